"""GPU parity of the bf16 entry points: bf16 in/out, fp32 scores/softmax/accumulate.  Oracle: the
fp32 CPU attention on the bf16-rounded inputs; tolerance stated by the task: max-abs <= 2e-2."""
import os

import numpy as np
import pytest

import oracle_lib as ol
from gpu_util import bf16_from_dev, bf16_problem, bf16_to_dev, call_legacy

pytestmark = pytest.mark.gpu
TOL = 2e-2


def run(pkg, cuda, bits, **kw):
    q, k, v = (bf16_to_dev(b, cuda) for b in bits)
    return bf16_from_dev(pkg.forward(q, k, v, **kw))


# kernels/attention_bf16_optimized_fused.cu:624-625
@pytest.mark.parametrize("shape", [(1, 4, 64, 512), (1, 4, 64, 2048), (1, 2, 32, 4096), (1, 1, 16, 8192)])
def test_reference_bf16_shape_list_drop_in(pkg, cuda, shape):
    B, H, L, D = shape
    bits, up = bf16_problem(B, H, L, L, D, 61, "uniform")
    q, k, v = (bf16_to_dev(b, cuda) for b in bits)
    for name, pe in (("attention_forward_bf16", ol.PE_NONE), ("attention_forward_sinusoidal_bf16", ol.PE_SINUSOIDAL),
                     ("attention_forward_rope_bf16", ol.PE_ROPE_INTERLEAVED)):
        got = bf16_from_dev(call_legacy(pkg, name, q, k, v))
        err = float(np.abs(got - ol.attention(*up, pe=pe)).max())
        assert err <= TOL, (name, shape, err)
        # a correct bf16 kernel is far inside the tolerance: output rounding is 2^-9 relative
        assert err <= 4e-3, (name, shape, err)


def test_bf16_hybrid_entry(pkg, cuda):
    B, H, L, D, rd = 1, 4, 64, 512, 128
    bits, up = bf16_problem(B, H, L, L, D, 62, "uniform")
    q, k, v = (bf16_to_dev(b, cuda) for b in bits)
    got = bf16_from_dev(call_legacy(pkg, "attention_forward_rope_bf16_v7", q, k, v, extra_ints=(rd,)))
    want = ol.attention(*up, pe=ol.PE_ROPE_Q_ONLY, rotary_dim=rd)
    assert float(np.abs(got - want).max()) <= 4e-3


@pytest.mark.parametrize("pe", [ol.PE_NONE, ol.PE_ROPE_HALF, ol.PE_ROPE_INTERLEAVED, ol.PE_SINUSOIDAL])
@pytest.mark.parametrize("shape", [(1, 2, 128, 128, 512), (1, 1, 256, 384, 512), (1, 1, 128, 256, 1024), (1, 2, 200, 136, 96)])
def test_bf16_both_paths_against_oracle(pkg, cuda, pe, shape):
    """Every shape runs on the CUDA-core path; shapes the tensor-core kernel takes also run on it."""
    B, H, Lq, Lk, D = shape
    bits, up = bf16_problem(B, H, Lq, Lk, D, 63, "normal")
    want = ol.attention(*up, pe=pe)
    got = run(pkg, cuda, bits, pe=pe, flags=pkg.FLAG_FORCE_GENERIC)
    assert pkg.last_path().startswith("splitd")
    assert float(np.abs(got - want).max()) <= TOL
    got = run(pkg, cuda, bits, pe=pe)
    err = float(np.abs(got - want).max())
    assert err <= TOL, (pkg.last_path(), shape, pe, err)
    # the one-kernel cluster pipeline, where it takes the shape
    got = run(pkg, cuda, bits, pe=pe, flags=pkg.FLAG_PREFER_ONE_KERNEL)
    if D <= 512 and D % 64 == 0 and Lq % 128 == 0 and Lk % 128 == 0 and pe != ol.PE_ROPE_HALF:
        assert pkg.last_path() == "tc_bf16"
    err = float(np.abs(got - want).max())
    assert err <= TOL, (pkg.last_path(), shape, pe, err)


@pytest.mark.parametrize("cfg", [
    ("cfg3 bf16 plain", 8, 16, 1024, 512, ol.PE_NONE),
    ("cfg4 bf16 rope-half", 4, 32, 2048, 1024, ol.PE_ROPE_HALF),
    ("cfg5 bf16 sinusoidal", 16, 32, 4096, 512, ol.PE_SINUSOIDAL),
    ("many units per cluster, sinusoidal", 2, 40, 1024, 512, ol.PE_SINUSOIDAL),
    ("many units per cluster, interleaved rope", 3, 30, 768, 256, ol.PE_ROPE_INTERLEAVED),
    ("single key block per unit", 1, 200, 128, 128, ol.PE_NONE),
    ("odd number of key blocks", 1, 90, 256, 384, ol.PE_SINUSOIDAL),
], ids=lambda c: c[0].replace(" ", "_").replace(",", ""))
def test_benchmark_bf16_configs_sampled(pkg, cuda, cfg):
    """Full benchmark shapes, inputs generated in HBM by the library; the oracle evaluates a
    stratified sample of rows (first/last, tile boundaries) of a few heads from the very bytes the
    device holds."""
    import torch
    name, B, H, L, D, pe = cfg
    n = B * H * L * D
    Q, K, V = (torch.empty(n, dtype=torch.bfloat16, device=cuda).view(B, H, L, D) for _ in range(3))
    for t, tid in ((Q, 0), (K, 1), (V, 2)):
        pkg.synth_fill(t, 44, tid, "normal")
    heads = [0, B * H // 2 + 1, B * H - 1]
    rows = sorted({0, 1, 63, 64, 127, min(128, L - 1), L // 2 + 5, L - 1})
    q3, k3, v3 = (t.view(B * H, L, D) for t in (Q, K, V))
    wants = []
    for h in heads:
        qs, ks, vs = (bf16_from_dev(t[h].contiguous()).reshape(1, 1, L, D) for t in (q3, k3, v3))
        wants.append(ol.attention_rows(qs, ks, vs, np.zeros(len(rows), np.int64), np.array(rows), pe=pe))
    # the default tensor-core path and, for the shapes it takes, the one-kernel cluster pipeline
    for prefer_pair in ((False, True) if D <= 512 else (False,)):
        out = pkg.forward(Q, K, V, pe=pe, flags=pkg.FLAG_PREFER_ONE_KERNEL if prefer_pair else 0)
        torch.cuda.synchronize()
        fused = D in (64, 128, 256)   # the one-kernel path (with an encoding: on encoded copies of Q and K)
        assert pkg.last_path() == ("tc_bf16" if prefer_pair else "tc_fused" if fused else "tc_wide")
        o = out.view(B * H, L, D)
        for h, want in zip(heads, wants):
            got = bf16_from_dev(o[h][rows].contiguous())
            err = float(np.abs(got - want).max())
            assert err <= TOL, (name, pkg.last_path(), h, err)
        assert bool(torch.isfinite(out.float()).all())
        del out, o


# Bounds a regression has to stay under; the tolerance of the task statement is TOL = 2e-2.  Observed on
# B200 with the stratified sample below: cfg3 1.2e-3, cfg4 1.1e-3, cfg5 1.6e-2.  The sinusoidal
# configuration is the thin one, and not because of the tables: the encoded operands q + pe, k + pe
# (magnitude up to 4) are rounded to bf16 once before the product (relative 2^-9 per element, about 3e-3 in
# a scaled score after 512 columns), and the encoding makes the softmax peaky, so a score error reaches the
# output undiluted.  Rotated operands (cfg4) are rounded the same way but meet a flat softmax over 2048 keys.
BENCH_REGRESSION_BOUND = {"cfg3": 2.5e-3, "cfg4": 2.5e-3, "cfg5": 1.9e-2}


@pytest.mark.parametrize("name,B,H,L,D,pe", [("cfg3", 8, 16, 1024, 512, ol.PE_NONE), ("cfg4", 4, 32, 2048, 1024, ol.PE_ROPE_HALF),
                                              ("cfg5", 16, 32, 4096, 512, ol.PE_SINUSOIDAL)], ids=["cfg3", "cfg4", "cfg5"])
def test_benchmark_bf16_error_on_a_stratified_sample_of_every_head(pkg, cuda, name, B, H, L, D, pe):
    """The three bf16 benchmark configurations at full size: EVERY (batch, head) slice is checked on 16 query
    rows (first and last rows, the rows on both sides of the 128- and 256-row tile boundaries, two rows
    that vary with the head) against the fp32 oracle evaluated on the very bytes the device holds; the
    configuration without an encoding also on two whole slices.  The maximum error is printed and held
    under a regression bound well inside the 2e-2 tolerance."""
    import os
    from concurrent.futures import ThreadPoolExecutor
    import torch
    Q, K, V = (torch.empty(B * H * L * D, dtype=torch.bfloat16, device=cuda).view(B, H, L, D) for _ in range(3))
    for t, tid in ((Q, 0), (K, 1), (V, 2)):
        pkg.synth_fill(t, 45, tid, "normal")
    out = pkg.forward(Q, K, V, pe=pe)
    torch.cuda.synchronize()
    assert pkg.last_path() == "tc_wide"
    q3, k3, v3, o3 = (t.view(B * H, L, D) for t in (Q, K, V, out))
    fixed = [0, 1, 126, 127, 128, 129, 255, 256, L // 2 - 1, L // 2, L - 257, L - 256, L - 2, L - 1]

    def rows_of(h):
        return sorted(set(fixed + [(37 * h + 11) % L, (101 * h + 300) % L]))

    def check(h, rows=None):
        rows = rows_of(h) if rows is None else rows
        ridx = torch.tensor(rows, device=cuda)
        qs = np.zeros((1, 1, L, D), np.float32)
        qs[0, 0, rows] = bf16_from_dev(q3[h][ridx].contiguous())
        ks, vs = (bf16_from_dev(t[h].contiguous()).reshape(1, 1, L, D) for t in (k3, v3))
        want = ol.attention_rows(qs, ks, vs, np.zeros(len(rows), np.int64), np.array(rows), pe=pe)
        got = bf16_from_dev(o3[h][ridx].contiguous())
        return float(np.abs(got - want).max())

    with ThreadPoolExecutor(max_workers=min(32, os.cpu_count() or 4)) as ex:
        errs = list(ex.map(check, range(B * H)))
        if pe == ol.PE_NONE:
            errs += list(ex.map(lambda h: check(h, list(range(L))), [3, B * H - 2]))
    worst = max(errs)
    print(f"\n[bf16 error] {name}: max_abs {worst:.3e} over {len(errs)} slice checks (mean of per-slice maxima {np.mean(errs):.3e}); "
          f"regression bound {BENCH_REGRESSION_BOUND[name]:.1e}, tolerance {TOL:.0e}")
    assert worst <= TOL, (name, worst)
    assert worst <= BENCH_REGRESSION_BOUND[name], (name, worst)
