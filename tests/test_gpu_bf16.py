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
        assert pkg.last_path() == ("tc_bf16" if prefer_pair else "tc_wide")
        o = out.view(B * H, L, D)
        for h, want in zip(heads, wants):
            got = bf16_from_dev(o[h][rows].contiguous())
            err = float(np.abs(got - want).max())
            assert err <= TOL, (name, pkg.last_path(), h, err)
        assert bool(torch.isfinite(out.float()).all())
        del out, o
