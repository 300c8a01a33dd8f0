"""GPU parity of the fp32 path: the CUDA library, called through its C ABI, against the CPU oracle
on the same seeded inputs.  Tolerance (stated by the task for fp32): max-abs <= 1e-4, and no
element with both abs > 1e-4 and rel > 1e-3 (the reference's AND rule, final/attention.cu:310)."""
import glob
import os

import numpy as np
import pytest

import oracle_lib as ol
from gpu_util import call_legacy, to_dev
from test_oracle import GOLD, KIND_PE, load_refcpu

pytestmark = pytest.mark.gpu

LEGACY = {"plain": "attention_forward_optimized", "rope": "attention_forward_rope_fused_v2",
          "sinus": "attention_forward_sinusoidal_fused"}


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLD, "refcpu_*.npz"))), ids=os.path.basename)
def test_drop_in_symbols_match_reference_cpu_fixtures(pkg, cuda, path):
    kind, (B, H, Lq, Lk, D), seed, rows, want = load_refcpu(path)
    Q, K, V = ol.make_qkv(B, H, Lq, Lk, D, seed, "uniform")
    got = call_legacy(pkg, LEGACY[kind], to_dev(Q, cuda), to_dev(K, cuda), to_dev(V, cuda)).cpu().numpy()
    res = ol.compare(got[:, :, rows, :], want)
    assert res["ok"], (kind, (B, H, Lq, Lk, D), pkg.last_path(), res)
    # and the whole output against the oracle run now
    res = ol.compare(got, ol.attention(Q, K, V, pe=KIND_PE[kind]))
    assert res["ok"], res


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLD, "sdpa_*.npz"))), ids=os.path.basename)
def test_reference_sdpa_golden_vectors(pkg, cuda, path):
    z = np.load(path)
    got = pkg.forward(to_dev(z["Q"], cuda), to_dev(z["K"], cuda), to_dev(z["V"], cuda)).cpu().numpy()
    res = ol.compare(got, z["output"])
    assert res["ok"], res


@pytest.mark.parametrize("shape", [(1, 4, 64, 64, 2048), (1, 4, 64, 64, 512), (1, 4, 64, 64, 4096),
                                   (1, 4, 64, 64, 8192), (1, 4, 32, 64, 4096)])
def test_benchmark_configs_fused_and_two_pass(pkg, cuda, shape):
    B, H, Lq, Lk, D = shape
    Q, K, V = ol.make_qkv(B, H, Lq, Lk, D, 43, "uniform")
    want = ol.attention(Q, K, V)
    q, k, v = (to_dev(x, cuda) for x in (Q, K, V))
    got = pkg.forward(q, k, v).cpu().numpy()
    assert pkg.last_path() == "splitd_tc"
    res = ol.compare(got, want)
    assert res["ok"] and res["max_abs"] <= 5e-6, res   # error-compensated tf32 keeps fp32 accuracy
    # twice more: both halves of the double-buffered score scratch, each cleared by the call before
    for _ in range(2):
        assert ol.compare(pkg.forward(q, k, v).cpu().numpy(), want)["ok"]
    got = pkg.forward(q, k, v, flags=pkg.FLAG_FORCE_GENERIC).cpu().numpy()
    assert pkg.last_path() == "splitd_fused"
    assert ol.compare(got, want)["ok"], ol.compare(got, want)
    got2 = pkg.forward(q, k, v, flags=pkg.FLAG_FORCE_TWO_PASS).cpu().numpy()
    assert pkg.last_path() == "splitd_two_pass"
    assert ol.compare(got2, want)["ok"], ol.compare(got2, want)
    # a second fused call right after: the shared score scratch must have been left clean
    got3 = pkg.forward(q, k, v).cpu().numpy()
    assert ol.compare(got3, want)["ok"]


@pytest.mark.parametrize("shape", [(1, 4, 64, 64, 2048), (1, 4, 64, 64, 512), (1, 4, 64, 64, 4096), (1, 4, 64, 64, 8192),
                                   (1, 4, 32, 64, 4096)])
def test_against_the_reference_gpu_kernel(pkg, cuda, shape):
    """The reference's own kernel (compiled from the reference tree into oracle/_ref) on the same GPU."""
    import torch
    ref = ol.ref()
    if ref is None:
        pytest.skip("oracle/_ref not available")
    B, H, Lq, Lk, D = shape
    Q, K, V = ol.make_qkv(B, H, Lq, Lk, D, 44, "uniform")
    q, k, v = (to_dev(x, cuda) for x in (Q, K, V))
    ref_out = torch.empty_like(q)
    torch.cuda.synchronize()
    ref.ref_attention_forward_optimized(q.data_ptr(), k.data_ptr(), v.data_ptr(), ref_out.data_ptr(), B, H, Lq, Lk, D)
    got = pkg.forward(q, k, v)
    res = ol.compare(got.cpu().numpy(), ref_out.cpu().numpy())
    assert res["ok"], res


@pytest.mark.parametrize("pe,rd", [(ol.PE_ROPE_INTERLEAVED, 0), (ol.PE_ROPE_INTERLEAVED, 32), (ol.PE_ROPE_HALF, 0),
                                   (ol.PE_ROPE_HALF, 64), (ol.PE_ROPE_HALF, 20), (ol.PE_SINUSOIDAL, 0), (ol.PE_ROPE_Q_ONLY, 64)])
@pytest.mark.parametrize("shape", [(1, 3, 24, 40, 128), (2, 2, 64, 64, 1024), (1, 2, 100, 150, 96)])
def test_positional_encodings_all_kinds(pkg, cuda, pe, rd, shape):
    B, H, Lq, Lk, D = shape
    Q, K, V = ol.make_qkv(B, H, Lq, Lk, D, 45, "uniform")
    want = ol.attention(Q, K, V, pe=pe, rotary_dim=(rd or None))
    got = pkg.forward(to_dev(Q, cuda), to_dev(K, cuda), to_dev(V, cuda), pe=pe, rotary_dim=rd).cpu().numpy()
    res = ol.compare(got, want)
    assert res["ok"], (pkg.last_path(), res)


@pytest.mark.parametrize("shape", [(1, 1, 1, 1, 8), (1, 1, 64, 64, 32), (1, 3, 17, 23, 100), (2, 5, 7, 64, 36), (1, 148, 16, 16, 64),
                                   (1, 2, 33, 9, 1028), (1, 37, 64, 64, 1024), (1, 1, 64, 64, 16384), (1, 1, 16, 16, 32768),
                                   (2, 4, 64, 40, 4096), (1, 8, 5, 3, 2052)])
def test_tensor_core_split_path_ragged_shapes(pkg, cuda, shape):
    """fp32 on the tensor cores: ragged lengths (rows beyond len are never loaded; key rows up to the next
    multiple of 8 are zero-filled), head_d that is not a multiple of 32 (zero-filled columns), one slice
    per head up to all SMs on one head, and the extreme head_d of kernels/attention_kernel_ultra_large.cu:414-419."""
    B, H, Lq, Lk, D = shape
    Q, K, V = ol.make_qkv(B, H, Lq, Lk, D, 50, "uniform")
    want = ol.attention(Q, K, V)
    q, k, v = (to_dev(x, cuda) for x in (Q, K, V))
    for rep in range(2):
        got = pkg.forward(q, k, v).cpu().numpy()
        assert pkg.last_path() == "splitd_tc", shape
        res = ol.compare(got, want)
        assert res["ok"] and res["max_abs"] <= 5e-6, (shape, rep, res)


def test_tensor_core_split_path_changing_head_counts(pkg, cuda):
    """Consecutive calls with different numbers of heads: each call clears what the previous one left in
    the other half of the score scratch, however many heads that was."""
    for (B, H, L, D) in [(1, 40, 64, 256), (1, 3, 64, 2048), (1, 100, 32, 128), (1, 1, 64, 4096), (1, 100, 32, 128), (1, 40, 64, 256)]:
        Q, K, V = ol.make_qkv(B, H, L, L, D, 51, "uniform")
        got = pkg.forward(to_dev(Q, cuda), to_dev(K, cuda), to_dev(V, cuda)).cpu().numpy()
        assert pkg.last_path() == "splitd_tc"
        res = ol.compare(got, ol.attention(Q, K, V))
        assert res["ok"] and res["max_abs"] <= 5e-6, ((B, H, L, D), res)


def test_forward_many_overlaps_consecutive_entries_correctly(pkg, cuda):
    """b200attn_forward_many launches an entry as the programmatic dependent of the one before it (its loads
    run under the other's tail).  Every entry of a long mixed batch must still be right, including an
    entry that reads the previous entry's output (the library detects that and does not overlap it)."""
    import torch
    shapes = [(1, 4, 64, 64, 2048), (1, 4, 64, 64, 512), (1, 4, 32, 64, 4096), (1, 2, 64, 64, 64), (1, 4, 64, 64, 8192),
              (1, 4, 64, 64, 2048), (1, 7, 16, 48, 256), (1, 4, 64, 64, 4096)] * 3
    probs, args = [], []
    for n, (B, H, Lq, Lk, D) in enumerate(shapes):
        Q, K, V = ol.make_qkv(B, H, Lq, Lk, D, 60 + n, "uniform")
        q, k, v = (to_dev(x, cuda) for x in (Q, K, V))
        o = torch.full_like(q, float("nan"))
        probs.append((Q, K, V, q, k, v, o))
        args.append(pkg.args_for(q, k, v, o, flags=pkg.FLAG_ASYNC))
    # a dependent pair at the end: the second reads the first one's output as its Q
    Q, K, V, q, k, v, o = probs[0]
    o2 = torch.full_like(q, float("nan"))
    args.append(pkg.args_for(o, k, v, o2, flags=pkg.FLAG_ASYNC))
    for rep in range(2):
        pkg.forward_many(args)
        torch.cuda.synchronize()
        for (Q, K, V, q, k, v, o) in probs:
            res = ol.compare(o.cpu().numpy(), ol.attention(Q, K, V))
            assert res["ok"] and res["max_abs"] <= 5e-6, (Q.shape, res)
        first = probs[0]
        want2 = ol.attention(first[6].cpu().numpy(), first[1], first[2])
        assert ol.compare(o2.cpu().numpy(), want2)["ok"]


def test_asynchronous_calls_on_two_streams_share_the_scratch_safely(pkg, cuda):
    """Two B200ATTN_FLAG_ASYNC calls on two different streams from one thread: the library orders the second
    after the first on the device (they share per-device scratch and tables), so both are right."""
    import torch
    s1, s2 = torch.cuda.Stream(device=cuda), torch.cuda.Stream(device=cuda)
    cases = []
    for n, (shape, pe) in enumerate([((1, 4, 64, 64, 2048), ol.PE_NONE), ((1, 4, 64, 64, 4096), ol.PE_NONE),
                                     ((1, 2, 64, 64, 512), ol.PE_SINUSOIDAL), ((1, 3, 96, 130, 64), ol.PE_ROPE_INTERLEAVED)]):
        B, H, Lq, Lk, D = shape
        Q, K, V = ol.make_qkv(B, H, Lq, Lk, D, 70 + n, "uniform")
        cases.append((Q, K, V, pe) + tuple(to_dev(x, cuda) for x in (Q, K, V)))
    torch.cuda.synchronize()
    for rep in range(3):
        outs = []
        for n, (Q, K, V, pe, q, k, v) in enumerate(cases):
            st = (s1, s2)[n % 2]
            outs.append(pkg.forward(q, k, v, pe=pe, stream=st.cuda_stream, flags=pkg.FLAG_ASYNC))
        s1.synchronize(); s2.synchronize()
        for (Q, K, V, pe, q, k, v), o in zip(cases, outs):
            res = ol.compare(o.cpu().numpy(), ol.attention(Q, K, V, pe=pe))
            assert res["ok"], (Q.shape, pe, rep, res)


def test_hybrid_entry_with_rotary_dim_zero_is_plain_attention(pkg, cuda):
    """The reference kernel rotates the columns d < rotary_dim (final/rope.cu:129-149): with 0 there is no
    rotation at all, and the hybrid entry is plain attention on Q and the K it was given."""
    import torch
    B, H, L, D = 1, 4, 64, 512
    Q, K, V = ol.make_qkv(B, H, L, L, D, 52, "uniform")
    q, k, v = (to_dev(x, cuda) for x in (Q, K, V))
    got = call_legacy(pkg, "attention_forward_rope_fused_v7_hybrid", q, k, v, extra_ints=(0,))
    assert ol.compare(got.cpu().numpy(), ol.attention(Q, K, V))["ok"]
    ref = ol.ref()
    if ref is not None and hasattr(ref, "ref_attention_forward_rope_fused_v7_hybrid"):
        ref_out = torch.empty_like(q)
        torch.cuda.synchronize()
        ref.ref_attention_forward_rope_fused_v7_hybrid(q.data_ptr(), k.data_ptr(), v.data_ptr(), ref_out.data_ptr(), B, H, L, L, D, 0)
        assert ol.compare(got.cpu().numpy(), ref_out.cpu().numpy())["ok"]


def test_rope_with_caller_supplied_caches_and_hybrid_entry(pkg, cuda):
    B, H, L, D, rd = 1, 4, 64, 512, 128
    Q, K, V = ol.make_qkv(B, H, L, L, D, 46, "uniform")
    c, s = ol.rope_cache(L, D)
    q, k, v = (to_dev(x, cuda) for x in (Q, K, V))
    got = call_legacy(pkg, "attention_forward_rope_fused", q, k, v, extra_ptrs=(to_dev(c, cuda), to_dev(s, cuda)))
    assert ol.compare(got.cpu().numpy(), ol.attention(Q, K, V, pe=ol.PE_ROPE_INTERLEAVED))["ok"]
    # hybrid: the caller pre-rotates K (first rd columns), the library rotates Q in the load
    c2, s2 = ol.rope_cache(L, rd)
    Kr = K.copy()
    Kr[..., 0:rd:2] = K[..., 0:rd:2] * c2[:, 0::2] - K[..., 1:rd:2] * s2[:, 0::2]
    Kr[..., 1:rd:2] = K[..., 0:rd:2] * s2[:, 0::2] + K[..., 1:rd:2] * c2[:, 0::2]
    got = call_legacy(pkg, "attention_forward_rope_fused_v7_hybrid", q, to_dev(Kr, cuda), v, extra_ints=(rd,))
    res = ol.compare(got.cpu().numpy(), ol.attention(Q, K, V, pe=ol.PE_ROPE_INTERLEAVED, rotary_dim=rd))
    assert res["ok"], res


@pytest.mark.parametrize("shape", [(1, 1, 1, 1, 8), (1, 1, 3, 5, 7), (1, 2, 5, 9, 30), (1, 1, 64, 64, 8), (3, 5, 2, 70, 12),
                                   (1, 1, 65, 129, 260), (1, 160, 16, 16, 64)])
def test_edge_shapes_ragged_and_odd_head_d(pkg, cuda, shape):
    B, H, Lq, Lk, D = shape
    Q, K, V = ol.make_qkv(B, H, Lq, Lk, D, 47, "uniform")
    for pe in (ol.PE_NONE, ol.PE_SINUSOIDAL):
        got = pkg.forward(to_dev(Q, cuda), to_dev(K, cuda), to_dev(V, cuda), pe=pe).cpu().numpy()
        res = ol.compare(got, ol.attention(Q, K, V, pe=pe))
        assert res["ok"], (shape, pe, pkg.last_path(), res)


def test_llama_style_shape_sampled(pkg, cuda):
    """final/attention.cu:522 (4,32,512,128): checked on sampled rows of every 8th head."""
    B, H, L, D = 4, 32, 512, 128
    Q, K, V = ol.make_qkv(B, H, L, L, D, 48, "uniform")
    got = pkg.forward(to_dev(Q, cuda), to_dev(K, cuda), to_dev(V, cuda)).cpu().numpy().reshape(B * H, L, D)
    bh = np.repeat(np.arange(0, B * H, 8), 4)
    rows = np.tile(np.array([0, 63, 64, 511]), len(bh) // 4)
    want = ol.attention_rows(Q, K, V, bh, rows)
    res = ol.compare(got[bh, rows], want)
    assert res["ok"], res


def test_properties_at_full_size(pkg, cuda):
    """Size-independent identities at the largest fp32 config: linearity in V, constant V, and
    outputs inside the per-column range of V (rows of P are convex weights)."""
    import torch
    B, H, L, D = 1, 4, 64, 8192
    Q, K, V = (to_dev(x, cuda) for x in ol.make_qkv(B, H, L, L, D, 49, "uniform"))
    V2 = torch.flip(V, dims=[2]).contiguous()
    o1, o2 = pkg.forward(Q, K, V), pkg.forward(Q, K, V2)
    o12 = pkg.forward(Q, K, (0.5 * V - 2.0 * V2).contiguous())
    assert (o12 - (0.5 * o1 - 2.0 * o2)).abs().max().item() < 2e-5
    oc = pkg.forward(Q, K, torch.full_like(V, 0.375))
    assert (oc - 0.375).abs().max().item() < 1e-6
    lo, hi = V.amin(dim=2, keepdim=True), V.amax(dim=2, keepdim=True)
    assert bool(((o1 >= lo - 1e-6) & (o1 <= hi + 1e-6)).all())
    # determinism of repeated calls up to the order of the fp32 score reduction
    assert (pkg.forward(Q, K, V) - o1).abs().max().item() < 1e-6


def test_error_status_instead_of_exit(pkg, cuda):
    import torch
    q = torch.zeros(1, 1, 4, 8, device=cuda)
    with pytest.raises(pkg.B200AttnError):
        pkg.forward(q, q, q, out=q)
    a = pkg.make_args(q.data_ptr(), q.data_ptr(), q.data_ptr(), torch.empty_like(q).data_ptr(), 1, 1, 4, 4, 8, pkg.F32,
                      pe=pkg.PE_ROPE_INTERLEAVED, rotary_dim=10)
    assert pkg.lib().b200attn_forward_ex(C_byref(a)) == 1


def C_byref(a):
    import ctypes
    return ctypes.byref(a)
