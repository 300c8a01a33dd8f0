"""GPU test of b200attn_forward_static, the entry point for callers that cannot allocate device
memory when they need attention (code living under a framework allocator that owns the device, or a
latency-critical loop that cannot afford the implicit synchronisation of an allocation): its scratch is a fixed array inside the library image.  Called
through the C ABI twice in a row (the array is shared by all calls and keeps the previous call's
contents, so the second call must not be disturbed by the first) and compared with the regular
entry point under the fp32 tolerance of the other tests (max-abs 1e-4 / rel 1e-3).

This file sorts last so that a run stopping at the first failure has already run everything else."""
import ctypes as C

import numpy as np
import pytest

import oracle_lib as ol
from gpu_util import to_dev

pytestmark = pytest.mark.gpu


def call_static(pkg, q, k, v):
    import torch
    out = torch.full_like(q, float("nan"))
    B, H, Lq, D = q.shape
    rc = pkg.lib().b200attn_forward_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, H, Lq, k.shape[2], D,
                                           torch.cuda.current_stream().cuda_stream)
    assert rc == 0, pkg.lib().b200attn_static_last_error()
    torch.cuda.synchronize()
    return out


def test_static_scratch_entry_matches_regular_entry_twice_in_a_row(pkg, cuda):
    first = (1, 4, 64, 64, 2048)
    second = (2, 3, 32, 48, 520)     # different shape right after: sees whatever the first call left in the array
    outs = []
    for shape, seed in ((first, 91), (second, 92), (first, 93)):
        B, H, Lq, Lk, D = shape
        Q, K, V = ol.make_qkv(B, H, Lq, Lk, D, seed, "uniform")
        q, k, v = (to_dev(x, cuda) for x in (Q, K, V))
        got = call_static(pkg, q, k, v).cpu().numpy()
        ref = pkg.forward(q, k, v).cpu().numpy()
        res = ol.compare(got, ref)
        assert res["ok"], (shape, res)
        res = ol.compare(got, ol.attention(Q, K, V))
        assert res["ok"], (shape, res)
        outs.append(got)
    assert np.isfinite(outs[0]).all() and np.isfinite(outs[2]).all()


def test_static_scratch_entry_rejects_what_does_not_fit(pkg, cuda):
    import torch
    L = pkg.lib()
    q = torch.zeros(1, 1, 128, 64, device=cuda)
    o = torch.empty_like(q)
    st = torch.cuda.current_stream().cuda_stream
    assert L.b200attn_forward_static(q.data_ptr(), q.data_ptr(), q.data_ptr(), o.data_ptr(), 1, 1, 128, 128, 64, st) == 5   # len > 64
    assert b"64" in L.b200attn_static_last_error()
    # 100 heads x 64 x 64 scores = 1.6 MB: beyond the 1 MiB array
    qq = torch.zeros(1, 100, 64, 16, device=cuda)
    oo = torch.empty_like(qq)
    assert L.b200attn_forward_static(qq.data_ptr(), qq.data_ptr(), qq.data_ptr(), oo.data_ptr(), 1, 100, 64, 64, 16, st) == 5
    assert b"static scratch" in L.b200attn_static_last_error()
    # every other limit holds (148 heads x 16 x 16 scores are 150 KB), but a head gets one slice and a slice
    # of 8192 columns does not fit an SM's shared memory
    qw = torch.zeros(1, 148, 16, 8192, device=cuda)
    ow = torch.empty_like(qw)
    assert L.b200attn_forward_static(qw.data_ptr(), qw.data_ptr(), qw.data_ptr(), ow.data_ptr(), 1, 148, 16, 16, 8192, st) == 5
    assert b"one slice per SM" in L.b200attn_static_last_error()
    assert L.b200attn_forward_static(None, None, None, None, 1, 1, 4, 4, 8, st) == 1
