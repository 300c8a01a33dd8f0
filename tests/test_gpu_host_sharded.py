"""GPU tests of the host-buffer entry point, the (batch, head) sharded launcher and the device
input generator, all through the C ABI."""
import ctypes as C

import numpy as np
import pytest

import oracle_lib as ol
from gpu_util import to_dev

pytestmark = pytest.mark.gpu


def test_forward_host_pageable_and_pinned(pkg, cuda):
    import torch
    B, H, L, D = 1, 4, 64, 2048
    Q, K, V = ol.make_qkv(B, H, L, L, D, 71, "uniform")
    want = ol.attention(Q, K, V, pe=ol.PE_SINUSOIDAL)
    out = np.empty_like(Q)
    pkg.forward_host(torch.from_numpy(Q), torch.from_numpy(K), torch.from_numpy(V), torch.from_numpy(out), pe=pkg.PE_SINUSOIDAL)
    assert ol.compare(out, want)["ok"]
    qp, kp, vp = (torch.from_numpy(x).pin_memory() for x in (Q, K, V))
    op = torch.empty_like(qp).pin_memory()
    pkg.forward_host(qp, kp, vp, op, pe=pkg.PE_SINUSOIDAL)
    assert ol.compare(op.numpy(), want)["ok"]


def test_forward_host_pipelined_chunks_equal_device_call(pkg, cuda):
    """A problem large enough to be cut into chunks of heads whose copy-in, compute and copy-out
    overlap: the result must equal the single device call on the same bytes."""
    import torch
    B, H, L, D = 2, 40, 1024, 512
    Q, K, V = (torch.empty(B, H, L, D, dtype=torch.bfloat16, device=cuda) for _ in range(3))
    for t, tid in ((Q, 0), (K, 1), (V, 2)):
        pkg.synth_fill(t, 73, tid, "normal")
    want = pkg.forward(Q, K, V, pe=pkg.PE_SINUSOIDAL).cpu()
    hq, hk, hv = (t.cpu().pin_memory() for t in (Q, K, V))
    ho = torch.empty_like(hq).pin_memory()
    for _ in range(2):   # twice: the second call reuses the staging buffers
        ho.zero_()
        pkg.forward_host(hq, hk, hv, ho, pe=pkg.PE_SINUSOIDAL)
        assert torch.equal(ho.view(torch.int16), want.view(torch.int16))


def test_sharded_launcher_equals_single_call(pkg, cuda):
    """Two shards placed on the devices that exist (both on device 0 when there is one GPU): the
    launcher needs no collective because (b,h) slices are contiguous slabs."""
    import torch
    B, H, L, D = 2, 3, 48, 256
    Q, K, V = ol.make_qkv(B, H, L, L, D, 72, "uniform")
    want = ol.attention(Q, K, V, pe=ol.PE_ROPE_HALF)
    ndev = min(2, torch.cuda.device_count())
    devices = [g % ndev for g in range(2)]
    begin, count = pkg.shard_ranges(B * H, 2)
    flat = lambda x: x.reshape(B * H, L, D)
    parts = []
    for g in range(2):
        d = torch.device(f"cuda:{devices[g]}")
        sl = slice(begin[g], begin[g] + count[g])
        parts.append(tuple(to_dev(flat(x)[sl], d) for x in (Q, K, V)) + (torch.empty(count[g], L, D, device=d),))
    arr = lambda i: (C.c_void_p * 2)(*[parts[g][i].data_ptr() for g in range(2)])
    proto = pkg.make_args(None, None, None, None, 0, 0, L, L, D, pkg.F32, pe=pkg.PE_ROPE_HALF)
    rc = pkg.lib().b200attn_forward_sharded(C.byref(proto), 2, (C.c_int * 2)(*devices), arr(0), arr(1), arr(2), arr(3),
                                            (C.c_int * 2)(*count))
    pkg.check(rc)
    got = np.concatenate([parts[g][3].cpu().numpy() for g in range(2)]).reshape(B, H, L, D)
    assert ol.compare(got, want)["ok"]
    # a failing device ordinal is reported as a status, not a crash
    rc = pkg.lib().b200attn_forward_sharded(C.byref(proto), 1, (C.c_int * 1)(63), arr(0), arr(1), arr(2), arr(3), (C.c_int * 1)(1))
    assert rc != 0 and len(pkg.lib().b200attn_last_error()) > 0
    torch.cuda.set_device(0)


@pytest.mark.parametrize("dtype,pe,shape", [("f32", "none", (2, 4, 64, 64, 2048)), ("bf16", "sinusoidal", (2, 8, 512, 512, 512)),
                                            ("bf16", "rope_half", (1, 6, 256, 256, 1024))])
def test_sharded_launcher_on_different_physical_gpus(pkg, cuda, dtype, pe, shape):
    """b200attn_forward_sharded with one shard per physical GPU (needs at least two; skipped otherwise):
    every device runs its contiguous range of (batch, head) slices on its own stream, and the result
    equals the single-GPU call on the same bytes bit for bit (bf16) or within the fp32 tolerance."""
    import torch
    ndev = torch.cuda.device_count()
    if ndev < 2:
        pytest.skip("needs two GPUs")
    B, H, Lq, Lk, D = shape
    td = torch.float32 if dtype == "f32" else torch.bfloat16
    pe_id = {"none": pkg.PE_NONE, "sinusoidal": pkg.PE_SINUSOIDAL, "rope_half": pkg.PE_ROPE_HALF}[pe]
    Q, K, V = (torch.empty(B, H, L, D, dtype=td, device=cuda) for L in (Lq, Lk, Lk))
    for t, tid in ((Q, 0), (K, 1), (V, 2)):
        pkg.synth_fill(t, 75, tid, "uniform" if dtype == "f32" else "normal")
    want = pkg.forward(Q, K, V, pe=pe_id)
    torch.cuda.synchronize()
    G = min(ndev, 4)
    begin, count = pkg.shard_ranges(B * H, G)
    parts = []
    for g in range(G):
        d = torch.device(f"cuda:{g}")
        sl = slice(begin[g], begin[g] + count[g])
        parts.append(tuple(t.view(B * H, -1, D)[sl].to(d) for t in (Q, K, V)) + (torch.empty(count[g], Lq, D, dtype=td, device=d),))
    arr = lambda i: (C.c_void_p * G)(*[parts[g][i].data_ptr() for g in range(G)])
    proto = pkg.make_args(None, None, None, None, 0, 0, Lq, Lk, D, pkg.F32 if dtype == "f32" else pkg.BF16, pe=pe_id)
    for rep in range(2):
        rc = pkg.lib().b200attn_forward_sharded(C.byref(proto), G, (C.c_int * G)(*range(G)), arr(0), arr(1), arr(2), arr(3), (C.c_int * G)(*count))
        pkg.check(rc)
        got = torch.cat([parts[g][3].to(cuda) for g in range(G)]).view(B, H, Lq, D)
        if dtype == "bf16":
            assert torch.equal(got.view(torch.int16), want.view(torch.int16))
        else:
            assert (got - want).abs().max().item() <= 2e-6
    torch.cuda.set_device(0)


def test_device_generator_matches_host_generator(pkg, cuda):
    import torch
    n = 1 << 16
    t = pkg.synth_fill(torch.empty(n, device=cuda), 43, 1, "uniform")
    assert np.array_equal(t.cpu().numpy(), ol.synth_uniform((n,), 43, 1))
    g = pkg.synth_fill(torch.empty(n, device=cuda), 44, 2, "normal").cpu().numpy()
    h = ol.synth_normal((n,), 44, 2)
    # libm and the device math library may differ in the last place of logf/cosf
    assert np.abs(g - h).max() < 1e-5
    b = pkg.synth_fill(torch.empty(n, device=cuda, dtype=torch.bfloat16), 44, 2, "normal")
    hb = ol.from_bf16_bits(ol.to_bf16_bits(h))
    gb = b.float().cpu().numpy()
    assert np.mean(gb != hb) < 1e-3


def test_launch_counter_moves(pkg, cuda):
    import torch
    q = torch.rand(1, 2, 16, 64, device=cuda)
    n0 = pkg.launch_count()
    pkg.forward(q, q.clone(), q.clone())
    assert pkg.launch_count() > n0
