"""Helpers shared by the GPU parity tests: every call goes through the C ABI of the library."""
import ctypes as C

import numpy as np

import oracle_lib as ol


def to_dev(x, dev):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).to(dev)


def bf16_to_dev(bits, dev):
    import torch
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).to(dev).view(torch.bfloat16)


def bf16_from_dev(t):
    import torch
    return ol.from_bf16_bits(t.view(torch.int16).cpu().numpy().view(np.uint16))


def call_legacy(pkg, name, Q, K, V, extra_ptrs=(), extra_ints=()):
    """Calls a drop-in symbol (void return, device pointers, blocking) on torch tensors."""
    import torch
    out = torch.full_like(Q, float("nan"))
    B, H, Lq, D = Q.shape
    Lk = K.shape[2]
    fn = getattr(pkg.lib(), name)
    ptrs = [Q.data_ptr(), K.data_ptr(), V.data_ptr(), out.data_ptr()] + [t.data_ptr() for t in extra_ptrs]
    torch.cuda.synchronize()
    fn(*ptrs, B, H, Lq, Lk, D, *extra_ints)
    return out


def bf16_problem(B, H, Lq, Lk, D, seed, dist="normal"):
    """bf16 inputs (bits) and their exact fp32 up-casts for the oracle."""
    Q, K, V = ol.make_qkv(B, H, Lq, Lk, D, seed, dist)
    bits = tuple(ol.to_bf16_bits(x) for x in (Q, K, V))
    up = tuple(ol.from_bf16_bits(b) for b in bits)
    return bits, up
