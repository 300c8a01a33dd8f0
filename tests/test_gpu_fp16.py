"""GPU parity of fp16 in / out (fp32 accumulation) against the fp32 CPU oracle evaluated on the fp16-rounded
inputs: what kernels/attention_kernel_fp16.cu:194 (attention_forward_fp16) covers in the reference.  fp16
carries three more mantissa bits than bf16, so the bound asserted here is tighter than the bf16 tolerance
of 2e-2: max-abs <= 4e-3."""
import numpy as np
import pytest

import oracle_lib as ol

pytestmark = pytest.mark.gpu
TOL = 4e-3


def problem(B, H, Lq, Lk, D, seed, dist):
    Q, K, V = ol.make_qkv(B, H, Lq, Lk, D, seed, dist)
    h = tuple(x.astype(np.float16) for x in (Q, K, V))
    return h, tuple(x.astype(np.float32) for x in h)


def run(pkg, cuda, h, **kw):
    import torch
    q, k, v = (torch.from_numpy(x).to(cuda) for x in h)
    out = pkg.forward(q, k, v, **kw)
    torch.cuda.synchronize()
    return out.float().cpu().numpy()


@pytest.mark.parametrize("shape", [(1, 4, 64, 64, 512), (1, 4, 64, 64, 2048), (1, 2, 32, 32, 4096), (1, 1, 16, 16, 8192), (1, 3, 40, 70, 100)], ids=str)
@pytest.mark.parametrize("pe", [ol.PE_NONE, ol.PE_ROPE_INTERLEAVED, ol.PE_ROPE_HALF, ol.PE_SINUSOIDAL], ids=["none", "rope", "rope_half", "sinusoidal"])
def test_fp16_short_sequences_wide_heads(pkg, cuda, shape, pe):
    """The reference's shape list (final/attention.cu:517-524) in fp16, every encoding: split-head_d kernels."""
    B, H, Lq, Lk, D = shape
    h, up = problem(B, H, Lq, Lk, D, 101, "uniform")
    got = run(pkg, cuda, h, pe=pe)
    assert pkg.last_path().startswith("splitd")
    err = float(np.abs(got - ol.attention(*up, pe=pe)).max())
    assert err <= TOL, (shape, pe, pkg.last_path(), err)


@pytest.mark.parametrize("shape", [(2, 4, 512, 512, 512), (1, 2, 256, 384, 1024), (1, 3, 384, 128, 64)], ids=str)
def test_fp16_on_the_tensor_cores(pkg, cuda, shape):
    B, H, Lq, Lk, D = shape
    h, up = problem(B, H, Lq, Lk, D, 102, "normal")
    got = run(pkg, cuda, h)
    assert pkg.last_path() == ("tc_fused" if D in (64, 128, 256) else "tc_wide")
    err = float(np.abs(got - ol.attention(*up)).max())
    assert err <= TOL, (shape, err)
    # with an encoding: encoded fp16 copies of Q and K (fp32 arithmetic, one rounding), then the same kernels
    for pe in (ol.PE_ROPE_HALF, ol.PE_SINUSOIDAL, ol.PE_ROPE_Q_ONLY):
        want = ol.attention(*up, pe=pe)
        if pe == ol.PE_ROPE_Q_ONLY:   # the caller keeps K rotated
            kr = ol.apply_rope(up[1]).astype(np.float16)
            want = ol.attention(ol.apply_rope(up[0]), kr.astype(np.float32), up[2])
            got = run(pkg, cuda, (h[0], kr, h[2]), pe=pe)
        else:
            got = run(pkg, cuda, h, pe=pe)
        assert pkg.last_path() == ("tc_fused" if D in (64, 128, 256) else "tc_wide")
        assert float(np.abs(got - want).max()) <= 4e-3, pe


@pytest.mark.parametrize("shape", [(1, 16, 4, 4096, 128), (1, 4, 48, 2000, 64), (1, 32, 1, 8192, 128), (1, 3, 20, 777, 128)], ids=str)
def test_fp16_decode(pkg, cuda, shape):
    B, H, Lq, Lk, D = shape
    h, up = problem(B, H, Lq, Lk, D, 103, "normal")
    got = run(pkg, cuda, h)
    assert pkg.last_path() == "tc_decode"
    err = float(np.abs(got - ol.attention(*up)).max())
    assert err <= TOL, (shape, err)
