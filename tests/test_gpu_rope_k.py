"""GPU parity of the "rotate K once" producer (b200attn_rope_k), of attention on a pre-rotated K (the
*_Q_ONLY encodings, both pairings) and of caller-supplied cos/sin caches on the tensor-core path, against
the CPU oracle.  fp32: max-abs <= 1e-4 (rotation itself: a few ulp); bf16: max-abs <= 2e-2."""
import numpy as np
import pytest

import oracle_lib as ol
from gpu_util import bf16_from_dev, bf16_problem, bf16_to_dev, to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("half", [False, True], ids=["interleaved", "half"])
@pytest.mark.parametrize("shape,rd,pos0", [((2, 3, 40, 128), 0, 0), ((1, 4, 64, 2048), 128, 0), ((1, 2, 17, 100), 20, 5),
                                           ((2, 2, 300, 64), 0, 1000), ((1, 1, 9, 30), 6, 0)])
def test_rope_k_matches_the_oracle_rotation_fp32(pkg, cuda, half, shape, rd, pos0):
    B, H, L, D = shape
    X = ol.synth_uniform((B, H, L, D), 81, 1)
    want = ol.apply_rope(X, half=half, rotary_dim=(rd or None), pos0=pos0)
    got = pkg.rope_k(to_dev(X, cuda), pairing=pkg.PE_ROPE_HALF if half else pkg.PE_ROPE_INTERLEAVED, rotary_dim=rd, pos0=pos0)
    # sincosf on the device and libm on the host differ in the last place at large angles
    assert float(np.abs(got.cpu().numpy() - want).max()) <= (2e-6 if pos0 == 0 else 2e-4)
    # from caller caches (the reference's layout) the result is the same arithmetic on the same numbers
    c, s = ol.rope_cache(pos0 + L, rd or D)
    got = pkg.rope_k(to_dev(X, cuda), pairing=pkg.PE_ROPE_HALF if half else pkg.PE_ROPE_INTERLEAVED, rotary_dim=rd, pos0=pos0,
                     cos_cache=to_dev(c, cuda), sin_cache=to_dev(s, cuda))
    assert float(np.abs(got.cpu().numpy() - want).max()) <= 5e-7


@pytest.mark.parametrize("half", [False, True], ids=["interleaved", "half"])
def test_rope_k_bf16_in_place_and_single_rounding(pkg, cuda, half):
    import torch
    B, H, L, D = 2, 4, 256, 512
    bits = ol.to_bf16_bits(ol.synth_normal((B, H, L, D), 82, 1))
    want = ol.from_bf16_bits(ol.to_bf16_bits(ol.apply_rope(ol.from_bf16_bits(bits), half=half)))
    x = bf16_to_dev(bits, cuda)
    pkg.rope_k(x, out=x, pairing=pkg.PE_ROPE_HALF if half else pkg.PE_ROPE_INTERLEAVED)   # in place
    torch.cuda.synchronize()
    got = bf16_from_dev(x)
    # the product is fp32 and rounded once: at most one bf16 ulp where device and host sincos differ in the last place
    assert np.mean(got != want) < 2e-3 and float(np.abs(got - want).max()) <= 4e-2


@pytest.mark.parametrize("half", [False, True], ids=["interleaved", "half"])
@pytest.mark.parametrize("shape", [(1, 4, 64, 64, 512), (1, 2, 100, 150, 96)])
def test_attention_on_k_rotated_by_rope_k_fp32(pkg, cuda, half, shape):
    B, H, Lq, Lk, D = shape
    Q, K, V = ol.make_qkv(B, H, Lq, Lk, D, 83, "uniform")
    want = ol.attention(Q, K, V, pe=ol.PE_ROPE_HALF if half else ol.PE_ROPE_INTERLEAVED)
    q, k, v = (to_dev(x, cuda) for x in (Q, K, V))
    kr = pkg.rope_k(k, pairing=pkg.PE_ROPE_HALF if half else pkg.PE_ROPE_INTERLEAVED)
    got = pkg.forward(q, kr, v, pe=pkg.PE_ROPE_HALF_Q_ONLY if half else pkg.PE_ROPE_Q_ONLY).cpu().numpy()
    res = ol.compare(got, want)
    assert res["ok"], (pkg.last_path(), res)


@pytest.mark.parametrize("half", [False, True], ids=["interleaved", "half"])
@pytest.mark.parametrize("shape", [(1, 3, 256, 512, 512), (1, 2, 384, 256, 1024)])
def test_attention_on_k_rotated_by_rope_k_bf16_on_the_tensor_cores(pkg, cuda, half, shape):
    """The KV-cache contract at tensor-core speed for both pairings: K is rotated once by b200attn_rope_k
    (rounded to bf16 once, which is also what the fused path does) and attention rotates Q only."""
    B, H, Lq, Lk, D = shape
    bits, up = bf16_problem(B, H, Lq, Lk, D, 84, "normal")
    want = ol.attention(*up, pe=ol.PE_ROPE_HALF if half else ol.PE_ROPE_INTERLEAVED)
    q, k, v = (bf16_to_dev(b, cuda) for b in bits)
    kr = pkg.rope_k(k, pairing=pkg.PE_ROPE_HALF if half else pkg.PE_ROPE_INTERLEAVED)
    got = bf16_from_dev(pkg.forward(q, kr, v, pe=pkg.PE_ROPE_HALF_Q_ONLY if half else pkg.PE_ROPE_Q_ONLY))
    assert pkg.last_path() == "tc_wide"
    err = float(np.abs(got - want).max())
    assert err <= 8e-3, err
    # and the fused call (library rotates both) agrees with it to bf16 rounding
    fused = bf16_from_dev(pkg.forward(q, k, v, pe=pkg.PE_ROPE_HALF if half else pkg.PE_ROPE_INTERLEAVED))
    assert float(np.abs(got - fused).max()) <= 8e-3


@pytest.mark.parametrize("pe", [ol.PE_ROPE_INTERLEAVED, ol.PE_ROPE_HALF, ol.PE_ROPE_Q_ONLY], ids=["interleaved", "half", "q_only"])
def test_caller_supplied_caches_on_the_tensor_core_path(pkg, cuda, pe):
    """cos/sin caches in the reference's layout (final/rope.cu:20-40) with a base the library would not
    have used by itself: the tensor-core path takes them (a table is made from them on every call)."""
    B, H, L, D, base = 1, 3, 256, 512, 500.0
    bits, up = bf16_problem(B, H, L, L, D, 85, "normal")
    c, s = ol.rope_cache(L, D, base)
    if pe == ol.PE_ROPE_Q_ONLY:
        kr = ol.from_bf16_bits(ol.to_bf16_bits(ol.apply_rope(up[1], base=base)))
        want = ol.attention(up[0], up[1], up[2], pe=ol.PE_ROPE_INTERLEAVED, base=base)
        kbits = ol.to_bf16_bits(kr)
    else:
        want = ol.attention(*up, pe=pe, base=base)
        kbits = bits[1]
    got = bf16_from_dev(pkg.forward(bf16_to_dev(bits[0], cuda), bf16_to_dev(kbits, cuda), bf16_to_dev(bits[2], cuda), pe=pe,
                                    cos_cache=to_dev(c, cuda), sin_cache=to_dev(s, cuda)))
    assert pkg.last_path() == "tc_wide"
    err = float(np.abs(got - want).max())
    assert err <= 8e-3, err
