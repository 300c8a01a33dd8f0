"""GPU parity of the decode / cross-attention regime (few queries, many keys; bf16): key splits on the
tensor cores plus the combine kernel, against the fp32 CPU oracle on the bf16-rounded inputs.  Tolerance
(stated by the task for bf16): max-abs <= 2e-2; a tighter bound is asserted as well."""
import numpy as np
import pytest

import oracle_lib as ol
from gpu_util import bf16_from_dev, bf16_problem, bf16_to_dev, to_dev

pytestmark = pytest.mark.gpu
TOL = 2e-2


def run(pkg, cuda, bits, **kw):
    q, k, v = (bf16_to_dev(b, cuda) for b in bits)
    return bf16_from_dev(pkg.forward(q, k, v, **kw))


@pytest.mark.parametrize("shape", [(1, 32, 1, 8192, 128), (1, 32, 4, 32768, 128), (2, 3, 64, 1000, 128), (1, 5, 7, 129, 64),
                                   (1, 160, 3, 700, 128), (1, 1, 16, 5000, 64)], ids=str)
def test_decode_plain(pkg, cuda, shape):
    B, H, Lq, Lk, D = shape
    bits, up = bf16_problem(B, H, Lq, Lk, D, 91, "normal")
    got = run(pkg, cuda, bits)
    assert pkg.last_path() == "tc_decode"
    err = float(np.abs(got - ol.attention(*up)).max())
    assert err <= 4e-3, (shape, err)
    # a second call right after (scratch and rings reused)
    assert float(np.abs(run(pkg, cuda, bits) - got).max()) == 0.0


@pytest.mark.parametrize("pe", [ol.PE_ROPE_INTERLEAVED, ol.PE_ROPE_HALF, ol.PE_SINUSOIDAL], ids=["interleaved", "half", "sinusoidal"])
@pytest.mark.parametrize("shape", [(1, 32, 1, 8192, 128), (1, 8, 4, 32768, 128), (1, 6, 33, 900, 128)], ids=str)
def test_decode_with_the_encoding_applied_in_the_load(pkg, cuda, pe, shape):
    """Positions: query row i -> i, key j -> j (final/rope.cu:129, 307), K encoded chunk by chunk between TMA
    arrival and MMA."""
    B, H, Lq, Lk, D = shape
    bits, up = bf16_problem(B, H, Lq, Lk, D, 92, "normal")
    got = run(pkg, cuda, bits, pe=pe)
    assert pkg.last_path() == "tc_decode"
    err = float(np.abs(got - ol.attention(*up, pe=pe)).max())
    assert err <= TOL and err <= 1.5e-2, (shape, pe, err)


@pytest.mark.parametrize("half", [False, True], ids=["interleaved", "half"])
def test_decode_on_a_rotated_key_cache(pkg, cuda, half):
    """The KV-cache use: K rotated once by b200attn_rope_k, attention rotates the queries only; partial
    rotary_dim for the interleaved pairing; D = 64 for it as well."""
    for (B, H, Lq, Lk, D, rd) in [(1, 16, 2, 4096, 128, 0), (1, 4, 5, 3000, 128, 0 if half else 64), (1, 4, 1, 2048, 64, 0)]:
        if half and D != 128:
            continue
        bits, up = bf16_problem(B, H, Lq, Lk, D, 93, "normal")
        want = ol.attention(*up, pe=ol.PE_ROPE_HALF if half else ol.PE_ROPE_INTERLEAVED, rotary_dim=(rd or None))
        q, k, v = (bf16_to_dev(b, cuda) for b in bits)
        kr = pkg.rope_k(k, pairing=pkg.PE_ROPE_HALF if half else pkg.PE_ROPE_INTERLEAVED, rotary_dim=rd)
        got = bf16_from_dev(pkg.forward(q, kr, v, pe=pkg.PE_ROPE_HALF_Q_ONLY if half else pkg.PE_ROPE_Q_ONLY, rotary_dim=rd))
        assert pkg.last_path() == "tc_decode"
        err = float(np.abs(got - want).max())
        assert err <= 8e-3, ((B, H, Lq, Lk, D, rd), err)


def test_decode_with_caller_caches(pkg, cuda):
    B, H, Lq, Lk, D, base = 1, 8, 3, 2000, 128, 777.0
    bits, up = bf16_problem(B, H, Lq, Lk, D, 94, "normal")
    c, s = ol.rope_cache(Lk, D, base)
    for pe in (ol.PE_ROPE_INTERLEAVED, ol.PE_ROPE_HALF):
        got = run(pkg, cuda, bits, pe=pe, cos_cache=to_dev(c, cuda), sin_cache=to_dev(s, cuda))
        assert pkg.last_path() == "tc_decode"
        err = float(np.abs(got - ol.attention(*up, pe=pe, base=base)).max())
        assert err <= 8e-3, (pe, err)


def test_wide_head_cross_attention_runs_on_the_general_path(pkg, cuda):
    """head_d 512 with few queries is outside the decode kernel (head_d 64 / 128): it runs, correctly, on the
    split-head_d kernels."""
    B, H, Lq, Lk, D = 4, 8, 16, 4096, 512
    bits, up = bf16_problem(B, H, Lq, Lk, D, 95, "normal")
    for pe in (ol.PE_ROPE_INTERLEAVED, ol.PE_ROPE_HALF):
        got = run(pkg, cuda, bits, pe=pe)
        err = float(np.abs(got - ol.attention(*up, pe=pe)).max())
        assert err <= TOL, (pe, pkg.last_path(), err)
