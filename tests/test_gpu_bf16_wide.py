"""GPU parity of the wide-head tensor-core path (head_d > 512, or rotate-half RoPE): score tiles by
tcgen05 with both operands streamed, scores kept relative to tile maxima, then P V per block of
output columns.  Oracle: fp32 CPU attention on the bf16-rounded inputs, max-abs <= 2e-2."""
import os

import numpy as np
import pytest

import oracle_lib as ol
from gpu_util import bf16_from_dev, bf16_problem, bf16_to_dev

pytestmark = pytest.mark.gpu
TOL = 2e-2


def run(pkg, cuda, bits, **kw):
    q, k, v = (bf16_to_dev(b, cuda) for b in bits)
    return bf16_from_dev(pkg.forward(q, k, v, **kw))


@pytest.mark.parametrize("pe", [ol.PE_NONE, ol.PE_ROPE_HALF], ids=["plain", "rope_half"])
@pytest.mark.parametrize("shape", [
    (1, 1, 128, 128, 1024),     # one tile, half-filled key tile
    (1, 2, 256, 256, 1024),
    (2, 3, 512, 512, 1024),     # more query tiles than key tiles
    (1, 2, 256, 1024, 1024),    # more key tiles than query tiles
    (1, 2, 384, 128, 1024),     # a single key tile
    (1, 2, 128, 768, 1024),     # a single query tile
    (1, 1, 256, 384, 768),      # output column blocks of 384, odd number of key blocks
    (1, 1, 128, 256, 640),      # output column blocks of 320 (MMA N = 256 + 64)
    (1, 1, 128, 256, 2048),     # four output column blocks
    (1, 3, 256, 256, 256),      # narrow head: only rotate-half comes here
    (1, 2, 256, 512, 1024),     # as many query tiles as key tiles: pairing q mod nkt, positions not shared
    (1, 1, 640, 256, 1024),     # five query tiles on one key tile
    (1, 1, 768, 512, 512),      # six query tiles on two key tiles
], ids=lambda s: "x".join(map(str, s)))
def test_wide_path_against_oracle(pkg, cuda, pe, shape):
    B, H, Lq, Lk, D = shape
    bits, up = bf16_problem(B, H, Lq, Lk, D, 71, "normal")
    want = ol.attention(*up, pe=pe)
    got = run(pkg, cuda, bits, pe=pe)
    if D > 512 or pe == ol.PE_ROPE_HALF:
        assert pkg.last_path() == "tc_wide"
    err = float(np.abs(got - want).max())
    assert err <= TOL, (shape, pe, err)
    assert err <= 8e-3, (shape, pe, err)   # far inside the tolerance on these sizes


def test_wide_path_in_several_passes_over_the_heads(pkg, cuda):
    """A small scratch cap makes the library process the heads in groups."""
    B, H, L, D = 1, 5, 512, 1024
    bits, up = bf16_problem(B, H, L, L, D, 72, "normal")
    want = ol.attention(*up, pe=ol.PE_ROPE_HALF)
    pkg.set_option(pkg.OPT_SCORE_SCRATCH_MB, 1)   # 512 x 512 bf16 scores are 512 KiB per head: two heads per pass
    try:
        got = run(pkg, cuda, bits, pe=ol.PE_ROPE_HALF)
    finally:
        pkg.set_option(pkg.OPT_SCORE_SCRATCH_MB, 2048)
    assert pkg.last_path() == "tc_wide"
    assert float(np.abs(got - want).max()) <= 8e-3


def test_wide_path_twice_in_a_row_same_result(pkg, cuda):
    bits, up = bf16_problem(1, 4, 256, 512, 1024, 73, "normal")
    a = run(pkg, cuda, bits, pe=ol.PE_ROPE_HALF)
    b = run(pkg, cuda, bits, pe=ol.PE_ROPE_HALF)
    assert np.array_equal(a, b)


@pytest.mark.parametrize("pe", [ol.PE_SINUSOIDAL, ol.PE_ROPE_INTERLEAVED], ids=["sinusoidal", "rope_pairs"])
@pytest.mark.parametrize("shape", [
    (1, 2, 256, 256, 1024),
    (1, 2, 512, 256, 1024),
    (1, 1, 128, 768, 1024),
    (1, 1, 256, 384, 768),
    (1, 1, 128, 256, 2048),
], ids=lambda s: "x".join(map(str, s)))
def test_wide_path_other_encodings(pkg, cuda, pe, shape):
    B, H, Lq, Lk, D = shape
    bits, up = bf16_problem(B, H, Lq, Lk, D, 74, "normal")
    want = ol.attention(*up, pe=pe)
    got = run(pkg, cuda, bits, pe=pe)
    assert pkg.last_path() == "tc_wide"
    err = float(np.abs(got - want).max())
    assert err <= TOL, (shape, pe, err)


def test_wide_path_partial_rotary_dim_and_q_only(pkg, cuda):
    B, H, L, D, rd = 1, 2, 256, 1024, 256
    bits, up = bf16_problem(B, H, L, L, D, 75, "normal")
    for pe in (ol.PE_ROPE_INTERLEAVED, ol.PE_ROPE_Q_ONLY):
        want = ol.attention(*up, pe=pe, rotary_dim=rd)
        got = run(pkg, cuda, bits, pe=pe, rotary_dim=rd)
        assert pkg.last_path() == "tc_wide"
        assert float(np.abs(got - want).max()) <= TOL, pe


@pytest.mark.parametrize("pe", [ol.PE_NONE, ol.PE_SINUSOIDAL, ol.PE_ROPE_INTERLEAVED, ol.PE_ROPE_HALF])
def test_narrow_heads_on_the_two_kernel_path(pkg, cuda, pe):
    """head_d <= 512 runs here too (the one-kernel pipeline only when asked for)."""
    bits, up = bf16_problem(1, 3, 384, 512, 512, 76, "normal")
    want = ol.attention(*up, pe=pe)
    got = run(pkg, cuda, bits, pe=pe)
    assert pkg.last_path() == "tc_wide"
    assert float(np.abs(got - want).max()) <= TOL
