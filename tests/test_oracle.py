"""CPU tests of the oracle: it must agree with every golden vector the reference holds for the
path (its torch SDPA vectors), with outputs of the reference's own CPU routines (committed
fixtures, and live when oracle/_ref is built), and with itself under the identities used to
cover what the reference has no vectors for (rotate-half pairing, sampled rows, bf16 rounding)."""
import glob
import os

import numpy as np
import pytest

import oracle_lib as ol

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
KIND_PE = {"plain": ol.PE_NONE, "rope": ol.PE_ROPE_INTERLEAVED, "sinus": ol.PE_SINUSOIDAL}


def load_refcpu(path):
    z = np.load(path)
    B, H, Lq, Lk, D = (int(x) for x in z["shape"])
    return str(z["kind"]), (B, H, Lq, Lk, D), int(z["seed"]), z["rows"], z["out_rows"]


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLD, "sdpa_*.npz"))), ids=os.path.basename)
def test_oracle_matches_reference_sdpa_golden(path):
    z = np.load(path)
    out = ol.attention(z["Q"], z["K"], z["V"])
    # the goldens came from torch SDPA (different summation order): 5e-6 abs is fp32 round-off here
    assert np.abs(out - z["output"]).max() < 5e-6
    # and against a float64 recompute of the same inputs
    Q, K, V = (z[k].astype(np.float64) for k in ("Q", "K", "V"))
    s = np.einsum("bhid,bhjd->bhij", Q, K) / np.sqrt(Q.shape[-1])
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    assert np.abs(out - np.einsum("bhij,bhjd->bhid", p, V)).max() < 5e-6


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLD, "refcpu_*.npz"))), ids=os.path.basename)
def test_oracle_bit_exact_with_reference_cpu_fixture(path):
    kind, (B, H, Lq, Lk, D), seed, rows, want = load_refcpu(path)
    Q, K, V = ol.make_qkv(B, H, Lq, Lk, D, seed, "uniform")
    out = ol.attention(Q, K, V, pe=KIND_PE[kind])
    assert np.array_equal(out[:, :, rows, :], want)


def test_fixture_count():
    assert len(glob.glob(os.path.join(GOLD, "sdpa_*.npz"))) == 6
    assert len(glob.glob(os.path.join(GOLD, "refcpu_*.npz"))) >= 25


@pytest.mark.parametrize("shape", [(1, 2, 8, 8, 16), (2, 3, 17, 29, 40), (1, 1, 64, 64, 256)])
def test_oracle_bit_exact_with_live_reference(shape):
    ref = ol.ref()
    if ref is None:
        pytest.skip("oracle/_ref not built (reference tree absent)")
    B, H, Lq, Lk, D = shape
    Q, K, V = ol.make_qkv(B, H, Lq, Lk, D, 7, "uniform")
    f = ol._f
    out = np.empty_like(Q)
    ref.ref_attention_cpu(f(Q), f(K), f(V), f(out), B, H, Lq, Lk, D)
    assert np.array_equal(out, ol.attention(Q, K, V))
    L = max(Lq, Lk)
    c = np.empty((L, D), np.float32); s = np.empty((L, D), np.float32)
    ref.ref_precompute_rope_cache(f(c), f(s), L, D, 10000.0)
    c2, s2 = ol.rope_cache(L, D)
    assert np.array_equal(c, c2) and np.array_equal(s, s2)
    ref.ref_attention_rope_cpu(f(Q), f(K), f(V), f(out), f(c), f(s), B, H, Lq, Lk, D)
    assert np.array_equal(out, ol.attention(Q, K, V, pe=ol.PE_ROPE_INTERLEAVED))
    st = np.empty((L, D), np.float32); ct = np.empty((L, D), np.float32)
    ref.ref_generate_sinusoidal_embeddings_cpu(f(st), f(ct), L, D)
    st2, ct2 = ol.sinusoidal_tables(L, D)
    assert np.array_equal(st, st2) and np.array_equal(ct, ct2)
    ref.ref_attention_sinusoidal_cpu(f(Q), f(K), f(V), f(st), f(ct), f(out), B, H, Lq, Lk, D)
    assert np.array_equal(out, ol.attention(Q, K, V, pe=ol.PE_SINUSOIDAL))


def test_rotate_half_equals_interleaved_under_column_permutation():
    B, H, L, D = 1, 2, 24, 64
    Q, K, V = ol.make_qkv(B, H, L, L, D, 11, "uniform")
    perm = np.empty(D, dtype=np.int64)
    perm[0::2] = np.arange(D // 2)
    perm[1::2] = np.arange(D // 2) + D // 2
    a = ol.attention(Q, K, V, pe=ol.PE_ROPE_HALF)
    b = ol.attention(np.ascontiguousarray(Q[..., perm]), np.ascontiguousarray(K[..., perm]), V, pe=ol.PE_ROPE_INTERLEAVED)
    assert np.abs(a - b).max() < 2e-6


def test_partial_rotation_leaves_tail_columns_alone():
    B, H, L, D, rd = 1, 1, 8, 32, 16
    Q, K, V = ol.make_qkv(B, H, L, L, D, 12, "uniform")
    a = ol.attention(Q, K, V, pe=ol.PE_ROPE_INTERLEAVED, rotary_dim=rd)
    # rotating only the first rd columns == full rotation of a problem whose tail scores are added unrotated
    c, s = ol.rope_cache(L, rd)
    def rot(X):
        Y = X.copy()
        Y[..., 0:rd:2] = X[..., 0:rd:2] * c[:, 0::2] - X[..., 1:rd:2] * s[:, 0::2]
        Y[..., 1:rd:2] = X[..., 0:rd:2] * s[:, 0::2] + X[..., 1:rd:2] * c[:, 0::2]
        return Y
    b = ol.attention(rot(Q), rot(K), V)
    assert np.abs(a - b).max() < 1e-6
    # q-only kind: K is taken as given
    d = ol.attention(Q, rot(K), V, pe=ol.PE_ROPE_Q_ONLY, rotary_dim=rd)
    assert np.abs(a - d).max() < 1e-6


def test_sampled_rows_equal_full_evaluation():
    B, H, Lq, Lk, D = 2, 2, 12, 20, 32
    Q, K, V = ol.make_qkv(B, H, Lq, Lk, D, 13, "normal")
    bh = np.array([0, 0, 2, 3, 3]); rows = np.array([0, 11, 5, 1, 7])
    for pe in (ol.PE_NONE, ol.PE_ROPE_INTERLEAVED, ol.PE_ROPE_HALF, ol.PE_SINUSOIDAL):
        full = ol.attention(Q, K, V, pe=pe).reshape(B * H, Lq, D)
        got = ol.attention_rows(Q, K, V, bh, rows, pe=pe)
        assert np.array_equal(got, full[bh, rows])


def test_bf16_rounding_is_round_to_nearest_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.0e38, 1e-40, 0.0], dtype=np.float32)
    bits = ol.to_bf16_bits(x)
    back = ol.from_bf16_bits(bits)
    import torch
    want = torch.from_numpy(x).to(torch.bfloat16).float().numpy()
    assert np.array_equal(back, want)
    r = np.random.default_rng(0).standard_normal(4096).astype(np.float32)
    assert np.array_equal(ol.from_bf16_bits(ol.to_bf16_bits(r)), torch.from_numpy(r).to(torch.bfloat16).float().numpy())


def test_synthetic_generator_numpy_equals_c():
    n = 1000
    import ctypes as C
    a = np.empty(n, np.float32)
    ol.oracle().oracle_fill_uniform(ol._f(a), n, 43, 2, 0)
    assert np.array_equal(a, ol.synth_uniform((n,), 43, 2))
    assert a.min() >= -1.0 and a.max() < 1.0 and abs(float(a.mean())) < 0.1
    g = ol.synth_normal((20000,), 44, 1)
    assert abs(float(g.mean())) < 0.03 and abs(float(g.std()) - 1.0) < 0.03 and np.isfinite(g).all()


def test_compare_rule():
    want = np.array([1.0, 0.0, 1e-6], np.float32)
    assert ol.compare(want + np.float32(5e-5), want)["ok"]
    assert not ol.compare(want + np.float32(2e-4), want)["ok"]
