"""ctypes bindings for the CPU oracle (oracle/attn_oracle.c) and, when it has been built, for the
reference project's own code (oracle/_ref/libref_attn.so).  Test infrastructure only."""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import build as oracle_build  # noqa: E402

PE_NONE, PE_ROPE_INTERLEAVED, PE_ROPE_HALF, PE_SINUSOIDAL, PE_ROPE_Q_ONLY = 0, 1, 2, 3, 4
PE_ROPE_HALF_Q_ONLY = 5   # the library rotates Q only; the oracle is given the rotated K (see apply_rope)

_fp = C.POINTER(C.c_float)
_i64 = C.c_longlong


def _f(a):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_fp)


_oracle = None
_ref = None


def oracle():
    global _oracle
    if _oracle is None:
        lib = C.CDLL(oracle_build.build_oracle())
        lib.oracle_attention_f32.argtypes = [_fp] * 4 + [C.c_int] * 5
        lib.oracle_rope_cache.argtypes = [_fp, _fp, C.c_int, C.c_int, C.c_float]
        lib.oracle_sinusoidal_tables.argtypes = [_fp, _fp, C.c_int, C.c_int]
        lib.oracle_attention_pe_f32.argtypes = [_fp] * 4 + [C.c_int] * 5 + [C.c_int, C.c_int, C.c_float, _i64, _i64]
        lib.oracle_attention_pe_f32.restype = C.c_int
        lib.oracle_attention_rope_f32.argtypes = [_fp] * 6 + [C.c_int] * 5
        lib.oracle_attention_sinusoidal_f32.argtypes = [_fp] * 6 + [C.c_int] * 5
        lib.oracle_attention_pe_rows_f32.argtypes = [_fp] * 4 + [C.c_int] * 3 + [C.c_int, C.c_int, C.c_float,
                                                                                C.POINTER(_i64), C.POINTER(C.c_int), C.c_int]
        lib.oracle_round_to_bf16.argtypes = [_fp, C.POINTER(C.c_uint16), _i64]
        lib.oracle_bf16_upcast.argtypes = [C.POINTER(C.c_uint16), _fp, _i64]
        lib.oracle_fill_uniform.argtypes = [_fp, _i64, C.c_uint64, C.c_uint64, _i64]
        lib.oracle_fill_normal.argtypes = [_fp, _i64, C.c_uint64, C.c_uint64, _i64]
        _oracle = lib
    return _oracle


def ref():
    """The reference project's own code, or None when oracle/_ref has not been built."""
    global _ref
    if _ref is None:
        path = oracle_build.build_ref()
        if path is None:
            return None
        lib = C.CDLL(path)
        lib.ref_attention_cpu.argtypes = [_fp] * 4 + [C.c_int] * 5
        lib.ref_precompute_rope_cache.argtypes = [_fp, _fp, C.c_int, C.c_int, C.c_float]
        lib.ref_attention_rope_cpu.argtypes = [_fp] * 6 + [C.c_int] * 5
        lib.ref_generate_sinusoidal_embeddings_cpu.argtypes = [_fp, _fp, C.c_int, C.c_int]
        lib.ref_attention_sinusoidal_cpu.argtypes = [_fp] * 6 + [C.c_int] * 5
        for name in ("ref_attention_forward_optimized", "ref_attention_forward_rope_fused_v2",
                     "ref_attention_forward_bf16", "ref_attention_forward_sinusoidal_bf16"):
            getattr(lib, name).argtypes = [C.c_void_p] * 4 + [C.c_int] * 5
        lib.ref_attention_forward_rope_fused.argtypes = [C.c_void_p] * 6 + [C.c_int] * 5
        lib.ref_attention_forward_rope_fused_v7_hybrid.argtypes = [C.c_void_p] * 4 + [C.c_int] * 6
        lib.ref_attention_forward_sinusoidal_v5.argtypes = [C.c_void_p] * 4 + [C.c_int] * 5
        lib.ref_attention_forward_sinusoidal_v5.restype = C.c_int
        _ref = lib
    return _ref


# ---------------------------------------------------------------------------------------------
# oracle wrappers (numpy in, numpy out)
# ---------------------------------------------------------------------------------------------
def attention(Q, K, V, pe=PE_NONE, rotary_dim=None, base=10000.0):
    """Q [B,H,Lq,D], K/V [B,H,Lk,D] float32 -> out [B,H,Lq,D] float32."""
    B, H, Lq, D = Q.shape
    Lk = K.shape[2]
    rd = D if rotary_dim is None else rotary_dim
    out = np.empty_like(Q)
    rc = oracle().oracle_attention_pe_f32(_f(Q), _f(K), _f(V), _f(out), B, H, Lq, Lk, D, pe, rd, base, 0, B * H)
    assert rc == 0
    return out


def attention_rows(Q, K, V, bh, rows, pe=PE_NONE, rotary_dim=None, base=10000.0):
    """Sampled rows of a large problem: returns [n, D]; (bh[r], rows[r]) must be grouped by bh."""
    B, H, Lq, D = Q.shape
    Lk = K.shape[2]
    rd = D if rotary_dim is None else rotary_dim
    bh = np.ascontiguousarray(bh, dtype=np.int64)
    rows = np.ascontiguousarray(rows, dtype=np.int32)
    out = np.empty((len(bh), D), dtype=np.float32)
    oracle().oracle_attention_pe_rows_f32(_f(Q), _f(K), _f(V), _f(out), Lq, Lk, D, pe, rd, base,
                                          bh.ctypes.data_as(C.POINTER(_i64)),
                                          rows.ctypes.data_as(C.POINTER(C.c_int)), len(bh))
    return out


def rope_cache(max_len, rotary_dim, base=10000.0):
    c = np.empty((max_len, rotary_dim), dtype=np.float32)
    s = np.empty((max_len, rotary_dim), dtype=np.float32)
    oracle().oracle_rope_cache(_f(c), _f(s), max_len, rotary_dim, base)
    return c, s


def apply_rope(X, half=False, rotary_dim=None, base=10000.0, pos0=0):
    """RoPE of every (b,h) slice of X [B,H,L,D] with positions pos0 + l: oracle_apply_rope_interleaved
    (final/rope.cu:1418-1437) or its rotate-half counterpart, on caches from oracle_rope_cache."""
    X = np.ascontiguousarray(X, dtype=np.float32)
    B, H, L, D = X.shape
    rd = D if rotary_dim is None else rotary_dim
    c, s = rope_cache(pos0 + L, rd, base)
    c, s = np.ascontiguousarray(c[pos0:]), np.ascontiguousarray(s[pos0:])
    out = np.empty_like(X)
    fn = oracle().oracle_apply_rope_half if half else oracle().oracle_apply_rope_interleaved
    xf, of = X.reshape(B * H, L, D), out.reshape(B * H, L, D)
    for i in range(B * H):
        fn(_f(xf[i]), _f(of[i]), _f(c), _f(s), L, D, rd)
    return out


def sinusoidal_tables(max_len, D):
    s = np.empty((max_len, D), dtype=np.float32)
    c = np.empty((max_len, D), dtype=np.float32)
    oracle().oracle_sinusoidal_tables(_f(s), _f(c), max_len, D)
    return s, c


def to_bf16_bits(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    oracle().oracle_round_to_bf16(_f(x), out.ctypes.data_as(C.POINTER(C.c_uint16)), x.size)
    return out


def from_bf16_bits(b):
    b = np.ascontiguousarray(b, dtype=np.uint16)
    return (b.astype(np.uint32) << 16).view(np.float32)


# ---------------------------------------------------------------------------------------------
# synthetic inputs: counter-based generator (same arithmetic as oracle_fill_* and the device fill)
# ---------------------------------------------------------------------------------------------
def _splitmix64(x):
    x = (x + np.uint64(0x9E3779B97F4A7C15))
    x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return x ^ (x >> np.uint64(31))


def _counter(n, seed, tensor_id, index0=0):
    with np.errstate(over="ignore"):
        base = (np.uint64(seed) << np.uint64(40)) + (np.uint64(tensor_id) << np.uint64(36)) + np.uint64(index0)
        return _splitmix64(np.arange(n, dtype=np.uint64) + base)


def synth_uniform(shape, seed, tensor_id):
    n = int(np.prod(shape))
    with np.errstate(over="ignore"):
        u = _counter(n, seed, tensor_id)
    v = (u >> np.uint64(40)).astype(np.float32) * np.float32(1.0 / 16777216.0)
    return (np.float32(-1.0) + np.float32(2.0) * v).astype(np.float32).reshape(shape)


def synth_normal(shape, seed, tensor_id):
    """Box-Muller; evaluated by the C oracle so that libm rounding is the same everywhere on the host."""
    n = int(np.prod(shape))
    out = np.empty(n, dtype=np.float32)
    oracle().oracle_fill_normal(_f(out), n, seed, tensor_id, 0)
    return out.reshape(shape)


def make_qkv(B, H, Lq, Lk, D, seed, dist="uniform"):
    gen = synth_uniform if dist == "uniform" else synth_normal
    return (gen((B, H, Lq, D), seed, 0), gen((B, H, Lk, D), seed, 1), gen((B, H, Lk, D), seed, 2))


# ---------------------------------------------------------------------------------------------
# comparison rule: the reference's AND-of-failures test (final/attention.cu:296-331) with the
# tolerances this library is held to (max-abs 1e-4, rel 1e-3 for fp32)
# ---------------------------------------------------------------------------------------------
def compare(got, want, abs_tol=1e-4, rel_tol=1e-3):
    got = np.asarray(got, dtype=np.float32)
    want = np.asarray(want, dtype=np.float32)
    ad = np.abs(got - want)
    rd = ad / (np.abs(want) + np.float32(1e-8))
    bad = int(np.count_nonzero((ad > abs_tol) & (rd > rel_tol)))
    finite = bool(np.isfinite(got).all())
    return {"max_abs": float(ad.max()) if ad.size else 0.0, "bad": bad, "finite": finite,
            "ok": finite and bad == 0 and (float(ad.max()) if ad.size else 0.0) <= abs_tol}
