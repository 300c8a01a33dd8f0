"""b200attn: thin ctypes binding of lib/libb200attn.so (the C ABI of include/b200attn.h).

This module is host-side convenience for the tests and the benchmark: it passes torch device
pointers to the C entry points.  All arithmetic is in the CUDA library; there is no fallback, and
loading fails when the shared library has not been built.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# B200ATTN_LIB names another build of the same library (a profiling build, an older build to compare with)
LIB_PATH = os.environ.get("B200ATTN_LIB") or os.path.join(_HERE, "lib", "libb200attn.so")

F32, BF16, F16 = 0, 1, 2
PE_NONE, PE_ROPE_INTERLEAVED, PE_ROPE_HALF, PE_SINUSOIDAL, PE_ROPE_Q_ONLY, PE_ROPE_HALF_Q_ONLY = 0, 1, 2, 3, 4, 5
FLAG_ASYNC, FLAG_FORCE_GENERIC, FLAG_FORCE_TWO_PASS, FLAG_PREFER_ONE_KERNEL, FLAG_NO_OVERLAP, FLAG_TWO_KERNELS = 1, 2, 4, 8, 16, 32
OPT_SCORE_SCRATCH_MB, OPT_SPIN_LIMIT = 1, 2
OK = 0

# every symbol include/b200attn.h declares (checked by the CPU test-suite against the header)
DROP_IN_SYMBOLS = (
    "attention_forward_optimized", "attention_forward_bf16", "attention_forward_rope_fused_v2",
    "attention_forward_rope_fused", "attention_forward_rope_fused_v7_hybrid", "attention_forward_rope_bf16",
    "attention_forward_rope_bf16_v7", "attention_forward_sinusoidal_fused", "attention_forward_sinusoidal_bf16",
)


class Args(C.Structure):
    _fields_ = [
        ("struct_size", C.c_size_t),
        ("Q", C.c_void_p), ("K", C.c_void_p), ("V", C.c_void_p), ("out", C.c_void_p),
        ("batch_sz", C.c_int), ("num_heads", C.c_int), ("len_q", C.c_int), ("len_k", C.c_int), ("head_d", C.c_int),
        ("dtype", C.c_int), ("pe", C.c_int), ("rotary_dim", C.c_int), ("rope_base", C.c_float),
        ("cos_cache", C.c_void_p), ("sin_cache", C.c_void_p),
        ("stream", C.c_void_p), ("flags", C.c_uint),
    ]


class B200AttnError(RuntimeError):
    def __init__(self, status, message):
        super().__init__(f"b200attn status {status}: {message}")
        self.status = status


_lib = None


def lib():
    """The loaded shared library (raises if it has not been built: there is no CPU path)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(f"{LIB_PATH} is missing: run `python accelerated-final-project_b200/build.py`")
        L = C.CDLL(LIB_PATH)
        five = [C.c_int] * 5
        for name in ("attention_forward_optimized", "attention_forward_bf16", "attention_forward_rope_fused_v2",
                     "attention_forward_rope_bf16", "attention_forward_sinusoidal_fused", "attention_forward_sinusoidal_bf16"):
            getattr(L, name).argtypes = [C.c_void_p] * 4 + five
            getattr(L, name).restype = None
        L.attention_forward_rope_fused.argtypes = [C.c_void_p] * 6 + five
        L.attention_forward_rope_fused.restype = None
        for name in ("attention_forward_rope_fused_v7_hybrid", "attention_forward_rope_bf16_v7"):
            getattr(L, name).argtypes = [C.c_void_p] * 4 + five + [C.c_int]
            getattr(L, name).restype = None
        L.b200attn_forward_ex.argtypes = [C.POINTER(Args)]
        L.b200attn_forward_ex.restype = C.c_int
        L.b200attn_forward_many.argtypes = [C.POINTER(Args), C.c_int]
        L.b200attn_forward_many.restype = C.c_int
        L.b200attn_forward_host.argtypes = [C.POINTER(Args)]
        L.b200attn_forward_host.restype = C.c_int
        L.b200attn_forward_sharded.argtypes = [C.POINTER(Args), C.c_int, C.POINTER(C.c_int)] + \
            [C.POINTER(C.c_void_p)] * 4 + [C.POINTER(C.c_int)]
        L.b200attn_forward_sharded.restype = C.c_int
        L.b200attn_shard_ranges.argtypes = [C.c_longlong, C.c_int, C.POINTER(C.c_longlong), C.POINTER(C.c_longlong)]
        L.b200attn_shard_ranges.restype = None
        L.b200attn_last_error.restype = C.c_char_p
        L.b200attn_last_path.restype = C.c_char_p
        L.b200attn_launch_count.restype = C.c_ulonglong
        L.b200attn_version.restype = C.c_char_p
        L.b200attn_release_workspace.restype = None
        L.b200attn_forward_static.argtypes = [C.c_void_p] * 4 + [C.c_int] * 5 + [C.c_void_p]
        L.b200attn_forward_static.restype = C.c_int
        L.b200attn_static_last_error.restype = C.c_char_p
        L.b200attn_synth_fill.argtypes = [C.c_void_p, C.c_longlong, C.c_ulonglong, C.c_ulonglong, C.c_longlong,
                                          C.c_int, C.c_int, C.c_void_p]
        L.b200attn_synth_fill.restype = C.c_int
        L.b200attn_rope_k.argtypes = [C.c_void_p, C.c_void_p] + [C.c_int] * 7 + [C.c_float, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
        L.b200attn_rope_k.restype = C.c_int
        L.b200attn_set_option.argtypes = [C.c_int, C.c_longlong]
        L.b200attn_set_option.restype = C.c_int
        L.b200attn_debug_kernel_times.argtypes = [C.c_int, C.POINTER(C.c_double)]
        L.b200attn_debug_kernel_times.restype = C.c_int
        L.b200attn_debug_lost_arrival.argtypes = [C.c_uint, C.c_uint]
        L.b200attn_debug_lost_arrival.restype = None
        _lib = L
    return _lib


def make_args(Q, K, V, out, B, H, Lq, Lk, D, dtype, pe=PE_NONE, rotary_dim=0, rope_base=0.0,
              cos_cache=None, sin_cache=None, stream=None, flags=0):
    """Q, K, V, out, cos_cache, sin_cache are raw addresses (ints)."""
    return Args(C.sizeof(Args), Q, K, V, out, B, H, Lq, Lk, D, dtype, pe, rotary_dim, rope_base,
                cos_cache, sin_cache, stream, flags)


def dtype_of(t):
    import torch
    return {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}[t.dtype]


def check(status):
    if status != OK:
        raise B200AttnError(status, lib().b200attn_last_error().decode())


def forward(Q, K, V, out=None, pe=PE_NONE, rotary_dim=0, rope_base=0.0, cos_cache=None, sin_cache=None,
            stream=None, flags=0):
    """Attention forward on torch CUDA tensors Q [B,H,Lq,D], K/V [B,H,Lk,D] (float32 or bfloat16,
    contiguous) through b200attn_forward_ex.  Returns `out`."""
    import torch
    assert Q.is_cuda and K.is_cuda and V.is_cuda and Q.is_contiguous() and K.is_contiguous() and V.is_contiguous()
    B, H, Lq, D = Q.shape
    Lk = K.shape[2]
    dtype = dtype_of(Q)
    if out is None:
        out = torch.empty_like(Q)
    if stream is None:
        stream = torch.cuda.current_stream(Q.device).cuda_stream
    a = make_args(Q.data_ptr(), K.data_ptr(), V.data_ptr(), out.data_ptr(), B, H, Lq, Lk, D, dtype, pe, rotary_dim,
                  rope_base, cos_cache.data_ptr() if cos_cache is not None else None,
                  sin_cache.data_ptr() if sin_cache is not None else None, stream, flags)
    with torch.cuda.device(Q.device):
        check(lib().b200attn_forward_ex(C.byref(a)))
    return out


def args_for(Q, K, V, out, pe=PE_NONE, rotary_dim=0, rope_base=0.0, stream=None, flags=0):
    """A filled b200attn_args for torch CUDA tensors (for forward_many)."""
    import torch
    B, H, Lq, D = Q.shape
    if stream is None:
        stream = torch.cuda.current_stream(Q.device).cuda_stream
    return make_args(Q.data_ptr(), K.data_ptr(), V.data_ptr(), out.data_ptr(), B, H, Lq, K.shape[2], D,
                     dtype_of(Q), pe, rotary_dim, rope_base, None, None, stream, flags)


def kernel_times(enable, collect=False):
    """Per-kernel timing of the two-kernel bf16 path (b200attn_debug_kernel_times).  With collect,
    returns {"scores_encode": (ms, launches), "scores": (...), "pv": (...)} for the launches recorded
    since the last collection."""
    out = (C.c_double * 6)() if collect else None
    check(lib().b200attn_debug_kernel_times(1 if enable else 0, out))
    if not collect:
        return None
    return {k: (out[i], int(out[3 + i])) for i, k in enumerate(("scores_encode", "scores", "pv"))}


def forward_many(arg_list):
    """Enqueues a list of b200attn_args through one b200attn_forward_many call."""
    arr = (Args * len(arg_list))(*arg_list)
    check(lib().b200attn_forward_many(arr, len(arg_list)))


def forward_host(Q, K, V, out, pe=PE_NONE, rotary_dim=0, rope_base=0.0, flags=0):
    """Same through b200attn_forward_host: Q, K, V, out are HOST torch tensors (pinned or pageable)."""
    import torch
    B, H, Lq, D = Q.shape
    Lk = K.shape[2]
    dtype = dtype_of(Q)
    a = make_args(Q.data_ptr(), K.data_ptr(), V.data_ptr(), out.data_ptr(), B, H, Lq, Lk, D, dtype, pe, rotary_dim,
                  rope_base, None, None, None, flags)
    check(lib().b200attn_forward_host(C.byref(a)))
    return out


def rope_k(X, out=None, pairing=PE_ROPE_INTERLEAVED, rotary_dim=0, rope_base=0.0, pos0=0, cos_cache=None, sin_cache=None, stream=None):
    """RoPE(X) for a torch CUDA tensor [B,H,L,D] through b200attn_rope_k.  Returns `out`."""
    import torch
    B, H, L, D = X.shape
    if out is None:
        out = torch.empty_like(X)
    if stream is None:
        stream = torch.cuda.current_stream(X.device).cuda_stream
    with torch.cuda.device(X.device):
        check(lib().b200attn_rope_k(X.data_ptr(), out.data_ptr(), B, H, L, D, F32 if X.dtype == torch.float32 else BF16, pairing, rotary_dim,
                                    rope_base, pos0, cos_cache.data_ptr() if cos_cache is not None else None,
                                    sin_cache.data_ptr() if sin_cache is not None else None, stream))
    return out


def set_option(option, value):
    check(lib().b200attn_set_option(option, value))


def shard_ranges(total_bh, n_parts):
    begin = (C.c_longlong * n_parts)()
    count = (C.c_longlong * n_parts)()
    lib().b200attn_shard_ranges(total_bh, n_parts, begin, count)
    return list(begin), list(count)


def synth_fill(t, seed, tensor_id, dist="uniform", index0=0, stream=None):
    """Fills a torch CUDA tensor (float32 / bfloat16) with the library's synthetic inputs."""
    import torch
    dtype = F32 if t.dtype == torch.float32 else BF16
    if stream is None:
        stream = torch.cuda.current_stream(t.device).cuda_stream
    with torch.cuda.device(t.device):
        check(lib().b200attn_synth_fill(t.data_ptr(), t.numel(), seed, tensor_id, index0,
                                        0 if dist == "uniform" else 1, dtype, stream))
    return t


def last_path():
    return lib().b200attn_last_path().decode()


def launch_count():
    return int(lib().b200attn_launch_count())
