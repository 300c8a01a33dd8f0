#!/usr/bin/env python3
"""Generates the committed golden fixtures in this folder.  Needs the reference tree (read-only)
and oracle/_ref built from it; run once in the development container:

    python tests/golden/make_golden.py

Two kinds of fixtures:

  sdpa_<name>.npz      the reference's own golden vectors (pytorch_reference_data/*.bin: fp32
                       inputs and torch SDPA outputs).  tiny/small are kept whole; of the
                       hdim* sets head 0 is kept with all its keys/values and the leading
                       32768/head_d query rows (heads and query rows are independent).
  refcpu_<case>.npz    outputs of the reference's own CPU routines (attention_cpu,
                       attention_rope_cpu, attention_sinusoidal_cpu) on this repo's counter-based
                       synthetic inputs, for the reference's test shape lists.  Inputs are not
                       stored (they are regenerated from the seed); of the output only a few rows
                       per (b,h) are stored for the large shapes.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import oracle_lib as ol  # noqa: E402

# the reference project's tree: B200ATTN_REFERENCE_ROOT, else a directory `reference` beside this repository
REF = os.environ.get("B200ATTN_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference")

SDPA_SETS = [  # scripts/generate_pytorch_reference.py:87-94
    (1, 1, 4, 8, "tiny"), (1, 2, 8, 16, "small"), (1, 4, 64, 512, "hdim512"),
    (1, 4, 64, 2048, "hdim2048"), (1, 2, 32, 4096, "hdim4096"), (1, 1, 16, 8192, "hdim8192"),
]

# (name, kind, B, H, Lq, Lk, D, seed); shapes from final/attention.cu:488-522, final/rope.cu:1917-1928,
# final/sinusoidal.cu:1270-1276, plus the cross-attention and head_d sweep shapes of the benchmark configs
REFCPU_CASES = [
    ("plain_1_1_4_8", "plain", 1, 1, 4, 4, 8, 101),
    ("plain_1_2_8_16", "plain", 1, 2, 8, 8, 16, 102),
    ("plain_2_4_32_32", "plain", 2, 4, 32, 32, 32, 103),
    ("plain_2_8_64_64", "plain", 2, 8, 64, 64, 64, 104),
    ("plain_cross_1_2_16_32_32", "plain", 1, 2, 16, 32, 32, 105),
    ("plain_1_4_16_64", "plain", 1, 4, 16, 16, 64, 106),
    ("plain_2_8_64_128", "plain", 2, 8, 64, 64, 128, 107),
    ("plain_1_4_64_512", "plain", 1, 4, 64, 64, 512, 108),
    ("plain_1_4_64_2048", "plain", 1, 4, 64, 64, 2048, 43),
    ("plain_1_4_64_4096", "plain", 1, 4, 64, 64, 4096, 109),
    ("plain_1_4_64_8192", "plain", 1, 4, 64, 64, 8192, 110),
    ("plain_cross_1_4_32_64_4096", "plain", 1, 4, 32, 64, 4096, 111),
    ("plain_1_2_32_4096", "plain", 1, 2, 32, 32, 4096, 112),
    ("plain_1_1_16_8192", "plain", 1, 1, 16, 16, 8192, 113),
    ("plain_1_2_200_96", "plain", 1, 2, 200, 136, 96, 114),
    ("rope_1_1_4_8", "rope", 1, 1, 4, 4, 8, 201),
    ("rope_1_2_8_16", "rope", 1, 2, 8, 8, 16, 202),
    ("rope_2_4_32_32", "rope", 2, 4, 32, 32, 32, 203),
    ("rope_1_4_16_64", "rope", 1, 4, 16, 16, 64, 204),
    ("rope_1_4_64_128", "rope", 1, 4, 64, 64, 128, 205),
    ("rope_1_4_64_512", "rope", 1, 4, 64, 64, 512, 206),
    ("rope_1_4_64_2048", "rope", 1, 4, 64, 64, 2048, 207),
    ("rope_cross_1_2_16_48_64", "rope", 1, 2, 16, 48, 64, 208),
    ("sinus_1_4_64_512", "sinus", 1, 4, 64, 64, 512, 301),
    ("sinus_1_4_64_2048", "sinus", 1, 4, 64, 64, 2048, 302),
    ("sinus_1_2_32_4096", "sinus", 1, 2, 32, 32, 4096, 303),
    ("sinus_1_2_8_16", "sinus", 1, 2, 8, 8, 16, 304),
    ("sinus_cross_1_2_16_48_64", "sinus", 1, 2, 16, 48, 64, 305),
]
MAX_FULL = 1 << 16  # outputs up to this many elements are stored whole


def kept_rows(Lq):
    return sorted(set([0, 1, Lq // 2, Lq - 1]) & set(range(Lq)))


def ref_cpu(kind, Q, K, V):
    lib = ol.ref()
    B, H, Lq, D = Q.shape
    Lk = K.shape[2]
    out = np.empty_like(Q)
    f = ol._f
    if kind == "plain":
        lib.ref_attention_cpu(f(Q), f(K), f(V), f(out), B, H, Lq, Lk, D)
    elif kind == "rope":
        L = max(Lq, Lk)
        c = np.empty((L, D), np.float32)
        s = np.empty((L, D), np.float32)
        lib.ref_precompute_rope_cache(f(c), f(s), L, D, 10000.0)
        lib.ref_attention_rope_cpu(f(Q), f(K), f(V), f(out), f(c), f(s), B, H, Lq, Lk, D)
    elif kind == "sinus":
        L = max(Lq, Lk)
        st = np.empty((L, D), np.float32)
        ct = np.empty((L, D), np.float32)
        lib.ref_generate_sinusoidal_embeddings_cpu(f(st), f(ct), L, D)
        lib.ref_attention_sinusoidal_cpu(f(Q), f(K), f(V), f(st), f(ct), f(out), B, H, Lq, Lk, D)
    else:
        raise ValueError(kind)
    return out


def main():
    assert ol.ref() is not None, "build oracle/_ref first (python oracle/build.py)"
    for b, h, l, d, name in SDPA_SETS:
        arrs = {}
        for t in ("Q", "K", "V", "output"):
            a = np.fromfile(os.path.join(REF, "pytorch_reference_data", f"pytorch_ref_{name}_{t}.bin"),
                            dtype=np.float32).reshape(b, h, l, d)
            if a.size > (1 << 15):
                a = a[:, :1]                      # head 0 only (heads are independent)
                if t in ("Q", "output"):
                    a = a[:, :, :max(1, (1 << 15) // d)]  # leading query rows only (rows are independent)
            arrs[t] = np.ascontiguousarray(a)
        np.savez(os.path.join(HERE, f"sdpa_{name}.npz"), **arrs)
        print("sdpa", name, arrs["Q"].shape)
    for name, kind, B, H, Lq, Lk, D, seed in REFCPU_CASES:
        Q, K, V = ol.make_qkv(B, H, Lq, Lk, D, seed, "uniform")
        out = ref_cpu(kind, Q, K, V)
        if out.size <= MAX_FULL:
            rows = np.arange(Lq)
        else:
            rows = np.array(kept_rows(Lq))
        np.savez(os.path.join(HERE, f"refcpu_{name}.npz"), kind=kind, shape=np.array([B, H, Lq, Lk, D]),
                 seed=seed, rows=rows, out_rows=np.ascontiguousarray(out[:, :, rows, :]))
        print("refcpu", name, out[:, :, rows, :].shape)


if __name__ == "__main__":
    main()
