// Tensor-core (tcgen05) bf16 forward: placeholder interface while the kernel is brought up.
#pragma once

#include <atomic>

#include "../../include/b200attn.h"
#include "common.cuh"

namespace b200attn {

struct TcTables {
    void release() {}
};

inline bool tc_bf16_supported(const b200attn_args &, int) { return false; }
inline const char *tc_bf16_error() { return ""; }
inline int tc_bf16_run(const b200attn_args &, int, float, TcTables &, unsigned *, int, unsigned, cudaStream_t,
                       std::atomic<unsigned long long> *) {
    return -1;
}

}  // namespace b200attn
