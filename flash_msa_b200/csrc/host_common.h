// Host-side helpers shared by the C-ABI entry points: status codes and launch checking.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/flash_msa_b200.h"

namespace fmsa {

inline int check_launch() {
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FMSA_OK : FMSA_ERR_CUDA;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

}  // namespace fmsa

#define FMSA_REQUIRE(cond)                     \
    do {                                       \
        if (!(cond)) return FMSA_ERR_ARGUMENT; \
    } while (0)
