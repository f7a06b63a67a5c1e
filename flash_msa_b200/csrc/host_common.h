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

// Head-count relations every entry point relies on (the reference checks the same ones in
// flash_msa/flash_msa.py:44-53 and flash_msa/warmup/flash_msa_warmup.py:34-43).
inline bool problem_ok(const fmsa_problem* pb) {
    return pb && pb->B > 0 && pb->S > 0 && pb->S % 128 == 0 && pb->Hq > 0 && pb->Hkv > 0 && pb->Hp > 0 && pb->Hpkv > 0 &&
           pb->Hq % pb->Hkv == 0 && pb->Hq % pb->Hp == 0 && pb->Hp % pb->Hpkv == 0 && pb->Hp % pb->Hkv == 0 &&
           (pb->dtype == FMSA_DTYPE_BF16 || pb->dtype == FMSA_DTYPE_FP16);
}

// Per-device facts that never change are looked up once (the launchers run on the critical path of every step).
inline int device_sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    if (cached[dev] == 0) {
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
        cached[dev] = sms;
    }
    return cached[dev];
}
// Raises a kernel's dynamic shared-memory limit once per (kernel, device).  Up to 16 kernels.
inline bool ensure_smem_attr(const void* func, size_t bytes) {
    struct Entry { const void* f; unsigned long long done; };
    static Entry table[16] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    for (auto& e : table) {
        if (e.f == func || e.f == nullptr) {
            if (e.f == func && (e.done >> dev & 1ull)) return true;
            if (cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)) != cudaSuccess)
                return false;
            e.f = func;
            e.done |= 1ull << dev;
            return true;
        }
    }
    return cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)) == cudaSuccess;
}

inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

}  // namespace fmsa

#define FMSA_REQUIRE(cond)                     \
    do {                                       \
        if (!(cond)) return FMSA_ERR_ARGUMENT; \
    } while (0)
