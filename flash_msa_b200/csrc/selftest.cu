// Known-answer hook for the tensor-core plumbing: one 128x128x128 product computed with exactly
// the device primitives the attention kernels use (swizzled operand tiles filled by cp.async or
// TMA, tcgen05.mma with K-major or MN-major descriptors, a TMEM accumulator, tcgen05.ld).
#include "host_common.h"
#include "sm100.cuh"
#include "tma_host.h"

namespace fmsa {
namespace {

__global__ void __launch_bounds__(128) umma_selftest_kernel(const __nv_bfloat16* __restrict__ a,
                                                            const __nv_bfloat16* __restrict__ b, float* __restrict__ d,
                                                            int a_mn, int b_mn, int use_tma,
                                                            const __grid_constant__ CUtensorMap tmap_a,
                                                            const __grid_constant__ CUtensorMap tmap_b,
                                                            int* __restrict__ status) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // dynamic shared memory is only guaranteed 16-byte aligned: align by hand
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t tile_a = base, tile_b = base + kTileBytes;
    __shared__ __align__(8) uint64_t bars[2];
    __shared__ uint32_t tmem_slot;
    const int tid = threadIdx.x, warp = tid >> 5;
    const uint32_t bar_mma = smem_u32(&bars[0]), bar_tma = smem_u32(&bars[1]);

    if (tid == 0) {
        mbar_init(bar_mma, 1);
        mbar_init(bar_tma, 1);
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(&tmem_slot), 128);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_slot;

    bool ok = true;
    if (use_tma) {
        if (tid == 0) {
            mbar_arrive_expect_tx(bar_tma, 2 * kTileBytes);
            tma_load_2d(tile_a, &tmap_a, 0, 0, bar_tma);
            tma_load_2d(tile_a + kPanelBytes, &tmap_a, 64, 0, bar_tma);
            tma_load_2d(tile_b, &tmap_b, 0, 0, bar_tma);
            tma_load_2d(tile_b + kPanelBytes, &tmap_b, 64, 0, bar_tma);
        }
        ok = mbar_wait(bar_tma, 0);
    } else {
        load_tile_async<128>(tile_a, a, 128, tid);
        load_tile_async<128>(tile_b, b, 128, tid);
        cp_async_commit();
        cp_async_wait<0>();
        fence_async_smem();
    }
    if (__syncthreads_or(!ok)) {
        if (tid == 0) atomicMax(status, kStatusWaitTimeout);
    } else {
        if (tid == 0) {
            tc_fence_after_sync();
            if (a_mn) {
                if (b_mn) umma_tile_128<true, true>(tmem, tile_a, tile_b, false);
                else umma_tile_128<true, false>(tmem, tile_a, tile_b, false);
            } else {
                if (b_mn) umma_tile_128<false, true>(tmem, tile_a, tile_b, false);
                else umma_tile_128<false, false>(tmem, tile_a, tile_b, false);
            }
            umma_commit(bar_mma);
        }
        ok = mbar_wait(bar_mma, 0);
        if (__syncthreads_or(!ok)) {
            if (tid == 0) atomicMax(status, kStatusWaitTimeout);
        } else {
            tc_fence_after_sync();
            const int row = warp * 32 + (tid & 31);
#pragma unroll 1
            for (int c = 0; c < 128; c += 32) {
                uint32_t r[32];
                tmem_ld32(tmem_addr(tmem, warp, c), r);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) d[row * 128 + c + i] = __uint_as_float(r[i]);
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 128);
}

}  // namespace
}  // namespace fmsa

extern "C" int fmsa_abi_version(void) { return 2; }

extern "C" int fmsa_umma_selftest(const void* a, const void* b, float* d, int a_mn, int b_mn, int use_tma, int* status,
                                  void* stream) {
    using namespace fmsa;
    FMSA_REQUIRE(a && b && d && status);
    FMSA_REQUIRE(aligned16(a) && aligned16(b));
    CUtensorMap ta, tb;
    memset(&ta, 0, sizeof(ta));
    memset(&tb, 0, sizeof(tb));
    if (use_tma) {
        if (!make_tmap_rows(&ta, a, 128, 256, 128) || !make_tmap_rows(&tb, b, 128, 256, 128)) return FMSA_ERR_CUDA;
    }
    const size_t smem = 2 * kTileBytes + 1024;
    if (cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) !=
        cudaSuccess)
        return FMSA_ERR_CUDA;
    umma_selftest_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), d, a_mn, b_mn, use_tma, ta, tb, status);
    return check_launch();
}
