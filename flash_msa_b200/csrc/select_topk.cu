// Per-row top-k over materialised fp32 block scores: the bandwidth half of block selection.
//
// One warp owns one query row.  The warp keeps its current best `Kb` entries as a sorted list
// spread over the lanes (entry e lives in register e/32 of lane e%32), reads the row's causally
// visible scores 32 at a time, filters them against the current Kb-th entry with one ballot and
// inserts the survivors with shuffle shifts.  The total order is (score descending, block index
// ascending), the row's own block is forced first and unused slots keep the sentinel NB - the
// order and conventions of the reference's register insertion
// (flash_msa/msa_select_cutedsl.py:219-225, 315-317, 370-392).
#include "host_common.h"
#include "sm100.cuh"

namespace fmsa {
namespace {

__device__ __forceinline__ bool beats(float av, int ai, float bv, int bi) {
    return av > bv || (av == bv && ai < bi);
}

template <int KPL>
__global__ void __launch_bounds__(256) topk_rows_kernel(const float* __restrict__ scores, int32_t* __restrict__ out,
                                                        int64_t total_rows, int S, int NB, int Kb) {
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    if (row >= total_rows) return;
    const int q = static_cast<int>(row % S);
    const int local = q >> 7;
    const int nvalid = local + 1;
    const float* srow = scores + row * NB;

    float lv[KPL];
    int li[KPL];
#pragma unroll
    for (int k = 0; k < KPL; ++k) {
        lv[k] = -INFINITY;
        li[k] = NB;
    }
    const int kt = (Kb - 1) >> 5, lt = (Kb - 1) & 31;   // position of the Kb-th entry
    float tv = -INFINITY;

    // Sorted insertion of (cv, ci) with shift; the last entry of the list falls out.  Candidates arrive in ascending
    // block index, so an entry of equal score that is already in the list has the lower index and stays ahead: the
    // position is decided by the scores alone (a strict comparison), except for the forced own block (`by_index`).
    auto insert = [&](float cv, int ci, bool by_index) {
        float inv = cv;
        int ini = ci;
        bool placed = false;
#pragma unroll
        for (int k = 0; k < KPL; ++k) {
            const unsigned bm = placed ? 0xffffffffu
                                       : __ballot_sync(0xffffffffu, by_index ? beats(cv, ci, lv[k], li[k]) : (cv > lv[k]));
            if (bm != 0) {
                const int first = __ffs(bm) - 1;
                const float outv = __shfl_sync(0xffffffffu, lv[k], 31);
                const int outi = __shfl_sync(0xffffffffu, li[k], 31);
                const float upv = __shfl_up_sync(0xffffffffu, lv[k], 1);
                const int upi = __shfl_up_sync(0xffffffffu, li[k], 1);
                if (lane > first) {
                    lv[k] = upv;
                    li[k] = upi;
                } else if (lane == first) {
                    lv[k] = inv;
                    li[k] = ini;
                }
                inv = outv;
                ini = outi;
                placed = true;
            }
        }
    };
    // the current Kb-th entry: what a candidate has to beat (refreshed once per batch of 32 candidates, not after every
    // insertion: a stale, lower bar only lets a candidate through that the insertion then places beyond the Kb-th slot)
    auto refresh_bar = [&]() {
        tv = __shfl_sync(0xffffffffu, lv[kt], lt);
    };

    int base = 0;
    if (KPL == 1) {
        // The first 32 candidates would nearly all be inserted one by one (the list is still empty):
        // sort them with a bitonic network instead (15 compare-exchange steps).  Same total order, so
        // the list is the one the insertions would have built.
        const int j = lane;
        const bool have = (j < nvalid) && (j != local);
        const float s = have ? srow[j] : -INFINITY;
        const bool ok = have && s > -INFINITY;   // a score of -inf (or NaN) never enters the list
        float v = ok ? s : -INFINITY;
        int id = ok ? j : NB;
#pragma unroll
        for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
            for (int jj = k >> 1; jj > 0; jj >>= 1) {
                const float pv = __shfl_xor_sync(0xffffffffu, v, jj);
                const int pi = __shfl_xor_sync(0xffffffffu, id, jj);
                // descending overall: inside a block of k lanes whose bit k is clear the better entry goes
                // to the lower lane, in the other blocks to the upper lane (k = 32: one block, bit clear)
                const bool want_better = ((lane & jj) == 0) == ((lane & k) == 0);
                const bool partner_better = beats(pv, pi, v, id);
                if (partner_better == want_better && (pv != v || pi != id)) {
                    v = pv;
                    id = pi;
                }
            }
        }
        lv[0] = v;
        li[0] = id;
        base = 32;
    }
    insert(INFINITY, local, true);   // the row's own block is forced first
    refresh_bar();

    for (; base < nvalid; base += 32) {
        const int j = base + lane;
        const bool have = (j < nvalid) && (j != local);
        const float s = have ? srow[j] : -INFINITY;
        // a score of -inf (or NaN) never enters the list: such a slot keeps the sentinel
        // (a candidate that only ties the bar loses to it: the entry in the list has the lower block index)
        unsigned mask = __ballot_sync(0xffffffffu, have && s > -INFINITY && s > tv);
        while (mask) {
            const int src = __ffs(mask) - 1;
            mask &= mask - 1;
            insert(__shfl_sync(0xffffffffu, s, src), base + src, false);
        }
        refresh_bar();
    }
    int32_t* orow = out + row * Kb;
#pragma unroll
    for (int k = 0; k < KPL; ++k) {
        const int e = k * 32 + lane;
        if (e < Kb) orow[e] = li[k];
    }
}

}  // namespace
}  // namespace fmsa

extern "C" int fmsa_select_topk(const float* block_scores, int32_t* block_indices, int64_t rows_bh, int32_t S,
                                int32_t top_k_blocks, void* stream) {
    using namespace fmsa;
    FMSA_REQUIRE(block_scores && block_indices);
    FMSA_REQUIRE(rows_bh >= 0 && S > 0 && S % kBlock == 0);
    const int NB = S / kBlock;
    FMSA_REQUIRE(top_k_blocks >= 1 && top_k_blocks <= NB);
    if (top_k_blocks > FMSA_MAX_TOPK_BLOCKS) return FMSA_ERR_UNSUPPORTED;
    const int64_t total = rows_bh * S;
    if (total == 0) return FMSA_OK;
    const int64_t grid = (total + 7) / 8;
    FMSA_REQUIRE(grid <= 0x7fffffffLL);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const dim3 g(static_cast<unsigned>(grid));
    if (top_k_blocks <= 32)
        topk_rows_kernel<1><<<g, 256, 0, st>>>(block_scores, block_indices, total, S, NB, top_k_blocks);
    else if (top_k_blocks <= 64)
        topk_rows_kernel<2><<<g, 256, 0, st>>>(block_scores, block_indices, total, S, NB, top_k_blocks);
    else
        topk_rows_kernel<4><<<g, 256, 0, st>>>(block_scores, block_indices, total, S, NB, top_k_blocks);
    return check_launch();
}
