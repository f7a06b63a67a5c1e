// Proxy block scores: the tensor-core half of block selection.
//
// For every (batch, proxy head, query row q) and every causally visible key block j <= q/128
//     block_scores[q][j] = max over visible keys k of block j of  scale * Qp[q] . Kp[k]
// (flash_msa/tests/testing_model.py:75-88; the reference kernel computes the same maxima inside
// msa_select_cutedsl.py:238-306 but rounds each score to bf16 first, which this kernel does not).
// Entries with j > q/128 are left untouched; the top-k kernel never reads them.
//
// One CTA owns a 128-row query tile of one (batch, proxy head) and walks the key blocks 0..i.
// Warp-specialised: warp 0 feeds K tiles by TMA through a two-stage ring, warp 1 issues
// tcgen05.mma into one of two TMEM accumulators, warps 2-5 read an accumulator back (one row per
// thread), take the masked row maximum and stage it in shared memory so that global stores are
// row-contiguous.
//
// Fused selection (LK > 0, top_k_blocks <= LK): the thread that owns a row sees the row's block scores one by one, in
// ascending block index, so it can keep the row's best LK blocks in a sorted register list and write block_indices
// itself; block_scores is then never written and the separate top-k kernel is not needed.  The order is the one of
// the top-k kernel (score descending, equal scores by ascending block index, own block first, sentinel NB): a new
// score goes behind every entry that is at least as large, and the own block is put in front at the end.
#include "host_common.h"
#include "sm100.cuh"
#include "tma_host.h"

namespace fmsa {
namespace {

constexpr int kScoreStageCols = 16;   // key blocks staged per flush

struct ScoreSmem {
    uint64_t q_full, k_full[2], k_empty[2], s_full[2], s_empty[2];
    uint32_t tmem_slot;
    float stage[128][kScoreStageCols + 1];
};

template <bool FP16, int LK>
__global__ void __launch_bounds__(192) select_scores_kernel(const __grid_constant__ CUtensorMap tmap_q,
                                                            const __grid_constant__ CUtensorMap tmap_k,
                                                            float* __restrict__ block_scores, int Hp, int pg, int S,
                                                            int NB, float scale, const int32_t* __restrict__ doc_start,
                                                            int32_t* __restrict__ block_indices, int Kb,
                                                            int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t tile_q = tiles, tile_k0 = tiles + kTileBytes;
    ScoreSmem* sm = reinterpret_cast<ScoreSmem*>(smem_raw + (tiles - smem_u32(smem_raw)) + 3 * kTileBytes);

    // The warp index goes through a shuffle so that the compiler knows it, and every branch on the warp's
    // role, to be uniform across the warp: the issuer's descriptor arithmetic can then use the uniform datapath.
    const int tid = threadIdx.x, warp = __shfl_sync(0xffffffffu, tid >> 5, 0), lane = tid & 31;
    const int qt = NB - 1 - static_cast<int>(blockIdx.x);   // longest tiles first
    const int bp = blockIdx.y;
    const int b = bp / Hp, p = bp % Hp, kph = p / pg;

    if (tid == 0) {
        mbar_init(smem_u32(&sm->q_full), 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&sm->k_full[i]), 1);
            mbar_init(smem_u32(&sm->k_empty[i]), 1);
            mbar_init(smem_u32(&sm->s_full[i]), 1);
            mbar_init(smem_u32(&sm->s_empty[i]), 128);
        }
        fence_mbar_init();
        prefetch_tmap(&tmap_q);
        prefetch_tmap(&tmap_k);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&sm->tmem_slot), 256);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = __shfl_sync(0xffffffffu, sm->tmem_slot, 0);
    bool ok = true;

    if (warp == 0) {
        if (lane == 0) {
            mbar_arrive_expect_tx(smem_u32(&sm->q_full), kTileBytes);
            tma_load_tile(tile_q, &tmap_q, qt * kBlock, p, b, smem_u32(&sm->q_full));
            for (int j = 0; j <= qt && ok; ++j) {
                const int st = j & 1;
                if (j >= 2) ok = mbar_wait(smem_u32(&sm->k_empty[st]), ((j >> 1) - 1) & 1);
                if (!ok) break;
                mbar_arrive_expect_tx(smem_u32(&sm->k_full[st]), kTileBytes);
                tma_load_tile(tile_k0 + st * kTileBytes, &tmap_k, j * kBlock, kph, b, smem_u32(&sm->k_full[st]));
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            ok = mbar_wait(smem_u32(&sm->q_full), 0);
            for (int j = 0; j <= qt && ok; ++j) {
                const int st = j & 1;
                ok = mbar_wait(smem_u32(&sm->k_full[st]), (j >> 1) & 1);
                if (ok && j >= 2) ok = mbar_wait(smem_u32(&sm->s_empty[st]), ((j >> 1) - 1) & 1);
                if (!ok) break;
                tc_fence_after_sync();
                umma_tile_128<false, false, FP16>(tmem + st * 128, tile_q, tile_k0 + st * kTileBytes, false);
                umma_commit(smem_u32(&sm->k_empty[st]));
                umma_commit(smem_u32(&sm->s_full[st]));
            }
        }
    } else {
        const int quarter = warp & 3;            // TMEM lane quarter this warp may read
        const int r = quarter * 32 + lane;        // row of the query tile
        // Document masking of a packed sequence: keys before the first token of the row's document are hidden
        // (lo = 0 without documents).
        const int lo = doc_start ? doc_start[static_cast<int64_t>(b) * S + qt * kBlock + r] : 0;
        const int lo_blk = lo >> 7, lo_col = lo & 127;
        constexpr int kList = LK > 0 ? LK : 1;
        float lv[kList];   // fused selection: the row's best blocks so far, best first
        int li[kList];
#pragma unroll
        for (int i = 0; i < kList; ++i) {
            lv[i] = -INFINITY;
            li[i] = NB;
        }
        // (value, block) goes behind every entry that is at least as large; the last entry falls out
        auto list_insert = [&](float val, int blk) {
#pragma unroll
            for (int i = kList - 1; i > 0; --i) {
                const bool shift = lv[i - 1] < val;           // entry i-1 moves down to i
                const bool here = !shift && lv[i] < val;      // the new entry lands at i
                lv[i] = shift ? lv[i - 1] : (here ? val : lv[i]);
                li[i] = shift ? li[i - 1] : (here ? blk : li[i]);
            }
            if (lv[0] < val) {
                lv[0] = val;
                li[0] = blk;
            }
        };
        for (int j = 0; j <= qt; ++j) {
            const int st = j & 1;
            ok = mbar_wait(smem_u32(&sm->s_full[st]), (j >> 1) & 1);
            if (!ok) break;   // every lane of the warp waits on the same phase: uniform
            tc_fence_after_sync();
            // The factor `scale` is positive, so it is applied once to the row maximum instead of to every logit
            // (rounding is monotone: the result is the same bit for bit).  Only the diagonal block needs the causal
            // mask; every other block is a plain maximum over 128 values, taken three at a time with the loads of
            // the next 32 columns already in flight.
            float m = -INFINITY;
            const bool low_edge = (j == lo_blk) && lo_col > 0;   // the row's document starts inside this block
            if (j == qt || __any_sync(0xffffffffu, low_edge)) {
                const int c_lo = low_edge ? lo_col : 0, c_hi = (j == qt) ? r : 127;
#pragma unroll 1
                for (int c = 0; c < 128; c += 32) {
                    uint32_t v[32];
                    tmem_ld32(tmem_addr(tmem + st * 128, quarter, c), v);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) m = (c + i >= c_lo && c + i <= c_hi) ? fmaxf(m, __uint_as_float(v[i])) : m;
                }
            } else {
                uint32_t v[2][32];
                tmem_ld32(tmem_addr(tmem + st * 128, quarter, 0), v[0]);
#pragma unroll
                for (int c = 0; c < 128; c += 32) {
                    const int cur = (c >> 5) & 1;
                    tmem_ld_wait();
                    if (c + 32 < 128) tmem_ld32(tmem_addr(tmem + st * 128, quarter, c + 32), v[cur ^ 1]);
#pragma unroll
                    for (int i = 0; i < 32; i += 2) m = fmax3(m, __uint_as_float(v[cur][i]), __uint_as_float(v[cur][i + 1]));
                }
            }
            m *= scale;
            if (j < lo_blk) m = -INFINITY;   // the whole block lies before the row's document
            tc_fence_before_sync();
            mbar_arrive(smem_u32(&sm->s_empty[st]));
            if (LK > 0) {
                // (a score of -inf or NaN never enters; the own block is forced in after the loop)
                if (j < qt && __any_sync(0xffffffffu, m > lv[kList - 1])) list_insert(m, j);
                continue;
            }
            sm->stage[r][j % kScoreStageCols] = m;
            if ((j % kScoreStageCols) == kScoreStageCols - 1 || j == qt) {
                __syncwarp();
                const int j0 = j - (j % kScoreStageCols);
                const int ncol = j - j0 + 1;
                // the warp owns rows quarter*32 .. +31 of the stage: write them row-contiguously
                for (int e = lane; e < 32 * kScoreStageCols; e += 32) {
                    const int rr = e / kScoreStageCols, cc = e % kScoreStageCols;
                    if (cc < ncol) {
                        float* orow = block_scores + (static_cast<int64_t>(bp) * S + qt * kBlock + quarter * 32 + rr) * NB;
                        orow[j0 + cc] = sm->stage[quarter * 32 + rr][cc];
                    }
                }
                __syncwarp();
            }
        }
        if (LK > 0 && ok) {
            // the row's own block always comes first (flash_msa/tests/testing_model.py:90-94)
            list_insert(INFINITY, qt);
            int32_t* orow = block_indices + (static_cast<int64_t>(bp) * S + qt * kBlock + r) * Kb;
#pragma unroll
            for (int i = 0; i < kList; ++i)
                if (i < Kb) orow[i] = li[i];
        }
    }
    if (!ok) atomicMax(status, kStatusWaitTimeout);
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 256);
}

}  // namespace
}  // namespace fmsa

namespace fmsa {
namespace {

template <bool FP16, int LK>
int launch_select(const CUtensorMap& tq, const CUtensorMap& tk, float* block_scores, int32_t* block_indices, int B, int Hp,
                  int Hpkv, int S, int Kb, float scale, const int32_t* doc_start, int32_t* status, cudaStream_t st) {
    const int NB = S / kBlock;
    const size_t smem = 3 * kTileBytes + 1024 + sizeof(ScoreSmem);
    if (!ensure_smem_attr(reinterpret_cast<const void*>(select_scores_kernel<FP16, LK>), smem)) return FMSA_ERR_CUDA;
    const dim3 grid(static_cast<unsigned>(NB), static_cast<unsigned>(B * Hp));
    select_scores_kernel<FP16, LK><<<grid, 192, smem, st>>>(tq, tk, block_scores, Hp, Hp / Hpkv, S, NB, scale, doc_start,
                                                           block_indices, Kb, status);
    return check_launch();
}

int select_common(const fmsa_tensor* q_proxy, const fmsa_tensor* k_proxy, float* block_scores, int32_t* block_indices,
                  int32_t B, int32_t Hp, int32_t Hpkv, int32_t S, int32_t Kb, float scale, int32_t dtype,
                  const int32_t* doc_start, int32_t* status, void* stream) {
    FMSA_REQUIRE(q_proxy && k_proxy && q_proxy->ptr && k_proxy->ptr && status);
    FMSA_REQUIRE(B > 0 && Hp > 0 && Hpkv > 0 && Hp % Hpkv == 0 && S > 0 && S % kBlock == 0);
    FMSA_REQUIRE(dtype == FMSA_DTYPE_BF16 || dtype == FMSA_DTYPE_FP16);
    FMSA_REQUIRE(scale > 0.f);   // the kernel scales the block maximum, not every logit
    FMSA_REQUIRE(static_cast<int64_t>(B) * Hp <= 65535);
    FMSA_REQUIRE(tma_compatible(q_proxy->ptr, q_proxy->stride_b, q_proxy->stride_h, q_proxy->stride_s));
    FMSA_REQUIRE(tma_compatible(k_proxy->ptr, k_proxy->stride_b, k_proxy->stride_h, k_proxy->stride_s));
    CUtensorMap tq, tk;
    if (!make_tmap_bhsd(&tq, q_proxy->ptr, B, Hp, S, q_proxy->stride_b, q_proxy->stride_h, q_proxy->stride_s, 128) ||
        !make_tmap_bhsd(&tk, k_proxy->ptr, B, Hpkv, S, k_proxy->stride_b, k_proxy->stride_h, k_proxy->stride_s, 128))
        return FMSA_ERR_CUDA;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool fp16 = dtype == FMSA_DTYPE_FP16;
#define FMSA_SELECT(LKV)                                                                                              \
    (fp16 ? launch_select<true, LKV>(tq, tk, block_scores, block_indices, B, Hp, Hpkv, S, Kb, scale, doc_start, status, st) \
          : launch_select<false, LKV>(tq, tk, block_scores, block_indices, B, Hp, Hpkv, S, Kb, scale, doc_start, status, st))
    if (Kb == 0) return FMSA_SELECT(0);
    if (Kb <= 8) return FMSA_SELECT(8);
    if (Kb <= 16) return FMSA_SELECT(16);
    if (Kb <= 32) return FMSA_SELECT(32);
    return FMSA_SELECT(64);
#undef FMSA_SELECT
}

}  // namespace
}  // namespace fmsa

extern "C" int fmsa_select_scores(const fmsa_tensor* q_proxy, const fmsa_tensor* k_proxy, float* block_scores,
                                  int32_t B, int32_t Hp, int32_t Hpkv, int32_t S, float scale, int32_t dtype,
                                  const int32_t* doc_start, int32_t* status, void* stream) {
    using namespace fmsa;
    FMSA_REQUIRE(block_scores);
    return select_common(q_proxy, k_proxy, block_scores, nullptr, B, Hp, Hpkv, S, 0, scale, dtype, doc_start, status, stream);
}

extern "C" int fmsa_select_fused(const fmsa_tensor* q_proxy, const fmsa_tensor* k_proxy, int32_t* block_indices, int32_t B,
                                 int32_t Hp, int32_t Hpkv, int32_t S, int32_t top_k_blocks, float scale, int32_t dtype,
                                 const int32_t* doc_start, int32_t* status, void* stream) {
    using namespace fmsa;
    FMSA_REQUIRE(block_indices && S > 0 && top_k_blocks >= 1 && top_k_blocks <= S / kBlock);
    if (top_k_blocks > FMSA_FUSED_SELECT_MAX_BLOCKS) return FMSA_ERR_UNSUPPORTED;
    return select_common(q_proxy, k_proxy, nullptr, block_indices, B, Hp, Hpkv, S, top_k_blocks, scale, dtype, doc_start, status,
                         stream);
}
