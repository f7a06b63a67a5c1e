// Sparse MSA forward, key-block stationary.
//
// Selection is per query ROW, so the rows that attend to one key block are scattered over the
// sequence.  The work unit is therefore a key block: unit (batch b, KV head g, key block j) keeps
// K_j, V_j (and the proxy keys Kp_j) resident in shared memory and walks the reverse-index row of
// every proxy head of the group in chunks of 128 gathered query rows; each chunk is run once per
// main head of the proxy head (the heads share the selection) and once more for the proxy head
// itself, which only needs its log-sum-exp.
//
// A tile (128 gathered rows of one head against the 128 keys of the block):
//     S = Q_g K_j^T                tcgen05.mma, K-major x K-major, fp32 in TMEM
//     m, P = exp2(S*c - m), l      one thread per row (TMEM lane), P rounded to bf16 into smem
//     O_part = P V_j               tcgen05.mma, K-major x MN-major
//     partial (O_part / l in bf16, lse = m + log l) is written to the edge's slot;
// a combine kernel merges the <= Kb partials of every query row (fmsa_sparse_fwd_combine).
// This mirrors the numerics of the reference path, which merges bf16 partial outputs of
// FlashAttention calls in fp32 (flash_msa/sparse_flash_varlen.py:169-244,
// flash_msa/csrc/reverse_index_cuda.cu:235-309) but without its host loop, gathers and syncs.
//
// `dense` mode runs the same tiles over every causal (query block, key block) pair with an
// implicit schedule: it is the warmup forward (flash_msa/warmup/msa_forward_cutedsl_warmup.py:22-67)
// and the full-sequence proxy log-sum-exp (warmup/msa_backward_cutedsl_warmup.py:83-114).
//
// Scheduling: persistent CTAs (one per SM) take units from a global counter, early key blocks
// (the long rows under causality) first.  CTA-wide phases are separated by block barriers; the
// gather of the next tile and the epilogue of the previous tile overlap the current tile.
#include "host_common.h"
#include "msa_common.cuh"
#include "sm100.cuh"
#include "tma_host.h"

namespace fmsa {
namespace {

struct FwdParams {
    const __nv_bfloat16* q;
    int64_t q_sb, q_sh, q_ss;
    const __nv_bfloat16* qp;
    int64_t qp_sb, qp_sh, qp_ss;
    const int32_t* row_ptr;
    const int32_t* col_q;
    __nv_bfloat16* o_part;   // [(edge - edge_base) * mpp + head][128]
    float* lse_part;         // [(edge - edge_base) * (mpp + 1) + head], head == mpp is the proxy head
    int32_t* counter;
    int32_t* status;
    int S, NB, Hq, Hkv, Hp, mpp, ppk, pg;
    int g_begin, G;
    int with_proxy, dense;
    float scale_log2e;
};

struct FwdSmem {
    uint64_t bar_kv, bar_kp, bar_s, bar_o[2];
    uint32_t tmem_slot;
    int32_t unit;
    int32_t rows[2][128];
    float inv_l[2][128];
};

constexpr int kFwdThreads = 256;
constexpr size_t kFwdSmemBytes = 6 * kTileBytes + 1024 + sizeof(FwdSmem);

struct TileMeta {   // what the epilogue of a finished main tile needs
    int64_t slot0;  // (edge - edge_base) of tile row 0
    int nrows;
    int head;       // head inside the proxy group
    int obuf;
};

__global__ void __launch_bounds__(kFwdThreads, 1) sparse_fwd_kernel(const __grid_constant__ CUtensorMap tmap_k,
                                                                    const __grid_constant__ CUtensorMap tmap_v,
                                                                    const __grid_constant__ CUtensorMap tmap_kp,
                                                                    const FwdParams P) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t tile_k = tiles, tile_v = tiles + kTileBytes, tile_kp = tiles + 2 * kTileBytes;
    const uint32_t tile_q0 = tiles + 3 * kTileBytes, tile_p = tiles + 5 * kTileBytes;
    FwdSmem* sm = reinterpret_cast<FwdSmem*>(smem_raw + (tiles - smem_u32(smem_raw)) + 6 * kTileBytes);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quarter = warp & 3, row = quarter * 32 + lane;
    const uint32_t bar_kv = smem_u32(&sm->bar_kv), bar_kp = smem_u32(&sm->bar_kp), bar_s = smem_u32(&sm->bar_s);

    if (tid == 0) {
        mbar_init(bar_kv, 1);
        mbar_init(bar_kp, 1);
        mbar_init(bar_s, 1);
        mbar_init(smem_u32(&sm->bar_o[0]), 1);
        mbar_init(smem_u32(&sm->bar_o[1]), 1);
        fence_mbar_init();
        prefetch_tmap(&tmap_k);
        prefetch_tmap(&tmap_v);
        prefetch_tmap(&tmap_kp);
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(&sm->tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = sm->tmem_slot;
    const uint32_t tmem_s = tmem, tmem_o0 = tmem + 128;

    const int hpc = P.mpp + (P.with_proxy ? 1 : 0);   // tiles per chunk
    const int lse_stride = P.mpp + 1;
    const int64_t edge_base = P.dense ? dense_edge_base(static_cast<int64_t>(P.g_begin) * P.ppk, P.S, P.NB)
                                      : static_cast<int64_t>(P.row_ptr[static_cast<int64_t>(P.g_begin) * P.ppk * P.NB]);
    uint32_t ph_kv = 0, ph_kp = 0, ph_s = 0;
    uint32_t mt = 0;   // main tiles issued so far (selects the O accumulator and its barrier phase)
    bool bad = false;

    for (;;) {
        if (tid == 0) sm->unit = atomicAdd(P.counter, 1);
        __syncthreads();
        const int u = sm->unit;
        __syncthreads();
        if (u >= P.G * P.NB) break;
        const int j = u / P.G;
        const int g = P.g_begin + u % P.G;
        const int b = g / P.Hkv, kvh = g % P.Hkv;
        if (tid == 0) {
            mbar_arrive_expect_tx(bar_kv, 2 * kTileBytes);
            tma_load_tile(tile_k, &tmap_k, j * kBlock, kvh, b, bar_kv);
            tma_load_tile(tile_v, &tmap_v, j * kBlock, kvh, b, bar_kv);
        }
        bool kv_ready = false;

        for (int pp = 0; pp < P.ppk; ++pp) {
            const int p = kvh * P.ppk + pp;
            const int64_t bp = static_cast<int64_t>(b) * P.Hp + p;
            int64_t e0;
            int n;
            if (P.dense) {
                e0 = dense_edge_base(bp, P.S, P.NB) + dense_row_offset(j, P.S);
                n = P.S - j * kBlock;
            } else {
                e0 = P.row_ptr[bp * P.NB + j];
                n = P.row_ptr[bp * P.NB + j + 1] - static_cast<int>(e0);
            }
            if (n <= 0) continue;
            bool kp_ready = false;
            if (P.with_proxy && tid == 0) {
                mbar_arrive_expect_tx(bar_kp, kTileBytes);
                tma_load_tile(tile_kp, &tmap_kp, j * kBlock, p / P.pg, b, bar_kp);
            }
            const int nchunks = (n + kBlock - 1) / kBlock;
            const int ntiles = nchunks * hpc;
            const __nv_bfloat16* q_b = P.q + static_cast<int64_t>(b) * P.q_sb;
            const __nv_bfloat16* qp_bp = P.qp + static_cast<int64_t>(b) * P.qp_sb + static_cast<int64_t>(p) * P.qp_sh;

            auto stage_rows = [&](int chunk) {
                if (tid < kBlock) {
                    const int at = chunk * kBlock + tid;
                    int qid = -1;
                    if (at < n) {
                        qid = P.dense ? (j * kBlock + at) : P.col_q[e0 + at];
                        if (static_cast<unsigned>(qid) >= static_cast<unsigned>(P.S) || (qid >> 7) < j) {
                            atomicMax(P.status, kStatusBadIndex);
                            qid = -1;
                        }
                    }
                    sm->rows[chunk & 1][tid] = qid;
                }
            };
            auto issue_gather = [&](int t) {
                const int chunk = t / hpc, hh = t % hpc;
                const uint32_t dst = tile_q0 + (t & 1) * kTileBytes;
                if (hh < P.mpp)
                    gather_tile_async<kFwdThreads>(dst, q_b + static_cast<int64_t>(p * P.mpp + hh) * P.q_sh, P.q_ss,
                                                   sm->rows[chunk & 1], tid);
                else
                    gather_tile_async<kFwdThreads>(dst, qp_bp, P.qp_ss, sm->rows[chunk & 1], tid);
                cp_async_commit();
            };

            stage_rows(0);
            __syncthreads();
            issue_gather(0);

            TileMeta prev{};
            bool pv_pending = false;

            for (int t = 0; t < ntiles; ++t) {
                const int chunk = t / hpc, hh = t % hpc;
                const bool is_proxy = hh == P.mpp;
                const uint32_t qbuf = tile_q0 + (t & 1) * kTileBytes;
                cp_async_wait<0>();
                fence_async_smem();
                __syncthreads();
                if (tid == 0) {
                    if (!kv_ready) bad |= !mbar_wait(bar_kv, ph_kv);
                    if (is_proxy && !kp_ready) bad |= !mbar_wait(bar_kp, ph_kp);
                    tc_fence_after_sync();
                    umma_tile_128<false, false>(tmem_s, qbuf, is_proxy ? tile_kp : tile_k, false);
                    umma_commit(bar_s);
                }
                if (!kv_ready) {
                    kv_ready = true;
                    ph_kv ^= 1;
                }
                if (is_proxy && !kp_ready) {
                    kp_ready = true;
                    ph_kp ^= 1;
                }
                // prefetch the next tile's rows while the tensor core works
                if (t + 1 < ntiles) {
                    const int nchunk = (t + 1) / hpc;
                    if (nchunk != chunk) {
                        stage_rows(nchunk);
                        __syncthreads();
                    }
                    issue_gather(t + 1);
                }
                bad |= !mbar_wait(bar_s, ph_s);
                ph_s ^= 1;
                if (__syncthreads_or(bad)) {
                    bad = true;
                    goto abort;
                }
                tc_fence_after_sync();

                const int nrows = min(kBlock, n - chunk * kBlock);
                if (warp < 4) {
                    // ---------------- softmax of tile t: one row per thread ----------------
                    const int qid = sm->rows[chunk & 1][row];
                    const int limit = (qid >= 0 && (qid >> 7) == j) ? (qid & 127) : 127;
                    float m = -INFINITY;
#pragma unroll 1
                    for (int c = 0; c < 128; c += 32) {
                        uint32_t v[32];
                        tmem_ld32(tmem_addr(tmem_s, quarter, c), v);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const float x = __uint_as_float(v[i]) * P.scale_log2e;
                            m = (c + i <= limit) ? fmaxf(m, x) : m;
                        }
                    }
                    if (pv_pending && !is_proxy)   // P buffer is still being read by the previous P*V
                        bad |= !mbar_wait(smem_u32(&sm->bar_o[prev.obuf]), ((mt - 1) >> 1) & 1);
                    float l = 0.f;
#pragma unroll 1
                    for (int c = 0; c < 128; c += 32) {
                        uint32_t v[32];
                        tmem_ld32(tmem_addr(tmem_s, quarter, c), v);
                        tmem_ld_wait();
                        uint32_t pk[16];
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            float p0 = fast_exp2(__uint_as_float(v[i]) * P.scale_log2e - m);
                            float p1 = fast_exp2(__uint_as_float(v[i + 1]) * P.scale_log2e - m);
                            p0 = (c + i <= limit) ? p0 : 0.f;
                            p1 = (c + i + 1 <= limit) ? p1 : 0.f;
                            l += p0 + p1;
                            pk[i >> 1] = pack_bf16(p0, p1);
                        }
                        if (!is_proxy) {
#pragma unroll
                            for (int k8 = 0; k8 < 4; ++k8)
                                st_shared_v4(tile_p + swz_offset(row, (c >> 3) + k8), pk[4 * k8], pk[4 * k8 + 1],
                                             pk[4 * k8 + 2], pk[4 * k8 + 3]);
                        }
                    }
                    if (row < nrows && qid >= 0) {
                        const int64_t slot = e0 - edge_base + chunk * kBlock + row;
                        P.lse_part[slot * lse_stride + hh] = (m + __log2f(l)) * kLn2;
                    }
                    if (!is_proxy) sm->inv_l[mt & 1][row] = 1.f / l;
                    fence_async_smem();
                } else if (pv_pending) {
                    // ---------------- epilogue of the previous main tile ----------------
                    bad |= !mbar_wait(smem_u32(&sm->bar_o[prev.obuf]), ((mt - 1) >> 1) & 1);
                    tc_fence_after_sync();
                    const float il = sm->inv_l[prev.obuf][row];
                    const bool live = row < prev.nrows;
                    __nv_bfloat16* dst = P.o_part + ((prev.slot0 + row) * P.mpp + prev.head) * kHeadDim;
#pragma unroll 1
                    for (int c = 0; c < 128; c += 32) {
                        uint32_t v[32];
                        tmem_ld32(tmem_addr(tmem_o0 + prev.obuf * 128, quarter, c), v);
                        tmem_ld_wait();
                        if (live) {
#pragma unroll
                            for (int k8 = 0; k8 < 4; ++k8) {
                                uint4 w;
                                w.x = pack_bf16(__uint_as_float(v[8 * k8 + 0]) * il, __uint_as_float(v[8 * k8 + 1]) * il);
                                w.y = pack_bf16(__uint_as_float(v[8 * k8 + 2]) * il, __uint_as_float(v[8 * k8 + 3]) * il);
                                w.z = pack_bf16(__uint_as_float(v[8 * k8 + 4]) * il, __uint_as_float(v[8 * k8 + 5]) * il);
                                w.w = pack_bf16(__uint_as_float(v[8 * k8 + 6]) * il, __uint_as_float(v[8 * k8 + 7]) * il);
                                *reinterpret_cast<uint4*>(dst + c + 8 * k8) = w;
                            }
                        }
                    }
                }
                tc_fence_before_sync();
                if (__syncthreads_or(bad)) {
                    bad = true;
                    goto abort;
                }
                pv_pending = false;
                if (!is_proxy) {
                    if (tid == 0) {
                        tc_fence_after_sync();
                        umma_tile_128<false, true>(tmem_o0 + (mt & 1) * 128, tile_p, tile_v, false);
                        umma_commit(smem_u32(&sm->bar_o[mt & 1]));
                    }
                    prev.slot0 = e0 - edge_base + static_cast<int64_t>(chunk) * kBlock;
                    prev.nrows = nrows;
                    prev.head = hh;
                    prev.obuf = mt & 1;
                    ++mt;
                    pv_pending = true;
                }
            }
            // drain: the last main tile of this (unit, proxy head)
            if (pv_pending) {
                bad |= !mbar_wait(smem_u32(&sm->bar_o[prev.obuf]), ((mt - 1) >> 1) & 1);
                tc_fence_after_sync();
                if (warp >= 4 && !bad) {
                    const float il = sm->inv_l[prev.obuf][row];
                    const bool live = row < prev.nrows;
                    __nv_bfloat16* dst = P.o_part + ((prev.slot0 + row) * P.mpp + prev.head) * kHeadDim;
#pragma unroll 1
                    for (int c = 0; c < 128; c += 32) {
                        uint32_t v[32];
                        tmem_ld32(tmem_addr(tmem_o0 + prev.obuf * 128, quarter, c), v);
                        tmem_ld_wait();
                        if (live) {
#pragma unroll
                            for (int k8 = 0; k8 < 4; ++k8) {
                                uint4 w;
                                w.x = pack_bf16(__uint_as_float(v[8 * k8 + 0]) * il, __uint_as_float(v[8 * k8 + 1]) * il);
                                w.y = pack_bf16(__uint_as_float(v[8 * k8 + 2]) * il, __uint_as_float(v[8 * k8 + 3]) * il);
                                w.z = pack_bf16(__uint_as_float(v[8 * k8 + 4]) * il, __uint_as_float(v[8 * k8 + 5]) * il);
                                w.w = pack_bf16(__uint_as_float(v[8 * k8 + 6]) * il, __uint_as_float(v[8 * k8 + 7]) * il);
                                *reinterpret_cast<uint4*>(dst + c + 8 * k8) = w;
                            }
                        }
                    }
                }
                tc_fence_before_sync();
                if (__syncthreads_or(bad)) {
                    bad = true;
                    goto abort;
                }
            }
        }
        if (!kv_ready) {   // no proxy head of this unit had any edge: still consume the K/V load
            if (tid == 0) bad |= !mbar_wait(bar_kv, ph_kv);
            ph_kv ^= 1;
            if (__syncthreads_or(bad)) {
                bad = true;
                goto abort;
            }
        }
    }
abort:
    cp_async_wait<0>();
    if (bad && tid == 0) atomicMax(P.status, kStatusWaitTimeout);
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 512);
}

// -------------------------------------------------------------------------------------------
// combine: merge the partials of every query row
// -------------------------------------------------------------------------------------------
struct CombineParams {
    const __nv_bfloat16* o_part;
    const float* lse_part;
    const int32_t* edge_pos;   // sparse: [B*Hp, S, Kb]
    const int32_t* row_ptr;
    __nv_bfloat16* out;        // [B, S, Hq*128]
    float* lse;                // [B, Hq, S]
    float* lse_proxy;          // [B, Hp, S] or null
    int S, NB, Hq, Hp, mpp, ppk, Kb;
    int g_begin, G, dense;
};

__global__ void __launch_bounds__(256) combine_kernel(const CombineParams P) {
    const int lane = threadIdx.x & 31;
    const int64_t w = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    const int64_t bp0 = static_cast<int64_t>(P.g_begin) * P.ppk;
    const int64_t nrows = static_cast<int64_t>(P.G) * P.ppk * P.S;
    if (w >= nrows) return;
    const int64_t bp = bp0 + w / P.S;
    const int q = static_cast<int>(w % P.S);
    const int b = static_cast<int>(bp / P.Hp), p = static_cast<int>(bp % P.Hp);
    const int64_t edge_base = P.dense ? dense_edge_base(bp0, P.S, P.NB) : static_cast<int64_t>(P.row_ptr[bp0 * P.NB]);
    const int nslots = P.dense ? (q >> 7) + 1 : P.Kb;
    const int lse_stride = P.mpp + 1;
    const int32_t* erow = P.dense ? nullptr : P.edge_pos + (bp * P.S + q) * P.Kb;

    auto slot_of = [&](int s) -> int64_t {
        if (s >= nslots) return -1;
        if (P.dense) return dense_edge_base(bp, P.S, P.NB) + dense_row_offset(s, P.S) + (q - s * kBlock) - edge_base;
        const int e = erow[s];
        return e < 0 ? -1 : static_cast<int64_t>(e) - edge_base;
    };

    const int nheads = P.mpp + (P.lse_proxy ? 1 : 0);
    for (int hh = 0; hh < nheads; ++hh) {
        // pass A: log-sum-exp over the slots
        float m = -INFINITY, sum = 0.f;
        for (int s0 = 0; s0 < nslots; s0 += 32) {
            const int64_t sl = slot_of(s0 + lane);
            if (sl >= 0) {
                const float x = P.lse_part[sl * lse_stride + hh];
                const float mn = fmaxf(m, x);
                sum = sum * __expf(m - mn) + __expf(x - mn);
                m = mn;
            }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float mo = __shfl_xor_sync(0xffffffffu, m, off);
            const float so = __shfl_xor_sync(0xffffffffu, sum, off);
            const float mn = fmaxf(m, mo);
            const float a = (m == -INFINITY) ? 0.f : sum * __expf(m - mn);
            const float c = (mo == -INFINITY) ? 0.f : so * __expf(mo - mn);
            sum = a + c;
            m = mn;
        }
        const float total = m + __logf(sum);
        if (hh == P.mpp) {
            if (lane == 0) P.lse_proxy[bp * P.S + q] = total;
            continue;
        }
        const int h = p * P.mpp + hh;
        if (lane == 0) P.lse[(static_cast<int64_t>(b) * P.Hq + h) * P.S + q] = total;
        // pass B: weighted sum of the partial outputs; lane owns columns 4*lane..4*lane+3
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
        for (int s0 = 0; s0 < nslots; s0 += 32) {
            const int64_t sl = slot_of(s0 + lane);
            const float wgt = sl >= 0 ? __expf(P.lse_part[sl * lse_stride + hh] - total) : 0.f;
            const int cnt = min(32, nslots - s0);
            for (int i = 0; i < cnt; ++i) {
                const int64_t si = __shfl_sync(0xffffffffu, sl, i);
                const float wi = __shfl_sync(0xffffffffu, wgt, i);
                if (si < 0) continue;
                const uint2 raw = *reinterpret_cast<const uint2*>(P.o_part + (si * P.mpp + hh) * kHeadDim + lane * 4);
                const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
                const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
                a0 += wi * __low2float(lo);
                a1 += wi * __high2float(lo);
                a2 += wi * __low2float(hi);
                a3 += wi * __high2float(hi);
            }
        }
        uint2 o;
        o.x = pack_bf16(a0, a1);
        o.y = pack_bf16(a2, a3);
        *reinterpret_cast<uint2*>(P.out + (static_cast<int64_t>(b) * P.S + q) * (static_cast<int64_t>(P.Hq) * kHeadDim) +
                                  static_cast<int64_t>(h) * kHeadDim + lane * 4) = o;
    }
}

}  // namespace
}  // namespace fmsa

extern "C" int64_t fmsa_fwd_partial_slots(const fmsa_problem* pb, int32_t g_count, int32_t dense) {
    using namespace fmsa;
    if (!problem_ok(pb) || g_count <= 0) return 0;
    const int64_t ppk = pb->Hp / pb->Hkv;
    const int NB = pb->S / kBlock;
    return dense ? g_count * ppk * dense_edges_per_bp(pb->S, NB) : g_count * ppk * static_cast<int64_t>(pb->S) * pb->top_k_blocks;
}

extern "C" int fmsa_sparse_fwd(const fmsa_problem* pb, const fmsa_tensor* q, const fmsa_tensor* k, const fmsa_tensor* v,
                               const fmsa_tensor* q_proxy, const fmsa_tensor* k_proxy, const int32_t* row_ptr,
                               const int32_t* col_q, void* o_part, float* lse_part, int64_t part_slots, int32_t g_begin,
                               int32_t g_count, int32_t with_proxy, int32_t dense, int32_t* counter, int32_t* status,
                               void* stream) {
    using namespace fmsa;
    FMSA_REQUIRE(problem_ok(pb));
    FMSA_REQUIRE(q && k && v && q->ptr && k->ptr && v->ptr && o_part && lse_part && counter && status);
    FMSA_REQUIRE(dense || (row_ptr && col_q));
    FMSA_REQUIRE(!with_proxy || (q_proxy && k_proxy && q_proxy->ptr && k_proxy->ptr));
    FMSA_REQUIRE(g_begin >= 0 && g_count > 0 && g_begin + g_count <= pb->B * pb->Hkv);
    FMSA_REQUIRE(dense || (pb->top_k_blocks >= 1 && pb->top_k_blocks <= pb->S / kBlock));
    FMSA_REQUIRE(pb->scale > 0.f);
    if (part_slots < fmsa_fwd_partial_slots(pb, g_count, dense)) return FMSA_ERR_WORKSPACE;
    FMSA_REQUIRE(tma_compatible(k->ptr, k->stride_b, k->stride_h, k->stride_s));
    FMSA_REQUIRE(tma_compatible(v->ptr, v->stride_b, v->stride_h, v->stride_s));
    FMSA_REQUIRE(tma_compatible(q->ptr, q->stride_b, q->stride_h, q->stride_s));
    const fmsa_tensor* kp = with_proxy ? k_proxy : k;
    if (with_proxy) {
        FMSA_REQUIRE(tma_compatible(kp->ptr, kp->stride_b, kp->stride_h, kp->stride_s));
        FMSA_REQUIRE(tma_compatible(q_proxy->ptr, q_proxy->stride_b, q_proxy->stride_h, q_proxy->stride_s));
    }
    CUtensorMap tk, tv, tkp;
    if (!make_tmap_bhsd(&tk, k->ptr, pb->B, pb->Hkv, pb->S, k->stride_b, k->stride_h, k->stride_s, 128) ||
        !make_tmap_bhsd(&tv, v->ptr, pb->B, pb->Hkv, pb->S, v->stride_b, v->stride_h, v->stride_s, 128) ||
        !make_tmap_bhsd(&tkp, kp->ptr, pb->B, with_proxy ? pb->Hpkv : pb->Hkv, pb->S, kp->stride_b, kp->stride_h, kp->stride_s, 128))
        return FMSA_ERR_CUDA;

    FwdParams P;
    P.q = static_cast<const __nv_bfloat16*>(q->ptr);
    P.q_sb = q->stride_b; P.q_sh = q->stride_h; P.q_ss = q->stride_s;
    P.qp = with_proxy ? static_cast<const __nv_bfloat16*>(q_proxy->ptr) : P.q;
    P.qp_sb = with_proxy ? q_proxy->stride_b : 0; P.qp_sh = with_proxy ? q_proxy->stride_h : 0;
    P.qp_ss = with_proxy ? q_proxy->stride_s : 0;
    P.row_ptr = row_ptr; P.col_q = col_q;
    P.o_part = static_cast<__nv_bfloat16*>(o_part); P.lse_part = lse_part;
    P.counter = counter; P.status = status;
    P.S = pb->S; P.NB = pb->S / kBlock; P.Hq = pb->Hq; P.Hkv = pb->Hkv; P.Hp = pb->Hp;
    P.mpp = pb->Hq / pb->Hp; P.ppk = pb->Hp / pb->Hkv; P.pg = pb->Hp / pb->Hpkv;
    P.g_begin = g_begin; P.G = g_count; P.with_proxy = with_proxy ? 1 : 0; P.dense = dense ? 1 : 0;
    P.scale_log2e = pb->scale * kLog2e;

    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return FMSA_ERR_CUDA;
    if (cudaFuncSetAttribute(sparse_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kFwdSmemBytes)) !=
        cudaSuccess)
        return FMSA_ERR_CUDA;
    if (cudaMemsetAsync(counter, 0, sizeof(int32_t), st) != cudaSuccess) return FMSA_ERR_CUDA;
    const int64_t units = static_cast<int64_t>(g_count) * P.NB;
    const int grid = static_cast<int>(units < sms ? units : sms);
    sparse_fwd_kernel<<<grid, kFwdThreads, kFwdSmemBytes, st>>>(tk, tv, tkp, P);
    return check_launch();
}

extern "C" int fmsa_sparse_fwd_combine(const fmsa_problem* pb, const void* o_part, const float* lse_part,
                                       const int32_t* edge_pos, const int32_t* row_ptr, void* out, float* lse,
                                       float* lse_proxy, int32_t g_begin, int32_t g_count, int32_t dense, void* stream) {
    using namespace fmsa;
    FMSA_REQUIRE(problem_ok(pb));
    FMSA_REQUIRE(o_part && lse_part && out && lse);
    FMSA_REQUIRE(dense || (edge_pos && row_ptr));
    FMSA_REQUIRE(g_begin >= 0 && g_count > 0 && g_begin + g_count <= pb->B * pb->Hkv);
    CombineParams P;
    P.o_part = static_cast<const __nv_bfloat16*>(o_part); P.lse_part = lse_part; P.edge_pos = edge_pos; P.row_ptr = row_ptr;
    P.out = static_cast<__nv_bfloat16*>(out); P.lse = lse; P.lse_proxy = lse_proxy;
    P.S = pb->S; P.NB = pb->S / kBlock; P.Hq = pb->Hq; P.Hp = pb->Hp; P.mpp = pb->Hq / pb->Hp; P.ppk = pb->Hp / pb->Hkv;
    P.Kb = pb->top_k_blocks; P.g_begin = g_begin; P.G = g_count; P.dense = dense ? 1 : 0;
    const int64_t rows = static_cast<int64_t>(g_count) * P.ppk * P.S;
    const int64_t grid = (rows + 7) / 8;
    FMSA_REQUIRE(grid <= 0x7fffffffLL);
    combine_kernel<<<static_cast<unsigned>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(P);
    return check_launch();
}
