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
// Scheduling: persistent CTAs (one per SM) take sub-units of reverse-index rows from a global counter;
// inside a CTA the roles (softmax, gather, MMA issue) run decoupled, see sparse_fwd_kernel.
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
    float* stat_part;        // [(edge - edge_base) * (mpp + 1) + head][2] = (row max in the log2 domain, row sum);
                             // head == mpp is the proxy head
    int32_t* counter;
    int32_t* status;
    int S, NB, Hq, Hkv, Hp, mpp, ppk, pg;
    int g_begin, G;
    int with_proxy, dense;
    int64_t n_subunits;
    float scale_log2e;
};

struct FwdSmem {
    uint64_t bar_kv, bar_kp, bar_done;
    uint64_t q_full[2];              // Q rows of a tile have landed (arrivals: the gather group)
    uint64_t s_full[2], s_empty[2];  // S accumulator written by the tensor core / read by the softmax group
    uint64_t p_full;                 // P written to shared memory (arrivals: the softmax group)
    uint64_t o_full[2], o_empty[2];  // O accumulator written by the tensor core / read back by the softmax group
    uint64_t unit_full[4];           // a sub-unit index has been published in unit_ring
    int32_t unit_ring[4];
    uint32_t tmem_slot;
    int32_t rows[8][128];            // query positions of the chunks in flight (ring)
    float rmax[4][128];              // row maxima of the four column groups
    float lsum[4][128];              // row sums of the four column groups
};

constexpr int kFwdSoftmax = 512;                              // 16 warps: thread = (tile row, 32 columns)
constexpr int kFwdStore = 256;                                // 8 warps: row lists and cp.async gathers of the Q rows
constexpr int kFwdThreads = kFwdSoftmax + kFwdStore + 32;     // + one warp that issues tcgen05.mma
constexpr size_t kFwdSmemBytes = 6 * kTileBytes + 1024 + sizeof(FwdSmem);

// Warp-specialised forward.  Three roles run decoupled and meet only through mbarriers:
//   warps 0-15  softmax group : thread = (tile row, 32-column group); reads S from TMEM, writes P (bf16)
//                               to shared memory and the per-row (max, sum) to global memory; while it
//                               would wait for the next S it writes the finished O^T accumulator of the
//                               previous tile out as unnormalised bf16 partial rows (thread = head-dimension
//                               lane x 32 tile rows);
//   warps 16-23 gather group  : draws the work, stages the row lists and gathers the Q rows two tiles
//                               ahead (cp.async);
//   warp 24     issuer        : loads K_j, V_j, Kp_j by TMA and issues S(t+1) = Q K^T, then
//                               O^T(t) = V^T P^T(t), so the softmax of one tile overlaps the products of
//                               its neighbours and the store of the tile before.  All its lanes run the
//                               same code; only lane 0's tcgen05 instructions take effect (a lone
//                               diverged lane is scheduled late).
// Work is drawn from a global counter by one thread of the gather group and published to the other
// roles through a four-entry ring, so every role walks the same sequence of sub-units.
// TMEM: S[2] at columns 0 and 128, O^T[2] at 256 and 384.
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
    const int role = warp < 16 ? 0 : (warp < 24 ? 1 : 2);   // 0 softmax group, 1 store group, 2 issuer
    const int quarter = warp & 3;                            // TMEM lane quarter this warp may read
    const int row = quarter * 32 + lane;                     // softmax: tile row; store: head-dimension index
    const uint32_t elect = (lane == 0) ? 1u : 0u;
    const uint32_t bar_kv = smem_u32(&sm->bar_kv), bar_kp = smem_u32(&sm->bar_kp), bar_done = smem_u32(&sm->bar_done);
    const uint32_t p_full = smem_u32(&sm->p_full);
    auto B2 = [&](uint64_t* arr, uint32_t i) { return smem_u32(&arr[i & 1]); };

    if (tid == 0) {
        mbar_init(bar_kv, 1);
        mbar_init(bar_kp, 1);
        mbar_init(bar_done, 1);
        mbar_init(p_full, kFwdSoftmax / 32);   // one arrival per warp: hundreds of arrivals on one barrier serialise
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&sm->q_full[i]), kFwdStore / 32);
            mbar_init(smem_u32(&sm->s_full[i]), 1);
            mbar_init(smem_u32(&sm->s_empty[i]), kFwdSoftmax / 32);
            mbar_init(smem_u32(&sm->o_full[i]), 1);
            mbar_init(smem_u32(&sm->o_empty[i]), kFwdSoftmax / 32);
        }
        for (int i = 0; i < 4; ++i) mbar_init(smem_u32(&sm->unit_full[i]), 1);
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
    const uint32_t tmem_s0 = tmem, tmem_o0 = tmem + 256;

    const int hpc = P.mpp + (P.with_proxy ? 1 : 0);   // tiles per chunk
    const int lse_stride = P.mpp + 1;
    const int64_t edge_base = P.dense ? dense_edge_base(static_cast<int64_t>(P.g_begin) * P.ppk, P.S, P.NB)
                                      : static_cast<int64_t>(P.row_ptr[static_cast<int64_t>(P.g_begin) * P.ppk * P.NB]);
    uint32_t gt = 0;    // tiles seen so far by this CTA (every role counts the same sequence)
    uint32_t mt = 0;    // main-head tiles seen so far
    uint32_t nsub = 0;  // sub-units with work seen so far
    uint32_t cbase = 0; // chunks of the sub-units seen so far: row lists live in ring entry (cbase + chunk - chunk0) % 8,
                        // so the lists of a new sub-unit never land on entries the softmax group still reads
    bool bad = false;   // a bounded wait gave up: later waits are skipped, the status word is set at the end
    auto wait = [&](uint32_t bar, uint32_t parity) {
        if (!bad) bad = !mbar_wait(bar, parity);
    };
    auto warp_arrive = [&](uint32_t bar) {   // every lane has finished (and fenced) its part; one arrival per warp
        __syncwarp();
        if (lane == 0) mbar_arrive(bar);
    };

    for (uint32_t draw = 0;; ++draw) {
        // One thread draws the work and publishes it in a ring.  It passes over sub-units that lie
        // beyond the end of their row, so every published entry has work (or is the end marker) and
        // the drawing thread, whose own role needs the other roles' results to finish a sub-unit,
        // cannot get more than three entries ahead of the slowest role: a ring of four is enough.
        if (tid == kFwdSoftmax) {
            int64_t u;
            for (;;) {
                u = atomicAdd(P.counter, 1);
                if (u >= P.n_subunits) break;
                const SubUnit su = decode_subunit(u, P.NB, P.ppk);
                int n;
                if (P.dense) {
                    n = P.S - su.j * kBlock;
                } else {
                    const int g = P.g_begin + su.g;
                    const int64_t r = (static_cast<int64_t>(g / P.Hkv) * P.Hp + (g % P.Hkv) * P.ppk + su.pp) * P.NB + su.j;
                    n = P.row_ptr[r + 1] - P.row_ptr[r];
                }
                if (su.chunk0 * kBlock < n) break;
            }
            sm->unit_ring[draw & 3] = static_cast<int32_t>(u < P.n_subunits ? u : P.n_subunits);
            mbar_arrive(smem_u32(&sm->unit_full[draw & 3]));
        }
        wait(smem_u32(&sm->unit_full[draw & 3]), (draw >> 2) & 1);
        const int64_t u = sm->unit_ring[draw & 3];
        if (u >= P.n_subunits) break;
        const SubUnit su = decode_subunit(u, P.NB, P.ppk);
        const int j = su.j;
        const int g = P.g_begin + su.g;
        const int b = g / P.Hkv, kvh = g % P.Hkv;
        const int p = kvh * P.ppk + su.pp;
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
        const int chunk0 = su.chunk0;
        const int chunk1 = min((n + kBlock - 1) / kBlock, chunk0 + kChunksPerSubUnit);
        if (chunk1 <= chunk0) continue;   // this sub-unit lies beyond the end of the row
        const int ntiles = (chunk1 - chunk0) * hpc;

        if (role == 2) {
            // =========================== issuer ===========================
            if (nsub > 0) wait(bar_done, (nsub - 1) & 1);   // every product of the previous sub-unit has finished
            if (elect) {
                mbar_arrive_expect_tx(bar_kv, 2 * kTileBytes);
                tma_load_tile(tile_k, &tmap_k, j * kBlock, kvh, b, bar_kv);
                tma_load_tile(tile_v, &tmap_v, j * kBlock, kvh, b, bar_kv);
                if (P.with_proxy) {
                    mbar_arrive_expect_tx(bar_kp, kTileBytes);
                    tma_load_tile(tile_kp, &tmap_kp, j * kBlock, p / P.pg, b, bar_kp);
                }
            }
            __syncwarp();
            wait(bar_kv, nsub & 1);
            bool kp_ready = false;
            auto issue_s = [&](bool proxy, uint32_t gtile) {
                if (proxy && !kp_ready) {
                    wait(bar_kp, nsub & 1);
                    kp_ready = true;
                }
                wait(B2(sm->q_full, gtile), (gtile >> 1) & 1);
                if (gtile >= 2) wait(B2(sm->s_empty, gtile), ((gtile >> 1) - 1) & 1);
                tc_fence_after_sync();
                umma_tile_128<false, false>(tmem_s0 + (gtile & 1) * 128, tile_q0 + (gtile & 1) * kTileBytes,
                                            proxy ? tile_kp : tile_k, false, elect);
                umma_commit(B2(sm->s_full, gtile), elect);
            };
            issue_s(false, gt);
            int hh = 0;
            for (int t = 0; t < ntiles; ++t, ++gt) {
                const bool is_proxy = hh == P.mpp;
                int hh1 = hh + 1;
                if (hh1 == hpc) hh1 = 0;
                if (t + 1 < ntiles) issue_s(hh1 == P.mpp, gt + 1);     // S of the next tile first: the softmax group never starves
                if (!is_proxy) {
                    wait(p_full, mt & 1);
                    if (mt >= 2) wait(B2(sm->o_empty, mt), ((mt >> 1) - 1) & 1);
                    tc_fence_after_sync();
                    umma_tile_128<true, false>(tmem_o0 + (mt & 1) * 128, tile_v, tile_p, false, elect);   // O^T = V_j^T P^T
                    umma_commit(B2(sm->o_full, mt), elect);
                    ++mt;
                }
                hh = hh1;
            }
            umma_commit(bar_done, elect);
            if (P.with_proxy && !kp_ready) wait(bar_kp, nsub & 1);   // (every chunk has a proxy tile, so this never waits)
        } else if (role == 0) {
            // =========================== softmax group ===========================
            const int cg = warp >> 2, c0 = cg * 32;
            int hh = 0, chunk = chunk0;
            // The finished O^T of a main tile is written out by the softmax warps themselves (32 tile rows per
            // warp), in the time they would otherwise spend waiting for the next S: leaving it to the gather
            // warps made them the bottleneck.  TMEM lane = head-dimension index, column = tile row: the 32 lanes
            // of a warp store 64 contiguous bytes of ONE partial row per instruction.
            bool pending = false;        // O^T of main tile prev_mt has not been written out by this warp yet
            uint32_t prev_mt = 0;
            int prev_head = 0, prev_nrows = 0;
            int64_t prev_slot0 = 0;
            auto store_share = [&]() {
                wait(B2(sm->o_full, prev_mt), (prev_mt >> 1) & 1);   // P*V of that tile has finished (and has read P)
                tc_fence_after_sync();
                const int64_t rstride = static_cast<int64_t>(P.mpp) * kHeadDim;
#pragma unroll
                for (int c = 0; c < 32; c += 16) {
                    uint32_t v[16];
                    tmem_ld16(tmem_addr(tmem_o0 + (prev_mt & 1) * 128, quarter, 32 * cg + c), v);
                    tmem_ld_wait();
                    if (c == 16) {
                        tc_fence_before_sync();
                        warp_arrive(B2(sm->o_empty, prev_mt));
                    }
                    store_transposed_bf16_16(P.o_part + ((prev_slot0 + 32 * cg + c) * P.mpp + prev_head) * kHeadDim + row, rstride, v,
                                             32 * cg + c, prev_nrows);
                }
                pending = false;
            };
            for (int t = 0; t < ntiles; ++t, ++gt) {
                const bool is_proxy = hh == P.mpp;
                const int sb = gt & 1;
                const int nrows = min(kBlock, n - chunk * kBlock);
                wait(B2(sm->s_full, gt), (gt >> 1) & 1);
                tc_fence_after_sync();
                // (the row list was published by the gather group before it released the Q rows S was computed from)
                const int qid = sm->rows[(cbase + chunk - chunk0) & 7][row];
                const bool live = qid >= 0;
                // only the first chunk of a reverse-index row can hold rows of the key block itself
                const bool masked = (chunk == 0);
                const int limit = (masked && live && (qid >> 7) == j) ? (qid & 127) : 127;
                const uint32_t ts = tmem_s0 + sb * 128;
                float mloc = -INFINITY;
#pragma unroll
                for (int c = 0; c < 32; c += 16) {
                    uint32_t v[16];
                    tmem_ld16(tmem_addr(ts, quarter, c0 + c), v);
                    tmem_ld_wait();
                    if (masked) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) mloc = (c0 + c + i <= limit) ? fmaxf(mloc, __uint_as_float(v[i])) : mloc;
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; i += 2) mloc = fmax3(mloc, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
                    }
                }
                sm->rmax[cg][row] = mloc;               // raw logits: scale > 0, so the maximum commutes with it
                named_barrier_sync(1 + quarter, 128);   // the four warps that share these 32 rows
                const float m = fmaxf(fmaxf(sm->rmax[0][row], sm->rmax[1][row]), fmaxf(sm->rmax[2][row], sm->rmax[3][row])) *
                                P.scale_log2e;
                if (pending) store_share();   // (also: P*V of the previous main tile has read P)
                uint64_t l2 = f2_pack(0.f, 0.f);
                const uint64_t sc2 = f2_pack(P.scale_log2e, P.scale_log2e), nm2 = f2_pack(-m, -m);
#pragma unroll
                for (int c = 0; c < 32; c += 16) {
                    uint32_t v[16];
                    tmem_ld16(tmem_addr(ts, quarter, c0 + c), v);
                    tmem_ld_wait();
                    uint32_t pk[8];
#pragma unroll
                    for (int i = 0; i < 16; i += 2) {
                        float p0, p1;
                        f2_unpack(f2_fma(f2_pack(__uint_as_float(v[i]), __uint_as_float(v[i + 1])), sc2, nm2), p0, p1);
                        p0 = fast_exp2(p0);
                        p1 = fast_exp2(p1);
                        if (masked) {
                            p0 = (c0 + c + i <= limit) ? p0 : 0.f;
                            p1 = (c0 + c + i + 1 <= limit) ? p1 : 0.f;
                        }
                        l2 = f2_add(l2, f2_pack(p0, p1));
                        pk[i >> 1] = pack_bf16(p0, p1);
                    }
                    if (!is_proxy) {
#pragma unroll
                        for (int k8 = 0; k8 < 2; ++k8)
                            st_shared_v4(tile_p + swz_offset(row, ((c0 + c) >> 3) + k8), pk[4 * k8], pk[4 * k8 + 1],
                                         pk[4 * k8 + 2], pk[4 * k8 + 3]);
                    }
                }
                float l, l_hi;
                f2_unpack(l2, l, l_hi);
                l += l_hi;
                tc_fence_before_sync();
                warp_arrive(B2(sm->s_empty, gt));
                if (!is_proxy) {
                    fence_async_smem();
                    warp_arrive(p_full);
                    pending = true;
                    prev_mt = mt;
                    prev_head = hh;
                    prev_nrows = nrows;
                    prev_slot0 = e0 - edge_base + static_cast<int64_t>(chunk) * kBlock;
                    ++mt;
                }
                sm->lsum[cg][row] = l;
                named_barrier_sync(1 + quarter, 128);
                if (cg == 0 && live && row < nrows) {
                    const int64_t slot = e0 - edge_base + static_cast<int64_t>(chunk) * kBlock + row;
                    float2* st = reinterpret_cast<float2*>(P.stat_part) + slot * lse_stride + hh;
                    *st = make_float2(m, sm->lsum[0][row] + sm->lsum[1][row] + sm->lsum[2][row] + sm->lsum[3][row]);
                }
                if (++hh == hpc) {
                    hh = 0;
                    ++chunk;
                }
            }
            if (pending) store_share();
        } else {
            // =========================== gather group ===========================
            const int etid = tid - kFwdSoftmax;
            const GatherLane glane = make_gather_lane(etid);
            const __nv_bfloat16* q_b = P.q + static_cast<int64_t>(b) * P.q_sb;
            const __nv_bfloat16* qp_bp = P.qp + static_cast<int64_t>(b) * P.qp_sb + static_cast<int64_t>(p) * P.qp_sh;
            auto stage_rows = [&](int chunk) {
                if (etid < kBlock) {
                    const int at = chunk * kBlock + etid;
                    int qid = -1;
                    if (at < n) {
                        qid = P.dense ? (j * kBlock + at) : P.col_q[e0 + at];
                        if (static_cast<unsigned>(qid) >= static_cast<unsigned>(P.S) || (qid >> 7) < j) {
                            atomicMax(P.status, kStatusBadIndex);
                            qid = -1;
                        }
                    }
                    sm->rows[(cbase + chunk - chunk0) & 7][etid] = qid;
                }
            };
            // 256 threads move a 128-row tile: thread (r0 = etid/16, 16-byte chunk etid%16) covers rows r0 + 16k
            auto gather_q = [&](int hh, int chunk, uint32_t gtile) {
                const uint32_t dst = tile_q0 + (gtile & 1) * kTileBytes;
                const int* rows = sm->rows[(cbase + chunk - chunk0) & 7];
                const __nv_bfloat16* base = (hh < P.mpp) ? q_b + static_cast<int64_t>(p * P.mpp + hh) * P.q_sh : qp_bp;
                const int64_t stride = (hh < P.mpp) ? P.q_ss : P.qp_ss;
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const int rowid = rows[glane.r0 + 16 * k];
                    const bool ok = rowid >= 0;
                    cp_async_16(dst + glane.dst_off + k * 2048, base + static_cast<int64_t>(ok ? rowid : 0) * stride + glane.col, ok);
                }
            };
            // tile walk (head, chunk) for tiles t+1, t+2, t+3 without divisions
            int hh1 = 1, chunk_1 = chunk0;
            if (hh1 == hpc) { hh1 = 0; ++chunk_1; }
            int hh2 = hh1 + 1, chunk_2 = chunk_1;
            if (hh2 == hpc) { hh2 = 0; ++chunk_2; }
            // prologue: row lists of the first three tiles, Q rows of the first two
            stage_rows(chunk0);
            if (ntiles > 1 && chunk_1 != chunk0) stage_rows(chunk_1);
            if (ntiles > 2 && chunk_2 != chunk_1) stage_rows(chunk_2);
            named_barrier_sync(5, kFwdStore);
            if (gt >= 2) wait(B2(sm->s_full, gt), ((gt >> 1) - 1) & 1);        // the Q buffers' last readers are done
            if (gt >= 1) wait(B2(sm->s_full, gt + 1), (((gt + 1) >> 1) - 1) & 1);
            gather_q(0, chunk0, gt);
            cp_async_commit();
            if (ntiles > 1) gather_q(hh1, chunk_1, gt + 1);
            cp_async_commit();
            cp_async_wait<1>();
            fence_async_smem();
            warp_arrive(B2(sm->q_full, gt));
            for (int t = 0; t < ntiles; ++t, ++gt) {
                int hh3 = hh2 + 1, chunk_3 = chunk_2;
                if (hh3 == hpc) { hh3 = 0; ++chunk_3; }
                // Q rows of tile t+2 go into the buffer S(t) has finished reading
                if (t + 2 < ntiles) {
                    wait(B2(sm->s_full, gt), (gt >> 1) & 1);
                    gather_q(hh2, chunk_2, gt + 2);
                }
                cp_async_commit();
                if (t + 3 < ntiles && chunk_3 != chunk_2) stage_rows(chunk_3);
                if (t + 1 < ntiles) {
                    cp_async_wait<1>();     // tile t+1 has landed (t+2 may still be in flight)
                    fence_async_smem();
                    warp_arrive(B2(sm->q_full, gt + 1));
                }
                named_barrier_sync(5, kFwdStore);   // row list of tile t+3 visible to the whole group before its gather
                hh1 = hh2; chunk_1 = chunk_2;
                hh2 = hh3; chunk_2 = chunk_3;
            }
        }
        cbase += static_cast<uint32_t>(chunk1 - chunk0);
        ++nsub;
    }
    cp_async_wait<0>();
    if (role == 2 && nsub > 0) wait(bar_done, (nsub - 1) & 1);
    if (bad) atomicMax(P.status, kStatusWaitTimeout);
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

    const float2* stats = reinterpret_cast<const float2*>(P.lse_part);
    const int nheads = P.mpp + (P.lse_proxy ? 1 : 0);
    for (int hh = 0; hh < nheads; ++hh) {
        // pass A: every partial carries (row max m in the log2 domain, row sum l); merge them
        float m = -INFINITY, sum = 0.f;
        for (int s0 = 0; s0 < nslots; s0 += 32) {
            const int64_t sl = slot_of(s0 + lane);
            if (sl >= 0) {
                const float2 st = stats[sl * lse_stride + hh];
                const float mn = fmaxf(m, st.x);
                sum = sum * fast_exp2(m - mn) + st.y * fast_exp2(st.x - mn);
                m = mn;
            }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float mo = __shfl_xor_sync(0xffffffffu, m, off);
            const float so = __shfl_xor_sync(0xffffffffu, sum, off);
            const float mn = fmaxf(m, mo);
            const float a = (m == -INFINITY) ? 0.f : sum * fast_exp2(m - mn);
            const float c = (mo == -INFINITY) ? 0.f : so * fast_exp2(mo - mn);
            sum = a + c;
            m = mn;
        }
        const float total = (m + __log2f(sum)) * kLn2;   // natural-log LSE of the whole row
        if (hh == P.mpp) {
            if (lane == 0) P.lse_proxy[bp * P.S + q] = total;
            continue;
        }
        const int h = p * P.mpp + hh;
        if (lane == 0) P.lse[(static_cast<int64_t>(b) * P.Hq + h) * P.S + q] = total;
        // pass B: weighted sum of the unnormalised partial outputs; lane owns columns 4*lane..4*lane+3
        const float inv = 1.f / sum;
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
        for (int s0 = 0; s0 < nslots; s0 += 32) {
            const int64_t sl = slot_of(s0 + lane);
            const float wgt = sl >= 0 ? fast_exp2(stats[sl * lse_stride + hh].x - m) * inv : 0.f;
            const int cnt = min(32, nslots - s0);
#pragma unroll 4
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

// Wide variant for Hq/Hp <= 8: the partial rows of all main heads of one edge are contiguous
// (mpp * 256 bytes), so a warp reads them with 16-byte loads per lane in one sweep instead of one
// 256-byte row at a time; weights go through shared memory.
// KITER = number of 512-byte sweeps per edge record: Hq/Hp <= 2*KITER.  Templated so that the common
// small head ratios keep few accumulators in registers and reach a high occupancy (the kernel is
// bound by memory latency).
constexpr int kWideMaxHeads = 8;
template <int KITER>
__global__ void __launch_bounds__(256, (KITER <= 2) ? 4 : 2) combine_wide_kernel(const CombineParams P) {
    constexpr int kWideMaxHeads = 2 * KITER;
    __shared__ float wsm[8][32][kWideMaxHeads + 1];
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const int64_t w = static_cast<int64_t>(blockIdx.x) * 8 + wib;
    const int64_t bp0 = static_cast<int64_t>(P.g_begin) * P.ppk;
    if (w >= static_cast<int64_t>(P.G) * P.ppk * P.S) return;
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
    const float2* stats = reinterpret_cast<const float2*>(P.lse_part);
    const int nheads = P.mpp + (P.lse_proxy ? 1 : 0);

    // pass A: merged (max, sum) of every head over all slots
    float hm[kWideMaxHeads + 1], hs[kWideMaxHeads + 1];
#pragma unroll
    for (int hh = 0; hh <= kWideMaxHeads; ++hh) {
        hm[hh] = -INFINITY;
        hs[hh] = 0.f;
    }
    for (int s0 = 0; s0 < nslots; s0 += 32) {
        const int64_t sl = slot_of(s0 + lane);
#pragma unroll
        for (int hh = 0; hh <= kWideMaxHeads; ++hh) {
            if (hh < nheads && sl >= 0) {
                const float2 st = stats[sl * lse_stride + hh];
                const float mn = fmaxf(hm[hh], st.x);
                hs[hh] = hs[hh] * fast_exp2(hm[hh] - mn) + st.y * fast_exp2(st.x - mn);
                hm[hh] = mn;
            }
        }
    }
#pragma unroll
    for (int hh = 0; hh <= kWideMaxHeads; ++hh) {
        if (hh < nheads) {
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                const float mo = __shfl_xor_sync(0xffffffffu, hm[hh], off);
                const float so = __shfl_xor_sync(0xffffffffu, hs[hh], off);
                const float mn = fmaxf(hm[hh], mo);
                const float a = (hm[hh] == -INFINITY) ? 0.f : hs[hh] * fast_exp2(hm[hh] - mn);
                const float c = (mo == -INFINITY) ? 0.f : so * fast_exp2(mo - mn);
                hs[hh] = a + c;
                hm[hh] = mn;
            }
            const float total = (hm[hh] + __log2f(hs[hh])) * kLn2;
            if (lane == 0) {
                if (hh == P.mpp) P.lse_proxy[bp * P.S + q] = total;
                else P.lse[(static_cast<int64_t>(b) * P.Hq + p * P.mpp + hh) * P.S + q] = total;
            }
        }
    }
    // pass B: lane owns 16-byte chunks ck = k*32 + lane of the mpp*128-element edge record
    const int nchunk = P.mpp * 16;
    float acc[KITER][8];
#pragma unroll
    for (int k = 0; k < KITER; ++k)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[k][e] = 0.f;
    for (int s0 = 0; s0 < nslots; s0 += 32) {
        const int64_t sl = slot_of(s0 + lane);
        __syncwarp();
#pragma unroll
        for (int hh = 0; hh < kWideMaxHeads; ++hh)
            if (hh < P.mpp) wsm[wib][lane][hh] = sl >= 0 ? fast_exp2(stats[sl * lse_stride + hh].x - hm[hh]) / hs[hh] : 0.f;
        __syncwarp();
        const int cnt = min(32, nslots - s0);
#pragma unroll 4
        for (int i = 0; i < cnt; ++i) {
            const int64_t si = __shfl_sync(0xffffffffu, sl, i);
            if (si < 0) continue;
            const __nv_bfloat16* rec = P.o_part + si * P.mpp * kHeadDim;
#pragma unroll
            for (int k = 0; k < KITER; ++k) {
                const int ck = k * 32 + lane;
                if (ck < nchunk) {
                    const float wgt = wsm[wib][i][ck >> 4];
                    const uint4 raw = *reinterpret_cast<const uint4*>(rec + ck * 8);
                    const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const __nv_bfloat162 v2 = *reinterpret_cast<const __nv_bfloat162*>(&u[e]);
                        acc[k][2 * e] += wgt * __low2float(v2);
                        acc[k][2 * e + 1] += wgt * __high2float(v2);
                    }
                }
            }
        }
    }
    __nv_bfloat16* orow = P.out + (static_cast<int64_t>(b) * P.S + q) * (static_cast<int64_t>(P.Hq) * kHeadDim) +
                          static_cast<int64_t>(p) * P.mpp * kHeadDim;
#pragma unroll
    for (int k = 0; k < KITER; ++k) {
        const int ck = k * 32 + lane;
        if (ck < nchunk) {
            uint4 o;
            o.x = pack_bf16(acc[k][0], acc[k][1]);
            o.y = pack_bf16(acc[k][2], acc[k][3]);
            o.z = pack_bf16(acc[k][4], acc[k][5]);
            o.w = pack_bf16(acc[k][6], acc[k][7]);
            *reinterpret_cast<uint4*>(orow + ck * 8) = o;
        }
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
    P.o_part = static_cast<__nv_bfloat16*>(o_part); P.stat_part = lse_part;
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
    P.n_subunits = g_count * subunits_per_group(P.NB, P.ppk, kChunksPerSubUnit);
    FMSA_REQUIRE(P.n_subunits < 0x7fffffffLL);
    const int grid = static_cast<int>(P.n_subunits < sms ? P.n_subunits : sms);
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
    const dim3 cg(static_cast<unsigned>(grid));
    cudaStream_t cst = static_cast<cudaStream_t>(stream);
    if (P.mpp <= 2)
        combine_wide_kernel<1><<<cg, 256, 0, cst>>>(P);
    else if (P.mpp <= 4)
        combine_wide_kernel<2><<<cg, 256, 0, cst>>>(P);
    else if (P.mpp <= 6)
        combine_wide_kernel<3><<<cg, 256, 0, cst>>>(P);
    else if (P.mpp <= 8)
        combine_wide_kernel<4><<<cg, 256, 0, cst>>>(P);
    else
        combine_kernel<<<static_cast<unsigned>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(P);
    return check_launch();
}
