// Fused MSA backward, key-block stationary: dQ, dK, dV and the on-the-fly KL gradients dQp, dKp.
//
// Work unit = (batch, KV head, key block j), exactly as in the forward: K_j and V_j stay in shared
// memory, the unit walks the reverse-index row of every proxy head of its group in chunks of 128
// gathered query rows.  For each chunk the main heads of the proxy head run one after another.  Scores
// are computed TRANSPOSED (TMEM lane = key, column = query) so that P^T and dS^T, written back into TMEM
// as bf16 over the columns S^T and dP^T occupied, are the TMEM operands of the dV and dK products:
//     S^T = K_j Q_g^T           dP^T = V_j dO_g^T                   (both operands in shared memory)
//     P^T = exp2(S^T*c - lse)   dS^T = P^T o (dP^T - delta)         (fp32, rounded to bf16)
//     dV += P^T dO_g            dK += dS^T Q_g                      (A operand in TMEM; accumulators stay in
//                                                                    TMEM for the whole sub-unit)
//     dQ  = dS K_j                                                  (dS^T also goes to shared memory)
// while every thread sums the P of its (key, queries) over the heads: the KL teacher.
// Then one proxy tile:
//     Sp^T = Kp_j Qp_g^T        p_px = exp2(Sp^T*c - lse_proxy)     dSp^T = p_px - teacher/mpp
//     dKp = dSp^T Qp_g, dQp = dSp Kp_j.
// dQ and dQp leave as bf16 per-edge partial rows (a combine kernel sums them per query row, applying
// scale and scale/(B*Hp*S)); dK, dV (once per sub-unit) and dKp (once per proxy tile) are added to fp32
// accumulators with vector reductions and cast afterwards.
//
// Formulas and rounding points follow the reference kernel
// (flash_msa/msa_backward_cutedsl.py:456-733: P and dS rounded to the input type before the
// second products, ds_px = c*(p_px - teacher)) and flash_msa/flash_msa.py:99-125 (delta, 1/(B*Hp*S),
// grad_kl applied afterwards on the device).  Differences: the teacher is summed from the unrounded P in
// fp16 pairs, and dSp is rounded to bf16 before the 1/(B*Hp*S) factor is applied.
// `dense` mode is the warmup backward (flash_msa/warmup/msa_backward_cutedsl_warmup.py:117-191):
// every causal (query block, key block) pair, with the schedule implied instead of built on the host.
#include <cuda_fp16.h>

#include <type_traits>

#include "host_common.h"
#include "msa_common.cuh"
#include "sm100.cuh"
#include "tma_host.h"

namespace fmsa {
namespace {

#ifdef FMSA_TRACE
// Debug builds only: cycles each warp of CTA 0 spent inside its role (slot 0) and inside waits of kind 1..7.
__device__ unsigned long long g_bwd_trace[20][8];
#endif

struct BwdParams {
    // Row-gather views: element row (b, h, s) of q / d_out / q_proxy is matrix row b*row_b + h*row_h + s*row_s.
    int64_t q_row_b, q_row_h, q_row_s;
    int64_t do_row_b, do_row_h, do_row_s;
    int64_t qp_row_b, qp_row_h, qp_row_s;
    int32_t q_rows_total, do_rows_total, qp_rows_total;   // first row index outside each view (reads as zeros)
    const float *lse, *lse_proxy, *delta;   // [B,Hq,S], [B,Hp,S], [B,Hq,S]
    const int32_t* row_ptr;
    const int32_t* col_q;
    const int32_t* doc_start;   // [B,S] first token of each token's document (packed sequences), or null
    __nv_bfloat16* dq_part;    // [(edge - edge_base) * mpp + head][128]: per-edge dQ contributions (unscaled)
    __nv_bfloat16* dqp_part;   // [(edge - edge_base)][128]: per-edge dQp contributions (unscaled)
    int64_t part_slots;        // slots per plane of the two buffers above
    int split;                 // 1: every contribution is stored as a bf16 pair (value, rounding remainder) in two planes
    // fp32, zero-initialised: [B,Hpkv,S,128], [B,Hkv,S,128] x2
    float *dkp_acc, *dk_acc, *dv_acc;
    int32_t* counter;
    int32_t* status;
    int S, NB, Hq, Hkv, Hp, Hpkv, mpp, ppk, pg;
    int g_begin, G;
    int64_t n_subunits;
    int with_kl, dense;
    float scale_log2e;
    float* kl_value;        // optional: += KL(teacher || proxy) summed over this launch's rows, / (B*Hp*S)
    float kl_value_scale;   // ln(2) / (B*Hp*S)
};

struct BwdUnit {   // (kept small: the control block shares the last 3 KB of shared memory with the row statistics)
    int64_t e0;
    int32_t n;
    uint16_t j, b, kvh, p, chunk0;   // (B*Hp < 65536 and S/128 <= 2048 are required by the entry point)
    int16_t chunk1;                  // < 0: no more work
};

constexpr int kBwdUnitRing = 8;

// Per-tile facts about the 128 gathered query rows (= TMEM columns), staged for the compute groups.
struct alignas(16) BwdRowStats {   // (filled and read with 16-byte vector accesses)
    float neg_lse[128];    // -lse * log2(e); -inf for a dead row, whose probabilities then come out as 0
    float neg_delta[128];  // -delta
    uint8_t limit[128];    // last visible key of the row inside this key block (127 = all)
    uint8_t low[128];      // first visible key (0 = all, 128 = none): document masking; written only with documents
    int32_t any_low;       // some row of the tile has low > 0
};

struct BwdCtrl {
    uint64_t k_full, v_full, kv_empty, acc_full, acc_free;
    uint64_t q_full[2], q_empty[2], do_full[2], do_empty[2], st_full[2], st_empty[2];
    uint64_t sdp_full, pds_full, dq_full, r0_free, ds_free, dkp_full, r1_free;
    uint64_t unit_full[kBwdUnitRing];
    BwdUnit units[kBwdUnitRing];
    BwdRowStats stats[2];
    uint32_t tmem_slot;
    int32_t abort_flag;
};

// Roles (warp index): 0-3 compute group A (queries 0..63 of a tile), 4-7 compute group B (queries 64..127),
// 8-11 output group, 12-15 row gather (Q, dO, Qp; Kp_j), 16 K/V loads and row statistics, 17 MMA issue (18, 19 only
// take part in the block-wide steps).  A TMA row gather costs the issuing warp ~65 cycles whatever its size, so the
// 128 gathers of a tile are spread over four warps.
constexpr int kBwdGatherWarps = 4;
constexpr int kBwdThreads = 20 * 32;
// Registers per thread after the warpgroups re-divide the register file (setmaxnreg).  A CTA of 640 threads is
// launched with 96 registers per thread; an increase can only be served from what the other warpgroups of the
// same CTA gave up, so the five warpgroups must not ask for more than 5 x 96 in total (a warpgroup that asks for
// registers nobody released waits forever).
constexpr int kBwdRegsLaunch = 96, kBwdRegsCompute = 136, kBwdRegsOutput = 88, kBwdRegsGather = 56, kBwdRegsMisc = 64;
static_assert(2 * kBwdRegsCompute + kBwdRegsOutput + kBwdRegsGather + kBwdRegsMisc <= 5 * kBwdRegsLaunch,
              "register re-division must balance");
static_assert(kBwdRegsLaunch == (65536 / kBwdThreads) / 8 * 8, "registers per thread at launch");
constexpr size_t kBwdTileBytes = 7 * static_cast<size_t>(kTileBytes);   // K, V, Q x2, dO x2, dS^T
constexpr size_t kBwdSmemBytes = 232448;                                 // everything a CTA can have
static_assert(kBwdTileBytes + sizeof(BwdCtrl) <= kBwdSmemBytes, "shared memory budget of one CTA");
constexpr int kStatusBadSmem = 3;   // the dynamic shared memory window does not start on a 1024-byte boundary

// Warp-specialised backward.  Every role walks the same sequence of sub-units (published by the gather warp in a
// ring) and of tiles.  TMEM (512 columns):
//   R0 [0,128)   S^T, overwritten in place by P^T (bf16: queries 0..63 in columns 0..31, queries 64..127 in columns
//                64..95), then dQ (lane = query).  Proxy tile: Sp^T, dSp^T parked in place, then dQp.
//   R1 [128,256) dP^T, overwritten by dS^T in the same split.  Proxy tile: dKp^T (lane = head dimension).
//   R2 [256,384) dV, R3 [384,512) dK (lane = key), accumulated over the sub-unit.
// Issue order of a main tile t (one full product always lies between a product that reads a TMEM operand and a
// later one that overwrites those columns):
//   [compute(t) done]  dV += P^T dO,  dK += dS^T Q,  dQ = dS K -> R0,  dP^T(t+1) -> R1,  [dQ read out]  S^T(t+1) -> R0.
// Hand-offs (mbarriers; one arrival per warp or per tcgen05.commit): q_full/do_full (TMA bytes) <- q_empty/do_empty;
// st_full <- st_empty (row statistics); sdp_full (S^T and dP^T of a tile), pds_full (P^T, dS^T written), dq_full,
// r0_free (dQ read out), ds_free (the dS^T tile, which doubles as the staging tile of the dQ store, is reusable),
// dkp_full / r1_free (proxy tile), acc_full / acc_free (dV, dK flushed at the end of a sub-unit).
// VARLEN: document masking of packed sequences (P.doc_start given).  A separate instantiation, so that the plain kernel
// carries none of its registers or code.
template <bool FP16, bool VARLEN>
__global__ void __launch_bounds__(kBwdThreads, 1) sparse_bwd_kernel(const __grid_constant__ CUtensorMap tmap_q,
                                                                    const __grid_constant__ CUtensorMap tmap_do,
                                                                    const __grid_constant__ CUtensorMap tmap_qp,
                                                                    const __grid_constant__ CUtensorMap tmap_k,
                                                                    const __grid_constant__ CUtensorMap tmap_v,
                                                                    const __grid_constant__ CUtensorMap tmap_kp,
                                                                    const __grid_constant__ CUtensorMap tmap_dq,
                                                                    const __grid_constant__ CUtensorMap tmap_dqp,
                                                                    const BwdParams P) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
    if ((tiles - smem_u32(smem_raw)) + kBwdTileBytes + sizeof(BwdCtrl) > kBwdSmemBytes) {
        if (threadIdx.x == 0) atomicMax(P.status, kStatusBadSmem);
        return;
    }
    const uint32_t tile_k = tiles, tile_v = tiles + kTileBytes;
    const uint32_t tile_q0 = tiles + 2 * kTileBytes, tile_do0 = tiles + 4 * kTileBytes, tile_ds = tiles + 6 * kTileBytes;
    BwdCtrl* sm = reinterpret_cast<BwdCtrl*>(smem_raw + (tiles - smem_u32(smem_raw)) + kBwdTileBytes);

    const int tid = threadIdx.x, warp = __shfl_sync(0xffffffffu, tid >> 5, 0), lane = tid & 31;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;   // TMEM lane of this thread: key (compute, dKp/dV/dK read-out) or query (dQ read-out)
    const uint32_t elect = (lane == 0) ? 1u : 0u;
    auto BAR = [&](uint64_t& b) { return smem_u32(&b); };

    if (tid == 0) {
        mbar_init(BAR(sm->k_full), 1);
        mbar_init(BAR(sm->v_full), 1);
        mbar_init(BAR(sm->kv_empty), 1);
        mbar_init(BAR(sm->acc_full), 1);
        mbar_init(BAR(sm->acc_free), 4);
        for (int i = 0; i < 2; ++i) {
            mbar_init(BAR(sm->q_full[i]), kBwdGatherWarps);
            mbar_init(BAR(sm->q_empty[i]), 1);
            mbar_init(BAR(sm->do_full[i]), kBwdGatherWarps);
            mbar_init(BAR(sm->do_empty[i]), 1);
            mbar_init(BAR(sm->st_full[i]), 1);
            mbar_init(BAR(sm->st_empty[i]), 8);
        }
        mbar_init(BAR(sm->sdp_full), 1);
        mbar_init(BAR(sm->pds_full), 8);
        mbar_init(BAR(sm->dq_full), 1);
        mbar_init(BAR(sm->r0_free), 4);
        mbar_init(BAR(sm->ds_free), 1);
        mbar_init(BAR(sm->dkp_full), 1);
        mbar_init(BAR(sm->r1_free), 4);
        for (int i = 0; i < kBwdUnitRing; ++i) mbar_init(BAR(sm->unit_full[i]), 1);
        sm->abort_flag = 0;
        fence_mbar_init();
        prefetch_tmap(&tmap_q);
        prefetch_tmap(&tmap_do);
        prefetch_tmap(&tmap_k);
        prefetch_tmap(&tmap_v);
        prefetch_tmap(&tmap_dq);
        if (P.with_kl) {
            prefetch_tmap(&tmap_qp);
            prefetch_tmap(&tmap_kp);
            prefetch_tmap(&tmap_dqp);
        }
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(&sm->tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = sm->tmem_slot;
    const uint32_t r0 = tmem, r1 = tmem + 128, r2 = tmem + 256, r3 = tmem + 384;

    const int hpc = P.mpp + (P.with_kl ? 1 : 0);   // tiles per chunk
    const int64_t edge_base = P.dense ? dense_edge_base(static_cast<int64_t>(P.g_begin) * P.ppk, P.S, P.NB)
                                      : static_cast<int64_t>(P.row_ptr[static_cast<int64_t>(P.g_begin) * P.ppk * P.NB]);
    volatile int* abort_flag = &sm->abort_flag;
    bool bad = false;   // a bounded wait gave up (here or in another role): the thread stops taking work
#ifdef FMSA_TRACE
    unsigned long long trace_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const long long trace_t0 = clock64();
#endif
    auto wait = [&](uint32_t bar, uint32_t parity, int kind = 1) {   // every lane of the warp calls it; the result is warp-uniform
#ifdef FMSA_TRACE
        const long long w0 = clock64();
#endif
        if (!bad) bad = __any_sync(0xffffffffu, !mbar_wait_abortable(bar, parity, abort_flag));
#ifdef FMSA_TRACE
        trace_acc[kind & 7] += static_cast<unsigned long long>(clock64() - w0);
#endif
        (void)kind;
    };
    auto group_or = [&](int id, bool flag) -> bool {   // 128-thread barrier that also ORs a flag
        uint32_t r;
        asm volatile(
            "{\n"
            ".reg .pred p, q;\n"
            "setp.ne.b32 q, %1, 0;\n"
            "barrier.cta.red.or.pred p, %2, 128, q;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(r)
            : "r"(flag ? 1u : 0u), "r"(id)
            : "memory");
        return r != 0;
    };
    auto warp_arrive = [&](uint32_t bar) {
        __syncwarp();
        if (lane == 0) mbar_arrive(bar);
    };

    uint32_t gt = 0;     // tiles seen so far by this CTA (every role counts the same sequence)
    uint32_t pt = 0;     // proxy tiles seen so far
    uint32_t nsub = 0;   // sub-units seen so far
    float kl_acc = 0.f;  // compute groups: this thread's share of sum t * (log2 t - log2 p_proxy)

    // Next sub-unit of the common sequence (false: no more work, or the CTA is giving up).  The gather warp draws the
    // work and publishes the decoded sub-unit; it passes over sub-units that lie beyond the end of their row, so
    // every published entry has work (or is the end marker).  The roles are at most a few tiles apart, fewer than the
    // ring has entries.
    auto next_unit = [&](uint32_t draw, BwdUnit& ud, auto may_draw) -> bool {
        const uint32_t uslot = draw & (kBwdUnitRing - 1);
        if (decltype(may_draw)::value && warp == 12 && lane == 0) {
            BwdUnit nu;
            nu.chunk1 = -1;
            for (;;) {
                const int64_t u = atomicAdd(P.counter, 1);
                if (u >= P.n_subunits) break;
                const SubUnit su = decode_subunit(u, P.NB, P.ppk);
                const int g = P.g_begin + su.g;
                const int b = g / P.Hkv, kvh = g % P.Hkv, p = kvh * P.ppk + su.pp;
                const int64_t bp = static_cast<int64_t>(b) * P.Hp + p;
                int64_t e0;
                int n;
                if (P.dense) {
                    e0 = dense_edge_base(bp, P.S, P.NB) + dense_row_offset(su.j, P.S);
                    n = P.S - su.j * kBlock;
                } else {
                    e0 = P.row_ptr[bp * P.NB + su.j];
                    n = P.row_ptr[bp * P.NB + su.j + 1] - static_cast<int>(e0);
                }
                if (su.chunk0 * kBlock < n) {
                    nu.j = static_cast<uint16_t>(su.j); nu.b = static_cast<uint16_t>(b); nu.kvh = static_cast<uint16_t>(kvh);
                    nu.p = static_cast<uint16_t>(p); nu.n = n; nu.e0 = e0;
                    nu.chunk0 = static_cast<uint16_t>(su.chunk0);
                    nu.chunk1 = static_cast<int16_t>(min((n + kBlock - 1) / kBlock, su.chunk0 + kChunksPerSubUnit));
                    break;
                }
            }
            sm->units[uslot] = nu;
            mbar_arrive(BAR(sm->unit_full[uslot]));
        }
        wait(BAR(sm->unit_full[uslot]), (draw / kBwdUnitRing) & 1, 7);
        if (warp >= 8 && warp < 12) bad = group_or(1, bad);
        if (bad) return false;
        ud = sm->units[uslot];
        return ud.chunk1 >= 0;
    };
    // query position of row `at` of a reverse-index row, -1 when there is none (or the index is bad)
    auto row_qid = [&](const BwdUnit& ud, int at) -> int {
        if (at >= ud.n) return -1;
        const int q = P.dense ? (ud.j * kBlock + at) : P.col_q[ud.e0 + at];
        if (static_cast<unsigned>(q) >= static_cast<unsigned>(P.S) || (q >> 7) < ud.j) {
            atomicMax(P.status, kStatusBadIndex);
            return -1;
        }
        return q;
    };

    // Every role has its own loop over the common sequence of sub-units (separate loops keep the register
    // allocation of one role from being charged with the live values of the others).
    if (warp >= 16) {
        reg_dec<kBwdRegsMisc>();
        if (warp == 17) {
            // =========================== MMA issue ===========================
            BwdUnit ud;
            for (uint32_t draw = 0; next_unit(draw, ud, std::false_type{}); ++draw, ++nsub) {
                const int ntiles = (ud.chunk1 - ud.chunk0) * hpc;
                wait(BAR(sm->k_full), nsub & 1, 6);
                wait(BAR(sm->v_full), nsub & 1, 6);
                // S^T and dP^T of tile g (running index), whose predecessor was tile g-1
                auto issue_front = [&](uint32_t g, bool proxy, bool prev_proxy) {
                    const uint32_t s = g & 1, ph = (g >> 1) & 1;
                    const uint32_t tq = tile_q0 + s * kTileBytes, tdo = tile_do0 + s * kTileBytes;
                    wait(BAR(sm->do_full[s]), ph, 1);
                    if (!proxy) {
                        if (g >= 1 && prev_proxy) wait(BAR(sm->r1_free), (pt - 1) & 1, 4);   // dKp has been read out of R1
                        tc_fence_after_sync();
                        if (!bad) umma_tile_128<false, false, FP16>(r1, tile_v, tdo, false, elect);   // dP^T = V_j dO_g^T
                    }
                    wait(BAR(sm->q_full[s]), ph, 2);
                    if (g >= 1) wait(BAR(sm->r0_free), (g - 1) & 1, 3);                       // dQ / dQp has been read out of R0
                    tc_fence_after_sync();
                    if (!bad) {
                        umma_tile_128<false, false, FP16>(r0, proxy ? tdo : tile_k, tq, false, elect);   // S^T = K_j Q_g^T  (Sp^T = Kp_j Qp_g^T)
                        umma_commit(BAR(sm->sdp_full), elect);
                    }
                };
                issue_front(gt, false, P.with_kl != 0);   // (a sub-unit ends with a proxy tile when there are any)
                int hh = 0;
                for (int t = 0; t < ntiles && !bad; ++t, ++gt) {
                    const bool is_proxy = hh == P.mpp;
                    const uint32_t s = gt & 1;
                    const uint32_t tq = tile_q0 + s * kTileBytes, tdo = tile_do0 + s * kTileBytes;
                    int hh1 = hh + 1;
                    if (hh1 == hpc) hh1 = 0;
                    wait(BAR(sm->pds_full), gt & 1, 5);
                    tc_fence_after_sync();
                    if (!is_proxy) {
                        if (t == 0 && nsub > 0) wait(BAR(sm->acc_free), (nsub - 1) & 1, 6);   // dV, dK of the previous sub-unit flushed
                        if (!bad) {
                            umma_tile_128_ts<true, FP16>(r2, r0, r0 + 64, tdo, t != 0, elect);    // dV += P^T dO_g
                            umma_commit(BAR(sm->do_empty[s]), elect);
                            umma_tile_128_ts<true, FP16>(r3, r1, r1 + 64, tq, t != 0, elect);     // dK += dS^T Q_g
                            umma_commit(BAR(sm->q_empty[s]), elect);
                            umma_tile_128<true, true, FP16>(r0, tile_ds, tile_k, false, elect);   // dQ = dS K_j
                            umma_commit(BAR(sm->dq_full), elect);
                        }
                    } else {
                        if (!bad) {
                            umma_tile_128<true, false, FP16>(r1, tq, tile_ds, false, elect);      // dKp^T = Qp_g^T dSp  (lane = head dim)
                            umma_commit(BAR(sm->dkp_full), elect);
                            umma_tile_128<true, true, FP16>(r0, tile_ds, tdo, false, elect);      // dQp = dSp Kp_j
                            umma_commit(BAR(sm->dq_full), elect);
                            umma_commit(BAR(sm->q_empty[s]), elect);
                            umma_commit(BAR(sm->do_empty[s]), elect);
                        }
                        ++pt;
                    }
                    if (t + 1 < ntiles) issue_front(gt + 1, hh1 == P.mpp, is_proxy);
                    hh = hh1;
                }
                if (!bad) {
                    umma_commit(BAR(sm->kv_empty), elect);
                    umma_commit(BAR(sm->acc_full), elect);
                }
            }
        } else if (warp == 16) {
            // =========================== K / V loads, row statistics ===========================
            BwdUnit ud;
            for (uint32_t draw = 0; next_unit(draw, ud, std::false_type{}); ++draw, ++nsub) {
                const int64_t bp = static_cast<int64_t>(ud.b) * P.Hp + ud.p;
                if (nsub > 0) wait(BAR(sm->kv_empty), (nsub - 1) & 1, 1);
                if (!bad && lane == 0) {
                    mbar_arrive_expect_tx(BAR(sm->k_full), kTileBytes);
                    tma_load_tile(tile_k, &tmap_k, ud.j * kBlock, ud.kvh, ud.b, BAR(sm->k_full));
                    mbar_arrive_expect_tx(BAR(sm->v_full), kTileBytes);
                    tma_load_tile(tile_v, &tmap_v, ud.j * kBlock, ud.kvh, ud.b, BAR(sm->v_full));
                }
                __syncwarp();
                for (int chunk = ud.chunk0; chunk < ud.chunk1 && !bad; ++chunk) {
                    int qid[4];
                    uint32_t lim4 = 0, low4 = 0;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        qid[i] = row_qid(ud, chunk * kBlock + 4 * lane + i);
                        const uint32_t lim = (qid[i] >= 0 && (qid[i] >> 7) == ud.j) ? static_cast<uint32_t>(qid[i] & 127) : 127u;
                        lim4 |= lim << (8 * i);
                        if (VARLEN && qid[i] >= 0) {
                            const int lo = P.doc_start[static_cast<int64_t>(ud.b) * P.S + qid[i]];
                            const int lb = lo >> 7;
                            low4 |= static_cast<uint32_t>(lb < ud.j ? 0 : (lb == ud.j ? (lo & 127) : 128)) << (8 * i);
                        }
                    }
                    const bool any_low = VARLEN && __any_sync(0xffffffffu, low4 != 0);
                    for (int hh = 0; hh < hpc && !bad; ++hh, ++gt) {
                        const uint32_t s = gt & 1;
                        const bool proxy = hh == P.mpp;
                        float nl[4], dl[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            nl[i] = -INFINITY;
                            dl[i] = 0.f;
                            if (qid[i] >= 0) {
                                if (proxy) {
                                    nl[i] = -P.lse_proxy[bp * P.S + qid[i]] * kLog2e;
                                } else {
                                    const int64_t at = (static_cast<int64_t>(ud.b) * P.Hq + ud.p * P.mpp + hh) * P.S + qid[i];
                                    nl[i] = -P.lse[at] * kLog2e;
                                    dl[i] = -P.delta[at];
                                }
                            }
                        }
                        if (gt >= 2) wait(BAR(sm->st_empty[s]), ((gt >> 1) - 1) & 1, 2);
                        if (bad) break;
                        BwdRowStats* st = &sm->stats[s];
                        reinterpret_cast<float4*>(st->neg_lse)[lane] = make_float4(nl[0], nl[1], nl[2], nl[3]);
                        reinterpret_cast<float4*>(st->neg_delta)[lane] = make_float4(dl[0], dl[1], dl[2], dl[3]);
                        reinterpret_cast<uint32_t*>(st->limit)[lane] = lim4;
                        if (VARLEN) {
                            reinterpret_cast<uint32_t*>(st->low)[lane] = low4;
                            if (lane == 0) st->any_low = any_low ? 1 : 0;
                        }
                        warp_arrive(BAR(sm->st_full[s]));
                    }
                }
            }
        }
    } else if (warp >= 12) {
        reg_dec<kBwdRegsGather>();
        // =========================== row gather ===========================
        // Gather warp g fetches rows 32g .. 32g+31 of every tile: lanes 0..15 issue the dO rows (dP^T is issued before
        // S^T), lanes 16..31 the Q rows; a lane takes row quad (lane/2)%8 and 64-column panel lane%2.  Lane r holds the
        // query position of row 32g + r.  In a proxy tile the Q stage takes the Qp rows and the dO stage the proxy keys
        // of the block (one ordinary tile load by the first gather warp).
        const int g = warp - 12;
        const int quad = (lane >> 1) & 7, panel = lane & 1;
        const bool q_lane = lane >= 16;
        BwdUnit ud;
        for (uint32_t draw = 0; next_unit(draw, ud, std::true_type{}); ++draw, ++nsub) {
            const int64_t q_base = static_cast<int64_t>(ud.b) * P.q_row_b + static_cast<int64_t>(ud.p) * P.mpp * P.q_row_h;
            const int64_t do_base = static_cast<int64_t>(ud.b) * P.do_row_b + static_cast<int64_t>(ud.p) * P.mpp * P.do_row_h;
            const int64_t qp_base = static_cast<int64_t>(ud.b) * P.qp_row_b + static_cast<int64_t>(ud.p) * P.qp_row_h;
            for (int chunk = ud.chunk0; chunk < ud.chunk1 && !bad; ++chunk) {
                const int q = row_qid(ud, chunk * kBlock + 32 * g + lane);
                int qr[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) qr[i] = __shfl_sync(0xffffffffu, q, 4 * quad + i);
                for (int hh = 0; hh < hpc && !bad; ++hh, ++gt) {
                    const uint32_t s = gt & 1, ph = (gt >> 1) & 1;
                    const bool proxy = hh == P.mpp;
                    const uint32_t qf = BAR(sm->q_full[s]), df = BAR(sm->do_full[s]);
                    const uint32_t off = panel * kPanelBytes + (32 * g + 4 * quad) * 128;
                    if (gt >= 2) {
                        wait(BAR(sm->do_empty[s]), ph ^ 1, 1);
                        wait(BAR(sm->q_empty[s]), ph ^ 1, 2);
                    }
                    if (bad) break;
                    if (lane == 0) {
                        mbar_arrive_expect_tx(qf, kTileBytes / kBwdGatherWarps);
                        if (!proxy) {
                            mbar_arrive_expect_tx(df, kTileBytes / kBwdGatherWarps);
                        } else if (g == 0) {
                            mbar_arrive_expect_tx(df, kTileBytes);
                            tma_load_tile(tile_do0 + s * kTileBytes, &tmap_kp, ud.j * kBlock, ud.p / P.pg, ud.b, df);
                        } else {
                            mbar_arrive(df);
                        }
                    }
                    __syncwarp();
                    int r[4];
                    if (!q_lane) {
                        if (!proxy) {
                            const int64_t base = do_base + static_cast<int64_t>(hh) * P.do_row_h;
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                r[i] = qr[i] >= 0 ? static_cast<int>(base + qr[i] * P.do_row_s) : P.do_rows_total;
                            tma_gather4(tile_do0 + s * kTileBytes + off, &tmap_do, panel * 64, r[0], r[1], r[2], r[3], df);
                        }
                    } else if (proxy) {
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            r[i] = qr[i] >= 0 ? static_cast<int>(qp_base + qr[i] * P.qp_row_s) : P.qp_rows_total;
                        tma_gather4(tile_q0 + s * kTileBytes + off, &tmap_qp, panel * 64, r[0], r[1], r[2], r[3], qf);
                    } else {
                        const int64_t base = q_base + static_cast<int64_t>(hh) * P.q_row_h;
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            r[i] = qr[i] >= 0 ? static_cast<int>(base + qr[i] * P.q_row_s) : P.q_rows_total;
                        tma_gather4(tile_q0 + s * kTileBytes + off, &tmap_q, panel * 64, r[0], r[1], r[2], r[3], qf);
                    }
                }
            }
        }
    } else if (warp >= 8) {
        reg_dec<kBwdRegsOutput>();
        // =========================== output group ===========================
        const int otid = tid - 8 * 32;
        // Reads accumulator `acc` (lane = key row of the block) and adds it to the fp32 rows starting at `dst`.
        auto flush_rows = [&](uint32_t acc, float* dst) {
            float* drow = dst + static_cast<int64_t>(row) * kHeadDim;
#pragma unroll 1
            for (int c = 0; c < 128; c += 32) {
                uint32_t v[32];
                tmem_ld32(tmem_addr(acc, quarter, c), v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; i += 4)
                    red_add_v4(drow + c + i, __uint_as_float(v[i]), __uint_as_float(v[i + 1]), __uint_as_float(v[i + 2]),
                               __uint_as_float(v[i + 3]));
            }
        };
        BwdUnit ud;
        for (uint32_t draw = 0; next_unit(draw, ud, std::false_type{}); ++draw, ++nsub) {
            const int ntiles = (ud.chunk1 - ud.chunk0) * hpc;
            const int64_t slot_base = ud.e0 - edge_base;
            const int kph = ud.p / P.pg;
            int hh = 0, chunk = ud.chunk0;
            for (int t = 0; t < ntiles && !bad; ++t, ++gt) {
                const bool is_proxy = hh == P.mpp;
                const int nrows = min(kBlock, ud.n - chunk * kBlock);
                const int64_t slot0 = slot_base + static_cast<int64_t>(chunk) * kBlock;
                const bool full = nrows == kBlock;
                if (is_proxy) {
                    wait(BAR(sm->dkp_full), pt & 1, 1);
                    if (!bad) {
                        tc_fence_after_sync();
                        {
                            // dKp^T: lane = head-dimension index, column = key row: the 32 lanes of a warp add to 32
                            // consecutive floats of one row per instruction
                            float* kbase = P.dkp_acc + ((static_cast<int64_t>(ud.b) * P.Hpkv + kph) * P.S + ud.j * kBlock) * kHeadDim + row;
#pragma unroll 1
                            for (int c = 0; c < 128; c += 32) {
                                uint32_t v[32];
                                tmem_ld32(tmem_addr(r1, quarter, c), v);
                                tmem_ld_wait();
#pragma unroll
                                for (int i = 0; i < 32; ++i) atomicAdd(kbase + static_cast<int64_t>(c + i) * kHeadDim, __uint_as_float(v[i]));
                            }
                        }
                        tc_fence_before_sync();
                        warp_arrive(BAR(sm->r1_free));
                    }
                    ++pt;
                }
                wait(BAR(sm->dq_full), gt & 1, 2);
                bad = group_or(1, bad);
                if (bad) break;
                tc_fence_after_sync();
                // With `split` the row leaves twice: rounded to bf16, and the remainder of that rounding (a second plane of
                // the partial buffers, `part_slots` slots further on), so that the sum over many edges keeps fp32-like accuracy.
                const int nparts = P.split ? 2 : 1;
                for (int part = 0; part < nparts; ++part) {
                    if (part > 0 && full) named_barrier_sync(1, 128);   // the staging tile's first store has read it
                    const int64_t pslot0 = slot0 + part * P.part_slots;
                    __nv_bfloat16* grow = is_proxy ? P.dqp_part + (pslot0 + row) * kHeadDim
                                                   : P.dq_part + ((pslot0 + row) * P.mpp + hh) * kHeadDim;
#pragma unroll 1
                    for (int c = 0; c < 128; c += 32) {
                        uint32_t v[32];
                        tmem_ld32(tmem_addr(r0, quarter, c), v);
                        tmem_ld_wait();
                        uint32_t pk[16];
                        if (part == 0) {
#pragma unroll
                            for (int i = 0; i < 16; ++i) pk[i] = pack_act<FP16>(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
                        } else {
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                const float x0 = __uint_as_float(v[2 * i]), x1 = __uint_as_float(v[2 * i + 1]);
                                pk[i] = pack_act<FP16>(x0 - act_round<FP16>(x0), x1 - act_round<FP16>(x1));
                            }
                        }
                        if (full) {
                            // the dS^T tile is free (dQ has been computed): it stages the rows for one TMA tile store
#pragma unroll
                            for (int k8 = 0; k8 < 4; ++k8)
                                st_shared_v4(tile_ds + swz_offset(row, (c >> 3) + k8), pk[4 * k8], pk[4 * k8 + 1], pk[4 * k8 + 2],
                                             pk[4 * k8 + 3]);
                        } else if (row < nrows) {
#pragma unroll
                            for (int k8 = 0; k8 < 4; ++k8)
                                *reinterpret_cast<uint4*>(grow + c + 8 * k8) =
                                    make_uint4(pk[4 * k8], pk[4 * k8 + 1], pk[4 * k8 + 2], pk[4 * k8 + 3]);
                        }
                    }
                    if (part == nparts - 1) {
                        tc_fence_before_sync();
                        warp_arrive(BAR(sm->r0_free));
                    }
                    if (full) {
                        fence_async_smem();
                        named_barrier_sync(1, 128);
                        if (otid == 0) {
                            const void* tm = is_proxy ? static_cast<const void*>(&tmap_dqp) : static_cast<const void*>(&tmap_dq);
                            tma_store_3d(tm, tile_ds, 0, is_proxy ? 0 : hh, static_cast<int>(pslot0));
                            tma_store_3d(tm, tile_ds + kPanelBytes, 64, is_proxy ? 0 : hh, static_cast<int>(pslot0));
                            tma_store_commit();
                            tma_store_wait_read();
                        }
                    }
                }
                if (otid == 0) mbar_arrive(BAR(sm->ds_free));
                if (++hh == hpc) {
                    hh = 0;
                    ++chunk;
                }
            }
            if (!bad) {
                // sub-unit epilogue: add this sub-unit's share of dV_j and dK_j
                wait(BAR(sm->acc_full), nsub & 1, 3);
                if (!bad) {
                    tc_fence_after_sync();
                    const int64_t at = ((static_cast<int64_t>(ud.b) * P.Hkv + ud.kvh) * P.S + ud.j * kBlock) * kHeadDim;
                    flush_rows(r2, P.dv_acc + at);
                    flush_rows(r3, P.dk_acc + at);
                    tc_fence_before_sync();
                    warp_arrive(BAR(sm->acc_free));
                }
            }
        }
        if (otid == 0) tma_store_wait_all();
    } else {
        reg_inc<kBwdRegsCompute>();
        // =========================== compute groups ===========================
        // Thread = (key `row`, the 64 queries of its group).  Reads S^T and dP^T, writes P^T and dS^T back into
        // TMEM over them (bf16) and dS^T into the shared tile that feeds dQ = dS K.
        const int hf = warp >> 2;          // which half of the queries
        const int cbase = hf * 64;
        const float2 sc2 = make_float2(P.scale_log2e, P.scale_log2e);
        const float inv_mpp = 1.f / static_cast<float>(P.mpp);
        const bool with_kl = P.with_kl != 0;
        // sum over the main heads of P for this thread's 64 queries: the KL teacher, as packed fp16 pairs
        // (values in [0,1], at most Hq/Hp addends; the result is rounded to bf16 anyway)
        __half2 teacher[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) teacher[i] = __floats2half2_rn(0.f, 0.f);
        BwdUnit ud;
        for (uint32_t draw = 0; next_unit(draw, ud, std::false_type{}); ++draw, ++nsub) {
            const int ntiles = (ud.chunk1 - ud.chunk0) * hpc;
            int hh = 0, chunk = ud.chunk0;
            for (int t = 0; t < ntiles && !bad; ++t, ++gt) {
                const bool is_proxy = hh == P.mpp;
                const uint32_t s = gt & 1;
                wait(BAR(sm->st_full[s]), (gt >> 1) & 1, 1);
                wait(BAR(sm->sdp_full), gt & 1, 3);
                if (bad) break;
                tc_fence_after_sync();
                const BwdRowStats* st = &sm->stats[s];
                // only the first chunk of a reverse-index row can hold rows of the key block itself
                const bool own = (chunk == 0);
                const bool masked = own || (VARLEN && st->any_low != 0);
                // The body is instantiated per (masked, proxy) combination: the common tile (neither) must not pay for
                // predicated-off mask arithmetic or per-element branches in its inner loop, which is bound by instruction issue.
                auto compute_tile = [&](auto masked_c, auto proxy_c) __attribute__((always_inline)) {
                    constexpr bool kMasked = decltype(masked_c)::value;
                    constexpr bool kProxy = decltype(proxy_c)::value;
                    // Software pipeline over four 16-column pieces: the TMEM loads of piece c+1 are in flight while piece c
                    // is worked on (tcgen05.wait::ld waits for every load issued so far, hence the order wait, issue, compute).
                    uint32_t sv[2][16], dv[2][16];
                    tmem_ld16(tmem_addr(r0, quarter, cbase), sv[0]);
                    if (!kProxy) tmem_ld16(tmem_addr(r1, quarter, cbase), dv[0]);
#pragma unroll
                    for (int c = 0; c < 64; c += 16) {
                        const int cur = (c >> 4) & 1;
                        tmem_ld_wait();
                        if (c + 16 < 64) {
                            tmem_ld16(tmem_addr(r0, quarter, cbase + c + 16), sv[cur ^ 1]);
                            if (!kProxy) tmem_ld16(tmem_addr(r1, quarter, cbase + c + 16), dv[cur ^ 1]);
                        }
                        uint32_t lim[4] = {0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu};
                        uint32_t lw[4] = {0u, 0u, 0u, 0u};
                        if (kMasked) {
                            if (own) {
                                const uint4 l4 = *reinterpret_cast<const uint4*>(&st->limit[cbase + c]);
                                lim[0] = l4.x; lim[1] = l4.y; lim[2] = l4.z; lim[3] = l4.w;
                            }
                            if (VARLEN) {
                                const uint4 w4 = *reinterpret_cast<const uint4*>(&st->low[cbase + c]);
                                lw[0] = w4.x; lw[1] = w4.y; lw[2] = w4.z; lw[3] = w4.w;
                            }
                        }
                        uint32_t pk[8], dk[8];
#pragma unroll
                        for (int i = 0; i < 16; i += 2) {
                            const float2 nl2 = *reinterpret_cast<const float2*>(&st->neg_lse[cbase + c + i]);
                            const float2 a = f2_fma(f2_from_bits(sv[cur][i], sv[cur][i + 1]), sc2, nl2);   // log2 of the probability
                            float p0 = fast_exp2(a.x);
                            float p1 = fast_exp2(a.y);
                            if (kMasked) {
                                const int l0 = static_cast<int>((lim[i >> 2] >> (8 * (i & 3))) & 0xffu);
                                const int l1 = static_cast<int>((lim[i >> 2] >> (8 * ((i + 1) & 3))) & 0xffu);
                                if (VARLEN) {
                                    const int w0 = static_cast<int>((lw[i >> 2] >> (8 * (i & 3))) & 0xffu);
                                    const int w1 = static_cast<int>((lw[i >> 2] >> (8 * ((i + 1) & 3))) & 0xffu);
                                    p0 = (row <= l0 && row >= w0) ? p0 : 0.f;
                                    p1 = (row <= l1 && row >= w1) ? p1 : 0.f;
                                } else {
                                    p0 = (row <= l0) ? p0 : 0.f;
                                    p1 = (row <= l1) ? p1 : 0.f;
                                }
                            }
                            const int ti = (c + i) >> 1;
                            if (!kProxy) {
                                // dS = P o (dP - delta)
                                const float2 nd2 = *reinterpret_cast<const float2*>(&st->neg_delta[cbase + c + i]);
                                const float2 d = f2_mul(make_float2(p0, p1), f2_add(f2_from_bits(dv[cur][i], dv[cur][i + 1]), nd2));
                                pk[i >> 1] = pack_act<FP16>(p0, p1);
                                dk[i >> 1] = pack_act<FP16>(d.x, d.y);
                                if (with_kl) teacher[ti] = __hadd2(teacher[ti], __floats2half2_rn(p0, p1));
                            } else {
                                const float2 tt = __half22float2(teacher[ti]);
                                const float t0 = tt.x * inv_mpp, t1 = tt.y * inv_mpp;
                                dk[i >> 1] = pack_act<FP16>(p0 - t0, p1 - t1);
                                if (P.kl_value) {   // KL(teacher || proxy) = sum t (ln t - ln p); t = 0 contributes nothing
                                    kl_acc += (t0 > 0.f) ? t0 * (fast_log2(t0) - a.x) : 0.f;
                                    kl_acc += (t1 > 0.f) ? t1 * (fast_log2(t1) - a.y) : 0.f;
                                }
                                teacher[ti] = __floats2half2_rn(0.f, 0.f);
                            }
                        }
                        // bf16 operands back into TMEM over the columns this thread has consumed: two queries per column.
                        // (In a proxy tile dSp^T is only parked in R0 until it can go to shared memory, see below.)
                        if (!kProxy) {
                            tmem_st8(tmem_addr(r0, quarter, cbase + (c >> 1)), pk);
                            tmem_st8(tmem_addr(r1, quarter, cbase + (c >> 1)), dk);
                        } else {
                            tmem_st8(tmem_addr(r0, quarter, cbase + (c >> 1)), dk);
                        }
                    }
                };
                if (masked) {
                    if (is_proxy) compute_tile(std::true_type{}, std::true_type{});
                    else compute_tile(std::true_type{}, std::false_type{});
                } else {
                    if (is_proxy) compute_tile(std::false_type{}, std::true_type{});
                    else compute_tile(std::false_type{}, std::false_type{});
                }
                tmem_st_wait();
                // dS^T also goes to the shared tile that feeds dQ = dS K (row = key, columns = queries).  That tile doubles
                // as the staging buffer of the previous tile's dQ store, so it is the last thing this tile touches: the
                // arithmetic above overlaps the previous tile's read-out.
                if (gt >= 1) wait(BAR(sm->ds_free), (gt - 1) & 1, 2);
                if (bad) break;
                {
                    uint32_t ds[32];
                    tmem_ld32(tmem_addr(is_proxy ? r0 : r1, quarter, cbase), ds);
                    tmem_ld_wait();
#pragma unroll
                    for (int k8 = 0; k8 < 8; ++k8)
                        st_shared_v4(tile_ds + swz_offset(row, (cbase >> 3) + k8), ds[4 * k8], ds[4 * k8 + 1], ds[4 * k8 + 2],
                                     ds[4 * k8 + 3]);
                }
                fence_async_smem();
                tc_fence_before_sync();
                warp_arrive(BAR(sm->pds_full));
                warp_arrive(BAR(sm->st_empty[s]));
                if (++hh == hpc) {
                    hh = 0;
                    ++chunk;
                }
            }
        }
    }
#ifdef FMSA_TRACE
    if (blockIdx.x == 0 && lane == 0) {
        trace_acc[0] = static_cast<unsigned long long>(clock64() - trace_t0);
        for (int i = 0; i < 8; ++i) g_bwd_trace[warp][i] = trace_acc[i];
    }
#endif
    if (P.kl_value && warp < 8) {
        for (int o = 16; o > 0; o >>= 1) kl_acc += __shfl_xor_sync(0xffffffffu, kl_acc, o);
        if (lane == 0) atomicAdd(P.kl_value, kl_acc * P.kl_value_scale);
    }
    if (bad) {
        atomicMax(P.status, kStatusWaitTimeout);
        // Give loads and products that are still in flight time to finish before shared memory and TMEM are released.
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000) __nanosleep(1000);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 512);
}

// -------------------------------------------------------------------------------------------
// dq[b,h,q,:] = sum over the row's edges of dq_part;  dq_proxy likewise, times the upstream
// gradient of kl_loss (a device scalar).  One warp per (batch*proxy head, query row).
// -------------------------------------------------------------------------------------------
struct BwdCombineParams {
    const __nv_bfloat16* dq_part;
    const __nv_bfloat16* dqp_part;
    const int32_t* edge_pos;   // sparse: [B*Hp, S, Kb]
    const int32_t* row_ptr;
    __nv_bfloat16* dq;         // (B,Hq,S,128) view: element strides below
    __nv_bfloat16* dqp;        // (B,Hp,S,128) view or null
    int32_t dq_sb, dq_sh, dq_ss, dqp_sb, dqp_sh, dqp_ss;   // element strides of the two views (each below 2^31)
    const float* grad_kl;      // device scalar or null (= 1)
    float scale, kl_out_scale; // factors the backward kernel left out of its partial rows
    int S, NB, Hq, Hp, mpp, ppk, Kb;
    int g_begin, G, dense;
    int split;              // the partial buffers hold a second plane (rounding remainders) part_slots slots further on
    int64_t part_slots;
};

template <bool FP16>
__global__ void __launch_bounds__(256) bwd_combine_kernel(const BwdCombineParams P) {
    const int lane = threadIdx.x & 31;
    const int64_t w = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    const int64_t bp0 = static_cast<int64_t>(P.g_begin) * P.ppk;
    if (w >= static_cast<int64_t>(P.G) * P.ppk * P.S) return;
    const int64_t bp = bp0 + w / P.S;
    const int q = static_cast<int>(w % P.S);
    const int b = static_cast<int>(bp / P.Hp), p = static_cast<int>(bp % P.Hp);
    const int64_t edge_base = P.dense ? dense_edge_base(bp0, P.S, P.NB) : static_cast<int64_t>(P.row_ptr[bp0 * P.NB]);
    const int nslots = P.dense ? (q >> 7) + 1 : P.Kb;
    const int32_t* erow = P.dense ? nullptr : P.edge_pos + (bp * P.S + q) * P.Kb;
    auto slot_of = [&](int s) -> int64_t {
        if (s >= nslots) return -1;
        if (P.dense) return dense_edge_base(bp, P.S, P.NB) + dense_row_offset(s, P.S) + (q - s * kBlock) - edge_base;
        const int e = erow[s];
        return e < 0 ? -1 : static_cast<int64_t>(e) - edge_base;
    };
    const float gk = ((P.dqp && P.grad_kl) ? *P.grad_kl : 1.f) * P.kl_out_scale;
    const int nheads = P.mpp + (P.dqp ? 1 : 0);
    for (int hh = 0; hh < nheads; ++hh) {
        const bool proxy = hh == P.mpp;
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
        for (int s0 = 0; s0 < nslots; s0 += 32) {
            const int64_t sl = slot_of(s0 + lane);
            const int cnt = min(32, nslots - s0);
#pragma unroll 4
            for (int i = 0; i < cnt; ++i) {
                const int64_t si = __shfl_sync(0xffffffffu, sl, i);
                if (si < 0) continue;
                for (int part = 0; part <= P.split; ++part) {
                    const int64_t sp = si + part * P.part_slots;
                    const __nv_bfloat16* src = proxy ? P.dqp_part + sp * kHeadDim : P.dq_part + (sp * P.mpp + hh) * kHeadDim;
                    const uint2 raw = *reinterpret_cast<const uint2*>(src + lane * 4);
                    const uint32_t lo = raw.x;
                    const uint32_t hi = raw.y;
                    a0 += act_lo<FP16>(lo);
                    a1 += act_hi<FP16>(lo);
                    a2 += act_lo<FP16>(hi);
                    a3 += act_hi<FP16>(hi);
                }
            }
        }
        uint2 o;
        if (proxy) {
            o.x = pack_act<FP16>(a0 * gk, a1 * gk);
            o.y = pack_act<FP16>(a2 * gk, a3 * gk);
            *reinterpret_cast<uint2*>(P.dqp + (static_cast<int64_t>(b) * P.dqp_sb + static_cast<int64_t>(p) * P.dqp_sh + static_cast<int64_t>(q) * P.dqp_ss) + lane * 4) = o;
        } else {
            o.x = pack_act<FP16>(a0 * P.scale, a1 * P.scale);
            o.y = pack_act<FP16>(a2 * P.scale, a3 * P.scale);
            *reinterpret_cast<uint2*>(P.dq + (static_cast<int64_t>(b) * P.dq_sb + static_cast<int64_t>(p * P.mpp + hh) * P.dq_sh + static_cast<int64_t>(q) * P.dq_ss) + lane * 4) = o;
        }
    }
}

// Wide variant for Hq/Hp <= 8: one sweep over the contiguous mpp*256-byte record of each edge.
template <int KITER, bool SPLIT, bool FP16>   // Hq/Hp <= 2*KITER: few accumulators, high occupancy (latency bound)
__global__ void __launch_bounds__(256, (KITER <= 2) ? 4 : 2) bwd_combine_wide_kernel(const BwdCombineParams P) {
    const int lane = threadIdx.x & 31;
    const int64_t w = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    const int64_t bp0 = static_cast<int64_t>(P.g_begin) * P.ppk;
    if (w >= static_cast<int64_t>(P.G) * P.ppk * P.S) return;
    const int64_t bp = bp0 + w / P.S;
    const int q = static_cast<int>(w % P.S);
    const int b = static_cast<int>(bp / P.Hp), p = static_cast<int>(bp % P.Hp);
    const int64_t edge_base = P.dense ? dense_edge_base(bp0, P.S, P.NB) : static_cast<int64_t>(P.row_ptr[bp0 * P.NB]);
    const int nslots = P.dense ? (q >> 7) + 1 : P.Kb;
    const int32_t* erow = P.dense ? nullptr : P.edge_pos + (bp * P.S + q) * P.Kb;
    auto slot_of = [&](int s) -> int64_t {
        if (s >= nslots) return -1;
        if (P.dense) return dense_edge_base(bp, P.S, P.NB) + dense_row_offset(s, P.S) + (q - s * kBlock) - edge_base;
        const int e = erow[s];
        return e < 0 ? -1 : static_cast<int64_t>(e) - edge_base;
    };
    const int nchunk = P.mpp * 16;
    float acc[KITER][8];
#pragma unroll
    for (int k = 0; k < KITER; ++k)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[k][e] = 0.f;
    float pa0 = 0.f, pa1 = 0.f, pa2 = 0.f, pa3 = 0.f;   // proxy row: lane owns columns 4*lane..+3
    // Four edges at a time: every load of the group is issued before the first sum (the kernel is bound by memory
    // latency; left to itself the compiler batches the loads only when the register budget happens to allow it).
    const bool has_proxy = P.dqp != nullptr;
    for (int s0 = 0; s0 < nslots; s0 += 32) {
        const int sl = static_cast<int>(slot_of(s0 + lane));   // slot numbers of a pass fit 31 bits
        const int cnt = min(32, nslots - s0);
        for (int i = 0; i < cnt; i += 4) {
            int si[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int v = __shfl_sync(0xffffffffu, sl, (i + u) & 31);
                si[u] = (i + u < cnt) ? v : -1;
            }
#pragma unroll
            for (int part = 0; part < (SPLIT ? 2 : 1); ++part) {
                uint4 raw[4][KITER];
                uint2 praw[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int64_t sp = static_cast<int64_t>(si[u]) + part * P.part_slots;
                    const __nv_bfloat16* rec = P.dq_part + sp * P.mpp * kHeadDim;
#pragma unroll
                    for (int k = 0; k < KITER; ++k) {
                        const int ck = k * 32 + lane;
                        raw[u][k] = (si[u] >= 0 && ck < nchunk) ? *reinterpret_cast<const uint4*>(rec + ck * 8) : make_uint4(0, 0, 0, 0);
                    }
                    praw[u] = (si[u] >= 0 && has_proxy) ? *reinterpret_cast<const uint2*>(P.dqp_part + sp * kHeadDim + lane * 4)
                                                        : make_uint2(0, 0);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
#pragma unroll
                    for (int k = 0; k < KITER; ++k) {
                        const uint32_t w4[4] = {raw[u][k].x, raw[u][k].y, raw[u][k].z, raw[u][k].w};
                        if constexpr (KITER >= 3) {   // packed adds pay at 120-128 registers and two CTAs per SM, not at 64
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float2 a = f2_add(make_float2(acc[k][2 * e], acc[k][2 * e + 1]),
                                                        make_float2(act_lo<FP16>(w4[e]), act_hi<FP16>(w4[e])));
                                acc[k][2 * e] = a.x;
                                acc[k][2 * e + 1] = a.y;
                            }
                        } else {
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                acc[k][2 * e] += act_lo<FP16>(w4[e]);
                                acc[k][2 * e + 1] += act_hi<FP16>(w4[e]);
                            }
                        }
                    }
                    pa0 += act_lo<FP16>(praw[u].x);
                    pa1 += act_hi<FP16>(praw[u].x);
                    pa2 += act_lo<FP16>(praw[u].y);
                    pa3 += act_hi<FP16>(praw[u].y);
                }
            }
        }
    }
#pragma unroll
    for (int k = 0; k < KITER; ++k) {
        const int ck = k * 32 + lane;
        if (ck < nchunk) {
            const int hh = ck >> 4, col = (ck & 15) * 8;
            uint4 o;
            o.x = pack_act<FP16>(acc[k][0] * P.scale, acc[k][1] * P.scale);
            o.y = pack_act<FP16>(acc[k][2] * P.scale, acc[k][3] * P.scale);
            o.z = pack_act<FP16>(acc[k][4] * P.scale, acc[k][5] * P.scale);
            o.w = pack_act<FP16>(acc[k][6] * P.scale, acc[k][7] * P.scale);
            *reinterpret_cast<uint4*>(P.dq + (static_cast<int64_t>(b) * P.dq_sb + static_cast<int64_t>(p * P.mpp + hh) * P.dq_sh + static_cast<int64_t>(q) * P.dq_ss) + col) = o;
        }
    }
    if (P.dqp) {
        const float gk = (P.grad_kl ? *P.grad_kl : 1.f) * P.kl_out_scale;
        uint2 o;
        o.x = pack_act<FP16>(pa0 * gk, pa1 * gk);
        o.y = pack_act<FP16>(pa2 * gk, pa3 * gk);
        *reinterpret_cast<uint2*>(P.dqp + (static_cast<int64_t>(b) * P.dqp_sb + static_cast<int64_t>(p) * P.dqp_sh + static_cast<int64_t>(q) * P.dqp_ss) + lane * 4) = o;
    }
}

// -------------------------------------------------------------------------------------------
// delta[b,h,q] = sum_d out[b,q,h,d] * dout[b,q,h,d]   (flash_msa/flash_msa.py:99)
// -------------------------------------------------------------------------------------------
// One CTA per (batch, 32 consecutive query positions): half-warp g takes positions 2g and 2g+1 and walks the heads,
// each lane reading 16 bytes of the `out` row and of the `dout` row (a half-warp covers one 256-byte row per load, four
// rows in flight); the sums meet in shared memory so that delta leaves in 128-byte runs along the sequence.
template <bool FP16>
__global__ void __launch_bounds__(256) delta_kernel(const __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ dout,
                                                    int64_t do_sb, int64_t do_ss, int64_t do_sh, float* __restrict__ delta,
                                                    int B, int S, int Hq) {
    extern __shared__ float sdelta[];   // [Hq][32]
    const int lane = threadIdx.x & 31, l16 = lane & 15;
    const int g = threadIdx.x >> 4;   // half-warp 0..15
    const int qblocks = S >> 5;
    const int b = blockIdx.x / qblocks, q0 = (blockIdx.x % qblocks) << 5;
    auto dot8 = [](const uint4& a, const uint4& d) {
        return act_lo<FP16>(a.x) * act_lo<FP16>(d.x) + act_hi<FP16>(a.x) * act_hi<FP16>(d.x) + act_lo<FP16>(a.y) * act_lo<FP16>(d.y) +
               act_hi<FP16>(a.y) * act_hi<FP16>(d.y) + act_lo<FP16>(a.z) * act_lo<FP16>(d.z) + act_hi<FP16>(a.z) * act_hi<FP16>(d.z) +
               act_lo<FP16>(a.w) * act_lo<FP16>(d.w) + act_hi<FP16>(a.w) * act_hi<FP16>(d.w);
    };
#pragma unroll
    for (int qq = 0; qq < 2; ++qq) {
        const int ql = 2 * g + qq, q = q0 + ql;
        const __nv_bfloat16* orow = out + (static_cast<int64_t>(b) * S + q) * Hq * kHeadDim + l16 * 8;
        const __nv_bfloat16* drow = dout + b * do_sb + q * do_ss + l16 * 8;
        int h = 0;
        for (; h + 4 <= Hq; h += 4) {
            uint4 a[4], d[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                a[i] = *reinterpret_cast<const uint4*>(orow + static_cast<int64_t>(h + i) * kHeadDim);
                d[i] = *reinterpret_cast<const uint4*>(drow + (h + i) * do_sh);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float sum = dot8(a[i], d[i]);
#pragma unroll
                for (int off = 8; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
                if (l16 == 0) sdelta[(h + i) * 32 + ql] = sum;
            }
        }
        for (; h < Hq; ++h) {
            const uint4 a = *reinterpret_cast<const uint4*>(orow + static_cast<int64_t>(h) * kHeadDim);
            const uint4 d = *reinterpret_cast<const uint4*>(drow + h * do_sh);
            float sum = dot8(a, d);
#pragma unroll
            for (int off = 8; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
            if (l16 == 0) sdelta[h * 32 + ql] = sum;
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < Hq * 32; i += 256)
        delta[(static_cast<int64_t>(b) * Hq + (i >> 5)) * S + q0 + (i & 31)] = sdelta[i];
}

// dst = bf16(src * const_scale * factor), factor = *scale_ptr when given (the upstream kl gradient lives on the
// device: flash_msa/flash_msa.py:122-125) else 1.
template <bool FP16>
__global__ void __launch_bounds__(256) cast_scaled_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int64_t n4,
                                                          const float* __restrict__ scale_ptr, float const_scale) {
    const float f = (scale_ptr ? *scale_ptr : 1.f) * const_scale;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const float4 v = reinterpret_cast<const float4*>(src)[i];
        uint2 o;
        o.x = pack_act<FP16>(v.x * f, v.y * f);
        o.y = pack_act<FP16>(v.z * f, v.w * f);
        reinterpret_cast<uint2*>(dst)[i] = o;
    }
}

// The same cast with a strided destination: src is contiguous fp32 [B,H,S,128], dst a (B,H,S,128) view given by
// element strides (a gradient written straight into (B,S,H,128) storage).  One thread per four elements.
template <bool FP16>
__global__ void __launch_bounds__(256) cast_scaled_rows_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                                               int64_t sb, int64_t sh, int64_t ss, int H, int S, int64_t n4,
                                                               const float* __restrict__ scale_ptr, float const_scale) {
    const float f = (scale_ptr ? *scale_ptr : 1.f) * const_scale;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const int64_t rowi = i >> 5;                // 32 float4 per row of 128
        const int c4 = static_cast<int>(i & 31);
        const int sq = static_cast<int>(rowi % S);
        const int64_t bh = rowi / S;
        const int h = static_cast<int>(bh % H);
        const int64_t b = bh / H;
        const float4 v = reinterpret_cast<const float4*>(src)[i];
        uint2 o;
        o.x = pack_act<FP16>(v.x * f, v.y * f);
        o.y = pack_act<FP16>(v.z * f, v.w * f);
        *reinterpret_cast<uint2*>(dst + b * sb + h * sh + sq * ss + c4 * 4) = o;
    }
}

}  // namespace
}  // namespace fmsa

extern "C" int fmsa_cast_scaled_rows(const float* src, const fmsa_tensor* dst, int32_t B, int32_t H, int32_t S,
                                     const float* scale_ptr, float const_scale, int32_t dtype, void* stream) {
    using namespace fmsa;
    FMSA_REQUIRE(src && dst && dst->ptr && B > 0 && H > 0 && S > 0);
    FMSA_REQUIRE(dtype == FMSA_DTYPE_BF16 || dtype == FMSA_DTYPE_FP16);
    FMSA_REQUIRE(aligned16(src) && (reinterpret_cast<uintptr_t>(dst->ptr) & 7u) == 0);
    FMSA_REQUIRE(dst->stride_b % 4 == 0 && dst->stride_h % 4 == 0 && dst->stride_s % 4 == 0);
    const int64_t n4 = static_cast<int64_t>(B) * H * S * (kHeadDim / 4);
    int64_t grid = (n4 + 255) / 256;
    if (grid > 148 * 16) grid = 148 * 16;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == FMSA_DTYPE_FP16)
        cast_scaled_rows_kernel<true><<<static_cast<unsigned>(grid), 256, 0, st>>>(
            src, static_cast<__nv_bfloat16*>(const_cast<void*>(dst->ptr)), dst->stride_b, dst->stride_h, dst->stride_s, H, S, n4, scale_ptr, const_scale);
    else
        cast_scaled_rows_kernel<false><<<static_cast<unsigned>(grid), 256, 0, st>>>(
            src, static_cast<__nv_bfloat16*>(const_cast<void*>(dst->ptr)), dst->stride_b, dst->stride_h, dst->stride_s, H, S, n4, scale_ptr, const_scale);
    return check_launch();
}

extern "C" int fmsa_bwd_delta(const void* out, const fmsa_tensor* d_out, float* delta, int32_t B, int32_t S, int32_t Hq,
                              int32_t dtype, void* stream) {
    using namespace fmsa;
    FMSA_REQUIRE(out && d_out && d_out->ptr && delta && B > 0 && S > 0 && Hq > 0);
    FMSA_REQUIRE(dtype == FMSA_DTYPE_BF16 || dtype == FMSA_DTYPE_FP16);
    FMSA_REQUIRE(aligned16(out) && aligned16(d_out->ptr));
    FMSA_REQUIRE(d_out->stride_b % 8 == 0 && d_out->stride_h % 8 == 0 && d_out->stride_s % 8 == 0);
    const int64_t grid = static_cast<int64_t>(B) * (S / 32);
    FMSA_REQUIRE(S % 32 == 0 && grid <= 0x7fffffffLL && Hq * 32 * sizeof(float) <= 48 * 1024);
    const size_t smem = static_cast<size_t>(Hq) * 32 * sizeof(float);
    if (dtype == FMSA_DTYPE_FP16)
        delta_kernel<true><<<static_cast<unsigned>(grid), 256, smem, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(d_out->ptr), d_out->stride_b, d_out->stride_s,
        d_out->stride_h, delta, B, S, Hq);
    else
        delta_kernel<false><<<static_cast<unsigned>(grid), 256, smem, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(d_out->ptr), d_out->stride_b, d_out->stride_s,
        d_out->stride_h, delta, B, S, Hq);
    return check_launch();
}

extern "C" int fmsa_cast_scaled(const float* src, void* dst, int64_t n, const float* scale_ptr, float const_scale,
                                int32_t dtype, void* stream) {
    using namespace fmsa;
    FMSA_REQUIRE(src && dst && n >= 0 && n % 4 == 0);
    FMSA_REQUIRE(dtype == FMSA_DTYPE_BF16 || dtype == FMSA_DTYPE_FP16);
    FMSA_REQUIRE(aligned16(src) && (reinterpret_cast<uintptr_t>(dst) & 7u) == 0);
    if (n == 0) return FMSA_OK;
    const int64_t n4 = n / 4;
    int64_t grid = (n4 + 255) / 256;
    if (grid > 148 * 16) grid = 148 * 16;
    if (dtype == FMSA_DTYPE_FP16)
        cast_scaled_kernel<true><<<static_cast<unsigned>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(
            src, static_cast<__nv_bfloat16*>(dst), n4, scale_ptr, const_scale);
    else
        cast_scaled_kernel<false><<<static_cast<unsigned>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(
            src, static_cast<__nv_bfloat16*>(dst), n4, scale_ptr, const_scale);
    return check_launch();
}

extern "C" int fmsa_sparse_bwd(const fmsa_problem* pb, const fmsa_tensor* q, const fmsa_tensor* k, const fmsa_tensor* v,
                               const fmsa_tensor* q_proxy, const fmsa_tensor* k_proxy, const fmsa_tensor* d_out,
                               const float* lse, const float* lse_proxy, const float* delta, const int32_t* row_ptr,
                               const int32_t* col_q, void* dq_part, void* dqp_part, int64_t part_slots, int32_t split,
                               float* dkp_acc, float* dk_acc, float* dv_acc, int32_t g_begin, int32_t g_count, int32_t with_kl,
                               int32_t dense, float* kl_value, int32_t* counter, int32_t* status, void* stream) {
    using namespace fmsa;
    FMSA_REQUIRE(problem_ok(pb));
    FMSA_REQUIRE(q && k && v && d_out && q->ptr && k->ptr && v->ptr && d_out->ptr);
    FMSA_REQUIRE(lse && delta && dq_part && dk_acc && dv_acc && counter && status);
    FMSA_REQUIRE(dense || (row_ptr && col_q));
    FMSA_REQUIRE(!with_kl || (q_proxy && k_proxy && q_proxy->ptr && k_proxy->ptr && lse_proxy && dqp_part && dkp_acc));
    FMSA_REQUIRE(g_begin >= 0 && g_count > 0 && g_begin + g_count <= pb->B * pb->Hkv);
    FMSA_REQUIRE(dense || (pb->top_k_blocks >= 1 && pb->top_k_blocks <= pb->S / kBlock));
    FMSA_REQUIRE(pb->scale > 0.f);
    FMSA_REQUIRE(static_cast<int64_t>(pb->B) * pb->Hp <= 65535 && pb->S / kBlock <= 32767);   // 16-bit fields of the sub-unit record
    if (part_slots < fmsa_fwd_partial_slots(pb, g_count, dense)) return FMSA_ERR_WORKSPACE;
    FMSA_REQUIRE(tma_compatible(k->ptr, k->stride_b, k->stride_h, k->stride_s));
    FMSA_REQUIRE(tma_compatible(v->ptr, v->stride_b, v->stride_h, v->stride_s));
    FMSA_REQUIRE(tma_compatible(q->ptr, q->stride_b, q->stride_h, q->stride_s));
    FMSA_REQUIRE(tma_compatible(d_out->ptr, d_out->stride_b, d_out->stride_h, d_out->stride_s));
    if (with_kl) {
        FMSA_REQUIRE(tma_compatible(q_proxy->ptr, q_proxy->stride_b, q_proxy->stride_h, q_proxy->stride_s));
        FMSA_REQUIRE(tma_compatible(k_proxy->ptr, k_proxy->stride_b, k_proxy->stride_h, k_proxy->stride_s));
    }
    FMSA_REQUIRE(aligned16(dk_acc) && aligned16(dv_acc) && (!with_kl || aligned16(dkp_acc)));
    FMSA_REQUIRE(aligned16(dq_part) && (!with_kl || aligned16(dqp_part)));
    FMSA_REQUIRE(gather_compatible(q->ptr, q->stride_b, q->stride_h, q->stride_s));
    FMSA_REQUIRE(gather_compatible(d_out->ptr, d_out->stride_b, d_out->stride_h, d_out->stride_s));
    if (with_kl) FMSA_REQUIRE(gather_compatible(q_proxy->ptr, q_proxy->stride_b, q_proxy->stride_h, q_proxy->stride_s));
    FMSA_REQUIRE(part_slots > 0 && part_slots * (split ? 2 : 1) < 0x7fffffffLL);
    const fmsa_tensor* qpx = with_kl ? q_proxy : q;
    const fmsa_tensor* kpx = with_kl ? k_proxy : k;
    const int h_qpx = with_kl ? pb->Hp : pb->Hq, h_kpx = with_kl ? pb->Hpkv : pb->Hkv;
    const uint64_t q_rows = gather_rows(pb->B, pb->Hq, pb->S, q->stride_b, q->stride_h, q->stride_s);
    const uint64_t do_rows = gather_rows(pb->B, pb->Hq, pb->S, d_out->stride_b, d_out->stride_h, d_out->stride_s);
    const uint64_t qp_rows = gather_rows(pb->B, h_qpx, pb->S, qpx->stride_b, qpx->stride_h, qpx->stride_s);
    CUtensorMap tq, tdo, tqp, tk, tv, tkp, tdq, tdqp;
    if (!make_tmap_gather(&tq, q->ptr, q_rows) || !make_tmap_gather(&tdo, d_out->ptr, do_rows) ||
        !make_tmap_gather(&tqp, qpx->ptr, qp_rows) ||
        !make_tmap_bhsd(&tk, k->ptr, pb->B, pb->Hkv, pb->S, k->stride_b, k->stride_h, k->stride_s, 128) ||
        !make_tmap_bhsd(&tv, v->ptr, pb->B, pb->Hkv, pb->S, v->stride_b, v->stride_h, v->stride_s, 128) ||
        !make_tmap_bhsd(&tkp, kpx->ptr, pb->B, h_kpx, pb->S, kpx->stride_b, kpx->stride_h, kpx->stride_s, 128) ||
        !make_tmap_partials_swz(&tdq, dq_part, static_cast<uint64_t>(part_slots) * (split ? 2 : 1),
                                static_cast<uint64_t>(pb->Hq / pb->Hp)) ||
        !make_tmap_partials_swz(&tdqp, with_kl ? dqp_part : dq_part, static_cast<uint64_t>(part_slots) * (split ? 2 : 1), 1))
        return FMSA_ERR_CUDA;

    BwdParams P;
    P.q_row_b = q->stride_b / 128; P.q_row_h = q->stride_h / 128; P.q_row_s = q->stride_s / 128;
    P.do_row_b = d_out->stride_b / 128; P.do_row_h = d_out->stride_h / 128; P.do_row_s = d_out->stride_s / 128;
    P.qp_row_b = qpx->stride_b / 128; P.qp_row_h = qpx->stride_h / 128; P.qp_row_s = qpx->stride_s / 128;
    P.q_rows_total = static_cast<int32_t>(q_rows); P.do_rows_total = static_cast<int32_t>(do_rows);
    P.qp_rows_total = static_cast<int32_t>(qp_rows);
    P.lse = lse; P.lse_proxy = lse_proxy; P.delta = delta;
    P.row_ptr = row_ptr; P.col_q = col_q; P.doc_start = pb->doc_start;
    P.dq_part = static_cast<__nv_bfloat16*>(dq_part); P.dqp_part = static_cast<__nv_bfloat16*>(dqp_part);
    P.part_slots = part_slots; P.split = split ? 1 : 0;
    P.dkp_acc = dkp_acc; P.dk_acc = dk_acc; P.dv_acc = dv_acc;
    P.counter = counter; P.status = status;
    P.S = pb->S; P.NB = pb->S / kBlock; P.Hq = pb->Hq; P.Hkv = pb->Hkv; P.Hp = pb->Hp; P.Hpkv = pb->Hpkv;
    P.mpp = pb->Hq / pb->Hp; P.ppk = pb->Hp / pb->Hkv; P.pg = pb->Hp / pb->Hpkv;
    P.g_begin = g_begin; P.G = g_count;
    P.with_kl = with_kl ? 1 : 0; P.dense = dense ? 1 : 0;
    P.scale_log2e = pb->scale * kLog2e;
    P.kl_value = with_kl ? kl_value : nullptr;
    P.kl_value_scale = kLn2 / (static_cast<float>(pb->B) * pb->Hp * pb->S);

    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int sms = device_sm_count();
    const bool fp16 = pb->dtype == FMSA_DTYPE_FP16;
    const bool varlen = P.doc_start != nullptr;
    const void* kfn = fp16 ? (varlen ? reinterpret_cast<const void*>(sparse_bwd_kernel<true, true>) : reinterpret_cast<const void*>(sparse_bwd_kernel<true, false>))
                           : (varlen ? reinterpret_cast<const void*>(sparse_bwd_kernel<false, true>) : reinterpret_cast<const void*>(sparse_bwd_kernel<false, false>));
    if (sms <= 0 || !ensure_smem_attr(kfn, kBwdSmemBytes)) return FMSA_ERR_CUDA;
    if (cudaMemsetAsync(counter, 0, sizeof(int32_t), st) != cudaSuccess) return FMSA_ERR_CUDA;
    P.n_subunits = g_count * subunits_per_group(P.NB, P.ppk, kChunksPerSubUnit);
    FMSA_REQUIRE(P.n_subunits < 0x7fffffffLL);
    const int grid = static_cast<int>(P.n_subunits < sms ? P.n_subunits : sms);
    if (fp16 && varlen) sparse_bwd_kernel<true, true><<<grid, kBwdThreads, kBwdSmemBytes, st>>>(tq, tdo, tqp, tk, tv, tkp, tdq, tdqp, P);
    else if (fp16) sparse_bwd_kernel<true, false><<<grid, kBwdThreads, kBwdSmemBytes, st>>>(tq, tdo, tqp, tk, tv, tkp, tdq, tdqp, P);
    else if (varlen) sparse_bwd_kernel<false, true><<<grid, kBwdThreads, kBwdSmemBytes, st>>>(tq, tdo, tqp, tk, tv, tkp, tdq, tdqp, P);
    else sparse_bwd_kernel<false, false><<<grid, kBwdThreads, kBwdSmemBytes, st>>>(tq, tdo, tqp, tk, tv, tkp, tdq, tdqp, P);
    return check_launch();
}

extern "C" int fmsa_sparse_bwd_combine(const fmsa_problem* pb, const void* dq_part, const void* dqp_part,
                                       int64_t part_slots, int32_t split, const int32_t* edge_pos, const int32_t* row_ptr,
                                       const fmsa_tensor* dq, const fmsa_tensor* dq_proxy, const float* grad_kl,
                                       int32_t g_begin, int32_t g_count, int32_t dense, void* stream) {
    using namespace fmsa;
    FMSA_REQUIRE(problem_ok(pb));
    FMSA_REQUIRE(dq_part && dq && dq->ptr);
    FMSA_REQUIRE(dense || (edge_pos && row_ptr));
    FMSA_REQUIRE(!dq_proxy || (dq_proxy->ptr && dqp_part));
    FMSA_REQUIRE(aligned16(dq->ptr) && dq->stride_b % 8 == 0 && dq->stride_h % 8 == 0 && dq->stride_s % 8 == 0);
    FMSA_REQUIRE(!dq_proxy || (aligned16(dq_proxy->ptr) && dq_proxy->stride_b % 8 == 0 && dq_proxy->stride_h % 8 == 0 &&
                               dq_proxy->stride_s % 8 == 0));
    FMSA_REQUIRE(g_begin >= 0 && g_count > 0 && g_begin + g_count <= pb->B * pb->Hkv);
    FMSA_REQUIRE(!split || part_slots > 0);
    BwdCombineParams P;
    P.dq_part = static_cast<const __nv_bfloat16*>(dq_part); P.dqp_part = static_cast<const __nv_bfloat16*>(dqp_part);
    P.edge_pos = edge_pos; P.row_ptr = row_ptr;
    P.split = split ? 1 : 0; P.part_slots = part_slots;
    auto fits = [](int64_t x) { return x >= 0 && x < 0x7fffffffLL; };
    FMSA_REQUIRE(fits(dq->stride_b) && fits(dq->stride_h) && fits(dq->stride_s));
    FMSA_REQUIRE(!dq_proxy || (fits(dq_proxy->stride_b) && fits(dq_proxy->stride_h) && fits(dq_proxy->stride_s)));
    P.dq = static_cast<__nv_bfloat16*>(const_cast<void*>(dq->ptr));
    P.dq_sb = static_cast<int32_t>(dq->stride_b); P.dq_sh = static_cast<int32_t>(dq->stride_h); P.dq_ss = static_cast<int32_t>(dq->stride_s);
    P.dqp = dq_proxy ? static_cast<__nv_bfloat16*>(const_cast<void*>(dq_proxy->ptr)) : nullptr;
    P.dqp_sb = dq_proxy ? static_cast<int32_t>(dq_proxy->stride_b) : 0; P.dqp_sh = dq_proxy ? static_cast<int32_t>(dq_proxy->stride_h) : 0;
    P.dqp_ss = dq_proxy ? static_cast<int32_t>(dq_proxy->stride_s) : 0;
    P.grad_kl = grad_kl;
    P.S = pb->S; P.NB = pb->S / kBlock; P.Hq = pb->Hq; P.Hp = pb->Hp; P.mpp = pb->Hq / pb->Hp; P.ppk = pb->Hp / pb->Hkv;
    P.Kb = pb->top_k_blocks; P.g_begin = g_begin; P.G = g_count; P.dense = dense ? 1 : 0;
    P.scale = pb->scale;
    P.kl_out_scale = pb->scale / (static_cast<float>(pb->B) * pb->Hp * pb->S);
    const int64_t rows = static_cast<int64_t>(g_count) * P.ppk * P.S;
    const int64_t grid = (rows + 7) / 8;
    FMSA_REQUIRE(grid <= 0x7fffffffLL);
    const dim3 cg(static_cast<unsigned>(grid));
    cudaStream_t cst = static_cast<cudaStream_t>(stream);
    const bool fp16 = pb->dtype == FMSA_DTYPE_FP16;
#define FMSA_BWD_COMBINE(K)                                                                          \
    do {                                                                                             \
        if (fp16) {                                                                                  \
            if (P.split) bwd_combine_wide_kernel<K, true, true><<<cg, 256, 0, cst>>>(P);             \
            else bwd_combine_wide_kernel<K, false, true><<<cg, 256, 0, cst>>>(P);                    \
        } else {                                                                                     \
            if (P.split) bwd_combine_wide_kernel<K, true, false><<<cg, 256, 0, cst>>>(P);            \
            else bwd_combine_wide_kernel<K, false, false><<<cg, 256, 0, cst>>>(P);                   \
        }                                                                                            \
    } while (0)
    if (P.mpp > 8) {
        if (fp16) bwd_combine_kernel<true><<<cg, 256, 0, cst>>>(P);
        else bwd_combine_kernel<false><<<cg, 256, 0, cst>>>(P);
    } else if (P.mpp <= 2) {
        FMSA_BWD_COMBINE(1);
    } else if (P.mpp <= 4) {
        FMSA_BWD_COMBINE(2);
    } else if (P.mpp <= 6) {
        FMSA_BWD_COMBINE(3);
    } else {
        FMSA_BWD_COMBINE(4);
    }
#undef FMSA_BWD_COMBINE
    return check_launch();
}

#ifdef FMSA_TRACE
extern "C" int fmsa_debug_bwd_trace(unsigned long long* host_out) {
    return cudaMemcpyFromSymbol(host_out, fmsa::g_bwd_trace, sizeof(unsigned long long) * 20 * 8) == cudaSuccess ? 0 : -4;
}
#endif
