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
//     S = Q_g K_j^T                tcgen05.mma, both operands in shared memory, fp32 in TMEM
//     m, P = exp2(S*c - m), l      one thread per row (TMEM lane); P goes back into TMEM as bf16,
//                                  over the columns S occupied
//     O_part = P V_j               tcgen05.mma with P as the TMEM operand
//     the partial (O_part unnormalised in bf16, row max m and row sum l) is written to the edge's slot;
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
// inside a CTA the roles (row gather, K/V loads, MMA issue, softmax x2, output) run decoupled and meet
// only through mbarriers, see sparse_fwd_kernel.
#include <type_traits>

#include "host_common.h"
#include "msa_common.cuh"
#include "sm100.cuh"
#include "tma_host.h"

namespace fmsa {
namespace {

#ifdef FMSA_TRACE
// Debug builds only: cycles each warp of CTA 0 spent inside its role (slot 0) and inside waits of kind 1..7.
__device__ unsigned long long g_fwd_trace[24][8];
#endif

struct FwdParams {
    // Row-gather views of q and q_proxy: element row (b, h, s) is matrix row b*row_b + h*row_h + s*row_s.
    int64_t q_row_b, q_row_h, q_row_s;
    int64_t qp_row_b, qp_row_h, qp_row_s;
    int32_t q_rows_total, qp_rows_total;   // first row index outside the views (reads as zeros)
    const int32_t* row_ptr;
    const int32_t* col_q;
    const int32_t* doc_start;   // [B,S] first token of each token's document (packed sequences), or null
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

// A sub-unit as the drawing thread publishes it to the other roles.
struct UnitDesc {
    int32_t j, b, kvh, p, n, chunk0, chunk1, pad;   // chunk1 < 0: no more work
    int64_t e0;                                      // position of the reverse-index row in col_q / the slot space
};

constexpr int kFwdQStages = 3;
constexpr int kUnitRing = 16;
constexpr int kLimitRing = 8;

struct FwdCtrl {
    uint64_t k_full, k_empty, v_full, v_empty, kp_full, kp_empty;
    uint64_t q_full[kFwdQStages], q_empty[kFwdQStages];
    uint64_t s_full[3], p_full[3], s_free[3];
    uint64_t o_full, o_empty;
    uint64_t unit_full[kUnitRing];
    UnitDesc units[kUnitRing];
    alignas(16) uint8_t limits[kLimitRing][128];   // per chunk in flight: last visible key of each row (127 = all)
    uint32_t tmem_slot;
    int32_t abort_flag;
};

// Roles (warp index): 0-3 softmax group A (tiles with an even running index), 4-7 softmax group B
// (odd tiles), 8-11 output group, 12-19 row gather, 20 K/V loads, 21 MMA issue (22, 23 only take
// part in the block-wide steps).  A TMA row gather costs the issuing warp ~65 cycles whatever its size, so the 64
// gathers of a tile are spread over eight warps.
constexpr int kFwdGatherWarps = 8;
constexpr int kFwdThreads = 24 * 32;
// Registers per thread after the warpgroups re-divide the register file (setmaxnreg).  A CTA of 768 threads is
// launched with 80 registers per thread; an increase can only be served from what the other warpgroups of the
// same CTA gave up, so the six warpgroups must not ask for more than 6 x 80 in total (a warpgroup that asks for
// registers nobody released waits forever).
constexpr int kFwdRegsLaunch = 80, kFwdRegsSoftmax = 128, kFwdRegsOutput = 80, kFwdRegsGather = 48, kFwdRegsMisc = 48;
static_assert(2 * kFwdRegsSoftmax + kFwdRegsOutput + 2 * kFwdRegsGather + kFwdRegsMisc <= 6 * kFwdRegsLaunch,
              "register re-division must balance");
static_assert(kFwdRegsLaunch == (65536 / kFwdThreads) / 8 * 8, "registers per thread at launch");
constexpr size_t kFwdTileBytes = static_cast<size_t>(3 + kFwdQStages + 1) * kTileBytes;   // K, V, Kp, Q stages, output staging
constexpr size_t kFwdSmemBytes = kFwdTileBytes + 1024 + sizeof(FwdCtrl);
static_assert(kFwdSmemBytes <= 232448, "shared memory budget of one CTA");

// Warp-specialised forward.  Every role walks the same sequence of sub-units (published by the first gather warp in
// a ring) and, inside a sub-unit, the same sequence of tiles: for each chunk of 128 rows, the main heads of the proxy
// head, then the proxy head.  Hand-offs (all mbarriers, one arrival per warp or per tcgen05.commit):
//   gather warps  q_full[stage] (TMA bytes)  <- q_empty[stage] (commit after S)
//   K/V warp      k_full/v_full/kp_full      <- k_empty/kp_empty (commit after the last S of a sub-unit), v_empty
//   MMA warp      S runs two tiles ahead of P V; s_full[t%3], o_full; s_free[t%3] when tile t no longer needs its S columns
//   softmax       p_full[t%3] when P is in TMEM (or, for a proxy tile, when S has been read)
//   output group  o_empty when the O accumulator has been read
// TMEM: three S accumulators at columns 0, 128 and 256 (tile t uses number t%3; P overwrites the first 64 columns of
// its S), one O accumulator at 384.  With three S accumulators the product S(t+2) does not have to wait for P V(t),
// so a softmax group finds its next S finished when it comes back for it; the price is a single O accumulator, i.e.
// P V(t+1) waits until O(t) has been read out, which takes far less time than a softmax.
// The register file is re-divided between the warpgroups (setmaxnreg): the softmax and output groups get what the
// gather and issue warps do not need.
// VARLEN: document masking of packed sequences (P.doc_start given).  A separate instantiation, so that the plain kernel
// carries none of its registers or code.
template <bool FP16, bool VARLEN>
__global__ void __launch_bounds__(kFwdThreads, 1) sparse_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q,
                                                                    const __grid_constant__ CUtensorMap tmap_qp,
                                                                    const __grid_constant__ CUtensorMap tmap_k,
                                                                    const __grid_constant__ CUtensorMap tmap_v,
                                                                    const __grid_constant__ CUtensorMap tmap_kp,
                                                                    const __grid_constant__ CUtensorMap tmap_o,
                                                                    const FwdParams P) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t tile_k = tiles, tile_v = tiles + kTileBytes, tile_kp = tiles + 2 * kTileBytes;
    const uint32_t tile_q0 = tiles + 3 * kTileBytes, tile_o = tiles + (3 + kFwdQStages) * kTileBytes;
    FwdCtrl* sm = reinterpret_cast<FwdCtrl*>(smem_raw + (tiles - smem_u32(smem_raw)) + kFwdTileBytes);

    const int tid = threadIdx.x, warp = __shfl_sync(0xffffffffu, tid >> 5, 0), lane = tid & 31;
    const int quarter = warp & 3;              // TMEM lane quarter this warp may access
    const int row = quarter * 32 + lane;       // softmax / output: tile row of this thread
    const uint32_t elect = (lane == 0) ? 1u : 0u;
    auto BAR = [&](uint64_t& b) { return smem_u32(&b); };

    if (tid == 0) {
        mbar_init(BAR(sm->k_full), 1);
        mbar_init(BAR(sm->k_empty), 1);
        mbar_init(BAR(sm->v_full), 1);
        mbar_init(BAR(sm->v_empty), 1);
        mbar_init(BAR(sm->kp_full), 1);
        mbar_init(BAR(sm->kp_empty), 1);
        for (int i = 0; i < kFwdQStages; ++i) {
            mbar_init(BAR(sm->q_full[i]), kFwdGatherWarps);
            mbar_init(BAR(sm->q_empty[i]), 1);
        }
        for (int i = 0; i < 3; ++i) {
            mbar_init(BAR(sm->s_full[i]), 1);
            mbar_init(BAR(sm->p_full[i]), 4);
            mbar_init(BAR(sm->s_free[i]), 1);
        }
        mbar_init(BAR(sm->o_full), 1);
        mbar_init(BAR(sm->o_empty), 4);
        for (int i = 0; i < kUnitRing; ++i) mbar_init(BAR(sm->unit_full[i]), 1);
        sm->abort_flag = 0;
        fence_mbar_init();
        prefetch_tmap(&tmap_q);
        prefetch_tmap(&tmap_qp);
        prefetch_tmap(&tmap_k);
        prefetch_tmap(&tmap_v);
        prefetch_tmap(&tmap_kp);
        prefetch_tmap(&tmap_o);
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(&sm->tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = sm->tmem_slot;
    const uint32_t tmem_s0 = tmem, tmem_o0 = tmem + 384;

    const int hpc = P.mpp + (P.with_proxy ? 1 : 0);   // tiles per chunk
    const int lse_stride = P.mpp + 1;
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
    // block barrier of one 128-thread group that also ORs a flag: the roles that use named barriers must
    // leave their loops together
    auto group_or = [&](int id, bool flag) -> bool {
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
    auto warp_arrive = [&](uint32_t bar) {   // every lane has finished (and fenced) its part; one arrival per warp
        __syncwarp();
        if (lane == 0) mbar_arrive(bar);
    };

    uint32_t gt = 0;     // tiles seen so far by this CTA (every role counts the same sequence)
    uint32_t mt = 0;     // main-head tiles seen so far
    uint32_t nsub = 0;   // sub-units seen so far
    uint32_t cbase = 0;  // chunks of the sub-units seen so far: the row limits of chunk c of a sub-unit live in ring
                         // entry (cbase + c - chunk0) % kLimitRing
    uint32_t qs = 0, qph = 0;   // gather warps / MMA warp: Q stage of tile gt and the phase bit of its barriers
    uint32_t sb = 0, sph = 0;   // MMA warp / softmax groups: S accumulator of tile gt (gt % 3) and the phase bit of its barriers

    // Next sub-unit of the common sequence (false: no more work, or the CTA is giving up).  The first gather warp draws
    // the work and publishes the decoded sub-unit; it passes over sub-units that lie beyond the end of their row, so
    // every published entry has work (or is the end marker).  The roles are at most a handful of tiles apart (Q stages
    // + S and O accumulators), far fewer than the ring has entries.
    auto next_unit = [&](uint32_t draw, UnitDesc& ud, auto may_draw) -> bool {
        const uint32_t uslot = draw & (kUnitRing - 1);
        if (decltype(may_draw)::value && warp == 12 && lane == 0) {
            UnitDesc nu;
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
                    nu.j = su.j; nu.b = b; nu.kvh = kvh; nu.p = p; nu.n = n; nu.e0 = e0;
                    nu.chunk0 = su.chunk0;
                    nu.chunk1 = min((n + kBlock - 1) / kBlock, su.chunk0 + kChunksPerSubUnit);
                    break;
                }
            }
            sm->units[uslot] = nu;
            mbar_arrive(BAR(sm->unit_full[uslot]));
        }
        wait(BAR(sm->unit_full[uslot]), (draw / kUnitRing) & 1, 7);
        if (warp >= 8 && warp < 12) bad = group_or(1, bad);
        if (bad) return false;
        ud = sm->units[uslot];
        return ud.chunk1 >= 0;
    };

    // Every role has its own loop over the common sequence of sub-units.
    if (warp >= 20) {
        reg_dec<kFwdRegsMisc>();
        if (warp == 21) {
            // =========================== MMA issue ===========================
            UnitDesc ud;
            for (uint32_t draw = 0; next_unit(draw, ud, std::false_type{}); ++draw, ++nsub) {
                const int ntiles = (ud.chunk1 - ud.chunk0) * hpc;
                wait(BAR(sm->k_full), nsub & 1, 5);
                bool kp_ready = false, v_ready = false;
                uint32_t gts = gt;            // running index of the next S to issue, its accumulator and phase bit
                uint32_t ssb = sb, ssph = sph;
                int hs = 0;                   // its head
                int s_issued = 0;
                auto next_s = [&]() {
                    if (s_issued == ntiles) return;
                    const bool proxy = hs == P.mpp;
                    if (proxy && !kp_ready) {
                        wait(BAR(sm->kp_full), nsub & 1, 5);
                        kp_ready = true;
                    }
                    wait(BAR(sm->q_full[qs]), qph, 1);
                    if (gts >= 3) wait(BAR(sm->s_free[ssb]), ssph ^ 1, 2);
                    tc_fence_after_sync();
                    if (!bad) {
                        umma_tile_128<false, false, FP16>(tmem_s0 + ssb * 128, tile_q0 + qs * kTileBytes, proxy ? tile_kp : tile_k, false,
                                                    elect);
                        umma_commit(BAR(sm->s_full[ssb]), elect);
                        umma_commit(BAR(sm->q_empty[qs]), elect);
                    }
                    if (++qs == kFwdQStages) {
                        qs = 0;
                        qph ^= 1;
                    }
                    if (++ssb == 3) {
                        ssb = 0;
                        ssph ^= 1;
                    }
                    ++gts;
                    if (++hs == hpc) hs = 0;
                    if (++s_issued == ntiles && !bad) {
                        umma_commit(BAR(sm->k_empty), elect);    // every S of this sub-unit has been issued
                        umma_commit(BAR(sm->kp_empty), elect);
                    }
                };
                next_s();
                next_s();
                int hh = 0;
                for (int t = 0; t < ntiles && !bad; ++t, ++gt) {
                    const bool is_proxy = hh == P.mpp;
                    next_s();   // S runs two tiles ahead: the softmax groups never starve
                    wait(BAR(sm->p_full[sb]), sph, 3);
                    if (!is_proxy) {
                        if (!v_ready) {
                            wait(BAR(sm->v_full), nsub & 1, 5);
                            v_ready = true;
                        }
                        if (mt >= 1) wait(BAR(sm->o_empty), (mt - 1) & 1, 4);
                        tc_fence_after_sync();
                        if (!bad) {
                            const uint32_t ts = tmem_s0 + sb * 128;
                            umma_tile_128_ts<true, FP16>(tmem_o0, ts, ts + 32, tile_v, false, elect);   // O = P V_j
                            umma_commit(BAR(sm->o_full), elect);
                        }
                        ++mt;
                    }
                    if (!bad) umma_commit(BAR(sm->s_free[sb]), elect);
                    if (++sb == 3) {
                        sb = 0;
                        sph ^= 1;
                    }
                    if (++hh == hpc) hh = 0;
                }
                if (!bad) umma_commit(BAR(sm->v_empty), elect);
            }
        } else if (warp == 20) {
            // =========================== K / V / Kp loads ===========================
            UnitDesc ud;
            for (uint32_t draw = 0; next_unit(draw, ud, std::false_type{}); ++draw, ++nsub) {
                if (nsub > 0) wait(BAR(sm->k_empty), (nsub - 1) & 1);
                if (!bad && lane == 0) {
                    mbar_arrive_expect_tx(BAR(sm->k_full), kTileBytes);
                    tma_load_tile(tile_k, &tmap_k, ud.j * kBlock, ud.kvh, ud.b, BAR(sm->k_full));
                }
                if (P.with_proxy) {
                    if (nsub > 0) wait(BAR(sm->kp_empty), (nsub - 1) & 1);
                    if (!bad && lane == 0) {
                        mbar_arrive_expect_tx(BAR(sm->kp_full), kTileBytes);
                        tma_load_tile(tile_kp, &tmap_kp, ud.j * kBlock, ud.p / P.pg, ud.b, BAR(sm->kp_full));
                    }
                }
                if (nsub > 0) wait(BAR(sm->v_empty), (nsub - 1) & 1);
                if (!bad && lane == 0) {
                    mbar_arrive_expect_tx(BAR(sm->v_full), kTileBytes);
                    tma_load_tile(tile_v, &tmap_v, ud.j * kBlock, ud.kvh, ud.b, BAR(sm->v_full));
                }
                __syncwarp();
            }
        }
    } else if (warp >= 12) {
        reg_dec<kFwdRegsGather>();
        // =========================== row gather ===========================
        // Gather warp g fetches rows 16g .. 16g+15 of every tile: lanes 0..7 issue one gather4 each (row quad
        // lane/2, 64-column panel lane%2).  Lanes 0..15 hold the query positions of the warp's rows.
        const int g = warp - 12;
        const int quad = (lane >> 1) & 3, panel = lane & 1;
        UnitDesc ud;
        for (uint32_t draw = 0; next_unit(draw, ud, std::true_type{}); ++draw, ++nsub) {
            const int64_t q_base = static_cast<int64_t>(ud.b) * P.q_row_b + static_cast<int64_t>(ud.p) * P.mpp * P.q_row_h;
            const int64_t qp_base = static_cast<int64_t>(ud.b) * P.qp_row_b + static_cast<int64_t>(ud.p) * P.qp_row_h;
            for (int chunk = ud.chunk0; chunk < ud.chunk1 && !bad; ++chunk) {
                int q = -1;
                if (lane < 16) {
                    const int at = chunk * kBlock + 16 * g + lane;
                    if (at < ud.n) {
                        q = P.dense ? (ud.j * kBlock + at) : P.col_q[ud.e0 + at];
                        if (static_cast<unsigned>(q) >= static_cast<unsigned>(P.S) || (q >> 7) < ud.j) {
                            atomicMax(P.status, kStatusBadIndex);
                            q = -1;
                        }
                    }
                    sm->limits[(cbase + chunk - ud.chunk0) & (kLimitRing - 1)][16 * g + lane] =
                        (q >= 0 && (q >> 7) == ud.j) ? static_cast<uint8_t>(q & 127) : static_cast<uint8_t>(127);

                }
                int qr[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) qr[i] = __shfl_sync(0xffffffffu, q, 4 * quad + i);
                for (int hh = 0; hh < hpc && !bad; ++hh, ++gt) {
                    if (gt >= kFwdQStages) wait(BAR(sm->q_empty[qs]), qph ^ 1);
                    if (bad) break;
                    const uint32_t full = BAR(sm->q_full[qs]);
                    if (lane == 0) mbar_arrive_expect_tx(full, kTileBytes / kFwdGatherWarps);
                    __syncwarp();
                    const bool proxy = hh == P.mpp;
                    const int64_t base = proxy ? qp_base : q_base + static_cast<int64_t>(hh) * P.q_row_h;
                    const int64_t rs = proxy ? P.qp_row_s : P.q_row_s;
                    const int oob = proxy ? P.qp_rows_total : P.q_rows_total;
                    int r[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) r[i] = qr[i] >= 0 ? static_cast<int>(base + qr[i] * rs) : oob;
                    const uint32_t dst = tile_q0 + qs * kTileBytes + panel * kPanelBytes + (16 * g + 4 * quad) * 128;
                    const void* tm = proxy ? static_cast<const void*>(&tmap_qp) : static_cast<const void*>(&tmap_q);
                    if (lane < 8) tma_gather4(dst, tm, panel * 64, r[0], r[1], r[2], r[3], full);
                    if (++qs == kFwdQStages) {
                        qs = 0;
                        qph ^= 1;
                    }
                }
            }
            cbase += static_cast<uint32_t>(ud.chunk1 - ud.chunk0);
        }
    } else if (warp >= 8) {
        reg_inc<kFwdRegsOutput>();
        // =========================== output group ===========================
        // Thread = row of the O accumulator: bf16, staged in the operand layout, one TMA tile store per panel.
        // The last, partial chunk of a reverse-index row is written row by row (its slots end where the next
        // row's begin).
        const int otid = tid - 8 * 32;
        UnitDesc ud;
        for (uint32_t draw = 0; next_unit(draw, ud, std::false_type{}); ++draw, ++nsub) {
            const int ntiles = (ud.chunk1 - ud.chunk0) * hpc;
            const int64_t slot_base = ud.e0 - edge_base;   // slot of the first row of the reverse-index row
            int hh = 0, chunk = ud.chunk0;
            for (int t = 0; t < ntiles && !bad; ++t) {
                if (hh != P.mpp) {
                    const int nrows = min(kBlock, ud.n - chunk * kBlock);
                    const int64_t slot0 = slot_base + static_cast<int64_t>(chunk) * kBlock;
                    const bool full = nrows == kBlock;
                    const uint32_t to = tmem_o0;
                    if (otid == 0) tma_store_wait_read();   // the staging tile's previous store has read it
                    wait(BAR(sm->o_full), mt & 1);
                    bad = group_or(1, bad);
                    if (bad) break;
                    tc_fence_after_sync();
                    __nv_bfloat16* grow = P.o_part + ((slot0 + row) * P.mpp + hh) * kHeadDim;
#pragma unroll
                    for (int c = 0; c < 128; c += 32) {
                        uint32_t v[32];
                        tmem_ld32(tmem_addr(to, quarter, c), v);
                        tmem_ld_wait();
                        uint32_t pk[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) pk[i] = pack_act<FP16>(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
                        if (full) {
#pragma unroll
                            for (int k8 = 0; k8 < 4; ++k8)
                                st_shared_v4(tile_o + swz_offset(row, (c >> 3) + k8), pk[4 * k8], pk[4 * k8 + 1], pk[4 * k8 + 2],
                                             pk[4 * k8 + 3]);
                        } else if (row < nrows) {
#pragma unroll
                            for (int k8 = 0; k8 < 4; ++k8)
                                *reinterpret_cast<uint4*>(grow + c + 8 * k8) =
                                    make_uint4(pk[4 * k8], pk[4 * k8 + 1], pk[4 * k8 + 2], pk[4 * k8 + 3]);
                        }
                    }
                    tc_fence_before_sync();
                    warp_arrive(BAR(sm->o_empty));
                    if (full) {
                        fence_async_smem();
                        named_barrier_sync(1, 128);
                        if (otid == 0) {
                            tma_store_3d(&tmap_o, tile_o, 0, hh, static_cast<int>(slot0));
                            tma_store_3d(&tmap_o, tile_o + kPanelBytes, 64, hh, static_cast<int>(slot0));
                            tma_store_commit();
                        }
                    }
                    ++mt;
                }
                if (++hh == hpc) {
                    hh = 0;
                    ++chunk;
                }
            }
        }
        if (otid == 0) tma_store_wait_all();
    } else {
        reg_inc<kFwdRegsSoftmax>();
        // =========================== softmax groups ===========================
        const uint32_t wg = static_cast<uint32_t>(warp >> 2);
        const float2 sc2 = make_float2(P.scale_log2e, P.scale_log2e);
        UnitDesc ud;
        for (uint32_t draw = 0; next_unit(draw, ud, std::false_type{}); ++draw, ++nsub) {
            const int ntiles = (ud.chunk1 - ud.chunk0) * hpc;
            const int64_t slot_base = ud.e0 - edge_base;
            int hh = 0, chunk = ud.chunk0;
            int low = 0, low_chunk = -1;   // document masking: first visible key of this thread's row in the chunk `low_chunk`
            for (int t = 0; t < ntiles && !bad; ++t, ++gt) {
                if ((gt & 1) == wg) {
                    if (VARLEN && low_chunk != chunk) {
                        // Keys before the first token of the row's document are hidden (0 = none of this block, 128 = all
                        // of it).  The row looks its own query position and document start up: shared memory has no room
                        // for a second per-row array, and only packed-sequence calls pay for the two loads.
                        const int at = chunk * kBlock + row;
                        low = 0;
                        if (at < ud.n) {
                            const int q = P.dense ? (ud.j * kBlock + at) : P.col_q[ud.e0 + at];
                            if (static_cast<unsigned>(q) < static_cast<unsigned>(P.S)) {
                                const int lo = P.doc_start[static_cast<int64_t>(ud.b) * P.S + q];
                                const int lb = lo >> 7;
                                low = lb < ud.j ? 0 : (lb == ud.j ? (lo & 127) : 128);
                            }
                        }
                        low_chunk = chunk;
                    }
                    const uint32_t ts = tmem_s0 + sb * 128;
                    const bool is_proxy = hh == P.mpp;
                    const int nrows = min(kBlock, ud.n - chunk * kBlock);
                    wait(BAR(sm->s_full[sb]), sph);
                    if (bad) break;
                    tc_fence_after_sync();
                    // only the first chunk of a reverse-index row can hold rows of the key block itself
                    const bool masked = (chunk == 0) || (VARLEN && __any_sync(0xffffffffu, low > 0));
                    const int limit = (chunk == 0) ? sm->limits[(cbase + chunk - ud.chunk0) & (kLimitRing - 1)][row] : 127;
                    float m = 0.f, l = 0.f;
                    {
                        const bool kMasked = masked, kProxy = is_proxy;
                        // Two passes over the 128 logits of the row (maximum, then exponentials), software-pipelined over
                        // 32-column pieces: the TMEM load of the next piece is in flight while this one is worked on
                        // (tcgen05.wait::ld waits for every load issued so far, hence the order wait, issue, compute).
                        // The loops run over PAIRS of pieces and are not unrolled further: the softmax code of a tile has
                        // to stay small enough for the instruction cache, which five roles share.
                        uint32_t ba[32], bb[32];
                        float mloc = -INFINITY;
                        auto piece_max = [&](const uint32_t (&v)[32], int c) __attribute__((always_inline)) {
                            if (kMasked) {
                                const int lc = limit - c, wc = low - c;
#pragma unroll
                                for (int i = 0; i < 32; ++i) mloc = (i <= lc && (!VARLEN || i >= wc)) ? fmaxf(mloc, __uint_as_float(v[i])) : mloc;
                            } else {
#pragma unroll
                                for (int i = 0; i < 32; i += 2) mloc = fmax3(mloc, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
                            }
                        };
                        tmem_ld32(tmem_addr(ts, quarter, 0), ba);
#pragma unroll 1
                        for (int c = 0; c < 128; c += 64) {
                            tmem_ld_wait();
                            tmem_ld32(tmem_addr(ts, quarter, c + 32), bb);
                            piece_max(ba, c);
                            tmem_ld_wait();
                            tmem_ld32(tmem_addr(ts, quarter, (c + 64) & 127), ba);   // (the last one fetches piece 0 again, for pass 2)
                            piece_max(bb, c + 32);
                        }
                        m = mloc * P.scale_log2e;   // raw logits: scale > 0, so the maximum commutes with it
                        // (dense schedule with documents: a row may see nothing of this block; a finite stand-in for
                        // -inf keeps the merge of the partial statistics free of inf - inf)
                        if (VARLEN) m = fmaxf(m, -1.0e30f);
                        const float2 nm2 = make_float2(-m, -m);
                        float2 l2 = make_float2(0.f, 0.f);
                        auto piece_exp = [&](const uint32_t (&v)[32], int c) __attribute__((always_inline)) {
                            uint32_t pk[16];
                            const int lc = limit - c, wc = low - c;
#pragma unroll
                            for (int i = 0; i < 32; i += 2) {
                                const float2 a = f2_fma(f2_from_bits(v[i], v[i + 1]), sc2, nm2);
                                float p0 = fast_exp2(a.x);
                                float p1 = fast_exp2(a.y);
                                if (kMasked) {
                                    p0 = (i <= lc && (!VARLEN || i >= wc)) ? p0 : 0.f;
                                    p1 = (i + 1 <= lc && (!VARLEN || i + 1 >= wc)) ? p1 : 0.f;
                                }
                                l2 = f2_add(l2, make_float2(p0, p1));
                                pk[i >> 1] = pack_act<FP16>(p0, p1);
                            }
                            // P (bf16, two keys per column) over S columns this thread has already consumed
                            if (!kProxy) tmem_st16(tmem_addr(ts, quarter, c >> 1), pk);
                        };
#pragma unroll 1
                        for (int c = 0; c < 128; c += 64) {
                            tmem_ld_wait();
                            tmem_ld32(tmem_addr(ts, quarter, c + 32), bb);
                            piece_exp(ba, c);
                            tmem_ld_wait();
                            if (c == 0) tmem_ld32(tmem_addr(ts, quarter, 64), ba);
                            piece_exp(bb, c + 32);
                        }
                        l = l2.x + l2.y;
                    }
                    if (!is_proxy) tmem_st_wait();
                    tc_fence_before_sync();
                    warp_arrive(BAR(sm->p_full[sb]));
                    if (row < nrows) {
                        const int64_t slot = slot_base + static_cast<int64_t>(chunk) * kBlock + row;
                        reinterpret_cast<float2*>(P.stat_part)[slot * lse_stride + hh] = make_float2(m, l);
                    }
                }
                if (++sb == 3) {
                    sb = 0;
                    sph ^= 1;
                }
                if (++hh == hpc) {
                    hh = 0;
                    ++chunk;
                }
            }
            cbase += static_cast<uint32_t>(ud.chunk1 - ud.chunk0);
        }
    }
#ifdef FMSA_TRACE
    if (blockIdx.x == 0 && lane == 0) {
        trace_acc[0] = static_cast<unsigned long long>(clock64() - trace_t0);
        for (int i = 0; i < 8; ++i) g_fwd_trace[warp][i] = trace_acc[i];
    }
#endif
    if (bad) {
        atomicMax(P.status, kStatusWaitTimeout);
        // Give loads that are still in flight time to land before the CTA's shared memory is released.
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000) __nanosleep(1000);
    }
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

template <bool FP16>
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
                const uint32_t lo = raw.x;
                const uint32_t hi = raw.y;
                a0 += wi * act_lo<FP16>(lo);
                a1 += wi * act_hi<FP16>(lo);
                a2 += wi * act_lo<FP16>(hi);
                a3 += wi * act_hi<FP16>(hi);
            }
        }
        uint2 o;
        o.x = pack_act<FP16>(a0, a1);
        o.y = pack_act<FP16>(a2, a3);
        *reinterpret_cast<uint2*>(P.out + (static_cast<int64_t>(b) * P.S + q) * (static_cast<int64_t>(P.Hq) * kHeadDim) +
                                  static_cast<int64_t>(h) * kHeadDim + lane * 4) = o;
    }
}

// Wide form for Hq/Hp <= 8, two kernels.  The partial rows of all main heads of one edge are contiguous (mpp * 256
// bytes), so a warp reads them with 16-byte loads per lane in sweeps of 512 bytes.
//   combine_lse_kernel   one thread per (query row, edge): loads the (max, sum) pairs of all heads of its edge at once,
//                        merges them across the row's lanes and writes the row's log-sum-exp per head (and the proxy's).
//   combine_rows_kernel  one warp per query row: an edge's weight exp2(m_edge - m_row) / l_row equals
//                        exp2(m_edge - lse_row * log2 e), so with the row's log-sum-exp already in memory nothing but the
//                        edge positions stands between the kernel and its loads: the partial rows and row maxima of four
//                        edges are in flight before the first sum.
// As one kernel (statistics, then weights through shared memory, then the rows) the same work took 0.443 ms at B=2,
// S=8192, Hq=32, top-k 16 blocks on a B200; the two kernels take 0.062 + 0.338 ms.
constexpr int kWideMaxHeads = 8;

// Slot (record number inside the partial buffers of this pass) of edge `s` of query row (bp, q), or -1.
template <bool DENSE>
struct CombineRow {
    int64_t bp;
    int q, b, p, nslots;
    int64_t edge_base;
    const int32_t* erow;
    __device__ __forceinline__ CombineRow(const CombineParams& P, int64_t w) {
        const int64_t bp0 = static_cast<int64_t>(P.g_begin) * P.ppk;
        bp = bp0 + w / P.S;
        q = static_cast<int>(w % P.S);
        b = static_cast<int>(bp / P.Hp);
        p = static_cast<int>(bp % P.Hp);
        edge_base = DENSE ? dense_edge_base(bp0, P.S, P.NB) : static_cast<int64_t>(P.row_ptr[bp0 * P.NB]);
        nslots = DENSE ? (q >> 7) + 1 : P.Kb;
        erow = DENSE ? nullptr : P.edge_pos + (bp * P.S + q) * P.Kb;
    }
    __device__ __forceinline__ int slot_of(const CombineParams& P, int s) const {   // slot numbers of a pass fit 31 bits
        if (s >= nslots) return -1;
        if (DENSE) return static_cast<int>(dense_edge_base(bp, P.S, P.NB) + dense_row_offset(s, P.S) + (q - s * kBlock) - edge_base);
        const int e = erow[s];
        return e < 0 ? -1 : static_cast<int>(e - edge_base);
    }
};

template <int LPR, bool DENSE>   // lanes per query row: 16 (two rows per warp, at most 16 edges per row) or 32
__global__ void __launch_bounds__(256) combine_lse_kernel(const CombineParams P) {
    constexpr int kMaxHeads = kWideMaxHeads + 1;
    const int lane = threadIdx.x & 31, l = lane % LPR;
    const int64_t nrows = static_cast<int64_t>(P.G) * P.ppk * P.S;
    const int64_t w0 = (static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5)) * (32 / LPR) + lane / LPR;
    const bool valid = w0 < nrows;   // (lanes of a row beyond the end still take part in the shuffles)
    const CombineRow<DENSE> row(P, valid ? w0 : nrows - 1);
    const int lse_stride = P.mpp + 1;
    const float2* stats = reinterpret_cast<const float2*>(P.lse_part);
    const int nheads = P.mpp + (P.lse_proxy ? 1 : 0);
    float hm[kMaxHeads], hs[kMaxHeads];
#pragma unroll
    for (int hh = 0; hh < kMaxHeads; ++hh) {
        hm[hh] = -INFINITY;
        hs[hh] = 0.f;
    }
    for (int s0 = 0; s0 < row.nslots; s0 += LPR) {
        const int sl = valid ? row.slot_of(P, s0 + l) : -1;
        const float2* rec = stats + static_cast<int64_t>(sl) * lse_stride;
#pragma unroll
        for (int hh = 0; hh < kMaxHeads; ++hh) {
            if (hh < nheads && sl >= 0) {
                const float2 st = rec[hh];
                const float mn = fmaxf(hm[hh], st.x);
                hs[hh] = hs[hh] * fast_exp2(hm[hh] - mn) + st.y * fast_exp2(st.x - mn);
                hm[hh] = mn;
            }
        }
    }
    // Across the row's lanes: first the maximum, then the sums brought to it (half the instructions of merging
    // (max, sum) pairs in every round; the kernel is bound by instruction issue, not by memory).
#pragma unroll
    for (int hh = 0; hh < kMaxHeads; ++hh) {
        if (hh < nheads) {
            float m = hm[hh];
#pragma unroll
            for (int off = LPR / 2; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
            float sum = (hm[hh] == -INFINITY) ? 0.f : hs[hh] * fast_exp2(hm[hh] - m);
#pragma unroll
            for (int off = LPR / 2; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
            if (l == 0 && valid) {
                const float total = (m + __log2f(sum)) * kLn2;   // natural-log LSE of the whole row
                if (hh == P.mpp) P.lse_proxy[row.bp * P.S + row.q] = total;
                else P.lse[(static_cast<int64_t>(row.b) * P.Hq + row.p * P.mpp + hh) * P.S + row.q] = total;
            }
        }
    }
}

template <int KITER, bool FP16, bool DENSE>   // Hq/Hp <= 2*KITER: few accumulators, high occupancy (the kernel is bound by memory latency)
__global__ void __launch_bounds__(256, (KITER <= 2) ? 4 : 2) combine_rows_kernel(const CombineParams P) {
    const int lane = threadIdx.x & 31;
    const int64_t w = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    if (w >= static_cast<int64_t>(P.G) * P.ppk * P.S) return;
    const CombineRow<DENSE> row(P, w);
    const int lse_stride = P.mpp + 1;
    const float2* stats = reinterpret_cast<const float2*>(P.lse_part);
    const int nchunk = P.mpp * 16;   // lane owns the 16-byte chunks ck = k*32 + lane of the mpp*128-element edge record
    float acc[KITER][8];
    float row_lse2[KITER];   // the row's log-sum-exp of the lane's head in each sweep, in the log2 domain
#pragma unroll
    for (int k = 0; k < KITER; ++k) {
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[k][e] = 0.f;
        const int hh = min((k * 32 + lane) >> 4, P.mpp - 1);
        row_lse2[k] = P.lse[(static_cast<int64_t>(row.b) * P.Hq + row.p * P.mpp + hh) * P.S + row.q] * kLog2e;
    }
    for (int s0 = 0; s0 < row.nslots; s0 += 32) {
        const int sl = row.slot_of(P, s0 + lane);
        const int cnt = min(32, row.nslots - s0);
        for (int i = 0; i < cnt; i += 4) {
            int si[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int v = __shfl_sync(0xffffffffu, sl, (i + u) & 31);
                si[u] = (i + u < cnt) ? v : -1;
            }
            uint4 raw[4][KITER];
            float em[4][KITER];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const __nv_bfloat16* rec = P.o_part + static_cast<int64_t>(si[u]) * P.mpp * kHeadDim;
#pragma unroll
                for (int k = 0; k < KITER; ++k) {
                    const int ck = k * 32 + lane;
                    const bool ok = si[u] >= 0 && ck < nchunk;
                    raw[u][k] = ok ? *reinterpret_cast<const uint4*>(rec + ck * 8) : make_uint4(0, 0, 0, 0);
                    em[u][k] = ok ? stats[static_cast<int64_t>(si[u]) * lse_stride + (ck >> 4)].x : -INFINITY;
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
#pragma unroll
                for (int k = 0; k < KITER; ++k) {
                    const uint32_t w4[4] = {raw[u][k].x, raw[u][k].y, raw[u][k].z, raw[u][k].w};
                    const float wgt = fast_exp2(em[u][k] - row_lse2[k]);   // an absent edge: exp2(-inf) = 0
                    // Packed two-wide FMAs pay at three and four sweeps (120-128 registers, two CTAs per SM: 4.45 -> 4.20 ms
                    // at Hq/Hp = 6, 64 edges per row); at one and two sweeps they cost registers the 64-register budget
                    // of four CTAs per SM does not have (0.392 -> 0.406 ms at Hq/Hp = 4, 16 edges per row).
                    if constexpr (KITER >= 3) {
                        const float2 wg2 = make_float2(wgt, wgt);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 a = f2_fma(wg2, make_float2(act_lo<FP16>(w4[e]), act_hi<FP16>(w4[e])),
                                                    make_float2(acc[k][2 * e], acc[k][2 * e + 1]));
                            acc[k][2 * e] = a.x;
                            acc[k][2 * e + 1] = a.y;
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            acc[k][2 * e] += wgt * act_lo<FP16>(w4[e]);
                            acc[k][2 * e + 1] += wgt * act_hi<FP16>(w4[e]);
                        }
                    }
                }
            }
        }
    }
    __nv_bfloat16* orow = P.out + (static_cast<int64_t>(row.b) * P.S + row.q) * (static_cast<int64_t>(P.Hq) * kHeadDim) +
                          static_cast<int64_t>(row.p) * P.mpp * kHeadDim;
#pragma unroll
    for (int k = 0; k < KITER; ++k) {
        const int ck = k * 32 + lane;
        if (ck < nchunk) {
            uint4 o;
            o.x = pack_act<FP16>(acc[k][0], acc[k][1]);
            o.y = pack_act<FP16>(acc[k][2], acc[k][3]);
            o.z = pack_act<FP16>(acc[k][4], acc[k][5]);
            o.w = pack_act<FP16>(acc[k][6], acc[k][7]);
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
    FMSA_REQUIRE(gather_compatible(q->ptr, q->stride_b, q->stride_h, q->stride_s));
    if (with_proxy) FMSA_REQUIRE(gather_compatible(q_proxy->ptr, q_proxy->stride_b, q_proxy->stride_h, q_proxy->stride_s));
    const fmsa_tensor* qpx = with_proxy ? q_proxy : q;
    const int hq_px = with_proxy ? pb->Hp : pb->Hq;
    const uint64_t q_rows = gather_rows(pb->B, pb->Hq, pb->S, q->stride_b, q->stride_h, q->stride_s);
    const uint64_t qp_rows = gather_rows(pb->B, hq_px, pb->S, qpx->stride_b, qpx->stride_h, qpx->stride_s);
    CUtensorMap tq, tqp, tk, tv, tkp, to;
    if (!make_tmap_gather(&tq, q->ptr, q_rows) || !make_tmap_gather(&tqp, qpx->ptr, qp_rows) ||
        !make_tmap_bhsd(&tk, k->ptr, pb->B, pb->Hkv, pb->S, k->stride_b, k->stride_h, k->stride_s, 128) ||
        !make_tmap_bhsd(&tv, v->ptr, pb->B, pb->Hkv, pb->S, v->stride_b, v->stride_h, v->stride_s, 128) ||
        !make_tmap_bhsd(&tkp, kp->ptr, pb->B, with_proxy ? pb->Hpkv : pb->Hkv, pb->S, kp->stride_b, kp->stride_h, kp->stride_s, 128) ||
        !make_tmap_partials_swz(&to, o_part, static_cast<uint64_t>(part_slots), static_cast<uint64_t>(pb->Hq / pb->Hp)))
        return FMSA_ERR_CUDA;
    FMSA_REQUIRE(aligned16(o_part) && part_slots < 0x7fffffffLL);

    FwdParams P;
    P.q_row_b = q->stride_b / 128; P.q_row_h = q->stride_h / 128; P.q_row_s = q->stride_s / 128;
    P.qp_row_b = qpx->stride_b / 128; P.qp_row_h = qpx->stride_h / 128; P.qp_row_s = qpx->stride_s / 128;
    P.q_rows_total = static_cast<int32_t>(q_rows); P.qp_rows_total = static_cast<int32_t>(qp_rows);
    P.row_ptr = row_ptr; P.col_q = col_q; P.doc_start = pb->doc_start;
    P.o_part = static_cast<__nv_bfloat16*>(o_part); P.stat_part = lse_part;
    P.counter = counter; P.status = status;
    P.S = pb->S; P.NB = pb->S / kBlock; P.Hq = pb->Hq; P.Hkv = pb->Hkv; P.Hp = pb->Hp;
    P.mpp = pb->Hq / pb->Hp; P.ppk = pb->Hp / pb->Hkv; P.pg = pb->Hp / pb->Hpkv;
    P.g_begin = g_begin; P.G = g_count; P.with_proxy = with_proxy ? 1 : 0; P.dense = dense ? 1 : 0;
    P.scale_log2e = pb->scale * kLog2e;

    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int sms = device_sm_count();
    const bool fp16 = pb->dtype == FMSA_DTYPE_FP16;
    const bool varlen = P.doc_start != nullptr;
    const void* kfn = fp16 ? (varlen ? reinterpret_cast<const void*>(sparse_fwd_kernel<true, true>) : reinterpret_cast<const void*>(sparse_fwd_kernel<true, false>))
                           : (varlen ? reinterpret_cast<const void*>(sparse_fwd_kernel<false, true>) : reinterpret_cast<const void*>(sparse_fwd_kernel<false, false>));
    if (sms <= 0 || !ensure_smem_attr(kfn, kFwdSmemBytes)) return FMSA_ERR_CUDA;
    if (cudaMemsetAsync(counter, 0, sizeof(int32_t), st) != cudaSuccess) return FMSA_ERR_CUDA;
    P.n_subunits = g_count * subunits_per_group(P.NB, P.ppk, kChunksPerSubUnit);
    FMSA_REQUIRE(P.n_subunits < 0x7fffffffLL);
    const int grid = static_cast<int>(P.n_subunits < sms ? P.n_subunits : sms);
    if (fp16 && varlen) sparse_fwd_kernel<true, true><<<grid, kFwdThreads, kFwdSmemBytes, st>>>(tq, tqp, tk, tv, tkp, to, P);
    else if (fp16) sparse_fwd_kernel<true, false><<<grid, kFwdThreads, kFwdSmemBytes, st>>>(tq, tqp, tk, tv, tkp, to, P);
    else if (varlen) sparse_fwd_kernel<false, true><<<grid, kFwdThreads, kFwdSmemBytes, st>>>(tq, tqp, tk, tv, tkp, to, P);
    else sparse_fwd_kernel<false, false><<<grid, kFwdThreads, kFwdSmemBytes, st>>>(tq, tqp, tk, tv, tkp, to, P);
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
    const bool f16 = pb->dtype == FMSA_DTYPE_FP16;
    if (P.mpp > kWideMaxHeads) {
        if (f16) combine_kernel<true><<<cg, 256, 0, cst>>>(P);
        else combine_kernel<false><<<cg, 256, 0, cst>>>(P);
        return check_launch();
    }
    if (dense) combine_lse_kernel<32, true><<<cg, 256, 0, cst>>>(P);
    else if (P.Kb <= 16) combine_lse_kernel<16, false><<<dim3(static_cast<unsigned>((rows + 15) / 16)), 256, 0, cst>>>(P);
    else combine_lse_kernel<32, false><<<cg, 256, 0, cst>>>(P);
#define FMSA_ROWS2(K, F) (dense ? combine_rows_kernel<K, F, true><<<cg, 256, 0, cst>>>(P) : combine_rows_kernel<K, F, false><<<cg, 256, 0, cst>>>(P))
#define FMSA_ROWS(K) (f16 ? FMSA_ROWS2(K, true) : FMSA_ROWS2(K, false))
    if (P.mpp <= 2) FMSA_ROWS(1);
    else if (P.mpp <= 4) FMSA_ROWS(2);
    else if (P.mpp <= 6) FMSA_ROWS(3);
    else FMSA_ROWS(4);
#undef FMSA_ROWS2
#undef FMSA_ROWS
    return check_launch();
}

#ifdef FMSA_TRACE
extern "C" int fmsa_debug_fwd_trace(unsigned long long* host_out) {
    return cudaMemcpyFromSymbol(host_out, fmsa::g_fwd_trace, sizeof(unsigned long long) * 24 * 8) == cudaSuccess ? 0 : -4;
}
#endif
