// Fused MSA backward, key-block stationary: dQ, dK, dV and the on-the-fly KL gradients dQp, dKp.
//
// Work unit = (batch, KV head, key block j), exactly as in the forward: K_j and V_j stay in shared
// memory, the unit walks the reverse-index row of every proxy head of its group in chunks of 128
// gathered query rows.  For each chunk the main heads of the proxy head run one after another
//     S  = Q_g K_j^T            dP = dO_g V_j^T                     (tcgen05, K-major operands)
//     P  = exp2(S*c - lse)      dS = P o (dP - delta)               (fp32, rounded to bf16 in smem)
//     dV += P^T dO_g            dK += dS^T Q_g                      (MN-major operands, TMEM-resident
//                                                                    accumulators for the whole unit)
//     dQ  = dS K_j  -> scaled, reduced into the fp32 dQ buffer with vector red.add
// while every thread sums the bf16-rounded P of its (row, columns) over the heads: the KL teacher.
// Then one proxy tile:
//     Sp = Qp_g Kp_j^T          p_px = exp2(Sp*c - lse_proxy)       dSp = p_px - teacher/mpp
//     dQp = dSp Kp_j, dKp = dSp^T Qp_g -> scaled by scale/(B*Hp*S), reduced into fp32 buffers.
// The unit owns dK_j and dV_j, so they are written once, in bf16, without atomics.
//
// Formulas and rounding points follow the reference kernel
// (flash_msa/msa_backward_cutedsl.py:456-733: P and dS rounded to the input type before the
// second products, teacher averaged from the rounded P, ds_px = c*(p_px - teacher)) and
// flash_msa/flash_msa.py:99-125 (delta, 1/(B*Hp*S), grad_kl applied afterwards on the device).
// `dense` mode is the warmup backward (flash_msa/warmup/msa_backward_cutedsl_warmup.py:117-191):
// every causal (query block, key block) pair, with the schedule implied instead of built on the host.
#include <cuda_fp16.h>

#include "host_common.h"
#include "msa_common.cuh"
#include "sm100.cuh"
#include "tma_host.h"

namespace fmsa {
namespace {

struct BwdParams {
    const __nv_bfloat16 *q, *qp, *kp, *dout;
    int64_t q_sb, q_sh, q_ss;
    int64_t qp_sb, qp_sh, qp_ss;
    int64_t kp_sb, kp_sh, kp_ss;
    int64_t do_sb, do_sh, do_ss;
    const float *lse, *lse_proxy, *delta;   // [B,Hq,S], [B,Hp,S], [B,Hq,S]
    const int32_t* row_ptr;
    const int32_t* col_q;
    __nv_bfloat16* dq_part;    // [(edge - edge_base) * mpp + head][128]: per-edge dQ contributions
    __nv_bfloat16* dqp_part;   // [(edge - edge_base)][128]: per-edge dQp contributions (already * scale/(B*Hp*S))
    // fp32, zero-initialised: [B,Hpkv,S,128], [B,Hkv,S,128] x2
    float *dkp_acc, *dk_acc, *dv_acc;
    int32_t* counter;
    int32_t* status;
    int S, NB, Hq, Hkv, Hp, Hpkv, mpp, ppk, pg;
    int g_begin, G;
    int64_t n_subunits;
    int with_kl, dense;
    float scale, scale_log2e, kl_out_scale;   // kl_out_scale = scale / (B*Hp*S)
    float* kl_value;    // optional: += KL(teacher || proxy) summed over this launch's rows, / (B*Hp*S)
    float kl_value_scale;   // ln(2) / (B*Hp*S)
};

struct BwdSmem {
    uint64_t bar_kv, bar_a, bar_dq, bar_dv, bar_dk;
    uint32_t tmem_slot;
    int32_t unit;
    int32_t rows[3][128];
};

constexpr int kBwdWorkers = 512;            // 16 worker warps
constexpr int kBwdThreads = kBwdWorkers + 32;   // + one warp whose lane 0 only issues tcgen05.mma
constexpr size_t kBwdSmemBytes = 7 * kTileBytes + 1024 + sizeof(BwdSmem);

// Roles.  Worker warp w (0..15) may read TMEM lanes 32*(w%4)..+31 and owns the 32 accumulator
// columns starting at 32*(w/4).  Warp 16 is the MMA issuer: a thread that issues tcgen05.mma is held
// while the tensor core's queue is full, so it must not carry any other work.
//
// Shared memory: K_j, V_j (resident), two Q buffers (rows gathered one tile ahead), one dO buffer
// (refilled as soon as dV has consumed it), P and dS.
// TMEM (512 columns): [0,128) S, then dKp^T in a proxy tile; [128,256) dP, then dQ^T / dQp^T;
// [256,384) dV^T; [384,512) dK^T.
//
// Products of the second group are issued TRANSPOSED (M = head dimension): a TMEM lane is then a
// head-dimension index and a column a row of the output, so the 32 lanes of a warp write 32
// consecutive elements of ONE output row per instruction.
//
// Per tile:   issuer:  [S ahead] dP | ......... | dQ^T dV^T dK^T S(next) |
//             workers: gather Q(next), wait | P, dS | wait dQ, store it; refill dO; (dKp) |
// dQ and dQp leave the kernel as bf16 per-edge partial rows (summed per query row by
// bwd_combine_kernel): fp32 atomics for them would move ~6 GB through the L2 atomic units per step.
__global__ void __launch_bounds__(kBwdThreads, 1) sparse_bwd_kernel(const __grid_constant__ CUtensorMap tmap_k,
                                                                    const __grid_constant__ CUtensorMap tmap_v,
                                                                    const __grid_constant__ CUtensorMap tmap_dq,
                                                                    const __grid_constant__ CUtensorMap tmap_dqp,
                                                                    const BwdParams P) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t tile_k = tiles, tile_v = tiles + kTileBytes;
    const uint32_t tile_q0 = tiles + 2 * kTileBytes, tile_do = tiles + 4 * kTileBytes;
    const uint32_t tile_p = tiles + 5 * kTileBytes, tile_ds = tiles + 6 * kTileBytes;
    BwdSmem* sm = reinterpret_cast<BwdSmem*>(smem_raw + (tiles - smem_u32(smem_raw)) + 7 * kTileBytes);

    // The warp index goes through a shuffle so that the compiler knows it, and every branch on the warp's
    // role, to be uniform across the warp: the issuer's descriptor arithmetic can then use the uniform datapath.
    const int tid = threadIdx.x, warp = __shfl_sync(0xffffffffu, tid >> 5, 0), lane = tid & 31;
    const bool worker = warp < 16;
    const bool issuer = (warp == 16);            // the whole warp runs the issue sequence ...
    const uint32_t elect = (lane == 0) ? 1u : 0u;   // ... and only this lane's instructions take effect
    const int quarter = warp & 3, cg = (warp >> 2) & 3;
    const int row = quarter * 32 + lane, c0 = cg * 32;
    const GatherLane glane = make_gather_lane(tid & 511);
    const uint32_t bar_kv = smem_u32(&sm->bar_kv), bar_a = smem_u32(&sm->bar_a), bar_dq = smem_u32(&sm->bar_dq);
    const uint32_t bar_dv = smem_u32(&sm->bar_dv), bar_dk = smem_u32(&sm->bar_dk);

    if (tid == 0) {
        mbar_init(bar_kv, 1);
        mbar_init(bar_a, 1);
        mbar_init(bar_dq, 1);
        mbar_init(bar_dv, 1);
        mbar_init(bar_dk, 1);
        fence_mbar_init();
        prefetch_tmap(&tmap_k);
        prefetch_tmap(&tmap_v);
        prefetch_tmap(&tmap_dq);
        if (P.with_kl) prefetch_tmap(&tmap_dqp);
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(&sm->tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = __shfl_sync(0xffffffffu, sm->tmem_slot, 0);
    const uint32_t t_s = tmem, t_dp = tmem + 128, t_dv = tmem + 256, t_dk = tmem + 384;

    const int hpc = P.mpp + (P.with_kl ? 1 : 0);
    const float inv_mpp = 1.f / static_cast<float>(P.mpp);
    const int64_t edge_base = P.dense ? dense_edge_base(static_cast<int64_t>(P.g_begin) * P.ppk, P.S, P.NB)
                                      : static_cast<int64_t>(P.row_ptr[static_cast<int64_t>(P.g_begin) * P.ppk * P.NB]);
    uint32_t ph_kv = 0, ph_a = 0, ph_dq = 0, ph_dv = 0, ph_dk = 0;
    bool bad = false;   // a bounded wait gave up: later waits are skipped, the status word is set at the end
    float kl_acc = 0.f;   // this thread's share of sum t * (log2 t - log2 p_proxy), when the KL value is asked for

    for (;;) {
        if (tid == 0) sm->unit = atomicAdd(P.counter, 1);
        __syncthreads();
        const int u = __shfl_sync(0xffffffffu, sm->unit, 0);   // (uniform anyway; tells the compiler so)
        __syncthreads();
        if (u >= P.n_subunits) break;
        const SubUnit su = decode_subunit(u, P.NB, P.ppk);
        const int j = su.j;
        const int g = P.g_begin + su.g;
        const int b = g / P.Hkv, kvh = g % P.Hkv;
        const int p = kvh * P.ppk + su.pp;
        const int kph = p / P.pg;
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
        if (tid == 0) {
            mbar_arrive_expect_tx(bar_kv, 2 * kTileBytes);
            tma_load_tile(tile_k, &tmap_k, j * kBlock, kvh, b, bar_kv);
            tma_load_tile(tile_v, &tmap_v, j * kBlock, kvh, b, bar_kv);
        }
        const int ntiles = (chunk1 - chunk0) * hpc;
        const __nv_bfloat16* q_b = P.q + static_cast<int64_t>(b) * P.q_sb;
        const __nv_bfloat16* do_b = P.dout + static_cast<int64_t>(b) * P.do_sb;
        const __nv_bfloat16* qp_bp = P.qp + static_cast<int64_t>(b) * P.qp_sb + static_cast<int64_t>(p) * P.qp_sh;
        const __nv_bfloat16* kp_blk = P.kp + static_cast<int64_t>(b) * P.kp_sb + static_cast<int64_t>(kph) * P.kp_sh +
                                      static_cast<int64_t>(j) * kBlock * P.kp_ss;

        auto stage_rows = [&](int chunk, int rb) {
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
                sm->rows[rb][tid] = qid;
            }
        };
        // Q rows of a tile (main head hh or the proxy head) into Q buffer `par` (workers only)
        auto gather_q = [&](int hh, int rb, int par) {
            const uint32_t dst = tile_q0 + par * kTileBytes;
            if (hh < P.mpp)
                gather_tile_512(dst, q_b + static_cast<int64_t>(p * P.mpp + hh) * P.q_sh, P.q_ss, sm->rows[rb], glane);
            else
                gather_tile_512(dst, qp_bp, P.qp_ss, sm->rows[rb], glane);
        };
        // dO rows of a main tile, or the proxy keys Kp_j of a proxy tile, into the dO buffer
        auto gather_do = [&](int hh, int rb) {
            if (hh < P.mpp)
                gather_tile_512(tile_do, do_b + static_cast<int64_t>(p * P.mpp + hh) * P.do_sh, P.do_ss, sm->rows[rb], glane);
            else
                load_tile_512(tile_do, kp_blk, P.kp_ss, glane);
        };

        // ---- prologue: operands of tile 0, S of tile 0 ----
        stage_rows(chunk0, 0);
        if (ntiles > 1 && hpc == 1) stage_rows(chunk0 + 1, 1);
        __syncthreads();
        if (worker) {
            gather_q(0, 0, 0);
            gather_do(0, 0);
            cp_async_commit();
            cp_async_wait<0>();
            fence_async_smem();
        }
        __syncthreads();
        if (issuer) {
            if (!bad) bad = !mbar_wait(bar_kv, ph_kv);
            tc_fence_after_sync();
            umma_tile_128<false, false>(t_s, tile_q0, tile_k, false, elect);   // S(0); tile 0 is always a main head
        }
        ph_kv ^= 1;
        bool s_issued = true;
        bool kv_acc = false;       // dK/dV accumulators hold something
        bool dk_pending = false;   // bar_dk of the previous tile has not been waited for yet

        // sum over the main heads of P for this thread's 32 columns: the KL teacher.  Kept as packed
        // fp16 pairs (values in [0,1], at most Hq/Hp addends; the result is rounded to bf16 anyway).
        __half2 teacher[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) teacher[i] = __floats2half2_rn(0.f, 0.f);

        int hh = 0, chunk = chunk0, rb = 0;   // head, chunk and row-list buffer of the current tile
        for (int t = 0; t < ntiles; ++t) {
            const bool is_proxy = hh == P.mpp;
            const bool has_next = t + 1 < ntiles;
            // the next two tiles, without divisions
            int hh1 = hh + 1, chunk_1 = chunk, rb1 = rb;
            if (hh1 == hpc) {
                hh1 = 0;
                ++chunk_1;
                rb1 = (rb == 2) ? 0 : rb + 1;
            }
            int hh2 = hh1 + 1, chunk_2 = chunk_1, rb2 = rb1;
            if (hh2 == hpc) {
                hh2 = 0;
                ++chunk_2;
                rb2 = (rb1 == 2) ? 0 : rb1 + 1;
            }
            const bool next_proxy = has_next && (hh1 == P.mpp);
            const uint32_t qbuf = tile_q0 + (t & 1) * kTileBytes;
            const int nrows = min(kBlock, n - chunk * kBlock);
            const int64_t slot0 = e0 - edge_base + static_cast<int64_t>(chunk) * kBlock;

            // ---- A: issuer: S (unless issued ahead) and dP;  workers: fetch the next tile's Q rows ----
            if (issuer) {
                tc_fence_after_sync();
                if (is_proxy) {
                    umma_tile_128<false, false>(t_s, qbuf, tile_do, false, elect);              // Sp = Qp_g Kp_j^T
                } else {
                    if (!s_issued) umma_tile_128<false, false>(t_s, qbuf, tile_k, false, elect);   // S  = Q_g K_j^T
                    umma_tile_128<false, false>(t_dp, tile_do, tile_v, false, elect);           // dP = dO_g V_j^T
                }
                umma_commit(bar_a, elect);
            }
            if (worker) {
                // per-row statistics: only the loads are issued here; they are consumed after the waits below
                float raw_lse = INFINITY, row_delta = 0.f;   // +inf: exp2(-inf) = 0, a dead row contributes nothing
                int limit = 127;
                {
                    const int qid = sm->rows[rb][row];
                    if (qid >= 0) {
                        if ((qid >> 7) == j) limit = qid & 127;
                        if (is_proxy) {
                            raw_lse = P.lse_proxy[bp * P.S + qid];
                        } else {
                            const int64_t at = (static_cast<int64_t>(b) * P.Hq + p * P.mpp + hh) * P.S + qid;
                            raw_lse = P.lse[at];
                            row_delta = P.delta[at];
                        }
                    }
                }
                if (dk_pending) {          // dK^T of the previous tile still reads the other Q buffer
                    if (!bad) bad = !mbar_wait(bar_dk, ph_dk);
                    ph_dk ^= 1;
                }
                if (has_next) gather_q(hh1, rb1, (t + 1) & 1);
                cp_async_commit();
                if (!bad) bad = !mbar_wait(bar_a, ph_a);
                ph_a ^= 1;
                tc_fence_after_sync();
                if (t + 2 < ntiles && chunk_2 != chunk_1) stage_rows(chunk_2, rb2);

                // ---- B: P, dS (or dSp) for this thread's (row, 32 columns) ----
                // Only the first chunk of a reverse-index row can hold rows of the key block itself
                // (they are the smallest query positions), so only there the causal mask is needed.
                const bool masked = (chunk == 0);
                const float neg_lse = -raw_lse * kLog2e;
                const uint64_t sc2 = f2_pack(P.scale_log2e, P.scale_log2e), nl2 = f2_pack(neg_lse, neg_lse);
                const uint64_t nd2 = f2_pack(-row_delta, -row_delta);
#pragma unroll
                for (int c = 0; c < 32; c += 16) {
                    uint32_t sv[16], dv[16];
                    tmem_ld16(tmem_addr(t_s, quarter, c0 + c), sv);
                    if (!is_proxy) tmem_ld16(tmem_addr(t_dp, quarter, c0 + c), dv);
                    tmem_ld_wait();
                    uint32_t pk[8], dk[8];
#pragma unroll
                    for (int i = 0; i < 16; i += 2) {
                        float a0, a1;   // log2 of the probability
                        f2_unpack(f2_fma(f2_pack(__uint_as_float(sv[i]), __uint_as_float(sv[i + 1])), sc2, nl2), a0, a1);
                        float p0 = fast_exp2(a0);
                        float p1 = fast_exp2(a1);
                        if (masked) {
                            p0 = (c0 + c + i <= limit) ? p0 : 0.f;
                            p1 = (c0 + c + i + 1 <= limit) ? p1 : 0.f;
                        }
                        if (!is_proxy) {
                            const uint64_t pp = f2_pack(p0, p1);
                            float d0, d1;   // dS = P o (dP - delta)
                            f2_unpack(f2_mul(pp, f2_add(f2_pack(__uint_as_float(dv[i]), __uint_as_float(dv[i + 1])), nd2)), d0, d1);
                            pk[i >> 1] = pack_bf16(p0, p1);
                            dk[i >> 1] = pack_bf16(d0, d1);
                            teacher[(c + i) >> 1] = __hadd2(teacher[(c + i) >> 1], __floats2half2_rn(p0, p1));
                        } else {
                            const float2 tt = __half22float2(teacher[(c + i) >> 1]);
                            const float t0 = tt.x * inv_mpp, t1 = tt.y * inv_mpp;
                            dk[i >> 1] = pack_bf16(p0 - t0, p1 - t1);
                            if (P.kl_value) {   // KL(teacher || proxy) = sum t (ln t - ln p); t = 0 contributes nothing
                                kl_acc += (t0 > 0.f) ? t0 * (fast_log2(t0) - a0) : 0.f;
                                kl_acc += (t1 > 0.f) ? t1 * (fast_log2(t1) - a1) : 0.f;
                            }
                            teacher[(c + i) >> 1] = __floats2half2_rn(0.f, 0.f);
                        }
                    }
#pragma unroll
                    for (int k8 = 0; k8 < 2; ++k8) {
                        const uint32_t off = swz_offset(row, ((c0 + c) >> 3) + k8);
                        if (!is_proxy) st_shared_v4(tile_p + off, pk[4 * k8], pk[4 * k8 + 1], pk[4 * k8 + 2], pk[4 * k8 + 3]);
                        st_shared_v4(tile_ds + off, dk[4 * k8], dk[4 * k8 + 1], dk[4 * k8 + 2], dk[4 * k8 + 3]);
                    }
                }
                cp_async_wait<0>();      // Q rows of the next tile have landed
                fence_async_smem();
                tc_fence_before_sync();
            }
            __syncthreads();

            // ---- C: issuer: dV^T (frees the dO and P buffers), dQ^T, dK^T, S of the next main tile ----
            const bool s_ahead = has_next && !next_proxy && !is_proxy;
            if (issuer) {
                tc_fence_after_sync();
                if (is_proxy) {
                    umma_tile_128<true, false>(t_dp, tile_do, tile_ds, false, elect);   // dQp^T = Kp_j^T dSp^T
                    umma_commit(bar_dq, elect);
                    umma_commit(bar_dv, elect);
                    umma_tile_128<true, true>(t_s, qbuf, tile_ds, false, elect);        // dKp^T = Qp_g^T dSp
                    umma_commit(bar_dk, elect);
                } else {
                    umma_tile_128<true, true>(t_dv, tile_do, tile_p, kv_acc, elect);    // dV^T += dO_g^T P  (frees dO and P)
                    umma_commit(bar_dv, elect);
                    umma_tile_128<true, false>(t_dp, tile_k, tile_ds, false, elect);    // dQ^T  = K_j^T dS^T
                    umma_commit(bar_dq, elect);
                    umma_tile_128<true, true>(t_dk, qbuf, tile_ds, kv_acc, elect);      // dK^T += Q_g^T dS
                    umma_commit(bar_dk, elect);
                    if (s_ahead) umma_tile_128<false, false>(t_s, tile_q0 + ((t + 1) & 1) * kTileBytes, tile_k, false, elect);
                }
            }
            if (!is_proxy) kv_acc = true;
            s_issued = s_ahead;
            dk_pending = true;

            // ---- D: workers: refill the dO buffer, write dQ^T out, reduce dKp^T ----
            if (worker) {
                if (!bad) bad = !mbar_wait(bar_dv, ph_dv);
                ph_dv ^= 1;
                if (has_next) gather_do(hh1, rb1);
                cp_async_commit();
                if (!bad) bad = !mbar_wait(bar_dq, ph_dq);
                ph_dq ^= 1;
                tc_fence_after_sync();
                {
                    // This thread holds head-dimension index `row` of the output rows c0 .. c0+31 (the
                    // factor scale, or scale/(B*Hp*S) for the proxy, is applied by the combine kernel).
                    // A full chunk is transposed through the P buffer (free since dV^T) into dense
                    // [row][d] order and leaves with ONE TMA tile store; the partial last chunk of a
                    // reverse-index row is written directly.
                    const bool full = (nrows == kBlock);
                    __nv_bfloat16* dst = is_proxy ? P.dqp_part + (slot0 + c0) * kHeadDim + row
                                                  : P.dq_part + ((slot0 + c0) * P.mpp + hh) * kHeadDim + row;
                    const int64_t rstride = is_proxy ? kHeadDim : static_cast<int64_t>(P.mpp) * kHeadDim;
#pragma unroll
                    for (int c = 0; c < 32; c += 16) {
                        uint32_t v[16];
                        tmem_ld16(tmem_addr(t_dp, quarter, c0 + c), v);
                        tmem_ld_wait();
                        if (full) {
                            const uint32_t sbase = tile_p + static_cast<uint32_t>((c0 + c) * 256 + row * 2);
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                const __nv_bfloat16 hv = __float2bfloat16_rn(__uint_as_float(v[i]));
                                asm volatile("st.shared.b16 [%0], %1;" ::"r"(sbase + i * 256), "h"(*reinterpret_cast<const uint16_t*>(&hv)) : "memory");
                            }
                        } else {
                            store_transposed_bf16_16(dst + c * rstride, rstride, v, c0 + c, nrows);
                        }
                    }
                    if (full) {
                        fence_async_smem();
                        named_barrier_sync(5, kBwdWorkers);
                        if (tid == 0) {
                            if (is_proxy) tma_store_3d(&tmap_dqp, tile_p, 0, 0, static_cast<int>(slot0));
                            else tma_store_3d(&tmap_dq, tile_p, 0, hh, static_cast<int>(slot0));
                            tma_store_commit();
                        }
                    }
                }
                if (is_proxy) {
                    if (!bad) bad = !mbar_wait(bar_dk, ph_dk);
                    ph_dk ^= 1;
                    tc_fence_after_sync();
                    float* kbase = P.dkp_acc + ((static_cast<int64_t>(b) * P.Hpkv + kph) * P.S + j * kBlock + c0) * kHeadDim + row;
#pragma unroll
                    for (int c = 0; c < 32; c += 16) {
                        uint32_t v[16];
                        tmem_ld16(tmem_addr(t_s, quarter, c0 + c), v);
                        tmem_ld_wait();
#pragma unroll
#pragma unroll
                        for (int i = 0; i < 16; ++i) atomicAdd(kbase + (c + i) * kHeadDim, __uint_as_float(v[i]));
                    }
                }
                cp_async_wait<0>();      // dO rows (or Kp_j) of the next tile have landed
                if (tid == 0) tma_store_wait_read();   // the P buffer may be overwritten by the next tile
                fence_async_smem();
                tc_fence_before_sync();
            }
            if (is_proxy) dk_pending = false;
            __syncthreads();
            hh = hh1;
            chunk = chunk_1;
            rb = rb1;
        }
        // ---- sub-unit epilogue: add this sub-unit's share of dK_j and dV_j ----
        if (worker) {
            if (dk_pending) {
                if (!bad) bad = !mbar_wait(bar_dk, ph_dk);
                ph_dk ^= 1;
            }
            tc_fence_after_sync();
            // accumulators are transposed: lane = head-dimension index, column = key row of the block
            const int64_t at = ((static_cast<int64_t>(b) * P.Hkv + kvh) * P.S + j * kBlock) * kHeadDim + row;
#pragma unroll 1
            for (int which = 0; which < 2; ++which) {
                float* dst = (which == 0 ? P.dv_acc : P.dk_acc) + at;
#pragma unroll
                for (int c = 0; c < 32; c += 16) {
                    uint32_t v[16];
                    tmem_ld16(tmem_addr(which == 0 ? t_dv : t_dk, quarter, c0 + c), v);
                    tmem_ld_wait();
                    if (kv_acc) {
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            atomicAdd(dst + static_cast<int64_t>(c0 + c + i) * kHeadDim, __uint_as_float(v[i]));
                    }
                }
            }
            tc_fence_before_sync();
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    if (tid == 0) tma_store_wait_all();
    if (P.kl_value && worker) {
        for (int o = 16; o > 0; o >>= 1) kl_acc += __shfl_xor_sync(0xffffffffu, kl_acc, o);
        if (lane == 0) atomicAdd(P.kl_value, kl_acc * P.kl_value_scale);
    }
    if (bad) atomicMax(P.status, kStatusWaitTimeout);
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
    __nv_bfloat16* dq;         // [B,Hq,S,128]
    __nv_bfloat16* dqp;        // [B,Hp,S,128] or null
    const float* grad_kl;      // device scalar or null (= 1)
    float scale, kl_out_scale; // factors the backward kernel left out of its partial rows
    int S, NB, Hq, Hp, mpp, ppk, Kb;
    int g_begin, G, dense;
};

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
                const __nv_bfloat16* src = proxy ? P.dqp_part + si * kHeadDim : P.dq_part + (si * P.mpp + hh) * kHeadDim;
                const uint2 raw = *reinterpret_cast<const uint2*>(src + lane * 4);
                const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
                const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
                a0 += __low2float(lo);
                a1 += __high2float(lo);
                a2 += __low2float(hi);
                a3 += __high2float(hi);
            }
        }
        uint2 o;
        if (proxy) {
            o.x = pack_bf16(a0 * gk, a1 * gk);
            o.y = pack_bf16(a2 * gk, a3 * gk);
            *reinterpret_cast<uint2*>(P.dqp + (bp * P.S + q) * kHeadDim + lane * 4) = o;
        } else {
            o.x = pack_bf16(a0 * P.scale, a1 * P.scale);
            o.y = pack_bf16(a2 * P.scale, a3 * P.scale);
            *reinterpret_cast<uint2*>(P.dq + ((static_cast<int64_t>(b) * P.Hq + p * P.mpp + hh) * P.S + q) * kHeadDim + lane * 4) = o;
        }
    }
}

// Wide variant for Hq/Hp <= 8: one sweep over the contiguous mpp*256-byte record of each edge.
template <int KITER>   // Hq/Hp <= 2*KITER: few accumulators, high occupancy (latency bound)
__global__ void __launch_bounds__(256, (KITER <= 2) ? 4 : 3) bwd_combine_wide_kernel(const BwdCombineParams P) {
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
    for (int s0 = 0; s0 < nslots; s0 += 32) {
        const int64_t sl = slot_of(s0 + lane);
        const int cnt = min(32, nslots - s0);
#pragma unroll 4
        for (int i = 0; i < cnt; ++i) {
            const int64_t si = __shfl_sync(0xffffffffu, sl, i);
            if (si < 0) continue;
            const __nv_bfloat16* rec = P.dq_part + si * P.mpp * kHeadDim;
#pragma unroll
            for (int k = 0; k < KITER; ++k) {
                const int ck = k * 32 + lane;
                if (ck < nchunk) {
                    const uint4 raw = *reinterpret_cast<const uint4*>(rec + ck * 8);
                    const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const __nv_bfloat162 v2 = *reinterpret_cast<const __nv_bfloat162*>(&u[e]);
                        acc[k][2 * e] += __low2float(v2);
                        acc[k][2 * e + 1] += __high2float(v2);
                    }
                }
            }
            if (P.dqp) {
                const uint2 raw = *reinterpret_cast<const uint2*>(P.dqp_part + si * kHeadDim + lane * 4);
                const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
                const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
                pa0 += __low2float(lo);
                pa1 += __high2float(lo);
                pa2 += __low2float(hi);
                pa3 += __high2float(hi);
            }
        }
    }
#pragma unroll
    for (int k = 0; k < KITER; ++k) {
        const int ck = k * 32 + lane;
        if (ck < nchunk) {
            const int hh = ck >> 4, col = (ck & 15) * 8;
            uint4 o;
            o.x = pack_bf16(acc[k][0] * P.scale, acc[k][1] * P.scale);
            o.y = pack_bf16(acc[k][2] * P.scale, acc[k][3] * P.scale);
            o.z = pack_bf16(acc[k][4] * P.scale, acc[k][5] * P.scale);
            o.w = pack_bf16(acc[k][6] * P.scale, acc[k][7] * P.scale);
            *reinterpret_cast<uint4*>(P.dq + ((static_cast<int64_t>(b) * P.Hq + p * P.mpp + hh) * P.S + q) * kHeadDim + col) = o;
        }
    }
    if (P.dqp) {
        const float gk = (P.grad_kl ? *P.grad_kl : 1.f) * P.kl_out_scale;
        uint2 o;
        o.x = pack_bf16(pa0 * gk, pa1 * gk);
        o.y = pack_bf16(pa2 * gk, pa3 * gk);
        *reinterpret_cast<uint2*>(P.dqp + (bp * P.S + q) * kHeadDim + lane * 4) = o;
    }
}

// -------------------------------------------------------------------------------------------
// delta[b,h,q] = sum_d out[b,q,h,d] * dout[b,q,h,d]   (flash_msa/flash_msa.py:99)
// -------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) delta_kernel(const __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ dout,
                                                    int64_t do_sb, int64_t do_ss, int64_t do_sh, float* __restrict__ delta,
                                                    int B, int S, int Hq) {
    const int lane = threadIdx.x & 31;
    const int64_t w = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    if (w >= static_cast<int64_t>(B) * S * Hq) return;
    const int h = static_cast<int>(w % Hq);
    const int64_t bq = w / Hq;
    const int q = static_cast<int>(bq % S);
    const int b = static_cast<int>(bq / S);
    const uint2 a = *reinterpret_cast<const uint2*>(out + w * kHeadDim + lane * 4);
    const uint2 d = *reinterpret_cast<const uint2*>(dout + b * do_sb + q * do_ss + h * do_sh + lane * 4);
    const __nv_bfloat162 a0 = *reinterpret_cast<const __nv_bfloat162*>(&a.x), a1 = *reinterpret_cast<const __nv_bfloat162*>(&a.y);
    const __nv_bfloat162 d0 = *reinterpret_cast<const __nv_bfloat162*>(&d.x), d1 = *reinterpret_cast<const __nv_bfloat162*>(&d.y);
    float s = __low2float(a0) * __low2float(d0) + __high2float(a0) * __high2float(d0) + __low2float(a1) * __low2float(d1) +
              __high2float(a1) * __high2float(d1);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (lane == 0) delta[(static_cast<int64_t>(b) * Hq + h) * S + q] = s;
}

// dst = bf16(src * const_scale * factor), factor = *scale_ptr when given (the upstream kl gradient lives on the
// device: flash_msa/flash_msa.py:122-125) else 1.
__global__ void __launch_bounds__(256) cast_scaled_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int64_t n4,
                                                          const float* __restrict__ scale_ptr, float const_scale) {
    const float f = (scale_ptr ? *scale_ptr : 1.f) * const_scale;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const float4 v = reinterpret_cast<const float4*>(src)[i];
        uint2 o;
        o.x = pack_bf16(v.x * f, v.y * f);
        o.y = pack_bf16(v.z * f, v.w * f);
        reinterpret_cast<uint2*>(dst)[i] = o;
    }
}

}  // namespace
}  // namespace fmsa

extern "C" int fmsa_bwd_delta(const void* out, const fmsa_tensor* d_out, float* delta, int32_t B, int32_t S, int32_t Hq,
                              void* stream) {
    using namespace fmsa;
    FMSA_REQUIRE(out && d_out && d_out->ptr && delta && B > 0 && S > 0 && Hq > 0);
    FMSA_REQUIRE((reinterpret_cast<uintptr_t>(out) & 7u) == 0 && (reinterpret_cast<uintptr_t>(d_out->ptr) & 7u) == 0);
    FMSA_REQUIRE(d_out->stride_b % 4 == 0 && d_out->stride_h % 4 == 0 && d_out->stride_s % 4 == 0);
    const int64_t rows = static_cast<int64_t>(B) * S * Hq;
    const int64_t grid = (rows + 7) / 8;
    FMSA_REQUIRE(grid <= 0x7fffffffLL);
    delta_kernel<<<static_cast<unsigned>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(d_out->ptr), d_out->stride_b, d_out->stride_s,
        d_out->stride_h, delta, B, S, Hq);
    return check_launch();
}

extern "C" int fmsa_cast_scaled(const float* src, void* dst, int64_t n, const float* scale_ptr, float const_scale,
                                void* stream) {
    using namespace fmsa;
    FMSA_REQUIRE(src && dst && n >= 0 && n % 4 == 0);
    FMSA_REQUIRE(aligned16(src) && (reinterpret_cast<uintptr_t>(dst) & 7u) == 0);
    if (n == 0) return FMSA_OK;
    const int64_t n4 = n / 4;
    int64_t grid = (n4 + 255) / 256;
    if (grid > 148 * 16) grid = 148 * 16;
    cast_scaled_kernel<<<static_cast<unsigned>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        src, static_cast<__nv_bfloat16*>(dst), n4, scale_ptr, const_scale);
    return check_launch();
}

extern "C" int fmsa_sparse_bwd(const fmsa_problem* pb, const fmsa_tensor* q, const fmsa_tensor* k, const fmsa_tensor* v,
                               const fmsa_tensor* q_proxy, const fmsa_tensor* k_proxy, const fmsa_tensor* d_out,
                               const float* lse, const float* lse_proxy, const float* delta, const int32_t* row_ptr,
                               const int32_t* col_q, void* dq_part, void* dqp_part, int64_t part_slots, float* dkp_acc,
                               float* dk_acc, float* dv_acc, int32_t g_begin, int32_t g_count, int32_t with_kl,
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
    if (part_slots < fmsa_fwd_partial_slots(pb, g_count, dense)) return FMSA_ERR_WORKSPACE;
    FMSA_REQUIRE(tma_compatible(k->ptr, k->stride_b, k->stride_h, k->stride_s));
    FMSA_REQUIRE(tma_compatible(v->ptr, v->stride_b, v->stride_h, v->stride_s));
    FMSA_REQUIRE(tma_compatible(q->ptr, q->stride_b, q->stride_h, q->stride_s));
    FMSA_REQUIRE(tma_compatible(d_out->ptr, d_out->stride_b, d_out->stride_h, d_out->stride_s));
    if (with_kl) {
        FMSA_REQUIRE(tma_compatible(q_proxy->ptr, q_proxy->stride_b, q_proxy->stride_h, q_proxy->stride_s));
        FMSA_REQUIRE(tma_compatible(k_proxy->ptr, k_proxy->stride_b, k_proxy->stride_h, k_proxy->stride_s));
    }
    FMSA_REQUIRE(aligned16(dq_part) && aligned16(dk_acc) && aligned16(dv_acc) &&
                 (!with_kl || (aligned16(dqp_part) && aligned16(dkp_acc))));
    CUtensorMap tk, tv, tdq, tdqp;
    if (!make_tmap_bhsd(&tk, k->ptr, pb->B, pb->Hkv, pb->S, k->stride_b, k->stride_h, k->stride_s, 128) ||
        !make_tmap_bhsd(&tv, v->ptr, pb->B, pb->Hkv, pb->S, v->stride_b, v->stride_h, v->stride_s, 128) ||
        !make_tmap_partials(&tdq, dq_part, part_slots, pb->Hq / pb->Hp) ||
        !make_tmap_partials(&tdqp, with_kl ? dqp_part : dq_part, part_slots, 1))
        return FMSA_ERR_CUDA;

    BwdParams P;
    P.q = static_cast<const __nv_bfloat16*>(q->ptr);
    P.q_sb = q->stride_b; P.q_sh = q->stride_h; P.q_ss = q->stride_s;
    P.dout = static_cast<const __nv_bfloat16*>(d_out->ptr);
    P.do_sb = d_out->stride_b; P.do_sh = d_out->stride_h; P.do_ss = d_out->stride_s;
    if (with_kl) {
        P.qp = static_cast<const __nv_bfloat16*>(q_proxy->ptr);
        P.qp_sb = q_proxy->stride_b; P.qp_sh = q_proxy->stride_h; P.qp_ss = q_proxy->stride_s;
        P.kp = static_cast<const __nv_bfloat16*>(k_proxy->ptr);
        P.kp_sb = k_proxy->stride_b; P.kp_sh = k_proxy->stride_h; P.kp_ss = k_proxy->stride_s;
    } else {
        P.qp = P.q; P.qp_sb = P.qp_sh = P.qp_ss = 0;
        P.kp = P.q; P.kp_sb = P.kp_sh = P.kp_ss = 0;
    }
    P.lse = lse; P.lse_proxy = lse_proxy; P.delta = delta;
    P.row_ptr = row_ptr; P.col_q = col_q;
    P.dq_part = static_cast<__nv_bfloat16*>(dq_part); P.dqp_part = static_cast<__nv_bfloat16*>(dqp_part);
    P.dkp_acc = dkp_acc; P.dk_acc = dk_acc; P.dv_acc = dv_acc;
    P.counter = counter; P.status = status;
    P.S = pb->S; P.NB = pb->S / kBlock; P.Hq = pb->Hq; P.Hkv = pb->Hkv; P.Hp = pb->Hp; P.Hpkv = pb->Hpkv;
    P.mpp = pb->Hq / pb->Hp; P.ppk = pb->Hp / pb->Hkv; P.pg = pb->Hp / pb->Hpkv;
    P.g_begin = g_begin; P.G = g_count;
    P.with_kl = with_kl ? 1 : 0; P.dense = dense ? 1 : 0;
    P.scale = pb->scale; P.scale_log2e = pb->scale * kLog2e;
    P.kl_out_scale = pb->scale / (static_cast<float>(pb->B) * pb->Hp * pb->S);
    P.kl_value = with_kl ? kl_value : nullptr;
    P.kl_value_scale = kLn2 / (static_cast<float>(pb->B) * pb->Hp * pb->S);

    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return FMSA_ERR_CUDA;
    if (cudaFuncSetAttribute(sparse_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kBwdSmemBytes)) !=
        cudaSuccess)
        return FMSA_ERR_CUDA;
    if (cudaMemsetAsync(counter, 0, sizeof(int32_t), st) != cudaSuccess) return FMSA_ERR_CUDA;
    P.n_subunits = g_count * subunits_per_group(P.NB, P.ppk, kChunksPerSubUnit);
    FMSA_REQUIRE(P.n_subunits < 0x7fffffffLL);
    const int grid = static_cast<int>(P.n_subunits < sms ? P.n_subunits : sms);
    sparse_bwd_kernel<<<grid, kBwdThreads, kBwdSmemBytes, st>>>(tk, tv, tdq, tdqp, P);
    return check_launch();
}

extern "C" int fmsa_sparse_bwd_combine(const fmsa_problem* pb, const void* dq_part, const void* dqp_part,
                                       const int32_t* edge_pos, const int32_t* row_ptr, void* dq, void* dq_proxy,
                                       const float* grad_kl, int32_t g_begin, int32_t g_count, int32_t dense,
                                       void* stream) {
    using namespace fmsa;
    FMSA_REQUIRE(problem_ok(pb));
    FMSA_REQUIRE(dq_part && dq);
    FMSA_REQUIRE(dense || (edge_pos && row_ptr));
    FMSA_REQUIRE(!dq_proxy || dqp_part);
    FMSA_REQUIRE(g_begin >= 0 && g_count > 0 && g_begin + g_count <= pb->B * pb->Hkv);
    BwdCombineParams P;
    P.dq_part = static_cast<const __nv_bfloat16*>(dq_part); P.dqp_part = static_cast<const __nv_bfloat16*>(dqp_part);
    P.edge_pos = edge_pos; P.row_ptr = row_ptr;
    P.dq = static_cast<__nv_bfloat16*>(dq); P.dqp = static_cast<__nv_bfloat16*>(dq_proxy); P.grad_kl = grad_kl;
    P.S = pb->S; P.NB = pb->S / kBlock; P.Hq = pb->Hq; P.Hp = pb->Hp; P.mpp = pb->Hq / pb->Hp; P.ppk = pb->Hp / pb->Hkv;
    P.Kb = pb->top_k_blocks; P.g_begin = g_begin; P.G = g_count; P.dense = dense ? 1 : 0;
    P.scale = pb->scale;
    P.kl_out_scale = pb->scale / (static_cast<float>(pb->B) * pb->Hp * pb->S);
    const int64_t rows = static_cast<int64_t>(g_count) * P.ppk * P.S;
    const int64_t grid = (rows + 7) / 8;
    FMSA_REQUIRE(grid <= 0x7fffffffLL);
    const dim3 cg(static_cast<unsigned>(grid));
    cudaStream_t cst = static_cast<cudaStream_t>(stream);
    if (P.mpp <= 2)
        bwd_combine_wide_kernel<1><<<cg, 256, 0, cst>>>(P);
    else if (P.mpp <= 4)
        bwd_combine_wide_kernel<2><<<cg, 256, 0, cst>>>(P);
    else if (P.mpp <= 6)
        bwd_combine_wide_kernel<3><<<cg, 256, 0, cst>>>(P);
    else if (P.mpp <= 8)
        bwd_combine_wide_kernel<4><<<cg, 256, 0, cst>>>(P);
    else
        bwd_combine_kernel<<<static_cast<unsigned>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(P);
    return check_launch();
}
