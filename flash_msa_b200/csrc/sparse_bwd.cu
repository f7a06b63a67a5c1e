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
    float *dq_acc, *dqp_acc, *dkp_acc;      // fp32 [B,Hq,S,128], [B,Hp,S,128], [B,Hpkv,S,128], zero-initialised
    __nv_bfloat16 *dk, *dv;                 // [B,Hkv,S,128]
    int32_t* counter;
    int32_t* status;
    int S, NB, Hq, Hkv, Hp, Hpkv, mpp, ppk, pg;
    int units_g;     // number of (batch, KV head) groups
    int with_kl, dense;
    float scale, scale_log2e, kl_out_scale;   // kl_out_scale = scale / (B*Hp*S)
};

struct BwdSmem {
    uint64_t bar_kv, bar_a, bar_b;
    uint32_t tmem_slot;
    int32_t unit;
    int32_t rows[2][128];
};

constexpr int kBwdThreads = 256;
constexpr size_t kBwdSmemBytes = 6 * kTileBytes + 1024 + sizeof(BwdSmem);

__global__ void __launch_bounds__(kBwdThreads, 1) sparse_bwd_kernel(const __grid_constant__ CUtensorMap tmap_k,
                                                                    const __grid_constant__ CUtensorMap tmap_v,
                                                                    const BwdParams P) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t tile_k = tiles, tile_v = tiles + kTileBytes;
    const uint32_t tile_q = tiles + 2 * kTileBytes, tile_do = tiles + 3 * kTileBytes;
    const uint32_t tile_p = tiles + 4 * kTileBytes, tile_ds = tiles + 5 * kTileBytes;
    BwdSmem* sm = reinterpret_cast<BwdSmem*>(smem_raw + (tiles - smem_u32(smem_raw)) + 6 * kTileBytes);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quarter = warp & 3, half = warp >> 2;
    const int row = quarter * 32 + lane, c0 = half * 64;
    const uint32_t bar_kv = smem_u32(&sm->bar_kv), bar_a = smem_u32(&sm->bar_a), bar_b = smem_u32(&sm->bar_b);

    if (tid == 0) {
        mbar_init(bar_kv, 1);
        mbar_init(bar_a, 1);
        mbar_init(bar_b, 1);
        fence_mbar_init();
        prefetch_tmap(&tmap_k);
        prefetch_tmap(&tmap_v);
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(&sm->tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = sm->tmem_slot;
    const uint32_t t_s = tmem, t_dp = tmem + 128, t_dv = tmem + 256, t_dk = tmem + 384;

    const int hpc = P.mpp + (P.with_kl ? 1 : 0);
    const float inv_mpp = 1.f / static_cast<float>(P.mpp);
    uint32_t ph_kv = 0, ph_a = 0, ph_b = 0;
    bool bad = false;

    for (;;) {
        if (tid == 0) sm->unit = atomicAdd(P.counter, 1);
        __syncthreads();
        const int u = sm->unit;
        __syncthreads();
        if (u >= P.units_g * P.NB) break;
        const int j = u / P.units_g;
        const int g = u % P.units_g;
        const int b = g / P.Hkv, kvh = g % P.Hkv;
        if (tid == 0) {
            mbar_arrive_expect_tx(bar_kv, 2 * kTileBytes);
            tma_load_tile(tile_k, &tmap_k, j * kBlock, kvh, b, bar_kv);
            tma_load_tile(tile_v, &tmap_v, j * kBlock, kvh, b, bar_kv);
        }
        bool kv_ready = false;
        bool kv_acc = false;   // dK/dV accumulators hold something

        for (int pp = 0; pp < P.ppk; ++pp) {
            const int p = kvh * P.ppk + pp;
            const int kph = p / P.pg;
            const int64_t bp = static_cast<int64_t>(b) * P.Hp + p;
            int64_t e0 = 0;
            int n;
            if (P.dense) {
                n = P.S - j * kBlock;
            } else {
                e0 = P.row_ptr[bp * P.NB + j];
                n = P.row_ptr[bp * P.NB + j + 1] - static_cast<int>(e0);
            }
            if (n <= 0) continue;
            const int nchunks = (n + kBlock - 1) / kBlock;
            const int ntiles = nchunks * hpc;
            const __nv_bfloat16* q_b = P.q + static_cast<int64_t>(b) * P.q_sb;
            const __nv_bfloat16* do_b = P.dout + static_cast<int64_t>(b) * P.do_sb;
            const __nv_bfloat16* qp_bp = P.qp + static_cast<int64_t>(b) * P.qp_sb + static_cast<int64_t>(p) * P.qp_sh;
            const __nv_bfloat16* kp_blk = P.kp + static_cast<int64_t>(b) * P.kp_sb + static_cast<int64_t>(kph) * P.kp_sh +
                                          static_cast<int64_t>(j) * kBlock * P.kp_ss;

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
                if (hh < P.mpp) {
                    const int h = p * P.mpp + hh;
                    gather_tile_async<kBwdThreads>(tile_q, q_b + static_cast<int64_t>(h) * P.q_sh, P.q_ss, sm->rows[chunk & 1], tid);
                    gather_tile_async<kBwdThreads>(tile_do, do_b + static_cast<int64_t>(h) * P.do_sh, P.do_ss, sm->rows[chunk & 1], tid);
                } else {
                    gather_tile_async<kBwdThreads>(tile_q, qp_bp, P.qp_ss, sm->rows[chunk & 1], tid);
                    load_tile_async<kBwdThreads>(tile_do, kp_blk, P.kp_ss, tid);
                }
                cp_async_commit();
            };

            stage_rows(0);
            __syncthreads();
            issue_gather(0);

            float teacher[64];
#pragma unroll
            for (int i = 0; i < 64; ++i) teacher[i] = 0.f;

            for (int t = 0; t < ntiles; ++t) {
                const int chunk = t / hpc, hh = t % hpc;
                const bool is_proxy = hh == P.mpp;
                const int qid = sm->rows[chunk & 1][row];
                const bool live = qid >= 0;
                const int limit = (live && (qid >> 7) == j) ? (qid & 127) : 127;
                // per-row statistics: issue the loads before waiting on anything
                float row_lse = 0.f, row_delta = 0.f;
                if (live) {
                    if (is_proxy) {
                        row_lse = P.lse_proxy[bp * P.S + qid];
                    } else {
                        const int64_t at = (static_cast<int64_t>(b) * P.Hq + p * P.mpp + hh) * P.S + qid;
                        row_lse = P.lse[at];
                        row_delta = P.delta[at];
                    }
                }
                cp_async_wait<0>();
                fence_async_smem();
                __syncthreads();
                if (tid == 0) {
                    if (!kv_ready) bad |= !mbar_wait(bar_kv, ph_kv);
                    tc_fence_after_sync();
                    if (is_proxy) {
                        umma_tile_128<false, false>(t_s, tile_q, tile_do, false);           // Sp = Qp_g Kp_j^T
                    } else {
                        umma_tile_128<false, false>(t_s, tile_q, tile_k, false);            // S  = Q_g K_j^T
                        umma_tile_128<false, false>(t_dp, tile_do, tile_v, false);          // dP = dO_g V_j^T
                    }
                    umma_commit(bar_a);
                }
                if (!kv_ready) {
                    kv_ready = true;
                    ph_kv ^= 1;
                }
                bad |= !mbar_wait(bar_a, ph_a);
                ph_a ^= 1;
                if (__syncthreads_or(bad)) {
                    bad = true;
                    goto abort;
                }
                tc_fence_after_sync();

                const float neg_lse = -row_lse * kLog2e;
                if (!is_proxy) {
#pragma unroll
                    for (int c = 0; c < 64; c += 32) {
                        uint32_t sv[32], dv[32];
                        tmem_ld32(tmem_addr(t_s, quarter, c0 + c), sv);
                        tmem_ld32(tmem_addr(t_dp, quarter, c0 + c), dv);
                        tmem_ld_wait();
                        uint32_t pk[16], dk[16];
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            float p0 = fast_exp2(fmaf(__uint_as_float(sv[i]), P.scale_log2e, neg_lse));
                            float p1 = fast_exp2(fmaf(__uint_as_float(sv[i + 1]), P.scale_log2e, neg_lse));
                            p0 = (live && c0 + c + i <= limit) ? p0 : 0.f;
                            p1 = (live && c0 + c + i + 1 <= limit) ? p1 : 0.f;
                            const float d0 = p0 * (__uint_as_float(dv[i]) - row_delta);
                            const float d1 = p1 * (__uint_as_float(dv[i + 1]) - row_delta);
                            const __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
                            pk[i >> 1] = *reinterpret_cast<const uint32_t*>(&pb);
                            dk[i >> 1] = pack_bf16(d0, d1);
                            if (P.with_kl) {
                                teacher[c + i] += __low2float(pb);
                                teacher[c + i + 1] += __high2float(pb);
                            }
                        }
#pragma unroll
                        for (int k8 = 0; k8 < 4; ++k8) {
                            const uint32_t off = swz_offset(row, ((c0 + c) >> 3) + k8);
                            st_shared_v4(tile_p + off, pk[4 * k8], pk[4 * k8 + 1], pk[4 * k8 + 2], pk[4 * k8 + 3]);
                            st_shared_v4(tile_ds + off, dk[4 * k8], dk[4 * k8 + 1], dk[4 * k8 + 2], dk[4 * k8 + 3]);
                        }
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < 64; c += 32) {
                        uint32_t sv[32];
                        tmem_ld32(tmem_addr(t_s, quarter, c0 + c), sv);
                        tmem_ld_wait();
                        uint32_t dk[16];
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            float p0 = fast_exp2(fmaf(__uint_as_float(sv[i]), P.scale_log2e, neg_lse));
                            float p1 = fast_exp2(fmaf(__uint_as_float(sv[i + 1]), P.scale_log2e, neg_lse));
                            p0 = (live && c0 + c + i <= limit) ? p0 : 0.f;
                            p1 = (live && c0 + c + i + 1 <= limit) ? p1 : 0.f;
                            dk[i >> 1] = pack_bf16(p0 - teacher[c + i] * inv_mpp, p1 - teacher[c + i + 1] * inv_mpp);
                            teacher[c + i] = 0.f;
                            teacher[c + i + 1] = 0.f;
                        }
#pragma unroll
                        for (int k8 = 0; k8 < 4; ++k8)
                            st_shared_v4(tile_ds + swz_offset(row, ((c0 + c) >> 3) + k8), dk[4 * k8], dk[4 * k8 + 1],
                                         dk[4 * k8 + 2], dk[4 * k8 + 3]);
                    }
                }
                fence_async_smem();
                tc_fence_before_sync();
                __syncthreads();
                if (tid == 0) {
                    tc_fence_after_sync();
                    if (is_proxy) {
                        umma_tile_128<false, true>(t_s, tile_ds, tile_do, false);    // dQp = dSp Kp_j
                        umma_tile_128<true, true>(t_dp, tile_ds, tile_q, false);     // dKp = dSp^T Qp_g
                    } else {
                        umma_tile_128<true, true>(t_dv, tile_p, tile_do, kv_acc);    // dV += P^T dO_g
                        umma_tile_128<true, true>(t_dk, tile_ds, tile_q, kv_acc);    // dK += dS^T Q_g
                        umma_tile_128<false, true>(t_s, tile_ds, tile_k, false);     // dQ  = dS K_j
                    }
                    umma_commit(bar_b);
                }
                if (!is_proxy) kv_acc = true;
                bad |= !mbar_wait(bar_b, ph_b);
                ph_b ^= 1;
                if (__syncthreads_or(bad)) {
                    bad = true;
                    goto abort;
                }
                tc_fence_after_sync();
                // the operand tiles are free again: start fetching the next tile
                if (t + 1 < ntiles) {
                    const int nchunk = (t + 1) / hpc;
                    if (nchunk != chunk) {
                        stage_rows(nchunk);
                        __syncthreads();
                    }
                    issue_gather(t + 1);
                }
                // epilogue: reduce dQ (or dQp and dKp) into the fp32 buffers
                {
                    const float osc = is_proxy ? P.kl_out_scale : P.scale;
                    float* dst = nullptr;
                    if (live) {
                        dst = is_proxy ? P.dqp_acc + (bp * P.S + qid) * kHeadDim
                                       : P.dq_acc + ((static_cast<int64_t>(b) * P.Hq + p * P.mpp + hh) * P.S + qid) * kHeadDim;
                    }
#pragma unroll 1
                    for (int c = 0; c < 64; c += 32) {
                        uint32_t v[32];
                        tmem_ld32(tmem_addr(t_s, quarter, c0 + c), v);
                        tmem_ld_wait();
                        if (live) {
#pragma unroll
                            for (int i = 0; i < 32; i += 4)
                                red_add_v4(dst + c0 + c + i, __uint_as_float(v[i]) * osc, __uint_as_float(v[i + 1]) * osc,
                                           __uint_as_float(v[i + 2]) * osc, __uint_as_float(v[i + 3]) * osc);
                        }
                    }
                    if (is_proxy) {
                        float* kdst = P.dkp_acc + ((static_cast<int64_t>(b) * P.Hpkv + kph) * P.S + j * kBlock + row) * kHeadDim;
#pragma unroll 1
                        for (int c = 0; c < 64; c += 32) {
                            uint32_t v[32];
                            tmem_ld32(tmem_addr(t_dp, quarter, c0 + c), v);
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 32; i += 4)
                                red_add_v4(kdst + c0 + c + i, __uint_as_float(v[i]) * osc, __uint_as_float(v[i + 1]) * osc,
                                           __uint_as_float(v[i + 2]) * osc, __uint_as_float(v[i + 3]) * osc);
                        }
                    }
                }
                tc_fence_before_sync();
            }
            __syncthreads();
        }
        if (!kv_ready) {
            if (tid == 0) bad |= !mbar_wait(bar_kv, ph_kv);
            ph_kv ^= 1;
            if (__syncthreads_or(bad)) {
                bad = true;
                goto abort;
            }
        }
        // unit epilogue: the unit owns dK_j and dV_j
        {
            tc_fence_after_sync();
            const int64_t at = ((static_cast<int64_t>(b) * P.Hkv + kvh) * P.S + j * kBlock + row) * kHeadDim + c0;
#pragma unroll 1
            for (int which = 0; which < 2; ++which) {
                __nv_bfloat16* dst = (which == 0 ? P.dv : P.dk) + at;
                const float osc = which == 0 ? 1.f : P.scale;
#pragma unroll 1
                for (int c = 0; c < 64; c += 32) {
                    uint32_t v[32];
                    if (kv_acc) {
                        tmem_ld32(tmem_addr(which == 0 ? t_dv : t_dk, quarter, c0 + c), v);
                        tmem_ld_wait();
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = 0u;
                    }
#pragma unroll
                    for (int k8 = 0; k8 < 4; ++k8) {
                        uint4 w;
                        w.x = pack_bf16(__uint_as_float(v[8 * k8 + 0]) * osc, __uint_as_float(v[8 * k8 + 1]) * osc);
                        w.y = pack_bf16(__uint_as_float(v[8 * k8 + 2]) * osc, __uint_as_float(v[8 * k8 + 3]) * osc);
                        w.z = pack_bf16(__uint_as_float(v[8 * k8 + 4]) * osc, __uint_as_float(v[8 * k8 + 5]) * osc);
                        w.w = pack_bf16(__uint_as_float(v[8 * k8 + 6]) * osc, __uint_as_float(v[8 * k8 + 7]) * osc);
                        *reinterpret_cast<uint4*>(dst + c + 8 * k8) = w;
                    }
                }
            }
            tc_fence_before_sync();
            __syncthreads();
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

// dst = bf16(src * factor), factor = *scale_ptr when given (the upstream kl gradient lives on the
// device: flash_msa/flash_msa.py:122-125) else 1.
__global__ void __launch_bounds__(256) cast_scaled_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int64_t n4,
                                                          const float* __restrict__ scale_ptr) {
    const float f = scale_ptr ? *scale_ptr : 1.f;
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

extern "C" int fmsa_cast_scaled(const float* src, void* dst, int64_t n, const float* scale_ptr, void* stream) {
    using namespace fmsa;
    FMSA_REQUIRE(src && dst && n >= 0 && n % 4 == 0);
    FMSA_REQUIRE(aligned16(src) && (reinterpret_cast<uintptr_t>(dst) & 7u) == 0);
    if (n == 0) return FMSA_OK;
    const int64_t n4 = n / 4;
    int64_t grid = (n4 + 255) / 256;
    if (grid > 148 * 16) grid = 148 * 16;
    cast_scaled_kernel<<<static_cast<unsigned>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        src, static_cast<__nv_bfloat16*>(dst), n4, scale_ptr);
    return check_launch();
}

extern "C" int fmsa_sparse_bwd(const fmsa_problem* pb, const fmsa_tensor* q, const fmsa_tensor* k, const fmsa_tensor* v,
                               const fmsa_tensor* q_proxy, const fmsa_tensor* k_proxy, const fmsa_tensor* d_out,
                               const float* lse, const float* lse_proxy, const float* delta, const int32_t* row_ptr,
                               const int32_t* col_q, float* dq_acc, float* dqp_acc, float* dkp_acc, void* dk, void* dv,
                               int32_t with_kl, int32_t dense, int32_t* counter, int32_t* status, void* stream) {
    using namespace fmsa;
    FMSA_REQUIRE(problem_ok(pb));
    FMSA_REQUIRE(q && k && v && d_out && q->ptr && k->ptr && v->ptr && d_out->ptr);
    FMSA_REQUIRE(lse && delta && dq_acc && dk && dv && counter && status);
    FMSA_REQUIRE(dense || (row_ptr && col_q));
    FMSA_REQUIRE(!with_kl || (q_proxy && k_proxy && q_proxy->ptr && k_proxy->ptr && lse_proxy && dqp_acc && dkp_acc));
    FMSA_REQUIRE(pb->scale > 0.f);
    FMSA_REQUIRE(tma_compatible(k->ptr, k->stride_b, k->stride_h, k->stride_s));
    FMSA_REQUIRE(tma_compatible(v->ptr, v->stride_b, v->stride_h, v->stride_s));
    FMSA_REQUIRE(tma_compatible(q->ptr, q->stride_b, q->stride_h, q->stride_s));
    FMSA_REQUIRE(tma_compatible(d_out->ptr, d_out->stride_b, d_out->stride_h, d_out->stride_s));
    if (with_kl) {
        FMSA_REQUIRE(tma_compatible(q_proxy->ptr, q_proxy->stride_b, q_proxy->stride_h, q_proxy->stride_s));
        FMSA_REQUIRE(tma_compatible(k_proxy->ptr, k_proxy->stride_b, k_proxy->stride_h, k_proxy->stride_s));
    }
    FMSA_REQUIRE(aligned16(dq_acc) && aligned16(dk) && aligned16(dv) && (!with_kl || (aligned16(dqp_acc) && aligned16(dkp_acc))));
    CUtensorMap tk, tv;
    if (!make_tmap_bhsd(&tk, k->ptr, pb->B, pb->Hkv, pb->S, k->stride_b, k->stride_h, k->stride_s, 128) ||
        !make_tmap_bhsd(&tv, v->ptr, pb->B, pb->Hkv, pb->S, v->stride_b, v->stride_h, v->stride_s, 128))
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
    P.dq_acc = dq_acc; P.dqp_acc = dqp_acc; P.dkp_acc = dkp_acc;
    P.dk = static_cast<__nv_bfloat16*>(dk); P.dv = static_cast<__nv_bfloat16*>(dv);
    P.counter = counter; P.status = status;
    P.S = pb->S; P.NB = pb->S / kBlock; P.Hq = pb->Hq; P.Hkv = pb->Hkv; P.Hp = pb->Hp; P.Hpkv = pb->Hpkv;
    P.mpp = pb->Hq / pb->Hp; P.ppk = pb->Hp / pb->Hkv; P.pg = pb->Hp / pb->Hpkv;
    P.units_g = pb->B * pb->Hkv;
    P.with_kl = with_kl ? 1 : 0; P.dense = dense ? 1 : 0;
    P.scale = pb->scale; P.scale_log2e = pb->scale * kLog2e;
    P.kl_out_scale = pb->scale / (static_cast<float>(pb->B) * pb->Hp * pb->S);

    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return FMSA_ERR_CUDA;
    if (cudaFuncSetAttribute(sparse_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kBwdSmemBytes)) !=
        cudaSuccess)
        return FMSA_ERR_CUDA;
    if (cudaMemsetAsync(counter, 0, sizeof(int32_t), st) != cudaSuccess) return FMSA_ERR_CUDA;
    const int64_t units = static_cast<int64_t>(P.units_g) * P.NB;
    const int grid = static_cast<int>(units < sms ? units : sms);
    sparse_bwd_kernel<<<grid, kBwdThreads, kBwdSmemBytes, st>>>(tk, tv, P);
    return check_launch();
}
