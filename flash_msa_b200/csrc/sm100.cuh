// Blackwell (sm_100a) device primitives shared by every tensor-core kernel of the library:
// mbarriers with bounded waits, tensor-memory (TMEM) allocation, tcgen05.mma issue with
// shared-memory matrix descriptors, TMEM loads, cp.async row gathers into the 128-byte
// swizzled operand layout, and TMA tile loads.
//
// Operand tile convention used everywhere: a tile is 128 rows x 128 bf16 columns, stored as two
// "panels" of 64 columns.  Panel p starts at byte p*16384; row r of a panel starts at r*128;
// the 16-byte chunk c (0..7) of that row sits at chunk position c ^ (r & 7)  (the SWIZZLE_128B
// pattern, tile base 1024-byte aligned).  The same bytes serve
//   * as a K-major operand   (rows = M or N index, columns = reduction index), and
//   * as an MN-major operand (rows = reduction index, columns = M or N index),
// which is what lets one gathered Q tile feed both S = Q K^T and dK = dS^T Q.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fmsa {

constexpr int kBlock = 128;              // tokens per key / query block
constexpr int kHeadDim = 128;            // head dimension (fixed by the reference: flash_msa.py:54-55)
constexpr int kTileBytes = 128 * 128 * 2;
constexpr int kPanelBytes = 128 * 64 * 2;
constexpr unsigned kParkNs = 20000;      // suspend-time hint of a parked barrier wait
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// Status words written by kernels into the caller's status buffer (0 = ok).
constexpr int kStatusWaitTimeout = 1;    // a bounded mbarrier wait gave up
constexpr int kStatusBadIndex = 2;       // an index read from metadata was out of range

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// try_wait with a suspend-time hint: the thread is parked by the hardware until the phase completes or
// about `hint_ns` have passed, instead of spinning.  (Spinning pollers were measured to execute a third
// of all instructions of the attention kernels, which are bound by instruction issue.)
__device__ __forceinline__ bool mbar_try_wait_parked(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit_ns` of wall time (about two seconds by default) and returns false.
// The polling loop is kept out of line: the warp-specialised kernels have dozens of wait sites, and
// their code has to stay small enough for the instruction cache (several roles run different code
// at the same time, and a kernel much above 100 KB was measured to run several times slower).
constexpr uint64_t kWaitLimitNs = 2000000000ull;
static __device__ __noinline__ bool mbar_wait_poll(uint32_t bar, uint32_t parity, uint64_t limit_ns) {
    const uint64_t t0 = global_timer_ns();
    for (;;) {
        if (mbar_try_wait_parked(bar, parity, kParkNs)) return true;
        if (global_timer_ns() - t0 > limit_ns) return false;
    }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint64_t limit_ns = kWaitLimitNs) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_poll(bar, parity, limit_ns);
}
// (Inlined: a kernel that re-divides its registers between warpgroups with setmaxnreg cannot make calls.)
// Variant for kernels whose roles run decoupled: `abort_flag` is a word in shared memory that any thread sets
// when one of its waits ran out.  Every other waiter sees it within one parking period and gives up as well,
// so the whole CTA leaves its loops together instead of each role waiting out its own limit in turn.
static __device__ __forceinline__ bool mbar_wait_poll_abortable(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    // Kept as small as possible: this loop is inlined at every wait site of the warp-specialised kernels, whose
    // code has to fit the instruction cache.  The clock and the abort flag are looked at once per 64 parked tries
    // (a parked try returns after kParkNs at the latest), the time limit is counted in such rounds.
    uint32_t tries = 0;
    uint64_t t0 = 0;
    for (;;) {
        if (mbar_try_wait_parked(bar, parity, kParkNs)) return true;
        if ((++tries & 63u) != 0) continue;
        if (*abort_flag) return false;
        const uint64_t now = global_timer_ns();
        if (t0 == 0) t0 = now;
        if (now - t0 > kWaitLimitNs) {
            *abort_flag = 1;
            return false;
        }
    }
}
__device__ __forceinline__ bool mbar_wait_abortable(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_poll_abortable(bar, parity, abort_flag);
}

// Re-division of the register file between the warpgroups of a CTA (all four warps of a warpgroup execute it).
template <int N>
__device__ __forceinline__ void reg_dec() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_inc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}

// ---------------------------------------------------------------------------------------------
// proxy / tcgen05 fences
// ---------------------------------------------------------------------------------------------
// Makes shared-memory writes done with ordinary stores or cp.async visible to the async proxy
// (tcgen05.mma and TMA read shared memory through it).
__device__ __forceinline__ void fence_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// TMEM allocation (one full warp executes these)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// ---------------------------------------------------------------------------------------------
// tcgen05.mma (kind::f16: bf16 x bf16 -> fp32 in TMEM), M = 128, one CTA
// ---------------------------------------------------------------------------------------------
// Instruction descriptor: D fp32, A/B bf16 (or fp16: format code 0 instead of 1), M = 128, N = n; a_mn / b_mn
// select MN-major operands.
__host__ __device__ constexpr uint32_t umma_idesc(int n, bool a_mn, bool b_mn, bool fp16 = false) {
    return (1u << 4) | ((fp16 ? 0u : 1u) << 7) | ((fp16 ? 0u : 1u) << 10) | ((a_mn ? 1u : 0u) << 15) |
           ((b_mn ? 1u : 0u) << 16) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
}

// Shared-memory matrix descriptor, SWIZZLE_128B, descriptor version 1.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu) | (static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16) |
           (static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) | (2ull << 61);
}
// Descriptor of reduction step `ks` (16 reduction elements each, 8 steps per 128) of a tile used
// K-major (rows are the M/N index).  Eight-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile, int ks) {
    return umma_desc(tile + (ks >> 2) * kPanelBytes + (ks & 3) * 32, 16, 1024);
}
// Same tile used MN-major (rows are the reduction index): a step is 16 rows = 2048 bytes; the two
// 64-column halves of the M/N extent are one panel (16384 bytes) apart.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile, int ks) {
    return umma_desc(tile + ks * 2048, kPanelBytes, 1024);
}

// `elect` != 0 selects the lane that really issues.  The predicate sits inside the instruction so
// that a whole warp can run the issue sequence without diverging: a lone lane that branches away
// from its warp after a block barrier was measured to be scheduled thousands of cycles late.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate, uint32_t elect = 1u) {
    asm volatile(
        "{\n"
        ".reg .pred p, q;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "setp.ne.b32 q, %5, 0;\n"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(elect)
        : "memory");
}
// Arrives once on `bar` when every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar, uint32_t elect = 1u) {
    asm volatile(
        "{\n"
        ".reg .pred q;\n"
        "setp.ne.b32 q, %1, 0;\n"
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
        "}\n" ::"r"(bar),
        "r"(elect)
        : "memory");
}

// One full 128x128x128 product D (+)= A * B^T issued by the calling thread (8 instructions).
// The descriptors of the eight reduction steps differ from the first one only in the 14-bit
// address field (a tile lies below 256 KB, so the field never carries): K-major steps advance by
// 32 bytes inside a panel and jump to the second panel after four steps; MN-major steps advance
// by 16 rows = 2048 bytes.  Adding the encoded step to the low word keeps the issue loop at a few
// instructions per MMA, which matters because a single thread feeds the tensor core.
__host__ __device__ constexpr uint32_t umma_kstep(bool mn_major, int ks) {
    return mn_major ? static_cast<uint32_t>(ks) * (2048u >> 4)
                    : static_cast<uint32_t>(ks >> 2) * (kPanelBytes >> 4) + static_cast<uint32_t>(ks & 3) * 2u;
}
// The eight instructions sit in ONE asm block (two predicate set-ups and two 64-bit adds per step with
// immediate step sizes), so the issuing warp spends as few issue slots per MMA as possible.
template <bool A_MN, bool B_MN, bool FP16 = false>
__device__ __forceinline__ void umma_tile_128(uint32_t d_tmem, uint32_t a_tile, uint32_t b_tile, bool accumulate,
                                              uint32_t elect = 1u) {
    constexpr uint32_t idesc = umma_idesc(128, A_MN, B_MN, FP16);
    const uint64_t a0 = A_MN ? desc_mnmajor(a_tile, 0) : desc_kmajor(a_tile, 0);
    const uint64_t b0 = B_MN ? desc_mnmajor(b_tile, 0) : desc_kmajor(b_tile, 0);
#define FMSA_UMMA_STEP(AI, BI)                                                  \
    "add.s64 a, %1, " #AI ";\n"                                                 \
    "add.s64 b, %2, " #BI ";\n"                                                 \
    "@q tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, t;\n"
    asm volatile(
        "{\n"
        ".reg .pred p, q, t;\n"
        ".reg .b64 a, b;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "setp.ne.b32 q, %5, 0;\n"
        "setp.eq.b32 t, %5, %5;\n"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        FMSA_UMMA_STEP(%6, %13) FMSA_UMMA_STEP(%7, %14) FMSA_UMMA_STEP(%8, %15) FMSA_UMMA_STEP(%9, %16)
        FMSA_UMMA_STEP(%10, %17) FMSA_UMMA_STEP(%11, %18) FMSA_UMMA_STEP(%12, %19)
        "}\n" ::"r"(d_tmem),
        "l"(a0), "l"(b0), "r"(idesc), "r"(accumulate ? 1u : 0u), "r"(elect),
        "n"(umma_kstep(A_MN, 1)), "n"(umma_kstep(A_MN, 2)), "n"(umma_kstep(A_MN, 3)), "n"(umma_kstep(A_MN, 4)),
        "n"(umma_kstep(A_MN, 5)), "n"(umma_kstep(A_MN, 6)), "n"(umma_kstep(A_MN, 7)),
        "n"(umma_kstep(B_MN, 1)), "n"(umma_kstep(B_MN, 2)), "n"(umma_kstep(B_MN, 3)), "n"(umma_kstep(B_MN, 4)),
        "n"(umma_kstep(B_MN, 5)), "n"(umma_kstep(B_MN, 6)), "n"(umma_kstep(B_MN, 7))
        : "memory");
#undef FMSA_UMMA_STEP
}

// ---------------------------------------------------------------------------------------------
// TMEM loads: warp w of a warpgroup reads lanes 32*(w%4)..+31; thread i gets lane 32*(w%4)+i
// and 32 consecutive fp32 columns.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// TMEM address of (lane quarter of this warp, column).
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, int warp_in_group, int col) {
    return base + (static_cast<uint32_t>(warp_in_group * 32) << 16) + static_cast<uint32_t>(col);
}

// TMEM stores: the mirror image of the loads above (thread i of warp w writes lane 32*(w%4)+i).
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(r[0]),
                 "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// tcgen05.mma with the A operand in TMEM ("TS" form): D[128 x 128] (+)= A[128 x 128] * B^T.
// A is a 128 x 128 bf16 matrix whose row m lives in TMEM lane m; a 32-bit column holds the two
// consecutive reduction elements (2c, 2c+1), the even one in the low half, so the whole operand
// takes 64 columns and one instruction (16 reduction elements) reads 8 of them.  The operand may
// be split: `a_lo` is the TMEM address of reduction elements 0..63 (32 columns), `a_hi` that of
// elements 64..127.  B is a shared-memory tile as in umma_tile_128.
// ---------------------------------------------------------------------------------------------
template <bool B_MN, bool FP16 = false>
__device__ __forceinline__ void umma_tile_128_ts(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_tile,
                                                 bool accumulate, uint32_t elect = 1u) {
    constexpr uint32_t idesc = umma_idesc(128, false, B_MN, FP16);
    const uint64_t b0 = B_MN ? desc_mnmajor(b_tile, 0) : desc_kmajor(b_tile, 0);
#define FMSA_UMMA_TS_STEP(AREG, AOFF, BI)                                       \
    "add.u32 a, " #AREG ", " #AOFF ";\n"                                        \
    "add.s64 b, %3, " #BI ";\n"                                                 \
    "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %4, t;\n"
    asm volatile(
        "{\n"
        ".reg .pred p, q, t;\n"
        ".reg .b64 b;\n"
        ".reg .b32 a;\n"
        "setp.ne.b32 p, %5, 0;\n"
        "setp.ne.b32 q, %6, 0;\n"
        "setp.eq.b32 t, %6, %6;\n"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %3, %4, p;\n"
        FMSA_UMMA_TS_STEP(%1, 8, %7) FMSA_UMMA_TS_STEP(%1, 16, %8) FMSA_UMMA_TS_STEP(%1, 24, %9)
        FMSA_UMMA_TS_STEP(%2, 0, %10) FMSA_UMMA_TS_STEP(%2, 8, %11) FMSA_UMMA_TS_STEP(%2, 16, %12)
        FMSA_UMMA_TS_STEP(%2, 24, %13)
        "}\n" ::"r"(d_tmem),
        "r"(a_lo), "r"(a_hi), "l"(b0), "r"(idesc), "r"(accumulate ? 1u : 0u), "r"(elect),
        "n"(umma_kstep(B_MN, 1)), "n"(umma_kstep(B_MN, 2)), "n"(umma_kstep(B_MN, 3)), "n"(umma_kstep(B_MN, 4)),
        "n"(umma_kstep(B_MN, 5)), "n"(umma_kstep(B_MN, 6)), "n"(umma_kstep(B_MN, 7))
        : "memory");
#undef FMSA_UMMA_TS_STEP
}

// ---------------------------------------------------------------------------------------------
// cp.async row gather into a swizzled tile
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;   // src-size 0 writes 16 zero bytes
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ uint32_t swz_offset(int row, int chunk16) {
    // chunk16: 16-byte chunk index 0..15 within the 256-byte row
    return static_cast<uint32_t>((chunk16 >> 3) * kPanelBytes + row * 128 + (((chunk16 & 7) ^ (row & 7)) << 4));
}

// Every thread of the CTA calls this.  Row r of the tile is copied from `base + rows[r]*stride`
// (elements); a negative row id produces a row of zeros.  `rows` may live in shared memory.
template <int NTHREADS>
__device__ __forceinline__ void gather_tile_async(uint32_t tile, const __nv_bfloat16* base, int64_t stride,
                                                  const int* rows, int tid) {
#pragma unroll 4
    for (int it = tid; it < 128 * 16; it += NTHREADS) {
        const int r = it >> 4, c16 = it & 15;
        const int row = rows[r];
        const bool ok = row >= 0;
        const __nv_bfloat16* src = base + static_cast<int64_t>(ok ? row : 0) * stride + c16 * 8;
        cp_async_16(tile + swz_offset(r, c16), src, ok);
    }
}
// Contiguous variant: tile row r comes from `base + (row0 + r)*stride`.
template <int NTHREADS>
__device__ __forceinline__ void load_tile_async(uint32_t tile, const __nv_bfloat16* base, int64_t stride, int tid) {
#pragma unroll 4
    for (int it = tid; it < 128 * 16; it += NTHREADS) {
        const int r = it >> 4, c16 = it & 15;
        cp_async_16(tile + swz_offset(r, c16), base + static_cast<int64_t>(r) * stride + c16 * 8, true);
    }
}

// Lean 512-thread variants used by the attention kernels.  Thread `tid` always moves the same
// 16-byte chunk column of rows tid/16 + 32k (k = 0..3), so its swizzled destination offset is a
// per-thread constant plus k * 4096 bytes; only the source row changes.
struct GatherLane {
    uint32_t dst_off;   // swizzled offset of (row tid/16, chunk tid%16) inside a tile
    int r0;             // tid / 16
    int col;            // element offset of the chunk inside the 128-element row
};
__device__ __forceinline__ GatherLane make_gather_lane(int tid) {
    GatherLane g;
    g.r0 = tid >> 4;
    g.col = (tid & 15) * 8;
    g.dst_off = swz_offset(g.r0, tid & 15);
    return g;
}
__device__ __forceinline__ void gather_tile_512(uint32_t tile, const __nv_bfloat16* base, int64_t stride, const int* rows,
                                                const GatherLane& g) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int row = rows[g.r0 + 32 * k];
        const bool ok = row >= 0;
        cp_async_16(tile + g.dst_off + k * 4096, base + static_cast<int64_t>(ok ? row : 0) * stride + g.col, ok);
    }
}
__device__ __forceinline__ void load_tile_512(uint32_t tile, const __nv_bfloat16* base, int64_t stride, const GatherLane& g) {
#pragma unroll
    for (int k = 0; k < 4; ++k)
        cp_async_16(tile + g.dst_off + k * 4096, base + static_cast<int64_t>(g.r0 + 32 * k) * stride + g.col, true);
}

// ---------------------------------------------------------------------------------------------
// TMA: 2-D tile load (64 columns x 128 rows box, SWIZZLE_128B) signalled on an mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(tmap), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

// 4-D variant for (B, H, S, 128) activations: coordinates {column, s, h, b}.
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void* tmap, int x, int s, int h, int b, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
        "l"(tmap), "r"(x), "r"(s), "r"(h), "r"(b), "r"(bar)
        : "memory");
}
// Loads the 128-row tile starting at sequence position s0 of (b, h) as two 64-column panels.
// The caller has already posted expect_tx(kTileBytes) on `bar`.
__device__ __forceinline__ void tma_load_tile(uint32_t tile, const void* tmap, int s0, int h, int b, uint32_t bar) {
    tma_load_4d(tile, tmap, 0, s0, h, b, bar);
    tma_load_4d(tile + kPanelBytes, tmap, 64, s0, h, b, bar);
}
// TMA row gather: four rows r0..r3 of a 2-D bf16 matrix (tensor map with a 64-column x 1-row box, 128-byte
// swizzle), 64 columns starting at `col`, land as four consecutive 128-byte rows at `dst`.  `dst` must be
// 512-byte aligned inside a 1024-byte aligned tile so that the swizzle pattern matches the operand layout.
// A row index outside the matrix yields a row of zeros.  Completes 512 bytes on `bar`.
__device__ __forceinline__ void tma_gather4(uint32_t dst, const void* tmap, int col, int r0, int r1, int r2, int r3,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3, %4, %5, %6}], [%7];" ::"r"(dst),
        "l"(tmap), "r"(col), "r"(r0), "r"(r1), "r"(r2), "r"(r3), "r"(bar)
        : "memory");
}
// TMA tile STORE shared -> global (bulk-group completion).  The source tile must have been made
// visible to the async proxy (fence_async_smem + a barrier) before the elected thread issues it.
__device__ __forceinline__ void tma_store_2d(const void* tmap, uint32_t src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(tmap), "r"(src), "r"(x),
                 "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tma_store_3d(const void* tmap, uint32_t src, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(tmap), "r"(src),
                 "r"(x), "r"(y), "r"(z)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until the bulk stores committed so far have finished READING shared memory.
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// Waits until they are complete (globally visible at kernel end anyway; used before exit).
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void named_barrier_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

__device__ __forceinline__ void prefetch_tmap(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ---------------------------------------------------------------------------------------------
// small math helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float fast_log2(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Packed fp32 pairs (sm_100 executes fma/add/mul on two floats per instruction) and 3-input max:
// they halve the instruction count of the element-wise softmax / dS arithmetic, which is issue bound.
// The compiler's own float2 built-ins are used so that it can keep the pairs in adjacent registers
// (inline asm on 64-bit operands costs extra moves around every instruction).
__device__ __forceinline__ float2 f2_fma(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 f2_add(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 f2_mul(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 f2_from_bits(uint32_t lo, uint32_t hi) { return make_float2(__uint_as_float(lo), __uint_as_float(hi)); }
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// The same for the activation type of a kernel instantiation: bf16 (FP16 = false) or fp16.  A packed pair sits in
// one 32-bit word, the first element in the low half.
template <bool FP16>
__device__ __forceinline__ uint32_t pack_act(float lo, float hi) {
    if (FP16) {
        __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
    return pack_bf16(lo, hi);
}
template <bool FP16>
__device__ __forceinline__ float act_round(float x) {
    return FP16 ? __half2float(__float2half_rn(x)) : bf16_round(x);
}
template <bool FP16>
__device__ __forceinline__ float act_lo(uint32_t w) {
    if (FP16) return __low2float(*reinterpret_cast<const __half2*>(&w));
    return __low2float(*reinterpret_cast<const __nv_bfloat162*>(&w));   // (a conversion the compiler can fold into the consumer; a shift is not)
}
template <bool FP16>
__device__ __forceinline__ float act_hi(uint32_t w) {
    if (FP16) return __high2float(*reinterpret_cast<const __half2*>(&w));
    return __high2float(*reinterpret_cast<const __nv_bfloat162*>(&w));
}

// Stores 16 accumulator values of a TRANSPOSED tile (this lane = head-dimension index d, value i =
// output row row0+i) as bf16: the 32 lanes of a warp write 64 contiguous bytes of one output row per
// instruction.  `dst` points at (row row0, element d); rows are `rstride` elements apart; rows >=
// nvalid are skipped (the test is uniform over the warp).  (Exchanging values between lane pairs
// to write packed 4-byte pairs was measured slower than one bf16 per lane.)
__device__ __forceinline__ void store_transposed_bf16_16(__nv_bfloat16* dst, int64_t rstride, const uint32_t (&v)[16],
                                                         int row0, int nvalid) {
    if (row0 + 16 <= nvalid) {
#pragma unroll
        for (int i = 0; i < 16; ++i) dst[i * rstride] = __float2bfloat16_rn(__uint_as_float(v[i]));
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i)
            if (row0 + i < nvalid) dst[i * rstride] = __float2bfloat16_rn(__uint_as_float(v[i]));
    }
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

}  // namespace fmsa
