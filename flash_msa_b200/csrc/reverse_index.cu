// Deterministic reverse index: a CSR that lists, for every (batch, proxy head, key block), the
// query positions that selected that block, in ascending order.
//
// Four small kernels, no global atomics and no host synchronisation:
//   1. count : one CTA per (batch*proxy head, query block) builds a shared-memory bitmap
//              "row r selected key block j" and writes the per-(query block, key block) counts;
//   2. colscan: one thread per (batch*proxy head, key block) turns the counts of its column into
//              exclusive offsets over the query blocks and records the column total;
//   3. rowscan: a single CTA turns the totals into row_ptr;
//   4. fill  : the bitmap is rebuilt and every edge gets position
//              row_ptr + block offset + (number of lower rows of its block that chose the key block).
// The edge rule `0 <= kb < NB && kb <= q/128` is the reference's
// (flash_msa/csrc/reverse_index_cuda.cu:41); its atomics-based slot assignment (:118) is replaced
// by ranks, so the output is a pure function of the input.
#include <mutex>

#include "host_common.h"
#include "sm100.cuh"

namespace fmsa {
namespace {

// Shared memory of the count and fill kernels: the bitmap words[j*4 + w] (rows 32w..32w+31 of the query block that
// selected key block j), then the query block's 128 x Kb selections, copied in with 16-byte loads (the rows of a
// query block are contiguous).  Thread r works on row r and walks its Kb slots starting at slot r % Kb, so that the
// lanes of a warp touch different banks.
__device__ __forceinline__ int32_t* stage_rows(uint32_t* words, const int32_t* idx_rows, int NB, int Kb) {
    int32_t* tile = reinterpret_cast<int32_t*>(words + NB * 4);
    const int4* src = reinterpret_cast<const int4*>(idx_rows);
    int4* dst = reinterpret_cast<int4*>(tile);
    for (int t = threadIdx.x; t < kBlock * Kb / 4; t += blockDim.x) dst[t] = src[t];
    for (int t = threadIdx.x; t < NB * 4; t += blockDim.x) words[t] = 0u;
    __syncthreads();
    return tile;
}
__device__ __forceinline__ int rotated_slot(int s, int r, int Kb) {
    const int x = s + (r % Kb);
    return x >= Kb ? x - Kb : x;
}
__device__ __forceinline__ void build_bitmap(uint32_t* words, const int32_t* tile, int NB, int Kb, int qblk) {
    const int r = threadIdx.x;   // 128 threads: one per row
    const int32_t* row = tile + r * Kb;
    for (int s = 0; s < Kb; ++s) {
        const int j = row[rotated_slot(s, r, Kb)];
        if (static_cast<unsigned>(j) < static_cast<unsigned>(NB) && j <= qblk) atomicOr(&words[j * 4 + (r >> 5)], 1u << (r & 31));
    }
    __syncthreads();
}

__global__ void __launch_bounds__(128) rix_count_kernel(const int32_t* __restrict__ idx, uint8_t* __restrict__ counts,
                                                        int S, int NB, int Kb) {
    extern __shared__ __align__(16) uint32_t words[];
    const int qblk = blockIdx.x;
    const int64_t bp = blockIdx.y;
    const int32_t* tile = stage_rows(words, idx + (bp * S + static_cast<int64_t>(qblk) * kBlock) * Kb, NB, Kb);
    build_bitmap(words, tile, NB, Kb, qblk);
    uint8_t* crow = counts + (bp * NB + qblk) * NB;
    for (int j = threadIdx.x; j <= qblk; j += blockDim.x) {
        const int c = __popc(words[j * 4]) + __popc(words[j * 4 + 1]) + __popc(words[j * 4 + 2]) + __popc(words[j * 4 + 3]);
        crow[j] = static_cast<uint8_t>(c);   // <= 128
    }
}

__global__ void rix_colscan_kernel(const uint8_t* __restrict__ counts, int32_t* __restrict__ blk_off,
                                   int32_t* __restrict__ totals, int64_t rows_bh, int NB) {
    const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= rows_bh * NB) return;
    const int64_t bp = t / NB;
    const int j = static_cast<int>(t % NB);
    int run = 0;
    for (int i = j; i < NB; ++i) {
        const int64_t at = (bp * NB + i) * NB + j;
        blk_off[at] = run;
        run += counts[at];
    }
    totals[t] = run;
}

__global__ void __launch_bounds__(1024) rix_rowscan_kernel(const int32_t* __restrict__ totals,
                                                           int32_t* __restrict__ row_ptr, int64_t n) {
    __shared__ int64_t part[1024];
    const int tid = threadIdx.x;
    const int64_t per = (n + 1023) / 1024;
    const int64_t lo = tid * per, hi = (lo + per < n) ? lo + per : n;
    int64_t sum = 0;
    for (int64_t i = lo; i < hi; ++i) sum += totals[i];
    part[tid] = sum;
    __syncthreads();
    // Hillis-Steele inclusive scan over 1024 partials
    for (int off = 1; off < 1024; off <<= 1) {
        const int64_t v = (tid >= off) ? part[tid - off] : 0;
        __syncthreads();
        part[tid] += v;
        __syncthreads();
    }
    int64_t run = part[tid] - sum;
    for (int64_t i = lo; i < hi; ++i) {
        row_ptr[i] = static_cast<int32_t>(run);
        run += totals[i];
    }
    if (tid == 1023) row_ptr[n] = static_cast<int32_t>(part[1023]);
}

__global__ void __launch_bounds__(128) rix_fill_kernel(const int32_t* __restrict__ idx, const int32_t* __restrict__ blk_off,
                                                       const int32_t* __restrict__ row_ptr, int32_t* __restrict__ col_q,
                                                       int32_t* __restrict__ edge_pos, int S, int NB, int Kb) {
    extern __shared__ __align__(16) uint32_t words[];
    const int qblk = blockIdx.x;
    const int64_t bp = blockIdx.y;
    const int64_t row0 = bp * S + static_cast<int64_t>(qblk) * kBlock;
    int32_t* tile = stage_rows(words, idx + row0 * Kb, NB, Kb);
    build_bitmap(words, tile, NB, Kb, qblk);
    const int r = threadIdx.x;
    const int q = qblk * kBlock + r;
    int32_t* row = tile + r * Kb;   // the selections of row r; each is replaced by its edge position
    const int32_t* rp = row_ptr + bp * NB;
    const int32_t* bo = blk_off + (bp * NB + qblk) * NB;
    const int w = r >> 5;
    const uint32_t below = (1u << (r & 31)) - 1u;
    for (int s = 0; s < Kb; ++s) {
        const int at = rotated_slot(s, r, Kb);
        const int j = row[at];
        int pos = -1;
        if (static_cast<unsigned>(j) < static_cast<unsigned>(NB) && j <= qblk) {
            int rank = __popc(words[j * 4 + w] & below);
            for (int ww = 0; ww < w; ++ww) rank += __popc(words[j * 4 + ww]);
            pos = rp[j] + bo[j] + rank;
            col_q[pos] = q;
        }
        row[at] = pos;
    }
    __syncthreads();
    // edge positions of the query block leave as one contiguous run
    const int4* src = reinterpret_cast<const int4*>(tile);
    int4* dst = reinterpret_cast<int4*>(edge_pos + row0 * Kb);
    for (int t = threadIdx.x; t < kBlock * Kb / 4; t += blockDim.x) dst[t] = src[t];
}

struct RixWorkspace {
    uint8_t* counts;
    int32_t* blk_off;
    int32_t* totals;
    size_t bytes;
};

RixWorkspace carve(void* base, int64_t rows_bh, int NB) {
    RixWorkspace w;
    const size_t n2 = static_cast<size_t>(rows_bh) * NB * NB;
    size_t off = 0;
    w.counts = reinterpret_cast<uint8_t*>(static_cast<char*>(base) + off);
    off += static_cast<size_t>(round_up(static_cast<int64_t>(n2), 256));
    w.blk_off = reinterpret_cast<int32_t*>(static_cast<char*>(base) + off);
    off += static_cast<size_t>(round_up(static_cast<int64_t>(n2 * 4), 256));
    w.totals = reinterpret_cast<int32_t*>(static_cast<char*>(base) + off);
    off += static_cast<size_t>(round_up(static_cast<int64_t>(rows_bh) * NB * 4, 256));
    w.bytes = off;
    return w;
}

}  // namespace

// Launch sequence shared with any other entry point that supplies its own scratch memory.
int reverse_index_launch(const int32_t* block_indices, int32_t* row_ptr, int32_t* col_q, int32_t* edge_pos,
                         int64_t rows_bh, int32_t S, int32_t Kb, void* scratch, cudaStream_t st) {
    const int NB = S / kBlock;
    const RixWorkspace w = carve(scratch, rows_bh, NB);
    const dim3 grid(static_cast<unsigned>(NB), static_cast<unsigned>(rows_bh));
    const size_t smem = static_cast<size_t>(NB) * 16 + static_cast<size_t>(kBlock) * Kb * sizeof(int32_t);
    constexpr size_t kSmemCap = 160 * 1024;   // NB <= 2048 and Kb <= 128 need 96 KB; the attribute is set once, to the cap
    if (smem > kSmemCap || (reinterpret_cast<uintptr_t>(block_indices) & 15u) != 0 || (reinterpret_cast<uintptr_t>(edge_pos) & 15u) != 0)
        return FMSA_ERR_UNSUPPORTED;
    if (!ensure_smem_attr(reinterpret_cast<const void*>(rix_count_kernel), kSmemCap) ||
        !ensure_smem_attr(reinterpret_cast<const void*>(rix_fill_kernel), kSmemCap))
        return FMSA_ERR_CUDA;
    rix_count_kernel<<<grid, 128, smem, st>>>(block_indices, w.counts, S, NB, Kb);
    const int64_t cols = rows_bh * NB;
    rix_colscan_kernel<<<static_cast<unsigned>((cols + 127) / 128), 128, 0, st>>>(w.counts, w.blk_off, w.totals, rows_bh, NB);
    rix_rowscan_kernel<<<1, 1024, 0, st>>>(w.totals, row_ptr, cols);
    rix_fill_kernel<<<grid, 128, smem, st>>>(block_indices, w.blk_off, row_ptr, col_q, edge_pos, S, NB, Kb);
    return check_launch();
}

size_t reverse_index_scratch_bytes(int64_t rows_bh, int32_t S) {
    return carve(nullptr, rows_bh, S / kBlock).bytes;
}

// -------------------------------------------------------------------------------------------
// Allocation-free variant: the scratch lives in the library image.
// -------------------------------------------------------------------------------------------
// Every GPU that loads the library holds these bytes until the process exits.
static __device__ __align__(256) unsigned char g_rix_static_scratch[FMSA_STATIC_SCRATCH_BYTES];

// In host code the array's name is only a handle for the runtime, not a device address, so the
// address is asked for once per device (with that device current) and cached.
static int static_scratch_address(void** out) {
    constexpr int kMaxDevices = 64;
    static void* cached[kMaxDevices] = {nullptr};
    static std::mutex guard;
    std::lock_guard<std::mutex> lock(guard);
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return FMSA_ERR_CUDA;
    if (cached[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_rix_static_scratch) != cudaSuccess || p == nullptr) return FMSA_ERR_CUDA;
        cached[dev] = p;
    }
    *out = cached[dev];
    return FMSA_OK;
}

}  // namespace fmsa

extern "C" int fmsa_reverse_index_static(const int32_t* block_indices, int32_t* row_ptr, int32_t* col_q,
                                         int32_t* edge_pos, int64_t rows_bh, int32_t S, int32_t top_k_blocks,
                                         void* stream) {
    using namespace fmsa;
    FMSA_REQUIRE(block_indices && row_ptr && col_q && edge_pos);
    FMSA_REQUIRE(rows_bh > 0 && rows_bh <= 65535 && S > 0 && S % kBlock == 0);
    const int NB = S / kBlock;
    FMSA_REQUIRE(top_k_blocks >= 1 && top_k_blocks <= NB);
    FMSA_REQUIRE(rows_bh * static_cast<int64_t>(S) * top_k_blocks < 0x7fffffffLL);
    if (NB > 2048) return FMSA_ERR_UNSUPPORTED;
    // the problem must fit the built-in scratch; larger ones need fmsa_reverse_index and a workspace
    if (reverse_index_scratch_bytes(rows_bh, S) > static_cast<size_t>(FMSA_STATIC_SCRATCH_BYTES)) return FMSA_ERR_WORKSPACE;
    void* scratch = nullptr;
    const int rc = static_scratch_address(&scratch);
    if (rc != FMSA_OK) return rc;
    // Nothing in the scratch has to start at zero: every count, offset and total a kernel reads
    // was written earlier in the same call, so stale contents of a previous call are never seen.
    return reverse_index_launch(block_indices, row_ptr, col_q, edge_pos, rows_bh, S, top_k_blocks, scratch,
                                static_cast<cudaStream_t>(stream));
}

extern "C" size_t fmsa_reverse_index_workspace_bytes(int64_t rows_bh, int32_t S) {
    if (rows_bh <= 0 || S <= 0 || S % fmsa::kBlock != 0) return 0;
    return fmsa::reverse_index_scratch_bytes(rows_bh, S);
}

extern "C" int fmsa_reverse_index(const int32_t* block_indices, int32_t* row_ptr, int32_t* col_q, int32_t* edge_pos,
                                  int64_t rows_bh, int32_t S, int32_t top_k_blocks, void* workspace,
                                  size_t workspace_bytes, void* stream) {
    using namespace fmsa;
    FMSA_REQUIRE(block_indices && row_ptr && col_q && edge_pos && workspace);
    FMSA_REQUIRE(rows_bh > 0 && rows_bh <= 65535 && S > 0 && S % kBlock == 0);
    const int NB = S / kBlock;
    FMSA_REQUIRE(top_k_blocks >= 1 && top_k_blocks <= NB);
    FMSA_REQUIRE(rows_bh * static_cast<int64_t>(S) * top_k_blocks < 0x7fffffffLL);
    if (NB > 2048) return FMSA_ERR_UNSUPPORTED;   // bitmap must fit in shared memory (NB*16 bytes)
    FMSA_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255u) == 0);
    if (workspace_bytes < reverse_index_scratch_bytes(rows_bh, S)) return FMSA_ERR_WORKSPACE;
    return reverse_index_launch(block_indices, row_ptr, col_q, edge_pos, rows_bh, S, top_k_blocks, workspace,
                                static_cast<cudaStream_t>(stream));
}
