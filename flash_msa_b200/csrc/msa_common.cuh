// Index arithmetic shared by the forward, combine and backward kernels.
#pragma once

#include <stdint.h>

#include "sm100.cuh"

namespace fmsa {

// Dense (warmup) schedule: the "reverse-index row" of key block j of one (batch, proxy head) is
// every query position >= 128*j, in order.  Rows are laid out back to back, so the edge of
// (key block j, query q) sits at  bp*S*(NB+1)/2 + j*S - 128*j*(j-1)/2 + (q - 128*j).
__host__ __device__ __forceinline__ int64_t dense_edges_per_bp(int S, int NB) {
    return static_cast<int64_t>(S) * (NB + 1) / 2;
}
__host__ __device__ __forceinline__ int64_t dense_edge_base(int64_t bp, int S, int NB) {
    return bp * dense_edges_per_bp(S, NB);
}
__host__ __device__ __forceinline__ int64_t dense_row_offset(int j, int S) {
    return static_cast<int64_t>(j) * S - static_cast<int64_t>(kBlock) * j * (j - 1) / 2;
}

// -------------------------------------------------------------------------------------------
// Work decomposition shared by the forward and the backward.
//
// A reverse-index row (batch, proxy head, key block j) can hold anything from one chunk of 128
// query rows to all S - 128*j later rows (a "sink" block).  To keep the persistent CTAs balanced a
// row is cut into sub-units of at most kChunksPerSubUnit chunks.  The number of rows is only known
// on the device, so the sub-units are enumerated for the worst case (NB - j chunks) and a CTA that
// draws a sub-unit beyond the real end of its row simply skips it.
//
// Order: (batch, KV head) group major, then sub-unit index s (chunks 8s .. 8s+7 of a row), then key
// block ascending, then proxy head of the group.  Group-major order keeps the rows that the active
// CTAs gather from and reduce into (a few heads of Q, dO) resident in L2.  Inside a group, putting s
// outermost makes neighbouring sub-units alike in size (for a given s the rows of neighbouring key
// blocks are about equally long, and the sub-units that lie beyond the end of their row cluster
// together), so both a dynamic work counter and a static round-robin deal stay balanced.
// -------------------------------------------------------------------------------------------
constexpr int kChunksPerSubUnit = 8;

// Key blocks j that can have a sub-unit s: NB - j > C*s, i.e. j < NB - C*s.
__host__ __device__ __forceinline__ int64_t subunits_per_group(int NB, int ppk, int C) {
    int64_t total = 0;
    for (int s = 0; s * C < NB; ++s) total += NB - s * C;
    return total * ppk;
}

struct SubUnit {
    int g, j, pp, chunk0;
};
__device__ __forceinline__ SubUnit decode_subunit(int64_t u, int NB, int ppk) {
    constexpr int C = kChunksPerSubUnit;
    const int64_t per_group = subunits_per_group(NB, ppk, C);
    SubUnit su;
    su.g = static_cast<int>(u / per_group);
    const int64_t r = u % per_group;
    su.pp = static_cast<int>(r % ppk);
    int64_t x = r / ppk;
    int s = 0;
    while (x >= NB - s * C) {   // at most NB/C iterations
        x -= NB - s * C;
        ++s;
    }
    su.j = static_cast<int>(x);
    su.chunk0 = s * C;
    return su;
}

}  // namespace fmsa
