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

}  // namespace fmsa
