// Strided copy between pinned host memory and the device for the host-buffer pipeline
// (flash_msa_b200/host.py): a (batch, head range) chunk of a [B,S,H*128] tensor is `rows` pieces of
// `width` bytes, `pitch` bytes apart.  A thin wrapper so that the Python side needs no CUDA runtime
// binding of its own; the direction is inferred from the pointers (unified addressing).
#include <cuda_runtime.h>

#include "../../include/flash_msa_b200.h"
#include "host_common.h"

extern "C" int fmsa_copy2d_async(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width,
                                 size_t rows, void* stream) {
    FMSA_REQUIRE(dst && src && width > 0 && rows > 0 && dst_pitch >= width && src_pitch >= width);
    const cudaError_t e = cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width, rows, cudaMemcpyDefault,
                                            static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? FMSA_OK : FMSA_ERR_CUDA;
}
