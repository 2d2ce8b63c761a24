/*
 * bam_fused.cuh -- library-internal wrappers of the public fused launch (include/bam/launch.cuh).
 */
#ifndef BAM_FUSED_CUH
#define BAM_FUSED_CUH

#include <cuda_runtime.h>

#include "bam/launch.cuh"
#include "bam_internal.h"

extern thread_local cudaError_t g_last_cuda;
#define CK(x)                                              \
    do {                                                   \
        cudaError_t e_ = (x);                              \
        if (e_ != cudaSuccess) { g_last_cuda = e_; (void)cudaGetLastError(); return BAM_ECUDA; } \
    } while (0)

template <class Work>
static int launch_fused(bam_ctrl* c, const Work& w, cudaStream_t s)
{
    uint32_t grid = 0;
    cudaError_t e = bam::launch_fused(c->emu, w, s, c->max_grid, &grid);
    if (e == cudaErrorInvalidConfiguration) { (void)cudaGetLastError(); return BAM_EINVAL; }
    CK(e);
    c->last_grid = grid;
    return BAM_OK;
}

template <class Work>
static int fused_geometry(bam_ctrl* c, uint32_t* grid)
{
    cudaError_t e = cudaSuccess;
    uint32_t g = bam::fused_max_grid<Work>(&e);
    CK(e);
    if (c->max_grid && g > c->max_grid) g = c->max_grid;
    *grid = g;
    return BAM_OK;
}

/* wrapping 64-bit sum of one value per lane, added to *out by lane 0 */
__device__ __forceinline__ void warp_sum_to(uint64_t v, uint64_t* out)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31u) == 0u && out) bam::red_add_relaxed(out, v);
}

#endif
