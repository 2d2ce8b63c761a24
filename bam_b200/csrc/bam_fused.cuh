/*
 * bam_fused.cuh -- the fused cooperative launch shared by every workload of libbam_b200.so.
 *
 * A workload kernel waits on completions that the emulated controller produces, so both must be
 * running at the same time.  They are therefore ONE cooperative launch (co-residency of all
 * blocks is guaranteed by cudaLaunchCooperativeKernel or the launch fails): blocks
 * [0, n_ctrl_blocks) run bam::emu_controller_main, the remaining blocks are persistent workers
 * that stride over the workload (a functor called with its worker-block index and the number of
 * worker blocks).  The controller blocks leave when the last worker block has finished.
 */
#ifndef BAM_FUSED_CUH
#define BAM_FUSED_CUH

#include <cuda_runtime.h>

#include "bam/array.cuh"
#include "bam/emu_ctrl.cuh"
#include "bam_internal.h"

extern thread_local cudaError_t g_last_cuda;
#define CK(x)                                              \
    do {                                                   \
        cudaError_t e_ = (x);                              \
        if (e_ != cudaSuccess) { g_last_cuda = e_; (void)cudaGetLastError(); return BAM_ECUDA; } \
    } while (0)

/* Dynamic shared memory of every block of a fused launch: the controller blocks use it as their
 * bulk-copy stages; it has to be the same size for all blocks of one grid. */
extern __shared__ __align__(128) uint8_t bam_dyn_smem[];
#define BAM_FUSED_SMEM BAM_EMU_SMEM_BYTES

template <class Work>
__global__ void __launch_bounds__(BAM_THREADS, BAM_MIN_BLOCKS)
bam_fused(const __grid_constant__ bam_emu_d_t emu, const __grid_constant__ Work work)
{
    if (blockIdx.x < emu.n_ctrl_blocks) {
        bam::emu_controller_main(emu, bam_dyn_smem);
        return;
    }
    work(blockIdx.x - emu.n_ctrl_blocks, gridDim.x - emu.n_ctrl_blocks);
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        bam::red_add_release(emu.consumers_remaining, 0xffffffffu);
    }
}

template <class Work>
static int launch_fused(bam_ctrl* c, const Work& w, cudaStream_t s)
{
    static thread_local int blocks_per_sm = 0;
    if (blocks_per_sm == 0) {
        int nb = 0;
        CK(cudaFuncSetAttribute(bam_fused<Work>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)BAM_FUSED_SMEM));
        CK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, bam_fused<Work>, BAM_THREADS, BAM_FUSED_SMEM));
        if (nb < 1) return BAM_EINVAL;
        blocks_per_sm = nb;
    }
    uint32_t grid = (uint32_t)blocks_per_sm * (uint32_t)c->num_sms;
    if (c->max_grid && grid > c->max_grid) grid = c->max_grid;
    if (grid <= c->emu.n_ctrl_blocks) return BAM_EINVAL;
    const uint32_t n_work = grid - c->emu.n_ctrl_blocks;
    CK(cudaMemcpyAsync(c->emu.consumers_remaining, &n_work, sizeof n_work, cudaMemcpyHostToDevice, s));
    bam_emu_d_t emu = c->emu;
    void* args[] = { (void*)&emu, (void*)&w };
    CK(cudaLaunchCooperativeKernel((const void*)bam_fused<Work>, dim3(grid), dim3(BAM_THREADS), args, BAM_FUSED_SMEM, s));
    c->last_grid = grid;
    return BAM_OK;
}

template <class Work>
static int fused_geometry(bam_ctrl* c, uint32_t* grid)
{
    int nb = 0;
    CK(cudaFuncSetAttribute(bam_fused<Work>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)BAM_FUSED_SMEM));
    CK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, bam_fused<Work>, BAM_THREADS, BAM_FUSED_SMEM));
    *grid = (uint32_t)nb * (uint32_t)c->num_sms;
    if (c->max_grid && *grid > c->max_grid) *grid = c->max_grid;
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
