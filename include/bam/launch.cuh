/*
 * bam/launch.cuh -- the fused cooperative launch every kernel that reads through the cache uses.
 *
 * A kernel that calls bam::array<T>::operator[] waits on completions that the emulated NVMe
 * controller produces, so both must be running at the same time.  Separate launches that wait
 * on each other are not guaranteed to run together; therefore they are ONE cooperative launch
 * (co-residency of all blocks is guaranteed by cudaLaunchCooperativeKernel, or the launch fails):
 * blocks [0, emu.n_ctrl_blocks) run bam::emu_controller_main, the remaining blocks are
 * persistent workers.  The workload is a functor
 *
 *     struct Work { ...; __device__ void operator()(uint32_t worker_block, uint32_t n_worker_blocks) const; };
 *
 * that strides over its own units (the reference's kernels index by blockIdx/threadIdx over a grid
 * as large as the problem; here worker_block / n_worker_blocks play that role in a grid-stride
 * loop).  The controller blocks leave when the last worker block has finished.
 */
#ifndef BAM_LAUNCH_CUH
#define BAM_LAUNCH_CUH

#include <cuda_runtime.h>

#include "array.cuh"
#include "emu_ctrl.cuh"

#define BAM_THREADS 256               /* threads per block of every fused launch              */
#ifndef BAM_MIN_BLOCKS
#define BAM_MIN_BLOCKS 3              /* resident blocks per SM the kernels are compiled for  */
#endif

/* Dynamic shared memory of every block of a fused launch (BAM_EMU_SMEM_BYTES): the controller
 * blocks use it as their bulk-copy stages, workers may stage cache pages in it; it has to be the
 * same size for all blocks of one grid. */
extern __shared__ __align__(128) uint8_t bam_dyn_smem[];
#define BAM_FUSED_SMEM BAM_EMU_SMEM_BYTES

/* A workload may ask for another register budget than the default: `static constexpr int min_blocks = 2;` in
 * the functor compiles its kernel for two resident blocks per SM (128 registers per thread instead of 80). */
template <class Work, class = void>
struct fused_min_blocks { static constexpr int value = BAM_MIN_BLOCKS; };
template <class Work>
struct fused_min_blocks<Work, decltype((void)Work::min_blocks)> { static constexpr int value = Work::min_blocks; };

template <class Work>
__global__ void __launch_bounds__(BAM_THREADS, fused_min_blocks<Work>::value)
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

namespace bam {

/* Blocks of bam_fused<Work> that are co-resident on the current device (0 on error). */
template <class Work>
inline uint32_t fused_max_grid(cudaError_t* err = nullptr)
{
    int dev = 0, sms = 0, nb = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(bam_fused<Work>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)BAM_FUSED_SMEM);
    if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, bam_fused<Work>, BAM_THREADS, BAM_FUSED_SMEM);
    if (err) *err = e;
    return e == cudaSuccess ? (uint32_t)nb * (uint32_t)sms : 0u;
}

/* Launch `work` fused with the controller described by `emu` (bam_ctrl_emu_descriptor) on stream
 * s.  max_grid caps the total number of blocks (0 = the cap the descriptor carries, and without one all
 * blocks that are co-resident).  Asynchronous. */
template <class Work>
inline cudaError_t launch_fused(const bam_emu_d_t& emu, const Work& work, cudaStream_t s = 0, uint32_t max_grid = 0,
                                uint32_t* grid_out = nullptr)
{
    cudaError_t e = cudaSuccess;
    uint32_t grid = fused_max_grid<Work>(&e);
    if (e != cudaSuccess) return e;
    if (max_grid == 0) max_grid = emu.max_grid;              /* the controller's own cap (bam_ctrl_set_max_grid) */
    if (max_grid && grid > max_grid) grid = max_grid;
    if (grid <= emu.n_ctrl_blocks) return cudaErrorInvalidConfiguration;
    const uint32_t n_work = grid - emu.n_ctrl_blocks;
    e = cudaMemcpyAsync(emu.consumers_remaining, &n_work, sizeof n_work, cudaMemcpyHostToDevice, s);
    if (e != cudaSuccess) return e;
    bam_emu_d_t emu_copy = emu;
    void* args[] = { (void*)&emu_copy, (void*)&work };
    e = cudaLaunchCooperativeKernel((const void*)bam_fused<Work>, dim3(grid), dim3(BAM_THREADS), args, BAM_FUSED_SMEM, s);
    if (grid_out) *grid_out = grid;
    return e;
}

}  // namespace bam
#endif
