/* util.h -- cuda_err_chk as in the reference's include/util.h:23-43 (prints, does not abort). */
#ifndef BAM_COMPAT_UTIL_H
#define BAM_COMPAT_UTIL_H
#include <cuda_runtime.h>
#include <cstdio>
#define cuda_err_chk(ans) { bam_gpu_assert((ans), __FILE__, __LINE__); }
inline void bam_gpu_assert(cudaError_t code, const char* file, int line)
{
    if (code != cudaSuccess) fprintf(stderr, "GPUassert: %s %s %d\n", cudaGetErrorString(code), file, line);
}
#endif
