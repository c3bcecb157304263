// Launcher for the reference's activation quantizer with resident buffers (test and benchmark infrastructure,
// never linked into the shipped library).  The reference only exposes its kernel through q8_1()
// (src/cuda/q8_1.cu:148-193), which allocates, copies and frees around every launch; timing the kernel itself
// needs a call that takes device pointers.  The kernel is the reference's own, compiled from its source where it
// lies and linked here by name (relocatable device code); only its prototype (src/cuda/q8_1.cu:20-29) and the
// launch geometry of q8_1() (:172-183: 128 threads, grid (rows, ceil(K / 512), 1)) are restated.
#include <cstdint>

#include <cuda_runtime.h>

__global__ void quantize_q8_1_kernel(const float *__restrict__ x, void *__restrict__ vy, const int64_t ne0_0, const int64_t s0_1,
                                     const int64_t s0_2, const int64_t s0_3, const int64_t ne0, const int64_t ne1,
                                     const int64_t ne2);

extern "C" int jq_ref_quantize_q8_1_device(const float *d_x, void *d_y, int64_t K, int64_t M, cudaStream_t stream) {
    const int block_size = 128;
    const dim3 blocks((unsigned)M, (unsigned)((K + 4 * block_size - 1) / (4 * block_size)), 1);
    quantize_q8_1_kernel<<<blocks, dim3(block_size, 1, 1), 0, stream>>>(d_x, d_y, K, K, K * M, K * M, K, M, 1);
    return (int)cudaGetLastError();
}
