// BENCHMARK-ONLY baseline, not part of the product and never linked into it: the library sort that the reference calls
// (cub::DeviceRadixSort::SortPairs, src/GPU_SACA.cu:1849 of the reference) timed on this box on the same record shape as
// the product's own radix sort, so that the two numbers stand side by side in bench.py's output.
#include <cub/cub.cuh>
#include <cuda_runtime.h>

#include <cstdint>

namespace
{

__global__ void fill_kernel(unsigned long long* keys, unsigned int* vals, unsigned long long n, unsigned long long seed)
{
    const unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
    if(i >= n) return;
    unsigned long long x = i + seed;
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    keys[i] = x ^ (x >> 31);
    vals[i] = (unsigned int)i;
}

}   // namespace

// Sorts n random (64-bit key, 32-bit value) records on key bits [0, bits) `reps` times (after one untimed run) and writes the
// average device milliseconds of one sort to *ms_out. Returns 0, or a cudaError_t.
extern "C" int cub_sort_pairs_ms(unsigned long long n, int bits, int reps, double* ms_out)
{
    unsigned long long *k0 = nullptr, *k1 = nullptr, *src = nullptr;
    unsigned int *v0 = nullptr, *v1 = nullptr;
    void* tmp = nullptr;
    size_t tmp_bytes = 0;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    cudaError_t rc = cudaSuccess;
    float total = 0;
#define CK(x) do { rc = (x); if(rc != cudaSuccess) goto done; } while(0)
    CK(cudaMalloc(&k0, n * 8)); CK(cudaMalloc(&k1, n * 8)); CK(cudaMalloc(&src, n * 8));
    CK(cudaMalloc(&v0, n * 4)); CK(cudaMalloc(&v1, n * 4));
    fill_kernel<<<unsigned((n + 255) / 256), 256>>>(src, v0, n, 12345);
    {
        cub::DoubleBuffer<unsigned long long> dk(k0, k1);
        cub::DoubleBuffer<unsigned int> dv(v0, v1);
        CK(cub::DeviceRadixSort::SortPairs(nullptr, tmp_bytes, dk, dv, (int64_t)n, 0, bits));
    }
    CK(cudaMalloc(&tmp, tmp_bytes));
    CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
    for(int r = 0; r <= reps; ++r)
    {
        CK(cudaMemcpy(k0, src, n * 8, cudaMemcpyDeviceToDevice));
        cub::DoubleBuffer<unsigned long long> dk(k0, k1);
        cub::DoubleBuffer<unsigned int> dv(v0, v1);
        CK(cudaEventRecord(e0));
        CK(cub::DeviceRadixSort::SortPairs(tmp, tmp_bytes, dk, dv, (int64_t)n, 0, bits));
        CK(cudaEventRecord(e1));
        CK(cudaEventSynchronize(e1));
        float ms = 0;
        CK(cudaEventElapsedTime(&ms, e0, e1));
        if(r > 0) total += ms;
    }
    *ms_out = reps > 0 ? total / reps : 0.0;
done:
#undef CK
    if(e0) cudaEventDestroy(e0);
    if(e1) cudaEventDestroy(e1);
    cudaFree(tmp); cudaFree(k0); cudaFree(k1); cudaFree(src); cudaFree(v0); cudaFree(v1);
    return (int)rc;
}
