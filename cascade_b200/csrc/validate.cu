// Exact, full check of a 5-byte suffix array against its text, on the device: the array is a permutation of [0, n) and
// every neighbouring pair is in suffix order. The order of a pair needs one symbol and one rank each: T[x] < T[y], or the
// symbols are equal and the suffix at x + 1 ranks before the suffix at y + 1, where the (empty) suffix at n ranks before
// all others. By induction over the suffix lengths this holds for every pair exactly when the whole array is sorted.
//
// It stands for test::is_permutation + test::is_correct_SA (test/end-to-end.cpp:11-80), the reference's own validator,
// which does the same three sweeps on the host with OpenMP.
#include "common.cuh"

namespace
{

// result words: [0] entries out of range, [1] entries seen before (duplicates), [2] pairs out of order, [3] lowest rank i
// whose pair (i - 1, i) is out of order (or ~0)
template <typename R>
__global__ void validate_mark_kernel(const u8* __restrict__ sa40, const u64 n, u32* __restrict__ seen, R* __restrict__ rank, u64* __restrict__ result)
{
    const u64 stride = u64(gridDim.x) * blockDim.x;
    for(u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    {
        const u64 x = sa40_load(sa40, i);
        if(x >= n) { atomicAdd(result + 0, 1ull); continue; }
        const u32 bit = 1u << (x & 31);
        const u32 old = atomicOr(seen + (x >> 5), bit);
        if(old & bit) atomicAdd(result + 1, 1ull);
        else rank[x] = R(i);
    }
}

template <typename R>
__global__ void validate_order_kernel(const u16* __restrict__ T, const u8* __restrict__ sa40, const u64 n, const R* __restrict__ rank, u64* __restrict__ result)
{
    const u64 stride = u64(gridDim.x) * blockDim.x;
    for(u64 i = 1 + u64(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    {
        const u64 x = sa40_load(sa40, i - 1), y = sa40_load(sa40, i);
        if(x >= n || y >= n) continue;          // counted by the first sweep
        const u16 a = T[x], b = T[y];
        bool bad = false;
        if(a > b) bad = true;
        else if(a == b)
        {
            // rank of the following suffix, the empty suffix first
            const long long rx = (x + 1 < n) ? (long long)rank[x + 1] : -1;
            const long long ry = (y + 1 < n) ? (long long)rank[y + 1] : -1;
            bad = rx >= ry;
        }
        if(bad)
        {
            atomicAdd(result + 2, 1ull);
            atomicMin(result + 3, i);
        }
    }
}

template <typename R>
int run_validate(csa_ctx* ctx, const u16* T, u64 n, const u8* sa40, void* ws, u64* result)
{
    const size_t seen_bytes = align_up256(div_up(n, 32) * 4);
    u32* seen = static_cast<u32*>(ws);
    R* rank = reinterpret_cast<R*>(static_cast<u8*>(ws) + seen_bytes);
    CSA_CUDA(ctx, cudaMemsetAsync(seen, 0, seen_bytes, ctx->stream));
    const u64 init[4] = {0, 0, 0, ~0ull};
    CSA_CUDA(ctx, cudaMemcpyAsync(result, init, sizeof(init), cudaMemcpyHostToDevice, ctx->stream));
    const unsigned blocks = unsigned(div_up(n, 256) < 148 * 16 ? div_up(n, 256) : 148 * 16);
    validate_mark_kernel<R><<<blocks, 256, 0, ctx->stream>>>(sa40, n, seen, rank, result);
    CSA_LAUNCH_CHECK(ctx);
    validate_order_kernel<R><<<blocks, 256, 0, ctx->stream>>>(T, sa40, n, rank, result);
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

}   // namespace

extern "C" size_t csa_validate_workspace_bytes(uint64_t n)
{
    const size_t rank_bytes = size_t(n) * (n <= (1ull << 32) ? 4 : 8);
    return align_up256(div_up(n, 32) * 4) + align_up256(rank_bytes) + 256;
}

extern "C" int csa_validate_sa(csa_ctx* ctx, const uint16_t* text_dev, uint64_t n, const uint8_t* sa40_dev, void* workspace_dev, size_t workspace_bytes,
                               uint64_t* result_dev)
{
    if(!ctx || !text_dev || !sa40_dev || !workspace_dev || !result_dev) return csa_fail(ctx, CSA_E_INVALID, "csa_validate_sa: null argument");
    if(n == 0 || n > (1ull << 40)) return csa_fail(ctx, CSA_E_INVALID, "csa_validate_sa: n out of range");
    if(workspace_bytes < csa_validate_workspace_bytes(n)) return csa_fail(ctx, CSA_E_NOMEM, "csa_validate_sa: workspace too small");
    if(reinterpret_cast<uintptr_t>(sa40_dev) & 3) return csa_fail(ctx, CSA_E_INVALID, "csa_validate_sa: the suffix array must be 4-byte aligned");
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    if(n <= (1ull << 32)) return run_validate<u32>(ctx, text_dev, n, sa40_dev, workspace_dev, reinterpret_cast<u64*>(result_dev));
    return run_validate<u64>(ctx, text_dev, n, sa40_dev, workspace_dev, reinterpret_cast<u64*>(result_dev));
}
