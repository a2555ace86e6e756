// Texts of other symbol widths. The reference instantiates its builder for 1-, 2- and 4-byte symbols
// (src/GPU_SACA.cu:2400-2402, src/Query_Engine.cu:1684-1686). The kernels of this library work on 16-bit symbols; a text of
// another width is first mapped onto 16-bit symbols in a way that keeps the numeric order of the symbols, which keeps the order
// of the suffixes and therefore the suffix array: bytes widen as they are; 32-bit symbols are replaced by their ranks among the
// distinct symbols of the text, which works while there are at most 65536 of them (more are refused: CSA_E_LIMIT).
#include "common.cuh"

namespace
{

__global__ void widen_u8_kernel(const u8* __restrict__ in, const u64 n, u16* __restrict__ out)
{
    const u64 stride = u64(gridDim.x) * blockDim.x;
    for(u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = u16(in[i]);
}

// One bit per possible 32-bit symbol: 2^27 words.
constexpr u64 BITMAP_WORDS = u64(1) << 27;
constexpr u32 GROUPS = 1u << 16, WORDS_PER_GROUP = 1u << 11;      // 65536 groups of 65536 symbols

__global__ void mark_symbols_kernel(const u32* __restrict__ in, const u64 n, u32* __restrict__ bitmap)
{
    const u64 stride = u64(gridDim.x) * blockDim.x;
    for(u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    {
        const u32 v = in[i], bit = 1u << (v & 31);
        if((bitmap[v >> 5] & bit) == 0) atomicOr(bitmap + (v >> 5), bit);      // most symbols have been seen already
    }
}

// Distinct symbols per group of 65536 symbols (one block of 256 threads per group; 8 words per thread).
__global__ void __launch_bounds__(256) count_groups_kernel(const u32* __restrict__ bitmap, u32* __restrict__ group_count)
{
    __shared__ u32 s[8];
    const u32* w = bitmap + u64(blockIdx.x) * WORDS_PER_GROUP;
    u32 c = 0;
    for(u32 k = threadIdx.x; k < WORDS_PER_GROUP; k += 256) c += __popc(w[k]);
    for(int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xFFFFFFFFu, c, o);
    if(lane_id() == 0) s[threadIdx.x >> 5] = c;
    __syncthreads();
    if(threadIdx.x == 0) { u32 t = 0; for(int k = 0; k < 8; ++k) t += s[k]; group_count[blockIdx.x] = t; }
}

// Exclusive sums of the 65536 group counts (one block), and the total.
__global__ void __launch_bounds__(1024) scan_groups_kernel(const u32* __restrict__ group_count, u32* __restrict__ group_first, u64* __restrict__ total)
{
    __shared__ u32 s[32];
    __shared__ u32 carry;
    if(threadIdx.x == 0) carry = 0;
    __syncthreads();
    for(u32 base = 0; base < GROUPS; base += 1024)
    {
        const u32 v = group_count[base + threadIdx.x];
        u32 inc = v;
        for(int o = 1; o < 32; o <<= 1) { const u32 t = __shfl_up_sync(0xFFFFFFFFu, inc, o); if(int(lane_id()) >= o) inc += t; }
        if(lane_id() == 31) s[threadIdx.x >> 5] = inc;
        __syncthreads();
        u32 pre = carry;
        for(u32 w = 0; w < (threadIdx.x >> 5); ++w) pre += s[w];
        group_first[base + threadIdx.x] = pre + inc - v;
        __syncthreads();
        if(threadIdx.x == 1023) carry = pre + inc;
        __syncthreads();
    }
    if(threadIdx.x == 0) *total = carry;
}

// The distinct symbols in ascending order (at most 65536, checked by the caller): one warp per non-empty group walks its words.
__global__ void __launch_bounds__(32) list_alphabet_kernel(const u32* __restrict__ bitmap, const u32* __restrict__ group_count, const u32* __restrict__ group_first,
                                                          u32* __restrict__ alphabet)
{
    const u32 g = blockIdx.x;
    if(group_count[g] == 0) return;
    const u32* w = bitmap + u64(g) * WORDS_PER_GROUP;
    u32 at = group_first[g];
    for(u32 k0 = 0; k0 < WORDS_PER_GROUP; k0 += 32)
    {
        const u32 word = w[k0 + lane_id()];
        const u32 c = __popc(word);
        u32 inc = c;
        for(int o = 1; o < 32; o <<= 1) { const u32 t = __shfl_up_sync(0xFFFFFFFFu, inc, o); if(int(lane_id()) >= o) inc += t; }
        u32 o = at + inc - c;
        for(u32 b = word; b != 0; b &= b - 1) alphabet[o++] = (g << 16) | ((k0 + lane_id()) << 5) | u32(__ffs(b) - 1);
        at += __shfl_sync(0xFFFFFFFFu, inc, 31);
    }
}

__global__ void rank_symbols_kernel(const u32* __restrict__ in, const u64 n, const u32* __restrict__ alphabet, const u32 distinct, u16* __restrict__ out)
{
    const u64 stride = u64(gridDim.x) * blockDim.x;
    for(u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    {
        const u32 v = in[i];
        u32 a = 0, b = distinct - 1;          // v is in the alphabet
        while(a < b)
        {
            const u32 mid = (a + b) >> 1;
            if(__ldg(alphabet + mid) < v) a = mid + 1; else b = mid;
        }
        out[i] = u16(a);
    }
}

unsigned grid_for(u64 n) { const u64 b = div_up(n, 256); return unsigned(b < 148 * 16 ? (b ? b : 1) : 148 * 16); }

}   // namespace

extern "C" int csa_text_from_u8(csa_ctx* ctx, const uint8_t* text_dev, uint64_t n, uint16_t* out_dev)
{
    if(!ctx || !text_dev || !out_dev) return csa_fail(ctx, CSA_E_INVALID, "csa_text_from_u8: null argument");
    if(n == 0) return CSA_OK;
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    widen_u8_kernel<<<grid_for(n), 256, 0, ctx->stream>>>(text_dev, n, out_dev);
    CSA_LAUNCH_CHECK(ctx);
    CSA_CUDA(ctx, cudaMemsetAsync(out_dev + n, 0, CSA_TEXT_PAD * 2, ctx->stream));
    return CSA_OK;
}

extern "C" int csa_text_from_u32(csa_ctx* ctx, const uint32_t* text_dev, uint64_t n, uint16_t* out_dev, uint32_t* alphabet_dev, uint32_t* distinct)
{
    if(!ctx || !text_dev || !out_dev || !alphabet_dev || !distinct) return csa_fail(ctx, CSA_E_INVALID, "csa_text_from_u32: null argument");
    *distinct = 0;
    if(n == 0) return CSA_OK;
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    void* ws = nullptr;
    CSA_TRY(csa_aux(ctx, BITMAP_WORDS * 4 + 2 * size_t(GROUPS) * 4 + 1024, &ws));
    u32* bitmap = static_cast<u32*>(ws);
    u32* group_count = bitmap + BITMAP_WORDS;
    u32* group_first = group_count + GROUPS;
    u64* total_d = ctx->d_scalars + 14;
    CSA_CUDA(ctx, cudaMemsetAsync(bitmap, 0, BITMAP_WORDS * 4, ctx->stream));
    mark_symbols_kernel<<<grid_for(n), 256, 0, ctx->stream>>>(text_dev, n, bitmap);
    CSA_LAUNCH_CHECK(ctx);
    count_groups_kernel<<<GROUPS, 256, 0, ctx->stream>>>(bitmap, group_count);
    CSA_LAUNCH_CHECK(ctx);
    scan_groups_kernel<<<1, 1024, 0, ctx->stream>>>(group_count, group_first, total_d);
    CSA_LAUNCH_CHECK(ctx);
    CSA_CUDA(ctx, cudaMemcpyAsync(ctx->h_scalars + 14, total_d, 8, cudaMemcpyDeviceToHost, ctx->stream));
    CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    const u64 total = ctx->h_scalars[14];
    if(total > 65536) return csa_fail(ctx, CSA_E_LIMIT, "csa_text_from_u32: " + std::to_string(total) + " distinct symbols; at most 65536 map onto 16-bit symbols");
    *distinct = u32(total);
    list_alphabet_kernel<<<GROUPS, 32, 0, ctx->stream>>>(bitmap, group_count, group_first, alphabet_dev);
    CSA_LAUNCH_CHECK(ctx);
    rank_symbols_kernel<<<grid_for(n), 256, 0, ctx->stream>>>(text_dev, n, alphabet_dev, u32(total), out_dev);
    CSA_LAUNCH_CHECK(ctx);
    CSA_CUDA(ctx, cudaMemsetAsync(out_dev + n, 0, CSA_TEXT_PAD * 2, ctx->stream));
    return CSA_OK;
}
