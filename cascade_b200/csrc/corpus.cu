// Seeded synthetic corpora with the shape of the tokenized corpora the reference is run on (u16 token ids,
// 0xFFFF written before each document; dataset/tokenize-corpus.py:4-7 of the reference describes that layout).
// Every symbol is a pure function of (seed, position), so the host and the device produce the same text and any
// part of it can be made alone.
//
//   position i is a separator iff a document ended at i - 1; a document ends after each of its tokens with
//   probability 1 / mean_doc (geometric lengths >= 1, mean mean_doc); position 0 is a separator;
//   every other position holds a token drawn by inverse CDF from 64-bit thresholds (Zipf, made by the caller).
#include "common.cuh"

namespace
{

__host__ __device__ __forceinline__ u64 hash64(u64 x)
{
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

__host__ __device__ __forceinline__ bool doc_ends_after(u64 seed, u64 j, u32 mean_doc)
{
    return hash64(seed * 0x9E3779B97F4A7C15ull + 2 * j + 1) % mean_doc == 0;
}

__host__ __device__ __forceinline__ bool is_separator(u64 seed, u64 i, u32 mean_doc)
{
    if(i == 0) return true;
    // sep(i) = ends(i-1) and not sep(i-1): count the run of end flags that stops at i - 1.
    u64 run = 0, j = i;
    while(j > 0 && doc_ends_after(seed, j - 1, mean_doc)) { ++run; --j; }
    if(j == 0) return (i & 1) == 0;       // the run reaches the start of the text, whose position 0 is a separator
    return (run & 1) == 1;
}

__host__ __device__ __forceinline__ u16 token_at(u64 seed, u64 i, const u64* cdf, u32 vocab)
{
    const u64 u = hash64(seed * 0xD1B54A32D192ED03ull + 2 * i);
    u32 a = 0, b = vocab - 1;           // first rank whose threshold is not below u
    while(a < b)
    {
        const u32 mid = (a + b) >> 1;
        if(u <= cdf[mid]) b = mid; else a = mid + 1;
    }
    return u16(a);
}

__host__ __device__ __forceinline__ u16 symbol_at(u64 seed, u64 i, u32 mean_doc, const u64* cdf, u32 vocab)
{
    return is_separator(seed, i, mean_doc) ? u16(0xFFFF) : token_at(seed, i, cdf, vocab);
}

__global__ void gen_corpus_kernel(u16* __restrict__ T, const u64 first, const u64 n, const u64 seed, const u32 mean_doc, const u64* __restrict__ cdf, const u32 vocab)
{
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if(i < n) T[i] = symbol_at(seed, first + i, mean_doc, cdf, vocab);
}

}   // namespace

extern "C" int csa_gen_corpus_dev(csa_ctx* ctx, uint16_t* text, uint64_t n, uint64_t seed, uint32_t mean_doc, const uint64_t* cdf, uint32_t vocab)
{
    if(!ctx || !text || !cdf || mean_doc == 0 || vocab == 0 || vocab > 65535) return csa_fail(ctx, CSA_E_INVALID, "csa_gen_corpus_dev: bad argument");
    if(n == 0) return CSA_OK;
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    gen_corpus_kernel<<<unsigned(div_up(n, 256)), 256, 0, ctx->stream>>>(text, 0, n, seed, mean_doc, reinterpret_cast<const u64*>(cdf), vocab);
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

extern "C" int csa_gen_corpus_dev_window(csa_ctx* ctx, uint16_t* text, uint64_t first, uint64_t count, uint64_t seed, uint32_t mean_doc, const uint64_t* cdf, uint32_t vocab)
{
    if(!ctx || !text || !cdf || mean_doc == 0 || vocab == 0 || vocab > 65535) return csa_fail(ctx, CSA_E_INVALID, "csa_gen_corpus_dev_window: bad argument");
    if(count == 0) return CSA_OK;
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    for(u64 at = 0; at < count; at += u64(1) << 30)
    {
        const u64 c = count - at < (u64(1) << 30) ? count - at : (u64(1) << 30);
        gen_corpus_kernel<<<unsigned(div_up(c, 256)), 256, 0, ctx->stream>>>(text + at, first + at, c, seed, mean_doc, reinterpret_cast<const u64*>(cdf), vocab);
        CSA_LAUNCH_CHECK(ctx);
    }
    return CSA_OK;
}

extern "C" int csa_gen_corpus_host(uint16_t* text, uint64_t first, uint64_t count, uint64_t seed, uint32_t mean_doc, const uint64_t* cdf, uint32_t vocab)
{
    if(!text || !cdf || mean_doc == 0 || vocab == 0 || vocab > 65535) return CSA_E_INVALID;
    #pragma omp parallel for schedule(static)
    for(u64 k = 0; k < count; ++k)
        text[k] = symbol_at(seed, first + k, mean_doc, reinterpret_cast<const u64*>(cdf), vocab);
    return CSA_OK;
}
