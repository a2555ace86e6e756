// Bulk exchange of ranks between the GPUs of a sharded build. The inverse array is cut by text position into one shard
// per GPU. Fine-grained loads and stores into a peer's shard are correct but slow once a shard spans gigabytes, so ranks
// travel as the reference's messages do (one message = a position and a rank, include/message.hpp:22-61; collated by
// destination, include/GPU_SACA.cuh:291-353), only over NVLink instead of host RAM: a GPU sorts its records into one
// bucket per destination GPU, the buckets cross as plain contiguous copies into the destination's inbox, and the
// destination applies them to its own shard. Reads work the same way with a request and a response leg.
#include "common.cuh"
#include "part.cuh"

namespace
{

constexpr int EX_BLOCK = 256, EX_ITEMS = 8, EX_TILE = EX_BLOCK * EX_ITEMS;

__device__ __forceinline__ u32 owner_of(u64 x, u64 shard) { return u32(x / shard); }

template <bool PACKED>
__global__ void __launch_bounds__(EX_BLOCK) count_owners_kernel(const u32* __restrict__ pos, const u64* __restrict__ packed, const u64 count, const u64 h,
                                                                const u64 n, const u64 shard, const u32 gpus, u64* __restrict__ counts)
{
    __shared__ u32 c[CSA_MAX_GPUS];
    if(threadIdx.x < CSA_MAX_GPUS) c[threadIdx.x] = 0;
    __syncthreads();
    u32 mine[CSA_MAX_GPUS];
    #pragma unroll
    for(int g = 0; g < CSA_MAX_GPUS; ++g) mine[g] = 0;
    for(int i = 0; i < EX_ITEMS; ++i)
    {
        const u64 k = u64(blockIdx.x) * EX_TILE + u64(i) * EX_BLOCK + threadIdx.x;
        if(k >= count) break;
        const u64 x = PACKED ? (packed[k] >> 32) : u64(pos[k]) + h;
        if(x >= n) continue;
        const u32 o = owner_of(x, shard);
        #pragma unroll
        for(int g = 0; g < CSA_MAX_GPUS; ++g) mine[g] += (o == u32(g));
    }
    #pragma unroll
    for(int g = 0; g < CSA_MAX_GPUS; ++g)
    {
        u32 v = mine[g];
        for(int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
        if(lane_id() == 0 && v) atomicAdd(&c[g], v);
    }
    __syncthreads();
    if(threadIdx.x < gpus && c[threadIdx.x]) atomicAdd(&counts[threadIdx.x], u64(c[threadIdx.x]));
}

// One block buckets EX_TILE records: counts per destination in shared memory, reserves one run per destination with one
// atomic on the destination's cursor, then writes each record into its run.
template <bool PACKED>
__global__ void __launch_bounds__(EX_BLOCK) bucket_kernel(const u32* __restrict__ pos, const u64* __restrict__ packed, const u64 count, const u64 h,
                                                          const u64 n, const u64 shard, const u32 gpus, u64* __restrict__ cursor,
                                                          u32* __restrict__ req_out, u32* __restrict__ perm_out, u64* __restrict__ upd_out)
{
    __shared__ u32 c[CSA_MAX_GPUS];
    __shared__ u64 base[CSA_MAX_GPUS];
    if(threadIdx.x < CSA_MAX_GPUS) c[threadIdx.x] = 0;
    __syncthreads();
    u32 own[EX_ITEMS], r[EX_ITEMS];
    u64 x[EX_ITEMS];
    #pragma unroll
    for(int i = 0; i < EX_ITEMS; ++i)
    {
        const u64 k = u64(blockIdx.x) * EX_TILE + u64(i) * EX_BLOCK + threadIdx.x;
        own[i] = 0xFFFFFFFFu;
        if(k < count)
        {
            x[i] = PACKED ? (packed[k] >> 32) : u64(pos[k]) + h;
            if(x[i] < n) own[i] = owner_of(x[i], shard);
        }
        // lanes with the same destination share one shared-memory atomic
        const u32 o = own[i];
        u32 peers = __match_any_sync(0xFFFFFFFFu, o);
        u32 old = 0;
        if(o != 0xFFFFFFFFu && (peers & lanemask_lt()) == 0) old = atomicAdd(&c[o], u32(__popc(peers)));
        old = __shfl_sync(0xFFFFFFFFu, old, __ffs(peers) - 1);
        r[i] = old + __popc(peers & lanemask_lt());
    }
    __syncthreads();
    if(threadIdx.x < gpus && c[threadIdx.x]) base[threadIdx.x] = atomicAdd(&cursor[threadIdx.x], u64(c[threadIdx.x]));
    __syncthreads();
    #pragma unroll
    for(int i = 0; i < EX_ITEMS; ++i)
    {
        if(own[i] == 0xFFFFFFFFu) continue;
        const u64 k = u64(blockIdx.x) * EX_TILE + u64(i) * EX_BLOCK + threadIdx.x;
        const u64 at = base[own[i]] + r[i];
        const u32 local = u32(x[i] - u64(own[i]) * shard);
        if(PACKED) upd_out[at] = (u64(local) << 32) | (packed[k] & 0xFFFFFFFFull);
        else { req_out[at] = local; perm_out[at] = u32(k); }
    }
}

__global__ void serve_requests_kernel(const u32* __restrict__ isa_local, const u32* __restrict__ req, const u64 count, u32* __restrict__ resp)
{
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if(i < count) resp[i] = isa_local[req[i]];
}

__global__ void apply_updates_kernel(u32* __restrict__ isa_local, const u64* __restrict__ upd, const u64 count, const u64 first_position)
{
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if(i < count) { const u64 u = upd[i]; isa_local[(u >> 32) - first_position] = u32(u); }
}

__global__ void keys_init_kernel(const u32* __restrict__ head, const u32* __restrict__ pos, const u64 count, const u64 n, const u64 h, const int sec_bits,
                                 u64* __restrict__ keys)
{
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if(i >= count) return;
    const u64 x = u64(pos[i]) + h;
    keys[i] = (u64(head[i]) << sec_bits) | (x >= n ? (n - 1 + h - x) : 0ull);
}

__global__ void keys_add_kernel(const u32* __restrict__ perm, const u32* __restrict__ resp, const u64 count, const u64 h, u64* __restrict__ keys)
{
    const u64 j = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if(j < count) keys[perm[j]] += u64(resp[j]) + h;
}

// Updates into 256 buckets by the top 8 bits of their position, for a list that holds every position of [0, n) exactly once:
// bucket b then holds exactly the positions [b << low_bits, (b + 1) << low_bits) and starts at entry b << low_bits, so nothing
// has to be counted first; and as the order inside a bucket does not matter, a record's place in its tile's run is simply what
// a shared-memory atomic hands out (no stable ranking, no look-back): a block counts, reserves one run per bucket with an
// atomic on the bucket's cursor, stages its records by bucket and writes coalesced runs. cursor: 256 words, zeroed.
constexpr int BU_BLOCK = 256, BU_ITEMS = 16, BU_TILE = BU_BLOCK * BU_ITEMS;
__global__ void __launch_bounds__(BU_BLOCK) bucket_updates_kernel(const u64* __restrict__ in, const u64 count, const int low_bits, u64* __restrict__ out,
                                                                  u64* __restrict__ cursor, u64* __restrict__ dev_status)
{
    __shared__ u64 stage[BU_TILE];
    __shared__ u64 base[256];         // entry of `out` where the tile's run of the bucket starts, minus the run's start in the tile
    __shared__ u32 cnt[256];
    __shared__ u32 warp_tot[8];
    const u32 tid = threadIdx.x;
    const u64 tile_first = u64(blockIdx.x) * BU_TILE;
    const u32 valid = (count - tile_first < u64(BU_TILE)) ? u32(count - tile_first) : u32(BU_TILE);
    cnt[tid] = 0;
    __syncthreads();
    u64 u[BU_ITEMS];
    u32 r[BU_ITEMS];
    #pragma unroll
    for(int k = 0; k < BU_ITEMS; ++k)
    {
        const u32 j = tid + k * BU_BLOCK;
        if(j < valid) u[k] = __ldcs(in + tile_first + j);
    }
    #pragma unroll
    for(int k = 0; k < BU_ITEMS; ++k)
    {
        const u32 j = tid + k * BU_BLOCK;
        if(j < valid) r[k] = atomicAdd(&cnt[u32(u[k] >> (32 + low_bits)) & 255u], 1u);
    }
    __syncthreads();
    // exclusive scan of the 256 counts (one per thread), then the runs' places
    const u32 c = cnt[tid];
    u32 inc = c;
    #pragma unroll
    for(int o = 1; o < 32; o <<= 1)
    {
        const u32 t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
        if(int(tid & 31) >= o) inc += t;
    }
    if((tid & 31) == 31) warp_tot[tid >> 5] = inc;
    __syncthreads();
    u32 pre = 0;
    for(u32 w = 0; w < (tid >> 5); ++w) pre += warp_tot[w];
    const u32 start = pre + inc - c;
    if(c) base[tid] = (u64(tid) << low_bits) + atomicAdd(reinterpret_cast<unsigned long long*>(cursor + tid), (unsigned long long)c) - start;
    cnt[tid] = start;
    __syncthreads();
    #pragma unroll
    for(int k = 0; k < BU_ITEMS; ++k)
    {
        const u32 j = tid + k * BU_BLOCK;
        if(j < valid) stage[cnt[u32(u[k] >> (32 + low_bits)) & 255u] + r[k]] = u[k];
    }
    __syncthreads();
    #pragma unroll
    for(int k = 0; k < BU_ITEMS; ++k)
    {
        const u32 j = tid + k * BU_BLOCK;
        if(j < valid)
        {
            const u64 v = stage[j];
            const u64 at = base[u32(v >> (32 + low_bits)) & 255u] + j;
            if(at < count) out[at] = v;
            else atomicOr(reinterpret_cast<unsigned long long*>(dev_status), (unsigned long long)CSA_ST_RANGE);    // the list did not cover every position once
        }
    }
}

// Up to CSA_MAX_GPUS contiguous copies in one launch, each possibly into another GPU's memory: every SM streams a share of
// every segment, so the copies to all peers run side by side over NVLink instead of one after another.
struct Copy_Segments
{
    void* dst[CSA_MAX_GPUS];
    const void* src[CSA_MAX_GPUS];
    u64 words[CSA_MAX_GPUS];        // 4-byte words
    u32 count;
};

__global__ void __launch_bounds__(256) copy_segments_kernel(const Copy_Segments segs)
{
    // Blocks are dealt to the segments round robin, so that all destinations are written at the same time: if every GPU
    // wrote to GPU 0 first, then to GPU 1, ... each destination's link would carry all traffic in turn while the others idle.
    const u32 k = blockIdx.x % segs.count;
    const u64 lane_block = blockIdx.x / segs.count, blocks = (gridDim.x - k + segs.count - 1) / segs.count;      // blocks that serve segment k
    const u64 first = lane_block * blockDim.x + threadIdx.x, stride = blocks * blockDim.x;
    const u64 words = segs.words[k];
    const bool wide = ((reinterpret_cast<uintptr_t>(segs.dst[k]) | reinterpret_cast<uintptr_t>(segs.src[k])) & 15) == 0;
    const u32* s1 = static_cast<const u32*>(segs.src[k]);
    u32* d1 = static_cast<u32*>(segs.dst[k]);
    if(wide)
    {
        const uint4* s4 = static_cast<const uint4*>(segs.src[k]);
        uint4* d4 = static_cast<uint4*>(segs.dst[k]);
        const u64 quads = words >> 2;
        for(u64 i = first; i < quads; i += stride) d4[i] = s4[i];
        for(u64 i = (quads << 2) + first; i < words; i += stride) d1[i] = s1[i];
    }
    else
        for(u64 i = first; i < words; i += stride) d1[i] = s1[i];
}

}   // namespace

int launch_copy_segments(csa_ctx* ctx, void* const* dst, const void* const* src, const u64* bytes, u32 count)
{
    Copy_Segments segs;
    segs.count = 0;
    u64 total = 0;
    for(u32 k = 0; k < count && segs.count < CSA_MAX_GPUS; ++k)
    {
        if(bytes[k] == 0) continue;
        segs.dst[segs.count] = dst[k]; segs.src[segs.count] = src[k]; segs.words[segs.count] = bytes[k] / 4;
        total += bytes[k];
        ++segs.count;
    }
    if(segs.count == 0) return CSA_OK;
    const u64 want = div_up(total / 16 + 1, 256 * 4);
    unsigned blocks = unsigned(want < 148 * 8 ? (want < 1 ? 1 : want) : 148 * 8);
    if(blocks < segs.count) blocks = segs.count;        // every segment needs a block
    copy_segments_kernel<<<blocks, 256, 0, ctx->stream>>>(segs);
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

int launch_count_owners(csa_ctx* ctx, const u32* pos, const u64* packed, u64 count, u64 h, u64 n, u64 shard, u32 gpus, u64* counts)
{
    if(count == 0) return CSA_OK;
    (void)packed;
    count_owners_kernel<false><<<unsigned(div_up(count, EX_TILE)), EX_BLOCK, 0, ctx->stream>>>(pos, packed, count, h, n, shard, gpus, counts);
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

int launch_bucket_requests(csa_ctx* ctx, const u32* pos, u64 count, u64 h, u64 n, u64 shard, u32 gpus, u64* cursor, u32* req_out, u32* perm_out)
{
    if(count == 0) return CSA_OK;
    bucket_kernel<false><<<unsigned(div_up(count, EX_TILE)), EX_BLOCK, 0, ctx->stream>>>(pos, nullptr, count, h, n, shard, gpus, cursor, req_out, perm_out, nullptr);
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

int launch_serve_requests(csa_ctx* ctx, const u32* isa_local, const u32* req, u64 count, u32* resp)
{
    if(count == 0) return CSA_OK;
    serve_requests_kernel<<<unsigned(div_up(count, 256)), 256, 0, ctx->stream>>>(isa_local, req, count, resp);
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

int launch_apply_updates(csa_ctx* ctx, u32* isa_local, const u64* upd, u64 count, u64 first_position)
{
    if(count == 0) return CSA_OK;
    apply_updates_kernel<<<unsigned(div_up(count, 256)), 256, 0, ctx->stream>>>(isa_local, upd, count, first_position);
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

int launch_keys_init(csa_ctx* ctx, const u32* head, const u32* pos, u64 count, u64 n, u64 h, int sec_bits, u64* keys)
{
    if(count == 0) return CSA_OK;
    keys_init_kernel<<<unsigned(div_up(count, 256)), 256, 0, ctx->stream>>>(head, pos, count, n, h, sec_bits, keys);
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

int launch_keys_add(csa_ctx* ctx, const u32* perm, const u32* resp, u64 count, u64 h, u64* keys)
{
    if(count == 0) return CSA_OK;
    keys_add_kernel<<<unsigned(div_up(count, 256)), 256, 0, ctx->stream>>>(perm, resp, count, h, keys);
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

int apply_updates_in_address_order(csa_ctx* ctx, u32* isa_local, u64* upd, u64* alt, u64 count, int position_bits, void* sort_ws, size_t sort_ws_bytes,
                                   bool every_position_once)
{
    if(count == 0) return CSA_OK;
    const u64* list = upd;
    // Worth a pass only when the array is much larger than L2 and the list is long enough to pay for the pass.
    if(position_bits > 24 && count >= (u64(1) << 20))
    {
        // 8 bits measured best at 2e9 positions: a stretch of the array per bucket (31 MB) stays in L2; 6 bits do not, 10-12 cost a second pass
        if(every_position_once && sort_ws_bytes >= 256 * sizeof(u64))
        {
            u64* cursor = static_cast<u64*>(sort_ws);
            CSA_CUDA(ctx, cudaMemsetAsync(cursor, 0, 256 * sizeof(u64), ctx->stream));
            bucket_updates_kernel<<<unsigned(div_up(count, BU_TILE)), BU_BLOCK, 0, ctx->stream>>>(upd, count, position_bits - 8, alt, cursor, ctx->d_status);
            CSA_LAUNCH_CHECK(ctx);
            list = alt;
        }
        else
        {
            const int top = 32 + position_bits, begin = top - 8;
            int in_alt = 0;
            CSA_TRY(csa_sort_pairs(ctx, reinterpret_cast<uint64_t*>(upd), reinterpret_cast<uint64_t*>(alt), nullptr, nullptr, 4, count, begin, top, sort_ws, sort_ws_bytes, &in_alt));
            list = in_alt ? alt : upd;
        }
    }
    return launch_apply_updates(ctx, isa_local, list, count, 0);
}
