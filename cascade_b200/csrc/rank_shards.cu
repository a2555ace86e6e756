// A rank store that is sharded by position over several GPUs, seen from one of them: sorting a list of positions (requests or
// rank messages) into one run per owning GPU before the caller's collective carries the runs, answering the requests that
// arrived for this GPU's stretch, and applying the messages that arrived for it. The reference keeps one inbox per partition
// on the host and fills it with messages (include/message.hpp:22-61, src/Partition_Backend.cpp:516-553); here the owner of a
// position is position / stretch and the runs cross NVLink.
#include "common.cuh"
#include "sort.cuh"

namespace
{

__global__ void owner_count_kernel(const u64* __restrict__ pos, const u64 count, const u64 stretch, const u32 owners, u64* __restrict__ counts, u64* __restrict__ dev_status)
{
    __shared__ u32 s_cnt[CSA_MAX_GPUS];
    if(threadIdx.x < CSA_MAX_GPUS) s_cnt[threadIdx.x] = 0;
    __syncthreads();
    u32 mine[CSA_MAX_GPUS];
    #pragma unroll
    for(int g = 0; g < CSA_MAX_GPUS; ++g) mine[g] = 0;
    const u64 stride = u64(gridDim.x) * blockDim.x;
    for(u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride)
    {
        const u64 o = pos[i] / stretch;
        if(o >= owners) { atomicOr(dev_status, (u64)CSA_ST_RANGE); continue; }
        #pragma unroll
        for(int g = 0; g < CSA_MAX_GPUS; ++g) mine[g] += (o == u64(g));
    }
    #pragma unroll
    for(int g = 0; g < CSA_MAX_GPUS; ++g)
    {
        u32 v = mine[g];
        #pragma unroll
        for(int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
        if(lane_id() == 0 && v) atomicAdd(&s_cnt[g], v);
    }
    __syncthreads();
    if(threadIdx.x < owners && s_cnt[threadIdx.x]) atomicAdd(reinterpret_cast<unsigned long long*>(counts + threadIdx.x), (unsigned long long)s_cnt[threadIdx.x]);
}

__global__ void iota_kernel(u32* __restrict__ out, const u64 count)
{
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if(i < count) out[i] = u32(i);
}

// cursor[g]: where owner g's run starts, advanced as the run fills. The lanes of a warp with one owner take their places with
// one atomic. The order inside a run is arbitrary; order[j] remembers where the j-th entry of the runs came from.
__global__ void owner_scatter_kernel(const u64* __restrict__ pos, const u32* __restrict__ payload, const u64 count, const u64 stretch, const u32 owners,
                                     u64* __restrict__ cursor, u64* __restrict__ pos_out, u32* __restrict__ payload_out, u32* __restrict__ order)
{
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    u32 g = 0xFFFFFFFFu;
    u64 x = 0;
    if(i < count) { x = pos[i]; const u64 o = x / stretch; if(o < owners) g = u32(o); }
    const u32 peers = __match_any_sync(0xFFFFFFFFu, g);
    u64 base = 0;
    if(g != 0xFFFFFFFFu && (peers & lanemask_lt()) == 0) base = atomicAdd(reinterpret_cast<unsigned long long*>(cursor + g), (unsigned long long)__popc(peers));
    base = __shfl_sync(0xFFFFFFFFu, base, __ffs(peers) - 1);
    if(g == 0xFFFFFFFFu) return;
    const u64 slot = base + __popc(peers & lanemask_lt());
    pos_out[slot] = x;
    if(payload) payload_out[slot] = payload[i];
    if(order) order[slot] = u32(i);
}

__global__ void shard_read_kernel(const u32* __restrict__ shard, const u64 first, const u64 positions, const u64* __restrict__ asked, const u64 count,
                                  u32* __restrict__ answers, u64* __restrict__ dev_status)
{
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if(i >= count) return;
    const u64 at = asked[i] - first;
    if(asked[i] >= first && at < positions) answers[i] = shard[at];
    else { answers[i] = 0; atomicOr(dev_status, (u64)CSA_ST_RANGE); }
}

__global__ void shard_apply_kernel(u32* __restrict__ shard, const u64 first, const u64 positions, const u64* __restrict__ pos, const u32* __restrict__ ranks,
                                   const u64 count, u64* __restrict__ dev_status)
{
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if(i >= count) return;
    const u64 at = pos[i] - first;
    if(pos[i] >= first && at < positions) shard[at] = ranks[i];
    else atomicOr(dev_status, (u64)CSA_ST_RANGE);
}

__global__ void unbucket_kernel(const u32* __restrict__ order, const u32* __restrict__ values, const u64 count, u32* __restrict__ out)
{
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if(i < count) out[order[i]] = values[i];
}

__global__ void outbox_positions_kernel(const u32* __restrict__ lo, const u8* __restrict__ hi, const u64 count, u64* __restrict__ pos)
{
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if(i < count) pos[i] = (u64(hi[i]) << 32) | lo[i];
}

}   // namespace

extern "C" int csa_bucket_by_owner(csa_ctx* ctx, const uint64_t* positions_dev, const uint32_t* payload_dev, uint64_t count, uint64_t stretch, uint32_t owners,
                                   uint64_t* counts_host, uint64_t* positions_out_dev, uint32_t* payload_out_dev, uint32_t* order_dev)
{
    if(!ctx || !counts_host || owners == 0 || owners > CSA_MAX_GPUS || stretch == 0) return csa_fail(ctx, CSA_E_INVALID, "csa_bucket_by_owner: bad argument");
    for(u32 g = 0; g < owners; ++g) counts_host[g] = 0;
    if(count == 0) return CSA_OK;
    if(!positions_dev || !positions_out_dev || (payload_dev && !payload_out_dev)) return csa_fail(ctx, CSA_E_INVALID, "csa_bucket_by_owner: null buffer");
    if(count >= (u64(1) << 32)) return csa_fail(ctx, CSA_E_LIMIT, "csa_bucket_by_owner: at most 2^32 - 1 entries a call");
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    u64* counts_dev = ctx->d_scalars + 32;            // CSA_MAX_GPUS words, then as many cursors
    u64* cursor_dev = counts_dev + CSA_MAX_GPUS;
    CSA_CUDA(ctx, cudaMemsetAsync(counts_dev, 0, sizeof(u64) * CSA_MAX_GPUS, ctx->stream));
    const unsigned blocks = unsigned(div_up(count, 256) < 148 * 8 ? div_up(count, 256) : 148 * 8);
    owner_count_kernel<<<blocks, 256, 0, ctx->stream>>>(reinterpret_cast<const u64*>(positions_dev), count, stretch, owners, counts_dev, ctx->d_status);
    CSA_LAUNCH_CHECK(ctx);
    CSA_CUDA(ctx, cudaMemcpyAsync(ctx->h_scalars + 32, counts_dev, sizeof(u64) * CSA_MAX_GPUS, cudaMemcpyDeviceToHost, ctx->stream));
    CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    u64 at = 0;
    for(u32 g = 0; g < owners; ++g) { counts_host[g] = ctx->h_scalars[32 + g]; ctx->h_scalars[32 + CSA_MAX_GPUS + g] = at; at += counts_host[g]; }
    if(at != count) { u64 bits = 0; const int rc = csa_sync(ctx, reinterpret_cast<uint64_t*>(&bits)); return rc != CSA_OK ? rc : csa_fail(ctx, CSA_E_DEVICE, "csa_bucket_by_owner: a position beyond the last owner"); }
    CSA_CUDA(ctx, cudaMemcpyAsync(cursor_dev, ctx->h_scalars + 32 + CSA_MAX_GPUS, sizeof(u64) * CSA_MAX_GPUS, cudaMemcpyHostToDevice, ctx->stream));
    owner_scatter_kernel<<<unsigned(div_up(count, 256)), 256, 0, ctx->stream>>>(reinterpret_cast<const u64*>(positions_dev), payload_dev, count, stretch, owners, cursor_dev,
                                                                                reinterpret_cast<u64*>(positions_out_dev), payload_out_dev, order_dev);
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

extern "C" int csa_order_by_address(csa_ctx* ctx, uint64_t* positions_dev, uint64_t* positions_alt_dev, uint32_t* payload_dev, uint32_t* payload_alt_dev, uint64_t count,
                                    int begin_bit, int end_bit, uint64_t stretch, uint32_t owners, int payload_is_index, uint64_t* counts_host, void* workspace_dev,
                                    size_t workspace_bytes, int* in_alt)
{
    if(!ctx || !counts_host || !in_alt || owners == 0 || owners > CSA_MAX_GPUS || stretch == 0 || begin_bit < 0 || end_bit > 64 || begin_bit >= end_bit)
        return csa_fail(ctx, CSA_E_INVALID, "csa_order_by_address: bad argument");
    if(begin_bit < 63 && stretch % (u64(1) << begin_bit) != 0) return csa_fail(ctx, CSA_E_INVALID, "csa_order_by_address: a stretch must be whole address buckets");
    *in_alt = 0;
    for(u32 g = 0; g < owners; ++g) counts_host[g] = 0;
    if(count == 0) return CSA_OK;
    if(!positions_dev || !positions_alt_dev || !payload_dev || !payload_alt_dev) return csa_fail(ctx, CSA_E_INVALID, "csa_order_by_address: null buffer");
    if(count >= (u64(1) << 32)) return csa_fail(ctx, CSA_E_LIMIT, "csa_order_by_address: at most 2^32 - 1 entries a call");
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    u64* counts_dev = ctx->d_scalars + 40;            // CSA_MAX_GPUS words
    CSA_CUDA(ctx, cudaMemsetAsync(counts_dev, 0, sizeof(u64) * CSA_MAX_GPUS, ctx->stream));
    const unsigned blocks = unsigned(div_up(count, 256) < 148 * 8 ? div_up(count, 256) : 148 * 8);
    owner_count_kernel<<<blocks, 256, 0, ctx->stream>>>(reinterpret_cast<const u64*>(positions_dev), count, stretch, owners, counts_dev, ctx->d_status);
    CSA_LAUNCH_CHECK(ctx);
    if(payload_is_index)
    {
        iota_kernel<<<unsigned(div_up(count, 256)), 256, 0, ctx->stream>>>(payload_dev, count);
        CSA_LAUNCH_CHECK(ctx);
    }
    CSA_CUDA(ctx, cudaMemcpyAsync(ctx->h_scalars + 40, counts_dev, sizeof(u64) * CSA_MAX_GPUS, cudaMemcpyDeviceToHost, ctx->stream));
    // one or two digit passes on the address bits from begin_bit up: owners' runs follow one another, addresses inside a run sweep upwards
    CSA_TRY(csa_sort_pairs(ctx, positions_dev, positions_alt_dev, payload_dev, payload_alt_dev, 4, count, begin_bit, end_bit, workspace_dev, workspace_bytes, in_alt));
    CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    u64 total = 0;
    for(u32 g = 0; g < owners; ++g) { counts_host[g] = ctx->h_scalars[40 + g]; total += counts_host[g]; }
    if(total != count) { u64 bits = 0; const int rc = csa_sync(ctx, reinterpret_cast<uint64_t*>(&bits)); return rc != CSA_OK ? rc : csa_fail(ctx, CSA_E_DEVICE, "csa_order_by_address: a position beyond the last owner"); }
    return CSA_OK;
}

extern "C" int csa_rank_shard_read(csa_ctx* ctx, const uint32_t* shard_dev, uint64_t first, uint64_t positions, const uint64_t* asked_dev, uint64_t count,
                                   uint32_t* answers_dev)
{
    if(!ctx || (count && (!shard_dev || !asked_dev || !answers_dev))) return csa_fail(ctx, CSA_E_INVALID, "csa_rank_shard_read: null argument");
    if(count == 0) return CSA_OK;
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    shard_read_kernel<<<unsigned(div_up(count, 256)), 256, 0, ctx->stream>>>(shard_dev, first, positions, reinterpret_cast<const u64*>(asked_dev), count, answers_dev, ctx->d_status);
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

extern "C" int csa_rank_shard_apply(csa_ctx* ctx, uint32_t* shard_dev, uint64_t first, uint64_t positions, const uint64_t* positions_dev, const uint32_t* ranks_dev,
                                    uint64_t count)
{
    if(!ctx || (count && (!shard_dev || !positions_dev || !ranks_dev))) return csa_fail(ctx, CSA_E_INVALID, "csa_rank_shard_apply: null argument");
    if(count == 0) return CSA_OK;
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    shard_apply_kernel<<<unsigned(div_up(count, 256)), 256, 0, ctx->stream>>>(shard_dev, first, positions, reinterpret_cast<const u64*>(positions_dev), ranks_dev, count, ctx->d_status);
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

extern "C" int csa_unbucket(csa_ctx* ctx, const uint32_t* order_dev, const uint32_t* values_dev, uint64_t count, uint32_t* out_dev)
{
    if(!ctx || (count && (!order_dev || !values_dev || !out_dev))) return csa_fail(ctx, CSA_E_INVALID, "csa_unbucket: null argument");
    if(count == 0) return CSA_OK;
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    unbucket_kernel<<<unsigned(div_up(count, 256)), 256, 0, ctx->stream>>>(order_dev, values_dev, count, out_dev);
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

extern "C" int csa_outbox_positions(csa_ctx* ctx, const uint32_t* pos_lo_dev, const uint8_t* pos_hi_dev, uint64_t count, uint64_t* positions_dev)
{
    if(!ctx || (count && (!pos_lo_dev || !pos_hi_dev || !positions_dev))) return csa_fail(ctx, CSA_E_INVALID, "csa_outbox_positions: null argument");
    if(count == 0) return CSA_OK;
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    outbox_positions_kernel<<<unsigned(div_up(count, 256)), 256, 0, ctx->stream>>>(pos_lo_dev, pos_hi_dev, count, reinterpret_cast<u64*>(positions_dev));
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}
