// The context: stream, device status word, pinned scalars and the grow-only scratch arena.
#include "common.cuh"
#include "sort.cuh"

#include <new>

extern "C" const char* csa_version(void) { return "cascade_b200 0.1 (sm_100a)"; }

extern "C" int csa_ctx_create(int device, csa_ctx** out)
{
    if(!out) return CSA_E_INVALID;
    *out = nullptr;
    csa_ctx* ctx = new(std::nothrow) csa_ctx();
    if(!ctx) return CSA_E_NOMEM;
    ctx->device = device;
    auto fail = [&](cudaError_t e) { std::fprintf(stderr, "csa_ctx_create: %s\n", cudaGetErrorString(e)); delete ctx; return CSA_E_CUDA; };
    cudaError_t e;
    if((e = cudaSetDevice(device)) != cudaSuccess) return fail(e);
    if((e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking)) != cudaSuccess) return fail(e);
    if((e = cudaMalloc(&ctx->d_status, sizeof(u64))) != cudaSuccess) return fail(e);
    if((e = cudaMemset(ctx->d_status, 0, sizeof(u64))) != cudaSuccess) return fail(e);
    if((e = cudaMalloc(&ctx->d_scalars, 64 * sizeof(u64))) != cudaSuccess) return fail(e);
    if((e = cudaMemset(ctx->d_scalars, 0, 64 * sizeof(u64))) != cudaSuccess) return fail(e);
    if((e = cudaMallocHost(&ctx->h_scalars, 64 * sizeof(u64))) != cudaSuccess) return fail(e);
    std::memset(ctx->h_scalars, 0, 64 * sizeof(u64));
    *out = ctx;
    return CSA_OK;
}

extern "C" void csa_ctx_destroy(csa_ctx* ctx)
{
    if(!ctx) return;
    cudaSetDevice(ctx->device);
    if(ctx->stream) cudaStreamSynchronize(ctx->stream);
    sort_free_timing(ctx);
    for(int g = 0; g < CSA_MAX_GPUS; ++g) if(ctx->peer_open[g]) cudaIpcCloseMemHandle(ctx->peer_base[g]);
    if(ctx->arena) cudaFree(ctx->arena);
    if(ctx->aux) cudaFree(ctx->aux);
    if(ctx->d_status) cudaFree(ctx->d_status);
    if(ctx->d_scalars) cudaFree(ctx->d_scalars);
    if(ctx->h_scalars) cudaFreeHost(ctx->h_scalars);
    if(ctx->host_aux) cudaFreeHost(ctx->host_aux);
    if(ctx->symbol_table) cudaFree(ctx->symbol_table);
    for(int l = 0; l < csa_ctx::LANES; ++l)
    {
        if(ctx->lane_event[l]) cudaEventDestroy(ctx->lane_event[l]);
        if(ctx->lane[l]) { cudaStreamSynchronize(ctx->lane[l]); cudaStreamDestroy(ctx->lane[l]); }
    }
    if(ctx->stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
}

extern "C" int csa_sync(csa_ctx* ctx, uint64_t* status_bits)
{
    if(!ctx) return CSA_E_INVALID;
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    CSA_CUDA(ctx, cudaMemcpyAsync(ctx->h_scalars + 63, ctx->d_status, sizeof(u64), cudaMemcpyDeviceToHost, ctx->stream));
    CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    const u64 bits = ctx->h_scalars[63];
    if(status_bits) *status_bits = bits;
    if(bits != 0)
    {
        CSA_CUDA(ctx, cudaMemsetAsync(ctx->d_status, 0, sizeof(u64), ctx->stream));
        CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        ctx->err = "device status word is non-zero: " + std::to_string(bits);
        return CSA_E_DEVICE;
    }
    return CSA_OK;
}

extern "C" const char* csa_last_error(const csa_ctx* ctx) { return ctx ? ctx->err.c_str() : ""; }
extern "C" void* csa_ctx_stream(csa_ctx* ctx) { return ctx ? static_cast<void*>(ctx->stream) : nullptr; }
extern "C" uint64_t csa_kernel_launches(const csa_ctx* ctx) { return ctx ? ctx->counters[0] : 0; }

extern "C" void csa_reset_counters(csa_ctx* ctx)
{
    if(!ctx) return;
    for(auto& c : ctx->counters) c = 0;
    sort_reset_timing(ctx);
}

int csa_lanes(csa_ctx* ctx)
{
    for(int l = 0; l < csa_ctx::LANES; ++l)
    {
        if(!ctx->lane[l]) CSA_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->lane[l], cudaStreamNonBlocking));
        if(!ctx->lane_event[l]) CSA_CUDA(ctx, cudaEventCreateWithFlags(&ctx->lane_event[l], cudaEventDisableTiming));
    }
    return CSA_OK;
}

int csa_arena(csa_ctx* ctx, size_t bytes, void** out)
{
    if(bytes > ctx->arena_bytes)
    {
        CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        if(ctx->arena) { cudaFree(ctx->arena); ctx->arena = nullptr; ctx->arena_bytes = 0; }
        // A little head-room, so that a slightly larger request later (another deal of the partitions, say) does not regrow the
        // arena: other GPUs may still hold a mapping of it, and its memory is not given back before they let go.
        const size_t want = bytes + bytes / 16;
        cudaError_t e = cudaMalloc(&ctx->arena, want);
        if(e == cudaSuccess) bytes = want;
        else { cudaGetLastError(); e = cudaMalloc(&ctx->arena, bytes); }
        if(e != cudaSuccess)
        {
            cudaGetLastError();
            ctx->err = "device allocation of " + std::to_string(bytes) + " bytes failed: " + cudaGetErrorString(e);
            return CSA_E_NOMEM;
        }
        ctx->arena_bytes = bytes;
    }
    *out = ctx->arena;
    return CSA_OK;
}

int csa_aux(csa_ctx* ctx, size_t bytes, void** out)
{
    if(bytes > ctx->aux_bytes)
    {
        CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        if(ctx->aux) { cudaFree(ctx->aux); ctx->aux = nullptr; ctx->aux_bytes = 0; }
        const cudaError_t e = cudaMalloc(&ctx->aux, bytes);
        if(e != cudaSuccess)
        {
            cudaGetLastError();
            ctx->err = "device allocation of " + std::to_string(bytes) + " bytes failed: " + cudaGetErrorString(e);
            return CSA_E_NOMEM;
        }
        ctx->aux_bytes = bytes;
    }
    *out = ctx->aux;
    return CSA_OK;
}

int csa_host_aux(csa_ctx* ctx, size_t bytes, void** out)
{
    if(bytes > ctx->host_aux_bytes)
    {
        CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        if(ctx->host_aux) { cudaFreeHost(ctx->host_aux); ctx->host_aux = nullptr; ctx->host_aux_bytes = 0; }
        const cudaError_t e = cudaMallocHost(&ctx->host_aux, bytes);
        if(e != cudaSuccess)
        {
            cudaGetLastError();
            ctx->err = "pinned host allocation of " + std::to_string(bytes) + " bytes failed: " + cudaGetErrorString(e);
            return CSA_E_NOMEM;
        }
        ctx->host_aux_bytes = bytes;
    }
    *out = ctx->host_aux;
    return CSA_OK;
}
