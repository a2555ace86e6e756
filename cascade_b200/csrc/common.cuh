// Shared declarations of the device library: the context, status codes, launch checks and small
// device helpers. Everything here is internal; the public C ABI is include/cascade_b200.h.
#pragma once

#include "../../include/cascade_b200.h"

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>

typedef unsigned long long u64;
typedef unsigned int u32;
typedef unsigned short u16;
typedef unsigned char u8;

// Bits of the device status word (csa_sync reports them).
enum : u64
{
    CSA_ST_LOOKBACK_TIMEOUT = 1ull << 0,   // a bounded wait on a predecessor tile ran out
    CSA_ST_BULK_TIMEOUT     = 1ull << 1,   // a bounded wait on a bulk shared-memory copy ran out
    CSA_ST_RANGE            = 1ull << 2,   // an index fell outside its array; the access was skipped
    CSA_ST_UNSERVED         = 1ull << 3,   // an invariant of the doubling step did not hold
};

// One per (device, host thread): a stream, the device status word, a grow-only scratch arena and pinned
// scalars for the small device-to-host reads of the build loop.
struct csa_ctx
{
    int device = 0;
    cudaStream_t stream = nullptr;
    u64* d_status = nullptr;       // device status word
    u64* h_scalars = nullptr;      // pinned, 64 words
    u64* d_scalars = nullptr;      // device, 64 words
    void* arena = nullptr;         // grow-only scratch
    size_t arena_bytes = 0;
    void* aux = nullptr;           // a second grow-only buffer, for data that must survive a regrowth of the arena
    size_t aux_bytes = 0;
    void* host_aux = nullptr;      // grow-only pinned host scratch (pinning gigabytes takes seconds: kept between builds)
    size_t host_aux_bytes = 0;
    std::string err;
    u64 counters[16] = {0};        // launch and byte counters for the benchmark
    const u32* symbol_range = nullptr;     // optional first-symbol table of csa_partition_ids (see partition_install_symbol_ranges)
    u32* symbol_table = nullptr;           // the table's memory where csa_install_pivots made it (65536 words, owned)
    bool ties_in_any_order = false;        // set by callers whose sorts may leave records of equal keys in any order (see radix_sort.cu)
    void* pass_timer = nullptr;            // digit-pass event timing of the sorts on this context (owned by radix_sort.cu)
    // Extra streams ("lanes") of the chunked host-batch pipelines, each with an event; made on first use.
    static constexpr int LANES = 3;
    cudaStream_t lane[LANES] = {nullptr, nullptr, nullptr};
    cudaEvent_t lane_event[LANES] = {nullptr, nullptr, nullptr};
    // Mappings of other GPUs' arenas opened through CUDA IPC (multi-GPU builds), kept while the peers' handles stay the same.
    void* peer_base[CSA_MAX_GPUS] = {nullptr};
    unsigned char peer_handle[CSA_MAX_GPUS][64] = {{0}};
    bool peer_open[CSA_MAX_GPUS] = {false};
};

// While one of these lives, the context's sorts may leave records of equal keys in any order (their first pass is then
// the cheap unordered one). The builds use it: tied suffixes are re-sorted by the next generation anyway.
struct Ties_In_Any_Order
{
    csa_ctx* ctx;
    explicit Ties_In_Any_Order(csa_ctx* c) : ctx(c) { ctx->ties_in_any_order = true; }
    ~Ties_In_Any_Order() { ctx->ties_in_any_order = false; }
    Ties_In_Any_Order(const Ties_In_Any_Order&) = delete;
    Ties_In_Any_Order& operator=(const Ties_In_Any_Order&) = delete;
};

#define CSA_CUDA(ctx, call)                                                                             \
    do {                                                                                                \
        const cudaError_t e_ = (call);                                                                  \
        if(e_ != cudaSuccess)                                                                           \
        {                                                                                               \
            (ctx)->err = std::string(#call) + ": " + cudaGetErrorString(e_);                            \
            return CSA_E_CUDA;                                                                          \
        }                                                                                               \
    } while(0)

#define CSA_TRY(expr)                       \
    do {                                    \
        const int r_ = (expr);              \
        if(r_ != CSA_OK) return r_;         \
    } while(0)

#define CSA_LAUNCH_CHECK(ctx)                                                                           \
    do {                                                                                                \
        const cudaError_t e_ = cudaGetLastError();                                                      \
        if(e_ != cudaSuccess)                                                                           \
        {                                                                                               \
            (ctx)->err = std::string("kernel launch at ") + __FILE__ + ":" + std::to_string(__LINE__)   \
                         + ": " + cudaGetErrorString(e_);                                               \
            return CSA_E_CUDA;                                                                          \
        }                                                                                               \
        (ctx)->counters[0]++;                                                                           \
    } while(0)

static inline int csa_fail(csa_ctx* ctx, int code, const std::string& why)
{
    if(ctx) ctx->err = why;
    return code;
}

// Makes the context's lanes (streams and events) if they do not exist yet.
int csa_lanes(csa_ctx* ctx);

// While one of these lives, the context's calls are queued on another stream than its own.
struct On_Stream
{
    csa_ctx* ctx;
    cudaStream_t saved;
    On_Stream(csa_ctx* c, cudaStream_t s) : ctx(c), saved(c->stream) { c->stream = s; }
    ~On_Stream() { ctx->stream = saved; }
    On_Stream(const On_Stream&) = delete;
    On_Stream& operator=(const On_Stream&) = delete;
};

// Returns in *out a scratch pointer of at least `bytes` bytes from the context's grow-only arena.
int csa_arena(csa_ctx* ctx, size_t bytes, void** out);
int csa_aux(csa_ctx* ctx, size_t bytes, void** out);
int csa_host_aux(csa_ctx* ctx, size_t bytes, void** out);

static inline size_t align_up256(size_t b) { return (b + 255) & ~size_t(255); }
static inline u64 div_up(u64 a, u64 b) { return (a + b - 1) / b; }
static inline int bits_for(u64 max_value) { int b = 0; while(b < 64 && (max_value >> b) != 0) ++b; return b; }   // bits to hold max_value

// A bump allocator over a caller's workspace, 256-byte aligned pieces.
struct Carver
{
    char* p; size_t left; bool ok = true;
    Carver(void* base, size_t bytes) : p(static_cast<char*>(base)), left(bytes) {}
    template <typename T> T* take(u64 count)
    {
        const size_t b = (count * sizeof(T) + 255) & ~size_t(255);
        if(b > left) { ok = false; return nullptr; }
        T* r = reinterpret_cast<T*>(p); p += b; left -= b; return r;
    }
};

#ifdef __CUDACC__

__device__ __forceinline__ u32 lane_id() { return threadIdx.x & 31; }
__device__ __forceinline__ u32 lanemask_lt() { u32 m; asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m)); return m; }

__device__ __forceinline__ u32 ld_relaxed_u32(const u32* p)
{
    u32 v; asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v;
}
__device__ __forceinline__ void st_relaxed_u32(u32* p, u32 v)
{
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ u64 ld_relaxed_u64(const u64* p)
{
    u64 v; asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory"); return v;
}

// The 4 symbols T[i, i+4) packed most-significant first: numeric order of the word = order of the symbols.
// T must be readable up to i + 4.
__device__ __forceinline__ u64 pack4(const u16* T, u64 i)
{
    return (u64(T[i]) << 48) | (u64(T[i + 1]) << 32) | (u64(T[i + 2]) << 16) | u64(T[i + 3]);
}

// 5-byte little-endian entry at rank r of an array whose base is 4-byte aligned and which is readable up to
// the 4-byte word past the entry.
__device__ __forceinline__ u64 sa40_load(const u8* sa, u64 r)
{
    const u64 b = 5 * r;
    const u32* w = reinterpret_cast<const u32*>(sa + (b & ~u64(3)));
    const u64 v = (u64(__ldg(w + 1)) << 32) | __ldg(w);
    return (v >> ((b & 3) * 8)) & 0xFFFFFFFFFFull;
}

#endif
