// Least-significant-digit radix sort of (64-bit key, 32- or 64-bit value) records, 8 bits per pass, each pass
// ONE sweep over the records: a tile ranks its records by digit with warp-level multisplit (match.any), publishes
// its per-digit counts, finds its global offsets by looking back over the tiles before it (decoupled look-back),
// stages the records in shared memory in digit order and writes them out in coalesced runs.
//
// It stands where the reference calls cub::DeviceRadixSort::SortPairs (src/GPU_SACA.cu:1175, 1203, 1783, 1849);
// no library sort is used.
#include "common.cuh"
#include "sort.cuh"

#include <vector>

namespace
{

constexpr int RADIX_BITS = 8;
constexpr int RADIX = 1 << RADIX_BITS;
constexpr u32 FLAG_SHIFT = 30;
constexpr u32 COUNT_MASK = (1u << FLAG_SHIFT) - 1;
constexpr u32 FLAG_AGGREGATE = 1u << FLAG_SHIFT;
constexpr u32 FLAG_PREFIX = 2u << FLAG_SHIFT;
constexpr u64 PORTION = 1ull << 29;         // records per launch of a pass: tile counts stay below 2^30
constexpr u32 LOOKBACK_SPIN_LIMIT = 1u << 22;

// Digit histograms of every pass in one read of the keys. hist holds [passes][RADIX] 32-bit counts for this portion.
template <int BLOCK>
__global__ void __launch_bounds__(BLOCK) histogram_kernel(const u64* __restrict__ keys, const u64 n, const int begin_bit, const int passes,
                                                         u32* __restrict__ hist)
{
    __shared__ u32 h[8 * RADIX];
    for(int i = threadIdx.x; i < passes * RADIX; i += BLOCK) h[i] = 0;
    __syncthreads();

    const u64 pairs = n >> 1;   // 128-bit loads of two keys
    const ulonglong2* k2 = reinterpret_cast<const ulonglong2*>(keys);
    const u64 stride = u64(gridDim.x) * BLOCK;
    // Whole warps take part in every round so that the match instruction sees a full mask.
    const u64 rounds = (pairs + stride - 1) / stride;
    u64 i = u64(blockIdx.x) * BLOCK + threadIdx.x;
    for(u64 r = 0; r < rounds; ++r, i += stride)
    {
        const bool live = i < pairs;
        ulonglong2 v = make_ulonglong2(0, 0);
        if(live) v = k2[i];
        #pragma unroll 1
        for(int p = 0; p < passes; ++p)
        {
            const int sh = begin_bit + p * RADIX_BITS;
            const u32 d0 = live ? u32(v.x >> sh) & (RADIX - 1) : RADIX;       // RADIX = "no record"
            const u32 d1 = live ? u32(v.y >> sh) & (RADIX - 1) : RADIX;
            const u32 m0 = __match_any_sync(0xFFFFFFFFu, d0);
            const u32 m1 = __match_any_sync(0xFFFFFFFFu, d1);
            if(live)
            {
                if(lane_id() == u32(__ffs(m0) - 1)) atomicAdd(&h[p * RADIX + d0], __popc(m0));
                if(lane_id() == u32(__ffs(m1) - 1)) atomicAdd(&h[p * RADIX + d1], __popc(m1));
            }
        }
    }
    if((n & 1) && blockIdx.x == 0 && threadIdx.x == 0)
    {
        const u64 k = keys[n - 1];
        for(int p = 0; p < passes; ++p) atomicAdd(&h[p * RADIX + (u32(k >> (begin_bit + p * RADIX_BITS)) & (RADIX - 1))], 1u);
    }
    __syncthreads();
    for(int i2 = threadIdx.x; i2 < passes * RADIX; i2 += BLOCK)
        if(h[i2] != 0) atomicAdd(&hist[i2], h[i2]);
}

// From the portions' histograms: the global base offset of every (portion, pass, digit), and for every pass
// whether a single digit holds all n records (such a pass moves nothing and is skipped).
// hist: [portions][passes][RADIX] u32. base: same shape, u64. skip: [passes] u64.
__global__ void __launch_bounds__(RADIX) digit_base_kernel(const u32* __restrict__ hist, const int portions, const int passes, const u64 n,
                                                          u64* __restrict__ base, u64* __restrict__ skip)
{
    __shared__ u64 warp_tot[RADIX / 32];
    __shared__ int s_skip;
    const int p = blockIdx.x, d = threadIdx.x;
    if(d == 0) s_skip = 0;
    __syncthreads();
    u64 total = 0;
    for(int P = 0; P < portions; ++P) total += hist[(u64(P) * passes + p) * RADIX + d];
    if(total == n) s_skip = 1;
    // exclusive scan of `total` over the 256 digits
    u64 inc = total;
    for(int o = 1; o < 32; o <<= 1)
    {
        const u64 t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
        if(int(lane_id()) >= o) inc += t;
    }
    if(lane_id() == 31) warp_tot[d >> 5] = inc;
    __syncthreads();
    u64 pre = 0;
    for(int w = 0; w < (d >> 5); ++w) pre += warp_tot[w];
    u64 run = pre + inc - total;
    for(int P = 0; P < portions; ++P)
    {
        const u64 idx = (u64(P) * passes + p) * RADIX + d;
        base[idx] = run;
        run += hist[idx];
    }
    if(d == 0) skip[p] = u64(s_skip);
}

template <int BLOCK, int ITEMS, typename V>
struct Pass_Smem
{
    static constexpr int TILE = BLOCK * ITEMS;
    static constexpr int WARPS = BLOCK / 32;
    static constexpr size_t bytes = size_t(TILE) * 8 + size_t(TILE) * sizeof(V) + size_t(WARPS) * RADIX * 4 + RADIX * 4 + RADIX * 8 + 64;
};

// One digit pass over one portion of the records. status: [tiles][RADIX] words, zeroed before the launch;
// tile_counter: one zeroed word. digit_base: [RADIX] global offsets of this portion and pass.
template <int BLOCK, int ITEMS, typename V>
__global__ void __launch_bounds__(BLOCK) onesweep_pass_kernel(const u64* __restrict__ keys_in, u64* __restrict__ keys_out, const V* __restrict__ vals_in,
                                                             V* __restrict__ vals_out, const u64 n, const int shift,
                                                             const u64* __restrict__ digit_base, u32* __restrict__ status, u32* __restrict__ tile_counter,
                                                             u64* __restrict__ dev_status)
{
    constexpr int TILE = BLOCK * ITEMS;
    constexpr int WARPS = BLOCK / 32;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    u64* const stage_keys = reinterpret_cast<u64*>(smem_raw);
    V* const stage_vals = reinterpret_cast<V*>(smem_raw + size_t(TILE) * 8);
    u32* const warp_hist = reinterpret_cast<u32*>(smem_raw + size_t(TILE) * 8 + size_t(TILE) * sizeof(V));
    u32* const tile_excl = warp_hist + WARPS * RADIX;
    u64* const g_off = reinterpret_cast<u64*>(tile_excl + RADIX);
    u32* const misc = reinterpret_cast<u32*>(g_off + RADIX);   // [0] tile id, [1..8] warp totals of the digit scan

    const u32 tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    // Tiles are taken in launch order of the blocks that run, so that every tile a block waits on is already running.
    if(tid == 0) misc[0] = atomicAdd(tile_counter, 1u);
    for(int i = tid; i < WARPS * RADIX; i += BLOCK) warp_hist[i] = 0;
    __syncthreads();
    const u32 tile = misc[0];
    const u64 tile_base = u64(tile) * TILE;
    if(tile_base >= n) return;
    const u32 valid = (n - tile_base < u64(TILE)) ? u32(n - tile_base) : u32(TILE);

    // Warp-striped load: a warp owns 32 * ITEMS consecutive records; item i of lane l is record i * 32 + l of them.
    u64 key[ITEMS];
    const u32 warp_first = warp * 32 * ITEMS;
    #pragma unroll
    for(int i = 0; i < ITEMS; ++i)
    {
        const u32 idx = warp_first + i * 32 + lane;
        key[i] = (idx < valid) ? keys_in[tile_base + idx] : ~0ull;
    }

    // Rank of every record among the records of its digit within the warp, and the warp's digit counts.
    u16 rank[ITEMS];
    u32* const wh = warp_hist + warp * RADIX;
    #pragma unroll
    for(int i = 0; i < ITEMS; ++i)
    {
        const u32 d = u32(key[i] >> shift) & (RADIX - 1);
        const u32 peers = __match_any_sync(0xFFFFFFFFu, d);
        const u32 leader = __ffs(peers) - 1;
        u32 old = 0;
        if(lane == leader) { old = wh[d]; wh[d] = old + __popc(peers); }
        old = __shfl_sync(0xFFFFFFFFu, old, leader);
        rank[i] = u16(old + __popc(peers & lanemask_lt()));
        __syncwarp();
    }
    __syncthreads();

    // Per digit: exclusive offsets of the warps, and the tile's count. Records past the end carry digit 255 and
    // rank last, so they only have to leave the count.
    u32 count = 0;
    if(tid < RADIX)
    {
        u32 sum = 0;
        #pragma unroll
        for(int w = 0; w < WARPS; ++w)
        {
            const u32 t = warp_hist[w * RADIX + tid];
            warp_hist[w * RADIX + tid] = sum;
            sum += t;
        }
        if(tid == RADIX - 1) sum -= (u32(TILE) - valid);
        count = sum;
        st_relaxed_u32(status + u64(tile) * RADIX + tid, (tile == 0 ? FLAG_PREFIX : FLAG_AGGREGATE) | count);
    }

    // Exclusive scan of the tile's digit counts.
    {
        u32 inc = count;
        if(tid < RADIX)
        {
            #pragma unroll
            for(int o = 1; o < 32; o <<= 1)
            {
                const u32 t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
                if(int(lane) >= o) inc += t;
            }
            if(lane == 31) misc[1 + warp] = inc;
        }
        __syncthreads();
        if(tid < RADIX)
        {
            u32 pre = 0;
            for(u32 w = 0; w < warp; ++w) pre += misc[1 + w];
            tile_excl[tid] = pre + inc - count;
        }
    }

    // Look back over the tiles before this one for the records of this digit that precede the tile.
    if(tid < RADIX)
    {
        u32 before = 0;
        if(tile > 0)
        {
            bool gave_up = false;
            for(long long t = (long long)tile - 1; t >= 0; --t)
            {
                const u32* const slot = status + u64(t) * RADIX + tid;
                u32 s = ld_relaxed_u32(slot);
                u32 spins = 0;
                while((s >> FLAG_SHIFT) == 0)
                {
                    if(++spins > LOOKBACK_SPIN_LIMIT || ((spins & 255u) == 0 && (ld_relaxed_u64(dev_status) & CSA_ST_LOOKBACK_TIMEOUT)))
                    {
                        gave_up = true;
                        break;
                    }
                    __nanosleep(40);
                    s = ld_relaxed_u32(slot);
                }
                if(gave_up) break;
                before += s & COUNT_MASK;
                if((s >> FLAG_SHIFT) == 2) break;
            }
            if(gave_up) atomicOr(dev_status, (u64)CSA_ST_LOOKBACK_TIMEOUT);
            st_relaxed_u32(status + u64(tile) * RADIX + tid, FLAG_PREFIX | ((before + count) & COUNT_MASK));
        }
        g_off[tid] = digit_base[tid] + before - tile_excl[tid];
    }
    __syncthreads();

    // Stage the records in digit order.
    #pragma unroll
    for(int i = 0; i < ITEMS; ++i)
    {
        const u32 d = u32(key[i] >> shift) & (RADIX - 1);
        const u32 pos = tile_excl[d] + wh[d] + rank[i];
        const u32 idx = warp_first + i * 32 + lane;
        rank[i] = u16(pos);
        if(idx < valid) stage_keys[pos] = key[i];
    }
    #pragma unroll
    for(int i = 0; i < ITEMS; ++i)
    {
        const u32 idx = warp_first + i * 32 + lane;
        if(idx < valid) stage_vals[rank[i]] = vals_in[tile_base + idx];
    }
    __syncthreads();

    // Write out: consecutive threads write consecutive records of a digit's run.
    #pragma unroll
    for(int k = 0; k < ITEMS; ++k)
    {
        const u32 p = tid + k * BLOCK;
        if(p < valid)
        {
            const u64 kk = stage_keys[p];
            const u64 dst = g_off[u32(kk >> shift) & (RADIX - 1)] + p;
            keys_out[dst] = kk;
            vals_out[dst] = stage_vals[p];
        }
    }
}

template <int BLOCK, int ITEMS, typename V>
int launch_pass(csa_ctx* ctx, const u64* kin, u64* kout, const V* vin, V* vout, u64 n, int shift, const u64* digit_base, u32* status, u32* counter)
{
    using S = Pass_Smem<BLOCK, ITEMS, V>;
    static bool configured[64] = {false};
    auto kern = onesweep_pass_kernel<BLOCK, ITEMS, V>;
    if(!configured[ctx->device & 63])
    {
        CSA_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(S::bytes)));
        configured[ctx->device & 63] = true;
    }
    const u64 tiles = div_up(n, S::TILE);
    CSA_CUDA(ctx, cudaMemsetAsync(status, 0, tiles * RADIX * sizeof(u32), ctx->stream));
    CSA_CUDA(ctx, cudaMemsetAsync(counter, 0, sizeof(u32), ctx->stream));
    kern<<<unsigned(tiles), BLOCK, S::bytes, ctx->stream>>>(kin, kout, vin, vout, n, shift, digit_base, status, counter, ctx->d_status);
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

constexpr int PASS_BLOCK = 256;
constexpr int PASS_ITEMS = 16;
constexpr int PASS_TILE = PASS_BLOCK * PASS_ITEMS;

struct Pass_Timer
{
    bool on = false;
    std::vector<cudaEvent_t> ev;    // pairs
    u64 passes = 0, records = 0;
};
Pass_Timer g_timer[64];

}   // namespace

size_t csa_sort_workspace_bytes(uint64_t n)
{
    const u64 portions = n == 0 ? 1 : div_up(n, PORTION);
    const u64 tiles = div_up(n < PORTION ? n : PORTION, PASS_TILE) + 1;
    return size_t(tiles) * RADIX * 4 + 256            // tile status
         + 256                                         // tile counter
         + size_t(portions) * 8 * RADIX * 4 + 256      // histograms
         + size_t(portions) * 8 * RADIX * 8 + 256      // digit bases
         + 4096;
}

int csa_set_pass_timing(csa_ctx* ctx, int on)
{
    if(!ctx) return CSA_E_INVALID;
    g_timer[ctx->device & 63].on = on != 0;
    return CSA_OK;
}

int csa_get_pass_timing(csa_ctx* ctx, double* total_ms, uint64_t* passes, uint64_t* records)
{
    if(!ctx) return CSA_E_INVALID;
    Pass_Timer& t = g_timer[ctx->device & 63];
    CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    double ms = 0;
    for(size_t i = 0; i + 1 < t.ev.size(); i += 2)
    {
        float e = 0;
        CSA_CUDA(ctx, cudaEventElapsedTime(&e, t.ev[i], t.ev[i + 1]));
        ms += e;
    }
    if(total_ms) *total_ms = ms;
    if(passes) *passes = t.passes;
    if(records) *records = t.records;
    return CSA_OK;
}

void sort_reset_timing(csa_ctx* ctx)
{
    Pass_Timer& t = g_timer[ctx->device & 63];
    for(auto e : t.ev) cudaEventDestroy(e);
    t.ev.clear();
    t.passes = t.records = 0;
}

int csa_sort_pairs(csa_ctx* ctx, uint64_t* keys, uint64_t* keys_alt, void* vals, void* vals_alt, uint32_t val_bytes, uint64_t n,
                   int begin_bit, int end_bit, void* workspace, size_t workspace_bytes, int* in_alt)
{
    if(!ctx || !in_alt) return CSA_E_INVALID;
    *in_alt = 0;
    if(begin_bit < 0 || end_bit > 64 || begin_bit > end_bit || (val_bytes != 4 && val_bytes != 8)) return csa_fail(ctx, CSA_E_INVALID, "csa_sort_pairs: bad bit range or value width");
    if(n <= 1 || begin_bit == end_bit) return CSA_OK;
    if(!keys || !keys_alt || !vals || !vals_alt || !workspace) return csa_fail(ctx, CSA_E_INVALID, "csa_sort_pairs: null buffer");
    if(workspace_bytes < csa_sort_workspace_bytes(n)) return csa_fail(ctx, CSA_E_NOMEM, "csa_sort_pairs: workspace too small");
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));

    const int passes = (end_bit - begin_bit + RADIX_BITS - 1) / RADIX_BITS;
    const int portions = int(div_up(n, PORTION));
    Carver cv(workspace, workspace_bytes);
    const u64 tiles_max = div_up(n < PORTION ? n : PORTION, PASS_TILE) + 1;
    u32* status = cv.take<u32>(tiles_max * RADIX);
    u32* counter = cv.take<u32>(64);
    u32* hist = cv.take<u32>(u64(portions) * 8 * RADIX);
    u64* base = cv.take<u64>(u64(portions) * 8 * RADIX);
    if(!cv.ok) return csa_fail(ctx, CSA_E_NOMEM, "csa_sort_pairs: workspace too small");

    CSA_CUDA(ctx, cudaMemsetAsync(hist, 0, u64(portions) * passes * RADIX * sizeof(u32), ctx->stream));
    for(int P = 0; P < portions; ++P)
    {
        const u64 first = u64(P) * PORTION, cnt = (n - first < PORTION ? n - first : PORTION);
        const unsigned blocks = unsigned(cnt / (2 * 256 * 8) < 1 ? 1 : (cnt / (2 * 256 * 8) > 148 * 8 ? 148 * 8 : cnt / (2 * 256 * 8)));
        histogram_kernel<256><<<blocks, 256, 0, ctx->stream>>>(reinterpret_cast<const u64*>(keys) + first, cnt, begin_bit, passes, hist + u64(P) * passes * RADIX);
        CSA_LAUNCH_CHECK(ctx);
    }
    u64* d_skip = ctx->d_scalars + 32;
    digit_base_kernel<<<passes, RADIX, 0, ctx->stream>>>(hist, portions, passes, n, base, d_skip);
    CSA_LAUNCH_CHECK(ctx);
    CSA_CUDA(ctx, cudaMemcpyAsync(ctx->h_scalars + 32, d_skip, passes * sizeof(u64), cudaMemcpyDeviceToHost, ctx->stream));
    CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    u64 skip[8];
    for(int p = 0; p < passes; ++p) skip[p] = ctx->h_scalars[32 + p];

    Pass_Timer& timer = g_timer[ctx->device & 63];
    u64* kin = reinterpret_cast<u64*>(keys); u64* kout = reinterpret_cast<u64*>(keys_alt);
    void* vin = vals; void* vout = vals_alt;
    int flips = 0;
    for(int p = 0; p < passes; ++p)
    {
        if(skip[p]) continue;
        const int shift = begin_bit + p * RADIX_BITS;
        cudaEvent_t e0 = nullptr, e1 = nullptr;
        if(timer.on)
        {
            CSA_CUDA(ctx, cudaEventCreate(&e0));
            CSA_CUDA(ctx, cudaEventCreate(&e1));
            CSA_CUDA(ctx, cudaEventRecord(e0, ctx->stream));
        }
        for(int P = 0; P < portions; ++P)
        {
            const u64 first = u64(P) * PORTION, cnt = (n - first < PORTION ? n - first : PORTION);
            const u64* db = base + (u64(P) * passes + p) * RADIX;
            if(val_bytes == 4)
                CSA_TRY((launch_pass<PASS_BLOCK, PASS_ITEMS, u32>(ctx, kin + first, kout, static_cast<const u32*>(vin) + first, static_cast<u32*>(vout), cnt, shift, db, status, counter)));
            else
                CSA_TRY((launch_pass<PASS_BLOCK, PASS_ITEMS, u64>(ctx, kin + first, kout, static_cast<const u64*>(vin) + first, static_cast<u64*>(vout), cnt, shift, db, status, counter)));
        }
        if(timer.on)
        {
            CSA_CUDA(ctx, cudaEventRecord(e1, ctx->stream));
            timer.ev.push_back(e0); timer.ev.push_back(e1);
            timer.passes++; timer.records += n;
        }
        ctx->counters[1]++;          // digit passes
        ctx->counters[2] += n;       // records moved
        u64* tk = kin; kin = kout; kout = tk;
        void* tv = vin; vin = vout; vout = tv;
        ++flips;
    }
    *in_alt = flips & 1;
    return CSA_OK;
}
