// Least-significant-digit radix sort of (64-bit key, 32- or 64-bit value) records, 8 bits per pass, each pass
// ONE sweep over the records: a tile ranks its records by digit with warp-level multisplit (match.any), publishes
// its per-digit counts, finds its global offsets by looking back over the tiles before it (decoupled look-back),
// stages the records in shared memory in digit order and writes them out in coalesced runs.
// Every pass is stable. Where the caller accepts records of equal keys in any order (the suffix-array builds do), the
// first pass is replaced by a cheaper unordered one (first_pass_kernel below): it has no earlier order to keep.
//
// It stands where the reference calls cub::DeviceRadixSort::SortPairs (src/GPU_SACA.cu:1175, 1203, 1783, 1849);
// no library sort is used.
#include "common.cuh"
#include "sort.cuh"

#include <algorithm>
#include <atomic>
#include <vector>

namespace
{

constexpr int RADIX_BITS = 8;
constexpr int RADIX = 1 << RADIX_BITS;
constexpr u32 FLAG_SHIFT = 30;
constexpr u32 COUNT_MASK = (1u << FLAG_SHIFT) - 1;
constexpr u32 FLAG_AGGREGATE = 1u << FLAG_SHIFT;
constexpr u32 FLAG_PREFIX = 2u << FLAG_SHIFT;
u64 PORTION = 1ull << 29;                   // records per launch of a pass: tile counts stay below 2^30 (tests may lower it)
constexpr u32 LOOKBACK_SPIN_LIMIT = 1u << 22;
// The limit that the kernels read (a test lowers it through csa_debug_set so that a wait which cannot succeed ends at once).
__device__ u32 g_lookback_spin_limit = LOOKBACK_SPIN_LIMIT;
u32 g_first_tile = 0;                        // test hook: value that a pass's tile counter starts from (0 in every real run)
constexpr int LOOKBACK_BATCH = 8;
constexpr int GAVE_UP_WORD = 32;           // word of a block's scratch words in shared memory that says a look-back wait ran out
constexpr int HIST_UNROLL = 4;             // 16-byte loads in flight per thread of the histogram kernel

// The digit of a pass that starts at bit `shift` holds min(8, end_bit - shift) bits.
__host__ __device__ __forceinline__ u32 digit_mask(int shift, int end_bit)
{
    const int w = end_bit - shift;
    return w >= RADIX_BITS ? u32(RADIX - 1) : ((1u << w) - 1);
}

// Digit histograms of every pass in one read of the keys. hist holds [passes][RADIX] 64-bit counts of the whole array.
template <int BLOCK>
__device__ __forceinline__ void histogram_body(const u64* __restrict__ keys, const u64 n, const int begin_bit, const int end_bit, const int passes,
                                               u64* __restrict__ hist, const u64 pass_stride, const u32 block_index, const u32 block_count)
{
    // One private histogram per warp keeps the shared-memory atomics of different warps apart; lanes of a warp that
    // hold the same digit still meet, and when all 32 do (a digit that is constant over long stretches, as the high bytes
    // of token ids are) one lane counts for the warp.
    constexpr int WARPS = BLOCK / 32;
    extern __shared__ u32 h[];                       // [WARPS][passes][RADIX]
    const int per_warp = passes * RADIX;
    for(int i = threadIdx.x; i < WARPS * per_warp; i += BLOCK) h[i] = 0;
    __syncthreads();
    u32* const mine = h + (threadIdx.x >> 5) * per_warp;

    // 128-bit loads of two keys, HIST_UNROLL of them in flight per thread: the kernel is a single read of the keys and
    // needs tens of KB outstanding per SM to keep the memory busy. A key is shifted and masked to its sorted bits once,
    // after which the digit of pass p is byte p of it.
    // A list that starts on an odd 8-byte boundary leaves its first key to the scalar tail below.
    const u64 odd_lead = (n > 0 && (reinterpret_cast<uintptr_t>(keys) & 8)) ? 1 : 0;
    const u64 pairs = (n - odd_lead) >> 1;
    const ulonglong2* k2 = reinterpret_cast<const ulonglong2*>(keys + odd_lead);
    const int width = end_bit - begin_bit;
    const u64 width_mask = width >= 64 ? ~0ull : ((1ull << width) - 1);
    const u64 chunk = u64(BLOCK) * HIST_UNROLL;
    const u64 stride = u64(block_count) * chunk;
    const u64 rounds = (pairs + stride - 1) / stride;       // whole warps take part in every round: the votes see a full mask
    u64 i = u64(block_index) * chunk + threadIdx.x;
    for(u64 r = 0; r < rounds; ++r, i += stride)
    {
        u64 k[2 * HIST_UNROLL];
        bool live[HIST_UNROLL];
        bool mine_live = true;
        #pragma unroll
        for(int j = 0; j < HIST_UNROLL; ++j)
        {
            live[j] = i + u64(j) * BLOCK < pairs;
            mine_live = mine_live && live[j];
            ulonglong2 v = make_ulonglong2(0, 0);
            if(live[j]) v = k2[i + u64(j) * BLOCK];
            k[2 * j] = (v.x >> begin_bit) & width_mask;
            k[2 * j + 1] = (v.y >> begin_bit) & width_mask;
        }
        // Bits in which any key of the warp differs from the first key of lane 0: a pass whose byte of them is zero has one
        // digit in the whole warp (the high bytes of token ids over long stretches), and one lane counts for all.
        const u64 k0 = __shfl_sync(0xFFFFFFFFu, k[0], 0);
        u64 diff = 0;
        #pragma unroll
        for(int j = 0; j < 2 * HIST_UNROLL; ++j) diff |= k[j] ^ k0;
        const u32 diff_lo = __reduce_or_sync(0xFFFFFFFFu, u32(diff)), diff_hi = __reduce_or_sync(0xFFFFFFFFu, u32(diff >> 32));
        const bool all_live = __all_sync(0xFFFFFFFFu, mine_live);
        #pragma unroll
        for(int p = 0; p < 8; ++p)
        {
            if(p >= passes) break;
            const u32 dbyte = ((p < 4 ? diff_lo : diff_hi) >> (8 * (p & 3))) & 0xFFu;
            if(all_live && dbyte == 0)
            {
                if(lane_id() == 0) atomicAdd(&mine[p * RADIX + (u32(k0 >> (8 * p)) & 0xFFu)], u32(64 * HIST_UNROLL));
            }
            else
            {
                #pragma unroll
                for(int j = 0; j < HIST_UNROLL; ++j)
                    if(live[j])
                    {
                        atomicAdd(&mine[p * RADIX + (u32(k[2 * j] >> (8 * p)) & 0xFFu)], 1u);
                        atomicAdd(&mine[p * RADIX + (u32(k[2 * j + 1] >> (8 * p)) & 0xFFu)], 1u);
                    }
            }
        }
    }
    if(block_index == 0 && threadIdx.x == 0)
    {
        // the keys outside the 16-byte pairs: the first of an odd start, the last of an odd remainder
        u64 rest[2];
        int rests = 0;
        if(odd_lead) rest[rests++] = keys[0];
        if((n - odd_lead) & 1) rest[rests++] = keys[n - 1];
        for(int e = 0; e < rests; ++e)
            for(int p = 0; p < passes; ++p)
                atomicAdd(&mine[p * RADIX + (u32(rest[e] >> (begin_bit + p * RADIX_BITS)) & digit_mask(begin_bit + p * RADIX_BITS, end_bit))], 1u);
    }
    __syncthreads();
    for(int i2 = threadIdx.x; i2 < per_warp; i2 += BLOCK)
    {
        u32 t = 0;
        #pragma unroll
        for(int w = 0; w < WARPS; ++w) t += h[w * per_warp + i2];
        if(t != 0) atomicAdd(&hist[u64(i2 / RADIX) * pass_stride + (i2 % RADIX)], u64(t));
    }
}

template <int BLOCK>
__global__ void __launch_bounds__(BLOCK) histogram_kernel(const u64* __restrict__ keys, const u64 n, const int begin_bit, const int end_bit, const int passes,
                                                         u64* __restrict__ hist)
{
    histogram_body<BLOCK>(keys, n, begin_bit, end_bit, passes, hist, RADIX, blockIdx.x, gridDim.x);
}

// The same for many segments of one array in one launch: blockIdx.y is the segment, hist is [passes][segments][RADIX].
template <int BLOCK>
__global__ void __launch_bounds__(BLOCK) seg_histogram_kernel(const u64* __restrict__ keys, const u64* __restrict__ seg_off, const u32 segs, const int begin_bit,
                                                             const int end_bit, const int passes, u64* __restrict__ hist)
{
    const u32 s = blockIdx.y;
    const u64 first = seg_off[s], count = seg_off[s + 1] - first;
    if(count == 0) return;
    histogram_body<BLOCK>(keys + first, count, begin_bit, end_bit, passes, hist + u64(s) * RADIX, u64(segs) * RADIX, blockIdx.x, gridDim.x);
}

// From the histograms: for every pass the global offset of each digit's first record (what the first launch of the pass
// starts from; a later launch starts from the offsets that the launch before it leaves behind), and whether a single
// digit holds all n records (such a pass moves nothing and is skipped).
// hist: [passes][RADIX]. base: [passes][launches + 1][RADIX], of which slot 0 is written here. skip: [passes].
__global__ void __launch_bounds__(RADIX) digit_base_kernel(const u64* __restrict__ hist, const int launches, const u64 n,
                                                          u64* __restrict__ base, u64* __restrict__ skip)
{
    __shared__ u64 warp_tot[RADIX / 32];
    __shared__ int s_skip;
    const int p = blockIdx.x, d = threadIdx.x;
    if(d == 0) s_skip = 0;
    __syncthreads();
    const u64 total = hist[u64(p) * RADIX + d];
    if(total == n) s_skip = 1;
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
    base[(u64(p) * (launches + 1)) * RADIX + d] = pre + inc - total;
    if(d == 0) skip[p] = u64(s_skip);
}

template <int BLOCK, int ITEMS, typename V>
struct Pass_Smem
{
    static constexpr int TILE = BLOCK * ITEMS;
    static constexpr int WARPS = BLOCK / 32;
    static constexpr size_t bytes = size_t(TILE) * 8 + size_t(TILE) * sizeof(V) + size_t(WARPS) * RADIX * 4 + RADIX * 4 + RADIX * 8 + 256;
};

// One digit pass over one launch's share of the records. status: [tiles][RADIX] words, zeroed before the launch;
// tile_counter: one zeroed word. digit_base: [RADIX] global offsets at which this launch's records of each digit start;
// the launch's last tile leaves in next_base the offsets at which the next launch's start.
template <int BLOCK, int ITEMS, typename V, int MATCH_BITS, bool FULL>
__device__ __forceinline__ void onesweep_tile(const u64* __restrict__ keys_in, u64* __restrict__ keys_out, const V* __restrict__ vals_in,
                                              V* __restrict__ vals_out, const u64 n, const int shift, const u32 dmask,
                                              const u64* __restrict__ digit_base, u64* __restrict__ next_base, u32* __restrict__ status,
                                              u64* __restrict__ dev_status, const u32 tile, const u32 valid_records, const u32 first_tile, const u64 tile_base)
{
    // tile: the tile's index among the status words; first_tile: the index of the first tile of the run of records that this
    // tile belongs to (0 for a sort of one array; a segment's first tile in a segmented sort: nothing before it is looked at);
    // tile_base: the tile's first record; n: the end of the run.
    constexpr int TILE = BLOCK * ITEMS;
    constexpr int WARPS = BLOCK / 32;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    u64* const stage_keys = reinterpret_cast<u64*>(smem_raw);
    V* const stage_vals = reinterpret_cast<V*>(smem_raw + size_t(TILE) * 8);
    u32* const warp_hist = reinterpret_cast<u32*>(smem_raw + size_t(TILE) * 8 + size_t(TILE) * sizeof(V));
    u32* const tile_excl = warp_hist + WARPS * RADIX;
    u64* const g_off = reinterpret_cast<u64*>(tile_excl + RADIX);
    u32* const misc = reinterpret_cast<u32*>(g_off + RADIX);   // [0] tile id, [1..] warp totals of the digit scan

    const u32 tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const u32 valid = FULL ? u32(TILE) : valid_records;     // a full tile needs no bounds checks

    // Warp-striped load: a warp owns 32 * ITEMS consecutive records; item i of lane l is record i * 32 + l of them.
    // Keys and values are requested together so that one memory round trip covers both.
    u64 key[ITEMS];
    V val[ITEMS];
    const u32 warp_first = warp * 32 * ITEMS;
    #pragma unroll
    for(int i = 0; i < ITEMS; ++i)
    {
        const u32 idx = warp_first + i * 32 + lane;
        key[i] = (FULL || idx < valid) ? keys_in[tile_base + idx] : ~0ull;
    }
    #pragma unroll
    for(int i = 0; i < ITEMS; ++i)
    {
        const u32 idx = warp_first + i * 32 + lane;
        if(vals_in != nullptr && (FULL || idx < valid)) val[i] = vals_in[tile_base + idx];
    }

    // Rank of every record among the records of its digit within the warp, and the warp's digit counts. The lanes that
    // hold a digit find one another (warp-level multisplit): the high bits of the digit by one match.any, whose cost grows
    // with the number of distinct values, and the low bits by one ballot each; the lowest lane of a group adds the group's
    // size to the warp's counter of the digit and hands the old value round. The steps run as separate sweeps over the
    // items so that their latencies overlap; shared-memory atomics of one warp take effect in program order, which keeps
    // the ranks stable.
    // Ranks are below the tile size (at most 8192), so two share a register; digits are taken from the keys again where
    // needed; the sweeps run over chunks of 8 items so that their temporaries stay few: this leaves registers for more
    // items per thread, i.e. larger tiles with longer runs per digit and fewer look-backs per record.
    u32 rank2[(ITEMS + 1) / 2];
    u32* const wh = warp_hist + warp * RADIX;
    constexpr int CHUNK = 8;
    #pragma unroll
    for(int c = 0; c < ITEMS; c += CHUNK)
    {
        u32 peers[CHUNK], old[CHUNK];
        #pragma unroll
        for(int j = 0; j < CHUNK; ++j)
        {
            if(c + j >= ITEMS) break;
            const u32 d = u32(key[c + j] >> shift) & dmask;
            u32 m = (MATCH_BITS > 0) ? __match_any_sync(0xFFFFFFFFu, d >> (RADIX_BITS - MATCH_BITS)) : 0xFFFFFFFFu;
            #pragma unroll
            for(int b = 0; b < RADIX_BITS - MATCH_BITS; ++b)
            {
                const u32 sel = 0u - ((d >> b) & 1u);                       // all ones if the bit is set
                const u32 v = __ballot_sync(0xFFFFFFFFu, sel != 0);
                m &= ~(v ^ sel);                                            // lanes whose bit equals this lane's
            }
            peers[j] = m;
        }
        #pragma unroll
        for(int j = 0; j < CHUNK; ++j)
        {
            if(c + j >= ITEMS) break;
            old[j] = 0;
            if((peers[j] & lanemask_lt()) == 0) old[j] = atomicAdd(&wh[u32(key[c + j] >> shift) & dmask], u32(__popc(peers[j])));    // lowest lane of the group
        }
        #pragma unroll
        for(int j = 0; j < CHUNK; ++j)
        {
            if(c + j >= ITEMS) break;
            const u32 r = __shfl_sync(0xFFFFFFFFu, old[j], __ffs(peers[j]) - 1) + __popc(peers[j] & lanemask_lt());
            if(((c + j) & 1) == 0) rank2[(c + j) >> 1] = r; else rank2[(c + j) >> 1] |= r << 16;
        }
    }
    __syncthreads();

    // Per digit: the tile's count, then (after a scan of the counts over the digits) the offset within the tile at which
    // each warp's records of the digit start. Records past the end carry the largest digit and rank last, so they only
    // have to leave the count.
    u32 count = 0;
    u32 wcount[WARPS];
    if(tid < RADIX)
    {
        #pragma unroll
        for(int w = 0; w < WARPS; ++w) { wcount[w] = warp_hist[w * RADIX + tid]; count += wcount[w]; }
        if(!FULL && tid == dmask) count -= (u32(TILE) - valid);      // dmask is the digit of the all-ones filler key
        st_relaxed_u32(status + u64(tile) * RADIX + tid, (tile == first_tile ? FLAG_PREFIX : FLAG_AGGREGATE) | count);
    }
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
            u32 run = pre + inc - count;
            tile_excl[tid] = run;
            #pragma unroll
            for(int w = 0; w < WARPS; ++w) { warp_hist[w * RADIX + tid] = run; run += wcount[w]; }
        }
    }

    __syncthreads();

    // Look back over the tiles before this one for the records of this digit that precede the tile.
    if(tid < RADIX)
    {
        u32 before = 0;
        if(tile > first_tile)
        {
            // The status words of LOOKBACK_BATCH earlier tiles are requested at once, so that a long walk costs one memory
            // round trip per batch instead of one per tile; a word that is still empty is polled (with a bound) in place.
            bool gave_up = false, done = false;
            const u32 spin_limit = g_lookback_spin_limit;
            const long long t_first = (long long)first_tile;
            long long t = (long long)tile - 1;
            while(t >= t_first && !done && !gave_up)
            {
                u32 s[LOOKBACK_BATCH];
                #pragma unroll
                for(int j = 0; j < LOOKBACK_BATCH; ++j)
                    s[j] = (t - j >= t_first) ? ld_relaxed_u32(status + u64(t - j) * RADIX + tid) : FLAG_PREFIX;
                #pragma unroll
                for(int j = 0; j < LOOKBACK_BATCH; ++j)
                {
                    if(done || gave_up || t - j < t_first) break;
                    u32 v = s[j];
                    u32 spins = 0;
                    while((v >> FLAG_SHIFT) == 0)
                    {
                        if(++spins > spin_limit || ((spins & 255u) == 0 && (ld_relaxed_u64(dev_status) & CSA_ST_LOOKBACK_TIMEOUT)))
                        {
                            gave_up = true;
                            break;
                        }
                        __nanosleep(20);
                        v = ld_relaxed_u32(status + u64(t - j) * RADIX + tid);
                    }
                    if(gave_up) break;
                    before += v & COUNT_MASK;
                    if((v >> FLAG_SHIFT) == 2) done = true;
                }
                t -= LOOKBACK_BATCH;
            }
            if(gave_up) { atomicOr(dev_status, (u64)CSA_ST_LOOKBACK_TIMEOUT); misc[GAVE_UP_WORD] = 1; }
            // published even then, so that the tiles after this one end their waits too
            st_relaxed_u32(status + u64(tile) * RADIX + tid, FLAG_PREFIX | ((before + count) & COUNT_MASK));
        }
        const u64 db = digit_base[tid];
        if(next_base != nullptr && tile_base + TILE >= n) next_base[tid] = db + before + count;     // the last tile has seen every record of the launch
        g_off[tid] = db + before - tile_excl[tid];
    }
    __syncthreads();
    if(misc[GAVE_UP_WORD]) return;      // a wait ran out: the offsets are not known, nothing is written (the status word tells the host)

    // Stage the records in digit order.
    #pragma unroll
    for(int i = 0; i < ITEMS; ++i)
    {
        const u32 idx = warp_first + i * 32 + lane;
        const u32 pos = ((rank2[i >> 1] >> ((i & 1) * 16)) & 0xFFFFu) + wh[u32(key[i] >> shift) & dmask];
        if(FULL || idx < valid)
        {
            stage_keys[pos] = key[i];
            if(vals_in != nullptr) stage_vals[pos] = val[i];
        }
    }
    __syncthreads();

    // Write out: consecutive threads write consecutive records of a digit's run.
    #pragma unroll
    for(int k = 0; k < ITEMS; ++k)
    {
        const u32 p = tid + k * BLOCK;
        if(FULL || p < valid)
        {
            const u64 kk = stage_keys[p];
            const u64 dst = g_off[u32(kk >> shift) & dmask] + p;
            keys_out[dst] = kk;
            if(vals_in != nullptr) vals_out[dst] = stage_vals[p];
        }
    }
}

template <int BLOCK, int ITEMS, typename V, int MATCH_BITS>
__global__ void __launch_bounds__(BLOCK) onesweep_pass_kernel(const u64* __restrict__ keys_in, u64* __restrict__ keys_out, const V* __restrict__ vals_in,
                                                             V* __restrict__ vals_out, const u64 n, const int shift, const u32 dmask,
                                                             const u64* __restrict__ digit_base, u64* __restrict__ next_base, u32* __restrict__ status,
                                                             u32* __restrict__ tile_counter, u64* __restrict__ dev_status)
{
    constexpr int TILE = BLOCK * ITEMS;
    constexpr int WARPS = BLOCK / 32;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    u32* const warp_hist = reinterpret_cast<u32*>(smem_raw + size_t(TILE) * 8 + size_t(TILE) * sizeof(V));
    u32* const misc = reinterpret_cast<u32*>(smem_raw + size_t(TILE) * 8 + size_t(TILE) * sizeof(V) + size_t(WARPS) * RADIX * 4 + RADIX * 4 + RADIX * 8);

    // Tiles are taken in launch order of the blocks that run, so that every tile a block waits on is already running.
    if(threadIdx.x == 0) { misc[0] = atomicAdd(tile_counter, 1u); misc[GAVE_UP_WORD] = 0; }
    for(int i = threadIdx.x; i < WARPS * RADIX; i += BLOCK) warp_hist[i] = 0;
    __syncthreads();
    const u32 tile = misc[0];
    const u64 tile_base = u64(tile) * TILE;
    if(tile_base >= n) return;
    if(n - tile_base >= u64(TILE))
        onesweep_tile<BLOCK, ITEMS, V, MATCH_BITS, true>(keys_in, keys_out, vals_in, vals_out, n, shift, dmask, digit_base, next_base, status, dev_status, tile, u32(TILE),
                                                         0u, tile_base);
    else
        onesweep_tile<BLOCK, ITEMS, V, MATCH_BITS, false>(keys_in, keys_out, vals_in, vals_out, n, shift, dmask, digit_base, next_base, status, dev_status, tile,
                                                          u32(n - tile_base), 0u, tile_base);
}

// The segment that holds tile `t`: the last s with seg_tile0[s] <= t (seg_tile0 has segs + 1 ascending entries).
__device__ __forceinline__ u32 segment_of_tile(const u32* __restrict__ seg_tile0, const u32 segs, const u32 t)
{
    u32 a = 0, b = segs - 1;
    while(a < b)
    {
        const u32 mid = (a + b + 1) >> 1;
        if(__ldg(seg_tile0 + mid) <= t) a = mid; else b = mid - 1;
    }
    return a;
}

// One digit pass over MANY segments of one array in one launch: every segment is sorted on its own (its tiles look back no
// further than its first tile, its records stay inside its range). digit_base: [segments][RADIX] offsets in the whole array;
// skip: [segments], what the segment does in this pass (see seg_plan_kernel): 0 sort; 1 copy its records over unchanged (the
// digit is the same for all of them), so that all segments change buffers together; 2 nothing.
template <int BLOCK, int ITEMS, typename V, int MATCH_BITS>
__global__ void __launch_bounds__(BLOCK) onesweep_seg_pass_kernel(const u64* __restrict__ keys_in, u64* __restrict__ keys_out, const V* __restrict__ vals_in,
                                                                 V* __restrict__ vals_out, const u64* __restrict__ seg_off, const u32* __restrict__ seg_tile0,
                                                                 const u32 segs, const int shift, const u32 dmask, const u64* __restrict__ digit_base,
                                                                 const u32* __restrict__ skip, u32* __restrict__ status, u32* __restrict__ tile_counter,
                                                                 u64* __restrict__ dev_status)
{
    constexpr int TILE = BLOCK * ITEMS;
    constexpr int WARPS = BLOCK / 32;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    u32* const warp_hist = reinterpret_cast<u32*>(smem_raw + size_t(TILE) * 8 + size_t(TILE) * sizeof(V));
    u32* const misc = reinterpret_cast<u32*>(smem_raw + size_t(TILE) * 8 + size_t(TILE) * sizeof(V) + size_t(WARPS) * RADIX * 4 + RADIX * 4 + RADIX * 8);
    if(threadIdx.x == 0)
    {
        const u32 t = atomicAdd(tile_counter, 1u);
        misc[0] = t;
        misc[GAVE_UP_WORD] = 0;
        misc[GAVE_UP_WORD + 1] = t < __ldg(seg_tile0 + segs) ? segment_of_tile(seg_tile0, segs, t) : 0xFFFFFFFFu;
    }
    for(int i = threadIdx.x; i < WARPS * RADIX; i += BLOCK) warp_hist[i] = 0;
    __syncthreads();
    const u32 tile = misc[0], s = misc[GAVE_UP_WORD + 1];
    if(s == 0xFFFFFFFFu) return;
    const u32 first_tile = __ldg(seg_tile0 + s);
    const u64 seg_first = seg_off[s], seg_end = seg_off[s + 1];
    const u64 tile_base = seg_first + u64(tile - first_tile) * TILE;
    if(tile_base >= seg_end) return;
    const u32 valid = seg_end - tile_base >= u64(TILE) ? u32(TILE) : u32(seg_end - tile_base);
    const u32 mode = __ldg(skip + s);
    if(mode == 2) return;
    if(mode == 1)
    {
        for(u32 i = threadIdx.x; i < valid; i += BLOCK)
        {
            keys_out[tile_base + i] = keys_in[tile_base + i];
            if(vals_in != nullptr) vals_out[tile_base + i] = vals_in[tile_base + i];
        }
        return;
    }
    const u64* const db = digit_base + u64(s) * RADIX;
    if(valid == u32(TILE))
        onesweep_tile<BLOCK, ITEMS, V, MATCH_BITS, true>(keys_in, keys_out, vals_in, vals_out, seg_end, shift, dmask, db, nullptr, status, dev_status, tile, u32(TILE),
                                                         first_tile, tile_base);
    else
        onesweep_tile<BLOCK, ITEMS, V, MATCH_BITS, false>(keys_in, keys_out, vals_in, vals_out, seg_end, shift, dmask, db, nullptr, status, dev_status, tile, valid,
                                                          first_tile, tile_base);
}

// What a segment does in each pass of a segmented sort. skip: [passes][segments], 1 where the pass's digit is constant inside
// the segment; it is rewritten in place as 0 = sort, 1 = copy the records over unchanged, 2 = nothing at all. Two passes
// in a row that a segment would copy through leave its records in the buffer where they were, so both can do nothing; of a
// run of such passes only the last one of an odd run copies. first_sorts: pass 0 sorts every segment whatever its flag says
// (the unordered first pass has no copy-through form).
__global__ void seg_plan_kernel(u32* __restrict__ skip, const u32 segs, const int passes, const int first_sorts)
{
    const u32 s = blockIdx.x * blockDim.x + threadIdx.x;
    if(s >= segs) return;
    int p = 0;
    if(first_sorts && passes > 0) { skip[s] = 0; p = 1; }
    while(p < passes)
    {
        if(skip[u64(p) * segs + s] == 0) { ++p; continue; }
        int e = p;
        while(e < passes && skip[u64(e) * segs + s] != 0) ++e;        // the run [p, e) is skipped
        const int pairs = (e - p) / 2;
        for(int k = p; k < p + 2 * pairs; ++k) skip[u64(k) * segs + s] = 2;
        if((e - p) & 1) skip[u64(e - 1) * segs + s] = 1;
        p = e;
    }
}

// Digit offsets and skip flags of a segmented sort. hist: [passes][segments][RADIX]; base likewise, offsets in the whole array;
// skip: [passes][segments].
__global__ void __launch_bounds__(RADIX) seg_digit_base_kernel(const u64* __restrict__ hist, const u64* __restrict__ seg_off, const u32 segs, u64* __restrict__ base,
                                                              u32* __restrict__ skip)
{
    __shared__ u64 warp_tot[RADIX / 32];
    __shared__ int s_skip;
    const u32 p = blockIdx.x, s = blockIdx.y, d = threadIdx.x;
    if(d == 0) s_skip = 0;
    __syncthreads();
    const u64 n = seg_off[s + 1] - seg_off[s];
    const u64 at = (u64(p) * segs + s) * RADIX;
    const u64 total = hist[at + d];
    if(total == n) s_skip = 1;
    u64 inc = total;
    for(int o = 1; o < 32; o <<= 1)
    {
        const u64 t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
        if(int(lane_id()) >= o) inc += t;
    }
    if(lane_id() == 31) warp_tot[d >> 5] = inc;
    __syncthreads();
    u64 pre = seg_off[s];
    for(u32 w = 0; w < (d >> 5); ++w) pre += warp_tot[w];
    base[at + d] = pre + inc - total;
    if(d == 0) skip[u64(p) * segs + s] = u32(s_skip);
}

template <int BLOCK, int ITEMS, typename V, int MATCH_BITS>
int launch_pass(csa_ctx* ctx, const u64* kin, u64* kout, const V* vin, V* vout, u64 n, int shift, u32 dmask, const u64* digit_base, u64* next_base, u32* status, u32* counter)
{
    using S = Pass_Smem<BLOCK, ITEMS, V>;
    static std::atomic<bool> configured[64];      // several host threads (one per GPU) may come here at once; setting the attribute twice is harmless
    auto kern = onesweep_pass_kernel<BLOCK, ITEMS, V, MATCH_BITS>;
    if(!configured[ctx->device & 63])
    {
        CSA_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(S::bytes)));
        configured[ctx->device & 63] = true;
    }
    const u64 tiles = div_up(n, S::TILE);
    // The tile counter lies right before the status words (csa_sort_pairs carves them so): one clear covers both.
    if(reinterpret_cast<unsigned char*>(counter) + 256 == reinterpret_cast<unsigned char*>(status))
        CSA_CUDA(ctx, cudaMemsetAsync(counter, 0, 256 + tiles * RADIX * sizeof(u32), ctx->stream));
    else
    {
        CSA_CUDA(ctx, cudaMemsetAsync(status, 0, tiles * RADIX * sizeof(u32), ctx->stream));
        CSA_CUDA(ctx, cudaMemsetAsync(counter, 0, sizeof(u32), ctx->stream));
    }
    if(g_first_tile != 0)       // test hook only
    {
        static u32 start_value;
        start_value = g_first_tile;
        CSA_CUDA(ctx, cudaMemcpyAsync(counter, &start_value, sizeof(u32), cudaMemcpyHostToDevice, ctx->stream));
    }
    kern<<<unsigned(tiles), BLOCK, S::bytes, ctx->stream>>>(kin, kout, vin, vout, n, shift, dmask, digit_base, next_base, status, counter, ctx->d_status);
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

// ---- the first pass of a sort whose caller accepts records of equal keys in any order --------------------------------
// The least significant digit's pass has no earlier order to keep, so it need not be stable: a record's place among its
// tile's records of the same digit is whatever a shared-memory atomic hands out, and a tile's run of a digit goes where
// an atomic on the digit's global cursor puts it. No warp-level matching, no look-back, a third of the instructions: the
// pass runs near copy speed. The later passes are stable as before, so the result is a correct sort whose ties come in
// no particular order (the doubling steps re-sort ties anyway). cursor: the pass's digit offsets; they are advanced.
constexpr int FP_BLOCK = 256, FP_ITEMS = 16, FP_TILE = FP_BLOCK * FP_ITEMS;
constexpr int FP_COPIES = 4;     // counters per digit, taken by lane: a digit that many records share (the low byte of a frequent token id) then serialises a quarter as many lanes of an atomic instruction
constexpr size_t FP_SMEM = size_t(FP_TILE) * 12 + RADIX * 8 + RADIX * FP_COPIES * 4 + 64;
__device__ __forceinline__ void first_pass_tile(const u64* __restrict__ keys_in, u64* __restrict__ keys_out, const u32* __restrict__ vals_in,
                                                u32* __restrict__ vals_out, const u64 tile_first, const u32 valid, const int shift, const u32 dmask,
                                                u64* __restrict__ cursor)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    u64* const stage_keys = reinterpret_cast<u64*>(smem_raw);
    u64* const base = stage_keys + FP_TILE;                         // output entry of the tile's run of a digit, minus the run's start in the tile
    u32* const stage_vals = reinterpret_cast<u32*>(base + RADIX);
    u32* const cnt = stage_vals + FP_TILE;                          // [digit][copy]
    u32* const warp_tot = cnt + RADIX * FP_COPIES;
    static_assert(FP_BLOCK == RADIX, "one thread per digit");
    const u32 tid = threadIdx.x, copy = tid & (FP_COPIES - 1);
    #pragma unroll
    for(int j = 0; j < FP_COPIES; ++j) cnt[tid * FP_COPIES + j] = 0;
    __syncthreads();
    u64 k[FP_ITEMS];
    u32 v[FP_ITEMS], r[FP_ITEMS];
    #pragma unroll
    for(int i = 0; i < FP_ITEMS; ++i)
    {
        const u32 j = tid + i * FP_BLOCK;
        if(j < valid) k[i] = keys_in[tile_first + j];
    }
    #pragma unroll
    for(int i = 0; i < FP_ITEMS; ++i)
    {
        const u32 j = tid + i * FP_BLOCK;
        if(vals_in != nullptr && j < valid) v[i] = vals_in[tile_first + j];
    }
    #pragma unroll
    for(int i = 0; i < FP_ITEMS; ++i)
    {
        const u32 j = tid + i * FP_BLOCK;
        if(j < valid) r[i] = atomicAdd(&cnt[(u32(k[i] >> shift) & dmask) * FP_COPIES + copy], 1u);
    }
    __syncthreads();
    // thread d: the digit's count over its copies, an exclusive scan over the digits, and the copies' starts inside the run
    u32 cc[FP_COPIES];
    u32 c = 0;
    #pragma unroll
    for(int j = 0; j < FP_COPIES; ++j) { cc[j] = cnt[tid * FP_COPIES + j]; c += cc[j]; }
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
    if(c) base[tid] = atomicAdd(reinterpret_cast<unsigned long long*>(cursor + tid), (unsigned long long)c) - start;
    {
        u32 run = start;
        #pragma unroll
        for(int j = 0; j < FP_COPIES; ++j) { cnt[tid * FP_COPIES + j] = run; run += cc[j]; }
    }
    __syncthreads();
    #pragma unroll
    for(int i = 0; i < FP_ITEMS; ++i)
    {
        const u32 j = tid + i * FP_BLOCK;
        if(j < valid)
        {
            const u32 at = cnt[(u32(k[i] >> shift) & dmask) * FP_COPIES + copy] + r[i];
            stage_keys[at] = k[i];
            if(vals_in != nullptr) stage_vals[at] = v[i];
        }
    }
    __syncthreads();
    #pragma unroll
    for(int i = 0; i < FP_ITEMS; ++i)
    {
        const u32 j = tid + i * FP_BLOCK;
        if(j < valid)
        {
            const u64 kk = stage_keys[j];
            const u64 dst = base[u32(kk >> shift) & dmask] + j;
            keys_out[dst] = kk;
            if(vals_in != nullptr) vals_out[dst] = stage_vals[j];
        }
    }
}

__global__ void __launch_bounds__(FP_BLOCK) first_pass_kernel(const u64* __restrict__ keys_in, u64* __restrict__ keys_out, const u32* __restrict__ vals_in,
                                                             u32* __restrict__ vals_out, const u64 n, const int shift, const u32 dmask,
                                                             u64* __restrict__ cursor)
{
    const u64 tile_first = u64(blockIdx.x) * FP_TILE;
    const u32 valid = (n - tile_first < u64(FP_TILE)) ? u32(n - tile_first) : u32(FP_TILE);
    first_pass_tile(keys_in, keys_out, vals_in, vals_out, tile_first, valid, shift, dmask, cursor);
}

// The same over many segments in one launch: a block's tile lies inside one segment and uses that segment's cursors
// (cursor: [segments][RADIX], each segment's digit offsets in the whole array).
__global__ void __launch_bounds__(FP_BLOCK) first_pass_seg_kernel(const u64* __restrict__ keys_in, u64* __restrict__ keys_out, const u32* __restrict__ vals_in,
                                                                 u32* __restrict__ vals_out, const u64* __restrict__ seg_off, const u32* __restrict__ seg_tile0,
                                                                 const u32 segs, const int shift, const u32 dmask, u64* __restrict__ cursor)
{
    __shared__ u32 s_seg;
    if(threadIdx.x == 0) s_seg = segment_of_tile(seg_tile0, segs, blockIdx.x);
    __syncthreads();
    const u32 s = s_seg;
    const u64 tile_first = seg_off[s] + u64(blockIdx.x - __ldg(seg_tile0 + s)) * FP_TILE, seg_end = seg_off[s + 1];
    if(tile_first >= seg_end) return;
    const u32 valid = (seg_end - tile_first < u64(FP_TILE)) ? u32(seg_end - tile_first) : u32(FP_TILE);
    first_pass_tile(keys_in, keys_out, vals_in, vals_out, tile_first, valid, shift, dmask, cursor + u64(s) * RADIX);
}

int launch_first_pass(csa_ctx* ctx, const u64* kin, u64* kout, const u32* vin, u32* vout, u64 n, int shift, u32 dmask, u64* cursor)
{
    static std::atomic<bool> configured[64];
    if(!configured[ctx->device & 63])
    {
        CSA_CUDA(ctx, cudaFuncSetAttribute(first_pass_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(FP_SMEM)));
        configured[ctx->device & 63] = true;
    }
    first_pass_kernel<<<unsigned(div_up(n, FP_TILE)), FP_BLOCK, FP_SMEM, ctx->stream>>>(kin, kout, vin, vout, n, shift, dmask, cursor);
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

// Shapes of the pass kernel to choose from (block size x items per thread); the smallest tile sizes the workspace.
int g_variant = 0;
constexpr int PASS_TILE = 4096;     // smallest tile among the variants

template <typename V>
int launch_pass_variant(csa_ctx* ctx, const u64* kin, u64* kout, const V* vin, V* vout, u64 n, int shift, u32 dmask, const u64* db, u64* nb, u32* status,
                        u32* counter)
{
    switch(g_variant)
    {
    case 1: return launch_pass<256, 16, V, 3>(ctx, kin, kout, vin, vout, n, shift, dmask, db, nb, status, counter);
    case 2: return launch_pass<256, 20, V, 3>(ctx, kin, kout, vin, vout, n, shift, dmask, db, nb, status, counter);
    case 3: return launch_pass<256, 24, V, 3>(ctx, kin, kout, vin, vout, n, shift, dmask, db, nb, status, counter);
    case 4: return launch_pass<256, 28, V, 3>(ctx, kin, kout, vin, vout, n, shift, dmask, db, nb, status, counter);
    case 5: return launch_pass<384, 16, V, 3>(ctx, kin, kout, vin, vout, n, shift, dmask, db, nb, status, counter);
    case 6: return launch_pass<512, 8, V, 3>(ctx, kin, kout, vin, vout, n, shift, dmask, db, nb, status, counter);
    default:
        // 24 records per thread hold in 128 registers with 4-byte values; 8-byte values spill beyond 16.
        if constexpr(sizeof(V) == 4) return launch_pass<256, 24, V, 3>(ctx, kin, kout, vin, vout, n, shift, dmask, db, nb, status, counter);
        else return launch_pass<256, 16, V, 3>(ctx, kin, kout, vin, vout, n, shift, dmask, db, nb, status, counter);
    }
}

struct Pass_Timer
{
    bool on = false;
    std::vector<cudaEvent_t> ev;    // pairs
    u64 passes = 0, records = 0, bytes = 0;
};

Pass_Timer& timer_of(csa_ctx* ctx)
{
    if(!ctx->pass_timer) ctx->pass_timer = new Pass_Timer();
    return *static_cast<Pass_Timer*>(ctx->pass_timer);
}

}   // namespace

extern "C" int csa_debug_set(int key, uint64_t value)
{
    if(key == 0 && value >= 12 && value <= 29) { PORTION = 1ull << value; return CSA_OK; }
    if(key == 1 && value <= 5) { g_variant = int(value); return CSA_OK; }
    if(key == 2 && value >= 1 && value <= LOOKBACK_SPIN_LIMIT)     // on the current device
    {
        const u32 v = u32(value);
        return cudaMemcpyToSymbol(g_lookback_spin_limit, &v, sizeof(v)) == cudaSuccess ? CSA_OK : CSA_E_CUDA;
    }
    if(key == 3 && value <= 1) { g_first_tile = u32(value); return CSA_OK; }
    if(key == 4 && value < (1ull << 40)) { stream_set_position_offset(value); return CSA_OK; }
    return CSA_E_INVALID;
}

// Device address of the digit histograms ([pass][RADIX] 64-bit counts) that the last csa_sort_pairs of n records left in
// its workspace (the same carving as in csa_sort_pairs).
const u64* sort_workspace_histograms(void* workspace, size_t workspace_bytes, u64 n)
{
    Carver cv(workspace, workspace_bytes);
    const u64 tiles_max = div_up(n < PORTION ? n : PORTION, PASS_TILE) + 1;
    cv.take<u32>(64);
    cv.take<u32>(tiles_max * RADIX);
    return cv.take<u64>(u64(8) * RADIX);
}

size_t csa_sort_workspace_bytes(uint64_t n)
{
    const u64 portions = n == 0 ? 1 : div_up(n, PORTION);
    const u64 tiles = div_up(n < PORTION ? n : PORTION, PASS_TILE) + 1;
    return size_t(tiles) * RADIX * 4 + 256            // tile status
         + 256                                         // tile counter
         + size_t(8) * RADIX * 8 + 256                 // histograms
         + size_t(portions + 1) * 8 * RADIX * 8 + 256  // digit bases of every launch
         + 4096;
}

int csa_set_pass_timing(csa_ctx* ctx, int on)
{
    if(!ctx) return CSA_E_INVALID;
    timer_of(ctx).on = on != 0;
    return CSA_OK;
}

int csa_get_pass_timing(csa_ctx* ctx, double* total_ms, uint64_t* passes, uint64_t* records, uint64_t* bytes)
{
    if(!ctx) return CSA_E_INVALID;
    Pass_Timer& t = timer_of(ctx);
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
    if(bytes) *bytes = t.bytes;
    return CSA_OK;
}

void sort_free_timing(csa_ctx* ctx)
{
    if(!ctx->pass_timer) return;
    Pass_Timer* t = static_cast<Pass_Timer*>(ctx->pass_timer);
    for(auto e : t->ev) cudaEventDestroy(e);
    delete t;
    ctx->pass_timer = nullptr;
}

void sort_reset_timing(csa_ctx* ctx)
{
    Pass_Timer& t = timer_of(ctx);
    for(auto e : t.ev) cudaEventDestroy(e);
    t.ev.clear();
    t.passes = t.records = t.bytes = 0;
}

int csa_sort_pairs(csa_ctx* ctx, uint64_t* keys, uint64_t* keys_alt, void* vals, void* vals_alt, uint32_t val_bytes, uint64_t n,
                   int begin_bit, int end_bit, void* workspace, size_t workspace_bytes, int* in_alt)
{
    if(!ctx || !in_alt) return CSA_E_INVALID;
    *in_alt = 0;
    if(begin_bit < 0 || end_bit > 64 || begin_bit > end_bit || (val_bytes != 4 && val_bytes != 8)) return csa_fail(ctx, CSA_E_INVALID, "csa_sort_pairs: bad bit range or value width");
    if(n <= 1 || begin_bit == end_bit) return CSA_OK;
    if(!keys || !keys_alt || !workspace || ((vals == nullptr) != (vals_alt == nullptr))) return csa_fail(ctx, CSA_E_INVALID, "csa_sort_pairs: null buffer");
    if(workspace_bytes < csa_sort_workspace_bytes(n)) return csa_fail(ctx, CSA_E_NOMEM, "csa_sort_pairs: workspace too small");
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));

    const int passes = (end_bit - begin_bit + RADIX_BITS - 1) / RADIX_BITS;
    const int portions = int(div_up(n, PORTION));
    Carver cv(workspace, workspace_bytes);
    const u64 tiles_max = div_up(n < PORTION ? n : PORTION, PASS_TILE) + 1;
    u32* counter = cv.take<u32>(64);                     // 256 bytes, directly before the status words
    u32* status = cv.take<u32>(tiles_max * RADIX);
    u64* hist = cv.take<u64>(u64(8) * RADIX);
    u64* base = cv.take<u64>(u64(portions + 1) * 8 * RADIX);
    if(!cv.ok) return csa_fail(ctx, CSA_E_NOMEM, "csa_sort_pairs: workspace too small");

    {
        static std::atomic<bool> hist_configured[64];
        if(!hist_configured[ctx->device & 63])
        {
            CSA_CUDA(ctx, cudaFuncSetAttribute(histogram_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 8 * RADIX * 4));
            hist_configured[ctx->device & 63] = true;
        }
    }
    CSA_CUDA(ctx, cudaMemsetAsync(hist, 0, u64(passes) * RADIX * sizeof(u64), ctx->stream));
    for(int P = 0; P < portions; ++P)
    {
        const u64 first = u64(P) * PORTION, cnt = (n - first < PORTION ? n - first : PORTION);
        const unsigned blocks = unsigned(cnt / (2 * 256 * HIST_UNROLL) < 1 ? 1 : (cnt / (2 * 256 * HIST_UNROLL) > 148 * 3 ? 148 * 3 : cnt / (2 * 256 * HIST_UNROLL)));
        histogram_kernel<256><<<blocks, 256, size_t(8) * passes * RADIX * 4, ctx->stream>>>(reinterpret_cast<const u64*>(keys) + first, cnt, begin_bit, end_bit, passes, hist);
        CSA_LAUNCH_CHECK(ctx);
    }
    u64* d_skip = ctx->d_scalars + 32;
    digit_base_kernel<<<passes, RADIX, 0, ctx->stream>>>(hist, portions, n, base, d_skip);
    CSA_LAUNCH_CHECK(ctx);
    CSA_CUDA(ctx, cudaMemcpyAsync(ctx->h_scalars + 32, d_skip, passes * sizeof(u64), cudaMemcpyDeviceToHost, ctx->stream));
    CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    u64 skip[8];
    for(int p = 0; p < passes; ++p) skip[p] = ctx->h_scalars[32 + p];

    Pass_Timer& timer = timer_of(ctx);
    u64* kin = reinterpret_cast<u64*>(keys); u64* kout = reinterpret_cast<u64*>(keys_alt);
    void* vin = vals; void* vout = vals_alt;
    int flips = 0;
    // The first pass that moves anything may leave ties in any order where the caller said so (4-byte values or none).
    bool first_pass_free = ctx->ties_in_any_order && (val_bytes == 4 || vals == nullptr);
    for(int p = 0; p < passes; ++p)
    {
        if(skip[p]) continue;
        const int shift = begin_bit + p * RADIX_BITS;
        const bool unordered = first_pass_free;
        first_pass_free = false;
        cudaEvent_t e0 = nullptr, e1 = nullptr;
        if(timer.on && !unordered)          // the timer is the digit-pass kernel's: the unordered pass is another kernel
        {
            CSA_CUDA(ctx, cudaEventCreate(&e0));
            CSA_CUDA(ctx, cudaEventCreate(&e1));
            CSA_CUDA(ctx, cudaEventRecord(e0, ctx->stream));
        }
        for(int P = 0; P < portions; ++P)
        {
            const u64 first = u64(P) * PORTION, cnt = (n - first < PORTION ? n - first : PORTION);
            u64* db = base + (u64(p) * (portions + 1) + P) * RADIX;
            if(unordered)       // one set of cursors serves all launches of the pass
                CSA_TRY(launch_first_pass(ctx, kin + first, kout, vin ? static_cast<const u32*>(vin) + first : nullptr, static_cast<u32*>(vout), cnt, shift,
                                          digit_mask(shift, end_bit), base + u64(p) * (portions + 1) * RADIX));
            else if(val_bytes == 4 || vin == nullptr)
                CSA_TRY(launch_pass_variant<u32>(ctx, kin + first, kout, vin ? static_cast<const u32*>(vin) + first : nullptr, static_cast<u32*>(vout), cnt, shift, digit_mask(shift, end_bit), db, db + RADIX, status, counter));
            else
                CSA_TRY(launch_pass_variant<u64>(ctx, kin + first, kout, static_cast<const u64*>(vin) + first, static_cast<u64*>(vout), cnt, shift, digit_mask(shift, end_bit), db, db + RADIX, status, counter));
        }
        if(timer.on && !unordered)
        {
            CSA_CUDA(ctx, cudaEventRecord(e1, ctx->stream));
            timer.ev.push_back(e0); timer.ev.push_back(e1);
            timer.passes++; timer.records += n; timer.bytes += 2 * n * (8 + (vin ? val_bytes : 0));
        }
        ctx->counters[1]++;          // digit passes
        ctx->counters[2] += n;       // records moved
        if(vin == nullptr) ctx->counters[3] += n;     // of which without a value (16 instead of 24 bytes per record and pass)
        u64* tk = kin; kin = kout; kout = tk;
        void* tv = vin; vin = vout; vout = tv;
        ++flips;
    }
    *in_alt = flips & 1;
    return CSA_OK;
}

// ---- many segments of one array, sorted in one set of launches ----------------------------------------------------------------
// Generation 0 of a build sorts every partition on its own; done one partition at a time that is a dozen launches and one
// read-back per partition. Here all partitions go through each digit pass together: one histogram launch, one launch for the
// digit offsets, one launch per pass, no read-back. A pass whose digit is constant inside a segment copies that segment's
// records over unchanged instead of being skipped, so that all segments change buffers together.

namespace
{

constexpr int SEG_BLOCK = 256, SEG_ITEMS = 24, SEG_MATCH = 3, SEG_TILE = SEG_BLOCK * SEG_ITEMS;

}   // namespace

size_t sort_segments_workspace_bytes(u64 n, u32 segs)
{
    const u64 tiles = n / SEG_TILE + segs + 2;
    return align_up256(tiles * RADIX * 4) + 256                                   // tile counter, then the tile status words
         + 2 * align_up256(size_t(8) * segs * RADIX * 8)                          // histograms and digit offsets of every pass and segment
         + align_up256(size_t(8) * segs * 4)                                      // skip flags
         + align_up256(size_t(segs + 1) * 8) + 2 * align_up256(size_t(segs + 1) * 4) + 4096;
}

int sort_segments(csa_ctx* ctx, u64* keys, u64* keys_alt, u32* vals, u32* vals_alt, const u64* seg_off_host, u32 segs, int begin_bit, int end_bit, void* workspace,
                  size_t workspace_bytes, int* in_alt)
{
    *in_alt = 0;
    if(segs == 0 || begin_bit < 0 || end_bit > 64 || begin_bit >= end_bit) return csa_fail(ctx, CSA_E_INVALID, "segmented sort: bad argument");
    const u64 n = seg_off_host[segs];
    if(n == 0) return CSA_OK;
    if(workspace_bytes < sort_segments_workspace_bytes(n, segs)) return csa_fail(ctx, CSA_E_NOMEM, "segmented sort: workspace too small");
    const int passes = (end_bit - begin_bit + RADIX_BITS - 1) / RADIX_BITS;
    std::vector<u32> tile0(segs + 1), tile0_fp(segs + 1);
    u64 t = 0, tf = 0;
    for(u32 s = 0; s < segs; ++s)
    {
        const u64 c = seg_off_host[s + 1] - seg_off_host[s];
        if(c >= (u64(1) << 30)) return csa_fail(ctx, CSA_E_LIMIT, "segmented sort: a segment holds 2^30 records or more");
        tile0[s] = u32(t); tile0_fp[s] = u32(tf);
        t += div_up(c, SEG_TILE); tf += div_up(c, FP_TILE);
    }
    if(t >= (u64(1) << 31) || tf >= (u64(1) << 31)) return csa_fail(ctx, CSA_E_LIMIT, "segmented sort: too many tiles");
    tile0[segs] = u32(t); tile0_fp[segs] = u32(tf);

    Carver cv(workspace, workspace_bytes);
    u32* counter = cv.take<u32>(64);
    u32* status = cv.take<u32>((t + 1) * RADIX);
    u64* hist = cv.take<u64>(u64(8) * segs * RADIX);
    u64* base = cv.take<u64>(u64(8) * segs * RADIX);
    u32* skip = cv.take<u32>(u64(8) * segs);
    u64* seg_off = cv.take<u64>(segs + 1);
    u32* seg_tile0 = cv.take<u32>(segs + 1);
    u32* seg_tile0_fp = cv.take<u32>(segs + 1);
    if(!cv.ok || reinterpret_cast<unsigned char*>(counter) + 256 != reinterpret_cast<unsigned char*>(status)) return csa_fail(ctx, CSA_E_NOMEM, "segmented sort: workspace too small");
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    // the tables go up from pageable memory: the copies are done when the calls return
    CSA_CUDA(ctx, cudaMemcpyAsync(seg_off, seg_off_host, size_t(segs + 1) * 8, cudaMemcpyHostToDevice, ctx->stream));
    CSA_CUDA(ctx, cudaMemcpyAsync(seg_tile0, tile0.data(), size_t(segs + 1) * 4, cudaMemcpyHostToDevice, ctx->stream));
    CSA_CUDA(ctx, cudaMemcpyAsync(seg_tile0_fp, tile0_fp.data(), size_t(segs + 1) * 4, cudaMemcpyHostToDevice, ctx->stream));
    CSA_CUDA(ctx, cudaMemsetAsync(hist, 0, u64(passes) * segs * RADIX * 8, ctx->stream));

    using S = Pass_Smem<SEG_BLOCK, SEG_ITEMS, u32>;
    auto pass_kern = onesweep_seg_pass_kernel<SEG_BLOCK, SEG_ITEMS, u32, SEG_MATCH>;
    {
        static std::atomic<bool> configured[64];
        if(!configured[ctx->device & 63])
        {
            CSA_CUDA(ctx, cudaFuncSetAttribute(pass_kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(S::bytes)));
            CSA_CUDA(ctx, cudaFuncSetAttribute(seg_histogram_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 8 * RADIX * 4));
            CSA_CUDA(ctx, cudaFuncSetAttribute(first_pass_seg_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(FP_SMEM)));
            configured[ctx->device & 63] = true;
        }
    }
    // blocks per segment of the histogram: enough to fill the device over all segments
    const unsigned hx = unsigned(std::max<u64>(1, std::min<u64>(148 * 4 / segs + 1, div_up(n / segs + 1, 2 * 256 * HIST_UNROLL))));
    seg_histogram_kernel<256><<<dim3(hx, segs), 256, size_t(8) * passes * RADIX * 4, ctx->stream>>>(keys, seg_off, segs, begin_bit, end_bit, passes, hist);
    CSA_LAUNCH_CHECK(ctx);
    seg_digit_base_kernel<<<dim3(passes, segs), RADIX, 0, ctx->stream>>>(hist, seg_off, segs, base, skip);
    CSA_LAUNCH_CHECK(ctx);
    seg_plan_kernel<<<unsigned(div_up(segs, 256)), 256, 0, ctx->stream>>>(skip, segs, passes, ctx->ties_in_any_order ? 1 : 0);
    CSA_LAUNCH_CHECK(ctx);

    Pass_Timer& timer = timer_of(ctx);
    // With pass timing on (the benchmark), the records that each pass really moves are counted: the plan comes back once, which
    // drains the stream; an untimed sort reads nothing back.
    std::vector<u64> moved(passes, n);
    if(timer.on)
    {
        std::vector<u32> modes(size_t(passes) * segs);
        CSA_CUDA(ctx, cudaMemcpyAsync(modes.data(), skip, modes.size() * 4, cudaMemcpyDeviceToHost, ctx->stream));
        CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        for(int p = 0; p < passes; ++p)
        {
            moved[p] = 0;
            for(u32 sg = 0; sg < segs; ++sg) if(modes[size_t(p) * segs + sg] != 2) moved[p] += seg_off_host[sg + 1] - seg_off_host[sg];
        }
    }
    u64* kin = keys; u64* kout = keys_alt;
    u32* vin = vals; u32* vout = vals_alt;
    for(int p = 0; p < passes; ++p)
    {
        const int shift = begin_bit + p * RADIX_BITS;
        const u32 dmask = digit_mask(shift, end_bit);
        const bool unordered = p == 0 && ctx->ties_in_any_order;
        if(unordered)
        {
            first_pass_seg_kernel<<<unsigned(tf), FP_BLOCK, FP_SMEM, ctx->stream>>>(kin, kout, vin, vout, seg_off, seg_tile0_fp, segs, shift, dmask, base);
            CSA_LAUNCH_CHECK(ctx);
        }
        else
        {
            cudaEvent_t e0 = nullptr, e1 = nullptr;
            if(timer.on)
            {
                CSA_CUDA(ctx, cudaEventCreate(&e0));
                CSA_CUDA(ctx, cudaEventCreate(&e1));
                CSA_CUDA(ctx, cudaEventRecord(e0, ctx->stream));
            }
            CSA_CUDA(ctx, cudaMemsetAsync(counter, 0, 256 + t * RADIX * sizeof(u32), ctx->stream));
            pass_kern<<<unsigned(t), SEG_BLOCK, S::bytes, ctx->stream>>>(kin, kout, vin, vout, seg_off, seg_tile0, segs, shift, dmask, base + u64(p) * segs * RADIX,
                                                                        skip + u64(p) * segs, status, counter, ctx->d_status);
            CSA_LAUNCH_CHECK(ctx);
            if(timer.on)
            {
                CSA_CUDA(ctx, cudaEventRecord(e1, ctx->stream));
                timer.ev.push_back(e0); timer.ev.push_back(e1);
                timer.passes++; timer.records += moved[p]; timer.bytes += 2 * moved[p] * (8 + (vin ? 4 : 0));
            }
        }
        ctx->counters[1]++;
        ctx->counters[2] += moved[p];
        u64* tk = kin; kin = kout; kout = tk;
        u32* tv = vin; vin = vout; vout = tv;
    }
    *in_alt = passes & 1;
    return CSA_OK;
}

extern "C" size_t csa_sort_segments_workspace_bytes(uint64_t n, uint32_t segments) { return sort_segments_workspace_bytes(n, segments ? segments : 1); }

extern "C" int csa_sort_segments(csa_ctx* ctx, uint64_t* keys, uint64_t* keys_alt, uint32_t* vals, uint32_t* vals_alt, const uint64_t* seg_off_host, uint32_t segments,
                                 int begin_bit, int end_bit, void* workspace, size_t workspace_bytes, int* in_alt)
{
    if(!ctx || !in_alt || !keys || !keys_alt || !seg_off_host || !workspace || ((vals == nullptr) != (vals_alt == nullptr)))
        return csa_fail(ctx, CSA_E_INVALID, "csa_sort_segments: null argument");
    for(uint32_t s = 0; s < segments; ++s)
        if(seg_off_host[s + 1] < seg_off_host[s]) return csa_fail(ctx, CSA_E_INVALID, "csa_sort_segments: offsets must not decrease");
    if(segments && seg_off_host[0] != 0) return csa_fail(ctx, CSA_E_INVALID, "csa_sort_segments: the first segment starts at record 0");
    return sort_segments(ctx, reinterpret_cast<u64*>(keys), reinterpret_cast<u64*>(keys_alt), vals, vals_alt, reinterpret_cast<const u64*>(seg_off_host), segments,
                         begin_bit, end_bit, workspace, workspace_bytes, in_alt);
}

// ---- the sort for callers that must not allocate ---------------------------------------------------------------------
//
// Some hosts of this library run where device allocation is off the table: a plugin called in the middle of another
// runtime's step, whose memory pool owns the whole device and treats a foreign cudaMalloc as an error (or would stall on
// it, since cudaMalloc synchronises the device), or a service that has been told to stay inside a fixed memory budget
// after start-up. csa_sort_pairs needs a context (which allocates) and a workspace. The entry point below needs neither:
// its scratch (tile status words, digit histograms and offsets, a status word) is a fixed array in the library's device
// image, which every GPU that loads the library holds from load to exit.

namespace
{

constexpr u64 STATIC_SORT_MAX = CSA_STATIC_SORT_MAX_RECORDS;
constexpr int ST_BLOCK = 512, ST_ITEMS = 8, ST_MATCH = 3, ST_TILE = ST_BLOCK * ST_ITEMS;
constexpr size_t ST_OFF_STATUS = 0;                                                        // [tiles][RADIX] u32
constexpr size_t ST_OFF_COUNTER = ST_OFF_STATUS + (STATIC_SORT_MAX / ST_TILE + 1) * RADIX * 4; // tile counter
constexpr size_t ST_OFF_HIST = ST_OFF_COUNTER + 256;                                       // [8][RADIX] u64
constexpr size_t ST_OFF_BASE = ST_OFF_HIST + size_t(8) * RADIX * 8;                        // [8][2][RADIX] u64
constexpr size_t ST_OFF_SKIP = ST_OFF_BASE + size_t(8) * 2 * RADIX * 8;                    // [8] u64 (written, not read)
constexpr size_t ST_OFF_DEVSTATUS = ST_OFF_SKIP + 256;                                     // one u64
constexpr size_t ST_BYTES = ST_OFF_DEVSTATUS + 256;

// Device code could name this array directly; host code must not pass its name to a kernel (on the host the name is only
// a stand-in for the symbol), so the host asks the runtime for the array's device address once per device.
static __device__ __align__(256) unsigned char g_static_scratch[ST_BYTES];
unsigned char* g_static_scratch_addr[64] = {nullptr};

}   // namespace

extern "C" int csa_sort_pairs_static(void* stream_, uint64_t* keys, uint64_t* keys_alt, uint32_t* vals, uint32_t* vals_alt, uint64_t n,
                                     int begin_bit, int end_bit, int* in_alt)
{
    if(!in_alt) return CSA_E_INVALID;
    *in_alt = 0;
    if(begin_bit < 0 || end_bit > 64 || begin_bit > end_bit) return CSA_E_INVALID;
    if(n > STATIC_SORT_MAX)
    {
        std::fprintf(stderr, "csa_sort_pairs_static: %llu records exceed the fixed scratch's maximum of %llu; use csa_sort_pairs\n",
                     (unsigned long long)n, (unsigned long long)STATIC_SORT_MAX);
        return CSA_E_LIMIT;
    }
    if(n <= 1 || begin_bit == end_bit) return CSA_OK;
    if(!keys || !keys_alt || !vals || !vals_alt) return CSA_E_INVALID;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);

    int dev = 0;
    if(cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return CSA_E_CUDA;
    auto kern = onesweep_pass_kernel<ST_BLOCK, ST_ITEMS, u32, ST_MATCH>;
    using S = Pass_Smem<ST_BLOCK, ST_ITEMS, u32>;
    if(!g_static_scratch_addr[dev])
    {
        // Set-up, once per device, with that device current: the array's device address, and the kernel's shared-memory size.
        void* p = nullptr;
        if(cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || !p) { cudaGetLastError(); return CSA_E_CUDA; }
        if(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(S::bytes)) != cudaSuccess) { cudaGetLastError(); return CSA_E_CUDA; }
        if(cudaFuncSetAttribute(histogram_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 8 * RADIX * 4) != cudaSuccess) { cudaGetLastError(); return CSA_E_CUDA; }
        g_static_scratch_addr[dev] = static_cast<unsigned char*>(p);
    }
    unsigned char* const base_addr = g_static_scratch_addr[dev];
    u32* const status = reinterpret_cast<u32*>(base_addr + ST_OFF_STATUS);
    u32* const counter = reinterpret_cast<u32*>(base_addr + ST_OFF_COUNTER);
    u64* const hist = reinterpret_cast<u64*>(base_addr + ST_OFF_HIST);
    u64* const base = reinterpret_cast<u64*>(base_addr + ST_OFF_BASE);
    u64* const skip = reinterpret_cast<u64*>(base_addr + ST_OFF_SKIP);
    u64* const dev_status = reinterpret_cast<u64*>(base_addr + ST_OFF_DEVSTATUS);

    const int passes = (end_bit - begin_bit + RADIX_BITS - 1) / RADIX_BITS;
    const u64 tiles = div_up(n, ST_TILE);
    // The array keeps the last call's contents: everything that must start at zero is cleared here.
    if(cudaMemsetAsync(base_addr + ST_OFF_COUNTER, 0, ST_BYTES - ST_OFF_COUNTER, stream) != cudaSuccess) return CSA_E_CUDA;
    const unsigned hblocks = unsigned(n / (2 * 256 * HIST_UNROLL) < 1 ? 1 : (n / (2 * 256 * HIST_UNROLL) > 148 * 3 ? 148 * 3 : n / (2 * 256 * HIST_UNROLL)));
    histogram_kernel<256><<<hblocks, 256, size_t(8) * passes * RADIX * 4, stream>>>(reinterpret_cast<const u64*>(keys), n, begin_bit, end_bit, passes, hist);
    digit_base_kernel<<<passes, RADIX, 0, stream>>>(hist, 1, n, base, skip);
    u64* kin = reinterpret_cast<u64*>(keys); u64* kout = reinterpret_cast<u64*>(keys_alt);
    u32* vin = vals; u32* vout = vals_alt;
    for(int p = 0; p < passes; ++p)     // every pass runs (no read-back decides about skipping), so the result's place is known
    {
        const int shift = begin_bit + p * RADIX_BITS;
        if(cudaMemsetAsync(status, 0, tiles * RADIX * sizeof(u32), stream) != cudaSuccess) return CSA_E_CUDA;
        if(cudaMemsetAsync(counter, 0, sizeof(u32), stream) != cudaSuccess) return CSA_E_CUDA;
        u64* db = base + u64(p) * 2 * RADIX;
        kern<<<unsigned(tiles), ST_BLOCK, S::bytes, stream>>>(kin, kout, vin, vout, n, shift, digit_mask(shift, end_bit), db, db + RADIX, status, counter, dev_status);
        u64* tk = kin; kin = kout; kout = tk;
        u32* tv = vin; vin = vout; vout = tv;
    }
    if(cudaGetLastError() != cudaSuccess) return CSA_E_CUDA;
    u64 bits = 0;
    if(cudaMemcpyAsync(&bits, dev_status, sizeof(bits), cudaMemcpyDeviceToHost, stream) != cudaSuccess) return CSA_E_CUDA;
    if(cudaStreamSynchronize(stream) != cudaSuccess) return CSA_E_CUDA;
    *in_alt = passes & 1;
    return bits == 0 ? CSA_OK : CSA_E_DEVICE;
}
