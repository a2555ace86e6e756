// K-gram sampling, splitter selection, partition ids and the scatter of suffix positions into partitions.
// A partition is the set of suffixes whose K-gram (first CSA_K symbols, zero-padded past the text's end) lies
// between two splitters, so it owns a fixed, contiguous range of the final suffix array.
//
// Reference behaviour followed: GPU_SACA::select_pivots (src/GPU_SACA.cu:290-364), compute_partition_IDs_kernel
// (include/GPU_SACA.cuh:23-73) and the host scatter of GPU_SACA::partition (src/GPU_SACA.cu:795-826).
#include "common.cuh"
#include "part.cuh"

#include <algorithm>
#include <utility>
#include <atomic>
#include <vector>

namespace
{

__host__ __device__ __forceinline__ u64 mix64(u64 x)
{
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

__global__ void sample_kgrams_kernel(const u16* __restrict__ T, const u64 n, const u64 n_samples, const u64 seed, u64* __restrict__ out)
{
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if(i >= n_samples) return;
    const u64 pos = mix64(seed * 0x100000001B3ull + i) % n;
    out[2 * i] = pack4(T, pos);             // the zero padding after the text makes short suffixes pad with zeros
    out[2 * i + 1] = pack4(T, pos + 4);
}

constexpr u32 BULK_WAIT_LIMIT = 1u << 16;   // each try may itself block for a while

__device__ __forceinline__ u32 smem_addr(const void* p) { return u32(__cvta_generic_to_shared(p)); }

// Copies `bytes` bytes (a multiple of 16, from a 16-byte aligned global address to a 16-byte aligned shared address)
// with one bulk asynchronous copy that signals `bar`. Called by one thread.
__device__ __forceinline__ void bulk_copy_to_shared(void* dst, const void* src, u32 bytes, u64* bar)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smem_addr(bar)), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(smem_addr(dst)), "l"(src), "r"(bytes), "r"(smem_addr(bar)) : "memory");
}

// Waits, with a bound, for phase `parity` of `bar`. Returns false if the bound ran out.
__device__ __forceinline__ bool bulk_wait(u64* bar, u32 parity)
{
    for(u32 spin = 0; spin < BULK_WAIT_LIMIT; ++spin)
    {
        u32 done;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(smem_addr(bar)), "r"(parity) : "memory");
        if(done) return true;
    }
    return false;
}

// Partition ids of the positions [first, first + count). A block takes a tile of BLOCK * ITEMS consecutive positions:
// the text window of the tile (tile + K - 1 symbols) arrives in shared memory by one bulk copy, a thread slides a
// K-gram over its ITEMS positions and searches the splitters, kept in shared memory too.
template <int BLOCK, int ITEMS>
__global__ void __launch_bounds__(BLOCK) partition_ids_kernel(const u16* __restrict__ T, const u64 n, const u64 first, const u64 count,
                                                             const u64* __restrict__ pivots, const u32 p, const u32* __restrict__ first_symbol_range,
                                                             u16* __restrict__ pid_out, u64* __restrict__ hist, u64* __restrict__ dev_status)
{
    constexpr int TILE = BLOCK * ITEMS;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    u16* const win = reinterpret_cast<u16*>(smem_raw);                               // TILE + 8 symbols
    u64* const bar = reinterpret_cast<u64*>(smem_raw + (TILE + 8) * 2);               // one mbarrier
    u64* const piv = reinterpret_cast<u64*>(smem_raw + (TILE + 8) * 2 + 16);          // 2 (p-1) words
    u32* const cnt = reinterpret_cast<u32*>(piv + 2 * (p > 1 ? p - 1 : 1));           // p counters

    const u32 tid = threadIdx.x;
    const u64 tile_first = first + u64(blockIdx.x) * TILE;          // `first` is a multiple of 8: the copy starts 16-byte aligned
    const u64 tile_count = (first + count - tile_first < u64(TILE)) ? first + count - tile_first : u64(TILE);

    if(tid == 0)
    {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(smem_addr(bar)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if(tid == 0)
    {
        // Readable symbols from the tile's start: the text and its zero padding, rounded down to whole 16-byte pieces.
        const u64 readable = ((n + CSA_TEXT_PAD - tile_first) / 8) * 8;
        const u64 want = TILE + 8;
        bulk_copy_to_shared(win, T + tile_first, u32((readable < want ? readable : want) * 2), bar);
    }
    for(u32 i = tid; i < 2 * (p - 1); i += BLOCK) piv[i] = pivots[i];
    for(u32 i = tid; i < p; i += BLOCK) cnt[i] = 0;
    __syncthreads();
    if(!bulk_wait(bar, 0))
    {
        atomicOr(dev_status, (u64)CSA_ST_BULK_TIMEOUT);
        bulk_wait(bar, 0);      // a second bounded wait for the copy still in flight before the block leaves
        return;
    }

    const u32 local = tid * ITEMS;
    if(local < tile_count)
    {
        u64 hi = (u64(win[local]) << 48) | (u64(win[local + 1]) << 32) | (u64(win[local + 2]) << 16) | u64(win[local + 3]);
        u64 lo = (u64(win[local + 4]) << 48) | (u64(win[local + 5]) << 32) | (u64(win[local + 6]) << 16) | u64(win[local + 7]);
        u16 ids[ITEMS];
        #pragma unroll
        for(int k = 0; k < ITEMS; ++k)
        {
            // lower bound: the first splitter that is not smaller than the K-gram, searched inside the range of partitions
            // that the K-gram's first symbol allows (a 65536-entry table; most symbols allow one partition only)
            u32 a = 0, b = p - 1;
            if(first_symbol_range != nullptr)
            {
                const u32 r = __ldg(first_symbol_range + u32(hi >> 48));
                a = r & 0xFFFFu; b = r >> 16;
            }
            while(a < b)
            {
                const u32 mid = (a + b) >> 1;
                const u64 ph = piv[2 * mid], pl = piv[2 * mid + 1];
                const bool le = (hi < ph) || (hi == ph && lo <= pl);
                if(le) b = mid; else a = mid + 1;
            }
            ids[k] = u16(a);
            if(local + k < tile_count) atomicAdd(&cnt[a], 1u);
            hi = (hi << 16) | (lo >> 48);
            lo = (lo << 16) | u64(win[local + k + 8]);
        }
        if(pid_out == nullptr) { /* sizes only */ }
        else if(local + ITEMS <= tile_count)
        {
            if constexpr(ITEMS % 8 == 0)
            {
                uint4* dst = reinterpret_cast<uint4*>(pid_out + (tile_first - first) + local);
                #pragma unroll
                for(int k = 0; k < ITEMS; k += 8)
                    dst[k / 8] = make_uint4(u32(ids[k]) | (u32(ids[k + 1]) << 16), u32(ids[k + 2]) | (u32(ids[k + 3]) << 16),
                                            u32(ids[k + 4]) | (u32(ids[k + 5]) << 16), u32(ids[k + 6]) | (u32(ids[k + 7]) << 16));
            }
            else
            {
                #pragma unroll
                for(int k = 0; k < ITEMS; ++k) pid_out[(tile_first - first) + local + k] = ids[k];
            }
        }
        else
        {
            for(int k = 0; k < ITEMS; ++k)
                if(local + k < tile_count) pid_out[(tile_first - first) + local + k] = ids[k];
        }
    }
    __syncthreads();
    for(u32 i = tid; i < p; i += BLOCK)
        if(cnt[i]) atomicAdd(&hist[i], u64(cnt[i]));
}

// Scatter of positions by partition id. A block takes BLOCK * ITEMS positions: counts them by partition in shared
// memory, reserves one run per partition with a single atomic on the partition's cursor, and writes every position
// into its run. Runs of a partition from different blocks follow one another in the order the blocks reserve them.
template <int BLOCK, int ITEMS>
__global__ void __launch_bounds__(BLOCK) scatter_by_pid_kernel(const u16* __restrict__ pid, const u64 first, const u64 count, const u32 p,
                                                              u32* const* __restrict__ part_base, u64* __restrict__ cursor)
{
    constexpr int TILE = BLOCK * ITEMS;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    u64* const base = reinterpret_cast<u64*>(smem_raw);        // p
    u32* const cnt = reinterpret_cast<u32*>(base + p);          // p
    const u32 tid = threadIdx.x;
    const u64 tile_first = u64(blockIdx.x) * TILE;
    for(u32 i = tid; i < p; i += BLOCK) cnt[i] = 0;
    __syncthreads();
    u16 id[ITEMS];
    u32 r[ITEMS];
    #pragma unroll
    for(int k = 0; k < ITEMS; ++k)
    {
        const u64 idx = tile_first + tid + u64(k) * BLOCK;
        if(idx < count)
        {
            id[k] = pid[idx];
            r[k] = atomicAdd(&cnt[id[k]], 1u);
        }
    }
    __syncthreads();
    for(u32 i = tid; i < p; i += BLOCK)
        if(cnt[i]) base[i] = atomicAdd(&cursor[i], u64(cnt[i]));
    __syncthreads();
    #pragma unroll
    for(int k = 0; k < ITEMS; ++k)
    {
        const u64 idx = tile_first + tid + u64(k) * BLOCK;
        if(idx < count) part_base[id[k]][base[id[k]] + r[k]] = u32(first + idx);
    }
}


// The same scatter for up to 256 partitions, built like a digit pass of the radix sort: the lanes of a warp that hold the
// same partition id find one another with ballots, warps keep private counters, the block reserves one run per partition
// with a single atomic on the partition's cursor, positions are staged in shared memory in partition order and written
// out as coalesced runs. Within a block's run the positions stay in increasing order.
template <int BLOCK, int ITEMS>
__global__ void __launch_bounds__(BLOCK) scatter_by_pid_ranked_kernel(const u16* __restrict__ pid, const u64 first, const u64 count, const u32 p,
                                                                     const int id_bits, u32* const* __restrict__ part_base, u64* __restrict__ cursor)
{
    constexpr int TILE = BLOCK * ITEMS;
    constexpr int WARPS = BLOCK / 32;
    constexpr int BINS = 256;
    __shared__ u32 stage[TILE];
    __shared__ u32 warp_cnt[WARPS * BINS];
    __shared__ u32 bin_start[BINS];       // start of the partition's records inside the tile
    __shared__ u64 bin_base[BINS];        // where the tile's run of the partition starts in the partition's array, minus bin_start
    __shared__ u32 scan_tot[BINS / 32];
    const u32 tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const u64 tile_first = u64(blockIdx.x) * TILE;
    const u32 valid = (count - tile_first < u64(TILE)) ? u32(count - tile_first) : u32(TILE);
    for(int i = tid; i < WARPS * BINS; i += BLOCK) warp_cnt[i] = 0;
    __syncthreads();

    u32 id[ITEMS], rank[ITEMS];
    const u32 warp_first = warp * 32 * ITEMS;
    #pragma unroll
    for(int i = 0; i < ITEMS; ++i)
    {
        const u32 idx = warp_first + i * 32 + lane;
        id[i] = (idx < valid) ? u32(pid[tile_first + idx]) : (BINS - 1);     // fillers rank last in the last bin
    }
    u32* const wc = warp_cnt + warp * BINS;
    {
        u32 peers[ITEMS], old[ITEMS];
        #pragma unroll
        for(int i = 0; i < ITEMS; ++i)
        {
            u32 m = 0xFFFFFFFFu;
            for(int b = 0; b < id_bits; ++b)
            {
                const u32 sel = 0u - ((id[i] >> b) & 1u);
                const u32 v = __ballot_sync(0xFFFFFFFFu, sel != 0);
                m &= ~(v ^ sel);
            }
            const u32 idx = warp_first + i * 32 + lane;
            // fillers must not meet real records of the last bin: split them off by their validity
            const u32 live = __ballot_sync(0xFFFFFFFFu, idx < valid);
            m &= (idx < valid) ? live : ~live;
            peers[i] = m;
        }
        #pragma unroll
        for(int i = 0; i < ITEMS; ++i)
        {
            const u32 idx = warp_first + i * 32 + lane;
            old[i] = 0;
            if(idx < valid && (peers[i] & lanemask_lt()) == 0) old[i] = atomicAdd(&wc[id[i]], u32(__popc(peers[i])));
        }
        #pragma unroll
        for(int i = 0; i < ITEMS; ++i)
            rank[i] = __shfl_sync(0xFFFFFFFFu, old[i], __ffs(peers[i]) - 1) + __popc(peers[i] & lanemask_lt());
    }
    __syncthreads();
    // per partition: the warps' offsets, the tile's count, an exclusive scan over the partitions, and the run's place
    u32 cnt = 0;
    u32 wsum[WARPS];
    if(tid < BINS)
    {
        #pragma unroll
        for(int w = 0; w < WARPS; ++w) { wsum[w] = warp_cnt[w * BINS + tid]; cnt += wsum[w]; }
    }
    u32 inc = cnt;
    if(tid < BINS)
    {
        #pragma unroll
        for(int o = 1; o < 32; o <<= 1)
        {
            const u32 t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
            if(int(lane) >= o) inc += t;
        }
        if(lane == 31) scan_tot[warp] = inc;
    }
    __syncthreads();
    if(tid < BINS)
    {
        u32 pre = 0;
        for(u32 w = 0; w < warp; ++w) pre += scan_tot[w];
        u32 run = pre + inc - cnt;
        bin_start[tid] = run;
        if(cnt && tid < p) bin_base[tid] = atomicAdd(&cursor[tid], u64(cnt)) - run;
        #pragma unroll
        for(int w = 0; w < WARPS; ++w) { warp_cnt[w * BINS + tid] = run; run += wsum[w]; }
    }
    __syncthreads();
    // Positions are staged in partition order; at write-out a record's partition is found again from its place in the tile
    // by a search over the partitions' starts (256 entries, 8 steps).
    #pragma unroll
    for(int i = 0; i < ITEMS; ++i)
    {
        const u32 idx = warp_first + i * 32 + lane;
        if(idx < valid) stage[wc[id[i]] + rank[i]] = u32(first + tile_first + idx);
    }
    __syncthreads();
    #pragma unroll
    for(int k = 0; k < ITEMS; ++k)
    {
        const u32 j = tid + k * BLOCK;
        if(j < valid)
        {
            u32 a = 0, b = BINS - 1;            // the last partition whose start is not after j
            while(a < b)
            {
                const u32 mid = (a + b + 1) >> 1;
                if(bin_start[mid] <= j) a = mid; else b = mid - 1;
            }
            part_base[a][bin_base[a] + j] = stage[j];
        }
    }
}


// The ranked scatter with the generation-0 keys made on the way: a tile covers consecutive text positions, so the four
// symbols a key packs come from one contiguous window of the text (read once, coalesced, into shared memory) instead of
// one 32-byte sector per suffix later, when the positions of a partition lie scattered over the text. The key goes to the
// same slot of `keys` as the position goes to in `sa`. text_limit = number of readable symbols (text and padding).
template <int BLOCK, int ITEMS>
__global__ void __launch_bounds__(BLOCK) scatter_keys_ranked_kernel(const u16* __restrict__ T, const u64 text_limit, const u16* __restrict__ pid,
                                                                   const u64 first, const u64 count, const u32 p, const int id_bits,
                                                                   const u64* __restrict__ part_off, u64* __restrict__ cursor,
                                                                   u32* __restrict__ sa, u64* __restrict__ keys)
{
    constexpr int TILE = BLOCK * ITEMS;
    constexpr int WARPS = BLOCK / 32;
    constexpr int BINS = 256;
    constexpr int WINDOW = TILE + 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    u64* const stage_key = reinterpret_cast<u64*>(smem_raw);                          // TILE
    u64* const bin_base = stage_key + TILE;                                           // BINS: slot in `sa` of the tile's run, minus bin_start
    u32* const stage_pos = reinterpret_cast<u32*>(bin_base + BINS);                   // TILE
    u32* const warp_cnt = stage_pos + TILE;                                           // WARPS * BINS
    u32* const scan_tot = warp_cnt + WARPS * BINS;                                    // 8
    u16* const window = reinterpret_cast<u16*>(scan_tot + 8);                         // WINDOW symbols
    u8* const stage_id = reinterpret_cast<u8*>(window + WINDOW);                      // TILE
    const u32 tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const u64 tile_first = u64(blockIdx.x) * TILE;
    const u32 valid = (count - tile_first < u64(TILE)) ? u32(count - tile_first) : u32(TILE);
    for(int i = tid; i < WARPS * BINS; i += BLOCK) warp_cnt[i] = 0;

    // the text window of the tile: symbols [first + tile_first, + TILE + 8)
    {
        const u64 w0 = first + tile_first;
        if((reinterpret_cast<uintptr_t>(T + w0) & 15) == 0)
        {
            for(u32 v = tid; v < WINDOW / 8; v += BLOCK)
            {
                const u64 a = w0 + u64(v) * 8;
                uint4 t = make_uint4(0, 0, 0, 0);
                if(a + 8 <= text_limit) t = *reinterpret_cast<const uint4*>(T + a);
                else
                {
                    u16 e[8];
                    #pragma unroll
                    for(int j = 0; j < 8; ++j) e[j] = (a + j < text_limit) ? T[a + j] : u16(0);
                    t = make_uint4(u32(e[0]) | (u32(e[1]) << 16), u32(e[2]) | (u32(e[3]) << 16), u32(e[4]) | (u32(e[5]) << 16), u32(e[6]) | (u32(e[7]) << 16));
                }
                reinterpret_cast<uint4*>(window)[v] = t;
            }
        }
        else
        {
            for(u32 v = tid; v < WINDOW; v += BLOCK) window[v] = (w0 + v < text_limit) ? T[w0 + v] : u16(0);
        }
    }
    __syncthreads();

    u32 id[ITEMS];
    u32 rank2[(ITEMS + 1) / 2];
    const u32 warp_first = warp * 32 * ITEMS;
    #pragma unroll
    for(int i = 0; i < ITEMS; ++i)
    {
        const u32 idx = warp_first + i * 32 + lane;
        id[i] = (idx < valid) ? u32(pid[tile_first + idx]) : (BINS - 1);     // fillers rank last in the last bin
    }
    u32* const wc = warp_cnt + warp * BINS;
    constexpr int CHUNK = 8;
    #pragma unroll
    for(int c = 0; c < ITEMS; c += CHUNK)
    {
        u32 peers[CHUNK], old[CHUNK];
        #pragma unroll
        for(int j = 0; j < CHUNK; ++j)
        {
            u32 m = 0xFFFFFFFFu;
            for(int b = 0; b < id_bits; ++b)
            {
                const u32 sel = 0u - ((id[c + j] >> b) & 1u);
                const u32 v = __ballot_sync(0xFFFFFFFFu, sel != 0);
                m &= ~(v ^ sel);
            }
            const u32 idx = warp_first + (c + j) * 32 + lane;
            // fillers must not meet real records of the last bin: split them off by their validity
            const u32 live = __ballot_sync(0xFFFFFFFFu, idx < valid);
            m &= (idx < valid) ? live : ~live;
            peers[j] = m;
        }
        #pragma unroll
        for(int j = 0; j < CHUNK; ++j)
        {
            const u32 idx = warp_first + (c + j) * 32 + lane;
            old[j] = 0;
            if(idx < valid && (peers[j] & lanemask_lt()) == 0) old[j] = atomicAdd(&wc[id[c + j]], u32(__popc(peers[j])));
        }
        #pragma unroll
        for(int j = 0; j < CHUNK; ++j)
        {
            const u32 r = __shfl_sync(0xFFFFFFFFu, old[j], __ffs(peers[j]) - 1) + __popc(peers[j] & lanemask_lt());
            if(((c + j) & 1) == 0) rank2[(c + j) >> 1] = r; else rank2[(c + j) >> 1] |= r << 16;
        }
    }
    __syncthreads();
    // per partition: the warps' offsets, the tile's count, an exclusive scan over the partitions, and the run's place
    static_assert(BLOCK >= BINS, "one thread per partition");
    u32 cnt = 0;
    u32 wsum[WARPS];
    if(tid < BINS)
    {
        #pragma unroll
        for(int w = 0; w < WARPS; ++w) { wsum[w] = warp_cnt[w * BINS + tid]; cnt += wsum[w]; }
    }
    u32 inc = cnt;
    if(tid < BINS)
    {
        #pragma unroll
        for(int o = 1; o < 32; o <<= 1)
        {
            const u32 t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
            if(int(lane) >= o) inc += t;
        }
        if(lane == 31) scan_tot[warp] = inc;
    }
    __syncthreads();
    if(tid < BINS)
    {
        u32 pre = 0;
        for(u32 w = 0; w < warp; ++w) pre += scan_tot[w];
        u32 run = pre + inc - cnt;
        if(cnt && tid < p) bin_base[tid] = part_off[tid] + atomicAdd(&cursor[tid], u64(cnt)) - run;
        #pragma unroll
        for(int w = 0; w < WARPS; ++w) { warp_cnt[w * BINS + tid] = run; run += wsum[w]; }
    }
    __syncthreads();
    #pragma unroll
    for(int i = 0; i < ITEMS; ++i)
    {
        const u32 idx = warp_first + i * 32 + lane;
        if(idx < valid)
        {
            const u32 at = wc[id[i]] + ((rank2[i >> 1] >> ((i & 1) * 16)) & 0xFFFFu);
            stage_pos[at] = u32(first + tile_first + idx);
            stage_key[at] = (u64(window[idx]) << 48) | (u64(window[idx + 1]) << 32) | (u64(window[idx + 2]) << 16) | u64(window[idx + 3]);
            stage_id[at] = u8(id[i]);
        }
    }
    __syncthreads();
    #pragma unroll
    for(int k = 0; k < ITEMS; ++k)
    {
        const u32 j = tid + k * BLOCK;
        if(j < valid)
        {
            const u64 dst = bin_base[stage_id[j]] + j;
            sa[dst] = stage_pos[j];
            keys[dst] = stage_key[j];
        }
    }
}

}   // namespace

extern "C" int csa_sample_kgrams(csa_ctx* ctx, const uint16_t* text, uint64_t n, uint64_t n_samples, uint64_t seed, uint64_t* samples)
{
    if(!ctx || !text || !samples || n == 0) return csa_fail(ctx, CSA_E_INVALID, "csa_sample_kgrams: bad argument");
    if(n_samples == 0) return CSA_OK;
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    sample_kgrams_kernel<<<unsigned(div_up(n_samples, 256)), 256, 0, ctx->stream>>>(text, n, n_samples, seed, reinterpret_cast<u64*>(samples));
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

extern "C" int csa_select_pivots(const uint64_t* samples, uint64_t n_samples, uint32_t p, uint64_t* pivots, uint32_t* p_out)
{
    if(!samples || !p_out || p == 0 || (p > 1 && !pivots)) return CSA_E_INVALID;
    if(p > CSA_MAX_PARTITIONS) return CSA_E_LIMIT;
    std::vector<std::pair<u64, u64>> s(n_samples);
    for(u64 i = 0; i < n_samples; ++i) s[i] = {samples[2 * i], samples[2 * i + 1]};
    // Only the p-1 order statistics at equal strides are needed: they are placed by nested selections (O(n log p))
    // instead of a full sort.
    std::vector<u64> want;
    for(u32 j = 1; j < p && n_samples > 0; ++j)
    {
        const u64 at = (u64(j) * n_samples) / p;
        want.push_back(at == 0 ? 0 : at - 1);
    }
    struct Job { u64 lo, hi; size_t a, b; };           // select want[a, b) inside s[lo, hi)
    std::vector<Job> jobs;
    if(!want.empty()) jobs.push_back({0, n_samples, 0, want.size()});
    while(!jobs.empty())
    {
        const Job j = jobs.back();
        jobs.pop_back();
        if(j.a >= j.b || j.lo >= j.hi) continue;
        const size_t m = (j.a + j.b) / 2;
        const u64 r = want[m];
        std::nth_element(s.begin() + j.lo, s.begin() + r, s.begin() + j.hi);
        jobs.push_back({j.lo, r, j.a, m});
        jobs.push_back({r + 1, j.hi, m + 1, j.b});
    }
    u32 made = 0;
    for(size_t k = 0; k < want.size(); ++k)
    {
        const auto& c = s[want[k]];
        if(made > 0 && pivots[2 * (made - 1)] == c.first && pivots[2 * (made - 1) + 1] == c.second) continue;    // equal K-grams never split
        pivots[2 * made] = c.first;
        pivots[2 * made + 1] = c.second;
        ++made;
    }
    *p_out = made + 1;
    return CSA_OK;
}

constexpr int PID_BLOCK = 256, PID_ITEMS = 16;

__global__ void split_samples_kernel(const u64* __restrict__ samples, const u64 count, u64* __restrict__ hi, u32* __restrict__ idx)
{
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if(i < count) { hi[i] = samples[2 * i]; idx[i] = u32(i); }
}

// Optional table for csa_partition_ids, kept in the context: for every first symbol the lowest and the highest partition
// that a K-gram starting with it can fall into (low and high 16 bits). Installed by partition_install_symbol_ranges.

int partition_install_symbol_ranges(csa_ctx* ctx, const u64* pivots_host, u32 p, u32* table_dev)
{
    if(table_dev == nullptr) { ctx->symbol_range = nullptr; return CSA_OK; }
    std::vector<u32> t(65536);
    // pid(k) = number of splitters smaller than k. For K-grams starting with s: from pid(s,0,...,0) to pid(s,FFFF,...,FFFF).
    u32 a = 0, b = 0;
    for(u32 s = 0; s < 65536; ++s)
    {
        const u64 lo_h = u64(s) << 48, hi_h = lo_h | 0x0000FFFFFFFFFFFFull;
        while(a < p - 1 && (pivots_host[2 * a] < lo_h)) ++a;                                     // splitters < (lo_h, 0): hi word smaller
        while(b < p - 1 && (pivots_host[2 * b] < hi_h || (pivots_host[2 * b] == hi_h && pivots_host[2 * b + 1] < ~0ull))) ++b;
        t[s] = a | (b << 16);
    }
    CSA_CUDA(ctx, cudaMemcpyAsync(table_dev, t.data(), 65536 * 4, cudaMemcpyHostToDevice, ctx->stream));
    CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    ctx->symbol_range = table_dev;
    return CSA_OK;
}

extern "C" int csa_install_pivots(csa_ctx* ctx, const uint64_t* pivots_host, uint32_t p)
{
    if(!ctx || p > CSA_MAX_PARTITIONS || (p > 1 && !pivots_host)) return csa_fail(ctx, CSA_E_INVALID, "csa_install_pivots: bad argument");
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    if(p <= 1) return partition_install_symbol_ranges(ctx, nullptr, 0, nullptr);
    if(!ctx->symbol_table) CSA_CUDA(ctx, cudaMalloc(&ctx->symbol_table, 65536 * sizeof(u32)));
    return partition_install_symbol_ranges(ctx, reinterpret_cast<const u64*>(pivots_host), p, ctx->symbol_table);
}

extern "C" int csa_partition_ids(csa_ctx* ctx, const uint16_t* text, uint64_t n, uint64_t first, uint64_t count, const uint64_t* pivots,
                                 uint32_t p, uint16_t* pid, uint64_t* hist)
{
    if(!ctx || !text || !hist || p == 0 || (p > 1 && !pivots) || first + count > n) return csa_fail(ctx, CSA_E_INVALID, "csa_partition_ids: bad argument");
    if(p > CSA_MAX_PARTITIONS) return csa_fail(ctx, CSA_E_LIMIT, "csa_partition_ids: too many partitions");
    if((reinterpret_cast<uintptr_t>(text) & 15) || (first & 7) || (reinterpret_cast<uintptr_t>(pid) & 15))
        return csa_fail(ctx, CSA_E_INVALID, "csa_partition_ids: text and pid must be 16-byte aligned and `first` a multiple of 8");
    if(count == 0) return CSA_OK;
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    constexpr int TILE = PID_BLOCK * PID_ITEMS;
    const size_t smem = (TILE + 8) * 2 + 16 + size_t(2) * (p > 1 ? p - 1 : 1) * 8 + size_t(p) * 4;
    auto kern = partition_ids_kernel<PID_BLOCK, PID_ITEMS>;
    CSA_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    kern<<<unsigned(div_up(count, TILE)), PID_BLOCK, smem, ctx->stream>>>(text, n, first, count, reinterpret_cast<const u64*>(pivots), p, ctx->symbol_range, pid,
                                                                          reinterpret_cast<u64*>(hist), ctx->d_status);
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

extern "C" int csa_scatter_by_pid(csa_ctx* ctx, const uint16_t* pid, uint64_t first, uint64_t count, uint32_t p, uint32_t* const* part_base,
                                  uint64_t* cursor)
{
    if(!ctx || !pid || !part_base || !cursor || p == 0) return csa_fail(ctx, CSA_E_INVALID, "csa_scatter_by_pid: bad argument");
    if(p > CSA_MAX_PARTITIONS) return csa_fail(ctx, CSA_E_LIMIT, "csa_scatter_by_pid: too many partitions");
    if(first + count > 0xFFFFFFFFull) return csa_fail(ctx, CSA_E_LIMIT, "csa_scatter_by_pid: positions must fit 32 bits");
    if(count == 0) return CSA_OK;
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    if(p <= 256)
    {
        constexpr int RB = 512, RI = 8;
        scatter_by_pid_ranked_kernel<RB, RI><<<unsigned(div_up(count, RB * RI)), RB, 0, ctx->stream>>>(pid, first, count, p, bits_for(p - 1), part_base,
                                                                                                     reinterpret_cast<u64*>(cursor));
        CSA_LAUNCH_CHECK(ctx);
        return CSA_OK;
    }
    constexpr int TILE = PID_BLOCK * PID_ITEMS;
    const size_t smem = size_t(p) * 12;
    auto kern = scatter_by_pid_kernel<PID_BLOCK, PID_ITEMS>;
    CSA_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    kern<<<unsigned(div_up(count, TILE)), PID_BLOCK, smem, ctx->stream>>>(pid, first, count, p, part_base, reinterpret_cast<u64*>(cursor));
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}


// Scatter of the positions [first, first + count) into `sa` by partition id together with their generation-0 keys into
// the same slots of `keys`; partition q owns the slots from part_off[q] on (device array). Up to 256 partitions.
int launch_scatter_with_keys(csa_ctx* ctx, const u16* T, u64 text_limit, const u16* pid, u64 first, u64 count, u32 p, const u64* part_off, u64* cursor,
                             u32* sa, u64* keys)
{
    if(p == 0 || p > 256) return csa_fail(ctx, CSA_E_LIMIT, "scatter with keys: 1 to 256 partitions");
    if(first + count > 0xFFFFFFFFull) return csa_fail(ctx, CSA_E_LIMIT, "scatter with keys: positions must fit 32 bits");
    if(count == 0) return CSA_OK;
    constexpr int SB = 256, SI = 16, TILE = SB * SI;
    constexpr size_t smem = size_t(TILE) * 8 + 256 * 8 + size_t(TILE) * 4 + size_t(SB / 32) * 256 * 4 + 8 * 4 + size_t(TILE + 8) * 2 + TILE;
    auto kern = scatter_keys_ranked_kernel<SB, SI>;
    static std::atomic<bool> configured[64];
    if(!configured[ctx->device & 63])
    {
        CSA_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        configured[ctx->device & 63] = true;
    }
    kern<<<unsigned(div_up(count, TILE)), SB, smem, ctx->stream>>>(T, text_limit, pid, first, count, p, bits_for(p - 1), part_off, cursor, sa, keys);
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

// Samples K-grams, orders them (the first words by the device's radix sort, ties on the first word by their second words
// on the host) and picks the splitters as csa_select_pivots does. scratch must hold pick_splitters_scratch_bytes(n_samples).
size_t pick_splitters_scratch_bytes(u64 n_samples)
{
    return align_up256(n_samples * 16) + 2 * align_up256(n_samples * 8) + 2 * align_up256(n_samples * 4) + align_up256(csa_sort_workspace_bytes(n_samples)) + 1024;
}

namespace
{
int order_samples_and_pick(csa_ctx* ctx, const u64* samples, u64 n_samples, u32 p, u64* hiA, u64* hiB, u32* ixA, u32* ixB, void* ws, size_t wsb, u64* pivots_host, u32* p_out);
}

int pick_splitters(csa_ctx* ctx, const u16* T, u64 n, u32 p, u64 seed, u64 n_samples, void* scratch, size_t scratch_bytes, u64* pivots_host, u32* p_out)
{
    Carver cv(scratch, scratch_bytes);
    u64* samples = cv.take<u64>(2 * n_samples);
    u64* hiA = cv.take<u64>(n_samples);
    u64* hiB = cv.take<u64>(n_samples);
    u32* ixA = cv.take<u32>(n_samples);
    u32* ixB = cv.take<u32>(n_samples);
    const size_t wsb = csa_sort_workspace_bytes(n_samples);
    void* ws = cv.take<u8>(wsb);
    if(!cv.ok) return csa_fail(ctx, CSA_E_NOMEM, "splitters: scratch too small");
    CSA_TRY(csa_sample_kgrams(ctx, T, n, n_samples, seed, reinterpret_cast<uint64_t*>(samples)));
    return order_samples_and_pick(ctx, samples, n_samples, p, hiA, hiB, ixA, ixB, ws, wsb, pivots_host, p_out);
}

// The same from samples that lie in device memory already (a text sharded over several GPUs: every GPU samples its stretch
// and the samples meet by the caller's all-gather). The scratch comes from the context's arena.
extern "C" int csa_select_pivots_dev(csa_ctx* ctx, const uint64_t* samples_dev, uint64_t n_samples, uint32_t p, uint64_t* pivots_host, uint32_t* p_out)
{
    if(!ctx || !samples_dev || !pivots_host || !p_out || n_samples == 0 || p == 0 || p > CSA_MAX_PARTITIONS) return csa_fail(ctx, CSA_E_INVALID, "csa_select_pivots_dev: bad argument");
    if(n_samples >= (u64(1) << 31)) return csa_fail(ctx, CSA_E_LIMIT, "csa_select_pivots_dev: too many samples");
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    const size_t wsb = csa_sort_workspace_bytes(n_samples);
    const size_t need = 2 * align_up256(n_samples * 8) + 2 * align_up256(n_samples * 4) + align_up256(wsb) + 1024;
    void* scratch = nullptr;
    CSA_TRY(csa_arena(ctx, need, &scratch));
    Carver cv(scratch, ctx->arena_bytes);
    u64* hiA = cv.take<u64>(n_samples);
    u64* hiB = cv.take<u64>(n_samples);
    u32* ixA = cv.take<u32>(n_samples);
    u32* ixB = cv.take<u32>(n_samples);
    void* ws = cv.take<u8>(wsb);
    if(!cv.ok) return csa_fail(ctx, CSA_E_NOMEM, "csa_select_pivots_dev: scratch too small");
    return order_samples_and_pick(ctx, reinterpret_cast<const u64*>(samples_dev), n_samples, p, hiA, hiB, ixA, ixB, ws, wsb, reinterpret_cast<u64*>(pivots_host), p_out);
}

namespace
{
int order_samples_and_pick(csa_ctx* ctx, const u64* samples, u64 n_samples, u32 p, u64* hiA, u64* hiB, u32* ixA, u32* ixB, void* ws, size_t wsb, u64* pivots_host, u32* p_out)
{
    split_samples_kernel<<<unsigned(div_up(n_samples, 256)), 256, 0, ctx->stream>>>(samples, n_samples, hiA, ixA);
    CSA_LAUNCH_CHECK(ctx);
    int in_alt = 0;
    CSA_TRY(csa_sort_pairs(ctx, reinterpret_cast<uint64_t*>(hiA), reinterpret_cast<uint64_t*>(hiB), ixA, ixB, 4, n_samples, 0, 64, ws, wsb, &in_alt));
    std::vector<u64> all(2 * n_samples);
    std::vector<u32> order(n_samples);
    CSA_CUDA(ctx, cudaMemcpyAsync(all.data(), samples, all.size() * 8, cudaMemcpyDeviceToHost, ctx->stream));
    CSA_CUDA(ctx, cudaMemcpyAsync(order.data(), in_alt ? ixB : ixA, order.size() * 4, cudaMemcpyDeviceToHost, ctx->stream));
    CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    // runs of equal first words are put in order of their second words
    for(u64 a = 0; a < n_samples; )
    {
        u64 b = a + 1;
        while(b < n_samples && all[2 * u64(order[b])] == all[2 * u64(order[a])]) ++b;
        if(b - a > 1) std::sort(order.begin() + a, order.begin() + b, [&](u32 x, u32 y) { return all[2 * u64(x) + 1] < all[2 * u64(y) + 1]; });
        a = b;
    }
    u32 made = 0;
    for(u32 j = 1; j < p && n_samples > 0; ++j)
    {
        const u64 at = (u64(j) * n_samples) / p;
        const u64 k = order[at == 0 ? 0 : at - 1];
        const u64 h = all[2 * k], l = all[2 * k + 1];
        if(made > 0 && pivots_host[2 * (made - 1)] == h && pivots_host[2 * (made - 1) + 1] == l) continue;      // equal K-grams never split
        pivots_host[2 * made] = h;
        pivots_host[2 * made + 1] = l;
        ++made;
    }
    *p_out = made + 1;
    return CSA_OK;
}
}   // namespace
