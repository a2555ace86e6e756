// Prefix doubling inside partitions: key building for the initial sort and for every later generation, and the
// scan-based step that turns a sorted list of tied suffixes into new slots, new ranks and the next active list.
//
// State kept by a build, per GPU: `sa` (local slots -> text positions, in current order), the inverse array `isa`
// (text position -> global rank of the head of the suffix's group, sharded by position over the GPUs), and the
// active list (head slot, position) of the suffixes that are still tied with a neighbour.
//
// Reference behaviour followed, not its code: initial ranking and filtering (src/GPU_SACA.cu:1111-1331 with
// initialize_key_group_ranks_and_mark_active_flags_kernel, include/GPU_SACA.cuh:191-208), re-ranking of generation
// t >= 1 (src/GPU_SACA.cu:1714-1995; rank_key_groups..., refine_primary_keys_kernel, include/GPU_SACA.cuh:218-280)
// and the stable split into active and retired suffixes (cub::DevicePartition::Flagged at src/GPU_SACA.cu:1253, 1917).
// The reference pushes ranks to partitions as messages and joins them by search; here a rank is written straight
// into the position-sharded inverse array (on the GPU that owns the position) and read from there.
#include "common.cuh"
#include "part.cuh"

namespace
{

__device__ __forceinline__ u32* isa_slot(const Isa_View& v, u64 x)
{
    if(v.gpus == 1) return v.shard[0] + x;
    const u64 g = x / v.shard_size;
    return v.shard[g] + (x - g * v.shard_size);
}

__device__ __forceinline__ u64 global_of(const Slot_Map& m, u32 slot)
{
    if(m.segs == 0) return m.base + slot;
    u32 a = 0, b = m.segs - 1;             // the last local partition that starts at or before the slot
    while(a < b)
    {
        const u32 mid = (a + b + 1) >> 1;
        if(__ldg(m.seg_first + mid) <= slot) a = mid; else b = mid - 1;
    }
    return __ldg(m.seg_delta + a) + slot;
}

__global__ void keys_gen0_kernel(const u16* __restrict__ T, const u32* __restrict__ pos, const u64 count, u64* __restrict__ keys)
{
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if(i < count) keys[i] = pack4(T, pos[i]);
}

__global__ void keys_gen_kernel(const u32* __restrict__ head, const u32* __restrict__ pos, const u64 count, const u64 n, const u64 h,
                                const int sec_bits, const Isa_View isa, u64* __restrict__ keys)
{
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if(i >= count) return;
    const u64 x = u64(pos[i]) + h;
    const u64 sec = (x < n) ? u64(*isa_slot(isa, x)) + h : (n - 1 + h - x);
    keys[i] = (u64(head[i]) << sec_bits) | sec;
}

// ---- block-wide scans over RANK_BLOCK threads ------------------------------------------------------------------

__device__ __forceinline__ u32 warp_inclusive_max(u32 v)
{
    #pragma unroll
    for(int o = 1; o < 32; o <<= 1)
    {
        const u32 t = __shfl_up_sync(0xFFFFFFFFu, v, o);
        if(int(lane_id()) >= o) v = max(v, t);
    }
    return v;
}

__device__ __forceinline__ u32 warp_inclusive_sum(u32 v)
{
    #pragma unroll
    for(int o = 1; o < 32; o <<= 1)
    {
        const u32 t = __shfl_up_sync(0xFFFFFFFFu, v, o);
        if(int(lane_id()) >= o) v += t;
    }
    return v;
}

// Heads are carried as (index + 1), 0 meaning "no head seen yet".
struct Tile_Flags
{
    u32 prim_head;   // bit i: record i of the thread starts a group of equal primaries
    u32 full_head;   // bit i: record i starts a group of equal full keys
    u32 active;      // bit i: record i is tied with a neighbour on the full key
};

// Loads the thread's RANK_ITEMS consecutive keys (with the neighbours on both sides) and derives the flags.
__device__ __forceinline__ Tile_Flags load_flags(const u64* __restrict__ keys, const u64 count, const u64 first, const int prim_shift,
                                                 u64 (&k)[RANK_ITEMS])
{
    Tile_Flags f{0, 0, 0};
    if(first >= count) return f;
    u64 prev = (first > 0) ? keys[first - 1] : 0;
    if(first + RANK_ITEMS <= count && ((reinterpret_cast<uintptr_t>(keys + first) & 15) == 0))
    {
        const ulonglong2* v = reinterpret_cast<const ulonglong2*>(keys + first);
        #pragma unroll
        for(int i = 0; i < RANK_ITEMS; i += 2) { const ulonglong2 t = v[i / 2]; k[i] = t.x; k[i + 1] = t.y; }
    }
    else
    {
        #pragma unroll
        for(int i = 0; i < RANK_ITEMS; ++i) k[i] = (first + i < count) ? keys[first + i] : 0;
    }
    const u64 after = (first + RANK_ITEMS < count) ? keys[first + RANK_ITEMS] : 0;
    #pragma unroll
    for(int i = 0; i < RANK_ITEMS; ++i)
    {
        if(first + i >= count) break;
        const u64 p = (i == 0) ? prev : k[i - 1];
        const bool is_first = (first + i == 0);
        const bool fh = is_first || (k[i] != p);
        const bool ph = is_first || (prim_shift < 64 && (k[i] >> prim_shift) != (p >> prim_shift));
        const bool has_next = (first + i + 1 < count);
        const u64 nx = (i + 1 < RANK_ITEMS) ? k[i + 1] : after;
        const bool next_head = !has_next || (nx != k[i]);
        if(fh) f.full_head |= 1u << i;
        if(ph) f.prim_head |= 1u << i;
        if(!(fh && next_head)) f.active |= 1u << i;
    }
    return f;
}

// Phase 1: per tile, the last group heads (as index + 1) and the number of active records.
__global__ void __launch_bounds__(RANK_BLOCK) rank_tile_kernel(const u64* __restrict__ keys, const u64 count, const int prim_shift, u32* __restrict__ agg)
{
    __shared__ u32 s_prim[RANK_BLOCK / 32], s_full[RANK_BLOCK / 32], s_act[RANK_BLOCK / 32];
    const u64 first = u64(blockIdx.x) * RANK_TILE + u64(threadIdx.x) * RANK_ITEMS;
    u64 k[RANK_ITEMS];
    const Tile_Flags f = load_flags(keys, count, first, prim_shift, k);
    u32 lp = f.prim_head ? u32(first) + (31 - __clz(f.prim_head)) + 1 : 0;
    u32 lf = f.full_head ? u32(first) + (31 - __clz(f.full_head)) + 1 : 0;
    u32 ac = __popc(f.active);
    #pragma unroll
    for(int o = 16; o > 0; o >>= 1)
    {
        lp = max(lp, __shfl_xor_sync(0xFFFFFFFFu, lp, o));
        lf = max(lf, __shfl_xor_sync(0xFFFFFFFFu, lf, o));
        ac += __shfl_xor_sync(0xFFFFFFFFu, ac, o);
    }
    if(lane_id() == 0) { s_prim[threadIdx.x >> 5] = lp; s_full[threadIdx.x >> 5] = lf; s_act[threadIdx.x >> 5] = ac; }
    __syncthreads();
    if(threadIdx.x == 0)
    {
        u32 a = 0, b = 0, c = 0;
        for(int w = 0; w < RANK_BLOCK / 32; ++w) { a = max(a, s_prim[w]); b = max(b, s_full[w]); c += s_act[w]; }
        agg[3 * u64(blockIdx.x)] = a;
        agg[3 * u64(blockIdx.x) + 1] = b;
        agg[3 * u64(blockIdx.x) + 2] = c;
    }
}

// Phase 2: one block turns the tile aggregates into carries: exclusive running maxima of the heads and the exclusive
// running sum of the active counts, which starts at the current length of the next list; the length is then advanced.
__global__ void __launch_bounds__(1024) rank_carry_kernel(u32* __restrict__ agg, const u64 tiles, u64* __restrict__ act_count)
{
    __shared__ u32 s_a[32], s_b[32];
    __shared__ u64 s_c[32];
    __shared__ u32 carry_a, carry_b;
    __shared__ u64 carry_c;
    if(threadIdx.x == 0) { carry_a = 0; carry_b = 0; carry_c = *act_count; }
    __syncthreads();
    for(u64 base = 0; base < tiles; base += 1024)
    {
        const u64 t = base + threadIdx.x;
        u32 a = 0, b = 0; u32 c = 0;
        if(t < tiles) { a = agg[3 * t]; b = agg[3 * t + 1]; c = agg[3 * t + 2]; }
        const u32 ia = warp_inclusive_max(a), ib = warp_inclusive_max(b), ic = warp_inclusive_sum(c);
        if(lane_id() == 31) { s_a[threadIdx.x >> 5] = ia; s_b[threadIdx.x >> 5] = ib; s_c[threadIdx.x >> 5] = ic; }
        __syncthreads();
        u32 pa = carry_a, pb = carry_b; u64 pc = carry_c;
        for(u32 w = 0; w < (threadIdx.x >> 5); ++w) { pa = max(pa, s_a[w]); pb = max(pb, s_b[w]); pc += s_c[w]; }
        // exclusive values for this tile
        const u32 ea = max(pa, __shfl_up_sync(0xFFFFFFFFu, ia, 1) * (lane_id() > 0));
        const u32 eb = max(pb, __shfl_up_sync(0xFFFFFFFFu, ib, 1) * (lane_id() > 0));
        const u64 ec = pc + (ic - c);
        __syncthreads();
        if(threadIdx.x == 1023) { carry_a = max(pa, ia); carry_b = max(pb, ib); carry_c = pc + ic; }
        if(t < tiles)
        {
            agg[3 * t] = ea; agg[3 * t + 1] = eb;
            // the running sum may pass 2^32 only if the list does, which the build's size limit excludes
            agg[3 * t + 2] = u32(ec);
        }
        __syncthreads();
    }
    if(threadIdx.x == 0) *act_count = carry_c;
}

// Phase 3: every record gets its slot and rank; tied records go to the next list.
// `pos` may be the very slot range of `sa` that the records go to (generation 0 sorts in place): such a record is not rewritten.
__global__ void __launch_bounds__(RANK_BLOCK) rank_apply_kernel(const u64* __restrict__ keys, const u32* pos, const u64 count,
                                                               const int prim_shift, const u32 fixed_head, const Isa_View isa, const Slot_Map map,
                                                               u32* sa, u32* __restrict__ next_head, u32* __restrict__ next_pos,
                                                               const u32* __restrict__ agg, u64* __restrict__ updates)
{
    __shared__ u32 s_prim[RANK_BLOCK / 32], s_full[RANK_BLOCK / 32], s_act[RANK_BLOCK / 32];
    __shared__ u32 s_next_head[RANK_TILE], s_next_pos[RANK_TILE];     // the tile's tied records, gathered for a coalesced write
    const u64 first = u64(blockIdx.x) * RANK_TILE + u64(threadIdx.x) * RANK_ITEMS;
    // Everything the block reads is asked for at once: the tile's carries, the thread's positions, then its keys.
    const u32 carry_p = agg[3 * u64(blockIdx.x)], carry_f = agg[3 * u64(blockIdx.x) + 1];
    const u32 out_base = agg[3 * u64(blockIdx.x) + 2];      // where the tile's tied records start in the next list
    // A thread's records are consecutive: positions come in and updates go out as 16-byte vectors where the thread's
    // stretch is whole and aligned (every tile but the last is, as the lists start on 16-byte boundaries).
    const bool whole = first + RANK_ITEMS <= count;
    u32 ps[RANK_ITEMS];
    if(whole && ((reinterpret_cast<uintptr_t>(pos + first) & 15) == 0))
    {
        const uint4* v = reinterpret_cast<const uint4*>(pos + first);
        #pragma unroll
        for(int i = 0; i < RANK_ITEMS; i += 4) { const uint4 t = v[i / 4]; ps[i] = t.x; ps[i + 1] = t.y; ps[i + 2] = t.z; ps[i + 3] = t.w; }
    }
    else
    {
        #pragma unroll
        for(int i = 0; i < RANK_ITEMS; ++i) ps[i] = (first + i < count) ? pos[first + i] : 0;
    }
    u64 k[RANK_ITEMS];
    const Tile_Flags f = load_flags(keys, count, first, prim_shift, k);

    // Thread-local last heads and active count, then block-wide exclusive scans with the tile's carries.
    const u32 lp = f.prim_head ? u32(first) + (31 - __clz(f.prim_head)) + 1 : 0;
    const u32 lf = f.full_head ? u32(first) + (31 - __clz(f.full_head)) + 1 : 0;
    const u32 ac = __popc(f.active);
    const u32 ip = warp_inclusive_max(lp), ifl = warp_inclusive_max(lf), ia = warp_inclusive_sum(ac);
    if(lane_id() == 31) { s_prim[threadIdx.x >> 5] = ip; s_full[threadIdx.x >> 5] = ifl; s_act[threadIdx.x >> 5] = ia; }
    __syncthreads();
    u32 run_p = carry_p, run_f = carry_f;
    u32 out = 0, tile_active = 0;
    for(u32 w = 0; w < RANK_BLOCK / 32; ++w)
    {
        if(w < (threadIdx.x >> 5)) { run_p = max(run_p, s_prim[w]); run_f = max(run_f, s_full[w]); out += s_act[w]; }
        tile_active += s_act[w];
    }
    {
        const u32 up = __shfl_up_sync(0xFFFFFFFFu, ip, 1), uf = __shfl_up_sync(0xFFFFFFFFu, ifl, 1);
        if(lane_id() > 0) { run_p = max(run_p, up); run_f = max(run_f, uf); }
        out += ia - ac;
    }
    if(first < count)
    {
        const bool vector_updates = updates && whole && ((reinterpret_cast<uintptr_t>(updates + first) & 15) == 0);
        u64 up[RANK_ITEMS];

        #pragma unroll
        for(int i = 0; i < RANK_ITEMS; ++i)
        {
            const u64 idx = first + i;
            if(idx >= count) break;
            if(f.prim_head & (1u << i)) run_p = u32(idx) + 1;
            if(f.full_head & (1u << i)) run_f = u32(idx) + 1;
            const u32 group_start = run_p - 1, sub_start = run_f - 1;      // indices into the sorted list
            const u32 head = (prim_shift < 64) ? u32(k[i] >> prim_shift) : fixed_head;
            const u32 slot = head + (u32(idx) - group_start);
            const u32 new_head = head + (sub_start - group_start);
            if(sa + slot != pos + idx) sa[slot] = ps[i];
            // The new rank goes straight into the inverse array, or, when the array is spread over several GPUs, into a list
            // of (position, rank) updates that is applied in address order (and, over several GPUs, routed to the positions' owners).
            const u32 global_rank = u32(global_of(map, head) + (new_head - head));      // a group lies inside one partition
            up[i] = (u64(ps[i]) << 32) | global_rank;
            if(updates) { if(!vector_updates) updates[idx] = up[i]; }
            else *isa_slot(isa, ps[i]) = global_rank;
            if(f.active & (1u << i))
            {
                s_next_head[out] = new_head;
                s_next_pos[out] = ps[i];
                ++out;
            }
        }
        if(vector_updates)
        {
            ulonglong2* dst = reinterpret_cast<ulonglong2*>(updates + first);
            #pragma unroll
            for(int i = 0; i < RANK_ITEMS; i += 2) dst[i / 2] = make_ulonglong2(up[i], up[i + 1]);
        }
    }
    __syncthreads();
    for(u32 j = threadIdx.x; j < tile_active; j += RANK_BLOCK)
    {
        next_head[out_base + j] = s_next_head[j];
        next_pos[out_base + j] = s_next_pos[j];
    }
}

__global__ void pack_sa40_kernel(const u32* __restrict__ sa, const u64 count, u8* __restrict__ out)
{
    // A thread packs 16 entries = 80 bytes = five 16-byte stores.
    const u64 g = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    const u64 first = g * 16;
    if(first >= count) return;
    if(first + 16 <= count)
    {
        u32 v[16];
        const uint4* src = reinterpret_cast<const uint4*>(sa + first);
        #pragma unroll
        for(int i = 0; i < 4; ++i) { const uint4 t = src[i]; v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w; }
        // byte stream: entry e occupies bytes [5e, 5e+5) = v[e] little-endian then a zero byte
        u32 w[20];
        #pragma unroll
        for(int j = 0; j < 20; ++j) w[j] = 0;
        #pragma unroll
        for(int e = 0; e < 16; ++e)
        {
            const int b = 5 * e, wi = b >> 2, sh = (b & 3) * 8;
            w[wi] |= v[e] << sh;
            if(sh) w[wi + 1] |= v[e] >> (32 - sh);
        }
        uint4* dst = reinterpret_cast<uint4*>(out + first * 5);
        #pragma unroll
        for(int i = 0; i < 5; ++i) dst[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
    }
    else
    {
        for(u64 r = first; r < count; ++r)
        {
            const u32 x = sa[r];
            out[5 * r] = u8(x); out[5 * r + 1] = u8(x >> 8); out[5 * r + 2] = u8(x >> 16); out[5 * r + 3] = u8(x >> 24); out[5 * r + 4] = 0;
        }
    }
}

}   // namespace

int launch_keys_gen0(csa_ctx* ctx, const u16* T, const u32* pos, u64 count, u64* keys)
{
    if(count == 0) return CSA_OK;
    keys_gen0_kernel<<<unsigned(div_up(count, 256)), 256, 0, ctx->stream>>>(T, pos, count, keys);
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

int launch_keys_gen(csa_ctx* ctx, const u32* head, const u32* pos, u64 count, u64 n, u64 h, int sec_bits, Isa_View isa, u64* keys)
{
    if(count == 0) return CSA_OK;
    keys_gen_kernel<<<unsigned(div_up(count, 256)), 256, 0, ctx->stream>>>(head, pos, count, n, h, sec_bits, isa, keys);
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

int launch_rank_and_compact(csa_ctx* ctx, const u64* keys, const u32* pos, u64 count, int prim_shift, u32 fixed_head, Isa_View isa,
                            Slot_Map map, u32* sa, u32* next_head, u32* next_pos, u64* act_count, u32* scratch, u64* updates)
{
    if(count == 0) return CSA_OK;
    const u64 tiles = div_up(count, RANK_TILE);
    rank_tile_kernel<<<unsigned(tiles), RANK_BLOCK, 0, ctx->stream>>>(keys, count, prim_shift, scratch);
    CSA_LAUNCH_CHECK(ctx);
    rank_carry_kernel<<<1, 1024, 0, ctx->stream>>>(scratch, tiles, act_count);
    CSA_LAUNCH_CHECK(ctx);
    rank_apply_kernel<<<unsigned(tiles), RANK_BLOCK, 0, ctx->stream>>>(keys, pos, count, prim_shift, fixed_head, isa, map, sa, next_head,
                                                                       next_pos, scratch, updates);
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

int launch_pack_sa40(csa_ctx* ctx, const u32* sa, u64 count, u8* sa40)
{
    if(count == 0) return CSA_OK;
    pack_sa40_kernel<<<unsigned(div_up(div_up(count, 16), 256)), 256, 0, ctx->stream>>>(sa, count, sa40);
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}
