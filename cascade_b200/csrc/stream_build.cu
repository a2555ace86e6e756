// The build with the partition as the unit of device work, for texts whose suffix lists do not fit the device and for
// positions beyond 32 bits (up to 2^40, 5-byte lanes as in the reference, include/lane.hpp:22-26).
//
// What stays on the device for the whole build is small and position-indexed: the text (2 bytes per position) and the rank
// store R (4 bytes per position: the rank of the suffix inside its part). What is large and rank-ordered, the parts' suffix
// lists (5-byte lanes and 4-byte ranks, 9 bytes per suffix), lives in host memory and streams through the device one part
// at a time, as the reference streams partitions through its three dispatcher threads (src/GPU_SACA.cu:1334-1608):
//
//   generation 0 of a part   (sort_and_init_rank_and_filter, src/GPU_SACA.cu:1111-1331)   csa_rank_gen0
//   generation t of a part   (sort_and_re_rank_and_filter,   src/GPU_SACA.cu:1714-1995)   csa_rank_gen
//   the exchange between two generations (messages, include/message.hpp:22-61)              csa_exchange_messages
//   the final order of a part (scatter_to_rank_order, src/GPU_SACA.cu:2106-2164)           csa_rank_order
//
// Ranks are local to a part (below 2^31, include/bit-layout.hpp:51-68), so a (rank, rank of the suffix h further on)
// pair fits one 64-bit sort key whatever the text's length. That needs the reference's invariant: suffixes that are
// still tied always take their second rank from one and the same part. It holds because the sort key of generation 0
// ends in a tag, the part of the suffix 3 symbols further on (the reference's forward tag, include/bit-layout.hpp:92-106):
// two suffixes that tie on (3 symbols, tag) have their successors in one part, and by induction so have suffixes that
// tie on (rank, second rank) later. The tag of a suffix that ends within 3 symbols is 0, 1 or 2 by its length, below every
// part's tag, so short suffixes are alone in their group from the start and a tied suffix always has h symbols left.
//
// Where the reference pushes (target, rank) messages into the host inboxes of other partitions and joins them by search,
// a part here writes its new ranks as (position, rank) messages into an outbox on the device, and the exchange applies
// them to R after the generation's last part: every read of a generation sees the ranks of the generation before.
#include "common.cuh"
#include "part.cuh"

#include "sort.cuh"

#include <atomic>
#include <cerrno>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <thread>
#include <vector>

#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

struct csa_store
{
    int device = 0;
    const u16* text = nullptr;      // borrowed: n symbols + CSA_TEXT_PAD zeros
    u64 n = 0;
    u32* rank = nullptr;            // R: n words, owned
    const u16* pid = nullptr;       // borrowed: partition id of every position (generation 0 only)
    u16* part_of_pid = nullptr;     // owned: p entries
    u32 p = 0;
    u32 parts = 0;                  // 1 + the largest entry of part_of_pid
    u64 position_offset = 0;        // test hook: lanes carry position + offset
    // the outbox of one generation: positions (low 32 bits and high 8 bits apart, so that every store is aligned) and ranks
    u32* box_lo = nullptr;
    u8* box_hi = nullptr;
    u32* box_ranks = nullptr;
    u64 box_capacity = 0;
    std::atomic<u64> box_count{0};
    bool owns_rank = true, owns_box = true;     // false where the caller lent the memory
};

namespace
{

u64 g_position_offset = 0;          // test hook (csa_debug_set key 4): what new stores add to every position in a lane

constexpr int SR_BLOCK = 256, SR_ITEMS = 8, SR_TILE = SR_BLOCK * SR_ITEMS;

__device__ __forceinline__ void lane_store(u8* lanes, u64 i, u64 v)
{
    u8* d = lanes + 5 * i;
    d[0] = u8(v); d[1] = u8(v >> 8); d[2] = u8(v >> 16); d[3] = u8(v >> 24); d[4] = u8(v >> 32);
}

__global__ void unpack_lanes_kernel(const u8* __restrict__ lanes, const u64 count, const u64 offset, u64* __restrict__ pos)
{
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if(i < count) pos[i] = sa40_load(lanes, i) - offset;
}

// Generation 0: key = 3 symbols, most significant first, then the 16-bit tag of the suffix 3 symbols on.
__global__ void stream_keys0_kernel(const u16* __restrict__ T, const u64 n, const u16* __restrict__ pid, const u16* __restrict__ part_of_pid,
                                    const u64* __restrict__ pos, const u64 count, u64* __restrict__ keys, u32* __restrict__ idx, u64* __restrict__ dev_status)
{
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if(i >= count) return;
    const u64 x = pos[i];
    if(x >= n) { atomicOr(dev_status, (u64)CSA_ST_RANGE); keys[i] = 0; idx[i] = u32(i); return; }
    const u64 next = x + 3;
    const u64 tag = next < n ? u64(part_of_pid[pid[next]]) + 3 : (n + 2 - next);
    keys[i] = (u64(T[x]) << 48) | (u64(T[x + 1]) << 32) | (u64(T[x + 2]) << 16) | tag;
    idx[i] = u32(i);
}

// Generation t: key = (rank, rank of the suffix h symbols on), both local to their parts.
__global__ void stream_keys_kernel(const u32* __restrict__ R, const u64 n, const u64 h, const u64* __restrict__ pos, const u32* __restrict__ ranks,
                                   const u64 count, u64* __restrict__ keys, u32* __restrict__ idx, u64* __restrict__ dev_status)
{
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if(i >= count) return;
    const u64 x = pos[i] + h;
    u32 sec = 0;
    if(x < n) sec = R[x];
    else atomicOr(dev_status, (u64)CSA_ST_UNSERVED);       // a tied suffix has h symbols left: see the head of this file
    keys[i] = (u64(ranks[i]) << 32) | sec;
    idx[i] = u32(i);
}

// Generation 0 from keys that the caller made, and generation t from second ranks that the caller fetched (a rank store
// sharded over several GPUs answers them): the list's own order.
__global__ void given_keys0_kernel(const u64* __restrict__ given, const u64 count, u64* __restrict__ keys, u32* __restrict__ idx)
{
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if(i >= count) return;
    keys[i] = given[i];
    idx[i] = u32(i);
}

__global__ void given_second_kernel(const u32* __restrict__ second, const u32* __restrict__ ranks, const u64 count, u64* __restrict__ keys, u32* __restrict__ idx)
{
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if(i >= count) return;
    keys[i] = (u64(ranks[i]) << 32) | second[i];
    idx[i] = u32(i);
}

__global__ void lane_positions_kernel(const u8* __restrict__ lanes, const u64 count, const u64 offset, const u64 add, u64* __restrict__ out)
{
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if(i < count) out[i] = sa40_load(lanes, i) - offset + add;
}

__device__ __forceinline__ u32 sr_warp_max(u32 v)
{
    #pragma unroll
    for(int o = 1; o < 32; o <<= 1) { const u32 t = __shfl_up_sync(0xFFFFFFFFu, v, o); if(int(lane_id()) >= o) v = max(v, t); }
    return v;
}
__device__ __forceinline__ u32 sr_warp_sum(u32 v)
{
    #pragma unroll
    for(int o = 1; o < 32; o <<= 1) { const u32 t = __shfl_up_sync(0xFFFFFFFFu, v, o); if(int(lane_id()) >= o) v += t; }
    return v;
}

struct Sr_Flags { u32 prim_head, full_head, active; };

// Flags of a thread's SR_ITEMS consecutive records of the sorted list. prim_shift = 64: the whole list is one group.
__device__ __forceinline__ Sr_Flags sr_flags(const u64* __restrict__ keys, const u64 count, const u64 first, const int prim_shift, u64 (&k)[SR_ITEMS])
{
    Sr_Flags f{0, 0, 0};
    if(first >= count) return f;
    const u64 prev = first > 0 ? keys[first - 1] : 0;
    #pragma unroll
    for(int i = 0; i < SR_ITEMS; ++i) k[i] = (first + i < count) ? keys[first + i] : 0;
    const u64 after = (first + SR_ITEMS < count) ? keys[first + SR_ITEMS] : 0;
    #pragma unroll
    for(int i = 0; i < SR_ITEMS; ++i)
    {
        if(first + i >= count) break;
        const u64 p = i == 0 ? prev : k[i - 1];
        const bool is_first = first + i == 0;
        const bool fh = is_first || k[i] != p;
        const bool ph = is_first || (prim_shift < 64 && (k[i] >> prim_shift) != (p >> prim_shift));
        const bool has_next = first + i + 1 < count;
        const u64 nx = i + 1 < SR_ITEMS ? k[i + 1] : after;
        const bool next_head = !has_next || nx != k[i];
        if(fh) f.full_head |= 1u << i;
        if(ph) f.prim_head |= 1u << i;
        if(!(fh && next_head)) f.active |= 1u << i;
    }
    return f;
}

// Step 1: per tile, the last heads (as index + 1, 0 = none) and the number of tied records.
__global__ void __launch_bounds__(SR_BLOCK) stream_rank_tile_kernel(const u64* __restrict__ keys, const u64 count, const int prim_shift, u32* __restrict__ agg)
{
    __shared__ u32 s_p[SR_BLOCK / 32], s_f[SR_BLOCK / 32], s_a[SR_BLOCK / 32];
    const u64 first = u64(blockIdx.x) * SR_TILE + u64(threadIdx.x) * SR_ITEMS;
    u64 k[SR_ITEMS];
    const Sr_Flags f = sr_flags(keys, count, first, prim_shift, k);
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
    if(lane_id() == 0) { s_p[threadIdx.x >> 5] = lp; s_f[threadIdx.x >> 5] = lf; s_a[threadIdx.x >> 5] = ac; }
    __syncthreads();
    if(threadIdx.x == 0)
    {
        u32 a = 0, b = 0, c = 0;
        for(int w = 0; w < SR_BLOCK / 32; ++w) { a = max(a, s_p[w]); b = max(b, s_f[w]); c += s_a[w]; }
        agg[3 * u64(blockIdx.x)] = a; agg[3 * u64(blockIdx.x) + 1] = b; agg[3 * u64(blockIdx.x) + 2] = c;
    }
}

// Step 2: one block makes the tiles' carries: exclusive running maxima of the heads, exclusive running sum of the tied counts,
// and the total of the tied records.
__global__ void __launch_bounds__(1024) stream_rank_carry_kernel(u32* __restrict__ agg, const u64 tiles, u64* __restrict__ total_active)
{
    __shared__ u32 s_a[32], s_b[32], s_c[32];
    __shared__ u32 carry_a, carry_b, carry_c;
    if(threadIdx.x == 0) { carry_a = 0; carry_b = 0; carry_c = 0; }
    __syncthreads();
    for(u64 base = 0; base < tiles; base += 1024)
    {
        const u64 t = base + threadIdx.x;
        u32 a = 0, b = 0, c = 0;
        if(t < tiles) { a = agg[3 * t]; b = agg[3 * t + 1]; c = agg[3 * t + 2]; }
        const u32 ia = sr_warp_max(a), ib = sr_warp_max(b), ic = sr_warp_sum(c);
        if(lane_id() == 31) { s_a[threadIdx.x >> 5] = ia; s_b[threadIdx.x >> 5] = ib; s_c[threadIdx.x >> 5] = ic; }
        __syncthreads();
        u32 pa = carry_a, pb = carry_b, pc = carry_c;
        for(u32 w = 0; w < (threadIdx.x >> 5); ++w) { pa = max(pa, s_a[w]); pb = max(pb, s_b[w]); pc += s_c[w]; }
        const u32 ua = __shfl_up_sync(0xFFFFFFFFu, ia, 1), ub = __shfl_up_sync(0xFFFFFFFFu, ib, 1);
        const u32 ea = lane_id() > 0 ? max(pa, ua) : pa, eb = lane_id() > 0 ? max(pb, ub) : pb;
        const u32 ec = pc + (ic - c);
        __syncthreads();
        if(threadIdx.x == 1023) { carry_a = max(pa, ia); carry_b = max(pb, ib); carry_c = pc + ic; }
        if(t < tiles) { agg[3 * t] = ea; agg[3 * t + 1] = eb; agg[3 * t + 2] = ec; }
        __syncthreads();
    }
    if(threadIdx.x == 0) *total_active = carry_c;
}

// Step 3: every record gets its new rank and its place in the part's reordered list (tied records first, in rank order, then
// the records that retire now); its (position, rank) goes straight into R (generation 0, when nothing reads R yet) or into the
// outbox (later generations).
__global__ void __launch_bounds__(SR_BLOCK) stream_rank_apply_kernel(const u64* __restrict__ keys, const u32* __restrict__ idx, const u64* __restrict__ pos,
                                                                    const u64 count, const int prim_shift, const u64 offset, const u32* __restrict__ agg,
                                                                    const u64* __restrict__ total_active, u64* __restrict__ out_pos, u32* __restrict__ out_ranks,
                                                                    u32* __restrict__ R, u32* __restrict__ box_lo, u8* __restrict__ box_hi, u32* __restrict__ box_ranks,
                                                                    const u64 box_first)
{
    __shared__ u32 s_p[SR_BLOCK / 32], s_f[SR_BLOCK / 32], s_a[SR_BLOCK / 32];
    const u64 first = u64(blockIdx.x) * SR_TILE + u64(threadIdx.x) * SR_ITEMS;
    const u32 carry_p = agg[3 * u64(blockIdx.x)], carry_f = agg[3 * u64(blockIdx.x) + 1], tile_act = agg[3 * u64(blockIdx.x) + 2];
    const u64 total = *total_active;
    u64 k[SR_ITEMS];
    const Sr_Flags f = sr_flags(keys, count, first, prim_shift, k);
    const u32 lp = f.prim_head ? u32(first) + (31 - __clz(f.prim_head)) + 1 : 0;
    const u32 lf = f.full_head ? u32(first) + (31 - __clz(f.full_head)) + 1 : 0;
    const u32 ac = __popc(f.active);
    const u32 ip = sr_warp_max(lp), ifl = sr_warp_max(lf), ia = sr_warp_sum(ac);
    if(lane_id() == 31) { s_p[threadIdx.x >> 5] = ip; s_f[threadIdx.x >> 5] = ifl; s_a[threadIdx.x >> 5] = ia; }
    __syncthreads();
    u32 run_p = carry_p, run_f = carry_f, act_before = tile_act;
    for(u32 w = 0; w < (threadIdx.x >> 5); ++w) { run_p = max(run_p, s_p[w]); run_f = max(run_f, s_f[w]); act_before += s_a[w]; }
    {
        const u32 up = __shfl_up_sync(0xFFFFFFFFu, ip, 1), uf = __shfl_up_sync(0xFFFFFFFFu, ifl, 1);
        if(lane_id() > 0) { run_p = max(run_p, up); run_f = max(run_f, uf); }
        act_before += ia - ac;
    }
    if(first >= count) return;
    #pragma unroll
    for(int i = 0; i < SR_ITEMS; ++i)
    {
        const u64 j = first + i;
        if(j >= count) break;
        if(f.prim_head & (1u << i)) run_p = u32(j) + 1;
        if(f.full_head & (1u << i)) run_f = u32(j) + 1;
        const u32 old_rank = prim_shift < 64 ? u32(k[i] >> prim_shift) : 0;
        const u32 new_rank = old_rank + ((run_f - 1) - (run_p - 1));
        const bool tied = (f.active >> i) & 1u;
        const u64 slot = tied ? u64(act_before) : total + (j - act_before);
        if(tied) ++act_before;
        const u64 x = pos[idx[j]];
        out_pos[slot] = x + offset;
        out_ranks[slot] = new_rank;
        if(box_lo) { box_lo[box_first + j] = u32(x); box_hi[box_first + j] = u8(x >> 32); box_ranks[box_first + j] = new_rank; }
        else R[x] = new_rank;
    }
}

__global__ void apply_messages_kernel(const u32* __restrict__ box_lo, const u8* __restrict__ box_hi, const u32* __restrict__ box_ranks, const u64 count, const u64 n,
                                      u32* __restrict__ R, u64* __restrict__ dev_status)
{
    const u64 stride = u64(gridDim.x) * blockDim.x;
    for(u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride)
    {
        const u64 x = (u64(box_hi[i]) << 32) | box_lo[i];
        if(x < n) R[x] = box_ranks[i];
        else atomicOr(dev_status, (u64)CSA_ST_RANGE);
    }
}

__global__ void rank_order_kernel(const u8* __restrict__ lanes, const u32* __restrict__ ranks, const u64 count, u8* __restrict__ out, u64* __restrict__ dev_status)
{
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if(i >= count) return;
    const u64 r = ranks[i];
    if(r >= count) { atomicOr(dev_status, (u64)CSA_ST_RANGE); return; }
    lane_store(out, r, sa40_load(lanes, i));
}

// 5-byte lanes from 64-bit positions: a thread packs 16 entries = 80 bytes = five 16-byte stores (out is 16-byte aligned).
__global__ void pack_lanes_kernel(const u64* __restrict__ pos, const u64 count, u8* __restrict__ out)
{
    const u64 first = (u64(blockIdx.x) * blockDim.x + threadIdx.x) * 16;
    if(first >= count) return;
    if(first + 16 <= count)
    {
        u32 w[20];
        #pragma unroll
        for(int j = 0; j < 20; ++j) w[j] = 0;
        #pragma unroll
        for(int e = 0; e < 16; ++e)
        {
            const u64 v = pos[first + e] & 0xFFFFFFFFFFull;
            const int b = 5 * e, wi = b >> 2, sh = (b & 3) * 8;        // 40 bits from bit sh of word wi on
            w[wi] |= u32(v << sh);
            w[wi + 1] |= u32(v >> (32 - sh));
        }
        uint4* dst = reinterpret_cast<uint4*>(out + first * 5);
        #pragma unroll
        for(int i = 0; i < 5; ++i) dst[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
    }
    else
        for(u64 r = first; r < count; ++r) lane_store(out, r, pos[r]);
}

// Histogram of the parts over a stretch of partition ids, and the scatter of the stretch's positions into per-part runs of a
// staging buffer (5-byte lanes). part_first: where each part's run starts in the staging buffer; cursor: running fill.
__global__ void count_parts_kernel(const u16* __restrict__ pid, const u64 count, const u16* __restrict__ part_of_pid, const u32 parts, u64* __restrict__ hist)
{
    extern __shared__ u32 s_cnt[];
    for(u32 i = threadIdx.x; i < parts; i += blockDim.x) s_cnt[i] = 0;
    __syncthreads();
    const u64 stride = u64(gridDim.x) * blockDim.x;
    for(u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) atomicAdd(&s_cnt[part_of_pid[pid[i]]], 1u);
    __syncthreads();
    for(u32 i = threadIdx.x; i < parts; i += blockDim.x) if(s_cnt[i]) atomicAdd(reinterpret_cast<unsigned long long*>(hist + i), (unsigned long long)s_cnt[i]);
}

// A block takes 256 * SP_ITEMS consecutive positions, a thread SP_ITEMS of them (one 16-byte load of partition ids where the
// window is aligned), so that the chain of dependent loads (id -> part -> is the part wanted) is paid once per 8 positions. The
// block counts its positions per part in shared memory (a warp's lanes with one part share one atomic), takes its places in the
// parts' runs with ONE global atomic per part that it holds, and then writes: the global cursors see a few dozen atomics per
// block instead of one per warp and part.
// KEYS: also write the generation-0 key beside every lane (3 symbols, then the tag of the suffix 3 symbols on), for a text
// that is sharded by position: T[i] is the symbol at position first + i and pid[i] its partition; both are readable 3 entries
// past `count` wherever those positions exist (the neighbour's first entries), and T is zero past the text's end.
constexpr int SP_ITEMS = 8;

template <bool KEYS>
__global__ void __launch_bounds__(256) scatter_parts_kernel(const u16* __restrict__ T, const u16* __restrict__ pid, const u64 first, const u64 count, const u64 n,
                                                            const u64 offset, const u16* __restrict__ part_of_pid, const u32 parts,
                                                            const u64* __restrict__ part_first, u64* __restrict__ cursor, u8* __restrict__ lanes,
                                                            u64* __restrict__ keys)
{
    extern __shared__ __align__(8) unsigned char sp_smem[];
    u64* const s_base = reinterpret_cast<u64*>(sp_smem);                   // [parts] where the block's records of a part start in the part's run
    u32* const s_cnt = reinterpret_cast<u32*>(sp_smem + size_t(parts) * 8); // [parts]
    for(u32 t = threadIdx.x; t < parts; t += blockDim.x) s_cnt[t] = 0;
    __syncthreads();
    const u64 i0 = (u64(blockIdx.x) * blockDim.x + threadIdx.x) * SP_ITEMS;
    u16 id[SP_ITEMS];
    if(i0 + SP_ITEMS <= count && (reinterpret_cast<uintptr_t>(pid + i0) & 15) == 0)
    {
        const uint4 v = *reinterpret_cast<const uint4*>(pid + i0);
        id[0] = u16(v.x); id[1] = u16(v.x >> 16); id[2] = u16(v.y); id[3] = u16(v.y >> 16);
        id[4] = u16(v.z); id[5] = u16(v.z >> 16); id[6] = u16(v.w); id[7] = u16(v.w >> 16);
    }
    else
    {
        #pragma unroll
        for(int j = 0; j < SP_ITEMS; ++j) id[j] = i0 + j < count ? pid[i0 + j] : u16(0);
    }
    u32 part[SP_ITEMS];
    #pragma unroll
    for(int j = 0; j < SP_ITEMS; ++j) part[j] = i0 + j < count ? u32(part_of_pid[id[j]]) : 0xFFFFFFFFu;
    u64 run_first[SP_ITEMS];
    #pragma unroll
    for(int j = 0; j < SP_ITEMS; ++j) run_first[j] = (part[j] != 0xFFFFFFFFu && part[j] < parts) ? part_first[part[j]] : ~0ull;     // ~0: not wanted now
    u32 place[SP_ITEMS];
    #pragma unroll
    for(int j = 0; j < SP_ITEMS; ++j)
    {
        const bool live = run_first[j] != ~0ull;
        place[j] = 0;
        if(__ballot_sync(0xFFFFFFFFu, live) == 0) continue;
        const u32 key_part = live ? part[j] : 0xFFFFFFFFu;
        const u32 peers = __match_any_sync(0xFFFFFFFFu, key_part);
        u32 base = 0;
        if(live && (peers & lanemask_lt()) == 0) base = atomicAdd(&s_cnt[key_part], u32(__popc(peers)));
        base = __shfl_sync(0xFFFFFFFFu, base, __ffs(peers) - 1);
        place[j] = base + __popc(peers & lanemask_lt());
    }
    __syncthreads();
    for(u32 t = threadIdx.x; t < parts; t += blockDim.x)
        if(s_cnt[t]) s_base[t] = atomicAdd(reinterpret_cast<unsigned long long*>(cursor + t), (unsigned long long)s_cnt[t]);
    __syncthreads();
    #pragma unroll
    for(int j = 0; j < SP_ITEMS; ++j)
    {
        if(run_first[j] == ~0ull) continue;
        const u64 slot = run_first[j] + s_base[part[j]] + place[j];
        const u64 i = i0 + j, x = first + i;
        lane_store(lanes, slot, x + offset);
        if(KEYS)
        {
            const u64 next = x + 3;
            const u64 tag = next < n ? u64(part_of_pid[pid[i + 3]]) + 3 : (n + 2 - next);
            keys[slot] = (u64(T[i]) << 48) | (u64(T[i + 1]) << 32) | (u64(T[i + 2]) << 16) | tag;
        }
    }
}

size_t part_workspace_bytes(u64 count)
{
    const u64 c = count ? count : 1;
    return align_up256(5 * c + 64) * 2 + align_up256(4 * c + 64) * 4 + align_up256(8 * c + 64) * 4 + align_up256(csa_sort_workspace_bytes(c))
         + align_up256(div_up(c, SR_TILE) * 12 + 256) + 4096;
}

bool is_host_pointer(const void* p)
{
    cudaPointerAttributes attr;
    const bool ok = cudaPointerGetAttributes(&attr, p) == cudaSuccess;
    cudaGetLastError();
    return !ok || attr.type == cudaMemoryTypeHost || attr.type == cudaMemoryTypeUnregistered;
}

// The common body of csa_rank_gen0 (h = 0) and csa_rank_gen.
// given_keys: generation 0 with the caller's keys (device memory, in the order of in->lanes); given_second: generation t
// with the caller's second ranks. With either, the store's text, partition ids and rank array are not read, and every new
// rank leaves as a message.
int rank_part(csa_ctx* ctx, csa_store* st, const csa_part* in, u64 h, csa_part_result* out, const u64* given_keys = nullptr, const u32* given_second = nullptr)
{
    if(!ctx || !st || !in || !out) return csa_fail(ctx, CSA_E_INVALID, "part job: null argument");
    out->active = 0; out->messages = 0;
    const u64 S = in->count;
    if(S == 0) return CSA_OK;
    if(S >= (u64(1) << 31)) return csa_fail(ctx, CSA_E_LIMIT, "part job: a part holds fewer than 2^31 suffixes");
    if(!in->lanes || !out->lanes || !out->ranks || (h > 0 && !in->ranks)) return csa_fail(ctx, CSA_E_INVALID, "part job: null buffer");
    if(h == 0 && !given_keys && !st->pid) return csa_fail(ctx, CSA_E_INVALID, "part job: generation 0 needs the store's partition ids");
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    const size_t need = part_workspace_bytes(S);
    void* ws = nullptr;
    CSA_TRY(csa_arena(ctx, need, &ws));
    Carver cv(ws, ctx->arena_bytes);
    u8* lanes_in = cv.take<u8>(5 * S + 64);
    u8* lanes_out = cv.take<u8>(5 * S + 64);
    u32* ranks_in = cv.take<u32>(S + 16);
    u32* ranks_out = cv.take<u32>(S + 16);
    u32* idxA = cv.take<u32>(S + 16);
    u32* idxB = cv.take<u32>(S + 16);
    u64* pos = cv.take<u64>(S + 8);
    u64* keysA = cv.take<u64>(S + 8);
    u64* keysB = cv.take<u64>(S + 8);
    u64* pos_out = cv.take<u64>(S + 8);
    const size_t sort_ws_bytes = csa_sort_workspace_bytes(S);
    void* sort_ws = cv.take<u8>(sort_ws_bytes);
    u32* agg = cv.take<u32>(div_up(S, SR_TILE) * 3 + 64);
    if(!cv.ok) return csa_fail(ctx, CSA_E_NOMEM, "part job: workspace too small");

    // in: lanes (and ranks) from wherever the caller keeps them
    CSA_CUDA(ctx, cudaMemcpyAsync(lanes_in, in->lanes, 5 * S, cudaMemcpyDefault, ctx->stream));
    CSA_CUDA(ctx, cudaMemsetAsync(lanes_in + 5 * S, 0, 8, ctx->stream));
    if(h > 0) CSA_CUDA(ctx, cudaMemcpyAsync(ranks_in, in->ranks, 4 * S, cudaMemcpyDefault, ctx->stream));
    const unsigned blocks = unsigned(div_up(S, 256));
    unpack_lanes_kernel<<<blocks, 256, 0, ctx->stream>>>(lanes_in, S, st->position_offset, pos);
    CSA_LAUNCH_CHECK(ctx);
    int bits = 64, prim_shift = 64;
    if(given_keys)
        given_keys0_kernel<<<blocks, 256, 0, ctx->stream>>>(given_keys, S, keysA, idxA);
    else if(h == 0)
        stream_keys0_kernel<<<blocks, 256, 0, ctx->stream>>>(st->text, st->n, st->pid, st->part_of_pid, pos, S, keysA, idxA, ctx->d_status);
    else
    {
        if(given_second) given_second_kernel<<<blocks, 256, 0, ctx->stream>>>(given_second, ranks_in, S, keysA, idxA);
        else stream_keys_kernel<<<blocks, 256, 0, ctx->stream>>>(st->rank, st->n, h, pos, ranks_in, S, keysA, idxA, ctx->d_status);
        bits = 64; prim_shift = 32;
    }
    CSA_LAUNCH_CHECK(ctx);
    int in_alt = 0;
    {
        const Ties_In_Any_Order free_ties(ctx);       // ties are what the next generation sorts
        CSA_TRY(csa_sort_pairs(ctx, reinterpret_cast<uint64_t*>(keysA), reinterpret_cast<uint64_t*>(keysB), idxA, idxB, 4, S, 0, bits, sort_ws, sort_ws_bytes, &in_alt));
    }
    const u64* ks = in_alt ? keysB : keysA;
    const u32* is = in_alt ? idxB : idxA;

    // messages: generation 0 writes R itself (nothing reads R before generation 1); later generations fill the outbox
    u64 box_first = 0;
    const bool boxed = h > 0 || given_keys != nullptr;
    if(boxed)
    {
        box_first = st->box_count.fetch_add(S);
        if(box_first + S > st->box_capacity) return csa_fail(ctx, CSA_E_NOMEM, "part job: the store's outbox is full (csa_store_reserve_messages)");
    }
    const u64 tiles = div_up(S, SR_TILE);
    u64* total_d = ctx->d_scalars + 12;
    stream_rank_tile_kernel<<<unsigned(tiles), SR_BLOCK, 0, ctx->stream>>>(ks, S, prim_shift, agg);
    CSA_LAUNCH_CHECK(ctx);
    stream_rank_carry_kernel<<<1, 1024, 0, ctx->stream>>>(agg, tiles, total_d);
    CSA_LAUNCH_CHECK(ctx);
    stream_rank_apply_kernel<<<unsigned(tiles), SR_BLOCK, 0, ctx->stream>>>(ks, is, pos, S, prim_shift, st->position_offset, agg, total_d, pos_out, ranks_out, st->rank,
                                                                          boxed ? st->box_lo : nullptr, boxed ? st->box_hi : nullptr, boxed ? st->box_ranks : nullptr, box_first);
    CSA_LAUNCH_CHECK(ctx);
    pack_lanes_kernel<<<unsigned(div_up(div_up(S, 16), 256)), 256, 0, ctx->stream>>>(pos_out, S, lanes_out);
    CSA_LAUNCH_CHECK(ctx);
    CSA_CUDA(ctx, cudaMemcpyAsync(ctx->h_scalars + 12, total_d, 8, cudaMemcpyDeviceToHost, ctx->stream));
    CSA_CUDA(ctx, cudaMemcpyAsync(ctx->h_scalars + 13, ctx->d_status, 8, cudaMemcpyDeviceToHost, ctx->stream));
    CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if(ctx->h_scalars[13] != 0) { u64 b = 0; return csa_sync(ctx, reinterpret_cast<uint64_t*>(&b)); }
    out->active = ctx->h_scalars[12];
    out->messages = boxed ? S : 0;
    // out: queued behind the job; complete after csa_sync
    CSA_CUDA(ctx, cudaMemcpyAsync(out->lanes, lanes_out, 5 * S, cudaMemcpyDefault, ctx->stream));
    CSA_CUDA(ctx, cudaMemcpyAsync(out->ranks, ranks_out, 4 * S, cudaMemcpyDefault, ctx->stream));
    return CSA_OK;
}

}   // namespace

void stream_set_position_offset(u64 offset) { g_position_offset = offset; }

extern "C" size_t csa_part_workspace_bytes(uint64_t count) { return part_workspace_bytes(count); }

extern "C" int csa_store_create(csa_ctx* ctx, const uint16_t* text_dev, uint64_t n, const uint16_t* pid_dev, const uint16_t* part_of_pid_host, uint32_t p,
                                uint32_t* rank_store_dev, csa_store** out)
{
    if(!ctx || !text_dev || !out || n == 0 || p == 0 || p > CSA_MAX_PARTITIONS || !part_of_pid_host) return csa_fail(ctx, CSA_E_INVALID, "csa_store_create: bad argument");
    if(n + g_position_offset >= (u64(1) << 40)) return csa_fail(ctx, CSA_E_LIMIT, "csa_store_create: positions must fit 40 bits");
    *out = nullptr;
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    csa_store* st = new(std::nothrow) csa_store();
    if(!st) return CSA_E_NOMEM;
    st->device = ctx->device; st->text = text_dev; st->n = n; st->pid = pid_dev; st->p = p; st->position_offset = g_position_offset;
    if(rank_store_dev) { st->rank = rank_store_dev; st->owns_rank = false; }
    if((!rank_store_dev && cudaMalloc(&st->rank, n * 4 + 64) != cudaSuccess) || cudaMalloc(&st->part_of_pid, size_t(p) * 2 + 64) != cudaSuccess)
    {
        cudaGetLastError();
        if(st->rank && st->owns_rank) cudaFree(st->rank);
        delete st;
        return csa_fail(ctx, CSA_E_NOMEM, "csa_store_create: no device memory for the rank store");
    }
    for(u32 q = 0; q < p; ++q) if(u32(part_of_pid_host[q]) + 1 > st->parts) st->parts = u32(part_of_pid_host[q]) + 1;
    CSA_CUDA(ctx, cudaMemcpyAsync(st->part_of_pid, part_of_pid_host, size_t(p) * 2, cudaMemcpyHostToDevice, ctx->stream));
    CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    *out = st;
    return CSA_OK;
}

extern "C" void csa_store_destroy(csa_store* st)
{
    if(!st) return;
    cudaSetDevice(st->device);
    if(st->rank && st->owns_rank) cudaFree(st->rank);
    if(st->part_of_pid) cudaFree(st->part_of_pid);
    if(st->owns_box) { if(st->box_lo) cudaFree(st->box_lo); if(st->box_hi) cudaFree(st->box_hi); if(st->box_ranks) cudaFree(st->box_ranks); }
    delete st;
}

extern "C" void csa_store_drop_partition_ids(csa_store* st) { if(st) st->pid = nullptr; }

extern "C" int csa_store_reserve_messages(csa_ctx* ctx, csa_store* st, uint64_t messages)
{
    if(!ctx || !st) return csa_fail(ctx, CSA_E_INVALID, "csa_store_reserve_messages: null argument");
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    st->box_count.store(0);
    if(!st->owns_box && messages > st->box_capacity) return csa_fail(ctx, CSA_E_NOMEM, "csa_store_reserve_messages: the outbox lent by the caller is too small");
    if(messages > st->box_capacity)
    {
        CSA_CUDA(ctx, cudaDeviceSynchronize());
        if(st->box_lo) cudaFree(st->box_lo);
        if(st->box_hi) cudaFree(st->box_hi);
        if(st->box_ranks) cudaFree(st->box_ranks);
        st->box_lo = nullptr; st->box_hi = nullptr; st->box_ranks = nullptr; st->box_capacity = 0;
        if(cudaMalloc(&st->box_lo, messages * 4 + 64) != cudaSuccess || cudaMalloc(&st->box_hi, messages + 64) != cudaSuccess ||
           cudaMalloc(&st->box_ranks, messages * 4 + 64) != cudaSuccess)
        {
            cudaGetLastError();
            if(st->box_lo) { cudaFree(st->box_lo); st->box_lo = nullptr; }
            if(st->box_hi) { cudaFree(st->box_hi); st->box_hi = nullptr; }
            return csa_fail(ctx, CSA_E_NOMEM, "csa_store_reserve_messages: no device memory for the outbox");
        }
        st->box_capacity = messages;
    }
    return CSA_OK;
}

extern "C" int csa_store_use_outbox(csa_store* st, uint32_t* pos_lo_dev, uint8_t* pos_hi_dev, uint32_t* ranks_dev, uint64_t capacity)
{
    const int given = (pos_lo_dev != nullptr) + (pos_hi_dev != nullptr) + (ranks_dev != nullptr);
    if(!st || (given != 0 && given != 3)) return CSA_E_INVALID;
    cudaSetDevice(st->device);
    if(st->owns_box)
    {
        cudaDeviceSynchronize();
        if(st->box_lo) cudaFree(st->box_lo);
        if(st->box_hi) cudaFree(st->box_hi);
        if(st->box_ranks) cudaFree(st->box_ranks);
    }
    st->box_lo = pos_lo_dev; st->box_hi = pos_hi_dev; st->box_ranks = ranks_dev;
    st->box_capacity = given ? capacity : 0;
    st->owns_box = given == 0;
    st->box_count.store(0);
    return CSA_OK;
}

extern "C" uint64_t csa_store_outbox_count(const csa_store* st) { return st ? st->box_count.load() : 0; }

extern "C" int csa_store_apply_messages(csa_ctx* ctx, csa_store* st, const uint32_t* pos_lo_dev, const uint8_t* pos_hi_dev, const uint32_t* ranks_dev, uint64_t count)
{
    if(!ctx || !st || (count && (!pos_lo_dev || !pos_hi_dev || !ranks_dev))) return csa_fail(ctx, CSA_E_INVALID, "csa_store_apply_messages: null argument");
    if(count == 0) return CSA_OK;
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    const unsigned blocks = unsigned(div_up(count, 256) < 148 * 16 ? div_up(count, 256) : 148 * 16);
    apply_messages_kernel<<<blocks, 256, 0, ctx->stream>>>(pos_lo_dev, pos_hi_dev, ranks_dev, count, st->n, st->rank, ctx->d_status);
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

extern "C" int csa_part_sizes(csa_ctx* ctx, csa_store* st, uint64_t first, uint64_t count, uint32_t parts, uint64_t* hist_dev)
{
    if(!ctx || !st || !st->pid || !hist_dev || parts == 0 || parts > CSA_MAX_PARTITIONS || first + count > st->n) return csa_fail(ctx, CSA_E_INVALID, "csa_part_sizes: bad argument");
    if(count == 0) return CSA_OK;
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    count_parts_kernel<<<148 * 4, 256, size_t(parts) * 4, ctx->stream>>>(st->pid + first, count, st->part_of_pid, parts, reinterpret_cast<u64*>(hist_dev));
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

extern "C" int csa_scatter_lanes(csa_ctx* ctx, csa_store* st, uint64_t first, uint64_t count, const uint64_t* part_first_dev, uint64_t* cursor_dev, uint8_t* lanes_dev)
{
    if(!ctx || !st || !st->pid || !part_first_dev || !cursor_dev || !lanes_dev || first + count > st->n) return csa_fail(ctx, CSA_E_INVALID, "csa_scatter_lanes: bad argument");
    if(count == 0) return CSA_OK;
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    scatter_parts_kernel<false><<<unsigned(div_up(count, 256 * SP_ITEMS)), 256, size_t(st->parts) * 12, ctx->stream>>>(nullptr, st->pid + first, first, count, st->n, st->position_offset,
                                                                                                                      st->part_of_pid, st->parts, reinterpret_cast<const u64*>(part_first_dev),
                                                                                                                      reinterpret_cast<u64*>(cursor_dev), lanes_dev, nullptr);
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

extern "C" int csa_rank_gen0(csa_ctx* ctx, csa_store* st, const csa_part* in, csa_part_result* out) { return rank_part(ctx, st, in, 0, out); }

extern "C" int csa_rank_gen(csa_ctx* ctx, csa_store* st, const csa_part* in, uint64_t h, csa_part_result* out)
{
    if(h == 0) return csa_fail(ctx, CSA_E_INVALID, "csa_rank_gen: h must be positive");
    return rank_part(ctx, st, in, h, out);
}

extern "C" int csa_rank_gen0_keys(csa_ctx* ctx, csa_store* st, const csa_part* in, const uint64_t* keys_dev, csa_part_result* out)
{
    if(!keys_dev) return csa_fail(ctx, CSA_E_INVALID, "csa_rank_gen0_keys: null keys");
    return rank_part(ctx, st, in, 0, out, reinterpret_cast<const u64*>(keys_dev), nullptr);
}

extern "C" int csa_rank_gen_ranks(csa_ctx* ctx, csa_store* st, const csa_part* in, const uint32_t* second_ranks_dev, csa_part_result* out)
{
    if(!second_ranks_dev) return csa_fail(ctx, CSA_E_INVALID, "csa_rank_gen_ranks: null second ranks");
    return rank_part(ctx, st, in, 1, out, nullptr, second_ranks_dev);
}

extern "C" int csa_part_positions(csa_ctx* ctx, csa_store* st, const uint8_t* lanes, uint64_t count, uint64_t add, uint64_t* positions_dev)
{
    if(!ctx || !st || (count && (!lanes || !positions_dev))) return csa_fail(ctx, CSA_E_INVALID, "csa_part_positions: null argument");
    if(count == 0) return CSA_OK;
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    void* ws = nullptr;
    CSA_TRY(csa_arena(ctx, align_up256(5 * count + 64), &ws));
    u8* lanes_in = static_cast<u8*>(ws);
    CSA_CUDA(ctx, cudaMemcpyAsync(lanes_in, lanes, 5 * count, cudaMemcpyDefault, ctx->stream));
    CSA_CUDA(ctx, cudaMemsetAsync(lanes_in + 5 * count, 0, 8, ctx->stream));
    lane_positions_kernel<<<unsigned(div_up(count, 256)), 256, 0, ctx->stream>>>(lanes_in, count, st->position_offset, add, reinterpret_cast<u64*>(positions_dev));
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

extern "C" int csa_scatter_lanes_keys(csa_ctx* ctx, csa_store* st, const uint16_t* text_window_dev, const uint16_t* pid_window_dev, uint64_t first, uint64_t count,
                                      const uint64_t* part_first_dev, uint64_t* cursor_dev, uint8_t* lanes_dev, uint64_t* keys_dev)
{
    if(!ctx || !st || !text_window_dev || !pid_window_dev || !part_first_dev || !cursor_dev || !lanes_dev || !keys_dev || first + count > st->n)
        return csa_fail(ctx, CSA_E_INVALID, "csa_scatter_lanes_keys: bad argument");
    if(count == 0) return CSA_OK;
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    scatter_parts_kernel<true><<<unsigned(div_up(count, 256 * SP_ITEMS)), 256, size_t(st->parts) * 12, ctx->stream>>>(text_window_dev, pid_window_dev, first, count, st->n, st->position_offset,
                                                                                               st->part_of_pid, st->parts, reinterpret_cast<const u64*>(part_first_dev),
                                                                                               reinterpret_cast<u64*>(cursor_dev), lanes_dev, reinterpret_cast<u64*>(keys_dev));
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

extern "C" int csa_exchange_messages(csa_ctx* ctx, csa_store* st, uint64_t* applied)
{
    if(!ctx || !st) return csa_fail(ctx, CSA_E_INVALID, "csa_exchange_messages: null argument");
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    const u64 c = st->box_count.load();
    if(applied) *applied = c;
    if(c == 0) return CSA_OK;
    const unsigned blocks = unsigned(div_up(c, 256) < 148 * 16 ? div_up(c, 256) : 148 * 16);
    apply_messages_kernel<<<blocks, 256, 0, ctx->stream>>>(st->box_lo, st->box_hi, st->box_ranks, c, st->n, st->rank, ctx->d_status);
    CSA_LAUNCH_CHECK(ctx);
    st->box_count.store(0);
    u64 bits = 0;
    return csa_sync(ctx, reinterpret_cast<uint64_t*>(&bits));
}

extern "C" int csa_rank_order(csa_ctx* ctx, const uint8_t* lanes, const uint32_t* ranks, uint64_t count, uint8_t* sa40_out)
{
    if(!ctx || !lanes || !ranks || !sa40_out) return csa_fail(ctx, CSA_E_INVALID, "csa_rank_order: null argument");
    if(count == 0) return CSA_OK;
    if(count >= (u64(1) << 31)) return csa_fail(ctx, CSA_E_LIMIT, "csa_rank_order: a part holds fewer than 2^31 suffixes");
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    void* ws = nullptr;
    CSA_TRY(csa_arena(ctx, align_up256(5 * count + 64) * 2 + align_up256(4 * count + 64) + 1024, &ws));
    Carver cv(ws, ctx->arena_bytes);
    u8* lanes_in = cv.take<u8>(5 * count + 64);
    u8* lanes_out = cv.take<u8>(5 * count + 64);
    u32* ranks_in = cv.take<u32>(count + 16);
    if(!cv.ok) return csa_fail(ctx, CSA_E_NOMEM, "csa_rank_order: workspace too small");
    CSA_CUDA(ctx, cudaMemcpyAsync(lanes_in, lanes, 5 * count, cudaMemcpyDefault, ctx->stream));
    CSA_CUDA(ctx, cudaMemsetAsync(lanes_in + 5 * count, 0, 8, ctx->stream));
    CSA_CUDA(ctx, cudaMemcpyAsync(ranks_in, ranks, 4 * count, cudaMemcpyDefault, ctx->stream));
    rank_order_kernel<<<unsigned(div_up(count, 256)), 256, 0, ctx->stream>>>(lanes_in, ranks_in, count, lanes_out, ctx->d_status);
    CSA_LAUNCH_CHECK(ctx);
    CSA_CUDA(ctx, cudaMemcpyAsync(sa40_out, lanes_out, 5 * count, cudaMemcpyDefault, ctx->stream));
    return CSA_OK;
}

// ---- the host pipeline: the whole build, parts streamed through the device --------------------------------------------------

namespace
{

struct Dev_Buffer
{
    void* p = nullptr;
    ~Dev_Buffer() { if(p) cudaFree(p); }
    int alloc(csa_ctx* ctx, size_t bytes)
    {
        if(cudaMalloc(&p, bytes) != cudaSuccess) { cudaGetLastError(); p = nullptr; return csa_fail(ctx, CSA_E_NOMEM, "streamed build: device allocation of " + std::to_string(bytes) + " bytes failed"); }
        return CSA_OK;
    }
};

double ms_since(const std::chrono::steady_clock::time_point& t0)
{
    return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
}

}   // namespace

namespace
{
bool write_all(int fd, const void* from, size_t bytes, u64 at)
{
    const u8* p = static_cast<const u8*>(from);
    while(bytes > 0)
    {
        const ssize_t w = ::pwrite(fd, p, bytes < (size_t(1) << 30) ? bytes : (size_t(1) << 30), off_t(at));
        if(w <= 0) { if(w < 0 && errno == EINTR) continue; return false; }
        p += w; at += u64(w); bytes -= size_t(w);
    }
    return true;
}

bool read_all(int fd, void* to, size_t bytes, u64 at)
{
    u8* p = static_cast<u8*>(to);
    while(bytes > 0)
    {
        const ssize_t r = ::pread(fd, p, bytes < (size_t(1) << 30) ? bytes : (size_t(1) << 30), off_t(at));
        if(r <= 0) { if(r < 0 && errno == EINTR) continue; return false; }
        p += r; at += u64(r); bytes -= size_t(r);
    }
    return true;
}

// The files of the parts whose lists do not fit the host bound: per part one file of lanes and one of ranks, in a directory
// of this build's own below the scratch directory (the reference stripes such files over its scratch roots,
// include/GPU_SACA.cuh:95-118). Everything is removed when the build ends, however it ends.
struct Part_Files
{
    std::vector<std::string> dirs;
    std::vector<int> lanes_fd, ranks_fd;
    std::vector<std::string> names;
    std::atomic<u64> bytes_read{0}, bytes_written{0};

    // scratch: one directory, or several separated by colons; part u's files go to directory u modulo their number.
    bool open_parts(const char* scratch, u32 first, u32 parts)
    {
        static std::atomic<unsigned> serial{0};
        const std::string own = "/cascade_b200_" + std::to_string(long(::getpid())) + "_" + std::to_string(serial.fetch_add(1));
        const std::string all(scratch);
        for(size_t at = 0; at <= all.size();)
        {
            size_t end = all.find(':', at);
            if(end == std::string::npos) end = all.size();
            if(end > at)
            {
                const std::string dir = all.substr(at, end - at) + own;
                if(::mkdir(dir.c_str(), 0700) != 0) return false;
                dirs.push_back(dir);
            }
            at = end + 1;
        }
        if(dirs.empty()) return false;
        lanes_fd.assign(parts, -1);
        ranks_fd.assign(parts, -1);
        for(u32 u = first; u < parts; ++u)
            for(int kind = 0; kind < 2; ++kind)
            {
                names.push_back(dirs[u % dirs.size()] + "/part_" + std::to_string(u) + (kind ? ".ranks" : ".lanes"));
                const int fd = ::open(names.back().c_str(), O_RDWR | O_CREAT | O_EXCL, 0600);
                if(fd < 0) return false;
                (kind ? ranks_fd : lanes_fd)[u] = fd;
            }
        return true;
    }
    bool read(int fd, void* to, size_t bytes, u64 at) { bytes_read += bytes; return read_all(fd, to, bytes, at); }
    bool write(int fd, const void* from, size_t bytes, u64 at) { bytes_written += bytes; return write_all(fd, from, bytes, at); }
    ~Part_Files()
    {
        for(int fd : lanes_fd) if(fd >= 0) ::close(fd);
        for(int fd : ranks_fd) if(fd >= 0) ::close(fd);
        for(const std::string& f : names) ::unlink(f.c_str());
        for(const std::string& d : dirs) ::rmdir(d.c_str());
    }
};
}

extern "C" int csa_build_sa_tiered(csa_ctx* ctx, const uint16_t* text_host, uint64_t n, uint32_t p, uint64_t seed, uint8_t* sa40_host,
                                   const csa_tier_options* options, csa_build_stats* stats)
{
    if(!ctx || !text_host || !options) return csa_fail(ctx, CSA_E_INVALID, "streamed build: null argument");
    if(!sa40_host && !options->output_path) return csa_fail(ctx, CSA_E_INVALID, "streamed build: neither an output array nor an output file");
    uint64_t part_suffixes = options->part_suffixes;
    if(n == 0) return csa_fail(ctx, CSA_E_INVALID, "streamed build: empty text");
    if(p == 0 || p > CSA_MAX_PARTITIONS) return csa_fail(ctx, CSA_E_LIMIT, "streamed build: partition count out of range");
    if(n + g_position_offset >= (u64(1) << 40)) return csa_fail(ctx, CSA_E_LIMIT, "streamed build: positions must fit 40 bits");
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    csa_build_stats local_stats;
    csa_build_stats& bs = stats ? *stats : local_stats;
    std::memset(&bs, 0, sizeof(bs));
    bs.n = n;
    const u64 launches_before = ctx->counters[0], passes_before = ctx->counters[1], records_before = ctx->counters[2];
    const auto t_start = std::chrono::steady_clock::now();
    const u64 offset = g_position_offset;

    // ---- text and partition ids on the device ------------------------------------------------------------------------------
    Dev_Buffer text_b, pid_b, small_b, stage_b;
    CSA_TRY(text_b.alloc(ctx, (n + CSA_TEXT_PAD) * 2 + 256));
    CSA_TRY(pid_b.alloc(ctx, n * 2 + 256));
    u16* T = static_cast<u16*>(text_b.p);
    u16* pid = static_cast<u16*>(pid_b.p);
    CSA_CUDA(ctx, cudaMemcpyAsync(T, text_host, n * 2, cudaMemcpyHostToDevice, ctx->stream));
    CSA_CUDA(ctx, cudaMemsetAsync(T + n, 0, CSA_TEXT_PAD * 2, ctx->stream));
    constexpr u64 MAX_SAMPLES = 1u << 19;
    const size_t split_bytes = align_up256(pick_splitters_scratch_bytes(MAX_SAMPLES));
    CSA_TRY(small_b.alloc(ctx, split_bytes + align_up256(size_t(2) * p * 8) + 3 * align_up256(size_t(CSA_MAX_PARTITIONS) * 8) + align_up256(65536 * 4) + 4096));
    Carver sc(small_b.p, split_bytes + align_up256(size_t(2) * p * 8) + 3 * align_up256(size_t(CSA_MAX_PARTITIONS) * 8) + align_up256(65536 * 4) + 4096);
    void* split_scratch = sc.take<u8>(split_bytes);
    u64* pivots_dev = sc.take<u64>(2 * u64(p));
    u64* hist_dev = sc.take<u64>(CSA_MAX_PARTITIONS);
    u64* part_first_dev = sc.take<u64>(CSA_MAX_PARTITIONS);
    u64* cursor_dev = sc.take<u64>(CSA_MAX_PARTITIONS);
    u32* symbol_range = sc.take<u32>(65536);
    if(!sc.ok) return csa_fail(ctx, CSA_E_NOMEM, "streamed build: scratch too small");

    u32 p_eff = 1;
    std::vector<u64> pivots(2 * size_t(p));
    if(p > 1)
    {
        u64 n_samples = u64(32) * p * u64(bits_for(n));
        if(n_samples > MAX_SAMPLES) n_samples = MAX_SAMPLES;
        if(n_samples < 1024) n_samples = 1024;
        CSA_TRY(pick_splitters(ctx, T, n, p, seed, n_samples, split_scratch, pick_splitters_scratch_bytes(MAX_SAMPLES), pivots.data(), &p_eff));
        if(p_eff > 1) CSA_CUDA(ctx, cudaMemcpyAsync(pivots_dev, pivots.data(), size_t(2) * (p_eff - 1) * 8, cudaMemcpyHostToDevice, ctx->stream));
    }
    bs.partitions = p_eff;
    CSA_CUDA(ctx, cudaMemsetAsync(hist_dev, 0, size_t(p_eff) * 8, ctx->stream));
    if(p_eff > 1) CSA_TRY(partition_install_symbol_ranges(ctx, pivots.data(), p_eff, symbol_range));
    constexpr u64 PID_CHUNK = u64(1) << 28;
    int pid_rc = CSA_OK;
    for(u64 first = 0; first < n && pid_rc == CSA_OK; first += PID_CHUNK)
        pid_rc = csa_partition_ids(ctx, T, n, first, n - first < PID_CHUNK ? n - first : PID_CHUNK, reinterpret_cast<const uint64_t*>(pivots_dev), p_eff, pid + first,
                                   reinterpret_cast<uint64_t*>(hist_dev));
    partition_install_symbol_ranges(ctx, nullptr, 0, nullptr);
    CSA_TRY(pid_rc);
    std::vector<u64> part_size(p_eff);
    CSA_CUDA(ctx, cudaMemcpyAsync(part_size.data(), hist_dev, size_t(p_eff) * 8, cudaMemcpyDeviceToHost, ctx->stream));
    CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));

    // ---- parts: runs of whole partitions, each below the size asked for (and below 2^31) -----------------------------------
    if(part_suffixes == 0) part_suffixes = u64(1) << 27;
    if(part_suffixes >= (u64(1) << 31)) part_suffixes = (u64(1) << 31) - 1;
    std::vector<u16> part_of_pid(p_eff);
    std::vector<u64> part_off(1, 0);
    {
        u64 cur = 0, total = 0;
        for(u32 q = 0; q < p_eff; ++q)
        {
            if(part_size[q] >= (u64(1) << 31)) return csa_fail(ctx, CSA_E_LIMIT, "streamed build: a partition holds 2^31 suffixes or more; ask for more partitions");
            if(cur > 0 && cur + part_size[q] > part_suffixes) { part_off.push_back(total); cur = 0; }
            part_of_pid[q] = u16(part_off.size() - 1);
            cur += part_size[q];
            total += part_size[q];
            if(part_size[q] > bs.max_partition) bs.max_partition = part_size[q];
        }
        part_off.push_back(total);
        if(total != n) return csa_fail(ctx, CSA_E_DEVICE, "streamed build: partition sizes do not add up to n");
    }
    const u32 parts = u32(part_off.size() - 1);
    u64 largest_part = 0;
    for(u32 u = 0; u < parts; ++u) if(part_off[u + 1] - part_off[u] > largest_part) largest_part = part_off[u + 1] - part_off[u];

    csa_store* st = nullptr;
    CSA_TRY(csa_store_create(ctx, T, n, pid, part_of_pid.data(), p_eff, nullptr, &st));
    struct Store_Guard { csa_store* s; ~Store_Guard() { csa_store_destroy(s); } } store_guard{st};

    // ---- tiers: the first parts keep their lists in host memory while the bound allows, the others keep them in files --------
    u32 first_file_part = parts;
    if(options->host_list_bytes != ~uint64_t(0))
        for(u32 u = 0; u < parts; ++u)
            if(9 * part_off[u + 1] > options->host_list_bytes) { first_file_part = u; break; }
    const bool files_in_use = first_file_part < parts;
    if(files_in_use && !options->scratch_dir)
        return csa_fail(ctx, CSA_E_NOMEM, "streamed build: the lists pass the host bound and no scratch directory is given");
    Part_Files files;
    if(files_in_use && !files.open_parts(options->scratch_dir, first_file_part, parts))
        return csa_fail(ctx, CSA_E_INVALID, "streamed build: cannot create the part files in the scratch directory");
    struct Fd_Guard { int fd = -1; ~Fd_Guard() { if(fd >= 0) ::close(fd); } } out_file;
    if(options->output_path)
    {
        out_file.fd = ::open(options->output_path, O_WRONLY | O_CREAT | O_TRUNC, 0644);
        if(out_file.fd < 0 || ::ftruncate(out_file.fd, off_t(5 * n)) != 0) return csa_fail(ctx, CSA_E_INVALID, "streamed build: cannot create the output file");
    }
    u64 largest_file_part = 0;
    for(u32 u = first_file_part; u < parts; ++u) if(part_off[u + 1] - part_off[u] > largest_file_part) largest_file_part = part_off[u + 1] - part_off[u];
    const u64 host_suffixes = part_off[first_file_part];
    constexpr u64 CHUNK = u64(1) << 27;
    const u64 chunk_cap = n < CHUNK ? n : CHUNK;
    // One pinned array of the context (a second build of this size pins nothing): the ranks of the host parts, their lanes when
    // there is no output array to keep them in, two buffers through which the lanes of the file parts reach their files, and
    // this thread's buffers for a file part (lanes, ranks, ordered lanes).
    const size_t bounce_bytes = files_in_use ? align_up256(5 * largest_file_part + 64) * 2 + align_up256(4 * largest_file_part + 64) : 0;
    const size_t ranks_bytes = align_up256(host_suffixes * 4 + 64);
    const size_t own_lanes_bytes = sa40_host ? 0 : align_up256(host_suffixes * 5 + 64);
    const size_t to_files_bytes = files_in_use ? 2 * align_up256(5 * chunk_cap + 256) : 0;
    void* pinned_p = nullptr;
    CSA_TRY(csa_host_aux(ctx, ranks_bytes + own_lanes_bytes + to_files_bytes + bounce_bytes + 256, &pinned_p));
    u8* const pinned = static_cast<u8*>(pinned_p);
    u32* const ranks_host = reinterpret_cast<u32*>(pinned);
    u8* const host_lanes = sa40_host ? sa40_host : pinned + ranks_bytes;
    u8* const to_files[2] = {pinned + ranks_bytes + own_lanes_bytes, pinned + ranks_bytes + own_lanes_bytes + to_files_bytes / 2};
    // Where the lists of host part u lie.
    auto lanes_of = [&](u32 u) { return host_lanes + 5 * part_off[u]; };
    auto ranks_of = [&](u32 u) { return ranks_host + part_off[u]; };
    const double ms_pinned = ms_since(t_start);
    {
        // Stretch by stretch: count the stretch's positions by part, scatter them into per-part runs of a staging buffer, and
        // copy every run to its part's place on the host. Two staging buffers and a second stream let the copies of one
        // stretch run under the scatter of the next.
        CSA_TRY(stage_b.alloc(ctx, 2 * align_up256(5 * chunk_cap + 256)));
        u8* const staging[2] = {static_cast<u8*>(stage_b.p), static_cast<u8*>(stage_b.p) + align_up256(5 * chunk_cap + 256)};
        CSA_TRY(csa_lanes(ctx));
        cudaStream_t copy_stream = ctx->lane[0];
        cudaEvent_t scattered = ctx->lane_event[0], copied[2] = {ctx->lane_event[1], ctx->lane_event[2]};
        std::vector<u64> filled(parts, 0), chunk_hist(parts), chunk_first(parts);
        u64 k = 0;
        for(u64 first = 0; first < n; first += CHUNK, ++k)
        {
            const u64 c = n - first < CHUNK ? n - first : CHUNK;
            u8* const stage = staging[k & 1];
            CSA_CUDA(ctx, cudaMemsetAsync(hist_dev, 0, size_t(parts) * 8, ctx->stream));
            count_parts_kernel<<<148 * 4, 256, size_t(parts) * 4, ctx->stream>>>(pid + first, c, st->part_of_pid, parts, hist_dev);
            CSA_LAUNCH_CHECK(ctx);
            CSA_CUDA(ctx, cudaMemcpyAsync(chunk_hist.data(), hist_dev, size_t(parts) * 8, cudaMemcpyDeviceToHost, ctx->stream));
            CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            u64 at = 0;
            for(u32 u = 0; u < parts; ++u) { chunk_first[u] = at; at += chunk_hist[u]; }
            CSA_CUDA(ctx, cudaMemcpyAsync(part_first_dev, chunk_first.data(), size_t(parts) * 8, cudaMemcpyHostToDevice, ctx->stream));
            CSA_CUDA(ctx, cudaMemsetAsync(cursor_dev, 0, size_t(parts) * 8, ctx->stream));
            if(k >= 2) CSA_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, copied[k & 1], 0));       // the copies out of this staging buffer, two stretches ago
            scatter_parts_kernel<false><<<unsigned(div_up(c, 256 * SP_ITEMS)), 256, size_t(parts) * 12, ctx->stream>>>(nullptr, pid + first, first, c, n, offset, st->part_of_pid, parts, part_first_dev,
                                                                                                                     cursor_dev, stage, nullptr);
            CSA_LAUNCH_CHECK(ctx);
            CSA_CUDA(ctx, cudaEventRecord(scattered, ctx->stream));
            CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));       // chunk_first is a host array that the next stretch rewrites
            CSA_CUDA(ctx, cudaStreamWaitEvent(copy_stream, scattered, 0));
            for(u32 u = 0; u < first_file_part; ++u)
            {
                if(chunk_hist[u] == 0) continue;
                CSA_CUDA(ctx, cudaMemcpyAsync(lanes_of(u) + 5 * filled[u], stage + 5 * chunk_first[u], 5 * chunk_hist[u], cudaMemcpyDeviceToHost, copy_stream));
                filled[u] += chunk_hist[u];
            }
            if(files_in_use)
            {
                // The runs of the file parts follow one another in the staging buffer: one copy to the host, then one write per part.
                const u64 from = chunk_first[first_file_part], bytes = 5 * (c - from);
                u8* const via = to_files[k & 1];
                if(bytes) CSA_CUDA(ctx, cudaMemcpyAsync(via, stage + 5 * from, bytes, cudaMemcpyDeviceToHost, copy_stream));
                CSA_CUDA(ctx, cudaEventRecord(copied[k & 1], copy_stream));
                CSA_CUDA(ctx, cudaStreamSynchronize(copy_stream));
                for(u32 u = first_file_part; u < parts; ++u)
                {
                    if(chunk_hist[u] == 0) continue;
                    if(!files.write(files.lanes_fd[u], via + 5 * (chunk_first[u] - from), 5 * chunk_hist[u], 5 * filled[u]))
                        return csa_fail(ctx, CSA_E_INVALID, "streamed build: writing a part file failed");
                    filled[u] += chunk_hist[u];
                }
            }
            else
                CSA_CUDA(ctx, cudaEventRecord(copied[k & 1], copy_stream));
        }
        CSA_CUDA(ctx, cudaStreamSynchronize(copy_stream));
        for(u32 u = 0; u < parts; ++u) if(filled[u] != part_off[u + 1] - part_off[u]) return csa_fail(ctx, CSA_E_DEVICE, "streamed build: a part's lanes do not add up");
    }
    cudaFree(stage_b.p); stage_b.p = nullptr;
    bs.ms_partition = ms_since(t_start);

    // ---- three workers, each with its own context (stream and scratch), take the parts one by one ---------------------------
    constexpr int WORKERS = 3;
    csa_ctx* wctx[WORKERS] = {ctx, nullptr, nullptr};
    struct Ctx_Guard { csa_ctx** c; ~Ctx_Guard() { for(int i = 1; i < WORKERS; ++i) if(c[i]) csa_ctx_destroy(c[i]); } } ctx_guard{wctx};
    const int workers = parts < u32(WORKERS) ? int(parts) : WORKERS;
    for(int w = 1; w < workers; ++w)
        if(csa_ctx_create(ctx->device, &wctx[w]) != CSA_OK) return csa_fail(ctx, CSA_E_CUDA, "streamed build: cannot create a worker context");
    // A worker's buffers for a file part: its lanes, its ranks, and the lanes in their final order.
    struct Bounce { u8* lanes; u32* ranks; u8* ordered; } bounce[WORKERS] = {};
    if(files_in_use)
        for(int w = 0; w < workers; ++w)
        {
            u8* base = pinned + ranks_bytes + own_lanes_bytes + to_files_bytes;
            if(w > 0)
            {
                void* own = nullptr;
                if(csa_host_aux(wctx[w], bounce_bytes + 256, &own) != CSA_OK) return csa_fail(ctx, CSA_E_NOMEM, "streamed build: cannot pin a worker's buffers");
                base = static_cast<u8*>(own);
            }
            bounce[w].lanes = base;
            bounce[w].ordered = base + align_up256(5 * largest_file_part + 64);
            bounce[w].ranks = reinterpret_cast<u32*>(base + 2 * align_up256(5 * largest_file_part + 64));
        }
    auto worker_of = [&](csa_ctx* c) { for(int w = 0; w < workers; ++w) if(wctx[w] == c) return w; return 0; };
    auto io_failed = [&](csa_ctx* c) { return csa_fail(c, CSA_E_INVALID, "streamed build: reading or writing a part file failed"); };
    std::vector<u64> active(parts);
    // Runs job(context, part) over all parts on the workers; returns the first error.
    auto over_parts = [&](auto job) -> int
    {
        std::atomic<u32> next{0};
        std::atomic<int> first_rc{CSA_OK};
        std::string why[WORKERS];
        auto body = [&](int w)
        {
            cudaSetDevice(ctx->device);
            for(;;)
            {
                const u32 u = next.fetch_add(1);
                if(u >= parts || first_rc.load() != CSA_OK) break;
                int rc = job(wctx[w], u);
                if(rc == CSA_OK) { u64 b = 0; rc = csa_sync(wctx[w], reinterpret_cast<uint64_t*>(&b)); }
                if(rc != CSA_OK) { int expected = CSA_OK; if(first_rc.compare_exchange_strong(expected, rc)) why[w] = wctx[w]->err; break; }
            }
        };
        std::vector<std::thread> pool;
        for(int w = 1; w < workers; ++w) pool.emplace_back(body, w);
        body(0);
        for(auto& t : pool) t.join();
        if(first_rc.load() != CSA_OK) for(int w = 0; w < WORKERS; ++w) if(!why[w].empty()) ctx->err = why[w];
        return first_rc.load();
    };

    // ---- generation 0 ----------------------------------------------------------------------------------------------------------
    const auto t_gen0 = std::chrono::steady_clock::now();
    CSA_TRY(over_parts([&](csa_ctx* c, u32 u) -> int
    {
        const u64 S = part_off[u + 1] - part_off[u];
        if(u < first_file_part)
        {
            csa_part in{lanes_of(u), nullptr, S, u};
            csa_part_result out{lanes_of(u), ranks_of(u), 0, 0};
            const int rc = csa_rank_gen0(c, st, &in, &out);
            active[u] = out.active;
            return rc;
        }
        const Bounce& b = bounce[worker_of(c)];
        if(!files.read(files.lanes_fd[u], b.lanes, 5 * S, 0)) return io_failed(c);
        csa_part in{b.lanes, nullptr, S, u};
        csa_part_result out{b.lanes, b.ranks, 0, 0};
        CSA_TRY(csa_rank_gen0(c, st, &in, &out));
        active[u] = out.active;
        u64 status = 0;
        CSA_TRY(csa_sync(c, reinterpret_cast<uint64_t*>(&status)));
        if(!files.write(files.lanes_fd[u], b.lanes, 5 * S, 0) || !files.write(files.ranks_fd[u], b.ranks, 4 * S, 0)) return io_failed(c);
        return CSA_OK;
    }));
    csa_store_drop_partition_ids(st);
    cudaFree(pid_b.p); pid_b.p = nullptr;
    u64 total_active = 0;
    for(u32 u = 0; u < parts; ++u) total_active += active[u];
    bs.active_after_gen0 = total_active;
    bs.ms_gen0 = ms_since(t_gen0);
    const bool debug = std::getenv("CSA_DEBUG") != nullptr;
    if(debug) std::fprintf(stderr, "[csa streamed] n=%llu partitions=%u parts=%u largest part=%llu active after generation 0: %llu; text, ids and pinned ranks after %.0f ms, "
                           "lanes on the host after %.0f ms\n", (unsigned long long)n, p_eff, parts, (unsigned long long)largest_part, (unsigned long long)total_active,
                           ms_pinned, bs.ms_partition);

    // ---- doubling generations ------------------------------------------------------------------------------------------------
    const auto t_dbl = std::chrono::steady_clock::now();
    u64 h = 3;
    u32 gen = 0;
    while(total_active > 0)
    {
        if(gen < 48) bs.active_per_gen[gen] = total_active;
        CSA_TRY(csa_store_reserve_messages(ctx, st, total_active));
        CSA_TRY(over_parts([&](csa_ctx* c, u32 u) -> int
        {
            if(active[u] == 0) return CSA_OK;
            if(u < first_file_part)
            {
                csa_part in{lanes_of(u), ranks_of(u), active[u], u};
                csa_part_result out{lanes_of(u), ranks_of(u), 0, 0};
                const int rc = csa_rank_gen(c, st, &in, h, &out);
                active[u] = out.active;
                return rc;
            }
            // Only the tied suffixes, which lead the part's lists, travel.
            const Bounce& b = bounce[worker_of(c)];
            const u64 tied = active[u];
            if(!files.read(files.lanes_fd[u], b.lanes, 5 * tied, 0) || !files.read(files.ranks_fd[u], b.ranks, 4 * tied, 0)) return io_failed(c);
            csa_part in{b.lanes, b.ranks, tied, u};
            csa_part_result out{b.lanes, b.ranks, 0, 0};
            CSA_TRY(csa_rank_gen(c, st, &in, h, &out));
            active[u] = out.active;
            u64 status = 0;
            CSA_TRY(csa_sync(c, reinterpret_cast<uint64_t*>(&status)));
            if(!files.write(files.lanes_fd[u], b.lanes, 5 * tied, 0) || !files.write(files.ranks_fd[u], b.ranks, 4 * tied, 0)) return io_failed(c);
            return CSA_OK;
        }));
        uint64_t applied = 0;
        CSA_TRY(csa_exchange_messages(ctx, st, &applied));
        u64 next_total = 0;
        for(u32 u = 0; u < parts; ++u) next_total += active[u];
        if(debug) std::fprintf(stderr, "[csa streamed] generation %u: h=%llu active %llu -> %llu (%llu messages)\n", gen + 1, (unsigned long long)h,
                               (unsigned long long)total_active, (unsigned long long)next_total, (unsigned long long)applied);
        total_active = next_total;
        ++gen;
        if(h > (u64(1) << 41)) return csa_fail(ctx, CSA_E_DEVICE, "streamed build: doubling did not terminate");
        h *= 2;
    }
    bs.generations = gen;
    bs.ms_doubling = ms_since(t_dbl);

    // ---- every part into its final order, in place in the output array ------------------------------------------------------------
    const auto t_out = std::chrono::steady_clock::now();
    CSA_TRY(over_parts([&](csa_ctx* c, u32 u) -> int
    {
        const u64 S = part_off[u + 1] - part_off[u];
        u64 status = 0;
        if(u < first_file_part)
        {
            CSA_TRY(csa_rank_order(c, lanes_of(u), ranks_of(u), S, lanes_of(u)));
            if(out_file.fd < 0) return CSA_OK;
            CSA_TRY(csa_sync(c, reinterpret_cast<uint64_t*>(&status)));
            return write_all(out_file.fd, lanes_of(u), 5 * S, 5 * part_off[u]) ? CSA_OK : io_failed(c);
        }
        const Bounce& b = bounce[worker_of(c)];
        if(!files.read(files.lanes_fd[u], b.lanes, 5 * S, 0) || !files.read(files.ranks_fd[u], b.ranks, 4 * S, 0)) return io_failed(c);
        CSA_TRY(csa_rank_order(c, b.lanes, b.ranks, S, b.ordered));
        CSA_TRY(csa_sync(c, reinterpret_cast<uint64_t*>(&status)));
        if(sa40_host) std::memcpy(sa40_host + 5 * part_off[u], b.ordered, 5 * S);
        if(out_file.fd >= 0 && !write_all(out_file.fd, b.ordered, 5 * S, 5 * part_off[u])) return io_failed(c);
        return CSA_OK;
    }));
    bs.host_parts = first_file_part;
    bs.file_parts = parts - first_file_part;
    bs.file_bytes_read = files.bytes_read.load();
    bs.file_bytes_written = files.bytes_written.load();
    bs.ms_output = ms_since(t_out);
    bs.ms_total = ms_since(t_start);
    for(int w = 0; w < workers; ++w)
    {
        bs.kernel_launches += wctx[w]->counters[0] - (w == 0 ? launches_before : 0);
        bs.sort_passes += wctx[w]->counters[1] - (w == 0 ? passes_before : 0);
        bs.sort_records += wctx[w]->counters[2] - (w == 0 ? records_before : 0);
    }
    return CSA_OK;
}

extern "C" int csa_build_sa_streamed(csa_ctx* ctx, const uint16_t* text_host, uint64_t n, uint32_t p, uint64_t seed, uint8_t* sa40_host,
                                     uint64_t part_suffixes, csa_build_stats* stats)
{
    if(!sa40_host) return csa_fail(ctx, CSA_E_INVALID, "streamed build: null argument");
    csa_tier_options options{};
    options.part_suffixes = part_suffixes;
    options.host_list_bytes = ~uint64_t(0);
    return csa_build_sa_tiered(ctx, text_host, n, p, seed, sa40_host, &options, stats);
}
