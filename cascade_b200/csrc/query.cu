// Batched count / locate queries over a suffix-array index: a sample table of packed K-grams (every stride-th
// suffix) brackets each boundary of a query's interval, and a binary search of the suffix array inside the bracket
// finds it exactly. Results equal ref::find_one's (include/CPU_Reference.hpp:42-73).
//
// Reference behaviour followed: Sample_Table build_kernel (src/Sample_Table.cu:26-31), the bracket rules of
// table_kernel (src/Query_Engine.cu:205-279), search_kernel (:369-418) and certify_kernel (:665-686). Locate has no
// counterpart there; it lists SA[lo + k] in rank order.
#include "common.cuh"

namespace
{

__global__ void table_build_kernel(const u16* __restrict__ T, const u8* __restrict__ sa40, const u64 n, const u64 stride, const u64 entries,
                                   u64* __restrict__ table)
{
    const u64 j = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if(j >= entries) return;
    const u64 pos = sa40_load(sa40, j * stride);
    if(pos >= n) { table[2 * j] = 0; table[2 * j + 1] = 0; return; }
    table[2 * j] = pack4(T, pos);          // the text's zero padding pads short suffixes
    table[2 * j + 1] = pack4(T, pos + 4);
}

// Order of the suffix at `pos`, truncated to m symbols, against the pattern: -1, 0 or 1; a suffix that ends before
// m symbols while still matching is smaller (ref::cmp_suffix_pattern, include/CPU_Reference.hpp:26-36).
__device__ __forceinline__ int cmp_suffix_pattern(const u16* __restrict__ T, const u64 n, const u64 pos, const u16* __restrict__ P, const u64 m)
{
    const u64 len = (n - pos < m) ? n - pos : m;
    for(u64 i = 0; i < len; ++i)
    {
        const u16 a = T[pos + i], b = P[i];
        if(a != b) return a < b ? -1 : 1;
    }
    return len < m ? -1 : 0;
}

// The ranks that can hold the two boundaries of a query's interval, from the sample table alone.
struct Brackets { u64 lo_first, lo_last, hi_first, hi_last; };

__device__ __forceinline__ Brackets table_brackets(const csa_index& idx, const u16* __restrict__ P, const u64 m)
{
    const u64 stride = idx.stride;
    const u64 ne = idx.sa_entries ? idx.sa_entries : idx.n;      // entries of the suffix array (a slice of it in a sharded index)
    // The pattern's first min(m, K) symbols, packed like a table key, and the mask of those symbols.
    const u32 mm = m < CSA_K ? u32(m) : u32(CSA_K);
    u64 qh = 0, ql = 0;
    for(u32 k = 0; k < mm; ++k)
    {
        if(k < 4) qh |= u64(P[k]) << (48 - 16 * k);
        else ql |= u64(P[k]) << (48 - 16 * (k - 4));
    }
    const u64 mask_h = mm >= 4 ? ~0ull : ~0ull << (64 - 16 * mm);
    const u64 mask_l = mm <= 4 ? 0ull : (mm == 8 ? ~0ull : ~0ull << (64 - 16 * (mm - 4)));

    const u64 J = (ne + stride - 1) / stride;
    const ulonglong2* const tab = reinterpret_cast<const ulonglong2*>(idx.table);
    // a = table keys (masked) smaller than the pattern's; b = those not greater.
    u64 a, b;
    {
        u64 x = 0, y = J;
        while(x < y)
        {
            const u64 mid = x + ((y - x) >> 1);
            const ulonglong2 t = tab[mid];
            const u64 th = t.x & mask_h, tl = t.y & mask_l;
            if(th < qh || (th == qh && tl < ql)) x = mid + 1; else y = mid;
        }
        a = x;
        // b lies at or shortly after a unless the pattern's K-gram is very frequent: gallop from a (1, 2, 4, ... keys ahead)
        // to the first key that is greater, then bisect what is left. Every probe is a dependent random read, and this
        // spares about twenty of them per query.
        y = J;
        for(u64 step = 1; x < y; step <<= 1)
        {
            const u64 mid = (x + step - 1 < y) ? x + step - 1 : y - 1;
            const ulonglong2 t = tab[mid];
            const u64 th = t.x & mask_h, tl = t.y & mask_l;
            if(th < qh || (th == qh && tl <= ql)) x = mid + 1; else { y = mid; break; }
        }
        while(x < y)
        {
            const u64 mid = x + ((y - x) >> 1);
            const ulonglong2 t = tab[mid];
            const u64 th = t.x & mask_h, tl = t.y & mask_l;
            if(th < qh || (th == qh && tl <= ql)) x = mid + 1; else y = mid;
        }
        b = x;
    }
    // Sampled rank j * stride carries table key j. Ranks up to (a-1) stride are smaller than the pattern; ranks from
    // b stride on are greater.
    Brackets br;
    br.lo_first = (a == 0) ? 0 : (a - 1) * stride + 1;
    br.hi_last = (b >= J) ? ne : b * stride;
    br.lo_last = br.hi_last;
    br.hi_first = br.lo_first;
    if(m <= CSA_K)
    {
        // Every suffix whose masked key equals the pattern's matches it, except suffixes that end inside the pattern and
        // owe the equality to zero padding; there are fewer than m of them and they need the pattern to end in a zero.
        const u64 e = (P[m - 1] == 0) ? m - 1 : 0;
        const u64 cap = a * stride + e;
        if(cap < br.lo_last) br.lo_last = cap;
        if(b > 0 && (b - 1) * stride + 1 > br.hi_first) br.hi_first = (b - 1) * stride + 1;
    }
    return br;
}

// Both boundaries of the interval by binary search inside the brackets. `sa_lo` / `sa_hi` are what entry r of the suffix
// array is read from in each search: the array itself, or a gathered window shifted so that the same r addresses it.
__device__ __forceinline__ void search_brackets(const csa_index& idx, const Brackets& br, const u16* __restrict__ P, const u64 m, const u8* sa_lo,
                                                const u8* sa_hi, u64& lo_out, u64& hi_out)
{
    const u64 n = idx.n;
    const u16* const T = idx.text;
    u64 x = br.lo_first, y = br.lo_last;
    while(x < y)
    {
        const u64 mid = x + ((y - x) >> 1);
        if(cmp_suffix_pattern(T, n, sa40_load(sa_lo, mid), P, m) < 0) x = mid + 1; else y = mid;
    }
    lo_out = x;
    x = (br.hi_first > x) ? br.hi_first : x;
    y = br.hi_last;
    if(x > y) x = y;
    // most patterns occur a few times: the end of the interval is galloped to from its start, then bisected
    for(u64 step = 1; x < y; step <<= 1)
    {
        const u64 mid = (x + step - 1 < y) ? x + step - 1 : y - 1;
        if(cmp_suffix_pattern(T, n, sa40_load(sa_hi, mid), P, m) <= 0) x = mid + 1; else { y = mid; break; }
    }
    while(x < y)
    {
        const u64 mid = x + ((y - x) >> 1);
        if(cmp_suffix_pattern(T, n, sa40_load(sa_hi, mid), P, m) <= 0) x = mid + 1; else y = mid;
    }
    hi_out = x;
}

__global__ void find_kernel(const csa_index idx, const u64* __restrict__ off, const u16* __restrict__ sym, const u64 q, u64* __restrict__ itv)
{
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if(i >= q) return;
    const u64 m = off[i + 1] - off[i];
    const u16* const P = sym + (off[i] - off[0]);
    if(m == 0) { itv[2 * i] = 0; itv[2 * i + 1] = idx.sa_entries ? idx.sa_entries : idx.n; return; }
    if(idx.sa_entries != 0 && idx.sa_entries < idx.n)
    {
        // One slice of a sharded array: most patterns lie wholly before or wholly after it, which its first and last suffix
        // tell with two comparisons; only a pattern that falls inside the slice's range is searched for.
        const u64 e = idx.sa_entries;
        if(cmp_suffix_pattern(idx.text, idx.n, sa40_load(idx.sa40, 0), P, m) > 0) { itv[2 * i] = 0; itv[2 * i + 1] = 0; return; }
        if(cmp_suffix_pattern(idx.text, idx.n, sa40_load(idx.sa40, e - 1), P, m) < 0) { itv[2 * i] = e; itv[2 * i + 1] = e; return; }
    }
    const Brackets br = table_brackets(idx, P, m);
    u64 lo, hi;
    search_brackets(idx, br, P, m, idx.sa40, idx.sa40, lo, hi);
    itv[2 * i] = lo;
    itv[2 * i + 1] = hi;
}

// ---- the same search when the suffix array lies in pinned host memory -------------------------------------------------
// Every probe of the array would be a PCIe round trip, so the entries of both brackets are first gathered into device
// memory, one warp per query with 16-byte loads (the reference's gather_kernel, src/Query_Engine.cu:334-354, does the same
// for its pinned plan), and the binary searches then run on the gathered windows. A bracket wider than WINDOW_ENTRIES
// (a long pattern whose K-gram prefix is very frequent) is searched in place.
constexpr u32 WINDOW_ENTRIES = 64;
constexpr u32 WINDOW_BYTES = 352;       // 5 * (WINDOW_ENTRIES + 1) entries' bytes + alignment slack + the load overrun, in 16-byte pieces

__global__ void brackets_kernel(const csa_index idx, const u64* __restrict__ off, const u16* __restrict__ sym, const u64 q, Brackets* __restrict__ out)
{
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if(i >= q) return;
    const u64 m = off[i + 1] - off[i];
    Brackets br{0, 0, 0, 0};
    if(m > 0) br = table_brackets(idx, sym + (off[i] - off[0]), m);
    out[i] = br;
}

__device__ __forceinline__ bool window_fits(u64 first, u64 last) { return last - first <= WINDOW_ENTRIES; }

__global__ void gather_windows_kernel(const u8* __restrict__ sa40, const Brackets* __restrict__ br, const u64 q, u8* __restrict__ win)
{
    const u64 w = (u64(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if(w >= q) return;
    const Brackets b = br[w];
    #pragma unroll
    for(int side = 0; side < 2; ++side)
    {
        const u64 first = side ? b.hi_first : b.lo_first, last = side ? b.hi_last : b.lo_last;
        if(last < first || !window_fits(first, last)) continue;
        if(side == 1 && b.hi_first == b.lo_first && b.hi_last == b.lo_last) continue;     // one window serves both searches (patterns longer than K)
        const u64 byte0 = (5 * first) & ~u64(15), byte1 = 5 * last + 5 + 4;       // entry `last` may be probed; a load reads 8 bytes
        const u32 pieces = u32((byte1 - byte0 + 15) >> 4);
        const uint4* src = reinterpret_cast<const uint4*>(sa40 + byte0);
        uint4* dst = reinterpret_cast<uint4*>(win + (2 * w + side) * WINDOW_BYTES);
        if(lane_id() < pieces && lane_id() < WINDOW_BYTES / 16) dst[lane_id()] = src[lane_id()];
    }
}

__global__ void search_windows_kernel(const csa_index idx, const u64* __restrict__ off, const u16* __restrict__ sym, const u64 q,
                                      const Brackets* __restrict__ brs, const u8* __restrict__ win, u64* __restrict__ itv)
{
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if(i >= q) return;
    const u64 m = off[i + 1] - off[i];
    if(m == 0) { itv[2 * i] = 0; itv[2 * i + 1] = idx.sa_entries ? idx.sa_entries : idx.n; return; }
    const Brackets br = brs[i];
    // A window holds the array's bytes from (5 first) & ~15 on; shifting its base back by that much lets rank r address it.
    const u8* sa_lo = idx.sa40;
    const u8* sa_hi = idx.sa40;
    if(br.lo_last >= br.lo_first && window_fits(br.lo_first, br.lo_last)) sa_lo = win + (2 * i) * WINDOW_BYTES - ((5 * br.lo_first) & ~u64(15));
    if(br.hi_last >= br.hi_first && window_fits(br.hi_first, br.hi_last))
    {
        const bool shared = br.hi_first == br.lo_first && br.hi_last == br.lo_last;
        sa_hi = win + (2 * i + (shared ? 0 : 1)) * WINDOW_BYTES - ((5 * br.hi_first) & ~u64(15));
    }
    u64 lo, hi;
    search_brackets(idx, br, sym + (off[i] - off[0]), m, sa_lo, sa_hi, lo, hi);
    itv[2 * i] = lo;
    itv[2 * i + 1] = hi;
}

// One warp per query: row i of pos receives SA[lo + k], k < min(max_pos, hi - lo).
__global__ void locate_rows_kernel(const u8* __restrict__ sa40, const u64* __restrict__ itv, const u64 q, const u32 max_pos, u64* __restrict__ pos,
                                   u32* __restrict__ cnt)
{
    const u64 w = (u64(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if(w >= q) return;
    const u64 lo = itv[2 * w], hi = itv[2 * w + 1];
    const u64 c = (hi - lo < max_pos) ? hi - lo : max_pos;
    if(lane_id() == 0) cnt[w] = u32(c);
    for(u64 k = lane_id(); k < c; k += 32) pos[w * max_pos + k] = sa40_load(sa40, lo + k);
}

// The same into one packed array: query i's positions start at pos_off[i].
__global__ void locate_packed_kernel(const u8* __restrict__ sa40, const u64* __restrict__ itv, const u64 q, const u32 max_pos,
                                     const u64* __restrict__ pos_off, u64* __restrict__ pos)
{
    const u64 w = (u64(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if(w >= q) return;
    const u64 lo = itv[2 * w], hi = itv[2 * w + 1];
    const u64 c = (hi - lo < max_pos) ? hi - lo : max_pos;
    const u64 o = pos_off[w];
    for(u64 k = lane_id(); k < c; k += 32) pos[o + k] = sa40_load(sa40, lo + k);
}

// Sharded locate: the columns of a global interval's row that fall into this slice of the suffix array.
__global__ void locate_window_kernel(const u8* __restrict__ sa40, const u64 sa_first, const u64 sa_entries, const u64* __restrict__ itv, const u64 q,
                                     const u32 max_pos, u64* __restrict__ pos)
{
    const u64 w = (u64(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if(w >= q) return;
    const u64 lo = itv[2 * w], hi = itv[2 * w + 1];
    const u64 c = (hi - lo < max_pos) ? hi - lo : max_pos;
    for(u64 k = lane_id(); k < c; k += 32)
    {
        const u64 r = lo + k;
        if(r >= sa_first && r < sa_first + sa_entries) pos[w * max_pos + k] = sa40_load(sa40, r - sa_first);
    }
}

// Sharded locate into ONE packed array: the entries of a global interval's first max_pos ranks that fall into this slice go to
// pos[pos_off[i] + k] (rank lo + k); the other entries are left as they are, so packed arrays that all shards write into, starting
// from zeros, add up to the packed positions of the whole index.
__global__ void locate_window_packed_kernel(const u8* __restrict__ sa40, const u64 sa_first, const u64 sa_entries, const u64* __restrict__ itv, const u64 q,
                                            const u32 max_pos, const u64* __restrict__ pos_off, u64* __restrict__ pos)
{
    const u64 w = (u64(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if(w >= q) return;
    const u64 lo = itv[2 * w], hi = itv[2 * w + 1];
    const u64 c = (hi - lo < max_pos) ? hi - lo : max_pos;
    if(c == 0 || lo + c <= sa_first || lo >= sa_first + sa_entries) return;
    const u64 o = pos_off[w];
    for(u64 k = lane_id(); k < c; k += 32)
    {
        const u64 r = lo + k;
        if(r >= sa_first && r < sa_first + sa_entries) pos[o + k] = sa40_load(sa40, r - sa_first);
    }
}

__global__ void counts_kernel(const u64* __restrict__ itv, const u64 q, const u32 max_pos, u32* __restrict__ cnt)
{
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if(i >= q) return;
    const u64 d = itv[2 * i + 1] - itv[2 * i];
    cnt[i] = u32(d < max_pos ? d : max_pos);
}

// Exclusive prefix sums of 32-bit counts into 64-bit offsets (off[count] = total), in three steps without waits:
// block sums, a one-block scan of them, and the per-block scans.
constexpr int SCAN_BLOCK = 256, SCAN_ITEMS = 8, SCAN_TILE = SCAN_BLOCK * SCAN_ITEMS;

__global__ void __launch_bounds__(SCAN_BLOCK) scan_sums_kernel(const u32* __restrict__ in, const u64 count, u64* __restrict__ sums)
{
    __shared__ u64 s[SCAN_BLOCK / 32];
    u64 v = 0;
    const u64 first = u64(blockIdx.x) * SCAN_TILE + u64(threadIdx.x) * SCAN_ITEMS;
    for(int i = 0; i < SCAN_ITEMS; ++i) if(first + i < count) v += in[first + i];
    for(int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    if(lane_id() == 0) s[threadIdx.x >> 5] = v;
    __syncthreads();
    if(threadIdx.x == 0) { u64 t = 0; for(int w = 0; w < SCAN_BLOCK / 32; ++w) t += s[w]; sums[blockIdx.x] = t; }
}

__global__ void __launch_bounds__(1024) scan_carry_kernel(u64* __restrict__ sums, const u64 tiles, u64* __restrict__ total)
{
    __shared__ u64 s[32];
    __shared__ u64 carry;
    if(threadIdx.x == 0) carry = 0;
    __syncthreads();
    for(u64 base = 0; base < tiles; base += 1024)
    {
        const u64 t = base + threadIdx.x;
        const u64 v = (t < tiles) ? sums[t] : 0;
        u64 inc = v;
        for(int o = 1; o < 32; o <<= 1) { const u64 u = __shfl_up_sync(0xFFFFFFFFu, inc, o); if(int(lane_id()) >= o) inc += u; }
        if(lane_id() == 31) s[threadIdx.x >> 5] = inc;
        __syncthreads();
        u64 pre = carry;
        for(u32 w = 0; w < (threadIdx.x >> 5); ++w) pre += s[w];
        __syncthreads();
        if(t < tiles) sums[t] = pre + inc - v;
        if(threadIdx.x == 1023) carry = pre + inc;
        __syncthreads();
    }
    if(threadIdx.x == 0) *total = carry;
}

__global__ void __launch_bounds__(SCAN_BLOCK) scan_apply_kernel(const u32* __restrict__ in, const u64 count, const u64* __restrict__ sums,
                                                               const u64* __restrict__ total, u64* __restrict__ out)
{
    __shared__ u64 s[SCAN_BLOCK / 32];
    const u64 first = u64(blockIdx.x) * SCAN_TILE + u64(threadIdx.x) * SCAN_ITEMS;
    u32 v[SCAN_ITEMS];
    u64 mine = 0;
    for(int i = 0; i < SCAN_ITEMS; ++i) { v[i] = (first + i < count) ? in[first + i] : 0; mine += v[i]; }
    u64 inc = mine;
    for(int o = 1; o < 32; o <<= 1) { const u64 u = __shfl_up_sync(0xFFFFFFFFu, inc, o); if(int(lane_id()) >= o) inc += u; }
    if(lane_id() == 31) s[threadIdx.x >> 5] = inc;
    __syncthreads();
    u64 run = sums[blockIdx.x] + inc - mine;
    for(u32 w = 0; w < (threadIdx.x >> 5); ++w) run += s[w];
    for(int i = 0; i < SCAN_ITEMS; ++i)
    {
        if(first + i < count) out[first + i] = run;
        run += v[i];
    }
    if(blockIdx.x == 0 && threadIdx.x == 0) out[count] = *total;
}

__global__ void certify_kernel(const csa_index idx, const u64* __restrict__ off, const u16* __restrict__ sym, const u64 q, const u64* __restrict__ itv,
                               u64* __restrict__ result)
{
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if(i >= q) return;
    const u64 n = idx.n, m = off[i + 1] - off[i], lo = itv[2 * i], hi = itv[2 * i + 1];
    const u16* const P = sym + (off[i] - off[0]);
    bool ok = true;
    if(lo > hi || hi > n) ok = false;
    else if(m == 0) ok = (lo == 0 && hi == n);
    else
    {
        if(lo > 0 && cmp_suffix_pattern(idx.text, n, sa40_load(idx.sa40, lo - 1), P, m) >= 0) ok = false;
        if(ok && lo < hi && (cmp_suffix_pattern(idx.text, n, sa40_load(idx.sa40, lo), P, m) != 0
                             || cmp_suffix_pattern(idx.text, n, sa40_load(idx.sa40, hi - 1), P, m) != 0)) ok = false;
        if(ok && hi < n && cmp_suffix_pattern(idx.text, n, sa40_load(idx.sa40, hi), P, m) <= 0) ok = false;
    }
    if(!ok)
    {
        atomicAdd(&result[0], 1ull);
        atomicMin(&result[1], i);
    }
}

int check_index(csa_ctx* ctx, const csa_index* index)
{
    if(!ctx || !index || !index->text || !index->sa40 || !index->table || index->n == 0 || index->stride == 0)
        return csa_fail(ctx, CSA_E_INVALID, "query: incomplete index");
    if(reinterpret_cast<uintptr_t>(index->sa40) & 3) return csa_fail(ctx, CSA_E_INVALID, "query: the suffix array must be 4-byte aligned");
    if(reinterpret_cast<uintptr_t>(index->table) & 15) return csa_fail(ctx, CSA_E_INVALID, "query: the sample table must be 16-byte aligned");
    return CSA_OK;
}

int exclusive_sum(csa_ctx* ctx, const u32* in, u64 count, u64* out, u64* sums_scratch, u64* total_dev)
{
    const u64 tiles = div_up(count, SCAN_TILE);
    if(tiles == 0) { CSA_CUDA(ctx, cudaMemsetAsync(out, 0, 8, ctx->stream)); CSA_CUDA(ctx, cudaMemsetAsync(total_dev, 0, 8, ctx->stream)); return CSA_OK; }
    scan_sums_kernel<<<unsigned(tiles), SCAN_BLOCK, 0, ctx->stream>>>(in, count, sums_scratch);
    CSA_LAUNCH_CHECK(ctx);
    scan_carry_kernel<<<1, 1024, 0, ctx->stream>>>(sums_scratch, tiles, total_dev);
    CSA_LAUNCH_CHECK(ctx);
    scan_apply_kernel<<<unsigned(tiles), SCAN_BLOCK, 0, ctx->stream>>>(in, count, sums_scratch, total_dev, out);
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

}   // namespace

extern "C" int csa_table_build(csa_ctx* ctx, const uint16_t* text, uint64_t n, const uint8_t* sa40, uint64_t stride, uint64_t* table)
{
    if(!ctx || !text || !sa40 || !table || n == 0 || stride == 0) return csa_fail(ctx, CSA_E_INVALID, "csa_table_build: bad argument");
    if(reinterpret_cast<uintptr_t>(sa40) & 3) return csa_fail(ctx, CSA_E_INVALID, "csa_table_build: the suffix array must be 4-byte aligned");
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    const u64 entries = div_up(n, stride);
    table_build_kernel<<<unsigned(div_up(entries, 256)), 256, 0, ctx->stream>>>(text, sa40, n, stride, entries, reinterpret_cast<u64*>(table));
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

extern "C" int csa_table_build_slice(csa_ctx* ctx, const uint16_t* text, uint64_t n, const uint8_t* sa40_slice, uint64_t sa_entries, uint64_t stride,
                                     uint64_t* table)
{
    if(!ctx || !text || !sa40_slice || !table || n == 0 || stride == 0 || sa_entries > n) return csa_fail(ctx, CSA_E_INVALID, "csa_table_build_slice: bad argument");
    if(reinterpret_cast<uintptr_t>(sa40_slice) & 3) return csa_fail(ctx, CSA_E_INVALID, "csa_table_build_slice: the slice must start 4-byte aligned");
    if(sa_entries == 0) return CSA_OK;
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    const u64 entries = div_up(sa_entries, stride);
    table_build_kernel<<<unsigned(div_up(entries, 256)), 256, 0, ctx->stream>>>(text, sa40_slice, n, stride, entries, reinterpret_cast<u64*>(table));
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

extern "C" int csa_locate_window(csa_ctx* ctx, const csa_index* index, const uint64_t* itv, uint64_t q, uint32_t max_pos, uint64_t* pos)
{
    CSA_TRY(check_index(ctx, index));
    if(q == 0) return CSA_OK;
    if(!itv || !pos || max_pos == 0) return csa_fail(ctx, CSA_E_INVALID, "csa_locate_window: bad argument");
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    const u64 ne = index->sa_entries ? index->sa_entries : index->n;
    locate_window_kernel<<<unsigned(div_up(q * 32, 256)), 256, 0, ctx->stream>>>(index->sa40, index->sa_first, ne, reinterpret_cast<const u64*>(itv), q, max_pos,
                                                                                 reinterpret_cast<u64*>(pos));
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

extern "C" int csa_locate_window_packed(csa_ctx* ctx, const csa_index* index, const uint64_t* itv, uint64_t q, uint32_t max_pos, uint32_t* cnt, uint64_t* pos_off,
                                        uint64_t* pos, uint64_t* total)
{
    CSA_TRY(check_index(ctx, index));
    if(q == 0) return CSA_OK;
    if(!itv || !cnt || !pos_off || !pos || !total || max_pos == 0) return csa_fail(ctx, CSA_E_INVALID, "csa_locate_window_packed: bad argument");
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    void* ws = nullptr;
    CSA_TRY(csa_aux(ctx, align_up256((div_up(q, SCAN_TILE) + 1) * 8), &ws));
    counts_kernel<<<unsigned(div_up(q, 256)), 256, 0, ctx->stream>>>(reinterpret_cast<const u64*>(itv), q, max_pos, cnt);
    CSA_LAUNCH_CHECK(ctx);
    CSA_TRY(exclusive_sum(ctx, cnt, q, reinterpret_cast<u64*>(pos_off), static_cast<u64*>(ws), reinterpret_cast<u64*>(total)));
    const u64 ne = index->sa_entries ? index->sa_entries : index->n;
    locate_window_packed_kernel<<<unsigned(div_up(q * 32, 256)), 256, 0, ctx->stream>>>(index->sa40, index->sa_first, ne, reinterpret_cast<const u64*>(itv), q, max_pos,
                                                                                        reinterpret_cast<const u64*>(pos_off), reinterpret_cast<u64*>(pos));
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

extern "C" int csa_find(csa_ctx* ctx, const csa_index* index, const uint64_t* off, const uint16_t* sym, uint64_t q, uint64_t* itv)
{
    CSA_TRY(check_index(ctx, index));
    if(q == 0) return CSA_OK;
    if(!off || !itv) return csa_fail(ctx, CSA_E_INVALID, "csa_find: null buffer");
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    cudaPointerAttributes attr;
    const bool sa_on_host = cudaPointerGetAttributes(&attr, index->sa40) == cudaSuccess && attr.type == cudaMemoryTypeHost;
    cudaGetLastError();
    if(!sa_on_host)
    {
        find_kernel<<<unsigned(div_up(q, 128)), 128, 0, ctx->stream>>>(*index, reinterpret_cast<const u64*>(off), sym, q, reinterpret_cast<u64*>(itv));
        CSA_LAUNCH_CHECK(ctx);
        return CSA_OK;
    }
    // Suffix array in pinned host memory: brackets from the table, the brackets' entries gathered over PCIe, search on the
    // device. Batches of 2^20 queries bound the window buffer (about 0.8 GB).
    constexpr u64 BATCH = u64(1) << 20;
    const u64 per = (q < BATCH ? q : BATCH);
    void* aux = nullptr;
    CSA_TRY(csa_aux(ctx, align_up256(per * sizeof(Brackets)) + align_up256(per * 2 * WINDOW_BYTES + 256), &aux));
    Brackets* brs = static_cast<Brackets*>(aux);
    u8* win = static_cast<u8*>(aux) + align_up256(per * sizeof(Brackets));
    for(u64 first = 0; first < q; first += BATCH)
    {
        const u64 c = (q - first < BATCH ? q - first : BATCH);
        const u64* o = reinterpret_cast<const u64*>(off) + first;
        // The kernels address pattern i at sym + (off[i] - off[0]) of the offsets they are given, so a later batch gets the
        // symbol pointer moved on by the symbols that precede it.
        const u16* sy = sym;
        if(first > 0)
        {
            u64 begin[2] = {0, 0};
            CSA_CUDA(ctx, cudaMemcpyAsync(&begin[0], off, 8, cudaMemcpyDefault, ctx->stream));
            CSA_CUDA(ctx, cudaMemcpyAsync(&begin[1], o, 8, cudaMemcpyDefault, ctx->stream));
            CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            sy = sym + (begin[1] - begin[0]);
        }
        brackets_kernel<<<unsigned(div_up(c, 128)), 128, 0, ctx->stream>>>(*index, o, sy, c, brs);
        CSA_LAUNCH_CHECK(ctx);
        gather_windows_kernel<<<unsigned(div_up(c * 32, 256)), 256, 0, ctx->stream>>>(index->sa40, brs, c, win);
        CSA_LAUNCH_CHECK(ctx);
        search_windows_kernel<<<unsigned(div_up(c, 128)), 128, 0, ctx->stream>>>(*index, o, sy, c, brs, win, reinterpret_cast<u64*>(itv) + 2 * first);
        CSA_LAUNCH_CHECK(ctx);
    }
    return CSA_OK;
}

extern "C" int csa_locate(csa_ctx* ctx, const csa_index* index, const uint64_t* itv, uint64_t q, uint32_t max_pos, uint64_t* pos, uint32_t* cnt)
{
    CSA_TRY(check_index(ctx, index));
    if(q == 0) return CSA_OK;
    if(!itv || !pos || !cnt || max_pos == 0) return csa_fail(ctx, CSA_E_INVALID, "csa_locate: bad argument");
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    locate_rows_kernel<<<unsigned(div_up(q * 32, 256)), 256, 0, ctx->stream>>>(index->sa40, reinterpret_cast<const u64*>(itv), q, max_pos,
                                                                               reinterpret_cast<u64*>(pos), cnt);
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

extern "C" int csa_certify(csa_ctx* ctx, const csa_index* index, const uint64_t* off, const uint16_t* sym, uint64_t q, const uint64_t* itv,
                           uint64_t* result)
{
    CSA_TRY(check_index(ctx, index));
    if(!result) return csa_fail(ctx, CSA_E_INVALID, "csa_certify: null result");
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    const u64 init[2] = {0, ~0ull};
    CSA_CUDA(ctx, cudaMemcpyAsync(result, init, sizeof(init), cudaMemcpyHostToDevice, ctx->stream));
    CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if(q == 0) return CSA_OK;
    if(!off || !itv) return csa_fail(ctx, CSA_E_INVALID, "csa_certify: null buffer");
    certify_kernel<<<unsigned(div_up(q, 128)), 128, 0, ctx->stream>>>(*index, reinterpret_cast<const u64*>(off), sym, q,
                                                                      reinterpret_cast<const u64*>(itv), reinterpret_cast<u64*>(result));
    CSA_LAUNCH_CHECK(ctx);
    return CSA_OK;
}

namespace
{

__global__ void add_base_kernel(u64* __restrict__ off, const u64 count, const u64 base)
{
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if(i < count) off[i] += base;
}

constexpr u64 HOST_CHUNK_QUERIES = u64(1) << 18;     // the reference's chunk of a host batch (include/Query_Engine.hpp:94-100)

// Device buffers of one lane of the host-batch pipeline.
struct Lane_Buffers
{
    u64* off; u16* sym; u64* itv; u32* cnt; u64* poff; u64* sums; u64* pos;
};

}   // namespace

// The host batch runs as chunks of 2^18 queries over three streams, as Query_Engine::find does (src/Query_Engine.cu:1355-1516):
// while one chunk's results cross PCIe to the host, the next chunk's search runs and the one after is on its way in. A
// chunk's positions are copied out once the host knows how many there are, one chunk behind the searches.
extern "C" int csa_query_host(csa_ctx* ctx, const csa_index* index, const uint64_t* off_host, const uint16_t* sym_host, uint64_t q, uint32_t max_pos,
                              uint64_t* itv_host, uint32_t* cnt_host, uint64_t* pos_off_host, uint64_t* pos_host, uint64_t pos_capacity,
                              uint64_t* pos_total)
{
    CSA_TRY(check_index(ctx, index));
    if(pos_total) *pos_total = 0;
    if(q == 0) return CSA_OK;
    if(!off_host || !itv_host) return csa_fail(ctx, CSA_E_INVALID, "csa_query_host: null buffer");
    const bool want_pos = max_pos > 0 && pos_host && cnt_host && pos_off_host;
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    CSA_TRY(csa_lanes(ctx));
    // With the suffix array in host memory the search itself uses the context's one window buffer: one lane then.
    cudaPointerAttributes attr;
    const bool sa_on_host = cudaPointerGetAttributes(&attr, index->sa40) == cudaSuccess && attr.type == cudaMemoryTypeHost;
    cudaGetLastError();
    const u64 chunks = div_up(q, HOST_CHUNK_QUERIES);
    const int lanes = sa_on_host ? 1 : int(chunks < u64(csa_ctx::LANES) ? chunks : u64(csa_ctx::LANES));
    const u64 cq_max = q < HOST_CHUNK_QUERIES ? q : HOST_CHUNK_QUERIES;
    u64 sym_max = 0;
    for(u64 c = 0; c < chunks; ++c)
    {
        const u64 first = c * HOST_CHUNK_QUERIES, cq = (q - first < HOST_CHUNK_QUERIES ? q - first : HOST_CHUNK_QUERIES);
        if(off_host[first + cq] < off_host[first]) return csa_fail(ctx, CSA_E_INVALID, "csa_query_host: offsets must not decrease");
        const u64 sc = off_host[first + cq] - off_host[first];
        if(sc > sym_max) sym_max = sc;
    }
    const size_t b_off = align_up256((cq_max + 1) * 8), b_sym = align_up256(sym_max * 2 + 16), b_itv = align_up256(cq_max * 16), b_cnt = align_up256(cq_max * 4),
                 b_poff = align_up256((cq_max + 1) * 8), b_sums = align_up256((div_up(cq_max, SCAN_TILE) + 1) * 8),
                 b_pos = want_pos ? align_up256(size_t(cq_max) * max_pos * 8) : 0;
    const size_t per_lane = b_off + b_sym + b_itv + b_cnt + b_poff + b_sums + b_pos;
    void* ws = nullptr;
    CSA_TRY(csa_arena(ctx, per_lane * lanes + 4096, &ws));
    Lane_Buffers L[csa_ctx::LANES];
    for(int l = 0; l < lanes; ++l)
    {
        u8* p = static_cast<u8*>(ws) + per_lane * l;
        L[l].off = reinterpret_cast<u64*>(p); p += b_off;
        L[l].sym = reinterpret_cast<u16*>(p); p += b_sym;
        L[l].itv = reinterpret_cast<u64*>(p); p += b_itv;
        L[l].cnt = reinterpret_cast<u32*>(p); p += b_cnt;
        L[l].poff = reinterpret_cast<u64*>(p); p += b_poff;
        L[l].sums = reinterpret_cast<u64*>(p); p += b_sums;
        L[l].pos = reinterpret_cast<u64*>(p);
    }
    CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));       // whatever the caller queued on the context's own stream comes first

    // search of chunk c: batch in, intervals out, counts, offsets inside the chunk, positions packed in the lane's buffer
    auto search = [&](u64 c) -> int
    {
        const int l = int(c % u64(lanes));
        const u64 first = c * HOST_CHUNK_QUERIES, cq = (q - first < HOST_CHUNK_QUERIES ? q - first : HOST_CHUNK_QUERIES);
        const u64 sc = off_host[first + cq] - off_host[first];
        const On_Stream on(ctx, ctx->lane[l]);
        CSA_CUDA(ctx, cudaMemcpyAsync(L[l].off, off_host + first, (cq + 1) * 8, cudaMemcpyHostToDevice, ctx->stream));
        if(sc) CSA_CUDA(ctx, cudaMemcpyAsync(L[l].sym, sym_host + (off_host[first] - off_host[0]), sc * 2, cudaMemcpyHostToDevice, ctx->stream));
        CSA_TRY(csa_find(ctx, index, reinterpret_cast<uint64_t*>(L[l].off), L[l].sym, cq, reinterpret_cast<uint64_t*>(L[l].itv)));
        CSA_CUDA(ctx, cudaMemcpyAsync(itv_host + 2 * first, L[l].itv, cq * 16, cudaMemcpyDeviceToHost, ctx->stream));
        if(want_pos)
        {
            counts_kernel<<<unsigned(div_up(cq, 256)), 256, 0, ctx->stream>>>(L[l].itv, cq, max_pos, L[l].cnt);
            CSA_LAUNCH_CHECK(ctx);
            u64* total_d = ctx->d_scalars + 8 + l;
            CSA_TRY(exclusive_sum(ctx, L[l].cnt, cq, L[l].poff, L[l].sums, total_d));
            locate_packed_kernel<<<unsigned(div_up(cq * 32, 256)), 256, 0, ctx->stream>>>(index->sa40, L[l].itv, cq, max_pos, L[l].poff, L[l].pos);
            CSA_LAUNCH_CHECK(ctx);
            CSA_CUDA(ctx, cudaMemcpyAsync(ctx->h_scalars + 8 + l, total_d, 8, cudaMemcpyDeviceToHost, ctx->stream));
            CSA_CUDA(ctx, cudaMemcpyAsync(cnt_host + first, L[l].cnt, cq * 4, cudaMemcpyDeviceToHost, ctx->stream));
        }
        CSA_CUDA(ctx, cudaEventRecord(ctx->lane_event[l], ctx->stream));
        return CSA_OK;
    };
    // delivery of chunk c, once its search is over: its positions go behind those of the chunks before it
    u64 base = 0;
    bool overflow = false;
    auto deliver = [&](u64 c) -> int
    {
        if(!want_pos) return CSA_OK;
        const int l = int(c % u64(lanes));
        const u64 first = c * HOST_CHUNK_QUERIES, cq = (q - first < HOST_CHUNK_QUERIES ? q - first : HOST_CHUNK_QUERIES);
        CSA_CUDA(ctx, cudaEventSynchronize(ctx->lane_event[l]));
        const u64 total = ctx->h_scalars[8 + l];
        const On_Stream on(ctx, ctx->lane[l]);
        if(base)
        {
            add_base_kernel<<<unsigned(div_up(cq, 256)), 256, 0, ctx->stream>>>(L[l].poff, cq, base);
            CSA_LAUNCH_CHECK(ctx);
        }
        CSA_CUDA(ctx, cudaMemcpyAsync(pos_off_host + first, L[l].poff, cq * 8, cudaMemcpyDeviceToHost, ctx->stream));
        if(base + total > pos_capacity) overflow = true;
        else if(total) CSA_CUDA(ctx, cudaMemcpyAsync(pos_host + base, L[l].pos, total * 8, cudaMemcpyDeviceToHost, ctx->stream));
        base += total;
        return CSA_OK;
    };
    // With two or more lanes the delivery of a chunk is issued after the search of the next one (which runs on another lane);
    // one lane takes the chunks one by one.
    const bool pipelined = lanes >= 2;
    int rc = CSA_OK;
    for(u64 c = 0; c < chunks && rc == CSA_OK; ++c)
    {
        rc = search(c);
        if(rc != CSA_OK) break;
        if(!pipelined) rc = deliver(c);
        else if(c >= 1) rc = deliver(c - 1);
    }
    if(rc == CSA_OK && pipelined) rc = deliver(chunks - 1);
    for(int l = 0; l < lanes; ++l) cudaStreamSynchronize(ctx->lane[l]);      // on every path: the lanes' buffers are the arena's
    CSA_TRY(rc);
    if(want_pos)
    {
        pos_off_host[q] = base;
        if(pos_total) *pos_total = base;
        if(overflow) return csa_fail(ctx, CSA_E_NOMEM, "csa_query_host: the positions buffer is too small");
    }
    u64 bits = 0;
    return csa_sync(ctx, reinterpret_cast<uint64_t*>(&bits));
}
