// The build of a whole suffix array on one GPU with text and all intermediates resident in HBM:
// sample K-grams -> splitters -> partition ids -> scatter positions into partitions (each a fixed contiguous range
// of the suffix array) -> per partition: sort by the first 4 symbols and rank (generation 0) -> doubling generations
// over the suffixes that are still tied -> 5-byte output.
//
// It stands for GPU_SACA::build_SA (src/GPU_SACA.cu:124-216): select_pivots (:290), partition (:737), initial_rank
// (:1052), exponentiate_prefix (:1998) and concatenate_partitions (:2167), for a text that fits the device.
#include "common.cuh"
#include "part.cuh"
#include "sort.cuh"

#include <cstdlib>
#include <vector>

namespace
{

struct Phase_Events
{
    cudaEvent_t e[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    ~Phase_Events() { for(auto x : e) if(x) cudaEventDestroy(x); }
};

size_t align256(size_t b) { return (b + 255) & ~size_t(255); }

struct Build_Layout
{
    size_t keys, pos, head, isa, sa, sort_ws, scratch, small, upd, total;
};

Build_Layout layout_for(u64 n, u32 p)
{
    Build_Layout L;
    const u64 cap = n;
    L.keys = align256(cap * 8);
    L.pos = align256(cap * 4);
    L.head = align256(cap * 4);
    L.isa = align256(n * 4);
    L.sa = align256(n * 4 + 64);
    const size_t one = csa_sort_workspace_bytes(n), many = sort_segments_workspace_bytes(n, p ? p : 1);
    L.sort_ws = align256(one > many ? one : many);
    L.scratch = align256(div_up(n, RANK_TILE) * 3 * 4 + 256);
    L.small = align256(size_t(p) * 8) * 3 + align256(size_t(2) * p * 8) + align256(pick_splitters_scratch_bytes(size_t(1) << 19)) + align256(65536 * 4) + 4096;   // hist, cursors, bases, pivots, splitter scratch, first-symbol table
    L.upd = align256(cap * 8);     // (position, rank) updates of one step, applied to `isa` in address order
    L.total = 2 * L.keys + 2 * L.pos + L.head + L.isa + L.sa + L.sort_ws + L.scratch + L.small + L.upd + 4096;
    return L;
}

constexpr u64 MAX_SAMPLES = 1u << 19;     // 2 words each: 8 MiB

int build_core(csa_ctx* ctx, const u16* T, const u64 n, u32 p, const u64 seed, u8* sa40, csa_build_stats* stats, void* ws, size_t ws_bytes)
{
    csa_build_stats local_stats;
    csa_build_stats& st = stats ? *stats : local_stats;
    std::memset(&st, 0, sizeof(st));
    st.n = n;
    const u64 launches_before = ctx->counters[0], passes_before = ctx->counters[1], records_before = ctx->counters[2];

    Phase_Events ev;
    for(auto& x : ev.e) CSA_CUDA(ctx, cudaEventCreate(&x));
    CSA_CUDA(ctx, cudaEventRecord(ev.e[0], ctx->stream));

    const Build_Layout L = layout_for(n, p);
    Carver cv(ws, ws_bytes);
    u64* keysA = cv.take<u64>(L.keys / 8);
    u64* keysB = cv.take<u64>(L.keys / 8);
    u32* posA = cv.take<u32>(L.pos / 4);
    u32* posB = cv.take<u32>(L.pos / 4);
    u32* head = cv.take<u32>(L.head / 4);
    u32* isa = cv.take<u32>(L.isa / 4);
    u32* sa = cv.take<u32>(L.sa / 4);
    void* sort_ws = cv.take<u8>(L.sort_ws);
    u32* scratch = cv.take<u32>(L.scratch / 4);
    u64* hist = cv.take<u64>(p);
    u64* cursor = cv.take<u64>(p);
    u32** part_base = cv.take<u32*>(p);
    u64* pivots_dev = cv.take<u64>(2 * u64(p));
    void* samples_dev = cv.take<u8>(align256(pick_splitters_scratch_bytes(MAX_SAMPLES)));
    u64* upd = cv.take<u64>(L.upd / 8);
    u32* symbol_range = cv.take<u32>(65536);
    if(!cv.ok) return csa_fail(ctx, CSA_E_NOMEM, "build: workspace too small");
    u16* pid = reinterpret_cast<u16*>(keysB);      // partition ids live only until the scatter; the keys come later

    // ---- splitters ---------------------------------------------------------------------------------------
    u32 p_eff = 1;
    std::vector<u64> pivots(2 * size_t(p));
    if(p > 1)
    {
        u64 n_samples = u64(32) * p * u64(bits_for(n));
        if(n_samples > MAX_SAMPLES) n_samples = MAX_SAMPLES;
        if(n_samples < 1024) n_samples = 1024;
        CSA_TRY(pick_splitters(ctx, T, n, p, seed, n_samples, samples_dev, pick_splitters_scratch_bytes(MAX_SAMPLES), pivots.data(), &p_eff));
        if(p_eff > 1) CSA_CUDA(ctx, cudaMemcpyAsync(pivots_dev, pivots.data(), size_t(2) * (p_eff - 1) * 8, cudaMemcpyHostToDevice, ctx->stream));
    }
    st.partitions = p_eff;

    const Ties_In_Any_Order free_ties(ctx);     // from here on the sorts order suffixes whose ties the next generation resolves

    // ---- partition ids and sizes ---------------------------------------------------------------------------
    CSA_CUDA(ctx, cudaMemsetAsync(hist, 0, size_t(p_eff) * 8, ctx->stream));
    if(p_eff > 1) CSA_TRY(partition_install_symbol_ranges(ctx, pivots.data(), p_eff, symbol_range));
    const int pid_rc = csa_partition_ids(ctx, T, n, 0, n, reinterpret_cast<const uint64_t*>(pivots_dev), p_eff, pid, reinterpret_cast<uint64_t*>(hist));
    partition_install_symbol_ranges(ctx, nullptr, 0, nullptr);
    CSA_TRY(pid_rc);
    std::vector<u64> part_size(p_eff), part_off(p_eff + 1, 0);
    CSA_CUDA(ctx, cudaMemcpyAsync(part_size.data(), hist, size_t(p_eff) * 8, cudaMemcpyDeviceToHost, ctx->stream));
    CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    u64 max_part = 0;
    for(u32 q = 0; q < p_eff; ++q) { part_off[q + 1] = part_off[q] + part_size[q]; if(part_size[q] > max_part) max_part = part_size[q]; }
    if(part_off[p_eff] != n) return csa_fail(ctx, CSA_E_DEVICE, "build: partition sizes do not add up to n");
    st.max_partition = max_part;

    // ---- scatter positions into the partitions' slot ranges ------------------------------------------------
    // With up to 256 partitions the scatter also leaves every suffix's generation-0 key in the same slot of keysA.
    const bool keys_from_scatter = p_eff <= 256;
    if(keys_from_scatter)
    {
        CSA_CUDA(ctx, cudaMemcpyAsync(hist, part_off.data(), size_t(p_eff) * 8, cudaMemcpyHostToDevice, ctx->stream));
        CSA_CUDA(ctx, cudaMemsetAsync(cursor, 0, size_t(p_eff) * 8, ctx->stream));
        CSA_TRY(launch_scatter_with_keys(ctx, T, n + CSA_TEXT_PAD, pid, 0, n, p_eff, hist, cursor, sa, keysA));
    }
    else
    {
        std::vector<u32*> bases(p_eff);
        for(u32 q = 0; q < p_eff; ++q) bases[q] = sa + part_off[q];
        CSA_CUDA(ctx, cudaMemcpyAsync(part_base, bases.data(), size_t(p_eff) * sizeof(u32*), cudaMemcpyHostToDevice, ctx->stream));
        CSA_CUDA(ctx, cudaMemsetAsync(cursor, 0, size_t(p_eff) * 8, ctx->stream));
        CSA_TRY(csa_scatter_by_pid(ctx, pid, 0, n, p_eff, part_base, reinterpret_cast<uint64_t*>(cursor)));
        CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));   // `bases` must outlive the copy
    }
    CSA_CUDA(ctx, cudaEventRecord(ev.e[1], ctx->stream));

    // ---- generation 0: per partition, sort by the first 4 symbols and rank ---------------------------------
    Isa_View iv;
    std::memset(&iv, 0, sizeof(iv));
    iv.shard[0] = isa; iv.shard_size = n; iv.gpus = 1;
    const Slot_Map whole{nullptr, nullptr, 0, 0};      // one GPU: local slots are global ranks
    u64* act_count = ctx->d_scalars;       // running length of the next active list
    CSA_CUDA(ctx, cudaMemsetAsync(act_count, 0, 8, ctx->stream));
    // All partitions go through every digit pass together (one launch per pass, no read-back) unless one of them is too large
    // for the segmented sort's tile counts; CSA_GEN0_BY_PARTITION=1 asks for the one-by-one form.
    bool together = max_part < (u64(1) << 30) && n < (u64(1) << 32);
    if(const char* e = std::getenv("CSA_GEN0_BY_PARTITION")) together = together && std::atoi(e) == 0;
    if(together)
    {
        if(!keys_from_scatter) CSA_TRY(launch_keys_gen0(ctx, T, sa, n, keysA));
        int in_alt = 0;
        CSA_TRY(sort_segments(ctx, keysA, keysB, sa, posB, part_off.data(), p_eff, 0, 64, sort_ws, L.sort_ws, &in_alt));
        // Ranked as one list: the partitions follow one another in suffix order, so the whole array is in key order; a group
        // of equal keys that meets a partition's border is one group (as in a build with fewer partitions).
        CSA_TRY(launch_rank_and_compact(ctx, in_alt ? keysB : keysA, in_alt ? posB : sa, n, 64, 0, iv, whole, sa, head, posA, act_count, scratch, upd));
    }
    for(u32 q = 0; q < p_eff && !together; ++q)
    {
        const u64 S = part_size[q], first = part_off[q];
        if(S == 0) continue;
        // The partition's keys: already in its slots of keysA, or made now from its positions.
        u64* const kq = keys_from_scatter ? keysA + first : keysA;
        if(!keys_from_scatter) CSA_TRY(launch_keys_gen0(ctx, T, sa + first, S, kq));
        int in_alt = 0;
        CSA_TRY(csa_sort_pairs(ctx, reinterpret_cast<uint64_t*>(kq), reinterpret_cast<uint64_t*>(keysB), sa + first, posB, 4, S, 0, 64, sort_ws,
                               L.sort_ws, &in_alt));
        const u64* ks = in_alt ? keysB : kq;
        const u32* ps = in_alt ? posB : sa + first;
        CSA_TRY(launch_rank_and_compact(ctx, ks, ps, S, 64, u32(first), iv, whole, sa, head, posA, act_count, scratch, upd + first));
    }
    // The ranks of generation 0 reach the inverse array in address order: one keys-only digit pass, then a streaming apply.
    const int position_bits = bits_for(n - 1);
    CSA_TRY(apply_updates_in_address_order(ctx, isa, upd, keysA, n, position_bits, sort_ws, L.sort_ws, true));     // every position was ranked once
    CSA_CUDA(ctx, cudaMemcpyAsync(ctx->h_scalars, act_count, 8, cudaMemcpyDeviceToHost, ctx->stream));
    CSA_CUDA(ctx, cudaEventRecord(ev.e[2], ctx->stream));
    CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    u64 active = ctx->h_scalars[0];
    st.active_after_gen0 = active;
    const bool debug = std::getenv("CSA_DEBUG") != nullptr;
    if(debug) std::fprintf(stderr, "[csa] n=%llu partitions=%u largest=%llu active after generation 0: %llu\n", n, p_eff, max_part, active);

    // ---- doubling generations -------------------------------------------------------------------------------
    u32* pos_cur = posA; u32* pos_other = posB;
    u64 h = 4;
    u32 gen = 0;
    const int prim_bits = bits_for(n - 1) < 1 ? 1 : bits_for(n - 1);
    while(active > 0)
    {
        if(gen < 48) st.active_per_gen[gen] = active;
        const int sec_bits = bits_for(n - 1 + h);
        if(sec_bits + prim_bits > 64) return csa_fail(ctx, CSA_E_LIMIT, "build: rank pair does not fit a 64-bit key");
        CSA_TRY(launch_keys_gen(ctx, head, pos_cur, active, n, h, sec_bits, iv, keysA));
        int in_alt = 0;
        CSA_TRY(csa_sort_pairs(ctx, reinterpret_cast<uint64_t*>(keysA), reinterpret_cast<uint64_t*>(keysB), pos_cur, pos_other, 4, active, 0,
                               sec_bits + prim_bits, sort_ws, L.sort_ws, &in_alt));
        const u64* ks = in_alt ? keysB : keysA;
        u32* ps = in_alt ? pos_other : pos_cur;
        u32* pn = in_alt ? pos_cur : pos_other;
        CSA_CUDA(ctx, cudaMemsetAsync(act_count, 0, 8, ctx->stream));
        CSA_TRY(launch_rank_and_compact(ctx, ks, ps, active, sec_bits, 0, iv, whole, sa, head, pn, act_count, scratch, upd));
        CSA_TRY(apply_updates_in_address_order(ctx, isa, upd, const_cast<u64*>(ks), active, position_bits, sort_ws, L.sort_ws));
        CSA_CUDA(ctx, cudaMemcpyAsync(ctx->h_scalars, act_count, 8, cudaMemcpyDeviceToHost, ctx->stream));
        CSA_CUDA(ctx, cudaMemcpyAsync(ctx->h_scalars + 1, ctx->d_status, 8, cudaMemcpyDeviceToHost, ctx->stream));
        CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        if(ctx->h_scalars[1] != 0) { u64 b = 0; return csa_sync(ctx, reinterpret_cast<uint64_t*>(&b)); }
        if(debug) std::fprintf(stderr, "[csa] generation %u: h=%llu active %llu -> %llu (key bits %d)\n", gen + 1, h, active, ctx->h_scalars[0], sec_bits + prim_bits);
        active = ctx->h_scalars[0];
        pos_cur = pn; pos_other = ps;
        ++gen;
        if(h > (u64(1) << 40)) return csa_fail(ctx, CSA_E_DEVICE, "build: doubling did not terminate");
        h *= 2;
    }
    st.generations = gen;
    CSA_CUDA(ctx, cudaEventRecord(ev.e[3], ctx->stream));

    // ---- output ------------------------------------------------------------------------------------------------
    CSA_TRY(launch_pack_sa40(ctx, sa, n, sa40));
    CSA_CUDA(ctx, cudaEventRecord(ev.e[4], ctx->stream));
    u64 bits = 0;
    CSA_TRY(csa_sync(ctx, reinterpret_cast<uint64_t*>(&bits)));

    float ms = 0;
    cudaEventElapsedTime(&ms, ev.e[0], ev.e[1]); st.ms_partition = ms;
    cudaEventElapsedTime(&ms, ev.e[1], ev.e[2]); st.ms_gen0 = ms;
    cudaEventElapsedTime(&ms, ev.e[2], ev.e[3]); st.ms_doubling = ms;
    cudaEventElapsedTime(&ms, ev.e[3], ev.e[4]); st.ms_output = ms;
    cudaEventElapsedTime(&ms, ev.e[0], ev.e[4]); st.ms_total = ms;
    st.kernel_launches = ctx->counters[0] - launches_before;
    st.sort_passes = ctx->counters[1] - passes_before;
    st.sort_records = ctx->counters[2] - records_before;
    return CSA_OK;
}

int check_build_args(csa_ctx* ctx, const void* text, u64 n, u32 p, const void* out)
{
    if(!ctx || !text || !out) return csa_fail(ctx, CSA_E_INVALID, "build: null argument");
    if(n == 0) return csa_fail(ctx, CSA_E_INVALID, "build: empty text");
    if(p == 0 || p > CSA_MAX_PARTITIONS) return csa_fail(ctx, CSA_E_LIMIT, "build: partition count out of range");
    if(n >= (u64(1) << 32) - (u64(1) << 26)) return csa_fail(ctx, CSA_E_LIMIT, "build: this build addresses fewer than 2^32 - 2^26 suffixes per call");
    return CSA_OK;
}

}   // namespace

extern "C" size_t csa_build_device_bytes(uint64_t n, uint32_t p)
{
    return layout_for(n, p ? p : 1).total;
}

extern "C" int csa_build_sa(csa_ctx* ctx, const uint16_t* text, uint64_t n, uint32_t p, uint64_t seed, uint8_t* sa40, csa_build_stats* stats)
{
    CSA_TRY(check_build_args(ctx, text, n, p, sa40));
    if((reinterpret_cast<uintptr_t>(text) & 15) || (reinterpret_cast<uintptr_t>(sa40) & 15))
        return csa_fail(ctx, CSA_E_INVALID, "build: text and output must be 16-byte aligned");
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    const size_t bytes = layout_for(n, p).total;
    void* ws = nullptr;
    CSA_TRY(csa_arena(ctx, bytes, &ws));
    return build_core(ctx, text, n, p, seed, sa40, stats, ws, bytes);
}

extern "C" int csa_build_sa_host(csa_ctx* ctx, const uint16_t* text_host, uint64_t n, uint32_t p, uint64_t seed, uint8_t* sa40_host, csa_build_stats* stats)
{
    CSA_TRY(check_build_args(ctx, text_host, n, p, sa40_host));
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));
    const size_t core = layout_for(n, p).total;
    const size_t text_bytes = align256((n + CSA_TEXT_PAD) * 2), out_bytes = align256(5 * n + CSA_SA_PAD_BYTES);
    const size_t bytes = core + text_bytes + out_bytes;
    void* ws = nullptr;
    CSA_TRY(csa_arena(ctx, bytes, &ws));
    u8* base = static_cast<u8*>(ws);
    u16* text_dev = reinterpret_cast<u16*>(base);
    u8* out_dev = base + text_bytes;
    CSA_CUDA(ctx, cudaMemcpyAsync(text_dev, text_host, n * 2, cudaMemcpyHostToDevice, ctx->stream));
    CSA_CUDA(ctx, cudaMemsetAsync(text_dev + n, 0, CSA_TEXT_PAD * 2, ctx->stream));
    CSA_TRY(build_core(ctx, text_dev, n, p, seed, out_dev, stats, base + text_bytes + out_bytes, core));
    CSA_CUDA(ctx, cudaMemcpyAsync(sa40_host, out_dev, 5 * n, cudaMemcpyDeviceToHost, ctx->stream));
    CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return CSA_OK;
}
