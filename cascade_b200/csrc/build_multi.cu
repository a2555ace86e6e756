// The suffix-array build spread over the GPUs of one box, one process per GPU.
//
// Sharding: a partition (a fixed contiguous range of the suffix array) is owned by one GPU for the whole build; the
// inverse array `isa` (rank of every text position) is cut into equal shards by position, one per GPU. A position
// travels to the owner of its partition as a store into the peer's memory (CUDA IPC mapping of the peer's arena, NVLink
// through NVSwitch), in runs of one partition. A rank travels to the owner of its text position as a message, as in the
// reference (include/message.hpp:22-61), but over NVLink instead of host RAM or files (src/Partition_Backend.cpp:516-553):
// every GPU buckets its (rank, position) updates by destination GPU, the buckets cross as contiguous copies into the
// destinations' inboxes, and each GPU applies its inbox to its own shard; reads of ranks take a request and a response
// leg of the same kind. Since a shard is addressed directly by position, no join by search is needed
// (join_messages_kernel, include/GPU_SACA.cuh:362-389). Fine-grained peer loads and stores into a shard of several
// gigabytes were measured to be far slower than these bulk copies, which is why ranks are not written in place.
// The ranks meet at host barriers (the caller's all-gather) between the steps. No device-side waits on peers.
#include "common.cuh"
#include "part.cuh"
#include "sort.cuh"

#include <chrono>
#include <unistd.h>
#include <cstdlib>
#include <vector>

extern "C" int csa_plan_shards(const uint64_t* hist_all, uint32_t p, uint32_t world, uint32_t policy, uint64_t* part_off, uint32_t* owner,
                               uint64_t* local_first, uint64_t* local_count, uint64_t* cursor_all)
{
    if(!hist_all || !part_off || !owner || !local_first || !local_count || !cursor_all || p == 0 || world == 0 || world > CSA_MAX_GPUS || policy > 1)
        return CSA_E_INVALID;
    part_off[0] = 0;
    for(uint32_t q = 0; q < p; ++q)
    {
        uint64_t size = 0;
        for(uint32_t g = 0; g < world; ++g) { cursor_all[uint64_t(g) * p + q] = size; size += hist_all[uint64_t(g) * p + q]; }
        part_off[q + 1] = part_off[q] + size;
    }
    const uint64_t n = part_off[p];
    if(policy == 1 && p >= world)
    {
        // Interleaved: neighbouring partitions go to different GPUs. Suffixes that start with frequent symbols stay tied
        // for longer, and they are neighbours in the suffix array, so dealing partitions round spreads the later
        // generations' work as well as the first one's.
        for(uint32_t q = 0; q < p; ++q) owner[q] = q % world;
    }
    else
    {
        // Contiguous: a partition goes to the GPU in whose equal share of the suffix array its middle falls.
        uint32_t last = 0;
        for(uint32_t q = 0; q < p; ++q)
        {
            const uint64_t mid = part_off[q] + (part_off[q + 1] - part_off[q]) / 2;
            uint32_t g = n == 0 ? 0 : uint32_t((static_cast<unsigned __int128>(mid) * world) / n);
            if(g >= world) g = world - 1;
            if(g < last) g = last;
            owner[q] = g;
            last = g;
        }
    }
    for(uint32_t g = 0; g < world; ++g) local_count[g] = 0;
    for(uint32_t q = 0; q < p; ++q)        // a GPU keeps its partitions one after another, in increasing order
    {
        local_first[q] = local_count[owner[q]];
        local_count[owner[q]] += part_off[q + 1] - part_off[q];
    }
    return CSA_OK;
}

namespace
{

struct Multi_Layout
{
    size_t keys, pos, head, isa, sa, sort_ws, scratch, pid, small, xin, resp, upd, total;
};

Multi_Layout multi_layout(u64 n_local, u64 shard, u32 p)
{
    Multi_Layout L;
    const u64 cap = n_local ? n_local : 1;
    L.keys = align_up256(cap * 8);
    L.pos = align_up256(cap * 4);
    L.head = align_up256(cap * 4);
    L.isa = align_up256(shard * 4 + 64);
    L.sa = align_up256(cap * 4 + 64);
    const size_t one = csa_sort_workspace_bytes(cap > shard ? cap : shard), many = sort_segments_workspace_bytes(cap, p);
    L.sort_ws = align_up256(one > many ? one : many);
    L.scratch = align_up256(div_up(cap, RANK_TILE) * 3 * 4 + 256);
    L.pid = 0;
    L.small = align_up256(size_t(p) * 8) * 5 + align_up256(size_t(2) * p * 8) + 4096;
    L.xin = align_up256(shard * 8 + 64);        // inbox of the bulk exchange: updates (8 bytes) or requests + responses (4 + 4)
    L.resp = align_up256(cap * 4 + 64);         // responses to this GPU's requests
    L.upd = align_up256((cap > shard ? cap : shard) * 8 + 64);   // (position, rank) updates before they are bucketed; pass buffer of the apply
    L.total = L.isa + L.sa + 2 * L.keys + 2 * L.pos + L.head + L.sort_ws + L.scratch + L.pid + L.small + L.xin + L.resp + L.upd + 4096;
    return L;
}

struct Peer_Info
{
    unsigned char handle[64];
    u64 off_isa, off_sa, off_xin, off_resp, off_keys, arena_bytes;
    u64 process, arena_address;     // ranks that are threads of one process reach one another's arenas directly
    int device;
};

// Every all-gather of the build carries a status word in front of its payload and has one fixed size, so that a rank which
// fails on its own (an allocation, a capacity check, a CUDA error) can say so in whichever all-gather its peers reach next:
// all ranks then leave the build at the same step instead of writing into, or waiting for, a rank that has gone.
constexpr size_t GATHER_PAYLOAD = size_t(CSA_MAX_PARTITIONS) * 8;
constexpr size_t GATHER_BYTES = 16 + GATHER_PAYLOAD;

struct Gather_State
{
    bool comm_failed = false;       // the caller's all-gather itself failed: the ranks can no longer meet
    bool peers_know = false;        // a non-zero status has crossed: every rank is leaving
};

int gather(csa_ctx* ctx, const csa_comm* comm, Gather_State& gs, const void* send, void* recv, u64 bytes, u64 my_status = 0)
{
    if(bytes > GATHER_PAYLOAD) return csa_fail(ctx, CSA_E_INVALID, "multi-GPU build: all-gather payload too large");
    if(my_status == 0) CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));      // a barrier: this rank's queued device work is done first
    std::vector<unsigned char> msg(GATHER_BYTES, 0), all(GATHER_BYTES * comm->world);
    std::memcpy(msg.data(), &my_status, 8);
    if(bytes) std::memcpy(msg.data() + 16, send, bytes);
    if(comm->allgather(comm->user, msg.data(), all.data(), GATHER_BYTES) != 0)
    {
        gs.comm_failed = true;
        return csa_fail(ctx, CSA_E_COMM, "the caller's all-gather failed");
    }
    for(u32 g = 0; g < comm->world; ++g)
    {
        u64 status = 0;
        std::memcpy(&status, all.data() + size_t(g) * GATHER_BYTES, 8);
        if(status != 0)
        {
            gs.peers_know = true;
            return csa_fail(ctx, g == comm->rank ? int(status) : CSA_E_COMM,
                            g == comm->rank ? ctx->err : "multi-GPU build: rank " + std::to_string(g) + " left the build with status " + std::to_string(status));
        }
    }
    if(recv) for(u32 g = 0; g < comm->world; ++g) std::memcpy(static_cast<unsigned char*>(recv) + size_t(g) * bytes, all.data() + size_t(g) * GATHER_BYTES + 16, bytes);
    return CSA_OK;
}

int barrier(csa_ctx* ctx, const csa_comm* comm, Gather_State& gs)
{
    u64 token = comm->rank, all[CSA_MAX_GPUS];
    return gather(ctx, comm, gs, &token, all, sizeof(u64));
}

int build_multi_body(csa_ctx* ctx, const csa_comm* comm, Gather_State& gs, const uint16_t* T, uint64_t n, uint32_t p, uint64_t seed, uint8_t* sa40,
                     uint64_t capacity_entries, uint64_t* seg_first, uint64_t* seg_count, uint32_t* seg_c, csa_build_stats* stats);

}   // namespace

extern "C" int csa_build_sa_multi(csa_ctx* ctx, const csa_comm* comm, const uint16_t* T, uint64_t n, uint32_t p, uint64_t seed, uint8_t* sa40,
                                  uint64_t capacity_entries, uint64_t* seg_first, uint64_t* seg_count, uint32_t* seg_c, csa_build_stats* stats)
{
    if(!ctx || !comm || !comm->allgather || !T || !sa40 || !seg_first || !seg_count || !seg_c) return csa_fail(ctx, CSA_E_INVALID, "multi-GPU build: null argument");
    if(comm->world == 0 || comm->world > CSA_MAX_GPUS || comm->rank >= comm->world) return csa_fail(ctx, CSA_E_INVALID, "multi-GPU build: bad rank or world size");
    Gather_State gs;
    int rc = build_multi_body(ctx, comm, gs, T, n, p, seed, sa40, capacity_entries, seg_first, seg_count, seg_c, stats);
    const std::string why = ctx->err;
    // A rank that failed on its own tells the others in the all-gather they reach next; then every rank, failed or not, drains
    // its stream and passes one last barrier, so that no arena is reused or freed while a peer's copy into it is in flight.
    if(rc != CSA_OK && !gs.comm_failed && !gs.peers_know) gather(ctx, comm, gs, nullptr, nullptr, 0, u64(rc));
    cudaStreamSynchronize(ctx->stream);
    if(!gs.comm_failed)
    {
        Gather_State last;
        const int brc = barrier(ctx, comm, last);
        if(rc == CSA_OK) rc = brc;
    }
    if(rc != CSA_OK && !why.empty()) ctx->err = why;
    return rc;
}

namespace
{

int build_multi_body(csa_ctx* ctx, const csa_comm* comm, Gather_State& gs, const uint16_t* T, uint64_t n, uint32_t p, uint64_t seed, uint8_t* sa40,
                     uint64_t capacity_entries, uint64_t* seg_first, uint64_t* seg_count, uint32_t* seg_c, csa_build_stats* stats)
{
    const u32 G = comm->world, me = comm->rank;
    if(n == 0 || p == 0 || p > CSA_MAX_PARTITIONS) return csa_fail(ctx, CSA_E_LIMIT, "multi-GPU build: n or partition count out of range");
    if(n >= (u64(1) << 32) - (u64(1) << 26)) return csa_fail(ctx, CSA_E_LIMIT, "multi-GPU build: this build addresses fewer than 2^32 - 2^26 suffixes");
    if((reinterpret_cast<uintptr_t>(T) & 15) || (reinterpret_cast<uintptr_t>(sa40) & 15)) return csa_fail(ctx, CSA_E_INVALID, "multi-GPU build: text and output must be 16-byte aligned");
    CSA_CUDA(ctx, cudaSetDevice(ctx->device));

    csa_build_stats local_stats;
    csa_build_stats& st = stats ? *stats : local_stats;
    std::memset(&st, 0, sizeof(st));
    st.n = n;
    const u64 launches_before = ctx->counters[0], passes_before = ctx->counters[1], records_before = ctx->counters[2];
    const bool debug = std::getenv("CSA_DEBUG") != nullptr;
    auto wall0 = std::chrono::steady_clock::now();
    auto lap = [&](const char* what)       // debug only: wall time since the last lap, after draining the stream
    {
        if(!debug) return;
        cudaStreamSynchronize(ctx->stream);
        const auto now = std::chrono::steady_clock::now();
        std::fprintf(stderr, "[csa %u/%u]   %-28s %8.2f ms\n", comm->rank, comm->world, what, std::chrono::duration<double, std::milli>(now - wall0).count());
        wall0 = now;
    };

    cudaEvent_t ev[5];
    for(auto& e : ev) CSA_CUDA(ctx, cudaEventCreate(&e));
    struct Ev_Guard { cudaEvent_t* e; ~Ev_Guard() { for(int i = 0; i < 5; ++i) cudaEventDestroy(e[i]); } } ev_guard{ev};
    CSA_CUDA(ctx, cudaEventRecord(ev[0], ctx->stream));

    // Position shards: equal, a multiple of 8 positions so that text windows start 16-byte aligned.
    // They are also whole address buckets (the top 8 bits of a position), so that a list of updates ordered by bucket is a
    // sequence of per-owner runs.
    const int position_bits = bits_for(n - 1);
    const int bucket_shift = position_bits > 8 ? position_bits - 8 : 0;
    const u64 shard_unit = (u64(1) << bucket_shift) > 8 ? (u64(1) << bucket_shift) : 8;
    const u64 shard = div_up(div_up(n, G), shard_unit) * shard_unit;
    const u64 my_first = u64(me) * shard < n ? u64(me) * shard : n;
    const u64 my_count = (my_first + shard <= n) ? shard : n - my_first;

    // ---- splitters: every rank samples the same positions of the same text, so all get the same splitters ----------
    constexpr u64 MAX_SAMPLES = 1u << 19;
    void* ws = nullptr;
    const size_t pre_bytes = align_up256(pick_splitters_scratch_bytes(MAX_SAMPLES)) + align_up256(size_t(2) * p * 8) + align_up256(size_t(p) * 8) + 4096;
    CSA_TRY(csa_arena(ctx, pre_bytes, &ws));
    // The partition ids of this rank's positions are made once, before the arena gets its final size, so they live apart.
    void* aux = nullptr;
    CSA_TRY(csa_aux(ctx, align_up256(shard * 2 + 64) + align_up256(65536 * 4), &aux));
    u16* const pid = static_cast<u16*>(aux);
    u32* const symbol_range = reinterpret_cast<u32*>(static_cast<u8*>(aux) + align_up256(shard * 2 + 64));
    u32 p_eff = 1;
    std::vector<u64> pivots(2 * size_t(p));
    std::vector<u64> my_hist(p, 0);
    {
        Carver cv(ws, ctx->arena_bytes);
        u64* samples_dev = reinterpret_cast<u64*>(cv.take<u8>(align_up256(pick_splitters_scratch_bytes(MAX_SAMPLES))));
        u64* pivots_dev = cv.take<u64>(2 * u64(p));
        u64* hist = cv.take<u64>(p);
        if(!cv.ok) return csa_fail(ctx, CSA_E_NOMEM, "multi-GPU build: arena too small");
        if(p > 1)
        {
            u64 n_samples = u64(32) * p * u64(bits_for(n));
            if(n_samples > MAX_SAMPLES) n_samples = MAX_SAMPLES;
            if(n_samples < 1024) n_samples = 1024;
            CSA_TRY(pick_splitters(ctx, T, n, p, seed, n_samples, samples_dev, pick_splitters_scratch_bytes(MAX_SAMPLES), pivots.data(), &p_eff));
            if(p_eff > 1) CSA_CUDA(ctx, cudaMemcpyAsync(pivots_dev, pivots.data(), size_t(2) * (p_eff - 1) * 8, cudaMemcpyHostToDevice, ctx->stream));
        }
        // ids and sizes of the partitions over this rank's positions
        CSA_CUDA(ctx, cudaMemsetAsync(hist, 0, size_t(p_eff) * 8, ctx->stream));
        if(p_eff > 1) CSA_TRY(partition_install_symbol_ranges(ctx, pivots.data(), p_eff, symbol_range));
        const int pid_rc = my_count ? csa_partition_ids(ctx, T, n, my_first, my_count, reinterpret_cast<const uint64_t*>(pivots_dev), p_eff, pid, reinterpret_cast<uint64_t*>(hist)) : CSA_OK;
        partition_install_symbol_ranges(ctx, nullptr, 0, nullptr);
        CSA_TRY(pid_rc);
        CSA_CUDA(ctx, cudaMemcpyAsync(my_hist.data(), hist, size_t(p_eff) * 8, cudaMemcpyDeviceToHost, ctx->stream));
        CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    }
    st.partitions = p_eff;
    lap("splitters + sizes");
    const Ties_In_Any_Order free_ties(ctx);     // from here on the sorts order suffixes whose ties the next generation resolves

    // ---- plan: the same on every rank ------------------------------------------------------------------------------
    std::vector<u64> hist_all(size_t(G) * p_eff), send_hist(my_hist.begin(), my_hist.begin() + p_eff);
    CSA_TRY(gather(ctx, comm, gs, send_hist.data(), hist_all.data(), size_t(p_eff) * 8));
    std::vector<u64> part_off(p_eff + 1), local_first(p_eff), local_count(G), cursor_all(size_t(G) * p_eff);
    std::vector<u32> owner(p_eff);
    if(csa_plan_shards(reinterpret_cast<const uint64_t*>(hist_all.data()), p_eff, G, comm->policy, reinterpret_cast<uint64_t*>(part_off.data()), owner.data(),
                       reinterpret_cast<uint64_t*>(local_first.data()), reinterpret_cast<uint64_t*>(local_count.data()),
                       reinterpret_cast<uint64_t*>(cursor_all.data())) != CSA_OK)
        return csa_fail(ctx, CSA_E_INVALID, "multi-GPU build: shard plan failed");
    if(part_off[p_eff] != n) return csa_fail(ctx, CSA_E_DEVICE, "multi-GPU build: partition sizes do not add up to n");
    const u64 n_local = local_count[me];
    u64 max_part = 0, n_local_max = 0;
    for(u32 q = 0; q < p_eff; ++q) if(part_off[q + 1] - part_off[q] > max_part) max_part = part_off[q + 1] - part_off[q];
    for(u32 g = 0; g < G; ++g) if(local_count[g] > n_local_max) n_local_max = local_count[g];
    st.max_partition = max_part;
    // This rank's slice of the suffix array: its partitions' global ranges, in the order in which they lie in its output.
    std::vector<u32> seg_first_local;
    std::vector<u64> seg_delta;
    *seg_c = 0;
    for(u32 q = 0; q < p_eff; ++q)
    {
        if(owner[q] != me) continue;
        seg_first[*seg_c] = part_off[q];
        seg_count[*seg_c] = part_off[q + 1] - part_off[q];
        ++*seg_c;
        seg_first_local.push_back(u32(local_first[q]));
        seg_delta.push_back(part_off[q] - local_first[q]);
    }
    if(n_local > capacity_entries) return csa_fail(ctx, CSA_E_NOMEM, "multi-GPU build: the output buffer holds fewer entries than this rank's slice");

    // ---- arena of the final size; peers map one another's arenas ---------------------------------------------------
    // Every rank sizes its arena for the largest slice, so the layout (and the offsets of isa and sa) is the same everywhere.
    const Multi_Layout L = multi_layout(n_local_max, shard, p_eff);
    CSA_TRY(csa_arena(ctx, L.total, &ws));
    Carver cv(ws, ctx->arena_bytes);
    u32* isa = cv.take<u32>(L.isa / 4);
    u32* sa = cv.take<u32>(L.sa / 4);
    u64* keysA = cv.take<u64>(L.keys / 8);
    u64* keysB = cv.take<u64>(L.keys / 8);
    u32* posA = cv.take<u32>(L.pos / 4);
    u32* posB = cv.take<u32>(L.pos / 4);
    u32* head = cv.take<u32>(L.head / 4);
    void* sort_ws = cv.take<u8>(L.sort_ws);
    u32* scratch = cv.take<u32>(L.scratch / 4);
    u64* hist = cv.take<u64>(p_eff);
    u64* cursor = cv.take<u64>(p_eff);
    u32** part_base = cv.take<u32*>(p_eff);
    u64* pivots_dev = cv.take<u64>(2 * u64(p_eff));
    u32* seg_first_dev = cv.take<u32>(p_eff);
    u64* seg_delta_dev = cv.take<u64>(p_eff);
    u8* xin = cv.take<u8>(L.xin);
    u32* resp_in = cv.take<u32>(L.resp / 4);
    u64* upd = cv.take<u64>(L.upd / 8);
    if(!cv.ok) return csa_fail(ctx, CSA_E_NOMEM, "multi-GPU build: arena too small");
    if(p_eff > 1) CSA_CUDA(ctx, cudaMemcpyAsync(pivots_dev, pivots.data(), size_t(2) * (p_eff - 1) * 8, cudaMemcpyHostToDevice, ctx->stream));

    Peer_Info mine;
    std::memset(&mine, 0, sizeof(mine));
    if(G > 1)
    {
        cudaIpcMemHandle_t h;
        CSA_CUDA(ctx, cudaIpcGetMemHandle(&h, ctx->arena));      // used by the ranks of other processes only
        static_assert(sizeof(h) == 64, "IPC handle size");
        std::memcpy(mine.handle, &h, 64);
    }
    mine.off_isa = reinterpret_cast<u8*>(isa) - static_cast<u8*>(ctx->arena);
    mine.off_sa = reinterpret_cast<u8*>(sa) - static_cast<u8*>(ctx->arena);
    mine.off_xin = xin - static_cast<u8*>(ctx->arena);
    mine.off_resp = reinterpret_cast<u8*>(resp_in) - static_cast<u8*>(ctx->arena);
    mine.off_keys = reinterpret_cast<u8*>(keysA) - static_cast<u8*>(ctx->arena);
    mine.arena_bytes = ctx->arena_bytes;
    mine.process = u64(getpid());
    mine.arena_address = reinterpret_cast<u64>(ctx->arena);
    mine.device = ctx->device;
    std::vector<Peer_Info> peers(G);
    CSA_TRY(gather(ctx, comm, gs, &mine, peers.data(), sizeof(Peer_Info)));
    u8* peer_arena[CSA_MAX_GPUS];
    for(u32 g = 0; g < G; ++g)
    {
        if(g == me) { peer_arena[g] = static_cast<u8*>(ctx->arena); continue; }
        if(peers[g].process == mine.process)
        {
            // a rank that is a thread of this process: its arena is addressed as it is, once peer access is on
            if(peers[g].device != ctx->device)
            {
                const cudaError_t e = cudaDeviceEnablePeerAccess(peers[g].device, 0);
                if(e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) { ctx->err = std::string("cudaDeviceEnablePeerAccess: ") + cudaGetErrorString(e); return CSA_E_CUDA; }
                cudaGetLastError();
            }
            peer_arena[g] = reinterpret_cast<u8*>(peers[g].arena_address);
            continue;
        }
        if(ctx->peer_open[g] && std::memcmp(ctx->peer_handle[g], peers[g].handle, 64) != 0)
        {
            cudaIpcCloseMemHandle(ctx->peer_base[g]);
            ctx->peer_open[g] = false;
        }
        if(!ctx->peer_open[g])
        {
            cudaIpcMemHandle_t h;
            std::memcpy(&h, peers[g].handle, 64);
            void* base = nullptr;
            CSA_CUDA(ctx, cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
            ctx->peer_base[g] = base;
            std::memcpy(ctx->peer_handle[g], peers[g].handle, 64);
            ctx->peer_open[g] = true;
        }
        peer_arena[g] = static_cast<u8*>(ctx->peer_base[g]);
    }
    lap("plan + arena + peer maps");
    Isa_View iv;
    std::memset(&iv, 0, sizeof(iv));
    iv.gpus = G; iv.shard_size = shard;
    for(u32 g = 0; g < G; ++g) iv.shard[g] = reinterpret_cast<u32*>(peer_arena[g] + peers[g].off_isa);

    // ---- bulk routes between the GPUs ---------------------------------------------------------------------------------
    // counts_dev: G words on the device; C: the all-gathered matrix, C[s * G + d] = records that GPU s sends to GPU d.
    u64* counts_dev = ctx->d_scalars + 16;
    u64* cursor_dev = ctx->d_scalars + 24;
    std::vector<u64> C(size_t(G) * G);
    u64 route_bytes = 0;
    auto exchange_counts = [&]() -> int
    {
        u64 mine_c[CSA_MAX_GPUS];
        CSA_CUDA(ctx, cudaMemcpyAsync(ctx->h_scalars + 16, counts_dev, G * 8, cudaMemcpyDeviceToHost, ctx->stream));
        CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        for(u32 g = 0; g < G; ++g) mine_c[g] = ctx->h_scalars[16 + g];
        CSA_TRY(gather(ctx, comm, gs, mine_c, C.data(), G * 8));
        u64 off = 0;
        for(u32 d = 0; d < G; ++d) { ctx->h_scalars[24 + d] = off; off += C[size_t(me) * G + d]; }
        CSA_CUDA(ctx, cudaMemcpyAsync(cursor_dev, ctx->h_scalars + 24, G * 8, cudaMemcpyHostToDevice, ctx->stream));
        return CSA_OK;
    };
    auto out_off = [&](u32 s, u32 d) { u64 o = 0; for(u32 x = 0; x < d; ++x) o += C[size_t(s) * G + x]; return o; };    // in s's bucketed buffer
    auto in_off = [&](u32 s, u32 d) { u64 o = 0; for(u32 x = 0; x < s; ++x) o += C[size_t(x) * G + d]; return o; };     // in d's inbox
    auto inbox_total = [&]() { u64 o = 0; for(u32 x = 0; x < G; ++x) o += C[size_t(x) * G + me]; return o; };
    // Routes `count` (position << 32 | rank) updates from `list` to the positions' owners and applies what arrives here.
    auto route_updates = [&](u64* list, u64 count, u64* bucketed) -> int
    {
        // One keys-only digit pass orders the updates by the top 8 bits of their position. Shards are whole buckets, so the
        // ordered list is one run per destination GPU, and inside a run the positions sweep the destination's shard once:
        // the destination applies each run as it arrived, with L2-sized locality and no pass of its own.
        int in_alt = 0;
        u64 hist_host[256];
        std::memset(hist_host, 0, sizeof(hist_host));
        if(count > 1)
        {
            CSA_TRY(csa_sort_pairs(ctx, reinterpret_cast<uint64_t*>(list), reinterpret_cast<uint64_t*>(bucketed), nullptr, nullptr, 4, count,
                                   32 + bucket_shift, 32 + position_bits, sort_ws, L.sort_ws, &in_alt));
            CSA_CUDA(ctx, cudaMemcpyAsync(hist_host, sort_workspace_histograms(sort_ws, L.sort_ws, count), sizeof(hist_host), cudaMemcpyDeviceToHost, ctx->stream));
            CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        }
        const u64* ordered = in_alt ? bucketed : list;
        u64 mine_c[CSA_MAX_GPUS];
        for(u32 g = 0; g < G; ++g) mine_c[g] = 0;
        if(count == 1)
        {
            u64 one = 0;
            CSA_CUDA(ctx, cudaMemcpyAsync(&one, list, 8, cudaMemcpyDeviceToHost, ctx->stream));
            CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            mine_c[(one >> 32) / shard] = 1;
        }
        else
        {
            const u64 buckets_per_shard = shard >> bucket_shift;
            for(u32 bkt = 0; bkt < 256; ++bkt)
            {
                if(hist_host[bkt] == 0) continue;
                const u64 g = bucket_shift ? bkt / buckets_per_shard : (u64(bkt) / shard);
                if(g >= G) return csa_fail(ctx, CSA_E_DEVICE, "multi-GPU build: an update's position lies outside the text");
                mine_c[g] += hist_host[bkt];
            }
        }
        CSA_TRY(gather(ctx, comm, gs, mine_c, C.data(), G * 8));
        if(inbox_total() > shard) return csa_fail(ctx, CSA_E_DEVICE, "multi-GPU build: more rank updates than positions in a shard");
        {
            void* dsts[CSA_MAX_GPUS]; const void* srcs[CSA_MAX_GPUS]; u64 bytes[CSA_MAX_GPUS];
            for(u32 d = 0; d < G; ++d)
            {
                const u64 c = C[size_t(me) * G + d];
                dsts[d] = reinterpret_cast<u64*>(peer_arena[d] + peers[d].off_xin) + in_off(me, d);
                srcs[d] = ordered + out_off(me, d);
                bytes[d] = c * 8;
                if(d != me) route_bytes += c * 8;
            }
            CSA_TRY(launch_copy_segments(ctx, dsts, srcs, bytes, G));
        }
        CSA_TRY(barrier(ctx, comm, gs));                                   // every inbox is complete
        CSA_TRY(launch_apply_updates(ctx, isa, reinterpret_cast<const u64*>(xin), inbox_total(), u64(me) * shard));
        return CSA_OK;
    };
    // Builds keys[k] = head[k] << sec_bits | secondary(pos[k] + h) for the active list, fetching the ranks from their owners.
    auto route_keys = [&](const u32* heads, const u32* poss, u64 count, u64 h, int sec_bits, u64* keys, u32* req_out, u32* perm) -> int
    {
        CSA_CUDA(ctx, cudaMemsetAsync(counts_dev, 0, G * 8, ctx->stream));
        CSA_TRY(launch_count_owners(ctx, poss, nullptr, count, h, n, shard, G, counts_dev));
        CSA_TRY(exchange_counts());             // also: every GPU has applied the updates of the step before
        if(inbox_total() > shard) return csa_fail(ctx, CSA_E_DEVICE, "multi-GPU build: more rank requests than positions in a shard");
        CSA_TRY(launch_bucket_requests(ctx, poss, count, h, n, shard, G, cursor_dev, req_out, perm));
        u32* const req_in = reinterpret_cast<u32*>(xin);
        u32* const resp_out = req_in + shard;
        {
            void* dsts[CSA_MAX_GPUS]; const void* srcs[CSA_MAX_GPUS]; u64 bytes[CSA_MAX_GPUS];
            for(u32 d = 0; d < G; ++d)
            {
                const u64 c = C[size_t(me) * G + d];
                dsts[d] = reinterpret_cast<u32*>(peer_arena[d] + peers[d].off_xin) + in_off(me, d);
                srcs[d] = req_out + out_off(me, d);
                bytes[d] = c * 4;
                if(d != me) route_bytes += c * 4;
            }
            CSA_TRY(launch_copy_segments(ctx, dsts, srcs, bytes, G));
        }
        CSA_TRY(barrier(ctx, comm, gs));                                   // every request has arrived
        CSA_TRY(launch_serve_requests(ctx, isa, req_in, inbox_total(), resp_out));
        {
            void* dsts[CSA_MAX_GPUS]; const void* srcs[CSA_MAX_GPUS]; u64 bytes[CSA_MAX_GPUS];
            for(u32 s2 = 0; s2 < G; ++s2)
            {
                const u64 c = C[size_t(s2) * G + me];
                dsts[s2] = reinterpret_cast<u32*>(peer_arena[s2] + peers[s2].off_resp) + out_off(s2, me);
                srcs[s2] = resp_out + in_off(s2, me);
                bytes[s2] = c * 4;
                if(s2 != me) route_bytes += c * 4;
            }
            CSA_TRY(launch_copy_segments(ctx, dsts, srcs, bytes, G));
        }
        CSA_TRY(launch_keys_init(ctx, heads, poss, count, n, h, sec_bits, keys));
        CSA_TRY(barrier(ctx, comm, gs));                                   // every response has arrived
        u64 asked = 0;
        for(u32 d = 0; d < G; ++d) asked += C[size_t(me) * G + d];
        CSA_TRY(launch_keys_add(ctx, perm, resp_in, asked, h, keys));
        return CSA_OK;
    };

    // ---- partition ids of this rank's positions, then the scatter to the partitions' owners ------------------------
    u64 peer_bytes = 0;
    const bool keys_travel = p_eff <= 256;
    {
        // Positions are first grouped by partition in a local buffer (one run per partition), then every run crosses to the
        // partition's owner as one contiguous copy: long coalesced transfers instead of scattered peer stores.
        u32* const local = reinterpret_cast<u32*>(upd);
        std::vector<u32*> bases(p_eff);
        std::vector<u64> local_off(p_eff + 1, 0);
        for(u32 q = 0; q < p_eff; ++q) { local_off[q + 1] = local_off[q] + hist_all[size_t(me) * p_eff + q]; bases[q] = local + local_off[q]; }
        CSA_CUDA(ctx, cudaMemsetAsync(cursor, 0, size_t(p_eff) * 8, ctx->stream));
        u64* const local_keys = reinterpret_cast<u64*>(xin);       // the inbox is idle until the first rank exchange
        if(keys_travel)
        {
            // The rank that scans a stretch of the text packs every suffix's generation-0 key from the text window it has in
            // shared memory anyway; (position, key) cross together, and the owner never reads the text at random.
            CSA_CUDA(ctx, cudaMemcpyAsync(hist, local_off.data(), size_t(p_eff) * 8, cudaMemcpyHostToDevice, ctx->stream));
            if(my_count) CSA_TRY(launch_scatter_with_keys(ctx, T, n + CSA_TEXT_PAD, pid, my_first, my_count, p_eff, hist, cursor, local, local_keys));
        }
        else
        {
            CSA_CUDA(ctx, cudaMemcpyAsync(part_base, bases.data(), size_t(p_eff) * sizeof(u32*), cudaMemcpyHostToDevice, ctx->stream));
            if(my_count) CSA_TRY(csa_scatter_by_pid(ctx, pid, my_first, my_count, p_eff, part_base, reinterpret_cast<uint64_t*>(cursor)));
        }
        for(u32 k = 0; k < p_eff; ++k)
        {
            const u32 q = (k + me) % p_eff;     // every rank starts with another partition, so the copies of one moment go to different GPUs
            const u64 c = hist_all[size_t(me) * p_eff + q];
            if(c == 0) continue;
            const u32 o = owner[q];
            const u64 slot = local_first[q] + cursor_all[size_t(me) * p_eff + q];
            u32* dst = reinterpret_cast<u32*>(peer_arena[o] + peers[o].off_sa) + slot;
            CSA_CUDA(ctx, cudaMemcpyAsync(dst, local + local_off[q], c * 4, cudaMemcpyDefault, ctx->stream));
            if(keys_travel)
            {
                u64* kdst = reinterpret_cast<u64*>(peer_arena[o] + peers[o].off_keys) + slot;
                CSA_CUDA(ctx, cudaMemcpyAsync(kdst, local_keys + local_off[q], c * 8, cudaMemcpyDefault, ctx->stream));
            }
            if(o != me) peer_bytes += c * (keys_travel ? 12 : 4);
        }
        CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    }
    CSA_CUDA(ctx, cudaEventRecord(ev[1], ctx->stream));
    lap("ids + scatter");
    CSA_TRY(barrier(ctx, comm, gs));        // every position has reached its owner
    lap("barrier");

    // ---- generation 0 over this rank's partitions -------------------------------------------------------------------
    u64* act_count = ctx->d_scalars;
    CSA_CUDA(ctx, cudaMemsetAsync(act_count, 0, 8, ctx->stream));
    if(!seg_delta.empty())
    {
        CSA_CUDA(ctx, cudaMemcpyAsync(seg_first_dev, seg_first_local.data(), seg_first_local.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
        CSA_CUDA(ctx, cudaMemcpyAsync(seg_delta_dev, seg_delta.data(), seg_delta.size() * 8, cudaMemcpyHostToDevice, ctx->stream));
    }
    const Slot_Map slot_map{seg_first_dev, seg_delta_dev, u32(seg_delta.size()), 0};
    // This rank's partitions are sorted together (one launch per digit pass, no read-back) and then ranked one by one: they are
    // not neighbours in the suffix array, so a group of equal keys must not run across the border of two of them.
    std::vector<u64> seg_off_local;
    for(u32 q = 0; q < p_eff; ++q) if(owner[q] == me) seg_off_local.push_back(local_first[q]);
    seg_off_local.push_back(n_local);
    const bool together = max_part < (u64(1) << 30) && n_local > 0;
    int all_in_alt = 0;
    if(together)
    {
        if(!keys_travel) CSA_TRY(launch_keys_gen0(ctx, T, sa, n_local, keysA));
        CSA_TRY(sort_segments(ctx, keysA, keysB, sa, posB, seg_off_local.data(), u32(seg_off_local.size() - 1), 0, 64, sort_ws, L.sort_ws, &all_in_alt));
    }
    for(u32 q = 0; q < p_eff; ++q)
    {
        if(owner[q] != me) continue;
        const u64 S = part_off[q + 1] - part_off[q], first = local_first[q];
        if(S == 0) continue;
        const u64* ks; const u32* ps;
        if(together) { ks = (all_in_alt ? keysB : keysA) + first; ps = (all_in_alt ? posB : sa) + first; }
        else
        {
            u64* const kq = keys_travel ? keysA + first : keysA;
            if(!keys_travel) CSA_TRY(launch_keys_gen0(ctx, T, sa + first, S, kq));
            int in_alt = 0;
            CSA_TRY(csa_sort_pairs(ctx, reinterpret_cast<uint64_t*>(kq), reinterpret_cast<uint64_t*>(keysB), sa + first, posB, 4, S, 0, 64, sort_ws,
                                   L.sort_ws, &in_alt));
            ks = in_alt ? keysB : kq;
            ps = in_alt ? posB : sa + first;
        }
        CSA_TRY(launch_rank_and_compact(ctx, ks, ps, S, 64, u32(first), iv, Slot_Map{nullptr, nullptr, 0, part_off[q] - first}, sa, head, posA, act_count, scratch, G > 1 ? upd + first : nullptr));
    }
    lap("generation 0 sorts + ranks");
    if(G > 1) CSA_TRY(route_updates(upd, n_local, keysA));      // generation 0's ranks go to the owners of their positions
    st.peer_bytes_per_gen[0] = peer_bytes + route_bytes;
    lap("generation 0 rank exchange");
    CSA_CUDA(ctx, cudaMemcpyAsync(ctx->h_scalars, act_count, 8, cudaMemcpyDeviceToHost, ctx->stream));
    CSA_CUDA(ctx, cudaEventRecord(ev[2], ctx->stream));
    CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    u64 active = ctx->h_scalars[0];
    u64 counts[CSA_MAX_GPUS];
    CSA_TRY(gather(ctx, comm, gs, &active, counts, sizeof(u64)));     // also the barrier after generation 0's rank writes
    u64 total_active = 0;
    for(u32 g = 0; g < G; ++g) total_active += counts[g];
    st.active_after_gen0 = total_active;
    if(debug) std::fprintf(stderr, "[csa %u/%u] n=%llu local=%llu partitions=%u active after generation 0: %llu (all ranks %llu)\n", me, G, (unsigned long long)n, n_local,
                           p_eff, active, total_active);

    // ---- doubling generations: all ranks run the same number of them ------------------------------------------------
    u32* pos_cur = posA; u32* pos_other = posB;
    u64 h = 4;
    u32 gen = 0;
    const int prim_bits = bits_for(n_local_max ? n_local_max - 1 : 0) < 1 ? 1 : bits_for(n_local_max - 1);
    while(total_active > 0)
    {
        if(gen < 48) st.active_per_gen[gen] = total_active;
        const int sec_bits = bits_for(n - 1 + h);
        if(sec_bits + prim_bits > 64) return csa_fail(ctx, CSA_E_LIMIT, "multi-GPU build: rank pair does not fit a 64-bit key");
        if(G > 1) CSA_TRY(route_keys(head, pos_cur, active, h, sec_bits, keysA, reinterpret_cast<u32*>(keysB), reinterpret_cast<u32*>(keysB) + n_local_max));
        else CSA_TRY(launch_keys_gen(ctx, head, pos_cur, active, n, h, sec_bits, iv, keysA));
        lap("keys (rank requests)");
        int in_alt = 0;
        if(active) CSA_TRY(csa_sort_pairs(ctx, reinterpret_cast<uint64_t*>(keysA), reinterpret_cast<uint64_t*>(keysB), pos_cur, pos_other, 4, active, 0,
                                          sec_bits + prim_bits, sort_ws, L.sort_ws, &in_alt));
        const u64* ks = in_alt ? keysB : keysA;
        u32* ps = in_alt ? pos_other : pos_cur;
        u32* pn = in_alt ? pos_cur : pos_other;
        CSA_CUDA(ctx, cudaMemsetAsync(act_count, 0, 8, ctx->stream));
        CSA_TRY(launch_rank_and_compact(ctx, ks, ps, active, sec_bits, 0, iv, slot_map, sa, head, pn, act_count, scratch, G > 1 ? upd : nullptr));
        lap("sort + ranks");
        if(G > 1) CSA_TRY(route_updates(upd, active, const_cast<u64*>(ks)));
        lap("rank exchange");     // the sorted keys are spent: their buffer holds the buckets
        CSA_CUDA(ctx, cudaMemcpyAsync(ctx->h_scalars, act_count, 8, cudaMemcpyDeviceToHost, ctx->stream));
        CSA_CUDA(ctx, cudaMemcpyAsync(ctx->h_scalars + 1, ctx->d_status, 8, cudaMemcpyDeviceToHost, ctx->stream));
        CSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        u64 mine2[2] = {ctx->h_scalars[0], ctx->h_scalars[1]}, all2[2 * CSA_MAX_GPUS];
        CSA_TRY(gather(ctx, comm, gs, mine2, all2, sizeof(mine2)));    // the barrier after this generation's rank writes
        u64 next_total = 0, any_status = 0;
        for(u32 g = 0; g < G; ++g) { next_total += all2[2 * g]; any_status |= all2[2 * g + 1]; }
        if(any_status != 0) { u64 b = 0; csa_sync(ctx, reinterpret_cast<uint64_t*>(&b)); return csa_fail(ctx, CSA_E_DEVICE, "multi-GPU build: a rank reported a device status"); }
        if(debug) std::fprintf(stderr, "[csa %u/%u] generation %u: h=%llu active %llu -> %llu (all ranks %llu)\n", me, G, gen + 1, h, active, mine2[0], next_total);
        if(gen + 1 < 49)
        {
            u64 before = 0;
            for(u32 g2 = 0; g2 <= gen && g2 < 49; ++g2) before += st.peer_bytes_per_gen[g2];
            st.peer_bytes_per_gen[gen + 1] = peer_bytes + route_bytes - before;
        }
        active = mine2[0];
        total_active = next_total;
        pos_cur = pn; pos_other = ps;
        ++gen;
        if(h > (u64(1) << 40)) return csa_fail(ctx, CSA_E_DEVICE, "multi-GPU build: doubling did not terminate");
        h *= 2;
    }
    st.generations = gen;
    CSA_CUDA(ctx, cudaEventRecord(ev[3], ctx->stream));

    // ---- this rank's slice of the output ------------------------------------------------------------------------------
    CSA_TRY(launch_pack_sa40(ctx, sa, n_local, sa40));
    CSA_CUDA(ctx, cudaEventRecord(ev[4], ctx->stream));
    u64 bits = 0;
    CSA_TRY(csa_sync(ctx, reinterpret_cast<uint64_t*>(&bits)));     // the caller of this body passes the last barrier

    float ms = 0;
    cudaEventElapsedTime(&ms, ev[0], ev[1]); st.ms_partition = ms;
    cudaEventElapsedTime(&ms, ev[1], ev[2]); st.ms_gen0 = ms;
    cudaEventElapsedTime(&ms, ev[2], ev[3]); st.ms_doubling = ms;
    cudaEventElapsedTime(&ms, ev[3], ev[4]); st.ms_output = ms;
    cudaEventElapsedTime(&ms, ev[0], ev[4]); st.ms_total = ms;
    st.kernel_launches = ctx->counters[0] - launches_before;
    st.sort_passes = ctx->counters[1] - passes_before;
    st.sort_records = ctx->counters[2] - records_before;
    st.peer_bytes = peer_bytes + route_bytes;
    return CSA_OK;
}

}   // namespace
