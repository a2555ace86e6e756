// Internal declarations of the build's translation units.
#pragma once
#include "common.cuh"

// The inverse suffix array (rank of every text position), split by position into equal shards, one per GPU.
// A kernel reads and writes any shard through these pointers; with one GPU there is one shard.
struct Isa_View
{
    u32* shard[CSA_MAX_GPUS];
    u64 shard_size;     // positions per shard
    u32 gpus;
};

// Installs (table_dev = 65536 words) or removes (null) the first-symbol table that narrows csa_partition_ids' search on this
// context's device. It must be removed before the table's memory is reused.
int partition_install_symbol_ranges(csa_ctx* ctx, const u64* pivots_host, u32 p, u32* table_dev);

// Global rank of a local slot. A GPU's local slots hold its partitions one after another; a partition's global range starts
// at its own offset, so global = local + a per-partition difference. With segs = 0 the difference is `base` for all slots.
struct Slot_Map
{
    const u32* seg_first;   // local first slot of every local partition, ascending
    const u64* seg_delta;   // global first slot minus local first slot
    u32 segs;
    u64 base;
};

// Samples, orders and picks up to p-1 splitters on the device (ties finished on the host); the result equals
// csa_sample_kgrams + csa_select_pivots. scratch holds pick_splitters_scratch_bytes(n_samples) bytes of device memory.
size_t pick_splitters_scratch_bytes(u64 n_samples);
int pick_splitters(csa_ctx* ctx, const u16* T, u64 n, u32 p, u64 seed, u64 n_samples, void* scratch, size_t scratch_bytes, u64* pivots_host, u32* p_out);

// Scatter of positions by partition id that also writes each suffix's generation-0 key (its first 4 symbols) into the same
// slot of `keys` as its position takes in `sa`; part_off (device) holds every partition's first slot. p <= 256.
int launch_scatter_with_keys(csa_ctx* ctx, const u16* T, u64 text_limit, const u16* pid, u64 first, u64 count, u32 p, const u64* part_off, u64* cursor,
                             u32* sa, u64* keys);
// key[i] = the 4 symbols at position pos[i], packed most-significant first.
int launch_keys_gen0(csa_ctx* ctx, const u16* T, const u32* pos, u64 count, u64* keys);

// key[j] = (head[j] << sec_bits) | secondary(pos[j] + h), where secondary(x) = isa[x] + h for x < n and
// n - 1 + h - x past the end of the text (shorter suffixes first).
int launch_keys_gen(csa_ctx* ctx, const u32* head, const u32* pos, u64 count, u64 n, u64 h, int sec_bits, Isa_View isa, u64* keys);

// After a sort of `count` (key, pos) records: places every suffix in its new slot, writes its new rank into the
// inverse suffix array, and appends the suffixes that are still tied to the next active list.
//   prim_shift < 64: records are grouped by key >> prim_shift, which is the group's first local slot;
//   prim_shift = 64: all records form one group whose first local slot is fixed_head.
// `map` turns local slots into global ranks. *act_count (device) is the running length of the next list.
// scratch holds 3 words per tile of RANK_TILE records.
constexpr int RANK_BLOCK = 256, RANK_ITEMS = 8, RANK_TILE = RANK_BLOCK * RANK_ITEMS;
// If `updates` is non-null the new ranks are not written into the inverse array but listed there, record i of the sorted
// list as (position << 32) | rank, for a bulk exchange between GPUs.
int launch_rank_and_compact(csa_ctx* ctx, const u64* keys, const u32* pos, u64 count, int prim_shift, u32 fixed_head, Isa_View isa,
                            Slot_Map map, u32* sa, u32* next_head, u32* next_pos, u64* act_count, u32* scratch, u64* updates = nullptr);

// ---- bulk exchange of ranks between GPUs (exchange.cu) ----------------------------------------------------------------
// counts[g] += the records whose position (offset by h; positions at or past n are skipped) lies in shard g.
int launch_count_owners(csa_ctx* ctx, const u32* pos, const u64* packed, u64 count, u64 h, u64 n, u64 shard, u32 gpus, u64* counts);
// Requests: for record k with x = pos[k] + h < n, writes x's index inside its shard and k into the bucket of x's owner.
// cursor[g] must hold the bucket starts; they are advanced.
int launch_bucket_requests(csa_ctx* ctx, const u32* pos, u64 count, u64 h, u64 n, u64 shard, u32 gpus, u64* cursor, u32* req_out, u32* perm_out);
// count (<= CSA_MAX_GPUS) contiguous copies, of a multiple of 4 bytes each, in one launch; destinations may be peer memory.
int launch_copy_segments(csa_ctx* ctx, void* const* dst, const void* const* src, const u64* bytes, u32 count);
// resp[i] = isa_local[req[i]]
int launch_serve_requests(csa_ctx* ctx, const u32* isa_local, const u32* req, u64 count, u32* resp);
// isa_local[high 32 bits - first_position] = low 32 bits
int launch_apply_updates(csa_ctx* ctx, u32* isa_local, const u64* upd, u64 count, u64 first_position = 0);
// The same after one keys-only radix pass on the top bits of the index (positions_bits of them are in use), so that the
// writes of one stretch of the list fall into one L2-sized stretch of the array. alt holds count records; sort_ws is a
// sort workspace. Short lists are applied directly.
int apply_updates_in_address_order(csa_ctx* ctx, u32* isa_local, u64* upd, u64* alt, u64 count, int position_bits, void* sort_ws, size_t sort_ws_bytes,
                                   bool every_position_once = false);
// keys[k] = head[k] << sec_bits | (n - 1 + h - x if x = pos[k] + h >= n, else 0)
int launch_keys_init(csa_ctx* ctx, const u32* head, const u32* pos, u64 count, u64 n, u64 h, int sec_bits, u64* keys);
// keys[perm[j]] += resp[j] + h
int launch_keys_add(csa_ctx* ctx, const u32* perm, const u32* resp, u64 count, u64 h, u64* keys);

// sa40[5 r, 5 r + 5) = sa[r], little-endian, for r < count.
int launch_pack_sa40(csa_ctx* ctx, const u32* sa, u64 count, u8* sa40);
