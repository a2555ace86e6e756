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

// key[i] = the 4 symbols at position pos[i], packed most-significant first.
int launch_keys_gen0(csa_ctx* ctx, const u16* T, const u32* pos, u64 count, u64* keys);

// key[j] = (head[j] << sec_bits) | secondary(pos[j] + h), where secondary(x) = isa[x] + h for x < n and
// n - 1 + h - x past the end of the text (shorter suffixes first).
int launch_keys_gen(csa_ctx* ctx, const u32* head, const u32* pos, u64 count, u64 n, u64 h, int sec_bits, Isa_View isa, u64* keys);

// After a sort of `count` (key, pos) records: places every suffix in its new slot, writes its new rank into the
// inverse suffix array, and appends the suffixes that are still tied to the next active list.
//   prim_shift < 64: records are grouped by key >> prim_shift, which is the group's first local slot;
//   prim_shift = 64: all records form one group whose first local slot is fixed_head.
// slot_base is the global rank of local slot 0. *act_count (device) is the running length of the next list.
// scratch holds 3 words per tile of RANK_TILE records.
constexpr int RANK_BLOCK = 256, RANK_ITEMS = 8, RANK_TILE = RANK_BLOCK * RANK_ITEMS;
int launch_rank_and_compact(csa_ctx* ctx, const u64* keys, const u32* pos, u64 count, int prim_shift, u32 fixed_head, Isa_View isa,
                            u64 slot_base, u32* sa, u32* next_head, u32* next_pos, u64* act_count, u32* scratch);

// sa40[5 r, 5 r + 5) = sa[r], little-endian, for r < count.
int launch_pack_sa40(csa_ctx* ctx, const u32* sa, u64 count, u8* sa40);
