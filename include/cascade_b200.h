/* C ABI of the B200 (sm_100a) suffix-array builder and batched query engine.
 *
 * Every entry point takes plain pointers and sizes, returns an int status (CSA_OK = 0) and never exits,
 * traps or throws. Device work is queued on the context's stream; csa_sync waits for it and reports the
 * device status word. Pointers named *_dev are device addresses on the context's device (or, where
 * stated, host memory that the device can address); pointers named *_host are ordinary host memory.
 *
 * The reference has no FFI layer: its host classes launch kernels directly. Each entry point below names
 * the reference call site (path within the reference project) whose device work it replaces.
 */
#ifndef CASCADE_B200_H
#define CASCADE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes. */
enum
{
    CSA_OK = 0,
    CSA_E_INVALID = 1,      /* a bad argument */
    CSA_E_CUDA = 2,         /* a CUDA call failed; csa_last_error has its text */
    CSA_E_NOMEM = 3,        /* device or host memory ran out, or a workspace was too small */
    CSA_E_LIMIT = 4,        /* a size beyond what the build supports (n, partition size, key bits) */
    CSA_E_DEVICE = 5,       /* the device status word is non-zero (csa_sync gives its bits) */
    CSA_E_COMM = 6          /* the multi-GPU exchange callback failed */
};

/* Symbols of zero padding that must follow the text in device memory (the reference keeps 64 bytes,
 * include/sa40.hpp:27; the tiled text-window copies here want 64 symbols). */
#define CSA_TEXT_PAD 64
/* Bytes of padding that must follow a 5-byte suffix array in memory (include/sa40.hpp:32). */
#define CSA_SA_PAD_BYTES 128
/* Symbols of a pivot / sample-table key (two 64-bit words of four u16 symbols; include/Packed_Prefix.hpp:20-34). */
#define CSA_K 8
/* Most partitions of a build (the splitters of a partition-id search are kept in shared memory). */
#define CSA_MAX_PARTITIONS 4096
/* Most GPUs of one build. */
#define CSA_MAX_GPUS 8

typedef struct csa_ctx csa_ctx;

/* ---- context ---------------------------------------------------------------------------------------- */

/* One context per (device, host thread): a stream, a status word and scratch. Replaces the per-dispatcher
 * stream and buffer set of src/GPU_SACA.cu:48-86,534-590. */
int csa_ctx_create(int device, csa_ctx** out);
void csa_ctx_destroy(csa_ctx* ctx);
/* Waits for the context's stream. If status_bits is non-null it receives the device status word; a non-zero
 * word makes the call return CSA_E_DEVICE and clears the word. Replaces synchronize_or_abort (src/utility.cpp:20-30). */
int csa_sync(csa_ctx* ctx, uint64_t* status_bits);
/* Text of the last error of this context ("" if none). The pointer stays valid until the next call on ctx. */
const char* csa_last_error(const csa_ctx* ctx);
/* The context's cudaStream_t, for callers that order their own work against it. */
void* csa_ctx_stream(csa_ctx* ctx);
/* Launches of this library's kernels on ctx since the last reset, and a reset. */
uint64_t csa_kernel_launches(const csa_ctx* ctx);
void csa_reset_counters(csa_ctx* ctx);
/* Library version string. */
const char* csa_version(void);

/* ---- LSD radix sort (replaces the cub::DeviceRadixSort::SortPairs calls of src/GPU_SACA.cu:1175,1203,1783,1849) */

/* Bytes of workspace that csa_sort_pairs needs for n records. */
size_t csa_sort_workspace_bytes(uint64_t n);
/* Stable least-significant-digit radix sort of n (64-bit key, value) records on key bits [begin_bit, end_bit),
 * 8 bits per pass, each pass one sweep over the records. val_bytes is 4 or 8. The records ping-pong between
 * (keys, vals) and (keys_alt, vals_alt); *in_alt is set to 1 if the sorted records end in the alt buffers, else 0.
 * Passes whose digit is the same for every key are skipped. With vals_dev and vals_alt_dev both null only keys are sorted. */
int csa_sort_pairs(csa_ctx* ctx, uint64_t* keys_dev, uint64_t* keys_alt_dev, void* vals_dev, void* vals_alt_dev,
                   uint32_t val_bytes, uint64_t n, int begin_bit, int end_bit, void* workspace_dev, size_t workspace_bytes,
                   int* in_alt);
/* Many segments of one record array, each sorted on its own (stable, 32-bit values or none), in one set of launches and
 * without a read-back: segment s holds the records [seg_off_host[s], seg_off_host[s + 1]) (seg_off_host[0] = 0, fewer than 2^30
 * records per segment). Every pass runs (a pass whose digit is constant inside a segment copies that segment over), so
 * *in_alt = number of passes & 1. This is how a build's generation 0 sorts all its partitions at once; it stands where the
 * reference sorts partition after partition (src/GPU_SACA.cu:1175, 1203). */
size_t csa_sort_segments_workspace_bytes(uint64_t n, uint32_t segments);
int csa_sort_segments(csa_ctx* ctx, uint64_t* keys_dev, uint64_t* keys_alt_dev, uint32_t* vals_dev, uint32_t* vals_alt_dev,
                      const uint64_t* seg_off_host, uint32_t segments, int begin_bit, int end_bit, void* workspace_dev,
                      size_t workspace_bytes, int* in_alt);
/* Most records of one csa_sort_pairs_static call. */
#define CSA_STATIC_SORT_MAX_RECORDS (1ull << 22)
/* The same sort for callers that cannot allocate device memory (no counterpart in the reference). It takes no context
 * and no workspace: its scratch is a fixed array of about 1.1 MB inside the library's device image, which each GPU that
 * loads the library holds until the process exits, so n is limited to CSA_STATIC_SORT_MAX_RECORDS (CSA_E_LIMIT beyond,
 * with a line on stderr). It calls no cudaMalloc, cudaFree or other allocating routine. Keys are 64-bit, values 32-bit;
 * every pass runs, so *in_alt = number of passes & 1. The work is queued on `stream` (a cudaStream_t, or null) of the
 * current device and the call returns after it has finished, with CSA_E_DEVICE if a bounded wait ran out.
 * The first call on each device also looks up the array's device address and sizes the kernel's shared memory. Every call
 * synchronises `stream` before it returns. All calls share the one array: calls that overlap on the GPU (two streams, two
 * threads) race on it, so keep them one after another per device. */
int csa_sort_pairs_static(void* stream, uint64_t* keys_dev, uint64_t* keys_alt_dev, uint32_t* vals_dev, uint32_t* vals_alt_dev,
                          uint64_t n, int begin_bit, int end_bit, int* in_alt);
/* Test hooks. key 0: log2 of the most records one launch of a digit pass takes (12..29, default 29); larger sorts run
 * as several launches per pass. key 2: polls after which a tile of a digit pass gives up waiting for the tile before it
 * (1..2^22, default 2^22), on the current device. key 3: 1 makes the tile numbering of csa_sort_pairs' passes start at 1,
 * so that tile 0 never comes and every wait of the pass runs out (0 restores it): the sort then returns normally, nothing
 * of the failed pass is written, and csa_sync reports CSA_E_DEVICE with bit 0 (a look-back wait ran out) in its status
 * word. No device fault is involved. key 4: an offset that stores created afterwards (csa_store_create,
 * csa_build_sa_streamed) add to every position they put into a lane and take off again when they read one, so that a small
 * text exercises lanes above 2^32; the suffix array of such a build holds position + offset. */
int csa_debug_set(int key, uint64_t value);
/* Average device time of the digit passes of the sorts run on ctx since the last csa_reset_counters, measured
 * with CUDA events on the context's stream when pass timing is on (csa_set_pass_timing): total milliseconds,
 * the passes timed, the records they moved and the algorithmic bytes of that (one read and one write of every record). */
int csa_set_pass_timing(csa_ctx* ctx, int on);
int csa_get_pass_timing(csa_ctx* ctx, double* total_ms, uint64_t* passes, uint64_t* records, uint64_t* bytes);

/* ---- build: sampling and partitioning ---------------------------------------------------------------- */

/* Packs the K-gram (CSA_K symbols, two big-endian-packed 64-bit words, zero-padded past the text's end) at
 * n_samples pseudo-random positions drawn from seed into samples_dev (2 words each, unsorted).
 * Replaces the sampling loop of GPU_SACA::select_pivots (src/GPU_SACA.cu:290-312). */
int csa_sample_kgrams(csa_ctx* ctx, const uint16_t* text_dev, uint64_t n, uint64_t n_samples, uint64_t seed,
                      uint64_t* samples_dev);
/* Host side of select_pivots (src/GPU_SACA.cu:313-364): sorts the samples and picks up to p-1 distinct pivots
 * (inclusive upper bounds) at equal strides, so that equal K-grams never split. pivots_host holds 2 (p-1)
 * words; *p_out receives the partition count actually formed (<= p). */
int csa_select_pivots(const uint64_t* samples_host, uint64_t n_samples, uint32_t p, uint64_t* pivots_host, uint32_t* p_out);
/* The same choice from samples in device memory, ordered by the device's radix sort (only runs of samples that tie on their
 * first word are put in order on the host): for samples gathered from several GPUs, whose order on the host would cost tens of
 * milliseconds at 2^19 samples. */
int csa_select_pivots_dev(csa_ctx* ctx, const uint64_t* samples_dev, uint64_t n_samples, uint32_t p, uint64_t* pivots_host, uint32_t* p_out);
/* For the positions [first, first + count) of the text: partition id = min{q : kgram(i) <= pivot[q]}, written to
 * pid_dev[i - first], and the partitions' sizes added into hist_dev[p]. Replaces compute_partition_IDs_kernel
 * (include/GPU_SACA.cuh:23-73, launched at src/GPU_SACA.cu:939). pivots_dev holds 2 (p-1) words. */
int csa_partition_ids(csa_ctx* ctx, const uint16_t* text_dev, uint64_t n, uint64_t first, uint64_t count,
                      const uint64_t* pivots_dev, uint32_t p, uint16_t* pid_dev, uint64_t* hist_dev);
/* Optional, before csa_partition_ids: from the same pivots in host memory, a table in the context that gives, for every
 * first symbol, the range of partitions a K-gram starting with it can fall into; the search of csa_partition_ids then starts
 * from that range (most symbols allow one partition only). p = 0 removes the table; pivots of another build need another call. */
int csa_install_pivots(csa_ctx* ctx, const uint64_t* pivots_host, uint32_t p);
/* Scatters the positions [first, first + count) into their partitions: position i goes to
 * part_base_dev[pid] [ cursor_dev[pid]++ ], 4 bytes each. part_base_dev holds p device pointers (they may
 * point into another GPU's memory); cursor_dev holds p running offsets. Replaces the host scatter of
 * GPU_SACA::partition (src/GPU_SACA.cu:795-826). */
int csa_scatter_by_pid(csa_ctx* ctx, const uint16_t* pid_dev, uint64_t first, uint64_t count, uint32_t p,
                       uint32_t* const* part_base_dev, uint64_t* cursor_dev);

/* ---- build: whole suffix array ------------------------------------------------------------------------ */

typedef struct csa_build_stats
{
    uint64_t n;                 /* suffixes */
    uint32_t partitions;        /* partitions formed */
    uint32_t generations;       /* doubling generations run after the initial sort */
    uint64_t max_partition;     /* largest partition, in suffixes */
    uint64_t active_after_gen0; /* suffixes still tied after the initial sort */
    uint64_t sort_passes;       /* radix digit passes run */
    uint64_t sort_records;      /* records moved by those passes */
    uint64_t kernel_launches;   /* kernels of this library launched by the build */
    uint64_t peer_bytes;        /* bytes read from or written to other GPUs' memory (multi-GPU builds) */
    double ms_partition;        /* device milliseconds by phase, from CUDA events */
    double ms_gen0;
    double ms_doubling;
    double ms_output;
    double ms_total;
    double ms_sort_passes;      /* total of the digit passes, when pass timing is on */
    uint64_t active_per_gen[48];
    uint64_t peer_bytes_per_gen[49];    /* multi-GPU builds: bytes this GPU wrote into other GPUs' memory; [0] = partition phase and
                                         * generation 0 (positions, keys, first ranks), [t] = doubling generation t (rank requests,
                                         * responses and updates) */
    uint32_t host_parts;        /* csa_build_sa_tiered: parts whose lists stayed in host memory */
    uint32_t file_parts;        /*   and parts whose lists went through files */
    uint64_t file_bytes_read;   /*   bytes read from and written to those files */
    uint64_t file_bytes_written;
} csa_build_stats;

/* Device bytes that csa_build_sa allocates for a text of n symbols in p partitions (beyond text and output). */
size_t csa_build_device_bytes(uint64_t n, uint32_t p);
/* Builds the suffix array of text_dev[0, n) (n < 2^32 - 2^26; CSA_TEXT_PAD zero symbols must follow the text)
 * into sa40_dev as 5-byte little-endian entries in numeric symbol order with shorter suffixes first
 * (5 n bytes are written; the buffer must hold 5 n + CSA_SA_PAD_BYTES). p is the number of partitions asked for
 * (K-gram splitters, CSA_K symbols); seed drives the sampling only (the suffix array does not depend on it).
 * Replaces GPU_SACA::build_SA (src/GPU_SACA.cu:124-216) for a text resident in device memory. */
int csa_build_sa(csa_ctx* ctx, const uint16_t* text_dev, uint64_t n, uint32_t p, uint64_t seed, uint8_t* sa40_dev,
                 csa_build_stats* stats);
/* The same from host buffers: copies text_host[0, n) to the device, builds, and copies the 5 n output bytes to
 * sa40_host. Pinned host buffers make the copies asynchronous and fast; pageable ones work. This is the call that
 * stands for `cascade <text> <sa>` (src/main.cu:12-46) once the files are in memory. */
int csa_build_sa_host(csa_ctx* ctx, const uint16_t* text_host, uint64_t n, uint32_t p, uint64_t seed, uint8_t* sa40_host,
                      csa_build_stats* stats);

/* ---- texts of other symbol widths ---------------------------------------------------------------------------------------- */

/* The reference instantiates its builder and its query engine for 1-, 2- and 4-byte symbols (src/GPU_SACA.cu:2400-2402,
 * src/Query_Engine.cu:1684-1686). This library's kernels take 16-bit symbols; a text of another width is first mapped onto
 * them in a way that keeps the numeric order of the symbols, hence the order of the suffixes, hence the suffix array (which
 * holds positions, not symbols): out_dev receives n symbols and CSA_TEXT_PAD zeros, ready for the builds above.
 * csa_text_from_u8: bytes widen as they are; patterns of a query widen the same way.
 * csa_text_from_u32: every symbol is replaced by its rank among the distinct symbols of the text; alphabet_dev (65536 words)
 * receives the distinct symbols in ascending order and *distinct their number; more than 65536 are refused with CSA_E_LIMIT
 * (8-byte lanes and wider keys, include/lane.hpp's IDX_LANE_BYTES = 8, are not built). A pattern maps through the same
 * alphabet; a pattern symbol that the text does not contain cannot be mapped, and such a pattern does not occur. */
int csa_text_from_u8(csa_ctx* ctx, const uint8_t* text_dev, uint64_t n, uint16_t* out_dev);
int csa_text_from_u32(csa_ctx* ctx, const uint32_t* text_dev, uint64_t n, uint16_t* out_dev, uint32_t* alphabet_dev, uint32_t* distinct);

/* ---- build, one part at a time (suffix lists in host memory, positions up to 2^40) ---------------------------------- */

/* A part is a run of whole partitions, i.e. one contiguous range of the suffix array, small enough to be ranked on the
 * device in one go (fewer than 2^31 suffixes). Its suffix list travels as 5-byte little-endian position lanes
 * (include/lane.hpp:22-26) with 4-byte ranks that are local to the part (include/bit-layout.hpp:51-68). The device keeps,
 * for the whole build, only what is indexed by text position: the text and the store of every position's rank. */
typedef struct csa_store csa_store;

typedef struct csa_part
{
    const uint8_t* lanes;   /* count lanes; device memory, or host memory (pinned makes the copies asynchronous) */
    const uint32_t* ranks;  /* the suffixes' ranks of the generation before (null at generation 0) */
    uint64_t count;         /* generation 0: the whole part; later: its still-tied suffixes, which lead the part's list */
    uint32_t part;          /* number of the part, in suffix order */
} csa_part;

typedef struct csa_part_result
{
    uint8_t* lanes;         /* count lanes, reordered: the suffixes that are still tied, in rank order, then those that retired now */
    uint32_t* ranks;        /* their new ranks inside the part (final for the retired ones) */
    uint64_t active;        /* out: how many are still tied */
    uint64_t messages;      /* out: (position, rank) messages left in the store's outbox for csa_exchange_messages */
} csa_part_result;

/* The store of one build on ctx's device: text_dev (n symbols + CSA_TEXT_PAD zeros) and pid_dev (the partition id of every
 * position, from csa_partition_ids; needed until generation 0 is over, then csa_store_drop_partition_ids lets the caller
 * free it) are borrowed; part_of_pid_host[p] gives the part of every partition (non-decreasing). The rank store (4 n bytes)
 * is allocated here unless rank_store_dev lends n words (a caller that shares the ranks between GPUs keeps them in memory that
 * its collectives can name). Part jobs of different contexts may run on one store at the same time. */
int csa_store_create(csa_ctx* ctx, const uint16_t* text_dev, uint64_t n, const uint16_t* pid_dev, const uint16_t* part_of_pid_host,
                     uint32_t p, uint32_t* rank_store_dev, csa_store** out);
void csa_store_drop_partition_ids(csa_store* store);
void csa_store_destroy(csa_store* store);
/* Empties the outbox and makes room for `messages` messages (9 bytes each): call before the part jobs of a generation >= 1
 * with the number of suffixes that are still tied over all parts. */
int csa_store_reserve_messages(csa_ctx* ctx, csa_store* store, uint64_t messages);
/* Several GPUs, one store each (every GPU holds the whole text and a replica of the rank store, and ranks the parts it
 * owns): the caller lends the outbox, `capacity` messages as three arrays (the low 32 bits of the positions, their high 8
 * bits, the ranks; all null takes it back), so that after a generation it can gather all GPUs' outboxes with its own
 * collective (NCCL over NVLink) and apply each of them to its replica with csa_store_apply_messages (queued on ctx's
 * stream); csa_store_outbox_count tells how many messages the GPU's own jobs left. Generation 0 writes the replica directly:
 * the replicas, zero before it, are then added up by the caller (every position is written by exactly one GPU). */
int csa_store_use_outbox(csa_store* store, uint32_t* pos_lo_dev, uint8_t* pos_hi_dev, uint32_t* ranks_dev, uint64_t capacity);
uint64_t csa_store_outbox_count(const csa_store* store);
int csa_store_apply_messages(csa_ctx* ctx, csa_store* store, const uint32_t* pos_lo_dev, const uint8_t* pos_hi_dev,
                             const uint32_t* ranks_dev, uint64_t count);
/* The positions [first, first + count) grouped by part, from the store's partition ids: csa_part_sizes adds the number of
 * positions of every part into hist_dev[parts]; csa_scatter_lanes writes the positions as lanes into lanes_dev, part u's from
 * lane part_first_dev[u] + cursor_dev[u] on (the cursors are advanced; the order inside a part is arbitrary; parts whose
 * part_first_dev entry is all ones are left out, so that a caller can fill a buffer with a few parts at a time). Replaces the host
 * scatter of GPU_SACA::partition (src/GPU_SACA.cu:795-826, Suffix_Buffer::add include/Suffix_Buffer.hpp:80-93) for 5-byte lanes. */
int csa_part_sizes(csa_ctx* ctx, csa_store* store, uint64_t first, uint64_t count, uint32_t parts, uint64_t* hist_dev);
int csa_scatter_lanes(csa_ctx* ctx, csa_store* store, uint64_t first, uint64_t count, const uint64_t* part_first_dev,
                      uint64_t* cursor_dev, uint8_t* lanes_dev);
/* Device bytes of ctx's scratch that a part job of `count` suffixes takes (about 63 bytes per suffix). */
size_t csa_part_workspace_bytes(uint64_t count);
/* Generation 0 of one part: sorts its suffixes by their first 3 symbols and the part of the suffix that follows those,
 * ranks them (rank = index of the group's first suffix in the sorted part), writes every rank into the store and returns
 * the list with the tied suffixes first. `active` is valid on return; the lists are complete after csa_sync(ctx).
 * in and out may name the same memory. Replaces sort_and_init_rank_and_filter (src/GPU_SACA.cu:1111-1331). */
int csa_rank_gen0(csa_ctx* ctx, csa_store* store, const csa_part* in, csa_part_result* out);
/* Generation t >= 1 of one part, h = 3 * 2^(t-1): sorts the tied suffixes by (rank, stored rank of the suffix h symbols on),
 * refines the ranks, and leaves one (position, new rank) message per suffix in the outbox; the store itself is not changed,
 * so every part of a generation reads the ranks of the generation before. Replaces sort_and_re_rank_and_filter
 * (src/GPU_SACA.cu:1714-1995) with its message emission (include/GPU_SACA.cuh:291-353). */
int csa_rank_gen(csa_ctx* ctx, csa_store* store, const csa_part* in, uint64_t h, csa_part_result* out);
/* The same jobs for a text and a rank store that are sharded by position over several GPUs (no replica of either): the GPU
 * that holds a stretch of the text makes the generation-0 keys of its positions, and second ranks are fetched from the GPUs
 * that own them, before the job runs. The reference keeps every partition's positions and inboxes apart in the same way and
 * joins them by messages (src/Partition_Backend.cpp:516-553); here the caller's collective carries them between the GPUs.
 * csa_scatter_lanes_keys: as csa_scatter_lanes over the window [first, first + count) of the text, writing beside every lane
 *   its generation-0 key (3 symbols, then the tag of the suffix 3 symbols on). text_window_dev[i] is the symbol at position
 *   first + i and pid_window_dev[i] its partition id; both must be readable 3 entries past `count` where those positions
 *   exist, and the text must read as zero past its end. The store's own text and partition ids are not read.
 * csa_rank_gen0_keys: generation 0 of a part from such keys (device memory, in the order of in->lanes). Every suffix's first
 *   rank leaves as a message in the outbox (csa_store_use_outbox); the store's rank array is not written.
 * csa_part_positions: positions_dev[i] = position of lanes[i] + add, as 64-bit words: the addresses whose ranks generation t
 *   needs (add = h). lanes may be host or device memory.
 * csa_rank_gen_ranks: generation t of a part with second_ranks_dev[i] = the stored rank of the suffix h symbols after
 *   in->lanes[i] (device memory), however the caller got it. Messages as in csa_rank_gen. */
int csa_scatter_lanes_keys(csa_ctx* ctx, csa_store* store, const uint16_t* text_window_dev, const uint16_t* pid_window_dev, uint64_t first,
                           uint64_t count, const uint64_t* part_first_dev, uint64_t* cursor_dev, uint8_t* lanes_dev, uint64_t* keys_dev);
int csa_rank_gen0_keys(csa_ctx* ctx, csa_store* store, const csa_part* in, const uint64_t* keys_dev, csa_part_result* out);
int csa_part_positions(csa_ctx* ctx, csa_store* store, const uint8_t* lanes, uint64_t count, uint64_t add, uint64_t* positions_dev);
int csa_rank_gen_ranks(csa_ctx* ctx, csa_store* store, const csa_part* in, const uint32_t* second_ranks_dev, csa_part_result* out);
/* The rank store sharded by position, one stretch of `stretch` positions per GPU (owner = position / stretch), seen from one GPU:
 * csa_bucket_by_owner: sorts count (< 2^32) positions into one run per owner, in owner order; counts_host[g] = length of owner
 *   g's run (valid on return: the call waits for the counts). payload (32-bit words that travel with the positions) and order
 *   (order_dev[j] = index in the input of the j-th entry of the runs) are optional. The order inside a run is arbitrary.
 * csa_rank_shard_read: answers_dev[i] = shard_dev[asked_dev[i] - first] for requests that arrived for this GPU's stretch
 *   [first, first + positions); a request outside it sets the range bit of the status word and reads as 0.
 * csa_rank_shard_apply: shard_dev[positions_dev[i] - first] = ranks_dev[i] for the messages that arrived for this stretch.
 * csa_unbucket: out_dev[order_dev[j]] = values_dev[j]: answers back into the order in which the requests were made.
 * csa_outbox_positions: the outbox's positions (csa_store_use_outbox keeps them as low 32 and high 8 bits) as 64-bit words. */
int csa_bucket_by_owner(csa_ctx* ctx, const uint64_t* positions_dev, const uint32_t* payload_dev, uint64_t count, uint64_t stretch, uint32_t owners,
                        uint64_t* counts_host, uint64_t* positions_out_dev, uint32_t* payload_out_dev, uint32_t* order_dev);
/* csa_order_by_address: the same runs per owner, with the addresses inside a run in ascending order of their bits
 * [begin_bit, end_bit): one digit pass of the radix sort per 8 bits. A stretch must be whole address buckets (a multiple of
 * 2^begin_bit), and end_bit must cover the highest position. The owner then reads or writes its stretch of the rank store in
 * address order, bucket by bucket, instead of at random. Positions and payload are sorted between the two buffers given for
 * each (*in_alt = 1: the result is in the alt buffers); payload_is_index fills the payload with 0, 1, 2, ... first, which
 * makes it the `order` of csa_unbucket. workspace: csa_sort_workspace_bytes(count). */
int csa_order_by_address(csa_ctx* ctx, uint64_t* positions_dev, uint64_t* positions_alt_dev, uint32_t* payload_dev, uint32_t* payload_alt_dev,
                         uint64_t count, int begin_bit, int end_bit, uint64_t stretch, uint32_t owners, int payload_is_index, uint64_t* counts_host,
                         void* workspace_dev, size_t workspace_bytes, int* in_alt);
int csa_rank_shard_read(csa_ctx* ctx, const uint32_t* shard_dev, uint64_t first, uint64_t positions, const uint64_t* asked_dev, uint64_t count,
                        uint32_t* answers_dev);
int csa_rank_shard_apply(csa_ctx* ctx, uint32_t* shard_dev, uint64_t first, uint64_t positions, const uint64_t* positions_dev, const uint32_t* ranks_dev,
                         uint64_t count);
int csa_unbucket(csa_ctx* ctx, const uint32_t* order_dev, const uint32_t* values_dev, uint64_t count, uint32_t* out_dev);
int csa_outbox_positions(csa_ctx* ctx, const uint32_t* pos_lo_dev, const uint8_t* pos_hi_dev, uint64_t count, uint64_t* positions_dev);
/* After the last part of a generation: applies the outbox to the rank store and empties it; *applied = messages applied.
 * Stands where the reference routes messages to the inboxes of their target partitions between two generations
 * (src/Partition_Backend.cpp:516-553, include/message.hpp:22-61). */
int csa_exchange_messages(csa_ctx* ctx, csa_store* store, uint64_t* applied);
/* The final order of a part: sa40_out[5 ranks[i], +5) = lanes[i] for i < count (ranks must be a permutation of [0, count)).
 * Input and output may be host or device memory and may be the same. Replaces scatter_to_rank_order
 * (src/GPU_SACA.cu:2106-2164). Complete after csa_sync(ctx). */
int csa_rank_order(csa_ctx* ctx, const uint8_t* lanes, const uint32_t* ranks, uint64_t count, uint8_t* sa40_out);
/* The whole build driven part by part, as the reference's drive_pipeline does (src/GPU_SACA.cu:1334-1608): text_host[0, n)
 * goes to the device, positions are grouped by part into sa40_host itself (5 bytes per suffix, the part's range of the output),
 * three worker threads with a context each stream the parts through csa_rank_gen0 / csa_rank_gen / csa_rank_order, and
 * sa40_host ends as the suffix array. n up to 2^40 - 1; device memory: 8 n bytes (text, rank store, partition ids until
 * generation 0 is over) + 9 bytes per tied suffix of a generation + three part workspaces; host memory: 4 n bytes pinned for
 * the ranks besides the caller's buffers. part_suffixes bounds a part's size (0: 2^27). */
int csa_build_sa_streamed(csa_ctx* ctx, const uint16_t* text_host, uint64_t n, uint32_t p, uint64_t seed, uint8_t* sa40_host,
                          uint64_t part_suffixes, csa_build_stats* stats);
/* Where the lists of csa_build_sa_tiered live. The reference plans three tiers for a partition's lists: device memory,
 * pinned host memory, files (src/GPU_SACA.cu:38-121, chosen from GPU_SACA_RAM_BUDGET and GPU_SACA_SCRATCH, include/GPU_SACA.cuh:95-118). */
typedef struct csa_tier_options
{
    uint64_t part_suffixes;     /* bound on a part's size, as in csa_build_sa_streamed (0: 2^27) */
    uint64_t host_list_bytes;   /* host memory that the parts' lists may take, 9 bytes a suffix: the parts are taken in order
                                 * while their lists fit below it, all later parts keep theirs in files. All ones: no bound */
    const char* scratch_dir;    /* an existing directory for those files, or several separated by colons (part u's files go to
                                 * directory u modulo their number); the build makes a directory of its own in each and removes
                                 * it at the end. May be null if the bound is never passed (CSA_E_NOMEM if it then is) */
    const char* output_path;    /* if not null, the suffix array is also written to this file (5 n bytes), part by part */
} csa_tier_options;
/* csa_build_sa_streamed with the lists in tiers: host memory up to a bound, files beyond it. A file part's lists are read into
 * pinned buffers of the worker that takes the part (only the tied suffixes after generation 0), processed and written
 * back, so host memory holds the host parts' lists (4 bytes a suffix for ranks, 5 more if sa40_host is null), 14 bytes per
 * suffix of the largest file part for each of the three workers, and two buffers of 5 * 2^27 bytes. sa40_host may be null
 * when output_path is given: the array then exists only in the file, as with the reference's Output_File
 * (src/GPU_SACA.cu:1404-1409). Stands where the reference's Residency_Plan and Spill_Store stand. */
int csa_build_sa_tiered(csa_ctx* ctx, const uint16_t* text_host, uint64_t n, uint32_t p, uint64_t seed, uint8_t* sa40_host,
                        const csa_tier_options* options, csa_build_stats* stats);

/* ---- validation -------------------------------------------------------------------------------------------- */

/* Exact check of a whole 5-byte suffix array in device memory against its text: every entry is below n, no entry occurs
 * twice (so the array is a permutation), and every neighbouring pair is in order: T[x] < T[y], or the symbols are equal
 * and the suffix at x + 1 ranks before the suffix at y + 1 (the empty suffix at n before all). result_dev receives four
 * words: entries out of range, duplicate entries, pairs out of order, and the lowest rank i whose pair (i - 1, i) is out
 * of order (~0 if none); the array is the suffix array exactly when the first three are zero. The work is queued on the
 * context's stream. workspace_dev holds csa_validate_workspace_bytes(n) bytes (a bit per position and a rank per
 * position: 4 bytes for n <= 2^32, else 8). Replaces test::is_correct_SA (test/end-to-end.cpp:11-80). */
size_t csa_validate_workspace_bytes(uint64_t n);
int csa_validate_sa(csa_ctx* ctx, const uint16_t* text_dev, uint64_t n, const uint8_t* sa40_dev, void* workspace_dev,
                    size_t workspace_bytes, uint64_t* result_dev);

/* ---- build on several GPUs of one box (one process per GPU) ------------------------------------------------ */

/* All-gather of `bytes` bytes per rank between the ranks' HOST buffers: recv holds world * bytes, rank r's part at
 * r * bytes. It also serves as a barrier. Returns 0 on success. The caller supplies it (torch.distributed, MPI, threads). */
typedef int (*csa_allgather_fn)(void* user, const void* send, void* recv, uint64_t bytes);
typedef struct csa_comm
{
    uint32_t rank, world;       /* world <= CSA_MAX_GPUS */
    uint32_t policy;            /* how partitions are dealt to GPUs: 0 = contiguous blocks, 1 = interleaved (q mod world) */
    csa_allgather_fn allgather;
    void* user;
} csa_comm;

/* A ready-made communicator for ranks that run on one box: the all-gather goes through a POSIX shared-memory object
 * called `name` (the same string on every rank, unique to the job; at most 48 KB per rank and call). Every rank calls
 * csa_comm_open_shm before the first build and csa_comm_close_shm after the last (one rank passes unlink_name = 1).
 * Rank 0 makes the object, replacing a leftover of the same name; the other ranks wait for it. Waits are bounded (two
 * minutes unless the environment variable CASCADE_COMM_TIMEOUT_S or csa_comm_shm_set_timeout says otherwise): a rank that
 * never arrives makes the others fail with CSA_E_COMM. */
int csa_comm_open_shm(const char* name, uint32_t rank, uint32_t world, uint32_t policy, csa_comm* out);
int csa_comm_shm_set_timeout(csa_comm* comm, double seconds);
void csa_comm_close_shm(csa_comm* comm, int unlink_name);

/* Host-side plan of a sharded build, the same on every rank: from every rank's partition sizes over its share of the
 * positions (hist_all[world][p]) the partitions' global offsets part_off[p + 1], their owners owner[p] (policy 0: contiguous
 * blocks of partitions balanced by size, so a GPU owns one contiguous slice of the suffix array; policy 1: partition q goes
 * to GPU q mod world, which also spreads the partitions that stay tied for many generations), the slot inside its owner's
 * local array at which each partition starts (local_first[p]; a GPU keeps its partitions one after another in increasing
 * order), the GPUs' totals local_count[world], and for every (rank, partition) the offset inside the partition at which
 * that rank's positions go (cursor_all[world][p]). Stands where the reference keeps every partition on its one GPU
 * (src/GPU_SACA.cu:982-985). */
int csa_plan_shards(const uint64_t* hist_all, uint32_t p, uint32_t world, uint32_t policy, uint64_t* part_off, uint32_t* owner,
                    uint64_t* local_first, uint64_t* local_count, uint64_t* cursor_all);
/* The build of csa_build_sa spread over comm->world GPUs. Every rank passes the whole text in its own device memory
 * (same n, p, seed everywhere). Whole partitions are owned by one GPU; positions travel to their partition's owner and
 * ranks to the owner of their text position in bulk copies between the GPUs' memories (CUDA IPC mappings, NVLink); the
 * ranks meet at host barriers between the steps. A rank receives the suffix-array entries of its partitions, one
 * partition after another, as 5-byte entries at sa40_dev, which must hold capacity_entries entries (CSA_E_NOMEM if too
 * few): segment k of the output holds the global ranks [seg_first[k], seg_first[k] + seg_count[k]); *seg_c segments, at
 * most p (the arrays must hold p words).
 * Replaces the host-mediated exchange of the reference (messages through RAM or files, src/Partition_Backend.cpp:516-553). */
int csa_build_sa_multi(csa_ctx* ctx, const csa_comm* comm, const uint16_t* text_dev, uint64_t n, uint32_t p, uint64_t seed,
                       uint8_t* sa40_dev, uint64_t capacity_entries, uint64_t* seg_first, uint64_t* seg_count, uint32_t* seg_c,
                       csa_build_stats* stats);

/* ---- query engine ------------------------------------------------------------------------------------- */

typedef struct csa_index
{
    const uint16_t* text;   /* n symbols + CSA_TEXT_PAD zero symbols, device memory */
    const uint8_t* sa40;    /* 5 n bytes + CSA_SA_PAD_BYTES; device memory, or pinned host memory mapped for the device */
    const uint64_t* table;  /* sample table: 2 words per sampled suffix, ceil(n / stride) entries; device memory */
    uint64_t n;             /* symbols of the text */
    uint64_t stride;
    uint64_t sa_entries;    /* entries of sa40: 0 or n for the whole suffix array, fewer for a slice of it (a shard) */
    uint64_t sa_first;      /* global rank of the slice's first entry */
} csa_index;

/* table_dev[j] = the K-gram of suffix SA[j * stride], zero-padded past the text's end, for j < ceil(n / stride).
 * Replaces Sample_Table::build / build_kernel (src/Sample_Table.cu:26-31,218-288). */
int csa_table_build(csa_ctx* ctx, const uint16_t* text_dev, uint64_t n, const uint8_t* sa40_dev, uint64_t stride,
                    uint64_t* table_dev);
/* SA intervals of q queries: query i is sym_dev[off_dev[i] - off_dev[0], ...) of length off_dev[i+1] - off_dev[i];
 * itv_dev receives {lo, hi} pairs. Semantics of ref::find_one (include/CPU_Reference.hpp:42-73). Replaces
 * Query_Engine::find_async (src/Query_Engine.cu:1314) with its rank and search kernels (:176-279, :369-418). */
int csa_find(csa_ctx* ctx, const csa_index* index, const uint64_t* off_dev, const uint16_t* sym_dev, uint64_t q,
             uint64_t* itv_dev);
/* Positions of each query: SA[lo + k] for k < min(max_pos, hi - lo), in rank order, written to row i of
 * pos_dev (q rows of max_pos words); cnt_dev[i] = the number written. The reference has no locate output
 * (include/query-file.hpp:18-19); this is the definition its intervals imply. */
int csa_locate(csa_ctx* ctx, const csa_index* index, const uint64_t* itv_dev, uint64_t q, uint32_t max_pos,
               uint64_t* pos_dev, uint32_t* cnt_dev);
/* Sharded indexes: when sa40 holds the slice [sa_first, sa_first + sa_entries) of the suffix array (the table built over that
 * slice with csa_table_build, passing the slice and its entry count as n_entries), csa_find returns for every query the
 * number of the slice's suffixes that are smaller than the pattern (lo) and the number that are not greater (hi). Summed
 * over the slices of all shards these are the global interval. csa_locate_window then writes, for a GLOBAL interval, the
 * positions whose global ranks lie in this slice into their columns of the q x max_pos rows (column k holds rank lo + k) and
 * leaves the other columns untouched; rows that all shards write into, starting from zeros, add up to the full rows.
 * The reference has one index on one GPU; sharding by SA range is this engine's. */
int csa_table_build_slice(csa_ctx* ctx, const uint16_t* text_dev, uint64_t n, const uint8_t* sa40_slice_dev, uint64_t sa_entries,
                          uint64_t stride, uint64_t* table_dev);
int csa_locate_window(csa_ctx* ctx, const csa_index* index, const uint64_t* itv_global_dev, uint64_t q, uint32_t max_pos,
                      uint64_t* pos_dev);
/* The same into one packed array, which is what should cross between GPUs (the rows are mostly empty): cnt_dev[i] =
 * min(max_pos, hi - lo), pos_off_dev[q + 1] = their exclusive sums (the same on every shard, being made from the global
 * intervals), *total_dev = their sum; this slice's share of query i's positions goes to pos_dev[pos_off[i] + k]. pos_dev must
 * hold the total (at most q max_pos words) and be zero before the first shard writes. csa_find on a slice first compares the
 * pattern with the slice's first and last suffix and answers at once when the pattern lies outside the slice's range. */
int csa_locate_window_packed(csa_ctx* ctx, const csa_index* index, const uint64_t* itv_global_dev, uint64_t q, uint32_t max_pos,
                             uint32_t* cnt_dev, uint64_t* pos_off_dev, uint64_t* pos_dev, uint64_t* total_dev);
/* Interval certificate of ref::certify (include/CPU_Reference.hpp:79-101) for every query: result_dev[0] = number
 * of failing queries, result_dev[1] = first failing query (or ~0). Replaces certify_kernel (src/Query_Engine.cu:665-686). */
int csa_certify(csa_ctx* ctx, const csa_index* index, const uint64_t* off_dev, const uint16_t* sym_dev, uint64_t q,
                const uint64_t* itv_dev, uint64_t* result_dev);
/* Count + locate from host buffers: copies the batch to the device, finds the intervals, lists up to max_pos
 * positions per query and copies the results back: itv_host {lo, hi} pairs, cnt_host[i] = positions listed for query i,
 * pos_off_host[q + 1] = their offsets into pos_host (packed, rank order), *pos_total = their number. pos_host must hold
 * pos_capacity words; CSA_E_NOMEM if that is too few (then *pos_total says how many are needed). Pass max_pos = 0 (or
 * null position buffers) for counts only. Stands for Query_Engine::find (src/Query_Engine.cu:1355). */
int csa_query_host(csa_ctx* ctx, const csa_index* index, const uint64_t* off_host, const uint16_t* sym_host, uint64_t q,
                   uint32_t max_pos, uint64_t* itv_host, uint32_t* cnt_host, uint64_t* pos_off_host, uint64_t* pos_host,
                   uint64_t pos_capacity, uint64_t* pos_total);

/* Where an index of n symbols goes, by the rules of the reference's planner (Query_Engine::plan / ::fit,
 * src/Query_Engine.cu:822-1006): the first plan that fits the budgets less their margins (a sixteenth, at least 1 GiB), with the
 * finest table stride from 32 on that the device still holds when stride is 0. Plans: 'A' text and suffix array in device
 * memory; 'B' text in device memory, suffix array in pinned host memory (brackets gathered over PCIe; strides up to 64). The
 * reference's plans C and D search on the host and are not offered. sa_tier: 0 any, 1 device, 2 pinned. plan = 0 and `why`
 * say so when nothing fits. Host code only. */
typedef struct csa_query_placement
{
    uint32_t plan, key_words;
    uint64_t stride, table_bytes, device_bytes, host_bytes;
    uint64_t device_budget, host_budget, device_margin, host_margin;
    uint64_t chunk_queries, chunk_symbols;      /* a lane's chunk of a host batch (csa_query_host runs three lanes) */
    char why[512];
} csa_query_placement;
int csa_query_plan(uint64_t n, uint64_t device_budget, uint64_t host_budget, uint64_t stride, int sa_tier, csa_query_placement* out);

/* ---- synthetic workloads (seeded; the same integers on host and device) -------------------------------- */

/* Fills text[0, n) with the Zipf corpus: separators 0xFFFF before documents of geometric length (mean mean_doc),
 * tokens drawn by inverse CDF from cdf[vocab] (64-bit thresholds). The device and host forms give the same symbols. */
int csa_gen_corpus_dev(csa_ctx* ctx, uint16_t* text_dev, uint64_t n, uint64_t seed, uint32_t mean_doc,
                       const uint64_t* cdf_dev, uint32_t vocab);
/* The symbols first .. first + count - 1 of the same corpus into text_dev[0, count): one GPU's stretch of a sharded text. */
int csa_gen_corpus_dev_window(csa_ctx* ctx, uint16_t* text_dev, uint64_t first, uint64_t count, uint64_t seed, uint32_t mean_doc,
                              const uint64_t* cdf_dev, uint32_t vocab);
int csa_gen_corpus_host(uint16_t* text_host, uint64_t first, uint64_t count, uint64_t seed, uint32_t mean_doc,
                        const uint64_t* cdf_host, uint32_t vocab);

/* A query batch with the semantics of the reference's `query gen` (src/query.cu:826-882): std::mt19937_64(seed);
 * kind 0 = substrings of text_host (length lens[rng() % len_c], place rng() % (n - len + 1)); kind 1 = random symbols
 * rng() % vocab. off_out holds q + 1 offsets, sym_out up to sym_capacity symbols (CSA_E_NOMEM if too few). Host only. */
int csa_gen_queries_host(int kind, const uint16_t* text_host, uint64_t n, uint64_t q, const uint32_t* lens, uint32_t len_c,
                         uint64_t vocab, uint64_t seed, uint64_t* off_out, uint16_t* sym_out, uint64_t sym_capacity);
/* FNV-1a-64 over the little-endian counts hi - lo of q {lo, hi} pairs: `counts_hash` of include/query-file.hpp:228-263. */
uint64_t csa_counts_hash(const uint64_t* itv_host, uint64_t q);

#ifdef __cplusplus
}
#endif

#endif
