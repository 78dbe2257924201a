/*
 * doksparse.h -- C ABI of libdoksparse.so: the batched closed-hashing map of DeMoriarty/DOKSparse
 * (sparse_dok 0.1.9.2) and the DOK tensor paths built on it, as hand-written CUDA for sm_100a.
 *
 * The reference has no FFI of its own: its native boundary is a CuPy RawKernel launch with raw
 * data_ptr() integers (sparse_dok/components/cuda/closed_hashmap_impl.py:123-143).  Every entry
 * point below names the reference launcher / kernel it replaces.  All pointers are DEVICE pointers
 * unless a parameter says "host"; `stream` is a cudaStream_t passed as void*.  Nothing here
 * allocates device memory, synchronises the stream, or throws: every call returns a dok_status.
 *
 * Key identity is the reference's 64-bit "uuid" (second hash), not the key bytes
 * (closed_hashmap_impl_class.cu:280-312, 368-427, 459-484).  The uuid is reproduced bit for bit;
 * the start slot is free (the slot layout is not part of the contract) and is derived from the uuid
 * and the first-hash parameters with a 64-bit mixer.
 *
 * Storage of a table (owned by the caller, 128-byte aligned, sized by dok_table_layout): n_slots slots of
 * slot_bytes (32, 64, 128, or a larger multiple of 128 for very wide rows):
 *     { int64 tag | value (padded to 8) | key row (padded to 8) | int64 stamp (if it fits without growing the slot) }
 * at the offsets dok_table_layout reports (value_offset is always 8, key_offset = 8 + padded value bytes, stamp_offset
 * behind the key row or -1).
 * tag = uuid, -1 empty, -3 tombstone, -2 blocked padding slot (slots n_buckets .. n_slots-1).  These are the
 * reference's _uuid, _values and _keys arrays interleaved.  On B200 every access instruction that touches a table
 * much larger than L2 costs the same, whatever it moves, while lanes that fall into one 128-byte line share the
 * cost; so an operation's tag, value and key sit in one line, a line is a probe group of 4 / 2 / 1 slots, and four
 * adjacent lanes read a group with one request.
 *   stamp : separate n_slots int64 array, zero-initialised; needed by dok_map_set / dok_dok_set_dense only when
 *           the layout reports stamp_offset == -1 (no room in the slot); NULL otherwise.
 */
#ifndef DOKSPARSE_H
#define DOKSPARSE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DOK_MAX_KEY_SIZE 8      /* key elements per row */
#define DOK_MAX_VALUE_BYTES 248 /* value bytes per row  */
#define DOK_MAX_SELECTOR_NDIM 8 /* dims of a broadcast selector shape */
#define DOK_MAX_SHARDS 64

#define DOK_TAG_EMPTY (-1LL)   /* cuda_closed_hashmap.py:36 */
#define DOK_TAG_REMOVED (-3LL) /* cuda_closed_hashmap.py:37 */

typedef enum dok_status {
  DOK_OK = 0,
  DOK_BAD_ARG = 1,       /* null pointer, size out of range, unsupported width */
  DOK_CUDA_ERROR = 2,    /* a launch failed; dok_last_cuda_error() has the code */
  DOK_TOO_LARGE = 3      /* request exceeds a fixed capacity (static scratch) */
} dok_status;

/* element type codes of key rows */
typedef enum dok_dtype {
  DOK_I8 = 0, DOK_U8 = 1, DOK_I16 = 2, DOK_I32 = 3, DOK_I64 = 4,
  DOK_F16 = 5, DOK_BF16 = 6, DOK_F32 = 7, DOK_F64 = 8
} dok_dtype;

/* Hash parameters, given UNPERMUTED, as the Python object holds them (cuda_closed_hashmap.py:66-113).
 * Second hash = the uuid, the key's identity, reproduced bit for bit:
 *   uuid  = | prod_i ( ((int64)key_i * alpha2[c] + beta2[c]) % prime2[c] ) |,  c = key_perm[i],
 * wrapping int64, C remainder, value cast of key_i (closed_hashmap_impl_class.cu:98-107, parameters indexed
 * through keyPerm as in :54-63).  The first hash (:87-96) places rows in the reference; here alpha1 / beta1 only
 * feed the start slot, mix(uuid, prod_i (key_i * (alpha1[c] | 1) + beta1[c])), so that keys whose uuids collide
 * but whose first hashes differ -- which the reference tells apart -- stay apart here as well.  prime1 is not
 * used.  |prime2[c]| must be >= 2. */
typedef struct dok_hash_params {
  int32_t key_size;    /* 1..DOK_MAX_KEY_SIZE */
  int32_t key_dtype;   /* dok_dtype of the caller's key rows */
  int64_t alpha2[DOK_MAX_KEY_SIZE];
  int64_t beta2[DOK_MAX_KEY_SIZE];
  int64_t prime2[DOK_MAX_KEY_SIZE];
  int64_t alpha1[DOK_MAX_KEY_SIZE];
  int64_t beta1[DOK_MAX_KEY_SIZE];
  int64_t prime1[DOK_MAX_KEY_SIZE];
  int32_t key_perm[DOK_MAX_KEY_SIZE]; /* storage column of key element i (set_key_permuted, :144-150) */
} dok_hash_params;

typedef struct dok_table {
  void *slots;
  int64_t *stamp;      /* separate stamp array, or NULL (see above) */
  int64_t n_buckets;   /* slots visible to the caller */
  int32_t slot_bytes;  /* as reported by dok_table_layout */
  int32_t value_bytes;
  int32_t key_bytes;   /* key_size * bytes per key element */
  int32_t reserved;
} dok_table;

typedef struct dok_layout_info {
  int32_t slot_bytes;
  int32_t slots_per_group; /* slots per 128-byte probe group (1 for slots wider than 128 bytes) */
  int32_t value_offset;    /* offsets inside a slot */
  int32_t key_offset;
  int32_t stamp_offset;    /* -1: the stamps need a separate array */
  int32_t reserved;
  int64_t n_slots;         /* n_buckets rounded up to whole groups */
  int64_t total_bytes;     /* n_slots * slot_bytes */
} dok_layout_info;

/* Counters written by the mutating calls (device int64[DOK_N_COUNTERS], ADDED to, not reset). */
enum {
  DOK_CNT_CLAIMED_EMPTY = 0, /* slots claimed from the empty state            */
  DOK_CNT_REUSED_REMOVED = 1,/* tombstones reused                              */
  DOK_CNT_FAILED = 2,        /* rows not stored: table full                    */
  DOK_CNT_HITS = 3,          /* rows found (get / exists / remove / overwrite) */
  DOK_CNT_DUPLICATES = 4,    /* rows of a set batch that lost to a later duplicate */
  DOK_CNT_PROBES = 5,        /* total slots inspected (only when probe counting is requested) */
  DOK_N_COUNTERS = 8
};

/* Selector view for the fused DOK kernels: ndim index tensors broadcast to one shape
 * (sparse_dok_tensor.py:220-300 produces them; sparse_dok/util.py:295-310 and
 * tensor_accessor.cu:1-121 are the reference's packing and accessor).  Strides in ELEMENTS, 0 for a
 * broadcast dim.  Element e of the row-major linearisation of `sizes` addresses
 * ptr[d][ sum_j idx_j * strides[d][j] ]. */
typedef struct dok_selectors {
  int32_t ndim;            /* number of index tensors = key_size of the DOK map */
  int32_t selector_ndim;   /* dims of the common shape, 0..DOK_MAX_SELECTOR_NDIM */
  int64_t sizes[DOK_MAX_SELECTOR_NDIM];
  const int64_t *ptr[DOK_MAX_KEY_SIZE];
  int64_t strides[DOK_MAX_KEY_SIZE][DOK_MAX_SELECTOR_NDIM];
} dok_selectors;

int dok_version(void);
int dok_last_cuda_error(void);          /* cudaError_t of the last failed launch on this thread */
int64_t dok_launch_count(void);         /* kernels launched by this library in this process so far */
/* slot geometry and allocation size for a table; DOK_BAD_ARG if the widths are unsupported */
int dok_table_layout(int value_bytes, int key_bytes, int64_t n_buckets, dok_layout_info *out);

/* Fills the tags (DOK_TAG_EMPTY, blocked for padding slots; values untouched) and zeroes the stamps.
 * Replaces `torch.zeros(n_buckets) + empty_marker`, cuda_closed_hashmap.py:40. */
int dok_map_init(const dok_table *t, void *stream);

/* uuid (and this library's start slot) of each key row.  uuid_out / slot_out may be NULL; t may be NULL when
 * slot_out is.
 * Replaces nothing on the reference's hot path; CudaClosedHashmap.get_uuid
 * (cuda_closed_hashmap.py:302-319) is the closest relative but bit-casts floats, which the kernels do not. */
int dok_map_uuid(const dok_table *t, const dok_hash_params *hp, const void *keys, int64_t n,
                 int64_t *uuid_out, int64_t *slot_out, void *stream);

/* Batched lookup.  out_values[n, value_bytes] receives the stored row on a hit and `fallback`
 * (HOST pointer to value_bytes bytes, NULL = zeros) on a miss; out_found[n] is 0/1.  counters may be NULL.
 * Replaces ClosedHashmapImplCuda.get + closed_hashmap_get (closed_hashmap_impl.py:50-145,
 * closed_hashmap_impl.cu:6-85) including the launcher's two pre-fills. */
int dok_map_get(const dok_table *t, const dok_hash_params *hp, const void *keys, int64_t n,
                void *out_values, uint8_t *out_found, const void *fallback, int64_t *counters, void *stream);

/* dok_map_get that also adds the number of slots inspected to counters[DOK_CNT_PROBES] (mean probe length
 * = probes / n); fallback is zeros.  No counterpart in the reference. */
int dok_map_get_probe_stats(const dok_table *t, const dok_hash_params *hp, const void *keys, int64_t n,
                            void *out_values, uint8_t *out_found, int64_t *counters, void *stream);

/* Insert-or-assign, ONE kernel, for batches whose rows have pairwise different uuids (rows with equal
 * uuid race: one of them wins, rows may tear).  out_stored[n] may be NULL.
 * Replaces ClosedHashmapImplCuda.set + closed_hashmap_set (closed_hashmap_impl.py:147-213,
 * closed_hashmap_impl.cu:87-156, ClosedHashmap::set closed_hashmap_impl_class.cu:368-427). */
int dok_map_set_unique(const dok_table *t, const dok_hash_params *hp, const void *keys, const void *values,
                       int64_t n, uint8_t *out_stored, int64_t *counters, void *stream);

/* Insert-or-assign for any batch: rows with equal uuid resolve to the LAST row in batch order, exactly one
 * slot per uuid, rows never torn (what a serial run of the reference kernel produces).  Two kernels: the first
 * finds or claims each row's slot, raises the slot's stamp to (epoch, row) with atomicMax and lets the first row
 * to arrive write key and value; the second runs only if the first met equal uuids, and lets each such slot's
 * last row rewrite it.  slot_scratch: device int64[n + 1], contents irrelevant.  epoch: 1..2^30-1, strictly larger
 * than any epoch used on this table since its stamps were last zeroed.  n < 2^32. */
int dok_map_set(const dok_table *t, const dok_hash_params *hp, const void *keys, const void *values,
                int64_t n, int64_t *slot_scratch, int64_t epoch, uint8_t *out_stored, int64_t *counters,
                void *stream);

/* Batched removal: the slot's tag becomes DOK_TAG_REMOVED, key/value bytes stay.  With equal uuids in the
 * batch exactly one row reports 1.  Replaces ClosedHashmapImplCuda.remove + closed_hashmap_remove
 * (closed_hashmap_impl.py:215-278, closed_hashmap_impl.cu:158-220). */
int dok_map_remove(const dok_table *t, const dok_hash_params *hp, const void *keys, int64_t n,
                   uint8_t *out_removed, int64_t *counters, void *stream);

/* counters[DOK_CNT_HITS] += number of rows present; out_flags may be NULL.
 * Replaces ClosedHashmap::exists as used by sparse_dok_count_items
 * (closed_hashmap_impl_class.cu:253-278, sparse_dok_tensor_impl.cu:3-56). */
int dok_map_count_exists(const dok_table *t, const dok_hash_params *hp, const void *keys, int64_t n,
                         uint8_t *out_flags, int64_t *counters, void *stream);

/* Number of DISTINCT uuids of the batch that are absent from the table: what `set` needs before it can
 * decide on a rehash (replaces the pre-get + `unique(dim=0)` of cuda_closed_hashmap.py:350-363 for keys
 * whose uuid is injective).  scratch_tags: device int64[scratch_slots], scratch_slots >= 2*n; it is
 * (re)initialised by the call.  Adds the count to counters[DOK_CNT_CLAIMED_EMPTY]. */
int dok_map_count_new(const dok_table *t, const dok_hash_params *hp, const void *keys, int64_t n,
                      int64_t *scratch_tags, int64_t scratch_slots, int64_t *counters, void *stream);

/* dok_map_count_new without a caller-supplied scratch buffer (no counterpart in the reference, and none among
 * the entry points above: it exists for hosts that cannot allocate).  The tag set lives in a fixed 8 MiB array
 * inside the library image, held by every GPU that loads the library.  n may not exceed
 * dok_static_scratch_max_rows() (2^19): larger batches return DOK_TOO_LARGE and launch nothing.  The first call
 * on a device resolves the array's device address; make it before any stream capture.  All calls on a device
 * share the array: each refills what it uses, and calls that overlap on the GPU race.  Never calls cudaMalloc,
 * cudaFree or another allocating routine.  Adds the count to counters[DOK_CNT_CLAIMED_EMPTY]. */
int64_t dok_static_scratch_max_rows(void);
int dok_map_count_new_static(const dok_table *t, const dok_hash_params *hp, const void *keys, int64_t n,
                             int64_t *counters, void *stream);

/* ---- sliced batches -------------------------------------------------------------------------------------
 * The same three operations on a batch that arrives as n_slices slices of slice_rows rows each (keys / values /
 * outputs are [n_slices * slice_rows] rows, slice s at row s * slice_rows), of which only the first
 * slice_counts[s] rows (device int64[n_slices]) are in use.  The counts are read ON THE DEVICE, so a caller that
 * does not know them yet -- an owner shard whose inbox other GPUs are still filling when it enqueues its work -- can
 * launch without a host synchronisation: the grid covers whole slices and blocks beyond the count leave at once.
 * Batch order (what decides "last row wins") is slice by slice.  abort_flag (device int64, may be NULL): a non-zero
 * value when the kernel runs turns the whole call into a no-op.  Outputs of unused rows are not written.
 * slot_scratch: int64[n_slices * slice_rows + 1].  No counterpart in the reference (single GPU, sizes known). */
int dok_map_get_sliced(const dok_table *t, const dok_hash_params *hp, const void *keys, int64_t n_slices,
                       int64_t slice_rows, const int64_t *slice_counts, const int64_t *abort_flag, void *out_values,
                       uint8_t *out_found, const void *fallback, int64_t *counters, void *stream);
int dok_map_set_sliced(const dok_table *t, const dok_hash_params *hp, const void *keys, const void *values,
                       int64_t n_slices, int64_t slice_rows, const int64_t *slice_counts, const int64_t *abort_flag,
                       int64_t *slot_scratch, int64_t epoch, int assume_unique, int64_t *counters, void *stream);
int dok_map_remove_sliced(const dok_table *t, const dok_hash_params *hp, const void *keys, int64_t n_slices,
                          int64_t slice_rows, const int64_t *slice_counts, const int64_t *abort_flag,
                          uint8_t *out_removed, int64_t *counters, void *stream);

/* ---- tables beyond the TLB's reach ------------------------------------------------------------------------
 * A random access into a slot array larger than what the GPU's TLB covers (64 GiB on B200) costs a page walk, and
 * the lookup rate falls to a third at 114 GB.  Every entry point above therefore works through such a table in
 * PASSES over the batch: pass w serves only the rows whose probe chain starts in the w-th window of the slot array,
 * so that one launch touches a range the TLB covers.  Results are identical to a single pass; the caller sees
 * nothing but the launch count.  A table of at most single_pass_limit bytes is served in one pass, a larger one in
 * ceil(bytes / window_bytes) windows (defaults 72 GiB and 58 GiB).  The setting is process-wide; tests use small
 * values to exercise the passes on small tables.  dok_table_passes reports the passes for a table (-1: bad table).
 * No counterpart in the reference (32-bit bucket indices keep its tables far below this size). */
int dok_set_window_bytes(int64_t single_pass_limit, int64_t window_bytes);
int dok_table_passes(const dok_table *t);

/* Live-slot compaction in slot order (replaces nonempty_mask + the boolean-mask gathers of
 * cuda_closed_hashmap.py:157-172, 233-234).  Step 1 counts per tile and scans:
 *   tile_offsets: device int64[dok_compact_tiles(n_buckets) + 1]; the last element is the live count.
 * Step 2 scatters; any of keys_out [count, key_size] (columns permuted by key_perm like keys()),
 * values_out [count, value_bytes], uuid_out [count] may be NULL.  keys_transposed != 0 writes
 * keys_out as [key_size, count] (what SparseDOKTensor.indices() returns, sparse_dok_tensor.py:156-162). */
int64_t dok_compact_tiles(int64_t n_buckets);
int dok_map_compact_count(const dok_table *t, int64_t *tile_offsets, void *stream);
int dok_map_compact_scatter(const dok_table *t, const dok_hash_params *hp, const int64_t *tile_offsets,
                            void *keys_out, int keys_transposed, void *values_out, int64_t *uuid_out,
                            void *stream);

/* ---- fused DOK tensor paths: keys are formed on the fly from broadcast selector views ---------------- */

/* Dense gather with fill: out[e] = stored value or `fallback` (HOST, NULL = zeros).
 * Replaces the stack + transpose + get of SparseDOKTensor.__getitem__ (sparse_dok_tensor.py:302-315). */
int dok_dok_get(const dok_table *t, const dok_hash_params *hp, const dok_selectors *sel,
                void *out_values, uint8_t *out_found, const void *fallback, int64_t *counters, void *stream);

/* Replaces sparse_dok_count_items (sparse_dok_tensor_impl.cu:3-56, launcher sparse_dok_tensor_impl.py:56-108). */
int dok_dok_count_exists(const dok_table *t, const dok_hash_params *hp, const dok_selectors *sel,
                         int64_t *counters, void *stream);

/* Insert-or-assign of a broadcast dense source, last selector element wins on duplicates, zeros stored.
 * src_strides in elements of value_bytes; slot_scratch int64[n + 1].  Replaces sparse_dok_set_items_dense
 * (sparse_dok_tensor_impl.cu:270-313, launcher sparse_dok_tensor_impl.py:412-474). */
int dok_dok_set_dense(const dok_table *t, const dok_hash_params *hp, const dok_selectors *sel,
                      const void *src, const int64_t *src_strides, int64_t *slot_scratch, int64_t epoch,
                      int64_t *counters, void *stream);

/* Tombstones every selected element that is present; counters[DOK_CNT_HITS] += removed.
 * Replaces sparse_dok_zero_items (sparse_dok_tensor_impl.cu:58-108). */
int dok_dok_zero_items(const dok_table *t, const dok_hash_params *hp, const dok_selectors *sel,
                       int64_t *counters, void *stream);

/* Sparse gather in one kernel (replaces sparse_dok_get_items, sparse_dok_tensor_impl.cu:110-160, launcher
 * sparse_dok_tensor_impl.py:148-232): every selected element that is stored in src is inserted into dst -- an
 * initialised table with int64 keys of max(selector_ndim, 1) elements, the same value_bytes and room for the hits --
 * under its index tuple in the selection's shape.  counters[DOK_CNT_HITS] += hits, [DOK_CNT_CLAIMED_EMPTY] += rows
 * inserted, [DOK_CNT_FAILED] += rows that found dst full.  DOK_TOO_LARGE for tables served in several passes. */
int dok_dok_gather_insert(const dok_table *src, const dok_hash_params *src_hp, const dok_selectors *sel,
                          const dok_table *dst, const dok_hash_params *dst_hp, int64_t *counters, void *stream);

/* from_dense: counts the non-zero elements of a contiguous dense tensor (step 1), then inserts
 * (unravelled index -> value) for each of them (step 2) without materialising COO indices.
 * Replaces tensor.to_sparse() + coalesce + set of SparseDOKTensor.from_dense (sparse_dok_tensor.py:71-90).
 * elem_bytes in {1,2,4,8} (= value_bytes of the table); is_float != 0 makes -0.0 count as zero;
 * sizes[ndim] is the dense shape, ndim = hp->key_size, keys are int64. */
int dok_dense_count_nonzero(const void *dense, int64_t numel, int elem_bytes, int is_float, int64_t *count_out,
                            void *stream);

/* rehash in one pass (replaces cuda_closed_hashmap.py:456-468: two boolean-mask gathers and a full set): every live
 * slot of src is hashed with dst's parameters and inserted into dst (initialised, same key and value widths, same
 * key_perm); key bytes and values are copied as stored.  counters[DOK_CNT_CLAIMED_EMPTY] += rows inserted,
 * counters[DOK_CNT_FAILED] += rows that found dst full. */
int dok_map_reinsert(const dok_table *src, const dok_table *dst, const dok_hash_params *dst_hp, int64_t *counters,
                     void *stream);

/* flatten / reshape in one pass (replaces the indices() / values() round trips of sparse_dok_tensor.py:479-514):
 * every live slot of src (int64 index keys of shape src_sizes[src_hp->key_size], row-major) is re-keyed to the index
 * tuple of the same linear position in dst_sizes[dst_hp->key_size] and inserted with its value into dst (an initialised
 * table with the same value_bytes and enough room).  counters[DOK_CNT_CLAIMED_EMPTY] += rows inserted,
 * counters[DOK_CNT_FAILED] += rows that found dst full. */
int dok_dok_rekey_insert(const dok_table *src, const dok_hash_params *src_hp, const int64_t *src_sizes /* host */,
                         const dok_table *dst, const dok_hash_params *dst_hp, const int64_t *dst_sizes /* host */,
                         int64_t *counters, void *stream);
int dok_dense_insert_nonzero(const dok_table *t, const dok_hash_params *hp, const void *dense,
                             const int64_t *sizes /* host */, int64_t numel, int is_float, int64_t *counters,
                             void *stream);

/* ---- hash-sharded table: batch routing (no counterpart in the reference, which is single-GPU) ------- */

/* Owner shard of each row: mulhi64(mix(uuid ^ salt), n_shards).  Stable partition of a batch by owner:
 * step 1 computes every row's owner (owners[n], one byte per row), a per-tile histogram and its scan ->
 * tile_offsets int64[dok_partition_offset_words(n, n_shards)] (the offsets, their total, and the scan's scratch behind
 * them) and shard_counts int64[2 * n_shards]: rows per
 * owner, then the same rounded up to multiples of 16 rows;
 * step 2 scatters key rows of key_bytes (and value rows, if values != NULL) into keys_out/values_out grouped by
 * owner, order within an owner preserved.  Each owner's segment starts at the sum of the ROUNDED counts before it
 * (so every segment is 16-byte aligned for the exchange); the rows of the gap behind a segment are left unwritten
 * and must be ignored by the receiver.  keys_out/values_out need dok_partition_capacity(n, n_shards) rows.
 * dest_index[n] (may be NULL) receives each row's position in that grouped order (for dok_shard_unpermute). */
int64_t dok_partition_tiles(int64_t n);
int64_t dok_partition_offset_words(int64_t n, int n_shards);
int64_t dok_partition_capacity(int64_t n, int n_shards);
int dok_shard_partition_count(const dok_hash_params *hp, const void *keys, int64_t n, int n_shards, uint8_t *owners,
                              int64_t *tile_offsets, int64_t *shard_counts, void *stream);
int dok_shard_partition_scatter(const void *keys, int key_bytes, const void *values, int value_bytes, int64_t n,
                                int n_shards, const uint8_t *owners, const int64_t *tile_offsets,
                                const int64_t *shard_counts, void *keys_out, void *values_out, int64_t *dest_index,
                                void *stream);

/* The same scatter with one destination per owner: peer_keys[o] / peer_values[o] are the owner GPU's receive
 * buffers mapped into this process (dok_peer_open; this rank's own buffer for o == rank) and peer_row0[o] >= 0 the
 * row at which THIS rank's segment starts inside them.  The rows cross NVLink as plain stores while the batch is
 * being partitioned; no exchange pass follows.  dest_index is as above (positions in this rank's own grouped order,
 * where the owner's answers will be placed).  The caller orders the launch against the owners' reads (a collective
 * on the stream before the owners touch the rows, double buffering against the next batch). */
int dok_shard_partition_scatter_peer(const void *keys, int key_bytes, const void *values, int value_bytes, int64_t n,
                                     int n_shards, const uint8_t *owners, const int64_t *tile_offsets,
                                     const int64_t *shard_counts, void *const *peer_keys, void *const *peer_values,
                                     const int64_t *peer_row0, int64_t *dest_index, void *stream);

/* Sliced exchange: every (source rank, owner) pair has a slice of slice_rows rows at a fixed place in the owner's
 * inbox, so a source needs nobody else's counts to know where its rows go, and no rank's host ever waits for a count.
 *  - dok_shard_partition_check_slices (after dok_shard_partition_count): raises the sticky word *status to 1 when an
 *    owner's rows exceed slice_rows, or when force != 0 (the caller already knows the batch cannot go this way).
 *  - dok_shard_partition_scatter_sliced: stores this rank's rows for owner o at slice_keys[o] / slice_values[o]
 *    (the start of this rank's slice in owner o's inbox: peer memory, or local for o == this rank), stores the row
 *    count at count_dst[o] (int64 in the owner's memory; always, also for n == 0), and writes dest_index[i] =
 *    owner * slice_rows + position: where the answer for row i will be in this rank's result region.  With
 *    *status != 0 nothing but zero counts is stored.
 *  - dok_copy_counted: min(*count, max_rows) rows of up to two row arrays (answer values and flags) to another
 *    place -- the asker's result region on another GPU -- in 16-byte pieces; a no-op when *abort_flag != 0.
 *    All four pointers 16-byte aligned; dst_b / src_b may be NULL.
 *  - dok_shard_token_prepare / dok_shard_token_finish bracket the all-reduce(MAX) that closes a send stage: prepare
 *    writes token[3] = {*status, signature, -signature}; after the reduction finish sets token[0] non-zero when any
 *    rank overflowed or the ranks' signatures differ (they submitted different operations), and raises *status to it.
 *    token[0] is the abort_flag of that operation's apply kernels.
 * The owner applies what it received with the *_sliced map operations.  The caller orders the stages with
 * stream-ordered collectives (nothing here waits on another GPU).  No counterpart in the reference. */
int dok_shard_partition_check_slices(const int64_t *shard_counts, int n_shards, int64_t slice_rows, int force,
                                     int64_t *status, void *stream);
int dok_shard_partition_scatter_sliced(const void *keys, int key_bytes, const void *values, int value_bytes, int64_t n,
                                       int n_shards, const uint8_t *owners, const int64_t *tile_offsets,
                                       const int64_t *shard_counts, void *const *slice_keys, void *const *slice_values,
                                       int64_t *const *count_dst, int64_t slice_rows, const int64_t *status,
                                       int64_t *dest_index, void *stream);
int dok_shard_token_prepare(const int64_t *status, int64_t signature, int64_t *token, void *stream);
/* Blocks of the two partition passes (dok_shard_partition_count and the scatter calls): 0 = one block per tile of
 * 2048 rows (the default); a positive number caps the grid and every block walks several tiles, which leaves room
 * on the SMs for the table kernels of another operation in flight.  Process-wide.  No counterpart in the reference. */
int dok_set_routing_blocks(int blocks);
int dok_shard_token_finish(int64_t *token, int64_t *status, void *stream);
int dok_copy_counted(void *dst_a, const void *src_a, int row_bytes_a, void *dst_b, const void *src_b, int row_bytes_b,
                     int64_t max_rows, const int64_t *count, const int64_t *abort_flag, void *stream);

/* Exchange arena: device memory of this process that other processes of the node map (CUDA IPC, peer access over
 * NVLink).  dok_peer_alloc allocates outside any caching allocator (an IPC handle names a whole allocation);
 * dok_peer_export fills a DOK_PEER_HANDLE_BYTES handle to send to the peers; dok_peer_open maps a peer's handle. */
#define DOK_PEER_HANDLE_BYTES 64
int dok_peer_alloc(int64_t bytes, void **ptr_out);
int dok_peer_free(void *ptr);
int dok_peer_export(void *ptr, uint8_t *handle_out);
int dok_peer_open(const uint8_t *handle, void **ptr_out);
int dok_peer_close(void *ptr);

/* n_words (<= 1024) int64 words from device memory to PINNED host memory (cudaHostAlloc / torch pin_memory), written
 * by a kernel through the mapped address instead of a copy-engine transfer, so that the read-back of the row counts
 * does not queue behind bulk device-to-host copies of other streams.  Complete when the stream reaches this point. */
int dok_words_to_pinned(const int64_t *src, int64_t *pinned_dst, int n_words, void *stream);

/* out_values[i] = grouped_values[dest_index[i]], out_found[i] = grouped_found[dest_index[i]].  abort_flag (device
 * int64, may be NULL): non-zero when the kernel runs = nothing is read or written (the operation was skipped and
 * dest_index holds nothing). */
int dok_shard_unpermute(const void *grouped_values, const uint8_t *grouped_found, const int64_t *dest_index,
                        int value_bytes, int64_t n, void *out_values, uint8_t *out_found, const int64_t *abort_flag,
                        void *stream);

/* Diagnostic: n_reads independent random 16-byte reads over buf[0, bytes) (one per thread).  Timed by the caller,
 * it gives the rate at which this GPU serves random requests; for buffers much larger than L2 that rate bounds
 * every probing kernel.  sink may be NULL.  No counterpart in the reference. */
int dok_diag_random_reads(const void *buf, int64_t bytes, int64_t n_reads, uint64_t seed, int64_t *sink, void *stream);
/* The same with a chosen request shape: `lanes` adjacent lanes read bytes_per_lane each of one random aligned unit
 * (supported: 8x1, 16x1, 32x1, 32x2, 32x4, 16x4 = requests of 8 ... 128 bytes).  Under a profiler the DRAM bytes per
 * request of the different shapes show the granule of a random access (128 bytes on B200, whatever is asked for). */
int dok_diag_random_requests(const void *buf, int64_t bytes, int64_t n_requests, int bytes_per_lane, int lanes,
                             uint64_t seed, int64_t *sink, void *stream);

/* owner_out[i] = owner shard of row i (diagnostics; the partition computes the same value internally) */
int dok_shard_owner(const dok_hash_params *hp, const void *keys, int64_t n, int n_shards, int32_t *owner_out,
                    void *stream);

#ifdef __cplusplus
}
#endif
#endif /* DOKSPARSE_H */
