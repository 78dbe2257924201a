// Batch routing for the hash-sharded table (declared in include/doksparse.h): a stable partition of a batch by
// owner shard, and the inverse permutation applied to the results.  The reference is single-GPU and has no
// counterpart; what is preserved is its single-table semantics: rows keep their batch order inside each owner's
// segment, so "last row wins" on the owner equals "last row wins" on one big table.
#include "dok_host.cuh"

#define DOK_PART_ROUNDS 8
#define DOK_PART_TILE (DOK_TPB * DOK_PART_ROUNDS)
// Every owner's segment starts on a multiple of this many rows, so that it starts 16-byte aligned whatever the row
// width (NCCL moves unaligned segments several times slower).  The rows of the gap behind a segment are not
// written; the receiver learns the exact row count of each segment and ignores them.
#define DOK_SEGMENT_ALIGN_ROWS 16

__device__ __forceinline__ void dok_copy_row(char *dst, const char *src, int bytes) {
  if ((bytes & 7) == 0) for (int i = 0; i < (bytes >> 3); i++) ((ull_t *)dst)[i] = ((const ull_t *)src)[i];
  else if ((bytes & 3) == 0) for (int i = 0; i < (bytes >> 2); i++) ((unsigned *)dst)[i] = ((const unsigned *)src)[i];
  else if ((bytes & 1) == 0) for (int i = 0; i < (bytes >> 1); i++) ((unsigned short *)dst)[i] = ((const unsigned short *)src)[i];
  else for (int i = 0; i < bytes; i++) dst[i] = src[i];
}

// Tile = DOK_PART_TILE consecutive rows; thread t of the block owns rows base + r * DOK_TPB + t, r = 0 .. ROUNDS-1,
// so the row order inside a tile is (round, warp, lane).
//
// Pass 1: owner shard of every row, kept as one byte per row for the second pass (the uuid is the expensive part
// of routing: one 64-bit remainder per key element), and the rows per owner of each tile.  The lanes of a warp
// that share an owner are found with one match; their first lane adds the group's size to the tile's histogram.
static __global__ void __launch_bounds__(DOK_TPB) k_part_count(DevHash hp, RowKeys keys, int n_shards, ll_t tiles,
                                                               uint8_t *__restrict__ owners,
                                                               ll_t *__restrict__ tile_counts) {
  __shared__ int hist[DOK_MAX_SHARDS];
  const int lane = threadIdx.x & 31;
  for (ll_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    if (threadIdx.x < DOK_MAX_SHARDS) hist[threadIdx.x] = 0;
    __syncthreads();
    const ll_t base = tile * DOK_PART_TILE;
#pragma unroll
    for (int r = 0; r < DOK_PART_ROUNDS; r++) {
      const ll_t e = base + r * DOK_TPB + threadIdx.x;
      int owner = -1;
      if (e < keys.n) {
        owner = dok_owner_shard(keys.hash(hp, e).uuid, n_shards);
        owners[e] = (uint8_t)owner;
      }
      const unsigned peers = __match_any_sync(0xffffffffu, owner);
      if (owner >= 0 && (peers & ((1u << lane) - 1u)) == 0) atomicAdd(&hist[owner], __popc(peers));
    }
    __syncthreads();
    // the thread that reads a counter is the one that clears it for the next tile
    if (threadIdx.x < n_shards) tile_counts[(ll_t)threadIdx.x * tiles + tile] = hist[threadIdx.x];
  }
}

// In-place exclusive scan of a[0 .. n); a[n] receives the total.  Three small launches: sums of chunks of
// DOK_SCAN_CHUNK elements (coalesced), a scan of those sums by one block, and the scan of every chunk on top of its
// offset.  (One block walking the whole array -- 131 K tile counts for 32 Mi rows and 8 owners -- took longer than the
// partition pass it follows.)
#define DOK_SCAN_CHUNK 2048
__device__ __forceinline__ ll_t dok_block_sum(ll_t v, ll_t *warp_sums) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = v;
  __syncthreads();
  ll_t total = 0;
  for (int w = 0; w < (int)(blockDim.x >> 5); w++) total += warp_sums[w];
  __syncthreads();
  return total;
}
static __global__ void __launch_bounds__(256) k_scan_chunk_sums(const ll_t *__restrict__ a, ll_t n, ll_t *__restrict__ sums) {
  __shared__ ll_t warp_sums[8];
  const ll_t base = (ll_t)blockIdx.x * DOK_SCAN_CHUNK;
  ll_t v = 0;
#pragma unroll
  for (int r = 0; r < DOK_SCAN_CHUNK / 256; r++) {
    const ll_t i = base + r * 256 + threadIdx.x;
    if (i < n) v += a[i];
  }
  const ll_t total = dok_block_sum(v, warp_sums);
  if (threadIdx.x == 0) sums[blockIdx.x] = total;
}
// exclusive scan of sums[0 .. m) by one block, sums[m] = total (m = chunks: 64 for the case above)
static __global__ void __launch_bounds__(1024) k_scan_sums(ll_t *sums, ll_t m) {
  __shared__ ll_t partial[1024];
  const ll_t per = (m + 1023) / 1024;
  const ll_t lo = threadIdx.x * per, hi = lo + per < m ? lo + per : m;
  ll_t s = 0;
  for (ll_t i = lo; i < hi; i++) s += sums[i];
  partial[threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.x < 32) {                       // one warp scans the 1024 partial sums, 32 per lane
    ll_t run = 0;
    for (int i = 0; i < 32; i++) run += partial[threadIdx.x * 32 + i];
    ll_t inc = run;
    for (int d = 1; d < 32; d <<= 1) {
      const ll_t up = __shfl_up_sync(0xffffffffu, inc, d);
      if ((int)threadIdx.x >= d) inc += up;
    }
    ll_t start = inc - run;
    for (int i = 0; i < 32; i++) { const ll_t v = partial[threadIdx.x * 32 + i]; partial[threadIdx.x * 32 + i] = start; start += v; }
    if (threadIdx.x == 31) sums[m] = inc;
  }
  __syncthreads();
  ll_t run = partial[threadIdx.x];
  for (ll_t i = lo; i < hi; i++) { const ll_t v = sums[i]; sums[i] = run; run += v; }
}
static __global__ void __launch_bounds__(256) k_scan_chunks(ll_t *__restrict__ a, ll_t n, const ll_t *__restrict__ sums, ll_t m) {
  __shared__ ll_t warp_sums[8];
  __shared__ ll_t carry;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const ll_t base = (ll_t)blockIdx.x * DOK_SCAN_CHUNK;
  if (threadIdx.x == 0) carry = sums[blockIdx.x];
  __syncthreads();
  for (int r = 0; r < DOK_SCAN_CHUNK / 256; r++) {
    const ll_t i = base + r * 256 + threadIdx.x;
    const ll_t v = i < n ? a[i] : 0;
    ll_t inc = v;
    for (int d = 1; d < 32; d <<= 1) {
      const ll_t up = __shfl_up_sync(0xffffffffu, inc, d);
      if (lane >= d) inc += up;
    }
    if (lane == 31) warp_sums[warp] = inc;
    __syncthreads();
    ll_t before = carry;
    for (int w = 0; w < warp; w++) before += warp_sums[w];
    if (i < n) a[i] = before + inc - v;
    __syncthreads();
    if (threadIdx.x == 255) carry = before + inc;
    __syncthreads();
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) a[n] = sums[m];
}
// scratch: int64[n / DOK_SCAN_CHUNK + 2]
static int dok_exclusive_scan(ll_t *a, ll_t n, ll_t *scratch, cudaStream_t st) {
  const ll_t chunks = (n + DOK_SCAN_CHUNK - 1) / DOK_SCAN_CHUNK;
  if (chunks == 0) {                             // nothing to scan: the total is zero
    if (cudaMemsetAsync(a, 0, sizeof(ll_t), st) != cudaSuccess) return dok_check_launch();
    return DOK_OK;
  }
  k_scan_chunk_sums<<<(unsigned)chunks, 256, 0, st>>>(a, n, scratch);
  int rc = dok_check_launch();
  if (rc != DOK_OK) return rc;
  k_scan_sums<<<1, 1024, 0, st>>>(scratch, chunks);
  rc = dok_check_launch();
  if (rc != DOK_OK) return rc;
  k_scan_chunks<<<(unsigned)chunks, 256, 0, st>>>(a, n, scratch, chunks);
  return dok_check_launch();
}

// shard_counts[0 .. P) = rows per owner, shard_counts[P .. 2P) = the same rounded up to whole alignment units
static __global__ void k_part_shard_counts(const ll_t *tile_offsets, int n_shards, ll_t tiles, ll_t *shard_counts) {
  const int o = threadIdx.x;
  if (o < n_shards) {
    const ll_t c = tile_offsets[(ll_t)(o + 1) * tiles] - tile_offsets[(ll_t)o * tiles];
    shard_counts[o] = c;
    shard_counts[n_shards + o] = (c + DOK_SEGMENT_ALIGN_ROWS - 1) / DOK_SEGMENT_ALIGN_ROWS * DOK_SEGMENT_ALIGN_ROWS;
  }
}

// Where the rows of each owner go.  Local exchange buffer: every owner the same base, row0 < 0 = "at the start of
// the owner's segment in this rank's grouped order".  Peer exchange: base = the owner GPU's receive buffer (mapped into this process), row0 = where THIS rank's segment
// starts inside it; the rows then cross NVLink as plain stores while the tile is being partitioned, and no separate
// exchange pass follows.
struct PartDest {
  char *keys[DOK_MAX_SHARDS];
  char *values[DOK_MAX_SHARDS];
  ll_t row0[DOK_MAX_SHARDS];
  // Sliced exchange (slice_rows > 0): every (source, owner) pair has a slice of slice_rows rows at a FIXED place in
  // the owner's inbox, so a source needs nobody's counts to know where its rows go; dest_index is the row's place in
  // the asker's result region, owner * slice_rows + position.  *status != 0 (a slice overflowed somewhere, now or
  // earlier) makes the launch a no-op: the host repeats the operation over the exact exchange.
  ll_t slice_rows;
  const ll_t *status;
};

// Pass 2: every row to its place.  Rows of one owner keep their batch order: inside a tile the place of a row is
// the number of same-owner rows before it in (round, warp, lane) order -- per-(round, warp) counts from warp
// matches, one exclusive scan per owner over the ROUNDS * warps counts, and the row's rank among its warp's
// same-owner lanes -- behind the tile's offset from pass 1.
// STAGED: the tile's rows are first sorted by owner in shared memory and then written out run by run, so that
// consecutive threads store consecutive rows of one owner: with 8 owners a warp's 32 rows would otherwise leave as
// 8 pieces of ~32 bytes each, which wastes most of an NVLink packet (and of a memory transaction).  Needs
// DOK_PART_TILE * (kb + vb) bytes of dynamic shared memory; wide rows take the direct path.
// dest_index[e] is always the row's position in THIS rank's grouped order (segments at the padded local offsets),
// which is where the owner's answer for the row will be found.
template <bool STAGED>
static __global__ void __launch_bounds__(DOK_TPB, 6) k_part_scatter(RowKeys keys, int kb, const char *__restrict__ values,
                                                                 int vb, const uint8_t *__restrict__ owners,
                                                                 int n_shards, ll_t tiles,
                                                                 const ll_t *__restrict__ tile_offsets,
                                                                 const ll_t *__restrict__ shard_counts,
                                                                 const __grid_constant__ PartDest dst,
                                                                 ll_t *__restrict__ dest_index) {
  constexpr int WARPS = DOK_TPB / 32, CELLS = DOK_PART_ROUNDS * WARPS;        // cells of one owner, in row order
  // dynamic shared memory: before[n_shards][CELLS] (same-owner rows of the tile before cell (round, warp)), then,
  // STAGED, the key rows of the tile sorted by owner and the value rows
  extern __shared__ __align__(16) char dyn_smem[];
  int (*before)[CELLS] = (int (*)[CELLS])dyn_smem;
  char *stage = dyn_smem + (size_t)n_shards * CELLS * sizeof(int);
  __shared__ int tile_total[DOK_MAX_SHARDS];      // rows of the owner in this tile
  __shared__ int sorted_start[DOK_MAX_SHARDS + 1];// STAGED: first sorted position of the owner's run in the tile
  __shared__ ll_t tile_first[DOK_MAX_SHARDS];     // rows of this owner in earlier tiles
  __shared__ ll_t local_start[DOK_MAX_SHARDS];    // start of the owner's segment in this rank's grouped order
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (dst.status != nullptr && *dst.status != 0) return;       // uniform over the grid
  // one thread per owner fetches its words (a single thread walking the owners would wait for 2 * n_shards dependent
  // loads at the head of every block)
  if ((int)threadIdx.x < n_shards) local_start[threadIdx.x] = shard_counts[n_shards + threadIdx.x];
  __syncthreads();
  if (threadIdx.x == 0) {
    ll_t padded = 0;                              // owner o's segment starts at the sum of the padded counts before it
    for (int o = 0; o < n_shards; o++) {
      const ll_t c = local_start[o];
      local_start[o] = padded;
      padded += c;
    }
  }
  char *stage_values = stage + (size_t)DOK_PART_TILE * kb;      // cell counts are a multiple of 16 bytes: still aligned
  for (ll_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    for (int i = threadIdx.x; i < n_shards * CELLS; i += DOK_TPB) ((int *)dyn_smem)[i] = 0;
    if ((int)threadIdx.x < n_shards)
      tile_first[threadIdx.x] = tile_offsets[(ll_t)threadIdx.x * tiles + tile] - tile_offsets[(ll_t)threadIdx.x * tiles];
    __syncthreads();
    const ll_t base = tile * DOK_PART_TILE;
    int owner[DOK_PART_ROUNDS];
    int rank[DOK_PART_ROUNDS];                    // same-owner lanes of the warp below this one
#pragma unroll
    for (int r = 0; r < DOK_PART_ROUNDS; r++) {
      const ll_t e = base + r * DOK_TPB + threadIdx.x;
      owner[r] = e < keys.n ? (int)owners[e] : -1;
      const unsigned peers = __match_any_sync(0xffffffffu, owner[r]);
      rank[r] = __popc(peers & ((1u << lane) - 1u));
      if (owner[r] >= 0 && rank[r] == 0) before[owner[r]][r * WARPS + warp] = __popc(peers);
    }
    __syncthreads();
    for (int o = warp; o < n_shards; o += WARPS) {  // exclusive scan of the owner's CELLS counts by one warp
      int run = 0;
#pragma unroll
      for (int c0 = 0; c0 < CELLS; c0 += 32) {
        const int v = before[o][c0 + lane];
        int inc = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const int up = __shfl_up_sync(0xffffffffu, inc, d);
          if (lane >= d) inc += up;
        }
        before[o][c0 + lane] = run + inc - v;
        run += __shfl_sync(0xffffffffu, inc, 31);
      }
      if (lane == 0) tile_total[o] = run;
    }
    __syncthreads();
    if (!STAGED) {
#pragma unroll
      for (int r = 0; r < DOK_PART_ROUNDS; r++) {
        if (owner[r] < 0) continue;
        const int o = owner[r];
        const ll_t e = base + r * DOK_TPB + threadIdx.x;
        const ll_t in_segment = tile_first[o] + before[o][r * WARPS + warp] + rank[r];
        if (dest_index) dest_index[e] = (dst.slice_rows > 0 ? (ll_t)o * dst.slice_rows : local_start[o]) + in_segment;
        const ll_t row = (dst.row0[o] >= 0 ? dst.row0[o] : local_start[o]) + in_segment;
        dok_copy_row(dst.keys[o] + row * kb, (const char *)keys.keys + e * kb, kb);
        if (values) dok_copy_row(dst.values[o] + row * vb, values + e * vb, vb);
      }
      __syncthreads();                            // the cells are cleared for the next tile
      continue;
    }
    if (threadIdx.x == 0) {
      int run = 0;
      for (int o = 0; o < n_shards; o++) { sorted_start[o] = run; run += tile_total[o]; }
      sorted_start[n_shards] = run;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < DOK_PART_ROUNDS; r++) {
      if (owner[r] < 0) continue;
      const int o = owner[r];
      const ll_t e = base + r * DOK_TPB + threadIdx.x;
      const int in_tile = before[o][r * WARPS + warp] + rank[r];
      if (dest_index) dest_index[e] = (dst.slice_rows > 0 ? (ll_t)o * dst.slice_rows : local_start[o]) + tile_first[o] + in_tile;
      const int pos = sorted_start[o] + in_tile;
      dok_copy_row(stage + (size_t)pos * kb, (const char *)keys.keys + e * kb, kb);
      if (values) dok_copy_row(stage_values + (size_t)pos * vb, values + e * vb, vb);
    }
    __syncthreads();
    const int tile_rows = sorted_start[n_shards];
    for (int i = threadIdx.x; i < tile_rows; i += DOK_TPB) {
      int o = 0;                                  // the run that sorted position i belongs to
      while (sorted_start[o + 1] <= i) o++;
      const ll_t row = (dst.row0[o] >= 0 ? dst.row0[o] : local_start[o]) + tile_first[o] + (i - sorted_start[o]);
      dok_copy_row(dst.keys[o] + row * kb, stage + (size_t)i * kb, kb);
      if (values) dok_copy_row(dst.values[o] + row * vb, stage_values + (size_t)i * vb, vb);
    }
    __syncthreads();                              // the staging area and the cells are reused by the next tile
  }
}

// Blocks of the two partition passes: one per tile by default; a smaller number makes every block walk several tiles,
// which leaves room on the SMs for the table kernels of another operation running at the same time.
static std::atomic<int> g_routing_blocks{0};
static unsigned dok_routing_grid(ll_t tiles) {
  const int cap = g_routing_blocks.load(std::memory_order_relaxed);
  return (unsigned)(cap > 0 && tiles > cap ? cap : tiles);
}

// staged when the tile's rows fit the shared memory a block may ask for without crowding out its neighbours
#define DOK_PART_STAGE_LIMIT (64 * 1024)
static int dok_launch_scatter(const RowKeys &rk, int kb, const char *values, int vb, const uint8_t *owners, int n_shards,
                              const ll_t *tile_offsets, const ll_t *shard_counts, const PartDest &dst, ll_t *dest_index,
                              cudaStream_t st) {
  const ll_t tiles = dok_partition_tiles(rk.n);
  const size_t stage_bytes = (size_t)DOK_PART_TILE * (size_t)(kb + (values ? vb : 0));
  const size_t cell_bytes = (size_t)n_shards * DOK_PART_ROUNDS * (DOK_TPB / 32) * sizeof(int);
  if (n_shards > 2 && stage_bytes <= DOK_PART_STAGE_LIMIT) {
    // more than the 48 KiB a kernel gets by default: the attribute is per device, and setting it again is cheap
    cudaFuncSetAttribute(k_part_scatter<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, DOK_PART_STAGE_LIMIT + 16 * 1024);
    k_part_scatter<true><<<dok_routing_grid(tiles), DOK_TPB, cell_bytes + stage_bytes, st>>>(rk, kb, values, vb, owners, n_shards, tiles,
                                                                                     tile_offsets, shard_counts, dst, dest_index);
  } else {
    k_part_scatter<false><<<dok_routing_grid(tiles), DOK_TPB, cell_bytes, st>>>(rk, kb, values, vb, owners, n_shards, tiles, tile_offsets,
                                                                        shard_counts, dst, dest_index);
  }
  return dok_check_launch();
}

// Sliced exchange: rows per owner as above, and the sticky status word is raised when an owner's rows do not fit
// its slice (or the caller already knows that the batch cannot go this way: force != 0).
static __global__ void k_part_check_slices(const ll_t *shard_counts, int n_shards, ll_t slice_rows, int force, ll_t *status) {
  const int o = threadIdx.x;
  if ((o < n_shards && shard_counts[o] > slice_rows) || (o == 0 && force)) *status = 1;
}

// The source tells every owner how many rows it put into its slice of that owner's inbox (a store into the owner's
// memory, like the rows themselves).  Always launched, also for an empty batch: the owner must not see the count of
// an earlier use of the slice.
struct CountDest { ll_t *at[DOK_MAX_SHARDS]; };
static __global__ void k_part_publish_counts(const ll_t *shard_counts, int n_shards, const __grid_constant__ CountDest dst,
                                             const ll_t *status) {
  const int o = threadIdx.x;
  if (o < n_shards && dst.at[o] != nullptr) *dst.at[o] = (status != nullptr && *status != 0) ? 0 : shard_counts[o];
}

// The token of one operation, before and after its all-reduce(MAX) over the ranks: {sticky status, signature,
// -signature} goes in; what comes out tells every rank, on the device, whether any rank overflowed (now or earlier)
// and whether all ranks submitted the same operation (max(signature) == -max(-signature)).  Either makes token[0]
// non-zero, which the apply kernels read as "do nothing", and raises this rank's sticky status.
static __global__ void k_token_prepare(const ll_t *status, ll_t signature, ll_t *token) {
  token[0] = *status;
  token[1] = signature;
  token[2] = -signature;
}
static __global__ void k_token_finish(ll_t *token, ll_t *status) {
  if (token[1] + token[2] != 0 && token[0] == 0) token[0] = 1;
  if (token[0] > *status) *status = token[0];
}

// min(*count, max_rows) rows of two row arrays (the answers of a lookup: values and flags) to another place, usually
// the asker's memory on another GPU: consecutive threads move consecutive 16-byte pieces, so the stores cross NVLink as
// full packets.  The row count is read on the device; both sources and destinations are 16-byte aligned.
static __global__ void __launch_bounds__(256) k_copy_counted(char *__restrict__ dst_a, const char *__restrict__ src_a, int rb_a,
                                                             char *__restrict__ dst_b, const char *__restrict__ src_b, int rb_b,
                                                             ll_t max_rows, const ll_t *count, const ll_t *abort) {
  if (abort != nullptr && *abort != 0) return;
  ll_t rows = *count;
  if (rows > max_rows) rows = max_rows;
  const ll_t stride = (ll_t)gridDim.x * blockDim.x;
  const ll_t first = (ll_t)blockIdx.x * blockDim.x + threadIdx.x;
#pragma unroll
  for (int which = 0; which < 2; which++) {
    char *dst = which ? dst_b : dst_a;
    const char *src = which ? src_b : src_a;
    const ll_t bytes = rows * (which ? rb_b : rb_a);
    if (dst == nullptr || bytes == 0) continue;
    const ll_t whole = bytes >> 4;
    for (ll_t i = first; i < whole; i += stride) ((uint4 *)dst)[i] = ((const uint4 *)src)[i];
    const ll_t tail = whole << 4;
    if (first < bytes - tail) dst[tail + first] = src[tail + first];
  }
}

static __global__ void __launch_bounds__(DOK_TPB) k_unpermute(const char *__restrict__ grouped_values,
                                                              const uint8_t *__restrict__ grouped_found,
                                                              const ll_t *__restrict__ dest_index, int vb, ll_t n,
                                                              char *__restrict__ out_values, uint8_t *__restrict__ out_found,
                                                              const ll_t *abort) {
  if (abort != nullptr && *abort != 0) return;      // the operation was skipped: dest_index was never written
  const ll_t i = (ll_t)blockIdx.x * DOK_TPB + threadIdx.x;
  if (i >= n) return;
  const ll_t g = dest_index[i];
  if (out_values) dok_copy_row(out_values + i * vb, grouped_values + g * vb, vb);
  if (out_found) out_found[i] = grouped_found[g];
}

extern "C" {

int64_t dok_partition_tiles(int64_t n) { return (n + DOK_PART_TILE - 1) / DOK_PART_TILE; }
int64_t dok_partition_offset_words(int64_t n, int n_shards) {
  const int64_t cells = (int64_t)n_shards * dok_partition_tiles(n);
  return cells + 1 + (cells + DOK_SCAN_CHUNK - 1) / DOK_SCAN_CHUNK + 2;      // offsets, total, scan scratch
}
int64_t dok_partition_capacity(int64_t n, int n_shards) { return n + (int64_t)n_shards * (DOK_SEGMENT_ALIGN_ROWS - 1); }

int dok_shard_partition_count(const dok_hash_params *hp, const void *keys, int64_t n, int n_shards, uint8_t *owners,
                              int64_t *tile_offsets, int64_t *shard_counts, void *stream) {
  DevHash dh;
  if (!dok_make_hash(hp, &dh) || n < 0 || n > DOK_MAX_BATCH || n_shards < 1 || n_shards > DOK_MAX_SHARDS) return DOK_BAD_ARG;
  if (!tile_offsets || !shard_counts || (n > 0 && (!keys || !owners))) return DOK_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const ll_t tiles = dok_partition_tiles(n);
  if (tiles > 0) {
    RowKeys rk{keys, n};
    k_part_count<<<dok_routing_grid(tiles), DOK_TPB, 0, st>>>(dh, rk, n_shards, tiles, owners, (ll_t *)tile_offsets);
    int rc = dok_check_launch();
    if (rc != DOK_OK) return rc;
  }
  const ll_t cells = (ll_t)n_shards * tiles;
  int rc = dok_exclusive_scan((ll_t *)tile_offsets, cells, (ll_t *)tile_offsets + cells + 1, st);
  if (rc != DOK_OK) return rc;
  k_part_shard_counts<<<1, DOK_MAX_SHARDS, 0, st>>>((const ll_t *)tile_offsets, n_shards, tiles, (ll_t *)shard_counts);
  return dok_check_launch();
}

int dok_shard_partition_scatter(const void *keys, int key_bytes, const void *values, int value_bytes, int64_t n,
                                int n_shards, const uint8_t *owners, const int64_t *tile_offsets,
                                const int64_t *shard_counts, void *keys_out, void *values_out, int64_t *dest_index,
                                void *stream) {
  if (n < 0 || n > DOK_MAX_BATCH || n_shards < 1 || n_shards > DOK_MAX_SHARDS) return DOK_BAD_ARG;
  if (n == 0) return DOK_OK;
  if (!keys || key_bytes < 1 || !owners || !tile_offsets || !shard_counts || !keys_out) return DOK_BAD_ARG;
  if (values && (!values_out || value_bytes < 1 || value_bytes > DOK_MAX_VALUE_BYTES)) return DOK_BAD_ARG;
  RowKeys rk{keys, n};
  // every owner's segment lies in the same local buffer, at the prefix sum of the padded counts, which the kernel
  // derives from shard_counts on the device (row0 < 0 asks for that): the host never needs the counts here
  PartDest dst;
  memset(&dst, 0, sizeof(dst));
  for (int o = 0; o < n_shards; o++) { dst.keys[o] = (char *)keys_out; dst.values[o] = (char *)values_out; dst.row0[o] = -1; }
  return dok_launch_scatter(rk, key_bytes, (const char *)values, value_bytes, owners, n_shards, (const ll_t *)tile_offsets,
                            (const ll_t *)shard_counts, dst, (ll_t *)dest_index, (cudaStream_t)stream);
}

int dok_shard_partition_scatter_peer(const void *keys, int key_bytes, const void *values, int value_bytes, int64_t n,
                                     int n_shards, const uint8_t *owners, const int64_t *tile_offsets,
                                     const int64_t *shard_counts, void *const *peer_keys, void *const *peer_values,
                                     const int64_t *peer_row0, int64_t *dest_index, void *stream) {
  if (n < 0 || n > DOK_MAX_BATCH || n_shards < 1 || n_shards > DOK_MAX_SHARDS) return DOK_BAD_ARG;
  if (n == 0) return DOK_OK;
  if (!keys || key_bytes < 1 || !owners || !tile_offsets || !shard_counts || !peer_keys || !peer_row0) return DOK_BAD_ARG;
  if (values && (!peer_values || value_bytes < 1 || value_bytes > DOK_MAX_VALUE_BYTES)) return DOK_BAD_ARG;
  PartDest dst;
  memset(&dst, 0, sizeof(dst));
  for (int o = 0; o < n_shards; o++) {
    if (!peer_keys[o] || peer_row0[o] < 0 || (values && !peer_values[o])) return DOK_BAD_ARG;
    dst.keys[o] = (char *)peer_keys[o];
    dst.values[o] = values ? (char *)peer_values[o] : nullptr;
    dst.row0[o] = peer_row0[o];
  }
  RowKeys rk{keys, n};
  return dok_launch_scatter(rk, key_bytes, (const char *)values, value_bytes, owners, n_shards, (const ll_t *)tile_offsets,
                            (const ll_t *)shard_counts, dst, (ll_t *)dest_index, (cudaStream_t)stream);
}

int dok_shard_partition_check_slices(const int64_t *shard_counts, int n_shards, int64_t slice_rows, int force,
                                     int64_t *status, void *stream) {
  if (!shard_counts || !status || n_shards < 1 || n_shards > DOK_MAX_SHARDS || slice_rows < 1) return DOK_BAD_ARG;
  k_part_check_slices<<<1, DOK_MAX_SHARDS, 0, (cudaStream_t)stream>>>((const ll_t *)shard_counts, n_shards, slice_rows, force,
                                                                      (ll_t *)status);
  return dok_check_launch();
}

int dok_shard_partition_scatter_sliced(const void *keys, int key_bytes, const void *values, int value_bytes, int64_t n,
                                       int n_shards, const uint8_t *owners, const int64_t *tile_offsets,
                                       const int64_t *shard_counts, void *const *slice_keys, void *const *slice_values,
                                       int64_t *const *count_dst, int64_t slice_rows, const int64_t *status,
                                       int64_t *dest_index, void *stream) {
  if (n < 0 || n > DOK_MAX_BATCH || n_shards < 1 || n_shards > DOK_MAX_SHARDS || slice_rows < 1) return DOK_BAD_ARG;
  if (!shard_counts || !slice_keys || !count_dst || !status || key_bytes < 1) return DOK_BAD_ARG;
  if (values && (!slice_values || value_bytes < 1 || value_bytes > DOK_MAX_VALUE_BYTES)) return DOK_BAD_ARG;
  if (n > 0 && (!keys || !owners || !tile_offsets)) return DOK_BAD_ARG;
  PartDest dst;
  CountDest cd;
  memset(&dst, 0, sizeof(dst));
  memset(&cd, 0, sizeof(cd));
  for (int o = 0; o < n_shards; o++) {
    if (!slice_keys[o] || !count_dst[o] || (values && !slice_values[o])) return DOK_BAD_ARG;
    dst.keys[o] = (char *)slice_keys[o];
    dst.values[o] = values ? (char *)slice_values[o] : nullptr;
    dst.row0[o] = 0;
    cd.at[o] = (ll_t *)count_dst[o];
  }
  dst.slice_rows = slice_rows;
  dst.status = (const ll_t *)status;
  cudaStream_t st = (cudaStream_t)stream;
  k_part_publish_counts<<<1, DOK_MAX_SHARDS, 0, st>>>((const ll_t *)shard_counts, n_shards, cd, (const ll_t *)status);
  int rc = dok_check_launch();
  if (rc != DOK_OK || n == 0) return rc;
  RowKeys rk{keys, n};
  return dok_launch_scatter(rk, key_bytes, (const char *)values, value_bytes, owners, n_shards, (const ll_t *)tile_offsets,
                            (const ll_t *)shard_counts, dst, (ll_t *)dest_index, st);
}

int dok_set_routing_blocks(int blocks) {
  if (blocks < 0) return DOK_BAD_ARG;
  g_routing_blocks.store(blocks, std::memory_order_relaxed);
  return DOK_OK;
}

int dok_shard_token_prepare(const int64_t *status, int64_t signature, int64_t *token, void *stream) {
  if (!status || !token) return DOK_BAD_ARG;
  k_token_prepare<<<1, 1, 0, (cudaStream_t)stream>>>((const ll_t *)status, (ll_t)signature, (ll_t *)token);
  return dok_check_launch();
}

int dok_shard_token_finish(int64_t *token, int64_t *status, void *stream) {
  if (!status || !token) return DOK_BAD_ARG;
  k_token_finish<<<1, 1, 0, (cudaStream_t)stream>>>((ll_t *)token, (ll_t *)status);
  return dok_check_launch();
}

int dok_copy_counted(void *dst_a, const void *src_a, int row_bytes_a, void *dst_b, const void *src_b, int row_bytes_b,
                     int64_t max_rows, const int64_t *count, const int64_t *abort_flag, void *stream) {
  if (!count || max_rows < 0 || (dst_a && (!src_a || row_bytes_a < 1)) || (dst_b && (!src_b || row_bytes_b < 1))) return DOK_BAD_ARG;
  if ((((uintptr_t)dst_a | (uintptr_t)src_a | (uintptr_t)dst_b | (uintptr_t)src_b) & 15) != 0) return DOK_BAD_ARG;
  if (max_rows == 0 || (!dst_a && !dst_b)) return DOK_OK;
  const ll_t pieces = (max_rows * (ll_t)(row_bytes_a > row_bytes_b ? row_bytes_a : row_bytes_b) + 15) / 16;
  ll_t blocks = (pieces + 255) / 256;
  if (blocks > 148 * 4) blocks = 148 * 4;
  k_copy_counted<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((char *)dst_a, (const char *)src_a, row_bytes_a, (char *)dst_b,
                                                                     (const char *)src_b, row_bytes_b, max_rows,
                                                                     (const ll_t *)count, (const ll_t *)abort_flag);
  return dok_check_launch();
}

/* ---- exchange arena: device memory that the other ranks of the node map into their address space ------------ */

int dok_peer_alloc(int64_t bytes, void **ptr_out) {
  if (bytes < 1 || !ptr_out) return DOK_BAD_ARG;
  void *p = nullptr;
  const cudaError_t err = cudaMalloc(&p, (size_t)bytes);
  if (err != cudaSuccess) { dok_last_error_slot() = (int)err; cudaGetLastError(); return DOK_CUDA_ERROR; }
  *ptr_out = p;
  return DOK_OK;
}

int dok_peer_free(void *ptr) {
  if (!ptr) return DOK_OK;
  const cudaError_t err = cudaFree(ptr);
  if (err != cudaSuccess) { dok_last_error_slot() = (int)err; cudaGetLastError(); return DOK_CUDA_ERROR; }
  return DOK_OK;
}

int dok_peer_export(void *ptr, uint8_t *handle_out /* DOK_PEER_HANDLE_BYTES */) {
  if (!ptr || !handle_out) return DOK_BAD_ARG;
  cudaIpcMemHandle_t h;
  const cudaError_t err = cudaIpcGetMemHandle(&h, ptr);
  if (err != cudaSuccess) { dok_last_error_slot() = (int)err; cudaGetLastError(); return DOK_CUDA_ERROR; }
  static_assert(sizeof(h) == DOK_PEER_HANDLE_BYTES, "handle size");
  memcpy(handle_out, &h, sizeof(h));
  return DOK_OK;
}

int dok_peer_open(const uint8_t *handle, void **ptr_out) {
  if (!handle || !ptr_out) return DOK_BAD_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void *p = nullptr;
  const cudaError_t err = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (err != cudaSuccess) { dok_last_error_slot() = (int)err; cudaGetLastError(); return DOK_CUDA_ERROR; }
  *ptr_out = p;
  return DOK_OK;
}

int dok_peer_close(void *ptr) {
  if (!ptr) return DOK_OK;
  const cudaError_t err = cudaIpcCloseMemHandle(ptr);
  if (err != cudaSuccess) { dok_last_error_slot() = (int)err; cudaGetLastError(); return DOK_CUDA_ERROR; }
  return DOK_OK;
}

int dok_shard_unpermute(const void *grouped_values, const uint8_t *grouped_found, const int64_t *dest_index,
                        int value_bytes, int64_t n, void *out_values, uint8_t *out_found, const int64_t *abort_flag,
                        void *stream) {
  if (n < 0 || n > DOK_MAX_BATCH) return DOK_BAD_ARG;
  if (n == 0) return DOK_OK;
  if (!dest_index || (out_values && (!grouped_values || value_bytes < 1)) || (out_found && !grouped_found)) return DOK_BAD_ARG;
  k_unpermute<<<(unsigned)((n + DOK_TPB - 1) / DOK_TPB), DOK_TPB, 0, (cudaStream_t)stream>>>(
      (const char *)grouped_values, grouped_found, (const ll_t *)dest_index, value_bytes, n, (char *)out_values, out_found,
      (const ll_t *)abort_flag);
  return dok_check_launch();
}

/* A few words from device memory into PINNED host memory by a kernel store (pinned memory is mapped into the
 * device's address space), not by a copy: a copy would queue on the device-to-host copy engine behind whatever
 * bulk result transfer another stream has in flight, and the host waits for these words (the per-owner row counts)
 * before it can size the exchange. */
static __global__ void k_words_to_host(const ll_t *__restrict__ src, volatile ll_t *dst, int n) {
  if ((int)threadIdx.x < n) dst[threadIdx.x] = src[threadIdx.x];
  __threadfence_system();
}

int dok_words_to_pinned(const int64_t *src, int64_t *pinned_dst, int n_words, void *stream) {
  if (!src || !pinned_dst || n_words < 1 || n_words > 1024) return DOK_BAD_ARG;
  k_words_to_host<<<1, 1024, 0, (cudaStream_t)stream>>>((const ll_t *)src, (volatile ll_t *)pinned_dst, n_words);
  return dok_check_launch();
}

/* owner shard of each row (diagnostics and host-side tests of the routing) */
static __global__ void k_owner(DevHash hp, RowKeys keys, int n_shards, int *owner_out) {
  const ll_t e = (ll_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e < keys.n) owner_out[e] = dok_owner_shard(keys.hash(hp, e).uuid, n_shards);
}

int dok_shard_owner(const dok_hash_params *hp, const void *keys, int64_t n, int n_shards, int32_t *owner_out,
                    void *stream) {
  DevHash dh;
  if (!dok_make_hash(hp, &dh) || n < 0 || n_shards < 1 || n_shards > DOK_MAX_SHARDS || (n > 0 && (!keys || !owner_out))) return DOK_BAD_ARG;
  if (n == 0) return DOK_OK;
  RowKeys rk{keys, n};
  k_owner<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(dh, rk, n_shards, owner_out);
  return dok_check_launch();
}

}  // extern "C"
