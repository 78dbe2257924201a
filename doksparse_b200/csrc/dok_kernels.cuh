// Kernel templates of the closed-hashing map: batched get / set / remove / exists / count-new and the
// compaction of live slots.  They are templated on the slot width SB (32, 64, 128 bytes: quad-cooperative walk,
// one 128-byte group per request; 0: slots wider than a line, serial walk) and on the key source (contiguous key
// rows, or the index tensors of a DOK selector), so that the map entry points (map_api.cu) and the fused DOK
// entry points (dok_api.cu) share them.  One CUDA thread owns one batch element, as in the reference kernels
// (sparse_dok/components/cuda/closed_hashmap_impl.cu); misses write the fallback from the kernel, and counters
// are accumulated on the device so that the host never has to synchronise.
//
// No thread of a warp returns early: the cooperative walk needs all 32 lanes.
#pragma once
#include "dok_host.cuh"

// ---------------------------------------------------------------------------------------------------------
// get
// ---------------------------------------------------------------------------------------------------------
template <int SB, int LW, class Keys>
__global__ void __launch_bounds__(DOK_TPB, (LW == 2 ? (SB == 32 ? 8 : 6) : 1)) k_get(DevTable t, DevHash hp, Keys keys, char *__restrict__ out_values,
                                                    uint8_t *__restrict__ out_found, Fallback fb, ll_t *counters,
                                                    int count_probes) {
  __shared__ BlockTally tally;
  if (keys.idle()) return;
  if (counters) dok_tally_begin(tally);
  ll_t e;
  bool active = keys.row(e);
  KeyHash kh{0, 0};
  if (active) kh = keys.hash(hp, e);
  active = dok_in_window(t, kh, active);
  int probes = 0;
  // on a hit the quad writes the value from the registers that hold the line
  const Located loc = dok_locate<SB, LW, false>(t, kh, e, active, &probes, EmitValue<(SB == 0 ? 32 : SB), LW>{t, out_values});
  const int hit = active && loc.found >= 0;
  if (active) {
    char *dst = out_values + e * (ll_t)t.vb;
    if (SB == 0 && hit) dok_load_value(t, loc.found, dst);
    if (!hit) dok_store_fallback(t, fb, dst);
  }
  if (active && out_found) out_found[e] = (uint8_t)hit;
  if (counters) {
    dok_tally_add(tally, DOK_CNT_HITS, hit);
    dok_tally_flush(tally, counters, nullptr);
    if (count_probes) dok_warp_add(counters + DOK_CNT_PROBES, probes);
  }
}

#define DOK_DISPATCH_SB(t, CALL)                        \
  switch ((t).sb) {                                     \
    case 32: { constexpr int SB = 32; CALL; break; }    \
    case 64: { constexpr int SB = 64; CALL; break; }    \
    case 128: { constexpr int SB = 128; CALL; break; }  \
    default: { constexpr int SB = 0; CALL; break; }     \
  }

// launch grid of a batch: one thread per row; sliced batches put the slice in gridDim.y
inline dim3 dok_grid(const RowKeys &k) {
  if (k.slice_rows == 0) return dim3((unsigned)((k.n + DOK_TPB - 1) / DOK_TPB));
  return dim3((unsigned)((k.slice_rows + DOK_TPB - 1) / DOK_TPB), (unsigned)(k.n / k.slice_rows));
}
inline dim3 dok_grid(const SelKeys &k) { return dim3((unsigned)((k.n + DOK_TPB - 1) / DOK_TPB)); }

template <class Keys>
inline int launch_get(const DevTable &t, const DevHash &hp, const Keys &keys, void *out_values, uint8_t *out_found,
                      const void *fallback, int64_t *counters, int count_probes, cudaStream_t st) {
  const ll_t n = keys.n;
  if (n == 0) return DOK_OK;
  Fallback fb;
  memset(&fb, 0, sizeof(fb));
  if (fallback) memcpy(&fb, fallback, (size_t)t.vb);
  const dim3 grid = dok_grid(keys);
  int rc = DOK_OK;
  if (t.vb <= 8 && t.sb <= 128) {   // tag and value fit the first 16 bytes of the slot: half the load width (or less)
    DOK_DISPATCH_SB(t, DOK_FOR_WINDOWS(t, rc, (k_get<(SB == 0 ? 32 : SB), 2, Keys><<<grid, DOK_TPB, 0, st>>>(
                                                  wt, hp, keys, (char *)out_values, out_found, fb, (ll_t *)counters, count_probes))));
  } else
    DOK_DISPATCH_SB(t, DOK_FOR_WINDOWS(t, rc, (k_get<SB, 4, Keys><<<grid, DOK_TPB, 0, st>>>(wt, hp, keys, (char *)out_values, out_found,
                                                                                           fb, (ll_t *)counters, count_probes))));
  return rc;
}

// ---------------------------------------------------------------------------------------------------------
// set
// ---------------------------------------------------------------------------------------------------------

// Value row of batch element e into its slot, and the key row too when this row claimed the slot.  A row that
// found its uuid already stored leaves the stored key alone: the reference rewrites it
// (closed_hashmap_impl_class.cu:384-386), but with the same bytes unless two different keys share a uuid, and every
// store to the table costs a request.  Floating-point keys are the exception -- their value cast makes different
// keys share a uuid as a rule -- so they are rewritten like in the reference.
template <class Keys, class Values>
__device__ __forceinline__ void dok_write_row(const DevTable &t, const DevHash &hp, const Keys &keys, const Values &values,
                                              ll_t e, ll_t slot, bool with_key) {
  if (with_key) keys.store_key(hp, e, dok_key_row(t, slot));
  dok_store_value(t, slot, values.row(t, e));
}

// One kernel, for batches whose rows have pairwise different uuids.
template <int SB, class Keys, class Values>
__global__ void __launch_bounds__(DOK_TPB, 4) k_set_unique(DevTable t, DevHash hp, Keys keys, Values values,
                                                        uint8_t *__restrict__ out_stored, ll_t *counters) {
  __shared__ BlockTally tally;
  if (keys.idle()) return;
  if (counters) dok_tally_begin(tally);
  ll_t e;
  bool active = keys.row(e);
  KeyHash kh{0, 0};
  if (active) kh = keys.hash(hp, e);
  active = dok_in_window(t, kh, active);
  int outcome = -1;
  const ll_t slot = dok_find_or_claim<SB>(t, kh, active, &outcome);
  if (active) {
    if (slot >= 0) dok_write_row(t, hp, keys, values, e, slot, outcome != DOK_OUT_FOUND || hp.dtype >= DOK_F16);
    if (out_stored) out_stored[e] = (uint8_t)(slot >= 0);
  }
  if (counters) {
    dok_tally_add(tally, DOK_CNT_CLAIMED_EMPTY, outcome == DOK_OUT_CLAIMED_EMPTY);
    dok_tally_add(tally, DOK_CNT_REUSED_REMOVED, outcome == DOK_OUT_REUSED);
    dok_tally_add(tally, DOK_CNT_FAILED, outcome == DOK_OUT_FAILED);
    dok_tally_add(tally, DOK_CNT_HITS, outcome == DOK_OUT_FOUND);
    dok_tally_flush(tally, counters, nullptr);
  }
}

// Stamp word of a slot during a general set: (epoch << 33) | (row << 1) | conflict.  The epoch of a call is
// larger than every epoch used on the table before, so an atomicMax leaves the LAST row of this batch that
// targets the slot; the low bit records that more than one row of the batch did.
__device__ __forceinline__ ll_t dok_stamp(ll_t epoch, ll_t row) { return (epoch << 33) | (row << 1); }

// First kernel of the general set.  Find or claim the slot, store the row there and raise the slot's stamp --
// for a batch without equal uuids that is all there is to do.  A row that finds the slot already stamped in
// this epoch sets the conflict bit and counts a duplicate (in slot_out[n], zeroed by the host before the
// launch); the second kernel then lets the slot's last row rewrite it.
template <int SB, class Keys, class Values>
__global__ void __launch_bounds__(DOK_TPB, 6) k_set_claim(DevTable t, DevHash hp, Keys keys, Values values,
                                                       ll_t *__restrict__ slot_out, ll_t epoch,
                                                       uint8_t *__restrict__ out_stored, ll_t *counters) {
  __shared__ BlockTally tally;
  if (keys.idle()) return;
  dok_tally_begin(tally);
  ll_t e;
  bool active = keys.row(e);
  KeyHash kh{0, 0};
  if (active) kh = keys.hash(hp, e);
  active = dok_in_window(t, kh, active);
  int outcome = -1, dup = 0;
  const ll_t slot = dok_find_or_claim<SB>(t, kh, active, &outcome);
  if (active) {
    slot_out[e] = slot;
    if (slot >= 0) {
      // the row is stored without waiting for the stamp's answer: the two requests travel together.  If the slot
      // turns out to be shared, whatever the racing stores left is rewritten by the second kernel.
      ll_t *stamp = dok_stamp_ptr(t, slot);
      dok_write_row(t, hp, keys, values, e, slot, outcome != DOK_OUT_FOUND || hp.dtype >= DOK_F16);
      const ll_t old = (ll_t)atomicMax(stamp, dok_stamp(epoch, e));
      if ((old >> 33) == epoch) {
        atomicOr((ull_t *)stamp, 1ULL);
        dup = 1;
      }
    }
    if (out_stored) out_stored[e] = (uint8_t)(slot >= 0);
  }
  dok_tally_add(tally, DOK_TALLY_EXTRA, dup);
  if (counters) {
    dok_tally_add(tally, DOK_CNT_CLAIMED_EMPTY, outcome == DOK_OUT_CLAIMED_EMPTY);
    dok_tally_add(tally, DOK_CNT_REUSED_REMOVED, outcome == DOK_OUT_REUSED);
    dok_tally_add(tally, DOK_CNT_FAILED, outcome == DOK_OUT_FAILED);
    dok_tally_add(tally, DOK_CNT_HITS, outcome == DOK_OUT_FOUND);
    dok_tally_add(tally, DOK_CNT_DUPLICATES, dup);
  }
  dok_tally_flush(tally, counters, slot_out + keys.count());
}

// Second kernel: does nothing unless the first one counted duplicates.  Then the row that owns a conflicted
// slot's stamp (the last row of the batch for that slot) rewrites key and value: one writer per slot, after
// every first-kernel write has completed, so rows cannot tear and the last row wins.
template <class Keys, class Values>
__global__ void __launch_bounds__(DOK_TPB) k_set_resolve(DevTable t, DevHash hp, Keys keys, Values values,
                                                         const ll_t *__restrict__ slot_in, ll_t epoch) {
  if (slot_in[keys.count()] == 0) return;        // the first kernel met no duplicate: every row is already in place
  if (keys.idle()) return;
  // a few blocks per SM stride over the rows: the usual launch has nothing to do, and a grid of one block per 256
  // rows would cost a millisecond at 2^28 rows just to find that out
  const ll_t span = keys.span(), stride = (ll_t)gridDim.x * DOK_TPB;
  for (ll_t j = (ll_t)blockIdx.x * DOK_TPB + threadIdx.x; j < span; j += stride) {
    ll_t e;
    if (!keys.at(j, e)) continue;
    const ll_t slot = slot_in[e];
    if (slot < 0) continue;
    if (t.win_hi != 0) {                         // windowed passes: by the slot's own group (each slot has one pass)
      const ll_t g = slot / t.spg;
      if (g < t.win_lo || g >= t.win_hi) continue;
    }
    if (__ldcg(dok_stamp_ptr(t, slot)) != (dok_stamp(epoch, e) | 1)) continue;
    dok_write_row(t, hp, keys, values, e, slot, true);
  }
}

// contiguous value rows [n, value_bytes]
template <class Keys, class Values>
inline int launch_set_general(const DevTable &t, const DevHash &hp, const Keys &keys, const Values &values,
                              int64_t *slot_scratch, int64_t epoch, uint8_t *out_stored, int64_t *counters, cudaStream_t st) {
  if (cudaMemsetAsync(slot_scratch + keys.n, 0, sizeof(int64_t), st) != cudaSuccess) return dok_check_launch();
  const dim3 grid = dok_grid(keys);
  int rc = DOK_OK;
  DOK_DISPATCH_SB(t, DOK_FOR_WINDOWS(t, rc, (k_set_claim<SB><<<grid, DOK_TPB, 0, st>>>(wt, hp, keys, values, (ll_t *)slot_scratch,
                                                                                       (ll_t)epoch, out_stored, (ll_t *)counters))));
  if (rc != DOK_OK) return rc;
  dim3 few = grid;
  if (few.x > 148 * 8) few.x = 148 * 8;
  DOK_FOR_WINDOWS(t, rc, (k_set_resolve<<<few, DOK_TPB, 0, st>>>(wt, hp, keys, values, (const ll_t *)slot_scratch, (ll_t)epoch)));
  return rc;
}

inline int launch_set(const DevTable &t, const DevHash &hp, const RowKeys &keys, const char *values, int64_t *slot_scratch,
                      int64_t epoch, uint8_t *out_stored, int64_t *counters, cudaStream_t st) {
  RowValues rv{values};
  return launch_set_general(t, hp, keys, rv, slot_scratch, epoch, out_stored, counters, st);
}

inline int launch_set_unique(const DevTable &t, const DevHash &hp, const RowKeys &keys, const char *values,
                             uint8_t *out_stored, int64_t *counters, cudaStream_t st) {
  RowValues rv{values};
  const dim3 grid = dok_grid(keys);
  int rc = DOK_OK;
  DOK_DISPATCH_SB(t, DOK_FOR_WINDOWS(t, rc, (k_set_unique<SB><<<grid, DOK_TPB, 0, st>>>(wt, hp, keys, rv, out_stored, (ll_t *)counters))));
  return rc;
}

// ---------------------------------------------------------------------------------------------------------
// remove / exists / count-new
// ---------------------------------------------------------------------------------------------------------

// REMOVE = 1: the tag is swapped to the tombstone by CAS so that equal uuids in one batch report exactly once
// (ClosedHashmap::remove, closed_hashmap_impl_class.cu:459-484, stores it non-atomically).
template <int SB, int REMOVE, class Keys>
__global__ void __launch_bounds__(DOK_TPB) k_find(DevTable t, DevHash hp, Keys keys, uint8_t *__restrict__ out_flags,
                                                  ll_t *counters) {
  __shared__ BlockTally tally;
  if (keys.idle()) return;
  if (counters) dok_tally_begin(tally);
  ll_t e;
  bool active = keys.row(e);
  KeyHash kh{0, 0};
  if (active) kh = keys.hash(hp, e);
  active = dok_in_window(t, kh, active);
  const Located loc = dok_locate<SB, 1, false>(t, kh, e, active, nullptr, NoEmit());
  int hit = active && loc.found >= 0;
  if (REMOVE && hit) hit = dok_cas_tag(t, loc.found, kh.uuid, DOK_REMOVED) == kh.uuid;
  if (active && out_flags) out_flags[e] = (uint8_t)hit;
  if (counters) {
    dok_tally_add(tally, DOK_CNT_HITS, hit);
    dok_tally_flush(tally, counters, nullptr);
  }
}

template <int REMOVE, class Keys>
inline int launch_find(const DevTable &t, const DevHash &hp, const Keys &keys, uint8_t *out_flags, int64_t *counters,
                       cudaStream_t st) {
  const dim3 grid = dok_grid(keys);
  int rc = DOK_OK;
  DOK_DISPATCH_SB(t, DOK_FOR_WINDOWS(t, rc, (k_find<SB, REMOVE><<<grid, DOK_TPB, 0, st>>>(wt, hp, keys, out_flags, (ll_t *)counters))));
  return rc;
}

static __global__ void k_fill_i64(ll_t *p, ll_t n, ll_t v) {
  for (ll_t i = (ll_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (ll_t)gridDim.x * blockDim.x) p[i] = v;
}

// Rows absent from the table insert their uuid into a scratch tag set; the number of successful claims is the
// number of distinct absent uuids.
template <int SB, class Keys>
__global__ void __launch_bounds__(DOK_TPB) k_count_new(DevTable t, DevHash hp, Keys keys, ll_t *__restrict__ scratch,
                                                       ll_t scratch_slots, ll_t *counters) {
  __shared__ BlockTally tally;
  if (keys.idle()) return;
  dok_tally_begin(tally);
  ll_t e;
  bool active = keys.row(e);
  KeyHash kh{0, 0};
  if (active) kh = keys.hash(hp, e);
  active = dok_in_window(t, kh, active);
  const Located loc = dok_locate<SB, 1, false>(t, kh, e, active, nullptr, NoEmit());
  int claimed = 0;
  if (active && loc.found < 0) {
    const ll_t uuid = kh.uuid;
    ll_t slot = (ll_t)__umul64hi(dok_mix64((ull_t)uuid ^ 0x5851f42d4c957f2dULL), (ull_t)scratch_slots);
    for (ll_t i = 0; i < scratch_slots; i++) {
      ll_t tag = __ldcg(&scratch[slot]);
      if (tag == DOK_EMPTY) {
        tag = (ll_t)atomicCAS((ull_t *)&scratch[slot], (ull_t)DOK_EMPTY, (ull_t)uuid);
        if (tag == DOK_EMPTY) { claimed = 1; break; }
      }
      if (tag == uuid) break;
      if (++slot == scratch_slots) slot = 0;
    }
  }
  dok_tally_add(tally, DOK_CNT_CLAIMED_EMPTY, claimed);
  dok_tally_flush(tally, counters, nullptr);
}

// ---------------------------------------------------------------------------------------------------------
// rehash: live slots of one table straight into another
// ---------------------------------------------------------------------------------------------------------

// One thread per SOURCE slot: the stored key row of a live slot is hashed with the destination's parameters and
// inserted, key bytes and value copied as they are (both tables store key element i in column perm[i]).  Replaces
// the reference's rehash = two boolean-mask gathers plus a full `set` with its pre-get and unique
// (cuda_closed_hashmap.py:456-468) and this library's own compaction + insert.  Live keys are pairwise different,
// so every row claims a fresh slot; tombstones stay behind.
template <int SB>
__global__ void __launch_bounds__(DOK_TPB) k_reinsert(DevTable src, DevTable dst, DevHash hp, ll_t *counters) {
  const ll_t stride = (ll_t)gridDim.x * DOK_TPB;
  int claimed = 0, failed = 0;
  for (ll_t base = (ll_t)blockIdx.x * DOK_TPB; base < src.nb; base += stride) {       // uniform over the block
    const ll_t s = base + threadIdx.x;
    bool active = false;
    if (s < src.nb) active = dok_load_tag(src, s) >= 0;   // uuids are non-negative; empty, tombstone, padding are not
    KeyHash kh{0, 0};
    const char *krow = dok_key_row(src, active ? s : 0);
    if (active) {
      ll_t k = dok_key_elem(krow, hp.dtype, hp.perm[0]);
      ll_t u = dok_uuid_term(k, hp.a[0], hp.b[0], hp.p[0], hp.m[0]);
      ull_t h = (ull_t)k * (ull_t)hp.a1[0] + (ull_t)hp.b1[0];
      for (int i = 1; i < hp.ks; i++) {
        k = dok_key_elem(krow, hp.dtype, hp.perm[i]);
        u = (ll_t)((ull_t)u * (ull_t)dok_uuid_term(k, hp.a[i], hp.b[i], hp.p[i], hp.m[i]));
        h *= (ull_t)k * (ull_t)hp.a1[i] + (ull_t)hp.b1[i];
      }
      kh = KeyHash{dok_llabs(u), (ll_t)h};
    }
    active = dok_in_window(dst, kh, active);
    int outcome = -1;
    const ll_t slot = dok_find_or_claim<SB>(dst, kh, active, &outcome);
    if (active && slot >= 0) {
      char *drow = dok_key_row(dst, slot);
      if ((dst.kb & 7) == 0) for (int i = 0; i < (dst.kb >> 3); i++) ((ull_t *)drow)[i] = ((const ull_t *)krow)[i];
      else if ((dst.kb & 3) == 0) for (int i = 0; i < (dst.kb >> 2); i++) ((unsigned *)drow)[i] = ((const unsigned *)krow)[i];
      else if ((dst.kb & 1) == 0) for (int i = 0; i < (dst.kb >> 1); i++) ((unsigned short *)drow)[i] = ((const unsigned short *)krow)[i];
      else for (int i = 0; i < dst.kb; i++) drow[i] = krow[i];
      dok_store_value(dst, slot, dok_value_ptr(src, s));
    }
    claimed += outcome == DOK_OUT_CLAIMED_EMPTY || outcome == DOK_OUT_REUSED;
    failed += outcome == DOK_OUT_FAILED;
  }
  if (counters) {
    dok_warp_add(counters + DOK_CNT_CLAIMED_EMPTY, claimed);
    dok_warp_add(counters + DOK_CNT_FAILED, failed);
  }
}

// ---------------------------------------------------------------------------------------------------------
// init / uuid
// ---------------------------------------------------------------------------------------------------------

static __global__ void k_init(DevTable t) {
  const ll_t stride = (ll_t)gridDim.x * blockDim.x;
  for (ll_t i = (ll_t)blockIdx.x * blockDim.x + threadIdx.x; i < t.n_slots; i += stride) {
    *dok_tag_ptr(t, i) = i < t.nb ? DOK_EMPTY : DOK_BLOCKED;
    if (t.stamp_off >= 0 || t.stamp) *dok_stamp_ptr(t, i) = 0;
  }
}

template <class Keys>
__global__ void k_uuid(DevTable t, DevHash hp, Keys keys, ll_t *uuid_out, ll_t *slot_out) {
  const ll_t e = (ll_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= keys.count()) return;
  const KeyHash kh = keys.hash(hp, e);
  if (uuid_out) uuid_out[e] = kh.uuid;
  if (slot_out) slot_out[e] = t.n_groups > 0 ? dok_start_group(kh, t) * t.spg : 0;
}

// ---------------------------------------------------------------------------------------------------------
// compaction of live slots in slot order
// ---------------------------------------------------------------------------------------------------------
#define DOK_COMPACT_ROUNDS 8
#define DOK_COMPACT_TILE (DOK_TPB * DOK_COMPACT_ROUNDS)

__device__ __forceinline__ bool dok_is_live(ll_t tag) { return tag != DOK_EMPTY && tag != DOK_REMOVED && tag != DOK_BLOCKED; }

static __global__ void __launch_bounds__(DOK_TPB) k_compact_count(DevTable t, ll_t *tile_counts) {
  __shared__ int warp_sums[DOK_TPB / 32];
  const ll_t base = (ll_t)blockIdx.x * DOK_COMPACT_TILE;
  int c = 0;
#pragma unroll
  for (int r = 0; r < DOK_COMPACT_ROUNDS; r++) {
    const ll_t slot = base + r * DOK_TPB + threadIdx.x;
    if (slot < t.nb) c += dok_is_live(__ldcs(dok_tag_ptr(t, slot)));
  }
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    int s = 0;
    for (int w = 0; w < DOK_TPB / 32; w++) s += warp_sums[w];
    tile_counts[blockIdx.x] = s;
  }
}

// In-place exclusive scan of a[0..n) by one block; a[n] receives the total.
static __global__ void __launch_bounds__(1024) k_exclusive_scan(ll_t *a, ll_t n) {
  __shared__ ll_t partial[1024];
  const ll_t per = (n + 1023) / 1024;
  const ll_t lo = threadIdx.x * per, hi = lo + per < n ? lo + per : n;
  ll_t s = 0;
  for (ll_t i = lo; i < hi; i++) s += a[i];
  partial[threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    ll_t run = 0;
    for (int i = 0; i < 1024; i++) { const ll_t v = partial[i]; partial[i] = run; run += v; }
    a[n] = run;
  }
  __syncthreads();
  ll_t run = partial[threadIdx.x];
  for (ll_t i = lo; i < hi; i++) { const ll_t v = a[i]; a[i] = run; run += v; }
}

static __global__ void __launch_bounds__(DOK_TPB) k_compact_scatter(DevTable t, DevHash hp, const ll_t *__restrict__ tile_offsets,
                                                             ll_t total_tiles, char *keys_out, int keys_transposed,
                                                             char *values_out, ll_t *uuid_out) {
  __shared__ int warp_sums[DOK_TPB / 32];
  __shared__ int round_base;
  const ll_t base = (ll_t)blockIdx.x * DOK_COMPACT_TILE;
  const ll_t count = tile_offsets[total_tiles];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) round_base = 0;
  __syncthreads();
  const ll_t tile_out = tile_offsets[blockIdx.x];
  for (int r = 0; r < DOK_COMPACT_ROUNDS; r++) {
    const ll_t slot = base + r * DOK_TPB + threadIdx.x;
    ll_t tag = DOK_EMPTY;
    if (slot < t.nb) tag = __ldcs(dok_tag_ptr(t, slot));
    const bool live = dok_is_live(tag);
    const unsigned ballot = __ballot_sync(0xffffffffu, live);
    if (lane == 0) warp_sums[warp] = __popc(ballot);
    __syncthreads();
    int before = round_base;
    for (int w = 0; w < warp; w++) before += warp_sums[w];
    before += __popc(ballot & ((1u << lane) - 1u));
    if (live) {
      const ll_t pos = tile_out + before;
      if (uuid_out) uuid_out[pos] = tag;
      if (values_out) dok_load_value(t, slot, values_out + pos * (ll_t)t.vb);
      if (keys_out) {
        // keys(): column i of the output is storage column key_perm[i] (cuda_closed_hashmap.py:165)
        const char *src = dok_key_row(t, slot);
        for (int i = 0; i < hp.ks; i++) {
          const ll_t o = keys_transposed ? ((ll_t)i * count + pos) : (pos * hp.ks + i);
          switch (hp.elem_bytes) {
            case 8: ((ll_t *)keys_out)[o] = ((const ll_t *)src)[hp.perm[i]]; break;
            case 4: ((int *)keys_out)[o] = ((const int *)src)[hp.perm[i]]; break;
            case 2: ((short *)keys_out)[o] = ((const short *)src)[hp.perm[i]]; break;
            default: keys_out[o] = src[hp.perm[i]]; break;
          }
        }
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int s = 0;
      for (int w = 0; w < DOK_TPB / 32; w++) s += warp_sums[w];
      round_base += s;
    }
    __syncthreads();
  }
}

