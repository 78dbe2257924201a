// Kernel templates of the closed-hashing map: batched get / set / remove / exists / count-new and the
// compaction of live slots.  They are templated on the key source (contiguous key rows, or index tensors of a
// DOK selector) so that the map entry points (map_api.cu) and the fused DOK entry points (dok_api.cu) share them.
// One CUDA thread handles one batch element, as in the reference kernels
// (sparse_dok/components/cuda/closed_hashmap_impl.cu), but each hit costs one bucket row (tag + value in the
// same 32-byte sector), misses write the fallback from the kernel, and counters are accumulated on the device
// so that the host never has to synchronise.
#pragma once
#include "dok_host.cuh"

// ---------------------------------------------------------------------------------------------------------
// get
// ---------------------------------------------------------------------------------------------------------

// 16-byte load that allocates in L2 only: the table is touched at random, L1 lines would be dead on arrival.
__device__ __forceinline__ ulonglong2 dok_ld16(const char *p) {
  return __ldcg((const ulonglong2 *)p);
}

// Writes `vb` bytes of a value held in the registers w[0..NW) to an output row.
template <int NW>
__device__ __forceinline__ void dok_store_out(char *dst, const ull_t (&w)[NW], int vb) {
  if ((vb & 7) == 0) {
#pragma unroll
    for (int i = 0; i < NW; i++) if (i * 8 < vb) ((ull_t *)dst)[i] = w[i];
  } else if ((vb & 3) == 0) {
#pragma unroll
    for (int i = 0; i < NW * 2; i++) if (i * 4 < vb) ((unsigned *)dst)[i] = (unsigned)(w[i >> 1] >> ((i & 1) * 32));
  } else if ((vb & 1) == 0) {
#pragma unroll
    for (int i = 0; i < NW * 4; i++) if (i * 2 < vb) ((unsigned short *)dst)[i] = (unsigned short)(w[i >> 2] >> ((i & 3) * 16));
  } else {
#pragma unroll
    for (int i = 0; i < NW * 8; i++) if (i < vb) dst[i] = (char)(w[i >> 3] >> ((i & 7) * 8));
  }
}

// UNITS = bucket_bytes / 16 for 1 and 2 (the value then lives in registers after one or two 16-byte loads of
// the probed row); UNITS = 0 is the generic path for wider rows.
template <int UNITS, class Keys>
__global__ void __launch_bounds__(DOK_TPB) k_get(DevTable t, DevHash hp, Keys keys, char *__restrict__ out_values,
                                                 uint8_t *__restrict__ out_found, Fallback fb, ll_t *counters,
                                                 int count_probes) {
  const ll_t e = (ll_t)blockIdx.x * DOK_TPB + threadIdx.x;
  int hit = 0, probes = 0;
  if (e < keys.count()) {
    const KeyHash kh = keys.hash(hp, e);
    const ll_t uuid = kh.uuid;
    char *dst = out_values + e * (ll_t)t.vb;
    if (UNITS == 1 || UNITS == 2) {
      constexpr int NW = UNITS == 1 ? 1 : 3;
      ull_t w[NW];
      ll_t slot = dok_start_bucket(kh, t.nb, t.nb_magic);
      for (ll_t i = 0; i < t.nb; i++) {
        const char *row = t.buckets + slot * (ll_t)(UNITS * 16);
        const ulonglong2 u0 = dok_ld16(row);
        ulonglong2 u1;
        if (UNITS == 2) u1 = dok_ld16(row + 16);
        probes++;
        const ll_t tag = (ll_t)u0.x;
        if (tag == uuid) {
          w[0] = u0.y;
          if (UNITS == 2) { w[1] = u1.x; w[2] = u1.y; }
          hit = 1;
          break;
        }
        if (tag == DOK_EMPTY) break;
        if (++slot == t.nb) slot = 0;
      }
      if (hit) dok_store_out<NW>(dst, w, t.vb);
      else dok_store_fallback(t, fb, dst);
    } else {
      const ll_t slot = dok_find(t, kh, &probes);
      hit = slot >= 0;
      if (hit) dok_load_value(t, slot, dst);
      else dok_store_fallback(t, fb, dst);
    }
    if (out_found) out_found[e] = (uint8_t)hit;
  }
  if (counters) {
    dok_warp_add(counters + DOK_CNT_HITS, hit);
    if (count_probes) dok_warp_add(counters + DOK_CNT_PROBES, probes);
  }
}

template <class Keys>
inline int launch_get(const DevTable &t, const DevHash &hp, const Keys &keys, void *out_values, uint8_t *out_found,
                      const void *fallback, int64_t *counters, int count_probes, cudaStream_t st) {
  const ll_t n = keys.n;
  if (n == 0) return DOK_OK;
  Fallback fb;
  memset(&fb, 0, sizeof(fb));
  if (fallback) memcpy(&fb, fallback, (size_t)t.vb);
  const unsigned grid = (unsigned)((n + DOK_TPB - 1) / DOK_TPB);
  if (t.bb == 16)
    k_get<1, Keys><<<grid, DOK_TPB, 0, st>>>(t, hp, keys, (char *)out_values, out_found, fb, (ll_t *)counters, count_probes);
  else if (t.bb == 32)
    k_get<2, Keys><<<grid, DOK_TPB, 0, st>>>(t, hp, keys, (char *)out_values, out_found, fb, (ll_t *)counters, count_probes);
  else
    k_get<0, Keys><<<grid, DOK_TPB, 0, st>>>(t, hp, keys, (char *)out_values, out_found, fb, (ll_t *)counters, count_probes);
  return dok_check_launch();
}

// ---------------------------------------------------------------------------------------------------------
// set
// ---------------------------------------------------------------------------------------------------------

template <class Keys, class Values>
__global__ void __launch_bounds__(DOK_TPB) k_set_unique(DevTable t, DevHash hp, Keys keys, Values values,
                                                        uint8_t *__restrict__ out_stored, ll_t *counters) {
  const ll_t e = (ll_t)blockIdx.x * DOK_TPB + threadIdx.x;
  int outcome = -1;
  if (e < keys.count()) {
    const ll_t slot = dok_find_or_claim(t, keys.hash(hp, e), &outcome);
    if (slot >= 0) {
      keys.store_key(hp, e, t.keys + slot * (ll_t)t.kb);
      dok_store_value(t, slot, values.row(t, e));
    }
    if (out_stored) out_stored[e] = (uint8_t)(slot >= 0);
  }
  if (counters) {
    dok_warp_add(counters + DOK_CNT_CLAIMED_EMPTY, outcome == DOK_OUT_CLAIMED_EMPTY);
    dok_warp_add(counters + DOK_CNT_REUSED_REMOVED, outcome == DOK_OUT_REUSED);
    dok_warp_add(counters + DOK_CNT_FAILED, outcome == DOK_OUT_FAILED);
    dok_warp_add(counters + DOK_CNT_HITS, outcome == DOK_OUT_FOUND);
  }
}

// First kernel of the general set: find or claim the slot, remember it, and raise the slot's stamp to
// (epoch << 32 | row).  The stamp of a slot can only have been written with a smaller epoch before this
// call, so after the kernel it names the LAST row of this batch that targets the slot.
template <class Keys>
__global__ void __launch_bounds__(DOK_TPB) k_set_claim(DevTable t, DevHash hp, Keys keys, ll_t *__restrict__ slot_out,
                                                       ll_t epoch, ll_t *counters) {
  const ll_t e = (ll_t)blockIdx.x * DOK_TPB + threadIdx.x;
  int outcome = -1, dup = 0;
  if (e < keys.count()) {
    const ll_t slot = dok_find_or_claim(t, keys.hash(hp, e), &outcome);
    slot_out[e] = slot;
    if (slot >= 0) {
      const ll_t mine = (epoch << 32) | e;
      const ll_t old = (ll_t)atomicMax((ll_t *)&t.stamp[slot], mine);
      dup = (old >> 32) == epoch;   // another row of this batch already stamped the slot
    }
  }
  if (counters) {
    dok_warp_add(counters + DOK_CNT_CLAIMED_EMPTY, outcome == DOK_OUT_CLAIMED_EMPTY);
    dok_warp_add(counters + DOK_CNT_REUSED_REMOVED, outcome == DOK_OUT_REUSED);
    dok_warp_add(counters + DOK_CNT_FAILED, outcome == DOK_OUT_FAILED);
    dok_warp_add(counters + DOK_CNT_HITS, outcome == DOK_OUT_FOUND);
    dok_warp_add(counters + DOK_CNT_DUPLICATES, dup);
  }
}

// Second kernel: the row whose index equals the slot's stamp writes key and value; every other row of the
// batch that targeted the slot lost to a later duplicate.  One writer per slot: rows cannot tear.
template <class Keys, class Values>
__global__ void __launch_bounds__(DOK_TPB) k_set_write(DevTable t, DevHash hp, Keys keys, Values values,
                                                       const ll_t *__restrict__ slot_in, ll_t epoch,
                                                       uint8_t *__restrict__ out_stored) {
  const ll_t e = (ll_t)blockIdx.x * DOK_TPB + threadIdx.x;
  if (e >= keys.count()) return;
  const ll_t slot = slot_in[e];
  if (out_stored) out_stored[e] = (uint8_t)(slot >= 0);
  if (slot < 0) return;
  if (__ldcg(&t.stamp[slot]) != ((epoch << 32) | e)) return;
  keys.store_key(hp, e, t.keys + slot * (ll_t)t.kb);
  dok_store_value(t, slot, values.row(t, e));
}

// ---------------------------------------------------------------------------------------------------------
// remove / exists / count-new
// ---------------------------------------------------------------------------------------------------------

// REMOVE = 1: the tag is swapped to the tombstone by CAS so that equal uuids in one batch report exactly once
// (ClosedHashmap::remove, closed_hashmap_impl_class.cu:459-484, stores it non-atomically).
template <int REMOVE, class Keys>
__global__ void __launch_bounds__(DOK_TPB) k_find(DevTable t, DevHash hp, Keys keys, uint8_t *__restrict__ out_flags,
                                                  ll_t *counters) {
  const ll_t e = (ll_t)blockIdx.x * DOK_TPB + threadIdx.x;
  int hit = 0;
  if (e < keys.count()) {
    const KeyHash kh = keys.hash(hp, e);
    const ll_t slot = dok_find(t, kh, nullptr);
    hit = slot >= 0;
    if (REMOVE && hit) hit = dok_cas_tag(t, slot, kh.uuid, DOK_REMOVED) == kh.uuid;
    if (out_flags) out_flags[e] = (uint8_t)hit;
  }
  dok_warp_add(counters ? counters + DOK_CNT_HITS : nullptr, hit);
}

static __global__ void k_fill_i64(ll_t *p, ll_t n, ll_t v) {
  for (ll_t i = (ll_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (ll_t)gridDim.x * blockDim.x) p[i] = v;
}

// Rows absent from the table insert their uuid into a scratch tag set; the number of successful claims is the
// number of distinct absent uuids.
template <class Keys>
__global__ void __launch_bounds__(DOK_TPB) k_count_new(DevTable t, DevHash hp, Keys keys, ll_t *__restrict__ scratch,
                                                       ll_t scratch_slots, ll_t *counters) {
  const ll_t e = (ll_t)blockIdx.x * DOK_TPB + threadIdx.x;
  int claimed = 0;
  if (e < keys.count()) {
    const KeyHash kh = keys.hash(hp, e);
    const ll_t uuid = kh.uuid;
    if (dok_find(t, kh, nullptr) < 0) {
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
  }
  dok_warp_add(counters + DOK_CNT_CLAIMED_EMPTY, claimed);
}

// ---------------------------------------------------------------------------------------------------------
// init / uuid
// ---------------------------------------------------------------------------------------------------------

static __global__ void k_init(DevTable t) {
  const ll_t stride = (ll_t)gridDim.x * blockDim.x;
  for (ll_t i = (ll_t)blockIdx.x * blockDim.x + threadIdx.x; i < t.nb; i += stride) {
    *dok_tag_ptr(t, i) = DOK_EMPTY;
    if (t.stamp) t.stamp[i] = 0;
  }
}

template <class Keys>
__global__ void k_uuid(DevTable t, DevHash hp, Keys keys, ll_t *uuid_out, ll_t *bucket_out) {
  const ll_t e = (ll_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= keys.count()) return;
  const KeyHash kh = keys.hash(hp, e);
  if (uuid_out) uuid_out[e] = kh.uuid;
  if (bucket_out) bucket_out[e] = t.nb > 0 ? dok_start_bucket(kh, t.nb, t.nb_magic) : 0;
}

// ---------------------------------------------------------------------------------------------------------
// compaction of live slots in slot order
// ---------------------------------------------------------------------------------------------------------
#define DOK_COMPACT_ROUNDS 8
#define DOK_COMPACT_TILE (DOK_TPB * DOK_COMPACT_ROUNDS)

__device__ __forceinline__ bool dok_is_live(ll_t tag) { return tag != DOK_EMPTY && tag != DOK_REMOVED; }

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
        const char *src = t.keys + slot * (ll_t)t.kb;
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

