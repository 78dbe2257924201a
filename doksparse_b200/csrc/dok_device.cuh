// Device-side building blocks shared by the kernels of libdoksparse.so (sm_100a).
//
// Semantics follow the reference's ClosedHashmap class
// (sparse_dok/components/cuda/closed_hashmap_impl_class.cu): key identity is the 64-bit uuid, tags are
// uuid / -1 (empty) / -3 (tombstone), probing is linear, a lookup stops at the first empty tag and steps
// over tombstones.  What differs on purpose is the memory layout and the start slot.
//
// Layout.  On B200, when the table is much larger than L2, every load / store / atomic INSTRUCTION-LANE that
// touches it costs the same (~48 G per second over the whole GPU, measured; a second access to a sector that
// was just read costs as much as a new random line), while lanes of one instruction that fall into the same
// 128-byte line count once.  So an operation should touch its line with as few instructions as possible, and
// adjacent lanes should share them.  A slot is {int64 tag | value | key row | stamp (if room)} padded to 32, 64
// or 128 bytes (tag first, value right behind it), a 128-byte line is a GROUP of 4, 2 or 1 slots, and probing
// starts at a group boundary.  The four
// lanes of a quad read one group with ONE coalesced 128-byte request (32 bytes per lane) and resolve a lookup
// from registers: tags, value and key of all its slots are then on chip.  The probe order is still plain linear
// probing over slots (group after group); only the start is aligned.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "../../include/doksparse.h"

typedef long long ll_t;
typedef unsigned long long ull_t;

#define DOK_EMPTY (-1LL)
#define DOK_REMOVED (-3LL)
#define DOK_TPB 256

// ---------------------------------------------------------------------------------------------------------
// Hash parameters in device-ready form: already permuted by key_perm (element i of the caller's key row uses
// a[i], b[i], p[i]) and with a magic reciprocal per prime so that the truncated remainder needs no division.
// ---------------------------------------------------------------------------------------------------------
struct DevHash {
  int ks;                       // key elements per row
  int dtype;                    // dok_dtype of the key rows
  int elem_bytes;               // bytes of one key element
  int pad_;
  ll_t a[DOK_MAX_KEY_SIZE];     // alpha2[key_perm[i]]   -- second hash: the uuid (key identity)
  ll_t b[DOK_MAX_KEY_SIZE];     // beta2[key_perm[i]]
  ull_t p[DOK_MAX_KEY_SIZE];    // |prime2[key_perm[i]]|  (>= 2)
  ull_t m[DOK_MAX_KEY_SIZE];    // floor(2^64 / p)
  ll_t a1[DOK_MAX_KEY_SIZE];    // alpha1[key_perm[i]], forced odd -- first-hash terms: they only decorrelate the
  ll_t b1[DOK_MAX_KEY_SIZE];    // beta1[key_perm[i]]                 probe chains of keys whose uuids collide
  int perm[DOK_MAX_KEY_SIZE];   // storage column of key element i
};

struct KeyHash { ll_t uuid; ll_t hash1; };   // hash1: product of the linear first-hash terms (see dok_start_group)

struct DevTable {
  char *slots;      // n_slots * sb bytes, 128-byte aligned
  ll_t *stamp;      // [n_slots] duplicate-resolution stamps when they do not fit in the slot, else nullptr
  ll_t nb;          // slots the caller sees (0 .. nb-1); slots nb .. n_slots-1 are blocked padding
  ll_t n_slots;     // n_groups * spg
  ll_t n_groups;    // probe groups: 128-byte lines of spg slots (sb <= 128), single slots otherwise
  int sb;           // slot bytes: 32, 64, 128, or a larger multiple of 128
  int spg;          // slots per group: 128 / sb, or 1 for sb > 128
  int vb;           // value bytes
  int kb;           // key row bytes
  int val_off;      // slot offset of the value: always 8, right behind the tag
  int key_off;      // slot offset of the key row: 8 + round_up(vb, 8)
  int stamp_off;    // slot offset of the stamp (behind the key row), -1 when `stamp` is a separate array
  int vwords;       // ceil(vb / 8)
  // Window of probe groups served by this launch; win_hi == 0: the whole table.  A slot array larger than the
  // reach of the GPU's TLB (64 GiB of 2 MiB pages on B200: random reads fall from 45 G/s to 13 G/s at 114 GB) is
  // worked through in passes, each pass taking only the rows whose chain STARTS inside its window, so that one
  // pass touches a range the TLB covers.
  ll_t win_lo, win_hi;
};

#define DOK_BLOCKED (-2LL)   // tag of padding slots: never empty, never a tombstone, never a uuid (uuids are >= 0)

// One factor of the uuid product: ((int64)k * a + b) % p with wrapping arithmetic and the C remainder
// (sign of the dividend), closed_hashmap_impl_class.cu:100,103.  q = mulhi(|x|, floor(2^64/p)) is
// floor(|x|/p) or one less, so a single conditional subtraction finishes the remainder.
__device__ __forceinline__ ll_t dok_uuid_term(ll_t k, ll_t a, ll_t b, ull_t p, ull_t m) {
  const ll_t x = (ll_t)((ull_t)k * (ull_t)a + (ull_t)b);
  const ull_t ux = x < 0 ? (0ULL - (ull_t)x) : (ull_t)x;
  const ull_t q = __umul64hi(ux, m);
  ull_t r = ux - q * p;
  if (r >= p) r -= p;
  return x < 0 ? -(ll_t)r : (ll_t)r;
}

__device__ __forceinline__ ll_t dok_llabs(ll_t v) {  // llabs; INT64_MIN stays INT64_MIN like the device's
  return v < 0 ? (ll_t)(0ULL - (ull_t)v) : v;
}

// `(ll_t) key[i]`: the reference converts key elements by VALUE (closed_hashmap_impl_class.cu:89-103), so a
// float key is truncated toward zero.  The plain C++ casts below compile to the same conversions the
// reference's JIT build uses.
__device__ __forceinline__ ll_t dok_key_elem(const void *keys, int dtype, ll_t idx) {
  switch (dtype) {
    case DOK_I64: return ((const ll_t *)keys)[idx];
    case DOK_I32: return (ll_t)((const int *)keys)[idx];
    case DOK_F32: return (ll_t)((const float *)keys)[idx];
    case DOK_I16: return (ll_t)((const short *)keys)[idx];
    case DOK_I8: return (ll_t)((const signed char *)keys)[idx];
    case DOK_U8: return (ll_t)((const unsigned char *)keys)[idx];
    case DOK_F64: return (ll_t)((const double *)keys)[idx];
    case DOK_F16: return __half2ll_rz(((const __half *)keys)[idx]);
    default: return (ll_t)__bfloat162float(((const __nv_bfloat16 *)keys)[idx]);
  }
}

// Mixer (the 64-bit finaliser of MurmurHash3); with a multiply-high range reduction any table size works
// without a modulo.
__device__ __forceinline__ ull_t dok_mix64(ull_t h) {
  h ^= h >> 33; h *= 0xff51afd7ed558ccdULL;
  h ^= h >> 33; h *= 0xc4ceb9fe1a85ec53ULL;
  h ^= h >> 33;
  return h;
}
// Start group.  In the reference two keys whose uuids collide are still told apart as long as their probe
// chains (first hash modulo n_buckets) do not meet; a uuid collision is not rare there, because alpha2 may be
// drawn as 0 (cuda_closed_hashmap.py:100), which makes one key element drop out of the uuid.  To keep that
// property the start group mixes the uuid with a second function of the key built from the first hash's
// parameters, prod_i (key_i * (alpha1_i | 1) + beta1_i) (wrapping, no modulo: it only has to differ where the
// keys differ): keys that collide in the uuid alone get unrelated chains.
__device__ __forceinline__ ll_t dok_start_group(const KeyHash &h, const DevTable &t) {
  return (ll_t)__umul64hi(dok_mix64((ull_t)h.uuid ^ ((ull_t)h.hash1 * 0x9e3779b97f4a7c15ULL)), (ull_t)t.n_groups);
}
// does this launch serve the row?  (rows outside the window belong to another pass over the same batch)
__device__ __forceinline__ bool dok_in_window(const DevTable &t, const KeyHash &h, bool active) {
  if (t.win_hi == 0 || !active) return active;
  const ll_t g = dok_start_group(h, t);
  return g >= t.win_lo && g < t.win_hi;
}
#define DOK_SHARD_SALT 0x9e3779b97f4a7c15ULL
__device__ __forceinline__ int dok_owner_shard(ll_t uuid, int n_shards) {
  return (int)__umul64hi(dok_mix64((ull_t)uuid ^ DOK_SHARD_SALT), (ull_t)n_shards);
}

// ---------------------------------------------------------------------------------------------------------
// Key sources.  A key source yields, for batch element e, the uuid of its key and can write the key's raw
// bytes into a table key row.  Keys are never held in a register array (key_size is a run-time value):
// elements are re-read where needed, which stays in L1.
// ---------------------------------------------------------------------------------------------------------
struct RowKeys {          // contiguous [n, ks] rows of the key dtype (closed_hashmap_impl.cu:51-60)
  const void *keys;
  ll_t n;
  // Sliced batches (the inbox of a sharded table): the rows come as gridDim.y slices of `slice_rows` rows each, of
  // which only the first slice_counts[y] are in use -- a count that only the DEVICE knows at launch time (another
  // GPU wrote it), so the grid covers whole slices and blocks beyond the count leave at once.  A non-zero *abort
  // (the exchange overflowed somewhere) turns the launch into a no-op.  Batch element e = y * slice_rows + row.
  ll_t slice_rows = 0;
  const ll_t *slice_counts = nullptr;
  const ll_t *abort = nullptr;
  __device__ __forceinline__ ll_t count() const { return n; }
  // batch element of the calling thread and whether it exists
  __device__ __forceinline__ bool row(ll_t &e) const {
    const ll_t j = (ll_t)blockIdx.x * DOK_TPB + threadIdx.x;
    if (slice_rows == 0) { e = j; return j < n; }
    e = (ll_t)blockIdx.y * slice_rows + j;
    return j < slice_rows && j < slice_counts[blockIdx.y];
  }
  // the same for position j of the batch (of slice blockIdx.y), for kernels that stride over the rows
  __device__ __forceinline__ bool at(ll_t j, ll_t &e) const {
    if (slice_rows == 0) { e = j; return j < n; }
    e = (ll_t)blockIdx.y * slice_rows + j;
    return j < slice_rows && j < slice_counts[blockIdx.y];
  }
  __device__ __forceinline__ ll_t span() const { return slice_rows == 0 ? n : slice_rows; }
  // block-uniform: nothing for this block to do
  __device__ __forceinline__ bool idle() const {
    if (slice_rows == 0) return false;
    if (abort != nullptr && *abort != 0) return true;
    return (ll_t)blockIdx.x * DOK_TPB >= slice_counts[blockIdx.y];
  }
  // get_uuid of the reference (closed_hashmap_impl_class.cu:98-107) and the chain-decorrelating product, in one
  // pass over the key
  __device__ __forceinline__ KeyHash hash(const DevHash &hp, ll_t e) const {
    if (hp.ks == 1 && hp.dtype == DOK_I64) {          // the common case, kept free of loops and type dispatch
      const ll_t k = ((const ll_t *)keys)[e];
      return KeyHash{dok_llabs(dok_uuid_term(k, hp.a[0], hp.b[0], hp.p[0], hp.m[0])),
                     (ll_t)((ull_t)k * (ull_t)hp.a1[0] + (ull_t)hp.b1[0])};
    }
    ll_t k = dok_key_elem(keys, hp.dtype, e * hp.ks);
    ll_t u = dok_uuid_term(k, hp.a[0], hp.b[0], hp.p[0], hp.m[0]);
    ull_t h = (ull_t)k * (ull_t)hp.a1[0] + (ull_t)hp.b1[0];
    for (int i = 1; i < hp.ks; i++) {
      k = dok_key_elem(keys, hp.dtype, e * hp.ks + i);
      u = (ll_t)((ull_t)u * (ull_t)dok_uuid_term(k, hp.a[i], hp.b[i], hp.p[i], hp.m[i]));
      h *= (ull_t)k * (ull_t)hp.a1[i] + (ull_t)hp.b1[i];
    }
    return KeyHash{dok_llabs(u), (ll_t)h};
  }
  // set_key_permuted (closed_hashmap_impl_class.cu:144-150): storage column perm[i] <- key element i
  __device__ __forceinline__ void store_key(const DevHash &hp, ll_t e, char *dst_row) const {
    const char *src = (const char *)keys + e * (ll_t)hp.ks * hp.elem_bytes;
    switch (hp.elem_bytes) {
      case 8: for (int i = 0; i < hp.ks; i++) ((ll_t *)dst_row)[hp.perm[i]] = ((const ll_t *)src)[i]; break;
      case 4: for (int i = 0; i < hp.ks; i++) ((int *)dst_row)[hp.perm[i]] = ((const int *)src)[i]; break;
      case 2: for (int i = 0; i < hp.ks; i++) ((short *)dst_row)[hp.perm[i]] = ((const short *)src)[i]; break;
      default: for (int i = 0; i < hp.ks; i++) dst_row[hp.perm[i]] = src[i]; break;
    }
  }
};

// ndim int64 index tensors broadcast to one shape; element e of the row-major linearisation of `sizes`.
// Replaces StrictTensorAccessor::get_index_from_offset + get (tensor_accessor.cu:70-87) as used by
// sparse_dok_tensor_impl.cu:36-42.
struct SelKeys {
  dok_selectors s;
  ll_t n;
  __device__ __forceinline__ ll_t count() const { return n; }
  __device__ __forceinline__ bool row(ll_t &e) const { e = (ll_t)blockIdx.x * DOK_TPB + threadIdx.x; return e < n; }
  __device__ __forceinline__ bool at(ll_t j, ll_t &e) const { e = j; return j < n; }
  __device__ __forceinline__ ll_t span() const { return n; }
  __device__ __forceinline__ bool idle() const { return false; }
  // element offsets of batch element e into each of the ndim index tensors (fully unrolled over the
  // maximum ndim with predication, so `off` stays in registers)
  __device__ __forceinline__ void offsets(ll_t e, ll_t (&off)[DOK_MAX_KEY_SIZE]) const {
#pragma unroll
    for (int d = 0; d < DOK_MAX_KEY_SIZE; d++) off[d] = 0;
    if (n <= 0xffffffffLL) {           // 32-bit index arithmetic: the common case, far cheaper than 64-bit division
      unsigned rem = (unsigned)e;
      for (int j = s.selector_ndim - 1; j >= 0; j--) {
        const unsigned size = (unsigned)s.sizes[j];
        const unsigned q = rem / size;
        const ll_t idx = (ll_t)(rem - q * size);
        rem = q;
#pragma unroll
        for (int d = 0; d < DOK_MAX_KEY_SIZE; d++) if (d < s.ndim) off[d] += idx * s.strides[d][j];
      }
    } else {
      ull_t rem = (ull_t)e;
      for (int j = s.selector_ndim - 1; j >= 0; j--) {
        const ull_t size = (ull_t)s.sizes[j];
        const ull_t q = rem / size;
        const ll_t idx = (ll_t)(rem - q * size);
        rem = q;
#pragma unroll
        for (int d = 0; d < DOK_MAX_KEY_SIZE; d++) if (d < s.ndim) off[d] += idx * s.strides[d][j];
      }
    }
  }
  __device__ __forceinline__ KeyHash hash(const DevHash &hp, ll_t e) const {
    ll_t off[DOK_MAX_KEY_SIZE];
    offsets(e, off);
    ll_t k = s.ptr[0][off[0]];
    ll_t u = dok_uuid_term(k, hp.a[0], hp.b[0], hp.p[0], hp.m[0]);
    ull_t h = (ull_t)k * (ull_t)hp.a1[0] + (ull_t)hp.b1[0];
#pragma unroll
    for (int d = 1; d < DOK_MAX_KEY_SIZE; d++)
      if (d < s.ndim) {
        k = s.ptr[d][off[d]];
        u = (ll_t)((ull_t)u * (ull_t)dok_uuid_term(k, hp.a[d], hp.b[d], hp.p[d], hp.m[d]));
        h *= (ull_t)k * (ull_t)hp.a1[d] + (ull_t)hp.b1[d];
      }
    return KeyHash{dok_llabs(u), (ll_t)h};
  }
  __device__ __forceinline__ void store_key(const DevHash &hp, ll_t e, char *dst_row) const {
    ll_t off[DOK_MAX_KEY_SIZE];
    offsets(e, off);
#pragma unroll
    for (int d = 0; d < DOK_MAX_KEY_SIZE; d++)
      if (d < s.ndim) ((ll_t *)dst_row)[hp.perm[d]] = s.ptr[d][off[d]];
  }
};

// ---------------------------------------------------------------------------------------------------------
// Slot access
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ char *dok_slot_ptr(const DevTable &t, ll_t slot) { return t.slots + slot * (ll_t)t.sb; }
__device__ __forceinline__ ll_t *dok_tag_ptr(const DevTable &t, ll_t slot) { return (ll_t *)dok_slot_ptr(t, slot); }
__device__ __forceinline__ ll_t dok_load_tag(const DevTable &t, ll_t slot) {
  return __ldcg(dok_tag_ptr(t, slot));   // L2 is the point of coherence for the CAS claims
}
__device__ __forceinline__ ll_t dok_cas_tag(const DevTable &t, ll_t slot, ll_t expect, ll_t desired) {
  return (ll_t)atomicCAS((ull_t *)dok_tag_ptr(t, slot), (ull_t)expect, (ull_t)desired);
}
__device__ __forceinline__ ll_t *dok_stamp_ptr(const DevTable &t, ll_t slot) {
  return t.stamp_off >= 0 ? (ll_t *)(dok_slot_ptr(t, slot) + t.stamp_off) : t.stamp + slot;
}
__device__ __forceinline__ char *dok_value_ptr(const DevTable &t, ll_t slot) { return dok_slot_ptr(t, slot) + t.val_off; }
__device__ __forceinline__ char *dok_key_row(const DevTable &t, ll_t slot) { return dok_slot_ptr(t, slot) + t.key_off; }

// `nbytes` (1..8) of the little-endian word `w` to dst, with the widest stores the alignment `align` (a power
// of two that divides both dst and nbytes' positions) allows
__device__ __forceinline__ void dok_store_word(char *dst, ull_t w, int nbytes, int align) {
  if (nbytes == 8 && align >= 8) { *(ull_t *)dst = w; return; }
  if (align >= 4) {
    *(unsigned *)dst = (unsigned)w;
    if (nbytes > 4) *(unsigned *)(dst + 4) = (unsigned)(w >> 32);
    return;
  }
  if (align >= 2) {
    for (int i = 0; i < nbytes; i += 2) *(unsigned short *)(dst + i) = (unsigned short)(w >> (8 * i));
    return;
  }
  for (int i = 0; i < nbytes; i++) dst[i] = (char)(w >> (8 * i));
}

// What a walk of one key's chain found.  found >= 0: the slot holding the uuid.  Otherwise `empty` is the first
// empty slot of the chain (-1: the whole table was walked without meeting one) and `tomb` the first tombstone
// met before it (-1: none) -- the two places ClosedHashmap::set may claim (closed_hashmap_impl_class.cu:368-427).
struct Located { ll_t found, empty, tomb; };

// Slot-by-slot walk by ONE lane: the reference's loop (closed_hashmap_impl_class.cu:280-312, 368-407) from this
// library's start slot.  Used for slots wider than a line.
__device__ __forceinline__ Located dok_locate_serial(const DevTable &t, const KeyHash &kh, int *probes) {
  Located r{-1, -1, -1};
  ll_t slot = dok_start_group(kh, t) * t.spg;
  ll_t i = 0;
  for (; i < t.n_slots; i++) {
    const ll_t tag = dok_load_tag(t, slot);
    if (tag == kh.uuid) { r.found = slot; i++; break; }
    if (tag == DOK_EMPTY) { r.empty = slot; i++; break; }
    if (tag == DOK_REMOVED && r.tomb < 0) r.tomb = slot;
    if (++slot == t.n_slots) slot = 0;
  }
  if (probes) *probes = (int)i;
  return r;
}

// No-op hit handler for walks that only need the slot.
struct NoEmit {
  template <int LW>
  __device__ __forceinline__ void operator()(ll_t, int, const ull_t (&)[LW]) const {}
};

// LW 8-byte words of a line chunk with one load that allocates in L2 only (L2 is the point of coherence for the
// CAS claims; the table is touched at random, so L1 lines would be dead on arrival)
template <int LW>
__device__ __forceinline__ void dok_load_words(const char *p, ull_t (&w)[LW]) {
  if constexpr (LW == 4) {
    asm volatile("ld.global.cg.v4.u64 {%0,%1,%2,%3}, [%4];" : "=l"(w[0]), "=l"(w[1]), "=l"(w[2]), "=l"(w[3]) : "l"(p));
  } else if constexpr (LW == 2) {
    const ulonglong2 v = __ldcg((const ulonglong2 *)p);
    w[0] = v.x; w[1] = v.y;
  } else {
    w[0] = __ldcg((const ull_t *)p);
  }
}

// The same walk for the 32 keys of a warp, one 128-byte group per request.  Lane i owns key i.  The four lanes of
// a quad serve the quad's four keys together, in PASSES: in a pass each lane loads, for every key of the quad that
// is still unresolved, the first LW words of its 32 bytes of that key's current group (one coalesced request per
// line: 1 word = the tags only, 2 = tag and an 8-byte value, 4 = everything; all requests of a pass are issued
// before any answer is looked at), compares its tag, and packs one match bit and one empty bit per key and slot
// into ONE 32-bit word (byte r = key r: bits 0-3 match, bits 4-7 empty, by slot).  Two xor-shuffles OR the quad's
// words together; every lane then knows the outcome of all four keys, and the owner lanes advance their own
// state once per pass.  With TOMB the tombstone bits travel in a second word (set needs them, lookups do not).
// The number of dependent memory round trips of a warp is the longest chain among its 32 keys (in groups), and
// rounds in which no quad of the warp has work are skipped (the decision is warp-uniform).
// On a hit, `emit(e_r, slot_in_group, words)` runs on all four lanes while they still hold the line: e_r is the
// batch element of the key, words the calling lane's chunk.
// Every lane of the warp must call this (inactive lanes pass active = false), with CONSECUTIVE batch elements e in
// consecutive lanes.  SB = slot bytes (32, 64, 128).  Slot indices are 32-bit here: the host refuses cooperative
// tables of 2^32 - 1 slots or more.
template <int SB, int LW, bool TOMB, class Emit>
__device__ __forceinline__ Located dok_locate_quad(const DevTable &t, const KeyHash &kh, ll_t e, bool active,
                                                   int *probes, const Emit &emit) {
  constexpr int SPG = 128 / SB;
  constexpr unsigned FULL = 0xffffffffu;
  constexpr unsigned NONE = 0xffffffffu;              // group index of a lane with nothing (left) to do
  const unsigned lane = threadIdx.x & 31u, l = lane & 3u, base = lane & ~3u;
  const bool has_tag = ((32u * l) % SB) == 0;         // does this lane's chunk start with a slot's tag?
  const unsigned my_slot = (32u * l) / SB;            // slot (within the group) the chunk belongs to
  const ll_t e_quad = e - l;                          // batch element of the quad's first lane (elements are consecutive)
  const unsigned n_groups = (unsigned)t.n_groups;     // < 2^32 (checked on the host)
  const char *my_base = t.slots + 32 * l;
  // results as 32-bit group-relative codes until the end: slot = group * SPG + position
  unsigned found = NONE, empty = NONE, tomb = NONE;
  unsigned group = active ? (unsigned)dok_start_group(kh, t) : NONE;
  unsigned walked = 0;

  // what the owner lane does with the outcome of one inspected group: m / me / tb = match, match-or-empty and
  // tombstone bits by slot
  auto advance = [&](unsigned m, unsigned me, unsigned tb) {
    const int pos = me ? __ffs(me) - 1 : -1;
    const unsigned first_slot = group * SPG;
    walked++;
    if (TOMB && tomb == NONE) {
      const unsigned before = pos >= 0 ? (tb & ((1u << pos) - 1u)) : tb;
      if (before) tomb = first_slot + __ffs(before) - 1;
    }
    if (pos >= 0) {
      if ((m >> pos) & 1u) found = first_slot + pos; else empty = first_slot + pos;
      group = NONE;
    } else {
      group = (group + 1 == n_groups) ? 0u : group + 1;
      if (walked == n_groups) group = NONE;           // every group inspected: no empty slot anywhere
    }
  };

  // ---- first groups of the quad's four keys: four requests in flight, one packed exchange
  {
    ull_t w[4][LW];
    unsigned g[4];
#pragma unroll
    for (unsigned r = 0; r < 4; r++) {
      g[r] = __shfl_sync(FULL, group, base + r);
      if (g[r] != NONE) dok_load_words<LW>(my_base + (ull_t)g[r] * 128u, w[r]);
    }
    unsigned bits = 0, tbits = 0;
#pragma unroll
    for (unsigned r = 0; r < 4; r++) {
      const ll_t uuid_r = __shfl_sync(FULL, kh.uuid, base + r);
      if (has_tag && g[r] != NONE) {
        const ll_t tag = (ll_t)w[r][0];
        bits |= ((unsigned)(tag == uuid_r) | ((unsigned)(tag == DOK_EMPTY) << 4)) << (8u * r + my_slot);
        if (TOMB) tbits |= (unsigned)(tag == DOK_REMOVED) << (4u * r + my_slot);
      }
    }
    bits |= __shfl_xor_sync(FULL, bits, 1);
    bits |= __shfl_xor_sync(FULL, bits, 2);
    if (TOMB) {
      tbits |= __shfl_xor_sync(FULL, tbits, 1);
      tbits |= __shfl_xor_sync(FULL, tbits, 2);
    }
#pragma unroll
    for (unsigned r = 0; r < 4; r++) {                // hits: hand the line to the emitter while it is in registers
      const unsigned m = (bits >> (8u * r)) & 0xfu, me = (m | (bits >> (8u * r + 4u))) & 0xfu;
      if (me) {
        const int pos = __ffs(me) - 1;
        if ((m >> pos) & 1u) emit(e_quad + r, pos, w[r]);
      }
    }
    if (group != NONE) {
      const unsigned mine = bits >> (8u * l);
      advance(mine & 0xfu, (mine | (mine >> 4)) & 0xfu, TOMB ? (tbits >> (4u * l)) & 0xfu : 0u);
    }
  }

  // ---- keys whose chain runs into further groups (few below 90 % load): one key per quad and iteration
  for (;;) {
    const unsigned pend = __ballot_sync(FULL, group != NONE);
    if (pend == 0) break;
    const unsigned quad = (pend >> base) & 0xfu;
    const unsigned r = quad ? (unsigned)(__ffs(quad) - 1) : 0u;     // the quad's lowest unfinished key
    unsigned g_r = __shfl_sync(FULL, group, base + r);
    if (!quad) g_r = NONE;
    const ll_t uuid_r = __shfl_sync(FULL, kh.uuid, base + r);
    ull_t wl[LW];
    if (g_r != NONE) dok_load_words<LW>(my_base + (ull_t)g_r * 128u, wl);
    const ll_t tag = (has_tag && g_r != NONE) ? (ll_t)wl[0] : DOK_BLOCKED;
    unsigned bits = ((unsigned)(tag == uuid_r) | ((unsigned)(tag == DOK_EMPTY) << 4) |
                     (TOMB ? (unsigned)(tag == DOK_REMOVED) << 8 : 0u)) << my_slot;
    bits |= __shfl_xor_sync(FULL, bits, 1);
    bits |= __shfl_xor_sync(FULL, bits, 2);
    const unsigned m = bits & 0xfu, me = (bits | (bits >> 4)) & 0xfu;
    if (me) {
      const int pos = __ffs(me) - 1;
      if ((m >> pos) & 1u) emit(e_quad + r, pos, wl);
    }
    if (l == r && group != NONE) advance(m, me, (bits >> 8) & 0xfu);
  }
  if (probes) *probes = (int)walked;
  Located res;
  res.found = found == NONE ? -1 : (ll_t)found;
  res.empty = empty == NONE ? -1 : (ll_t)empty;
  res.tomb = tomb == NONE ? -1 : (ll_t)tomb;
  return res;
}

// Hit handler of `get`: the lanes of the quad write the value straight from the registers that hold the line, so
// a hit needs no second access to the table.  LW = 2 serves 32-byte slots whose value is one word behind the tag.
template <int SB, int LW>
struct EmitValue {
  const DevTable &t;
  char *out_values;
  __device__ __forceinline__ void operator()(ll_t e_r, int pos, const ull_t (&w)[LW]) const {
    const int l = (int)(threadIdx.x & 3u);
    char *dst = out_values + e_r * (ll_t)t.vb;
    if constexpr (SB == 32 && LW == 2) {
      if (l == pos) {
        if (t.vb == 8) *(ull_t *)dst = w[1];
        else dok_store_word(dst, w[1], t.vb, (t.vb & -t.vb));
      }
    } else {
      const int start = pos * SB + 8 - 32 * l;             // offset of the value relative to this lane's chunk
      const int align = (t.vb & -t.vb) < 8 ? (t.vb & -t.vb) : 8;
#pragma unroll
      for (int j = 0; j < LW; j++) {
        const int rel = 8 * j - start;
        if (rel >= 0 && rel < t.vb) dok_store_word(dst + rel, w[j], t.vb - rel < 8 ? t.vb - rel : 8, align);
      }
    }
  }
};

// SB == 0 selects the serial walk (slots wider than one line); emit is not called there.
template <int SB, int LW, bool TOMB, class Emit>
__device__ __forceinline__ Located dok_locate(const DevTable &t, const KeyHash &kh, ll_t e, bool active, int *probes,
                                              const Emit &emit) {
  if constexpr (SB == 0) {
    if (active) return dok_locate_serial(t, kh, probes);
    if (probes) *probes = 0;
    return Located{-1, -1, -1};
  } else {
    return dok_locate_quad<SB, LW, TOMB>(t, kh, e, active, probes, emit);
  }
}

enum { DOK_OUT_FOUND = 0, DOK_OUT_CLAIMED_EMPTY = 1, DOK_OUT_REUSED = 2, DOK_OUT_FAILED = 3 };

// Insert-or-find by one lane, slot by slot (ClosedHashmap::set, closed_hashmap_impl_class.cu:368-427, without
// the row stores).  Phase 1 walks the chain: a matching tag is a hit; the first tombstone is remembered; at the
// first empty tag the slot is claimed by CAS unless a tombstone was seen.  Phase 2 starts at the remembered
// tombstone and tries tombstone->uuid, then empty->uuid, slot by slot.  Unlike the reference, a CAS that loses
// to the SAME uuid joins that slot instead of walking on, so equal uuids of one batch always meet in one slot.
static __device__ __forceinline__ ll_t dok_find_or_claim_serial(const DevTable &t, const KeyHash &kh, int *outcome) {
  const ll_t uuid = kh.uuid;
  ll_t slot = dok_start_group(kh, t) * t.spg;
  ll_t first_removed = -1;
  for (ll_t i = 0; i < t.n_slots; i++) {
    ll_t tag = dok_load_tag(t, slot);
    if (tag == DOK_EMPTY && first_removed < 0) {
      tag = dok_cas_tag(t, slot, DOK_EMPTY, uuid);
      if (tag == DOK_EMPTY) { *outcome = DOK_OUT_CLAIMED_EMPTY; return slot; }
    }
    if (tag == uuid) { *outcome = DOK_OUT_FOUND; return slot; }
    if (tag == DOK_EMPTY) break;                       // a tombstone was seen earlier: go reuse it
    if (tag == DOK_REMOVED && first_removed < 0) first_removed = slot;
    if (++slot == t.n_slots) slot = 0;
  }
  if (first_removed >= 0) {
    slot = first_removed;
    for (ll_t i = 0; i < t.n_slots; i++) {
      ll_t old = dok_cas_tag(t, slot, DOK_REMOVED, uuid);
      if (old == DOK_REMOVED) { *outcome = DOK_OUT_REUSED; return slot; }
      if (old == DOK_EMPTY) {
        old = dok_cas_tag(t, slot, DOK_EMPTY, uuid);
        if (old == DOK_EMPTY) { *outcome = DOK_OUT_CLAIMED_EMPTY; return slot; }
      }
      if (old == uuid) { *outcome = DOK_OUT_FOUND; return slot; }
      if (++slot == t.n_slots) slot = 0;
    }
  }
  *outcome = DOK_OUT_FAILED;
  return -1;
}

// Insert-or-find for the 32 keys of a warp: one cooperative walk tells every owner lane where its uuid is or
// where the chain offers a place (first tombstone, else first empty slot); the owner claims that place with one
// CAS.  Losing the CAS to the same uuid means a twin row of the batch claimed it: join.  Losing it to another
// uuid is rare; that lane redoes the whole operation with the serial walk.  Every lane of the warp must call.
template <int SB>
__device__ __forceinline__ ll_t dok_find_or_claim(const DevTable &t, const KeyHash &kh, bool active, int *outcome) {
  const Located loc = dok_locate<SB, 1, true>(t, kh, 0, active, nullptr, NoEmit());   // the tags are all a claim needs
  if (!active) return -1;
  if (loc.found >= 0) { *outcome = DOK_OUT_FOUND; return loc.found; }
  if (loc.tomb >= 0) {
    const ll_t old = dok_cas_tag(t, loc.tomb, DOK_REMOVED, kh.uuid);
    if (old == DOK_REMOVED) { *outcome = DOK_OUT_REUSED; return loc.tomb; }
    if (old == kh.uuid) { *outcome = DOK_OUT_FOUND; return loc.tomb; }
  } else if (loc.empty >= 0) {
    const ll_t old = dok_cas_tag(t, loc.empty, DOK_EMPTY, kh.uuid);
    if (old == DOK_EMPTY) { *outcome = DOK_OUT_CLAIMED_EMPTY; return loc.empty; }
    if (old == kh.uuid) { *outcome = DOK_OUT_FOUND; return loc.empty; }
  } else {
    *outcome = DOK_OUT_FAILED;       // no match, no tombstone, no empty slot: the table is full
    return -1;
  }
  return dok_find_or_claim_serial(t, kh, outcome);
}

// value row (vb bytes at `src`, alignment of the widest power of two dividing vb, capped at 8) -> slot
__device__ __forceinline__ void dok_store_value(const DevTable &t, ll_t slot, const char *src) {
  ull_t *dst = (ull_t *)dok_value_ptr(t, slot);
  if (t.vb == 8) { *dst = *(const ull_t *)src; return; }
  if (t.vb == 4) { *(unsigned *)dst = *(const unsigned *)src; return; }
  if ((t.vb & 7) == 0) {
    for (int w = 0; w < t.vwords; w++) dst[w] = ((const ull_t *)src)[w];
  } else if ((t.vb & 3) == 0) {
    unsigned *d32 = (unsigned *)dst;
    for (int w = 0; w < (t.vb >> 2); w++) d32[w] = ((const unsigned *)src)[w];
  } else if ((t.vb & 1) == 0) {
    unsigned short *d16 = (unsigned short *)dst;
    for (int w = 0; w < (t.vb >> 1); w++) d16[w] = ((const unsigned short *)src)[w];
  } else {
    char *d8 = (char *)dst;
    for (int w = 0; w < t.vb; w++) d8[w] = src[w];
  }
}

// slot -> value row
__device__ __forceinline__ void dok_load_value(const DevTable &t, ll_t slot, char *dst) {
  const ull_t *src = (const ull_t *)dok_value_ptr(t, slot);
  if (t.vb == 8) { *(ull_t *)dst = __ldcg(src); return; }
  if (t.vb == 4) { *(unsigned *)dst = __ldcg((const unsigned *)src); return; }
  if ((t.vb & 7) == 0) {
    for (int w = 0; w < t.vwords; w++) ((ull_t *)dst)[w] = __ldcg(src + w);
  } else if ((t.vb & 3) == 0) {
    for (int w = 0; w < (t.vb >> 2); w++) ((unsigned *)dst)[w] = __ldcg((const unsigned *)src + w);
  } else if ((t.vb & 1) == 0) {
    for (int w = 0; w < (t.vb >> 1); w++) ((unsigned short *)dst)[w] = __ldcg((const unsigned short *)src + w);
  } else {
    for (int w = 0; w < t.vb; w++) dst[w] = __ldcg((const char *)src + w);
  }
}

struct Fallback { ull_t w[DOK_MAX_VALUE_BYTES / 8]; };   // miss fill, passed by value

__device__ __forceinline__ void dok_store_fallback(const DevTable &t, const Fallback &fb, char *dst) {
  const char *src = (const char *)fb.w;
  if (t.vb == 8) { *(ull_t *)dst = fb.w[0]; return; }
  if (t.vb == 4) { *(unsigned *)dst = (unsigned)fb.w[0]; return; }
  if ((t.vb & 7) == 0) {
    for (int w = 0; w < t.vwords; w++) ((ull_t *)dst)[w] = fb.w[w];
  } else if ((t.vb & 3) == 0) {
    for (int w = 0; w < (t.vb >> 2); w++) ((unsigned *)dst)[w] = ((const unsigned *)src)[w];
  } else if ((t.vb & 1) == 0) {
    for (int w = 0; w < (t.vb >> 1); w++) ((unsigned short *)dst)[w] = ((const unsigned short *)src)[w];
  } else {
    for (int w = 0; w < t.vb; w++) dst[w] = src[w];
  }
}

// Per-launch counters.  The counters of a launch are a handful of global addresses, and atomics on one address are
// served one after the other, so a million per-warp atomics on one word cost about as much as the probing itself.
// A block therefore tallies in shared memory (one vote and one shared atomic per warp and counter) and the LAST warp
// of the block to finish adds the block's totals to global memory: one global atomic per block and counter, and no
// barrier at the end of the kernel, where warps finish at very different times.
// Slots 0 .. 7 go to counters[slot] (the dok_counter indices), slot 8 to `extra`.  Every thread of the block must
// call begin and flush, and every lane of a warp must call add together.
#define DOK_TALLY_SLOTS 9
#define DOK_TALLY_EXTRA 8
struct BlockTally { int v[DOK_TALLY_SLOTS]; int done; };

__device__ __forceinline__ void dok_tally_begin(BlockTally &b) {
  if (threadIdx.x < DOK_TALLY_SLOTS) b.v[threadIdx.x] = 0;
  if (threadIdx.x == DOK_TALLY_SLOTS) b.done = 0;
  __syncthreads();
}
__device__ __forceinline__ void dok_tally_add(BlockTally &b, int slot, int pred) {
  const unsigned m = __ballot_sync(0xffffffffu, pred);
  if ((threadIdx.x & 31) == 0 && m) atomicAdd(&b.v[slot], __popc(m));
}
__device__ __forceinline__ void dok_tally_flush(BlockTally &b, ll_t *counters, ll_t *extra) {
  __syncwarp();
  int last = 0;
  if ((threadIdx.x & 31) == 0) {
    __threadfence_block();
    last = atomicAdd(&b.done, 1) == (int)(blockDim.x >> 5) - 1;
  }
  last = __shfl_sync(0xffffffffu, last, 0);
  if (!last) return;
  const int k = threadIdx.x & 31;
  if (k < DOK_TALLY_SLOTS) {
    const int c = ((volatile int *)b.v)[k];
    ll_t *dst = k < DOK_TALLY_EXTRA ? (counters ? counters + k : nullptr) : extra;
    if (c && dst) atomicAdd((ull_t *)dst, (ull_t)c);
  }
}

// warp sum + one atomicAdd per warp (replaces warp_sum + atomicAdd of sparse_dok_tensor_impl.cu:52-55).
// Every lane of the warp must call it.
__device__ __forceinline__ void dok_warp_add(ll_t *counter, int v) {
  if (counter == nullptr) return;
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0 && v) atomicAdd((ull_t *)counter, (ull_t)v);
}
