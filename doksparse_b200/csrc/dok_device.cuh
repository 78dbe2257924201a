// Device-side building blocks shared by the kernels of libdoksparse.so (sm_100a).
//
// Semantics follow the reference's ClosedHashmap class
// (sparse_dok/components/cuda/closed_hashmap_impl_class.cu): key identity is the 64-bit uuid, tags are
// uuid / -1 (empty) / -3 (tombstone), probing is linear, a lookup stops at the first empty tag and steps
// over tombstones.  What differs on purpose is the memory layout (tag and value share one bucket row so that
// a hit costs one 32-byte sector) and the start bucket (a mixer of the uuid instead of the reference's first
// hash, whose product form clusters badly on power-of-two tables).
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
  ll_t a1[DOK_MAX_KEY_SIZE];    // alpha1[key_perm[i]]   -- first hash: only decorrelates the probe chains of
  ll_t b1[DOK_MAX_KEY_SIZE];    // beta1[key_perm[i]]       keys whose uuids collide (see dok_start_bucket)
  ull_t p1[DOK_MAX_KEY_SIZE];   // |prime1[key_perm[i]]|
  ull_t m1[DOK_MAX_KEY_SIZE];   // floor(2^64 / p1)
  int perm[DOK_MAX_KEY_SIZE];   // storage column of key element i
};

struct KeyHash { ll_t uuid; ll_t hash1; };

struct DevTable {
  char *buckets;    // n_buckets * bb bytes: {int64 tag; value; pad}
  char *keys;       // n_buckets * kb bytes
  ll_t *stamp;      // n_buckets or nullptr
  ll_t nb;
  ull_t nb_magic;   // floor(2^64 / nb)
  int bb;           // bucket bytes (multiple of 16)
  int vb;           // value bytes
  int kb;           // key row bytes
  int vwords;       // ceil(vb / 8)
};

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
// Start bucket.  In the reference two keys whose uuids collide are still told apart as long as their probe
// chains (first hash modulo n_buckets) do not meet; a uuid collision is not rare there, because alpha2 may be
// drawn as 0 (cuda_closed_hashmap.py:100), which makes one key element drop out of the uuid.  To keep that
// property the start bucket mixes the uuid with the reference's first hash reduced modulo n_buckets: keys
// that collide in BOTH collide here too, keys that collide in the uuid only get unrelated chains.
__device__ __forceinline__ ll_t dok_start_bucket(const KeyHash &h, ll_t nb, ull_t nb_magic) {
  const ull_t h1 = (ull_t)h.hash1;
  ull_t r = h1 - __umul64hi(h1, nb_magic) * (ull_t)nb;       // h1 % nb
  if (r >= (ull_t)nb) r -= (ull_t)nb;
  return (ll_t)__umul64hi(dok_mix64((ull_t)h.uuid ^ ((r + 1) * 0x9e3779b97f4a7c15ULL)), (ull_t)nb);
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
  __device__ __forceinline__ ll_t count() const { return n; }
  // get_uuid and get_hash of the reference (closed_hashmap_impl_class.cu:87-107) in one pass over the key
  __device__ __forceinline__ KeyHash hash(const DevHash &hp, ll_t e) const {
    ll_t k = dok_key_elem(keys, hp.dtype, e * hp.ks);
    ll_t u = dok_uuid_term(k, hp.a[0], hp.b[0], hp.p[0], hp.m[0]);
    ll_t h = dok_uuid_term(k, hp.a1[0], hp.b1[0], hp.p1[0], hp.m1[0]);
    for (int i = 1; i < hp.ks; i++) {
      k = dok_key_elem(keys, hp.dtype, e * hp.ks + i);
      u = (ll_t)((ull_t)u * (ull_t)dok_uuid_term(k, hp.a[i], hp.b[i], hp.p[i], hp.m[i]));
      h = (ll_t)((ull_t)h * (ull_t)dok_uuid_term(k, hp.a1[i], hp.b1[i], hp.p1[i], hp.m1[i]));
    }
    return KeyHash{dok_llabs(u), dok_llabs(h)};
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
    ll_t h = dok_uuid_term(k, hp.a1[0], hp.b1[0], hp.p1[0], hp.m1[0]);
#pragma unroll
    for (int d = 1; d < DOK_MAX_KEY_SIZE; d++)
      if (d < s.ndim) {
        k = s.ptr[d][off[d]];
        u = (ll_t)((ull_t)u * (ull_t)dok_uuid_term(k, hp.a[d], hp.b[d], hp.p[d], hp.m[d]));
        h = (ll_t)((ull_t)h * (ull_t)dok_uuid_term(k, hp.a1[d], hp.b1[d], hp.p1[d], hp.m1[d]));
      }
    return KeyHash{dok_llabs(u), dok_llabs(h)};
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
// Bucket access
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ ll_t *dok_tag_ptr(const DevTable &t, ll_t slot) {
  return (ll_t *)(t.buckets + slot * (ll_t)t.bb);
}
__device__ __forceinline__ ll_t dok_load_tag(const DevTable &t, ll_t slot) {
  return __ldcg(dok_tag_ptr(t, slot));   // L2 is the point of coherence for the CAS claims
}
__device__ __forceinline__ ll_t dok_cas_tag(const DevTable &t, ll_t slot, ll_t expect, ll_t desired) {
  return (ll_t)atomicCAS((ull_t *)dok_tag_ptr(t, slot), (ull_t)expect, (ull_t)desired);
}

// Lookup: returns the slot holding `uuid`, or -1 (ClosedHashmap::get / exists,
// closed_hashmap_impl_class.cu:253-312).  The loop is bounded by n_buckets like the reference's.
__device__ __forceinline__ ll_t dok_find(const DevTable &t, const KeyHash &kh, int *probes) {
  const ll_t uuid = kh.uuid;
  ll_t slot = dok_start_bucket(kh, t.nb, t.nb_magic);
  for (ll_t i = 0; i < t.nb; i++) {
    const ll_t tag = dok_load_tag(t, slot);
    if (tag == uuid) { if (probes) *probes = (int)i + 1; return slot; }
    if (tag == DOK_EMPTY) { if (probes) *probes = (int)i + 1; return -1; }
    if (++slot == t.nb) slot = 0;
  }
  if (probes) *probes = (int)t.nb;
  return -1;
}

enum { DOK_OUT_FOUND = 0, DOK_OUT_CLAIMED_EMPTY = 1, DOK_OUT_REUSED = 2, DOK_OUT_FAILED = 3 };

// Insert-or-find (ClosedHashmap::set, closed_hashmap_impl_class.cu:368-427, without the row stores).
// Phase 1 walks the chain: a matching tag is a hit; the first tombstone is remembered; at the first empty
// tag the slot is claimed by CAS unless a tombstone was seen.  Phase 2 starts at the remembered tombstone and
// tries tombstone->uuid, then empty->uuid, slot by slot.  Unlike the reference, a CAS that loses to the SAME
// uuid joins that slot instead of walking on, so that equal uuids of one batch always meet in one slot.
__device__ __forceinline__ ll_t dok_find_or_claim(const DevTable &t, const KeyHash &kh, int *outcome) {
  const ll_t uuid = kh.uuid;
  ll_t slot = dok_start_bucket(kh, t.nb, t.nb_magic);
  ll_t first_removed = -1;
  for (ll_t i = 0; i < t.nb; i++) {
    ll_t tag = dok_load_tag(t, slot);
    if (tag == DOK_EMPTY && first_removed < 0) {
      tag = dok_cas_tag(t, slot, DOK_EMPTY, uuid);
      if (tag == DOK_EMPTY) { *outcome = DOK_OUT_CLAIMED_EMPTY; return slot; }
    }
    if (tag == uuid) { *outcome = DOK_OUT_FOUND; return slot; }
    if (tag == DOK_EMPTY) break;                       // a tombstone was seen earlier: go reuse it
    if (tag == DOK_REMOVED && first_removed < 0) first_removed = slot;
    if (++slot == t.nb) slot = 0;
  }
  if (first_removed >= 0) {
    slot = first_removed;
    for (ll_t i = 0; i < t.nb; i++) {
      ll_t old = dok_cas_tag(t, slot, DOK_REMOVED, uuid);
      if (old == DOK_REMOVED) { *outcome = DOK_OUT_REUSED; return slot; }
      if (old == DOK_EMPTY) {
        old = dok_cas_tag(t, slot, DOK_EMPTY, uuid);
        if (old == DOK_EMPTY) { *outcome = DOK_OUT_CLAIMED_EMPTY; return slot; }
      }
      if (old == uuid) { *outcome = DOK_OUT_FOUND; return slot; }
      if (++slot == t.nb) slot = 0;
    }
  }
  *outcome = DOK_OUT_FAILED;
  return -1;
}

// value row (vb bytes at `src`, alignment of the widest power of two dividing vb, capped at 8) -> bucket
__device__ __forceinline__ void dok_store_value(const DevTable &t, ll_t slot, const char *src) {
  ull_t *dst = (ull_t *)(t.buckets + slot * (ll_t)t.bb + 8);
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

// bucket -> value row
__device__ __forceinline__ void dok_load_value(const DevTable &t, ll_t slot, char *dst) {
  const ull_t *src = (const ull_t *)(t.buckets + slot * (ll_t)t.bb + 8);
  if ((t.vb & 7) == 0) {
    for (int w = 0; w < t.vwords; w++) ((ull_t *)dst)[w] = src[w];
  } else if ((t.vb & 3) == 0) {
    for (int w = 0; w < (t.vb >> 2); w++) ((unsigned *)dst)[w] = ((const unsigned *)src)[w];
  } else if ((t.vb & 1) == 0) {
    for (int w = 0; w < (t.vb >> 1); w++) ((unsigned short *)dst)[w] = ((const unsigned short *)src)[w];
  } else {
    for (int w = 0; w < t.vb; w++) dst[w] = ((const char *)src)[w];
  }
}

struct Fallback { ull_t w[DOK_MAX_VALUE_BYTES / 8]; };   // miss fill, passed by value

__device__ __forceinline__ void dok_store_fallback(const DevTable &t, const Fallback &fb, char *dst) {
  const char *src = (const char *)fb.w;
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

// warp sum + one atomicAdd per warp (replaces warp_sum + atomicAdd of sparse_dok_tensor_impl.cu:52-55)
__device__ __forceinline__ void dok_warp_add(ll_t *counter, int v) {
  if (counter == nullptr) return;
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0 && v) atomicAdd((ull_t *)counter, (ull_t)v);
}
