/*
 * TEST INFRASTRUCTURE ONLY -- the product path never links, imports or runs this file.
 * Only the test-suite, the smoke check and the benchmark's CPU-baseline leg use it,
 * and there only as the checker / the timed CPU baseline.
 *
 * A plain-C restatement of the reference hash map algorithm of
 * DeMoriarty/DOKSparse (sparse_dok 0.1.9.2), on the reference's own storage layout:
 *   keys   [n_buckets, key_size]   (element type = key dtype)
 *   values [n_buckets, value_row_bytes]  (opaque bytes)
 *   uuid   [n_buckets] int64, -1 = empty, -3 = removed (tombstone)
 * Because the start bucket is computed with the reference's first hash, a serial run of
 * this file produces the same slot layout as a serial run of the reference kernels;
 * tests/test_oracle_vs_ref.py checks the raw arrays for equality against the reference's
 * own source compiled for the host (oracle/_ref).
 *
 * Pinning: the reference ships no tests or golden vectors.  This restatement is pinned
 * against outputs of the reference's own kernel source run on the host (oracle/_ref) and
 * against fixtures generated from it (tests/golden).
 *
 * Each function cites the reference lines it follows (paths relative to the reference
 * checkout, sparse_dok/components/cuda/...).
 */
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_MAX_KEY_SIZE 8
#define ORC_EMPTY (-1LL)
#define ORC_REMOVED (-3LL)

/* element type codes (shared with the product's C header by value) */
enum {
  ORC_I8 = 0, ORC_U8 = 1, ORC_I16 = 2, ORC_I32 = 3, ORC_I64 = 4,
  ORC_F16 = 5, ORC_BF16 = 6, ORC_F32 = 7, ORC_F64 = 8
};

typedef struct orc_map {
  int32_t key_size;        /* number of key elements, <= ORC_MAX_KEY_SIZE */
  int32_t key_dtype;       /* element type code of the keys */
  int32_t value_row_bytes; /* bytes of one value row (opaque) */
  int32_t _pad;
  /* hash parameters exactly as the Python object holds them (NOT permuted) */
  int64_t prime1[ORC_MAX_KEY_SIZE], prime2[ORC_MAX_KEY_SIZE];
  int64_t alpha1[ORC_MAX_KEY_SIZE], alpha2[ORC_MAX_KEY_SIZE];
  int64_t beta1[ORC_MAX_KEY_SIZE], beta2[ORC_MAX_KEY_SIZE];
  int64_t key_perm[ORC_MAX_KEY_SIZE];
  int64_t n_buckets;
  void *keys;      /* [n_buckets, key_size] */
  void *values;    /* [n_buckets, value_row_bytes] */
  int64_t *uuid;   /* [n_buckets] */
} orc_map;

static int orc_elem_bytes(int dtype) {
  switch (dtype) {
    case ORC_I8: case ORC_U8: return 1;
    case ORC_I16: case ORC_F16: case ORC_BF16: return 2;
    case ORC_I32: case ORC_F32: return 4;
    default: return 8;
  }
}

/* float -> int64 by VALUE, round toward zero.  The device conversion saturates and maps NaN
 * to 0 (PTX cvt.rzi.s64.f32/f64); the same is defined here for out-of-range inputs, where the
 * C cast would be undefined. */
static int64_t orc_double_to_i64(double v) {
  if (v != v) return 0;
  if (v >= 9223372036854775808.0) return INT64_MAX;
  if (v <= -9223372036854775808.0) return INT64_MIN;
  return (int64_t)v;
}

static float orc_half_to_float(uint16_t h) {
  uint32_t sign = (uint32_t)(h >> 15) << 31, exp = (h >> 10) & 31, man = h & 1023, bits;
  if (exp == 0) {
    if (man == 0) bits = sign;
    else {
      int e = -1;
      do { e++; man <<= 1; } while (!(man & 1024));
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 1023) << 13);
    }
  } else if (exp == 31) bits = sign | 0x7f800000u | (man << 13);
  else bits = sign | ((exp + 112) << 23) | (man << 13);
  float f; memcpy(&f, &bits, 4); return f;
}

/* `(ll_t) key[i]` of closed_hashmap_impl_class.cu:89,92,100,103: a value cast, not a bit cast */
static int64_t orc_key_elem_as_i64(const void *row, int dtype, int i) {
  switch (dtype) {
    case ORC_I8: return ((const int8_t *)row)[i];
    case ORC_U8: return ((const uint8_t *)row)[i];
    case ORC_I16: return ((const int16_t *)row)[i];
    case ORC_I32: return ((const int32_t *)row)[i];
    case ORC_I64: return ((const int64_t *)row)[i];
    case ORC_F16: return orc_double_to_i64(orc_half_to_float(((const uint16_t *)row)[i]));
    case ORC_BF16: {
      uint32_t bits = (uint32_t)((const uint16_t *)row)[i] << 16; float f; memcpy(&f, &bits, 4);
      return orc_double_to_i64(f);
    }
    case ORC_F32: return orc_double_to_i64(((const float *)row)[i]);
    default: return orc_double_to_i64(((const double *)row)[i]);
  }
}

/* wrapping signed arithmetic, written with unsigned operands */
static int64_t wmul(int64_t a, int64_t b) { return (int64_t)((uint64_t)a * (uint64_t)b); }
static int64_t wadd(int64_t a, int64_t b) { return (int64_t)((uint64_t)a + (uint64_t)b); }
static int64_t wabs(int64_t a) { return a < 0 ? (int64_t)(0ULL - (uint64_t)a) : a; } /* llabs; INT64_MIN stays */
/* C truncated remainder (sign of the dividend); |p| >= 2 is required by the callers */
static int64_t trem(int64_t a, int64_t p) { return a % p; }

/* get_hash / get_uuid, closed_hashmap_impl_class.cu:87-107, with the parameters indexed through
 * keyPerm as the kernels' constructor does (:54-63): element i of the caller's key uses parameter
 * keyPerm[i]. */
static void orc_hash_uuid_row(const orc_map *m, const void *key_row, int64_t *hash, int64_t *uuid) {
  int64_t h = 0, u = 0;
  for (int i = 0; i < m->key_size; i++) {
    const int64_t k = orc_key_elem_as_i64(key_row, m->key_dtype, i);
    const int64_t c = m->key_perm[i];
    const int64_t th = trem(wadd(wmul(k, m->alpha1[c]), m->beta1[c]), m->prime1[c]);
    const int64_t tu = trem(wadd(wmul(k, m->alpha2[c]), m->beta2[c]), m->prime2[c]);
    if (i == 0) { h = th; u = tu; } else { h = wmul(h, th); u = wmul(u, tu); }
  }
  *hash = wabs(h);
  *uuid = wabs(u);
}

static const char *orc_row(const void *base, int64_t i, int64_t row_bytes) {
  return (const char *)base + i * row_bytes;
}

/* set_key_permuted, closed_hashmap_impl_class.cu:144-150: storage column keyPerm[i] <- key[i] */
static void orc_store_key(const orc_map *m, int64_t address, const void *key_row) {
  const int eb = orc_elem_bytes(m->key_dtype);
  char *dst = (char *)m->keys + address * (int64_t)m->key_size * eb;
  for (int i = 0; i < m->key_size; i++)
    memcpy(dst + m->key_perm[i] * eb, (const char *)key_row + (int64_t)i * eb, (size_t)eb);
}

static void orc_store_value(const orc_map *m, int64_t address, const void *value_row) {
  memcpy((char *)m->values + address * (int64_t)m->value_row_bytes, value_row, (size_t)m->value_row_bytes);
}

static int64_t orc_cas(int64_t *p, int64_t expect, int64_t desired) {
  __atomic_compare_exchange_n(p, &expect, desired, 0, __ATOMIC_SEQ_CST, __ATOMIC_SEQ_CST);
  return expect;
}

/* ClosedHashmap::get, closed_hashmap_impl_class.cu:280-312 (exists, :253-278, when out_value is
 * NULL): probe linearly from hash % n_buckets, stop at the empty marker, step over tombstones. */
static int orc_get_one(const orc_map *m, const void *key_row, void *out_value) {
  int64_t hash, uuid;
  orc_hash_uuid_row(m, key_row, &hash, &uuid);
  for (int64_t i = 0; i < m->n_buckets; i++) {
    /* (hashCode + i) % numBuckets; hashCode can be INT64_MIN only through llabs overflow */
    const int64_t address = trem(wadd(hash, i), m->n_buckets);
    const int64_t cand = __atomic_load_n(&m->uuid[address], __ATOMIC_RELAXED);
    if (cand == ORC_EMPTY) break;
    if (cand == uuid) {
      if (out_value) memcpy(out_value, orc_row(m->values, address, m->value_row_bytes), (size_t)m->value_row_bytes);
      return 1;
    }
  }
  return 0;
}

/* ClosedHashmap::set, closed_hashmap_impl_class.cu:368-427 */
static int orc_set_one(const orc_map *m, const void *key_row, const void *value_row) {
  int64_t start, uuid, first_removed = -1;
  orc_hash_uuid_row(m, key_row, &start, &uuid);
  for (int64_t i = 0; i < m->n_buckets; i++) {
    const int64_t address = trem(wadd(start, i), m->n_buckets);
    const int64_t cand = __atomic_load_n(&m->uuid[address], __ATOMIC_RELAXED);
    if (cand == uuid) {                       /* :382-388 insert-or-assign */
      orc_store_key(m, address, key_row);
      orc_store_value(m, address, value_row);
      return 1;
    }
    if (cand == ORC_REMOVED && first_removed == -1) first_removed = address;   /* :390-393 */
    if (cand == ORC_EMPTY) {                  /* :395-406 */
      if (first_removed == -1) {
        /* set_uuid_if_empty takes `int address` (:184): the truncation is reproduced */
        if (orc_cas(&m->uuid[(int)address], ORC_EMPTY, uuid) == ORC_EMPTY) {
          orc_store_key(m, address, key_row);
          orc_store_value(m, address, value_row);
          return 1;
        }
      } else break;
    }
  }
  if (first_removed != -1) {                  /* :409-425 */
    for (int64_t i = 0; i < m->n_buckets; i++) {
      const int64_t address = trem(wadd(first_removed, i), m->n_buckets);
      if (orc_cas(&m->uuid[(int)address], ORC_REMOVED, uuid) == ORC_REMOVED ||
          orc_cas(&m->uuid[(int)address], ORC_EMPTY, uuid) == ORC_EMPTY) {
        orc_store_key(m, address, key_row);
        orc_store_value(m, address, value_row);
        return 1;
      }
    }
  }
  return 0;
}

/* ClosedHashmap::remove, closed_hashmap_impl_class.cu:459-484: plain store of the tombstone */
static int orc_remove_one(const orc_map *m, const void *key_row) {
  int64_t hash, uuid;
  orc_hash_uuid_row(m, key_row, &hash, &uuid);
  for (int64_t i = 0; i < m->n_buckets; i++) {
    const int64_t address = trem(wadd(hash, i), m->n_buckets);
    const int64_t cand = __atomic_load_n(&m->uuid[address], __ATOMIC_RELAXED);
    if (cand == ORC_EMPTY) break;
    if (cand == uuid) { __atomic_store_n(&m->uuid[address], ORC_REMOVED, __ATOMIC_RELAXED); return 1; }
  }
  return 0;
}

/* ---- batched entry points: one emulated thread per key (closed_hashmap_impl.cu), serial when
 * n_threads <= 1 (canonical order), else contiguous ranges over pthreads (timed CPU baseline). ---- */

enum { OP_GET, OP_SET, OP_REMOVE, OP_EXISTS };

typedef struct {
  const orc_map *m; int op; int64_t lo, hi;
  const char *keys; const char *in_values; char *out_values; uint8_t *flags; int64_t count;
} orc_job;

static void *orc_worker(void *arg) {
  orc_job *j = (orc_job *)arg;
  const orc_map *m = j->m;
  const int64_t kb = (int64_t)m->key_size * orc_elem_bytes(m->key_dtype), vb = m->value_row_bytes;
  int64_t count = 0;
  for (int64_t i = j->lo; i < j->hi; i++) {
    const char *key = j->keys + i * kb;
    int ok = 0;
    switch (j->op) {
      case OP_GET: ok = orc_get_one(m, key, j->out_values + i * vb); break;
      case OP_SET: ok = orc_set_one(m, key, j->in_values + i * vb); break;
      case OP_REMOVE: ok = orc_remove_one(m, key); break;
      default: ok = orc_get_one(m, key, NULL); break;
    }
    if (j->flags) j->flags[i] = (uint8_t)ok;
    count += ok;
  }
  j->count = count;
  return NULL;
}

static int64_t orc_run(const orc_map *m, int op, const void *keys, const void *in_values, void *out_values,
                       uint8_t *flags, int64_t n, int n_threads) {
  if (n_threads < 1) n_threads = 1;
  if (n_threads > 256) n_threads = 256;
  orc_job jobs[256];
  pthread_t tids[256];
  const int64_t per = (n + n_threads - 1) / n_threads;
  int used = 0;
  for (int t = 0; t < n_threads; t++) {
    int64_t lo = t * per, hi = lo + per < n ? lo + per : n;
    if (lo >= hi) break;
    jobs[used] = (orc_job){m, op, lo, hi, (const char *)keys, (const char *)in_values, (char *)out_values, flags, 0};
    used++;
  }
  if (used <= 1) { if (used == 1) orc_worker(&jobs[0]); }
  else {
    for (int t = 0; t < used; t++) pthread_create(&tids[t], NULL, orc_worker, &jobs[t]);
    for (int t = 0; t < used; t++) pthread_join(tids[t], NULL);
  }
  int64_t total = 0;
  for (int t = 0; t < used; t++) total += jobs[t].count;
  return total;
}

/* get launcher + kernel: closed_hashmap_impl.py:102-111 pre-fills `values` with the fallback row and the
 * flags with zero; the kernel (closed_hashmap_impl.cu:70-84) writes the flag always and the value row only
 * on a hit.  fallback == NULL means zeros (:88-93). Returns the number of hits. */
int64_t orc_get(const orc_map *m, const void *keys, int64_t n, void *out_values, const void *fallback,
                uint8_t *out_found, int n_threads) {
  for (int64_t i = 0; i < n; i++) {
    char *dst = (char *)out_values + i * (int64_t)m->value_row_bytes;
    if (fallback) memcpy(dst, fallback, (size_t)m->value_row_bytes); else memset(dst, 0, (size_t)m->value_row_bytes);
  }
  return orc_run(m, OP_GET, keys, NULL, out_values, out_found, n, n_threads);
}

/* closed_hashmap_impl.cu:87-156.  Returns the number of stored rows (is_stored true). */
int64_t orc_set(const orc_map *m, const void *keys, const void *values, int64_t n, uint8_t *out_stored, int n_threads) {
  return orc_run(m, OP_SET, keys, values, NULL, out_stored, n, n_threads);
}

/* closed_hashmap_impl.cu:158-220.  Returns the number of removed rows. */
int64_t orc_remove(const orc_map *m, const void *keys, int64_t n, uint8_t *out_removed, int n_threads) {
  return orc_run(m, OP_REMOVE, keys, NULL, NULL, out_removed, n, n_threads);
}

/* `exists` per key: the count is what sparse_dok_count_items accumulates
 * (sparse_dok_tensor_impl.cu:47-55). out_flags may be NULL. */
int64_t orc_count_exists(const orc_map *m, const void *keys, int64_t n, uint8_t *out_flags, int n_threads) {
  return orc_run(m, OP_EXISTS, keys, NULL, NULL, out_flags, n, n_threads);
}

/* both hashes for a batch of keys (no table access) */
void orc_hash_uuid(const orc_map *m, const void *keys, int64_t n, int64_t *hash_out, int64_t *uuid_out) {
  const int64_t kb = (int64_t)m->key_size * orc_elem_bytes(m->key_dtype);
  for (int64_t i = 0; i < n; i++) {
    int64_t h, u;
    orc_hash_uuid_row(m, (const char *)keys + i * kb, &h, &u);
    if (hash_out) hash_out[i] = h;
    if (uuid_out) uuid_out[i] = u;
  }
}

int orc_sizeof_map(void) { return (int)sizeof(orc_map); }
