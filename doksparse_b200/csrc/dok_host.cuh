// Host-side helpers shared by the translation units of libdoksparse.so: argument validation, conversion of the
// C-ABI structs into device-ready form, launch error capture.
#pragma once
#include <string.h>
#include "dok_device.cuh"

#define DOK_MAX_BATCH 0xffffffffLL   // row indices are packed into 32 bits of the set stamp

// contiguous value rows [n, value_bytes]
struct RowValues {
  const char *values;
  __device__ __forceinline__ const char *row(const DevTable &t, ll_t e) const { return values + e * (ll_t)t.vb; }
};

inline int &dok_last_error_slot() {
  static thread_local int last = 0;
  return last;
}

// number of kernels this library has launched in this process (every launch is followed by dok_check_launch)
inline long long &dok_launch_counter() {
  static long long count = 0;
  return count;
}

inline int dok_check_launch() {
  dok_launch_counter()++;
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    dok_last_error_slot() = (int)err;
    return DOK_CUDA_ERROR;
  }
  return DOK_OK;
}

inline int dok_dtype_bytes(int dtype) {
  switch (dtype) {
    case DOK_I8: case DOK_U8: return 1;
    case DOK_I16: case DOK_F16: case DOK_BF16: return 2;
    case DOK_I32: case DOK_F32: return 4;
    case DOK_I64: case DOK_F64: return 8;
    default: return 0;
  }
}

// Permutes the hash parameters by key_perm (what the reference's kernel-side constructor does,
// closed_hashmap_impl_class.cu:54-63) and precomputes floor(2^64 / p) per prime.
inline bool dok_make_hash(const dok_hash_params *hp, DevHash *out) {
  if (!hp || hp->key_size < 1 || hp->key_size > DOK_MAX_KEY_SIZE) return false;
  const int eb = dok_dtype_bytes(hp->key_dtype);
  if (eb == 0) return false;
  memset(out, 0, sizeof(*out));
  out->ks = hp->key_size;
  out->dtype = hp->key_dtype;
  out->elem_bytes = eb;
  unsigned seen = 0;
  for (int i = 0; i < hp->key_size; i++) {
    const int c = hp->key_perm[i];
    if (c < 0 || c >= hp->key_size || (seen >> c) & 1u) return false;
    seen |= 1u << c;
    const long long prime = hp->prime2[c];
    const unsigned long long p = prime < 0 ? (0ULL - (unsigned long long)prime) : (unsigned long long)prime;
    if (p < 2) return false;
    const long long prime1 = hp->prime1[c];
    const unsigned long long p1 = prime1 < 0 ? (0ULL - (unsigned long long)prime1) : (unsigned long long)prime1;
    if (p1 < 2) return false;
    out->a[i] = hp->alpha2[c];
    out->b[i] = hp->beta2[c];
    out->p[i] = p;
    out->m[i] = (unsigned long long)((((unsigned __int128)1) << 64) / p);
    out->a1[i] = hp->alpha1[c];
    out->b1[i] = hp->beta1[c];
    out->p1[i] = p1;
    out->m1[i] = (unsigned long long)((((unsigned __int128)1) << 64) / p1);
    out->perm[i] = c;
  }
  return true;
}

inline bool dok_make_table(const dok_table *t, const DevHash *dh, DevTable *out) {
  if (!t || !t->buckets || t->n_buckets < 1) return false;
  if (t->value_bytes < 1 || t->value_bytes > DOK_MAX_VALUE_BYTES) return false;
  const int bb = (8 + t->value_bytes + 15) / 16 * 16;
  if (t->bucket_bytes != bb) return false;
  out->buckets = (char *)t->buckets;
  out->keys = (char *)t->keys;
  out->stamp = (ll_t *)t->stamp;
  out->nb = t->n_buckets;
  out->nb_magic = t->n_buckets > 1 ? (unsigned long long)((((unsigned __int128)1) << 64) / (unsigned long long)t->n_buckets) : 0ULL;
  out->bb = bb;
  out->vb = t->value_bytes;
  out->kb = dh ? dh->ks * dh->elem_bytes : 0;
  out->vwords = (t->value_bytes + 7) / 8;
  return true;
}
