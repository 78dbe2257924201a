/*
 * TEST INFRASTRUCTURE ONLY -- never imported by the product path.
 *
 * The reference's own closed_hashmap_{get,set,remove} kernels
 * (sparse_dok/components/cuda/closed_hashmap_impl.cu:6-85, 87-156, 158-220),
 * compiled for the GPU from the files the reference concatenates
 * (closed_hashmap_impl.py:22-27: head, smem_tensor, closed_hashmap_impl_class,
 * closed_hashmap_impl) and launched the way its launcher does
 * (closed_hashmap_impl.py:121-143: ceil(n / (TPB*KPT)) blocks of TPB threads).
 * The reference compiles this text with CuPy at run time; CuPy is not
 * available, so nvcc does it ahead of time with the same placeholder values
 * passed as -D macros.  The sources are read in place; nothing is copied.
 *
 * Used (a) by GPU tests as a second oracle: this library's results against the
 * reference kernels on the same device, and (b) by the reference arm of the
 * benchmark for a kernel-only figure of the reference on the same GPU.
 */
#include <cuda_runtime.h>
#include "head.cu"
#include "smem_tensor.cu"
#include "closed_hashmap_impl_class.cu"
#include "closed_hashmap_impl.cu"

#define REFGPU_HASH_PARAMS                                                     \
  const ll_t *p1, const ll_t *p2, const ll_t *a1, const ll_t *a2,              \
      const ll_t *b1, const ll_t *b2, const ll_t *perm
#define REFGPU_HASH_ARGS p1, p2, a1, a2, b1, b2, perm

static inline unsigned refgpu_blocks(ll_t n) {
  return (unsigned)((n + (ll_t)_TPB_ * _KPT_ - 1) / ((ll_t)_TPB_ * _KPT_));
}

extern "C" {

int refgpu_key_size() { return _KEYSIZE_; }
int refgpu_value_size() { return _VALUESIZE_; }
int refgpu_key_bytes() { return (int)sizeof(KeyType); }
int refgpu_value_bytes() { return (int)sizeof(ValueType); }

/* All pointers are device pointers.  Returns the cudaError_t of the launch. */
int refgpu_get(REFGPU_HASH_PARAMS, const KeyType *keys, ValueType *values,
               KeyType *all_keys, ValueType *all_values, ll_t *all_uuids,
               const ValueType *fallback, uint8_t *is_found, ll_t n_keys,
               ll_t n_buckets, void *stream) {
  if (n_keys <= 0) return 0;
  closed_hashmap_get<<<refgpu_blocks(n_keys), _TPB_, 0, (cudaStream_t)stream>>>(
      REFGPU_HASH_ARGS, keys, values, all_keys, all_values, all_uuids, fallback,
      is_found, n_keys, n_buckets);
  return (int)cudaGetLastError();
}

int refgpu_set(REFGPU_HASH_PARAMS, const KeyType *keys, const ValueType *values,
               KeyType *all_keys, ValueType *all_values, ll_t *all_uuids,
               uint8_t *is_stored, ll_t n_keys, ll_t n_buckets, void *stream) {
  if (n_keys <= 0) return 0;
  closed_hashmap_set<<<refgpu_blocks(n_keys), _TPB_, 0, (cudaStream_t)stream>>>(
      REFGPU_HASH_ARGS, keys, values, all_keys, all_values, all_uuids,
      is_stored, n_keys, n_buckets);
  return (int)cudaGetLastError();
}

int refgpu_remove(REFGPU_HASH_PARAMS, const KeyType *keys, KeyType *all_keys,
                  ValueType *all_values, ll_t *all_uuids, uint8_t *is_removed,
                  ll_t n_keys, ll_t n_buckets, void *stream) {
  if (n_keys <= 0) return 0;
  closed_hashmap_remove<<<refgpu_blocks(n_keys), _TPB_, 0, (cudaStream_t)stream>>>(
      REFGPU_HASH_ARGS, keys, all_keys, all_values, all_uuids, is_removed,
      n_keys, n_buckets);
  return (int)cudaGetLastError();
}

}  /* extern "C" */
