/*
 * TEST INFRASTRUCTURE ONLY -- never imported by the product path.
 *
 * Runs the reference's own closed_hashmap_{get,set,remove} kernels
 * (sparse_dok/components/cuda/closed_hashmap_impl.cu:6-85, 87-156, 158-220) on
 * the host by looping over the emulated (blockIdx.x, threadIdx.x) grid that the
 * reference launcher uses (closed_hashmap_impl.py:121-122: ceil(n/256) blocks
 * of 256 threads, one key per thread).
 *
 * One shared object is built per (key type, value type, key size, value size):
 * the reference's textual placeholders _KEYTYPE_, _VALUETYPE_, _KEYSIZE_,
 * _VALUESIZE_, _TPB_, _KPT_ (closed_hashmap_impl.py:33-40) are passed as -D
 * macros by oracle/Makefile.
 *
 * n_threads == 1 is the serial, canonical order (thread 0 of block 0 first);
 * n_threads > 1 distributes blocks over host threads and is only used as a
 * timed CPU baseline.
 */
#include "ref_shim.h"
#include "closed_hashmap_impl_class.cu"
#include "closed_hashmap_impl.cu"

#define REF_ARGS_HASH                                                          \
  const ll_t *p1, const ll_t *p2, const ll_t *a1, const ll_t *a2,              \
      const ll_t *b1, const ll_t *b2, const ll_t *perm

extern "C" {

int ref_key_size() { return _KEYSIZE_; }
int ref_value_size() { return _VALUESIZE_; }
int ref_key_bytes() { return (int)sizeof(KeyType); }
int ref_value_bytes() { return (int)sizeof(ValueType); }

void ref_get(REF_ARGS_HASH, const KeyType *keys, ValueType *values,
             KeyType *all_keys, ValueType *all_values, ll_t *all_uuids,
             const ValueType *fallback, uint8_t *is_found, ll_t n_keys,
             ll_t n_buckets, int n_threads) {
  const ll_t n_blocks = (n_keys + _TPB_ * _KPT_ - 1) / (_TPB_ * _KPT_);
  ref_for_each_block(n_blocks, n_threads, [=](ll_t b) {
    for (int t = 0; t < _TPB_; t++) {
      blockIdx.x = (int)b;
      threadIdx.x = t;
      closed_hashmap_get(p1, p2, a1, a2, b1, b2, perm, keys, values, all_keys,
                         all_values, all_uuids, fallback, is_found, n_keys,
                         n_buckets);
    }
  });
}

void ref_set(REF_ARGS_HASH, const KeyType *keys, const ValueType *values,
             KeyType *all_keys, ValueType *all_values, ll_t *all_uuids,
             uint8_t *is_stored, ll_t n_keys, ll_t n_buckets, int n_threads) {
  const ll_t n_blocks = (n_keys + _TPB_ * _KPT_ - 1) / (_TPB_ * _KPT_);
  ref_for_each_block(n_blocks, n_threads, [=](ll_t b) {
    for (int t = 0; t < _TPB_; t++) {
      blockIdx.x = (int)b;
      threadIdx.x = t;
      closed_hashmap_set(p1, p2, a1, a2, b1, b2, perm, keys, values, all_keys,
                         all_values, all_uuids, is_stored, n_keys, n_buckets);
    }
  });
}

void ref_remove(REF_ARGS_HASH, const KeyType *keys, KeyType *all_keys,
                ValueType *all_values, ll_t *all_uuids, uint8_t *is_removed,
                ll_t n_keys, ll_t n_buckets, int n_threads) {
  const ll_t n_blocks = (n_keys + _TPB_ * _KPT_ - 1) / (_TPB_ * _KPT_);
  ref_for_each_block(n_blocks, n_threads, [=](ll_t b) {
    for (int t = 0; t < _TPB_; t++) {
      blockIdx.x = (int)b;
      threadIdx.x = t;
      closed_hashmap_remove(p1, p2, a1, a2, b1, b2, perm, keys, all_keys,
                            all_values, all_uuids, is_removed, n_keys,
                            n_buckets);
    }
  });
}

/* The two device hash functions on their own (closed_hashmap_impl_class.cu:87-107),
 * through the permuting constructor (:32-64) exactly as the kernels build it. */
void ref_hash_uuid(REF_ARGS_HASH, const KeyType *keys, ll_t *hash_out,
                   ll_t *uuid_out, ll_t n_keys) {
  ClosedHashmap<KeyType, ValueType, _KEYSIZE_, _VALUESIZE_> hashmap(
      p1, p2, a1, a2, b1, b2, perm, nullptr, nullptr, nullptr, 1, -1, -3);
  for (ll_t i = 0; i < n_keys; i++) {
    KeyType key[_KEYSIZE_];
    for (int j = 0; j < _KEYSIZE_; j++) key[j] = keys[i * _KEYSIZE_ + j];
    hash_out[i] = hashmap.get_hash(key);
    uuid_out[i] = hashmap.get_uuid(key);
  }
}

}  /* extern "C" */
