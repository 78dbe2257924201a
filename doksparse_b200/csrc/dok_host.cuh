// Host-side helpers shared by the translation units of libdoksparse.so: argument validation, conversion of the
// C-ABI structs into device-ready form, launch error capture.
#pragma once
#include <string.h>
#include <atomic>
#include "dok_device.cuh"

#define DOK_MAX_BATCH 0xffffffffLL   // row indices are packed into 32 bits of the set stamp
#define DOK_MAX_EPOCH 0x3fffffffLL   // 30 bits of the stamp above the row index and the conflict bit

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
inline std::atomic<long long> &dok_launch_counter() {
  static std::atomic<long long> count{0};
  return count;
}

inline int dok_check_launch() {
  dok_launch_counter().fetch_add(1, std::memory_order_relaxed);
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
    out->a[i] = hp->alpha2[c];
    out->b[i] = hp->beta2[c];
    out->p[i] = p;
    out->m[i] = (unsigned long long)((((unsigned __int128)1) << 64) / p);
    out->a1[i] = hp->alpha1[c] | 1;     // odd: the linear term is then injective in the key element
    out->b1[i] = hp->beta1[c];
    out->perm[i] = c;
  }
  return true;
}

// Slot geometry for (value_bytes, key_bytes): {tag 8 | value, padded to 8 | key row, padded to 8 | stamp 8 if it
// fits without growing the slot}, padded to 32, 64 or 128 bytes (4, 2 or 1 slots per 128-byte line); wider rows
// take a whole number of lines and always carry their stamp.
struct DokLayout { int sb, spg, val_off, key_off, stamp_off; };

inline bool dok_layout(int value_bytes, int key_bytes, DokLayout *out) {
  if (value_bytes < 1 || value_bytes > DOK_MAX_VALUE_BYTES || key_bytes < 1 || key_bytes > 8 * DOK_MAX_KEY_SIZE) return false;
  const int key_off = 8 + (value_bytes + 7) / 8 * 8;
  const int need = key_off + (key_bytes + 7) / 8 * 8;      // without the stamp
  int sb;
  if (need <= 128) { sb = 32; while (sb < need) sb *= 2; }
  else sb = (need + 8 + 127) / 128 * 128;
  out->sb = sb;
  out->spg = sb <= 128 ? 128 / sb : 1;
  out->val_off = 8;
  out->key_off = key_off;
  out->stamp_off = need + 8 <= sb ? need : -1;
  return true;
}

inline bool dok_make_table(const dok_table *t, DevTable *out) {
  if (!t || !t->slots || t->n_buckets < 1) return false;
  DokLayout lay;
  if (!dok_layout(t->value_bytes, t->key_bytes, &lay) || t->slot_bytes != lay.sb) return false;
  out->slots = (char *)t->slots;
  out->stamp = (ll_t *)t->stamp;
  out->nb = t->n_buckets;
  out->n_groups = (t->n_buckets + lay.spg - 1) / lay.spg;
  out->n_slots = out->n_groups * lay.spg;
  out->sb = lay.sb;
  out->spg = lay.spg;
  out->vb = t->value_bytes;
  out->kb = t->key_bytes;
  out->val_off = lay.val_off;
  out->key_off = lay.key_off;
  out->stamp_off = lay.stamp_off;
  out->vwords = (t->value_bytes + 7) / 8;
  out->win_lo = out->win_hi = 0;
  if (lay.sb <= 128 && out->n_slots >= 0xffffffffLL) return false;    // the cooperative walk keeps slot indices in 32 bits
  return true;
}

// Passes over a batch for tables beyond the TLB's reach (see DevTable::win_lo).  Measured on B200 (2 MiB pages):
// random 16-byte reads run at 46.8 / 44.6 / 40.2 / 28.4 / 18.1 / 13.9 G/s over 4 / 64 / 72 / 80 / 96 / 114 GiB, i.e. the
// TLB covers 64 GiB and a walk-bound regime follows; a pass costs about a quarter more per row than an unfiltered
// launch.  So: one pass up to single_pass_limit, beyond it ceil(bytes / window_bytes) windows of equal size.
struct DokWindowCfg { long long single_pass_limit, window_bytes; };
inline DokWindowCfg &dok_window_cfg() {
  static DokWindowCfg cfg{72LL << 30, 58LL << 30};
  return cfg;
}
inline int dok_window_passes(const DevTable &t) {
  const long long bytes = t.n_groups * (long long)(t.sb <= 128 ? 128 : t.sb) + (t.stamp ? t.n_slots * 8 : 0);
  const DokWindowCfg &cfg = dok_window_cfg();
  if (bytes <= cfg.single_pass_limit) return 1;
  const long long passes = (bytes + cfg.window_bytes - 1) / cfg.window_bytes;
  return (int)(passes < t.n_groups ? passes : t.n_groups);
}
inline DevTable dok_window(const DevTable &t, int w, int passes) {
  DevTable o = t;
  o.win_lo = o.win_hi = 0;
  if (passes > 1) {
    o.win_lo = (ll_t)((__int128)t.n_groups * w / passes);
    o.win_hi = (ll_t)((__int128)t.n_groups * (w + 1) / passes);
  }
  return o;
}
// runs LAUNCH (which uses the DevTable `wt`) once per window and leaves the first failure in `rc`
#define DOK_FOR_WINDOWS(dt, rc, LAUNCH)                                        \
  do {                                                                         \
    const int passes_ = dok_window_passes(dt);                                 \
    for (int w_ = 0; w_ < passes_ && (rc) == DOK_OK; w_++) {                   \
      const DevTable wt = dok_window(dt, w_, passes_);                         \
      LAUNCH;                                                                  \
      (rc) = dok_check_launch();                                               \
    }                                                                          \
  } while (0)

// true when a general set can run on this table: the stamps are in the slots or the caller supplied the array
inline bool dok_has_stamps(const DevTable &t) { return t.stamp_off >= 0 || t.stamp != nullptr; }
