// C-ABI entry points of the fused DOK tensor paths (declared in include/doksparse.h): the keys of a batch are
// formed on the fly from broadcast index tensors (or from the position of a non-zero element of a dense
// tensor) instead of being materialised as an int64[n, ndim] matrix first.
#include "dok_kernels.cuh"

// dense source of __setitem__ viewed through the selector's common shape (strides in elements, 0 = broadcast);
// replaces the extra StrictTensorAccessor of sparse_dok_set_items_dense (sparse_dok_tensor_impl.cu:290,309).
struct StridedValues {
  const char *src;
  int selector_ndim;
  ll_t sizes[DOK_MAX_SELECTOR_NDIM];
  ll_t strides[DOK_MAX_SELECTOR_NDIM];
  __device__ __forceinline__ const char *row(const DevTable &t, ll_t e) const {
    ull_t rem = (ull_t)e;
    ll_t off = 0;
    for (int j = selector_ndim - 1; j >= 0; j--) {
      const ull_t size = (ull_t)sizes[j];
      const ull_t q = rem / size;
      off += (ll_t)(rem - q * size) * strides[j];
      rem = q;
    }
    return src + off * (ll_t)t.vb;
  }
};

static bool prepare(const dok_table *t, const dok_hash_params *hp, DevTable *dt, DevHash *dh) {
  if (!dok_make_hash(hp, dh) || !dok_make_table(t, dt)) return false;
  return dt->kb == dh->ks * dh->elem_bytes;
}


static bool make_sel(const dok_selectors *sel, const DevHash &dh, SelKeys *out) {
  if (!sel || sel->ndim != dh.ks || dh.dtype != DOK_I64) return false;
  if (sel->selector_ndim < 0 || sel->selector_ndim > DOK_MAX_SELECTOR_NDIM) return false;
  ll_t n = 1;
  for (int j = 0; j < sel->selector_ndim; j++) {
    if (sel->sizes[j] < 0) return false;
    n *= sel->sizes[j];
  }
  for (int d = 0; d < sel->ndim; d++) if (n > 0 && !sel->ptr[d]) return false;
  out->s = *sel;
  out->n = n;
  return n <= DOK_MAX_BATCH;
}

// ---- from_dense ------------------------------------------------------------------------------------------

template <typename T>
__device__ __forceinline__ bool dok_nonzero(T bits, int is_float) {
  // `x != 0`: for floating types both signed zeros compare equal to zero, NaN does not
  return is_float ? (T)(bits << 1) != 0 : bits != 0;
}

template <typename T>
__global__ void __launch_bounds__(DOK_TPB) k_dense_count(const T *__restrict__ dense, ll_t numel, int is_float, ll_t *count_out) {
  int c = 0;
  const ll_t stride = (ll_t)gridDim.x * DOK_TPB;
  for (ll_t i = (ll_t)blockIdx.x * DOK_TPB + threadIdx.x; i < numel; i += stride) c += dok_nonzero<T>(__ldcs(dense + i), is_float);
  dok_warp_add(count_out, c);
}

struct DenseShape { int ndim; ll_t sizes[DOK_MAX_KEY_SIZE]; };

// A block takes DOK_DENSE_SPAN consecutive elements at a time: every thread looks at DOK_DENSE_ROUNDS of them
// (coalesced), the non-zero ones are collected in shared memory (position inside the span and value), and the block
// then inserts the collected elements 256 at a time with every lane busy.  At the 1 % density of BASELINE config 3 a
// warp of the one-element-per-thread form ran the whole cooperative insert for a single active lane.
#define DOK_DENSE_ROUNDS 8
#define DOK_DENSE_SPAN (DOK_TPB * DOK_DENSE_ROUNDS)

template <int SB, typename T>
__global__ void __launch_bounds__(DOK_TPB) k_dense_insert(DevTable t, DevHash hp, const T *__restrict__ dense, ll_t numel,
                                                          int is_float, DenseShape shape, ll_t *counters) {
  __shared__ T found_value[DOK_DENSE_SPAN];
  __shared__ unsigned short found_at[DOK_DENSE_SPAN];
  __shared__ int n_found;
  const ll_t stride = (ll_t)gridDim.x * DOK_DENSE_SPAN;
  int claimed = 0, reused = 0, failed = 0, hits = 0;
  for (ll_t base = (ll_t)blockIdx.x * DOK_DENSE_SPAN; base < numel; base += stride) {     // uniform over the block
    if (threadIdx.x == 0) n_found = 0;
    __syncthreads();
#pragma unroll
    for (int r = 0; r < DOK_DENSE_ROUNDS; r++) {
      const int j = r * DOK_TPB + (int)threadIdx.x;
      const ll_t i = base + j;
      T v = 0;
      bool nz = false;
      if (i < numel) {
        v = __ldcs(dense + i);
        nz = dok_nonzero<T>(v, is_float);
      }
      const unsigned votes = __ballot_sync(0xffffffffu, nz);
      int at = 0;
      if ((threadIdx.x & 31) == 0 && votes) at = atomicAdd(&n_found, __popc(votes));
      at = __shfl_sync(0xffffffffu, at, 0) + __popc(votes & ((1u << (threadIdx.x & 31)) - 1u));
      if (nz) {
        found_value[at] = v;
        found_at[at] = (unsigned short)j;
      }
    }
    __syncthreads();
    const int total = n_found;
    for (int first = 0; first < total; first += DOK_TPB) {                                // uniform over the block
      const int k = first + (int)threadIdx.x;
      bool active = k < total;
      int outcome = -1;
      T v = 0;
      ll_t idx[DOK_MAX_KEY_SIZE];
      KeyHash kh{0, 0};
      if (active) {
        v = found_value[k];
        // unravel the row-major position into the index tuple; each index is one factor of the hash products
        ull_t rem = (ull_t)(base + found_at[k]);
#pragma unroll
        for (int d = DOK_MAX_KEY_SIZE - 1; d >= 0; d--) {
          idx[d] = 0;
          if (d < shape.ndim) {
            const ull_t size = (ull_t)shape.sizes[d];
            const ull_t q = rem / size;
            idx[d] = (ll_t)(rem - q * size);
            rem = q;
          }
        }
        ll_t u = dok_uuid_term(idx[0], hp.a[0], hp.b[0], hp.p[0], hp.m[0]);
        ull_t h = (ull_t)idx[0] * (ull_t)hp.a1[0] + (ull_t)hp.b1[0];
#pragma unroll
        for (int d = 1; d < DOK_MAX_KEY_SIZE; d++)
          if (d < shape.ndim) {
            u = (ll_t)((ull_t)u * (ull_t)dok_uuid_term(idx[d], hp.a[d], hp.b[d], hp.p[d], hp.m[d]));
            h *= (ull_t)idx[d] * (ull_t)hp.a1[d] + (ull_t)hp.b1[d];
          }
        kh = KeyHash{dok_llabs(u), (ll_t)h};
      }
      active = dok_in_window(t, kh, active);
      const ll_t slot = dok_find_or_claim<SB>(t, kh, active, &outcome);
      if (active && slot >= 0) {
        ll_t *krow = (ll_t *)dok_key_row(t, slot);
#pragma unroll
        for (int d = 0; d < DOK_MAX_KEY_SIZE; d++) if (d < shape.ndim) krow[hp.perm[d]] = idx[d];
        *(T *)dok_value_ptr(t, slot) = v;
      }
      claimed += outcome == DOK_OUT_CLAIMED_EMPTY;
      reused += outcome == DOK_OUT_REUSED;
      failed += outcome == DOK_OUT_FAILED;
      hits += outcome == DOK_OUT_FOUND;
    }
    __syncthreads();                                     // the lists are rewritten by the next span
  }
  if (counters) {
    dok_warp_add(counters + DOK_CNT_CLAIMED_EMPTY, claimed);
    dok_warp_add(counters + DOK_CNT_REUSED_REMOVED, reused);
    dok_warp_add(counters + DOK_CNT_FAILED, failed);
    dok_warp_add(counters + DOK_CNT_HITS, hits);
  }
}

// ---- flatten / reshape: re-key + re-insert in one pass ----------------------------------------------------

struct Rekey {
  int old_ndim, new_ndim;
  int old_perm[DOK_MAX_KEY_SIZE];       // storage column of logical index d in the source table
  ll_t old_strides[DOK_MAX_KEY_SIZE];   // row-major strides of the source shape (logical order)
  ll_t new_sizes[DOK_MAX_KEY_SIZE];     // destination shape
};

// One thread per SOURCE slot: a live slot's index tuple is linearised in the old shape, unravelled in the new one
// and inserted with its value into the destination table -- no compaction of the source, no intermediate tensors
// (the reference goes through indices()/values() and, for reshape, through a whole intermediate flattened tensor:
// sparse_dok_tensor.py:479-514).  Distinct positions stay distinct, so every insert claims a fresh slot.
template <int SB>
__global__ void __launch_bounds__(DOK_TPB) k_rekey_insert(DevTable src, DevTable dst, DevHash hp, Rekey rk, ll_t *counters) {
  const ll_t stride = (ll_t)gridDim.x * DOK_TPB;
  int claimed = 0, failed = 0;
  for (ll_t base = (ll_t)blockIdx.x * DOK_TPB; base < src.nb; base += stride) {       // uniform over the block
    const ll_t s = base + threadIdx.x;
    bool active = false;
    ll_t idx[DOK_MAX_KEY_SIZE];
    KeyHash kh{0, 0};
    if (s < src.nb) {
      const ll_t tag = dok_load_tag(src, s);
      active = tag >= 0;                                  // uuids are non-negative; empty, tombstone, padding are not
    }
    if (active) {
      const ll_t *krow = (const ll_t *)dok_key_row(src, s);
      ull_t linear = 0;
#pragma unroll
      for (int d = 0; d < DOK_MAX_KEY_SIZE; d++)
        if (d < rk.old_ndim) linear += (ull_t)krow[rk.old_perm[d]] * (ull_t)rk.old_strides[d];
#pragma unroll
      for (int d = DOK_MAX_KEY_SIZE - 1; d >= 0; d--) {
        idx[d] = 0;
        if (d < rk.new_ndim) {
          const ull_t size = (ull_t)rk.new_sizes[d];
          const ull_t q = linear / size;
          idx[d] = (ll_t)(linear - q * size);
          linear = q;
        }
      }
      ll_t u = dok_uuid_term(idx[0], hp.a[0], hp.b[0], hp.p[0], hp.m[0]);
      ull_t h = (ull_t)idx[0] * (ull_t)hp.a1[0] + (ull_t)hp.b1[0];
#pragma unroll
      for (int d = 1; d < DOK_MAX_KEY_SIZE; d++)
        if (d < rk.new_ndim) {
          u = (ll_t)((ull_t)u * (ull_t)dok_uuid_term(idx[d], hp.a[d], hp.b[d], hp.p[d], hp.m[d]));
          h *= (ull_t)idx[d] * (ull_t)hp.a1[d] + (ull_t)hp.b1[d];
        }
      kh = KeyHash{dok_llabs(u), (ll_t)h};
    }
    active = dok_in_window(dst, kh, active);
    int outcome = -1;
    const ll_t slot = dok_find_or_claim<SB>(dst, kh, active, &outcome);
    if (active && slot >= 0) {
      ll_t *krow = (ll_t *)dok_key_row(dst, slot);
#pragma unroll
      for (int d = 0; d < DOK_MAX_KEY_SIZE; d++) if (d < rk.new_ndim) krow[hp.perm[d]] = idx[d];
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

// ---- sparse gather: lookup over the selectors and insert of the hits into a second table, one kernel -----

// One thread per selector element: the key formed from the selectors is looked up in `src`; a hit is inserted into
// `dst` under the element's POSITION in the selection (its index tuple in the selection's shape, int64), with the
// stored value.  Positions are pairwise different, so every insert claims a fresh slot.  Replaces
// sparse_dok_get_items (sparse_dok_tensor_impl.cu:110-160), which does the same per thread.
template <int SBS, int SBD>
__global__ void __launch_bounds__(DOK_TPB) k_gather_insert(DevTable src, DevHash shp, SelKeys sel, DevTable dst, DevHash dhp,
                                                           ll_t *counters) {
  ll_t e;
  const bool active = sel.row(e);
  KeyHash kh{0, 0};
  if (active) kh = sel.hash(shp, e);
  const Located loc = dok_locate<SBS, 1, false>(src, kh, e, active, nullptr, NoEmit());
  const bool hit = active && loc.found >= 0;
  ll_t idx[DOK_MAX_KEY_SIZE];
  KeyHash kd{0, 0};
  if (hit) {
    // the element's index tuple in the selection's shape (row-major); a 0-dim selection is position (0,)
    ull_t rem = (ull_t)e;
#pragma unroll
    for (int d = DOK_MAX_KEY_SIZE - 1; d >= 0; d--) {
      idx[d] = 0;
      if (d < sel.s.selector_ndim) {
        const ull_t size = (ull_t)sel.s.sizes[d];
        const ull_t q = rem / size;
        idx[d] = (ll_t)(rem - q * size);
        rem = q;
      }
    }
    ll_t u = dok_uuid_term(idx[0], dhp.a[0], dhp.b[0], dhp.p[0], dhp.m[0]);
    ull_t h = (ull_t)idx[0] * (ull_t)dhp.a1[0] + (ull_t)dhp.b1[0];
#pragma unroll
    for (int d = 1; d < DOK_MAX_KEY_SIZE; d++)
      if (d < dhp.ks) {
        u = (ll_t)((ull_t)u * (ull_t)dok_uuid_term(idx[d], dhp.a[d], dhp.b[d], dhp.p[d], dhp.m[d]));
        h *= (ull_t)idx[d] * (ull_t)dhp.a1[d] + (ull_t)dhp.b1[d];
      }
    kd = KeyHash{dok_llabs(u), (ll_t)h};
  }
  int outcome = -1;
  const ll_t slot = dok_find_or_claim<SBD>(dst, kd, hit, &outcome);
  if (hit && slot >= 0) {
    ll_t *krow = (ll_t *)dok_key_row(dst, slot);
#pragma unroll
    for (int d = 0; d < DOK_MAX_KEY_SIZE; d++) if (d < dhp.ks) krow[dhp.perm[d]] = idx[d];
    dok_store_value(dst, slot, dok_value_ptr(src, loc.found));
  }
  if (counters) {
    dok_warp_add(counters + DOK_CNT_HITS, hit);
    dok_warp_add(counters + DOK_CNT_CLAIMED_EMPTY, outcome == DOK_OUT_CLAIMED_EMPTY || outcome == DOK_OUT_REUSED);
    dok_warp_add(counters + DOK_CNT_FAILED, outcome == DOK_OUT_FAILED);
  }
}

static unsigned streaming_grid(ll_t numel) {
  const ll_t blocks = (numel + DOK_TPB - 1) / DOK_TPB;
  const ll_t cap = 148 * 8;   // 8 resident blocks of 256 threads per SM
  return (unsigned)(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
}

extern "C" {

int dok_dok_get(const dok_table *t, const dok_hash_params *hp, const dok_selectors *sel, void *out_values,
                uint8_t *out_found, const void *fallback, int64_t *counters, void *stream) {
  DevHash dh;
  DevTable dt;
  SelKeys sk;
  if (!prepare(t, hp, &dt, &dh) || !make_sel(sel, dh, &sk)) return DOK_BAD_ARG;
  if (sk.n > 0 && !out_values) return DOK_BAD_ARG;
  return launch_get(dt, dh, sk, out_values, out_found, fallback, counters, 0, (cudaStream_t)stream);
}

int dok_dok_count_exists(const dok_table *t, const dok_hash_params *hp, const dok_selectors *sel, int64_t *counters,
                         void *stream) {
  DevHash dh;
  DevTable dt;
  SelKeys sk;
  if (!prepare(t, hp, &dt, &dh) || !make_sel(sel, dh, &sk) || !counters) return DOK_BAD_ARG;
  if (sk.n == 0) return DOK_OK;
  return launch_find<0>(dt, dh, sk, nullptr, counters, (cudaStream_t)stream);
}

int dok_dok_zero_items(const dok_table *t, const dok_hash_params *hp, const dok_selectors *sel, int64_t *counters,
                       void *stream) {
  DevHash dh;
  DevTable dt;
  SelKeys sk;
  if (!prepare(t, hp, &dt, &dh) || !make_sel(sel, dh, &sk) || !counters) return DOK_BAD_ARG;
  if (sk.n == 0) return DOK_OK;
  return launch_find<1>(dt, dh, sk, nullptr, counters, (cudaStream_t)stream);
}

int dok_dok_set_dense(const dok_table *t, const dok_hash_params *hp, const dok_selectors *sel, const void *src,
                      const int64_t *src_strides, int64_t *slot_scratch, int64_t epoch, int64_t *counters,
                      void *stream) {
  DevHash dh;
  DevTable dt;
  SelKeys sk;
  if (!prepare(t, hp, &dt, &dh) || !make_sel(sel, dh, &sk)) return DOK_BAD_ARG;
  if (sk.n == 0) return DOK_OK;
  if (!src || !src_strides || !slot_scratch || !dok_has_stamps(dt) || epoch < 1 || epoch > DOK_MAX_EPOCH) return DOK_BAD_ARG;
  StridedValues sv;
  sv.src = (const char *)src;
  sv.selector_ndim = sel->selector_ndim;
  for (int j = 0; j < DOK_MAX_SELECTOR_NDIM; j++) {
    sv.sizes[j] = j < sel->selector_ndim ? sel->sizes[j] : 1;
    sv.strides[j] = j < sel->selector_ndim ? src_strides[j] : 0;
  }
  return launch_set_general(dt, dh, sk, sv, slot_scratch, epoch, nullptr, counters, (cudaStream_t)stream);
}

int dok_dok_gather_insert(const dok_table *src, const dok_hash_params *src_hp, const dok_selectors *sel,
                          const dok_table *dst, const dok_hash_params *dst_hp, int64_t *counters, void *stream) {
  DevHash sh, dh;
  DevTable st_, dt;
  SelKeys sk;
  if (!prepare(src, src_hp, &st_, &sh) || !prepare(dst, dst_hp, &dt, &dh) || !make_sel(sel, sh, &sk)) return DOK_BAD_ARG;
  if (dh.dtype != DOK_I64 || st_.vb != dt.vb || dh.ks != (sel->selector_ndim > 0 ? sel->selector_ndim : 1)) return DOK_BAD_ARG;
  if (st_.sb > 128 || dt.sb > 128) return DOK_BAD_ARG;                 // DOK tables: int64 index keys, one value element
  if (dok_window_passes(st_) > 1 || dok_window_passes(dt) > 1) return DOK_TOO_LARGE;   // callers take the two-step route
  if (sk.n == 0) return DOK_OK;
  const unsigned grid = (unsigned)((sk.n + DOK_TPB - 1) / DOK_TPB);
  cudaStream_t st = (cudaStream_t)stream;
#define DOK_GATHER(SBS) \
  switch (dt.sb) { \
    case 32: k_gather_insert<SBS, 32><<<grid, DOK_TPB, 0, st>>>(st_, sh, sk, dt, dh, (ll_t *)counters); break; \
    case 64: k_gather_insert<SBS, 64><<<grid, DOK_TPB, 0, st>>>(st_, sh, sk, dt, dh, (ll_t *)counters); break; \
    default: k_gather_insert<SBS, 128><<<grid, DOK_TPB, 0, st>>>(st_, sh, sk, dt, dh, (ll_t *)counters); break; \
  }
  switch (st_.sb) {
    case 32: DOK_GATHER(32); break;
    case 64: DOK_GATHER(64); break;
    default: DOK_GATHER(128); break;
  }
#undef DOK_GATHER
  return dok_check_launch();
}

int dok_dok_rekey_insert(const dok_table *src, const dok_hash_params *src_hp, const int64_t *src_sizes,
                         const dok_table *dst, const dok_hash_params *dst_hp, const int64_t *dst_sizes,
                         int64_t *counters, void *stream) {
  DevHash sh, dh;
  DevTable st_, dt;
  if (!prepare(src, src_hp, &st_, &sh) || !prepare(dst, dst_hp, &dt, &dh)) return DOK_BAD_ARG;
  if (sh.dtype != DOK_I64 || dh.dtype != DOK_I64 || !src_sizes || !dst_sizes || st_.vb != dt.vb) return DOK_BAD_ARG;
  Rekey rk;
  memset(&rk, 0, sizeof(rk));
  rk.old_ndim = sh.ks;
  rk.new_ndim = dh.ks;
  ll_t old_total = 1, new_total = 1;
  for (int d = sh.ks - 1; d >= 0; d--) {
    if (src_sizes[d] < 1) return DOK_BAD_ARG;
    rk.old_strides[d] = old_total;
    rk.old_perm[d] = sh.perm[d];
    old_total *= src_sizes[d];
  }
  for (int d = 0; d < dh.ks; d++) {
    if (dst_sizes[d] < 1) return DOK_BAD_ARG;
    rk.new_sizes[d] = dst_sizes[d];
    new_total *= dst_sizes[d];
  }
  if (old_total != new_total) return DOK_BAD_ARG;
  const unsigned grid = streaming_grid(st_.nb);
  int rc = DOK_OK;
  DOK_DISPATCH_SB(dt, DOK_FOR_WINDOWS(dt, rc, (k_rekey_insert<SB><<<grid, DOK_TPB, 0, (cudaStream_t)stream>>>(st_, wt, dh, rk, (ll_t *)counters))));
  return rc;
}

int dok_dense_count_nonzero(const void *dense, int64_t numel, int elem_bytes, int is_float, int64_t *count_out,
                            void *stream) {
  if (numel < 0 || !count_out || (numel > 0 && !dense)) return DOK_BAD_ARG;
  if (numel == 0) return DOK_OK;
  const unsigned grid = streaming_grid(numel);
  cudaStream_t st = (cudaStream_t)stream;
  switch (elem_bytes) {
    case 1: k_dense_count<unsigned char><<<grid, DOK_TPB, 0, st>>>((const unsigned char *)dense, numel, is_float, (ll_t *)count_out); break;
    case 2: k_dense_count<unsigned short><<<grid, DOK_TPB, 0, st>>>((const unsigned short *)dense, numel, is_float, (ll_t *)count_out); break;
    case 4: k_dense_count<unsigned><<<grid, DOK_TPB, 0, st>>>((const unsigned *)dense, numel, is_float, (ll_t *)count_out); break;
    case 8: k_dense_count<ull_t><<<grid, DOK_TPB, 0, st>>>((const ull_t *)dense, numel, is_float, (ll_t *)count_out); break;
    default: return DOK_BAD_ARG;
  }
  return dok_check_launch();
}

int dok_dense_insert_nonzero(const dok_table *t, const dok_hash_params *hp, const void *dense, const int64_t *sizes,
                             int64_t numel, int is_float, int64_t *counters, void *stream) {
  DevHash dh;
  DevTable dt;
  if (!prepare(t, hp, &dt, &dh) || dh.dtype != DOK_I64 || !sizes || numel < 0) return DOK_BAD_ARG;
  if (numel == 0) return DOK_OK;
  if (!dense) return DOK_BAD_ARG;
  DenseShape shape;
  shape.ndim = dh.ks;
  ll_t prod = 1;
  for (int d = 0; d < DOK_MAX_KEY_SIZE; d++) {
    shape.sizes[d] = d < dh.ks ? sizes[d] : 1;
    if (shape.sizes[d] < 1) return DOK_BAD_ARG;
    prod *= shape.sizes[d];
  }
  if (prod != numel) return DOK_BAD_ARG;
  const unsigned grid = streaming_grid((numel + DOK_DENSE_ROUNDS - 1) / DOK_DENSE_ROUNDS);
  cudaStream_t st = (cudaStream_t)stream;
  int rc = DOK_OK;
  switch (dt.vb) {
    case 1: DOK_DISPATCH_SB(dt, DOK_FOR_WINDOWS(dt, rc, (k_dense_insert<SB, unsigned char><<<grid, DOK_TPB, 0, st>>>(wt, dh, (const unsigned char *)dense, numel, is_float, shape, (ll_t *)counters)))); break;
    case 2: DOK_DISPATCH_SB(dt, DOK_FOR_WINDOWS(dt, rc, (k_dense_insert<SB, unsigned short><<<grid, DOK_TPB, 0, st>>>(wt, dh, (const unsigned short *)dense, numel, is_float, shape, (ll_t *)counters)))); break;
    case 4: DOK_DISPATCH_SB(dt, DOK_FOR_WINDOWS(dt, rc, (k_dense_insert<SB, unsigned><<<grid, DOK_TPB, 0, st>>>(wt, dh, (const unsigned *)dense, numel, is_float, shape, (ll_t *)counters)))); break;
    case 8: DOK_DISPATCH_SB(dt, DOK_FOR_WINDOWS(dt, rc, (k_dense_insert<SB, ull_t><<<grid, DOK_TPB, 0, st>>>(wt, dh, (const ull_t *)dense, numel, is_float, shape, (ll_t *)counters)))); break;
    default: return DOK_BAD_ARG;
  }
  return rc;
}

}  // extern "C"
