/*
 * TEST INFRASTRUCTURE ONLY -- never imported by the product path.
 *
 * Runs the reference's fused DOK kernels sparse_dok_count_items,
 * sparse_dok_zero_items and sparse_dok_set_items_dense
 * (sparse_dok/components/cuda/sparse_dok_tensor_impl.cu:3-56, 58-108, 270-313)
 * on the host.  They are emulated with one thread per block (_TPB_=1, _EPT_=1):
 * every emulated thread is then lane 0, so the "lane 0 adds the warp total"
 * epilogue (:52-55) adds each thread's own count and the totals equal the
 * device result.  The argument blocks are the reference's own:
 *   hashmap args  = CudaClosedHashmap._kernel_args(as_list=False)
 *                   (sparse_dok/components/cuda_closed_hashmap.py:131-155)
 *   accessor args = util.get_tensor_accessor_argument_array
 *                   (sparse_dok/util.py:295-310)
 * built by the Python side of the oracle with host pointers.
 *
 * Placeholders _SELECTORNDIM_, _NDIM_, _VALUETYPE_ are -D macros.
 */
#include "ref_shim.h"
#include "tensor_accessor.cu"
#include "closed_hashmap_impl_class.cu"
#include "sparse_dok_tensor_impl.cu"

extern "C" {

int refdok_selector_ndim() { return _SELECTORNDIM_; }
int refdok_ndim() { return _NDIM_; }
int refdok_value_bytes() { return (int)sizeof(value_t); }

void refdok_count_items(const ll_t *hashmap_args, const ll_t *accessor_args,
                        const ll_t *real_selector_accessor, ll_t *counts,
                        ll_t n_selector_elements) {
  for (ll_t b = 0; b < n_selector_elements; b++) {
    blockIdx.x = (int)b;
    threadIdx.x = 0;
    sparse_dok_count_items(hashmap_args, accessor_args, real_selector_accessor,
                           counts, n_selector_elements);
  }
}

void refdok_zero_items(const ll_t *hashmap_args, const ll_t *accessor_args,
                       const ll_t *real_selector_accessor, ll_t *n_removed,
                       ll_t n_selector_elements) {
  for (ll_t b = 0; b < n_selector_elements; b++) {
    blockIdx.x = (int)b;
    threadIdx.x = 0;
    sparse_dok_zero_items(hashmap_args, accessor_args, real_selector_accessor,
                          n_removed, n_selector_elements);
  }
}

void refdok_set_items_dense(const ll_t *hashmap_args, const ll_t *accessor_args,
                            const ll_t *real_selector_accessor,
                            ll_t n_selector_elements) {
  for (ll_t b = 0; b < n_selector_elements; b++) {
    blockIdx.x = (int)b;
    threadIdx.x = 0;
    sparse_dok_set_items_dense(hashmap_args, accessor_args,
                               real_selector_accessor, n_selector_elements);
  }
}

}  /* extern "C" */
