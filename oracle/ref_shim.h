/*
 * TEST INFRASTRUCTURE ONLY -- never imported by the product path.
 *
 * Host shim that lets g++ compile the reference's own CUDA C++ text
 * (sparse_dok/components/cuda/closed_hashmap_impl_class.cu,
 *  closed_hashmap_impl.cu, tensor_accessor.cu, sparse_dok_tensor_impl.cu)
 * without modification.  The reference sources are #included by path at build
 * time from the read-only reference checkout; nothing from them is copied here.
 *
 * What the reference prelude (sparse_dok/components/cuda/head.cu:23,32-34,152-188)
 * provides on the device is re-provided here for the host:
 *   ll_t / ull_t typedefs, CUDA_DEVICE_INLINE, the signed 64-bit atomicCAS /
 *   atomicAdd wrappers, __threadfence, and the threadIdx / blockIdx builtins
 *   (thread-local so that several host threads can emulate CUDA threads).
 * Build with -fwrapv: the reference hash relies on wrapping signed overflow
 * (closed_hashmap_impl_class.cu:88-107).
 */
#pragma once
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <thread>
#include <vector>

typedef long long ll_t;
typedef unsigned long long ull_t;

#define CUDA_DEVICE_INLINE inline
#define __global__
#define __device__
#define __forceinline__ inline

struct ref_dim3_t { int x, y, z; };
static thread_local ref_dim3_t threadIdx = {0, 0, 0};
static thread_local ref_dim3_t blockIdx = {0, 0, 0};

static inline void __threadfence() { __atomic_thread_fence(__ATOMIC_SEQ_CST); }

static inline ll_t atomicCAS(ll_t *address, ll_t compare, ll_t val) {
  ll_t expected = compare;
  __atomic_compare_exchange_n(address, &expected, val, false, __ATOMIC_SEQ_CST, __ATOMIC_SEQ_CST);
  return expected;  /* old value, like CUDA's atomicCAS */
}

template <typename T, typename U>
static inline T atomicAdd(T *address, U val) {
  return __atomic_fetch_add(address, (T)val, __ATOMIC_SEQ_CST);
}

/* reduce.cu's warp_sum uses shuffles.  The DOK kernels are emulated with one
 * thread per block (_TPB_=1), so every thread is lane 0 and the warp sum of a
 * single lane is the identity. */
template <typename T, int N>
static inline void warp_sum(T &value) { (void)value; }

/* Runs body(b) for b in [0, n_blocks): in order on the calling thread when
 * n_threads <= 1 (the canonical serial order), otherwise split into contiguous
 * ranges over n_threads std::threads. */
template <typename F>
static inline void ref_for_each_block(ll_t n_blocks, int n_threads, F body) {
  if (n_threads <= 1 || n_blocks < 2) {
    for (ll_t b = 0; b < n_blocks; b++) body(b);
    return;
  }
  std::vector<std::thread> pool;
  const ll_t per = (n_blocks + n_threads - 1) / n_threads;
  for (int t = 0; t < n_threads; t++) {
    const ll_t lo = t * per, hi = (lo + per < n_blocks) ? lo + per : n_blocks;
    if (lo >= hi) break;
    pool.emplace_back([=]() { for (ll_t b = lo; b < hi; b++) body(b); });
  }
  for (auto &th : pool) th.join();
}
