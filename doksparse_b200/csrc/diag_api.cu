// Diagnostic entry point (declared in include/doksparse.h): the rate at which this GPU serves independent random
// 16-byte reads over a buffer.  For buffers much larger than L2 it is the ceiling of any probing kernel, because
// every access instruction-lane costs the same whatever it moves; the benchmark reports it next to the roofline.
#include "dok_host.cuh"

static __global__ void __launch_bounds__(256) k_random_reads(const char *__restrict__ buf, ull_t n_units, ll_t n, ull_t seed,
                                                            ll_t *sink) {
  const ll_t i = (ll_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= n) return;
  const ull_t u = __umul64hi(dok_mix64((ull_t)i + seed), n_units);
  const ulonglong2 v = __ldcg((const ulonglong2 *)(buf + u * 16));
  if ((v.x ^ v.y) == 0x9e3779b97f4a7c15ULL && sink) *sink = (ll_t)v.x;      // keeps the load alive
}

// The same with a chosen request shape: `lanes` (1, 2, 4) adjacent lanes read `bytes_per_lane` (8, 16, 32) each of ONE
// random, naturally aligned unit of lanes * bytes_per_lane bytes, i.e. requests of 8 ... 128 bytes.  Counting DRAM
// bytes per request under ncu for the different shapes shows what a random access costs in DRAM traffic.
template <int BYTES, int LANES>
static __global__ void __launch_bounds__(256) k_random_requests(const char *__restrict__ buf, ull_t n_units, ll_t n_threads,
                                                                ull_t seed, ll_t *sink) {
  const ll_t i = (ll_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= n_threads) return;
  const ull_t unit = __umul64hi(dok_mix64((ull_t)(i / LANES) + seed), n_units);
  const char *p = buf + unit * (ull_t)(BYTES * LANES) + (ull_t)(i % LANES) * BYTES;
  ull_t acc;
  if (BYTES == 8) {
    acc = __ldcg((const ull_t *)p);
  } else if (BYTES == 16) {
    const ulonglong2 v = __ldcg((const ulonglong2 *)p);
    acc = v.x ^ v.y;
  } else {
    ull_t a, b, c, d;
    asm volatile("ld.global.cg.v4.u64 {%0,%1,%2,%3}, [%4];" : "=l"(a), "=l"(b), "=l"(c), "=l"(d) : "l"(p));
    acc = a ^ b ^ c ^ d;
  }
  if (acc == 0x9e3779b97f4a7c15ULL && sink) *sink = (ll_t)acc;      // keeps the load alive
}

extern "C" int dok_diag_random_requests(const void *buf, int64_t bytes, int64_t n_requests, int bytes_per_lane, int lanes,
                                        uint64_t seed, int64_t *sink, void *stream) {
  if (!buf || n_requests < 1 || bytes < (int64_t)bytes_per_lane * lanes) return DOK_BAD_ARG;
  const ull_t units = (ull_t)(bytes / ((int64_t)bytes_per_lane * lanes));
  const ll_t threads = n_requests * lanes;
  const unsigned grid = (unsigned)((threads + 255) / 256);
  cudaStream_t st = (cudaStream_t)stream;
#define DOK_REQ(B, LN) k_random_requests<B, LN><<<grid, 256, 0, st>>>((const char *)buf, units, threads, seed, (ll_t *)sink)
  if (bytes_per_lane == 8 && lanes == 1) DOK_REQ(8, 1);
  else if (bytes_per_lane == 16 && lanes == 1) DOK_REQ(16, 1);
  else if (bytes_per_lane == 32 && lanes == 1) DOK_REQ(32, 1);
  else if (bytes_per_lane == 32 && lanes == 2) DOK_REQ(32, 2);
  else if (bytes_per_lane == 32 && lanes == 4) DOK_REQ(32, 4);
  else if (bytes_per_lane == 16 && lanes == 4) DOK_REQ(16, 4);
  else return DOK_BAD_ARG;
#undef DOK_REQ
  return dok_check_launch();
}

extern "C" int dok_diag_random_reads(const void *buf, int64_t bytes, int64_t n_reads, uint64_t seed, int64_t *sink,
                                     void *stream) {
  if (!buf || bytes < 16 || n_reads < 1) return DOK_BAD_ARG;
  k_random_reads<<<(unsigned)((n_reads + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const char *)buf, (ull_t)(bytes / 16), n_reads, seed, (ll_t *)sink);
  return dok_check_launch();
}
