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

extern "C" int dok_diag_random_reads(const void *buf, int64_t bytes, int64_t n_reads, uint64_t seed, int64_t *sink,
                                     void *stream) {
  if (!buf || bytes < 16 || n_reads < 1) return DOK_BAD_ARG;
  k_random_reads<<<(unsigned)((n_reads + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const char *)buf, (ull_t)(bytes / 16), n_reads, seed, (ll_t *)sink);
  return dok_check_launch();
}
