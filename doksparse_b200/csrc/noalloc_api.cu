// dok_map_count_new_static: dok_map_count_new for callers that cannot hand the library a scratch buffer.
//
// Who that is: a host program that binds this C ABI directly (no PyTorch caching allocator behind it) and has
// committed its device memory up front -- a table sized to most of the GPU, the rest reserved -- or that answers
// requests in a loop where a cudaMalloc / cudaFree pair per call is not acceptable, because both synchronise the
// whole device.  Such a caller still needs the exact number of distinct new keys of a batch before it can decide
// whether the table must grow, and that count needs a scratch tag set.  Here the set lives in a fixed array inside
// the library image: every GPU that loads libdoksparse.so holds these 8 MiB until the process exits.
//
// Limits and rules:
//   * at most DOK_STATIC_SCRATCH_ROWS rows per call (the tag set holds twice as many slots); larger batches are
//     refused with DOK_TOO_LARGE, nothing is launched;
//   * the first call on a device looks up the array's device address (cudaGetSymbolAddress, once per device, with
//     that device current) -- make that first call before any stream capture begins;
//   * the array is shared by all calls on a device and keeps the previous call's tags, so every call refills the
//     part it uses before counting; two calls that overlap on the GPU (different streams, or different host
//     threads) race on it -- issue them on one stream, or serialise them yourself;
//   * no cudaMalloc, cudaFree or any other allocating routine is called.
#include <mutex>
#include "dok_kernels.cuh"

#define DOK_STATIC_SCRATCH_ROWS (1 << 19)
#define DOK_STATIC_SCRATCH_SLOTS (2 * DOK_STATIC_SCRATCH_ROWS)
#define DOK_MAX_DEVICES 64

// In host code this name is only a handle for the runtime, never a device address.
static __device__ __align__(256) long long dok_static_scratch[DOK_STATIC_SCRATCH_SLOTS];

static std::mutex g_scratch_mutex;
static long long *g_scratch_ptr[DOK_MAX_DEVICES];     // device address of dok_static_scratch, per device

// Device address of the static scratch on the CURRENT device, looked up once per device.
static int static_scratch_address(long long **out) {
  int dev = -1;
  const cudaError_t dev_err = cudaGetDevice(&dev);
  if (dev_err != cudaSuccess || dev < 0 || dev >= DOK_MAX_DEVICES) {
    dok_last_error_slot() = (int)(dev_err != cudaSuccess ? dev_err : cudaErrorInvalidDevice);
    cudaGetLastError();
    return DOK_CUDA_ERROR;
  }
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void *p = nullptr;
    const cudaError_t err = cudaGetSymbolAddress(&p, dok_static_scratch);
    if (err != cudaSuccess || p == nullptr) {
      dok_last_error_slot() = (int)err;
      return DOK_CUDA_ERROR;
    }
    g_scratch_ptr[dev] = (long long *)p;
  }
  *out = g_scratch_ptr[dev];
  return DOK_OK;
}

extern "C" {

int64_t dok_static_scratch_max_rows(void) { return DOK_STATIC_SCRATCH_ROWS; }

int dok_map_count_new_static(const dok_table *t, const dok_hash_params *hp, const void *keys, int64_t n,
                             int64_t *counters, void *stream) {
  DevHash dh;
  DevTable dt;
  if (!dok_make_hash(hp, &dh) || !dok_make_table(t, &dt) || dt.kb != dh.ks * dh.elem_bytes || n < 0) return DOK_BAD_ARG;
  if (n > DOK_STATIC_SCRATCH_ROWS) return DOK_TOO_LARGE;    // the fixed tag set cannot hold 2 * n slots
  if (n == 0) return DOK_OK;
  if (!keys || !counters) return DOK_BAD_ARG;
  long long *scratch = nullptr;
  int rc = static_scratch_address(&scratch);
  if (rc != DOK_OK) return rc;
  // the tag set of this call: 2 * n slots, refilled because the array still holds the previous call's tags
  const ll_t slots = 2 * n;
  const ll_t blocks = (slots + 255) / 256;
  cudaStream_t st = (cudaStream_t)stream;
  k_fill_i64<<<(unsigned)(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, st>>>(scratch, slots, DOK_EMPTY);
  rc = dok_check_launch();
  if (rc != DOK_OK) return rc;
  RowKeys rk{keys, n};
  const unsigned grid = (unsigned)((n + DOK_TPB - 1) / DOK_TPB);
  rc = DOK_OK;
  DOK_DISPATCH_SB(dt, DOK_FOR_WINDOWS(dt, rc, (k_count_new<SB><<<grid, DOK_TPB, 0, st>>>(wt, dh, rk, scratch, slots, (ll_t *)counters))));
  return rc;
}

}  // extern "C"
