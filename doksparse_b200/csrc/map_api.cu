// C-ABI entry points of the hash map proper (declared in include/doksparse.h).
#include "dok_kernels.cuh"

// ---------------------------------------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------------------------------------
extern "C" {

int dok_version(void) { return 1; }
int dok_last_cuda_error(void) { return dok_last_error_slot(); }
int64_t dok_launch_count(void) { return dok_launch_counter(); }

int dok_bucket_bytes(int value_bytes) {
  if (value_bytes < 1 || value_bytes > DOK_MAX_VALUE_BYTES) return -1;
  const int bb = (8 + value_bytes + 15) / 16 * 16;
  return bb < 16 ? 16 : bb;
}

int dok_map_init(const dok_table *t, void *stream) {
  DevTable dt;
  if (!dok_make_table(t, nullptr, &dt)) return DOK_BAD_ARG;
  const ll_t blocks = (dt.nb + 255) / 256;
  k_init<<<(unsigned)(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, (cudaStream_t)stream>>>(dt);
  return dok_check_launch();
}

int dok_map_uuid(const dok_table *t, const dok_hash_params *hp, const void *keys, int64_t n, int64_t *uuid_out,
                 int64_t *bucket_out, void *stream) {
  DevHash dh;
  DevTable dt;
  memset(&dt, 0, sizeof(dt));
  if (!dok_make_hash(hp, &dh) || n < 0 || (n > 0 && !keys)) return DOK_BAD_ARG;
  if (t && t->n_buckets > 0) {
    dt.nb = t->n_buckets;
    dt.nb_magic = dt.nb > 1 ? (ull_t)((((unsigned __int128)1) << 64) / (ull_t)dt.nb) : 0ULL;
  }
  if (n == 0) return DOK_OK;
  RowKeys rk{keys, n};
  k_uuid<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(dt, dh, rk, (ll_t *)uuid_out, (ll_t *)bucket_out);
  return dok_check_launch();
}

int dok_map_get(const dok_table *t, const dok_hash_params *hp, const void *keys, int64_t n, void *out_values,
                uint8_t *out_found, const void *fallback, int64_t *counters, void *stream) {
  DevHash dh;
  DevTable dt;
  if (!dok_make_hash(hp, &dh) || !dok_make_table(t, &dh, &dt) || n < 0 || n > DOK_MAX_BATCH) return DOK_BAD_ARG;
  if (n > 0 && (!keys || !out_values)) return DOK_BAD_ARG;
  RowKeys rk{keys, n};
  return launch_get(dt, dh, rk, out_values, out_found, fallback, counters, 0, (cudaStream_t)stream);
}

int dok_map_get_probe_stats(const dok_table *t, const dok_hash_params *hp, const void *keys, int64_t n,
                            void *out_values, uint8_t *out_found, int64_t *counters, void *stream) {
  DevHash dh;
  DevTable dt;
  if (!dok_make_hash(hp, &dh) || !dok_make_table(t, &dh, &dt) || n < 0 || n > DOK_MAX_BATCH || !counters) return DOK_BAD_ARG;
  if (n > 0 && (!keys || !out_values)) return DOK_BAD_ARG;
  RowKeys rk{keys, n};
  return launch_get(dt, dh, rk, out_values, out_found, nullptr, counters, 1, (cudaStream_t)stream);
}

int dok_map_set_unique(const dok_table *t, const dok_hash_params *hp, const void *keys, const void *values,
                       int64_t n, uint8_t *out_stored, int64_t *counters, void *stream) {
  DevHash dh;
  DevTable dt;
  if (!dok_make_hash(hp, &dh) || !dok_make_table(t, &dh, &dt) || n < 0 || n > DOK_MAX_BATCH) return DOK_BAD_ARG;
  if (n == 0) return DOK_OK;
  if (!keys || !values) return DOK_BAD_ARG;
  RowKeys rk{keys, n};
  RowValues rv{(const char *)values};
  k_set_unique<<<(unsigned)((n + DOK_TPB - 1) / DOK_TPB), DOK_TPB, 0, (cudaStream_t)stream>>>(
      dt, dh, rk, rv, out_stored, (ll_t *)counters);
  return dok_check_launch();
}

int dok_map_set(const dok_table *t, const dok_hash_params *hp, const void *keys, const void *values, int64_t n,
                int64_t *slot_scratch, int64_t epoch, uint8_t *out_stored, int64_t *counters, void *stream) {
  DevHash dh;
  DevTable dt;
  if (!dok_make_hash(hp, &dh) || !dok_make_table(t, &dh, &dt) || n < 0 || n > DOK_MAX_BATCH) return DOK_BAD_ARG;
  if (n == 0) return DOK_OK;
  if (!keys || !values || !slot_scratch || !dt.stamp || epoch < 1 || epoch > 0x7fffffffLL) return DOK_BAD_ARG;
  RowKeys rk{keys, n};
  RowValues rv{(const char *)values};
  const unsigned grid = (unsigned)((n + DOK_TPB - 1) / DOK_TPB);
  k_set_claim<<<grid, DOK_TPB, 0, (cudaStream_t)stream>>>(dt, dh, rk, (ll_t *)slot_scratch, (ll_t)epoch, (ll_t *)counters);
  int rc = dok_check_launch();
  if (rc != DOK_OK) return rc;
  k_set_write<<<grid, DOK_TPB, 0, (cudaStream_t)stream>>>(dt, dh, rk, rv, (const ll_t *)slot_scratch, (ll_t)epoch, out_stored);
  return dok_check_launch();
}

int dok_map_remove(const dok_table *t, const dok_hash_params *hp, const void *keys, int64_t n, uint8_t *out_removed,
                   int64_t *counters, void *stream) {
  DevHash dh;
  DevTable dt;
  if (!dok_make_hash(hp, &dh) || !dok_make_table(t, &dh, &dt) || n < 0 || n > DOK_MAX_BATCH) return DOK_BAD_ARG;
  if (n == 0) return DOK_OK;
  if (!keys) return DOK_BAD_ARG;
  RowKeys rk{keys, n};
  k_find<1><<<(unsigned)((n + DOK_TPB - 1) / DOK_TPB), DOK_TPB, 0, (cudaStream_t)stream>>>(dt, dh, rk, out_removed, (ll_t *)counters);
  return dok_check_launch();
}

int dok_map_count_exists(const dok_table *t, const dok_hash_params *hp, const void *keys, int64_t n,
                         uint8_t *out_flags, int64_t *counters, void *stream) {
  DevHash dh;
  DevTable dt;
  if (!dok_make_hash(hp, &dh) || !dok_make_table(t, &dh, &dt) || n < 0 || n > DOK_MAX_BATCH) return DOK_BAD_ARG;
  if (n == 0) return DOK_OK;
  if (!keys) return DOK_BAD_ARG;
  RowKeys rk{keys, n};
  k_find<0><<<(unsigned)((n + DOK_TPB - 1) / DOK_TPB), DOK_TPB, 0, (cudaStream_t)stream>>>(dt, dh, rk, out_flags, (ll_t *)counters);
  return dok_check_launch();
}

int dok_map_count_new(const dok_table *t, const dok_hash_params *hp, const void *keys, int64_t n,
                      int64_t *scratch_tags, int64_t scratch_slots, int64_t *counters, void *stream) {
  DevHash dh;
  DevTable dt;
  if (!dok_make_hash(hp, &dh) || !dok_make_table(t, &dh, &dt) || n < 0 || n > DOK_MAX_BATCH) return DOK_BAD_ARG;
  if (n == 0) return DOK_OK;
  if (!keys || !scratch_tags || !counters || scratch_slots < 2 * n) return DOK_BAD_ARG;
  const ll_t blocks = (scratch_slots + 255) / 256;
  k_fill_i64<<<(unsigned)(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, (cudaStream_t)stream>>>(
      (ll_t *)scratch_tags, scratch_slots, DOK_EMPTY);
  int rc = dok_check_launch();
  if (rc != DOK_OK) return rc;
  RowKeys rk{keys, n};
  k_count_new<<<(unsigned)((n + DOK_TPB - 1) / DOK_TPB), DOK_TPB, 0, (cudaStream_t)stream>>>(
      dt, dh, rk, (ll_t *)scratch_tags, scratch_slots, (ll_t *)counters);
  return dok_check_launch();
}

int64_t dok_compact_tiles(int64_t n_buckets) { return (n_buckets + DOK_COMPACT_TILE - 1) / DOK_COMPACT_TILE; }

int dok_map_compact_count(const dok_table *t, int64_t *tile_offsets, void *stream) {
  DevTable dt;
  if (!dok_make_table(t, nullptr, &dt) || !tile_offsets) return DOK_BAD_ARG;
  const ll_t tiles = dok_compact_tiles(dt.nb);
  k_compact_count<<<(unsigned)tiles, DOK_TPB, 0, (cudaStream_t)stream>>>(dt, (ll_t *)tile_offsets);
  int rc = dok_check_launch();
  if (rc != DOK_OK) return rc;
  k_exclusive_scan<<<1, 1024, 0, (cudaStream_t)stream>>>((ll_t *)tile_offsets, tiles);
  return dok_check_launch();
}

int dok_map_compact_scatter(const dok_table *t, const dok_hash_params *hp, const int64_t *tile_offsets, void *keys_out,
                            int keys_transposed, void *values_out, int64_t *uuid_out, void *stream) {
  DevHash dh;
  DevTable dt;
  if (!dok_make_hash(hp, &dh) || !dok_make_table(t, &dh, &dt) || !tile_offsets) return DOK_BAD_ARG;
  const ll_t tiles = dok_compact_tiles(dt.nb);
  k_compact_scatter<<<(unsigned)tiles, DOK_TPB, 0, (cudaStream_t)stream>>>(
      dt, dh, (const ll_t *)tile_offsets, tiles, (char *)keys_out, keys_transposed, (char *)values_out, (ll_t *)uuid_out);
  return dok_check_launch();
}

}  // extern "C"
