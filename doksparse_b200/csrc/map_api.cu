// C-ABI entry points of the hash map proper (declared in include/doksparse.h).
#include "dok_kernels.cuh"

static bool prepare(const dok_table *t, const dok_hash_params *hp, DevTable *dt, DevHash *dh) {
  if (!dok_make_hash(hp, dh) || !dok_make_table(t, dt)) return false;
  return dt->kb == dh->ks * dh->elem_bytes;
}

static unsigned grid_for(ll_t n) { return (unsigned)((n + DOK_TPB - 1) / DOK_TPB); }

extern "C" {

int dok_version(void) { return 2; }
int dok_last_cuda_error(void) { return dok_last_error_slot(); }
int64_t dok_launch_count(void) { return dok_launch_counter(); }

int dok_table_layout(int value_bytes, int key_bytes, int64_t n_buckets, dok_layout_info *out) {
  DokLayout lay;
  if (!out || n_buckets < 1 || !dok_layout(value_bytes, key_bytes, &lay)) return DOK_BAD_ARG;
  out->slot_bytes = lay.sb;
  out->slots_per_group = lay.spg;
  out->value_offset = lay.val_off;
  out->key_offset = lay.key_off;
  out->stamp_offset = lay.stamp_off;
  out->reserved = 0;
  out->n_slots = (n_buckets + lay.spg - 1) / lay.spg * lay.spg;
  out->total_bytes = out->n_slots * lay.sb;
  return DOK_OK;
}

int dok_map_init(const dok_table *t, void *stream) {
  DevTable dt;
  if (!dok_make_table(t, &dt)) return DOK_BAD_ARG;
  const ll_t blocks = (dt.n_slots + 255) / 256;
  k_init<<<(unsigned)(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, (cudaStream_t)stream>>>(dt);
  return dok_check_launch();
}

int dok_map_uuid(const dok_table *t, const dok_hash_params *hp, const void *keys, int64_t n, int64_t *uuid_out,
                 int64_t *slot_out, void *stream) {
  DevHash dh;
  DevTable dt;
  memset(&dt, 0, sizeof(dt));
  if (!dok_make_hash(hp, &dh) || n < 0 || (n > 0 && !keys)) return DOK_BAD_ARG;
  if (t && !dok_make_table(t, &dt)) return DOK_BAD_ARG;
  if (slot_out && !t) return DOK_BAD_ARG;
  if (n == 0) return DOK_OK;
  RowKeys rk{keys, n};
  k_uuid<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(dt, dh, rk, (ll_t *)uuid_out, (ll_t *)slot_out);
  return dok_check_launch();
}

int dok_map_get(const dok_table *t, const dok_hash_params *hp, const void *keys, int64_t n, void *out_values,
                uint8_t *out_found, const void *fallback, int64_t *counters, void *stream) {
  DevHash dh;
  DevTable dt;
  if (!prepare(t, hp, &dt, &dh) || n < 0 || n > DOK_MAX_BATCH) return DOK_BAD_ARG;
  if (n > 0 && (!keys || !out_values)) return DOK_BAD_ARG;
  RowKeys rk{keys, n};
  return launch_get(dt, dh, rk, out_values, out_found, fallback, counters, 0, (cudaStream_t)stream);
}

int dok_map_get_probe_stats(const dok_table *t, const dok_hash_params *hp, const void *keys, int64_t n,
                            void *out_values, uint8_t *out_found, int64_t *counters, void *stream) {
  DevHash dh;
  DevTable dt;
  if (!prepare(t, hp, &dt, &dh) || n < 0 || n > DOK_MAX_BATCH || !counters) return DOK_BAD_ARG;
  if (n > 0 && (!keys || !out_values)) return DOK_BAD_ARG;
  RowKeys rk{keys, n};
  return launch_get(dt, dh, rk, out_values, out_found, nullptr, counters, 1, (cudaStream_t)stream);
}

int dok_map_set_unique(const dok_table *t, const dok_hash_params *hp, const void *keys, const void *values,
                       int64_t n, uint8_t *out_stored, int64_t *counters, void *stream) {
  DevHash dh;
  DevTable dt;
  if (!prepare(t, hp, &dt, &dh) || n < 0 || n > DOK_MAX_BATCH) return DOK_BAD_ARG;
  if (n == 0) return DOK_OK;
  if (!keys || !values) return DOK_BAD_ARG;
  RowKeys rk{keys, n};
  return launch_set_unique(dt, dh, rk, (const char *)values, out_stored, counters, (cudaStream_t)stream);
}

int dok_map_set(const dok_table *t, const dok_hash_params *hp, const void *keys, const void *values, int64_t n,
                int64_t *slot_scratch, int64_t epoch, uint8_t *out_stored, int64_t *counters, void *stream) {
  DevHash dh;
  DevTable dt;
  if (!prepare(t, hp, &dt, &dh) || n < 0 || n > DOK_MAX_BATCH) return DOK_BAD_ARG;
  if (n == 0) return DOK_OK;
  if (!keys || !values || !slot_scratch || !dok_has_stamps(dt) || epoch < 1 || epoch > DOK_MAX_EPOCH) return DOK_BAD_ARG;
  RowKeys rk{keys, n};
  return launch_set(dt, dh, rk, (const char *)values, slot_scratch, epoch, out_stored, counters, (cudaStream_t)stream);
}

int dok_map_remove(const dok_table *t, const dok_hash_params *hp, const void *keys, int64_t n, uint8_t *out_removed,
                   int64_t *counters, void *stream) {
  DevHash dh;
  DevTable dt;
  if (!prepare(t, hp, &dt, &dh) || n < 0 || n > DOK_MAX_BATCH) return DOK_BAD_ARG;
  if (n == 0) return DOK_OK;
  if (!keys) return DOK_BAD_ARG;
  RowKeys rk{keys, n};
  return launch_find<1>(dt, dh, rk, out_removed, counters, (cudaStream_t)stream);
}

int dok_map_count_exists(const dok_table *t, const dok_hash_params *hp, const void *keys, int64_t n,
                         uint8_t *out_flags, int64_t *counters, void *stream) {
  DevHash dh;
  DevTable dt;
  if (!prepare(t, hp, &dt, &dh) || n < 0 || n > DOK_MAX_BATCH) return DOK_BAD_ARG;
  if (n == 0) return DOK_OK;
  if (!keys) return DOK_BAD_ARG;
  RowKeys rk{keys, n};
  return launch_find<0>(dt, dh, rk, out_flags, counters, (cudaStream_t)stream);
}

int dok_map_count_new(const dok_table *t, const dok_hash_params *hp, const void *keys, int64_t n,
                      int64_t *scratch_tags, int64_t scratch_slots, int64_t *counters, void *stream) {
  DevHash dh;
  DevTable dt;
  if (!prepare(t, hp, &dt, &dh) || n < 0 || n > DOK_MAX_BATCH) return DOK_BAD_ARG;
  if (n == 0) return DOK_OK;
  if (!keys || !scratch_tags || !counters || scratch_slots < 2 * n) return DOK_BAD_ARG;
  const ll_t blocks = (scratch_slots + 255) / 256;
  k_fill_i64<<<(unsigned)(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, (cudaStream_t)stream>>>(
      (ll_t *)scratch_tags, scratch_slots, DOK_EMPTY);
  int rc = dok_check_launch();
  if (rc != DOK_OK) return rc;
  RowKeys rk{keys, n};
  rc = DOK_OK;
  DOK_DISPATCH_SB(dt, DOK_FOR_WINDOWS(dt, rc, (k_count_new<SB><<<grid_for(n), DOK_TPB, 0, (cudaStream_t)stream>>>(
                                                  wt, dh, rk, (ll_t *)scratch_tags, scratch_slots, (ll_t *)counters))));
  return rc;
}

/* ---- sliced batches: rows whose count only the device knows (the inbox of a sharded table) ---------------------- */

static bool sliced_keys(const void *keys, int64_t n_slices, int64_t slice_rows, const int64_t *slice_counts,
                        const int64_t *abort_flag, RowKeys *out) {
  if (!keys || !slice_counts || n_slices < 1 || n_slices > 65535 || slice_rows < 1) return false;
  if (slice_rows > DOK_MAX_BATCH / n_slices) return false;
  out->keys = keys;
  out->n = n_slices * slice_rows;
  out->slice_rows = slice_rows;
  out->slice_counts = (const ll_t *)slice_counts;
  out->abort = (const ll_t *)abort_flag;
  return true;
}

int dok_map_get_sliced(const dok_table *t, const dok_hash_params *hp, const void *keys, int64_t n_slices,
                       int64_t slice_rows, const int64_t *slice_counts, const int64_t *abort_flag, void *out_values,
                       uint8_t *out_found, const void *fallback, int64_t *counters, void *stream) {
  DevHash dh;
  DevTable dt;
  RowKeys rk;
  if (!prepare(t, hp, &dt, &dh) || !sliced_keys(keys, n_slices, slice_rows, slice_counts, abort_flag, &rk) || !out_values)
    return DOK_BAD_ARG;
  return launch_get(dt, dh, rk, out_values, out_found, fallback, counters, 0, (cudaStream_t)stream);
}

int dok_map_set_sliced(const dok_table *t, const dok_hash_params *hp, const void *keys, const void *values,
                       int64_t n_slices, int64_t slice_rows, const int64_t *slice_counts, const int64_t *abort_flag,
                       int64_t *slot_scratch, int64_t epoch, int assume_unique, int64_t *counters, void *stream) {
  DevHash dh;
  DevTable dt;
  RowKeys rk;
  if (!prepare(t, hp, &dt, &dh) || !sliced_keys(keys, n_slices, slice_rows, slice_counts, abort_flag, &rk) || !values)
    return DOK_BAD_ARG;
  if (assume_unique) return launch_set_unique(dt, dh, rk, (const char *)values, nullptr, counters, (cudaStream_t)stream);
  if (!slot_scratch || !dok_has_stamps(dt) || epoch < 1 || epoch > DOK_MAX_EPOCH) return DOK_BAD_ARG;
  return launch_set(dt, dh, rk, (const char *)values, slot_scratch, epoch, nullptr, counters, (cudaStream_t)stream);
}

int dok_map_remove_sliced(const dok_table *t, const dok_hash_params *hp, const void *keys, int64_t n_slices,
                          int64_t slice_rows, const int64_t *slice_counts, const int64_t *abort_flag,
                          uint8_t *out_removed, int64_t *counters, void *stream) {
  DevHash dh;
  DevTable dt;
  RowKeys rk;
  if (!prepare(t, hp, &dt, &dh) || !sliced_keys(keys, n_slices, slice_rows, slice_counts, abort_flag, &rk)) return DOK_BAD_ARG;
  return launch_find<1>(dt, dh, rk, out_removed, counters, (cudaStream_t)stream);
}

/* ---- passes over tables beyond the TLB's reach ----------------------------------------------------------------- */

int dok_set_window_bytes(int64_t single_pass_limit, int64_t window_bytes) {
  if (single_pass_limit < 0 || window_bytes < 128) return DOK_BAD_ARG;
  dok_window_cfg().single_pass_limit = single_pass_limit;
  dok_window_cfg().window_bytes = window_bytes;
  return DOK_OK;
}

int dok_table_passes(const dok_table *t) {
  DevTable dt;
  if (!dok_make_table(t, &dt)) return -1;
  return dok_window_passes(dt);
}

int64_t dok_compact_tiles(int64_t n_buckets) { return (n_buckets + DOK_COMPACT_TILE - 1) / DOK_COMPACT_TILE; }

int dok_map_compact_count(const dok_table *t, int64_t *tile_offsets, void *stream) {
  DevTable dt;
  if (!dok_make_table(t, &dt) || !tile_offsets) return DOK_BAD_ARG;
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
  if (!prepare(t, hp, &dt, &dh) || !tile_offsets) return DOK_BAD_ARG;
  const ll_t tiles = dok_compact_tiles(dt.nb);
  k_compact_scatter<<<(unsigned)tiles, DOK_TPB, 0, (cudaStream_t)stream>>>(
      dt, dh, (const ll_t *)tile_offsets, tiles, (char *)keys_out, keys_transposed, (char *)values_out, (ll_t *)uuid_out);
  return dok_check_launch();
}

int dok_map_reinsert(const dok_table *src, const dok_table *dst, const dok_hash_params *dst_hp, int64_t *counters,
                     void *stream) {
  DevHash dh;
  DevTable st_, dt;
  if (!prepare(dst, dst_hp, &dt, &dh) || !dok_make_table(src, &st_)) return DOK_BAD_ARG;
  if (st_.kb != dt.kb || st_.vb != dt.vb) return DOK_BAD_ARG;
  ll_t blocks = (st_.nb + DOK_TPB - 1) / DOK_TPB;
  if (blocks > 148 * 8) blocks = 148 * 8;            // 8 resident blocks of 256 threads per SM, grid-stride over the slots
  if (blocks < 1) blocks = 1;
  int rc = DOK_OK;
  DOK_DISPATCH_SB(dt, DOK_FOR_WINDOWS(dt, rc, (k_reinsert<SB><<<(unsigned)blocks, DOK_TPB, 0, (cudaStream_t)stream>>>(
                                                  st_, wt, dh, (ll_t *)counters))));
  return rc;
}

}  // extern "C"
