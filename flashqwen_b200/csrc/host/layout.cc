// Layout arithmetic of the paged KV cache (no CUDA).
#include "../../../include/fqb.h"
#include "../errors.h"

extern "C" {

int fqb_kv_layout_query(int kv_heads_local, fqb_kv_layout* out) {
  if (!out || kv_heads_local <= 0) return fqb::set_error(FQB_ERR_INVALID, "kv_layout_query: bad argument");
  out->kv_heads_local = kv_heads_local;
  out->head_dim = FQB_HEAD_DIM;
  out->block_tokens = FQB_BLOCK_TOKENS;
  out->row_elems = static_cast<int64_t>(kv_heads_local) * FQB_HEAD_DIM;
  out->plane_elems = out->row_elems * FQB_BLOCK_TOKENS;
  out->block_elems = out->plane_elems * FQB_PLANES;
  out->block_bytes = out->block_elems * 2;
  return FQB_OK;
}

int64_t fqb_kv_pool_bytes(int num_blocks, int kv_heads_local) {
  if (num_blocks < 0 || kv_heads_local <= 0) return 0;
  return static_cast<int64_t>(num_blocks) * FQB_PLANES * FQB_BLOCK_TOKENS * kv_heads_local * FQB_HEAD_DIM * 2;
}

}  // extern "C"
