// TEST INFRASTRUCTURE ONLY. extern "C" doors onto the reference's KV-append kernel and its
// head-norm + RoPE kernel, compiled from the reference tree where it lies (include path from
// oracle/Makefile; nothing is copied). Output goes to oracle/_ref/.
//
// KvStore's constructor sizes the pool from cudaMemGetInfo (engine/src/kv_store.cu:10-46), which
// is not wanted on a shared GPU, so the append kernel is launched here on a caller-owned cache
// with the launch shape of KvStore::StoreKV (engine/src/kv_store.cu:66-75).
#include "kv_store.cu"  // engine/src/kv_store.cu of the FlashQwen tree
#include "kernels.cu"   // engine/src/kernels.cu (HeadNormRope)

extern "C" {

void ref_store_kv(void* cache, int n_heads, int n_kv, int head_dim, const void* qkv, const int* bt,
                  int bt_stride, const int* bt_row, const int* pos, int M, void* stream) {
  int q_dim = n_heads * head_dim, kv_dim = n_kv * head_dim;
  int n = M * kv_dim, threads = 256;
  if (n <= 0) return;
  fq::StoreKvKernel<<<(n + threads - 1) / threads, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const fq::bf16*>(qkv), q_dim + 2 * kv_dim, q_dim, q_dim + kv_dim,
      static_cast<fq::bf16*>(cache), bt, bt_stride, kv_dim, bt_row, pos, M);
}

// engine/src/kernels.cu:133-139
void ref_head_norm_rope(void* buf, const float* wq, const float* wk, const float* cos_tab,
                        const float* sin_tab, const int* pos, int M, int n_q, int n_kv,
                        int head_dim, int stride, float eps, void* stream) {
  if (M <= 0) return;
  fq::LaunchHeadNormRope(static_cast<fq::bf16*>(buf), wq, wk, cos_tab, sin_tab, pos, M, n_q, n_kv,
                         head_dim, stride, eps, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
