// TEST INFRASTRUCTURE ONLY. Thin extern "C" doors onto the reference's own attention launchers,
// compiled from the reference tree where it lies (the include path is given by oracle/Makefile;
// no reference source is copied into this repository). Output goes to oracle/_ref/.
#include "attn_cute.cu"  // engine/src/attn_cute.cu of the FlashQwen tree

extern "C" {

// engine/src/attn_cute.h:14-20
void ref_attn_decode(const void* q, int q_stride, const void* cache_kv, void* out, int n_heads,
                     int n_kv, int head_dim, const int* pos, const int* qstart,
                     const int* decode_rids, int n_decode, const int* bt, int max_blocks,
                     int block_size, float scale, float* pm, float* pl, float* pa, void* stream) {
  fq::LaunchAttnDecodeCute(static_cast<const __nv_bfloat16*>(q), q_stride,
                           static_cast<const __nv_bfloat16*>(cache_kv),
                           static_cast<__nv_bfloat16*>(out), n_heads, n_kv, head_dim, pos, qstart,
                           decode_rids, n_decode, bt, max_blocks, block_size, scale, pm, pl, pa,
                           static_cast<cudaStream_t>(stream));
}

// engine/src/attn_cute.h:7-12
void ref_attn_prefill(const void* q, int q_stride, const void* cache_kv, void* out, int n_heads,
                      int n_kv, int head_dim, const int* pos, const int* qstart, const int* qlen,
                      const int* rids, int R, int max_qlen, const int* bt, int max_blocks,
                      int block_size, float scale, void* stream) {
  fq::LaunchAttnPrefillCute(static_cast<const __nv_bfloat16*>(q), q_stride,
                            static_cast<const __nv_bfloat16*>(cache_kv),
                            static_cast<__nv_bfloat16*>(out), n_heads, n_kv, head_dim, pos, qstart,
                            qlen, rids, R, max_qlen, bt, max_blocks, block_size, scale,
                            static_cast<cudaStream_t>(stream));
}

// engine/src/kernels.cuh:33-37
int ref_decode_max_ksplit() { return fq::kMaxKsplit; }
int ref_decode_max_heads() { return fq::kDecodeMaxHeads; }

}  // extern "C"
