// The engine's two attention launcher symbols (engine/src/attn_cute.h:7-20), defined on top of the
// C ABI so that an engine linked against libfqb instead of its own attn_cute.cu needs no change at
// the call sites (engine/src/model_runtime.cu:271-283). Their signatures lack the pool's block
// count and the scratch size; fqb_engine_configure() holds both. The launchers return void: the
// first failure is kept for fqb_engine_status().
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>
#include <mutex>
#include <string>

#include "../../../include/fqb.h"
#include "../errors.h"

namespace {

std::atomic<int> g_num_blocks{0};
std::atomic<long long> g_partial_slots{0};
std::atomic<int> g_first_error{FQB_OK};
std::mutex g_message_lock;
std::string g_message;

void keep(int rc) {
  if (rc == FQB_OK) return;
  int expected = FQB_OK;
  if (g_first_error.compare_exchange_strong(expected, rc)) {
    std::lock_guard<std::mutex> hold(g_message_lock);
    g_message = fqb_last_error();
  }
}

bool configured(const char* who) {
  if (g_num_blocks.load() > 0) return true;
  keep(fqb::set_error(FQB_ERR_STATE, "%s: fqb_engine_configure() has not been called", who));
  return false;
}

}  // namespace

extern "C" {

int fqb_engine_configure(int num_blocks, int64_t partial_slots) {
  if (num_blocks <= 0 || partial_slots < 0)
    return fqb::set_error(FQB_ERR_INVALID, "fqb_engine_configure: num_blocks %d, partial_slots %lld", num_blocks,
                          static_cast<long long>(partial_slots));
  // The engine's scratch must at least serve one sequence on this GPU (a launch cuts the page list into
  // a number of pieces that follows the SM count); an engine started with very few slots would otherwise
  // learn of it only at its first decode step.
  long long least = -1;
  for (int n_kv = 1; n_kv <= 8; n_kv *= 2) {
    const long long need = fqb_attn_decode_slots_needed(1, n_kv);
    if (need < 0) break;  // no usable CUDA device in this process (yet): the launches will check
    if (least < 0 || need < least) least = need;
  }
  if (least >= 0 && partial_slots < least)
    return fqb::set_error(FQB_ERR_WORKSPACE,
                          "fqb_engine_configure: %lld partial slots cannot serve a single sequence on this GPU "
                          "(%lld needed); the engine's DecodePartialFloats(slots) gives slots*1024",
                          static_cast<long long>(partial_slots), least);
  g_num_blocks.store(num_blocks);
  g_partial_slots.store(partial_slots);
  g_first_error.store(FQB_OK);
  std::lock_guard<std::mutex> hold(g_message_lock);
  g_message.clear();
  return FQB_OK;
}

int fqb_engine_status(void) { return g_first_error.load(); }

const char* fqb_engine_error(void) {
  static thread_local std::string copy;
  std::lock_guard<std::mutex> hold(g_message_lock);
  copy = g_message;
  return copy.c_str();
}

}  // extern "C"

namespace fq {

void LaunchAttnPrefillCute(const __nv_bfloat16* q, int q_stride, const __nv_bfloat16* cache_kv,
                           __nv_bfloat16* out, int n_heads, int n_kv, int head_dim, const int* pos,
                           const int* qstart, const int* qlen, const int* rids, int R, int max_qlen,
                           const int* bt, int max_blocks, int block_size, float scale, cudaStream_t s) {
  if (!configured("LaunchAttnPrefillCute")) return;
  keep(fqb_attn_prefill(q, q_stride, cache_kv, g_num_blocks.load(), out, n_heads, n_kv, head_dim, pos, qstart,
                        qlen, rids, R, max_qlen, bt, max_blocks, block_size, scale, s));
}

void LaunchAttnDecodeCute(const __nv_bfloat16* q, int q_stride, const __nv_bfloat16* cache_kv,
                          __nv_bfloat16* out, int n_heads, int n_kv, int head_dim, const int* pos,
                          const int* qstart, const int* decode_rids, int n_decode, const int* bt,
                          int max_blocks, int block_size, float scale, float* pm, float* pl, float* pa,
                          cudaStream_t s) {
  if (!configured("LaunchAttnDecodeCute")) return;
  keep(fqb_attn_decode(q, q_stride, cache_kv, g_num_blocks.load(), out, n_heads, n_kv, head_dim, pos, qstart,
                       decode_rids, n_decode, bt, max_blocks, block_size, scale, pm, pl, pa,
                       g_partial_slots.load(), s));
}

}  // namespace fq
