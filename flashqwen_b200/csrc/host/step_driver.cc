// Step driver: the engine's scheduling loop and per-step runtime around the attention path, as host
// code over the C ABI. It stands where the FlashQwen engine has Scheduler (engine/src/scheduler.cc:59-154,
// engine/src/scheduler.h:19-118) and the attention-related half of ModelRuntime
// (engine/src/model_runtime.cu:47-108 PrepareInputs, :227-283 RunLayers / RunLayersBody,
// engine/src/model_runtime.h:160-201 GraphCache). The model itself is not here: two callbacks stand in
// for it -- one produces the step's fused qkv rows (embedding + QKV projection in the engine), one
// consumes the attention output and returns the sampled tokens (o_proj ... sampler in the engine).
//
// Differences from the reference, by design:
//   * the step's metadata (positions, request index, qstart, qlen, decode / prefill request lists, packed
//     block tables) lives in ONE pinned buffer and goes to the device with one copy instead of eight;
//   * a pure-decode step runs per layer {RMSNorm + RoPE, fused KV append + decode attention} and is
//     replayed from a cache of CUDA graphs keyed (rows, decode requests) as in the reference; a mixed
//     step runs {RMSNorm + RoPE + append, decode attention, prefill attention} eagerly;
//   * errors come back as status codes; nothing exits.
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <deque>
#include <memory>
#include <numeric>
#include <vector>

#include "../../../include/fqb.h"
#include "../errors.h"

namespace {

constexpr int kRowSlack = 16;  // engine/src/model_runtime.cu:45

#define DRV_CUDA(call)                                                                               \
  do {                                                                                               \
    cudaError_t e_ = (call);                                                                         \
    if (e_ != cudaSuccess) return fqb::set_error(FQB_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e_)); \
  } while (0)
#define DRV_TRY(call)          \
  do {                         \
    int rc_ = (call);          \
    if (rc_ != FQB_OK) return rc_; \
  } while (0)

// engine/src/scheduler.h:26-118 (class Request), without sinks and sampling parameters
struct Request {
  int id = 0;
  std::vector<int32_t> prompt, output, blocks;
  int max_new = 0, max_ctx = 0;
  int computed = 0, num_new = 0, cached_blocks = 0;
  uint64_t last_hash = 0;

  int NumTokens() const { return static_cast<int>(prompt.size() + output.size()); }
  int Remaining() const { return NumTokens() - computed; }
  int TokenAt(int i) const {
    const int p = static_cast<int>(prompt.size());
    return i < p ? prompt[i] : output[i - p];
  }
  bool IsFinished() const { return static_cast<int>(output.size()) >= max_new || NumTokens() >= max_ctx; }
  void ResetForRecompute() { computed = cached_blocks = 0, last_hash = 0; }
};

// engine/src/model_runtime.h:160-201: capture once, replay; most recently used first, 64 entries
struct GraphCache {
  struct Entry {
    int k0, k1;
    cudaGraphExec_t exec;
  };
  std::vector<Entry> entries;
  static constexpr size_t kMaxEntries = 64;
  ~GraphCache() {
    for (auto& e : entries) cudaGraphExecDestroy(e.exec);
  }
};

template <class T>
struct DevBuf {
  T* p = nullptr;
  ~DevBuf() {
    if (p) cudaFree(p);
  }
  int alloc(size_t n) { DRV_CUDA(cudaMalloc(reinterpret_cast<void**>(&p), n * sizeof(T))); return FQB_OK; }
};
template <class T>
struct PinBuf {
  T* p = nullptr;
  ~PinBuf() {
    if (p) cudaFreeHost(p);
  }
  int alloc(size_t n) { DRV_CUDA(cudaMallocHost(reinterpret_cast<void**>(&p), n * sizeof(T))); return FQB_OK; }
};

}  // namespace

struct fqb_driver {
  fqb_driver_config cfg{};
  fqb_rows_fn rows_fn = nullptr;
  fqb_sample_fn sample_fn = nullptr;
  void* user = nullptr;
  std::vector<void*> pools;  // caller-owned per-layer caches
  fqb_alloc* alloc = nullptr;
  cudaStream_t stream = nullptr;

  int max_rows = 0, max_blocks = 0, row_elems = 0, q_dim = 0, kv_dim = 0;
  // one metadata buffer: [pos | req | qstart | qlen | decode_rids | prefill_rids | bt], fixed offsets (ints)
  size_t o_pos = 0, o_req = 0, o_qstart = 0, o_qlen = 0, o_drids = 0, o_prids = 0, o_bt = 0, meta_ints = 0;
  PinBuf<int32_t> h_meta;
  DevBuf<int32_t> d_meta;
  PinBuf<uint16_t> h_rows, h_out;   // [n_layers][max_rows][row_elems], [n_layers][max_rows][q_dim]
  DevBuf<uint16_t> d_rows, d_out;
  DevBuf<float> d_cos, d_sin, d_wq, d_wk, d_pm, d_pl, d_pa;
  DevBuf<int32_t> d_plan;
  int64_t partial_slots = 0;
  GraphCache graphs;

  std::deque<std::unique_ptr<Request>> waiting;
  std::vector<std::unique_ptr<Request>> running;
  int next_id = 0, step_no = 0;
  fqb_driver_stats stats{};

  // the step being built
  std::vector<Request*> batch;
  std::vector<int32_t> tokens, logits_rows, sampled;
  int n_rows = 0, n_req = 0, n_decode = 0, n_prefill = 0, prefill_max_qlen = 1;

  ~fqb_driver() {
    if (alloc) fqb_alloc_destroy(alloc);
    if (stream) cudaStreamDestroy(stream);
  }

  int32_t* hm(size_t off) { return h_meta.p + off; }
  int32_t* dm(size_t off) { return d_meta.p + off; }

  // ---- engine/src/scheduler.cc:59-110 ------------------------------------------------------------
  void Release(Request* r) {
    int len = static_cast<int>(r->blocks.size());
    if (len) fqb_alloc_free_table(alloc, r->blocks.data(), &len);
    r->blocks.clear();
  }
  void Retire(Request* r) {
    Release(r);
    for (auto it = running.begin(); it != running.end(); ++it)
      if (it->get() == r) {
        running.erase(it);
        return;
      }
  }
  // Grow: blocks for `upto` tokens; when the pool is dry the youngest other running request is
  // preempted (blocks freed, recomputed on resume) until it fits.
  enum GrowResult { kGrown, kGrownAfterPreempting, kRetired };
  GrowResult Grow(Request* r, int upto) {
    bool preempted = false;
    for (;;) {
      const int need = fqb_alloc_blocks_for(upto);
      int len = static_cast<int>(r->blocks.size());
      r->blocks.resize(std::max(need, len));
      const int rc = fqb_alloc_grow(alloc, r->blocks.data(), &len, static_cast<int>(r->blocks.size()), upto);
      r->blocks.resize(len);
      if (rc == FQB_OK) return preempted ? kGrownAfterPreempting : kGrown;
      int k = static_cast<int>(running.size()) - 1;
      while (k >= 0 && running[k].get() == r) --k;
      if (k < 0) {  // alone and still too large for the pool: over capacity
        ++stats.over_capacity;
        Retire(r);
        return kRetired;
      }
      Release(running[k].get());
      running[k]->ResetForRecompute();
      waiting.push_front(std::move(running[k]));
      running.erase(running.begin() + k);
      ++stats.preemptions;
      preempted = true;
    }
  }
  void AcquirePrefix(Request* r) {
    if (!cfg.use_prefix_cache) return;
    std::vector<int32_t> all(r->NumTokens());
    for (int i = 0; i < r->NumTokens(); ++i) all[i] = r->TokenAt(i);
    const int cap = std::max(1, (r->NumTokens() - 1) / FQB_BLOCK_TOKENS);
    r->blocks.resize(cap);
    uint64_t last = 0;
    const int nb = fqb_acquire_prefix(alloc, all.data(), r->NumTokens(), r->blocks.data(), cap, &last);
    r->blocks.resize(std::max(nb, 0));
    if (nb > 0) {  // Request::AdoptPrefix
      r->computed = nb * FQB_BLOCK_TOKENS;
      r->cached_blocks = nb;
      r->last_hash = last;
      stats.prefix_hit_blocks += nb;
    }
  }
  void CacheBlocks(Request* r) {
    std::vector<int32_t> all(r->NumTokens());
    for (int i = 0; i < r->NumTokens(); ++i) all[i] = r->TokenAt(i);
    uint64_t last = r->last_hash;
    const int n = fqb_cache_blocks(alloc, all.data(), r->computed, r->blocks.data(), r->cached_blocks, &last);
    if (n >= 0) {
      r->cached_blocks = n;
      r->last_hash = last;
    }
  }
  void Refill() {
    while (static_cast<int>(running.size()) < cfg.n_slots && !waiting.empty()) {
      if (waiting.front()->blocks.empty()) AcquirePrefix(waiting.front().get());
      running.push_back(std::move(waiting.front()));
      waiting.pop_front();
    }
  }
  // engine/src/scheduler.cc:112-143 BuildBatch + Request::EmitChunk: shortest remaining first (decodes
  // outrank prefill chunks), one merged batch under the token budget, restart after a preemption.
  bool BuildBatch() {
    std::vector<int> order;
    for (bool restart = true; restart;) {
      restart = false;
      batch.clear();
      tokens.clear();
      logits_rows.clear();
      n_rows = n_req = 0;
      order.resize(running.size());
      std::iota(order.begin(), order.end(), 0);
      std::stable_sort(order.begin(), order.end(),
                       [&](int a, int b) { return running[a]->Remaining() < running[b]->Remaining(); });
      int budget = cfg.token_budget;
      for (int idx : order) {
        if (budget <= 0) break;
        Request* r = running[idx].get();
        const int remaining = r->Remaining();
        if (remaining <= 0) continue;
        int n = std::min(remaining, budget);
        if (remaining > 1) n = std::min(n, cfg.prefill_chunk);
        // The build starts over whenever the running set changed: after the request itself was retired
        // (as the reference does) and also after a preemption -- the reference goes on with indices that
        // the erase has shifted; starting over gives the same batch wherever that is well defined, because
        // the blocks already obtained stay with their requests.
        if (Grow(r, r->computed + n) != kGrown) {
          restart = true;
          break;
        }
        for (int k = 0; k < n; ++k) {
          hm(o_pos)[n_rows] = r->computed + k;
          hm(o_req)[n_rows] = n_req;
          tokens.push_back(r->TokenAt(r->computed + k));
          ++n_rows;
        }
        if (r->computed + n == r->NumTokens()) logits_rows.push_back(n_rows - 1);
        r->num_new = n;
        batch.push_back(r);
        ++n_req;
        budget -= n;
      }
    }
    return !batch.empty();
  }

  int RunLayers();
  int LayerBody(bool pure_decode);
  int Step();
};

// ---- engine/src/model_runtime.cu:235-283: the attention calls of every layer ------------------------
int fqb_driver::LayerBody(bool pure_decode) {
  const fqb_driver_config& c = cfg;
  const int k_off = q_dim, v_off = q_dim + kv_dim;
  if (pure_decode)
    DRV_TRY(fqb_attn_decode_plan(dm(o_pos), dm(o_qstart), dm(o_drids), n_decode, max_blocks, d_plan.p, stream));
  for (int l = 0; l < c.n_layers; ++l) {
    uint16_t* rows = d_rows.p + static_cast<size_t>(l) * max_rows * row_elems;
    uint16_t* out = d_out.p + static_cast<size_t>(l) * max_rows * q_dim;
    if (pure_decode) {
      // LaunchHeadNormRope, then StoreKV + LaunchAttnDecodeCute as one kernel; the kernel in front of the
      // fused call writes only the rows, never the cached history
      DRV_TRY(fqb_norm_rope_append(nullptr, c.num_blocks, c.kv_heads, c.q_heads, rows, row_elems, 0, k_off, v_off,
                                   d_wq.p, d_wk.p, d_cos.p, d_sin.p, c.rms_eps, nullptr, max_blocks, nullptr,
                                   dm(o_pos), n_rows, stream));
      DRV_TRY(fqb_append_attn_decode(pools[l], c.num_blocks, c.kv_heads, rows, row_elems, 0, k_off, v_off, out,
                                     FQB_HEAD_DIM, nullptr, nullptr, nullptr, d_plan.p, n_decode, dm(o_bt), max_blocks,
                                     FQB_BLOCK_TOKENS, c.scale, d_pm.p, d_pl.p, d_pa.p, partial_slots,
                                     FQB_DECODE_HISTORY_STABLE, stream));
    } else {
      DRV_TRY(fqb_norm_rope_append(pools[l], c.num_blocks, c.kv_heads, c.q_heads, rows, row_elems, 0, k_off, v_off,
                                   d_wq.p, d_wk.p, d_cos.p, d_sin.p, c.rms_eps, dm(o_bt), max_blocks, dm(o_req),
                                   dm(o_pos), n_rows, stream));
      DRV_TRY(fqb_attn_decode(rows, row_elems, pools[l], c.num_blocks, out, c.q_heads, c.kv_heads, FQB_HEAD_DIM,
                              dm(o_pos), dm(o_qstart), dm(o_drids), n_decode, dm(o_bt), max_blocks, FQB_BLOCK_TOKENS,
                              c.scale, d_pm.p, d_pl.p, d_pa.p, partial_slots, stream));
      DRV_TRY(fqb_attn_prefill(rows, row_elems, pools[l], c.num_blocks, out, c.q_heads, c.kv_heads, FQB_HEAD_DIM,
                               dm(o_pos), dm(o_qstart), dm(o_qlen), dm(o_prids), n_prefill, prefill_max_qlen,
                               dm(o_bt), max_blocks, FQB_BLOCK_TOKENS, c.scale, stream));
    }
  }
  return FQB_OK;
}

// engine/src/model_runtime.cu:227-233 + GraphCache::Run: pure-decode steps replay a captured graph
int fqb_driver::RunLayers() {
  const bool pure_decode = n_prefill == 0 && n_decode > 0;
  if (!pure_decode || !cfg.use_graphs) return LayerBody(pure_decode);
  auto& es = graphs.entries;
  for (auto it = es.begin(); it != es.end(); ++it)
    if (it->k0 == n_rows && it->k1 == n_decode) {
      GraphCache::Entry hit = *it;
      es.erase(it);
      es.insert(es.begin(), hit);
      DRV_CUDA(cudaGraphLaunch(hit.exec, stream));
      ++stats.graph_replays;
      return FQB_OK;
    }
  DRV_CUDA(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
  const int rc = LayerBody(true);
  cudaGraph_t g = nullptr;
  const cudaError_t ce = cudaStreamEndCapture(stream, &g);
  if (rc != FQB_OK) {
    if (g) cudaGraphDestroy(g);
    return rc;
  }
  if (ce != cudaSuccess) return fqb::set_error(FQB_ERR_CUDA, "cudaStreamEndCapture: %s", cudaGetErrorString(ce));
  cudaGraphExec_t exec = nullptr;
  const cudaError_t ie = cudaGraphInstantiate(&exec, g, 0);
  cudaGraphDestroy(g);
  if (ie != cudaSuccess) return fqb::set_error(FQB_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(ie));
  while (es.size() >= GraphCache::kMaxEntries) {
    cudaGraphExecDestroy(es.back().exec);
    es.pop_back();
  }
  es.insert(es.begin(), GraphCache::Entry{n_rows, n_decode, exec});
  ++stats.graph_captures;
  DRV_CUDA(cudaGraphLaunch(exec, stream));
  return FQB_OK;
}

// engine/src/scheduler.cc:145-154 Step + engine/src/model_runtime.cu:295-310 Forward
int fqb_driver::Step() {
  Refill();
  if (!BuildBatch()) return 0;
  // ---- PrepareInputs: the derived metadata, written straight into the pinned buffer ----
  std::vector<const int32_t*> tabs(n_req);
  std::vector<int32_t> lens(n_req);
  for (int i = 0; i < n_req; ++i) {
    tabs[i] = batch[i]->blocks.data();
    lens[i] = static_cast<int32_t>(batch[i]->blocks.size());
  }
  int32_t counts[3] = {0, 0, 1};
  DRV_TRY(fqb_step_pack(hm(o_req), n_rows, n_req, tabs.data(), lens.data(), max_blocks, hm(o_bt), hm(o_qstart),
                        hm(o_qlen), hm(o_drids), hm(o_prids), counts));
  n_decode = counts[0];
  n_prefill = counts[1];
  prefill_max_qlen = counts[2];
  // the model stand-in fills the step's rows for every layer
  rows_fn(user, step_no, n_rows, tokens.data(), hm(o_pos), hm(o_req), h_rows.p, max_rows);
  const size_t used_ints = o_bt + static_cast<size_t>(n_req) * max_blocks;
  DRV_CUDA(cudaMemcpyAsync(d_meta.p, h_meta.p, used_ints * sizeof(int32_t), cudaMemcpyHostToDevice, stream));
  DRV_CUDA(cudaMemcpy2DAsync(d_rows.p, static_cast<size_t>(max_rows) * row_elems * 2, h_rows.p,
                             static_cast<size_t>(max_rows) * row_elems * 2, static_cast<size_t>(n_rows) * row_elems * 2,
                             cfg.n_layers, cudaMemcpyHostToDevice, stream));
  const uint64_t replays_before = stats.graph_replays;
  DRV_TRY(RunLayers());
  DRV_CUDA(cudaMemcpy2DAsync(h_out.p, static_cast<size_t>(max_rows) * q_dim * 2, d_out.p,
                             static_cast<size_t>(max_rows) * q_dim * 2, static_cast<size_t>(n_rows) * q_dim * 2,
                             cfg.n_layers, cudaMemcpyDeviceToHost, stream));
  DRV_CUDA(cudaStreamSynchronize(stream));
  DRV_TRY(fqb_device_status(nullptr));
  // ---- the rest of the model + sampler ----
  fqb_step_view v{};
  v.step = step_no;
  v.n_rows = n_rows;
  v.n_req = n_req;
  v.n_decode = n_decode;
  v.n_prefill = n_prefill;
  v.prefill_max_qlen = prefill_max_qlen;
  v.bt_stride = max_blocks;
  v.row_capacity = max_rows;
  v.from_graph = stats.graph_replays != replays_before;
  v.tokens = tokens.data();
  v.pos = hm(o_pos);
  v.req = hm(o_req);
  v.qstart = hm(o_qstart);
  v.qlen = hm(o_qlen);
  v.decode_rids = hm(o_drids);
  v.prefill_rids = hm(o_prids);
  v.bt = hm(o_bt);
  v.n_logits = static_cast<int32_t>(logits_rows.size());
  v.logits_rows = logits_rows.data();
  std::vector<int32_t> ids(n_req);
  for (int i = 0; i < n_req; ++i) ids[i] = batch[i]->id;
  v.request_ids = ids.data();
  sampled.assign(logits_rows.size(), 0);
  sample_fn(user, &v, h_out.p, sampled.data());
  // ---- CurrentBatch::Apply, CacheBlocks, Retire (engine/src/scheduler.h:138-145, scheduler.cc:150-153) ----
  for (Request* r : batch) r->computed += r->num_new;
  size_t s = 0;
  std::vector<Request*> finished;
  for (Request* r : batch)
    if (r->Remaining() == 0) {
      r->output.push_back(sampled[s++]);
      if (r->IsFinished()) finished.push_back(r);
    }
  if (cfg.use_prefix_cache)
    for (Request* r : batch) CacheBlocks(r);
  for (Request* r : finished) {
    Retire(r);
    ++stats.finished;
  }
  ++stats.steps;
  stats.decode_rows += n_decode;
  stats.prefill_rows += n_rows - n_decode;
  ++step_no;
  return 1;
}

extern "C" {

void fqb_rope_tables(float* cos_tab, float* sin_tab, int n_pos, int head_dim, float theta) {
  const int half = head_dim / 2;
  for (int p = 0; p < n_pos; ++p)
    for (int i = 0; i < half; ++i) {
      const float inv = std::pow(theta, -2.0f * i / head_dim);
      const float ang = p * inv;
      cos_tab[static_cast<size_t>(p) * half + i] = std::cos(ang);
      sin_tab[static_cast<size_t>(p) * half + i] = std::sin(ang);
    }
}

int fqb_driver_create(const fqb_driver_config* cfg, void* const* layer_caches, const float* wq, const float* wk,
                      fqb_rows_fn rows_fn, fqb_sample_fn sample_fn, void* user, fqb_driver** out) {
  if (!cfg || !layer_caches || !wq || !wk || !rows_fn || !sample_fn || !out)
    return fqb::set_error(FQB_ERR_INVALID, "driver_create: null pointer");
  const fqb_driver_config& c = *cfg;
  if (c.n_layers <= 0 || c.num_blocks <= 0 || c.kv_heads <= 0 || c.q_heads != c.kv_heads * FQB_GQA_GROUP ||
      c.n_slots <= 0 || c.token_budget <= 0 || c.prefill_chunk <= 0 || c.max_ctx < FQB_BLOCK_TOKENS)
    return fqb::set_error(FQB_ERR_INVALID, "driver_create: bad configuration");
  if (c.num_blocks < fqb_alloc_blocks_for(c.max_ctx))  // engine/src/kv_store.cu:30-38
    return fqb::set_error(FQB_ERR_NOMEM, "driver_create: a pool of %d blocks cannot hold one sequence of %d tokens",
                          c.num_blocks, c.max_ctx);
  std::unique_ptr<fqb_driver> d(new fqb_driver);
  d->cfg = c;
  d->rows_fn = rows_fn;
  d->sample_fn = sample_fn;
  d->user = user;
  d->pools.assign(layer_caches, layer_caches + c.n_layers);
  d->alloc = fqb_alloc_create(c.num_blocks);
  if (!d->alloc) return FQB_ERR_INVALID;
  d->max_rows = std::max(1, c.token_budget) + kRowSlack;
  d->max_blocks = fqb_alloc_blocks_for(c.max_ctx);
  d->q_dim = c.q_heads * FQB_HEAD_DIM;
  d->kv_dim = c.kv_heads * FQB_HEAD_DIM;
  d->row_elems = d->q_dim + 2 * d->kv_dim;
  const size_t slots = static_cast<size_t>(c.n_slots), rows = static_cast<size_t>(d->max_rows);
  // every section starts on a 16-byte boundary
  auto up4 = [](size_t x) { return (x + 3) & ~static_cast<size_t>(3); };
  d->o_pos = 0;
  d->o_req = up4(d->o_pos + rows);
  d->o_qstart = up4(d->o_req + rows);
  d->o_qlen = up4(d->o_qstart + slots);
  d->o_drids = up4(d->o_qlen + slots);
  d->o_prids = up4(d->o_drids + slots);
  d->o_bt = up4(d->o_prids + slots);
  d->meta_ints = d->o_bt + slots * d->max_blocks;
  DRV_CUDA(cudaStreamCreate(&d->stream));
  DRV_TRY(d->h_meta.alloc(d->meta_ints));
  DRV_TRY(d->d_meta.alloc(d->meta_ints));
  std::memset(d->h_meta.p, 0, d->meta_ints * sizeof(int32_t));
  DRV_CUDA(cudaMemset(d->d_meta.p, 0, d->meta_ints * sizeof(int32_t)));
  const size_t nl = static_cast<size_t>(c.n_layers);
  DRV_TRY(d->h_rows.alloc(nl * rows * d->row_elems));
  DRV_TRY(d->d_rows.alloc(nl * rows * d->row_elems));
  DRV_TRY(d->h_out.alloc(nl * rows * d->q_dim));
  DRV_TRY(d->d_out.alloc(nl * rows * d->q_dim));
  DRV_CUDA(cudaMemset(d->d_out.p, 0, nl * rows * d->q_dim * 2));
  const size_t tab = static_cast<size_t>(c.max_ctx) * (FQB_HEAD_DIM / 2);
  std::vector<float> hc(tab), hs(tab);
  fqb_rope_tables(hc.data(), hs.data(), c.max_ctx, FQB_HEAD_DIM, c.rope_theta);
  DRV_TRY(d->d_cos.alloc(tab));
  DRV_TRY(d->d_sin.alloc(tab));
  DRV_TRY(d->d_wq.alloc(FQB_HEAD_DIM));
  DRV_TRY(d->d_wk.alloc(FQB_HEAD_DIM));
  DRV_CUDA(cudaMemcpy(d->d_cos.p, hc.data(), tab * 4, cudaMemcpyHostToDevice));
  DRV_CUDA(cudaMemcpy(d->d_sin.p, hs.data(), tab * 4, cudaMemcpyHostToDevice));
  DRV_CUDA(cudaMemcpy(d->d_wq.p, wq, FQB_HEAD_DIM * 4, cudaMemcpyHostToDevice));
  DRV_CUDA(cudaMemcpy(d->d_wk.p, wk, FQB_HEAD_DIM * 4, cudaMemcpyHostToDevice));
  d->partial_slots = fqb_attn_decode_partial_slots(c.n_slots, c.q_heads, d->max_blocks);
  DRV_TRY(d->d_pm.alloc(d->partial_slots));
  DRV_TRY(d->d_pl.alloc(d->partial_slots));
  DRV_TRY(d->d_pa.alloc(static_cast<size_t>(d->partial_slots) * FQB_HEAD_DIM));
  DRV_TRY(d->d_plan.alloc(4 * slots + 4));
  *out = d.release();
  return FQB_OK;
}

void fqb_driver_destroy(fqb_driver* d) { delete d; }

int fqb_driver_submit(fqb_driver* d, const int32_t* prompt, int n_prompt, int max_new) {
  if (!d || !prompt || n_prompt <= 0 || max_new <= 0)
    return fqb::set_error(FQB_ERR_INVALID, "driver_submit: bad arguments");
  if (n_prompt >= d->cfg.max_ctx)
    return fqb::set_error(FQB_ERR_SHAPE, "driver_submit: a prompt of %d tokens does not fit max_ctx %d", n_prompt,
                          d->cfg.max_ctx);
  std::unique_ptr<Request> r(new Request);
  r->id = d->next_id++;
  r->prompt.assign(prompt, prompt + n_prompt);
  r->max_new = max_new;
  r->max_ctx = d->cfg.max_ctx;
  const int id = r->id;
  d->waiting.push_back(std::move(r));
  return id;
}

int fqb_driver_busy(const fqb_driver* d) { return d && (!d->waiting.empty() || !d->running.empty()) ? 1 : 0; }

int fqb_driver_step(fqb_driver* d) {
  if (!d) return fqb::set_error(FQB_ERR_INVALID, "driver_step: null handle");
  return d->Step();
}

int fqb_driver_get_stats(const fqb_driver* d, fqb_driver_stats* out) {
  if (!d || !out) return fqb::set_error(FQB_ERR_INVALID, "driver_get_stats: null pointer");
  *out = d->stats;
  out->free_blocks = fqb_alloc_num_free(d->alloc);
  out->running = static_cast<int32_t>(d->running.size());
  out->waiting = static_cast<int32_t>(d->waiting.size());
  return FQB_OK;
}

}  // extern "C"
