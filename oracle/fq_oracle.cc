// TEST INFRASTRUCTURE ONLY -- never linked into, loaded by, or called from the product library.
//
// Scalar C++ host oracle for the paged-KV attention path of the FlashQwen engine. Each function
// restates, on the CPU and in the plainest possible form, what one reference routine computes;
// the reference location it follows (path:line inside the FlashQwen tree) is given beside it.
// Integer / byte work (indexing, append, block copies, allocator, hashes, step metadata) is meant
// to be compared bit-for-bit. Attention is computed as an exact fp32/double softmax with a single
// bf16 rounding at the output; it does not imitate the reference's split order, __expf or the
// P->bf16 rounding of the prefill kernel (an optional switch does the latter for triage).
//
// Parity status: pinned. The attention, append and norm+RoPE functions are checked against
// outputs of the reference's own CUDA kernels (rebuilt for sm_100a and run on a B200; fixtures
// under tests/golden/), the allocator against a trace produced by the reference's
// block_allocator.h compiled on the host (same folder).
//
// Build: see oracle/Makefile (g++ -O2 -ffp-contract=off, no CUDA needed).

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <unordered_map>
#include <vector>

namespace {

constexpr int kTok = 16;     // tokens per page            engine/src/kv_layout.h:5
constexpr int kPlanes = 2;   // K plane then V plane       engine/src/kv_layout.h:7
constexpr int kHd = 128;     // head_dim                   engine/src/model_spec.h:15

inline float bf2f(uint16_t b) {
  uint32_t u = static_cast<uint32_t>(b) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

// round-to-nearest-even, NaN kept quiet (what __float2bfloat16 / cutlass::bfloat16_t do)
inline uint16_t f2bf(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}

template <class F>
void parallel_for(int n, int nthreads, F&& body) {
  if (nthreads <= 1 || n <= 1) {
    for (int i = 0; i < n; ++i) body(i);
    return;
  }
  std::atomic<int> next{0};
  std::vector<std::thread> pool;
  int nt = std::min(nthreads, n);
  for (int t = 0; t < nt; ++t)
    pool.emplace_back([&] {
      for (int i = next.fetch_add(1); i < n; i = next.fetch_add(1)) body(i);
    });
  for (auto& th : pool) th.join();
}

}  // namespace

extern "C" {

// ---------------------------------------------------------------------------------------------
// KV append: engine/src/kv_store.cu:48-64 (StoreKvKernel) and :66-75 (offsets k_off/v_off).
// cache is [num_blocks][2][16][kv_dim] bf16. For each row m the K and V slices of the fused qkv
// row go to block bt[bt_row[m]][pos[m]/16], slot pos[m]%16.
// ---------------------------------------------------------------------------------------------
void orc_kv_append(uint16_t* cache, int kv_dim, const uint16_t* qkv, int src_stride, int k_off,
                   int v_off, const int32_t* bt, int bt_stride, const int32_t* bt_row,
                   const int32_t* pos, int M) {
  const int64_t plane = static_cast<int64_t>(kTok) * kv_dim;
  for (int m = 0; m < M; ++m) {
    const int32_t* row_bt = bt + static_cast<int64_t>(bt_row[m]) * bt_stride;
    int p = pos[m];
    int64_t dst = static_cast<int64_t>(row_bt[p / kTok]) * kPlanes * plane +
                  static_cast<int64_t>(p % kTok) * kv_dim;
    const uint16_t* src = qkv + static_cast<int64_t>(m) * src_stride;
    for (int i = 0; i < kv_dim; ++i) {
      cache[dst + i] = src[k_off + i];
      cache[dst + plane + i] = src[v_off + i];
    }
  }
}

// ---------------------------------------------------------------------------------------------
// fp8 KV variant (the reference names fp8 KV as its next lever, docs/optimization.md:119-120, and has
// no such path; the format is defined here). K and V rows are stored as e4m3 bytes,
// cache8 [num_blocks][2][16][kv_dim] u8, with one fp32 scale per (token, kv head, plane),
// scales [num_blocks][n_kv][2][16]: s = amax / 448 over the head's 128 values (s = 1 when the row is
// all zero), stored byte = e4m3(x * (448 / amax)) rounded to nearest even and saturated to +-448;
// a value reads back as e4m3_to_float(byte) * s. Every step is a single IEEE fp32 operation, so a
// device implementation that uses the same operations matches bit for bit.
// ---------------------------------------------------------------------------------------------
static inline float e4m3_to_f32(uint8_t b) {
  const int e = (b >> 3) & 15, m = b & 7;
  float v = e == 0 ? std::ldexp(static_cast<float>(m), -9) : std::ldexp(1.0f + m / 8.0f, e - 7);
  if (e == 15 && m == 7) v = NAN;
  return (b & 0x80) ? -v : v;
}

static inline uint8_t f32_to_e4m3(float f) {
  const uint8_t sign = std::signbit(f) ? 0x80 : 0;
  float a = std::fabs(f);
  if (a != a) return sign | 0x7F;
  if (a >= 464.0f) return sign | 0x7E;  // 464 is halfway to the next step above 448: saturates
  if (a == 0.0f) return sign;
  int ex;
  std::frexp(a, &ex);                   // a = m * 2^ex, m in [0.5, 1): a in [2^(ex-1), 2^ex)
  int e = ex - 1;
  if (e < -6) e = -6;                   // subnormals share the quantum of the smallest normal binade
  const float quantum = std::ldexp(1.0f, e - 3);
  const float q = std::nearbyint(a / quantum);  // round to nearest even (default rounding mode); exact division
  const float v = q * quantum;
  if (v > 448.0f) return sign | 0x7E;
  if (v < std::ldexp(1.0f, -6)) return sign | static_cast<uint8_t>(q);  // subnormal: q = 0..7
  int ev;
  const float mv = std::frexp(v, &ev);  // v = mv * 2^ev, mv in [0.5, 1)
  const int be = ev - 1 + 7;
  const int bm = static_cast<int>((mv * 2.0f - 1.0f) * 8.0f);
  return sign | static_cast<uint8_t>((be << 3) | bm);
}

uint8_t orc_f32_to_e4m3(float f) { return f32_to_e4m3(f); }
float orc_e4m3_to_f32(uint8_t b) { return e4m3_to_f32(b); }

void orc_kv_append_fp8(uint8_t* cache8, float* scales, int kv_dim, const uint16_t* qkv, int src_stride,
                       int k_off, int v_off, const int32_t* bt, int bt_stride, const int32_t* bt_row,
                       const int32_t* pos, int M) {
  const int n_kv = kv_dim / kHd;
  const int64_t plane = static_cast<int64_t>(kTok) * kv_dim;
  for (int m = 0; m < M; ++m) {
    const int32_t* row_bt = bt + static_cast<int64_t>(bt_row[m]) * bt_stride;
    const int p = pos[m];
    const int64_t blk = row_bt[p / kTok];
    const uint16_t* src = qkv + static_cast<int64_t>(m) * src_stride;
    for (int pl = 0; pl < 2; ++pl)
      for (int h = 0; h < n_kv; ++h) {
        const uint16_t* x = src + (pl ? v_off : k_off) + h * kHd;
        float amax = 0.f;
        for (int d = 0; d < kHd; ++d) amax = std::max(amax, std::fabs(bf2f(x[d])));
        const float s = amax > 0.f ? amax / 448.0f : 1.0f;
        const float inv = amax > 0.f ? 448.0f / amax : 0.0f;
        scales[((blk * n_kv + h) * 2 + pl) * kTok + p % kTok] = s;
        uint8_t* dst = cache8 + (blk * kPlanes + pl) * plane + static_cast<int64_t>(p % kTok) * kv_dim + h * kHd;
        for (int d = 0; d < kHd; ++d) dst[d] = f32_to_e4m3(bf2f(x[d]) * inv);
      }
  }
}

// Blocks of the fp8 cache read back as bf16 (no reference counterpart; the format is the one of
// orc_kv_append_fp8): out block i = block list[i], every value bf16(e4m3_to_float(byte) * scale) --
// the product is one fp32 multiplication, the conversion rounds to nearest even.
void orc_dequant_blocks_fp8(const uint8_t* cache8, const float* scales, int kv_dim, const int32_t* list, int n,
                            uint16_t* out) {
  const int n_kv = kv_dim / kHd;
  const int64_t plane = static_cast<int64_t>(kTok) * kv_dim;
  for (int i = 0; i < n; ++i) {
    const int64_t blk = list[i];
    for (int pl = 0; pl < 2; ++pl)
      for (int t = 0; t < kTok; ++t)
        for (int h = 0; h < n_kv; ++h) {
          const float s = scales[((blk * n_kv + h) * 2 + pl) * kTok + t];
          const uint8_t* src = cache8 + (blk * kPlanes + pl) * plane + static_cast<int64_t>(t) * kv_dim + h * kHd;
          uint16_t* dst = out + (static_cast<int64_t>(i) * kPlanes + pl) * plane + static_cast<int64_t>(t) * kv_dim + h * kHd;
          for (int d = 0; d < kHd; ++d) dst[d] = f2bf(e4m3_to_f32(src[d]) * s);
        }
  }
}

// Decode attention over the fp8 cache: orc_attn_decode with every K / V value read back as
// e4m3_to_float(byte) * scale (exact in fp32: 4 significant bits times a float).
void orc_attn_decode_fp8(const uint16_t* q, int q_stride, const uint8_t* cache8, const float* scales,
                         uint16_t* out, int n_heads, int n_kv, const int32_t* pos, const int32_t* qstart,
                         const int32_t* decode_rids, int n_decode, const int32_t* bt, int max_blocks,
                         float scale, int nthreads) {
  const int kv_dim = n_kv * kHd;
  const int group = n_heads / n_kv;
  const int64_t plane = static_cast<int64_t>(kTok) * kv_dim;
  parallel_for(n_decode * n_heads, nthreads, [&](int job) {
    int di = job / n_heads, h = job % n_heads;
    int r = decode_rids[di], flat = qstart[r], qpos = pos[flat];
    int kvh = h / group;
    const int32_t* row_bt = bt + static_cast<int64_t>(r) * max_blocks;
    const uint16_t* qv = q + static_cast<int64_t>(flat) * q_stride + static_cast<int64_t>(h) * kHd;
    float qf[kHd];
    for (int d = 0; d < kHd; ++d) qf[d] = bf2f(qv[d]);
    int n = qpos + 1;
    std::vector<float> s(n > 0 ? n : 0);
    float mx = -INFINITY;
    for (int t = 0; t < n; ++t) {
      const int64_t blk = row_bt[t / kTok];
      const int64_t base = blk * kPlanes * plane + static_cast<int64_t>(t % kTok) * kv_dim + static_cast<int64_t>(kvh) * kHd;
      const float ks = scales[((blk * n_kv + kvh) * 2 + 0) * kTok + t % kTok];
      float dot = 0.f;
      for (int d = 0; d < kHd; ++d) dot += qf[d] * (e4m3_to_f32(cache8[base + d]) * ks);
      s[t] = dot * scale;
      mx = std::max(mx, s[t]);
    }
    double acc[kHd];
    for (int d = 0; d < kHd; ++d) acc[d] = 0.0;
    double denom = 0.0;
    for (int t = 0; t < n; ++t) {
      float p = std::exp(s[t] - mx);
      denom += p;
      const int64_t blk = row_bt[t / kTok];
      const int64_t base = blk * kPlanes * plane + plane + static_cast<int64_t>(t % kTok) * kv_dim + static_cast<int64_t>(kvh) * kHd;
      const float vs = scales[((blk * n_kv + kvh) * 2 + 1) * kTok + t % kTok];
      for (int d = 0; d < kHd; ++d) acc[d] += static_cast<double>(p) * (e4m3_to_f32(cache8[base + d]) * vs);
    }
    uint16_t* o = out + (static_cast<int64_t>(flat) * n_heads + h) * kHd;
    for (int d = 0; d < kHd; ++d)
      o[d] = f2bf(denom > 0.0 ? static_cast<float>(acc[d] / denom) : 0.f);
  });
}

// ---------------------------------------------------------------------------------------------
// Decode attention: engine/src/attn_cute.cu:165-238 (split + combine collapse to one exact
// softmax). For decode sequence di: r = decode_rids[di], flat = qstart[r], qpos = pos[flat];
// query head h attends keys 0..qpos inclusive of kv head h / (n_heads / n_kv); the score is
// (q . k) * scale; out[(flat * n_heads + h) * 128 + d] in bf16. A sequence with no key (qpos < 0)
// gets zeros (attn_cute.cu:236, inv = 0 when the sum is not positive).
// ---------------------------------------------------------------------------------------------
void orc_attn_decode(const uint16_t* q, int q_stride, const uint16_t* cache, uint16_t* out,
                     int n_heads, int n_kv, const int32_t* pos, const int32_t* qstart,
                     const int32_t* decode_rids, int n_decode, const int32_t* bt, int max_blocks,
                     float scale, int nthreads) {
  const int kv_dim = n_kv * kHd;
  const int group = n_heads / n_kv;
  const int64_t plane = static_cast<int64_t>(kTok) * kv_dim;
  parallel_for(n_decode * n_heads, nthreads, [&](int job) {
    int di = job / n_heads, h = job % n_heads;
    int r = decode_rids[di], flat = qstart[r], qpos = pos[flat];
    int kvh = h / group;
    const int32_t* row_bt = bt + static_cast<int64_t>(r) * max_blocks;
    const uint16_t* qv = q + static_cast<int64_t>(flat) * q_stride + static_cast<int64_t>(h) * kHd;
    float qf[kHd];
    for (int d = 0; d < kHd; ++d) qf[d] = bf2f(qv[d]);
    int n = qpos + 1;
    std::vector<float> s(n > 0 ? n : 0);
    float mx = -INFINITY;
    for (int t = 0; t < n; ++t) {
      int64_t base = static_cast<int64_t>(row_bt[t / kTok]) * kPlanes * plane +
                     static_cast<int64_t>(t % kTok) * kv_dim + static_cast<int64_t>(kvh) * kHd;
      float dot = 0.f;
      for (int d = 0; d < kHd; ++d) dot += qf[d] * bf2f(cache[base + d]);
      s[t] = dot * scale;
      mx = std::max(mx, s[t]);
    }
    double acc[kHd];
    for (int d = 0; d < kHd; ++d) acc[d] = 0.0;
    double denom = 0.0;
    for (int t = 0; t < n; ++t) {
      float p = std::exp(s[t] - mx);
      denom += p;
      int64_t base = static_cast<int64_t>(row_bt[t / kTok]) * kPlanes * plane + plane +
                     static_cast<int64_t>(t % kTok) * kv_dim + static_cast<int64_t>(kvh) * kHd;
      for (int d = 0; d < kHd; ++d) acc[d] += static_cast<double>(p) * bf2f(cache[base + d]);
    }
    uint16_t* o = out + (static_cast<int64_t>(flat) * n_heads + h) * kHd;
    for (int d = 0; d < kHd; ++d)
      o[d] = f2bf(denom > 0.0 ? static_cast<float>(acc[d] / denom) : 0.f);
  });
}

// ---------------------------------------------------------------------------------------------
// Chunked-prefill attention: engine/src/attn_cute.cu:30-147. For prefill request r = rids[z],
// rows qs..qs+ql-1 (qs = qstart[r], ql = qlen[r]) are contiguous; row i attends key positions
// kpos <= pos[qs+i] (attn_cute.cu:116) read through r's block-table row. mirror_p != 0 rounds
// the probabilities to bf16 before the PV sum, as the reference's tensor-core path does
// (attn_cute.cu:128).
// ---------------------------------------------------------------------------------------------
void orc_attn_prefill(const uint16_t* q, int q_stride, const uint16_t* cache, uint16_t* out,
                      int n_heads, int n_kv, const int32_t* pos, const int32_t* qstart,
                      const int32_t* qlen, const int32_t* rids, int R, const int32_t* bt,
                      int max_blocks, float scale, int mirror_p, int nthreads) {
  const int kv_dim = n_kv * kHd;
  const int group = n_heads / n_kv;
  const int64_t plane = static_cast<int64_t>(kTok) * kv_dim;
  std::vector<std::pair<int, int>> jobs;  // (z, row)
  for (int z = 0; z < R; ++z)
    for (int i = 0; i < qlen[rids[z]]; ++i) jobs.emplace_back(z, i);
  parallel_for(static_cast<int>(jobs.size()), nthreads, [&](int j) {
    int r = rids[jobs[j].first], i = jobs[j].second;
    int row = qstart[r] + i, qp = pos[row];
    const int32_t* row_bt = bt + static_cast<int64_t>(r) * max_blocks;
    int n = qp + 1;
    std::vector<float> s(n > 0 ? n : 0);
    for (int h = 0; h < n_heads; ++h) {
      int kvh = h / group;
      const uint16_t* qv =
          q + static_cast<int64_t>(row) * q_stride + static_cast<int64_t>(h) * kHd;
      float qf[kHd];
      for (int d = 0; d < kHd; ++d) qf[d] = bf2f(qv[d]);
      float mx = -INFINITY;
      for (int t = 0; t < n; ++t) {
        int64_t base = static_cast<int64_t>(row_bt[t / kTok]) * kPlanes * plane +
                       static_cast<int64_t>(t % kTok) * kv_dim + static_cast<int64_t>(kvh) * kHd;
        float dot = 0.f;
        for (int d = 0; d < kHd; ++d) dot += qf[d] * bf2f(cache[base + d]);
        s[t] = dot * scale;
        mx = std::max(mx, s[t]);
      }
      double acc[kHd];
      for (int d = 0; d < kHd; ++d) acc[d] = 0.0;
      double denom = 0.0;
      for (int t = 0; t < n; ++t) {
        float p = std::exp(s[t] - mx);
        denom += p;
        float pv = mirror_p ? bf2f(f2bf(p)) : p;
        int64_t base = static_cast<int64_t>(row_bt[t / kTok]) * kPlanes * plane + plane +
                       static_cast<int64_t>(t % kTok) * kv_dim + static_cast<int64_t>(kvh) * kHd;
        for (int d = 0; d < kHd; ++d) acc[d] += static_cast<double>(pv) * bf2f(cache[base + d]);
      }
      uint16_t* o = out + (static_cast<int64_t>(row) * n_heads + h) * kHd;
      for (int d = 0; d < kHd; ++d)
        o[d] = f2bf(denom > 0.0 ? static_cast<float>(acc[d] / denom) : 0.f);
    }
  });
}

// ---------------------------------------------------------------------------------------------
// RoPE tables: engine/src/model_runtime.cu:111-126. [n_pos][head_dim/2] fp32,
// inv = powf(theta, -2 i / head_dim), ang = p * inv (fp32), cos/sin of the fp32 angle.
// ---------------------------------------------------------------------------------------------
void orc_rope_tables(float* cos_tab, float* sin_tab, int n_pos, int head_dim, float theta) {
  int half = head_dim / 2;
  for (int p = 0; p < n_pos; ++p)
    for (int i = 0; i < half; ++i) {
      float inv = std::pow(theta, -2.0f * i / head_dim);
      float ang = p * inv;
      cos_tab[static_cast<int64_t>(p) * half + i] = std::cos(ang);
      sin_tab[static_cast<int64_t>(p) * half + i] = std::sin(ang);
    }
}

// ---------------------------------------------------------------------------------------------
// Per-head RMSNorm + NeoX rotary embedding in place on the q and k heads of a fused qkv row:
// engine/src/kernels.cu:97-131. Head g < n_q uses weight wq, n_q <= g < n_q+n_kv uses wk; V is
// untouched. Sum of squares follows the reference's pairwise halving order (stride 64,32,..,1)
// so that an IEEE device implementation with the same tree can match bit for bit;
// inv = 1/sqrt(mean + eps) is IEEE here (the reference's fast-math rsqrtf may differ by an ulp).
// ---------------------------------------------------------------------------------------------
void orc_head_norm_rope(uint16_t* buf, const float* wq, const float* wk, const float* cos_tab,
                        const float* sin_tab, const int32_t* pos, int M, int n_q, int n_kv,
                        int head_dim, int stride, float eps) {
  int half = head_dim / 2;
  std::vector<float> sq(head_dim), y(head_dim);
  for (int m = 0; m < M; ++m)
    for (int g = 0; g < n_q + n_kv; ++g) {
      uint16_t* v = buf + static_cast<int64_t>(m) * stride + static_cast<int64_t>(g) * head_dim;
      const float* w = g < n_q ? wq : wk;
      for (int t = 0; t < head_dim; ++t) {
        float x = bf2f(v[t]);
        sq[t] = x * x;
      }
      for (int s = head_dim / 2; s > 0; s >>= 1)
        for (int t = 0; t < s; ++t) sq[t] = sq[t] + sq[t + s];
      float inv = 1.0f / std::sqrt(sq[0] / head_dim + eps);
      for (int t = 0; t < head_dim; ++t) y[t] = bf2f(v[t]) * inv * w[t];
      const float* cb = cos_tab + static_cast<int64_t>(pos[m]) * half;
      const float* sb = sin_tab + static_cast<int64_t>(pos[m]) * half;
      for (int t = 0; t < half; ++t) {
        float a = y[t] * cb[t];
        float b = y[t + half] * sb[t];
        float c = y[t + half] * cb[t];
        float d = y[t] * sb[t];
        v[t] = f2bf(a - b);
        v[t + half] = f2bf(c + d);
      }
    }
}

// ---------------------------------------------------------------------------------------------
// Prefix-block copies (no reference kernel: the reference only ever aliases full blocks,
// engine/src/scheduler.cc:30-40). copy: cache[dst] <- cache[src] for each pair, whole page, both
// planes, pairs applied in order. gather: out[i] <- cache[list[i]].
// ---------------------------------------------------------------------------------------------
void orc_copy_blocks(uint16_t* cache, int kv_dim, const int32_t* pairs, int n_pairs) {
  const int64_t blk = static_cast<int64_t>(kPlanes) * kTok * kv_dim;
  for (int i = 0; i < n_pairs; ++i)
    std::memmove(cache + pairs[2 * i + 1] * blk, cache + pairs[2 * i] * blk, blk * 2);
}

void orc_gather_blocks(const uint16_t* cache, int kv_dim, const int32_t* list, int n,
                       uint16_t* out) {
  const int64_t blk = static_cast<int64_t>(kPlanes) * kTok * kv_dim;
  for (int i = 0; i < n; ++i) std::memcpy(out + i * blk, cache + list[i] * blk, blk * 2);
}

// ---------------------------------------------------------------------------------------------
// Prefix hash chain: engine/src/scheduler.cc:16-24. Golden-ratio seed xor, then per token
// xor / FNV-prime multiply / rotate-left 27; 0 is remapped to 1 because 0 means "no hash".
// ---------------------------------------------------------------------------------------------
uint64_t orc_hash_block(uint64_t parent, const int32_t* tokens, int n) {
  uint64_t h = parent ^ 0x9E3779B97F4A7C15ull;
  for (int i = 0; i < n; ++i) {
    h ^= static_cast<uint64_t>(static_cast<uint32_t>(tokens[i]));
    h *= 0x100000001B3ull;
    h = (h << 27) | (h >> 37);
  }
  return h ? h : 1;
}

// ---------------------------------------------------------------------------------------------
// Step metadata: engine/src/model_runtime.cu:54-91. qlen[r] = rows of request r, qstart =
// exclusive prefix sum, request is decode iff qlen == 1, else prefill; returns max prefill qlen
// (at least 1). Block tables are packed with row stride bt_stride; entries past a request's own
// length are left as they were (the reference does not clear the stale tail).
// out_counts = {n_decode, n_prefill, prefill_max_qlen}.
// ---------------------------------------------------------------------------------------------
void orc_step_pack(const int32_t* req_index, int n_rows, int n_req, int32_t* qstart,
                   int32_t* qlen, int32_t* decode_rids, int32_t* prefill_rids,
                   int32_t* out_counts) {
  for (int r = 0; r < n_req; ++r) qlen[r] = 0;
  for (int t = 0; t < n_rows; ++t) qlen[req_index[t]]++;
  int acc = 0;
  for (int r = 0; r < n_req; ++r) {
    qstart[r] = acc;
    acc += qlen[r];
  }
  int nd = 0, np = 0, mx = 1;
  for (int r = 0; r < n_req; ++r) {
    if (qlen[r] == 1)
      decode_rids[nd++] = r;
    else {
      prefill_rids[np++] = r;
      mx = std::max(mx, qlen[r]);
    }
  }
  out_counts[0] = nd;
  out_counts[1] = np;
  out_counts[2] = mx;
}

// ---------------------------------------------------------------------------------------------
// Block allocator: engine/src/block_allocator.h:21-101, restated with index-linked lists.
// Free blocks form an LRU queue initialised 0..N-1. alloc pops the front, drops that block's
// hash mapping and sets refcount 1. free decrements and at zero appends to the LRU back keeping
// the hash. lookup(hash) returns the mapped block (taking it out of the queue if it was free)
// and increments its refcount, or -1. insert(b, hash) does nothing when b already carries a hash
// or the hash is already mapped.
// ---------------------------------------------------------------------------------------------
struct OrcAlloc {
  int n;
  std::vector<int> ref, prev, next;   // prev/next = -2 when not queued
  std::vector<uint64_t> hash;
  std::unordered_map<uint64_t, int> map;
  int head = -1, tail = -1, nfree = 0;
  void push_back(int b) {
    prev[b] = tail;
    next[b] = -1;
    if (tail >= 0) next[tail] = b; else head = b;
    tail = b;
    ++nfree;
  }
  void unlink(int b) {
    int p = prev[b], q = next[b];
    if (p >= 0) next[p] = q; else head = q;
    if (q >= 0) prev[q] = p; else tail = p;
    prev[b] = next[b] = -2;
    --nfree;
  }
};

void* orc_alloc_create(int num_blocks) {
  auto* a = new OrcAlloc;
  a->n = num_blocks;
  a->ref.assign(num_blocks, 0);
  a->prev.assign(num_blocks, -2);
  a->next.assign(num_blocks, -2);
  a->hash.assign(num_blocks, 0);
  for (int b = 0; b < num_blocks; ++b) a->push_back(b);
  return a;
}
void orc_alloc_destroy(void* h) { delete static_cast<OrcAlloc*>(h); }
int orc_alloc_num_free(void* h) { return static_cast<OrcAlloc*>(h)->nfree; }
int orc_alloc_refcount(void* h, int b) { return static_cast<OrcAlloc*>(h)->ref[b]; }
uint64_t orc_alloc_block_hash(void* h, int b) { return static_cast<OrcAlloc*>(h)->hash[b]; }

int orc_alloc_one(void* h) {  // -1 when the pool is dry
  auto* a = static_cast<OrcAlloc*>(h);
  if (a->head < 0) return -1;
  int b = a->head;
  a->unlink(b);
  if (a->hash[b]) {
    auto it = a->map.find(a->hash[b]);
    if (it != a->map.end() && it->second == b) a->map.erase(it);
    a->hash[b] = 0;
  }
  a->ref[b] = 1;
  return b;
}
void orc_alloc_free_one(void* h, int b) {
  auto* a = static_cast<OrcAlloc*>(h);
  if (--a->ref[b] == 0) a->push_back(b);
}
// grows table (length *len, capacity cap) to ceil(n_tok/16) entries; 1 = ok, 0 = pool dry
int orc_alloc_grow(void* h, int32_t* table, int* len, int cap, int n_tok) {
  int need = (n_tok + kTok - 1) / kTok;
  while (*len < need && *len < cap) {
    int b = orc_alloc_one(h);
    if (b < 0) return 0;
    table[(*len)++] = b;
  }
  return *len >= need ? 1 : 0;
}
int orc_alloc_lookup(void* h, uint64_t hash) {
  auto* a = static_cast<OrcAlloc*>(h);
  auto it = a->map.find(hash);
  if (it == a->map.end()) return -1;
  int b = it->second;
  if (a->ref[b] == 0) a->unlink(b);
  ++a->ref[b];
  return b;
}
void orc_alloc_insert(void* h, int b, uint64_t hash) {
  auto* a = static_cast<OrcAlloc*>(h);
  if (a->hash[b]) return;
  if (a->map.count(hash)) return;
  a->hash[b] = hash;
  a->map[hash] = b;
}

// Prefix acquisition: engine/src/scheduler.cc:27-44. Looks up at most (n_tokens-1)/16 full
// blocks, chaining hashes from parent 0, stops at the first miss. Returns the number of blocks
// adopted (computed tokens = that * 16) and writes the last hash of the chain.
int orc_acquire_prefix(void* h, const int32_t* tokens, int n_tokens, int32_t* table,
                       uint64_t* last_hash) {
  int limit = (n_tokens - 1) / kTok;
  uint64_t parent = 0;
  int nb = 0;
  for (; nb < limit; ++nb) {
    uint64_t hv = orc_hash_block(parent, tokens + nb * kTok, kTok);
    int b = orc_alloc_lookup(h, hv);
    if (b < 0) break;
    table[nb] = b;
    parent = hv;
  }
  *last_hash = nb > 0 ? parent : 0;
  return nb;
}

// Publishing computed blocks: engine/src/scheduler.cc:46-57. Full blocks [cached, computed/16)
// are hashed onward from *last_hash and inserted; returns the new cached-block count.
int orc_cache_blocks(void* h, const int32_t* tokens, int computed, const int32_t* table,
                     int cached, uint64_t* last_hash) {
  int full = computed / kTok;
  uint64_t parent = *last_hash;
  for (int i = cached; i < full; ++i) {
    parent = orc_hash_block(parent, tokens + i * kTok, kTok);
    orc_alloc_insert(h, table[i], parent);
  }
  *last_hash = parent;
  return full;
}

// Copy-on-write rule (defined for this project; the reference shares only full blocks so it
// never fires there): before a sequence writes token position `pos` into its block
// table[pos/16], if that block has refcount > 1 and pos%16 != 0, take a fresh block b', record
// (old, b') as a copy pair, put b' into the table and drop one reference of the old block.
// Returns 1 if a pair was produced, 0 if not needed, -1 if the pool is dry.
int orc_cow_prepare(void* h, int32_t* table, int pos, int32_t* pair) {
  auto* a = static_cast<OrcAlloc*>(h);
  int idx = pos / kTok;
  int b = table[idx];
  if (a->ref[b] <= 1 || pos % kTok == 0) return 0;
  int nb = orc_alloc_one(h);
  if (nb < 0) return -1;
  pair[0] = b;
  pair[1] = nb;
  table[idx] = nb;
  orc_alloc_free_one(h, b);
  return 1;
}

int orc_hardware_threads() { return static_cast<int>(std::thread::hardware_concurrency()); }

}  // extern "C"
