// Kernel 3, Blackwell tensor-core version: chunked-prefill paged attention on tcgen05 / TMEM.
//
// Same operator as prefill_kernel (semantics of the reference's CutePrefillKernel,
// engine/src/attn_cute.cu:30-147 of the FlashQwen tree). One CTA = 32 query rows x the 4 query
// heads of one kv head = a 128-row MMA tile (row = head * 32 + query row); keys are consumed 64 at
// a time (4 pages).
//
//   TMA warp    producer: per page and plane two 2 KiB boxes (one per 64-dim half) placed so
//               that a 64-key K tile / V tile is a canonical 128-byte-swizzled UMMA operand
//               ([half][key][64 dims], 8-key groups 1024 bytes apart); STAGES-deep ring of 32 KiB stages.
//   MMA warps   one thread of each issues tcgen05.mma: the first S = Q K^T (M128 N64, 8 k-steps of 16 dims, both
//               operands K-major) into one of two 64-column TMEM buffers, and O += P V
//               (M128 N128, 4 k-steps of 16 keys, V MN-major) into a 128-column TMEM accumulator (issued by
//               the second warp). P is the A operand either from tensor memory (TS: it overwrites the
//               first 32 columns of its S tile as bf16 pairs) or from a swizzled shared-memory tile.
//               The S issuer runs up to two tiles ahead of the softmax, so the tensor pipe works while the
//               softmax runs; all descriptors are built once, the issue loops only add k-step offsets.
//   warps 0-3 (and 4-7 with two row groups per CTA)
//               softmax: thread = one row (one TMEM lane): tcgen05.ld of its 64 scores, scale,
//               causal mask, running max without any shuffle, exp2, P -> bf16.
//               The accumulator is rescaled in TMEM only when a row's max grew by more than 2^8
//               since the scale in use (the probabilities stay exact relative to that scale).
// Completion is tracked with mbarriers (tcgen05.commit for MMA groups); every wait is bounded and
// ends in a status code. A kernel that allocates tensor memory runs one CTA per SM here; the CTA
// allocates 256 columns per row group and frees them before exit.
// This file also holds the building blocks (descriptors, TMEM access, fences) that the key-split
// kernel in prefill_tc_ks.cuh, the default, is made of.
#pragma once

#include "common.cuh"
#include "prefill.cuh"

namespace fqb {

constexpr int kTcGroupRows = 32;  // query rows per group (x 4 q heads = one 128-row MMA tile)
constexpr int kTcBN = 64;         // keys per tile
constexpr int kTcGroupCols = 256; // TMEM columns per group: S0 [0,64), S1 [64,128), O [128,256)

// G = row groups per CTA (1 or 2): each group is a 128-row MMA tile with its own Q, P, S and O; the
// groups share the K/V stages, so with G = 2 every K/V tile fetched from L2 feeds twice the math and
// the softmax of one group overlaps the MMAs of the other.
template <int G, int STAGES, bool TS = true>
struct TcSmem {
  static constexpr int kQ = 0;                                   // G x [2 k-blocks][128 rows][128 B]
  static constexpr int kKV = G * 32768;                          // stages x {K 16 KiB, V 16 KiB}
  static constexpr int kStage = 32768;
  static constexpr int kP = kKV + STAGES * kStage;               // G x 2 x [128 rows][128 B]
  static constexpr int kBars = kP + (TS ? 0 : G * 2 * 16384);      // no P tiles when P lives in TMEM
  static constexpr int kTmemSlot = kBars + 32 * 8;
  static constexpr int kTotal = kTmemSlot + 16;
  static constexpr int kAlloc = kTotal;                          // base must be 1024-byte aligned (checked)
  static constexpr int kThreads = (4 * G + 3) * 32;              // softmax warps, TMA warp, two MMA-issue warps
  static constexpr int kRows = G * kTcGroupRows;                 // query rows per CTA
};

// ---- UMMA descriptors -----------------------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle: start address, leading / stride byte offsets
// in 16-byte units, descriptor version 1 (sm_100), layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}
// Instruction descriptor for kind::f16: fp32 accumulate, bf16 A and B, A K-major, B K- or MN-major.
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a), "l"(b), "r"(idesc), "r"(acc)
      : "memory");
}
// the same MMA with the A operand read from tensor memory (128 lanes x 8 columns of bf16 pairs)
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void proxy_fence_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// 16 consecutive fp32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const float* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(
          taddr),
      "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
      "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
      "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
      "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15]))
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 4-D tiled load of a 2 KiB box {64 dims, 16 tokens, 1 half, 1 plane, 1 block}
__device__ __forceinline__ void tma_load_half(void* dst, const CUtensorMap* m, uint64_t* bar, int half, int plane,
                                              int blk) {
  tma_load_page(dst, m, bar, 0, 0, half, plane, blk);
}

// TS: P stays in tensor memory (it overwrites the first 32 columns of the S tile it came from, as
// packed bf16 pairs) and is the A operand of the PV MMA from there, instead of going through a
// swizzled shared-memory tile.
template <int G, int STAGES, bool TS>
__global__ void __launch_bounds__(TcSmem<G, STAGES, TS>::kThreads, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap tmap, const PrefillParams P) {
  using L = TcSmem<G, STAGES, TS>;
  static_assert(G >= 1 && G <= 2 && STAGES >= 2 && STAGES <= 5, "barrier block and TMEM are laid out for these");
  constexpr int kCols = G * kTcGroupCols;
  constexpr int kProducerWarp = 4 * G, kMmaWarp = 4 * G + 1;  // warp 4G+2 issues PV
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if ((smem_u32(smem) & 1023u) != 0) {  // the swizzled operand tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) report(FQB_ERR_INVALID, kKidPrefill, static_cast<int>(smem_u32(smem)));
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
  uint64_t* kv_full = bars;        // [5]  producer -> MMA (tx bytes)
  uint64_t* kv_empty = bars + 5;   // [5]  MMA commit -> producer
  // per group gi at bars + 10 + 10*gi: s_full[2] (MMA commit -> softmax), s_free[2] (softmax, 1 per warp ->
  // MMA), p_full[2] (softmax, 1 per warp -> MMA), o_done[2] (MMA commit -> softmax), q_full. S, P and
  // their barriers are double-buffered by tile parity, so the softmax of tile k+1 never waits for the
  // MMA round trip of tile k (a single P buffer tied every tile to two cross-warp hand-offs).
  auto s_full = [&](int gi, int b) { return bars + 10 + 10 * gi + b; };
  auto s_free = [&](int gi, int b) { return bars + 10 + 10 * gi + 2 + b; };
  auto p_full = [&](int gi, int b) { return bars + 10 + 10 * gi + 4 + b; };
  auto o_done = [&](int gi, int b) { return bars + 10 + 10 * gi + 6 + b; };
  auto q_full = [&](int gi) { return bars + 10 + 10 * gi + 8; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kTmemSlot);

  // Longest jobs first: CTAs are handed out in blockIdx order (x fastest, z slowest), a job's length
  // is its last visible key position, and one CTA per SM runs at a time, so the z-th CTA plane takes
  // the request with the z-th longest key range (ranked here on the device; up to 32 requests, more
  // keep their given order) and x walks its query tiles from the last one down.
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int zsel = blockIdx.z;
  if (gridDim.z > 1 && gridDim.z <= 32) {
    int len = -1;
    if (lane < static_cast<int>(gridDim.z)) {
      const int rr = P.rids[lane];
      const int n = P.qlen[rr];
      len = n > 0 ? P.pos[P.qstart[rr] + n - 1] : -1;
    }
    int rank = 0;
    for (int j = 0; j < static_cast<int>(gridDim.z); ++j) {
      const int other = __shfl_sync(0xffffffffu, len, j);
      rank += (other > len || (other == len && j < lane)) ? 1 : 0;
    }
    const unsigned hit = __ballot_sync(0xffffffffu, lane < static_cast<int>(gridDim.z) && rank == static_cast<int>(blockIdx.z));
    zsel = hit ? __ffs(hit) - 1 : static_cast<int>(blockIdx.z);
  }
  const int r = P.rids[zsel];
  const int kvh = blockIdx.y;
  const int qtile = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);  // long tiles first
  const int ql = P.qlen[r], qs = P.qstart[r];
  const int q0 = qtile * L::kRows;
  if (q0 >= ql) return;  // before any allocation; the whole CTA leaves together

  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "n"(kCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    tma_prefetch_desc(&tmap);
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    for (int gi = 0; gi < G; ++gi) {
      for (int b = 0; b < 2; ++b) {
        mbar_init(s_full(gi, b), 1);
        mbar_init(s_free(gi, b), 4);
      }
      for (int b = 0; b < 2; ++b) {
        mbar_init(p_full(gi, b), 4);
        mbar_init(o_done(gi, b), 1);
      }
      mbar_init(q_full(gi), 4);
    }
    mbar_fence_init();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  // Per group: last visible key position of its rows and the number of 64-key tiles it consumes.
  // A later group has later rows, so the CTA loads max over the groups (pages up to cta_last).
  int g_last[G], g_tiles[G];
  int cta_last = -1;
#pragma unroll
  for (int gi = 0; gi < G; ++gi) {
    const int first = q0 + gi * kTcGroupRows;
    int lp = -1;
    if (first < ql) {
      lp = P.pos[qs + min(first + kTcGroupRows, ql) - 1];
      if (lp >= P.max_blocks * kTok) {
        if (tid == 0) report(FQB_ERR_INDEX, kKidPrefill, lp);
        lp = P.max_blocks * kTok - 1;
      }
    }
    g_last[gi] = lp;
    g_tiles[gi] = lp < 0 ? 0 : lp / kTcBN + 1;
    cta_last = max(cta_last, lp);
  }
  const int npages = cta_last < 0 ? 0 : cta_last / kTok + 1;
  const int ntiles = cta_last < 0 ? 0 : cta_last / kTcBN + 1;
  bool dead = false;
  auto wait = [&](uint64_t* bar, uint32_t parity, int what) {
    if (!dead && !mbar_wait_bounded(bar, parity)) {
      dead = true;
      report(FQB_ERR_TIMEOUT, kKidPrefill, what);
    }
  };

  if (warp < 4 * G) {
    // =========================== softmax warps: one thread per MMA row ===========================
    const int gi = warp >> 2;            // row group
    const int row = tid & 127;           // MMA row inside the group = head * 32 + query row
    const int g = warp & 3, qi = lane;
    const int qrow = q0 + gi * kTcGroupRows + qi;
    const bool valid = qrow < ql;
    uint8_t* q_smem = smem + L::kQ + gi * 32768;
    uint8_t* p_group = smem + L::kP + gi * 2 * 16384;
    const int my_tiles = g_tiles[gi];
    {
      const uint4* src = reinterpret_cast<const uint4*>(
          P.q + static_cast<long long>(qs + (valid ? qrow : q0)) * P.q_stride + (kvh * kGroup + g) * kHd);
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const uint4 v = valid ? __ldg(src + c) : make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(q_smem + (c >> 3) * 16384 + row * 128 + (((c & 7) ^ (row & 7)) << 4)) = v;
      }
    }
    proxy_fence_async();
    __syncwarp();
    if (lane == 0) mbar_arrive(q_full(gi));  // one arrival per warp: 128 arrivals on one word serialise
    const int qp = valid ? P.pos[qs + qrow] : -1;
    const uint32_t lane_addr = tmem + gi * kTcGroupCols + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    float m_used = kNegBig, l = 0.f;

#pragma unroll 1
    for (int k = 0; k < my_tiles; ++k) {
      const int b = k & 1;
      wait(s_full(gi, b), (k >> 1) & 1, k);
      tc_fence_after();
      float x[kTcBN];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld16(lane_addr + b * 64 + c * 16, x + c * 16);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (!TS && lane == 0) mbar_arrive(s_free(gi, b));  // with TS the S tile is free only after PV has read P from it
      const int k0 = k * kTcBN;
      if (k0 + kTcBN - 1 > qp) {  // the tile crosses this row's causal edge (or lies beyond it)
#pragma unroll
        for (int j = 0; j < kTcBN; ++j)
          if (k0 + j > qp) x[j] = kNegBig;
      }
      // four independent chains each for the max and for the sum: a single warp per scheduler has
      // nothing else to hide the dependent-issue latency of one long chain
      float mx0 = kNegBig, mx1 = kNegBig, mx2 = kNegBig, mx3 = kNegBig;
#pragma unroll
      for (int j = 0; j < kTcBN; j += 4) {
        mx0 = fmaxf(mx0, x[j]);
        mx1 = fmaxf(mx1, x[j + 1]);
        mx2 = fmaxf(mx2, x[j + 2]);
        mx3 = fmaxf(mx3, x[j + 3]);
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * P.scale_log2;  // scale > 0: max commutes
      const float m_new = fmaxf(m_used, mx);
      const bool grow = m_new > m_used + 8.f;  // keep the scale in use unless the max moved by > 2^8
      const float f = grow ? fast_exp2(m_used - m_new) : 1.f;
      if (grow) {
        m_used = m_new;
        l *= f;
      }
      float sm0 = 0.f, sm1 = 0.f, sm2 = 0.f, sm3 = 0.f;
      uint32_t pk[kTcBN / 2];
      const float neg_m = -m_used;
#pragma unroll
      for (int j = 0; j < kTcBN; j += 4) {
        const float p0 = fast_exp2(fmaf(x[j], P.scale_log2, neg_m));
        const float p1 = fast_exp2(fmaf(x[j + 1], P.scale_log2, neg_m));
        const float p2 = fast_exp2(fmaf(x[j + 2], P.scale_log2, neg_m));
        const float p3 = fast_exp2(fmaf(x[j + 3], P.scale_log2, neg_m));
        sm0 += p0; sm1 += p1; sm2 += p2; sm3 += p3;
        pk[j >> 1] = pack_bf16(p0, p1);
        pk[(j >> 1) + 1] = pack_bf16(p2, p3);
      }
      l += (sm0 + sm1) + (sm2 + sm3);
      // O is touched only when some row of the warp moved its scale: then PV of the tile before must
      // have finished. Otherwise only P[b] must be free again, i.e. PV of tile k-2 has finished.
      const bool any_grow = k > 0 && __any_sync(0xffffffffu, grow);
      if (any_grow) {
        wait(o_done(gi, (k - 1) & 1), ((k - 1) >> 1) & 1, 1000 + k);
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          float o[16];
          tmem_ld16(lane_addr + 128 + c * 16, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] *= f;
          tmem_st16(lane_addr + 128 + c * 16, o);
        }
        tmem_wait_st();
      } else if (k >= 2) {
        wait(o_done(gi, b), ((k - 2) >> 1) & 1, 1500 + k);
      }
      if (TS) {
        // P over the first 32 columns of S[b]: column c = keys 2c (low half) and 2c+1 (high half)
        float pf[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) pf[c] = __uint_as_float(pk[c]);
        tmem_st16(lane_addr + b * 64, pf);
        tmem_st16(lane_addr + b * 64 + 16, pf + 16);
        tmem_wait_st();
      } else {
        uint8_t* p_smem = p_group + b * 16384;
#pragma unroll
        for (int c = 0; c < 8; ++c)
          *reinterpret_cast<uint4*>(p_smem + row * 128 + ((c ^ (row & 7)) << 4)) =
              make_uint4(pk[c * 4], pk[c * 4 + 1], pk[c * 4 + 2], pk[c * 4 + 3]);
      }
      if (k == ntiles - 1) {
        // key slots past the CTA's last position (never written, or pages that do not exist): clear
        // their V rows so that 0 * garbage cannot reach an accumulator. Keys between this group's
        // and the CTA's last position are real data another group still needs; they stay.
        const int nvalid = cta_last - k0 + 1;
        uint8_t* vst = smem + L::kKV + (k % STAGES) * L::kStage + 16384;
        for (int idx = row; idx < (kTcBN - nvalid) * 16; idx += 128) {
          const int vr = nvalid + (idx >> 4), c = idx & 15;
          *reinterpret_cast<uint4*>(vst + (c >> 3) * 8192 + vr * 128 + ((c & 7) << 4)) = make_uint4(0, 0, 0, 0);
        }
      }
      proxy_fence_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full(gi, b));
    }
    // ---- epilogue: O / l -> bf16 -> out ----
    if (my_tiles > 0) {
      wait(o_done(gi, (my_tiles - 1) & 1), ((my_tiles - 1) >> 1) & 1, 2000);
      tc_fence_after();
    }
    const float inv = (l > 0.f && my_tiles > 0) ? 1.f / l : 0.f;
    __nv_bfloat16* orow = P.out + (static_cast<long long>(qs + qrow) * P.n_heads + kvh * kGroup + g) * kHd;
#pragma unroll 1
    for (int c = 0; c < 8; ++c) {
      float o[16];
      if (my_tiles > 0) {
        tmem_ld16(lane_addr + 128 + c * 16, o);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) o[i] = 0.f;
      }
      if (valid) {
        uint4 a, bq;
        a.x = pack_bf16(o[0] * inv, o[1] * inv);   a.y = pack_bf16(o[2] * inv, o[3] * inv);
        a.z = pack_bf16(o[4] * inv, o[5] * inv);   a.w = pack_bf16(o[6] * inv, o[7] * inv);
        bq.x = pack_bf16(o[8] * inv, o[9] * inv);  bq.y = pack_bf16(o[10] * inv, o[11] * inv);
        bq.z = pack_bf16(o[12] * inv, o[13] * inv); bq.w = pack_bf16(o[14] * inv, o[15] * inv);
        *reinterpret_cast<uint4*>(orow + c * 16) = a;
        *reinterpret_cast<uint4*>(orow + c * 16 + 8) = bq;
      }
    }
    tc_fence_before();
  } else if (warp == kProducerWarp) {
    // =========================== TMA producer ===========================
    const int* btr = P.bt + static_cast<long long>(r) * P.max_blocks;
#pragma unroll 1
    for (int k = 0; k < ntiles; ++k) {
      const int stage = k % STAGES;
      const int pg0 = k * 4;
      const int npg = min(4, npages - pg0);
      const int mine = lane < npg ? __ldg(btr + pg0 + lane) : 0;
      if (k >= STAGES) wait(&kv_empty[stage], ((k / STAGES) - 1) & 1, 3000 + k);
      if (lane < npg && static_cast<unsigned>(mine) >= static_cast<unsigned>(P.num_blocks))
        report(FQB_ERR_INDEX, kKidPrefill, mine);  // the loads below then read zeros
      uint8_t* st = smem + L::kKV + stage * L::kStage;
      if (lane == 0) mbar_expect_tx(&kv_full[stage], static_cast<uint32_t>(npg) * kPageBytes);
      __syncwarp();
      if (lane < npg) {
#pragma unroll
        for (int plane = 0; plane < 2; ++plane)
#pragma unroll
          for (int half = 0; half < 2; ++half)
            tma_load_half(st + plane * 16384 + half * 8192 + lane * 2048, &tmap, &kv_full[stage], kvh * 2 + half,
                          plane, mine);
      }
    }
  } else if (warp == kMmaWarp) {
    // =========================== S = Q K^T issuer (one thread) ===========================
    // Issuing is the hot loop of a single thread, so every descriptor is built once up front and
    // the loop only adds the k-step offsets (16-byte units) to the low word.
    if (lane == 0) {
      constexpr uint32_t kIdescS = umma_idesc(128, kTcBN, false);
      uint64_t qd[G], kd[STAGES];
#pragma unroll
      for (int gi = 0; gi < G; ++gi) qd[gi] = umma_desc(smem_u32(smem + L::kQ + gi * 32768), 16, 1024);
#pragma unroll
      for (int st = 0; st < STAGES; ++st) kd[st] = umma_desc(smem_u32(smem + L::kKV + st * L::kStage), 16, 1024);
#pragma unroll
      for (int gi = 0; gi < G; ++gi)
        if (g_tiles[gi] > 0) wait(q_full(gi), 0, 4000 + gi);
      tc_fence_after();
      int stage = 0;
      uint32_t kv_par = 0;
#pragma unroll 1
      for (int k = 0; k < ntiles; ++k) {
        const int b = k & 1;
        wait(&kv_full[stage], kv_par, 5000 + k);
        uint64_t kdesc = kd[0];
#pragma unroll
        for (int st = 1; st < STAGES; ++st) kdesc = stage == st ? kd[st] : kdesc;
        // One group after the other: measured, a tcgen05.mma of these shapes costs about
        // 80 + 0.55 * N clocks whether or not its neighbours are independent, and finishing one
        // group's S early lets its softmax start while the other group's MMAs still issue.
#pragma unroll
        for (int gi = 0; gi < G; ++gi) {
          if (k >= g_tiles[gi]) continue;  // this group's rows cannot see the tile
          if (k >= 2) {
            if (TS) wait(o_done(gi, b), ((k - 2) >> 1) & 1, 6000 + k);  // PV of tile k-2 has read P out of this tile
            else wait(s_free(gi, b), ((k >> 1) - 1) & 1, 6000 + k);
          }
          tc_fence_after();
          const uint32_t d = tmem + gi * kTcGroupCols + b * 64;
#pragma unroll
          for (int kb = 0; kb < 2; ++kb)
#pragma unroll
            for (int j = 0; j < 4; ++j)
              umma_bf16(d, qd[gi] + ((kb * 16384 + j * 32) >> 4), kdesc + ((kb * 8192 + j * 32) >> 4), kIdescS,
                        (kb | j) ? 1u : 0u);
          umma_commit(s_full(gi, b));
        }
        if (++stage == STAGES) {
          stage = 0;
          kv_par ^= 1u;
        }
      }
    }
    tc_fence_before();
  } else {
    // =========================== O += P V issuer (one thread) ===========================
    if (lane == 0) {
      constexpr uint32_t kIdescO = umma_idesc(128, kHd, true);
      uint64_t pd[G][2], vd[STAGES];
#pragma unroll
      for (int gi = 0; gi < G; ++gi)
#pragma unroll
        for (int b = 0; b < 2; ++b) pd[gi][b] = umma_desc(smem_u32(smem + L::kP + (gi * 2 + b) * 16384), 16, 1024);
#pragma unroll
      for (int st = 0; st < STAGES; ++st)
        vd[st] = umma_desc(smem_u32(smem + L::kKV + st * L::kStage + 16384), 8192, 1024);
      int stage = 0;
#pragma unroll 1
      for (int t = 0; t < ntiles; ++t) {
        const int b = t & 1;
        uint64_t vdesc = vd[0];
#pragma unroll
        for (int st = 1; st < STAGES; ++st) vdesc = stage == st ? vd[st] : vdesc;
#pragma unroll
        for (int gi = 0; gi < G; ++gi) {
          if (t >= g_tiles[gi]) continue;
          // P of the tile is in shared memory; S of the tile (and so the K/V stage) was complete
          // before the softmax could produce it
          wait(p_full(gi, b), (t >> 1) & 1, 7000 + t);
          tc_fence_after();
          const uint32_t d = tmem + gi * kTcGroupCols + 128;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (TS)
              umma_bf16_ts(d, tmem + gi * kTcGroupCols + b * 64 + j * 8, vdesc + ((j * 2048) >> 4), kIdescO,
                           (t | j) ? 1u : 0u);
            else
              umma_bf16(d, pd[gi][b] + ((j * 32) >> 4), vdesc + ((j * 2048) >> 4), kIdescO, (t | j) ? 1u : 0u);
          }
          umma_commit(o_done(gi, b));
        }
        umma_commit(&kv_empty[stage]);  // all PV of the tile issued; its S finished before P existed
        if (++stage == STAGES) stage = 0;
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(kCols) : "memory");
  }
}

}  // namespace fqb
