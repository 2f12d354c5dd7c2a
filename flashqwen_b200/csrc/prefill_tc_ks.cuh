// Kernel 3: chunked-prefill paged attention on tcgen05 / tensor memory, key-split form.
//
// Operator semantics follow the reference's CutePrefillKernel / LaunchAttnPrefillCute
// (engine/src/attn_cute.cu:30-163 of the FlashQwen tree): rows of one request are contiguous, row i
// sees key positions <= pos[qstart+i], the scale is applied after Q K^T, probabilities are rounded to
// bf16 before P V, bf16 output at out[(row*n_heads + h)*128 + d]. The design is not the reference's:
//
//   * One CTA = 32 query rows x the 4 query heads of one kv head = one 128-row MMA tile
//     (row = head * 32 + query row); keys are consumed 64 at a time (4 pages). The CTA's two warp
//     groups take the two HALVES OF THE KEY RANGE of that tile: each group has its own K/V ring, S
//     tiles and O accumulator in tensor memory and its own softmax warps, both run concurrently (the
//     tensor pipe stays fed by two independent pipelines), and at the end group 0 merges group 1's
//     (max, sum) from shared memory and its O straight out of tensor memory by log-sum-exp. With
//     skewed histories (one request at 7000 cached tokens beside one at 0) the longest jobs decide the
//     run time; the split halves them without any scratch in global memory.
//   * TMA warps (one per half): per page and plane two 2 KiB boxes (one per 64-dim half) placed so
//     that a 64-key K tile / V tile is a canonical 128-byte-swizzled UMMA operand
//     ([half][key][64 dims], 8-key groups 1024 bytes apart); 3-deep ring of 32 KiB stages per half.
//   * One thread issues S = Q K^T (M128 N64, 8 k-steps of 16 dims, both operands K-major) into one of
//     two 64-column TMEM buffers per half; another issues O += P V (M128 N128, 4 k-steps of 16 keys,
//     V MN-major) with P read from tensor memory: the softmax overwrites the first 32 columns of its
//     S tile with packed bf16 pairs.
//   * Softmax warps: thread = one row (one TMEM lane): tcgen05.ld of its 64 scores, causal mask,
//     running max without any shuffle (three-input max), scale and subtract, sums as two-wide fp32
//     instructions, exp2, P -> bf16. The accumulator is rescaled in TMEM only
//     when a row's max grew by more than 2^8 since the scale in use (the probabilities stay exact
//     relative to that scale).
// Completion is tracked with mbarriers (tcgen05.commit for MMA groups); every wait is bounded and
// ends in a status code. A kernel that allocates tensor memory runs one CTA per SM here; the CTA
// allocates 512 columns and frees them before exit.
#pragma once

#include <cmath>

#include "umma.cuh"

namespace fqb {

struct PrefillParams {
  const __nv_bfloat16* q;
  int q_stride;
  __nv_bfloat16* out;
  int n_heads, n_kv;
  const int* pos;
  const int* qstart;
  const int* qlen;
  const int* rids;
  const int* bt;
  int max_blocks, num_blocks;
  float scale_log2;  // softmax scale * log2(e), > 0
};

constexpr int kTcGroupRows = 32;  // query rows per CTA (x 4 q heads = one 128-row MMA tile)
constexpr int kTcBN = 64;         // keys per tile
constexpr int kTcGroupCols = 256; // TMEM columns per key half: S0 [0,64), S1 [64,128), O [128,256)

template <int STAGES>
struct TcKsSmem {
  static constexpr int kQ = 0;                                  // [2 k-blocks][128 rows][128 B]
  static constexpr int kKV = 32768;                             // 2 rings x STAGES x {K 16 KiB, V 16 KiB}
  static constexpr int kStage = 32768;
  static constexpr int kRing = STAGES * kStage;
  static constexpr int kBars = kKV + 2 * kRing;
  static constexpr int kTmemSlot = kBars + 40 * 8;
  static constexpr int kMl = kTmemSlot + 16;                    // group 1's {row sum, row maximum}: 2 x 128 floats
  static constexpr int kTotal = kMl + 2 * 128 * 4;
  static constexpr int kAlloc = kTotal;                         // base must be 1024-byte aligned (checked)
  static constexpr int kThreads = 12 * 32;                      // 8 softmax, 2 TMA, S issuer, PV issuer
};

template <int STAGES>
__global__ void __launch_bounds__(TcKsSmem<STAGES>::kThreads, 1)
prefill_tc_ks_kernel(const __grid_constant__ CUtensorMap tmap, const PrefillParams P) {
  using L = TcKsSmem<STAGES>;
  static_assert(STAGES == 3 && L::kTotal <= 232448, "two rings of 3 x 32 KiB plus Q fill the 227 KiB");
  constexpr int kCols = 2 * kTcGroupCols;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) report(FQB_ERR_INVALID, kKidPrefill, static_cast<int>(smem_u32(smem)));
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
  // per group gi at bars + 16*gi: kv_full[3], kv_empty[3], s_full[2], p_full[2], o_done[2]; q_full at 32
  auto kv_full = [&](int gi, int s) { return bars + 16 * gi + s; };
  auto kv_empty = [&](int gi, int s) { return bars + 16 * gi + 3 + s; };
  auto s_full = [&](int gi, int b) { return bars + 16 * gi + 6 + b; };
  auto p_full = [&](int gi, int b) { return bars + 16 * gi + 8 + b; };
  auto o_done = [&](int gi, int b) { return bars + 16 * gi + 10 + b; };
  uint64_t* q_full = bars + 32;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kTmemSlot);

  // Longest jobs first: CTAs are handed out in blockIdx order (x fastest, z slowest), a job's length is
  // its last visible key position, and one CTA per SM runs at a time, so the z-th CTA plane takes the
  // request with the z-th longest key range (ranked here on the device; up to 32 requests, more keep
  // their given order) and x walks its query tiles from the last one down. The loads that rank the
  // requests also bring every request's row count, first row and the position of this query tile's last
  // row, one request per lane, so once the CTA knows which request it serves nothing more has to be
  // fetched before the block table.
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kvh = blockIdx.y;
  const int qtile = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
  const int q0 = qtile * kTcGroupRows;
  int r, ql, qs, tile_last;
  if (gridDim.z > 1 && gridDim.z <= 32) {
    int rr = 0, n = 0, s0 = 0, len = -1, tl = -1;
    if (lane < static_cast<int>(gridDim.z)) {
      rr = P.rids[lane];
      n = P.qlen[rr];
      s0 = P.qstart[rr];
      len = n > 0 ? P.pos[s0 + n - 1] : -1;
      tl = q0 < n ? P.pos[s0 + min(q0 + kTcGroupRows, n) - 1] : -1;
    }
    int rank = 0;
    for (int j = 0; j < static_cast<int>(gridDim.z); ++j) {
      const int other = __shfl_sync(0xffffffffu, len, j);
      rank += (other > len || (other == len && j < lane)) ? 1 : 0;
    }
    const unsigned hit =
        __ballot_sync(0xffffffffu, lane < static_cast<int>(gridDim.z) && rank == static_cast<int>(blockIdx.z));
    const int zsel = hit ? __ffs(hit) - 1 : static_cast<int>(blockIdx.z);
    r = __shfl_sync(0xffffffffu, rr, zsel);
    ql = __shfl_sync(0xffffffffu, n, zsel);
    qs = __shfl_sync(0xffffffffu, s0, zsel);
    tile_last = __shfl_sync(0xffffffffu, tl, zsel);
  } else {
    r = P.rids[blockIdx.z];
    ql = P.qlen[r];
    qs = P.qstart[r];
    tile_last = q0 < ql ? P.pos[qs + min(q0 + kTcGroupRows, ql) - 1] : -1;
  }
  if (q0 >= ql) return;  // before any allocation; the whole CTA leaves together

  if (warp == 10) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "n"(kCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    tma_prefetch_desc(&tmap);
    for (int gi = 0; gi < 2; ++gi) {
      for (int s = 0; s < STAGES; ++s) {
        mbar_init(kv_full(gi, s), 1);
        mbar_init(kv_empty(gi, s), 1);
      }
      for (int b = 0; b < 2; ++b) {
        mbar_init(s_full(gi, b), 1);
        mbar_init(p_full(gi, b), 4);
        mbar_init(o_done(gi, b), 1);
      }
    }
    mbar_init(q_full, 4);
    mbar_fence_init();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  int last_pos = tile_last;
  if (last_pos >= P.max_blocks * kTok) {
    if (tid == 0) report(FQB_ERR_INDEX, kKidPrefill, last_pos);
    last_pos = P.max_blocks * kTok - 1;
  }
  const int npages = last_pos < 0 ? 0 : last_pos / kTok + 1;
  const int ntiles = last_pos < 0 ? 0 : last_pos / kTcBN + 1;
  // group 0 takes tiles [0, cut), group 1 takes [cut, ntiles)
  const int cut = (ntiles + 1) / 2;
  auto g_begin = [&](int gi) { return gi == 0 ? 0 : cut; };
  auto g_count = [&](int gi) { return gi == 0 ? cut : ntiles - cut; };
  bool dead = false;
  auto wait = [&](uint64_t* bar, uint32_t parity, int what) {
    if (!dead && !mbar_wait_bounded(bar, parity)) {
      dead = true;
      report(FQB_ERR_TIMEOUT, kKidPrefill, what);
    }
  };
  float* ml = reinterpret_cast<float*>(smem + L::kMl);

  if (warp < 8) {
    // =========================== softmax warps: one thread per MMA row, per key half ===========================
    const int gi = warp >> 2;
    const int row = tid & 127;
    const int g = warp & 3, qi = lane;
    const int qrow = q0 + qi;
    const bool valid = qrow < ql;
    const int my_begin = g_begin(gi), my_tiles = g_count(gi);
    if (gi == 0) {  // group 0's warps load the shared Q tile
      const uint4* src = reinterpret_cast<const uint4*>(
          P.q + static_cast<long long>(qs + (valid ? qrow : q0)) * P.q_stride + (kvh * kGroup + g) * kHd);
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const uint4 v = valid ? __ldg(src + c) : make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(smem + L::kQ + (c >> 3) * 16384 + row * 128 + (((c & 7) ^ (row & 7)) << 4)) = v;
      }
      proxy_fence_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(q_full);
    }
    const int qp = valid ? P.pos[qs + qrow] : -1;
    const uint32_t lane_addr = tmem + gi * kTcGroupCols + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    float m_used = kNegBig, l = 0.f;

#pragma unroll 1
    for (int i = 0; i < my_tiles; ++i) {
      const int b = i & 1;
      const int k = my_begin + i;
      wait(s_full(gi, b), (i >> 1) & 1, k);
      tc_fence_after();
      float x[kTcBN];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld16(lane_addr + b * 64 + c * 16, x + c * 16);
      tmem_wait_ld();
      const int k0 = k * kTcBN;
      // Keys this row may not see get a score of -inf, so their probability is exactly 0 whatever the
      // scale: ex2(fma(-inf, scale, -m)) = 0. A tile in which the row sees no key at all (the upper key
      // half of a row near the start of the chunk) then leaves the row's maximum, sum and O untouched:
      // its tile maximum is -inf, m_used stays the finite value it had (at least kNegBig), nothing grows.
      // (Masking with a large finite number instead goes wrong exactly there: the maximum in use
      // becomes the rounded product of that number and the scale, and the exponent of a masked key the
      // rounding residue of the same product, about +-1e21 -- inf for half of all scales.)
      if (k0 + kTcBN - 1 > qp) {
#pragma unroll
        for (int j = 0; j < kTcBN; ++j)
          if (k0 + j > qp) x[j] = -INFINITY;
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int j = 0; j < kTcBN; j += 8) {
        mx0 = fmax3(mx0, x[j], x[j + 1]);
        mx1 = fmax3(mx1, x[j + 2], x[j + 3]);
        mx2 = fmax3(mx2, x[j + 4], x[j + 5]);
        mx3 = fmax3(mx3, x[j + 6], x[j + 7]);
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * P.scale_log2;
      const float m_new = fmaxf(m_used, mx);
      const bool grow = m_new > m_used + 8.f;
      const float f = grow ? fast_exp2(m_used - m_new) : 1.f;
      if (grow) {
        m_used = m_new;
        l *= f;
      }
      float2 sm0 = make_float2(0.f, 0.f), sm1 = make_float2(0.f, 0.f);
      float pf[kTcBN / 2];
      const float2 sc2 = make_float2(P.scale_log2, P.scale_log2), nm2 = make_float2(-m_used, -m_used);
#pragma unroll
      for (int j = 0; j < kTcBN; j += 4) {
        float2 e0 = ffma2(make_float2(x[j], x[j + 1]), sc2, nm2);
        float2 e1 = ffma2(make_float2(x[j + 2], x[j + 3]), sc2, nm2);
        e0.x = fast_exp2(e0.x); e0.y = fast_exp2(e0.y);
        e1.x = fast_exp2(e1.x); e1.y = fast_exp2(e1.y);
        sm0 = fadd2(sm0, e0);
        sm1 = fadd2(sm1, e1);
        pf[j >> 1] = __uint_as_float(pack_bf16(e0.x, e0.y));
        pf[(j >> 1) + 1] = __uint_as_float(pack_bf16(e1.x, e1.y));
      }
      l += (sm0.x + sm0.y) + (sm1.x + sm1.y);
      const bool any_grow = i > 0 && __any_sync(0xffffffffu, grow);
      if (any_grow) {  // PV of the tile before must have finished before O is rescaled
        wait(o_done(gi, (i - 1) & 1), ((i - 1) >> 1) & 1, 1000 + k);
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          float o[16];
          tmem_ld16(lane_addr + 128 + c * 16, o);
          tmem_wait_ld();
#pragma unroll
          for (int q = 0; q < 16; ++q) o[q] *= f;
          tmem_st16(lane_addr + 128 + c * 16, o);
        }
        tmem_wait_st();
      }
      // P over the first 32 columns of S[b] (column c = keys 2c and 2c+1)
      tmem_st16(lane_addr + b * 64, pf);
      tmem_st16(lane_addr + b * 64 + 16, pf + 16);
      tmem_wait_st();
      if (k == ntiles - 1) {  // key slots past the last position: clear their V rows (0 * garbage)
        const int nvalid = last_pos - k0 + 1;
        uint8_t* vst = smem + L::kKV + gi * L::kRing + (i % STAGES) * L::kStage + 16384;
        for (int idx = row; idx < (kTcBN - nvalid) * 16; idx += 128) {
          const int vr = nvalid + (idx >> 4), c = idx & 15;
          *reinterpret_cast<uint4*>(vst + (c >> 3) * 8192 + vr * 128 + ((c & 7) << 4)) = make_uint4(0, 0, 0, 0);
        }
        proxy_fence_async();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full(gi, b));
    }
    if (my_tiles > 0) {
      wait(o_done(gi, (my_tiles - 1) & 1), ((my_tiles - 1) >> 1) & 1, 2000 + gi);
      tc_fence_after();
    }
    // ---- merge the two key halves ----
    // Group 1 publishes only its row sums and maxima (shared memory); its O stays in tensor memory, where
    // group 0's thread of the same row can read it: a warp reaches the 32 TMEM lanes of its quarter in ALL
    // columns, and warps w and w + 4 are in the same quarter.
    if (gi == 1) {
      ml[row] = my_tiles > 0 ? l : 0.f;
      ml[128 + row] = my_tiles > 0 ? m_used : kNegBig;
    }
    tc_fence_before();
    asm volatile("bar.sync 1, 256;" ::: "memory");  // the 8 softmax warps only
    tc_fence_after();
    if (gi == 0) {
      const float l1 = ml[row], m1 = ml[128 + row];
      const float m0 = my_tiles > 0 ? m_used : kNegBig;
      const float mm = fmaxf(m0, m1);
      const float f0 = my_tiles > 0 ? fast_exp2(m0 - mm) : 0.f, f1 = l1 > 0.f ? fast_exp2(m1 - mm) : 0.f;
      const float lt = l * f0 + l1 * f1;
      const float inv = lt > 0.f ? 1.f / lt : 0.f;
      const bool other = g_count(1) > 0;  // same for the whole CTA
      __nv_bfloat16* orow = P.out + (static_cast<long long>(qs + qrow) * P.n_heads + kvh * kGroup + g) * kHd;
#pragma unroll 1
      for (int c = 0; c < 8; ++c) {
        float o[16], o1[16];
        if (my_tiles > 0) tmem_ld16(lane_addr + 128 + c * 16, o);
        if (other) tmem_ld16(lane_addr + kTcGroupCols + 128 + c * 16, o1);
        tmem_wait_ld();
#pragma unroll
        for (int q = 0; q < 16; ++q)
          o[q] = ((my_tiles > 0 ? o[q] * f0 : 0.f) + (other && f1 > 0.f ? o1[q] * f1 : 0.f)) * inv;
        if (valid) {
          uint4 a, bq;
          a.x = pack_bf16(o[0], o[1]);    a.y = pack_bf16(o[2], o[3]);
          a.z = pack_bf16(o[4], o[5]);    a.w = pack_bf16(o[6], o[7]);
          bq.x = pack_bf16(o[8], o[9]);   bq.y = pack_bf16(o[10], o[11]);
          bq.z = pack_bf16(o[12], o[13]); bq.w = pack_bf16(o[14], o[15]);
          *reinterpret_cast<uint4*>(orow + c * 16) = a;
          *reinterpret_cast<uint4*>(orow + c * 16 + 8) = bq;
        }
      }
    }
    tc_fence_before();
  } else if (warp < 10) {
    // =========================== TMA producers, one per key half ===========================
    const int gi = warp - 8;
    const int my_begin = g_begin(gi), my_tiles = g_count(gi);
    const int* btr = P.bt + static_cast<long long>(r) * P.max_blocks;
#pragma unroll 1
    for (int i = 0; i < my_tiles; ++i) {
      const int stage = i % STAGES;
      const int pg0 = (my_begin + i) * 4;
      const int npg = min(4, npages - pg0);
      const int mine = lane < npg ? __ldg(btr + pg0 + lane) : 0;
      if (i >= STAGES) wait(kv_empty(gi, stage), ((i / STAGES) - 1) & 1, 3000 + i);
      if (lane < npg && static_cast<unsigned>(mine) >= static_cast<unsigned>(P.num_blocks))
        report(FQB_ERR_INDEX, kKidPrefill, mine);
      uint8_t* st = smem + L::kKV + gi * L::kRing + stage * L::kStage;
      if (lane == 0) mbar_expect_tx(kv_full(gi, stage), static_cast<uint32_t>(npg) * kPageBytes);
      __syncwarp();
      if (lane < npg) {
#pragma unroll
        for (int plane = 0; plane < 2; ++plane)
#pragma unroll
          for (int half = 0; half < 2; ++half)
            tma_load_half(st + plane * 16384 + half * 8192 + lane * 2048, &tmap, kv_full(gi, stage), kvh * 2 + half,
                          plane, mine);
      }
    }
  } else if (warp == 10) {
    // =========================== S = Q K^T issuer (one thread, both halves) ===========================
    if (lane == 0) {
      constexpr uint32_t kIdescS = umma_idesc(128, kTcBN, false);
      const uint64_t qd = umma_desc(smem_u32(smem + L::kQ), 16, 1024);
      wait(q_full, 0, 4000);
      tc_fence_after();
      const int most = max(g_count(0), g_count(1));
#pragma unroll 1
      for (int i = 0; i < most; ++i) {
        const int b = i & 1, stage = i % STAGES;
#pragma unroll
        for (int gi = 0; gi < 2; ++gi) {
          if (i >= g_count(gi)) continue;
          wait(kv_full(gi, stage), (i / STAGES) & 1, 5000 + i);
          if (i >= 2) wait(o_done(gi, b), ((i - 2) >> 1) & 1, 6000 + i);  // PV two tiles back has read P out of S[b]
          tc_fence_after();
          const uint64_t kd = umma_desc(smem_u32(smem + L::kKV + gi * L::kRing + stage * L::kStage), 16, 1024);
          const uint32_t d = tmem + gi * kTcGroupCols + b * 64;
#pragma unroll
          for (int kb = 0; kb < 2; ++kb)
#pragma unroll
            for (int j = 0; j < 4; ++j)
              umma_bf16(d, qd + ((kb * 16384 + j * 32) >> 4), kd + ((kb * 8192 + j * 32) >> 4), kIdescS,
                        (kb | j) ? 1u : 0u);
          umma_commit(s_full(gi, b));
        }
      }
    }
    tc_fence_before();
  } else {
    // =========================== O += P V issuer (one thread, both halves) ===========================
    if (lane == 0) {
      constexpr uint32_t kIdescO = umma_idesc(128, kHd, true);
      const int most = max(g_count(0), g_count(1));
#pragma unroll 1
      for (int i = 0; i < most; ++i) {
        const int b = i & 1, stage = i % STAGES;
#pragma unroll
        for (int gi = 0; gi < 2; ++gi) {
          if (i >= g_count(gi)) continue;
          wait(p_full(gi, b), (i >> 1) & 1, 7000 + i);
          tc_fence_after();
          const uint64_t vd = umma_desc(smem_u32(smem + L::kKV + gi * L::kRing + stage * L::kStage + 16384), 8192, 1024);
          const uint32_t d = tmem + gi * kTcGroupCols + 128;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            umma_bf16_ts(d, tmem + gi * kTcGroupCols + b * 64 + j * 8, vd + ((j * 2048) >> 4), kIdescO,
                         (i | j) ? 1u : 0u);
          umma_commit(o_done(gi, b));
          umma_commit(kv_empty(gi, stage));
        }
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 10) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(kCols) : "memory");
  }
}

}  // namespace fqb
