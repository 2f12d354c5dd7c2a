// Kernel 3: chunked-prefill paged attention (causal over the chunk, full over the cached history).
//
// Operator semantics follow the reference's CutePrefillKernel / LaunchAttnPrefillCute
// (engine/src/attn_cute.cu:30-163 of the FlashQwen tree): rows of one request are contiguous,
// row i sees key positions <= pos[qstart+i], scale applied after QK^T, probabilities rounded to
// bf16 before PV, bf16 output at out[(row*n_heads + h)*128 + d]. The design differs:
//
//   * one CTA serves a tile of BM query rows for ALL 4 query heads of one kv head (the reference
//     runs one head per CTA and so fetches every K/V page 4 times);
//   * K/V pages arrive through a ring of TMA tensor loads (same 8 KiB box as decode) issued by a
//     dedicated producer warp under full/empty mbarriers, so loads overlap the math (the reference
//     loads synchronously between four __syncthreads per page);
//   * block-table entries are fetched 32 at a time by the producer warp, ahead of use;
//   * QK^T and PV run on tensor cores (mma.sync m16n8k16, fp32 accumulate), 16 query rows of one
//     head per warp.
#pragma once

#include "common.cuh"

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
  float scale_log2;
};

// RT row tiles of 16 rows each -> BM = 16*RT query rows, 4*RT consumer warps + 1 producer warp
template <int RT, int NS>
struct PrefillCfg {
  static constexpr int kConsumers = 4 * RT;
  static constexpr int kThreads = (kConsumers + 1) * 32;
  static constexpr int kBM = 16 * RT;
  static constexpr int kSmem = NS * kPageBytes + 2 * NS * 8 + 1024;
};

template <int RT, int NS, int MINB>
__global__ void __launch_bounds__(PrefillCfg<RT, NS>::kThreads, MINB)
prefill_kernel(const __grid_constant__ CUtensorMap tmap, const PrefillParams P) {
  using C = PrefillCfg<RT, NS>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + NS * kPageBytes);
  uint64_t* empty = full + NS;

  const int r = P.rids[blockIdx.z];
  const int kvh = blockIdx.y;
  const int qtile = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);  // long tiles first
  const int ql = P.qlen[r], qs = P.qstart[r];
  const int q0 = qtile * C::kBM;
  if (q0 >= ql) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    tma_prefetch_desc(&tmap);
    for (int i = 0; i < NS; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], C::kConsumers);
    }
    mbar_fence_init();
  }
  __syncthreads();

  const int qlast = min(q0 + C::kBM, ql) - 1;
  int last_pos = P.pos[qs + qlast];
  if (last_pos >= P.max_blocks * kTok) {
    report(FQB_ERR_INDEX, kKidPrefill, last_pos);
    last_pos = P.max_blocks * kTok - 1;
  }
  const int ntiles = last_pos / kTok + 1;  // pages 0..ntiles-1 (<= 0 when last_pos < 0)
  const int* btr = P.bt + static_cast<long long>(r) * P.max_blocks;

  if (warp == C::kConsumers) {
    // ---------------- producer warp ----------------
    int slot = 0;
    uint32_t phase = 0;
    bool dead = false;
    int cur = lane < ntiles ? __ldg(btr + lane) : 0;
    for (int base = 0; base < ntiles; base += 32) {
      const int nxt_idx = base + 32 + lane;
      const int nxt = nxt_idx < ntiles ? __ldg(btr + nxt_idx) : 0;
      const int cnt = min(32, ntiles - base);
      for (int i = 0; i < cnt; ++i) {
        const int blk = __shfl_sync(0xffffffffu, cur, i);
        const int kt = base + i;
        if (kt >= NS) {  // slot was used before: wait until every consumer warp released it
          if (!dead && !mbar_wait_bounded(&empty[slot], phase ^ 1u)) {
            dead = true;
            report(FQB_ERR_TIMEOUT, kKidPrefill, kt);
          }
        }
        if (static_cast<unsigned>(blk) >= static_cast<unsigned>(P.num_blocks))
          report(FQB_ERR_INDEX, kKidPrefill, blk);  // the load reads zeros
        if (lane == 0) {
          mbar_expect_tx(&full[slot], kPageBytes);
          tma_load_page(smem + slot * kPageBytes, &tmap, &full[slot], 0, 0, kvh * 2, 0, blk);
        }
        slot = (slot + 1 == NS) ? 0 : slot + 1;
        if (slot == 0) phase ^= 1u;
      }
      cur = nxt;
    }
    return;
  }

  // ---------------- consumer warps ----------------
  const int hsub = warp & 3, rt = warp >> 2;
  const int head = kvh * kGroup + hsub;
  const int g = lane >> 2, t = lane & 3;
  const int row_lo = q0 + rt * 16 + g, row_hi = row_lo + 8;  // rows inside the request
  const bool ok_lo = row_lo < ql, ok_hi = row_hi < ql;
  const int qp_lo = ok_lo ? P.pos[qs + row_lo] : -1;
  const int qp_hi = ok_hi ? P.pos[qs + row_hi] : -1;
  // smallest / largest visible position over the warp's 16 rows, for skipping and mask elision
  int wmin = ok_lo ? qp_lo : 0x7fffffff, wmax = max(qp_lo, qp_hi);
  if (ok_hi) wmin = min(wmin, qp_hi);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    wmin = min(wmin, __shfl_xor_sync(0xffffffffu, wmin, o));
    wmax = max(wmax, __shfl_xor_sync(0xffffffffu, wmax, o));
  }

  uint32_t qa[8][4];
  {
    const uint32_t* qlo = reinterpret_cast<const uint32_t*>(
        P.q + static_cast<long long>(qs + row_lo) * P.q_stride + head * kHd);
    const uint32_t* qhi = reinterpret_cast<const uint32_t*>(
        P.q + static_cast<long long>(qs + row_hi) * P.q_stride + head * kHd);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      qa[ks][0] = ok_lo ? __ldg(qlo + ks * 8 + t) : 0u;
      qa[ks][1] = ok_hi ? __ldg(qhi + ks * 8 + t) : 0u;
      qa[ks][2] = ok_lo ? __ldg(qlo + ks * 8 + t + 4) : 0u;
      qa[ks][3] = ok_hi ? __ldg(qhi + ks * 8 + t + 4) : 0u;
    }
  }
  float o[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m_lo = kNegBig, m_hi = kNegBig, l_lo = 0.f, l_hi = 0.f;

  const int mat = lane >> 3;
  const int k_tok = ((mat >> 1) << 3) + (lane & 7), k_sel = mat & 1;
  const int v_tok = ((mat & 1) << 3) + (lane & 7), v_sel = mat >> 1;
  int slot = 0;
  uint32_t phase = 0;
  bool dead = false;

#pragma unroll 1
  for (int kt = 0; kt < ntiles; ++kt) {
    if (!dead && !mbar_wait_bounded(&full[slot], phase)) {
      dead = true;
      report(FQB_ERR_TIMEOUT, kKidPrefill, kt);
    }
    if (kt * kTok <= wmax) {  // some row of this warp sees the page
      if (kt == ntiles - 1 && last_pos - kt * kTok + 1 < kTok) {
        // token slots past the chunk's last position were never written: their V rows may hold
        // anything (0 * NaN would poison PV). Every warp clears them before its own reads;
        // the warps store the same zeros, so the overlap is harmless.
        uint8_t* st = smem + slot * kPageBytes;
        if (lane < 16)
          for (int row = last_pos - kt * kTok + 1; row < kTok; ++row)
            *reinterpret_cast<uint4*>(st + kPlaneBytes + (lane >> 3) * kHalfBytes + row * 128 +
                                      ((lane & 7) << 4)) = make_uint4(0, 0, 0, 0);
        __syncwarp();
      }
      const uint32_t kbase = smem_u32(smem + slot * kPageBytes), vbase = kbase + kPlaneBytes;
      float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(kbase + page_chunk_off(k_tok, ks * 2 + k_sel), b0, b1, b2, b3);
        mma_bf16(s0, qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
        mma_bf16(s1, qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b2, b3);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        s0[i] *= P.scale_log2;
        s1[i] *= P.scale_log2;
      }
      if (kt * kTok + kTok - 1 > wmin) {  // page crosses the causal edge of some row
        const int k0 = kt * kTok + 2 * t;
        if (k0 > qp_lo) s0[0] = kNegBig;
        if (k0 + 1 > qp_lo) s0[1] = kNegBig;
        if (k0 > qp_hi) s0[2] = kNegBig;
        if (k0 + 1 > qp_hi) s0[3] = kNegBig;
        if (k0 + 8 > qp_lo) s1[0] = kNegBig;
        if (k0 + 9 > qp_lo) s1[1] = kNegBig;
        if (k0 + 8 > qp_hi) s1[2] = kNegBig;
        if (k0 + 9 > qp_hi) s1[3] = kNegBig;
      }
      float mx_lo = fmaxf(fmaxf(s0[0], s0[1]), fmaxf(s1[0], s1[1]));
      float mx_hi = fmaxf(fmaxf(s0[2], s0[3]), fmaxf(s1[2], s1[3]));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
      const float c_lo = fast_exp2(m_lo - mn_lo), c_hi = fast_exp2(m_hi - mn_hi);
      m_lo = mn_lo;
      m_hi = mn_hi;
      s0[0] = fast_exp2(s0[0] - mn_lo); s0[1] = fast_exp2(s0[1] - mn_lo);
      s1[0] = fast_exp2(s1[0] - mn_lo); s1[1] = fast_exp2(s1[1] - mn_lo);
      s0[2] = fast_exp2(s0[2] - mn_hi); s0[3] = fast_exp2(s0[3] - mn_hi);
      s1[2] = fast_exp2(s1[2] - mn_hi); s1[3] = fast_exp2(s1[3] - mn_hi);
      l_lo = l_lo * c_lo + ((s0[0] + s0[1]) + (s1[0] + s1[1]));
      l_hi = l_hi * c_hi + ((s0[2] + s0[3]) + (s1[2] + s1[3]));
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        o[j][0] *= c_lo; o[j][1] *= c_lo;
        o[j][2] *= c_hi; o[j][3] *= c_hi;
      }
      const uint32_t pa0 = pack_bf16(s0[0], s0[1]), pa1 = pack_bf16(s0[2], s0[3]);
      const uint32_t pa2 = pack_bf16(s1[0], s1[1]), pa3 = pack_bf16(s1[2], s1[3]);
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_trans(vbase + page_chunk_off(v_tok, jj * 2 + v_sel), b0, b1, b2, b3);
        mma_bf16(o[2 * jj], pa0, pa1, pa2, pa3, b0, b1);
        mma_bf16(o[2 * jj + 1], pa0, pa1, pa2, pa3, b2, b3);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[slot]);
    slot = (slot + 1 == NS) ? 0 : slot + 1;
    if (slot == 0) phase ^= 1u;
  }

  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  const float i_lo = l_lo > 0.f ? 1.f / l_lo : 0.f, i_hi = l_hi > 0.f ? 1.f / l_hi : 0.f;
  if (ok_lo) {
    uint32_t* dst = reinterpret_cast<uint32_t*>(
        P.out + (static_cast<long long>(qs + row_lo) * P.n_heads + head) * kHd);
#pragma unroll
    for (int j = 0; j < 16; ++j) dst[j * 4 + t] = pack_bf16(o[j][0] * i_lo, o[j][1] * i_lo);
  }
  if (ok_hi) {
    uint32_t* dst = reinterpret_cast<uint32_t*>(
        P.out + (static_cast<long long>(qs + row_hi) * P.n_heads + head) * kHd);
#pragma unroll
    for (int j = 0; j < 16; ++j) dst[j * 4 + t] = pack_bf16(o[j][2] * i_hi, o[j][3] * i_hi);
  }
}

}  // namespace fqb
