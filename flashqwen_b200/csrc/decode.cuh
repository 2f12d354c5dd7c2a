// Kernel 2: GQA-shared split-K paged decode attention and its log-sum-exp combine.
//
// Operator semantics follow the reference's LaunchAttnDecodeCute
// (engine/src/attn_cute.cu:165-261 of the FlashQwen tree): decode sequence di attends keys
// 0..qpos inclusive, one kv head serves its 4 query heads, fp32 accumulation, bf16 output at
// out[(flat*n_heads + h)*128 + d]. The design is not the reference's:
//
//   * Work is the flat list of page slices (sequence, kv head, page), each 8 KiB (K and V rows of
//     one head of one 16-token page). The list is cut into equal contiguous ranges, one per
//     persistent CTA, on the device from the actual context lengths -- the grid depends only on
//     the SM count, so the launch can sit in a CUDA graph while lengths change.
//   * Each warp owns a private ring of NS page buffers in shared memory filled by single-thread
//     TMA tensor loads (5-D box, 128-byte swizzle) that complete on the ring's mbarriers; the
//     warp that consumes a buffer refills it, so there is no cross-warp handshake in the stream
//     and loads run ahead across (sequence, head) boundaries.
//   * Scores and PV products use mma.sync m16n8k16 with the 4 query heads as rows 0..3 of the
//     16-row A tile (rows 4..15 are zero padding): S[4x16] = Q[4x128] K^T, O[4x128] += P[4x16] V.
//   * A (sequence, head) pair that lies inside one CTA is normalised and written straight to
//     `out`; a pair cut by a CTA boundary leaves one unnormalised partial per CTA
//     (slot = pair index + CTA index) and the combine kernel merges them.
#pragma once

#include "common.cuh"

namespace fqb {

constexpr int kMinSlicesPerCta = 16;

struct DecodeParams {
  const __nv_bfloat16* q;
  int q_stride;
  __nv_bfloat16* out;
  int n_heads, n_kv;
  const int* pos;
  const int* qstart;
  const int* rids;
  int n_decode;
  const int* bt;
  int max_blocks, num_blocks;
  float scale_log2;  // softmax scale * log2(e)
  float* pm;
  float* pl;
  float* pa;
  long long partial_slots;
};

// Tail of pm / pl reused as integers to hand the partition to the combine kernel:
//   pm_i[slots-1] = slices per CTA (W); pm_i[slots-2-di] = first page index of sequence di in the
//   flat list (exclusive prefix sum of pages); pl_i[slots-2-di] = pages of sequence di.
__device__ __forceinline__ int* meta_w(const DecodeParams& P) {
  return reinterpret_cast<int*>(P.pm) + (P.partial_slots - 1);
}
__device__ __forceinline__ int* meta_cum(const DecodeParams& P, int di) {
  return reinterpret_cast<int*>(P.pm) + (P.partial_slots - 2 - di);
}
__device__ __forceinline__ int* meta_np(const DecodeParams& P, int di) {
  return reinterpret_cast<int*>(P.pl) + (P.partial_slots - 2 - di);
}

// MAXD = sequences per launch (the host loops over larger batches)
template <int NW, int NS, int MAXD>
struct DecodeSmem {
  static constexpr int kStageBytes = NW * NS * kPageBytes;
  static constexpr int kBarOff = kStageBytes;
  static constexpr int kQOff = kBarOff + NW * NS * 8;
  static constexpr int kMoOff = kQOff + 2 * kGroup * kHd * 2;
  static constexpr int kMmOff = kMoOff + NW * kGroup * kHd * 4;
  static constexpr int kMlOff = kMmOff + NW * kGroup * 4;
  static constexpr int kROff = kMlOff + NW * kGroup * 4;
  static constexpr int kFlatOff = kROff + MAXD * 4;
  static constexpr int kQposOff = kFlatOff + MAXD * 4;
  static constexpr int kCumOff = kQposOff + MAXD * 4;
  static constexpr int kTotal = kCumOff + (MAXD + 1) * 4;
  static constexpr int kAlloc = kTotal + 1024;  // slack for manual 1024-byte alignment
};

// Walks the items (maximal runs of pages of one (sequence, kv head) pair) of a CTA's range.
struct ItemCursor {
  int off;     // flat slice offset of the current item's first page; >= hi when exhausted
  int di, kvh;
  int pb, pe;  // page range [pb, pe) of the item
  int np;      // pages of the whole sequence
};

__device__ __forceinline__ void item_at(ItemCursor& c, int off, int hi, int n_decode, int n_kv,
                                        const int* s_cum, const int* s_qpos) {
  c.off = off;
  if (off >= hi) return;
  // largest di with s_cum[di] * n_kv <= off (s_cum[n_decode] * n_kv = total > off)
  int lo = 0, up = n_decode;
  while (up - lo > 1) {
    int mid = (lo + up) >> 1;
    if (s_cum[mid] * n_kv <= off) lo = mid; else up = mid;
  }
  c.di = lo;
  c.np = s_qpos[lo] / kTok + 1;
  int rem = off - s_cum[lo] * n_kv;
  c.kvh = rem / c.np;
  c.pb = rem - c.kvh * c.np;
  c.pe = min(c.np, c.pb + (hi - off));
}

template <int NW, int NS, int MINB, int MAXD>
__global__ void __launch_bounds__(NW * 32, MINB)
decode_split_kernel(const __grid_constant__ CUtensorMap tmap, const DecodeParams P) {
  using L = DecodeSmem<NW, NS, MAXD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem + L::kQOff);
  float* s_mo = reinterpret_cast<float*>(smem + L::kMoOff);
  float* s_mm = reinterpret_cast<float*>(smem + L::kMmOff);
  float* s_ml = reinterpret_cast<float*>(smem + L::kMlOff);
  int* s_r = reinterpret_cast<int*>(smem + L::kROff);
  int* s_flat = reinterpret_cast<int*>(smem + L::kFlatOff);
  int* s_qpos = reinterpret_cast<int*>(smem + L::kQposOff);
  int* s_cum = reinterpret_cast<int*>(smem + L::kCumOff);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_decode = P.n_decode, n_kv = P.n_kv;

  if (tid == 0) {
    tma_prefetch_desc(&tmap);
    for (int i = 0; i < NW * NS; ++i) mbar_init(&bars[i], 1);
    mbar_fence_init();
  }
  // ---- per-sequence metadata (3 dependent loads) and the page prefix sum ----
  for (int di = tid; di < n_decode; di += NW * 32) {
    int r = P.rids[di];
    int flat = P.qstart[r];
    int qp = P.pos[flat];
    if (qp >= P.max_blocks * kTok) {
      report(FQB_ERR_INDEX, kKidDecode, qp);
      qp = P.max_blocks * kTok - 1;
    }
    if (qp < -1) qp = -1;
    s_r[di] = r;
    s_flat[di] = flat;
    s_qpos[di] = qp;
  }
  __syncthreads();
  if (warp == 0) {
    constexpr int kPer = MAXD / 32;
    int sum = 0;
    for (int i = 0; i < kPer; ++i) {
      int idx = lane * kPer + i;
      if (idx < n_decode) sum += (s_qpos[idx] + kTok) / kTok;  // qpos/16+1, 0 when qpos = -1
    }
    int incl = sum;
    for (int o = 1; o < 32; o <<= 1) {
      int y = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += y;
    }
    int run = incl - sum;
    for (int i = 0; i < kPer; ++i) {
      int idx = lane * kPer + i;
      if (idx < n_decode) {
        s_cum[idx] = run;
        run += (s_qpos[idx] + kTok) / kTok;
      }
    }
    int total = __shfl_sync(0xffffffffu, incl, 31);
    if (lane == 0) s_cum[n_decode] = total;
  }
  __syncthreads();

  const int total_slices = s_cum[n_decode] * n_kv;
  const int nb = static_cast<int>(gridDim.x);
  const int W = max(kMinSlicesPerCta, (total_slices + nb - 1) / nb);
  if (blockIdx.x == 0) {
    for (int di = tid; di < n_decode; di += NW * 32) {
      *meta_cum(P, di) = s_cum[di];
      *meta_np(P, di) = (s_qpos[di] + kTok) / kTok;
    }
    if (tid == 0) *meta_w(P) = W;
  }
  const long long lo_ll = static_cast<long long>(blockIdx.x) * W;
  if (lo_ll >= total_slices) return;  // whole CTA leaves together; nothing in flight
  const int lo = static_cast<int>(lo_ll);
  const int hi = min(total_slices, lo + W);

  uint8_t* my_stage = smem + warp * NS * kPageBytes;
  uint64_t* my_bar = bars + warp * NS;
  bool dead = false;  // a wait ran out: stop waiting, finish the control flow, status is set

  // ---- producer cursor: next page this warp will request ----
  ItemCursor pc;
  item_at(pc, lo, hi, n_decode, n_kv, s_cum, s_qpos);
  int p_page = pc.pb + warp;
  int p_blk = 0;
  int islot = 0;
  auto prod_settle = [&]() {  // move to the next item until this warp has a page in it
    while (pc.off < hi && p_page >= pc.pe) {
      item_at(pc, pc.off + (pc.pe - pc.pb), hi, n_decode, n_kv, s_cum, s_qpos);
      p_page = pc.pb + warp;
    }
    if (pc.off < hi)
      p_blk = __ldg(P.bt + static_cast<long long>(s_r[pc.di]) * P.max_blocks + p_page);
  };
  auto prod_issue = [&]() {
    if (pc.off >= hi) return;
    if (static_cast<unsigned>(p_blk) >= static_cast<unsigned>(P.num_blocks))
      report(FQB_ERR_INDEX, kKidDecode, p_blk);  // the load below then reads zeros
    if (lane == 0) {
      mbar_expect_tx(&my_bar[islot], kPageBytes);
      tma_load_page(my_stage + islot * kPageBytes, &tmap, &my_bar[islot], 0, 0, pc.kvh * 2, 0,
                    p_blk);
    }
    islot = (islot + 1 == NS) ? 0 : islot + 1;
    p_page += NW;
    prod_settle();
  };
  prod_settle();
#pragma unroll 1
  for (int s = 0; s < NS; ++s) prod_issue();

  // ---- consumer ----
  ItemCursor cc;
  item_at(cc, lo, hi, n_decode, n_kv, s_cum, s_qpos);
  int cslot = 0;
  uint32_t cphase = 0;
  int qbuf = 0;
  // q rows of the first item: 4 heads x 128 bf16 = 64 chunks of 16 bytes
  if (tid < 64)
    cp_async16(sQ + tid * 8, P.q + static_cast<long long>(s_flat[cc.di]) * P.q_stride +
                                 cc.kvh * (kGroup * kHd) + tid * 8);
  cp_async_commit();

  const int g = lane >> 2, t = lane & 3;
  const int mat = lane >> 3;
  const int k_tok = ((mat >> 1) << 3) + (lane & 7), k_sel = mat & 1;
  const int v_tok = ((mat & 1) << 3) + (lane & 7), v_sel = mat >> 1;

#pragma unroll 1
  while (cc.off < hi) {
    cp_async_wait_all();
    __syncthreads();  // q of this item visible; merge buffers of the previous item free
    ItemCursor nx;
    item_at(nx, cc.off + (cc.pe - cc.pb), hi, n_decode, n_kv, s_cum, s_qpos);
    if (nx.off < hi && tid < 64)
      cp_async16(sQ + (qbuf ^ 1) * (kGroup * kHd) + tid * 8,
                 P.q + static_cast<long long>(s_flat[nx.di]) * P.q_stride +
                     nx.kvh * (kGroup * kHd) + tid * 8);
    cp_async_commit();

    uint32_t qa[8][2];
    {
      const uint32_t* qw = reinterpret_cast<const uint32_t*>(sQ + qbuf * (kGroup * kHd));
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        qa[ks][0] = g < kGroup ? qw[(g * kHd + ks * 16 + 2 * t) >> 1] : 0u;
        qa[ks][1] = g < kGroup ? qw[(g * kHd + ks * 16 + 2 * t + 8) >> 1] : 0u;
      }
    }
    float o[16][4];
#pragma unroll
    for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float m = kNegBig, l = 0.f;
    const int qpos = s_qpos[cc.di];

#pragma unroll 1
    for (int page = cc.pb + warp; page < cc.pe; page += NW) {
      if (!dead && !mbar_wait_bounded(&my_bar[cslot], cphase)) {
        dead = true;
        report(FQB_ERR_TIMEOUT, kKidDecode, page);
      }
      uint8_t* st = my_stage + cslot * kPageBytes;
      const int nvalid = min(kTok, qpos - page * kTok + 1);
      if (nvalid < kTok) {
        // tail of the sequence's last page was never written: its V rows may hold anything
        if (lane < 16)
          for (int row = nvalid; row < kTok; ++row)
            *reinterpret_cast<uint4*>(st + kPlaneBytes + (lane >> 3) * kHalfBytes + row * 128 +
                                      ((lane & 7) << 4)) = make_uint4(0, 0, 0, 0);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
      }
      const uint32_t kbase = smem_u32(st), vbase = kbase + kPlaneBytes;
      float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(kbase + page_chunk_off(k_tok, ks * 2 + k_sel), b0, b1, b2, b3);
        mma_bf16(s0, qa[ks][0], 0u, qa[ks][1], 0u, b0, b1);
        mma_bf16(s1, qa[ks][0], 0u, qa[ks][1], 0u, b2, b3);
      }
      float x00 = s0[0] * P.scale_log2, x01 = s0[1] * P.scale_log2;
      float x10 = s1[0] * P.scale_log2, x11 = s1[1] * P.scale_log2;
      if (nvalid < kTok) {
        if (2 * t >= nvalid) x00 = kNegBig;
        if (2 * t + 1 >= nvalid) x01 = kNegBig;
        if (2 * t + 8 >= nvalid) x10 = kNegBig;
        if (2 * t + 9 >= nvalid) x11 = kNegBig;
      }
      float mx = fmaxf(fmaxf(x00, x01), fmaxf(x10, x11));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float mnew = fmaxf(m, mx);
      const float corr = fast_exp2(m - mnew);
      m = mnew;
      const float p00 = fast_exp2(x00 - mnew), p01 = fast_exp2(x01 - mnew);
      const float p10 = fast_exp2(x10 - mnew), p11 = fast_exp2(x11 - mnew);
      l = l * corr + ((p00 + p01) + (p10 + p11));
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        o[j][0] *= corr;
        o[j][1] *= corr;
      }
      const uint32_t pa0 = pack_bf16(p00, p01), pa2 = pack_bf16(p10, p11);
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_trans(vbase + page_chunk_off(v_tok, jj * 2 + v_sel), b0, b1, b2, b3);
        mma_bf16(o[2 * jj], pa0, 0u, pa2, 0u, b0, b1);
        mma_bf16(o[2 * jj + 1], pa0, 0u, pa2, 0u, b2, b3);
      }
      __syncwarp();  // every lane has read the buffer before it is refilled
      cslot = (cslot + 1 == NS) ? 0 : cslot + 1;
      if (cslot == 0) cphase ^= 1u;
      prod_issue();
    }

    // ---- merge the warps' partial softmax states of this item ----
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (g < kGroup) {
      float* dst = s_mo + (warp * kGroup + g) * kHd + 2 * t;
#pragma unroll
      for (int j = 0; j < 16; ++j)
        *reinterpret_cast<float2*>(dst + j * 8) = make_float2(o[j][0], o[j][1]);
      if (t == 0) {
        s_mm[warp * kGroup + g] = m;
        s_ml[warp * kGroup + g] = l;
      }
    }
    __syncthreads();
    if (tid < kGroup * 32) {
      const int h = tid >> 5, d4 = (tid & 31) * 4;
      float gm = kNegBig;
#pragma unroll
      for (int w = 0; w < NW; ++w) gm = fmaxf(gm, s_mm[w * kGroup + h]);
      float gl = 0.f;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        const float c = fast_exp2(s_mm[w * kGroup + h] - gm);
        gl += s_ml[w * kGroup + h] * c;
        const float4 v = *reinterpret_cast<const float4*>(s_mo + (w * kGroup + h) * kHd + d4);
        acc.x += v.x * c; acc.y += v.y * c; acc.z += v.z * c; acc.w += v.w * c;
      }
      const int head = cc.kvh * kGroup + h;
      if (cc.pb == 0 && cc.pe == cc.np) {
        const float inv = gl > 0.f ? 1.f / gl : 0.f;
        uint2 pk;
        pk.x = pack_bf16(acc.x * inv, acc.y * inv);
        pk.y = pack_bf16(acc.z * inv, acc.w * inv);
        *reinterpret_cast<uint2*>(P.out + (static_cast<long long>(s_flat[cc.di]) * P.n_heads + head) *
                                              kHd + d4) = pk;
      } else {
        const long long slot =
            (static_cast<long long>(cc.di) * n_kv + cc.kvh + blockIdx.x) * kGroup + h;
        if ((tid & 31) == 0) {
          P.pm[slot] = gm;
          P.pl[slot] = gl;
        }
        *reinterpret_cast<float4*>(P.pa + slot * kHd + d4) = acc;
      }
    }
    cc = nx;
    qbuf ^= 1;
  }
}

// One CTA per (sequence, kv head): merges the partials of a pair that was cut by CTA boundaries
// of the split kernel, writes zeros for a sequence without keys, and leaves pairs that the split
// kernel finished on its own untouched. 128 threads = 4 heads x 32 lanes x 4 dims.
__global__ void __launch_bounds__(128)
decode_combine_kernel(const DecodeParams P) {
  const int di = blockIdx.x / P.n_kv, kvh = blockIdx.x - di * P.n_kv;
  const int tid = threadIdx.x, h = tid >> 5, d4 = (tid & 31) * 4;
  const int W = *meta_w(P);
  const int cum = *meta_cum(P, di), np = *meta_np(P, di);
  const int head = kvh * kGroup + h;
  if (np <= 0) {
    const int flat = P.qstart[P.rids[di]];
    *reinterpret_cast<uint2*>(P.out + (static_cast<long long>(flat) * P.n_heads + head) * kHd + d4) =
        make_uint2(0u, 0u);
    return;
  }
  const int start = cum * P.n_kv + kvh * np;
  const int b0 = start / W, b1 = (start + np - 1) / W;
  if (b0 == b1) return;
  const long long pair = static_cast<long long>(di) * P.n_kv + kvh;
  float gm = kNegBig;
  for (int b = b0; b <= b1; ++b) gm = fmaxf(gm, P.pm[(pair + b) * kGroup + h]);
  float gl = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int b = b0; b <= b1; ++b) {
    const long long slot = (pair + b) * kGroup + h;
    const float c = fast_exp2(P.pm[slot] - gm);
    gl += P.pl[slot] * c;
    const float4 v = *reinterpret_cast<const float4*>(P.pa + slot * kHd + d4);
    acc.x += v.x * c; acc.y += v.y * c; acc.z += v.z * c; acc.w += v.w * c;
  }
  const float inv = gl > 0.f ? 1.f / gl : 0.f;
  const int flat = P.qstart[P.rids[di]];
  uint2 pk;
  pk.x = pack_bf16(acc.x * inv, acc.y * inv);
  pk.y = pack_bf16(acc.z * inv, acc.w * inv);
  *reinterpret_cast<uint2*>(P.out + (static_cast<long long>(flat) * P.n_heads + head) * kHd + d4) = pk;
}

}  // namespace fqb
