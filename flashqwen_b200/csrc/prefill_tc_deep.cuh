// Kernel 3, deep-pipeline form of the tcgen05 / TMEM prefill kernel.
//
// What clock-stamped timelines of the two-group kernels (prefill_tc_kernel, prefill_tc_ks_kernel) showed:
// per group, S for tile i+1 can only be issued once the PV MMA of tile i-1 has finished (P lives in the S
// buffer it came from and there are two buffers), so S, softmax and PV of a group run one after the other
// and two such chains per SM overlap only as far as they happen to be out of phase; and every mbarrier
// wait costs about 175 clocks even when the barrier completed long ago, which the thread that issues S
// pays twice per 64-key tile and group.
// Here a CTA is ONE 128-row tile (32 query rows x 4 q heads of a kv head) over 128-key tiles: the S issuer
// pays its waits once per 128 keys and its MMAs are M128 N128 (an N64 instruction holds the pipe as long
// as an N128 one), and tensor memory holds THREE S buffers (3 x 128 columns) beside O (128 columns), so S
// runs two tiles ahead of the softmax and never waits for it; measured in steady state, the S and PV
// issue windows then alternate without a gap (the tensor pipe is busy ~90 % of the time, at 110-125 clocks
// per MMA under load against 64 alone). K and V travel in separate rings of three
// 32 KiB slots ([2 blocks of 64 dims][128 keys][128 B], 128-byte swizzled as TMA writes it): a K slot is
// free again when its S MMA is done, a V slot when its PV MMA is done.
//
// Warps: 0-15 softmax, four threads per score row with 32 keys each (warps w, w + 4, w + 8, w + 12 address
// the same TMEM lanes and agree on the row maximum through 2-byte shared-memory slots and a 128-thread
// named barrier; two threads per row measured the same, and taking the exp2, the bf16 pack or the row sums
// out altogether does not change the run time: in this kernel the softmax is not what the others wait for),
// 16 K producer, 17 V producer, 18 S issuer (+ TMEM alloc), 19 PV issuer.
// The building blocks (descriptors, TMEM access, barriers) are those of prefill_tc.cuh.
#pragma once

#include "prefill_tc.cuh"

namespace fqb {

struct TcDeepSmem {
  static constexpr int kTile = 128;                             // keys per tile
  static constexpr int kSlots = 3;                              // K slots, V slots and S buffers
  static constexpr int kQ = 0;                                  // [2 k-blocks][128 rows][128 B]
  static constexpr int kK = 32768;                              // kSlots x 32 KiB
  static constexpr int kSlot = 32768;
  static constexpr int kV = kK + kSlots * kSlot;
  static constexpr int kBars = kV + kSlots * kSlot;
  static constexpr int kTmemSlot = kBars + 32 * 8;
  static constexpr int kXch = kTmemSlot + 16;                   // [tile parity][key quarter][128 rows] bf16 row maxima
  static constexpr int kTotal = kXch + 2 * 4 * 128 * 2;
  static constexpr int kAlloc = kTotal;                         // base must be 1024-byte aligned (checked)
  static constexpr int kThreads = 20 * 32;
  static constexpr int kOCol = kSlots * kTile;                  // O accumulator behind the S buffers
};

__global__ void __launch_bounds__(TcDeepSmem::kThreads, 1)
prefill_tc_deep_kernel(const __grid_constant__ CUtensorMap tmap, const PrefillParams P) {
  using L = TcDeepSmem;
  static_assert(L::kTotal <= 232448, "227 KiB of shared memory per CTA");
  static_assert(L::kOCol + kHd <= 512, "S buffers and O fit tensor memory");
  constexpr int kCols = 512;
  constexpr int kT = L::kTile, kN = L::kSlots;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) report(FQB_ERR_INVALID, kKidPrefill, static_cast<int>(smem_u32(smem)));
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
  auto k_full = [&](int s) { return bars + s; };
  auto k_empty = [&](int s) { return bars + 3 + s; };
  auto v_full = [&](int s) { return bars + 6 + s; };
  auto v_empty = [&](int s) { return bars + 9 + s; };
  auto s_full = [&](int b) { return bars + 12 + b; };
  auto p_full = [&](int b) { return bars + 15 + b; };
  auto o_done = [&](int b) { return bars + 18 + b; };
  uint64_t* q_full = bars + 21;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kTmemSlot);

  // Longest request first; the ranking loads also bring this query tile's metadata (see prefill_tc_ks_kernel).
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

  if (warp == 18) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "n"(kCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    tma_prefetch_desc(&tmap);
    for (int s = 0; s < kN; ++s) {
      mbar_init(k_full(s), 1);
      mbar_init(k_empty(s), 1);
      mbar_init(v_full(s), 1);
      mbar_init(v_empty(s), 1);
      mbar_init(s_full(s), 1);
      mbar_init(p_full(s), 16);
      mbar_init(o_done(s), 1);
    }
    mbar_init(q_full, 16);
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
  const int ntiles = last_pos < 0 ? 0 : last_pos / kT + 1;
  bool dead = false;
  auto wait = [&](uint64_t* bar, uint32_t parity, int what) {
    if (!dead && !mbar_wait_bounded(bar, parity)) {
      dead = true;
      report(FQB_ERR_TIMEOUT, kKidPrefill, what);
    }
  };

  if (warp < 16) {
    // ============ softmax warps: four threads per MMA row (32 keys of the tile each) ============
    const int q4 = warp & 3;   // TMEM lane quarter = q head
    const int ch = warp >> 2;  // which 32 keys of each 128-key tile
    const int row = q4 * 32 + lane;
    const int g = q4, qi = lane;
    const int qrow = q0 + qi;
    const bool valid = qrow < ql;
    const int row_bar = 2 + q4;  // named barrier of this row's four warps
    {
      const uint4* src = reinterpret_cast<const uint4*>(
          P.q + static_cast<long long>(qs + (valid ? qrow : q0)) * P.q_stride + (kvh * kGroup + g) * kHd);
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        const int c = ch * 4 + cc;
        const uint4 v = valid ? __ldg(src + c) : make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(smem + L::kQ + (c >> 3) * 16384 + row * 128 + (((c & 7) ^ (row & 7)) << 4)) = v;
      }
      proxy_fence_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(q_full);
    }
    const int qp = valid ? P.pos[qs + qrow] : -1;
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(q4 * 32) << 16);
    __nv_bfloat16* xch = reinterpret_cast<__nv_bfloat16*>(smem + L::kXch);  // [parity][ch][128]
    float m_used = kNegBig, l = 0.f;

#pragma unroll 1
    for (int i = 0; i < ntiles; ++i) {
      const int b = i % kN;
      wait(s_full(b), (i / kN) & 1, i);
      tc_fence_after();
      float x[32];
      tmem_ld16(lane_addr + b * kT + ch * 32, x);
      tmem_ld16(lane_addr + b * kT + ch * 32 + 16, x + 16);
      tmem_wait_ld();
      const int k0 = i * kT + ch * 32;
      if (k0 + 31 > qp) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (k0 + j > qp) x[j] = kNegBig;
      }
      float mx0 = kNegBig, mx1 = kNegBig, mx2 = kNegBig, mx3 = kNegBig;
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        mx0 = fmaxf(mx0, x[j]);
        mx1 = fmaxf(mx1, x[j + 1]);
        mx2 = fmaxf(mx2, x[j + 2]);
        mx3 = fmaxf(mx3, x[j + 3]);
      }
      // The row's four threads agree on one maximum: each publishes its own rounded UP to bf16 (so the
      // agreed value is never below the true maximum and exp2 cannot overflow; the maximum is only a
      // scaling reference) and all take the largest. Slots alternate with the tile parity, so one
      // barrier per tile is enough.
      const __nv_bfloat16 mine = __float2bfloat16_ru(fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * P.scale_log2);
      __nv_bfloat16* slots = xch + (i & 1) * 512 + row;
      slots[ch * 128] = mine;
      asm volatile("bar.sync %0, 128;" ::"r"(row_bar) : "memory");
      const float mx = fmaxf(fmaxf(__bfloat162float(slots[0]), __bfloat162float(slots[128])),
                             fmaxf(__bfloat162float(slots[256]), __bfloat162float(slots[384])));
      const float m_new = fmaxf(m_used, mx);
      const bool grow = m_new > m_used + 8.f;
      const float f = grow ? fast_exp2(m_used - m_new) : 1.f;
      if (grow) {
        m_used = m_new;
        l *= f;
      }
      const bool any_grow = i > 0 && __any_sync(0xffffffffu, grow);
      if (any_grow) {  // PV of the tile before must be done before O is rescaled; none later is issued yet
        wait(o_done((i - 1) % kN), ((i - 1) / kN) & 1, 1000 + i);
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {  // this thread's 32 of the 128 dims
          float o[16];
          tmem_ld16(lane_addr + L::kOCol + ch * 32 + c * 16, o);
          tmem_wait_ld();
#pragma unroll
          for (int q = 0; q < 16; ++q) o[q] *= f;
          tmem_st16(lane_addr + L::kOCol + ch * 32 + c * 16, o);
        }
      }
      // P over the first 64 columns of S[b] (column c = keys 2c and 2c+1); all four threads of the row have
      // their scores in registers by now (the barrier above came after the loads)
      float sm0 = 0.f, sm1 = 0.f, sm2 = 0.f, sm3 = 0.f;
      const float neg_m = -m_used;
      float pf[16];
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        const float p0 = fast_exp2(fmaf(x[j], P.scale_log2, neg_m));
        const float p1 = fast_exp2(fmaf(x[j + 1], P.scale_log2, neg_m));
        const float p2 = fast_exp2(fmaf(x[j + 2], P.scale_log2, neg_m));
        const float p3 = fast_exp2(fmaf(x[j + 3], P.scale_log2, neg_m));
        sm0 += p0; sm1 += p1; sm2 += p2; sm3 += p3;
        pf[j >> 1] = __uint_as_float(pack_bf16(p0, p1));
        pf[(j >> 1) + 1] = __uint_as_float(pack_bf16(p2, p3));
      }
      tmem_st16(lane_addr + b * kT + ch * 16, pf);
      l += (sm0 + sm1) + (sm2 + sm3);
      tmem_wait_st();
      if (i == ntiles - 1) {  // key slots past the last position: clear their V rows (0 * garbage)
        const int nvalid = last_pos - i * kT + 1;
        wait(v_full(i % kN), (i / kN) & 1, 1500 + i);
        uint8_t* vst = smem + L::kV + (i % kN) * L::kSlot;
        for (int idx = row + ch * 128; idx < (kT - nvalid) * 16; idx += 512) {
          const int vr = nvalid + (idx >> 4), c = idx & 15;
          *reinterpret_cast<uint4*>(vst + (c >> 3) * 16384 + vr * 128 + ((c & 7) << 4)) = make_uint4(0, 0, 0, 0);
        }
        proxy_fence_async();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full(b));
    }
    if (ntiles > 0) {
      wait(o_done((ntiles - 1) % kN), ((ntiles - 1) / kN) & 1, 2000);
      tc_fence_after();
    }
    // the row sum is the sum of its four threads' sums (over the finished maximum slots)
    float* lsum = reinterpret_cast<float*>(smem + L::kXch);  // [ch][128]
    lsum[ch * 128 + row] = l;
    asm volatile("bar.sync %0, 128;" ::"r"(row_bar) : "memory");
    const float lt = (lsum[row] + lsum[128 + row]) + (lsum[256 + row] + lsum[384 + row]);
    const float inv = lt > 0.f ? 1.f / lt : 0.f;
    __nv_bfloat16* orow = P.out + (static_cast<long long>(qs + qrow) * P.n_heads + kvh * kGroup + g) * kHd + ch * 32;
#pragma unroll 1
    for (int c = 0; c < 2; ++c) {
      float o[16];
      if (ntiles > 0) {
        tmem_ld16(lane_addr + L::kOCol + ch * 32 + c * 16, o);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int q = 0; q < 16; ++q) o[q] = 0.f;
      }
      if (valid) {
        uint4 a, bq;
        a.x = pack_bf16(o[0] * inv, o[1] * inv);     a.y = pack_bf16(o[2] * inv, o[3] * inv);
        a.z = pack_bf16(o[4] * inv, o[5] * inv);     a.w = pack_bf16(o[6] * inv, o[7] * inv);
        bq.x = pack_bf16(o[8] * inv, o[9] * inv);    bq.y = pack_bf16(o[10] * inv, o[11] * inv);
        bq.z = pack_bf16(o[12] * inv, o[13] * inv);  bq.w = pack_bf16(o[14] * inv, o[15] * inv);
        *reinterpret_cast<uint4*>(orow + c * 16) = a;
        *reinterpret_cast<uint4*>(orow + c * 16 + 8) = bq;
      }
    }
    tc_fence_before();
  } else if (warp < 18) {
    // ============ TMA producers: warp 16 fills the K slots, warp 17 the V slots ============
    const int plane = warp - 16;
    const int* btr = P.bt + static_cast<long long>(r) * P.max_blocks;
#pragma unroll 1
    for (int i = 0; i < ntiles; ++i) {
      const int slot = i % kN;
      const int pg0 = i * 8;
      const int npg = min(8, npages - pg0);
      const int mine = lane < npg ? __ldg(btr + pg0 + lane) : 0;
      if (i >= kN) wait(plane == 0 ? k_empty(slot) : v_empty(slot), ((i / kN) - 1) & 1, 3000 + i);
      if (lane < npg && static_cast<unsigned>(mine) >= static_cast<unsigned>(P.num_blocks))
        report(FQB_ERR_INDEX, kKidPrefill, mine);
      uint8_t* st = smem + (plane == 0 ? L::kK : L::kV) + slot * L::kSlot;
      uint64_t* full = plane == 0 ? k_full(slot) : v_full(slot);
      if (lane == 0) mbar_expect_tx(full, static_cast<uint32_t>(npg) * kPlaneBytes);
      __syncwarp();
      if (lane < npg) {
#pragma unroll
        for (int half = 0; half < 2; ++half)
          tma_load_half(st + half * 16384 + lane * 2048, &tmap, full, kvh * 2 + half, plane, mine);
      }
    }
  } else if (warp == 18) {
    // ============ S = Q K^T issuer: up to two tiles ahead of the softmax ============
    if (lane == 0) {
      constexpr uint32_t kIdescS = umma_idesc(128, kT, false);
      const uint64_t qd = umma_desc(smem_u32(smem + L::kQ), 16, 1024);
      wait(q_full, 0, 4000);
      tc_fence_after();
#pragma unroll 1
      for (int i = 0; i < ntiles; ++i) {
        const int b = i % kN;
        wait(k_full(b), (i / kN) & 1, 5000 + i);
        if (i >= kN) wait(o_done(b), ((i / kN) - 1) & 1, 6000 + i);  // PV of tile i - 3 has read P out of S[b]
        tc_fence_after();
        const uint64_t kd = umma_desc(smem_u32(smem + L::kK + b * L::kSlot), 16, 1024);
        const uint32_t d = tmem + b * kT;
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int j = 0; j < 4; ++j)
            umma_bf16(d, qd + ((kb * 16384 + j * 32) >> 4), kd + ((kb * 16384 + j * 32) >> 4), kIdescS,
                      (kb | j) ? 1u : 0u);
        umma_commit(s_full(b));
        umma_commit(k_empty(b));
      }
    }
    tc_fence_before();
  } else {
    // ============ O += P V issuer ============
    if (lane == 0) {
      constexpr uint32_t kIdescO = umma_idesc(128, kHd, true);
#pragma unroll 1
      for (int i = 0; i < ntiles; ++i) {
        const int b = i % kN;
        wait(p_full(b), (i / kN) & 1, 7000 + i);
        wait(v_full(b), (i / kN) & 1, 8000 + i);
        tc_fence_after();
        const uint64_t vd = umma_desc(smem_u32(smem + L::kV + b * L::kSlot), 16384, 1024);
        const uint32_t d = tmem + L::kOCol;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          umma_bf16_ts(d, tmem + b * kT + j * 8, vd + ((j * 2048) >> 4), kIdescO, (i | j) ? 1u : 0u);
        umma_commit(o_done(b));
        umma_commit(v_empty(b));
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 18) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(kCols) : "memory");
  }
}

}  // namespace fqb
