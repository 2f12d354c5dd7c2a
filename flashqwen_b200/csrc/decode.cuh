// Kernel 2: GQA-shared split-K paged decode attention with the log-sum-exp combine fused in, and
// optionally the KV append of the step's new token fused in as well.
//
// Operator semantics follow the reference's LaunchAttnDecodeCute
// (engine/src/attn_cute.cu:165-261 of the FlashQwen tree): decode sequence di attends keys
// 0..qpos inclusive, one kv head serves its 4 query heads, fp32 accumulation, bf16 output at
// out[(flat*n_heads + h)*128 + d]. The design is not the reference's:
//
//   * Work is the flat list of pages of all sequences (sequence-major). It is cut into contiguous
//     SEGMENTS of equal cost (a page counts 1, a sequence end inside the segment a few pages), one
//     per (CTA, warp group) of a persistent grid, on the device from the actual context lengths --
//     the grid depends only on the SM count, so the launch can sit in a CUDA graph while lengths
//     change. Warp w serves kv head w % HEADS of segment
//     blockIdx.x * SUB + w / HEADS: with all local heads in one CTA (HEADS == NW) the loads a CTA has
//     in flight cover whole 64 KiB pages (all heads of K and V are adjacent in memory); with one or
//     two local heads the SUB warps that share a head take neighbouring segments.
//   * Each warp owns a private ring of NS page buffers (8 KiB: K and V rows of one head of one
//     16-token page) filled by single-thread TMA tensor loads (5-D box, 128-byte swizzle) that
//     complete on the ring's mbarriers. The warp that consumes a buffer refills it, so the stream
//     has no cross-warp handshake and no block barrier at all, and runs ahead across sequence
//     boundaries.
//   * Scores and PV products use mma.sync m16n8k16 with the 4 query heads as rows 0..3 of the
//     16-row A tile (rows 4..15 are zero padding): S[4x16] = Q[4x128] K^T, O[4x128] += P[4x16] V.
//     The query rows of the next sequence are fetched into registers while the current one runs.
//   * A (sequence, head) pair that lies inside one segment is normalised and written straight to
//     `out`. A pair cut by segment boundaries leaves one unnormalised partial per segment and takes a
//     ticket on the pair's arrival counter; the warp that takes the last ticket merges the
//     partials (log-sum-exp) and writes `out` -- no second kernel, no inter-CTA waiting.
//   * Fused append (the step's new token, engine/src/kv_store.cu:48-75): exactly one warp per
//     (sequence, head) streams the sequence's last page; it copies the new K and V rows from the
//     fused qkv row into the cache and into the page buffer it has just received, so the token takes
//     part in the attention without a separate append kernel in front.
#pragma once

#include <cuda_fp8.h>

#include "common.cuh"

namespace fqb {

constexpr int kMaxPeers = 8;
constexpr int kMaxPending = 8;  // cut sequences a warp may leave behind before it settles them (<= 32)

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
  unsigned epoch;  // differs from launch to launch, never 0
  int kvh_base;    // first kv head this launch serves (launches cover 8, 4, 2 or 1 heads each)
  int mode;        // kDecodeWaitFirst / kDecodeNoWait / kDecodeWaitRows, see below
  int sync_first;  // 1: wait for every earlier kernel BEFORE letting the next launch start
  int end_weight;  // what a sequence end inside a segment is charged, in pages, when the page list is cut
  int groups;      // head groups of the launch: CTA b serves heads kvh_base + (b % groups) * HEADS ... of segment b / groups
  const int* plan; // optional step plan {r, flat, qpos, page prefix}[n_decode] + total (decode_plan_kernel)
  const float* scales;  // fp8 cache only: [num_blocks][n_kv][2 planes][16 tokens] fp32
  float* scales_w;      // fp8 cache with the fused append: the same array, written for the step's token
  // fused append of the new token (cache_w == nullptr: none). The rows are qkv + flat * q_stride
  // seen from q: K of cache head kvh at q + k_rel + kvh*128, V at q + v_rel + kvh*128.
  __nv_bfloat16* cache_w;
  long long k_rel, v_rel;
  // Reassembly over G GPUs (n_peers == 0: none). A finished row also goes to every rank's buffer
  // peer_out[r] of full rows [rows][peer_heads][128] at head column peer_col + (local head); plain
  // stores, the pointers may be peer memory. When the last warp of the launch has arrived on `arrive`
  // it bumps this rank's publish counter seq and stores the new value into every rank's flag word
  // peer_flag[r] (release, system scope): "rank `rank` has delivered publish number v of this slot".
  int n_peers;
  __nv_bfloat16* peer_out[kMaxPeers];
  unsigned* peer_flag[kMaxPeers];
  int peer_heads, peer_col;
  unsigned* seq;
  unsigned long long* arrive;
};

// What a launch waits for before it touches anything but the step metadata:
//   kDecodeWaitFirst  the kernel launched before it has completed (always safe);
//   kDecodeNoWait     nothing: that kernel writes nothing this launch reads (the wait moves to the very
//                     end, where it only keeps kernels completing in order);
//   kDecodeWaitRows   the page ring is filled first -- that kernel writes none of the cached keys
//                     0..qpos-1 -- and only then the launch waits, before it reads the q / K / V rows of
//                     the step, which that kernel may have produced.
enum { kDecodeWaitFirst = 0, kDecodeNoWait = 1, kDecodeWaitRows = 2 };

// Scratch layout. Partial (sequence di, segment b, kv head, q head g) lives at slot
// ((di + b) * n_kv + kvh) * 4 + g of pm / pl / pa: along the flat page list the cuts are sequence
// boundaries and segment boundaries, so di + b numbers the pieces uniquely. The arrival counters
// (one 64-bit word per (sequence, kv head)) sit at the end of pl.
__host__ __device__ inline long long decode_counter_base(long long partial_slots, int n_pairs) {
  return (partial_slots - 2LL * n_pairs) & ~1LL;  // float index into pl, 8-byte aligned
}
__host__ __device__ inline long long decode_slots_needed(int n_decode, int n_kv, int segments) {
  return (static_cast<long long>(n_decode) + segments) * n_kv * kGroup + 2LL * n_decode * n_kv + 2;
}

// Takes a ticket on an arrival counter {epoch : 32 | count : 32}. A word whose epoch field is not
// this launch's (stale or never initialised memory) counts as empty, so the scratch needs no
// clearing; the caller that gets the last ticket clears the word for a replay with the same epoch.
__device__ __forceinline__ bool take_ticket_is_last(unsigned long long* c, unsigned epoch, int total) {
  unsigned long long seen = *reinterpret_cast<volatile unsigned long long*>(c);
  unsigned cnt = 0;
  for (int tries = 0; tries < 4096; ++tries) {
    cnt = (static_cast<unsigned>(seen >> 32) == epoch) ? static_cast<unsigned>(seen) + 1u : 1u;
    const unsigned long long want = (static_cast<unsigned long long>(epoch) << 32) | cnt;
    const unsigned long long old = atomicCAS(c, seen, want);
    if (old == seen) return cnt == static_cast<unsigned>(total);
    seen = old;
  }
  report(FQB_ERR_TIMEOUT, kKidCombine, total);
  return false;
}

// One page slice of the fp8 cache: [2 planes][16 tokens][128 e4m3 bytes] + its 32 scales.
constexpr int kPageBytes8 = 2 * kTok * kHd;  // 4096
constexpr int kScaleBytes8 = 2 * kTok * 4;   // 128
constexpr float kPScale8 = 256.f;            // P is scaled up before it is rounded to f16 (fp8 path)

template <int NW, int NS, int MAXD, bool FP8 = false>
struct DecodeSmem {
  static constexpr int kSlice = FP8 ? kPageBytes8 : kPageBytes;
  static constexpr int kStageBytes = NW * NS * kSlice;
  static constexpr int kScaleOff = kStageBytes;                      // fp8: NW * NS x 128 bytes of scales
  static constexpr int kBarOff = kScaleOff + (FP8 ? NW * NS * kScaleBytes8 : 0);
  static constexpr int kROff = kBarOff + NW * NS * 8;
  static constexpr int kFlatOff = kROff + MAXD * 4;
  static constexpr int kQposOff = kFlatOff + MAXD * 4;
  static constexpr int kCumOff = kQposOff + MAXD * 4;
  static constexpr int kArriveOff = kCumOff + (MAXD + 1) * 4;  // warps of this CTA that are through (reassembly)
  static constexpr int kPendOff = kArriveOff + 4;              // per warp: cut sequences whose ticket is still to be taken
  static constexpr int kTotal = kPendOff + NW * kMaxPending * 4;
  static constexpr int kAlloc = kTotal + 1024;  // slack for manual 1024-byte alignment
};

// An item is a maximal run of pages of one sequence inside a segment.
struct ItemCursor {
  int off;     // flat page offset of the item's first page; >= hi when exhausted
  int di;
  int pb, pe;  // page range [pb, pe) inside the sequence
  int np;      // pages of the whole sequence
};

__device__ __forceinline__ void item_at(ItemCursor& c, int off, int hi, int n_decode, const int* s_cum) {
  c.off = off;
  if (off >= hi) return;
  int lo = 0, up = n_decode;  // largest di with s_cum[di] <= off (s_cum[n_decode] = total > off)
  while (up - lo > 1) {
    const int mid = (lo + up) >> 1;
    if (s_cum[mid] <= off) lo = mid; else up = mid;
  }
  c.di = lo;
  c.np = s_cum[lo + 1] - s_cum[lo];
  c.pb = off - s_cum[lo];
  c.pe = min(c.np, c.pb + (hi - off));
}

// Merges the partials of pair (di, kvh) left by segments b0..b1 and writes the 4 query heads' rows.
// One warp: lane -> q head g = lane / 8 and dims (lane % 8) * 4 + 32 * i, i < 4. The partials are
// fetched four segments at a time, all loads of a batch in flight together: a sequence cut over many
// segments would otherwise pay one L2 round trip per segment.
__device__ __forceinline__ void merge_pair(const DecodeParams& P, int di, int kvh, int b0, int b1, int flat,
                                           int lane) {
  const int g = lane >> 3, sub8 = lane & 7, dbase = sub8 * 4;
  const long long stride = static_cast<long long>(P.n_kv) * kGroup;  // slots from one segment to the next
  const long long slot_b0 = ((static_cast<long long>(di) + b0) * P.n_kv + kvh) * kGroup + g;
  const int n = b1 - b0 + 1;
  float gm = kNegBig;
  for (int i = sub8; i < n; i += 8) gm = fmaxf(gm, __ldcg(P.pm + slot_b0 + i * stride));
  gm = fmaxf(gm, __shfl_xor_sync(0xffffffffu, gm, 1));
  gm = fmaxf(gm, __shfl_xor_sync(0xffffffffu, gm, 2));
  gm = fmaxf(gm, __shfl_xor_sync(0xffffffffu, gm, 4));
  float gl = 0.f;
  float4 acc[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int i0 = 0; i0 < n; i0 += 4) {
    float pm4[4], pl4[4];
    float4 v[4][4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long slot = slot_b0 + min(i0 + u, n - 1) * stride;  // past the end: reload the last one, weight 0
      pm4[u] = __ldcg(P.pm + slot);
      pl4[u] = __ldcg(P.pl + slot);
#pragma unroll
      for (int i = 0; i < 4; ++i) v[u][i] = __ldcg(reinterpret_cast<const float4*>(P.pa + slot * kHd + dbase + 32 * i));
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float c = i0 + u < n ? fast_exp2(pm4[u] - gm) : 0.f;
      gl += pl4[u] * c;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[i].x += v[u][i].x * c; acc[i].y += v[u][i].y * c; acc[i].z += v[u][i].z * c; acc[i].w += v[u][i].w * c;
      }
    }
  }
  const float inv = gl > 0.f ? 1.f / gl : 0.f;
  uint2 pk[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    pk[i].x = pack_bf16(acc[i].x * inv, acc[i].y * inv);
    pk[i].y = pack_bf16(acc[i].z * inv, acc[i].w * inv);
  }
  __nv_bfloat16* o = P.out + (static_cast<long long>(flat) * P.n_heads + kvh * kGroup + g) * kHd + dbase;
#pragma unroll
  for (int i = 0; i < 4; ++i) *reinterpret_cast<uint2*>(o + 32 * i) = pk[i];
  for (int r = 0; r < P.n_peers; ++r) {
    __nv_bfloat16* po =
        P.peer_out[r] + (static_cast<long long>(flat) * P.peer_heads + P.peer_col + kvh * kGroup + g) * kHd + dbase;
#pragma unroll
    for (int i = 0; i < 4; ++i) *reinterpret_cast<uint2*>(po + 32 * i) = pk[i];
  }
}

// Step plan: what every decode launch of a step derives from pos / qstart / decode_rids, computed
// once. plan[4*di .. 4*di+3] = {request r, flat row, last key position (clamped, -1 = no key), first
// page index in the flat page list}; plan[4*n] = total pages. One CTA, up to 1024 sequences.
__global__ void __launch_bounds__(1024)
decode_plan_kernel(const int* __restrict__ pos, const int* __restrict__ qstart, const int* __restrict__ rids,
                   int n_decode, int max_blocks, int* __restrict__ plan) {
  __shared__ int s_pages[1024];
  __shared__ int s_warp[32];
  const int di = threadIdx.x, lane = di & 31, warp = di >> 5;
  int r = 0, flat = 0, qp = -1;
  if (di < n_decode) {
    r = rids[di];
    flat = qstart[r];
    qp = pos[flat];
    if (qp >= max_blocks * kTok) {
      report(FQB_ERR_INDEX, kKidDecode, qp);
      qp = max_blocks * kTok - 1;
    }
    if (qp < 0) qp = -1;
  }
  const int pages = di < n_decode ? (qp + kTok) / kTok : 0;
  int incl = pages;
  for (int o = 1; o < 32; o <<= 1) {
    const int y = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += y;
  }
  if (lane == 31) s_warp[warp] = incl;
  s_pages[di] = incl - pages;
  __syncthreads();
  if (warp == 0) {
    int w = s_warp[lane];
    int wi = w;
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += y;
    }
    s_warp[lane] = wi - w;
    if (lane == 31) plan[4 * n_decode] = wi;
  }
  __syncthreads();
  if (di < n_decode)
    reinterpret_cast<int4*>(plan)[di] = make_int4(r, flat, qp, s_pages[di] + s_warp[warp]);
}

// Reassembly, consumer side: returns once every rank has delivered publish number seq[0] of the slot,
// i.e. flags[r] >= this rank's own publish count (all ranks make the same calls in the same order, and
// this kernel follows this rank's own publishing launch on the stream). One warp, lane r polls rank r's
// word in LOCAL memory. The wait is bounded by time: past the limit it records FQB_ERR_TIMEOUT and returns.
__global__ void __launch_bounds__(32)
gather_wait_kernel(const unsigned* __restrict__ flags, const unsigned* __restrict__ seq, int world,
                   unsigned long long limit_ns) {
  pdl_launch_dependents();
  pdl_wait();  // the publishing launch of this rank has completed: seq holds its number
  const int lane = threadIdx.x;
  if (lane >= world) return;
  const unsigned want = *reinterpret_cast<const volatile unsigned*>(seq);
  unsigned long long t0;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
  for (;;) {
    unsigned have;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(have) : "l"(flags + lane) : "memory");
    if (static_cast<int>(have - want) >= 0) return;
    unsigned long long now;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
    if (now - t0 > limit_ns) {
      report(FQB_ERR_TIMEOUT, kKidGather, lane);
      return;
    }
    __nanosleep(200);
  }
}

// The same for every slot of the control block, one after the other (at the end of a step).
__global__ void __launch_bounds__(32)
gather_wait_all_kernel(const unsigned* __restrict__ flags, const unsigned* __restrict__ seq, int slots, int world,
                       unsigned long long limit_ns) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x;
  if (lane >= world) return;
  unsigned long long t0;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
  for (int s = 0; s < slots; ++s) {
    const unsigned want = *reinterpret_cast<const volatile unsigned*>(seq + s);
    for (;;) {
      unsigned have;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(have) : "l"(flags + s * world + lane) : "memory");
      if (static_cast<int>(have - want) >= 0) break;
      unsigned long long now;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
      if (now - t0 > limit_ns) {
        report(FQB_ERR_TIMEOUT, kKidGather, s * 16 + lane);
        return;
      }
      __nanosleep(200);
    }
  }
}

// Publishes every slot of the control block at once: launched without overlap after the last kernel that
// stored rows into the peers' buffers, so those stores have been performed. One thread per slot bumps the
// slot's counter; one thread per (slot, rank) stores it into that rank's flag word for this rank.
struct PublishAllParams {
  unsigned* seq;               // this rank's publish counters [slots]
  unsigned* flags[kMaxPeers];  // every rank's flag words [slots][world]
  int slots, world, rank;
};
__global__ void __launch_bounds__(256)
gather_publish_all_kernel(const PublishAllParams P) {
  __shared__ unsigned s_seq[256];
  const int tid = threadIdx.x;
  for (int base = 0; base < P.slots; base += 256) {
    const int n = min(256, P.slots - base);
    if (tid < n) s_seq[tid] = atomicAdd(P.seq + base + tid, 1u) + 1u;
    __threadfence_system();
    __syncthreads();
    for (int i = tid; i < n * P.world; i += 256) {
      const int s = i / P.world, r = i - s * P.world;
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(P.flags[r] + static_cast<size_t>(base + s) * P.world + P.rank),
                   "r"(s_seq[s])
                   : "memory");
    }
    __syncthreads();
  }
}

// HEADS = local kv heads served by the launch (1, 2, 4 or 8); the CTA's NW warps form SUB = NW / HEADS
// groups of HEADS warps, and group `sub` of CTA b owns segment b * SUB + sub of the flat page list.
// FP8: the cache holds e4m3 bytes with one fp32 scale per (token, head, plane). A page slice is 4 KiB
// (+ 128 bytes of scales, a second copy on the same barrier). K and V are widened to f16 in registers
// (exact) and the products run as f16 MMAs; the K scale multiplies the score column, the V scale the
// probability, so no element is ever multiplied by its scale one at a time. The contraction over the
// 128 dims and the order of the output dims are permuted so that every lane fetches 16 contiguous
// bytes: lane (g, t) reads dims [32t, 32t+32) of its two key tokens for Q K^T, and dims [16g, 16g+16) of
// its four value tokens for P V, whose accumulator columns then hold dims 32t+j and 32t+16+j.
template <int NW, int NS, int HEADS, int MINB, int MAXD, bool FP8 = false, bool APPEND = true>
__global__ void __launch_bounds__(NW * 32, MINB)
decode_kernel(const __grid_constant__ CUtensorMap tmap, const DecodeParams P) {
  using L = DecodeSmem<NW, NS, MAXD, FP8>;
  constexpr int kSlice = L::kSlice;
  constexpr int SUB = NW / HEADS;
  static_assert(NW % HEADS == 0, "warps must divide evenly over the heads");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  int* s_r = reinterpret_cast<int*>(smem + L::kROff);
  int* s_flat = reinterpret_cast<int*>(smem + L::kFlatOff);
  int* s_qpos = reinterpret_cast<int*>(smem + L::kQposOff);
  int* s_cum = reinterpret_cast<int*>(smem + L::kCumOff);
  unsigned* s_arrive = reinterpret_cast<unsigned*>(smem + L::kArriveOff);
  int* s_pend = reinterpret_cast<int*>(smem + L::kPendOff) + (threadIdx.x >> 5) * kMaxPending;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_decode = P.n_decode;
  // A launch may cover groups * HEADS heads with CTAs of HEADS heads each (CTA b: group b % groups, CTA
  // index b / groups within the group), which puts more, smaller CTAs on an SM than one CTA for all heads.
  const int cta = static_cast<int>(blockIdx.x) / P.groups;
  const int kvh = P.kvh_base + (static_cast<int>(blockIdx.x) % P.groups) * HEADS + warp % HEADS, sub = warp / HEADS;

  // The next kernel on the stream may start its own prologue now. This kernel's prologue reads
  // only the step metadata (rids, qstart, pos, bt), which the kernel before it never writes.
  if (!P.sync_first) pdl_launch_dependents();
  if (tid == 0) {
    tma_prefetch_desc(&tmap);
    for (int i = 0; i < NW * NS; ++i) mbar_init(&bars[i], 1);
    mbar_fence_init();
    *s_arrive = 0u;
  }
  // ---- per-sequence metadata and the page prefix sum ----
  // With a step plan (built once per step, the same for all layers) this is one coalesced load;
  // without it, three dependent loads per sequence and a scan.
  const bool planned = P.plan != nullptr;
  if (planned) {
    for (int di = tid; di < n_decode; di += NW * 32) {
      const int4 e = __ldg(reinterpret_cast<const int4*>(P.plan) + di);
      s_r[di] = e.x;
      s_flat[di] = e.y;
      s_qpos[di] = e.z;
      s_cum[di] = e.w;
    }
    if (tid == 0) s_cum[n_decode] = __ldg(P.plan + 4 * n_decode);
  } else
  for (int di = tid; di < n_decode; di += NW * 32) {
    const int r = P.rids[di];
    const int flat = P.qstart[r];
    int qp = P.pos[flat];
    if (qp >= P.max_blocks * kTok) {
      report(FQB_ERR_INDEX, kKidDecode, qp);
      qp = P.max_blocks * kTok - 1;
    }
    if (qp < 0) qp = -1;
    s_r[di] = r;
    s_flat[di] = flat;
    s_qpos[di] = qp;
  }
  // kDecodeWaitFirst: q, the cache and the scratch may be written by the kernel before this one, so
  // wait for it here. A sync_first launch (the one that re-enters scratch region 0) waits first in
  // every mode and only then lets the next launch start, so every launch after it begins with all
  // older launches complete.
  bool waited = false;
  if (P.mode == kDecodeWaitFirst || P.sync_first) {
    pdl_wait();
    waited = true;
  }
  if (P.sync_first) pdl_launch_dependents();
  __syncthreads();
  if (warp == 0 && !planned) {
    constexpr int kPer = MAXD / 32;
    int sum = 0;
    for (int i = 0; i < kPer; ++i) {
      const int idx = lane * kPer + i;
      if (idx < n_decode) sum += (s_qpos[idx] + kTok) / kTok;  // qpos/16+1, 0 when qpos = -1
    }
    int incl = sum;
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += y;
    }
    int run = incl - sum;
    for (int i = 0; i < kPer; ++i) {
      const int idx = lane * kPer + i;
      if (idx < n_decode) {
        s_cum[idx] = run;
        run += (s_qpos[idx] + kTok) / kTok;
      }
    }
    const int total = __shfl_sync(0xffffffffu, incl, 31);
    if (lane == 0) s_cum[n_decode] = total;
  }
  if (!planned) __syncthreads();  // the scan's results; a plan was complete at the barrier above
  // From here on the warps of the CTA never meet again: each one streams its own segment.

  const int total_pages = s_cum[n_decode];
  const int nseg = (static_cast<int>(gridDim.x) / P.groups) * SUB;
  const int seg = cta * SUB + sub;
  // The list is cut into segments of equal COST, not of equal length: a sequence that ends inside a
  // segment costs its warp a fixed amount on top of its pages (the row or partial to write, one more
  // ticket and possibly a merge at the end, a new set of q rows), and with equal lengths the launch
  // ends with the warps that have several such ends. So position x of the weighted list is page
  // x - end_weight * (sequences before it), each sequence is followed by end_weight positions that
  // hold no page, and segment s covers positions [s W, (s+1) W).
  const int w_end = P.end_weight;
  const long long total_w = total_pages + static_cast<long long>(w_end) * n_decode;
  const int W = max(2, static_cast<int>((total_w + nseg - 1) / nseg));  // positions per segment
  auto page_at = [&](long long x) {  // the first page at or after weighted position x
    if (x >= total_w) return total_pages;
    int a = 0, b = n_decode;  // largest a with s_cum[a] + w_end * a <= x
    while (b - a > 1) {
      const int mid = (a + b) >> 1;
      if (s_cum[mid] + static_cast<long long>(w_end) * mid <= x) a = mid; else b = mid;
    }
    const int o = static_cast<int>(x - (s_cum[a] + static_cast<long long>(w_end) * a));
    return s_cum[a] + min(o, s_cum[a + 1] - s_cum[a]);
  };
  auto segment_of = [&](int di, int page_in_seq) {
    return static_cast<int>((s_cum[di] + static_cast<long long>(w_end) * di + page_in_seq) / W);
  };
  const int lo = page_at(static_cast<long long>(seg) * W);
  const int hi = page_at(static_cast<long long>(seg + 1) * W);
  unsigned long long* counters =
      reinterpret_cast<unsigned long long*>(P.pl + decode_counter_base(P.partial_slots, n_decode * P.n_kv));

  uint8_t* my_stage = smem + warp * NS * kSlice;
  uint8_t* my_scale = smem + L::kScaleOff + warp * NS * kScaleBytes8;  // fp8 only
  uint64_t* my_bar = bars + warp * NS;
  bool dead = false;  // a wait ran out: stop waiting, finish the control flow, status is set

  // ---- producer cursor: next page this warp will request ----
  ItemCursor pc;
  item_at(pc, lo, hi, n_decode, s_cum);
  int p_page = pc.pb;
  int p_blk = 0;
  int islot = 0;
  // Moves to the next item until this warp has a page in it; with `load` it also fetches that
  // page's block id (used one page later, so the fetch is off the critical path in steady state).
  auto prod_settle = [&](bool load) {
    while (pc.off < hi && p_page >= pc.pe) {
      item_at(pc, pc.off + (pc.pe - pc.pb), hi, n_decode, s_cum);
      p_page = pc.pb;
    }
    if (load && pc.off < hi)
      p_blk = __ldg(P.bt + static_cast<long long>(s_r[pc.di]) * P.max_blocks + p_page);
  };
  auto prod_issue = [&](bool load_next) {
    if (pc.off >= hi) return;
    if (static_cast<unsigned>(p_blk) >= static_cast<unsigned>(P.num_blocks))
      report(FQB_ERR_INDEX, kKidDecode, p_blk);  // the load below then reads zeros
    if (lane == 0) {
      if constexpr (FP8) {
        const bool ok = static_cast<unsigned>(p_blk) < static_cast<unsigned>(P.num_blocks);
        mbar_expect_tx(&my_bar[islot], kPageBytes8 + kScaleBytes8);
        tma_load_page(my_stage + islot * kPageBytes8, &tmap, &my_bar[islot], 0, 0, kvh, 0, p_blk);
        bulk_load(my_scale + islot * kScaleBytes8,
                  P.scales + (static_cast<long long>(ok ? p_blk : 0) * P.n_kv + kvh) * (2 * kTok), kScaleBytes8,
                  &my_bar[islot]);
      } else {
        mbar_expect_tx(&my_bar[islot], kPageBytes);
        tma_load_page(my_stage + islot * kPageBytes, &tmap, &my_bar[islot], 0, 0, kvh * 2, 0, p_blk);
      }
    }
    islot = (islot + 1 == NS) ? 0 : islot + 1;
    p_page += 1;
    prod_settle(load_next);
  };
  // Filling the ring: the block ids of this warp's first NS pages are fetched with ONE load (lane j
  // takes the j-th page) instead of NS dependent ones.
  prod_settle(false);
  {
    const int n_first = pc.off < hi ? min(NS, pc.pe - p_page) : 0;
    const int pre = lane < n_first
                        ? __ldg(P.bt + static_cast<long long>(s_r[pc.di]) * P.max_blocks + p_page + lane)
                        : 0;
#pragma unroll
    for (int s = 0; s < NS; ++s) {
      if (s < n_first) {
        p_blk = __shfl_sync(0xffffffffu, pre, s);
        prod_issue(s + 1 >= n_first);  // the last prefetched page goes back to the one-ahead scheme
      } else {
        prod_issue(true);
      }
    }
  }
  // kDecodeWaitRows: the pages requested above hold only keys that were cached before the kernel
  // ahead of this one began; the q / K / V rows of the step may be its product, so wait for it now.
  if (P.mode == kDecodeWaitRows && !waited) pdl_wait();

  if (blockIdx.x == 0 && P.kvh_base == 0)
    for (int di = tid; di < n_decode; di += NW * 32)
      if (s_qpos[di] < 0) {  // no key at all: the row is zero (the reference's inv = 0 case)
        uint4* o = reinterpret_cast<uint4*>(P.out + static_cast<long long>(s_flat[di]) * P.n_heads * kHd);
        for (int i = 0; i < P.n_heads * kHd / 8; ++i) o[i] = make_uint4(0, 0, 0, 0);
        for (int r = 0; r < P.n_peers; ++r) {
          uint4* po = reinterpret_cast<uint4*>(
              P.peer_out[r] + (static_cast<long long>(s_flat[di]) * P.peer_heads + P.peer_col) * kHd);
          for (int i = 0; i < P.n_heads * kHd / 8; ++i) po[i] = make_uint4(0, 0, 0, 0);
        }
      }

  // ---- consumer ----
  const int g = lane >> 2, t = lane & 3;
  const int mat = lane >> 3;
  const int k_tok = ((mat >> 1) << 3) + (lane & 7), k_sel = mat & 1;
  const int v_tok = ((mat & 1) << 3) + (lane & 7), v_sel = mat >> 1;
  // A-fragment words of this lane inside the 4 x 128 q block of a kv head (rows g >= 4 are padding)
  auto load_q = [&](uint32_t (&dst)[8][2], int di) {
    const uint32_t* qw = reinterpret_cast<const uint32_t*>(
        P.q + static_cast<long long>(s_flat[di]) * P.q_stride + kvh * (kGroup * kHd) + (g & 3) * kHd);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const uint32_t a = __ldg(qw + ks * 8 + t), b = __ldg(qw + ks * 8 + t + 4);
      dst[ks][0] = g < kGroup ? a : 0u;
      dst[ks][1] = g < kGroup ? b : 0u;
    }
  };

  // fp8 path: lane (g, t) holds q dims [32t, 32t+32) of head g as f16 pairs, two words per k-step
  auto load_q8 = [&](uint32_t (&dst)[8][2], int di) {
    const uint4* qv = reinterpret_cast<const uint4*>(
        P.q + static_cast<long long>(s_flat[di]) * P.q_stride + kvh * (kGroup * kHd) + (g & 3) * kHd + 32 * t);
#pragma unroll
    for (int c = 0; c < 4; ++c) {  // 8 bf16 = k-steps 2c and 2c+1
      const uint4 v = __ldg(qv + c);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float lo_f = __uint_as_float(w[i] << 16), hi_f = __uint_as_float(w[i] & 0xffff0000u);
        const uint32_t h = pack_f16(lo_f, hi_f);
        dst[2 * c + (i >> 1)][i & 1] = g < kGroup ? h : 0u;
      }
    }
  };
  auto fetch_q = [&](uint32_t (&dst)[8][2], int di) {
    if constexpr (FP8) load_q8(dst, di); else load_q(dst, di);
  };

  bool wrote_rows = blockIdx.x == 0 && P.kvh_base == 0;  // CTA 0 may have written the zero rows above
  // A sequence cut by segment boundaries costs its warp a fence, an atomic round trip and, for the last
  // arriver, a merge: about 6 us measured, during which the warp's ring stands still. So the partial
  // is only stored when the item ends; the tickets are taken later -- when the warp has no more pages to
  // stream (or kMaxPending items are waiting) -- for all waiting items at once, one lane per item, their
  // round trips in flight together; then the merges this warp has won, one after the other.
  int n_pend = 0;
  auto settle = [&]() {
    __syncwarp();  // the lanes' partial stores are ordered before the fences below
    int di_mine = -1, b0 = 0, b1 = 0, last = 0;
    if (lane < n_pend) {
      di_mine = s_pend[lane];
      const int np_seq = s_cum[di_mine + 1] - s_cum[di_mine];
      b0 = segment_of(di_mine, 0);
      b1 = segment_of(di_mine, np_seq - 1);
      unsigned long long* c = counters + static_cast<long long>(di_mine) * P.n_kv + kvh;
      __threadfence();
      last = take_ticket_is_last(c, P.epoch, b1 - b0 + 1) ? 1 : 0;
      __threadfence();
    }
    unsigned won = __ballot_sync(0xffffffffu, last != 0);
    while (won) {
      const int src = __ffs(won) - 1;
      won &= won - 1;
      const int di = __shfl_sync(0xffffffffu, di_mine, src);
      const int sb0 = __shfl_sync(0xffffffffu, b0, src), sb1 = __shfl_sync(0xffffffffu, b1, src);
      merge_pair(P, di, kvh, sb0, sb1, s_flat[di], lane);
      wrote_rows = true;
      if (lane == 0) counters[static_cast<long long>(di) * P.n_kv + kvh] = 0ull;
    }
    n_pend = 0;
    __syncwarp();
  };
  ItemCursor cc;
  item_at(cc, lo, hi, n_decode, s_cum);
  int cslot = 0;
  uint32_t cphase = 0;
  uint32_t qa[8][2], qn[8][2];
  if (cc.off < hi) fetch_q(qa, cc.di);
  const long long plane_elems = static_cast<long long>(kTok) * P.n_kv * kHd;

#pragma unroll 1
  while (cc.off < hi) {
    ItemCursor nx;
    item_at(nx, cc.off + (cc.pe - cc.pb), hi, n_decode, s_cum);
    if (nx.off < hi) fetch_q(qn, nx.di);  // lands while this item is processed

    float o[16][4];
#pragma unroll
    for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float m = kNegBig, l = 0.f;
    const int qpos = s_qpos[cc.di];
    const int flat = s_flat[cc.di];

#pragma unroll 1
    for (int page = cc.pb; page < cc.pe; ++page) {
      // fused append: this warp is the only one that streams the sequence's last page for this head
      // (every shape comes in two builds: where registers are short -- 168 per thread with three or six CTAs
      // per SM -- the fused append's code costs the attention-only kernel a few per cent)
      const bool appends = APPEND && P.cache_w != nullptr && page == cc.np - 1;
      uint4 new_row = make_uint4(0, 0, 0, 0);
      int a_blk = 0;
      if (appends) {  // lane -> plane = lane / 16 (K, V), 16-byte chunk lane % 16 of the head's 256-byte row
        a_blk = __ldg(P.bt + static_cast<long long>(s_r[cc.di]) * P.max_blocks + page);
        new_row = *reinterpret_cast<const uint4*>(P.q + static_cast<long long>(flat) * P.q_stride +
                                                  (lane < 16 ? P.k_rel : P.v_rel) + kvh * kHd + (lane & 15) * 8);
      }
      if (!dead && !mbar_wait_bounded(&my_bar[cslot], cphase)) {
        dead = true;
        report(FQB_ERR_TIMEOUT, kKidDecode, page);
      }
      uint8_t* st = my_stage + cslot * kSlice;
      const int nvalid = min(kTok, qpos - page * kTok + 1);
      if constexpr (!FP8) {
        if (appends) {
          const int slot = qpos & (kTok - 1), plane = lane >> 4;
          if (static_cast<unsigned>(a_blk) < static_cast<unsigned>(P.num_blocks))
            *reinterpret_cast<uint4*>(P.cache_w + (static_cast<long long>(a_blk) * FQB_PLANES + plane) * plane_elems +
                                      static_cast<long long>(slot) * (P.n_kv * kHd) + kvh * kHd + (lane & 15) * 8) = new_row;
          *reinterpret_cast<uint4*>(st + plane * kPlaneBytes + page_chunk_off(slot, lane & 15)) = new_row;
        }
        if (nvalid < kTok) {
          // tail of the sequence's last page was never written: its V rows may hold anything
          if (lane < 16)
            for (int row = nvalid; row < kTok; ++row)
              *reinterpret_cast<uint4*>(st + kPlaneBytes + (lane >> 3) * kHalfBytes + row * 128 +
                                        ((lane & 7) << 4)) = make_uint4(0, 0, 0, 0);
        }
        if (appends || nvalid < kTok) {
          // generic-proxy writes into a buffer the async proxy (TMA) refills later
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
        // the running maximum moves on the first pages of a sequence and rarely afterwards: the
        // accumulator is rescaled only on pages where some row's maximum grew
        if (__any_sync(0xffffffffu, mx > m)) {
          const float mnew = fmaxf(m, mx);
          const float corr = fast_exp2(m - mnew);
          m = mnew;
          l *= corr;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            o[j][0] *= corr;
            o[j][1] *= corr;
          }
        }
        const float p00 = fast_exp2(x00 - m), p01 = fast_exp2(x01 - m);
        const float p10 = fast_exp2(x10 - m), p11 = fast_exp2(x11 - m);
        l += (p00 + p01) + (p10 + p11);
        const uint32_t pa0 = pack_bf16(p00, p01), pa2 = pack_bf16(p10, p11);
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4_trans(vbase + page_chunk_off(v_tok, jj * 2 + v_sel), b0, b1, b2, b3);
          mma_bf16(o[2 * jj], pa0, 0u, pa2, 0u, b0, b1);
          mma_bf16(o[2 * jj + 1], pa0, 0u, pa2, 0u, b2, b3);
        }
      } else {
        if (appends) {
          // The step's token in the fp8 format: lanes 0..15 hold the K row of this head, lanes 16..31 the V
          // row, 8 values each; one scale per row (amax / 448), bytes e4m3(x * (448 / amax)) -- the
          // operations of kv_append_fp8_kernel, so the cache gets the same bytes. The row goes to the
          // cache and into the slice that has just arrived (swizzled like the rest of it), its scale to
          // the scale array and to the slice's scales.
          const int slot = qpos & (kTok - 1), plane = lane >> 4, l16 = lane & 15;
          const uint32_t w[4] = {new_row.x, new_row.y, new_row.z, new_row.w};
          float x[8];
          float amax = 0.f;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            x[2 * k] = __uint_as_float(w[k] << 16);
            x[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
            amax = fmaxf(amax, fmaxf(fabsf(x[2 * k]), fabsf(x[2 * k + 1])));
          }
#pragma unroll
          for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
          const float sq = amax > 0.f ? __fdiv_rn(amax, 448.0f) : 1.0f;
          const float inv = amax > 0.f ? __fdiv_rn(448.0f, amax) : 0.0f;
          uint32_t b[4];
#pragma unroll
          for (int k = 0; k < 4; ++k)
            b[k] = __nv_cvt_float2_to_fp8x2(make_float2(__fmul_rn(x[2 * k], inv), __fmul_rn(x[2 * k + 1], inv)),
                                            __NV_SATFINITE, __NV_E4M3);
          const uint2 bytes = make_uint2(b[0] | (b[1] << 16), b[2] | (b[3] << 16));
          if (static_cast<unsigned>(a_blk) < static_cast<unsigned>(P.num_blocks)) {
            uint8_t* c8 = reinterpret_cast<uint8_t*>(P.cache_w);
            *reinterpret_cast<uint2*>(c8 + ((static_cast<long long>(a_blk) * FQB_PLANES + plane) * kTok + slot) *
                                               (static_cast<long long>(P.n_kv) * kHd) + kvh * kHd + l16 * 8) = bytes;
            if (l16 == 0)
              P.scales_w[((static_cast<long long>(a_blk) * P.n_kv + kvh) * 2 + plane) * kTok + slot] = sq;
          }
          *reinterpret_cast<uint2*>(st + plane * (kPageBytes8 / 2) + slot * 128 + (((l16 >> 1) ^ (slot & 7)) << 4) +
                                    (l16 & 1) * 8) = bytes;
          if (l16 == 0) reinterpret_cast<float*>(my_scale + cslot * kScaleBytes8)[plane * kTok + slot] = sq;
        }
        if (nvalid < kTok) {
          // tail of the sequence's last page was never written: bytes there may decode to NaN
          for (int row = nvalid; row < kTok; ++row)
            if (lane < 8) *reinterpret_cast<uint4*>(st + kPageBytes8 / 2 + row * 128 + (lane << 4)) = make_uint4(0, 0, 0, 0);
        }
        if (appends || nvalid < kTok) {
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
        }
        const float* sc = reinterpret_cast<const float*>(my_scale + cslot * kScaleBytes8);
        const uint32_t kbase = smem_u32(st), vbase = kbase + kPageBytes8 / 2;
        // ---- S = Q K^T: key tokens g (tile 0) and g + 8 (tile 1), this lane's 32 dims of each ----
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
        {
          uint32_t kw[2][8];
#pragma unroll
          for (int tile = 0; tile < 2; ++tile) {
            const int tok = g + 8 * tile;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
              uint32_t x0, x1, x2, x3;
              asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                           : "=r"(x0), "=r"(x1), "=r"(x2), "=r"(x3)
                           : "r"(kbase + tok * 128 + (((2 * t + c) ^ (tok & 7)) << 4)));
              kw[tile][4 * c] = x0; kw[tile][4 * c + 1] = x1; kw[tile][4 * c + 2] = x2; kw[tile][4 * c + 3] = x3;
            }
          }
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            uint32_t b0, b1, b2, b3;
            e4m3x4_to_f16x2x2(kw[0][ks], b0, b1);
            e4m3x4_to_f16x2x2(kw[1][ks], b2, b3);
            mma_f16(s0, qa[ks][0], 0u, qa[ks][1], 0u, b0, b1);
            mma_f16(s1, qa[ks][0], 0u, qa[ks][1], 0u, b2, b3);
          }
        }
        const float2 ka = *reinterpret_cast<const float2*>(sc + 2 * t), kb = *reinterpret_cast<const float2*>(sc + 8 + 2 * t);
        float2 va = *reinterpret_cast<const float2*>(sc + kTok + 2 * t), vb = *reinterpret_cast<const float2*>(sc + kTok + 8 + 2 * t);
        float x00 = s0[0] * (ka.x * P.scale_log2), x01 = s0[1] * (ka.y * P.scale_log2);
        float x10 = s1[0] * (kb.x * P.scale_log2), x11 = s1[1] * (kb.y * P.scale_log2);
        if (nvalid < kTok) {  // scores and value scales of slots that were never written are not trusted
          if (2 * t >= nvalid) { x00 = kNegBig; va.x = 0.f; }
          if (2 * t + 1 >= nvalid) { x01 = kNegBig; va.y = 0.f; }
          if (2 * t + 8 >= nvalid) { x10 = kNegBig; vb.x = 0.f; }
          if (2 * t + 9 >= nvalid) { x11 = kNegBig; vb.y = 0.f; }
        }
        float mx = fmaxf(fmaxf(x00, x01), fmaxf(x10, x11));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        if (__any_sync(0xffffffffu, mx > m)) {  // rescale only where some row's maximum grew
          const float mnew = fmaxf(m, mx);
          const float corr = fast_exp2(m - mnew);
          m = mnew;
          l *= corr;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            o[j][0] *= corr;
            o[j][1] *= corr;
          }
        }
        const float p00 = fast_exp2(x00 - m), p01 = fast_exp2(x01 - m);
        const float p10 = fast_exp2(x10 - m), p11 = fast_exp2(x11 - m);
        l += (p00 + p01) + (p10 + p11);
        const uint32_t pa0 = pack_f16(p00 * (va.x * kPScale8), p01 * (va.y * kPScale8));
        const uint32_t pa2 = pack_f16(p10 * (vb.x * kPScale8), p11 * (vb.y * kPScale8));
        // ---- O += P V: value tokens 2t, 2t+1, 2t+8, 2t+9, dims 16g .. 16g+15 (accumulator tile j = dim 16g+j) ----
        uint32_t vr[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int tok = 2 * t + (i & 1) + 8 * (i >> 1);
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                       : "=r"(vr[i][0]), "=r"(vr[i][1]), "=r"(vr[i][2]), "=r"(vr[i][3])
                       : "r"(vbase + tok * 128 + ((g ^ (tok & 7)) << 4)));
        }
#pragma unroll
        for (int wd = 0; wd < 4; ++wd) {
          // bytes (j, j+1) of rows 0/1 interleaved, then (j+2, j+3): two key pairs per permute
          const uint32_t e01a = __byte_perm(vr[0][wd], vr[1][wd], 0x5140), e01b = __byte_perm(vr[0][wd], vr[1][wd], 0x7362);
          const uint32_t e23a = __byte_perm(vr[2][wd], vr[3][wd], 0x5140), e23b = __byte_perm(vr[2][wd], vr[3][wd], 0x7362);
          uint32_t u0, u1, u2, u3, w0, w1, w2, w3;
          e4m3x4_to_f16x2x2(e01a, u0, u1);
          e4m3x4_to_f16x2x2(e23a, w0, w1);
          e4m3x4_to_f16x2x2(e01b, u2, u3);
          e4m3x4_to_f16x2x2(e23b, w2, w3);
          mma_f16(o[4 * wd + 0], pa0, 0u, pa2, 0u, u0, w0);
          mma_f16(o[4 * wd + 1], pa0, 0u, pa2, 0u, u1, w1);
          mma_f16(o[4 * wd + 2], pa0, 0u, pa2, 0u, u2, w2);
          mma_f16(o[4 * wd + 3], pa0, 0u, pa2, 0u, u3, w3);
        }
      }
      __syncwarp();  // every lane has read the buffer before it is refilled
      cslot = (cslot + 1 == NS) ? 0 : cslot + 1;
      if (cslot == 0) cphase ^= 1u;
      prod_issue(true);
    }

    // ---- end of item: this warp's softmax state of (cc.di, kvh) over its pages ----
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const bool whole = cc.pb == 0 && cc.pe == cc.np;
    if constexpr (FP8) {  // P carried a factor of kPScale8
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        o[j][0] *= 1.f / kPScale8;
        o[j][1] *= 1.f / kPScale8;
      }
    }
    if (whole) {
      // the pair lies inside this segment: straight from registers to `out`
      wrote_rows = true;
      if (g < kGroup) {
        const float inv = l > 0.f ? 1.f / l : 0.f;
        if constexpr (!FP8) {
          uint32_t w[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) w[j] = pack_bf16(o[j][0] * inv, o[j][1] * inv);
          uint32_t* dst = reinterpret_cast<uint32_t*>(
              P.out + (static_cast<long long>(flat) * P.n_heads + kvh * kGroup + g) * kHd);
#pragma unroll
          for (int j = 0; j < 16; ++j) dst[j * 4 + t] = w[j];
          for (int r = 0; r < P.n_peers; ++r) {
            uint32_t* pd = reinterpret_cast<uint32_t*>(
                P.peer_out[r] + (static_cast<long long>(flat) * P.peer_heads + P.peer_col + kvh * kGroup + g) * kHd);
#pragma unroll
            for (int j = 0; j < 16; ++j) pd[j * 4 + t] = w[j];
          }
        } else {
          // accumulator tile j holds dims 32t + j (column 0) and 32t + 16 + j (column 1): 32 contiguous dims
          uint4 w[4];
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            w[2 * c].x = pack_bf16(o[0][c] * inv, o[1][c] * inv);
            w[2 * c].y = pack_bf16(o[2][c] * inv, o[3][c] * inv);
            w[2 * c].z = pack_bf16(o[4][c] * inv, o[5][c] * inv);
            w[2 * c].w = pack_bf16(o[6][c] * inv, o[7][c] * inv);
            w[2 * c + 1].x = pack_bf16(o[8][c] * inv, o[9][c] * inv);
            w[2 * c + 1].y = pack_bf16(o[10][c] * inv, o[11][c] * inv);
            w[2 * c + 1].z = pack_bf16(o[12][c] * inv, o[13][c] * inv);
            w[2 * c + 1].w = pack_bf16(o[14][c] * inv, o[15][c] * inv);
          }
          uint4* dst = reinterpret_cast<uint4*>(
              P.out + (static_cast<long long>(flat) * P.n_heads + kvh * kGroup + g) * kHd + 32 * t);
#pragma unroll
          for (int i = 0; i < 4; ++i) dst[i] = w[i];
          for (int r = 0; r < P.n_peers; ++r) {
            uint4* pd = reinterpret_cast<uint4*>(
                P.peer_out[r] + (static_cast<long long>(flat) * P.peer_heads + P.peer_col + kvh * kGroup + g) * kHd + 32 * t);
#pragma unroll
            for (int i = 0; i < 4; ++i) pd[i] = w[i];
          }
        }
      }
    } else {
      const long long slot0 = ((static_cast<long long>(cc.di) + seg) * P.n_kv + kvh) * kGroup;
      if (g < kGroup) {
        if constexpr (!FP8) {
          float* dst = P.pa + (slot0 + g) * kHd + 2 * t;
#pragma unroll
          for (int j = 0; j < 16; ++j) *reinterpret_cast<float2*>(dst + j * 8) = make_float2(o[j][0], o[j][1]);
        } else {
          float4* dst = reinterpret_cast<float4*>(P.pa + (slot0 + g) * kHd + 32 * t);
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int i = 0; i < 4; ++i)
              dst[4 * c + i] = make_float4(o[4 * i][c], o[4 * i + 1][c], o[4 * i + 2][c], o[4 * i + 3][c]);
        }
        if (t == 0) {
          P.pm[slot0 + g] = m;
          P.pl[slot0 + g] = l;
        }
      }
      if (lane == 0) s_pend[n_pend] = cc.di;
      ++n_pend;
    }
    if (n_pend == kMaxPending || (nx.off >= hi && n_pend > 0)) settle();
    cc = nx;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      qa[ks][0] = qn[ks][0];
      qa[ks][1] = qn[ks][1];
    }
  }
  // ---- reassembly: tell every rank that this rank's rows of the launch are in its buffer ----
  // Fences are cumulative, so the expensive ones are few: a warp orders its lanes' stores before lane 0
  // with the warp barrier and hands them to its CTA with a CTA-scope fence and an arrival in shared
  // memory; the CTA's last warp makes them (and its own) visible to the GPU with ONE device-scope fence
  // -- that one returns only when the stores have been performed, wherever their memory is -- and arrives
  // on the slot's word with one plain atomic add (hundreds of warps in a compare-and-swap loop on one word
  // serialise for tens of microseconds); the launch's last CTA issues the one system-scope fence and then
  // stores the publish number into every rank's flag word (relaxed: the fence before them orders them
  // after everything the arrivals have handed over). It also puts the word back to zero, which is why
  // two launches that can overlap must not share a slot.
  if (P.n_peers > 0 && P.arrive != nullptr) {  // (null: the caller publishes later, for all slots at once)
    __syncwarp();
    if (lane == 0) {
      if (wrote_rows) __threadfence_block();
      if (atomicAdd(s_arrive, 1u) + 1u == static_cast<unsigned>(NW)) {
        __threadfence();
        unsigned* word = reinterpret_cast<unsigned*>(P.arrive);
        if (atomicAdd(word, 1u) + 1u == gridDim.x) {
          *word = 0u;
          const unsigned v = atomicAdd(P.seq, 1u) + 1u;
          __threadfence_system();
          for (int r = 0; r < P.n_peers; ++r)
            asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(P.peer_flag[r]), "r"(v) : "memory");
        }
      }
    }
  }
  // A kernel never completes before the one launched ahead of it: one warp of CTA 0 stays until that
  // one is done. Only one -- a CTA that waits keeps its shared memory, and with every CTA waiting a
  // quarter of each CTA's residency was spent idle here instead of hosting the next launch.
  if (blockIdx.x == 0 && warp == 0) pdl_wait();
}

}  // namespace fqb
