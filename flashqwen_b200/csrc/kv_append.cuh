// Kernel 1: KV append through the block table, and its fused form with per-head RMSNorm + RoPE.
//
// Semantics follow the reference's StoreKvKernel (engine/src/kv_store.cu:48-64 of the FlashQwen
// tree) and HeadNormRopeKernel (engine/src/kernels.cu:97-131). The reference moves one 2-byte
// element per thread with two integer divisions and three dependent index loads each; here one
// CTA takes one token row, looks its page up once, and moves the row with 16-byte loads/stores.
#pragma once

#include <cuda_fp8.h>

#include "common.cuh"

namespace fqb {

struct AppendParams {
  __nv_bfloat16* cache;
  int num_blocks;
  int row_elems;  // kv_heads_local * 128
  const __nv_bfloat16* qkv;
  int src_stride, k_off, v_off;
  const int* bt;
  int bt_stride;
  const int* bt_row;
  const int* pos;
  int M;
};

// Element offset of token slot (block, pos%16) of the K plane; the V plane is plane_elems later.
__device__ __forceinline__ bool append_dst(const AppendParams& P, int m, int kid, long long& dst) {
  const int p = P.pos[m];
  const int page = p / kTok;
  if (p < 0 || page >= P.bt_stride) {
    report(FQB_ERR_INDEX, kid, p);
    return false;
  }
  const int blk = P.bt[static_cast<long long>(P.bt_row[m]) * P.bt_stride + page];
  if (static_cast<unsigned>(blk) >= static_cast<unsigned>(P.num_blocks)) {
    report(FQB_ERR_INDEX, kid, blk);
    return false;
  }
  const long long plane = static_cast<long long>(kTok) * P.row_elems;
  dst = static_cast<long long>(blk) * FQB_PLANES * plane + static_cast<long long>(p % kTok) * P.row_elems;
  return true;
}

__global__ void __launch_bounds__(256)
kv_append_kernel(const AppendParams P) {
  const int m = blockIdx.x;
  pdl_launch_dependents();  // the attention kernel that follows may run its metadata prologue now
  pdl_wait();               // the rows were produced by the kernel before this one
  long long dst;
  if (!append_dst(P, m, kKidAppend, dst)) return;
  const int vecs = P.row_elems / 8;  // 16-byte vectors per plane row
  const long long plane = static_cast<long long>(kTok) * P.row_elems;
  const __nv_bfloat16* src = P.qkv + static_cast<long long>(m) * P.src_stride;
  for (int v = threadIdx.x; v < 2 * vecs; v += blockDim.x) {
    const int pl = v >= vecs;
    const int i = v - pl * vecs;
    const uint4 val = __ldg(reinterpret_cast<const uint4*>(src + (pl ? P.v_off : P.k_off)) + i);
    *(reinterpret_cast<uint4*>(P.cache + dst + pl * plane) + i) = val;
  }
}

// fp8 form of the append: each head's 128 K (and V) values are stored as e4m3 bytes with one fp32
// scale per (token, head, plane): s = amax / 448 (1 for an all-zero row), byte = e4m3(x * (448 / amax))
// rounded to nearest even, saturating. cache is [num_blocks][2][16][row_elems] BYTES (P.cache is used
// as a byte pointer), scales [num_blocks][heads][2][16] fp32. One warp per (plane, head); every step is
// one IEEE operation, so the host restatement gives the same bytes.
__global__ void __launch_bounds__(256)
kv_append_fp8_kernel(const AppendParams P, float* __restrict__ scales) {
  const int m = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();
  pdl_wait();
  long long dst;  // element offset of the token slot in the K plane; elements are bytes here
  if (!append_dst(P, m, kKidAppend, dst)) return;
  const int heads = P.row_elems / kHd;
  const int p = P.pos[m];
  const long long blk = dst / (static_cast<long long>(FQB_PLANES) * kTok * P.row_elems);
  const long long plane = static_cast<long long>(kTok) * P.row_elems;
  uint8_t* cache8 = reinterpret_cast<uint8_t*>(P.cache);
  const __nv_bfloat16* src = P.qkv + static_cast<long long>(m) * P.src_stride;
  for (int hd = warp; hd < 2 * heads; hd += 8) {
    const int pl = hd >= heads, h = hd - pl * heads;
    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(src + (pl ? P.v_off : P.k_off) + h * kHd) + lane);
    const float x0 = __uint_as_float(raw.x << 16), x1 = __uint_as_float(raw.x & 0xffff0000u);
    const float x2 = __uint_as_float(raw.y << 16), x3 = __uint_as_float(raw.y & 0xffff0000u);
    float amax = fmaxf(fmaxf(fabsf(x0), fabsf(x1)), fmaxf(fabsf(x2), fabsf(x3)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float s = amax > 0.f ? __fdiv_rn(amax, 448.0f) : 1.0f;
    const float inv = amax > 0.f ? __fdiv_rn(448.0f, amax) : 0.0f;
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(__fmul_rn(x0, inv), __fmul_rn(x1, inv)), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(__fmul_rn(x2, inv), __fmul_rn(x3, inv)), __NV_SATFINITE, __NV_E4M3);
    *reinterpret_cast<uint32_t*>(cache8 + dst + pl * plane + h * kHd + 4 * lane) = lo | (hi << 16);
    if (lane == 0) scales[((blk * heads + h) * 2 + pl) * kTok + p % kTok] = s;
  }
}

// Blocks of the fp8 cache read back as bf16 into a dense buffer [n][2][16][row_elems]: out block i is
// block list[i], every value bf16(e4m3_to_float(byte) * scale), the product one fp32 multiplication (so
// the host restatement gives the same bits). For the chunked prefill of a request whose history lives in
// the fp8 cache: its pages are read back once per chunk into a staging pool that the prefill kernel
// attends. One warp per (plane, token) row of the block: a lane turns 16 bytes into 16 bf16 at a time.
__global__ void __launch_bounds__(256)
dequant_blocks_fp8_kernel(const uint8_t* __restrict__ cache8, const float* __restrict__ scales, int num_blocks,
                          int heads, const int* __restrict__ list, __nv_bfloat16* __restrict__ out) {
  const int i = blockIdx.x;
  const int blk = __ldg(list + i);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (static_cast<unsigned>(blk) >= static_cast<unsigned>(num_blocks)) {
    if (threadIdx.x == 0 && blockIdx.y == 0) report(FQB_ERR_INDEX, kKidBlocks, blk);
    return;
  }
  const int row_elems = heads * kHd;
  const int chunks = row_elems / 16;  // 16-byte chunks of a row; 8 per head
  for (int r = blockIdx.y * 8 + warp; r < 2 * kTok; r += gridDim.y * 8) {
    const int pl = r / kTok, t = r % kTok;
    const long long row = (static_cast<long long>(pl) * kTok + t) * row_elems;
    const uint8_t* src = cache8 + static_cast<long long>(blk) * 2 * kTok * row_elems + row;
    __nv_bfloat16* dst = out + static_cast<long long>(i) * 2 * kTok * row_elems + row;
    for (int c = lane; c < chunks; c += 32) {
      const float s = __ldg(scales + ((static_cast<long long>(blk) * heads + (c >> 3)) * 2 + pl) * kTok + t);
      const uint4 b = __ldg(reinterpret_cast<const uint4*>(src) + c);
      const uint32_t w[4] = {b.x, b.y, b.z, b.w};
      uint32_t o[8];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        uint32_t h01, h23;
        e4m3x4_to_f16x2x2(w[k], h01, h23);
        const float2 f01 = f16x2_to_f32x2(h01), f23 = f16x2_to_f32x2(h23);
        o[2 * k] = pack_bf16(__fmul_rn(f01.x, s), __fmul_rn(f01.y, s));
        o[2 * k + 1] = pack_bf16(__fmul_rn(f23.x, s), __fmul_rn(f23.y, s));
      }
      reinterpret_cast<uint4*>(dst)[2 * c] = make_uint4(o[0], o[1], o[2], o[3]);
      reinterpret_cast<uint4*>(dst)[2 * c + 1] = make_uint4(o[4], o[5], o[6], o[7]);
    }
  }
}

struct NormRopeParams {
  AppendParams a;       // a.qkv is written in place, so the pointer is cast back to mutable
  int q_heads, kv_heads;
  int q_off;
  const float* wq;
  const float* wk;
  const float* cos_tab;
  const float* sin_tab;
  float eps;
};

// One warp per head of the row. Lane l holds dims {2l, 2l+1, 64+2l, 65+2l}: the two rotary
// partners are lane-local and the xor-shuffle butterfly below adds squares in the order
// (t, t+64), then strides 32, 16, 8, 4, 2, 1 -- the reference's shared-memory halving tree --
// so an IEEE evaluation is reproducible on the host bit for bit.
__global__ void __launch_bounds__(256)
norm_rope_append_kernel(const NormRopeParams P) {
  const int m = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();
  pdl_wait();
  // P.a.cache == nullptr: norm + rope only (the append is left to the decode kernel that follows)
  const bool store = P.a.cache != nullptr;
  long long dst = 0;
  bool ok;
  if (store) {
    ok = append_dst(P.a, m, kKidNormRope, dst);
  } else {
    ok = P.a.pos[m] >= 0;
    if (!ok) report(FQB_ERR_INDEX, kKidNormRope, P.a.pos[m]);
  }
  __nv_bfloat16* row = const_cast<__nv_bfloat16*>(P.a.qkv) + static_cast<long long>(m) * P.a.src_stride;
  const int p = P.a.pos[m];
  const float2 cs = ok ? __ldg(reinterpret_cast<const float2*>(P.cos_tab + static_cast<long long>(p) * 64) + lane)
                       : make_float2(1.f, 1.f);
  const float2 sn = ok ? __ldg(reinterpret_cast<const float2*>(P.sin_tab + static_cast<long long>(p) * 64) + lane)
                       : make_float2(0.f, 0.f);
  const int nheads = P.q_heads + P.kv_heads;
  for (int hd = warp; hd < nheads; hd += 8) {
    const bool is_k = hd >= P.q_heads;
    __nv_bfloat16* v = row + (is_k ? P.a.k_off + (hd - P.q_heads) * kHd : P.q_off + hd * kHd);
    const float* w = is_k ? P.wk : P.wq;
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(v + 2 * lane);
    const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(v + 64 + 2 * lane);
    const float x0 = __low2float(lo), x1 = __high2float(lo);
    const float x2 = __low2float(hi), x3 = __high2float(hi);
    float s0 = __fadd_rn(__fmul_rn(x0, x0), __fmul_rn(x2, x2));  // dims t, t+64
    float s1 = __fadd_rn(__fmul_rn(x1, x1), __fmul_rn(x3, x3));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      s0 = __fadd_rn(s0, __shfl_xor_sync(0xffffffffu, s0, o));
      s1 = __fadd_rn(s1, __shfl_xor_sync(0xffffffffu, s1, o));
    }
    const float ss = __fadd_rn(s0, s1);
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, static_cast<float>(kHd)), P.eps)));
    const float2 w_lo = __ldg(reinterpret_cast<const float2*>(w) + lane);
    const float2 w_hi = __ldg(reinterpret_cast<const float2*>(w + 64) + lane);
    const float y0 = __fmul_rn(__fmul_rn(x0, inv), w_lo.x), y1 = __fmul_rn(__fmul_rn(x1, inv), w_lo.y);
    const float y2 = __fmul_rn(__fmul_rn(x2, inv), w_hi.x), y3 = __fmul_rn(__fmul_rn(x3, inv), w_hi.y);
    const float r0 = __fsub_rn(__fmul_rn(y0, cs.x), __fmul_rn(y2, sn.x));
    const float r1 = __fsub_rn(__fmul_rn(y1, cs.y), __fmul_rn(y3, sn.y));
    const float r2 = __fadd_rn(__fmul_rn(y2, cs.x), __fmul_rn(y0, sn.x));
    const float r3 = __fadd_rn(__fmul_rn(y3, cs.y), __fmul_rn(y1, sn.y));
    const __nv_bfloat162 out_lo = __floats2bfloat162_rn(r0, r1), out_hi = __floats2bfloat162_rn(r2, r3);
    if (ok) {
      *reinterpret_cast<__nv_bfloat162*>(v + 2 * lane) = out_lo;
      *reinterpret_cast<__nv_bfloat162*>(v + 64 + 2 * lane) = out_hi;
      if (is_k && store) {
        __nv_bfloat16* c = P.a.cache + dst + (hd - P.q_heads) * kHd;
        *reinterpret_cast<__nv_bfloat162*>(c + 2 * lane) = out_lo;
        *reinterpret_cast<__nv_bfloat162*>(c + 64 + 2 * lane) = out_hi;
      }
    }
  }
  if (!ok || !store) return;
  const int vecs = P.a.row_elems / 8;
  const long long plane = static_cast<long long>(kTok) * P.a.row_elems;
  for (int i = threadIdx.x; i < vecs; i += blockDim.x)
    *(reinterpret_cast<uint4*>(P.a.cache + dst + plane) + i) =
        __ldg(reinterpret_cast<const uint4*>(row + P.a.v_off) + i);
}

}  // namespace fqb
