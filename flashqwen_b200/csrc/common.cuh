// Shared device helpers for the libfqb kernels (sm_100a): bounded mbarrier waits, TMA tensor
// loads, ldmatrix / mma.sync wrappers, the device status word and host-side error plumbing.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/fqb.h"

namespace fqb {

constexpr int kTok = FQB_BLOCK_TOKENS;  // tokens per page
constexpr int kHd = FQB_HEAD_DIM;       // head dim
constexpr int kGroup = FQB_GQA_GROUP;   // q heads per kv head
// One TMA box = the K and V slices of one kv head of one page:
// [2 planes][2 halves of 64 dims][16 tokens][64 bf16], 128-byte swizzled rows.
constexpr int kPageBytes = 2 * 2 * kTok * 64 * 2;  // 8192
constexpr int kPlaneBytes = kPageBytes / 2;         // 4096
constexpr int kHalfBytes = kPlaneBytes / 2;         // 2048

// ids written to the status word so a failure names its kernel
enum KernelId { kKidAppend = 1, kKidDecode = 2, kKidCombine = 3, kKidPrefill = 4, kKidBlocks = 5,
                kKidNormRope = 6, kKidGather = 7 };

// {code, kernel id, blockIdx.x, value}; first failure wins
__device__ int g_status[4];

__device__ __forceinline__ void report(int code, int kid, int value) {
  if (atomicCAS(&g_status[0], 0, code) == 0) {
    g_status[1] = kid;
    g_status[2] = static_cast<int>(blockIdx.x);
    g_status[3] = value;
  }
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier ------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One poll: the thread may be suspended until the phase completes, but for no longer than about
// kSuspendNs (without the hint the limit is the system's own, which is not documented; the prefill
// kernel, whose warps hand tiles to one another through mbarriers, ran 8 % faster with the hint).
constexpr uint32_t kSuspendNs = 10000;
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(kSuspendNs)
      : "memory");
  return ok != 0;
}
// Waits for the phase with the given parity and gives up after kWaitNs of the global timer (read every
// 64th poll; a poll itself blocks for a hardware-defined short time, which is why the bound is one of
// time and not of polls). Returns false on give-up.
constexpr unsigned long long kWaitNs = 500ull * 1000 * 1000;
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
#pragma unroll 1
  for (int i = 0; i < 64; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
#pragma unroll 1
  while (global_ns() - t0 < kWaitNs) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}

// ---- TMA -----------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 5-D tiled load of one page slice into shared memory; completion is signalled on bar as bytes.
__device__ __forceinline__ void tma_load_page(void* dst, const CUtensorMap* m, uint64_t* bar,
                                              int c0, int c1, int c2, int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6, %7}], [%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3),
      "r"(c4)
      : "memory");
}

// ---- programmatic dependent launch ---------------------------------------------------------------
// launch_dependents lets the next kernel on the stream (if it was launched with the programmatic
// serialization attribute) begin while this one still runs; wait blocks until the kernel launched
// before this one has completed and its writes are visible. Both are no-ops for plain launches.
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- cp.async (16-byte, for the small q rows) -----------------------------------------------
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// ---- tensor-core fragments -----------------------------------------------------------------
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                        uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                              uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
// D(16x8, fp32) += A(16x16, bf16) * B(16x8, bf16)
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// D(16x8, fp32) += A(16x16, f16) * B(16x8, f16)
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                        uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// two e4m3 bytes (low byte first) -> f16x2 (low half first); exact
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t two_bytes) {
  uint32_t r;
  asm("{\n\t.reg .b16 s;\n\tcvt.u16.u32 s, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, s;\n\t}" : "=r"(r) : "r"(two_bytes));
  return r;
}
// four e4m3 bytes -> two f16x2 words (bytes 0,1 and bytes 2,3); exact
__device__ __forceinline__ void e4m3x4_to_f16x2x2(uint32_t four_bytes, uint32_t& lo, uint32_t& hi) {
  asm("{\n\t.reg .b16 a, b;\n\tmov.b32 {a, b}, %2;\n\tcvt.rn.f16x2.e4m3x2 %0, a;\n\tcvt.rn.f16x2.e4m3x2 %1, b;\n\t}"
      : "=r"(lo), "=r"(hi)
      : "r"(four_bytes));
}
// an f16x2 word as two floats (low half first); exact
__device__ __forceinline__ float2 f16x2_to_f32x2(uint32_t h) {
  float2 f;
  asm("{\n\t.reg .b16 a, b;\n\tmov.b32 {a, b}, %2;\n\tcvt.f32.f16 %0, a;\n\tcvt.f32.f16 %1, b;\n\t}"
      : "=f"(f.x), "=f"(f.y)
      : "r"(h));
  return f;
}
__device__ __forceinline__ uint32_t pack_f16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// 1-D bulk copy global -> shared, completion on bar as bytes (16-byte aligned addresses and size)
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Two fp32 operations per instruction (sm_100): d = a * b + c and d = a + b on register pairs, and the
// maximum of three values in one instruction.
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(d)
      : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)),
        "l"(*reinterpret_cast<unsigned long long*>(&c)));
  return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
  unsigned long long d;
  asm("add.rn.f32x2 %0, %1, %2;"
      : "=l"(d)
      : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)));
  return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Byte offset of the 16-byte chunk holding dims [8*c16, 8*c16+8) of token `tok` inside one
// plane of a page slice laid out by the TMA box above (128-byte swizzle: chunk ^= tok & 7).
__device__ __forceinline__ uint32_t page_chunk_off(int tok, int c16) {
  return static_cast<uint32_t>((c16 >> 3) * kHalfBytes + tok * 128 + (((c16 & 7) ^ (tok & 7)) << 4));
}

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kNegBig = -1.0e30f;

}  // namespace fqb
