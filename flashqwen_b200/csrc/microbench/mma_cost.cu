// Microbenchmark behind the figures quoted in the prefill kernels: clocks per tcgen05.mma (cta_group::1,
// kind::f16, M128 K16) for N = 64 / 128 / 256, both operands in shared memory or A in tensor memory, one or
// two accumulators, one or two issuing warps. Operands are zeros; descriptors are those of the kernels.
//   nvcc -std=c++17 -O3 -gencode arch=compute_100a,code=sm_100a -o mma_cost mma_cost.cu && ./mma_cost
#include <cstdio>
#include "../prefill_tc.cuh"
using namespace fqb;

// mode 0: SS same D; 1: SS alternating two D; 2: TS (A in TMEM), B MN-major; 3: two issuer warps, SS
template <int N, int MODE>
__global__ void __launch_bounds__(128, 1) k(long long* out, int reps) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ uint64_t bar[2];
  __shared__ uint32_t slot;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < 98304 / 16; i += 128) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(&slot)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) { mbar_init(&bar[0], 1); mbar_init(&bar[1], 1); mbar_fence_init(); }
  proxy_fence_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&slot);
  const int issuers = MODE == 3 ? 2 : 1;
  if (warp < issuers && lane == 0) {
    constexpr uint32_t idesc = umma_idesc(128, N, MODE == 2);
    const uint64_t ad = umma_desc(smem_u32(smem), 16, 1024);
    const uint64_t bd = MODE == 2 ? umma_desc(smem_u32(smem + 32768), N == 128 ? 16384 : 8192, 1024)
                                  : umma_desc(smem_u32(smem + 32768), 16, 1024);
    const uint32_t d0 = tmem + warp * 256;
    long long t0 = clock64();
    for (int i = 0; i < reps; ++i) {
      const int j = i & 3, kb = (i >> 2) & 1;
      if (MODE == 2)
        umma_bf16_ts(d0 + 256 * 0 + 128, d0 + j * 8, bd + ((j * 2048) >> 4), idesc, i ? 1u : 0u);
      else
        umma_bf16((MODE == 1 && (i & 1)) ? d0 + 256 : d0, ad + ((kb * 16384 + j * 32) >> 4),
                  bd + ((kb * (N * 128) + j * 32) >> 4), idesc, i > 1 ? 1u : 0u);
    }
    long long t1 = clock64();
    umma_commit(&bar[warp]);
    bool ok = mbar_wait_bounded(&bar[warp], 0);
    long long t2 = clock64();
    if (blockIdx.x == 0) { out[warp * 3] = t1 - t0; out[warp * 3 + 1] = t2 - t0; out[warp * 3 + 2] = ok; }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
  }
}

template <int N, int MODE>
void run(const char* name, int grid) {
  long long* d; cudaMalloc(&d, 64); cudaMemset(d, 0, 64);
  cudaFuncSetAttribute(k<N, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 98304);
  const int reps = 512;
  for (int it = 0; it < 2; ++it) k<N, MODE><<<grid, 128, 98304>>>(d, reps);
  cudaError_t e = cudaDeviceSynchronize();
  long long h[8]; cudaMemcpy(h, d, 64, cudaMemcpyDeviceToHost);
  double flop = 2.0 * 128 * N * 16;
  printf("%-28s grid %3d N %3d: issue %6.1f clk/mma, done %6.1f clk/mma (%.0f flop/clk/SM) ok=%lld %s", name, grid, N,
         (double)h[0] / reps, (double)h[1] / reps, flop * (MODE == 3 ? 2 : 1) / ((double)h[1] / reps), h[2], cudaGetErrorString(e));
  if (MODE == 3) printf(" | warp1 done %6.1f", (double)h[4] / reps);
  printf("\n");
  cudaFree(d);
}

int main() {
  for (int grid : {1, 148}) {
    run<64, 0>("SS same D", grid);
    run<128, 0>("SS same D", grid);
    run<256, 0>("SS same D", grid);
    run<64, 1>("SS two D alternating", grid);
    run<128, 1>("SS two D alternating", grid);
    run<128, 2>("TS B mn-major", grid);
    run<64, 3>("SS two issuer warps", grid);
    run<128, 3>("SS two issuer warps", grid);
  }
  return 0;
}
