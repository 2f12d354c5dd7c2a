// Microbenchmark behind the figures quoted in the prefill kernels: what one thread pays for an mbarrier
// wait whose phase completed long ago, for the tcgen05 fences, for tcgen05.commit + wait, for clock64(),
// and how long a blocked wait takes to wake up after another warp arrives.
//   nvcc -std=c++17 -O3 -gencode arch=compute_100a,code=sm_100a -o wait_cost wait_cost.cu && ./wait_cost
#include <cstdio>
#include "../prefill_tc.cuh"
using namespace fqb;
__global__ void __launch_bounds__(128, 1) k(long long* out) {
  __shared__ uint64_t bar[4];
  __shared__ uint32_t slot;
  const int tid = threadIdx.x, warp = tid >> 5;
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 64;" ::"r"(smem_u32(&slot)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) { for (int i = 0; i < 4; ++i) mbar_init(&bar[i], 1); mbar_fence_init(); }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&slot);
  if (tid == 0) {
    mbar_arrive(&bar[0]);                      // phase 0 of bar[0] complete
    const int N = 256;
    long long t0 = clock64();
    int ok = 0;
    for (int i = 0; i < N; ++i) ok += mbar_wait_bounded(&bar[0], 0) ? 1 : 0;   // satisfied wait
    long long t1 = clock64();
    for (int i = 0; i < N; ++i) tc_fence_after();
    long long t2 = clock64();
    for (int i = 0; i < N; ++i) tc_fence_before();
    long long t3 = clock64();
    // commit with nothing outstanding + wait for it, alternating phases on bar[1]
    for (int i = 0; i < N; ++i) { umma_commit(&bar[1]); ok += mbar_wait_bounded(&bar[1], i & 1) ? 1 : 0; }
    long long t4 = clock64();
    long long acc = 0;
    for (int i = 0; i < N; ++i) acc += clock64();
    long long t5 = clock64();
    // arrive by this thread then wait (phase flips each time) on bar[2]
    for (int i = 0; i < N; ++i) { mbar_arrive(&bar[2]); ok += mbar_wait_bounded(&bar[2], i & 1) ? 1 : 0; }
    long long t6 = clock64();
    out[0] = (t1 - t0) / N; out[1] = (t2 - t1) / N; out[2] = (t3 - t2) / N; out[3] = (t4 - t3) / N;
    out[4] = (t5 - t4) / N; out[5] = (t6 - t5) / N; out[6] = ok; out[7] = acc & 1;
  }
  tc_fence_before(); __syncthreads();
  if (warp == 0) { tc_fence_after(); asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 64;" ::"r"(tmem) : "memory"); }
}
// cross-thread: warp 1 arrives every ~2000 clk, warp 0 thread waits; measures wake-up latency after the arrive
__global__ void __launch_bounds__(64, 1) k2(long long* out) {
  __shared__ uint64_t bar;
  __shared__ volatile long long t_arrive[64];
  const int tid = threadIdx.x;
  if (tid == 0) { mbar_init(&bar, 1); mbar_fence_init(); }
  __syncthreads();
  const int N = 32;
  if (tid == 32) {
    for (int i = 0; i < N; ++i) {
      long long t = clock64();
      while (clock64() - t < 3000) {}
      t_arrive[i] = clock64();
      mbar_arrive(&bar);
    }
  } else if (tid == 0) {
    long long sum = 0, mx = 0;
    for (int i = 0; i < N; ++i) {
      mbar_wait_bounded(&bar, i & 1);
      long long t = clock64();
      long long d = t - t_arrive[i];
      sum += d; if (d > mx) mx = d;
    }
    out[8] = sum / N; out[9] = mx;
  }
}
int main() {
  long long* d; cudaMalloc(&d, 128); cudaMemset(d, 0, 128);
  k<<<1, 128>>>(d); k2<<<1, 64>>>(d);
  cudaError_t e = cudaDeviceSynchronize();
  long long h[16]; cudaMemcpy(h, d, 128, cudaMemcpyDeviceToHost);
  printf("%s\nsatisfied wait %lld clk | fence::after %lld | fence::before %lld | commit+wait %lld | clock64 %lld | arrive+wait %lld | ok %lld\n",
         cudaGetErrorString(e), h[0], h[1], h[2], h[3], h[4], h[5], h[6]);
  printf("cross-thread wake-up after arrive: avg %lld clk, max %lld clk\n", h[8], h[9]);
  return 0;
}
