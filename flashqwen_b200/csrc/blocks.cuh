// Kernel 4: whole-page copies for prefix-cache copy-on-write, and gather / scatter of a block
// list into a contiguous buffer. The reference has no such kernel (it only aliases full blocks,
// engine/src/scheduler.cc:27-44 of the FlashQwen tree); a page is 2*16*row_elems bf16 and is
// moved as 16-byte vectors, 16 KiB per CTA.
#pragma once

#include "common.cuh"

namespace fqb {

constexpr int kCopyChunkVecs = 1024;  // 16 KiB per CTA

struct BlockMoveParams {
  void* const* layers;   // device array of layer base pointers, or nullptr
  uint4* cache;          // used when layers == nullptr
  uint4* lin;            // contiguous buffer for gather / scatter
  const int* idx;        // pairs (copy) or list (gather / scatter)
  int n;                 // pairs or list entries
  int num_blocks;
  int block_vecs;        // 16-byte vectors per page
  int mode;              // 0 copy, 1 gather, 2 scatter
};

__global__ void __launch_bounds__(256)
block_move_kernel(const BlockMoveParams P) {
  const int i = blockIdx.x;
  uint4* base = P.layers ? static_cast<uint4*>(P.layers[blockIdx.z]) : P.cache;
  const uint4* src;
  uint4* dst;
  if (P.mode == 0) {
    const int s = P.idx[2 * i], d = P.idx[2 * i + 1];
    if (static_cast<unsigned>(s) >= static_cast<unsigned>(P.num_blocks) ||
        static_cast<unsigned>(d) >= static_cast<unsigned>(P.num_blocks)) {
      report(FQB_ERR_INDEX, kKidBlocks, s);
      return;
    }
    src = base + static_cast<long long>(s) * P.block_vecs;
    dst = base + static_cast<long long>(d) * P.block_vecs;
  } else {
    const int b = P.idx[i];
    if (static_cast<unsigned>(b) >= static_cast<unsigned>(P.num_blocks)) {
      report(FQB_ERR_INDEX, kKidBlocks, b);
      return;
    }
    uint4* in_cache = base + static_cast<long long>(b) * P.block_vecs;
    uint4* in_lin = P.lin + static_cast<long long>(i) * P.block_vecs;
    src = P.mode == 1 ? in_cache : in_lin;
    dst = P.mode == 1 ? in_lin : in_cache;
  }
  const int v0 = blockIdx.y * kCopyChunkVecs;
  const int v1 = min(P.block_vecs, v0 + kCopyChunkVecs);
#pragma unroll 4
  for (int v = v0 + threadIdx.x; v < v1; v += 256) dst[v] = src[v];
}

}  // namespace fqb
