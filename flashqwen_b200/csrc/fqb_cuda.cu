// libfqb, CUDA side: the extern "C" operators declared in include/fqb.h. Host code here only
// validates scalar arguments, builds the TMA descriptor of the cache and enqueues kernels on the
// caller's stream; it allocates nothing and never synchronises (fqb_device_status excepted).
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <atomic>
#include <mutex>

#include "blocks.cuh"
#include "common.cuh"
#include "decode.cuh"
#include "errors.h"
#include "kv_append.cuh"
#include "prefill_tc_ks.cuh"

namespace fqb {
namespace {

int cuda_fail(cudaError_t e, const char* what) {
  return set_error(FQB_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}
#define FQB_CUDA_TRY(call)                                   \
  do {                                                       \
    cudaError_t e_ = (call);                                 \
    if (e_ != cudaSuccess) return cuda_fail(e_, #call);      \
  } while (0)

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

struct DeviceInfo {
  int sm_count = 0;
};
int device_info(DeviceInfo& out) {
  static std::mutex mu;
  static DeviceInfo cache[64];
  int dev = 0;
  FQB_CUDA_TRY(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lk(mu);
  if (dev < 0 || dev >= 64) return set_error(FQB_ERR_CUDA, "device ordinal %d out of range", dev);
  if (cache[dev].sm_count == 0) {
    int n = 0;
    FQB_CUDA_TRY(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
    cache[dev].sm_count = n;
  }
  out = cache[dev];
  return FQB_OK;
}

// ---- TMA descriptor of one layer's cache ------------------------------------------------------
// The cache [num_blocks][2][16][row_elems] is described as a 5-D tensor whose innermost
// dimension is 64 bf16 (128 bytes, the widest row the 128-byte swizzle takes):
//   d0 = 64 dims, d1 = 16 tokens, d2 = row_elems/64 half-heads, d3 = 2 planes, d4 = blocks.
// One box {64,16,2,2,1} is the K and V slice of one kv head of one page (8 KiB) and lands in
// shared memory as [plane][half][token][64] with rows of 128 bytes, which ldmatrix then reads
// without bank conflicts.
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

int get_encode(EncodeFn& fn) {
  static EncodeFn cached = nullptr;
  static std::mutex mu;
  std::lock_guard<std::mutex> lk(mu);
  if (!cached) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    FQB_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres));
    if (qres != cudaDriverEntryPointSuccess || !p)
      return set_error(FQB_ERR_CUDA, "cuTensorMapEncodeTiled not available from this driver");
    cached = reinterpret_cast<EncodeFn>(p);
  }
  fn = cached;
  return FQB_OK;
}

// half_boxes = false: box {64,16,2,2,1} = one 8 KiB page slice (K and V, both halves) per load.
// half_boxes = true : box {64,16,1,1,1} = one 2 KiB half of one plane, so that the caller can place
//                     the pieces as a UMMA operand tile.
int make_cache_map(const void* cache, int num_blocks, int kv_heads_local, CUtensorMap& map, bool half_boxes = false) {
  struct Entry {
    const void* ptr;
    int nb, kvh;
    bool half;
    CUtensorMap map;
  };
  constexpr int kCache = 128;
  static thread_local Entry lru[kCache];
  static thread_local int used = 0, next = 0;
  for (int i = 0; i < used; ++i)
    if (lru[i].ptr == cache && lru[i].nb == num_blocks && lru[i].kvh == kv_heads_local && lru[i].half == half_boxes) {
      map = lru[i].map;
      return FQB_OK;
    }
  EncodeFn enc;
  if (int rc = get_encode(enc)) return rc;
  const cuuint64_t row_bytes = static_cast<cuuint64_t>(kv_heads_local) * kHd * 2;
  cuuint64_t dims[5] = {64, static_cast<cuuint64_t>(kTok), static_cast<cuuint64_t>(kv_heads_local) * 2, 2,
                        static_cast<cuuint64_t>(num_blocks)};
  cuuint64_t strides[4] = {row_bytes, 128, row_bytes * kTok, row_bytes * kTok * 2};
  cuuint32_t box[5] = {64, static_cast<cuuint32_t>(kTok), half_boxes ? 1u : 2u, half_boxes ? 1u : 2u, 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(cache), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(FQB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
  Entry& e = lru[next];
  e.ptr = cache;
  e.nb = num_blocks;
  e.kvh = kv_heads_local;
  e.half = half_boxes;
  e.map = map;
  next = (next + 1) % kCache;
  if (used < kCache) ++used;
  return FQB_OK;
}

// fp8 cache [num_blocks][2][16][kv_heads*128] bytes as a 5-D tensor of bytes:
//   d0 = 128 bytes of one head, d1 = 16 tokens, d2 = heads, d3 = 2 planes, d4 = blocks.
// One box {128,16,1,2,1} is the K and V slice of one kv head of one page (4 KiB), rows of 128 bytes,
// 128-byte swizzle.
int make_cache_map_fp8(const void* cache8, int num_blocks, int kv_heads_local, CUtensorMap& map) {
  struct Entry {
    const void* ptr;
    int nb, kvh;
    CUtensorMap map;
  };
  constexpr int kCache = 64;
  static thread_local Entry lru[kCache];
  static thread_local int used = 0, next = 0;
  for (int i = 0; i < used; ++i)
    if (lru[i].ptr == cache8 && lru[i].nb == num_blocks && lru[i].kvh == kv_heads_local) {
      map = lru[i].map;
      return FQB_OK;
    }
  EncodeFn enc;
  if (int rc = get_encode(enc)) return rc;
  const cuuint64_t row_bytes = static_cast<cuuint64_t>(kv_heads_local) * kHd;
  cuuint64_t dims[5] = {static_cast<cuuint64_t>(kHd), static_cast<cuuint64_t>(kTok), static_cast<cuuint64_t>(kv_heads_local),
                        2, static_cast<cuuint64_t>(num_blocks)};
  cuuint64_t strides[4] = {row_bytes, static_cast<cuuint64_t>(kHd), row_bytes * kTok, row_bytes * kTok * 2};
  cuuint32_t box[5] = {static_cast<cuuint32_t>(kHd), static_cast<cuuint32_t>(kTok), 1, 2, 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 5, const_cast<void*>(cache8), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(FQB_ERR_CUDA, "cuTensorMapEncodeTiled (fp8 cache) failed with CUresult %d", static_cast<int>(r));
  Entry& e = lru[next];
  e.ptr = cache8;
  e.nb = num_blocks;
  e.kvh = kv_heads_local;
  e.map = map;
  next = (next + 1) % kCache;
  if (used < kCache) ++used;
  return FQB_OK;
}

int check_attn_shape(int n_heads, int n_kv, int head_dim, int block_size) {
  if (head_dim != kHd) return set_error(FQB_ERR_SHAPE, "head_dim %d: only 128 is supported", head_dim);
  if (block_size != kTok) return set_error(FQB_ERR_SHAPE, "block_size %d: only 16 is supported", block_size);
  if (n_kv <= 0 || n_heads != n_kv * kGroup)
    return set_error(FQB_ERR_SHAPE, "n_heads %d / n_kv %d: the GQA group must be 4", n_heads, n_kv);
  return FQB_OK;
}

// ---- decode configurations -----------------------------------------------------------------------
// One launch serves HEADS local kv heads (8, 4, 2 or 1; other head counts are covered by several
// launches). A CTA's NW warps form SUB = NW / HEADS groups, each group streams its own segment of the
// flat page list, so a launch of `grid` CTAs cuts the list into grid * SUB segments.
template <int NW_, int NS_, int HEADS_, int MINB_, int MAXD_>
struct DecodeCfg {
  static constexpr int NW = NW_, NS = NS_, HEADS = HEADS_, MINB = MINB_, MAXD = MAXD_, SUB = NW_ / HEADS_;
};
using DecodeCfg8 = DecodeCfg<8, 3, 8, 1, 512>;
using DecodeCfg4 = DecodeCfg<4, 3, 4, 2, 256>;
using DecodeCfg2 = DecodeCfg<4, 3, 2, 2, 256>;
using DecodeCfg1 = DecodeCfg<4, 3, 1, 2, 256>;
// The 1-head shape of launches that wait for nothing: two warps per CTA with rings of 2 and six
// launches resident per SM instead of four warps with rings of 3 and two launches. A launch then cuts the
// page list into half as many segments, so a warp's fixed costs (block-table and TMA round trips before
// its first page, partial, ticket and merge after its last) are spread over twice the pages, and six
// launches at different stages hide them better than two: 11.4 instead of 12.3 us per launch of 68.6 MB
// (one of 8 kv heads, 64 sequences). Rings of 3 with four resident launches measured 11.6 on the same
// GPU, eight resident launches 12.7, three warps per CTA 12.0 (four resident) and 14.6 (three), one warp
// per CTA 12.0-12.1; the same change for the 2-head shape measured no difference, and the 4-head shape
// loses more in the launches that wait (rings of 2) than it gains.
using DecodeCfg1I = DecodeCfg<2, 2, 1, 6, 256>;
// fp8 cache: slices are half the size, so the rings are twice as deep for the same bytes in flight
using Decode8Cfg4 = DecodeCfg<4, 6, 4, 2, 256>;
using Decode8Cfg2 = DecodeCfg<4, 6, 2, 2, 256>;
using Decode8Cfg1 = DecodeCfg<4, 6, 1, 2, 256>;
// fp8 launches that wait for nothing: three CTAs resident per SM instead of two (rings of 4). The fp8
// kernel is bound by the issue rate of its one warp per scheduler (unpacking e4m3 costs instructions, not
// bytes), and 168 registers per thread hold all but 32 bytes of its state, so twelve resident warps
// instead of eight give 5.26 instead of 4.59 TB/s on configuration 2 (0.80 instead of 0.70 of the copy
// peak). The bf16 4-head shape gains nothing from the same change (it is at the copy peak with two).
using Decode8Cfg4I = DecodeCfg<4, 4, 4, 3, 256>;
using Decode8Cfg2I = DecodeCfg<4, 4, 2, 3, 256>;
using Decode8Cfg1I = DecodeCfg<4, 4, 1, 3, 256>;

// CTAs per SM of a default-mode launch of the 4-, 2- and 1-head shapes (build-time choice; measured on
// B200 with every launch waiting for the one before it: 1 beats 2 for the 4-head and the 1-head shape).
#ifndef FQB_DEFAULT_CTAS_PER_SM
#define FQB_DEFAULT_CTAS_PER_SM 1
#endif
constexpr int kDefaultCtas = FQB_DEFAULT_CTAS_PER_SM;

// Most segments any launch of a call makes when its n_kv local heads are covered by launches of 8
// (default mode only), 4, 2 and 1 heads. Default mode: one CTA per SM for the 8-head shape, two for the
// others; overlapped modes: one CTA per SM. The scratch is indexed with the call's n_kv, so the largest
// launch decides.
// Layout of a rank's reassembly control block (32-bit words): flags [slots][world] | publish counters
// [slots] | arrival words [slots] (64-bit, 8-byte aligned).
size_t gather_seq_offset(int slots, int world) { return static_cast<size_t>(slots) * world; }
size_t gather_arrive_offset(int slots, int world) { return (gather_seq_offset(slots, world) + slots + 1) & ~size_t(1); }

int max_segments(int n_kv, int sm_count, bool overlapped, bool fp8 = false) {
  int seg = 0, left = n_kv;
  const int per = overlapped ? 1 : kDefaultCtas;
  if (!overlapped && left >= 8) {
    seg = sm_count * DecodeCfg8::SUB;
    left %= 8;
  }
  if (left >= 4) {
    seg = seg > sm_count * per * DecodeCfg4::SUB ? seg : sm_count * per * DecodeCfg4::SUB;
    left %= 4;
  }
  if (left >= 2) {
    seg = seg > sm_count * per * DecodeCfg2::SUB ? seg : sm_count * per * DecodeCfg2::SUB;
    left %= 2;
  }
  if (left >= 1) {
    const int sub = overlapped && !fp8 ? DecodeCfg1I::SUB : DecodeCfg1::SUB;  // Decode8Cfg1 has DecodeCfg1's groups
    seg = seg > sm_count * per * sub ? seg : sm_count * per * sub;
  }
  return seg;
}

// What a sequence end inside a segment is charged when a launch cuts its page list into segments of equal
// cost, in pages. Measured with every launch waiting for the one before it (fused call, per launch):
// 58.4 -> 51.0 us at 4 local heads, 33.7 -> 30.7 at 2, 25.8 -> 23.7 at 1, 91.0 -> 90.7 at 8; 4 to 8 pages
// give the same within noise, launches that wait for nothing do not change.
constexpr int kEndWeightPages = 6;

unsigned next_epoch() {
  static std::atomic<unsigned> counter{0x5eed0000u};
  unsigned e = ++counter;
  while (e == 0) e = ++counter;
  return e;
}

// Building with -DFQB_NO_PDL turns every launch into a plain one (debugging aid).
constexpr bool pdl_enabled() {
#ifdef FQB_NO_PDL
  return false;
#else
  return true;
#endif
}

// Set by fqb_attn_decode_plan: the next launch this thread makes goes out WITHOUT the programmatic
// attribute, i.e. it starts only when the plan kernel has completed and its writes are visible. Every
// later kernel of the step starts after that one has started, so a plan read in a prologue (before the
// reader's own wait) is always the finished plan. Early starts alone would not give that: a kernel that
// begins at its predecessor's trigger sees only what was visible before the predecessor began.
thread_local bool t_plain_next = false;
thread_local cudaStream_t t_plain_stream = nullptr;  // the stream the plan kernel went to

// Launches `kern` with or without the programmatic-serialization attribute.
template <class... KArgs, class... Args>
cudaError_t launch_ex(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl,
                      Args... args) {
  if (t_plain_next && st == t_plain_stream) {  // a launch on another stream leaves the flag for the plan's stream
    pdl = false;
    t_plain_next = false;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (pdl && pdl_enabled()) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

// Opts the prefill kernel in to its dynamic shared memory once per device and thread, then launches
// (query tiles of 32 rows, kv heads, requests).
int launch_prefill(int max_qlen, int n_kv, int R, const CUtensorMap& map, const PrefillParams& P, cudaStream_t st) {
  using L = TcKsSmem<3>;
  auto kern = prefill_tc_ks_kernel<3>;
  static thread_local int attr_dev = -1;
  int dev = 0;
  FQB_CUDA_TRY(cudaGetDevice(&dev));
  if (attr_dev != dev) {
    FQB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kAlloc));
    attr_dev = dev;
  }
  dim3 grid((max_qlen + kTcGroupRows - 1) / kTcGroupRows, n_kv, R);
  kern<<<grid, L::kThreads, L::kAlloc, st>>>(map, P);
  FQB_CUDA_TRY(cudaGetLastError());
  return FQB_OK;
}

// The build with or without the fused append's code, by whether the call appends.
#define FQB_LAUNCH(Cfg, FP8, ...) \
  (cache_w ? launch_decode<Cfg, FP8, true>(__VA_ARGS__) : launch_decode<Cfg, FP8, false>(__VA_ARGS__))

// ctas_per_sm: how many CTAs of THIS launch go on each SM (the kernel may allow more to be resident,
// so that the CTAs of the launch after it can move in beside them).
template <class Cfg, bool FP8 = false, bool APPEND = true>
int launch_decode(const CUtensorMap& map, DecodeParams P, const int* rids, int n_decode, int sm_count,
                  int ctas_per_sm, bool pdl, cudaStream_t st) {
  using L = DecodeSmem<Cfg::NW, Cfg::NS, Cfg::MAXD, FP8>;
  auto kern = decode_kernel<Cfg::NW, Cfg::NS, Cfg::HEADS, Cfg::MINB, Cfg::MAXD, FP8, APPEND>;
  static thread_local int attr_dev = -1;
  int dev = 0;
  FQB_CUDA_TRY(cudaGetDevice(&dev));
  if (attr_dev != dev) {
    FQB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kAlloc));
    attr_dev = dev;
  }
  int grid = sm_count * ctas_per_sm;
  grid -= grid % P.groups;  // the same number of CTAs for every head group of the launch
  for (int base = 0; base < n_decode; base += Cfg::MAXD) {
    P.rids = rids + base;
    P.n_decode = n_decode - base < Cfg::MAXD ? n_decode - base : Cfg::MAXD;
    const long long need = decode_slots_needed(P.n_decode, P.n_kv, grid / P.groups * Cfg::SUB);
    if (need > P.partial_slots)
      return set_error(FQB_ERR_WORKSPACE, "decode scratch: %lld partial slots needed, %lld given", need,
                       P.partial_slots);
    P.epoch = next_epoch();
    // a second batch of the same call shares the scratch with the first: it must not overlap it
    FQB_CUDA_TRY(launch_ex(kern, dim3(grid), dim3(Cfg::NW * 32), L::kAlloc, st, pdl && base == 0, map, P));
  }
  return FQB_OK;
}

// Independent launches may overlap the launch before them, so consecutive launches must not share
// scratch. The caller's scratch is cut into regions used in rotation; the launch that wraps around
// to region 0 is a plain launch (it waits for everything before it), so a region is never reused
// while an earlier launch could still touch it.
constexpr int kMaxRegions = 64;
struct ScratchTurn {
  const void* key;
  unsigned count;
};
int next_region(const void* key, int regions) {
  constexpr int kTable = 16;
  static thread_local ScratchTurn table[kTable];
  static thread_local int victim = 0;
  for (int i = 0; i < kTable; ++i)
    if (table[i].key == key) return static_cast<int>(table[i].count++ % static_cast<unsigned>(regions));
  table[victim].key = key;
  table[victim].count = 1;
  victim = (victim + 1) % kTable;
  return 0;
}

}  // namespace
}  // namespace fqb

using namespace fqb;

extern "C" {

const char* fqb_version(void) { return "libfqb 0.1 (sm_100a)"; }

int fqb_kv_append(void* cache, int num_blocks, int kv_heads_local, const void* qkv, int src_stride,
                  int k_off, int v_off, const int32_t* bt, int bt_stride, const int32_t* bt_row,
                  const int32_t* pos, int M, void* stream) {
  if (M <= 0) return FQB_OK;
  if (!cache || !qkv || !bt || !bt_row || !pos) return set_error(FQB_ERR_INVALID, "kv_append: null pointer");
  if (num_blocks <= 0 || kv_heads_local <= 0 || bt_stride <= 0)
    return set_error(FQB_ERR_INVALID, "kv_append: non-positive size");
  if (!aligned16(cache) || !aligned16(qkv) || (src_stride % 8) || (k_off % 8) || (v_off % 8))
    return set_error(FQB_ERR_INVALID, "kv_append: pointers, src_stride, k_off and v_off must keep 16-byte alignment");
  AppendParams P{static_cast<__nv_bfloat16*>(cache), num_blocks, kv_heads_local * kHd,
                 static_cast<const __nv_bfloat16*>(qkv), src_stride, k_off, v_off, bt, bt_stride, bt_row, pos, M};
  FQB_CUDA_TRY(launch_ex(kv_append_kernel, dim3(M), dim3(256), 0, static_cast<cudaStream_t>(stream), true, P));
  return FQB_OK;
}

int fqb_norm_rope_append(void* cache, int num_blocks, int kv_heads_local, int q_heads_local, void* qkv,
                         int src_stride, int q_off, int k_off, int v_off, const float* wq, const float* wk,
                         const float* cos_tab, const float* sin_tab, float eps, const int32_t* bt,
                         int bt_stride, const int32_t* bt_row, const int32_t* pos, int M, void* stream) {
  if (M <= 0) return FQB_OK;
  // cache == NULL: RMSNorm + RoPE only (LaunchHeadNormRope alone); bt / bt_row are then not read
  if (!qkv || !pos || !wq || !wk || !cos_tab || !sin_tab || (cache && (!bt || !bt_row)))
    return set_error(FQB_ERR_INVALID, "norm_rope_append: null pointer");
  if (kv_heads_local <= 0 || q_heads_local < 0 || (cache && (num_blocks <= 0 || bt_stride <= 0)))
    return set_error(FQB_ERR_INVALID, "norm_rope_append: non-positive size");
  if (!aligned16(cache) || !aligned16(qkv) || (src_stride % 8) || (q_off % 8) || (k_off % 8) || (v_off % 8) ||
      (reinterpret_cast<uintptr_t>(cos_tab) & 7u) || (reinterpret_cast<uintptr_t>(sin_tab) & 7u) ||
      (reinterpret_cast<uintptr_t>(wq) & 7u) || (reinterpret_cast<uintptr_t>(wk) & 7u))
    return set_error(FQB_ERR_INVALID, "norm_rope_append: misaligned pointer or offset");
  NormRopeParams P;
  P.a = AppendParams{static_cast<__nv_bfloat16*>(cache), num_blocks, kv_heads_local * kHd,
                     static_cast<const __nv_bfloat16*>(qkv), src_stride, k_off, v_off, bt, bt_stride, bt_row, pos, M};
  P.q_heads = q_heads_local;
  P.kv_heads = kv_heads_local;
  P.q_off = q_off;
  P.wq = wq;
  P.wk = wk;
  P.cos_tab = cos_tab;
  P.sin_tab = sin_tab;
  P.eps = eps;
  FQB_CUDA_TRY(launch_ex(norm_rope_append_kernel, dim3(M), dim3(256), 0, static_cast<cudaStream_t>(stream), true, P));
  return FQB_OK;
}

int64_t fqb_attn_decode_partial_slots(int max_decode, int n_heads_local, int max_blocks) {
  (void)max_blocks;  // the split count follows the SM count, not the context length
  if (max_decode <= 0 || n_heads_local <= 0) return 0;
  // One region holds the partials of (sequences + segments) pieces plus the arrival counters of a
  // launch of at most 512 sequences. Overlapping launches rotate through
  // regions; re-entering the first one is a sync point whose cost is shared by all regions, so
  // give as many as fit in about 128 Ki slots (64 MiB of pa), at least 16, at most 64.
  const int n_kv = n_heads_local / kGroup;
  // sized for a GPU of up to 256 SMs
  const long long one =
      (decode_slots_needed(max_decode < 512 ? max_decode : 512, n_kv, max_segments(n_kv, 256, false)) + 3) & ~3LL;
  long long regions = (128 * 1024) / one;
  if (regions < 16) regions = 16;
  if (regions > kMaxRegions) regions = kMaxRegions;
  return regions * one;
}

static int decode_impl(const void* q, int q_stride, const void* cache, int num_blocks, void* out, int n_heads,
                       int n_kv, int head_dim, const int32_t* pos, const int32_t* qstart,
                       const int32_t* decode_rids, int n_decode, const int32_t* bt, int max_blocks, int block_size,
                       float scale, float* pm, float* pl, float* pa, int64_t partial_slots, unsigned flags,
                       const int32_t* plan, void* cache_w, long long k_rel, long long v_rel, const fqb_gather* gather,
                       const float* scales, void* stream);

int64_t fqb_kv_pool_bytes_fp8(int num_blocks, int kv_heads_local) {
  if (num_blocks <= 0 || kv_heads_local <= 0) return 0;
  return static_cast<int64_t>(num_blocks) * FQB_PLANES * kTok * kv_heads_local * kHd;
}
int64_t fqb_kv_scale_bytes_fp8(int num_blocks, int kv_heads_local) {
  if (num_blocks <= 0 || kv_heads_local <= 0) return 0;
  return static_cast<int64_t>(num_blocks) * kv_heads_local * FQB_PLANES * kTok * 4;
}

int fqb_kv_append_fp8(void* cache8, float* scales, int num_blocks, int kv_heads_local, const void* qkv, int src_stride,
                      int k_off, int v_off, const int32_t* bt, int bt_stride, const int32_t* bt_row, const int32_t* pos,
                      int M, void* stream) {
  if (M <= 0) return FQB_OK;
  if (!cache8 || !scales || !qkv || !bt || !bt_row || !pos) return set_error(FQB_ERR_INVALID, "kv_append_fp8: null pointer");
  if (num_blocks <= 0 || kv_heads_local <= 0 || bt_stride <= 0)
    return set_error(FQB_ERR_INVALID, "kv_append_fp8: non-positive size");
  if (!aligned16(cache8) || !aligned16(scales) || !aligned16(qkv) || (src_stride % 8) || (k_off % 8) || (v_off % 8))
    return set_error(FQB_ERR_INVALID, "kv_append_fp8: pointers, src_stride, k_off and v_off must keep 16-byte alignment");
  AppendParams P{static_cast<__nv_bfloat16*>(cache8), num_blocks, kv_heads_local * kHd,
                 static_cast<const __nv_bfloat16*>(qkv), src_stride, k_off, v_off, bt, bt_stride, bt_row, pos, M};
  FQB_CUDA_TRY(launch_ex(kv_append_fp8_kernel, dim3(M), dim3(256), 0, static_cast<cudaStream_t>(stream), true, P, scales));
  return FQB_OK;
}

int fqb_dequant_blocks_fp8(const void* cache8, const float* scales, int num_blocks, int kv_heads_local,
                           const int32_t* list, int n, void* out, void* stream) {
  if (n <= 0) return FQB_OK;
  if (!cache8 || !scales || !list || !out) return set_error(FQB_ERR_INVALID, "dequant_blocks_fp8: null pointer");
  if (num_blocks <= 0 || kv_heads_local <= 0) return set_error(FQB_ERR_INVALID, "dequant_blocks_fp8: non-positive size");
  if (!aligned16(cache8) || !aligned16(scales) || !aligned16(out))
    return set_error(FQB_ERR_INVALID, "dequant_blocks_fp8: misaligned pointer");
  if (n > 2147483647 / 2) return set_error(FQB_ERR_SHAPE, "dequant_blocks_fp8: too many blocks");
  // a block has 32 (plane, token) rows, one per warp: four CTAs of eight warps
  dequant_blocks_fp8_kernel<<<dim3(n, 4), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(cache8), scales, num_blocks, kv_heads_local, list, static_cast<__nv_bfloat16*>(out));
  FQB_CUDA_TRY(cudaGetLastError());
  return FQB_OK;
}

int fqb_attn_decode_fp8(const void* q, int q_stride, const void* cache8, const float* scales, int num_blocks, void* out,
                        int n_heads, int n_kv, int head_dim, const int32_t* pos, const int32_t* qstart,
                        const int32_t* decode_rids, int n_decode, const int32_t* bt, int max_blocks, int block_size,
                        float scale, float* pm, float* pl, float* pa, int64_t partial_slots, unsigned flags,
                        void* stream) {
  if (n_decode <= 0) return FQB_OK;
  if (!scales) return set_error(FQB_ERR_INVALID, "attn_decode_fp8: null pointer");
  if (flags & FQB_DECODE_HISTORY_STABLE)
    return set_error(FQB_ERR_INVALID, "attn_decode_fp8: FQB_DECODE_HISTORY_STABLE belongs to fqb_append_attn_decode");
  return decode_impl(q, q_stride, cache8, num_blocks, out, n_heads, n_kv, head_dim, pos, qstart, decode_rids, n_decode,
                     bt, max_blocks, block_size, scale, pm, pl, pa, partial_slots, flags, nullptr, nullptr, 0, 0, nullptr,
                     scales, stream);
}

int64_t fqb_attn_decode_slots_needed(int n_decode, int n_kv) {
  if (n_decode <= 0 || n_kv <= 0) return 0;
  DeviceInfo di;
  if (int rc = device_info(di)) return rc;
  return decode_slots_needed(n_decode < 512 ? n_decode : 512, n_kv, max_segments(n_kv, di.sm_count, false));
}

int fqb_attn_decode_plan(const int32_t* pos, const int32_t* qstart, const int32_t* decode_rids, int n_decode,
                         int max_blocks, int32_t* plan, void* stream) {
  if (n_decode <= 0) return FQB_OK;
  if (!pos || !qstart || !decode_rids || !plan) return set_error(FQB_ERR_INVALID, "attn_decode_plan: null pointer");
  if (n_decode > FQB_PLAN_MAX_DECODE)
    return set_error(FQB_ERR_SHAPE, "attn_decode_plan: %d sequences, at most %d", n_decode, FQB_PLAN_MAX_DECODE);
  if (reinterpret_cast<uintptr_t>(plan) & 15u) return set_error(FQB_ERR_INVALID, "attn_decode_plan: plan must be 16-byte aligned");
  decode_plan_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(pos, qstart, decode_rids, n_decode, max_blocks,
                                                                        plan);
  FQB_CUDA_TRY(cudaGetLastError());
  t_plain_next = true;
  t_plain_stream = static_cast<cudaStream_t>(stream);
  return FQB_OK;
}

// cache_w != nullptr: the launch also appends the new token's K / V rows (fqb_append_attn_decode).
static int decode_impl(const void* q, int q_stride, const void* cache, int num_blocks, void* out, int n_heads,
                       int n_kv, int head_dim, const int32_t* pos, const int32_t* qstart,
                       const int32_t* decode_rids, int n_decode, const int32_t* bt, int max_blocks, int block_size,
                       float scale, float* pm, float* pl, float* pa, int64_t partial_slots, unsigned flags,
                       const int32_t* plan, void* cache_w, long long k_rel, long long v_rel, const fqb_gather* gather,
                       const float* scales, void* stream) {
  if (n_decode <= 0 && !gather) return FQB_OK;
  const bool fp8 = scales != nullptr;
  if (plan && (n_decode > 256 || (reinterpret_cast<uintptr_t>(plan) & 15u)))
    return set_error(FQB_ERR_INVALID, "attn_decode: a step plan serves at most 256 sequences per call and must be 16-byte aligned");
  if (int rc = check_attn_shape(n_heads, n_kv, head_dim, block_size)) return rc;
  if (!q || !cache || !out || !pos || !qstart || !decode_rids || !bt || !pm || !pl || !pa)
    return set_error(FQB_ERR_INVALID, "attn_decode: null pointer");
  if (num_blocks <= 0 || max_blocks <= 0 || partial_slots <= 0)
    return set_error(FQB_ERR_INVALID, "attn_decode: non-positive size");
  if (!(scale > 0.f) || !std::isfinite(scale))
    return set_error(FQB_ERR_INVALID, "attn_decode: the softmax scale must be positive and finite");
  if (!aligned16(q) || !aligned16(cache) || !aligned16(out) || !aligned16(pa) || (q_stride % 8) ||
      (reinterpret_cast<uintptr_t>(pl) & 7u) || (reinterpret_cast<uintptr_t>(pm) & 3u))
    return set_error(FQB_ERR_INVALID, "attn_decode: q, cache, out, pa and q_stride must keep 16-byte alignment, pl 8");
  if ((flags & FQB_DECODE_INDEPENDENT) && (flags & FQB_DECODE_HISTORY_STABLE))
    return set_error(FQB_ERR_INVALID, "attn_decode: FQB_DECODE_INDEPENDENT and FQB_DECODE_HISTORY_STABLE exclude each other");
  DeviceInfo di;
  if (int rc = device_info(di)) return rc;
  CUtensorMap map;
  if (int rc = fp8 ? make_cache_map_fp8(cache, num_blocks, n_kv, map) : make_cache_map(cache, num_blocks, n_kv, map)) return rc;
  if (fp8 && (!aligned16(scales) || (q_stride % 8)))
    return set_error(FQB_ERR_INVALID, "attn_decode_fp8: scales and q rows must keep 16-byte alignment");
  DecodeParams P;
  P.q = static_cast<const __nv_bfloat16*>(q);
  P.q_stride = q_stride;
  P.out = static_cast<__nv_bfloat16*>(out);
  P.n_heads = n_heads;
  P.n_kv = n_kv;
  P.scales = scales;
  P.scales_w = cache_w ? const_cast<float*>(scales) : nullptr;  // the fused fp8 append writes the token's scales
  P.pos = pos;
  P.qstart = qstart;
  P.rids = decode_rids;
  P.n_decode = n_decode;
  P.bt = bt;
  P.max_blocks = max_blocks;
  P.num_blocks = num_blocks;
  P.scale_log2 = scale * kLog2e;
  P.pm = pm;
  P.pl = pl;
  P.pa = pa;
  P.partial_slots = partial_slots;
  P.mode = kDecodeWaitFirst;
  P.sync_first = 0;
  P.end_weight = kEndWeightPages;
  P.groups = 1;
  P.plan = plan;
  P.cache_w = static_cast<__nv_bfloat16*>(cache_w);
  P.k_rel = k_rel;
  P.v_rel = v_rel;
  P.n_peers = 0;
  if (gather) {
    const fqb_gather& g = *gather;
    if (g.world < 1 || g.world > kMaxPeers || g.rank < 0 || g.rank >= g.world || g.slot < 0 || g.slot >= g.slots ||
        !g.control)
      return set_error(FQB_ERR_INVALID, "attn_decode: bad reassembly descriptor (world %d, rank %d, slot %d of %d)",
                       g.world, g.rank, g.slot, g.slots);
    if (n_decode <= 0 || n_decode > 256 || (n_kv != 1 && n_kv != 2 && n_kv != 4))
      return set_error(FQB_ERR_SHAPE, "attn_decode: reassembly takes calls that go out as ONE launch: 1 to 256 "
                                      "sequences and 1, 2 or 4 local kv heads (got %d, %d)", n_decode, n_kv);
    P.n_peers = g.world;
    for (int r = 0; r < g.world; ++r) {
      if (!g.out[r] || !g.flags[r] || !aligned16(g.out[r]))
        return set_error(FQB_ERR_INVALID, "attn_decode: reassembly pointer of rank %d missing or misaligned", r);
      P.peer_out[r] = static_cast<__nv_bfloat16*>(g.out[r]);
      P.peer_flag[r] = static_cast<unsigned*>(g.flags[r]) + static_cast<size_t>(g.slot) * g.world + g.rank;
    }
    P.peer_heads = g.world * n_heads;
    P.peer_col = g.rank * n_heads;
    unsigned* ctl = static_cast<unsigned*>(g.control);
    P.seq = ctl + gather_seq_offset(g.slots, g.world) + g.slot;
    P.arrive = (flags & FQB_GATHER_PUBLISH_LATER)
                   ? nullptr
                   : reinterpret_cast<unsigned long long*>(ctl + gather_arrive_offset(g.slots, g.world)) + g.slot;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  // ---- launches that wait for nothing: one CTA per SM per launch, two launches resident side by side (four
  // of the 1-head shape) ----
  // Such a launch may touch the scratch while the launch before it still merges its partials, so
  // consecutive launches rotate through regions of the scratch.
  if ((flags & FQB_DECODE_INDEPENDENT) && pdl_enabled() && n_decode <= 256) {
    const int64_t need = (decode_slots_needed(n_decode, n_kv, max_segments(n_kv, di.sm_count, true, fp8)) + 3) & ~int64_t(3);
    int regions = static_cast<int>(partial_slots / need);
    if (regions > kMaxRegions) regions = kMaxRegions;
    if (regions >= 2) {
      const int region = next_region(pm, regions);
      P.pm = pm + region * need;
      P.pl = pl + region * need;
      P.pa = pa + region * need * kHd;
      P.partial_slots = need;
      P.mode = kDecodeNoWait;
      // The launch that re-enters region 0 waits for all earlier kernels before it lets the next
      // launch start (sync_first): a region is reused one full rotation later, and between any launch and
      // its region's previous user lies such a sync point, so the earlier user has always completed.
      P.sync_first = region == 0 ? 1 : 0;
      const bool pdl = true;
      for (int base = 0; base < n_kv;) {
        const int left = n_kv - base;
        P.kvh_base = base;
        int rc, took;
        if (left >= 4) { rc = fp8 ? FQB_LAUNCH(Decode8Cfg4I, true, map, P, decode_rids, n_decode, di.sm_count, 1, pdl, st) : FQB_LAUNCH(DecodeCfg4, false, map, P, decode_rids, n_decode, di.sm_count, 1, pdl, st); took = 4; }
        else if (left >= 2) { rc = fp8 ? FQB_LAUNCH(Decode8Cfg2I, true, map, P, decode_rids, n_decode, di.sm_count, 1, pdl, st) : FQB_LAUNCH(DecodeCfg2, false, map, P, decode_rids, n_decode, di.sm_count, 1, pdl, st); took = 2; }
        else { rc = fp8 ? FQB_LAUNCH(Decode8Cfg1I, true, map, P, decode_rids, n_decode, di.sm_count, 1, pdl, st) : FQB_LAUNCH(DecodeCfg1I, false, map, P, decode_rids, n_decode, di.sm_count, 1, pdl, st); took = 1; }
        if (rc != FQB_OK) return rc;
        base += took;
        P.sync_first = 0;  // later launches of the call serve other heads: disjoint partials and counters
      }
      return FQB_OK;
    }
  }

  // ---- FQB_DECODE_HISTORY_STABLE: the default geometry below, but every warp requests its first pages
  // BEFORE it waits for the kernel in front. Nothing but the page ring is touched before that wait (the
  // scratch, q and `out` after it), so the scratch needs no rotation. A call that needs several launches
  // (5, 6, 7 ... heads) lets only the first one start early: the later ones follow a launch of this same
  // call, which writes the cache.
  if ((flags & FQB_DECODE_HISTORY_STABLE) && pdl_enabled()) P.mode = kDecodeWaitRows;

  // ---- default: the launch waits for the kernel before it after its metadata prologue ----
  // cover the local heads with launches of 8, 4, 2 or 1 heads (one launch for 8, 4, 2, 1 heads)
  for (int base = 0; base < n_kv;) {
    const int left = n_kv - base;
    P.kvh_base = base;
    int rc, took;
    if (left >= 8 && fp8) {
      // fp8, 8 heads, the launch waits: two head groups of four heads in one launch, three 4-warp CTAs per
      // SM (12 warps where the 8-head shape has 8; the kernel is bound by its issue rate, see Decode8Cfg4I)
      P.groups = 2;
      rc = FQB_LAUNCH(Decode8Cfg4I, true, map, P, decode_rids, n_decode, di.sm_count, 3, true, st);
      P.groups = 1;
      took = 8;
    }
    else if (left >= 8) { rc = FQB_LAUNCH(DecodeCfg8, false, map, P, decode_rids, n_decode, di.sm_count, 1, true, st); took = 8; }
    else if (left >= 4) { rc = fp8 ? FQB_LAUNCH(Decode8Cfg4, true, map, P, decode_rids, n_decode, di.sm_count, kDefaultCtas, true, st) : FQB_LAUNCH(DecodeCfg4, false, map, P, decode_rids, n_decode, di.sm_count, kDefaultCtas, true, st); took = 4; }
    else if (left >= 2) { rc = fp8 ? FQB_LAUNCH(Decode8Cfg2, true, map, P, decode_rids, n_decode, di.sm_count, kDefaultCtas, true, st) : FQB_LAUNCH(DecodeCfg2, false, map, P, decode_rids, n_decode, di.sm_count, kDefaultCtas, true, st); took = 2; }
    else { rc = fp8 ? FQB_LAUNCH(Decode8Cfg1, true, map, P, decode_rids, n_decode, di.sm_count, kDefaultCtas, true, st) : FQB_LAUNCH(DecodeCfg1, false, map, P, decode_rids, n_decode, di.sm_count, kDefaultCtas, true, st); took = 1; }
    if (rc != FQB_OK) return rc;
    base += took;
    P.mode = kDecodeWaitFirst;
  }
  return FQB_OK;
}

int fqb_attn_decode_ex(const void* q, int q_stride, const void* cache, int num_blocks, void* out, int n_heads,
                       int n_kv, int head_dim, const int32_t* pos, const int32_t* qstart,
                       const int32_t* decode_rids, int n_decode, const int32_t* bt, int max_blocks, int block_size,
                       float scale, float* pm, float* pl, float* pa, int64_t partial_slots, unsigned flags,
                       void* stream) {
  if (flags & FQB_DECODE_HISTORY_STABLE)
    return set_error(FQB_ERR_INVALID, "attn_decode: FQB_DECODE_HISTORY_STABLE belongs to fqb_append_attn_decode "
                                      "(a separate append kernel in front writes the cache this call reads)");
  return decode_impl(q, q_stride, cache, num_blocks, out, n_heads, n_kv, head_dim, pos, qstart, decode_rids, n_decode,
                     bt, max_blocks, block_size, scale, pm, pl, pa, partial_slots, flags, nullptr, nullptr, 0, 0, nullptr, nullptr, stream);
}

int fqb_attn_decode_planned(const void* q, int q_stride, const void* cache, int num_blocks, void* out, int n_heads,
                            int n_kv, int head_dim, const int32_t* plan, int n_decode, const int32_t* bt,
                            int max_blocks, int block_size, float scale, float* pm, float* pl, float* pa,
                            int64_t partial_slots, unsigned flags, void* stream) {
  if (n_decode > 0 && !plan) return set_error(FQB_ERR_INVALID, "attn_decode_planned: null plan");
  if (flags & FQB_DECODE_HISTORY_STABLE)
    return set_error(FQB_ERR_INVALID, "attn_decode_planned: FQB_DECODE_HISTORY_STABLE belongs to fqb_append_attn_decode");
  // pos / qstart / decode_rids are not read when a plan is given; the plan pointer stands in for them
  return decode_impl(q, q_stride, cache, num_blocks, out, n_heads, n_kv, head_dim, plan, plan, plan, n_decode, bt,
                     max_blocks, block_size, scale, pm, pl, pa, partial_slots, flags, plan, nullptr, 0, 0, nullptr, nullptr, stream);
}

int fqb_attn_decode(const void* q, int q_stride, const void* cache, int num_blocks, void* out, int n_heads,
                    int n_kv, int head_dim, const int32_t* pos, const int32_t* qstart, const int32_t* decode_rids,
                    int n_decode, const int32_t* bt, int max_blocks, int block_size, float scale, float* pm,
                    float* pl, float* pa, int64_t partial_slots, void* stream) {
  return fqb_attn_decode_ex(q, q_stride, cache, num_blocks, out, n_heads, n_kv, head_dim, pos, qstart, decode_rids,
                            n_decode, bt, max_blocks, block_size, scale, pm, pl, pa, partial_slots, 0u, stream);
}

static int append_decode(void* cache, int num_blocks, int kv_heads_local, const void* qkv, int src_stride, int q_off,
                         int k_off, int v_off, void* out, int head_dim, const int32_t* pos, const int32_t* qstart,
                         const int32_t* decode_rids, const int32_t* plan, int n_decode, const int32_t* bt,
                         int max_blocks, int block_size, float scale, float* pm, float* pl, float* pa,
                         int64_t partial_slots, unsigned flags, const fqb_gather* gather, float* scales, void* stream) {
  if (n_decode <= 0 && !gather) return FQB_OK;
  if (!qkv) return set_error(FQB_ERR_INVALID, "append_attn_decode: null pointer");
  if (!aligned16(qkv) || (src_stride % 8) || (q_off % 8) || (k_off % 8) || (v_off % 8) || q_off < 0 || k_off < 0 || v_off < 0)
    return set_error(FQB_ERR_INVALID, "append_attn_decode: qkv, src_stride, q_off, k_off and v_off must keep 16-byte alignment");
  if (!plan && (!pos || !qstart || !decode_rids))
    return set_error(FQB_ERR_INVALID, "append_attn_decode: give pos / qstart / decode_rids or a step plan");
  const __nv_bfloat16* q = static_cast<const __nv_bfloat16*>(qkv) + q_off;
  const int32_t* m0 = plan ? plan : pos;
  const int32_t* m1 = plan ? plan : qstart;
  const int32_t* m2 = plan ? plan : decode_rids;
  return decode_impl(q, src_stride, cache, num_blocks, out, kv_heads_local * kGroup, kv_heads_local, head_dim, m0, m1, m2,
                     n_decode, bt, max_blocks, block_size, scale, pm, pl, pa, partial_slots, flags, plan, cache,
                     static_cast<long long>(k_off) - q_off, static_cast<long long>(v_off) - q_off, gather, scales, stream);
}

int fqb_append_attn_decode(void* cache, int num_blocks, int kv_heads_local, const void* qkv, int src_stride, int q_off,
                           int k_off, int v_off, void* out, int head_dim, const int32_t* pos, const int32_t* qstart,
                           const int32_t* decode_rids, const int32_t* plan, int n_decode, const int32_t* bt,
                           int max_blocks, int block_size, float scale, float* pm, float* pl, float* pa,
                           int64_t partial_slots, unsigned flags, void* stream) {
  return append_decode(cache, num_blocks, kv_heads_local, qkv, src_stride, q_off, k_off, v_off, out, head_dim, pos, qstart,
                       decode_rids, plan, n_decode, bt, max_blocks, block_size, scale, pm, pl, pa, partial_slots, flags,
                       nullptr, nullptr, stream);
}

int fqb_append_attn_decode_fp8(void* cache8, float* scales, int num_blocks, int kv_heads_local, const void* qkv,
                               int src_stride, int q_off, int k_off, int v_off, void* out, int head_dim,
                               const int32_t* pos, const int32_t* qstart, const int32_t* decode_rids, const int32_t* plan,
                               int n_decode, const int32_t* bt, int max_blocks, int block_size, float scale, float* pm,
                               float* pl, float* pa, int64_t partial_slots, unsigned flags, void* stream) {
  if (n_decode <= 0) return FQB_OK;
  if (!scales) return set_error(FQB_ERR_INVALID, "append_attn_decode_fp8: null pointer");
  return append_decode(cache8, num_blocks, kv_heads_local, qkv, src_stride, q_off, k_off, v_off, out, head_dim, pos, qstart,
                       decode_rids, plan, n_decode, bt, max_blocks, block_size, scale, pm, pl, pa, partial_slots, flags,
                       nullptr, scales, stream);
}

int fqb_append_attn_decode_gather(void* cache, int num_blocks, int kv_heads_local, const void* qkv, int src_stride,
                                  int q_off, int k_off, int v_off, void* out, int head_dim, const int32_t* pos,
                                  const int32_t* qstart, const int32_t* decode_rids, const int32_t* plan, int n_decode,
                                  const int32_t* bt, int max_blocks, int block_size, float scale, float* pm, float* pl,
                                  float* pa, int64_t partial_slots, unsigned flags, const fqb_gather* gather,
                                  void* stream) {
  if (!gather) return set_error(FQB_ERR_INVALID, "append_attn_decode_gather: null reassembly descriptor");
  return append_decode(cache, num_blocks, kv_heads_local, qkv, src_stride, q_off, k_off, v_off, out, head_dim, pos, qstart,
                       decode_rids, plan, n_decode, bt, max_blocks, block_size, scale, pm, pl, pa, partial_slots, flags,
                       gather, nullptr, stream);
}

int64_t fqb_gather_control_bytes(int slots, int world) {
  if (slots <= 0 || world <= 0 || world > kMaxPeers) return 0;
  return static_cast<int64_t>(gather_arrive_offset(slots, world)) * 4 + static_cast<int64_t>(slots) * 8;
}

int fqb_gather_wait(const fqb_gather* g, void* stream) {
  if (!g || !g->control || g->world < 1 || g->world > kMaxPeers || g->slot < 0 || g->slot >= g->slots)
    return set_error(FQB_ERR_INVALID, "gather_wait: bad reassembly descriptor");
  const unsigned* ctl = static_cast<const unsigned*>(g->control);
  const unsigned long long limit_ns = static_cast<unsigned long long>(g->timeout_ms > 0 ? g->timeout_ms : 1000) * 1000000ull;
  FQB_CUDA_TRY(launch_ex(gather_wait_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), true,
                         ctl + static_cast<size_t>(g->slot) * g->world, ctl + gather_seq_offset(g->slots, g->world) + g->slot,
                         g->world, limit_ns));
  return FQB_OK;
}

int fqb_gather_wait_all(const fqb_gather* g, void* stream) {
  if (!g || !g->control || g->world < 1 || g->world > kMaxPeers || g->slots < 1)
    return set_error(FQB_ERR_INVALID, "gather_wait_all: bad reassembly descriptor");
  const unsigned* ctl = static_cast<const unsigned*>(g->control);
  const unsigned long long limit_ns = static_cast<unsigned long long>(g->timeout_ms > 0 ? g->timeout_ms : 1000) * 1000000ull;
  FQB_CUDA_TRY(launch_ex(gather_wait_all_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), true, ctl,
                         ctl + gather_seq_offset(g->slots, g->world), g->slots, g->world, limit_ns));
  return FQB_OK;
}

int fqb_gather_publish_all(const fqb_gather* g, void* stream) {
  if (!g || !g->control || g->world < 1 || g->world > kMaxPeers || g->rank < 0 || g->rank >= g->world || g->slots < 1)
    return set_error(FQB_ERR_INVALID, "gather_publish_all: bad reassembly descriptor");
  PublishAllParams P;
  unsigned* ctl = static_cast<unsigned*>(g->control);
  P.seq = ctl + gather_seq_offset(g->slots, g->world);
  for (int r = 0; r < kMaxPeers; ++r) P.flags[r] = nullptr;
  for (int r = 0; r < g->world; ++r) {
    if (!g->flags[r]) return set_error(FQB_ERR_INVALID, "gather_publish_all: control block of rank %d missing", r);
    P.flags[r] = static_cast<unsigned*>(g->flags[r]);
  }
  P.slots = g->slots;
  P.world = g->world;
  P.rank = g->rank;
  // a plain launch: it starts when every earlier kernel of the stream has completed
  gather_publish_all_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(P);
  FQB_CUDA_TRY(cudaGetLastError());
  return FQB_OK;
}

// ---- set-up helpers for the reassembly buffers: memory another process on this node can map ----
int fqb_peer_alloc(int64_t bytes, void** ptr) {
  if (bytes <= 0 || !ptr) return set_error(FQB_ERR_INVALID, "peer_alloc: bad arguments");
  FQB_CUDA_TRY(cudaMalloc(ptr, static_cast<size_t>(bytes)));
  FQB_CUDA_TRY(cudaMemset(*ptr, 0, static_cast<size_t>(bytes)));
  return FQB_OK;
}
int fqb_peer_free(void* ptr) {
  if (ptr) FQB_CUDA_TRY(cudaFree(ptr));
  return FQB_OK;
}
int fqb_peer_export(void* ptr, void* handle64) {
  static_assert(sizeof(cudaIpcMemHandle_t) == FQB_PEER_HANDLE_BYTES, "handle size");
  if (!ptr || !handle64) return set_error(FQB_ERR_INVALID, "peer_export: null pointer");
  cudaIpcMemHandle_t h;
  FQB_CUDA_TRY(cudaIpcGetMemHandle(&h, ptr));
  std::memcpy(handle64, &h, sizeof h);
  return FQB_OK;
}
int fqb_peer_open(const void* handle64, void** ptr) {
  if (!handle64 || !ptr) return set_error(FQB_ERR_INVALID, "peer_open: null pointer");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, sizeof h);
  FQB_CUDA_TRY(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return FQB_OK;
}
int fqb_peer_close(void* ptr) {
  if (ptr) FQB_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
  return FQB_OK;
}

// ---- decode attention for callers that cannot provide scratch -------------------------------------
// Scratch of fqb_attn_decode_static: pm | pl | pa for kStaticSlots partial slots, 4.06 MiB, part of
// the library image on every GPU that loads it. Device code could name the array directly; host
// code cannot -- on the host the symbol is only a stand-in -- so its device address is looked up
// once per device with cudaGetSymbolAddress and handed to the kernel like any caller's scratch.
constexpr long long kStaticSlots = 8192;
static __device__ __align__(256) float g_decode_static_scratch[kStaticSlots * (2 + FQB_HEAD_DIM)];

namespace fqb {
namespace {
int static_scratch_address(float** out) {
  static std::mutex mu;
  static float* addr[64] = {};
  int dev = 0;
  FQB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return set_error(FQB_ERR_CUDA, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lk(mu);
  if (!addr[dev]) {
    float* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_decode_static_scratch);
    if (e != cudaSuccess || !p)
      return set_error(FQB_ERR_CUDA, "attn_decode_static: cudaGetSymbolAddress failed on device %d: %s", dev,
                       cudaGetErrorString(e));
    addr[dev] = p;
  }
  *out = addr[dev];
  return FQB_OK;
}
}  // namespace
}  // namespace fqb

int fqb_attn_decode_static(const void* q, int q_stride, const void* cache, int num_blocks, void* out, int n_heads,
                           int n_kv, int head_dim, const int32_t* pos, const int32_t* qstart,
                           const int32_t* decode_rids, int n_decode, const int32_t* bt, int max_blocks,
                           int block_size, float scale, void* stream) {
  if (n_decode <= 0) return FQB_OK;
  // what the launches of this call would need, worked out before anything is launched
  DeviceInfo di;
  if (int rc = device_info(di)) return rc;
  const long long need = n_kv > 0 ? decode_slots_needed(n_decode, n_kv, max_segments(n_kv, di.sm_count, false)) : 0;
  if (n_decode > FQB_STATIC_MAX_DECODE || n_kv > FQB_STATIC_MAX_KV_HEADS || need > kStaticSlots)
    return set_error(FQB_ERR_WORKSPACE,
                     "attn_decode_static: %d sequences x %d kv heads is beyond the built-in scratch (at most %d "
                     "sequences; 1, 2, 4 or 8 kv heads; %lld of %lld partial slots needed on this GPU); use "
                     "fqb_attn_decode with your own scratch",
                     n_decode, n_kv, FQB_STATIC_MAX_DECODE, need, kStaticSlots);
  float* base = nullptr;
  if (int rc = fqb::static_scratch_address(&base)) return rc;
  // the arrival counters inside the scratch are tagged with a per-launch number, so nothing has to
  // be zeroed between calls even though the array keeps the previous call's contents
  return fqb_attn_decode_ex(q, q_stride, cache, num_blocks, out, n_heads, n_kv, head_dim, pos, qstart, decode_rids,
                            n_decode, bt, max_blocks, block_size, scale, base, base + kStaticSlots,
                            base + 2 * kStaticSlots, kStaticSlots, 0u, stream);
}

int fqb_attn_prefill(const void* q, int q_stride, const void* cache, int num_blocks, void* out, int n_heads,
                     int n_kv, int head_dim, const int32_t* pos, const int32_t* qstart, const int32_t* qlen,
                     const int32_t* rids, int R, int max_qlen, const int32_t* bt, int max_blocks, int block_size,
                     float scale, void* stream) {
  if (R <= 0) return FQB_OK;
  if (int rc = check_attn_shape(n_heads, n_kv, head_dim, block_size)) return rc;
  if (!q || !cache || !out || !pos || !qstart || !qlen || !rids || !bt)
    return set_error(FQB_ERR_INVALID, "attn_prefill: null pointer");
  if (num_blocks <= 0 || max_blocks <= 0 || max_qlen <= 0)
    return set_error(FQB_ERR_INVALID, "attn_prefill: non-positive size");
  if (!aligned16(cache)) return set_error(FQB_ERR_INVALID, "attn_prefill: misaligned cache pointer");
  if (!(scale > 0.f) || !std::isfinite(scale))
    return set_error(FQB_ERR_INVALID, "attn_prefill: the softmax scale must be positive and finite");
  if (n_kv > 65535 || R > 65535) return set_error(FQB_ERR_SHAPE, "attn_prefill: n_kv or R above 65535");
  if (!aligned16(q) || !aligned16(out) || (q_stride % 8))
    return set_error(FQB_ERR_INVALID, "attn_prefill: q, out and q_stride must keep 16-byte alignment");
  CUtensorMap map;
  if (int rc = make_cache_map(cache, num_blocks, n_kv, map, true)) return rc;
  PrefillParams P;
  P.q = static_cast<const __nv_bfloat16*>(q);
  P.q_stride = q_stride;
  P.out = static_cast<__nv_bfloat16*>(out);
  P.n_heads = n_heads;
  P.n_kv = n_kv;
  P.pos = pos;
  P.qstart = qstart;
  P.qlen = qlen;
  P.rids = rids;
  P.bt = bt;
  P.max_blocks = max_blocks;
  P.num_blocks = num_blocks;
  P.scale_log2 = scale * kLog2e;
  return launch_prefill(max_qlen, n_kv, R, map, P, static_cast<cudaStream_t>(stream));
}

static int block_move(void* const* layers, int n_layers, void* cache, void* lin, int num_blocks,
                      int kv_heads_local, const int32_t* idx, int n, int mode, void* stream, const char* who) {
  if (n <= 0) return FQB_OK;
  if ((!cache && !layers) || !idx || (mode != 0 && !lin)) return set_error(FQB_ERR_INVALID, "%s: null pointer", who);
  if (num_blocks <= 0 || kv_heads_local <= 0 || n_layers <= 0)
    return set_error(FQB_ERR_INVALID, "%s: non-positive size", who);
  if ((cache && !aligned16(cache)) || (lin && !aligned16(lin)))
    return set_error(FQB_ERR_INVALID, "%s: misaligned pointer", who);
  if (n_layers > 65535) return set_error(FQB_ERR_SHAPE, "%s: more than 65535 layers", who);
  BlockMoveParams P;
  P.layers = layers;
  P.cache = static_cast<uint4*>(cache);
  P.lin = static_cast<uint4*>(lin);
  P.idx = idx;
  P.n = n;
  P.num_blocks = num_blocks;
  P.block_vecs = FQB_PLANES * kTok * kv_heads_local * kHd / 8;
  P.mode = mode;
  dim3 grid(n, (P.block_vecs + kCopyChunkVecs - 1) / kCopyChunkVecs, n_layers);
  block_move_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(P);
  FQB_CUDA_TRY(cudaGetLastError());
  return FQB_OK;
}

int fqb_copy_blocks(void* cache, int num_blocks, int kv_heads_local, const int32_t* pairs, int n_pairs,
                    void* stream) {
  return block_move(nullptr, 1, cache, nullptr, num_blocks, kv_heads_local, pairs, n_pairs, 0, stream,
                    "copy_blocks");
}
int fqb_copy_blocks_layers(void* const* layer_caches, int n_layers, int num_blocks, int kv_heads_local,
                           const int32_t* pairs, int n_pairs, void* stream) {
  if (n_pairs > 0 && !layer_caches) return set_error(FQB_ERR_INVALID, "copy_blocks_layers: null pointer");
  return block_move(layer_caches, n_layers, nullptr, nullptr, num_blocks, kv_heads_local, pairs, n_pairs, 0,
                    stream, "copy_blocks_layers");
}
int fqb_gather_blocks(const void* cache, int num_blocks, int kv_heads_local, const int32_t* list, int n,
                      void* out, void* stream) {
  return block_move(nullptr, 1, const_cast<void*>(cache), out, num_blocks, kv_heads_local, list, n, 1, stream,
                    "gather_blocks");
}
int fqb_scatter_blocks(void* cache, int num_blocks, int kv_heads_local, const int32_t* list, int n,
                       const void* in, void* stream) {
  return block_move(nullptr, 1, cache, const_cast<void*>(in), num_blocks, kv_heads_local, list, n, 2, stream,
                    "scatter_blocks");
}

int fqb_device_status(int32_t* detail) {
  int h[4] = {0, 0, 0, 0};
  FQB_CUDA_TRY(cudaMemcpyFromSymbol(h, g_status, sizeof(h)));
  if (detail) std::memcpy(detail, h, sizeof(h));
  if (h[0] != 0)
    return set_error(h[0], "device status: code %d from kernel %d, block %d, value %d", h[0], h[1], h[2], h[3]);
  return FQB_OK;
}

int fqb_device_status_reset(void) {
  const int z[4] = {0, 0, 0, 0};
  FQB_CUDA_TRY(cudaMemcpyToSymbol(g_status, z, sizeof(z)));
  return FQB_OK;
}

}  // extern "C"
