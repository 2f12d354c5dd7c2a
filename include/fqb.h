/* fqb.h -- C ABI of libfqb: paged-KV attention operators for NVIDIA B200 (sm_100a).
 *
 * The library replaces, operator for operator, the paged-KV attention path of the FlashQwen C++
 * engine. Every entry point names the reference interface it stands in for as
 * "replaces: <path>:<lines>" (paths inside the FlashQwen tree).
 *
 * Conventions (the same ones the reference call sites observe):
 *   - every data pointer is a DEVICE pointer owned by the caller unless its comment says "host";
 *   - no entry point allocates device memory, synchronises the device or the stream, or reads
 *     device data on the host; all work is enqueued on the `stream` argument (a cudaStream_t
 *     passed as void*), so the calls may be captured into a CUDA graph;
 *   - launch geometry depends only on scalar arguments, never on context lengths;
 *   - index arrays are 32-bit int; offsets into the cache are computed in 64 bits;
 *   - the return value is FQB_OK (0) or a negative FQB_ERR_* code; nothing exits or throws.
 *     fqb_last_error() gives the text of the calling thread's last failure.
 *
 * KV cache layout of one layer on one GPU (bf16):
 *     cache[num_blocks][2 planes: K, V][16 tokens][kv_heads_local * 128]
 * kv_heads_local is 8 on a single GPU and 8/G when the KV heads are sharded over G GPUs.
 */
#ifndef FQB_H_
#define FQB_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FQB_BLOCK_TOKENS 16 /* replaces: engine/src/kv_layout.h:5 (kKvBlock)  */
#define FQB_PLANES 2        /* replaces: engine/src/kv_layout.h:7 (kKvPlanes) */
#define FQB_HEAD_DIM 128    /* engine/src/model_spec.h:15                      */
#define FQB_GQA_GROUP 4     /* q heads per kv head, engine/src/attn_cute.cu:17 */

enum {
  FQB_OK = 0,
  FQB_ERR_INVALID = -1,   /* null pointer, negative size, misaligned pointer            */
  FQB_ERR_SHAPE = -2,     /* head_dim != 128, group != 4, block_size != 16 and the like  */
  FQB_ERR_CUDA = -3,      /* a CUDA runtime / driver call failed (text in last_error)     */
  FQB_ERR_WORKSPACE = -4, /* partial-result scratch too small for this launch            */
  FQB_ERR_TIMEOUT = -5,   /* device status: a bounded wait inside a kernel ran out       */
  FQB_ERR_INDEX = -6,     /* device status: a block id / position outside its range      */
  FQB_ERR_NOMEM = -7,     /* host allocator: block pool exhausted                        */
  FQB_ERR_STATE = -8      /* host allocator: refcount underflow, unknown block, bad handle */
};

const char* fqb_version(void);
const char* fqb_strerror(int code);
const char* fqb_last_error(void);

/* ---- layout -------------------------------------------------------------------------------
 * replaces: engine/src/kv_store.h:33-35 (KV / NumBlocks / BlockSize) and the sizing arithmetic
 * of engine/src/kv_store.cu:21-23. All counts are in bf16 elements unless named *_bytes. */
typedef struct fqb_kv_layout {
  int32_t kv_heads_local;
  int32_t head_dim;
  int32_t block_tokens;
  int64_t row_elems;   /* kv_heads_local * 128: one token's K (or V) across local heads */
  int64_t plane_elems; /* 16 * row_elems                                                  */
  int64_t block_elems; /* 2 * plane_elems                                                 */
  int64_t block_bytes; /* block_elems * 2                                                 */
} fqb_kv_layout;

int fqb_kv_layout_query(int kv_heads_local, fqb_kv_layout* out /* host */);
int64_t fqb_kv_pool_bytes(int num_blocks, int kv_heads_local);

/* ---- kernel 1: KV append ------------------------------------------------------------------
 * replaces: engine/src/kv_store.h:29-31 KvStore::StoreKV and engine/src/kv_store.cu:48-75.
 * For each row m < M copies the K slice qkv[m*src_stride + k_off ..+row_elems) and the V slice
 * (v_off) into block bt[bt_row[m]*bt_stride + pos[m]/16], token slot pos[m]%16. k_off / v_off
 * are element offsets of this GPU's first kv head inside the fused row; both, src_stride and the
 * base pointers must keep 16-byte alignment. M <= 0 is a no-op. */
int fqb_kv_append(void* cache, int num_blocks, int kv_heads_local, const void* qkv, int src_stride,
                  int k_off, int v_off, const int32_t* bt, int bt_stride, const int32_t* bt_row,
                  const int32_t* pos, int M, void* stream);

/* Fused variant: applies per-head RMSNorm (weights wq / wk, fp32, 128 each) and NeoX rotary
 * embedding to the q and k heads of every fused row in place, exactly as
 * engine/src/kernels.cu:97-139 LaunchHeadNormRope does, and appends the resulting K and the
 * untouched V to the cache as fqb_kv_append does -- one pass over the rows instead of two.
 * replaces: the pair of calls at engine/src/model_runtime.cu:263-268.
 * q_heads_local / kv_heads_local heads starting at element offsets q_off / k_off / v_off.
 * cos_tab / sin_tab are [n_pos][64] fp32 tables (engine/src/model_runtime.cu:111-126).
 * cache == NULL: RMSNorm + RoPE only, nothing is stored (LaunchHeadNormRope by itself) -- for a
 * pure-decode step whose append happens inside fqb_append_attn_decode. */
int fqb_norm_rope_append(void* cache, int num_blocks, int kv_heads_local, int q_heads_local,
                         void* qkv, int src_stride, int q_off, int k_off, int v_off,
                         const float* wq, const float* wk, const float* cos_tab,
                         const float* sin_tab, float eps, const int32_t* bt, int bt_stride,
                         const int32_t* bt_row, const int32_t* pos, int M, void* stream);

/* ---- kernel 2: GQA-shared split-K paged decode attention + LSE combine ---------------------
 * replaces: engine/src/attn_cute.h:14-20 LaunchAttnDecodeCute (engine/src/attn_cute.cu:165-261).
 * For decode sequence di < n_decode: r = decode_rids[di], flat = qstart[r], qpos = pos[flat];
 * q head h (row q + flat*q_stride + h*128) attends keys 0..qpos of kv head h/4 through block
 * table row bt + r*max_blocks; out[(flat*n_heads + h)*128 + d] receives bf16.
 * n_heads / n_kv are the LOCAL head counts (q already points at this GPU's first head).
 *
 * pm, pl (partial_slots floats each) and pa (partial_slots*128 floats) are the split-K scratch,
 * as at the reference call site (engine/src/model_runtime.cu:191-194, kernels.cuh:33-37).
 * The split count is decided on the device from the actual context lengths and limited by
 * partial_slots; fqb_attn_decode_partial_slots() returns a size that never limits it.
 * num_blocks bounds the block ids (ids outside [0,num_blocks) read zeros and raise
 * FQB_ERR_INDEX in the device status). n_decode <= 0 is a no-op. */
int64_t fqb_attn_decode_partial_slots(int max_decode, int n_heads_local, int max_blocks);
/* The exact number of partial slots fqb_attn_decode (flags = 0) needs for n_decode sequences and n_kv
 * local kv heads on the CURRENT device (it follows the SM count), or a negative FQB_ERR_* code. */
int64_t fqb_attn_decode_slots_needed(int n_decode, int n_kv);

int fqb_attn_decode(const void* q, int q_stride, const void* cache, int num_blocks, void* out,
                    int n_heads, int n_kv, int head_dim, const int32_t* pos, const int32_t* qstart,
                    const int32_t* decode_rids, int n_decode, const int32_t* bt, int max_blocks,
                    int block_size, float scale, float* pm, float* pl, float* pa,
                    int64_t partial_slots, void* stream);

/* fqb_attn_decode with flags. Every launch of this library lets the kernel after it begin early
 * (programmatic dependent launch) and itself waits for the kernel before it only after its own
 * prologue, which reads nothing but pos / qstart / decode_rids / bt -- those four arrays must be final
 * (written by copies, or by kernels that an ordinary launch has followed) before the kernel launched
 * immediately before this call starts; the engine fills them with copies at the start of the step,
 * engine/src/model_runtime.cu:295-302.
 *   FQB_DECODE_INDEPENDENT  the caller states that the kernel launched immediately before this call
 *       writes NOTHING this call reads (q, cache, metadata) and does not read `out`. The launch then
 *       streams KV while that kernel is still running; consecutive calls rotate through up to 64
 *       regions of the scratch and the launch that re-enters the first region completes all earlier
 *       work before any later launch may start, so scratch is never shared by two live launches. Meant for back-to-back attention over independent
 *       caches (micro-batches, benchmarks); without the flag the call is always safe. */
#define FQB_DECODE_INDEPENDENT 1u
int fqb_attn_decode_ex(const void* q, int q_stride, const void* cache, int num_blocks, void* out,
                       int n_heads, int n_kv, int head_dim, const int32_t* pos,
                       const int32_t* qstart, const int32_t* decode_rids, int n_decode,
                       const int32_t* bt, int max_blocks, int block_size, float scale, float* pm,
                       float* pl, float* pa, int64_t partial_slots, unsigned flags, void* stream);

/* Step plan. The per-sequence values every decode launch derives from pos / qstart / decode_rids
 * (request, flat row, last key position, page prefix sum) are the same for all layers of a step:
 * fqb_attn_decode_plan computes them once (one small kernel) into plan[4*n_decode + 1] int32 (device,
 * 16-byte aligned), and fqb_attn_decode_planned takes the plan instead of the three arrays, which
 * turns each launch's three dependent metadata loads and its scan into one coalesced load. No
 * reference counterpart (the reference recomputes per launch, engine/src/attn_cute.cu:172). The plan
 * is valid while pos / qstart / decode_rids are unchanged; at most FQB_PLAN_MAX_DECODE sequences to
 * build and 256 per planned call. Results are identical to fqb_attn_decode_ex. Build the plan and make
 * the step's launches from ONE thread on ONE stream: the first launch that thread makes on the plan's
 * stream after fqb_attn_decode_plan waits for the plan in full (it is an ordinary launch), which is what
 * makes the plan visible to the prologues of all later launches on that stream. */
#define FQB_PLAN_MAX_DECODE 1024
int fqb_attn_decode_plan(const int32_t* pos, const int32_t* qstart, const int32_t* decode_rids,
                         int n_decode, int max_blocks, int32_t* plan, void* stream);
int fqb_attn_decode_planned(const void* q, int q_stride, const void* cache, int num_blocks, void* out,
                            int n_heads, int n_kv, int head_dim, const int32_t* plan, int n_decode,
                            const int32_t* bt, int max_blocks, int block_size, float scale, float* pm,
                            float* pl, float* pa, int64_t partial_slots, unsigned flags, void* stream);

/* Fused pair: KV append of the step's new token + decode attention, one kernel.
 * replaces: the call pair KvStore::StoreKV + LaunchAttnDecodeCute of a pure-decode step
 * (engine/src/model_runtime.cu:267-273; the steps the engine replays from CUDA graphs,
 * engine/src/model_runtime.cu:227-233). For decode sequence di (r = decode_rids[di], flat = qstart[r],
 * p = pos[flat]) the K and V rows of the fused row qkv + flat*src_stride (local heads at element
 * offsets k_off / v_off, as for fqb_kv_append) are written to token slot p of block
 * bt[r*max_blocks + p/16], and the q heads at q_off attend keys 0..p including that row; out as for
 * fqb_attn_decode. The cache afterwards is bit-identical to fqb_kv_append over the same rows. Exactly
 * one warp per (sequence, kv head) streams the sequence's last page; that warp stores the row and puts
 * it into the page it has just loaded, so no other kernel has to run in front. Rows of prefill requests
 * in a mixed step still go through fqb_kv_append (appending a decode row twice is harmless).
 * Either pos / qstart / decode_rids or a step plan (fqb_attn_decode_plan; then the three may be NULL).
 * The block that receives the row must be private to the sequence (fqb_cow_prepare first).
 * flags: 0, FQB_DECODE_INDEPENDENT, or
 *   FQB_DECODE_HISTORY_STABLE  the caller states that the kernel launched immediately before this call
 *       writes none of the CACHED keys this call reads (positions < p of the decode sequences) and none
 *       of the metadata; it may well produce the qkv rows. The launch then requests its first pages
 *       while that kernel still runs and waits for it only before it reads the rows -- the dependency
 *       the engine's layer loop really has (the kernel in front is the QKV projection or the q/k norm,
 *       engine/src/model_runtime.cu:259-265; the layer's cache was last written one step earlier).
 *       Not valid directly after a kernel that writes this cache (fqb_copy_blocks, fqb_kv_append,
 *       fqb_scatter_blocks): use flags = 0 there. */
#define FQB_DECODE_HISTORY_STABLE 2u
int fqb_append_attn_decode(void* cache, int num_blocks, int kv_heads_local, const void* qkv, int src_stride,
                           int q_off, int k_off, int v_off, void* out, int head_dim, const int32_t* pos,
                           const int32_t* qstart, const int32_t* decode_rids, const int32_t* plan, int n_decode,
                           const int32_t* bt, int max_blocks, int block_size, float scale, float* pm, float* pl,
                           float* pa, int64_t partial_slots, unsigned flags, void* stream);

/* ---- fp8 (e4m3) KV cache: kernels 1 and 2 over half the bytes ------------------------------------
 * No reference counterpart: the reference names an fp8 KV cache as its next lever and has none
 * (docs/optimization.md:119-120); the format is defined here. cache8 is
 * [num_blocks][2][16][kv_heads_local*128] e4m3 bytes and scales [num_blocks][kv_heads_local][2][16] fp32:
 * one scale per (token, kv head, plane), s = amax / 448 over the head's 128 values (1 for an all-zero
 * row); a stored byte is e4m3(x * (448 / amax)), round to nearest even, saturating; a value reads back
 * as e4m3_to_float(byte) * s. fqb_kv_append_fp8 quantises the rows as fqb_kv_append copies them (same
 * arguments); the bytes and scales are reproducible bit for bit on the host. fqb_attn_decode_fp8 is
 * fqb_attn_decode_ex over that cache: K and V are widened to f16 in registers (exact), the K scale
 * multiplies the score, the V scale the probability; flags 0 or FQB_DECODE_INDEPENDENT. Against the
 * exact softmax over the DEQUANTISED cache the outputs agree to the same 2e-2 as the bf16 kernels;
 * against the bf16 cache they differ by the quantisation itself (about 2^-4 relative per K / V value). */
int64_t fqb_kv_pool_bytes_fp8(int num_blocks, int kv_heads_local);
int64_t fqb_kv_scale_bytes_fp8(int num_blocks, int kv_heads_local);
int fqb_kv_append_fp8(void* cache8, float* scales, int num_blocks, int kv_heads_local, const void* qkv, int src_stride,
                      int k_off, int v_off, const int32_t* bt, int bt_stride, const int32_t* bt_row,
                      const int32_t* pos, int M, void* stream);
/* Blocks of the fp8 cache read back as bf16: out is a dense pool [n][2][16][kv_heads_local*128] bf16 in the
 * layout of the bf16 cache, out block i = block list[i] (device array), every value
 * bf16(e4m3_to_float(byte) * scale), reproducible bit for bit on the host. For the chunked prefill of a
 * request whose history lives in the fp8 cache: read its pages back into a staging pool, append the
 * chunk's rows to the staging pool with fqb_kv_append (and to the fp8 cache with fqb_kv_append_fp8), and
 * run fqb_attn_prefill over the staging pool with the block table 0, 1, 2, ... Ids outside
 * [0, num_blocks) raise FQB_ERR_INDEX in the device status and leave their output block untouched. */
int fqb_dequant_blocks_fp8(const void* cache8, const float* scales, int num_blocks, int kv_heads_local,
                           const int32_t* list, int n, void* out, void* stream);
/* fqb_append_attn_decode over the fp8 cache: the step's token is quantised (the bytes and the scale
 * fqb_kv_append_fp8 would store) by the warp that streams its page, written to cache8 / scales and attended
 * in the same kernel; arguments and flags as fqb_append_attn_decode, scales is read and written. */
int fqb_append_attn_decode_fp8(void* cache8, float* scales, int num_blocks, int kv_heads_local, const void* qkv,
                               int src_stride, int q_off, int k_off, int v_off, void* out, int head_dim,
                               const int32_t* pos, const int32_t* qstart, const int32_t* decode_rids, const int32_t* plan,
                               int n_decode, const int32_t* bt, int max_blocks, int block_size, float scale, float* pm,
                               float* pl, float* pa, int64_t partial_slots, unsigned flags, void* stream);
int fqb_attn_decode_fp8(const void* q, int q_stride, const void* cache8, const float* scales, int num_blocks, void* out,
                        int n_heads, int n_kv, int head_dim, const int32_t* pos, const int32_t* qstart,
                        const int32_t* decode_rids, int n_decode, const int32_t* bt, int max_blocks, int block_size,
                        float scale, float* pm, float* pl, float* pa, int64_t partial_slots, unsigned flags,
                        void* stream);

/* ---- reassembly of the per-head outputs over G GPUs of one node, inside the decode kernel -----------
 * No reference counterpart (the reference is single-GPU). With the KV heads sharded over G GPUs every
 * rank produces [rows][(32/G)*128]; where full rows are wanted on every GPU, the kernel that finishes a
 * row stores it straight into every rank's buffer of full rows [rows][32*128] (plain stores over
 * NVLink into peer memory, no multicast, no library kernel on peer memory), instead of a separate
 * all-gather per layer afterwards. When the launch's last warp is through, the rank bumps its publish
 * counter for the slot and stores it into every rank's flag word. fqb_gather_wait enqueues a one-warp
 * kernel that returns once all G ranks have delivered the slot's current publish; it polls local memory
 * only and gives up after timeout_ms (default 1000) with FQB_ERR_TIMEOUT in the device status.
 * Set-up, once: every rank allocates its buffers and one zeroed control block of
 * fqb_gather_control_bytes(slots, world) bytes with fqb_peer_alloc, exports them (fqb_peer_export, 64-byte
 * handles passed through any host channel) and opens the others' (fqb_peer_open). A slot is one
 * independent sequence of publishes (one per layer, say). All ranks make the same calls in the same
 * order. Two calls of one rank whose kernels can overlap (FQB_DECODE_INDEPENDENT) must use different slots. A rank may overwrite a peer's buffer of slot s as soon as it reaches its next call for s: put the
 * consumer of a slot (and a fqb_gather_wait) on every rank's stream before that rank's next call for it.
 * The calls take no CUDA graph parameters that change between replays, so they can be captured. */
#define FQB_PEER_HANDLE_BYTES 64
typedef struct fqb_gather {
  int32_t world, rank;   /* ranks of the node sharing the heads, this rank           */
  int32_t slots, slot;   /* publish sequences in the control block, the one to use   */
  void* out[8];          /* every rank's buffer of full rows for this call; out[rank] is local */
  void* flags[8];        /* every rank's control block (its start); flags[rank] is local        */
  void* control;         /* this rank's control block                                          */
  int32_t timeout_ms;    /* fqb_gather_wait gives up after this long; 0 = 1000                  */
} fqb_gather;
int64_t fqb_gather_control_bytes(int slots, int world);
/* fqb_append_attn_decode that also delivers the rows to every rank and publishes. One launch per call:
 * 1..256 sequences, 1, 2 or 4 local kv heads. */
int fqb_append_attn_decode_gather(void* cache, int num_blocks, int kv_heads_local, const void* qkv, int src_stride,
                                  int q_off, int k_off, int v_off, void* out, int head_dim, const int32_t* pos,
                                  const int32_t* qstart, const int32_t* decode_rids, const int32_t* plan, int n_decode,
                                  const int32_t* bt, int max_blocks, int block_size, float scale, float* pm, float* pl,
                                  float* pa, int64_t partial_slots, unsigned flags, const fqb_gather* gather,
                                  void* stream);
int fqb_gather_wait(const fqb_gather* gather, void* stream);
/* The same wait for every slot of the control block in one kernel (end of a step). */
int fqb_gather_wait_all(const fqb_gather* gather, void* stream);
/* FQB_GATHER_PUBLISH_LATER (a flag of fqb_append_attn_decode_gather): the kernel still stores every
 * finished row into all ranks' buffers, but neither counts its warps in nor publishes. A launch that the
 * next one waits for then ends without a system-wide fence and a round of flag stores over NVLink (about
 * 15 us per launch where every launch waits for the one before it). The caller publishes all slots at
 * once with fqb_gather_publish_all after the last such launch of the step: a one-CTA kernel, launched
 * without overlap, so every earlier kernel of the stream has completed and its stores have been performed
 * when it bumps each slot's publish counter and stores it into every rank's flag words. All ranks make
 * the same number of publishes per slot, as with the in-kernel form. */
#define FQB_GATHER_PUBLISH_LATER 4u
int fqb_gather_publish_all(const fqb_gather* gather, void* stream);
int fqb_peer_alloc(int64_t bytes, void** ptr /* host: receives a zeroed device allocation */);
int fqb_peer_free(void* ptr);
int fqb_peer_export(void* ptr, void* handle64 /* host, FQB_PEER_HANDLE_BYTES */);
int fqb_peer_open(const void* handle64 /* host */, void** ptr /* host: receives the mapped peer pointer */);
int fqb_peer_close(void* ptr);

/* Decode attention without caller scratch. No counterpart in the reference (its call site always
 * passes pm / pl / pa): this entry point exists for callers that have no device memory to give and
 * no way to get any at the point of the call -- an engine that handed all free VRAM to its KV pool
 * at start-up, as the FlashQwen engine does (engine/src/kv_store.cu:10-46), so a later cudaMalloc
 * fails; code between cudaStreamBeginCapture and cudaStreamEndCapture, where cudaMalloc is not
 * allowed; a plugin inside a host that owns every device allocation. It runs the same kernel as
 * fqb_attn_decode with the split-K scratch taken from a fixed 4.06 MiB array inside the library's
 * own device image (resident on every GPU that loads the library until the process exits), and it
 * calls no allocating routine of any kind.
 *   Limits: n_decode <= FQB_STATIC_MAX_DECODE and n_kv one of 1, 2, 4, 8 (<= FQB_STATIC_MAX_KV_HEADS).
 *   Any other head count (3, 5, 6, 7) goes out as several launches whose partials do not fit the
 *   array; so does the full 64 x 8 case on a GPU with more than 159 SMs (B200 has 148). What does not
 *   fit is worked out before anything is launched: the call returns FQB_ERR_WORKSPACE, names the
 *   limit in fqb_last_error() and launches nothing.
 *   First call on each device: looks up the array's device address (cudaGetSymbolAddress, with that
 *   device current). Make that first call outside any stream capture; later calls may be captured
 *   like the other operators.
 *   All calls on a device share the one array, which keeps whatever the previous call left in it.
 *   Nothing in it needs clearing (the arrival counters are tagged per launch), but two calls whose
 *   kernels can overlap on the GPU -- different streams, or FQB_DECODE_INDEPENDENT-style pipelining --
 *   race on it: issue them on one stream, one after the other. */
#define FQB_STATIC_MAX_DECODE 64
#define FQB_STATIC_MAX_KV_HEADS 8
int fqb_attn_decode_static(const void* q, int q_stride, const void* cache, int num_blocks, void* out,
                           int n_heads, int n_kv, int head_dim, const int32_t* pos,
                           const int32_t* qstart, const int32_t* decode_rids, int n_decode,
                           const int32_t* bt, int max_blocks, int block_size, float scale,
                           void* stream);

/* ---- kernel 3: chunked-prefill paged attention ---------------------------------------------
 * replaces: engine/src/attn_cute.h:7-12 LaunchAttnPrefillCute (engine/src/attn_cute.cu:30-163).
 * For prefill request r = rids[z], z < R: rows qstart[r] .. qstart[r]+qlen[r]-1 are contiguous,
 * row i attends key positions <= pos[qstart[r]+i] through bt + r*max_blocks; output layout as
 * for decode. max_qlen bounds qlen over the R requests. R <= 0 is a no-op. */
int fqb_attn_prefill(const void* q, int q_stride, const void* cache, int num_blocks, void* out,
                     int n_heads, int n_kv, int head_dim, const int32_t* pos,
                     const int32_t* qstart, const int32_t* qlen, const int32_t* rids, int R,
                     int max_qlen, const int32_t* bt, int max_blocks, int block_size, float scale,
                     void* stream);

/* ---- kernel 4: prefix-cache block copy (copy-on-write) and gather --------------------------
 * No reference kernel exists: the reference shares only full blocks by aliasing block-table
 * entries (engine/src/scheduler.cc:27-44) and so never copies. These operators add copy-on-write
 * for a partially filled shared tail block and a contiguous export of a block list.
 * copy:   cache[pairs[2i+1]] <- cache[pairs[2i]] (whole page, both planes). Destinations must be
 *         distinct from each other and from every source.
 * gather: out[i] <- cache[list[i]], out is [n][2][16][row_elems].
 * scatter: the inverse of gather, cache[list[i]] <- in[i]. */
int fqb_copy_blocks(void* cache, int num_blocks, int kv_heads_local, const int32_t* pairs,
                    int n_pairs, void* stream);
int fqb_copy_blocks_layers(void* const* layer_caches /* device array of n_layers pointers */,
                           int n_layers, int num_blocks, int kv_heads_local, const int32_t* pairs,
                           int n_pairs, void* stream);
int fqb_gather_blocks(const void* cache, int num_blocks, int kv_heads_local, const int32_t* list,
                      int n, void* out, void* stream);
int fqb_scatter_blocks(void* cache, int num_blocks, int kv_heads_local, const int32_t* list, int n,
                       const void* in, void* stream);

/* ---- device status --------------------------------------------------------------------------
 * The kernels never trap and never wait without a limit. A bounded wait that runs out, or an
 * index outside its range, is recorded in a status word in the library's own device memory and
 * the kernel carries on without touching memory it should not. fqb_device_status() copies the
 * word back (it synchronises the device: call it at the step boundary, where the reference
 * checks its own CUDA errors, engine/src/model_runtime.cu:309) and returns FQB_OK,
 * FQB_ERR_TIMEOUT or FQB_ERR_INDEX; detail[0..3] (host, optional) receives
 * {code, kernel id, block index, value}. fqb_device_status_reset() clears it. */
int fqb_device_status(int32_t* detail /* host, may be NULL */);
int fqb_device_status_reset(void);

/* ---- the engine's launcher symbols -----------------------------------------------------------
 * libfqb also defines, as C++ symbols with the engine's own signatures, the two attention
 * launchers of engine/src/attn_cute.h:7-20:
 *   void fq::LaunchAttnPrefillCute(const __nv_bfloat16* q, int q_stride, const __nv_bfloat16* cache_kv,
 *        __nv_bfloat16* out, int n_heads, int n_kv, int head_dim, const int* pos, const int* qstart,
 *        const int* qlen, const int* rids, int R, int max_qlen, const int* bt, int max_blocks,
 *        int block_size, float scale, cudaStream_t s);
 *   void fq::LaunchAttnDecodeCute(... const int* decode_rids, int n_decode, const int* bt, int max_blocks,
 *        int block_size, float scale, float* pm, float* pl, float* pa, cudaStream_t s);
 * so an engine built without attn_cute.cu and linked against libfqb resolves its existing calls
 * (engine/src/model_runtime.cu:271-283) here. Those signatures carry neither the pool's block count
 * nor the scratch size, which the kernels need for their tensor map and bounds checks:
 * fqb_engine_configure() supplies both once, after the pool and the decode scratch are allocated
 * (num_blocks = KvStore::NumBlocks(), engine/src/kv_store.h:37; partial_slots = the float count of
 * pm, DecodePartialFloats(slots), engine/src/kernels.cuh:33-37). The launchers return void as the
 * engine's do; a failed call is kept (first one wins) and fqb_engine_status() returns its code,
 * with the message in fqb_engine_error(). Before fqb_engine_configure() they fail with
 * FQB_ERR_STATE and launch nothing. */
int fqb_engine_configure(int num_blocks, int64_t partial_slots);
int fqb_engine_status(void);
const char* fqb_engine_error(void);

/* ---- host side: block allocator with prefix cache (no CUDA) ---------------------------------
 * replaces: engine/src/block_allocator.h:21-101 (class BlockAllocator) and the prefix functions
 * of engine/src/scheduler.cc:16-57. One handle = one pool of block ids [0, num_blocks);
 * not thread-safe, like the reference (one engine thread). */
typedef struct fqb_alloc fqb_alloc;

fqb_alloc* fqb_alloc_create(int num_blocks);
void fqb_alloc_destroy(fqb_alloc* a);
int fqb_alloc_num_blocks(const fqb_alloc* a);
int fqb_alloc_num_free(const fqb_alloc* a);                  /* BlockAllocator::NumFree  */
int fqb_alloc_blocks_for(int n_tokens);                      /* BlockAllocator::BlocksFor */
int fqb_alloc_refcount(const fqb_alloc* a, int block);
uint64_t fqb_alloc_block_hash(const fqb_alloc* a, int block);
int fqb_alloc_one(fqb_alloc* a);                             /* AllocOne: id or FQB_ERR_NOMEM */
int fqb_alloc_free_one(fqb_alloc* a, int block);             /* FreeOne                    */
int fqb_alloc_free_table(fqb_alloc* a, int32_t* table, int* len); /* Free: frees all, *len=0 */
/* Grow: extend table (*len entries, room for cap) to cover n_tokens. FQB_ERR_NOMEM when the pool
 * runs dry; the blocks obtained so far stay in the table (the caller preempts and retries). */
int fqb_alloc_grow(fqb_alloc* a, int32_t* table, int* len, int cap, int n_tokens);
int fqb_alloc_cache_lookup(fqb_alloc* a, uint64_t hash);     /* CacheLookup: id or -1 (miss) */
int fqb_alloc_cache_insert(fqb_alloc* a, int block, uint64_t hash); /* CacheInsert          */

/* replaces: engine/src/scheduler.cc:16-24 HashBlock */
uint64_t fqb_hash_block(uint64_t parent, const int32_t* tokens, int n);
/* replaces: engine/src/scheduler.cc:27-44 AcquirePrefix (+ Request::AdoptPrefix,
 * engine/src/scheduler.h:54-58). Returns the number of blocks adopted into table[0..); the
 * request's computed-token count becomes that * 16. *last_hash receives the chain hash. */
int fqb_acquire_prefix(fqb_alloc* a, const int32_t* tokens, int n_tokens, int32_t* table, int cap,
                       uint64_t* last_hash);
/* replaces: engine/src/scheduler.cc:46-57 CacheBlocks. Returns the new cached-block count. */
int fqb_cache_blocks(fqb_alloc* a, const int32_t* tokens, int computed, const int32_t* table,
                     int cached_blocks, uint64_t* last_hash);
/* Copy-on-write decision before writing token position pos of a sequence: when the target block
 * is shared (refcount > 1) and the write does not start the block, a private block replaces it in
 * the table and pair[0..1] = {shared, private} must be copied (fqb_copy_blocks) before the append.
 * Returns 1 (pair produced), 0 (nothing to do) or FQB_ERR_NOMEM. */
int fqb_cow_prepare(fqb_alloc* a, int32_t* table, int pos, int32_t* pair);

/* ---- host side: step metadata ----------------------------------------------------------------
 * replaces: engine/src/model_runtime.cu:54-91 (PackBlockTables, SplitDecodePrefill). All host
 * pointers. counts = {n_decode, n_prefill, prefill_max_qlen}. tables[r] / table_len[r] are the
 * requests' block tables, packed into bt_out with row stride bt_stride (tail left untouched). */
int fqb_step_pack(const int32_t* req_index, int n_rows, int n_req, const int32_t* const* tables,
                  const int32_t* table_len, int bt_stride, int32_t* bt_out, int32_t* qstart,
                  int32_t* qlen, int32_t* decode_rids, int32_t* prefill_rids, int32_t* counts);

/* ---- host side: step driver -----------------------------------------------------------------------
 * The engine's scheduling loop and the attention part of its per-step runtime, driven through the
 * operators above. replaces: engine/src/scheduler.cc:59-154 and engine/src/scheduler.h:19-118 (Request,
 * Grow with preempt-by-recompute, Refill, BuildBatch under a token budget, Step), and of
 * engine/src/model_runtime.cu the input preparation (:47-108, here ONE pinned buffer and one copy for all
 * step metadata instead of eight), RunLayers (:227-233: pure-decode steps replayed from CUDA graphs keyed
 * (rows, decode requests), engine/src/model_runtime.h:160-201) and the attention calls of RunLayersBody
 * (:259-283). The model is not part of it: `rows` stands in for embedding + QKV projection and fills the
 * step's fused qkv rows (bf16 bits) for every layer, rows_host[layer * row_capacity + row][row_elems];
 * `sample` stands in for everything after attention: it receives the attention output of every layer,
 * out_host[layer * row_capacity + row][q_heads*128], and writes one token per entry of logits_rows.
 * Both run on the calling thread inside fqb_driver_step. The caller owns the per-layer caches
 * ([num_blocks][2][16][kv_heads*128] bf16 each); fqb_driver_create allocates the driver's own staging
 * buffers once, steps allocate nothing. A pure-decode step runs, per layer, RMSNorm + RoPE and then
 * fqb_append_attn_decode (FQB_DECODE_HISTORY_STABLE); a mixed step fqb_norm_rope_append, fqb_attn_decode
 * and fqb_attn_prefill. One thread drives a handle, like the engine thread. */
typedef struct fqb_driver fqb_driver;
typedef struct fqb_driver_config {
  int32_t n_layers, num_blocks, kv_heads, q_heads;
  int32_t n_slots;        /* concurrent sequences, engine/src/args.h:14 */
  int32_t token_budget;   /* rows per step, engine/src/args.h:16          */
  int32_t prefill_chunk;  /* engine/src/args.h:17                          */
  int32_t max_ctx;
  int32_t use_prefix_cache, use_graphs;
  float scale, rms_eps, rope_theta;
} fqb_driver_config;
typedef struct fqb_step_view {   /* all pointers: host, valid during the callback */
  int32_t step, n_rows, n_req, n_decode, n_prefill, prefill_max_qlen, bt_stride, row_capacity, from_graph, n_logits;
  const int32_t *tokens, *pos, *req, *qstart, *qlen, *decode_rids, *prefill_rids, *bt, *logits_rows, *request_ids;
} fqb_step_view;
typedef struct fqb_driver_stats {
  uint64_t steps, graph_captures, graph_replays, preemptions, over_capacity, prefix_hit_blocks, finished, decode_rows,
      prefill_rows;
  int32_t free_blocks, running, waiting;
} fqb_driver_stats;
typedef void (*fqb_rows_fn)(void* user, int step, int n_rows, const int32_t* tokens, const int32_t* pos,
                            const int32_t* req, uint16_t* rows_host, int row_capacity);
typedef void (*fqb_sample_fn)(void* user, const fqb_step_view* view, const uint16_t* out_host, int32_t* sampled);

/* replaces: RopeTables::Build, engine/src/model_runtime.cu:111-126 (host arrays [n_pos][head_dim/2]) */
void fqb_rope_tables(float* cos_tab, float* sin_tab, int n_pos, int head_dim, float theta);
int fqb_driver_create(const fqb_driver_config* cfg, void* const* layer_caches /* host array of device pointers */,
                      const float* wq, const float* wk /* host, 128 each: q / k norm weights */, fqb_rows_fn rows,
                      fqb_sample_fn sample, void* user, fqb_driver** out);
void fqb_driver_destroy(fqb_driver* d);
/* Scheduler::Submit: queues a request; returns its id (>= 0) or a negative code. */
int fqb_driver_submit(fqb_driver* d, const int32_t* prompt, int n_prompt, int max_new);
int fqb_driver_busy(const fqb_driver* d);
/* Scheduler::Step: 1 = a step ran, 0 = nothing to run, negative = error (the step is lost). */
int fqb_driver_step(fqb_driver* d);
int fqb_driver_get_stats(const fqb_driver* d, fqb_driver_stats* out);

#ifdef __cplusplus
}
#endif
#endif /* FQB_H_ */
