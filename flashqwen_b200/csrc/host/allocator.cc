// Host half of the paged KV cache: block ids, reference counts, LRU reuse and the prefix cache.
// CUDA-free. Behaviour follows the reference's BlockAllocator
// (engine/src/block_allocator.h:21-101 of the FlashQwen tree) and the scheduler's prefix functions
// (engine/src/scheduler.cc:16-57); the data structures do not: the LRU queue is a pair of index
// arrays threaded through the blocks (no node allocation per push), and the hash -> block map is
// an open-addressing table sized once for the pool.
#include <cstdint>
#include <cstring>
#include <new>
#include <vector>

#include "../../../include/fqb.h"
#include "../errors.h"

namespace fqb {
namespace {
constexpr int kNil = -1;
constexpr int kOut = -2;  // not in the free queue
}  // namespace
}  // namespace fqb

struct fqb_alloc {
  int n = 0;
  std::vector<int32_t> ref, prv, nxt;
  std::vector<uint64_t> hash;  // content hash of the block, 0 = none
  int head = fqb::kNil, tail = fqb::kNil, n_free = 0;

  // open addressing, linear probing, tombstones; key 0 = empty, value kOut = tombstone
  std::vector<uint64_t> keys;
  std::vector<int32_t> vals;
  uint32_t mask = 0;
  int live = 0, tomb = 0;

  void queue_push(int b) {
    prv[b] = tail;
    nxt[b] = fqb::kNil;
    if (tail != fqb::kNil) nxt[tail] = b; else head = b;
    tail = b;
    ++n_free;
  }
  void queue_remove(int b) {
    const int p = prv[b], q = nxt[b];
    if (p != fqb::kNil) nxt[p] = q; else head = q;
    if (q != fqb::kNil) prv[q] = p; else tail = p;
    prv[b] = nxt[b] = fqb::kOut;
    --n_free;
  }
  static uint32_t mix(uint64_t h) {
    h ^= h >> 33;
    h *= 0xff51afd7ed558ccdull;
    h ^= h >> 33;
    return static_cast<uint32_t>(h);
  }
  int map_find(uint64_t key) const {  // slot index or -1
    for (uint32_t i = mix(key) & mask;; i = (i + 1) & mask) {
      if (keys[i] == key && vals[i] != fqb::kOut) return static_cast<int>(i);
      if (keys[i] == 0 && vals[i] != fqb::kOut) return -1;
    }
  }
  void map_rebuild() {
    std::vector<uint64_t> ok;
    std::vector<int32_t> ov;
    ok.swap(keys);
    ov.swap(vals);
    keys.assign(ok.size(), 0);
    vals.assign(ov.size(), 0);
    tomb = 0;
    for (size_t i = 0; i < ok.size(); ++i)
      if (ok[i] != 0 && ov[i] != fqb::kOut) {
        uint32_t j = mix(ok[i]) & mask;
        while (keys[j] != 0) j = (j + 1) & mask;
        keys[j] = ok[i];
        vals[j] = ov[i];
      }
  }
  void map_put(uint64_t key, int b) {
    if ((live + tomb + 1) * 2 > static_cast<int>(mask)) map_rebuild();
    uint32_t i = mix(key) & mask;
    while (keys[i] != 0 && vals[i] != fqb::kOut) i = (i + 1) & mask;
    if (vals[i] == fqb::kOut) --tomb;
    keys[i] = key;
    vals[i] = b;
    ++live;
  }
  void map_erase_slot(int slot) {
    keys[slot] = 0;
    vals[slot] = fqb::kOut;
    --live;
    ++tomb;
  }
  bool valid(int b) const { return b >= 0 && b < n; }
};

extern "C" {

fqb_alloc* fqb_alloc_create(int num_blocks) {
  if (num_blocks <= 0) {
    fqb::set_error(FQB_ERR_INVALID, "alloc_create: num_blocks %d", num_blocks);
    return nullptr;
  }
  fqb_alloc* a = new (std::nothrow) fqb_alloc;
  if (!a) return nullptr;
  a->n = num_blocks;
  a->ref.assign(num_blocks, 0);
  a->prv.assign(num_blocks, fqb::kOut);
  a->nxt.assign(num_blocks, fqb::kOut);
  a->hash.assign(num_blocks, 0);
  uint32_t cap = 16;
  while (cap < static_cast<uint32_t>(num_blocks) * 4u) cap <<= 1;  // live <= n, so load stays under 1/2
  a->keys.assign(cap, 0);
  a->vals.assign(cap, 0);
  a->mask = cap - 1;
  for (int b = 0; b < num_blocks; ++b) a->queue_push(b);
  return a;
}

void fqb_alloc_destroy(fqb_alloc* a) { delete a; }
int fqb_alloc_num_blocks(const fqb_alloc* a) { return a ? a->n : FQB_ERR_STATE; }
int fqb_alloc_num_free(const fqb_alloc* a) { return a ? a->n_free : FQB_ERR_STATE; }
int fqb_alloc_blocks_for(int n_tokens) { return (n_tokens + FQB_BLOCK_TOKENS - 1) / FQB_BLOCK_TOKENS; }

int fqb_alloc_refcount(const fqb_alloc* a, int block) {
  if (!a || !a->valid(block)) return fqb::set_error(FQB_ERR_STATE, "alloc_refcount: bad handle or block %d", block);
  return a->ref[block];
}
uint64_t fqb_alloc_block_hash(const fqb_alloc* a, int block) {
  return (a && a->valid(block)) ? a->hash[block] : 0;
}

int fqb_alloc_one(fqb_alloc* a) {
  if (!a) return fqb::set_error(FQB_ERR_STATE, "alloc_one: null handle");
  if (a->head == fqb::kNil) return fqb::set_error(FQB_ERR_NOMEM, "alloc_one: pool of %d blocks is dry", a->n);
  const int b = a->head;
  a->queue_remove(b);
  if (a->hash[b]) {  // a cached block is being recycled: its prefix entry dies with it
    const int slot = a->map_find(a->hash[b]);
    if (slot >= 0 && a->vals[slot] == b) a->map_erase_slot(slot);
    a->hash[b] = 0;
  }
  a->ref[b] = 1;
  return b;
}

int fqb_alloc_free_one(fqb_alloc* a, int block) {
  if (!a || !a->valid(block)) return fqb::set_error(FQB_ERR_STATE, "free_one: bad handle or block %d", block);
  if (a->ref[block] <= 0) return fqb::set_error(FQB_ERR_STATE, "free_one: block %d is not held", block);
  if (--a->ref[block] == 0) a->queue_push(block);  // most recently freed is reused last; hash kept
  return FQB_OK;
}

int fqb_alloc_free_table(fqb_alloc* a, int32_t* table, int* len) {
  if (!a || !table || !len) return fqb::set_error(FQB_ERR_STATE, "free_table: null argument");
  int rc = FQB_OK;
  for (int i = 0; i < *len; ++i) {
    const int r = fqb_alloc_free_one(a, table[i]);
    if (r != FQB_OK) rc = r;
  }
  *len = 0;
  return rc;
}

int fqb_alloc_grow(fqb_alloc* a, int32_t* table, int* len, int cap, int n_tokens) {
  if (!a || !table || !len) return fqb::set_error(FQB_ERR_STATE, "alloc_grow: null argument");
  const int need = fqb_alloc_blocks_for(n_tokens);
  if (need > cap) return fqb::set_error(FQB_ERR_INVALID, "alloc_grow: %d blocks needed, table holds %d", need, cap);
  while (*len < need) {
    const int b = fqb_alloc_one(a);
    if (b < 0) return b;
    table[(*len)++] = b;
  }
  return FQB_OK;
}

int fqb_alloc_cache_lookup(fqb_alloc* a, uint64_t hash) {
  if (!a || hash == 0) return -1;
  const int slot = a->map_find(hash);
  if (slot < 0) return -1;
  const int b = a->vals[slot];
  if (a->ref[b] == 0) a->queue_remove(b);  // resurrect a freed block that still holds the prefix
  ++a->ref[b];
  return b;
}

int fqb_alloc_cache_insert(fqb_alloc* a, int block, uint64_t hash) {
  if (!a || !a->valid(block)) return fqb::set_error(FQB_ERR_STATE, "cache_insert: bad handle or block %d", block);
  if (hash == 0) return fqb::set_error(FQB_ERR_INVALID, "cache_insert: hash 0 is reserved");
  if (a->hash[block] != 0) return FQB_OK;       // block already published
  if (a->map_find(hash) >= 0) return FQB_OK;    // content already cached elsewhere
  a->hash[block] = hash;
  a->map_put(hash, block);
  return FQB_OK;
}

uint64_t fqb_hash_block(uint64_t parent, const int32_t* tokens, int n) {
  uint64_t h = parent ^ 0x9E3779B97F4A7C15ull;
  for (int i = 0; i < n; ++i) {
    h ^= static_cast<uint64_t>(static_cast<uint32_t>(tokens[i]));
    h *= 0x100000001B3ull;
    h = (h << 27) | (h >> 37);
  }
  return h ? h : 1;
}

int fqb_acquire_prefix(fqb_alloc* a, const int32_t* tokens, int n_tokens, int32_t* table, int cap,
                       uint64_t* last_hash) {
  if (!a || !tokens || !table || !last_hash) return fqb::set_error(FQB_ERR_STATE, "acquire_prefix: null argument");
  // the last token is always left to compute, so only (n-1)/16 full blocks may be adopted
  int limit = n_tokens > 0 ? (n_tokens - 1) / FQB_BLOCK_TOKENS : 0;
  if (limit > cap) limit = cap;
  uint64_t chain = 0;
  int nb = 0;
  while (nb < limit) {
    const uint64_t h = fqb_hash_block(chain, tokens + nb * FQB_BLOCK_TOKENS, FQB_BLOCK_TOKENS);
    const int b = fqb_alloc_cache_lookup(a, h);
    if (b < 0) break;
    table[nb++] = b;
    chain = h;
  }
  *last_hash = nb > 0 ? chain : 0;
  return nb;
}

int fqb_cache_blocks(fqb_alloc* a, const int32_t* tokens, int computed, const int32_t* table, int cached_blocks,
                     uint64_t* last_hash) {
  if (!a || !tokens || !table || !last_hash) return fqb::set_error(FQB_ERR_STATE, "cache_blocks: null argument");
  const int full = computed / FQB_BLOCK_TOKENS;
  uint64_t chain = *last_hash;
  for (int i = cached_blocks; i < full; ++i) {
    chain = fqb_hash_block(chain, tokens + i * FQB_BLOCK_TOKENS, FQB_BLOCK_TOKENS);
    const int rc = fqb_alloc_cache_insert(a, table[i], chain);
    if (rc != FQB_OK) return rc;
  }
  *last_hash = chain;
  return full;
}

int fqb_cow_prepare(fqb_alloc* a, int32_t* table, int pos, int32_t* pair) {
  if (!a || !table || !pair || pos < 0) return fqb::set_error(FQB_ERR_STATE, "cow_prepare: bad argument");
  const int idx = pos / FQB_BLOCK_TOKENS;
  const int shared = table[idx];
  if (!a->valid(shared)) return fqb::set_error(FQB_ERR_STATE, "cow_prepare: block %d out of range", shared);
  if (a->ref[shared] <= 1 || pos % FQB_BLOCK_TOKENS == 0) return 0;
  const int fresh = fqb_alloc_one(a);
  if (fresh < 0) return fresh;
  pair[0] = shared;
  pair[1] = fresh;
  table[idx] = fresh;
  fqb_alloc_free_one(a, shared);
  return 1;
}

int fqb_step_pack(const int32_t* req_index, int n_rows, int n_req, const int32_t* const* tables,
                  const int32_t* table_len, int bt_stride, int32_t* bt_out, int32_t* qstart, int32_t* qlen,
                  int32_t* decode_rids, int32_t* prefill_rids, int32_t* counts) {
  if (n_rows < 0 || n_req < 0 || (n_rows > 0 && !req_index) || !qstart || !qlen || !decode_rids ||
      !prefill_rids || !counts)
    return fqb::set_error(FQB_ERR_INVALID, "step_pack: bad argument");
  std::memset(qlen, 0, sizeof(int32_t) * static_cast<size_t>(n_req));
  for (int t = 0; t < n_rows; ++t) {
    const int r = req_index[t];
    if (r < 0 || r >= n_req) return fqb::set_error(FQB_ERR_INVALID, "step_pack: row %d names request %d", t, r);
    ++qlen[r];
  }
  int running = 0, nd = 0, np = 0, longest = 1;
  for (int r = 0; r < n_req; ++r) {
    qstart[r] = running;
    running += qlen[r];
    if (qlen[r] == 1) {
      decode_rids[nd++] = r;
    } else {
      prefill_rids[np++] = r;
      if (qlen[r] > longest) longest = qlen[r];
    }
  }
  counts[0] = nd;
  counts[1] = np;
  counts[2] = longest;
  if (tables && bt_out) {
    if (!table_len) return fqb::set_error(FQB_ERR_INVALID, "step_pack: table_len missing");
    for (int r = 0; r < n_req; ++r) {
      if (table_len[r] > bt_stride)
        return fqb::set_error(FQB_ERR_INVALID, "step_pack: request %d has %d blocks, stride is %d", r,
                              table_len[r], bt_stride);
      std::memcpy(bt_out + static_cast<size_t>(r) * bt_stride, tables[r], sizeof(int32_t) * table_len[r]);
    }
  }
  return FQB_OK;
}

}  // extern "C"
