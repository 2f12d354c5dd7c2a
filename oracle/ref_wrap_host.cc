// TEST INFRASTRUCTURE ONLY. extern "C" doors onto the reference's header-only, CUDA-free
// BlockAllocator (engine/src/block_allocator.h), compiled from the reference tree where it lies
// (include path from oracle/Makefile; nothing is copied). Output goes to oracle/_ref/.
#include <cstdint>
#include <vector>

#include "block_allocator.h"

extern "C" {

void* ref_alloc_create(int n) { return new fq::BlockAllocator(n); }
void ref_alloc_destroy(void* h) { delete static_cast<fq::BlockAllocator*>(h); }
int ref_alloc_num_free(void* h) { return static_cast<fq::BlockAllocator*>(h)->NumFree(); }
int ref_alloc_one(void* h) {
  int b = -1;
  return static_cast<fq::BlockAllocator*>(h)->AllocOne(b) ? b : -1;
}
void ref_alloc_free_one(void* h, int b) { static_cast<fq::BlockAllocator*>(h)->FreeOne(b); }
int ref_alloc_grow(void* h, int32_t* table, int* len, int cap, int n_tok) {
  std::vector<int> bt(table, table + *len);
  bool ok = static_cast<fq::BlockAllocator*>(h)->Grow(bt, n_tok);
  for (size_t i = *len; i < bt.size() && static_cast<int>(i) < cap; ++i) table[i] = bt[i];
  *len = static_cast<int>(bt.size());
  return ok ? 1 : 0;
}
int ref_alloc_lookup(void* h, uint64_t hash) {
  return static_cast<fq::BlockAllocator*>(h)->CacheLookup(hash);
}
void ref_alloc_insert(void* h, int b, uint64_t hash) {
  static_cast<fq::BlockAllocator*>(h)->CacheInsert(b, hash);
}

}  // extern "C"
