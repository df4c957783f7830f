// How kernels address one layer's keys and values inside a paged pool.
//
// A pool is [entries][num_pages][2 (K, V)][kv_heads][page_size][head_dim] (one layer's pages lie together);
// a view fixes the entry (the layer), so
//   K(page, head, slot, d) = base + page * page_stride + (head * page_size + slot) * head_dim + d
//   V(...)                 = the same + v_offset
// The page of position p of segment s is block_table[s * table_stride + p / page_size].
// The reference uses the same block-major idea with a fixed page of 16
// (crates/kir/src/cuda/attention/prim.rs:217; docs/specrt-scheduler.md:20-22).
#pragma once
#include "common.cuh"

struct IbKvView {
  void* base;              // first element of this layer's K in page 0
  long long page_stride;   // elements between consecutive pages
  long long v_offset;      // elements from a K element to the V element of the same place
  const int* block_table;  // [segments][table_stride]
  int table_stride;
  int page_size;
  int num_pages;
  int kv_heads;
  int head_dim;
  int dtype;  // IB_F32 or IB_BF16
};

namespace ib {

// Element offset of (position, kv head) in a view, or -1 when the table has no valid page there.
__device__ __forceinline__ long long kv_offset(const IbKvView& kv, int seg, int pos, int head) {
  int page = kv.block_table[(size_t)seg * kv.table_stride + pos / kv.page_size];
  if (page < 0 || page >= kv.num_pages) return -1;
  return (long long)page * kv.page_stride + ((long long)head * kv.page_size + pos % kv.page_size) * kv.head_dim;
}

}  // namespace ib
