// Building blocks of the warp-level tensor-core attention kernels: 16-byte asynchronous copies
// into swizzled shared-memory tiles, ldmatrix fragment loads and the m16n8k16 bfloat16 MMA.
//
// A tile of ROWS rows of HD bfloat16 is stored as HD/64 blocks of [ROWS][64 elements]: rows of 128
// bytes, the 16-byte chunk c of row r at chunk position c ^ (r & 7). This is the layout a TMA copy
// with the 128-byte swizzle writes (so tiles may be filled by TMA or by cp.async), and it keeps
// both row-wise stores and the 8x8 ldmatrix reads free of bank conflicts.
#pragma once
#include "common.cuh"

namespace mt {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

template <int HD, int ROWS>
__device__ __forceinline__ uint32_t tile_offset(int row, int chunk) {  // byte offset inside a tile; chunk < HD / 8
  return (uint32_t)((chunk >> 3) * ROWS * 128 + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void st_shared_zero16(uint32_t smem_dst) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(smem_dst), "r"(0u) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

// D (16x8, float32) += A (16x16, row) * B (16x8, col), bfloat16 operands.
// Thread (g = lane / 4, t = lane % 4) holds: A a0 (row g, k 2t..), a1 (row g+8, k 2t..), a2 (row g, k 2t+8..),
// a3 (row g+8, k 2t+8..); B b0 (k 2t.., n g), b1 (k 2t+8.., n g); D d0,d1 (row g, n 2t, 2t+1), d2,d3 (row g+8).
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// A fragments of a 16-row tile for k-step kk (16 values of the head dimension).
template <int HD, int ROWS>
__device__ __forceinline__ void load_a_frag(uint32_t tile, int row0, int kk, int lane, uint32_t (&a)[4]) {
  int row = row0 + (lane & 7) + 8 * ((lane >> 3) & 1);
  ldmatrix_x4(tile + tile_offset<HD, ROWS>(row, 2 * kk + (lane >> 4)), a[0], a[1], a[2], a[3]);
}
// B fragments of K for the product Q K^T: keys key0..key0+15 (two n-tiles), k-step kk.
// r0,r1 = b0,b1 of keys key0..+7; r2,r3 = b0,b1 of keys key0+8..+15.
template <int HD, int ROWS>
__device__ __forceinline__ void load_k_frag(uint32_t tile, int key0, int kk, int lane, uint32_t (&r)[4]) {
  int row = key0 + (lane & 7) + 8 * (lane >> 4);
  ldmatrix_x4(tile + tile_offset<HD, ROWS>(row, 2 * kk + ((lane >> 3) & 1)), r[0], r[1], r[2], r[3]);
}
// B fragments of V for the product P V: keys key0..key0+15 (one k-step), dims 16*dp..16*dp+15 (two n-tiles).
// r0,r1 = b0,b1 of dims 16dp..+7; r2,r3 = b0,b1 of dims 16dp+8..+15.
template <int HD, int ROWS>
__device__ __forceinline__ void load_v_frag(uint32_t tile, int key0, int dp, int lane, uint32_t (&r)[4]) {
  int row = key0 + (lane & 7) + 8 * ((lane >> 3) & 1);
  ldmatrix_x4_trans(tile + tile_offset<HD, ROWS>(row, 2 * dp + (lane >> 4)), r[0], r[1], r[2], r[3]);
}

}  // namespace mt
