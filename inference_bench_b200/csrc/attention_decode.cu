// Decode attention over the paged cache, bfloat16, split over the context.
//
// One CTA = one decoded token's kv head and one 64-key slice of its context. The query heads that
// share the kv head (the GQA group, up to 16) are the rows of a 16-row MMA tile, so keys and values
// are read from memory once per group. Each of the 4 warps takes 16 keys of the slice:
// S = Q K^T (m16n8k16 bfloat16 MMAs, float32 accumulators), softmax statistics in float32 base 2,
// O = P V; the warps' partial results are merged in shared memory and written to scratch as an
// unnormalised (max, sum, O) triple per (token, head, slice). A second kernel merges the slices.
// Slices are cut at fixed absolute key positions, so a token's result does not depend on the batch.
// Reference design: crates/kir/src/cuda/attention/decode.rs, combine.rs (split-KV with packed GQA rows).
#include <cuda.h>

#include "kv_view.cuh"
#include "mma_tiles.cuh"
#include "sm100.cuh"
#include "tma_host.cuh"

namespace {

constexpr int kWarps = 4;
constexpr int kKeysPerWarp = 16;                 // 16 or 32
constexpr int kTile = kWarps * kKeysPerWarp;     // keys per tile; a CTA walks tiles_per_slice of them
constexpr int kNT = kKeysPerWarp / 8;            // 8-key MMA column tiles per warp
constexpr int kKS = kKeysPerWarp / 16;           // 16-key MMA steps per warp

// How the visible keys [lo, pos] of a decoded token are cut into slices of `tps` tiles from tile `tile_lo` on.
// tiles_per_slice > 0: slices of that many tiles at fixed absolute positions. 0: the token's own visible
// tiles in max_slices equal parts of at least kMinTiles tiles, so that every token gives about as many
// units of work, of about equal size, whatever its length.
constexpr int kMinTiles = 2;
__device__ __forceinline__ void slice_plan(int pos, int window, int max_slices, int tiles_per_slice, int& lo, int& tile_lo, int& tps) {
  lo = window > 0 ? max(0, pos - window + 1) : 0;
  if (tiles_per_slice > 0) {
    tile_lo = 0;
    tps = tiles_per_slice;
    return;
  }
  tile_lo = lo / kTile;
  const int tiles = pos / kTile - tile_lo + 1;
  tps = max(kMinTiles, (tiles + max_slices - 1) / max_slices);
}

template <int HD>
__global__ void __launch_bounds__(kWarps * 32)
    decode_split_kernel(const __nv_bfloat16* __restrict__ q, IbKvView kv, const int* __restrict__ dec_tokens,
                        const int* __restrict__ positions, const int* __restrict__ seg_of_token, int window, float scale_log2e,
                        float* __restrict__ part_o, float* __restrict__ part_ml, int heads, int max_slices, int tiles_per_slice,
                        unsigned* __restrict__ status) {
  constexpr int CPR = HD / 8;              // 16-byte chunks per row
  constexpr int TILE = kTile * HD * 2;     // bytes of one K (or V) tile
  extern __shared__ __align__(1024) uint8_t smem[];
  // layout: Q tile [16][HD] | 2 stages x (K tile, V tile) | key offsets [2][kTile]; the merge buffers reuse the tiles
  const uint32_t q_s = mt::smem_u32(smem);
  const uint32_t kv_s = q_s + 16 * HD * 2;
  long long* offs = (long long*)(smem + 16 * HD * 2 + 4 * TILE);

  // What the kernel before this one in the stream writes is q and the key and value of each token's
  // own position; the index arrays, the block table and every older key and value were complete
  // before the step began. So the first tile of older keys is requested before the dependency
  // wait (it then travels while the kernel before still runs); q and the row of the token's own
  // position are fetched after it.
  ib::pdl_launch_dependents();
  const int kvh = blockIdx.x, item = blockIdx.y, slice = blockIdx.z;
  const int t = dec_tokens[item];
  const int pos = positions[t], seg = seg_of_token[t];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int slice_keys = tiles_per_slice * kTile;
  const int k_begin = max(lo, slice * slice_keys), k_end = min(pos + 1, (slice + 1) * slice_keys);
  if (k_begin >= k_end) return;
  const int tile_begin = k_begin / kTile, tile_end = (k_end - 1) / kTile + 1;
  const int group = heads / kv.kv_heads;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, tq = lane & 3;
  const __nv_bfloat16* base = (const __nv_bfloat16*)kv.base;

  // One thread per key looks its page up; then all threads copy 16-byte chunks.
  // `own_later`: leave out the row of the token's own position (it is not written yet); it is fetched after the wait.
  auto load_tile = [&](int tile, int stage, bool own_later = false) {
    long long* o = offs + stage * kTile;
    if (tid < kTile) {
      int key = tile * kTile + tid;
      long long off = (key >= k_begin && key < k_end) ? ib::kv_offset(kv, seg, key, kvh) : -2;
      if (off == -1) atomicOr(status, IB_ERR_BAD_PAGE);
      o[tid] = off;
    }
    __syncthreads();
    const uint32_t k_s = kv_s + stage * 2 * TILE, v_s = k_s + TILE;
    for (int idx = tid; idx < kTile * CPR; idx += kWarps * 32) {
      int row = idx / CPR, c = idx % CPR;
      long long off = o[row];
      if (own_later && tile * kTile + row == pos) continue;
      uint32_t kd = k_s + mt::tile_offset<HD, kTile>(row, c), vd = v_s + mt::tile_offset<HD, kTile>(row, c);
      if (off >= 0) {
        mt::cp_async16(kd, base + off + c * 8);
        mt::cp_async16(vd, base + off + kv.v_offset + c * 8);
      } else {
        mt::st_shared_zero16(kd);
        mt::st_shared_zero16(vd);
      }
    }
  };

  // ---- the first tile of older keys, then (after the dependency wait) Q and the token's own row
  load_tile(tile_begin, 0, true);
  ib::pdl_wait();
  if (pos / kTile == tile_begin && pos >= k_begin && pos < k_end) {
    const long long off = offs[pos % kTile];
    const int row = pos % kTile;
    for (int c = tid; c < CPR; c += kWarps * 32) {
      const uint32_t kd = kv_s + mt::tile_offset<HD, kTile>(row, c), vd = kd + TILE;
      if (off >= 0) {
        mt::cp_async16(kd, base + off + c * 8);
        mt::cp_async16(vd, base + off + kv.v_offset + c * 8);
      } else {
        mt::st_shared_zero16(kd);
        mt::st_shared_zero16(vd);
      }
    }
  }
  // Q: rows = the group's heads, zero rows above
  for (int idx = tid; idx < 16 * CPR; idx += kWarps * 32) {
    int row = idx / CPR, c = idx % CPR;
    uint32_t dst = q_s + mt::tile_offset<HD, 16>(row, c);
    if (row < group)
      mt::cp_async16(dst, q + ((size_t)t * heads + (size_t)kvh * group + row) * HD + c * 8);
    else
      mt::st_shared_zero16(dst);
  }
  mt::cp_async_commit();

  // ---- running softmax state of this warp's share of the keys (rows g and g+8 of the 16-row tile)
  const int wkey = warp * kKeysPerWarp;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[HD / 8][4];
#pragma unroll
  for (int n = 0; n < HD / 8; n++)
#pragma unroll
    for (int e = 0; e < 4; e++) o[n][e] = 0.f;

  for (int tile = tile_begin; tile < tile_end; tile++) {
    const int stage = (tile - tile_begin) & 1;
    const uint32_t k_s = kv_s + stage * 2 * TILE, v_s = k_s + TILE;
    if (tile + 1 < tile_end) {
      load_tile(tile + 1, stage ^ 1);
      mt::cp_async_commit();
      mt::cp_async_wait<1>();
    } else {
      mt::cp_async_wait<0>();
    }
    __syncthreads();
    // S = Q K^T for this warp's keys of the tile
    float s[kNT][4];
#pragma unroll
    for (int j = 0; j < kNT; j++)
#pragma unroll
      for (int e = 0; e < 4; e++) s[j][e] = 0.f;
#pragma unroll
    for (int kk = 0; kk < HD / 16; kk++) {
      uint32_t a[4], b[4];
      mt::load_a_frag<HD, 16>(q_s, 0, kk, lane, a);
#pragma unroll
      for (int pr = 0; pr < kKS; pr++) {
        mt::load_k_frag<HD, kTile>(k_s, wkey + 16 * pr, kk, lane, b);
        mt::mma_16816(s[2 * pr], a, b[0], b[1]);
        mt::mma_16816(s[2 * pr + 1], a, b[2], b[3]);
      }
    }
    // mask, running max
    float mn[2] = {m[0], m[1]};
#pragma unroll
    for (int j = 0; j < kNT; j++)
#pragma unroll
      for (int e = 0; e < 4; e++) {
        int key = tile * kTile + wkey + 8 * j + 2 * tq + (e & 1);
        float v = (key >= k_begin && key < k_end) ? s[j][e] * scale_log2e : -INFINITY;
        s[j][e] = v;
        mn[e >> 1] = fmaxf(mn[e >> 1], v);
      }
    float mu[2], corr[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
      mn[r] = fmaxf(mn[r], __shfl_xor_sync(0xffffffffu, mn[r], 1));
      mn[r] = fmaxf(mn[r], __shfl_xor_sync(0xffffffffu, mn[r], 2));
      mu[r] = mn[r] == -INFINITY ? 0.f : mn[r];
      corr[r] = exp2f(m[r] - mu[r]);   // 0 while m is still -inf
      m[r] = mn[r];
      l[r] *= corr[r];
    }
    if (tile > tile_begin) {
#pragma unroll
      for (int n = 0; n < HD / 8; n++) {
        o[n][0] *= corr[0];
        o[n][1] *= corr[0];
        o[n][2] *= corr[1];
        o[n][3] *= corr[1];
      }
    }
    uint32_t p[kKS][4];  // A fragments of P, one per 16-key step
#pragma unroll
    for (int j = 0; j < kNT; j++) {
      float e0 = exp2f(s[j][0] - mu[0]), e1 = exp2f(s[j][1] - mu[0]), e2 = exp2f(s[j][2] - mu[1]), e3 = exp2f(s[j][3] - mu[1]);
      l[0] += e0 + e1;
      l[1] += e2 + e3;
      p[j >> 1][(j & 1) * 2] = mt::pack_bf16(e0, e1);
      p[j >> 1][(j & 1) * 2 + 1] = mt::pack_bf16(e2, e3);
    }
    // O += P V over this warp's keys
#pragma unroll
    for (int ks = 0; ks < kKS; ks++)
#pragma unroll
      for (int dp = 0; dp < HD / 16; dp++) {
        uint32_t b[4];
        mt::load_v_frag<HD, kTile>(v_s, wkey + 16 * ks, dp, lane, b);
        mt::mma_16816(o[2 * dp], p[ks], b[0], b[1]);
        mt::mma_16816(o[2 * dp + 1], p[ks], b[2], b[3]);
      }
    __syncthreads();  // every warp is done with this stage before it is loaded again
  }
#pragma unroll
  for (int r = 0; r < 2; r++) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
  // ---- merge the four warps through shared memory (the tiles are no longer needed); only the
  // rows that are real heads of the group are stored
  float* ml_s = (float*)smem;                                  // [warps][16][2], in the Q tile
  float* o_s = (float*)(smem + 16 * HD * 2);                   // [warps][16][HD], in the K and V tiles
  if (tq == 0) {
    ml_s[(warp * 16 + g) * 2] = m[0];
    ml_s[(warp * 16 + g) * 2 + 1] = l[0];
    ml_s[(warp * 16 + g + 8) * 2] = m[1];
    ml_s[(warp * 16 + g + 8) * 2 + 1] = l[1];
  }
#pragma unroll
  for (int n = 0; n < HD / 8; n++) {
    int d = 8 * n + 2 * tq;
    if (g < group) *(float2*)&o_s[(warp * 16 + g) * HD + d] = make_float2(o[n][0], o[n][1]);
    if (g + 8 < group) *(float2*)&o_s[(warp * 16 + g + 8) * HD + d] = make_float2(o[n][2], o[n][3]);
  }
  __syncthreads();
  for (int idx = tid; idx < group * HD; idx += kWarps * 32) {
    int row = idx / HD, d = idx % HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; w++) M = fmaxf(M, ml_s[(w * 16 + row) * 2]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; w++) {
      float mw = ml_s[(w * 16 + row) * 2];
      float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
      L += ml_s[(w * 16 + row) * 2 + 1] * f;
      O += o_s[(w * 16 + row) * HD + d] * f;
    }
    size_t slot = ((size_t)item * heads + (size_t)kvh * group + row) * max_slices + slice;
    part_o[slot * HD + d] = O;
    if (d == 0) {
      part_ml[slot * 2] = M;
      part_ml[slot * 2 + 1] = L;
    }
  }
}

// out[token][head] = sum over the slices that hold visible keys of O_s 2^(m_s - M) / sum of l_s 2^(m_s - M).
// One CTA per (head, token): kCombineThreads threads as [slice lanes][head_dim / 4]; a thread sums every
// lane-th slice for four values of the head, and the lanes are added in order through shared memory.
constexpr int kCombineThreads = 256;

template <int HD>
__global__ void __launch_bounds__(kCombineThreads)
    decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, const int* __restrict__ dec_tokens,
                          const int* __restrict__ positions, int window, __nv_bfloat16* __restrict__ out, int heads, int max_slices,
                          int tiles_per_slice, unsigned* __restrict__ status) {
  constexpr int DQ = HD / 4;
  constexpr int SG = kCombineThreads / DQ;
  __shared__ float4 o_red[SG][DQ];
  __shared__ float m_red[SG], l_red[SG];
  ib::pdl_launch_dependents();
  const int h = blockIdx.x, item = blockIdx.y;
  const int t = dec_tokens[item];
  const int pos = positions[t];
  int lo, tile_lo, tps;
  slice_plan(pos, window, max_slices, tiles_per_slice, lo, tile_lo, tps);
  const int s_begin = (lo / kTile - tile_lo) / tps;
  int s_end = (pos / kTile - tile_lo) / tps + 1;
  if (s_end > max_slices) {   // the caller's max_slices does not cover this position: nothing beyond the scratch is read, and the status says so
    if (threadIdx.x == 0) atomicOr(status, IB_ERR_INTERNAL);
    s_end = max_slices;
  }
  const size_t slot0 = ((size_t)item * heads + h) * max_slices;
  const int sg = threadIdx.x / DQ, dq = threadIdx.x % DQ;
  ib::pdl_wait();
  // the thread's first slice (with up to SG slices, its only one) is requested whole before anything is waited for:
  // one trip to memory instead of two, one after the other
  const int s0 = s_begin + sg;
  const bool have = s0 < s_end;
  float m0 = -INFINITY, l0 = 0.f;
  float4 v0 = make_float4(0.f, 0.f, 0.f, 0.f);
  if (have) {
    m0 = part_ml[(slot0 + s0) * 2];
    l0 = part_ml[(slot0 + s0) * 2 + 1];
    v0 = *(const float4*)&part_o[(slot0 + s0) * HD + 4 * dq];
  }
  float mx = m0;
  for (int s = s0 + SG; s < s_end; s += SG) mx = fmaxf(mx, part_ml[(slot0 + s) * 2]);
  if (dq == 0) m_red[sg] = mx;
  __syncthreads();
  float M = -INFINITY;
#pragma unroll
  for (int i = 0; i < SG; i++) M = fmaxf(M, m_red[i]);
  float Lp = 0.f;
  float4 Op = make_float4(0.f, 0.f, 0.f, 0.f);
  if (have) {
    const float f = exp2f(m0 - M);
    Lp = l0 * f;
    Op = make_float4(v0.x * f, v0.y * f, v0.z * f, v0.w * f);
  }
  for (int s = s0 + SG; s < s_end; s += SG) {
    const float f = exp2f(part_ml[(slot0 + s) * 2] - M);
    Lp += part_ml[(slot0 + s) * 2 + 1] * f;
    const float4 v = *(const float4*)&part_o[(slot0 + s) * HD + 4 * dq];
    Op.x += v.x * f;
    Op.y += v.y * f;
    Op.z += v.z * f;
    Op.w += v.w * f;
  }
  o_red[sg][dq] = Op;
  if (dq == 0) l_red[sg] = Lp;
  __syncthreads();
  if (sg == 0) {
    float Lsum = 0.f;
    float4 O = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < SG; i++) {
      Lsum += l_red[i];
      const float4 v = o_red[i][dq];
      O.x += v.x;
      O.y += v.y;
      O.z += v.z;
      O.w += v.w;
    }
    if (!(Lsum > 0.f)) {
      O = make_float4(0.f, 0.f, 0.f, 0.f);
      Lsum = 1.f;
    }
    uint2 packed = make_uint2(mt::pack_bf16(O.x / Lsum, O.y / Lsum), mt::pack_bf16(O.z / Lsum, O.w / Lsum));
    *(uint2*)&out[((size_t)t * heads + h) * HD + 4 * dq] = packed;
  }
}

// ---------------------------------------------------------------- the streaming variant
//
// The same slices, the same arithmetic and the same scratch, but CTAs that stay: a CTA takes every
// gridDim.x-th unit (slice, token, kv head), and a fifth warp runs ahead of the four computing warps
// through a ring of kRing tiles that TMA box copies fill (one box per page, plane and 64 values of
// the head dimension). The ring does not drain where a unit ends, so copies are in flight all the
// time; with one short-lived CTA per unit the memory system idles while each CTA looks its pages
// up and while it merges its warps. Needs the tensor map of the pool (ib_make_kv_map).
constexpr int kRing = 3;
constexpr int kMeta = 256;   // decoded tokens whose row, position and segment are kept in shared memory

__device__ __forceinline__ void bar_sync_compute() { asm volatile("bar.sync 1, %0;" ::"n"(kWarps * 32) : "memory"); }

// What the fused form works from instead of finished queries: the products of the q/k/v projection as the
// matrix-product kernel left them (float32 partial sums [P][T][(heads + 2 kv_heads) * head_dim]), the
// per-head norm scales (or null) and the step's rotation tables (or null). The kernel then norms and turns
// the queries itself, and the CTA whose slice holds a token's own position does the same for its key,
// stores key and value in the cache (write_kv) and attends to them from shared memory: the own position
// is never read back from the cache, so nothing this kernel copies depends on the kernel before it.
struct RawQkv {
  const float* qkv;
  int P;
  long long stride_p;
  const float* q_norm_w;
  const float* k_norm_w;
  float eps;
  const float* cos_t;
  const float* sin_t;
  int write_kv;
};

template <int HD, bool FUSED>
__global__ void __launch_bounds__((kWarps + 1) * 32, 2)
    decode_stream_kernel(const __nv_bfloat16* __restrict__ q, RawQkv raw, IbKvView kv, const int* __restrict__ dec_tokens, const int* __restrict__ positions,
                         const int* __restrict__ seg_of_token, int window, float scale_log2e, float* __restrict__ part_o,
                         float* __restrict__ part_ml, int heads, int n_dec, int max_slices, int tiles_per_slice, int merge_cols,
                         const __grid_constant__ CUtensorMap kv_map, long long view_row0, unsigned long long wait_ns, unsigned* __restrict__ status) {
  constexpr int CPR = HD / 8;
  constexpr int TILE = kTile * HD * 2;
  constexpr int HB = HD / 64;
  extern __shared__ __align__(1024) uint8_t smem[];
  const int group = heads / kv.kv_heads;
  // layout: kRing x (K tile, V tile) | Q tile [16][HD] | (max, sum) [warps][16] | O [warps][group][merge_cols] | barriers | flag | token table | own key, value, scores
  uint8_t* ring = smem;
  const uint32_t q_s = mt::smem_u32(smem + kRing * 2 * TILE);
  float* ml_s = (float*)(smem + kRing * 2 * TILE + 16 * HD * 2);
  float* o_s = ml_s + kWarps * 16 * 2;
  uint64_t* full = (uint64_t*)(o_s + kWarps * group * merge_cols);
  uint64_t* empty = full + kRing;
  volatile int* gave_up = (volatile int*)(empty + kRing);
  int* meta = (int*)(empty + kRing) + 2;   // [kMeta][3]
  float* k_own = (float*)(meta + 3 * kMeta);   // fused form: the token's own key and value (bfloat16 values), and its scores per head
  float* v_own = k_own + HD;
  float* s_own = v_own + HD;                   // [16]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if ((mt::smem_u32(smem) & 1023u) != 0) {   // the swizzle of the box copies counts from 1024-byte boundaries
    if (tid == 0) atomicOr(status, IB_ERR_INTERNAL);
    return;
  }
  if (tid == 0) {
    for (int s = 0; s < kRing; s++) {
      sm100::mbar_init(&full[s], 1);
      sm100::mbar_init(&empty[s], kWarps);
    }
    *gave_up = 0;
    sm100::fence_barrier_init();
  }
  __syncthreads();
  ib::pdl_launch_dependents();

  const int n_units = max_slices * n_dec * kv.kv_heads;
  // Row, position and segment of the first kMeta decoded tokens, fetched once: opening a unit then costs
  // no chain of loads from global memory. Index arrays and the block table were complete before the
  // step began, so they are read without waiting for the kernel before.
  for (int i = tid; i < min(n_dec, kMeta); i += (kWarps + 1) * 32) {
    const int tt = dec_tokens[i];
    meta[3 * i] = tt;
    meta[3 * i + 1] = positions[tt];
    meta[3 * i + 2] = seg_of_token[tt];
  }
  __syncthreads();
  // unit -> what it covers; false when it holds no visible key
  int kvh, item, slice, t, pos, seg, k_begin, k_end;
  bool has_own = false;   // fused form: the unit's slice holds the token's own position
  auto open_unit = [&](int u) {
    kvh = u % kv.kv_heads;
    const int r = u / kv.kv_heads;
    item = r % n_dec;
    slice = r / n_dec;
    if (item < kMeta) {
      t = meta[3 * item];
      pos = meta[3 * item + 1];
      seg = meta[3 * item + 2];
    } else {
      t = dec_tokens[item];
      pos = positions[t];
      seg = seg_of_token[t];
    }
    int lo, tile_lo, tps;
    slice_plan(pos, window, max_slices, tiles_per_slice, lo, tile_lo, tps);
    k_begin = max(lo, (tile_lo + slice * tps) * kTile);
    k_end = min(pos + 1, (tile_lo + (slice + 1) * tps) * kTile);
    if constexpr (FUSED) {   // the own position comes from the projection, not from the cache
      has_own = k_begin < k_end && k_end == pos + 1;
      if (has_own) k_end = pos;
      return has_own || k_begin < k_end;
    }
    return k_begin < k_end;
  };
  auto next_unit = [&](int u) {   // the first unit from u on, in this CTA's stride, that holds a visible key; opened
    while (u < n_units && !open_unit(u)) u += gridDim.x;
    return u;
  };

  if (warp == kWarps) {
    // ---------------- the copying warp
    // A lane owns one box of every tile: box b_pg of the tile's keys (a page, where a page holds fewer keys than a tile),
    // plane b_plane and 64-value block b_hb. What does not change from tile to tile is computed once, and the row of a box in
    // the pool when its page is looked up (32 boxes at a time, one per lane): the loop over the tiles divides nothing.
    const int box_rows = min(kv.page_size, kTile);   // rows of one box: a page, or the tile's part of a larger page
    const int ppt = kTile / box_rows;                // boxes per tile, plane and 64-value block
    const int boxes = ppt * HB * 2;
    const int boxes_per_page = kv.page_size / box_rows;
    const long long rows_per_page = kv.page_stride / HD;
    const int v_rows = (int)(kv.v_offset / HD);
    const int b_pg = lane / (HB * 2), b_plane = (lane / HB) & 1, b_hb = lane % HB;
    const bool has_box = lane < boxes;
    const uint32_t box_bytes = (uint32_t)box_rows * 128;
    const uint32_t dst_lane = b_plane * TILE + b_hb * kTile * 128 + b_pg * box_bytes;
    uint32_t n = 0;        // tiles sent so far
    int stage = 0;
    uint32_t parity = 1;   // of the stage's "empty" barrier
    bool waited = false;   // the kernel before this one writes only the rows of the tokens' own positions
    bool ok = true;
    for (int u = next_unit(blockIdx.x); u < n_units && ok; u = next_unit(u + gridDim.x)) {
      const int tile_begin = k_begin / kTile, tile_end = k_begin < k_end ? (k_end - 1) / kTile + 1 : tile_begin;
      int held_row = -1;   // where in the pool the K rows of box (tile_begin * ppt + rel + lane) begin, or -1: nothing to copy
      for (int tile = tile_begin; tile < tile_end; tile++, n++) {
        const int rel = (tile - tile_begin) * ppt;
        if ((rel & 31) == 0) {
          const int box = tile_begin * ppt + rel + lane;
          const int key0 = box * box_rows;
          held_row = -1;
          if (key0 < k_end && key0 + box_rows > k_begin) {
            const int col = boxes_per_page == 1 ? box : box / boxes_per_page;
            const int page = col < kv.table_stride ? kv.block_table[(size_t)seg * kv.table_stride + col] : -1;
            if (page >= 0 && page < kv.num_pages)
              held_row = (int)((long long)page * rows_per_page + view_row0 + (long long)kvh * kv.page_size + (key0 - col * kv.page_size));
            else
              atomicOr(status, IB_ERR_BAD_PAGE);
          }
        }
        const int row = __shfl_sync(0xffffffffu, held_row, (rel + b_pg) & 31);
        const bool mine = has_box && row >= 0;
        const unsigned vmask = __ballot_sync(0xffffffffu, mine);
        const int n_ok = __popc(vmask);
        if (!FUSED && !waited && pos >= tile * kTile && pos < (tile + 1) * kTile) {
          ib::pdl_wait();
          waited = true;
        }
        if (lane == 0) ok = sm100::mbar_wait(&empty[stage], parity, wait_ns);
        ok = __shfl_sync(0xffffffffu, ok, 0) && !*gave_up;
        if (!ok) break;
        uint8_t* k_t = ring + stage * 2 * TILE;
        if (n_ok != boxes) {   // boxes that are not copied (no visible key in them, or no page) are cleared: a masked key's value still meets a zero weight
          for (int b = 0; b < boxes; b++) {
            if ((vmask >> b) & 1) continue;
            const uint32_t d0 = mt::smem_u32(k_t) + ((b / HB) & 1) * TILE + (b % HB) * kTile * 128 + (b / (HB * 2)) * box_bytes;
            for (int idx = lane; idx < box_rows * 8; idx += 32) mt::st_shared_zero16(d0 + idx * 16);
          }
          sm100::fence_proxy_async();
          __syncwarp();
        }
        if (lane == 0) sm100::mbar_arrive_expect_tx(&full[stage], (uint32_t)n_ok * box_bytes);
        if (mine) sm100::tma_load_2d(k_t + dst_lane, &kv_map, b_hb * 64, row + b_plane * v_rows, &full[stage]);
        if (++stage == kRing) stage = 0, parity ^= 1;
      }
    }
    if (!ok) {   // a wait ran out: say so, and let the copies in flight land before the shared memory goes
      if (lane == 0) {
        *gave_up = 1;
        atomicOr(status, IB_ERR_WAIT_TIMEOUT);
        for (uint32_t j = n > kRing ? n - kRing : 0; j < n; j++) sm100::mbar_wait(&full[j % kRing], (j / kRing) & 1, wait_ns);
      }
    }
    return;
  }

  // ---------------- the four computing warps
  const int g = lane >> 2, tq = lane & 3;
  const int wkey = warp * kKeysPerWarp;
  ib::pdl_wait();   // q comes from the kernel before
  uint32_t n = 0;
  bool dead = false;
  for (int idx = tid; idx < 16 * CPR; idx += kWarps * 32)   // rows above the group stay zero
    if (idx / CPR >= group) mt::st_shared_zero16(q_s + mt::tile_offset<HD, 16>(idx / CPR, idx % CPR));
  auto fetch_q = [&]() {   // the opened unit's query rows into the Q tile
    for (int idx = tid; idx < group * CPR; idx += kWarps * 32) {
      const int row = idx / CPR, c = idx % CPR;
      mt::cp_async16(q_s + mt::tile_offset<HD, 16>(row, c), q + ((size_t)t * heads + (size_t)kvh * group + row) * HD + c * 8);
    }
    mt::cp_async_commit();
  };
  // ---- the fused form: one head of the projection's output -> summed, normed, turned; E values per lane
  constexpr int E = HD / 32;
  const int R = (heads + 2 * kv.kv_heads) * HD;
  auto load_head = [&](int j, float (&v)[E]) {   // the sum, in order, of the partial products of head j
    const float* src = raw.qkv + (size_t)t * R + (size_t)j * HD + lane * E;
#pragma unroll
    for (int e = 0; e < E; e++) v[e] = 0.f;
    for (int p = 0; p < raw.P; p++) {
      if constexpr (E == 4) {
        const float4 a = *(const float4*)(src + p * raw.stride_p);
        v[0] += a.x, v[1] += a.y, v[2] += a.z, v[3] += a.w;
      } else {
        const float2 a = *(const float2*)(src + p * raw.stride_p);
        v[0] += a.x, v[1] += a.y;
      }
    }
  };
  auto load_two_heads = [&](int j1, float (&v1)[E], int j2, float (&v2)[E]) {   // two heads, their loads side by side
    const float* s1 = raw.qkv + (size_t)t * R + (size_t)j1 * HD + lane * E;
    const float* s2 = raw.qkv + (size_t)t * R + (size_t)j2 * HD + lane * E;
#pragma unroll
    for (int e = 0; e < E; e++) v1[e] = 0.f, v2[e] = 0.f;
    for (int p = 0; p < raw.P; p++) {
      if constexpr (E == 4) {
        const float4 a = *(const float4*)(s1 + p * raw.stride_p), b = *(const float4*)(s2 + p * raw.stride_p);
        v1[0] += a.x, v1[1] += a.y, v1[2] += a.z, v1[3] += a.w;
        v2[0] += b.x, v2[1] += b.y, v2[2] += b.z, v2[3] += b.w;
      } else {
        const float2 a = *(const float2*)(s1 + p * raw.stride_p), b = *(const float2*)(s2 + p * raw.stride_p);
        v1[0] += a.x, v1[1] += a.y;
        v2[0] += b.x, v2[1] += b.y;
      }
    }
  };
  // (the norm's weights and the rotation's table entries are requested by the caller beside the partial products,
  // not here after the sums: one trip to memory, not three one after the other)
  auto finish_head = [&](bool norm, const float (&nw)[E], bool turn, const float (&c)[E], const float (&sn)[E], float (&v)[E]) {   // norm and rotation
    if (norm) {
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < E; e++) ss += v[e] * v[e];
      ss = ib::warp_sum(ss);
      const float inv = rsqrtf(ss / (float)HD + raw.eps);
#pragma unroll
      for (int e = 0; e < E; e++) v[e] = nw[e] * (v[e] * inv);
    }
    if (turn && raw.cos_t) {
#pragma unroll
      for (int e = 0; e < E; e++) {
        const float other = __shfl_xor_sync(0xffffffffu, v[e], 16);
        v[e] = lane < 16 ? v[e] * c[e] - other * sn[e] : v[e] * c[e] + other * sn[e];
      }
    }
  };
  auto q_row_addr = [&](int row) { return q_s + mt::tile_offset<HD, 16>(row, lane * E / 8) + (lane * E * 2) % 16; };   // this lane's E values of a Q row
  auto make_unit_inputs = [&]() {   // the opened unit's query rows, and its own key and value if its slice holds them
    const bool own_mine = has_own && warp < 2;   // warp 0: the key (normed and turned); warp 1: the value
    float vo[E], c[E], sn[E], qw[E], kw[E];
#pragma unroll
    for (int e = 0; e < E; e++) {
      c[e] = raw.cos_t ? raw.cos_t[(size_t)t * (HD / 2) + (lane & 15) * E + e] : 1.f;
      sn[e] = raw.cos_t ? raw.sin_t[(size_t)t * (HD / 2) + (lane & 15) * E + e] : 0.f;
      qw[e] = raw.q_norm_w ? raw.q_norm_w[lane * E + e] : 1.f;
      kw[e] = own_mine && warp == 0 && raw.k_norm_w ? raw.k_norm_w[lane * E + e] : 1.f;
    }
    const int own_j = warp == 0 ? heads + kvh : heads + kv.kv_heads + kvh;
    const bool together = own_mine && warp < group;   // the own key or value is requested together with the warp's first query row
    if (own_mine && !together) load_head(own_j, vo);
    for (int row = warp; row < group; row += kWarps) {
      float v[E];
      if (together && row == warp)
        load_two_heads(own_j, vo, kvh * group + row, v);
      else
        load_head(kvh * group + row, v);
      finish_head(raw.q_norm_w != nullptr, qw, true, c, sn, v);
      if constexpr (E == 4)
        asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(q_row_addr(row)), "r"(mt::pack_bf16(v[0], v[1])), "r"(mt::pack_bf16(v[2], v[3])) : "memory");
      else
        asm volatile("st.shared.b32 [%0], %1;" ::"r"(q_row_addr(row)), "r"(mt::pack_bf16(v[0], v[1])) : "memory");
    }
    if (own_mine) {
      float (&v)[E] = vo;
      finish_head(warp == 0 && raw.k_norm_w != nullptr, kw, warp == 0, c, sn, v);
      __nv_bfloat16 b[E];
      float* own = warp == 0 ? k_own : v_own;
#pragma unroll
      for (int e = 0; e < E; e++) {
        b[e] = __float2bfloat16_rn(v[e]);
        own[lane * E + e] = __bfloat162float(b[e]);
      }
      if (raw.write_kv) {
        const long long off = ib::kv_offset(kv, seg, pos, kvh);
        if (off < 0) {
          if (lane == 0) atomicOr(status, IB_ERR_BAD_PAGE);
        } else {
          __nv_bfloat16* dst = (__nv_bfloat16*)kv.base + off + (warp == 0 ? 0 : kv.v_offset) + lane * E;
          if constexpr (E == 4)
            *(uint2*)dst = *(const uint2*)b;
          else
            *(uint32_t*)dst = *(const uint32_t*)b;
        }
      }
    }
  };
  auto own_scores = [&]() {   // s_own[row] = scale * q_row . k_own, from the rounded values the tensor core would see
    for (int row = warp; row < group; row += kWarps) {
      float dot = 0.f;
      uint32_t w0, w1 = 0;
      if constexpr (E == 4)
        asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(w0), "=r"(w1) : "r"(q_row_addr(row)));
      else
        asm volatile("ld.shared.b32 %0, [%1];" : "=r"(w0) : "r"(q_row_addr(row)));
      dot += __uint_as_float(w0 << 16) * k_own[lane * E] + __uint_as_float(w0 & 0xffff0000u) * k_own[lane * E + 1];
      if constexpr (E == 4) dot += __uint_as_float(w1 << 16) * k_own[lane * E + 2] + __uint_as_float(w1 & 0xffff0000u) * k_own[lane * E + 3];
      dot = ib::warp_sum(dot);
      if (lane == 0) s_own[row] = dot * scale_log2e;
    }
  };

  int u = next_unit(blockIdx.x);
  if (!FUSED && u < n_units) fetch_q();
  while (u < n_units) {
    if constexpr (FUSED) {
      bar_sync_compute();   // every warp is done with the last unit's Q tile and merge buffers
      make_unit_inputs();
    } else {
      mt::cp_async_wait<0>();
    }
    bar_sync_compute();   // the Q tile is whole; every warp is done with the last unit's merge buffers
    uint32_t qa[HD / 16][4];
#pragma unroll
    for (int kk = 0; kk < HD / 16; kk++) mt::load_a_frag<HD, 16>(q_s, 0, kk, lane, qa[kk]);
    if (FUSED && has_own) own_scores();
    if (!FUSED) bar_sync_compute();   // every warp holds its fragments: the Q tile is free for the next unit's rows, which travel during this unit
    const bool own_here = has_own;
    const int u_next = next_unit(u + gridDim.x);
    if (!FUSED && u_next < n_units) fetch_q();
    open_unit(u);
    const int tile_begin = k_begin / kTile, tile_end = k_begin < k_end ? (k_end - 1) / kTile + 1 : tile_begin;

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; i++)
#pragma unroll
      for (int e = 0; e < 4; e++) o[i][e] = 0.f;

    for (int tile = tile_begin; tile < tile_end; tile++, n++) {
      const int stage = n % kRing;
      // After a wait that ran out nothing is waited for any more; the loops still run to their ends,
      // so that every warp meets the others at the barriers (the results are then void, and the status says so).
      if (!dead) {
        if (!sm100::mbar_wait(&full[stage], (n / kRing) & 1, wait_ns)) {
          *gave_up = 1;
          if (lane == 0) atomicOr(status, IB_ERR_WAIT_TIMEOUT);
        }
        if (*gave_up) dead = true;
      }
      __syncwarp();
      const uint32_t k_s = mt::smem_u32(ring + stage * 2 * TILE), v_s = k_s + TILE;
      float s[kNT][4];
#pragma unroll
      for (int j = 0; j < kNT; j++)
#pragma unroll
        for (int e = 0; e < 4; e++) s[j][e] = 0.f;
#pragma unroll
      for (int kk = 0; kk < HD / 16; kk++) {
        uint32_t b[4];
#pragma unroll
        for (int pr = 0; pr < kKS; pr++) {
          mt::load_k_frag<HD, kTile>(k_s, wkey + 16 * pr, kk, lane, b);
          mt::mma_16816(s[2 * pr], qa[kk], b[0], b[1]);
          mt::mma_16816(s[2 * pr + 1], qa[kk], b[2], b[3]);
        }
      }
      float mn[2] = {m[0], m[1]};
#pragma unroll
      for (int j = 0; j < kNT; j++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
          const int key = tile * kTile + wkey + 8 * j + 2 * tq + (e & 1);
          const float v = (key >= k_begin && key < k_end) ? s[j][e] * scale_log2e : -INFINITY;
          s[j][e] = v;
          mn[e >> 1] = fmaxf(mn[e >> 1], v);
        }
      float mu[2], corr[2];
#pragma unroll
      for (int r = 0; r < 2; r++) {
        mn[r] = fmaxf(mn[r], __shfl_xor_sync(0xffffffffu, mn[r], 1));
        mn[r] = fmaxf(mn[r], __shfl_xor_sync(0xffffffffu, mn[r], 2));
        mu[r] = mn[r] == -INFINITY ? 0.f : mn[r];
        corr[r] = exp2f(m[r] - mu[r]);   // 0 while m is still -inf
        m[r] = mn[r];
        l[r] *= corr[r];
      }
      if (tile > tile_begin) {
#pragma unroll
        for (int i = 0; i < HD / 8; i++) {
          o[i][0] *= corr[0];
          o[i][1] *= corr[0];
          o[i][2] *= corr[1];
          o[i][3] *= corr[1];
        }
      }
      uint32_t p[kKS][4];
#pragma unroll
      for (int j = 0; j < kNT; j++) {
        const float e0 = exp2f(s[j][0] - mu[0]), e1 = exp2f(s[j][1] - mu[0]), e2 = exp2f(s[j][2] - mu[1]), e3 = exp2f(s[j][3] - mu[1]);
        l[0] += e0 + e1;
        l[1] += e2 + e3;
        p[j >> 1][(j & 1) * 2] = mt::pack_bf16(e0, e1);
        p[j >> 1][(j & 1) * 2 + 1] = mt::pack_bf16(e2, e3);
      }
#pragma unroll
      for (int ks = 0; ks < kKS; ks++)
#pragma unroll
        for (int dp = 0; dp < HD / 16; dp++) {
          uint32_t b[4];
          mt::load_v_frag<HD, kTile>(v_s, wkey + 16 * ks, dp, lane, b);
          mt::mma_16816(o[2 * dp], p[ks], b[0], b[1]);
          mt::mma_16816(o[2 * dp + 1], p[ks], b[2], b[3]);
        }
      __syncwarp();
      if (lane == 0) sm100::mbar_arrive(&empty[stage]);   // this warp has read what it needs of the stage
    }
#pragma unroll
    for (int r = 0; r < 2; r++) {
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
    // merge the four warps; only the rows that are heads of the group are kept
    if (tq == 0) {
      ml_s[(warp * 16 + g) * 2] = m[0];
      ml_s[(warp * 16 + g) * 2 + 1] = l[0];
      ml_s[(warp * 16 + g + 8) * 2] = m[1];
      ml_s[(warp * 16 + g + 8) * 2 + 1] = l[1];
    }
    // (the O buffer holds merge_cols of the head's values at a time, so that large groups do not cost the second CTA of the SM)
    for (int c0 = 0; c0 < HD; c0 += merge_cols) {
    if (c0) bar_sync_compute();   // every warp is done reading the pass before
#pragma unroll
    for (int i = 0; i < HD / 8; i++) {
      const int d = 8 * i + 2 * tq - c0;
      if (d < 0 || d >= merge_cols) continue;
      if (g < group) *(float2*)&o_s[(warp * group + g) * merge_cols + d] = make_float2(o[i][0], o[i][1]);
      if (g + 8 < group) *(float2*)&o_s[(warp * group + g + 8) * merge_cols + d] = make_float2(o[i][2], o[i][3]);
    }
    bar_sync_compute();
    for (int idx = tid; idx < group * merge_cols; idx += kWarps * 32) {
      const int row = idx / merge_cols, dl = idx % merge_cols, d = c0 + dl;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < kWarps; w++) M = fmaxf(M, ml_s[(w * 16 + row) * 2]);
      if (FUSED && own_here) M = fmaxf(M, s_own[row]);
      float Lsum = 0.f, O = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; w++) {
        const float mw = ml_s[(w * 16 + row) * 2];
        const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
        Lsum += ml_s[(w * 16 + row) * 2 + 1] * f;
        O += o_s[(w * group + row) * merge_cols + dl] * f;
      }
      if (FUSED && own_here) {   // the token's own key and value, as one more partial result
        const float f = exp2f(s_own[row] - M);
        Lsum += f;
        O += v_own[d] * f;
      }
      const size_t slot = ((size_t)item * heads + (size_t)kvh * group + row) * max_slices + slice;
      part_o[slot * HD + d] = O;
      if (d == 0) {
        part_ml[slot * 2] = M;
        part_ml[slot * 2 + 1] = Lsum;
      }
    }
    }
    u = u_next;
  }
}

// Values of a head that the merge buffer of the streaming kernel holds at a time: all of them while
// four warps' rows of the group fit 8 KiB (groups up to 4 at head size 128), else a half, a quarter, ...
inline int stream_merge_cols(int group, int hd) {
  int w = hd;
  while (w > 8 && kWarps * group * w * 4 > 8192) w >>= 1;
  return w;
}

template <int HD, bool FUSED>
int launch_stream(const void* q, const RawQkv* raw, const IbKvView* kv, const int* dec_tokens, int n_dec, const int* positions, const int* seg_of_token,
                  int window, float scale, float* part_o, float* part_ml, void* out, int heads, int max_slices, int tiles_per_slice,
                  const CUtensorMap* kv_map, long long view_row0, unsigned* status, cudaStream_t stream) {
  const int group = heads / kv->kv_heads;
  const int merge_cols = stream_merge_cols(group, HD);
  const int smem = kRing * 2 * kTile * HD * 2 + 16 * HD * 2 + kWarps * 16 * 2 * 4 + kWarps * group * merge_cols * 4 + 2 * kRing * 8 + 16 + kMeta * 12 +
                   (2 * HD + 16) * 4;
  static int reserved = 0, per_sm = 0, sms = 0;
  if (smem != reserved) {
    cudaError_t e = cudaFuncSetAttribute(decode_stream_kernel<HD, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    IB_CHECK_ARG(e == cudaSuccess, "attention_decode_stream: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_stream_kernel<HD, FUSED>, (kWarps + 1) * 32, smem);
    IB_CHECK_ARG(e == cudaSuccess && per_sm >= 1, "attention_decode_stream: no CTA fits an SM with %d bytes of shared memory", smem);
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    reserved = smem;
  }
  const long long units = (long long)max_slices * n_dec * kv->kv_heads;
  IB_CHECK_ARG(units < (1ll << 31), "attention_decode_stream: %lld units", units);
  const int grid = (int)(units < (long long)sms * per_sm ? units : (long long)sms * per_sm);
  const RawQkv none = {};
  ib::launch(decode_stream_kernel<HD, FUSED>, grid, (kWarps + 1) * 32, smem, stream, (const __nv_bfloat16*)q, raw ? *raw : none, *kv, dec_tokens,
             positions, seg_of_token, window, scale * 1.4426950408889634f, part_o, part_ml, heads, n_dec, max_slices, tiles_per_slice, merge_cols,
             *kv_map, view_row0, ib_wait_limit_ns(), status);
  IB_CHECK_LAUNCH("attention_decode_stream split");
  ib::launch(decode_combine_kernel<HD>, dim3(heads, n_dec), kCombineThreads, 0, stream, part_o, part_ml, dec_tokens, positions, window, (__nv_bfloat16*)out, heads,
             max_slices, tiles_per_slice, status);
  IB_CHECK_LAUNCH("attention_decode_stream combine");
  return 0;
}

template <int HD>
int launch(const void* q, const IbKvView* kv, const int* dec_tokens, int n_dec, const int* positions, const int* seg_of_token, int window,
           float scale, float* part_o, float* part_ml, void* out, int heads, int max_slices, int tiles_per_slice, unsigned* status,
           cudaStream_t stream) {
  constexpr int smem = 16 * HD * 2 + 4 * kTile * HD * 2 + 2 * kTile * 8;   // Q, two stages of K and V, key offsets
  static_assert(kWarps * 16 * HD * 4 <= 4 * kTile * HD * 2, "the merge buffer must fit in the tiles");
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(decode_split_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    IB_CHECK_ARG(e == cudaSuccess, "attention_decode: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  dim3 grid(kv->kv_heads, n_dec, max_slices);
  ib::launch(decode_split_kernel<HD>, grid, kWarps * 32, smem, stream, (const __nv_bfloat16*)q, *kv, dec_tokens, positions, seg_of_token, window,
             scale * 1.4426950408889634f, part_o, part_ml, heads, max_slices, tiles_per_slice, status);
  IB_CHECK_LAUNCH("attention_decode split");
  ib::launch(decode_combine_kernel<HD>, dim3(heads, n_dec), kCombineThreads, 0, stream, part_o, part_ml, dec_tokens, positions, window, (__nv_bfloat16*)out, heads,
             max_slices, tiles_per_slice, status);
  IB_CHECK_LAUNCH("attention_decode combine");
  return 0;
}

}  // namespace

// Attention for decoded tokens (one query position each). dec_tokens[i] is the flat row of the i-th
// decoded token in q/out/positions/seg_of_token. Scratch: part_o float32 [n_dec * heads * max_slices * head_dim],
// part_ml float32 [n_dec * heads * max_slices * 2]. A CTA handles a slice of tiles_per_slice tiles of
// ib_attention_decode_tile() keys; max_slices slices must cover every position in use. Slices are cut at
// multiples of their size, so for a given tiles_per_slice a token's result does not depend on the batch.
// Keys and values are copied with cp.async, so every page size is served.
extern "C" int ib_attention_decode_tile() { return kTile; }

// Describes a whole cache pool [executions, pages, 2, kv_heads, page_size, head_dim] (bfloat16) to TMA
// as a matrix of [all rows, head_dim] read in boxes of [page_size rows, 64 columns] with the 128-byte
// swizzle. `map_out` receives the 128-byte tensor map that the attention entry points take.
// Returns 1 with a message when the geometry cannot be served (the kernels then copy with cp.async).
extern "C" int ib_make_kv_map(void* map_out, const void* pool_base, long long total_rows, int head_dim, int page_size) {
  IB_CHECK_ARG(map_out && pool_base && total_rows > 0, "make_kv_map: null pointer or no rows");
  IB_CHECK_ARG(head_dim % 64 == 0, "make_kv_map: head_dim %d is not a multiple of 64", head_dim);
  IB_CHECK_ARG(page_size % 8 == 0 && (kTile % page_size == 0 || page_size % kTile == 0), "make_kv_map: page size %d is not a multiple of 8 that divides %d or a multiple of it", page_size, kTile);
  IB_CHECK_ARG(total_rows < (1ll << 31), "make_kv_map: %lld rows exceed the 32-bit coordinate range", total_rows);
  tma_host::EncodeTiledFn fn = tma_host::encode_fn();
  IB_CHECK_ARG(fn, "make_kv_map: the driver has no cuTensorMapEncodeTiled");
  cuuint64_t dims[2] = {(cuuint64_t)head_dim, (cuuint64_t)total_rows};
  cuuint64_t strides[1] = {(cuuint64_t)head_dim * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)(page_size < kTile ? page_size : kTile)};   // a page, or the tile's part of a larger one
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn((CUtensorMap*)map_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pool_base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  IB_CHECK_ARG(r == CUDA_SUCCESS, "make_kv_map: cuTensorMapEncodeTiled failed with code %d", (int)r);
  return 0;
}

extern "C" int ib_attention_decode(const void* q, const IbKvView* kv, const int* dec_tokens, int n_dec, const int* positions,
                                   const int* seg_of_token, int window, float scale, float* part_o, float* part_ml, void* out, int heads,
                                   int max_slices, int tiles_per_slice, unsigned* status, cudaStream_t stream) {
  if (n_dec == 0) return 0;
  IB_CHECK_ARG(kv && kv->base && kv->block_table, "attention_decode: the cache view has a null pointer");
  IB_CHECK_ARG(tiles_per_slice >= 1 && tiles_per_slice <= 1024, "attention_decode: %d tiles per slice", tiles_per_slice);
  IB_CHECK_ARG(kv->dtype == IB_BF16, "attention_decode: the cache must be bfloat16");
  IB_CHECK_ARG(kv->kv_heads > 0 && heads % kv->kv_heads == 0 && heads / kv->kv_heads <= 16,
               "attention_decode: %d query heads on %d kv heads (groups of up to 16 are supported)", heads, kv->kv_heads);
  IB_CHECK_ARG(n_dec > 0 && n_dec <= 65535 && max_slices > 0 && max_slices <= 65535, "attention_decode: bad sizes n=%d slices=%d", n_dec, max_slices);
  if (kv->head_dim == 128)
    return launch<128>(q, kv, dec_tokens, n_dec, positions, seg_of_token, window, scale, part_o, part_ml, out, heads, max_slices, tiles_per_slice,
                       status, stream);
  if (kv->head_dim == 64)
    return launch<64>(q, kv, dec_tokens, n_dec, positions, seg_of_token, window, scale, part_o, part_ml, out, heads, max_slices, tiles_per_slice,
                      status, stream);
  return ib_set_error("attention_decode: head_dim %d has no tensor-core kernel (64 and 128 have)", kv->head_dim);
}

namespace {
int stream_entry(const void* q, const RawQkv* raw, const IbKvView* kv, const int* dec_tokens, int n_dec, const int* positions, const int* seg_of_token,
                 int window, float scale, float* part_o, float* part_ml, void* out, int heads, int max_slices, int tiles_per_slice,
                 const void* kv_map, long long view_row0, unsigned* status, cudaStream_t stream) {
  if (n_dec == 0) return 0;
  IB_CHECK_ARG(kv && kv->base && kv->block_table && kv_map, "attention_decode_stream: the cache view or the tensor map is a null pointer");
  IB_CHECK_ARG(kv->page_size % 8 == 0 && (kTile % kv->page_size == 0 || kv->page_size % kTile == 0),
               "attention_decode_stream: page size %d is not a multiple of 8 that divides %d or a multiple of %d", kv->page_size, kTile, kTile);
  IB_CHECK_ARG(tiles_per_slice >= 0 && tiles_per_slice <= 1024, "attention_decode_stream: %d tiles per slice", tiles_per_slice);
  IB_CHECK_ARG(kv->dtype == IB_BF16, "attention_decode_stream: the cache must be bfloat16");
  IB_CHECK_ARG(kv->kv_heads > 0 && heads % kv->kv_heads == 0 && heads / kv->kv_heads <= 16,
               "attention_decode_stream: %d query heads on %d kv heads (groups of up to 16 are supported)", heads, kv->kv_heads);
  IB_CHECK_ARG(n_dec > 0 && n_dec <= 65535 && max_slices > 0 && max_slices <= 65535, "attention_decode_stream: bad sizes n=%d slices=%d", n_dec, max_slices);
  IB_CHECK_ARG(kv->page_stride % kv->head_dim == 0 && kv->v_offset % kv->head_dim == 0, "attention_decode_stream: strides are not whole rows");
  const CUtensorMap* map = (const CUtensorMap*)kv_map;
  if (kv->head_dim == 128) {
    if (raw) return launch_stream<128, true>(q, raw, kv, dec_tokens, n_dec, positions, seg_of_token, window, scale, part_o, part_ml, out, heads, max_slices,
                                             tiles_per_slice, map, view_row0, status, stream);
    return launch_stream<128, false>(q, raw, kv, dec_tokens, n_dec, positions, seg_of_token, window, scale, part_o, part_ml, out, heads, max_slices,
                                     tiles_per_slice, map, view_row0, status, stream);
  }
  if (kv->head_dim == 64) {
    if (raw) return launch_stream<64, true>(q, raw, kv, dec_tokens, n_dec, positions, seg_of_token, window, scale, part_o, part_ml, out, heads, max_slices,
                                            tiles_per_slice, map, view_row0, status, stream);
    return launch_stream<64, false>(q, raw, kv, dec_tokens, n_dec, positions, seg_of_token, window, scale, part_o, part_ml, out, heads, max_slices,
                                    tiles_per_slice, map, view_row0, status, stream);
  }
  return ib_set_error("attention_decode_stream: head_dim %d has no tensor-core kernel (64 and 128 have)", kv->head_dim);
}
}  // namespace

// The streaming variant: the same arguments and scratch; kv_map is required, and the page size must be a
// multiple of 8 that divides the tile or a multiple of the tile. tiles_per_slice = 0 cuts every token's
// visible keys into max_slices equal slices (of two tiles at least) instead of slices at fixed positions.
extern "C" int ib_attention_decode_stream(const void* q, const IbKvView* kv, const int* dec_tokens, int n_dec, const int* positions,
                                          const int* seg_of_token, int window, float scale, float* part_o, float* part_ml, void* out,
                                          int heads, int max_slices, int tiles_per_slice, const void* kv_map, long long view_row0,
                                          unsigned* status, cudaStream_t stream) {
  IB_CHECK_ARG(q || n_dec == 0, "attention_decode_stream: q is a null pointer");
  return stream_entry(q, nullptr, kv, dec_tokens, n_dec, positions, seg_of_token, window, scale, part_o, part_ml, out, heads, max_slices,
                      tiles_per_slice, kv_map, view_row0, status, stream);
}

// The same from the output of the q/k/v projection (float32 partial sums qkv [P][T][(heads + 2 kv_heads) * head_dim],
// stride_p elements apart), for steps of decoded tokens only: sums the partial products, applies the per-head
// norms (q_norm_w, k_norm_w: float32 [head_dim] or null) and the rotation (cos_t, sin_t: float32 [T][head_dim / 2]
// or null) to queries and keys, stores every token's key and value at its position in the cache (write_kv) and
// attends. It stands for ib_qk_norm_rope_kv followed by ib_attention_decode_stream.
extern "C" int ib_attention_decode_fused(const float* qkv, int P, long long stride_p, const float* q_norm_w, const float* k_norm_w, float eps,
                                         const float* cos_t, const float* sin_t, int write_kv, const IbKvView* kv, const int* dec_tokens,
                                         int n_dec, const int* positions, const int* seg_of_token, int window, float scale, float* part_o,
                                         float* part_ml, void* out, int heads, int max_slices, int tiles_per_slice, const void* kv_map,
                                         long long view_row0, unsigned* status, cudaStream_t stream) {
  if (n_dec == 0) return 0;
  IB_CHECK_ARG(qkv && P >= 1 && stride_p > 0, "attention_decode_fused: no projection output (P=%d)", P);
  IB_CHECK_ARG(((uintptr_t)qkv % 16) == 0 && stride_p % 4 == 0, "attention_decode_fused: the projection output must be 16-byte aligned");
  IB_CHECK_ARG((cos_t == nullptr) == (sin_t == nullptr), "attention_decode_fused: cos and sin tables come together");
  const RawQkv raw = {qkv, P, stride_p, q_norm_w, k_norm_w, eps, cos_t, sin_t, write_kv};
  return stream_entry(nullptr, &raw, kv, dec_tokens, n_dec, positions, seg_of_token, window, scale, part_o, part_ml, out, heads, max_slices,
                      tiles_per_slice, kv_map, view_row0, status, stream);
}

// ---------------------------------------------------------------- the variant that allocates nothing
#include <mutex>

#include "attention_decode_noalloc.h"

// Scratch of the no-allocation entry point: [part_o | part_ml] of one call. In host code this name
// is only a handle for cudaGetSymbolAddress, never a pointer a kernel may be given.
static __device__ __align__(256) float g_decode_noalloc_scratch[IB_DECODE_NOALLOC_MAX_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {nullptr};
std::mutex g_noalloc_mutex;

// Device address of the scratch array on the current device, looked up once per device.
int noalloc_scratch(float** ptr) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  IB_CHECK_ARG(e == cudaSuccess, "attention_decode_noalloc: cudaGetDevice failed: %s", cudaGetErrorString(e));
  IB_CHECK_ARG(dev >= 0 && dev < kMaxDevices, "attention_decode_noalloc: device %d is beyond the %d this library tracks", dev, kMaxDevices);
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (!g_noalloc_ptr[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_decode_noalloc_scratch);
    IB_CHECK_ARG(e == cudaSuccess && p, "attention_decode_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
    g_noalloc_ptr[dev] = p;
  }
  *ptr = g_noalloc_ptr[dev];
  return 0;
}
}  // namespace

extern "C" int ib_attention_decode_noalloc(const void* q, const IbKvView* kv, const int* dec_tokens, int n_dec, const int* positions,
                                           const int* seg_of_token, int window, float scale, void* out, int heads, int max_slices,
                                           int tiles_per_slice, unsigned* status, cudaStream_t stream) {
  if (n_dec == 0) return 0;
  IB_CHECK_ARG(kv, "attention_decode_noalloc: the cache view is null");
  IB_CHECK_ARG(n_dec > 0 && heads > 0 && max_slices > 0 && kv->head_dim > 0, "attention_decode_noalloc: bad sizes n=%d heads=%d slices=%d", n_dec,
               heads, max_slices);
  const unsigned long long slots = (unsigned long long)n_dec * heads * max_slices;
  const unsigned long long need = slots * (unsigned long long)(kv->head_dim + 2);
  IB_CHECK_ARG(need <= IB_DECODE_NOALLOC_MAX_FLOATS,
               "attention_decode_noalloc: %d tokens x %d heads x %d slices x (head_dim %d + 2) = %llu float32 values, more than the fixed scratch of %u; "
               "use ib_attention_decode with scratch of your own",
               n_dec, heads, max_slices, kv->head_dim, need, IB_DECODE_NOALLOC_MAX_FLOATS);
  float* scratch = nullptr;
  if (noalloc_scratch(&scratch)) return 1;
  float* part_o = scratch;
  float* part_ml = scratch + slots * kv->head_dim;
  return ib_attention_decode(q, kv, dec_tokens, n_dec, positions, seg_of_token, window, scale, part_o, part_ml, out, heads, max_slices, tiles_per_slice,
                             status, stream);
}
