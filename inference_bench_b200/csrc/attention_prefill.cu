// Causal attention for prompt portions over the paged cache, bfloat16, flash style.
//
// One CTA = 64 consecutive query rows of one segment and one query head; warp w owns rows 16w..16w+15.
// Keys are walked in tiles of 64 through the block table (cp.async into swizzled shared memory,
// double buffered); S = Q K^T and O += P V run on m16n8k16 bfloat16 MMAs with float32 accumulators,
// the softmax keeps a running max and sum in float32 base 2. A row at position p sees keys
// lo..p, lo = max(0, p - window + 1) with a window, else 0; the keys of earlier portions are already
// in the cache, and this portion's own keys were written there before this kernel runs.
// Reference design: crates/kir/src/cuda/attention/flash_mma.rs (128-query tiles, f16 hi/lo MMAs).
#include "kv_view.cuh"
#include "mma_tiles.cuh"

namespace {

constexpr int BM = 64, BN = 64, kWarps = 4;

template <int HD>
__device__ __forceinline__ void load_kv_tile(uint32_t k_s, uint32_t v_s, const IbKvView& kv, const __nv_bfloat16* base, int seg, int kvh,
                                             int key0, int key_lo, int key_hi, int tid, unsigned* status) {
  constexpr int CPR = HD / 8;
  for (int idx = tid; idx < BN * CPR; idx += kWarps * 32) {
    int row = idx / CPR, c = idx % CPR;
    int key = key0 + row;
    long long off = (key >= key_lo && key <= key_hi) ? ib::kv_offset(kv, seg, key, kvh) : -2;
    uint32_t kd = k_s + mt::tile_offset<HD, BN>(row, c), vd = v_s + mt::tile_offset<HD, BN>(row, c);
    if (off >= 0) {
      mt::cp_async16(kd, base + off + c * 8);
      mt::cp_async16(vd, base + off + kv.v_offset + c * 8);
    } else {
      if (off == -1) atomicOr(status, IB_ERR_BAD_PAGE);
      mt::st_shared_zero16(kd);
      mt::st_shared_zero16(vd);
    }
  }
}

template <int HD>
__global__ void __launch_bounds__(kWarps * 32)
    prefill_kernel(const __nv_bfloat16* __restrict__ q, IbKvView kv, const int* __restrict__ tile_seg, const int* __restrict__ tile_row0,
                   const int* __restrict__ seg_start, const int* __restrict__ seg_pos0, int window, float scale_log2e,
                   __nv_bfloat16* __restrict__ out, int heads, unsigned* __restrict__ status) {
  constexpr int CPR = HD / 8;
  constexpr int TILE = BN * HD * 2;
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t q_s = mt::smem_u32(smem);                // [64][HD]
  const uint32_t kv_s = q_s + BM * HD * 2;                // 2 stages x (K tile, V tile)

  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int tile = blockIdx.x, h = blockIdx.y;
  const int seg = tile_seg[tile], row0 = tile_row0[tile];
  const int n = seg_start[seg + 1] - seg_start[seg];
  const int rows = min(BM, n - row0);
  const int t0 = seg_start[seg] + row0;
  const int pos_first = seg_pos0[seg] + row0, pos_last = pos_first + rows - 1;
  const int kvh = h / (heads / kv.kv_heads);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, tq = lane & 3;
  const __nv_bfloat16* base = (const __nv_bfloat16*)kv.base;

  const int key_lo = window > 0 ? max(0, pos_first - window + 1) : 0;
  const int kt_begin = key_lo / BN, kt_end = pos_last / BN + 1;

  for (int idx = tid; idx < BM * CPR; idx += kWarps * 32) {
    int row = idx / CPR, c = idx % CPR;
    uint32_t dst = q_s + mt::tile_offset<HD, BM>(row, c);
    if (row < rows)
      mt::cp_async16(dst, q + ((size_t)(t0 + row) * heads + h) * HD + c * 8);
    else
      mt::st_shared_zero16(dst);
  }
  load_kv_tile<HD>(kv_s, kv_s + TILE, kv, base, seg, kvh, kt_begin * BN, key_lo, pos_last, tid, status);
  mt::cp_async_commit();

  uint32_t qa[HD / 16][4];
  float o[HD / 8][4];
#pragma unroll
  for (int nn = 0; nn < HD / 8; nn++)
#pragma unroll
    for (int e = 0; e < 4; e++) o[nn][e] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  const int my_pos[2] = {pos_first + warp * 16 + g, pos_first + warp * 16 + g + 8};

  for (int kt = kt_begin; kt < kt_end; kt++) {
    const int stage = (kt - kt_begin) & 1;
    const uint32_t k_s = kv_s + stage * 2 * TILE, v_s = k_s + TILE;
    if (kt + 1 < kt_end) {
      const uint32_t nk = kv_s + (stage ^ 1) * 2 * TILE;
      load_kv_tile<HD>(nk, nk + TILE, kv, base, seg, kvh, (kt + 1) * BN, key_lo, pos_last, tid, status);
      mt::cp_async_commit();
      mt::cp_async_wait<1>();
    } else {
      mt::cp_async_wait<0>();
    }
    __syncthreads();
    if (kt == kt_begin) {
#pragma unroll
      for (int kk = 0; kk < HD / 16; kk++) mt::load_a_frag<HD, BM>(q_s, warp * 16, kk, lane, qa[kk]);
    }
    const int key0 = kt * BN;
    // skip tiles wholly outside this warp's rows' sight (after their last position or before their window)
    const int w_first = pos_first + warp * 16, w_last = w_first + 15;
    const bool visible = key0 <= w_last && (window <= 0 || key0 + BN - 1 > w_first - window);
    if (visible) {
      float s[BN / 8][4];
#pragma unroll
      for (int j = 0; j < BN / 8; j++)
#pragma unroll
        for (int e = 0; e < 4; e++) s[j][e] = 0.f;
#pragma unroll
      for (int kk = 0; kk < HD / 16; kk++) {
#pragma unroll
        for (int pr = 0; pr < BN / 16; pr++) {
          uint32_t b[4];
          mt::load_k_frag<HD, BN>(k_s, 16 * pr, kk, lane, b);
          mt::mma_16816(s[2 * pr], qa[kk], b[0], b[1]);
          mt::mma_16816(s[2 * pr + 1], qa[kk], b[2], b[3]);
        }
      }
      float mt_[2] = {m[0], m[1]};
#pragma unroll
      for (int j = 0; j < BN / 8; j++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
          const int key = key0 + 8 * j + 2 * tq + (e & 1);
          const int p = my_pos[e >> 1];
          const bool live = key <= p && (window <= 0 || key > p - window);
          const float v = live ? s[j][e] * scale_log2e : -INFINITY;
          s[j][e] = v;
          mt_[e >> 1] = fmaxf(mt_[e >> 1], v);
        }
      float corr[2], mu[2];
#pragma unroll
      for (int r = 0; r < 2; r++) {
        mt_[r] = fmaxf(mt_[r], __shfl_xor_sync(0xffffffffu, mt_[r], 1));
        mt_[r] = fmaxf(mt_[r], __shfl_xor_sync(0xffffffffu, mt_[r], 2));
        mu[r] = mt_[r] == -INFINITY ? 0.f : mt_[r];
        corr[r] = exp2f(m[r] - mu[r]);   // m = -inf at the start gives 0
        m[r] = mt_[r];
        l[r] *= corr[r];
      }
#pragma unroll
      for (int nn = 0; nn < HD / 8; nn++) {
        o[nn][0] *= corr[0];
        o[nn][1] *= corr[0];
        o[nn][2] *= corr[1];
        o[nn][3] *= corr[1];
      }
      uint32_t p[BN / 16][4];
#pragma unroll
      for (int j = 0; j < BN / 8; j++) {
        float e0 = exp2f(s[j][0] - mu[0]), e1 = exp2f(s[j][1] - mu[0]), e2 = exp2f(s[j][2] - mu[1]), e3 = exp2f(s[j][3] - mu[1]);
        l[0] += e0 + e1;
        l[1] += e2 + e3;
        p[j >> 1][(j & 1) * 2] = mt::pack_bf16(e0, e1);
        p[j >> 1][(j & 1) * 2 + 1] = mt::pack_bf16(e2, e3);
      }
#pragma unroll
      for (int ks = 0; ks < BN / 16; ks++)
#pragma unroll
        for (int dp = 0; dp < HD / 16; dp++) {
          uint32_t b[4];
          mt::load_v_frag<HD, BN>(v_s, 16 * ks, dp, lane, b);
          mt::mma_16816(o[2 * dp], p[ks], b[0], b[1]);
          mt::mma_16816(o[2 * dp + 1], p[ks], b[2], b[3]);
        }
    }
    __syncthreads();  // every warp is done with this stage before the next load overwrites it
  }
#pragma unroll
  for (int r = 0; r < 2; r++) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
  const float inv[2] = {l[0] > 0.f ? 1.f / l[0] : 0.f, l[1] > 0.f ? 1.f / l[1] : 0.f};
#pragma unroll
  for (int r = 0; r < 2; r++) {
    const int row = warp * 16 + g + 8 * r;
    if (row >= rows) continue;
    __nv_bfloat16* dst = out + ((size_t)(t0 + row) * heads + h) * HD;
#pragma unroll
    for (int nn = 0; nn < HD / 8; nn++)
      *(uint32_t*)(dst + 8 * nn + 2 * tq) = mt::pack_bf16(o[nn][2 * r] * inv[r], o[nn][2 * r + 1] * inv[r]);
  }
}

template <int HD>
int launch(const void* q, const IbKvView* kv, const int* tile_seg, const int* tile_row0, int n_tiles, const int* seg_start, const int* seg_pos0,
           int window, float scale, void* out, int heads, unsigned* status, cudaStream_t stream) {
  constexpr int smem = BM * HD * 2 + 4 * BN * HD * 2;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    IB_CHECK_ARG(e == cudaSuccess, "attention_prefill: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  ib::launch(prefill_kernel<HD>, dim3(n_tiles, heads), kWarps * 32, smem, stream, (const __nv_bfloat16*)q, *kv, tile_seg, tile_row0, seg_start, seg_pos0,
                                                                         window, scale * 1.4426950408889634f, (__nv_bfloat16*)out, heads, status);
  IB_CHECK_LAUNCH("attention_prefill");
  return 0;
}

}  // namespace

// Attention for query tiles of 64 rows: tile i covers rows tile_row0[i].. of segment tile_seg[i].
extern "C" int ib_attention_prefill(const void* q, const IbKvView* kv, const int* tile_seg, const int* tile_row0, int n_tiles,
                                    const int* seg_start, const int* seg_pos0, int window, float scale, void* out, int heads, unsigned* status,
                                    cudaStream_t stream) {
  if (n_tiles == 0) return 0;
  IB_CHECK_ARG(kv && kv->base && kv->block_table, "attention_prefill: the cache view has a null pointer");
  IB_CHECK_ARG(kv->dtype == IB_BF16, "attention_prefill: the cache must be bfloat16");
  IB_CHECK_ARG(kv->kv_heads > 0 && heads % kv->kv_heads == 0, "attention_prefill: %d query heads are not a multiple of %d kv heads", heads,
               kv->kv_heads);
  IB_CHECK_ARG(n_tiles > 0 && heads <= 65535, "attention_prefill: bad sizes tiles=%d heads=%d", n_tiles, heads);
  if (kv->head_dim == 128) return launch<128>(q, kv, tile_seg, tile_row0, n_tiles, seg_start, seg_pos0, window, scale, out, heads, status, stream);
  if (kv->head_dim == 64) return launch<64>(q, kv, tile_seg, tile_row0, n_tiles, seg_start, seg_pos0, window, scale, out, heads, status, stream);
  return ib_set_error("attention_prefill: head_dim %d has no tensor-core kernel (64 and 128 have)", kv->head_dim);
}
