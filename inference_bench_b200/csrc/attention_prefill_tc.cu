// Causal attention for prompt portions on the sm_100a tensor cores (tcgen05), bfloat16.
//
// One CTA = 128 consecutive query rows of one segment and one query head. Row i is lane i of tensor
// memory; two threads share a row (warps w and w + 4 may both read lanes 32 (w % 4) .. + 31), each
// taking half of the columns, so a row's maximum costs one exchange through shared memory and no
// shuffles. Keys are walked in tiles of 64 through the block table:
//   S = Q K^T   tcgen05.mma, A = Q tile, B = K tile, both K-major in shared memory, S in TMEM (2 buffers)
//   softmax     each thread reads its row of S from TMEM, keeps a running max and sum in float32
//               (base 2), writes P as bfloat16 into a K-major shared tile
//   O += P V    tcgen05.mma, A = P tile, B = V tile read as an N-contiguous operand, O stays in TMEM
// O is rescaled in TMEM only when a row's maximum grows by more than 2^8 (the values of P stay
// within bfloat16 and float32 range meanwhile, and the final division uses the same reference
// maximum), so most tiles cost no pass over O. K and V tiles are fetched with cp.async one to
// two tiles ahead. Two CTAs share an SM: while one does its softmax the other's MMAs run.
// Reference design: crates/kir/src/cuda/attention/flash_mma.rs (mma.sync, f16 hi/lo operands).
#include "kv_view.cuh"
#include "mma_tiles.cuh"
#include "sm100.cuh"

namespace {

constexpr int BM = 128, BN = 64, kThreads = 256;
constexpr float kRescaleThreshold = 8.f;  // log2 units

// Shared tiles are [rows][64 elements] blocks of 128-byte rows (one block per 64 head dims), 16-byte
// chunk c of row r stored at chunk c ^ (r & 7): the layout TMA's 128-byte swizzle would produce and
// the tcgen05 descriptors expect.
__device__ __forceinline__ uint32_t blk_offset(int rows, int r, int cc) {  // cc: 16-byte chunk index along the row of HD elements
  return (uint32_t)((cc >> 3) * rows * 128 + r * 128 + (((cc & 7) ^ (r & 7)) << 4));
}

// 2^x, hardware approximation (relative error about 2^-22); 2^-inf = 0
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 2^x on the FMA and integer pipes, for x <= 8 or so: x = n + f with |f| <= 1/2, a degree-5 polynomial
// for 2^f (relative error below 3e-6) and n added into the exponent. The special-function unit is the
// busiest pipe of this kernel, so half of the exponentials are computed this way.
__device__ __forceinline__ float ex2_poly(float x) {
  x = fmaxf(x, -125.f);
  const float t = x + 12582912.f;          // 1.5 * 2^23: the integer nearest to x sits in the low mantissa bits
  const float f = x - (t - 12582912.f);
  float p = fmaf(f, 1.3333558e-3f, 9.6181291e-3f);
  p = fmaf(p, f, 5.5504109e-2f);
  p = fmaf(p, f, 2.4022651e-1f);
  p = fmaf(p, f, 6.9314718e-1f);
  p = fmaf(p, f, 1.f);
  return __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
}
// two float32 -> packed bfloat16 with integer rounding (half up), no conversion instructions
__device__ __forceinline__ uint32_t pack_bf16_int(float lo, float hi) {
  return __byte_perm(__float_as_uint(lo) + 0x8000u, __float_as_uint(hi) + 0x8000u, 0x7632);
}

template <int HD>
struct Smem {
  static constexpr int kQ = BM * HD * 2, kKV = BN * HD * 2, kP = BM * BN * 2;
  static constexpr int oQ = 0, oK = kQ, oV = kQ + 2 * kKV, oP = kQ + 4 * kKV, oBar = oP + kP, oOffs = oBar + 32;
  // barriers and the tmem slot, then where the keys of two tiles live in the cache (int32, in rows of
  // head_dim elements; -1 = no such key, -2 = its page is missing). Two CTAs of this size fit one SM
  // (113 KiB each beside the 1 KiB the system keeps per CTA), which is why nothing else may be added:
  // the two threads of a row exchange their maxima through the row's own 128 bytes of the P tile.
  static constexpr int kBytes = oOffs + 2 * BN * 4;
  static_assert(kBytes <= 113 * 1024, "two CTAs must fit one SM");
};

template <int HD>
__global__ void __launch_bounds__(kThreads, 2)
    prefill_tc_kernel(const __nv_bfloat16* __restrict__ q, IbKvView kv, const int* __restrict__ tile_seg, const int* __restrict__ tile_row0,
                      const int* __restrict__ seg_start, const int* __restrict__ seg_pos0, int window, float scale_log2e,
                      __nv_bfloat16* __restrict__ out, int heads, int n_tiles, unsigned long long wait_ns, unsigned* __restrict__ status) {
  using SM = Smem<HD>;
  constexpr int CPR = HD / 8;               // 16-byte chunks per row of a Q/K/V tile
  constexpr int kTmemCols = 256;            // S0 [0,64) | S1 [64,128) | O [128, 128+HD)
  extern __shared__ __align__(1024) uint8_t sm[];
  if (sm100::smem_u32(sm) & 1023u) {  // the swizzled tiles need 1024-byte alignment; never seen, but never assumed
    if (threadIdx.x == 0) atomicOr(status, IB_ERR_INTERNAL);
    return;
  }
  const uint32_t q_s = sm100::smem_u32(sm + SM::oQ), k_s = sm100::smem_u32(sm + SM::oK), v_s = sm100::smem_u32(sm + SM::oV),
                 p_s = sm100::smem_u32(sm + SM::oP);
  uint64_t* bar_s = (uint64_t*)(sm + SM::oBar);  // [2]
  uint64_t* bar_o = bar_s + 2;
  uint32_t* tmem_slot = (uint32_t*)(bar_o + 1);
  int* offs = (int*)(sm + SM::oOffs);  // [2][BN], by tile parity

  const int tid = threadIdx.x, warp = tid >> 5;
  const int half = warp >> 2;                       // which half of the columns this thread takes
  const int row = (warp & 3) * 32 + (tid & 31);     // its query row = its tensor-memory lane
  auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"((warp & 3) + 1) : "memory"); };  // the two warps that share 32 rows
  ib::pdl_launch_dependents();
  if (tid == 0) {
    sm100::mbar_init(&bar_s[0], 1);
    sm100::mbar_init(&bar_s[1], 1);
    sm100::mbar_init(bar_o, 1);
    sm100::fence_barrier_init();
  }
  if (warp == 0) {
    sm100::tmem_alloc(tmem_slot, kTmemCols);
    sm100::tmem_relinquish();
  }
  sm100::tc_fence_before();
  __syncthreads();
  sm100::tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t t_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16);  // this warp's quarter of the lanes
  ib::pdl_wait();

  // heads vary fastest, and the caller lists the tiles with the most keys first: the longest CTAs start
  // first whatever their head, and the heads that share a kv head run side by side
  const int tile = blockIdx.y, h = blockIdx.x;
  const int seg = tile_seg[tile], row0 = tile_row0[tile];
  const int n = seg_start[seg + 1] - seg_start[seg];
  const int rows = min(BM, n - row0);
  const int t0 = seg_start[seg] + row0;
  const int pos_first = seg_pos0[seg] + row0, pos_last = pos_first + rows - 1;
  const int my_pos = pos_first + row;
  const int kvh = h / (heads / kv.kv_heads);
  const __nv_bfloat16* base = (const __nv_bfloat16*)kv.base;
  const int key_lo = window > 0 ? max(0, pos_first - window + 1) : 0;
  const int kt_begin = key_lo / BN, kt_end = pos_last / BN + 1;
  const int n_kt = kt_end - kt_begin;

  // One thread per key looks up where the key lives (once per tile, kept for the K and the V copy).
  // The lookup reads the block table from memory, so it is started one tile before its result is
  // needed: look_up() returns the row in a register, post() puts it into shared memory a tile later.
  auto look_up = [&](int kt) -> int {
    int o = -1;
    if (tid < BN) {
      const int key = kt * BN + tid;
      if (key >= key_lo && key <= pos_last) {
        const long long off = ib::kv_offset(kv, seg, key, kvh);
        o = off < 0 ? -2 : (int)(off / HD);      // elements -> rows of head_dim elements (offsets are whole rows)
      }
    }
    return o;
  };
  auto post = [&](int kt, int o) {
    if (tid < BN) {
      if (o == -2) atomicOr(status, IB_ERR_BAD_PAGE);
      offs[(kt & 1) * BN + tid] = o;
    }
  };
  // copies one K or V tile (64 keys) into a swizzled buffer; keys outside [key_lo, pos_last] become zero
  const int my_cc = tid % CPR, my_r0 = tid / CPR;
  auto load_kv = [&](uint32_t dst, int kt, long long plane) {
    const int* o = offs + (kt & 1) * BN;
    const __nv_bfloat16* src = base + plane + my_cc * 8;
#pragma unroll
    for (int r = my_r0; r < BN; r += kThreads / CPR) {
      const int off = o[r];
      const uint32_t d = dst + blk_offset(BN, r, my_cc);
      if (off >= 0)
        mt::cp_async16(d, src + (size_t)off * HD);
      else
        mt::st_shared_zero16(d);
    }
  };

  // ---- prologue: Q, K0, V0 (copy group), K1 (copy group); S_0 is issued as soon as Q and K0 are in
  for (int idx = tid; idx < BM * CPR; idx += kThreads) {
    const int r = idx / CPR, cc = idx % CPR;
    const uint32_t d = q_s + blk_offset(BM, r, cc);
    if (r < rows)
      mt::cp_async16(d, q + ((size_t)(t0 + r) * heads + h) * HD + cc * 8);
    else
      mt::st_shared_zero16(d);
  }
  post(kt_begin, look_up(kt_begin));
  if (n_kt > 1) post(kt_begin + 1, look_up(kt_begin + 1));
  int next_rows = n_kt > 2 ? look_up(kt_begin + 2) : -1;   // of tile 2, posted when tile 0 is processed
  __syncthreads();
  load_kv(k_s, kt_begin, 0);
  load_kv(v_s, kt_begin, kv.v_offset);
  mt::cp_async_commit();
  if (n_kt > 1) load_kv(k_s + SM::kKV, kt_begin + 1, 0);
  mt::cp_async_commit();
  mt::cp_async_wait<1>();
  mt::cp_async_commit();   // an empty group in the place of a V fetch, so that the loop's group counts hold from tile 0
  sm100::fence_proxy_async();
  __syncthreads();

  constexpr uint32_t idesc_s = sm100::idesc_bf16_f32(BM, BN);
  constexpr uint32_t idesc_o = sm100::idesc_bf16_f32_b_mn(BM, HD);
  auto issue_s = [&](int j) {  // S_j = Q K_j^T into S buffer j & 1
    const uint32_t kb = k_s + (j & 1) * SM::kKV;
#pragma unroll
    for (int kk = 0; kk < HD / 16; kk++) {
      const uint64_t da = sm100::smem_desc_sw128(q_s + (kk >> 2) * BM * 128) + 2 * (kk & 3);
      const uint64_t db = sm100::smem_desc_sw128(kb + (kk >> 2) * BN * 128) + 2 * (kk & 3);
      sm100::mma_bf16_ss(tmem + (j & 1) * BN, da, db, idesc_s, kk != 0);
    }
    sm100::mma_commit(&bar_s[j & 1]);
  };
  auto issue_o = [&](int j) {  // O += P_j V_j
    const uint32_t vb = v_s + (j & 1) * SM::kKV;
#pragma unroll
    for (int ks = 0; ks < BN / 16; ks++) {
      const uint64_t da = sm100::smem_desc_sw128(p_s) + 2 * ks;
      const uint64_t db = sm100::smem_desc_sw128_mn(vb + ks * 16 * 128, BN * 128);
      sm100::mma_bf16_ss(tmem + 2 * BN, da, db, idesc_o, (j | ks) != 0);
    }
    sm100::mma_commit(bar_o);
  };
  if (tid == 0) issue_s(0);

  // Per tile j:  wait S_j | issue S_{j+1} (runs during this tile's softmax) | fetch K_{j+2} |
  //              read S_j, softmax | wait P V of tile j-1 | fetch V_{j+1} | write P_j | issue P V of tile j
  float m_ref = -INFINITY, l = 0.f;
  bool ok = true;
  for (int j = 0; j < n_kt && ok; j++) {
    const int kt = kt_begin + j;
    ok = sm100::mbar_wait(&bar_s[j & 1], (j >> 1) & 1, wait_ns);   // S_j is done: its K buffer is free
    if (!ok) {
      atomicOr(status, IB_ERR_WAIT_TIMEOUT);
      break;
    }
    sm100::tc_fence_after();
    if (j + 2 < n_kt) post(kt + 2, next_rows);
    if (j + 3 < n_kt) next_rows = look_up(kt + 3);
    mt::cp_async_wait<1>();                                 // K of tile j+1 has landed (all but the newest group, a V)
    sm100::fence_proxy_async();
    sm100::tc_fence_before();
    __syncthreads();
    if (tid == 0 && j + 1 < n_kt) {
      sm100::tc_fence_after();
      issue_s(j + 1);
    }
    if (j + 2 < n_kt) load_kv(k_s + (j & 1) * SM::kKV, kt + 2, 0);
    mt::cp_async_commit();

    // ---- this thread's half of its row of S
    constexpr int HC = BN / 2;
    uint32_t sr[HC];
    sm100::tmem_ld_32x32b_x32(t_lane + (j & 1) * BN + half * HC, sr);
    sm100::tmem_ld_wait();
    const int key0 = kt * BN + half * HC;
    const bool need_mask = kt * BN + BN - 1 > pos_first || kt * BN < key_lo || (window > 0 && kt * BN <= pos_last - window);
    float tile_max = -INFINITY;   // of the raw products; the scale (positive) is applied once below
    if (need_mask) {
#pragma unroll
      for (int c = 0; c < HC; c++) {
        const int key = key0 + c;
        const bool live = key <= my_pos && key >= key_lo && (window <= 0 || key > my_pos - window);
        if (!live) sr[c] = 0xff800000u;  // -inf
      }
    }
#pragma unroll
    for (int c = 0; c < HC; c++) tile_max = fmaxf(tile_max, __uint_as_float(sr[c]));
    // ---- P V of tile j-1 must be finished before O, the P tile or its V buffer are touched
    if (j > 0) {
      ok = sm100::mbar_wait(bar_o, (j - 1) & 1, wait_ns);
      if (!ok) {
        atomicOr(status, IB_ERR_WAIT_TIMEOUT);
        break;
      }
      sm100::tc_fence_after();
    }
    if (j + 1 < n_kt) load_kv(v_s + ((j + 1) & 1) * SM::kKV, kt + 1, kv.v_offset);
    mt::cp_async_commit();
    // ---- the row's maximum: the two halves meet in the row's own bytes of the (now free) P tile
    float* mine = (float*)(sm + SM::oP + row * 128);
    mine[half] = tile_max;
    pair_sync();
    tile_max = fmaxf(tile_max, mine[half ^ 1]) * scale_log2e;
    pair_sync();   // both have read before either writes P over it
    // ---- reference maximum: moved only when a row's maximum grew a lot (or at the first tile).
    // Both threads of a row see the same numbers here, so both warps take the same branch.
    const bool grow = tile_max > m_ref + kRescaleThreshold || (m_ref == -INFINITY && tile_max > -INFINITY);
    if (j == 0) {
      m_ref = tile_max;
    } else if (__any_sync(0xffffffffu, grow)) {
      const float m_new = fmaxf(m_ref, tile_max);
      const float f = m_new == -INFINITY ? 1.f : ex2(m_ref - m_new);  // 0 when m_ref was -inf
      l *= f;
      m_ref = m_new;
#pragma unroll 1
      for (int c0 = half * (HD / 2); c0 < (half + 1) * (HD / 2); c0 += 32) {   // this thread's half of the columns of O
        uint32_t o[32];
        sm100::tmem_ld_32x32b_x32(t_lane + 2 * BN + c0, o);
        sm100::tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; c++) o[c] = __float_as_uint(__uint_as_float(o[c]) * f);
        sm100::tmem_st_32x32b_x32(t_lane + 2 * BN + c0, o);
      }
      sm100::tmem_st_wait();
    }
    const float mu = m_ref == -INFINITY ? 0.f : m_ref;
    // ---- P = 2^(S - m_ref) as bfloat16 into the shared P tile (this thread's half of its row)
#pragma unroll
    for (int c8 = 0; c8 < HC / 8; c8++) {
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const float p0 = ex2(fmaf(__uint_as_float(sr[c8 * 8 + 2 * e]), scale_log2e, -mu));
        const float p1 = ex2_poly(fmaf(__uint_as_float(sr[c8 * 8 + 2 * e + 1]), scale_log2e, -mu));
        l += p0 + p1;
        w[e] = pack_bf16_int(p0, p1);
      }
      asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(p_s + blk_offset(BM, row, half * (HC / 8) + c8)), "r"(w[0]), "r"(w[1]),
                   "r"(w[2]), "r"(w[3])
                   : "memory");
    }
    // ---- V of tile j has landed (all but the two newest copy groups); hand P and V over to the MMA
    mt::cp_async_wait<2>();
    sm100::fence_proxy_async();
    sm100::tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      sm100::tc_fence_after();
      issue_o(j);
    }
  }
  // ---- O / l -> out
  if (ok) {
    ok = sm100::mbar_wait(bar_o, (n_kt - 1) & 1, wait_ns);
    if (!ok) atomicOr(status, IB_ERR_WAIT_TIMEOUT);
  }
  sm100::tc_fence_after();
  {  // the row's sum is the sum of its two halves (the P tile is free again: the last P V has finished)
    float* mine = (float*)(sm + SM::oP + row * 128);
    mine[half] = l;
    pair_sync();
    l += mine[half ^ 1];
  }
  if (__all_sync(0xffffffffu, ok)) {
    const float inv = l > 0.f ? 1.f / l : 0.f;
    __nv_bfloat16* dst = out + ((size_t)(t0 + row) * heads + h) * HD;
#pragma unroll 1
    for (int c0 = half * (HD / 2); c0 < (half + 1) * (HD / 2); c0 += 32) {
      uint32_t o[32];
      sm100::tmem_ld_32x32b_x32(t_lane + 2 * BN + c0, o);
      sm100::tmem_ld_wait();
      if (row < rows) {
#pragma unroll
        for (int c = 0; c < 32; c += 8) {
          uint4 w;
          w.x = mt::pack_bf16(__uint_as_float(o[c]) * inv, __uint_as_float(o[c + 1]) * inv);
          w.y = mt::pack_bf16(__uint_as_float(o[c + 2]) * inv, __uint_as_float(o[c + 3]) * inv);
          w.z = mt::pack_bf16(__uint_as_float(o[c + 4]) * inv, __uint_as_float(o[c + 5]) * inv);
          w.w = mt::pack_bf16(__uint_as_float(o[c + 6]) * inv, __uint_as_float(o[c + 7]) * inv);
          *(uint4*)(dst + c0 + c) = w;
        }
      }
    }
  }
  mt::cp_async_wait<0>();
  sm100::tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    sm100::tmem_dealloc(tmem, kTmemCols);
  }
}

template <int HD>
int launch(const void* q, const IbKvView* kv, const int* tile_seg, const int* tile_row0, int n_tiles, const int* seg_start, const int* seg_pos0,
           int window, float scale, void* out, int heads, unsigned* status, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<HD>::kBytes);
    IB_CHECK_ARG(e == cudaSuccess, "attention_prefill_tc: cannot reserve %d bytes of shared memory: %s", Smem<HD>::kBytes, cudaGetErrorString(e));
    configured = true;
  }
  ib::launch(prefill_tc_kernel<HD>, dim3(heads, n_tiles), kThreads, Smem<HD>::kBytes, stream, (const __nv_bfloat16*)q, *kv, tile_seg, tile_row0,
             seg_start, seg_pos0, window, scale * 1.4426950408889634f, (__nv_bfloat16*)out, heads, n_tiles, ib_wait_limit_ns(), status);
  IB_CHECK_LAUNCH("attention_prefill_tc");
  return 0;
}

}  // namespace

// Attention for query tiles of 128 rows: tile i covers rows tile_row0[i].. of segment tile_seg[i].
// List the tiles that see the most keys first: they are started in that order.
extern "C" int ib_attention_prefill_tc(const void* q, const IbKvView* kv, const int* tile_seg, const int* tile_row0, int n_tiles,
                                       const int* seg_start, const int* seg_pos0, int window, float scale, void* out, int heads,
                                       unsigned* status, cudaStream_t stream) {
  if (n_tiles == 0) return 0;
  IB_CHECK_ARG(kv && kv->base && kv->block_table, "attention_prefill_tc: the cache view has a null pointer");
  IB_CHECK_ARG(kv->dtype == IB_BF16, "attention_prefill_tc: the cache must be bfloat16");
  IB_CHECK_ARG(kv->kv_heads > 0 && heads % kv->kv_heads == 0, "attention_prefill_tc: %d query heads are not a multiple of %d kv heads", heads,
               kv->kv_heads);
  IB_CHECK_ARG(n_tiles > 0 && n_tiles <= 65535, "attention_prefill_tc: %d query tiles (at most 65535 per launch)", n_tiles);
  if (kv->head_dim == 128) return launch<128>(q, kv, tile_seg, tile_row0, n_tiles, seg_start, seg_pos0, window, scale, out, heads, status, stream);
  if (kv->head_dim == 64) return launch<64>(q, kv, tile_seg, tile_row0, n_tiles, seg_start, seg_pos0, window, scale, out, heads, status, stream);
  return ib_set_error("attention_prefill_tc: head_dim %d has no tensor-core kernel (64 and 128 have)", kv->head_dim);
}
