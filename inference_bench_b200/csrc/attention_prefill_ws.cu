// Causal attention for prompt portions on the sm_100a tensor cores, bfloat16, with the work of a CTA
// divided among warps that do one thing each:
//   warps 0-3  softmax: thread i owns query row i = lane i of tensor memory. It reads its row of S
//              (64 keys) from tensor memory, keeps the running maximum and sum (float32, base 2), and
//              writes P = 2^(S - m) as bfloat16 back into tensor memory over the first half of S.
//   warp 4     issues the MMAs: S_j = Q K_j^T (A = Q, B = K, both from shared memory) one tile ahead,
//              O += P_j V_j (A = P from tensor memory, B = V from shared memory), and one commit after each:
//              the first tells the softmax threads that S is there and the K warp that the K buffer is free,
//              the second tells the V warp that the V buffer is free and the softmax threads that O has the tile.
//   warp 5, 6  copy: one the K tiles, one the V tiles, through the block table by TMA box copies (one per page
//              and 64 values of the head dimension, each issued by a lane of its own) into two and three buffers,
//              as soon as one is free. A lane looks up the page of one box in 32; the loop divides nothing.
// Nobody waits at a CTA-wide barrier inside the loop: the roles meet at mbarriers only, so the
// tensor core works on S_{j+1} while the softmax threads are busy with tile j, and the copies run
// ahead of both. O is rescaled (in tensor memory, by the softmax threads) only when a row's maximum
// grows by more than 2^8, so most tiles touch O by MMA alone. Two CTAs share an SM. The warps that issue
// (MMAs, copies) run one instruction stream each, and the loop is as fast as the slowest of them: what
// they do per tile is kept to the instructions themselves (descriptors are a constant apart, buffers and
// parities are counted, a wait that is already over costs one try).
// Needs the tensor map of the cache pool (ib_make_kv_map): page sizes that are a multiple of 8 and
// divide 64, or a multiple of 64. Reference design: crates/kir/src/cuda/attention/flash_mma.rs.
#include <cuda.h>

#include "kv_view.cuh"
#include "mma_tiles.cuh"
#include "sm100.cuh"

namespace {

constexpr int BM = 128, BN = 64;
constexpr int kSoftmaxWarps = 4, kThreads = (kSoftmaxWarps + 3) * 32;
constexpr float kRescaleThreshold = 8.f;  // log2 units
constexpr int KS = 2, VS = 3;             // buffers for K tiles and for V tiles (what two CTAs per SM leave room for)
static_assert(KS == 2 && VS >= 2 && VS <= 4, "K buffer j % KS goes with S buffer j & 1; the parity argument for v_empty needs VS >= 2");
constexpr int kMufu = 4;                  // of every four exponentials, how many the special-function unit computes (0, 2 or 4)

__device__ __forceinline__ uint32_t blk_offset(int rows, int r, int cc) {  // 16-byte chunk cc of row r in [rows][64]-element blocks, 128-byte swizzle
  return (uint32_t)((cc >> 3) * rows * 128 + r * 128 + (((cc & 7) ^ (r & 7)) << 4));
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 2^x for two values on the FMA and integer pipes (relative error below 3e-6), for x <= 8 or so, with the
// two-wide float32 instructions of sm_100: x = n + f with |f| <= 1/2, a degree-5 polynomial for 2^f, n added
// into the exponent. The special-function unit is a bottleneck of this kernel, so part of the exponentials go this way.
__device__ __forceinline__ float2 ex2_poly2(float2 x) {
  x.x = fmaxf(x.x, -125.f);
  x.y = fmaxf(x.y, -125.f);
  const float2 big = make_float2(12582912.f, 12582912.f);   // 1.5 * 2^23: the integer nearest to x sits in the low mantissa bits
  const float2 t = __fadd2_rn(x, big);
  const float2 r = __fadd2_rn(t, make_float2(-12582912.f, -12582912.f));
  const float2 f = __ffma2_rn(r, make_float2(-1.f, -1.f), x);
  float2 p = __ffma2_rn(f, make_float2(1.3333558e-3f, 1.3333558e-3f), make_float2(9.6181291e-3f, 9.6181291e-3f));
  p = __ffma2_rn(p, f, make_float2(5.5504109e-2f, 5.5504109e-2f));
  p = __ffma2_rn(p, f, make_float2(2.4022651e-1f, 2.4022651e-1f));
  p = __ffma2_rn(p, f, make_float2(6.9314718e-1f, 6.9314718e-1f));
  p = __ffma2_rn(p, f, make_float2(1.f, 1.f));
  return make_float2(__int_as_float(__float_as_int(p.x) + (__float_as_int(t.x) << 23)), __int_as_float(__float_as_int(p.y) + (__float_as_int(t.y) << 23)));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {   // round to nearest even, one instruction
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ void bar_sync_softmax() { asm volatile("bar.sync 1, %0;" ::"n"(kSoftmaxWarps * 32) : "memory"); }

template <int HD>
struct Smem {
  static constexpr int kQ = BM * HD * 2, kKV = BN * HD * 2;
  static constexpr int oQ = 0, oK = kQ, oV = kQ + KS * kKV, oBar = kQ + (KS + VS) * kKV;
  // barriers: k_full[KS] v_full[VS] v_empty[VS] s_full[2] p_full[2] q_full; then the tmem slot and the flag
  static constexpr int kBars = KS + 2 * VS + 5;
  static constexpr int kBytes = oBar + kBars * 8 + 16;
  static_assert(kBytes <= 113 * 1024, "two CTAs must fit one SM");
};

template <int HD>
__global__ void __launch_bounds__(kThreads, 2)
    prefill_ws_kernel(const __nv_bfloat16* __restrict__ q, IbKvView kv, const int* __restrict__ tile_seg, const int* __restrict__ tile_row0,
                      const int* __restrict__ seg_start, const int* __restrict__ seg_pos0, int window, float scale_log2e,
                      __nv_bfloat16* __restrict__ out, int heads, const __grid_constant__ CUtensorMap kv_map, long long view_row0,
                      unsigned long long wait_ns, unsigned* __restrict__ status) {
  using SM = Smem<HD>;
  constexpr int CPR = HD / 8, HB = HD / 64;
  constexpr int kTmemCols = 256;            // S0 [0,64) | S1 [64,128) | O [128, 128+HD); P_j lies over the first 32 columns of S_j
  extern __shared__ __align__(1024) uint8_t sm[];
  if (sm100::smem_u32(sm) & 1023u) {
    if (threadIdx.x == 0) atomicOr(status, IB_ERR_INTERNAL);
    return;
  }
  const uint32_t q_s = sm100::smem_u32(sm + SM::oQ), k_s = sm100::smem_u32(sm + SM::oK), v_s = sm100::smem_u32(sm + SM::oV);
  uint64_t* bars = (uint64_t*)(sm + SM::oBar);
  uint64_t *k_full = bars, *v_full = bars + KS, *v_empty = bars + KS + VS, *s_full = bars + KS + 2 * VS, *p_full = s_full + 2, *q_full = s_full + 4;
  uint32_t* tmem_slot = (uint32_t*)(bars + SM::kBars);
  volatile int* gave_up = (volatile int*)(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  ib::pdl_launch_dependents();
  if (tid == 0) {
    for (int i = 0; i < KS; i++) sm100::mbar_init(&k_full[i], 1);
    for (int i = 0; i < VS; i++) {
      sm100::mbar_init(&v_full[i], 1);
      sm100::mbar_init(&v_empty[i], 1);
    }
    for (int i = 0; i < 2; i++) {
      sm100::mbar_init(&s_full[i], 1);
      sm100::mbar_init(&p_full[i], kSoftmaxWarps);
    }
    sm100::mbar_init(q_full, 1);
    *gave_up = 0;
    sm100::fence_barrier_init();
  }
  if (warp == kSoftmaxWarps) {
    sm100::tmem_alloc(tmem_slot, kTmemCols);
    sm100::tmem_relinquish();
  }
  sm100::tc_fence_before();
  __syncthreads();
  sm100::tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  // heads vary fastest, and the caller lists the tiles with the most keys first
  const int tile = blockIdx.y, h = blockIdx.x;
  const int seg = tile_seg[tile], row0 = tile_row0[tile];
  const int n = seg_start[seg + 1] - seg_start[seg];
  const int rows = min(BM, n - row0);
  const int t0 = seg_start[seg] + row0;
  const int pos_first = seg_pos0[seg] + row0, pos_last = pos_first + rows - 1;
  const int kvh = h / (heads / kv.kv_heads);
  const int key_lo = window > 0 ? max(0, pos_first - window + 1) : 0;
  const int kt_begin = key_lo / BN, kt_end = pos_last / BN + 1;
  const int n_kt = kt_end - kt_begin;
  // a wait that ran out: say so once, and from then on nobody waits (the results are void, the status says so)
  auto wait = [&](uint64_t* bar, uint32_t parity) {
    if (sm100::mbar_try_wait(bar, parity) || *gave_up) return;
    if (!sm100::mbar_wait(bar, parity, wait_ns)) {
      *gave_up = 1;
      atomicOr(status, IB_ERR_WAIT_TIMEOUT);
    }
  };

  if (warp > kSoftmaxWarps) {
    // ------------------------------------------------------------ the copying warps: one for the K tiles, one for the V tiles
    // One lane owns one box of every tile: box b_pg of the tile's keys (a page, where a page holds fewer than 64 keys) and
    // the 64-value block b_hb of the head. What does not change from tile to tile is computed once; the row of a box in the
    // pool is computed when its page is looked up (32 boxes at a time, one per lane), so the loop divides nothing.
    ib::pdl_wait();   // the kernel before wrote this portion's keys and values
    const int box_rows = min(kv.page_size, BN);
    const int ppt = BN / box_rows, boxes = ppt * HB;
    const int boxes_per_page = kv.page_size / box_rows;
    const long long rows_per_page = kv.page_stride / HD;
    const int v_rows = (int)(kv.v_offset / HD);
    const int b_pg = lane / HB, b_hb = lane % HB;
    const bool has_box = lane < boxes;
    const uint32_t box_bytes = (uint32_t)box_rows * 128;
    const int plane = warp - kSoftmaxWarps - 1;   // 0: this warp copies K tiles, 1: V tiles
    const int n_buf = plane ? VS : KS;
    uint8_t* const dst0 = sm + (plane ? SM::oV : SM::oK) + b_hb * BN * 128 + b_pg * box_bytes;
    uint64_t* const full0 = plane ? v_full : k_full;
    int held_row = -1;   // the row in the pool where the K rows of the box that this lane looked up begin, or -1: nothing to copy
    int st = 0;
    uint32_t par = 1;   // the parity to wait for before a buffer is filled again: of s_full (K), of v_empty (V)
    for (int j = 0; j < n_kt; j++) {
      const int rel = j * ppt;
      if ((rel & 31) == 0) {   // the pages of the next 32 boxes, one per lane
        const int box = kt_begin * ppt + rel + lane;
        const int key0 = box * box_rows;
        held_row = -1;
        if (key0 <= pos_last && key0 + box_rows > key_lo) {
          const int col = boxes_per_page == 1 ? box : box / boxes_per_page;
          const int page = col < kv.table_stride ? kv.block_table[(size_t)seg * kv.table_stride + col] : -1;
          if (page >= 0 && page < kv.num_pages)
            held_row = (int)((long long)page * rows_per_page + view_row0 + (long long)kvh * kv.page_size + (key0 - col * kv.page_size));
          else
            atomicOr(status, IB_ERR_BAD_PAGE);
        }
      }
      const int row = __shfl_sync(0xffffffffu, held_row, (rel + b_pg) & 31);
      const bool ok = has_box && row >= 0;
      const unsigned vmask = __ballot_sync(0xffffffffu, ok);
      const int n_ok = __popc(vmask);
      const uint32_t bytes = (uint32_t)n_ok * box_bytes;
      // the K buffer of tile j is free when S of tile j - 2 is there (the MMA warp's commit to s_full says both); the V buffer
      // when P V of the tile that used it has finished
      uint64_t* const empty = plane ? &v_empty[st] : j >= KS ? &s_full[st] : nullptr;
      uint8_t* const dst = dst0 + st * SM::kKV;
      if (lane == 0 && empty) wait(empty, par);
      __syncwarp();
      if (n_ok != boxes) {   // boxes that are not copied (no visible key, or no page) are cleared: the tile's edge, seldom
        for (int b = 0; b < boxes; b++) {
          if ((vmask >> b) & 1) continue;
          const uint32_t d0 = sm100::smem_u32(dst) + ((b % HB) - b_hb) * BN * 128 + ((b / HB) - b_pg) * (int)box_bytes;
          for (int idx = lane; idx < box_rows * 8; idx += 32) mt::st_shared_zero16(d0 + idx * 16);
        }
        sm100::fence_proxy_async();
        __syncwarp();
      }
      if (lane == 0) sm100::mbar_arrive_expect_tx(&full0[st], bytes);
      if (ok) sm100::tma_load_2d(dst, &kv_map, b_hb * 64, row + plane * v_rows, &full0[st]);
      if (++st == n_buf) st = 0, par ^= 1;
    }
  } else if (warp == kSoftmaxWarps) {
    // ------------------------------------------------------------ the MMA warp (one lane issues)
    if (lane == 0) {
      constexpr uint32_t idesc_s = sm100::idesc_bf16_f32(BM, BN);
      constexpr uint32_t idesc_o = sm100::idesc_bf16_f32_b_mn(BM, HD);
      // Only the address field of a shared-memory descriptor changes from one MMA to the next (16-byte units), so every
      // operand is the first one's descriptor plus a constant; buffers and parities are counted, not divided.
      const uint64_t dq0 = sm100::smem_desc_sw128(q_s), dk0 = sm100::smem_desc_sw128(k_s), dv0 = sm100::smem_desc_sw128_mn(v_s, BN * 128);
      int ks = 0, vs = 0;
      uint32_t k_par = 0, v_par = 0;
      auto issue_s = [&](int j) {  // S_j = Q K_j^T into S buffer j & 1 (= K buffer ks); its commit also frees the K buffer
        wait(&k_full[ks], k_par);
        sm100::tc_fence_after();
        const uint64_t dk = dk0 + (uint64_t)(ks * (SM::kKV >> 4));
#pragma unroll
        for (int kk = 0; kk < HD / 16; kk++) {
          const uint64_t step = (uint64_t)(2 * (kk & 3));
          sm100::mma_bf16_ss(tmem + ks * BN, dq0 + (uint64_t)(((kk >> 2) * BM * 128) >> 4) + step, dk + (uint64_t)(((kk >> 2) * BN * 128) >> 4) + step,
                             idesc_s, kk != 0);
        }
        sm100::mma_commit(&s_full[ks]);
        if (++ks == KS) ks = 0, k_par ^= 1;
      };
      wait(q_full, 0);
      issue_s(0);
      for (int j = 0; j < n_kt; j++) {
        if (j + 1 < n_kt) issue_s(j + 1);
        wait(&p_full[j & 1], (j >> 1) & 1);
        wait(&v_full[vs], v_par);
        sm100::tc_fence_after();
        const uint64_t dv = dv0 + (uint64_t)(vs * (SM::kKV >> 4));
#pragma unroll
        for (int kstep = 0; kstep < BN / 16; kstep++)   // O += P_j V_j, P from tensor memory: 16 keys = 8 columns per step
          sm100::mma_bf16_ts(tmem + 2 * BN, tmem + (j & 1) * BN + kstep * 8, dv + (uint64_t)((kstep * 16 * 128) >> 4), idesc_o, (j | kstep) != 0);
        sm100::mma_commit(&v_empty[vs]);   // O has tile j, and the V buffer is free
        if (++vs == VS) vs = 0, v_par ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------ the softmax warps: thread = query row
    const int row = tid;
    const uint32_t t_lane = tmem + ((uint32_t)(warp * 32) << 16);
    const int my_pos = pos_first + row;
    ib::pdl_wait();   // q comes from the kernel before
    for (int idx = tid; idx < BM * CPR; idx += kSoftmaxWarps * 32) {
      const int r = idx / CPR, cc = idx % CPR;
      const uint32_t d = q_s + blk_offset(BM, r, cc);
      if (r < rows)
        mt::cp_async16(d, q + ((size_t)(t0 + r) * heads + h) * HD + cc * 8);
      else
        mt::st_shared_zero16(d);
    }
    mt::cp_async_commit();
    mt::cp_async_wait<0>();
    sm100::fence_proxy_async();
    bar_sync_softmax();
    if (tid == 0) sm100::mbar_arrive(q_full);

    float m_ref = -INFINITY, l = 0.f;
    for (int j = 0; j < n_kt; j++) {
      const int kt = kt_begin + j;
      wait(&s_full[j & 1], (j >> 1) & 1);
      sm100::tc_fence_after();
      uint32_t sr[BN];
      sm100::tmem_ld_32x32b_x32(t_lane + (j & 1) * BN, sr);
      sm100::tmem_ld_32x32b_x32(t_lane + (j & 1) * BN + 32, sr + 32);
      sm100::tmem_ld_wait();
      const int key0 = kt * BN;
      const bool need_mask = key0 + BN - 1 > pos_first || key0 < key_lo || (window > 0 && key0 <= pos_last - window);
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < BN; c++) {
          const int key = key0 + c;
          const bool live = key <= my_pos && key >= key_lo && (window <= 0 || key > my_pos - window);
          if (!live) sr[c] = 0xff800000u;  // -inf
        }
      }
      // the maximum of the raw products (the positive scale is applied once below): four chains of three-input maxima
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < BN; c += 8) {
#pragma unroll
        for (int e = 0; e < 4; e++) mx[e] = max3(mx[e], __uint_as_float(sr[c + 2 * e]), __uint_as_float(sr[c + 2 * e + 1]));
      }
      const float tile_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale_log2e;
      // the reference maximum moves only when a row's maximum grew a lot (or at the first tile); then O,
      // which P V of the tile before may still be adding to, is rescaled once that MMA has finished
      const bool grow = tile_max > m_ref + kRescaleThreshold || (m_ref == -INFINITY && tile_max > -INFINITY);
      if (j == 0) {
        m_ref = tile_max;
      } else if (__any_sync(0xffffffffu, grow)) {
        // P V of tile t commits to v_empty[t % VS]. A parity wait tells a phase from the one before it only; here the barrier
        // of tile j - 1 has seen tile j - 1 - VS (S_j is ready, and P V of tile j - 2 was issued before it) and cannot have
        // seen tile j - 1 + VS (its P is not written yet), so the parity of tile j - 1 is not mistaken.
        wait(&v_empty[(j - 1) % VS], ((j - 1) / VS) & 1);
        sm100::tc_fence_after();
        const float m_new = grow ? fmaxf(m_ref, tile_max) : m_ref;
        const float f = m_new == -INFINITY ? 1.f : ex2(m_ref - m_new);  // 1 for rows that keep their reference, 0 when it was -inf
        l *= f;
        m_ref = m_new;
#pragma unroll 1
        for (int c0 = 0; c0 < HD; c0 += 32) {
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
      // P = 2^(S - m_ref) as bfloat16, two to a column, over the first 32 columns of S_j
      // (of every four keys, kMufu go through the special-function unit and the rest through the polynomial)
      uint32_t w[BN / 2];
      const float2 sc2 = make_float2(scale_log2e, scale_log2e), nmu2 = make_float2(-mu, -mu);
      float2 la = make_float2(0.f, 0.f), lb = make_float2(0.f, 0.f);
#pragma unroll
      for (int c = 0; c < BN; c += 4) {
        const float2 a = __ffma2_rn(make_float2(__uint_as_float(sr[c]), __uint_as_float(sr[c + 1])), sc2, nmu2);
        const float2 b = __ffma2_rn(make_float2(__uint_as_float(sr[c + 2]), __uint_as_float(sr[c + 3])), sc2, nmu2);
        const float2 pa = kMufu >= 2 ? make_float2(ex2(a.x), ex2(a.y)) : ex2_poly2(a);
        const float2 pb = kMufu >= 4 ? make_float2(ex2(b.x), ex2(b.y)) : ex2_poly2(b);
        la = __fadd2_rn(la, pa);
        lb = __fadd2_rn(lb, pb);
        w[c / 2] = pack_bf16x2(pa.x, pa.y);
        w[c / 2 + 1] = pack_bf16x2(pb.x, pb.y);
      }
      l += (la.x + la.y) + (lb.x + lb.y);
      sm100::tmem_st_32x32b_x32(t_lane + (j & 1) * BN, w);
      sm100::tmem_st_wait();
      sm100::tc_fence_before();
      __syncwarp();
      if (lane == 0) sm100::mbar_arrive(&p_full[j & 1]);
    }
    // ---- O / l -> out
    wait(&v_empty[(n_kt - 1) % VS], ((n_kt - 1) / VS) & 1);
    sm100::tc_fence_after();
    if (!*gave_up) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = out + ((size_t)(t0 + row) * heads + h) * HD;
#pragma unroll 1
      for (int c0 = 0; c0 < HD; c0 += 32) {
        uint32_t o[32];
        sm100::tmem_ld_32x32b_x32(t_lane + 2 * BN + c0, o);
        sm100::tmem_ld_wait();
        if (row < rows) {
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            uint4 v;
            v.x = mt::pack_bf16(__uint_as_float(o[c]) * inv, __uint_as_float(o[c + 1]) * inv);
            v.y = mt::pack_bf16(__uint_as_float(o[c + 2]) * inv, __uint_as_float(o[c + 3]) * inv);
            v.z = mt::pack_bf16(__uint_as_float(o[c + 4]) * inv, __uint_as_float(o[c + 5]) * inv);
            v.w = mt::pack_bf16(__uint_as_float(o[c + 6]) * inv, __uint_as_float(o[c + 7]) * inv);
            *(uint4*)(dst + c0 + c) = v;
          }
        }
      }
    }
  }
  // every role is done: the MMAs have finished (the softmax threads waited for the last one), copies have landed (every tile was used)
  sm100::tc_fence_before();
  __syncthreads();
  if (warp == kSoftmaxWarps) {
    __syncwarp();
    sm100::tmem_dealloc(tmem, kTmemCols);
  }
}

template <int HD>
int launch(const void* q, const IbKvView* kv, const int* tile_seg, const int* tile_row0, int n_tiles, const int* seg_start, const int* seg_pos0,
           int window, float scale, void* out, int heads, const CUtensorMap* kv_map, long long view_row0, unsigned* status, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(prefill_ws_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<HD>::kBytes);
    IB_CHECK_ARG(e == cudaSuccess, "attention_prefill_ws: cannot reserve %d bytes of shared memory: %s", Smem<HD>::kBytes, cudaGetErrorString(e));
    configured = true;
  }
  ib::launch(prefill_ws_kernel<HD>, dim3(heads, n_tiles), kThreads, Smem<HD>::kBytes, stream, (const __nv_bfloat16*)q, *kv, tile_seg, tile_row0,
             seg_start, seg_pos0, window, scale * 1.4426950408889634f, (__nv_bfloat16*)out, heads, *kv_map, view_row0, ib_wait_limit_ns(), status);
  IB_CHECK_LAUNCH("attention_prefill_ws");
  return 0;
}

}  // namespace

// Attention for query tiles of 128 rows: tile i covers rows tile_row0[i].. of segment tile_seg[i]; list the
// tiles that see the most keys first. kv_map: the tensor map of the view's pool (ib_make_kv_map), view_row0
// the pool row where this view's keys of page 0, head 0 start.
extern "C" int ib_attention_prefill_ws(const void* q, const IbKvView* kv, const int* tile_seg, const int* tile_row0, int n_tiles,
                                       const int* seg_start, const int* seg_pos0, int window, float scale, void* out, int heads,
                                       const void* kv_map, long long view_row0, unsigned* status, cudaStream_t stream) {
  if (n_tiles == 0) return 0;
  IB_CHECK_ARG(kv && kv->base && kv->block_table && kv_map, "attention_prefill_ws: the cache view or the tensor map is a null pointer");
  IB_CHECK_ARG(kv->dtype == IB_BF16, "attention_prefill_ws: the cache must be bfloat16");
  IB_CHECK_ARG(kv->page_size % 8 == 0 && (BN % kv->page_size == 0 || kv->page_size % BN == 0),
               "attention_prefill_ws: page size %d is not a multiple of 8 that divides %d or a multiple of %d", kv->page_size, BN, BN);
  IB_CHECK_ARG(kv->kv_heads > 0 && heads % kv->kv_heads == 0, "attention_prefill_ws: %d query heads are not a multiple of %d kv heads", heads,
               kv->kv_heads);
  IB_CHECK_ARG(n_tiles > 0 && n_tiles <= 65535, "attention_prefill_ws: %d query tiles (at most 65535 per launch)", n_tiles);
  IB_CHECK_ARG(kv->page_stride % kv->head_dim == 0 && kv->v_offset % kv->head_dim == 0, "attention_prefill_ws: strides are not whole rows");
  if (kv->head_dim == 128)
    return launch<128>(q, kv, tile_seg, tile_row0, n_tiles, seg_start, seg_pos0, window, scale, out, heads, (const CUtensorMap*)kv_map, view_row0,
                       status, stream);
  if (kv->head_dim == 64)
    return launch<64>(q, kv, tile_seg, tile_row0, n_tiles, seg_start, seg_pos0, window, scale, out, heads, (const CUtensorMap*)kv_map, view_row0,
                      status, stream);
  return ib_set_error("attention_prefill_ws: head_dim %d has no tensor-core kernel (64 and 128 have)", kv->head_dim);
}
