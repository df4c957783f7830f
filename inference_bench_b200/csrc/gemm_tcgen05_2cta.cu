// The large-tile matrix product on CTA pairs: out[t][n] = sum_k x[t][k] * w[n][k], bfloat16 operands,
// float32 accumulation, for prompts (256 tokens per tile; 128 with the SwiGLU epilogue).
//
// Two CTAs of a cluster (two neighbouring SMs) work on one 256 (rows of W) x 256 (tokens) tile with
// tcgen05.mma.cta_group::2: each CTA loads its own 128 rows of W and its own 128 of the 256 tokens,
// the MMA reads both halves of the token tile from the two SMs' shared memory, and each CTA's
// tensor memory receives the 128 x 256 block of its rows. Per FLOP this moves half the token-tile
// bytes of the single-CTA kernel, which is what limits that one. With two accumulators per CTA
// (gate rows and up rows of a SwiGLU feed-forward) the epilogue writes silu(gate) * up directly.
//
// Roles per CTA: warp 0 issues its TMA loads (completion is counted on the leader CTA's barrier),
// warp 1 of the leader CTA issues the MMAs for the pair and signals both CTAs' barriers, warps 2-5
// store this CTA's accumulator rows. No load uses cluster multicast. Every wait is bounded.
// The reference's equivalent is its mma.sync tile kernel (crates/kir/src/cuda/gemm/core.rs:14-155).
#include <cuda.h>

#include <cuda_bf16.h>

#include "kv_view.cuh"
#include "sm100.cuh"
#include "tma_host.cuh"

namespace {

constexpr int BM = 128;      // rows of W per CTA (256 per pair)
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;
constexpr int EPI_STORE = 0, EPI_SWIGLU = 1, EPI_ADD = 2;   // float32 out; bfloat16 silu(gate) * up; float32 out += product
constexpr int EPI_QKV = 3;   // the q/k/v projection finished in the epilogue: per-head norm, rotation, queries out, keys and values into the cache
constexpr int kQkvHead = 128;   // head size of the EPI_QKV form: a head is 128 accumulator columns
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;   // clears the bit that tells the two CTAs of a pair apart in a shared::cluster address

// BN: tokens per tile = accumulator columns (each CTA loads half of them)
template <int MT, int BN>
struct Tile {
  static constexpr int kABytes = BM * BK * 2, kBBytes = (BN / 2) * BK * 2;
  static constexpr int kStageBytes = MT * kABytes + kBBytes;
  static constexpr int kStages = (200 * 1024) / kStageBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /* alignment slack */ + 256 /* barriers */ + 1024 /* norm scales of EPI_QKV */;
  static constexpr int kAccSets = 512 / (MT * BN);   // accumulator sets that fit tensor memory
};

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {   // round to nearest even
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sm100::smem_u32(slot)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc2(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
// TMA tile load whose completion bytes are counted on the barrier at the same offset in the pair's leader CTA.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          sm100::smem_u32(smem_dst)),
      "l"(m), "r"(x), "r"(y), "r"(sm100::smem_u32(bar) & kPeerBitMask)
      : "memory");
}
__device__ __forceinline__ void mma_bf16_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at this offset in both CTAs of the pair once the MMAs issued so far are done.
__device__ __forceinline__ void mma_commit_pair(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(sm100::smem_u32(bar)),
               "h"((uint16_t)3)
               : "memory");
}

// Arrive on the barrier at this offset in the pair's leader CTA (from either CTA).
__device__ __forceinline__ void arrive_on_leader(uint64_t* bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(sm100::smem_u32(bar) & kPeerBitMask) : "memory");
}

// What the EPI_QKV epilogue works with. The product is taken the other way round there: the tokens are the
// rows of the MMA (tensor-memory lanes: a thread of the epilogue owns a token) and the rows of the fused
// [q | k | v] weight are its columns, so that a head's 128 values of a token sit in one thread: the norm is a
// sum inside the thread, the rotation partner (d + 64) is the thread's own, and a token's head goes out as one
// contiguous row. What `qk_norm_rope_kv` computes from the stored product, with the same formulas:
// per-head RMSNorm of q and k heads (scales or null), half rotation by the step's tables (or null), queries
// as bfloat16 [tokens][heads * 128], keys and values into the paged cache at the token's position.
struct QkvEpi {
  const float* q_norm_w;
  const float* k_norm_w;
  float eps;
  const float* cos_t;   // [tokens][64]
  const float* sin_t;
  const int* positions;
  const int* seg_of_token;
  __nv_bfloat16* q_out;
  IbKvView kv;
  int write_kv;
  int heads;
};

// Persistent: each CTA pair walks tiles pair, pair + n_pairs, ... (token tiles vary fastest, so the
// pairs that work at the same time share rows of W). The TMA warps run ahead into the next tile
// while the accumulator of the last one is stored; with one accumulator per tile (MT = 1) tensor
// memory holds two of them, so the next tile's MMAs also run during that store.
template <int MT, int EPI, int BN>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_2cta_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, void* __restrict__ out_, int T, int N,
                     int K, int token_tiles, int total_tiles, int second_off, unsigned long long wait_ns, unsigned* __restrict__ status, const QkvEpi qe) {
  using TL = Tile<MT, BN>;
  constexpr int STAGES = TL::kStages;
  constexpr int BNH = BN / 2;
  constexpr int NBUF = TL::kAccSets >= 2 ? 2 : 1;   // accumulator sets in use
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = sm100::smem_u32(smem_raw);
  uint8_t* tiles = smem_raw + (((raw + 1023u) & ~1023u) - raw);   // the same offset in both CTAs: same kernel, same launch
  uint64_t* full = (uint64_t*)(tiles + STAGES * TL::kStageBytes);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;   // [NBUF]
  uint64_t* acc_empty = acc_full + 2;    // [NBUF], used in the leader CTA
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  float* norm_s = (float*)(tiles + STAGES * TL::kStageBytes + 256);   // EPI_QKV: q scales [128], k scales [128]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();          // 0 = leader
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int nkt = (K + BK - 1) / BK;
  constexpr int kColsPerPair = EPI == EPI_SWIGLU ? 2 * BM : 2 * BM * MT;

  ib::pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      sm100::mbar_init(&full[s], 1);
      sm100::mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; b++) {
      sm100::mbar_init(&acc_full[b], 1);
      sm100::mbar_init(&acc_empty[b], 8);   // four epilogue warps in each of the two CTAs
    }
    sm100::fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc2(tmem_slot, 512);
    tmem_relinquish2();
  }
  if constexpr (EPI == EPI_QKV) {   // the norm scales are weights: nothing earlier in the stream writes them
    for (int i = threadIdx.x; i < 2 * kQkvHead; i += kThreads) {
      const float* src = i < kQkvHead ? qe.q_norm_w : qe.k_norm_w;
      norm_s[i] = src ? src[i % kQkvHead] : 1.f;
    }
  }
  sm100::tc_fence_before();
  __syncthreads();
  cluster_sync();   // both CTAs' barriers exist before either signals the other's
  sm100::tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  // W rows of accumulator m of this CTA for the pair's row block rb: plain tiles stack 256-row pairs;
  // SwiGLU takes gate rows and, second_off on, up rows
  auto w_row = [&](int rb, int m) {
    const int n_pair = rb * kColsPerPair;
    return EPI == EPI_SWIGLU ? n_pair + (int)rank * BM + m * second_off : n_pair + m * 2 * BM + (int)rank * BM;
  };

  if (warp == 0) {
    if (sm100::elect_one()) {
      sm100::prefetch_tensormap(&tmap_w);
      sm100::prefetch_tensormap(&tmap_x);
      bool waited = false, ok = true;
      int it = 0;   // k-tiles sent so far, over all tiles: stage = it % STAGES
      for (int tile = pair; tile < total_tiles && ok; tile += n_pairs) {
        const int t0 = (tile % token_tiles) * BN, rb = tile / token_tiles;
        for (int i = 0; i < nkt; i++, it++) {
          const int s = it % STAGES;
          if (!sm100::mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1, wait_ns)) {
            atomicOr(status, IB_ERR_WAIT_TIMEOUT);
            ok = false;
            break;
          }
          uint8_t* a = tiles + s * TL::kStageBytes;
          if (rank == 0) sm100::mbar_arrive_expect_tx(&full[s], 2 * TL::kStageBytes);   // the leader counts both CTAs' bytes
          if (EPI == EPI_QKV && !waited) {   // there the rows are the tokens, which the kernel before wrote
            ib::pdl_wait();
            waited = true;
          }
#pragma unroll
          for (int m = 0; m < MT; m++) tma_load_2d_pair(a + m * TL::kABytes, &tmap_w, i * BK, w_row(rb, m), &full[s]);
          if (!waited) {   // the weights above do not depend on earlier kernels; x does
            ib::pdl_wait();
            waited = true;
          }
          tma_load_2d_pair(a + MT * TL::kABytes, &tmap_x, i * BK, t0 + (int)rank * BNH, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (rank == 0 && sm100::elect_one()) {
      constexpr uint32_t idesc = sm100::idesc_bf16_f32(2 * BM, BN);
      bool ok = true;
      int it = 0, tl = 0;
      for (int tile = pair; tile < total_tiles && ok; tile += n_pairs, tl++) {
        const int b = tl % NBUF;
        if (tl >= NBUF && !sm100::mbar_wait(&acc_empty[b], ((tl / NBUF) - 1) & 1, wait_ns)) {   // the accumulator's last contents have been stored
          atomicOr(status, IB_ERR_WAIT_TIMEOUT);
          ok = false;
          break;
        }
        sm100::tc_fence_after();
        for (int i = 0; i < nkt; i++, it++) {
          const int s = it % STAGES;
          if (!sm100::mbar_wait(&full[s], (it / STAGES) & 1, wait_ns)) {
            atomicOr(status, IB_ERR_WAIT_TIMEOUT);
            ok = false;
            break;
          }
          sm100::tc_fence_after();
          const uint32_t a_addr = sm100::smem_u32(tiles + s * TL::kStageBytes);
          const uint64_t db = sm100::smem_desc_sw128(a_addr + MT * TL::kABytes);
#pragma unroll
          for (int m = 0; m < MT; m++) {
            const uint64_t da = sm100::smem_desc_sw128(a_addr + m * TL::kABytes);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; k++) mma_bf16_ss_pair(tmem + b * MT * BN + m * BN, da + 2 * k, db + 2 * k, idesc, (i | k) != 0);
          }
          mma_commit_pair(&empty[s]);
        }
        if (ok) mma_commit_pair(&acc_full[b]);
      }
    }
  } else {
    const int q = warp & 3;
    ib::pdl_wait();
    const uint32_t lane_addr = tmem + ((uint32_t)(q * 32) << 16);
    int tl = 0;
    for (int tile = pair; tile < total_tiles; tile += n_pairs, tl++) {
      const int b = tl % NBUF;
      const int t0 = (tile % token_tiles) * BN, n_pair = (tile / token_tiles) * kColsPerPair;
      bool ok = sm100::mbar_wait(&acc_full[b], (tl / NBUF) & 1, wait_ns);
      if (!ok && lane == 0) atomicOr(status, IB_ERR_WAIT_TIMEOUT);
      sm100::tc_fence_after();
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if constexpr (EPI == EPI_QKV) {
        // this thread's token, and the (up to) two heads of the tile: columns [0,128) and [128,256) of the accumulator
        const int tok = n_pair + (int)rank * BM + q * 32 + lane;
        const bool live = tok < N;
        const int kvh = qe.kv.kv_heads;
        int pos = 0, seg = 0;
        if (live && qe.write_kv) {
          pos = qe.positions[tok];
          seg = qe.seg_of_token[tok];
        }
        const float* cs = qe.cos_t ? qe.cos_t + (size_t)tok * (kQkvHead / 2) : nullptr;
        const float* sn = qe.sin_t ? qe.sin_t + (size_t)tok * (kQkvHead / 2) : nullptr;
#pragma unroll 1
        for (int hh = 0; hh < BN / kQkvHead; hh++) {
          const int j = t0 / kQkvHead + hh;   // head slot: q heads, then k heads, then v heads
          if (j * kQkvHead >= T) break;
          const bool is_q = j < qe.heads, is_k = !is_q && j < qe.heads + kvh;
          if (!is_q && !qe.write_kv) continue;
          const uint32_t col0 = lane_addr + b * MT * BN + hh * kQkvHead;
          const float* nw = is_q ? (qe.q_norm_w ? norm_s : nullptr) : (is_k && qe.k_norm_w ? norm_s + kQkvHead : nullptr);
          float inv = 1.f;
          if (nw) {   // sum of squares over the head, d rising (uniform branch: every lane of the warp reads tensor memory)
            float ss = 0.f;
#pragma unroll 1
            for (int c0 = 0; c0 < kQkvHead; c0 += 32) {
              uint32_t r[32];
              sm100::tmem_ld_32x32b_x32(col0 + c0, r);
              sm100::tmem_ld_wait();
#pragma unroll
              for (int c = 0; c < 32; c++) ss = __fmaf_rn(__uint_as_float(r[c]), __uint_as_float(r[c]), ss);
            }
            inv = rsqrtf(ss / (float)kQkvHead + qe.eps);
          }
          // destination row of this token's head
          __nv_bfloat16* dst = nullptr;
          if (live) {
            if (is_q) {
              dst = qe.q_out + ((size_t)tok * qe.heads + j) * kQkvHead;
            } else {
              const long long off = ib::kv_offset(qe.kv, seg, pos, is_k ? j - qe.heads : j - qe.heads - kvh);
              if (off < 0)
                atomicOr(status, IB_ERR_BAD_PAGE);
              else
                dst = (__nv_bfloat16*)qe.kv.base + off + (is_k ? 0 : qe.kv.v_offset);
            }
          }
          const bool turn = (is_q || is_k) && cs != nullptr;
#pragma unroll 1
          for (int c0 = 0; c0 < kQkvHead / 2; c0 += 32) {   // values d = c0 + c and their rotation partners d + 64
            uint32_t lo[32], hi[32];
            sm100::tmem_ld_32x32b_x32(col0 + c0, lo);
            sm100::tmem_ld_32x32b_x32(col0 + kQkvHead / 2 + c0, hi);
            sm100::tmem_ld_wait();
            if (dst) {
#pragma unroll
              for (int c4 = 0; c4 < 32; c4 += 4) {
                float a[4], bb[4];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                  a[e] = __uint_as_float(lo[c4 + e]);
                  bb[e] = __uint_as_float(hi[c4 + e]);
                  if (nw) {
                    a[e] = nw[c0 + c4 + e] * (a[e] * inv);
                    bb[e] = nw[kQkvHead / 2 + c0 + c4 + e] * (bb[e] * inv);
                  }
                }
                if (turn) {
                  const float4 c = *(const float4*)(cs + c0 + c4), sgn = *(const float4*)(sn + c0 + c4);
                  const float cv[4] = {c.x, c.y, c.z, c.w}, sv[4] = {sgn.x, sgn.y, sgn.z, sgn.w};
#pragma unroll
                  for (int e = 0; e < 4; e++) {
                    const float x0 = a[e], x1 = bb[e];
                    a[e] = __fmaf_rn(x1, -sv[e], __fmul_rn(x0, cv[e]));
                    bb[e] = __fmaf_rn(x0, sv[e], __fmul_rn(x1, cv[e]));
                  }
                }
                lo[c4 / 2] = pack_bf16x2(a[0], a[1]);
                lo[c4 / 2 + 1] = pack_bf16x2(a[2], a[3]);
                hi[c4 / 2] = pack_bf16x2(bb[0], bb[1]);
                hi[c4 / 2 + 1] = pack_bf16x2(bb[2], bb[3]);
              }
#pragma unroll
              for (int v = 0; v < 4; v++) {
                *(uint4*)(dst + c0 + 8 * v) = make_uint4(lo[4 * v], lo[4 * v + 1], lo[4 * v + 2], lo[4 * v + 3]);
                *(uint4*)(dst + kQkvHead / 2 + c0 + 8 * v) = make_uint4(hi[4 * v], hi[4 * v + 1], hi[4 * v + 2], hi[4 * v + 3]);
              }
            }
          }
        }
      } else if constexpr (EPI == EPI_STORE || EPI == EPI_ADD) {
        float* dst = (float*)out_;
#pragma unroll 1
        for (int m = 0; m < MT; m++) {
          const int n = n_pair + m * 2 * BM + (int)rank * BM + q * 32 + lane;
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 32) {
            uint32_t r[32];
            sm100::tmem_ld_32x32b_x32(lane_addr + b * MT * BN + m * BN + c0, r);
            sm100::tmem_ld_wait();
            if (n < N) {
              if constexpr (EPI == EPI_ADD) {   // every element belongs to one thread of one CTA: a plain read, add, write
                float old[32];
#pragma unroll
                for (int c = 0; c < 32; c++) old[c] = t0 + c0 + c < T ? dst[(size_t)(t0 + c0 + c) * N + n] : 0.f;
#pragma unroll
                for (int c = 0; c < 32; c++) r[c] = __float_as_uint(old[c] + __uint_as_float(r[c]));
              }
#pragma unroll
              for (int c = 0; c < 32; c++) {
                const int t = t0 + c0 + c;
                if (t < T) dst[(size_t)t * N + n] = __uint_as_float(r[c]);
              }
            }
          }
        }
      } else {
        __nv_bfloat16* dst = (__nv_bfloat16*)out_;
        const int n = n_pair + (int)rank * BM + q * 32 + lane;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t g[32], u[32];
          sm100::tmem_ld_32x32b_x32(lane_addr + b * MT * BN + c0, g);
          sm100::tmem_ld_32x32b_x32(lane_addr + b * MT * BN + BN + c0, u);
          sm100::tmem_ld_wait();
          if (n < N) {
#pragma unroll
            for (int c = 0; c < 32; c++) {
              const int t = t0 + c0 + c;
              const float gv = __uint_as_float(g[c]), uv = __uint_as_float(u[c]);
              if (t < T) dst[(size_t)t * N + n] = __float2bfloat16_rn(__fdividef(gv, 1.f + __expf(-gv)) * uv);
            }
          }
        }
      }
      // this warp has read its part of the accumulator: tell the leader's MMA warp
      sm100::tc_fence_before();
      __syncwarp();
      if (lane == 0) arrive_on_leader(&acc_empty[b]);
    }
  }
  sm100::tc_fence_before();
  __syncthreads();
  cluster_sync();   // neither CTA leaves (or frees tensor memory) while its partner may still signal it
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc2(tmem, 512);
  }
}

int make_tmap(CUtensorMap* m, const void* ptr, int rows, int K, int box_rows) {
  tma_host::EncodeTiledFn fn = tma_host::encode_fn();
  IB_CHECK_ARG(fn, "gemm_tcgen05_2cta: the driver has no cuTensorMapEncodeTiled");
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  IB_CHECK_ARG(r == CUDA_SUCCESS, "gemm_tcgen05_2cta: cuTensorMapEncodeTiled failed with code %d", (int)r);
  return 0;
}

template <int MT, int EPI, int BN>
int launch(const void* x, const void* w, void* out, int T, int N, int K, int w_rows, int second_off, unsigned* status, cudaStream_t stream,
           const QkvEpi& qe = QkvEpi{}) {
  using TL = Tile<MT, BN>;
  IB_CHECK_ARG(T > 0 && N > 0 && K > 0 && K % 8 == 0, "gemm_tcgen05_2cta: bad sizes T=%d N=%d K=%d (K must be a multiple of 8)", T, N, K);
  IB_CHECK_ARG(((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0, "gemm_tcgen05_2cta: operands must be 16-byte aligned");
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_2cta_kernel<MT, EPI, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, TL::kSmemBytes);
    IB_CHECK_ARG(e == cudaSuccess, "gemm_tcgen05_2cta: cannot reserve %d bytes of shared memory: %s", TL::kSmemBytes, cudaGetErrorString(e));
    configured = true;
  }
  CUtensorMap tw, tx;
  if (make_tmap(&tw, w, w_rows, K, BM)) return 1;
  if (make_tmap(&tx, x, T, K, BN / 2)) return 1;
  const int cols_per_pair = EPI == EPI_SWIGLU ? 2 * BM : 2 * BM * MT;
  const int token_tiles = (T + BN - 1) / BN, row_blocks = (N + cols_per_pair - 1) / cols_per_pair;
  const int total_tiles = token_tiles * row_blocks;
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  const int n_pairs = total_tiles < sm_count / 2 ? total_tiles : sm_count / 2;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * n_pairs);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = TL::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = ib_pdl_enabled();
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_2cta_kernel<MT, EPI, BN>, tw, tx, out, T, N, K, token_tiles, total_tiles, second_off, ib_wait_limit_ns(), status, qe);
  IB_CHECK_ARG(e == cudaSuccess, "gemm_tcgen05_2cta: launch failed: %s", cudaGetErrorString(e));
  return 0;
}

}  // namespace

// x [T, K], w [N, K] bfloat16 -> out [T, N] float32, 256 x 256 tiles on CTA pairs (meant for T >= 256).
extern "C" int ib_gemm_tcgen05_2cta(const void* x, const void* w, float* out, int T, int N, int K, unsigned* status, cudaStream_t stream) {
  if (T == 0 || N == 0) return 0;
  return launch<1, EPI_STORE, 256>(x, w, out, T, N, K, N, 0, status, stream);
}

// The same product added to what out [T, N] float32 holds (the residual stream), in place.
extern "C" int ib_gemm_tcgen05_2cta_add(const void* x, const void* w, float* out, int T, int N, int K, unsigned* status, cudaStream_t stream) {
  if (T == 0 || N == 0) return 0;
  return launch<1, EPI_ADD, 256>(x, w, out, T, N, K, N, 0, status, stream);
}

// w [2*I, K] = gate rows then up rows -> act [T, I] bfloat16 = silu(x gate^T) * (x up^T), on CTA pairs.
extern "C" int ib_gemm_swiglu_tcgen05_2cta(const void* x, const void* w, void* act, int T, int I, int K, unsigned* status, cudaStream_t stream) {
  if (T == 0 || I == 0) return 0;
  return launch<2, EPI_SWIGLU, 128>(x, w, act, T, I, K, 2 * I, I, status, stream);
}

// The q/k/v projection with its epilogue: x [T, K] bfloat16 and w [(heads + 2 kv_heads) * 128, K] bfloat16 (q rows, k rows, v rows)
// -> q_out [T, heads * 128] bfloat16 normed and turned, and (write_kv) keys and values of each token at its position
// in the paged cache; what ib_gemm_tcgen05_2cta followed by ib_qk_norm_rope_kv gives, without the float32 product
// in memory between them. Head size 128, a bfloat16 cache, the whole head turned (cos_t, sin_t [T, 64]) or none of it.
extern "C" int ib_gemm_qkv_tcgen05_2cta(const void* x, const void* w, int T, int K, const float* q_norm_w, const float* k_norm_w, float eps,
                                        const float* cos_t, const float* sin_t, const int* positions, const int* seg_of_token, void* q_out,
                                        const IbKvView* kv, int write_kv, int heads, unsigned* status, cudaStream_t stream) {
  if (T == 0) return 0;
  IB_CHECK_ARG(kv && q_out && positions && seg_of_token, "gemm_qkv_tcgen05_2cta: a null pointer");
  IB_CHECK_ARG(kv->head_dim == kQkvHead, "gemm_qkv_tcgen05_2cta: head size %d (this form has 128)", kv->head_dim);
  IB_CHECK_ARG(!write_kv || (kv->base && kv->block_table && kv->dtype == IB_BF16), "gemm_qkv_tcgen05_2cta: the cache must be bfloat16");
  IB_CHECK_ARG(heads > 0 && kv->kv_heads > 0, "gemm_qkv_tcgen05_2cta: %d heads, %d kv heads", heads, kv->kv_heads);
  IB_CHECK_ARG((cos_t == nullptr) == (sin_t == nullptr), "gemm_qkv_tcgen05_2cta: one rotation table without the other");
  IB_CHECK_ARG(((uintptr_t)q_out & 15) == 0 && ((uintptr_t)kv->base & 15) == 0 && ((uintptr_t)cos_t & 15) == 0 && ((uintptr_t)sin_t & 15) == 0,
               "gemm_qkv_tcgen05_2cta: outputs and tables must be 16-byte aligned");
  QkvEpi qe = {q_norm_w, k_norm_w, eps, cos_t, sin_t, positions, seg_of_token, (__nv_bfloat16*)q_out, *kv, write_kv, heads};
  const int N = (heads + 2 * kv->kv_heads) * kQkvHead;
  // the other way round: the tokens are the rows of the product, the weight's rows its columns
  return launch<1, EPI_QKV, 256>(w, x, nullptr, N, T, K, T, 0, status, stream, qe);
}
