// out[p][t][n] = sum over split p's k-range of x[t][k] * w[n][k]: bfloat16 operands, float32
// accumulation in tensor memory, on the sm_100a tensor cores (tcgen05.mma fed by TMA).
//
// The weight matrix sits in the MMA's M dimension (128 rows of W per MMA) and the tokens in its N
// dimension (16 to 256 per CTA), so the same kernel streams weights at memory speed for a handful
// of decoded tokens and runs large tiles for a prompt. Both operands are K-major in memory, which
// is how [rows, K] row-major tensors already are: no transposes anywhere.
//
// A CTA may hold two accumulators (MT = 2) that share the token tile: either two neighbouring
// 128-row blocks of W (a 256 x BN output tile, half the token-tile traffic per FLOP), or a block of
// gate rows and the matching block of up rows of a SwiGLU feed-forward, whose epilogue then writes
// silu(gate) * up in bfloat16 directly and the [T, 2I] intermediate never exists in memory.
//
// CTA = 6 warps: warp 0 issues TMA loads, warp 1 owns tensor memory and issues the MMAs, warps 2-5
// read the accumulators back (tcgen05.ld: warp w may touch lanes 32*(w%4)..+31) and store.
// The reference's equivalent is its mma.sync tile kernel (crates/kir/src/cuda/gemm/core.rs:14-155)
// with the ACT epilogue for gate/up (core.rs:199-213).
#include <cuda.h>

#include "sm100.cuh"
#include "tma_host.cuh"

namespace {

constexpr int BM = 128;     // weight rows per MMA (MMA M)
constexpr int BK = 64;      // k per stage: 64 bfloat16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;  // k per tcgen05.mma of kind::f16
constexpr int kThreads = 192;
constexpr int EPI_STORE = 0;   // float32 partial products
constexpr int EPI_SWIGLU = 1;  // accumulator 0 = gate, accumulator 1 = up -> bfloat16 silu(gate) * up
constexpr int EPI_SWIGLU_HALF = 2;  // one accumulator: rows 0-63 = 64 gate rows, rows 64-127 = the matching 64 up rows -> bfloat16 silu(gate) * up
// (for a handful of tokens: as many CTAs as the plain product has, I / 64, so the weights stream as fast, and neither the
// float32 [T, 2I] intermediate nor the SiLU-mul kernel exists)

template <int BN, int MT>
struct Tile {
  static constexpr int kABytes = BM * BK * 2;            // one 128-row block of W
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = MT * kABytes + kBBytes;
  // few tokens: shallower pipelines so that two CTAs share an SM and more loads are in flight
  static constexpr int kStages = MT == 2 ? (BN >= 256 ? 3 : 4) : (BN >= 256 ? 4 : (BN >= 128 ? 6 : (BN >= 64 ? 4 : (BN >= 32 ? 5 : 6))));
  static constexpr int kCols = MT * BN;
  static constexpr int kTmemCols = kCols <= 32 ? 32 : (kCols <= 64 ? 64 : (kCols <= 128 ? 128 : (kCols <= 256 ? 256 : 512)));
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /* alignment slack */ + 256 /* barriers */;
};

template <int BN, int MT, int EPI>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, void* __restrict__ out_, int T,
                        int N, int K, int ktiles_per_split, int second_off, unsigned long long wait_ns, int starve, unsigned* __restrict__ status) {
  // wait_ns: the limit of every wait below. starve != 0 (the wait-limit test only): the copying warp sends nothing, so that
  // the waits run out the way they would if a copy never landed, and the kernel has to unwind through its ordinary path.
  using TL = Tile<BN, MT>;
  constexpr int STAGES = TL::kStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = sm100::smem_u32(smem_raw);
  uint8_t* tiles = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  uint64_t* full = (uint64_t*)(tiles + STAGES * TL::kStageBytes);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // first output column of this CTA, and the W row where each accumulator's block starts
  // (token tiles vary fastest in the grid: the CTAs that share a block of W run together, so W comes
  // from memory once and the much smaller x stays in L2)
  const int n0 = blockIdx.y * (EPI == EPI_SWIGLU_HALF ? BM / 2 : EPI == EPI_SWIGLU ? BM : BM * MT);
  const int t0 = blockIdx.x * BN, split = blockIdx.z;
  const int total_kt = (K + BK - 1) / BK;
  const int kt_begin = split * ktiles_per_split;
  const int kt_end = min(total_kt, kt_begin + ktiles_per_split);
  const int nkt = max(0, kt_end - kt_begin);

  ib::pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      sm100::mbar_init(&full[s], 1);
      sm100::mbar_init(&empty[s], 1);
    }
    sm100::mbar_init(acc_full, 1);
    sm100::fence_barrier_init();
  }
  if (warp == 1) {
    sm100::tmem_alloc(tmem_slot, TL::kTmemCols);
    sm100::tmem_relinquish();
  }
  sm100::tc_fence_before();
  __syncthreads();
  sm100::tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (!starve && sm100::elect_one()) {
      sm100::prefetch_tensormap(&tmap_w);
      sm100::prefetch_tensormap(&tmap_x);
      // The weights do not depend on earlier kernels: fill the pipeline with them before waiting
      // for the kernel that produces x, then send the x tiles after.
      auto load_w = [&](uint8_t* a, int kt, uint64_t* bar) {   // this CTA's rows of W for k-tile kt
        if constexpr (EPI == EPI_SWIGLU_HALF) {   // tmap_w's box has 64 rows here: gate rows, then the up rows second_off further on
          sm100::tma_load_2d(a, &tmap_w, kt * BK, n0, bar);
          sm100::tma_load_2d(a + TL::kABytes / 2, &tmap_w, kt * BK, n0 + second_off, bar);
        } else {
#pragma unroll
          for (int m = 0; m < MT; m++) sm100::tma_load_2d(a + m * TL::kABytes, &tmap_w, kt * BK, n0 + m * second_off, bar);
        }
      };
      const int first = min(nkt, STAGES);
      for (int i = 0; i < first; i++) {
        sm100::mbar_arrive_expect_tx(&full[i], TL::kStageBytes);
        load_w(tiles + i * TL::kStageBytes, kt_begin + i, &full[i]);
      }
      ib::pdl_wait();
      for (int i = 0; i < first; i++)
        sm100::tma_load_2d(tiles + i * TL::kStageBytes + MT * TL::kABytes, &tmap_x, (kt_begin + i) * BK, t0, &full[i]);
      for (int i = first; i < nkt; i++) {
        const int s = i % STAGES;
        if (!sm100::mbar_wait(&empty[s], ((i / STAGES) & 1) ^ 1, wait_ns)) {
          atomicOr(status, IB_ERR_WAIT_TIMEOUT);
          break;
        }
        uint8_t* a = tiles + s * TL::kStageBytes;
        sm100::mbar_arrive_expect_tx(&full[s], TL::kStageBytes);
        load_w(a, kt_begin + i, &full[s]);
        sm100::tma_load_2d(a + MT * TL::kABytes, &tmap_x, (kt_begin + i) * BK, t0, &full[s]);
      }
    }
  } else if (warp == 1) {
    if (sm100::elect_one()) {
      constexpr uint32_t idesc = sm100::idesc_bf16_f32(BM, BN);
      bool ok = true;
      for (int i = 0; i < nkt && ok; i++) {
        const int s = i % STAGES;
        if (!sm100::mbar_wait(&full[s], (i / STAGES) & 1, wait_ns)) {
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
          for (int k = 0; k < BK / UMMA_K; k++) {
            // inside the 128-byte swizzle row the next 16 k-values are 32 bytes on: +2 in the >>4 address field
            sm100::mma_bf16_ss(tmem + m * BN, da + 2 * k, db + 2 * k, idesc, (i | k) != 0);
          }
        }
        sm100::mma_commit(&empty[s]);
      }
      if (ok) sm100::mma_commit(acc_full);
    }
  } else {
    // Epilogue: this warp's quarter of the 128 accumulator lanes.
    const int q = warp & 3;
    ib::pdl_wait();   // the output buffer may still be in use by an earlier kernel
    bool ok = true;
    if (nkt > 0) {
      ok = sm100::mbar_wait(acc_full, 0, wait_ns);
      if (!ok && lane == 0) atomicOr(status, IB_ERR_WAIT_TIMEOUT);
      sm100::tc_fence_after();
    }
    ok = __all_sync(0xffffffffu, ok);
    constexpr int CH = BN < 32 ? 16 : 32;
    const uint32_t lane_addr = tmem + ((uint32_t)(q * 32) << 16);
    if (ok && EPI == EPI_STORE) {
      float* dst = (float*)out_ + (size_t)split * T * N;
#pragma unroll 1
      for (int m = 0; m < MT; m++) {
        const int n = n0 + m * BM + q * 32 + lane;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += CH) {
          uint32_t r[CH];
          if (nkt > 0) {
            if constexpr (CH == 32)
              sm100::tmem_ld_32x32b_x32(lane_addr + m * BN + c0, r);
            else
              sm100::tmem_ld_32x32b_x16(lane_addr + m * BN + c0, r);
            sm100::tmem_ld_wait();
          } else {
#pragma unroll
            for (int c = 0; c < CH; c++) r[c] = 0u;
          }
          if (n < N) {
#pragma unroll
            for (int c = 0; c < CH; c++) {
              const int t = t0 + c0 + c;
              if (t < T) dst[(size_t)t * N + n] = __uint_as_float(r[c]);
            }
          }
        }
      }
    }
    if (ok && EPI == EPI_SWIGLU) {
      __nv_bfloat16* dst = (__nv_bfloat16*)out_;
      const int n = n0 + q * 32 + lane;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += CH) {
        uint32_t g[CH], u[CH];
        if constexpr (CH == 32) {
          sm100::tmem_ld_32x32b_x32(lane_addr + c0, g);
          sm100::tmem_ld_32x32b_x32(lane_addr + BN + c0, u);
        } else {
          sm100::tmem_ld_32x32b_x16(lane_addr + c0, g);
          sm100::tmem_ld_32x32b_x16(lane_addr + BN + c0, u);
        }
        sm100::tmem_ld_wait();
        if (n < N) {
#pragma unroll
          for (int c = 0; c < CH; c++) {
            const int t = t0 + c0 + c;
            const float gv = __uint_as_float(g[c]), uv = __uint_as_float(u[c]);
            if (t < T) dst[(size_t)t * N + n] = __float2bfloat16_rn(__fdividef(gv, 1.f + __expf(-gv)) * uv);
          }
        }
      }
    }
    if constexpr (EPI == EPI_SWIGLU_HALF) {
      // Lanes 0-63 of the accumulator (warps with q = 0, 1) hold gate rows, lanes 64-127 (q = 2, 3) the matching up rows. The up
      // half goes through shared memory (the pipeline's stages are free once the accumulator is complete) to the warps that
      // hold the gate half, which apply the activation and store. All four warps meet at a barrier of their own, whatever ok says.
      float* up_s = (float*)tiles;   // [64][BN]
      uint32_t r[CH];
      static_assert(BN <= 64, "the half-and-half form is for few tokens");
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += CH) {
        if (ok) {
          if constexpr (CH == 32)
            sm100::tmem_ld_32x32b_x32(lane_addr + c0, r);
          else
            sm100::tmem_ld_32x32b_x16(lane_addr + c0, r);
          sm100::tmem_ld_wait();
        }
        if (ok && q >= 2) {
#pragma unroll
          for (int c = 0; c < CH; c++) up_s[(c0 + c) * 64 + (q - 2) * 32 + lane] = __uint_as_float(r[c]);   // [token][row]: no bank conflicts
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (ok && q < 2) {
          __nv_bfloat16* dst = (__nv_bfloat16*)out_;
          const int n = n0 + q * 32 + lane;
          if (n < N) {
#pragma unroll
            for (int c = 0; c < CH; c++) {
              const int t = t0 + c0 + c;
              const float gv = __uint_as_float(r[c]), uv = up_s[(c0 + c) * 64 + q * 32 + lane];
              if (t < T) dst[(size_t)t * N + n] = __float2bfloat16_rn(__fdividef(gv, 1.f + __expf(-gv)) * uv);
            }
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");   // the buffer is read before the next chunk overwrites it
      }
    }
  }
  sm100::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    sm100::tmem_dealloc(tmem, TL::kTmemCols);
  }
}

// ---------------------------------------------------------------- host side
// A [rows, K] row-major bfloat16 matrix read in boxes of [box_rows, 64] with the 128-byte swizzle;
// out-of-range rows and columns read as zero.
int make_tmap(CUtensorMap* m, const void* ptr, int rows, int K, int box_rows) {
  tma_host::EncodeTiledFn fn = tma_host::encode_fn();
  IB_CHECK_ARG(fn, "gemm_tcgen05: the driver has no cuTensorMapEncodeTiled");
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  IB_CHECK_ARG(r == CUDA_SUCCESS, "gemm_tcgen05: cuTensorMapEncodeTiled failed with code %d (rows=%d K=%d box_rows=%d)", (int)r, rows, K, box_rows);
  return 0;
}

template <int BN, int MT, int EPI>
int launch(const CUtensorMap& tw, const CUtensorMap& tx, void* out, int T, int N, int K, int splits, int kt_per_split, int second_off,
           unsigned* status, cudaStream_t stream, int starve = 0) {
  using TL = Tile<BN, MT>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, MT, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, TL::kSmemBytes);
    IB_CHECK_ARG(e == cudaSuccess, "gemm_tcgen05: cannot reserve %d bytes of shared memory: %s", TL::kSmemBytes, cudaGetErrorString(e));
    configured = true;
  }
  const int cols_per_cta = EPI == EPI_SWIGLU_HALF ? BM / 2 : EPI == EPI_SWIGLU ? BM : BM * MT;
  dim3 grid((T + BN - 1) / BN, (N + cols_per_cta - 1) / cols_per_cta, splits);
  IB_CHECK_ARG(grid.y <= 65535, "gemm_tcgen05: N=%d gives more than 65535 row blocks", N);
  ib::launch(gemm_tcgen05_kernel<BN, MT, EPI>, grid, kThreads, TL::kSmemBytes, stream, tw, tx, out, T, N, K, kt_per_split, second_off, ib_wait_limit_ns(), starve, status);
  IB_CHECK_LAUNCH("gemm_tcgen05");
  return 0;
}

int check_common(const char* name, const void* x, const void* w, int T, int N, int K, int bn) {
  IB_CHECK_ARG(T > 0 && N > 0 && K > 0, "%s: bad sizes T=%d N=%d K=%d", name, T, N, K);
  IB_CHECK_ARG(K % 8 == 0, "%s: K=%d must be a multiple of 8 (TMA needs 16-byte row pitch)", name, K);
  IB_CHECK_ARG(((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0, "%s: operands must be 16-byte aligned", name);
  return 0;
}

}  // namespace

// x [T, K] bfloat16, w [N, K] bfloat16 -> out [splits, T, N] float32. bn: tokens per CTA (16, 32, 64,
// 128 or 256); splits: how many CTAs share one output tile's k-range (each writes its own partial);
// wide != 0: 256 rows of w per CTA (two accumulators) instead of 128, for bn 128 and 256.
extern "C" int ib_gemm_tcgen05(const void* x, const void* w, float* out, int T, int N, int K, int bn, int splits, int wide, unsigned* status,
                               cudaStream_t stream) {
  if (T == 0 || N == 0) return 0;
  if (check_common("gemm_tcgen05", x, w, T, N, K, bn)) return 1;
  const int total_kt = (K + BK - 1) / BK;
  IB_CHECK_ARG(splits >= 1 && splits <= total_kt && splits <= 65535, "gemm_tcgen05: %d splits for %d k-tiles", splits, total_kt);
  const int kt_per_split = (total_kt + splits - 1) / splits;
  IB_CHECK_ARG((splits - 1) * kt_per_split < total_kt, "gemm_tcgen05: %d splits of %d k-tiles leave one empty (%d k-tiles)", splits, kt_per_split,
               total_kt);
  CUtensorMap tw, tx;
  if (make_tmap(&tw, w, N, K, BM)) return 1;
  if (make_tmap(&tx, x, T, K, bn)) return 1;
  if (wide) {
    switch (bn) {
      case 128: return launch<128, 2, EPI_STORE>(tw, tx, out, T, N, K, splits, kt_per_split, BM, status, stream);
      case 256: return launch<256, 2, EPI_STORE>(tw, tx, out, T, N, K, splits, kt_per_split, BM, status, stream);
      default: return ib_set_error("gemm_tcgen05: the wide tile takes token tiles of 128 or 256, not %d", bn);
    }
  }
  switch (bn) {
    case 16: return launch<16, 1, EPI_STORE>(tw, tx, out, T, N, K, splits, kt_per_split, 0, status, stream);
    case 32: return launch<32, 1, EPI_STORE>(tw, tx, out, T, N, K, splits, kt_per_split, 0, status, stream);
    case 64: return launch<64, 1, EPI_STORE>(tw, tx, out, T, N, K, splits, kt_per_split, 0, status, stream);
    case 128: return launch<128, 1, EPI_STORE>(tw, tx, out, T, N, K, splits, kt_per_split, 0, status, stream);
    case 256: return launch<256, 1, EPI_STORE>(tw, tx, out, T, N, K, splits, kt_per_split, 0, status, stream);
    default: return ib_set_error("gemm_tcgen05: token tile %d is not one of 16, 32, 64, 128, 256", bn);
  }
}

// The wait-limit test's entry: ib_gemm_tcgen05 for up to 16 tokens whose copying warp sends nothing. Every wait in the
// kernel then runs out after the limit set with ib_set_wait_limit_ms: the status word gets IB_ERR_WAIT_TIMEOUT, nothing
// is stored, tensor memory is given back and the kernel returns. No copy is in flight at any time.
extern "C" int ib_test_gemm_tcgen05_starved(const void* x, const void* w, float* out, int T, int N, int K, unsigned* status, cudaStream_t stream) {
  if (check_common("test_gemm_tcgen05_starved", x, w, T, N, K, 16)) return 1;
  IB_CHECK_ARG(T <= 16, "test_gemm_tcgen05_starved: up to 16 tokens, got %d", T);
  IB_CHECK_ARG(ib_wait_limit_ns() <= 100000000ull, "test_gemm_tcgen05_starved: set a wait limit of 100 ms or less first (it is %llu ns)", ib_wait_limit_ns());
  const int total_kt = (K + BK - 1) / BK;
  CUtensorMap tw, tx;
  if (make_tmap(&tw, w, N, K, BM)) return 1;
  if (make_tmap(&tx, x, T, K, 16)) return 1;
  return launch<16, 1, EPI_STORE>(tw, tx, out, T, N, K, 1, total_kt, 0, status, stream, 1);
}

// SwiGLU front half in one kernel: w [2*I, K] = gate rows then up rows; act [T, I] bfloat16 =
// silu(x gate^T) * (x up^T). bn: 16 or 32 tokens per CTA, or 64 with half != 0 (64 gate rows and their 64 up rows in one
// accumulator: I must be a multiple of 64), or 64, 128 or 256 (128 gate rows and 128 up rows in two accumulators).
extern "C" int ib_gemm_swiglu_tcgen05(const void* x, const void* w, void* act, int T, int I, int K, int bn, int half, unsigned* status,
                                      cudaStream_t stream) {
  if (T == 0 || I == 0) return 0;
  if (check_common("gemm_swiglu_tcgen05", x, w, T, I, K, bn)) return 1;
  const int total_kt = (K + BK - 1) / BK;
  CUtensorMap tw, tx;
  if (bn == 16 || bn == 32 || (bn == 64 && half)) {
    IB_CHECK_ARG(I % 64 == 0, "gemm_swiglu_tcgen05: with %d tokens per CTA the intermediate size must be a multiple of 64, not %d", bn, I);
    if (make_tmap(&tw, w, 2 * I, K, BM / 2)) return 1;
    if (make_tmap(&tx, x, T, K, bn)) return 1;
    if (bn == 16) return launch<16, 1, EPI_SWIGLU_HALF>(tw, tx, act, T, I, K, 1, total_kt, I, status, stream);
    if (bn == 32) return launch<32, 1, EPI_SWIGLU_HALF>(tw, tx, act, T, I, K, 1, total_kt, I, status, stream);
    return launch<64, 1, EPI_SWIGLU_HALF>(tw, tx, act, T, I, K, 1, total_kt, I, status, stream);
  }
  if (make_tmap(&tw, w, 2 * I, K, BM)) return 1;
  if (make_tmap(&tx, x, T, K, bn)) return 1;
  switch (bn) {
    case 64: return launch<64, 2, EPI_SWIGLU>(tw, tx, act, T, I, K, 1, total_kt, I, status, stream);
    case 128: return launch<128, 2, EPI_SWIGLU>(tw, tx, act, T, I, K, 1, total_kt, I, status, stream);
    case 256: return launch<256, 2, EPI_SWIGLU>(tw, tx, act, T, I, K, 1, total_kt, I, status, stream);
    default: return ib_set_error("gemm_swiglu_tcgen05: token tile %d is not one of 16, 32, 64, 128, 256", bn);
  }
}
