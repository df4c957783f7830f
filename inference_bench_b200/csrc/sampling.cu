// Next-token choice on the device, one block per logits row.
//
// Temperature 0: argmax, the lowest index winning ties. Otherwise Gumbel-max over the candidates
// that survive top-k, top-p and min-p, on v = logit / T: token = argmax_i (v_i + g_i),
// g_i = -ln(-ln u_i), u_i from an integer hash of (seed, step, i). Same semantics and the same
// hash as the reference's sample_rows (crates/kir/tests/golden/prims/prims_sm120.cu:34-39,
// 51-163, 208-250); the threshold search here is a byte-wise radix descent for top-k and a
// bisection with ordered block sums for top-p, so a row's result never depends on thread timing.
#include "common.cuh"

namespace {

constexpr int kThreads = 1024;

struct RowParams {  // six 32-bit words per row, as the reference packs them (crates/specrt/src/runtime/step.rs:76-85)
  float inv_temp;   // 0 = greedy
  unsigned seed;
  unsigned step;
  int top_k;    // 0 = off
  float top_p;  // 1 = off
  float min_p;  // 0 = off
};

__device__ __forceinline__ float gumbel(unsigned seed, unsigned step, unsigned i) {
  unsigned x = seed * 747796405u + step * 2891336453u + i * 2246822519u + 1u;
  x ^= x >> 16;
  x *= 2246822507u;
  x ^= x >> 13;
  x *= 3266489909u;
  x ^= x >> 16;
  float u = ((float)(x >> 8) + 0.5f) / 16777216.0f;
  return -logf(-logf(u));
}

// Monotone map float -> unsigned (larger float, larger key).
__device__ __forceinline__ unsigned order_key(float v) {
  unsigned b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float order_value(unsigned k) { return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k); }

__device__ float block_max(float v, float* scratch) {
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = ib::warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = lane < (blockDim.x >> 5) ? scratch[lane] : -INFINITY;
  return ib::warp_max(r);
}

// The k-th largest value of v_i = row[i] * inv_temp, by four passes over one byte of the key each.
__device__ float kth_largest(const float* row, int V, float inv_temp, int k) {
  __shared__ unsigned hist[256];
  __shared__ unsigned sh_prefix;
  __shared__ int sh_need;
  unsigned prefix = 0, mask = 0;
  int need = k;
  for (int pass = 0; pass < 4; pass++) {
    int shift = 24 - 8 * pass;
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      unsigned key = order_key(row[i] * inv_temp);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int c = need, b = 255;
      for (; b > 0; b--) {
        if ((int)hist[b] >= c) break;
        c -= (int)hist[b];
      }
      sh_need = c;
      sh_prefix = prefix | ((unsigned)b << shift);
    }
    __syncthreads();
    need = sh_need;
    prefix = sh_prefix;
    mask |= 255u << shift;
    __syncthreads();
  }
  return order_value(prefix);
}

__device__ float mass_at_least(const float* row, int V, float inv_temp, float m, float floor_v, float* scratch) {
  float z = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    float v = row[i] * inv_temp;
    if (v >= floor_v) z += expf(v - m);
  }
  return ib::block_sum(z, scratch);
}

// Stage 1, one block per row: the candidate threshold on v = logit / T. Rows that are greedy or
// have no filter leave at once with -inf.
__global__ void __launch_bounds__(kThreads) sample_threshold_kernel(const float* __restrict__ logits, int V, const RowParams* __restrict__ params,
                                                                    float* __restrict__ threshold) {
  __shared__ float scratch[32];
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const float* row = logits + (size_t)blockIdx.x * V;
  const RowParams p = params[blockIdx.x];
  const bool use_k = p.top_k > 0 && p.top_k < V, use_p = p.top_p < 1.f, use_m = p.min_p > 0.f;
  if (!(p.inv_temp > 0.f) || !(use_k || use_p || use_m)) {
    if (threadIdx.x == 0) threshold[blockIdx.x] = -INFINITY;
    return;
  }
  float thr = -INFINITY;
  float m = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) m = fmaxf(m, row[i] * p.inv_temp);
  m = block_max(m, scratch);
  if (use_k) thr = kth_largest(row, V, p.inv_temp, p.top_k);
  if (use_p) {
    // Largest threshold whose candidates (also above the top-k threshold) hold mass >= top_p * total.
    float z = mass_at_least(row, V, p.inv_temp, m, thr, scratch);
    float target = fmaxf(p.top_p, 1e-9f) * z;
    float lo = thr > -INFINITY ? thr : m - 88.f;
    float hi = nextafterf(m, INFINITY);
    for (int it = 0; it < 64; it++) {
      float mid = 0.5f * (lo + hi);
      if (mid <= lo || mid >= hi) break;
      if (mass_at_least(row, V, p.inv_temp, m, mid, scratch) >= target)
        lo = mid;
      else
        hi = mid;
    }
    // Snap to the smallest candidate value >= lo.
    float low = INFINITY;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      float v = row[i] * p.inv_temp;
      if (v >= lo) low = fminf(low, v);
    }
    low = -block_max(-low, scratch);
    thr = fmaxf(thr, low);
  }
  if (use_m) thr = fmaxf(thr, m + logf(p.min_p));
  if (threadIdx.x == 0) threshold[blockIdx.x] = thr;
}

__device__ __forceinline__ void better(float& bv, int& bi, float ov, int oi) {  // the lowest index wins ties
  if (ov > bv || (ov == bv && oi < bi)) {
    bv = ov;
    bi = oi;
  }
}

// Best (value, index) of a block of kPickThreads threads; valid in thread 0.
constexpr int kPickThreads = 256;
__device__ void block_best(float& bv, int& bi) {
  __shared__ float sv[kPickThreads / 32];
  __shared__ int si[kPickThreads / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) better(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
  if (lane == 0) {
    sv[warp] = bv;
    si[warp] = bi;
  }
  __syncthreads();
  if (warp == 0) {
    bv = lane < kPickThreads / 32 ? sv[lane] : -INFINITY;
    bi = lane < kPickThreads / 32 ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) better(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
  }
}

// Stage 2, grid (chunks, rows): the best candidate of one chunk of the vocabulary.
__global__ void __launch_bounds__(kPickThreads) sample_pick_kernel(const float* __restrict__ logits, int V, const RowParams* __restrict__ params,
                                                                   const float* __restrict__ threshold, float* __restrict__ part_v,
                                                                   int* __restrict__ part_i, int chunk) {
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int r = blockIdx.y;
  const float* row = logits + (size_t)r * V;
  const RowParams p = params[r];
  const bool sampling = p.inv_temp > 0.f;
  const float thr = threshold[r];
  const int begin = blockIdx.x * chunk, end = min(V, begin + chunk);
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = begin + threadIdx.x; i < end; i += kPickThreads) {
    float v = row[i];
    if (sampling) {
      v *= p.inv_temp;
      if (v < thr) continue;
      v += gumbel(p.seed, p.step, (unsigned)i);
    }
    better(bv, bi, v, i);
  }
  block_best(bv, bi);
  if (threadIdx.x == 0) {
    part_v[r * gridDim.x + blockIdx.x] = bv;
    part_i[r * gridDim.x + blockIdx.x] = bi;
  }
}

// Stage 3, one warp per row: the best of the chunks.
// With `status` the step's status word is copied to tokens[gridDim.x], so the host gets it in the transfer that brings the tokens.
__global__ void sample_final_kernel(const float* __restrict__ part_v, const int* __restrict__ part_i, int chunks, int* __restrict__ tokens,
                                    const unsigned* __restrict__ status) {
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int r = blockIdx.x;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int c = threadIdx.x; c < chunks; c += 32) better(bv, bi, part_v[r * chunks + c], part_i[r * chunks + c]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) better(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
  if (threadIdx.x == 0) tokens[r] = bi == 0x7fffffff ? 0 : bi;
  if (status && r == 0 && threadIdx.x == 0) tokens[gridDim.x] = (int)*status;
}

// After a decode step: feed every row's sampled token back as its next input, move its position on
// by one, count its sampling step, and log the token. With this at the end of a captured decode
// step the graph can be replayed many times with no host work in between; the host reads the log
// afterwards (the reference's argmax_advance does the same for one row:
// crates/kir/tests/golden/prims/prims_sm120.cu:252-294).
__global__ void advance_rows_kernel(const int* __restrict__ sampled, int* __restrict__ token_in, int* __restrict__ positions,
                                    int* __restrict__ pos0, RowParams* __restrict__ params, int* __restrict__ history, int* __restrict__ count,
                                    int rows, int history_len) {
  // No early launch of the kernels that follow: the attention kernels of the next step read
  // `positions` before their own dependency wait, so nothing of the next step may start before
  // the rows are written. The next kernel starts when this one has finished.
  ib::pdl_wait();
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  int c = count[0];
  if (i < rows) {
    int tok = sampled[i];
    token_in[i] = tok;
    positions[i] += 1;
    pos0[i] += 1;
    params[i].step += 1;
    if (c < history_len) history[(size_t)c * rows + i] = tok;
  }
  __syncthreads();
  if (i == 0) count[0] = c + 1;
}

}  // namespace

extern "C" int ib_advance_rows(const int* sampled, int* token_in, int* positions, int* pos0, void* params, int* history, int* count, int rows,
                               int history_len, cudaStream_t stream) {
  if (rows == 0) return 0;
  IB_CHECK_ARG(rows > 0 && rows <= 1024 && history_len >= 0, "advance_rows: bad sizes rows=%d history=%d", rows, history_len);
  ib::launch(advance_rows_kernel, 1, 1024, 0, stream, sampled, token_in, positions, pos0, (RowParams*)params, history, count, rows, history_len);
  IB_CHECK_LAUNCH("advance_rows");
  return 0;
}

// chunks of the vocabulary per row in stage 2
extern "C" int ib_sample_chunks(int V) { return V <= 4096 ? 1 : (V + 4095) / 4096 > 64 ? 64 : (V + 4095) / 4096; }

// logits float32 [rows, V], params [rows] of six words -> tokens int32 [rows].
// scratch: float32 [rows * (1 + 2 * ib_sample_chunks(V))] (threshold, then per-chunk best values and indices).
// status: null, or the device status word, whose value is then stored in tokens[rows] (tokens has rows + 1 entries).
extern "C" int ib_sample_rows(const float* logits, int rows, int V, const void* params, int* tokens, float* scratch, const unsigned* status,
                              cudaStream_t stream) {
  if (rows == 0) return 0;
  IB_CHECK_ARG(rows > 0 && rows <= 65535 && V > 0, "sample_rows: bad sizes rows=%d V=%d", rows, V);
  const int chunks = ib_sample_chunks(V);
  const int chunk = (V + chunks - 1) / chunks;
  float* threshold = scratch;
  float* part_v = scratch + rows;
  int* part_i = (int*)(part_v + (size_t)rows * chunks);
  ib::launch(sample_threshold_kernel, rows, kThreads, 0, stream, logits, V, (const RowParams*)params, threshold);
  IB_CHECK_LAUNCH("sample_rows threshold");
  ib::launch(sample_pick_kernel, dim3(chunks, rows), kPickThreads, 0, stream, logits, V, (const RowParams*)params, threshold, part_v, part_i, chunk);
  IB_CHECK_LAUNCH("sample_rows pick");
  ib::launch(sample_final_kernel, rows, 32, 0, stream, part_v, part_i, chunks, tokens, status);
  IB_CHECK_LAUNCH("sample_rows final");
  return 0;
}
