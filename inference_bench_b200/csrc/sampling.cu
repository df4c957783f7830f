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

__global__ void __launch_bounds__(kThreads) sample_rows_kernel(const float* __restrict__ logits, int V, const RowParams* __restrict__ params,
                                                               int* __restrict__ tokens) {
  __shared__ float scratch[32];
  __shared__ float best_v[kThreads / 32];
  __shared__ int best_i[kThreads / 32];
  const float* row = logits + (size_t)blockIdx.x * V;
  const RowParams p = params[blockIdx.x];
  const bool sampling = p.inv_temp > 0.f;
  float thr = -INFINITY;
  if (sampling) {
    float m = -INFINITY;
    for (int i = threadIdx.x; i < V; i += blockDim.x) m = fmaxf(m, row[i] * p.inv_temp);
    m = block_max(m, scratch);
    if (p.top_k > 0 && p.top_k < V) thr = kth_largest(row, V, p.inv_temp, p.top_k);
    if (p.top_p < 1.f) {
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
    if (p.min_p > 0.f) thr = fmaxf(thr, m + logf(p.min_p));
  }
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    float v = row[i];
    if (sampling) {
      v *= p.inv_temp;
      if (v < thr) continue;
      v += gumbel(p.seed, p.step, (unsigned)i);
    }
    if (v > bv || (v == bv && i < bi)) {
      bv = v;
      bi = i;
    }
  }
  // Reduce (value, index) with the lowest index winning ties.
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) {
      bv = ov;
      bi = oi;
    }
  }
  __syncthreads();
  if (lane == 0) {
    best_v[warp] = bv;
    best_i[warp] = bi;
  }
  __syncthreads();
  if (warp == 0) {
    bv = lane < (blockDim.x >> 5) ? best_v[lane] : -INFINITY;
    bi = lane < (blockDim.x >> 5) ? best_i[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    if (lane == 0) tokens[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
  }
}

// After a decode step: feed every row's sampled token back as its next input, move its position on
// by one, count its sampling step, and log the token. With this at the end of a captured decode
// step the graph can be replayed many times with no host work in between; the host reads the log
// afterwards (the reference's argmax_advance does the same for one row:
// crates/kir/tests/golden/prims/prims_sm120.cu:252-294).
__global__ void advance_rows_kernel(const int* __restrict__ sampled, int* __restrict__ token_in, int* __restrict__ positions,
                                    int* __restrict__ pos0, RowParams* __restrict__ params, int* __restrict__ history, int* __restrict__ count,
                                    int rows, int history_len) {
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
  advance_rows_kernel<<<1, 1024, 0, stream>>>(sampled, token_in, positions, pos0, (RowParams*)params, history, count, rows, history_len);
  IB_CHECK_LAUNCH("advance_rows");
  return 0;
}

extern "C" int ib_sample_rows(const float* logits, int rows, int V, const void* params, int* tokens, cudaStream_t stream) {
  if (rows == 0) return 0;
  IB_CHECK_ARG(rows > 0 && V > 0, "sample_rows: bad sizes rows=%d V=%d", rows, V);
  sample_rows_kernel<<<rows, kThreads, 0, stream>>>(logits, V, (const RowParams*)params, tokens);
  IB_CHECK_LAUNCH("sample_rows");
  return 0;
}
