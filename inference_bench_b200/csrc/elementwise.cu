// Row-wise kernels of the decoder: embedding gather, residual add fused with RMSNorm, rotation
// tables, SiLU-mul. All arithmetic is float32; only the stored activation may be bfloat16.
//
// What the reference computes: embed crates/kir/src/prims.rs:387, RMSNorm
// crates/kir/tests/golden/rmsnorm_sm120.cu:19-29, swiglu crates/kir/tests/golden/swiglu_silu.cu:1-11.
#include <stdarg.h>
#include <stdio.h>

#include <type_traits>

#include "common.cuh"

static thread_local char g_error[512] = "";
extern "C" const char* ib_last_error() { return g_error; }
int ib_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return 1;
}

static int g_pdl = 1;
extern "C" int ib_pdl_enabled() { return g_pdl; }
extern "C" void ib_set_pdl(int on) { g_pdl = on ? 1 : 0; }

static unsigned long long g_wait_limit_ns = 2000000000ull;  // 2 s
extern "C" unsigned long long ib_wait_limit_ns() { return g_wait_limit_ns; }
extern "C" void ib_set_wait_limit_ms(int ms) { g_wait_limit_ns = (unsigned long long)(ms > 0 ? ms : 1) * 1000000ull; }

namespace {

// ---------------------------------------------------------------- embedding
template <typename W>
__global__ void embed_kernel(const W* __restrict__ table, const int* __restrict__ tokens, float* __restrict__ x, int H, int V,
                             unsigned* __restrict__ status) {
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  int t = blockIdx.y;
  int tok = tokens[t];
  if (tok < 0 || tok >= V) {
    if (threadIdx.x == 0 && blockIdx.x == 0) atomicOr(status, IB_ERR_BAD_TOKEN);
    tok = 0;
  }
  const W* src = table + (size_t)tok * H;
  float* dst = x + (size_t)t * H;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < H; i += gridDim.x * blockDim.x) dst[i] = ib::to_f32<W>(src[i]);
}

// ---------------------------------------------------------------- residual add + RMSNorm
// One block per output row r. Source row t = rows ? rows[r] : r.
//   v = x[t] + sum_p delta[p][t]   (partials summed in order p = 0..P-1, then added to x)
//   if write_x: x[t] = v
//   out[r] = w * (v * rsqrt(mean(v^2) + eps))
// The row lives in dynamic shared memory (H floats) between the two passes.
// VEC = 4 when H is a multiple of 4 (16-byte loads), else 1.
// Sum of squares of a row, in one fixed order whatever kernel computes it (so a token's norm does not
// depend on how many rows share the launch): float4 number f of the row belongs to thread f % 1024 of
// a block of 1024; a thread adds its float4s in rising order; the 1024 sums are added as 32 warps
// (shuffle tree), then the 32 warp sums (the same tree). sq4 pins the order inside a float4.
__device__ __forceinline__ float sq4(float4 v) { return __fmaf_rn(v.w, v.w, __fmaf_rn(v.z, v.z, __fmaf_rn(v.y, v.y, __fmul_rn(v.x, v.x)))); }

// HELD (a few rows only): every partial sum of a thread's four values is requested before the first is used, so that the
// row costs one trip to memory whatever the number of splits; with more rows the loads of four at a time are the faster
// form (the rows' requests then stand in one another's way, and in the way of the next product's weights).
constexpr int kHeld = 9;

template <typename O, int VEC, bool HELD>
__global__ void __launch_bounds__(1024) add_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ delta, int P, size_t delta_stride,
                                   const float* __restrict__ w, O* __restrict__ out, const int* __restrict__ rows, int H, float eps,
                                   int write_x) {
  extern __shared__ __align__(16) float row[];
  __shared__ float scratch[32];
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int r = blockIdx.x;
  const int t = rows ? rows[r] : r;
  float* xr = x + (size_t)t * H;
  const float* dr = delta + (size_t)t * H;
  float ss = 0.f;
  if constexpr (VEC == 4) {
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      float4 v = *(const float4*)(xr + i);
      if (P > 0) {
        float4 d;
        int p = 1;
        if constexpr (HELD) {
          float4 part[kHeld];
#pragma unroll
          for (int q = 0; q < kHeld; q++)
            if (q < P) part[q] = *(const float4*)(dr + q * delta_stride + i);
          d = part[0];
#pragma unroll
          for (int q = 1; q < kHeld; q++)
            if (q < P) d.x += part[q].x, d.y += part[q].y, d.z += part[q].z, d.w += part[q].w;
          p = P < kHeld ? P : kHeld;
        } else {
          d = *(const float4*)(dr + i);
        }
        for (; !HELD && p + 3 < P; p += 4) {   // four independent loads in flight, added in order
          const float4 a = *(const float4*)(dr + p * delta_stride + i), b = *(const float4*)(dr + (p + 1) * delta_stride + i),
                       c = *(const float4*)(dr + (p + 2) * delta_stride + i), e = *(const float4*)(dr + (p + 3) * delta_stride + i);
          d.x = (((d.x + a.x) + b.x) + c.x) + e.x;
          d.y = (((d.y + a.y) + b.y) + c.y) + e.y;
          d.z = (((d.z + a.z) + b.z) + c.z) + e.z;
          d.w = (((d.w + a.w) + b.w) + c.w) + e.w;
        }
        if (!HELD && p < P) {   // the one to three that are left: requested together as well, added in order
          const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
          const float4 a = *(const float4*)(dr + p * delta_stride + i), b = p + 1 < P ? *(const float4*)(dr + (p + 1) * delta_stride + i) : zero,
                       c = p + 2 < P ? *(const float4*)(dr + (p + 2) * delta_stride + i) : zero;
          d.x += a.x, d.y += a.y, d.z += a.z, d.w += a.w;
          if (p + 1 < P) d.x += b.x, d.y += b.y, d.z += b.z, d.w += b.w;
          if (p + 2 < P) d.x += c.x, d.y += c.y, d.z += c.z, d.w += c.w;
          p = P;
        }
        for (; p < P; p++) {   // (the held form's partial sums beyond what it holds)
          const float4 a = *(const float4*)(dr + p * delta_stride + i);
          d.x += a.x, d.y += a.y, d.z += a.z, d.w += a.w;
        }
        v.x += d.x, v.y += d.y, v.z += d.z, v.w += d.w;
        if (write_x) *(float4*)(xr + i) = v;
      }
      *(float4*)(row + i) = v;
      ss = __fadd_rn(ss, sq4(v));
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float v = xr[i];
      if (P > 0) {
        float d = dr[i];
        for (int p = 1; p < P; p++) d += dr[p * delta_stride + i];
        v += d;
        if (write_x) xr[i] = v;
      }
      row[i] = v;
      ss += v * v;
    }
  }
  ss = ib::block_sum(ss, scratch);   // VEC == 4 runs with 1024 threads: the fixed order
  const float inv = rsqrtf(ss / (float)H + eps);
  O* o = out + (size_t)r * H;
  if constexpr (VEC == 4) {
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      const float4 v = *(const float4*)(row + i), g = *(const float4*)(w + i);
      const float a = g.x * (v.x * inv), b = g.y * (v.y * inv), c = g.z * (v.z * inv), d = g.w * (v.w * inv);
      if constexpr (sizeof(O) == 4) {
        *(float4*)((float*)o + i) = make_float4(a, b, c, d);
      } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        *(uint2*)((__nv_bfloat16*)o + i) = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
      }
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = ib::from_f32<O>(w[i] * (row[i] * inv));
  }
}

// The same for many rows at once (prompt portions): 128 threads per row, the row kept in registers
// (NV float4 per thread, H <= 512 * NV), so that a thread has NV independent loads in flight and
// sixteen rows share an SM; the one-CTA-of-1024-threads form above is the faster one for a few rows.
template <typename O, int NV>
__global__ void __launch_bounds__(128) add_rmsnorm_rows_kernel(float* __restrict__ x, const float* __restrict__ delta, int P, size_t delta_stride,
                                                                const float* __restrict__ w, O* __restrict__ out, const int* __restrict__ rows,
                                                                int H, float eps, int write_x) {
  __shared__ float scratch[32];
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int r = blockIdx.x;
  const int t = rows ? rows[r] : r;
  float* xr = x + (size_t)t * H;
  const float* dr = delta + (size_t)t * H;
  float4 v[NV];
#pragma unroll
  for (int k = 0; k < NV; k++) {
    const int i = (k * 128 + threadIdx.x) * 4;
    v[k] = i < H ? *(const float4*)(xr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (P > 0) {
#pragma unroll
    for (int k = 0; k < NV; k++) {
      const int i = (k * 128 + threadIdx.x) * 4;
      if (i >= H) continue;
      float4 d = *(const float4*)(dr + i);
      for (int p = 1; p < P; p++) {
        const float4 a = *(const float4*)(dr + p * delta_stride + i);
        d.x += a.x, d.y += a.y, d.z += a.z, d.w += a.w;
      }
      v[k].x += d.x, v[k].y += d.y, v[k].z += d.z, v[k].w += d.w;
      if (write_x) *(float4*)(xr + i) = v[k];
    }
  }
  // the fixed order: float4 k * 128 + tid is thread (k % 8) * 128 + tid of the block of 1024, so each of this
  // block's warps holds, for every k < 8, exactly one warp of the 1024
  float part[8];
#pragma unroll
  for (int k = 0; k < 8; k++) {
    part[k] = (k < NV && (k * 128 + threadIdx.x) * 4 < H) ? sq4(v[k < NV ? k : 0]) : 0.f;
    if (k + 8 < NV && ((k + 8) * 128 + threadIdx.x) * 4 < H) part[k] = __fadd_rn(part[k], sq4(v[k + 8 < NV ? k + 8 : 0]));
    part[k] = ib::warp_sum(part[k]);
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) {
#pragma unroll
    for (int k = 0; k < 8; k++) scratch[4 * k + (threadIdx.x >> 5)] = part[k];
  }
  __syncthreads();
  const float ss = ib::warp_sum(scratch[threadIdx.x & 31]);
  const float inv = rsqrtf(ss / (float)H + eps);
  O* o = out + (size_t)r * H;
#pragma unroll
  for (int k = 0; k < NV; k++) {
    const int i = (k * 128 + threadIdx.x) * 4;
    if (i >= H) continue;
    const float4 g = *(const float4*)(w + i);
    const float a = g.x * (v[k].x * inv), b = g.y * (v[k].y * inv), c = g.z * (v[k].z * inv), d = g.w * (v[k].w * inv);
    if constexpr (sizeof(O) == 4) {
      *(float4*)((float*)o + i) = make_float4(a, b, c, d);
    } else {
      __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
      *(uint2*)((__nv_bfloat16*)o + i) = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
    }
  }
}

// ---------------------------------------------------------------- rotation tables
// cos/sin[t][i] of angle = float(position[t]) * inv_freq[i], float32 throughout
// (crates/kir/tests/golden/attention/RopeKvWrite_bf16x2_sm120.cu:32-35).
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq, float* __restrict__ cos_t,
                                  float* __restrict__ sin_t, int T, int half) {
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= T * half) return;
  int t = idx / half, i = idx - t * half;
  float ang = (float)positions[t] * inv_freq[i];
  float s, c;
  sincosf(ang, &s, &c);
  cos_t[idx] = c;
  sin_t[idx] = s;
}

// ---------------------------------------------------------------- SiLU-mul
// gu[p][t][0:I] = gate, gu[p][t][I:2I] = up (partials summed first); act = g / (1 + exp(-g)) * u.
template <typename O>
__global__ void silu_mul_kernel(const float* __restrict__ gu, int P, size_t stride, O* __restrict__ act, int I) {
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  int t = blockIdx.y;
  const float* row = gu + (size_t)t * 2 * I;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < I; i += gridDim.x * blockDim.x) {
    float g = row[i], u = row[I + i];
    for (int p = 1; p < P; p++) {
      g += row[p * stride + i];
      u += row[p * stride + I + i];
    }
    act[(size_t)t * I + i] = ib::from_f32<O>((g / (1.f + expf(-g))) * u);
  }
}

}  // namespace

extern "C" int ib_embed(const void* table, int table_dtype, const int* tokens, float* x, int T, int H, int V, unsigned* status,
                        cudaStream_t stream) {
  if (T == 0) return 0;
  IB_CHECK_ARG(T > 0 && H > 0 && V > 0, "embed: bad sizes T=%d H=%d V=%d", T, H, V);
  IB_CHECK_ARG(T <= 65535, "embed: T=%d rows exceed the grid limit 65535", T);
  dim3 grid((H + 255) / 256, T);
  if (table_dtype == IB_F32)
    ib::launch(embed_kernel<float>, grid, 256, 0, stream, (const float*)table, tokens, x, H, V, status);
  else if (table_dtype == IB_BF16)
    ib::launch(embed_kernel<__nv_bfloat16>, grid, 256, 0, stream, (const __nv_bfloat16*)table, tokens, x, H, V, status);
  else
    return ib_set_error("embed: unknown table dtype %d", table_dtype);
  IB_CHECK_LAUNCH("embed");
  return 0;
}

extern "C" int ib_add_rmsnorm(float* x, const float* delta, int P, long long delta_stride, const float* w, void* out, int out_dtype,
                              const int* rows, int n_rows, int H, float eps, int write_x, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  IB_CHECK_ARG(n_rows > 0 && H > 0 && P >= 0, "add_rmsnorm: bad sizes rows=%d H=%d P=%d", n_rows, H, P);
  IB_CHECK_ARG(!(rows && write_x), "add_rmsnorm: a gathered call must not write x back");
  size_t smem = (size_t)H * sizeof(float);
  IB_CHECK_ARG(smem <= 200 * 1024, "add_rmsnorm: hidden size %d needs %zu bytes of shared memory, more than 200 KiB", H, smem);
  const bool vec = H % 4 == 0 && ((uintptr_t)x % 16 == 0) && (!delta || (uintptr_t)delta % 16 == 0) && ((uintptr_t)w % 16 == 0) &&
                   ((uintptr_t)out % 16 == 0) && (delta_stride % 4 == 0);
  if (vec && n_rows >= 256 && H <= 8192) {   // many rows: the register form
    auto go_rows = [&](auto* o) {
      using O = std::remove_pointer_t<decltype(o)>;
      const int nv = (H + 511) / 512;
      if (nv <= 1) ib::launch(add_rmsnorm_rows_kernel<O, 1>, n_rows, 128, 0, stream, x, delta, P, (size_t)delta_stride, w, o, rows, H, eps, write_x);
      else if (nv <= 2) ib::launch(add_rmsnorm_rows_kernel<O, 2>, n_rows, 128, 0, stream, x, delta, P, (size_t)delta_stride, w, o, rows, H, eps, write_x);
      else if (nv <= 4) ib::launch(add_rmsnorm_rows_kernel<O, 4>, n_rows, 128, 0, stream, x, delta, P, (size_t)delta_stride, w, o, rows, H, eps, write_x);
      else if (nv <= 8) ib::launch(add_rmsnorm_rows_kernel<O, 8>, n_rows, 128, 0, stream, x, delta, P, (size_t)delta_stride, w, o, rows, H, eps, write_x);
      else ib::launch(add_rmsnorm_rows_kernel<O, 16>, n_rows, 128, 0, stream, x, delta, P, (size_t)delta_stride, w, o, rows, H, eps, write_x);
    };
    if (out_dtype == IB_F32) go_rows((float*)out);
    else if (out_dtype == IB_BF16) go_rows((__nv_bfloat16*)out);
    else return ib_set_error("add_rmsnorm: unknown output dtype %d", out_dtype);
    IB_CHECK_LAUNCH("add_rmsnorm");
    return 0;
  }
  constexpr int kFewRows = 4;   // up to here the form that requests every partial sum at once (measured: faster for 1 to 4 rows)
  int threads = vec ? 1024 : (H >= 1024 ? 1024 : (H >= 512 ? 512 : (H >= 256 ? 256 : 128)));   // 16-byte form: always 1024, the fixed summation order
  auto go = [&](auto kernel, auto* o) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ib::launch(kernel, n_rows, threads, smem, stream, x, delta, P, (size_t)delta_stride, w, o, rows, H, eps, write_x);
  };
  if (out_dtype == IB_F32) {
    if (vec) go(add_rmsnorm_kernel<float, 4, false>, (float*)out);
    else go(add_rmsnorm_kernel<float, 1, false>, (float*)out);
  } else if (out_dtype == IB_BF16) {
    if (vec && n_rows <= kFewRows) go(add_rmsnorm_kernel<__nv_bfloat16, 4, true>, (__nv_bfloat16*)out);
    else if (vec) go(add_rmsnorm_kernel<__nv_bfloat16, 4, false>, (__nv_bfloat16*)out);
    else go(add_rmsnorm_kernel<__nv_bfloat16, 1, false>, (__nv_bfloat16*)out);
  } else {
    return ib_set_error("add_rmsnorm: unknown output dtype %d", out_dtype);
  }
  IB_CHECK_LAUNCH("add_rmsnorm");
  return 0;
}

extern "C" int ib_rope_table(const int* positions, const float* inv_freq, float* cos_t, float* sin_t, int T, int half,
                             cudaStream_t stream) {
  if (T == 0 || half == 0) return 0;
  IB_CHECK_ARG(T > 0 && half > 0, "rope_table: bad sizes T=%d half=%d", T, half);
  long long n = (long long)T * half;
  ib::launch(rope_table_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, positions, inv_freq, cos_t, sin_t, T, half);
  IB_CHECK_LAUNCH("rope_table");
  return 0;
}

extern "C" int ib_silu_mul(const float* gu, int P, long long stride, void* act, int act_dtype, int T, int I, cudaStream_t stream) {
  if (T == 0) return 0;
  IB_CHECK_ARG(T > 0 && I > 0 && P >= 1, "silu_mul: bad sizes T=%d I=%d P=%d", T, I, P);
  IB_CHECK_ARG(T <= 65535, "silu_mul: T=%d rows exceed the grid limit 65535", T);
  dim3 grid((I + 255) / 256, T);
  if (grid.x > 64) grid.x = 64;
  if (act_dtype == IB_F32)
    ib::launch(silu_mul_kernel<float>, grid, 256, 0, stream, gu, P, (size_t)stride, (float*)act, I);
  else if (act_dtype == IB_BF16)
    ib::launch(silu_mul_kernel<__nv_bfloat16>, grid, 256, 0, stream, gu, P, (size_t)stride, (__nv_bfloat16*)act, I);
  else
    return ib_set_error("silu_mul: unknown output dtype %d", act_dtype);
  IB_CHECK_LAUNCH("silu_mul");
  return 0;
}
