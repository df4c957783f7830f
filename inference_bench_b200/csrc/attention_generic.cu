// Generic attention kernels: any head size (even, up to 256), any number of heads and groups, any
// page size; float32 or bfloat16 storage with float32 arithmetic. They serve the float32 path of
// the whole model and every bfloat16 shape that has no tensor-core specialisation.
//
//  * qk_norm_rope_kv: sums the split-K partials of the qkv projection, applies the per-head RMSNorm
//    to q and k, rotates them, writes q out and k/v into the paged cache
//    (reference: crates/kir/src/cuda/attention/common.rs:49-96, rope.rs:13-23).
//  * attention_generic: one warp per (token, query head); online softmax over the keys that the
//    token may see (causal, optional window), read through the block table. Prefill portions and
//    decoded tokens are the same case here: a token at position p reads keys lo..p
//    (mask: crates/kir/src/cuda/attention/flash_mma.rs:193).
#include <type_traits>

#include "kv_view.cuh"

namespace {

constexpr int kWarps = 4;
constexpr int kMaxHeadDim = 256;

template <typename A, typename C>
__global__ void qk_norm_rope_kv_kernel(const float* __restrict__ qkv, int P, size_t stride_p, const float* __restrict__ q_norm_w,
                                       const float* __restrict__ k_norm_w, float eps, const float* __restrict__ cos_t,
                                       const float* __restrict__ sin_t, int rot_half, const int* __restrict__ positions,
                                       const int* __restrict__ seg_of_token, A* __restrict__ q_out, IbKvView kv, int write_kv, int T,
                                       int heads, unsigned* __restrict__ status) {
  __shared__ float vec[kWarps][kMaxHeadDim];
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int hd = kv.head_dim, kvh = kv.kv_heads;
  const int slots = heads + 2 * kvh;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  long long item = (long long)blockIdx.x * kWarps + warp;
  if (item >= (long long)T * slots) return;
  const int t = (int)(item / slots), j = (int)(item % slots);
  const int R = slots * hd;
  const bool is_q = j < heads, is_k = !is_q && j < heads + kvh;
  if (!is_q && !write_kv) return;
  const float* src = qkv + (size_t)t * R + (size_t)j * hd;
  float* v = vec[warp];
  float ss = 0.f;
  for (int d = lane; d < hd; d += 32) {
    float a = src[d];
    for (int p = 1; p < P; p++) a += src[p * stride_p + d];
    v[d] = a;
    ss += a * a;
  }
  __syncwarp();
  const float* nw = is_q ? q_norm_w : (is_k ? k_norm_w : nullptr);
  if (nw) {
    ss = ib::warp_sum(ss);
    float inv = rsqrtf(ss / (float)hd + eps);
    for (int d = lane; d < hd; d += 32) v[d] = nw[d] * (v[d] * inv);
    __syncwarp();
  }
  if ((is_q || is_k) && cos_t && rot_half > 0) {
    // Half rotation over the first 2*rot_half dims: pair (d, d + rot_half).
    for (int d = lane; d < rot_half; d += 32) {
      float c = cos_t[(size_t)t * rot_half + d], s = sin_t[(size_t)t * rot_half + d];
      float a = v[d], b = v[d + rot_half];
      v[d] = a * c - b * s;
      v[d + rot_half] = b * c + a * s;
    }
    __syncwarp();
  }
  if (is_q) {
    A* dst = q_out + (size_t)t * heads * hd + (size_t)j * hd;
    for (int d = lane; d < hd; d += 32) dst[d] = ib::from_f32<A>(v[d]);
    return;
  }
  const int head = is_k ? j - heads : j - heads - kvh;
  long long off = ib::kv_offset(kv, seg_of_token[t], positions[t], head);
  if (off < 0) {
    if (lane == 0) atomicOr(status, IB_ERR_BAD_PAGE);
    return;
  }
  C* dst = (C*)kv.base + off + (is_k ? 0 : kv.v_offset);
  for (int d = lane; d < hd; d += 32) dst[d] = ib::from_f32<C>(v[d]);
}

// The same for head sizes 64 and 128 with the whole head rotated (or none of it): a lane holds
// HD/32 consecutive values, so loads and stores are 8 or 16 bytes wide, the norm is one warp sum,
// and the rotation partner (d + HD/2) sits in lane ^ 16.
template <int HD, typename A, typename C, int PER>
__global__ void qk_norm_rope_kv_vec_kernel(const float* __restrict__ qkv, int P, size_t stride_p, const float* __restrict__ q_norm_w,
                                           const float* __restrict__ k_norm_w, float eps, const float* __restrict__ cos_t,
                                           const float* __restrict__ sin_t, const int* __restrict__ positions,
                                           const int* __restrict__ seg_of_token, A* __restrict__ q_out, IbKvView kv, int write_kv, int T,
                                           int heads, unsigned* __restrict__ status) {
  // blockIdx.x is the token; a warp takes PER consecutive heads of it (q heads, then k heads, then v heads)
  // and loads them all before it works on any: with many tokens (PER = 4) that keeps four loads per lane
  // in flight; with few, PER = 1 keeps the chain short. No division anywhere: this kernel is bound by
  // its instruction count as much as by memory.
  constexpr int E = HD / 32;
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int kvh = kv.kv_heads, slots = heads + 2 * kvh;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int j0 = (blockIdx.y * kWarps + warp) * PER;
  // what every head of the token shares, fetched once per warp with wide loads and requested before the partial products
  // (one trip to memory for all of it, not one after the other): norm scales, the token's
  // rotation (the sine with the sign of this lane's half: d < HD/2: v cos - partner sin; d >= HD/2: v cos + partner sin)
  float qw[E], kw[E], cs[E], sn[E];
  auto load_vec = [&](const float* src, float (&dst)[E]) {
    if constexpr (E == 4) {
      const float4 a = *(const float4*)src;
      dst[0] = a.x, dst[1] = a.y, dst[2] = a.z, dst[3] = a.w;
    } else {
      const float2 a = *(const float2*)src;
      dst[0] = a.x, dst[1] = a.y;
    }
  };
  if (q_norm_w) load_vec(q_norm_w + lane * E, qw);
  if (k_norm_w) load_vec(k_norm_w + lane * E, kw);
  if (cos_t) {
    load_vec(cos_t + (size_t)t * (HD / 2) + (lane & 15) * E, cs);
    load_vec(sin_t + (size_t)t * (HD / 2) + (lane & 15) * E, sn);
  }
  float v[PER][E];
#pragma unroll
  for (int u = 0; u < PER; u++) {
#pragma unroll
    for (int e = 0; e < E; e++) v[u][e] = 0.f;
    const int j = j0 + u;
    if (j >= slots || (j >= heads && !write_kv)) continue;
    const float* src = qkv + (size_t)t * slots * HD + (size_t)j * HD + lane * E;
    for (int p = 0; p < P; p++) {
      if constexpr (E == 4) {
        const float4 a = *(const float4*)(src + p * stride_p);
        v[u][0] += a.x, v[u][1] += a.y, v[u][2] += a.z, v[u][3] += a.w;
      } else {
        const float2 a = *(const float2*)(src + p * stride_p);
        v[u][0] += a.x, v[u][1] += a.y;
      }
    }
  }
  if (cos_t && lane < 16) {   // (used only now, so that nothing waited for it above)
#pragma unroll
    for (int e = 0; e < E; e++) sn[e] = -sn[e];
  }
#pragma unroll
  for (int u = 0; u < PER; u++) {
    const int j = j0 + u;
    if (j >= slots) continue;
    const bool is_q = j < heads, is_k = !is_q && j < heads + kvh;
    if (!is_q && !write_kv) continue;
    if (is_q ? q_norm_w != nullptr : (is_k && k_norm_w != nullptr)) {
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < E; e++) ss += v[u][e] * v[u][e];
      ss = ib::warp_sum(ss);
      const float inv = rsqrtf(ss / (float)HD + eps);
#pragma unroll
      for (int e = 0; e < E; e++) v[u][e] = (is_q ? qw[e] : kw[e]) * (v[u][e] * inv);
    }
    if ((is_q || is_k) && cos_t) {
#pragma unroll
      for (int e = 0; e < E; e++) {
        const float other = __shfl_xor_sync(0xffffffffu, v[u][e], 16);
        v[u][e] = __fmaf_rn(other, sn[e], __fmul_rn(v[u][e], cs[e]));
      }
    }
    auto store = [&](auto* dst) {
      using D = std::remove_pointer_t<decltype(dst)>;
      if constexpr (sizeof(D) == 4) {
        if constexpr (E == 4) *(float4*)dst = make_float4(v[u][0], v[u][1], v[u][2], v[u][3]);
        else *(float2*)dst = make_float2(v[u][0], v[u][1]);
      } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(v[u][0], v[u][1]);
        if constexpr (E == 4) {
          __nv_bfloat162 hi = __floats2bfloat162_rn(v[u][2], v[u][3]);
          *(uint2*)dst = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
        } else {
          *(uint32_t*)dst = *(uint32_t*)&lo;
        }
      }
    };
    if (is_q) {
      store(q_out + (size_t)t * heads * HD + (size_t)j * HD + lane * E);
      continue;
    }
    const int head = is_k ? j - heads : j - heads - kvh;
    const long long off = ib::kv_offset(kv, seg_of_token[t], positions[t], head);
    if (off < 0) {
      if (lane == 0) atomicOr(status, IB_ERR_BAD_PAGE);
      continue;
    }
    store((C*)kv.base + off + (is_k ? 0 : kv.v_offset) + lane * E);
  }
}

// acc registers: lane owns dims lane, lane+32, ... (up to 8 for head_dim 256).
template <typename A, typename C>
__global__ void attention_generic_kernel(const A* __restrict__ q, IbKvView kv, const int* __restrict__ positions,
                                         const int* __restrict__ seg_of_token, int window, float scale, A* __restrict__ out, int T,
                                         int heads, unsigned* __restrict__ status) {
  __shared__ float qs[kWarps][kMaxHeadDim];
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int hd = kv.head_dim;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  long long item = (long long)blockIdx.x * kWarps + warp;
  if (item >= (long long)T * heads) return;
  const int t = (int)(item / heads), h = (int)(item % heads);
  const int kvhead = h / (heads / kv.kv_heads);
  const int pos = positions[t], seg = seg_of_token[t];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const A* qrow = q + (size_t)t * heads * hd + (size_t)h * hd;
  for (int d = lane; d < hd; d += 32) qs[warp][d] = ib::to_f32<A>(qrow[d]);
  __syncwarp();
  float acc[kMaxHeadDim / 32];
#pragma unroll
  for (int r = 0; r < kMaxHeadDim / 32; r++) acc[r] = 0.f;
  float m = -INFINITY, l = 0.f;
  const C* base = (const C*)kv.base;
  for (int k0 = lo; k0 <= pos; k0 += 32) {
    int key = k0 + lane;
    long long off = -1;
    float s = -INFINITY;
    if (key <= pos) {
      off = ib::kv_offset(kv, seg, key, kvhead);
      if (off < 0) {
        atomicOr(status, IB_ERR_BAD_PAGE);
      } else {
        const C* kr = base + off;
        float dot = 0.f;
        for (int d = 0; d < hd; d++) dot += qs[warp][d] * ib::to_f32<C>(kr[d]);
        s = dot * scale;
      }
    }
    float m_new = fmaxf(m, ib::warp_max(s));
    if (m_new == -INFINITY) continue;  // every key of this chunk was unreadable
    float corr = expf(m - m_new);
    float p = s == -INFINITY ? 0.f : expf(s - m_new);
    l = l * corr + ib::warp_sum(p);
#pragma unroll
    for (int r = 0; r < kMaxHeadDim / 32; r++) acc[r] *= corr;
    int n = min(32, pos - k0 + 1);
    for (int jj = 0; jj < n; jj++) {
      float pj = __shfl_sync(0xffffffffu, p, jj);
      long long oj = __shfl_sync(0xffffffffu, off, jj);
      if (oj < 0) continue;
      const C* vr = base + oj + kv.v_offset;
#pragma unroll
      for (int r = 0; r < kMaxHeadDim / 32; r++) {
        int d = lane + 32 * r;
        if (d < hd) acc[r] += pj * ib::to_f32<C>(vr[d]);
      }
    }
    m = m_new;
  }
  float inv = l > 0.f ? 1.f / l : 0.f;
  A* orow = out + (size_t)t * heads * hd + (size_t)h * hd;
#pragma unroll
  for (int r = 0; r < kMaxHeadDim / 32; r++) {
    int d = lane + 32 * r;
    if (d < hd) orow[d] = ib::from_f32<A>(acc[r] * inv);
  }
}

int check_view(const char* name, const IbKvView* kv, int heads) {
  IB_CHECK_ARG(kv && kv->base && kv->block_table, "%s: the cache view has a null pointer", name);
  IB_CHECK_ARG(kv->head_dim > 0 && kv->head_dim <= kMaxHeadDim && kv->head_dim % 2 == 0,
               "%s: head_dim %d is not supported (even sizes up to %d)", name, kv->head_dim, kMaxHeadDim);
  IB_CHECK_ARG(kv->kv_heads > 0 && heads > 0 && heads % kv->kv_heads == 0, "%s: %d query heads are not a multiple of %d kv heads", name,
               heads, kv->kv_heads);
  IB_CHECK_ARG(kv->page_size > 0 && kv->num_pages > 0 && kv->table_stride > 0, "%s: bad page geometry", name);
  IB_CHECK_ARG(kv->dtype == IB_F32 || kv->dtype == IB_BF16, "%s: unknown cache dtype %d", name, kv->dtype);
  return 0;
}

}  // namespace

extern "C" int ib_qk_norm_rope_kv(const float* qkv, int P, long long stride_p, const float* q_norm_w, const float* k_norm_w, float eps,
                                  const float* cos_t, const float* sin_t, int rot_half, const int* positions, const int* seg_of_token,
                                  void* q_out, int act_dtype, const IbKvView* kv, int write_kv, int T, int heads, unsigned* status,
                                  cudaStream_t stream) {
  if (T == 0) return 0;
  if (check_view("qk_norm_rope_kv", kv, heads)) return 1;
  IB_CHECK_ARG(P >= 1 && T > 0, "qk_norm_rope_kv: bad sizes T=%d P=%d", T, P);
  IB_CHECK_ARG(rot_half >= 0 && 2 * rot_half <= kv->head_dim, "qk_norm_rope_kv: rotary size %d exceeds head_dim %d", 2 * rot_half,
               kv->head_dim);
  IB_CHECK_ARG((act_dtype == IB_F32 && kv->dtype == IB_F32) || (act_dtype == IB_BF16 && kv->dtype == IB_BF16),
               "qk_norm_rope_kv: activation dtype %d and cache dtype %d must match", act_dtype, kv->dtype);
  long long items = (long long)T * (heads + 2 * kv->kv_heads);
  unsigned blocks = (unsigned)((items + kWarps - 1) / kWarps);
  const int hd = kv->head_dim;
  const bool aligned = ((uintptr_t)qkv % 16 == 0) && (stride_p % 4 == 0) && ((uintptr_t)q_out % 16 == 0) && ((uintptr_t)kv->base % 16 == 0);
  const bool vec = (hd == 64 || hd == 128) && (rot_half == 0 || 2 * rot_half == hd) && aligned;
  const float* cs = rot_half ? cos_t : nullptr;
  if (vec) {
    const int slots = heads + 2 * kv->kv_heads;
    auto go = [&](auto kernel, int per, auto* qo) {
      const dim3 grid((unsigned)T, (unsigned)((slots + kWarps * per - 1) / (kWarps * per)));
      ib::launch(kernel, grid, kWarps * 32, 0, stream, qkv, P, (size_t)stride_p, q_norm_w, k_norm_w, eps, cs, sin_t, positions, seg_of_token, qo, *kv,
                 write_kv, T, heads, status);
    };
    const bool many = (long long)T * slots >= 8192;   // a prompt portion: four heads per warp; a few decoded tokens: one
    if (act_dtype == IB_F32 && hd == 128) {
      if (many) go(qk_norm_rope_kv_vec_kernel<128, float, float, 4>, 4, (float*)q_out);
      else go(qk_norm_rope_kv_vec_kernel<128, float, float, 1>, 1, (float*)q_out);
    } else if (act_dtype == IB_F32) {
      if (many) go(qk_norm_rope_kv_vec_kernel<64, float, float, 4>, 4, (float*)q_out);
      else go(qk_norm_rope_kv_vec_kernel<64, float, float, 1>, 1, (float*)q_out);
    } else if (hd == 128) {
      if (many) go(qk_norm_rope_kv_vec_kernel<128, __nv_bfloat16, __nv_bfloat16, 4>, 4, (__nv_bfloat16*)q_out);
      else go(qk_norm_rope_kv_vec_kernel<128, __nv_bfloat16, __nv_bfloat16, 1>, 1, (__nv_bfloat16*)q_out);
    } else {
      if (many) go(qk_norm_rope_kv_vec_kernel<64, __nv_bfloat16, __nv_bfloat16, 4>, 4, (__nv_bfloat16*)q_out);
      else go(qk_norm_rope_kv_vec_kernel<64, __nv_bfloat16, __nv_bfloat16, 1>, 1, (__nv_bfloat16*)q_out);
    }
  }
  else if (act_dtype == IB_F32)
    ib::launch(qk_norm_rope_kv_kernel<float, float>, blocks, kWarps * 32, 0, stream, qkv, P, (size_t)stride_p, q_norm_w, k_norm_w, eps, cos_t, sin_t,
                                                                            rot_half, positions, seg_of_token, (float*)q_out, *kv, write_kv,
                                                                            T, heads, status);
  else
    ib::launch(qk_norm_rope_kv_kernel<__nv_bfloat16, __nv_bfloat16>, blocks, kWarps * 32, 0, stream, 
        qkv, P, (size_t)stride_p, q_norm_w, k_norm_w, eps, cos_t, sin_t, rot_half, positions, seg_of_token, (__nv_bfloat16*)q_out, *kv,
        write_kv, T, heads, status);
  IB_CHECK_LAUNCH("qk_norm_rope_kv");
  return 0;
}

extern "C" int ib_attention_generic(const void* q, int act_dtype, const IbKvView* kv, const int* positions, const int* seg_of_token,
                                    int window, float scale, void* out, int T, int heads, unsigned* status, cudaStream_t stream) {
  if (T == 0) return 0;
  if (check_view("attention_generic", kv, heads)) return 1;
  IB_CHECK_ARG((act_dtype == IB_F32 && kv->dtype == IB_F32) || (act_dtype == IB_BF16 && kv->dtype == IB_BF16),
               "attention_generic: activation dtype %d and cache dtype %d must match", act_dtype, kv->dtype);
  long long items = (long long)T * heads;
  unsigned blocks = (unsigned)((items + kWarps - 1) / kWarps);
  if (act_dtype == IB_F32)
    ib::launch(attention_generic_kernel<float, float>, blocks, kWarps * 32, 0, stream, (const float*)q, *kv, positions, seg_of_token, window, scale,
                                                                              (float*)out, T, heads, status);
  else
    ib::launch(attention_generic_kernel<__nv_bfloat16, __nv_bfloat16>, blocks, kWarps * 32, 0, stream, 
        (const __nv_bfloat16*)q, *kv, positions, seg_of_token, window, scale, (__nv_bfloat16*)out, T, heads, status);
  IB_CHECK_LAUNCH("attention_generic");
  return 0;
}
