// Shared device helpers and the error convention of the kernel library.
//
// Every exported function is `extern "C" int ib_*(…, cudaStream_t stream)`: 0 on success, a
// non-zero code after ib_set_error() stored a message that ib_last_error() returns. Kernels are
// launched on the caller's stream and never synchronise.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define IB_F32 0
#define IB_BF16 1

extern "C" const char* ib_last_error();
int ib_set_error(const char* fmt, ...);

#define IB_CHECK_ARG(cond, ...)                 \
  do {                                          \
    if (!(cond)) return ib_set_error(__VA_ARGS__); \
  } while (0)

#define IB_CHECK_LAUNCH(name)                                                          \
  do {                                                                                 \
    cudaError_t e__ = cudaGetLastError();                                              \
    if (e__ != cudaSuccess) return ib_set_error("%s: %s", name, cudaGetErrorString(e__)); \
  } while (0)

// Error bits that kernels set in the device-side status word (read by the host after a step).
#define IB_ERR_BAD_PAGE 1u      // a block table entry that a kernel had to use was negative or out of range
#define IB_ERR_BAD_TOKEN 2u     // a token id outside the vocabulary
#define IB_ERR_WAIT_TIMEOUT 4u  // a bounded wait on an mbarrier ran out
#define IB_ERR_INTERNAL 8u      // a kernel found one of its own assumptions broken and did nothing

// Programmatic dependent launch: a kernel may be scheduled while the kernel before it in the stream
// is still running; it runs its own set-up, and ib::pdl_wait() then blocks until everything earlier
// in the stream has finished and its writes are visible. Nothing before pdl_wait() may read memory
// that an earlier kernel writes, nor write memory at all.
extern "C" int ib_pdl_enabled();
extern "C" void ib_set_pdl(int on);

// How long a bounded wait inside a kernel (on an mbarrier) may last before the kernel gives up, sets
// IB_ERR_WAIT_TIMEOUT in the status word and unwinds. Launchers pass it to their kernels as an argument.
extern "C" unsigned long long ib_wait_limit_ns();
extern "C" void ib_set_wait_limit_ms(int ms);

namespace ib {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... Exp, typename... Act>
inline cudaError_t launch(void (*kernel)(Exp...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Act&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = ib_pdl_enabled();
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<Exp>(args)...);
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result. `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = lane < nwarps ? scratch[lane] : 0.f;
  return warp_sum(r);
}

}  // namespace ib
