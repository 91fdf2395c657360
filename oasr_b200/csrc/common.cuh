// Shared device/host helpers for the sm_100a kernels of the encoder hot path.
//
// Everything here is header-only: element-type traits, 128-bit vector access,
// warp/block reductions, the activation functor table and the error plumbing
// of the C-ABI (thread-local message + integer status).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/oasr_b200.h"

namespace ob {

// ---------------------------------------------------------------------------
// Error plumbing (host)
// ---------------------------------------------------------------------------
int set_error(int code, const char* fmt, ...);  // defined in capi.cu
int check_launch(const char* what);             // cudaGetLastError -> status

#define OB_REQUIRE(cond, code, ...)                  \
  do {                                               \
    if (!(cond)) return ::ob::set_error((code), __VA_ARGS__); \
  } while (0)

inline bool is_aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// ---------------------------------------------------------------------------
// Element traits
// ---------------------------------------------------------------------------
template <typename T>
struct Elem;
template <>
struct Elem<float> {
  static constexpr int kVec = 4;  // elements per 128-bit access
  __device__ static float to_f(float v) { return v; }
  __device__ static float from_f(float v) { return v; }
};
template <>
struct Elem<__half> {
  static constexpr int kVec = 8;
  __device__ static float to_f(__half v) { return __half2float(v); }
  __device__ static __half from_f(float v) { return __float2half_rn(v); }
};
template <>
struct Elem<__nv_bfloat16> {
  static constexpr int kVec = 8;
  __device__ static float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ static __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};

// 128-bit packet of T.
template <typename T>
struct alignas(16) Pack {
  T v[Elem<T>::kVec];
};

template <typename T>
__device__ __forceinline__ Pack<T> ld128(const T* p) {
  Pack<T> r;
  *reinterpret_cast<uint4*>(&r) = *reinterpret_cast<const uint4*>(p);
  return r;
}
template <typename T>
__device__ __forceinline__ Pack<T> ld128_nc(const T* p) {
  Pack<T> r;
  *reinterpret_cast<uint4*>(&r) = __ldg(reinterpret_cast<const uint4*>(p));
  return r;
}
// Streaming load: data is read exactly once, do not keep it in L1.
template <typename T>
__device__ __forceinline__ Pack<T> ld128_stream(const T* p) {
  Pack<T> r;
  uint4 u;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w)
               : "l"(p));
  *reinterpret_cast<uint4*>(&r) = u;
  return r;
}
template <typename T>
__device__ __forceinline__ void st128(T* p, const Pack<T>& r) {
  *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&r);
}

// ---------------------------------------------------------------------------
// Reductions
// ---------------------------------------------------------------------------
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

// Block-wide sum for blocks of up to 1024 threads; `red` holds >= 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[wid] = v;
  __syncthreads();
  if (wid == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    float t = lane < nw ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// ---------------------------------------------------------------------------
// Activations.  Ids follow the reference's ActivationType enum
// (include/oasr/common/types.h:49-56): 0 relu, 1 gelu (tanh form), 2 swish,
// 4 gelu (erf form).  -1 is "identity" (no counterpart id in the reference).
// ---------------------------------------------------------------------------
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }

template <int kAct>
__device__ __forceinline__ float apply_act(float x) {
  if constexpr (kAct == OASR_ACT_RELU) {
    return fmaxf(x, 0.f);
  } else if constexpr (kAct == OASR_ACT_GELU_TANH) {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    return 0.5f * x * (1.f + tanhf(k0 * (x + k1 * x * x * x)));
  } else if constexpr (kAct == OASR_ACT_SWISH) {
    return x * sigmoid_f(x);
  } else if constexpr (kAct == OASR_ACT_GELU_ERF) {
    return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));
  } else {
    return x;
  }
}

__device__ __forceinline__ float apply_act_rt(float x, int act) {
  switch (act) {
    case OASR_ACT_RELU: return apply_act<OASR_ACT_RELU>(x);
    case OASR_ACT_GELU_TANH: return apply_act<OASR_ACT_GELU_TANH>(x);
    case OASR_ACT_SWISH: return apply_act<OASR_ACT_SWISH>(x);
    case OASR_ACT_GELU_ERF: return apply_act<OASR_ACT_GELU_ERF>(x);
    default: return x;
  }
}

// One-MUFU forms for epilogues whose result is rounded to a 16-bit type anyway: tanh.approx has
// a relative error of about 2^-11, below half an ulp of bf16 and of the same order as fp16's.
__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float sigmoid_fast(float x) { return fmaf(0.5f, tanh_approx(0.5f * x), 0.5f); }
__device__ __forceinline__ float swish_fast(float x) {
  const float h = 0.5f * x;
  return fmaf(h, tanh_approx(h), h);
}
__device__ __forceinline__ float apply_act_fast(float x, int act) {
  switch (act) {
    case OASR_ACT_RELU: return fmaxf(x, 0.f);
    case OASR_ACT_GELU_TANH: {
      const float k0 = 0.7978845608028654f, k1 = 0.044715f;
      const float h = 0.5f * x;
      return fmaf(h, tanh_approx(k0 * fmaf(k1 * x * x, x, x)), h);
    }
    case OASR_ACT_SWISH: return swish_fast(x);
    case OASR_ACT_GELU_ERF: return apply_act<OASR_ACT_GELU_ERF>(x);
    default: return x;
  }
}

inline bool act_is_known(int act) {
  return act == OASR_ACT_NONE || act == OASR_ACT_RELU || act == OASR_ACT_GELU_TANH ||
         act == OASR_ACT_SWISH || act == OASR_ACT_GELU_ERF;
}

// Dispatch a lambda on the element type named by an oasr_dtype id.
#define OB_DISPATCH_FLOAT(dtype, T, ...)                                  \
  [&]() -> int {                                                          \
    switch (dtype) {                                                      \
      case OASR_DT_F32: { using T = float; return __VA_ARGS__(); }        \
      case OASR_DT_F16: { using T = __half; return __VA_ARGS__(); }       \
      case OASR_DT_BF16: { using T = __nv_bfloat16; return __VA_ARGS__(); } \
      default: return ::ob::set_error(OASR_ERR_DTYPE, "unsupported dtype id %d", (int)(dtype)); \
    }                                                                     \
  }()

#define OB_DISPATCH_HALF(dtype, T, ...)                                   \
  [&]() -> int {                                                          \
    switch (dtype) {                                                      \
      case OASR_DT_F16: { using T = __half; return __VA_ARGS__(); }       \
      case OASR_DT_BF16: { using T = __nv_bfloat16; return __VA_ARGS__(); } \
      default: return ::ob::set_error(OASR_ERR_DTYPE, "dtype id %d: only fp16/bf16 are supported here", (int)(dtype)); \
    }                                                                     \
  }()

extern unsigned long long* g_trace_buffer;  // nullable diagnostics buffer (capi.cu), see oasr_b200_trace_buffer
int sm_count();  // cached multiprocessor count of the current device (capi.cu)

// Launch with programmatic stream serialisation (the kernel must call grid_dep_wait() before it touches
// global memory): its blocks may be scheduled while the previous kernel of the stream drains.  The "pdl"
// tunable switches the attribute (default 1; 0 = plain stream order).
extern int g_pdl;
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = g_pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

}  // namespace ob
