// First convolution of the Conv2d subsampling front end: one input channel,
// k x k taps, stride s, + bias + ReLU, fp32 features in, 16-bit NHWC out
// (oasr/models/conformer/model.py:433-444 runs it as a generic NHWC
// Conv2dActivation; with a single input channel it is a 9-tap stencil per
// output channel, HBM-bound on its output: 2*C bytes per output position).
// The features are read in fp32 and the products accumulated in fp32, so the
// only rounding is the one on store.
#include "common.cuh"

namespace ob {
namespace {

struct Conv1Args {
  void* out;            // (B, T1, F1, C) 16-bit
  const float* in;      // (B, T, F) fp32
  const float* weight;  // (C, k, k) fp32
  const float* bias;    // (C) fp32
  const int32_t* t1_limit;  // nullable (B): output frames >= limit are skipped
  int B, T, F, C, T1, F1, k, s;
};

// One warp per output position; lane l owns channels [l*8, l*8+8) of every 256-channel group.
template <typename T>
__global__ void __launch_bounds__(256) subsample_conv1_kernel(Conv1Args a) {
  extern __shared__ float sm[];  // [k*k][C] weights, then [C] bias
  const int taps = a.k * a.k;
  float* sw = sm;
  float* sb = sm + taps * a.C;
  for (int i = threadIdx.x; i < taps * a.C; i += blockDim.x) {
    const int tap = i / a.C, c = i - tap * a.C;
    sw[i] = a.weight[c * taps + tap];
  }
  for (int i = threadIdx.x; i < a.C; i += blockDim.x) sb[i] = a.bias[i];
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int64_t total = static_cast<int64_t>(a.B) * a.T1 * a.F1;
  const int64_t wstride = static_cast<int64_t>(gridDim.x) * warps_per_block;
  T* out = static_cast<T*>(a.out);
  for (int64_t pos = static_cast<int64_t>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5); pos < total;
       pos += wstride) {
    const int f1 = static_cast<int>(pos % a.F1);
    const int t1 = static_cast<int>((pos / a.F1) % a.T1);
    const int b = static_cast<int>(pos / (static_cast<int64_t>(a.F1) * a.T1));
    if (a.t1_limit && t1 >= a.t1_limit[b]) continue;
    // lane i < taps loads input tap i, then every lane reads all taps by shuffle
    float xin = 0.f;
    if (lane < taps) {
      const int i = lane / a.k, j = lane - i * a.k;
      xin = a.in[(static_cast<int64_t>(b) * a.T + (t1 * a.s + i)) * a.F + (f1 * a.s + j)];
    }
    for (int c0 = lane * 8; c0 < a.C; c0 += 256) {
      float acc[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] = sb[c0 + q];
      for (int tap = 0; tap < taps; ++tap) {
        const float x = __shfl_sync(0xffffffffu, xin, tap);
        const float4 w0 = *reinterpret_cast<const float4*>(sw + tap * a.C + c0);
        const float4 w1 = *reinterpret_cast<const float4*>(sw + tap * a.C + c0 + 4);
        acc[0] = fmaf(x, w0.x, acc[0]); acc[1] = fmaf(x, w0.y, acc[1]);
        acc[2] = fmaf(x, w0.z, acc[2]); acc[3] = fmaf(x, w0.w, acc[3]);
        acc[4] = fmaf(x, w1.x, acc[4]); acc[5] = fmaf(x, w1.y, acc[5]);
        acc[6] = fmaf(x, w1.z, acc[6]); acc[7] = fmaf(x, w1.w, acc[7]);
      }
      Pack<T> o;
#pragma unroll
      for (int q = 0; q < 8; ++q) o.v[q] = Elem<T>::from_f(fmaxf(acc[q], 0.f));
      st128(out + pos * a.C + c0, o);
    }
  }
}

}  // namespace
}  // namespace ob

extern "C" {

int oasr_b200_subsample_conv1(void* out, const float* in, const float* weight, const float* bias,
                              const int32_t* t1_limit, int64_t B, int64_t T, int64_t F, int64_t C, int64_t kernel,
                              int64_t stride, int dtype, void* stream) {
  using namespace ob;
  OB_REQUIRE(B >= 0 && T > 0 && F > 0 && C > 0 && kernel > 0 && stride > 0, OASR_ERR_INVALID,
             "subsample_conv1: bad shape");
  OB_REQUIRE(kernel * kernel <= 32, OASR_ERR_UNSUPPORTED, "subsample_conv1: at most 32 taps (got %lld x %lld)",
             (long long)kernel, (long long)kernel);
  OB_REQUIRE(C % 8 == 0, OASR_ERR_ALIGN, "subsample_conv1: channel count must be a multiple of 8");
  OB_REQUIRE(T >= kernel && F >= kernel, OASR_ERR_INVALID, "subsample_conv1: input smaller than the kernel");
  if (B == 0) return OASR_OK;
  OB_REQUIRE(out && in && weight && bias, OASR_ERR_INVALID, "subsample_conv1: null pointer argument");
  OB_REQUIRE(is_aligned(out, 16), OASR_ERR_ALIGN, "subsample_conv1: out must be 16-byte aligned");
  Conv1Args a{out, in, weight, bias, t1_limit, (int)B, (int)T, (int)F, (int)C,
              (int)((T - kernel) / stride + 1), (int)((F - kernel) / stride + 1), (int)kernel, (int)stride};
  const size_t smem = (static_cast<size_t>(kernel * kernel) * C + C) * sizeof(float);
  OB_REQUIRE(smem <= 200 * 1024, OASR_ERR_UNSUPPORTED, "subsample_conv1: weights do not fit in shared memory");
  const int64_t total = B * a.T1 * a.F1;
  int64_t grid = (total + 7) / 8;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 4;
  if (grid > cap) grid = cap;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return OB_DISPATCH_HALF(dtype, T_, [&]() -> int {
    auto kern = subsample_conv1_kernel<T_>;
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return set_error(OASR_ERR_CUDA, "subsample_conv1: %s", cudaGetErrorString(e));
    }
    kern<<<static_cast<unsigned>(grid), 256, smem, s>>>(a);
    return check_launch("subsample_conv1 launch");
  });
}

}  // extern "C"
