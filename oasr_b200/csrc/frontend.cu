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

// A thread owns 8 output channels for the whole kernel (weights and bias in registers) and walks
// output positions; the C/8 threads of one position write C*2 contiguous bytes.  The k*k input
// taps of a position are the same address for all its threads (one broadcast load each).
template <typename T, int kK>
__global__ void __launch_bounds__(256) subsample_conv1_kernel(Conv1Args a) {
  constexpr int kTaps = kK * kK;
  const int groups = a.C / 8;                 // threads per position
  const int lanes = blockDim.x / groups;      // positions handled concurrently by a block
  const int cg = threadIdx.x % groups;
  const int pl = threadIdx.x / groups;
  if (pl >= lanes) return;
  const int c0 = cg * 8;
  float w[kTaps][8], bias[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    bias[q] = a.bias[c0 + q];
#pragma unroll
    for (int tap = 0; tap < kTaps; ++tap) w[tap][q] = a.weight[(c0 + q) * kTaps + tap];
  }
  // blockIdx.y = batch row; positions (t1, f1) of that row are walked with 32-bit arithmetic
  const int b = blockIdx.y;
  int t1_end = a.T1;
  if (a.t1_limit) t1_end = min(t1_end, a.t1_limit[b]);
  const unsigned total = static_cast<unsigned>(t1_end) * a.F1;
  const unsigned stride = gridDim.x * lanes;
  const float* __restrict__ xin = a.in + static_cast<int64_t>(b) * a.T * a.F;
  T* __restrict__ out = static_cast<T*>(a.out) + static_cast<int64_t>(b) * a.T1 * a.F1 * a.C + c0;
  for (unsigned pos = blockIdx.x * lanes + pl; pos < total; pos += stride) {
    const unsigned t1 = pos / static_cast<unsigned>(a.F1);
    const unsigned f1 = pos - t1 * a.F1;
    const float* x = xin + (t1 * a.s) * a.F + f1 * a.s;
    float acc[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) acc[q] = bias[q];
#pragma unroll
    for (int i = 0; i < kK; ++i) {
#pragma unroll
      for (int j = 0; j < kK; ++j) {
        const float xv = __ldg(x + i * a.F + j);
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[q] = fmaf(xv, w[i * kK + j][q], acc[q]);
      }
    }
    Pack<T> o;
#pragma unroll
    for (int q = 0; q < 8; ++q) o.v[q] = Elem<T>::from_f(fmaxf(acc[q], 0.f));
    st128(out + static_cast<int64_t>(pos) * a.C, o);
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
  OB_REQUIRE(kernel == 3 || kernel == 5, OASR_ERR_UNSUPPORTED, "subsample_conv1: kernel size 3 or 5 (got %lld)",
             (long long)kernel);
  OB_REQUIRE(C / 8 <= 256, OASR_ERR_UNSUPPORTED, "subsample_conv1: at most 2048 output channels");
  OB_REQUIRE(C % 8 == 0, OASR_ERR_ALIGN, "subsample_conv1: channel count must be a multiple of 8");
  OB_REQUIRE(T >= kernel && F >= kernel, OASR_ERR_INVALID, "subsample_conv1: input smaller than the kernel");
  if (B == 0) return OASR_OK;
  OB_REQUIRE(out && in && weight && bias, OASR_ERR_INVALID, "subsample_conv1: null pointer argument");
  OB_REQUIRE(is_aligned(out, 16), OASR_ERR_ALIGN, "subsample_conv1: out must be 16-byte aligned");
  Conv1Args a{out, in, weight, bias, t1_limit, (int)B, (int)T, (int)F, (int)C,
              (int)((T - kernel) / stride + 1), (int)((F - kernel) / stride + 1), (int)kernel, (int)stride};
  const int groups = (int)(C / 8);
  const int block = (256 / groups) * groups;      // whole positions per block
  const int lanes = block / groups;
  OB_REQUIRE(B <= 65535 && static_cast<int64_t>(a.T1) * a.F1 < (int64_t(1) << 31), OASR_ERR_INVALID,
             "subsample_conv1: batch or frame count too large");
  const int64_t per_row = static_cast<int64_t>(a.T1) * a.F1;
  int64_t gx = (per_row + lanes - 1) / lanes;
  const int64_t cap = (static_cast<int64_t>(sm_count()) * 8 + B - 1) / B;
  if (gx > cap) gx = cap;
  if (gx < 1) gx = 1;
  dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(B));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return OB_DISPATCH_HALF(dtype, T_, [&]() -> int {
    if (kernel == 3) subsample_conv1_kernel<T_, 3><<<grid, block, 0, s>>>(a);
    else subsample_conv1_kernel<T_, 5><<<grid, block, 0, s>>>(a);
    return check_launch("subsample_conv1 launch");
  });
}

}  // extern "C"
