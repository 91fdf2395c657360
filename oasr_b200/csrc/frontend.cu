// First convolution of the Conv2d subsampling front end: one input channel,
// k x k taps, stride s, + bias + ReLU, fp32 features in, 16-bit NHWC out
// (oasr/models/conformer/model.py:433-444 runs it as a generic NHWC
// Conv2dActivation; with a single input channel it is a 9-tap stencil per
// output channel, HBM-bound on its output: 2*C bytes per output position).
// The features are read in fp32 and the products accumulated in fp32, so the
// only rounding is the one on store.
#include "common.cuh"

namespace ob {
namespace conv1_mma {   // conv1_mma.cu: the parity-split 3x3 / stride-2 form on the tensor cores
bool supported(int64_t B, int64_t C);
int run(void* out, const float* in, const float* weight, const float* bias, const int32_t* t1_limit, int64_t B, int64_t T,
        int64_t F, int64_t C, int dtype, cudaStream_t s);
}  // namespace conv1_mma
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

// Fast form for the common 3x3 / stride-2 case.  A block stages the 2R+1 feature frames that R
// output frames need in shared memory (one coalesced pass), then thread (row r, channel group g)
// walks the F1 positions of output frame t1_0 + r: the taps come from shared memory as warp
// broadcasts (two new columns per input row and position, the third is carried over), the 72
// multiply-adds of its 8 channels are 36 packed fp32x2 FMAs, and the C/8 threads of a position
// write C*2 contiguous bytes.
// kS2d selects the output layout: 0 = NHWC (B, T1, F1, C); 1 = parity-split
// (B, ceil(T1/2), 4, ceil(F1/2)+pad, C) with plane index (t1 & 1) * 2 + (f1 & 1) and rows (t1 / 2,
// f1 / 2), so that every tap of a following 3x3 / stride-2 convolution reads a dense box.
template <typename T, bool kS2d>
__global__ void __launch_bounds__(256) subsample_conv1_k3s2_kernel(Conv1Args a, int rows_per_block, int TH, int FH) {
  extern __shared__ float xs[];   // (2R+1) x F
  const int groups = a.C / 8;
  const int cg = threadIdx.x % groups;
  const int r = threadIdx.x / groups;
  const int b = blockIdx.y;
  const int t1_0 = blockIdx.x * rows_per_block;
  int t1_end = a.T1;
  if (a.t1_limit) t1_end = min(t1_end, a.t1_limit[b]);
  if (t1_0 >= t1_end) return;
  const int in_rows = min(2 * rows_per_block + 1, a.T - 2 * t1_0);
  const float* __restrict__ xin = a.in + (static_cast<int64_t>(b) * a.T + 2 * t1_0) * a.F;
  for (int i = threadIdx.x; i < in_rows * a.F; i += blockDim.x) xs[i] = __ldg(xin + i);
  const int c0 = cg * 8;
  float2 w[9][4], bias[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    bias[q] = make_float2(a.bias[c0 + 2 * q], a.bias[c0 + 2 * q + 1]);
#pragma unroll
    for (int tap = 0; tap < 9; ++tap)
      w[tap][q] = make_float2(a.weight[(c0 + 2 * q) * 9 + tap], a.weight[(c0 + 2 * q + 1) * 9 + tap]);
  }
  __syncthreads();
  const int t1 = t1_0 + r;
  if (r >= rows_per_block || t1 >= t1_end) return;
  const float* x0 = xs + (2 * r) * a.F;
  const float* x1 = x0 + a.F;
  const float* x2 = x1 + a.F;
  T* out;
  int64_t pos_stride_even, odd_offset;
  if constexpr (kS2d) {
    // plane (t1&1)*2 + fpar of frame pair t1/2; consecutive f1 of equal parity are C apart
    out = static_cast<T*>(a.out) + ((static_cast<int64_t>(b) * TH + (t1 >> 1)) * 4 + (t1 & 1) * 2) * FH * a.C + c0;
    pos_stride_even = a.C;
    odd_offset = static_cast<int64_t>(FH) * a.C;
  } else {
    out = static_cast<T*>(a.out) + (static_cast<int64_t>(b) * a.T1 + t1) * a.F1 * a.C + c0;
    pos_stride_even = 0;
    odd_offset = 0;
  }
  float c00 = x0[0], c10 = x1[0], c20 = x2[0];
  for (int f1 = 0; f1 < a.F1; ++f1) {
    const float c01 = x0[2 * f1 + 1], c02 = x0[2 * f1 + 2];
    const float c11 = x1[2 * f1 + 1], c12 = x1[2 * f1 + 2];
    const float c21 = x2[2 * f1 + 1], c22 = x2[2 * f1 + 2];
    const float xv[9] = {c00, c01, c02, c10, c11, c12, c20, c21, c22};
    float2 acc[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) acc[q] = bias[q];
#pragma unroll
    for (int tap = 0; tap < 9; ++tap) {
      const float2 xx = make_float2(xv[tap], xv[tap]);
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[q] = __ffma2_rn(xx, w[tap][q], acc[q]);
    }
    Pack<T> o;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      o.v[2 * q] = Elem<T>::from_f(fmaxf(acc[q].x, 0.f));
      o.v[2 * q + 1] = Elem<T>::from_f(fmaxf(acc[q].y, 0.f));
    }
    if constexpr (kS2d) st128(out + (f1 & 1) * odd_offset + (f1 >> 1) * pos_stride_even, o);
    else st128(out + static_cast<int64_t>(f1) * a.C, o);
    c00 = c02; c10 = c12; c20 = c22;
  }
}

template <typename T>
int launch_k3s2(const Conv1Args& a, bool s2d, cudaStream_t s) {
  const int groups = a.C / 8;
  const int R = 256 / groups;
  const size_t smem = static_cast<size_t>(2 * R + 1) * a.F * sizeof(float);
  dim3 grid(static_cast<unsigned>((a.T1 + R - 1) / R), static_cast<unsigned>(a.B));
  const int TH = (a.T1 + 1) / 2, FH = (a.F1 + 1) / 2;
  if (s2d) subsample_conv1_k3s2_kernel<T, true><<<grid, 256, smem, s>>>(a, R, TH, FH);
  else subsample_conv1_k3s2_kernel<T, false><<<grid, 256, smem, s>>>(a, R, TH, FH);
  return check_launch("subsample_conv1 launch");
}

bool k3s2_applies(const Conv1Args& a) {
  const int groups = a.C / 8;
  return a.k == 3 && a.s == 2 && groups >= 1 && groups <= 256 && 256 % groups == 0 &&
         static_cast<size_t>(2 * (256 / groups) + 1) * a.F * sizeof(float) <= 48 * 1024;
}

// Depthwise 3x3 / stride-2 Conv2d on NHWC 16-bit data with causal-style zero padding (pad_lo columns before, pad_hi
// after on the frequency axis; tpad_lo / tpad_hi frames on the time axis -- equal to the frequency pads offline, zero
// for a streaming chunk whose left context is the cached tail prepended by the caller): the depthwise half of a stage
// of the FastConformer 8x subsampling stack (oasr/models/nemotron/subsampling.py:204-224, padding geometry :39-53,
// streaming form :156-189).  HBM-bound: a thread
// owns 8 channels of one output position (9 x 16-byte loads, 72 FMAs, one 16-byte store); output frames at or past
// out_len[b] (nullable) are written as zeros, which is the reference's per-stage time mask.
struct Dw2dArgs {
  void* out;
  const void* in;
  const void* weight;   // (C, 3, 3) 16-bit
  const void* bias;     // nullable (C)
  const int32_t* out_len;
  const int32_t* in_len;   // nullable: input frames >= in_len[b] count as zeros (whatever the buffer holds there)
  int B, T, F, C, To, Fo, pad_lo;   // pad_lo: zero columns before the first frequency bin
  int tpad_lo;                        // zero frames before the first input frame
};

// kHoist: 256 % (C/8) == 0, so a thread keeps one channel group for its whole grid-stride walk; the weights sit in
// shared memory as fp32 and the nine 16-byte input loads of a position are issued together.
template <typename T, bool kHoist>
__global__ void __launch_bounds__(256, 2) depthwise_conv2d_k3s2_kernel(Dw2dArgs a) {
  const int groups = a.C / 8;
  const int64_t positions = static_cast<int64_t>(a.B) * a.To * a.Fo;
  const T* wt = static_cast<const T*>(a.weight);
  const T* in = static_cast<const T*>(a.in);
  if constexpr (kHoist) {
    const int cg = threadIdx.x % groups;
    const int c0 = cg * 8;
    const int lanes = 256 / groups;                 // positions per block and step
    // weights as fp32 [tap][channel] (+ the bias row) in shared memory: a thread reads its 8 channels of a tap as two
    // 16-byte words, consecutive threads consecutive words
    extern __shared__ float dw2d_smem[];
    float* sw = dw2d_smem;
    for (int e = threadIdx.x; e < 10 * a.C; e += 256) {
      const int k = e / a.C, c = e - k * a.C;
      sw[e] = k < 9 ? Elem<T>::to_f(wt[c * 9 + k]) : (a.bias ? Elem<T>::to_f(static_cast<const T*>(a.bias)[c]) : 0.f);
    }
    __syncthreads();
    // positions fit 32 bits (the host checks); the per-stream limits are re-read only when the stream changes, so the
    // input loads of a position do not wait on them
    const uint32_t pstride = gridDim.x * static_cast<uint32_t>(lanes);
    const uint32_t npos = static_cast<uint32_t>(positions);
    const uint32_t per_b = static_cast<uint32_t>(a.To) * a.Fo;
    int cur_b = -1, lim_out = 0, t_end = 0;
    for (uint32_t pos = blockIdx.x * static_cast<uint32_t>(lanes) + threadIdx.x / groups; pos < npos; pos += pstride) {
      const int b = static_cast<int>(pos / per_b);
      const uint32_t rem = pos - static_cast<uint32_t>(b) * per_b;
      const int to = static_cast<int>(rem / a.Fo);
      const int fo = static_cast<int>(rem - static_cast<uint32_t>(to) * a.Fo);
      if (b != cur_b) {
        cur_b = b;
        lim_out = a.out_len ? a.out_len[b] : a.To;
        t_end = a.in_len ? min(a.T, a.in_len[b]) : a.T;
      }
      const bool live = to < lim_out;
      Pack<T> x[9];
      bool ok[9];
#pragma unroll
      for (int di = 0; di < 3; ++di) {
        const int t = 2 * to + di - a.tpad_lo;
#pragma unroll
        for (int dj = 0; dj < 3; ++dj) {
          const int f = 2 * fo + dj - a.pad_lo;
          ok[di * 3 + dj] = live && t >= 0 && t < t_end && f >= 0 && f < a.F;
          if (ok[di * 3 + dj]) x[di * 3 + dj] = ld128(in + ((static_cast<int64_t>(b) * a.T + t) * a.F + f) * a.C + c0);
        }
      }
      float acc[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] = live ? sw[9 * a.C + c0 + q] : 0.f;
#pragma unroll
      for (int k = 0; k < 9; ++k) {
        if (ok[k]) {
          const float4 w0 = *reinterpret_cast<const float4*>(sw + k * a.C + c0);
          const float4 w1 = *reinterpret_cast<const float4*>(sw + k * a.C + c0 + 4);
          const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
          for (int q = 0; q < 8; ++q) acc[q] = fmaf(Elem<T>::to_f(x[k].v[q]), w[q], acc[q]);
        }
      }
      Pack<T> o;
#pragma unroll
      for (int q = 0; q < 8; ++q) o.v[q] = Elem<T>::from_f(acc[q]);
      st128(static_cast<T*>(a.out) + static_cast<int64_t>(pos) * a.C + c0, o);
    }
  } else {
    const int64_t total = positions * groups;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
      const int cg = static_cast<int>(i % groups);
      int64_t r = i / groups;
      const int fo = static_cast<int>(r % a.Fo);
      r /= a.Fo;
      const int to = static_cast<int>(r % a.To);
      const int b = static_cast<int>(r / a.To);
      const int c0 = cg * 8;
      float acc[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] = 0.f;
      const bool live = !a.out_len || to < a.out_len[b];
      const int t_end = a.in_len ? min(a.T, a.in_len[b]) : a.T;
      if (live) {
        if (a.bias) {
          const Pack<T> bb = ld128(static_cast<const T*>(a.bias) + c0);
#pragma unroll
          for (int q = 0; q < 8; ++q) acc[q] = Elem<T>::to_f(bb.v[q]);
        }
#pragma unroll
        for (int di = 0; di < 3; ++di) {
          const int t = 2 * to + di - a.tpad_lo;
          if (t < 0 || t >= t_end) continue;
#pragma unroll
          for (int dj = 0; dj < 3; ++dj) {
            const int f = 2 * fo + dj - a.pad_lo;
            if (f < 0 || f >= a.F) continue;
            const Pack<T> x = ld128(in + ((static_cast<int64_t>(b) * a.T + t) * a.F + f) * a.C + c0);
#pragma unroll
            for (int q = 0; q < 8; ++q)
              acc[q] = fmaf(Elem<T>::to_f(x.v[q]), Elem<T>::to_f(wt[(c0 + q) * 9 + di * 3 + dj]), acc[q]);
          }
        }
      }
      Pack<T> o;
#pragma unroll
      for (int q = 0; q < 8; ++q) o.v[q] = Elem<T>::from_f(acc[q]);
      st128(static_cast<T*>(a.out) + ((static_cast<int64_t>(b) * a.To + to) * a.Fo + fo) * a.C + c0, o);
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
  OB_REQUIRE(B <= 65535, OASR_ERR_INVALID, "subsample_conv1: batch too large");
  if (k3s2_applies(a)) {
    return OB_DISPATCH_HALF(dtype, T_, [&]() -> int { return launch_k3s2<T_>(a, false, static_cast<cudaStream_t>(stream)); });
  }
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

int oasr_b200_subsample_conv1_s2d(void* out, const float* in, const float* weight, const float* bias,
                                  const int32_t* t1_limit, int64_t B, int64_t T, int64_t F, int64_t C, int dtype,
                                  void* stream) {
  using namespace ob;
  OB_REQUIRE(B >= 0 && T >= 3 && F >= 3 && C > 0, OASR_ERR_INVALID, "subsample_conv1_s2d: bad shape");
  if (B == 0) return OASR_OK;
  OB_REQUIRE(out && in && weight && bias, OASR_ERR_INVALID, "subsample_conv1_s2d: null pointer argument");
  OB_REQUIRE(C % 8 == 0 && is_aligned(out, 16), OASR_ERR_ALIGN,
             "subsample_conv1_s2d: channels must be a multiple of 8 and out 16-byte aligned");
  OB_REQUIRE(B <= 65535, OASR_ERR_INVALID, "subsample_conv1_s2d: batch too large");
  if (conv1_mma::supported(B, C) && (dtype == OASR_DT_BF16 || dtype == OASR_DT_F16))
    return conv1_mma::run(out, in, weight, bias, t1_limit, B, T, F, C, dtype, static_cast<cudaStream_t>(stream));
  Conv1Args a{out, in, weight, bias, t1_limit, (int)B, (int)T, (int)F, (int)C, (int)((T - 3) / 2 + 1),
              (int)((F - 3) / 2 + 1), 3, 2};
  OB_REQUIRE(k3s2_applies(a), OASR_ERR_UNSUPPORTED,
             "subsample_conv1_s2d: channels / 8 must be a power of two <= 256 (got C = %lld)", (long long)C);
  return OB_DISPATCH_HALF(dtype, T_, [&]() -> int { return launch_k3s2<T_>(a, true, static_cast<cudaStream_t>(stream)); });
}

int oasr_b200_depthwise_conv2d_k3s2(void* out, const void* in, const void* weight, const void* bias,
                                    const int32_t* out_len, const int32_t* in_len, int64_t B, int64_t T, int64_t F, int64_t C, int64_t pad_lo,
                                    int64_t pad_hi, int64_t time_pad_lo, int64_t time_pad_hi, int dtype, void* stream) {
  using namespace ob;
  OB_REQUIRE(B >= 0 && T > 0 && F > 0 && C > 0 && pad_lo >= 0 && pad_hi >= 0 && time_pad_lo >= 0 && time_pad_hi >= 0,
             OASR_ERR_INVALID, "depthwise_conv2d_k3s2: bad shape");
  OB_REQUIRE(T + time_pad_lo + time_pad_hi >= 3 && F + pad_lo + pad_hi >= 3, OASR_ERR_INVALID,
             "depthwise_conv2d_k3s2: padded input smaller than the kernel");
  if (B == 0) return OASR_OK;
  OB_REQUIRE(out && in && weight, OASR_ERR_INVALID, "depthwise_conv2d_k3s2: null pointer argument");
  OB_REQUIRE(C % 8 == 0 && is_aligned(out, 16) && is_aligned(in, 16) && (!bias || is_aligned(bias, 16)), OASR_ERR_ALIGN,
             "depthwise_conv2d_k3s2: channels must be a multiple of 8 and the tensors 16-byte aligned");
  Dw2dArgs a{out, in, weight, bias, out_len, in_len, (int)B, (int)T, (int)F, (int)C,
             (int)((T + time_pad_lo + time_pad_hi - 3) / 2 + 1), (int)((F + pad_lo + pad_hi - 3) / 2 + 1), (int)pad_lo,
             (int)time_pad_lo};
  const int groups = (int)(C / 8);
  const bool hoist = 256 % groups == 0 && C <= 1024 && B * a.To * a.Fo < (int64_t(1) << 31);     // 40 bytes of shared memory per channel
  const int64_t total = B * a.To * a.Fo * groups;
  int64_t g = (total + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count()) * (hoist ? 2 : 16);   // hoisted: one resident wave, weights staged once
  if (g > cap) g = cap;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return OB_DISPATCH_HALF(dtype, T_, [&]() -> int {
    if (hoist) depthwise_conv2d_k3s2_kernel<T_, true><<<static_cast<unsigned>(g), 256, 10 * C * sizeof(float), s>>>(a);
    else depthwise_conv2d_k3s2_kernel<T_, false><<<static_cast<unsigned>(g), 256, 0, s>>>(a);
    return check_launch("depthwise_conv2d_k3s2 launch");
  });
}

}  // extern "C"
