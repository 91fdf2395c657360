// Depthwise conv1d over channels-last rows (padded batch or packed segments),
// with optional per-channel affine (folded inference BatchNorm) and activation,
// and the streaming causal form with a rolling state.
//
// HBM-bound.  Fast path: a thread owns a channel pair and a run of kTile
// consecutive output frames; the K-frame input window slides through registers
// so every input frame is loaded once per thread ((kTile+K-1)/kTile re-read
// factor, served by L1/L2), weights live in registers, lanes of a warp touch
// 32 adjacent channel pairs (128 contiguous bytes per frame).  Algorithmic
// bytes per frame of C channels in a 16-bit type: 4C (+2KC weights once).
// The reference kernel launches one CTA of C/8 threads per output frame and
// re-reads all K taps and weights per frame (include/oasr/conv/conv1d.cuh:23-113).
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace ob {
int g_dw_path = 2;  // "dwconv_path": 2 (default) = rolling register-window kernel for kernel sizes 9 / 15, the run-at-once streaming
                    // kernel for the other sizes up to 15; 0 = the run-at-once kernel for all of them; 1 = shared-memory tiled kernel
namespace {

template <typename T>
struct Pair;
template <>
struct Pair<float> {
  __device__ static float2 ld(const float* p) { return *reinterpret_cast<const float2*>(p); }
  __device__ static void st(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
};
template <>
struct Pair<__half> {
  __device__ static float2 ld(const __half* p) { return __half22float2(*reinterpret_cast<const __half2*>(p)); }
  __device__ static void st(__half* p, float a, float b) { *reinterpret_cast<__half2*>(p) = __floats2half2_rn(a, b); }
};
template <>
struct Pair<__nv_bfloat16> {
  __device__ static float2 ld(const __nv_bfloat16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
  }
  __device__ static void st(__nv_bfloat16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
  }
};

struct DwArgs {
  void* out;
  const void* in;
  const void* weight;        // (K, C)
  const void* bias;          // nullable (C)
  const float* post_scale;   // nullable (C) fp32: y = y*scale + shift applied after bias
  const float* post_shift;   // nullable (C) fp32
  const int32_t* cu_seqlens; // nullable: packed mode, (S+1)
  const float* right_fill;   // nullable (C) fp32: value of the frames just past a segment's end
  const int32_t* fill_frames;// with right_fill: how many such frames each segment has (S)
  int64_t batch;             // batch size or number of segments
  int seq_len;               // padded mode: frames per batch row
  int out_len;               // padded mode: output frames per batch row
  int channels;
  int kernel_size;
  int pad_left;
  int act;
  // generic path only
  const void* mask;
  int mask_is_bool;
  int add_input;
};

constexpr int kTile = 8;

template <typename T, int K, bool kAffine, bool kAct>
__global__ void __launch_bounds__(128) dwconv_window_kernel(DwArgs a) {
  const int cp = blockIdx.x * blockDim.x + threadIdx.x;  // channel pair
  const int C = a.channels;
  if (cp * 2 >= C) return;
  const int c = cp * 2;
  const int64_t b = blockIdx.z;
  int64_t in_row0, out_row0;
  int TL, OL;
  if (a.cu_seqlens) {
    const int s0 = a.cu_seqlens[b], s1 = a.cu_seqlens[b + 1];
    TL = s1 - s0;
    OL = TL;
    in_row0 = s0;
    out_row0 = s0;
  } else {
    TL = a.seq_len;
    OL = a.out_len;
    in_row0 = b * a.seq_len;
    out_row0 = b * a.out_len;
  }
  const int t0 = blockIdx.y * kTile;
  if (t0 >= OL) return;
  float f0 = 0.f, f1 = 0.f;
  int fill_end = TL;  // frames in [TL, fill_end) read the fill value instead of zero
  if (a.right_fill) {
    f0 = a.right_fill[c];
    f1 = a.right_fill[c + 1];
    fill_end = TL + a.fill_frames[b];
  }
  const T* __restrict__ in = static_cast<const T*>(a.in) + in_row0 * C + c;
  T* __restrict__ out = static_cast<T*>(a.out) + out_row0 * C + c;
  const T* __restrict__ w = static_cast<const T*>(a.weight) + c;

  float w0[K], w1[K];
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const float2 ww = Pair<T>::ld(w + static_cast<int64_t>(k) * C);
    w0[k] = ww.x;
    w1[k] = ww.y;
  }
  float b0 = 0.f, b1 = 0.f;
  if (a.bias) {
    const float2 bb = Pair<T>::ld(static_cast<const T*>(a.bias) + c);
    b0 = bb.x;
    b1 = bb.y;
  }
  float sc0 = 1.f, sc1 = 1.f, sh0 = 0.f, sh1 = 0.f;
  if constexpr (kAffine) {
    sc0 = a.post_scale[c];
    sc1 = a.post_scale[c + 1];
    sh0 = a.post_shift[c];
    sh1 = a.post_shift[c + 1];
  }

  // All kTile + K - 1 input frames of this thread's run are loaded up front (independent loads,
  // full memory-level parallelism), then the outputs are computed from registers.
  constexpr int kWin = kTile + K - 1;
  float x0[kWin], x1[kWin];
  const int first = t0 - a.pad_left;
#pragma unroll
  for (int k = 0; k < kWin; ++k) {
    const int ti = first + k;
    float2 v = make_float2(0.f, 0.f);
    if (ti >= 0 && ti < TL) v = Pair<T>::ld(in + static_cast<int64_t>(ti) * C);
    else if (ti >= TL && ti < fill_end) v = make_float2(f0, f1);
    x0[k] = v.x;
    x1[k] = v.y;
  }
#pragma unroll
  for (int j = 0; j < kTile; ++j) {
    const int t = t0 + j;
    if (t < OL) {
      float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
      for (int k = 0; k < K; ++k) {
        acc0 = fmaf(x0[j + k], w0[k], acc0);
        acc1 = fmaf(x1[j + k], w1[k], acc1);
      }
      acc0 += b0;
      acc1 += b1;
      if constexpr (kAffine) {
        acc0 = fmaf(acc0, sc0, sh0);
        acc1 = fmaf(acc1, sc1, sh1);
      }
      if constexpr (kAct) {
        acc0 = apply_act_rt(acc0, a.act);
        acc1 = apply_act_rt(acc1, a.act);
      }
      Pair<T>::st(out + static_cast<int64_t>(t) * C, acc0, acc1);
    }
  }
}

// Shared-memory tiled form (the fast path when channels*sizeof(T) is a multiple of 16): a block
// of 256 threads stages kTT + K - 1 input frames x up to 512 channels with 16-byte coalesced
// loads (all independent: the whole tile is in flight at once), then every thread slides a
// K-frame register window down its channel pair and writes kTT outputs.
constexpr int kTT = 32;
constexpr int kCB = 512;  // channels per block

template <typename T, int K, bool kAffine, bool kAct>
__global__ void __launch_bounds__(256) dwconv_tile_kernel(DwArgs a) {
  extern __shared__ __align__(16) uint8_t dw_smem[];
  T* tile = reinterpret_cast<T*>(dw_smem);
  const int C = a.channels;
  const int cb0 = blockIdx.y * kCB;
  const int cw = min(kCB, C - cb0);          // channels of this block (multiple of 16 bytes / sizeof(T))
  const int64_t b = blockIdx.z;
  int64_t in_row0, out_row0;
  int TL, OL;
  if (a.cu_seqlens) {
    const int s0 = a.cu_seqlens[b], s1 = a.cu_seqlens[b + 1];
    TL = s1 - s0; OL = TL; in_row0 = s0; out_row0 = s0;
  } else {
    TL = a.seq_len; OL = a.out_len; in_row0 = b * a.seq_len; out_row0 = b * a.out_len;
  }
  const int t0 = blockIdx.x * kTT;
  if (t0 >= OL) return;
  int fill_end = TL;
  if (a.right_fill) fill_end = TL + a.fill_frames[b];
  constexpr int kRows = kTT + K - 1;
  constexpr int kPer16 = 16 / sizeof(T);
  const int chunks_per_row = cw / kPer16;
  const int first = t0 - a.pad_left;
  const T* __restrict__ in = static_cast<const T*>(a.in) + in_row0 * C + cb0;
  // ---- stage the input tile: four independent 16-byte loads in flight per thread ----
  const int n_chunks = kRows * chunks_per_row;
  for (int i0 = threadIdx.x; i0 < n_chunks; i0 += 4 * blockDim.x) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = i0 + u * blockDim.x;
      v[u] = make_uint4(0, 0, 0, 0);
      if (i < n_chunks) {
        const int r = i / chunks_per_row, ch = i - r * chunks_per_row;
        const int ti = first + r;
        if (ti >= 0 && ti < TL) {
          v[u] = __ldg(reinterpret_cast<const uint4*>(in + static_cast<int64_t>(ti) * C) + ch);
        } else if (ti >= TL && ti < fill_end) {
          Pack<T> pk;
#pragma unroll
          for (int q = 0; q < kPer16; ++q) pk.v[q] = Elem<T>::from_f(a.right_fill[cb0 + ch * kPer16 + q]);
          v[u] = *reinterpret_cast<uint4*>(&pk);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = i0 + u * blockDim.x;
      if (i < n_chunks) {
        const int r = i / chunks_per_row, ch = i - r * chunks_per_row;
        *reinterpret_cast<uint4*>(tile + r * cw + ch * kPer16) = v[u];
      }
    }
  }
  // ---- per-thread constants (overlaps with the tile loads) ----
  const int c = threadIdx.x * 2;
  const bool active = c < cw;
  float w0[K], w1[K], b0 = 0.f, b1 = 0.f, sc0 = 1.f, sc1 = 1.f, sh0 = 0.f, sh1 = 0.f;
  if (active) {
    const T* __restrict__ w = static_cast<const T*>(a.weight) + cb0 + c;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const float2 ww = Pair<T>::ld(w + static_cast<int64_t>(k) * C);
      w0[k] = ww.x; w1[k] = ww.y;
    }
    if (a.bias) {
      const float2 bb = Pair<T>::ld(static_cast<const T*>(a.bias) + cb0 + c);
      b0 = bb.x; b1 = bb.y;
    }
    if constexpr (kAffine) {
      sc0 = a.post_scale[cb0 + c]; sc1 = a.post_scale[cb0 + c + 1];
      sh0 = a.post_shift[cb0 + c]; sh1 = a.post_shift[cb0 + c + 1];
    }
  }
  __syncthreads();
  if (!active) return;
  T* __restrict__ out = static_cast<T*>(a.out) + out_row0 * C + cb0 + c;
  float x0[K], x1[K];
#pragma unroll
  for (int k = 0; k < K - 1; ++k) {
    const float2 v = Pair<T>::ld(tile + k * cw + c);
    x0[k] = v.x; x1[k] = v.y;
  }
#pragma unroll
  for (int j = 0; j < kTT; ++j) {
    const int t = t0 + j;
    if (t < OL) {
      const float2 v = Pair<T>::ld(tile + (j + K - 1) * cw + c);
      x0[K - 1] = v.x; x1[K - 1] = v.y;
      float acc0 = b0, acc1 = b1;
#pragma unroll
      for (int k = 0; k < K; ++k) {
        acc0 = fmaf(x0[k], w0[k], acc0);
        acc1 = fmaf(x1[k], w1[k], acc1);
      }
      if constexpr (kAffine) {
        acc0 = fmaf(acc0, sc0, sh0);
        acc1 = fmaf(acc1, sc1, sh1);
      }
      if constexpr (kAct) {
        if constexpr (sizeof(T) == 2) {
          acc0 = apply_act_fast(acc0, a.act);
          acc1 = apply_act_fast(acc1, a.act);
        } else {
          acc0 = apply_act_rt(acc0, a.act);
          acc1 = apply_act_rt(acc1, a.act);
        }
      }
      Pair<T>::st(out + static_cast<int64_t>(t) * C, acc0, acc1);
#pragma unroll
      for (int k = 0; k < K - 1; ++k) { x0[k] = x0[k + 1]; x1[k] = x1[k + 1]; }
    }
  }
}

template <typename T, int K>
int launch_tile(const DwArgs& a, int max_out_len, cudaStream_t s) {
  const int cw = a.channels < kCB ? a.channels : kCB;
  const size_t smem = static_cast<size_t>(kTT + K - 1) * cw * sizeof(T);
  dim3 block(256);
  dim3 grid((max_out_len + kTT - 1) / kTT, (a.channels + kCB - 1) / kCB, static_cast<unsigned>(a.batch));
  const bool affine = a.post_scale != nullptr;
  const bool act = a.act != OASR_ACT_NONE;
#define OB_DW_TILE(AFF, ACT)                                                                         \
  do {                                                                                               \
    auto kern = dwconv_tile_kernel<T, K, AFF, ACT>;                                                  \
    if (smem > 48 * 1024) {                                                                          \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) return set_error(OASR_ERR_CUDA, "depthwise_conv1d: %s", cudaGetErrorString(e)); \
    }                                                                                                \
    kern<<<grid, block, smem, s>>>(a);                                                               \
  } while (0)
  if (affine && act) OB_DW_TILE(true, true);
  else if (affine) OB_DW_TILE(true, false);
  else if (act) OB_DW_TILE(false, true);
  else OB_DW_TILE(false, false);
#undef OB_DW_TILE
  return check_launch("depthwise_conv1d (tiled) kernel launch");
}

// Register-streaming form for 16-bit element types (the default fast path): no shared memory and
// no block-wide barrier.  A thread owns one channel pair; a warp's 32-bit loads of one frame are
// one coalesced 128-byte request.  All kST + K - 1 frames of a thread's run are requested up front
// (independent loads), then the K-deep window rotates through statically indexed registers and the
// taps are packed two-channel fp32 FMAs (fma.rn.f32x2).  Neighbouring tiles re-read the K-1 halo
// frames from L2.
constexpr int kST = 32;

template <typename T>
__device__ __forceinline__ float2 unpack_pair(uint32_t u);
template <>
__device__ __forceinline__ float2 unpack_pair<__nv_bfloat16>(uint32_t u) {
  return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
}
template <>
__device__ __forceinline__ float2 unpack_pair<__half>(uint32_t u) {
  return __half22float2(*reinterpret_cast<const __half2*>(&u));
}
template <typename T>
__device__ __forceinline__ uint32_t pack_pair(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack_pair<__half>(float a, float b) {
  const __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// kAct: 0 = none, 1 = swish, 2 = any other id (run-time switch).  Swish is separate so that the unrolled tap
// loop does not carry the never-taken activations between the instructions it executes (instruction fetch).
template <typename T, int K, bool kAffine, int kAct>
__global__ void __launch_bounds__(256, 2) dwconv_stream_kernel(DwArgs a) {
  static_assert(sizeof(T) == 2, "16-bit element types only");
  ptx::grid_dep_launch();   // no-ops unless launched with programmatic stream serialisation
  ptx::grid_dep_wait();
  const int C = a.channels;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 2;
  if (c >= C) return;
  const int64_t b = blockIdx.z;
  int64_t in_row0, out_row0;
  int TL, OL;
  if (a.cu_seqlens) {
    const int s0 = a.cu_seqlens[b], s1 = a.cu_seqlens[b + 1];
    TL = s1 - s0; OL = TL; in_row0 = s0; out_row0 = s0;
  } else {
    TL = a.seq_len; OL = a.out_len; in_row0 = b * a.seq_len; out_row0 = b * a.out_len;
  }
  const int t0 = blockIdx.x * kST;
  if (t0 >= OL) return;
  int fill_end = TL;
  uint32_t fill = 0;
  if (a.right_fill) {
    fill_end = TL + a.fill_frames[b];
    fill = pack_pair<T>(a.right_fill[c], a.right_fill[c + 1]);
  }
  const uint32_t* __restrict__ in = reinterpret_cast<const uint32_t*>(static_cast<const T*>(a.in) + in_row0 * C + c);
  const int64_t row_u32 = C / 2;
  const int first = t0 - a.pad_left;
  constexpr int kRows = kST + K - 1;
  uint32_t raw[kRows];
#pragma unroll
  for (int r = 0; r < kRows; ++r) {
    const int ti = first + r;
    uint32_t v = 0;
    if (ti >= 0 && ti < TL) v = __ldg(in + ti * row_u32);
    else if (ti >= TL && ti < fill_end) v = fill;
    raw[r] = v;
  }
  float2 w[K];
  {
    const uint32_t* __restrict__ wp = reinterpret_cast<const uint32_t*>(static_cast<const T*>(a.weight) + c);
#pragma unroll
    for (int k = 0; k < K; ++k) w[k] = unpack_pair<T>(__ldg(wp + k * row_u32));
  }
  float2 bias = make_float2(0.f, 0.f), sc = make_float2(1.f, 1.f), sh = make_float2(0.f, 0.f);
  if (a.bias) bias = unpack_pair<T>(__ldg(reinterpret_cast<const uint32_t*>(static_cast<const T*>(a.bias) + c)));
  if constexpr (kAffine) {
    sc = *reinterpret_cast<const float2*>(a.post_scale + c);
    sh = *reinterpret_cast<const float2*>(a.post_shift + c);
  }
  uint32_t* __restrict__ out = reinterpret_cast<uint32_t*>(static_cast<T*>(a.out) + out_row0 * C + c);
  float2 x[K];
#pragma unroll
  for (int k = 0; k < K - 1; ++k) x[k] = unpack_pair<T>(raw[k]);
#pragma unroll
  for (int j = 0; j < kST; ++j) {
    x[(j + K - 1) % K] = unpack_pair<T>(raw[j + K - 1]);
    float2 acc = bias;
#pragma unroll
    for (int k = 0; k < K; ++k) acc = __ffma2_rn(x[(j + k) % K], w[k], acc);
    if constexpr (kAffine) acc = __ffma2_rn(acc, sc, sh);
    if constexpr (kAct == 1) {
      acc.x = swish_fast(acc.x);
      acc.y = swish_fast(acc.y);
    } else if constexpr (kAct == 2) {
      acc.x = apply_act_fast(acc.x, a.act);
      acc.y = apply_act_fast(acc.y, a.act);
    }
    if (t0 + j < OL) out[(t0 + j) * row_u32] = pack_pair<T>(acc.x, acc.y);
  }
}

// Rolling form of the streaming kernel: a thread owns one channel pair over a run of kRollRuns * K consecutive output
// frames.  The K-deep window of unpacked inputs and a K-deep queue of packed inputs requested K frames ahead both
// rotate through statically indexed registers (the frame loop is unrolled by K), so a thread keeps 2K + K registers of
// data instead of the whole run, every input frame is loaded once per run (halo (K - 1) / run instead of (K - 1) / 32),
// and an output costs its K two-channel FMAs, one load, the unpack / pack, the activation and the store.
constexpr int kRollRuns = 4;   // 2 and 4 measure the same (0.253-0.256 ms for the 12 launches of a step), 8 is slower (0.349)

template <typename T, int K, bool kAffine, int kAct>
__global__ void __launch_bounds__(128, 4) dwconv_roll_kernel(DwArgs a) {
  static_assert(sizeof(T) == 2, "16-bit element types only");
  ptx::grid_dep_launch();   // no-ops unless launched with programmatic stream serialisation
  ptx::grid_dep_wait();
  constexpr int kRun = kRollRuns * K;
  const int C = a.channels;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 2;
  if (c >= C) return;
  const int64_t b = blockIdx.z;
  int64_t in_row0, out_row0;
  int TL, OL;
  if (a.cu_seqlens) {
    const int s0 = a.cu_seqlens[b], s1 = a.cu_seqlens[b + 1];
    TL = s1 - s0; OL = TL; in_row0 = s0; out_row0 = s0;
  } else {
    TL = a.seq_len; OL = a.out_len; in_row0 = b * a.seq_len; out_row0 = b * a.out_len;
  }
  const int t0 = blockIdx.x * kRun;
  if (t0 >= OL) return;
  int fill_end = TL;
  uint32_t fill = 0;
  if (a.right_fill) {
    fill_end = TL + a.fill_frames[b];
    fill = pack_pair<T>(a.right_fill[c], a.right_fill[c + 1]);
  }
  const uint32_t* __restrict__ in = reinterpret_cast<const uint32_t*>(static_cast<const T*>(a.in) + in_row0 * C + c);
  const int64_t row_u32 = C / 2;
  auto fetch = [&](int ti) -> uint32_t {    // input frame ti of the segment: data, the fill value past its end, else zero
    uint32_t v = 0;
    if (ti >= 0 && ti < TL) v = __ldg(in + ti * row_u32);
    else if (ti >= TL && ti < fill_end) v = fill;
    return v;
  };
  float2 w[K];
  {
    const uint32_t* __restrict__ wp = reinterpret_cast<const uint32_t*>(static_cast<const T*>(a.weight) + c);
#pragma unroll
    for (int k = 0; k < K; ++k) w[k] = unpack_pair<T>(__ldg(wp + k * row_u32));
  }
  float2 bias = make_float2(0.f, 0.f);
  if (a.bias) bias = unpack_pair<T>(__ldg(reinterpret_cast<const uint32_t*>(static_cast<const T*>(a.bias) + c)));
  if constexpr (kAffine) {   // fold y * scale + shift into the taps and the bias
    const float2 sc = *reinterpret_cast<const float2*>(a.post_scale + c);
    const float2 sh = *reinterpret_cast<const float2*>(a.post_shift + c);
#pragma unroll
    for (int k = 0; k < K; ++k) w[k] = make_float2(w[k].x * sc.x, w[k].y * sc.y);
    bias = make_float2(fmaf(bias.x, sc.x, sh.x), fmaf(bias.y, sc.y, sh.y));
  }
  const int first = t0 - a.pad_left;          // input frame under tap 0 of output t0
  float2 x[K];                                 // x[s]: the unpacked frame whose index is congruent to s (mod K) from `first`
  uint32_t q[K];                               // q[s]: the packed frame K positions after x[s]
#pragma unroll
  for (int k = 0; k < K - 1; ++k) x[k] = unpack_pair<T>(fetch(first + k));
  q[K - 1] = fetch(first + K - 1);
#pragma unroll
  for (int k = 0; k < K - 1; ++k) q[k] = fetch(first + K + k);
  uint32_t* __restrict__ out = reinterpret_cast<uint32_t*>(static_cast<T*>(a.out) + out_row0 * C + c);
  const int t_end = min(OL, t0 + kRun);
#pragma unroll 1
  for (int base = t0; base < t_end; base += K) {
#pragma unroll
    for (int s = 0; s < K; ++s) {
      // output base + s: window frames (base + s - t0) + 0 .. K-1 from `first`; the newest one sits in slot (s + K - 1) % K
      const int slot = (s + K - 1) % K;
      x[slot] = unpack_pair<T>(q[slot]);
      q[slot] = fetch(first + (base - t0) + s + 2 * K - 1);
      float2 acc = bias;
#pragma unroll
      for (int k = 0; k < K; ++k) acc = __ffma2_rn(x[(s + k) % K], w[k], acc);
      if constexpr (kAct == 1) {
        const float2 h = __fmul2_rn(acc, make_float2(0.5f, 0.5f));
        acc = __ffma2_rn(h, make_float2(tanh_approx(h.x), tanh_approx(h.y)), h);
      } else if constexpr (kAct == 2) {
        acc.x = apply_act_fast(acc.x, a.act);
        acc.y = apply_act_fast(acc.y, a.act);
      }
      if (base + s < t_end) out[(base + s) * row_u32] = pack_pair<T>(acc.x, acc.y);
    }
  }
}

template <typename T, int K>
int launch_roll(const DwArgs& a, int max_out_len, cudaStream_t s) {
  if constexpr (sizeof(T) != 2) {
    return set_error(OASR_ERR_DTYPE, "depthwise_conv1d: rolling kernel is 16-bit only");
  } else {
    const int pairs = a.channels / 2;
    const int threads = pairs >= 128 ? 128 : ((pairs + 31) / 32) * 32;
    constexpr int kRun = kRollRuns * K;
    dim3 block(threads);
    dim3 grid((max_out_len + kRun - 1) / kRun, (pairs + threads - 1) / threads, static_cast<unsigned>(a.batch));
    const bool affine = a.post_scale != nullptr;
    const int act = a.act == OASR_ACT_NONE ? 0 : (a.act == OASR_ACT_SWISH ? 1 : 2);
    if (affine) {
      if (act == 1) launch_pdl(dwconv_roll_kernel<T, K, true, 1>, grid, block, 0, s, a);
      else if (act == 0) launch_pdl(dwconv_roll_kernel<T, K, true, 0>, grid, block, 0, s, a);
      else launch_pdl(dwconv_roll_kernel<T, K, true, 2>, grid, block, 0, s, a);
    } else {
      if (act == 1) launch_pdl(dwconv_roll_kernel<T, K, false, 1>, grid, block, 0, s, a);
      else if (act == 0) launch_pdl(dwconv_roll_kernel<T, K, false, 0>, grid, block, 0, s, a);
      else launch_pdl(dwconv_roll_kernel<T, K, false, 2>, grid, block, 0, s, a);
    }
    return check_launch("depthwise_conv1d (rolling) kernel launch");
  }
}

template <typename T, int K>
int launch_stream(const DwArgs& a, int max_out_len, cudaStream_t s) {
  if constexpr (sizeof(T) != 2) {
    return set_error(OASR_ERR_DTYPE, "depthwise_conv1d: streaming kernel is 16-bit only");
  } else {
    const int pairs = a.channels / 2;
    const int threads = pairs >= 256 ? 256 : ((pairs + 31) / 32) * 32;
    dim3 block(threads);
    dim3 grid((max_out_len + kST - 1) / kST, (pairs + threads - 1) / threads, static_cast<unsigned>(a.batch));
    const bool affine = a.post_scale != nullptr;
    const int act = a.act == OASR_ACT_NONE ? 0 : (a.act == OASR_ACT_SWISH ? 1 : 2);
    if (affine) {
      if (act == 1) launch_pdl(dwconv_stream_kernel<T, K, true, 1>, grid, block, 0, s, a);
      else if (act == 0) launch_pdl(dwconv_stream_kernel<T, K, true, 0>, grid, block, 0, s, a);
      else launch_pdl(dwconv_stream_kernel<T, K, true, 2>, grid, block, 0, s, a);
    } else {
      if (act == 1) launch_pdl(dwconv_stream_kernel<T, K, false, 1>, grid, block, 0, s, a);
      else if (act == 0) launch_pdl(dwconv_stream_kernel<T, K, false, 0>, grid, block, 0, s, a);
      else launch_pdl(dwconv_stream_kernel<T, K, false, 2>, grid, block, 0, s, a);
    }
    return check_launch("depthwise_conv1d (streaming) kernel launch");
  }
}

// Any kernel size / channel count, optional mask and add_input
// (include/oasr/conv/conv1d.cuh:23-113 semantics).  One thread per output element.
template <typename T>
__global__ void __launch_bounds__(256) dwconv_generic_kernel(DwArgs a) {
  const int C = a.channels;
  const int64_t total = a.batch * a.out_len * C;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const T* mask_t = static_cast<const T*>(a.mask);
  const uint8_t* mask_b = static_cast<const uint8_t*>(a.mask);
  auto mask_at = [&](int64_t b, int t) -> float {
    if (!a.mask) return 1.f;
    const int64_t i = b * a.seq_len + t;
    return a.mask_is_bool ? (mask_b[i] ? 1.f : 0.f) : Elem<T>::to_f(mask_t[i]);
  };
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int c = static_cast<int>(i % C);
    const int t = static_cast<int>((i / C) % a.out_len);
    const int64_t b = i / (static_cast<int64_t>(C) * a.out_len);
    const T* in = static_cast<const T*>(a.in) + b * a.seq_len * C + c;
    const T* w = static_cast<const T*>(a.weight) + c;
    float acc = 0.f;
    for (int k = 0; k < a.kernel_size; ++k) {
      const int ti = t - a.pad_left + k;
      if (ti < 0 || ti >= a.seq_len) continue;
      float v = Elem<T>::to_f(in[static_cast<int64_t>(ti) * C]);
      v *= mask_at(b, ti);
      acc = fmaf(v, Elem<T>::to_f(w[static_cast<int64_t>(k) * C]), acc);
    }
    if (a.bias) acc += Elem<T>::to_f(static_cast<const T*>(a.bias)[c]);
    if (a.post_scale) acc = fmaf(acc, a.post_scale[c], a.post_shift[c]);
    if (a.add_input) acc += Elem<T>::to_f(in[static_cast<int64_t>(t) * C]) * mask_at(b, t);
    if (a.mask) acc *= mask_at(b, t);
    acc = apply_act_rt(acc, a.act);
    static_cast<T*>(a.out)[i] = Elem<T>::from_f(acc);
  }
}

template <typename T, int K>
int launch_window(const DwArgs& a, int max_out_len, cudaStream_t s) {
  dim3 block(128);
  dim3 grid((a.channels / 2 + 127) / 128, (max_out_len + kTile - 1) / kTile, static_cast<unsigned>(a.batch));
  const bool affine = a.post_scale != nullptr;
  const bool act = a.act != OASR_ACT_NONE;
  if (affine && act) dwconv_window_kernel<T, K, true, true><<<grid, block, 0, s>>>(a);
  else if (affine) dwconv_window_kernel<T, K, true, false><<<grid, block, 0, s>>>(a);
  else if (act) dwconv_window_kernel<T, K, false, true><<<grid, block, 0, s>>>(a);
  else dwconv_window_kernel<T, K, false, false><<<grid, block, 0, s>>>(a);
  return check_launch("depthwise_conv1d kernel launch");
}

template <typename T>
int launch_dw(const DwArgs& a, int max_out_len, cudaStream_t s) {
  const bool plain = a.mask == nullptr && !a.add_input;
  const bool fast = plain && a.channels % 2 == 0 && is_aligned(a.in, 2 * sizeof(T)) &&
                    is_aligned(a.out, 2 * sizeof(T)) && is_aligned(a.weight, 2 * sizeof(T)) &&
                    (!a.bias || is_aligned(a.bias, 2 * sizeof(T))) && a.batch <= 65535 &&
                    (max_out_len + kTile - 1) / kTile <= 65535;
  const bool tiled = fast && (a.channels * sizeof(T)) % 16 == 0 && (a.channels % kCB == 0 || a.channels < kCB) &&
                     is_aligned(a.in, 16) && (max_out_len + kTT - 1) / kTT <= 65535 &&
                     (a.channels + kCB - 1) / kCB <= 65535;
  const bool stream = fast && sizeof(T) == 2 && is_aligned(a.in, 4) && is_aligned(a.out, 4) && is_aligned(a.weight, 4) &&
                      (!a.bias || is_aligned(a.bias, 4)) && (!a.post_scale || (is_aligned(a.post_scale, 8) && is_aligned(a.post_shift, 8))) &&
                      (max_out_len + kST - 1) / kST <= 65535 && a.kernel_size <= 15 && g_dw_path != 1;
  if (stream && g_dw_path == 2) {
    switch (a.kernel_size) {
      case 9: return launch_roll<T, 9>(a, max_out_len, s);
      case 15: return launch_roll<T, 15>(a, max_out_len, s);
      default: break;
    }
  }
  if (stream) {
    switch (a.kernel_size) {
      case 3: return launch_stream<T, 3>(a, max_out_len, s);
      case 5: return launch_stream<T, 5>(a, max_out_len, s);
      case 7: return launch_stream<T, 7>(a, max_out_len, s);
      case 9: return launch_stream<T, 9>(a, max_out_len, s);
      case 11: return launch_stream<T, 11>(a, max_out_len, s);
      case 15: return launch_stream<T, 15>(a, max_out_len, s);
      default: break;
    }
  }
  if (tiled) {
    switch (a.kernel_size) {
      case 3: return launch_tile<T, 3>(a, max_out_len, s);
      case 5: return launch_tile<T, 5>(a, max_out_len, s);
      case 7: return launch_tile<T, 7>(a, max_out_len, s);
      case 9: return launch_tile<T, 9>(a, max_out_len, s);
      case 11: return launch_tile<T, 11>(a, max_out_len, s);
      case 15: return launch_tile<T, 15>(a, max_out_len, s);
      case 31: return launch_tile<T, 31>(a, max_out_len, s);
      default: break;
    }
  }
  if (fast) {
    switch (a.kernel_size) {
      case 3: return launch_window<T, 3>(a, max_out_len, s);
      case 5: return launch_window<T, 5>(a, max_out_len, s);
      case 7: return launch_window<T, 7>(a, max_out_len, s);
      case 9: return launch_window<T, 9>(a, max_out_len, s);
      case 11: return launch_window<T, 11>(a, max_out_len, s);
      case 15: return launch_window<T, 15>(a, max_out_len, s);
      case 31: return launch_window<T, 31>(a, max_out_len, s);
      default: break;
    }
  }
  if (a.cu_seqlens) {
    return set_error(OASR_ERR_UNSUPPORTED,
                     "packed depthwise conv supports kernel sizes 3/5/7/9/11/15/31 and even channel counts");
  }
  int64_t total = a.batch * a.out_len * a.channels;
  int64_t g = (total + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  if (g > cap) g = cap;
  dwconv_generic_kernel<T><<<static_cast<unsigned>(g), 256, 0, s>>>(a);
  return check_launch("depthwise_conv1d (generic) kernel launch");
}

// ---------------------------------------------------------------------------
// Streaming causal conv with rolling state.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) causal_conv_kernel(T* __restrict__ out, const T* __restrict__ in,
                                                          const T* __restrict__ state,
                                                          const T* __restrict__ weight,  // (C, K)
                                                          const T* __restrict__ bias, int64_t batch,
                                                          int seq_len, int C, int K) {
  const int64_t total = batch * seq_len * C;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int SL = K - 1;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int c = static_cast<int>(i % C);
    const int t = static_cast<int>((i / C) % seq_len);
    const int64_t b = i / (static_cast<int64_t>(C) * seq_len);
    float acc = 0.f;
    for (int k = 0; k < K; ++k) {
      const int pos = t - SL + k;
      const float v = pos < 0 ? Elem<T>::to_f(state[(b * SL + (SL + pos)) * C + c])
                              : Elem<T>::to_f(in[(b * seq_len + pos) * C + c]);
      acc = fmaf(v, Elem<T>::to_f(weight[static_cast<int64_t>(c) * K + k]), acc);
    }
    if (bias) acc += Elem<T>::to_f(bias[c]);
    out[i] = Elem<T>::from_f(acc);
  }
}

// One thread owns one (batch, channel) column of the state and walks it in
// ascending order, so the in-place left shift reads every slot before it is
// overwritten.
template <typename T>
__global__ void __launch_bounds__(256) causal_state_update_kernel(T* __restrict__ state,
                                                                  const T* __restrict__ in, int64_t batch,
                                                                  int seq_len, int C, int SL) {
  const int64_t total = batch * C;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int c = static_cast<int>(i % C);
  const int64_t b = i / C;
  T* st = state + b * SL * C + c;
  const T* x = in + b * seq_len * C + c;
  if (seq_len >= SL) {
    for (int s = 0; s < SL; ++s) st[static_cast<int64_t>(s) * C] = x[static_cast<int64_t>(seq_len - SL + s) * C];
  } else {
    const int shift = SL - seq_len;
    for (int s = 0; s < shift; ++s) st[static_cast<int64_t>(s) * C] = st[static_cast<int64_t>(s + seq_len) * C];
    for (int s = shift; s < SL; ++s) st[static_cast<int64_t>(s) * C] = x[static_cast<int64_t>(s - shift) * C];
  }
}

// xcat[b] = [state[slot[b]] (SL rows) ; x[b] (T rows)], 16-byte pieces.
__global__ void __launch_bounds__(256) conv_state_concat_kernel(uint8_t* __restrict__ xcat,
                                                                const uint8_t* __restrict__ state,
                                                                const int64_t* __restrict__ slots,
                                                                const uint8_t* __restrict__ x, int64_t B, int SL, int T,
                                                                int64_t row_bytes, int64_t num_slots) {
  const int64_t pieces = row_bytes / 16;
  const int64_t total = B * (SL + T) * pieces;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t piece = i % pieces;
    const int64_t row = i / pieces;
    const int r = static_cast<int>(row % (SL + T));
    const int64_t b = row / (SL + T);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < SL) {
      const int64_t slot = slots[b];   // a slot id outside the buffer reads as an empty (zero) left context
      if (slot >= 0 && slot < num_slots) v = *reinterpret_cast<const uint4*>(state + (slot * SL + r) * row_bytes + piece * 16);
    } else {
      v = *reinterpret_cast<const uint4*>(x + (b * T + (r - SL)) * row_bytes + piece * 16);
    }
    *reinterpret_cast<uint4*>(xcat + row * row_bytes + piece * 16) = v;
  }
}
// state[slot[b]] = last SL rows of xcat[b] (read from xcat, so the update cannot race with itself).
__global__ void __launch_bounds__(256) conv_state_update_kernel(uint8_t* __restrict__ state,
                                                                const int64_t* __restrict__ slots,
                                                                const uint8_t* __restrict__ xcat, int64_t B, int SL,
                                                                int T, int64_t row_bytes, int64_t num_slots) {
  const int64_t pieces = row_bytes / 16;
  const int64_t total = B * SL * pieces;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t piece = i % pieces;
    const int64_t row = i / pieces;
    const int r = static_cast<int>(row % SL);
    const int64_t b = row / SL;
    const int64_t slot = slots[b];
    if (slot < 0 || slot >= num_slots) continue;   // never a write outside the state buffer
    *reinterpret_cast<uint4*>(state + (slot * SL + r) * row_bytes + piece * 16) =
        *reinterpret_cast<const uint4*>(xcat + (b * (SL + T) + T + r) * row_bytes + piece * 16);
  }
}

}  // namespace

}  // namespace ob

extern "C" {

int oasr_b200_conv_state_concat(void* xcat, void* state, int64_t num_slots, const int64_t* slot_ids, const void* x,
                                int64_t B, int64_t state_len, int64_t T, int64_t channels, int dtype, void* stream) {
  using namespace ob;
  OB_REQUIRE(B >= 0 && state_len >= 0 && T > 0 && channels > 0 && num_slots >= 0, OASR_ERR_INVALID,
             "conv_state_concat: bad shape");
  if (B == 0) return OASR_OK;
  OB_REQUIRE(xcat && state && slot_ids && x, OASR_ERR_INVALID, "conv_state_concat: null pointer argument");
  const int64_t es = dtype == OASR_DT_F32 ? 4 : 2;
  OB_REQUIRE(dtype == OASR_DT_F32 || dtype == OASR_DT_F16 || dtype == OASR_DT_BF16, OASR_ERR_DTYPE,
             "conv_state_concat: unsupported dtype id %d", dtype);
  const int64_t row_bytes = channels * es;
  OB_REQUIRE(row_bytes % 16 == 0 && is_aligned(xcat, 16) && is_aligned(state, 16) && is_aligned(x, 16), OASR_ERR_ALIGN,
             "conv_state_concat: rows must be multiples of 16 bytes and 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  int64_t g = (B * (state_len + T) * (row_bytes / 16) + 255) / 256;
  if (g > cap) g = cap;
  conv_state_concat_kernel<<<static_cast<unsigned>(g), 256, 0, s>>>(
      static_cast<uint8_t*>(xcat), static_cast<const uint8_t*>(state), slot_ids, static_cast<const uint8_t*>(x), B,
      (int)state_len, (int)T, row_bytes, num_slots);
  if (int rc = check_launch("conv_state_concat launch")) return rc;
  if (state_len == 0) return OASR_OK;
  g = (B * state_len * (row_bytes / 16) + 255) / 256;
  if (g > cap) g = cap;
  conv_state_update_kernel<<<static_cast<unsigned>(g), 256, 0, s>>>(static_cast<uint8_t*>(state), slot_ids,
                                                                   static_cast<const uint8_t*>(xcat), B, (int)state_len,
                                                                   (int)T, row_bytes, num_slots);
  return check_launch("conv_state_update launch");
}

int oasr_b200_depthwise_conv1d_affine(void* out, const void* in, const void* weight, const void* bias,
                                      const float* post_scale, const float* post_shift, int64_t batch,
                                      int64_t seq_len, int64_t channels, int64_t kernel_size, int64_t pad_left,
                                      int64_t pad_right, int activation, int dtype, void* stream) {
  using namespace ob;
  OB_REQUIRE(batch >= 0 && seq_len >= 0 && channels > 0 && kernel_size > 0 && pad_left >= 0 && pad_right >= 0,
             OASR_ERR_INVALID, "depthwise_conv1d_affine: bad shape");
  const int64_t out_len = seq_len + pad_left + pad_right - kernel_size + 1;
  OB_REQUIRE(out_len > 0, OASR_ERR_INVALID, "depthwise_conv1d_affine has invalid output length %lld", (long long)out_len);
  if (batch == 0) return OASR_OK;
  OB_REQUIRE(out && in && weight, OASR_ERR_INVALID, "depthwise_conv1d_affine: null pointer argument");
  OB_REQUIRE((post_scale == nullptr) == (post_shift == nullptr), OASR_ERR_INVALID,
             "depthwise_conv1d_affine: post_scale and post_shift go together");
  OB_REQUIRE(act_is_known(activation), OASR_ERR_INVALID, "depthwise_conv1d_affine: unknown activation id %d", activation);
  DwArgs a{};
  a.out = out; a.in = in; a.weight = weight; a.bias = bias; a.post_scale = post_scale; a.post_shift = post_shift;
  a.batch = batch; a.seq_len = (int)seq_len; a.out_len = (int)out_len; a.channels = (int)channels;
  a.kernel_size = (int)kernel_size; a.pad_left = (int)pad_left; a.act = activation;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return OB_DISPATCH_FLOAT(dtype, T, [&]() -> int { return launch_dw<T>(a, (int)out_len, s); });
}

int oasr_b200_depthwise_conv1d_packed(void* out, const void* in, const void* weight, const void* bias,
                                      const float* post_scale, const float* post_shift, const float* right_fill,
                                      const int32_t* fill_frames, const int32_t* cu_seqlens, int64_t num_segs,
                                      int64_t max_seg_len, int64_t channels, int64_t kernel_size, int activation,
                                      int dtype, void* stream) {
  using namespace ob;
  OB_REQUIRE(num_segs >= 0 && max_seg_len >= 0 && channels > 0 && kernel_size > 0, OASR_ERR_INVALID,
             "depthwise_conv1d_packed: bad shape");
  if (num_segs == 0 || max_seg_len == 0) return OASR_OK;
  OB_REQUIRE(out && in && weight && cu_seqlens, OASR_ERR_INVALID, "depthwise_conv1d_packed: null pointer argument");
  OB_REQUIRE(kernel_size % 2 == 1, OASR_ERR_INVALID, "depthwise_conv1d_packed needs an odd kernel size");
  OB_REQUIRE((post_scale == nullptr) == (post_shift == nullptr), OASR_ERR_INVALID,
             "depthwise_conv1d_packed: post_scale and post_shift go together");
  OB_REQUIRE((right_fill == nullptr) == (fill_frames == nullptr), OASR_ERR_INVALID,
             "depthwise_conv1d_packed: right_fill and fill_frames go together");
  OB_REQUIRE(act_is_known(activation), OASR_ERR_INVALID, "depthwise_conv1d_packed: unknown activation id %d", activation);
  DwArgs a{};
  a.out = out; a.in = in; a.weight = weight; a.bias = bias;
  a.post_scale = post_scale; a.post_shift = post_shift; a.cu_seqlens = cu_seqlens;
  a.right_fill = right_fill; a.fill_frames = fill_frames;
  a.batch = num_segs; a.channels = (int)channels;
  a.kernel_size = (int)kernel_size; a.pad_left = ((int)kernel_size - 1) / 2; a.act = activation;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return OB_DISPATCH_FLOAT(dtype, T, [&]() -> int { return launch_dw<T>(a, (int)max_seg_len, s); });
}

int oasr_b200_depthwise_conv1d_packed_causal(void* out, const void* in, const void* weight, const void* bias,
                                             const int32_t* cu_seqlens, int64_t num_segs, int64_t max_seg_len,
                                             int64_t channels, int64_t kernel_size, int activation, int dtype,
                                             void* stream) {
  using namespace ob;
  OB_REQUIRE(num_segs >= 0 && max_seg_len >= 0 && channels > 0 && kernel_size > 0, OASR_ERR_INVALID,
             "depthwise_conv1d_packed_causal: bad shape");
  if (num_segs == 0 || max_seg_len == 0) return OASR_OK;
  OB_REQUIRE(out && in && weight && cu_seqlens, OASR_ERR_INVALID,
             "depthwise_conv1d_packed_causal: null pointer argument");
  OB_REQUIRE(act_is_known(activation), OASR_ERR_INVALID, "depthwise_conv1d_packed_causal: unknown activation id %d",
             activation);
  DwArgs a{};
  a.out = out; a.in = in; a.weight = weight; a.bias = bias; a.cu_seqlens = cu_seqlens;
  a.batch = num_segs; a.channels = (int)channels;
  a.kernel_size = (int)kernel_size; a.pad_left = (int)kernel_size - 1; a.act = activation;   // all padding on the left
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return OB_DISPATCH_FLOAT(dtype, T, [&]() -> int { return launch_dw<T>(a, (int)max_seg_len, s); });
}

int oasr_b200_depthwise_conv1d(void* out, const void* in, const void* weight, const void* bias,
                               int64_t batch, int64_t seq_len, int64_t channels, int64_t kernel_size,
                               int64_t pad_left, int64_t pad_right, const void* mask, int mask_is_bool,
                               int add_input, int activation, int dtype, void* stream) {
  using namespace ob;
  OB_REQUIRE(batch == 0 || (out && in && weight), OASR_ERR_INVALID, "depthwise_conv1d: null pointer argument");
  OB_REQUIRE(batch >= 0 && seq_len >= 0 && channels > 0 && kernel_size > 0 && pad_left >= 0 && pad_right >= 0,
             OASR_ERR_INVALID, "depthwise_conv1d: bad shape");
  OB_REQUIRE(channels < (1 << 24) && seq_len < (1 << 30) && kernel_size < (1 << 16), OASR_ERR_INVALID,
             "depthwise_conv1d: extent too large");
  const int64_t out_len = seq_len + pad_left + pad_right - kernel_size + 1;
  OB_REQUIRE(out_len > 0, OASR_ERR_INVALID, "depthwise_conv1d has invalid output length %lld", (long long)out_len);
  OB_REQUIRE(!(mask || add_input) || out_len == seq_len, OASR_ERR_INVALID,
             "depthwise_conv1d: mask / add_input need out_len == seq_len");
  OB_REQUIRE(activation == OASR_ACT_NONE || activation == OASR_ACT_SWISH, OASR_ERR_INVALID,
             "depthwise_conv1d: activation must be none or swish");
  if (batch == 0) return OASR_OK;
  DwArgs a{};
  a.out = out; a.in = in; a.weight = weight; a.bias = bias;
  a.batch = batch; a.seq_len = (int)seq_len; a.out_len = (int)out_len; a.channels = (int)channels;
  a.kernel_size = (int)kernel_size; a.pad_left = (int)pad_left; a.act = activation;
  a.mask = mask; a.mask_is_bool = mask_is_bool; a.add_input = add_input;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return OB_DISPATCH_FLOAT(dtype, T, [&]() -> int { return launch_dw<T>(a, (int)out_len, s); });
}

int oasr_b200_causal_conv1d(void* out, const void* in, void* state, const void* weight, const void* bias,
                            int64_t batch, int64_t seq_len, int64_t channels, int64_t kernel_size, int dtype,
                            void* stream) {
  using namespace ob;
  OB_REQUIRE(out && in && state && weight, OASR_ERR_INVALID, "causal_conv1d: null pointer argument");
  OB_REQUIRE(batch >= 0 && seq_len > 0 && channels > 0 && kernel_size > 1, OASR_ERR_INVALID,
             "causal_conv1d: bad shape");
  if (batch == 0) return OASR_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return OB_DISPATCH_FLOAT(dtype, T, [&]() -> int {
    const int64_t total = batch * seq_len * channels;
    int64_t g = (total + 255) / 256;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
    if (g > cap) g = cap;
    causal_conv_kernel<T><<<static_cast<unsigned>(g), 256, 0, s>>>(
        static_cast<T*>(out), static_cast<const T*>(in), static_cast<const T*>(state),
        static_cast<const T*>(weight), static_cast<const T*>(bias), batch, (int)seq_len, (int)channels,
        (int)kernel_size);
    if (int rc = check_launch("causal_conv1d kernel launch")) return rc;
    const int64_t cols = batch * channels;
    causal_state_update_kernel<T><<<static_cast<unsigned>((cols + 255) / 256), 256, 0, s>>>(
        static_cast<T*>(state), static_cast<const T*>(in), batch, (int)seq_len, (int)channels,
        (int)kernel_size - 1);
    return check_launch("causal_conv1d state update launch");
  });
}

}  // extern "C"
