// Row normalisation kernels: LayerNorm / RMSNorm with optional fused residual
// add, optional activation, and inference BatchNorm over channels-last rows.
//
// HBM-bound.  Fast path: one warp owns one row, the whole row lives in
// registers (one global read, one global write), statistics by warp shuffles,
// 128-bit coalesced accesses (lane l of chunk c touches elements
// [(c*32+l)*8, +8)).  Algorithmic bytes per row of width H in a 16-bit type:
// LN 4H, add+LN+residual 8H (include/oasr/norm.cuh:28-93,396-484 in the
// reference make 3-4 passes over the row from global memory instead).
#include <cuda_fp8.h>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace ob {
namespace {

constexpr int kGran = 8;  // elements per lane per chunk

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&f)[kGran]) {
  if constexpr (sizeof(T) == 4) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
    f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  } else {
    Pack<T> v = ld128(p);
#pragma unroll
    for (int i = 0; i < kGran; ++i) f[i] = Elem<T>::to_f(v.v[i]);
  }
}
template <typename T>
__device__ __forceinline__ void load8_param(const T* p, float (&f)[kGran]) {
  if constexpr (sizeof(T) == 4) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p));
    const float4 b = __ldg(reinterpret_cast<const float4*>(p + 4));
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
    f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  } else {
    Pack<T> v = ld128_nc(p);
#pragma unroll
    for (int i = 0; i < kGran; ++i) f[i] = Elem<T>::to_f(v.v[i]);
  }
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&f)[kGran]) {
  if constexpr (sizeof(T) == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
  } else {
    Pack<T> v;
#pragma unroll
    for (int i = 0; i < kGran; ++i) v.v[i] = Elem<T>::from_f(f[i]);
    st128(p, v);
  }
}

struct NormArgs {
  void* out;
  void* res_out;      // nullable
  const void* in;
  const void* res;    // nullable
  const void* weight;
  const void* bias;   // nullable
  int64_t rows;
  int hidden;
  float eps;
  float alpha;
  int act;
};

// TIn: type of in/residual; TOut: type of out/res_out; TW: type of weight/bias.
template <typename TIn, typename TOut, typename TW, int kChunks, bool kRms, bool kAdd, bool kAct>
__global__ void __launch_bounds__(128) norm_warp_rows_kernel(NormArgs a) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= a.rows) return;
  const int H = a.hidden;
  const TIn* in = static_cast<const TIn*>(a.in) + row * H;
  const TIn* res = kAdd ? static_cast<const TIn*>(a.res) + row * H : nullptr;
  TOut* out = static_cast<TOut*>(a.out) + row * H;
  TOut* res_out = (kAdd && a.res_out) ? static_cast<TOut*>(a.res_out) + row * H : nullptr;

  float x[kChunks][kGran];
  float sum = 0.f;
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    const int e = (c * 32 + lane) * kGran;
    if (e < H) {
      load8(in + e, x[c]);
      if constexpr (kAdd) {
        float r[kGran];
        load8(res + e, r);
#pragma unroll
        for (int i = 0; i < kGran; ++i) x[c][i] = fmaf(a.alpha, x[c][i], r[i]);
        if (res_out) store8(res_out + e, x[c]);
      }
#pragma unroll
      for (int i = 0; i < kGran; ++i) sum += kRms ? x[c][i] * x[c][i] : x[c][i];
    } else {
#pragma unroll
      for (int i = 0; i < kGran; ++i) x[c][i] = 0.f;
    }
  }
  sum = warp_sum(sum);
  float mean = 0.f, rstd;
  if constexpr (kRms) {
    rstd = rsqrtf(sum / H + a.eps);
  } else {
    mean = sum / H;
    float sq = 0.f;
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
      const int e = (c * 32 + lane) * kGran;
      if (e < H) {
#pragma unroll
        for (int i = 0; i < kGran; ++i) {
          const float d = x[c][i] - mean;
          sq = fmaf(d, d, sq);
        }
      }
    }
    sq = warp_sum(sq);
    rstd = rsqrtf(sq / H + a.eps);
  }
  const TW* w = static_cast<const TW*>(a.weight);
  const TW* b = static_cast<const TW*>(a.bias);
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    const int e = (c * 32 + lane) * kGran;
    if (e < H) {
      float g[kGran], y[kGran];
      load8_param(w + e, g);
#pragma unroll
      for (int i = 0; i < kGran; ++i) y[i] = (x[c][i] - mean) * rstd * g[i];
      if (b) {
        float bb[kGran];
        load8_param(b + e, bb);
#pragma unroll
        for (int i = 0; i < kGran; ++i) y[i] += bb[i];
      }
      if constexpr (kAct) {
#pragma unroll
        for (int i = 0; i < kGran; ++i) y[i] = apply_act_rt(y[i], a.act);
      }
      store8(out + e, y);
    }
  }
}

// Any width: one block per row, scalar accesses, row re-read from global.
template <typename TIn, typename TOut, typename TW, bool kRms, bool kAdd, bool kAct>
__global__ void __launch_bounds__(256) norm_block_rows_kernel(NormArgs a) {
  __shared__ float red[33];
  const int64_t row = blockIdx.x;
  const int H = a.hidden;
  const TIn* in = static_cast<const TIn*>(a.in) + row * H;
  const TIn* res = kAdd ? static_cast<const TIn*>(a.res) + row * H : nullptr;
  TOut* out = static_cast<TOut*>(a.out) + row * H;
  TOut* res_out = (kAdd && a.res_out) ? static_cast<TOut*>(a.res_out) + row * H : nullptr;
  auto value = [&](int i) -> float {
    float v = Elem<TIn>::to_f(in[i]);
    if constexpr (kAdd) v = fmaf(a.alpha, v, Elem<TIn>::to_f(res[i]));
    return v;
  };
  float s = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = value(i);
    s += kRms ? v * v : v;
  }
  s = block_sum(s, red);
  float mean = 0.f, rstd;
  if constexpr (kRms) {
    rstd = rsqrtf(s / H + a.eps);
  } else {
    mean = s / H;
    float sq = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      const float d = value(i) - mean;
      sq = fmaf(d, d, sq);
    }
    sq = block_sum(sq, red);
    rstd = rsqrtf(sq / H + a.eps);
  }
  const TW* w = static_cast<const TW*>(a.weight);
  const TW* b = static_cast<const TW*>(a.bias);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = value(i);
    float y = (v - mean) * rstd * Elem<TW>::to_f(w[i]);
    if (b) y += Elem<TW>::to_f(b[i]);
    if constexpr (kAct) y = apply_act_rt(y, a.act);
    // The sum is written after every read of in/res at this index by this
    // thread, so res_out may alias in or res.
    if (res_out) res_out[i] = Elem<TOut>::from_f(v);
    out[i] = Elem<TOut>::from_f(y);
  }
}

template <typename TIn, typename TOut, typename TW, bool kRms, bool kAdd, bool kAct>
int launch_norm(const NormArgs& a, cudaStream_t stream) {
  if (a.rows == 0) return OASR_OK;
  const int H = a.hidden;
  const bool fast = (H % kGran == 0) && H <= 16 * 32 * kGran && is_aligned(a.in, 16) &&
                    is_aligned(a.out, 16) && is_aligned(a.weight, 16) &&
                    (!a.bias || is_aligned(a.bias, 16)) && (!a.res || is_aligned(a.res, 16)) &&
                    (!a.res_out || is_aligned(a.res_out, 16));
  if (fast) {
    const int packs = H / kGran;
    const int chunks = (packs + 31) / 32;
    const int warps = 4;
    const unsigned grid = static_cast<unsigned>((a.rows + warps - 1) / warps);
#define OB_NORM_CASE(C)                                                                          \
  norm_warp_rows_kernel<TIn, TOut, TW, C, kRms, kAdd, kAct><<<grid, warps * 32, 0, stream>>>(a)
    if (chunks <= 1) OB_NORM_CASE(1);
    else if (chunks <= 2) OB_NORM_CASE(2);
    else if (chunks <= 4) OB_NORM_CASE(4);
    else if (chunks <= 8) OB_NORM_CASE(8);
    else OB_NORM_CASE(16);
#undef OB_NORM_CASE
  } else {
    norm_block_rows_kernel<TIn, TOut, TW, kRms, kAdd, kAct>
        <<<static_cast<unsigned>(a.rows), 256, 0, stream>>>(a);
  }
  return check_launch("norm kernel launch");
}

int validate_norm(const void* out, const void* in, const void* weight, int64_t rows, int64_t hidden,
                  int act) {
  OB_REQUIRE(rows == 0 || (out && in && weight), OASR_ERR_INVALID, "norm: null pointer argument");
  OB_REQUIRE(rows >= 0 && hidden > 0, OASR_ERR_INVALID, "norm: bad shape rows=%lld hidden=%lld",
             (long long)rows, (long long)hidden);
  OB_REQUIRE(hidden <= (1 << 24), OASR_ERR_INVALID, "norm: hidden=%lld is too large", (long long)hidden);
  OB_REQUIRE(rows < (int64_t(1) << 31), OASR_ERR_INVALID, "norm: rows=%lld is too large", (long long)rows);
  OB_REQUIRE(act_is_known(act), OASR_ERR_INVALID, "norm: unknown activation id %d", act);
  return OASR_OK;
}

template <bool kRms>
int norm_entry(void* out, void* res_out, const void* in, const void* res, const void* weight,
               const void* bias, int64_t rows, int64_t hidden, double eps, double alpha, int act,
               int dtype, bool add, void* stream) {
  if (int rc = validate_norm(out, in, weight, rows, hidden, act)) return rc;
  if (add) OB_REQUIRE(rows == 0 || res != nullptr, OASR_ERR_INVALID, "add-norm: residual pointer is null");
  NormArgs a{out, res_out, in, res, weight, bias, rows, (int)hidden, (float)eps, (float)alpha, act};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return OB_DISPATCH_FLOAT(dtype, T, [&]() -> int {
    if (add) {
      if (act != OASR_ACT_NONE) return launch_norm<T, T, T, kRms, true, true>(a, s);
      return launch_norm<T, T, T, kRms, true, false>(a, s);
    }
    if (act != OASR_ACT_NONE) return launch_norm<T, T, T, kRms, false, true>(a, s);
    return launch_norm<T, T, T, kRms, false, false>(a, s);
  });
}

// ---------------------------------------------------------------------------
// BatchNorm (inference) over channels-last rows.
// ---------------------------------------------------------------------------
struct BnArgs {
  void* out;
  const void* in;
  const void *w, *b, *mean, *var;
  int64_t rows;
  int channels;
  float eps;
  int act;
};

// Each thread keeps one 8-channel column group for the whole kernel, so the
// per-channel scale/shift are computed once per thread.
template <typename T, bool kAct>
__global__ void __launch_bounds__(256) batch_norm_vec_kernel(BnArgs a) {
  const int ppr = a.channels / kGran;  // packs per row
  const int64_t total = a.rows * ppr;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;  // multiple of ppr
  if (tid >= total) return;
  const int c0 = static_cast<int>(tid % ppr) * kGran;
  float g[kGran], bb[kGran], mu[kGran], vv[kGran], scale[kGran], shift[kGran];
  load8_param(static_cast<const T*>(a.w) + c0, g);
  load8_param(static_cast<const T*>(a.b) + c0, bb);
  load8_param(static_cast<const T*>(a.mean) + c0, mu);
  load8_param(static_cast<const T*>(a.var) + c0, vv);
#pragma unroll
  for (int i = 0; i < kGran; ++i) {
    scale[i] = g[i] * rsqrtf(vv[i] + a.eps);
    shift[i] = bb[i] - mu[i] * scale[i];
  }
  const T* in = static_cast<const T*>(a.in);
  T* out = static_cast<T*>(a.out);
  for (int64_t p = tid; p < total; p += nthreads) {
    float x[kGran];
    load8(in + p * kGran, x);
#pragma unroll
    for (int i = 0; i < kGran; ++i) {
      x[i] = fmaf(x[i], scale[i], shift[i]);
      if constexpr (kAct) x[i] = apply_act_rt(x[i], a.act);
    }
    store8(out + p * kGran, x);
  }
}

template <typename T, bool kAct>
__global__ void __launch_bounds__(256) batch_norm_scalar_kernel(BnArgs a) {
  const int64_t total = a.rows * a.channels;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += nthreads) {
    const int c = static_cast<int>(i % a.channels);
    const float scale = Elem<T>::to_f(static_cast<const T*>(a.w)[c]) *
                        rsqrtf(Elem<T>::to_f(static_cast<const T*>(a.var)[c]) + a.eps);
    float y = (Elem<T>::to_f(static_cast<const T*>(a.in)[i]) - Elem<T>::to_f(static_cast<const T*>(a.mean)[c])) * scale +
              Elem<T>::to_f(static_cast<const T*>(a.b)[c]);
    if constexpr (kAct) y = apply_act_rt(y, a.act);
    static_cast<T*>(a.out)[i] = Elem<T>::from_f(y);
  }
}

int64_t gcd64(int64_t x, int64_t y) {
  while (y) { int64_t t = x % y; x = y; y = t; }
  return x;
}

template <typename T, bool kAct>
int launch_bn(const BnArgs& a, cudaStream_t s) {
  if (a.rows == 0) return OASR_OK;
  const bool fast = a.channels % kGran == 0 && is_aligned(a.in, 16) && is_aligned(a.out, 16) &&
                    is_aligned(a.w, 16) && is_aligned(a.b, 16) && is_aligned(a.mean, 16) &&
                    is_aligned(a.var, 16);
  const int block = 256;
  if (fast) {
    const int64_t ppr = a.channels / kGran;
    const int64_t total = a.rows * ppr;
    // grid*block must be a multiple of ppr so that a thread's column is fixed.
    const int64_t unit = ppr / gcd64(ppr, block);  // grid must be a multiple of this
    int64_t want = (total + block - 1) / block;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
    if (want > cap) want = cap;
    int64_t grid = ((want + unit - 1) / unit) * unit;
    batch_norm_vec_kernel<T, kAct><<<static_cast<unsigned>(grid), block, 0, s>>>(a);
  } else {
    int64_t grid = (a.rows * a.channels + block - 1) / block;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
    if (grid > cap) grid = cap;
    batch_norm_scalar_kernel<T, kAct><<<static_cast<unsigned>(grid), block, 0, s>>>(a);
  }
  return check_launch("batch_norm kernel launch");
}

// ---------------------------------------------------------------------------
// Residual-stream step of the fused encoder layer.  The residual stream is
// fp32; sub-layer outputs and normalised activations are 16-bit:
//   s = res_in + alpha * y                                (fp32; y nullable)
//   mode 0:  res_out = s,          h = LN_a(s)
//   mode 1:  res_out = s,          h = s * scale_a + shift_a     (folded inference BatchNorm)
//   mode 2:  res_out = LN_a(s),    h = LN_b(res_out)             (layer tail: norm_final, then the
//                                                                 next layer's first pre-norm)
// One warp per row, the row stays in registers (12*H bytes of traffic per row
// for a 16-bit y: 4H + 2H read, 4H + 2H written).
// ---------------------------------------------------------------------------
struct AddNormArgs {
  void* h_out;          // T
  float* res_out;       // nullable (mode 0/1: sum is not kept)
  const float* res_in;
  const void* y;        // T, nullable
  float alpha;
  const void *w_a, *b_a;        // T (LN) ; mode 1: fp32 scale / shift
  const void *w_b, *b_b;        // T (mode 2)
  int64_t rows;
  int hidden;
  float eps;
  int split_out;        // h rows are [hi | lo] (2*hidden wide): x = hi + lo with both parts 16-bit
  uint8_t* q_out;       // nullable: the h row once more in 8 bits, quantised per row exactly as quantize_rows(h) would
  float* q_scale;       // its row scales
  int q_kind;           // OASR_Q8_FP8_E4M3 / OASR_Q8_INT8
};

// The per-token quantisation of the row of h this warp has just produced: `v` holds the lane's final values (before
// their rounding to T); scale = amax(|round_T(v)|) / qmax and q = cvt(round_T(v) / scale), the arithmetic of
// quantize_rows_kernel (quant.cu) on the stored 16-bit row, so the two routes give the same bytes.
template <typename T, int kChunks>
__device__ __forceinline__ void quantise_row(const AddNormArgs& a, int64_t row, int lane, float (&v)[kChunks][kGran]) {
  const int H = a.hidden;
  float amax = 0.f;
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    if ((c * 32 + lane) * kGran < H) {
#pragma unroll
      for (int i = 0; i < kGran; ++i) {
        v[c][i] = Elem<T>::to_f(Elem<T>::from_f(v[c][i]));
        amax = fmaxf(amax, fabsf(v[c][i]));
      }
    }
  }
  amax = warp_max(amax);
  const float qmax = a.q_kind == OASR_Q8_FP8_E4M3 ? 448.f : 127.f;
  const float sc = amax > 0.f ? amax / qmax : 1.f;
  const float inv = 1.f / sc;
  if (lane == 0) a.q_scale[row] = sc;
  uint8_t* qr = a.q_out + row * H;
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    const int e = (c * 32 + lane) * kGran;
    if (e < H) {
      uint32_t w[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t packed = 0;
#pragma unroll
        for (int i = 0; i < 4; i += 2) {
          const float x0 = v[c][h * 4 + i] * inv, x1 = v[c][h * 4 + i + 1] * inv;
          uint32_t two;
          if (a.q_kind == OASR_Q8_FP8_E4M3) {
            two = __nv_cvt_float2_to_fp8x2(make_float2(x0, x1), __NV_SATFINITE, __NV_E4M3);
          } else {
            const int ia = max(-127, min(127, __float2int_rn(x0))), ib = max(-127, min(127, __float2int_rn(x1)));
            two = (static_cast<uint32_t>(ia) & 0xffu) | ((static_cast<uint32_t>(ib) & 0xffu) << 8);
          }
          packed |= two << (8 * i);
        }
        w[h] = packed;
      }
      *reinterpret_cast<uint2*>(qr + e) = make_uint2(w[0], w[1]);
    }
  }
}

// h row stride and the split store: hi = round(x), lo = round(x - hi).
template <typename T>
__device__ __forceinline__ void store_h(T* h, int e, int H, const float (&v)[kGran], bool split) {
  if (!split) {
    store8(h + e, v);
    return;
  }
  float hi[kGran], lo[kGran];
#pragma unroll
  for (int i = 0; i < kGran; ++i) {
    hi[i] = Elem<T>::to_f(Elem<T>::from_f(v[i]));
    lo[i] = v[i] - hi[i];
  }
  store8(h + e, hi);
  store8(h + H + e, lo);
}

template <int kChunks>
__device__ __forceinline__ void row_layer_norm(float (&x)[kChunks][kGran], int H, int lane, float eps) {
  float sum = 0.f;
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    if ((c * 32 + lane) * kGran < H) {
#pragma unroll
      for (int i = 0; i < kGran; ++i) sum += x[c][i];
    }
  }
  const float mean = warp_sum(sum) / H;
  float sq = 0.f;
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    if ((c * 32 + lane) * kGran < H) {
#pragma unroll
      for (int i = 0; i < kGran; ++i) {
        const float d = x[c][i] - mean;
        sq = fmaf(d, d, sq);
      }
    }
  }
  const float rstd = rsqrtf(warp_sum(sq) / H + eps);
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
#pragma unroll
    for (int i = 0; i < kGran; ++i) x[c][i] = (x[c][i] - mean) * rstd;
  }
}

template <typename T, int kChunks, int kMode>
__global__ void __launch_bounds__(128) add_norm_f32_kernel(AddNormArgs a) {
  ptx::grid_dep_launch();   // no-ops unless launched with programmatic stream serialisation
  ptx::grid_dep_wait();
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= a.rows) return;
  const int H = a.hidden;
  const float* res = a.res_in ? a.res_in + row * H : nullptr;
  const T* y = a.y ? static_cast<const T*>(a.y) + row * H : nullptr;
  float x[kChunks][kGran];
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    const int e = (c * 32 + lane) * kGran;
    if (e < H) {
      if (res) {
        load8(res + e, x[c]);
      } else {
#pragma unroll
        for (int i = 0; i < kGran; ++i) x[c][i] = 0.f;
      }
      if (y) {
        float yy[kGran];
        load8(y + e, yy);
#pragma unroll
        for (int i = 0; i < kGran; ++i) x[c][i] = fmaf(a.alpha, yy[i], x[c][i]);
      }
      if (kMode != 2 && a.res_out) store8(a.res_out + row * H + e, x[c]);
    } else {
#pragma unroll
      for (int i = 0; i < kGran; ++i) x[c][i] = 0.f;
    }
  }
  const bool split = a.split_out != 0;
  T* h = static_cast<T*>(a.h_out) + row * H * (split ? 2 : 1);
  if constexpr (kMode == 1) {
    const float* sc = static_cast<const float*>(a.w_a);
    const float* sh = static_cast<const float*>(a.b_a);
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
      const int e = (c * 32 + lane) * kGran;
      if (e < H) {
        float s8[kGran], t8[kGran];
        load8_param(sc + e, s8);
        load8_param(sh + e, t8);
#pragma unroll
        for (int i = 0; i < kGran; ++i) x[c][i] = fmaf(x[c][i], s8[i], t8[i]);
        store_h(h, e, H, x[c], split);
      }
    }
    if (a.q_out) quantise_row<T, kChunks>(a, row, lane, x);
    return;
  } else {
    row_layer_norm<kChunks>(x, H, lane, a.eps);
    const T* w = static_cast<const T*>(a.w_a);
    const T* b = static_cast<const T*>(a.b_a);
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
      const int e = (c * 32 + lane) * kGran;
      if (e < H) {
        float g[kGran], bb[kGran];
        load8_param(w + e, g);
        load8_param(b + e, bb);
#pragma unroll
        for (int i = 0; i < kGran; ++i) x[c][i] = fmaf(x[c][i], g[i], bb[i]);
        if constexpr (kMode == 0) store_h(h, e, H, x[c], split);
        else store8(a.res_out + row * H + e, x[c]);
      }
    }
    if constexpr (kMode == 2) {
      row_layer_norm<kChunks>(x, H, lane, a.eps);
      const T* w2 = static_cast<const T*>(a.w_b);
      const T* b2 = static_cast<const T*>(a.b_b);
#pragma unroll
      for (int c = 0; c < kChunks; ++c) {
        const int e = (c * 32 + lane) * kGran;
        if (e < H) {
          float g[kGran], bb[kGran];
          load8_param(w2 + e, g);
          load8_param(b2 + e, bb);
#pragma unroll
          for (int i = 0; i < kGran; ++i) x[c][i] = fmaf(x[c][i], g[i], bb[i]);
          store_h(h, e, H, x[c], split);
        }
      }
    }
    if (a.q_out) quantise_row<T, kChunks>(a, row, lane, x);
  }
}

template <typename T, int kMode>
int launch_add_norm(const AddNormArgs& a, cudaStream_t s) {
  const int chunks = (a.hidden / kGran + 31) / 32;
  const int warps = 4;
  const unsigned grid = static_cast<unsigned>((a.rows + warps - 1) / warps);
#define OB_AN_CASE(C) launch_pdl(add_norm_f32_kernel<T, C, kMode>, dim3(grid), dim3(warps * 32), 0, s, a)
  if (chunks <= 1) OB_AN_CASE(1);
  else if (chunks <= 2) OB_AN_CASE(2);
  else if (chunks <= 4) OB_AN_CASE(4);
  else OB_AN_CASE(8);
#undef OB_AN_CASE
  return check_launch("add_norm_f32 launch");
}

}  // namespace

}  // namespace ob

extern "C" {

int oasr_b200_add_norm_f32(void* h_out, float* res_out, const float* res_in, const void* y, double alpha, int mode,
                           const void* w_a, const void* b_a, const void* w_b, const void* b_b, int64_t rows,
                           int64_t hidden, double eps, int split_out, int dtype, void* stream) {
  return oasr_b200_add_norm_f32_q8(h_out, res_out, res_in, y, alpha, mode, w_a, b_a, w_b, b_b, rows, hidden, eps, split_out,
                                   nullptr, nullptr, 0, dtype, stream);
}

int oasr_b200_add_norm_f32_q8(void* h_out, float* res_out, const float* res_in, const void* y, double alpha, int mode,
                              const void* w_a, const void* b_a, const void* w_b, const void* b_b, int64_t rows,
                              int64_t hidden, double eps, int split_out, void* q_out, float* q_scale, int q_kind,
                              int dtype, void* stream) {
  using namespace ob;
  OB_REQUIRE(!q_out || (q_scale && (q_kind == OASR_Q8_FP8_E4M3 || q_kind == OASR_Q8_INT8) && !split_out && is_aligned(q_out, 16)),
             OASR_ERR_INVALID, "add_norm_f32_q8: the 8-bit output needs its scales, a kind of 1 (fp8 e4m3) or 2 (int8), 16-byte alignment and split_out = 0");
  OB_REQUIRE(rows >= 0 && hidden > 0, OASR_ERR_INVALID, "add_norm_f32: bad shape");
  if (rows == 0) return OASR_OK;
  OB_REQUIRE(h_out && (res_in || y) && w_a && b_a, OASR_ERR_INVALID, "add_norm_f32: null pointer argument");
  OB_REQUIRE(mode >= 0 && mode <= 2, OASR_ERR_INVALID, "add_norm_f32: mode must be 0, 1 or 2");
  OB_REQUIRE(mode != 2 || (res_out && w_b && b_b), OASR_ERR_INVALID, "add_norm_f32: mode 2 needs res_out and the second norm");
  OB_REQUIRE(hidden % 8 == 0 && hidden <= 2048, OASR_ERR_UNSUPPORTED,
             "add_norm_f32: hidden must be a multiple of 8 and at most 2048 (got %lld)", (long long)hidden);
  OB_REQUIRE(is_aligned(h_out, 16) && (!res_in || is_aligned(res_in, 16)) && (!res_out || is_aligned(res_out, 16)) &&
                 (!y || is_aligned(y, 16)) && is_aligned(w_a, 16) && is_aligned(b_a, 16) &&
                 (!w_b || is_aligned(w_b, 16)) && (!b_b || is_aligned(b_b, 16)),
             OASR_ERR_ALIGN, "add_norm_f32: pointers must be 16-byte aligned");
  AddNormArgs a{h_out, res_out, res_in, y, (float)alpha, w_a, b_a, w_b, b_b, rows, (int)hidden, (float)eps, split_out,
                static_cast<uint8_t*>(q_out), q_scale, q_kind};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return OB_DISPATCH_HALF(dtype, T, [&]() -> int {
    if (mode == 0) return launch_add_norm<T, 0>(a, s);
    if (mode == 1) return launch_add_norm<T, 1>(a, s);
    return launch_add_norm<T, 2>(a, s);
  });
}

int oasr_b200_layer_norm(void* out, const void* in, const void* weight, const void* bias, int64_t rows,
                         int64_t hidden, double eps, int dtype, void* stream) {
  return ob::norm_entry<false>(out, nullptr, in, nullptr, weight, bias, rows, hidden, eps, 1.0,
                               OASR_ACT_NONE, dtype, false, stream);
}
int oasr_b200_layer_norm_activation(void* out, const void* in, const void* weight, const void* bias,
                                    int64_t rows, int64_t hidden, double eps, int activation, int dtype,
                                    void* stream) {
  return ob::norm_entry<false>(out, nullptr, in, nullptr, weight, bias, rows, hidden, eps, 1.0, activation,
                               dtype, false, stream);
}
int oasr_b200_add_layer_norm(void* out, const void* in, const void* residual, const void* weight,
                             const void* bias, int64_t rows, int64_t hidden, double eps, double alpha,
                             int dtype, void* stream) {
  return ob::norm_entry<false>(out, nullptr, in, residual, weight, bias, rows, hidden, eps, alpha,
                               OASR_ACT_NONE, dtype, true, stream);
}
int oasr_b200_add_layer_norm_residual(void* out, void* residual_out, const void* in, const void* residual,
                                      const void* weight, const void* bias, int64_t rows, int64_t hidden,
                                      double eps, double alpha, int dtype, void* stream) {
  if (!residual_out && rows > 0) return ob::set_error(OASR_ERR_INVALID, "add_layer_norm_residual: residual_out is null");
  return ob::norm_entry<false>(out, residual_out, in, residual, weight, bias, rows, hidden, eps, alpha,
                               OASR_ACT_NONE, dtype, true, stream);
}
int oasr_b200_rms_norm(void* out, const void* in, const void* weight, const void* bias, int64_t rows,
                       int64_t hidden, double eps, int dtype, void* stream) {
  return ob::norm_entry<true>(out, nullptr, in, nullptr, weight, bias, rows, hidden, eps, 1.0, OASR_ACT_NONE,
                              dtype, false, stream);
}
int oasr_b200_rms_norm_activation(void* out, const void* in, const void* weight, const void* bias,
                                  int64_t rows, int64_t hidden, double eps, int activation, int dtype,
                                  void* stream) {
  return ob::norm_entry<true>(out, nullptr, in, nullptr, weight, bias, rows, hidden, eps, 1.0, activation,
                              dtype, false, stream);
}
int oasr_b200_add_rms_norm(void* out, const void* in, const void* residual, const void* weight,
                           const void* bias, int64_t rows, int64_t hidden, double eps, double alpha, int dtype,
                           void* stream) {
  return ob::norm_entry<true>(out, nullptr, in, residual, weight, bias, rows, hidden, eps, alpha,
                              OASR_ACT_NONE, dtype, true, stream);
}
int oasr_b200_add_rms_norm_residual(void* out, void* residual_out, const void* in, const void* residual,
                                    const void* weight, const void* bias, int64_t rows, int64_t hidden,
                                    double eps, double alpha, int dtype, void* stream) {
  if (!residual_out && rows > 0) return ob::set_error(OASR_ERR_INVALID, "add_rms_norm_residual: residual_out is null");
  return ob::norm_entry<true>(out, residual_out, in, residual, weight, bias, rows, hidden, eps, alpha,
                              OASR_ACT_NONE, dtype, true, stream);
}

int oasr_b200_batch_norm(void* out, const void* in, const void* weight, const void* bias,
                         const void* running_mean, const void* running_var, int64_t rows, int64_t channels,
                         double eps, int activation, int dtype, void* stream) {
  using namespace ob;
  OB_REQUIRE(rows == 0 || (out && in && weight && bias && running_mean && running_var), OASR_ERR_INVALID,
             "batch_norm: null pointer argument");
  OB_REQUIRE(rows >= 0 && channels > 0 && channels < (1 << 24), OASR_ERR_INVALID,
             "batch_norm: bad shape rows=%lld channels=%lld", (long long)rows, (long long)channels);
  OB_REQUIRE(act_is_known(activation), OASR_ERR_INVALID, "batch_norm: unknown activation id %d", activation);
  BnArgs a{out, in, weight, bias, running_mean, running_var, rows, (int)channels, (float)eps, activation};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return OB_DISPATCH_FLOAT(dtype, T, [&]() -> int {
    if (activation != OASR_ACT_NONE) return launch_bn<T, true>(a, s);
    return launch_bn<T, false>(a, s);
  });
}

}  // extern "C"
