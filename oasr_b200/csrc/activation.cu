// GLU and swish: pure-bandwidth elementwise kernels, 128-bit accesses,
// grid sized as a multiple of the SM count.  Algorithmic bytes (16-bit type):
// GLU 6C per output row of width C, swish 4 per element.
#include "common.cuh"

namespace ob {
namespace {

template <typename T>
__global__ void __launch_bounds__(256) glu_vec_kernel(T* __restrict__ out, const T* __restrict__ in,
                                                      int64_t rows, int channels) {
  constexpr int V = Elem<T>::kVec;
  const int ppr = channels / V;
  const int64_t total = rows * ppr;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t p = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; p < total; p += stride) {
    const int64_t r = p / ppr;
    const int c = static_cast<int>(p - r * ppr) * V;
    const T* row = in + r * 2 * channels;
    const Pack<T> a = ld128_stream(row + c);
    const Pack<T> g = ld128_stream(row + channels + c);
    Pack<T> o;
#pragma unroll
    for (int i = 0; i < V; ++i) o.v[i] = Elem<T>::from_f(Elem<T>::to_f(a.v[i]) * sigmoid_f(Elem<T>::to_f(g.v[i])));
    st128(out + r * channels + c, o);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) glu_scalar_kernel(T* __restrict__ out, const T* __restrict__ in,
                                                         int64_t rows, int channels) {
  const int64_t total = rows * channels;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t r = i / channels;
    const int c = static_cast<int>(i - r * channels);
    const float a = Elem<T>::to_f(in[r * 2 * channels + c]);
    const float g = Elem<T>::to_f(in[r * 2 * channels + channels + c]);
    out[i] = Elem<T>::from_f(a * sigmoid_f(g));
  }
}

template <typename T>
__global__ void __launch_bounds__(256) swish_vec_kernel(T* __restrict__ out, const T* __restrict__ in,
                                                        int64_t packs) {
  constexpr int V = Elem<T>::kVec;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t p = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; p < packs; p += stride) {
    const Pack<T> a = ld128_stream(in + p * V);
    Pack<T> o;
#pragma unroll
    for (int i = 0; i < V; ++i) o.v[i] = Elem<T>::from_f(apply_act<OASR_ACT_SWISH>(Elem<T>::to_f(a.v[i])));
    st128(out + p * V, o);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) swish_scalar_kernel(T* __restrict__ out, const T* __restrict__ in,
                                                           int64_t begin, int64_t numel) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = begin + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < numel; i += stride) {
    out[i] = Elem<T>::from_f(apply_act<OASR_ACT_SWISH>(Elem<T>::to_f(in[i])));
  }
}

unsigned grid_for(int64_t work_items, int block) {
  int64_t g = (work_items + block - 1) / block;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<unsigned>(g);
}

}  // namespace
}  // namespace ob

namespace ob {
namespace {

// Transformer-XL relative shift + scale + attention mask in one pass: bd (B, H, T, ld) holds the scores of query i
// against the 2T-1 relative positions (column p = distance T-1-p); key j of query i sits at column (T-1) + j - i.
// out (B, H, T, T) = visible(b, i, j) ? bd[b, h, i, T-1+j-i] * scale : floor, with the chunked-limited window
// (query chunk - key chunk in [0, left_chunks], chunks of `chunk` frames) and key padding j < lengths[b]
// (oasr/models/nemotron/encoder.py:82-96 rel_shift, :124-149 chunked_limited_mask, :343-348 mask floor).
template <typename T>
__global__ void __launch_bounds__(256) relshift_bias_kernel(T* __restrict__ out, const T* __restrict__ bd,
                                                            const int32_t* __restrict__ lengths, int B, int H, int Tn, int ld, int ld_out,
                                                            int64_t bd_sb, int64_t bd_sh,
                                                            float scale, int chunk, int left_chunks, float floor_v) {
  // One warp per output row (b, h, i): the visible keys of a row are one interval [lo, hi), so the per-element work is a
  // compare, a 2-byte load at a row-constant offset and a store; the row decomposition is done once per warp.
  const int lane = threadIdx.x & 31;
  const int64_t rows = static_cast<int64_t>(B) * H * Tn;
  const int64_t wstride = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  const T floor_t = Elem<T>::from_f(floor_v);
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows; row += wstride) {
    const int64_t r = row / Tn;               // b * H + h
    const int i = static_cast<int>(row - r * Tn);
    const int b = static_cast<int>(r / H);
    const int h = static_cast<int>(r - static_cast<int64_t>(b) * H);
    const int qc = i / chunk;
    const int lo = max(0, (qc - left_chunks) * chunk);
    const int hi = min(min((qc + 1) * chunk, Tn), lengths[b]);
    const T* src = bd + b * bd_sb + h * bd_sh + static_cast<int64_t>(i) * ld + (Tn - 1 - i);
    T* dst = out + row * ld_out;
#pragma unroll 4
    for (int j = lane; j < Tn; j += 32) {
      T v = floor_t;
      if (j >= lo && j < hi) v = Elem<T>::from_f(Elem<T>::to_f(src[j]) * scale);
      dst[j] = v;
    }
  }
}

// Packed form: scores bd (H, total, ld) over packed rows, one block-diagonal bias segment per stream.  Segment s is
// (H, len_s, roundup8(len_s)) at offsets[s]; a warp finds its row's segment by bisection of cu_seqlens.
template <typename T>
__global__ void __launch_bounds__(256) relshift_bias_packed_kernel(T* __restrict__ out, const T* __restrict__ bd,
                                                                   const int32_t* __restrict__ cu, const int64_t* __restrict__ offsets,
                                                                   int S, int H, int total, int Tn, int ld, float scale,
                                                                   int chunk, int left_chunks, float floor_v) {
  const int lane = threadIdx.x & 31;
  const int64_t rows = static_cast<int64_t>(H) * total;
  const int64_t wstride = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  const T floor_t = Elem<T>::from_f(floor_v);
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows; row += wstride) {
    const int h = static_cast<int>(row / total);
    const int r = static_cast<int>(row - static_cast<int64_t>(h) * total);
    int lo_s = 0, hi_s = S;                    // largest s with cu[s] <= r
    while (hi_s - lo_s > 1) {
      const int mid = (lo_s + hi_s) >> 1;
      if (cu[mid] <= r) lo_s = mid; else hi_s = mid;
    }
    const int s0 = cu[lo_s];
    const int len = cu[lo_s + 1] - s0;
    const int i = r - s0;
    if (i >= len) continue;                    // rows past the last segment
    const int ld_s = (len + 7) & ~7;
    const int qc = i / chunk;
    const int lo = max(0, (qc - left_chunks) * chunk);
    const int hi = min((qc + 1) * chunk, len);
    const T* src = bd + row * ld + (Tn - 1 - i);
    T* dst = out + offsets[lo_s] + (static_cast<int64_t>(h) * len + i) * ld_s;
#pragma unroll 4
    for (int j = lane; j < ld_s; j += 32) {
      T v = floor_t;
      if (j >= lo && j < hi) v = Elem<T>::from_f(Elem<T>::to_f(src[j]) * scale);
      dst[j] = v;
    }
  }
}

}  // namespace
}  // namespace ob

namespace ob {
// Streaming form of the same bias: B streams, Tq new query frames each, keys = the stream's cached frames followed by
// the chunk.  One warp per output row (b, h, i).
template <typename T>
__global__ void __launch_bounds__(256) relshift_bias_stream_kernel(T* __restrict__ out, const T* __restrict__ bd,
                                                                   const int32_t* __restrict__ cached,
                                                                   const int32_t* __restrict__ offsets, int B, int H, int Tq,
                                                                   int ld, int ld_out, int Lmax, int64_t bd_sh, float scale,
                                                                   int chunk, int left_chunks, float floor_v) {
  const int lane = threadIdx.x & 31;
  const int64_t rows = static_cast<int64_t>(B) * H * Tq;
  const int64_t wstride = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  const T floor_t = Elem<T>::from_f(floor_v);
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows; row += wstride) {
    const int64_t r = row / Tq;               // b * H + h
    const int i = static_cast<int>(row - r * Tq);
    const int b = static_cast<int>(r / H);
    const int h = static_cast<int>(r - static_cast<int64_t>(b) * H);
    const int c = cached[b];
    const int keys = c + Tq;
    const int q_abs = offsets[b] + i;
    const int k_abs0 = offsets[b] - c;        // absolute frame of key 0 (never negative: only real frames are cached)
    const int qc = q_abs / chunk;
    // distance of key j from query i is c + i - j; the projected table has the embedding of distance d at row Lmax - 1 - d
    const T* src = bd + h * bd_sh + (static_cast<int64_t>(b) * Tq + i) * ld + (Lmax - 1 - c - i);
    T* dst = out + row * ld_out;
    for (int j = lane; j < ld_out; j += 32) {
      T v = floor_t;
      if (j < keys) {
        const int diff = qc - (k_abs0 + j) / chunk;
        if (diff >= 0 && diff <= left_chunks) v = Elem<T>::from_f(Elem<T>::to_f(src[j]) * scale);
      }
      dst[j] = v;
    }
  }
}
}  // namespace ob

extern "C" {

int oasr_b200_relshift_bias_stream(void* out, const void* bd, const int32_t* cached, const int32_t* offsets, int64_t B,
                                   int64_t H, int64_t Tq, int64_t ld, int64_t ld_out, int64_t Lmax, int64_t bd_stride_h,
                                   double scale, int64_t chunk, int64_t left_chunks, double floor_value, int dtype,
                                   void* stream) {
  using namespace ob;
  OB_REQUIRE(B >= 0 && H > 0 && Tq > 0 && Lmax >= Tq && ld >= 2 * Lmax - 1 && ld_out > 0 && chunk > 0 && left_chunks >= 0,
             OASR_ERR_INVALID, "relshift_bias_stream: bad shape");
  if (B == 0) return OASR_OK;
  OB_REQUIRE(out && bd && cached && offsets, OASR_ERR_INVALID, "relshift_bias_stream: null pointer argument");
  const int64_t rows = B * H * Tq;
  int64_t g = (rows + 7) / 8;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  if (g > cap) g = cap;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return OB_DISPATCH_HALF(dtype, T_, [&]() -> int {
    relshift_bias_stream_kernel<T_><<<static_cast<unsigned>(g), 256, 0, s>>>(
        static_cast<T_*>(out), static_cast<const T_*>(bd), cached, offsets, (int)B, (int)H, (int)Tq, (int)ld, (int)ld_out,
        (int)Lmax, bd_stride_h ? bd_stride_h : B * Tq * ld, (float)scale, (int)chunk, (int)left_chunks, (float)floor_value);
    return check_launch("relshift_bias_stream launch");
  });
}

int oasr_b200_relshift_bias_packed(void* out, const void* bd, const int32_t* cu_seqlens, const int64_t* bias_offsets,
                                   int64_t num_segs, int64_t H, int64_t total, int64_t T, int64_t ld, double scale,
                                   int64_t chunk, int64_t left_chunks, double floor_value, int dtype, void* stream) {
  using namespace ob;
  OB_REQUIRE(num_segs >= 0 && H > 0 && total >= 0 && T > 0 && ld >= 2 * T - 1 && chunk > 0 && left_chunks >= 0 &&
                 H * total < (int64_t(1) << 40) && total < (int64_t(1) << 31),
             OASR_ERR_INVALID, "relshift_bias_packed: bad shape");
  if (num_segs == 0 || total == 0) return OASR_OK;
  OB_REQUIRE(out && bd && cu_seqlens && bias_offsets, OASR_ERR_INVALID, "relshift_bias_packed: null pointer argument");
  if (chunk > T) chunk = T;
  if (left_chunks > T) left_chunks = T;
  const int64_t rows = H * total;
  int64_t g = (rows + 7) / 8;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  if (g > cap) g = cap;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return OB_DISPATCH_HALF(dtype, T_, [&]() -> int {
    relshift_bias_packed_kernel<T_><<<static_cast<unsigned>(g), 256, 0, s>>>(
        static_cast<T_*>(out), static_cast<const T_*>(bd), cu_seqlens, bias_offsets, (int)num_segs, (int)H, (int)total, (int)T,
        (int)ld, (float)scale, (int)chunk, (int)left_chunks, (float)floor_value);
    return check_launch("relshift_bias_packed launch");
  });
}

int oasr_b200_relshift_bias(void* out, const void* bd, const int32_t* lengths, int64_t B, int64_t H, int64_t T, int64_t ld,
                            int64_t ld_out, int64_t bd_stride_b, int64_t bd_stride_h, double scale, int64_t chunk, int64_t left_chunks, double floor_value, int dtype, void* stream) {
  using namespace ob;
  OB_REQUIRE(B >= 0 && H > 0 && T > 0 && ld >= 2 * T - 1 && ld_out >= T && chunk > 0 && left_chunks >= 0, OASR_ERR_INVALID,
             "relshift_bias: bad shape");
  if (B == 0) return OASR_OK;
  OB_REQUIRE(out && bd && lengths, OASR_ERR_INVALID, "relshift_bias: null pointer argument");
  const int64_t rows = B * H * T;
  if (chunk > T) chunk = T;              // every frame is in chunk 0 either way; keeps the interval arithmetic in int range
  if (left_chunks > T) left_chunks = T;
  int64_t g = (rows + 7) / 8;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  if (g > cap) g = cap;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return OB_DISPATCH_HALF(dtype, T_, [&]() -> int {
    relshift_bias_kernel<T_><<<static_cast<unsigned>(g), 256, 0, s>>>(static_cast<T_*>(out), static_cast<const T_*>(bd), lengths,
                                                                      (int)B, (int)H, (int)T, (int)ld, (int)ld_out, bd_stride_b ? bd_stride_b : H * T * ld,
                                                                      bd_stride_h ? bd_stride_h : T * ld, (float)scale, (int)chunk,
                                                                      (int)left_chunks, (float)floor_value);
    return check_launch("relshift_bias launch");
  });
}


int oasr_b200_glu(void* out, const void* in, int64_t rows, int64_t channels, int dtype, void* stream) {
  using namespace ob;
  OB_REQUIRE(rows == 0 || (out && in), OASR_ERR_INVALID, "glu: null pointer argument");
  OB_REQUIRE(rows >= 0 && channels > 0 && channels < (1 << 24), OASR_ERR_INVALID,
             "glu: bad shape rows=%lld channels=%lld", (long long)rows, (long long)channels);
  if (rows == 0) return OASR_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return OB_DISPATCH_FLOAT(dtype, T, [&]() -> int {
    constexpr int V = Elem<T>::kVec;
    if (channels % V == 0 && is_aligned(in, 16) && is_aligned(out, 16)) {
      glu_vec_kernel<T><<<grid_for(rows * (channels / V), 256), 256, 0, s>>>(
          static_cast<T*>(out), static_cast<const T*>(in), rows, (int)channels);
    } else {
      glu_scalar_kernel<T><<<grid_for(rows * channels, 256), 256, 0, s>>>(
          static_cast<T*>(out), static_cast<const T*>(in), rows, (int)channels);
    }
    return check_launch("glu kernel launch");
  });
}

int oasr_b200_swish(void* out, const void* in, int64_t numel, int dtype, void* stream) {
  using namespace ob;
  OB_REQUIRE(numel == 0 || (out && in), OASR_ERR_INVALID, "swish: null pointer argument");
  OB_REQUIRE(numel >= 0, OASR_ERR_INVALID, "swish: negative element count");
  if (numel == 0) return OASR_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return OB_DISPATCH_FLOAT(dtype, T, [&]() -> int {
    constexpr int V = Elem<T>::kVec;
    int64_t vec_elems = 0;
    if (is_aligned(in, 16) && is_aligned(out, 16)) {
      const int64_t packs = numel / V;
      vec_elems = packs * V;
      if (packs > 0) {
        swish_vec_kernel<T><<<grid_for(packs, 256), 256, 0, s>>>(static_cast<T*>(out),
                                                                  static_cast<const T*>(in), packs);
      }
    }
    if (vec_elems < numel) {
      swish_scalar_kernel<T><<<grid_for(numel - vec_elems, 256), 256, 0, s>>>(
          static_cast<T*>(out), static_cast<const T*>(in), vec_elems, numel);
    }
    return check_launch("swish kernel launch");
  });
}

}  // extern "C"
