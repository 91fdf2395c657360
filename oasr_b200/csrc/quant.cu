// Row-wise dynamic quantisation to one byte per element for the 8-bit GEMM kinds:
//   scale[r] = amax(x[r, :]) / qmax,  q[r, c] = round(x[r, c] / scale[r])
// with qmax = 448 and round-to-nearest-even into fp8 e4m3 (saturating), or qmax = 127 and
// round-to-nearest into int8.  Per token on activations, per output channel on weights.
// HBM-bound: 2*cols bytes read + cols bytes written per row (the second pass over the row hits L1/L2).
// One warp per row, 16-byte loads, 8-byte stores.  The reference has no quantised path
// (oasr/layers/linear.py:7 names a future one); the arithmetic is restated on the CPU in oracle/ops.py.
#include <cuda_fp8.h>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace ob {
namespace {

template <typename T, int kKind>
__global__ void __launch_bounds__(256) quantize_rows_kernel(uint8_t* __restrict__ q, float* __restrict__ scale,
                                                            const T* __restrict__ x, int64_t rows, int cols) {
  ptx::grid_dep_launch();   // no-ops unless launched with programmatic stream serialisation
  ptx::grid_dep_wait();
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* __restrict__ xr = x + row * cols;
  float amax = 0.f;
  for (int c = lane * 8; c < cols; c += 256) {
    const Pack<T> v = ld128(xr + c);
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(Elem<T>::to_f(v.v[i])));
  }
  amax = warp_max(amax);
  constexpr float kQmax = kKind == OASR_Q8_FP8_E4M3 ? 448.f : 127.f;
  const float sc = amax > 0.f ? amax / kQmax : 1.f;
  const float inv = 1.f / sc;
  if (lane == 0) scale[row] = sc;
  uint8_t* __restrict__ qr = q + row * cols;
  for (int c = lane * 8; c < cols; c += 256) {
    const Pack<T> v = ld128(xr + c);
    uint32_t w[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t packed = 0;
#pragma unroll
      for (int i = 0; i < 4; i += 2) {
        const float a = Elem<T>::to_f(v.v[h * 4 + i]) * inv, b = Elem<T>::to_f(v.v[h * 4 + i + 1]) * inv;
        uint32_t two;
        if constexpr (kKind == OASR_Q8_FP8_E4M3) {
          two = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
        } else {
          const int ia = max(-127, min(127, __float2int_rn(a))), ib = max(-127, min(127, __float2int_rn(b)));
          two = (static_cast<uint32_t>(ia) & 0xffu) | ((static_cast<uint32_t>(ib) & 0xffu) << 8);
        }
        packed |= two << (8 * i);
      }
      w[h] = packed;
    }
    *reinterpret_cast<uint2*>(qr + c) = make_uint2(w[0], w[1]);
  }
}

}  // namespace
}  // namespace ob

extern "C" {

int oasr_b200_quantize_rows(void* q, float* scale, const void* x, int64_t rows, int64_t cols, int kind, int dtype,
                            void* stream) {
  using namespace ob;
  OB_REQUIRE(rows >= 0 && cols > 0, OASR_ERR_INVALID, "quantize_rows: bad shape");
  OB_REQUIRE(kind == OASR_Q8_FP8_E4M3 || kind == OASR_Q8_INT8, OASR_ERR_INVALID, "quantize_rows: kind must be 1 (fp8 e4m3) or 2 (int8)");
  if (rows == 0) return OASR_OK;
  OB_REQUIRE(q && scale && x, OASR_ERR_INVALID, "quantize_rows: null pointer argument");
  OB_REQUIRE(cols % 16 == 0 && is_aligned(q, 16) && is_aligned(x, 16), OASR_ERR_ALIGN,
             "quantize_rows: cols must be a multiple of 16 and the pointers 16-byte aligned");
  OB_REQUIRE(cols < (1 << 30) && (rows + 7) / 8 < (int64_t(1) << 31), OASR_ERR_INVALID, "quantize_rows: extent too large");
  const unsigned grid = static_cast<unsigned>((rows + 7) / 8);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return OB_DISPATCH_HALF(dtype, T, [&]() -> int {
    if (kind == OASR_Q8_FP8_E4M3)
      launch_pdl(quantize_rows_kernel<T, OASR_Q8_FP8_E4M3>, dim3(grid), dim3(256), 0, s, static_cast<uint8_t*>(q), scale, static_cast<const T*>(x), rows, (int)cols);
    else
      launch_pdl(quantize_rows_kernel<T, OASR_Q8_INT8>, dim3(grid), dim3(256), 0, s, static_cast<uint8_t*>(q), scale, static_cast<const T*>(x), rows, (int)cols);
    return check_launch("quantize_rows launch");
  });
}

}  // extern "C"
