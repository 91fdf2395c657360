// Paged KV-cache data movement and row gather/scatter.  Byte work, bit-exact
// by construction; HBM-bound (one read + one write of every moved byte),
// 128-bit accesses where the row size allows.
//
// Index rule (oasr/cache/paged_kv.py:23-40 in the reference): logical frame
// pos = offsets[b] + t of stream b lives at physical pool row
//   block_table[b, pos / block_size] * block_size + pos % block_size.
#include <cuda_fp8.h>

#include "common.cuh"

namespace ob {
namespace {

struct PagedWriteArgs {
  uint8_t *k_pool, *v_pool;
  const uint8_t *k_new, *v_new;
  const int32_t* block_table;
  const int32_t* offsets;
  int64_t B, Hkv, T, D;
  int64_t stride_b, stride_h, stride_t;  // elements
  int64_t blocks_per_seq, block_size, num_blocks;
  int elem_bytes;
};

// One thread moves one 16-byte (or narrower, `VB`-byte) piece of one (b, t, h) row for K and V.
template <int VB>
__global__ void __launch_bounds__(256) paged_kv_write_kernel(PagedWriteArgs a) {
  const int64_t row_bytes = a.D * a.elem_bytes;
  const int64_t pieces = row_bytes / VB;
  const int64_t total = a.B * a.T * a.Hkv * pieces;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t piece = i % pieces;
    int64_t r = i / pieces;
    const int64_t h = r % a.Hkv;
    r /= a.Hkv;
    const int64_t t = r % a.T;
    const int64_t b = r / a.T;
    const int64_t pos = static_cast<int64_t>(a.offsets[b]) + t;
    const int64_t logical = pos / a.block_size;
    if (pos < 0 || logical >= a.blocks_per_seq) continue;  // outside the table: dropped, never written
    const int64_t page = a.block_table[b * a.blocks_per_seq + logical];
    if (page < 0 || page >= a.num_blocks) continue;
    const int64_t dst_row = page * a.block_size + pos % a.block_size;
    const int64_t dst = ((dst_row * a.Hkv + h) * a.D) * a.elem_bytes + piece * VB;
    const int64_t src = (b * a.stride_b + h * a.stride_h + t * a.stride_t) * a.elem_bytes + piece * VB;
    if constexpr (VB == 16) {
      *reinterpret_cast<uint4*>(a.k_pool + dst) = *reinterpret_cast<const uint4*>(a.k_new + src);
      *reinterpret_cast<uint4*>(a.v_pool + dst) = *reinterpret_cast<const uint4*>(a.v_new + src);
    } else {
      for (int j = 0; j < VB; ++j) {
        a.k_pool[dst + j] = a.k_new[src + j];
        a.v_pool[dst + j] = a.v_new[src + j];
      }
    }
  }
}

struct PagedGatherArgs {
  uint8_t *k_out, *v_out;
  const uint8_t *k_pool, *v_pool;
  const int32_t* block_table;
  int64_t B, Hkv, D, blocks_per_seq, block_size, num_blocks;
  int elem_bytes;
};

// out[b, h, j*bs + w, :] = pool[table[b, j], w, h, :]
template <int VB>
__global__ void __launch_bounds__(256) paged_kv_gather_kernel(PagedGatherArgs a) {
  const int64_t row_bytes = a.D * a.elem_bytes;
  const int64_t pieces = row_bytes / VB;
  const int64_t Tk = a.blocks_per_seq * a.block_size;
  const int64_t total = a.B * a.Hkv * Tk * pieces;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t piece = i % pieces;
    int64_t r = i / pieces;
    const int64_t pos = r % Tk;
    r /= Tk;
    const int64_t h = r % a.Hkv;
    const int64_t b = r / a.Hkv;
    int64_t page = a.block_table[b * a.blocks_per_seq + pos / a.block_size];
    const bool valid = page >= 0 && page < a.num_blocks;
    const int64_t src_row = page * a.block_size + pos % a.block_size;
    const int64_t src = ((src_row * a.Hkv + h) * a.D) * a.elem_bytes + piece * VB;
    const int64_t dst = i * VB;
    if constexpr (VB == 16) {
      const uint4 z = make_uint4(0, 0, 0, 0);
      *reinterpret_cast<uint4*>(a.k_out + dst) = valid ? *reinterpret_cast<const uint4*>(a.k_pool + src) : z;
      *reinterpret_cast<uint4*>(a.v_out + dst) = valid ? *reinterpret_cast<const uint4*>(a.v_pool + src) : z;
    } else {
      for (int j = 0; j < VB; ++j) {
        a.k_out[dst + j] = valid ? a.k_pool[src + j] : 0;
        a.v_out[dst + j] = valid ? a.v_pool[src + j] : 0;
      }
    }
  }
}

// Row gather / scatter with int64 indices; rows are multiples of 16 bytes.  `table_rows` is the row count of the
// indexed side (source of a gather, destination of a scatter): an index outside [0, table_rows) never becomes an
// address -- a gather writes a zero row for it, a scatter skips it.
template <bool kScatter>
__global__ void __launch_bounds__(256) move_rows_kernel(uint8_t* __restrict__ out, const uint8_t* __restrict__ in,
                                                        const int64_t* __restrict__ index, int64_t n,
                                                        int64_t row_bytes, int64_t table_rows) {
  const int64_t pieces = row_bytes / 16;
  const int64_t total = n * pieces;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t r = i / pieces, piece = i - r * pieces;
    const int64_t j = index[r];
    if constexpr (kScatter) {
      if (j < 0 || j >= table_rows) continue;
      *reinterpret_cast<uint4*>(out + j * row_bytes + piece * 16) =
          *reinterpret_cast<const uint4*>(in + r * row_bytes + piece * 16);
    } else {
      uint4 v = make_uint4(0, 0, 0, 0);
      if (j >= 0 && j < table_rows) v = *reinterpret_cast<const uint4*>(in + j * row_bytes + piece * 16);
      *reinterpret_cast<uint4*>(out + r * row_bytes + piece * 16) = v;
    }
  }
}

// fp8 page write: the same index rule, every 16-bit value divided by its head's scale and rounded to e4m3
// (round to nearest even, saturating at +-448).  One thread converts 8 consecutive values of K and of V.
struct PagedWriteFp8Args {
  uint8_t *k_pool, *v_pool;
  const void *k_new, *v_new;
  const float *k_scale, *v_scale;   // [Hkv]
  const int32_t* block_table;
  const int32_t* offsets;
  int64_t B, Hkv, T, D;
  int64_t stride_b, stride_h, stride_t;  // elements
  int64_t blocks_per_seq, block_size, num_blocks;
};

template <typename T>
__device__ __forceinline__ uint2 to_e4m3x8(const Pack<T>& v, float inv) {
  uint32_t w[2];
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(Elem<T>::to_f(v.v[hh * 4]) * inv, Elem<T>::to_f(v.v[hh * 4 + 1]) * inv),
                                                 __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(Elem<T>::to_f(v.v[hh * 4 + 2]) * inv, Elem<T>::to_f(v.v[hh * 4 + 3]) * inv),
                                                 __NV_SATFINITE, __NV_E4M3);
    w[hh] = lo | (hi << 16);
  }
  return make_uint2(w[0], w[1]);
}

template <typename T>
__global__ void __launch_bounds__(256) paged_kv_write_fp8_kernel(PagedWriteFp8Args a) {
  const int64_t pieces = a.D / 8;
  const int64_t total = a.B * a.T * a.Hkv * pieces;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t piece = i % pieces;
    int64_t r = i / pieces;
    const int64_t h = r % a.Hkv;
    r /= a.Hkv;
    const int64_t t = r % a.T;
    const int64_t b = r / a.T;
    const int64_t pos = static_cast<int64_t>(a.offsets[b]) + t;
    const int64_t logical = pos / a.block_size;
    if (pos < 0 || logical >= a.blocks_per_seq) continue;  // outside the table: dropped, never written
    const int64_t page = a.block_table[b * a.blocks_per_seq + logical];
    if (page < 0 || page >= a.num_blocks) continue;
    const int64_t dst_row = page * a.block_size + pos % a.block_size;
    const int64_t dst = (dst_row * a.Hkv + h) * a.D + piece * 8;
    const int64_t src = b * a.stride_b + h * a.stride_h + t * a.stride_t + piece * 8;
    const Pack<T> kv = ld128(static_cast<const T*>(a.k_new) + src);
    const Pack<T> vv = ld128(static_cast<const T*>(a.v_new) + src);
    *reinterpret_cast<uint2*>(a.k_pool + dst) = to_e4m3x8<T>(kv, 1.f / a.k_scale[h]);
    *reinterpret_cast<uint2*>(a.v_pool + dst) = to_e4m3x8<T>(vv, 1.f / a.v_scale[h]);
  }
}

unsigned grid_for(int64_t items) {
  int64_t g = (items + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<unsigned>(g);
}

}  // namespace
}  // namespace ob

extern "C" {

int oasr_b200_paged_kv_write(void* k_pool, void* v_pool, const void* k_new, const void* v_new,
                             const int32_t* block_table, const int32_t* offsets, int64_t B, int64_t Hkv, int64_t T,
                             int64_t D, int64_t stride_b, int64_t stride_h, int64_t stride_t, int64_t blocks_per_seq,
                             int64_t block_size, int64_t num_blocks, int elem_bytes, void* stream) {
  using namespace ob;
  OB_REQUIRE(k_pool && v_pool && k_new && v_new && block_table && offsets, OASR_ERR_INVALID,
             "paged_kv_write: null pointer argument");
  OB_REQUIRE(B >= 0 && Hkv > 0 && T >= 0 && D > 0 && blocks_per_seq > 0 && block_size > 0 && num_blocks > 0,
             OASR_ERR_INVALID, "paged_kv_write: bad shape");
  OB_REQUIRE(elem_bytes == 1 || elem_bytes == 2 || elem_bytes == 4, OASR_ERR_INVALID,
             "paged_kv_write: elem_bytes must be 1, 2 or 4");
  if (B == 0 || T == 0) return OASR_OK;
  PagedWriteArgs a{static_cast<uint8_t*>(k_pool), static_cast<uint8_t*>(v_pool),
                   static_cast<const uint8_t*>(k_new), static_cast<const uint8_t*>(v_new), block_table, offsets,
                   B, Hkv, T, D, stride_b, stride_h, stride_t, blocks_per_seq, block_size, num_blocks, elem_bytes};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t row_bytes = D * elem_bytes;
  const bool vec = row_bytes % 16 == 0 && (stride_b * elem_bytes) % 16 == 0 && (stride_h * elem_bytes) % 16 == 0 &&
                   (stride_t * elem_bytes) % 16 == 0 && is_aligned(k_pool, 16) && is_aligned(v_pool, 16) &&
                   is_aligned(k_new, 16) && is_aligned(v_new, 16);
  if (vec) {
    paged_kv_write_kernel<16><<<grid_for(B * T * Hkv * (row_bytes / 16)), 256, 0, s>>>(a);
  } else {
    a.elem_bytes = elem_bytes;
    // piece = one element
    if (elem_bytes == 1) paged_kv_write_kernel<1><<<grid_for(B * T * Hkv * D), 256, 0, s>>>(a);
    else if (elem_bytes == 2) paged_kv_write_kernel<2><<<grid_for(B * T * Hkv * D), 256, 0, s>>>(a);
    else paged_kv_write_kernel<4><<<grid_for(B * T * Hkv * D), 256, 0, s>>>(a);
  }
  return check_launch("paged_kv_write launch");
}

int oasr_b200_paged_kv_write_fp8(void* k_pool, void* v_pool, const void* k_new, const void* v_new, const float* k_scale,
                                 const float* v_scale, const int32_t* block_table, const int32_t* offsets, int64_t B,
                                 int64_t Hkv, int64_t T, int64_t D, int64_t stride_b, int64_t stride_h, int64_t stride_t,
                                 int64_t blocks_per_seq, int64_t block_size, int64_t num_blocks, int dtype, void* stream) {
  using namespace ob;
  OB_REQUIRE(k_pool && v_pool && k_new && v_new && k_scale && v_scale && block_table && offsets, OASR_ERR_INVALID,
             "paged_kv_write_fp8: null pointer argument");
  OB_REQUIRE(B >= 0 && Hkv > 0 && T >= 0 && D > 0 && blocks_per_seq > 0 && block_size > 0 && num_blocks > 0,
             OASR_ERR_INVALID, "paged_kv_write_fp8: bad shape");
  OB_REQUIRE(D % 8 == 0 && stride_b % 8 == 0 && stride_h % 8 == 0 && stride_t % 8 == 0 && is_aligned(k_new, 16) &&
                 is_aligned(v_new, 16) && is_aligned(k_pool, 8) && is_aligned(v_pool, 8),
             OASR_ERR_ALIGN, "paged_kv_write_fp8: head_dim and strides must be multiples of 8 elements, sources 16-byte aligned");
  if (B == 0 || T == 0) return OASR_OK;
  PagedWriteFp8Args a{static_cast<uint8_t*>(k_pool), static_cast<uint8_t*>(v_pool), k_new, v_new, k_scale, v_scale,
                      block_table, offsets, B, Hkv, T, D, stride_b, stride_h, stride_t, blocks_per_seq, block_size, num_blocks};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned grid = grid_for(B * T * Hkv * (D / 8));
  return OB_DISPATCH_HALF(dtype, T_, [&]() -> int {
    paged_kv_write_fp8_kernel<T_><<<grid, 256, 0, s>>>(a);
    return check_launch("paged_kv_write_fp8 launch");
  });
}

int oasr_b200_paged_kv_gather(void* k_out, void* v_out, const void* k_pool, const void* v_pool,
                              const int32_t* block_table, int64_t B, int64_t Hkv, int64_t D, int64_t blocks_per_seq,
                              int64_t block_size, int64_t num_blocks, int elem_bytes, void* stream) {
  using namespace ob;
  OB_REQUIRE(k_out && v_out && k_pool && v_pool && block_table, OASR_ERR_INVALID,
             "paged_kv_gather: null pointer argument");
  OB_REQUIRE(B >= 0 && Hkv > 0 && D > 0 && blocks_per_seq >= 0 && block_size > 0 && num_blocks > 0, OASR_ERR_INVALID,
             "paged_kv_gather: bad shape");
  OB_REQUIRE(elem_bytes == 1 || elem_bytes == 2 || elem_bytes == 4, OASR_ERR_INVALID,
             "paged_kv_gather: elem_bytes must be 1, 2 or 4");
  if (B == 0 || blocks_per_seq == 0) return OASR_OK;
  PagedGatherArgs a{static_cast<uint8_t*>(k_out), static_cast<uint8_t*>(v_out),
                    static_cast<const uint8_t*>(k_pool), static_cast<const uint8_t*>(v_pool), block_table,
                    B, Hkv, D, blocks_per_seq, block_size, num_blocks, elem_bytes};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t row_bytes = D * elem_bytes;
  const int64_t rows = B * Hkv * blocks_per_seq * block_size;
  const bool vec = row_bytes % 16 == 0 && is_aligned(k_out, 16) && is_aligned(v_out, 16) && is_aligned(k_pool, 16) &&
                   is_aligned(v_pool, 16);
  if (vec) paged_kv_gather_kernel<16><<<grid_for(rows * (row_bytes / 16)), 256, 0, s>>>(a);
  else if (elem_bytes == 1) paged_kv_gather_kernel<1><<<grid_for(rows * D), 256, 0, s>>>(a);
  else if (elem_bytes == 2) paged_kv_gather_kernel<2><<<grid_for(rows * D), 256, 0, s>>>(a);
  else paged_kv_gather_kernel<4><<<grid_for(rows * D), 256, 0, s>>>(a);
  return check_launch("paged_kv_gather launch");
}

int oasr_b200_gather_rows(void* out, const void* in, const int64_t* index, int64_t n_out, int64_t row_bytes,
                          int64_t in_rows, void* stream) {
  using namespace ob;
  OB_REQUIRE(out && in && index, OASR_ERR_INVALID, "gather_rows: null pointer argument");
  OB_REQUIRE(in_rows >= 0, OASR_ERR_INVALID, "gather_rows: negative source row count");
  OB_REQUIRE(n_out >= 0 && row_bytes > 0 && row_bytes % 16 == 0, OASR_ERR_ALIGN,
             "gather_rows: row size must be a positive multiple of 16 bytes (got %lld)", (long long)row_bytes);
  OB_REQUIRE(is_aligned(out, 16) && is_aligned(in, 16), OASR_ERR_ALIGN, "gather_rows: pointers must be 16-byte aligned");
  if (n_out == 0) return OASR_OK;
  move_rows_kernel<false><<<grid_for(n_out * (row_bytes / 16)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint8_t*>(out), static_cast<const uint8_t*>(in), index, n_out, row_bytes, in_rows);
  return check_launch("gather_rows launch");
}

int oasr_b200_scatter_rows(void* out, const void* in, const int64_t* index, int64_t n_in, int64_t row_bytes,
                           int64_t out_rows, void* stream) {
  using namespace ob;
  OB_REQUIRE(out && in && index, OASR_ERR_INVALID, "scatter_rows: null pointer argument");
  OB_REQUIRE(out_rows >= 0, OASR_ERR_INVALID, "scatter_rows: negative destination row count");
  OB_REQUIRE(n_in >= 0 && row_bytes > 0 && row_bytes % 16 == 0, OASR_ERR_ALIGN,
             "scatter_rows: row size must be a positive multiple of 16 bytes (got %lld)", (long long)row_bytes);
  OB_REQUIRE(is_aligned(out, 16) && is_aligned(in, 16), OASR_ERR_ALIGN, "scatter_rows: pointers must be 16-byte aligned");
  if (n_in == 0) return OASR_OK;
  move_rows_kernel<true><<<grid_for(n_in * (row_bytes / 16)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint8_t*>(out), static_cast<const uint8_t*>(in), index, n_in, row_bytes, out_rows);
  return check_launch("scatter_rows launch");
}

}  // extern "C"
