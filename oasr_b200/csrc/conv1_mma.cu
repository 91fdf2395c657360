// First subsampling convolution (1 -> C channels, 3x3, stride 2, + bias + ReLU; fp32 features in, 16-bit out in the
// parity-split layout the second convolution reads) on the tensor cores.
//
// As a stencil on the CUDA cores this step costs 72 multiply-adds, 4 conversions and a 16-byte store per 8 outputs
// and is bound by instruction issue at about 2.4x its HBM time.  As a GEMM the instruction count per output drops
// by an order of magnitude and the step becomes what it should be, a 2*C-bytes-per-position HBM write:
//   out[row, n] = relu( sum_k A[row, k] * W[n, k] ),   K = 32
// with both operands split in two bf16 terms so that the products keep fp32-like accuracy (error about 2^-16
// relative, 100x below the 16-bit rounding of the output):
//   A[row] = [ x_hi(9) | x_lo(9) | x_hi(9) | 1 | 1 | 0 0 0 ],   W[n] = [ w_hi(9) | w_hi(9) | w_lo(9) | b_hi | b_lo | 0 0 0 ]
// (x = the 9 feature taps of the position, x_hi = bf16(x), x_lo = bf16(x - x_hi); likewise w and the bias b).
// Reference: Conv2dActivation on a one-channel NHWC input, oasr/models/conformer/model.py:433-444.
//
// Rows are the slots of the parity-split output (B, TH, 4, FH, C) in memory order, so that a tile of 128 rows is
// 128 consecutive slots of ONE utterance and leaves as plain 2-D TMA boxes; only the slots of frame pairs below
// the utterance's t1_limit are computed (a contiguous prefix of its region); slots inside that prefix that lie past
// the frame limit or the last frequency bin come out as zeros.
//   warp 0       builds the weight operand once (all warps help), then issues the MMAs (2 K steps x C/256 halves)
//   warps 1-4    producers: one row each -- 9 feature loads, split, four swizzled 16-byte stores (A is double-buffered)
//   warps 5-12   epilogue: tcgen05.ld (thread = row), ReLU, round, swizzled staging, TMA store; two accumulator
//                stages of 256 columns, so the MMAs of the next half run under the epilogue of this one
// Every wait is bounded (mbar_wait); on give-up the CTA drains and raises the device status word.
#include <cuda.h>

#include <type_traits>

#include "common.cuh"
#include "device_status.cuh"
#include "sm100_ptx.cuh"
#include "tma_host.cuh"

namespace ob {
namespace conv1_mma {

int g_enabled = 1;   // tunable conv1_mma

constexpr int BM = 128;
constexpr int kProdWarps = 4;
constexpr int kEpiWarps = 8;
constexpr int kThreads = 32 * (1 + kProdWarps + kEpiWarps);
constexpr int kMaxBatch = 1024;
constexpr int kRowBytes = 128;          // one swizzle row: 64 bf16 slots, 32 of them used
constexpr int kABytes = BM * kRowBytes;

struct Params {
  const float* in;          // (B, T, F) fp32
  const float* weight;      // (C, 3, 3) fp32
  const float* bias;        // (C) fp32
  const int32_t* t1_limit;  // nullable (B)
  int B, T, F, C, T1, F1, TH, FH;
  uint32_t* status;
};

template <int C>
struct Smem {
  static constexpr int kBBytes = C * kRowBytes;
  static constexpr int kAOffset = kBBytes;
  static constexpr int kEpiOffset = kAOffset + 2 * kABytes;
  static constexpr int kWarpEpi = 2 * 4096;                 // two 32 x 64 16-bit staging buffers per epilogue warp
  static constexpr int kCumOffset = kEpiOffset + kEpiWarps * kWarpEpi;
  static constexpr int kBarOffset = kCumOffset + ((kMaxBatch + 1) * 4 + 15) / 16 * 16;
  static_assert(kBarOffset % 8 == 0, "mbarriers are 8-byte objects");
  static constexpr int kNumBars = 8;
  static constexpr int kDynamic = kBarOffset + kNumBars * 8 + 16 + 1024;
};

__device__ __forceinline__ uint32_t bf16_bits(float f) {
  return static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(f)));
}
__device__ __forceinline__ float bf16_round(float f) { return __bfloat162float(__float2bfloat16_rn(f)); }

// 32 operand entries of one row (as 16 packed bf16 pairs) from 9 values: [hi | lo | hi | one one 0 0 0] when
// kFeature, [hi | hi | lo | v9_hi v9_lo 0 0 0] for a weight row (v9 = its bias).
template <bool kFeature>
__device__ __forceinline__ void build_row(const float (&v)[9], float v9, uint32_t (&out)[16]) {
  uint32_t e[32];
#pragma unroll
  for (int k = 0; k < 9; ++k) {
    const float hi = bf16_round(v[k]);
    const uint32_t h = bf16_bits(hi), l = bf16_bits(v[k] - hi);
    e[k] = h;
    e[9 + k] = kFeature ? l : h;
    e[18 + k] = kFeature ? h : l;
  }
  if (kFeature) {
    e[27] = e[28] = 0x3F80u;                     // 1.0
  } else {
    const float hi = bf16_round(v9);
    e[27] = bf16_bits(hi);
    e[28] = bf16_bits(v9 - hi);
  }
  e[29] = e[30] = e[31] = 0;
#pragma unroll
  for (int i = 0; i < 16; ++i) out[i] = e[2 * i] | (e[2 * i + 1] << 16);
}

// Row r of a K-major, 128-byte-swizzled operand tile: the 16-byte chunk c of the row sits at chunk c ^ (r & 7).
__device__ __forceinline__ void store_row(uint8_t* tile, int r, const uint32_t (&w)[16]) {
  uint8_t* row = tile + (r >> 3) * 1024 + (r & 7) * 128;
#pragma unroll
  for (int c = 0; c < 4; ++c)
    *reinterpret_cast<uint4*>(row + ((c ^ (r & 7)) << 4)) = make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
}

template <typename T>
__device__ __forceinline__ uint32_t pack_relu2(uint32_t a, uint32_t b);
template <>
__device__ __forceinline__ uint32_t pack_relu2<__nv_bfloat16>(uint32_t a, uint32_t b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(fmaxf(__uint_as_float(a), 0.f), fmaxf(__uint_as_float(b), 0.f));
  return *reinterpret_cast<uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack_relu2<__half>(uint32_t a, uint32_t b) {
  __half2 v = __floats2half2_rn(fmaxf(__uint_as_float(a), 0.f), fmaxf(__uint_as_float(b), 0.f));
  return *reinterpret_cast<uint32_t*>(&v);
}

template <typename T, int C>
__global__ void __launch_bounds__(kThreads, 1) conv1_mma_kernel(const __grid_constant__ CUtensorMap tmap_out, const Params p) {
  using S = Smem<C>;
  constexpr int kHalves = C / 256;
  constexpr uint32_t kIdesc = ptx::umma_idesc_f16(true, BM, 256);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sB = smem;
  uint8_t* sA = smem + S::kAOffset;
  int32_t* cum = reinterpret_cast<int32_t*>(smem + S::kCumOffset);    // cum[b] = tiles of utterances < b
  uint64_t* a_full = reinterpret_cast<uint64_t*>(smem + S::kBarOffset);
  uint64_t* a_empty = a_full + 2;
  uint64_t* t_full = a_empty + 2;
  uint64_t* t_empty = t_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(t_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int slots_per_b = p.TH * 4 * p.FH;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&a_full[i], kProdWarps);
      ptx::mbar_init(&a_empty[i], 1);
      ptx::mbar_init(&t_full[i], 1);
      ptx::mbar_init(&t_empty[i], kEpiWarps);
    }
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&tmap_out);
  }
  if (warp == 0) {
    __syncwarp();                                  // lane 0 rejoins the warp before the warp-wide allocation
    ptx::tmem_alloc(tmem_slot, 512);
    ptx::tmem_relinquish();
    // tiles per utterance -> exclusive prefix, 32 utterances per lane
    const int per_lane = (p.B + 31) / 32;
    int mine = 0;
    for (int i = 0; i < per_lane; ++i) {
      const int b = lane * per_lane + i;
      if (b < p.B) {
        const int t1_end = p.t1_limit ? min(p.T1, max(p.t1_limit[b], 0)) : p.T1;
        mine += (((t1_end + 1) >> 1) * 4 * p.FH + BM - 1) / BM;
      }
    }
    int incl = mine;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += o;
    }
    int run = incl - mine;
    for (int i = 0; i < per_lane; ++i) {
      const int b = lane * per_lane + i;
      if (b < p.B) {
        cum[b] = run;
        const int t1_end = p.t1_limit ? min(p.T1, max(p.t1_limit[b], 0)) : p.T1;
        run += (((t1_end + 1) >> 1) * 4 * p.FH + BM - 1) / BM;
      }
    }
    if (lane == 31) cum[p.B] = incl;
  }
  // weight operand: one row per output channel, built once by all threads
  for (int n = threadIdx.x; n < C; n += kThreads) {
    float w[9];
#pragma unroll
    for (int k = 0; k < 9; ++k) w[k] = p.weight[n * 9 + k];
    uint32_t row[16];
    build_row<false>(w, p.bias[n], row);
    store_row(sB, n, row);
  }
  ptx::fence_proxy_async_smem();
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const int num_tiles = cum[p.B];

  // utterance of a tile: the last b with cum[b] <= tile
  auto find_b = [&](int tile) {
    int lo = 0, hi = p.B - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (cum[mid] <= tile) lo = mid; else hi = mid - 1;
    }
    return lo;
  };

  if (warp == 0) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      bool ok = true;
      int n = 0;
      const uint32_t b_addr = ptx::smem_u32(sB);
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++n) {
        const int s = n & 1;
        if (!ptx::mbar_wait(&a_full[s], (n >> 1) & 1, abort_flag)) { ok = false; break; }
        ptx::tc_fence_after_sync();
        const uint32_t a_addr = ptx::smem_u32(sA + s * kABytes);
#pragma unroll
        for (int half = 0; half < kHalves; ++half) {
          const int u = n * kHalves + half;
          const int acc = u & 1;
          if (!ptx::mbar_wait(&t_empty[acc], ((u >> 1) & 1) ^ 1u, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after_sync();
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            const uint64_t adesc = ptx::smem_desc_kmajor_sw128(a_addr + k * 32);
            const uint64_t bdesc = ptx::smem_desc_kmajor_sw128(b_addr + half * 256 * kRowBytes + k * 32);
            ptx::umma_f16(tmem_base + acc * 256, adesc, bdesc, kIdesc, k != 0 ? 1u : 0u);
          }
          ptx::umma_commit(&t_full[acc]);
        }
        if (ok) ptx::umma_commit(&a_empty[s]);
      }
      if (!ok && p.status) atomicOr(p.status, kStatusGemmMma);
    }
    __syncwarp();
  } else if (warp <= kProdWarps) {
    // ------------------------------ producers: thread = row of the tile ------------------------------
    const int r = (warp - 1) * 32 + lane;
    bool ok = true;
    int n = 0;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++n) {
      const int s = n & 1;
      const int b = find_b(tile);
      const int slot = (tile - cum[b]) * BM + r;
      const int t1_end = p.t1_limit ? min(p.T1, max(p.t1_limit[b], 0)) : p.T1;
      const int fh = slot % p.FH;
      const int rest = slot / p.FH;
      const int plane = rest & 3;
      const int t1 = 2 * (rest >> 2) + (plane >> 1);
      const int f1 = 2 * fh + (plane & 1);
      const bool valid = slot < slots_per_b && t1 < t1_end && f1 < p.F1;
      float x[9];
      if (valid) {
        const float* src = p.in + (static_cast<int64_t>(b) * p.T + 2 * t1) * p.F + 2 * f1;
#pragma unroll
        for (int i = 0; i < 3; ++i)
#pragma unroll
          for (int j = 0; j < 3; ++j) x[i * 3 + j] = __ldg(src + i * p.F + j);
      }
      uint32_t row[16];
      if (valid) {
        build_row<true>(x, 0.f, row);
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) row[i] = 0;
      }
      if (!ptx::mbar_wait(&a_empty[s], ((n >> 1) & 1) ^ 1u, abort_flag)) { ok = false; break; }
      store_row(sA + s * kABytes, r, row);
      ptx::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&a_full[s]);
    }
    if (!ok && lane == 0 && p.status) atomicOr(p.status, kStatusGemmProducer);
  } else {
    // ------------------------------ epilogue: thread = (row, 128-column slice of the half) ------------------------------
    const int ew = warp - (1 + kProdWarps);
    const int q = warp & 3;                        // TMEM lane quarter this warp may access
    const int slice = ew >> 2;
    uint8_t* stage = smem + S::kEpiOffset + ew * S::kWarpEpi;
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    bool ok = true;
    int n = 0;
    int piece = 0;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++n) {
      const int b = find_b(tile);
      const int slot0 = (tile - cum[b]) * BM + q * 32;
      const bool live = slot0 < slots_per_b;       // a band wholly past the utterance's region has no storage
#pragma unroll 1
      for (int half = 0; half < kHalves; ++half) {
        const int u = n * kHalves + half;
        const int acc = u & 1;
        if (!ptx::mbar_wait(&t_full[acc], (u >> 1) & 1, abort_flag)) { ok = false; break; }
        ptx::tc_fence_after_sync();
        const uint32_t t_acc = tmem_base + lane_base + acc * 256 + slice * 128;
#pragma unroll 1
        for (int c = 0; c < 2; ++c, ++piece) {
          uint32_t v[64];
          ptx::tmem_ld_32x64(t_acc + c * 64, v);
          uint8_t* buf = stage + (piece & 1) * 4096;
          if (lane == 0) ptx::bulk_wait_group_read<1>();       // the store issued from this buffer two pieces ago has read it
          __syncwarp();
          ptx::tmem_ld_wait();
          uint8_t* row = buf + lane * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            *reinterpret_cast<uint4*>(row + ((j ^ (lane & 7)) << 4)) =
                make_uint4(pack_relu2<T>(v[8 * j], v[8 * j + 1]), pack_relu2<T>(v[8 * j + 2], v[8 * j + 3]),
                           pack_relu2<T>(v[8 * j + 4], v[8 * j + 5]), pack_relu2<T>(v[8 * j + 6], v[8 * j + 7]));
          }
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (live) ptx::tma_store_3d(&tmap_out, buf, half * 256 + slice * 128 + c * 64, slot0, b);
            ptx::bulk_commit_group();
          }
        }
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&t_empty[acc]);
      }
    }
    if (lane == 0) ptx::bulk_wait_group<0>();
    if (!ok && lane == 0 && p.status) atomicOr(p.status, kStatusGemmEpilogue);
  }

  // Teardown.  After an abandoned wait, give work that may still be in flight time to land before shared memory and
  // tensor memory are released.
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, 512);
  }
}

bool supported(int64_t B, int64_t C) { return g_enabled != 0 && (C == 256 || C == 512) && B >= 1 && B <= kMaxBatch; }

template <typename T, int C>
int launch(void* out, const Params& p, int dtype, cudaStream_t s) {
  using S = Smem<C>;
  static_assert(S::kDynamic <= 232448, "shared memory budget of one CTA");
  auto kern = conv1_mma_kernel<T, C>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kDynamic);
    if (e != cudaSuccess) return set_error(OASR_ERR_CUDA, "subsample_conv1_s2d: cannot reserve %d bytes of shared memory: %s",
                                           S::kDynamic, cudaGetErrorString(e));
    attr_done = true;
  }
  CUtensorMap to;
  const uint64_t slots = static_cast<uint64_t>(p.TH) * 4 * p.FH;
  uint64_t dims[3] = {static_cast<uint64_t>(C), slots, static_cast<uint64_t>(p.B)};
  uint64_t str[3] = {0, static_cast<uint64_t>(C) * 2, static_cast<uint64_t>(C) * 2 * slots};
  uint32_t box[3] = {64, 32, 1};
  if (int rc = make_tensor_map(&to, tma_dtype(dtype), 3, out, dims, str, box)) return rc;
  // an upper bound of the tile count sizes the grid; the kernel derives the exact list from t1_limit
  const int64_t max_tiles = static_cast<int64_t>(p.B) * ((static_cast<int64_t>(slots) + BM - 1) / BM);
  int64_t grid = sm_count();
  if (max_tiles < grid) grid = max_tiles;
  if (grid < 1) grid = 1;
  kern<<<static_cast<unsigned>(grid), kThreads, S::kDynamic, s>>>(to, p);
  return check_launch("subsample_conv1_s2d (tensor-core) launch");
}

int run(void* out, const float* in, const float* weight, const float* bias, const int32_t* t1_limit, int64_t B, int64_t T,
        int64_t F, int64_t C, int dtype, cudaStream_t s) {
  Params p{};
  p.in = in; p.weight = weight; p.bias = bias; p.t1_limit = t1_limit;
  p.B = static_cast<int>(B); p.T = static_cast<int>(T); p.F = static_cast<int>(F); p.C = static_cast<int>(C);
  p.T1 = static_cast<int>((T - 3) / 2 + 1); p.F1 = static_cast<int>((F - 3) / 2 + 1);
  p.TH = (p.T1 + 1) / 2; p.FH = (p.F1 + 1) / 2;
  p.status = device_status_ptr();
  return OB_DISPATCH_HALF(dtype, T_, [&]() -> int {
    if (C == 512) return launch<T_, 512>(out, p, dtype, s);
    return launch<T_, 256>(out, p, dtype, s);
  });
}

}  // namespace conv1_mma
}  // namespace ob
