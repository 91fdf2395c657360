// Second subsampling convolution (3x3, stride 2, C_in -> N channels, + bias + ReLU) as an implicit GEMM on CTA pairs.
//
// Same problem and operand layouts as the conv scheduler of gemm.cu (the first conv's output in the parity-split
// layout, so that tap (kh, kw) of a block of `tpt` output frames x `f2` positions is ONE dense 5-D TMA box; K block =
// (tap, 64 input channels); output rows written straight into the packed (total_frames * f2, N) matrix the embed
// Linear reads), i.e. Conv2dActivation of oasr/models/conformer/model.py:433-449 (reference kernels
// include/oasr/conv/conv2d.cuh:78-86, oasr/functionals/conv.py:765-793) followed by pack_hidden
// (oasr/models/conformer/packing.py:204-216).
//
// What differs is the tile.  The single-CTA 128 x 256 tile pulls 47 KB of operands per 512 tensor clocks (94
// B/clk per SM, 27 TB/s over the GPU), more than the L2 delivers, and runs at half the tensor rate.  Here the two
// CTAs of a cluster each hold ONE conv tile (their own 128 accumulator rows, possibly of different utterances) and
// together issue tcgen05 cta_group::2 instructions of M 256 x N 256 over ALL N output channels: each CTA stages its
// own A box and half of the weight rows of every instruction, 48 KB per 1024 tensor clocks.  With K = 9 * C_in = 4608
// the main loop is 72 K blocks long, so that the epilogue, which cannot overlap the next tile's main loop (the 128 x
// 512 fp32 accumulator is all of a CTA's tensor memory), is a small share.  No multicast; every wait is bounded.
#include <cuda.h>

#include <type_traits>

#include "common.cuh"
#include "device_status.cuh"
#include "sm100_ptx.cuh"
#include "tma_host.cuh"

namespace ob {
namespace conv2_pair {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kEpiWarps = 8;
constexpr int kThreads = 64 + 32 * kEpiWarps;

struct Params {
  int N;                    // output channels
  int groups;               // utterances
  const int32_t* offsets;   // cu[0..groups]: packed output frame offsets
  int conv_f2;              // output positions per output frame
  int conv_tpt;             // output frames per tile = 128 / conv_f2
  int conv_cblocks;         // input channels / 64
  int num_k_blocks;         // 9 * conv_cblocks
  void* D;                  // (total_frames * f2, N)
  const void* bias;         // T[N], nullable
  uint32_t* status;
};

template <int N, int kStages>
struct Smem {
  static constexpr int kHalves = N > 256 ? N / 256 : 1;
  static constexpr int kNI = N / kHalves;
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBHalfBytes = (kNI / 2) * BK * 2;
  static constexpr int kBBytes = kHalves * kBHalfBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = kStages * kStageBytes;
  static constexpr int kNumBars = 2 * kStages + 2;
  static constexpr int kDynamic = kBarOffset + kNumBars * 8 + 16 + 1024;
};

template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

struct Item {
  int b, t0;           // utterance, first output frame of the tile
  int64_t out_row;     // first output row
  int64_t row_end;     // rows >= row_end are not stored
  bool valid;
};

// w-th conv tile in (utterance, frame block) order; invalid past the last one.
__device__ __forceinline__ Item find_item(const Params& p, int64_t w) {
  Item it{0, 0, 0, 0, false};
  for (int b = 0; b < p.groups; ++b) {
    const int lo = p.offsets[b], hi = p.offsets[b + 1];
    const int frames = hi - lo;
    const int tiles = (frames + p.conv_tpt - 1) / p.conv_tpt;
    if (w < tiles) {
      it.b = b;
      it.t0 = static_cast<int>(w) * p.conv_tpt;
      it.out_row = static_cast<int64_t>(lo + it.t0) * p.conv_f2;
      it.row_end = static_cast<int64_t>(lo + min(it.t0 + p.conv_tpt, frames)) * p.conv_f2;
      it.valid = true;
      return it;
    }
    w -= tiles;
  }
  return it;
}

template <typename T, int N, int kStages>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
conv2_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const Params p) {
  using S = Smem<N, kStages>;
  constexpr int kHalves = S::kHalves;
  constexpr int kNI = S::kNI;
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
  constexpr uint32_t kIdesc = ptx::umma_idesc_f16(kBf16, 2 * BM, kNI);
  constexpr uint32_t kTmemCols = N;
  const uint32_t cta_rank = ptx::cluster_ctarank();

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + kStages * S::kABytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::kBarOffset);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tfull_bar = empty_bar + kStages;
  uint64_t* tempty_bar = tfull_bar + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      ptx::mbar_init(&full_bar[i], 1);
      ptx::mbar_init(&empty_bar[i], 1);
    }
    ptx::mbar_init(tfull_bar, 1);
    ptx::mbar_init(tempty_bar, kEpiWarps * 2);
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async_smem();
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(tmem_slot, kTmemCols);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before_sync();
  ptx::cluster_sync();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  ptx::grid_dep_launch();
  ptx::grid_dep_wait();

  // The pair of iteration `it` takes conv tiles 2w and 2w+1 with w = cluster + it * clusters: rank 0 the even one.  A pair
  // whose second tile does not exist (the very last one) lets rank 1 recompute rank 0's tile and store nothing.
  const int64_t num_clusters = static_cast<int64_t>(gridDim.x >> 1);
  const int64_t first = static_cast<int64_t>(blockIdx.x >> 1);
  const uint32_t a_box_bytes = static_cast<uint32_t>(p.conv_tpt * p.conv_f2 * 128);

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int64_t w = first; ok; w += num_clusters) {
        const Item lead = find_item(p, 2 * w);
        if (!lead.valid) break;
        Item mine = cta_rank == 0 ? lead : find_item(p, 2 * w + 1);
        if (!mine.valid) mine = lead;
        for (int kb = 0; kb < p.num_k_blocks; ++kb) {
          if (!ptx::mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          const uint32_t lead_full = ptx::map_to_cta(&full_bar[stage], 0);
          if (cta_rank == 0) ptx::mbar_expect_tx(&full_bar[stage], 2 * (a_box_bytes + S::kBBytes));
          // K block kb = (tap, 64-channel block).  Tap (kh, kw) of output (t2, f2) reads input frame 2*t2 + kh, feature
          // 2*f2 + kw: parity plane (kh&1)*2 + (kw&1), rows (t2 + kh/2, f2 + kw/2) -- one dense box of tpt x f2 rows x 64
          // channels.  Rows past the box stay stale in shared memory: they only feed accumulator rows never stored.
          const int tap = kb / p.conv_cblocks, cb = kb - tap * p.conv_cblocks;
          const int kh = tap / 3, kw = tap - 3 * kh;
          ptx::tma_load_5d_pair(sA + stage * S::kABytes, &tmap_a, cb * BK, kw >> 1, (kh & 1) * 2 + (kw & 1),
                                mine.t0 + (kh >> 1), mine.b, lead_full);
#pragma unroll
          for (int j = 0; j < kHalves; ++j)
            ptx::tma_load_3d_pair(sB + stage * S::kBBytes + j * S::kBHalfBytes, &tmap_b, kb * BK,
                                  j * kNI + static_cast<int>(cta_rank) * (kNI / 2), 0, lead_full);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok && p.status) atomicOr(p.status, kStatusGemmProducer);
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA) -------------------
    if (lane == 0 && cta_rank == 0) {
      int stage = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int64_t w = first; ok; w += num_clusters) {
        if (!find_item(p, 2 * w).valid) break;
        if (!ptx::mbar_wait(tempty_bar, acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        ptx::tc_fence_after_sync();
        for (int kb = 0; kb < p.num_k_blocks; ++kb) {
          if (!ptx::mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after_sync();
          const uint32_t a_addr = ptx::smem_u32(sA + stage * S::kABytes);
          const uint32_t b_addr = ptx::smem_u32(sB + stage * S::kBBytes);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t adesc = ptx::smem_desc_kmajor_sw128(a_addr + k * UMMA_K * 2);
#pragma unroll
            for (int j = 0; j < kHalves; ++j) {
              const uint64_t bdesc = ptx::smem_desc_kmajor_sw128(b_addr + j * S::kBHalfBytes + k * UMMA_K * 2);
              ptx::umma_f16_pair(tmem_base + j * kNI, adesc, bdesc, kIdesc, (kb | k) != 0 ? 1u : 0u);
            }
          }
          ptx::umma_commit_pair(&empty_bar[stage], 3);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (ok) ptx::umma_commit_pair(tfull_bar, 3);
        acc_phase ^= 1u;
      }
      if (!ok && p.status) atomicOr(p.status, kStatusGemmMma);
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue: thread = (tile row, column half) ---------------
    const int ew = warp - 2;
    const int q = warp & 3;
    const int slice = ew >> 2;
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    const int tile_row = q * 32 + lane;
    const T* bias = static_cast<const T*>(p.bias);
    constexpr int kCols = N / 2;                   // columns per warp
    uint32_t tile_phase = 0;
    bool ok = true;
    for (int64_t w = first; ok; w += num_clusters) {
      const Item lead = find_item(p, 2 * w);
      if (!lead.valid) break;
      Item mine = cta_rank == 0 ? lead : find_item(p, 2 * w + 1);
      const bool have = mine.valid;
      if (!ptx::mbar_wait(tfull_bar, tile_phase, abort_flag)) { ok = false; break; }
      tile_phase ^= 1u;
      ptx::tc_fence_after_sync();
      const int64_t row = mine.out_row + tile_row;
      const bool row_ok = have && tile_row < p.conv_tpt * p.conv_f2 && row < mine.row_end;
      T* drow = static_cast<T*>(p.D) + row * N;
#pragma unroll 1
      for (int c0 = 0; c0 < kCols; c0 += 32) {
        const int col = slice * kCols + c0;
        uint32_t r[32];
        ptx::tmem_ld_32x32(tmem_base + lane_base + col, r);
        ptx::tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[g * 8 + i]);
            if (bias) {
              Pack<T> bb = ld128_nc(bias + col + g * 8);
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] += Elem<T>::to_f(bb.v[i]);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = fmaxf(v[i], 0.f);
            uint4 o;
            o.x = pack2<T>(v[0], v[1]); o.y = pack2<T>(v[2], v[3]);
            o.z = pack2<T>(v[4], v[5]); o.w = pack2<T>(v[6], v[7]);
            *reinterpret_cast<uint4*>(drow + col + g * 8) = o;
          }
        }
      }
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(ptx::map_to_cta(tempty_bar, 0));
    }
    if (!ok && lane == 0 && p.status) atomicOr(p.status, kStatusGemmEpilogue);
  }

  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  ptx::tc_fence_before_sync();
  ptx::cluster_sync();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

int g_enabled = 1;   // "conv2_pairs" tunable: 0 keeps the second subsampling conv on the single-CTA kernel

bool supported(int64_t C, int64_t N) { return g_enabled && (N == 128 || N == 256 || N == 512) && C % 64 == 0; }

template <int N> struct StagesFor;
template <> struct StagesFor<512> { static constexpr int v = 4; };   // 48 KB per stage
template <> struct StagesFor<256> { static constexpr int v = 6; };   // 32 KB per stage
template <> struct StagesFor<128> { static constexpr int v = 8; };   // 24 KB per stage

template <typename T, int N>
int launch(const CUtensorMap& ta, const void* w2, int64_t K, const Params& p, int64_t max_items, int dtype, cudaStream_t s) {
  constexpr int kStages = StagesFor<N>::v;
  using S = Smem<N, kStages>;
  static_assert(S::kDynamic <= 232448, "shared memory budget of one CTA");
  auto kern = conv2_pair_kernel<T, N, kStages>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kDynamic);
  if (e != cudaSuccess) return set_error(OASR_ERR_CUDA, "subsample_conv2: cannot reserve %d bytes of shared memory: %s",
                                         S::kDynamic, cudaGetErrorString(e));
  CUtensorMap tb;
  uint64_t bdims[3] = {(uint64_t)K, (uint64_t)N, 1};
  uint64_t bstr[3] = {0, (uint64_t)K * 2, (uint64_t)K * 2 * (uint64_t)N};
  uint32_t bbox[3] = {BK, (uint32_t)(S::kNI / 2), 1};
  if (int rc = make_tensor_map(&tb, tma_dtype(dtype), 3, w2, bdims, bstr, bbox)) return rc;
  int64_t clusters = sm_count() / 2;
  const int64_t pairs = (max_items + 1) / 2;
  if (pairs < clusters) clusters = pairs;
  if (clusters < 1) clusters = 1;
  launch_pdl(kern, dim3(static_cast<unsigned>(2 * clusters)), dim3(kThreads), S::kDynamic, s, ta, tb, p);
  return check_launch("subsample_conv2 (CTA pairs) launch");
}

// Called by oasr_b200_subsample_conv2 after its argument checks, with the A tensor map it built.
int run(const CUtensorMap& ta, void* out, const void* w2, const void* bias, const int32_t* cu_frames, int64_t B, int64_t C,
        int64_t N, int64_t F2, int tpt, int64_t total_frames, int dtype, cudaStream_t s) {
  Params p{};
  p.N = static_cast<int>(N); p.groups = static_cast<int>(B); p.offsets = cu_frames;
  p.conv_f2 = static_cast<int>(F2); p.conv_tpt = tpt; p.conv_cblocks = static_cast<int>(C / 64);
  p.num_k_blocks = 9 * p.conv_cblocks;
  p.D = out; p.bias = bias; p.status = device_status_ptr();
  const int64_t max_items = total_frames / tpt + B;   // upper bound of the conv tiles (the kernel finds the exact end)
  return OB_DISPATCH_HALF(dtype, T, [&]() -> int {
    switch (N) {
      case 512: return launch<T, 512>(ta, w2, 9 * C, p, max_items, dtype, s);
      case 256: return launch<T, 256>(ta, w2, 9 * C, p, max_items, dtype, s);
      default: return launch<T, 128>(ta, w2, 9 * C, p, max_items, dtype, s);
    }
  });
}

}  // namespace conv2_pair
}  // namespace ob
