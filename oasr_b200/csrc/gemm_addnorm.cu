// Linear + residual add + LayerNorm in ONE kernel for the residual-stream steps of the encoder layer:
//
//   y = A[M,K] . B[N,K]^T + bias            (16-bit operands, fp32 accumulate, never rounded)
//   s = res_in + alpha * y                  (fp32 residual stream in a blocked layout, see res_block_offset;
//                                            res_in nullable)
//   mode 0:  res_out = s,        h = LN_a(s)
//   mode 1:  res_out = s,        h = s * w_a + b_a          (fp32 per-channel scale/shift: a folded BatchNorm)
//   mode 2:  res_out = LN_a(s),  h = LN_b(res_out)          (optionally h as [hi | lo], 2N wide)
//
// It replaces a GEMM launch, the 16-bit round trip of y through HBM and an add+norm launch
// (ConformerEncoderLayer.forward_packed: `x = residual + alpha * sub(x); x = norm(x)`,
// oasr/models/conformer/model.py:722-751; fused reference form include/oasr/norm.cuh:396-484).
//
// Shape of the kernel.  The whole output row must sit in one CTA for the row statistics, so a CTA
// owns 128 rows x N columns (N = 128, 256 or 512 = the fp32 columns of tensor memory).  Two CTAs of
// a cluster form a pair that computes 256 rows with tcgen05 cta_group::2: each CTA stages its own
// 128 rows of A and HALF of the B rows of every instruction, so per flop a CTA writes and reads
// half the B bytes in shared memory -- at K = 512 shared-memory bandwidth, not the tensor pipe, is
// what limits a single-CTA 128 x 256 tile.  No multicast: every CTA loads its own bytes.
//   warp 0   TMA producer (A tile + its B rows per 64-wide K block, kStages-deep ring)
//   warp 1   MMA issuer (leader CTA only; N/256 instructions of N<=256 per K16 step) + TMEM owner
//   warps 2-17  epilogue, four threads per output row (tcgen05.ld 32x32b: lane = row; the four warps that share a
//             TMEM lane quarter take one quarter of the row's columns each -- the passes below are chains of load
//             latencies, so what they need is warps to switch between; two per scheduler left the SM idle 3/4 of the time):
//     pass 1  s = res + alpha*(acc + bias) per 16-column chunk; the residual stream lives in HBM in 32 x 32
//             blocks laid out so that a warp (lane = row) reads and writes half a block with four coalesced 512-byte
//             accesses straight from registers (the next chunk is requested before this one is processed, the
//             first one under the main loop); s also goes back into the accumulator's own TMEM columns; running
//             sums for mean / variance about the slice's first value, combined across the four slices through
//             shared memory
//     pass 2  re-reads s from TMEM, normalises, rounds once, stages 32 x 32 pieces (64-byte swizzle, two chunks each)
//             and TMA-stores them (mode 2: writes LN_a(s) as fp32 instead, keeps it in TMEM, pass 3 stores h)
// Every wait is bounded (mbar_wait); on give-up the CTA drains and raises the device status word.
#include <cuda.h>

#include <type_traits>

#include "common.cuh"
#include "device_status.cuh"
#include "sm100_ptx.cuh"
#include "tma_host.cuh"

namespace ob {
namespace gan {

constexpr int BM = 128;      // rows per CTA (= TMEM lanes)
constexpr int BK = 64;       // K elements per stage (128-byte rows)
constexpr int UMMA_K = 16;
constexpr int kEpiWarps = 16; // four warps per TMEM lane quarter: each handles one quarter of the row's columns
constexpr int kThreads = 64 + 32 * kEpiWarps;
constexpr int kChunk = 16;   // columns per epilogue step (two steps fill one 32 x 32 h piece)
constexpr int kSlices = kEpiWarps / 4;   // column slices of a row (threads that share a row)
// per epilogue warp: one 32 x 32 16-bit staging buffer for h (2 KB, 64-byte swizzle)
constexpr int kWarpEpiBytes = 2048;

struct Params {
  int M, N, K;
  int num_k_blocks;
  int num_pairs;           // 256-row tiles
  const void* bias;        // T[N], nullable
  float alpha;
  int mode;                // 0, 1, 2 as above
  int split_out;           // mode 2: h rows are [hi | lo]
  const float* res_in;     // fp32 residual stream in the blocked layout described at the top, nullable
  float* res_out;          // same layout, nullable unless mode 2; may alias res_in
  const void *w_a, *b_a;   // T[N] (mode 1: float[N])
  const void *w_b, *b_b;   // T[N], mode 2
  float eps;
  uint32_t* status;
  unsigned long long* trace;   // nullable: CTA 0 writes clock stamps of its phases here (diagnostics)
};

template <int N, int kStages>
struct Smem {
  static constexpr int kHalves = N > 256 ? N / 256 : 1;     // MMA instructions per K16 step
  static constexpr int kNI = N / kHalves;                   // N of one instruction (pair-wide)
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBHalfBytes = (kNI / 2) * BK * 2;    // this CTA's B rows of one instruction
  static constexpr int kBBytes = kHalves * kBHalfBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kRing = kStages * kStageBytes;
  static constexpr int kWarpEpi = kWarpEpiBytes;
  static constexpr int kEpiOffset = kRing;
  static constexpr int kBarOffset = kEpiOffset + kEpiWarps * kWarpEpi;
  static constexpr int kNumBars = 2 * kStages + 2 + 2;
  static constexpr int kTotal = kBarOffset + kNumBars * 8 + 16;
  static constexpr int kDynamic = kTotal + 1024;
};

// The epilogue passes are bound by their instruction count: the element-wise arithmetic runs two columns per
// instruction (fp32x2 add / mul / fma, each component rounded exactly as the scalar operation).
__device__ __forceinline__ float2 f2at(const float* f, int i) { return make_float2(f[2 * i], f[2 * i + 1]); }
__device__ __forceinline__ float2 pairu(const uint32_t* r, int i) {
  return make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
}
__device__ __forceinline__ float2 splat(float x) { return make_float2(x, x); }
__device__ __forceinline__ float u2f(uint32_t u) { return __uint_as_float(u); }
__device__ __forceinline__ uint32_t f2u(float f) { return __float_as_uint(f); }

template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// 16 consecutive parameters (16-bit or fp32) starting at p as floats; warp-uniform addresses (broadcast loads).
template <typename P>
__device__ __forceinline__ void load_params16(const P* p, float (&f)[16]) {
  if constexpr (std::is_same<P, float>::value) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(p) + i);
      f[4 * i] = v.x; f[4 * i + 1] = v.y; f[4 * i + 2] = v.z; f[4 * i + 3] = v.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      Pack<P> v = ld128_nc(p + 8 * i);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[8 * i + j] = Elem<P>::to_f(v.v[j]);
    }
  }
}

// Blocked layout of the fp32 residual stream: the matrix is cut into blocks of 32 rows x 32 columns, blocks of a
// row band back to back (band-major); inside a block the 16-byte piece j (columns 4j..4j+3) of row l sits at
// float4 index j*32 + l.  A warp whose lane l owns row l of a band then moves a block with eight fully
// coalesced 512-byte accesses, no staging in shared memory.
__device__ __forceinline__ int64_t res_block_offset(int band, int chunk, int n_chunks) {
  return (static_cast<int64_t>(band) * n_chunks + chunk) * 1024;   // in floats
}
__device__ __forceinline__ float4 ld_res(const float* p) {
  float4 v;
  asm volatile("ld.global.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ void stamp(const Params& p, int slot) {
  if (p.trace != nullptr && blockIdx.x == 0) p.trace[slot] = static_cast<unsigned long long>(clock64());
}

template <typename T, int N, int kStages>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_addnorm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_h, const Params p) {
  using S = Smem<N, kStages>;
  constexpr int kHalves = S::kHalves;
  constexpr int kNI = S::kNI;
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
  constexpr uint32_t kIdesc = ptx::umma_idesc_f16(kBf16, 2 * BM, kNI);
  constexpr uint32_t kTmemCols = N;              // 128, 256 or 512: a power of two >= 32
  constexpr int kChunks = N / kChunk;
  const uint32_t cta_rank = ptx::cluster_ctarank();

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + kStages * S::kABytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::kBarOffset);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tfull_bar = empty_bar + kStages;
  uint64_t* tempty_bar = tfull_bar + 1;
  uint64_t* stat_bar = tempty_bar + 1;           // [2]: every warp has published its slice's row statistics
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(stat_bar + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      ptx::mbar_init(&full_bar[i], 1);
      ptx::mbar_init(&empty_bar[i], 1);
    }
    ptx::mbar_init(tfull_bar, 1);
    ptx::mbar_init(tempty_bar, kEpiWarps * 2);   // the leader waits for both CTAs' epilogue warps
    ptx::mbar_init(&stat_bar[0], kEpiWarps);
    ptx::mbar_init(&stat_bar[1], kEpiWarps);
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async_smem();
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_b);
    ptx::prefetch_tensormap(&tmap_h);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(tmem_slot, kTmemCols);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before_sync();
  ptx::cluster_sync();                           // the peer's barriers exist before anything targets them
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  ptx::grid_dep_launch();
  ptx::grid_dep_wait();

  const int num_clusters = static_cast<int>(gridDim.x >> 1);
  const int first_pair = static_cast<int>(blockIdx.x >> 1);
  if (threadIdx.x == 0) stamp(p, 0);

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int pair = first_pair; ok && pair < p.num_pairs; pair += num_clusters) {
        const int a_row = pair * 2 * BM + static_cast<int>(cta_rank) * BM;
        for (int kb = 0; kb < p.num_k_blocks; ++kb) {
          if (!ptx::mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          // both CTAs' bytes are credited to the leader's barrier; only the leader arrives on it
          const uint32_t lead_full = ptx::map_to_cta(&full_bar[stage], 0);
          if (cta_rank == 0) ptx::mbar_expect_tx(&full_bar[stage], 2 * S::kStageBytes);
          if (kb == 0) stamp(p, 1);
          ptx::tma_load_3d_pair(sA + stage * S::kABytes, &tmap_a, kb * BK, a_row, 0, lead_full);
#pragma unroll
          for (int j = 0; j < kHalves; ++j) {
            // instruction j covers output columns [j*kNI, (j+1)*kNI): this CTA supplies rows rank*kNI/2 .. of them
            ptx::tma_load_3d_pair(sB + stage * S::kBBytes + j * S::kBHalfBytes, &tmap_b, kb * BK,
                                  j * kNI + static_cast<int>(cta_rank) * (kNI / 2), 0, lead_full);
          }
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
      for (int pair = first_pair; ok && pair < p.num_pairs; pair += num_clusters) {
        if (!ptx::mbar_wait(tempty_bar, acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        ptx::tc_fence_after_sync();
        for (int kb = 0; kb < p.num_k_blocks; ++kb) {
          if (!ptx::mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after_sync();
          if (kb == 0) stamp(p, 2);
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
          ptx::umma_commit_pair(&empty_bar[stage], 3);    // frees the stage in both CTAs
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (ok) ptx::umma_commit_pair(tfull_bar, 3);      // the accumulators of both CTAs are complete
        stamp(p, 3);
        acc_phase ^= 1u;
      }
      if (!ok && p.status) atomicOr(p.status, kStatusGemmMma);
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue: thread = (output row, column slice) ---------------
    const int ew = warp - 2;                       // epilogue warp index 0..15
    const int q = warp & 3;                        // TMEM lane quarter this warp may access
    const int slice = ew >> 2;                     // which quarter of the row's columns this warp handles
    constexpr int kLocal = kChunks / kSlices;      // 16-column chunks per thread (even: two chunks make one h piece)
    static_assert(kLocal >= 2 && kLocal % 2 == 0, "a thread fills whole 32-column h pieces");
    const int c_lo = slice * kLocal;
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    uint8_t* hbuf = smem + S::kEpiOffset + ew * S::kWarpEpi;            // 2 KB: one 32 x 32 h piece; also the statistics mailbox
    uint8_t* quarter_bufs = smem + S::kEpiOffset + (ew & 3) * S::kWarpEpi;   // + 4 * t * kWarpEpi: the warps of this lane quarter
    uint32_t tile_phase = 0;
    bool ok = true;
    const T* bias = static_cast<const T*>(p.bias);
    const int sw64 = (lane >> 1) & 3;              // chunk XOR of this thread's row in a 64-byte-swizzled buffer

    // 16 values rounded to T into half `half` of this thread's 64-byte row of the staging buffer
    auto half_row_store = [&](const float (&v)[16], int half) {
      uint8_t* row = hbuf + lane * 64;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        *reinterpret_cast<uint4*>(row + (((2 * half + c) ^ sw64) << 4)) =
            make_uint4(pack2<T>(v[8 * c], v[8 * c + 1]), pack2<T>(v[8 * c + 2], v[8 * c + 3]),
                       pack2<T>(v[8 * c + 4], v[8 * c + 5]), pack2<T>(v[8 * c + 6], v[8 * c + 7]));
      }
    };
    // Before the staging buffer is rewritten: the TMA store issued from it has read it.
    auto h_buffer_free = [&]() {
      if (lane == 0) ptx::bulk_wait_group_read<0>();
      __syncwarp();
    };
    // The 32 x 32 piece in the staging buffer leaves for columns [col, col + 32) of the output rows of this warp.
    auto h_piece_out = [&](int col, int row0_, bool live) {
      ptx::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        if (live) ptx::tma_store_3d(&tmap_h, hbuf, col, row0_, 0);
        ptx::bulk_commit_group();
      }
    };
    // Row statistics of the four column slices -> statistics of the whole row.  Every thread mails (mean, M2) of its
    // slice to the four warps of its lane quarter (their staging buffers are idle at that point: every store has read
    // its buffer before the previous tile ended, and no h is staged before the statistics are known), all warps meet
    // on an mbarrier (bounded wait), and each thread combines the four entries of its own buffer in slice order, so
    // that the four threads of a row get bit-identical mean / rstd.
    auto combine_stats = [&](int which, float pivot_, float sum_, float sq_, float& mean_, float& rstd_) -> bool {
      constexpr float n_s = static_cast<float>(N / kSlices);
      const float m_s = sum_ / n_s;                              // mean of (x - pivot) over the slice
      const float mean_s = pivot_ + m_s;
      const float m2_s = fmaxf(sq_ - sum_ * m_s, 0.f);           // sum of squared deviations from the slice mean
#pragma unroll
      for (int t = 0; t < kSlices; ++t)
        *reinterpret_cast<float2*>(quarter_bufs + t * 4 * S::kWarpEpi + which * 1024 + (slice * 32 + lane) * 8) =
            make_float2(mean_s, m2_s);
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&stat_bar[which]);
      if (!ptx::mbar_wait(&stat_bar[which], tile_phase, abort_flag)) return false;
      float n = 0.f, mean = 0.f, m2 = 0.f;
#pragma unroll
      for (int t = 0; t < kSlices; ++t) {
        const float2 o = *reinterpret_cast<const float2*>(hbuf + which * 1024 + (t * 32 + lane) * 8);
        const float delta = o.x - mean;
        const float n_new = n + n_s;
        mean += delta * (n_s / n_new);
        m2 += o.y + delta * delta * (n * n_s / n_new);
        n = n_new;
      }
      mean_ = mean;
      rstd_ = rsqrtf(m2 / static_cast<float>(N) + p.eps);
      __syncwarp();                                              // every lane has read its mailbox before h is staged over it
      return true;
    };
    // The per-column parameters (bias, gamma / beta or scale / shift) are read by every thread, 16 at a time, from
    // warp-uniform addresses: pull their lines into L1 once, under the main loop, so that the per-chunk loads hit.
    {
      auto prefetch_vec = [&](const void* ptr, int bytes) {
        if (ptr == nullptr) return;
        const char* b = static_cast<const char*>(ptr);
        for (int off = (ew * 32 + lane) * 128; off < bytes; off += kEpiWarps * 32 * 128)
          asm volatile("prefetch.global.L1 [%0];" ::"l"(b + off));
      };
      const int pbytes = N * (p.mode == 1 ? 4 : 2);
      prefetch_vec(p.bias, N * 2);
      prefetch_vec(p.w_a, pbytes);
      prefetch_vec(p.b_a, pbytes);
      prefetch_vec(p.w_b, N * 2);
      prefetch_vec(p.b_b, N * 2);
    }

    for (int pair = first_pair; ok && pair < p.num_pairs; pair += num_clusters) {
      const int row0 = pair * 2 * BM + static_cast<int>(cta_rank) * BM + q * 32;   // first row of this warp (a 32-row band)
      const bool warp_live = row0 < p.M;           // a band wholly past M has no storage: it neither loads nor stores
      const uint32_t t_acc = tmem_base + lane_base;
      const bool use_rin = p.res_in != nullptr && warp_live;
      const bool store_res = p.res_out != nullptr && warp_live;
      const int band = row0 >> 5;
      // this thread's pieces of 16-column chunk c: the half (c & 1) of residual block (band, c >> 1), float4 index
      // ((c & 1) * 4 + j) * 32 + lane, j = 0..3
      auto res_ptr = [&](const float* base, int c) {
        return base + res_block_offset(band, c >> 1, N / 32) + ((c & 1) * 128 + lane) * 4;
      };
      float4 nxt[4];
      if (use_rin) {                               // the first chunk travels under the main loop
        const float* src = res_ptr(p.res_in, c_lo);
#pragma unroll
        for (int j = 0; j < 4; ++j) nxt[j] = ld_res(src + j * 128);
      }

      if (!ptx::mbar_wait(tfull_bar, tile_phase, abort_flag)) { ok = false; break; }
      ptx::tc_fence_after_sync();
      if (ew == 0 && lane == 0) stamp(p, 4);

      // ---------------- pass 1: s = res + alpha * (acc + bias), statistics about the slice's first value ----------------
      float pivot = 0.f;
      float2 sum2 = make_float2(0.f, 0.f), sq2v = make_float2(0.f, 0.f);
#pragma unroll 1
      for (int i = 0; i < kLocal; ++i) {
        const int c = c_lo + i;
        uint32_t r[16];
        ptx::tmem_ld_32x16(t_acc + c * kChunk, r);
        float s[16];
        if (use_rin) {
#pragma unroll
          for (int j = 0; j < 4; ++j) { s[4 * j] = nxt[j].x; s[4 * j + 1] = nxt[j].y; s[4 * j + 2] = nxt[j].z; s[4 * j + 3] = nxt[j].w; }
          if (i + 1 < kLocal) {                    // the next chunk is in flight while this one is processed
            const float* src = res_ptr(p.res_in, c + 1);
#pragma unroll
            for (int j = 0; j < 4; ++j) nxt[j] = ld_res(src + j * 128);
          }
        } else {
#pragma unroll
          for (int k = 0; k < 16; ++k) s[k] = 0.f;
        }
        float bb[16];
        if (bias) load_params16(bias + c * kChunk, bb);
        ptx::tmem_ld_wait();
        if (bias) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const float2 t = __ffma2_rn(splat(p.alpha), __fadd2_rn(pairu(r, k), f2at(bb, k)), f2at(s, k));
            s[2 * k] = t.x; s[2 * k + 1] = t.y;
          }
        } else {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const float2 t = __ffma2_rn(splat(p.alpha), pairu(r, k), f2at(s, k));
            s[2 * k] = t.x; s[2 * k + 1] = t.y;
          }
        }
        if (store_res && p.mode != 2) {
          float* dst = const_cast<float*>(res_ptr(p.res_out, c));
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *reinterpret_cast<float4*>(dst + j * 128) = make_float4(s[4 * j], s[4 * j + 1], s[4 * j + 2], s[4 * j + 3]);
        }
        if (p.mode == 1) {
          // affine pre-norm: no statistics, h leaves in this pass
          float sc[16], sh[16], o[16];
          load_params16(static_cast<const float*>(p.w_a) + c * kChunk, sc);
          load_params16(static_cast<const float*>(p.b_a) + c * kChunk, sh);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const float2 t = __ffma2_rn(f2at(s, k), f2at(sc, k), f2at(sh, k));
            o[2 * k] = t.x; o[2 * k + 1] = t.y;
          }
          if ((c & 1) == 0) h_buffer_free();
          half_row_store(o, c & 1);
          if (c & 1) h_piece_out((c >> 1) * 32, row0, warp_live);
        } else {
          if (i == 0) pivot = s[0];
#pragma unroll
          for (int k = 0; k < 8; ++k) {     // even and odd columns keep separate running sums, added at the end
            const float2 d = __fadd2_rn(f2at(s, k), splat(-pivot));
            sum2 = __fadd2_rn(sum2, d);
            sq2v = __ffma2_rn(d, d, sq2v);
          }
#pragma unroll
          for (int k = 0; k < 16; ++k) r[k] = f2u(s[k]);
          ptx::tmem_st_32x16(t_acc + c * kChunk, r);
        }
      }
      if (ew == 0 && lane == 0) stamp(p, 5);

      if (p.mode != 1) {
        ptx::tmem_st_wait();                       // pass 1's writes of s are in TMEM before anything reads them back
        float mean, rstd;
        if (!combine_stats(0, pivot, sum2.x + sum2.y, sq2v.x + sq2v.y, mean, rstd)) { ok = false; break; }
        const T* g1 = static_cast<const T*>(p.w_a);
        const T* b1 = static_cast<const T*>(p.b_a);
        if (p.mode == 2) {
          // ---------------- pass 2 (mode 2): res_out = LN_a(s), kept in TMEM, statistics of it ----------------
          float pivot2 = 0.f;
          float2 sumb = make_float2(0.f, 0.f), sqb = make_float2(0.f, 0.f);
#pragma unroll 1
          for (int i = 0; i < kLocal; ++i) {
            const int c = c_lo + i;
            uint32_t r[16];
            ptx::tmem_ld_32x16(t_acc + c * kChunk, r);
            float gg[16], bb[16], v[16];
            load_params16(g1 + c * kChunk, gg);
            load_params16(b1 + c * kChunk, bb);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const float2 t = __ffma2_rn(__fmul2_rn(__fadd2_rn(pairu(r, k), splat(-mean)), splat(rstd)), f2at(gg, k), f2at(bb, k));
              v[2 * k] = t.x; v[2 * k + 1] = t.y;
            }
            if (i == 0) pivot2 = v[0];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const float2 d = __fadd2_rn(f2at(v, k), splat(-pivot2));
              sumb = __fadd2_rn(sumb, d);
              sqb = __ffma2_rn(d, d, sqb);
            }
#pragma unroll
            for (int k = 0; k < 16; ++k) r[k] = f2u(v[k]);
            ptx::tmem_st_32x16(t_acc + c * kChunk, r);
            if (store_res) {
              float* dst = const_cast<float*>(res_ptr(p.res_out, c));
#pragma unroll
              for (int j = 0; j < 4; ++j)
                *reinterpret_cast<float4*>(dst + j * 128) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            }
          }
          if (ew == 0 && lane == 0) stamp(p, 6);
          ptx::tmem_st_wait();
          if (!combine_stats(1, pivot2, sumb.x + sumb.y, sqb.x + sqb.y, mean, rstd)) { ok = false; break; }
          g1 = static_cast<const T*>(p.w_b);
          b1 = static_cast<const T*>(p.b_b);
        }
        // ---------------- last pass: h = LN(row in TMEM), rounded once, 32 x 32 pieces out by TMA ----------------
        // With split_out the pass runs twice: h = hi + lo with hi = round16(h) into columns [0, N), then
        // lo = round16(h - hi) into columns [N, 2N).
        const int parts = p.split_out ? 2 : 1;
#pragma unroll 1
        for (int part = 0; part < parts; ++part) {
#pragma unroll 1
          for (int i = 0; i < kLocal; ++i) {
            const int c = c_lo + i;
            uint32_t r[16];
            ptx::tmem_ld_32x16(t_acc + c * kChunk, r);
            float gg[16], bb[16], v[16];
            load_params16(g1 + c * kChunk, gg);
            load_params16(b1 + c * kChunk, bb);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const float2 t = __ffma2_rn(__fmul2_rn(__fadd2_rn(pairu(r, k), splat(-mean)), splat(rstd)), f2at(gg, k), f2at(bb, k));
              v[2 * k] = t.x; v[2 * k + 1] = t.y;
            }
            if (part == 1) {
#pragma unroll
              for (int k = 0; k < 16; ++k) v[k] = v[k] - Elem<T>::to_f(Elem<T>::from_f(v[k]));
            }
            if ((c & 1) == 0) h_buffer_free();
            half_row_store(v, c & 1);
            if (c & 1) h_piece_out(part * N + (c >> 1) * 32, row0, warp_live);
          }
        }
      }
      if (ew == 0 && lane == 0) stamp(p, 7);
      // Tile done.  All of this warp's stores have read the staging buffer (the quarter's warps write statistics into
      // it during the next tile); then the accumulator columns go back to the leader's MMA issuer.
      if (lane == 0) ptx::bulk_wait_group_read<0>();
      __syncwarp();
      tile_phase ^= 1u;
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(ptx::map_to_cta(tempty_bar, 0));
    }
    if (lane == 0) ptx::bulk_wait_group<0>();      // every h piece has landed
    if (ew == 0 && lane == 0) stamp(p, 8);
    if (!ok && lane == 0 && p.status) atomicOr(p.status, kStatusGemmEpilogue);
  }

  // Teardown.  After an abandoned wait, give copies that may still be in flight time to land before shared
  // memory and TMEM are released.  Neither CTA may leave while the leader's MMAs can still read the peer's
  // shared memory or the peer can still arrive on the leader's barriers.
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
  if (threadIdx.x == 0) stamp(p, 9);
}

template <int N> struct StagesFor;
template <> struct StagesFor<512> { static constexpr int v = 4; };   // 48 KB per stage + 32 KB of h staging
template <> struct StagesFor<256> { static constexpr int v = 5; };   // 32 KB per stage
template <> struct StagesFor<128> { static constexpr int v = 6; };   // 24 KB per stage

struct Call {
  void* h_out;
  float* res_out;
  const float* res_in;
  const void *A, *B;
  int64_t M, N, K;
  int dtype;
  Params p;
};

template <typename T, int N>
int launch(const Call& c, cudaStream_t s) {
  constexpr int kStages = StagesFor<N>::v;
  using S = Smem<N, kStages>;
  static_assert(S::kDynamic <= 232448, "shared memory budget of one CTA");
  auto kern = gemm_addnorm_kernel<T, N, kStages>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kDynamic);
    if (e != cudaSuccess) return set_error(OASR_ERR_CUDA, "gemm_add_norm_f32: cannot reserve %d bytes of shared memory: %s",
                                           S::kDynamic, cudaGetErrorString(e));
    attr_done = true;
  }
  CUtensorMap ta, tb, th;
  const uint64_t M = static_cast<uint64_t>(c.M), K = static_cast<uint64_t>(c.K);
  {
    uint64_t dims[3] = {K, M, 1};
    uint64_t str[3] = {0, K * 2, K * 2 * M};
    uint32_t box[3] = {BK, BM, 1};
    if (int rc = make_tensor_map(&ta, tma_dtype(c.dtype), 3, c.A, dims, str, box)) return rc;
  }
  {
    uint64_t dims[3] = {K, static_cast<uint64_t>(N), 1};
    uint64_t str[3] = {0, K * 2, K * 2 * N};
    uint32_t box[3] = {BK, static_cast<uint32_t>(S::kNI / 2), 1};
    if (int rc = make_tensor_map(&tb, tma_dtype(c.dtype), 3, c.B, dims, str, box)) return rc;
  }
  {
    const uint64_t w = static_cast<uint64_t>(N) * (c.p.split_out ? 2 : 1);
    uint64_t dims[3] = {w, M, 1};
    uint64_t str[3] = {0, w * 2, w * 2 * M};
    uint32_t box[3] = {32, 32, 1};
    if (int rc = make_tensor_map(&th, tma_dtype(c.dtype), 3, c.h_out, dims, str, box, CU_TENSOR_MAP_SWIZZLE_64B)) return rc;
  }
  int64_t clusters = sm_count() / 2;
  if (c.p.num_pairs < clusters) clusters = c.p.num_pairs;
  if (clusters < 1) clusters = 1;
  launch_pdl(kern, dim3(static_cast<unsigned>(2 * clusters)), dim3(kThreads), S::kDynamic, s, ta, tb, th, c.p);
  return check_launch("gemm_add_norm_f32 launch");
}

}  // namespace gan
}  // namespace ob

extern "C" {


int oasr_b200_gemm_add_norm_supported(int64_t N, int64_t K) {
  return (N == 128 || N == 256 || N == 512) && K >= 64 && K % 8 == 0 ? 1 : 0;
}

int oasr_b200_gemm_add_norm_f32(void* h_out, float* res_out, const float* res_in, const void* A, const void* B,
                                const void* bias, int64_t M, int64_t N, int64_t K, double alpha, int mode,
                                const void* w_a, const void* b_a, const void* w_b, const void* b_b, double eps,
                                int split_out, int dtype, void* stream) {
  using namespace ob;
  using namespace ob::gan;
  OB_REQUIRE(M >= 0 && N > 0 && K > 0, OASR_ERR_INVALID, "gemm_add_norm_f32: bad shape M=%lld N=%lld K=%lld", (long long)M,
             (long long)N, (long long)K);
  if (M == 0) return OASR_OK;
  OB_REQUIRE(oasr_b200_gemm_add_norm_supported(N, K), OASR_ERR_UNSUPPORTED,
             "gemm_add_norm_f32: the output row must fill tensor memory exactly (N = 128, 256 or 512) and K must be a "
             "multiple of 8, at least 64 (got N=%lld K=%lld); use gemm + add_norm_f32 for other widths",
             (long long)N, (long long)K);
  OB_REQUIRE(h_out && A && B && w_a && b_a, OASR_ERR_INVALID, "gemm_add_norm_f32: null pointer argument");
  OB_REQUIRE(mode >= 0 && mode <= 2, OASR_ERR_INVALID, "gemm_add_norm_f32: mode must be 0, 1 or 2");
  OB_REQUIRE(mode != 2 || (res_out && w_b && b_b), OASR_ERR_INVALID, "gemm_add_norm_f32: mode 2 needs res_out and the second norm");
  OB_REQUIRE(!split_out || mode == 2, OASR_ERR_INVALID, "gemm_add_norm_f32: the [hi | lo] output exists for mode 2 only");
  OB_REQUIRE(M < (int64_t(1) << 31) && K < (1 << 30), OASR_ERR_INVALID, "gemm_add_norm_f32: extent too large");
  OB_REQUIRE(is_aligned(h_out, 16) && is_aligned(A, 16) && is_aligned(B, 16) && (!bias || is_aligned(bias, 16)) &&
                 (!res_in || is_aligned(res_in, 16)) && (!res_out || is_aligned(res_out, 16)) && is_aligned(w_a, 16) &&
                 is_aligned(b_a, 16) && (!w_b || is_aligned(w_b, 16)) && (!b_b || is_aligned(b_b, 16)),
             OASR_ERR_ALIGN, "gemm_add_norm_f32: pointers must be 16-byte aligned");
  Call c{};
  c.h_out = h_out; c.res_out = res_out; c.res_in = res_in; c.A = A; c.B = B;
  c.M = M; c.N = N; c.K = K; c.dtype = dtype;
  Params& p = c.p;
  p.M = static_cast<int>(M); p.N = static_cast<int>(N); p.K = static_cast<int>(K);
  p.num_k_blocks = static_cast<int>((K + BK - 1) / BK);
  p.num_pairs = static_cast<int>((M + 2 * BM - 1) / (2 * BM));
  p.bias = bias; p.alpha = static_cast<float>(alpha); p.mode = mode; p.split_out = split_out ? 1 : 0;
  p.res_in = res_in; p.res_out = res_out;
  p.w_a = w_a; p.b_a = b_a; p.w_b = w_b; p.b_b = b_b; p.eps = static_cast<float>(eps);
  p.status = device_status_ptr();
  p.trace = g_trace_buffer;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return OB_DISPATCH_HALF(dtype, T, [&]() -> int {
    switch (N) {
      case 512: return launch<T, 512>(c, s);
      case 256: return launch<T, 256>(c, s);
      default: return launch<T, 128>(c, s);
    }
  });
}

}  // extern "C"
