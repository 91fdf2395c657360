// GEMM family on the 5th-generation tensor cores:
//   D[M,N] = epilogue(A[M,K] . B[N,K]^T + bias[N]),  A/B fp16 or bf16, fp32 accumulate.
//
// One persistent, warp-specialised kernel (192 or 320 threads, one CTA per SM):
//   warp 0   TMA producer: streams 128x64 A tiles and BNx64 B tiles (128-byte
//            swizzle) into a kStages-deep shared-memory ring, one mbarrier pair
//            (full/empty) per stage;
//   warp 1   MMA issuer: one elected thread issues tcgen05.mma (M=128, N=BN,
//            K=16) four times per stage into a TMEM accumulator and commits the
//            stage back to the producer; owns the TMEM allocation (2 x BN
//            columns, so the epilogue of tile i overlaps the main loop of i+1);
//   warps 2-5 (and 6-9 for the store / GLU epilogues) epilogue: tcgen05.ld the
//            accumulator (lane = row, 32 columns per load), apply bias /
//            activation / residual / GLU / log-softmax in fp32, round once, stage
//            128-byte row pieces in swizzled shared memory and TMA-store them.
// Tensor-pipe bound; algorithmic flops 2*M*N*K.  No cluster launch and no TMA
// multicast: every CTA loads its own operands.
//
// The reference reaches the same tensor cores through CUTLASS 3.x with one
// fixed 128x128x128 tile (include/oasr/gemm/gemm.cuh:57-59,
// oasr/jit/gemm.py:863-880); epilogue numerics follow its fusion functors
// (include/oasr/common/epilogue_functors.h): fp32 accumulate, + bias in fp32,
// activation in fp32, one rounding to the output type.
#include <cuda.h>

#include <cstdlib>
#include <type_traits>

#include "common.cuh"
#include "device_status.cuh"
#include "sm100_ptx.cuh"
#include "tma_host.cuh"

namespace ob {
namespace gemm {

constexpr int BM = 128;   // rows per tile (= UMMA M, = TMEM lanes)
constexpr int BK = 64;    // K elements per stage (= 128 bytes = one swizzle row)
constexpr int UMMA_K = 16;
constexpr int kEpiWarps = 4;  // per group; store / GLU epilogues run two groups (8 warps)

enum Epi { kEpiStore = 0, kEpiResid = 1, kEpiGlu = 2, kEpiLsm = 3 };
enum Sched { kSchedDense = 0, kSchedGroup = 1, kSchedSweep = 2, kSchedConv = 3 };

struct Params {
  int M, N, K;            // per-problem extents (N = output columns)
  int batch;              // dense: number of independent problems (bmm)
  int num_m_tiles, num_n_tiles, num_k_blocks;
  int groups;             // grouped: number of groups
  const int32_t* offsets; // grouped: cumulative end rows (device)
  void* D;                // output (T, or float for kEpiResid / fp32 log-probs)
  const void* bias;       // nullable, T[N] (GLU: T[2N])
  const float* R_in;      // kEpiResid
  float alpha;
  int act;
  int out_f32;            // kEpiLsm: 1 = fp32 output, 0 = T output
  int lsm_passes;         // kEpiLsm: 2 = statistics sweep + normalised-output sweep; 1 = statistics only (argmax, no output)
  int32_t* argmax;        // kEpiLsm: nullable
  uint32_t* status;       // device status word (nullable)
  int dup_cols;           // kDup: output columns [0, dup_cols) of the GEMM are stored twice (see gemm_body)
  // kSchedConv (3x3 / stride-2 convolution as an implicit GEMM over a parity-split NHWC input):
  // 8-bit operand kinds: D = (A_q . B_q^T) * a_scale[row] * b_scale[col] (+ bias)
  const float* a_scale;   // [M] per-row (per-token) scales of A
  const float* b_scale;   // [N] (GLU: [2N]) per-row (per-output-channel) scales of B
  int conv_f2;            // output positions per output frame (rows of one frame in a tile)
  int conv_tpt;           // output frames per 128-row tile = 128 / conv_f2
  int conv_cblocks;       // input channels / 64
};

struct Tile {
  int a_row, a_batch;   // TMA coordinates of the A tile
  int b_row, b_batch;   // TMA coordinates of the B tile
  int64_t out_row;      // first output row of the tile
  int64_t row_end;      // rows >= row_end are not stored
  int n0;               // first output column
  int pass, n_idx;      // sweep scheduler only
};

template <int kSched, int BN, int kCtas = 1>
struct Scheduler {
  const Params& p;
  uint32_t rank = 0;  // CTA rank inside a pair (kCtas == 2)
  __device__ explicit Scheduler(const Params& p_) : p(p_) {}
  // Does this CTA have an iter-th work item?  The MMA issuer needs nothing else from the scheduler,
  // and a tile boundary is where a stalled issuer starves the tensor pipe.
  __device__ bool has(int iter) const {
    if constexpr (kSched == kSchedDense) {
      const uint32_t ctas = kCtas == 2 ? (gridDim.x >> 1) : gridDim.x;
      const uint32_t first = kCtas == 2 ? (blockIdx.x >> 1) : blockIdx.x;
      const uint32_t total = static_cast<uint32_t>(p.num_m_tiles) * p.num_n_tiles * p.batch;
      return first + static_cast<uint32_t>(iter) * ctas < total;
    } else if constexpr (kSched == kSchedSweep) {
      return blockIdx.x + static_cast<uint32_t>(iter / (p.lsm_passes * p.num_n_tiles)) * gridDim.x < static_cast<uint32_t>(p.num_m_tiles);
    } else {
      Tile t;
      return get(iter, t);
    }
  }
  // iter-th work item of this CTA; false when the CTA has no more work.
  __device__ bool get(int iter, Tile& t) const {
    if constexpr (kSched == kSchedDense && kCtas == 2) {
      // a pair of CTAs owns a 256-row x BN tile: CTA `rank` holds rows [m*256 + rank*128, +128) of A and
      // rows [n*BN + rank*BN/2, +BN/2) of B (GLU: rank 0 the value rows, rank 1 the gate rows)
      const int64_t per_batch = static_cast<int64_t>(p.num_m_tiles) * p.num_n_tiles;
      const int64_t w = (blockIdx.x >> 1) + static_cast<int64_t>(iter) * (gridDim.x >> 1);
      if (w >= per_batch * p.batch) return false;
      const int b = static_cast<int>(w / per_batch);
      const int r = static_cast<int>(w - b * per_batch);
      const int m = r / p.num_n_tiles, n = r - m * p.num_n_tiles;
      t.a_row = m * 2 * BM + static_cast<int>(rank) * BM; t.a_batch = b;
      t.b_row = n * BN + static_cast<int>(rank) * (BN / 2); t.b_batch = b;
      t.out_row = static_cast<int64_t>(b) * p.M + t.a_row;
      t.row_end = static_cast<int64_t>(b) * p.M + p.M;
      t.n0 = n * BN;
      t.pass = 0; t.n_idx = n;
      return true;
    } else if constexpr (kSched == kSchedDense) {
      // tile counts fit 32 bits (the host checks); 64-bit divisions here would sit on every role's tile boundary
      const uint32_t per_batch = static_cast<uint32_t>(p.num_m_tiles) * p.num_n_tiles;
      const uint32_t w = blockIdx.x + static_cast<uint32_t>(iter) * gridDim.x;
      if (w >= per_batch * p.batch) return false;
      const int b = p.batch == 1 ? 0 : static_cast<int>(w / per_batch);
      const int r = static_cast<int>(w - b * per_batch);
      const int m = r / p.num_n_tiles, n = r - m * p.num_n_tiles;
      t.a_row = m * BM; t.a_batch = b;
      t.b_row = n * BN; t.b_batch = b;
      t.out_row = static_cast<int64_t>(b) * p.M + m * BM;
      t.row_end = static_cast<int64_t>(b) * p.M + p.M;
      t.n0 = n * BN;
      t.pass = 0; t.n_idx = n;
      return true;
    } else if constexpr (kSched == kSchedGroup) {
      int64_t w = blockIdx.x + static_cast<int64_t>(iter) * gridDim.x;
      int start = 0;
      for (int g = 0; g < p.groups; ++g) {
        const int end = p.offsets[g];
        const int rows = end - start;
        const int64_t tiles = static_cast<int64_t>((rows + BM - 1) / BM) * p.num_n_tiles;
        if (w < tiles) {
          const int m = static_cast<int>(w / p.num_n_tiles), n = static_cast<int>(w - static_cast<int64_t>(m) * p.num_n_tiles);
          t.a_row = start + m * BM; t.a_batch = 0;
          t.b_row = n * BN; t.b_batch = g;
          t.out_row = t.a_row;
          t.row_end = end;
          t.n0 = n * BN;
          t.pass = 0; t.n_idx = n;
          return true;
        }
        w -= tiles;
        start = end;
      }
      return false;
    } else if constexpr (kSched == kSchedConv) {
      // work item = (utterance b, block of conv_tpt output frames, column tile); `offsets` holds the
      // packed output frame offsets cu[0..groups] (cu[b+1] - cu[b] valid output frames of utterance b)
      int64_t w = blockIdx.x + static_cast<int64_t>(iter) * gridDim.x;
      const int n = static_cast<int>(w % p.num_n_tiles);
      int64_t mt = w / p.num_n_tiles;
      for (int b = 0; b < p.groups; ++b) {
        const int lo = p.offsets[b], hi = p.offsets[b + 1];
        const int frames = hi - lo;
        const int tiles = (frames + p.conv_tpt - 1) / p.conv_tpt;
        if (mt < tiles) {
          const int t0 = static_cast<int>(mt) * p.conv_tpt;
          t.a_row = t0; t.a_batch = b;
          t.b_row = n * BN; t.b_batch = 0;
          t.out_row = static_cast<int64_t>(lo + t0) * p.conv_f2;
          t.row_end = static_cast<int64_t>(lo + min(t0 + p.conv_tpt, frames)) * p.conv_f2;
          t.n0 = n * BN;
          t.pass = 0; t.n_idx = n;
          return true;
        }
        mt -= tiles;
      }
      return false;
    } else {
      const int per_row_tile = p.lsm_passes * p.num_n_tiles;
      const int64_t m = blockIdx.x + static_cast<int64_t>(iter / per_row_tile) * gridDim.x;
      if (m >= p.num_m_tiles) return false;
      const int sub = iter % per_row_tile;
      t.pass = sub / p.num_n_tiles;
      t.n_idx = sub - t.pass * p.num_n_tiles;
      t.a_row = static_cast<int>(m) * BM; t.a_batch = 0;
      t.b_row = t.n_idx * BN; t.b_batch = 0;
      t.out_row = m * BM;
      t.row_end = p.M;
      t.n0 = t.n_idx * BN;
      return true;
    }
  }
};

template <int BN, int kStages, int kCtas = 1>
struct Smem {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = (BN / kCtas) * BK * 2;  // a CTA of a pair holds half of the B tile
  static constexpr int kStageOut = kStages * (kABytes + kBBytes);  // 2 x 16 KB output staging (128 rows x 128 B)
  static constexpr int kOutBytes = BM * 128;
  static constexpr int kBarOffset = kStageOut + 2 * kOutBytes;
  static constexpr int kNumBars = 2 * kStages + 4;
  static constexpr int kTotal = kBarOffset + kNumBars * 8 + 16;
  static constexpr int kDynamic = kTotal + 1024;  // slack for manual 1024-byte alignment
};

__device__ __forceinline__ float bits_f(uint32_t u) { return __uint_as_float(u); }

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

// 8 consecutive bias values as floats (T is 16-bit; p is 16-byte aligned).
template <typename T>
__device__ __forceinline__ void load_bias8(const T* p, float (&f)[8]) {
  Pack<T> v = ld128_nc(p);
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = Elem<T>::to_f(v.v[i]);
}

// Output path: the epilogue warps write 128-byte row pieces into a swizzled staging tile and one
// thread stores the tile with TMA (clipped at the tensor edge).  Grouped problems keep per-thread
// stores because a tile may end inside the tensor (at a group boundary).
template <int kSched, int kEpi>
constexpr bool uses_tma_store() { return kSched != kSchedGroup && kSched != kSchedConv && kEpi != kEpiResid; }
// Epilogue warp groups (4 warps = all 128 TMEM lanes each).  With a single warp per scheduler the
// epilogue's load / convert / store chain is latency-bound and slower than the main loop of a
// K = 512 tile; two groups take alternate 64-column chunks of the accumulator.
template <int kSched, int kEpi>
constexpr int epi_groups() { return (uses_tma_store<kSched, kEpi>() && (kEpi == kEpiStore || kEpi == kEpiGlu)) ? 2 : 1; }
template <int kSched, int kEpi>
constexpr int threads_for() { return 64 + 32 * kEpiWarps * epi_groups<kSched, kEpi>(); }

// kCtas == 2: the kernel is launched in clusters of two CTAs that share one 256-row MMA
// (tcgen05 cta_group::2).  Each CTA loads its own 128 A rows and its own half of the B tile (no
// multicast), the leader CTA (rank 0) issues the MMAs for both, every CTA drains its own 128
// accumulator rows.  Per flop this halves the B bytes a CTA pulls from L2, which is what limits the
// single-CTA 128 x 256 tile.
// kKind: 0 = 16-bit operands of type T; 1 = fp8 e4m3 operands (kind::f8f6f4, fp32 accumulators); 2 = signed
// int8 operands (kind::i8, int32 accumulators).  For the 8-bit kinds T is the OUTPUT type, a K block is 128
// elements (the same 128 bytes per shared-memory row) and the epilogue multiplies by the row and column scales.
template <typename T, int BN, int kStages, int kSched, int kEpi, int kCtas, int kKind = 0, bool kDup = false>
__device__ __forceinline__ void gemm_body(const CUtensorMap& tmap_a, const CUtensorMap& tmap_b,
                                          const CUtensorMap& tmap_d, const Params& p) {
  using S = Smem<BN, kStages, kCtas>;
  constexpr bool kTmaStore = uses_tma_store<kSched, kEpi>();
  constexpr int kGroups = epi_groups<kSched, kEpi>();
  constexpr uint32_t kTmemCols = 2 * BN;  // 128, 256 or 512: a power of two >= 32
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
  constexpr uint32_t kIdesc = kKind == 0 ? ptx::umma_idesc_f16(kBf16, BM * kCtas, BN)
                            : kKind == 1 ? ptx::umma_idesc_8bit(1, 0, 0, BM, BN)
                                         : ptx::umma_idesc_8bit(2, 1, 1, BM, BN);
  constexpr int kBKe = kKind == 0 ? BK : 2 * BK;  // K elements per stage
  static_assert(kKind == 0 || (kCtas == 1 && kSched == kSchedDense && (kEpi == kEpiStore || kEpi == kEpiGlu)),
                "8-bit kinds: dense problems, store / GLU epilogues, single-CTA tiles");
  static_assert(kCtas == 1 || (kSched == kSchedDense && kTmaStore), "CTA pairs: dense problems with TMA stores");
  const uint32_t cta_rank = kCtas == 2 ? ptx::cluster_ctarank() : 0u;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + kStages * S::kABytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::kBarOffset);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tfull_bar = empty_bar + kStages;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      ptx::mbar_init(&full_bar[i], 1);
      ptx::mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&tfull_bar[i], 1);
      ptx::mbar_init(&tempty_bar[i], kEpiWarps * kGroups * kCtas);  // the leader waits for both CTAs' epilogues
    }
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async_smem();
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_b);
    if (kTmaStore) ptx::prefetch_tensormap(&tmap_d);
  }
  if (warp == 1) {
    if constexpr (kCtas == 2) {
      ptx::tmem_alloc_pair(tmem_slot, kTmemCols);
      ptx::tmem_relinquish_pair();
    } else {
      ptx::tmem_alloc(tmem_slot, kTmemCols);
      ptx::tmem_relinquish();
    }
  }
  ptx::tc_fence_before_sync();
  if constexpr (kCtas == 2) ptx::cluster_sync();  // the peer's barriers are initialised before anything targets them
  else __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // set-up done: let the next kernel of the stream start its own set-up, then wait for the previous kernel's
  // results (no-ops unless launched with programmatic stream serialisation)
  ptx::grid_dep_launch();
  ptx::grid_dep_wait();

  Scheduler<kSched, BN, kCtas> sched(p);
  sched.rank = cta_rank;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      Tile t;
      bool ok = true;
      for (int iter = 0; ok && sched.get(iter, t); ++iter) {
        for (int kb = 0; kb < p.num_k_blocks; ++kb) {
          if (!ptx::mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          if constexpr (kCtas == 2) {
            // both CTAs' bytes are credited to the leader's barrier; only the leader arrives on it
            const uint32_t lead_full = ptx::map_to_cta(&full_bar[stage], 0);
            if (cta_rank == 0) ptx::mbar_expect_tx(&full_bar[stage], 2 * (S::kABytes + S::kBBytes));
            ptx::tma_load_3d_pair(sA + stage * S::kABytes, &tmap_a, kb * BK, t.a_row, t.a_batch, lead_full);
            int b_row = t.b_row;
            if constexpr (kEpi == kEpiGlu) b_row = (cta_rank == 0 ? 0 : p.N) + t.n0 / 2;  // value | gate rows
            ptx::tma_load_3d_pair(sB + stage * S::kBBytes, &tmap_b, kb * BK, b_row, t.b_batch, lead_full);
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
            continue;
          }
          if constexpr (kSched == kSchedConv) {
            // K block kb = (tap, 64-channel block).  Tap (kh, kw) of output (t2, f2) reads input frame
            // 2*t2 + kh, feature 2*f2 + kw: parity plane (kh&1)*2 + (kw&1), rows (t2 + kh/2, f2 + kw/2) --
            // one dense box of conv_tpt x conv_f2 rows x 64 channels.  Rows past the box stay stale in
            // shared memory: they only feed accumulator rows that are never stored.
            const int tap = kb / p.conv_cblocks, cb = kb - tap * p.conv_cblocks;
            const int kh = tap / 3, kw = tap - 3 * kh;
            ptx::mbar_expect_tx(&full_bar[stage], static_cast<uint32_t>(p.conv_tpt * p.conv_f2 * 128) + S::kBBytes);
            ptx::tma_load_5d(sA + stage * S::kABytes, &tmap_a, cb * BK, kw >> 1, (kh & 1) * 2 + (kw & 1),
                             t.a_row + (kh >> 1), t.a_batch, &full_bar[stage]);
            ptx::tma_load_3d(sB + stage * S::kBBytes, &tmap_b, kb * BK, t.b_row, t.b_batch, &full_bar[stage]);
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
            continue;
          }
          ptx::mbar_expect_tx(&full_bar[stage], S::kABytes + S::kBBytes);
          ptx::tma_load_3d(sA + stage * S::kABytes, &tmap_a, kb * kBKe, t.a_row, t.a_batch, &full_bar[stage]);
          if constexpr (kEpi == kEpiGlu) {
            // value rows [n0/2, +BN/2) and gate rows [N + n0/2, +BN/2) of the 2N-row weight
            ptx::tma_load_3d(sB + stage * S::kBBytes, &tmap_b, kb * kBKe, t.b_row / 2, t.b_batch, &full_bar[stage]);
            ptx::tma_load_3d(sB + stage * S::kBBytes + S::kBBytes / 2, &tmap_b, kb * kBKe, p.N + t.b_row / 2,
                             t.b_batch, &full_bar[stage]);
          } else {
            ptx::tma_load_3d(sB + stage * S::kBBytes, &tmap_b, kb * kBKe, t.b_row, t.b_batch, &full_bar[stage]);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok && p.status) atomicOr(p.status, kStatusGemmProducer);
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0 && cta_rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int iter = 0; ok && sched.has(iter); ++iter) {
        const int acc = iter & 1;
        const uint32_t acc_phase = (iter >> 1) & 1u;
        if (!ptx::mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < p.num_k_blocks; ++kb) {
          if (!ptx::mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after_sync();
          const uint32_t a_addr = ptx::smem_u32(sA + stage * S::kABytes);
          const uint32_t b_addr = ptx::smem_u32(sB + stage * S::kBBytes);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t adesc = ptx::smem_desc_kmajor_sw128(a_addr + k * UMMA_K * 2);
            const uint64_t bdesc = ptx::smem_desc_kmajor_sw128(b_addr + k * UMMA_K * 2);
            if constexpr (kCtas == 2) ptx::umma_f16_pair(d_tmem, adesc, bdesc, kIdesc, (kb | k) != 0 ? 1u : 0u);
            else if constexpr (kKind == 1) ptx::umma_f8(d_tmem, adesc, bdesc, kIdesc, (kb | k) != 0 ? 1u : 0u);
            else if constexpr (kKind == 2) ptx::umma_i8(d_tmem, adesc, bdesc, kIdesc, (kb | k) != 0 ? 1u : 0u);
            else ptx::umma_f16(d_tmem, adesc, bdesc, kIdesc, (kb | k) != 0 ? 1u : 0u);
          }
          if constexpr (kCtas == 2) ptx::umma_commit_pair(&empty_bar[stage], 3);  // frees the stage in both CTAs
          else ptx::umma_commit(&empty_bar[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (ok) {
          if constexpr (kCtas == 2) ptx::umma_commit_pair(&tfull_bar[acc], 3);
          else ptx::umma_commit(&tfull_bar[acc]);
        }
      }
      if (!ok && p.status) atomicOr(p.status, kStatusGemmMma);
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    Tile t;
    bool ok = true;
    // kEpiLsm running statistics of this thread's row
    float run_max = -INFINITY, run_sum = 0.f, lse = 0.f;
    int run_arg = 0;
    // TMA-store staging: `w` is this thread's 128 bytes of row (q*32+lane) for output columns
    // starting at `col`; the 128 x 128 B tile goes out as one box at (col, row0, batch).  With two
    // warp groups each group owns one staging buffer and one named barrier; a single group
    // alternates between the two buffers.
    const int grp = (warp - 2) >> 2;
    uint8_t* stage_out = smem + S::kStageOut;
    int out_buf = 0;
    const bool issuer = ((warp - 2) & 3) == 0 && lane == 0;
    const int tile_row = q * 32 + lane;
    // Two-group form: every warp stages and stores its own 32 rows, so no barrier couples the warps and their
    // load / convert / store chains overlap.  A warp owns two 32-row x 64-byte buffers (64-byte swizzle); a unit
    // of 32 output columns goes out per store, and a buffer is rewritten only after the store before the most
    // recent one has finished reading it.
    auto stage32_and_store = [&](const uint32_t* w16, int col, const Tile& tt) {
      if (lane == 0) ptx::bulk_wait_group_read<1>();
      __syncwarp();
      uint8_t* buf = stage_out + ((warp - 2) * 2 + out_buf) * 2048;
      uint8_t* row = buf + lane * 64;
      const int swz = (lane >> 1) & 3;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        *reinterpret_cast<uint4*>(row + ((c ^ swz) << 4)) = make_uint4(w16[4 * c], w16[4 * c + 1], w16[4 * c + 2], w16[4 * c + 3]);
      }
      ptx::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0 && tt.a_row + q * 32 < p.M) {
        ptx::tma_store_3d(&tmap_d, buf, col, tt.a_row + q * 32, tt.a_batch);
        ptx::bulk_commit_group();
      }
      out_buf ^= 1;
    };
    auto stage_and_store = [&](const uint32_t (&w)[32], int col, const Tile& tt) {
      if (issuer) ptx::bulk_wait_group_read<1>();  // the store that last used this buffer has finished reading it
      ptx::named_barrier_sync(1 + grp, kEpiWarps * 32);
      uint8_t* row = stage_out + out_buf * S::kOutBytes + tile_row * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        *reinterpret_cast<uint4*>(row + ((c ^ (tile_row & 7)) * 16)) = make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
      }
      ptx::fence_proxy_async_smem();
      ptx::named_barrier_sync(1 + grp, kEpiWarps * 32);
      if (issuer) {
        ptx::tma_store_3d(&tmap_d, stage_out + out_buf * S::kOutBytes, col, tt.a_row, tt.a_batch);
        ptx::bulk_commit_group();
      }
      out_buf ^= 1;
    };
    // 32 accumulator columns -> 16 packed words of `w` (kHalf = which half), bias and activation in fp32
    // accumulator word -> float (int32 accumulators of kind::i8 are converted), and this thread's row scale
    auto acc_f = [](uint32_t u) -> float {
      if constexpr (kKind == 2) return __int2float_rn(static_cast<int>(u));
      else return __uint_as_float(u);
    };
    float row_scale = 1.f;
    // act_c: 0 = none, 1 = swish, 2 = any other id (run-time switch).  Compile-time so that the instructions a
    // tile executes are contiguous: with the switch inlined per element, the never-taken activations sit between
    // the executed instructions and the loop runs at the speed of instruction fetch.
    auto finish32 = [&](const uint32_t (&r)[32], uint32_t (&w)[32], auto half_c, auto act_c, int col0, const T* bias) {
      constexpr int kHalf = decltype(half_c)::value;
      constexpr int kAct = decltype(act_c)::value;
#pragma unroll
      for (int g8 = 0; g8 < 4; ++g8) {
        const int col = col0 + g8 * 8;
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = acc_f(r[g8 * 8 + i]);
        if constexpr (kKind != 0) {
          if (col < p.N) {
            const float4 s0 = *reinterpret_cast<const float4*>(p.b_scale + col);
            const float4 s1 = *reinterpret_cast<const float4*>(p.b_scale + col + 4);
            v[0] *= row_scale * s0.x; v[1] *= row_scale * s0.y; v[2] *= row_scale * s0.z; v[3] *= row_scale * s0.w;
            v[4] *= row_scale * s1.x; v[5] *= row_scale * s1.y; v[6] *= row_scale * s1.z; v[7] *= row_scale * s1.w;
          }
        }
        if (bias && col < p.N) {
          float bb[8];
          load_bias8(bias + col, bb);
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] += bb[i];
        }
        if constexpr (kAct == 1) {
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = swish_fast(v[i]);
        } else if constexpr (kAct == 2) {
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = apply_act_fast(v[i], p.act);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) w[kHalf * 16 + g8 * 4 + i] = pack2<T>(v[2 * i], v[2 * i + 1]);
      }
    };
    for (int iter = 0; ok && sched.get(iter, t); ++iter) {
      const int acc = iter & 1;
      const uint32_t acc_phase = (iter >> 1) & 1u;
      if (!ptx::mbar_wait(&tfull_bar[acc], acc_phase, abort_flag)) { ok = false; break; }
      ptx::tc_fence_after_sync();
      const int64_t row = t.out_row + q * 32 + lane;
      const bool row_ok = row < t.row_end;
      const uint32_t t_acc = tmem_base + lane_base + acc * BN;
      if constexpr (kKind != 0) row_scale = row_ok ? p.a_scale[row] : 0.f;

      if constexpr (kEpi == kEpiStore && kTmaStore) {
        // group `grp` takes the 64-column chunks grp, grp + kGroups, ...; the TMEM load of the next 32
        // columns is always in flight while the current 32 are converted
        const T* bias = static_cast<const T*>(p.bias);
        const int nchunks = (min(BN, p.N - t.n0) + 63) / 64;
        // one 64-column TMEM load per chunk; the next chunk's load is issued as soon as this chunk has been
        // converted, under the staging and the stores
        // kDup (the fused q/q/k/v projection): the first dup_cols columns of the product are stored twice, at output
        // columns [0, dup_cols) and [dup_cols, 2*dup_cols), each copy with the bias of its OUTPUT column; the other
        // columns move right by dup_cols.  bias is indexed by output column; tiles do not straddle dup_cols.
        const int shift = (kDup && t.n0 >= p.dup_cols) ? p.dup_cols : 0;
        const bool twice = kDup && t.n0 < p.dup_cols;
        auto store_tile = [&](auto act_c) {
          uint32_t r[64], w[32];
          int ci = grp;
          if (ci < nchunks) ptx::tmem_ld_32x64(t_acc + ci * 64, r);
#pragma unroll 1
          for (; ci < nchunks; ci += kGroups) {
            const int c0 = ci * 64;
            ptx::tmem_ld_wait();
            finish32(reinterpret_cast<const uint32_t(&)[32]>(r[0]), w, std::integral_constant<int, 0>{}, act_c, t.n0 + c0, bias ? bias + shift : bias);
            finish32(reinterpret_cast<const uint32_t(&)[32]>(r[32]), w, std::integral_constant<int, 1>{}, act_c, t.n0 + c0 + 32, bias ? bias + shift : bias);
            if constexpr (kDup && kGroups == 2) {
              if (twice) {
                uint32_t w2[32];
                finish32(reinterpret_cast<const uint32_t(&)[32]>(r[0]), w2, std::integral_constant<int, 0>{}, act_c, t.n0 + c0, bias ? bias + p.dup_cols : bias);
                finish32(reinterpret_cast<const uint32_t(&)[32]>(r[32]), w2, std::integral_constant<int, 1>{}, act_c, t.n0 + c0 + 32, bias ? bias + p.dup_cols : bias);
                stage32_and_store(w2, t.n0 + c0 + p.dup_cols, t);
                if (t.n0 + c0 + 32 < p.N) stage32_and_store(w2 + 16, t.n0 + c0 + 32 + p.dup_cols, t);
              }
            }
            if (ci + kGroups < nchunks) ptx::tmem_ld_32x64(t_acc + (ci + kGroups) * 64, r);
            if constexpr (kGroups == 2) {
              stage32_and_store(w, t.n0 + c0 + shift, t);
              if (t.n0 + c0 + 32 < p.N) stage32_and_store(w + 16, t.n0 + c0 + 32 + shift, t);
            } else {
              stage_and_store(w, t.n0 + c0, t);
            }
          }
          ptx::tmem_ld_wait();
        };
        if (p.act == OASR_ACT_NONE) store_tile(std::integral_constant<int, 0>{});
        else if (p.act == OASR_ACT_SWISH) store_tile(std::integral_constant<int, 1>{});
        else store_tile(std::integral_constant<int, 2>{});
      } else if constexpr (kEpi == kEpiStore) {
        T* drow = static_cast<T*>(p.D) + row * p.N;
        const T* bias = static_cast<const T*>(p.bias);
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          if (t.n0 + c0 >= p.N) break;
          uint32_t r[32];
          ptx::tmem_ld_32x32(t_acc + c0, r);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int col = t.n0 + c0 + g * 8;
            if (col < p.N) {
              float v[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] = bits_f(r[g * 8 + i]);
              if (bias) {
                float bb[8];
                load_bias8(bias + col, bb);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] += bb[i];
              }
              if (p.act != OASR_ACT_NONE) {
      #pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = apply_act_fast(v[i], p.act);
              }
              if (row_ok) {
                uint4 o;
                o.x = pack2<T>(v[0], v[1]); o.y = pack2<T>(v[2], v[3]);
                o.z = pack2<T>(v[4], v[5]); o.w = pack2<T>(v[6], v[7]);
                *reinterpret_cast<uint4*>(drow + col) = o;
              }
            }
          }
        }
      } else if constexpr (kEpi == kEpiResid) {
        float* orow = static_cast<float*>(p.D) + row * p.N;
        const float* rrow = p.R_in ? p.R_in + row * p.N : nullptr;   // null: D = alpha * (A.B^T + bias)
        const T* bias = static_cast<const T*>(p.bias);
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          if (t.n0 + c0 >= p.N) break;
          uint32_t r[32];
          ptx::tmem_ld_32x32(t_acc + c0, r);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int col = t.n0 + c0 + g * 8;
            if (col < p.N) {
              float v[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] = bits_f(r[g * 8 + i]);
              if (bias) {
                float bb[8];
                load_bias8(bias + col, bb);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] += bb[i];
              }
              if (row_ok) {
                float4 r0 = make_float4(0.f, 0.f, 0.f, 0.f), r1 = r0;
                if (rrow) {
                  r0 = *reinterpret_cast<const float4*>(rrow + col);
                  r1 = *reinterpret_cast<const float4*>(rrow + col + 4);
                }
                float4 o0, o1;
                o0.x = fmaf(p.alpha, v[0], r0.x); o0.y = fmaf(p.alpha, v[1], r0.y);
                o0.z = fmaf(p.alpha, v[2], r0.z); o0.w = fmaf(p.alpha, v[3], r0.w);
                o1.x = fmaf(p.alpha, v[4], r1.x); o1.y = fmaf(p.alpha, v[5], r1.y);
                o1.z = fmaf(p.alpha, v[6], r1.z); o1.w = fmaf(p.alpha, v[7], r1.w);
                *reinterpret_cast<float4*>(orow + col) = o0;
                *reinterpret_cast<float4*>(orow + col + 4) = o1;
              }
            }
          }
        }
      } else if constexpr (kEpi == kEpiGlu && kTmaStore) {
        // accumulator columns [0, BN/2) hold the value half, [BN/2, BN) the gate half
        constexpr int HN = BN / 2;
        const int n0 = t.n0 / 2;
        const T* bias = static_cast<const T*>(p.bias);
#pragma unroll 1
        for (int c0 = grp * 64; c0 < HN; c0 += 64 * kGroups) {
          if (n0 + c0 >= p.N) break;
          uint32_t w[32];
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            uint32_t rv[32], rg[32];
            ptx::tmem_ld_32x32(t_acc + c0 + half * 32, rv);
            ptx::tmem_ld_32x32(t_acc + HN + c0 + half * 32, rg);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const int col = n0 + c0 + half * 32 + g * 8;
              float v[8], gt[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) { v[i] = acc_f(rv[g * 8 + i]); gt[i] = acc_f(rg[g * 8 + i]); }
              if constexpr (kKind != 0) {
                if (col < p.N) {
#pragma unroll
                  for (int i = 0; i < 8; ++i) {
                    v[i] *= row_scale * p.b_scale[col + i];
                    gt[i] *= row_scale * p.b_scale[p.N + col + i];
                  }
                }
              }
              if (bias && col < p.N) {
                float bb[8];
                load_bias8(bias + col, bb);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] += bb[i];
                load_bias8(bias + p.N + col, bb);
#pragma unroll
                for (int i = 0; i < 8; ++i) gt[i] += bb[i];
              }
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] *= sigmoid_fast(gt[i]);
#pragma unroll
              for (int i = 0; i < 4; ++i) w[half * 16 + g * 4 + i] = pack2<T>(v[2 * i], v[2 * i + 1]);
            }
            if constexpr (kGroups == 2) {
              if (n0 + c0 + half * 32 < p.N) stage32_and_store(w + half * 16, n0 + c0 + half * 32, t);
            }
          }
          if constexpr (kGroups == 1) stage_and_store(w, n0 + c0, t);
        }
      } else if constexpr (kEpi == kEpiGlu) {
        // accumulator columns [0, BN/2) hold the value half, [BN/2, BN) the gate half
        constexpr int HN = BN / 2;
        const int n0 = t.n0 / 2;
        T* drow = static_cast<T*>(p.D) + row * p.N;
        const T* bias = static_cast<const T*>(p.bias);
#pragma unroll 1
        for (int c0 = 0; c0 < HN; c0 += 32) {
          if (n0 + c0 >= p.N) break;
          uint32_t rv[32], rg[32];
          ptx::tmem_ld_32x32(t_acc + c0, rv);
          ptx::tmem_ld_32x32(t_acc + HN + c0, rg);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int col = n0 + c0 + g * 8;
            if (col < p.N) {
              float v[8], gt[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) { v[i] = bits_f(rv[g * 8 + i]); gt[i] = bits_f(rg[g * 8 + i]); }
              if (bias) {
                float bb[8];
                load_bias8(bias + col, bb);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] += bb[i];
                load_bias8(bias + p.N + col, bb);
#pragma unroll
                for (int i = 0; i < 8; ++i) gt[i] += bb[i];
              }
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] *= sigmoid_fast(gt[i]);
              if (row_ok) {
                uint4 o;
                o.x = pack2<T>(v[0], v[1]); o.y = pack2<T>(v[2], v[3]);
                o.z = pack2<T>(v[4], v[5]); o.w = pack2<T>(v[6], v[7]);
                *reinterpret_cast<uint4*>(drow + col) = o;
              }
            }
          }
        }
      } else {
        // kEpiLsm.  Pass 0: running (max, sum of exp, argmax) of the row over all
        // column tiles.  Pass 1: the same products again, written as logit - lse.
        const T* bias = static_cast<const T*>(p.bias);
        if (t.pass == 0 && t.n_idx == 0) { run_max = -INFINITY; run_sum = 0.f; run_arg = 0; }
        uint32_t wout[32];
        // 32 accumulator columns starting at tile column cc; kHalf selects the half of `wout` a
        // 16-bit output chunk fills (compile-time so that `wout` stays in registers)
        auto process32 = [&](int cc, auto half_c) {
          constexpr int kHalf = decltype(half_c)::value;
          uint32_t r[32];
          ptx::tmem_ld_32x32(t_acc + cc, r);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int col = t.n0 + cc + g * 8;
            if (col < p.N) {
              float v[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] = bits_f(r[g * 8 + i]);
              if (bias) {
                float bb[8];
                load_bias8(bias + col, bb);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] += bb[i];
              }
              if (t.pass == 0) {
                float m8 = v[0];
                int a8 = 0;
#pragma unroll
                for (int i = 1; i < 8; ++i) {
                  if (v[i] > m8) { m8 = v[i]; a8 = i; }
                }
                if (m8 > run_max) {
                  run_sum *= __expf(run_max - m8);  // exp(-inf) = 0 on the first group
                  run_max = m8;
                  run_arg = col + a8;
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) run_sum += __expf(v[i] - run_max);
              } else if constexpr (kTmaStore) {
                if (p.out_f32) {
#pragma unroll
                  for (int i = 0; i < 8; ++i) wout[g * 8 + i] = __float_as_uint(v[i] - lse);
                } else {
#pragma unroll
                  for (int i = 0; i < 4; ++i) wout[kHalf * 16 + g * 4 + i] = pack2<T>(v[2 * i] - lse, v[2 * i + 1] - lse);
                }
              } else if (row_ok) {
                if (p.out_f32) {
                  float* orow = static_cast<float*>(p.D) + row * p.N + col;
                  *reinterpret_cast<float4*>(orow) = make_float4(v[0] - lse, v[1] - lse, v[2] - lse, v[3] - lse);
                  *reinterpret_cast<float4*>(orow + 4) = make_float4(v[4] - lse, v[5] - lse, v[6] - lse, v[7] - lse);
                } else {
                  uint4 o;
                  o.x = pack2<T>(v[0] - lse, v[1] - lse); o.y = pack2<T>(v[2] - lse, v[3] - lse);
                  o.z = pack2<T>(v[4] - lse, v[5] - lse); o.w = pack2<T>(v[6] - lse, v[7] - lse);
                  *reinterpret_cast<uint4*>(static_cast<T*>(p.D) + row * p.N + col) = o;
                }
              }
            }
          }
        };
        const bool storing = kTmaStore && t.pass == 1;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 64) {
          if (t.n0 + c0 >= p.N) break;
          process32(c0, std::integral_constant<int, 0>{});
          if (storing && p.out_f32) stage_and_store(wout, t.n0 + c0, t);         // 32 fp32 columns = 128 bytes
          if (t.n0 + c0 + 32 < p.N) {
            process32(c0 + 32, std::integral_constant<int, 1>{});
            if (storing && p.out_f32) stage_and_store(wout, t.n0 + c0 + 32, t);
          }
          if (storing && !p.out_f32) stage_and_store(wout, t.n0 + c0, t);        // 64 16-bit columns = 128 bytes
        }
        if (t.pass == 0 && t.n_idx == p.num_n_tiles - 1) {
          lse = run_max + __logf(run_sum);
          if (row_ok && p.argmax) p.argmax[row] = run_arg;
        }
      }

      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if constexpr (kCtas == 2) ptx::mbar_arrive_cluster(ptx::map_to_cta(&tempty_bar[acc], 0));
        else ptx::mbar_arrive(&tempty_bar[acc]);
      }
    }
    if (kTmaStore && (kGroups == 2 ? lane == 0 : issuer)) ptx::bulk_wait_group<0>();  // all output tiles have left shared memory and landed
    if (!ok && lane == 0 && p.status) atomicOr(p.status, kStatusGemmEpilogue);
  }

  // Teardown.  After an abandoned wait, give copies that may still be in
  // flight time to land before shared memory and TMEM are released.
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if constexpr (kCtas == 2) {
    // neither CTA may leave (or release TMEM) while the leader's MMAs can still read the peer's shared
    // memory or the peer can still arrive on the leader's barriers
    ptx::tc_fence_before_sync();
    ptx::cluster_sync();
  }
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    if constexpr (kCtas == 2) ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
    else ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <typename T, int BN, int kStages, int kSched, int kEpi>
__global__ void __launch_bounds__(threads_for<kSched, kEpi>(), 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_d, const Params p) {
  gemm_body<T, BN, kStages, kSched, kEpi, 1>(tmap_a, tmap_b, tmap_d, p);
}

template <typename T>
__global__ void __launch_bounds__(threads_for<kSchedDense, kEpiStore>(), 1)
gemm_tcgen05_dup_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                        const __grid_constant__ CUtensorMap tmap_d, const Params p) {
  gemm_body<T, 256, 4, kSchedDense, kEpiStore, 1, 0, true>(tmap_a, tmap_b, tmap_d, p);
}

template <typename T, int BN, int kStages, int kEpi, int kKind>
__global__ void __launch_bounds__(threads_for<kSchedDense, kEpi>(), 1)
gemm_tcgen05_q8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                       const __grid_constant__ CUtensorMap tmap_d, const Params p) {
  gemm_body<T, BN, kStages, kSchedDense, kEpi, 1, kKind>(tmap_a, tmap_b, tmap_d, p);
}

template <typename T, int kStages, int kEpi>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(threads_for<kSchedDense, kEpi>(), 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         const __grid_constant__ CUtensorMap tmap_d, const Params p) {
  gemm_body<T, 256, kStages, kSchedDense, kEpi, 2>(tmap_a, tmap_b, tmap_d, p);
}

// ---------------------------------------------------------------------------
// Small / odd problems: plain CUDA-core kernel (one thread per output).  Keeps
// every shape the reference accepts on the GPU; not a performance path.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) gemm_simt_kernel(T* __restrict__ D, const T* __restrict__ A,
                                                        const T* __restrict__ B, const T* __restrict__ bias,
                                                        int64_t M, int N, int K, int act, int64_t strideA,
                                                        int64_t strideB, int64_t strideD) {
  const int64_t batch = blockIdx.z;
  A += batch * strideA; B += batch * strideB; D += batch * strideD;
  const int64_t total = M * N;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t m = i / N;
    const int n = static_cast<int>(i - m * N);
    const T* a = A + m * K;
    const T* b = B + static_cast<int64_t>(n) * K;
    float acc = 0.f;
    for (int k = 0; k < K; ++k) acc = fmaf(Elem<T>::to_f(a[k]), Elem<T>::to_f(b[k]), acc);
    if (bias) acc += Elem<T>::to_f(bias[n]);
    acc = apply_act_rt(acc, act);
    D[i] = Elem<T>::from_f(acc);
  }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
int g_force_bn = 0;  // 0 = heuristic; otherwise 64 / 128 / 256 (set through oasr_b200_set_tunable)
int g_lsm_path = 0;   // CTC head: 0 = by size, 1 = one fused two-sweep kernel, 2 = fp32 logits GEMM + in-place row kernel
int g_use_pairs = 0; // 1 = large dense problems run on CTA pairs (cta_group::2); 0 (default) = single-CTA tiles.
                     // Measured on B200 (M 17.5k, K 512..2048): pairs are 5-20 % slower than single-CTA tiles here.

template <typename T, int BN, int kStages, int kSched, int kEpi>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td, const Params& p, int64_t work_items,
           cudaStream_t s) {
  using S = Smem<BN, kStages>;
  auto kern = gemm_tcgen05_kernel<T, BN, kStages, kSched, kEpi>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kDynamic);
    if (e != cudaSuccess) return set_error(OASR_ERR_CUDA, "gemm: cannot reserve %d bytes of shared memory: %s",
                                           S::kDynamic, cudaGetErrorString(e));
    attr_done = true;
  }
  int64_t grid = work_items < sm_count() ? work_items : sm_count();
  if (grid < 1) grid = 1;
  launch_pdl(kern, dim3(static_cast<unsigned>(grid)), dim3(threads_for<kSched, kEpi>()), S::kDynamic, s, ta, tb, td, p);
  return check_launch("tcgen05 gemm launch");
}

template <typename T, int BN, int kStages, int kEpi, int kKind>
int launch_q8(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td, const Params& p, int64_t work_items,
              cudaStream_t s) {
  using S = Smem<BN, kStages>;
  auto kern = gemm_tcgen05_q8_kernel<T, BN, kStages, kEpi, kKind>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kDynamic);
    if (e != cudaSuccess) return set_error(OASR_ERR_CUDA, "gemm_q8: cannot reserve %d bytes of shared memory: %s",
                                           S::kDynamic, cudaGetErrorString(e));
    attr_done = true;
  }
  int64_t grid = work_items < sm_count() ? work_items : sm_count();
  if (grid < 1) grid = 1;
  launch_pdl(kern, dim3(static_cast<unsigned>(grid)), dim3(threads_for<kSchedDense, kEpi>()), S::kDynamic, s, ta, tb, td, p);
  return check_launch("tcgen05 8-bit gemm launch");
}

constexpr int kPairStages = 6;  // 32 KB per stage and CTA (+32 KB staging = 224 KB)

template <typename T, int kEpi>
int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td, const Params& p,
                int64_t work_items, cudaStream_t s) {
  using S = Smem<256, kPairStages, 2>;
  auto kern = gemm_tcgen05_pair_kernel<T, kPairStages, kEpi>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kDynamic);
    if (e != cudaSuccess) return set_error(OASR_ERR_CUDA, "gemm: cannot reserve %d bytes of shared memory: %s",
                                           S::kDynamic, cudaGetErrorString(e));
    attr_done = true;
  }
  int64_t clusters = sm_count() / 2;
  if (work_items < clusters) clusters = work_items;
  if (clusters < 1) clusters = 1;
  kern<<<static_cast<unsigned>(2 * clusters), threads_for<kSchedDense, kEpi>(), S::kDynamic, s>>>(ta, tb, td, p);
  return check_launch("tcgen05 pair gemm launch");
}

// stage counts: as deep as fits beside the barriers in ~200 KB
template <int BN> struct StagesFor;
template <> struct StagesFor<64> { static constexpr int v = 7; };   // 24 KB / stage
template <> struct StagesFor<128> { static constexpr int v = 5; };  // 32 KB / stage
template <> struct StagesFor<256> { static constexpr int v = 4; };  // 48 KB / stage (+32 KB staging = 224 KB)

int pick_bn(int64_t m_tiles_total, int64_t N, int64_t K = 512) {
  if (g_force_bn == 64 || g_force_bn == 128 || g_force_bn == 256) return g_force_bn;
  const int sms = sm_count();
  double best = 1e30;
  int best_bn = 128;
  const int cand[3] = {256, 128, 64};
  // relative cost per output column of the narrower tiles: small at K = 512, where a tile is bound by its epilogue,
  // growing with K as the main loop takes over (a 128-wide tile moves 1.4x the operand bytes per flop; measured
  // 1.08 / 1.25 at K = 512, 1.45 / 2.0 at K >= 2048)
  const double kf = K <= 512 ? 0.0 : (K >= 2048 ? 1.0 : static_cast<double>(K - 512) / 1536.0);
  const double unit_cost[3] = {1.0, 1.08 + 0.37 * kf, 1.25 + 0.75 * kf};
  for (int i = 0; i < 3; ++i) {
    const int bn = cand[i];
    const int64_t tiles = m_tiles_total * ((N + bn - 1) / bn);
    const int64_t waves = (tiles + sms - 1) / sms;
    const double cost = static_cast<double>(waves) * bn * unit_cost[i];
    if (cost < best) { best = cost; best_bn = bn; }
  }
  return best_bn;
}

// In-place log-softmax (+ first-maximum index) of fp32 rows, N % 8 == 0: a block per row, the row held in registers
// (up to 8192 columns; longer rows are re-read), max and sum reduced across the block.
__global__ void __launch_bounds__(256) log_softmax_rows_f32_kernel(float* __restrict__ x, int32_t* __restrict__ argmax,
                                                                   int M, int N) {
  constexpr int kCache = 8;
  __shared__ float s_val[8];
  __shared__ int s_idx[8];
  __shared__ float s_bcast[2];
  const int n4 = N >> 2;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int row = blockIdx.x; row < M; row += gridDim.x) {
    float4* xr = reinterpret_cast<float4*>(x + static_cast<int64_t>(row) * N);
    float4 c[kCache];
    float best = -INFINITY;
    int arg = 0x7fffffff;
    auto see = [&](const float4& v, int col) {
      if (v.x > best) { best = v.x; arg = col; }
      if (v.y > best) { best = v.y; arg = col + 1; }
      if (v.z > best) { best = v.z; arg = col + 2; }
      if (v.w > best) { best = v.w; arg = col + 3; }
    };
#pragma unroll
    for (int k = 0; k < kCache; ++k) {
      const int ch = threadIdx.x + k * 256;
      if (ch < n4) { c[k] = xr[ch]; see(c[k], ch * 4); }
    }
    for (int ch = threadIdx.x + kCache * 256; ch < n4; ch += 256) see(xr[ch], ch * 4);
    // block maximum, ties to the smaller column
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ov > best || (ov == best && oi < arg)) { best = ov; arg = oi; }
    }
    if (lane == 0) { s_val[warp] = best; s_idx[warp] = arg; }
    __syncthreads();
    if (warp == 0) {
      float bv = lane < 8 ? s_val[lane] : -INFINITY;
      int bi = lane < 8 ? s_idx[lane] : 0x7fffffff;
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
      }
      if (lane == 0) {
        s_bcast[0] = bv;
        if (argmax) argmax[row] = bi;
      }
    }
    __syncthreads();
    const float mx = s_bcast[0];
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < kCache; ++k) {
      if (threadIdx.x + k * 256 < n4)
        sum += __expf(c[k].x - mx) + __expf(c[k].y - mx) + __expf(c[k].z - mx) + __expf(c[k].w - mx);
    }
    for (int ch = threadIdx.x + kCache * 256; ch < n4; ch += 256) {
      const float4 v = xr[ch];
      sum += __expf(v.x - mx) + __expf(v.y - mx) + __expf(v.z - mx) + __expf(v.w - mx);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) s_val[warp] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) t += s_val[w];
      s_bcast[1] = mx + __logf(t);
    }
    __syncthreads();
    const float lse = s_bcast[1];
#pragma unroll
    for (int k = 0; k < kCache; ++k) {
      const int ch = threadIdx.x + k * 256;
      if (ch < n4) xr[ch] = make_float4(c[k].x - lse, c[k].y - lse, c[k].z - lse, c[k].w - lse);
    }
    for (int ch = threadIdx.x + kCache * 256; ch < n4; ch += 256) {
      const float4 v = xr[ch];
      xr[ch] = make_float4(v.x - lse, v.y - lse, v.z - lse, v.w - lse);
    }
    __syncthreads();   // s_val / s_bcast are reused by the next row
  }
}

// The split CTC head wins where the fused kernel cannot fill the GPU (one CTA per 128-row tile).  Measured on B200 at
// N = 5008, K = 512: split 25 us per 1024 rows (103 us at M = 4096), fused flat at 310-320 us up to one tile per SM;
// they cross at 96 row tiles.
bool lsm_split_wins(int64_t M, int64_t N, int64_t K) {
  (void)N; (void)K;
  return (M + BM - 1) / BM <= (5 * sm_count()) / 8;
}

struct Problem {
  int sched, epi;
  int64_t M, N, K, batch, groups;
  const void *A, *B;
  Params p;
  int64_t lda = 0, a_bs = 0, ldb = 0, b_bs = 0;   // element strides of A / B rows and batches; 0 = packed
};

template <typename T>
int make_maps(const Problem& pr, int bn, int dtype, CUtensorMap* ta, CUtensorMap* tb, bool pair) {
  // A: (K, rows, batch); B: (K, rows, batch)
  const int64_t a_rows = pr.sched == kSchedGroup ? pr.M : pr.M;
  const int64_t a_batch = pr.sched == kSchedDense ? pr.batch : 1;
  const int64_t b_rows = pr.epi == kEpiGlu ? 2 * pr.N : pr.N;
  const int64_t b_batch = pr.sched == kSchedDense ? pr.batch : (pr.sched == kSchedGroup ? pr.groups : 1);
  uint64_t adims[3] = {(uint64_t)pr.K, (uint64_t)a_rows, (uint64_t)a_batch};
  uint64_t astr[3] = {0, (uint64_t)(pr.lda ? pr.lda : pr.K) * 2,
                      pr.a_bs ? (uint64_t)pr.a_bs * 2 : (uint64_t)pr.K * 2 * (uint64_t)a_rows};
  uint32_t abox[3] = {BK, BM, 1};
  if (int rc = make_tensor_map(ta, tma_dtype(dtype), 3, pr.A, adims, astr, abox)) return rc;
  uint64_t bdims[3] = {(uint64_t)pr.K, (uint64_t)b_rows, (uint64_t)b_batch};
  uint64_t bstr[3] = {0, (uint64_t)(pr.ldb ? pr.ldb : pr.K) * 2,
                      pr.b_bs ? (uint64_t)pr.b_bs * 2 : (uint64_t)pr.K * 2 * (uint64_t)b_rows};
  uint32_t bbox[3] = {BK, (uint32_t)((pr.epi == kEpiGlu || pair) ? bn / 2 : bn), 1};
  return make_tensor_map(tb, tma_dtype(dtype), 3, pr.B, bdims, bstr, bbox);
}

template <typename T, int kSched, int kEpi>
int run_typed(Problem& pr, int dtype, cudaStream_t s) {
  Params& p = pr.p;
  int64_t m_tiles_total;
  if (kSched == kSchedGroup) m_tiles_total = (pr.M + BM - 1) / BM + pr.groups;
  else m_tiles_total = ((pr.M + BM - 1) / BM) * (kSched == kSchedDense ? pr.batch : 1);
  const int64_t n_eff = kEpi == kEpiGlu ? 2 * pr.N : pr.N;  // accumulator columns
  int bn = kEpi == kEpiLsm ? (g_force_bn ? g_force_bn : 256) : pick_bn(m_tiles_total, n_eff, pr.K);
  if (kEpi == kEpiGlu && bn < 128) bn = 128;  // half tiles of >= 64 columns
  constexpr bool kPairCapable = kSched == kSchedDense && (kEpi == kEpiStore || kEpi == kEpiGlu);
  const bool pair = kPairCapable && g_use_pairs && g_force_bn == 0 && pr.M >= 1024 && n_eff >= 256 && pr.K >= 128;
  if (pair) bn = 256;
  p.num_m_tiles = static_cast<int>((pr.M + BM - 1) / BM);
  if (pair) p.num_m_tiles = static_cast<int>((pr.M + 2 * BM - 1) / (2 * BM));
  p.num_n_tiles = static_cast<int>((n_eff + bn - 1) / bn);
  p.num_k_blocks = static_cast<int>((pr.K + BK - 1) / BK);
  CUtensorMap ta, tb, td;
  if (int rc = make_maps<T>(pr, bn, dtype, &ta, &tb, pair)) return rc;
  if (uses_tma_store<kSched, kEpi>() && p.D != nullptr) {
    // output (N, M, batch): one 128-row x 128-byte box per store
    const bool f32 = kEpi == kEpiLsm && p.out_f32;
    const uint64_t es = f32 ? 4 : 2;
    uint64_t ddims[3] = {(uint64_t)pr.N, (uint64_t)pr.M, (uint64_t)(kSched == kSchedDense ? pr.batch : 1)};
    uint64_t dstr[3] = {0, (uint64_t)pr.N * es, (uint64_t)pr.N * es * (uint64_t)pr.M};
    constexpr bool kHalfUnits = epi_groups<kSched, kEpi>() == 2;   // 32-column stores from 64-byte-swizzled staging
    uint32_t dbox[3] = {(f32 || kHalfUnits) ? 32u : 64u, kHalfUnits ? 32u : (uint32_t)BM, 1};  // two-group epilogues store per warp
    if (int rc = make_tensor_map(&td, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : tma_dtype(dtype), 3, p.D, ddims, dstr, dbox,
                                 kHalfUnits ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  } else {
    td = ta;
  }
  int64_t work;
  if (kSched == kSchedSweep) work = p.num_m_tiles;
  else work = m_tiles_total * p.num_n_tiles;
  OB_REQUIRE(work < (int64_t(1) << 31), OASR_ERR_INVALID, "gemm: too many output tiles (%lld)", (long long)work);
  if constexpr (kPairCapable) {
    if (pair) return launch_pair<T, kEpi>(ta, tb, td, p, static_cast<int64_t>(p.num_m_tiles) * p.num_n_tiles * pr.batch, s);
  }
  switch (bn) {
    case 256: return launch<T, 256, StagesFor<256>::v, kSched, kEpi>(ta, tb, td, p, work, s);
    case 128: return launch<T, 128, StagesFor<128>::v, kSched, kEpi>(ta, tb, td, p, work, s);
    default: return launch<T, 64, StagesFor<64>::v, kSched, kEpi>(ta, tb, td, p, work, s);
  }
}

template <int kSched, int kEpi>
int run(Problem& pr, int dtype, cudaStream_t s) {
  pr.p.status = device_status_ptr();
  return OB_DISPATCH_HALF(dtype, T, [&]() -> int { return run_typed<T, kSched, kEpi>(pr, dtype, s); });
}

int validate_common(const char* op, const void* D, const void* A, const void* B, const void* bias, int64_t M,
                    int64_t N, int64_t K) {
  OB_REQUIRE(M == 0 || (D && A && B), OASR_ERR_INVALID, "%s: null pointer argument", op);
  OB_REQUIRE(M >= 0 && N > 0 && K > 0, OASR_ERR_INVALID, "%s: bad shape M=%lld N=%lld K=%lld", op, (long long)M,
             (long long)N, (long long)K);
  OB_REQUIRE(N % 8 == 0 && K % 8 == 0, OASR_ERR_ALIGN,
             "%s needs both free dimensions 8-aligned, got N=%lld K=%lld. Pad the projection at the model layer "
             "(align_out_features / pad_output_projection).",
             op, (long long)N, (long long)K);
  OB_REQUIRE(is_aligned(A, 16) && is_aligned(B, 16) && is_aligned(D, 16) && (!bias || is_aligned(bias, 16)),
             OASR_ERR_ALIGN, "%s: operand pointers must be 16-byte aligned", op);
  OB_REQUIRE(M < (int64_t(1) << 31) && N < (1 << 30) && K < (1 << 30), OASR_ERR_INVALID, "%s: extent too large", op);
  return OASR_OK;
}

// Shapes the tensor-core kernel does not take: fewer than 16 columns of K.
bool use_simt(int64_t M, int64_t N, int64_t K) { return K < 16 || M * N * K < 32 * 32 * 32; }

template <typename T>
int launch_simt(void* D, const void* A, const void* B, const void* bias, int64_t batch, int64_t M, int64_t N,
                int64_t K, int act, cudaStream_t s) {
  if (M == 0 || batch == 0) return OASR_OK;
  int64_t g = (M * N + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  if (g > cap) g = cap;
  dim3 grid(static_cast<unsigned>(g), 1, static_cast<unsigned>(batch));
  gemm_simt_kernel<T><<<grid, 256, 0, s>>>(static_cast<T*>(D), static_cast<const T*>(A), static_cast<const T*>(B),
                                           static_cast<const T*>(bias), M, (int)N, (int)K, act, M * K, N * K, M * N);
  return check_launch("simt gemm launch");
}

// 8-bit operand GEMM: A_q (M, K) and B_q (N or 2N, K) hold one byte per element.
template <typename T, int kEpi, int kKind>
int run_q8_typed(Params& p, const void* A, const void* B, int64_t M, int64_t N, int64_t K, int out_dtype, cudaStream_t s) {
  const int64_t n_eff = kEpi == kEpiGlu ? 2 * N : N;
  const int64_t m_tiles = (M + BM - 1) / BM;
  int bn = pick_bn(m_tiles, n_eff, K / 2);   // 8-bit operands: half the bytes per K element
  if (kEpi == kEpiGlu && bn < 128) bn = 128;
  p.num_m_tiles = static_cast<int>(m_tiles);
  p.num_n_tiles = static_cast<int>((n_eff + bn - 1) / bn);
  p.num_k_blocks = static_cast<int>((K + 2 * BK - 1) / (2 * BK));
  CUtensorMap ta, tb, td;
  uint64_t adims[3] = {(uint64_t)K, (uint64_t)M, 1};
  uint64_t astr[3] = {0, (uint64_t)K, (uint64_t)K * (uint64_t)M};
  uint32_t abox[3] = {2 * BK, BM, 1};
  if (int rc = make_tensor_map(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, A, adims, astr, abox)) return rc;
  uint64_t bdims[3] = {(uint64_t)K, (uint64_t)n_eff, 1};
  uint64_t bstr[3] = {0, (uint64_t)K, (uint64_t)K * (uint64_t)n_eff};
  uint32_t bbox[3] = {2 * BK, (uint32_t)(kEpi == kEpiGlu ? bn / 2 : bn), 1};
  if (int rc = make_tensor_map(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, B, bdims, bstr, bbox)) return rc;
  uint64_t ddims[3] = {(uint64_t)N, (uint64_t)M, 1};
  uint64_t dstr[3] = {0, (uint64_t)N * 2, (uint64_t)N * 2 * (uint64_t)M};
  uint32_t dbox[3] = {32u, 32u, 1};  // two-group epilogues store 32 x 32 pieces per warp
  if (int rc = make_tensor_map(&td, tma_dtype(out_dtype), 3, p.D, ddims, dstr, dbox, CU_TENSOR_MAP_SWIZZLE_64B)) return rc;
  const int64_t work = m_tiles * p.num_n_tiles;
  OB_REQUIRE(work < (int64_t(1) << 31), OASR_ERR_INVALID, "gemm_q8: too many output tiles");
  switch (bn) {
    case 256: return launch_q8<T, 256, StagesFor<256>::v, kEpi, kKind>(ta, tb, td, p, work, s);
    case 128: return launch_q8<T, 128, StagesFor<128>::v, kEpi, kKind>(ta, tb, td, p, work, s);
    default: return launch_q8<T, 64, StagesFor<64>::v, kEpi, kKind>(ta, tb, td, p, work, s);
  }
}

}  // namespace gemm

// The same convolution on CTA pairs over all output channels (conv2_pair.cu).
namespace conv2_pair {
bool supported(int64_t C, int64_t N);
int run(const CUtensorMap& ta, void* out, const void* w2, const void* bias, const int32_t* cu_frames, int64_t B, int64_t C,
        int64_t N, int64_t F2, int tpt, int64_t total_frames, int dtype, cudaStream_t s);
}  // namespace conv2_pair

// Internal C++ entry: reference GEMM on CUDA cores (tests compare the
// tensor-core kernel against it on the device).
int gemm_simt_reference(void* D, const void* A, const void* B, const void* bias, int64_t M, int64_t N, int64_t K,
                        int act, int dtype, cudaStream_t s) {
  return OB_DISPATCH_HALF(dtype, T, [&]() -> int {
    return gemm::launch_simt<T>(D, A, B, bias, 1, M, N, K, act, s);
  });
}

}  // namespace ob

extern "C" {

int oasr_b200_gemm(void* D, const void* A, const void* B, const void* bias, int64_t M, int64_t N, int64_t K,
                   int activation, int dtype, void* stream) {
  using namespace ob;
  using namespace ob::gemm;
  if (int rc = validate_common("gemm", D, A, B, bias, M, N, K)) return rc;
  OB_REQUIRE(act_is_known(activation), OASR_ERR_INVALID, "gemm: unknown activation id %d", activation);
  if (M == 0) return OASR_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (use_simt(M, N, K)) return gemm_simt_reference(D, A, B, bias, M, N, K, activation, dtype, s);
  Problem pr{};
  pr.sched = kSchedDense; pr.epi = kEpiStore;
  pr.M = M; pr.N = N; pr.K = K; pr.batch = 1; pr.A = A; pr.B = B;
  pr.p.M = (int)M; pr.p.N = (int)N; pr.p.K = (int)K; pr.p.batch = 1;
  pr.p.D = D; pr.p.bias = bias; pr.p.act = activation; pr.p.alpha = 1.f;
  return run<kSchedDense, kEpiStore>(pr, dtype, s);
}

int oasr_b200_gemm_dup_first_supported(int64_t N, int64_t K, int64_t dup_cols) {
  return N > 0 && K >= 16 && K % 8 == 0 && dup_cols > 0 && dup_cols <= N && N % 256 == 0 && dup_cols % 256 == 0 ? 1 : 0;
}

int oasr_b200_gemm_dup_first(void* D, const void* A, const void* B, const void* bias, int64_t M, int64_t N, int64_t K,
                             int64_t dup_cols, int dtype, void* stream) {
  using namespace ob;
  using namespace ob::gemm;
  if (int rc = validate_common("gemm_dup_first", D, A, B, bias, M, N, K)) return rc;
  OB_REQUIRE(oasr_b200_gemm_dup_first_supported(N, K, dup_cols) != 0, OASR_ERR_UNSUPPORTED,
             "gemm_dup_first: N and dup_cols must be multiples of 256 with 0 < dup_cols <= N (got N=%lld dup_cols=%lld)",
             (long long)N, (long long)dup_cols);
  if (M == 0) return OASR_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  Problem pr{};
  pr.sched = kSchedDense; pr.epi = kEpiStore;
  pr.M = M; pr.N = N; pr.K = K; pr.batch = 1; pr.A = A; pr.B = B;
  Params& p = pr.p;
  p.M = (int)M; p.N = (int)N; p.K = (int)K; p.batch = 1;
  p.D = D; p.bias = bias; p.act = OASR_ACT_NONE; p.alpha = 1.f;
  p.dup_cols = (int)dup_cols;
  p.status = device_status_ptr();
  p.num_m_tiles = static_cast<int>((M + BM - 1) / BM);
  p.num_n_tiles = static_cast<int>(N / 256);
  p.num_k_blocks = static_cast<int>((K + BK - 1) / BK);
  return OB_DISPATCH_HALF(dtype, T, [&]() -> int {
    CUtensorMap ta, tb, td;
    if (int rc = make_maps<T>(pr, 256, dtype, &ta, &tb, false)) return rc;
    const uint64_t n_out = static_cast<uint64_t>(N + dup_cols);
    uint64_t ddims[3] = {n_out, (uint64_t)M, 1};
    uint64_t dstr[3] = {0, n_out * 2, n_out * 2 * (uint64_t)M};
    uint32_t dbox[3] = {32u, 32u, 1};                       // the two-group epilogue stores 32 x 32 pieces per warp
    if (int rc = make_tensor_map(&td, tma_dtype(dtype), 3, D, ddims, dstr, dbox, CU_TENSOR_MAP_SWIZZLE_64B)) return rc;
    using S = Smem<256, 4>;
    auto kern = gemm_tcgen05_dup_kernel<T>;
    static bool attr_done = false;
    if (!attr_done) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kDynamic);
      if (e != cudaSuccess) return set_error(OASR_ERR_CUDA, "gemm_dup_first: cannot reserve %d bytes of shared memory: %s",
                                             S::kDynamic, cudaGetErrorString(e));
      attr_done = true;
    }
    const int64_t work = static_cast<int64_t>(p.num_m_tiles) * p.num_n_tiles;
    int64_t grid = work < sm_count() ? work : sm_count();
    if (grid < 1) grid = 1;
    launch_pdl(kern, dim3(static_cast<unsigned>(grid)), dim3(threads_for<kSchedDense, kEpiStore>()), S::kDynamic, s, ta, tb, td, p);
    return check_launch("tcgen05 gemm (duplicated first block) launch");
  });
}

int oasr_b200_gemm_q8(void* D, const void* A_q, const float* a_scale, const void* B_q, const float* b_scale,
                      const void* bias, int64_t M, int64_t N, int64_t K, int activation, int glu, int kind,
                      int out_dtype, void* stream) {
  using namespace ob;
  using namespace ob::gemm;
  OB_REQUIRE(M == 0 || (D && A_q && B_q && a_scale && b_scale), OASR_ERR_INVALID, "gemm_q8: null pointer argument");
  OB_REQUIRE(M >= 0 && N > 0 && K > 0, OASR_ERR_INVALID, "gemm_q8: bad shape M=%lld N=%lld K=%lld", (long long)M,
             (long long)N, (long long)K);
  OB_REQUIRE(kind == OASR_Q8_FP8_E4M3 || kind == OASR_Q8_INT8, OASR_ERR_INVALID, "gemm_q8: kind must be 1 (fp8 e4m3) or 2 (int8)");
  OB_REQUIRE(N % 8 == 0 && K % 16 == 0, OASR_ERR_ALIGN, "gemm_q8 needs N a multiple of 8 and K a multiple of 16 (got N=%lld K=%lld)",
             (long long)N, (long long)K);
  OB_REQUIRE(is_aligned(A_q, 16) && is_aligned(B_q, 16) && is_aligned(D, 16) && is_aligned(b_scale, 16) &&
                 (!bias || is_aligned(bias, 16)),
             OASR_ERR_ALIGN, "gemm_q8: operand pointers must be 16-byte aligned");
  OB_REQUIRE(act_is_known(activation) && (!glu || activation == OASR_ACT_NONE), OASR_ERR_INVALID,
             "gemm_q8: unknown activation id %d (none with glu)", activation);
  OB_REQUIRE(M < (int64_t(1) << 31) && N < (1 << 30) && K < (1 << 30), OASR_ERR_INVALID, "gemm_q8: extent too large");
  if (M == 0) return OASR_OK;
  Params p{};
  p.M = (int)M; p.N = (int)N; p.K = (int)K; p.batch = 1;
  p.D = D; p.bias = bias; p.act = activation; p.alpha = 1.f;
  p.a_scale = a_scale; p.b_scale = b_scale; p.status = device_status_ptr();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return OB_DISPATCH_HALF(out_dtype, T, [&]() -> int {
    if (kind == OASR_Q8_FP8_E4M3)
      return glu ? run_q8_typed<T, kEpiGlu, 1>(p, A_q, B_q, M, N, K, out_dtype, s)
                 : run_q8_typed<T, kEpiStore, 1>(p, A_q, B_q, M, N, K, out_dtype, s);
    return glu ? run_q8_typed<T, kEpiGlu, 2>(p, A_q, B_q, M, N, K, out_dtype, s)
               : run_q8_typed<T, kEpiStore, 2>(p, A_q, B_q, M, N, K, out_dtype, s);
  });
}

int oasr_b200_gemm_residual_f32(float* R_out, const float* R_in, const void* A, const void* B, const void* bias,
                                int64_t M, int64_t N, int64_t K, double alpha, int dtype, void* stream) {
  using namespace ob;
  using namespace ob::gemm;
  if (int rc = validate_common("gemm_residual_f32", R_out, A, B, bias, M, N, K)) return rc;
  OB_REQUIRE(M == 0 || !R_in || is_aligned(R_in, 16), OASR_ERR_ALIGN, "gemm_residual_f32: residual pointer unaligned");
  if (M == 0) return OASR_OK;
  Problem pr{};
  pr.sched = kSchedDense; pr.epi = kEpiResid;
  pr.M = M; pr.N = N; pr.K = K; pr.batch = 1; pr.A = A; pr.B = B;
  pr.p.M = (int)M; pr.p.N = (int)N; pr.p.K = (int)K; pr.p.batch = 1;
  pr.p.D = R_out; pr.p.R_in = R_in; pr.p.bias = bias; pr.p.act = OASR_ACT_NONE; pr.p.alpha = (float)alpha;
  return run<kSchedDense, kEpiResid>(pr, dtype, static_cast<cudaStream_t>(stream));
}

int oasr_b200_gemm_glu(void* D, const void* A, const void* B, const void* bias, int64_t M, int64_t N, int64_t K,
                       int dtype, void* stream) {
  using namespace ob;
  using namespace ob::gemm;
  if (int rc = validate_common("gemm_glu", D, A, B, bias, M, N, K)) return rc;
  if (M == 0) return OASR_OK;
  Problem pr{};
  pr.sched = kSchedDense; pr.epi = kEpiGlu;
  pr.M = M; pr.N = N; pr.K = K; pr.batch = 1; pr.A = A; pr.B = B;
  pr.p.M = (int)M; pr.p.N = (int)N; pr.p.K = (int)K; pr.p.batch = 1;
  pr.p.D = D; pr.p.bias = bias; pr.p.act = OASR_ACT_NONE; pr.p.alpha = 1.f;
  return run<kSchedDense, kEpiGlu>(pr, dtype, static_cast<cudaStream_t>(stream));
}

int oasr_b200_bmm(void* D, const void* A, const void* B, int64_t batch, int64_t M, int64_t N, int64_t K, int dtype,
                  void* stream) {
  using namespace ob;
  using namespace ob::gemm;
  if (int rc = validate_common("bmm", D, A, B, nullptr, M, N, K)) return rc;
  OB_REQUIRE(batch >= 0 && batch < 65536, OASR_ERR_INVALID, "bmm: bad batch %lld", (long long)batch);
  if (M == 0 || batch == 0) return OASR_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (use_simt(M, N, K)) {
    return OB_DISPATCH_HALF(dtype, T, [&]() -> int {
      return launch_simt<T>(D, A, B, nullptr, batch, M, N, K, OASR_ACT_NONE, s);
    });
  }
  Problem pr{};
  pr.sched = kSchedDense; pr.epi = kEpiStore;
  pr.M = M; pr.N = N; pr.K = K; pr.batch = batch; pr.A = A; pr.B = B;
  pr.p.M = (int)M; pr.p.N = (int)N; pr.p.K = (int)K; pr.p.batch = (int)batch;
  pr.p.D = D; pr.p.act = OASR_ACT_NONE; pr.p.alpha = 1.f;
  return run<kSchedDense, kEpiStore>(pr, dtype, s);
}

int oasr_b200_bmm_strided(void* D, const void* A, const void* B, int64_t batch, int64_t M, int64_t N, int64_t K,
                          int64_t lda, int64_t stride_a, int64_t ldb, int64_t stride_b, int dtype, void* stream) {
  using namespace ob;
  using namespace ob::gemm;
  if (int rc = validate_common("bmm_strided", D, A, B, nullptr, M, N, K)) return rc;
  OB_REQUIRE(batch >= 0 && batch < 65536, OASR_ERR_INVALID, "bmm_strided: bad batch %lld", (long long)batch);
  OB_REQUIRE(lda >= K && ldb >= K && stride_a > 0 && stride_b > 0 && lda % 8 == 0 && ldb % 8 == 0 && stride_a % 8 == 0 &&
                 stride_b % 8 == 0,
             OASR_ERR_ALIGN, "bmm_strided: row and batch strides must be positive multiples of 8 elements, rows >= K");
  if (M == 0 || batch == 0) return OASR_OK;
  OB_REQUIRE(!use_simt(M, N, K), OASR_ERR_UNSUPPORTED,
             "bmm_strided: shape (%lld, %lld, %lld) is below the tensor-core kernel's range; use bmm on packed operands",
             (long long)M, (long long)N, (long long)K);
  Problem pr{};
  pr.sched = kSchedDense; pr.epi = kEpiStore;
  pr.M = M; pr.N = N; pr.K = K; pr.batch = batch; pr.A = A; pr.B = B;
  pr.lda = lda; pr.a_bs = stride_a; pr.ldb = ldb; pr.b_bs = stride_b;
  pr.p.M = (int)M; pr.p.N = (int)N; pr.p.K = (int)K; pr.p.batch = (int)batch;
  pr.p.D = D; pr.p.act = OASR_ACT_NONE; pr.p.alpha = 1.f;
  return run<kSchedDense, kEpiStore>(pr, dtype, static_cast<cudaStream_t>(stream));
}

int oasr_b200_group_gemm(void* D, const void* A, const void* B, const int32_t* offsets, int64_t L, int64_t groups,
                         int64_t N, int64_t K, int dtype, void* stream) {
  using namespace ob;
  using namespace ob::gemm;
  if (int rc = validate_common("group_gemm", D, A, B, nullptr, L, N, K)) return rc;
  OB_REQUIRE(offsets != nullptr && groups > 0 && groups < 65536, OASR_ERR_INVALID, "group_gemm: bad offsets/groups");
  if (L == 0) return OASR_OK;
  Problem pr{};
  pr.sched = kSchedGroup; pr.epi = kEpiStore;
  pr.M = L; pr.N = N; pr.K = K; pr.batch = 1; pr.groups = groups; pr.A = A; pr.B = B;
  pr.p.M = (int)L; pr.p.N = (int)N; pr.p.K = (int)K; pr.p.batch = 1; pr.p.groups = (int)groups;
  pr.p.offsets = offsets;
  pr.p.D = D; pr.p.act = OASR_ACT_NONE; pr.p.alpha = 1.f;
  return run<kSchedGroup, kEpiStore>(pr, dtype, static_cast<cudaStream_t>(stream));
}

int oasr_b200_subsample_conv2(void* out, const void* x1, const void* w2, const void* bias, const int32_t* cu_frames,
                              int64_t B, int64_t T1, int64_t F1, int64_t C, int64_t N, int64_t total_frames, int dtype,
                              void* stream) {
  using namespace ob;
  using namespace ob::gemm;
  OB_REQUIRE(B >= 0 && T1 >= 3 && F1 >= 3 && C > 0 && N > 0 && total_frames >= 0, OASR_ERR_INVALID,
             "subsample_conv2: bad shape");
  if (B == 0 || total_frames == 0) return OASR_OK;
  OB_REQUIRE(out && x1 && w2 && cu_frames, OASR_ERR_INVALID, "subsample_conv2: null pointer argument");
  OB_REQUIRE(C % 64 == 0 && N % 8 == 0, OASR_ERR_ALIGN,
             "subsample_conv2: input channels must be a multiple of 64 and output channels of 8 (got %lld, %lld)",
             (long long)C, (long long)N);
  OB_REQUIRE(is_aligned(out, 16) && is_aligned(x1, 16) && is_aligned(w2, 16) && (!bias || is_aligned(bias, 16)),
             OASR_ERR_ALIGN, "subsample_conv2: operand pointers must be 16-byte aligned");
  const int64_t F2 = (F1 - 3) / 2 + 1, TH = (T1 + 1) / 2, FH = (F1 + 1) / 2;
  OB_REQUIRE(F2 >= 1 && F2 <= BM, OASR_ERR_UNSUPPORTED, "subsample_conv2: at most %d output positions per frame", BM);
  OB_REQUIRE(B < 65536 && total_frames * F2 < (int64_t(1) << 31), OASR_ERR_INVALID, "subsample_conv2: extent too large");
  const int tpt = static_cast<int>(BM / F2);
  const int64_t K = 9 * C;
  Params p{};
  p.M = static_cast<int>(total_frames * F2); p.N = static_cast<int>(N); p.K = static_cast<int>(K); p.batch = 1;
  p.groups = static_cast<int>(B); p.offsets = cu_frames;
  p.D = out; p.bias = bias; p.act = OASR_ACT_RELU; p.alpha = 1.f;
  p.conv_f2 = static_cast<int>(F2); p.conv_tpt = tpt; p.conv_cblocks = static_cast<int>(C / 64);
  p.status = device_status_ptr();
  int bn = N >= 256 ? 256 : (N >= 128 ? 128 : 64);
  if (g_force_bn == 64 || g_force_bn == 128 || g_force_bn == 256) bn = g_force_bn;
  p.num_m_tiles = 0;
  p.num_n_tiles = static_cast<int>((N + bn - 1) / bn);
  p.num_k_blocks = static_cast<int>(K / BK);
  CUtensorMap ta, tb;
  {
    uint64_t dims[5] = {(uint64_t)C, (uint64_t)FH, 4, (uint64_t)TH, (uint64_t)B};
    uint64_t str[5] = {0, (uint64_t)C * 2, (uint64_t)FH * C * 2, (uint64_t)4 * FH * C * 2, (uint64_t)TH * 4 * FH * C * 2};
    uint32_t box[5] = {BK, (uint32_t)F2, 1, (uint32_t)tpt, 1};
    if (int rc = make_tensor_map(&ta, tma_dtype(dtype), 5, x1, dims, str, box)) return rc;
    if (g_force_bn == 0 && conv2_pair::supported(C, N))
      return conv2_pair::run(ta, out, w2, bias, cu_frames, B, C, N, F2, tpt, total_frames, dtype, static_cast<cudaStream_t>(stream));
    uint64_t bdims[3] = {(uint64_t)K, (uint64_t)N, 1};
    uint64_t bstr[3] = {0, (uint64_t)K * 2, (uint64_t)K * 2 * (uint64_t)N};
    uint32_t bbox[3] = {BK, (uint32_t)bn, 1};
    if (int rc = make_tensor_map(&tb, tma_dtype(dtype), 3, w2, bdims, bstr, bbox)) return rc;
  }
  const int64_t work = (total_frames / tpt + B) * p.num_n_tiles;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return OB_DISPATCH_HALF(dtype, T, [&]() -> int {
    switch (bn) {
      case 256: return launch<T, 256, StagesFor<256>::v, kSchedConv, kEpiStore>(ta, tb, ta, p, work, s);
      case 128: return launch<T, 128, StagesFor<128>::v, kSchedConv, kEpiStore>(ta, tb, ta, p, work, s);
      default: return launch<T, 64, StagesFor<64>::v, kSchedConv, kEpiStore>(ta, tb, ta, p, work, s);
    }
  });
}

int oasr_b200_gemm_log_softmax(void* out, const void* A, const void* B, const void* bias, int64_t M, int64_t N,
                               int64_t K, int dtype, int out_dtype, int32_t* argmax, void* stream) {
  using namespace ob;
  using namespace ob::gemm;
  // out == NULL with argmax != NULL: only the per-row index of the first maximum is wanted (greedy CTC search);
  // one sweep over the vocabulary, nothing but 4 bytes per row is written
  const bool tokens_only = out == nullptr && argmax != nullptr;
  if (int rc = validate_common("gemm_log_softmax", tokens_only ? static_cast<const void*>(A) : out, A, B, bias, M, N, K)) return rc;
  OB_REQUIRE(out_dtype == OASR_DT_F32 || out_dtype == dtype, OASR_ERR_DTYPE,
             "gemm_log_softmax: out dtype must be fp32 or the activation dtype");
  if (M == 0) return OASR_OK;
  // Two forms.  The fused kernel sweeps the vocabulary twice per 128-row tile (statistics, then the same products
  // written normalised) and never writes logits; it keeps one CTA per row tile, so it needs about as many row tiles
  // as SMs.  The split form writes fp32 logits into `out` with the dense scheduler (every SM busy at any M) and
  // normalises the rows in place: one GEMM instead of two for a second pass over the output.
  const bool split_ok = out_dtype == OASR_DT_F32 && !use_simt(M, N, K) && !tokens_only;
  const bool split = split_ok && (g_lsm_path == 2 || (g_lsm_path == 0 && lsm_split_wins(M, N, K)));
  if (split) {
    Problem pg{};
    pg.sched = kSchedDense; pg.epi = kEpiResid;
    pg.M = M; pg.N = N; pg.K = K; pg.batch = 1; pg.A = A; pg.B = B;
    pg.p.M = (int)M; pg.p.N = (int)N; pg.p.K = (int)K; pg.p.batch = 1;
    pg.p.D = out; pg.p.R_in = nullptr; pg.p.bias = bias; pg.p.act = OASR_ACT_NONE; pg.p.alpha = 1.f;
    if (int rc = run<kSchedDense, kEpiResid>(pg, dtype, static_cast<cudaStream_t>(stream))) return rc;
    int64_t g = M < static_cast<int64_t>(sm_count()) * 8 ? M : static_cast<int64_t>(sm_count()) * 8;
    log_softmax_rows_f32_kernel<<<static_cast<unsigned>(g), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<float*>(out), argmax, (int)M, (int)N);
    return check_launch("log_softmax_rows launch");
  }
  Problem pr{};
  pr.sched = kSchedSweep; pr.epi = kEpiLsm;
  pr.M = M; pr.N = N; pr.K = K; pr.batch = 1; pr.A = A; pr.B = B;
  pr.p.M = (int)M; pr.p.N = (int)N; pr.p.K = (int)K; pr.p.batch = 1;
  pr.p.D = out; pr.p.bias = bias; pr.p.act = OASR_ACT_NONE; pr.p.alpha = 1.f;
  pr.p.out_f32 = out_dtype == OASR_DT_F32 ? 1 : 0;
  pr.p.lsm_passes = tokens_only ? 1 : 2;
  pr.p.argmax = argmax;
  return run<kSchedSweep, kEpiLsm>(pr, dtype, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
