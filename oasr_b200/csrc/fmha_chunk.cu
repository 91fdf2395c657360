// Streaming-chunk attention: a handful of new query frames (<= 16) of every stream against that
// stream's paged K/V history, with the Conformer relative-position term.
//
//   out[b, i, h, :] = softmax_j( ((q_i+u).k_j + (q_i+v).p_{pos_start[b]+j}) * scale ) . v_j ,  j < seqlens[b]
//
// With 16 query rows the contraction is tiny (about 24 flop per byte of K/V/P read) and the
// kernel is bound by how fast pages stream out of HBM, so the layout is chosen for memory-level
// parallelism, not for the tensor pipe: one WARP owns one (stream, head) and runs its own
// two-stage TMA ring of 32-key slices (K page rows, the matching rows of the projected position
// table, V page rows; 128-byte swizzle) behind per-warp mbarriers -- no block-wide barrier after
// set-up, eight independent pipelines per CTA, ~100 KB of loads in flight per SM.  The 16-row
// products run on warp-level m16n8k16 MMAs fed by ldmatrix (a 128-row tcgen05 tile would waste 7/8
// of its rows here); the softmax is the usual online form in the log2 domain with fp32 state.
//
// Reference semantics: RelPositionMultiHeadedAttention.forward_paged
// (oasr/layers/attention/attention.py:388-470) + paged fmha (oasr/functionals/attention.py:369-551):
// every new frame sees the whole cached window and the whole chunk; keys >= seqlens[b] are masked.
#include <cuda.h>
#include <cuda_fp8.h>

#include <type_traits>

#include "common.cuh"
#include "device_status.cuh"
#include "sm100_ptx.cuh"
#include "tma_host.cuh"

namespace ob {
int g_fmha_chunk_path = 1;  // 1 = this kernel where it applies; 0 = always the 128-row tcgen05 kernel ("fmha_chunk_path")

namespace fmha_chunk {

constexpr int kWarps = 8;
constexpr int kKeys = 32;                   // keys per pipeline stage
constexpr int kStages = 2;
constexpr int kTileBytes = kKeys * 128;     // 32 rows x 64 x 2 B
constexpr int kStageBytes = 3 * kTileBytes; // K | pos | V
constexpr int kSmemBars = kWarps * kStages * kStageBytes;
constexpr int kSmemTotal = kSmemBars + kWarps * kStages * 8 + 16;
constexpr int kSmemDynamic = kSmemTotal + 1024;
constexpr int D = 64;

struct Params {
  const uint8_t* qkv4;   // rows (b*Tq + i), 4*d wide: [q+u | q+v | k | v]
  int64_t ld;            // elements per qkv4 row
  int B, H, Tq;
  float scale_log2;
  const int32_t* seqlens;
  const int32_t* pos_start;
  const int32_t* block_table;
  int blocks_per_seq, block_size, num_blocks;
  void* out;             // (B*Tq, H*D)
  uint32_t* status;
  const float* k_scale;  // fp8 pages: [H] per-head scales of the K / V codes (x ~ code * scale)
  const float* v_scale;
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}
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

// fp8 pages (kFp8): K and V arrive as e4m3 codes (64 bytes per key, plain layout) in the first 4 KB of a stage, the
// position rows behind them; the warp converts the codes to fp16 into two working tiles in the swizzled layout the
// ldmatrix path reads ("shared-memory-staged" dequantisation: one cvt per value pair, exact), multiplies q+u by the
// K scale once when it loads it (as fp16) and the output by the V scale once at the end.  The content product and
// P.V then run as fp16 MMAs, the position product stays in T; all accumulate in the same fp32 registers.
// Per warp: 2 stages x 8 KB + 2 x 4 KB working tiles = the same 24 KB as the 16-bit ring.
template <typename T, bool kFp8>
__global__ void __launch_bounds__(kWarps * 32, 1)
fmha_chunk_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                  const __grid_constant__ CUtensorMap map_pos, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kStageB = kFp8 ? 2 * (kTileBytes / 2) + kTileBytes : kStageBytes;   // fp8: K8 2 KB | V8 2 KB | pos 4 KB
  constexpr int kPosOff = kFp8 ? kTileBytes : kTileBytes;                           // position rows sit 4 KB into a stage either way
  using TC = typename std::conditional<kFp8, __half, T>::type;                      // operand type of the content / P.V MMAs
  uint8_t* ring = smem + warp * kStages * kStageBytes;
  uint8_t* work = ring + kStages * kStageB;                                         // fp8 only: K and V working tiles (fp16)
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kSmemBars) + warp * kStages;
  volatile uint32_t* abort_flag = reinterpret_cast<uint32_t*>(smem + kSmemBars + kWarps * kStages * 8);
  if (threadIdx.x == 0) *abort_flag = 0;
  if (lane == 0) {
    for (int s = 0; s < kStages; ++s) ptx::mbar_init(&bars[s], 1);
    ptx::fence_barrier_init();
    ptx::fence_proxy_async_smem();
  }
  __syncthreads();
  ptx::grid_dep_launch();   // no-ops unless launched with programmatic stream serialisation
  ptx::grid_dep_wait();
  bool ok = true;
  const int item = blockIdx.x * kWarps + warp;
  const bool live = item < p.B * p.H;   // warp-uniform; dead warps skip to the common exit
  if (live) {
    const int b = item / p.H, h = item - b * p.H;
    const int kv_len = min(max(p.seqlens[b], 0), p.blocks_per_seq * p.block_size);
    const int n_it = (kv_len + kKeys - 1) / kKeys;
    const int pos0 = p.pos_start[b];
    const int g = lane >> 2, t = lane & 3;
    T* out = static_cast<T*>(p.out) + (static_cast<int64_t>(b) * p.Tq * p.H + h) * D;
    const int64_t out_ld = static_cast<int64_t>(p.H) * D;
    if (n_it == 0) {   // no visible key: zero rows
      for (int i = lane; i < p.Tq * (D / 8); i += 32)
        *reinterpret_cast<uint4*>(out + (i / (D / 8)) * out_ld + (i % (D / 8)) * 8) = make_uint4(0, 0, 0, 0);
    } else {
      // this stream's page ids, two per lane (the host guarantees blocks_per_seq <= 64)
      const int32_t* row = p.block_table + static_cast<int64_t>(b) * p.blocks_per_seq;
      int pg_lo = lane < p.blocks_per_seq ? row[lane] : 0;
      int pg_hi = lane + 32 < p.blocks_per_seq ? row[lane + 32] : 0;
      pg_lo = min(max(pg_lo, 0), p.num_blocks - 1);
      pg_hi = min(max(pg_hi, 0), p.num_blocks - 1);
      const bool small_pages = p.block_size == 16;   // else block_size is a multiple of 32
      auto issue = [&](int it, int s) {   // warp-collective: shuffles by all lanes, TMA by lane 0
        const int key0 = it * kKeys;
        int col0 = min(key0 / p.block_size, p.blocks_per_seq - 1);
        int col1 = min(col0 + 1, p.blocks_per_seq - 1);
        const int a0 = __shfl_sync(0xffffffffu, pg_lo, col0 & 31), a1 = __shfl_sync(0xffffffffu, pg_hi, col0 & 31);
        const int c0 = __shfl_sync(0xffffffffu, pg_lo, col1 & 31), c1 = __shfl_sync(0xffffffffu, pg_hi, col1 & 31);
        const int page0 = col0 < 32 ? a0 : a1, page1 = col1 < 32 ? c0 : c1;
        if (lane == 0) {
          uint8_t* dst = ring + s * kStageB;
          ptx::fence_proxy_async_smem();
          ptx::mbar_expect_tx(&bars[s], kStageB);
          if constexpr (kFp8) {
            if (small_pages) {
              ptx::tma_load_4d(dst, &map_k, 0, 0, h, page0, &bars[s]);
              ptx::tma_load_4d(dst + 16 * 64, &map_k, 0, 0, h, page1, &bars[s]);
              ptx::tma_load_4d(dst + kTileBytes / 2, &map_v, 0, 0, h, page0, &bars[s]);
              ptx::tma_load_4d(dst + kTileBytes / 2 + 16 * 64, &map_v, 0, 0, h, page1, &bars[s]);
            } else {
              const int r0 = key0 % p.block_size;
              ptx::tma_load_4d(dst, &map_k, 0, r0, h, page0, &bars[s]);
              ptx::tma_load_4d(dst + kTileBytes / 2, &map_v, 0, r0, h, page0, &bars[s]);
            }
          } else if (small_pages) {
            ptx::tma_load_4d(dst, &map_k, 0, 0, h, page0, &bars[s]);
            ptx::tma_load_4d(dst + 16 * 128, &map_k, 0, 0, h, page1, &bars[s]);
            ptx::tma_load_4d(dst + 2 * kTileBytes, &map_v, 0, 0, h, page0, &bars[s]);
            ptx::tma_load_4d(dst + 2 * kTileBytes + 16 * 128, &map_v, 0, 0, h, page1, &bars[s]);
          } else {
            const int r0 = key0 % p.block_size;
            ptx::tma_load_4d(dst, &map_k, 0, r0, h, page0, &bars[s]);
            ptx::tma_load_4d(dst + 2 * kTileBytes, &map_v, 0, r0, h, page0, &bars[s]);
          }
          ptx::tma_load_4d(dst + kPosOff, &map_pos, 0, pos0 + key0, h, 0, &bars[s]);
        }
      };
      issue(0, 0);
      if (n_it > 1) issue(1, 1);

      // Q fragments (A operand, 16 x 64 each) straight from global memory; rows >= Tq are zero
      uint32_t qu[4][4], qv[4][4];
      {
        const int64_t d = static_cast<int64_t>(p.H) * D;
        const T* q = reinterpret_cast<const T*>(p.qkv4) + static_cast<int64_t>(b) * p.Tq * p.ld + h * D;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int r = g + (e & 1) * 8, c = kk * 16 + 2 * t + (e >> 1) * 8;
            uint32_t a = 0, bb = 0;
            if (r < p.Tq) {
              a = __ldg(reinterpret_cast<const uint32_t*>(q + r * p.ld + c));
              bb = __ldg(reinterpret_cast<const uint32_t*>(q + r * p.ld + d + c));
            }
            if constexpr (kFp8) {   // q+u as fp16, times the K scale of this head
              const float ks = p.k_scale[h];
              float2 f;
              if constexpr (std::is_same<T, __nv_bfloat16>::value) f = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&a));
              else f = __half22float2(*reinterpret_cast<__half2*>(&a));
              const __half2 hq = __floats2half2_rn(f.x * ks, f.y * ks);
              a = *reinterpret_cast<const uint32_t*>(&hq);
            }
            qu[kk][e] = a;
            qv[kk][e] = bb;
          }
        }
      }
      float o[8][4];
#pragma unroll
      for (int n = 0; n < 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
      float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

      for (int it = 0; it < n_it; ++it) {
        const int s = it % kStages;
        const bool arrived = ptx::mbar_wait(&bars[s], (it / kStages) & 1u, abort_flag);
        if (!__all_sync(0xffffffffu, arrived)) { ok = false; break; }
        const uint32_t stage = ptx::smem_u32(ring + s * kStageB);
        if constexpr (kFp8) {
          // 2 x 2 KB of codes -> 2 x 4 KB of fp16 in the swizzled 128-byte-row layout; lane handles 16-byte pieces
#pragma unroll
          for (int which = 0; which < 2; ++which) {
            const uint8_t* src = ring + s * kStageB + which * (kTileBytes / 2);
            uint8_t* dstw = work + which * kTileBytes;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int piece = lane + 32 * u, key = piece >> 2, part = piece & 3;   // 16 codes = d 16*part .. +15 of one key
              const uint4 c = *reinterpret_cast<const uint4*>(src + piece * 16);
              const uint32_t cw[4] = {c.x, c.y, c.z, c.w};
              uint32_t hw[8];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(cw[i] & 0xffffu), __NV_E4M3);
                const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(cw[i] >> 16), __NV_E4M3);
                hw[2 * i] = static_cast<uint32_t>(lo.x) | (static_cast<uint32_t>(lo.y) << 16);
                hw[2 * i + 1] = static_cast<uint32_t>(hi.x) | (static_cast<uint32_t>(hi.y) << 16);
              }
              uint8_t* rowp = dstw + key * 128;
              *reinterpret_cast<uint4*>(rowp + (((2 * part) ^ (key & 7)) << 4)) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
              *reinterpret_cast<uint4*>(rowp + (((2 * part + 1) ^ (key & 7)) << 4)) = make_uint4(hw[4], hw[5], hw[6], hw[7]);
            }
          }
          __syncwarp();
        }
        const uint32_t k_tile = kFp8 ? ptx::smem_u32(work) : stage;
        const uint32_t v_tile = kFp8 ? ptx::smem_u32(work + kTileBytes) : stage + 2 * kTileBytes;
        const uint32_t p_tile = stage + kPosOff;
        // ---- S = (q+u).K^T + (q+v).P^T : 16 x 32 in four 8-key accumulators ----
        float sc[4][4];
#pragma unroll
        for (int n = 0; n < 4; ++n) {
          sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
          const int r = n * 8 + (lane & 7);
#pragma unroll
          for (int kp = 0; kp < 2; ++kp) {
            const uint32_t off = r * 128 + (((kp * 4 + (lane >> 3)) ^ (r & 7)) << 4);
            uint32_t kb[4], pb[4];
            ldmatrix_x4(kb, k_tile + off);
            ldmatrix_x4(pb, p_tile + off);
            mma16816<TC>(sc[n], qu[2 * kp], kb[0], kb[1]);
            mma16816<TC>(sc[n], qu[2 * kp + 1], kb[2], kb[3]);
            mma16816<T>(sc[n], qv[2 * kp], pb[0], pb[1]);
            mma16816<T>(sc[n], qv[2 * kp + 1], pb[2], pb[3]);
          }
        }
        // ---- online softmax (log2 domain); rows g and g+8 ----
        const int key0 = it * kKeys;
        float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < 4; ++n) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int key = key0 + n * 8 + 2 * t + (e & 1);
            const float x = key < kv_len ? sc[n][e] * p.scale_log2 : -INFINITY;
            sc[n][e] = x;
            tmax[e >> 1] = fmaxf(tmax[e >> 1], x);
          }
        }
        float alpha[2], m_use[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
          tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
          const float m_new = fmaxf(m_run[r], tmax[r]);
          m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;
          alpha[r] = (m_run[r] == -INFINITY) ? 0.f : exp2f(m_run[r] - m_use[r]);
          m_run[r] = m_new;
        }
        uint32_t pa[2][4];
        float rs[2] = {0.f, 0.f};
#pragma unroll
        for (int n = 0; n < 4; ++n) {
          const float p0 = exp2f(sc[n][0] - m_use[0]), p1 = exp2f(sc[n][1] - m_use[0]);
          const float p2 = exp2f(sc[n][2] - m_use[1]), p3 = exp2f(sc[n][3] - m_use[1]);
          rs[0] += p0 + p1;
          rs[1] += p2 + p3;
          pa[n >> 1][(n & 1) * 2] = pack2<TC>(p0, p1);
          pa[n >> 1][(n & 1) * 2 + 1] = pack2<TC>(p2, p3);
        }
        l_run[0] = l_run[0] * alpha[0] + rs[0];
        l_run[1] = l_run[1] * alpha[1] + rs[1];
#pragma unroll
        for (int n = 0; n < 8; ++n) {
          o[n][0] *= alpha[0]; o[n][1] *= alpha[0];
          o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
        }
        // ---- O += P.V : V rows are keys, so the B fragments come through a transposing ldmatrix ----
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
          const int r = kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
#pragma unroll
          for (int np = 0; np < 4; ++np) {
            const uint32_t off = r * 128 + (((2 * np + (lane >> 4)) ^ (r & 7)) << 4);
            uint32_t vb[4];
            ldmatrix_x4_trans(vb, v_tile + off);
            mma16816<TC>(o[2 * np], pa[kk], vb[0], vb[1]);
            mma16816<TC>(o[2 * np + 1], pa[kk], vb[2], vb[3]);
          }
        }
        __syncwarp();
        if (it + kStages < n_it) issue(it + kStages, s);
      }
      if (ok) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
          l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
        }
        float inv0 = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f;
        float inv1 = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
        if constexpr (kFp8) {
          inv0 *= p.v_scale[h];
          inv1 *= p.v_scale[h];
        }
#pragma unroll
        for (int n = 0; n < 8; ++n) {
          const int c = n * 8 + 2 * t;
          if (g < p.Tq) *reinterpret_cast<uint32_t*>(out + g * out_ld + c) = pack2<T>(o[n][0] * inv0, o[n][1] * inv0);
          if (g + 8 < p.Tq)
            *reinterpret_cast<uint32_t*>(out + (g + 8) * out_ld + c) = pack2<T>(o[n][2] * inv1, o[n][3] * inv1);
        }
      } else if (lane == 0 && p.status) {
        atomicOr(p.status, kStatusFmhaLoad);
      }
    }
  }
  // A warp that gave up may still have copies in flight into its ring: hold the CTA's shared
  // memory for a bounded while before returning it.
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
}

int make_map(CUtensorMap* m, int dtype, const void* base, int64_t rows, int64_t heads, int64_t batch,
             int64_t stride_row, int64_t stride_head, int64_t stride_batch, int box_rows) {
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)rows, (uint64_t)heads, (uint64_t)batch};
  uint64_t str[4] = {0, (uint64_t)stride_row * 2, (uint64_t)stride_head * 2, (uint64_t)stride_batch * 2};
  uint32_t box[4] = {64, (uint32_t)box_rows, 1, 1};
  return make_tensor_map(m, tma_dtype(dtype), 4, base, dims, str, box);
}

// fp8 pool (num_blocks, block_size, H, 64) of one-byte codes: 64-byte rows, plain (unswizzled) boxes
int make_map_u8(CUtensorMap* m, const void* base, int64_t block_size, int64_t heads, int64_t num_blocks, int box_rows) {
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)block_size, (uint64_t)heads, (uint64_t)num_blocks};
  uint64_t str[4] = {0, (uint64_t)heads * D, (uint64_t)D, (uint64_t)block_size * heads * D};
  uint32_t box[4] = {64, (uint32_t)box_rows, 1, 1};
  return make_tensor_map(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, base, dims, str, box, CU_TENSOR_MAP_SWIZZLE_NONE);
}

bool applies(int64_t Tq, int64_t block_size, int64_t blocks_per_seq) {
  return g_fmha_chunk_path && Tq <= 16 && (block_size == 16 || block_size % 32 == 0) && blocks_per_seq <= 64;
}
bool applies_fp8(int64_t Tq, int64_t block_size, int64_t blocks_per_seq) {
  return Tq <= 16 && (block_size == 16 || block_size % 32 == 0) && blocks_per_seq <= 64;
}

template <typename T, bool kFp8>
int launch(const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mp, const Params& p, unsigned grid, cudaStream_t stream) {
  auto kern = fmha_chunk_kernel<T, kFp8>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemDynamic);
    if (e != cudaSuccess)
      return set_error(OASR_ERR_CUDA, "fmha_paged_relpos: cannot reserve %d bytes of shared memory: %s", kSmemDynamic,
                       cudaGetErrorString(e));
    attr_done = true;
  }
  launch_pdl(kern, dim3(grid), dim3(kWarps * 32), kSmemDynamic, stream, mk, mv, mp, p);
  return check_launch("fmha_paged_relpos (chunk kernel) launch");
}

// k_scale / v_scale null: 16-bit pools; otherwise the pools hold fp8 e4m3 codes with per-head scales.
int run(void* out, const void* qkv4, void* k_pool, void* v_pool, const float* k_scale, const float* v_scale, const void* pos,
        int64_t pos_rows, int64_t pos_stride, const int32_t* pos_start, const int32_t* block_table, const int32_t* seqlens,
        int64_t B, int64_t Tq, int64_t H, int64_t blocks_per_seq, int64_t block_size, int64_t num_blocks, double scale,
        int dtype, cudaStream_t stream) {
  const int64_t d = H * D;
  const int box_rows = block_size == 16 ? 16 : 32;
  const bool fp8 = k_scale != nullptr;
  CUtensorMap mk, mv, mp;
  if (fp8) {
    if (int rc = make_map_u8(&mk, k_pool, block_size, H, num_blocks, box_rows)) return rc;
    if (int rc = make_map_u8(&mv, v_pool, block_size, H, num_blocks, box_rows)) return rc;
  } else {
    if (int rc = make_map(&mk, dtype, k_pool, block_size, H, num_blocks, H * D, D, block_size * H * D, box_rows)) return rc;
    if (int rc = make_map(&mv, dtype, v_pool, block_size, H, num_blocks, H * D, D, block_size * H * D, box_rows)) return rc;
  }
  if (int rc = make_map(&mp, dtype, pos, pos_rows, H, 1, pos_stride, D, pos_stride * pos_rows, kKeys)) return rc;
  Params p{};
  p.qkv4 = static_cast<const uint8_t*>(qkv4);
  p.ld = 4 * d;
  p.B = (int)B; p.H = (int)H; p.Tq = (int)Tq;
  p.scale_log2 = static_cast<float>(scale * 1.4426950408889634);
  p.seqlens = seqlens; p.pos_start = pos_start; p.block_table = block_table;
  p.blocks_per_seq = (int)blocks_per_seq; p.block_size = (int)block_size; p.num_blocks = (int)num_blocks;
  p.out = out; p.status = device_status_ptr();
  p.k_scale = k_scale; p.v_scale = v_scale;
  const unsigned grid = (unsigned)((B * H + kWarps - 1) / kWarps);
  return OB_DISPATCH_HALF(dtype, T, [&]() -> int {
    return fp8 ? launch<T, true>(mk, mv, mp, p, grid, stream) : launch<T, false>(mk, mv, mp, p, grid, stream);
  });
}

}  // namespace fmha_chunk
}  // namespace ob
