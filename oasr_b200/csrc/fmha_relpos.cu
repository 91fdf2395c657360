// Packed relative-position attention (head_dim 64), the form the offline Conformer layer runs:
//   out[i,:] = softmax_j( ((q_i+u).k_j + (q_i+v).p_j) * scale ) . v_j      over the keys j of row i's segment
// (RelPositionMultiHeadedAttention._forward_packed, oasr/layers/attention/attention.py:323-386).
//
// Same tcgen05 / TMEM / TMA pipeline as fmha.cu, sized so that TWO CTAs share an SM: at head_dim 64 a tile's
// tensor work (0.8k clocks) is a fraction of its softmax (3k) and of the latencies around it (TMEM loads,
// MUFU, barrier hand-offs, 3k clocks before a CTA's first scores arrive), so one CTA per SM leaves every unit
// under 20 % busy; a second resident CTA fills those gaps.  To fit twice:
//   keys are walked in tiles of 64 (K | pos 16 KB, V 8 KB per stage, two stages),
//   P has a single 16 KB buffer (the softmax folds O of tile j-1, which proves P.V of tile j-1 is done, before
//   it rewrites P for tile j),
//   TMEM holds S[2] (2 x 64 columns) and O[2] (2 x 64 columns) = 256 columns,
// i.e. 96 KB of shared memory and half of TMEM per CTA.
// 160 threads: warp 4 lane 0 issues TMA loads and MMAs, warps 0-3 own one query row per thread.
// Only the length mask exists here (keys >= segment length); bias, causal masks, key starts, paged K/V and
// head_dim 128 stay on the general kernel in fmha.cu.  Every wait is bounded.
#include <cuda.h>

#include <type_traits>

#include "common.cuh"
#include "device_status.cuh"
#include "sm100_ptx.cuh"
#include "tma_host.cuh"

namespace ob {
int g_fmha_relpos_path = 1;  // 1 = this kernel for the packed relative-position form; 0 = the general kernel ("fmha_relpos_path")

namespace fmha_relpos {

constexpr int BQ = 128, BKV = 64, D = 64;
constexpr int kThreads = 160;
constexpr int kQBytes = 2 * 128 * 128;          // [q+u | q+v]: two atoms of 128 rows x 128 B
constexpr int kKBytes = 2 * BKV * 128;          // [k | pos] per stage
constexpr int kVBytes = BKV * 128;
constexpr int kPBytes = BQ * 128;               // 128 rows x 64 keys
constexpr int kOffQ = 0, kOffK = kOffQ + kQBytes, kOffV = kOffK + 2 * kKBytes, kOffP = kOffV + 2 * kVBytes;
constexpr int kOffBar = kOffP + kPBytes;
constexpr int kNumBars = 12;
constexpr int kSmemDynamic = kOffBar + kNumBars * 8 + 16 + 1024;
constexpr uint32_t kTmemCols = 256, kColS = 0, kColO = 128;

struct Params {
  int H;
  float scale_log2;
  const int32_t* cu;
  void* out;
  uint32_t* status;
};

__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
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

template <typename T>
__global__ void __launch_bounds__(kThreads, 2)
fmha_relpos64_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_q2,
                     const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_pos,
                     const __grid_constant__ CUtensorMap map_v, const Params p) {
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
  constexpr uint32_t kIdescQK = ptx::umma_idesc_f16(kBf16, BQ, BKV, false, false);
  constexpr uint32_t kIdescPV = ptx::umma_idesc_f16(kBf16, BQ, D, false, true);  // V is MN-major
  constexpr float kNegInf = -INFINITY;

  ptx::grid_dep_launch();   // no-ops unless launched with programmatic stream serialisation
  ptx::grid_dep_wait();
  const int q0 = blockIdx.x * BQ, h = blockIdx.y, seg = blockIdx.z;
  const int row0 = p.cu[seg], kv_len = p.cu[seg + 1] - row0;
  if (q0 >= kv_len) return;  // CTA-uniform (queries and keys of a segment are the same rows)
  const int nkv = (kv_len + BKV - 1) / BKV;
  const int rows_valid = min(BQ, kv_len - q0);
  const int64_t out_ld = static_cast<int64_t>(p.H) * D;
  T* out = static_cast<T*>(p.out) + (static_cast<int64_t>(row0 + q0) * p.H + h) * D;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + kOffQ;
  uint8_t* sK = smem + kOffK;
  uint8_t* sV = smem + kOffV;
  uint8_t* sP = smem + kOffP;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBar);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;    // [2]
  uint64_t* kv_empty = bars + 3;   // [2]
  uint64_t* s_full = bars + 5;     // [2]
  uint64_t* s_free = bars + 7;     // [2]
  uint64_t* p_full = bars + 9;     // [1]
  uint64_t* po_done = bars + 10;   // [2]  P.V into O[b] finished: O[b] is ready and P may be rewritten
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    ptx::mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&kv_full[i], 1);
      ptx::mbar_init(&kv_empty[i], 1);
      ptx::mbar_init(&s_full[i], 1);
      ptx::mbar_init(&s_free[i], BQ);
      ptx::mbar_init(&po_done[i], 1);
    }
    ptx::mbar_init(p_full, BQ);
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == 4) {
    ptx::tmem_alloc(tmem_slot, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // =================== TMA producer + MMA issuer (one thread) ===================
    if (lane == 0) {
      bool ok = true;
      auto load_kv = [&](int t, int b) {
        const int key0 = t * BKV;
        ptx::mbar_expect_tx(&kv_full[b], kKBytes + kVBytes);
        uint8_t* dk = sK + b * kKBytes;
        ptx::tma_load_4d(dk, &map_k, 0, row0 + key0, h, 0, &kv_full[b]);
        ptx::tma_load_4d(dk + BKV * 128, &map_pos, 0, key0, h, 0, &kv_full[b]);
        ptx::tma_load_4d(sV + b * kVBytes, &map_v, 0, row0 + key0, h, 0, &kv_full[b]);
      };
      auto issue_qk = [&](int b) {   // S[b] = [q+u | q+v] . [k | pos]^T : K = 128 in eight steps of 16
        const uint32_t a_addr = ptx::smem_u32(sQ);
        const uint32_t b_addr = ptx::smem_u32(sK + b * kKBytes);
        const uint32_t d_tmem = tmem_base + kColS + b * BKV;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t adesc = ptx::smem_desc_kmajor_sw128(a_addr + (kk / 4) * (128 * 128) + (kk % 4) * 32);
          const uint64_t bdesc = ptx::smem_desc_kmajor_sw128(b_addr + (kk / 4) * (BKV * 128) + (kk % 4) * 32);
          ptx::umma_f16(d_tmem, adesc, bdesc, kIdescQK, kk != 0 ? 1u : 0u);
        }
        ptx::umma_commit(&s_full[b]);
      };
      auto issue_pv = [&](int b) {   // O[b] = P . V_b : K = 64 keys in four steps of 16
        const uint32_t a_addr = ptx::smem_u32(sP);
        const uint32_t b_addr = ptx::smem_u32(sV + b * kVBytes);
        const uint32_t d_tmem = tmem_base + kColO + b * D;
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          const uint64_t adesc = ptx::smem_desc_kmajor_sw128(a_addr + kk * 32);
          const uint64_t bdesc = ptx::smem_desc_mnmajor_sw128(b_addr + kk * 2048, BKV * 128, 1024);
          ptx::umma_f16(d_tmem, adesc, bdesc, kIdescPV, kk != 0 ? 1u : 0u);
        }
        ptx::umma_commit(&po_done[b]);
        ptx::umma_commit(&kv_empty[b]);
      };
      ptx::mbar_expect_tx(q_full, kQBytes);
      ptx::tma_load_4d(sQ, &map_q, 0, row0 + q0, h, 0, q_full);
      ptx::tma_load_4d(sQ + 128 * 128, &map_q2, 0, row0 + q0, h, 0, q_full);
      load_kv(0, 0);
      if (nkv > 1) load_kv(1, 1);
      ok = ptx::mbar_wait(q_full, 0, abort_flag) && ptx::mbar_wait(&kv_full[0], 0, abort_flag);
      if (ok) {
        ptx::tc_fence_after_sync();
        issue_qk(0);
      }
      for (int j = 0; ok && j < nkv; ++j) {
        const int b = j & 1;
        const uint32_t ph = (j >> 1) & 1u;
        if (j + 1 < nkv) {
          const int nb = (j + 1) & 1;
          const uint32_t nph = ((j + 1) >> 1) & 1u;
          // S[nb] was last read by the softmax of tile j-1
          ok = ptx::mbar_wait(&kv_full[nb], nph, abort_flag) && ptx::mbar_wait(&s_free[nb], nph ^ 1u, abort_flag);
          if (!ok) break;
          ptx::tc_fence_after_sync();
          issue_qk(nb);
        }
        ok = ptx::mbar_wait(p_full, static_cast<uint32_t>(j) & 1u, abort_flag);   // P of tile j written
        if (!ok) break;
        ptx::tc_fence_after_sync();
        issue_pv(b);
        if (j + 2 < nkv) {
          ok = ptx::mbar_wait(&kv_empty[b], ph, abort_flag);
          if (!ok) break;
          load_kv(j + 2, b);
        }
      }
      if (!ok && p.status) atomicOr(p.status, kStatusFmhaMma);
    }
    __syncwarp();
  } else {
    // =========================== softmax / output (thread = row) ===========================
    const int r = threadIdx.x;  // 0..127
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const bool row_ok = r < rows_valid;
    float m_run = kNegInf, l_run = 0.f, alpha_prev = 1.f;
    float o[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o[i] = 0.f;
    bool ok = true;
    auto fold_o = [&](int t) -> bool {  // o = o * alpha_prev + O_t
      const int b = t & 1;
      if (!ptx::mbar_wait(&po_done[b], (t >> 1) & 1u, abort_flag)) return false;
      ptx::tc_fence_after_sync();
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t v[32];
        ptx::tmem_ld_32x32(tmem_base + lane_base + kColO + b * D + c0, v);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c0 + i] = fmaf(o[c0 + i], alpha_prev, __uint_as_float(v[i]));
      }
      ptx::tc_fence_before_sync();
      return true;
    };
    for (int j = 0; ok && j < nkv; ++j) {
      const int b = j & 1;
      const int key0 = j * BKV;
      if (!ptx::mbar_wait(&s_full[b], (j >> 1) & 1u, abort_flag)) { ok = false; break; }
      ptx::tc_fence_after_sync();
      const uint32_t t_s = tmem_base + lane_base + kColS + b * BKV;
      // ---- pass 1: row max of the raw scores (32-key blocks inside the valid keys need no mask) ----
      float tile_max = kNegInf;
#pragma unroll 1
      for (int c0 = 0; c0 < BKV; c0 += 32) {
        if (key0 + c0 >= kv_len) break;
        uint32_t v[32];
        ptx::tmem_ld_32x32(t_s + c0, v);
        ptx::tmem_ld_wait();
        if (key0 + c0 + 32 <= kv_len) {
#pragma unroll
          for (int i = 0; i < 32; ++i) tile_max = fmaxf(tile_max, __uint_as_float(v[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) tile_max = fmaxf(tile_max, key0 + c0 + i < kv_len ? __uint_as_float(v[i]) : kNegInf);
        }
      }
      tile_max *= p.scale_log2;   // the scale is positive
      const float m_new = fmaxf(m_run, tile_max);
      const float m_use = (m_new == kNegInf) ? 0.f : m_new;  // empty-row clamp
      const float alpha = (m_run == kNegInf) ? 0.f : ex2_fast(m_run - m_use);
      // ---- O of tile j-1 (also proves that P.V of tile j-1 has finished reading P) ----
      if (j >= 1) {
        if (!fold_o(j - 1)) { ok = false; break; }
      }
      // ---- pass 2: exponentiate, sum, round, write P (K-major, 128-byte swizzle) ----
      float row_sum = 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < BKV; c0 += 32) {
        uint32_t packed[16];
        if (key0 + c0 >= kv_len) {   // P of keys past the end is zero (V rows there hold other segments' finite values)
#pragma unroll
          for (int i = 0; i < 16; ++i) packed[i] = 0u;
        } else {
          uint32_t v[32];
          ptx::tmem_ld_32x32(t_s + c0, v);
          ptx::tmem_ld_wait();
          const bool full = key0 + c0 + 32 <= kv_len;
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float p0 = ex2_fast(fmaf(__uint_as_float(v[i]), p.scale_log2, -m_use));
            float p1 = ex2_fast(fmaf(__uint_as_float(v[i + 1]), p.scale_log2, -m_use));
            if (!full) {
              p0 = key0 + c0 + i < kv_len ? p0 : 0.f;
              p1 = key0 + c0 + i + 1 < kv_len ? p1 : 0.f;
            }
            row_sum += p0 + p1;
            packed[i / 2] = pack2<T>(p0, p1);
          }
        }
        // keys c0..c0+31 of row r: 16-byte chunks c0/8 .. +3, XOR-swizzled by r%8
        uint8_t* row_base = sP + r * 128;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int chunk = (c0 / 8 + q4) ^ (r & 7);
          *reinterpret_cast<uint4*>(row_base + chunk * 16) =
              make_uint4(packed[q4 * 4], packed[q4 * 4 + 1], packed[q4 * 4 + 2], packed[q4 * 4 + 3]);
        }
      }
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(&s_free[b]);
      ptx::fence_proxy_async_smem();
      ptx::mbar_arrive(p_full);
      l_run = l_run * alpha + row_sum;
      m_run = m_new;
      alpha_prev = alpha;
    }
    if (ok) ok = fold_o(nkv - 1);
    if (ok && row_ok) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      T* orow = out + static_cast<int64_t>(r) * out_ld;
#pragma unroll
      for (int c = 0; c < D; c += 8) {
        uint4 w;
        w.x = pack2<T>(o[c] * inv, o[c + 1] * inv);
        w.y = pack2<T>(o[c + 2] * inv, o[c + 3] * inv);
        w.z = pack2<T>(o[c + 4] * inv, o[c + 5] * inv);
        w.w = pack2<T>(o[c + 6] * inv, o[c + 7] * inv);
        *reinterpret_cast<uint4*>(orow + c) = w;
      }
    }
    if (!ok && lane == 0 && p.status) atomicOr(p.status, kStatusFmhaSoftmax);
  }

  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 4) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

int make_map(CUtensorMap* m, int dtype, const void* base, int64_t rows, int64_t heads, int64_t stride_row, int box_rows) {
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)rows, (uint64_t)heads, 1};
  uint64_t str[4] = {0, (uint64_t)stride_row * 2, (uint64_t)D * 2, (uint64_t)stride_row * 2 * (uint64_t)rows};
  uint32_t box[4] = {64, (uint32_t)box_rows, 1, 1};
  return make_tensor_map(m, tma_dtype(dtype), 4, base, dims, str, box);
}

int run(void* out, const void* qkv4, const void* pos, int64_t pos_rows, int64_t pos_stride, const int32_t* cu_seqlens,
        int64_t num_segs, int64_t max_seqlen, int64_t total, int64_t H, double scale, int dtype, cudaStream_t stream) {
  const int64_t d = H * D, ld = 4 * d;
  const uint8_t* base = static_cast<const uint8_t*>(qkv4);
  CUtensorMap mq, mq2, mk, mp, mv;
  if (int rc = make_map(&mq, dtype, base, total, H, ld, BQ)) return rc;
  if (int rc = make_map(&mq2, dtype, base + d * 2, total, H, ld, BQ)) return rc;
  if (int rc = make_map(&mk, dtype, base + 2 * d * 2, total, H, ld, BKV)) return rc;
  if (int rc = make_map(&mv, dtype, base + 3 * d * 2, total, H, ld, BKV)) return rc;
  if (int rc = make_map(&mp, dtype, pos, pos_rows, H, pos_stride, BKV)) return rc;
  Params p{};
  p.H = (int)H;
  p.scale_log2 = static_cast<float>(scale * 1.4426950408889634);
  p.cu = cu_seqlens; p.out = out; p.status = device_status_ptr();
  dim3 grid((unsigned)((max_seqlen + BQ - 1) / BQ), (unsigned)H, (unsigned)num_segs);
  return OB_DISPATCH_HALF(dtype, T, [&]() -> int {
    auto kern = fmha_relpos64_kernel<T>;
    static bool attr_done = false;
    if (!attr_done) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemDynamic);
      if (e == cudaSuccess) e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
      if (e != cudaSuccess)
        return set_error(OASR_ERR_CUDA, "fmha_varlen_relpos: cannot reserve %d bytes of shared memory: %s", kSmemDynamic,
                         cudaGetErrorString(e));
      attr_done = true;
    }
    launch_pdl(kern, grid, dim3(kThreads), kSmemDynamic, stream, mq, mq2, mk, mp, mv, p);
    return check_launch("fmha_varlen_relpos (two CTAs per SM) launch");
  });
}

}  // namespace fmha_relpos
}  // namespace ob
