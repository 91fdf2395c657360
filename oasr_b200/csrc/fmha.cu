// Fused multi-head attention on tcgen05 / TMEM / TMA: dense (+bias, lengths,
// starts, causal), packed variable-length (+packed block-diagonal bias), paged
// KV (+bias) and the Conformer relative-position form that computes the
// position term as a second K-dimension atom instead of reading a bias.
//
//   out[i,:] = softmax_j( (q_i . k_j) * scale + bias[i,j] ) . v_j       (fp32 softmax)
//
// One CTA owns 128 query rows of one (batch|segment, head) and walks the keys
// in tiles of 128.  160 threads:
//   warp 4, one thread: TMA producer and tcgen05.mma issuer
//       S[b]  = Q . K_j^T      (M=128, N=128, K = 64 per atom, 1-2 atoms)  -> TMEM
//       O[b]  = P_j . V_j      (M=128, N=D,   K = 128)                      -> TMEM
//     K/V tiles are double-buffered in shared memory (128-byte swizzle), S and
//     O are double-buffered in TMEM (2x128 + 2xD columns), so QK^T of tile j+1
//     runs under the softmax of tile j;
//   warps 0-3: thread r owns query row r.  Pass 1 reads the S row from TMEM,
//     applies scale, bias and masks in the log2 domain, writes it back and
//     takes the row maximum; pass 2 exponentiates, sums, rounds P to the
//     16-bit input type and writes it to shared memory in the K-major swizzled
//     layout the P.V MMA reads.  The running output is rescaled in registers
//     (o = o * 2^(m_old - m_new) + O_j), so TMEM is never read-modified-written.
// A row with no visible key produces zeros (running max -inf is clamped to 0,
// the row sum stays 0), as in the reference kernel
// (oasr/kernels/cute/softmax.py:141-146,176-181).  Keys outside [start, len)
// and, with `causal`, keys j > i are masked after the bias
// (oasr/kernels/cute/mask.py:102-117).  GQA: query head h reads KV head
// h / (H / Hkv).  The reference runs this path through PyTorch SDPA on sm_100
// (oasr/functionals/attention.py:511-530, 181-220).
//
// Tensor-pipe bound for long keys; algorithmic flops 4*Tq*Tk*D (+2*Tq*Tk*D for
// the in-kernel position term).
#include <cuda.h>

#include <cmath>
#include <type_traits>

#include "common.cuh"
#include "device_status.cuh"
#include "sm100_ptx.cuh"
#include "tma_host.cuh"

namespace ob {
namespace fmha {

constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int kThreads = 160;
constexpr int kAtomBytes = 128 * 128;  // 128 rows x 128 bytes

enum Mode { kDense = 0, kVarlen = 1, kPaged = 2 };

struct Params {
  int mode;
  int B, H, Hkv, Tq, Tk;
  float scale_log2;  // softmax scale * log2(e)
  int causal;
  int relpos;        // second Q/K atom comes from the q2 / k2 tensor maps
  const int32_t* seqlens;
  const int32_t* seqstarts;
  const int32_t* cu_q;
  const int32_t* cu_k;
  const int32_t* block_table;
  int blocks_per_seq, block_size, num_blocks;
  const void* bias;
  int64_t bias_sb, bias_sh, bias_sq;  // dense / paged bias strides (elements)
  const void* bias_offsets;           // varlen: per-segment start (elements)
  int bias_off_i64;
  int bias_ld8;                       // varlen: bias rows of a segment are roundup8(Tk_s) elements apart (16-byte aligned rows)
  const int32_t* pos_start;           // relpos + paged: first position row of each stream's key 0
  int out_token_major;                // dense/paged: out is (B*Tq, H*D) rows instead of (B,H,Tq,D)
  void* out;
  uint32_t* status;
};

struct Maps {
  CUtensorMap q, q2, k, k2, v;
};

template <int D, int kAtoms>
struct Smem {
  static constexpr int kVAtoms = D / 64;
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + kAtoms * kAtomBytes;
  static constexpr int kV = kK + 2 * kAtoms * kAtomBytes;
  static constexpr int kP = kV + 2 * kVAtoms * kAtomBytes;
  static constexpr int kBar = kP + 2 * 2 * kAtomBytes;
  static constexpr int kNumBars = 1 + 2 * 6;
  static constexpr int kTotal = kBar + kNumBars * 8 + 16;
  static constexpr int kDynamic = kTotal + 1024;
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

template <typename T>
__device__ __forceinline__ float unpack_lo(uint32_t w) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) return __uint_as_float(w << 16);
  else return __half2float(__ushort_as_half(static_cast<unsigned short>(w & 0xffffu)));
}
template <typename T>
__device__ __forceinline__ float unpack_hi(uint32_t w) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) return __uint_as_float(w & 0xffff0000u);
  else return __half2float(__ushort_as_half(static_cast<unsigned short>(w >> 16)));
}

__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// kGeneral = false: no bias, no causal mask, no key start -- the only mask is key < kv_len (the packed
// relative-position path and plain attention).  The softmax then never writes scores back to TMEM and the
// code a tile executes stays small.
template <typename T, int D, int kAtoms, bool kGeneral>
__global__ void __launch_bounds__(kThreads, 1)
fmha_tcgen05_kernel(const __grid_constant__ Maps maps, const Params p) {
  using S = Smem<D, kAtoms>;
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
  constexpr uint32_t kIdescQK = ptx::umma_idesc_f16(kBf16, BQ, BKV, false, false);
  constexpr uint32_t kIdescPV = ptx::umma_idesc_f16(kBf16, BQ, D, false, true);  // V is MN-major
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColS = 0, kColO = 256;
  constexpr float kNegInf = -INFINITY;

  // no-ops unless launched with programmatic stream serialisation; cu_seqlens / seqlens below are already
  // global reads, so the wait comes first
  ptx::grid_dep_launch();
  ptx::grid_dep_wait();
  // ---- which rows / keys does this CTA own ---------------------------------
  const int q0 = blockIdx.x * BQ;
  const int h = blockIdx.y;
  const int bz = blockIdx.z;
  const int hkv = h / (p.H / p.Hkv);
  int tq_seg, q_row_c1, q_c3, kv_row_c1, kv_c3, kv_len, kv_start = 0;
  int64_t out_row0;         // element offset of (row q0, this head) in out
  int64_t out_row_stride;   // elements between consecutive query rows
  if (p.mode == kVarlen) {
    const int qa = p.cu_q[bz], qb = p.cu_q[bz + 1], ka = p.cu_k[bz], kb = p.cu_k[bz + 1];
    tq_seg = qb - qa;
    kv_len = kb - ka;
    q_row_c1 = qa + q0; q_c3 = 0;
    kv_row_c1 = ka; kv_c3 = 0;
    out_row_stride = static_cast<int64_t>(p.H) * D;
    out_row0 = (static_cast<int64_t>(qa + q0) * p.H + h) * D;
  } else {
    tq_seg = p.Tq;
    kv_len = p.seqlens ? min(p.seqlens[bz], p.Tk) : p.Tk;
    if (p.seqstarts) kv_start = max(p.seqstarts[bz], 0);
    q_row_c1 = q0; q_c3 = bz;
    kv_row_c1 = 0; kv_c3 = bz;
    if (p.out_token_major) {
      out_row_stride = static_cast<int64_t>(p.H) * D;
      out_row0 = ((static_cast<int64_t>(bz) * p.Tq + q0) * p.H + h) * D;
    } else {
      out_row_stride = D;
      out_row0 = ((static_cast<int64_t>(bz) * p.H + h) * p.Tq + q0) * D;
    }
  }
  if (q0 >= tq_seg) return;  // CTA-uniform
  int kv_end = kv_len;
  if (p.causal) kv_end = min(kv_end, q0 + BQ);
  const int tile_begin = kv_start / BKV;
  const int tile_end = (kv_end + BKV - 1) / BKV;
  const int nkv = max(tile_end - tile_begin, 0);
  T* out = static_cast<T*>(p.out) + out_row0;
  const int rows_valid = min(BQ, tq_seg - q0);

  if (nkv == 0) {  // nothing visible: zero rows, no pipeline (CTA-uniform)
    for (int i = threadIdx.x; i < rows_valid * (D / 8); i += blockDim.x) {
      const int r = i / (D / 8), c = (i % (D / 8)) * 8;
      *reinterpret_cast<uint4*>(out + r * out_row_stride + c) = make_uint4(0, 0, 0, 0);
    }
    return;
  }

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + S::kQ;
  uint8_t* sK = smem + S::kK;
  uint8_t* sV = smem + S::kV;
  uint8_t* sP = smem + S::kP;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kBar);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;    // [2]
  uint64_t* kv_empty = bars + 3;   // [2]
  uint64_t* s_full = bars + 5;     // [2]
  uint64_t* s_free = bars + 7;     // [2]
  uint64_t* p_full = bars + 9;     // [2]
  uint64_t* po_done = bars + 11;   // [2]  P.V of buffer b finished: O[b] is ready and P[b] may be rewritten
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + S::kNumBars);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // Barrier block: q_full, kv_full[2], kv_empty[2], s_full[2], s_free[2], p_full[2], po_done[2] = 13.
  // O[b] and P[b] need no "free" barrier of their own: a softmax thread folds O[b] of tile j-2 (which
  // also proves P.V of tile j-2 has finished reading P[b]) before it arrives on p_full[b] for tile j.
  if (threadIdx.x == 0) {
    ptx::mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&kv_full[i], 1);
      ptx::mbar_init(&kv_empty[i], 1);
      ptx::mbar_init(&s_full[i], 1);
      ptx::mbar_init(&s_free[i], BQ);
      ptx::mbar_init(&p_full[i], BQ);
      ptx::mbar_init(&po_done[i], 1);
    }
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
      constexpr uint32_t kKVBytes = (kAtoms + S::kVAtoms) * kAtomBytes;
      auto load_kv = [&](int t /*tile index within [0,nkv)*/, int b) {
        const int key0 = (tile_begin + t) * BKV;
        ptx::mbar_expect_tx(&kv_full[b], kKVBytes);
        uint8_t* dk = sK + b * kAtoms * kAtomBytes;
        uint8_t* dv = sV + b * S::kVAtoms * kAtomBytes;
        if (p.mode == kPaged) {
          const int bs = p.block_size;
          const int pages = BKV / bs;
          for (int pg = 0; pg < pages; ++pg) {
            int col = key0 / bs + pg;
            if (col >= p.blocks_per_seq) col = p.blocks_per_seq - 1;  // masked keys: any valid page
            int page = p.block_table[static_cast<int64_t>(bz) * p.blocks_per_seq + col];
            page = min(max(page, 0), p.num_blocks - 1);
            if (p.relpos) {
              ptx::tma_load_4d(dk + pg * bs * 128, &maps.k, 0, 0, hkv, page, &kv_full[b]);
            } else {
#pragma unroll
              for (int a = 0; a < kAtoms; ++a)
                ptx::tma_load_4d(dk + a * kAtomBytes + pg * bs * 128, &maps.k, a * 64, 0, hkv, page, &kv_full[b]);
            }
#pragma unroll
            for (int a = 0; a < S::kVAtoms; ++a)
              ptx::tma_load_4d(dv + a * kAtomBytes + pg * bs * 128, &maps.v, a * 64, 0, hkv, page, &kv_full[b]);
          }
          // position term of the keys of this tile: rows pos_start[b] + key0 ... of the projected table
          if (p.relpos) ptx::tma_load_4d(dk + kAtomBytes, &maps.k2, 0, p.pos_start[bz] + key0, h, 0, &kv_full[b]);
        } else {
          if (p.relpos) {
            ptx::tma_load_4d(dk, &maps.k, 0, kv_row_c1 + key0, hkv, kv_c3, &kv_full[b]);
            ptx::tma_load_4d(dk + kAtomBytes, &maps.k2, 0, key0, h, 0, &kv_full[b]);
          } else {
#pragma unroll
            for (int a = 0; a < kAtoms; ++a)
              ptx::tma_load_4d(dk + a * kAtomBytes, &maps.k, a * 64, kv_row_c1 + key0, hkv, kv_c3, &kv_full[b]);
          }
#pragma unroll
          for (int a = 0; a < S::kVAtoms; ++a)
            ptx::tma_load_4d(dv + a * kAtomBytes, &maps.v, a * 64, kv_row_c1 + key0, hkv, kv_c3, &kv_full[b]);
        }
      };
      auto issue_qk = [&](int b) {
        const uint32_t a_addr = ptx::smem_u32(sQ);
        const uint32_t b_addr = ptx::smem_u32(sK + b * kAtoms * kAtomBytes);
        const uint32_t d_tmem = tmem_base + kColS + b * BKV;
#pragma unroll
        for (int kk = 0; kk < kAtoms * 4; ++kk) {
          const uint32_t off = (kk / 4) * kAtomBytes + (kk % 4) * 32;
          ptx::umma_f16(d_tmem, ptx::smem_desc_kmajor_sw128(a_addr + off), ptx::smem_desc_kmajor_sw128(b_addr + off),
                        kIdescQK, kk != 0 ? 1u : 0u);
        }
        ptx::umma_commit(&s_full[b]);
      };
      auto issue_pv = [&](int b) {
        const uint32_t a_addr = ptx::smem_u32(sP + b * 2 * kAtomBytes);
        const uint32_t b_addr = ptx::smem_u32(sV + b * S::kVAtoms * kAtomBytes);
        const uint32_t d_tmem = tmem_base + kColO + b * D;
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          const uint64_t adesc = ptx::smem_desc_kmajor_sw128(a_addr + (kk / 4) * kAtomBytes + (kk % 4) * 32);
          // V tile: rows = keys (128 B each), 16 keys per MMA = 2048 B; atoms along D are kAtomBytes apart
          const uint64_t bdesc = ptx::smem_desc_mnmajor_sw128(b_addr + kk * 2048, kAtomBytes, 1024);
          ptx::umma_f16(d_tmem, adesc, bdesc, kIdescPV, kk != 0 ? 1u : 0u);
        }
        ptx::umma_commit(&po_done[b]);
        ptx::umma_commit(&kv_empty[b]);
      };

      // Q tile (+ second atom)
      ptx::mbar_expect_tx(q_full, kAtoms * kAtomBytes);
      if (p.relpos) {
        ptx::tma_load_4d(sQ, &maps.q, 0, q_row_c1, h, q_c3, q_full);
        ptx::tma_load_4d(sQ + kAtomBytes, &maps.q2, 0, q_row_c1, h, q_c3, q_full);
      } else {
#pragma unroll
        for (int a = 0; a < kAtoms; ++a) ptx::tma_load_4d(sQ + a * kAtomBytes, &maps.q, a * 64, q_row_c1, h, q_c3, q_full);
      }
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
        // P[b] written and O[b] of tile j-2 consumed (the softmax threads fold O[b] before they
        // arrive on p_full[b] for tile j)
        ok = ptx::mbar_wait(&p_full[b], ph, abort_flag);
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
    const int row_in_seq = q0 + r;
    // bias row pointer
    const T* bias_row = nullptr;
    if (p.bias) {
      const T* bias = static_cast<const T*>(p.bias);
      if (p.mode == kVarlen) {
        const int64_t off = p.bias_off_i64 ? static_cast<const int64_t*>(p.bias_offsets)[bz]
                                           : static_cast<int64_t>(static_cast<const int32_t*>(p.bias_offsets)[bz]);
        bias_row = bias + off + (static_cast<int64_t>(h) * tq_seg + row_in_seq) * (p.bias_ld8 ? ((kv_len + 7) & ~7) : kv_len);
      } else {
        bias_row = bias + bz * p.bias_sb + h * p.bias_sh + static_cast<int64_t>(row_in_seq) * p.bias_sq;
      }
    }
    const bool row_ok = r < rows_valid;
    const bool bias_vec = bias_row && (p.mode == kDense || (p.mode == kVarlen && p.bias_ld8)) &&
                          (reinterpret_cast<uintptr_t>(bias_row) & 15u) == 0;
    const int bias_cols = p.mode == kDense ? p.Tk : ((kv_len + 7) & ~7);   // columns of a bias row that exist in memory
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
      const uint32_t ph = (j >> 1) & 1u;
      const int key0 = (tile_begin + j) * BKV;
      if (!ptx::mbar_wait(&s_full[b], ph, abort_flag)) { ok = false; break; }
      ptx::tc_fence_after_sync();
      const uint32_t t_s = tmem_base + lane_base + kColS + b * BKV;
      float tile_max = kNegInf, m_new, m_use, alpha, row_sum = 0.f;
      uint8_t* p_tile = sP + b * 2 * kAtomBytes;
      // keys c0..c0+31 of row r: atom c0/64, 16-byte chunks (c0%64)/8 .. +3, XOR-swizzled by r%8
      auto write_p = [&](const uint32_t (&packed)[16], int c0) {
        uint8_t* row_base = p_tile + (c0 / 64) * kAtomBytes + r * 128;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int chunk = ((c0 % 64) / 8 + q4) ^ (r & 7);
          *reinterpret_cast<uint4*>(row_base + chunk * 16) =
              make_uint4(packed[q4 * 4], packed[q4 * 4 + 1], packed[q4 * 4 + 2], packed[q4 * 4 + 3]);
        }
      };
      if constexpr (!kGeneral) {
        // ---- pass 1: row max of the raw scores; 32-key blocks that end inside the valid keys need no mask ----
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
        m_new = fmaxf(m_run, tile_max);
        m_use = (m_new == kNegInf) ? 0.f : m_new;  // empty-row clamp
        alpha = (m_run == kNegInf) ? 0.f : ex2_fast(m_run - m_use);
        // ---- pass 2: exponentiate, sum, round, write P (K-major, 128-byte swizzle) ----
#pragma unroll 1
        for (int c0 = 0; c0 < BKV; c0 += 32) {
          uint32_t packed[16];
          if (key0 + c0 >= kv_len) {   // P of keys past the end is zero (V rows there may hold anything finite)
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
          write_p(packed, c0);
        }
      } else {
      // ---- pass 1: row max.  Interior tiles without a bias need no mask and no write-back: the max of
      // the raw scores is taken and the (positive) scale applied in pass 2.  Edge tiles and biased tiles
      // get scale, bias and masks applied here (log2 domain) and written back to TMEM. ----
      const bool plain_tile = !bias_row && !p.causal && key0 + BKV <= kv_len && key0 >= kv_start;
      if (plain_tile) {
#pragma unroll 1
        for (int c0 = 0; c0 < BKV; c0 += 32) {
          uint32_t v[32];
          ptx::tmem_ld_32x32(t_s + c0, v);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) tile_max = fmaxf(tile_max, __uint_as_float(v[i]));
        }
        tile_max *= p.scale_log2;
      } else {
        // kInterior: every key of the tile is inside [kv_start, kv_len) and there is no causal edge, so the
        // per-element visibility test drops out (the usual tile when the masks arrive through the bias)
        auto biased_pass = [&](auto interior_c) {
        constexpr bool kInterior = decltype(interior_c)::value;
#pragma unroll 1
        for (int c0 = 0; c0 < BKV; c0 += 32) {
          uint32_t v[32];
          ptx::tmem_ld_32x32(t_s + c0, v);
          // bias of keys c0..c0+31 of this row, packed two per word: 16-byte loads where the row is aligned and the
          // group of 8 lies inside the bias width, element loads (predicated on the key range) otherwise
          uint32_t bw[16];
          if (bias_row && row_ok) {
            const T* bp = bias_row + key0 + c0;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const int kg = key0 + c0 + g * 8;
              if (bias_vec && kg + 8 <= bias_cols) {
                const uint4 w = __ldg(reinterpret_cast<const uint4*>(bp + g * 8));
                bw[g * 4] = w.x; bw[g * 4 + 1] = w.y; bw[g * 4 + 2] = w.z; bw[g * 4 + 3] = w.w;
              } else {
#pragma unroll
                for (int e = 0; e < 8; e += 2) {
                  const float b0 = kg + e < kv_len ? Elem<T>::to_f(__ldg(bp + g * 8 + e)) : 0.f;
                  const float b1 = kg + e + 1 < kv_len ? Elem<T>::to_f(__ldg(bp + g * 8 + e + 1)) : 0.f;
                  bw[g * 4 + e / 2] = pack2<T>(b0, b1);
                }
              }
            }
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) bw[i] = 0u;
          }
          ptx::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = key0 + c0 + i;
            const float bf = (i & 1) ? unpack_hi<T>(bw[i / 2]) : unpack_lo<T>(bw[i / 2]);
            float x = fmaf(bf, 1.4426950408889634f, __uint_as_float(v[i]) * p.scale_log2);
            if constexpr (!kInterior) {
              const bool visible = key < kv_len && key >= kv_start && !(p.causal && key > row_in_seq);
              x = visible ? x : kNegInf;
            }
            tile_max = fmaxf(tile_max, x);
            v[i] = __float_as_uint(x);
          }
          ptx::tmem_st_32x32(t_s + c0, v);
        }
        };
        if (!p.causal && key0 + BKV <= kv_len && key0 >= kv_start) biased_pass(std::true_type{});
        else biased_pass(std::false_type{});
        ptx::tmem_st_wait();
      }
      m_new = fmaxf(m_run, tile_max);
      m_use = (m_new == kNegInf) ? 0.f : m_new;  // empty-row clamp
      alpha = (m_run == kNegInf) ? 0.f : exp2f(m_run - m_use);
      const float pscale = plain_tile ? p.scale_log2 : 1.f;   // pass 2 computes exp2(x * pscale - m_use)
      // ---- pass 2: exponentiate, sum, round, write P (K-major, 128-byte swizzle) ----
      // P[b] is free: this thread folded O of tile j-2 (po_done[b]) in the previous iteration.
#pragma unroll 1
      for (int c0 = 0; c0 < BKV; c0 += 32) {
        uint32_t v[32];
        ptx::tmem_ld_32x32(t_s + c0, v);
        ptx::tmem_ld_wait();
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = ex2_fast(fmaf(__uint_as_float(v[i]), pscale, -m_use));   // ex2(-inf) = +0: masked keys
          const float p1 = ex2_fast(fmaf(__uint_as_float(v[i + 1]), pscale, -m_use));
          row_sum += p0 + p1;
          packed[i / 2] = pack2<T>(p0, p1);
        }
        write_p(packed, c0);
      }
      }
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(&s_free[b]);
      ptx::fence_proxy_async_smem();
      ptx::mbar_arrive(&p_full[b]);
      l_run = l_run * alpha + row_sum;
      m_run = m_new;
      // ---- fold the previous tile's output while P.V of this tile runs ----
      if (j >= 1) {
        if (!fold_o(j - 1)) { ok = false; break; }
      }
      alpha_prev = alpha;
    }
    if (ok) ok = fold_o(nkv - 1);
    if (ok && row_ok) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      T* orow = out + static_cast<int64_t>(r) * out_row_stride;
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

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
// 4-D map over a (rows, heads, D) style tensor: dims {D, rows, heads, batch}, box {64, box_rows, 1, 1}.
int make_map(CUtensorMap* m, int dtype, const void* base, int D, int64_t rows, int64_t heads, int64_t batch,
             int64_t stride_row, int64_t stride_head, int64_t stride_batch, int box_rows) {
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)rows, (uint64_t)heads, (uint64_t)batch};
  uint64_t str[4] = {0, (uint64_t)stride_row * 2, (uint64_t)stride_head * 2, (uint64_t)stride_batch * 2};
  uint32_t box[4] = {64, (uint32_t)box_rows, 1, 1};
  return make_tensor_map(m, tma_dtype(dtype), 4, base, dims, str, box);
}

template <typename T, int D, int kAtoms, bool kGeneral>
int launch_k(const Maps& maps, const Params& p, dim3 grid, cudaStream_t s) {
  using S = Smem<D, kAtoms>;
  auto kern = fmha_tcgen05_kernel<T, D, kAtoms, kGeneral>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kDynamic);
    if (e != cudaSuccess)
      return set_error(OASR_ERR_CUDA, "fmha: cannot reserve %d bytes of shared memory: %s", S::kDynamic,
                       cudaGetErrorString(e));
    attr_done = true;
  }
  launch_pdl(kern, grid, dim3(kThreads), S::kDynamic, s, maps, p);
  return check_launch("fmha launch");
}

template <typename T, int D, int kAtoms>
int launch(const Maps& maps, const Params& p, dim3 grid, cudaStream_t s) {
  const bool general = p.bias != nullptr || p.causal || p.seqstarts != nullptr;
  return general ? launch_k<T, D, kAtoms, true>(maps, p, grid, s) : launch_k<T, D, kAtoms, false>(maps, p, grid, s);
}

int dispatch(const Maps& maps, const Params& p, int D, int dtype, dim3 grid, cudaStream_t s) {
  return OB_DISPATCH_HALF(dtype, T, [&]() -> int {
    if (D == 64 && p.relpos) return launch<T, 64, 2>(maps, p, grid, s);
    if (D == 64) return launch<T, 64, 1>(maps, p, grid, s);
    if (D == 128 && !p.relpos) return launch<T, 128, 2>(maps, p, grid, s);
    return set_error(OASR_ERR_UNSUPPORTED, "fmha: head_dim %d is not supported (64 and 128 are)", D);
  });
}

bool stride_ok(int64_t s) { return s % 8 == 0; }

}  // namespace fmha

namespace fmha_relpos {  // fmha_relpos.cu: packed relative-position form, two CTAs per SM
int run(void* out, const void* qkv4, const void* pos, int64_t pos_rows, int64_t pos_stride, const int32_t* cu_seqlens,
        int64_t num_segs, int64_t max_seqlen, int64_t total, int64_t H, double scale, int dtype, const int2* items,
        const int32_t* n_items, cudaStream_t stream);
constexpr int kPlanMaxSegs = 1024;
int64_t plan_bytes(int64_t num_segs, int64_t H, int64_t total);
int plan(void* plan_buf, const int32_t* cu_seqlens, int64_t num_segs, int64_t H, cudaStream_t stream);
}  // namespace fmha_relpos
extern int g_fmha_relpos_path;

namespace fmha_chunk {   // fmha_chunk.cu: warp-per-(stream, head) kernel for <= 16 query frames
bool applies(int64_t Tq, int64_t block_size, int64_t blocks_per_seq);
bool applies_fp8(int64_t Tq, int64_t block_size, int64_t blocks_per_seq);
int run(void* out, const void* qkv4, void* k_pool, void* v_pool, const float* k_scale, const float* v_scale, const void* pos,
        int64_t pos_rows, int64_t pos_stride, const int32_t* pos_start, const int32_t* block_table, const int32_t* seqlens,
        int64_t B, int64_t Tq, int64_t H, int64_t blocks_per_seq, int64_t block_size, int64_t num_blocks, double scale,
        int dtype, cudaStream_t stream);
}  // namespace fmha_chunk

}  // namespace ob

extern "C" {

int64_t oasr_b200_fmha_relpos_plan_bytes(int64_t num_segs, int64_t H, int64_t total) {
  if (num_segs < 0 || H <= 0 || total < 0) return -1;
  return ob::fmha_relpos::plan_bytes(num_segs, H, total);
}

int oasr_b200_fmha_relpos_plan(void* plan, int64_t plan_bytes, const int32_t* cu_seqlens, int64_t num_segs, int64_t H,
                               int64_t total, void* stream) {
  using namespace ob;
  OB_REQUIRE(num_segs >= 0 && H > 0 && H <= 32767 && total >= 0, OASR_ERR_INVALID, "fmha_relpos_plan: bad shape");
  if (num_segs == 0) return OASR_OK;
  OB_REQUIRE(plan && cu_seqlens && is_aligned(plan, 16), OASR_ERR_INVALID, "fmha_relpos_plan: null or unaligned pointer");
  OB_REQUIRE(num_segs <= fmha_relpos::kPlanMaxSegs, OASR_ERR_UNSUPPORTED,
             "fmha_relpos_plan: at most %d segments (got %lld); run oasr_b200_fmha_varlen_relpos without a plan",
             fmha_relpos::kPlanMaxSegs, (long long)num_segs);
  OB_REQUIRE(plan_bytes >= fmha_relpos::plan_bytes(num_segs, H, total), OASR_ERR_INVALID,
             "fmha_relpos_plan: plan buffer of %lld bytes, %lld needed", (long long)plan_bytes,
             (long long)fmha_relpos::plan_bytes(num_segs, H, total));
  return fmha_relpos::plan(plan, cu_seqlens, num_segs, H, static_cast<cudaStream_t>(stream));
}

static int fmha_varlen_relpos_impl(void* out, const void* qkv4, const void* pos, int64_t pos_rows, int64_t pos_stride,
                                   const int32_t* cu_seqlens, int64_t num_segs, int64_t max_seqlen, int64_t total,
                                   int64_t H, double scale, const void* plan, int dtype, void* stream_);

int oasr_b200_fmha_varlen_relpos(void* out, const void* qkv4, const void* pos, int64_t pos_rows,
                                 int64_t pos_stride, const int32_t* cu_seqlens, int64_t num_segs,
                                 int64_t max_seqlen, int64_t total, int64_t H, double scale, int dtype,
                                 void* stream_) {
  return fmha_varlen_relpos_impl(out, qkv4, pos, pos_rows, pos_stride, cu_seqlens, num_segs, max_seqlen, total, H, scale,
                                 nullptr, dtype, stream_);
}

int oasr_b200_fmha_varlen_relpos_planned(void* out, const void* qkv4, const void* pos, int64_t pos_rows,
                                         int64_t pos_stride, const int32_t* cu_seqlens, int64_t num_segs,
                                         int64_t max_seqlen, int64_t total, int64_t H, double scale, const void* plan,
                                         int dtype, void* stream_) {
  return fmha_varlen_relpos_impl(out, qkv4, pos, pos_rows, pos_stride, cu_seqlens, num_segs, max_seqlen, total, H, scale,
                                 plan, dtype, stream_);
}

static int fmha_varlen_relpos_impl(void* out, const void* qkv4, const void* pos, int64_t pos_rows, int64_t pos_stride,
                                   const int32_t* cu_seqlens, int64_t num_segs, int64_t max_seqlen, int64_t total,
                                   int64_t H, double scale, const void* plan, int dtype, void* stream_) {
  using namespace ob;
  using namespace ob::fmha;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int D = 64;
  if (num_segs == 0 || max_seqlen == 0 || total == 0) return OASR_OK;
  OB_REQUIRE(out && qkv4 && pos && cu_seqlens, OASR_ERR_INVALID, "fmha_varlen_relpos: null pointer argument");
  OB_REQUIRE(pos_rows >= max_seqlen, OASR_ERR_INVALID, "fmha_varlen_relpos: pos must cover max_seqlen rows");
  OB_REQUIRE(num_segs <= 65535 && H <= 65535, OASR_ERR_INVALID, "fmha_varlen_relpos: segment / head count too large");
  OB_REQUIRE(is_aligned(out, 16) && is_aligned(qkv4, 16) && is_aligned(pos, 16) && pos_stride % 8 == 0,
             OASR_ERR_ALIGN, "fmha_varlen_relpos: operands must be 16-byte aligned");
  if (num_segs == 0 || max_seqlen == 0 || total == 0) return OASR_OK;
  if (g_fmha_relpos_path)
    return fmha_relpos::run(out, qkv4, pos, pos_rows, pos_stride, cu_seqlens, num_segs, max_seqlen, total, H, scale, dtype,
                            plan ? reinterpret_cast<const int2*>(static_cast<const int32_t*>(plan) + 4) : nullptr,
                            static_cast<const int32_t*>(plan), stream);
  const int64_t d = H * D, ld = 4 * d;
  const uint8_t* base = static_cast<const uint8_t*>(qkv4);
  Maps maps;
  if (int rc = make_map(&maps.q, dtype, base, D, total, H, 1, ld, D, ld * total, BQ)) return rc;
  if (int rc = make_map(&maps.q2, dtype, base + d * 2, D, total, H, 1, ld, D, ld * total, BQ)) return rc;
  if (int rc = make_map(&maps.k, dtype, base + 2 * d * 2, D, total, H, 1, ld, D, ld * total, BKV)) return rc;
  if (int rc = make_map(&maps.v, dtype, base + 3 * d * 2, D, total, H, 1, ld, D, ld * total, BKV)) return rc;
  if (int rc = make_map(&maps.k2, dtype, pos, D, pos_rows, H, 1, pos_stride, D, pos_stride * pos_rows, BKV)) return rc;
  Params p{};
  p.mode = kVarlen; p.B = (int)num_segs; p.H = (int)H; p.Hkv = (int)H; p.Tq = (int)max_seqlen; p.Tk = (int)max_seqlen;
  p.scale_log2 = static_cast<float>(scale * 1.4426950408889634);
  p.relpos = 1; p.cu_q = cu_seqlens; p.cu_k = cu_seqlens; p.out = out; p.status = device_status_ptr();
  dim3 grid((unsigned)((max_seqlen + BQ - 1) / BQ), (unsigned)H, (unsigned)num_segs);
  return dispatch(maps, p, D, dtype, grid, stream);
}


int oasr_b200_fmha_paged_relpos(void* out, const void* qkv4, void* k_pool, void* v_pool, const void* pos,
                                int64_t pos_rows, int64_t pos_stride, const int32_t* pos_start,
                                const int32_t* block_table, const int32_t* seqlens, int64_t B, int64_t Tq, int64_t H,
                                int64_t blocks_per_seq, int64_t block_size, int64_t num_blocks, double scale,
                                int dtype, void* stream) {
  using namespace ob;
  using namespace ob::fmha;
  const int D = 64;
  OB_REQUIRE(B >= 0 && Tq >= 0 && H > 0, OASR_ERR_INVALID, "fmha_paged_relpos: bad shape");
  if (B == 0 || Tq == 0) return OASR_OK;
  OB_REQUIRE(out && qkv4 && k_pool && v_pool && pos && pos_start && block_table && seqlens, OASR_ERR_INVALID,
             "fmha_paged_relpos: null pointer argument");
  OB_REQUIRE(Tq <= BQ, OASR_ERR_UNSUPPORTED, "fmha_paged_relpos: at most %d query frames per stream", BQ);
  OB_REQUIRE(block_size > 0 && blocks_per_seq > 0 && num_blocks > 0 && BKV % block_size == 0 && block_size % 8 == 0,
             OASR_ERR_UNSUPPORTED,
             "fmha_paged_relpos: block size must divide 128 and be a multiple of 8 (got %lld)", (long long)block_size);
  OB_REQUIRE(is_aligned(out, 16) && is_aligned(qkv4, 16) && is_aligned(k_pool, 16) && is_aligned(v_pool, 16) &&
                 is_aligned(pos, 16) && pos_stride % 8 == 0,
             OASR_ERR_ALIGN, "fmha_paged_relpos: operands must be 16-byte aligned");
  OB_REQUIRE(B <= 65535 && H <= 65535, OASR_ERR_INVALID, "fmha_paged_relpos: batch / head count too large");
  if (fmha_chunk::applies(Tq, block_size, blocks_per_seq))
    return fmha_chunk::run(out, qkv4, k_pool, v_pool, nullptr, nullptr, pos, pos_rows, pos_stride, pos_start, block_table,
                           seqlens, B, Tq, H, blocks_per_seq, block_size, num_blocks, scale, dtype,
                           static_cast<cudaStream_t>(stream));
  const int64_t d = H * D, ld = 4 * d;
  const uint8_t* base = static_cast<const uint8_t*>(qkv4);
  Maps maps;
  if (int rc = make_map(&maps.q, dtype, base, D, Tq, H, B, ld, D, Tq * ld, BQ)) return rc;
  if (int rc = make_map(&maps.q2, dtype, base + d * 2, D, Tq, H, B, ld, D, Tq * ld, BQ)) return rc;
  if (int rc = make_map(&maps.k, dtype, k_pool, D, block_size, H, num_blocks, H * D, D, block_size * H * D,
                        (int)block_size))
    return rc;
  if (int rc = make_map(&maps.v, dtype, v_pool, D, block_size, H, num_blocks, H * D, D, block_size * H * D,
                        (int)block_size))
    return rc;
  if (int rc = make_map(&maps.k2, dtype, pos, D, pos_rows, H, 1, pos_stride, D, pos_stride * pos_rows, BKV)) return rc;
  Params p{};
  p.mode = kPaged; p.B = (int)B; p.H = (int)H; p.Hkv = (int)H; p.Tq = (int)Tq;
  p.Tk = (int)(blocks_per_seq * block_size);
  p.scale_log2 = static_cast<float>(scale * 1.4426950408889634);
  p.relpos = 1; p.seqlens = seqlens; p.pos_start = pos_start; p.out_token_major = 1;
  p.block_table = block_table; p.blocks_per_seq = (int)blocks_per_seq; p.block_size = (int)block_size;
  p.num_blocks = (int)num_blocks;
  p.out = out; p.status = device_status_ptr();
  dim3 grid(1, (unsigned)H, (unsigned)B);
  return dispatch(maps, p, D, dtype, grid, static_cast<cudaStream_t>(stream));
}

int oasr_b200_fmha_paged_relpos_fp8(void* out, const void* qkv4, void* k_pool, void* v_pool, const float* k_scale,
                                    const float* v_scale, const void* pos, int64_t pos_rows, int64_t pos_stride,
                                    const int32_t* pos_start, const int32_t* block_table, const int32_t* seqlens, int64_t B,
                                    int64_t Tq, int64_t H, int64_t blocks_per_seq, int64_t block_size, int64_t num_blocks,
                                    double scale, int dtype, void* stream) {
  using namespace ob;
  OB_REQUIRE(B >= 0 && Tq >= 0 && H > 0, OASR_ERR_INVALID, "fmha_paged_relpos_fp8: bad shape");
  if (B == 0 || Tq == 0) return OASR_OK;
  OB_REQUIRE(out && qkv4 && k_pool && v_pool && k_scale && v_scale && pos && pos_start && block_table && seqlens,
             OASR_ERR_INVALID, "fmha_paged_relpos_fp8: null pointer argument");
  OB_REQUIRE(block_size > 0 && blocks_per_seq > 0 && num_blocks > 0, OASR_ERR_INVALID, "fmha_paged_relpos_fp8: bad page geometry");
  OB_REQUIRE(fmha_chunk::applies_fp8(Tq, block_size, blocks_per_seq), OASR_ERR_UNSUPPORTED,
             "fmha_paged_relpos_fp8: at most 16 query frames, pages of 16 or a multiple of 32 frames, at most 64 pages per stream");
  OB_REQUIRE(is_aligned(out, 16) && is_aligned(qkv4, 16) && is_aligned(k_pool, 16) && is_aligned(v_pool, 16) &&
                 is_aligned(pos, 16) && pos_stride % 8 == 0,
             OASR_ERR_ALIGN, "fmha_paged_relpos_fp8: operands must be 16-byte aligned");
  return fmha_chunk::run(out, qkv4, k_pool, v_pool, k_scale, v_scale, pos, pos_rows, pos_stride, pos_start, block_table,
                         seqlens, B, Tq, H, blocks_per_seq, block_size, num_blocks, scale, dtype,
                         static_cast<cudaStream_t>(stream));
}

static int fmha_dense_or_paged(void* out, const void* q, const void* k, const void* v, const int64_t* q_strides,
                   const int64_t* k_strides, const int64_t* v_strides, const void* bias, int64_t bias_stride_b,
                   int64_t bias_stride_h, int64_t bias_stride_q, const int32_t* seqlens, const int32_t* seqstarts,
                   const int32_t* block_table, int64_t blocks_per_seq, int64_t block_size, int64_t num_blocks,
                   int64_t B, int64_t H, int64_t Hkv, int64_t Tq, int64_t Tk, int64_t D, double scale, int causal,
                   int dtype, void* stream, int out_token_major) {
  using namespace ob;
  using namespace ob::fmha;
  OB_REQUIRE(B >= 0 && H > 0 && Hkv > 0 && Tq >= 0 && Tk >= 0 && D > 0, OASR_ERR_INVALID, "fmha: bad shape");
  OB_REQUIRE(H % Hkv == 0, OASR_ERR_INVALID, "fmha: H (%lld) must be divisible by H_kv (%lld)", (long long)H,
             (long long)Hkv);
  if (B == 0 || Tq == 0) return OASR_OK;
  OB_REQUIRE(out && q && k && v, OASR_ERR_INVALID, "fmha: null pointer argument");
  OB_REQUIRE(is_aligned(out, 16) && is_aligned(q, 16) && is_aligned(k, 16) && is_aligned(v, 16), OASR_ERR_ALIGN,
             "fmha: q/k/v/out must be 16-byte aligned");
  OB_REQUIRE(!seqstarts || seqlens, OASR_ERR_INVALID, "fmha: cache_seqstarts requires cache_seqlens");
  OB_REQUIRE(B <= 65535 && H <= 65535, OASR_ERR_INVALID, "fmha: batch / head count too large");
  OB_REQUIRE(D == 64 || D == 128, OASR_ERR_UNSUPPORTED, "fmha: head_dim %lld is not supported (64 and 128 are)",
             (long long)D);
  const bool paged = block_table != nullptr;
  const int64_t qs[3] = {q_strides ? q_strides[0] : H * Tq * D, q_strides ? q_strides[1] : Tq * D,
                         q_strides ? q_strides[2] : D};
  OB_REQUIRE(stride_ok(qs[0]) && stride_ok(qs[1]) && stride_ok(qs[2]), OASR_ERR_ALIGN,
             "fmha: q strides must be multiples of 8 elements");
  Maps maps;
  Params p{};
  if (int rc = make_map(&maps.q, dtype, q, (int)D, Tq, H, B, qs[2], qs[1], qs[0], BQ)) return rc;
  maps.q2 = maps.q;
  if (paged) {
    OB_REQUIRE(block_size > 0 && blocks_per_seq > 0 && num_blocks > 0 && BKV % block_size == 0 && block_size % 8 == 0,
               OASR_ERR_UNSUPPORTED,
               "fmha: paged mode needs a block size that divides 128 and is a multiple of 8 (got %lld)",
               (long long)block_size);
    Tk = blocks_per_seq * block_size;
    // pools (num_blocks, block_size, Hkv, D) -> dims {D, block_size, Hkv, num_blocks}
    if (int rc = make_map(&maps.k, dtype, k, (int)D, block_size, Hkv, num_blocks, Hkv * D, D, block_size * Hkv * D,
                          (int)block_size))
      return rc;
    if (int rc = make_map(&maps.v, dtype, v, (int)D, block_size, Hkv, num_blocks, Hkv * D, D, block_size * Hkv * D,
                          (int)block_size))
      return rc;
    p.mode = kPaged;
    p.block_table = block_table; p.blocks_per_seq = (int)blocks_per_seq; p.block_size = (int)block_size;
    p.num_blocks = (int)num_blocks;
  } else {
    const int64_t ks[3] = {k_strides ? k_strides[0] : Hkv * Tk * D, k_strides ? k_strides[1] : Tk * D,
                           k_strides ? k_strides[2] : D};
    const int64_t vs[3] = {v_strides ? v_strides[0] : Hkv * Tk * D, v_strides ? v_strides[1] : Tk * D,
                           v_strides ? v_strides[2] : D};
    OB_REQUIRE(stride_ok(ks[0]) && stride_ok(ks[1]) && stride_ok(ks[2]) && stride_ok(vs[0]) && stride_ok(vs[1]) &&
                   stride_ok(vs[2]),
               OASR_ERR_ALIGN, "fmha: k/v strides must be multiples of 8 elements");
    if (Tk == 0) {
      // no keys at all: every row is empty -> zeros
      cudaError_t e = cudaMemsetAsync(out, 0, (size_t)B * H * Tq * D * 2, static_cast<cudaStream_t>(stream));
      if (e != cudaSuccess) return set_error(OASR_ERR_CUDA, "fmha: memset failed: %s", cudaGetErrorString(e));
      return OASR_OK;
    }
    if (int rc = make_map(&maps.k, dtype, k, (int)D, Tk, Hkv, B, ks[2], ks[1], ks[0], BKV)) return rc;
    if (int rc = make_map(&maps.v, dtype, v, (int)D, Tk, Hkv, B, vs[2], vs[1], vs[0], BKV)) return rc;
    p.mode = kDense;
  }
  maps.k2 = maps.k;
  p.B = (int)B; p.H = (int)H; p.Hkv = (int)Hkv; p.Tq = (int)Tq; p.Tk = (int)Tk;
  p.scale_log2 = static_cast<float>(scale * 1.4426950408889634);
  p.causal = causal; p.seqlens = seqlens; p.seqstarts = seqstarts;
  p.bias = bias; p.bias_sb = bias_stride_b; p.bias_sh = bias_stride_h; p.bias_sq = bias_stride_q;
  p.out = out; p.out_token_major = out_token_major; p.status = device_status_ptr();
  dim3 grid((unsigned)((Tq + BQ - 1) / BQ), (unsigned)H, (unsigned)B);
  return dispatch(maps, p, (int)D, dtype, grid, static_cast<cudaStream_t>(stream));
}

int oasr_b200_fmha(void* out, const void* q, const void* k, const void* v, const int64_t* q_strides,
                   const int64_t* k_strides, const int64_t* v_strides, const void* bias, int64_t bias_stride_b,
                   int64_t bias_stride_h, int64_t bias_stride_q, const int32_t* seqlens, const int32_t* seqstarts,
                   const int32_t* block_table, int64_t blocks_per_seq, int64_t block_size, int64_t num_blocks,
                   int64_t B, int64_t H, int64_t Hkv, int64_t Tq, int64_t Tk, int64_t D, double scale, int causal,
                   int dtype, void* stream) {
  return fmha_dense_or_paged(out, q, k, v, q_strides, k_strides, v_strides, bias, bias_stride_b, bias_stride_h,
                             bias_stride_q, seqlens, seqstarts, block_table, blocks_per_seq, block_size, num_blocks, B, H,
                             Hkv, Tq, Tk, D, scale, causal, dtype, stream, 0);
}

int oasr_b200_fmha_bthd(void* out, const void* q, const void* k, const void* v, const int64_t* q_strides,
                        const int64_t* k_strides, const int64_t* v_strides, const void* bias, int64_t bias_stride_b,
                        int64_t bias_stride_h, int64_t bias_stride_q, const int32_t* seqlens, const int32_t* seqstarts,
                        const int32_t* block_table, int64_t blocks_per_seq, int64_t block_size, int64_t num_blocks,
                        int64_t B, int64_t H, int64_t Hkv, int64_t Tq, int64_t Tk, int64_t D, double scale, int causal,
                        int dtype, void* stream) {
  return fmha_dense_or_paged(out, q, k, v, q_strides, k_strides, v_strides, bias, bias_stride_b, bias_stride_h,
                             bias_stride_q, seqlens, seqstarts, block_table, blocks_per_seq, block_size, num_blocks, B, H,
                             Hkv, Tq, Tk, D, scale, causal, dtype, stream, 1);
}

static int fmha_varlen_impl(void* out, const void* q, const void* k, const void* v, int64_t q_ld, int64_t k_ld,
                           int64_t v_ld, const void* bias, const void* bias_offsets, int bias_offsets_is_i64,
                           int bias_rows_padded8, const int32_t* cu_seqlens_q,
                          const int32_t* cu_seqlens_k, int64_t num_segs, int64_t total_q, int64_t total_k,
                          int64_t max_seqlen_q, int64_t H, int64_t Hkv, int64_t D, double scale, int dtype,
                          void* stream) {
  using namespace ob;
  using namespace ob::fmha;
  OB_REQUIRE(num_segs >= 0 && total_q >= 0 && total_k >= 0 && max_seqlen_q >= 0 && H > 0 && Hkv > 0 && D > 0,
             OASR_ERR_INVALID, "fmha_varlen: bad shape");
  OB_REQUIRE(H % Hkv == 0, OASR_ERR_INVALID, "fmha_varlen: H (%lld) must be divisible by H_kv (%lld)", (long long)H,
             (long long)Hkv);
  if (num_segs == 0 || total_q == 0 || max_seqlen_q == 0) return OASR_OK;
  OB_REQUIRE(out && q && k && v && cu_seqlens_q && cu_seqlens_k, OASR_ERR_INVALID, "fmha_varlen: null pointer argument");
  OB_REQUIRE((bias == nullptr) == (bias_offsets == nullptr), OASR_ERR_INVALID,
             "fmha_varlen: attn_bias and bias_offsets must be provided together");
  OB_REQUIRE(is_aligned(out, 16) && is_aligned(q, 16) && is_aligned(k, 16) && is_aligned(v, 16), OASR_ERR_ALIGN,
             "fmha_varlen: q/k/v/out must be 16-byte aligned");
  OB_REQUIRE(D == 64 || D == 128, OASR_ERR_UNSUPPORTED,
             "fmha_varlen: head_dim %lld is not supported (64 and 128 are)", (long long)D);
  OB_REQUIRE(num_segs <= 65535 && H <= 65535, OASR_ERR_INVALID, "fmha_varlen: segment / head count too large");
  if (q_ld == 0) q_ld = H * D;
  if (k_ld == 0) k_ld = Hkv * D;
  if (v_ld == 0) v_ld = Hkv * D;
  OB_REQUIRE(q_ld >= H * D && k_ld >= Hkv * D && v_ld >= Hkv * D && stride_ok(q_ld) && stride_ok(k_ld) && stride_ok(v_ld),
             OASR_ERR_ALIGN, "fmha_varlen: row strides must cover a row and be multiples of 8 elements");
  Maps maps;
  if (int rc = make_map(&maps.q, dtype, q, (int)D, total_q, H, 1, q_ld, D, q_ld * total_q, BQ)) return rc;
  const int64_t tk = total_k > 0 ? total_k : 1;
  if (int rc = make_map(&maps.k, dtype, k, (int)D, tk, Hkv, 1, k_ld, D, k_ld * tk, BKV)) return rc;
  if (int rc = make_map(&maps.v, dtype, v, (int)D, tk, Hkv, 1, v_ld, D, v_ld * tk, BKV)) return rc;
  maps.q2 = maps.q;
  maps.k2 = maps.k;
  Params p{};
  p.mode = kVarlen; p.B = (int)num_segs; p.H = (int)H; p.Hkv = (int)Hkv; p.Tq = (int)max_seqlen_q; p.Tk = 0;
  p.scale_log2 = static_cast<float>(scale * 1.4426950408889634);
  p.cu_q = cu_seqlens_q; p.cu_k = cu_seqlens_k;
  p.bias = bias; p.bias_offsets = bias_offsets; p.bias_off_i64 = bias_offsets_is_i64;
  p.bias_ld8 = bias_rows_padded8;
  p.out = out; p.status = device_status_ptr();
  dim3 grid((unsigned)((max_seqlen_q + BQ - 1) / BQ), (unsigned)H, (unsigned)num_segs);
  return dispatch(maps, p, (int)D, dtype, grid, static_cast<cudaStream_t>(stream));
}

int oasr_b200_fmha_varlen(void* out, const void* q, const void* k, const void* v, const void* bias,
                          const void* bias_offsets, int bias_offsets_is_i64, const int32_t* cu_seqlens_q,
                          const int32_t* cu_seqlens_k, int64_t num_segs, int64_t total_q, int64_t total_k,
                          int64_t max_seqlen_q, int64_t H, int64_t Hkv, int64_t D, double scale, int dtype,
                          void* stream) {
  return fmha_varlen_impl(out, q, k, v, 0, 0, 0, bias, bias_offsets, bias_offsets_is_i64, 0, cu_seqlens_q, cu_seqlens_k,
                          num_segs, total_q, total_k, max_seqlen_q, H, Hkv, D, scale, dtype, stream);
}

int oasr_b200_fmha_varlen_strided(void* out, const void* q, const void* k, const void* v, int64_t q_row_stride,
                                  int64_t k_row_stride, int64_t v_row_stride, const void* bias,
                                  const void* bias_offsets, int bias_offsets_is_i64, int bias_rows_padded8,
                                  const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, int64_t num_segs,
                                  int64_t total_q, int64_t total_k, int64_t max_seqlen_q, int64_t H, int64_t Hkv,
                                  int64_t D, double scale, int dtype, void* stream) {
  return fmha_varlen_impl(out, q, k, v, q_row_stride, k_row_stride, v_row_stride, bias, bias_offsets,
                          bias_offsets_is_i64, bias_rows_padded8, cu_seqlens_q, cu_seqlens_k, num_segs, total_q, total_k,
                          max_seqlen_q, H, Hkv, D, scale, dtype, stream);
}

}  // extern "C"
