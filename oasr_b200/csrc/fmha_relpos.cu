// Packed relative-position attention (head_dim 64), the form the offline Conformer layer runs:
//   out[i,:] = softmax_j( ((q_i+u).k_j + (q_i+v).p_j) * scale ) . v_j      over the keys j of row i's segment
// (RelPositionMultiHeadedAttention._forward_packed, oasr/layers/attention/attention.py:323-386).
//
// Same tcgen05 / TMEM / TMA pipeline as fmha.cu, sized so that TWO CTAs share an SM: at head_dim 64 a tile's
// tensor work (0.4k clocks for 128 queries x 64 keys) is a fraction of its softmax (2k) and of the latencies around it
// (TMEM loads, MUFU, barrier hand-offs), so one CTA per SM leaves every unit under 20 % busy; a second resident CTA
// fills those gaps.  To fit twice:
//   keys are walked in tiles of 64 (K | pos 16 KB, V 8 KB per stage, two stages),
//   P has a single 16 KB buffer (a softmax thread waits for P.V of tile j-1 before it rewrites P for tile j; by
//   then that short MMA has long finished, because the exponentials of tile j were computed in between),
//   TMEM holds S[2] (2 x 64 columns) and ONE O (64 columns) that every P.V accumulates into = 192 of 256 columns,
// i.e. 96 KB of shared memory and half of TMEM per CTA.
// PERSISTENT: the grid is two CTAs per SM and every CTA walks work items (segment, head, 128-row query tile) number
// blockIdx.x, + gridDim.x, ... of a list that holds the longest segments first (plan_kernel below, built on the device
// once per batch; without a list the items are enumerated in (segment, head, tile) order).  Stages and barriers are
// indexed by the CTA's running key-tile count, so the pipeline carries on from one item into the next: a fresh CTA
// needs 3.5-5k clocks before its first scores arrive, which one CTA per item paid 1,300 times per launch of the
// headline batch (72 -> 55 us per launch).
// 192 threads: warp 4 lane 0 issues the MMAs, warp 5 lane 0 the TMA loads (a stage's refill waits for the MMAs that
// read it; in one thread with the MMA issue those waits made that thread's per-tile path as long as a tile's softmax),
// warps 0-3 own one query row per thread.
// Softmax per tile and row: ONE TMEM load of the 64 scores into registers (S is handed back to the MMA issuer at
// once), running max with a LAZY rescale -- the reference maximum only moves, and O (in TMEM) and the running sum
// are only rescaled, when the tile's maximum exceeds it by more than 2^8, so exponentials stay below 256 and the
// common case costs nothing -- then exp2 (scale / subtract and the row sum as packed fp32x2 operations on tiles
// without masked keys: 1.3k -> 0.8k clocks for the 64 exponentials of a thread; optionally a share of them as a
// degree-3 polynomial on the FMA pipe, off by default: measured slower), bf16/fp16 P into swizzled shared memory.
// O leaves TMEM once per item, scaled by 1 / sum; the next item's first P.V waits until every row has read it.
// K | pos of tile j+2 is requested as soon as Q.K^T of tile j has finished, V of tile j+2 when P.V of tile j has: the
// two have separate stage barriers.
// Only the length mask exists here (keys >= segment length); bias, causal masks, key starts, paged K/V and
// head_dim 128 stay on the general kernel in fmha.cu.  Every wait is bounded.
#include <cuda.h>

#include <type_traits>

#include "common.cuh"
#include "device_status.cuh"
#include "sm100_ptx.cuh"
#include "tma_host.cuh"

namespace ob {
int g_fmha_relpos_path = 1;   // 1 = this kernel for the packed relative-position form; 0 = the general kernel ("fmha_relpos_path")
int g_fmha_poly = 0;          // exponentials per four on the FMA pipe in this kernel ("fmha_poly": 0, 1, 2); measured on B200
                              // (config-2 batch): 66.0 / 66.9 / 68.9 us per launch for 0 / 1 / 2 -- the softmax is bound by
                              // instruction issue, not by the MUFU unit, so the extra FMA work does not pay

namespace fmha_relpos {

constexpr int BQ = 128, BKV = 64, D = 64;
constexpr int kThreads = 192;   // 4 softmax warps, the MMA issuer's warp, the TMA producer's warp
constexpr int kQBytes = 2 * 128 * 128;          // [q+u | q+v]: two atoms of 128 rows x 128 B
constexpr int kKBytes = 2 * BKV * 128;          // [k | pos] per stage
constexpr int kVBytes = BKV * 128;
constexpr int kPBytes = BQ * 128;               // 128 rows x 64 keys
constexpr int kOffQ = 0, kOffK = kOffQ + kQBytes, kOffV = kOffK + 2 * kKBytes, kOffP = kOffV + 2 * kVBytes;
constexpr int kOffBar = kOffP + kPBytes;
constexpr int kNumBars = 16;
constexpr int kSmemDynamic = kOffBar + kNumBars * 8 + 16 + 1024;
constexpr uint32_t kTmemCols = 256, kColS = 0, kColO = 128;
constexpr float kLazyLog2 = 8.f;   // rescale only when the row maximum grows by more than 2^8

struct Params {
  int H;
  float scale_log2;
  const int32_t* cu;
  void* out;
  uint32_t* status;
  const int2* items;           // nullable: work items (segment, head << 16 | query tile), longest segments first
  const int32_t* n_items;      // device count of `items`
  int natural_items;           // items == null: num_segs * H * qtiles, item i = (segment, head, query tile) in that order
  int qtiles;                  // query tiles of the longest segment
  unsigned long long* trace;   // nullable diagnostics buffer: the CTA (0, 0, trace_seg) stamps its phases
  int trace_seg;
};
__device__ __forceinline__ void stamp(const Params& p, int slot) {
  if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && static_cast<int>(blockIdx.z) == p.trace_seg)
    p.trace[slot] = static_cast<unsigned long long>(clock64());
}

__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 2^x on the FMA / ALU pipes: round x to the nearest integer n with the 1.5 * 2^23 trick, 2^(x - n) by a cubic on
// [-0.5, 0.5] (relative error 6e-4, below the rounding of a 16-bit P), n added to the exponent field.
__device__ __forceinline__ float ex2_poly(float x) {
  x = fmaxf(x, -125.f);
  const float magic = 12582912.f;                      // 0x4B400000
  const float xr = x + magic;
  const int n = __float_as_int(xr) - 0x4B400000;
  const float f = x - (xr - magic);
  const float pl = fmaf(fmaf(fmaf(0.0555041f, f, 0.2402265f), f, 0.6931472f), f, 1.0f);
  return __int_as_float(__float_as_int(pl) + (n << 23));
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

// kPoly: how many of every four exponentials run as a polynomial on the FMA pipe instead of the MUFU unit (0, 1 or 2)
template <typename T, int kPoly>
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
  if (threadIdx.x == 0) stamp(p, 0);
  if (p.trace != nullptr && threadIdx.x == 0) p.trace[64 + blockIdx.x * 4] = static_cast<unsigned long long>(clock64());
  // Persistent CTA: walks work items blockIdx.x, + gridDim.x, ... of the list (or of the natural enumeration).  All
  // roles decode the same items in the same order; an item whose query tile lies past its segment is skipped by all.
  const int n_items = p.items ? *p.n_items : p.natural_items;
  const int64_t out_ld = static_cast<int64_t>(p.H) * D;
  struct Item { int h, q0, row0, kv_len, nkv; };
  auto decode = [&](int it, Item& w) -> bool {
    int seg, qt;
    if (p.items) {
      const int2 v = p.items[it];
      seg = v.x; w.h = v.y >> 16; qt = v.y & 0xffff;
    } else {
      qt = it % p.qtiles;
      const int rest = it / p.qtiles;
      w.h = rest % p.H;
      seg = rest / p.H;
    }
    w.row0 = p.cu[seg];
    w.kv_len = p.cu[seg + 1] - w.row0;
    w.q0 = qt * BQ;
    w.nkv = (w.kv_len + BKV - 1) / BKV;
    return w.q0 < w.kv_len;
  };

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + kOffQ;
  uint8_t* sK = smem + kOffK;
  uint8_t* sV = smem + kOffV;
  uint8_t* sP = smem + kOffP;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBar);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;     // [2]  K | pos stage landed
  uint64_t* k_empty = bars + 3;    // [2]  Q.K^T of the stage's tile finished: the stage may be refilled (long before its V)
  uint64_t* s_full = bars + 5;     // [2]
  uint64_t* s_free = bars + 7;     // [2]
  uint64_t* p_full = bars + 9;     // [1]
  uint64_t* po_done = bars + 10;   // P.V of a tile has been accumulated into O: O is stable and P may be rewritten
  uint64_t* v_full = bars + 11;    // [2]  V stage landed
  uint64_t* v_empty = bars + 13;   // [2]  P.V of the stage's tile finished
  uint64_t* o_free = bars + 15;    // every softmax thread has read the item's O: the next item's first P.V may overwrite it
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    ptx::mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&k_full[i], 1);
      ptx::mbar_init(&k_empty[i], 1);
      ptx::mbar_init(&v_full[i], 1);
      ptx::mbar_init(&v_empty[i], 1);
      ptx::mbar_init(&s_full[i], 1);
      ptx::mbar_init(&s_free[i], BQ);
    }
    ptx::mbar_init(po_done, 1);
    ptx::mbar_init(p_full, BQ);
    ptx::mbar_init(o_free, BQ);
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
  if (threadIdx.x == 0) stamp(p, 1);

  // Every barrier that completes once per key tile is indexed by the CTA's running tile count g (stage g & 1, phase
  // g >> 1), which carries on from one item to the next, so the pipeline never drains between items.
  if (warp == 5) {
    // =================== TMA producer (one thread) ===================
    // Its own warp: the refill of a stage waits for the MMAs that read it, and those waits must not sit in the MMA
    // issuer's instruction stream (with both roles in one thread that thread's per-tile path, about 2k clocks of
    // serial waits and issues, was as long as the softmax of a tile and set the pace).
    if (lane == 0) {
      bool ok = true;
      int g = 0, done = 0;
      for (int it = blockIdx.x; ok && it < n_items; it += gridDim.x) {
        Item w;
        if (!decode(it, w)) continue;
        if (done > 0) {   // Q is single-buffered: the previous item's last Q.K^T (tile g-1) has finished
          if (!ptx::mbar_wait(&k_empty[(g - 1) & 1], ((g - 1) >> 1) & 1u, abort_flag)) { ok = false; break; }
        }
        ptx::mbar_expect_tx(q_full, kQBytes);
        ptx::tma_load_4d(sQ, &map_q, 0, w.row0 + w.q0, w.h, 0, q_full);
        ptx::tma_load_4d(sQ + 128 * 128, &map_q2, 0, w.row0 + w.q0, w.h, 0, q_full);
        for (int t = 0; ok && t < w.nkv; ++t) {
          const int gg = g + t, b = gg & 1;
          const int key0 = t * BKV;
          const uint32_t prev = ((gg - 2) >> 1) & 1u;         // phase of tile gg - 2, the stage's last user
          if (gg >= 2 && !ptx::mbar_wait(&k_empty[b], prev, abort_flag)) { ok = false; break; }   // its Q.K^T finished
          ptx::mbar_expect_tx(&k_full[b], kKBytes);
          uint8_t* dk = sK + b * kKBytes;
          ptx::tma_load_4d(dk, &map_k, 0, w.row0 + key0, w.h, 0, &k_full[b]);
          ptx::tma_load_4d(dk + BKV * 128, &map_pos, 0, key0, w.h, 0, &k_full[b]);
          if (gg >= 2 && !ptx::mbar_wait(&v_empty[b], prev, abort_flag)) { ok = false; break; }   // its P.V finished
          ptx::mbar_expect_tx(&v_full[b], kVBytes);
          ptx::tma_load_4d(sV + b * kVBytes, &map_v, 0, w.row0 + key0, w.h, 0, &v_full[b]);
        }
        g += w.nkv;
        ++done;
      }
      if (!ok && p.status) atomicOr(p.status, kStatusFmhaMma);
    }
    __syncwarp();
  } else if (warp == 4) {
    // =================== MMA issuer (one thread) ===================
    if (lane == 0) {
      bool ok = true;
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
        ptx::umma_commit(&k_empty[b]);
      };
      auto issue_pv = [&](int b, bool first) {   // O (+)= P . V_b : K = 64 keys in four steps of 16
        const uint32_t a_addr = ptx::smem_u32(sP);
        const uint32_t b_addr = ptx::smem_u32(sV + b * kVBytes);
        const uint32_t d_tmem = tmem_base + kColO;
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          const uint64_t adesc = ptx::smem_desc_kmajor_sw128(a_addr + kk * 32);
          const uint64_t bdesc = ptx::smem_desc_mnmajor_sw128(b_addr + kk * 2048, BKV * 128, 1024);
          ptx::umma_f16(d_tmem, adesc, bdesc, kIdescPV, (!first || kk != 0) ? 1u : 0u);
        }
        ptx::umma_commit(po_done);
        ptx::umma_commit(&v_empty[b]);
      };
      // scores of tile gg: its K | pos stage has landed and S[gg & 1] has been read by the softmax of tile gg - 2
      auto scores = [&](int gg) -> bool {
        const int b = gg & 1;
        const uint32_t ph = (gg >> 1) & 1u;
        if (!ptx::mbar_wait(&k_full[b], ph, abort_flag) || !ptx::mbar_wait(&s_free[b], ph ^ 1u, abort_flag)) return false;
        ptx::tc_fence_after_sync();
        issue_qk(b);
        return true;
      };
      // next item of this CTA at or after `it` whose query tile exists (n_items if none)
      auto next_item = [&](int it, Item& w) {
        while (it < n_items && !decode(it, w)) it += gridDim.x;
        return it;
      };
      int g = 0, done = 0;
      Item w, w2;
      int it = next_item(blockIdx.x, w);
      bool first_issued = false;               // the item's first scores were already issued under the previous item
      while (ok && it < n_items) {
        if (!first_issued) ok = ptx::mbar_wait(q_full, static_cast<uint32_t>(done) & 1u, abort_flag) && scores(g);
        first_issued = false;
        const int it2 = next_item(it + gridDim.x, w2);
        // Tile j: the scores of tile j+1 are issued first -- at the item's last tile those of the NEXT item's first
        // tile (its Q was loaded when this item's last Q.K^T finished), so that they are ready when the softmax
        // threads come out of this item's output -- then P.V of tile j, which waits for the softmax.
        for (int j = 0; ok && j < w.nkv; ++j) {
          const int gg = g + j, b = gg & 1;
          if (j + 1 < w.nkv) {
            if (!scores(gg + 1)) { ok = false; break; }
          } else if (it2 < n_items) {
            if (!ptx::mbar_wait(q_full, static_cast<uint32_t>(done + 1) & 1u, abort_flag) || !scores(gg + 1)) { ok = false; break; }
            first_issued = true;
          }
          ok = ptx::mbar_wait(p_full, static_cast<uint32_t>(gg) & 1u, abort_flag) &&
               ptx::mbar_wait(&v_full[b], (gg >> 1) & 1u, abort_flag);
          if (ok && j == 0 && done > 0) ok = ptx::mbar_wait(o_free, static_cast<uint32_t>(done - 1) & 1u, abort_flag);
          if (!ok) break;
          ptx::tc_fence_after_sync();
          issue_pv(b, j == 0);
        }
        g += w.nkv;
        ++done;
        it = it2;
        w = w2;
      }
      if (!ok && p.status) atomicOr(p.status, kStatusFmhaMma);
    }
    __syncwarp();
  } else {
    // =========================== softmax / output (thread = row) ===========================
    const int r = threadIdx.x;  // 0..127
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const uint32_t t_o = tmem_base + lane_base + kColO;
    bool ok = true;
    int g = 0;
    for (int it = blockIdx.x; ok && it < n_items; it += gridDim.x) {
    Item w;
    if (!decode(it, w)) continue;
    const int kv_len = w.kv_len, nkv = w.nkv;
    const bool row_ok = r < min(BQ, kv_len - w.q0);
    T* out = static_cast<T*>(p.out) + (static_cast<int64_t>(w.row0 + w.q0) * p.H + w.h) * D;
    float m_run = kNegInf, l_run = 0.f;   // m_run: the reference maximum the exponentials, l_run and O are relative to
    for (int j = 0; ok && j < nkv; ++j) {
      const int gg = g + j, b = gg & 1;
      const int key0 = j * BKV;
      if (!ptx::mbar_wait(&s_full[b], (gg >> 1) & 1u, abort_flag)) { ok = false; break; }
      ptx::tc_fence_after_sync();
      if (j == 0 && r == 0) stamp(p, 2);
      if (j == 3 && r == 0) stamp(p, 50);
      uint32_t v[64];
      ptx::tmem_ld_32x64(tmem_base + lane_base + kColS + b * BKV, v);
      ptx::tmem_ld_wait();
      if (j == 3 && r == 0) stamp(p, 51);
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(&s_free[b]);          // the scores live in registers now: S[b] may take tile j+2
      const bool full = key0 + BKV <= kv_len;   // tiles inside the valid keys need no mask
      if (!full) {   // the segment's last tile: keys past its end become -inf scores, i.e. P = exp2(-inf) = 0 below
#pragma unroll
        for (int i = 0; i < 64; ++i) v[i] = key0 + i < kv_len ? v[i] : 0xff800000u;
      }
      float mx[4] = {kNegInf, kNegInf, kNegInf, kNegInf};   // four independent chains
#pragma unroll
      for (int i = 0; i < 64; ++i) mx[i & 3] = fmaxf(mx[i & 3], __uint_as_float(v[i]));
      float tile_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      tile_max *= p.scale_log2;   // the scale is positive
      if (j == 3 && r == 0) stamp(p, 52);
      // Lazy rescale: the reference maximum moves only when this tile exceeds it by more than 2^kLazyLog2.
      float rescale = 1.f;
      bool moved = false;
      if (m_run == kNegInf) {
        m_run = (tile_max == kNegInf) ? 0.f : tile_max;      // first tile (empty-row clamp: no valid key -> 0)
      } else if (tile_max > m_run + kLazyLog2) {
        rescale = ex2_fast(m_run - tile_max);
        m_run = tile_max;
        moved = true;
      }
      // exponentiate, sum, round
      uint32_t packed[32];
      float row_sum = 0.f;
      if (kPoly == 0) {
        // every exponential on the MUFU unit: scale / subtract and the row sum as packed fp32x2 operations (masked
        // keys carry -inf and come out as exactly 0)
        const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
        const float2 nm2 = make_float2(-m_run, -m_run);
        float2 acc[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
        for (int i = 0; i < 64; i += 2) {
          const float2 x = __ffma2_rn(make_float2(__uint_as_float(v[i]), __uint_as_float(v[i + 1])), sc2, nm2);
          const float2 e = make_float2(ex2_fast(x.x), ex2_fast(x.y));
          acc[(i >> 1) & 1] = __fadd2_rn(acc[(i >> 1) & 1], e);
          packed[i / 2] = pack2<T>(e.x, e.y);
        }
        const float2 a = __fadd2_rn(acc[0], acc[1]);
        row_sum = a.x + a.y;
      } else {
        // keys 4k+3 (and 4k+1) of every group of four optionally on the FMA pipe; keys past the end give P = 0
#pragma unroll
        for (int i = 0; i < 64; i += 4) {
          float e0 = ex2_fast(fmaf(__uint_as_float(v[i]), p.scale_log2, -m_run));
          const float x1 = fmaf(__uint_as_float(v[i + 1]), p.scale_log2, -m_run);
          const float x3 = fmaf(__uint_as_float(v[i + 3]), p.scale_log2, -m_run);
          float e1 = kPoly >= 2 ? ex2_poly(x1) : ex2_fast(x1);
          float e2 = ex2_fast(fmaf(__uint_as_float(v[i + 2]), p.scale_log2, -m_run));
          float e3 = kPoly >= 1 ? ex2_poly(x3) : ex2_fast(x3);
          if (!full) {   // P of keys past the end is zero (V rows there hold other segments' finite values)
            e0 = key0 + i < kv_len ? e0 : 0.f;
            e1 = key0 + i + 1 < kv_len ? e1 : 0.f;
            e2 = key0 + i + 2 < kv_len ? e2 : 0.f;
            e3 = key0 + i + 3 < kv_len ? e3 : 0.f;
          }
          row_sum += (e0 + e1) + (e2 + e3);
          packed[i / 2] = pack2<T>(e0, e1);
          packed[i / 2 + 1] = pack2<T>(e2, e3);
        }
      }
      if (j == 3 && r == 0) stamp(p, 53);
      // P.V of tile j-1 has finished: P may be rewritten and O is stable (it is only touched here when the maximum moved)
      if (j >= 1) {
        if (!ptx::mbar_wait(po_done, static_cast<uint32_t>(gg - 1) & 1u, abort_flag)) { ok = false; break; }
        if (moved) {
          ptx::tc_fence_after_sync();
          uint32_t o[64];
          ptx::tmem_ld_32x64(t_o, o);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 64; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * rescale);
          ptx::tmem_st_32x32(t_o, reinterpret_cast<const uint32_t(&)[32]>(o[0]));
          ptx::tmem_st_32x32(t_o + 32, reinterpret_cast<const uint32_t(&)[32]>(o[32]));
          ptx::tmem_st_wait();
          ptx::tc_fence_before_sync();
        }
      }
      if (j == 3 && r == 0) stamp(p, 54);
      l_run = l_run * rescale + row_sum;
      // row r of P, K-major with the 128-byte swizzle: 16-byte chunk c (8 keys) sits at c ^ (r % 8)
      uint8_t* row_base = sP + r * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        *reinterpret_cast<uint4*>(row_base + ((c ^ (r & 7)) << 4)) =
            make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
      }
      if (j == 3 && r == 0) stamp(p, 55);
      ptx::fence_proxy_async_smem();
      ptx::mbar_arrive(p_full);
      if (r == 0 && j < 40) stamp(p, 3 + j);
    }
    if (ok) ok = ptx::mbar_wait(po_done, static_cast<uint32_t>(g + nkv - 1) & 1u, abort_flag);
    if (ok) {
      ptx::tc_fence_after_sync();
      uint32_t o[64];
      ptx::tmem_ld_32x64(t_o, o);
      ptx::tmem_ld_wait();
      if (row_ok) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        T* orow = out + static_cast<int64_t>(r) * out_ld;
#pragma unroll
        for (int c = 0; c < D; c += 8) {
          uint4 w;
          w.x = pack2<T>(__uint_as_float(o[c]) * inv, __uint_as_float(o[c + 1]) * inv);
          w.y = pack2<T>(__uint_as_float(o[c + 2]) * inv, __uint_as_float(o[c + 3]) * inv);
          w.z = pack2<T>(__uint_as_float(o[c + 4]) * inv, __uint_as_float(o[c + 5]) * inv);
          w.w = pack2<T>(__uint_as_float(o[c + 6]) * inv, __uint_as_float(o[c + 7]) * inv);
          *reinterpret_cast<uint4*>(orow + c) = w;
        }
      }
      if (r == 0) stamp(p, 60);
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(o_free);             // O is in registers: the next item's first P.V may overwrite it
    }
    g += nkv;
    }   // items
    if (p.trace != nullptr && r == 0) {   // diagnostics: this CTA's span and work
      p.trace[64 + blockIdx.x * 4 + 1] = static_cast<unsigned long long>(clock64());
      p.trace[64 + blockIdx.x * 4 + 2] = static_cast<unsigned long long>(g);
      unsigned smid;
      asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
      p.trace[64 + blockIdx.x * 4 + 3] = smid;
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
        int64_t num_segs, int64_t max_seqlen, int64_t total, int64_t H, double scale, int dtype, const int2* items,
        const int32_t* n_items, cudaStream_t stream) {
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
  p.trace = g_trace_buffer; p.trace_seg = 0;
  p.items = items; p.n_items = n_items;
  p.qtiles = static_cast<int>((max_seqlen + BQ - 1) / BQ);
  const int64_t natural = num_segs * H * p.qtiles;
  OB_REQUIRE(natural < (int64_t(1) << 31), OASR_ERR_INVALID, "fmha_varlen_relpos: too many work items");
  p.natural_items = static_cast<int>(natural);
  int64_t ctas = 2 * static_cast<int64_t>(sm_count());     // two resident CTAs per SM, each walking the item list
  if (natural < ctas) ctas = natural;
  dim3 grid(static_cast<unsigned>(ctas));
  auto launch_one = [&](auto kern) -> int {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemDynamic);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    if (e != cudaSuccess)
      return set_error(OASR_ERR_CUDA, "fmha_varlen_relpos: cannot reserve %d bytes of shared memory: %s", kSmemDynamic,
                       cudaGetErrorString(e));
    launch_pdl(kern, grid, dim3(kThreads), kSmemDynamic, stream, mq, mq2, mk, mp, mv, p);
    return check_launch("fmha_varlen_relpos (two CTAs per SM) launch");
  };
  return OB_DISPATCH_HALF(dtype, T, [&]() -> int {
    if (g_fmha_poly <= 0) return launch_one(fmha_relpos64_kernel<T, 0>);
    if (g_fmha_poly == 1) return launch_one(fmha_relpos64_kernel<T, 1>);
    return launch_one(fmha_relpos64_kernel<T, 2>);
  });
}


// Work list for the persistent kernel: items (segment, head, query tile) with the longest segments first, so that the
// CTAs that pick up the last items pick up short ones (a tile's cost is proportional to its segment's length).  One
// block; segments are ranked by counting (num_segs <= 1024), the items of rank r start at the prefix sum of the
// ranks before it.  plan = [int32 n_items, pad to 16 bytes][int2 items...].
constexpr int kPlanMaxSegs = 1024;
__global__ void __launch_bounds__(kPlanMaxSegs) plan_kernel(int32_t* plan, const int32_t* __restrict__ cu, int S, int H) {
  __shared__ int len[kPlanMaxSegs];
  __shared__ int seg_of_rank[kPlanMaxSegs];
  __shared__ int start[kPlanMaxSegs + 1];
  const int t = threadIdx.x;
  if (t < S) len[t] = cu[t + 1] - cu[t];
  __syncthreads();
  if (t < S) {
    int rank = 0;
    const int mine = len[t];
    for (int k = 0; k < S; ++k) rank += (len[k] > mine || (len[k] == mine && k < t)) ? 1 : 0;
    seg_of_rank[rank] = t;
  }
  __syncthreads();
  // inclusive scan of the items per rank (Hillis-Steele over S <= 1024 entries)
  int mine_items = 0;
  if (t < S) mine_items = ((len[seg_of_rank[t]] + BQ - 1) / BQ) * H;
  start[t + 1 <= kPlanMaxSegs ? t + 1 : kPlanMaxSegs] = 0;
  __syncthreads();
  if (t < S) start[t + 1] = mine_items;
  if (t == 0) start[0] = 0;
  __syncthreads();
  for (int d = 1; d < S; d <<= 1) {
    int add = 0;
    if (t < S && t + 1 - d >= 1) add = start[t + 1 - d];
    __syncthreads();
    if (t < S) start[t + 1] += add;
    __syncthreads();
  }
  if (t == 0) plan[0] = start[S];
  if (t < S) {
    const int seg = seg_of_rank[t];
    const int qt_n = (len[seg] + BQ - 1) / BQ;
    int2* items = reinterpret_cast<int2*>(plan + 4) + start[t];
    for (int qt = 0; qt < qt_n; ++qt)
      for (int h = 0; h < H; ++h) items[qt * H + h] = make_int2(seg, (h << 16) | qt);
  }
}

// every segment contributes H * ceil(len / 128) items: at most H * (total / 128 + num_segs) over all segments
int64_t plan_bytes(int64_t num_segs, int64_t H, int64_t total) { return 16 + 8 * H * (total / BQ + num_segs); }

int plan(void* plan_buf, const int32_t* cu_seqlens, int64_t num_segs, int64_t H, cudaStream_t stream) {
  plan_kernel<<<1, kPlanMaxSegs, 0, stream>>>(static_cast<int32_t*>(plan_buf), cu_seqlens, static_cast<int>(num_segs),
                                              static_cast<int>(H));
  return check_launch("fmha_relpos_plan launch");
}

}  // namespace fmha_relpos
}  // namespace ob
