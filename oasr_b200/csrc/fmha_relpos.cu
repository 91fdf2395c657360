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
//   TMEM holds S[2] (2 x 64 columns) and ONE O (64 columns + 16 that hold the row sum of P, see kIdescPV) that every
//   P.V accumulates into = 208 of 256 columns,
// i.e. 104 KB of shared memory (8 KB of it a constant block of ones) and half of TMEM per CTA.
// PERSISTENT: the grid is two CTAs per SM and every CTA walks work items (segment, head, 128-row query tile) of a
// list that holds the longest segments first (plan_kernel below, built on the device once per batch; without a list the
// items are enumerated in (segment, head, tile) order), dealt in rounds of gridDim.x items, forwards and backwards in
// turn.  Stages and barriers are indexed by the CTA's running key-tile count, so the pipeline carries on from one item
// into the next: a fresh CTA needs 3.5-5k clocks before its first scores arrive, which one CTA per item paid 1,300
// times per launch of the headline batch (72 -> 55 us per launch).
// 192 threads: warp 4 lane 0 issues the MMAs, warp 5 lane 0 the TMA loads, warps 0-3 own one query row per thread.
// The two single-thread roles are event loops over two cursors each (K | pos and V refills; scores and P.V): whichever
// operation has its inputs ready is issued, so scores run up to two tiles ahead of P.V, into the next item too, and
// an item's output is written by the softmax threads inside the next item's first tile, while that item's last P.V
// drains (55 -> 50 us); with the alternating deal (20-28 -> 22-26 key tiles per CTA) 45 us per launch, 44 us without the
// per-tile diagnostic stamps the softmax loop used to carry.
// Softmax per tile and row: ONE TMEM load of the 64 scores into registers (S is handed back to the MMA issuer at
// once), running max with a LAZY rescale -- the reference maximum only moves, and O (in TMEM) and the running sum
// are only rescaled, when the tile's maximum exceeds it by more than 2^8, so exponentials stay below 256 and the
// common case costs nothing -- then exp2 (scale / subtract as packed fp32x2 operations: 1.3k -> 0.8k clocks for the 64
// exponentials of a thread; the row sum is taken by the tensor core: P.V runs with N = 80 against [V | ones],
// 43.9 -> 43.3 us per launch; a share of the exponentials as a cubic on the FMA pipe measured slower: 45.4 / 56.2 /
// 60.3 us per launch with none / one / two of every four), bf16/fp16 P into swizzled shared memory.
// O leaves TMEM once per item, scaled by 1 / sum; the next item's first P.V waits until every row has read it.
// K | pos of tile j+2 is requested as soon as Q.K^T of tile j has finished, V of tile j+2 when P.V of tile j has: the
// two have separate stage barriers and separate cursors.
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

namespace fmha_relpos {

constexpr int BQ = 128, BKV = 64, D = 64;
constexpr int kThreads = 192;   // 4 softmax warps, the MMA issuer's warp, the TMA producer's warp
constexpr int kQBytes = 2 * 128 * 128;          // [q+u | q+v]: two atoms of 128 rows x 128 B
constexpr int kKBytes = 2 * BKV * 128;          // [k | pos] per stage
constexpr int kVBytes = BKV * 128;
constexpr int kPBytes = BQ * 128;               // 128 rows x 64 keys
constexpr int kOnesBytes = BKV * 128;           // a V-shaped block of ones: the P.V instruction's second block of 64 columns
constexpr int kOffQ = 0, kOffK = kOffQ + kQBytes, kOffV = kOffK + 2 * kKBytes, kOffP = kOffV + 2 * kVBytes;
constexpr int kOffOnes = kOffP + kPBytes;
constexpr int kOffBar = kOffOnes + kOnesBytes;
constexpr int kNumBars = 16;
constexpr int kSmemDynamic = kOffBar + kNumBars * 8 + 16 + 1024;
constexpr uint32_t kTmemCols = 256, kColS = 0, kColO = 128, kColSum = kColO + D;   // O | 16 columns that each hold the row sum of P
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
  unsigned long long* trace;   // nullable diagnostics buffer: CTA 0 stamps its start, every CTA its span, tile count and SM
  int trace_seg;
};
__device__ __forceinline__ void stamp(const Params& p, int slot) {
  if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && static_cast<int>(blockIdx.z) == p.trace_seg)
    p.trace[slot] = static_cast<unsigned long long>(clock64());
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
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
  // P.V with N = D + 16: columns D.. of the B operand come from a constant block of ones (the MN-major descriptor's
  // distance between 64-column blocks points there), so the accumulator's columns D..D+15 each receive the row sum of
  // the 16-bit P -- the sum the output is divided by leaves the tensor core with O instead of costing every softmax
  // thread an add per pair of keys.
  constexpr uint32_t kIdescPV = ptx::umma_idesc_f16(kBf16, BQ, D + 16, false, true);  // V is MN-major
  constexpr float kNegInf = -INFINITY;

  ptx::grid_dep_launch();   // no-ops unless launched with programmatic stream serialisation
  ptx::grid_dep_wait();
  if (threadIdx.x == 0) stamp(p, 0);
  if (p.trace != nullptr && threadIdx.x == 0) p.trace[64 + blockIdx.x * 4] = static_cast<unsigned long long>(clock64());
  // Persistent CTA: the items of the list (or of the natural enumeration) are dealt to the CTAs in rounds of gridDim.x,
  // forwards in even rounds and backwards in odd ones: the list holds the longest items first, so plain round-robin
  // would hand CTA 0 the longest item of every round (20 to 28 key tiles per CTA on the headline batch).  All roles
  // decode the same items in the same order; an item whose query tile lies past its segment is skipped by all.
  const int n_items = p.items ? *p.n_items : p.natural_items;
  auto item_of_round = [&](int round) -> int {
    const int G = static_cast<int>(gridDim.x), bid = static_cast<int>(blockIdx.x);
    const long long it = static_cast<long long>(round) * G + ((round & 1) ? G - 1 - bid : bid);
    return it < n_items ? static_cast<int>(it) : n_items;
  };
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
  uint8_t* sOnes = smem + kOffOnes;
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
  {
    const uint32_t one2 = kBf16 ? 0x3F803F80u : 0x3C003C00u;      // 1.0 | 1.0 in T
    for (int i = threadIdx.x; i < kOnesBytes / 16; i += kThreads)
      reinterpret_cast<uint4*>(sOnes)[i] = make_uint4(one2, one2, one2, one2);
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
  // The TMA producer and the MMA issuer each follow TWO cursors over the CTA's tile sequence and issue whichever of
  // their two next operations has its inputs ready (non-blocking barrier tests in a bounded polling loop):
  // a refill of K | pos never queues behind a V refill that waits for a later P.V, and P.V of a tile never queues
  // behind scores whose keys are still in flight.
  struct Cursor { int round, it, j, g, ord; Item w; };   // dealing round, item, key tile within it, running tile count, item ordinal of this CTA
  auto seek = [&](Cursor& c) {   // from c.round on: the CTA's next item whose query tile exists (c.it = n_items if none)
    Item w2;
    for (;; ++c.round) {
      c.it = item_of_round(c.round);
      if (c.it >= n_items) { c.it = n_items; return; }
      if (decode(c.it, w2)) { c.w = w2; return; }
    }
  };
  auto start = [&](Cursor& c) { c.j = 0; c.g = 0; c.ord = 0; c.round = 0; seek(c); };
  auto advance = [&](Cursor& c) {
    ++c.g;
    if (++c.j == c.w.nkv) {
      c.j = 0;
      ++c.ord;
      ++c.round;
      seek(c);
    }
  };
  constexpr uint32_t kIdleLimit = 1u << 24;   // polls without progress before the role gives up (a sleep between polls
                                              // measured slower: 45.4 / 46.0 / 46.3 / 46.7 us per launch for 0 / 20 / 40 / 100 ns)
  if (warp == 5) {
    // =================== TMA producer (one thread) ===================
    if (lane == 0) {
      bool ok = true;
      Cursor ck, cv;
      start(ck);
      start(cv);
      uint32_t idle = 0;
      while (ok && (ck.it < n_items || cv.it < n_items)) {   // either cursor may finish first
        bool progress = false;
        if (ck.it < n_items) {
          const int gg = ck.g, b = gg & 1;
          // the stage's last user was Q.K^T of tile gg - 2; Q is single-buffered: a new item's Q waits for the
          // previous item's last Q.K^T (tile gg - 1)
          bool ready = gg < 2 || ptx::mbar_test(&k_empty[b], ((gg - 2) >> 1) & 1u);
          if (ready && ck.j == 0 && ck.ord > 0) ready = ptx::mbar_test(&k_empty[(gg - 1) & 1], ((gg - 1) >> 1) & 1u);
          if (ready) {
            const Item& w = ck.w;
            if (ck.j == 0) {
              ptx::mbar_expect_tx(q_full, kQBytes);
              ptx::tma_load_4d(sQ, &map_q, 0, w.row0 + w.q0, w.h, 0, q_full);
              ptx::tma_load_4d(sQ + 128 * 128, &map_q2, 0, w.row0 + w.q0, w.h, 0, q_full);
            }
            const int key0 = ck.j * BKV;
            ptx::mbar_expect_tx(&k_full[b], kKBytes);
            uint8_t* dk = sK + b * kKBytes;
            ptx::tma_load_4d(dk, &map_k, 0, w.row0 + key0, w.h, 0, &k_full[b]);
            ptx::tma_load_4d(dk + BKV * 128, &map_pos, 0, key0, w.h, 0, &k_full[b]);
            advance(ck);
            progress = true;
          }
        }
        if (cv.it < n_items) {
          const int gg = cv.g, b = gg & 1;
          if (gg < 2 || ptx::mbar_test(&v_empty[b], ((gg - 2) >> 1) & 1u)) {   // P.V of tile gg - 2 finished
            ptx::mbar_expect_tx(&v_full[b], kVBytes);
            ptx::tma_load_4d(sV + b * kVBytes, &map_v, 0, cv.w.row0 + cv.j * BKV, cv.w.h, 0, &v_full[b]);
            advance(cv);
            progress = true;
          }
        }
        if (progress) {
          idle = 0;
        } else {
          if (++idle >= kIdleLimit) { *abort_flag = 1u; ok = false; }
          else if ((idle & 63u) == 63u && *abort_flag) ok = false;
        }
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
          const uint64_t bdesc = ptx::smem_desc_mnmajor_sw128(b_addr + kk * 2048, ptx::smem_u32(sOnes) - b_addr, 1024);
          ptx::umma_f16(d_tmem, adesc, bdesc, kIdescPV, (!first || kk != 0) ? 1u : 0u);
        }
        ptx::umma_commit(po_done);
        ptx::umma_commit(&v_empty[b]);
      };
      Cursor cq, cp;   // next scores, next P.V
      start(cq);
      start(cp);
      uint32_t idle = 0;
      while (ok && cp.it < n_items) {
        bool progress = false;
        if (cq.it < n_items) {
          // scores of tile g: its K | pos stage has landed, S[g & 1] has been read by the softmax of tile g - 2, and
          // (first tile of an item) the item's Q has landed.  They run ahead of P.V by up to two tiles, into the
          // next item too: its Q was requested when this item's last Q.K^T finished.
          const int b = cq.g & 1;
          const uint32_t ph = (cq.g >> 1) & 1u;
          if (ptx::mbar_test(&k_full[b], ph) && ptx::mbar_test(&s_free[b], ph ^ 1u) &&
              (cq.j != 0 || ptx::mbar_test(q_full, static_cast<uint32_t>(cq.ord) & 1u))) {
            ptx::tc_fence_after_sync();
            issue_qk(b);
            advance(cq);
            progress = true;
          }
        }
        if (cp.g < cq.g) {
          // P.V of tile g: P written, V landed, and (first tile of an item) every row has read the previous item's O
          const int b = cp.g & 1;
          if (ptx::mbar_test(p_full, static_cast<uint32_t>(cp.g) & 1u) && ptx::mbar_test(&v_full[b], (cp.g >> 1) & 1u) &&
              (cp.j != 0 || cp.ord == 0 || ptx::mbar_test(o_free, static_cast<uint32_t>(cp.ord - 1) & 1u))) {
            ptx::tc_fence_after_sync();
            issue_pv(b, cp.j == 0);
            advance(cp);
            progress = true;
          }
        }
        if (progress) {
          idle = 0;
        } else {
          if (++idle >= kIdleLimit) { *abort_flag = 1u; ok = false; }
          else if ((idle & 63u) == 63u && *abort_flag) ok = false;
        }
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
    // An item's output leaves TMEM inside the NEXT item's first tile, between that tile's exponentials and its P store
    // (the last P.V of the item finishes under them); the CTA's last item after the loop.
    bool pending = false;          // an item whose O has not been written out yet
    T* pending_row = nullptr;      // nullptr: the row lies past the segment's end
    auto write_out = [&]() {       // O is stable: P.V of the item's last tile has been waited for
      ptx::tc_fence_after_sync();
      uint32_t o[64], sm[16];
      ptx::tmem_ld_32x64(t_o, o);
      ptx::tmem_ld_32x16(t_o + D, sm);
      ptx::tmem_ld_wait();
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(o_free);    // O and the row sum are in registers: the next item's first P.V may overwrite them
      if (pending_row != nullptr) {
        const float l = __uint_as_float(sm[0]);
        const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
        for (int c = 0; c < D; c += 8) {
          uint4 w;
          w.x = pack2<T>(__uint_as_float(o[c]) * inv, __uint_as_float(o[c + 1]) * inv);
          w.y = pack2<T>(__uint_as_float(o[c + 2]) * inv, __uint_as_float(o[c + 3]) * inv);
          w.z = pack2<T>(__uint_as_float(o[c + 4]) * inv, __uint_as_float(o[c + 5]) * inv);
          w.w = pack2<T>(__uint_as_float(o[c + 6]) * inv, __uint_as_float(o[c + 7]) * inv);
          *reinterpret_cast<uint4*>(pending_row + c) = w;
        }
      }
      pending = false;
    };
    for (int round = 0; ok; ++round) {
    const int it = item_of_round(round);
    if (it >= n_items) break;
    Item w;
    if (!decode(it, w)) continue;
    const int kv_len = w.kv_len, nkv = w.nkv;
    const bool row_ok = r < min(BQ, kv_len - w.q0);
    T* out = static_cast<T*>(p.out) + (static_cast<int64_t>(w.row0 + w.q0) * p.H + w.h) * D;
    float m_run = kNegInf;   // the reference maximum the exponentials, O and the row sums (in TMEM) are relative to
    for (int j = 0; ok && j < nkv; ++j) {
      const int gg = g + j, b = gg & 1;
      const int key0 = j * BKV;
      if (!ptx::mbar_wait(&s_full[b], (gg >> 1) & 1u, abort_flag)) { ok = false; break; }
      ptx::tc_fence_after_sync();
      uint32_t v[64];
      ptx::tmem_ld_32x64(tmem_base + lane_base + kColS + b * BKV, v);
      ptx::tmem_ld_wait();
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(&s_free[b]);          // the scores live in registers now: S[b] may take tile j+2
      const bool full = key0 + BKV <= kv_len;   // tiles inside the valid keys need no mask
      if (!full) {   // the segment's last tile: keys past its end become -inf scores, i.e. P = exp2(-inf) = 0 below
#pragma unroll
        for (int i = 0; i < 64; ++i) v[i] = key0 + i < kv_len ? v[i] : 0xff800000u;
      }
      // eight independent chains of three-input maxima (four deep), then a three-level tree
      float mx[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float a = max3(__uint_as_float(v[c]), __uint_as_float(v[c + 8]), __uint_as_float(v[c + 16]));
        const float b2 = max3(a, __uint_as_float(v[c + 24]), __uint_as_float(v[c + 32]));
        const float c2 = max3(b2, __uint_as_float(v[c + 40]), __uint_as_float(v[c + 48]));
        mx[c] = fmaxf(c2, __uint_as_float(v[c + 56]));
      }
      float tile_max = max3(max3(mx[0], mx[1], mx[2]), max3(mx[3], mx[4], mx[5]), fmaxf(mx[6], mx[7]));
      tile_max *= p.scale_log2;   // the scale is positive
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
      {
        // every exponential on the MUFU unit, scale / subtract as packed fp32x2 operations (masked keys carry -inf and
        // come out as exactly 0); the row sums are taken by the tensor core (see kIdescPV)
        const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
        const float2 nm2 = make_float2(-m_run, -m_run);
#pragma unroll
        for (int i = 0; i < 64; i += 2) {
          const float2 x = __ffma2_rn(make_float2(__uint_as_float(v[i]), __uint_as_float(v[i + 1])), sc2, nm2);
          packed[i / 2] = pack2<T>(ex2_fast(x.x), ex2_fast(x.y));
        }
      }
      // P.V of tile j-1 has finished: P may be rewritten and O is stable (it is only touched here when the maximum moved)
      if (j >= 1 || pending) {
        if (!ptx::mbar_wait(po_done, static_cast<uint32_t>(gg - 1) & 1u, abort_flag)) { ok = false; break; }
        if (j == 0) {
          write_out();                 // the previous item's rows (the maximum cannot have moved on a first tile)
        } else if (moved) {
          ptx::tc_fence_after_sync();
          uint32_t o[64];
          ptx::tmem_ld_32x64(t_o, o);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 64; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * rescale);
          ptx::tmem_st_32x32(t_o, reinterpret_cast<const uint32_t(&)[32]>(o[0]));
          ptx::tmem_st_32x32(t_o + 32, reinterpret_cast<const uint32_t(&)[32]>(o[32]));
          uint32_t sm[16];                       // the running row sum is relative to the same maximum
          ptx::tmem_ld_32x16(t_o + D, sm);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) sm[i] = __float_as_uint(__uint_as_float(sm[i]) * rescale);
          ptx::tmem_st_32x16(t_o + D, sm);
          ptx::tmem_st_wait();
          ptx::tc_fence_before_sync();
        }
      }
      // row r of P, K-major with the 128-byte swizzle: 16-byte chunk c (8 keys) sits at c ^ (r % 8)
      uint8_t* row_base = sP + r * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        *reinterpret_cast<uint4*>(row_base + ((c ^ (r & 7)) << 4)) =
            make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
      }
      ptx::fence_proxy_async_smem();
      ptx::mbar_arrive(p_full);
    }
    pending = ok;
    pending_row = row_ok ? out + static_cast<int64_t>(r) * out_ld : nullptr;
    g += nkv;
    }   // items
    if (ok && pending) {
      ok = ptx::mbar_wait(po_done, static_cast<uint32_t>(g - 1) & 1u, abort_flag);
      if (ok) write_out();
    }
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
    return launch_one(fmha_relpos64_kernel<T>);
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
