// Native executor of the packed Conformer encoder + CTC head: one host call
// enqueues the whole fixed kernel sequence (13 launches per layer) on the
// caller's stream.  Host code only; every step is one of this library's own
// C-ABI kernels.  No allocation, no host synchronisation, launch order and
// kernel choice are pure functions of the shapes.
#include <atomic>
#include <cmath>
#include <vector>

#include "common.cuh"

namespace ob {
namespace {

struct Workspace {
  float* res;      // (M, d) fp32 residual stream
  uint8_t* h;      // (M, d)   16-bit normalised activation
  uint8_t* y;      // (M, d)   16-bit sub-layer output
  uint8_t* a_ffn;  // (M, ffn)
  uint8_t* qkv4;   // (M, 4d)
  uint8_t* att;    // (M, d)
  uint8_t* g;      // (M, d)
  uint8_t* cv;     // (M, d)
  uint8_t* h3;     // (M, 2d)  after_norm as [hi | lo]
  uint8_t* pos;    // (max_seg, L*d)
  uint8_t* att_plan;  // work list of the packed attention kernel (oasr_b200_fmha_relpos_plan)
  int64_t att_plan_bytes;
  uint8_t* q8;     // (M, max(ffn, d)) one byte per element: per-token quantised GEMM input (quant_kind != 0)
  float* qs;       // (M) its scales
  int64_t bytes;
};

int64_t align256(int64_t x) { return (x + 255) / 256 * 256; }

struct ChunkWorkspace {
  float* res;
  uint8_t *h, *y, *a_ffn, *qkv4, *att, *xcat, *g, *cv, *h3;
  uint8_t* q8;     // quant_kind != 0: per-token quantised input of the current Linear, one byte per element
  float* qs;       // its row scales
  int64_t bytes;
};

ChunkWorkspace carve_chunk(const oasr_b200_conformer_model& m, int64_t B, int64_t T, uint8_t* base) {
  ChunkWorkspace w{};
  const int64_t d = m.d_model, M = B * T, MC = B * (T + m.kernel - 1);
  int64_t off = 0;
  auto take = [&](int64_t bytes) {
    uint8_t* p = base ? base + off : nullptr;
    off += align256(bytes);
    return p;
  };
  w.res = reinterpret_cast<float*>(take(M * d * 4));
  w.h = take(M * d * 2);
  w.y = take(M * d * 2);
  w.a_ffn = take(M * m.ffn * 2);
  w.qkv4 = take(M * 4 * d * 2);
  w.att = take(M * d * 2);
  w.xcat = take(MC * d * 2);
  w.g = take(MC * d * 2);
  w.cv = take(M * d * 2);
  w.h3 = take(M * 2 * d * 2);
  if (m.quant_kind != 0) {
    const int64_t widest = M * m.ffn > MC * d ? M * m.ffn : MC * d;
    w.q8 = take(widest);
    w.qs = reinterpret_cast<float*>(take(MC * 4));
  }
  w.bytes = off;
  return w;
}

// Optional per-step timing of the executor: a CUDA-event pair around every step, on the launching
// stream.  Off by default; switched on for one call by a benchmark.
struct ProfRecord {
  const char* label;
  double flops;
  cudaEvent_t a, b;
};
bool g_prof_on = false;
}  // namespace
// 1 (default): the last Linear of every sub-layer runs fused with the residual add and the following norm
// (oasr_b200_gemm_add_norm_f32) where the model width allows it and the batch fills the GPU; 2: whenever the width
// allows it; 0: gemm + add_norm_f32 as two kernels.
int g_fused_addnorm = 1;
int g_qkv_dup = 1;   // "qkv_dup": 1 = the q/q/k/v projection computes its query block once and stores it twice (two biases)
namespace {
std::vector<ProfRecord> g_prof;

// Scratch of oasr_b200_conformer_encode_packed_noalloc: lives in the library image, so every GPU
// whose context loads the library holds these bytes until the process exits.
constexpr int64_t kStaticScratchBytes = int64_t(64) << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

void prof_clear() {
  for (auto& r : g_prof) {
    cudaEventDestroy(r.a);
    cudaEventDestroy(r.b);
  }
  g_prof.clear();
}

Workspace carve(const oasr_b200_conformer_model& m, int64_t M, int64_t max_seg, uint8_t* base) {
  Workspace w{};
  const int64_t d = m.d_model;
  int64_t off = 0;
  auto take = [&](int64_t bytes) {
    uint8_t* p = base ? base + off : nullptr;
    off += align256(bytes);
    return p;
  };
  w.res = reinterpret_cast<float*>(take((M + 31) / 32 * 32 * d * 4));   // rows padded to whole 32-row bands (blocked layout)
  w.h = take(M * d * 2);
  w.y = take(M * d * 2);
  w.a_ffn = take(M * m.ffn * 2);
  w.qkv4 = take(M * 4 * d * 2);
  w.att = take(M * d * 2);
  w.g = take(M * d * 2);
  w.cv = take(M * d * 2);
  w.h3 = take(M * 2 * d * 2);
  w.pos = take(max_seg * m.num_layers * d * 2);
  // the plan serves at most 1024 segments (beyond that attention runs unplanned), each of at least one frame
  w.att_plan_bytes = oasr_b200_fmha_relpos_plan_bytes(M < 1024 ? M : 1024, m.heads, M);
  w.att_plan = take(w.att_plan_bytes);
  if (m.quant_kind != 0) {
    w.q8 = take(M * (m.ffn > d ? m.ffn : d));
    w.qs = reinterpret_cast<float*>(take(M * 4));
  }
  w.bytes = off;
  return w;
}

}  // namespace
}  // namespace ob

extern "C" {

int64_t oasr_b200_conformer_workspace_bytes(const oasr_b200_conformer_model* model, int64_t total, int64_t max_seg) {
  if (!model || total < 0 || max_seg < 0) return -1;
  return ob::carve(*model, total, max_seg, nullptr).bytes;
}

#define OB_STEP(label, flops, call)                                        \
  do {                                                                     \
    ob::ProfRecord pr_{label, static_cast<double>(flops), nullptr, nullptr}; \
    if (ob::g_prof_on) {                                                   \
      cudaEventCreate(&pr_.a);                                             \
      cudaEventCreate(&pr_.b);                                             \
      cudaEventRecord(pr_.a, static_cast<cudaStream_t>(stream));           \
    }                                                                      \
    int rc_ = (call);                                                      \
    if (ob::g_prof_on) {                                                   \
      cudaEventRecord(pr_.b, static_cast<cudaStream_t>(stream));           \
      ob::g_prof.push_back(pr_);                                           \
    }                                                                      \
    if (rc_ != OASR_OK) return rc_;                                        \
  } while (0)

int oasr_b200_profile_enable(int on) {
  ob::prof_clear();
  ob::g_prof_on = on != 0;
  return OASR_OK;
}

int oasr_b200_profile_count(void) { return static_cast<int>(ob::g_prof.size()); }

int oasr_b200_profile_get(int index, const char** label, double* ms, double* flops) {
  if (index < 0 || index >= static_cast<int>(ob::g_prof.size()))
    return ob::set_error(OASR_ERR_INVALID, "profile_get: index %d out of range", index);
  const ob::ProfRecord& r = ob::g_prof[index];
  cudaError_t e = cudaEventSynchronize(r.b);
  float t = 0.f;
  if (e == cudaSuccess) e = cudaEventElapsedTime(&t, r.a, r.b);
  if (e != cudaSuccess) return ob::set_error(OASR_ERR_CUDA, "profile_get: %s", cudaGetErrorString(e));
  if (label) *label = r.label;
  if (ms) *ms = t;
  if (flops) *flops = r.flops;
  return OASR_OK;
}

int oasr_b200_conformer_encode_packed(const oasr_b200_conformer_model* model, const void* rows,
                                      const int32_t* cu_seqlens, const int32_t* fill_frames, int64_t num_segs,
                                      int64_t total, int64_t max_seg, void* workspace, int64_t workspace_bytes,
                                      float* log_probs, int32_t* argmax, void* stream) {
  using namespace ob;
  OB_REQUIRE(model && model->layers, OASR_ERR_INVALID, "conformer_encode_packed: null model");
  const oasr_b200_conformer_model& m = *model;
  OB_REQUIRE(m.num_layers > 0 && m.d_model > 0 && m.heads > 0 && m.d_model == m.heads * 64, OASR_ERR_UNSUPPORTED,
             "conformer_encode_packed: needs head_dim 64 (d_model %d, heads %d)", m.d_model, m.heads);
  OB_REQUIRE(num_segs >= 0 && total >= 0 && max_seg >= 0, OASR_ERR_INVALID, "conformer_encode_packed: bad shape");
  if (total == 0 || num_segs == 0) return OASR_OK;
  OB_REQUIRE(rows && cu_seqlens && workspace, OASR_ERR_INVALID, "conformer_encode_packed: null pointer argument");
  OB_REQUIRE(is_aligned(workspace, 256), OASR_ERR_ALIGN, "conformer_encode_packed: workspace must be 256-byte aligned");
  OB_REQUIRE(max_seg <= m.pe_rows, OASR_ERR_INVALID,
             "conformer_encode_packed: segment of %lld frames exceeds the positional table (%lld rows)",
             (long long)max_seg, (long long)m.pe_rows);
  Workspace w = carve(m, total, max_seg, static_cast<uint8_t*>(workspace));
  OB_REQUIRE(workspace_bytes >= w.bytes, OASR_ERR_INVALID, "conformer_encode_packed: workspace of %lld bytes, %lld needed",
             (long long)workspace_bytes, (long long)w.bytes);
  const int64_t M = total, d = m.d_model, L = m.num_layers;
  const int dt = m.dtype;
  const double scale = 1.0 / std::sqrt(64.0);
  const oasr_b200_conformer_layer* ly = m.layers;

  // embed Linear (+ LayerNorm with sqrt(d) folded) -> fp32 residual, and the first pre-norm
  // One Linear of the layer stack: 16-bit GEMM, or per-token quantisation of the input followed by the 8-bit GEMM
  // on the pre-quantised weight `qi` of the layer (order of oasr_b200_conformer_layer::q_w).
  const int qk = m.quant_kind;
  OB_REQUIRE(qk == 0 || qk == OASR_Q8_FP8_E4M3 || qk == OASR_Q8_INT8, OASR_ERR_INVALID, "conformer_encode_packed: bad quant_kind %d", qk);
#define OB_LINEAR(label, fl, out, in, wt, bs, lay, qi, N, K, act, glu)                                              \
  do {                                                                                                              \
    if (qk == 0) {                                                                                                  \
      if (glu) OB_STEP("gemm_glu " label, fl, oasr_b200_gemm_glu(out, in, wt, bs, M, N, K, dt, stream));              \
      else OB_STEP("gemm " label, fl, oasr_b200_gemm(out, in, wt, bs, M, N, K, act, dt, stream));                    \
    } else {                                                                                                        \
      OB_STEP("quantize_rows", 0, oasr_b200_quantize_rows(w.q8, w.qs, in, M, K, qk, dt, stream));                     \
      OB_STEP("gemm_q8 " label, fl, oasr_b200_gemm_q8(out, w.q8, w.qs, (lay).q_w[qi], (lay).q_s[qi], bs, M, N, K, act, glu, qk, dt, stream)); \
    }                                                                                                               \
  } while (0)
  // Last Linear of a sub-layer + residual step + norm: one fused kernel where the width allows it (16-bit GEMMs),
  // else the Linear into w.y followed by add_norm_f32.  `rin` is the residual input (null for the embed).
  // The fused kernel keeps the residual stream in its own blocked layout, add_norm_f32 row-major: one or the other
  // for the whole call.
  // The fused kernel gives one 256-row tile to a pair of SMs and cannot overlap a tile's epilogue with the next main
  // loop, so it pays only when its tiles fill the GPU: at least 80 % of the SM pairs busy in every round (measured on
  // B200, d 512: 16.7k rows, 66 of 74 pairs, fused 7.07 against 7.30 ms per step; 8.3k rows, 32 pairs, 4.69 against 4.34).
  const bool qkv_dup = qk == 0 && g_qkv_dup != 0 && M >= 128 && oasr_b200_gemm_dup_first_supported(3 * d, d, d) != 0;
  const int64_t pairs = (M + 255) / 256, slots = sm_count() / 2;
  const int64_t rounds = (pairs + slots - 1) / slots;
  const bool fills = g_fused_addnorm == 2 || pairs * 5 >= rounds * slots * 4;
  const bool fuse = qk == 0 && g_fused_addnorm != 0 && fills && oasr_b200_gemm_add_norm_supported(d, d) != 0 &&
                    oasr_b200_gemm_add_norm_supported(d, m.ffn) != 0 && oasr_b200_gemm_add_norm_supported(d, m.embed_in) != 0;
  // add + norm; with an 8-bit kind (and an unsplit h) the kernel also leaves the quantised row of h in w.q8 / w.qs for
  // the Linear that reads h next, which then skips its own quantisation launch (OB_LINEAR_H)
#define OB_ADD_NORM(hout, rout, rin, y_, alpha, mode, wa, ba, wb, bb, eps_, split)                                      \
  OB_STEP("add_norm", 0, oasr_b200_add_norm_f32_q8(hout, rout, rin, y_, alpha, mode, wa, ba, wb, bb, M, d, eps_, split,   \
                                                   (qk && !(split)) ? w.q8 : nullptr, (qk && !(split)) ? w.qs : nullptr, qk, dt, stream))
#define OB_LINEAR_H(label, fl, out, wt, bs, lay, qi, N, act, glu)                                                     \
  do {                                                                                                              \
    if (qk == 0) OB_LINEAR(label, fl, out, w.h, wt, bs, lay, qi, N, d, act, glu);                                     \
    else OB_STEP("gemm_q8 " label, fl, oasr_b200_gemm_q8(out, w.q8, w.qs, (lay).q_w[qi], (lay).q_s[qi], bs, M, N, d, act, glu, qk, dt, stream)); \
  } while (0)
#define OB_LINEAR_ADDNORM(label, fl, hout, rin, in, wt, bs, lay, qi, K, alpha, mode, wa, ba, wb, bb, eps_, split)       \
  do {                                                                                                              \
    if (fuse) {                                                                                                     \
      OB_STEP("gemm_addnorm " label, fl, oasr_b200_gemm_add_norm_f32(hout, w.res, rin, in, wt, bs, M, d, K, alpha, mode, wa, ba, \
                                                                    wb, bb, eps_, split, dt, stream));              \
    } else {                                                                                                        \
      OB_LINEAR(label, fl, w.y, in, wt, bs, lay, qi, d, K, OASR_ACT_NONE, 0);                                        \
      OB_ADD_NORM(hout, w.res, rin, w.y, alpha, mode, wa, ba, wb, bb, eps_, split);                                   \
    }                                                                                                               \
  } while (0)
  if (fuse) {
    if (m.embed_ln_w) {
      OB_STEP("gemm_addnorm embed", 2.0 * M * d * m.embed_in, oasr_b200_gemm_add_norm_f32(w.h, w.res, nullptr, rows, m.embed_w, m.embed_b, M, d, m.embed_in, 1.0, 2,
                                     m.embed_ln_w, m.embed_ln_b, ly[0].norm_ff_macaron_w, ly[0].norm_ff_macaron_b, 1e-5, 0, dt, stream));
    } else {
      OB_STEP("gemm_addnorm embed", 2.0 * M * d * m.embed_in, oasr_b200_gemm_add_norm_f32(w.h, w.res, nullptr, rows, m.embed_w, m.embed_b, M, d, m.embed_in, 1.0, 0,
                                     ly[0].norm_ff_macaron_w, ly[0].norm_ff_macaron_b, nullptr, nullptr, m.eps, 0, dt, stream));
    }
  } else {
  // The embedding is the first value of the fp32 residual stream: it goes there in fp32 straight from the GEMM's
  // epilogue (a 16-bit round trip here would put a rounding error on every element that all layers then carry).
  OB_STEP("gemm embed", 2.0 * M * d * m.embed_in, oasr_b200_gemm_residual_f32(w.res, nullptr, rows, m.embed_w, m.embed_b, M, d, m.embed_in, 1.0, dt, stream));
  if (m.embed_ln_w) {
    OB_ADD_NORM(w.h, w.res, w.res, nullptr, 0.0, 2, m.embed_ln_w, m.embed_ln_b, ly[0].norm_ff_macaron_w, ly[0].norm_ff_macaron_b, 1e-5, 0);
  } else {
    OB_ADD_NORM(w.h, nullptr, w.res, nullptr, 0.0, 0, ly[0].norm_ff_macaron_w, ly[0].norm_ff_macaron_b, nullptr, nullptr, m.eps, 0);
  }
  }
  // attention work list (longest segments first), once per batch; every layer reuses it
  const void* att_plan = nullptr;
  if (num_segs <= 1024 && oasr_b200_fmha_relpos_plan_bytes(num_segs, m.heads, M) <= w.att_plan_bytes) {
    OB_STEP("fmha_relpos_plan", 0, oasr_b200_fmha_relpos_plan(w.att_plan, w.att_plan_bytes, cu_seqlens, num_segs, m.heads, M, stream));
    att_plan = w.att_plan;
  }
  // linear_pos of every layer in one GEMM: (max_seg, d) x (L*d, d)^T
  OB_STEP("gemm linear_pos", 2.0 * max_seg * L * d * d, oasr_b200_gemm(w.pos, m.pe, m.pos_w_all, nullptr, max_seg, L * d, d, OASR_ACT_NONE, dt, stream));

  for (int64_t i = 0; i < L; ++i) {
    const oasr_b200_conformer_layer& l = ly[i];
    // macaron feed-forward
    OB_LINEAR_H("ffn_w1", 2.0 * M * m.ffn * d, w.a_ffn, l.ffm_w1, l.ffm_b1, l, 0, m.ffn, OASR_ACT_SWISH, 0);
    OB_LINEAR_ADDNORM("ffn_w2", 2.0 * M * m.ffn * d, w.h, w.res, w.a_ffn, l.ffm_w2, l.ffm_b2, l, 1, m.ffn, 0.5, 0, l.norm_mha_w,
                      l.norm_mha_b, nullptr, nullptr, m.eps, 0);
    // relative-position self-attention
    if (qkv_dup) {   // [Wq;Wk;Wv] are rows d.. of [Wq;Wq;Wk;Wv]: the query block once, stored as q+u and q+v
      OB_STEP("gemm qkv4", 2.0 * M * 3 * d * d, oasr_b200_gemm_dup_first(w.qkv4, w.h, static_cast<const uint8_t*>(l.qkv4_w) + d * d * 2, l.qkv4_b, M, 3 * d, d, d, dt, stream));
    } else {
      OB_LINEAR_H("qkv4", 2.0 * M * 3 * d * d /* algorithmic: the query block is issued twice */, w.qkv4, l.qkv4_w, l.qkv4_b, l, 2, 4 * d, OASR_ACT_NONE, 0);
    }
    OB_STEP("fmha_varlen_relpos", 0, oasr_b200_fmha_varlen_relpos_planned(w.att, w.qkv4, w.pos + i * d * 2, max_seg, L * d, cu_seqlens, num_segs,
                                         max_seg, M, m.heads, scale, att_plan, dt, stream));
    OB_LINEAR_ADDNORM("attn_out", 2.0 * M * d * d, w.h, w.res, w.att, l.out_w, l.out_b, l, 3, d, 1.0, 1, l.norm_conv_scale,
                      l.norm_conv_shift, nullptr, nullptr, m.eps, 0);
    // convolution module
    OB_LINEAR_H("pw1", 2.0 * M * 2 * d * d, w.g, l.pw1_w, l.pw1_b, l, 4, d, OASR_ACT_NONE, 1);
    OB_STEP("depthwise_conv1d_packed", 0, oasr_b200_depthwise_conv1d_packed(w.cv, w.g, l.dw_w, l.dw_b, l.conv_bn_scale, l.conv_bn_shift,
                                              fill_frames ? l.glu_of_bias : nullptr, fill_frames, cu_seqlens, num_segs,
                                              max_seg, d, m.kernel, OASR_ACT_SWISH, dt, stream));
    OB_LINEAR_ADDNORM("pw2", 2.0 * M * d * d, w.h, w.res, w.cv, l.pw2_w, l.pw2_b, l, 5, d, 1.0, 0, l.norm_ff_w, l.norm_ff_b, nullptr,
                      nullptr, m.eps, 0);
    // feed-forward, norm_final, then the next layer's first pre-norm (or after_norm, split for the head)
    OB_LINEAR_H("ffn_w1", 2.0 * M * m.ffn * d, w.a_ffn, l.ff_w1, l.ff_b1, l, 6, m.ffn, OASR_ACT_SWISH, 0);
    if (i + 1 < L) {
      OB_LINEAR_ADDNORM("ffn_w2", 2.0 * M * m.ffn * d, w.h, w.res, w.a_ffn, l.ff_w2, l.ff_b2, l, 7, m.ffn, 0.5, 2, l.norm_final_w,
                        l.norm_final_b, ly[i + 1].norm_ff_macaron_w, ly[i + 1].norm_ff_macaron_b, m.eps, 0);
    } else {
      OB_LINEAR_ADDNORM("ffn_w2", 2.0 * M * m.ffn * d, w.h3, w.res, w.a_ffn, l.ff_w2, l.ff_b2, l, 7, m.ffn, 0.5, 2, l.norm_final_w,
                        l.norm_final_b, m.after_norm_w, m.after_norm_b, m.eps, 1);
    }
  }
  if (log_probs || argmax) {   // log_probs == NULL: token-only head, one vocabulary sweep, no log-prob write
    OB_STEP("gemm_log_softmax", 2.0 * M * m.vocab_padded * d /* algorithmic; issued with the input split in two 16-bit terms (K = 2d) */, oasr_b200_gemm_log_softmax(log_probs, w.h3, m.ctc_w, m.ctc_b, M, m.vocab_padded, 2 * d, dt, OASR_DT_F32,
                                       argmax, stream));
  }
  return OASR_OK;
}

int64_t oasr_b200_conformer_noalloc_capacity_bytes(void) { return ob::kStaticScratchBytes; }

// Same work as oasr_b200_conformer_encode_packed, for callers that are not allowed to allocate
// device memory: a plugin living inside a host process that handed all of the GPU's memory to its
// own pool at start-up, code running between a framework's allocator hooks, or a real-time
// thread where a cudaMalloc (which may synchronise the whole device) is off limits.  They cannot
// bring a workspace, so the scratch is a fixed 64 MiB array inside the library.
//
// Set-up: the array's name is only a host-side handle here, not something a kernel can be given.
// The first call on each device -- made with that device current -- asks the runtime for the
// array's device address (cudaGetSymbolAddress), checks the result and keeps it for later calls
// on that device.  Make that first call outside of any stream capture.  It is also the moment the
// CUDA runtime loads this part of the library onto the device, which is when the 64 MiB are
// really reserved: a host whose pool takes all GPU memory should make one warm-up call per device
// (total = 0 is enough: the address is resolved before the empty batch returns) BEFORE the pool
// grabs the memory; later the call would fail with an out-of-memory status instead.  The per-device
// address is published atomically, so concurrent first calls are safe; they only repeat the lookup.
//
// Limits and sharing: a batch whose scratch need (oasr_b200_conformer_workspace_bytes) exceeds
// oasr_b200_conformer_noalloc_capacity_bytes() is refused with OASR_ERR_INVALID before anything
// is launched.  All calls on a device use the same array; it keeps whatever the previous call
// left there and no step depends on its initial contents (every buffer carved from it is fully
// written before it is read), so nothing is cleared.  Two calls whose kernels overlap on the GPU
// (different streams, or different host threads) would overwrite each other's intermediates:
// serialise them.  No cudaMalloc / cudaFree or allocating library routine is called.
int oasr_b200_conformer_encode_packed_noalloc(const oasr_b200_conformer_model* model, const void* rows,
                                              const int32_t* cu_seqlens, const int32_t* fill_frames,
                                              int64_t num_segs, int64_t total, int64_t max_seg, float* log_probs,
                                              int32_t* argmax, void* stream) {
  using namespace ob;
  OB_REQUIRE(model != nullptr, OASR_ERR_INVALID, "conformer_encode_packed_noalloc: null model");
  OB_REQUIRE(total >= 0 && max_seg >= 0, OASR_ERR_INVALID, "conformer_encode_packed_noalloc: bad shape");
  const int64_t need = carve(*model, total, max_seg, nullptr).bytes;
  OB_REQUIRE(need <= kStaticScratchBytes, OASR_ERR_INVALID,
             "conformer_encode_packed_noalloc: this batch needs %lld bytes of scratch but the built-in array holds "
             "%lld; send fewer frames per call or use oasr_b200_conformer_encode_packed with your own workspace",
             (long long)need, (long long)kStaticScratchBytes);
  static std::atomic<unsigned char*> scratch_of_device[64];
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  OB_REQUIRE(e == cudaSuccess && dev >= 0 && dev < 64, OASR_ERR_CUDA,
             "conformer_encode_packed_noalloc: cannot identify the current device (%s)", cudaGetErrorString(e));
  unsigned char* scratch = scratch_of_device[dev].load(std::memory_order_acquire);
  if (scratch == nullptr) {
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&scratch), g_static_scratch);
    OB_REQUIRE(e != cudaErrorMemoryAllocation, OASR_ERR_CUDA,
               "conformer_encode_packed_noalloc: device %d has no room left for the library's %lld-byte scratch array; make "
               "one warm-up call per device at start-up, before the host's pool takes the memory",
               dev, (long long)kStaticScratchBytes);
    OB_REQUIRE(e == cudaSuccess && scratch != nullptr, OASR_ERR_CUDA,
               "conformer_encode_packed_noalloc: the scratch array has no device address on device %d (%s)", dev,
               cudaGetErrorString(e));
    scratch_of_device[dev].store(scratch, std::memory_order_release);
  }
  return oasr_b200_conformer_encode_packed(model, rows, cu_seqlens, fill_frames, num_segs, total, max_seg, scratch,
                                           kStaticScratchBytes, log_probs, argmax, stream);
}

int64_t oasr_b200_conformer_chunk_workspace_bytes(const oasr_b200_conformer_model* model, int64_t B, int64_t T) {
  if (!model || B < 0 || T < 0) return -1;
  return ob::carve_chunk(*model, B, T, nullptr).bytes;
}

int oasr_b200_conformer_chunk_paged(const oasr_b200_conformer_model* model, const void* rows, int64_t B, int64_t T,
                                    void* const* k_pools, void* const* v_pools, const int32_t* block_table,
                                    const int32_t* cache_seqlens, const int32_t* total_seqlens,
                                    const int32_t* pos_start, int64_t blocks_per_seq, int64_t block_size,
                                    int64_t num_blocks, const float* kv_scales, void* cnn_state, int64_t num_slots,
                                    const int64_t* slot_ids,
                                    void* workspace, int64_t workspace_bytes, float* log_probs, int32_t* argmax,
                                    void* stream) {
  using namespace ob;
  OB_REQUIRE(model && model->layers, OASR_ERR_INVALID, "conformer_chunk_paged: null model");
  const oasr_b200_conformer_model& m = *model;
  OB_REQUIRE(m.d_model == m.heads * 64, OASR_ERR_UNSUPPORTED, "conformer_chunk_paged: needs head_dim 64");
  OB_REQUIRE(B >= 0 && T > 0 && T <= 128, OASR_ERR_INVALID, "conformer_chunk_paged: bad shape (B %lld, T %lld)",
             (long long)B, (long long)T);
  if (B == 0) return OASR_OK;
  OB_REQUIRE(rows && k_pools && v_pools && block_table && cache_seqlens && total_seqlens && pos_start && cnn_state &&
                 slot_ids && workspace,
             OASR_ERR_INVALID, "conformer_chunk_paged: null pointer argument");
  OB_REQUIRE(m.pos_proj && m.pos_proj_rows > 0, OASR_ERR_INVALID,
             "conformer_chunk_paged: the model has no projected positional table (pos_proj)");
  OB_REQUIRE(is_aligned(workspace, 256), OASR_ERR_ALIGN, "conformer_chunk_paged: workspace must be 256-byte aligned");
  const int qk = m.quant_kind;
  OB_REQUIRE(qk == 0 || qk == OASR_Q8_FP8_E4M3 || qk == OASR_Q8_INT8, OASR_ERR_INVALID, "conformer_chunk_paged: bad quant_kind %d", qk);
  ChunkWorkspace w = carve_chunk(m, B, T, static_cast<uint8_t*>(workspace));
  OB_REQUIRE(workspace_bytes >= w.bytes, OASR_ERR_INVALID, "conformer_chunk_paged: workspace of %lld bytes, %lld needed",
             (long long)workspace_bytes, (long long)w.bytes);
  const int64_t d = m.d_model, L = m.num_layers, M = B * T, SL = m.kernel - 1, MC = B * (T + SL);
  const int dt = m.dtype;
  const double scale = 1.0 / std::sqrt(64.0);
  const oasr_b200_conformer_layer* ly = m.layers;

  const bool qkv_dup = qk == 0 && g_qkv_dup != 0 && B * T >= 128 && oasr_b200_gemm_dup_first_supported(3 * m.d_model, m.d_model, m.d_model) != 0;
  // One Linear over `R` rows: 16-bit GEMM, or per-token quantisation of the input followed by the 8-bit GEMM on the
  // layer's pre-quantised weight `qi` (order of oasr_b200_conformer_layer::q_w), as in the offline executor.
#define OB_CHUNK_LINEAR(label, fl, out, in, wt, bs, lay, qi, R, N, K, act, glu)                                       \
  do {                                                                                                                \
    if (qk == 0) {                                                                                                    \
      if (glu) OB_STEP("gemm_glu " label, fl, oasr_b200_gemm_glu(out, in, wt, bs, R, N, K, dt, stream));                \
      else OB_STEP("gemm " label, fl, oasr_b200_gemm(out, in, wt, bs, R, N, K, act, dt, stream));                      \
    } else {                                                                                                          \
      OB_STEP("quantize_rows", 0, oasr_b200_quantize_rows(w.q8, w.qs, in, R, K, qk, dt, stream));                       \
      OB_STEP("gemm_q8 " label, fl, oasr_b200_gemm_q8(out, w.q8, w.qs, (lay).q_w[qi], (lay).q_s[qi], bs, R, N, K, act, glu, qk, dt, stream)); \
    }                                                                                                                 \
  } while (0)

  // a Linear over the M chunk rows whose input h the add + norm before it has already quantised (8-bit kinds)
#define OB_CHUNK_LINEAR_H(label, fl, out, wt, bs, lay, qi, N, act)                                                    \
  do {                                                                                                                \
    if (qk == 0) OB_CHUNK_LINEAR(label, fl, out, w.h, wt, bs, lay, qi, M, N, d, act, 0);                                \
    else OB_STEP("gemm_q8 " label, fl, oasr_b200_gemm_q8(out, w.q8, w.qs, (lay).q_w[qi], (lay).q_s[qi], bs, M, N, d, act, 0, qk, dt, stream)); \
  } while (0)
  // the embedding starts the fp32 residual stream unrounded (see the offline executor)
  OB_STEP("gemm embed", 2.0 * M * d * m.embed_in, oasr_b200_gemm_residual_f32(w.res, nullptr, rows, m.embed_w, m.embed_b, M, d, m.embed_in, 1.0, dt, stream));
  if (m.embed_ln_w) {
    OB_ADD_NORM(w.h, w.res, w.res, nullptr, 0.0, 2, m.embed_ln_w, m.embed_ln_b, ly[0].norm_ff_macaron_w, ly[0].norm_ff_macaron_b, 1e-5, 0);
  } else {
    OB_ADD_NORM(w.h, nullptr, w.res, nullptr, 0.0, 0, ly[0].norm_ff_macaron_w, ly[0].norm_ff_macaron_b, nullptr, nullptr, m.eps, 0);
  }
  for (int64_t i = 0; i < L; ++i) {
    const oasr_b200_conformer_layer& l = ly[i];
    OB_CHUNK_LINEAR_H("ffn_w1", 2.0 * M * m.ffn * d, w.a_ffn, l.ffm_w1, l.ffm_b1, l, 0, m.ffn, OASR_ACT_SWISH);
    OB_CHUNK_LINEAR("ffn_w2", 2.0 * M * m.ffn * d, w.y, w.a_ffn, l.ffm_w2, l.ffm_b2, l, 1, M, d, m.ffn, OASR_ACT_NONE, 0);
    OB_ADD_NORM(w.h, w.res, w.res, w.y, 0.5, 0, l.norm_mha_w, l.norm_mha_b, nullptr, nullptr, m.eps, 0);
    // attention: project, append the chunk's keys/values to the pages, attend over cache + chunk
    if (qkv_dup) {
      OB_STEP("gemm qkv4", 2.0 * M * 3 * d * d, oasr_b200_gemm_dup_first(w.qkv4, w.h, static_cast<const uint8_t*>(l.qkv4_w) + d * d * 2, l.qkv4_b, M, 3 * d, d, d, dt, stream));
    } else {
      OB_CHUNK_LINEAR_H("qkv4", 2.0 * M * 3 * d * d, w.qkv4, l.qkv4_w, l.qkv4_b, l, 2, 4 * d, OASR_ACT_NONE);
    }
    if (kv_scales) {   // fp8 pages: per-head scales of this layer, K then V
      const float* ks = kv_scales + static_cast<int64_t>(i) * 2 * m.heads;
      const float* vs = ks + m.heads;
      OB_STEP("paged_kv_write", 0, oasr_b200_paged_kv_write_fp8(k_pools[i], v_pools[i], w.qkv4 + 2 * d * 2, w.qkv4 + 3 * d * 2,
                                       ks, vs, block_table, cache_seqlens, B, m.heads, T, 64, T * 4 * d, 64, 4 * d,
                                       blocks_per_seq, block_size, num_blocks, dt, stream));
      OB_STEP("fmha_paged_relpos", 0, oasr_b200_fmha_paged_relpos_fp8(w.att, w.qkv4, k_pools[i], v_pools[i], ks, vs,
                                       static_cast<const uint8_t*>(m.pos_proj) + i * d * 2, m.pos_proj_rows, L * d,
                                       pos_start, block_table, total_seqlens, B, T, m.heads, blocks_per_seq, block_size,
                                       num_blocks, scale, dt, stream));
    } else {
      OB_STEP("paged_kv_write", 0, oasr_b200_paged_kv_write(k_pools[i], v_pools[i], w.qkv4 + 2 * d * 2, w.qkv4 + 3 * d * 2,
                                       block_table, cache_seqlens, B, m.heads, T, 64, T * 4 * d, 64, 4 * d, blocks_per_seq,
                                       block_size, num_blocks, 2, stream));
      OB_STEP("fmha_paged_relpos", 0, oasr_b200_fmha_paged_relpos(w.att, w.qkv4, k_pools[i], v_pools[i],
                                       static_cast<const uint8_t*>(m.pos_proj) + i * d * 2, m.pos_proj_rows, L * d,
                                       pos_start, block_table, total_seqlens, B, T, m.heads, blocks_per_seq, block_size,
                                       num_blocks, scale, dt, stream));
    }
    OB_CHUNK_LINEAR("attn_out", 2.0 * M * d * d, w.y, w.att, l.out_w, l.out_b, l, 3, M, d, d, OASR_ACT_NONE, 0);
    OB_ADD_NORM(w.h, w.res, w.res, w.y, 1.0, 1, l.norm_conv_scale, l.norm_conv_shift, nullptr, nullptr, m.eps, 0);
    // convolution module with the cached left context
    OB_STEP("conv_state_concat", 0, oasr_b200_conv_state_concat(w.xcat, static_cast<uint8_t*>(cnn_state) + i * num_slots * SL * d * 2,
                                     num_slots, slot_ids, w.h, B, SL, T, d, dt, stream));
    OB_CHUNK_LINEAR("pw1", 2.0 * MC * 2 * d * d, w.g, w.xcat, l.pw1_w, l.pw1_b, l, 4, MC, d, d, OASR_ACT_NONE, 1);
    OB_STEP("depthwise_conv1d", 0, oasr_b200_depthwise_conv1d_affine(w.cv, w.g, l.dw_w, l.dw_b, l.conv_bn_scale, l.conv_bn_shift,
                                     B, T + SL, d, m.kernel, 0, 0, OASR_ACT_SWISH, dt, stream));
    OB_CHUNK_LINEAR("pw2", 2.0 * M * d * d, w.y, w.cv, l.pw2_w, l.pw2_b, l, 5, M, d, d, OASR_ACT_NONE, 0);
    OB_ADD_NORM(w.h, w.res, w.res, w.y, 1.0, 0, l.norm_ff_w, l.norm_ff_b, nullptr, nullptr, m.eps, 0);
    OB_CHUNK_LINEAR_H("ffn_w1", 2.0 * M * m.ffn * d, w.a_ffn, l.ff_w1, l.ff_b1, l, 6, m.ffn, OASR_ACT_SWISH);
    OB_CHUNK_LINEAR("ffn_w2", 2.0 * M * m.ffn * d, w.y, w.a_ffn, l.ff_w2, l.ff_b2, l, 7, M, d, m.ffn, OASR_ACT_NONE, 0);
    if (i + 1 < L) {
      OB_ADD_NORM(w.h, w.res, w.res, w.y, 0.5, 2, l.norm_final_w, l.norm_final_b, ly[i + 1].norm_ff_macaron_w, ly[i + 1].norm_ff_macaron_b, m.eps, 0);
    } else {
      OB_ADD_NORM(w.h3, w.res, w.res, w.y, 0.5, 2, l.norm_final_w, l.norm_final_b, m.after_norm_w, m.after_norm_b, m.eps, 1);
    }
  }
  if (log_probs || argmax) {   // log_probs == NULL: token-only head, one vocabulary sweep, no log-prob write
    OB_STEP("gemm_log_softmax", 2.0 * M * m.vocab_padded * d /* algorithmic; issued with the input split in two 16-bit terms (K = 2d) */, oasr_b200_gemm_log_softmax(log_probs, w.h3, m.ctc_w, m.ctc_b, M, m.vocab_padded, 2 * d, dt, OASR_DT_F32,
                                       argmax, stream));
  }
  return OASR_OK;
}

}  // extern "C"
