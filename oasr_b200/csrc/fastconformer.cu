// Native executor of the packed FastConformer / Nemotron layer stack: one host call enqueues the whole fixed
// kernel sequence of NemotronEncoder.forward's layer loop (oasr/models/nemotron/encoder.py:217-267, 542-583) on the
// caller's stream -- per layer 17 launches (21 with an 8-bit kind: the add + norm kernels also write the quantised
// row for the Linear behind them) of this library's own C-ABI kernels: macaron FFN, Transformer-XL
// relative-position attention (q projected once per global bias, position scores as one batched GEMM over heads,
// one kernel for the relative shift + scale + chunked-limited window, head_dim 128 attention with that bias),
// conv module (GLU GEMM, causal depthwise conv per segment, LayerNorm + SiLU, pointwise GEMM), second FFN, with the
// fp32 residual stream and the fused add + LayerNorm between the sub-layers; with an 8-bit kind every Linear is a
// per-token quantisation of its input followed by the fp8 / int8 GEMM on the pre-quantised weight.  Host code only: no allocation, no host
// synchronisation; launch order and kernel choice are pure functions of the shapes.  The rows are the valid frames of
// all utterances back to back (no padding frame is ever computed).
#include <cmath>

#include "common.cuh"

namespace ob {
namespace {

struct FcWorkspace {
  float* res;      // (M, C)   fp32 residual stream
  uint8_t* h;      // (M, C)   16-bit normalised activation
  uint8_t* y;      // (M, C)   16-bit sub-layer output
  uint8_t* a_ffn;  // (M, F)
  uint8_t* qkv4;   // (M, 4C)
  uint8_t* att;    // (M, C)
  uint8_t* g;      // (M, C)
  uint8_t* cv;     // (M, C)
  uint8_t* rel_k;  // (Pp, C)  projected relative-position table of the current layer
  uint8_t* bd;     // (H, M, Pp) position scores
  uint8_t* bias;   // bias_numel elements: block-diagonal attention bias
  uint8_t* q8;     // (M, max(C, F)) 8-bit kinds: the per-token quantised input of the current Linear
  float* qs;       // (M) its row scales
  int64_t bytes;
};

int64_t fc_align(int64_t x) { return (x + 255) / 256 * 256; }

FcWorkspace fc_carve(const oasr_b200_fastconformer_model& m, int64_t M, int64_t table_rows, int64_t bias_numel, uint8_t* base) {
  FcWorkspace w{};
  const int64_t C = m.hidden;
  int64_t off = 0;
  auto take = [&](int64_t bytes) {
    uint8_t* p = base ? base + off : nullptr;
    off += fc_align(bytes);
    return p;
  };
  w.res = reinterpret_cast<float*>(take(M * C * 4));
  w.h = take(M * C * 2);
  w.y = take(M * C * 2);
  w.a_ffn = take(M * m.ffn * 2);
  w.qkv4 = take(M * 4 * C * 2);
  w.att = take(M * C * 2);
  w.g = take(M * C * 2);
  w.cv = take(M * C * 2);
  w.rel_k = take(table_rows * C * 2);
  w.bd = take(static_cast<int64_t>(m.heads) * M * table_rows * 2);
  w.bias = take(bias_numel * 2);
  if (m.quant_kind != 0) {
    w.q8 = take(M * (m.ffn > C ? m.ffn : C));
    w.qs = reinterpret_cast<float*>(take(M * 4));
  }
  w.bytes = off;
  return w;
}

}  // namespace
}  // namespace ob

extern "C" {

int64_t oasr_b200_fastconformer_workspace_bytes(const oasr_b200_fastconformer_model* model, int64_t total,
                                                int64_t table_rows, int64_t bias_numel) {
  if (!model || total < 0 || table_rows < 0 || bias_numel < 0) return -1;
  return ob::fc_carve(*model, total, table_rows, bias_numel, nullptr).bytes;
}

#define FC_STEP(call)                  \
  do {                                 \
    int rc_ = (call);                  \
    if (rc_ != OASR_OK) return rc_;    \
  } while (0)

int oasr_b200_fastconformer_layers_packed(const oasr_b200_fastconformer_model* model, const void* rows, int rows_f32, float* out,
                                          const void* rel_table, int64_t table_rows, const int32_t* cu_seqlens,
                                          const int64_t* bias_offsets, int64_t bias_numel, int64_t num_segs,
                                          int64_t total, int64_t max_seg, void* workspace, int64_t workspace_bytes,
                                          void* stream) {
  using namespace ob;
  OB_REQUIRE(model && model->layers, OASR_ERR_INVALID, "fastconformer_layers_packed: null model");
  const oasr_b200_fastconformer_model& m = *model;
  OB_REQUIRE(m.num_layers > 0 && m.hidden > 0 && m.heads > 0 && m.hidden % m.heads == 0 &&
                 (m.hidden / m.heads == 64 || m.hidden / m.heads == 128),
             OASR_ERR_UNSUPPORTED, "fastconformer_layers_packed: head_dim must be 64 or 128 (hidden %d, heads %d)", m.hidden,
             m.heads);
  OB_REQUIRE(m.kernel > 0 && m.ffn > 0 && m.right_context >= 0, OASR_ERR_INVALID, "fastconformer_layers_packed: bad model geometry");
  OB_REQUIRE(num_segs >= 0 && total >= 0 && max_seg >= 0 && bias_numel >= 0, OASR_ERR_INVALID, "fastconformer_layers_packed: bad shape");
  if (total == 0 || num_segs == 0) return OASR_OK;
  OB_REQUIRE(rows && out && rel_table && cu_seqlens && bias_offsets && workspace, OASR_ERR_INVALID,
             "fastconformer_layers_packed: null pointer argument");
  OB_REQUIRE(table_rows >= 2 * max_seg - 1 && table_rows % 8 == 0, OASR_ERR_INVALID,
             "fastconformer_layers_packed: the position table needs >= 2*max_seg-1 rows, a multiple of 8 (got %lld for %lld frames)",
             (long long)table_rows, (long long)max_seg);
  OB_REQUIRE(is_aligned(workspace, 256), OASR_ERR_ALIGN, "fastconformer_layers_packed: workspace must be 256-byte aligned");
  FcWorkspace w = fc_carve(m, total, table_rows, bias_numel, static_cast<uint8_t*>(workspace));
  OB_REQUIRE(workspace_bytes >= w.bytes, OASR_ERR_INVALID, "fastconformer_layers_packed: workspace of %lld bytes, %lld needed",
             (long long)workspace_bytes, (long long)w.bytes);
  const int64_t M = total, C = m.hidden, F = m.ffn, H = m.heads, D = C / H, L = m.num_layers, Pp = table_rows;
  const int dt = m.dtype;
  const size_t es = 2;
  const double scale = 1.0 / std::sqrt(static_cast<double>(D));
  const int64_t chunk = m.right_context + 1;
  const int64_t left_chunks = m.left_context >= 0 ? m.left_context / chunk : max_seg;
  const oasr_b200_fastconformer_layer* ly = m.layers;
  const double eps = m.eps;

  // One Linear: 16-bit GEMM, or per-token quantisation of the input followed by the 8-bit GEMM on the layer's
  // pre-quantised weight `qi` (order of oasr_b200_fastconformer_layer::q_w).
  const int qk = m.quant_kind;
  OB_REQUIRE(qk == 0 || qk == OASR_Q8_FP8_E4M3 || qk == OASR_Q8_INT8, OASR_ERR_INVALID, "fastconformer_layers_packed: bad quant_kind %d", qk);
#define FC_LINEAR(out, in, wt, bs, lay, qi, N, K, act, glu)                                                           \
  do {                                                                                                                \
    if (qk == 0) {                                                                                                    \
      if (glu) FC_STEP(oasr_b200_gemm_glu(out, in, wt, bs, M, N, K, dt, stream));                                       \
      else FC_STEP(oasr_b200_gemm(out, in, wt, bs, M, N, K, act, dt, stream));                                          \
    } else {                                                                                                          \
      OB_REQUIRE((lay).q_w[qi] && (lay).q_s[qi], OASR_ERR_INVALID, "fastconformer_layers_packed: layer without 8-bit weight %d", qi); \
      FC_STEP(oasr_b200_quantize_rows(w.q8, w.qs, in, M, K, qk, dt, stream));                                          \
      FC_STEP(oasr_b200_gemm_q8(out, w.q8, w.qs, (lay).q_w[qi], (lay).q_s[qi], bs, M, N, K, act, glu, qk, dt, stream)); \
    }                                                                                                                 \
  } while (0)

  // A Linear whose input h was produced (and, with an 8-bit kind, already quantised into w.q8 / w.qs) by the add + norm
  // directly before it.
#define FC_LINEAR_H(out, wt, bs, lay, qi, N, K, act, glu)                                                            \
  do {                                                                                                                \
    if (qk == 0) {                                                                                                    \
      FC_LINEAR(out, w.h, wt, bs, lay, qi, N, K, act, glu);                                                           \
    } else {                                                                                                          \
      OB_REQUIRE((lay).q_w[qi] && (lay).q_s[qi], OASR_ERR_INVALID, "fastconformer_layers_packed: layer without 8-bit weight %d", qi); \
      FC_STEP(oasr_b200_gemm_q8(out, w.q8, w.qs, (lay).q_w[qi], (lay).q_s[qi], bs, M, N, K, act, glu, qk, dt, stream)); \
    }                                                                                                                 \
  } while (0)
  // add + norm into w.h, and with an 8-bit kind the quantised row for the Linear that follows
#define FC_ADD_NORM(res_in_, y_, alpha_, mode_, wa, ba, wb, bb)                                                       \
  FC_STEP(oasr_b200_add_norm_f32_q8(w.h, res, res_in_, y_, alpha_, mode_, wa, ba, wb, bb, M, C, eps, 0,                \
                                    qk ? w.q8 : nullptr, qk ? w.qs : nullptr, qk, dt, stream))

  // the input rows (16-bit, or fp32 when rows_f32) start the fp32 residual stream; h = LN_ff1(x) of the first layer in
  // the same kernel
  float* res = w.res;
  if (rows_f32) {
    FC_ADD_NORM(static_cast<const float*>(rows), nullptr, 0.0, 0, ly[0].norm_ff1_w, ly[0].norm_ff1_b, nullptr, nullptr);
  } else {
    FC_ADD_NORM(nullptr, rows, 1.0, 0, ly[0].norm_ff1_w, ly[0].norm_ff1_b, nullptr, nullptr);
  }
  for (int64_t i = 0; i < L; ++i) {
    const oasr_b200_fastconformer_layer& l = ly[i];
    // macaron feed-forward: x += 0.5 * W2 silu(W1 h)
    FC_LINEAR_H(w.a_ffn, l.ff1_w1, l.ff1_b1, l, 0, F, C, OASR_ACT_SWISH, 0);
    FC_LINEAR(w.y, w.a_ffn, l.ff1_w2, l.ff1_b2, l, 1, C, F, OASR_ACT_NONE, 0);
    FC_ADD_NORM(res, w.y, 0.5, 0, l.norm_att_w, l.norm_att_b, nullptr, nullptr);
    // attention: [q+u | q+v | k | v] of every row, position scores (q+v) . rel_k^T per head, shifted bias, attention
    FC_LINEAR_H(w.qkv4, l.qkv4_w, l.qkv4_b, l, 2, 4 * C, C, OASR_ACT_NONE, 0);
    FC_STEP(oasr_b200_gemm(w.rel_k, rel_table, l.rel_w, nullptr, Pp, C, C, OASR_ACT_NONE, dt, stream));
    FC_STEP(oasr_b200_bmm_strided(w.bd, w.qkv4 + C * es, w.rel_k, H, M, Pp, D, 4 * C, D, C, D, dt, stream));
    FC_STEP(oasr_b200_relshift_bias_packed(w.bias, w.bd, cu_seqlens, bias_offsets, num_segs, H, M, max_seg, Pp, scale, chunk,
                                           left_chunks, m.mask_floor, dt, stream));
    FC_STEP(oasr_b200_fmha_varlen_strided(w.att, w.qkv4, w.qkv4 + 2 * C * es, w.qkv4 + 3 * C * es, 4 * C, 4 * C, 4 * C, w.bias,
                                          bias_offsets, 1, 1, cu_seqlens, cu_seqlens, num_segs, M, M, max_seg, H, H, D, scale, dt,
                                          stream));
    FC_LINEAR(w.y, w.att, l.o_w, l.o_b, l, 3, C, C, OASR_ACT_NONE, 0);
    FC_ADD_NORM(res, w.y, 1.0, 0, l.norm_conv_w, l.norm_conv_b, nullptr, nullptr);
    // conv module: pointwise + GLU, causal depthwise conv per segment, LayerNorm + SiLU, pointwise
    FC_LINEAR_H(w.g, l.pw1_w, l.pw1_b, l, 4, C, C, OASR_ACT_NONE, 1);
    FC_STEP(oasr_b200_depthwise_conv1d_packed_causal(w.cv, w.g, l.dw_w, l.dw_b, cu_seqlens, num_segs, max_seg, C, m.kernel, -1, dt,
                                                     stream));
    FC_STEP(oasr_b200_layer_norm_activation(w.g, w.cv, l.conv_norm_w, l.conv_norm_b, M, C, 1e-5, OASR_ACT_SWISH, dt, stream));
    FC_LINEAR(w.y, w.g, l.pw2_w, l.pw2_b, l, 5, C, C, OASR_ACT_NONE, 0);
    FC_ADD_NORM(res, w.y, 1.0, 0, l.norm_ff2_w, l.norm_ff2_b, nullptr, nullptr);
    // second feed-forward, norm_out, then the next layer's first pre-norm in the same kernel
    FC_LINEAR_H(w.a_ffn, l.ff2_w1, l.ff2_b1, l, 6, F, C, OASR_ACT_SWISH, 0);
    FC_LINEAR(w.y, w.a_ffn, l.ff2_w2, l.ff2_b2, l, 7, C, F, OASR_ACT_NONE, 0);
    if (i + 1 < L) {
      FC_ADD_NORM(res, w.y, 0.5, 2, l.norm_out_w, l.norm_out_b, ly[i + 1].norm_ff1_w, ly[i + 1].norm_ff1_b);
    } else {
      FC_STEP(oasr_b200_add_norm_f32(w.h, out, res, w.y, 0.5, 2, l.norm_out_w, l.norm_out_b, l.norm_out_w, l.norm_out_b, M, C, eps, 0,
                                     dt, stream));
    }
  }
  return OASR_OK;
}

}  // extern "C"
