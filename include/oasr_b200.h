/*
 * oasr_b200.h -- C-ABI of the B200 (sm_100a) encoder hot path.
 *
 * One shared library, liboasr_b200.so, exports every function below with C
 * linkage, plain device pointers and sizes.  Each entry point replaces one
 * TVM-FFI launcher of the reference (cited per function as <file>:<line> in
 * the reference tree).  Conventions shared by all entry points, following
 * the reference's launcher conventions (csrc/tvm_ffi_utils.h:36-168):
 *
 *   - the OUTPUT pointer comes first, inputs follow, optional tensors are
 *     nullable pointers, scalars are int64_t / double / int;
 *   - the caller owns and allocates every buffer; nothing is allocated per
 *     call, so every entry point may be recorded into a CUDA graph;
 *   - work is enqueued on the `stream` argument (a cudaStream_t passed as
 *     void*; NULL means the legacy default stream) and the call returns
 *     without synchronising;
 *   - the return value is 0 on success or a negative OASR_ERR_* code; no
 *     launch has happened when the code is negative.  The message for the
 *     calling thread is available from oasr_b200_last_error();
 *   - all pointers are device pointers unless the parameter comment says
 *     "host"; tensors are dense row-major with the trailing dimension
 *     contiguous;
 *   - `dtype` is an oasr_dtype id naming the element type of the activation
 *     tensors (and of weights unless stated otherwise).
 */
#ifndef OASR_B200_H_
#define OASR_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define OASR_API __declspec(dllexport)
#else
#define OASR_API __attribute__((visibility("default")))
#endif

/* Element type ids. */
enum oasr_dtype {
  OASR_DT_F32 = 0,
  OASR_DT_F16 = 1,
  OASR_DT_BF16 = 2,
  OASR_DT_FP8_E4M3 = 3,
  OASR_DT_INT8 = 4
};

/* Activation ids: the reference's ActivationType (include/oasr/common/types.h:49-56,
 * oasr/functionals/activation.py:13-25).  OASR_ACT_NONE has no reference id. */
enum oasr_activation {
  OASR_ACT_NONE = -1,
  OASR_ACT_RELU = 0,
  OASR_ACT_GELU_TANH = 1,
  OASR_ACT_SWISH = 2,
  OASR_ACT_GELU_ERF = 4
};

/* Status codes. */
enum oasr_status {
  OASR_OK = 0,
  OASR_ERR_INVALID = -1,   /* bad shape / size / null pointer            */
  OASR_ERR_DTYPE = -2,     /* element type not supported by this op      */
  OASR_ERR_ALIGN = -3,     /* pointer or extent violates an alignment    */
  OASR_ERR_CUDA = -4,      /* a CUDA runtime / driver call failed        */
  OASR_ERR_UNSUPPORTED = -5,
  OASR_ERR_DEVICE_WAIT = -6 /* a bounded device-side wait gave up        */
};

/* ---- library ---------------------------------------------------------- */

/* "oasr_b200 <version> sm_100a" */
OASR_API const char* oasr_b200_version(void);
/* Message of the last failing call made by this thread ("" if none). */
OASR_API const char* oasr_b200_last_error(void);
/* Reads and clears the device-side status word that kernels with bounded
 * waits (TMA / tcgen05 pipelines) write when a wait gives up.  Synchronises
 * `stream`.  Returns 0 when no kernel reported a problem, else
 * OASR_ERR_DEVICE_WAIT with the raw word in *word (nullable). */
OASR_API int oasr_b200_device_status(uint32_t* word /*host*/, void* stream);
/* Self-test of the bounded-wait path (no reference counterpart): launches one
 * small CTA in which one role waits, for at most `poll_limit` polls (64 ..
 * 2^20), on an mbarrier that nothing arrives on, and a second role waits on a
 * barrier the first would have signalled.  Both must give up, set bit 8
 * (0x100) of the device status word, release their tensor memory and return;
 * `report` (device, nullable, zero it first) receives 1 | 2 for the two
 * roles.  The next oasr_b200_device_status call then returns
 * OASR_ERR_DEVICE_WAIT and clears the word; kernels launched afterwards run
 * normally.  Nothing faults or hangs. */
/* Diagnostics (no reference counterpart): with a device buffer of 64 uint64
 * set, the first CTA of every following launch of the instrumented kernels
 * (the fused Linear+add+norm kernel, the packed relative-position attention
 * kernel) writes SM clock stamps of its phases there; NULL (the default)
 * switches it off.  Slots of the Linear+add+norm kernel: 0 start, 1 first
 * operand load, 2 first operands landed, 3 last MMA committed, 4 accumulator
 * seen by the epilogue, 5 / 6 / 7 ends of the epilogue passes, 8 stores
 * drained, 9 exit.  Attention kernel: 0 start, 1 set-up done, 2 first scores
 * seen, 3 + j end of the softmax of key tile j (j < 40), 60 output written. */
OASR_API int oasr_b200_trace_buffer(void* device_buffer /*nullable*/);
OASR_API int oasr_b200_selftest_bounded_wait(int64_t poll_limit, uint32_t* report /*device, nullable*/,
                                             void* stream);
/* Number of kernels this library has launched in this process so far
 * (host-side counter, one per launch; no reference counterpart). */
OASR_API unsigned long long oasr_b200_launch_count(void);
/* Process-wide integer tunables.  "gemm_bn": 0 = heuristic tile width, or 64 /
 * 128 / 256 to force it; "gemm_pairs": 1 lets large dense GEMMs run
 * on CTA pairs (tcgen05 cta_group::2), 0 (default) keeps single-CTA tiles;
 * "dwconv_path": 0 (default) = register-streaming depthwise conv where it
 * applies, 1 = the shared-memory tiled kernel; "fmha_chunk_path": 1 (default)
 * = paged rel-pos attention with <= 16 query frames runs the warp-per-(stream,
 * head) kernel, 0 = always the 128-row tcgen05 kernel; "fmha_relpos_path": 1 (default) =
 * packed relative-position attention on the two-CTAs-per-SM kernel (64-key tiles),
 * 0 = on the general kernel; "lsm_path": the CTC head, 0 (default) = by size, 1 = the fused two-sweep
 * kernel, 2 = fp32 logits GEMM + in-place row log-softmax kernel (fp32 output only); "pdl": 1 launches
 * the GEMM, attention, add+norm, depthwise-conv and quantise kernels with
 * programmatic stream serialisation (their set-up overlaps the previous
 * kernel's tail), 0 (default) = plain stream order (no reference counterpart; the reference selects tiles
 * through its JIT variant names, oasr/jit/gemm.py:863-880). */
OASR_API int oasr_b200_set_tunable(const char* name, int value);

/* ---- norms ------------------------------------------------------------ */
/* rows = product of leading dims, hidden = trailing dim.  weight/bias and the
 * batch-norm statistics have `hidden` elements of the activation dtype. */

/* out = LN(in).  Replaces layernorm (csrc/norm_jit_binding.cu:9, kernel
 * include/oasr/norm.cuh:28-93). */
OASR_API int oasr_b200_layer_norm(void* out, const void* in, const void* weight,
                                  const void* bias /*nullable*/, int64_t rows, int64_t hidden,
                                  double eps, int dtype, void* stream);
/* out = act(LN(in)).  Replaces layernorm_activation (csrc/norm_jit_binding.cu:28). */
OASR_API int oasr_b200_layer_norm_activation(void* out, const void* in, const void* weight,
                                             const void* bias /*nullable*/, int64_t rows,
                                             int64_t hidden, double eps, int activation, int dtype,
                                             void* stream);
/* out = LN(residual + alpha*in), sum kept in fp32.  Replaces addlayernorm
 * (csrc/norm_jit_binding.cu:17, kernel include/oasr/norm.cuh:307-382). */
OASR_API int oasr_b200_add_layer_norm(void* out, const void* in, const void* residual,
                                      const void* weight, const void* bias /*nullable*/,
                                      int64_t rows, int64_t hidden, double eps, double alpha,
                                      int dtype, void* stream);
/* As above and residual_out = cast(residual + alpha*in), rounded once.
 * Replaces addlayernorm_residual (csrc/norm_jit_binding.cu:19, kernel
 * include/oasr/norm.cuh:396-484). */
OASR_API int oasr_b200_add_layer_norm_residual(void* out, void* residual_out, const void* in,
                                               const void* residual, const void* weight,
                                               const void* bias /*nullable*/, int64_t rows,
                                               int64_t hidden, double eps, double alpha, int dtype,
                                               void* stream);
/* out = RMSNorm(in) (+bias).  Replaces rmsnorm (csrc/norm_jit_binding.cu:11,
 * kernel include/oasr/norm.cuh:99-147). */
OASR_API int oasr_b200_rms_norm(void* out, const void* in, const void* weight,
                                const void* bias /*nullable*/, int64_t rows, int64_t hidden,
                                double eps, int dtype, void* stream);
/* Replaces rmsnorm_activation (csrc/norm_jit_binding.cu:30). */
OASR_API int oasr_b200_rms_norm_activation(void* out, const void* in, const void* weight,
                                           const void* bias /*nullable*/, int64_t rows,
                                           int64_t hidden, double eps, int activation, int dtype,
                                           void* stream);
/* Replaces addrmsnorm (csrc/norm_jit_binding.cu:22). */
OASR_API int oasr_b200_add_rms_norm(void* out, const void* in, const void* residual,
                                    const void* weight, const void* bias /*nullable*/, int64_t rows,
                                    int64_t hidden, double eps, double alpha, int dtype,
                                    void* stream);
/* Replaces addrmsnorm_residual (csrc/norm_jit_binding.cu:24). */
OASR_API int oasr_b200_add_rms_norm_residual(void* out, void* residual_out, const void* in,
                                             const void* residual, const void* weight,
                                             const void* bias /*nullable*/, int64_t rows,
                                             int64_t hidden, double eps, double alpha, int dtype,
                                             void* stream);
/* Residual-stream step of the fused encoder layer: the residual stream is
 * fp32, sub-layer outputs y and normalised activations h are 16-bit.
 *   s = res_in + alpha * y   (either operand nullable = absent)
 *   mode 0: res_out = s (nullable), h = LN_a(s)
 *   mode 1: res_out = s (nullable), h = s * w_a + b_a with fp32 w_a/b_a (a
 *           folded inference BatchNorm used as pre-norm)
 *   mode 2: res_out = LN_a(s), h = LN_b(res_out)
 * It is the reference's `x = residual + alpha*sub(x); x = norm(x)` pairs
 * (oasr/models/conformer/model.py:722-751; fused form :602-663) with the sum
 * never rounded to 16 bits.  res_out may alias res_in.  hidden % 8 == 0,
 * hidden <= 2048.  With split_out = 1, h rows are 2*hidden wide and hold
 * [hi | lo] with hi = round16(h), lo = round16(h - hi): multiplied by a
 * weight laid out as [W | W] (W in 16 bits, twice) this gives the product with
 * the INPUT at close to fp32 precision (used for the CTC head, whose log-probs
 * are compared with an fp32 path: rounding the head's input to bf16 alone costs
 * 4e-4 mean-abs there, rounding its weight 1e-4). */
OASR_API int oasr_b200_add_norm_f32(void* h_out, float* res_out /*nullable*/,
                                    const float* res_in /*nullable*/,
                                    const void* y /*nullable*/, double alpha, int mode,
                                    const void* w_a, const void* b_a, const void* w_b /*mode 2*/,
                                    const void* b_b /*mode 2*/, int64_t rows, int64_t hidden,
                                    double eps, int split_out, int dtype, void* stream);
/* The same, with the h row also written in 8 bits for a following 8-bit GEMM
 * (no reference counterpart): q_out (rows, hidden) one byte per element and
 * q_scale fp32[rows] are what oasr_b200_quantize_rows(h) would produce -- the
 * scale is amax of the 16-bit h row / 448 (q_kind 1, fp8 e4m3) or / 127
 * (q_kind 2, int8) -- bit for bit, so the per-token quantisation launch and
 * its second read of h disappear.  q_out = NULL: exactly
 * oasr_b200_add_norm_f32.  split_out must be 0 with an 8-bit output. */
OASR_API int oasr_b200_add_norm_f32_q8(void* h_out, float* res_out /*nullable*/,
                                       const float* res_in /*nullable*/,
                                       const void* y /*nullable*/, double alpha, int mode,
                                       const void* w_a, const void* b_a, const void* w_b /*mode 2*/,
                                       const void* b_b /*mode 2*/, int64_t rows, int64_t hidden,
                                       double eps, int split_out, void* q_out /*nullable*/,
                                       float* q_scale, int q_kind, int dtype, void* stream);
/* Linear + residual step + norm in one kernel (no single reference
 * counterpart: it replaces gemm (csrc/gemm_jit_binding.cu:9-12) followed by
 * addlayernorm_residual (csrc/norm_jit_binding.cu:18-20, kernel
 * include/oasr/norm.cuh:396-484) as the layer composes them,
 * oasr/models/conformer/model.py:722-751):
 *   y = A[M,K] . B[N,K]^T + bias (fp32, never rounded), s = res_in + alpha*y,
 * then `mode` / w_a, b_a, w_b, b_b / split_out exactly as oasr_b200_add_norm_f32
 * (h_out 16-bit row-major [M,N] or [M,2N]).  The fp32 residual stream
 * (res_in, res_out; res_out may alias res_in) is NOT row-major here: it is
 * private to a chain of these calls and uses a blocked layout the kernel can
 * move without staging -- rows padded to a multiple of 32, blocks of 32 rows x
 * 32 columns stored band-major ((row/32) * (N/32) + col/32) * 1024 floats,
 * and inside a block element (row l, column 4j+e) at float (j*32 + l)*4 + e;
 * the buffers hold roundup32(M) * N floats.
 * The output row must fill tensor memory: N = 128, 256 or 512
 * (oasr_b200_gemm_add_norm_supported); other widths return
 * OASR_ERR_UNSUPPORTED and the caller composes gemm + add_norm_f32. */
OASR_API int oasr_b200_gemm_add_norm_f32(void* h_out, float* res_out /*nullable unless mode 2*/,
                                         const float* res_in /*nullable*/, const void* A,
                                         const void* B, const void* bias /*nullable*/, int64_t M,
                                         int64_t N, int64_t K, double alpha, int mode,
                                         const void* w_a, const void* b_a,
                                         const void* w_b /*mode 2*/, const void* b_b /*mode 2*/,
                                         double eps, int split_out, int dtype, void* stream);
OASR_API int oasr_b200_gemm_add_norm_supported(int64_t N, int64_t K);

/* Inference batch norm over channels-last rows, optional activation
 * (activation = OASR_ACT_NONE for plain BN).  Replaces batchnorm1d,
 * batchnorm_activation and batchnorm_swish (csrc/norm_jit_binding.cu:13,32,35;
 * kernels include/oasr/norm.cuh:153-187,779-813). */
OASR_API int oasr_b200_batch_norm(void* out, const void* in, const void* weight, const void* bias,
                                  const void* running_mean, const void* running_var, int64_t rows,
                                  int64_t channels, double eps, int activation, int dtype,
                                  void* stream);

/* ---- activations ------------------------------------------------------ */
/* out[r, c] = in[r, c] * sigmoid(in[r, channels + c]); in has 2*channels
 * columns.  Replaces glu (csrc/activation_jit_binding.cu:9, kernel
 * include/oasr/activation.cuh:25-60). */
OASR_API int oasr_b200_glu(void* out, const void* in, int64_t rows, int64_t channels, int dtype,
                           void* stream);
/* out = in * sigmoid(in).  Replaces swish (csrc/activation_jit_binding.cu:13,
 * kernel include/oasr/activation.cuh:66-87). */
OASR_API int oasr_b200_swish(void* out, const void* in, int64_t numel, int dtype, void* stream);

/* ---- depthwise conv1d -------------------------------------------------- */
/* in (batch, seq_len, channels), weight (kernel_size, channels), out
 * (batch, out_len, channels) with out_len = seq_len + pad_left + pad_right -
 * kernel_size + 1.  `mask` (nullable) is (batch, seq_len) in the activation
 * dtype (mask_is_bool = 0) or one byte per frame (mask_is_bool = 1) and is
 * applied to the input and to the output; add_input adds the (masked) input
 * frame before the output mask (both need out_len == seq_len).  activation is
 * OASR_ACT_NONE or OASR_ACT_SWISH.  Replaces depthwise_conv1d and
 * depthwise_conv1d_silu (csrc/conv_jit_binding.cu:9-13, kernels
 * include/oasr/conv/conv1d.cuh:23-181). */
OASR_API int oasr_b200_depthwise_conv1d(void* out, const void* in, const void* weight,
                                        const void* bias /*nullable*/, int64_t batch,
                                        int64_t seq_len, int64_t channels, int64_t kernel_size,
                                        int64_t pad_left, int64_t pad_right,
                                        const void* mask /*nullable*/, int mask_is_bool,
                                        int add_input, int activation, int dtype, void* stream);
/* Depthwise conv over PACKED segments: in/out (total, channels) rows,
 * segment s = rows [cu_seqlens[s], cu_seqlens[s+1]), each convolved alone with
 * (kernel_size-1)/2 zero frames on both sides -- the gapped-buffer scatter /
 * conv / gather of ConvolutionModule._forward_packed_noncausal
 * (oasr/models/conformer/model.py:223-233) without the gapped buffer.
 * post_scale/post_shift (nullable, fp32[channels]) apply y*scale+shift after
 * the bias (a folded inference BatchNorm, oasr/layers/norm.py:64-74), then the
 * activation.  right_fill (nullable, fp32[channels]) with fill_frames
 * (int32[S]) makes the first fill_frames[s] frames past a segment's end read
 * right_fill instead of zero: the value padded rows carry in the padded-batch
 * path, where they are zeroed BEFORE pointwise_conv1 (model.py:176-197). */
OASR_API int oasr_b200_depthwise_conv1d_packed(void* out, const void* in, const void* weight,
                                               const void* bias /*nullable*/,
                                               const float* post_scale /*nullable*/,
                                               const float* post_shift /*nullable*/,
                                               const float* right_fill /*nullable*/,
                                               const int32_t* fill_frames /*nullable*/,
                                               const int32_t* cu_seqlens, int64_t num_segs,
                                               int64_t max_seg_len, int64_t channels,
                                               int64_t kernel_size, int activation, int dtype,
                                               void* stream);
/* The same over packed segments with all kernel_size-1 zero frames on the LEFT (a causal conv: frame t
 * of a segment reads frames t-kernel_size+1 .. t of that segment), the packed form of the FastConformer conv module's
 * depthwise conv (oasr/models/nemotron/encoder.py CausalConv1d, padding (kernel_size-1, 0)). */
OASR_API int oasr_b200_depthwise_conv1d_packed_causal(void* out, const void* in, const void* weight,
                                                      const void* bias /*nullable*/, const int32_t* cu_seqlens,
                                                      int64_t num_segs, int64_t max_seg_len, int64_t channels,
                                                      int64_t kernel_size, int activation, int dtype, void* stream);
/* oasr_b200_depthwise_conv1d with a per-channel affine (fp32 post_scale /
 * post_shift, a folded inference BatchNorm) applied after the bias and before
 * the activation: depthwise_conv followed by BatchNormActivation of the conv
 * module (oasr/models/conformer/model.py:193-194) in one kernel. */
OASR_API int oasr_b200_depthwise_conv1d_affine(void* out, const void* in, const void* weight,
                                               const void* bias /*nullable*/,
                                               const float* post_scale /*nullable*/,
                                               const float* post_shift /*nullable*/, int64_t batch,
                                               int64_t seq_len, int64_t channels,
                                               int64_t kernel_size, int64_t pad_left,
                                               int64_t pad_right, int activation, int dtype,
                                               void* stream);
/* Conv-module left context of streaming chunks (ConvolutionModule.forward with
 * a cache, oasr/models/conformer/model.py:176-190, plus SlotTensor.gather /
 * scatter, oasr/cache/state.py:88-94): xcat[b] = [state[slot_ids[b]] ; x[b]]
 * with state (num_slots, state_len, channels), x (B, T, channels), xcat
 * (B, state_len + T, channels); afterwards state[slot_ids[b]] is set to the
 * last state_len rows of xcat[b].  A slot id outside [0, num_slots) reads as
 * a zero left context and is not written back. */
OASR_API int oasr_b200_conv_state_concat(void* xcat, void* state, int64_t num_slots,
                                         const int64_t* slot_ids, const void* x, int64_t B,
                                         int64_t state_len, int64_t T, int64_t channels, int dtype,
                                         void* stream);
/* Streaming causal depthwise conv with a rolling state: in (batch, seq_len,
 * channels), state (batch, kernel_size-1, channels) updated in place to the
 * last kernel_size-1 frames of [state, in], weight (channels, kernel_size).
 * Replaces causal_conv1d (csrc/conv_jit_binding.cu:14, kernels
 * include/oasr/conv/conv1d.cuh:187-269,450-473). */
OASR_API int oasr_b200_causal_conv1d(void* out, const void* in, void* state, const void* weight,
                                     const void* bias /*nullable*/, int64_t batch, int64_t seq_len,
                                     int64_t channels, int64_t kernel_size, int dtype,
                                     void* stream);

/* ---- subsampling front end --------------------------------------------- */
/* First Conv2d of the subsampling stack (one input channel): out (B,T1,F1,C)
 * NHWC 16-bit = relu(conv(in (B,T,F) fp32, weight (C,k,k) fp32, stride) + bias),
 * T1 = (T-k)/stride+1, F1 = (F-k)/stride+1.  t1_limit (nullable, int32[B])
 * skips output frames >= t1_limit[b] (frames only padding would consume).
 * Replaces the first Conv2dActivation of Conv2dSubsampling
 * (oasr/models/conformer/model.py:433-444, oasr/layers/conv.py:652-670). */
OASR_API int oasr_b200_subsample_conv1(void* out, const float* in, const float* weight,
                                       const float* bias, const int32_t* t1_limit /*nullable*/,
                                       int64_t B, int64_t T, int64_t F, int64_t C, int64_t kernel,
                                       int64_t stride, int dtype, void* stream);
/* The same convolution written in the parity-split layout the second
 * convolution reads: out (B, ceil(T1/2), 4, ceil(F1/2), C) with plane
 * (t1 & 1) * 2 + (f1 & 1) and rows (t1 / 2, f1 / 2); 3x3 taps, stride 2 only.
 * Positions no output frame < t1_limit[b] needs are left unwritten (no
 * reference counterpart: the reference keeps NHWC between the convolutions,
 * oasr/models/conformer/model.py:433-449). */
OASR_API int oasr_b200_subsample_conv1_s2d(void* out, const float* in, const float* weight,
                                           const float* bias, const int32_t* t1_limit /*nullable*/,
                                           int64_t B, int64_t T, int64_t F, int64_t C, int dtype,
                                           void* stream);
/* Depthwise 3x3 / stride-2 Conv2d on NHWC 16-bit data (B, T, F, C) with pad_lo zero columns before and pad_hi
 * after on the frequency axis and time_pad_lo / time_pad_hi zero frames on the time axis (offline: the same (2, 1)
 * on both axes; a streaming chunk passes (0, 0) in time and prepends its cached two frames instead,
 * oasr/models/nemotron/subsampling.py:156-189): out (B, To, Fo, C), To = (T+time_pad_lo+time_pad_hi-3)/2+1,
 * Fo = (F+pad_lo+pad_hi-3)/2+1.
 * weight (C, 3, 3), bias nullable (C); output frames >= out_len[b] (nullable int32[B]) are written as zeros and
 * input frames >= in_len[b] (nullable int32[B]) are read as zeros, whatever the buffer holds there.
 * The depthwise half of a FastConformer subsampling stage (oasr/models/nemotron/subsampling.py:39-53, 204-224);
 * its pointwise half is a GEMM over the (b, t, f) rows. */
OASR_API int oasr_b200_depthwise_conv2d_k3s2(void* out, const void* in, const void* weight,
                                             const void* bias /*nullable*/, const int32_t* out_len /*nullable*/,
                                             const int32_t* in_len /*nullable*/, int64_t B, int64_t T, int64_t F, int64_t C, int64_t pad_lo,
                                             int64_t pad_hi, int64_t time_pad_lo, int64_t time_pad_hi, int dtype, void* stream);
/* Second Conv2d of the subsampling stack (3x3, stride 2, C -> N channels, +
 * bias + ReLU) as an implicit GEMM on the tensor cores, writing only valid
 * output frames, already packed: out (total_frames, F2, N) with utterance b's
 * frames at rows [cu_frames[b], cu_frames[b+1]) (cu_frames: int32[B+1] on the
 * device), F2 = (F1-3)/2+1.  x1 is the parity-split output of
 * oasr_b200_subsample_conv1_s2d; w2 is (N, 3, 3, C) = (N, 9*C) row-major (taps
 * outermost, input channels innermost).  Replaces the second Conv2dActivation
 * of Conv2dSubsampling (oasr/models/conformer/model.py:445-449, CUTLASS implicit
 * GEMM include/oasr/conv/conv2d.cuh:78-86) and the pack_hidden gather after it
 * (oasr/models/conformer/packing.py:204-216). */
OASR_API int oasr_b200_subsample_conv2(void* out, const void* x1, const void* w2,
                                       const void* bias /*nullable*/, const int32_t* cu_frames,
                                       int64_t B, int64_t T1, int64_t F1, int64_t C, int64_t N,
                                       int64_t total_frames, int dtype, void* stream);

/* ---- GEMM family (tcgen05 / TMEM / TMA) -------------------------------- */
/* D[M,N] = act(A[M,K] . B[N,K]^T + bias[N]); A, B, D row-major, fp16 or
 * bf16, fp32 accumulation in tensor memory, one rounding on store.  N and K
 * must be multiples of 8 and all pointers 16-byte aligned.  activation =
 * OASR_ACT_NONE gives the plain GEMM.  Replaces gemm / gemm_activation
 * (csrc/gemm_jit_binding.cu:9-16, launchers csrc/gemm.cu:40-115). */
OASR_API int oasr_b200_gemm(void* D, const void* A, const void* B, const void* bias /*nullable*/,
                            int64_t M, int64_t N, int64_t K, int activation, int dtype,
                            void* stream);
/* D[M, N + dup_cols] from A[M,K] . B[N,K]^T (no reference counterpart: it serves the fused q/q/k/v projection,
 * oasr/layers/attention/attention.py:323-386, whose two query blocks q+u and q+v differ only in their bias): the
 * first dup_cols columns of the product are stored twice, at output columns [0, dup_cols) and [dup_cols, 2*dup_cols),
 * the remaining columns after them; bias (16-bit, N + dup_cols entries, nullable) is indexed by OUTPUT column, so the
 * two copies carry different biases.  The result equals oasr_b200_gemm with the first dup_cols rows of B repeated, bit
 * for bit, at three quarters of the products.  N and dup_cols multiples of 256 (oasr_b200_gemm_dup_first_supported). */
OASR_API int oasr_b200_gemm_dup_first_supported(int64_t N, int64_t K, int64_t dup_cols);
OASR_API int oasr_b200_gemm_dup_first(void* D, const void* A, const void* B, const void* bias /*nullable*/,
                                      int64_t M, int64_t N, int64_t K, int64_t dup_cols, int dtype, void* stream);
/* 8-bit operand kinds of the GEMM (no reference counterpart: the reference has no quantised path,
 * oasr/layers/linear.py:7 only names a future one).  D (M,N) 16-bit =
 * act( (A_q . B_q^T) * a_scale[m] * b_scale[n] + bias[n] ), A_q (M,K) and B_q (N,K) one byte per
 * element: kind OASR_Q8_FP8_E4M3 = fp8 e4m3 operands with fp32 accumulation (tcgen05 kind::f8f6f4),
 * OASR_Q8_INT8 = signed int8 operands with int32 accumulation (kind::i8).  a_scale fp32[M] per
 * token, b_scale fp32[N] per output channel.  glu != 0: B_q has 2N rows (value | gate), b_scale
 * and bias 2N entries, D = value * sigmoid(gate).  K % 16 == 0, N % 8 == 0. */
#define OASR_Q8_FP8_E4M3 1
#define OASR_Q8_INT8 2
OASR_API int oasr_b200_gemm_q8(void* D, const void* A_q, const float* a_scale, const void* B_q,
                               const float* b_scale, const void* bias /*nullable, 16-bit*/,
                               int64_t M, int64_t N, int64_t K, int activation, int glu, int kind,
                               int out_dtype, void* stream);
/* Row-wise dynamic quantisation: q (rows, cols) one byte per element and scale fp32[rows] with
 * x ~ q * scale; scale = amax(row) / 448 (fp8 e4m3, round to nearest, saturating) or amax / 127
 * (int8, round to nearest).  x 16-bit, cols % 16 == 0.  Used per token on activations and per
 * output channel on weights (no reference counterpart). */
OASR_API int oasr_b200_quantize_rows(void* q, float* scale, const void* x, int64_t rows, int64_t cols,
                                     int kind, int dtype, void* stream);
/* Residual form used by the fused encoder layer (no reference counterpart as
 * an operator; it is the reference's `residual + alpha * Linear(x)` pair,
 * oasr/models/conformer/model.py:722-751, with the sum kept in fp32):
 * R_out[M,N] (fp32) = R_in[M,N] (fp32) + alpha * (A . B^T + bias).  R_out may
 * alias R_in; R_in == NULL reads as zeros (a plain fp32-output GEMM: how the
 * embedding projection starts the residual stream without a 16-bit rounding). */
OASR_API int oasr_b200_gemm_residual_f32(float* R_out, const float* R_in, const void* A,
                                         const void* B, const void* bias /*nullable*/, int64_t M,
                                         int64_t N, int64_t K, double alpha, int dtype,
                                         void* stream);
/* GLU form: B has 2*N rows; D[M,N] = (A.B[:N]^T + bias[:N]) * sigmoid(A.B[N:]^T
 * + bias[N:]).  Equals pointwise_conv1 followed by glu
 * (oasr/models/conformer/model.py:191-192) without the (M, 2N) round trip. */
OASR_API int oasr_b200_gemm_glu(void* D, const void* A, const void* B,
                                const void* bias /*nullable*/, int64_t M, int64_t N, int64_t K,
                                int dtype, void* stream);
/* D[b] = A[b] . B[b]^T for b < batch; A (batch,M,K), B (batch,N,K).  Replaces
 * bmm (csrc/bmm.cu, oasr/functionals/gemm.py:262-299). */
OASR_API int oasr_b200_bmm(void* D, const void* A, const void* B, int64_t batch, int64_t M,
                           int64_t N, int64_t K, int dtype, void* stream);
/* bmm over strided views: row m of A[b] starts at A + b*stride_a + m*lda elements (likewise B with stride_b, ldb),
 * unit stride along K; all four strides are multiples of 8 elements.  D is packed (batch, M, N).  Lets the per-head
 * operands of an attention layer be read in place from a (tokens, heads, head_dim) projection (batch = head:
 * stride = head_dim, ld = heads*head_dim) instead of being copied head-major first. */
OASR_API int oasr_b200_bmm_strided(void* D, const void* A, const void* B, int64_t batch, int64_t M,
                                   int64_t N, int64_t K, int64_t lda, int64_t stride_a, int64_t ldb,
                                   int64_t stride_b, int dtype, void* stream);
/* Grouped GEMM: rows [offsets[g-1], offsets[g]) of A (L,K) times B[g] (N,K)^T.
 * `offsets` is a DEVICE int32 array of `groups` cumulative END rows; it is
 * read on the device (no host synchronisation, unlike the reference launcher
 * csrc/group_gemm.cu:54-57).  Replaces group_gemm
 * (csrc/group_gemm_jit_binding.cu:8-12). */
OASR_API int oasr_b200_group_gemm(void* D, const void* A, const void* B, const int32_t* offsets,
                                  int64_t L, int64_t groups, int64_t N, int64_t K, int dtype,
                                  void* stream);
/* CTC head: out[M,N] = log_softmax(A.B^T + bias) over N, logits never leave
 * the chip.  out_dtype is OASR_DT_F32 or the activation dtype.  Replaces
 * gemm_log_softmax (csrc/gemm_log_softmax_jit_binding.cu:8-11, kernel pair
 * include/oasr/gemm/gemm_log_softmax.cuh:124-166).  `argmax` (nullable,
 * int32[M]) receives the index of the first maximum of each row.  With
 * out == NULL and argmax != NULL only that index is produced (the input of a
 * greedy CTC search, oasr/functionals/ctc_decode.py:359): one sweep over the
 * vocabulary and 4 bytes written per row instead of the N log-probs. */
OASR_API int oasr_b200_gemm_log_softmax(void* out, const void* A, const void* B,
                                        const void* bias /*nullable*/, int64_t M, int64_t N,
                                        int64_t K, int dtype, int out_dtype,
                                        int32_t* argmax /*nullable*/, void* stream);

/* ---- attention --------------------------------------------------------- */
/* Dense or paged multi-head attention, the reference's fmha
 * (oasr/functionals/attention.py:369-551; kernel contract
 * oasr/kernels/cute/attention/fmha_sm80.py:552, mask rules
 * oasr/kernels/cute/mask.py:102-117):
 *   out[b,h,i,:] = softmax_j(q[b,h,i,:].k[b,h/(H/Hkv),j,:]*scale + bias[b,h,i,j]) . v
 * q (B,H,Tq,D) and dense k, v (B,Hkv,Tk,D) may be strided views: *_strides
 * (nullable = canonical) are HOST arrays of 3 element strides {batch, head,
 * row}, each a multiple of 8, with unit stride along D.  out is canonical
 * (B,H,Tq,D).  bias (nullable) is in the activation dtype with element strides
 * bias_stride_b / _h / _q and unit stride along keys.  seqlens / seqstarts
 * (nullable, int32[B]) keep keys in [start, len); causal masks j > i.  Rows
 * with no visible key produce zeros.  Paged mode (block_table != NULL): k, v
 * are pools (num_blocks, block_size, Hkv, D), block_table is int32
 * (B, blocks_per_seq), Tk is ignored (= blocks_per_seq * block_size).
 * D is 64 or 128. */
OASR_API int oasr_b200_fmha(void* out, const void* q, const void* k, const void* v,
                            const int64_t* q_strides /*host, nullable*/,
                            const int64_t* k_strides /*host, nullable*/,
                            const int64_t* v_strides /*host, nullable*/,
                            const void* bias /*nullable*/, int64_t bias_stride_b,
                            int64_t bias_stride_h, int64_t bias_stride_q,
                            const int32_t* seqlens /*nullable*/,
                            const int32_t* seqstarts /*nullable*/,
                            const int32_t* block_table /*nullable*/, int64_t blocks_per_seq,
                            int64_t block_size, int64_t num_blocks, int64_t B, int64_t H,
                            int64_t Hkv, int64_t Tq, int64_t Tk, int64_t D, double scale,
                            int causal, int dtype, void* stream);
/* Same attention, but out is written token-major, (B, Tq, H, D): the layout the output projection reads, which the
 * reference reaches with transpose(1, 2).contiguous() after its fmha call (oasr/layers/attention/attention.py). */
OASR_API int oasr_b200_fmha_bthd(void* out, const void* q, const void* k, const void* v,
                                 const int64_t* q_strides /*host, nullable*/,
                                 const int64_t* k_strides /*host, nullable*/,
                                 const int64_t* v_strides /*host, nullable*/,
                                 const void* bias /*nullable*/, int64_t bias_stride_b,
                                 int64_t bias_stride_h, int64_t bias_stride_q,
                                 const int32_t* seqlens /*nullable*/,
                                 const int32_t* seqstarts /*nullable*/,
                                 const int32_t* block_table /*nullable*/, int64_t blocks_per_seq,
                                 int64_t block_size, int64_t num_blocks, int64_t B, int64_t H,
                                 int64_t Hkv, int64_t Tq, int64_t Tk, int64_t D, double scale,
                                 int causal, int dtype, void* stream);
/* fmha_varlen (next declaration) over strided views: rows of q / k / v are *_row_stride elements apart (0 = packed;
 * multiples of 8), heads D apart, so the slices of one fused projection are read in place; with bias_rows_padded8 the
 * rows of bias segment s are roundup8(Tk_s) elements apart and the offsets multiples of 8, which lets the kernel fetch
 * the bias in 16-byte pieces. */
OASR_API int oasr_b200_fmha_varlen_strided(void* out, const void* q, const void* k, const void* v,
                                           int64_t q_row_stride, int64_t k_row_stride, int64_t v_row_stride,
                                           const void* bias /*nullable*/, const void* bias_offsets /*nullable*/,
                                           int bias_offsets_is_i64, int bias_rows_padded8,
                                           const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                           int64_t num_segs, int64_t total_q, int64_t total_k,
                                           int64_t max_seqlen_q, int64_t H, int64_t Hkv, int64_t D,
                                           double scale, int dtype, void* stream);
/* Packed variable-length attention, the reference's fmha_varlen
 * (oasr/functionals/attention.py:592-693): q, out (total_q,H,D); k, v
 * (total_k,Hkv,D); cu_seqlens_* int32[S+1]; bias (nullable) flat, segment s is
 * (H,Tq_s,Tk_s) row-major at bias_offsets[s] (int64[S+1] if
 * bias_offsets_is_i64 else int32[S+1]). */
OASR_API int oasr_b200_fmha_varlen(void* out, const void* q, const void* k, const void* v,
                                   const void* bias /*nullable*/,
                                   const void* bias_offsets /*nullable*/, int bias_offsets_is_i64,
                                   const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                   int64_t num_segs, int64_t total_q, int64_t total_k,
                                   int64_t max_seqlen_q, int64_t H, int64_t Hkv, int64_t D,
                                   double scale, int dtype, void* stream);

/* Conformer relative-position attention over packed rows, the whole of
 * RelPositionMultiHeadedAttention._forward_packed between linear_qkv and
 * linear_out (oasr/layers/attention/attention.py:323-386) in one kernel:
 *   score[i,j] = ((q_i+u).k_j + (q_i+v).p_j) * scale,  j within i's segment,
 * where the position term is a second 64-wide K-atom of the same MMA instead
 * of a materialised (S,H,Tm,Tm) bias.  qkv4 is (total, 4*H*64) rows
 * [q+u | q+v | k | v] (the fused projection with the query block duplicated
 * and pos_bias_u / pos_bias_v folded into its bias); pos is linear_pos(pe)
 * (pos_rows >= max_seqlen rows of H*64, row stride pos_stride elements);
 * out is (total, H*64).  Head dim is 64. */
OASR_API int oasr_b200_fmha_varlen_relpos(void* out, const void* qkv4, const void* pos,
                                          int64_t pos_rows, int64_t pos_stride,
                                          const int32_t* cu_seqlens, int64_t num_segs,
                                          int64_t max_seqlen, int64_t total, int64_t H,
                                          double scale, int dtype, void* stream);
/* Work list for oasr_b200_fmha_varlen_relpos_planned: the items (segment, head, 128-row query tile) of a packed
 * batch, longest segments first, so that the persistent kernel's last items are short ones.  Built on the device
 * from cu_seqlens (no host synchronisation), once per batch; every layer's attention call reuses it.  plan must hold
 * oasr_b200_fmha_relpos_plan_bytes(num_segs, H, total) bytes, 16-byte aligned; num_segs <= 1024 (larger batches run
 * the unplanned entry point, which walks the items in (segment, head, tile) order).  No reference counterpart. */
OASR_API int64_t oasr_b200_fmha_relpos_plan_bytes(int64_t num_segs, int64_t H, int64_t total);
OASR_API int oasr_b200_fmha_relpos_plan(void* plan, int64_t plan_bytes, const int32_t* cu_seqlens,
                                        int64_t num_segs, int64_t H, int64_t total, void* stream);
/* oasr_b200_fmha_varlen_relpos following a plan (NULL = the unplanned order). */
OASR_API int oasr_b200_fmha_varlen_relpos_planned(void* out, const void* qkv4, const void* pos, int64_t pos_rows,
                                                  int64_t pos_stride, const int32_t* cu_seqlens,
                                                  int64_t num_segs, int64_t max_seqlen, int64_t total, int64_t H,
                                                  double scale, const void* plan /*nullable*/, int dtype,
                                                  void* stream);

/* Streaming form of the above: the attention of
 * RelPositionMultiHeadedAttention._forward_paged (oasr/layers/attention/attention.py:229-280)
 * after the chunk's keys/values were written to the page pools.  qkv4 is
 * (B*Tq, 4*H*64) rows [q+u | q+v | k | v] of the chunk, k_pool / v_pool are
 * (num_blocks, block_size, H, 64), block_table int32 (B, blocks_per_seq),
 * seqlens int32[B] the visible keys per stream INCLUDING the chunk.  Key j of
 * stream b takes its position term from row pos_start[b] + j of pos (the
 * projected positional table linear_pos(pe), pos_rows x H*64, row stride
 * pos_stride), i.e. pos_start = offset - cached frames
 * (oasr/models/conformer/model.py:993-1001).  out is (B*Tq, H*64).  Tq <= 128. */
OASR_API int oasr_b200_fmha_paged_relpos(void* out, const void* qkv4, void* k_pool, void* v_pool,
                                         const void* pos, int64_t pos_rows, int64_t pos_stride,
                                         const int32_t* pos_start, const int32_t* block_table,
                                         const int32_t* seqlens, int64_t B, int64_t Tq, int64_t H,
                                         int64_t blocks_per_seq, int64_t block_size,
                                         int64_t num_blocks, double scale, int dtype, void* stream);

/* The same attention over fp8 pages: k_pool / v_pool hold e4m3 codes (one byte per element, same
 * (num_blocks, block_size, H, 64) layout) and k_scale / v_scale fp32[H] the per-head scales
 * (value ~ code * scale).  The codes are converted to fp16 in shared memory; Tq <= 16, pages of 16 or
 * a multiple of 32 frames, at most 64 pages per stream (no reference counterpart: the reference keeps
 * 16-bit pages, oasr/cache/block_pool.py:33-41). */
OASR_API int oasr_b200_fmha_paged_relpos_fp8(void* out, const void* qkv4, void* k_pool, void* v_pool,
                                             const float* k_scale, const float* v_scale, const void* pos,
                                             int64_t pos_rows, int64_t pos_stride, const int32_t* pos_start,
                                             const int32_t* block_table, const int32_t* seqlens,
                                             int64_t B, int64_t Tq, int64_t H, int64_t blocks_per_seq,
                                             int64_t block_size, int64_t num_blocks, double scale,
                                             int dtype, void* stream);

/* Attention bias of the FastConformer layer in one pass: out (B, H, T, T) 16-bit with row stride ld_out >= T
 * elements (a multiple of 8 lets the attention kernel fetch it in 16-byte pieces; columns T..ld_out-1 are not written) =
 * visible(b,i,j) ? bd[b,h,i,(T-1)+j-i] * scale : floor_value, where bd (B, H, T, ld >= 2T-1; batch / head strides bd_stride_b / _h elements) are the scores of the
 * position-biased queries against the 2T-1 projected relative positions, and visible = key j in the query's chunked-
 * limited window (i/chunk - j/chunk in [0, left_chunks]) and j < lengths[b].  Replaces rel_shift, the scale, the
 * window & padding mask and the masked_fill of oasr/models/nemotron/encoder.py:82-96, 124-149, 343-348. */
OASR_API int oasr_b200_relshift_bias(void* out, const void* bd, const int32_t* lengths, int64_t B, int64_t H,
                                     int64_t T, int64_t ld, int64_t ld_out, int64_t bd_stride_b /*0 = H*T*ld*/,
                                     int64_t bd_stride_h /*0 = T*ld*/, double scale, int64_t chunk,
                                     int64_t left_chunks, double floor_value, int dtype, void* stream);
/* Streaming form of the same bias (NemotronRelPositionAttention.forward_chunk and NemotronEncoder._streaming_mask,
 * oasr/models/nemotron/encoder.py:362-410, 680-720): B streams with Tq new query frames each; the keys of stream b
 * are its cached[b] cached frames followed by the chunk, and offsets[b] encoder frames were emitted before this chunk.
 * bd (H, B*Tq, ld) holds the position-biased queries against the projected relative table built for Lmax >=
 * max(cached) + Tq (row p = distance Lmax-1-p; ld >= 2*Lmax-1).  out (B, H, Tq, ld_out) 16-bit: key j < cached[b]+Tq
 * gets bd[distance cached[b] + i - j] * scale when it lies in the query's chunked-limited window over ABSOLUTE frame
 * positions, else floor_value; columns past the stream's keys get floor_value.  The reference prefills a window of
 * constant length with masked placeholders instead; the visible keys and their distances are the same. */
OASR_API int oasr_b200_relshift_bias_stream(void* out, const void* bd, const int32_t* cached,
                                            const int32_t* offsets, int64_t B, int64_t H, int64_t Tq,
                                            int64_t ld, int64_t ld_out, int64_t Lmax, int64_t bd_stride_h,
                                            double scale, int64_t chunk, int64_t left_chunks,
                                            double floor_value, int dtype, void* stream);

/* Packed form of the same bias: bd (H, total, ld >= 2T-1) holds the position scores of every packed row (rows
 * [cu_seqlens[s], cu_seqlens[s+1]) are stream s, at most T frames), and segment s of out is (H, len_s, roundup8(len_s))
 * at bias_offsets[s] elements: the block-diagonal bias oasr_b200_fmha_varlen_strided reads with bias_rows_padded8 = 1.
 * Only the chunked-limited window is masked; a segment holds no padding keys. */
OASR_API int oasr_b200_relshift_bias_packed(void* out, const void* bd, const int32_t* cu_seqlens,
                                            const int64_t* bias_offsets, int64_t num_segs, int64_t H,
                                            int64_t total, int64_t T, int64_t ld, double scale, int64_t chunk,
                                            int64_t left_chunks, double floor_value, int dtype, void* stream);

/* ---- paged KV cache ---------------------------------------------------- */
/* paged_kv_write with quantisation: 16-bit k_new / v_new (element strides as below, unit stride along
 * D) are divided by their head's scale and stored as fp8 e4m3 codes (round to nearest even,
 * saturating) in one-byte pools of the same layout; same index rule (no reference counterpart). */
OASR_API int oasr_b200_paged_kv_write_fp8(void* k_pool, void* v_pool, const void* k_new, const void* v_new,
                                          const float* k_scale, const float* v_scale,
                                          const int32_t* block_table, const int32_t* offsets, int64_t B,
                                          int64_t Hkv, int64_t T, int64_t D, int64_t stride_b,
                                          int64_t stride_h, int64_t stride_t, int64_t blocks_per_seq,
                                          int64_t block_size, int64_t num_blocks, int dtype, void* stream);
/* Scatter a chunk of new keys/values into the page pools.  k_new, v_new are
 * (B, Hkv, T, D) with element strides (sb, sh, st) and unit stride along D;
 * logical position offsets[b] + t of stream b lands in physical row
 * block_table[b, pos / block_size] * block_size + pos % block_size of the
 * pools (num_blocks, block_size, Hkv, D).  Replaces
 * PagedKVCache.write_kv_chunk / flat_write_index
 * (oasr/cache/paged_kv.py:23-40,63-137).  elem_bytes is 1, 2 or 4. */
OASR_API int oasr_b200_paged_kv_write(void* k_pool, void* v_pool, const void* k_new,
                                      const void* v_new, const int32_t* block_table,
                                      const int32_t* offsets, int64_t B, int64_t Hkv, int64_t T,
                                      int64_t D, int64_t stride_b, int64_t stride_h,
                                      int64_t stride_t, int64_t blocks_per_seq,
                                      int64_t block_size, int64_t num_blocks, int elem_bytes,
                                      void* stream);
/* Gather pages into dense (B, Hkv, blocks_per_seq*block_size, D) tensors.
 * Replaces gather_paged_kv (oasr/functionals/attention.py:153-178). */
OASR_API int oasr_b200_paged_kv_gather(void* k_out, void* v_out, const void* k_pool,
                                       const void* v_pool, const int32_t* block_table, int64_t B,
                                       int64_t Hkv, int64_t D, int64_t blocks_per_seq,
                                       int64_t block_size, int64_t num_blocks, int elem_bytes,
                                       void* stream);

/* ---- packed-layout glue ------------------------------------------------ */
/* out[i, :] = in[index[i], :] for i < n_out (rows of `row_bytes` bytes,
 * multiple of 16; index int64; `in` has `in_rows` rows and an index outside
 * [0, in_rows) writes a zero row instead of reading).  Covers
 * pack_hidden / the gapped-conv gather (oasr/models/conformer/packing.py:222-232,
 * oasr/models/conformer/model.py:223-233) and SlotTensor.gather
 * (oasr/cache/state.py:88-94). */
OASR_API int oasr_b200_gather_rows(void* out, const void* in, const int64_t* index, int64_t n_out,
                                   int64_t row_bytes, int64_t in_rows, void* stream);
/* out[index[i], :] = in[i, :] for i < n_in (index_copy_ along rows); `out` has
 * `out_rows` rows and an index outside [0, out_rows) is skipped. */
OASR_API int oasr_b200_scatter_rows(void* out, const void* in, const int64_t* index, int64_t n_in,
                                    int64_t row_bytes, int64_t out_rows, void* stream);

/* ---- feature front end ---------------------------------------------------- */
/* Kaldi-compatible log-mel FBANK features with optional global CMVN in one
 * kernel: snip_edges framing, per-frame DC removal, pre-emphasis (first sample
 * replicated), analysis window, zero-padded n_fft-point power spectrum, mel
 * filterbank, log(max(., log_floor)), then (x - cmvn_mean) * cmvn_istd.
 * Replaces the launcher chain stft_frame / rfft_power / mel_log
 * (csrc/features.cu:39-205, composed in oasr/features/batched.py:171-206) and
 * cmvn (oasr/functionals/norm.py:338-360).  waveforms (B, T) fp32; lengths (B)
 * int32 samples (nullable: every row is T long); window (frame_length) fp32;
 * mel_mat (num_mel, n_fft/2+1) fp32 with mel_lo / mel_hi (num_mel) int32 = the
 * non-zero bin range [lo, hi) of every filter; out (B, num_frames, num_mel)
 * fp32, frames that do not lie wholly inside their utterance are zeros.
 * n_fft: a power of two in [64, 2048], >= frame_length. */
OASR_API int oasr_b200_fbank(float* out, const float* waveforms, const int32_t* lengths /*nullable*/,
                             const float* window, const float* mel_mat, const int32_t* mel_lo,
                             const int32_t* mel_hi, const float* cmvn_mean /*nullable*/,
                             const float* cmvn_istd /*nullable*/, int64_t B, int64_t T,
                             int64_t num_frames, int64_t frame_length, int64_t frame_shift,
                             int64_t n_fft, int64_t num_mel, double preemph, double log_floor,
                             void* stream);

/* ---- greedy CTC decoding -------------------------------------------------- */
/* Per-frame argmax ids of packed utterances -> token rows: repeated ids are
 * dropped, then blanks, never across an utterance boundary (the rule of
 * csrc/decoder/ctc/cpu/ctc_greedy_search.cc:26-55).  The result has the layout
 * of the reference's GPU decoders for beam 1 (oasr/functionals/ctc_decode.py:
 * 313-412: tokens (batch, beam, max_len) int32, lengths (batch, beam), optional
 * emission frames), but is fed by the CTC head's fused argmax, so no log-probs
 * are written or read.  ids (total) int32 with utterance b at
 * [cu_seqlens[b], cu_seqlens[b+1]); tokens (batch, max_len) int32, entries past
 * lengths[b] = blank; lengths (batch) int32 = min(token count, max_len); times
 * (batch, max_len) int32 nullable: the frame (within its utterance) each token
 * was emitted at, -1 past the length. */
OASR_API int oasr_b200_ctc_greedy_collapse(int32_t* tokens, int32_t* lengths, int32_t* times /*nullable*/,
                                           const int32_t* ids, const int32_t* cu_seqlens, int64_t batch,
                                           int64_t max_len, int64_t blank, void* stream);

/* ---- encoder layer stack (native executor) ------------------------------ */
/* Device pointers to the prepared weights of one Conformer encoder layer
 * (ConformerEncoderLayer, oasr/models/conformer/model.py:499-752).  16-bit
 * tensors are in the model dtype, `float` ones are fp32.  Weight matrices are
 * [out_features, in_features] row-major as in the reference's Linear. */
typedef struct oasr_b200_conformer_layer {
  const void *norm_ff_macaron_w, *norm_ff_macaron_b;
  const void *ffm_w1, *ffm_b1, *ffm_w2, *ffm_b2;   /* feed_forward_macaron */
  const void *norm_mha_w, *norm_mha_b;
  const void *qkv4_w, *qkv4_b;   /* [Wq;Wq;Wk;Wv] (4d,d) and [bq+u;bq+v;bk;bv] */
  const void *out_w, *out_b;     /* self_attn.linear_out */
  const float *norm_conv_scale, *norm_conv_shift;  /* norm_conv as folded inference BatchNorm */
  const void *pw1_w, *pw1_b;     /* pointwise_conv1 (2d,d) */
  const void *dw_w, *dw_b;       /* depthwise_conv (K,d) */
  const float *conv_bn_scale, *conv_bn_shift;      /* conv_module.norm_activation folded */
  const float *glu_of_bias;      /* value of a zeroed row after pointwise_conv1 + GLU */
  const void *pw2_w, *pw2_b;
  const void *norm_ff_w, *norm_ff_b;
  const void *ff_w1, *ff_b1, *ff_w2, *ff_b2;       /* feed_forward */
  const void *norm_final_w, *norm_final_b;
  /* 8-bit copies of the eight Linear weights (one byte per element, same shapes) and their fp32
   * per-output-channel scales, in the order ffm_w1, ffm_w2, qkv4, out, pw1, pw2, ff_w1, ff_w2;
   * read only when the model's quant_kind is not 0 (no reference counterpart). */
  const void* q_w[8];
  const float* q_s[8];
} oasr_b200_conformer_layer;

typedef struct oasr_b200_conformer_model {
  int32_t d_model, heads, ffn, kernel, num_layers, vocab_padded, embed_in, dtype;
  double eps;
  const oasr_b200_conformer_layer* layers;   /* HOST array of num_layers entries */
  const void *embed_w, *embed_b;             /* embed Linear (d, embed_in) */
  const void *embed_ln_w, *embed_ln_b;       /* nullable: embed LayerNorm with sqrt(d) folded in */
  const void *pos_w_all;                     /* (num_layers*d, d): every layer's linear_pos */
  const void *pe;                            /* (pe_rows, d) positional table */
  int64_t pe_rows;
  const void *after_norm_w, *after_norm_b;
  const void *ctc_w, *ctc_b;                 /* (vocab_padded, 2d) head weight [W | W] for the two-term input, (vocab_padded) bias */
  const void *pos_proj;                      /* nullable: (pos_proj_rows, num_layers*d) = pe . pos_w_all^T, streaming */
  int64_t pos_proj_rows;
  int32_t quant_kind;                        /* 0 = 16-bit GEMMs; OASR_Q8_FP8_E4M3 / OASR_Q8_INT8: the eight Linear GEMMs of every
                                                layer run on 8-bit operands, activations quantised per token on the fly
                                                (offline entry point only) */
} oasr_b200_conformer_model;

/* Bytes of device scratch oasr_b200_conformer_encode_packed needs for `total`
 * packed frames with segments of at most `max_seg` frames. */
OASR_API int64_t oasr_b200_conformer_workspace_bytes(const oasr_b200_conformer_model* model,
                                                     int64_t total, int64_t max_seg);
/* The whole packed encoder + CTC head in one host call: embed Linear, the
 * layer stack of ConformerEncoder.forward_packed (oasr/models/conformer/model.py:830-868,
 * layer :709-752), after_norm and the fused CTC head (oasr/layers/ctc.py:48-51),
 * as a fixed sequence of this library's kernels on `stream`.  rows is
 * (total, embed_in): the gathered outputs of the subsampling convolutions.
 * fill_frames (nullable, int32[num_segs]) selects the padded-batch semantics
 * of the depthwise conv (see oasr_b200_depthwise_conv1d_packed).  log_probs
 * (nullable) is fp32 (total, vocab_padded); argmax (nullable) int32[total].
 * workspace must hold oasr_b200_conformer_workspace_bytes() bytes, 256-byte
 * aligned.  Nothing is allocated and the host never waits for the device. */
OASR_API int oasr_b200_conformer_encode_packed(const oasr_b200_conformer_model* model,
                                               const void* rows, const int32_t* cu_seqlens,
                                               const int32_t* fill_frames /*nullable*/,
                                               int64_t num_segs, int64_t total, int64_t max_seg,
                                               void* workspace, int64_t workspace_bytes,
                                               float* log_probs /*nullable*/,
                                               int32_t* argmax /*nullable*/, void* stream);

/* One streaming chunk for B streams: ConformerEncoder.forward_chunk_paged
 * (oasr/models/conformer/model.py:913-1023) + CTC head in one host call.
 * rows (B*T, embed_in) are the subsampled chunk frames; layer l appends its
 * keys/values at logical positions cache_seqlens[b].. to k_pools[l] / v_pools[l]
 * (HOST arrays of num_layers device pointers, pools (num_blocks, block_size, H,
 * 64)) through block_table (B, blocks_per_seq), attends over total_seqlens[b] =
 * cache_seqlens[b] + T keys with positions starting at pos_start[b] = offset[b] -
 * cache_seqlens[b], and runs the causal conv module on [cnn_state[l, slot_ids[b]] ;
 * chunk], updating cnn_state (num_layers, num_slots, kernel-1, d) in place.  The
 * caller allocated the chunk's pages before the call and advances cache_seqlens
 * after it, as with the reference's AttentionCacheManager.  T <= 128.  With the
 * model's quant_kind set, the eight Linear GEMMs of every layer run on 8-bit
 * operands as in the offline entry point (per-token quantisation of each input,
 * the layers' q_w / q_s). */
OASR_API int64_t oasr_b200_conformer_chunk_workspace_bytes(const oasr_b200_conformer_model* model,
                                                           int64_t B, int64_t T);
OASR_API int oasr_b200_conformer_chunk_paged(const oasr_b200_conformer_model* model,
                                             const void* rows, int64_t B, int64_t T,
                                             void* const* k_pools /*host*/,
                                             void* const* v_pools /*host*/,
                                             const int32_t* block_table,
                                             const int32_t* cache_seqlens,
                                             const int32_t* total_seqlens,
                                             const int32_t* pos_start, int64_t blocks_per_seq,
                                             int64_t block_size, int64_t num_blocks,
                                             const float* kv_scales /*nullable: fp8 pages, fp32 (num_layers, 2, heads) K then V scales*/,
                                             void* cnn_state, int64_t num_slots,
                                             const int64_t* slot_ids, void* workspace,
                                             int64_t workspace_bytes, float* log_probs /*nullable*/,
                                             int32_t* argmax /*nullable*/, void* stream);

/* This entry point has no counterpart in the reference.  It does what
 * oasr_b200_conformer_encode_packed does for callers that must not allocate
 * device memory (a plugin inside a process whose own pool already owns the
 * GPU's memory, code between a framework's allocator hooks, a latency-critical
 * thread that may not risk the device-wide stall of a cudaMalloc): the scratch
 * is a 64 MiB array built into the library instead of a caller workspace.
 * Inputs and outputs are still the caller's.  A batch that needs more scratch
 * than oasr_b200_conformer_noalloc_capacity_bytes() is refused with
 * OASR_ERR_INVALID and nothing is launched.  The first call on a device
 * resolves the array's device address; make it with that device current and
 * outside any stream capture.  That first call is also when the CUDA runtime
 * places the array on the device, so make one warm-up call per device (total
 * = 0 is enough) at start-up, BEFORE the host's pool takes the GPU's memory;
 * made later it fails with an out-of-memory status.  Serialise calls on a
 * device, the first one included.  All calls share the array (it keeps the last
 * call's contents; no step reads it before writing), so calls that overlap on
 * the GPU race with each other and must be serialised by the caller. */
OASR_API int oasr_b200_conformer_encode_packed_noalloc(const oasr_b200_conformer_model* model,
                                                       const void* rows,
                                                       const int32_t* cu_seqlens,
                                                       const int32_t* fill_frames /*nullable*/,
                                                       int64_t num_segs, int64_t total,
                                                       int64_t max_seg,
                                                       float* log_probs /*nullable*/,
                                                       int32_t* argmax /*nullable*/, void* stream);
/* Size in bytes of the built-in scratch array of the entry point above. */
OASR_API int64_t oasr_b200_conformer_noalloc_capacity_bytes(void);

/* Per-step timing of oasr_b200_conformer_encode_packed for benchmarks (no
 * reference counterpart).  profile_enable(1) clears the records and makes the
 * executor bracket every step with a CUDA-event pair on its stream;
 * profile_enable(0) stops recording and clears.  profile_get waits for record
 * `index` and returns its label (a static string), device milliseconds and
 * algorithmic flops (0 for steps that are not GEMMs). */
OASR_API int oasr_b200_profile_enable(int on);
OASR_API int oasr_b200_profile_count(void);
OASR_API int oasr_b200_profile_get(int index, const char** label /*host*/, double* ms /*host*/,
                                   double* flops /*host*/);

/* ---- FastConformer / Nemotron layer stack (native executor) ---------------- */
/* Device pointers to the prepared weights of one NemotronEncoderLayer
 * (oasr/models/nemotron/encoder.py:217-267): 16-bit tensors in the model
 * dtype, weight matrices [out_features, in_features] row-major, every bias
 * nullable.  qkv4_w is [Wq; Wq; Wk; Wv] (4C, C) with qkv4_b = [bq+u; bq+v; bk;
 * bv] (the two global biases of the Transformer-XL attention folded into two
 * copies of the query projection); rel_w is relative_k_proj (C, C); dw_w is the
 * causal depthwise conv as (kernel, C). */
typedef struct oasr_b200_fastconformer_layer {
  const void *norm_ff1_w, *norm_ff1_b;
  const void *ff1_w1, *ff1_b1, *ff1_w2, *ff1_b2;
  const void *norm_att_w, *norm_att_b;
  const void *qkv4_w, *qkv4_b, *rel_w, *o_w, *o_b;
  const void *norm_conv_w, *norm_conv_b;
  const void *pw1_w, *pw1_b, *dw_w, *dw_b, *conv_norm_w, *conv_norm_b, *pw2_w, *pw2_b;
  const void *norm_ff2_w, *norm_ff2_b;
  const void *ff2_w1, *ff2_b1, *ff2_w2, *ff2_b2;
  const void *norm_out_w, *norm_out_b;
  /* 8-bit kinds (model.quant_kind != 0): the eight Linear weights quantised per output channel
   * (oasr_b200_quantize_rows of the 16-bit weight) and their fp32 scales, in the order ff1_w1, ff1_w2, qkv4_w, o_w,
   * pw1_w, pw2_w, ff2_w1, ff2_w2.  rel_w stays 16-bit (it multiplies the small position table).  Unused otherwise. */
  const void* q_w[8];
  const float* q_s[8];
} oasr_b200_fastconformer_layer;

typedef struct oasr_b200_fastconformer_model {
  int32_t hidden, heads, ffn, kernel, num_layers, dtype;
  int32_t left_context;    /* sliding_window - 1 frames; < 0 = unlimited */
  int32_t right_context;   /* look-ahead frames; the trained attention chunk is right_context + 1 frames */
  double eps;              /* of the LayerNorms between the sub-layers (the conv module's own norm uses 1e-5) */
  double mask_floor;       /* finite additive floor of a masked key (-1e4, encoder.py:80) */
  const oasr_b200_fastconformer_layer* layers;   /* HOST array of num_layers entries */
  int32_t quant_kind;      /* 0 = 16-bit Linear GEMMs; OASR_Q8_FP8_E4M3 / OASR_Q8_INT8 = per-token quantised inputs x q_w */
} oasr_b200_fastconformer_model;

/* Bytes of device scratch oasr_b200_fastconformer_layers_packed needs for `total` packed frames, a relative-position
 * table of `table_rows` rows and an attention bias of `bias_numel` elements. */
OASR_API int64_t oasr_b200_fastconformer_workspace_bytes(const oasr_b200_fastconformer_model* model, int64_t total,
                                                         int64_t table_rows, int64_t bias_numel);
/* The layer loop of NemotronEncoder.forward (oasr/models/nemotron/encoder.py:542-583, layer :217-267, attention
 * :82-149 / 300-359, conv module :150-214) on the valid frames of all utterances back to back, as one fixed sequence
 * of this library's kernels on `stream`.  rows (total, hidden), 16-bit or (rows_f32 != 0) fp32: the post-subsampling
 * states of the valid frames (they start the fp32 residual stream, which lives in the workspace; rows is not written); out (total, hidden) fp32: the stack's output.
 * rel_table (table_rows, hidden) 16-bit:
 * sinusoid rows for relative positions max_seg-1 .. -(max_seg-1), then zero rows up to a multiple of 8.  cu_seqlens
 * int32[num_segs+1]; bias_offsets int64[num_segs+1], segment s = heads * len_s * roundup8(len_s) elements, bias_numel
 * their sum.  workspace: oasr_b200_fastconformer_workspace_bytes() bytes, 256-byte aligned.  Nothing is allocated and
 * the host never waits for the device. */
OASR_API int oasr_b200_fastconformer_layers_packed(const oasr_b200_fastconformer_model* model, const void* rows,
                                                   int rows_f32, float* out,
                                                   const void* rel_table, int64_t table_rows,
                                                   const int32_t* cu_seqlens, const int64_t* bias_offsets,
                                                   int64_t bias_numel, int64_t num_segs, int64_t total,
                                                   int64_t max_seg, void* workspace, int64_t workspace_bytes,
                                                   void* stream);

#ifdef __cplusplus
}
#endif
#endif /* OASR_B200_H_ */
