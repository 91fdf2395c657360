// Greedy CTC decoding of packed per-frame argmax ids on the GPU: drop repeated ids, then blanks, never across an
// utterance boundary (the rule of the reference's greedy search, csrc/decoder/ctc/cpu/ctc_greedy_search.cc:26-55;
// its GPU decoders take fp32 log-probs, oasr/functionals/ctc_decode.py:313-412, and return (batch, beam, max_len)
// int32 tokens, (batch, beam) lengths and optional emission frames -- this is that result for beam 1, fed by the
// CTC head's fused argmax so that no log-probs are ever written).  One block per utterance: a block-wide prefix
// sum over the keep flags gives every surviving token its output slot, so the order is deterministic.
#include "common.cuh"

namespace ob {
namespace ctc_greedy {

constexpr int kThreads = 256;

__global__ void __launch_bounds__(kThreads) collapse_kernel(int32_t* __restrict__ tokens, int32_t* __restrict__ lengths,
                                                          int32_t* __restrict__ times, const int32_t* __restrict__ ids,
                                                          const int32_t* __restrict__ cu_seqlens, int max_len, int blank) {
  __shared__ int warp_sums[kThreads / 32];
  __shared__ int carry;
  const int b = blockIdx.x;
  const int begin = cu_seqlens[b], end = cu_seqlens[b + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int32_t* out = tokens + static_cast<int64_t>(b) * max_len;
  int32_t* tout = times ? times + static_cast<int64_t>(b) * max_len : nullptr;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int base = begin; base < end; base += kThreads) {
    const int t = base + threadIdx.x;
    int id = blank;
    bool keep = false;
    if (t < end) {
      id = ids[t];
      const int prev = t > begin ? ids[t - 1] : -1;
      keep = id != prev && id != blank;
    }
    const unsigned ballot = __ballot_sync(0xffffffffu, keep);
    const int in_warp = __popc(ballot & ((1u << lane) - 1u));
    if (lane == 0) warp_sums[warp] = __popc(ballot);
    __syncthreads();
    int before = carry;
    for (int w = 0; w < warp; ++w) before += warp_sums[w];
    const int slot = before + in_warp;
    if (keep && slot < max_len) {
      out[slot] = id;
      if (tout) tout[slot] = t - begin;
    }
    __syncthreads();
    if (threadIdx.x == kThreads - 1) carry = before + in_warp + (keep ? 1 : 0);
    __syncthreads();
  }
  const int n = min(carry, max_len);
  if (threadIdx.x == 0) lengths[b] = n;
  // the tail of the row is defined too: blank ids (and -1 frames), so the row can be compared or copied whole
  for (int i = n + threadIdx.x; i < max_len; i += kThreads) {
    out[i] = blank;
    if (tout) tout[i] = -1;
  }
}

}  // namespace ctc_greedy
}  // namespace ob

extern "C" {

int oasr_b200_ctc_greedy_collapse(int32_t* tokens, int32_t* lengths, int32_t* times, const int32_t* ids,
                                  const int32_t* cu_seqlens, int64_t batch, int64_t max_len, int64_t blank, void* stream) {
  using namespace ob;
  OB_REQUIRE(batch >= 0 && max_len >= 0 && max_len < (int64_t(1) << 31), OASR_ERR_INVALID, "ctc_greedy_collapse: bad shape");
  if (batch == 0) return OASR_OK;
  OB_REQUIRE(lengths && cu_seqlens && (max_len == 0 || tokens), OASR_ERR_INVALID, "ctc_greedy_collapse: null pointer argument");
  OB_REQUIRE(ids != nullptr, OASR_ERR_INVALID, "ctc_greedy_collapse: null id pointer");
  ctc_greedy::collapse_kernel<<<static_cast<unsigned>(batch), ctc_greedy::kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      tokens, lengths, times, ids, cu_seqlens, static_cast<int>(max_len), static_cast<int>(blank));
  return check_launch("ctc_greedy_collapse launch");
}

}  // extern "C"
