// Kaldi-compatible log-mel filterbank features (FBANK) with optional global CMVN, one fused kernel:
//   frame (snip_edges) -> subtract the frame's mean -> pre-emphasis (first sample replicated) -> analysis window ->
//   zero-pad to n_fft -> power spectrum -> mel filterbank -> log(max(., floor)) -> (x - mean) * istd
// It replaces the reference's kernel chain stft_frame -> rfft_power -> mel_log (launchers csrc/features.cu:39-205,
// composed by oasr/features/batched.py:171-206; arithmetic of the torch route batched.py:209-268) and GlobalCMVN
// (oasr/layers/norm.py:571-584): frames, spectra and mel energies never reach HBM.
//
// One warp per frame.  The real FFT of n_fft points is a complex FFT of n_fft/2 points on z[n] = x[2n] + i x[2n+1]
// (radix-2, decimation in time, in shared memory, one __syncwarp per stage) followed by the usual split; all
// twiddles come from one table W[k] = exp(-2 pi i k / n_fft), k < n_fft/2, built per block.  The mel filterbank is
// applied from the dense (num_mel, n_fft/2+1) matrix the reference builds, but only over each filter's non-zero
// bin range.  HBM-bound in principle (4 B in per hop sample, 4 B out per mel bin); in practice a few dozen
// microseconds for a batch of a thousand audio-seconds, so the instruction count of the FFT is what it costs.
#include "common.cuh"

namespace ob {
namespace features {

constexpr int kWarps = 4;
constexpr int kMaxFft = 2048;

struct Args {
  const float* wave;       // (B, T)
  const int32_t* lengths;  // (B) samples, nullable = every row is T samples long
  const float* window;     // (frame_length)
  const float* mel;        // (num_mel, n_fft/2 + 1)
  const int32_t* mel_lo;   // (num_mel) first non-zero bin
  const int32_t* mel_hi;   // (num_mel) one past the last non-zero bin
  const float* cmvn_mean;  // (num_mel), nullable
  const float* cmvn_istd;  // (num_mel), nullable
  float* out;              // (B, num_frames, num_mel)
  int64_t B, T;
  int num_frames, frame_length, frame_shift, n_fft, log2_half, num_mel;
  float preemph, log_floor;
};

__global__ void __launch_bounds__(kWarps * 32) fbank_kernel(Args a) {
  extern __shared__ float fb_smem[];
  const int N = a.n_fft, Nh = N >> 1;
  float2* tw = reinterpret_cast<float2*>(fb_smem);                       // Nh entries
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* bufA = fb_smem + 2 * Nh + warp * (2 * N + 2);                   // N + 2 floats: samples, later the power spectrum
  float2* z = reinterpret_cast<float2*>(bufA + N + 2);                   // Nh complex values
  for (int k = threadIdx.x; k < Nh; k += blockDim.x) {
    float s, c;
    sincospif(2.0f * static_cast<float>(k) / static_cast<float>(N), &s, &c);
    tw[k] = make_float2(c, -s);
  }
  __syncthreads();
  const int64_t total = a.B * a.num_frames;
  const int L = a.frame_length;
  for (int64_t f = static_cast<int64_t>(blockIdx.x) * kWarps + warp; f < total; f += static_cast<int64_t>(gridDim.x) * kWarps) {
    const int64_t b = f / a.num_frames;
    const int t = static_cast<int>(f - b * a.num_frames);
    float* out = a.out + f * a.num_mel;
    const int64_t len = a.lengths ? a.lengths[b] : a.T;
    const int64_t start = static_cast<int64_t>(t) * a.frame_shift;
    if (start + L > len) {                       // not a whole frame of this utterance: outside its feature length
      for (int m = lane; m < a.num_mel; m += 32) out[m] = 0.f;
      continue;
    }
    const float* x = a.wave + b * a.T + start;
    // samples and their mean
    float sum = 0.f;
    for (int n = lane; n < L; n += 32) {
      const float v = x[n];
      bufA[n] = v;
      sum += v;
    }
    const float mean = warp_sum(sum) / static_cast<float>(L);
    __syncwarp();
    // DC removal, pre-emphasis, window, zero padding; packed as z[m] = y[2m] + i y[2m+1] at the bit-reversed index
    const int shift = 32 - a.log2_half;
    for (int m = lane; m < Nh; m += 32) {
      float y[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int n = 2 * m + e;
        float v = 0.f;
        if (n < L) {
          const float cur = bufA[n] - mean;
          const float prev = bufA[n > 0 ? n - 1 : 0] - mean;
          v = (cur - a.preemph * prev) * a.window[n];
        }
        y[e] = v;
      }
      z[__brev(static_cast<unsigned>(m)) >> shift] = make_float2(y[0], y[1]);
    }
    __syncwarp();
    // complex FFT of Nh points, radix 2: stage s joins blocks of half = 2^s
    for (int half = 1; half < Nh; half <<= 1) {
      const int tw_step = N / (2 * half) ;       // W_{2*half}^j = W_N^{j * N / (2*half)}
      for (int i = lane; i < (Nh >> 1); i += 32) {
        const int j = i & (half - 1);
        const int lo = ((i - j) << 1) + j;
        const float2 w = tw[j * tw_step];
        const float2 u = z[lo], v = z[lo + half];
        const float2 wv = make_float2(w.x * v.x - w.y * v.y, w.x * v.y + w.y * v.x);
        z[lo] = make_float2(u.x + wv.x, u.y + wv.y);
        z[lo + half] = make_float2(u.x - wv.x, u.y - wv.y);
      }
      __syncwarp();
    }
    // split into the spectrum of the real signal: X[k] = (Z[k] + conj Z[Nh-k]) / 2 - i W_N^k (Z[k] - conj Z[Nh-k]) / 2
    float* power = bufA;
    for (int k = lane; k <= Nh; k += 32) {
      const float2 zk = z[k == Nh ? 0 : k];
      const float2 zc = z[(Nh - k) == Nh ? 0 : (Nh - k)];
      const float er = 0.5f * (zk.x + zc.x), ei = 0.5f * (zk.y - zc.y);      // even part
      const float orr = 0.5f * (zk.x - zc.x), oi = 0.5f * (zk.y + zc.y);     // (Z[k] - conj Z[Nh-k]) / 2
      float2 w = k == Nh ? make_float2(-1.f, 0.f) : tw[k];
      // -i * w * (orr + i oi) = -i * ((w.x*orr - w.y*oi) + i (w.x*oi + w.y*orr)) = (w.x*oi + w.y*orr) - i (w.x*orr - w.y*oi)
      const float xr = er + (w.x * oi + w.y * orr);
      const float xi = ei - (w.x * orr - w.y * oi);
      power[k] = xr * xr + xi * xi;
    }
    __syncwarp();
    const int nfreq = Nh + 1;
    for (int m = lane; m < a.num_mel; m += 32) {
      const float* row = a.mel + static_cast<int64_t>(m) * nfreq;
      float acc = 0.f;
      for (int k = a.mel_lo[m]; k < a.mel_hi[m]; ++k) acc = fmaf(power[k], __ldg(row + k), acc);
      float v = logf(fmaxf(acc, a.log_floor));
      if (a.cmvn_mean) v = (v - a.cmvn_mean[m]) * a.cmvn_istd[m];
      out[m] = v;
    }
    __syncwarp();
  }
}

}  // namespace features
}  // namespace ob

extern "C" {

int oasr_b200_fbank(float* out, const float* waveforms, const int32_t* lengths, const float* window, const float* mel_mat,
                    const int32_t* mel_lo, const int32_t* mel_hi, const float* cmvn_mean, const float* cmvn_istd,
                    int64_t B, int64_t T, int64_t num_frames, int64_t frame_length, int64_t frame_shift, int64_t n_fft,
                    int64_t num_mel, double preemph, double log_floor, void* stream) {
  using namespace ob;
  using namespace ob::features;
  OB_REQUIRE(B >= 0 && T >= 0 && num_frames >= 0 && num_mel > 0, OASR_ERR_INVALID, "fbank: bad shape");
  if (B == 0 || num_frames == 0) return OASR_OK;
  OB_REQUIRE(out && waveforms && window && mel_mat && mel_lo && mel_hi, OASR_ERR_INVALID, "fbank: null pointer argument");
  OB_REQUIRE((cmvn_mean == nullptr) == (cmvn_istd == nullptr), OASR_ERR_INVALID, "fbank: CMVN needs both mean and istd");
  OB_REQUIRE(n_fft >= 64 && n_fft <= kMaxFft && (n_fft & (n_fft - 1)) == 0, OASR_ERR_UNSUPPORTED,
             "fbank: n_fft must be a power of two in [64, %d] (got %lld)", kMaxFft, (long long)n_fft);
  OB_REQUIRE(frame_length >= 2 && frame_length <= n_fft && frame_shift > 0, OASR_ERR_INVALID,
             "fbank: frame length %lld / shift %lld do not fit n_fft %lld", (long long)frame_length, (long long)frame_shift,
             (long long)n_fft);
  OB_REQUIRE((num_frames - 1) * frame_shift + frame_length <= T, OASR_ERR_INVALID,
             "fbank: %lld frames do not fit %lld samples", (long long)num_frames, (long long)T);
  Args a{};
  a.wave = waveforms; a.lengths = lengths; a.window = window; a.mel = mel_mat; a.mel_lo = mel_lo; a.mel_hi = mel_hi;
  a.cmvn_mean = cmvn_mean; a.cmvn_istd = cmvn_istd; a.out = out;
  a.B = B; a.T = T;
  a.num_frames = static_cast<int>(num_frames); a.frame_length = static_cast<int>(frame_length);
  a.frame_shift = static_cast<int>(frame_shift); a.n_fft = static_cast<int>(n_fft); a.num_mel = static_cast<int>(num_mel);
  int lg = 0;
  while ((int64_t(1) << lg) < n_fft / 2) ++lg;
  a.log2_half = lg;
  a.preemph = static_cast<float>(preemph); a.log_floor = static_cast<float>(log_floor);
  const int64_t total = B * num_frames;
  int64_t grid = (total + kWarps - 1) / kWarps;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  if (grid > cap) grid = cap;
  // twiddle table (n_fft/2 complex) + per warp n_fft + 2 floats of samples / power and n_fft/2 complex values
  const size_t smem = sizeof(float) * (static_cast<size_t>(n_fft) + kWarps * (2 * static_cast<size_t>(n_fft) + 2));
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(fbank_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return set_error(OASR_ERR_CUDA, "fbank: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
  }
  fbank_kernel<<<static_cast<unsigned>(grid), kWarps * 32, smem, static_cast<cudaStream_t>(stream)>>>(a);
  return check_launch("fbank launch");
}

}  // extern "C"
