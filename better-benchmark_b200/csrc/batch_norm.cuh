// Pieces shared by the translation units of the BatchNorm training forward: the parameter block and
// the step from the fp64 totals of a channel's shifted sums to its mean / invstd / running statistics.
#pragma once

#include "rowwise.cuh"

namespace b200 {

struct BatchNormParams {
  const void* x;
  void* y;
  const void* weight;  // may be null
  const void* bias;    // may be null
  float* running_mean;  // may be null (no update)
  float* running_var;
  float* save_mean;    // [C] fp32 out (may be null)
  float* save_invstd;  // [C] fp32 out (may be null)
  long long rows;      // N*H*W for channels-last; N for the general path
  int channels;
  long long spatial;   // general path: H*W
  long long sn, sc, ss;  // general path: element strides of (n, c, spatial)
  int w_dtype;
  float eps, momentum, one_minus_momentum, unbias;
  double count;  // elements per channel
  double inv_count;  // 1 / count (a multiplication by it replaces two fp64 divisions per channel)
  int relu;
  float* partials;  // [P][2][C]
  float* stats;     // [2][C] mean, invstd (scratch copy every CTA reads)
  unsigned int* bar;
  long long rows_per_cta;  // contiguous row range of each CTA
  int smem_tiles;          // stages of the shared-memory ring
  int local_stats;         // 1: every CTA combines all partials itself (one grid barrier instead of two)
  int deep;                // 1: a thread's chain of squares is long; it is carried in fp64 every 16 vectors
};

// The value every sum of a channel is shifted by. Any value works as long as all threads of all
// CTAs use the same one; the closer it is to the channel's mean, the less the variance
// (s2 - s1 * s1 / n) / n cancels, and the cancellation multiplies the rounding error of s2 by
// 1 + (shift - mean)^2 / var. The first element of the channel can sit three standard deviations
// away (a factor of ten); the mean of the channel's first sixteen rows (rows beyond the last one
// repeat it) rarely sits more than one. Both forms below add the same sixteen values in the same
// order with the same roundings, so they agree to the bit.
constexpr int BN_SHIFT_ROWS = 16;

// The shift is cut to eight significant bits (a bf16 value). With 16-bit inputs x - shift then
// has so few bits that the sums of the differences are exact or nearly so; with a full fp32 shift
// every addition would drop the same low bits of the shift and the errors would add up instead
// of cancelling (measured: the mean of 6.4 M bf16 values off by 2e-6 instead of 1e-8).
__device__ __forceinline__ float bn_round_shift(float v) {
  return __uint_as_float((__float_as_uint(v) + 0x8000u) & 0xffff0000u);
}

template <typename T>
__device__ __forceinline__ float bn_shift_scalar(const T* x, int c, int channels, long long rows) {
  float v[BN_SHIFT_ROWS];
#pragma unroll
  for (int r = 0; r < BN_SHIFT_ROWS; ++r) {
    const long long rr = r < rows ? r : rows - 1;
    v[r] = Elem<T>::to_f32(__ldg(x + rr * channels + c));
  }
  float s = 0.f;
#pragma unroll
  for (int r = 0; r < BN_SHIFT_ROWS; ++r) s = __fadd_rn(s, v[r]);
  return bn_round_shift(__fmul_rn(s, 1.0f / BN_SHIFT_ROWS));
}

// The same for the Elem<T>::V channels of vector column vc, as fp32 pairs.
template <typename T>
__device__ __forceinline__ void bn_shift_pairs(const T* x, int vc, int channels, long long rows,
                                               f32x2 (&shift)[Elem<T>::V / 2]) {
  constexpr int V = Elem<T>::V;
  uint4 raw[BN_SHIFT_ROWS];
#pragma unroll
  for (int r = 0; r < BN_SHIFT_ROWS; ++r) {
    const long long rr = r < rows ? r : rows - 1;
    raw[r] = ld_keep(x + rr * channels + (long long)vc * V);
  }
#pragma unroll
  for (int i = 0; i < V / 2; ++i) shift[i] = splat2(0.f);
#pragma unroll
  for (int r = 0; r < BN_SHIFT_ROWS; ++r) {
    f32x2 f[V / 2];
    Pairs<T>::unpack(raw[r], f);
#pragma unroll
    for (int i = 0; i < V / 2; ++i) shift[i] = add2(shift[i], f[i]);
  }
#pragma unroll
  for (int i = 0; i < V / 2; ++i) {
    float lo, hi;
    unpack2(mul2(shift[i], splat2(1.0f / BN_SHIFT_ROWS)), lo, hi);
    shift[i] = pack2(bn_round_shift(lo), bn_round_shift(hi));
  }
}

// Turns the fp64 totals of the shifted sums of one channel into mean / invstd and, for the one
// caller that owns the channel's global outputs, writes the saved and running statistics.
// have_old: the caller already holds the channel's running statistics (fetched while the sums
// were being formed, so that their latency is not waited for here).
__device__ __forceinline__ void bn_channel_stats(const BatchNormParams& p, int c, double s1, double s2, float shift,
                                                 bool write_global, float* mean_out, float* invstd_out,
                                                 bool have_old = false, float old_mean = 0.f, float old_var = 0.f) {
  // On the critical path of every launch (one thread per channel computes this while the others
  // wait), so no fp64 division or square root: a product with 1/count and the fp64 rsqrt.
  const double mean_shifted = s1 * p.inv_count;
  double var = (s2 - s1 * mean_shifted) * p.inv_count;
  if (var < 0.0) var = 0.0;
  const float mean = (float)((double)shift + mean_shifted);
  const float varf = (float)var;
  // 1 / sqrt(var + eps) from the fp64 variance, rounded once: within an ulp or two of the graph's
  // rsqrt(fp32(var) + eps), and the closest fp32 value to what the graph gives in fp64
  const float invstd = (float)rsqrt(var + (double)p.eps);
  *mean_out = mean;
  *invstd_out = invstd;
  if (write_global) {
    if (p.save_mean) p.save_mean[c] = mean;
    if (p.save_invstd) p.save_invstd[c] = invstd;
    if (p.running_mean) {
      if (!have_old) {
        old_mean = p.running_mean[c];
        old_var = p.running_var[c];
      }
      p.running_mean[c] = mean * p.momentum + old_mean * p.one_minus_momentum;
      p.running_var[c] = (varf * p.unbias) * p.momentum + old_var * p.one_minus_momentum;
    }
  }
}

// Many channels: the channels are dealt out to the WARPS of the grid (channel c to warp c / P of
// CTA c % P, P = CTAs = partial rows), so that all of them are combined at the same time and no
// CTA barrier is involved. The lanes split the partial rows, eight loads in flight each, fp64,
// fixed order; lane 0 derives the statistics and publishes them in p.stats for the second grid barrier.
template <typename T>
__device__ __forceinline__ void bn_stats_by_warps(const BatchNormParams& p, const T* x, int P) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  // a trailing partial warp (block sizes that are no multiple of 32) takes no channel
  for (int c = (int)blockIdx.x + warp * P; c < p.channels && warp < nwarps; c += P * nwarps) {
    const float shift = lane == 0 ? bn_shift_scalar<T>(x, c, p.channels, p.rows) : 0.f;
    double d1 = 0.0, d2 = 0.0;
    for (int g0 = lane; g0 < P; g0 += 8 * 32) {
      float a[8], b[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int g = g0 + u * 32;
        a[u] = g < P ? __ldcg(p.partials + ((long long)g * 2) * p.channels + c) : 0.f;
        b[u] = g < P ? __ldcg(p.partials + ((long long)g * 2 + 1) * p.channels + c) : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        d1 += (double)a[u];
        d2 += (double)b[u];
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      d1 += __shfl_xor_sync(0xffffffffu, d1, o);
      d2 += __shfl_xor_sync(0xffffffffu, d2, o);
    }
    if (lane == 0) {
      float mean, invstd;
      bn_channel_stats(p, c, d1, d2, shift, true, &mean, &invstd);
      p.stats[c] = mean;
      p.stats[p.channels + c] = invstd;
    }
  }
}

// Contiguous NCHW tensors (batch_norm_nchw.cu): one launch, the CTAs that share a channel form a
// thread-block cluster. Returns false when the shape does not fit (the caller takes another path).
template <typename T>
bool try_launch_batch_norm_nchw(const BatchNormParams& p, cudaStream_t st, int* rc);

}  // namespace b200
