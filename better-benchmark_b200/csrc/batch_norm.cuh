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
  int relu;
  float* partials;  // [P][2][C]
  float* stats;     // [2][C] mean, invstd (scratch copy every CTA reads)
  unsigned int* bar;
  long long rows_per_cta;  // contiguous row range of each CTA
  int smem_tiles;          // stages of the shared-memory ring
  int local_stats;         // 1: every CTA combines all partials itself (one grid barrier instead of two)
};

// Turns the fp64 totals of the shifted sums of one channel into mean / invstd and, for the one
// caller that owns the channel's global outputs, writes the saved and running statistics.
__device__ __forceinline__ void bn_channel_stats(const BatchNormParams& p, int c, double s1, double s2, float shift,
                                                 bool write_global, float* mean_out, float* invstd_out) {
  const double mean_shifted = s1 / p.count;
  double var = (s2 - s1 * mean_shifted) / p.count;
  if (var < 0.0) var = 0.0;
  const float mean = (float)((double)shift + mean_shifted);
  const float varf = (float)var;
  const float invstd = rsqrtf(varf + p.eps);
  *mean_out = mean;
  *invstd_out = invstd;
  if (write_global) {
    if (p.save_mean) p.save_mean[c] = mean;
    if (p.save_invstd) p.save_invstd[c] = invstd;
    if (p.running_mean) {
      p.running_mean[c] = mean * p.momentum + p.running_mean[c] * p.one_minus_momentum;
      p.running_var[c] = (varf * p.unbias) * p.momentum + p.running_var[c] * p.one_minus_momentum;
    }
  }
}

// Contiguous NCHW tensors (batch_norm_nchw.cu): one launch, the CTAs that share a channel form a
// thread-block cluster. Returns false when the shape does not fit (the caller takes another path).
template <typename T>
bool try_launch_batch_norm_nchw(const BatchNormParams& p, cudaStream_t st, int* rc);

}  // namespace b200
