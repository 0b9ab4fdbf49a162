// Pieces shared by the translation units of the LayerNorm / RMSNorm backward: the parameter block,
// the fp64 finalize of the per-group partial rows, and the launch-geometry helpers.
#pragma once

#include "rowwise.cuh"
#include "tile_stream.cuh"

namespace b200 {

struct NormBwdParams {
  const void* x;
  const void* dy;
  const void* w;      // may be null (treated as ones)
  const float* mean;  // LayerNorm only
  const float* rstd;
  void* dx;
  float* dw;  // may be null
  float* db;  // may be null
  long long rows;
  int n;
  long long x_row_stride, dy_row_stride;
  int dy_elem_stride;  // 1, or 0 when dy is one element broadcast over the whole tensor (dy_row_stride 0 too)
  int w_dtype;
  // dx element (r, c) lives at (r / seq) * dx_batch_stride + (r % seq) * dx_seq_stride
  //                            + (c / head_dim) * dx_head_stride + (c % head_dim)
  int seq, head_dim;
  FastDiv seq_div;  // rows < 2^31, so row / seq is a 32-bit fast division
  long long dx_batch_stride, dx_seq_stride, dx_head_stride;
  float n_f;
  float* partials;    // [groups][n] for dw, followed by [groups][n] for db
  double* level2;     // [2][slices][n]: second level of the fused finalize (may be null)
  unsigned int* bar;  // grid barrier words (cooperative variant)
  int groups;
  int fused;  // 1: barrier + finalize inside this launch
};

template <int V>
__device__ __forceinline__ void zero(float (&a)[V]) {
#pragma unroll
  for (int i = 0; i < V; ++i) a[i] = 0.f;
}

// Sum `groups` partial rows into out[0..n): each CTA takes 64-column chunks, its warps split the
// partial rows, fp64 accumulation, fixed order.
__device__ __forceinline__ void finalize_columns(const float* partials, int groups, int n, float* out,
                                                 double* smem /* [warps][64] */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int chunks = (n + 63) / 64;
  for (int chunk = blockIdx.x; chunk < chunks; chunk += gridDim.x) {
    const int c0 = chunk * 64 + lane, c1 = c0 + 32;
    double a0 = 0.0, a1 = 0.0;
    for (int g0 = warp; g0 < groups; g0 += 4 * nwarps) {  // eight loads in flight, then added in order
      float v0[4], v1[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int g = g0 + u * nwarps;
        const float* row = partials + (long long)g * n;
        v0[u] = (g < groups && c0 < n) ? __ldcg(row + c0) : 0.f;
        v1[u] = (g < groups && c1 < n) ? __ldcg(row + c1) : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        a0 += (double)v0[u];
        a1 += (double)v1[u];
      }
    }
    smem[warp * 64 + lane] = a0;
    smem[warp * 64 + 32 + lane] = a1;
    __syncthreads();
    if (warp == 0) {
      double s0 = 0.0, s1 = 0.0;
      for (int w = 0; w < nwarps; ++w) {
        s0 += smem[w * 64 + lane];
        s1 += smem[w * 64 + 32 + lane];
      }
      if (c0 < n) out[c0] = (float)s0;
      if (c1 < n) out[c1] = (float)s1;
    }
    __syncthreads();
  }
}

// Two-level variant for grids much larger than the number of 64-column chunks (narrow rows): with
// one chunk per CTA only n/64 CTAs would add up all the partial rows while the rest of the grid
// idles. Level 1: CTA b sums chunk b % chunks over the partial rows slice, slice + slices, ...
// (slice = b / chunks) and writes fp64 sums; a grid barrier; level 2: the first `chunks` CTAs add
// the slices in order. `which` selects the dw (0) or db (1) plane of `level2`.
__device__ __forceinline__ void finalize_level1(const float* partials, int groups, int n, double* level2, int slices,
                                                double* smem /* [warps][64] */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int chunks = (n + 63) / 64;
  if ((int)blockIdx.x >= chunks * slices) return;
  const int chunk = blockIdx.x % chunks, slice = blockIdx.x / chunks;
  const int c0 = chunk * 64 + lane, c1 = c0 + 32;
  double a0 = 0.0, a1 = 0.0;
  for (int k0 = warp; slice + slices * k0 < groups; k0 += 4 * nwarps) {
    float v0[4], v1[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int g = slice + slices * (k0 + u * nwarps);
      const float* row = partials + (long long)g * n;
      v0[u] = (g < groups && c0 < n) ? __ldcg(row + c0) : 0.f;
      v1[u] = (g < groups && c1 < n) ? __ldcg(row + c1) : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      a0 += (double)v0[u];
      a1 += (double)v1[u];
    }
  }
  smem[warp * 64 + lane] = a0;
  smem[warp * 64 + 32 + lane] = a1;
  __syncthreads();
  if (warp == 0) {
    double s0 = 0.0, s1 = 0.0;
    for (int w = 0; w < nwarps; ++w) {
      s0 += smem[w * 64 + lane];
      s1 += smem[w * 64 + 32 + lane];
    }
    if (c0 < n) level2[(long long)slice * n + c0] = s0;
    if (c1 < n) level2[(long long)slice * n + c1] = s1;
  }
  __syncthreads();
}

__device__ __forceinline__ void finalize_level2(const double* level2, int slices, int n, float* out) {
  const int chunks = (n + 63) / 64;
  if ((int)blockIdx.x >= chunks || threadIdx.x >= 64) return;
  const int c = blockIdx.x * 64 + threadIdx.x;
  if (c >= n) return;
  double s = 0.0;
  for (int k0 = 0; k0 < slices; k0 += 8) {  // eight loads in flight, added in order
    double v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u)
      v[u] = k0 + u < slices ? __ldcg(level2 + (long long)(k0 + u) * n + c) : 0.0;
#pragma unroll
    for (int u = 0; u < 8; ++u) s += v[u];
  }
  out[c] = (float)s;
}


// Warp reduction of N (2, 4 or 8) values per lane at once: in every step a lane keeps one half of
// its values and hands the other half to its partner, so N values need N - 1 + log2(32 / N)
// shuffles instead of 5 N.
template <int N>
__device__ __forceinline__ float warp_reduce_multi(float (&v)[N], int lane) {
  // After the call lane l holds the warp total of value l / (32 / N).
  int off = 16;
#pragma unroll
  for (int n = N; n > 1; n >>= 1) {
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < n / 2; ++i) {
      const float send = upper ? v[i] : v[i + n / 2];
      const float keep = upper ? v[i + n / 2] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
    off >>= 1;
  }
#pragma unroll
  for (int k = 0; k < 5; ++k) {
    if (off >= 1) {
      v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
      off >>= 1;
    }
  }
  return v[0];
}

// Warp-per-row kernel with per-warp copy rings (norm_bwd_warp.cu): rows of 33..256 vectors.
// Returns false when the shape does not fit (the caller takes another kernel); otherwise *rc is
// the launch status.
template <typename T, bool LN>
bool try_launch_norm_bwd_warp(NormBwdParams p, size_t scratch_bytes, bool cooperative, cudaStream_t st, int* rc);

unsigned int norm_bwd_warp_wait_timeouts();  // bounded waits of that kernel that ran out

}  // namespace b200
