// LayerNorm / RMSNorm forward over the last dimension, and row-wise var_mean.
//
// Replaces the Triton kernels of the row-normalisation repros in the reference
// (repros/canonical/var_mean_f8ec553e339e/oracle.py:50-84, var_mean_af505388b035/oracle.py:11-40,
// var_mean_f7906a6c6957/oracle.py:14-50, mean_f667cd8901af/oracle.py:36-72).
//
// Evaluation order, as the decomposed aten graphs have it:
//   LayerNorm: mean = sum(x)/n; var = sum((x-mean)^2)/(n-correction); rstd = 1/sqrt(var+eps)
//              y = ((x - mean) * rstd) * w + b
//   RMSNorm  : ms = sum(x*x)/n; rstd = 1/sqrt(ms+eps); y = (x * rstd) * w
// The variance is the centred second pass over the row held in registers. Statistics are fp32.
// Any of y, mean, rstd, var may be null (var_mean alone = no y, no rstd).
#include "rowwise.cuh"

namespace b200 {

struct NormFwdParams {
  const void* x;
  const void* w;  // may be null
  const void* b;  // may be null
  void* y;        // may be null
  float* mean_out;
  float* rstd_out;
  float* var_out;
  long long rows;
  int n;
  long long x_row_stride, y_row_stride;  // elements
  int w_dtype;
  float eps;
  float inv_n;      // 1 / n
  float inv_denom;  // 1 / (n - correction)
  int rms;
};

// rsqrtf is the 2-ulp hardware approximation aten's CUDA rsqrt uses as well.
__device__ __forceinline__ float precise_rsqrt(float v) { return rsqrtf(v); }

template <typename Tin, typename Tout, int CH, bool BLOCK>
__global__ void __launch_bounds__(BLOCK ? 512 : 256)
norm_fwd_resident_kernel(const NormFwdParams p) {
  constexpr int V = Elem<Tin>::V;
  __shared__ float red[32];
  const int lane = group_lane<BLOCK>();
  const int G = group_size<BLOCK>();
  const long long row = group_row<BLOCK>();
  if (row >= p.rows) return;

  const Tin* x = reinterpret_cast<const Tin*>(p.x) + row * p.x_row_stride;
  const int nv = p.n / V;

  uint4 raw[CH];
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int j = c * G + lane;
    if (j < nv) raw[c] = ld_stream(x + (long long)j * V);
  }
  float v[CH][V];
  float s = 0.f;
  if (p.rms) {
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      if (c * G + lane < nv) {
        Elem<Tin>::unpack(raw[c], v[c]);
#pragma unroll
        for (int i = 0; i < V; ++i) s += v[c][i] * v[c][i];
      }
    }
  } else {
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      if (c * G + lane < nv) {
        Elem<Tin>::unpack(raw[c], v[c]);
#pragma unroll
        for (int i = 0; i < V; ++i) s += v[c][i];
      }
    }
  }
  s = group_reduce<SumOp, BLOCK>(s, red);

  float mean = 0.f, var, rstd;
  if (p.rms) {
    var = s * p.inv_n;
    rstd = precise_rsqrt(var + p.eps);
  } else {
    mean = s * p.inv_n;
    float q = 0.f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int j = c * G + lane;
      if (j < nv) {
#pragma unroll
        for (int i = 0; i < V; ++i) {
          v[c][i] = v[c][i] - mean;  // keep the centred value: the output needs it again
          q += v[c][i] * v[c][i];
        }
      }
    }
    q = group_reduce<SumOp, BLOCK>(q, red);
    var = q * p.inv_denom;
    rstd = precise_rsqrt(var + p.eps);
  }
  if (lane == 0) {
    if (p.mean_out) p.mean_out[row] = mean;
    if (p.rstd_out) p.rstd_out[row] = rstd;
    if (p.var_out) p.var_out[row] = var;
  }
  if (p.y == nullptr) return;

  Tout* y = reinterpret_cast<Tout*>(p.y) + row * p.y_row_stride;
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int j = c * G + lane;
    if (j < nv) {
      float o[V];
#pragma unroll
      for (int i = 0; i < V; ++i) o[i] = v[c][i] * rstd;
      if (p.w) {
        float wf[V];
        load_param<V>(p.w, p.w_dtype, (long long)j * V, wf);
#pragma unroll
        for (int i = 0; i < V; ++i) o[i] = o[i] * wf[i];
      }
      if (p.b) {
        float bf[V];
        load_param<V>(p.b, p.w_dtype, (long long)j * V, bf);
#pragma unroll
        for (int i = 0; i < V; ++i) o[i] = o[i] + bf[i];
      }
      store_converted<Tout, V>(y + (long long)j * V, o);
    }
  }
}

// Element-wise kernel for ragged, unaligned or very long rows: one CTA per row, sweeps over
// global memory (the second and third sweep of a row that fits in L2 are served from there).
template <typename Tin, typename Tout>
__global__ void __launch_bounds__(1024) norm_fwd_streaming_kernel(const NormFwdParams p) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const Tin* x = reinterpret_cast<const Tin*>(p.x) + row * p.x_row_stride;

  float s = 0.f;
  for (long long i = threadIdx.x; i < p.n; i += blockDim.x) {
    const float f = Elem<Tin>::to_f32(x[i]);
    s += p.rms ? f * f : f;
  }
  s = block_reduce<SumOp>(s, red);
  float mean = 0.f, var, rstd;
  if (p.rms) {
    var = s * p.inv_n;
  } else {
    mean = s * p.inv_n;
    float q = 0.f;
    for (long long i = threadIdx.x; i < p.n; i += blockDim.x) {
      const float d = Elem<Tin>::to_f32(x[i]) - mean;
      q += d * d;
    }
    q = block_reduce<SumOp>(q, red);
    var = q * p.inv_denom;
  }
  rstd = precise_rsqrt(var + p.eps);
  if (threadIdx.x == 0) {
    if (p.mean_out) p.mean_out[row] = mean;
    if (p.rstd_out) p.rstd_out[row] = rstd;
    if (p.var_out) p.var_out[row] = var;
  }
  if (p.y == nullptr) return;
  Tout* y = reinterpret_cast<Tout*>(p.y) + row * p.y_row_stride;
  for (long long i = threadIdx.x; i < p.n; i += blockDim.x) {
    float o = (Elem<Tin>::to_f32(x[i]) - mean) * rstd;
    if (p.w) o = o * load_param1(p.w, p.w_dtype, i);
    if (p.b) o = o + load_param1(p.b, p.w_dtype, i);
    y[i] = Elem<Tout>::from_f32(o);
  }
}

template <typename Tin, typename Tout>
static int launch_norm_fwd(const NormFwdParams& p, bool vector_ok, cudaStream_t st) {
  constexpr int V = Elem<Tin>::V;
  if (p.rows > 0x7fffffffLL) return fail(B200_ERR_UNSUPPORTED, "norm_fwd: too many rows");
  RowGeometry g;
  if (vector_ok && p.n % V == 0 && pick_row_geometry(p.n / V, &g)) {
    if (!g.block) {
      const int rows_per_cta = g.threads / 32;
      const unsigned grid = (unsigned)((p.rows + rows_per_cta - 1) / rows_per_cta);
      switch (g.ch) {
        case 1: norm_fwd_resident_kernel<Tin, Tout, 1, false><<<grid, g.threads, 0, st>>>(p); break;
        case 2: norm_fwd_resident_kernel<Tin, Tout, 2, false><<<grid, g.threads, 0, st>>>(p); break;
        default: norm_fwd_resident_kernel<Tin, Tout, 4, false><<<grid, g.threads, 0, st>>>(p); break;
      }
    } else {
      const unsigned grid = (unsigned)p.rows;
      switch (g.ch) {
        case 2: norm_fwd_resident_kernel<Tin, Tout, 2, true><<<grid, g.threads, 0, st>>>(p); break;
        case 4: norm_fwd_resident_kernel<Tin, Tout, 4, true><<<grid, g.threads, 0, st>>>(p); break;
        default: norm_fwd_resident_kernel<Tin, Tout, 8, true><<<grid, g.threads, 0, st>>>(p); break;
      }
    }
  } else {
    int threads = 1024;
    while (threads > 64 && threads / 2 >= p.n) threads /= 2;
    norm_fwd_streaming_kernel<Tin, Tout><<<(unsigned)p.rows, threads, 0, st>>>(p);
  }
  return launch_status("b200_norm_fwd");
}

}  // namespace b200

using namespace b200;

extern "C" int b200_norm_fwd(const void* x, const void* weight, const void* bias, void* y,
                             float* mean_out, float* rstd_out, float* var_out, int64_t rows,
                             int64_t n, int64_t x_row_stride, int64_t y_row_stride,
                             int32_t x_dtype, int32_t w_dtype, int32_t y_dtype, double eps,
                             double correction, int32_t rms, void* stream) {
  if (!x) return fail(B200_ERR_INVALID, "b200_norm_fwd: null x");
  if (rows < 0 || n < 0 || n > 0x7fffffffLL)
    return fail(B200_ERR_INVALID, "b200_norm_fwd: bad sizes rows=%lld n=%lld", (long long)rows, (long long)n);
  if (rows == 0) return B200_OK;
  if (n == 0) return fail(B200_ERR_INVALID, "b200_norm_fwd: empty rows have no statistics");
  if (w_dtype < 0 || w_dtype > 2) return fail(B200_ERR_INVALID, "b200_norm_fwd: bad weight dtype");

  NormFwdParams p;
  p.x = x; p.w = weight; p.b = bias; p.y = y;
  p.mean_out = mean_out; p.rstd_out = rstd_out; p.var_out = var_out;
  p.rows = rows; p.n = (int)n;
  p.x_row_stride = x_row_stride; p.y_row_stride = y_row_stride;
  p.w_dtype = w_dtype; p.eps = (float)eps; p.rms = rms ? 1 : 0;
  p.inv_n = (float)(1.0 / (double)n);
  p.inv_denom = (float)(1.0 / ((double)n - correction));  // inf/NaN for n <= correction, as aten

  const int ib = dtype_size(x_dtype), ob = dtype_size(y_dtype), wb = dtype_size(w_dtype);
  const int v_in = 16 / ib;
  const int out_chunk = v_in * ob < 16 ? v_in * ob : 16;
  const int w_chunk = v_in * wb < 16 ? v_in * wb : 16;
  bool vec = aligned16(x) && (x_row_stride * ib) % 16 == 0;
  if (y) vec = vec && reinterpret_cast<uintptr_t>(y) % out_chunk == 0 && (y_row_stride * ob) % out_chunk == 0;
  if (weight) vec = vec && reinterpret_cast<uintptr_t>(weight) % w_chunk == 0;
  if (bias) vec = vec && reinterpret_cast<uintptr_t>(bias) % w_chunk == 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);

#define B200_NORM_CASE(TI, TO, DI, DO) \
  if (x_dtype == DI && y_dtype == DO) return launch_norm_fwd<TI, TO>(p, vec, st);
  B200_NORM_CASE(float, float, B200_F32, B200_F32)
  B200_NORM_CASE(__nv_bfloat16, __nv_bfloat16, B200_BF16, B200_BF16)
  B200_NORM_CASE(__half, __half, B200_F16, B200_F16)
  B200_NORM_CASE(__nv_bfloat16, float, B200_BF16, B200_F32)
  B200_NORM_CASE(__half, float, B200_F16, B200_F32)
  B200_NORM_CASE(float, __nv_bfloat16, B200_F32, B200_BF16)
  B200_NORM_CASE(float, __half, B200_F32, B200_F16)
#undef B200_NORM_CASE
  return fail(B200_ERR_UNSUPPORTED, "b200_norm_fwd: dtype pair (%d -> %d) not built", x_dtype, y_dtype);
}
