// Dropout -> residual add -> RMSNorm -> dropout, one pass over the row.
//
// The region (reference repros/canonical/mean_014afd4984e6/repro.py:24-47, a T5 block in training):
//   keep0 = T(rand(seed[i0])) > p          s   = T(T(keep0 * x) * scale)
//   sum   = residual + float(s)            rstd = rsqrt(mean(sum^2) + eps)
//   keep1 = rand(seed[i1]) > p             y   = T((keep1 * (w * (sum * rstd))) * scale)
// with scale = 1/(1-p) and outputs (keep0, sum, rstd, keep1, y).
//
// The random numbers are Philox4x32-10 (Salmon et al., SC'11): key = the 64-bit seed read from the
// seed tensor on the device, counter = (element index / 4, mask number); each call yields four
// consecutive elements' uniforms u = (bits >> 8) * 2^-24 in [0, 1). The reference's check treats
// the masks as stochastic outputs; everything else is a deterministic function of them.
//
// One warp owns a row: lane l holds vectors l, l+32, .. (8 elements each) in registers between the
// sum of squares and the normalisation, so x and residual are read once.
#include "common.cuh"

namespace b200 {
namespace {

__device__ __forceinline__ uint4 philox4x32_10(uint4 c, uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c.x), lo0 = 0xD2511F53u * c.x;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c.z), lo1 = 0xCD9E8D57u * c.z;
    c = make_uint4(hi1 ^ c.y ^ k0, lo1, hi0 ^ c.w ^ k1, lo0);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return c;
}

__device__ __forceinline__ float uniform01(uint32_t bits) { return (float)(bits >> 8) * 0x1p-24f; }

// Eight uniforms for the elements [e0, e0+8) of mask number `which`; e0 is a multiple of 8.
__device__ __forceinline__ void uniforms8(unsigned long long e0, uint32_t which, uint32_t k0, uint32_t k1,
                                          float (&u)[8]) {
  const unsigned long long g = e0 >> 2;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const unsigned long long gi = g + h;
    const uint4 r = philox4x32_10(make_uint4((uint32_t)gi, (uint32_t)(gi >> 32), which, 0u), k0, k1);
    u[4 * h + 0] = uniform01(r.x);
    u[4 * h + 1] = uniform01(r.y);
    u[4 * h + 2] = uniform01(r.z);
    u[4 * h + 3] = uniform01(r.w);
  }
}

struct DropoutNormParams {
  const void* x;
  const float* residual;
  const float* weight;
  const long long* seeds;
  int seed_index0, seed_index1;
  float p, p_narrow, scale, eps;
  unsigned char* keep0;
  float* sum;
  float* rstd;
  unsigned char* keep1;
  void* y;
  long long rows;
  int cols;
};

template <typename T, int CH>
__global__ void __launch_bounds__(128) dropout_rms_norm_kernel(DropoutNormParams p) {
  const int lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  const int nv = p.cols >> 3;  // vectors of 8 elements per row
  const unsigned long long s0 = (unsigned long long)p.seeds[p.seed_index0];
  const unsigned long long s1 = (unsigned long long)p.seeds[p.seed_index1];
  const uint32_t k00 = (uint32_t)s0, k01 = (uint32_t)(s0 >> 32);
  const uint32_t k10 = (uint32_t)s1, k11 = (uint32_t)(s1 >> 32);

  for (long long row = (long long)blockIdx.x * warps + (threadIdx.x >> 5); row < p.rows;
       row += (long long)gridDim.x * warps) {
    const unsigned long long row0 = (unsigned long long)row * (unsigned long long)p.cols;
    const T* xr = reinterpret_cast<const T*>(p.x) + row0;
    const float* rr = p.residual + row0;

    // every load of the row is issued before the first use
    uint4 xv[CH], ra[CH], rb[CH];
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int v = lane + 32 * c;
      if (v < nv) {
        xv[c] = ld_stream(xr + 8 * v);
        ra[c] = ld_stream(rr + 8 * v);
        rb[c] = ld_stream(rr + 8 * v + 4);
      }
    }

    float s[CH][8];
    float sq = 0.f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int v = lane + 32 * c;
      if (v < nv) {
        float xf[8], r[8], u[8];
        Elem<T>::unpack(xv[c], xf);
        const float4 a = *reinterpret_cast<const float4*>(&ra[c]);
        const float4 b = *reinterpret_cast<const float4*>(&rb[c]);
        r[0] = a.x; r[1] = a.y; r[2] = a.z; r[3] = a.w;
        r[4] = b.x; r[5] = b.y; r[6] = b.z; r[7] = b.w;
        uniforms8(row0 + 8ull * v, 0u, k00, k01, u);
        uint32_t m_lo = 0, m_hi = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const bool keep = Elem<T>::to_f32(Elem<T>::from_f32(u[i])) > p.p_narrow;
          if (i < 4) m_lo |= (keep ? 1u : 0u) << (8 * i);
          else m_hi |= (keep ? 1u : 0u) << (8 * (i - 4));
          const float kept = Elem<T>::to_f32(Elem<T>::from_f32(xf[i] * (keep ? 1.f : 0.f)));
          const float scaled = Elem<T>::to_f32(Elem<T>::from_f32(kept * p.scale));
          s[c][i] = r[i] + scaled;
          sq += s[c][i] * s[c][i];
        }
        *reinterpret_cast<uint2*>(p.keep0 + row0 + 8 * v) = make_uint2(m_lo, m_hi);
        float* so = p.sum + row0 + 8 * v;
        st_stream(so, make_uint4(__float_as_uint(s[c][0]), __float_as_uint(s[c][1]), __float_as_uint(s[c][2]),
                                 __float_as_uint(s[c][3])));
        st_stream(so + 4, make_uint4(__float_as_uint(s[c][4]), __float_as_uint(s[c][5]),
                                     __float_as_uint(s[c][6]), __float_as_uint(s[c][7])));
      }
    }
    sq = warp_reduce<SumOp>(sq);
    const float rstd = rsqrtf(sq / (float)p.cols + p.eps);
    if (lane == 0) p.rstd[row] = rstd;

    T* yr = reinterpret_cast<T*>(p.y) + row0;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int v = lane + 32 * c;
      if (v < nv) {
        float u[8], o[8];
        uniforms8(row0 + 8ull * v, 1u, k10, k11, u);
        const float4 wa = __ldg(reinterpret_cast<const float4*>(p.weight + 8 * v));
        const float4 wb = __ldg(reinterpret_cast<const float4*>(p.weight + 8 * v + 4));
        const float w[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
        uint32_t m_lo = 0, m_hi = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const bool keep = u[i] > p.p;
          if (i < 4) m_lo |= (keep ? 1u : 0u) << (8 * i);
          else m_hi |= (keep ? 1u : 0u) << (8 * (i - 4));
          const float normed = w[i] * (s[c][i] * rstd);
          o[i] = (normed * (keep ? 1.f : 0.f)) * p.scale;
        }
        *reinterpret_cast<uint2*>(p.keep1 + row0 + 8 * v) = make_uint2(m_lo, m_hi);
        st_stream(yr + 8 * v, Elem<T>::pack(o));
      }
    }
  }
}

template <typename T>
int launch_dropout_rms_norm(const DropoutNormParams& p, cudaStream_t st) {
  const int nv = p.cols >> 3;
  const int warps = 4;
  const long long want = (p.rows + warps - 1) / warps;
  const long long cap = (long long)device_info().sm_count * 32;
  const int grid = (int)(want < cap ? want : cap);
  if (nv <= 32) dropout_rms_norm_kernel<T, 1><<<grid, 32 * warps, 0, st>>>(p);
  else if (nv <= 64) dropout_rms_norm_kernel<T, 2><<<grid, 32 * warps, 0, st>>>(p);
  else if (nv <= 128) dropout_rms_norm_kernel<T, 4><<<grid, 32 * warps, 0, st>>>(p);
  else dropout_rms_norm_kernel<T, 8><<<grid, 32 * warps, 0, st>>>(p);
  return launch_status("b200_dropout_rms_norm");
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int b200_dropout_rms_norm(const void* x, const void* residual, const void* weight,
                                     const int64_t* seeds, int32_t seed_index0, int32_t seed_index1,
                                     double p, double eps, void* keep0, void* sum, void* rstd, void* keep1,
                                     void* y, int64_t rows, int64_t cols, int32_t x_dtype, void* stream) {
  if (rows < 0 || cols < 0) return fail(B200_ERR_INVALID, "b200_dropout_rms_norm: negative size");
  if (rows == 0) return B200_OK;
  if (!x || !residual || !weight || !seeds || !keep0 || !sum || !rstd || !keep1 || !y)
    return fail(B200_ERR_INVALID, "b200_dropout_rms_norm: null argument");
  if (seed_index0 < 0 || seed_index1 < 0) return fail(B200_ERR_INVALID, "b200_dropout_rms_norm: negative seed index");
  if (!(p >= 0.0 && p < 1.0)) return fail(B200_ERR_INVALID, "b200_dropout_rms_norm: p must be in [0, 1)");
  if (x_dtype != B200_BF16 && x_dtype != B200_F16)
    return fail(B200_ERR_UNSUPPORTED, "b200_dropout_rms_norm: x must be bf16 or fp16 (dtype %d)", x_dtype);
  if (cols == 0 || cols % 8 != 0 || cols > 2048)
    return fail(B200_ERR_UNSUPPORTED, "b200_dropout_rms_norm: row length %lld (supported: multiples of 8 up to 2048)",
                (long long)cols);
  if (!aligned16(x) || !aligned16(residual) || !aligned16(weight) || !aligned16(sum) || !aligned16(y) ||
      (reinterpret_cast<uintptr_t>(keep0) & 7u) || (reinterpret_cast<uintptr_t>(keep1) & 7u))
    return fail(B200_ERR_ALIGNMENT, "b200_dropout_rms_norm: tensors must be 16-byte aligned (masks 8-byte)");
  DropoutNormParams q;
  q.x = x;
  q.residual = static_cast<const float*>(residual);
  q.weight = static_cast<const float*>(weight);
  q.seeds = reinterpret_cast<const long long*>(seeds);
  q.seed_index0 = seed_index0;
  q.seed_index1 = seed_index1;
  q.p = (float)p;
  q.scale = (float)(1.0 / (1.0 - p));
  q.eps = (float)eps;
  q.keep0 = static_cast<unsigned char*>(keep0);
  q.sum = static_cast<float*>(sum);
  q.rstd = static_cast<float*>(rstd);
  q.keep1 = static_cast<unsigned char*>(keep1);
  q.y = y;
  q.rows = rows;
  q.cols = (int)cols;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (x_dtype == B200_BF16) {
    q.p_narrow = __bfloat162float(__float2bfloat16_rn((float)p));
    return launch_dropout_rms_norm<__nv_bfloat16>(q, st);
  }
  q.p_narrow = __half2float(__float2half_rn((float)p));
  return launch_dropout_rms_norm<__half>(q, st);
}
