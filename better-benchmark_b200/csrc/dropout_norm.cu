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
// consecutive elements' uniforms u = (bits >> 8) * 2^-24 in [0, 1); the comparisons with p are done on
// the 24-bit integers (thresholds computed on the host), which gives the same masks. The reference's check treats
// the masks as stochastic outputs; everything else is a deterministic function of them.
//
// One warp owns a row: lane l holds vectors l, l+32, .. (8 elements each) in registers between the
// sum of squares and the normalisation, so x and residual are read once.
#include "rowwise.cuh"

namespace b200 {
namespace {

// The ten round keys of one seed: key + r * (0x9E3779B9, 0xBB67AE85). They are the same for every
// element, so a kernel computes them once and every call only multiplies and xors.
struct PhiloxKeys {
  uint32_t k0[10], k1[10];
};
__device__ __forceinline__ PhiloxKeys philox_keys(unsigned long long seed) {
  PhiloxKeys k;
  uint32_t a = (uint32_t)seed, b = (uint32_t)(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    k.k0[r] = a;
    k.k1[r] = b;
    a += 0x9E3779B9u;
    b += 0xBB67AE85u;
  }
  return k;
}

__device__ __forceinline__ uint4 philox4x32_10(uint4 c, const PhiloxKeys& k) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c.x), lo0 = 0xD2511F53u * c.x;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c.z), lo1 = 0xCD9E8D57u * c.z;
    c = make_uint4(hi1 ^ c.y ^ k.k0[r], lo1, hi0 ^ c.w ^ k.k1[r], lo0);
  }
  return c;
}

// Random words for the elements [e0, e0+8) of mask number `which`; e0 is a multiple of 8.
__device__ __forceinline__ void random_words8(unsigned long long e0, uint32_t which, const PhiloxKeys& k,
                                              uint32_t (&w)[8]) {
  const unsigned long long g = e0 >> 2;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const unsigned long long gi = g + h;
    const uint4 r = philox4x32_10(make_uint4((uint32_t)gi, (uint32_t)(gi >> 32), which, 0u), k);
    w[4 * h + 0] = r.x;
    w[4 * h + 1] = r.y;
    w[4 * h + 2] = r.z;
    w[4 * h + 3] = r.w;
  }
}

struct DropoutNormParams {
  const void* x;
  const float* residual;
  const float* weight;
  const long long* seeds;
  int seed_index0, seed_index1;
  // An element is kept when the top 24 bits of its random word, n, satisfy n >= keep_from: the
  // uniform is u = n * 2^-24, and both "T(u) > T(p)" and "u > p" are monotonic in n, so the host
  // turns each into one integer threshold (see thresholds() below).
  uint32_t keep_from0, keep_from1;
  float scale, eps;
  unsigned char* keep0;
  float* sum;
  float* rstd;
  unsigned char* keep1;
  void* y;
  long long rows;
  int cols;
};

// Mask bytes (0 / 1) and the same mask as fp32 pairs for eight random words.
__device__ __forceinline__ void masks8(const uint32_t (&w)[8], uint32_t keep_from, uint2& bytes, f32x2 (&m)[4]) {
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const bool ka = (w[2 * j] >> 8) >= keep_from, kb = (w[2 * j + 1] >> 8) >= keep_from;
    const uint32_t two = (ka ? 1u : 0u) | (kb ? 0x100u : 0u);
    if (j < 2) lo |= two << (16 * j);
    else hi |= two << (16 * (j - 2));
    m[j] = pack2(ka ? 1.f : 0.f, kb ? 1.f : 0.f);
  }
  bytes = make_uint2(lo, hi);
}

template <typename T, int CH>
__global__ void __launch_bounds__(128) dropout_rms_norm_kernel(DropoutNormParams p) {
  const int lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  const int nv = p.cols >> 3;  // vectors of 8 elements per row
  const unsigned long long s0 = (unsigned long long)p.seeds[p.seed_index0];
  const unsigned long long s1 = (unsigned long long)p.seeds[p.seed_index1];
  const PhiloxKeys keys0 = philox_keys(s0), keys1 = philox_keys(s1);
  const f32x2 scale2 = splat2(p.scale);

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

    f32x2 s[CH][4];
    f32x2 sq2 = pack2(0.f, 0.f);
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int v = lane + 32 * c;
      if (v < nv) {
        f32x2 xp[4], r[4], m[4];
        Pairs<T>::unpack(xv[c], xp);
        {
          f32x2 t[2];
          Pairs<float>::unpack(ra[c], t);
          r[0] = t[0]; r[1] = t[1];
          Pairs<float>::unpack(rb[c], t);
          r[2] = t[0]; r[3] = t[1];
        }
        uint32_t w[8];
        random_words8(row0 + 8ull * v, 0u, keys0, w);
        uint2 bytes;
        masks8(w, p.keep_from0, bytes, m);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          // keep * x is already a value of T; its product with 1/(1-p) is rounded to T, as in the graph
          const f32x2 scaled = Pairs<T>::word(Pairs<T>::narrow(mul2(mul2(xp[j], m[j]), scale2)));
          s[c][j] = add2(r[j], scaled);
          sq2 = fma2(s[c][j], s[c][j], sq2);
        }
        *reinterpret_cast<uint2*>(p.keep0 + row0 + 8 * v) = bytes;
        float* so = p.sum + row0 + 8 * v;
        {
          const f32x2 t0[2] = {s[c][0], s[c][1]}, t1[2] = {s[c][2], s[c][3]};
          st_stream(so, Pairs<float>::pack(t0));
          st_stream(so + 4, Pairs<float>::pack(t1));
        }
      }
    }
    const float sq = warp_reduce<SumOp>(hsum2(sq2));
    const float rstd = rsqrtf(sq / (float)p.cols + p.eps);
    if (lane == 0) p.rstd[row] = rstd;
    const f32x2 rstd2 = splat2(rstd);

    T* yr = reinterpret_cast<T*>(p.y) + row0;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int v = lane + 32 * c;
      if (v < nv) {
        uint32_t w[8];
        random_words8(row0 + 8ull * v, 1u, keys1, w);
        uint2 bytes;
        f32x2 m[4], wt[4];
        masks8(w, p.keep_from1, bytes, m);
        {
          f32x2 t[2];
          Pairs<float>::unpack(ld_keep(p.weight + 8 * v), t);
          wt[0] = t[0]; wt[1] = t[1];
          Pairs<float>::unpack(ld_keep(p.weight + 8 * v + 4), t);
          wt[2] = t[0]; wt[3] = t[1];
        }
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          o[j] = Pairs<T>::narrow(mul2(mul2(mul2(wt[j], mul2(s[c][j], rstd2)), m[j]), scale2));
        *reinterpret_cast<uint2*>(p.keep1 + row0 + 8 * v) = bytes;
        st_stream(yr + 8 * v, make_uint4(o[0], o[1], o[2], o[3]));
      }
    }
  }
}

// CTAs per SM that the register allocation has to leave room for, by chunks per lane.
constexpr int min_ctas(int ch) { return ch <= 1 ? 7 : ch <= 3 ? 5 : ch == 4 ? 4 : 1; }

struct DropoutLayerNormParams {
  const void* x;
  const float* residual;
  const float* weight;
  const float* bias;
  const long long* seeds;
  int seed_index;
  uint32_t keep_from;  // as in DropoutNormParams
  float scale, eps;
  unsigned char* keep;
  float* xhat;
  float* y;
  float* rstd_over_n;
  long long rows;
  int cols;
};

// Dropout -> residual add -> LayerNorm (reference repros/canonical/var_mean_01fbd6c1b27f/repro.py:24-44):
//   keep = T(rand(seed[i])) > p;  sum = float(T(T(keep * x) * scale)) + residual;
//   var, mean = var_mean(sum);  rstd = rsqrt(var + eps);  xhat = (sum - mean) * rstd;
//   y = xhat * w + b;  outputs (keep, xhat, y, rstd / cols).
// Same row ownership as above; the variance is the centred sum of squares of the row in registers.
template <typename T, int CH>
__global__ void __launch_bounds__(128, min_ctas(CH)) dropout_layer_norm_kernel(DropoutLayerNormParams p) {
  const int lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  const int nv = p.cols >> 3;
  const unsigned long long seed = (unsigned long long)p.seeds[p.seed_index];
  const PhiloxKeys keys = philox_keys(seed);
  const f32x2 scale2 = splat2(p.scale);
  const float n = (float)p.cols;

  for (long long row = (long long)blockIdx.x * warps + (threadIdx.x >> 5); row < p.rows;
       row += (long long)gridDim.x * warps) {
    const unsigned long long row0 = (unsigned long long)row * (unsigned long long)p.cols;
    const T* xr = reinterpret_cast<const T*>(p.x) + row0;
    const float* rr = p.residual + row0;

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

    f32x2 s[CH][4];
    f32x2 sum2 = pack2(0.f, 0.f);
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int v = lane + 32 * c;
      if (v < nv) {
        f32x2 xp[4], r[4], m[4];
        Pairs<T>::unpack(xv[c], xp);
        {
          f32x2 t[2];
          Pairs<float>::unpack(ra[c], t);
          r[0] = t[0]; r[1] = t[1];
          Pairs<float>::unpack(rb[c], t);
          r[2] = t[0]; r[3] = t[1];
        }
        uint32_t w[8];
        random_words8(row0 + 8ull * v, 0u, keys, w);
        uint2 bytes;
        masks8(w, p.keep_from, bytes, m);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const f32x2 scaled = Pairs<T>::word(Pairs<T>::narrow(mul2(mul2(xp[j], m[j]), scale2)));
          s[c][j] = add2(scaled, r[j]);
          sum2 = add2(sum2, s[c][j]);
        }
        *reinterpret_cast<uint2*>(p.keep + row0 + 8 * v) = bytes;
      }
    }
    const float mean = warp_reduce<SumOp>(hsum2(sum2)) / n;
    const f32x2 mean2 = splat2(mean);
    f32x2 sq2 = pack2(0.f, 0.f);
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      if (lane + 32 * c < nv) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          s[c][j] = sub2(s[c][j], mean2);
          sq2 = fma2(s[c][j], s[c][j], sq2);
        }
      }
    }
    const float rstd = rsqrtf(warp_reduce<SumOp>(hsum2(sq2)) / n + p.eps);
    if (lane == 0) p.rstd_over_n[row] = rstd / n;
    const f32x2 rstd2 = splat2(rstd);

#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int v = lane + 32 * c;
      if (v < nv) {
        f32x2 wt[4], bs[4], xh[4], out[4];
        {
          f32x2 t[2];
          Pairs<float>::unpack(ld_keep(p.weight + 8 * v), t);
          wt[0] = t[0]; wt[1] = t[1];
          Pairs<float>::unpack(ld_keep(p.weight + 8 * v + 4), t);
          wt[2] = t[0]; wt[3] = t[1];
          Pairs<float>::unpack(ld_keep(p.bias + 8 * v), t);
          bs[0] = t[0]; bs[1] = t[1];
          Pairs<float>::unpack(ld_keep(p.bias + 8 * v + 4), t);
          bs[2] = t[0]; bs[3] = t[1];
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          xh[j] = mul2(s[c][j], rstd2);
          out[j] = add2(mul2(xh[j], wt[j]), bs[j]);
        }
        float* xo = p.xhat + row0 + 8 * v;
        float* yo = p.y + row0 + 8 * v;
        const f32x2 a0[2] = {xh[0], xh[1]}, a1[2] = {xh[2], xh[3]};
        const f32x2 b0[2] = {out[0], out[1]}, b1[2] = {out[2], out[3]};
        st_stream(xo, Pairs<float>::pack(a0));
        st_stream(xo + 4, Pairs<float>::pack(a1));
        st_stream(yo, Pairs<float>::pack(b0));
        st_stream(yo + 4, Pairs<float>::pack(b1));
      }
    }
  }
}

struct DropoutAddParams {
  const void* x;
  const float* residual;
  const long long* seeds;
  int seed_index;
  uint32_t keep_from;
  float scale;
  unsigned char* keep;
  float* sum;
  long long vecs;  // vectors of 8 elements
};

// Dropout -> residual add with no reduction (reference repros/canonical/pointwise_4b076ed1ff41/repro.py:24-32):
//   keep = T(rand(seed[i])) > p;  sum = residual + float(T(T(keep * x) * scale)).
// Flat over the elements, two vectors of 8 in flight per thread.
template <typename T>
__global__ void __launch_bounds__(256) dropout_add_kernel(DropoutAddParams p) {
  const PhiloxKeys keys = philox_keys((unsigned long long)p.seeds[p.seed_index]);
  const f32x2 scale2 = splat2(p.scale);
  const long long stride = (long long)gridDim.x * blockDim.x;
  const T* x = reinterpret_cast<const T*>(p.x);
  for (long long v0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; v0 < p.vecs; v0 += 2 * stride) {
    const long long vi[2] = {v0, v0 + stride};
    uint4 xv[2], ra[2], rb[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (vi[u] < p.vecs) {
        xv[u] = ld_stream(x + 8 * vi[u]);
        ra[u] = ld_stream(p.residual + 8 * vi[u]);
        rb[u] = ld_stream(p.residual + 8 * vi[u] + 4);
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (vi[u] < p.vecs) {
        f32x2 xp[4], r[4], m[4], s[4];
        Pairs<T>::unpack(xv[u], xp);
        {
          f32x2 t[2];
          Pairs<float>::unpack(ra[u], t);
          r[0] = t[0]; r[1] = t[1];
          Pairs<float>::unpack(rb[u], t);
          r[2] = t[0]; r[3] = t[1];
        }
        uint32_t w[8];
        random_words8(8ull * (unsigned long long)vi[u], 0u, keys, w);
        uint2 bytes;
        masks8(w, p.keep_from, bytes, m);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          s[j] = add2(r[j], Pairs<T>::word(Pairs<T>::narrow(mul2(mul2(xp[j], m[j]), scale2))));
        *reinterpret_cast<uint2*>(p.keep + 8 * vi[u]) = bytes;
        const f32x2 t0[2] = {s[0], s[1]}, t1[2] = {s[2], s[3]};
        st_stream(p.sum + 8 * vi[u], Pairs<float>::pack(t0));
        st_stream(p.sum + 8 * vi[u] + 4, Pairs<float>::pack(t1));
      }
    }
  }
}

// Smallest n in [0, 2^24] whose uniform n * 2^-24 is kept, for a predicate that is monotonic in n.
template <typename Keep>
uint32_t first_kept(Keep keep) {
  uint32_t lo = 0, hi = 1u << 24;  // the answer lies in [lo, hi]; hi = 2^24 means "never kept"
  while (lo < hi) {
    const uint32_t mid = lo + (hi - lo) / 2;
    if (keep((float)mid * 0x1p-24f)) hi = mid;
    else lo = mid + 1;
  }
  return lo;
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
  else if (nv <= 96) dropout_rms_norm_kernel<T, 3><<<grid, 32 * warps, 0, st>>>(p);
  else if (nv <= 128) dropout_rms_norm_kernel<T, 4><<<grid, 32 * warps, 0, st>>>(p);
  else if (nv <= 192) dropout_rms_norm_kernel<T, 6><<<grid, 32 * warps, 0, st>>>(p);
  else dropout_rms_norm_kernel<T, 8><<<grid, 32 * warps, 0, st>>>(p);
  return launch_status("b200_dropout_rms_norm");
}

template <typename T>
int launch_dropout_layer_norm(const DropoutLayerNormParams& p, cudaStream_t st) {
  const int nv = p.cols >> 3;
  const int warps = 4;
  const long long want = (p.rows + warps - 1) / warps;
  const long long cap = (long long)device_info().sm_count * 32;
  const int grid = (int)(want < cap ? want : cap);
  if (nv <= 32) dropout_layer_norm_kernel<T, 1><<<grid, 32 * warps, 0, st>>>(p);
  else if (nv <= 64) dropout_layer_norm_kernel<T, 2><<<grid, 32 * warps, 0, st>>>(p);
  else if (nv <= 96) dropout_layer_norm_kernel<T, 3><<<grid, 32 * warps, 0, st>>>(p);
  else if (nv <= 128) dropout_layer_norm_kernel<T, 4><<<grid, 32 * warps, 0, st>>>(p);
  else if (nv <= 192) dropout_layer_norm_kernel<T, 6><<<grid, 32 * warps, 0, st>>>(p);
  else dropout_layer_norm_kernel<T, 8><<<grid, 32 * warps, 0, st>>>(p);
  return launch_status("b200_dropout_layer_norm");
}

// ---- softmax(x + bias) followed by dropout -----------------------------------------------------
// The region (reference repros/canonical/amax_sum_089fdab8f22b/repro.py:24-46, attention
// probabilities of a T5 block in training), per row of `cols` scores:
//   logits = T(float(x) + bias)            amax = max(logits)       e = exp(logits - amax)
//   sum = sum(e)                           prob = T(e / sum)
//   keep = T(rand(seed[i])) > p            y = T(T(keep * prob) * scale)
// with outputs (logits, amax, sum, keep, y). x is a contiguous [B*H, Sq, cols] tensor of 16-bit
// elements; bias is fp32 [B, H, Sq, cols] with arbitrary element strides (the captured graph hands
// over a permuted tensor whose head dimension is the unit-stride one); all outputs are contiguous.
// A warp owns a row, a lane the 8-element vectors l, l + 32, ..; the row stays in registers from
// the load to the last store. Random numbers as in the kernels above (counter = flat element
// index / 4, mask number 0).
struct SoftmaxDropoutParams {
  const void* x;
  const float* bias;
  long long sb, sh, sq, sk;  // element strides of bias
  int heads, seq_q, cols;
  long long rows;            // B * H * Sq
  const long long* seeds;
  int seed_index;
  uint32_t keep_from;
  float scale;
  void* logits;
  float* amax;
  float* sum;
  unsigned char* keep;
  void* y;
};

template <typename T, int CH>
__global__ void __launch_bounds__(128) softmax_dropout_kernel(SoftmaxDropoutParams p) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const PhiloxKeys keys = philox_keys((unsigned long long)p.seeds[p.seed_index]);
  const int nv = p.cols >> 3;
  const T* x = reinterpret_cast<const T*>(p.x);
  T* logits = reinterpret_cast<T*>(p.logits);
  T* y = reinterpret_cast<T*>(p.y);
  for (long long row = (long long)blockIdx.x * 4 + warp; row < p.rows; row += (long long)gridDim.x * 4) {
    const long long bh = row / p.seq_q;
    const int q = (int)(row - bh * p.seq_q);
    const long long b = bh / p.heads;
    const int h = (int)(bh - b * p.heads);
    const float* brow = p.bias + b * p.sb + h * p.sh + q * p.sq;
    const long long base = row * p.cols;
    float l[CH][8];
    float mx = -INFINITY;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int v = lane + 32 * c;
      if (v < nv) {
        float f[8], bv[8];
        const uint4 raw = ld_stream(x + base + 8 * v);
#pragma unroll
        for (int j = 0; j < 8; ++j) bv[j] = __ldg(brow + (long long)(8 * v + j) * p.sk);
        Elem<T>::unpack(raw, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          l[c][j] = Elem<T>::to_f32(Elem<T>::from_f32(f[j] + bv[j]));  // the graph rounds the logits to T
          mx = fmaxf(mx, l[c][j]);
        }
        st_stream(logits + base + 8 * v, Elem<T>::pack(l[c]));
      }
    }
    mx = warp_reduce<MaxOp>(mx);
    float s = 0.f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      if (lane + 32 * c < nv) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          l[c][j] = expf(l[c][j] - mx);
          s += l[c][j];
        }
      }
    }
    s = warp_reduce<SumOp>(s);
    if (lane == 0) {
      p.amax[row] = mx;
      p.sum[row] = s;
    }
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int v = lane + 32 * c;
      if (v < nv) {
        uint32_t w[8];
        random_words8((unsigned long long)(base + 8 * v), 0u, keys, w);
        uint2 bytes;
        f32x2 m[4];
        masks8(w, p.keep_from, bytes, m);
        float o[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float ma, mb;
          unpack2(m[j], ma, mb);
          const float pa = Elem<T>::to_f32(Elem<T>::from_f32(l[c][2 * j] / s));
          const float pb = Elem<T>::to_f32(Elem<T>::from_f32(l[c][2 * j + 1] / s));
          o[2 * j] = (ma * pa) * p.scale;      // keep * prob is exact in T; one rounding at the end
          o[2 * j + 1] = (mb * pb) * p.scale;
        }
        *reinterpret_cast<uint2*>(p.keep + base + 8 * v) = bytes;
        st_stream(y + base + 8 * v, Elem<T>::pack(o));
      }
    }
  }
}

template <typename T>
int launch_softmax_dropout(const SoftmaxDropoutParams& p, cudaStream_t st) {
  const int nv = p.cols >> 3;
  const long long want = (p.rows + 3) / 4;
  const long long cap = (long long)device_info().sm_count * 32;
  const int grid = (int)(want < cap ? want : cap);
  if (nv <= 32) softmax_dropout_kernel<T, 1><<<grid, 128, 0, st>>>(p);
  else if (nv <= 64) softmax_dropout_kernel<T, 2><<<grid, 128, 0, st>>>(p);
  else softmax_dropout_kernel<T, 4><<<grid, 128, 0, st>>>(p);
  return launch_status("b200_softmax_dropout");
}

// Threshold of the mask whose draw is narrowed to the tensor dtype before the comparison with p.
uint32_t narrowed_keep_from(float pf, int x_dtype) {
  if (x_dtype == B200_BF16) {
    const float pn = __bfloat162float(__float2bfloat16_rn(pf));
    return first_kept([&](float u) { return __bfloat162float(__float2bfloat16_rn(u)) > pn; });
  }
  const float pn = __half2float(__float2half_rn(pf));
  return first_kept([&](float u) { return __half2float(__float2half_rn(u)) > pn; });
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
  const float pf = (float)p;
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
  // second mask: u > p in fp32; first mask: the draw and p are both narrowed to T before the comparison
  q.keep_from1 = first_kept([&](float u) { return u > pf; });
  q.keep_from0 = narrowed_keep_from(pf, x_dtype);
  if (q.keep_from0 >= (1u << 24) || q.keep_from1 >= (1u << 24))
    return fail(B200_ERR_UNSUPPORTED, "b200_dropout_rms_norm: p = %g keeps nothing at 24-bit resolution", p);
  if (x_dtype == B200_BF16) return launch_dropout_rms_norm<__nv_bfloat16>(q, st);
  return launch_dropout_rms_norm<__half>(q, st);
}

extern "C" int b200_dropout_layer_norm(const void* x, const void* residual, const void* weight, const void* bias,
                                       const int64_t* seeds, int32_t seed_index, double p, double eps, void* keep,
                                       void* xhat, void* y, void* rstd_over_n, int64_t rows, int64_t cols,
                                       int32_t x_dtype, void* stream) {
  if (rows < 0 || cols < 0) return fail(B200_ERR_INVALID, "b200_dropout_layer_norm: negative size");
  if (rows == 0) return B200_OK;
  if (!x || !residual || !weight || !bias || !seeds || !keep || !xhat || !y || !rstd_over_n)
    return fail(B200_ERR_INVALID, "b200_dropout_layer_norm: null argument");
  if (seed_index < 0) return fail(B200_ERR_INVALID, "b200_dropout_layer_norm: negative seed index");
  if (!(p >= 0.0 && p < 1.0)) return fail(B200_ERR_INVALID, "b200_dropout_layer_norm: p must be in [0, 1)");
  if (x_dtype != B200_BF16 && x_dtype != B200_F16)
    return fail(B200_ERR_UNSUPPORTED, "b200_dropout_layer_norm: x must be bf16 or fp16 (dtype %d)", x_dtype);
  if (cols == 0 || cols % 8 != 0 || cols > 2048)
    return fail(B200_ERR_UNSUPPORTED,
                "b200_dropout_layer_norm: row length %lld (supported: multiples of 8 up to 2048)", (long long)cols);
  if (!aligned16(x) || !aligned16(residual) || !aligned16(weight) || !aligned16(bias) || !aligned16(xhat) ||
      !aligned16(y) || (reinterpret_cast<uintptr_t>(keep) & 7u))
    return fail(B200_ERR_ALIGNMENT, "b200_dropout_layer_norm: tensors must be 16-byte aligned (mask 8-byte)");
  DropoutLayerNormParams q;
  q.x = x;
  q.residual = static_cast<const float*>(residual);
  q.weight = static_cast<const float*>(weight);
  q.bias = static_cast<const float*>(bias);
  q.seeds = reinterpret_cast<const long long*>(seeds);
  q.seed_index = seed_index;
  q.keep_from = narrowed_keep_from((float)p, x_dtype);
  if (q.keep_from >= (1u << 24))
    return fail(B200_ERR_UNSUPPORTED, "b200_dropout_layer_norm: p = %g keeps nothing at 24-bit resolution", p);
  q.scale = (float)(1.0 / (1.0 - p));
  q.eps = (float)eps;
  q.keep = static_cast<unsigned char*>(keep);
  q.xhat = static_cast<float*>(xhat);
  q.y = static_cast<float*>(y);
  q.rstd_over_n = static_cast<float*>(rstd_over_n);
  q.rows = rows;
  q.cols = (int)cols;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (x_dtype == B200_BF16) return launch_dropout_layer_norm<__nv_bfloat16>(q, st);
  return launch_dropout_layer_norm<__half>(q, st);
}

extern "C" int b200_dropout_add(const void* x, const void* residual, const int64_t* seeds, int32_t seed_index,
                                double p, void* keep, void* sum, int64_t n, int32_t x_dtype, void* stream) {
  if (n < 0) return fail(B200_ERR_INVALID, "b200_dropout_add: negative size");
  if (n == 0) return B200_OK;
  if (!x || !residual || !seeds || !keep || !sum) return fail(B200_ERR_INVALID, "b200_dropout_add: null argument");
  if (seed_index < 0) return fail(B200_ERR_INVALID, "b200_dropout_add: negative seed index");
  if (!(p >= 0.0 && p < 1.0)) return fail(B200_ERR_INVALID, "b200_dropout_add: p must be in [0, 1)");
  if (x_dtype != B200_BF16 && x_dtype != B200_F16)
    return fail(B200_ERR_UNSUPPORTED, "b200_dropout_add: x must be bf16 or fp16 (dtype %d)", x_dtype);
  if (n % 8 != 0) return fail(B200_ERR_UNSUPPORTED, "b200_dropout_add: %lld elements (supported: multiples of 8)", (long long)n);
  if (!aligned16(x) || !aligned16(residual) || !aligned16(sum) || (reinterpret_cast<uintptr_t>(keep) & 7u))
    return fail(B200_ERR_ALIGNMENT, "b200_dropout_add: tensors must be 16-byte aligned (mask 8-byte)");
  DropoutAddParams q;
  q.x = x;
  q.residual = static_cast<const float*>(residual);
  q.seeds = reinterpret_cast<const long long*>(seeds);
  q.seed_index = seed_index;
  q.keep_from = narrowed_keep_from((float)p, x_dtype);
  if (q.keep_from >= (1u << 24))
    return fail(B200_ERR_UNSUPPORTED, "b200_dropout_add: p = %g keeps nothing at 24-bit resolution", p);
  q.scale = (float)(1.0 / (1.0 - p));
  q.keep = static_cast<unsigned char*>(keep);
  q.sum = static_cast<float*>(sum);
  q.vecs = n / 8;
  const long long want = (q.vecs + 2 * 256 - 1) / (2 * 256);
  const long long cap = (long long)device_info().sm_count * 32;
  const int grid = (int)(want < cap ? want : cap);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (x_dtype == B200_BF16) dropout_add_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(q);
  else dropout_add_kernel<__half><<<grid, 256, 0, st>>>(q);
  return launch_status("b200_dropout_add");
}

extern "C" int b200_softmax_dropout(const void* x, const void* bias, int64_t batch, int64_t heads, int64_t seq_q,
                                    int64_t cols, int64_t bias_stride_b, int64_t bias_stride_h,
                                    int64_t bias_stride_q, int64_t bias_stride_k, const int64_t* seeds,
                                    int32_t seed_index, double p, void* logits, void* amax, void* sum, void* keep,
                                    void* y, int32_t x_dtype, void* stream) {
  if (batch < 0 || heads < 0 || seq_q < 0 || cols < 0) return fail(B200_ERR_INVALID, "b200_softmax_dropout: negative size");
  const long long rows = batch * heads * seq_q;
  if (rows == 0 || cols == 0) return B200_OK;
  if (!x || !bias || !seeds || !logits || !amax || !sum || !keep || !y)
    return fail(B200_ERR_INVALID, "b200_softmax_dropout: null argument");
  if (seed_index < 0) return fail(B200_ERR_INVALID, "b200_softmax_dropout: negative seed index");
  if (!(p >= 0.0 && p < 1.0)) return fail(B200_ERR_INVALID, "b200_softmax_dropout: p must be in [0, 1)");
  if (x_dtype != B200_BF16 && x_dtype != B200_F16)
    return fail(B200_ERR_UNSUPPORTED, "b200_softmax_dropout: x must be bf16 or fp16 (dtype %d)", x_dtype);
  if (cols % 8 != 0 || cols > 1024)
    return fail(B200_ERR_UNSUPPORTED, "b200_softmax_dropout: %lld columns (supported: multiples of 8 up to 1024)",
                (long long)cols);
  if (!aligned16(x) || !aligned16(logits) || !aligned16(y) || (reinterpret_cast<uintptr_t>(keep) & 7u))
    return fail(B200_ERR_ALIGNMENT, "b200_softmax_dropout: tensors must be 16-byte aligned (mask 8-byte)");
  SoftmaxDropoutParams q;
  q.x = x;
  q.bias = static_cast<const float*>(bias);
  q.sb = bias_stride_b; q.sh = bias_stride_h; q.sq = bias_stride_q; q.sk = bias_stride_k;
  q.heads = (int)heads; q.seq_q = (int)seq_q; q.cols = (int)cols;
  q.rows = rows;
  q.seeds = reinterpret_cast<const long long*>(seeds);
  q.seed_index = seed_index;
  q.keep_from = narrowed_keep_from((float)p, x_dtype);
  if (q.keep_from >= (1u << 24))
    return fail(B200_ERR_UNSUPPORTED, "b200_softmax_dropout: p = %g keeps nothing at 24-bit resolution", p);
  q.scale = (float)(1.0 / (1.0 - p));
  q.logits = logits;
  q.amax = static_cast<float*>(amax);
  q.sum = static_cast<float*>(sum);
  q.keep = static_cast<unsigned char*>(keep);
  q.y = y;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return x_dtype == B200_BF16 ? launch_softmax_dropout<__nv_bfloat16>(q, st) : launch_softmax_dropout<__half>(q, st);
}
