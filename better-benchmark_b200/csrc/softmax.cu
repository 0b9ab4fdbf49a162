// Row softmax / log_softmax with optional fused scale and additive (broadcast) mask.
//
// Replaces the single-tile and online Triton softmax kernels of the amax_sum* repro family
// (repros/canonical/amax_sum_20ccc18dda60/oracle.py:11-58, amax_sum_d16035e7b826/oracle.py:14-33,
// amax_sum_7079889cfc04/oracle.py:10-36 in the reference).
//
// Evaluation order follows the decomposed aten graph:
//   t = x [* scale] [+ mask]
//   f = float(t); m = amax(f); e = exp(f - m); s = sum(e); y = e / s      (softmax)
//                                           y = (f - m) - log(s)          (log_softmax)
// Two prologue flavours exist, because graphs differ in where they convert to fp32:
//   fp32   : x and mask are converted first; multiply and add run in fp32, nothing is rounded.
//   packed : (16-bit inputs) multiply and add run in the input dtype and their results are
//            rounded to it, as a 16-bit aten graph materialises them. The kernel does this with
//            packed two-element arithmetic: the product of two 16-bit values is exact in fp32,
//            so a packed multiply by a scale that is representable in the input dtype is
//            bit-identical to "convert, multiply in fp32, round"; a scale that is not
//            representable takes exactly that longer route. The packed add rounds the exact sum
//            once, where aten rounds the fp32 sum; the two differ only when the fp32 sum lands
//            exactly on a 16-bit rounding tie, by one 16-bit ulp of a logit.
// fp32 outputs: expf / logf and the IEEE division. 16-bit outputs: the natural exponential is
// evaluated pairwise as a hardware 2^y with the rounding of y compensated (the accuracy class of
// expf, see exp_pair_compensated in rowwise.cuh) and e / s as e * (1 / s) with a correctly rounded
// reciprocal; both deviations are three orders of magnitude below half a 16-bit ulp. Building with
// -DB200_SOFTMAX_FAST_EXP drops the compensation (the bare ex2.approx that Triton's tl.exp emits);
// that build is for measurements only.
#include "rowwise.cuh"

#include <type_traits>

namespace b200 {

#define B200_SOFTMAX_LOG 1
#define B200_SOFTMAX_SCALE 2
#define B200_SOFTMAX_ROUND 4  // packed prologue semantics for 16-bit inputs

struct SoftmaxParams {
  const void* x;
  const void* mask;  // may be null; same dtype as x
  void* y;
  long long rows;
  int n;
  RowMap xmap, mmap, ymap;
  float scale;
  int has_scale;
  int scale_exact16;  // scale survives a round trip through the input dtype
  int log_mode;
};

// Maximum that ignores NaN operands. aten.amax keeps NaNs, but a NaN element makes the sum, and
// with it every output of the row, NaN either way.
struct FastMax {
  static __device__ __forceinline__ float identity() { return -INFINITY; }
  static __device__ __forceinline__ float apply(float a, float b) { return fmaxf(a, b); }
};

// Packed two-element views of the 16-bit types.
template <typename T>
struct Pair;
template <>
struct Pair<__half> {
  using type = __half2;
  static __device__ __forceinline__ __half2 splat(float v) { return __float2half2_rn(v); }
  static __device__ __forceinline__ float2 widen(__half2 v) { return __half22float2(v); }
  static __device__ __forceinline__ __half2 narrow(float a, float b) { return __floats2half2_rn(a, b); }
};
template <>
struct Pair<__nv_bfloat16> {
  using type = __nv_bfloat162;
  static __device__ __forceinline__ __nv_bfloat162 splat(float v) { return __float2bfloat162_rn(v); }
  static __device__ __forceinline__ float2 widen(__nv_bfloat162 v) {
    const uint32_t w = *reinterpret_cast<const uint32_t*>(&v);
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
  }
  static __device__ __forceinline__ __nv_bfloat162 narrow(float a, float b) {
    return __floats2bfloat162_rn(a, b);
  }
};
template <>
struct Pair<float> {  // never instantiated for arithmetic; keeps the packed branch well-formed
  using type = float2;
};

// Final phases shared by both prologues. v holds this thread's fp32 logits as packed pairs.
// FASTEXP (16-bit outputs) uses the compensated pair exponential (exp_pair_compensated, the
// accuracy class of expf); fp32 outputs use expf itself.
template <typename Tout, int CH, int V, int G, bool FASTEXP, bool EXACT = false>
__device__ __forceinline__ void softmax_finish(f32x2 (&v)[CH][V / 2], float mx, float mx_raw, Tout* y, int nv,
                                               int lane, int gs, bool log_mode, bool valid, float* red) {
  const f32x2 mx2 = splat2(mx);
  f32x2 s2 = splat2(0.f);
  auto exp_pair = [](f32x2 d) {
    if constexpr (FASTEXP) {
#ifdef B200_SOFTMAX_FAST_EXP
      return exp_pair_fast(d);
#else
      return exp_pair_compensated(d);
#endif
    } else {
      float a, b;
      unpack2(d, a, b);
      return pack2(expf(a), expf(b));
    }
  };
  if (log_mode) {  // keep x - max (it may be -inf); the exponentials only feed the sum
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      if (EXACT || c * gs < nv) {  // group-uniform: skip slots no lane uses
#pragma unroll
        for (int i = 0; i < V / 2; ++i) {
          v[c][i] = sub2(v[c][i], mx2);
#ifndef B200_SOFTMAX_FAST_EXP
          if constexpr (FASTEXP) {
            float a, b;
            unpack2(v[c][i], a, b);
            a = a < -1e38f ? -1e38f : a;  // finite argument for the compensated exponential, NaN kept
            b = b < -1e38f ? -1e38f : b;
            s2 = add2(s2, exp_pair(pack2(a, b)));
          } else {
            s2 = add2(s2, exp_pair(v[c][i]));
          }
#else
          s2 = add2(s2, exp_pair(v[c][i]));
#endif
        }
      }
    }
  } else {
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      if (EXACT || c * gs < nv) {
#pragma unroll
        for (int i = 0; i < V / 2; ++i) {
          v[c][i] = exp_pair(sub2(v[c][i], mx2));
          s2 = add2(s2, v[c][i]);
        }
      }
    }
  }
  float sa, sb;
  unpack2(s2, sa, sb);
  float s = greduce<SumOp, G>(sa + sb, red);
  if (mx_raw == -INFINITY) s = NAN;  // every logit -inf: aten's x - max is NaN for the whole row

  f32x2 k2;  // second operand of the last step
  if (log_mode) {
    k2 = splat2(logf(s));
  } else {
    k2 = splat2(__frcp_rn(s));
  }
  if (!valid) return;
  Tout* yl = y + (long long)lane * V;  // slot c of this lane starts c * gs vectors further on
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    if (EXACT || c * gs + lane < nv) {
      f32x2 o[V / 2];
#pragma unroll
      for (int i = 0; i < V / 2; ++i) {
        if (log_mode) {
          o[i] = sub2(v[c][i], k2);
        } else if constexpr (sizeof(Tout) == 4) {
          float a, b;
          unpack2(v[c][i], a, b);
          o[i] = pack2(a / s, b / s);
        } else {
          o[i] = mul2(v[c][i], k2);
        }
      }
      store_pairs<Tout, V>(yl + (long long)c * gs * V, o);
    }
  }
}

template <typename Tin, typename Tout, int CH, int G, bool PACKED, bool EXACT = false>
__global__ void __launch_bounds__(G == 0 ? 512 : 256)
softmax_resident_kernel(const SoftmaxParams p) {
  constexpr int V = Elem<Tin>::V;
  constexpr bool FASTEXP = sizeof(Tout) == 2;
  __shared__ float red[32];
  const int lane = glane<G>();
  const int gs = gsize<G>();
  long long row = grow<G>();
  const bool valid = row < p.rows;  // lanes of a partly filled last CTA compute on the last row
  if (!valid) row = p.rows - 1;

  const Tin* x = reinterpret_cast<const Tin*>(p.x) + row_offset(p.xmap, row);
  const Tin* m = p.mask ? reinterpret_cast<const Tin*>(p.mask) + row_offset(p.mmap, row) : nullptr;
  Tout* y = reinterpret_cast<Tout*>(p.y) + row_offset(p.ymap, row);
  const int nv = p.n / V;

  // slot c of this lane starts c * gs vectors after the lane's first one: one pointer per tensor,
  // constant offsets per slot (gs is a compile-time constant for sub-warp and warp groups)
  const Tin* xl = x + (long long)lane * V;
  const Tin* ml = m ? m + (long long)lane * V : nullptr;
  uint4 raw[CH];
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    if (EXACT || c * gs + lane < nv) raw[c] = ld_stream(xl + (long long)c * gs * V);
  }

  f32x2 v[CH][V / 2];
  float mx = -INFINITY;

  // The compensated pair exponential needs finite arguments (inf - inf inside its compensation step would
  // give NaN where exp(-inf) is 0): logits are clamped to a finite floor AFTER the row maximum was
  // taken from the unclamped values. A row whose maximum is -inf (fully masked with -inf) makes
  // aten return NaN for the whole row; the same happens here through the sum (see below).
  constexpr float kFloor = sizeof(Tin) == 2 && !std::is_same<Tin, __nv_bfloat16>::value ? -60000.f : -1e38f;
  // log_softmax returns x - max - log(sum) itself, which may legitimately be -inf: there only the
  // exponential's argument is clamped (in softmax_finish), not the stored value.
#ifdef B200_SOFTMAX_FAST_EXP
  const bool clamp_now = false;  // 2^(-inf) is 0 in the plain exponential: nothing to protect
#else
  const bool clamp_now = FASTEXP && !p.log_mode;
#endif
  if constexpr (PACKED && sizeof(Tin) == 2) {
    using P2 = typename Pair<Tin>::type;
    const P2 neg_inf = Pair<Tin>::splat(-INFINITY);
    const P2 floor2 = Pair<Tin>::splat(kFloor);
    P2 mx2 = neg_inf;
    // One copy of the slot loop per combination of the (warp-uniform) prologue switches, so that
    // they are tested once per row and not once per 16-byte slot.
    //   SK: 0 no scale, 1 packed multiply (scale representable in Tin), 2 fp32 multiply + rounding
    auto prologue = [&](auto sk_tag, auto hm_tag, auto clamp_tag) {
      constexpr int SK = decltype(sk_tag)::value;
      constexpr bool HM = decltype(hm_tag)::value;
      constexpr bool CLAMP = decltype(clamp_tag)::value;
      const P2 s2 = Pair<Tin>::splat(p.scale);
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        P2 t[4];
        if (EXACT || c * gs + lane < nv) {
          const uint32_t w[4] = {raw[c].x, raw[c].y, raw[c].z, raw[c].w};
#pragma unroll
          for (int i = 0; i < 4; ++i) t[i] = *reinterpret_cast<const P2*>(&w[i]);
          if constexpr (SK == 1) {
#pragma unroll
            for (int i = 0; i < 4; ++i) t[i] = __hmul2(t[i], s2);
          } else if constexpr (SK == 2) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 f = Pair<Tin>::widen(t[i]);
              t[i] = Pair<Tin>::narrow(f.x * p.scale, f.y * p.scale);
            }
          }
          if constexpr (HM) {
            const uint4 mr = ld_keep(ml + (long long)c * gs * V);
            const uint32_t mw[4] = {mr.x, mr.y, mr.z, mr.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) t[i] = __hadd2(t[i], *reinterpret_cast<const P2*>(&mw[i]));
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) mx2 = __hmax2(mx2, t[i]);
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) t[i] = neg_inf;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const P2 u = CLAMP ? __hmax2_nan(t[i], floor2) : t[i];  // NaN stays NaN
          v[c][i] = Pairs<Tin>::word(*reinterpret_cast<const uint32_t*>(&u));
        }
      }
    };
    using I0 = std::integral_constant<int, 0>;
    using I1 = std::integral_constant<int, 1>;
    using I2 = std::integral_constant<int, 2>;
    auto with_mask_and_clamp = [&](auto sk_tag) {
      if (m != nullptr) {
        if (clamp_now) prologue(sk_tag, std::true_type{}, std::true_type{});
        else prologue(sk_tag, std::true_type{}, std::false_type{});
      } else {
        if (clamp_now) prologue(sk_tag, std::false_type{}, std::true_type{});
        else prologue(sk_tag, std::false_type{}, std::false_type{});
      }
    };
    if (!p.has_scale) with_mask_and_clamp(I0{});
    else if (p.scale_exact16) with_mask_and_clamp(I1{});
    else with_mask_and_clamp(I2{});
    const float2 mf = Pair<Tin>::widen(mx2);
    mx = greduce<FastMax, G>(fmaxf(mf.x, mf.y), red);
  } else {
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      float f[V];
      if (EXACT || c * gs + lane < nv) {
        Elem<Tin>::unpack(raw[c], f);
        if (p.has_scale) {
#pragma unroll
          for (int i = 0; i < V; ++i) f[i] = f[i] * p.scale;
        }
        if (m != nullptr) {
          float mf[V];
          Elem<Tin>::unpack(ld_keep(ml + (long long)c * gs * V), mf);
#pragma unroll
          for (int i = 0; i < V; ++i) f[i] = f[i] + mf[i];
        }
#pragma unroll
        for (int i = 0; i < V; ++i) mx = fmaxf(mx, f[i]);
      } else {
#pragma unroll
        for (int i = 0; i < V; ++i) f[i] = -INFINITY;
      }
      if (clamp_now) {
#pragma unroll
        for (int i = 0; i < V; ++i) f[i] = f[i] < kFloor ? kFloor : f[i];  // a NaN logit stays NaN
      }
#pragma unroll
      for (int i = 0; i < V / 2; ++i) v[c][i] = pack2(f[2 * i], f[2 * i + 1]);
    }
    mx = greduce<FastMax, G>(mx, red);
  }

  // Subtract the maximum of the CLAMPED values (so every difference is <= 0 and finite); the
  // unclamped maximum still decides whether the whole row was -inf.
  const float mx_raw = mx;
  if (clamp_now) mx = fmaxf(mx, kFloor);
  softmax_finish<Tout, CH, V, G, FASTEXP, EXACT>(v, mx, mx_raw, y, nv, lane, gs, p.log_mode != 0, valid, red);
}

// Element-wise kernel for rows that do not fit in registers or break the vector-path alignment
// rules: one CTA per row and three sweeps (max, sum of exp, write). Only the first sweep of a
// row comes from DRAM when the row fits in L2.
template <typename Tin, bool PACKED>
__device__ __forceinline__ float softmax_logit(const SoftmaxParams& p, const Tin* x, const Tin* m,
                                               long long i) {
  float t = Elem<Tin>::to_f32(x[i]);
  if (p.has_scale) {
    t = t * p.scale;
    if (PACKED) t = round_through<Tin>(t);
  }
  if (m != nullptr) {
    t = t + Elem<Tin>::to_f32(m[i]);
    if (PACKED) t = round_through<Tin>(t);
  }
  return t;
}

template <typename Tin, typename Tout, bool PACKED>
__global__ void __launch_bounds__(1024) softmax_streaming_kernel(const SoftmaxParams p) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const Tin* x = reinterpret_cast<const Tin*>(p.x) + row_offset(p.xmap, row);
  const Tin* m = p.mask ? reinterpret_cast<const Tin*>(p.mask) + row_offset(p.mmap, row) : nullptr;
  Tout* y = reinterpret_cast<Tout*>(p.y) + row_offset(p.ymap, row);

  float mx = -INFINITY;
  for (long long i = threadIdx.x; i < p.n; i += blockDim.x)
    mx = fmaxf(mx, softmax_logit<Tin, PACKED>(p, x, m, i));
  mx = block_reduce<FastMax>(mx, red);

  float s = 0.f;
  for (long long i = threadIdx.x; i < p.n; i += blockDim.x)
    s += expf(softmax_logit<Tin, PACKED>(p, x, m, i) - mx);
  s = block_reduce<SumOp>(s, red);

  const float ls = logf(s);
  const float inv = __frcp_rn(s);
  for (long long i = threadIdx.x; i < p.n; i += blockDim.x) {
    const float d = softmax_logit<Tin, PACKED>(p, x, m, i) - mx;
    float o;
    if (p.log_mode) {
      o = d - ls;
    } else if (sizeof(Tout) == 4) {
      o = expf(d) / s;
    } else {
      o = expf(d) * inv;
    }
    y[i] = Elem<Tout>::from_f32(o);
  }
}

// ----------------------------------------------------------------------------------------------
// Long or ragged rows (rows that do not fit the register-resident kernel, or whose length is not a
// whole number of 16-byte vectors): one CTA per row, two sweeps instead of three.
//   sweep 1: every thread keeps a running maximum m and the sum of exp(t - m) of its elements,
//            rescaling the sum when the maximum grows; the CTA then combines the (m, s) pairs:
//            M = max m_i, S = sum s_i * exp(m_i - M)
//   sweep 2: the row is read again - it was just read by this CTA, so for rows up to a few hundred
//            KB it comes from L2 - and y = exp(t - M) / S (or t - M - log S) is written.
// Both sweeps use 16-byte loads when the row starts on a 16-byte boundary (the ragged tail is read
// element by element) and 16-byte stores when the output row does. No mask; the optional scale is
// applied in fp32.
// ----------------------------------------------------------------------------------------------
template <typename Tout>
__device__ __forceinline__ f32x2 long_row_exp(f32x2 d) {
  if constexpr (sizeof(Tout) == 2) {
    return exp_pair_compensated(d);
  } else {
    float a, b;
    unpack2(d, a, b);
    return pack2(expf(a), expf(b));
  }
}

template <typename Tin, typename Tout>
__global__ void __launch_bounds__(1024) softmax_long_kernel(const SoftmaxParams p) {
  constexpr int V = Elem<Tin>::V;
  constexpr int P = V / 2;
  constexpr int U = 4;  // vectors in flight per thread
  constexpr float kFloor = -1e30f;  // finite stand-in for -inf inside the compensated exponential
  __shared__ float red[64];
  const long long row = blockIdx.x;
  const Tin* x = reinterpret_cast<const Tin*>(p.x) + row_offset(p.xmap, row);
  Tout* y = reinterpret_cast<Tout*>(p.y) + row_offset(p.ymap, row);
  const int tid = threadIdx.x, T_ = blockDim.x;
  const bool x_vec = (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
  const int nvec = x_vec ? p.n / V : 0;
  const int body = nvec * V;  // elements covered by whole vectors
  const f32x2 scale2 = splat2(p.has_scale ? p.scale : 1.0f);
  const bool scaled = p.has_scale != 0;

  // ---- sweep 1 ----------------------------------------------------------------------------------
  float m = -INFINITY, s = 0.f;
  auto absorb = [&](const f32x2 (&t)[P]) {  // one vector of logits into (m, s)
    float vm = -INFINITY;
#pragma unroll
    for (int i = 0; i < P; ++i) {
      float a, b;
      unpack2(t[i], a, b);
      vm = fmaxf(vm, fmaxf(a, b));
    }
    if (vm > m) {
      s = s * expf(fmaxf(m, kFloor) - vm);  // m = -inf the first time: the sum is still zero
      m = vm;
    }
    const f32x2 m2 = splat2(fmaxf(m, kFloor));
    f32x2 acc = splat2(0.f);
#pragma unroll
    for (int i = 0; i < P; ++i) {
      float a, b;
      unpack2(t[i], a, b);
      a = fmaxf(a, kFloor);  // NaN would be lost here, so NaN rows are caught through the maximum below
      b = fmaxf(b, kFloor);
      acc = add2(acc, long_row_exp<Tout>(sub2(pack2(a, b), m2)));
    }
    s += hsum2(acc);
  };
  bool saw_nan = false;
  for (int j0 = tid; j0 < nvec; j0 += U * T_) {
    uint4 raw[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int j = j0 + u * T_;
      if (j < nvec) raw[u] = ld_keep(x + (long long)j * V);  // read again in sweep 2: keep it cached
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int j = j0 + u * T_;
      if (j < nvec) {
        f32x2 t[P];
        Pairs<Tin>::unpack(raw[u], t);
        if (scaled) {
#pragma unroll
          for (int i = 0; i < P; ++i) t[i] = mul2(t[i], scale2);
        }
#pragma unroll
        for (int i = 0; i < P; ++i) {
          float a, b;
          unpack2(t[i], a, b);
          saw_nan |= (a != a) | (b != b);
        }
        absorb(t);
      }
    }
  }
  for (int i = body + tid; i < p.n; i += T_) {  // ragged tail, or the whole row when it is unaligned
    float t = Elem<Tin>::to_f32(x[i]);
    if (scaled) t = t * p.scale;
    saw_nan |= t != t;
    if (t > m) {
      s = s * expf(fmaxf(m, kFloor) - t);
      m = t;
    }
    s += expf(fmaxf(t, kFloor) - fmaxf(m, kFloor));
  }
  // CTA-wide (M, S)
  const float M = block_reduce<FastMax>(m, red);
  const float contrib = (m == -INFINITY) ? 0.f : s * expf(m - fmaxf(M, kFloor));
  float S = block_reduce<SumOp>(contrib, red);
  const float nan_any = block_reduce<FastMax>(saw_nan ? 1.f : 0.f, red);
  if (M == -INFINITY || nan_any > 0.f) S = NAN;  // aten: x - max is NaN for a row of -inf; NaN logits poison the row

  // ---- sweep 2 ----------------------------------------------------------------------------------
  const float logS = logf(S);
  const float inv = __frcp_rn(S);
  const float Mf = fmaxf(M, kFloor);
  const bool log_mode = p.log_mode != 0;
  auto finish = [&](float t) -> float {  // one logit -> one output value
    if (log_mode) return (t - M) - logS;
    const float e = expf(fmaxf(t, kFloor) - Mf);
    return sizeof(Tout) == 4 ? e / S : e * inv;
  };
  constexpr int VO = 16 / (int)sizeof(Tout);           // output elements per 16-byte store
  const bool y_vec = x_vec && (reinterpret_cast<uintptr_t>(y) & 15u) == 0 && V % VO == 0;
  const f32x2 M2 = splat2(Mf), inv2 = splat2(inv), logS2 = splat2(logS), Mraw2 = splat2(M);
  if (!y_vec) {
    // The output row does not start on a 16-byte boundary where the input row does (a ragged row
    // length, another element size): vectors are formed on the OUTPUT side - up to the first
    // boundary element by element, then 16-byte stores whose inputs are read element by element
    // (they were read a moment ago and come from L1 / L2), then the rest.
    int ho = (int)(((16u - (unsigned)(reinterpret_cast<uintptr_t>(y) & 15u)) & 15u) / sizeof(Tout));
    if (ho > p.n) ho = p.n;
    const int nout = (p.n - ho) / VO;
    for (int i = tid; i < ho; i += T_) {
      float t = Elem<Tin>::to_f32(x[i]);
      if (scaled) t = t * p.scale;
      y[i] = Elem<Tout>::from_f32(finish(t));
    }
    for (int j = tid; j < nout; j += T_) {
      const int i0 = ho + j * VO;
      float o[VO];
#pragma unroll
      for (int k = 0; k < VO; ++k) o[k] = Elem<Tin>::to_f32(x[i0 + k]);
#pragma unroll
      for (int k = 0; k < VO; ++k) {
        if (scaled) o[k] = o[k] * p.scale;
        o[k] = finish(o[k]);
      }
      store_converted<Tout, VO>(y + i0, o);
    }
    for (int i = ho + nout * VO + tid; i < p.n; i += T_) {
      float t = Elem<Tin>::to_f32(x[i]);
      if (scaled) t = t * p.scale;
      y[i] = Elem<Tout>::from_f32(finish(t));
    }
    return;
  }
  for (int j0 = tid; j0 < nvec; j0 += U * T_) {
    uint4 raw[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int j = j0 + u * T_;
      if (j < nvec) raw[u] = ld_stream(x + (long long)j * V);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int j = j0 + u * T_;
      if (j < nvec) {
        f32x2 t[P], o[P];
        Pairs<Tin>::unpack(raw[u], t);
#pragma unroll
        for (int i = 0; i < P; ++i) {
          if (scaled) t[i] = mul2(t[i], scale2);
          if (log_mode) {
            o[i] = sub2(sub2(t[i], Mraw2), logS2);
          } else {
            float a, b;
            unpack2(t[i], a, b);
            const f32x2 e = long_row_exp<Tout>(sub2(pack2(fmaxf(a, kFloor), fmaxf(b, kFloor)), M2));
            if constexpr (sizeof(Tout) == 4) {
              float ea, eb;
              unpack2(e, ea, eb);
              o[i] = pack2(ea / S, eb / S);
            } else {
              o[i] = mul2(e, inv2);
            }
          }
        }
        store_pairs<Tout, V>(y + (long long)j * V, o);
      }
    }
  }
  for (int i = body + tid; i < p.n; i += T_) {
    float t = Elem<Tin>::to_f32(x[i]);
    if (scaled) t = t * p.scale;
    y[i] = Elem<Tout>::from_f32(finish(t));
  }
}

template <typename Tin, typename Tout, bool PACKED>
static int launch_softmax(const SoftmaxParams& p, bool vector_ok, cudaStream_t st) {
  constexpr int V = Elem<Tin>::V;
  RowGeometry g;
  if (p.rows > 0x7fffffffLL) return fail(B200_ERR_UNSUPPORTED, "softmax: too many rows");
  if (vector_ok && p.n % V == 0 && pick_row_geometry(p.n / V, &g)) {
    set_path_tag(g.block ? "vector, row resident, CTA per row" : "vector, row resident, sub-warp rows");
    if (!g.block) {
      const int rows_per_cta = g.threads / g.g;
      const unsigned grid = (unsigned)((p.rows + rows_per_cta - 1) / rows_per_cta);
#define B200_SM_LAUNCH(GG, CC)                                                                   \
  do {                                                                                          \
    if (GG > 0 && p.n / V == (long long)GG * CC)                                                \
      softmax_resident_kernel<Tin, Tout, CC, GG, PACKED, (GG > 0)><<<grid, g.threads, 0, st>>>(p); \
    else                                                                                        \
      softmax_resident_kernel<Tin, Tout, CC, GG, PACKED, false><<<grid, g.threads, 0, st>>>(p);   \
  } while (0)
      if (g.g == 8) {
        if (g.ch == 1) B200_SM_LAUNCH(8, 1);
        else if (g.ch == 2) B200_SM_LAUNCH(8, 2);
        else B200_SM_LAUNCH(8, 4);
      } else if (g.g == 16) {
        B200_SM_LAUNCH(16, 4);
      } else {
        B200_SM_LAUNCH(32, 4);
      }
    } else {
      const unsigned grid = (unsigned)p.rows;
      if (g.ch == 2) B200_SM_LAUNCH(0, 2);
      else if (g.ch == 4) B200_SM_LAUNCH(0, 4);
      else B200_SM_LAUNCH(0, 8);
#undef B200_SM_LAUNCH
    }
  } else if (p.mask == nullptr && !PACKED && p.n >= 256) {
    int threads = (int)((p.n / V + 3) / 4);
    threads = (threads + 31) / 32 * 32;
    threads = threads < 128 ? 128 : (threads > 1024 ? 1024 : threads);
    set_path_tag("two sweeps, CTA per row");
    softmax_long_kernel<Tin, Tout><<<(unsigned)p.rows, threads, 0, st>>>(p);
  } else {
    int threads = 1024;
    while (threads > 64 && threads / 2 >= p.n) threads /= 2;
    set_path_tag("element-wise, three passes");
    softmax_streaming_kernel<Tin, Tout, PACKED><<<(unsigned)p.rows, threads, 0, st>>>(p);
  }
  return launch_status("b200_softmax");
}

template <typename Tin, typename Tout>
static int launch_softmax_pro(const SoftmaxParams& p, bool packed, bool vector_ok, cudaStream_t st) {
  if constexpr (sizeof(Tin) == 2) {
    if (packed) return launch_softmax<Tin, Tout, true>(p, vector_ok, st);
  }
  return launch_softmax<Tin, Tout, false>(p, vector_ok, st);
}

}  // namespace b200

using namespace b200;

static bool map_vector_ok(const RowMap& m, int elem_bytes, int chunk) {
  // every row start stays `chunk`-byte aligned when all outer strides are multiples of it
  return (m.s0 * elem_bytes) % chunk == 0 && (m.s1 * elem_bytes) % chunk == 0 &&
         (m.s2 * elem_bytes) % chunk == 0;
}

static bool survives_round_trip(float v, int dtype) {
  if (dtype == B200_F16) return __half2float(__float2half_rn(v)) == v;
  if (dtype == B200_BF16) return __bfloat162float(__float2bfloat16_rn(v)) == v;
  return true;
}

extern "C" int b200_softmax(const void* x, const void* mask, void* y, int64_t rows, int64_t n,
                            int64_t d1, int64_t d2, const int64_t* x_strides,
                            const int64_t* mask_strides, const int64_t* y_strides, int32_t in_dtype,
                            int32_t out_dtype, double scale, int32_t flags, void* stream) {
  if (!x || !y || !x_strides || !y_strides) return fail(B200_ERR_INVALID, "b200_softmax: null argument");
  if (rows < 0 || n < 0 || d1 < 1 || d2 < 1 || n > 0x7fffffffLL)
    return fail(B200_ERR_INVALID, "b200_softmax: bad sizes rows=%lld n=%lld", (long long)rows, (long long)n);
  if (mask && !mask_strides) return fail(B200_ERR_INVALID, "b200_softmax: mask without strides");
  if (rows == 0 || n == 0) return B200_OK;
  if (rows % (d1 * d2) != 0) return fail(B200_ERR_INVALID, "b200_softmax: rows not divisible by d1*d2");

  SoftmaxParams p;
  p.x = x; p.mask = mask; p.y = y; p.rows = rows; p.n = (int)n;
  if (rows > 0x7fffffffLL) return fail(B200_ERR_UNSUPPORTED, "b200_softmax: more than 2^31-1 rows");
  p.xmap = make_row_map(x_strides, d1, d2);
  p.ymap = make_row_map(y_strides, d1, d2);
  p.mmap = mask ? make_row_map(mask_strides, d1, d2) : make_row_map_flat(0);
  p.scale = (float)scale;
  p.has_scale = (flags & B200_SOFTMAX_SCALE) ? 1 : 0;
  p.scale_exact16 = survives_round_trip(p.scale, in_dtype) ? 1 : 0;
  p.log_mode = (flags & B200_SOFTMAX_LOG) ? 1 : 0;
  const bool packed = (flags & B200_SOFTMAX_ROUND) != 0 && in_dtype != B200_F32 &&
                      (p.has_scale || mask != nullptr);

  const int ib = dtype_size(in_dtype), ob = dtype_size(out_dtype);
  const int v_in = 16 / ib;
  const int out_chunk = v_in * ob < 16 ? v_in * ob : 16;
  bool vec = aligned16(x) && map_vector_ok(p.xmap, ib, 16) &&
             (reinterpret_cast<uintptr_t>(y) % out_chunk == 0) && map_vector_ok(p.ymap, ob, out_chunk);
  if (mask) vec = vec && aligned16(mask) && map_vector_ok(p.mmap, ib, 16);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);

#define B200_SOFTMAX_CASE(TI, TO, DI, DO) \
  if (in_dtype == DI && out_dtype == DO) return launch_softmax_pro<TI, TO>(p, packed, vec, st);
  B200_SOFTMAX_CASE(float, float, B200_F32, B200_F32)
  B200_SOFTMAX_CASE(__nv_bfloat16, __nv_bfloat16, B200_BF16, B200_BF16)
  B200_SOFTMAX_CASE(__half, __half, B200_F16, B200_F16)
  B200_SOFTMAX_CASE(__nv_bfloat16, float, B200_BF16, B200_F32)
  B200_SOFTMAX_CASE(__half, float, B200_F16, B200_F32)
  B200_SOFTMAX_CASE(float, __nv_bfloat16, B200_F32, B200_BF16)
  B200_SOFTMAX_CASE(float, __half, B200_F32, B200_F16)
#undef B200_SOFTMAX_CASE
  return fail(B200_ERR_UNSUPPORTED, "b200_softmax: dtype pair (%d -> %d) not built", in_dtype, out_dtype);
}
