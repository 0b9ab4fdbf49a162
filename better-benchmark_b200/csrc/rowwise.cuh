// Helpers shared by the row-wise families (row reductions, softmax, LayerNorm/RMSNorm forward).
//
// Work decomposition: a "group" of threads owns one row. The group is one warp (short rows,
// several rows per CTA, no block barrier) or the whole CTA (long rows). A row of n elements is
// nv = n / V sixteen-byte vectors; vector j belongs to group lane j % G and register slot j / G,
// so each slot is one fully coalesced G x 16-byte access and all of a thread's loads are issued
// before the first is consumed.
#pragma once

#include "common.cuh"

#include <cstdlib>

namespace b200 {

// Division by a run-time constant without a divide instruction: q = umulhi(n, mul) >> shr for
// 0 <= n < 2^31 (host side picks mul/shr for the divisor d >= 1).
struct FastDiv {
  unsigned int mul, shr, d;
};

inline FastDiv make_fast_div(long long d) {
  FastDiv f;
  f.d = (unsigned int)d;
  if (d <= 1) {
    f.mul = 0;
    f.shr = 0;
    return f;
  }
  unsigned int lg = 0;
  while ((1ull << lg) < (unsigned long long)d) ++lg;  // ceil(log2 d)
  const unsigned int p = 31 + lg;
  f.mul = (unsigned int)(((1ull << p) + (unsigned long long)d - 1) / (unsigned long long)d);
  f.shr = p - 32;
  return f;
}

__device__ __forceinline__ unsigned int fast_div(unsigned int n, const FastDiv& f) {
  return f.d == 1 ? n : (__umulhi(n, f.mul) >> f.shr);
}

// Maps a flat row index onto up to three outer dimensions with arbitrary element strides, so
// broadcast operands (stride 0) and non-contiguous views need no copy. row = (i0*d1 + i1)*d2 + i2.
// Rows are limited to 2^31 - 1 (checked by the host).
struct RowMap {
  long long s0, s1, s2;
  FastDiv d1, d2;
};

inline RowMap make_row_map(const int64_t* strides, long long d1, long long d2) {
  RowMap m;
  m.s0 = strides[0];
  m.s1 = strides[1];
  m.s2 = strides[2];
  m.d1 = make_fast_div(d1);
  m.d2 = make_fast_div(d2);
  return m;
}

inline RowMap make_row_map_flat(long long row_stride) {
  RowMap m;
  m.s0 = row_stride;
  m.s1 = m.s2 = 0;
  m.d1 = make_fast_div(1);
  m.d2 = make_fast_div(1);
  return m;
}

__device__ __forceinline__ long long row_offset(const RowMap& m, long long row) {
  if (m.d1.d == 1 && m.d2.d == 1) return row * m.s0;
  const unsigned int r = (unsigned int)row;
  const unsigned int t = fast_div(r, m.d2);
  const unsigned int i2 = r - t * m.d2.d;
  const unsigned int i0 = fast_div(t, m.d1);
  const unsigned int i1 = t - i0 * m.d1.d;
  return (long long)i0 * m.s0 + (long long)i1 * m.s1 + (long long)i2 * m.s2;
}

// ----------------------------------------------------------------------------------------------
// Packed fp32 pairs. sm_100 executes add/sub/mul/fma on two fp32 values held in one 64-bit
// register pair as ONE instruction (same per-lane arithmetic throughput, half the issue slots),
// with round-to-nearest on each half: numerically identical to the two scalar operations.
// ----------------------------------------------------------------------------------------------
typedef unsigned long long f32x2;

__device__ __forceinline__ f32x2 pack2(float a, float b) {
  f32x2 r;
  asm("mov.b64 %0, {%1,%2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& a, float& b) {
  asm("mov.b64 {%0,%1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ f32x2 splat2(float a) { return pack2(a, a); }
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ f32x2 sub2(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
// a*b+c with a single rounding per half: only where the evaluated graph has no separate
// multiply and add to mirror (polynomial/compensation steps, sums of squares for statistics).
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}

// 16-byte vector <-> packed fp32 pairs, converted word by word so that each pair is born in (and
// consumed from) an aligned register pair instead of being assembled from two scalars.
template <typename T>
struct Pairs;

template <>
struct Pairs<float> {
  static __device__ __forceinline__ void unpack(const uint4& r, f32x2 (&v)[2]) {
    asm("mov.b64 %0, {%1,%2};" : "=l"(v[0]) : "r"(r.x), "r"(r.y));
    asm("mov.b64 %0, {%1,%2};" : "=l"(v[1]) : "r"(r.z), "r"(r.w));
  }
  static __device__ __forceinline__ uint4 pack(const f32x2 (&v)[2]) {
    uint4 r;
    asm("mov.b64 {%0,%1}, %2;" : "=r"(r.x), "=r"(r.y) : "l"(v[0]));
    asm("mov.b64 {%0,%1}, %2;" : "=r"(r.z), "=r"(r.w) : "l"(v[1]));
    return r;
  }
};

template <>
struct Pairs<__nv_bfloat16> {
  static __device__ __forceinline__ f32x2 word(uint32_t w) {
    f32x2 r;  // bf16 -> fp32: the low element is a 16-bit shift, the high one a mask
    asm("{\n\t.reg .b32 lo, hi;\n\tshl.b32 lo, %1, 16;\n\tand.b32 hi, %1, 0xffff0000;\n\tmov.b64 %0, {lo,hi};\n\t}"
        : "=l"(r) : "r"(w));
    return r;
  }
  static __device__ __forceinline__ void unpack(const uint4& r, f32x2 (&v)[4]) {
    v[0] = word(r.x); v[1] = word(r.y); v[2] = word(r.z); v[3] = word(r.w);
  }
  static __device__ __forceinline__ uint32_t narrow(f32x2 v) {
    uint32_t r;
    asm("{\n\t.reg .b32 lo, hi;\n\tmov.b64 {lo,hi}, %1;\n\tcvt.rn.bf16x2.f32 %0, hi, lo;\n\t}" : "=r"(r) : "l"(v));
    return r;
  }
  static __device__ __forceinline__ uint4 pack(const f32x2 (&v)[4]) {
    return make_uint4(narrow(v[0]), narrow(v[1]), narrow(v[2]), narrow(v[3]));
  }
};

template <>
struct Pairs<__half> {
  static __device__ __forceinline__ f32x2 word(uint32_t w) {
    f32x2 r;
    asm("{\n\t.reg .b16 a, b;\n\t.reg .b32 lo, hi;\n\tmov.b32 {a,b}, %1;\n\tcvt.f32.f16 lo, a;\n\tcvt.f32.f16 hi, b;\n\t"
        "mov.b64 %0, {lo,hi};\n\t}"
        : "=l"(r) : "r"(w));
    return r;
  }
  static __device__ __forceinline__ void unpack(const uint4& r, f32x2 (&v)[4]) {
    v[0] = word(r.x); v[1] = word(r.y); v[2] = word(r.z); v[3] = word(r.w);
  }
  static __device__ __forceinline__ uint32_t narrow(f32x2 v) {
    uint32_t r;
    asm("{\n\t.reg .b32 lo, hi;\n\tmov.b64 {lo,hi}, %1;\n\tcvt.rn.f16x2.f32 %0, hi, lo;\n\t}" : "=r"(r) : "l"(v));
    return r;
  }
  static __device__ __forceinline__ uint4 pack(const f32x2 (&v)[4]) {
    return make_uint4(narrow(v[0]), narrow(v[1]), narrow(v[2]), narrow(v[3]));
  }
};

// Sum of the two halves of a pair.
__device__ __forceinline__ float hsum2(f32x2 v) {
  float a, b;
  unpack2(v, a, b);
  return a + b;
}

// Natural exponential of a pair for results that are rounded to a 16-bit type afterwards.
//
// exp_pair_compensated (the default): y = x * log2(e) is rounded to fp32 (yh); what that rounding
// and the rounding of the constant lost is recovered exactly as r = x - yh * ln 2 with one fused
// multiply-add (the product is exact inside the fma; r is the error of the exponent in natural
// units, |r| < 2^-20), 2^yh comes from the hardware approximation (relative error 2^-22) and the
// result is 2^yh * (1 + r). Relative error below 3.5e-7 for arguments down to -17 (below 6e-7 over
// the whole range): the accuracy class of expf (2 ulp), three orders of magnitude below half a
// bf16/fp16 ulp. The argument must be finite (inf - inf inside the fma would give NaN where
// exp(-inf) is 0): callers clamp to a finite floor first; NaN stays NaN.
// .ftz: results below 2^-126 become 0 instead of denormals; nothing a 16-bit output or the row sum
// can see.
__device__ __forceinline__ f32x2 exp_pair_compensated(f32x2 x) {
  const f32x2 yh = mul2(x, splat2(1.4426950216293335f));   // x * fl(log2 e), rounded
  const f32x2 r = fma2(yh, splat2(-0.6931471824645996f), x);  // x - yh * ln 2
  f32x2 p;
  asm("{\n\t.reg .f32 a, b, pa, pb;\n\tmov.b64 {a,b}, %1;\n\tex2.approx.ftz.f32 pa, a;\n\t"
      "ex2.approx.ftz.f32 pb, b;\n\tmov.b64 %0, {pa,pb};\n\t}"
      : "=l"(p) : "l"(yh));
  return fma2(p, r, p);
}

// exp_pair_fast (opt-in, -DB200_SOFTMAX_FAST_EXP): 2^(x * log2 e) with the hardware approximation
// alone, which is what Triton's tl.exp lowers to. Relative error <= 2^-22 + |x * log2 e| * 2^-24 * ln 2:
// below 1.3e-6 wherever an fp16 result is not zero (x > -17) and below 6e-6 over the whole bf16
// range. Not the natural-exponential accuracy the eager graphs have; kept for measurements.
__device__ __forceinline__ f32x2 exp_pair_fast(f32x2 x) {
  const f32x2 y = mul2(x, splat2(1.4426950216293335f));
  f32x2 r;
  asm("{\n\t.reg .f32 a, b, pa, pb;\n\tmov.b64 {a,b}, %1;\n\tex2.approx.ftz.f32 pa, a;\n\t"
      "ex2.approx.ftz.f32 pb, b;\n\tmov.b64 %0, {pa,pb};\n\t}"
      : "=l"(r) : "l"(y));
  return r;
}

template <bool BLOCK>
__device__ __forceinline__ int group_lane() {
  return BLOCK ? (int)threadIdx.x : (int)(threadIdx.x & 31);
}
template <bool BLOCK>
__device__ __forceinline__ int group_size() {
  return BLOCK ? (int)blockDim.x : 32;
}
template <bool BLOCK>
__device__ __forceinline__ long long group_row() {
  return BLOCK ? (long long)blockIdx.x
               : (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
}

// Store N fp32 values as N elements of Tout with the widest store the byte count allows
// (N * sizeof(Tout) is 8, 16 or 32 and `p` is aligned to min(16, that)).
template <typename Tout, int N>
__device__ __forceinline__ void store_converted(Tout* p, const float (&f)[N]) {
  if constexpr (sizeof(Tout) == 4) {
#pragma unroll
    for (int i = 0; i < N / 4; ++i) {
      uint4 o = make_uint4(__float_as_uint(f[4 * i]), __float_as_uint(f[4 * i + 1]),
                           __float_as_uint(f[4 * i + 2]), __float_as_uint(f[4 * i + 3]));
      st_stream(reinterpret_cast<float*>(p) + 4 * i, o);
    }
  } else if constexpr (N == 8) {
    st_stream(p, Elem<Tout>::pack(f));
  } else {
    static_assert(N == 4, "unexpected vector length");
    uint32_t w[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      if constexpr (sizeof(Tout) == 2) {
        Tout a = Elem<Tout>::from_f32(f[2 * i]);
        Tout b = Elem<Tout>::from_f32(f[2 * i + 1]);
        w[i] = (uint32_t)(*reinterpret_cast<unsigned short*>(&a)) |
               ((uint32_t)(*reinterpret_cast<unsigned short*>(&b)) << 16);
      }
    }
    asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(w[0]), "r"(w[1]) : "memory");
  }
}

// store_converted for values held as packed pairs (N values = N/2 pairs).
template <typename Tout, int N>
__device__ __forceinline__ void store_pairs(Tout* p, const f32x2 (&v)[N / 2]) {
  if constexpr (sizeof(Tout) == 4) {
#pragma unroll
    for (int i = 0; i < N / 4; ++i) {
      const f32x2 two[2] = {v[2 * i], v[2 * i + 1]};
      st_stream(reinterpret_cast<float*>(p) + 4 * i, Pairs<float>::pack(two));
    }
  } else if constexpr (N == 8) {
    st_stream(p, Pairs<Tout>::pack(v));
  } else {
    static_assert(N == 4, "unexpected vector length");
    const uint32_t w0 = Pairs<Tout>::narrow(v[0]), w1 = Pairs<Tout>::narrow(v[1]);
    asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(w0), "r"(w1) : "memory");
  }
}

// Load N consecutive parameter values (weight, bias) whose dtype is only known at run time.
// These operands are tiny and shared by every row, so they come through L1 (ld_keep).
// `p` + idx must be aligned to min(16, N * element size).
template <int N>
__device__ __forceinline__ void load_param(const void* base, int dtype, long long idx,
                                           float (&f)[N]) {
  if (dtype == B200_F32) {
    const float* q = reinterpret_cast<const float*>(base) + idx;
#pragma unroll
    for (int i = 0; i < N / 4; ++i) {
      uint4 r = ld_keep(q + 4 * i);
      f[4 * i] = __uint_as_float(r.x);
      f[4 * i + 1] = __uint_as_float(r.y);
      f[4 * i + 2] = __uint_as_float(r.z);
      f[4 * i + 3] = __uint_as_float(r.w);
    }
  } else {
    const unsigned short* q = reinterpret_cast<const unsigned short*>(base) + idx;
    uint32_t w[N / 2];
    if constexpr (N == 8) {
      uint4 r = ld_keep(q);
      w[0] = r.x; w[1] = r.y; w[2] = r.z; w[3] = r.w;
    } else {
      uint2 r = __ldg(reinterpret_cast<const uint2*>(q));
      w[0] = r.x; w[1] = r.y;
    }
#pragma unroll
    for (int i = 0; i < N / 2; ++i) {
      if (dtype == B200_BF16) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
      } else {
        float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
      }
    }
  }
}

// Scalar parameter load with run-time dtype.
__device__ __forceinline__ float load_param1(const void* base, int dtype, long long idx) {
  if (dtype == B200_F32) return __ldg(reinterpret_cast<const float*>(base) + idx);
  if (dtype == B200_BF16)
    return __bfloat162float(__ldg(reinterpret_cast<const __nv_bfloat16*>(base) + idx));
  return __half2float(__ldg(reinterpret_cast<const __half*>(base) + idx));
}

// Round an fp32 value to T and back: the rounding boundary a 16-bit intermediate tensor imposes.
template <typename T>
__device__ __forceinline__ float round_through(float v) {
  return Elem<T>::to_f32(Elem<T>::from_f32(v));
}

// ----------------------------------------------------------------------------------------------
// Register-resident rows: launch geometry and group helpers.
// A row of nv 16-byte vectors is owned by a group of G threads with CH register slots each
// (G * CH >= nv). Short rows use sub-warp groups of 8, 16 or 32 lanes with up to four slots, so
// that a thread still handles ~32 elements and the per-row bookkeeping (index arithmetic, two
// shuffle reductions, a reciprocal) is amortised; long rows use the whole CTA (G = 0).
//   nv <= 32   : G = 8,  CH = 1, 2 or 4      (256-thread CTA = 32 rows)
//   nv <= 64   : G = 16, CH = 4              (16 rows per CTA)
//   nv <= 128  : G = 32, CH = 4              (8 rows per CTA)
//   nv <= 4096 : G = 0 (CTA per row), CH = 2, 4 or 8, 96..512 threads
// ----------------------------------------------------------------------------------------------
struct RowGeometry {
  int g;        // lanes per row; 0 = the whole CTA
  int ch;       // register slots per thread
  int threads;  // CTA size
  bool block;   // g == 0
};

inline bool pick_row_geometry(long long nv, RowGeometry* g) {
  if (nv <= 0) return false;
  g->threads = 256;
  g->block = false;
  if (nv <= 32) {
    g->g = 8;
    g->ch = nv <= 8 ? 1 : (nv <= 16 ? 2 : 4);
    return true;
  }
  if (nv <= 64) {
    g->g = 16;
    g->ch = 4;
    return true;
  }
  if (nv <= 128) {
    g->g = 32;
    g->ch = 4;
    return true;
  }
  if (nv > 4096) return false;
  g->g = 0;
  g->block = true;
  // CTAs of about 128 threads for mid-size rows (measured on 4096 bf16 columns: 44.7 us with four
  // vectors per thread against 49.2 us with two), eight vectors per thread for the longest
  g->ch = nv <= 256 ? 2 : (nv <= 2048 ? 4 : 8);
  {
    static const int ch_env = [] { const char* e = getenv("B200_BLOCK_CH"); return e ? atoi(e) : 0; }();
    if (ch_env == 2 || ch_env == 4 || ch_env == 8) g->ch = ch_env;
  }
  long long t = (nv + g->ch - 1) / g->ch;
  t = (t + 31) / 32 * 32;
  g->threads = (int)t;
  return true;
}

template <int G>
__device__ __forceinline__ int glane() {
  return G == 0 ? (int)threadIdx.x : (int)(threadIdx.x & (G - 1));
}
template <int G>
__device__ __forceinline__ int gsize() {
  return G == 0 ? (int)blockDim.x : G;
}
template <int G>
__device__ __forceinline__ long long grow() {
  return G == 0 ? (long long)blockIdx.x
                : (long long)blockIdx.x * (blockDim.x / (G == 0 ? 1 : G)) + threadIdx.x / (G == 0 ? 1 : G);
}
// Reduction over the group; every lane of the warp must call it (sub-warp groups reduce side by
// side inside one shuffle).
template <typename Op, int G>
__device__ __forceinline__ float greduce(float v, float* scratch) {
  if constexpr (G == 0) {
    return block_reduce<Op>(v, scratch);
  } else {
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) v = Op::apply(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
  }
}

// Two sums over the group at once: the shuffle chains of the two values interleave, so the pair
// costs about one reduction's latency. `scratch` holds >= 64 floats.
template <int G>
__device__ __forceinline__ void greduce_sum2(float& a, float& b, float* scratch) {
  if constexpr (G == 0) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      a += __shfl_xor_sync(0xffffffffu, a, o);
      b += __shfl_xor_sync(0xffffffffu, b, o);
    }
    if (lane == 0) {
      scratch[warp] = a;
      scratch[32 + warp] = b;
    }
    __syncthreads();
    a = 0.f;
    b = 0.f;
    for (int w = 0; w < nwarps; ++w) {
      a += scratch[w];
      b += scratch[32 + w];
    }
    __syncthreads();
  } else {
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) {
      a += __shfl_xor_sync(0xffffffffu, a, o);
      b += __shfl_xor_sync(0xffffffffu, b, o);
    }
  }
}

}  // namespace b200
