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
// exp/log are the full-precision expf/logf. For 16-bit outputs e / s is evaluated as
// e * (1 / s) with a correctly rounded reciprocal; the extra fp32 rounding is far below half a
// 16-bit ulp. fp32 outputs use the IEEE division.
#include "rowwise.cuh"

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

// Final phases shared by both prologues: v holds the fp32 logits of this thread's slots.
template <typename Tout, int CH, int V, bool BLOCK>
__device__ __forceinline__ void softmax_finish(float (&v)[CH][V], float mx, Tout* y, int nv, int lane,
                                               int G, bool log_mode, float* red) {
  float s = 0.f;
  if (log_mode) {
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      if (c * G < nv) {  // group-uniform: skip slots no lane uses
#pragma unroll
        for (int i = 0; i < V; ++i) {
          v[c][i] = v[c][i] - mx;
          s += expf(v[c][i]);
        }
      }
    }
    s = group_reduce<SumOp, BLOCK>(s, red);
    const float ls = logf(s);
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int j = c * G + lane;
      if (j < nv) {
#pragma unroll
        for (int i = 0; i < V; ++i) v[c][i] = v[c][i] - ls;
        store_converted<Tout, V>(y + (long long)j * V, v[c]);
      }
    }
  } else {
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      if (c * G < nv) {
#pragma unroll
        for (int i = 0; i < V; ++i) {
          v[c][i] = expf(v[c][i] - mx);
          s += v[c][i];
        }
      }
    }
    s = group_reduce<SumOp, BLOCK>(s, red);
    const float inv = __frcp_rn(s);
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int j = c * G + lane;
      if (j < nv) {
#pragma unroll
        for (int i = 0; i < V; ++i) {
          if constexpr (sizeof(Tout) == 4) {
            v[c][i] = v[c][i] / s;
          } else {
            v[c][i] = v[c][i] * inv;
          }
        }
        store_converted<Tout, V>(y + (long long)j * V, v[c]);
      }
    }
  }
}

template <typename Tin, typename Tout, int CH, bool BLOCK, bool PACKED>
__global__ void __launch_bounds__(BLOCK ? 512 : 256)
softmax_resident_kernel(const SoftmaxParams p) {
  constexpr int V = Elem<Tin>::V;
  __shared__ float red[32];
  const int lane = group_lane<BLOCK>();
  const int G = group_size<BLOCK>();
  const long long row = group_row<BLOCK>();
  if (row >= p.rows) return;

  const Tin* x = reinterpret_cast<const Tin*>(p.x) + row_offset(p.xmap, row);
  const Tin* m = p.mask ? reinterpret_cast<const Tin*>(p.mask) + row_offset(p.mmap, row) : nullptr;
  Tout* y = reinterpret_cast<Tout*>(p.y) + row_offset(p.ymap, row);
  const int nv = p.n / V;

  uint4 raw[CH];
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int j = c * G + lane;
    if (j < nv) raw[c] = ld_stream(x + (long long)j * V);
  }

  float v[CH][V];
  float mx = -INFINITY;

  if constexpr (PACKED && sizeof(Tin) == 2) {
    using P2 = typename Pair<Tin>::type;
    const P2 neg_inf = Pair<Tin>::splat(-INFINITY);
    P2 mx2 = neg_inf;
    P2 t[CH][4];
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int j = c * G + lane;
      if (j < nv) {
        const uint32_t w[4] = {raw[c].x, raw[c].y, raw[c].z, raw[c].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) t[c][i] = *reinterpret_cast<const P2*>(&w[i]);
        if (p.has_scale) {
          if (p.scale_exact16) {
            const P2 s2 = Pair<Tin>::splat(p.scale);
#pragma unroll
            for (int i = 0; i < 4; ++i) t[c][i] = __hmul2(t[c][i], s2);
          } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 f = Pair<Tin>::widen(t[c][i]);
              t[c][i] = Pair<Tin>::narrow(f.x * p.scale, f.y * p.scale);
            }
          }
        }
        if (m != nullptr) {
          const uint4 mr = ld_keep(m + (long long)j * V);
          const uint32_t mw[4] = {mr.x, mr.y, mr.z, mr.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) t[c][i] = __hadd2(t[c][i], *reinterpret_cast<const P2*>(&mw[i]));
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) mx2 = __hmax2(mx2, t[c][i]);
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) t[c][i] = neg_inf;
      }
    }
    const float2 mf = Pair<Tin>::widen(mx2);
    mx = group_reduce<FastMax, BLOCK>(fmaxf(mf.x, mf.y), red);
#pragma unroll
    for (int c = 0; c < CH; ++c) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = Pair<Tin>::widen(t[c][i]);
        v[c][2 * i] = f.x;
        v[c][2 * i + 1] = f.y;
      }
    }
  } else {
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int j = c * G + lane;
      if (j < nv) {
        Elem<Tin>::unpack(raw[c], v[c]);
        if (p.has_scale) {
#pragma unroll
          for (int i = 0; i < V; ++i) v[c][i] = v[c][i] * p.scale;
        }
        if (m != nullptr) {
          float mf[V];
          Elem<Tin>::unpack(ld_keep(m + (long long)j * V), mf);
#pragma unroll
          for (int i = 0; i < V; ++i) v[c][i] = v[c][i] + mf[i];
        }
#pragma unroll
        for (int i = 0; i < V; ++i) mx = fmaxf(mx, v[c][i]);
      } else {
#pragma unroll
        for (int i = 0; i < V; ++i) v[c][i] = -INFINITY;
      }
    }
    mx = group_reduce<FastMax, BLOCK>(mx, red);
  }

  softmax_finish<Tout, CH, V, BLOCK>(v, mx, y, nv, lane, G, p.log_mode != 0, red);
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

template <typename Tin, typename Tout, bool PACKED>
static int launch_softmax(const SoftmaxParams& p, bool vector_ok, cudaStream_t st) {
  constexpr int V = Elem<Tin>::V;
  RowGeometry g;
  if (p.rows > 0x7fffffffLL) return fail(B200_ERR_UNSUPPORTED, "softmax: too many rows");
  if (vector_ok && p.n % V == 0 && pick_row_geometry(p.n / V, &g)) {
    if (!g.block) {
      const int rows_per_cta = g.threads / 32;
      const unsigned grid = (unsigned)((p.rows + rows_per_cta - 1) / rows_per_cta);
      switch (g.ch) {
        case 1: softmax_resident_kernel<Tin, Tout, 1, false, PACKED><<<grid, g.threads, 0, st>>>(p); break;
        case 2: softmax_resident_kernel<Tin, Tout, 2, false, PACKED><<<grid, g.threads, 0, st>>>(p); break;
        default: softmax_resident_kernel<Tin, Tout, 4, false, PACKED><<<grid, g.threads, 0, st>>>(p); break;
      }
    } else {
      const unsigned grid = (unsigned)p.rows;
      switch (g.ch) {
        case 2: softmax_resident_kernel<Tin, Tout, 2, true, PACKED><<<grid, g.threads, 0, st>>>(p); break;
        case 4: softmax_resident_kernel<Tin, Tout, 4, true, PACKED><<<grid, g.threads, 0, st>>>(p); break;
        default: softmax_resident_kernel<Tin, Tout, 8, true, PACKED><<<grid, g.threads, 0, st>>>(p); break;
      }
    }
  } else {
    int threads = 1024;
    while (threads > 64 && threads / 2 >= p.n) threads /= 2;
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
  p.xmap = RowMap{x_strides[0], x_strides[1], x_strides[2], (int)d1, (int)d2};
  p.ymap = RowMap{y_strides[0], y_strides[1], y_strides[2], (int)d1, (int)d2};
  p.mmap = mask ? RowMap{mask_strides[0], mask_strides[1], mask_strides[2], (int)d1, (int)d2}
                : RowMap{0, 0, 0, 1, 1};
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
