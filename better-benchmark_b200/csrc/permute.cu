// Layout-changing copies with a pointwise epilogue (optional scale, dtype conversion):
//   * general: up to four dimensions with arbitrary input strides into a contiguous output
//     (head split [B,S,H,D] -> [B,H,S,D], any permute + clone);
//   * transpose of the two innermost dimensions through a padded shared-memory tile, coalesced
//     row accesses on both sides;
//   * contiguous cast / scale (no layout change).
//
// Replaces the permuting pointwise Triton kernels of the reference:
// repros/canonical/pointwise_c0d19d490a2f/oracle.py:10-33 (head-split gather copy),
// pointwise_021e90d9c17d/oracle.py:10-51 (autotuned 2-D tile transpose),
// pointwise_8bb40810003c/oracle.py:11-15 and pointwise_95ed2ef35da9/oracle.py:10-44 (cast / scale).
//
// Pointwise semantics follow aten: the value is converted to fp32, multiplied by the scale (when
// given) and rounded once to the output dtype.
#include "rowwise.cuh"

#include <type_traits>
#include <cstdlib>

namespace b200 {

struct PermuteParams {
  const void* x;
  void* y;
  long long shape[4];      // OUTPUT shape, outermost first (unused leading dims are 1)
  long long in_stride[4];  // input stride of each OUTPUT dimension, in elements
  FastDiv d1, d2, d3;      // fast division by shape[1], shape[2], shape[3] (in units of the inner vector)
  long long total;         // output elements
  float scale;
  int has_scale;
};

// Activation bits of the mode word (after the optional scaling), each the fp32 expression of the
// decomposed aten graph: 2 ReLU (a NaN stays a NaN); 4 exact GELU, (x * 0.5) * (erf(x * 0.7071067811865476) + 1)
// (repros/canonical/pointwise_826ea0b5f6e4/repro.py:27-31); 8 SiLU, x / (exp(-x) + 1)
// (repros/canonical/pointwise_795cdbe23b17/repro.py:26-29).
// One activation per launch; ACT is its bit (0: none), so that each instantiation carries only the
// code it uses.
template <int ACT>
__device__ __forceinline__ float apply_activation(float f) {
  if constexpr (ACT == 2) f = f < 0.f ? 0.f : f;
  if constexpr (ACT == 4) f = (f * 0.5f) * (erff(f * 0.7071067811865476f) + 1.0f);
  if constexpr (ACT == 8) f = f / (expf(-f) + 1.0f);
  return f;
}

template <typename Tin, typename Tout, int ACT = 0>
__device__ __forceinline__ Tout convert_scaled(Tin v, float scale, int has_scale) {
  float f = Elem<Tin>::to_f32(v);
  if (has_scale & 1) f = f * scale;
  f = apply_activation<ACT>(f);
  return Elem<Tout>::from_f32(f);
}

// General kernel. VEC: the innermost output dimension is also unit-stride in the input and both
// sides are 16-byte friendly, so a thread moves VIN = 16 / sizeof(Tin) elements at once.
template <typename Tin, typename Tout, bool VEC>
__global__ void __launch_bounds__(256) permute_general_kernel(const PermuteParams p) {
  constexpr int VIN = VEC ? Elem<Tin>::V : 1;
  constexpr int U = VEC ? 4 : 1;  // independent 16-byte loads in flight per thread
  const long long units = p.total / VIN;
  // input offset of unit u: decompose u over (shape[0], shape[1], shape[2], shape[3] / VIN)
  auto in_offset = [&](long long u) {
    long long i3, i2, i1, i0;
    if (u < 0x7fffffffLL) {
      unsigned int r = (unsigned int)u;
      unsigned int q = fast_div(r, p.d3);
      i3 = r - q * p.d3.d; r = q;
      q = fast_div(r, p.d2);
      i2 = r - q * p.d2.d; r = q;
      q = fast_div(r, p.d1);
      i1 = r - q * p.d1.d;
      i0 = q;
    } else {
      long long rest = u;
      const long long n3 = p.d3.d, n2 = p.d2.d, n1 = p.d1.d;
      i3 = rest % n3; rest /= n3;
      i2 = rest % n2; rest /= n2;
      i1 = rest % n1;
      i0 = rest / n1;
    }
    return i0 * p.in_stride[0] + i1 * p.in_stride[1] + i2 * p.in_stride[2] + i3 * VIN * p.in_stride[3];
  };
  // a CTA takes blocks of U * blockDim consecutive output units (block b, b + grid, ...), so that
  // its U stores (and, for most layouts, loads) in flight per thread fall into one stretch of memory
  const long long stride = blockDim.x;
  const long long block = (long long)U * blockDim.x;
  for (long long u0 = (long long)blockIdx.x * block + threadIdx.x; u0 < units; u0 += (long long)gridDim.x * block) {
    if constexpr (VEC) {
      uint4 raw[U];
#pragma unroll
      for (int k = 0; k < U; ++k) {
        const long long u = u0 + k * stride;
        if (u < units) raw[k] = ld_stream(reinterpret_cast<const Tin*>(p.x) + in_offset(u));
      }
#pragma unroll
      for (int k = 0; k < U; ++k) {
        const long long u = u0 + k * stride;
        if (u < units) {
          Tout* dst = reinterpret_cast<Tout*>(p.y) + u * VIN;
          if (std::is_same<Tin, Tout>::value && !p.has_scale) {
            st_stream(reinterpret_cast<Tin*>(dst), raw[k]);  // plain copy: no conversion at all
          } else {
            float f[VIN];
            Elem<Tin>::unpack(raw[k], f);
            if (p.has_scale) {
#pragma unroll
              for (int i = 0; i < VIN; ++i) f[i] = f[i] * p.scale;
            }
            store_converted<Tout, VIN>(dst, f);
          }
        }
      }
    } else {
      const Tin* src = reinterpret_cast<const Tin*>(p.x) + in_offset(u0);
      reinterpret_cast<Tout*>(p.y)[u0] = convert_scaled<Tin, Tout>(*src, p.scale, p.has_scale);
    }
  }
}

// Transpose of the two innermost dimensions: output [batch, C, P] from input [batch, P, C]
// (input row stride in_row_stride, batch stride in_batch_stride). 64 x 64 element tiles; a warp
// reads and writes whole tile rows (64 consecutive elements), the transposition happens in shared
// memory (row pitch padded by one 4-byte word to spread the column reads over the banks).
struct TransposeParams {
  const void* x;
  void* y;
  long long batch, P, C;
  long long in_batch_stride, in_row_stride;
  float scale;
  int has_scale;
};

template <typename Tin, typename Tout>
__global__ void __launch_bounds__(256) transpose_tile_kernel(const TransposeParams p) {
  constexpr int TILE = 64;
  __shared__ float tile[TILE][TILE + 1];
  const long long b = blockIdx.z;
  const long long p0 = (long long)blockIdx.y * TILE, c0 = (long long)blockIdx.x * TILE;
  const Tin* src = reinterpret_cast<const Tin*>(p.x) + b * p.in_batch_stride;
  Tout* dst = reinterpret_cast<Tout*>(p.y) + b * p.P * p.C;
  // load: thread (ty, tx) walks rows of the input tile, columns contiguous
  for (int r = threadIdx.x / TILE; r < TILE; r += 256 / TILE) {
    const int c = threadIdx.x % TILE;
    const long long pr = p0 + r, pc = c0 + c;
    float v = 0.f;
    if (pr < p.P && pc < p.C) {
      v = Elem<Tin>::to_f32(src[pr * p.in_row_stride + pc]);
      if (p.has_scale) v = v * p.scale;
    }
    tile[r][c] = v;
  }
  __syncthreads();
  // store: rows of the output tile are columns of the input tile
  for (int r = threadIdx.x / TILE; r < TILE; r += 256 / TILE) {
    const int c = threadIdx.x % TILE;
    const long long oc = c0 + r, op = p0 + c;  // output row index = input column
    if (oc < p.C && op < p.P) dst[oc * p.P + op] = Elem<Tout>::from_f32(tile[c][r]);
  }
}

// Transpose of 16-bit elements without conversion, whole 64 x 64 tiles only: 16-byte accesses on
// both sides. The tile lives in shared memory as 64 rows of 32 words (two elements per word), row r
// rotated by 4 * (r / 8) words. A thread then reads, for one pair of input columns and eight
// consecutive input rows, eight words that fall into eight different banks, and splits them into two
// output vectors with byte permutes: eight consecutive elements of output row 2c and of row 2c + 1.
__global__ void __launch_bounds__(256) transpose16_tile_kernel(const TransposeParams p) {
  __shared__ __align__(16) uint32_t tile[64][32];
  const long long b = blockIdx.z;
  const long long p0 = (long long)blockIdx.y * 64, c0 = (long long)blockIdx.x * 64;
  const unsigned short* src = reinterpret_cast<const unsigned short*>(p.x) + b * p.in_batch_stride;
  unsigned short* dst = reinterpret_cast<unsigned short*>(p.y) + b * p.P * p.C;
  const int tid = threadIdx.x;
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int q = tid + k * 256;
    const int r = q >> 3, wv = q & 7;
    const uint4 v = ld_stream(reinterpret_cast<const __half*>(src + (p0 + r) * p.in_row_stride + c0 + wv * 8));
    *reinterpret_cast<uint4*>(&tile[r][(wv * 4 + 4 * (r >> 3)) & 31]) = v;
  }
  __syncthreads();
  const int ovc = tid & 7, cpair = tid >> 3;
  uint32_t w[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) w[j] = tile[ovc * 8 + j][(cpair + 4 * ovc) & 31];
  uint4 lo, hi;
  lo.x = __byte_perm(w[0], w[1], 0x5410); hi.x = __byte_perm(w[0], w[1], 0x7632);
  lo.y = __byte_perm(w[2], w[3], 0x5410); hi.y = __byte_perm(w[2], w[3], 0x7632);
  lo.z = __byte_perm(w[4], w[5], 0x5410); hi.z = __byte_perm(w[4], w[5], 0x7632);
  lo.w = __byte_perm(w[6], w[7], 0x5410); hi.w = __byte_perm(w[6], w[7], 0x7632);
  unsigned short* o = dst + (c0 + 2 * cpair) * p.P + p0 + ovc * 8;
  st_stream(reinterpret_cast<__half*>(o), lo);
  st_stream(reinterpret_cast<__half*>(o + p.P), hi);
}

// Batched transpose of SMALL matrices without conversion (a [P, C] matrix and its transpose fit in
// shared memory; e.g. the [49, 128] and [196, 64] attention tiles of
// repros/canonical/pointwise_021e90d9c17d/shapes.json, whose 49 rows fill a 64 x 64 tile only to
// three quarters and whose output rows of 49 elements do not start on 16-byte boundaries). The
// input matrix and the output matrix of one batch entry are each ONE contiguous block, so both are
// moved with 16-byte accesses as flat arrays; the transposition is the shared-memory gather in
// between: output element o = c * P + p comes from [p][c]. A CTA takes matrices b, b + grid, ...
template <typename E>  // E: unsigned short (16-bit elements) or unsigned int (32-bit elements)
__global__ void __launch_bounds__(256) transpose_small_kernel(const TransposeParams p, const int pitch) {
  constexpr int VE = 16 / (int)sizeof(E);
  extern __shared__ __align__(16) unsigned char small_smem[];
  E* tile = reinterpret_cast<E*>(small_smem);  // [P][pitch]
  const int P = (int)p.P, C = (int)p.C;
  const int nvec = P * C / VE;
  for (long long b = blockIdx.x; b < p.batch; b += gridDim.x) {
    const E* src = reinterpret_cast<const E*>(p.x) + b * p.in_batch_stride;
    E* dst = reinterpret_cast<E*>(p.y) + b * (long long)P * C;
    for (int j0 = threadIdx.x; j0 < nvec; j0 += 4 * 256) {  // four loads in flight per thread
      uint4 raws[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int j = j0 + u * 256;
        if (j < nvec) raws[u] = ld_stream(reinterpret_cast<const float*>(src) + (size_t)j * 4);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int j = j0 + u * 256;
        if (j >= nvec) continue;
        const uint4 raw = raws[u];
        const int e0 = j * VE;
        const int r = e0 / C, c0 = e0 - r * C;  // C is a multiple of VE: the vector stays in one row
        E* t = tile + r * pitch + c0;
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        if constexpr (sizeof(E) == 2) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            t[2 * k] = (E)(w[k] & 0xffffu);
            t[2 * k + 1] = (E)(w[k] >> 16);
          }
        } else {
#pragma unroll
          for (int k = 0; k < 4; ++k) t[k] = (E)w[k];
        }
      }
    }
    __syncthreads();
    for (int j = threadIdx.x; j < nvec; j += 256) {
      int o = j * VE;
      int c = o / P, r = o - c * P;
      uint32_t w[4];
      if constexpr (sizeof(E) == 2) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint32_t lo = tile[r * pitch + c];
          if (++r == P) { r = 0; ++c; }
          const uint32_t hi = tile[r * pitch + c];
          if (++r == P) { r = 0; ++c; }
          w[k] = lo | (hi << 16);
        }
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          w[k] = tile[r * pitch + c];
          if (++r == P) { r = 0; ++c; }
        }
      }
      st_stream(reinterpret_cast<float*>(dst) + (size_t)j * 4, make_uint4(w[0], w[1], w[2], w[3]));
    }
    __syncthreads();  // the tile is overwritten by the next matrix
  }
}

// Contiguous cast / scale / activation (has_scale: bit 0 multiply by scale; bits 1..3 ReLU, exact GELU, SiLU after it).
// ACT: the activation bit of the mode word (0: none); the plain cast / scale instantiation carries none of
// the activations' code (the erf and exp sequences cost registers and instruction-cache lines that a 5 us
// parameter cast would pay for without using them).
template <typename Tin, typename Tout, bool VEC, int ACT>
__global__ void __launch_bounds__(256, ACT >= 4 ? 3 : 4) cast_scale_kernel(const void* x, void* y, long long n, float scale,
                                                                            int mode_word) {
  const int has_scale = mode_word & 1;
  constexpr int VIN = VEC ? Elem<Tin>::V : 1;
  const long long units = n / VIN;
  const Tin* src = reinterpret_cast<const Tin*>(x);
  Tout* dst = reinterpret_cast<Tout*>(y);
  if constexpr (VEC) {
    // A CTA takes blocks of U * blockDim consecutive vectors (block b, b + grid, ...): its U loads
    // in flight per thread fall into one contiguous stretch of memory.
    constexpr int U = 4;
    const long long stride = blockDim.x;
    const long long block = (long long)U * blockDim.x;
    for (long long u0 = (long long)blockIdx.x * block + threadIdx.x; u0 < units; u0 += (long long)gridDim.x * block) {
      uint4 raw[U];
#pragma unroll
      for (int k = 0; k < U; ++k) {
        const long long u = u0 + k * stride;
        if (u < units) raw[k] = ld_stream(src + u * VIN);
      }
#pragma unroll
      for (int k = 0; k < U; ++k) {
        const long long u = u0 + k * stride;
        if (u < units) {
          float f[VIN];
          Elem<Tin>::unpack(raw[k], f);
          if (has_scale & 1) {
#pragma unroll
            for (int i = 0; i < VIN; ++i) f[i] = f[i] * scale;
          }
          if constexpr (ACT == 8 && sizeof(Tout) == 2) {
            // SiLU for a 16-bit result: exp(-x) from the compensated pair exponential (the accuracy
            // class of expf) and x * (1 / (e + 1)) with a correctly rounded reciprocal: 1.5 fp32 ulp,
            // three orders of magnitude below half an ulp of the output, at a third of the
            // instructions of expf and an IEEE division. The argument is clamped to the range in
            // which the result does not depend on it any more (the exponential needs finite inputs).
#pragma unroll
            for (int i = 0; i < VIN / 2; ++i) {
              const float a = f[2 * i], b = f[2 * i + 1];
              float ea, eb;
              unpack2(exp_pair_compensated(pack2(fminf(fmaxf(-a, -87.f), 88.f), fminf(fmaxf(-b, -87.f), 88.f))), ea, eb);
              f[2 * i] = a * __frcp_rn(ea + 1.0f);
              f[2 * i + 1] = b * __frcp_rn(eb + 1.0f);
            }
          } else if constexpr (ACT != 0) {
#pragma unroll
            for (int i = 0; i < VIN; ++i) f[i] = apply_activation<ACT>(f[i]);
          }
          store_converted<Tout, VIN>(dst + u * VIN, f);
        }
      }
    }
  } else {
    for (long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x; u < units;
         u += (long long)gridDim.x * blockDim.x)
      dst[u] = convert_scaled<Tin, Tout, ACT>(src[u], scale, has_scale);
  }
  if constexpr (VEC) {  // ragged tail
    const long long done = units * VIN;
    const long long t = done + (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t < n) dst[t] = convert_scaled<Tin, Tout, ACT>(src[t], scale, has_scale);
  }
}

// Grid of the flat streaming kernels: one CTA per 256 units up to `per_sm` CTAs per SM, which then
// loop. Many small CTAs keep the window of addresses that are in flight at any moment narrow; for
// the cast kernel 128 per SM measured best on a 262 M-element bf16 -> f32 cast (8: 331 us, 16: 299,
// 32: 279, 64: 268, 128: 263, 256: 285, one CTA per block: 331). B200_STREAM_CTAS_PER_SM overrides both.
static unsigned streaming_grid(long long units, long long default_per_sm = 16) {
  const long long ctas = (units + 255) / 256;
  static const long long env_per_sm = [] { const char* e = getenv("B200_STREAM_CTAS_PER_SM"); return e ? atoll(e) : 0LL; }();
  const long long per_sm = env_per_sm > 0 ? env_per_sm : default_per_sm;
  const long long cap = (long long)device_info().sm_count * per_sm;
  return (unsigned)(ctas < 1 ? 1 : (ctas > cap ? cap : ctas));
}

template <typename Tin, typename Tout>
static int launch_permute(const PermuteParams& p, bool vec, cudaStream_t st) {
  const long long units = vec ? p.total / Elem<Tin>::V : p.total;
  set_path_tag(vec ? "vector gather" : "element-wise gather");
  if (vec) permute_general_kernel<Tin, Tout, true><<<streaming_grid(units), 256, 0, st>>>(p);
  else permute_general_kernel<Tin, Tout, false><<<streaming_grid(units), 256, 0, st>>>(p);
  return launch_status("b200_permute_copy");
}

template <typename Tin, typename Tout>
static int launch_transpose(const TransposeParams& p, cudaStream_t st) {
  if constexpr (std::is_same<Tin, Tout>::value) {
    // small matrices that are not made of whole 64 x 64 tiles: flat 16-byte copies around a
    // shared-memory gather
    constexpr int VE = 16 / (int)sizeof(Tin);
    const long long elems = p.P * p.C;
    const bool tiles64 = sizeof(Tin) == 2 && p.P % 64 == 0 && p.C % 64 == 0;
    if (!p.has_scale && !tiles64 && elems * (long long)sizeof(Tin) <= 32 * 1024 && p.C % VE == 0 && elems % VE == 0 &&
        p.in_row_stride == p.C && p.in_batch_stride % VE == 0 && aligned16(p.x) && aligned16(p.y) && p.batch >= 1) {
      const int pitch = (int)p.C + 1;
      const size_t smem = (size_t)p.P * pitch * sizeof(Tin);
      if (smem <= 48 * 1024) {
        long long grid = p.batch;
        const long long cap = (long long)device_info().sm_count * 8;
        if (grid > cap) grid = cap;
        if constexpr (sizeof(Tin) == 2) transpose_small_kernel<unsigned short><<<(unsigned)grid, 256, smem, st>>>(p, pitch);
        else transpose_small_kernel<unsigned int><<<(unsigned)grid, 256, smem, st>>>(p, pitch);
        return launch_status("b200_transpose_copy [small matrices, flat 16-byte copies]");
      }
    }
  }
  dim3 grid((unsigned)((p.C + 63) / 64), (unsigned)((p.P + 63) / 64), (unsigned)p.batch);
  if constexpr (std::is_same<Tin, Tout>::value && sizeof(Tin) == 2) {
    const bool whole = p.P % 64 == 0 && p.C % 64 == 0 && !p.has_scale && p.in_row_stride % 8 == 0 &&
                       p.in_batch_stride % 8 == 0 && aligned16(p.x) && aligned16(p.y);
    if (whole) {
      transpose16_tile_kernel<<<grid, 256, 0, st>>>(p);
      return launch_status("b200_transpose_copy [16-byte tiles]");
    }
  }
  transpose_tile_kernel<Tin, Tout><<<grid, 256, 0, st>>>(p);
  return launch_status("b200_transpose_copy [element tiles]");
}

template <typename Tin, typename Tout>
static int launch_cast(const void* x, void* y, long long n, float scale, int has_scale, bool vec, cudaStream_t st) {
  const long long units = vec ? n / Elem<Tin>::V : n;
  set_path_tag(vec ? "vector" : "element-wise");
  const unsigned grid = streaming_grid(units > 0 ? units : 1, 128);
  auto go = [&](auto act_tag) {
    constexpr int ACT = decltype(act_tag)::value;
    if (vec) cast_scale_kernel<Tin, Tout, true, ACT><<<grid, 256, 0, st>>>(x, y, n, scale, has_scale);
    else cast_scale_kernel<Tin, Tout, false, ACT><<<grid, 256, 0, st>>>(x, y, n, scale, has_scale);
  };
  switch (has_scale & 14) {
    case 0: go(std::integral_constant<int, 0>{}); break;
    case 2: go(std::integral_constant<int, 2>{}); break;
    case 4: go(std::integral_constant<int, 4>{}); break;
    case 8: go(std::integral_constant<int, 8>{}); break;
    default: return fail(B200_ERR_INVALID, "b200_cast_scale: one activation at a time (mode %d)", has_scale);
  }
  return launch_status("b200_cast_scale");
}

}  // namespace b200

using namespace b200;

#define B200_DTYPE_PAIRS(MACRO)                                  \
  MACRO(float, float, B200_F32, B200_F32)                        \
  MACRO(__nv_bfloat16, __nv_bfloat16, B200_BF16, B200_BF16)      \
  MACRO(__half, __half, B200_F16, B200_F16)                      \
  MACRO(__nv_bfloat16, float, B200_BF16, B200_F32)               \
  MACRO(__half, float, B200_F16, B200_F32)                       \
  MACRO(float, __nv_bfloat16, B200_F32, B200_BF16)               \
  MACRO(float, __half, B200_F32, B200_F16)

extern "C" int b200_permute_copy(const void* x, void* y, const int64_t* out_shape, const int64_t* in_strides,
                                 int32_t in_dtype, int32_t out_dtype, double scale, int32_t has_scale,
                                 void* stream) {
  if (!x || !y || !out_shape || !in_strides) return fail(B200_ERR_INVALID, "b200_permute_copy: null argument");
  PermuteParams p;
  p.x = x; p.y = y; p.total = 1;
  for (int i = 0; i < 4; ++i) {
    if (out_shape[i] < 0) return fail(B200_ERR_INVALID, "b200_permute_copy: negative extent");
    p.shape[i] = out_shape[i];
    p.in_stride[i] = in_strides[i];
    p.total *= out_shape[i];
  }
  if (p.total == 0) return B200_OK;
  for (int i = 1; i < 4; ++i)
    if (out_shape[i] > 0x7fffffffLL) return fail(B200_ERR_UNSUPPORTED, "b200_permute_copy: extent beyond 2^31-1");
  p.scale = (float)scale; p.has_scale = has_scale ? 1 : 0;
  const int ib = dtype_size(in_dtype), ob = dtype_size(out_dtype);
  const int vin = 16 / ib;
  const int out_chunk = vin * ob < 16 ? vin * ob : 16;
  bool vec = in_strides[3] == 1 && out_shape[3] % vin == 0 && aligned16(x) &&
             reinterpret_cast<uintptr_t>(y) % out_chunk == 0;
  for (int i = 0; i < 3; ++i) vec = vec && (in_strides[i] * ib) % 16 == 0;
  p.d1 = make_fast_div(out_shape[1]);
  p.d2 = make_fast_div(out_shape[2]);
  p.d3 = make_fast_div(vec ? out_shape[3] / vin : out_shape[3]);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define B200_CASE(TI, TO, DI, DO) if (in_dtype == DI && out_dtype == DO) return launch_permute<TI, TO>(p, vec, st);
  B200_DTYPE_PAIRS(B200_CASE)
#undef B200_CASE
  return fail(B200_ERR_UNSUPPORTED, "b200_permute_copy: dtype pair (%d -> %d) not built", in_dtype, out_dtype);
}

extern "C" int b200_transpose_copy(const void* x, void* y, int64_t batch, int64_t rows, int64_t cols,
                                   int64_t in_batch_stride, int64_t in_row_stride, int32_t in_dtype,
                                   int32_t out_dtype, double scale, int32_t has_scale, void* stream) {
  if (!x || !y) return fail(B200_ERR_INVALID, "b200_transpose_copy: null argument");
  if (batch < 0 || rows < 0 || cols < 0) return fail(B200_ERR_INVALID, "b200_transpose_copy: negative size");
  if (batch == 0 || rows == 0 || cols == 0) return B200_OK;
  if (batch > 65535 || (rows + 63) / 64 > 65535)
    return fail(B200_ERR_UNSUPPORTED, "b200_transpose_copy: grid too large (fold batch dimensions)");
  TransposeParams p;
  p.x = x; p.y = y; p.batch = batch; p.P = rows; p.C = cols;
  p.in_batch_stride = in_batch_stride; p.in_row_stride = in_row_stride;
  p.scale = (float)scale; p.has_scale = has_scale ? 1 : 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define B200_CASE(TI, TO, DI, DO) if (in_dtype == DI && out_dtype == DO) return launch_transpose<TI, TO>(p, st);
  B200_DTYPE_PAIRS(B200_CASE)
#undef B200_CASE
  return fail(B200_ERR_UNSUPPORTED, "b200_transpose_copy: dtype pair (%d -> %d) not built", in_dtype, out_dtype);
}

extern "C" int b200_cast_scale(const void* x, void* y, int64_t n, int32_t in_dtype, int32_t out_dtype,
                               double scale, int32_t has_scale, void* stream) {
  if (n < 0) return fail(B200_ERR_INVALID, "b200_cast_scale: negative size");
  if (n == 0) return B200_OK;
  if (!x || !y) return fail(B200_ERR_INVALID, "b200_cast_scale: null argument");
  const int ib = dtype_size(in_dtype), ob = dtype_size(out_dtype);
  const int vin = 16 / ib;
  const int out_chunk = vin * ob < 16 ? vin * ob : 16;
  const bool vec = aligned16(x) && reinterpret_cast<uintptr_t>(y) % out_chunk == 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define B200_CASE(TI, TO, DI, DO) \
  if (in_dtype == DI && out_dtype == DO) return launch_cast<TI, TO>(x, y, n, (float)scale, has_scale & 15, vec, st);
  B200_DTYPE_PAIRS(B200_CASE)
#undef B200_CASE
  return fail(B200_ERR_UNSUPPORTED, "b200_cast_scale: dtype pair (%d -> %d) not built", in_dtype, out_dtype);
}
