// Helpers shared by the row-wise families (row reductions, softmax, LayerNorm/RMSNorm forward).
//
// Work decomposition: a "group" of threads owns one row. The group is one warp (short rows,
// several rows per CTA, no block barrier) or the whole CTA (long rows). A row of n elements is
// nv = n / V sixteen-byte vectors; vector j belongs to group lane j % G and register slot j / G,
// so each slot is one fully coalesced G x 16-byte access and all of a thread's loads are issued
// before the first is consumed.
#pragma once

#include "common.cuh"

namespace b200 {

// Maps a flat row index onto up to three outer dimensions with arbitrary element strides, so
// broadcast operands (stride 0) and non-contiguous views need no copy. row = (i0*d1 + i1)*d2 + i2.
struct RowMap {
  long long s0, s1, s2;
  int d1, d2;
};

__device__ __forceinline__ long long row_offset(const RowMap& m, long long row) {
  if (m.d1 == 1 && m.d2 == 1) return row * m.s0;
  const long long i2 = row % m.d2;
  const long long t = row / m.d2;
  const long long i1 = t % m.d1;
  const long long i0 = t / m.d1;
  return i0 * m.s0 + i1 * m.s1 + i2 * m.s2;
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

// Pick the launch geometry for a register-resident row: nv vectors per row.
//   warp mode  : nv <= 128 -> 256-thread CTAs (8 rows each), CH = 1, 2 or 4 slots
//   block mode : nv <= 4096 -> one CTA per row, CH = 2, 4 or 8 slots, 32..512 threads
// Returns false when the row does not fit (the caller then uses the streaming kernel).
struct RowGeometry {
  bool block;
  int ch;
  int threads;
};

inline bool pick_row_geometry(long long nv, RowGeometry* g) {
  if (nv <= 0) return false;
  if (nv <= 128) {
    g->block = false;
    g->threads = 256;
    g->ch = nv <= 32 ? 1 : (nv <= 64 ? 2 : 4);
    return true;
  }
  if (nv > 4096) return false;
  g->block = true;
  g->ch = nv <= 512 ? 2 : (nv <= 2048 ? 4 : 8);
  long long t = (nv + g->ch - 1) / g->ch;
  t = (t + 31) / 32 * 32;
  g->threads = (int)t;
  return true;
}

}  // namespace b200
