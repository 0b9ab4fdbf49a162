// Shared device/host helpers for the sm_100a oracle kernels.
//
// Everything here is header-only and included by each family's .cu file.
// Conventions used throughout the library:
//   * dtype codes: 0 = float32, 1 = bfloat16, 2 = float16 (B200_F32 / B200_BF16 / B200_F16)
//   * all arithmetic is fp32 (fp64 only for the final combination of split partial sums);
//     the translation units are compiled with -fmad=false so a*b+c is two rounded operations,
//     exactly as a decomposed aten graph evaluates it
//   * the "vector path" moves 16 bytes per thread per access and requires 16-byte aligned
//     row starts; every family also has an element-wise path for unaligned or ragged rows
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <string.h>

#define B200_F32 0
#define B200_BF16 1
#define B200_F16 2

// ----------------------------------------------------------------------------------------
// Host-side error state (thread local). Entry points return 0 on success, a negative
// B200_ERR_* code for an argument error found before any launch, or a positive cudaError_t
// when the launch itself was rejected.
// ----------------------------------------------------------------------------------------
#define B200_OK 0
#define B200_ERR_INVALID -1      // null pointer, negative size, bad enum
#define B200_ERR_UNSUPPORTED -2  // valid request this build has no kernel for
#define B200_ERR_ALIGNMENT -3    // pointer or stride breaks an alignment the caller promised
#define B200_ERR_WORKSPACE -4    // scratch buffer missing or too small
#define B200_ERR_DEVICE_WAIT -5  // a bounded device-side wait ran out (reported by b200_check_status)

namespace b200 {

char* last_error_buffer();  // defined in abi.cu (thread-local storage, 512 bytes)

inline int fail(int code, const char* fmt, ...) {
  char* buf = last_error_buffer();
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, 512, fmt, ap);
  va_end(ap);
  return code;
}

// Defined in abi.cu. note_launch counts a kernel launch for b200_launch_count() and remembers
// its name (with the path tag, if one was set since the previous launch) for b200_last_kernel().
// set_path_tag names the variant a launcher chose ("vector", "element-wise", "streaming", ...):
// a pointer to a string literal, consumed by the next note_launch on this thread.
void note_launch(const char* what);
void set_path_tag(const char* tag);

// Call after every kernel launch: counts it and reports a rejected launch.
inline int launch_status(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    fail((int)e, "%s: launch failed: %s", what, cudaGetErrorString(e));
    return (int)e;
  }
  note_launch(what);
  return B200_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int dtype_size(int dt) { return dt == B200_F32 ? 4 : 2; }

// Number of SMs and opt-in shared memory of the current device, cached per device.
struct DeviceInfo {
  int sm_count;
  int max_smem_optin;
  int l2_bytes;
};
const DeviceInfo& device_info();  // defined in abi.cu

// ----------------------------------------------------------------------------------------
// Element traits: 16-byte vectors of T, conversion to and from fp32.
// ----------------------------------------------------------------------------------------
template <typename T>
struct Elem;

template <>
struct Elem<float> {
  static constexpr int V = 4;  // elements per 16-byte vector
  static __device__ __forceinline__ float to_f32(float v) { return v; }
  static __device__ __forceinline__ float from_f32(float v) { return v; }
  static __device__ __forceinline__ void unpack(const uint4& r, float (&f)[4]) {
    f[0] = __uint_as_float(r.x);
    f[1] = __uint_as_float(r.y);
    f[2] = __uint_as_float(r.z);
    f[3] = __uint_as_float(r.w);
  }
  static __device__ __forceinline__ uint4 pack(const float (&f)[4]) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                      __float_as_uint(f[3]));
  }
};

template <>
struct Elem<__nv_bfloat16> {
  static constexpr int V = 8;
  static __device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
  static __device__ __forceinline__ void unpack(const uint4& r, float (&f)[8]) {
    // bf16 -> fp32 is a 16-bit left shift; two elements per 32-bit word, low half first.
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ uint4 pack(const float (&f)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 p = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&p);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};

template <>
struct Elem<__half> {
  static constexpr int V = 8;
  static __device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f32(float v) { return __float2half_rn(v); }
  static __device__ __forceinline__ void unpack(const uint4& r, float (&f)[8]) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
      float2 t = __half22float2(h);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
  static __device__ __forceinline__ uint4 pack(const float (&f)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 p = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&p);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};

// ----------------------------------------------------------------------------------------
// 16-byte global accesses with cache hints.
//   ld_stream : read-once data, bypass L1 allocation
//   ld_keep   : data that is read again soon (small broadcast operands) - default caching
//   st_stream : write-once results
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 r;
#ifdef B200_LD_STREAM_L2_EVICT_FIRST
  // build variant for measurements: read-once data is also the first candidate for eviction from L2
  uint64_t pol;
  asm("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p), "l"(pol));
#else
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
#endif
  return r;
}

__device__ __forceinline__ uint4 ld_keep(const void* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}

// Plain (coherent) 16-byte load: for data another CTA of the same grid wrote earlier.
__device__ __forceinline__ uint4 ld_coherent(const void* p) {
  uint4 r;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p)
               : "memory");
  return r;
}

__device__ __forceinline__ void st_stream(void* p, const uint4& v) {
#ifdef B200_ST_STREAM_DEFAULT
  // build variant for measurements: write-once results with the default cache policy
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
#else
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
#endif
}

__device__ __forceinline__ void st_default(void* p, const uint4& v) {
  *reinterpret_cast<uint4*>(p) = v;
}

// L2 eviction-priority policies (createpolicy) for data that should stay in, or leave, L2.
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint64_t l2_policy_evict_normal() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint4 ld_policy(const void* p, uint64_t pol) {
  uint4 r;
  asm volatile("ld.global.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p), "l"(pol)
               : "memory");
  return r;
}
__device__ __forceinline__ void st_policy(void* p, const uint4& v, uint64_t pol) {
  asm volatile("st.global.L2::cache_hint.v4.u32 [%0], {%1,%2,%3,%4}, %5;" ::"l"(p), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w), "l"(pol)
               : "memory");
}

// ----------------------------------------------------------------------------------------
// Reductions. Orders are fixed (butterfly within a warp, then warp 0..n-1 in sequence), so
// every launch of the same shape produces the same bits.
// ----------------------------------------------------------------------------------------
struct SumOp {
  static constexpr bool is_sum = true;
  static __device__ __forceinline__ float identity() { return 0.f; }
  static __device__ __forceinline__ float apply(float a, float b) { return a + b; }
};
struct MaxOp {
  static constexpr bool is_sum = false;
  static __device__ __forceinline__ float identity() { return -INFINITY; }
  // NaN-propagating maximum, as aten.amax: any NaN operand gives NaN.
  static __device__ __forceinline__ float apply(float a, float b) {
    float r;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));  // one instruction, NaN if either is NaN
    return r;
  }
  // the same on packed 16-bit pairs: a maximum is exact in any precision
  static __device__ __forceinline__ __half2 apply2(__half2 a, __half2 b) { return __hmax2_nan(a, b); }
  static __device__ __forceinline__ __nv_bfloat162 apply2(__nv_bfloat162 a, __nv_bfloat162 b) { return __hmax2_nan(a, b); }
};
struct MinOp {
  static constexpr bool is_sum = false;
  static __device__ __forceinline__ float identity() { return INFINITY; }
  static __device__ __forceinline__ float apply(float a, float b) {
    float r;
    asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
  }
  static __device__ __forceinline__ __half2 apply2(__half2 a, __half2 b) { return __hmin2_nan(a, b); }
  static __device__ __forceinline__ __nv_bfloat162 apply2(__nv_bfloat162 a, __nv_bfloat162 b) { return __hmin2_nan(a, b); }
};

template <typename Op>
__device__ __forceinline__ float warp_reduce(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = Op::apply(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide reduction; every thread returns the result. `scratch` holds >= 32 floats and is
// reusable immediately after return (two barriers inside).
template <typename Op>
__device__ __forceinline__ float block_reduce(float v, float* scratch) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_reduce<Op>(v);
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = Op::identity();
  for (int w = 0; w < nwarps; ++w) r = Op::apply(r, scratch[w]);
  __syncthreads();
  return r;
}

// Group reduce: a warp (BLOCK == false) or the whole CTA (BLOCK == true).
template <typename Op, bool BLOCK>
__device__ __forceinline__ float group_reduce(float v, float* scratch) {
  if constexpr (BLOCK) {
    return block_reduce<Op>(v, scratch);
  } else {
    return warp_reduce<Op>(v);
  }
}

// ----------------------------------------------------------------------------------------
// Grid-wide barrier for cooperative (co-resident) launches, with a bounded wait.
// `bar` points at four 32-bit words of global scratch that are zero before the launch:
//   [0] arrival counter, [1] error flag, [2] departure counter, [3] work counter of kernels that
//   hand out blocks dynamically (reset with the others).
// Each use of the barrier within one launch passes the next `phase` (1, 2, ..): the arrival
// counter only grows, and phase p completes when it reaches p * gridDim.x. Every CTA calls
// grid_barrier_depart() once after its last barrier; the last CTA to depart puts the counters
// back to zero, so the next launch on the same stream needs no memset. A wait that runs out
// sets the error flag (which stays set until the host clears the words) and returns false;
// callers then skip the remaining work, so the context stays usable and the host can report
// B200_ERR_DEVICE_WAIT.
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ bool grid_barrier(unsigned int* bar, unsigned int phase, int* smem_flag) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(&bar[0], 1u);
    const unsigned int target = phase * gridDim.x;
    int ok = 1;
    unsigned int spins = 0;
    while (true) {
      unsigned int seen;
      asm volatile("ld.global.acquire.gpu.u32 %0, [%1];" : "=r"(seen) : "l"(bar) : "memory");
      if (seen >= target) break;
      unsigned int err;
      asm volatile("ld.global.relaxed.gpu.u32 %0, [%1];" : "=r"(err) : "l"(bar + 1) : "memory");
      if (err != 0u || ++spins > (1u << 22)) {  // ~4M polls: a fraction of a second
        atomicExch(&bar[1], 1u);
        ok = 0;
        break;
      }
      if (spins > 4096) __nanosleep(64);  // poll tightly at first: the usual wait is a few microseconds
    }
    __threadfence();
    *smem_flag = ok;
  }
  __syncthreads();
  return *smem_flag != 0;
}

__device__ __forceinline__ void grid_barrier_depart(unsigned int* bar) {
  if (threadIdx.x == 0) {
    const unsigned int old = atomicAdd(&bar[2], 1u);
    if (old == gridDim.x - 1) {
      // Everyone has left every barrier of this launch (or gave up): reset for the next one.
      // The error flag is left alone on purpose.
      atomicExch(&bar[0], 0u);
      atomicExch(&bar[2], 0u);
      atomicExch(&bar[3], 0u);
      __threadfence();
    }
  }
}

// The occupancy query is a host-side calculation; cached per (kernel, block size, smem).
inline int cached_occupancy(const void* fn, int threads, size_t smem = 0) {
  struct Entry { const void* fn; int threads; size_t smem; int blocks; };
  static Entry cache[256];
  static int used = 0;
  for (int i = 0; i < used; ++i)
    if (cache[i].fn == fn && cache[i].threads == threads && cache[i].smem == smem) return cache[i].blocks;
  int blocks = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, fn, threads, smem) != cudaSuccess) {
    cudaGetLastError();
    blocks = 1;
  }
  if (blocks < 1) blocks = 1;
  if (used < 256) cache[used++] = Entry{fn, threads, smem, blocks};
  return blocks;
}

}  // namespace b200
