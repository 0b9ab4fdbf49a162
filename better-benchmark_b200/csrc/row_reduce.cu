// Row reductions over the last (contiguous) dimension: sum, mean, amax, amin.
//
// Replaces the row-form Triton kernels of the mean/sum/amax repros in the reference
// (repros/canonical/mean_c9e1a8113328/oracle.py:11-76 for the contiguous case,
// amax_sum_7079889cfc04/oracle.py:20-29 for the long-row loop).
//
// One warp (many short rows) or one CTA (few or long rows) streams a row once with eight
// 16-byte loads in flight per thread, accumulating in fp32 in V independent chains per thread,
// then a fixed-order shuffle/shared-memory tree. mean multiplies the sum by 1/n, as aten does.
#include "rowwise.cuh"

#include <type_traits>

namespace b200 {

#define B200_REDUCE_SUM 0
#define B200_REDUCE_MEAN 1
#define B200_REDUCE_AMAX 2
#define B200_REDUCE_AMIN 3

struct RowReduceParams {
  const void* x;
  void* out;
  long long rows;
  long long n;
  RowMap xmap;
  long long out_stride;
  int out_dtype;
  float post_scale;  // 1/n for mean, 1 otherwise
};

__device__ __forceinline__ void store_scalar(void* out, int dtype, long long idx, float v) {
  if (dtype == B200_F32) {
    reinterpret_cast<float*>(out)[idx] = v;
  } else if (dtype == B200_BF16) {
    reinterpret_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
  } else {
    reinterpret_cast<__half*>(out)[idx] = __float2half_rn(v);
  }
}

// U = 16-byte loads in flight per thread. Warp mode uses U = 4 and at most 32 registers so that
// 64 warps fit on an SM; block mode uses U = 8.
template <typename Tin, typename Op, bool BLOCK, bool VEC>
__global__ void __launch_bounds__(BLOCK ? 1024 : 256, BLOCK ? 1 : 8)
row_reduce_kernel(const RowReduceParams p) {
  constexpr int V = Elem<Tin>::V;
  constexpr int U = BLOCK ? 8 : 4;
  __shared__ __align__(8) float red[64];
  const int lane = group_lane<BLOCK>();
  const int G = group_size<BLOCK>();
  const long long row = group_row<BLOCK>();
  if (row >= p.rows) return;
  const Tin* x = reinterpret_cast<const Tin*>(p.x) + row_offset(p.xmap, row);

  float acc[V];
#pragma unroll
  for (int i = 0; i < V; ++i) acc[i] = Op::identity();

  long long done = 0;  // elements covered by the vector loop
  if constexpr (VEC && !Op::is_sum && sizeof(Tin) == 2) {
    // Maximum / minimum of 16-bit elements: exact in the storage type, so the vectors are folded
    // as packed pairs (one instruction per two elements, no conversion) and only the last pair
    // of each thread is widened.
    using P2 = typename std::conditional<std::is_same<Tin, __half>::value, __half2, __nv_bfloat162>::type;
    const long long nv = p.n / V;
    P2 m[4];
    {
      const Tin id = Elem<Tin>::from_f32(Op::identity());
      P2 idp;
      idp.x = id;
      idp.y = id;
#pragma unroll
      for (int i = 0; i < 4; ++i) m[i] = idp;
    }
    for (long long j0 = lane; j0 < nv; j0 += (long long)G * U) {
      uint4 raw[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long j = j0 + (long long)u * G;
        if (j < nv) raw[u] = ld_stream(x + j * V);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long j = j0 + (long long)u * G;
        if (j < nv) {
          const uint32_t w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
#pragma unroll
          for (int i = 0; i < 4; ++i) m[i] = Op::apply2(m[i], *reinterpret_cast<const P2*>(&w[i]));
        }
      }
    }
    const P2 a = Op::apply2(Op::apply2(m[0], m[1]), Op::apply2(m[2], m[3]));
    acc[0] = Op::apply(Elem<Tin>::to_f32(a.x), Elem<Tin>::to_f32(a.y));
    done = nv * V;
  } else if constexpr (VEC) {
    const long long nv = p.n / V;
    for (long long j0 = lane; j0 < nv; j0 += (long long)G * U) {
      uint4 raw[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long j = j0 + (long long)u * G;
        if (j < nv) raw[u] = ld_stream(x + j * V);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long j = j0 + (long long)u * G;
        if (j < nv) {
          float f[V];
          Elem<Tin>::unpack(raw[u], f);
#pragma unroll
          for (int i = 0; i < V; ++i) acc[i] = Op::apply(acc[i], f[i]);
        }
      }
    }
    done = nv * V;
  }
  for (long long i = done + lane; i < p.n; i += G)
    acc[0] = Op::apply(acc[0], Elem<Tin>::to_f32(x[i]));

  float r;
  if constexpr (Op::is_sum) {
    // Per-thread chains are short (tens of elements); everything above them is combined in
    // fp64 so that the result is the correctly rounded sum of the chain values.
    double d = 0.0;
#pragma unroll
    for (int i = 0; i < V; ++i) d += (double)acc[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
    if constexpr (BLOCK) {
      double* dred = reinterpret_cast<double*>(red);
      const int warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
      if ((threadIdx.x & 31) == 0) dred[warp] = d;
      __syncthreads();
      d = 0.0;
      for (int w = 0; w < nwarps; ++w) d += dred[w];
    }
    r = (float)d;
  } else {
#pragma unroll
    for (int w = V / 2; w > 0; w >>= 1) {
#pragma unroll
      for (int i = 0; i < w; ++i) acc[i] = Op::apply(acc[i], acc[i + w]);
    }
    r = group_reduce<Op, BLOCK>(acc[0], red);
  }
  if (lane == 0) store_scalar(p.out, p.out_dtype, row * p.out_stride, r * p.post_scale);
}

template <typename Tin, typename Op>
static int launch_row_reduce(const RowReduceParams& p, bool vec, cudaStream_t st) {
  constexpr int V = Elem<Tin>::V;
  const int sms = device_info().sm_count;
  // CTA-per-row geometry: about eight vectors per thread.
  int threads = (int)((p.n / V + 7) / 8);
  threads = (threads + 31) / 32 * 32;
  threads = threads < 64 ? 64 : (threads > 1024 ? 1024 : threads);
  // Tail model: work that needs more than one wave of resident CTAs loses the unfilled part of
  // its last wave. Warp-per-row (8 rows per 256-thread CTA, 8 CTAs per SM) needs enough rows to
  // fill the machine and rows short enough for one warp; otherwise one CTA per row.
  auto efficiency = [&](double units, double resident_per_sm) {
    const double waves = units / (sms * resident_per_sm);
    return waves <= 1.0 ? 1.0 : waves / (double)(long long)(waves + 0.999999);
  };
  const double eff_warp = efficiency((double)((p.rows + 7) / 8), 8.0);
  const double eff_block = efficiency((double)p.rows, (double)(2048 / threads > 32 ? 32 : 2048 / threads));
  const bool warp_mode = p.rows >= (long long)sms * 16 && p.n <= 16384 && eff_warp + 0.02 >= eff_block;
  set_path_tag(vec ? (warp_mode ? "vector, warp per row" : "vector, CTA per row")
                   : (warp_mode ? "element-wise, warp per row" : "element-wise, CTA per row"));
  if (warp_mode) {
    const long long grid = (p.rows + 7) / 8;
    if (grid > 0x7fffffffLL) return fail(B200_ERR_UNSUPPORTED, "row_reduce: too many rows");
    if (vec) row_reduce_kernel<Tin, Op, false, true><<<(unsigned)grid, 256, 0, st>>>(p);
    else row_reduce_kernel<Tin, Op, false, false><<<(unsigned)grid, 256, 0, st>>>(p);
  } else {
    if (p.rows > 0x7fffffffLL) return fail(B200_ERR_UNSUPPORTED, "row_reduce: too many rows");
    if (vec) row_reduce_kernel<Tin, Op, true, true><<<(unsigned)p.rows, threads, 0, st>>>(p);
    else row_reduce_kernel<Tin, Op, true, false><<<(unsigned)p.rows, threads, 0, st>>>(p);
  }
  return launch_status("b200_row_reduce");
}

template <typename Tin>
static int dispatch_row_reduce_op(const RowReduceParams& p, int op, bool vec, cudaStream_t st) {
  switch (op) {
    case B200_REDUCE_SUM:
    case B200_REDUCE_MEAN: return launch_row_reduce<Tin, SumOp>(p, vec, st);
    case B200_REDUCE_AMAX: return launch_row_reduce<Tin, MaxOp>(p, vec, st);
    case B200_REDUCE_AMIN: return launch_row_reduce<Tin, MinOp>(p, vec, st);
  }
  return fail(B200_ERR_INVALID, "b200_row_reduce: unknown op %d", op);
}

}  // namespace b200

using namespace b200;

extern "C" int b200_row_reduce(const void* x, void* out, int64_t rows, int64_t n, int64_t d1,
                               int64_t d2, const int64_t* x_strides, int64_t out_stride,
                               int32_t x_dtype, int32_t out_dtype, int32_t op, void* stream) {
  if (!x || !out || !x_strides) return fail(B200_ERR_INVALID, "b200_row_reduce: null argument");
  if (rows < 0 || n < 0 || d1 < 1 || d2 < 1)
    return fail(B200_ERR_INVALID, "b200_row_reduce: bad sizes rows=%lld n=%lld", (long long)rows, (long long)n);
  if (rows == 0) return B200_OK;
  if (rows % (d1 * d2) != 0) return fail(B200_ERR_INVALID, "b200_row_reduce: rows not divisible by d1*d2");
  if (n == 0 && (op == B200_REDUCE_AMAX || op == B200_REDUCE_AMIN))
    return fail(B200_ERR_INVALID, "b200_row_reduce: amax/amin of an empty row is undefined");

  RowReduceParams p;
  p.x = x; p.out = out; p.rows = rows; p.n = n;
  if (rows > 0x7fffffffLL) return fail(B200_ERR_UNSUPPORTED, "b200_row_reduce: more than 2^31-1 rows");
  p.xmap = make_row_map(x_strides, d1, d2);
  p.out_stride = out_stride; p.out_dtype = out_dtype;
  // mean of an empty row is 0 * (1/0) = NaN, as aten.mean returns
  p.post_scale = op == B200_REDUCE_MEAN ? 1.0f / (float)n : 1.0f;
  const int ib = dtype_size(x_dtype);
  const bool vec = aligned16(x) && (p.xmap.s0 * ib) % 16 == 0 && (p.xmap.s1 * ib) % 16 == 0 &&
                   (p.xmap.s2 * ib) % 16 == 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (x_dtype) {
    case B200_F32: return dispatch_row_reduce_op<float>(p, op, vec, st);
    case B200_BF16: return dispatch_row_reduce_op<__nv_bfloat16>(p, op, vec, st);
    case B200_F16: return dispatch_row_reduce_op<__half>(p, op, vec, st);
  }
  return fail(B200_ERR_INVALID, "b200_row_reduce: unknown dtype %d", x_dtype);
}
