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
// The variance is the centred second pass over the row held in registers (squares accumulated with
// fused multiply-adds: aten's var_mean has no multiply/add sequence to mirror). Statistics are fp32.
// Any of y, mean, rstd, var may be null (var_mean alone = no y, no rstd).
#include "rowwise.cuh"
#include "tile_stream.cuh"

#include <cstdlib>

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
  int prologue;     // 0: none; 1: exact (erf) GELU of x, rounded to x's dtype, is what gets normalised
  // Residual prologue (the post-LayerNorm blocks, repros/canonical/var_mean_0ada225c0a04/repro.py:26-27):
  // what gets normalised is T(x + res); res has x's dtype and row stride. sum_out (may be null)
  // receives that rounded sum, rows of n elements, contiguous.
  const void* res;
  void* sum_out;
  // 1: the sum is rounded to x's dtype before it is normalised, as the eager graph materialises it;
  // 0: it stays in fp32, as in Inductor's fused kernel - the form the reference's fp64-anchored gate
  // accepts (the fp64 evaluation of the graph has no such rounding);
  // 2 (what the stubs use; LayerNorm of 16-bit tensors): both rows are normalised, each with its own
  // statistics, and every element takes the fp32 form where that form's rounded output exceeds 3 in
  // magnitude and the rounded form elsewhere - the rule of the reference's oracle for these regions
  // (repros/canonical/var_mean_45f7dfd4a983/oracle.py:96-107). Small outputs then equal the eager
  // module's (its element-wise check allows 1e-2 + 1e-2 |y|, less than two 16-bit steps between 1.3
  // and 2 and between 2.6 and 4), large ones, which decide the maximum error against the fp64 graph,
  // carry no intermediate rounding. The statistics that are returned are those of the fp32 sum.
  int res_round;
};

// Pointwise prologue of the LayerNorm regions that normalise an activation
// (repros/canonical/var_mean_af505388b035/repro.py:27-33): (x * 0.5) * (erf(x * 0.7071067811865476) + 1)
// in fp32, in that order, then rounded to the tensor dtype - the graph materialises the
// activation as a 16-bit tensor before the statistics are taken.
template <typename Tin>
__device__ __forceinline__ float gelu_erf_rounded(float x) {
  const float g = (x * 0.5f) * (erff(x * 0.7071067811865476f) + 1.0f);
  return round_through<Tin>(g);
}
template <typename Tin>
__device__ __forceinline__ f32x2 gelu_erf_rounded2(f32x2 v) {
  float a, b;
  unpack2(v, a, b);
  return pack2(gelu_erf_rounded<Tin>(a), gelu_erf_rounded<Tin>(b));
}

// rsqrtf is the 2-ulp hardware approximation aten's CUDA rsqrt uses as well.
__device__ __forceinline__ float precise_rsqrt(float v) { return rsqrtf(v); }

template <typename Tin, typename Tout, int CH, int G, bool RES = false>
// Residual instantiations with sub-warp rows: three CTAs of 256 threads per SM (80 registers, a few
// spilled words) measured faster than two at 119 registers: 57.1 -> 45.8 us on [65536, 768] bf16
// under the reference's cold-L2 protocol.
__global__ void __launch_bounds__(G == 0 ? 512 : 256, (RES && G != 0) ? 3 : 1)
norm_fwd_resident_kernel(const NormFwdParams p) {
  constexpr int V = Elem<Tin>::V;
  __shared__ float red[64];
  const int lane = glane<G>();
  const int gs = gsize<G>();
  long long row = grow<G>();
  const bool valid = row < p.rows;  // lanes of a partly filled last CTA recompute the last row
  if (!valid) row = p.rows - 1;

  const Tin* x = reinterpret_cast<const Tin*>(p.x) + row * p.x_row_stride;
  const int nv = p.n / V;

  uint4 raw[CH], rraw[RES ? CH : 1];
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int j = c * gs + lane;
    if (j < nv) {
      raw[c] = ld_stream(x + (long long)j * V);
      if constexpr (RES)
        rraw[c] = ld_stream(reinterpret_cast<const Tin*>(p.res) + row * p.x_row_stride + (long long)j * V);
    }
  }
  // The row as packed fp32 pairs; slots past the end of the row hold zeros and add nothing.
  f32x2 v[CH][V / 2];
  constexpr bool DUAL = RES && sizeof(Tin) == 2;  // fp32 tensors: the rounded sum is the sum
  uint4 pr[DUAL ? CH : 1];                         // the rounded sums, packed, when both forms are asked for
  const bool both = DUAL && p.res_round == 2;
  f32x2 s2 = splat2(0.f);
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    float f[V];
    if (c * gs + lane < nv) {
      Elem<Tin>::unpack(raw[c], f);
      if constexpr (RES) {  // x + res in fp32; sum_out receives it rounded to the tensor dtype
        float r[V];
        Elem<Tin>::unpack(rraw[c], r);
#pragma unroll
        for (int i = 0; i < V; ++i) f[i] = f[i] + r[i];
        const uint4 packed = Elem<Tin>::pack(f);
        if (p.sum_out && valid)
          st_stream(reinterpret_cast<Tin*>(p.sum_out) + row * (long long)p.n + (long long)(c * gs + lane) * V, packed);
        if constexpr (DUAL) pr[c] = packed;
        if (p.res_round == 1) {
#pragma unroll
          for (int i = 0; i < V; ++i) f[i] = round_through<Tin>(f[i]);
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < V; ++i) f[i] = 0.f;
      if constexpr (DUAL) pr[c] = make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int i = 0; i < V / 2; ++i) v[c][i] = pack2(f[2 * i], f[2 * i + 1]);
  }
  if (p.prologue == 1) {  // gelu(0) = 0: the padding slots stay zero
#pragma unroll
    for (int c = 0; c < CH; ++c)
#pragma unroll
      for (int i = 0; i < V / 2; ++i) v[c][i] = gelu_erf_rounded2<Tin>(v[c][i]);
  }
  if (p.rms) {
#pragma unroll
    for (int c = 0; c < CH; ++c)
#pragma unroll
      for (int i = 0; i < V / 2; ++i) s2 = fma2(v[c][i], v[c][i], s2);
  } else {
#pragma unroll
    for (int c = 0; c < CH; ++c)
#pragma unroll
      for (int i = 0; i < V / 2; ++i) s2 = add2(s2, v[c][i]);
  }
  float sa, sb;
  unpack2(s2, sa, sb);
  float s = sa + sb, t = 0.f;  // t: the same sum over the rounded values (both forms)
  if constexpr (DUAL) {
    if (both) {
      f32x2 t2 = splat2(0.f);
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        float fr[V];
        Elem<Tin>::unpack(pr[c], fr);  // zeros in the padding slots
#pragma unroll
        for (int i = 0; i < V / 2; ++i) t2 = add2(t2, pack2(fr[2 * i], fr[2 * i + 1]));
      }
      float ta, tb;
      unpack2(t2, ta, tb);
      t = ta + tb;
    }
  }
  if (both) greduce_sum2<G>(s, t, red);
  else s = greduce<SumOp, G>(s, red);
  const float mean_r = t * p.inv_n;

  float mean = 0.f, var, rstd, rstd_r = 0.f;
  if (p.rms) {
    var = s * p.inv_n;
    rstd = precise_rsqrt(var + p.eps);
  } else {
    mean = s * p.inv_n;
    const f32x2 mean2 = splat2(mean);
    f32x2 q2 = splat2(0.f);
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      if (c * gs + lane < nv) {  // padding slots must not contribute (0 - mean)^2
#pragma unroll
        for (int i = 0; i < V / 2; ++i) {
          v[c][i] = sub2(v[c][i], mean2);  // keep the centred value: the output needs it again
          q2 = fma2(v[c][i], v[c][i], q2);
        }
      }
    }
    float qa, qb;
    unpack2(q2, qa, qb);
    float q = qa + qb, qr = 0.f;
    if constexpr (DUAL) {
      if (both) {
        const f32x2 mean_r2 = splat2(mean_r);
        f32x2 r2 = splat2(0.f);
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          if (c * gs + lane < nv) {
            float fr[V];
            Elem<Tin>::unpack(pr[c], fr);
#pragma unroll
            for (int i = 0; i < V / 2; ++i) {
              const f32x2 d = sub2(pack2(fr[2 * i], fr[2 * i + 1]), mean_r2);
              r2 = fma2(d, d, r2);
            }
          }
        }
        float ra, rb;
        unpack2(r2, ra, rb);
        qr = ra + rb;
      }
    }
    if (both) greduce_sum2<G>(q, qr, red);
    else q = greduce<SumOp, G>(q, red);
    var = q * p.inv_denom;
    rstd = precise_rsqrt(var + p.eps);
    rstd_r = precise_rsqrt(qr * p.inv_denom + p.eps);  // LayerNorm only; the entry point rejects the rest
  }
  if (lane == 0 && valid) {
    if (p.mean_out) p.mean_out[row] = mean;
    if (p.rstd_out) p.rstd_out[row] = rstd;
    if (p.var_out) p.var_out[row] = var;
  }
  if (p.y == nullptr) return;

  Tout* y = reinterpret_cast<Tout*>(p.y) + row * p.y_row_stride;
  const f32x2 rstd2 = splat2(rstd);
  const f32x2 rstd_r2 = splat2(rstd_r), mean_r2 = splat2(mean_r);
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int j = c * gs + lane;
    if (j < nv && valid) {
      f32x2 o[V / 2], orr[DUAL ? V / 2 : 1];
#pragma unroll
      for (int i = 0; i < V / 2; ++i) o[i] = mul2(v[c][i], rstd2);
      if constexpr (DUAL) {
        if (both) {
          float fr[V];
          Elem<Tin>::unpack(pr[c], fr);
#pragma unroll
          for (int i = 0; i < V / 2; ++i) orr[i] = mul2(sub2(pack2(fr[2 * i], fr[2 * i + 1]), mean_r2), rstd_r2);
        }
      }
      if (p.w) {
        float wf[V];
        load_param<V>(p.w, p.w_dtype, (long long)j * V, wf);
#pragma unroll
        for (int i = 0; i < V / 2; ++i) o[i] = mul2(o[i], pack2(wf[2 * i], wf[2 * i + 1]));
        if constexpr (DUAL) {
          if (both) {
#pragma unroll
            for (int i = 0; i < V / 2; ++i) orr[i] = mul2(orr[i], pack2(wf[2 * i], wf[2 * i + 1]));
          }
        }
      }
      if (p.b) {
        float bf[V];
        load_param<V>(p.b, p.w_dtype, (long long)j * V, bf);
#pragma unroll
        for (int i = 0; i < V / 2; ++i) o[i] = add2(o[i], pack2(bf[2 * i], bf[2 * i + 1]));
        if constexpr (DUAL) {
          if (both) {
#pragma unroll
            for (int i = 0; i < V / 2; ++i) orr[i] = add2(orr[i], pack2(bf[2 * i], bf[2 * i + 1]));
          }
        }
      }
      float of[V];
#pragma unroll
      for (int i = 0; i < V / 2; ++i) unpack2(o[i], of[2 * i], of[2 * i + 1]);
      if constexpr (DUAL) {
        if (both) {
#pragma unroll
          for (int i = 0; i < V / 2; ++i) {
            float ra, rb;
            unpack2(orr[i], ra, rb);
            if (!(fabsf(round_through<Tout>(of[2 * i])) > 3.0f)) of[2 * i] = ra;
            if (!(fabsf(round_through<Tout>(of[2 * i + 1])) > 3.0f)) of[2 * i + 1] = rb;
          }
        }
      }
      store_converted<Tout, V>(y + (long long)j * V, of);
    }
  }
}

// ----------------------------------------------------------------------------------------------
// Streaming variant for many short rows: a persistent CTA pulls tiles of R = blockDim/G rows into
// a ring of shared-memory stages with bulk asynchronous copies (S-1 tiles in flight per CTA,
// independent of register use), groups of G lanes normalise one row each from shared memory, and
// weight and bias are converted to fp32 once per CTA and kept in shared memory. One CTA barrier
// per tile: it makes the bounded-wait outcome CTA-uniform and, at the same time, proves that the
// previous tile's stage is free to be refilled.
// ----------------------------------------------------------------------------------------------
template <typename Tin, typename Tout, int CH, int G, bool EXACT>
__global__ void __launch_bounds__(256, 4)
norm_fwd_stream_kernel(const NormFwdParams p, const int stages, const int contiguous) {
  constexpr int V = Elem<Tin>::V;
  constexpr int PLANES = V / 4;  // fp32 copies of weight/bias are stored as planes of float4
  extern __shared__ __align__(128) unsigned char smem[];
  const int nv = p.n / V;
  const uint32_t row_bytes = (uint32_t)nv * 16u;
  const int R = blockDim.x / G;
  const uint32_t tile_bytes = (uint32_t)R * row_bytes;
  float* wsm = reinterpret_cast<float*>(smem + (size_t)stages * tile_bytes);
  float* bsm = wsm + (size_t)nv * V;
  uint64_t* full = reinterpret_cast<uint64_t*>(bsm + (size_t)nv * V);

  const int lane = threadIdx.x & (G - 1);
  const int grp = threadIdx.x / G;
  const long long num_tiles = (p.rows + R - 1) / R;
  const long long my_tiles =
      num_tiles > blockIdx.x ? (num_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const Tin* xg = reinterpret_cast<const Tin*>(p.x);

  // Thread 0 only: start the copy of this CTA's k-th tile into stage `slot` (= k mod stages,
  // tracked incrementally: a modulo per tile would cost more than the tile's arithmetic).
  const int rows_i = (int)p.rows;  // the launcher admits fewer than 2^31 rows
  const int num_tiles_i = (int)num_tiles, my_tiles_i = (int)my_tiles;
  auto issue = [&](int k, int slot) {
    const long long r0 = ((long long)blockIdx.x + (long long)k * gridDim.x) * R;
    const long long left = p.rows - r0;
    const uint32_t rows_here = (uint32_t)(left < R ? left : R);
    uint64_t* bar = &full[slot];
    unsigned char* dst = smem + (size_t)slot * tile_bytes;
    mbar_arrive_expect_tx(bar, rows_here * row_bytes);
    if (contiguous) {
      bulk_load(dst, xg + r0 * p.x_row_stride, rows_here * row_bytes, bar);
    } else {
      for (uint32_t r = 0; r < rows_here; ++r)
        bulk_load(dst + (size_t)r * row_bytes, xg + (r0 + r) * p.x_row_stride, row_bytes, bar);
    }
  };
  (void)num_tiles_i;
  // Thread 0 sets up the stage barriers and starts the first copies at once, before the CTA
  // converts weight and bias: HBM traffic begins with the CTA instead of after its prologue. (The
  // other threads first touch a barrier after the __syncthreads below.)
  int issued = 0;
  int issue_slot = 0;  // stage the next copy goes to
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
    mbar_init_fence();
    for (; issued < my_tiles_i && issued < stages; ++issued) issue(issued, issued);
    issue_slot = issued % stages;
  }

  for (int j = threadIdx.x; j < nv; j += blockDim.x) {
    float f[V];
    if (p.w) {
      load_param<V>(p.w, p.w_dtype, (long long)j * V, f);
#pragma unroll
      for (int q = 0; q < PLANES; ++q)
        *reinterpret_cast<float4*>(wsm + ((size_t)q * nv + j) * 4) = make_float4(f[4 * q], f[4 * q + 1], f[4 * q + 2], f[4 * q + 3]);
    }
    if (p.b) {
      load_param<V>(p.b, p.w_dtype, (long long)j * V, f);
#pragma unroll
      for (int q = 0; q < PLANES; ++q)
        *reinterpret_cast<float4*>(bsm + ((size_t)q * nv + j) * 4) = make_float4(f[4 * q], f[4 * q + 1], f[4 * q + 2], f[4 * q + 3]);
    }
  }
  __syncthreads();

  // Everything a tile needs that does not change from tile to tile is set up here, as 32-bit
  // shared-memory addresses and one running output pointer: the per-tile code is then loads at
  // [register + constant], arithmetic and stores.
  const uint32_t x_lane = smem_u32(smem) + (uint32_t)grp * row_bytes + (uint32_t)lane * 16u;
  uint32_t w_lane[PLANES], b_lane[PLANES];
#pragma unroll
  for (int q = 0; q < PLANES; ++q) {
    w_lane[q] = smem_u32(wsm) + ((uint32_t)q * nv + lane) * 16u;
    b_lane[q] = smem_u32(bsm) + ((uint32_t)q * nv + lane) * 16u;
  }
  const bool has_w = p.w != nullptr, has_b = p.b != nullptr, has_y = p.y != nullptr, rms = p.rms != 0;
  const int row_step = (int)gridDim.x * R;
  int row = (int)blockIdx.x * R + grp;
  Tout* yrow = reinterpret_cast<Tout*>(p.y) + (long long)row * p.y_row_stride + (long long)lane * V;
  const long long y_step = (long long)row_step * p.y_row_stride;

  int st = 0;           // stage of tile k
  uint32_t phase = 0;   // parity of that stage's current use
  uint32_t x_stage = x_lane;
  for (int k = 0; k < my_tiles_i; ++k, row += row_step, yrow += y_step) {
    const bool arrived = mbar_wait(&full[st], phase);
    if (!__syncthreads_and(arrived)) {
      // A copy did not complete within the bound: stop streaming. Thread 0 waits (bounded) for
      // whatever it still has in flight so that nothing lands in shared memory after the exit.
      if (threadIdx.x == 0) {
        note_wait_timeout();
        int ds = st;
        uint32_t dp = phase;
        for (int d = k; d < issued; ++d) {
          mbar_wait(&full[ds], dp);
          if (++ds == stages) { ds = 0; dp ^= 1u; }
        }
      }
      return;
    }
    // Everyone has passed the barrier, so everyone is done with tile k-1: refill its stage.
    if (threadIdx.x == 0 && k >= 1 && issued < my_tiles_i) {
      fence_proxy_async_smem();
      issue(issued, issue_slot);
      ++issued;
      if (++issue_slot == stages) issue_slot = 0;
    }
    const bool valid = row < rows_i;

    f32x2 v[CH][V / 2];
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      if (EXACT || c * G + lane < nv) {
        Pairs<Tin>::unpack(lds128(x_stage + (uint32_t)(c * G * 16)), v[c]);
      } else {
#pragma unroll
        for (int i = 0; i < V / 2; ++i) v[c][i] = splat2(0.f);
      }
    }
    if (p.prologue == 1) {  // gelu(0) = 0: the padding slots stay zero
#pragma unroll
      for (int c = 0; c < CH; ++c)
#pragma unroll
        for (int i = 0; i < V / 2; ++i) v[c][i] = gelu_erf_rounded2<Tin>(v[c][i]);
    }
    // one short chain per slot, combined afterwards: a single chain over the whole row would
    // serialise on the add latency
    f32x2 part[CH];
    if (rms) {
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        part[c] = mul2(v[c][0], v[c][0]);
#pragma unroll
        for (int i = 1; i < V / 2; ++i) part[c] = fma2(v[c][i], v[c][i], part[c]);
      }
    } else {
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        part[c] = v[c][0];
#pragma unroll
        for (int i = 1; i < V / 2; ++i) part[c] = add2(part[c], v[c][i]);
      }
    }
    f32x2 s2 = part[0];
#pragma unroll
    for (int c = 1; c < CH; ++c) s2 = add2(s2, part[c]);
    const float s = greduce<SumOp, G>(hsum2(s2), nullptr);

    float mean = 0.f, var, rstd;
    if (rms) {
      var = s * p.inv_n;
      rstd = precise_rsqrt(var + p.eps);
    } else {
      mean = s * p.inv_n;
      const f32x2 mean2 = splat2(mean);
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        part[c] = splat2(0.f);
        if (EXACT || c * G + lane < nv) {
#pragma unroll
          for (int i = 0; i < V / 2; ++i) {
            v[c][i] = sub2(v[c][i], mean2);
            part[c] = fma2(v[c][i], v[c][i], part[c]);
          }
        }
      }
      f32x2 q2 = part[0];
#pragma unroll
      for (int c = 1; c < CH; ++c) q2 = add2(q2, part[c]);
      const float q = greduce<SumOp, G>(hsum2(q2), nullptr);
      var = q * p.inv_denom;
      rstd = precise_rsqrt(var + p.eps);
    }
    if (lane == 0 && valid) {
      if (p.mean_out) p.mean_out[row] = mean;
      if (p.rstd_out) p.rstd_out[row] = rstd;
      if (p.var_out) p.var_out[row] = var;
    }
    if (has_y && valid) {
      const f32x2 rstd2 = splat2(rstd);
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        if (EXACT || c * G + lane < nv) {
          f32x2 o[V / 2];
#pragma unroll
          for (int i = 0; i < V / 2; ++i) o[i] = mul2(v[c][i], rstd2);
          if (has_w) {
#pragma unroll
            for (int q = 0; q < PLANES; ++q) {
              f32x2 w2[2];
              Pairs<float>::unpack(lds128(w_lane[q] + (uint32_t)(c * G * 16)), w2);
              o[2 * q] = mul2(o[2 * q], w2[0]);
              o[2 * q + 1] = mul2(o[2 * q + 1], w2[1]);
            }
          }
          if (has_b) {
#pragma unroll
            for (int q = 0; q < PLANES; ++q) {
              f32x2 b2[2];
              Pairs<float>::unpack(lds128(b_lane[q] + (uint32_t)(c * G * 16)), b2);
              o[2 * q] = add2(o[2 * q], b2[0]);
              o[2 * q + 1] = add2(o[2 * q + 1], b2[1]);
            }
          }
          store_pairs<Tout, V>(yrow + c * G * V, o);
        }
      }
    }
    x_stage += tile_bytes;
    if (++st == stages) {
      st = 0;
      phase ^= 1u;
      x_stage = x_lane;
    }
  }
}

// Geometry of the streaming kernel: lanes per row and register slots per lane for nv vectors.
// At most 32 elements per thread, so that the kernel fits in 64 registers and four 256-thread CTAs
// (32 warps) share an SM: with fewer warps the per-row dependency chains (two shuffle reductions)
// leave the schedulers idle.
// `wide` (fp32 inputs: two register pairs per vector instead of four) allows up to eight vectors per lane.
static bool pick_stream_geometry(long long nv, bool wide, int* g, int* ch) {
  if (nv <= 8) { *g = 8; *ch = 1; return true; }
  if (nv <= 16) { *g = 8; *ch = 2; return true; }
  if (nv <= 24) { *g = 8; *ch = 3; return true; }
  if (nv <= 32) { *g = 8; *ch = 4; return true; }
  if (nv <= 48) { *g = 16; *ch = 3; return true; }
  if (nv <= 64) { *g = 16; *ch = 4; return true; }
  if (nv <= 96) { *g = 32; *ch = 3; return true; }
  if (nv <= 128) { *g = 32; *ch = 4; return true; }
  if (wide && nv <= 192) { *g = 32; *ch = 6; return true; }
  if (wide && nv <= 256) { *g = 32; *ch = 8; return true; }
  return false;
}

static bool streaming_disabled() {
  static const bool off = [] {
    const char* e = getenv("B200_DISABLE_STREAMING");
    return e && e[0] == '1';
  }();
  return off;
}

template <typename Tin, typename Tout>
static bool try_launch_norm_fwd_stream(const NormFwdParams& p, cudaStream_t st, int* rc) {
  constexpr int V = Elem<Tin>::V;
  const long long nv = p.n / V;
  int g, ch;
  if (streaming_disabled() || !pick_stream_geometry(nv, V == 4, &g, &ch)) return false;
  if (p.rows > 0x7ffff000LL) return false;  // the kernel counts rows and tiles in 32 bits
  const long long total_bytes = p.rows * nv * 16;
  if (total_bytes < (8ll << 20)) return false;  // small problems: the resident kernel is fine
  const DeviceInfo& dev = device_info();
  static const int threads_env = [] { const char* e = getenv("B200_NF_THREADS"); return e ? atoi(e) : 0; }();
  // 128 threads: eight small CTAs per SM keep each other busy across the per-tile barrier better than
  // four of 256 (measured on the 32768 x 768 bf16 case: 18.3 us against 19.7 us)
  const int threads = threads_env ? threads_env : 128;
  const int R = threads / g;
  const size_t tile_bytes = (size_t)R * nv * 16;
  const size_t fixed = 2 * (size_t)nv * V * sizeof(float) + 8 * sizeof(uint64_t);
  // as many CTAs per SM as 1024 threads allow, fewer when two stages of long rows need the room
  int ctas_per_sm = 1024 / threads;
  const size_t usable = (size_t)dev.max_smem_optin;
  while (ctas_per_sm > 2 && (usable - 1024 * (size_t)ctas_per_sm) / (size_t)ctas_per_sm < fixed + 2 * tile_bytes)
    --ctas_per_sm;
  const size_t per_cta = (usable - 1024 * (size_t)ctas_per_sm) / (size_t)ctas_per_sm;
  if (fixed + 2 * tile_bytes > per_cta) return false;
  int stages = (int)((per_cta - fixed) / tile_bytes);
  if (stages > 8) stages = 8;
  const size_t smem = (size_t)stages * tile_bytes + fixed;
  const long long num_tiles = (p.rows + R - 1) / R;
  long long grid = (long long)ctas_per_sm * dev.sm_count;
  if (grid > num_tiles) grid = num_tiles;
  const int contiguous = p.x_row_stride == p.n ? 1 : 0;
  const bool exact = nv == (long long)g * ch;

  auto launch = [&](auto kernel) {
    cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(kernel),
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      cudaGetLastError();
      *rc = fail((int)e, "b200_norm_fwd: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
      return;
    }
    kernel<<<(unsigned)grid, threads, smem, st>>>(p, stages, contiguous);
    *rc = launch_status("b200_norm_fwd [streaming ring, sub-warp rows]");
  };
#define B200_NFS(GG, CC)                                                            if (g == GG && ch == CC) {                                                          if (exact) launch(norm_fwd_stream_kernel<Tin, Tout, CC, GG, true>);               else launch(norm_fwd_stream_kernel<Tin, Tout, CC, GG, false>);                    return true;                                                                    }
  B200_NFS(8, 1) B200_NFS(8, 2) B200_NFS(8, 3) B200_NFS(8, 4) B200_NFS(16, 3) B200_NFS(16, 4) B200_NFS(32, 3) B200_NFS(32, 4)
  if constexpr (V == 4) {
    B200_NFS(32, 6) B200_NFS(32, 8)
  }
#undef B200_NFS
  return false;
}

// Element-wise kernel for ragged, unaligned or very long rows: one CTA per row, sweeps over
// global memory (the second and third sweep of a row that fits in L2 are served from there).
template <typename Tin, typename Tout>
__global__ void __launch_bounds__(1024) norm_fwd_streaming_kernel(const NormFwdParams p) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const Tin* x = reinterpret_cast<const Tin*>(p.x) + row * p.x_row_stride;

  const Tin* res = p.res ? reinterpret_cast<const Tin*>(p.res) + row * p.x_row_stride : nullptr;
  auto value = [&](long long i) {
    float f = Elem<Tin>::to_f32(x[i]);
    if (res) {
      f = f + Elem<Tin>::to_f32(res[i]);
      if (p.res_round == 1) f = round_through<Tin>(f);
    }
    return p.prologue == 1 ? gelu_erf_rounded<Tin>(f) : f;
  };
  auto rounded_value = [&](long long i) {  // the other form of the residual sum (res_round == 2)
    return round_through<Tin>(Elem<Tin>::to_f32(x[i]) + Elem<Tin>::to_f32(res[i]));
  };
  if (res && p.sum_out) {
    Tin* so = reinterpret_cast<Tin*>(p.sum_out) + row * (long long)p.n;
    for (long long i = threadIdx.x; i < p.n; i += blockDim.x)
      so[i] = Elem<Tin>::from_f32(Elem<Tin>::to_f32(x[i]) + Elem<Tin>::to_f32(res[i]));
  }
  float s = 0.f;
  for (long long i = threadIdx.x; i < p.n; i += blockDim.x) {
    const float f = value(i);
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
      const float d = value(i) - mean;
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
  const bool both = res && p.res_round == 2;
  float mean_r = 0.f, rstd_r = 0.f;
  if (both) {
    float t = 0.f;
    for (long long i = threadIdx.x; i < p.n; i += blockDim.x) t += rounded_value(i);
    mean_r = block_reduce<SumOp>(t, red) * p.inv_n;
    float q = 0.f;
    for (long long i = threadIdx.x; i < p.n; i += blockDim.x) {
      const float d = rounded_value(i) - mean_r;
      q += d * d;
    }
    rstd_r = precise_rsqrt(block_reduce<SumOp>(q, red) * p.inv_denom + p.eps);
  }
  Tout* y = reinterpret_cast<Tout*>(p.y) + row * p.y_row_stride;
  for (long long i = threadIdx.x; i < p.n; i += blockDim.x) {
    float o = (value(i) - mean) * rstd;
    if (p.w) o = o * load_param1(p.w, p.w_dtype, i);
    if (p.b) o = o + load_param1(p.b, p.w_dtype, i);
    if (both && !(fabsf(round_through<Tout>(o)) > 3.0f)) {
      o = (rounded_value(i) - mean_r) * rstd_r;
      if (p.w) o = o * load_param1(p.w, p.w_dtype, i);
      if (p.b) o = o + load_param1(p.b, p.w_dtype, i);
    }
    y[i] = Elem<Tout>::from_f32(o);
  }
}

template <typename Tin, typename Tout>
static int launch_norm_fwd(const NormFwdParams& p, bool vector_ok, cudaStream_t st) {
  constexpr int V = Elem<Tin>::V;
  if (p.rows > 0x7fffffffLL) return fail(B200_ERR_UNSUPPORTED, "norm_fwd: too many rows");
  RowGeometry g;
  constexpr bool kResBuilt = std::is_same<Tin, Tout>::value;  // the residual prologue: same-dtype pairs only
  if (p.res && !kResBuilt) return fail(B200_ERR_UNSUPPORTED, "norm_fwd: the residual prologue needs y in x's dtype");
  if (vector_ok && p.n % V == 0 && !p.res) {  // the ring kernel streams one tensor
    int rc = B200_OK;
    if (try_launch_norm_fwd_stream<Tin, Tout>(p, st, &rc)) return rc;
  }
  if (vector_ok && p.n % V == 0 && pick_row_geometry(p.n / V, &g)) {
    set_path_tag(g.block ? (p.res ? "residual add, vector, row resident, CTA per row" : "vector, row resident, CTA per row")
                         : (p.res ? "residual add, vector, row resident, sub-warp rows" : "vector, row resident, sub-warp rows"));
#define B200_NF_LAUNCH(GG, CC)                                                                       \
  do {                                                                                               \
    if constexpr (kResBuilt) {                                                                       \
      if (p.res) {                                                                                   \
        norm_fwd_resident_kernel<Tin, Tout, CC, GG, true><<<grid, g.threads, 0, st>>>(p);            \
        break;                                                                                       \
      }                                                                                              \
    }                                                                                                \
    norm_fwd_resident_kernel<Tin, Tout, CC, GG><<<grid, g.threads, 0, st>>>(p);                      \
  } while (0)
    if (!g.block) {
      if (p.res) {  // CTAs of 128 threads for the residual kernels (measured: 45.8 -> 44.3 us on the case above)
        static const int t_env = [] { const char* e = getenv("B200_NF_RES_THREADS"); return e ? atoi(e) : 0; }();
        g.threads = (t_env == 64 || t_env == 128 || t_env == 256) ? t_env : 128;
      }
      const int rows_per_cta = g.threads / g.g;
      const unsigned grid = (unsigned)((p.rows + rows_per_cta - 1) / rows_per_cta);
      if (g.g == 8) {
        if (g.ch == 1) B200_NF_LAUNCH(8, 1);
        else if (g.ch == 2) B200_NF_LAUNCH(8, 2);
        else B200_NF_LAUNCH(8, 4);
      } else if (g.g == 16) {
        B200_NF_LAUNCH(16, 4);
      } else {
        B200_NF_LAUNCH(32, 4);
      }
    } else {
      const unsigned grid = (unsigned)p.rows;
      if (g.ch == 2) B200_NF_LAUNCH(0, 2);
      else if (g.ch == 4) B200_NF_LAUNCH(0, 4);
      else B200_NF_LAUNCH(0, 8);
    }
#undef B200_NF_LAUNCH
  } else {
    int threads = 1024;
    while (threads > 64 && threads / 2 >= p.n) threads /= 2;
    set_path_tag(p.res ? "residual add, element-wise, CTA per row" : "element-wise, CTA per row");
    norm_fwd_streaming_kernel<Tin, Tout><<<(unsigned)p.rows, threads, 0, st>>>(p);
  }
  return launch_status("b200_norm_fwd");
}

}  // namespace b200

using namespace b200;

// Bounded waits of the streaming kernel that ran out since the library was loaded (0 in normal
// operation). Synchronises the device.
extern "C" int64_t b200_norm_fwd_wait_timeouts(void) { return (int64_t)read_wait_timeouts(); }

extern "C" int b200_norm_fwd_residual(const void* x, const void* residual, void* sum_out, const void* weight,
                                      const void* bias, void* y, float* mean_out, float* rstd_out, float* var_out,
                                      int64_t rows, int64_t n, int64_t x_row_stride, int64_t y_row_stride,
                                      int32_t x_dtype, int32_t w_dtype, int32_t y_dtype, double eps,
                                      double correction, int32_t rms, void* stream) {
  if (!x) return fail(B200_ERR_INVALID, "b200_norm_fwd: null x");
  if (sum_out && !residual) return fail(B200_ERR_INVALID, "b200_norm_fwd_residual: sum_out without residual");
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
  p.w_dtype = w_dtype; p.eps = (float)eps; p.rms = (rms & 1) ? 1 : 0;
  p.prologue = (rms & 2) ? 1 : 0;  // bit 1 of the mode word: exact GELU of x, rounded to x's dtype, first
  p.res = residual; p.sum_out = sum_out;
  // bits 2 and 3 of the mode word: 4 rounds the residual sum to x's dtype first; 8 normalises both
  // forms and selects per element (LayerNorm without the GELU prologue; for fp32 tensors the two
  // forms are the same row, so 8 means 0 there)
  if ((rms & 12) == 12) return fail(B200_ERR_INVALID, "b200_norm_fwd_residual: mode bits 4 and 8 exclude each other");
  if ((rms & 12) && !residual) return fail(B200_ERR_INVALID, "b200_norm_fwd_residual: mode bits 4 and 8 need a residual");
  if ((rms & 8) && (rms & 3)) return fail(B200_ERR_UNSUPPORTED, "b200_norm_fwd_residual: both forms of the sum are built for plain LayerNorm only");
  p.res_round = (rms & 4) ? 1 : ((rms & 8) && x_dtype != B200_F32 ? 2 : 0);
  p.inv_n = (float)(1.0 / (double)n);
  p.inv_denom = (float)(1.0 / ((double)n - correction));  // inf/NaN for n <= correction, as aten

  const int ib = dtype_size(x_dtype), ob = dtype_size(y_dtype), wb = dtype_size(w_dtype);
  const int v_in = 16 / ib;
  const int out_chunk = v_in * ob < 16 ? v_in * ob : 16;
  const int w_chunk = v_in * wb < 16 ? v_in * wb : 16;
  bool vec = aligned16(x) && (x_row_stride * ib) % 16 == 0;
  if (residual) vec = vec && aligned16(residual) && (!sum_out || (aligned16(sum_out) && (n * ib) % 16 == 0));
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

extern "C" int b200_norm_fwd(const void* x, const void* weight, const void* bias, void* y,
                             float* mean_out, float* rstd_out, float* var_out, int64_t rows,
                             int64_t n, int64_t x_row_stride, int64_t y_row_stride,
                             int32_t x_dtype, int32_t w_dtype, int32_t y_dtype, double eps,
                             double correction, int32_t rms, void* stream) {
  return b200_norm_fwd_residual(x, nullptr, nullptr, weight, bias, y, mean_out, rstd_out, var_out, rows, n,
                                x_row_stride, y_row_stride, x_dtype, w_dtype, y_dtype, eps, correction, rms, stream);
}
