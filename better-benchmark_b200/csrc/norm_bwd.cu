// LayerNorm / RMSNorm backward: dx rows plus the dweight (and dbias) column reductions, in one
// pass over x and dy, with an optional head-major (B,S,H,D) -> (B,H,S,D) store of dx.
//
// Replaces the "mix-order" Triton kernels of the norm-backward repros in the reference
// (repros/canonical/sum_sum_2cd99e5eb23e/oracle.py:48-117 for RMSNorm,
// sum_sum_sum_3cac3bbf4e8f/oracle.py:100-193 for LayerNorm) and fuses the head split of
// pointwise_c0d19d490a2f/oracle.py:10-33 into the dx store.
//
// Evaluation order, as the decomposed aten graphs have it (g = dy * w):
//   RMSNorm  : dx = g*rstd + (((sum_row(g*x) * -0.5) * rstd^3) / n) * (x*2)
//              dw = sum_rows(dy * (x*rstd))
//   LayerNorm: xhat = (x-mean)*rstd
//              dx = (rstd/n) * ((g*n - sum_row(g)) - xhat*sum_row(g*xhat))
//              dw = sum_rows(dy * xhat),  db = sum_rows(dy)
//
// Structure: a persistent grid; each group of threads (a CTA for long rows, a warp for short
// ones) walks rows group, group+G, ..., keeps the next row's loads in flight while it reduces the
// current one, and accumulates its columns of dw/db in registers over all its rows. Each group
// then writes one fp32 partial row to scratch; after a grid-wide barrier (cooperative launch)
// the partial rows are summed in fp64, in a fixed order, into dw/db. No atomics: results are
// bit-reproducible. A two-launch variant (main + finalize) does the same without the barrier.
#include "norm_bwd.cuh"

#include <cstdlib>
#include <type_traits>

namespace b200 {

template <typename T, int CH, bool BLOCK, bool LN>
__global__ void __launch_bounds__(BLOCK ? 512 : 256)
norm_bwd_kernel(const NormBwdParams p) {
  constexpr int V = Elem<T>::V;
  __shared__ float2 red[2][16];
  __shared__ double fin[16 * 64];
  __shared__ int bar_ok;
  const int lane = group_lane<BLOCK>();
  const int G = group_size<BLOCK>();
  const int nv = p.n / V;
  const long long group = BLOCK ? (long long)blockIdx.x
                                : (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long group_stride = BLOCK ? (long long)gridDim.x : (long long)gridDim.x * (blockDim.x >> 5);

  float acc_w[CH][V], acc_b[LN ? CH : 1][V];
#pragma unroll
  for (int c = 0; c < CH; ++c) zero(acc_w[c]);
#pragma unroll
  for (int c = 0; c < (LN ? CH : 1); ++c) zero(acc_b[c]);

  // column offsets of this thread's slots inside a dx row (head-major aware)
  long long dx_col[CH];
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int col = (c * G + lane) * V;
    dx_col[c] = (long long)(col / p.head_dim) * p.dx_head_stride + (col % p.head_dim);
  }

  uint4 nx[CH], ny[CH];  // next row, in flight
  long long row = group;
  if (row < p.rows) {
    const T* xr = reinterpret_cast<const T*>(p.x) + row * p.x_row_stride;
    const T* yr = reinterpret_cast<const T*>(p.dy) + row * p.dy_row_stride;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int j = c * G + lane;
      if (j < nv) {
        nx[c] = ld_stream(xr + (long long)j * V);
        ny[c] = ld_stream(yr + (long long)j * V);
      }
    }
  }
  int parity = 0;
  // In block mode every thread of the CTA runs the same number of iterations (row is CTA-uniform),
  // so the barrier inside the loop is safe.
  while (row < p.rows) {
    uint4 cx[CH], cy[CH];
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      cx[c] = nx[c];
      cy[c] = ny[c];
    }
    const long long next = row + group_stride;
    if (next < p.rows) {
      const T* xr = reinterpret_cast<const T*>(p.x) + next * p.x_row_stride;
      const T* yr = reinterpret_cast<const T*>(p.dy) + next * p.dy_row_stride;
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        const int j = c * G + lane;
        if (j < nv) {
          nx[c] = ld_stream(xr + (long long)j * V);
          ny[c] = ld_stream(yr + (long long)j * V);
        }
      }
    }
    const float rstd = __ldg(p.rstd + row);
    const float mean = LN ? __ldg(p.mean + row) : 0.f;

    float xf[CH][V], gf[CH][V];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int j = c * G + lane;
      if (j < nv) {
        float dyf[V], wf[V];
        Elem<T>::unpack(cx[c], xf[c]);
        Elem<T>::unpack(cy[c], dyf);
        if (p.w) {
          load_param<V>(p.w, p.w_dtype, (long long)j * V, wf);
        } else {
#pragma unroll
          for (int i = 0; i < V; ++i) wf[i] = 1.f;
        }
#pragma unroll
        for (int i = 0; i < V; ++i) {
          if constexpr (LN) {
            xf[c][i] = (xf[c][i] - mean) * rstd;  // xhat
            gf[c][i] = dyf[i] * wf[i];
            s1 += gf[c][i];
            s2 += gf[c][i] * xf[c][i];
            acc_w[c][i] += dyf[i] * xf[c][i];
            acc_b[c][i] += dyf[i];
          } else {
            gf[c][i] = dyf[i] * wf[i];
            s2 += gf[c][i] * xf[c][i];
            acc_w[c][i] += dyf[i] * (xf[c][i] * rstd);
          }
        }
      }
    }
    // row sums
    if constexpr (BLOCK) {
      s1 = warp_reduce<SumOp>(s1);
      s2 = warp_reduce<SumOp>(s2);
      const int warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
      if ((threadIdx.x & 31) == 0) red[parity][warp] = make_float2(s1, s2);
      __syncthreads();
      s1 = 0.f;
      s2 = 0.f;
      for (int w = 0; w < nwarps; ++w) {
        const float2 t = red[parity][w];
        s1 += t.x;
        s2 += t.y;
      }
      parity ^= 1;
    } else {
      if constexpr (LN) s1 = warp_reduce<SumOp>(s1);
      s2 = warp_reduce<SumOp>(s2);
    }

    const unsigned int bi = fast_div((unsigned int)row, p.seq_div);
    const unsigned int si = (unsigned int)row - bi * (unsigned int)p.seq;
    T* dxr = reinterpret_cast<T*>(p.dx) + (long long)bi * p.dx_batch_stride + (long long)si * p.dx_seq_stride;
    float k;  // per-row coefficient
    if constexpr (LN) {
      k = rstd / p.n_f;
    } else {
      k = ((s2 * -0.5f) * (rstd * rstd * rstd)) / p.n_f;
    }
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int j = c * G + lane;
      if (j < nv) {
        float o[V];
#pragma unroll
        for (int i = 0; i < V; ++i) {
          if constexpr (LN) {
            o[i] = k * ((gf[c][i] * p.n_f - s1) - xf[c][i] * s2);
          } else {
            o[i] = gf[c][i] * rstd + k * (xf[c][i] * 2.0f);
          }
        }
        st_stream(dxr + dx_col[c], Elem<T>::pack(o));
      }
    }
    row = next;
  }

  // one partial row per group
  if (p.dw || p.db) {
    float* pw = p.partials + group * p.n;
    float* pb = p.partials + ((long long)p.groups + group) * p.n;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int j = c * G + lane;
      if (j < nv) {
        float4* dst = reinterpret_cast<float4*>(pw + (long long)j * V);
#pragma unroll
        for (int q = 0; q < V / 4; ++q)
          dst[q] = make_float4(acc_w[c][4 * q], acc_w[c][4 * q + 1], acc_w[c][4 * q + 2], acc_w[c][4 * q + 3]);
        if constexpr (LN) {
          if (p.db) {
            float4* dstb = reinterpret_cast<float4*>(pb + (long long)j * V);
#pragma unroll
            for (int q = 0; q < V / 4; ++q)
              dstb[q] = make_float4(acc_b[c][4 * q], acc_b[c][4 * q + 1], acc_b[c][4 * q + 2], acc_b[c][4 * q + 3]);
          }
        }
      }
    }
  }
  if (p.fused) {
    const bool ok = grid_barrier(p.bar, 1u, &bar_ok);
    if (ok) {
      if (p.dw) finalize_columns(p.partials, p.groups, p.n, p.dw, fin);
      if (LN && p.db) finalize_columns(p.partials + (long long)p.groups * p.n, p.groups, p.n, p.db, fin);
    }
    grid_barrier_depart(p.bar);
  }
}

// ----------------------------------------------------------------------------------------------
// Streaming variant of the CTA-per-row kernel: rows of x and dy arrive in a ring of shared-memory
// stages through bulk asynchronous copies (stages-1 rows of each in flight per CTA, whatever the
// register pressure), the weight is converted to fp32 once per CTA and kept in shared memory, and
// the arithmetic runs on packed fp32 pairs. The CTA barrier that publishes the row sums also
// proves that every thread has copied its part of the stage to registers, so the stage is
// refilled right after it.
// ----------------------------------------------------------------------------------------------
template <typename T, int CH, bool LN>
__global__ void __launch_bounds__(512, CH == 1 ? 2 : 1)
norm_bwd_stream_kernel(const NormBwdParams p, const int stages) {
  constexpr int V = Elem<T>::V;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(16) float2 red[2][16];
  __shared__ double fin[16 * 64];
  __shared__ int bar_ok;
  const int tid = threadIdx.x;
  const int T_ = blockDim.x;
  const int nv = p.n / V;
  const uint32_t row_bytes = (uint32_t)nv * 16u;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)stages * 2 * row_bytes);
  const T* xg = reinterpret_cast<const T*>(p.x);
  const T* dyg = reinterpret_cast<const T*>(p.dy);
  const long long my_rows = p.rows > blockIdx.x ? (p.rows - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

  if (tid == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
    mbar_init_fence();
  }
  __syncthreads();

  auto issue = [&](long long k, int slot) {  // thread 0 only; slot = k mod stages, tracked incrementally
    const long long row = (long long)blockIdx.x + k * gridDim.x;
    uint64_t* bar = &full[slot];
    unsigned char* dst = smem + (size_t)slot * 2 * row_bytes;
    mbar_arrive_expect_tx(bar, 2 * row_bytes);
    bulk_load(dst, xg + row * p.x_row_stride, row_bytes, bar);
    bulk_load(dst + row_bytes, dyg + row * p.dy_row_stride, row_bytes, bar);
  };
  long long issued = 0;
  int issue_slot = 0;
  if (tid == 0) {
    for (; issued < my_rows && issued < stages; ++issued) issue(issued, (int)issued);
    issue_slot = (int)(issued % stages);
  }

  // A thread owns the same columns in every row: its slice of the weight stays in registers.
  f32x2 wv[CH][V / 2];
  f32x2 acc_w[CH][V / 2], acc_b[LN ? CH : 1][V / 2];
  long long dx_col[CH];
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int j = c * T_ + tid;
    float wf[V];
    if (p.w && j < nv) {
      load_param<V>(p.w, p.w_dtype, (long long)j * V, wf);
    } else {
#pragma unroll
      for (int i = 0; i < V; ++i) wf[i] = 1.f;
    }
#pragma unroll
    for (int i = 0; i < V / 2; ++i) {
      wv[c][i] = pack2(wf[2 * i], wf[2 * i + 1]);
      acc_w[c][i] = splat2(0.f);
    }
    const int col = j * V;
    dx_col[c] = (long long)(col / p.head_dim) * p.dx_head_stride + (col % p.head_dim);
  }
#pragma unroll
  for (int c = 0; c < (LN ? CH : 1); ++c)
#pragma unroll
    for (int i = 0; i < V / 2; ++i) acc_b[c][i] = splat2(0.f);

  const int warp = tid >> 5, nwarps = T_ >> 5;
  const float inv_n = 1.0f / p.n_f;
  bool failed = false;
  int parity = 0;
  int st = 0;
  uint32_t phase = 0;
  for (long long k = 0; k < my_rows; ++k) {
    const long long row = (long long)blockIdx.x + k * gridDim.x;
    const bool arrived = mbar_wait(&full[st], phase);
    const unsigned char* sx = smem + (size_t)st * 2 * row_bytes;
    const unsigned char* sy = sx + row_bytes;
    const float rstd = __ldg(p.rstd + row);
    const float mean = LN ? __ldg(p.mean + row) : 0.f;
    const f32x2 rstd2 = splat2(rstd), mean2 = splat2(mean);

    f32x2 xv[CH][V / 2], gv[CH][V / 2];
    f32x2 s1 = splat2(0.f), s2 = splat2(0.f);
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int j = c * T_ + tid;
      if (j < nv) {
        float xf[V], dyf[V];
        Elem<T>::unpack(*reinterpret_cast<const uint4*>(sx + (size_t)j * 16), xf);
        Elem<T>::unpack(*reinterpret_cast<const uint4*>(sy + (size_t)j * 16), dyf);
#pragma unroll
        for (int i = 0; i < V / 2; ++i) {
          const f32x2 x2 = pack2(xf[2 * i], xf[2 * i + 1]);
          const f32x2 dy2 = pack2(dyf[2 * i], dyf[2 * i + 1]);
          const f32x2 g2 = mul2(dy2, wv[c][i]);
          gv[c][i] = g2;
          if constexpr (LN) {
            const f32x2 xhat = mul2(sub2(x2, mean2), rstd2);
            xv[c][i] = xhat;
            s1 = add2(s1, g2);
            s2 = add2(s2, mul2(g2, xhat));
            acc_w[c][i] = add2(acc_w[c][i], mul2(dy2, xhat));
            acc_b[c][i] = add2(acc_b[c][i], dy2);
          } else {
            xv[c][i] = x2;
            s2 = add2(s2, mul2(g2, x2));
            acc_w[c][i] = add2(acc_w[c][i], mul2(dy2, mul2(x2, rstd2)));
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < V / 2; ++i) xv[c][i] = gv[c][i] = splat2(0.f);
      }
    }
    float a, b, t1 = 0.f, t2;
    if constexpr (LN) {
      unpack2(s1, a, b);
      t1 = warp_reduce<SumOp>(a + b);
    }
    unpack2(s2, a, b);
    t2 = warp_reduce<SumOp>(a + b);
    if ((tid & 31) == 0) red[parity][warp] = make_float2(t1, t2);
    if (!__syncthreads_and(arrived)) {
      failed = true;
      if (tid == 0) {
        note_wait_timeout();
        atomicExch(&p.bar[1], 1u);  // lets the other CTAs leave the grid barrier at once
        int ds = st;
        uint32_t dp = phase;
        for (long long d = k; d < issued; ++d) {
          mbar_wait(&full[ds], dp);
          if (++ds == stages) { ds = 0; dp ^= 1u; }
        }
      }
      break;
    }
    if (tid == 0 && issued < my_rows) {  // every thread holds its part of this stage in registers
      fence_proxy_async_smem();
      issue(issued, issue_slot);
      ++issued;
      if (++issue_slot == stages) issue_slot = 0;
    }
    t1 = 0.f;
    t2 = 0.f;
    const float4* r4 = reinterpret_cast<const float4*>(red[parity]);
#pragma unroll
    for (int w = 0; w < 8; ++w) {  // two warps' (s1, s2) pairs per 16-byte read
      if (2 * w < nwarps) {
        const float4 t = r4[w];
        t1 += t.x;
        t2 += t.y;
        if (2 * w + 1 < nwarps) {
          t1 += t.z;
          t2 += t.w;
        }
      }
    }
    parity ^= 1;

    const unsigned int bi = fast_div((unsigned int)row, p.seq_div);
    const unsigned int si = (unsigned int)row - bi * (unsigned int)p.seq;
    T* dxr = reinterpret_cast<T*>(p.dx) + (long long)bi * p.dx_batch_stride + (long long)si * p.dx_seq_stride;
    // The division by n of the aten graph is a multiplication by 1/n here (exact for powers of
    // two, otherwise within one fp32 ulp of a per-row coefficient).
    float kf;
    if constexpr (LN) {
      kf = rstd * inv_n;
    } else {
      kf = ((t2 * -0.5f) * (rstd * rstd * rstd)) * inv_n;
    }
    const f32x2 k2 = splat2(kf), n2 = splat2(p.n_f), s1b = splat2(t1), s2b = splat2(t2), two2 = splat2(2.0f);
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int j = c * T_ + tid;
      if (j < nv) {
        float o[V];
#pragma unroll
        for (int i = 0; i < V / 2; ++i) {
          f32x2 r;
          if constexpr (LN) {
            r = mul2(k2, sub2(sub2(mul2(gv[c][i], n2), s1b), mul2(xv[c][i], s2b)));
          } else {
            r = add2(mul2(gv[c][i], rstd2), mul2(k2, mul2(xv[c][i], two2)));
          }
          unpack2(r, o[2 * i], o[2 * i + 1]);
        }
        st_stream(dxr + dx_col[c], Elem<T>::pack(o));
      }
    }
    if (++st == stages) {
      st = 0;
      phase ^= 1u;
    }
  }

  if (!failed && (p.dw || p.db)) {
    float* pw = p.partials + (long long)blockIdx.x * p.n;
    float* pb = p.partials + ((long long)p.groups + blockIdx.x) * p.n;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int j = c * T_ + tid;
      if (j < nv) {
        float f[V];
#pragma unroll
        for (int i = 0; i < V / 2; ++i) unpack2(acc_w[c][i], f[2 * i], f[2 * i + 1]);
#pragma unroll
        for (int q = 0; q < V / 4; ++q)
          reinterpret_cast<float4*>(pw + (long long)j * V)[q] = make_float4(f[4 * q], f[4 * q + 1], f[4 * q + 2], f[4 * q + 3]);
        if constexpr (LN) {
          if (p.db) {
#pragma unroll
            for (int i = 0; i < V / 2; ++i) unpack2(acc_b[c][i], f[2 * i], f[2 * i + 1]);
#pragma unroll
            for (int q = 0; q < V / 4; ++q)
              reinterpret_cast<float4*>(pb + (long long)j * V)[q] = make_float4(f[4 * q], f[4 * q + 1], f[4 * q + 2], f[4 * q + 3]);
          }
        }
      }
    }
  }
  if (p.fused) {
    const bool ok = !failed && grid_barrier(p.bar, 1u, &bar_ok);
    if (ok) {
      if (p.dw) finalize_columns(p.partials, p.groups, p.n, p.dw, fin);
      if (LN && p.db) finalize_columns(p.partials + (long long)p.groups * p.n, p.groups, p.n, p.db, fin);
    }
    grid_barrier_depart(p.bar);
  }
}

// ----------------------------------------------------------------------------------------------
// Row-tile variant of the streaming kernel for wide rows (one 16-byte vector per thread): a stage
// holds R consecutive rows of x and of dy, and everything that costs a fixed amount per row and
// thread - the wait on the stage, the warp reduction, the CTA barrier, the exchange of the warps'
// partial sums - is paid once per tile:
//   * the R (or 2R for LayerNorm) row sums of a thread are reduced across the warp together: in
//     every step a lane keeps one half of its values and hands the other half to its partner, so
//     R values need log2(R) + ... shuffles instead of 5R;
//   * the warps' partials of all rows of the tile go to shared memory as one small table
//     [value][warp] that every warp sums with one load per lane and a short butterfly.
// The second pass reads the stage again (keeping the vectors in registers costs more than it
// saves at 64 registers per thread), so a stage is refilled one tile after it was consumed.
// ----------------------------------------------------------------------------------------------
template <typename T, int R, bool LN, bool GROUPED>
__global__ void __launch_bounds__(512, 2)
norm_bwd_tile_kernel(const NormBwdParams p, const int stages, const int TG, const int groups_arg, const int wpg_inv) {
  constexpr int V = Elem<T>::V;
  constexpr int NVAL = R * (LN ? 2 : 1);  // row sums per tile: 2, 4 or 8
  constexpr int LPV = 32 / NVAL;          // lanes that share one value after the warp reduction
  constexpr int PER = NVAL / 2;           // table entries a lane sums in the second stage
  static_assert(NVAL == 2 || NVAL == 4 || NVAL == 8, "tile of 1, 2 or 4 rows");
  // Narrow rows: the CTA is GROUPS = blockDim.x / TG row groups of TG threads (TG a multiple of
  // 32, >= the vectors of a row). A tile is GROUPS * R consecutive rows, group g takes rows
  // g*R .. g*R+R-1 of it; thread t of every group owns the same columns. Wide rows: one group.
  constexpr int MAX_GROUPS = GROUPED ? 8 : 1;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(16) float red[2][MAX_GROUPS][NVAL][16];
  __shared__ int bar_ok;
  // the fp64 area of the final column sums reuses the ring once the last tile has been consumed
  // (the launcher keeps the ring at 8 KB or more)
  double* fin = reinterpret_cast<double*>(smem);
  const int lane = threadIdx.x & 31;
  // group of this thread = (warp index) / (warps per group), as a multiplication by the 16.16
  // reciprocal the launcher passes: a plain division here gets recomputed in the loop when
  // registers are short, and costs twenty instructions each time
  const int GROUPS = GROUPED ? groups_arg : 1;
  const int grp = GROUPED ? (int)((threadIdx.x >> 5) * (unsigned)wpg_inv) >> 16 : 0;
  const int tid = threadIdx.x - grp * TG;        // thread within its row group
  const int warp = tid >> 5;                     // warp within its row group
  const int TR = GROUPS * R;                     // rows per tile
  const int nv = p.n / V;
  const bool active = tid < nv;
  const uint32_t row_bytes = (uint32_t)nv * 16u;
  const uint32_t stage_bytes = 2u * TR * row_bytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)stages * stage_bytes);
  // LayerNorm keeps three register arrays per thread already (dweight, dbias, and the row data of
  // the pass at hand): its weight slice lives in shared memory as fp32, behind the barriers.
  float* wsm = reinterpret_cast<float*>(smem + (size_t)stages * stage_bytes + 8 * sizeof(uint64_t));
  const int rows = (int)p.rows;  // the launcher admits fewer than 2^31 rows
  const int tiles = (rows + TR - 1) / TR;
  const int my_tiles = tiles > (int)blockIdx.x ? (tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
  const int row_step = (int)gridDim.x * TR;

  for (int i = threadIdx.x; i < 2 * MAX_GROUPS * NVAL * 16; i += blockDim.x) (&red[0][0][0][0])[i] = 0.f;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
    mbar_init_fence();
  }
  __syncthreads();

  auto issue = [&](int k, int slot) {  // thread 0 only
    const T* xg = reinterpret_cast<const T*>(p.x);
    const T* dyg = reinterpret_cast<const T*>(p.dy);
    const long long row0 = ((long long)blockIdx.x + (long long)k * gridDim.x) * TR;
    const int nrows = p.rows - row0 < TR ? (int)(p.rows - row0) : TR;
    uint64_t* bar = &full[slot];
    unsigned char* dst = smem + (size_t)slot * stage_bytes;
    mbar_arrive_expect_tx(bar, 2u * nrows * row_bytes);
    if (p.x_row_stride == p.n && p.dy_row_stride == p.n) {
      bulk_load(dst, xg + row0 * p.n, nrows * row_bytes, bar);
      bulk_load(dst + TR * row_bytes, dyg + row0 * p.n, nrows * row_bytes, bar);
    } else {
      for (int r = 0; r < nrows; ++r) {
        bulk_load(dst + r * row_bytes, xg + (row0 + r) * p.x_row_stride, row_bytes, bar);
        bulk_load(dst + (TR + r) * row_bytes, dyg + (row0 + r) * p.dy_row_stride, row_bytes, bar);
      }
    }
  };
  int issued = 0, issue_slot = 0;
  if (threadIdx.x == 0) {
    for (; issued < my_tiles && issued < stages; ++issued) issue(issued, issued);
    issue_slot = issued % stages;
  }

  // A thread owns the same V columns in every row: weight slice and gradient sums in registers.
  f32x2 wv[LN ? 1 : V / 2], acc_w[V / 2], acc_b[LN ? V / 2 : 1];
  {
    float wf[V];
    if (p.w && active) {
      load_param<V>(p.w, p.w_dtype, (long long)tid * V, wf);
    } else {
#pragma unroll
      for (int i = 0; i < V; ++i) wf[i] = 1.f;
    }
#pragma unroll
    for (int i = 0; i < V / 2; ++i) {
      if constexpr (LN) {
        if (grp == 0 && active) {
          wsm[tid * V + 2 * i] = wf[2 * i];
          wsm[tid * V + 2 * i + 1] = wf[2 * i + 1];
        }
      } else {
        wv[i] = pack2(wf[2 * i], wf[2 * i + 1]);
      }
      acc_w[i] = splat2(0.f);
    }
#pragma unroll
    for (int i = 0; i < (LN ? V / 2 : 1); ++i) acc_b[i] = splat2(0.f);
    if constexpr (LN) {
      wv[0] = splat2(0.f);
      __syncthreads();  // the weight slice is read by every row group
    }
  }
  const f32x2* wrow = reinterpret_cast<const f32x2*>(wsm + (size_t)tid * V);
  auto weight = [&](int i) { return LN ? wrow[i] : wv[LN ? 0 : i]; };
  // dx offsets fit 32 bits (checked by the launcher): one 64-bit address per store.
  const int col = tid * V;
  const uint32_t dx_col = active ? (uint32_t)(col / p.head_dim) * (uint32_t)p.dx_head_stride + (uint32_t)(col % p.head_dim) : 0u;
  const bool one_batch_per_tile = p.seq % R == 0;  // tiles start at multiples of R
  T* const dx_base = reinterpret_cast<T*>(p.dx);
  const float inv_n = 1.0f / p.n_f;
  bool failed = false;
  int parity = 0, st = 0;
  uint32_t phase = 0;
  int row0 = (int)blockIdx.x * TR + grp * R;  // first row of this group in the current tile

  for (int k = 0; k < my_tiles; ++k, row0 += row_step) {
    const int nrows = rows - row0 < R ? (rows - row0 > 0 ? rows - row0 : 0) : R;
    float rstd[R], mean[LN ? R : 1];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      rstd[r] = r < nrows ? __ldg(p.rstd + row0 + r) : 0.f;
      if constexpr (LN) mean[r] = r < nrows ? __ldg(p.mean + row0 + r) : 0.f;
    }
    const bool arrived = mbar_wait(&full[st], phase);
    const unsigned char* sx = smem + (size_t)st * stage_bytes + (size_t)(grp * R) * row_bytes + (size_t)tid * 16;
    const unsigned char* sy = sx + (size_t)TR * row_bytes;
    const bool whole = active && nrows == R;  // uniform per warp except in the last warp of a ragged row

    // Pass 1: the row sums of this thread's columns.
    float vals[NVAL];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      f32x2 s1 = splat2(0.f), s2 = splat2(0.f);
      if (whole || (active && r < nrows)) {
        f32x2 x2[V / 2], dy2[V / 2];
        Pairs<T>::unpack(*reinterpret_cast<const uint4*>(sx + (size_t)r * row_bytes), x2);
        Pairs<T>::unpack(*reinterpret_cast<const uint4*>(sy + (size_t)r * row_bytes), dy2);
#pragma unroll
        for (int i = 0; i < V / 2; ++i) {
          const f32x2 g2 = mul2(dy2[i], weight(i));
          if constexpr (LN) {
            s1 = add2(s1, g2);
            s2 = add2(s2, mul2(g2, mul2(sub2(x2[i], splat2(mean[r])), splat2(rstd[r]))));
          } else {
            s2 = add2(s2, mul2(g2, x2[i]));
          }
        }
      }
      vals[LN ? 2 * r + 1 : r] = hsum2(s2);
      if constexpr (LN) vals[2 * r] = hsum2(s1);
    }
    const float mine = warp_reduce_multi<NVAL>(vals, lane);
    if ((lane & (LPV - 1)) == 0) red[parity][grp][lane / LPV][warp] = mine;

    if (!__syncthreads_and(arrived)) {
      failed = true;
      if (threadIdx.x == 0) {
        note_wait_timeout();
        atomicExch(&p.bar[1], 1u);  // lets the other CTAs leave the grid barrier at once
        int ds = st;
        uint32_t dp = phase;
        for (int d = k; d < issued; ++d) {
          mbar_wait(&full[ds], dp);
          if (++ds == stages) { ds = 0; dp ^= 1u; }
        }
      }
      break;
    }
    // The second pass reads this stage again; what the barrier proves is that the PREVIOUS tile's
    // stage has been read to the end by every thread: that one is refilled.
    if (threadIdx.x == 0 && k >= 1 && issued < my_tiles) {
      fence_proxy_async_smem();
      issue(issued, issue_slot);
      ++issued;
      if (++issue_slot == stages) issue_slot = 0;
    }

    // Second stage of the reduction: lane l sums PER consecutive entries of the [value][warp]
    // table, a butterfly over the LPV lanes of a value finishes it.
    float part;
    {
      const float* tp = &red[parity][grp][0][0] + lane * PER;
      if constexpr (PER == 1) {
        part = tp[0];
      } else if constexpr (PER == 2) {
        const float2 t = *reinterpret_cast<const float2*>(tp);
        part = t.x + t.y;
      } else {
        const float4 t = *reinterpret_cast<const float4*>(tp);
        part = (t.x + t.y) + (t.z + t.w);
      }
#pragma unroll
      for (int off = LPV / 2; off >= 1; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
    }
    parity ^= 1;

    // Pass 2: dx and the gradient sums.
    uint32_t off0 = 0;
    if (one_batch_per_tile) {
      const unsigned int bi = fast_div((unsigned int)row0, p.seq_div);
      const unsigned int si = (unsigned int)row0 - bi * (unsigned int)p.seq;
      off0 = bi * (uint32_t)p.dx_batch_stride + si * (uint32_t)p.dx_seq_stride + dx_col;
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const float t2 = __shfl_sync(0xffffffffu, part, (LN ? 2 * r + 1 : r) * LPV);
      const float t1 = LN ? __shfl_sync(0xffffffffu, part, (2 * r) * LPV) : 0.f;
      if (whole || (active && r < nrows)) {
        uint32_t off;
        if (one_batch_per_tile) {
          off = off0 + (uint32_t)r * (uint32_t)p.dx_seq_stride;
        } else {
          const unsigned int row = (unsigned int)(row0 + r);
          const unsigned int bi = fast_div(row, p.seq_div);
          const unsigned int si = row - bi * (unsigned int)p.seq;
          off = bi * (uint32_t)p.dx_batch_stride + si * (uint32_t)p.dx_seq_stride + dx_col;
        }
        f32x2 x2[V / 2], dy2[V / 2], o2[V / 2];
        Pairs<T>::unpack(*reinterpret_cast<const uint4*>(sx + (size_t)r * row_bytes), x2);
        Pairs<T>::unpack(*reinterpret_cast<const uint4*>(sy + (size_t)r * row_bytes), dy2);
        const f32x2 rstd2 = splat2(rstd[r]);
        if constexpr (LN) {
          // The division by n of the aten graph is a multiplication by 1/n here (exact for
          // powers of two, otherwise within one fp32 ulp of a per-row coefficient).
          const f32x2 k2 = splat2(rstd[r] * inv_n), n2 = splat2(p.n_f), s1b = splat2(t1), s2b = splat2(t2);
          const f32x2 mean2 = splat2(mean[r]);
#pragma unroll
          for (int i = 0; i < V / 2; ++i) {
            const f32x2 g2 = mul2(dy2[i], weight(i));
            const f32x2 xhat = mul2(sub2(x2[i], mean2), rstd2);
            acc_w[i] = add2(acc_w[i], mul2(dy2[i], xhat));
            acc_b[i] = add2(acc_b[i], dy2[i]);
            o2[i] = mul2(k2, sub2(sub2(mul2(g2, n2), s1b), mul2(xhat, s2b)));
          }
        } else {
          // dx = g*rstd + k*(x*2), k = (sum * -0.5) * rstd^3 / n; the doubling is exact, so it is
          // folded into the coefficient.
          const float kf = ((t2 * -0.5f) * (rstd[r] * rstd[r] * rstd[r])) * inv_n;
          const f32x2 k2 = splat2(kf * 2.0f);
#pragma unroll
          for (int i = 0; i < V / 2; ++i) {
            const f32x2 g2 = mul2(dy2[i], weight(i));
            acc_w[i] = add2(acc_w[i], mul2(dy2[i], mul2(x2[i], rstd2)));
            o2[i] = add2(mul2(g2, rstd2), mul2(k2, x2[i]));
          }
        }
        st_stream(dx_base + off, Pairs<T>::pack(o2));
      }
    }
    if (++st == stages) {
      st = 0;
      phase ^= 1u;
    }
  }

  // Per-CTA partial rows: the row groups are folded in a fixed order through the ring (free now).
  if (!failed && (p.dw || p.db)) {
    __syncthreads();  // every group is done with its last tile
    float* fold_w = reinterpret_cast<float*>(smem);             // [GROUPS][n]
    float* fold_b = fold_w + (size_t)GROUPS * p.n;              // [GROUPS][n]
    if (active) {
#pragma unroll
      for (int i = 0; i < V / 2; ++i) {
        unpack2(acc_w[i], fold_w[(size_t)grp * p.n + tid * V + 2 * i], fold_w[(size_t)grp * p.n + tid * V + 2 * i + 1]);
        if constexpr (LN) unpack2(acc_b[i], fold_b[(size_t)grp * p.n + tid * V + 2 * i],
                                  fold_b[(size_t)grp * p.n + tid * V + 2 * i + 1]);
      }
    }
    __syncthreads();
    float* pw = p.partials + (long long)blockIdx.x * p.n;
    float* pb = p.partials + ((long long)p.groups + blockIdx.x) * p.n;
    for (int c = threadIdx.x; c < p.n; c += blockDim.x) {
      float a = fold_w[c];
      for (int g = 1; g < GROUPS; ++g) a += fold_w[(size_t)g * p.n + c];
      pw[c] = a;
      if constexpr (LN) {
        if (p.db) {
          float b = fold_b[c];
          for (int g = 1; g < GROUPS; ++g) b += fold_b[(size_t)g * p.n + c];
          pb[c] = b;
        }
      }
    }
  }
  if (p.fused) {
    bool ok = !failed && grid_barrier(p.bar, 1u, &bar_ok);
    const int chunks = (p.n + 63) / 64;
    const int slices = (int)gridDim.x / chunks;
    if (ok && p.level2 != nullptr && slices >= 2) {
      double* l2w = p.level2;
      double* l2b = p.level2 + (long long)slices * p.n;
      if (p.dw) finalize_level1(p.partials, p.groups, p.n, l2w, slices, fin);
      if (LN && p.db) finalize_level1(p.partials + (long long)p.groups * p.n, p.groups, p.n, l2b, slices, fin);
      ok = grid_barrier(p.bar, 2u, &bar_ok);
      if (ok) {
        if (p.dw) finalize_level2(l2w, slices, p.n, p.dw);
        if (LN && p.db) finalize_level2(l2b, slices, p.n, p.db);
      }
    } else if (ok) {
      if (p.dw) finalize_columns(p.partials, p.groups, p.n, p.dw, fin);
      if (LN && p.db) finalize_columns(p.partials + (long long)p.groups * p.n, p.groups, p.n, p.db, fin);
    }
    grid_barrier_depart(p.bar);
  }
}

__global__ void __launch_bounds__(512) norm_bwd_finalize_kernel(const NormBwdParams p) {
  __shared__ double fin[16 * 64];
  if (p.dw) finalize_columns(p.partials, p.groups, p.n, p.dw, fin);
  if (p.db) finalize_columns(p.partials + (long long)p.groups * p.n, p.groups, p.n, p.db, fin);
}

// Element-wise kernels for rows the vector path cannot take (ragged n, unaligned pointers, a head
// size that is not a multiple of the vector length). Correct for every layout, not tuned.
template <typename T, bool LN>
__global__ void __launch_bounds__(256) norm_bwd_rows_general_kernel(const NormBwdParams p) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const T* x = reinterpret_cast<const T*>(p.x) + row * p.x_row_stride;
  const T* dy = reinterpret_cast<const T*>(p.dy) + row * p.dy_row_stride;
  const float rstd = p.rstd[row];
  const float mean = LN ? p.mean[row] : 0.f;
  float s1 = 0.f, s2 = 0.f;
  for (int i = threadIdx.x; i < p.n; i += blockDim.x) {
    const float w = p.w ? load_param1(p.w, p.w_dtype, i) : 1.f;
    const float g = Elem<T>::to_f32(dy[(long long)i * p.dy_elem_stride]) * w;
    const float xv = Elem<T>::to_f32(x[i]);
    if (LN) {
      const float xhat = (xv - mean) * rstd;
      s1 += g;
      s2 += g * xhat;
    } else {
      s2 += g * xv;
    }
  }
  s1 = block_reduce<SumOp>(s1, red);
  s2 = block_reduce<SumOp>(s2, red);
  T* dxr = reinterpret_cast<T*>(p.dx) + (row / p.seq) * p.dx_batch_stride + (row % p.seq) * p.dx_seq_stride;
  const float k = LN ? rstd / p.n_f : ((s2 * -0.5f) * (rstd * rstd * rstd)) / p.n_f;
  for (int i = threadIdx.x; i < p.n; i += blockDim.x) {
    const float w = p.w ? load_param1(p.w, p.w_dtype, i) : 1.f;
    const float g = Elem<T>::to_f32(dy[(long long)i * p.dy_elem_stride]) * w;
    const float xv = Elem<T>::to_f32(x[i]);
    float o;
    if (LN) {
      const float xhat = (xv - mean) * rstd;
      o = k * ((g * p.n_f - s1) - xhat * s2);
    } else {
      o = g * rstd + k * (xv * 2.0f);
    }
    dxr[(long long)(i / p.head_dim) * p.dx_head_stride + (i % p.head_dim)] = Elem<T>::from_f32(o);
  }
}

// One thread per column, rows split over blockIdx.y; partial rows go to scratch like the fast path.
template <typename T, bool LN>
__global__ void __launch_bounds__(128) norm_bwd_cols_general_kernel(const NormBwdParams p) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= p.n) return;
  const long long per = (p.rows + gridDim.y - 1) / gridDim.y;
  const long long r0 = (long long)blockIdx.y * per;
  const long long r1 = r0 + per < p.rows ? r0 + per : p.rows;
  float aw = 0.f, ab = 0.f;
  for (long long r = r0; r < r1; ++r) {
    const float xv = Elem<T>::to_f32(reinterpret_cast<const T*>(p.x)[r * p.x_row_stride + col]);
    const float dyv = Elem<T>::to_f32(reinterpret_cast<const T*>(p.dy)[r * p.dy_row_stride + (long long)col * p.dy_elem_stride]);
    const float rstd = p.rstd[r];
    if (LN) {
      aw += dyv * ((xv - p.mean[r]) * rstd);
      ab += dyv;
    } else {
      aw += dyv * (xv * rstd);
    }
  }
  p.partials[(long long)blockIdx.y * p.n + col] = aw;
  if (LN) p.partials[((long long)p.groups + blockIdx.y) * p.n + col] = ab;
}

static bool streaming_disabled() {
  static const bool off = [] {
    const char* e = getenv("B200_DISABLE_STREAMING");
    return e && e[0] == '1';
  }();
  return off;
}

// B200_NORM_BWD_TILE_ROWS=1|2 caps the rows per tile of the row-tile kernel (1: one row per
// barrier, the earlier kernel); for measurements.
static int tile_rows_override() {
  static const int v = [] {
    const char* e = getenv("B200_NORM_BWD_TILE_ROWS");
    return e ? atoi(e) : 0;
  }();
  return v;
}

// CTA-per-row streaming launch; returns false when the shape does not fit (caller falls back).
template <typename T, int CH, bool LN>
static bool try_launch_norm_bwd_stream(NormBwdParams p, int threads, size_t scratch_bytes, bool cooperative,
                                       cudaStream_t st, int* rc) {
  constexpr int V = Elem<T>::V;
  if (streaming_disabled() || p.rows < 1024) return false;
  const DeviceInfo& dev = device_info();
  const size_t row_bytes = (size_t)(p.n / V) * 16;
  const size_t static_bytes = 10 * 1024;  // red + fin + flags
  const size_t per_cta = ((size_t)dev.max_smem_optin - 2048) / 2;  // aim at two CTAs per SM
  const size_t fixed = 8 * sizeof(uint64_t);
  if (per_cta < static_bytes + fixed + 2 * 2 * row_bytes) return false;
  int stages = (int)((per_cta - static_bytes - fixed) / (2 * row_bytes));
  if (stages > 8) stages = 8;
  const size_t smem = (size_t)stages * 2 * row_bytes + fixed;
  auto kernel = norm_bwd_stream_kernel<T, CH, LN>;
  cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(kernel),
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  const int per_sm = cached_occupancy(reinterpret_cast<const void*>(kernel), threads, smem);
  long long grid = (long long)per_sm * dev.sm_count;
  if (grid > p.rows) grid = p.rows;
  if (p.dw || p.db) {
    const long long plane = (long long)p.n * sizeof(float);
    const long long max_groups = ((long long)scratch_bytes - 256) / (2 * plane);
    if (max_groups < 1) return false;
    if (grid > max_groups) grid = max_groups;
  }
  p.groups = (int)grid;
  p.fused = cooperative ? 1 : 0;
  if (cooperative) {
    int stages_arg = stages;
    void* args[] = {&p, &stages_arg};
    e = cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), dim3((unsigned)grid), dim3(threads),
                                    args, smem, st);
    if (e != cudaSuccess) {
      cudaGetLastError();
      *rc = fail((int)e, "b200_norm_bwd: cooperative launch failed: %s", cudaGetErrorString(e));
      return true;
    }
    note_launch("b200_norm_bwd [streaming, CTA per row, fused finalize]");
    *rc = B200_OK;
    return true;
  }
  kernel<<<(unsigned)grid, threads, smem, st>>>(p, stages);
  *rc = launch_status("b200_norm_bwd (streaming)");
  if (*rc == B200_OK && (p.dw || p.db)) {
    norm_bwd_finalize_kernel<<<(p.n + 63) / 64, 512, 0, st>>>(p);
    *rc = launch_status("b200_norm_bwd finalize");
  }
  return true;
}

// Row-tile streaming launch (one vector per thread); returns false when the shape does not fit.
template <typename T, int R, bool LN>
static bool try_launch_norm_bwd_tile(NormBwdParams p, int threads, size_t scratch_bytes, bool cooperative,
                                     cudaStream_t st, int* rc, int want_groups = 0) {
  constexpr int V = Elem<T>::V;
  if (streaming_disabled() || p.rows < 1024 || threads > 512) return false;
  {  // the kernel addresses dx with 32-bit element offsets
    const long long last = (p.rows / p.seq) * p.dx_batch_stride + (long long)(p.seq - 1) * p.dx_seq_stride +
                           (long long)(p.n / p.head_dim - 1) * p.dx_head_stride + p.head_dim;
    if (last >= 0x7fffffffLL || p.dx_batch_stride < 0 || p.dx_seq_stride < 0 || p.dx_head_stride < 0) return false;
  }
  const DeviceInfo& dev = device_info();
  // Narrow rows: several row groups of `threads` threads share a CTA of up to 512 threads, so that
  // there are still only two partial rows per SM to finalize. Wide rows: one group.
  const int tg = threads;
  int groups_per_cta = 512 / tg;
  if (groups_per_cta > 8) groups_per_cta = 8;
  static const int groups_env = [] { const char* e = getenv("B200_NORM_BWD_GROUPS"); return e ? atoi(e) : 0; }();
  if (groups_env > 0 && groups_env < groups_per_cta) groups_per_cta = groups_env;
  if (want_groups > 0 && want_groups < groups_per_cta) groups_per_cta = want_groups;
  if (groups_per_cta < 1) groups_per_cta = 1;
  threads = tg * groups_per_cta;
  const size_t stage_bytes = 2 * (size_t)groups_per_cta * (size_t)R * (size_t)(p.n / V) * 16;
  const size_t static_bytes = (groups_per_cta > 1 ? 8 : 1) * 2 * 8 * 16 * sizeof(float) + 256;  // row-sum tables + flags
  int ctas_per_sm = 1024 / threads;  // 64 registers per thread: 1024 threads per SM
  if (ctas_per_sm < 2) ctas_per_sm = 2;
  if (ctas_per_sm > 8) ctas_per_sm = 8;
  const size_t per_cta = ((size_t)dev.max_smem_optin - 1024 * (size_t)ctas_per_sm) / (size_t)ctas_per_sm;
  const size_t fixed = 8 * sizeof(uint64_t) + (LN ? (size_t)p.n * sizeof(float) : 0);  // barriers (+ fp32 weight)
  const int min_stages = groups_per_cta > 1 ? 2 : 3;
  if (per_cta < static_bytes + fixed + (size_t)min_stages * stage_bytes) return false;
  int stages = (int)((per_cta - static_bytes - fixed) / stage_bytes);
  if (stages > 8) stages = 8;
  // the ring doubles as the fold area [2][groups][n] fp32 and as the fp64 area of the finalize
  if ((size_t)stages * stage_bytes < 16 * 64 * sizeof(double) ||
      (size_t)stages * stage_bytes < 2 * (size_t)groups_per_cta * p.n * sizeof(float)) return false;
  const size_t smem = (size_t)stages * stage_bytes + fixed;
  auto kernel = groups_per_cta > 1 ? norm_bwd_tile_kernel<T, R, LN, true> : norm_bwd_tile_kernel<T, R, LN, false>;
  cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(kernel),
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  const int per_sm = cached_occupancy(reinterpret_cast<const void*>(kernel), threads, smem);
  long long grid = (long long)per_sm * dev.sm_count;
  const long long tiles = (p.rows + (long long)R * groups_per_cta - 1) / ((long long)R * groups_per_cta);
  if (grid > tiles) grid = tiles;
  if (p.dw || p.db) {
    const long long plane = (long long)p.n * sizeof(float);
    const long long max_groups = ((long long)scratch_bytes - 256) / (2 * plane);
    if (max_groups < 1) return false;
    if (grid > max_groups) grid = max_groups;
  }
  p.groups = (int)grid;
  p.fused = cooperative ? 1 : 0;
  p.level2 = nullptr;
  if (cooperative && (p.dw || p.db)) {  // room for the second level of the finalize behind the partial planes?
    const long long chunks = (p.n + 63) / 64;
    const long long slices = grid / chunks;
    const long long planes = 256 + 2LL * grid * p.n * (long long)sizeof(float);
    const long long need = (planes + 7) / 8 * 8 + 2LL * slices * p.n * (long long)sizeof(double);
    if (slices >= 2 && (long long)scratch_bytes >= need)
      p.level2 = reinterpret_cast<double*>(reinterpret_cast<char*>(p.bar) + (planes + 7) / 8 * 8);
  }
  int tg_arg = tg, groups_arg = groups_per_cta, wpg_inv_arg = (65536 + tg / 32 - 1) / (tg / 32);
  if (cooperative) {
    int stages_arg = stages;
    void* args[] = {&p, &stages_arg, &tg_arg, &groups_arg, &wpg_inv_arg};
    e = cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), dim3((unsigned)grid), dim3(threads),
                                    args, smem, st);
    if (e != cudaSuccess) {
      cudaGetLastError();
      *rc = fail((int)e, "b200_norm_bwd: cooperative launch failed: %s", cudaGetErrorString(e));
      return true;
    }
    note_launch(groups_per_cta > 1 ? "b200_norm_bwd [row tiles, row groups, fused finalize]" : "b200_norm_bwd [row tiles, fused finalize]");
    *rc = B200_OK;
    return true;
  }
  kernel<<<(unsigned)grid, threads, smem, st>>>(p, stages, tg_arg, groups_arg, wpg_inv_arg);
  *rc = launch_status("b200_norm_bwd (row tiles)");
  if (*rc == B200_OK && (p.dw || p.db)) {
    norm_bwd_finalize_kernel<<<(p.n + 63) / 64, 512, 0, st>>>(p);
    *rc = launch_status("b200_norm_bwd finalize");
  }
  return true;
}

template <typename T, int CH, bool BLOCK, bool LN>
static int launch_norm_bwd_fast(NormBwdParams p, int threads, size_t scratch_bytes, bool cooperative,
                                cudaStream_t st) {
  auto kernel = norm_bwd_kernel<T, CH, BLOCK, LN>;
  const int sms = device_info().sm_count;
  const int per_sm = cached_occupancy(reinterpret_cast<const void*>(kernel), threads);
  long long grid = (long long)per_sm * sms;
  const int groups_per_cta = BLOCK ? 1 : threads / 32;
  const long long max_useful = (p.rows + groups_per_cta - 1) / groups_per_cta;
  if (grid > max_useful) grid = max_useful;
  // scratch: 256 bytes of barrier words, then two planes of [groups][n] floats
  if (p.dw || p.db) {
    const long long plane = (long long)p.n * sizeof(float);
    const long long max_groups = ((long long)scratch_bytes - 256) / (2 * plane);
    if (max_groups < groups_per_cta)
      return fail(B200_ERR_WORKSPACE, "b200_norm_bwd: scratch of %zu bytes is too small (need >= %lld)",
                  scratch_bytes, 256 + 2 * plane * groups_per_cta);
    if (grid * groups_per_cta > max_groups) grid = max_groups / groups_per_cta;
  }
  p.groups = (int)(grid * groups_per_cta);
  p.fused = cooperative ? 1 : 0;
  if (cooperative) {
    void* args[] = {&p};
    cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), dim3((unsigned)grid),
                                                dim3(threads), args, 0, st);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail((int)e, "b200_norm_bwd: cooperative launch failed: %s", cudaGetErrorString(e));
    }
    note_launch(BLOCK ? "b200_norm_bwd [registers, CTA per row, fused finalize]" : "b200_norm_bwd [registers, warp per row, fused finalize]");
    return B200_OK;
  }
  kernel<<<(unsigned)grid, threads, 0, st>>>(p);
  int rc = launch_status("b200_norm_bwd");
  if (rc != B200_OK) return rc;
  if (p.dw || p.db) {
    const int chunks = (p.n + 63) / 64;
    norm_bwd_finalize_kernel<<<chunks, 512, 0, st>>>(p);
    rc = launch_status("b200_norm_bwd finalize");
  }
  return rc;
}

template <typename T, bool LN>
static int launch_norm_bwd(NormBwdParams p, bool vector_ok, size_t scratch_bytes, bool cooperative,
                           cudaStream_t st) {
  constexpr int V = Elem<T>::V;
  if (p.rows > 0x7fffffffLL) return fail(B200_ERR_UNSUPPORTED, "norm_bwd: too many rows");
  const long long nv = p.n / V;
  if (vector_ok && p.n % V == 0 && p.head_dim % V == 0 && nv <= 2048) {
    {  // rows of 33..256 vectors: warp per row, per-warp copy rings (norm_bwd_warp.cu)
      int rc = B200_OK;
      if (try_launch_norm_bwd_warp<T, LN>(p, scratch_bytes, cooperative, st, &rc)) return rc;
    }
  }
  // a broadcast scalar dy is read by the warp-per-row kernel above and by the element-wise kernels
  // below; the other vector kernels stream dy rows
  if (p.dy_elem_stride != 0 && vector_ok && p.n % V == 0 && p.head_dim % V == 0 && nv <= 2048) {
    if (nv <= 128) {
      if (nv > 32 && tile_rows_override() != 1) {  // column-owner CTAs of 2..4 warps, several rows per barrier
        int rc = B200_OK;
        const int narrow = (int)((nv + 31) / 32 * 32);
        // four rows per group and barrier when two stages of that fit (with fewer groups if need
        // be: more work per barrier beats more groups), else two rows
        for (int g = 512 / narrow; g >= 3; --g)
          if (try_launch_norm_bwd_tile<T, 4, LN>(p, narrow, scratch_bytes, cooperative, st, &rc, g)) return rc;
        if (try_launch_norm_bwd_tile<T, 2, LN>(p, narrow, scratch_bytes, cooperative, st, &rc)) return rc;
      }
      if (nv <= 32) return launch_norm_bwd_fast<T, 1, false, LN>(p, 256, scratch_bytes, cooperative, st);
      if (nv <= 64) return launch_norm_bwd_fast<T, 2, false, LN>(p, 256, scratch_bytes, cooperative, st);
      return launch_norm_bwd_fast<T, 4, false, LN>(p, 256, scratch_bytes, cooperative, st);
    }
    int rc = B200_OK;
    if (nv <= 512) {
      // streaming: one vector per thread (many warps, few registers, the weight slice resident)
      const int wide = (int)((nv + 31) / 32 * 32);
      if (tile_rows_override() != 1) {
        if (tile_rows_override() != 2 &&
            try_launch_norm_bwd_tile<T, 4, LN>(p, wide, scratch_bytes, cooperative, st, &rc)) return rc;
        if (try_launch_norm_bwd_tile<T, 2, LN>(p, wide, scratch_bytes, cooperative, st, &rc)) return rc;
      }
      if (try_launch_norm_bwd_stream<T, 1, LN>(p, wide, scratch_bytes, cooperative, st, &rc)) return rc;
      int threads = (int)((nv + 1) / 2);
      threads = (threads + 31) / 32 * 32;
      return launch_norm_bwd_fast<T, 2, true, LN>(p, threads, scratch_bytes, cooperative, st);
    }
    if (nv <= 1024) {
      int threads = (int)((nv + 1) / 2);
      threads = (threads + 31) / 32 * 32;
      if (try_launch_norm_bwd_stream<T, 2, LN>(p, threads, scratch_bytes, cooperative, st, &rc)) return rc;
    }
    int threads = (int)((nv + 3) / 4);
    threads = (threads + 31) / 32 * 32;
    if (try_launch_norm_bwd_stream<T, 4, LN>(p, threads, scratch_bytes, cooperative, st, &rc)) return rc;
    return launch_norm_bwd_fast<T, 4, true, LN>(p, threads, scratch_bytes, cooperative, st);
  }
  // general path: rows kernel + column kernel + finalize
  norm_bwd_rows_general_kernel<T, LN><<<(unsigned)p.rows, 256, 0, st>>>(p);
  int rc = launch_status("b200_norm_bwd rows [element-wise]");
  if (rc != B200_OK || !(p.dw || p.db)) return rc;
  const long long plane = (long long)p.n * sizeof(float);
  long long splits = ((long long)scratch_bytes - 256) / (2 * plane);
  if (splits < 1) return fail(B200_ERR_WORKSPACE, "b200_norm_bwd: scratch too small");
  if (splits > 64) splits = 64;
  if (splits > p.rows) splits = p.rows;
  p.groups = (int)splits;
  norm_bwd_cols_general_kernel<T, LN><<<dim3((p.n + 127) / 128, (unsigned)splits), 128, 0, st>>>(p);
  rc = launch_status("b200_norm_bwd cols");
  if (rc != B200_OK) return rc;
  norm_bwd_finalize_kernel<<<(p.n + 63) / 64, 512, 0, st>>>(p);
  return launch_status("b200_norm_bwd finalize");
}

}  // namespace b200

using namespace b200;

// Bounded waits of the streaming kernel that ran out since the library was loaded (0 in normal
// operation). Synchronises the device.
extern "C" int64_t b200_norm_bwd_wait_timeouts(void) {
  return (int64_t)read_wait_timeouts() + (int64_t)norm_bwd_warp_wait_timeouts();
}

// Bytes of scratch that let every path run its largest grid for rows of n elements: the barrier
// words, two planes (dweight, dbias) of one fp32 partial row per group, and the fp64 second level
// of the fused finalize. A group is a CTA (at most eight resident per SM), except in the
// warp-per-row register kernel that takes rows of up to 256 elements, where it is a warp (64 per
// SM). The launchers shrink their grids to whatever scratch they are given, so a smaller buffer
// costs speed, never correctness.
extern "C" int64_t b200_norm_bwd_scratch_bytes(int64_t n) {
  const int64_t sms = device_info().sm_count;
  const int64_t groups = (n <= 256 ? 64 : 8) * sms;
  const int64_t planes = 2 * groups * n * (int64_t)sizeof(float);
  const int64_t level2 = 2 * groups * 64 * (int64_t)sizeof(double);
  return 256 + planes + 64 + level2;
}

extern "C" int b200_norm_bwd(const void* x, const void* dy, const void* weight, const float* mean,
                             const float* rstd, void* dx, float* dweight, float* dbias, int64_t rows,
                             int64_t n, int64_t x_row_stride, int64_t dy_row_stride, int32_t x_dtype,
                             int32_t w_dtype, int32_t rms, int64_t seq, int64_t head_dim,
                             int64_t dx_batch_stride, int64_t dx_seq_stride, int64_t dx_head_stride,
                             void* scratch, int64_t scratch_bytes, int32_t flags, void* stream) {
  if (!x || !dy || !rstd || !dx) return fail(B200_ERR_INVALID, "b200_norm_bwd: null argument");
  if (!rms && !mean) return fail(B200_ERR_INVALID, "b200_norm_bwd: LayerNorm backward needs mean");
  if (rows < 0 || n <= 0 || n > 0x7fffffffLL || seq < 1 || head_dim < 1 || n % head_dim != 0)
    return fail(B200_ERR_INVALID, "b200_norm_bwd: bad sizes rows=%lld n=%lld seq=%lld head_dim=%lld",
                (long long)rows, (long long)n, (long long)seq, (long long)head_dim);
  if ((dweight || dbias) && (!scratch || scratch_bytes < 256))
    return fail(B200_ERR_WORKSPACE, "b200_norm_bwd: dweight/dbias need a scratch buffer");
  if ((dweight || dbias) && !aligned16(scratch)) return fail(B200_ERR_ALIGNMENT, "b200_norm_bwd: scratch must be 16-byte aligned");
  if (rms && dbias) return fail(B200_ERR_INVALID, "b200_norm_bwd: RMSNorm has no bias gradient");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (rows == 0) {
    if (dweight) cudaMemsetAsync(dweight, 0, n * sizeof(float), st);
    if (dbias) cudaMemsetAsync(dbias, 0, n * sizeof(float), st);
    return launch_status("b200_norm_bwd (empty)");
  }

  NormBwdParams p;
  p.x = x; p.dy = dy; p.w = weight; p.mean = mean; p.rstd = rstd; p.dx = dx; p.dw = dweight; p.db = dbias;
  p.rows = rows; p.n = (int)n; p.x_row_stride = x_row_stride; p.dy_row_stride = dy_row_stride;
  const bool dy_scalar = (flags & 2) != 0;  // dy points at ONE element that stands for the whole tensor
  p.dy_elem_stride = dy_scalar ? 0 : 1;
  if (dy_scalar) p.dy_row_stride = 0;
  p.w_dtype = w_dtype; p.seq = (int)seq; p.head_dim = (int)head_dim;
  p.seq_div = make_fast_div(seq);
  p.dx_batch_stride = dx_batch_stride; p.dx_seq_stride = dx_seq_stride; p.dx_head_stride = dx_head_stride;
  p.n_f = (float)n;
  p.bar = reinterpret_cast<unsigned int*>(scratch);
  p.partials = scratch ? reinterpret_cast<float*>(reinterpret_cast<char*>(scratch) + 256) : nullptr;
  p.groups = 0; p.fused = 0; p.level2 = nullptr;
  const bool cooperative = (flags & 1) == 0 && (dweight || dbias);

  const int eb = dtype_size(x_dtype), wb = dtype_size(w_dtype);
  const int v = 16 / eb;
  const int w_chunk = v * wb < 16 ? v * wb : 16;
  bool vec = aligned16(x) && (dy_scalar || aligned16(dy)) && aligned16(dx) && (x_row_stride * eb) % 16 == 0 &&
             (p.dy_row_stride * eb) % 16 == 0 && (dx_batch_stride * eb) % 16 == 0 &&
             (dx_seq_stride * eb) % 16 == 0 && (dx_head_stride * eb) % 16 == 0;
  if (weight) vec = vec && reinterpret_cast<uintptr_t>(weight) % w_chunk == 0;

#define B200_NBWD_CASE(TT, DT)                                                              \
  if (x_dtype == DT)                                                                        \
    return rms ? launch_norm_bwd<TT, false>(p, vec, (size_t)scratch_bytes, cooperative, st) \
               : launch_norm_bwd<TT, true>(p, vec, (size_t)scratch_bytes, cooperative, st);
  B200_NBWD_CASE(float, B200_F32)
  B200_NBWD_CASE(__nv_bfloat16, B200_BF16)
  B200_NBWD_CASE(__half, B200_F16)
#undef B200_NBWD_CASE
  return fail(B200_ERR_INVALID, "b200_norm_bwd: unknown dtype %d", x_dtype);
}
