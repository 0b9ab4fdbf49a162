// LayerNorm / RMSNorm backward for rows of 33..256 sixteen-byte vectors (hidden sizes of about
// 300 to 1024 elements): a warp per row, every warp with its own ring of copy stages.
//
// This is the shape class of most norm-backward points of the reference's corpus
// (repros/canonical/sum_sum_sum_3cac3bbf4e8f/oracle.py:100-193 LayerNorm,
// sum_sum_2cd99e5eb23e/oracle.py:48-117 RMSNorm; hidden 512..1024). The arithmetic is that of
// norm_bwd.cu (same evaluation order as the decomposed aten graphs, see there).
//
// Structure
//   * Persistent cooperative grid of 256-thread CTAs. Warp g of the grid takes rows g, g + G, ...
//   * A stage of a warp's ring holds one row of x and one row of dy, brought in by two bulk
//     asynchronous copies that lane 0 issues; the warp waits on the stage's mbarrier. There is no
//     CTA barrier in the row loop, and the bytes in flight (stages - 1 rows per warp) do not
//     depend on the registers the arithmetic needs.
//   * Lane l owns the 16-byte vectors l, l + 32, ... of every row: its columns never change, so
//     its slice of dweight / dbias is summed in registers over all rows of the warp. LayerNorm
//     reads its weight slice from shared memory (fp32, converted once per CTA); RMSNorm keeps it
//     in registers.
//   * Two sweeps over the stage: row sums first (one batched warp reduction), then dx and the
//     gradient sums. The stage is refilled as soon as the second sweep has read it.
//   * At the end the warps of a CTA fold their sums in a fixed order through shared memory into
//     ONE fp32 partial row per CTA; after the grid barrier the partial rows are added in fp64
//     (two-level when the grid is much larger than the number of 64-column chunks). No atomics:
//     results are bit-reproducible.
// Every wait is bounded; a wait that runs out makes the warp stop, wait (bounded) for its own
// copies and raise the error word of the grid barrier, so that all CTAs leave.
#include "norm_bwd.cuh"

namespace b200 {

namespace {

constexpr int kWarps = 8;  // warps per CTA

// DYS: dy is ONE element broadcast over the whole tensor (the captured graphs of the reference's
// norm-backward directories expand a 0-dim gradient, repros/canonical/sum_sum_2cd99e5eb23e/repro.py:26);
// nothing is read for it and a stage holds the row of x only.
template <typename T, int CH, bool LN, bool DYS>
__global__ void __launch_bounds__(kWarps * 32, (LN && DYS) ? 3 : 2)
norm_bwd_warp_kernel(const NormBwdParams p, const int stages, const int ring_bytes) {
  constexpr int V = Elem<T>::V;
  constexpr int P = V / 2;  // fp32 pairs per vector
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int bar_ok;
  __shared__ int cta_failed;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nv = p.n / V;
  const uint32_t row_bytes = (uint32_t)nv * 16u;
  const uint32_t stage_bytes = (DYS ? 1u : 2u) * row_bytes;
  // layout: [kWarps][stages][x row | dy row] | pad to ring_bytes | mbarriers [kWarps][8] | fp32 weight [CH][V/2][32] pairs (LayerNorm)
  unsigned char* ring = smem + (size_t)warp * stages * stage_bytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + ring_bytes) + warp * 8;
  float* wsm = reinterpret_cast<float*>(smem + ring_bytes + kWarps * 8 * sizeof(uint64_t));
  const int rows = (int)p.rows;  // the launcher admits fewer than 2^31 rows
  const int gwarp = (int)blockIdx.x * kWarps + warp;
  const int gstep = (int)gridDim.x * kWarps;
  const int my_rows = rows > gwarp ? (rows - gwarp + gstep - 1) / gstep : 0;

  if (threadIdx.x == 0) cta_failed = 0;
  if (lane == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
  }
  mbar_init_fence();

  const T* xg = reinterpret_cast<const T*>(p.x);
  const T* dyg = reinterpret_cast<const T*>(p.dy);
  auto issue = [&](int k, int slot) {  // lane 0 only
    const long long row = (long long)gwarp + (long long)k * gstep;
    unsigned char* dst = ring + (size_t)slot * stage_bytes;
    mbar_arrive_expect_tx(&full[slot], stage_bytes);
    bulk_load(dst, xg + row * p.x_row_stride, row_bytes, &full[slot]);
    if constexpr (!DYS) bulk_load(dst + row_bytes, dyg + row * p.dy_row_stride, row_bytes, &full[slot]);
  };
  const f32x2 dy_all = splat2(DYS ? Elem<T>::to_f32(__ldg(dyg)) : 0.f);

  // weight slice: registers (RMSNorm) or shared memory (LayerNorm, which already keeps two
  // gradient sums per column in registers)
  f32x2 wv[LN ? 1 : CH][P];
  if constexpr (LN) {
    // layout [vector slot c][pair i][lane] of fp32 pairs: the 32 lanes of a warp read 32 consecutive
    // 8-byte words, one shared-memory wavefront without bank conflicts
    for (int q = threadIdx.x; q < CH * 32; q += blockDim.x) {  // q = c * 32 + lane: vector q of the row
      float wf[V];
      if (p.w && q < nv) {
        load_param<V>(p.w, p.w_dtype, (long long)q * V, wf);
      } else {
#pragma unroll
        for (int i = 0; i < V; ++i) wf[i] = 1.f;
      }
      if constexpr (DYS) {  // one dy for the whole tensor: g = dy * w does not depend on the row
        const float dyf = Elem<T>::to_f32(__ldg(dyg));
#pragma unroll
        for (int i = 0; i < V; ++i) wf[i] = __fmul_rn(dyf, wf[i]);
      }
      const int c = q >> 5, l = q & 31;
#pragma unroll
      for (int i = 0; i < P; ++i) {
        wsm[((c * P + i) * 32 + l) * 2] = wf[2 * i];
        wsm[((c * P + i) * 32 + l) * 2 + 1] = wf[2 * i + 1];
      }
    }
#pragma unroll
    for (int i = 0; i < P; ++i) wv[0][i] = splat2(0.f);
  } else {
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int j = c * 32 + lane;
      float wf[V];
      if (p.w && j < nv) {
        load_param<V>(p.w, p.w_dtype, (long long)j * V, wf);
      } else {
#pragma unroll
        for (int i = 0; i < V; ++i) wf[i] = 1.f;
      }
#pragma unroll
      for (int i = 0; i < P; ++i) wv[c][i] = pack2(wf[2 * i], wf[2 * i + 1]);
    }
  }
  __syncthreads();  // barriers initialised, weight slice in place

  // LayerNorm with a scalar dy: g = dy * w is the same in every row, and so are sum(g) and the
  // term g * n - sum(g) of dx. They are computed once: sum(g) by every warp (same order, same
  // result), the per-column term into a second table behind the first.
  float g_sum = 0.f;
  float* asm_tab = wsm + CH * 32 * V;  // [CH][P][32] fp32 pairs, the layout of wsm
  if constexpr (LN && DYS) {
    f32x2 s1 = splat2(0.f);
    const f32x2* g_lane = reinterpret_cast<const f32x2*>(wsm) + lane;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      if (c * 32 + lane < nv) {
#pragma unroll
        for (int i = 0; i < P; ++i) s1 = add2(s1, g_lane[(c * P + i) * 32]);
      }
    }
    g_sum = warp_reduce<SumOp>(hsum2(s1));
    for (int q = threadIdx.x; q < CH * 32 * P; q += blockDim.x) {  // q = (c * P + i) * 32 + lane
      asm_tab[q * 2] = __fsub_rn(__fmul_rn(wsm[q * 2], p.n_f), g_sum);
      asm_tab[q * 2 + 1] = __fsub_rn(__fmul_rn(wsm[q * 2 + 1], p.n_f), g_sum);
    }
    __syncthreads();
  }

  int issued = 0;
  if (lane == 0) {
    for (; issued < my_rows && issued < stages; ++issued) issue(issued, issued);
  }
  issued = __shfl_sync(0xffffffffu, issued, 0);

  f32x2 acc_w[CH][P], acc_b[LN ? CH : 1][P];
  uint32_t dx_col[CH];
#pragma unroll
  for (int c = 0; c < CH; ++c) {
#pragma unroll
    for (int i = 0; i < P; ++i) acc_w[c][i] = splat2(0.f);
    const int col = (c * 32 + lane) * V;
    dx_col[c] = (uint32_t)(col / p.head_dim) * (uint32_t)p.dx_head_stride + (uint32_t)(col % p.head_dim);
  }
#pragma unroll
  for (int c = 0; c < (LN ? CH : 1); ++c)
#pragma unroll
    for (int i = 0; i < P; ++i) acc_b[c][i] = splat2(0.f);

  const uint32_t ring_addr = smem_u32(ring) + (uint32_t)lane * 16u;
  const f32x2* w_lane = reinterpret_cast<const f32x2*>(wsm) + lane;
  auto weight = [&](int c, int i) -> f32x2 {
    if constexpr (LN) {
      return w_lane[(c * P + i) * 32];
    } else {
      return wv[c][i];
    }
  };
  T* const dx_base = reinterpret_cast<T*>(p.dx);
  const float inv_n = 1.0f / p.n_f;
  int slot = 0;
  uint32_t phase = 0;
  int row = gwarp;

  // the row statistics are fetched one row ahead, so that their latency is never waited for
  float rstd_next = my_rows > 0 ? __ldg(p.rstd + row) : 0.f;
  float mean_next = (LN && my_rows > 0) ? __ldg(p.mean + row) : 0.f;
  for (int k = 0; k < my_rows; ++k, row += gstep) {
    const float rstd = rstd_next, mean = mean_next;
    if (k + 1 < my_rows) {
      rstd_next = __ldg(p.rstd + row + gstep);
      if constexpr (LN) mean_next = __ldg(p.mean + row + gstep);
    }
    const bool arrived = __all_sync(0xffffffffu, mbar_wait(&full[slot], phase));
    if (!arrived) {
      if (lane == 0) {
        note_wait_timeout();
        atomicExch(&p.bar[1], 1u);  // lets the other CTAs leave the grid barrier at once
        atomicExch(&cta_failed, 1);
        int ds = slot;
        uint32_t dp = phase;
        for (int d = k; d < issued; ++d) {  // none of this warp's copies may be in flight at exit
          mbar_wait(&full[ds], dp);
          if (++ds == stages) { ds = 0; dp ^= 1u; }
        }
      }
      break;
    }
    const uint32_t sx = ring_addr + (uint32_t)slot * stage_bytes;
    const uint32_t sy = sx + row_bytes;
    const f32x2 rstd2 = splat2(rstd), mean2 = splat2(mean);

    // Sweep 1: the row sums of this lane's columns.
    f32x2 s1 = splat2(0.f), s2 = splat2(0.f);
    if constexpr (LN && DYS) {
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        if (c * 32 + lane < nv) {
          f32x2 x2[P];
          Pairs<T>::unpack(lds128(sx + c * 512), x2);
#pragma unroll
          for (int i = 0; i < P; ++i) s2 = add2(s2, mul2(weight(c, i), mul2(sub2(x2[i], mean2), rstd2)));
        }
      }
    } else {
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      if (c * 32 + lane < nv) {
        f32x2 x2[P], dy2[P];
        Pairs<T>::unpack(lds128(sx + c * 512), x2);
        if constexpr (DYS) {
#pragma unroll
          for (int i = 0; i < P; ++i) dy2[i] = dy_all;
        } else {
          Pairs<T>::unpack(lds128(sy + c * 512), dy2);
        }
#pragma unroll
        for (int i = 0; i < P; ++i) {
          const f32x2 g2 = mul2(dy2[i], weight(c, i));
          if constexpr (LN) {
            s1 = add2(s1, g2);
            s2 = add2(s2, mul2(g2, mul2(sub2(x2[i], mean2), rstd2)));
          } else {
            s2 = add2(s2, mul2(g2, x2[i]));
          }
        }
      }
    }
    }
    float t1 = 0.f, t2;
    if constexpr (LN && DYS) {
      t1 = g_sum;
      t2 = warp_reduce<SumOp>(hsum2(s2));
    } else if constexpr (LN) {
      float vals[2] = {hsum2(s1), hsum2(s2)};
      const float mine = warp_reduce_multi<2>(vals, lane);  // lanes 0..15 hold sum 1, lanes 16..31 sum 2
      t1 = __shfl_sync(0xffffffffu, mine, 0);
      t2 = __shfl_sync(0xffffffffu, mine, 16);
    } else {
      t2 = warp_reduce<SumOp>(hsum2(s2));
    }

    // Sweep 2: dx and the gradient sums.
    uint32_t off0;
    {
      const unsigned int bi = fast_div((unsigned int)row, p.seq_div);
      const unsigned int si = (unsigned int)row - bi * (unsigned int)p.seq;
      off0 = bi * (uint32_t)p.dx_batch_stride + si * (uint32_t)p.dx_seq_stride;
    }
    if constexpr (LN && DYS) {
      // dweight = dy * sum(xhat): the sum of xhat is kept, the product is taken once at the end.
      const f32x2 k2 = splat2(rstd * inv_n), s2b = splat2(t2);
      const f32x2* a_lane = reinterpret_cast<const f32x2*>(asm_tab) + lane;
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        if (c * 32 + lane < nv) {
          f32x2 x2[P], o2[P];
          Pairs<T>::unpack(lds128(sx + c * 512), x2);
#pragma unroll
          for (int i = 0; i < P; ++i) {
            const f32x2 xhat = mul2(sub2(x2[i], mean2), rstd2);
            acc_w[c][i] = add2(acc_w[c][i], xhat);
            o2[i] = mul2(k2, sub2(a_lane[(c * P + i) * 32], mul2(xhat, s2b)));
          }
          st_stream(dx_base + off0 + dx_col[c], Pairs<T>::pack(o2));
        }
      }
    } else if constexpr (LN) {
      // The division by n of the aten graph is a multiplication by 1/n here (exact for powers of
      // two, otherwise within one fp32 ulp of a per-row coefficient).
      const f32x2 k2 = splat2(rstd * inv_n), n2 = splat2(p.n_f), s1b = splat2(t1), s2b = splat2(t2);
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        if (c * 32 + lane < nv) {
          f32x2 x2[P], dy2[P], o2[P];
          Pairs<T>::unpack(lds128(sx + c * 512), x2);
          if constexpr (DYS) {
#pragma unroll
            for (int i = 0; i < P; ++i) dy2[i] = dy_all;
          } else {
            Pairs<T>::unpack(lds128(sy + c * 512), dy2);
          }
#pragma unroll
          for (int i = 0; i < P; ++i) {
            const f32x2 g2 = mul2(dy2[i], weight(c, i));
            const f32x2 xhat = mul2(sub2(x2[i], mean2), rstd2);
            acc_w[c][i] = add2(acc_w[c][i], mul2(dy2[i], xhat));
            acc_b[c][i] = add2(acc_b[c][i], dy2[i]);
            o2[i] = mul2(k2, sub2(sub2(mul2(g2, n2), s1b), mul2(xhat, s2b)));
          }
          st_stream(dx_base + off0 + dx_col[c], Pairs<T>::pack(o2));
        }
      }
    } else {
      // dx = g*rstd + k*(x*2), k = (sum * -0.5) * rstd^3 / n; the doubling is exact, so it is
      // folded into the coefficient.
      const float kf = ((t2 * -0.5f) * (rstd * rstd * rstd)) * inv_n;
      const f32x2 k2 = splat2(kf * 2.0f);
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        if (c * 32 + lane < nv) {
          f32x2 x2[P], dy2[P], o2[P];
          Pairs<T>::unpack(lds128(sx + c * 512), x2);
          if constexpr (DYS) {
#pragma unroll
            for (int i = 0; i < P; ++i) dy2[i] = dy_all;
          } else {
            Pairs<T>::unpack(lds128(sy + c * 512), dy2);
          }
#pragma unroll
          for (int i = 0; i < P; ++i) {
            const f32x2 g2 = mul2(dy2[i], weight(c, i));
            acc_w[c][i] = add2(acc_w[c][i], mul2(dy2[i], mul2(x2[i], rstd2)));
            o2[i] = add2(mul2(g2, rstd2), mul2(k2, x2[i]));
          }
          st_stream(dx_base + off0 + dx_col[c], Pairs<T>::pack(o2));
        }
      }
    }

    // every lane has read the stage: refill it with the row `stages` further on
    __syncwarp();
    if (k + stages < my_rows) {
      if (lane == 0) {
        fence_proxy_async_smem();
        issue(k + stages, slot);
      }
      ++issued;
    }
    if (++slot == stages) {
      slot = 0;
      phase ^= 1u;
    }
  }

  // One partial row per CTA: the warps are folded in a fixed order through the ring (free now).
  __syncthreads();  // every warp is done with its rows (or gave up, with no copy in flight)
  const bool any_failed = cta_failed != 0;
  if (!any_failed && (p.dw || p.db)) {
    float* fold_w = reinterpret_cast<float*>(smem);   // [kWarps][n]
    float* fold_b = fold_w + (size_t)kWarps * p.n;    // [kWarps][n]
    if constexpr (LN && DYS) {
#pragma unroll
      for (int c = 0; c < CH; ++c) {
#pragma unroll
        for (int i = 0; i < P; ++i) {
          acc_w[c][i] = mul2(acc_w[c][i], dy_all);
          acc_b[c][i] = mul2(splat2((float)my_rows), dy_all);  // this warp's rows, each adding dy
        }
      }
    }
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int j = c * 32 + lane;
      if (j < nv) {
        float* dw = fold_w + (size_t)warp * p.n + (size_t)j * V;
#pragma unroll
        for (int i = 0; i < P; ++i) unpack2(acc_w[c][i], dw[2 * i], dw[2 * i + 1]);
        if constexpr (LN) {
          float* db = fold_b + (size_t)warp * p.n + (size_t)j * V;
#pragma unroll
          for (int i = 0; i < P; ++i) unpack2(acc_b[c][i], db[2 * i], db[2 * i + 1]);
        }
      }
    }
    __syncthreads();
    float* pw = p.partials + (long long)blockIdx.x * p.n;
    float* pb = p.partials + ((long long)p.groups + blockIdx.x) * p.n;
    for (int c = threadIdx.x; c < p.n; c += blockDim.x) {
      float a = fold_w[c];
#pragma unroll
      for (int g = 1; g < kWarps; ++g) a += fold_w[(size_t)g * p.n + c];
      pw[c] = a;
      if constexpr (LN) {
        if (p.db) {
          float b = fold_b[c];
#pragma unroll
          for (int g = 1; g < kWarps; ++g) b += fold_b[(size_t)g * p.n + c];
          pb[c] = b;
        }
      }
    }
    __syncthreads();  // the fold area doubles as the fp64 area of the finalize
  }
  if (p.fused) {
    double* fin = reinterpret_cast<double*>(smem);  // [warps][64] fp64, inside the ring
    bool ok = !any_failed && grid_barrier(p.bar, 1u, &bar_ok);
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

template <typename T, int CH, bool LN, bool DYS>
bool launch_warp_kernel_impl(NormBwdParams p, size_t scratch_bytes, cudaStream_t st, int* rc) {
  constexpr int V = Elem<T>::V;
  const DeviceInfo& dev = device_info();
  const int nv = p.n / V;
  const size_t stage_bytes = (DYS ? 1 : 2) * (size_t)nv * 16;
  // barriers (+ fp32 weight slots; a second table of the same size for LayerNorm with a scalar dy)
  const size_t fixed = kWarps * 8 * sizeof(uint64_t) + (LN ? (size_t)(DYS ? 2 : 1) * CH * 32 * V * sizeof(float) : 0);
  // the ring doubles as the fold area [2][kWarps][n] fp32 and as the fp64 area of the finalize
  size_t floor_bytes = 2 * (size_t)kWarps * p.n * sizeof(float);
  if (floor_bytes < 16 * 64 * sizeof(double)) floor_bytes = 16 * 64 * sizeof(double);
  int stages = 0, ctas_per_sm = (LN && DYS) ? 3 : 2;  // the scalar-dy LayerNorm form needs fewer registers
  for (; ctas_per_sm >= 1; --ctas_per_sm) {
    const size_t per_cta = ((size_t)dev.max_smem_optin - 1024 * (size_t)ctas_per_sm) / (size_t)ctas_per_sm;
    if (per_cta <= fixed + 256) continue;
    stages = (int)((per_cta - fixed - 256) / (kWarps * stage_bytes));
    if (stages >= 2) break;
  }
  if (stages < 2) return false;
  if (stages > 8) stages = 8;
  size_t ring_bytes = (size_t)stages * kWarps * stage_bytes;
  if (ring_bytes < floor_bytes) ring_bytes = floor_bytes;
  ring_bytes = (ring_bytes + 127) / 128 * 128;
  const size_t smem = ring_bytes + fixed;
  if (smem > (size_t)dev.max_smem_optin) return false;
  auto kernel = norm_bwd_warp_kernel<T, CH, LN, DYS>;
  cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(kernel),
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  const int per_sm = cached_occupancy(reinterpret_cast<const void*>(kernel), kWarps * 32, smem);
  long long grid = (long long)per_sm * dev.sm_count;
  const long long useful = (p.rows + kWarps - 1) / kWarps;
  if (grid > useful) grid = useful;
  if (p.dw || p.db) {
    const long long plane = (long long)p.n * sizeof(float);
    const long long max_groups = ((long long)scratch_bytes - 256) / (2 * plane);
    if (max_groups < 1) return false;
    if (grid > max_groups) grid = max_groups;
  }
  p.groups = (int)grid;
  p.fused = 1;
  p.level2 = nullptr;
  if (p.dw || p.db) {  // room for the second level of the finalize behind the partial planes?
    const long long chunks = (p.n + 63) / 64;
    const long long slices = grid / chunks;
    const long long planes = 256 + 2LL * grid * p.n * (long long)sizeof(float);
    const long long need = (planes + 7) / 8 * 8 + 2LL * slices * p.n * (long long)sizeof(double);
    if (slices >= 2 && (long long)scratch_bytes >= need)
      p.level2 = reinterpret_cast<double*>(reinterpret_cast<char*>(p.bar) + (planes + 7) / 8 * 8);
  }
  int stages_arg = stages, ring_arg = (int)ring_bytes;
  void* args[] = {&p, &stages_arg, &ring_arg};
  e = cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), dim3((unsigned)grid), dim3(kWarps * 32),
                                  args, smem, st);
  if (e != cudaSuccess) {
    cudaGetLastError();
    *rc = fail((int)e, "b200_norm_bwd: cooperative launch failed: %s", cudaGetErrorString(e));
    return true;
  }
  note_launch(DYS ? "b200_norm_bwd [warp per row, warp rings, scalar dy, fused finalize]"
                  : "b200_norm_bwd [warp per row, warp rings, fused finalize]");
  *rc = B200_OK;
  return true;
}

template <typename T, int CH, bool LN>
bool launch_warp_kernel(NormBwdParams p, size_t scratch_bytes, cudaStream_t st, int* rc) {
  return p.dy_elem_stride == 0 ? launch_warp_kernel_impl<T, CH, LN, true>(p, scratch_bytes, st, rc)
                               : launch_warp_kernel_impl<T, CH, LN, false>(p, scratch_bytes, st, rc);
}

}  // namespace

template <typename T, bool LN>
bool try_launch_norm_bwd_warp(NormBwdParams p, size_t scratch_bytes, bool cooperative, cudaStream_t st, int* rc) {
  constexpr int V = Elem<T>::V;
  static const bool off = [] {
    const char* e = getenv("B200_NORM_BWD_NO_WARP_RINGS");
    return e && e[0] == '1';
  }();
  if (off || !cooperative || !(p.dw || p.db)) return false;  // the kernel is the fused, single-launch form
  const long long nv = p.n / V;
  if (nv <= 32 || nv > (V == 4 ? 256 : 128) || p.rows >= 0x7fffffffLL) return false;
  {  // dx is addressed with 32-bit element offsets
    const long long last = (p.rows / p.seq) * p.dx_batch_stride + (long long)(p.seq - 1) * p.dx_seq_stride +
                           (long long)(p.n / p.head_dim - 1) * p.dx_head_stride + p.head_dim;
    if (last >= 0x7fffffffLL || p.dx_batch_stride < 0 || p.dx_seq_stride < 0 || p.dx_head_stride < 0) return false;
  }
  const int ch = (int)((nv + 31) / 32);
  switch (ch) {
    case 2: return launch_warp_kernel<T, 2, LN>(p, scratch_bytes, st, rc);
    case 3: return launch_warp_kernel<T, 3, LN>(p, scratch_bytes, st, rc);
    case 4: return launch_warp_kernel<T, 4, LN>(p, scratch_bytes, st, rc);
    default: break;
  }
  if constexpr (V == 4) {
    if (ch <= 6) return launch_warp_kernel<T, 6, LN>(p, scratch_bytes, st, rc);
    return launch_warp_kernel<T, 8, LN>(p, scratch_bytes, st, rc);
  }
  return false;
}

#define B200_INSTANTIATE(TT)                                                                              \
  template bool try_launch_norm_bwd_warp<TT, true>(NormBwdParams, size_t, bool, cudaStream_t, int*);      \
  template bool try_launch_norm_bwd_warp<TT, false>(NormBwdParams, size_t, bool, cudaStream_t, int*);
B200_INSTANTIATE(float)
B200_INSTANTIATE(__nv_bfloat16)
B200_INSTANTIATE(__half)
#undef B200_INSTANTIATE

unsigned int norm_bwd_warp_wait_timeouts() { return read_wait_timeouts(); }

}  // namespace b200
