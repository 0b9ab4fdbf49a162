// BatchNorm2d training forward: per-channel var_mean over (N,H,W), normalise, affine, optional
// ReLU, running-statistics update.
//
// Replaces the three-kernel Triton plan of the BatchNorm repros in the reference
// (repros/canonical/var_mean_42fad1ece813/oracle.py:11-46 partial sums, :49-87 finalize and
// running stats, :90-119 normalise pass that re-reads x from DRAM).
//
// Evaluation order, as the decomposed aten graph has it (var_mean_42fad1ece813/repro.py:23-58):
//   var, mean = var_mean(float(x), correction 0);  invstd = rsqrt(var + eps)
//   y = relu(cast(((x - mean) * invstd) * w + b))           (ReLU after the cast)
//   running_mean = mean*m + running_mean*(1-m)
//   running_var  = (var*unbias)*m + running_var*(1-m),  unbias = n/(n-1)
//
// Channels-last fast path (x viewed as [R = N*H*W, C], C contiguous): ONE cooperative kernel.
//   pass 1  every CTA owns a contiguous range of row tiles and accumulates, per channel, the
//           shifted sums S1 = sum(x - K), S2 = sum((x - K)^2) with K = x[0, c] (a value of the
//           channel itself, so S2 - S1^2/n does not cancel); the CTA's last tiles stay in shared
//           memory, and the loads carry an L2 evict-last hint.
//   barrier per-CTA partials -> channels are split over the CTAs, each combines its channels over
//           all partials in fp64, writes mean / invstd / running stats; second barrier.
//   pass 2  the CTA walks its tiles in REVERSE order: first the ones still in shared memory, then
//           the most recently read ones, which are the likeliest to still be in L2; y is written
//           with streaming stores so that it does not push x out of L2.
// DRAM traffic therefore approaches one read of x plus one write of y.
// Contiguous NCHW tensors take the single-launch cluster kernel of batch_norm_nchw.cu. Any other
// layout takes the three-launch general path: strided statistics, finalize, strided normalise.
#include "batch_norm.cuh"
#include "tile_stream.cuh"

#include <cstdlib>
#include <mutex>
#include <type_traits>

namespace b200 {

template <typename T, bool VECTOR>
__device__ __forceinline__ void bn_finalize_channel(const BatchNormParams& p, int c, int num_partials,
                                                    float shift) {
  // Called by one warp per channel: lanes split the partials, fp64 accumulation, fixed order.
  const int lane = threadIdx.x & 31;
  float old_mean = 0.f, old_var = 0.f;  // requested now, so that they do not cost a round trip after the sums
  if (lane == 0 && p.running_mean) {
    old_mean = __ldcg(p.running_mean + c);
    old_var = __ldcg(p.running_var + c);
  }
  double s1 = 0.0, s2 = 0.0;
  for (int g0 = lane; g0 < num_partials; g0 += 8 * 32) {  // eight pairs of loads in flight before any is used
    float a[8], b[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int g = g0 + u * 32;
      a[u] = g < num_partials ? __ldcg(p.partials + ((long long)g * 2) * p.channels + c) : 0.f;
      b[u] = g < num_partials ? __ldcg(p.partials + ((long long)g * 2 + 1) * p.channels + c) : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      s1 += (double)a[u];
      s2 += (double)b[u];
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s1 += __shfl_xor_sync(0xffffffffu, s1, o);
    s2 += __shfl_xor_sync(0xffffffffu, s2, o);
  }
  if (lane == 0) {
    float mean, invstd;
    bn_channel_stats(p, c, s1, s2, shift, true, &mean, &invstd, true, old_mean, old_var);
    p.stats[c] = mean;
    p.stats[p.channels + c] = invstd;
  }
}

// ----------------------------------------------------------------------------------------------
// Channels-last fused kernel (one CTA per SM, cooperative launch).
//
// x is streamed through a ring of shared-memory stages with bulk asynchronous copies, one
// contiguous tile of rows per copy. blockDim.x = vpr * rpp (vpr = C / V vector columns, rpp rows
// per pass over the CTA); a thread owns one vector column and walks the tile's rows rpp apart, so
// its per-channel accumulators and, later, its mean / invstd / weight / bias stay in registers.
//   pass 1  tiles 0 .. n-1 of the CTA's row range go through the ring; the last `stages` tiles
//           are simply never overwritten, so they are still in shared memory afterwards.
//   stats   per-CTA shifted sums -> grid barrier -> fp64 combine per channel -> grid barrier.
//   pass 2  tiles n-1 .. 0: first the ones still in shared memory, then the earlier ones, loaded
//           again in reverse order (most recently read first: the likeliest to sit in L2) into
//           the stage each one's successor just freed. y goes out with streaming stores.
// One CTA barrier per tile carries the bounded-wait verdict and frees the previous tile's stage.
// ----------------------------------------------------------------------------------------------
template <typename T, int U>
__global__ void __launch_bounds__(1024, 1)
batch_norm_cl_stream_kernel(const BatchNormParams p, const int stages, const int red_rows, const int red_bytes) {
  constexpr int V = Elem<T>::V;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int bar_ok;
  const int tid = threadIdx.x;
  const int T_ = blockDim.x;
  const int vpr = p.channels / V;
  const int rpp = T_ / vpr;
  const int vc = tid % vpr;
  const int tr = tid / vpr;
  const uint32_t row_bytes = (uint32_t)vpr * 16u;
  // A tile is U passes of the CTA over rpp rows: as a flat array of 16-byte vectors, thread tid
  // owns vectors tid, tid + T_, ..., which all fall into its vector column vc.
  const int tile_rows = rpp * U;
  const uint32_t tile_bytes = (uint32_t)tile_rows * row_bytes;
  float* red = reinterpret_cast<float*>(smem + (size_t)stages * tile_bytes);  // [2][red_rows][C], reused later
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)stages * tile_bytes + red_bytes);

  const T* x = reinterpret_cast<const T*>(p.x);
  // Tiles are dealt out round-robin: CTA b owns tiles b, b + gridDim, ... so that at any moment
  // the CTAs stream neighbouring addresses and finish within one tile of each other.
  const long long total_tiles = (p.rows + tile_rows - 1) / tile_rows;
  const int my_tiles =
      total_tiles > blockIdx.x ? (int)((total_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x) : 0;
  auto tile_row0 = [&](int k) { return ((long long)blockIdx.x + (long long)k * gridDim.x) * tile_rows; };
  if (tid == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
    mbar_init_fence();
  }
  __syncthreads();

  const uint64_t keep_policy = l2_policy_evict_last();
  const uint64_t drop_policy = l2_policy_evict_first();
  auto issue = [&](int k, int slot, uint64_t policy) {  // thread 0 only
    const long long r0 = tile_row0(k);
    const long long left = p.rows - r0;
    const uint32_t bytes = (uint32_t)(left < tile_rows ? left : tile_rows) * row_bytes;
    mbar_arrive_expect_tx(&full[slot], bytes);
    bulk_load_hint(smem + (size_t)slot * tile_bytes, x + r0 * p.channels, bytes, &full[slot], policy);
  };

#ifdef B200_BN_TIMING
  unsigned long long* tlog = reinterpret_cast<unsigned long long*>(p.stats + 2 * p.channels) + blockIdx.x * 8;
#define B200_TMARK(i)                                                        \
  if (tid == 0) {                                                            \
    unsigned long long t_;                                                   \
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                   \
    tlog[i] = t_;                                                            \
  }
#else
#define B200_TMARK(i)
#endif
  B200_TMARK(0)
  bool failed = false;
  uint32_t phase_bits = 0;  // bit s: parity of the next completion of stage s
  int issued = 0;           // pass 1: tiles whose copy has been started
  if (tid == 0) {
    for (; issued < my_tiles && issued < stages; ++issued) issue(issued, issued, keep_policy);
  }
  // What thread 0 still has in flight when a wait runs out: wait for it (bounded) before leaving.
  auto drain = [&](int first_stage_hint) {
    (void)first_stage_hint;
    for (int s = 0; s < stages; ++s) mbar_wait(&full[s], (phase_bits >> s) & 1u);
  };

  // ---- pass 1: shifted sums -------------------------------------------------------------------
  f32x2 shift[V / 2], s1[V / 2], s2[V / 2];
  bn_shift_pairs<T>(x, vc, p.channels, p.rows, shift);
#pragma unroll
  for (int i = 0; i < V / 2; ++i) s1[i] = s2[i] = splat2(0.f);
  // Long chains (huge tensors): every 8 tiles the thread moves its sums of squares into fp64 slots
  // of its own in the reduction area, which nothing else uses before the first pass ends.
  double* deep_acc = reinterpret_cast<double*>(red);  // [V][T_]
  if (p.deep) {
#pragma unroll
    for (int i = 0; i < V; ++i) deep_acc[i * T_ + tid] = 0.0;
  }
  auto deep_flush = [&]() {
#pragma unroll
    for (int i = 0; i < V / 2; ++i) {
      float a, b;
      unpack2(s2[i], a, b);
      deep_acc[(2 * i) * T_ + tid] += (double)a;
      deep_acc[(2 * i + 1) * T_ + tid] += (double)b;
      s2[i] = splat2(0.f);
    }
  };
  {
    int st = 0, issue_slot = issued % (stages > 0 ? stages : 1);
    for (int k = 0; k < my_tiles; ++k) {
      const bool arrived = mbar_wait(&full[st], (phase_bits >> st) & 1u);
      phase_bits ^= 1u << st;
      if (!__syncthreads_and(arrived)) {
        failed = true;
        break;
      }
      if (tid == 0 && k >= 1 && issued < my_tiles) {  // everyone is done with tile k-1
        fence_proxy_async_smem();
        issue(issued, issue_slot, keep_policy);
        ++issued;
        if (++issue_slot == stages) issue_slot = 0;
      }
      const long long left = p.rows - tile_row0(k);
      const int vecs = (int)(left < tile_rows ? left : tile_rows) * vpr;  // vectors in this tile
      const uint4* src = reinterpret_cast<const uint4*>(smem + (size_t)st * tile_bytes);
      uint4 raw[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (tid + u * T_ < vecs) raw[u] = src[tid + u * T_];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (tid + u * T_ < vecs) {
          float f[V];
          Elem<T>::unpack(raw[u], f);
#pragma unroll
          for (int i = 0; i < V / 2; ++i) {
            const f32x2 d = sub2(pack2(f[2 * i], f[2 * i + 1]), shift[i]);
            s1[i] = add2(s1[i], d);
            s2[i] = fma2(d, d, s2[i]);
          }
        }
      }
      if (p.deep && (k & 7) == 7) deep_flush();
      if (++st == stages) st = 0;
    }
  }
  if (p.deep) {  // the rest of the chain joins the fp64 part; from here on the sums are fp32 again
    deep_flush();
#pragma unroll
    for (int i = 0; i < V / 2; ++i)
      s2[i] = pack2((float)deep_acc[(2 * i) * T_ + tid], (float)deep_acc[(2 * i + 1) * T_ + tid]);
    __syncthreads();  // the reduction area is about to be rewritten
  }
  if (failed && tid == 0) {
    note_wait_timeout();
    atomicExch(&p.bar[1], 1u);
    // undo the flip of the stage whose wait ran out, then wait (bounded) for every stage in flight
    drain(0);
  }

  B200_TMARK(1)
  // ---- per-CTA partial sums ---------------------------------------------------------------------
  if (!failed) {
    float a1[V], a2[V];
#pragma unroll
    for (int i = 0; i < V / 2; ++i) {
      unpack2(s1[i], a1[2 * i], a1[2 * i + 1]);
      unpack2(s2[i], a2[2 * i], a2[2 * i + 1]);
    }
    float* r1 = red;
    float* r2 = red + (size_t)red_rows * p.channels;
    int my_red_row;
    bool writer = true;
    if (red_rows != rpp) {
      // vpr is a power of two <= 32: lanes vpr apart share a vector column; fold them first
      for (int off = vpr; off < 32; off <<= 1) {
#pragma unroll
        for (int i = 0; i < V; ++i) {
          a1[i] += __shfl_xor_sync(0xffffffffu, a1[i], off);
          a2[i] += __shfl_xor_sync(0xffffffffu, a2[i], off);
        }
      }
      my_red_row = tid >> 5;
      writer = (tid & 31) < vpr;
    } else {
      my_red_row = tr;
    }
    if (writer) {
#pragma unroll
      for (int i = 0; i < V; ++i) {
        r1[(size_t)my_red_row * p.channels + vc * V + i] = a1[i];
        r2[(size_t)my_red_row * p.channels + vc * V + i] = a2[i];
      }
    }
    __syncthreads();
    for (int c = tid; c < p.channels; c += T_) {
      float a = 0.f, b = 0.f;
      for (int k = 0; k < red_rows; ++k) {
        a += r1[(size_t)k * p.channels + c];
        b += r2[(size_t)k * p.channels + c];
      }
      p.partials[((long long)blockIdx.x * 2) * p.channels + c] = a;
      p.partials[((long long)blockIdx.x * 2 + 1) * p.channels + c] = b;
    }
  }
  B200_TMARK(2)
  bool ok = !failed && grid_barrier(p.bar, 1u, &bar_ok);
  B200_TMARK(3)

  // ---- channel statistics ------------------------------------------------------------------------
  // Few channels: every CTA sums all partials itself (coalesced reads of a table that sits in L2)
  // and keeps mean / invstd in shared memory; CTA 0 also writes the global statistics. No second
  // grid barrier. Many channels: the channels are dealt out to the CTAs, each combines its own
  // with all threads, and a second grid barrier publishes the table.
  double* dred = reinterpret_cast<double*>(red);
  float* stats_s = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(red) + (size_t)T_ * 16);
  const int P = gridDim.x;
  if (ok && p.local_stats) {
    const int C = p.channels;
    const int PG = T_ / C;  // groups of threads that split the partial rows
    const int c = tid % C, pg = tid / C;
    double d1 = 0.0, d2 = 0.0;
    if (pg < PG) {
      for (int g0 = pg; g0 < P; g0 += 8 * PG) {  // eight pairs of loads in flight before any is used
        float a[8], b[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int g = g0 + u * PG;
          a[u] = g < P ? __ldcg(p.partials + ((long long)g * 2) * C + c) : 0.f;
          b[u] = g < P ? __ldcg(p.partials + ((long long)g * 2 + 1) * C + c) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          d1 += (double)a[u];
          d2 += (double)b[u];
        }
      }
      dred[((size_t)pg * C + c) * 2] = d1;
      dred[((size_t)pg * C + c) * 2 + 1] = d2;
    }
    __syncthreads();
    if (tid < C) {
      double t1 = 0.0, t2 = 0.0;
      for (int g = 0; g < PG; ++g) {
        t1 += dred[((size_t)g * C + tid) * 2];
        t2 += dred[((size_t)g * C + tid) * 2 + 1];
      }
      float mean, invstd;
      bn_channel_stats(p, tid, t1, t2, bn_shift_scalar<T>(x, tid, p.channels, p.rows), blockIdx.x == 0, &mean, &invstd);
      stats_s[tid] = mean;
      stats_s[C + tid] = invstd;
    }
    __syncthreads();
  } else if (ok) {
    bn_stats_by_warps<T>(p, x, P);
    B200_TMARK(4)
    ok = grid_barrier(p.bar, 2u, &bar_ok);
  }
  B200_TMARK(5)

  // ---- pass 2: normalise, tiles in reverse order --------------------------------------------------
  if (ok && my_tiles > 0) {
    f32x2 mean2[V / 2], inv2[V / 2], w2[V / 2], b2[V / 2];
#pragma unroll
    for (int i = 0; i < V / 2; ++i) {
      const int c = vc * V + 2 * i;
      if (p.local_stats) {
        mean2[i] = pack2(stats_s[c], stats_s[c + 1]);
        inv2[i] = pack2(stats_s[p.channels + c], stats_s[p.channels + c + 1]);
      } else {
        mean2[i] = pack2(__ldcg(p.stats + c), __ldcg(p.stats + c + 1));
        inv2[i] = pack2(__ldcg(p.stats + p.channels + c), __ldcg(p.stats + p.channels + c + 1));
      }
      w2[i] = p.weight ? pack2(load_param1(p.weight, p.w_dtype, c), load_param1(p.weight, p.w_dtype, c + 1))
                       : splat2(1.f);
      b2[i] = p.bias ? pack2(load_param1(p.bias, p.w_dtype, c), load_param1(p.bias, p.w_dtype, c + 1))
                     : splat2(0.f);
    }
    T* y = reinterpret_cast<T*>(p.y);
    const int resident_from = my_tiles - (my_tiles < stages ? my_tiles : stages);  // tiles >= this are in smem
    int st = (my_tiles - 1) % stages;
    int next_load = resident_from - 1;  // next tile to bring back, descending
    for (int k = my_tiles - 1; k >= 0; --k) {
      bool arrived = true;
      if (k < resident_from) {
        arrived = mbar_wait(&full[st], (phase_bits >> st) & 1u);
        phase_bits ^= 1u << st;
      }
      if (!__syncthreads_and(arrived)) {
        failed = true;
        break;
      }
      if (tid == 0 && k < my_tiles - 1 && next_load >= 0) {
        // everyone is done with tile k+1: its stage takes tile k+1-stages (= next_load)
        int freed = st + 1;
        if (freed == stages) freed = 0;
        fence_proxy_async_smem();
        issue(next_load, freed, drop_policy);
        --next_load;
      }
      const long long r0 = tile_row0(k);
      const long long left = p.rows - r0;
      const int vecs = (int)(left < tile_rows ? left : tile_rows) * vpr;
      const uint4* src = reinterpret_cast<const uint4*>(smem + (size_t)st * tile_bytes);
      uint4* dst = reinterpret_cast<uint4*>(y + r0 * p.channels);
      // Vectors are read one by one (the compiler hoists what the register budget allows): the
      // per-channel constants already take half of the 64 registers a 1024-thread CTA may use.
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (tid + u * T_ >= vecs) continue;
        float f[V];
        Elem<T>::unpack(src[tid + u * T_], f);
        uint4 packed;
        if constexpr (sizeof(T) == 2) {
          using P2 = typename std::conditional<std::is_same<T, __half>::value, __half2, __nv_bfloat162>::type;
          uint32_t wds[4];
#pragma unroll
          for (int i = 0; i < V / 2; ++i) {
            f32x2 o = add2(mul2(mul2(sub2(pack2(f[2 * i], f[2 * i + 1]), mean2[i]), inv2[i]), w2[i]), b2[i]);
            float oa, ob;
            unpack2(o, oa, ob);
            P2 h;
            if constexpr (std::is_same<T, __half>::value) {
              h = __floats2half2_rn(oa, ob);
              if (p.relu) h = __hmax2_nan(h, __float2half2_rn(0.f));  // ReLU after the cast; NaN stays NaN
            } else {
              h = __floats2bfloat162_rn(oa, ob);
              if (p.relu) h = __hmax2_nan(h, __float2bfloat162_rn(0.f));
            }
            wds[i] = *reinterpret_cast<uint32_t*>(&h);
          }
          packed = make_uint4(wds[0], wds[1], wds[2], wds[3]);
        } else {
          float o[V];
#pragma unroll
          for (int i = 0; i < V / 2; ++i) {
            f32x2 r = add2(mul2(mul2(sub2(pack2(f[2 * i], f[2 * i + 1]), mean2[i]), inv2[i]), w2[i]), b2[i]);
            unpack2(r, o[2 * i], o[2 * i + 1]);
            if (p.relu) {
              o[2 * i] = o[2 * i] < 0.f ? 0.f : o[2 * i];
              o[2 * i + 1] = o[2 * i + 1] < 0.f ? 0.f : o[2 * i + 1];
            }
          }
          packed = Elem<T>::pack(o);
        }
        st_stream(dst + tid + u * T_, packed);
      }
      if (--st < 0) st = stages - 1;
    }
    if (failed && tid == 0) {
      note_wait_timeout();
      atomicExch(&p.bar[1], 1u);
      drain(0);
    }
  }
  B200_TMARK(6)
  grid_barrier_depart(p.bar);
}

// ----------------------------------------------------------------------------------------------
// Channels-last fused kernel with one private copy ring per WARP (vpr = C / V a power of two
// <= 32; one CTA of 32 warps per SM, cooperative launch).
//
// The CTA-wide ring above costs one CTA barrier per tile, which keeps 32 warps in lock step. Here:
//   * x is cut into blocks of 32 chunks (a chunk = 32 * U vectors = 512 * U bytes); CTA b takes the
//     blocks b, b + grid, b + 2 grid, ...; warp w of the CTA takes chunk w of each. The list is
//     fixed, so which thread sums which element never changes: the statistics are bit-reproducible.
//   * each warp streams its chunks through its own ring: lane 0 starts the bulk copies, all lanes
//     wait on the chunk's mbarrier, consume it, and after a __syncwarp lane 0 refills the slot.
//     No CTA barrier in either pass; warps drift apart and hide each other's latencies.
//   * the per-chunk bookkeeping is 32-bit and incremental (a chunk is 32 elements per lane: every
//     instruction spent on indices counts), and whole chunks - all but those of the very last
//     block - take a path without per-vector bounds checks.
//   pass 1  the CTA's blocks in order; a warp's last `stages` chunks are never overwritten (and are
//           loaded with the evict-first hint: they will not be read from L2 again).
//   stats   lanes that share a vector column are folded by shuffles, warps through shared memory,
//           CTAs through the scratch buffer and one grid barrier (two for many channels), fp64.
//   pass 2  the same blocks in reverse order: the resident chunks first, then the rest, each
//           loaded again into the slot its successor freed (most recently read first: the
//           likeliest to sit in L2).
// Every wait is bounded (mbar_wait); a wait that runs out makes the CTA raise the error word of the
// grid barrier, wait for its own copies, and skip the rest.
// ----------------------------------------------------------------------------------------------
template <typename T, int U>
__global__ void __launch_bounds__(1024, 1)
batch_norm_cl_warp_kernel(const BatchNormParams p, const int stages, const int red_bytes, const int nblocks,
                          const int flags) {
  constexpr int V = Elem<T>::V;
  constexpr uint32_t CHUNK_BYTES = 512u * U;
  constexpr uint32_t CV = 32 * U;  // vectors per chunk
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int bar_ok;
  __shared__ int cta_failed;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int T_ = blockDim.x;  // 1024
  const int vpr = p.channels / V;
  const int vc = lane & (vpr - 1);  // this lane's vector column, the same in every chunk
  // layout: [32 warps][stages][CHUNK_BYTES] | reduction area (red_bytes) | mbarriers [32][stages]
  unsigned char* ring = smem + (size_t)warp * stages * CHUNK_BYTES;
  float* red = reinterpret_cast<float*>(smem + (size_t)32 * stages * CHUNK_BYTES);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)32 * stages * CHUNK_BYTES + red_bytes) + warp * stages;
  const T* x = reinterpret_cast<const T*>(p.x);
  const uint32_t total_vecs = (uint32_t)(p.rows * vpr);  // the launcher admits fewer than 2^31 vectors

  // The shift of the channel this thread finalises later: fetched now, needed after the barrier.
  const float stat_shift = tid < p.channels ? bn_shift_scalar<T>(x, tid, p.channels, p.rows) : 0.f;

  if (tid == 0) cta_failed = 0;
  if (lane == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
  }
  mbar_init_fence();
  __syncthreads();

  // chunk k of this warp: vectors [first0 + k * step, ... + CV), clipped in the last block only
  const int n_chunks = nblocks > (int)blockIdx.x ? (nblocks - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
  const uint32_t first0 = ((uint32_t)blockIdx.x * 32u + (uint32_t)warp) * CV;
  const uint32_t step = (uint32_t)gridDim.x * 32u * CV;
  const int last_k = ((nblocks - 1) % (int)gridDim.x == (int)blockIdx.x) ? n_chunks - 1 : -1;  // chunk of the last block
  auto vecs_of = [&](int k, uint32_t first) -> int {
    if (k != last_k) return (int)CV;
    return first >= total_vecs ? 0 : (total_vecs - first < CV ? (int)(total_vecs - first) : (int)CV);
  };
  const uint64_t keep_policy = (flags & 2) ? l2_policy_evict_last() : l2_policy_evict_normal();
  const uint64_t drop_policy = l2_policy_evict_first();
  const uint4* xv = reinterpret_cast<const uint4*>(p.x);
  auto issue = [&](uint32_t first, int nv, int slot, uint64_t policy) {  // lane 0 only, nv > 0
    const uint32_t bytes = (uint32_t)nv * 16u;
    mbar_arrive_expect_tx(&full[slot], bytes);
    bulk_load_hint(ring + (size_t)slot * CHUNK_BYTES, xv + first, bytes, &full[slot], policy);
  };

#ifdef B200_BN_TIMING
  unsigned long long* tlog = reinterpret_cast<unsigned long long*>(p.stats + 2 * p.channels) + blockIdx.x * 8;
#define B200_WMARK(i)                                                        \
  {                                                                          \
    __syncthreads();                                                         \
    if (tid == 0) {                                                          \
      unsigned long long t_;                                                 \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                 \
      tlog[i] = t_;                                                          \
    }                                                                        \
  }
#else
#define B200_WMARK(i)
#endif
  B200_WMARK(0)
  bool failed = false;
  uint32_t phase_bits = 0;  // bit s: parity of the next completion of slot s
  uint32_t busy_bits = 0;   // bit s: slot s has a copy that was started and not yet waited for
  const int keep_until = n_chunks - stages;  // chunks from here on stay in shared memory

  // ---- pass 1: shifted sums -------------------------------------------------------------------
  f32x2 shift[V / 2], s1[V / 2], s2[V / 2];
  bn_shift_pairs<T>(x, vc, p.channels, p.rows, shift);
#pragma unroll
  for (int i = 0; i < V / 2; ++i) s1[i] = s2[i] = splat2(0.f);
  // Long chains (huge tensors): every 8 chunks the lane moves its sums of squares into fp64 slots
  // of its own in the reduction area, which nothing else uses before the first pass ends.
  double* deep_acc = reinterpret_cast<double*>(red);  // [V][1024]
  if (p.deep) {
#pragma unroll
    for (int i = 0; i < V; ++i) deep_acc[i * 1024 + tid] = 0.0;
  }
  auto deep_flush = [&]() {
#pragma unroll
    for (int i = 0; i < V / 2; ++i) {
      float a, b;
      unpack2(s2[i], a, b);
      deep_acc[(2 * i) * 1024 + tid] += (double)a;
      deep_acc[(2 * i + 1) * 1024 + tid] += (double)b;
      s2[i] = splat2(0.f);
    }
  };
  {
    uint32_t f = first0;
    for (int k = 0; k < stages && k < n_chunks; ++k, f += step) {  // fill the ring
      const int nv = vecs_of(k, f);
      if (nv > 0) {
        if (lane == 0) issue(f, nv, k, k < keep_until ? keep_policy : drop_policy);
        busy_bits |= 1u << k;
      }
    }
  }
  auto accumulate = [&](const uint4& raw) {
    f32x2 f[V / 2];
    Pairs<T>::unpack(raw, f);
#pragma unroll
    for (int i = 0; i < V / 2; ++i) {
      const f32x2 d = sub2(f[i], shift[i]);
      s1[i] = add2(s1[i], d);
      s2[i] = fma2(d, d, s2[i]);
    }
  };
  {
    int slot = 0;
    uint32_t first = first0;
    const uint32_t ahead = (uint32_t)stages * step;
    for (int k = 0; k < n_chunks; ++k, first += step) {
      const int nv = vecs_of(k, first);
      if (nv > 0) {
        const bool arrived = __all_sync(0xffffffffu, mbar_wait(&full[slot], (phase_bits >> slot) & 1u));
        if (!arrived) {
          failed = true;
          break;
        }
        phase_bits ^= 1u << slot;
        busy_bits &= ~(1u << slot);
        const uint4* src = reinterpret_cast<const uint4*>(ring + (size_t)slot * CHUNK_BYTES) + lane;
        if (nv == (int)CV) {  // a whole chunk: no bounds checks
#pragma unroll
          for (int u = 0; u < U; ++u) accumulate(src[u * 32]);
        } else {
#pragma unroll
          for (int u = 0; u < U; ++u)
            if (u * 32 + lane < nv) accumulate(src[u * 32]);
        }
        __syncwarp();
      }
      if (p.deep && (k & 7) == 7) deep_flush();
      if (k + stages < n_chunks) {  // refill the slot with the chunk `stages` further on
        const int nnv = vecs_of(k + stages, first + ahead);
        if (nnv > 0) {
          if (lane == 0) {
            fence_proxy_async_smem();
            issue(first + ahead, nnv, slot, k + stages < keep_until ? keep_policy : drop_policy);
          }
          busy_bits |= 1u << slot;
        }
      }
      if (++slot == stages) slot = 0;
    }
  }
  auto give_up = [&]() {  // after a wait ran out: tell everyone, then wait (bounded) for this warp's copies
    if (lane == 0) {
      note_wait_timeout();
      atomicExch(&p.bar[1], 1u);
      atomicExch(&cta_failed, 1);
      for (int s = 0; s < stages; ++s)
        if ((busy_bits >> s) & 1u) mbar_wait(&full[s], (phase_bits >> s) & 1u);
    }
    busy_bits = 0;
    __syncwarp();
  };
  if (failed) give_up();
  if (p.deep) {  // the rest of the chain joins the fp64 part; from here on the sums are fp32 again
    deep_flush();
#pragma unroll
    for (int i = 0; i < V / 2; ++i)
      s2[i] = pack2((float)deep_acc[(2 * i) * 1024 + tid], (float)deep_acc[(2 * i + 1) * 1024 + tid]);
    __syncthreads();  // the reduction area is about to be rewritten
  }

  B200_WMARK(1)
  // ---- per-CTA partial sums ---------------------------------------------------------------------
  {
    float a1[V], a2[V];
#pragma unroll
    for (int i = 0; i < V / 2; ++i) {
      unpack2(s1[i], a1[2 * i], a1[2 * i + 1]);
      unpack2(s2[i], a2[2 * i], a2[2 * i + 1]);
    }
    for (int off = vpr; off < 32; off <<= 1) {  // lanes vpr apart share a vector column
#pragma unroll
      for (int i = 0; i < V; ++i) {
        a1[i] += __shfl_xor_sync(0xffffffffu, a1[i], off);
        a2[i] += __shfl_xor_sync(0xffffffffu, a2[i], off);
      }
    }
    // red: [32 warps][2][C]; a second, smaller table [4][2][C] follows it
    const int C2 = 2 * p.channels;
    if (lane < vpr) {
#pragma unroll
      for (int i = 0; i < V; ++i) {
        red[(size_t)warp * C2 + vc * V + i] = a1[i];
        red[(size_t)warp * C2 + p.channels + vc * V + i] = a2[i];
      }
    }
    __syncthreads();
    failed = cta_failed != 0;
    float* red4 = red + (size_t)32 * C2;
    if (!failed) {
      // 32 rows -> 4 rows -> 1: consecutive threads take consecutive columns (no bank conflicts)
      for (int i = tid; i < 4 * C2; i += T_) {
        const int q = i / C2, c = i - q * C2;
        float a = 0.f;
#pragma unroll
        for (int r = 0; r < 8; ++r) a += red[(size_t)(q * 8 + r) * C2 + c];
        red4[i] = a;
      }
    }
    __syncthreads();
    if (!failed) {
      for (int c = tid; c < C2; c += T_) {
        const float a = (red4[c] + red4[C2 + c]) + (red4[2 * C2 + c] + red4[3 * C2 + c]);
        p.partials[(long long)blockIdx.x * C2 + c] = a;  // [cta][2][C]
      }
    }
  }
  // weight and bias of this lane's channels: fetched before the grid-wide wait, used after it
  f32x2 w2[V / 2], b2[V / 2];
#pragma unroll
  for (int i = 0; i < V / 2; ++i) {
    const int c = vc * V + 2 * i;
    w2[i] = p.weight ? pack2(load_param1(p.weight, p.w_dtype, c), load_param1(p.weight, p.w_dtype, c + 1))
                     : splat2(1.f);
    b2[i] = p.bias ? pack2(load_param1(p.bias, p.w_dtype, c), load_param1(p.bias, p.w_dtype, c + 1))
                   : splat2(0.f);
  }
  B200_WMARK(2)
  bool ok = !failed && grid_barrier(p.bar, 1u, &bar_ok);
  B200_WMARK(3)

  // ---- channel statistics (same scheme as the CTA-ring kernel) -----------------------------------
  double* dred = reinterpret_cast<double*>(red);
  float* stats_s = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(red) + (size_t)T_ * 16);
  const int P = gridDim.x;
  if (ok && p.local_stats) {
    const int C = p.channels;
    const int PG = T_ / C;
    const int c = tid % C, pg = tid / C;
    double d1 = 0.0, d2 = 0.0;
    if (pg < PG) {
      for (int g0 = pg; g0 < P; g0 += 12 * PG) {  // twelve pairs of loads in flight before any is used
        float a[12], b[12];
#pragma unroll
        for (int u = 0; u < 12; ++u) {
          const int g = g0 + u * PG;
          a[u] = g < P ? __ldcg(p.partials + ((long long)g * 2) * C + c) : 0.f;
          b[u] = g < P ? __ldcg(p.partials + ((long long)g * 2 + 1) * C + c) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 12; ++u) {
          d1 += (double)a[u];
          d2 += (double)b[u];
        }
      }
      dred[((size_t)pg * C + c) * 2] = d1;
      dred[((size_t)pg * C + c) * 2 + 1] = d2;
    }
    __syncthreads();
    if (tid < C) {
      double t1 = 0.0, t2 = 0.0;
      for (int g = 0; g < PG; ++g) {
        t1 += dred[((size_t)g * C + tid) * 2];
        t2 += dred[((size_t)g * C + tid) * 2 + 1];
      }
      float mean, invstd;
      bn_channel_stats(p, tid, t1, t2, stat_shift, blockIdx.x == 0, &mean, &invstd);
      stats_s[tid] = mean;
      stats_s[C + tid] = invstd;
    }
    __syncthreads();
  } else if (ok) {
    bn_stats_by_warps<T>(p, x, P);
    ok = grid_barrier(p.bar, 2u, &bar_ok);
  }

  B200_WMARK(5)
  // ---- pass 2: normalise, chunks in reverse order -------------------------------------------------
  if (ok && p.y && n_chunks > 0) {
    f32x2 mean2[V / 2], inv2[V / 2];
#pragma unroll
    for (int i = 0; i < V / 2; ++i) {
      const int c = vc * V + 2 * i;
      if (p.local_stats) {
        mean2[i] = pack2(stats_s[c], stats_s[c + 1]);
        inv2[i] = pack2(stats_s[p.channels + c], stats_s[p.channels + c + 1]);
      } else {
        mean2[i] = pack2(__ldcg(p.stats + c), __ldcg(p.stats + c + 1));
        inv2[i] = pack2(__ldcg(p.stats + p.channels + c), __ldcg(p.stats + p.channels + c + 1));
      }
    }
    const bool relu = p.relu != 0;
    auto normalise = [&](const uint4& raw, uint4* dst) {
      f32x2 f[V / 2], o[V / 2];
      Pairs<T>::unpack(raw, f);
#pragma unroll
      for (int i = 0; i < V / 2; ++i) o[i] = add2(mul2(mul2(sub2(f[i], mean2[i]), inv2[i]), w2[i]), b2[i]);
      uint4 packed = Pairs<T>::pack(o);
      if (relu) {  // ReLU after the cast, as the graph has it; NaN stays NaN
        if constexpr (std::is_same<T, __nv_bfloat16>::value) {
          const __nv_bfloat162 z = __float2bfloat162_rn(0.f);
          uint32_t* w = reinterpret_cast<uint32_t*>(&packed);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __hmax2_nan(*reinterpret_cast<__nv_bfloat162*>(&w[i]), z);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
          }
        } else if constexpr (std::is_same<T, __half>::value) {
          const __half2 z = __float2half2_rn(0.f);
          uint32_t* w = reinterpret_cast<uint32_t*>(&packed);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            __half2 h = __hmax2_nan(*reinterpret_cast<__half2*>(&w[i]), z);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
          }
        } else {
          float* w = reinterpret_cast<float*>(&packed);
#pragma unroll
          for (int i = 0; i < 4; ++i) w[i] = w[i] < 0.f ? 0.f : w[i];  // NaN < 0 is false: NaN stays
        }
      }
      st_stream(reinterpret_cast<T*>(dst), packed);
    };
    const int resident_from = n_chunks - (n_chunks < stages ? n_chunks : stages);  // chunks >= this are in smem
    int slot = (n_chunks - 1) % stages;
    uint32_t first = first0 + (uint32_t)(n_chunks - 1) * step;
    const uint32_t behind = (uint32_t)stages * step;
    uint4* yv = reinterpret_cast<uint4*>(p.y) + lane;
    for (int k = n_chunks - 1; k >= 0; --k, first -= step) {
      const int nv = vecs_of(k, first);
      if (nv > 0) {
        if (k < resident_from) {
          const bool arrived = __all_sync(0xffffffffu, mbar_wait(&full[slot], (phase_bits >> slot) & 1u));
          if (!arrived) {
            failed = true;
            break;
          }
          phase_bits ^= 1u << slot;
          busy_bits &= ~(1u << slot);
        }
        const uint4* src = reinterpret_cast<const uint4*>(ring + (size_t)slot * CHUNK_BYTES) + lane;
        uint4* dst = yv + first;
        if (nv == (int)CV) {
#pragma unroll
          for (int u = 0; u < U; ++u) normalise(src[u * 32], dst + u * 32);
        } else {
#pragma unroll
          for (int u = 0; u < U; ++u)
            if (u * 32 + lane < nv) normalise(src[u * 32], dst + u * 32);
        }
        __syncwarp();
      }
      if (k >= stages) {  // the slot takes the chunk `stages` before this one (never the last block: whole)
        if (lane == 0) {
          fence_proxy_async_smem();
          issue(first - behind, (int)CV, slot, drop_policy);
        }
        busy_bits |= 1u << slot;
      }
      if (--slot < 0) slot = stages - 1;
    }
    if (failed) give_up();
  }
  B200_WMARK(6)
  grid_barrier_depart(p.bar);
}

// ----------------------------------------------------------------------------------------------
// General path: x addressed as (n, c, s) with arbitrary strides.
// ----------------------------------------------------------------------------------------------
// Geometry of the fused kernel for vpr = C / V vector columns: CTA size (a multiple of both vpr
// and 32, at most 1024) and the number of rows of the shared-memory reduction area. When vpr is a
// power of two <= 32 the lanes of a warp that share a column are folded by shuffles first and the
// area has one row per warp; otherwise it has one row per thread row and the CTA is kept at <= 256
// threads so that it stays small. Returns 0 threads when there is no fit.
struct FusedGeometry {
  int threads;
  int red_rows;
};
static FusedGeometry fused_geometry(int vpr) {
  FusedGeometry g = {0, 0};
  if (vpr < 1 || vpr > 1024) return g;
  const bool pow2 = (vpr & (vpr - 1)) == 0;
  if (pow2 && vpr <= 32) {
    g.threads = 1024;
    g.red_rows = 1024 / 32;
    return g;
  }
  const int cap = vpr > 256 ? 1024 : 256;
  int rpp = cap / vpr;
  while (rpp > 0 && (vpr * rpp) % 32 != 0) --rpp;
  if (rpp == 0) return g;
  g.threads = vpr * rpp;
  g.red_rows = rpp;
  return g;
}

template <typename T>
__global__ void __launch_bounds__(256) batch_norm_stats_general_kernel(const BatchNormParams p) {
  __shared__ float red[32];
  const int c = blockIdx.x;
  const int split = blockIdx.y, splits = gridDim.y;
  const T* x = reinterpret_cast<const T*>(p.x);
  const float shift = Elem<T>::to_f32(x[(long long)c * p.sc]);
  const long long total = p.rows * p.spatial;
  const long long per = (total + splits - 1) / splits;
  const long long e0 = (long long)split * per;
  const long long e1 = e0 + per < total ? e0 + per : total;
  float s1 = 0.f, s2 = 0.f;
  for (long long e = e0 + threadIdx.x; e < e1; e += blockDim.x) {
    const long long n = e / p.spatial, s = e % p.spatial;
    const float d = Elem<T>::to_f32(x[n * p.sn + (long long)c * p.sc + s * p.ss]) - shift;
    s1 += d;
    s2 += d * d;
  }
  s1 = block_reduce<SumOp>(s1, red);
  s2 = block_reduce<SumOp>(s2, red);
  if (threadIdx.x == 0) {
    p.partials[((long long)split * 2) * p.channels + c] = s1;
    p.partials[((long long)split * 2 + 1) * p.channels + c] = s2;
  }
}

// rows_shift: the sums were shifted by bn_shift_scalar (channels-last flat path, p.rows = N*H*W)
// instead of by the channel's first element.
template <typename T>
__global__ void __launch_bounds__(256) batch_norm_finalize_general_kernel(const BatchNormParams p,
                                                                          int num_partials, int rows_shift) {
  const int warps = blockDim.x >> 5;
  const int c = blockIdx.x * warps + (threadIdx.x >> 5);
  if (c >= p.channels) return;
  const T* x = reinterpret_cast<const T*>(p.x);
  const float shift = rows_shift ? bn_shift_scalar<T>(x, c, p.channels, p.rows) : Elem<T>::to_f32(x[(long long)c * p.sc]);
  bn_finalize_channel<T, false>(p, c, num_partials, shift);
}

template <typename T>
__global__ void __launch_bounds__(256) batch_norm_apply_general_kernel(const BatchNormParams p) {
  const int c = blockIdx.x;
  const T* x = reinterpret_cast<const T*>(p.x);
  T* y = reinterpret_cast<T*>(p.y);
  const float mean = p.stats[c], invstd = p.stats[p.channels + c];
  const float w = p.weight ? load_param1(p.weight, p.w_dtype, c) : 1.f;
  const float b = p.bias ? load_param1(p.bias, p.w_dtype, c) : 0.f;
  const long long total = p.rows * p.spatial;
  const long long per = (total + gridDim.y - 1) / gridDim.y;
  const long long e0 = (long long)blockIdx.y * per;
  const long long e1 = e0 + per < total ? e0 + per : total;
  for (long long e = e0 + threadIdx.x; e < e1; e += blockDim.x) {
    const long long n = e / p.spatial, s = e % p.spatial;
    const long long off = n * p.sn + (long long)c * p.sc + s * p.ss;
    float o = ((Elem<T>::to_f32(x[off]) - mean) * invstd) * w + b;
    if (p.relu) o = o < 0.f ? 0.f : o;
    y[off] = Elem<T>::from_f32(o);
  }
}

// ----------------------------------------------------------------------------------------------
// Channels-last tensors with ANY channel count: three launches over the tensor as a flat array of
// 16-byte vectors (the corpus of the reference has channels-last BatchNorm points with 24, 36, 60,
// 92, 100, 480 ... channels; repros/canonical/var_mean_42fad1ece813/shapes.json).
//
// A vector holds V consecutive elements of the flat [rows * C] array, so it may straddle the end
// of a row. The pattern of channels under a vector repeats every PV = C / gcd(C, V) vectors
// (lcm(C, V) elements): vector i has phase i % PV and its element j belongs to channel
// (phase * V + j) % C. The CTA's vector range starts at a multiple of PV and blockDim.x is a
// multiple of PV, so a thread keeps its phase - its V channels - for the whole launch and its
// sums, and later its mean / invstd / weight / bias, stay in registers.
//   sums      CTA b takes vectors [b * per, (b + 1) * per): shifted sums per thread, the threads of
//             a phase folded in a fixed order (fp64), one fp32 partial row per CTA
//   finalize  a warp per channel (batch_norm_finalize_general_kernel)
//   apply     the same ranges walked from the end (what the sums pass read last is what L2 still
//             holds), y written with streaming stores
// ----------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256, 3) batch_norm_sums_cl_flat_kernel(const BatchNormParams p, long long vecs_per_cta,
                                                                      int PV, int rows_shift) {
  constexpr int V = Elem<T>::V;
  __shared__ float red[2 * 256 * V];  // [2][threads][V]
  const int tid = threadIdx.x, T_ = blockDim.x, C = p.channels;
  const int ph = tid % PV;
  const long long total = p.rows * C / V;
  const long long v0 = (long long)blockIdx.x * vecs_per_cta;
  long long v1 = v0 + vecs_per_cta;
  if (v1 > total) v1 = total;
  const T* xe = reinterpret_cast<const T*>(p.x);
  const uint4* x = reinterpret_cast<const uint4*>(p.x);
  // The shift of every channel (bn_shift_scalar: mean of its first sixteen rows, eight significant
  // bits; the finalize kernel forms the same value) is computed once per CTA into shared memory,
  // at most 2 * 256 * V channels per round, and every thread picks up its V channels.
  f32x2 shift[V / 2], s1[V / 2], s2[V / 2];
  f32x2 upper[V / 2];  // a thread's sum of squares moves here every 16 vectors: two short chains instead of one long one
#pragma unroll
  for (int i = 0; i < V / 2; ++i) shift[i] = s1[i] = s2[i] = upper[i] = splat2(0.f);
  if (!rows_shift) {  // short chains (small tensors): the channel's element of row 0 will do
#pragma unroll
    for (int i = 0; i < V / 2; ++i)
      shift[i] = pack2(Elem<T>::to_f32(__ldg(xe + (ph * V + 2 * i) % C)), Elem<T>::to_f32(__ldg(xe + (ph * V + 2 * i + 1) % C)));
  }
  for (int c0 = 0; rows_shift && c0 < C; c0 += 2 * 256 * V) {
    for (int c = c0 + tid; c < C && c < c0 + 2 * 256 * V; c += T_) red[c - c0] = bn_shift_scalar<T>(xe, c, C, p.rows);
    __syncthreads();
#pragma unroll
    for (int i = 0; i < V / 2; ++i) {
      const int ca = (ph * V + 2 * i) % C, cb = (ph * V + 2 * i + 1) % C;
      float lo, hi;
      unpack2(shift[i], lo, hi);
      if (ca >= c0 && ca < c0 + 2 * 256 * V) lo = red[ca - c0];
      if (cb >= c0 && cb < c0 + 2 * 256 * V) hi = red[cb - c0];
      shift[i] = pack2(lo, hi);
    }
    __syncthreads();
  }
  constexpr int U = 4;  // vectors in flight per thread (three CTAs per SM)
  int round = 0;
  for (long long v = v0 + tid; v < v1; v += (long long)U * T_) {
    uint4 raw[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = v + (long long)u * T_;
      if (i < v1) raw[u] = ld_stream(reinterpret_cast<const T*>(x + i));
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (v + (long long)u * T_ < v1) {
        f32x2 f[V / 2];
        Pairs<T>::unpack(raw[u], f);
#pragma unroll
        for (int i = 0; i < V / 2; ++i) {
          const f32x2 d = sub2(f[i], shift[i]);
          s1[i] = add2(s1[i], d);
          s2[i] = fma2(d, d, s2[i]);
        }
      }
    }
    if ((++round & 3) == 0) {
#pragma unroll
      for (int i = 0; i < V / 2; ++i) {
        upper[i] = add2(upper[i], s2[i]);
        s2[i] = splat2(0.f);
      }
    }
  }
  float* r1 = red;
  float* r2 = red + 256 * V;
#pragma unroll
  for (int i = 0; i < V / 2; ++i) {
    unpack2(s1[i], r1[tid * V + 2 * i], r1[tid * V + 2 * i + 1]);
    unpack2(add2(upper[i], s2[i]), r2[tid * V + 2 * i], r2[tid * V + 2 * i + 1]);
  }
  __syncthreads();
  const int period = PV * V;  // elements; a multiple of C
  for (int c = tid; c < C; c += T_) {
    double a = 0.0, b = 0.0;
    for (int idx = c; idx < period; idx += C) {  // every (phase, element) that lands on channel c
      const int col = idx / V, e = idx % V;
      for (int t = col; t < T_; t += PV) {
        a += (double)r1[t * V + e];
        b += (double)r2[t * V + e];
      }
    }
    p.partials[((long long)blockIdx.x * 2) * C + c] = (float)a;
    p.partials[((long long)blockIdx.x * 2 + 1) * C + c] = (float)b;
  }
}

template <typename T>
__global__ void __launch_bounds__(256, 3) batch_norm_apply_cl_flat_kernel(const BatchNormParams p, long long vecs_per_cta,
                                                                       int PV) {
  constexpr int V = Elem<T>::V;
  const int tid = threadIdx.x, T_ = blockDim.x, C = p.channels;
  const int ph = PV - 1 - tid % PV;  // the range ends on a multiple of PV: its last vector has phase PV - 1
  const long long total = p.rows * C / V;
  const long long v0 = (long long)blockIdx.x * vecs_per_cta;
  long long v1 = v0 + vecs_per_cta;
  if (v1 > total) v1 = total;  // total is a multiple of PV as well (the launcher checks)
  const uint4* x = reinterpret_cast<const uint4*>(p.x);
  uint4* y = reinterpret_cast<uint4*>(p.y);
  f32x2 mean2[V / 2], inv2[V / 2], w2[V / 2], b2[V / 2];
#pragma unroll
  for (int i = 0; i < V / 2; ++i) {
    const int c0 = (ph * V + 2 * i) % C, c1 = (ph * V + 2 * i + 1) % C;
    mean2[i] = pack2(p.stats[c0], p.stats[c1]);
    inv2[i] = pack2(p.stats[C + c0], p.stats[C + c1]);
    w2[i] = p.weight ? pack2(load_param1(p.weight, p.w_dtype, c0), load_param1(p.weight, p.w_dtype, c1)) : splat2(1.f);
    b2[i] = p.bias ? pack2(load_param1(p.bias, p.w_dtype, c0), load_param1(p.bias, p.w_dtype, c1)) : splat2(0.f);
  }
  const bool relu = p.relu != 0;
  constexpr int U = 8;
  for (long long v = v1 - 1 - tid; v >= v0; v -= (long long)U * T_) {
    uint4 raw[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = v - (long long)u * T_;
      if (i >= v0) raw[u] = ld_stream(reinterpret_cast<const T*>(x + i));
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = v - (long long)u * T_;
      if (i >= v0) {
        f32x2 f[V / 2];
        Pairs<T>::unpack(raw[u], f);
#pragma unroll
        for (int k = 0; k < V / 2; ++k) {
          f[k] = add2(mul2(mul2(sub2(f[k], mean2[k]), inv2[k]), w2[k]), b2[k]);
          if (relu) {
            float lo, hi;
            unpack2(f[k], lo, hi);
            f[k] = pack2(lo < 0.f ? 0.f : lo, hi < 0.f ? 0.f : hi);
          }
        }
        st_stream(reinterpret_cast<T*>(y + i), Pairs<T>::pack(f));
      }
    }
  }
}

// Returns false when the shape does not fit (the caller takes the element-wise path).
template <typename T>
static bool try_launch_batch_norm_cl_flat(BatchNormParams p, size_t scratch_bytes, cudaStream_t st, int* rc) {
  constexpr int V = Elem<T>::V;
  const DeviceInfo& dev = device_info();
  const long long C = p.channels;
  long long g = C, h = V;  // gcd(C, V)
  while (h) { const long long t = g % h; g = h; h = t; }
  const long long PV = C / g;
  const long long elems = p.rows * C;
  if (PV > 256 || elems % (PV * V) != 0) return false;  // whole periods only: every range ends on a multiple of PV
  const long long total = elems / V;
  const int threads = (int)(256 / PV * PV);
  const long long stats_floats = 2 * C;
  const long long room = ((long long)scratch_bytes - 256) / (long long)sizeof(float) - stats_floats;
  if (room < 2 * C) return false;
  long long splits = 8LL * dev.sm_count;
  if (splits > room / (2 * C)) splits = room / (2 * C);
  // at least one full round of loads (8 vectors) per thread: small tensors get few partial rows and a
  // short finalize
  if (splits * threads * 8 > total) splits = (total + threads * 8 - 1) / (threads * 8);
  if (splits < 1) splits = 1;
  long long per = (total + splits - 1) / splits;
  per = (per + PV - 1) / PV * PV;
  splits = (total + per - 1) / per;
  p.stats = p.partials + splits * 2 * C;
  const int rows_shift = per > 32LL * threads ? 1 : 0;  // more than 32 vectors per thread
  batch_norm_sums_cl_flat_kernel<T><<<(unsigned)splits, threads, 0, st>>>(p, per, (int)PV, rows_shift);
  *rc = launch_status("b200_batch_norm_fwd sums [channels-last, flat vectors]");
  if (*rc != B200_OK) return true;
  batch_norm_finalize_general_kernel<T><<<(p.channels + 7) / 8, 256, 0, st>>>(p, (int)splits, rows_shift);
  *rc = launch_status("b200_batch_norm_fwd finalize");
  if (*rc != B200_OK || !p.y) return true;
  batch_norm_apply_cl_flat_kernel<T><<<(unsigned)splits, threads, 0, st>>>(p, per, (int)PV);
  *rc = launch_status("b200_batch_norm_fwd apply [channels-last, flat vectors]");
  return true;
}

// Channels-last tensors smaller than this take the three flat launches: a cooperative launch with
// its grid-wide barriers costs more than two extra plain launches until the tensor is tens of MB.
constexpr long long kFlatBelowBytes = 8000000;  // measured: 3.2 MB 16.3 us flat / 21.3 us fused, 12.8 MB 27.5 / 24.1

// B200_BN_CTA_RING=1 keeps the CTA-wide ring for every shape (for measurements).
static bool warp_rings_disabled() {
  static const bool off = [] {
    const char* e = getenv("B200_BN_CTA_RING");
    return e && e[0] == '1';
  }();
  return off;
}

// Per-warp-ring launch; returns false when the shape does not fit (the CTA-ring kernel takes it).
template <typename T>
static bool try_launch_batch_norm_warp(BatchNormParams p, size_t scratch_bytes, cudaStream_t st, int* rc) {
  constexpr int V = Elem<T>::V;
  const DeviceInfo& dev = device_info();
  const int threads = 1024;
  const long long total_vecs = p.rows * (p.channels / V);
  long long grid = dev.sm_count;
  const long long stats_floats = 2LL * p.channels;
  const long long need = 256 + (grid * 2 * p.channels + stats_floats) * (long long)sizeof(float);
  if ((long long)scratch_bytes < need) return false;  // the caller's path reports the shortage
  // reduction area: [32 + 4][2][C] fp32, later reused for the fp64 combine + the CTA's stats table
  size_t red_bytes = 2ull * 36 * p.channels * sizeof(float);
  const size_t stats_area = (size_t)threads * 16 + 2ull * p.channels * sizeof(float);
  if (red_bytes < stats_area) red_bytes = stats_area;
  // more than 64 vectors per lane: the squares are carried in fp64, 8 bytes per channel of every lane
  p.deep = total_vecs > 64LL * threads * grid ? 1 : 0;
  if (p.deep && red_bytes < (size_t)threads * V * sizeof(double)) red_bytes = (size_t)threads * V * sizeof(double);
  red_bytes = (red_bytes + 127) / 128 * 128;
  p.local_stats = (p.channels <= threads && (long long)p.channels * grid <= 32768) ? 1 : 0;
  const size_t barrier_bytes = 32 * 8 * sizeof(uint64_t);
  const size_t budget = (size_t)dev.max_smem_optin - 1024;  // static shared variables
  if (budget < red_bytes + barrier_bytes + 32 * 2 * 1024) return false;
  const size_t per_warp = (budget - red_bytes - barrier_bytes) / 32;
  // 2 KB chunks when three or more fit, else 1 KB chunks
  const bool big = per_warp >= 3 * 2048;
  const size_t chunk = big ? 2048 : 1024;
  int stages = (int)(per_warp / chunk);
  if (stages > 8) stages = 8;
  if (stages < 2) return false;
  const size_t smem = 32 * (size_t)stages * chunk + red_bytes + barrier_bytes;
  // a block = 32 chunks (one per warp); CTA b takes blocks b, b + grid, ...
  const long long block_vecs = 32LL * (long long)(chunk / 16);
  const long long nblocks = (total_vecs + block_vecs - 1) / block_vecs;
  if (grid > nblocks) grid = nblocks;
  if (grid < 1) grid = 1;
  if (total_vecs >= 0x7fffffffLL - 4096) return false;  // the kernel counts vectors in 32 bits
  {
    const long long need2 = 256 + (grid * 2 * p.channels + stats_floats) * (long long)sizeof(float);
    if ((long long)scratch_bytes < need2) return false;
    p.local_stats = (p.channels <= threads && (long long)p.channels * grid <= 32768) ? 1 : 0;
  }
  const void* kernel = big ? reinterpret_cast<const void*>(batch_norm_cl_warp_kernel<T, 4>)
                           : reinterpret_cast<const void*>(batch_norm_cl_warp_kernel<T, 2>);
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  p.rows_per_cta = 0;
  p.smem_tiles = stages;
  p.stats = p.partials + grid * 2 * p.channels;
  int stages_arg = stages, red_bytes_arg = (int)red_bytes, nblocks_arg = (int)nblocks;
  int flags_arg = getenv("B200_BN_EVICT_LAST") ? 2 : 0;
  void* args[] = {&p, &stages_arg, &red_bytes_arg, &nblocks_arg, &flags_arg};
  e = cudaLaunchCooperativeKernel(kernel, dim3((unsigned)grid), dim3(threads), args, smem, st);
  if (e != cudaSuccess) {
    cudaGetLastError();
    *rc = fail((int)e, "b200_batch_norm_fwd: cooperative launch failed: %s", cudaGetErrorString(e));
    return true;
  }
  note_launch("b200_batch_norm_fwd [fused, channels-last, warp rings]");
  *rc = B200_OK;
  return true;
}

template <typename T>
static int launch_batch_norm(BatchNormParams p, bool channels_last_fast, bool channels_last, size_t scratch_bytes,
                             cudaStream_t st) {
  constexpr int V = Elem<T>::V;
  const DeviceInfo& dev = device_info();
  const long long stats_floats = 2LL * p.channels;
  if (channels_last_fast) {
    const int vpr = p.channels / V;
    if ((vpr & (vpr - 1)) == 0 && vpr <= 32 && !warp_rings_disabled()) {
      int rc = B200_OK;
      if (try_launch_batch_norm_warp<T>(p, scratch_bytes, st, &rc)) return rc;
    }
    const FusedGeometry geo = fused_geometry(vpr);
    const int threads = geo.threads;
    const int rpp = threads / vpr;
    // A tile is U = 2 passes of the CTA (U * threads * 16 bytes): 32 KB at 1024 threads, small
    // enough that the round-robin tile assignment leaves the CTAs within a few percent of each other.
    constexpr int passes = 2;
    auto kernel = batch_norm_cl_stream_kernel<T, passes>;
    const size_t row_bytes = (size_t)vpr * 16;
    const int tile_rows = rpp * passes;
    const size_t tile_bytes = (size_t)tile_rows * row_bytes;
    long long grid = dev.sm_count;  // one CTA per SM
    const long long total_tiles = (p.rows + tile_rows - 1) / tile_rows;
    if (grid > total_tiles) grid = total_tiles;
    const long long need = 256 + (grid * 2 * p.channels + stats_floats) * (long long)sizeof(float);
    if ((long long)scratch_bytes < need)
      return fail(B200_ERR_WORKSPACE, "b200_batch_norm_fwd: scratch of %zu bytes, need %lld", scratch_bytes, need);
    p.rows_per_cta = 0;  // unused: tiles are assigned round-robin
    // reduction area: the fp32 fold of pass 1, later reused for the fp64 combine (16 bytes per
    // thread) followed by the CTA's own mean / invstd table
    size_t red_bytes = 2ull * geo.red_rows * p.channels * sizeof(float);
    const size_t stats_area = (size_t)threads * 16 + 2ull * p.channels * sizeof(float);
    if (red_bytes < stats_area) red_bytes = stats_area;
    p.deep = total_tiles * passes > 64LL * grid ? 1 : 0;  // more than 64 vectors per thread
    if (p.deep && red_bytes < (size_t)threads * V * sizeof(double)) red_bytes = (size_t)threads * V * sizeof(double);
    red_bytes = (red_bytes + 15) / 16 * 16;
    p.local_stats = (p.channels <= threads && (long long)p.channels * grid <= 32768) ? 1 : 0;
    const size_t fixed = red_bytes + 8 * sizeof(uint64_t) + 256;
    if (fixed + 2 * tile_bytes > (size_t)dev.max_smem_optin)
      return fail(B200_ERR_UNSUPPORTED, "b200_batch_norm_fwd: %d channels need too much shared memory", p.channels);
    int stages = (int)(((size_t)dev.max_smem_optin - fixed) / tile_bytes);
    if (stages > 8) stages = 8;
    const size_t smem = (size_t)stages * tile_bytes + red_bytes + 8 * sizeof(uint64_t);
    p.smem_tiles = stages;
    cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(kernel),
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail((int)e, "b200_batch_norm_fwd: cannot reserve %zu bytes of shared memory: %s", smem,
                  cudaGetErrorString(e));
    }
    p.stats = p.partials + grid * 2 * p.channels;
    int stages_arg = stages, red_rows_arg = geo.red_rows, red_bytes_arg = (int)red_bytes;
    void* args[] = {&p, &stages_arg, &red_rows_arg, &red_bytes_arg};
    e = cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), dim3((unsigned)grid), dim3(threads),
                                    args, smem, st);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail((int)e, "b200_batch_norm_fwd: cooperative launch failed: %s", cudaGetErrorString(e));
    }
    note_launch("b200_batch_norm_fwd [fused, channels-last, CTA ring]");
    return B200_OK;
  }
  if (channels_last) {  // any channel count: the tensor as a flat array of vectors, three launches
    BatchNormParams q = p;
    q.rows = p.rows * p.spatial;
    int rc = B200_OK;
    if (try_launch_batch_norm_cl_flat<T>(q, scratch_bytes, st, &rc)) return rc;
  }
  {  // contiguous NCHW: one launch, a cluster of CTAs per channel (batch_norm_nchw.cu)
    int rc = B200_OK;
    if (try_launch_batch_norm_nchw<T>(p, st, &rc)) return rc;
  }
  // general path
  const long long total = p.rows * p.spatial;
  long long splits = total / 16384;
  if (splits < 1) splits = 1;
  if (splits > 64) splits = 64;
  const long long need = 256 + (splits * 2 * p.channels + stats_floats) * (long long)sizeof(float);
  if ((long long)scratch_bytes < need)
    return fail(B200_ERR_WORKSPACE, "b200_batch_norm_fwd: scratch of %zu bytes, need %lld", scratch_bytes, need);
  p.stats = p.partials + splits * 2 * p.channels;
  batch_norm_stats_general_kernel<T><<<dim3(p.channels, (unsigned)splits), 256, 0, st>>>(p);
  int rc = launch_status("b200_batch_norm_fwd stats [strided, element-wise]");
  if (rc != B200_OK) return rc;
  batch_norm_finalize_general_kernel<T><<<(p.channels + 7) / 8, 256, 0, st>>>(p, (int)splits, 0);
  rc = launch_status("b200_batch_norm_fwd finalize");
  if (rc != B200_OK) return rc;
  if (p.y) {
    batch_norm_apply_general_kernel<T><<<dim3(p.channels, (unsigned)splits), 256, 0, st>>>(p);
    rc = launch_status("b200_batch_norm_fwd apply [strided, element-wise]");
  }
  return rc;
}

}  // namespace b200

using namespace b200;

// Bounded waits of the fused kernel that ran out since the library was loaded (0 in normal
// operation). Synchronises the device.
extern "C" int64_t b200_batch_norm_wait_timeouts(void) { return (int64_t)read_wait_timeouts(); }

extern "C" int64_t b200_batch_norm_scratch_bytes(int64_t channels) {
  const int sms = device_info().sm_count;
  return 256 + ((int64_t)(sms > 64 ? sms : 64) * 2 * channels + 2 * channels) * (int64_t)sizeof(float);
}

// b200_batch_norm_fwd with the factor that turns the biased batch variance into the value blended
// into running_var given by the caller (unbiased_factor > 0) instead of n / (n - 1). A captured
// graph carries that factor as a literal of the shape it was captured at and applies it at every
// other shape point too; an oracle for such a graph has to do the same.
extern "C" int b200_batch_norm_fwd_ex(const void* x, void* y, const void* weight, const void* bias,
                                      float* running_mean, float* running_var, float* save_mean,
                                      float* save_invstd, int64_t batch, int64_t channels, int64_t spatial,
                                      int64_t stride_n, int64_t stride_c, int64_t stride_s,
                                      int32_t x_dtype, int32_t w_dtype, double eps, double momentum,
                                      double unbiased_factor, int32_t relu, void* scratch,
                                      int64_t scratch_bytes, void* stream) {
  if (!x || !y || !scratch) return fail(B200_ERR_INVALID, "b200_batch_norm_fwd: null argument");
  if (batch <= 0 || channels <= 0 || spatial <= 0 || channels > 0x7fffffffLL)
    return fail(B200_ERR_INVALID, "b200_batch_norm_fwd: bad sizes N=%lld C=%lld HW=%lld", (long long)batch,
                (long long)channels, (long long)spatial);
  if ((running_mean == nullptr) != (running_var == nullptr))
    return fail(B200_ERR_INVALID, "b200_batch_norm_fwd: running_mean and running_var come together");
  if (!aligned16(scratch)) return fail(B200_ERR_ALIGNMENT, "b200_batch_norm_fwd: scratch must be 16-byte aligned");

  BatchNormParams p;
  p.x = x; p.y = y; p.weight = weight; p.bias = bias;
  p.running_mean = running_mean; p.running_var = running_var;
  p.save_mean = save_mean; p.save_invstd = save_invstd;
  p.channels = (int)channels; p.spatial = spatial;
  p.sn = stride_n; p.sc = stride_c; p.ss = stride_s;
  p.w_dtype = w_dtype;
  p.eps = (float)eps; p.momentum = (float)momentum; p.one_minus_momentum = (float)(1.0 - momentum);
  const double count = (double)batch * (double)spatial;
  p.count = count;
  p.inv_count = 1.0 / count;
  p.unbias = unbiased_factor > 0.0 ? (float)unbiased_factor : (float)(count / (count - 1.0));
  p.relu = relu ? 1 : 0;
  p.bar = reinterpret_cast<unsigned int*>(scratch);
  p.partials = reinterpret_cast<float*>(reinterpret_cast<char*>(scratch) + 256);
  p.stats = nullptr; p.rows_per_cta = 0; p.smem_tiles = 0; p.local_stats = 0; p.deep = 0;

  const int eb = dtype_size(x_dtype);
  const int v = 16 / eb;
  // channels-last: c is the unit-stride dimension, rows are (n, s) pairs with a uniform stride of C
  const bool cl = stride_c == 1 && stride_s == channels && stride_n == spatial * channels;
  // the fused cooperative kernels take channel counts that make a power-of-two number (<= 32) of
  // vectors per row; B200_BN_CL_RING=1 sends every count the CTA-ring kernel can lay out there too
  static const bool ring_all = [] {
    const char* e = getenv("B200_BN_CL_RING");
    return e && e[0] == '1';
  }();
  // B200_BN_CL_FLAT_BELOW_MB=<n>: tensors below n MB take the three flat launches even when the fused
  // kernels could (measurement switch; the default threshold is kFlatBelowBytes)
  static const long long flat_below = [] {
    const char* e = getenv("B200_BN_CL_FLAT_BELOW_MB");
    return e ? atoll(e) * 1000000LL : kFlatBelowBytes;
  }();
  const long long vpr = channels % v == 0 ? channels / v : 0;
  const bool pow2 = vpr > 0 && vpr <= 32 && (vpr & (vpr - 1)) == 0;
  const bool small_tensor = batch * channels * spatial * (long long)eb < flat_below;
  const bool fast = cl && vpr > 0 && ((pow2 && !small_tensor) || ring_all) && fused_geometry((int)vpr).threads > 0 &&
                    aligned16(x) && aligned16(y);
  const bool cl_flat = cl && !fast && aligned16(x) && aligned16(y);
  if (fast) {
    p.rows = batch * spatial;
  } else {
    p.rows = batch;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (x_dtype) {
    case B200_F32: return launch_batch_norm<float>(p, fast, cl_flat, (size_t)scratch_bytes, st);
    case B200_BF16: return launch_batch_norm<__nv_bfloat16>(p, fast, cl_flat, (size_t)scratch_bytes, st);
    case B200_F16: return launch_batch_norm<__half>(p, fast, cl_flat, (size_t)scratch_bytes, st);
  }
  return fail(B200_ERR_INVALID, "b200_batch_norm_fwd: unknown dtype %d", x_dtype);
}

extern "C" int b200_batch_norm_fwd(const void* x, void* y, const void* weight, const void* bias,
                                   float* running_mean, float* running_var, float* save_mean,
                                   float* save_invstd, int64_t batch, int64_t channels, int64_t spatial,
                                   int64_t stride_n, int64_t stride_c, int64_t stride_s,
                                   int32_t x_dtype, int32_t w_dtype, double eps, double momentum,
                                   int32_t relu, void* scratch, int64_t scratch_bytes, void* stream) {
  return b200_batch_norm_fwd_ex(x, y, weight, bias, running_mean, running_var, save_mean, save_invstd, batch,
                                channels, spatial, stride_n, stride_c, stride_s, x_dtype, w_dtype, eps, momentum,
                                0.0, relu, scratch, scratch_bytes, stream);
}

// ----------------------------------------------------------------------------------------------
// BatchNorm forward for callers that cannot hand over scratch memory.
//
// Some hosts of this library are not allowed to allocate device memory at all: a serving process
// whose framework carves one arena at start-up and forbids plug-ins to call cudaMalloc (the call
// would also synchronise the whole device in the middle of a request), or an embedding where the
// only device buffers the caller owns are the tensors it was given. b200_batch_norm_fwd needs a
// scratch buffer from its caller; this variant brings its own: a fixed array in the library's
// device image. Every GPU that loads the library holds those bytes until the process exits, which
// is why the size is capped (B200_BN_STATIC_MAX_CHANNELS channels, about 1.3 MB).
//
// The array's name is only meaningful in device code. On the host it is a stand-in symbol, not a
// device address, so the address is looked up once per device with cudaGetSymbolAddress - on the
// first call made while that device is current - and kept. That first call therefore does a little
// set-up work and should be made before any stream capture begins.
//
// All calls on a device share the one array and it keeps whatever the previous call left in it.
// The only part that must start at zero, the grid-barrier words, is cleared on the stream before
// every launch; partial sums and statistics are fully rewritten before they are read. Two calls
// that overlap on the GPU (different streams, no ordering between them) would race on the array:
// callers must order them.
// ----------------------------------------------------------------------------------------------
#define B200_BN_STATIC_MAX_CHANNELS 1024
#define B200_BN_STATIC_MAX_GROUPS 160  // partial rows: one per CTA (<= SM count) or per split (<= 64)

namespace b200 {

constexpr size_t kBnStaticScratchBytes =
    256 + ((size_t)B200_BN_STATIC_MAX_GROUPS * 2 * B200_BN_STATIC_MAX_CHANNELS + 2 * B200_BN_STATIC_MAX_CHANNELS) *
              sizeof(float);

static __device__ __align__(256) unsigned char g_bn_static_scratch[kBnStaticScratchBytes];

// Device address of the array on the current device; looked up on first use per device.
static int bn_static_scratch_address(void** out) {
  static void* address[64] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail((int)e, "b200_batch_norm_fwd_static_scratch: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) return fail(B200_ERR_UNSUPPORTED, "b200_batch_norm_fwd_static_scratch: device index %d", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (address[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_bn_static_scratch);  // `dev` is the current device
    if (e != cudaSuccess || ptr == nullptr) {
      cudaGetLastError();
      return fail(e != cudaSuccess ? (int)e : B200_ERR_INVALID,
                  "b200_batch_norm_fwd_static_scratch: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    }
    address[dev] = ptr;
  }
  *out = address[dev];
  return B200_OK;
}

}  // namespace b200

extern "C" int b200_batch_norm_fwd_static_scratch(const void* x, void* y, const void* weight, const void* bias,
                                                  float* running_mean, float* running_var, float* save_mean,
                                                  float* save_invstd, int64_t batch, int64_t channels,
                                                  int64_t spatial, int64_t stride_n, int64_t stride_c,
                                                  int64_t stride_s, int32_t x_dtype, int32_t w_dtype, double eps,
                                                  double momentum, int32_t relu, void* stream) {
  if (channels > B200_BN_STATIC_MAX_CHANNELS)
    return fail(B200_ERR_UNSUPPORTED,
                "b200_batch_norm_fwd_static_scratch: %lld channels exceed the built-in scratch (max %d); "
                "use b200_batch_norm_fwd with a caller-provided scratch buffer",
                (long long)channels, B200_BN_STATIC_MAX_CHANNELS);
  if (channels > 0 && b200_batch_norm_scratch_bytes(channels) > (int64_t)kBnStaticScratchBytes)
    return fail(B200_ERR_UNSUPPORTED,
                "b200_batch_norm_fwd_static_scratch: this device needs %lld scratch bytes for %lld channels, "
                "the built-in array holds %zu",
                (long long)b200_batch_norm_scratch_bytes(channels), (long long)channels, kBnStaticScratchBytes);
  void* scratch = nullptr;
  int rc = bn_static_scratch_address(&scratch);
  if (rc != B200_OK) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(scratch, 0, 256, st);  // the barrier words must start at zero
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail((int)e, "b200_batch_norm_fwd_static_scratch: clearing the barrier words: %s", cudaGetErrorString(e));
  }
  return b200_batch_norm_fwd(x, y, weight, bias, running_mean, running_var, save_mean, save_invstd, batch,
                             channels, spatial, stride_n, stride_c, stride_s, x_dtype, w_dtype, eps, momentum,
                             relu, scratch, (int64_t)kBnStaticScratchBytes, stream);
}
