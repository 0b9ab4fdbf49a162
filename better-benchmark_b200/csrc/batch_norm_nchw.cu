// BatchNorm2d training forward (+ReLU, running statistics) on a contiguous NCHW tensor, in ONE
// launch.
//
// Most BatchNorm points of the reference's corpus are NCHW (95 of the 121 shape points of
// repros/canonical/var_mean_42fad1ece813/shapes.json), from 50 KB to 100 MB. Its Triton plan for
// them is one launch up to 1024 elements per channel and three launches (partial sums, finalize,
// normalise; oracle.py:11-119) above. Here a channel of at most 16 K elements is kept in the
// registers of one CTA (batch_norm_nchw_small_kernel, further down); larger channels take the
// two-pass kernel below, whose CTAs of one channel form a thread-block cluster and exchange their
// partial sums through distributed shared memory:
//
//   grid (S, C), cluster (S, 1, 1): CTA (s, c) owns images [s * ipc, (s + 1) * ipc) of channel c.
//   pass 1  every plane (the H*W contiguous elements of one image and channel) is walked by a
//           group of G lanes (G = 1 .. 32, chosen so that a lane gets at least ~64 bytes of a
//           plane): the unaligned head and tail of a plane element by element, its body with
//           16-byte loads. Shifted sums S1 = sum(x - K), S2 = sum((x - K)^2), K = x[0, c, 0, 0];
//           a lane's fp32 chain ends with its plane, everything above it is fp64.
//   combine the CTA's fp64 totals go to its shared memory; after a cluster barrier every CTA of the
//           cluster reads all S totals through distributed shared memory, in rank order, and
//           derives mean / invstd itself; rank 0 writes the saved and running statistics.
//   pass 2  the planes are walked again, LAST plane first (what pass 1 read last is what L1 / L2
//           still hold), and y is written with the same head / body / tail split, since y has x's
//           layout and therefore x's alignment.
// No global scratch, no grid-wide barrier, no atomics: bit-reproducible.
#include "batch_norm.cuh"

#include <cooperative_groups.h>

#include <cstdlib>

namespace b200 {

namespace {

namespace cg = cooperative_groups;

constexpr int kThreads = 256;

// Visits the HW elements of one plane with `G` lanes (lane = 0 .. G-1, G >= 2): scalar(i, value)
// for the elements before the first and after the last 16-byte boundary, vec(i, raw) for the
// aligned 16-byte vectors in between (i = element index of the vector's first element). All loads
// of the head, of the tail and of the first eight vectors of a lane are issued before any of them
// is consumed: a small plane costs ONE round trip to memory, not one per loop iteration.
template <typename T, typename FS, typename FV>
__device__ __forceinline__ void visit_plane(const T* plane, int hw, int lane, int G, FS&& scalar, FV&& vec) {
  constexpr int V = Elem<T>::V;
  constexpr int SU = V / 2;  // head and tail hold at most V - 1 elements: V / 2 per lane when G >= 2
  constexpr int U = 8;
  const int mis = (int)((reinterpret_cast<uintptr_t>(plane) / sizeof(T)) & (V - 1));
  int head = mis ? V - mis : 0;
  if (head > hw) head = hw;
  const int nvec = (hw - head) / V;
  const int tail0 = head + nvec * V;
  T hs[SU], ts[SU];
  uint4 raw[U];
#pragma unroll
  for (int u = 0; u < SU; ++u) {
    const int i = lane + u * G;
    if (i < head) hs[u] = plane[i];
    if (tail0 + i < hw) ts[u] = plane[tail0 + i];
  }
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int v = lane + u * G;
    if (v < nvec) raw[u] = ld_keep(plane + head + v * V);
  }
#pragma unroll
  for (int u = 0; u < SU; ++u) {
    const int i = lane + u * G;
    if (i < head) scalar(i, Elem<T>::to_f32(hs[u]));
    if (tail0 + i < hw) scalar(tail0 + i, Elem<T>::to_f32(ts[u]));
  }
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int v = lane + u * G;
    if (v < nvec) vec(head + v * V, raw[u]);
  }
  for (int v0 = lane + U * G; v0 < nvec; v0 += U * G) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int v = v0 + u * G;
      if (v < nvec) raw[u] = ld_keep(plane + head + v * V);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int v = v0 + u * G;
      if (v < nvec) vec(head + v * V, raw[u]);
    }
  }
}

// CLUSTER false: one CTA per channel, launched without a cluster (grid (1, C)).
template <typename T, bool CLUSTER>
__global__ void __launch_bounds__(kThreads)
batch_norm_nchw_cluster_kernel(const BatchNormParams p, const int imgs_per_cta, const int G) {
  constexpr int V = Elem<T>::V;
  constexpr int P = V / 2;
  __shared__ double warp_tot[kThreads / 32][2];
  __shared__ double cta_tot[2];   // read by the other CTAs of the cluster
  __shared__ float stat[2];       // mean, invstd of this channel
  const int tid = threadIdx.x, lane = tid % G, grp = tid / G, groups = kThreads / G;
  const int c = blockIdx.y;
  const int hw = (int)p.spatial;
  const int n_total = (int)p.rows;
  const int n0 = (int)blockIdx.x * imgs_per_cta;
  const int n1 = n0 + imgs_per_cta < n_total ? n0 + imgs_per_cta : n_total;
  const T* x = reinterpret_cast<const T*>(p.x);
  T* y = reinterpret_cast<T*>(p.y);
  const long long plane_stride = (long long)p.channels * hw;  // between images of one channel
  const T* xc = x + (long long)c * hw;
  T* yc = y + (long long)c * hw;
#ifdef B200_BN_TIMING
  long long tmark[8];
#define B200_NMARK(i) \
  if (tid == 0) tmark[i] = clock64();
#else
#define B200_NMARK(i)
#endif
  B200_NMARK(0)
  const float shift = Elem<T>::to_f32(__ldg(xc));  // the channel's first element: every CTA of the cluster reads the same one
  const f32x2 shift2 = splat2(shift);
  // everything pass 2 and the statistics need besides x is requested now, so that it arrives
  // while pass 1 runs instead of costing a round trip of its own later
  const float w = p.weight ? load_param1(p.weight, p.w_dtype, c) : 1.f;
  const float b = p.bias ? load_param1(p.bias, p.w_dtype, c) : 0.f;
  float old_mean = 0.f, old_var = 0.f;
  if (tid == 0 && p.running_mean) {
    old_mean = __ldcg(p.running_mean + c);
    old_var = __ldcg(p.running_var + c);
  }

  // ---- pass 1 ----------------------------------------------------------------------------------
  double d1 = 0.0, d2 = 0.0;
  for (int n = n0 + grp; n < n1; n += groups) {
    const T* plane = xc + (long long)n * plane_stride;
    float s1 = 0.f, s2 = 0.f;
    f32x2 a1 = splat2(0.f), a2 = splat2(0.f);
    visit_plane<T>(
        plane, hw, lane, G,
        [&](int, float xv) {
          const float d = xv - shift;
          s1 += d;
          s2 += d * d;
        },
        [&](int, const uint4& raw) {
          f32x2 f[P];
          Pairs<T>::unpack(raw, f);
#pragma unroll
          for (int k = 0; k < P; ++k) {
            const f32x2 d = sub2(f[k], shift2);
            a1 = add2(a1, d);
            a2 = fma2(d, d, a2);
          }
        });
    d1 += (double)s1 + (double)hsum2(a1);
    d2 += (double)s2 + (double)hsum2(a2);
  }
  B200_NMARK(1)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    d1 += __shfl_xor_sync(0xffffffffu, d1, o);
    d2 += __shfl_xor_sync(0xffffffffu, d2, o);
  }
  if ((tid & 31) == 0) {
    warp_tot[tid >> 5][0] = d1;
    warp_tot[tid >> 5][1] = d2;
  }
  __syncthreads();
  B200_NMARK(2)
  if (tid == 0) {
    double t1 = 0.0, t2 = 0.0;
    for (int w = 0; w < kThreads / 32; ++w) {
      t1 += warp_tot[w][0];
      t2 += warp_tot[w][1];
    }
    cta_tot[0] = t1;
    cta_tot[1] = t2;
  }
  if constexpr (CLUSTER) {
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();  // every CTA of the cluster has published its totals
    if (tid == 0) {
      double t1 = 0.0, t2 = 0.0;
      const unsigned int nb = cluster.num_blocks();
      for (unsigned int r = 0; r < nb; ++r) {  // rank order: the same sum in every CTA
        const double* remote = cluster.map_shared_rank(cta_tot, r);
        t1 += remote[0];
        t2 += remote[1];
      }
      float mean, invstd;
      bn_channel_stats(p, c, t1, t2, shift, cluster.block_rank() == 0, &mean, &invstd, true, old_mean, old_var);
      stat[0] = mean;
      stat[1] = invstd;
    }
    cluster.sync();  // nobody leaves (and gives up its shared memory) before everyone has read it; stat[] is visible
  } else {
    if (tid == 0) {
      float mean, invstd;
      bn_channel_stats(p, c, cta_tot[0], cta_tot[1], shift, true, &mean, &invstd, true, old_mean, old_var);
      stat[0] = mean;
      stat[1] = invstd;
    }
    B200_NMARK(3)
    __syncthreads();
  }
  B200_NMARK(4)
  if (p.y == nullptr) return;

  // ---- pass 2 ----------------------------------------------------------------------------------
  const float mean = stat[0], invstd = stat[1];
  const f32x2 mean2 = splat2(mean), invstd2 = splat2(invstd), w2 = splat2(w), b2 = splat2(b);
  const bool relu = p.relu != 0;
  // the groups walk the CTA's images from the last to the first
  for (int n = n1 - 1 - grp; n >= n0; n -= groups) {
    const T* plane = xc + (long long)n * plane_stride;
    T* out = yc + (long long)n * plane_stride;
    visit_plane<T>(
        plane, hw, lane, G,
        [&](int i, float xv) {
          float o = ((xv - mean) * invstd) * w + b;
          if (relu) o = o < 0.f ? 0.f : o;
          out[i] = Elem<T>::from_f32(o);
        },
        [&](int i, const uint4& raw) {
          f32x2 f[P];
          Pairs<T>::unpack(raw, f);
#pragma unroll
          for (int k = 0; k < P; ++k) {
            f[k] = add2(mul2(mul2(sub2(f[k], mean2), invstd2), w2), b2);
            if (relu) {
              float lo, hi;
              unpack2(f[k], lo, hi);
              f[k] = pack2(lo < 0.f ? 0.f : lo, hi < 0.f ? 0.f : hi);
            }
          }
          st_stream(out + i, Pairs<T>::pack(f));
        });
  }
  B200_NMARK(5)
#ifdef B200_BN_TIMING
  if (tid == 0 && blockIdx.x == 0 && p.partials) {
    long long* log = reinterpret_cast<long long*>(p.partials) + (long long)blockIdx.y * 8;
    for (int i = 0; i < 6; ++i) log[i] = tmark[i];
  }
#endif
}

// Sum over the CTA, the same value in every thread: a shuffle tree inside each warp, one word per
// warp through shared memory, and the same tree again over those words in every warp. Fixed
// order, so the result is reproducible. `part` belongs to this call alone (32 floats).
__device__ __forceinline__ float cta_sum_all(float v, float* part, int lane, int warp, int nwarps) {
  v = warp_reduce<SumOp>(v);
  if (nwarps == 1) return v;
  if (lane == 0) part[warp] = v;
  __syncthreads();
  return warp_reduce<SumOp>(lane < nwarps ? part[lane] : 0.f);
}

// W consecutive elements of a plane, moved with one access of W * sizeof(T) bytes.
template <typename T, int W>
struct alignas(W * sizeof(T)) PlaneVec {
  T v[W];
};

// Channels of at most 16 K elements (N * H * W): the shape class of two thirds of the BatchNorm
// points of the reference's corpus (tensors of 50 KB to a few MB, where a launch is a handful of
// dependent steps and every instruction on that path counts, not bytes). A CTA per channel; a
// thread keeps its K * W elements in registers, so x is read once, and it does nothing but
//   load -> sum -> mean -> centred sum of squares -> invstd -> normalise -> store
// with two CTA-wide sums. A plane (H * W contiguous elements) is cut into vectors of W elements
// (W = 8, 4, 2 or 1, the largest that divides H * W, so that no vector crosses a plane and every
// vector is aligned); vector e of the channel belongs to thread e % blockDim (slot e / blockDim).
// The two-pass form needs no shift and keeps everything in fp32: a thread adds at most 16 terms
// and the trees above it have ten levels.
template <typename T, int K, int W>
__global__ void __launch_bounds__(1024)
batch_norm_nchw_small_kernel(const BatchNormParams p, const FastDiv vpp_div) {
  __shared__ float part[2][32];
  using Vec = PlaneVec<T, W>;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = (int)blockDim.x >> 5;
  const int c = blockIdx.x;
  const unsigned int hw = (unsigned int)p.spatial;
  const unsigned int vpp = hw / W;  // vectors per plane
  const unsigned int nvec = (unsigned int)p.rows * vpp;
  const unsigned int plane_stride = (unsigned int)p.channels * hw;  // the launcher admits < 2^31 elements in all
  const T* xc = reinterpret_cast<const T*>(p.x) + (size_t)c * hw;
  unsigned int off[K];
  Vec raw[K];
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const unsigned int e = (unsigned int)k * blockDim.x + (unsigned int)tid;
    const unsigned int n = fast_div(e, vpp_div);
    off[k] = n * plane_stride + (e - n * vpp) * W;
    if (e < nvec) raw[k] = *reinterpret_cast<const Vec*>(xc + off[k]);
  }
  // what the end of the kernel needs besides x: requested now, used after the statistics
  const float w = p.weight ? load_param1(p.weight, p.w_dtype, c) : 1.f;
  const float b = p.bias ? load_param1(p.bias, p.w_dtype, c) : 0.f;
  float old_mean = 0.f, old_var = 0.f;
  if (tid == 0 && p.running_mean) {
    old_mean = __ldcg(p.running_mean + c);
    old_var = __ldcg(p.running_var + c);
  }
  float v[K][W];
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const unsigned int e = (unsigned int)k * blockDim.x + (unsigned int)tid;
#pragma unroll
    for (int j = 0; j < W; ++j) {
      v[k][j] = e < nvec ? Elem<T>::to_f32(raw[k].v[j]) : 0.f;
      s += v[k][j];
    }
  }
  const float inv_count = (float)p.inv_count;
  const float mean = cta_sum_all(s, part[0], lane, warp, nwarps) * inv_count;
  float q = 0.f;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const unsigned int e = (unsigned int)k * blockDim.x + (unsigned int)tid;
#pragma unroll
    for (int j = 0; j < W; ++j) {
      const float d = e < nvec ? v[k][j] - mean : 0.f;
      q += d * d;
    }
  }
  const float var = cta_sum_all(q, part[1], lane, warp, nwarps) * inv_count;
  const float invstd = __frsqrt_rn(var + p.eps);
  if (tid == 0) {
    if (p.save_mean) p.save_mean[c] = mean;
    if (p.save_invstd) p.save_invstd[c] = invstd;
    if (p.running_mean) {
      p.running_mean[c] = mean * p.momentum + old_mean * p.one_minus_momentum;
      p.running_var[c] = (var * p.unbias) * p.momentum + old_var * p.one_minus_momentum;
    }
  }
  if (p.y == nullptr) return;
  T* yc = reinterpret_cast<T*>(p.y) + (size_t)c * hw;
  const bool relu = p.relu != 0;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const unsigned int e = (unsigned int)k * blockDim.x + (unsigned int)tid;
    Vec out;
#pragma unroll
    for (int j = 0; j < W; ++j) {
      float o = ((v[k][j] - mean) * invstd) * w + b;
      if (relu) o = o < 0.f ? 0.f : o;
      out.v[j] = Elem<T>::from_f32(o);
    }
    if (e < nvec) *reinterpret_cast<Vec*>(yc + off[k]) = out;
  }
}

// At most 16 elements per thread; as few vectors per thread as 512 threads allow (1024 threads for
// the largest channels).
template <typename T, int W>
static void launch_small(const BatchNormParams& p, cudaStream_t st) {
  const long long nvec = p.rows * p.spatial / W;
  constexpr int KMAX = 16 / W;
  int K = 1;
  while (K < KMAX && nvec > 512LL * K) K *= 2;
  int threads = (int)((nvec + K - 1) / K);
  threads = (threads + 31) / 32 * 32;
  const FastDiv d = make_fast_div(p.spatial / W);
  const unsigned grid = (unsigned)p.channels;
  if (K == 1) batch_norm_nchw_small_kernel<T, 1, W><<<grid, threads, 0, st>>>(p, d);
  if constexpr (KMAX >= 2) if (K == 2) batch_norm_nchw_small_kernel<T, 2, W><<<grid, threads, 0, st>>>(p, d);
  if constexpr (KMAX >= 4) if (K == 4) batch_norm_nchw_small_kernel<T, 4, W><<<grid, threads, 0, st>>>(p, d);
  if constexpr (KMAX >= 8) if (K == 8) batch_norm_nchw_small_kernel<T, 8, W><<<grid, threads, 0, st>>>(p, d);
  if constexpr (KMAX >= 16) if (K == 16) batch_norm_nchw_small_kernel<T, 16, W><<<grid, threads, 0, st>>>(p, d);
}

}  // namespace

template <typename T>
bool try_launch_batch_norm_nchw(const BatchNormParams& p, cudaStream_t st, int* rc) {
  static const bool off = [] {
    const char* e = getenv("B200_BN_NO_NCHW_CLUSTER");
    return e && e[0] == '1';
  }();
  if (off) return false;
  // contiguous NCHW only: planes of `spatial` contiguous elements, channel after channel
  if (p.ss != 1 || p.sc != p.spatial || p.sn != (long long)p.channels * p.spatial) return false;
  if (p.rows < 1 || p.rows > 0x7fffffffLL || p.spatial < 1 || p.spatial > 0x3fffffffLL || p.channels > 65535) return false;
  const DeviceInfo& dev = device_info();
  const long long plane_vecs = (p.spatial * (long long)sizeof(T) + 15) / 16;
  // measurement switch: B200_BN_NCHW_FORCE=cta|cluster|registers picks the variant whatever the shape
  static const int force = [] {
    const char* e = getenv("B200_BN_NCHW_FORCE");
    if (!e) return 0;
    return e[0] == 'c' && e[1] == 't' ? 2 : (e[0] == 'c' ? 3 : (e[0] == 'r' ? 4 : 0));
  }();
  // channels of at most 16 K elements: the register-resident kernel, as few elements per thread as
  // 512 threads allow (1024 threads for the largest channels)
  {
    const long long elems = p.rows * p.spatial;
    const long long total = elems * p.channels;
    if ((force == 0 || force == 4) && elems <= 16384 && total < 0x7fffffffLL) {
      constexpr int WMAX = 16 / (int)sizeof(T);  // elements of a 16-byte access
      int W = WMAX;
      while (W > 1 && (p.spatial % W != 0 || reinterpret_cast<uintptr_t>(p.x) % (W * sizeof(T)) != 0 ||
                       reinterpret_cast<uintptr_t>(p.y) % (W * sizeof(T)) != 0))
        W /= 2;
      if (W == 8) { if constexpr (WMAX >= 8) launch_small<T, 8>(p, st); }
      else if (W == 4) launch_small<T, 4>(p, st);
      else if (W == 2) launch_small<T, 2>(p, st);
      else launch_small<T, 1>(p, st);
      *rc = launch_status("b200_batch_norm_fwd [NCHW, one launch, CTA per channel, channel in registers]");
      return true;
    }
  }
  // cluster size: enough CTAs to fill the machine twice over, at most 8 per channel, at most one per image
  // Several CTAs per channel (a cluster) only pay when a channel holds enough data to keep them
  // busy: launching clusters costs more than launching plain CTAs, and for channels of a few tens of
  // KB one CTA per channel was measured faster even when the channels do not fill the machine.
  int S = 1;
  if (p.rows * p.spatial * (long long)sizeof(T) >= 128 * 1024)
    while (S < 8 && (long long)p.channels * S < 2LL * dev.sm_count && 2 * S <= p.rows) S *= 2;
  if (force == 2) S = 1;
  if (force == 3 && S == 1 && p.rows >= 2) S = 2;
  const int ipc = (int)((p.rows + S - 1) / S);  // a CTA whose range starts beyond the last image simply has no planes
  // Lanes per plane. Few lanes per plane mean many planes in flight per CTA (a group walks its
  // planes one after the other, each a round trip to memory), many lanes mean few vectors per lane
  // and round: as few lanes as give every plane of the CTA its own group, but enough that a lane
  // holds at most eight vectors of a plane.
  int G = 32;
  while (G > 2 && kThreads / (G / 2) <= 2 * ipc && plane_vecs <= 8LL * (G / 2)) G /= 2;
  if (S == 1) {
    batch_norm_nchw_cluster_kernel<T, false><<<dim3(1, (unsigned)p.channels, 1), kThreads, 0, st>>>(p, ipc, G);
    *rc = launch_status("b200_batch_norm_fwd [NCHW, one launch, CTA per channel]");
    return true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)S, (unsigned)p.channels, 1);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)S;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, batch_norm_nchw_cluster_kernel<T, true>, p, ipc, G);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return false;  // the cluster launch was refused: the caller takes the three-launch path
  }
  *rc = launch_status("b200_batch_norm_fwd [NCHW, one launch, cluster per channel, DSMEM combine]");
  return true;
}

template bool try_launch_batch_norm_nchw<float>(const BatchNormParams&, cudaStream_t, int*);
template bool try_launch_batch_norm_nchw<__nv_bfloat16>(const BatchNormParams&, cudaStream_t, int*);
template bool try_launch_batch_norm_nchw<__half>(const BatchNormParams&, cudaStream_t, int*);

}  // namespace b200
