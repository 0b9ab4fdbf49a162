// BatchNorm2d training backward: per-channel sums of dy and dy * (x - mean), then
//   dx = ((dy - (x - mean) * k) - sum_dy / N) * (invstd * w),   k = (dot / N) * invstd^2
//   dweight = dot * invstd,   dbias = sum_dy
// with an optional activation-backward prologue on dy (leaky ReLU with a given slope; slope 0 is
// ReLU): dy' = act > 0 ? dy : dy * slope, rounded to the tensor dtype as the captured graphs do.
//
// Replaces the Triton plans of the BatchNorm-backward repros of the reference
// (repros/canonical/sum_sum_183b124c731f/oracle.py: per-channel partial sums, finalize, apply;
// repros/canonical/sum_sum_12fc8ebf8180/oracle.py: the same behind a leaky-ReLU backward).
// Evaluation order as in the decomposed aten graph (sum_sum_183b124c731f/repro.py:26-50):
//   sum_dy = sum(float(dy'));  dot = sum(float(dy') * (float(x) - mean))
//   c1 = sum_dy * (1/N);  c2 = (dot * (1/N)) * (invstd * invstd);  gs = invstd * w
//   dx = cast(((float(dy') - (float(x) - mean) * c2) - c1) * gs)
//
// Three launches: sums (a thread's own short chain in fp32, everything above it in fp64; per-CTA
// partials over a fixed split of the rows), finalize (fixed order, coefficient table), apply (each
// CTA walks its part of the rows backwards, so that it starts in what the sums pass left in L2).
// No atomics: bit-reproducible.
// Channels-last tensors whose channel count is a multiple of the 16-byte vector (at most 256
// vectors per row) take the vector kernels; every other layout the strided element-wise ones.
#include "rowwise.cuh"

#include <cooperative_groups.h>

#include <cstdlib>

namespace b200 {

struct BnBwdParams {
  const void* dy;
  const void* x;
  const void* act;     // may be null: no prologue
  const float* mean;   // [C]
  const float* invstd; // [C]
  const void* weight;  // may be null (ones)
  int w_dtype;
  void* dx;            // may be null: sums only
  float* dweight;      // may be null
  float* dbias;        // may be null
  long long rows;      // channels-last: N*H*W; general: N
  long long spatial;   // general: H*W
  long long sn, sc, ss;  // general: element strides of (n, c, spatial), shared by dy, x, act, dx
  int channels;
  float slope;
  float inv_count;     // 1 / (N*H*W)
  double* partials;    // [splits][2][C]: everything above a thread's own short fp32 chain is fp64
  float* coef;         // [4][C]: c1, c2, gs, mean
  int splits;
};

template <typename T>
__device__ __forceinline__ void bn_bwd_prologue(f32x2 (&g)[Elem<T>::V / 2], const uint4& act_raw, float slope) {
  constexpr int V = Elem<T>::V;
  f32x2 a[V / 2];
  Pairs<T>::unpack(act_raw, a);
  f32x2 scaled[V / 2];
#pragma unroll
  for (int i = 0; i < V / 2; ++i) scaled[i] = mul2(g[i], splat2(slope));
#pragma unroll
  for (int i = 0; i < V / 2; ++i) {
    float a0, a1, g0, g1, s0, s1;
    unpack2(a[i], a0, a1);
    unpack2(g[i], g0, g1);
    unpack2(scaled[i], s0, s1);
    g[i] = pack2(a0 > 0.f ? g0 : s0, a1 > 0.f ? g1 : s1);
  }
  if constexpr (sizeof(T) == 2) {  // the graph rounds dy' to the tensor dtype before it is used
    const uint4 r = Pairs<T>::pack(g);
    Pairs<T>::unpack(r, g);
  }
}

// Channels-last sums: the tensors are flat [rows * C] arrays of 16-byte vectors, whatever C is. A
// vector may straddle the end of a row; the pattern of channels under a vector repeats every
// PV = C / gcd(C, V) vectors: vector i has phase i % PV and its element j belongs to channel
// (phase * V + j) % C. blockDim.x and the CTA's range [b*per, (b+1)*per) are multiples of PV, so a
// thread keeps its phase - its V channels - for the whole launch.
template <typename T>
__global__ void __launch_bounds__(256) bn_bwd_sums_cl_kernel(const BnBwdParams p, long long vecs_per_cta, int PV) {
  constexpr int V = Elem<T>::V;
  __shared__ float red[2 * 256 * 8 / 8 * 8];  // [2][threads][V] fp32, V <= 8
  const int tid = threadIdx.x, T_ = blockDim.x, C = p.channels;
  const int ph = tid % PV;
  const long long total = p.rows * C / V;
  const long long v0 = (long long)blockIdx.x * vecs_per_cta;
  long long v1 = v0 + vecs_per_cta;
  if (v1 > total) v1 = total;
  const uint4* dy = reinterpret_cast<const uint4*>(p.dy);
  const uint4* x = reinterpret_cast<const uint4*>(p.x);
  const uint4* act = reinterpret_cast<const uint4*>(p.act);
  f32x2 mean2[V / 2], s1[V / 2], s2[V / 2];
#pragma unroll
  for (int i = 0; i < V / 2; ++i) {
    mean2[i] = pack2(__ldg(p.mean + (ph * V + 2 * i) % C), __ldg(p.mean + (ph * V + 2 * i + 1) % C));
    s1[i] = s2[i] = splat2(0.f);
  }
  constexpr int U = 4;  // vectors of each tensor in flight per thread
  for (long long v = v0 + tid; v < v1; v += (long long)U * T_) {
    uint4 rg[U], rx[U], ra[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = v + (long long)u * T_;
      if (i < v1) {
        rg[u] = ld_stream(reinterpret_cast<const T*>(dy + i));
        rx[u] = ld_stream(reinterpret_cast<const T*>(x + i));
        if (act) ra[u] = ld_stream(reinterpret_cast<const T*>(act + i));
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (v + (long long)u * T_ < v1) {
        f32x2 g[V / 2], xv[V / 2];
        Pairs<T>::unpack(rg[u], g);
        Pairs<T>::unpack(rx[u], xv);
        if (act) bn_bwd_prologue<T>(g, ra[u], p.slope);
#pragma unroll
        for (int i = 0; i < V / 2; ++i) {
          s1[i] = add2(s1[i], g[i]);
          s2[i] = add2(s2[i], mul2(g[i], sub2(xv[i], mean2[i])));
        }
      }
    }
  }
  // fold the threads of a column (tid, tid + vpr, ...) in a fixed order
  float* r1 = red;
  float* r2 = red + 256 * V;
#pragma unroll
  for (int i = 0; i < V / 2; ++i) {
    unpack2(s1[i], r1[tid * V + 2 * i], r1[tid * V + 2 * i + 1]);
    unpack2(s2[i], r2[tid * V + 2 * i], r2[tid * V + 2 * i + 1]);
  }
  __syncthreads();
  const int period = PV * V;  // elements; a multiple of C
  for (int c = tid; c < p.channels; c += T_) {
    double a = 0.0, b = 0.0;
    for (int idx = c; idx < period; idx += C) {  // every (phase, element) that lands on channel c
      const int col = idx / V, e = idx % V;
      for (int t = col; t < T_; t += PV) {
        a += (double)r1[t * V + e];
        b += (double)r2[t * V + e];
      }
    }
    p.partials[((long long)blockIdx.x * 2) * p.channels + c] = a;
    p.partials[((long long)blockIdx.x * 2 + 1) * p.channels + c] = b;
  }
}

// One CTA per channel: the partials are read with every thread (all loads of a thread are in
// flight together), combined in fp64 in a fixed order; thread 0 writes the outputs and the
// coefficient table.
__global__ void __launch_bounds__(256) bn_bwd_finalize_kernel(const BnBwdParams p) {
  __shared__ double red[2][8];
  const int c = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // what thread 0 needs after the sums: requested now, so that it does not cost a round trip then
  float invstd = 0.f, w = 1.f, mean = 0.f;
  if (tid == 0) {
    invstd = __ldg(p.invstd + c);
    mean = __ldg(p.mean + c);
    if (p.weight) w = load_param1(p.weight, p.w_dtype, c);
  }
  double s1 = 0.0, s2 = 0.0;
  for (int g0 = tid; g0 < p.splits; g0 += 256 * 4) {
    double a[4], b[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int g = g0 + u * 256;
      a[u] = g < p.splits ? p.partials[((long long)g * 2) * p.channels + c] : 0.0;
      b[u] = g < p.splits ? p.partials[((long long)g * 2 + 1) * p.channels + c] : 0.0;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      s1 += a[u];
      s2 += b[u];
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s1 += __shfl_xor_sync(0xffffffffu, s1, o);
    s2 += __shfl_xor_sync(0xffffffffu, s2, o);
  }
  if (lane == 0) {
    red[0][warp] = s1;
    red[1][warp] = s2;
  }
  __syncthreads();
  if (tid == 0) {
    s1 = s2 = 0.0;
    for (int w = 0; w < 8; ++w) {
      s1 += red[0][w];
      s2 += red[1][w];
    }
    const float sum_dy = (float)s1, dot = (float)s2;
    if (p.dbias) p.dbias[c] = sum_dy;
    if (p.dweight) p.dweight[c] = dot * invstd;
    p.coef[c] = sum_dy * p.inv_count;
    p.coef[p.channels + c] = (dot * p.inv_count) * (invstd * invstd);
    p.coef[2 * p.channels + c] = invstd * w;
    p.coef[3 * p.channels + c] = mean;
  }
}

// Apply pass. CTA b takes the same vectors [b*per, (b+1)*per) as in the sums pass but walks them
// from the end to the start: what the sums pass read last is what is still in L2, so the first
// part of this pass is served from there instead of DRAM (the two inputs together are larger than
// the L2, so walking forward again would find nothing). blockDim.x and `per` are multiples of vpr,
// so a thread stays in one vector column here too.
template <typename T>
__global__ void __launch_bounds__(256) bn_bwd_apply_cl_kernel(const BnBwdParams p, long long vecs_per_cta, int PV) {
  constexpr int V = Elem<T>::V;
  const int tid = threadIdx.x, T_ = blockDim.x, C = p.channels;
  const int ph = PV - 1 - tid % PV;  // the range ends on a multiple of PV: its last vector has phase PV - 1
  const long long total = p.rows * C / V;
  const long long v0 = (long long)blockIdx.x * vecs_per_cta;
  long long v1 = v0 + vecs_per_cta;
  if (v1 > total) v1 = total;
  const uint4* dy = reinterpret_cast<const uint4*>(p.dy);
  const uint4* x = reinterpret_cast<const uint4*>(p.x);
  const uint4* act = reinterpret_cast<const uint4*>(p.act);
  uint4* dx = reinterpret_cast<uint4*>(p.dx);
  f32x2 c1[V / 2], c2[V / 2], gs[V / 2], mean2[V / 2];
#pragma unroll
  for (int i = 0; i < V / 2; ++i) {
    const int c = (ph * V + 2 * i) % C, d = (ph * V + 2 * i + 1) % C;
    c1[i] = pack2(p.coef[c], p.coef[d]);
    c2[i] = pack2(p.coef[C + c], p.coef[C + d]);
    gs[i] = pack2(p.coef[2 * C + c], p.coef[2 * C + d]);
    mean2[i] = pack2(p.coef[3 * C + c], p.coef[3 * C + d]);
  }
  constexpr int U = 4;
  for (long long v = v1 - 1 - tid; v >= v0; v -= (long long)U * T_) {
    uint4 rg[U], rx[U], ra[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = v - (long long)u * T_;
      if (i >= v0) {
        rg[u] = ld_stream(reinterpret_cast<const T*>(dy + i));
        rx[u] = ld_stream(reinterpret_cast<const T*>(x + i));
        if (act) ra[u] = ld_stream(reinterpret_cast<const T*>(act + i));
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = v - (long long)u * T_;
      if (i >= v0) {
        f32x2 g[V / 2], xv[V / 2], o[V / 2];
        Pairs<T>::unpack(rg[u], g);
        Pairs<T>::unpack(rx[u], xv);
        if (act) bn_bwd_prologue<T>(g, ra[u], p.slope);
#pragma unroll
        for (int k = 0; k < V / 2; ++k)
          o[k] = mul2(sub2(sub2(g[k], mul2(sub2(xv[k], mean2[k]), c2[k])), c1[k]), gs[k]);
        st_stream(reinterpret_cast<T*>(dx + i), Pairs<T>::pack(o));
      }
    }
  }
}

// ---- general layout: element-wise, (n, c, s) strides ------------------------------------------
template <typename T>
__device__ __forceinline__ float bn_bwd_dy_general(const BnBwdParams& p, long long off) {
  float g = Elem<T>::to_f32(reinterpret_cast<const T*>(p.dy)[off]);
  if (p.act) {
    const float a = Elem<T>::to_f32(reinterpret_cast<const T*>(p.act)[off]);
    g = a > 0.f ? g : g * p.slope;
    g = Elem<T>::to_f32(Elem<T>::from_f32(g));
  }
  return g;
}

template <typename T>
__global__ void __launch_bounds__(256) bn_bwd_sums_general_kernel(const BnBwdParams p) {
  __shared__ double red[2][8];
  const int c = blockIdx.x;
  const long long total = p.rows * p.spatial;
  const long long per = (total + gridDim.y - 1) / gridDim.y;
  const long long e0 = (long long)blockIdx.y * per;
  const long long e1 = e0 + per < total ? e0 + per : total;
  const float mean = p.mean[c];
  float s1 = 0.f, s2 = 0.f;
  for (long long e = e0 + threadIdx.x; e < e1; e += blockDim.x) {
    const long long n = e / p.spatial, s = e % p.spatial;
    const long long off = n * p.sn + (long long)c * p.sc + s * p.ss;
    const float g = bn_bwd_dy_general<T>(p, off);
    s1 += g;
    s2 += g * (Elem<T>::to_f32(reinterpret_cast<const T*>(p.x)[off]) - mean);
  }
  double d1 = (double)s1, d2 = (double)s2;  // the threads' short chains are combined in fp64
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    d1 += __shfl_xor_sync(0xffffffffu, d1, o);
    d2 += __shfl_xor_sync(0xffffffffu, d2, o);
  }
  if ((threadIdx.x & 31) == 0) {
    red[0][threadIdx.x >> 5] = d1;
    red[1][threadIdx.x >> 5] = d2;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    d1 = d2 = 0.0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) {
      d1 += red[0][w];
      d2 += red[1][w];
    }
    p.partials[((long long)blockIdx.y * 2) * p.channels + c] = d1;
    p.partials[((long long)blockIdx.y * 2 + 1) * p.channels + c] = d2;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) bn_bwd_apply_general_kernel(const BnBwdParams p) {
  const int c = blockIdx.x;
  const long long total = p.rows * p.spatial;
  const long long per = (total + gridDim.y - 1) / gridDim.y;
  const long long e0 = (long long)blockIdx.y * per;
  const long long e1 = e0 + per < total ? e0 + per : total;
  const float c1 = p.coef[c], c2 = p.coef[p.channels + c], gs = p.coef[2 * p.channels + c], mean = p.coef[3 * p.channels + c];
  for (long long e = e0 + threadIdx.x; e < e1; e += blockDim.x) {
    const long long n = e / p.spatial, s = e % p.spatial;
    const long long off = n * p.sn + (long long)c * p.sc + s * p.ss;
    const float g = bn_bwd_dy_general<T>(p, off);
    const float xv = Elem<T>::to_f32(reinterpret_cast<const T*>(p.x)[off]);
    reinterpret_cast<T*>(p.dx)[off] = Elem<T>::from_f32(((g - (xv - mean) * c2) - c1) * gs);
  }
}

// ---- contiguous NCHW: one launch, a cluster of CTAs per channel ---------------------------------
// grid (S, C), cluster (S, 1, 1): CTA (s, c) owns images [s * ipc, (s + 1) * ipc) of channel c. A
// plane (the H*W contiguous elements of one image and channel) is walked by a group of G lanes: the
// unaligned head and tail element by element, the body with 16-byte accesses (dy, x, act and dx
// share the layout, hence the alignment); all loads of the head, the tail and the first four body
// vectors of a lane are issued before any is consumed, so a small plane costs one round trip to
// memory. Pass 1 sums dy' and dy' * (x - mean); the CTA totals (fp64) are exchanged through
// distributed shared memory after a cluster barrier and every CTA derives the coefficients itself;
// pass 2 walks the planes backwards (what was read last is still cached) and writes dx. No scratch,
// no atomics.
template <typename T, bool HAS_ACT, typename FS, typename FV>
__device__ __forceinline__ void bn_bwd_visit_plane(const T* dyp, const T* xp, const T* ap, int hw, int lane, int G,
                                                   float slope, FS&& scalar, FV&& vec) {
  constexpr int V = Elem<T>::V;
  constexpr int P = V / 2;
  constexpr int SU = V / 2;  // head and tail hold at most V - 1 elements: V / 2 per lane when G >= 2
  constexpr int U = 4;
  const int mis = (int)((reinterpret_cast<uintptr_t>(xp) / sizeof(T)) & (V - 1));
  int head = mis ? V - mis : 0;
  if (head > hw) head = hw;
  const int nvec = (hw - head) / V;
  const int tail0 = head + nvec * V;
  T sg[2 * SU], sx[2 * SU], sa[2 * SU];
  uint4 rg[U], rx[U], ra[U];
  auto sidx = [&](int u) { return u < SU ? lane + u * G : tail0 + lane + (u - SU) * G; };
  auto slive = [&](int u) { return u < SU ? lane + u * G < head : tail0 + lane + (u - SU) * G < hw; };
#pragma unroll
  for (int u = 0; u < 2 * SU; ++u) {
    if (slive(u)) {
      const int i = sidx(u);
      sg[u] = dyp[i];
      sx[u] = xp[i];
      if constexpr (HAS_ACT) sa[u] = ap[i];
    }
  }
  auto load_batch = [&](int v0) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int v = v0 + u * G;
      if (v < nvec) {
        rg[u] = ld_keep(dyp + head + v * V);
        rx[u] = ld_keep(xp + head + v * V);
        if constexpr (HAS_ACT) ra[u] = ld_keep(ap + head + v * V);
      }
    }
  };
  auto use_batch = [&](int v0) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int v = v0 + u * G;
      if (v < nvec) {
        f32x2 g[P], xv[P];
        Pairs<T>::unpack(rg[u], g);
        Pairs<T>::unpack(rx[u], xv);
        if constexpr (HAS_ACT) bn_bwd_prologue<T>(g, ra[u], slope);
        vec(head + v * V, g, xv);
      }
    }
  };
  load_batch(lane);
#pragma unroll
  for (int u = 0; u < 2 * SU; ++u) {
    if (slive(u)) {
      float g = Elem<T>::to_f32(sg[u]);
      if constexpr (HAS_ACT) {
        g = Elem<T>::to_f32(sa[u]) > 0.f ? g : g * slope;
        g = Elem<T>::to_f32(Elem<T>::from_f32(g));  // the graph rounds dy' to the tensor dtype
      }
      scalar(sidx(u), g, Elem<T>::to_f32(sx[u]));
    }
  }
  use_batch(lane);
  for (int v0 = lane + U * G; v0 < nvec; v0 += U * G) {
    load_batch(v0);
    use_batch(v0);
  }
}

// CLUSTER false: one CTA per channel, launched without a cluster (grid (1, C)).
template <typename T, bool HAS_ACT, bool CLUSTER>
__global__ void __launch_bounds__(256)
bn_bwd_nchw_cluster_kernel(const BnBwdParams p, const int imgs_per_cta, const int G) {
  namespace cg = cooperative_groups;
  constexpr int V = Elem<T>::V;
  constexpr int P = V / 2;
  __shared__ double warp_tot[8][2];
  __shared__ double cta_tot[2];  // read by the other CTAs of the cluster
  __shared__ float coef[2];      // c1, c2 of this channel
  const int tid = threadIdx.x, lane = tid % G, grp = tid / G, groups = 256 / G;
  const int c = blockIdx.y;
  const int hw = (int)p.spatial;
  const int n_total = (int)p.rows;
  const int n0 = (int)blockIdx.x * imgs_per_cta;
  const int n1 = n0 + imgs_per_cta < n_total ? n0 + imgs_per_cta : n_total;
  const long long plane_stride = (long long)p.channels * hw;
  const T* dyc = reinterpret_cast<const T*>(p.dy) + (long long)c * hw;
  const T* xc = reinterpret_cast<const T*>(p.x) + (long long)c * hw;
  const T* actc = HAS_ACT ? reinterpret_cast<const T*>(p.act) + (long long)c * hw : nullptr;
  T* dxc = p.dx ? reinterpret_cast<T*>(p.dx) + (long long)c * hw : nullptr;
  const float mean = __ldg(p.mean + c);
  const f32x2 mean2 = splat2(mean);
  const float slope = p.slope;
  const float invstd = __ldg(p.invstd + c);  // needed after the sums: requested now
  const float w = p.weight ? load_param1(p.weight, p.w_dtype, c) : 1.f;

  // ---- pass 1 ----------------------------------------------------------------------------------
  double d1 = 0.0, d2 = 0.0;
  for (int n = n0 + grp; n < n1; n += groups) {
    const long long off = (long long)n * plane_stride;
    float s1 = 0.f, s2 = 0.f;
    f32x2 a1 = splat2(0.f), a2 = splat2(0.f);
    bn_bwd_visit_plane<T, HAS_ACT>(
        dyc + off, xc + off, HAS_ACT ? actc + off : nullptr, hw, lane, G, slope,
        [&](int, float g, float xv) {
          s1 += g;
          s2 += g * (xv - mean);
        },
        [&](int, const f32x2 (&g)[P], const f32x2 (&xv)[P]) {
#pragma unroll
          for (int k = 0; k < P; ++k) {
            a1 = add2(a1, g[k]);
            a2 = add2(a2, mul2(g[k], sub2(xv[k], mean2)));
          }
        });
    d1 += (double)s1 + (double)hsum2(a1);
    d2 += (double)s2 + (double)hsum2(a2);
  }
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
  if (tid == 0) {
    double t1 = 0.0, t2 = 0.0;
    for (int w = 0; w < 8; ++w) {
      t1 += warp_tot[w][0];
      t2 += warp_tot[w][1];
    }
    cta_tot[0] = t1;
    cta_tot[1] = t2;
  }
  bool first = true;  // this CTA writes the channel's global outputs
  if constexpr (CLUSTER) {
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();  // every CTA of the cluster has published its totals
    first = cluster.block_rank() == 0;
    if (tid == 0) {
      double t1 = 0.0, t2 = 0.0;
      const unsigned int nb = cluster.num_blocks();
      for (unsigned int r = 0; r < nb; ++r) {  // rank order: the same sums in every CTA
        const double* remote = cluster.map_shared_rank(cta_tot, r);
        t1 += remote[0];
        t2 += remote[1];
      }
      coef[0] = (float)t1;
      coef[1] = (float)t2;
    }
    cluster.sync();  // nobody leaves before its totals were read
  } else {
    if (tid == 0) {
      coef[0] = (float)cta_tot[0];
      coef[1] = (float)cta_tot[1];
    }
    __syncthreads();
  }
  const float sum_dy = coef[0], dot = coef[1];
  if (first && tid == 0) {
    if (p.dbias) p.dbias[c] = sum_dy;
    if (p.dweight) p.dweight[c] = dot * invstd;
  }
  if (dxc == nullptr) return;

  // ---- pass 2 ----------------------------------------------------------------------------------
  const float c1 = sum_dy * p.inv_count, c2 = (dot * p.inv_count) * (invstd * invstd), gs = invstd * w;
  const f32x2 c1v = splat2(c1), c2v = splat2(c2), gsv = splat2(gs);
  for (int n = n1 - 1 - grp; n >= n0; n -= groups) {
    const long long off = (long long)n * plane_stride;
    T* out = dxc + off;
    bn_bwd_visit_plane<T, HAS_ACT>(
        dyc + off, xc + off, HAS_ACT ? actc + off : nullptr, hw, lane, G, slope,
        [&](int i, float g, float xv) { out[i] = Elem<T>::from_f32(((g - (xv - mean) * c2) - c1) * gs); },
        [&](int i, const f32x2 (&g)[P], const f32x2 (&xv)[P]) {
          f32x2 o[P];
#pragma unroll
          for (int k = 0; k < P; ++k)
            o[k] = mul2(sub2(sub2(g[k], mul2(sub2(xv[k], mean2), c2v)), c1v), gsv);
          st_stream(out + i, Pairs<T>::pack(o));
        });
  }
}

// ---- contiguous NCHW, channels of at most 8 K elements: the channel in registers ----------------
// A CTA per channel; a thread keeps its K * W elements of dy (after the activation prologue) and of
// x in registers, so both are read once, and the launch is load -> two sums -> coefficients -> dx.
// A plane (H * W contiguous elements) is cut into vectors of W elements (the largest of 8, 4, 2, 1
// that divides H * W: no vector crosses a plane, every vector is aligned); vector e of the channel
// belongs to thread e % blockDim, slot e / blockDim. For tensors of a few hundred KB a launch is a
// handful of dependent steps, and what counts is how few instructions lie on that path, not bytes.
// Both sums go through one pair of shuffle trees (fixed order, fp32: a thread adds at most 8 terms
// and the trees above it have ten levels).
template <typename T, int W>
struct alignas(W * sizeof(T)) BwdPlaneVec {
  T v[W];
};

template <typename T, int K, int W, bool HAS_ACT>
__global__ void __launch_bounds__(1024) bn_bwd_nchw_small_kernel(const BnBwdParams p, const FastDiv vpp_div) {
  __shared__ float part[2][32];
  using Vec = BwdPlaneVec<T, W>;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = (int)blockDim.x >> 5;
  const int c = blockIdx.x;
  const unsigned int hw = (unsigned int)p.spatial;
  const unsigned int vpp = hw / W;  // vectors per plane
  const unsigned int nvec = (unsigned int)p.rows * vpp;
  const unsigned int plane_stride = (unsigned int)p.channels * hw;  // the launcher admits < 2^31 elements in all
  const size_t base = (size_t)c * hw;
  const T* dyc = reinterpret_cast<const T*>(p.dy) + base;
  const T* xc = reinterpret_cast<const T*>(p.x) + base;
  const T* actc = HAS_ACT ? reinterpret_cast<const T*>(p.act) + base : nullptr;
  unsigned int off[K];
  Vec g_raw[K], x_raw[K], a_raw[HAS_ACT ? K : 1];
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const unsigned int e = (unsigned int)k * blockDim.x + (unsigned int)tid;
    const unsigned int n = fast_div(e, vpp_div);
    off[k] = n * plane_stride + (e - n * vpp) * W;
    if (e < nvec) {
      g_raw[k] = *reinterpret_cast<const Vec*>(dyc + off[k]);
      x_raw[k] = *reinterpret_cast<const Vec*>(xc + off[k]);
      if constexpr (HAS_ACT) a_raw[k] = *reinterpret_cast<const Vec*>(actc + off[k]);
    }
  }
  const float mean = __ldg(p.mean + c);
  const float invstd = __ldg(p.invstd + c);
  const float w = p.weight ? load_param1(p.weight, p.w_dtype, c) : 1.f;
  float g[K][W], xm[K][W];
  float s1 = 0.f, s2 = 0.f;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const unsigned int e = (unsigned int)k * blockDim.x + (unsigned int)tid;
#pragma unroll
    for (int j = 0; j < W; ++j) {
      g[k][j] = 0.f;
      xm[k][j] = 0.f;
      if (e < nvec) {
        float gv = Elem<T>::to_f32(g_raw[k].v[j]);
        if constexpr (HAS_ACT) {
          gv = Elem<T>::to_f32(a_raw[k].v[j]) > 0.f ? gv : gv * p.slope;
          gv = Elem<T>::to_f32(Elem<T>::from_f32(gv));  // the graph rounds dy' to the tensor dtype
        }
        g[k][j] = gv;
        xm[k][j] = Elem<T>::to_f32(x_raw[k].v[j]) - mean;
      }
      s1 += g[k][j];
      s2 += g[k][j] * xm[k][j];
    }
  }
  s1 = warp_reduce<SumOp>(s1);
  s2 = warp_reduce<SumOp>(s2);
  if (nwarps > 1) {
    if (lane == 0) {
      part[0][warp] = s1;
      part[1][warp] = s2;
    }
    __syncthreads();
    s1 = warp_reduce<SumOp>(lane < nwarps ? part[0][lane] : 0.f);
    s2 = warp_reduce<SumOp>(lane < nwarps ? part[1][lane] : 0.f);
  }
  if (tid == 0) {
    if (p.dbias) p.dbias[c] = s1;
    if (p.dweight) p.dweight[c] = s2 * invstd;
  }
  if (p.dx == nullptr) return;
  const float c1 = s1 * p.inv_count, c2 = (s2 * p.inv_count) * (invstd * invstd), gs = invstd * w;
  T* dxc = reinterpret_cast<T*>(p.dx) + base;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const unsigned int e = (unsigned int)k * blockDim.x + (unsigned int)tid;
    Vec out;
#pragma unroll
    for (int j = 0; j < W; ++j) out.v[j] = Elem<T>::from_f32(((g[k][j] - xm[k][j] * c2) - c1) * gs);
    if (e < nvec) *reinterpret_cast<Vec*>(dxc + off[k]) = out;
  }
}

template <typename T, int K, int W>
static void launch_bn_bwd_small_k(const BnBwdParams& p, int threads, const FastDiv& d, cudaStream_t st) {
  if (p.act) bn_bwd_nchw_small_kernel<T, K, W, true><<<(unsigned)p.channels, threads, 0, st>>>(p, d);
  else bn_bwd_nchw_small_kernel<T, K, W, false><<<(unsigned)p.channels, threads, 0, st>>>(p, d);
}

// At most 8 elements of each tensor per thread; as few vectors per thread as 512 threads allow.
template <typename T, int W>
static void launch_bn_bwd_small(const BnBwdParams& p, cudaStream_t st) {
  const long long nvec = p.rows * p.spatial / W;
  constexpr int KMAX = 8 / W;
  int K = 1;
  while (K < KMAX && nvec > 512LL * K) K *= 2;
  int threads = (int)((nvec + K - 1) / K);
  threads = (threads + 31) / 32 * 32;
  const FastDiv d = make_fast_div(p.spatial / W);
  if (K == 1) launch_bn_bwd_small_k<T, 1, W>(p, threads, d, st);
  if constexpr (KMAX >= 2) if (K == 2) launch_bn_bwd_small_k<T, 2, W>(p, threads, d, st);
  if constexpr (KMAX >= 4) if (K == 4) launch_bn_bwd_small_k<T, 4, W>(p, threads, d, st);
  if constexpr (KMAX >= 8) if (K == 8) launch_bn_bwd_small_k<T, 8, W>(p, threads, d, st);
}

template <typename T>
static bool try_launch_bn_bwd_nchw(const BnBwdParams& p, cudaStream_t st, int* rc) {
  static const bool off = [] {
    const char* e = getenv("B200_BN_NO_NCHW_CLUSTER");
    return e && e[0] == '1';
  }();
  if (off) return false;
  if (p.ss != 1 || p.sc != p.spatial || p.sn != (long long)p.channels * p.spatial) return false;
  if (p.rows < 1 || p.rows > 0x7fffffffLL || p.spatial < 1 || p.spatial > 0x3fffffffLL || p.channels > 65535) return false;
  if (!aligned16(p.dy) || !aligned16(p.x) || (p.act && !aligned16(p.act)) || (p.dx && !aligned16(p.dx))) return false;
  const DeviceInfo& dev = device_info();
  const long long plane_vecs = (p.spatial * (long long)sizeof(T) + 15) / 16;
  // measurement switch: B200_BN_NCHW_FORCE=cta|cluster|registers picks the variant whatever the shape
  static const int force = [] {
    const char* e = getenv("B200_BN_NCHW_FORCE");
    if (!e) return 0;
    return e[0] == 'c' && e[1] == 't' ? 2 : (e[0] == 'c' ? 3 : (e[0] == 'r' ? 4 : 0));
  }();
  {  // channels of at most 8 K elements: the register-resident kernel, as few elements per thread as 512 threads allow
    const long long elems = p.rows * p.spatial;
    if ((force == 0 || force == 4) && elems <= 8192 && elems * p.channels < 0x7fffffffLL) {
      constexpr int WMAX = 16 / (int)sizeof(T);  // elements of a 16-byte access
      int W = WMAX;
      while (W > 1 && p.spatial % W != 0) W /= 2;  // the tensors are 16-byte aligned (checked above)
      if (W == 8) { if constexpr (WMAX >= 8) launch_bn_bwd_small<T, 8>(p, st); }
      else if (W == 4) launch_bn_bwd_small<T, 4>(p, st);
      else if (W == 2) launch_bn_bwd_small<T, 2>(p, st);
      else launch_bn_bwd_small<T, 1>(p, st);
      *rc = launch_status("b200_batch_norm_bwd [NCHW, one launch, CTA per channel, channel in registers]");
      return true;
    }
  }
  int S = 1;  // several CTAs per channel only when a channel holds enough data (see batch_norm_nchw.cu)
  if (p.rows * p.spatial * (long long)sizeof(T) >= 128 * 1024)
    while (S < 8 && (long long)p.channels * S < 2LL * dev.sm_count && 2 * S <= p.rows) S *= 2;
  if (force == 2) S = 1;
  if (force == 3 && S == 1 && p.rows >= 2) S = 2;
  const int ipc = (int)((p.rows + S - 1) / S);  // a CTA whose range starts beyond the last image has no planes
  // lanes per plane: as few as give every plane of the CTA its own group, but enough that a lane
  // holds at most four vectors of each tensor of a plane (see batch_norm_nchw.cu)
  int G = 32;
  while (G > 2 && 256 / (G / 2) <= 2 * ipc && plane_vecs <= 4LL * (G / 2)) G /= 2;
  if (S == 1) {
    const dim3 grid(1, (unsigned)p.channels, 1);
    if (p.act) bn_bwd_nchw_cluster_kernel<T, true, false><<<grid, 256, 0, st>>>(p, ipc, G);
    else bn_bwd_nchw_cluster_kernel<T, false, false><<<grid, 256, 0, st>>>(p, ipc, G);
    *rc = launch_status("b200_batch_norm_bwd [NCHW, one launch, CTA per channel]");
    return true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)S, (unsigned)p.channels, 1);
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)S;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = p.act ? cudaLaunchKernelEx(&cfg, bn_bwd_nchw_cluster_kernel<T, true, true>, p, ipc, G)
                        : cudaLaunchKernelEx(&cfg, bn_bwd_nchw_cluster_kernel<T, false, true>, p, ipc, G);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  *rc = launch_status("b200_batch_norm_bwd [NCHW, one launch, cluster per channel, DSMEM combine]");
  return true;
}

template <typename T>
static int launch_bn_bwd(BnBwdParams p, bool fast, size_t scratch_bytes, cudaStream_t st) {
  constexpr int V = Elem<T>::V;
  const DeviceInfo& dev = device_info();
  const long long coef_floats = 4LL * p.channels;
  if (fast) {
    long long g = p.channels, h = V;  // gcd(C, V)
    while (h) { const long long t = g % h; g = h; h = t; }
    const int vpr = (int)(p.channels / g);  // PV: vectors after which the channel pattern repeats
    const int threads = 256 / vpr * vpr;  // a multiple of PV: a thread keeps its phase
    const long long total = p.rows * p.channels / V;
    long long splits = 8LL * dev.sm_count;  // eight CTAs per SM
    // at least two rounds of loads (8 vectors of each tensor) per thread: small tensors get few
    // partial rows and a short finalize
    if (splits * threads * 8 > total) splits = (total + threads * 8 - 1) / (threads * 8);
    if (splits < 1) splits = 1;
    long long per = (total + splits - 1) / splits;
    per = (per + vpr - 1) / vpr * vpr;  // whole rows per CTA: the column of a thread stays fixed
    splits = (total + per - 1) / per;
    const long long need = splits * 2 * p.channels * (long long)sizeof(double) + coef_floats * (long long)sizeof(float);
    if ((long long)scratch_bytes < need)
      return fail(B200_ERR_WORKSPACE, "b200_batch_norm_bwd: scratch of %zu bytes, need %lld", scratch_bytes, need);
    p.splits = (int)splits;
    p.coef = reinterpret_cast<float*>(p.partials + splits * 2 * p.channels);
    bn_bwd_sums_cl_kernel<T><<<(unsigned)splits, threads, 0, st>>>(p, per, vpr);
    int rc = launch_status("b200_batch_norm_bwd sums");
    if (rc != B200_OK) return rc;
    bn_bwd_finalize_kernel<<<p.channels, 256, 0, st>>>(p);
    rc = launch_status("b200_batch_norm_bwd finalize");
    if (rc != B200_OK || !p.dx) return rc;
    bn_bwd_apply_cl_kernel<T><<<(unsigned)splits, threads, 0, st>>>(p, per, vpr);
    return launch_status("b200_batch_norm_bwd apply [channels-last, vector]");
  }
  {  // contiguous NCHW: one launch, a cluster of CTAs per channel
    int rc = B200_OK;
    if (try_launch_bn_bwd_nchw<T>(p, st, &rc)) return rc;
  }
  const long long total = p.rows * p.spatial;
  long long splits = total / 16384;
  if (splits < 1) splits = 1;
  if (splits > 64) splits = 64;
  const long long need = splits * 2 * p.channels * (long long)sizeof(double) + coef_floats * (long long)sizeof(float);
  if ((long long)scratch_bytes < need)
    return fail(B200_ERR_WORKSPACE, "b200_batch_norm_bwd: scratch of %zu bytes, need %lld", scratch_bytes, need);
  p.splits = (int)splits;
  p.coef = reinterpret_cast<float*>(p.partials + splits * 2 * p.channels);
  bn_bwd_sums_general_kernel<T><<<dim3(p.channels, (unsigned)splits), 256, 0, st>>>(p);
  int rc = launch_status("b200_batch_norm_bwd sums");
  if (rc != B200_OK) return rc;
  bn_bwd_finalize_kernel<<<p.channels, 256, 0, st>>>(p);
  rc = launch_status("b200_batch_norm_bwd finalize");
  if (rc != B200_OK || !p.dx) return rc;
  bn_bwd_apply_general_kernel<T><<<dim3(p.channels, (unsigned)splits), 256, 0, st>>>(p);
  return launch_status("b200_batch_norm_bwd apply [strided, element-wise]");
}

}  // namespace b200

using namespace b200;

extern "C" int64_t b200_batch_norm_bwd_scratch_bytes(int64_t channels) {
  const int sms = device_info().sm_count;
  return (int64_t)(8 * sms > 64 ? 8 * sms : 64) * 2 * channels * (int64_t)sizeof(double) +
         4 * channels * (int64_t)sizeof(float);
}

// b200_batch_norm_bwd with the reciprocal element count given by the caller (inv_count > 0) instead
// of 1 / (batch * spatial). A captured graph carries 1/N as a literal of the shape it was captured
// at and applies it at every other shape point too; an oracle for such a graph has to do the same.
extern "C" int b200_batch_norm_bwd_ex(const void* dy, const void* x, const void* act, const float* mean,
                                      const float* invstd, const void* weight, void* dx, float* dweight,
                                      float* dbias, int64_t batch, int64_t channels, int64_t spatial,
                                      int64_t stride_n, int64_t stride_c, int64_t stride_s, int32_t x_dtype,
                                      int32_t w_dtype, double slope, double inv_count, void* scratch,
                                      int64_t scratch_bytes, void* stream) {
  if (!dy || !x || !mean || !invstd) return fail(B200_ERR_INVALID, "b200_batch_norm_bwd: null argument");
  if (batch < 0 || channels <= 0 || spatial < 0 || channels > 0x7fffffffLL)
    return fail(B200_ERR_INVALID, "b200_batch_norm_bwd: bad sizes");
  if (!scratch || scratch_bytes <= 0) return fail(B200_ERR_WORKSPACE, "b200_batch_norm_bwd: needs a scratch buffer");
  if (!aligned16(scratch)) return fail(B200_ERR_ALIGNMENT, "b200_batch_norm_bwd: scratch must be 16-byte aligned");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long count = batch * spatial;
  if (count == 0) {
    if (dweight) cudaMemsetAsync(dweight, 0, channels * sizeof(float), st);
    if (dbias) cudaMemsetAsync(dbias, 0, channels * sizeof(float), st);
    return launch_status("b200_batch_norm_bwd (empty)");
  }
  BnBwdParams p;
  p.dy = dy; p.x = x; p.act = act; p.mean = mean; p.invstd = invstd; p.weight = weight; p.w_dtype = w_dtype;
  p.dx = dx; p.dweight = dweight; p.dbias = dbias;
  p.spatial = spatial; p.sn = stride_n; p.sc = stride_c; p.ss = stride_s;
  p.channels = (int)channels; p.slope = (float)slope;
  p.inv_count = inv_count > 0.0 ? (float)inv_count : (float)(1.0 / (double)count);
  p.partials = reinterpret_cast<double*>(scratch);
  p.coef = nullptr; p.splits = 0;
  const int eb = dtype_size(x_dtype);
  const int v = 16 / eb;
  const bool cl = stride_c == 1 && stride_s == channels && stride_n == spatial * channels;
  // vectors after which the pattern of channels under a vector repeats: C / gcd(C, v); the flat
  // kernels need whole periods and at most 256 vectors in one
  long long g = channels, h = v;
  while (h) { const long long t = g % h; g = h; h = t; }
  const long long pv = channels / g;
  const bool fast = cl && pv >= 1 && pv <= 256 && (batch * spatial * channels) % (pv * v) == 0 && aligned16(dy) &&
                    aligned16(x) && (!act || aligned16(act)) && (!dx || aligned16(dx));
  p.rows = fast ? batch * spatial : batch;
  switch (x_dtype) {
    case B200_F32: return launch_bn_bwd<float>(p, fast, (size_t)scratch_bytes, st);
    case B200_BF16: return launch_bn_bwd<__nv_bfloat16>(p, fast, (size_t)scratch_bytes, st);
    case B200_F16: return launch_bn_bwd<__half>(p, fast, (size_t)scratch_bytes, st);
  }
  return fail(B200_ERR_INVALID, "b200_batch_norm_bwd: unknown dtype %d", x_dtype);
}

extern "C" int b200_batch_norm_bwd(const void* dy, const void* x, const void* act, const float* mean,
                                   const float* invstd, const void* weight, void* dx, float* dweight,
                                   float* dbias, int64_t batch, int64_t channels, int64_t spatial,
                                   int64_t stride_n, int64_t stride_c, int64_t stride_s, int32_t x_dtype,
                                   int32_t w_dtype, double slope, void* scratch, int64_t scratch_bytes,
                                   void* stream) {
  return b200_batch_norm_bwd_ex(dy, x, act, mean, invstd, weight, dx, dweight, dbias, batch, channels, spatial,
                                stride_n, stride_c, stride_s, x_dtype, w_dtype, slope, 0.0, scratch, scratch_bytes,
                                stream);
}
