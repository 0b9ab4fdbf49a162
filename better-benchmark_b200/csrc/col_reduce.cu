// Column reductions: x viewed as [batch, rows, cols] with cols contiguous, reduced over rows.
//
// Replaces the column-form Triton kernels of the sum/mean repros in the reference:
// repros/canonical/sum_eb86a17deab9/oracle.py:20-70 (atomic partial sums, grid (R/256, H/32)),
// sum_c2bf513c1ebf/oracle.py:10-29 (whole column in one tile) and the channels-last spatial mean
// of mean_c9e1a8113328/oracle.py:11-76 ([N, H*W, C] -> [N, C]).
//
// A thread owns one 16-byte vector column; the CTA's thread rows and, for tall inputs, several
// CTAs split the rows. With 2, 4 or 8 splits the CTAs of one reduction form a thread-block cluster:
// each leaves its folded partial result in its own shared memory and the first CTA of the cluster
// reads the others' through distributed shared memory, adds them in fp64 in a fixed order and
// writes the output - one launch, no scratch traffic. With more splits the partial results go to
// scratch as fp32 and a second launch combines them the same way. No float atomics either way:
// bit-reproducible (the reference's atomic variant is not, and its harness would classify such an
// output as stochastic).
#include "rowwise.cuh"

#include <cooperative_groups.h>

#include <cstdlib>

namespace b200 {

#define B200_COL_SUM 0
#define B200_COL_MEAN 1
#define B200_COL_AMAX 2

struct ColReduceParams {
  const void* x;
  void* out;
  float* partials;  // [splits][batch][cols]
  long long batch, rows, cols;
  long long x_batch_stride, x_row_stride;  // elements
  long long out_batch_stride;
  int out_dtype;
  int op;
  int splits;
  long long rows_per_split;
  float post_scale;
  int tx_log2;  // log2 of the lanes per thread row: 32 for wide tensors, fewer when cols / V < 32
};

__device__ __forceinline__ void store_out(void* out, int dtype, long long idx, float v) {
  if (dtype == B200_F32) reinterpret_cast<float*>(out)[idx] = v;
  else if (dtype == B200_BF16) reinterpret_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
  else reinterpret_cast<__half*>(out)[idx] = __float2half_rn(v);
}

// 256 threads = TY thread rows of TX lanes (TX = 32, or the power of two that covers cols / V when
// that is smaller, so that narrow tensors - a channels-last image with 64 channels is 8 vectors
// wide - still use every lane); grid = (column chunks of TX vectors, splits of the rows, batch).
// CLUSTER: the gridDim.y CTAs that split one reduction are one cluster (cluster dims (1, splits, 1)).
template <typename T, bool IS_MAX, bool VEC, bool CLUSTER>
__global__ void __launch_bounds__(512) col_reduce_kernel(const ColReduceParams p) {
  constexpr int V = VEC ? Elem<T>::V : 1;
  constexpr int U = 8;
  __shared__ float red[512 * V + 512];  // [TY][TX * V + 1]
  __shared__ float fold[CLUSTER ? 32 * V : 1];  // this CTA's folded columns, read by the cluster's first CTA
  const int TX = 1 << p.tx_log2, TY = (int)blockDim.x >> p.tx_log2;
  const int tx = threadIdx.x & (TX - 1), ty = threadIdx.x >> p.tx_log2;
  const int pitch = TX * V + 1;
  const long long col0 = ((long long)blockIdx.x * TX + tx) * V;
  const long long b = blockIdx.z;
  const long long r_begin = (long long)blockIdx.y * p.rows_per_split;
  long long r_end = r_begin + p.rows_per_split;
  if (r_end > p.rows) r_end = p.rows;
  const bool active = col0 < p.cols;
  const T* base = reinterpret_cast<const T*>(p.x) + b * p.x_batch_stride + col0;

  float acc[V];
#pragma unroll
  for (int i = 0; i < V; ++i) acc[i] = IS_MAX ? -INFINITY : 0.f;
  if (active) {
    for (long long r0 = r_begin + ty; r0 < r_end; r0 += (long long)TY * U) {
      if constexpr (VEC) {
        uint4 raw[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long r = r0 + (long long)TY * u;
          if (r < r_end) raw[u] = ld_stream(base + r * p.x_row_stride);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long r = r0 + (long long)TY * u;
          if (r < r_end) {
            float f[V];
            Elem<T>::unpack(raw[u], f);
#pragma unroll
            for (int i = 0; i < V; ++i) acc[i] = IS_MAX ? MaxOp::apply(acc[i], f[i]) : acc[i] + f[i];
          }
        }
      } else {
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long r = r0 + (long long)TY * u;
          if (r < r_end) {
            const float f = Elem<T>::to_f32(base[r * p.x_row_stride]);
            acc[0] = IS_MAX ? MaxOp::apply(acc[0], f) : acc[0] + f;
          }
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < V; ++i) red[ty * pitch + tx * V + i] = acc[i];
  __syncthreads();
  // thread rows are folded in a fixed order, one column per thread
  for (int c = threadIdx.x; c < TX * V; c += blockDim.x) {
    const long long col = (long long)blockIdx.x * TX * V + c;
    if (col >= p.cols) {
      if constexpr (CLUSTER) fold[c] = IS_MAX ? -INFINITY : 0.f;
      continue;
    }
    float r;
    if constexpr (IS_MAX) {
      r = red[c];
      for (int k = 1; k < TY; ++k) r = MaxOp::apply(r, red[k * pitch + c]);
    } else {
      double d = 0.0;  // above a thread's own chain the sum is carried in fp64
      for (int k = 0; k < TY; ++k) d += (double)red[k * pitch + c];
      r = (float)d;
    }
    if constexpr (CLUSTER) {
      fold[c] = r;
    } else if (p.splits == 1) {
      store_out(p.out, p.out_dtype, b * p.out_batch_stride + col, r * p.post_scale);
    } else {
      p.partials[((long long)blockIdx.y * p.batch + b) * p.cols + col] = r;
    }
  }
  if constexpr (CLUSTER) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();  // every CTA of the cluster has written its fold[]
    if (cluster.block_rank() == 0) {
      const unsigned int nblocks = cluster.num_blocks();
      for (int c = threadIdx.x; c < TX * V; c += blockDim.x) {
        const long long col = (long long)blockIdx.x * TX * V + c;
        if (col >= p.cols) continue;
        float r;
        if constexpr (IS_MAX) {
          r = fold[c];
          for (unsigned int k = 1; k < nblocks; ++k) r = MaxOp::apply(r, cluster.map_shared_rank(fold, k)[c]);
          store_out(p.out, p.out_dtype, b * p.out_batch_stride + col, r);
        } else {
          double d = (double)fold[c];
          for (unsigned int k = 1; k < nblocks; ++k) d += (double)cluster.map_shared_rank(fold, k)[c];
          store_out(p.out, p.out_dtype, b * p.out_batch_stride + col, (float)d * p.post_scale);
        }
      }
    }
    cluster.sync();  // nobody leaves (and gives up its shared memory) before the first CTA has read it
  }
}

// Combines the splits: a CTA takes 32 outputs (lanes), its eight warps take the splits w, w+8, ...
// with all their loads in flight together, and warp 0 adds the eight partial sums in order (fp64).
template <bool IS_MAX>
__global__ void __launch_bounds__(256) col_reduce_finalize_kernel(const ColReduceParams p) {
  __shared__ double red[8][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long total = p.batch * p.cols;
  const long long idx = (long long)blockIdx.x * 32 + lane;  // over batch * cols
  const bool live = idx < total;
  double r = IS_MAX ? -INFINITY : 0.0;
  for (int s0 = warp; s0 < p.splits; s0 += 8 * 8) {
    float v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int sp = s0 + 8 * u;
      v[u] = (live && sp < p.splits) ? p.partials[(long long)sp * total + idx] : (IS_MAX ? -INFINITY : 0.f);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) r = IS_MAX ? (double)MaxOp::apply((float)r, v[u]) : r + (double)v[u];
  }
  red[warp][lane] = r;
  __syncthreads();
  if (warp == 0 && live) {
    double t = red[0][lane];
#pragma unroll
    for (int w = 1; w < 8; ++w) t = IS_MAX ? (double)MaxOp::apply((float)t, (float)red[w][lane]) : t + red[w][lane];
    const long long b = idx / p.cols, col = idx - b * p.cols;
    store_out(p.out, p.out_dtype, b * p.out_batch_stride + col, IS_MAX ? (float)t : (float)t * p.post_scale);
  }
}

template <typename T>
static int launch_col_reduce(ColReduceParams p, bool vec, size_t scratch_bytes, cudaStream_t st) {
  const int sms = device_info().sm_count;
  const int v = vec ? Elem<T>::V : 1;
  const long long vcols = (p.cols + v - 1) / v;
  int tx_log2 = 5;
  while (tx_log2 > 0 && (1LL << (tx_log2 - 1)) >= vcols) --tx_log2;
  p.tx_log2 = tx_log2;
  const long long tx = 1LL << tx_log2;
  const long long chunks = (vcols + tx - 1) / tx;
  if (chunks > 0x7fffffffLL || p.batch > 65535) return fail(B200_ERR_UNSUPPORTED, "b200_col_reduce: grid too large");
  const long long base = chunks * p.batch;
  // (A single launch of one 512-thread CTA per reduction, without a split, was measured slower
  // than three splits plus the finalize launch on a batch of 256 images: 25.2 us against 22.6 us.)
  const int threads = 256;
  const long long ty = threads / tx;
  // Otherwise: enough 256-thread CTAs (eight resident per SM) to fill the machine about four times
  // over, every thread keeping at least eight rows. When a somewhat larger split count makes the
  // CTAs fill whole waves almost exactly, take that one: a grid of 4.1 CTAs per SM runs as long as
  // one of 5.
  const long long slots = 8LL * sms;
  long long max_splits = (p.rows + 8 * ty - 1) / (8 * ty);
  if (max_splits < 1) max_splits = 1;
  long long splits = (4LL * sms + base - 1) / base;
  if (splits > max_splits) splits = max_splits;
  for (long long s = splits; s <= max_splits && s <= 2 * splits; ++s) {
    const long long ctas = s * base;
    if (ctas < slots) continue;
    const long long waves = (ctas + slots - 1) / slots;
    if ((double)ctas / (double)(waves * slots) >= 0.97) {
      splits = s;
      break;
    }
  }
  {
    static const int splits_env = [] { const char* e = getenv("B200_COL_SPLITS"); return e ? atoi(e) : 0; }();
    if (splits_env > 0 && splits_env <= max_splits) splits = splits_env;
  }
  const long long cap = scratch_bytes / ((size_t)p.batch * p.cols * sizeof(float) + 1);
  if (splits > cap) splits = cap;
  if (splits > 65535) splits = 65535;
  if (splits < 1) splits = 1;
  p.splits = (int)splits;
  p.rows_per_split = (p.rows + splits - 1) / splits;
  const bool is_max = p.op == B200_COL_AMAX;
  // 2..8 splits: one cluster per reduction, combined through distributed shared memory
  static const bool clusters_off = [] { const char* e = getenv("B200_COL_NO_CLUSTER"); return e && e[0] == '1'; }();
  if (vec && !clusters_off && splits >= 2 && splits <= 8) {
    long long cs = splits <= 2 ? 2 : (splits <= 4 ? 4 : 8);
    while (cs > max_splits && cs > 2) cs /= 2;
    if (cs <= max_splits) {
      ColReduceParams q = p;
      q.splits = (int)cs;
      q.rows_per_split = (p.rows + cs - 1) / cs;
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3((unsigned)chunks, (unsigned)cs, (unsigned)p.batch);
      cfg.blockDim = dim3(threads);
      cfg.dynamicSmemBytes = 0;
      cfg.stream = st;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 1;
      attr[0].val.clusterDim.y = (unsigned)cs;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      cudaError_t e = is_max ? cudaLaunchKernelEx(&cfg, col_reduce_kernel<T, true, true, true>, q)
                             : cudaLaunchKernelEx(&cfg, col_reduce_kernel<T, false, true, true>, q);
      if (e == cudaSuccess) return launch_status("b200_col_reduce [vector, cluster of splits, DSMEM combine]");
      cudaGetLastError();  // the cluster launch was refused: take the two-launch path
    }
  }
  // More than 8 splits would need a second launch to combine them. For inputs up to about the size
  // of the L2, where a launch costs as much as the reduction itself, narrower column chunks (8
  // vectors = 128 contiguous bytes per row instead of 32) give enough CTAs with clusters of at most
  // 8 splits, and the reduction stays one launch.
  if (vec && !clusters_off && splits > 8 && p.tx_log2 > 3 &&
      (double)p.batch * (double)p.rows * (double)p.cols * sizeof(T) <= 128.0 * 1024 * 1024) {
    const long long chunks2 = (vcols + 7) / 8;
    const long long max_splits2 = (p.rows + 8 * 32 - 1) / (8 * 32);
    long long cs = 8;
    while (cs > max_splits2 && cs > 1) cs /= 2;
    if (cs >= 2 && 2 * chunks2 * p.batch * cs >= sms && chunks2 <= 0x7fffffffLL) {
      ColReduceParams q = p;
      q.tx_log2 = 3;
      q.splits = (int)cs;
      q.rows_per_split = (p.rows + cs - 1) / cs;
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3((unsigned)chunks2, (unsigned)cs, (unsigned)p.batch);
      cfg.blockDim = dim3(threads);
      cfg.dynamicSmemBytes = 0;
      cfg.stream = st;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 1;
      attr[0].val.clusterDim.y = (unsigned)cs;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      cudaError_t e = is_max ? cudaLaunchKernelEx(&cfg, col_reduce_kernel<T, true, true, true>, q)
                             : cudaLaunchKernelEx(&cfg, col_reduce_kernel<T, false, true, true>, q);
      if (e == cudaSuccess) return launch_status("b200_col_reduce [vector, narrow chunks, cluster of splits, DSMEM combine]");
      cudaGetLastError();
    }
  }
  dim3 grid((unsigned)chunks, (unsigned)splits, (unsigned)p.batch);
  set_path_tag(vec ? "vector" : "element-wise");
  if (is_max) {
    if (vec) col_reduce_kernel<T, true, true, false><<<grid, threads, 0, st>>>(p);
    else col_reduce_kernel<T, true, false, false><<<grid, threads, 0, st>>>(p);
  } else {
    if (vec) col_reduce_kernel<T, false, true, false><<<grid, threads, 0, st>>>(p);
    else col_reduce_kernel<T, false, false, false><<<grid, threads, 0, st>>>(p);
  }
  int rc = launch_status("b200_col_reduce");
  if (rc != B200_OK || splits == 1) return rc;
  const long long total = p.batch * p.cols;
  if (is_max) col_reduce_finalize_kernel<true><<<(unsigned)((total + 31) / 32), 256, 0, st>>>(p);
  else col_reduce_finalize_kernel<false><<<(unsigned)((total + 31) / 32), 256, 0, st>>>(p);
  return launch_status("b200_col_reduce finalize");
}

}  // namespace b200

using namespace b200;

extern "C" int b200_col_reduce(const void* x, void* out, int64_t batch, int64_t rows, int64_t cols,
                               int64_t x_batch_stride, int64_t x_row_stride, int64_t out_batch_stride,
                               int32_t x_dtype, int32_t out_dtype, int32_t op, void* scratch,
                               int64_t scratch_bytes, void* stream) {
  if (!x || !out) return fail(B200_ERR_INVALID, "b200_col_reduce: null argument");
  if (batch < 0 || rows < 0 || cols < 0) return fail(B200_ERR_INVALID, "b200_col_reduce: negative size");
  if (op < 0 || op > 2) return fail(B200_ERR_INVALID, "b200_col_reduce: unknown op %d", op);
  if (batch == 0 || cols == 0) return B200_OK;
  if (rows == 0 && op == B200_COL_AMAX) return fail(B200_ERR_INVALID, "b200_col_reduce: amax over zero rows");
  ColReduceParams p;
  p.x = x; p.out = out; p.partials = reinterpret_cast<float*>(scratch);
  p.batch = batch; p.rows = rows; p.cols = cols;
  p.x_batch_stride = x_batch_stride; p.x_row_stride = x_row_stride; p.out_batch_stride = out_batch_stride;
  p.out_dtype = out_dtype; p.op = op; p.splits = 1; p.rows_per_split = rows;
  p.post_scale = op == B200_COL_MEAN ? 1.0f / (float)rows : 1.0f;
  const int eb = dtype_size(x_dtype);
  const bool vec = aligned16(x) && (x_batch_stride * eb) % 16 == 0 && (x_row_stride * eb) % 16 == 0 &&
                   cols % (16 / eb) == 0;
  const size_t sb = scratch ? (size_t)scratch_bytes : 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (x_dtype) {
    case B200_F32: return launch_col_reduce<float>(p, vec, sb, st);
    case B200_BF16: return launch_col_reduce<__nv_bfloat16>(p, vec, sb, st);
    case B200_F16: return launch_col_reduce<__half>(p, vec, sb, st);
  }
  return fail(B200_ERR_INVALID, "b200_col_reduce: unknown dtype %d", x_dtype);
}
