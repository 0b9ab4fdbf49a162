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
// Any other layout (NCHW, channel counts that are not a multiple of the vector width) takes the
// three-launch general path: strided statistics, finalize, strided normalise.
#include "rowwise.cuh"

#include <mutex>

namespace b200 {

struct BatchNormParams {
  const void* x;
  void* y;
  const void* weight;  // may be null
  const void* bias;    // may be null
  float* running_mean;  // may be null (no update)
  float* running_var;
  float* save_mean;    // [C] fp32 out (may be null)
  float* save_invstd;  // [C] fp32 out (may be null)
  long long rows;      // N*H*W for channels-last; N for the general path
  int channels;
  long long spatial;   // general path: H*W
  long long sn, sc, ss;  // general path: element strides of (n, c, spatial)
  int w_dtype;
  float eps, momentum, one_minus_momentum, unbias;
  double count;  // elements per channel
  int relu;
  float* partials;  // [P][2][C]
  float* stats;     // [2][C] mean, invstd (scratch copy every CTA reads)
  unsigned int* bar;
  long long rows_per_cta;  // contiguous row range of each CTA (a multiple of rows-per-pass)
  int smem_tiles;          // tiles of each CTA kept in shared memory between the passes
};

template <typename T, bool VECTOR>
__device__ __forceinline__ void bn_finalize_channel(const BatchNormParams& p, int c, int num_partials,
                                                    float shift) {
  // Called by one warp per channel: lanes split the partials, fp64 accumulation, fixed order.
  const int lane = threadIdx.x & 31;
  double s1 = 0.0, s2 = 0.0;
  for (int g = lane; g < num_partials; g += 32) {
    s1 += (double)__ldcg(p.partials + ((long long)g * 2) * p.channels + c);
    s2 += (double)__ldcg(p.partials + ((long long)g * 2 + 1) * p.channels + c);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s1 += __shfl_xor_sync(0xffffffffu, s1, o);
    s2 += __shfl_xor_sync(0xffffffffu, s2, o);
  }
  if (lane == 0) {
    const double mean_shifted = s1 / p.count;
    double var = (s2 - s1 * mean_shifted) / p.count;
    if (var < 0.0) var = 0.0;
    const float mean = (float)((double)shift + mean_shifted);
    const float varf = (float)var;
    const float invstd = rsqrtf(varf + p.eps);
    p.stats[c] = mean;
    p.stats[p.channels + c] = invstd;
    if (p.save_mean) p.save_mean[c] = mean;
    if (p.save_invstd) p.save_invstd[c] = invstd;
    if (p.running_mean) {
      p.running_mean[c] = mean * p.momentum + p.running_mean[c] * p.one_minus_momentum;
      p.running_var[c] = (varf * p.unbias) * p.momentum + p.running_var[c] * p.one_minus_momentum;
    }
  }
}

// ----------------------------------------------------------------------------------------------
// Channels-last fused kernel. blockDim.x = vpr * rpp (vpr = C / V vectors per row, rpp = rows per
// pass); a tile is rpp * U rows. Dynamic shared memory: smem_tiles tiles of raw 16-byte vectors,
// followed by the reduction area.
// ----------------------------------------------------------------------------------------------
template <typename T, int U>
__global__ void __launch_bounds__(512, 1) batch_norm_cl_fused_kernel(const BatchNormParams p) {
  constexpr int V = Elem<T>::V;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ int bar_ok;
  const int T_ = blockDim.x;
  const int vpr = p.channels / V;
  const int rpp = T_ / vpr;
  const int vc = threadIdx.x % vpr;  // this thread's vector column
  const int tr = threadIdx.x / vpr;  // this thread's row inside a pass
  const long long tile_rows = (long long)rpp * U;
  const int tile_vecs = T_ * U;
  uint4* keep = reinterpret_cast<uint4*>(smem_raw);
  float* red = reinterpret_cast<float*>(smem_raw + (size_t)p.smem_tiles * tile_vecs * sizeof(uint4));

  const T* x = reinterpret_cast<const T*>(p.x);
  const long long row_begin = (long long)blockIdx.x * p.rows_per_cta;
  long long row_end = row_begin + p.rows_per_cta;
  if (row_end > p.rows) row_end = p.rows;
  const int my_tiles = row_end > row_begin ? (int)((row_end - row_begin + tile_rows - 1) / tile_rows) : 0;
  const int first_kept = my_tiles - p.smem_tiles;  // tiles with local index >= this stay in smem

  const uint64_t keep_policy = l2_policy_evict_last();

  // ---- pass 1: shifted sums -------------------------------------------------------------------
  float shift[V];
  {
    float f[V];
    Elem<T>::unpack(ld_keep(x + (long long)vc * V), f);  // row 0 of this thread's channels
#pragma unroll
    for (int i = 0; i < V; ++i) shift[i] = f[i];
  }
  float s1[V], s2[V];
#pragma unroll
  for (int i = 0; i < V; ++i) s1[i] = s2[i] = 0.f;

  for (int t = 0; t < my_tiles; ++t) {
    const long long r0 = row_begin + (long long)t * tile_rows + tr;
    uint4 raw[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long r = r0 + (long long)u * rpp;
      if (r < row_end) raw[u] = ld_policy(x + r * p.channels + (long long)vc * V, keep_policy);
    }
    const bool stash = t >= first_kept;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long r = r0 + (long long)u * rpp;
      if (r < row_end) {
        if (stash) keep[(size_t)(t - first_kept) * tile_vecs + u * T_ + threadIdx.x] = raw[u];
        float f[V];
        Elem<T>::unpack(raw[u], f);
#pragma unroll
        for (int i = 0; i < V; ++i) {
          const float d = f[i] - shift[i];
          s1[i] += d;
          s2[i] += d * d;
        }
      }
    }
  }
  // combine the rpp threads that share a vector column: red[2][rpp][C]
  {
    float* r1 = red;
    float* r2 = red + (size_t)rpp * p.channels;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      r1[(size_t)tr * p.channels + vc * V + i] = s1[i];
      r2[(size_t)tr * p.channels + vc * V + i] = s2[i];
    }
    __syncthreads();
    for (int c = threadIdx.x; c < p.channels; c += T_) {
      float a = 0.f, b = 0.f;
      for (int k = 0; k < rpp; ++k) {
        a += r1[(size_t)k * p.channels + c];
        b += r2[(size_t)k * p.channels + c];
      }
      p.partials[((long long)blockIdx.x * 2) * p.channels + c] = a;
      p.partials[((long long)blockIdx.x * 2 + 1) * p.channels + c] = b;
    }
  }
  bool ok = grid_barrier(p.bar, 1u, &bar_ok);

  // ---- channel statistics: warps of all CTAs split the channels -------------------------------
  if (ok) {
    const int warps_per_cta = T_ >> 5;  // blockDim.x is a multiple of 32 (checked by the host)
    const int gwarp = blockIdx.x * warps_per_cta + (threadIdx.x >> 5);
    const int total_warps = gridDim.x * warps_per_cta;
    for (int c = gwarp; c < p.channels; c += total_warps) {
      const float k = Elem<T>::to_f32(__ldg(x + c));
      bn_finalize_channel<T, true>(p, c, gridDim.x, k);
    }
    ok = grid_barrier(p.bar, 2u, &bar_ok);
  }

  // ---- pass 2: normalise, reverse tile order -----------------------------------------------------
  if (ok) {
    float mean[V], invstd[V], wv[V], bv[V];
#pragma unroll
    for (int i = 0; i < V; ++i) {
      mean[i] = __ldcg(p.stats + vc * V + i);
      invstd[i] = __ldcg(p.stats + p.channels + vc * V + i);
      wv[i] = p.weight ? load_param1(p.weight, p.w_dtype, vc * V + i) : 1.f;
      bv[i] = p.bias ? load_param1(p.bias, p.w_dtype, vc * V + i) : 0.f;
    }
    T* y = reinterpret_cast<T*>(p.y);
    const uint64_t drop_policy = l2_policy_evict_first();
    for (int t = my_tiles - 1; t >= 0; --t) {
      const long long r0 = row_begin + (long long)t * tile_rows + tr;
      uint4 raw[U];
      const bool stashed = t >= first_kept;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long r = r0 + (long long)u * rpp;
        if (r < row_end) {
          raw[u] = stashed ? keep[(size_t)(t - first_kept) * tile_vecs + u * T_ + threadIdx.x]
                           : ld_policy(x + r * p.channels + (long long)vc * V, drop_policy);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long r = r0 + (long long)u * rpp;
        if (r < row_end) {
          float f[V];
          Elem<T>::unpack(raw[u], f);
#pragma unroll
          for (int i = 0; i < V; ++i) {
            float o = ((f[i] - mean[i]) * invstd[i]) * wv[i] + bv[i];
            if (p.relu) o = o < 0.f ? 0.f : o;  // relu commutes with the monotone rounding below
            f[i] = o;
          }
          st_stream(y + r * p.channels + (long long)vc * V, Elem<T>::pack(f));
        }
      }
    }
  }
  grid_barrier_depart(p.bar);
}

// ----------------------------------------------------------------------------------------------
// General path: x addressed as (n, c, s) with arbitrary strides.
// ----------------------------------------------------------------------------------------------
// Rows per pass of the fused kernel for C / V = vpr vector columns: the largest count that keeps
// the CTA at <= 512 threads and a whole number of warps; 0 when there is none.
static int fused_rows_per_pass(int vpr) {
  if (vpr < 1 || vpr > 512) return 0;
  int rpp = 512 / vpr;
  while (rpp > 0 && (vpr * rpp) % 32 != 0) --rpp;
  return rpp;
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

template <typename T>
__global__ void __launch_bounds__(256) batch_norm_finalize_general_kernel(const BatchNormParams p,
                                                                          int num_partials) {
  const int warps = blockDim.x >> 5;
  const int c = blockIdx.x * warps + (threadIdx.x >> 5);
  if (c >= p.channels) return;
  const T* x = reinterpret_cast<const T*>(p.x);
  bn_finalize_channel<T, false>(p, c, num_partials, Elem<T>::to_f32(x[(long long)c * p.sc]));
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

template <typename T>
static int launch_batch_norm(BatchNormParams p, bool channels_last_fast, size_t scratch_bytes,
                             cudaStream_t st) {
  constexpr int V = Elem<T>::V;
  constexpr int U = 8;
  const DeviceInfo& dev = device_info();
  const long long stats_floats = 2LL * p.channels;
  if (channels_last_fast) {
    const int vpr = p.channels / V;
    const int rpp = fused_rows_per_pass(vpr);
    const int threads = vpr * rpp;
    auto kernel = batch_norm_cl_fused_kernel<T, U>;
    const long long tile_rows = (long long)rpp * U;
    const long long passes = (p.rows + rpp - 1) / rpp;
    long long grid = dev.sm_count;  // one CTA per SM
    if (grid > passes) grid = passes;
    const long long need = 256 + (grid * 2 * p.channels + stats_floats) * (long long)sizeof(float);
    if ((long long)scratch_bytes < need)
      return fail(B200_ERR_WORKSPACE, "b200_batch_norm_fwd: scratch of %zu bytes, need %lld", scratch_bytes, need);
    p.rows_per_cta = (passes + grid - 1) / grid * rpp;
    grid = (p.rows + p.rows_per_cta - 1) / p.rows_per_cta;
    const long long tiles_per_cta = (p.rows_per_cta + tile_rows - 1) / tile_rows;
    const size_t red_bytes = 2ull * rpp * p.channels * sizeof(float);
    const size_t tile_bytes = (size_t)threads * U * sizeof(uint4);
    long long room = (long long)dev.max_smem_optin - (long long)red_bytes - 1024;
    int smem_tiles = room > 0 ? (int)(room / (long long)tile_bytes) : 0;
    if (smem_tiles > tiles_per_cta) smem_tiles = (int)tiles_per_cta;
    p.smem_tiles = smem_tiles;
    const size_t smem = (size_t)smem_tiles * tile_bytes + red_bytes;
    if (red_bytes + 1024 > (size_t)dev.max_smem_optin)
      return fail(B200_ERR_UNSUPPORTED, "b200_batch_norm_fwd: %d channels need too much shared memory", p.channels);
    cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(kernel),
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail((int)e, "b200_batch_norm_fwd: cannot reserve %zu bytes of shared memory: %s", smem,
                  cudaGetErrorString(e));
    }
    p.stats = p.partials + grid * 2 * p.channels;
    void* args[] = {&p};
    e = cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), dim3((unsigned)grid), dim3(threads),
                                    args, smem, st);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail((int)e, "b200_batch_norm_fwd: cooperative launch failed: %s", cudaGetErrorString(e));
    }
    note_launch();
    return B200_OK;
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
  int rc = launch_status("b200_batch_norm_fwd stats");
  if (rc != B200_OK) return rc;
  batch_norm_finalize_general_kernel<T><<<(p.channels + 7) / 8, 256, 0, st>>>(p, (int)splits);
  rc = launch_status("b200_batch_norm_fwd finalize");
  if (rc != B200_OK) return rc;
  if (p.y) {
    batch_norm_apply_general_kernel<T><<<dim3(p.channels, (unsigned)splits), 256, 0, st>>>(p);
    rc = launch_status("b200_batch_norm_fwd apply");
  }
  return rc;
}

}  // namespace b200

using namespace b200;

extern "C" int64_t b200_batch_norm_scratch_bytes(int64_t channels) {
  const int sms = device_info().sm_count;
  return 256 + ((int64_t)(sms > 64 ? sms : 64) * 2 * channels + 2 * channels) * (int64_t)sizeof(float);
}

extern "C" int b200_batch_norm_fwd(const void* x, void* y, const void* weight, const void* bias,
                                   float* running_mean, float* running_var, float* save_mean,
                                   float* save_invstd, int64_t batch, int64_t channels, int64_t spatial,
                                   int64_t stride_n, int64_t stride_c, int64_t stride_s,
                                   int32_t x_dtype, int32_t w_dtype, double eps, double momentum,
                                   int32_t relu, void* scratch, int64_t scratch_bytes, void* stream) {
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
  p.unbias = (float)(count / (count - 1.0));
  p.relu = relu ? 1 : 0;
  p.bar = reinterpret_cast<unsigned int*>(scratch);
  p.partials = reinterpret_cast<float*>(reinterpret_cast<char*>(scratch) + 256);
  p.stats = nullptr; p.rows_per_cta = 0; p.smem_tiles = 0;

  const int eb = dtype_size(x_dtype);
  const int v = 16 / eb;
  // channels-last: c is the unit-stride dimension, rows are (n, s) pairs with a uniform stride of C
  const bool cl = stride_c == 1 && stride_s == channels && stride_n == spatial * channels;
  const bool fast = cl && channels % v == 0 && fused_rows_per_pass((int)(channels / v)) > 0 &&
                    aligned16(x) && aligned16(y);
  if (fast) {
    p.rows = batch * spatial;
  } else {
    p.rows = batch;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (x_dtype) {
    case B200_F32: return launch_batch_norm<float>(p, fast, (size_t)scratch_bytes, st);
    case B200_BF16: return launch_batch_norm<__nv_bfloat16>(p, fast, (size_t)scratch_bytes, st);
    case B200_F16: return launch_batch_norm<__half>(p, fast, (size_t)scratch_bytes, st);
  }
  return fail(B200_ERR_INVALID, "b200_batch_norm_fwd: unknown dtype %d", x_dtype);
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
