// Library-wide pieces of the C ABI: error text, version, device properties, status words.
#include "common.cuh"

#include <atomic>
#include <mutex>

namespace b200 {

char* last_error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

const DeviceInfo& device_info() {
  static DeviceInfo info[64];
  static bool have[64] = {false};
  static std::mutex mu;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  std::lock_guard<std::mutex> lock(mu);
  if (!have[dev]) {
    DeviceInfo d;
    d.sm_count = 148;
    d.max_smem_optin = 48 * 1024;
    d.l2_bytes = 0;
    cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    cudaDeviceGetAttribute(&d.l2_bytes, cudaDevAttrL2CacheSize, dev);
    info[dev] = d;
    have[dev] = true;
  }
  return info[dev];
}

static std::atomic<long long> g_launches{0};
static thread_local const char* t_path_tag = nullptr;
static thread_local char t_last_kernel[160] = {0};

void set_path_tag(const char* tag) { t_path_tag = tag; }

void note_launch(const char* what) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (t_path_tag)
    snprintf(t_last_kernel, sizeof(t_last_kernel), "%s [%s]", what, t_path_tag);
  else
    snprintf(t_last_kernel, sizeof(t_last_kernel), "%s", what);
  t_path_tag = nullptr;
}

}  // namespace b200

// Number of kernels this library has launched in this process (cooperative launches included).
extern "C" int64_t b200_launch_count(void) { return b200::g_launches.load(std::memory_order_relaxed); }

// Name of the kernel this thread launched last, with the variant the launcher chose in brackets
// (e.g. "b200_row_reduce [vector, warp per row]"); "" before the first launch. A diagnostic: sweep
// reports use it to tell tuned paths from the element-wise ones.
extern "C" const char* b200_last_kernel(void) { return b200::t_last_kernel; }

extern "C" const char* b200_last_error(void) { return b200::last_error_buffer(); }

extern "C" int b200_version(void) { return 1; }

extern "C" int b200_sm_count(void) { return b200::device_info().sm_count; }

extern "C" int b200_l2_bytes(void) { return b200::device_info().l2_bytes; }

// Reads the status words of a scratch buffer used by a cooperative kernel (see grid_barrier).
// Synchronises the stream: a diagnostic call, never part of a timed or captured region.
extern "C" int b200_check_status(const void* scratch, void* stream) {
  if (!scratch) return b200::fail(B200_ERR_INVALID, "b200_check_status: null scratch");
  unsigned int words[4] = {0, 0, 0, 0};
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(words, scratch, sizeof(words), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return b200::fail((int)e, "b200_check_status: %s", cudaGetErrorString(e));
  if (words[1] != 0)
    return b200::fail(B200_ERR_DEVICE_WAIT,
                      "a grid-wide wait ran out inside a cooperative kernel (arrivals=%u)", words[0]);
  return B200_OK;
}
