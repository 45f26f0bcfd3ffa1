// Library-wide host state: last-error text, per-device status word, device properties.
#include "common.h"

#include <cstring>
#include <mutex>

namespace b200ait {

std::atomic<uint64_t> g_kernel_launches{0};

namespace {
thread_local std::string g_last_error;
constexpr int kMaxDevices = 64;
std::mutex g_mutex;
int* g_status_word[kMaxDevices] = {};
int g_sm_count[kMaxDevices] = {};

int current_device() {
  int dev = 0;
  B200AIT_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) throw Error("device ordinal out of range");
  return dev;
}
}  // namespace

void set_last_error(const std::string& msg) { g_last_error = msg; }
const std::string& last_error() { return g_last_error; }

int* device_status_word() {
  const int dev = current_device();
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_status_word[dev]) {
    int* p = nullptr;
    B200AIT_CUDA_CHECK(cudaMalloc(&p, sizeof(int)));
    B200AIT_CUDA_CHECK(cudaMemset(p, 0, sizeof(int)));
    g_status_word[dev] = p;
  }
  return g_status_word[dev];
}

int sm_count() {
  const int dev = current_device();
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_sm_count[dev]) {
    int n = 0;
    B200AIT_CUDA_CHECK(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
    g_sm_count[dev] = n > 0 ? n : 1;
  }
  return g_sm_count[dev];
}

void opt_in_smem_once(std::atomic<uint64_t>& done, const void* kernel, int bytes) {
  const int dev = current_device();
  const uint64_t bit = 1ull << dev;
  if (done.load(std::memory_order_acquire) & bit) return;
  B200AIT_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  done.fetch_or(bit, std::memory_order_release);
}

}  // namespace b200ait

using namespace b200ait;

// Text of the last error raised on the calling thread by any b200ait_* / AITemplate* entry point.
B200AIT_EXPORT const char* b200ait_last_error() {
  return last_error().c_str();
}

// Reads and clears the current device's kernel status word (0 = no kernel reported a problem;
// otherwise the DeviceError code of the first bounded wait that gave up). Synchronises the device.
B200AIT_EXPORT int b200ait_device_status(int* status_out) {
  return guarded("b200ait_device_status", [&] {
    B200AIT_REQUIRE(status_out, "status_out is null");
    int* w = device_status_word();
    B200AIT_CUDA_CHECK(cudaDeviceSynchronize());
    B200AIT_CUDA_CHECK(cudaMemcpy(status_out, w, sizeof(int), cudaMemcpyDeviceToHost));
    if (*status_out != 0) B200AIT_CUDA_CHECK(cudaMemset(w, 0, sizeof(int)));
  });
}

B200AIT_EXPORT int b200ait_version() { return 1; }

// Number of kernels this library has launched in this process so far (all devices, all threads).
B200AIT_EXPORT int b200ait_kernel_launch_count(int64_t* count_out) {
  return guarded("b200ait_kernel_launch_count", [&] {
    B200AIT_REQUIRE(count_out, "count_out is null");
    *count_out = static_cast<int64_t>(g_kernel_launches.load(std::memory_order_relaxed));
  });
}

// ------------------------------------------------------------------------------------------------
// Peer buffers for multi-GPU runs (one process per GPU on one node): a buffer allocated here can be opened by
// the other ranks through a CUDA IPC handle, which gives them a pointer they can pass as an extra output of
// b200ait_gemm_rcr_multi_out. The handle is 64 opaque bytes that the caller ships to its peers.
B200AIT_EXPORT int b200ait_peer_alloc(int64_t bytes, void** ptr_out, void* handle64_out) {
  return b200ait::guarded("b200ait_peer_alloc", [&] {
    B200AIT_REQUIRE(ptr_out && handle64_out && bytes > 0, "b200ait_peer_alloc: bad argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    void* p = nullptr;
    B200AIT_CUDA_CHECK(cudaMalloc(&p, static_cast<size_t>(bytes)));
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
      cudaFree(p);
      B200AIT_CUDA_CHECK(e);
    }
    memcpy(handle64_out, &h, 64);
    *ptr_out = p;
  });
}
B200AIT_EXPORT int b200ait_peer_open(const void* handle64, void** ptr_out) {
  return b200ait::guarded("b200ait_peer_open", [&] {
    B200AIT_REQUIRE(handle64 && ptr_out, "b200ait_peer_open: bad argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    B200AIT_CUDA_CHECK(cudaIpcOpenMemHandle(ptr_out, h, cudaIpcMemLazyEnablePeerAccess));
  });
}
B200AIT_EXPORT int b200ait_peer_close(void* opened_ptr) {
  return b200ait::guarded("b200ait_peer_close", [&] { B200AIT_CUDA_CHECK(cudaIpcCloseMemHandle(opened_ptr)); });
}
B200AIT_EXPORT int b200ait_peer_free(void* allocated_ptr) {
  return b200ait::guarded("b200ait_peer_free", [&] { B200AIT_CUDA_CHECK(cudaFree(allocated_ptr)); });
}
