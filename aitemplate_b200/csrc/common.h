// Host-side helpers shared by every translation unit of libb200ait:
// thread-local last-error text, exception -> status conversion, the per-device
// status word that kernels write when a bounded wait gives up.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <stdexcept>
#include <string>

#define B200AIT_EXPORT extern "C" __attribute__((visibility("default")))

namespace b200ait {

void set_last_error(const std::string& msg);
const std::string& last_error();

// device pointer to this device's int status word (allocated on first use, zeroed)
int* device_status_word();

// Process-wide count of kernels this library has launched (every launch site calls count_launch();
// a launch made while a stream is being captured counts once, at capture).
extern std::atomic<uint64_t> g_kernel_launches;
inline void count_launch() { g_kernel_launches.fetch_add(1, std::memory_order_relaxed); }

// number of SMs of the current device (cached per device)
int sm_count();

// Raises a kernel's dynamic shared-memory limit once per device (bit i of `done` = device i).
void opt_in_smem_once(std::atomic<uint64_t>& done, const void* kernel, int bytes);

struct Error : public std::runtime_error {
  using std::runtime_error::runtime_error;
};

#define B200AIT_CUDA_CHECK(expr)                                                              \
  do {                                                                                        \
    cudaError_t _e = (expr);                                                                  \
    if (_e != cudaSuccess) {                                                                  \
      throw ::b200ait::Error(std::string(#expr " failed: ") + cudaGetErrorString(_e));        \
    }                                                                                         \
  } while (0)

#define B200AIT_REQUIRE(cond, msg)                       \
  do {                                                   \
    if (!(cond)) throw ::b200ait::Error(std::string(msg)); \
  } while (0)

// Runs `fn`, converts any exception into a nonzero status + last-error text.
template <class F>
int guarded(const char* where, F&& fn) {
  try {
    fn();
    return 0;
  } catch (const std::exception& e) {
    set_last_error(std::string(where) + ": " + e.what());
    return 1;
  } catch (...) {
    set_last_error(std::string(where) + ": unknown error");
    return 1;
  }
}

enum DType : int { kDTypeHalf = 1, kDTypeFloat = 2, kDTypeInt = 3, kDTypeBFloat16 = 6 };  // values of AITemplateDtype

}  // namespace b200ait
