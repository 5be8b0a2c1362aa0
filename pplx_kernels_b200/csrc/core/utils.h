// Host-side helpers: arithmetic, checked CUDA calls, assertions.
//
// Role parity: csrc/core/common_utils.h:15-24 (ceil_div / round_up / next_pow_2),
// csrc/core/cuda_utils.h:7-31 (CUDACHECK, get_sm_count) and csrc/core/utils.h:7-24
// (PPLX_ASSERT) of the reference.  The reference prints and calls exit()/trap on
// failure; here every failure is a C++ exception so that a Python caller sees an
// error it can handle and the process (and the GPU context) stays usable.
#pragma once

#include <cstddef>
#include <cstdint>
#include <sstream>
#include <stdexcept>
#include <string>

#include <cuda_runtime.h>

namespace pplx {

template <typename T>
constexpr __host__ __device__ T ceil_div(T a, T b) {
  return (a + b - 1) / b;
}

template <typename T>
constexpr __host__ __device__ T round_up(T a, T b) {
  return ceil_div<T>(a, b) * b;
}

constexpr __host__ __device__ uint32_t next_pow_2(uint32_t x) {
  uint32_t n = 1;
  while (n < x) n <<= 1;
  return n;
}

class Error : public std::runtime_error {
 public:
  using std::runtime_error::runtime_error;
};

[[noreturn]] inline void fail(const char* file, int line, const std::string& what) {
  std::ostringstream os;
  os << file << ":" << line << ": " << what;
  throw Error(os.str());
}

#define PPLX_CHECK(cond, msg)                                                    \
  do {                                                                           \
    if (!(cond)) {                                                               \
      std::ostringstream _os;                                                    \
      _os << "check failed: " #cond " -- " << msg;                               \
      ::pplx::fail(__FILE__, __LINE__, _os.str());                               \
    }                                                                            \
  } while (0)

#define PPLX_UNREACHABLE(msg) ::pplx::fail(__FILE__, __LINE__, std::string("unreachable: ") + msg)

#define CUDA_CHECK(expr)                                                         \
  do {                                                                           \
    cudaError_t _e = (expr);                                                     \
    if (_e != cudaSuccess) {                                                     \
      ::pplx::fail(__FILE__, __LINE__,                                           \
                   std::string(#expr " -> ") + cudaGetErrorName(_e) + ": " +     \
                       cudaGetErrorString(_e));                                  \
    }                                                                            \
  } while (0)

inline int current_device() {
  int d = 0;
  CUDA_CHECK(cudaGetDevice(&d));
  return d;
}

inline int get_sm_count(int device = -1) {
  if (device < 0) device = current_device();
  int n = 0;
  CUDA_CHECK(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device));
  return n;
}

// Reads an integer knob from the environment once; `fallback` when unset or malformed.
long env_long(const char* name, long fallback);

}  // namespace pplx
