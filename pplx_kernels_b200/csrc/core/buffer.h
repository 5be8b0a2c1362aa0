// RAII device / pinned-host buffers and POD strided views.
//
// Role parity: csrc/core/buffer.h:13-161 of the reference (HostBuffer,
// DeviceBuffer, Strided1D/2D/3D).  Differences: buffers are movable, zero-filled
// on request, and a pinned buffer can be mapped so the device can write into it
// (used for the host-visible mirror of the status block, which the kernel thread
// that records a failure fills in).
#pragma once

#include <cstring>
#include <utility>
#include <vector>

#include "utils.h"

namespace pplx {

template <typename T>
class DeviceBuffer {
 public:
  DeviceBuffer() = default;
  explicit DeviceBuffer(size_t n, bool zero = true) : n_(n) {
    if (n_ == 0) return;
    CUDA_CHECK(cudaMalloc(&ptr_, n_ * sizeof(T)));
    if (zero) CUDA_CHECK(cudaMemset(ptr_, 0, n_ * sizeof(T)));
  }
  DeviceBuffer(const DeviceBuffer&) = delete;
  DeviceBuffer& operator=(const DeviceBuffer&) = delete;
  DeviceBuffer(DeviceBuffer&& o) noexcept { swap(o); }
  DeviceBuffer& operator=(DeviceBuffer&& o) noexcept {
    if (this != &o) {
      release();
      swap(o);
    }
    return *this;
  }
  ~DeviceBuffer() { release(); }

  T* get() const { return ptr_; }
  size_t size() const { return n_; }
  size_t bytes() const { return n_ * sizeof(T); }

  void copy_from_host(const T* src, size_t n) {
    PPLX_CHECK(n <= n_, "copy_from_host overflow");
    CUDA_CHECK(cudaMemcpy(ptr_, src, n * sizeof(T), cudaMemcpyHostToDevice));
  }
  void copy_from_host(const std::vector<T>& v) { copy_from_host(v.data(), v.size()); }
  std::vector<T> to_host() const {
    std::vector<T> v(n_);
    if (n_) CUDA_CHECK(cudaMemcpy(v.data(), ptr_, n_ * sizeof(T), cudaMemcpyDeviceToHost));
    return v;
  }

 private:
  void release() {
    if (ptr_) cudaFree(ptr_);
    ptr_ = nullptr;
    n_ = 0;
  }
  void swap(DeviceBuffer& o) {
    std::swap(ptr_, o.ptr_);
    std::swap(n_, o.n_);
  }
  T* ptr_ = nullptr;
  size_t n_ = 0;
};

template <typename T>
class HostBuffer {
 public:
  HostBuffer() = default;
  explicit HostBuffer(size_t n, bool mapped = false) : n_(n) {
    if (n_ == 0) return;
    unsigned flags = mapped ? cudaHostAllocMapped : cudaHostAllocDefault;
    CUDA_CHECK(cudaHostAlloc(&ptr_, n_ * sizeof(T), flags));
    std::memset(ptr_, 0, n_ * sizeof(T));
  }
  HostBuffer(const HostBuffer&) = delete;
  HostBuffer& operator=(const HostBuffer&) = delete;
  HostBuffer(HostBuffer&& o) noexcept { swap(o); }
  HostBuffer& operator=(HostBuffer&& o) noexcept {
    if (this != &o) {
      release();
      swap(o);
    }
    return *this;
  }
  ~HostBuffer() { release(); }

  T* get() const { return ptr_; }
  size_t size() const { return n_; }
  T& operator[](size_t i) { return ptr_[i]; }
  const T& operator[](size_t i) const { return ptr_[i]; }

  // Device-side alias of a mapped allocation.
  T* device_ptr() const {
    T* d = nullptr;
    CUDA_CHECK(cudaHostGetDevicePointer(reinterpret_cast<void**>(&d), ptr_, 0));
    return d;
  }

 private:
  void release() {
    if (ptr_) cudaFreeHost(ptr_);
    ptr_ = nullptr;
    n_ = 0;
  }
  void swap(HostBuffer& o) {
    std::swap(ptr_, o.ptr_);
    std::swap(n_, o.n_);
  }
  T* ptr_ = nullptr;
  size_t n_ = 0;
};

// Strides are in elements of T.
template <typename T>
struct Strided1D {
  T* data = nullptr;
  int64_t stride = 1;
};

template <typename T>
struct Strided2D {
  T* data = nullptr;
  int64_t stride_row = 0;
  int64_t stride_col = 1;
};

template <typename T>
struct Strided3D {
  T* data = nullptr;
  int64_t stride_outer = 0;
  int64_t stride_row = 0;
  int64_t stride_col = 1;
};

}  // namespace pplx
