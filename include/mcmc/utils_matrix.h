// Source-compatible stand-ins for the reference's buffer types
// (include/mcmc/utils_matrix.h:39-150 there): DeviceMatrix<T> is an owning or
// viewing 2-D device buffer whose `swap` exchanges pointer, shape and view flag —
// the mechanism the reference's driver uses to rotate its parameter buffers
// (main.h:62-75).  Only what the HMC path uses is provided.
#pragma once
#include <cuda_runtime.h>
#include <cstddef>
#include <utility>
#include <vector>

template <typename T>
class DeviceMatrix {
 public:
  DeviceMatrix() = default;
  DeviceMatrix(size_t rows, size_t cols) : rows_(rows), cols_(cols) { cudaMalloc(&data_, nbytes()); }
  // filled with a constant, as DeviceMatrix(M, N, init_val, stream) of the reference
  DeviceMatrix(size_t rows, size_t cols, T init, const cudaStream_t& stream) : DeviceMatrix(rows, cols) {
    std::vector<T> h(rows * cols, init);
    cudaMemcpyAsync(data_, h.data(), nbytes(), cudaMemcpyHostToDevice, stream);
    cudaStreamSynchronize(stream);
  }
  // non-owning view
  DeviceMatrix(size_t rows, size_t cols, T* data) : view_(true), rows_(rows), cols_(cols), data_(data) {}
  DeviceMatrix(const DeviceMatrix&) = delete;
  DeviceMatrix& operator=(const DeviceMatrix&) = delete;
  ~DeviceMatrix() {
    if (!view_ && data_) cudaFree(data_);
  }
  T* ptr() { return data_; }
  const T* ptr() const { return data_; }
  size_t rows() const { return rows_; }
  size_t cols() const { return cols_; }
  size_t nel() const { return rows_ * cols_; }
  size_t nbytes() const { return nel() * sizeof(T); }
  void swap(DeviceMatrix& o) {
    std::swap(view_, o.view_);
    std::swap(rows_, o.rows_);
    std::swap(cols_, o.cols_);
    std::swap(data_, o.data_);
  }

 private:
  bool view_ = false;
  size_t rows_ = 0, cols_ = 0;
  T* data_ = nullptr;
};
