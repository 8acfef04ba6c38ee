// mcmc::read_data with the reference's signature (include/mcmc/io.h:42-80
// there): fills the device matrices from DATA_FNAME in the reference's text
// layout.  Sizes are checked like there; a failure throws instead of aborting.
// The features are returned UNSCALED, as the reference's read_data leaves them
// (its main_loop scales by 0.001 afterwards, main.h:162-164).
#pragma once
#include <stdexcept>
#include <string>
#include <vector>

#include "../mcmc_b200.h"
#include "global_params.h"
#include "utils_matrix.h"

namespace mcmc {

template <typename T>
void read_data(DeviceMatrix<T>& x_out, DeviceMatrix<T>& y_out, const char* path = DATA_FNAME) {
  static_assert(sizeof(T) == sizeof(float), "the library stores the dataset in FP32");
  if (x_out.rows() != (size_t)N_SAMPLES || x_out.cols() != (size_t)N_COLS)
    throw std::runtime_error("read_data: expected a data matrix of N_SAMPLES x N_COLS");
  if (y_out.rows() != (size_t)N_SAMPLES || y_out.cols() != (size_t)FEAT_DIM[NUM_LAYERS])
    throw std::runtime_error("read_data: expected a label matrix of N_SAMPLES x 1");
  std::vector<float> x((size_t)N_SAMPLES * N_COLS), y(N_SAMPLES);
  if (mcmc_b200_read_table(path, N_SAMPLES, TOTAL_COLS, SKIP_COLS, N_COLS, 1.0f, x.data(), y.data()) !=
      MCMC_B200_OK)
    throw std::runtime_error(std::string("read_data: ") + mcmc_b200_last_error());
  cudaMemcpy(x_out.ptr(), x.data(), x_out.nbytes(), cudaMemcpyHostToDevice);
  cudaMemcpy(y_out.ptr(), y.data(), y_out.nbytes(), cudaMemcpyHostToDevice);
}

}  // namespace mcmc
