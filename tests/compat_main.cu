// Builds against include/mcmc/main.h exactly as the reference's main.cu builds
// against its own headers, and exercises mcmc_step / log_acpt_prec / Network on
// device buffers.  Prints the numbers the Python test compares with the oracle.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "mcmc/io.h"
#include "mcmc/main.h"

int main(int argc, char** argv) {
  using namespace mcmc;
  if (argc > 1 && std::string(argv[1]) == "main_loop") {
    main_loop<float>();
    return 0;
  }
  if (argc > 2 && std::string(argv[1]) == "read_data") {  // the reference's reader signature (io.h:42-43)
    DeviceMatrix<float> data(N_SAMPLES, N_COLS), labels(N_SAMPLES, FEAT_DIM[NUM_LAYERS]);
    read_data(data, labels, argv[2]);
    std::printf("read %zu x %zu\n", data.rows(), data.cols());
    return 0;
  }
  cudaStream_t stream = cudaStreamPerThread;
  std::vector<float> hx((size_t)N_SAMPLES * N_COLS), hy(N_SAMPLES);
  mcmc_b200_synth_window(5, 0, N_SAMPLES, N_COLS, FEAT_DIM[1], hx.data(), hy.data(), nullptr);
  for (auto& v : hx) v *= 0.05f;
  DeviceMatrix<float> data(N_SAMPLES, N_COLS), labels(N_SAMPLES, 1);
  cudaMemcpy(data.ptr(), hx.data(), data.nbytes(), cudaMemcpyHostToDevice);
  cudaMemcpy(labels.ptr(), hy.data(), labels.nbytes(), cudaMemcpyHostToDevice);
  Network<float> net(stream);
  DeviceMatrix<float> loss_values(1, N_SAMPLES + NUM_PARAMS), prev_loss(1, N_SAMPLES + NUM_PARAMS),
      prev_mom(1, NUM_PARAMS);
  // bootstrap exactly as main.h:191-202: everything zero, one step
  mcmc_step<float, 1>(data, labels, net.w_prev, net.w_next, net.mom_prev, net.mom_next, net.grad_prev,
                      net.grad_cur, net.grad_next, loss_values, nullptr, 0.01f, stream);
  cudaMemcpyAsync(prev_loss.ptr(), loss_values.ptr(), loss_values.nbytes(), cudaMemcpyDeviceToDevice, stream);
  // momentum: a fixed pattern
  std::vector<float> hm(NUM_PARAMS);
  for (int i = 0; i < NUM_PARAMS; ++i) hm[i] = 0.5f * (float)((i * 37) % 11 - 5) / 5.f;
  cudaMemcpyAsync(prev_mom.ptr(), hm.data(), NUM_PARAMS * 4, cudaMemcpyHostToDevice, stream);
  cudaMemcpyAsync(net.mom_next.ptr(), hm.data(), NUM_PARAMS * 4, cudaMemcpyHostToDevice, stream);
  net.do_swap();
  const float eps = 0.02f;
  mcmc_step<float, 10>(data, labels, net.w_prev, net.w_next, net.mom_prev, net.mom_next, net.grad_prev,
                       net.grad_cur, net.grad_next, loss_values, nullptr, eps, stream);
  float* tmp_storage = nullptr;
  size_t tmp_bytes = 0;
  const float la = log_acpt_prec<float, N_SAMPLES, NUM_PARAMS>(nullptr, prev_loss.ptr(), loss_values.ptr(),
                                                               prev_mom.ptr(), net.mom_next.ptr(),
                                                               net.grad_cur.ptr(), nullptr, tmp_storage,
                                                               tmp_bytes, eps, stream);
  std::vector<float> w(NUM_PARAMS), g(NUM_PARAMS), gn(NUM_PARAMS);
  cudaMemcpy(w.data(), net.w_next.ptr(), NUM_PARAMS * 4, cudaMemcpyDeviceToHost);
  cudaMemcpy(g.data(), net.grad_cur.ptr(), NUM_PARAMS * 4, cudaMemcpyDeviceToHost);
  cudaMemcpy(gn.data(), net.grad_next.ptr(), NUM_PARAMS * 4, cudaMemcpyDeviceToHost);
  std::printf("log_acpt %.9g\n", la);
  double gnz = 0;
  for (float v : gn) gnz += v * v;
  std::printf("grad_next_sq %.9g\n", gnz);
  for (int i = 0; i < NUM_PARAMS; ++i) std::printf("w %d %.9g %.9g\n", i, w[i], g[i]);
  return 0;
}
