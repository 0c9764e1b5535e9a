// Test fixture: a caller written against the reference runtime's own names (GPUTransformer, TPGroup, tp_init,
// tp_group_barrier, moe_gpu_120b), compiled with the host compiler against include/moe_b200_shim.hpp and run by
// tests/test_shim_gpu.py.  One process, one host thread per GPU, as the reference runs its TP groups
// (getp-csrc/getp_run.cpp:3514-3517).  Usage: shim_caller <dir> <tp>; tensors are raw dumps in <dir>.
#include <cstdint>
#include <cstdio>
#include <fstream>
#include <string>
#include <thread>
#include <vector>

#include "moe_b200_shim.hpp"

static std::vector<uint8_t> slurp(const std::string &path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) { fprintf(stderr, "cannot read %s\n", path.c_str()); exit(2); }
  return std::vector<uint8_t>((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
}

int main(int argc, char **argv) {
  if (argc < 3) return 2;
  const std::string dir = argv[1];
  const int tp = atoi(argv[2]);
  int E, H, D, T;
  {
    FILE *f = fopen((dir + "/cfg.txt").c_str(), "r");
    if (!f || fscanf(f, "%d %d %d %d", &E, &H, &D, &T) != 4) return 2;
    fclose(f);
  }
  const auto w1c = slurp(dir + "/w1_codes.bin"), w1s = slurp(dir + "/w1_scales.bin"), b1 = slurp(dir + "/b1.bin");
  const auto w2c = slurp(dir + "/w2_codes.bin"), w2s = slurp(dir + "/w2_scales.bin"), b2 = slurp(dir + "/b2.bin");
  const auto rw = slurp(dir + "/router_w.bin"), rb = slurp(dir + "/router_b.bin");
  const auto x = slurp(dir + "/x.bin"), gain = slurp(dir + "/gain.bin");
  const int rows_local = T / tp;

  // start-up, as the reference's main thread does before it spawns its per-device threads
  for (int r = 0; r < tp; ++r) {
    if (cudaSetDevice(r) != cudaSuccess) return 3;
    moe_config cfg = {};
    cfg.hidden_dim = H; cfg.intermediate_dim = D; cfg.n_experts = E; cfg.experts_per_token = 4; cfg.n_layers = 1;
    cfg.swiglu_limit = 7.0f; cfg.swiglu_alpha = 1.702f; cfg.max_rows = T; cfg.tp_size = tp; cfg.tp_rank = r; cfg.device = r;
    moe_handle &h = moe_b200_handles()[r];
    int rc = moe_create(&cfg, &h);
    if (rc == MOE_OK)
      rc = moe_load_layer(h, 0, w1c.data(), w1s.data(), reinterpret_cast<const uint16_t *>(b1.data()), w2c.data(), w2s.data(),
                          reinterpret_cast<const uint16_t *>(b2.data()), reinterpret_cast<const float *>(rw.data()),
                          reinterpret_cast<const float *>(rb.data()));
    if (rc != MOE_OK) moe_b200_die(h, "start-up", rc);
    tp_init(tp_groups()[r], tp, r, tp);
  }
  if (tp > 1)
    for (int r = 0; r < tp; ++r) {
      cudaSetDevice(r);
      moe_b200_connect_group(tp_groups()[r]);
    }

  std::vector<uint8_t> out(x.size());
  std::vector<std::thread> threads;
  for (int r = 0; r < tp; ++r)
    threads.emplace_back([&, r] {
      cudaSetDevice(r);
      const size_t bytes = static_cast<size_t>(rows_local) * H * 2;
      void *d_x = nullptr, *d_gain = nullptr;
      cudaMalloc(&d_x, bytes);
      cudaMalloc(&d_gain, static_cast<size_t>(H) * 2);
      cudaMemcpy(d_x, x.data() + static_cast<size_t>(r) * bytes, bytes, cudaMemcpyHostToDevice);
      cudaMemcpy(d_gain, gain.data(), static_cast<size_t>(H) * 2, cudaMemcpyHostToDevice);
      cudaStream_t sMoe;
      cudaStreamCreate(&sMoe);
      GPUTransformer gt = {};
      gt.config.hidden_dim = H;
      gt.weights.rms_ffn_w = d_gain;
      gt.state.x = d_x;
      tp_group_barrier(tp_groups()[r]);
      moe_gpu_120b(&gt, 0, rows_local, 0, sMoe);       // x += MoE(rmsnorm(x) * gain), in place
      cudaStreamSynchronize(sMoe);
      const int rc = moe_synchronize(moe_b200_handles()[r]);
      if (rc != MOE_OK) moe_b200_die(moe_b200_handles()[r], "moe_synchronize", rc);
      cudaMemcpy(out.data() + static_cast<size_t>(r) * bytes, d_x, bytes, cudaMemcpyDeviceToHost);
      tp_group_barrier(tp_groups()[r]);
      cudaFree(d_x);
      cudaFree(d_gain);
      cudaStreamDestroy(sMoe);
    });
  for (auto &t : threads) t.join();
  for (int r = 0; r < tp; ++r) {
    cudaSetDevice(r);
    moe_destroy(moe_b200_handles()[r]);
  }
  std::ofstream f(dir + "/x_out.bin", std::ios::binary);
  f.write(reinterpret_cast<const char *>(out.data()), static_cast<std::streamsize>(out.size()));
  printf("shim_caller ok tp=%d\n", tp);
  return 0;
}
