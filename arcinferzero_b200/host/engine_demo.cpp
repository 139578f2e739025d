// Small program over the C++ mirror (engine.hpp): one FFN block of a dense layer as the reference's layer_ffn issues it
// (zero/engine_qwen.h:419-452): quantise -> gate (store) -> up (fused SwiGLU store mode) -> quantise -> down (add to
// the residual).  Prints a checksum; the GPU test compares it with the same sequence through the Python binding.
// usage: engine_demo <rows> <hidden> <ffn> <seed>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>

#include "engine.hpp"

static std::vector<uint8_t> random_q4k(int N, int K, uint32_t seed) {
  std::mt19937 rng(seed);
  std::vector<uint8_t> w((size_t)N * (K / 256) * 144);
  for (auto& b : w) b = (uint8_t)rng();
  for (size_t sb = 0; sb < w.size() / 144; ++sb) {  // fp16 d, dmin in a sane range: 0x1C00..0x2000 = 0.0039..0.0078
    const uint16_t d = (uint16_t)(0x1C00 + rng() % 0x400), m = (uint16_t)(0x1C00 + rng() % 0x400);
    memcpy(&w[sb * 144], &d, 2);
    memcpy(&w[sb * 144 + 2], &m, 2);
  }
  return w;
}

int main(int argc, char** argv) {
  const int T = argc > 1 ? atoi(argv[1]) : 40, E = argc > 2 ? atoi(argv[2]) : 512, F = argc > 3 ? atoi(argv[3]) : 1024;
  const uint32_t seed = argc > 4 ? (uint32_t)atoi(argv[4]) : 1;
  try {
    izb::Engine eng(0);
    const auto wg = random_q4k(F, E, seed), wu = random_q4k(F, E, seed + 1), wd = random_q4k(E, F, seed + 2);
    izb::GpuWeight Wg = eng.make_weight(IZB_Q4_K, wg.data(), F, E), Wu = eng.make_weight(IZB_Q4_K, wu.data(), F, E),
                   Wd = eng.make_weight(IZB_Q4_K, wd.data(), E, F);
    const int Mp = izb::Engine::pad_rows(T);
    eng.alloc_buffers(Mp, F > E ? F : E);
    std::mt19937 rng(seed + 3);
    std::normal_distribution<float> nd(0.0f, 1.0f);
    std::vector<float> x((size_t)T * E);
    for (auto& v : x) v = nd(rng);
    float *dx, *dh, *dres;
    cudaMalloc(&dx, x.size() * 4);
    cudaMalloc(&dh, (size_t)Mp * F * 4);
    cudaMalloc(&dres, (size_t)Mp * E * 4);
    cudaMemcpy(dx, x.data(), x.size() * 4, cudaMemcpyHostToDevice);
    cudaMemset(dres, 0, (size_t)Mp * E * 4);
    eng.set_rows(T);
    eng.quant_rows(dx, E, E, Mp);
    eng.matmul("gemm_gate", Wg, Mp, dh, F, 0, 0);
    eng.matmul("gemm_up", Wu, Mp, dh, F, 0, 2);      // h = up * silu(gate)
    eng.quant_rows(dh, F, F, Mp);
    eng.matmul("gemm_down", Wd, Mp, dres, E, 0, 1);  // residual += h Wd^T
    std::vector<float> out((size_t)T * E);
    cudaMemcpy(out.data(), dres, out.size() * 4, cudaMemcpyDeviceToHost);
    double sum = 0, sq = 0;
    for (float v : out) { sum += v; sq += (double)v * v; }
    printf("rows %d hidden %d ffn %d checksum %.6e l2 %.6e\n", T, E, F, sum, sq);
    // a bad shape must throw before anything is launched
    bool threw = false;
    try { eng.matmul("bad", Wg, Mp, dres, E, 0, 0); } catch (const std::runtime_error&) { threw = true; }  // Wg.K = E, rows hold F
    printf("shape error raised: %s\n", threw ? "yes" : "no");
    cudaFree(dx); cudaFree(dh); cudaFree(dres);
    return threw ? 0 : 2;
  } catch (const std::exception& e) {
    fprintf(stderr, "engine_demo: %s\n", e.what());
    return 1;
  }
}
