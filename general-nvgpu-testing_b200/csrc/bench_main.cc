// beam_bench: times one registry kernel from C++ through the C ABI, with the warm-up / pause / event-timed
// repetitions scheme of the reference's test_pipeline (cuda/cublas.cc:12-40: nrep warm-up launches, a 100 ms sleep,
// nrep launches between two CUDA events; nrep within [1, 64] as in set_default_nrep, cuda/main.cc:37-48, unless
// --nrep asks for more).  No Python, no torch: what a C++ caller of libbeam_b200.so measures.
//
//   beam_bench --kernel cutlass_gemmrc --m 8192 --n 8192 --k 8192 [--nrep 20]
//   beam_bench --kernel cutlass_gemmrc_spec --tb_m 256 --tb_n 128 ...
//   beam_bench --kernel cutlass_gemmrc_splitk --m 128 --n 256 --k 65536 [--slices 0] [--stable 1] [--sets 6]
//
// Split-K kernels are timed over `--sets` rotating input sets (more than the L2 holds, so every call reads HBM).
// Prints one JSON line.
#include <cuda_runtime.h>

#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "../../include/beam_b200.h"

#define CHECK_CUDA(expr)                                                                         \
  do {                                                                                           \
    cudaError_t e_ = (expr);                                                                     \
    if (e_ != cudaSuccess) {                                                                     \
      std::fprintf(stderr, "%s failed: %s\n", #expr, cudaGetErrorString(e_));                    \
      return 2;                                                                                  \
    }                                                                                            \
  } while (0)

namespace {

// fp32 -> fp16 bits, round to nearest even (values here are small and normal)
uint16_t to_half(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  x &= 0x7FFFFFFFu;
  if (x < 0x38800000u) return static_cast<uint16_t>(sign);  // below the smallest normal half: flush (inputs only)
  const uint32_t exp = (x >> 23) - 112, man = x & 0x7FFFFFu;
  uint32_t h = (exp << 10) | (man >> 13);
  const uint32_t rest = man & 0x1FFFu;
  if (rest > 0x1000u || (rest == 0x1000u && (h & 1u))) ++h;
  return static_cast<uint16_t>(sign | h);
}

// uniform in [-scale, scale) from a 64-bit LCG; reproducible across runs
void fill(std::vector<uint16_t>& v, uint64_t seed, float scale) {
  uint64_t s = seed * 6364136223846793005ull + 1442695040888963407ull;
  for (auto& e : v) {
    s = s * 6364136223846793005ull + 1442695040888963407ull;
    const float u = static_cast<float>((s >> 40) & 0xFFFFFF) / 8388608.0f - 1.0f;
    e = to_half(u * scale);
  }
}

struct Args {
  std::string kernel = "cutlass_gemmrc";
  int m = 8192, n = 8192, k = 8192, nrep = 20, tb_m = 128, tb_n = 128, slices = 0, stable = 0, sets = 0;
};

bool parse(int argc, char** argv, Args* a) {
  for (int i = 1; i + 1 < argc; i += 2) {
    const std::string key = argv[i];
    const char* val = argv[i + 1];
    if (key == "--kernel") a->kernel = val;
    else if (key == "--m") a->m = std::atoi(val);
    else if (key == "--n") a->n = std::atoi(val);
    else if (key == "--k") a->k = std::atoi(val);
    else if (key == "--nrep") a->nrep = std::atoi(val);
    else if (key == "--tb_m") a->tb_m = std::atoi(val);
    else if (key == "--tb_n") a->tb_n = std::atoi(val);
    else if (key == "--slices") a->slices = std::atoi(val);
    else if (key == "--stable") a->stable = std::atoi(val);
    else if (key == "--sets") a->sets = std::atoi(val);
    else return false;
  }
  return (argc % 2) == 1 && a->m > 0 && a->n > 0 && a->k > 0 && a->nrep >= 1;
}

}  // namespace

int main(int argc, char** argv) {
  Args a;
  if (!parse(argc, argv, &a)) {
    std::fprintf(stderr, "usage: beam_bench --kernel NAME --m M --n N --k K [--nrep R] [--tb_m .. --tb_n ..] "
                         "[--slices S] [--stable 0|1] [--sets N]\n");
    return 1;
  }
  const bool splitk = a.kernel.find("splitk") != std::string::npos;
  const int sets = a.sets > 0 ? a.sets : (splitk ? 6 : 1);
  const size_t ea = static_cast<size_t>(a.m) * a.k, eb = static_cast<size_t>(a.n) * a.k, ec = static_cast<size_t>(a.m) * a.n;
  std::vector<void*> dA(sets), dB(sets);
  void* dC = nullptr;
  {
    std::vector<uint16_t> ha(ea), hb(eb);
    for (int s = 0; s < sets; ++s) {
      fill(ha, 11 + 2 * s, splitk ? 1.0f : 0.17f);
      fill(hb, 12 + 2 * s, splitk ? 1.0f : 0.17f);
      CHECK_CUDA(cudaMalloc(&dA[s], ea * 2));
      CHECK_CUDA(cudaMalloc(&dB[s], eb * 2));
      CHECK_CUDA(cudaMemcpy(dA[s], ha.data(), ea * 2, cudaMemcpyHostToDevice));
      CHECK_CUDA(cudaMemcpy(dB[s], hb.data(), eb * 2, cudaMemcpyHostToDevice));
    }
  }
  CHECK_CUDA(cudaMalloc(&dC, ec * 2));
  CHECK_CUDA(cudaMemset(dC, 0, ec * 2));
  void* ws = nullptr;
  size_t ws_bytes = 0;
  beam_gemm_cfg cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  if (splitk) {
    cfg.tile_n = a.kernel == "cutlass_gemmrc_splitk_spec" ? a.tb_n : 0;
    cfg.split_k_slices = a.slices;
    cfg.flags = a.stable ? BEAM_FLAG_INPUTS_STABLE : 0;
    ws_bytes = beam_gemmrc_splitk_workspace_bytes(a.m, a.n, a.k, cfg.tile_n, a.slices);
    CHECK_CUDA(cudaMalloc(&ws, ws_bytes > 0 ? ws_bytes : 16));
  }
  cudaStream_t stream;
  CHECK_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
  auto launch = [&](int i) -> int {
    const void* A = dA[i % sets];
    const void* B = dB[i % sets];
    if (a.kernel == "custom_gemmrc_128x128") return beam_custom_gemmrc_128x128(A, B, dC, a.m, a.n, a.k, stream);
    if (a.kernel == "custom_gemmrc_128x256") return beam_custom_gemmrc_128x256(A, B, dC, a.m, a.n, a.k, stream);
    if (a.kernel == "cutlass_gemmrc") return beam_cutlass_gemmrc(A, B, dC, a.m, a.n, a.k, stream);
    if (a.kernel == "cutlass_gemmrc_spec")
      return beam_cutlass_gemmrc_spec(A, B, dC, a.m, a.n, a.k, a.tb_m, a.tb_n, 64, 64, stream);
    if (splitk) return beam_gemmrc_splitk_fp16(A, B, dC, a.m, a.n, a.k, &cfg, ws, ws_bytes, stream);
    return BEAM_ERR_INVALID_ARG;
  };
  for (int i = 0; i < a.nrep; ++i) {
    const int st = launch(i);
    if (st != BEAM_OK) {
      std::fprintf(stderr, "%s: %s [%s]\n", a.kernel.c_str(), beam_status_string(st), beam_last_cuda_error());
      return 3;
    }
  }
  CHECK_CUDA(cudaStreamSynchronize(stream));
  std::this_thread::sleep_for(std::chrono::milliseconds(100));
  cudaEvent_t e0, e1;
  CHECK_CUDA(cudaEventCreate(&e0));
  CHECK_CUDA(cudaEventCreate(&e1));
  CHECK_CUDA(cudaEventRecord(e0, stream));
  for (int i = 0; i < a.nrep; ++i) (void)launch(i);
  CHECK_CUDA(cudaEventRecord(e1, stream));
  CHECK_CUDA(cudaEventSynchronize(e1));
  float ms = 0.f;
  CHECK_CUDA(cudaEventElapsedTime(&ms, e0, e1));
  int word = 0;
  const int dev_st = beam_device_status(0, &word);
  const double per = static_cast<double>(ms) / a.nrep;
  const double tflops = 2.0 * a.m * a.n * static_cast<double>(a.k) / (per * 1e-3) * 1e-12;
  const double gbs = 2.0 * (static_cast<double>(ea) + eb + ec) / (per * 1e-3) * 1e-9;
  std::printf("{\"kernel\": \"%s\", \"m\": %d, \"n\": %d, \"k\": %d, \"nrep\": %d, \"input_sets\": %d, \"us_per_call\": %.3f, "
              "\"tflops\": %.2f, \"algorithmic_GBps\": %.1f, \"device_status\": %d, \"fault_word\": %d}\n",
              a.kernel.c_str(), a.m, a.n, a.k, a.nrep, sets, per * 1e3, tflops, gbs, dev_st, word);
  return dev_st == BEAM_OK ? 0 : 4;
}
