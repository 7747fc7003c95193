// Host-buffer entry point: the caller's A, B and C live in host memory.  B is copied whole; A is
// copied in row blocks, each block's GEMM is launched as soon as its rows have landed, and each
// block of C starts its way back as soon as it is computed, so that the two PCIe directions and
// the tensor cores work at the same time.  Staging buffers are per device, grow-only.
#include "host_entry.h"

#include <mutex>

#include "gemmrc_launch.h"

namespace beam {

namespace {

struct HostPath {
  void* dA = nullptr;
  void* dB = nullptr;
  void* dC = nullptr;
  size_t capA = 0, capB = 0, capC = 0;
  cudaStream_t s_in = nullptr, s_mm = nullptr, s_out = nullptr;
  static constexpr int kMaxBlocks = 64;
  cudaEvent_t landed[kMaxBlocks] = {};
  cudaEvent_t computed[kMaxBlocks] = {};
  bool ready = false;
};

HostPath g_host[64];
std::mutex g_host_mutex;

int grow(void** p, size_t* cap, size_t need) {
  if (*cap >= need) return BEAM_OK;
  if (*p) BEAM_CUDA_TRY(cudaFree(*p), "cudaFree(staging)");
  *p = nullptr;
  *cap = 0;
  BEAM_CUDA_TRY(cudaMalloc(p, need), "cudaMalloc(staging)");
  *cap = need;
  return BEAM_OK;
}

}  // namespace

int gemmrc_from_host(const void* A_host, const void* B_host, void* C_host, int m, int n, int k) {
  if (!A_host || !B_host || !C_host || m <= 0 || n <= 0 || k <= 0) return BEAM_ERR_INVALID_ARG;
  if ((k % 8) != 0 || (n % 8) != 0) return BEAM_ERR_ALIGNMENT;
  int st = BEAM_OK;
  DeviceCtx* ctx = current_device_ctx(&st);
  if (!ctx) return st;
  std::lock_guard<std::mutex> lock(g_host_mutex);
  HostPath& h = g_host[ctx->device];
  if (!h.ready) {
    BEAM_CUDA_TRY(cudaStreamCreateWithFlags(&h.s_in, cudaStreamNonBlocking), "stream");
    BEAM_CUDA_TRY(cudaStreamCreateWithFlags(&h.s_mm, cudaStreamNonBlocking), "stream");
    BEAM_CUDA_TRY(cudaStreamCreateWithFlags(&h.s_out, cudaStreamNonBlocking), "stream");
    for (int i = 0; i < HostPath::kMaxBlocks; ++i) {
      BEAM_CUDA_TRY(cudaEventCreateWithFlags(&h.landed[i], cudaEventDisableTiming), "event");
      BEAM_CUDA_TRY(cudaEventCreateWithFlags(&h.computed[i], cudaEventDisableTiming), "event");
    }
    h.ready = true;
  }
  const size_t bytesA = static_cast<size_t>(m) * k * 2, bytesB = static_cast<size_t>(n) * k * 2,
               bytesC = static_cast<size_t>(m) * n * 2;
  if ((st = grow(&h.dA, &h.capA, bytesA)) != BEAM_OK) return st;
  if ((st = grow(&h.dB, &h.capB, bytesB)) != BEAM_OK) return st;
  if ((st = grow(&h.dC, &h.capC, bytesC)) != BEAM_OK) return st;

  // Row blocks of A: multiples of 256 rows (a pair tile), about 16 blocks, at most kMaxBlocks.
  int rows_per_block = ((m + 15) / 16 + 255) / 256 * 256;
  while ((m + rows_per_block - 1) / rows_per_block > HostPath::kMaxBlocks) rows_per_block *= 2;
  const int blocks = (m + rows_per_block - 1) / rows_per_block;

  BEAM_CUDA_TRY(cudaMemcpyAsync(h.dB, B_host, bytesB, cudaMemcpyHostToDevice, h.s_in), "H2D B");
  GemmPlan plan;
  for (int b = 0; b < blocks; ++b) {
    const int r0 = b * rows_per_block;
    const int rows = (m - r0 < rows_per_block) ? (m - r0) : rows_per_block;
    const char* srcA = static_cast<const char*>(A_host) + static_cast<size_t>(r0) * k * 2;
    char* dstA = static_cast<char*>(h.dA) + static_cast<size_t>(r0) * k * 2;
    char* devC = static_cast<char*>(h.dC) + static_cast<size_t>(r0) * n * 2;
    char* dstC = static_cast<char*>(C_host) + static_cast<size_t>(r0) * n * 2;
    BEAM_CUDA_TRY(cudaMemcpyAsync(dstA, srcA, static_cast<size_t>(rows) * k * 2, cudaMemcpyHostToDevice, h.s_in),
                  "H2D A");
    BEAM_CUDA_TRY(cudaEventRecord(h.landed[b], h.s_in), "event record");
    BEAM_CUDA_TRY(cudaStreamWaitEvent(h.s_mm, h.landed[b], 0), "stream wait");
    st = launch_gemmrc(dstA, h.dB, devC, rows, n, k, plan, h.s_mm);
    if (st != BEAM_OK) return st;
    BEAM_CUDA_TRY(cudaEventRecord(h.computed[b], h.s_mm), "event record");
    BEAM_CUDA_TRY(cudaStreamWaitEvent(h.s_out, h.computed[b], 0), "stream wait");
    BEAM_CUDA_TRY(cudaMemcpyAsync(dstC, devC, static_cast<size_t>(rows) * n * 2, cudaMemcpyDeviceToHost, h.s_out),
                  "D2H C");
  }
  BEAM_CUDA_TRY(cudaStreamSynchronize(h.s_out), "sync");
  BEAM_CUDA_TRY(cudaStreamSynchronize(h.s_mm), "sync");
  BEAM_CUDA_TRY(cudaStreamSynchronize(h.s_in), "sync");
  return BEAM_OK;
}

}  // namespace beam
