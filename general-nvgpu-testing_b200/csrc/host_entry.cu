// Host-buffer entry points: the caller's A and C (and, in the first form, B) live in host memory.
//
// PCIe is the whole cost here (at 8192^3 the kernel needs 0.7 ms, the copies 5 to 6), and the link carries less in
// each direction when both are busy than when one is (measured on B200 hosts: 55 GB/s one way, about 79 GB/s for
// both together).  So the schedule is built to keep both directions busy for as long as possible: A and B go up in
// row blocks, alternating, and after every arrival the strip of C that has just become computable (the new rows of
// A against every row of B that has landed, or the new rows of B against every row of A) is multiplied and starts
// its way back at once.  The computable area grows like a square, C begins to flow after the second block instead
// of after all of B, and only the last strip's copy is left when the uploads end.  Copies in, kernels and copies
// out run on three streams ordered by events; staging buffers are per device and grow-only.
#include "host_entry.h"

#include <mutex>

#include "gemmrc_launch.h"

namespace beam {

namespace {

struct HostPath {
  std::mutex mutex;  // one call at a time per device (the staging buffers are shared)
  void* dA = nullptr;
  void* dB = nullptr;
  void* dC = nullptr;
  size_t capA = 0, capB = 0, capC = 0;
  cudaStream_t s_in = nullptr, s_mm = nullptr, s_out = nullptr;
  static constexpr int kMaxSteps = 64;
  cudaEvent_t landed[kMaxSteps] = {};
  cudaEvent_t computed[kMaxSteps] = {};
  bool ready = false;
};

HostPath g_host[64];

int grow(void** p, size_t* cap, size_t need) {
  if (*cap >= need) return BEAM_OK;
  if (*p) BEAM_CUDA_TRY(cudaFree(*p), "cudaFree(staging)");
  *p = nullptr;
  *cap = 0;
  BEAM_CUDA_TRY(cudaMalloc(p, need), "cudaMalloc(staging)");
  *cap = need;
  return BEAM_OK;
}

// Rows per block: about an eighth of the dimension, a multiple of 256 (a pair tile), so that fewer than
// kMaxSteps / 2 blocks cover it (the last regular block is cut in two, see next_block).
int block_rows(int dim) {
  int rows = ((dim + 7) / 8 + 255) / 256 * 256;
  while ((dim + rows - 1) / rows + 1 > HostPath::kMaxSteps / 2) rows *= 2;
  return rows;
}

// Rows of the next block when `left` rows remain: the regular block, except that the last regular block is cut in
// two, so that the strip whose copy back nothing overlaps any more (the last one) is half as long.
int next_block(int left, int blk) {
  if (left > blk) return blk;
  const int half = ((left + 1) / 2 + 255) / 256 * 256;
  return (left > 512 && half < left) ? half : left;
}

// The body of a call; any failure leaves work in flight on the internal streams, which the caller drains.
int run_pipeline(HostPath& h, const void* A_host, const void* B_host, const void* B_dev, void* C_host, int m, int n,
                 int k) {
  const size_t row_a = static_cast<size_t>(k) * 2, row_c = static_cast<size_t>(n) * 2;
  int st;
  if ((st = grow(&h.dA, &h.capA, static_cast<size_t>(m) * row_a)) != BEAM_OK) return st;
  if ((st = grow(&h.dC, &h.capC, static_cast<size_t>(m) * row_c)) != BEAM_OK) return st;
  const char* devB = static_cast<const char*>(B_dev);
  if (!devB) {
    if ((st = grow(&h.dB, &h.capB, static_cast<size_t>(n) * row_a)) != BEAM_OK) return st;
    devB = static_cast<const char*>(h.dB);
  }
  const int blk_a = block_rows(m), blk_b = block_rows(n);
  int a_done = 0, b_done = B_dev ? n : 0;  // rows of A / of B whose upload has been queued
  int step = 0;
  while (a_done < m || b_done < n) {
    // B goes first and the two alternate while both have rows left (the computable area stays close to a square).
    const bool take_b = b_done < n && (a_done >= m || b_done <= a_done);
    const int r0 = take_b ? b_done : a_done;
    const int rows = next_block(take_b ? n - r0 : m - r0, take_b ? blk_b : blk_a);
    const char* src = static_cast<const char*>(take_b ? B_host : A_host) + static_cast<size_t>(r0) * row_a;
    char* dst = (take_b ? static_cast<char*>(h.dB) : static_cast<char*>(h.dA)) + static_cast<size_t>(r0) * row_a;
    BEAM_CUDA_TRY(cudaMemcpyAsync(dst, src, static_cast<size_t>(rows) * row_a, cudaMemcpyHostToDevice, h.s_in), "H2D");
    BEAM_CUDA_TRY(cudaEventRecord(h.landed[step], h.s_in), "event record");
    // the strip of C that became computable: new rows x landed columns, or landed rows x new columns
    const int c_r0 = take_b ? 0 : r0, c_rows = take_b ? a_done : rows;
    const int c_c0 = take_b ? r0 : 0, c_cols = take_b ? rows : b_done;
    if (take_b)
      b_done += rows;
    else
      a_done += rows;
    if (c_rows > 0 && c_cols > 0) {
      BEAM_CUDA_TRY(cudaStreamWaitEvent(h.s_mm, h.landed[step], 0), "stream wait");
      GemmPlan plan;
      plan.ldc = n;
      plan.whole_tiles = 1;  // the copies set the pace here; whole tiles keep every strip's bits those of one whole GEMM
      // the headline tile (256 x 512 per CTA pair) once a strip fills most of a wave of them; 256 x 256 below that
      if (static_cast<long long>((c_rows + 255) / 256) * ((c_cols + 511) / 512) >= 48) plan.tile_n = 512;
      char* devC = static_cast<char*>(h.dC) + static_cast<size_t>(c_r0) * row_c + static_cast<size_t>(c_c0) * 2;
      st = launch_gemmrc(static_cast<const char*>(h.dA) + static_cast<size_t>(c_r0) * row_a,
                         devB + static_cast<size_t>(c_c0) * row_a, devC, c_rows, c_cols, k, plan, h.s_mm);
      if (st != BEAM_OK) return st;
      BEAM_CUDA_TRY(cudaEventRecord(h.computed[step], h.s_mm), "event record");
      BEAM_CUDA_TRY(cudaStreamWaitEvent(h.s_out, h.computed[step], 0), "stream wait");
      char* hostC = static_cast<char*>(C_host) + static_cast<size_t>(c_r0) * row_c + static_cast<size_t>(c_c0) * 2;
      BEAM_CUDA_TRY(cudaMemcpy2DAsync(hostC, row_c, devC, row_c, static_cast<size_t>(c_cols) * 2,
                                      static_cast<size_t>(c_rows), cudaMemcpyDeviceToHost, h.s_out),
                    "D2H C");
    }
    ++step;
  }
  return BEAM_OK;
}

int from_host(const void* A_host, const void* B_host, const void* B_dev, void* C_host, int m, int n, int k) {
  if (!A_host || !(B_host || B_dev) || !C_host || m <= 0 || n <= 0 || k <= 0) return BEAM_ERR_INVALID_ARG;
  if ((k % 8) != 0 || (n % 8) != 0) return BEAM_ERR_ALIGNMENT;
  if (B_dev && !aligned16(B_dev)) return BEAM_ERR_ALIGNMENT;
  int st = BEAM_OK;
  DeviceCtx* ctx = current_device_ctx(&st);
  if (!ctx) return st;
  HostPath& h = g_host[ctx->device];
  std::lock_guard<std::mutex> lock(h.mutex);
  if (!h.ready) {
    BEAM_CUDA_TRY(cudaStreamCreateWithFlags(&h.s_in, cudaStreamNonBlocking), "stream");
    BEAM_CUDA_TRY(cudaStreamCreateWithFlags(&h.s_mm, cudaStreamNonBlocking), "stream");
    BEAM_CUDA_TRY(cudaStreamCreateWithFlags(&h.s_out, cudaStreamNonBlocking), "stream");
    for (int i = 0; i < HostPath::kMaxSteps; ++i) {
      BEAM_CUDA_TRY(cudaEventCreateWithFlags(&h.landed[i], cudaEventDisableTiming), "event");
      BEAM_CUDA_TRY(cudaEventCreateWithFlags(&h.computed[i], cudaEventDisableTiming), "event");
    }
    h.ready = true;
  }
  st = run_pipeline(h, A_host, B_host, B_dev, C_host, m, n, k);
  // Success or not, nothing of this call may still be in flight when it returns: the next call reuses the staging
  // buffers and events, and the copies out target the caller's memory.
  const cudaError_t e_out = cudaStreamSynchronize(h.s_out);
  const cudaError_t e_mm = cudaStreamSynchronize(h.s_mm);
  const cudaError_t e_in = cudaStreamSynchronize(h.s_in);
  if (st != BEAM_OK) return st;
  BEAM_CUDA_TRY(e_out, "sync");
  BEAM_CUDA_TRY(e_mm, "sync");
  BEAM_CUDA_TRY(e_in, "sync");
  return BEAM_OK;
}

}  // namespace

int gemmrc_from_host(const void* A_host, const void* B_host, void* C_host, int m, int n, int k) {
  if (!B_host) return BEAM_ERR_INVALID_ARG;
  return from_host(A_host, B_host, nullptr, C_host, m, n, k);
}

int gemmrc_rows_from_host(const void* A_host, const void* B_dev, void* C_host, int m, int n, int k) {
  if (!B_dev) return BEAM_ERR_INVALID_ARG;
  return from_host(A_host, nullptr, B_dev, C_host, m, n, k);
}

}  // namespace beam
