// beam_gemmrc_splitk_noalloc: the split-K rc GEMM for callers that must not allocate.
//
// Who this is for.  The ordinary split-K entry points take a caller-provided workspace, which in practice the
// caller obtains from cudaMalloc or from torch's caching allocator.  Some callers cannot do that at the
// point where they need the GEMM: a host thread inside a latency-critical serving loop (cudaMalloc and
// cudaFree take the driver's allocator lock and cudaFree synchronises the whole device, stalling every
// stream), a process that has handed all device memory to another allocator at start-up so that a late
// cudaMalloc fails, or an embedding runtime whose policy is "no device allocation after initialisation".
// For them the fp32 partial tiles live in a fixed array that is part of this library's device image.
//
// What it costs.  The array is kStaticScratchBytes (16 MiB) of device memory on every GPU that loads the
// library, held until the process exits whether or not this entry point is ever called.  Problems whose
// partials do not fit (slices * M * N * 4 bytes > 16 MiB) are rejected with BEAM_ERR_WORKSPACE.
//
// What it does not do.  It calls no cudaMalloc, cudaFree, or allocating library routine, and it does not use
// the library's per-device context (whose first use allocates a fault word).  The first call on a device
// performs a one-time set-up for that device (symbol address lookup, kernel attributes) and is slower than
// the calls after it.
//
// Sharing.  Every call on a device uses the same array and the array keeps whatever the previous call left
// in it.  Nothing in it has to start at zero: each call's first kernel overwrites every partial element
// (all slices, rows < M, columns < N) that its reduction kernel later reads.  Two calls whose kernels
// overlap on the GPU (different streams, no dependency) race on the array and produce garbage; calls on
// one stream, or ordered by events, are safe.
#include <mutex>

#include "gemmrc_launch.h"
#include "gemmrc_umma.cuh"
#include "splitk_launch.h"

namespace beam {
namespace {

constexpr size_t kStaticScratchBytes = static_cast<size_t>(16) << 20;

// Device-resident scratch.  In host code this name is only a handle for cudaGetSymbolAddress: it is not
// a device address and must never be handed to a kernel as one.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

struct StaticSetup {
  bool ready = false;
  float* scratch = nullptr;  // device address of g_static_scratch on this device
  int sm_count = 0;
};
StaticSetup g_setup[64];
std::mutex g_setup_mutex;

using Kernel64 = GemmShape<64, 8, 1, kModeSplitK>;
using Kernel128 = GemmShape<128, 6, 1, kModeSplitK>;

// One-time per device, with that device current.
int setup_device(int dev, StaticSetup** out) {
  StaticSetup& s = g_setup[dev];
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!s.ready) {
    int major = 0, sms = 0, smem = 0;
    BEAM_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev), "device attribute");
    BEAM_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev), "device attribute");
    BEAM_CUDA_TRY(cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev), "device attribute");
    if (major != 10 || smem < Kernel128::kSmemBytes || smem < Kernel64::kSmemBytes) return BEAM_ERR_NO_DEVICE;
    void* ptr = nullptr;
    BEAM_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_scratch), "cudaGetSymbolAddress(static scratch)");
    if (!ptr) return BEAM_ERR_CUDA;
    BEAM_CUDA_TRY(cudaFuncSetAttribute(gemmrc_umma_kernel<64, 8, 1, kModeSplitK>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, Kernel64::kSmemBytes),
                  "cudaFuncSetAttribute(smem)");
    BEAM_CUDA_TRY(cudaFuncSetAttribute(gemmrc_umma_kernel<128, 6, 1, kModeSplitK>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, Kernel128::kSmemBytes),
                  "cudaFuncSetAttribute(smem)");
    s.scratch = static_cast<float*>(ptr);
    s.sm_count = sms;
    s.ready = true;
  }
  *out = &s;
  return BEAM_OK;
}

template <int BN, int kStages>
int launch_partials(const StaticSetup& s, const void* A, const void* B, void* C, int m, int n, int k, int slices,
                    int* fault_word, cudaStream_t stream) {
  using S = GemmShape<BN, kStages, 1, kModeSplitK>;
  GemmParams p = {};
  int st = encode_tmap_2d(&p.tm_a, A, 2, static_cast<uint64_t>(m), static_cast<uint64_t>(k),
                          static_cast<uint64_t>(k), S::kBM, S::kBK, true);
  if (st != BEAM_OK) return st;
  st = encode_tmap_2d(&p.tm_b, B, 2, static_cast<uint64_t>(n), static_cast<uint64_t>(k), static_cast<uint64_t>(k),
                      S::kBRows, S::kBK, true);
  if (st != BEAM_OK) return st;
  st = encode_tmap_3d_f32(&p.tm_s, s.scratch, static_cast<uint64_t>(slices), static_cast<uint64_t>(m),
                          static_cast<uint64_t>(n), 32, 32);
  if (st != BEAM_OK) return st;
  p.c = static_cast<__half*>(C);
  p.scratch = s.scratch;
  p.row_part = nullptr;
  p.tickets = nullptr;
  p.ln_queue = nullptr;
  p.gamma = nullptr;
  p.beta = nullptr;
  p.eps = 0.f;
  p.m = m;
  p.n = n;
  p.k = k;
  p.ldc = n;
  p.m_tiles = (m + S::kBM - 1) / S::kBM;
  p.n_tiles = (n + BN - 1) / BN;
  p.group_m = 1;
  p.slices = slices;
  p.hint_a = 0;
  p.hint_b = 0;
  p.hint_c = 0;
  p.n_peers = 0;
  p.flags = 0;
  p.fold = 0;
  p.bf16 = 0;
  p.ew_in = nullptr;
  p.ew_out = nullptr;
  p.ew_count = 0;
  p.status = fault_word;
  const long long items = static_cast<long long>(p.m_tiles) * p.n_tiles * slices;
  const int ctas = items < s.sm_count ? static_cast<int>(items) : s.sm_count;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(ctas), 1, 1);
  cfg.blockDim = dim3(S::kThreads, 1, 1);
  cfg.dynamicSmemBytes = S::kSmemBytes;
  cfg.stream = stream;
  BEAM_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemmrc_umma_kernel<BN, kStages, 1, kModeSplitK>, p),
                "cudaLaunchKernelEx(split-K partials)");
  return BEAM_OK;
}

}  // namespace
}  // namespace beam

extern "C" BEAM_API int beam_gemmrc_splitk_noalloc(const void* A, const void* B, void* C, int m, int n, int k,
                                                   int split_k_slices, int* device_fault_word, void* stream_) {
  using namespace beam;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int st = validate_gemm_args(A, B, C, m, n, k);
  if (st != BEAM_OK) return st;
  if (split_k_slices < 0) return BEAM_ERR_INVALID_ARG;
  if (m > 65535) return BEAM_ERR_UNSUPPORTED;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    (void)cudaGetLastError();
    return BEAM_ERR_NO_DEVICE;
  }
  StaticSetup* s = nullptr;
  st = setup_device(dev, &s);
  if (st != BEAM_OK) return st;

  // Tile choice and split rule of the workspace entry point's two-kernel form, computed without the library
  // context, with one difference: problems with M, N <= 64 are not folded here (they run the plain 64-wide tile,
  // one plane per slice), so for those shapes this entry is slower than the workspace one and its sum is
  // associated differently (equal within the parity tolerance, not bit for bit).
  const int bn = splitk_tile_n(n, 0);
  const int num_kb = (k + 63) / 64;
  int slices = split_k_slices;
  if (slices <= 0 || slices > num_kb || slices > 1024) {
    const long long tiles = static_cast<long long>((m + 127) / 128) * ((n + bn - 1) / bn);
    long long h = s->sm_count / (tiles > 0 ? tiles : 1);
    const long long cap = num_kb / 4 > 0 ? num_kb / 4 : 1;
    if (h > cap) h = cap;
    if (h > 256) h = 256;
    if (h < 1) h = 1;
    slices = static_cast<int>(h);
  }
  const size_t need = static_cast<size_t>(slices) * m * n * sizeof(float);
  if (need > kStaticScratchBytes) {
    // Clear refusal: the built-in scratch is fixed-size by design; use the workspace entry point instead.
    return BEAM_ERR_WORKSPACE;
  }

  if (bn == 64)
    st = launch_partials<64, 8>(*s, A, B, C, m, n, k, slices, device_fault_word, stream);
  else
    st = launch_partials<128, 6>(*s, A, B, C, m, n, k, slices, device_fault_word, stream);
  if (st != BEAM_OK) return st;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>((n + 127) / 128), static_cast<unsigned>(m), 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  BEAM_CUDA_TRY(cudaLaunchKernelEx(&cfg, splitk_reduce_kernel, static_cast<const float*>(s->scratch),
                                   static_cast<__half*>(C), m, n, slices),
                "cudaLaunchKernelEx(split-K reduce)");
  return BEAM_OK;
}
