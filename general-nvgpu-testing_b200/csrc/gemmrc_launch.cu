// Host launchers of the persistent UMMA kernels: validate the problem, pick the kernel
// instantiation named by the plan, build the TMA descriptors and launch on the caller's stream.
#include "gemmrc_launch.h"

#include <mutex>

#include "gemmrc_umma.cuh"
#include "gemm_ln_resident.cuh"
#include "gemmrc_dual.cuh"
#include "gemmrc_wide.cuh"
#include "layernorm_launch.h"
#include "splitk_launch.h"
#include "splitk_stream.cuh"

namespace beam {


namespace {

struct ExtraArgs {
  float* scratch = nullptr;
  const __half* gamma = nullptr;
  const __half* beta = nullptr;
  float eps = 0.f;
  int slices = 1;
  int l2_hints = 0;
  int flags = 0;
  int fold = 0;
  int bf16 = 0;
  int whole_tiles = 0;  // 1 = never cut the tiles of the last wave in two (256 x 256 tiles on pairs)
  int ldc = 0;  // row pitch of C in elements (0 = n): GEMM-mode kernels store C through a tensor map, so a pitch costs nothing
  const __half* ew_in = nullptr;
  __half* ew_out = nullptr;
  long long ew_count = 0;
  const void* peer_c[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};  // fused all-gather
  int n_peers = 0;
  float2* row_part = nullptr;
  int* tickets = nullptr;
  int* ln_queue = nullptr;
};

// How many 2-CTA clusters of `kernel` the device holds at once (a GPC with an odd number of free SMs leaves one
// unpaired, so this can be less than half the SM count).
template <typename Kernel>
int resident_pairs(Kernel kernel, int threads, int smem_bytes, int sm_count) {
  int pairs = sm_count / 2;
  cudaLaunchConfig_t probe = {};
  probe.gridDim = dim3(static_cast<unsigned>(sm_count / 2 * 2), 1, 1);
  probe.blockDim = dim3(static_cast<unsigned>(threads), 1, 1);
  probe.dynamicSmemBytes = static_cast<size_t>(smem_bytes);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  probe.attrs = attr;
  probe.numAttrs = 1;
  int n_clusters = 0;
  cudaError_t e = cudaOccupancyMaxActiveClusters(&n_clusters, kernel, &probe);
  if (e == cudaSuccess && n_clusters > 0 && n_clusters < pairs) pairs = n_clusters;
  (void)cudaGetLastError();
  return pairs > 0 ? pairs : 1;
}

template <int BN, int kStages, int kCta, int kMode>
int launch_instance(DeviceCtx* ctx, const void* A, const void* B, void* C, int m, int n, int k, int group_m,
                    int max_ctas, const ExtraArgs& ex, cudaStream_t stream) {
  using S = GemmShape<BN, kStages, kCta, kMode>;
  auto kernel = gemmrc_umma_kernel<BN, kStages, kCta, kMode>;

  // One-time per (instantiation, device): opt in to the large dynamic shared memory and, for
  // pairs, ask how many 2-CTA clusters fit on this part at once.
  static int configured_clusters[64] = {0};
  static std::mutex configure_mutex;
  int resident = 0;
  {
    std::lock_guard<std::mutex> lock(configure_mutex);
    resident = configured_clusters[ctx->device];
  }
  if (resident == 0) {
    std::lock_guard<std::mutex> lock(configure_mutex);
    if (S::kSmemBytes > ctx->max_smem_optin) return BEAM_ERR_UNSUPPORTED;
    BEAM_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kSmemBytes),
                  "cudaFuncSetAttribute(smem)");
    int clusters = ctx->sm_count / kCta;
    if (kCta == 2) clusters = resident_pairs(kernel, S::kThreads, S::kSmemBytes, ctx->sm_count);
    resident = clusters > 0 ? clusters : 1;
    configured_clusters[ctx->device] = resident;
  }

  GemmParams p = {};
  const bool fold = is_splitk_mode(kMode) && BN == 128 && kCta == 1 && ex.fold != 0;
  int st = encode_tmap_2d(&p.tm_a, A, 2, static_cast<uint64_t>(m), static_cast<uint64_t>(k),
                          static_cast<uint64_t>(k), fold ? S::kBM / 2 : S::kBM, S::kBK, true);
  if (st != BEAM_OK) return st;
  st = encode_tmap_2d(&p.tm_b, B, 2, static_cast<uint64_t>(n), static_cast<uint64_t>(k), static_cast<uint64_t>(k),
                      fold ? S::kBRows / 2 : S::kBRows, S::kBK, true);
  if (st != BEAM_OK) return st;
  p.fold = fold ? 1 : 0;
  p.bf16 = (kMode == kModeGemm) ? ex.bf16 : 0;
  p.ew_in = ex.ew_in;
  p.ew_out = ex.ew_out;
  p.ew_count = ex.ew_count;
  if (kMode == kModeGemm || kMode == kModeGemmSilu) {
    st = encode_tmap_2d(&p.tm_c, C, 2, static_cast<uint64_t>(m), static_cast<uint64_t>(n),
                        static_cast<uint64_t>(ex.ldc > 0 ? ex.ldc : n), 32, 64, true);
  } else {
    st = encode_tmap_3d_f32(&p.tm_s, ex.scratch, static_cast<uint64_t>(ex.slices) * (fold ? 2 : 1),
                            static_cast<uint64_t>(m),
                            static_cast<uint64_t>(n), 32, 32);
  }
  if (st != BEAM_OK) return st;
  if (kMode == kModeGemm) {
    for (int d = 0; d < ex.n_peers; ++d) {
      st = encode_tmap_2d(&p.tm_peer[d], ex.peer_c[d], 2, static_cast<uint64_t>(m), static_cast<uint64_t>(n),
                          static_cast<uint64_t>(n), 32, 64, true);
      if (st != BEAM_OK) return st;
    }
    p.n_peers = ex.n_peers;
  }
  p.c = static_cast<__half*>(C);
  p.scratch = ex.scratch;
  p.row_part = ex.row_part;
  p.tickets = ex.tickets;
  p.ln_queue = ex.ln_queue;
  p.gamma = ex.gamma;
  p.beta = ex.beta;
  p.eps = ex.eps;
  p.m = m;
  p.n = n;
  p.k = k;
  p.ldc = n;
  const int tile_m = S::kBM * kCta;
  p.m_tiles = (m + tile_m - 1) / tile_m;
  p.n_tiles = (n + BN - 1) / BN;
  p.group_m = group_m > 0 ? group_m : (kCta == 2 ? 8 : 16);
  p.slices = ex.slices;
  p.hint_a = (ex.l2_hints / 10) % 10;
  p.hint_b = ex.l2_hints % 10;
  p.hint_c = (ex.l2_hints / 100) % 10;
  p.flags = ex.flags;
  p.status = ctx->status_word;

  long long items = static_cast<long long>(p.m_tiles) * p.n_tiles * p.slices;
  int clusters = resident;
  if (max_ctas > 0 && max_ctas / kCta < clusters) clusters = max_ctas / kCta > 0 ? max_ctas / kCta : 1;
  if (S::kCutTiles) {
    // The last wave of the persistent grid: when its tiles occupy at most half of the pairs, they are cut into
    // 128-column halves, which occupy twice as many pairs for a shorter time (4096^3: 256 tiles on 74 pairs are
    // 3 waves and 34 tiles; as 68 halves those take 0.77 of a wave instead of a whole one, measured).  At most one
    // cut item per pair, and it is the pair's last: the kernel relies on both.
    st = encode_tmap_2d(&p.tm_b_tail, B, 2, static_cast<uint64_t>(n), static_cast<uint64_t>(k),
                        static_cast<uint64_t>(k), S::kBRows / 2, S::kBK, true);
    if (st != BEAM_OK) return st;
    const int last_wave = static_cast<int>(items % clusters);
    if (!ex.whole_tiles && last_wave > 0 && 2 * last_wave <= clusters && n > BN / 2 && k > 64) {
      p.tail_tiles = last_wave;
      items += last_wave;
    }
  }
  if (items < clusters) clusters = static_cast<int>(items);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(clusters * kCta), 1, 1);
  cfg.blockDim = dim3(S::kThreads, 1, 1);
  cfg.dynamicSmemBytes = S::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kCta;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (kMode == kModeLayerNorm) {
    // CTAs of this grid wait for one another (the drain of the second pass): place the whole grid or none of it.
    attr[cfg.numAttrs].id = cudaLaunchAttributeCooperative;
    attr[cfg.numAttrs].val.cooperative = 1;
    ++cfg.numAttrs;
  }
  if (is_splitk_mode(kMode) || kMode == kModeGemm) {
    // May start while the previous kernel on the stream drains; the kernel itself waits for that grid's
    // completion before its first global read or write.
    attr[cfg.numAttrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[cfg.numAttrs].val.programmaticStreamSerializationAllowed = 1;
    ++cfg.numAttrs;
  }
  BEAM_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, p), "cudaLaunchKernelEx(gemmrc_umma)");
  return BEAM_OK;
}

// 256 x 512 tiles on CTA pairs (gemmrc_wide.cuh).
template <int kStages, bool kTall>
int launch_wide_instance(DeviceCtx* ctx, const void* A, const void* B, void* C, int m, int n, int k, int group_m,
                         int max_ctas, const ExtraArgs& ex, cudaStream_t stream) {
  using S = WideShape<kStages>;
  auto kernel = gemmrc_wide_kernel<kStages, kTall>;
  static int configured_clusters[64] = {0};
  static std::mutex configure_mutex;
  int resident = 0;
  {
    std::lock_guard<std::mutex> lock(configure_mutex);
    resident = configured_clusters[ctx->device];
  }
  if (resident == 0) {
    std::lock_guard<std::mutex> lock(configure_mutex);
    if (S::kSmemBytes > ctx->max_smem_optin) return BEAM_ERR_UNSUPPORTED;
    BEAM_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kSmemBytes),
                  "cudaFuncSetAttribute(smem)");
    resident = resident_pairs(kernel, S::kThreads, S::kSmemBytes, ctx->sm_count);
    configured_clusters[ctx->device] = resident;
  }
  GemmParams p = {};
  int st = encode_tmap_2d(&p.tm_a, A, 2, static_cast<uint64_t>(m), static_cast<uint64_t>(k),
                          static_cast<uint64_t>(k), S::kBM, S::kBK, true);
  if (st != BEAM_OK) return st;
  st = encode_tmap_2d(&p.tm_b, B, 2, static_cast<uint64_t>(n), static_cast<uint64_t>(k), static_cast<uint64_t>(k),
                      S::kBRows, S::kBK, true);
  if (st != BEAM_OK) return st;
  st = encode_tmap_2d(&p.tm_c, C, 2, static_cast<uint64_t>(m), static_cast<uint64_t>(n),
                      static_cast<uint64_t>(ex.ldc > 0 ? ex.ldc : n), 32, 64, true);
  if (st != BEAM_OK) return st;
  for (int d = 0; d < ex.n_peers; ++d) {
    st = encode_tmap_2d(&p.tm_peer[d], ex.peer_c[d], 2, static_cast<uint64_t>(m), static_cast<uint64_t>(n),
                        static_cast<uint64_t>(n), 32, 64, true);
    if (st != BEAM_OK) return st;
  }
  p.n_peers = ex.n_peers;
  p.bf16 = ex.bf16;
  p.c = static_cast<__half*>(C);
  p.m = m;
  p.n = n;
  p.k = k;
  p.ldc = n;
  p.m_tiles = kTall ? (m + 511) / 512 : (m + 255) / 256;
  p.n_tiles = kTall ? (n + 255) / 256 : (n + S::kTileN - 1) / S::kTileN;
  p.group_m = group_m > 0 ? group_m : (kTall ? 8 : 16);
  p.slices = 1;
  p.lead_in = 2;
  p.lead_out = 2;
  p.hint_a = (ex.l2_hints / 10) % 10;
  p.hint_b = ex.l2_hints % 10;
  p.hint_c = (ex.l2_hints / 100) % 10;
  p.status = ctx->status_word;
  const long long items = static_cast<long long>(p.m_tiles) * p.n_tiles;
  int clusters = resident;
  if (max_ctas > 0 && max_ctas / 2 < clusters) clusters = max_ctas / 2 > 0 ? max_ctas / 2 : 1;
  if (items < clusters) clusters = static_cast<int>(items);
  if (max_ctas < 0 && items < 30000) clusters = static_cast<int>(items);  // one tile per pair, no persistence
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(clusters * 2), 1, 1);
  cfg.blockDim = dim3(S::kThreads, 1, 1);
  cfg.dynamicSmemBytes = S::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // a programmatic dependent of the kernel before it: set-up overlaps that kernel's tail (the kernel waits for it)
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  BEAM_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, p), "cudaLaunchKernelEx(gemmrc_wide)");
  return BEAM_OK;
}

// 128-wide tiles, two of them in flight per CTA or CTA pair (gemmrc_dual.cuh).
template <int kStages, int kCta>
int launch_dual_instance(DeviceCtx* ctx, const void* A, const void* B, void* C, int m, int n, int k, int group_m,
                         int max_ctas, const ExtraArgs& ex, cudaStream_t stream) {
  using S = DualShape<kStages, kCta>;
  auto kernel = gemmrc_dual_kernel<kStages, kCta>;
  static int configured_clusters[64] = {0};
  static std::mutex configure_mutex;
  int resident = 0;
  {
    std::lock_guard<std::mutex> lock(configure_mutex);
    resident = configured_clusters[ctx->device];
    if (resident == 0) {
      if (S::kSmemBytes > ctx->max_smem_optin) return BEAM_ERR_UNSUPPORTED;
      BEAM_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kSmemBytes),
                    "cudaFuncSetAttribute(smem)");
      resident = kCta == 2 ? resident_pairs(kernel, S::kThreads, S::kSmemBytes, ctx->sm_count) : ctx->sm_count;
      configured_clusters[ctx->device] = resident;
    }
  }
  GemmParams p = {};
  int st = encode_tmap_2d(&p.tm_a, A, 2, static_cast<uint64_t>(m), static_cast<uint64_t>(k),
                          static_cast<uint64_t>(k), S::kBM, S::kBK, true);
  if (st != BEAM_OK) return st;
  st = encode_tmap_2d(&p.tm_b, B, 2, static_cast<uint64_t>(n), static_cast<uint64_t>(k), static_cast<uint64_t>(k),
                      S::kBRows, S::kBK, true);
  if (st != BEAM_OK) return st;
  st = encode_tmap_2d(&p.tm_c, C, 2, static_cast<uint64_t>(m), static_cast<uint64_t>(n),
                      static_cast<uint64_t>(ex.ldc > 0 ? ex.ldc : n), 32, 64, true);
  if (st != BEAM_OK) return st;
  for (int d = 0; d < ex.n_peers; ++d) {
    st = encode_tmap_2d(&p.tm_peer[d], ex.peer_c[d], 2, static_cast<uint64_t>(m), static_cast<uint64_t>(n),
                        static_cast<uint64_t>(n), 32, 64, true);
    if (st != BEAM_OK) return st;
  }
  p.n_peers = ex.n_peers;
  p.bf16 = ex.bf16;
  p.c = static_cast<__half*>(C);
  p.m = m;
  p.n = n;
  p.k = k;
  p.ldc = n;
  p.m_tiles = (m + 2 * S::kBM * kCta - 1) / (2 * S::kBM * kCta);  // double tiles: two vertically adjacent tiles each
  p.n_tiles = (n + S::kBN - 1) / S::kBN;
  p.group_m = group_m > 0 ? group_m : (kCta == 2 ? 4 : 8);
  p.slices = 1;
  p.hint_a = (ex.l2_hints / 10) % 10;
  p.hint_b = ex.l2_hints % 10;
  p.hint_c = (ex.l2_hints / 100) % 10;
  p.status = ctx->status_word;
  const long long items = static_cast<long long>(p.m_tiles) * p.n_tiles;
  int clusters = resident;
  if (max_ctas > 0 && max_ctas / kCta < clusters) clusters = max_ctas / kCta > 0 ? max_ctas / kCta : 1;
  if (items < clusters) clusters = static_cast<int>(items);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(clusters * kCta), 1, 1);
  cfg.blockDim = dim3(S::kThreads, 1, 1);
  cfg.dynamicSmemBytes = S::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kCta;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  BEAM_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, p), "cudaLaunchKernelEx(gemmrc_dual)");
  return BEAM_OK;
}

// The one-kernel split-K (splitk_stream.cuh): one CTA per (tile, slice), launched cooperatively and as a programmatic
// dependent of whatever precedes it on the stream.  Returns BEAM_ERR_UNSUPPORTED when the grid does not fit at once.
template <int BN, int kStages, bool kFold>
int launch_stream_instance(DeviceCtx* ctx, const void* A, const void* B, void* C, int m, int n, int k,
                           const ExtraArgs& ex, cudaStream_t stream) {
  using S = StreamShape<BN, kStages>;
  auto kernel = splitk_stream_kernel<BN, kStages, kFold>;
  static int configured[64] = {0};
  static std::mutex configure_mutex;
  int max_ctas = 0;
  {
    std::lock_guard<std::mutex> lock(configure_mutex);
    if (configured[ctx->device] == 0) {
      if (S::kSmemBytes > ctx->max_smem_optin) return BEAM_ERR_UNSUPPORTED;
      BEAM_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kSmemBytes),
                    "cudaFuncSetAttribute(smem)");
      int per_sm = 0;
      BEAM_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, S::kThreads, S::kSmemBytes),
                    "cudaOccupancyMaxActiveBlocksPerMultiprocessor");
      configured[ctx->device] = per_sm > 0 ? per_sm * ctx->sm_count : -1;
    }
    max_ctas = configured[ctx->device];
  }
  GemmParams p = {};
  int st = encode_tmap_2d(&p.tm_a, A, 2, static_cast<uint64_t>(m), static_cast<uint64_t>(k), static_cast<uint64_t>(k),
                          kFold ? S::kBM / 2 : S::kBM, S::kBK, true);
  if (st != BEAM_OK) return st;
  st = encode_tmap_2d(&p.tm_b, B, 2, static_cast<uint64_t>(n), static_cast<uint64_t>(k), static_cast<uint64_t>(k),
                      kFold ? BN / 2 : BN, S::kBK, true);
  if (st != BEAM_OK) return st;
  const int planes = ex.slices * (kFold ? 2 : 1);
  st = encode_tmap_3d_f32(&p.tm_s, ex.scratch, static_cast<uint64_t>(planes), static_cast<uint64_t>(m),
                          static_cast<uint64_t>(n), 32, 32);
  if (st != BEAM_OK) return st;
  p.c = static_cast<__half*>(C);
  p.scratch = ex.scratch;
  p.m = m;
  p.n = n;
  p.k = k;
  p.ldc = n;
  p.m_tiles = (m + S::kBM - 1) / S::kBM;
  p.n_tiles = (n + BN - 1) / BN;
  p.group_m = 1;
  p.slices = ex.slices;
  p.flags = ex.flags;
  p.fold = kFold ? 1 : 0;
  p.status = ctx->status_word;
  const long long items = static_cast<long long>(p.m_tiles) * p.n_tiles * p.slices;
  // one wave that leaves the other half of every SM to the call before or after it
  if (items > ctx->sm_count || items > max_ctas) return BEAM_ERR_UNSUPPORTED;
  // Read-back view: every plane's share of one CTA in one copy.  The box holds all planes (at most 256) and as many
  // 32-byte granules as a CTA's share needs, the landing area holds and the group sums have room for.
  if (planes > 256) return BEAM_ERR_UNSUPPORTED;
  const long long granules = (static_cast<long long>(m) * n) >> 3;
  long long box_g = (granules + items - 1) / items;
  const long long fit = (S::kRingBytes - S::kSumsBytes) / 32 / planes;
  if (box_g > fit) box_g = fit;
  if (box_g > S::kMaxBoxGranules) box_g = S::kMaxBoxGranules;
  if (box_g < 1) return BEAM_ERR_UNSUPPORTED;
  st = encode_tmap_granules_f32(&p.tm_peer[0], ex.scratch, static_cast<uint64_t>(planes),
                                static_cast<uint64_t>(granules), static_cast<uint32_t>(planes),
                                static_cast<uint32_t>(box_g));
  if (st != BEAM_OK) return st;
  p.rb_granules = static_cast<int>(box_g);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(items), 1, 1);
  cfg.blockDim = dim3(S::kThreads, 1, 1);
  cfg.dynamicSmemBytes = S::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (!ctx->coop_without_pdl) {
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 2;
  }
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, p);
  if (e != cudaSuccess && cfg.numAttrs == 2 &&
      (e == cudaErrorNotSupported || e == cudaErrorInvalidValue || e == cudaErrorInvalidConfiguration)) {
    // This driver does not take a cooperative grid as a programmatic dependent: launch it as an ordinary
    // stream-ordered kernel from now on (griddepcontrol.wait then returns at once).
    (void)cudaGetLastError();
    ctx->coop_without_pdl = true;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, kernel, p);
  }
  if (e == cudaErrorCooperativeLaunchTooLarge) {
    (void)cudaGetLastError();
    return BEAM_ERR_UNSUPPORTED;
  }
  BEAM_CUDA_TRY(e, "cudaLaunchKernelEx(splitk_stream)");
  return BEAM_OK;
}

}  // namespace

int default_stages(int bn, int cta) {
  if (cta == 2) return bn == 256 ? 6 : 8;
  return bn == 256 ? 4 : (bn == 128 ? 6 : 8);
}

int validate_gemm_args(const void* A, const void* B, const void* C, int m, int n, int k) {
  if (!A || !B || !C) return BEAM_ERR_INVALID_ARG;
  if (m <= 0 || n <= 0 || k <= 0) return BEAM_ERR_INVALID_ARG;
  if (!aligned16(A) || !aligned16(B) || !aligned16(C)) return BEAM_ERR_ALIGNMENT;
  if ((k % 8) != 0 || (n % 8) != 0) return BEAM_ERR_ALIGNMENT;
  return BEAM_OK;
}

// ------------------------------------------------------------------------------- large GEMM
#define BEAM_GEMM_CASE(BN_, ST_, CTA_)                                                \
  if (plan.tile_n == BN_ && stages == ST_ && plan.cta_pair == CTA_)                   \
    return launch_instance<BN_, ST_, CTA_, kModeGemm>(ctx, A, B, C, m, n, k, plan.group_m, plan.max_ctas, ex, \
                                                      stream);

static int launch_gemmrc_ex(const void* A, const void* B, void* C, int m, int n, int k, const GemmPlan& plan,
                            ExtraArgs ex, cudaStream_t stream) {
  int st = validate_gemm_args(A, B, C, m, n, k);
  if (st != BEAM_OK) return st;
  DeviceCtx* ctx = current_device_ctx(&st);
  if (!ctx) return st;
  const int stages = plan.stages > 0 ? plan.stages : default_stages(plan.tile_n, plan.cta_pair);
  ex.l2_hints = plan.l2_hints;
  ex.bf16 = plan.bf16;
  ex.whole_tiles = plan.whole_tiles;
  if (plan.ldc != 0) {
    if (plan.ldc < n || (plan.ldc % 8) != 0) return BEAM_ERR_INVALID_ARG;  // rows of C must stay 16-byte aligned
    ex.ldc = plan.ldc;
  }
  if (plan.tile_n == 512 || plan.tile_m == 512) {
    // two-accumulator tiles: 256 x 512 (tile_n = 512) or 512 x 256 (tile_m = 512, tile_n = 256)
    if (plan.cta_pair != 2) return BEAM_ERR_UNSUPPORTED;
    const bool tall = plan.tile_m == 512;
    if (tall && plan.tile_n != 256) return BEAM_ERR_UNSUPPORTED;
    // Default: the 3-deep ring, which leaves room for two C staging buffers per epilogue warp.
    if (plan.stages == 0 || plan.stages == 3)
      return tall ? launch_wide_instance<3, true>(ctx, A, B, C, m, n, k, plan.group_m, plan.max_ctas, ex, stream)
                  : launch_wide_instance<3, false>(ctx, A, B, C, m, n, k, plan.group_m, plan.max_ctas, ex, stream);
    if (plan.stages == 4)
      return tall ? launch_wide_instance<4, true>(ctx, A, B, C, m, n, k, plan.group_m, plan.max_ctas, ex, stream)
                  : launch_wide_instance<4, false>(ctx, A, B, C, m, n, k, plan.group_m, plan.max_ctas, ex, stream);
    return BEAM_ERR_UNSUPPORTED;
  }
  if (plan.tile_n == 128 && plan.stages == 0 && plan.tiles_in_flight != 1) {
    // 128-wide tiles: two tiles in flight per CTA (pair), each with its own accumulator and issuing thread
    if (plan.cta_pair == 2)
      return launch_dual_instance<4, 2>(ctx, A, B, C, m, n, k, plan.group_m, plan.max_ctas, ex, stream);
    return launch_dual_instance<4, 1>(ctx, A, B, C, m, n, k, plan.group_m, plan.max_ctas, ex, stream);
  }
  BEAM_GEMM_CASE(256, 4, 2)
  BEAM_GEMM_CASE(256, 5, 2)
  BEAM_GEMM_CASE(256, 6, 2)
  BEAM_GEMM_CASE(128, 4, 2)
  BEAM_GEMM_CASE(128, 6, 2)
  BEAM_GEMM_CASE(128, 8, 2)
  BEAM_GEMM_CASE(256, 3, 1)
  BEAM_GEMM_CASE(256, 4, 1)
  BEAM_GEMM_CASE(128, 4, 1)
  BEAM_GEMM_CASE(128, 6, 1)
  BEAM_GEMM_CASE(64, 4, 1)
  BEAM_GEMM_CASE(64, 8, 1)
  return BEAM_ERR_UNSUPPORTED;
}
#undef BEAM_GEMM_CASE

int launch_gemmrc(const void* A, const void* B, void* C, int m, int n, int k, const GemmPlan& plan,
                  cudaStream_t stream) {
  return launch_gemmrc_ex(A, B, C, m, n, k, plan, ExtraArgs(), stream);
}

// Every destination (this GPU included) receives the rank's block at rows [rank * m, (rank + 1) * m) of its
// gathered buffer.  The tensor maps start at that block and span m rows, so the copy engine clips a tile that
// overhangs the block instead of spilling into the next rank's rows.
int launch_gemmrc_allgather(const void* A, const void* B, void* const* gathered, int world, int rank, int m, int n,
                            int k, const GemmPlan& plan, cudaStream_t stream) {
  if (!gathered || world < 1 || world > 8 || rank < 0 || rank >= world) return BEAM_ERR_INVALID_ARG;
  if (m <= 0 || n <= 0 || k <= 0) return BEAM_ERR_INVALID_ARG;
  const size_t block_bytes = static_cast<size_t>(m) * static_cast<size_t>(n) * 2;
  ExtraArgs ex;
  void* local = nullptr;
  for (int i = 0; i < world; ++i) {
    const int d = (rank + i) % world;  // self first, then the peers starting with the next rank
    if (!gathered[d]) return BEAM_ERR_INVALID_ARG;
    char* block = static_cast<char*>(gathered[d]) + static_cast<size_t>(rank) * block_bytes;
    if (!aligned16(block)) return BEAM_ERR_ALIGNMENT;
    if (i == 0)
      local = block;
    else
      ex.peer_c[ex.n_peers++] = block;
  }
  return launch_gemmrc_ex(A, B, local, m, n, k, plan, ex, stream);
}

// ------------------------------------------------------------------- GEMM with a co-scheduled SiLU
int launch_gemm_silu(const void* A, const void* B, void* C, int m, int n, int k, const void* x, void* y,
                     long long count, cudaStream_t stream) {
  int st = validate_gemm_args(A, B, C, m, n, k);
  if (st != BEAM_OK) return st;
  if (count < 0 || (count > 0 && (!x || !y))) return BEAM_ERR_INVALID_ARG;
  if (count > 0 && (!aligned16(x) || !aligned16(y))) return BEAM_ERR_ALIGNMENT;
  DeviceCtx* ctx = current_device_ctx(&st);
  if (!ctx) return st;
  ExtraArgs ex;
  ex.ew_in = static_cast<const __half*>(x);
  ex.ew_out = static_cast<__half*>(y);
  ex.ew_count = count;
  const long long pair_tiles = static_cast<long long>((m + 255) / 256) * ((n + 255) / 256);
  if (pair_tiles >= ctx->sm_count / 2)
    return launch_instance<256, 6, 2, kModeGemmSilu>(ctx, A, B, C, m, n, k, 0, 0, ex, stream);
  return launch_instance<128, 6, 1, kModeGemmSilu>(ctx, A, B, C, m, n, k, 0, 0, ex, stream);
}

// ---------------------------------------------------------------------------------- split-K
int splitk_tile_n(int n, int tile_n) {
  if (tile_n == 64 || tile_n == 128 || tile_n == 256) return tile_n;
  return n <= 64 ? 64 : 128;
}

// Split-K serves two kinds of problem.  Small M and N (the reference's 128 x 256 x 65536 and 64 x 64 x 131072) stream A
// and B once and are bound by HBM.  Medium M and N (512 x 512 x 8192, python/gemm_test.py:201 of the reference;
// 1024 x 1024 x 8192) have too few output tiles for the SMs but more arithmetic than memory time: with every SM at work
// 2 M N K flop take longer than 2 K (M + N) bytes once M N / (M + N) exceeds about 200 (B200: ~1500 TFLOP/s against
// ~6.5 TB/s).  Those want the 256-wide tile (UMMAs of N = 256 keep the tensor pipe busy from one issuing thread,
// N = 128 ones do not) and as many slices as fill the SMs.
bool splitk_compute_bound(int m, int n) {
  return static_cast<double>(m) * n >= 200.0 * (static_cast<double>(m) + n);
}

int splitk_pick_tile(int m, int n, int tile_n) {
  if (tile_n == 64 || tile_n == 128 || tile_n == 256) return tile_n;
  if (n >= 256 && splitk_compute_bound(m, n)) return 256;
  return splitk_tile_n(n, 0);
}

// Plain calls (each call waits for the one before it), measured on B200 with chains of dependent calls over
// HBM-cold inputs: two thirds of the SMs get a work item (128 x 256 x 65536: 16.1 us with 96 CTAs against 17.3 to
// 18.8 with 128 to 148; fewer CTAs drain sooner and the memory system is saturated either way); folded problems
// (M, N <= 64), which run as one kernel, do best with seven eighths (64 x 64 x 131072: 13.1 us with 128 slices
// against 14.3 with 74).  Never fewer than 4 k-blocks (256 of K) per slice, so that the fill of the TMA ring is
// amortised.  (The reference's model, cutlass_gemmrc_splitk.cu:44-57, targets the 108 SMs of an A100 and rounds
// to half waves.)
// Calls that carry BEAM_FLAG_INPUTS_STABLE overlap with their neighbours on the stream, so the grid is sized by
// bytes instead: about 650 KB of operand traffic per CTA (820 KB when the problem runs folded), which leaves room
// for two or three consecutive calls to stream side by side (measured optimum on B200 for 128x256x65536 and
// 64x64x131072).
int splitk_heuristic(int m, int n, int k, int tile_n, int flags) {
  const int bn = splitk_pick_tile(m, n, tile_n);
  const long long m_tiles = (m + 127) / 128, n_tiles = (n + bn - 1) / bn;
  const long long tiles = m_tiles * n_tiles;
  const int num_kb = (k + 63) / 64;
  int sms = 148;
  int err = 0;
  int dev = -1;
  if (cudaGetDevice(&dev) == cudaSuccess) {
    if (DeviceCtx* ctx = current_device_ctx(&err)) sms = ctx->sm_count;
  } else {
    (void)cudaGetLastError();
  }
  const bool folds = splitk_folds(m, n, tile_n);
  long long s = (folds ? sms * 7 / 8 : sms * 2 / 3) / (tiles > 0 ? tiles : 1);
  if (folds && s > 128) s = 128;  // a folded slice leaves two planes, and the one-kernel form reads back at most 256
  if (flags & BEAM_FLAG_INPUTS_STABLE) {
    s = sms / (tiles > 0 ? tiles : 1);
    if (folds) s = (s + 1) / 2;  // a folded slice leaves two planes: half as many slices reduce as fast
    // every N tile re-reads its rows of A, every M tile its rows of B (from L2 after the first reader)
    const double bytes = 2.0 * k * (static_cast<double>(m) * n_tiles + static_cast<double>(n) * m_tiles);
    const double per_cta = splitk_folds(m, n, tile_n) ? 820.0 * 1024.0 : 650.0 * 1024.0;  // folded rings hold more of K
    const long long by_bytes = static_cast<long long>(bytes / per_cta / static_cast<double>(tiles) + 0.5);
    if (by_bytes < s) s = by_bytes;
  }
  long long cap = num_kb / 4 > 0 ? num_kb / 4 : 1;
  if (!folds && splitk_compute_bound(m, n)) {
    // every SM a work item; slices of at least 8 k-blocks, so that a slice's arithmetic outweighs its partial plane
    s = sms / (tiles > 0 ? tiles : 1);
    cap = num_kb / 8 > 0 ? num_kb / 8 : 1;
  }
  if (s > cap) s = cap;
  if (s > 256) s = 256;
  if (s < 1) s = 1;
  return static_cast<int>(s);
}

// Problems with M, N <= 64 run "folded" (two k-blocks per UMMA, see gemmrc_umma.cuh) unless the caller insists
// on a 128- or 256-wide tile: K is then dealt out in steps of 128, and every slice leaves two partial planes.
bool splitk_folds(int m, int n, int tile_n) { return m <= 64 && n <= 64 && (tile_n == 0 || tile_n == 64); }

int splitk_resolve_slices(int m, int n, int k, int tile_n, int requested, int flags) {
  const int num_kb = (k + 63) / 64;
  const int steps = splitk_folds(m, n, tile_n) ? (num_kb + 1) / 2 : num_kb;
  if (requested > 0 && requested <= num_kb && requested <= 1024) return requested <= steps ? requested : steps;
  const int h = splitk_heuristic(m, n, k, tile_n, flags);
  return h <= steps ? h : steps;
}

size_t splitk_workspace_bytes(int m, int n, int k, int tile_n, int slices) {
  if (m <= 0 || n <= 0 || k <= 0) return 0;
  // sized for whichever of the two heuristics (plain calls, calls that may overlap) picks more slices
  const int s_plain = splitk_resolve_slices(m, n, k, tile_n, slices, 0);
  const int s_over = splitk_resolve_slices(m, n, k, tile_n, slices, BEAM_FLAG_INPUTS_STABLE);
  const int s = s_plain > s_over ? s_plain : s_over;
  const size_t planes = static_cast<size_t>(s) * (splitk_folds(m, n, tile_n) ? 2 : 1);
  return planes * static_cast<size_t>(m) * static_cast<size_t>(n) * sizeof(float);
}

// The one-kernel form needs every (tile, slice) resident at once (one CTA per SM) and a device that launches
// cooperative grids; BEAM_FLAG_SPLITK_TWO_KERNELS asks for the two-kernel form regardless.
static bool splitk_one_kernel(const DeviceCtx* ctx, int m, int n, int bn, int slices, int flags, bool fold) {
  if (flags & BEAM_FLAG_SPLITK_TWO_KERNELS) return false;
  if (!ctx->cooperative_launch) return false;
  if (bn > 128) return false;  // a 256-wide tile does not leave half of the SM free (see splitk_stream.cuh)
  // Where both forms apply the faster one was chosen by measurement (B200, chains of 24 calls, HBM-cold inputs): one
  // kernel for folded problems called plainly (13.1 against 15.0 us at 64 x 64 x 131072); two kernels otherwise
  // (16.1 against 18.4 us at 128 x 256 x 65536; calls that overlap their neighbours: 7.7 against 8.3 us folded, 11.9
  // against 12.4 us not).  Both forms pay about 8 us between the last UMMA and the next call's first load, a chain
  // of device-wide round trips of about a microsecond each (stores visible, barrier or kernel boundary, read back).
  if (!(flags & BEAM_FLAG_SPLITK_ONE_KERNEL) && (!fold || (flags & BEAM_FLAG_INPUTS_STABLE))) return false;
  if (slices * (fold ? 2 : 1) > 256) return false;  // the read-back copy holds at most 256 planes
  const long long items = static_cast<long long>((m + 127) / 128) * ((n + bn - 1) / bn) * slices;
  return items <= ctx->sm_count;
}

int splitk_describe(int m, int n, int k, int tile_n, int slices, int flags, int* info) {
  int st = BEAM_OK;
  DeviceCtx* ctx = current_device_ctx(&st);
  if (!ctx) return st;
  if (m <= 0 || n <= 0 || k <= 0 || slices < 0 || !info) return BEAM_ERR_INVALID_ARG;
  const bool fold = splitk_folds(m, n, tile_n);
  const int bn = fold ? 128 : splitk_pick_tile(m, n, tile_n);
  const int s = splitk_resolve_slices(m, n, k, tile_n, slices, flags);
  const bool one = splitk_one_kernel(ctx, m, n, bn, s, flags, fold);
  info[0] = bn;
  info[1] = s;
  info[2] = fold ? 1 : 0;
  info[3] = one ? 1 : 2;                                 // kernels per call
  info[4] = (one && ctx->coop_without_pdl) ? 0 : 1;      // first kernel is a programmatic dependent launch
  return BEAM_OK;
}

int launch_splitk(const void* A, const void* B, void* C, int m, int n, int k, int tile_n, int slices,
                  void* workspace, size_t workspace_bytes, cudaStream_t stream, int flags) {
  int st = validate_gemm_args(A, B, C, m, n, k);
  if (st != BEAM_OK) return st;
  if (slices < 0) return BEAM_ERR_INVALID_ARG;
  if (m > 65535) return BEAM_ERR_UNSUPPORTED;  // the reduction grid has one block row per output row
  DeviceCtx* ctx = current_device_ctx(&st);
  if (!ctx) return st;
  const bool fold = splitk_folds(m, n, tile_n);
  const int bn = fold ? 128 : splitk_pick_tile(m, n, tile_n);
  const int s = splitk_resolve_slices(m, n, k, tile_n, slices, flags);
  const int planes = fold ? 2 * s : s;
  const size_t need = static_cast<size_t>(planes) * m * n * sizeof(float);
  if (!workspace || workspace_bytes < need) return BEAM_ERR_WORKSPACE;
  if (!aligned16(workspace)) return BEAM_ERR_ALIGNMENT;

  ExtraArgs ex;
  ex.scratch = static_cast<float*>(workspace);
  ex.slices = s;
  ex.flags = flags & BEAM_FLAG_INPUTS_STABLE;
  ex.fold = fold ? 1 : 0;
  if (splitk_one_kernel(ctx, m, n, bn, s, flags, fold)) {
    // One kernel: partials, a grid-wide barrier, then every CTA sums its share of the output (same order as the
    // reduction kernel below, so the two paths agree bit for bit).
    if (bn == 64)
      st = launch_stream_instance<64, 4, false>(ctx, A, B, C, m, n, k, ex, stream);
    else
      st = fold ? launch_stream_instance<128, 3, true>(ctx, A, B, C, m, n, k, ex, stream)
                : launch_stream_instance<128, 3, false>(ctx, A, B, C, m, n, k, ex, stream);
    if (st != BEAM_ERR_UNSUPPORTED) return st;
    ctx->cooperative_launch = false;  // the grid does not fit at once on this device: two kernels from now on
  }
  if (bn == 64)
    st = launch_instance<64, 8, 1, kModeSplitK>(ctx, A, B, C, m, n, k, 1, 0, ex, stream);
  else if (bn == 128)
    st = launch_instance<128, 6, 1, kModeSplitK>(ctx, A, B, C, m, n, k, 1, 0, ex, stream);
  else
    st = launch_instance<256, 4, 1, kModeSplitK>(ctx, A, B, C, m, n, k, 1, 0, ex, stream);
  if (st != BEAM_OK) return st;

  // Fixed-order reduction, launched so that its blocks may become resident while the partial
  // kernel drains; it blocks in griddepcontrol.wait until every partial is written and visible.
  // Small outputs: a block per row x 128 columns, the eight groups of planes summed by eight warps side by side (the
  // shortest chain of dependent loads).  From 64 Ki outputs on: one thread per four columns (one wave of blocks).
  const bool flat = static_cast<long long>(m) * n >= 65536;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = flat ? dim3(static_cast<unsigned>((static_cast<long long>(m) * (n / 4) + 255) / 256), 1, 1)
                     : dim3(static_cast<unsigned>((n + 127) / 128), static_cast<unsigned>(m), 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  BEAM_CUDA_TRY(cudaLaunchKernelEx(&cfg, flat ? splitk_reduce_flat_kernel : splitk_reduce_kernel,
                                   static_cast<const float*>(workspace), static_cast<__half*>(C), m, n, planes),
                "cudaLaunchKernelEx(splitk_reduce)");
  return BEAM_OK;
}

// ------------------------------------------------------------------------ GEMM + LayerNorm
// Workspace layout: [fp32 panel M x N][(mean, M2) per row per 256-wide N tile][ticket per 128 rows]
// [queue: 16 control ints + one int per 128-row panel].  Tickets and queue are zeroed before each launch.
namespace {
constexpr int kLnTileN = 256;
struct LnLayout {
  size_t panel_bytes, part_off, part_bytes, ticket_off, ticket_bytes, queue_off, total;  // ticket_bytes covers the queue too
};
// `resident`: the TMEM-resident kernel runs (it needs no panel; its tickets, one int per 32 rows, take the panel's place).
LnLayout ln_layout(int m, int n, bool resident) {
  LnLayout l;
  const size_t n_tiles = static_cast<size_t>((n + kLnTileN - 1) / kLnTileN);
  const size_t panels = 2 * static_cast<size_t>((m + 255) / 256);  // both CTAs of every 256-row pair tile
  l.panel_bytes = resident ? ((static_cast<size_t>((m + 31) / 32) + 8) * sizeof(int) + 255) / 256 * 256
                           : (static_cast<size_t>(m) * n * sizeof(float) + 255) / 256 * 256;
  l.part_off = l.panel_bytes;
  l.part_bytes = (static_cast<size_t>(m) * n_tiles * sizeof(float2) + 255) / 256 * 256;
  l.ticket_off = l.part_off + l.part_bytes;
  l.ticket_bytes = (panels * sizeof(int) + 255) / 256 * 256 + ((16 + panels) * sizeof(int) + 255) / 256 * 256;
  l.queue_off = l.ticket_off + (panels * sizeof(int) + 255) / 256 * 256;
  l.total = l.ticket_off + l.ticket_bytes;
  return l;
}
constexpr int kLnResidentStages = 6;
// CTA pairs of the TMEM-resident kernel that the device holds at once, asked of the occupancy calculator once per
// device (which also opts the kernel in to its shared memory); 0 if the kernel cannot run there.
int ln_resident_pairs(DeviceCtx* ctx) {
  using S = LnResidentShape<kLnResidentStages>;
  static int cached[64] = {0};
  static std::mutex mutex;
  std::lock_guard<std::mutex> lock(mutex);
  int& pairs = cached[ctx->device];
  if (pairs == 0) {
    pairs = -1;
    if (S::kSmemBytes <= ctx->max_smem_optin &&
        cudaFuncSetAttribute(gemm_ln_resident_kernel<kLnResidentStages>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             S::kSmemBytes) == cudaSuccess)
      pairs = resident_pairs(gemm_ln_resident_kernel<kLnResidentStages>, S::kThreads, S::kSmemBytes, ctx->sm_count);
    (void)cudaGetLastError();
  }
  return pairs > 0 ? pairs : 0;
}
// CTA pairs of the current device (74 when there is none to ask: sizes can be queried without a GPU).
int ln_pairs() {
  int dev = -1, err = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) {
    if (DeviceCtx* ctx = current_device_ctx(&err)) return ln_resident_pairs(ctx);
  } else {
    (void)cudaGetLastError();
  }
  return 74;
}
bool ln_resident(int n) { return (n + kLnTileN - 1) / kLnTileN <= ln_pairs(); }
}  // namespace

// The TMEM-resident form (gemm_ln_resident.cuh): no parked panel, only statistics and tickets in the workspace.
template <int kStages>
int launch_ln_resident(DeviceCtx* ctx, const void* X, const void* W, void* out, const void* gamma, const void* beta,
                       float eps, int m, int n, int k, float2* row_part, int* tickets, size_t ticket_bytes,
                       cudaStream_t stream) {
  using S = LnResidentShape<kStages>;
  auto kernel = gemm_ln_resident_kernel<kStages>;
  const int pairs = ln_resident_pairs(ctx);  // also opts the kernel in to its shared memory, once per device
  if (pairs <= 0) return BEAM_ERR_UNSUPPORTED;
  GemmParams p = {};
  int st = encode_tmap_2d(&p.tm_a, X, 2, static_cast<uint64_t>(m), static_cast<uint64_t>(k),
                          static_cast<uint64_t>(k), S::kBM, S::kBK, true);
  if (st != BEAM_OK) return st;
  st = encode_tmap_2d(&p.tm_b, W, 2, static_cast<uint64_t>(n), static_cast<uint64_t>(k), static_cast<uint64_t>(k),
                      S::kBRows, S::kBK, true);
  if (st != BEAM_OK) return st;
  st = encode_tmap_2d(&p.tm_c, out, 2, static_cast<uint64_t>(m), static_cast<uint64_t>(n), static_cast<uint64_t>(n),
                      32, 64, true);
  if (st != BEAM_OK) return st;
  p.c = static_cast<__half*>(out);
  p.row_part = row_part;
  p.tickets = tickets;
  p.gamma = static_cast<const __half*>(gamma);
  p.beta = static_cast<const __half*>(beta);
  p.eps = eps;
  p.m = m;
  p.n = n;
  p.k = k;
  p.ldc = n;
  p.m_tiles = (m + 255) / 256;
  p.n_tiles = (n + S::kBN - 1) / S::kBN;
  p.status = ctx->status_word;
  BEAM_CUDA_TRY(cudaMemsetAsync(tickets, 0, ticket_bytes, stream), "cudaMemsetAsync(tickets)");
  const long long tiles = static_cast<long long>(p.m_tiles) * p.n_tiles;
  int clusters = pairs;
  if (tiles < clusters) clusters = static_cast<int>(tiles);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(clusters * 2), 1, 1);
  cfg.blockDim = dim3(S::kThreads, 1, 1);
  cfg.dynamicSmemBytes = S::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // CTAs of this grid wait for one another: a cooperative launch places the whole grid or none of it, so two such
  // grids launched on different streams cannot each hold half of the SMs and wait for the other half.
  attr[1].id = cudaLaunchAttributeCooperative;
  attr[1].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  BEAM_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, p), "cudaLaunchKernelEx(gemm_ln_resident)");
  return BEAM_OK;
}

size_t layernorm_workspace_bytes(int m, int n, int k) {
  (void)k;
  if (m <= 0 || n <= 0) return 0;
  return ln_layout(m, n, ln_resident(n)).total;
}

int launch_gemm_layernorm(const void* X, const void* W, void* out, const void* gamma, const void* beta, float eps,
                          int m, int n, int k, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  int st = validate_gemm_args(X, W, out, m, n, k);
  if (st != BEAM_OK) return st;
  if (!gamma || !beta || !(eps >= 0.f)) return BEAM_ERR_INVALID_ARG;
  if (!aligned16(gamma) || !aligned16(beta)) return BEAM_ERR_ALIGNMENT;
  const bool resident = ln_resident(n);
  const LnLayout l = ln_layout(m, n, resident);
  if (!workspace || workspace_bytes < l.total) return BEAM_ERR_WORKSPACE;
  if (!aligned16(workspace)) return BEAM_ERR_ALIGNMENT;
  DeviceCtx* ctx = current_device_ctx(&st);
  if (!ctx) return st;
  char* ws = static_cast<char*>(workspace);
  ExtraArgs ex;
  ex.scratch = reinterpret_cast<float*>(ws);
  ex.row_part = reinterpret_cast<float2*>(ws + l.part_off);
  ex.tickets = reinterpret_cast<int*>(ws + l.ticket_off);
  ex.ln_queue = reinterpret_cast<int*>(ws + l.queue_off);
  ex.gamma = static_cast<const __half*>(gamma);
  ex.beta = static_cast<const __half*>(beta);
  ex.eps = eps;
  const int n_tiles = (n + kLnTileN - 1) / kLnTileN;
  const int pairs = ctx->sm_count / 2;
  {
    // With at least as many resident CTA pairs as N tiles, the tiles can wait in TMEM for their rows' statistics
    // and nothing is parked: tickets (one int per 32 rows) go where the panel would have been.
    const size_t ticket_bytes = (static_cast<size_t>((m + 31) / 32) + 8) * sizeof(int);
    if (resident && ticket_bytes <= l.panel_bytes)
      return launch_ln_resident<kLnResidentStages>(ctx, X, W, out, gamma, beta, eps, m, n, k, ex.row_part,
                                   reinterpret_cast<int*>(ws), ticket_bytes, stream);
  }
  // More N tiles than CTA pairs (N > 256 * pairs): the pre-normalisation values are parked as an fp32 panel.
  // Operand loads carry the explicit normal policy here: with the second pass's scratch traffic sharing L2,
  // that kernel measured 3 % slower when its operand reads were left eligible for request coalescing.
  ex.l2_hints = 33;
  BEAM_CUDA_TRY(cudaMemsetAsync(ex.tickets, 0, l.ticket_bytes, stream), "cudaMemsetAsync(tickets)");
  // Rasterisation: one wave of resident CTAs should cover whole rows of tiles, so that a panel's N tiles are
  // computed close together in time and its parked values are still in L2 when they are normalised.
  const int group_m = (pairs + n_tiles - 1) / n_tiles;
  return launch_instance<kLnTileN, 5, 2, kModeLayerNorm>(ctx, X, W, out, m, n, k, group_m, 0, ex, stream);
}

}  // namespace beam
