// extern "C" surface of libbeam_b200: argument checking, registry-name presets, status plumbing.
// Nothing here touches torch; pointers and sizes only.
#include <cstring>

#include "gemmrc_launch.h"
#include "host_entry.h"
#include "layernorm_launch.h"
#include "splitk_launch.h"

using namespace beam;

extern "C" {

const char* beam_status_string(int status) {
  switch (status) {
    case BEAM_OK: return "ok";
    case BEAM_ERR_INVALID_ARG: return "invalid argument (null pointer, non-positive size or bad value)";
    case BEAM_ERR_UNSUPPORTED: return "unsupported shape, tile or split factor";
    case BEAM_ERR_ALIGNMENT: return "alignment: pointers must be 16-byte aligned, K and N multiples of 8";
    case BEAM_ERR_WORKSPACE: return "workspace missing or too small";
    case BEAM_ERR_CUDA: return "CUDA runtime call failed";
    case BEAM_ERR_TENSORMAP: return "TMA descriptor rejected by the driver";
    case BEAM_ERR_DEVICE_TIMEOUT: return "a kernel's bounded wait ran out";
    case BEAM_ERR_NO_DEVICE: return "no sm_100 CUDA device is current";
    default: return "unknown status";
  }
}

const char* beam_last_cuda_error(void) { return last_cuda_error_text(); }

const char* beam_version(void) { return "beam_b200 sm_100a (TMA + tcgen05)"; }

int beam_device_status(int clear, int* fault_word_out) {
  int st = BEAM_OK;
  DeviceCtx* ctx = current_device_ctx(&st);
  if (!ctx) return st;
  int word = 0;
  BEAM_CUDA_TRY(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  BEAM_CUDA_TRY(cudaMemcpy(&word, ctx->status_word, sizeof(int), cudaMemcpyDeviceToHost), "read fault word");
  if (fault_word_out) *fault_word_out = word;
  if (clear && word != 0) BEAM_CUDA_TRY(cudaMemset(ctx->status_word, 0, sizeof(int)), "clear fault word");
  return word == 0 ? BEAM_OK : BEAM_ERR_DEVICE_TIMEOUT;
}

int beam_gemmrc_fp16(const void* A, const void* B, void* C, int m, int n, int k, const beam_gemm_cfg* cfg,
                     void* stream) {
  GemmPlan plan;
  if (cfg) {
    if (cfg->tile_n) plan.tile_n = cfg->tile_n;
    if (cfg->cta_pair) plan.cta_pair = cfg->cta_pair;
    plan.stages = cfg->stages;
    plan.group_m = cfg->group_m;
    plan.max_ctas = cfg->max_ctas;
    plan.l2_hints = cfg->l2_hints;
    plan.bf16 = (cfg->flags & BEAM_FLAG_BF16) ? 1 : 0;
    plan.whole_tiles = (cfg->flags & BEAM_FLAG_WHOLE_TILES) ? 1 : 0;
    plan.tile_m = cfg->tile_m;
    plan.tiles_in_flight = cfg->tiles_in_flight;
    if (plan.tiles_in_flight < 0 || plan.tiles_in_flight > 2) return BEAM_ERR_INVALID_ARG;
    if (plan.tile_m != 0 && plan.tile_m != 512) return BEAM_ERR_INVALID_ARG;
    if (cfg->flags & ~(BEAM_FLAG_BF16 | BEAM_FLAG_WHOLE_TILES)) return BEAM_ERR_INVALID_ARG;
    if (plan.cta_pair != 1 && plan.cta_pair != 2) return BEAM_ERR_INVALID_ARG;
    if (plan.stages < 0 || plan.group_m < 0 || plan.max_ctas < -1 || plan.l2_hints < 0 || plan.l2_hints > 333)
      return BEAM_ERR_INVALID_ARG;
  }
  return launch_gemmrc(A, B, C, m, n, k, plan, static_cast<cudaStream_t>(stream));
}

int beam_gemmrc_fp16_allgather(const void* A_local, const void* B, void* const* C_gathered, int world, int rank,
                               int m_local, int n, int k, const beam_gemm_cfg* cfg, void* stream) {
  GemmPlan plan;
  if (cfg) {
    if (cfg->tile_n) plan.tile_n = cfg->tile_n;
    if (cfg->cta_pair) plan.cta_pair = cfg->cta_pair;
    plan.stages = cfg->stages;
    plan.group_m = cfg->group_m;
    if (plan.cta_pair != 1 && plan.cta_pair != 2) return BEAM_ERR_INVALID_ARG;
    if (plan.stages < 0 || plan.group_m < 0) return BEAM_ERR_INVALID_ARG;
  }
  // Default: 256 x 256 tiles on CTA pairs, also where the plain GEMM would take 256 x 512.  The NVLink store stream,
  // not the tensor pipe, sets the pace of this kernel, and smaller tiles feed it more evenly (8 GPUs, 8192 rows per
  // rank: 1.61 ms against 1.68 ms with 256 x 512 tiles; the stores alone take 1.41 ms).
  return launch_gemmrc_allgather(A_local, B, C_gathered, world, rank, m_local, n, k, plan,
                                 static_cast<cudaStream_t>(stream));
}

int beam_custom_gemmrc_128x128(const void* A, const void* B, void* C, int m, int n, int k, void* stream) {
  GemmPlan plan;
  plan.tile_n = 128;
  plan.cta_pair = 1;
  return launch_gemmrc(A, B, C, m, n, k, plan, static_cast<cudaStream_t>(stream));
}

int beam_custom_gemmrc_128x256(const void* A, const void* B, void* C, int m, int n, int k, void* stream) {
  GemmPlan plan;
  plan.tile_n = 256;
  plan.cta_pair = 1;
  return launch_gemmrc(A, B, C, m, n, k, plan, static_cast<cudaStream_t>(stream));
}

int beam_cutlass_gemmrc(const void* A, const void* B, void* C, int m, int n, int k, void* stream) {
  GemmPlan plan;  // 256 x 256 on a CTA pair ...
  // ... or 256 x 512 (both TMEM accumulators live) once there are enough tiles to keep every pair busy for
  // several waves: fewer operand bytes per flop through L2 and shared memory, worth ~7 % at 8192^3.
  const long long wide_tiles = static_cast<long long>((m + 255) / 256) * ((n + 511) / 512);
  if (m > 0 && n > 0 && wide_tiles >= 4 * 74) plan.tile_n = 512;
  return launch_gemmrc(A, B, C, m, n, k, plan, static_cast<cudaStream_t>(stream));
}

int beam_cutlass_gemmrc_spec(const void* A, const void* B, void* C, int m, int n, int k, int tb_m, int tb_n,
                             int warp_m, int warp_n, void* stream) {
  (void)warp_m;
  (void)warp_n;
  GemmPlan plan;
  if (tb_m == 128)
    plan.cta_pair = 1;
  else if (tb_m == 256)
    plan.cta_pair = 2;
  else if (tb_m == 512 && tb_n == 256) {  // two 256-row accumulators per CTA pair
    plan.cta_pair = 2;
    plan.tile_m = 512;
  } else
    return BEAM_ERR_UNSUPPORTED;
  if (tb_n != 128 && tb_n != 256 && !(tb_n == 512 && tb_m == 256)) return BEAM_ERR_UNSUPPORTED;
  plan.tile_n = tb_n;
  return launch_gemmrc(A, B, C, m, n, k, plan, static_cast<cudaStream_t>(stream));
}

size_t beam_gemmrc_splitk_workspace_bytes(int m, int n, int k, int tile_n, int split_k_slices) {
  return splitk_workspace_bytes(m, n, k, tile_n, split_k_slices);
}

int beam_gemmrc_splitk_heuristic(int m, int n, int k, int tile_n) { return splitk_heuristic(m, n, k, tile_n); }

int beam_gemmrc_splitk_describe(int m, int n, int k, int tile_n, int split_k_slices, int flags, int* info) {
  return splitk_describe(m, n, k, tile_n, split_k_slices, flags, info);
}

int beam_gemmrc_splitk_fp16(const void* A, const void* B, void* C, int m, int n, int k, const beam_gemm_cfg* cfg,
                            void* workspace, size_t workspace_bytes, void* stream) {
  int tile_n = 0, slices = 0, flags = 0;
  if (cfg) {
    tile_n = cfg->tile_n;
    slices = cfg->split_k_slices;
    flags = cfg->flags;
    if (tile_n != 0 && tile_n != 64 && tile_n != 128 && tile_n != 256) return BEAM_ERR_UNSUPPORTED;
    if (flags & ~(BEAM_FLAG_INPUTS_STABLE | BEAM_FLAG_SPLITK_TWO_KERNELS | BEAM_FLAG_SPLITK_ONE_KERNEL))
      return BEAM_ERR_INVALID_ARG;
    if ((flags & BEAM_FLAG_SPLITK_TWO_KERNELS) && (flags & BEAM_FLAG_SPLITK_ONE_KERNEL)) return BEAM_ERR_INVALID_ARG;
  }
  return launch_splitk(A, B, C, m, n, k, tile_n, slices, workspace, workspace_bytes,
                       static_cast<cudaStream_t>(stream), flags);
}

int beam_cutlass_gemmrc_splitk(const void* A, const void* B, void* C, int m, int n, int k, int split_k_slices,
                               void* workspace, size_t workspace_bytes, void* stream) {
  return launch_splitk(A, B, C, m, n, k, 0, split_k_slices, workspace, workspace_bytes,
                       static_cast<cudaStream_t>(stream));
}

int beam_cutlass_gemmrc_splitk_spec(const void* A, const void* B, void* C, int m, int n, int k, int tb_m,
                                    int tb_n, int warp_m, int warp_n, int split_k_slices, void* workspace,
                                    size_t workspace_bytes, void* stream) {
  (void)tb_m;
  (void)warp_m;
  (void)warp_n;
  if (tb_n != 64 && tb_n != 128 && tb_n != 256) return BEAM_ERR_UNSUPPORTED;
  return launch_splitk(A, B, C, m, n, k, tb_n, split_k_slices, workspace, workspace_bytes,
                       static_cast<cudaStream_t>(stream));
}

size_t beam_gemmrc_layernorm_workspace_bytes(int m, int n, int k) { return layernorm_workspace_bytes(m, n, k); }

int beam_gemmrc_layernorm(const void* X, const void* W, void* out, const void* gamma, const void* beta, float eps,
                          int m, int n, int k, void* workspace, size_t workspace_bytes, void* stream) {
  return launch_gemm_layernorm(X, W, out, gamma, beta, eps, m, n, k, workspace, workspace_bytes,
                               static_cast<cudaStream_t>(stream));
}

int beam_gemmrc_silu(const void* A, const void* B, void* C, int m, int n, int k, const void* x, void* y,
                     long long count, void* stream) {
  return launch_gemm_silu(A, B, C, m, n, k, x, y, count, static_cast<cudaStream_t>(stream));
}

int beam_gemmrc_fp16_host(const void* A_host, const void* B_host, void* C_host, int m, int n, int k) {
  return gemmrc_from_host(A_host, B_host, C_host, m, n, k);
}

int beam_gemmrc_fp16_host_rows(const void* A_host, const void* B_dev, void* C_host, int m, int n, int k) {
  return gemmrc_rows_from_host(A_host, B_dev, C_host, m, n, k);
}

}  // extern "C"
