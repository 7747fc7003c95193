// Launcher interface of the persistent UMMA kernels (implementation: gemmrc_launch.cu).
#pragma once

#include "host_common.h"

namespace beam {

struct GemmPlan {
  int tile_n = 256;   // UMMA N
  int tile_m = 0;     // 0 = 128 rows per CTA; 512 = two 256-row accumulators per CTA pair (with tile_n = 256)
  int cta_pair = 2;   // 1 or 2 CTAs per tile
  int stages = 0;     // 0 = deepest ring that fits
  int group_m = 0;    // 0 = default rasterisation group
  int max_ctas = 0;   // 0 = whole device
  int bf16 = 0;       // operands and result are bf16 instead of fp16
  int l2_hints = 0;   // decimal digits: tens = A loads, ones = B loads; 0 normal, 1 evict-first, 2 evict-last
  int ldc = 0;        // row pitch of C in elements (0 = n; a multiple of 8, at least n): C may be a block of columns
  int whole_tiles = 0;  // 256 x 256 on pairs: 1 = do not cut the last wave's tiles into 128-column halves
  int tiles_in_flight = 0;  // tile_n = 128 only: 0 or 2 = two tiles in flight per CTA (pair), 1 = one tile at a time
};

int default_stages(int tile_n, int cta_pair);
int validate_gemm_args(const void* A, const void* B, const void* C, int m, int n, int k);
int launch_gemmrc(const void* A, const void* B, void* C, int m, int n, int k, const GemmPlan& plan,
                  cudaStream_t stream);
// GEMM plus an independent y = silu(x) over `count` halves worked in by the epilogue warps.
int launch_gemm_silu(const void* A, const void* B, void* C, int m, int n, int k, const void* x, void* y,
                     long long count, cudaStream_t stream);
// Fused GEMM + all-gather: C of this rank's m rows goes to row block `rank` of every gathered[d] (d < world).
int launch_gemmrc_allgather(const void* A, const void* B, void* const* gathered, int world, int rank, int m, int n,
                            int k, const GemmPlan& plan, cudaStream_t stream);

}  // namespace beam
