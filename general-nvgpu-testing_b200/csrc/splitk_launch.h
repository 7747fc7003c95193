// Split-K rc GEMM: K-sliced UMMA kernel writing fp32 partials + fixed-order reduction kernel.
#pragma once

#include "host_common.h"

namespace beam {

// tile_n = 0 picks the tile from N; slices = 0 picks the split factor from the SM count.
int splitk_tile_n(int n, int tile_n);
// ... and from M and N: the 256-wide tile for problems with more arithmetic than memory time (see gemmrc_launch.cu).
int splitk_pick_tile(int m, int n, int tile_n);
bool splitk_folds(int m, int n, int tile_n);
int splitk_heuristic(int m, int n, int k, int tile_n, int flags = 0);
int splitk_resolve_slices(int m, int n, int k, int tile_n, int requested, int flags = 0);
size_t splitk_workspace_bytes(int m, int n, int k, int tile_n, int slices);
// info[0..4] = tile N, slices, folded (0/1), kernels per call (1 or 2), first kernel launched as a programmatic
// dependent (0/1) for this problem on the current device.
int splitk_describe(int m, int n, int k, int tile_n, int slices, int flags, int* info);
int launch_splitk(const void* A, const void* B, void* C, int m, int n, int k, int tile_n, int slices,
                  void* workspace, size_t workspace_bytes, cudaStream_t stream, int flags = 0);

}  // namespace beam
