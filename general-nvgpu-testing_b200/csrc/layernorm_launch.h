// Fused GEMM + LayerNorm: one persistent kernel, row panels owned by a CTA pair.
#pragma once

#include "host_common.h"

namespace beam {

size_t layernorm_workspace_bytes(int m, int n, int k);
int launch_gemm_layernorm(const void* X, const void* W, void* out, const void* gamma, const void* beta, float eps,
                          int m, int n, int k, void* workspace, size_t workspace_bytes, cudaStream_t stream);

}  // namespace beam
