// Host-buffer entry: H2D copies, GEMM and D2H copy pipelined over row blocks of A.
#pragma once

namespace beam {

int gemmrc_from_host(const void* A_host, const void* B_host, void* C_host, int m, int n, int k);

}  // namespace beam
