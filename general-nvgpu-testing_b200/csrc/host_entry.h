// Host-buffer entries: H2D copies, GEMMs and D2H copies pipelined over row blocks of A and B.
#pragma once

namespace beam {

// A, B, C in host memory.
int gemmrc_from_host(const void* A_host, const void* B_host, void* C_host, int m, int n, int k);
// A, C in host memory, B already on the device (a rank of a row-sharded job, which uploads B once or receives it
// from its peers over NVLink).
int gemmrc_rows_from_host(const void* A_host, const void* B_dev, void* C_host, int m, int n, int k);

}  // namespace beam
