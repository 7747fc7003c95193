// Host-side plumbing shared by the launchers: the per-device context (SM count, fault word;
// its one allocation happens at first use of a device), CUDA error bookkeeping, and the TMA
// tensor-map encoder fetched from the driver at run time.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <atomic>
#include <cstddef>
#include <cstdint>

#include "../../include/beam_b200.h"

namespace beam {

struct DeviceCtx {
  int device = -1;
  int sm_count = 0;
  int max_smem_optin = 0;
  int cc_major = 0, cc_minor = 0;
  int* status_word = nullptr;  // device memory, one int, zero while healthy
  std::atomic<bool> cooperative_launch{false}; // the device places cooperative grids of one CTA per SM
  std::atomic<bool> coop_without_pdl{false};   // set once a cooperative grid was refused as a programmatic dependent
  std::atomic<bool> ok{false};                 // published last (release); readers acquire
};

// Returns the context of the CUDA device that is current on the calling thread, creating it
// on first use (cudaMalloc of the 4-byte status word happens there, never on a later call).
// On failure returns nullptr and stores a BEAM_ERR_* code in *err.
DeviceCtx* current_device_ctx(int* err);

// 2-D row-major fp16/fp32 tensor map: `rows` x `cols` elements, row pitch `ld` elements,
// box = box_rows x box_cols, 128-byte swizzle when swizzle128 is set (box_cols * elem = 128 B).
int encode_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint64_t ld,
                   uint32_t box_rows, uint32_t box_cols, bool swizzle128);

// Dense 3-D fp32 tensor [planes][rows][cols], box 1 x box_rows x box_cols (box_cols * 4 = 128 B), 128-byte swizzle.
int encode_tmap_3d_f32(CUtensorMap* out, const void* base, uint64_t planes, uint64_t rows, uint64_t cols,
                       uint32_t box_rows, uint32_t box_cols);

// The same dense fp32 tensor [planes][rows * cols] seen as [planes][granules][8 floats] (32-byte granules, no
// swizzle), box = box_planes x box_granules x 8: the read-back view of the one-kernel split-K.
int encode_tmap_granules_f32(CUtensorMap* out, const void* base, uint64_t planes, uint64_t granules,
                             uint32_t box_planes, uint32_t box_granules);

// Records a CUDA runtime failure for beam_last_cuda_error() (thread-local text).
void note_cuda_error(cudaError_t e, const char* where);
const char* last_cuda_error_text();

#define BEAM_CUDA_TRY(expr, where)            \
  do {                                        \
    cudaError_t _e = (expr);                  \
    if (_e != cudaSuccess) {                  \
      ::beam::note_cuda_error(_e, where);     \
      (void)cudaGetLastError();               \
      return BEAM_ERR_CUDA;                   \
    }                                         \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace beam
