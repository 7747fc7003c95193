// Per-device context and TMA descriptor encoding for the beam_b200 library.
#include "host_common.h"

#include <cstdio>
#include <cstring>
#include <mutex>

namespace beam {

namespace {

constexpr int kMaxDevices = 64;
DeviceCtx g_ctx[kMaxDevices];
std::mutex g_ctx_mutex;

thread_local char t_cuda_error[256] = "";

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is looked up through the runtime so the library carries no link-time
// dependency on libcuda (it must load, and export its symbols, on a machine without a GPU).
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess) return nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// A descriptor is a pure function of (base, extents, pitch, box, type, swizzle), and callers come back with the
// same tensors call after call, so each host thread keeps the last few it encoded: a hit costs a short compare
// instead of a driver call.  (Base pointers are unique across devices under unified addressing.)
struct TmapKey {
  const void* base;
  uint64_t d0, d1, d2, pitch;
  uint32_t box0, box1, kind;
};
struct TmapSlot {
  TmapKey key;
  CUtensorMap map;
  bool used;
};
constexpr int kTmapSlots = 32;
thread_local TmapSlot t_tmaps[kTmapSlots];
thread_local unsigned t_tmap_next = 0;

bool tmap_lookup(const TmapKey& key, CUtensorMap* out) {
  for (int i = 0; i < kTmapSlots; ++i) {
    const TmapSlot& s = t_tmaps[i];
    if (s.used && s.key.base == key.base && s.key.d0 == key.d0 && s.key.d1 == key.d1 && s.key.d2 == key.d2 &&
        s.key.pitch == key.pitch && s.key.box0 == key.box0 && s.key.box1 == key.box1 && s.key.kind == key.kind) {
      std::memcpy(out, &s.map, sizeof(CUtensorMap));
      return true;
    }
  }
  return false;
}
void tmap_remember(const TmapKey& key, const CUtensorMap* map) {
  TmapSlot& s = t_tmaps[t_tmap_next++ % kTmapSlots];
  s.key = key;
  std::memcpy(&s.map, map, sizeof(CUtensorMap));
  s.used = true;
}

}  // namespace

void note_cuda_error(cudaError_t e, const char* where) {
  std::snprintf(t_cuda_error, sizeof(t_cuda_error), "%s: %s", where, cudaGetErrorString(e));
}
const char* last_cuda_error_text() { return t_cuda_error; }

DeviceCtx* current_device_ctx(int* err) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    if (e != cudaSuccess) note_cuda_error(e, "cudaGetDevice");
    (void)cudaGetLastError();
    *err = BEAM_ERR_NO_DEVICE;
    return nullptr;
  }
  DeviceCtx* c = &g_ctx[dev];
  if (c->ok.load(std::memory_order_acquire)) return c;
  std::lock_guard<std::mutex> lock(g_ctx_mutex);
  if (c->ok.load(std::memory_order_acquire)) return c;
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, dev);
  if (e != cudaSuccess) {
    note_cuda_error(e, "cudaGetDeviceProperties");
    (void)cudaGetLastError();
    *err = BEAM_ERR_NO_DEVICE;
    return nullptr;
  }
  if (prop.major != 10) {  // the kernels are built for sm_100a only
    std::snprintf(t_cuda_error, sizeof(t_cuda_error), "device %d is sm_%d%d, need sm_100", dev, prop.major,
                  prop.minor);
    *err = BEAM_ERR_NO_DEVICE;
    return nullptr;
  }
  c->device = dev;
  c->sm_count = prop.multiProcessorCount;
  c->max_smem_optin = static_cast<int>(prop.sharedMemPerBlockOptin);
  c->cc_major = prop.major;
  c->cc_minor = prop.minor;
  c->cooperative_launch = prop.cooperativeLaunch != 0;
  e = cudaMalloc(&c->status_word, 256);
  if (e == cudaSuccess) e = cudaMemset(c->status_word, 0, 256);
  if (e != cudaSuccess) {
    note_cuda_error(e, "status word");
    (void)cudaGetLastError();
    *err = BEAM_ERR_CUDA;
    return nullptr;
  }
  c->ok.store(true, std::memory_order_release);
  return c;
}

int encode_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint64_t ld,
                   uint32_t box_rows, uint32_t box_cols, bool swizzle128) {
  const TmapKey key = {base, cols, rows, 0, ld, box_cols, box_rows,
                       static_cast<uint32_t>(elem_bytes) | (swizzle128 ? 0x100u : 0u)};
  if (tmap_lookup(key, out)) return BEAM_OK;
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return BEAM_ERR_TENSORMAP;
  const cuuint64_t gdim[2] = {cols, rows};
  const cuuint64_t gstride[1] = {ld * static_cast<uint64_t>(elem_bytes)};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t estride[2] = {1, 1};
  const CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    std::snprintf(t_cuda_error, sizeof(t_cuda_error), "cuTensorMapEncodeTiled failed with CUresult %d",
                  static_cast<int>(r));
    return BEAM_ERR_TENSORMAP;
  }
  tmap_remember(key, out);
  return BEAM_OK;
}

// 3-D row-major fp32 tensor [planes][rows][cols] (dense), box = 1 x box_rows x box_cols, 128-byte swizzle.
int encode_tmap_3d_f32(CUtensorMap* out, const void* base, uint64_t planes, uint64_t rows, uint64_t cols,
                       uint32_t box_rows, uint32_t box_cols) {
  const TmapKey key = {base, cols, rows, planes, 0, box_cols, box_rows, 0x1000u};
  if (tmap_lookup(key, out)) return BEAM_OK;
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return BEAM_ERR_TENSORMAP;
  const cuuint64_t gdim[3] = {cols, rows, planes};
  const cuuint64_t gstride[2] = {cols * 4, rows * cols * 4};
  const cuuint32_t box[3] = {box_cols, box_rows, 1};
  const cuuint32_t estride[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), gdim, gstride, box, estride,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    std::snprintf(t_cuda_error, sizeof(t_cuda_error), "cuTensorMapEncodeTiled (3-D) failed with CUresult %d",
                  static_cast<int>(r));
    return BEAM_ERR_TENSORMAP;
  }
  tmap_remember(key, out);
  return BEAM_OK;
}

int encode_tmap_granules_f32(CUtensorMap* out, const void* base, uint64_t planes, uint64_t granules,
                             uint32_t box_planes, uint32_t box_granules) {
  const TmapKey key = {base, granules, planes, 0, 0, box_granules, box_planes, 0x2000u};
  if (tmap_lookup(key, out)) return BEAM_OK;
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return BEAM_ERR_TENSORMAP;
  const cuuint64_t gdim[3] = {8, granules, planes};
  const cuuint64_t gstride[2] = {32, granules * 32};
  const cuuint32_t box[3] = {8, box_granules, box_planes};
  const cuuint32_t estride[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), gdim, gstride, box, estride,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    std::snprintf(t_cuda_error, sizeof(t_cuda_error), "cuTensorMapEncodeTiled (granules) failed with CUresult %d",
                  static_cast<int>(r));
    return BEAM_ERR_TENSORMAP;
  }
  tmap_remember(key, out);
  return BEAM_OK;
}

}  // namespace beam
