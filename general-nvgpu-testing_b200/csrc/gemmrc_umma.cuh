// Persistent, warp-specialised fp16 rc GEMM for sm_100a:  C[M,N] = A[M,K] * B[N,K]^T.
//
// One CTA (kCta = 1) or a cta_group::2 pair of CTAs on neighbouring SMs (kCta = 2) owns an
// output tile of (128 * kCta) x BN.  Both operands are K-major, so TMA drops 128-byte-swizzled
// [rows x 64 halves] boxes straight into the layout the UMMA shared-memory descriptor reads.
//
//   warp 0      TMA producer   one lane: waits empty[s], arms full[s], issues the A and B box loads
//   warp 1      MMA issuer     one lane of the leader CTA: waits full[s], 4 x tcgen05.mma (K = 16 each)
//                              per 64-wide k-block into a TMEM accumulator, commits empty[s]; after
//                              the last k-block commits tmem_full[acc].  Also owns TMEM alloc/dealloc.
//   warps 2..5  epilogue       wait tmem_full[acc], tcgen05.ld 32 lanes x 32 columns at a time, lay each
//                              row's 128 bytes into a swizzled staging buffer, TMA-store the 32-row box
//                              (the copy engine clips rows >= M and columns >= N), then release the
//                              accumulator through tmem_empty[acc].
//
// TMEM holds two accumulators (2 x BN fp32 columns) so the epilogue of work item i overlaps the
// main loop of item i+1.  In pair mode each CTA loads its own 128 rows of A and its own BN/2 rows
// of B (plain per-CTA TMA loads that signal the leader's mbarrier), the leader's UMMA reads both
// CTAs' shared memory and writes both CTAs' TMEM, and completion is fanned out to both CTAs with
// the two-CTA form of tcgen05.commit.
//
// GEMM mode with 256 x 256 tiles on pairs runs two more warps (6: a second MMA issuer, 7: a second producer), idle
// except in a pair's last item when the launcher has cut the tiles of the last wave into halves (see kTail below).
// All GEMM-mode launches are programmatic dependents of the kernel before them on the stream: set-up overlaps that
// kernel's tail, the producer waits for its completion before the first load.
//
// Four epilogues share this pipeline:
//   kModeGemm       fp32 -> fp16, store C.
//   kModeSplitK     a work item is (tile, K slice); the fp32 partial goes to workspace[slice][M][N]
//                   and a second kernel sums the slices in index order.
//                   (Calls whose work items fit on the device at once run as one kernel instead: splitk_stream.cuh.)
//   kModeGemmSilu   the GEMM epilogue, plus an unrelated element-wise y = x / (1 + exp(-x)) over a second tensor
//                   that the epilogue warps work through, 1024 elements at a time, while they wait for their
//                   next accumulator (what the reference's cute_gemm_ln.cu co-schedules on a quarter of its CTAs).
//   kModeLayerNorm  tiles are walked in GEMM order (so A and B stay L2-resident).  Each tile's epilogue
//                   parks its fp32 values in a scratch panel, writes one (mean, M2) pair per row for
//                   its N range, and takes a ticket for its 128-row panel.  The CTA that draws the last
//                   ticket of a panel publishes the panel on a device-wide queue; after every tile each
//                   CTA claims a few 8-row chunks of published panels and normalises them (statistics
//                   merged in tile order, panel re-read from L2, gamma/beta applied, fp16 stored), so the
//                   second pass is spread over all SMs and hidden under the main loops.
#pragma once

#include "umma_common.cuh"

namespace beam {

enum GemmMode : int { kModeGemm = 0, kModeSplitK = 1, kModeLayerNorm = 2, kModeGemmSilu = 3 };
__host__ __device__ constexpr bool is_splitk_mode(int mode) { return mode == kModeSplitK; }

struct GemmParams {
  CUtensorMap tm_a;  // A  [M, K], box 128 x 64, 128 B swizzle
  CUtensorMap tm_b;  // B  [N, K], box (BN / kCta) x 64, 128 B swizzle
  CUtensorMap tm_b_tail;  // the same with half as many rows per box, for the half-width tiles of the last wave
  CUtensorMap tm_c;  // C  [M, N] fp16, store box 32 rows x 64 columns, 128 B swizzle
  CUtensorMap tm_s;  // scratch [slices][M][N] fp32, store box 1 x 32 rows x 32 columns, 128 B swizzle
  CUtensorMap tm_peer[7];  // fused all-gather: this rank's row block inside each peer GPU's gathered C
                           // (one-kernel split-K: [0] is the read-back view of the scratch, see splitk_stream.cuh)
  int n_peers;             // 0 = plain GEMM; else every C box is also stored to that many peers
  __half* c;         // fp16 output [M, ldc]
  float* scratch;    // split-K: partials [slices][M][N]; LayerNorm: fp32 panel store [M][N]
  float2* row_part;  // LayerNorm: (mean, M2) of every row over each N tile, [M][n_tiles]
  int* tickets;      // LayerNorm: arrival counter per 128-row panel, zero at launch
  int* ln_queue;     // LayerNorm: [0] panels published, [1] chunks claimed, [16 + i] i-th published panel + 1
  const __half* gamma;
  const __half* beta;
  float eps;
  int m, n, k;
  int ldc;
  int m_tiles;  // tiles of 128 * kCta rows
  int n_tiles;  // tiles of BN columns
  int group_m;  // M-tiles per rasterisation group (GEMM mode)
  int slices;   // split-K slices (1 otherwise)
  int hint_a;   // L2 eviction policy of the A loads: 0 normal, 1 evict-first, 2 evict-last
  int hint_b;   // same for the B loads
  int hint_c;   // same for the C stores (GEMM mode)
  int flags;    // BEAM_FLAG_* bits of the call
  const __half* ew_in;   // kModeGemmSilu: element-wise input, ew_count halves
  __half* ew_out;        // kModeGemmSilu: element-wise output
  long long ew_count;
  int bf16;     // GEMM mode: A, B, C are bf16 instead of fp16 (same kernels: descriptor bits and final rounding)
  int fold;     // split-K of a problem with M, N <= 64: two k-blocks share one 128 x 128 UMMA (see the producer)
  int lead_in;  // two-accumulator tiles: k-blocks issued half-major at the start of a tile (at least 1)
  int lead_out; // ... and at its end
  int tail_tiles;   // GEMM on CTA pairs, BN = 256: this many tiles at the end of the walk are cut into two 128-column halves
  int rb_granules;  // one-kernel split-K: 32-byte granules of every plane per read-back copy (box of tm_peer[0])
  int* status;  // device fault word
};

template <int BN, int kStages, int kCta, int kMode = kModeGemm>
struct GemmShape {
  static constexpr int kBM = 128;
  static constexpr int kBK = 64;
  static constexpr int kBRows = BN / kCta;
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = kBRows * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = 2 * BN;  // 128, 256 or 512: a power of two >= 32
  static constexpr int kBarBytes = 512;
  static constexpr int kStoreBufBytes = 32 * 128;  // one warp's box: 32 rows x 128 bytes
  // Staging buffers per epilogue warp: two for the output stores; LayerNorm keeps four, which also serve
  // as the landing ring of its second pass.
  static constexpr int kBufsPerWarp = (kMode == kModeLayerNorm) ? 4 : 2;
  static constexpr int kStagingBytes = 4 * kBufsPerWarp * kStoreBufBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + kBarBytes + 1024;  // + alignment slack
  // GEMM with 256 x 256 tiles on pairs has a seventh warp: the second UMMA-issuing thread of a cut tile.
  // (Even ring depths only: each issuing thread of a cut item takes every other k-block, and with an even depth it
  // meets a given stage once per pass of the ring, which is what a parity wait can tell apart.)
  static constexpr bool kCutTiles = kMode == kModeGemm && BN == 256 && kCta == 2 && kStages % 2 == 0;
  static constexpr int kThreads = kCutTiles ? 256 : 192;
  static_assert(kSmemBytes <= 232448, "exceeds the 227 KB of shared memory a CTA can opt in to");
  static_assert(BN == 64 || BN == 128 || BN == 256, "UMMA N of the tile");
  static_assert(kCta == 1 || kCta == 2, "one CTA or a pair");
  // mbarriers: full/empty per stage, 2 + 2 for TMEM, 16 for the LayerNorm landing ring; then 8 ints.
  static_assert((2 * kStages + 4 + 16) * 8 + 32 <= kBarBytes, "barrier block too small");
};

struct WorkItem {
  int mt, nt;        // tile coordinates
  int half;          // -1: the whole tile; 0 / 1: its left / right half (the cut tiles of the last wave)
  int kb0, kb1;      // k-block range [kb0, kb1)
  int slice;         // split-K slice index
};

// The j-th work item of the CTA (pair) whose first item index is `first` with `stride` CTAs (pairs)
// in the grid.  Returns false past the end.  All three roles call this with the same arguments and
// therefore walk identical sequences.
//   GEMM, LayerNorm: items are tiles; groups of `group_m` M-tiles are walked N-major so that tiles
//              in flight together share A rows and B rows in L2 (the reference's CTA remap at
//              cute_gemm_128x128.cu:23-33, restated for a persistent grid).
//              With kTail, the last p.tail_tiles tiles of that order are two items each, one per half: when the
//              tiles do not fill the last wave of a persistent grid by half, halves fill it twice as well and
//              the wave takes about half as long.
//   split-K:   items are (tile, slice), slice fastest; k-blocks are dealt out as evenly as possible.
// How one CTA (pair) walks the work: item j is `first + j * stride`.
struct Walk {
  int first, stride;
};

template <int kMode, bool kTail = false>
__device__ __forceinline__ bool work_item(const GemmParams& p, const Walk& walk, int j, int num_kb, WorkItem& w) {
  const int first = walk.first, stride = walk.stride;
  w.slice = 0;
  w.half = -1;
  w.kb0 = 0;
  w.kb1 = num_kb;
  if constexpr (!is_splitk_mode(kMode)) {
    int t = first + j * stride;
    if constexpr (kTail) {
      const int whole = p.m_tiles * p.n_tiles - p.tail_tiles;  // tiles before the cut ones
      if (t >= whole) {
        w.half = (t - whole) & 1;
        t = whole + ((t - whole) >> 1);
      }
    }
    if (t >= p.m_tiles * p.n_tiles) return false;
    const int per_group = p.group_m * p.n_tiles;
    const int g = t / per_group;
    const int first_m = g * p.group_m;
    const int rows = min(p.group_m, p.m_tiles - first_m);
    const int r = t - g * per_group;
    w.mt = first_m + r % rows;
    w.nt = r / rows;
    return true;
  } else {
    const int t = first + j * stride;
    if (t >= p.m_tiles * p.n_tiles * p.slices) return false;
    w.slice = t % p.slices;
    const int tile = t / p.slices;
    w.nt = tile % p.n_tiles;
    w.mt = tile / p.n_tiles;
    w.kb0 = static_cast<int>(static_cast<long long>(num_kb) * w.slice / p.slices);
    w.kb1 = static_cast<int>(static_cast<long long>(num_kb) * (w.slice + 1) / p.slices);
    return true;
  }
}

// Stores one staged 32 x 64 fp16 box of C: to this GPU's C and, in the fused all-gather, to the same place in
// every peer's gathered buffer (plain per-destination TMA stores over NVLink; one bulk group for all of them).
__device__ __forceinline__ void store_c_box(const GemmParams& p, uint32_t buf, int x, int y) {
  ptx::tma_store_2d_hint(&p.tm_c, buf, x, y, ptx::l2_policy(p.hint_c));
  for (int d = 0; d < p.n_peers; ++d) ptx::tma_store_2d(&p.tm_peer[d], buf, x, y);
  ptx::tma_store_commit();
}

// One warp applies y = x / (1 + exp(-x)) (fp32 math, fp16 in and out; cute_gemm_ln.cu:181-198 of the reference) to
// chunk `chunk` of 1024 elements: four coalesced 16-byte loads per lane in flight, then four stores.
__device__ __forceinline__ void silu_chunk(const GemmParams& p, long long chunk, uint32_t lane) {
  const long long base = chunk * 1024;
  uint4 v[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long e = base + (static_cast<long long>(i) * 32 + lane) * 8;
    v[i] = make_uint4(0, 0, 0, 0);
    if (e + 8 <= p.ew_count) v[i] = *reinterpret_cast<const uint4*>(p.ew_in + e);  // plain load: x may alias y
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long e = base + (static_cast<long long>(i) * 32 + lane) * 8;
    if (e + 8 <= p.ew_count) {
      __half2* h = reinterpret_cast<__half2*>(&v[i]);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 x = __half22float2(h[q]);
        h[q] = __floats2half2_rn(x.x / (1.f + __expf(-x.x)), x.y / (1.f + __expf(-x.y)));
      }
      *reinterpret_cast<uint4*>(p.ew_out + e) = v[i];
    } else if (e < p.ew_count) {  // the ragged last few elements, one at a time
      for (long long t = e; t < p.ew_count; ++t) {
        const float x = __half2float(p.ew_in[t]);
        p.ew_out[t] = __float2half_rn(x / (1.f + __expf(-x)));
      }
    }
  }
}

// Chan's parallel update of (count, mean, M2) with a block of `nb` values whose own mean and M2 are given.
__device__ __forceinline__ void welford_merge(float& n, float& mean, float& m2, float nb, float mean_b, float m2_b) {
  const float nn = n + nb;
  const float delta = mean_b - mean;
  const float f = nb / nn;
  mean += delta * f;
  m2 += m2_b + delta * delta * n * f;
  n = nn;
}

// ------------------------------------------------------------------ LayerNorm second pass
// Work unit of the second pass: 32 rows x 512 columns of a published panel, normalised by one warp.
constexpr int kLnUnitCols = 512;
constexpr int kLnQueueItems = 16;  // int offset of the published-panel list inside the queue block

__device__ __forceinline__ int ld_volatile_i32(const int* ptr) {
  return *reinterpret_cast<const volatile int*>(ptr);
}
__device__ __forceinline__ int ln_units_per_panel(int n) { return 4 * ((n + kLnUnitCols - 1) / kLnUnitCols); }

// One warp normalises unit `u` of the panel published in queue slot `slot`: lane = row.  Each lane merges its
// row's per-tile (mean, M2) in tile order, then the parked fp32 values come back through TMA as 32 x 32 boxes
// into the warp's four staging buffers (a four-deep ring, so three boxes are in flight while one is being
// consumed); every lane reads its row's 128 bytes, applies (x - mean) * rstd * gamma + beta and stores 64 bytes
// of fp16.  ring_count counts the boxes this warp has ever landed (selects buffer and mbarrier parity).
template <int BN>
__device__ __forceinline__ void ln_normalise_unit(const GemmParams& p, int panel, int u, uint32_t lane,
                                                  uint32_t buf_base, uint32_t bar_base, uint32_t& ring_count,
                                                  volatile int* cta_abort) {
  const int col_units = (p.n + kLnUnitCols - 1) / kLnUnitCols;
  const int row_base = panel * 128 + (u / col_units) * 32;
  const int col_base = (u % col_units) * kLnUnitCols;
  if (row_base >= p.m) return;
  const int boxes = (min(p.n, col_base + kLnUnitCols) - col_base + 31) / 32;
  auto issue = [&](int i) {  // lane 0 only
    const uint32_t k = ring_count + static_cast<uint32_t>(i);
    const uint32_t bar = bar_base + 8u * (k & 3u);
    ptx::mbar_arrive_expect_tx(bar, 4096);
    ptx::tma_load_3d(buf_base + (k & 3u) * 4096u, &p.tm_s, bar, col_base + i * 32, row_base, 0);
  };
  if (lane == 0) {
    for (int i = 0; i < min(4, boxes); ++i) issue(i);
  }
  // Statistics of this lane's row while the first boxes fly.
  const int row = row_base + static_cast<int>(lane);
  float mean = 0.f, rstd = 0.f;
  if (row < p.m) {
    float n_acc = 0.f, m2 = 0.f;
    const float2* parts = p.row_part + static_cast<size_t>(row) * p.n_tiles;
    for (int t0 = 0; t0 < p.n_tiles; t0 += 8) {
      float2 pt[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) pt[i] = (t0 + i < p.n_tiles) ? __ldcg(parts + t0 + i) : make_float2(0.f, 0.f);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (t0 + i < p.n_tiles)
          welford_merge(n_acc, mean, m2, static_cast<float>(min(BN, p.n - (t0 + i) * BN)), pt[i].x, pt[i].y);
    }
    rstd = rsqrtf(m2 / n_acc + p.eps);
  }
  __half* orow = p.c + static_cast<size_t>(row) * p.ldc;
  for (int i = 0; i < boxes; ++i) {
    const uint32_t k = ring_count + static_cast<uint32_t>(i);
    const uint32_t buf = buf_base + (k & 3u) * 4096u;
    if (!bounded_wait_warp(bar_base + 8u * (k & 3u), (k >> 2) & 1u, cta_abort, p.status, kFaultReduceWait, lane))
      break;
    uint4 x[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = ptx::ld_shared_v4(buf + lane * 128u + ((static_cast<uint32_t>(j) ^ (lane & 7u)) << 4));
    // The buffer may be refilled once every lane has read it; the fence orders these generic reads before
    // the copy engine's writes.
    ptx::fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0 && i + 4 < boxes) issue(i + 4);
    const int col = col_base + i * 32;
    if (row < p.m) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {  // 8 columns per step
        if (col + 8 * j < p.n) {
          const uint4 g = __ldg(reinterpret_cast<const uint4*>(p.gamma + col + 8 * j));
          const uint4 b = __ldg(reinterpret_cast<const uint4*>(p.beta + col + 8 * j));
          const __half2* g2 = reinterpret_cast<const __half2*>(&g);
          const __half2* b2 = reinterpret_cast<const __half2*>(&b);
          const uint32_t xs[8] = {x[2 * j].x, x[2 * j].y, x[2 * j].z, x[2 * j].w,
                                  x[2 * j + 1].x, x[2 * j + 1].y, x[2 * j + 1].z, x[2 * j + 1].w};
          uint32_t o[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 gf = __half22float2(g2[q]);
            const float2 bf = __half22float2(b2[q]);
            o[q] = ptx::pack_half2((__uint_as_float(xs[2 * q]) - mean) * rstd * gf.x + bf.x,
                                   (__uint_as_float(xs[2 * q + 1]) - mean) * rstd * gf.y + bf.y);
          }
          *reinterpret_cast<uint4*>(orow + col + 8 * j) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
    }
  }
  ring_count += static_cast<uint32_t>(boxes);
}

// One visit of a warp to the device-wide queue of panels whose statistics are complete.  Lane 0 claims at
// most one unit with atomicAdd on the claim counter.  A claim can run ahead of publication (the counter is
// bumped before the panel it falls into is published): such a unit stays in `pending` and is retried at the
// next visit.  Returns kLnWorked after normalising a unit, kLnAllDone when every unit of the problem has been
// claimed and this warp holds none, kLnIdle otherwise.
// deadline_ns != 0 (the drain after the last tile): past it, or once the CTA has aborted, report kLnAllDone.
enum LnVisit : int { kLnIdle = 0, kLnWorked = 1, kLnAllDone = 2 };
template <int BN>
__device__ __forceinline__ int ln_visit(const GemmParams& p, int& pending, uint32_t lane, uint32_t buf_base,
                                         uint32_t bar_base, uint32_t& ring_count, volatile int* cta_abort,
                                         uint64_t deadline_ns) {
  int* q = p.ln_queue;
  const int upp = ln_units_per_panel(p.n);
  const int total = ((p.m + 127) / 128) * upp;
  int unit = -1, panel = 0, done = 0;
  if (lane == 0) {
    if (pending < 0) {
      const int head = ld_volatile_i32(q + 1);
      if (head >= total) {
        done = 1;
      } else if (head < ld_volatile_i32(q) * upp) {
        const int c = atomicAdd(q + 1, 1);
        if (c >= total)
          done = 1;
        else
          pending = c;
      }
    }
    if (pending >= 0) {
      const int slot = pending / upp;
      if (slot < ld_volatile_i32(q)) {
        const int item = ld_volatile_i32(q + kLnQueueItems + slot);
        if (item != 0) {
          unit = pending % upp;
          panel = item - 1;
          pending = -1;
        }
      }
    }
    if (deadline_ns != 0 && unit < 0 && !done) {
      if (!*cta_abort && ptx::globaltimer_ns() > deadline_ns) {
        *cta_abort = 1;
        if (p.status) atomicCAS(p.status, 0, static_cast<int>(kFaultReduceWait));
      }
      if (*cta_abort) done = 1;
    }
  }
  unit = __shfl_sync(0xffffffffu, unit, 0);
  panel = __shfl_sync(0xffffffffu, panel, 0);
  done = __shfl_sync(0xffffffffu, done, 0);
  if (unit >= 0) {
    __threadfence();  // acquire side of the publication: panel data and statistics are visible below
    ln_normalise_unit<BN>(p, panel, unit, lane, buf_base, bar_base, ring_count, cta_abort);
    return kLnWorked;
  }
  return done != 0 ? kLnAllDone : kLnIdle;
}

// ------------------------------------------------------------------ split-K: fixed-order sum of the partials
// C[r][c] = fp16( sum over planes of partial[plane][r][c] ), the planes dealt to kReduceGroups groups of
// consecutive planes: inside a group the planes are added in ascending order, then the group sums are added
// in ascending group order.  The association depends only on the plane count, never on timing or on how the
// work is spread over threads, so results are bitwise reproducible, and the reduction kernel at the end of this
// file and the tail of the one-kernel path (splitk_stream.cuh) produce identical bits.
constexpr int kReduceGroups = 8;
constexpr int kReduceUnitsPerPass = 16;  // float4 output groups that 128 threads (8 groups x 16) reduce together

template <int BN, int kStages, int kCta, int kMode>
__global__ void __launch_bounds__((GemmShape<BN, kStages, kCta, kMode>::kThreads), 1)
    gemmrc_umma_kernel(const __grid_constant__ GemmParams p) {
  using S = GemmShape<BN, kStages, kCta, kMode>;
  extern __shared__ uint8_t smem_raw[];

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t cta_rank = (kCta == 2) ? ptx::cluster_ctarank() : 0u;
  const bool leader = cta_rank == 0;
  Walk walk;
  walk.stride = (kCta == 2) ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  walk.first = (kCta == 2) ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);

  // ---- shared-memory carve-up (tile buffers need 1024-byte alignment for the 128 B swizzle)
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t staging_base = smem_base + kStages * S::kStageBytes;  // 1024-aligned: stage sizes are multiples
  const uint32_t bar_base = staging_base + S::kStagingBytes;
  auto smem_a = [&](int s) { return smem_base + s * S::kStageBytes; };
  auto smem_b = [&](int s) { return smem_base + s * S::kStageBytes + S::kABytes; };
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tmem_full_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto tmem_empty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  auto ln_ring_bar = [&](uint32_t quad_) { return bar_base + 8u * (2 * kStages + 4 + 4 * quad_); };  // 4 per warp
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(
      smem_gen + kStages * S::kStageBytes + S::kStagingBytes + 8 * (2 * kStages + 4 + 16));
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  // Folded split-K (M, N <= 64; BN = 128, one CTA): a stage carries TWO k-blocks.  Rows 0..63 of the A box hold
  // A's rows for k-block 2i and rows 64..127 the same rows for k-block 2i + 1 (likewise B), so one M = 128,
  // N = 128 UMMA computes [A_2i; A_2i+1] x [B_2i; B_2i+1]^T, whose two diagonal 64 x 64 blocks are the wanted
  // products (the off-diagonal blocks are ignored).  No shared-memory row is zero fill, and the ring holds twice
  // as much of K.  The two diagonal blocks leave as two partial slices (2 * slice, 2 * slice + 1).
  constexpr bool kCanFold = is_splitk_mode(kMode) && BN == 128 && kCta == 1;
  // Cut tiles (GEMM on pairs, BN = 256): a pair's LAST item may be one 128-column half of a tile (the launcher cuts at
  // most one tile per pair).  Its B box has half the rows (tm_b_tail) and its UMMAs have N = 128.  One thread cannot
  // keep the tensor pipe busy with those (UMMAs into one accumulator complete one after the other, a UMMA of N = 128
  // is shorter than the gap between two completions, and one thread cannot issue them faster either), nor can one
  // thread issue a k-block's two copies in the time such a k-block takes.  So a cut item runs on two chains: warp 1
  // issues the even k-blocks into the left 128 columns of the item's accumulator, warp 6 the odd k-blocks into the
  // right 128 columns, each releasing the stages it read, and the epilogue adds the two halves; warp 7 issues the
  // item's B copies while warp 0 issues the A copies.  A cut tile's elements are thus the sum of two partial sums over
  // alternate k-blocks: a fixed order, but not that of a whole tile.  Warps 6 and 7 sleep on cut_start_bar and
  // cut_load_bar until warps 1 and 0 reach the cut item: a parity wait on a ring barrier is only meaningful within
  // one phase of the ring's position, so they must not look at the ring before.  Warp 6 reports the end of its chain
  // on cut_full_bar.  (The three mbarriers are slots of the LayerNorm mode's landing ring.)
  constexpr bool kTail = S::kCutTiles;
  const uint32_t cut_full_bar = bar_base + 8u * (2 * kStages + 4 + 8);
  const uint32_t cut_start_bar = bar_base + 8u * (2 * kStages + 4 + 9);
  const uint32_t cut_load_bar = bar_base + 8u * (2 * kStages + 4 + 10);
  const bool fold = kCanFold && p.fold != 0;
  const int num_kb = fold ? ((p.k + S::kBK - 1) / S::kBK + 1) / 2 : (p.k + S::kBK - 1) / S::kBK;
  auto load_stage = [&](int s, int kb, int row_a, int row_b, uint64_t pol_a_, uint64_t pol_b_) {  // one CTA per tile
    ptx::mbar_arrive_expect_tx(full_bar(s), S::kStageBytes);
    if (fold) {
      const int k0 = 2 * kb * S::kBK;
      ptx::tma_load_2d_hint(smem_a(s), &p.tm_a, full_bar(s), k0, row_a, pol_a_);
      ptx::tma_load_2d_hint(smem_a(s) + S::kABytes / 2, &p.tm_a, full_bar(s), k0 + S::kBK, row_a, pol_a_);
      ptx::tma_load_2d_hint(smem_b(s), &p.tm_b, full_bar(s), k0, row_b, pol_b_);
      ptx::tma_load_2d_hint(smem_b(s) + S::kBBytes / 2, &p.tm_b, full_bar(s), k0 + S::kBK, row_b, pol_b_);
    } else {
      ptx::tma_load_2d_hint(smem_a(s), &p.tm_a, full_bar(s), kb * S::kBK, row_a, pol_a_);
      ptx::tma_load_2d_hint(smem_b(s), &p.tm_b, full_bar(s), kb * S::kBK, row_b, pol_b_);
    }
  };
  uint32_t preloaded = 0;  // k-blocks of the first work item that thread 0 put in flight during set-up
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(tmem_full_bar(a), 1);
      ptx::mbar_init(tmem_empty_bar(a), 4 * kCta);  // one arrive per epilogue warp of each CTA
    }
    if constexpr (kMode == kModeLayerNorm) {
      for (uint32_t i = 0; i < 16; ++i) ptx::mbar_init(ln_ring_bar(0) + 8u * i, 1);
    }
    if constexpr (kTail) {
      ptx::mbar_init(cut_full_bar, 1);
      ptx::mbar_init(cut_start_bar, 1);
      ptx::mbar_init(cut_load_bar, 1);
    }
    *cta_abort = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&p.tm_a);
    ptx::prefetch_tensormap(&p.tm_b);
    if constexpr (is_splitk_mode(kMode) || kMode == kModeGemm) {
      // Launched as a programmatic dependent of the kernel before it on the stream (split-K: the previous call's
      // reduction): everything above may run while that grid drains; nothing below reads or writes global memory
      // before it has completed (the other threads pass the CTA barrier below after this wait).
      // Split-K with BEAM_FLAG_INPUTS_STABLE: the caller vouches that A and B are not that grid's outputs, and the
      // loads below may start at once; the partial stores wait for it in the epilogue either way.
      // (GEMM on pairs: only the producer threads read global memory before anything is written, and they wait
      // after the set-up barriers below instead, which then overlap the preceding grid's tail as well.)
      if (is_splitk_mode(kMode) ? !(p.flags & 1) : kCta == 1) ptx::grid_dependency_wait();
      // In turn, let the next kernel on the stream (this call's reduction kernel, or the next call) become
      // resident early; it blocks in its own griddepcontrol.wait until this grid is done.
      ptx::grid_launch_dependents();
    }
    if constexpr (kCta == 1) {
      // The ring starts empty, so the first loads need no wait: put them in flight before the CTA-wide
      // set-up barrier (TMEM allocation) instead of after it.  Thread 0 is also the producer thread.
      WorkItem w0;
      if (work_item<kMode, kTail>(p, walk, 0, num_kb, w0)) {
        const int row_a = w0.mt * S::kBM;
        const int row_b = w0.nt * BN;
        for (int kb = w0.kb0; kb < w0.kb1 && preloaded < static_cast<uint32_t>(kStages); ++kb, ++preloaded) {
          load_stage(static_cast<int>(preloaded), kb, row_a, row_b, ptx::l2_policy(p.hint_a),
                     ptx::l2_policy(p.hint_b));
        }
      }
    }
  }
  if (warp == 1) {
    ptx::tmem_alloc<kCta>(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), S::kTmemCols);
    ptx::tmem_relinquish<kCta>();
  }
  ptx::tc_fence_before();
  __syncthreads();
  if constexpr (kCta == 2) ptx::cluster_sync_all();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      if constexpr (kMode == kModeGemm && kCta == 2) ptx::grid_dependency_wait();  // before the first global read
      uint32_t it = 0;
      bool alive = true;
      const uint64_t pol_a = ptx::l2_policy(p.hint_a);
      const uint64_t pol_b = ptx::l2_policy(p.hint_b);
      WorkItem w;
      for (int j = 0; alive && work_item<kMode, kTail>(p, walk, j, num_kb, w); ++j) {
        int row_a = w.mt * (S::kBM * kCta) + static_cast<int>(cta_rank) * S::kBM;
        const bool cut = kTail && w.half >= 0;
        int row_b = cut ? w.nt * BN + w.half * (BN / 2) + static_cast<int>(cta_rank) * (S::kBRows / 2)
                        : w.nt * BN + static_cast<int>(cta_rank) * S::kBRows;
        const CUtensorMap* map_b = cut ? &p.tm_b_tail : &p.tm_b;
        const uint32_t pair_bytes = 2u * (S::kABytes + (cut ? S::kBBytes / 2 : S::kBBytes));
        int kb = w.kb0;
        if (j == 0) {  // these are already in flight
          kb += static_cast<int>(preloaded);
          it = preloaded;
        }
        if constexpr (kTail) {
          if (cut) ptx::mbar_arrive(cut_load_bar);  // wake the second producer thread, which loads this item's B boxes
        }
        for (; kb < w.kb1; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1u;
          if (!bounded_wait(empty_bar(s), ph ^ 1u, cta_abort, p.status, kFaultProducerWait)) {
            alive = false;
            break;
          }
          if constexpr (kCta == 1) {
            load_stage(s, kb, row_a, row_b, pol_a, pol_b);
          } else {
            // Both CTAs' bytes are counted on the leader's barrier; only the leader arms it.
            if (leader) ptx::mbar_arrive_expect_tx(full_bar(s), pair_bytes);
            const uint32_t lead_bar = ptx::mapa(full_bar(s), 0);
            ptx::tma_load_2d_pair_hint(smem_a(s), &p.tm_a, lead_bar, kb * S::kBK, row_a, pol_a);
            if (!cut) ptx::tma_load_2d_pair_hint(smem_b(s), map_b, lead_bar, kb * S::kBK, row_b, pol_b);
          }
        }
      }
    }
  } else if (warp == 7) {
    // ------------------------------------------------------------------ second TMA producer (cut tiles only)
    // One thread needs about as long to issue a k-block's two copies as the tensor pipe needs for a whole tile's
    // k-block, so a cut item, whose k-blocks take half as long, has its B boxes loaded by a thread of their own.
    if constexpr (kTail) {
      if (lane == 0) {
        const uint64_t pol_b = ptx::l2_policy(p.hint_b);
        WorkItem w;
        for (int j = 0; work_item<kMode, kTail>(p, walk, j, num_kb, w); ++j) {
          if (w.half < 0) continue;
          if (!bounded_wait(cut_load_bar, 0u, cta_abort, p.status, kFaultProducerWait, 30 * kWaitLimitNs)) break;
          const uint32_t it0 = static_cast<uint32_t>(j) * static_cast<uint32_t>(num_kb);
          const int row_b = w.nt * BN + w.half * (BN / 2) + static_cast<int>(cta_rank) * (S::kBRows / 2);
          uint32_t it = it0;
          for (int kb = w.kb0; kb < w.kb1; ++kb, ++it) {
            const int s = it % kStages;
            const uint32_t ph = (it / kStages) & 1u;
            if (!bounded_wait(empty_bar(s), ph ^ 1u, cta_abort, p.status, kFaultProducerWait)) break;
            ptx::tma_load_2d_pair_hint(smem_b(s), &p.tm_b_tail, ptx::mapa(full_bar(s), 0), kb * S::kBK, row_b,
                                       pol_b);
          }
          break;  // a pair has at most one cut item, its last
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && leader) {
      const uint32_t idesc = ptx::umma_idesc_f16_f32(S::kBM * kCta, BN) | (p.bf16 ? ptx::kIdescBf16Inputs : 0u);
      const uint32_t idesc_cut = ptx::umma_idesc_f16_f32(S::kBM * kCta, BN / 2) | (p.bf16 ? ptx::kIdescBf16Inputs : 0u);
      // The issuing thread is a single dependent instruction stream and, for N = 128, has only 256 clocks of tensor
      // work per k-block to hide behind: the stage index and barrier parity advance incrementally (no division), the
      // descriptors are the stage-0 descriptors plus a stride, and a k-block's four UMMAs are one instruction group.
      uint32_t stage = 0, parity = 0;
      const uint64_t a_desc0 = ptx::umma_desc_k_sw128(smem_a(0));
      const uint64_t b_desc0 = ptx::umma_desc_k_sw128(smem_b(0));
      constexpr uint64_t kDescStride = static_cast<uint64_t>(S::kStageBytes >> 4);
      bool alive = true;
      WorkItem w;
      for (int j = 0; alive && work_item<kMode, kTail>(p, walk, j, num_kb, w); ++j) {
        const uint32_t acc = static_cast<uint32_t>(j) & 1u;
        const uint32_t acc_ph = (static_cast<uint32_t>(j) >> 1) & 1u;
        {
          const bool drained = bounded_wait(tmem_empty_bar(acc), acc_ph ^ 1u, cta_abort, p.status, kFaultMmaWaitAcc);
          if (!drained) break;
        }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        if constexpr (kTail) {
          if (w.half >= 0) ptx::mbar_arrive(cut_start_bar);  // wake the second issuing thread
        }
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if constexpr (kTail) {
            if (w.half >= 0 && ((kb - w.kb0) & 1)) {  // the odd k-blocks of a cut item are the second thread's
              if (++stage == static_cast<uint32_t>(kStages)) {
                stage = 0;
                parity ^= 1u;
              }
              continue;
            }
          }
          {
            const bool landed = bounded_wait(full_bar(stage), parity, cta_abort, p.status, kFaultMmaWaitFull);
            if (!landed) {
              alive = false;
              break;
            }
          }
          ptx::tc_fence_after();
          if constexpr (kTail) {
            ptx::umma_f16_kblock<kCta>(d_tmem, a_desc0 + stage * kDescStride, b_desc0 + stage * kDescStride,
                                       w.half >= 0 ? idesc_cut : idesc, kb > w.kb0 ? 1u : 0u);
          } else {
            ptx::umma_f16_kblock<kCta>(d_tmem, a_desc0 + stage * kDescStride, b_desc0 + stage * kDescStride, idesc,
                                       kb > w.kb0 ? 1u : 0u);
          }
          if constexpr (kCta == 1)
            ptx::umma_commit<1>(empty_bar(stage));
          else
            ptx::umma_commit_pair_both(empty_bar(stage), 0x3);
          if (++stage == static_cast<uint32_t>(kStages)) {
            stage = 0;
            parity ^= 1u;
          }
        }
        if (alive) {
          if constexpr (kCta == 1)
            ptx::umma_commit<1>(tmem_full_bar(acc));
          else
            ptx::umma_commit_pair_both(tmem_full_bar(acc), 0x3);
        }
      }
    }
  } else if (warp == 6) {
    // ------------------------------------------------------------------ second MMA issuer (cut tiles only)
    if constexpr (kTail) {
      if (lane == 0 && leader) {
        const uint32_t idesc_cut =
            ptx::umma_idesc_f16_f32(S::kBM * kCta, BN / 2) | (p.bf16 ? ptx::kIdescBf16Inputs : 0u);
        const uint64_t a_desc0 = ptx::umma_desc_k_sw128(smem_a(0));
        const uint64_t b_desc0 = ptx::umma_desc_k_sw128(smem_b(0));
        constexpr uint64_t kDescStride = static_cast<uint64_t>(S::kStageBytes >> 4);
        WorkItem w;
        for (int j = 0; work_item<kMode, kTail>(p, walk, j, num_kb, w); ++j) {
          if (w.half < 0) continue;
          // every earlier item was a whole tile of num_kb k-blocks: that fixes the ring position of this one
          const uint32_t it0 = static_cast<uint32_t>(j) * static_cast<uint32_t>(num_kb);
          uint32_t stage = it0 % kStages, parity = (it0 / kStages) & 1u;
          const uint32_t acc = static_cast<uint32_t>(j) & 1u;
          // Until warp 1 has seen the item's accumulator drained and starts on it.  This wait spans all the whole
          // tiles before, hence the long limit; an abort anywhere in the CTA still ends it at once.
          if (!bounded_wait(cut_start_bar, 0u, cta_abort, p.status, kFaultMmaWaitAcc, 30 * kWaitLimitNs)) break;
          ptx::tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * BN + BN / 2;
          bool alive = true;
          for (int kb = w.kb0; kb < w.kb1; ++kb) {
            if ((kb - w.kb0) & 1) {
              if (!bounded_wait(full_bar(stage), parity, cta_abort, p.status, kFaultMmaWaitFull)) {
                alive = false;
                break;
              }
              ptx::tc_fence_after();
              ptx::umma_f16_kblock<kCta>(d_tmem, a_desc0 + stage * kDescStride, b_desc0 + stage * kDescStride,
                                         idesc_cut, kb > w.kb0 + 1 ? 1u : 0u);
              ptx::umma_commit_pair_both(empty_bar(stage), 0x3);
            }
            if (++stage == static_cast<uint32_t>(kStages)) {
              stage = 0;
              parity ^= 1u;
            }
          }
          if (alive) ptx::umma_commit_pair_both(cut_full_bar, 0x3);
          break;  // a pair has at most one cut item, its last
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const uint32_t quad = warp & 3u;  // TMEM lanes [32*quad, 32*quad+32) are this warp's to read
    const uint32_t row_in_tile = quad * 32u + lane;
    const uint32_t lead_empty0 = (kCta == 2) ? ptx::mapa(tmem_empty_bar(0), 0) : tmem_empty_bar(0);
    uint32_t store_count = 0;  // bulk stores this warp has issued (selects the staging buffer)
    // kModeGemmSilu: chunks of the element-wise tensor are dealt round-robin to the grid's epilogue warps
    const long long ew_chunks = (kMode == kModeGemmSilu) ? (p.ew_count + 1023) / 1024 : 0;
    const long long ew_stride = static_cast<long long>(gridDim.x) * 4;
    long long ew_chunk = static_cast<long long>(blockIdx.x) * 4 + quad;
    if constexpr (is_splitk_mode(kMode)) ptx::grid_dependency_wait();  // before this thread's first global write
    int ln_pending = -1;                               // LayerNorm: a unit this warp claimed ahead of its publication
    uint32_t ln_ring_count = 0;                        // LayerNorm: boxes this warp's landing ring has received
    const uint32_t ln_bufs = staging_base + quad * S::kBufsPerWarp * S::kStoreBufBytes;
    WorkItem w;
    for (int j = 0; work_item<kMode, kTail>(p, walk, j, num_kb, w); ++j) {
      const uint32_t acc = static_cast<uint32_t>(j) & 1u;
      const uint32_t acc_ph = (static_cast<uint32_t>(j) >> 1) & 1u;
      // Lane 0 polls (with back-off) for the whole warp, which stays converged for the .sync.aligned TMEM
      // loads below.
      bool ready;
      if constexpr (kMode == kModeGemmSilu) {
        // While the accumulator is not ready, this warp works through its share of the element-wise tensor.
        const uint64_t deadline = ptx::globaltimer_ns() + kWaitLimitNs;
        for (;;) {
          int hit = 0;
          if (lane == 0) hit = ptx::mbar_try_wait(tmem_full_bar(acc), acc_ph) ? 1 : 0;
          hit = __shfl_sync(0xffffffffu, hit, 0);
          if (hit) {
            ready = true;
            break;
          }
          if (ew_chunk < ew_chunks) {
            silu_chunk(p, ew_chunk, lane);
            ew_chunk += ew_stride;
          } else {
            __nanosleep(128);
            int give_up = 0;
            if (lane == 0) {
              if (!*cta_abort && ptx::globaltimer_ns() > deadline) {
                *cta_abort = 1;
                if (p.status) atomicCAS(p.status, 0, static_cast<int>(kFaultEpilogueWait));
              }
              give_up = *cta_abort;
            }
            if (__shfl_sync(0xffffffffu, give_up, 0)) {
              ready = false;
              break;
            }
          }
        }
      } else if constexpr (kMode == kModeLayerNorm) {
        // While the accumulator is not ready, this warp spends the time on the second pass: one unit of a
        // published panel per iteration (its staging buffers are idle: its stores have completed).
        const uint64_t deadline = ptx::globaltimer_ns() + kWaitLimitNs;
        bool pass2_done = false;
        for (;;) {
          int hit = 0;
          if (lane == 0) hit = ptx::mbar_try_wait(tmem_full_bar(acc), acc_ph) ? 1 : 0;
          hit = __shfl_sync(0xffffffffu, hit, 0);
          if (hit) {
            ready = true;
            break;
          }
          int did = kLnIdle;
          if (!pass2_done) {
            did = ln_visit<BN>(p, ln_pending, lane, ln_bufs, ln_ring_bar(quad), ln_ring_count, cta_abort, 0);
            pass2_done = did == kLnAllDone;
          }
          if (did != kLnWorked) {
            __nanosleep(128);
            int give_up = 0;
            if (lane == 0) {
              if (!*cta_abort && ptx::globaltimer_ns() > deadline) {
                *cta_abort = 1;
                if (p.status) atomicCAS(p.status, 0, static_cast<int>(kFaultEpilogueWait));
              }
              give_up = *cta_abort;
            }
            if (__shfl_sync(0xffffffffu, give_up, 0)) {
              ready = false;
              break;
            }
          }
        }
      } else {
        ready = bounded_wait_warp(tmem_full_bar(acc), acc_ph, cta_abort, p.status, kFaultEpilogueWait, lane);
      }
      if constexpr (kTail) {
        if (ready && w.half >= 0)  // the second issuing thread's chain (a pair's only cut item: phase 0)
          ready = bounded_wait_warp(cut_full_bar, 0u, cta_abort, p.status, kFaultEpilogueWait, lane);
      }
      if (!ready) break;
      ptx::tc_fence_after();
      const int row0 = w.mt * (S::kBM * kCta) + static_cast<int>(cta_rank) * S::kBM;  // first row of this CTA
      const int grow = row0 + static_cast<int>(row_in_tile);
      const bool cut = kTail && w.half >= 0;
      const int col0 = w.nt * BN + (cut ? w.half * (BN / 2) : 0);
      const uint32_t taddr = tmem_base + ((quad * 32u) << 16) + acc * BN;
      float st_n = 0.f, st_mean = 0.f, st_m2 = 0.f;  // LayerNorm: this row's statistics over this tile
      // One chunk = 128 bytes per row: 64 fp16 columns (GEMM) or 32 fp32 columns (split-K, LayerNorm).
      constexpr bool kHalfOut = (kMode == kModeGemm || kMode == kModeGemmSilu);  // fp16 C through tm_c
      constexpr int kChunkCols = kHalfOut ? 64 : 32;
      // Folded split-K: lanes 0..63 own the block in TMEM columns 0..63, lanes 64..127 the one in columns 64..127.
      const int fold_half = fold ? static_cast<int>(quad >> 1) : 0;
      const int c_begin = fold ? fold_half * 64 : 0;
      const int c_end = fold ? c_begin + 64 : (cut ? BN / 2 : BN);
#pragma unroll 1
      for (int c = c_begin; c < c_end; c += kChunkCols) {
        uint32_t out[32];  // this row's 128 bytes of the chunk
        if constexpr (kHalfOut) {
          uint32_t v0[32], v1[32];
          ptx::tmem_ld_32x32(taddr + c, v0);
          ptx::tmem_ld_32x32(taddr + c + 32, v1);
          ptx::tmem_ld_wait();
          if constexpr (kTail) {
            if (cut && w.kb1 - w.kb0 > 1) {  // warp-uniform: add the odd k-blocks' partial sums (the accumulator's other half)
              uint32_t u[32];
              ptx::tmem_ld_32x32(taddr + c + BN / 2, u);
              ptx::tmem_ld_wait();
#pragma unroll
              for (int q = 0; q < 32; ++q) v0[q] = __float_as_uint(__uint_as_float(v0[q]) + __uint_as_float(u[q]));
              ptx::tmem_ld_32x32(taddr + c + 32 + BN / 2, u);
              ptx::tmem_ld_wait();
#pragma unroll
              for (int q = 0; q < 32; ++q) v1[q] = __float_as_uint(__uint_as_float(v1[q]) + __uint_as_float(u[q]));
            }
          }
#pragma unroll
          for (int q = 0; q < 16; ++q) {
            out[q] = ptx::pack_out2(__uint_as_float(v0[2 * q]), __uint_as_float(v0[2 * q + 1]), p.bf16);
            out[16 + q] = ptx::pack_out2(__uint_as_float(v1[2 * q]), __uint_as_float(v1[2 * q + 1]), p.bf16);
          }
        } else {
          ptx::tmem_ld_32x32(taddr + c, out);
          ptx::tmem_ld_wait();
          if constexpr (kMode == kModeLayerNorm) {
            // Two-pass statistics of the (up to) 32 values in registers, merged into the row's running
            // (count, mean, M2).  Columns past N do not exist and are left out.
            const int valid = min(32, p.n - (col0 + c));
            if (valid > 0) {
              float sum = 0.f;
#pragma unroll
              for (int q = 0; q < 32; ++q) sum += (q < valid) ? __uint_as_float(out[q]) : 0.f;
              const float mb = sum / static_cast<float>(valid);
              float m2b = 0.f;
#pragma unroll
              for (int q = 0; q < 32; ++q) {
                const float d = __uint_as_float(out[q]) - mb;
                m2b += (q < valid) ? d * d : 0.f;
              }
              welford_merge(st_n, st_mean, st_m2, static_cast<float>(valid), mb, m2b);
            }
          }
        }
        // where the box goes: (x, y) in C / scratch coordinates, z = scratch plane
        const int box_x = fold ? c - c_begin : col0 + c;
        const int box_y = fold ? static_cast<int>(quad & 1u) * 32 : row0 + static_cast<int>(quad) * 32;
        const int box_z = fold ? 2 * w.slice + fold_half : w.slice;
        bool box_live = box_x < p.n && box_y < p.m;  // warp-uniform
        if (box_live) {
          // Before a staging buffer is rewritten, the bulk store that last read it must be done reading.
          constexpr uint32_t kBufs = S::kBufsPerWarp;
          const uint32_t buf = staging_base + (quad * kBufs + (store_count % kBufs)) * S::kStoreBufBytes;
          if (store_count >= kBufs) {
            if (lane == 0) ptx::tma_store_wait_read<kBufs - 1>();
            __syncwarp();
          }
          // Row `lane` of the box, 16-byte piece j at (j ^ (lane & 7)): the 128-byte swizzle the copy
          // engine expects, which also spreads each quarter-warp's stores over all banks.
          const uint32_t row_addr = buf + lane * 128u;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            ptx::st_shared_v4(row_addr + ((static_cast<uint32_t>(j) ^ (lane & 7u)) << 4), out[4 * j], out[4 * j + 1],
                              out[4 * j + 2], out[4 * j + 3]);
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if constexpr (kHalfOut) {
              store_c_box(p, buf, box_x, box_y);
            } else {
              ptx::tma_store_3d(&p.tm_s, buf, box_x, box_y, box_z);
              ptx::tma_store_commit();
            }
          }
          ++store_count;
        }
      }
      // The accumulator is drained: hand it back to the MMA issuer before the slow part below.
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (kCta == 1)
          ptx::mbar_arrive(tmem_empty_bar(acc));
        else
          ptx::mbar_arrive_cluster(lead_empty0 + 8u * acc);
      }
      if constexpr (kMode == kModeLayerNorm) {
        // Publish this row's (mean, M2) over the tile; once this warp's parked rows have landed, fence and take
        // one of the panel's tickets (four per tile, one per epilogue warp).  The warp that draws the panel's
        // last ticket publishes it for normalisation.
        if (grow < p.m) p.row_part[static_cast<size_t>(grow) * p.n_tiles + w.nt] = make_float2(st_mean, st_m2);
        if (lane == 0) ptx::tma_store_wait_all<0>();
        __syncwarp();
        __threadfence();
        __syncwarp();
        if (lane == 0 && row0 < p.m) {  // a pair's second CTA can sit wholly below the last row
          const int panel = row0 / S::kBM;
          if (atomicAdd(p.tickets + panel, 1) == 4 * p.n_tiles - 1) {
            __threadfence();
            const int slot = atomicAdd(p.ln_queue, 1);
            *reinterpret_cast<volatile int*>(p.ln_queue + kLnQueueItems + slot) = panel + 1;
          }
        }
      }
    }
    if constexpr (kMode == kModeGemmSilu) {
      for (; ew_chunk < ew_chunks; ew_chunk += ew_stride) silu_chunk(p, ew_chunk, lane);
    }
    if constexpr (kMode == kModeLayerNorm) {
      // No tiles left: keep normalising until every unit of the problem has been claimed and this warp's own
      // claim is done.  Other CTAs may still be computing, so this is a wait, and it is bounded.
      const uint64_t deadline = ptx::globaltimer_ns() + kWaitLimitNs;
      for (;;) {
        const int did = ln_visit<BN>(p, ln_pending, lane, ln_bufs, ln_ring_bar(quad), ln_ring_count, cta_abort, deadline);
        if (did == kLnAllDone) break;
        if (did == kLnIdle) __nanosleep(100);
      }
    }
  }

  // ---- teardown: bulk stores must have finished reading shared memory (and, for the kernels that follow,
  // writing global memory) before the CTA goes away; then everyone meets and the allocating warp frees TMEM
  if (warp >= 2 && lane == 0) {
    // A plain GEMM only needs its staging buffers back (the stores have READ them); their writes to C complete with
    // the grid like any other store.  Partials, LayerNorm panels and stores into peer GPUs are waited for in full.
    if (kMode == kModeGemm && p.n_peers == 0)
      ptx::tma_store_wait_read<0>();
    else
      ptx::tma_store_wait_all<0>();
  }
  __syncwarp();
  if (*cta_abort) abort_drain_delay();
  ptx::tc_fence_before();
  __syncthreads();
  if constexpr (kCta == 2) ptx::cluster_sync_all();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc<kCta>(tmem_base, S::kTmemCols);
  }
}

// Second kernel of the two-kernel split-K path: the same fixed-order sum with a block per row x 128 columns;
// thread (g, q) adds the slices of group g (a contiguous range, ascending) for 4 columns, then the 8 group
// sums are added in ascending g.
static __global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ partial,
                                                                   __half* __restrict__ c, int m, int n,
                                                                   int slices) {
  ptx::grid_launch_dependents();  // the next call's first kernel may set itself up while this grid runs
  ptx::grid_dependency_wait();    // partials of the producing kernel are complete and visible
  __shared__ float4 sums[kReduceGroups][32];
  const int q = threadIdx.x & 31;
  const int g = threadIdx.x >> 5;
  const int row = blockIdx.y;
  const int col = blockIdx.x * 128 + q * 4;
  const bool live = col < n;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (live) {
    const int s0 = slices * g / kReduceGroups;
    const int s1 = slices * (g + 1) / kReduceGroups;
    const size_t plane = static_cast<size_t>(m) * n;
    const float* src = partial + static_cast<size_t>(row) * n + col;
    constexpr int kBatch = 8;  // independent loads in flight; the additions stay in ascending slice order
    for (int s = s0; s < s1; s += kBatch) {
      float4 v[kBatch];
#pragma unroll
      for (int i = 0; i < kBatch; ++i)
        v[i] = (s + i < s1) ? __ldcg(reinterpret_cast<const float4*>(src + plane * (s + i)))
                            : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int i = 0; i < kBatch; ++i) {
        if (s + i < s1) {
          acc.x += v[i].x; acc.y += v[i].y; acc.z += v[i].z; acc.w += v[i].w;
        }
      }
    }
  }
  sums[g][q] = acc;
  __syncthreads();
  if (g == 0 && live) {
    float4 t = sums[0][q];
#pragma unroll
    for (int gg = 1; gg < kReduceGroups; ++gg) {
      const float4 u = sums[gg][q];
      t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
    }
    uint2 o;
    o.x = ptx::pack_half2(t.x, t.y);
    o.y = ptx::pack_half2(t.z, t.w);
    *reinterpret_cast<uint2*>(c + static_cast<size_t>(row) * n + col) = o;
  }
}


// The same sum for larger outputs (a split-K problem of 512 x 512 and up): one thread per 4 columns walks all the
// planes, eight loads in flight, and folds a group's sum into the total when the walk leaves the group, so the
// additions are those of splitk_reduce_kernel in the same order (bit-identical), without its block per row and
// its exchange through shared memory: with a million outputs that kernel needs seven waves of short blocks.
static __global__ void __launch_bounds__(256) splitk_reduce_flat_kernel(const float* __restrict__ partial,
                                                                        __half* __restrict__ c, int m, int n,
                                                                        int slices) {
  ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();
  const int quads = n >> 2;  // N is a multiple of 8
  const long long idx = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  if (idx >= static_cast<long long>(m) * quads) return;
  const int row = static_cast<int>(idx / quads);
  const int col = static_cast<int>(idx - static_cast<long long>(row) * quads) * 4;
  const size_t plane = static_cast<size_t>(m) * n;
  const float* src = partial + static_cast<size_t>(row) * n + col;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f), t = acc;
  int g = 0;
  int g_end = slices / kReduceGroups;  // slices * (g + 1) / kReduceGroups for g = 0
  auto fold = [&]() {
    if (g == 0) {
      t = acc;
    } else {
      t.x += acc.x; t.y += acc.y; t.z += acc.z; t.w += acc.w;
    }
    acc = make_float4(0.f, 0.f, 0.f, 0.f);
    ++g;
    g_end = slices * (g + 1) / kReduceGroups;
  };
  constexpr int kBatch = 8;
  for (int s = 0; s < slices; s += kBatch) {
    float4 v[kBatch];
#pragma unroll
    for (int i = 0; i < kBatch; ++i)
      v[i] = (s + i < slices) ? __ldcg(reinterpret_cast<const float4*>(src + plane * (s + i)))
                              : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      if (s + i < slices) {
        while (s + i >= g_end) fold();  // the walk has left group g (groups may be empty)
        acc.x += v[i].x; acc.y += v[i].y; acc.z += v[i].z; acc.w += v[i].w;
      }
    }
  }
  while (g < kReduceGroups) fold();
  uint2 o;
  o.x = ptx::pack_half2(t.x, t.y);
  o.y = ptx::pack_half2(t.z, t.w);
  *reinterpret_cast<uint2*>(c + static_cast<size_t>(row) * n + col) = o;
}

}  // namespace beam
