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
//   warps 2..5  epilogue       wait tmem_full[acc], tcgen05.ld 32 lanes x 32 columns at a time, then
//                              release the accumulator through tmem_empty[acc].
//
// TMEM holds two accumulators (2 x BN fp32 columns) so the epilogue of work item i overlaps the
// main loop of item i+1.  In pair mode each CTA loads its own 128 rows of A and its own BN/2 rows
// of B (plain per-CTA TMA loads that signal the leader's mbarrier), the leader's UMMA reads both
// CTAs' shared memory and writes both CTAs' TMEM, and completion is fanned out to both CTAs with
// the two-CTA form of tcgen05.commit.
//
// Three epilogues share this pipeline:
//   kModeGemm       fp32 -> fp16, store C.
//   kModeSplitK     a work item is (tile, K slice); the fp32 partial goes to workspace[slice][M][N]
//                   and a second kernel sums the slices in index order.
//   kModeLayerNorm  tiles are walked in GEMM order (so A and B stay L2-resident).  Each tile's epilogue
//                   parks its fp32 values in a scratch panel, writes one (mean, M2) pair per row for
//                   its N range, and takes a ticket for its 128-row panel.  The CTA that draws the last
//                   ticket of a panel merges the per-tile statistics in tile order, re-reads the panel
//                   (still in L2), normalises, applies gamma/beta and stores fp16.  Nobody waits.
#pragma once

#include "umma_common.cuh"

namespace beam {

enum GemmMode : int { kModeGemm = 0, kModeSplitK = 1, kModeLayerNorm = 2 };

struct GemmParams {
  CUtensorMap tm_a;  // A  [M, K], box 128 x 64, 128 B swizzle
  CUtensorMap tm_b;  // B  [N, K], box (BN / kCta) x 64, 128 B swizzle
  __half* c;         // fp16 output [M, ldc]
  float* scratch;    // split-K: partials [slices][M][N]; LayerNorm: fp32 panel store [M][N]
  float2* row_part;  // LayerNorm: (mean, M2) of every row over each N tile, [M][n_tiles]
  int* tickets;      // LayerNorm: arrival counter per 128-row panel, zero at launch
  const __half* gamma;
  const __half* beta;
  float eps;
  int m, n, k;
  int ldc;
  int m_tiles;  // tiles of 128 * kCta rows
  int n_tiles;  // tiles of BN columns
  int group_m;  // M-tiles per rasterisation group (GEMM mode)
  int slices;   // split-K slices (1 otherwise)
  int* status;  // device fault word
};

template <int BN, int kStages, int kCta>
struct GemmShape {
  static constexpr int kBM = 128;
  static constexpr int kBK = 64;
  static constexpr int kBRows = BN / kCta;
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = kBRows * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = 2 * BN;  // 128, 256 or 512: a power of two >= 32
  static constexpr int kBarBytes = 256;
  static constexpr int kSmemBytes = kStages * kStageBytes + kBarBytes + 1024;  // + alignment slack
  static constexpr int kThreads = 192;
  static_assert(BN == 64 || BN == 128 || BN == 256, "UMMA N of the tile");
  static_assert(kCta == 1 || kCta == 2, "one CTA or a pair");
  static_assert((2 * kStages + 4) * 8 + 16 <= kBarBytes, "barrier block too small");  // + tmem, abort, ticket
};

struct WorkItem {
  int mt, nt;        // tile coordinates
  int kb0, kb1;      // k-block range [kb0, kb1)
  int slice;         // split-K slice index
};

// The j-th work item of the CTA (pair) whose first item index is `first` with `stride` CTAs (pairs)
// in the grid.  Returns false past the end.  All three roles call this with the same arguments and
// therefore walk identical sequences.
//   GEMM, LayerNorm: items are tiles; groups of `group_m` M-tiles are walked N-major so that tiles
//              in flight together share A rows and B rows in L2 (the reference's CTA remap at
//              cute_gemm_128x128.cu:23-33, restated for a persistent grid).
//   split-K:   items are (tile, slice), slice fastest; k-blocks are dealt out as evenly as possible.
template <int kMode>
__device__ __forceinline__ bool work_item(const GemmParams& p, int first, int stride, int j, int num_kb,
                                          WorkItem& w) {
  w.slice = 0;
  w.kb0 = 0;
  w.kb1 = num_kb;
  if constexpr (kMode != kModeSplitK) {
    const int t = first + j * stride;
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

// Chan's parallel update of (count, mean, M2) with a block of `nb` values whose own mean and M2 are given.
__device__ __forceinline__ void welford_merge(float& n, float& mean, float& m2, float nb, float mean_b, float m2_b) {
  const float nn = n + nb;
  const float delta = mean_b - mean;
  const float f = nb / nn;
  mean += delta * f;
  m2 += m2_b + delta * delta * n * f;
  n = nn;
}

template <int BN, int kStages, int kCta, int kMode>
__global__ void __launch_bounds__(192, 1) gemmrc_umma_kernel(const __grid_constant__ GemmParams p) {
  using S = GemmShape<BN, kStages, kCta>;
  extern __shared__ uint8_t smem_raw[];

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t cta_rank = (kCta == 2) ? ptx::cluster_ctarank() : 0u;
  const bool leader = cta_rank == 0;
  const int stride = (kCta == 2) ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  const int first = (kCta == 2) ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);

  // ---- shared-memory carve-up (tile buffers need 1024-byte alignment for the 128 B swizzle)
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + kStages * S::kStageBytes;
  auto smem_a = [&](int s) { return smem_base + s * S::kStageBytes; };
  auto smem_b = [&](int s) { return smem_base + s * S::kStageBytes + S::kABytes; };
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tmem_full_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto tmem_empty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  volatile uint32_t* tmem_slot =
      reinterpret_cast<volatile uint32_t*>(smem_gen + kStages * S::kStageBytes + 8 * (2 * kStages + 4));
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* ticket_slot = reinterpret_cast<volatile int*>(tmem_slot + 2);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(tmem_full_bar(a), 1);
      ptx::mbar_init(tmem_empty_bar(a), 4 * kCta);  // one arrive per epilogue warp of each CTA
    }
    *cta_abort = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&p.tm_a);
    ptx::prefetch_tensormap(&p.tm_b);
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
  if constexpr (kMode == kModeSplitK) {
    // Let the reduction kernel's blocks become resident early; they block until this grid is done.
    if (threadIdx.x == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  }

  const int num_kb = (p.k + S::kBK - 1) / S::kBK;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool alive = true;
      WorkItem w;
      for (int j = 0; alive && work_item<kMode>(p, first, stride, j, num_kb, w); ++j) {
        const int row_a = w.mt * (S::kBM * kCta) + static_cast<int>(cta_rank) * S::kBM;
        const int row_b = w.nt * BN + static_cast<int>(cta_rank) * S::kBRows;
        for (int kb = w.kb0; kb < w.kb1; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1u;
          if (!bounded_wait(empty_bar(s), ph ^ 1u, cta_abort, p.status, kFaultProducerWait)) {
            alive = false;
            break;
          }
          if constexpr (kCta == 1) {
            ptx::mbar_arrive_expect_tx(full_bar(s), S::kStageBytes);
            ptx::tma_load_2d(smem_a(s), &p.tm_a, full_bar(s), kb * S::kBK, row_a);
            ptx::tma_load_2d(smem_b(s), &p.tm_b, full_bar(s), kb * S::kBK, row_b);
          } else {
            // Both CTAs' bytes are counted on the leader's barrier; only the leader arms it.
            if (leader) ptx::mbar_arrive_expect_tx(full_bar(s), 2 * S::kStageBytes);
            const uint32_t lead_bar = ptx::mapa(full_bar(s), 0);
            ptx::tma_load_2d_pair(smem_a(s), &p.tm_a, lead_bar, kb * S::kBK, row_a);
            ptx::tma_load_2d_pair(smem_b(s), &p.tm_b, lead_bar, kb * S::kBK, row_b);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = ptx::umma_idesc_f16_f32(S::kBM * kCta, BN);
      uint32_t it = 0;
      bool alive = true;
      WorkItem w;
      for (int j = 0; alive && work_item<kMode>(p, first, stride, j, num_kb, w); ++j) {
        const uint32_t acc = static_cast<uint32_t>(j) & 1u;
        const uint32_t acc_ph = (static_cast<uint32_t>(j) >> 1) & 1u;
        if (!bounded_wait(tmem_empty_bar(acc), acc_ph ^ 1u, cta_abort, p.status, kFaultMmaWaitAcc)) break;
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = w.kb0; kb < w.kb1; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1u;
          if (!bounded_wait(full_bar(s), ph, cta_abort, p.status, kFaultMmaWaitFull)) {
            alive = false;
            break;
          }
          ptx::tc_fence_after();
          const uint64_t a_desc = ptx::umma_desc_k_sw128(smem_a(s));
          const uint64_t b_desc = ptx::umma_desc_k_sw128(smem_b(s));
#pragma unroll
          for (int kk = 0; kk < S::kBK / 16; ++kk) {
            // +32 bytes (2 x 16 B units) along K inside the 128-byte swizzle atom per UMMA.
            ptx::umma_f16<kCta>(d_tmem, a_desc + 2u * kk, b_desc + 2u * kk, idesc,
                                (kb > w.kb0 || kk > 0) ? 1u : 0u);
          }
          if constexpr (kCta == 1)
            ptx::umma_commit<1>(empty_bar(s));
          else
            ptx::umma_commit_pair_both(empty_bar(s), 0x3);
        }
        if (alive) {
          if constexpr (kCta == 1)
            ptx::umma_commit<1>(tmem_full_bar(acc));
          else
            ptx::umma_commit_pair_both(tmem_full_bar(acc), 0x3);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const uint32_t quad = warp & 3u;  // TMEM lanes [32*quad, 32*quad+32) are this warp's to read
    const uint32_t row_in_tile = quad * 32u + lane;
    const uint32_t lead_empty0 = (kCta == 2) ? ptx::mapa(tmem_empty_bar(0), 0) : tmem_empty_bar(0);
    WorkItem w;
    for (int j = 0; work_item<kMode>(p, first, stride, j, num_kb, w); ++j) {
      const uint32_t acc = static_cast<uint32_t>(j) & 1u;
      const uint32_t acc_ph = (static_cast<uint32_t>(j) >> 1) & 1u;
      // Every lane polls; the vote keeps the warp together for the .sync.aligned TMEM loads below.
      const bool ready = bounded_wait(tmem_full_bar(acc), acc_ph, cta_abort, p.status, kFaultEpilogueWait);
      if (!__all_sync(0xffffffffu, ready)) break;
      ptx::tc_fence_after();
      const int row0 = w.mt * (S::kBM * kCta) + static_cast<int>(cta_rank) * S::kBM;  // first row of this CTA
      const int grow = row0 + static_cast<int>(row_in_tile);
      const int col0 = w.nt * BN;
      const uint32_t taddr = tmem_base + ((quad * 32u) << 16) + acc * BN;
      float st_n = 0.f, st_mean = 0.f, st_m2 = 0.f;  // LayerNorm: this row's statistics over this tile
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t v[32];
        ptx::tmem_ld_32x32(taddr + c, v);
        ptx::tmem_ld_wait();
        if constexpr (kMode == kModeGemm) {
          if (grow < p.m) {
            __half* crow = p.c + static_cast<size_t>(grow) * p.ldc + col0 + c;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              if (col0 + c + 8 * q < p.n) {  // N % 8 == 0, so a started group of 8 is whole
                uint4 o;
                o.x = ptx::pack_half2(__uint_as_float(v[8 * q + 0]), __uint_as_float(v[8 * q + 1]));
                o.y = ptx::pack_half2(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3]));
                o.z = ptx::pack_half2(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5]));
                o.w = ptx::pack_half2(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7]));
                *reinterpret_cast<uint4*>(crow + 8 * q) = o;
              }
            }
          }
        } else {
          // fp32 rows: split-K partial of this slice, or the parked LayerNorm panel.
          if (grow < p.m) {
            float* srow = p.scratch +
                          (static_cast<size_t>(w.slice) * p.m + static_cast<size_t>(grow)) * p.n + col0 + c;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              if (col0 + c + 4 * q < p.n) {
                __stcg(reinterpret_cast<uint4*>(srow + 4 * q),
                       make_uint4(v[4 * q + 0], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]));
              }
            }
          }
          if constexpr (kMode == kModeLayerNorm) {
            // Two-pass statistics of the (up to) 32 values in registers, merged into the row's running
            // (count, mean, M2).  Columns past N do not exist and are left out.
            const int valid = min(32, p.n - (col0 + c));
            if (valid > 0) {
              float s = 0.f;
#pragma unroll
              for (int q = 0; q < 32; ++q) s += (q < valid) ? __uint_as_float(v[q]) : 0.f;
              const float mb = s / static_cast<float>(valid);
              float m2b = 0.f;
#pragma unroll
              for (int q = 0; q < 32; ++q) {
                const float d = __uint_as_float(v[q]) - mb;
                m2b += (q < valid) ? d * d : 0.f;
              }
              welford_merge(st_n, st_mean, st_m2, static_cast<float>(valid), mb, m2b);
            }
          }
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
        // Publish this row's (mean, M2) over the tile, then take the panel's ticket.  The fence before
        // the barrier orders every epilogue thread's scratch and statistics stores before the ticket.
        if (grow < p.m) p.row_part[static_cast<size_t>(grow) * p.n_tiles + w.nt] = make_float2(st_mean, st_m2);
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");  // the 4 epilogue warps only
        if (warp == 2 && lane == 0) *ticket_slot = atomicAdd(p.tickets + row0 / S::kBM, 1);
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const bool last = (*ticket_slot == p.n_tiles - 1);
        if (last) {
          __threadfence();
          // Whole rows per warp, lane = column group: the panel is re-read and the output written in
          // 512-byte runs.  Every lane merges the row's per-tile statistics in tile order.
          const int rows_here = min(S::kBM, p.m - row0);
          for (int r = static_cast<int>(quad); r < rows_here; r += 4) {
            float n_acc = 0.f, mean = 0.f, m2 = 0.f;
            const float2* parts = p.row_part + static_cast<size_t>(row0 + r) * p.n_tiles;
            for (int t = 0; t < p.n_tiles; ++t) {
              const float2 pt = __ldcg(parts + t);
              welford_merge(n_acc, mean, m2, static_cast<float>(min(BN, p.n - t * BN)), pt.x, pt.y);
            }
            const float rstd = rsqrtf(m2 / n_acc + p.eps);
            const float* srow = p.scratch + static_cast<size_t>(row0 + r) * p.n;
            __half* orow = p.c + static_cast<size_t>(row0 + r) * p.ldc;
            for (int col = static_cast<int>(lane) * 8; col < p.n; col += 256) {
              const float4 x0 = __ldcg(reinterpret_cast<const float4*>(srow + col));
              const float4 x1 = __ldcg(reinterpret_cast<const float4*>(srow + col + 4));
              const uint4 g = __ldg(reinterpret_cast<const uint4*>(p.gamma + col));
              const uint4 b = __ldg(reinterpret_cast<const uint4*>(p.beta + col));
              const __half2* g2 = reinterpret_cast<const __half2*>(&g);
              const __half2* b2 = reinterpret_cast<const __half2*>(&b);
              const float xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
              uint32_t o[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const float2 gf = __half22float2(g2[q]);
                const float2 bf = __half22float2(b2[q]);
                const float y0 = (xs[2 * q] - mean) * rstd * gf.x + bf.x;
                const float y1 = (xs[2 * q + 1] - mean) * rstd * gf.y + bf.y;
                o[q] = ptx::pack_half2(y0, y1);
              }
              *reinterpret_cast<uint4*>(orow + col) = make_uint4(o[0], o[1], o[2], o[3]);
            }
          }
        }
      }
    }
  }

  // ---- teardown: everyone meets, then the allocating warp frees TMEM
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

// Second kernel of split-K: C[r][c] = fp16( sum over slices, in a fixed order, of partial[s][r][c] ).
// A block owns one row x 128 columns; thread (g, q) adds the slices of group g (a contiguous range,
// ascending) for 4 columns, then the 8 group sums are added in ascending g.  The association order
// depends only on the slice count, never on timing, so results are bitwise reproducible.
constexpr int kReduceGroups = 8;
static __global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ partial,
                                                            __half* __restrict__ c, int m, int n, int slices) {
  asm volatile("griddepcontrol.wait;" ::: "memory");  // partials of the producing kernel are complete
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
    int s = s0;
    for (; s + 4 <= s1; s += 4) {
      const float4 v0 = __ldcg(reinterpret_cast<const float4*>(src + plane * s));
      const float4 v1 = __ldcg(reinterpret_cast<const float4*>(src + plane * (s + 1)));
      const float4 v2 = __ldcg(reinterpret_cast<const float4*>(src + plane * (s + 2)));
      const float4 v3 = __ldcg(reinterpret_cast<const float4*>(src + plane * (s + 3)));
      acc.x += v0.x; acc.y += v0.y; acc.z += v0.z; acc.w += v0.w;
      acc.x += v1.x; acc.y += v1.y; acc.z += v1.z; acc.w += v1.w;
      acc.x += v2.x; acc.y += v2.y; acc.z += v2.z; acc.w += v2.w;
      acc.x += v3.x; acc.y += v3.y; acc.z += v3.z; acc.w += v3.w;
    }
    for (; s < s1; ++s) {
      const float4 v0 = __ldcg(reinterpret_cast<const float4*>(src + plane * s));
      acc.x += v0.x; acc.y += v0.y; acc.z += v0.z; acc.w += v0.w;
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

}  // namespace beam
