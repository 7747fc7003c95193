// Split-K rc GEMM as ONE kernel per call: C[M,N] = A[M,K] * B[N,K]^T for small M, N and huge K.
//
// Every CTA owns one (output tile, K slice): it streams its slice of A and B through a TMA ring into a TMEM
// accumulator, writes the fp32 partial tile to workspace[plane][M][N], meets the other CTAs at a grid-wide barrier
// (the grid is launched cooperatively: all CTAs are resident) and then sums its share of the output over all planes
// in the fixed order of splitk_reduce_kernel (gemmrc_umma.cuh), so one-kernel and two-kernel calls agree bit
// for bit.
//
// What a single call costs besides streaming its bytes was measured with time stamps (128 x 256 x 65536, 128 CTAs):
// 1.1 us between the previous kernel's exit and this one's entry, 2.0 us of set-up before the first load, 8.4 us
// from the last UMMA to the exit (1.3 us draining TMEM chunk by chunk, 0.7 us until the stores are visible, 1.8 us
// in the barrier, 4.6 us reading 64 KB of partials per CTA with ordinary loads).  This kernel is shaped by that:
//   * it needs less than half of an SM's shared memory and TMEM, so the next call's CTAs (a programmatic dependent
//     launch) become resident beside this call's and finish their whole set-up while this call is still running;
//   * the accumulator is pulled out of TMEM with all loads in flight at once and staged in the (by then idle)
//     operand ring, from where TMA stores move it to the workspace;
//   * after the barrier the partials come back as ONE tiled TMA copy per CTA (all planes of the CTA's share of
//     the output at once) and are summed from shared memory.
#pragma once

#include <cooperative_groups.h>

#include "gemmrc_umma.cuh"

namespace beam {

template <int BN, int kStages>
struct StreamShape {
  static constexpr int kBM = 128;
  static constexpr int kBK = 64;
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kRingBytes = kStages * kStageBytes;
  static constexpr int kTmemCols = BN < 32 ? 32 : BN;
  static constexpr int kBarBytes = 256;
  static constexpr int kSumsBytes = 32 * 1024;      // group sums of the final reduction: 8 groups x 256 float4
  static constexpr int kMaxBoxGranules = 128;       // 32-byte granules of one plane per read-back copy (256 units)
  static constexpr int kSmemBytes = kRingBytes + kBarBytes + 1024;  // + alignment slack
  static constexpr int kThreads = 192;
  // The drained accumulator (128 rows x BN fp32) is staged in the ring before it leaves through TMA.
  static_assert(kBM * BN * 4 <= kRingBytes, "the ring must hold one fp32 tile");
  static_assert(kSmemBytes <= 113 * 1024, "two CTAs must fit on one SM");
  static_assert(BN == 64 || BN == 128, "UMMA N of the tile (a 256-wide tile does not fit twice on an SM)");
  static_assert((2 * kStages + 2) * 8 + 16 <= kBarBytes, "barrier block too small");
};

namespace ptx {
// Untiled bulk copy global -> this CTA's shared memory; both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
               "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ float4 ld_shared_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}
}  // namespace ptx

// Problems with M, N <= 64 run "folded" (kFold): a stage carries TWO k-blocks, rows 0..63 of the A box hold A's rows
// for k-block 2i and rows 64..127 the same rows for k-block 2i + 1 (likewise B), so one M = 128, N = 128 UMMA
// computes [A_2i; A_2i+1] x [B_2i; B_2i+1]^T, whose two diagonal 64 x 64 blocks are the wanted products and leave as
// two planes (2 * slice, 2 * slice + 1).
template <int BN, int kStages, bool kFold>
__global__ void __launch_bounds__(192, 2) splitk_stream_kernel(const __grid_constant__ GemmParams p) {
  using S = StreamShape<BN, kStages>;
  static_assert(!kFold || BN == 128, "folding uses the 128 x 128 UMMA");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;

  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + S::kRingBytes;
  auto smem_a = [&](int s) { return smem_base + s * S::kStageBytes; };
  auto smem_b = [&](int s) { return smem_base + s * S::kStageBytes + S::kABytes; };
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  const uint32_t tmem_full_bar = bar_base + 8u * (2 * kStages);
  const uint32_t reduce_bar = bar_base + 8u * (2 * kStages + 1);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + S::kRingBytes + 8 * (2 * kStages + 2));
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  // ---- set-up: nothing here touches global memory, so it runs while the previous kernel on the stream is still busy
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    ptx::mbar_init(tmem_full_bar, 1);
    ptx::mbar_init(reduce_bar, 1);
    *cta_abort = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&p.tm_a);
    ptx::prefetch_tensormap(&p.tm_b);
    ptx::prefetch_tensormap(&p.tm_s);
    ptx::prefetch_tensormap(&p.tm_peer[0]);
    // The next kernel on the stream may become resident now; it blocks in its own griddepcontrol.wait.
    ptx::grid_launch_dependents();
  }
  if (warp == 1) {
    ptx::tmem_alloc<1>(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), S::kTmemCols);
    ptx::tmem_relinquish<1>();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // ---- this CTA's work item: slice fastest, then N tile, then M tile
  const int num_kb = kFold ? ((p.k + S::kBK - 1) / S::kBK + 1) / 2 : (p.k + S::kBK - 1) / S::kBK;
  const int item = static_cast<int>(blockIdx.x);
  const int slice = item % p.slices;
  const int tile = item / p.slices;
  const int nt = tile % p.n_tiles;
  const int mt = tile / p.n_tiles;
  const int kb0 = static_cast<int>(static_cast<long long>(num_kb) * slice / p.slices);
  const int kb1 = static_cast<int>(static_cast<long long>(num_kb) * (slice + 1) / p.slices);
  const bool has_work = mt < p.m_tiles && kb1 > kb0;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && has_work) {
      // A and B may be outputs of the previous kernel unless the caller vouches otherwise (BEAM_FLAG_INPUTS_STABLE).
      if (!(p.flags & 1)) ptx::grid_dependency_wait();
      const int row_a = mt * S::kBM;
      const int row_b = nt * BN;
      uint32_t it = 0;
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % kStages;
        const uint32_t ph = (it / kStages) & 1u;
        if (!bounded_wait(empty_bar(s), ph ^ 1u, cta_abort, p.status, kFaultProducerWait)) break;
        ptx::mbar_arrive_expect_tx(full_bar(s), S::kStageBytes);
        if constexpr (kFold) {
          const int k0 = 2 * kb * S::kBK;
          ptx::tma_load_2d(smem_a(s), &p.tm_a, full_bar(s), k0, row_a);
          ptx::tma_load_2d(smem_a(s) + S::kABytes / 2, &p.tm_a, full_bar(s), k0 + S::kBK, row_a);
          ptx::tma_load_2d(smem_b(s), &p.tm_b, full_bar(s), k0, row_b);
          ptx::tma_load_2d(smem_b(s) + S::kBBytes / 2, &p.tm_b, full_bar(s), k0 + S::kBK, row_b);
        } else {
          ptx::tma_load_2d(smem_a(s), &p.tm_a, full_bar(s), kb * S::kBK, row_a);
          ptx::tma_load_2d(smem_b(s), &p.tm_b, full_bar(s), kb * S::kBK, row_b);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && has_work) {
      const uint32_t idesc = ptx::umma_idesc_f16_f32(S::kBM, BN);
      uint32_t stage = 0, parity = 0;
      const uint64_t a_desc0 = ptx::umma_desc_k_sw128(smem_a(0));
      const uint64_t b_desc0 = ptx::umma_desc_k_sw128(smem_b(0));
      constexpr uint64_t kDescStride = static_cast<uint64_t>(S::kStageBytes >> 4);
      bool alive = true;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!bounded_wait(full_bar(stage), parity, cta_abort, p.status, kFaultMmaWaitFull)) {
          alive = false;
          break;
        }
        ptx::tc_fence_after();
        ptx::umma_f16_kblock<1>(tmem_base, a_desc0 + stage * kDescStride, b_desc0 + stage * kDescStride, idesc,
                                kb > kb0 ? 1u : 0u);
        ptx::umma_commit<1>(empty_bar(stage));
        if (++stage == static_cast<uint32_t>(kStages)) {
          stage = 0;
          parity ^= 1u;
        }
      }
      if (alive) ptx::umma_commit<1>(tmem_full_bar);
    }
  } else if (has_work) {
    // ------------------------------------------------------------------ epilogue (warps 2..5): partial tile -> workspace
    const uint32_t quad = warp & 3u;  // TMEM lanes [32*quad, 32*quad+32) are this warp's to read
    if (bounded_wait_warp(tmem_full_bar, 0, cta_abort, p.status, kFaultEpilogueWait, lane)) {
      ptx::tc_fence_after();
      // Every UMMA has retired, so the ring is idle: stage the whole tile there (box b of this warp at
      // quad * kBoxes + b, 4 KB each, 128-byte-swizzled rows) with all TMEM loads in flight at once.
      const int fold_half = kFold ? static_cast<int>(quad >> 1) : 0;
      const int c_begin = kFold ? fold_half * 64 : 0;
      constexpr int kCols = kFold ? 64 : BN;     // columns this warp drains
      constexpr int kBoxes = kCols / 32;
      constexpr int kBatch = 2;                  // boxes drained per pass: 2 x 32 registers in flight
      const uint32_t taddr = tmem_base + ((quad * 32u) << 16) + static_cast<uint32_t>(c_begin);
      const uint32_t stage_base = smem_base + quad * (kBoxes * 4096u);
      const uint32_t row_addr = lane * 128u;
      ptx::grid_dependency_wait();  // before this thread's first global write
#pragma unroll 1
      for (int b0 = 0; b0 < kBoxes; b0 += kBatch) {
        uint32_t v[kBatch][32];
#pragma unroll
        for (int b = 0; b < kBatch; ++b) ptx::tmem_ld_32x32(taddr + static_cast<uint32_t>((b0 + b) * 32), v[b]);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
          const uint32_t buf = stage_base + static_cast<uint32_t>(b0 + b) * 4096u;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            ptx::st_shared_v4(buf + row_addr + ((static_cast<uint32_t>(j) ^ (lane & 7u)) << 4), v[b][4 * j],
                              v[b][4 * j + 1], v[b][4 * j + 2], v[b][4 * j + 3]);
        }
      }
      ptx::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
#pragma unroll 1
        for (int b = 0; b < kBoxes; ++b) {
          // where the box goes: (x, y) in workspace coordinates, z = plane
          const int box_x = kFold ? b * 32 : nt * BN + b * 32;
          const int box_y = kFold ? static_cast<int>(quad & 1u) * 32 : mt * S::kBM + static_cast<int>(quad) * 32;
          const int box_z = kFold ? 2 * slice + fold_half : slice;
          if (box_x < p.n && box_y < p.m) ptx::tma_store_3d(&p.tm_s, stage_base + static_cast<uint32_t>(b) * 4096u, box_x, box_y, box_z);
        }
        ptx::tma_store_commit();
        ptx::tma_store_wait_all<0>();  // complete and visible to this thread; released to the grid below
      }
      __syncwarp();
    }
  }

  // ---- every CTA's partial is on its way to L2: meet, then sum.  All paths reach the barrier, including a CTA whose
  // bounded wait gave up (the fault word then tells the host that the result is invalid).
  // (No fence of our own here: the storing lanes have waited for their bulk stores to complete, and the grid barrier
  // releases at GPU scope after a CTA barrier and acquires on the way out.  A __threadfence() by every thread in
  // front of it cost 0.7 us per call.)
  cooperative_groups::this_grid().sync();
  {
    // The workspace is read back through a second tensor map that sees it as [planes][M * N / 8][8 floats]
    // ("granules" of 32 bytes, numbered row-major over the output): ONE tiled copy brings a run of granules of
    // EVERY plane into shared memory (plane s at offset s * rb_granules * 32).  Issuing a copy per plane from one
    // thread instead costs about 60 ns per copy, 4 us for 64 planes.  This CTA's share is granules [g0, g1).
    const int planes = p.slices * (kFold ? 2 : 1);
    const long long granules = (static_cast<long long>(p.m) * p.n) >> 3;
    const long long g0 = granules * blockIdx.x / gridDim.x;
    const long long g1 = granules * (blockIdx.x + 1) / gridDim.x;
    const int box_g = p.rb_granules;                       // granules per copy (what the tensor map's box holds)
    const uint32_t plane_bytes = static_cast<uint32_t>(box_g) * 32u;
    const uint32_t box_bytes = plane_bytes * static_cast<uint32_t>(planes);
    const int t = static_cast<int>(threadIdx.x);
    const int g = t >> 4, q = t & 15;
    const int s0 = planes * g / kReduceGroups, s1 = planes * (g + 1) / kReduceGroups;
    const int n4 = p.n >> 2;
    // group sums: [kReduceGroups][2 * box_g units] float4 at the tail of the ring (the host keeps box_g <= 128)
    float4* sums = reinterpret_cast<float4*>(smem_gen + S::kRingBytes - S::kSumsBytes);
    uint32_t pass = 0;
    for (long long gc = g0; gc < g1; gc += box_g, ++pass) {
      const int ng = static_cast<int>((g1 - gc < box_g) ? (g1 - gc) : box_g);  // granules of this pass that are ours
      if (threadIdx.x == 0) {
        ptx::mbar_arrive_expect_tx(reduce_bar, box_bytes);
        ptx::tma_load_3d(smem_base, &p.tm_peer[0], reduce_bar, 0, static_cast<int>(gc), 0);
      }
      // every thread waits on the barrier itself (whoever sees the phase complete sees the copied bytes); the
      // verdict is made uniform so that nobody is left behind at a CTA barrier
      const int landed = bounded_wait(reduce_bar, pass & 1u, cta_abort, p.status, kFaultReduceWait) ? 1 : 0;
      if (!__syncthreads_and(landed)) break;
      const int nu = 2 * ng;  // float4 units of this pass
      if (t < 128) {
        for (int u = q; u < nu; u += kReduceUnitsPerPass) {
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
          const uint32_t addr = smem_base + static_cast<uint32_t>(u) * 16u;
          for (int sp = s0; sp < s1; ++sp) {
            const float4 v = ptx::ld_shared_f4(addr + static_cast<uint32_t>(sp) * plane_bytes);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
          }
          sums[g * (2 * box_g) + u] = acc;
        }
      }
      __syncthreads();
      for (int u = t; u < nu; u += S::kThreads) {
        float4 r = sums[u];
#pragma unroll
        for (int gg = 1; gg < kReduceGroups; ++gg) {
          const float4 w = sums[gg * (2 * box_g) + u];
          r.x += w.x; r.y += w.y; r.z += w.z; r.w += w.w;
        }
        const long long unit = 2 * gc + u;
        uint2 o;
        o.x = ptx::pack_half2(r.x, r.y);
        o.y = ptx::pack_half2(r.z, r.w);
        *reinterpret_cast<uint2*>(p.c + (unit / n4) * p.n + (unit % n4) * 4) = o;
      }
      // the next pass's copy overwrites what this pass's loads read: generic reads before async writes
      ptx::fence_proxy_async_smem();
      __syncthreads();
    }
  }

  // ---- teardown
  if (*cta_abort) abort_drain_delay();
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc<1>(tmem_base, S::kTmemCols);
  }
}

}  // namespace beam
