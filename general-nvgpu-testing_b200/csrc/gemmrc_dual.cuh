// The N = 128 tile families (128 x 128 per CTA, 256 x 128 per CTA pair) with TWO output tiles in flight.
//
// A tcgen05.mma of N = 128, K = 16 is 64 clocks of tensor-pipe work, but consecutive UMMAs into the SAME
// accumulator retire only about every 120 clocks: the next one needs the previous result.  With one tile per
// CTA every instruction of the main loop targets the same accumulator, and the pipe idles for nearly half of
// the time.  Here a CTA (pair) works on two output tiles at once, the two vertically adjacent tiles of one N
// column, each with its own accumulator and its own issuing thread, so that the two dependent chains overlap.
// TMEM holds four 128-column accumulators: two being computed, two being drained by the epilogue.
//
// Both tiles multiply by the same rows of B, so a shared-memory stage carries the A box of each tile and ONE B box
// (a 128 x 128 tile needs 128 bytes per clock per SM from L2 at full tensor rate, which is all the L2 -> SM port
// delivers; sharing B brings the pair down to 96).  Work items are therefore pairs of tiles ("double tiles" of
// 2 x 128 x kCta rows), walked in the grouped raster of gemmrc_umma_kernel.  With an odd number of tile rows the
// last double tile's second tile lies below the matrix: its A box loads as zeros and its stores are skipped.
//
// Roles, barriers, staging and the TMA-store epilogue are those of gemmrc_umma_kernel in GEMM mode.
#pragma once

#include "gemmrc_umma.cuh"

namespace beam {

template <int kStages, int kCta>
struct DualShape {
  static constexpr int kBN = 128;
  static constexpr int kBM = 128;
  static constexpr int kBK = 64;
  static constexpr int kBRows = kBN / kCta;
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = kBRows * kBK * 2;
  static constexpr int kStageBytes = 2 * kABytes + kBBytes;  // [A of tile 0][A of tile 1][B, shared by both]
  static constexpr int kTmemCols = 4 * kBN;
  static constexpr int kBarBytes = 512;
  static constexpr int kStoreBufBytes = 32 * 128;
  static constexpr int kBufsPerWarp = 2;
  static constexpr int kStagingBytes = 4 * kBufsPerWarp * kStoreBufBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + kBarBytes + 1024;
  static constexpr int kThreads = 256;  // producer (A boxes), first issuer, four epilogue warps, second issuer, producer (B box)
  static_assert(kSmemBytes <= 232448, "exceeds the 227 KB of shared memory a CTA can opt in to");
  static_assert((2 * kStages + 4) * 8 + 32 <= kBarBytes, "barrier block too small");
  static_assert(kABytes % 1024 == 0 && kBBytes % 1024 == 0, "boxes must keep the 1024-byte alignment of the swizzle atom");
};

// Double tile `t` of the grouped raster (see work_item in gemmrc_umma.cuh; p.m_tiles counts double tiles here).
__device__ __forceinline__ void dual_item_coords(const GemmParams& p, int t, int& mt2, int& nt) {
  const int per_group = p.group_m * p.n_tiles;
  const int g = t / per_group;
  const int first_m = g * p.group_m;
  const int rows = min(p.group_m, p.m_tiles - first_m);
  const int r = t - g * per_group;
  mt2 = first_m + r % rows;
  nt = r / rows;
}

template <int kStages, int kCta>
__global__ void __launch_bounds__((DualShape<kStages, kCta>::kThreads), 1) gemmrc_dual_kernel(const __grid_constant__ GemmParams p) {
  using S = DualShape<kStages, kCta>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t cta_rank = (kCta == 2) ? ptx::cluster_ctarank() : 0u;
  const bool leader = cta_rank == 0;
  const int stride = (kCta == 2) ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  const int first = (kCta == 2) ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int items = p.m_tiles * p.n_tiles;  // double tiles

  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t staging_base = smem_base + kStages * S::kStageBytes;
  const uint32_t bar_base = staging_base + S::kStagingBytes;
  // stage s = [A of tile 0][A of tile 1][B]
  auto smem_a = [&](int s, int h) { return smem_base + s * S::kStageBytes + h * S::kABytes; };
  auto smem_b = [&](int s) { return smem_base + s * S::kStageBytes + 2 * S::kABytes; };
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tmem_full_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto tmem_empty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(
      smem_gen + kStages * S::kStageBytes + S::kStagingBytes + 8 * (2 * kStages + 4));
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int num_kb = (p.k + S::kBK - 1) / S::kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 2);  // both issuing threads commit the stage
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(tmem_full_bar(a), 2);  // ... and their accumulator
      ptx::mbar_init(tmem_empty_bar(a), 4 * kCta);  // one arrive per epilogue warp of each CTA
    }
    *cta_abort = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&p.tm_a);
    ptx::prefetch_tensormap(&p.tm_b);
    ptx::prefetch_tensormap(&p.tm_c);
    // A programmatic dependent of the kernel before it on the stream: the whole set-up may overlap that kernel's last
    // CTAs; the two producer threads wait for that grid before their first load, and nothing is written before data
    // has arrived.
    ptx::grid_launch_dependents();
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
      ptx::grid_dependency_wait();
      uint32_t it = 0;
      bool alive = true;
      const uint64_t pol_a = ptx::l2_policy(p.hint_a);
      for (int j = 0; alive && first + j * stride < items; ++j) {
        int mt2, nt;
        dual_item_coords(p, first + j * stride, mt2, nt);
        int row_a[2];
        for (int h = 0; h < 2; ++h) row_a[h] = (2 * mt2 + h) * (S::kBM * kCta) + static_cast<int>(cta_rank) * S::kBM;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1u;
          if (!bounded_wait(empty_bar(s), ph ^ 1u, cta_abort, p.status, kFaultProducerWait)) {
            alive = false;
            break;
          }
          if constexpr (kCta == 1) {
            ptx::mbar_arrive_expect_tx(full_bar(s), S::kStageBytes);
            for (int h = 0; h < 2; ++h)
              ptx::tma_load_2d_hint(smem_a(s, h), &p.tm_a, full_bar(s), kb * S::kBK, row_a[h], pol_a);
          } else {
            // Both CTAs' bytes are counted on the leader's barrier; only the leader arms it.
            if (leader) ptx::mbar_arrive_expect_tx(full_bar(s), 2 * S::kStageBytes);
            const uint32_t lead_bar = ptx::mapa(full_bar(s), 0);
            for (int h = 0; h < 2; ++h)
              ptx::tma_load_2d_pair_hint(smem_a(s, h), &p.tm_a, lead_bar, kb * S::kBK, row_a[h], pol_a);
          }
        }
      }
    }
  } else if (warp == 7) {
    // ------------------------------------------------------------------ second TMA producer: the B boxes
    // One thread issuing all three copies of a k-block cannot quite keep up with the two tiles' UMMAs at full clocks;
    // with the B box on a thread of its own the kernel gains 1.7 % (one CTA per tile) and 3.5 % (pairs) at 8192^3
    // (a thread per box is slower again).  Both producers walk the same items and wait on the same empty barriers.
    if (lane == 0) {
      ptx::grid_dependency_wait();
      uint32_t it = 0;
      bool alive = true;
      const uint64_t pol_b = ptx::l2_policy(p.hint_b);
      for (int j = 0; alive && first + j * stride < items; ++j) {
        int mt2, nt;
        dual_item_coords(p, first + j * stride, mt2, nt);
        const int row_b = nt * S::kBN + static_cast<int>(cta_rank) * S::kBRows;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1u;
          if (!bounded_wait(empty_bar(s), ph ^ 1u, cta_abort, p.status, kFaultProducerWait)) {
            alive = false;
            break;
          }
          if constexpr (kCta == 1)
            ptx::tma_load_2d_hint(smem_b(s), &p.tm_b, full_bar(s), kb * S::kBK, row_b, pol_b);
          else
            ptx::tma_load_2d_pair_hint(smem_b(s), &p.tm_b, ptx::mapa(full_bar(s), 0), kb * S::kBK, row_b, pol_b);
        }
      }
    }
  } else if (warp == 1 || warp == 6) {
    // ------------------------------------------------------------------ MMA issuers
    // One thread per tile of the pair (warp 1 the first tile, warp 6 the second).  A single thread issues a
    // tcgen05.mma about every 82 clocks at best, more than the 64 clocks an N = 128 instruction keeps the pipe busy
    // (one thread alternating between the two accumulators: 77.7 % of active cycles; 1212 -> 1301 TFLOP/s with two).
    // Each thread commits the stages it read and the accumulator it wrote; which thread's instruction reaches the
    // pipe first does not matter, the two never touch the same accumulator.
    if (lane == 0 && leader) {
      const uint32_t idesc = ptx::umma_idesc_f16_f32(S::kBM * kCta, S::kBN) | (p.bf16 ? ptx::kIdescBf16Inputs : 0u);
      const uint32_t mine = (warp == 6) ? 1u : 0u;  // which tile of the pair this thread issues
      uint32_t stage = 0, parity = 0;
      const uint64_t a_desc0 = ptx::umma_desc_k_sw128(smem_a(0, 0));
      const uint64_t b_desc0 = ptx::umma_desc_k_sw128(smem_b(0));
      constexpr uint64_t kDescStride = static_cast<uint64_t>(S::kStageBytes >> 4);
      constexpr uint64_t kDescTile = static_cast<uint64_t>(S::kABytes >> 4);  // from tile 0's A box to tile 1's
      bool alive = true;
      for (int j = 0; alive && first + j * stride < items; ++j) {
        const uint32_t acc = static_cast<uint32_t>(j) & 1u;  // which pair of accumulators
        const uint32_t acc_ph = (static_cast<uint32_t>(j) >> 1) & 1u;
        if (!bounded_wait(tmem_empty_bar(acc), acc_ph ^ 1u, cta_abort, p.status, kFaultMmaWaitAcc)) break;
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + (acc * 2u + mine) * S::kBN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!bounded_wait(full_bar(stage), parity, cta_abort, p.status, kFaultMmaWaitFull)) {
            alive = false;
            break;
          }
          ptx::tc_fence_after();
          ptx::umma_f16_kblock<kCta>(d_tmem, a_desc0 + stage * kDescStride + mine * kDescTile,
                                     b_desc0 + stage * kDescStride, idesc, kb > 0 ? 1u : 0u);
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
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const uint32_t quad = warp & 3u;  // TMEM lanes [32*quad, 32*quad+32) are this warp's to read
    const uint32_t lead_empty0 = (kCta == 2) ? ptx::mapa(tmem_empty_bar(0), 0) : tmem_empty_bar(0);
    uint32_t store_count = 0;
    for (int j = 0; first + j * stride < items; ++j) {
      const uint32_t acc = static_cast<uint32_t>(j) & 1u;
      const uint32_t acc_ph = (static_cast<uint32_t>(j) >> 1) & 1u;
      if (!bounded_wait_warp(tmem_full_bar(acc), acc_ph, cta_abort, p.status, kFaultEpilogueWait, lane)) break;
      ptx::tc_fence_after();
      int mt2, nt;
      dual_item_coords(p, first + j * stride, mt2, nt);
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        const int box_y = (2 * mt2 + h) * (S::kBM * kCta) + static_cast<int>(cta_rank) * S::kBM + static_cast<int>(quad) * 32;
        const int col0 = nt * S::kBN;
        const uint32_t taddr = tmem_base + ((quad * 32u) << 16) + (acc * 2u + static_cast<uint32_t>(h)) * S::kBN;
#pragma unroll 1
        for (int c = 0; c < S::kBN; c += 64) {
          uint32_t v0[32], v1[32], out[32];
          ptx::tmem_ld_32x32(taddr + c, v0);
          ptx::tmem_ld_32x32(taddr + c + 32, v1);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 16; ++q) {
            out[q] = ptx::pack_out2(__uint_as_float(v0[2 * q]), __uint_as_float(v0[2 * q + 1]), p.bf16);
            out[16 + q] = ptx::pack_out2(__uint_as_float(v1[2 * q]), __uint_as_float(v1[2 * q + 1]), p.bf16);
          }
          if (col0 + c < p.n && box_y < p.m) {  // warp-uniform
            const uint32_t buf = staging_base + (quad * S::kBufsPerWarp + (store_count % S::kBufsPerWarp)) * S::kStoreBufBytes;
            if (store_count >= static_cast<uint32_t>(S::kBufsPerWarp)) {
              if (lane == 0) ptx::tma_store_wait_read<S::kBufsPerWarp - 1>();
              __syncwarp();
            }
            const uint32_t row_addr = buf + lane * 128u;
#pragma unroll
            for (int jj = 0; jj < 8; ++jj)
              ptx::st_shared_v4(row_addr + ((static_cast<uint32_t>(jj) ^ (lane & 7u)) << 4), out[4 * jj], out[4 * jj + 1],
                                out[4 * jj + 2], out[4 * jj + 3]);
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) store_c_box(p, buf, col0 + c, box_y);
            ++store_count;
          }
        }
      }
      // both accumulators of the item are drained: hand the pair back to the issuer
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (kCta == 1)
          ptx::mbar_arrive(tmem_empty_bar(acc));
        else
          ptx::mbar_arrive_cluster(lead_empty0 + 8u * acc);
      }
    }
  }

  if (warp >= 2 && lane == 0) {  // staging buffers read; stores into peer GPUs are waited for in full
    if (p.n_peers == 0)
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

}  // namespace beam
