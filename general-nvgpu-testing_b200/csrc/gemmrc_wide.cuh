// 256 x 512 output tile per CTA pair: the large-GEMM kernel with both TMEM accumulators live at once.
//
// Same roles, barriers and TMA-store epilogue as gemmrc_umma_kernel in pair mode, but a k-block stage holds
// A (128 rows per CTA) and TWO B boxes (128 rows per CTA each, the two 256-column halves of the tile), and the
// leader issues tcgen05.mma (M = 256, N = 256) for both halves against the same A.  Per unit of math this
// moves 24 KB instead of 32 KB per CTA through L2 and shared memory, and a wave of 74 tiles touches fewer
// distinct operand rows per flop.
//
// The price: TMEM (512 columns) holds one tile, so the epilogue cannot hide behind the next tile's main loop
// by double-buffering.  It hides behind the ends of the main loops instead: the first and the last two
// k-blocks of a tile are issued half-major (half 0 of both, then half 1 of both), so half 0 completes early
// and is drained while half 1 finishes, and the issuer only needs half 0 back to start the next tile while
// half 1 is drained.  The drain of half 0 is the exposed part, so the epilogue is made short:
// eight warps (two per TMEM lane quadrant, 128 columns of each half apiece) pull a whole half into registers
// and hand it back before rounding or storing anything, so the hand-back does not wait for the C stores.
#pragma once

#include "gemmrc_umma.cuh"

namespace beam {

template <int kStages>
struct WideShape {
  static constexpr int kBM = 128;
  static constexpr int kBK = 64;
  static constexpr int kHalfN = 256;
  static constexpr int kTileN = 512;
  static constexpr int kBRows = kHalfN / 2;  // rows of one B half that one CTA of the pair loads
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBHalfBytes = kBRows * kBK * 2;
  static constexpr int kStageBytes = kABytes + 2 * kBHalfBytes;
  static constexpr int kTmemCols = 512;
  static constexpr int kBarBytes = 512;
  static constexpr int kStoreBufBytes = 32 * 128;
  static constexpr int kEpilogueWarps = 8;
  // A 3-deep ring leaves room for two staging buffers per epilogue warp; a 4-deep ring for one (a warp then
  // waits for its previous store to have read the buffer, which the TMEM loads and the rounding cover).
  static constexpr int kBufsPerWarp = (kStages <= 3) ? 2 : 1;
  static constexpr int kStagingBytes = kEpilogueWarps * kBufsPerWarp * kStoreBufBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + kBarBytes + 1024;
  static constexpr int kThreads = 64 + 32 * kEpilogueWarps;
  static_assert(kSmemBytes <= 232448, "exceeds the 227 KB of shared memory a CTA can opt in to");
  static_assert((2 * kStages + 4) * 8 + 16 <= kBarBytes, "barrier block too small");
};

// kTall = false: 256 x 512 tile, the two accumulators are the two 256-column halves (one A box, two B boxes
// per stage).  kTall = true: 512 x 256 tile, the two accumulators are the two 256-row halves (two A boxes, one
// B box per stage), and inside a k-block the UMMAs alternate between the halves so that consecutive
// instructions read the same B operand.
template <int kStages, bool kTall>
__global__ void __launch_bounds__(WideShape<kStages>::kThreads, 1) gemmrc_wide_kernel(const __grid_constant__ GemmParams p) {
  using S = WideShape<kStages>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t cta_rank = ptx::cluster_ctarank();
  const bool leader = cta_rank == 0;
  Walk walk;
  walk.stride = static_cast<int>(gridDim.x >> 1);
  walk.first = static_cast<int>(blockIdx.x >> 1);

  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t staging_base = smem_base + kStages * S::kStageBytes;
  const uint32_t bar_base = staging_base + S::kStagingBytes;
  // a stage is three 16 KB boxes; which of them hold A and B depends on the orientation
  auto smem_box = [&](int s, int i) { return smem_base + s * S::kStageBytes + i * S::kABytes; };
  auto smem_a = [&](int s, int h) { return smem_box(s, kTall ? h : 0); };
  auto smem_b = [&](int s, int h) { return smem_box(s, kTall ? 2 : 1 + h); };
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tmem_full_bar = [&](int h) { return bar_base + 8u * (2 * kStages + h); };       // one per accumulator half
  auto tmem_empty_bar = [&](int h) { return bar_base + 8u * (2 * kStages + 2 + h); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(
      smem_gen + kStages * S::kStageBytes + S::kStagingBytes + 8 * (2 * kStages + 4));
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    ptx::mbar_init(tmem_full_bar(0), 1);
    ptx::mbar_init(tmem_full_bar(1), 1);
    ptx::mbar_init(tmem_empty_bar(0), 2 * S::kEpilogueWarps);  // one arrive per epilogue warp of each CTA
    ptx::mbar_init(tmem_empty_bar(1), 2 * S::kEpilogueWarps);
    *cta_abort = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&p.tm_a);
    ptx::prefetch_tensormap(&p.tm_b);
    ptx::prefetch_tensormap(&p.tm_c);
    // Launched as a programmatic dependent of the kernel before it on the stream: this CTA may have become resident
    // and run the set-up (this block, the TMEM allocation, the barriers below) while that kernel's last CTAs were still
    // at work.  The producer thread waits for that grid before its first load; nothing is written before data arrives.
    // In turn, the next kernel on the stream may take SMs as this grid's CTAs leave them.
    ptx::grid_launch_dependents();
  }
  if (warp == 1) {
    ptx::tmem_alloc<2>(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), S::kTmemCols);
    ptx::tmem_relinquish<2>();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync_all();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int num_kb = (p.k + S::kBK - 1) / S::kBK;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      ptx::grid_dependency_wait();  // the preceding grid has completed: A and B may be its outputs
      uint32_t it = 0;
      bool alive = true;
      const uint64_t pol_a = ptx::l2_policy(p.hint_a);
      const uint64_t pol_b = ptx::l2_policy(p.hint_b);
      WorkItem w;
      for (int j = 0; alive && work_item<kModeGemm>(p, walk, j, num_kb, w); ++j) {
        // rows of the three boxes this CTA loads: (A, B half 0, B half 1) or (A half 0, A half 1, B)
        const int r0 = kTall ? w.mt * 512 + static_cast<int>(cta_rank) * S::kBM
                             : w.mt * 256 + static_cast<int>(cta_rank) * S::kBM;
        const int r1 = kTall ? r0 + 256 : w.nt * S::kTileN + static_cast<int>(cta_rank) * S::kBRows;
        const int r2 = kTall ? w.nt * 256 + static_cast<int>(cta_rank) * S::kBRows : r1 + S::kHalfN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1u;
          if (!bounded_wait(empty_bar(s), ph ^ 1u, cta_abort, p.status, kFaultProducerWait)) {
            alive = false;
            break;
          }
          if (leader) ptx::mbar_arrive_expect_tx(full_bar(s), 2 * S::kStageBytes);
          const uint32_t lead_bar = ptx::mapa(full_bar(s), 0);
          ptx::tma_load_2d_pair_hint(smem_box(s, 0), &p.tm_a, lead_bar, kb * S::kBK, r0, pol_a);
          ptx::tma_load_2d_pair_hint(smem_box(s, 1), kTall ? &p.tm_a : &p.tm_b, lead_bar, kb * S::kBK, r1,
                                     kTall ? pol_a : pol_b);
          ptx::tma_load_2d_pair_hint(smem_box(s, 2), &p.tm_b, lead_bar, kb * S::kBK, r2, pol_b);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA)
    if (lane == 0 && leader) {
      const uint32_t idesc = ptx::umma_idesc_f16_f32(256, S::kHalfN) | (p.bf16 ? ptx::kIdescBf16Inputs : 0u);
      uint32_t it = 0;
      bool alive = true;
      WorkItem w;
      auto issue_half = [&](int s, int h, bool first_kb) {
        const uint64_t a_desc = ptx::umma_desc_k_sw128(smem_a(s, h));
        const uint64_t b_desc = ptx::umma_desc_k_sw128(smem_b(s, h));
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(h) * S::kHalfN;
#pragma unroll
        for (int kk = 0; kk < S::kBK / 16; ++kk)
          ptx::umma_f16<2>(d_tmem, a_desc + 2u * kk, b_desc + 2u * kk, idesc, (!first_kb || kk > 0) ? 1u : 0u);
      };
      // A group of k-blocks issued half-major: half 0 of each (waiting for its bytes), then, after `between`,
      // half 1 of each, which is also where their stages are released.
      auto wait_landed = [&](uint32_t k) {
        const bool landed = bounded_wait(full_bar(k % kStages), (k / kStages) & 1u, cta_abort, p.status, kFaultMmaWaitFull);
        if (landed) ptx::tc_fence_after();
        return landed;
      };
      for (int j = 0; alive && work_item<kModeGemm>(p, walk, j, num_kb, w); ++j) {
        const uint32_t tile_ph = static_cast<uint32_t>(j) & 1u;
        // Tile boundary.  The first kLead k-blocks are issued half-major (needs only half 0 of the previous tile
        // back; half 1 is being drained meanwhile) and so are the last kLead (half 0 completes early and is drained
        // while half 1 finishes).  Longer groups pin more ring stages and starve the prefetch: two is the measured
        // optimum for a 3- or 4-deep ring.
        const int lead_in = num_kb < p.lead_in ? num_kb : p.lead_in;
        const int lead_out = (num_kb - lead_in) < p.lead_out ? (num_kb - lead_in) : p.lead_out;
        {
          const bool ok0 = bounded_wait(tmem_empty_bar(0), tile_ph ^ 1u, cta_abort, p.status, kFaultMmaWaitAcc);
          if (!ok0) break;
        }
        ptx::tc_fence_after();
        for (int g = 0; g < lead_in && alive; ++g) {
          alive = wait_landed(it + static_cast<uint32_t>(g));
          if (!alive) break;
          issue_half((it + static_cast<uint32_t>(g)) % kStages, 0, g == 0);
        }
        if (!alive) break;
        if (lead_in == num_kb) ptx::umma_commit_pair_both(tmem_full_bar(0), 0x3);  // half 0 is complete already
        {
          const bool ok1 = bounded_wait(tmem_empty_bar(1), tile_ph ^ 1u, cta_abort, p.status, kFaultMmaWaitAcc);
          if (!ok1) break;
        }
        ptx::tc_fence_after();
        for (int g = 0; g < lead_in; ++g) {
          const int s = (it + static_cast<uint32_t>(g)) % kStages;
          issue_half(s, 1, g == 0);
          ptx::umma_commit_pair_both(empty_bar(s), 0x3);
        }
        it += static_cast<uint32_t>(lead_in);
        for (int kb = lead_in; kb < num_kb - lead_out; ++kb, ++it) {
          alive = wait_landed(it);
          if (!alive) break;
          const int s = it % kStages;
          if (kTall) {
            // both halves multiply by the same B: alternate so that neighbouring UMMAs share the operand
            const uint64_t a0_desc = ptx::umma_desc_k_sw128(smem_a(s, 0));
            const uint64_t a1_desc = ptx::umma_desc_k_sw128(smem_a(s, 1));
            const uint64_t b_desc = ptx::umma_desc_k_sw128(smem_b(s, 0));
#pragma unroll
            for (int kk = 0; kk < S::kBK / 16; ++kk) {
              ptx::umma_f16<2>(tmem_base, a0_desc + 2u * kk, b_desc + 2u * kk, idesc, 1u);
              ptx::umma_f16<2>(tmem_base + S::kHalfN, a1_desc + 2u * kk, b_desc + 2u * kk, idesc, 1u);
            }
          } else {
            // both halves multiply the same A: alternate, and let the second UMMA of each pair take A from the
            // collector buffer the first one filled instead of reading shared memory again
            const uint64_t a_desc = ptx::umma_desc_k_sw128(smem_a(s, 0));
            const uint64_t b0_desc = ptx::umma_desc_k_sw128(smem_b(s, 0));
            const uint64_t b1_desc = ptx::umma_desc_k_sw128(smem_b(s, 1));
#pragma unroll
            for (int kk = 0; kk < S::kBK / 16; ++kk)
              ptx::umma_f16_pair_shared_a(tmem_base, tmem_base + S::kHalfN, a_desc + 2u * kk, b0_desc + 2u * kk,
                                          b1_desc + 2u * kk, idesc, 1u, 1u);
          }
          ptx::umma_commit_pair_both(empty_bar(s), 0x3);
        }
        if (!alive) break;
        if (lead_out == 0 && num_kb > lead_in) ptx::umma_commit_pair_both(tmem_full_bar(0), 0x3);
        if (lead_out > 0) {
          for (int g = 0; g < lead_out && alive; ++g) {
            alive = wait_landed(it + static_cast<uint32_t>(g));
            if (!alive) break;
            issue_half((it + static_cast<uint32_t>(g)) % kStages, 0, false);
          }
          if (!alive) break;
          ptx::umma_commit_pair_both(tmem_full_bar(0), 0x3);  // half 0 is complete: its drain starts now
          for (int g = 0; g < lead_out; ++g) {
            const int s = (it + static_cast<uint32_t>(g)) % kStages;
            issue_half(s, 1, false);
            ptx::umma_commit_pair_both(empty_bar(s), 0x3);
          }
          it += static_cast<uint32_t>(lead_out);
        }
        ptx::umma_commit_pair_both(tmem_full_bar(1), 0x3);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9, both CTAs)
    const uint32_t quad = warp & 3u;               // TMEM lane quadrant this warp may read
    const uint32_t col_half = (warp - 2u) >> 2;    // which 128 columns of each accumulator half it drains
    const uint32_t slot = warp - 2u;
    const uint32_t lead_empty0 = ptx::mapa(tmem_empty_bar(0), 0);
    const uint32_t lane_base = tmem_base + ((quad * 32u) << 16);
    // chunk i of a tile: half (i >> 1), columns col_half * 128 + (i & 1) * 64 of that half's accumulator
    auto chunk_col = [&](int i) { return (i >> 1) * S::kHalfN + static_cast<int>(col_half) * 128 + (i & 1) * 64; };
    // where chunk i lands in C relative to the tile's first row / column
    auto out_row = [&](int i) { return kTall ? (i >> 1) * 256 : 0; };
    auto out_col = [&](int i) { return kTall ? static_cast<int>(col_half) * 128 + (i & 1) * 64 : chunk_col(i); };
    uint32_t store_count = 0;
    WorkItem w;
    for (int j = 0; work_item<kModeGemm>(p, walk, j, num_kb, w); ++j) {
      {
        const bool ready = bounded_wait_warp(tmem_full_bar(0), static_cast<uint32_t>(j) & 1u, cta_abort, p.status,
                                             kFaultEpilogueWait, lane);
        if (!ready) break;
      }
      ptx::tc_fence_after();
      const int row0 = w.mt * (kTall ? 512 : 256) + static_cast<int>(cta_rank) * S::kBM + static_cast<int>(quad) * 32;
      const int tile_col0 = w.nt * (kTall ? 256 : S::kTileN);
      // Both halves are handed back as soon as their accumulators sit in registers, before anything is rounded or
      // stored: the issuer's wait then depends on TMEM load latency only, not on how fast the (bursty, all CTAs at
      // once) C stores drain the staging buffers.
      uint32_t va0[32], va1[32], vb0[32], vb1[32], out[32], out_b[32];
      auto load_chunk = [&](int i, uint32_t (&lo)[32], uint32_t (&hi)[32]) {
        ptx::tmem_ld_32x32(lane_base + chunk_col(i), lo);
        ptx::tmem_ld_32x32(lane_base + chunk_col(i) + 32, hi);
      };
      auto round_chunk = [&](const uint32_t (&lo)[32], const uint32_t (&hi)[32], uint32_t (&dst)[32]) {
#pragma unroll
        for (int q = 0; q < 16; ++q) {
          dst[q] = ptx::pack_out2(__uint_as_float(lo[2 * q]), __uint_as_float(lo[2 * q + 1]), p.bf16);
          dst[16 + q] = ptx::pack_out2(__uint_as_float(hi[2 * q]), __uint_as_float(hi[2 * q + 1]), p.bf16);
        }
      };
      auto release_half = [&](uint32_t h) {
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive_cluster(lead_empty0 + 8u * h);
      };
      auto stage_and_store = [&](int i, const uint32_t (&src)[32]) {
        const int col = tile_col0 + out_col(i);
        const int row = row0 + out_row(i);
        if (col < p.n && row < p.m) {
          constexpr uint32_t kBufs = S::kBufsPerWarp;
          const uint32_t buf = staging_base + (slot * kBufs + (store_count % kBufs)) * S::kStoreBufBytes;
          if (store_count >= kBufs) {
            if (lane == 0) ptx::tma_store_wait_read<kBufs - 1>();
            __syncwarp();
          }
          const uint32_t row_addr = buf + lane * 128u;
#pragma unroll
          for (int jj = 0; jj < 8; ++jj)
            ptx::st_shared_v4(row_addr + ((static_cast<uint32_t>(jj) ^ (lane & 7u)) << 4), src[4 * jj],
                              src[4 * jj + 1], src[4 * jj + 2], src[4 * jj + 3]);
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) store_c_box(p, buf, col, row);
          ++store_count;
        }
      };
      load_chunk(0, va0, va1);
      load_chunk(1, vb0, vb1);
      ptx::tmem_ld_wait();
      release_half(0);
      // Half 1 completes two half-k-blocks after half 0: that time goes into rounding half 0 and storing its first
      // chunk, so that once half 1 is complete nothing but its TMEM loads stands between it and its hand-back.
      round_chunk(va0, va1, out);
      stage_and_store(0, out);
      round_chunk(vb0, vb1, out_b);
      if (!bounded_wait_warp(tmem_full_bar(1), static_cast<uint32_t>(j) & 1u, cta_abort, p.status,
                             kFaultEpilogueWait, lane))
        break;
      ptx::tc_fence_after();
      load_chunk(2, va0, va1);
      load_chunk(3, vb0, vb1);
      ptx::tmem_ld_wait();
      release_half(1);
      stage_and_store(1, out_b);
      round_chunk(va0, va1, out);
      stage_and_store(2, out);
      round_chunk(vb0, vb1, out);
      stage_and_store(3, out);
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
  ptx::cluster_sync_all();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc<2>(tmem_base, S::kTmemCols);
  }
}

}  // namespace beam
