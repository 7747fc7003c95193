// Fused GEMM + LayerNorm whose pre-normalisation values never leave the SM.
//
// out[M,N] = LayerNorm_row(X[M,K] x W[N,K]^T) * gamma + beta.  A CTA pair (cta_group::2) owns 256 x 256 output
// tiles, walked in row-major tile order (all N tiles of a 256-row panel, then the next panel), and keeps TWO
// tiles in TMEM.  When a tile's UMMAs have retired, each epilogue warp reads its 32 rows once to compute the
// rows' (mean, M2) over the tile's columns, publishes them and takes a ticket for its 32-row block; the tile
// then STAYS in its accumulator while the pair computes its next tile in the other one.  Once a block's
// ticket count shows that all N tiles of those rows have published, the warp merges the per-tile statistics
// (Chan / Welford, tile order, so the result does not depend on timing), reads the accumulator a second
// time, applies (x - mean) * rstd * gamma + beta, stores fp16 through TMA and only then hands the
// accumulator back.  Nothing but the output and 8 bytes per row per tile of statistics touches global memory.
//
// Why this cannot deadlock: with at least as many resident pairs as N tiles, pair p's j-th tile is tile
// p + j * pairs, so consecutive tiles of a pair lie in different row panels and a panel's tiles lie in at most
// two consecutive rounds j.  A pair needs its round j-1 tile normalised before it can start round j+1; that
// needs the statistics of tiles of rounds <= j, and publishing a tile's statistics never waits for anything
// but its own UMMAs.  By induction over j every wait ends.  (The host only selects this kernel when the
// condition holds, and every wait here is bounded like all others in this library.)
#pragma once

#include "gemmrc_umma.cuh"

namespace beam {

template <int kStages>
struct LnResidentShape {
  static constexpr int kBM = 128;   // rows per CTA
  static constexpr int kBN = 256;   // UMMA N = tile width
  static constexpr int kBK = 64;
  static constexpr int kBRows = kBN / 2;  // rows of B one CTA of the pair loads
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = kBRows * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = 2 * kBN;
  static constexpr int kStoreBufBytes = 32 * 128;
  static constexpr int kBufsPerWarp = 2;
  static constexpr int kStagingBytes = 4 * kBufsPerWarp * kStoreBufBytes;
  static constexpr int kBarBytes = 512;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + kBarBytes + 1024;
  static constexpr int kThreads = 192;
  static_assert(kSmemBytes <= 232448, "exceeds the 227 KB of shared memory a CTA can opt in to");
  static_assert((2 * kStages + 4) * 8 + 16 <= kBarBytes, "barrier block too small");
};

// p.tickets: one int per 32 rows of the output (zeroed by the host before the launch).
// p.row_part: float2 (mean, M2) per row per 256-column tile.
template <int kStages>
__global__ void __launch_bounds__(192, 1) gemm_ln_resident_kernel(const __grid_constant__ GemmParams p) {
  using S = LnResidentShape<kStages>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t cta_rank = ptx::cluster_ctarank();
  const bool leader = cta_rank == 0;
  const int pairs = static_cast<int>(gridDim.x >> 1);
  const int first = static_cast<int>(blockIdx.x >> 1);
  const int tiles = p.m_tiles * p.n_tiles;
  const int my_tiles = first < tiles ? (tiles - first + pairs - 1) / pairs : 0;

  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t staging_base = smem_base + kStages * S::kStageBytes;
  const uint32_t bar_base = staging_base + S::kStagingBytes;
  auto smem_a = [&](int s) { return smem_base + s * S::kStageBytes; };
  auto smem_b = [&](int s) { return smem_base + s * S::kStageBytes + S::kABytes; };
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tmem_full_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto tmem_empty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(
      smem_gen + kStages * S::kStageBytes + S::kStagingBytes + 8 * (2 * kStages + 4));
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(tmem_full_bar(a), 1);
      ptx::mbar_init(tmem_empty_bar(a), 8);  // one arrive per epilogue warp of each CTA
    }
    *cta_abort = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&p.tm_a);
    ptx::prefetch_tensormap(&p.tm_b);
    ptx::prefetch_tensormap(&p.tm_c);
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
      uint32_t it = 0;
      bool alive = true;
      const uint64_t pol_a = ptx::l2_policy(p.hint_a);
      const uint64_t pol_b = ptx::l2_policy(p.hint_b);
      for (int j = 0; alive && j < my_tiles; ++j) {
        const int t = first + j * pairs;
        const int row_a = (t / p.n_tiles) * 256 + static_cast<int>(cta_rank) * S::kBM;
        const int row_b = (t % p.n_tiles) * S::kBN + static_cast<int>(cta_rank) * S::kBRows;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kStages;
          if (!bounded_wait(empty_bar(s), ((it / kStages) & 1u) ^ 1u, cta_abort, p.status, kFaultProducerWait)) {
            alive = false;
            break;
          }
          if (leader) ptx::mbar_arrive_expect_tx(full_bar(s), 2 * S::kStageBytes);
          const uint32_t lead_bar = ptx::mapa(full_bar(s), 0);
          ptx::tma_load_2d_pair_hint(smem_a(s), &p.tm_a, lead_bar, kb * S::kBK, row_a, pol_a);
          ptx::tma_load_2d_pair_hint(smem_b(s), &p.tm_b, lead_bar, kb * S::kBK, row_b, pol_b);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA)
    if (lane == 0 && leader) {
      const uint32_t idesc = ptx::umma_idesc_f16_f32(256, S::kBN);
      uint32_t stage = 0, parity = 0;
      const uint64_t a_desc0 = ptx::umma_desc_k_sw128(smem_a(0));
      const uint64_t b_desc0 = ptx::umma_desc_k_sw128(smem_b(0));
      constexpr uint64_t kDescStride = static_cast<uint64_t>(S::kStageBytes >> 4);
      bool alive = true;
      for (int j = 0; alive && j < my_tiles; ++j) {
        const uint32_t acc = static_cast<uint32_t>(j) & 1u;
        // the accumulator comes back only after the tile that used it last has been normalised and stored
        if (!bounded_wait(tmem_empty_bar(acc), ((static_cast<uint32_t>(j) >> 1) & 1u) ^ 1u, cta_abort, p.status,
                          kFaultMmaWaitAcc))
          break;
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * S::kBN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!bounded_wait(full_bar(stage), parity, cta_abort, p.status, kFaultMmaWaitFull)) {
            alive = false;
            break;
          }
          ptx::tc_fence_after();
          ptx::umma_f16_kblock<2>(d_tmem, a_desc0 + stage * kDescStride, b_desc0 + stage * kDescStride, idesc,
                                  kb > 0 ? 1u : 0u);
          ptx::umma_commit_pair_both(empty_bar(stage), 0x3);
          if (++stage == static_cast<uint32_t>(kStages)) {
            stage = 0;
            parity ^= 1u;
          }
        }
        if (alive) ptx::umma_commit_pair_both(tmem_full_bar(acc), 0x3);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const uint32_t quad = warp & 3u;
    const uint32_t lane_base = tmem_base + ((quad * 32u) << 16);
    const uint32_t lead_empty0 = ptx::mapa(tmem_empty_bar(0), 0);
    uint32_t store_count = 0;
    // first row of this warp's 32-row block inside tile t, and the block's ticket index
    auto block_row0 = [&](int t) {
      return (t / p.n_tiles) * 256 + static_cast<int>(cta_rank) * S::kBM + static_cast<int>(quad) * 32;
    };

    // First visit of a finished tile: statistics of this warp's rows over the tile's columns; the tile stays.
    auto publish_stats = [&](int j) {
      const int t = first + j * pairs;
      const int nt = t % p.n_tiles;
      const int row0 = block_row0(t);
      const int col0 = nt * S::kBN;
      const uint32_t taddr = lane_base + (static_cast<uint32_t>(j) & 1u) * S::kBN;
      ptx::tc_fence_after();
      float st_n = 0.f, st_mean = 0.f, st_m2 = 0.f;
      uint32_t v[2][32];
      ptx::tmem_ld_32x32(taddr, v[0]);
#pragma unroll
      for (int c = 0; c < S::kBN / 32; ++c) {
        ptx::tmem_ld_wait();
        if (c + 1 < S::kBN / 32) ptx::tmem_ld_32x32(taddr + (c + 1) * 32, v[(c + 1) & 1]);
        const int valid = min(32, p.n - (col0 + c * 32));
        if (valid > 0) {
          // two passes over the (up to) 32 values in registers, then a merge into the running (count, mean, M2)
          float sum = 0.f;
#pragma unroll
          for (int q = 0; q < 32; ++q) sum += (q < valid) ? __uint_as_float(v[c & 1][q]) : 0.f;
          const float mb = sum / static_cast<float>(valid);
          float m2b = 0.f;
#pragma unroll
          for (int q = 0; q < 32; ++q) {
            const float d = __uint_as_float(v[c & 1][q]) - mb;
            m2b += (q < valid) ? d * d : 0.f;
          }
          welford_merge(st_n, st_mean, st_m2, static_cast<float>(valid), mb, m2b);
        }
      }
      const int row = row0 + static_cast<int>(lane);
      if (row < p.m) p.row_part[static_cast<size_t>(row) * p.n_tiles + nt] = make_float2(st_mean, st_m2);
      __threadfence();
      __syncwarp();
      if (lane == 0 && row0 < p.m) atomicAdd(p.tickets + row0 / 32, 1);
    };

    // Second visit, once every tile of these rows has published: normalise from TMEM, store, release.
    auto normalise_and_release = [&](int j) {
      const int t = first + j * pairs;
      const int nt = t % p.n_tiles;
      const int row0 = block_row0(t);
      const int col0 = nt * S::kBN;
      const uint32_t acc = static_cast<uint32_t>(j) & 1u;
      const uint32_t taddr = lane_base + acc * S::kBN;
      __threadfence();  // acquire side of the ticket: the other tiles' statistics are visible below
      const int row = row0 + static_cast<int>(lane);
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
              welford_merge(n_acc, mean, m2, static_cast<float>(min(S::kBN, p.n - (t0 + i) * S::kBN)), pt[i].x,
                            pt[i].y);
        }
        rstd = rsqrtf(m2 / n_acc + p.eps);
      }
      ptx::tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < S::kBN; c += 64) {
        const int col = col0 + c;
        if (col >= p.n || row0 >= p.m) break;  // warp-uniform: nothing of this chunk (or block) exists
        uint32_t v0[32], v1[32], out[32];
        ptx::tmem_ld_32x32(taddr + c, v0);
        ptx::tmem_ld_32x32(taddr + c + 32, v1);
        // gamma and beta of the chunk's 64 columns: the same addresses in every lane (one broadcast each)
        uint4 g[8], b[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          g[i] = make_uint4(0, 0, 0, 0);
          b[i] = make_uint4(0, 0, 0, 0);
          if (col + 8 * i < p.n) {
            g[i] = __ldg(reinterpret_cast<const uint4*>(p.gamma + col + 8 * i));
            b[i] = __ldg(reinterpret_cast<const uint4*>(p.beta + col + 8 * i));
          }
        }
        ptx::tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 32; ++q) {  // output pair q = columns 2q, 2q + 1 of the chunk
          const uint32_t x0 = q < 16 ? v0[2 * q] : v1[2 * q - 32];
          const uint32_t x1 = q < 16 ? v0[2 * q + 1] : v1[2 * q - 31];
          const uint32_t gw = reinterpret_cast<const uint32_t*>(&g[q >> 2])[q & 3];
          const uint32_t bw = reinterpret_cast<const uint32_t*>(&b[q >> 2])[q & 3];
          const float2 gf = __half22float2(*reinterpret_cast<const __half2*>(&gw));
          const float2 bf = __half22float2(*reinterpret_cast<const __half2*>(&bw));
          out[q] = ptx::pack_half2((__uint_as_float(x0) - mean) * rstd * gf.x + bf.x,
                                   (__uint_as_float(x1) - mean) * rstd * gf.y + bf.y);
        }
        constexpr uint32_t kBufs = S::kBufsPerWarp;
        const uint32_t buf = staging_base + (quad * kBufs + (store_count % kBufs)) * S::kStoreBufBytes;
        if (store_count >= kBufs) {
          if (lane == 0) ptx::tma_store_wait_read<kBufs - 1>();
          __syncwarp();
        }
        const uint32_t row_addr = buf + lane * 128u;
#pragma unroll
        for (int jj = 0; jj < 8; ++jj)
          ptx::st_shared_v4(row_addr + ((static_cast<uint32_t>(jj) ^ (lane & 7u)) << 4), out[4 * jj], out[4 * jj + 1],
                            out[4 * jj + 2], out[4 * jj + 3]);
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          ptx::tma_store_2d(&p.tm_c, buf, col, row0);  // the copy engine clips rows >= M and columns >= N
          ptx::tma_store_commit();
        }
        ++store_count;
      }
      // every TMEM read of this tile is done: the issuer may overwrite the accumulator
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(lead_empty0 + 8u * acc);
    };

    int js = 0;  // next tile whose statistics are due
    int jn = 0;  // next tile to normalise (jn <= js <= jn + 2: two accumulators)
    uint64_t last_progress = ptx::globaltimer_ns();
    while (jn < my_tiles) {
      int action = 0;  // 1 publish statistics of tile js, 2 normalise tile jn, 3 give up
      if (lane == 0) {
        if (jn < js) {
          const int row0 = block_row0(first + jn * pairs);
          if (row0 >= p.m || ld_volatile_i32(p.tickets + row0 / 32) >= p.n_tiles) action = 2;
        }
        if (action == 0 && js < my_tiles && js - jn < 2 &&
            ptx::mbar_try_wait(tmem_full_bar(js & 1), (static_cast<uint32_t>(js) >> 1) & 1u))
          action = 1;
        if (action == 0) {
          if (!*cta_abort && ptx::globaltimer_ns() - last_progress > kWaitLimitNs) {
            *cta_abort = 1;
            if (p.status) atomicCAS(p.status, 0, static_cast<int>(kFaultReduceWait));
          }
          if (*cta_abort) action = 3;
        }
      }
      action = __shfl_sync(0xffffffffu, action, 0);
      if (action == 1) {
        publish_stats(js);
        ++js;
      } else if (action == 2) {
        normalise_and_release(jn);
        ++jn;
      } else if (action == 3) {
        break;
      } else {
        __nanosleep(64);
        continue;
      }
      last_progress = ptx::globaltimer_ns();
    }
  }

  if (warp >= 2 && lane == 0) ptx::tma_store_wait_all<0>();
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
