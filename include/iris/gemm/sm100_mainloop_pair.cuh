// Two-SM variant of the GEMM main loop: a cluster of two CTAs computes one 256 x BN output tile
// with tcgen05.mma.cta_group::2. Each CTA stages its own 128 rows of A and HALF of the B tile,
// so a stage is 32 KB instead of 48 KB (six stages fit instead of four, and B is read from L2
// once per pair instead of once per CTA); the leader CTA (cluster rank 0) issues the MMAs for
// both, each CTA's accumulator rows live in its own TMEM, and each CTA runs its own epilogue.
//
// Wiring (L = leader, P = peer):
//   full[s]        lives in L; both CTAs' TMA loads complete_tx on it (the .cta_group::2 load form
//                  with the leader's barrier address; no multicast anywhere); L's producer arms it
//                  with the byte count of both CTAs.
//   empty[s]       one per CTA; L's MMA thread releases both with one multicast tcgen05.commit.
//   tmem_full[b]   one per CTA, signalled by a multicast commit; tmem_empty[b] lives in L and
//                  counts the epilogue warps of both CTAs (the peer arrives remotely).
// Policies are the ones of sm100_mainloop.cuh; tile() is asked for PAIR tiles (its m index counts
// 256-row tiles) and every other hook sees 128-row tile indices (2 * pair_m + cluster rank).
// Only the row-major epilogue path is provided.
#pragma once
#include "sm100_mainloop.cuh"

namespace iris {
namespace gemm {

template <int BN_, bool kBKMajor_, int kStages_>
struct PairConfig {
  static constexpr int BN = BN_;
  static constexpr int kHalfN = BN_ / 2;
  static constexpr bool kBKMajor = kBKMajor_;
  static constexpr int kStages = kStages_;
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBoxes = kBKMajor_ ? 1 : (kHalfN + 63) / 64;
  static constexpr int kBBytes = kBKMajor_ ? kHalfN * kBK * 2 : kBBoxes * 8192;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kAccCols = 256;
  static constexpr int kTmemCols = 512;
  static constexpr int kEpiBytes = kEpiWarps * 2048;
  static constexpr int kSmemBytes = 1024 + kStages_ * kStageBytes + kEpiBytes + 256;
  static_assert(BN_ % 64 == 0 && BN_ <= 256, "pair tiles are 64, 128, 192 or 256 wide");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};

IRIS_HD uint32_t make_idesc_pair(int n, bool bf16, bool b_mn_major) {
  uint32_t fmt = bf16 ? 1u : 0u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(256 >> 4) << 24);
}

template <class Cfg, class Policy>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1) gemm_pair_kernel(const __grid_constant__ Policy pol) {
  extern __shared__ uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = ptx::cluster_ctarank();
  const bool leader = cta == 0;
  const Shape sh = pol.shape();

  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* stage_base = smem;
  uint8_t* epi_base = smem + Cfg::kStages * Cfg::kStageBytes;
  uint64_t* bars = (uint64_t*)(epi_base + Cfg::kEpiBytes);
  Pipeline pipe{bars, bars + Cfg::kStages, bars + 2 * Cfg::kStages, bars + 2 * Cfg::kStages + 2};
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * Cfg::kStages + 4);

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      ptx::mbar_init(&pipe.full[s], 1);
      ptx::mbar_init(&pipe.empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(&pipe.tmem_full[b], 1);
      ptx::mbar_init(&pipe.tmem_empty[b], 2 * kEpiWarps);
    }
    ptx::fence_mbar_init();
    ptx::fence_proxy_async();
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(tmem_slot, Cfg::kTmemCols);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();          // both CTAs' barriers exist before anyone signals remotely
  ptx::tc_fence_after();
  const uint32_t tmem_base = *(volatile uint32_t*)tmem_slot;

  const int num_tiles = pol.num_tiles();                  // pair tiles
  const int k_blocks = (sh.K + kBK - 1) / kBK;
  const int first = blockIdx.x >> 1, step = pol.gemm_ctas() >> 1;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) ptx::prefetch_tmap(pol.b_map());
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    typename Policy::State st;
    for (int t = first; t < num_tiles && ok; t += step) {
      int tmp, tn;
      pol.tile(t, tmp, tn);
      const int tm = 2 * tmp + (int)cta;
      for (int kb = 0; kb < k_blocks; ++kb) {
        ASource as;
        as.bn0 = tn * Cfg::BN;
        if (!pol.a_source(st, tm, kb, as)) { ok = false; break; }
        if (!ptx::mbar_wait<true>(&pipe.empty[s], ph ^ 1, kPipeTimeoutNs)) { pol.fail(kTimeoutPipeline); ok = false; break; }
        if (lane == 0) {
          uint8_t* sa = stage_base + s * Cfg::kStageBytes;
          uint8_t* sb = sa + Cfg::kABytes;
          if (leader) ptx::mbar_expect_tx(&pipe.full[s], 2 * Cfg::kStageBytes);
          ptx::tma_load_2d_pair(sa, as.map, &pipe.full[s], as.x, as.y);
          const int n0 = as.bn0 + (int)cta * Cfg::kHalfN;
          if constexpr (Cfg::kBKMajor) {
            ptx::tma_load_2d_pair(sb, pol.b_map(), &pipe.full[s], as.bk, n0);
          } else {
#pragma unroll
            for (int j = 0; j < Cfg::kBBoxes; ++j)
              ptx::tma_load_2d_pair(sb + j * 8192, pol.b_map(), &pipe.full[s], n0 + j * 64, as.bk);
          }
        }
        __syncwarp();
        if (++s == Cfg::kStages) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader only)
    if (leader) {
      const uint32_t idesc = make_idesc_pair(Cfg::BN, pol.is_bf16(), !Cfg::kBKMajor);
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      bool ok = true;
      for (int t = first; t < num_tiles && ok; t += step, ++it) {
        const int buf = it & 1;
        const uint32_t acc_ph = (it >> 1) & 1;
        if (!ptx::mbar_wait<true>(&pipe.tmem_empty[buf], acc_ph ^ 1, kPipeTimeoutNs)) { pol.fail(kTimeoutPipeline); break; }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * Cfg::kAccCols;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!ptx::mbar_wait<true>(&pipe.full[s], ph, kPipeTimeoutNs)) { pol.fail(kTimeoutPipeline); ok = false; break; }
          ptx::tc_fence_after();
          if (lane == 0) {
            const uint32_t sa = ptx::smem_u32(stage_base + s * Cfg::kStageBytes);
            const uint32_t sb = sa + Cfg::kABytes;
#pragma unroll
            for (int k = 0; k < kBK / kUmmaK; ++k) {
              uint64_t ad = desc_kmajor(sa + k * (kUmmaK * 2));
              uint64_t bd = Cfg::kBKMajor ? desc_kmajor(sb + k * (kUmmaK * 2)) : desc_mnmajor(sb + k * (kUmmaK * 128));
              ptx::mma_f16_pair(d_tmem, ad, bd, idesc, (kb | k) != 0);
            }
            ptx::mma_commit_pair(&pipe.empty[s], 3);
            if (kb == k_blocks - 1) ptx::mma_commit_pair(&pipe.tmem_full[buf], 3);
          }
          __syncwarp();
          if (++s == Cfg::kStages) { s = 0; ph ^= 1; }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (both CTAs)
    const int quarter = warp & 3;
    uint8_t* my_epi = epi_base + (warp - 2) * 2048;
    const bool bf16 = pol.is_bf16();
    const bool has_bias = pol.has_bias();
    typename Policy::State est;
    int it = 0;
    for (int t = first; t < num_tiles; t += step, ++it) {
      const int buf = it & 1;
      const uint32_t acc_ph = (it >> 1) & 1;
      int tmp, tn;
      pol.tile(t, tmp, tn);
      const int tm = 2 * tmp + (int)cta;
      const bool live = ptx::mbar_wait<true>(&pipe.tmem_full[buf], acc_ph, kPipeTimeoutNs);
      if (!live) {
        pol.fail(kTimeoutPipeline);
        break;
      }
      ptx::tc_fence_after();
      pol.begin_tile(est, tm, tn, my_epi);
      const uint32_t t_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * Cfg::kAccCols;
      const int row0 = pol.row_origin(est, tm) + quarter * 32;
      const float rb = has_bias ? pol.row_bias(row0 + lane) : 0.f;
#pragma unroll 1
      for (int c = 0; c < Cfg::BN / 32; ++c) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(t_addr + c * 32, r);
        ptx::tmem_ld_wait();
        if (c == Cfg::BN / 32 - 1) {
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if (leader) ptx::mbar_arrive(&pipe.tmem_empty[buf]);
            else ptx::mbar_arrive_cluster(&pipe.tmem_empty[buf], 0);
          }
        }
        const int col0 = tn * Cfg::BN + c * 32;
        uint32_t packed[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          float a = __uint_as_float(r[2 * j]) + rb, b = __uint_as_float(r[2 * j + 1]) + rb;
          if (has_bias) { a += pol.col_bias(col0 + 2 * j); b += pol.col_bias(col0 + 2 * j + 1); }
          if (bf16) {
            __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
            packed[j] = *(uint32_t*)&h;
          } else {
            __half2 h = __floats2half2_rn(a, b);
            packed[j] = *(uint32_t*)&h;
          }
        }
        const int sw = (lane >> 1) & 3;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 v = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
          *(uint4*)(my_epi + lane * 64 + ((j ^ sw) * 16)) = v;
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int rr = i * 8 + (lane >> 2), cc = lane & 3;
          uint4 v = *(uint4*)(my_epi + rr * 64 + ((cc ^ ((rr >> 1) & 3)) * 16));
          pol.store16(est, row0 + rr, col0 + cc * 8, v);
        }
        __syncwarp();
      }
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();          // the peer's smem and barriers stay alive until the leader is done
  ptx::tc_fence_after();
  if (warp == 1) ptx::tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
}

}  // namespace gemm
}  // namespace iris
