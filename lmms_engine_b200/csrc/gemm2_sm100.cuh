// Two-SM (CTA pair) variant of the persistent bf16 GEMM: one 256 x 256 output tile per
// pair, computed by tcgen05.mma.cta_group::2 (M = 256, N = 256, K = 16).
//
// Why a pair: a single SM that feeds a 128 x 256 tile reads 12 KB of operands from
// shared memory per K = 16 step while TMA writes another 12 KB into it, which is what
// keeps the one-CTA kernel near 83 % of the tensor pipe.  In a pair each SM stages only
// its own 128 rows of A and HALF of the B tile (128 of the 256 columns); the tensor cores
// of both SMs read both halves of B.  Per SM and K step that is 8 KB read + 8 KB written,
// and the ring holds six stages instead of four in the same shared memory.
//
// Roles per CTA (256 threads):
//   warp 0      TMA producer: loads this CTA's A rows and B half; the bytes of BOTH CTAs are
//               counted on the full barrier of the pair's leader (cluster rank 0), which alone
//               arrives on it (expecting twice a CTA's bytes): the second CTA makes no remote
//               arrive per stage, which would cost a cluster round trip per K block.
//               No load multicasts.
//   warp 1      MMA issuer, leader CTA only; stage release and accumulator hand-over go to
//               both CTAs with tcgen05.commit (multicast arrive on the same barrier offset).
//   warp 2      TMEM allocation (cta_group::2, 512 columns = two 256-column accumulators).
//   warps 4..7  epilogue of this CTA's 128 rows; they release the accumulator on the
//               leader's barrier (remote arrive from the second CTA).
//
// Every wait is bounded like in the one-CTA kernel; the pair re-converges on a cluster
// barrier before either CTA releases shared memory or TMEM.
#pragma once
#include "common.cuh"

namespace b200 {

constexpr int kStages2 = 6;
constexpr int kTile2M = 256;                           // rows of C per pair
constexpr int kHalfBytes = 128 * 64 * 2;               // one 128 x 64 bf16 operand tile
constexpr int kStage2Bytes = 2 * kHalfBytes;           // A rows + B half of one CTA
constexpr int kSmem2Bytes = kStages2 * kStage2Bytes + kEpiBytes + 1024 + 256;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the variable at `local` (a shared::cta address) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA loads of a CTA pair: the data lands in this CTA, the byte count on `bar_cluster`, which may be the
// peer's barrier.  No multicast: each CTA fetches its own operand tiles.
__device__ __forceinline__ void tma2_load_2d(uint32_t smem_dst, const CUtensorMap* m, uint32_t bar_cluster, int x,
                                             int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma2_load_3d(uint32_t smem_dst, const CUtensorMap* m, uint32_t bar_cluster, int x,
                                             int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tmem2_alloc(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem2_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem2_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma2_bf16_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at this shared-memory offset in BOTH CTAs once the MMAs issued so far have retired.
__device__ __forceinline__ void umma2_commit_both(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(mask)
      : "memory");
}

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmB2, const __grid_constant__ CUtensorMap tmC,
                  const __grid_constant__ CUtensorMap tmC2, const __grid_constant__ CUtensorMap tmC3,
                  const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  // the dynamic shared window starts at the same offset in both CTAs, so the aligned tiles do too
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* epi_smem = smem + kStages2 * kStage2Bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + kEpiBytes);
  uint64_t* full_bar = bars;                   // [kStages2]  used in the leader: its arrival + bytes of both CTAs
  uint64_t* empty_bar = bars + kStages2;       // [kStages2]  one per CTA, raised by the leader's commit
  uint64_t* tfull_bar = bars + 2 * kStages2;   // [2]         one per CTA, raised by the leader's commit
  uint64_t* tempty_bar = tfull_bar + 2;        // [2]         used in the leader: epilogue warps of both CTAs
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();      // 0 = leader
  const int pair = static_cast<int>(blockIdx.x) >> 1;
  const int n_pairs = static_cast<int>(gridDim.x) >> 1;
  const int tiles_m = p.n_tiles_m, tiles_n = p.n_tiles_n;
  const int n_tiles = tiles_m * tiles_n;
  const int n_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages2; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], 2 * kEpiWarps);
    }
    *abort_word = 0;
    fence_barrier_init();
  }
  if (warp == 2) {
    tmem2_alloc(tmem_slot, kTmemCols);
    tmem2_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto tile_active = [&](int mb, int nb) -> bool {
    if (EPI != EPI_SYMM) return true;
    return (nb + 1) * BN > mb * kTile2M;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t it = 0;
      bool ok = true;
      for (int t = pair; t < n_tiles && ok; t += n_pairs) {
        int mb, nb;
        tile_coords(t, tiles_m, tiles_n, mb, nb, p.group_m);
        if (!tile_active(mb, nb)) continue;
        const int m0 = mb * kTile2M + static_cast<int>(cta) * 128;
        // SWIGLU: the leader stages gate rows, the second CTA the matching up rows
        const int n0 = (EPI == EPI_SWIGLU) ? nb * 128 : nb * BN + static_cast<int>(cta) * 128;
        for (int kb = 0; kb < n_kb; ++kb, ++it) {
          const int s = it % kStages2;
          const uint32_t ph = (it / kStages2) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_word)) { ok = false; break; }
          const uint32_t sa = smem_u32(smem + s * kStage2Bytes);
          const uint32_t sb = sa + kHalfBytes;
          const uint32_t fb = map_to_cta(smem_u32(&full_bar[s]), 0);
          if (cta == 0) mbar_expect_tx(&full_bar[s], 2 * kStage2Bytes);
          const int k0 = kb * BK;
          if (!p.a_mn_major) {
            tma2_load_2d(sa, &tmA, fb, k0, m0);
          } else if (p.a_mn3d) {
            tma2_load_3d(sa, &tmA, fb, 0, k0, m0 / 64);
          } else {
#pragma unroll
            for (int c = 0; c < 2; ++c) tma2_load_2d(sa + c * 8192, &tmA, fb, m0 + c * 64, k0);
          }
          if (EPI == EPI_SWIGLU) {
            tma2_load_2d(sb, cta == 0 ? &tmB : &tmB2, fb, k0, n0);
          } else if (!p.b_mn_major) {
            tma2_load_2d(sb, &tmB, fb, k0, n0);
          } else if (p.b_mn3d) {
            tma2_load_3d(sb, &tmB, fb, 0, k0, n0 / 64);
          } else {
#pragma unroll
            for (int c = 0; c < 2; ++c) tma2_load_2d(sb + c * 8192, &tmB, fb, n0 + c * 64, k0);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    if (lane == 0 && cta == 0) {
      const uint32_t idesc = umma_idesc_bf16_major(kTile2M, BN, p.a_mn_major, p.b_mn_major);
      uint32_t it = 0, tl = 0;
      bool ok = true;
      for (int t = pair; t < n_tiles && ok; t += n_pairs) {
        int mb, nb;
        tile_coords(t, tiles_m, tiles_n, mb, nb, p.group_m);
        if (!tile_active(mb, nb)) continue;
        const int acc = tl & 1;
        const uint32_t acc_ph = (tl >> 1) & 1;
        if (!mbar_wait(&tempty_bar[acc], acc_ph ^ 1, abort_word)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < n_kb; ++kb, ++it) {
          const int s = it % kStages2;
          const uint32_t ph = (it / kStages2) & 1;
          if (!mbar_wait(&full_bar[s], ph, abort_word)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * kStage2Bytes);
          const uint32_t sb = sa + kHalfBytes;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            uint64_t ad, bd;
            if (!p.a_mn_major) {
              ad = umma_desc_sw128(sa + kk * 32);
            } else {
              ad = umma_desc_sw128(sa + kk * 2048);
              ad = (ad & ~(uint64_t(0x3FFF) << 16)) | (uint64_t(8192 >> 4) << 16);
            }
            if (!p.b_mn_major) {
              bd = umma_desc_sw128(sb + kk * 32);
            } else {
              bd = umma_desc_sw128(sb + kk * 2048);
              bd = (bd & ~(uint64_t(0x3FFF) << 16)) | (uint64_t(8192 >> 4) << 16);
            }
            umma2_bf16_ss(d_tmem, ad, bd, idesc, (kb | kk) != 0);
          }
          umma2_commit_both(&empty_bar[s]);
        }
        if (ok) umma2_commit_both(&tfull_bar[acc]);
        ++tl;
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ epilogue (warps 4..7, both CTAs)
    const int q = warp - 4;
    uint8_t* slab0 = epi_smem + q * 2 * kEpiSlabBytes;
    uint32_t tl = 0;
    int buf = 0;
    bool ok = true;
    for (int t = pair; t < n_tiles && ok; t += n_pairs) {
      int mb, nb;
      tile_coords(t, tiles_m, tiles_n, mb, nb, p.group_m);
      if (!tile_active(mb, nb)) continue;
      const int acc = tl & 1;
      const uint32_t acc_ph = (tl >> 1) & 1;
      if (!mbar_wait(&tfull_bar[acc], acc_ph, abort_word)) { ok = false; break; }
      tc_fence_after();
      const int m0 = mb * kTile2M + static_cast<int>(cta) * 128;
      const int row = m0 + q * 32 + lane;
      const uint32_t t_acc = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);

      if (EPI == EPI_PLAIN || EPI == EPI_STATS || EPI == EPI_SYMM) {
        const int n0 = nb * BN;
        float run_max = -INFINITY, run_sum = 0.f;
#pragma unroll 1
        for (int c64 = 0; c64 < BN / 64; ++c64) {
          uint8_t* slab = slab0 + buf * kEpiSlabBytes;
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(t_acc + c64 * 64 + h * 32, r);
            tmem_ld_wait();
            const int col0 = n0 + c64 * 64 + h * 32;
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
            if (EPI == EPI_PLAIN && p.bias != nullptr) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) v[j] += __bfloat162float(p.bias[col0 + j]);
            }
            if ((EPI == EPI_PLAIN || EPI == EPI_SYMM) && p.cin != nullptr && row < p.M) {
              const __nv_bfloat16* crow = p.cin + static_cast<size_t>(row) * p.ldcin + col0;
              if (col0 + 32 <= p.N) {
                const uint4* c4 = reinterpret_cast<const uint4*>(crow);
#pragma unroll
                for (int j4 = 0; j4 < 4; ++j4) {
                  uint4 u = c4[j4];
                  float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z),
                         f3 = unpack_bf16x2(u.w);
                  v[j4 * 8 + 0] += p.beta * f0.x; v[j4 * 8 + 1] += p.beta * f0.y;
                  v[j4 * 8 + 2] += p.beta * f1.x; v[j4 * 8 + 3] += p.beta * f1.y;
                  v[j4 * 8 + 4] += p.beta * f2.x; v[j4 * 8 + 5] += p.beta * f2.y;
                  v[j4 * 8 + 6] += p.beta * f3.x; v[j4 * 8 + 7] += p.beta * f3.y;
                }
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (col0 + j < p.N) v[j] += p.beta * __bfloat162float(crow[j]);
              }
            }
            uint32_t pk[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) pk[j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
            if (EPI == EPI_STATS) {
              float cmax = -INFINITY;
              float w[32];
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                float2 f = unpack_bf16x2(pk[j]);
                w[2 * j] = (col0 + 2 * j < p.N) ? f.x : -INFINITY;
                w[2 * j + 1] = (col0 + 2 * j + 1 < p.N) ? f.y : -INFINITY;
                cmax = fmaxf(cmax, fmaxf(w[2 * j], w[2 * j + 1]));
              }
              const float new_max = fmaxf(run_max, cmax);
              if (new_max > -INFINITY) {
                float s = 0.f;
#pragma unroll
                for (int j = 0; j < 32; ++j) s += __expf(w[j] - new_max);
                run_sum = run_sum * __expf(run_max - new_max) + s;
                run_max = new_max;
              }
            }
            uint8_t* srow = slab + lane * 128;
#pragma unroll
            for (int j4 = 0; j4 < 4; ++j4) {
              const int chunk = (h * 4 + j4) ^ (lane & 7);
              *reinterpret_cast<uint4*>(srow + chunk * 16) =
                  make_uint4(pk[j4 * 4], pk[j4 * 4 + 1], pk[j4 * 4 + 2], pk[j4 * 4 + 3]);
            }
            if (EPI == EPI_SYMM) {
              if (row < p.N) {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  const int orow = col0 + j;
                  if (orow > row && orow < p.M) {
                    const uint32_t w2 = pk[j >> 1];
                    const unsigned short bits = (j & 1) ? static_cast<unsigned short>(w2 >> 16)
                                                        : static_cast<unsigned short>(w2 & 0xFFFFu);
                    reinterpret_cast<unsigned short*>(p.cmirror)[static_cast<size_t>(orow) * p.ldc + row] = bits;
                  }
                }
              }
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmC, slab, n0 + c64 * 64, m0 + q * 32);
            tma_store_commit();
          }
          buf ^= 1;
        }
        if (EPI == EPI_STATS && row < p.M) p.stats[static_cast<size_t>(row) * tiles_n + nb] = make_float2(run_max, run_sum);
      } else {  // EPI_SWIGLU: accumulator cols [0,128) = gate, [128,256) = up
        const int n0 = nb * 128;
#pragma unroll 1
        for (int c64 = 0; c64 < 2; ++c64) {
          uint32_t pg[2][16], pu[2][16], phh[2][16];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t rg[32], ru[32];
            tmem_ld_32x32b_x32(t_acc + c64 * 64 + h * 32, rg);
            tmem_ld_32x32b_x32(t_acc + 128 + c64 * 64 + h * 32, ru);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              pg[h][j] = pack_bf16x2(__uint_as_float(rg[2 * j]) * p.alpha, __uint_as_float(rg[2 * j + 1]) * p.alpha);
              pu[h][j] = pack_bf16x2(__uint_as_float(ru[2 * j]) * p.alpha, __uint_as_float(ru[2 * j + 1]) * p.alpha);
              float2 g = unpack_bf16x2(pg[h][j]), u = unpack_bf16x2(pu[h][j]);
              phh[h][j] = pack_bf16x2(silu_f(g.x) * u.x, silu_f(g.y) * u.y);
            }
          }
          const int n_out = p.store_gu ? 3 : 1;
#pragma unroll 1
          for (int o = 0; o < n_out; ++o) {
            uint8_t* slab = slab0 + buf * kEpiSlabBytes;
            if (lane == 0) tma_store_wait_read<1>();
            __syncwarp();
            uint8_t* srow = slab + lane * 128;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
#pragma unroll
              for (int j4 = 0; j4 < 4; ++j4) {
                const int chunk = (h * 4 + j4) ^ (lane & 7);
                uint4 val;
                if (o == 0) val = make_uint4(phh[h][j4 * 4], phh[h][j4 * 4 + 1], phh[h][j4 * 4 + 2], phh[h][j4 * 4 + 3]);
                else if (o == 1) val = make_uint4(pg[h][j4 * 4], pg[h][j4 * 4 + 1], pg[h][j4 * 4 + 2], pg[h][j4 * 4 + 3]);
                else val = make_uint4(pu[h][j4 * 4], pu[h][j4 * 4 + 1], pu[h][j4 * 4 + 2], pu[h][j4 * 4 + 3]);
                *reinterpret_cast<uint4*>(srow + chunk * 16) = val;
              }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              const CUtensorMap* tm = (o == 0) ? &tmC : (o == 1 ? &tmC2 : &tmC3);
              tma_store_2d(tm, slab, n0 + c64 * 64, m0 + q * 32);
              tma_store_commit();
            }
            buf ^= 1;
          }
        }
      }
      // this warp has read its part of the accumulator: count it on the leader's barrier
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[acc]), 0));
      ++tl;
    }
    if (lane == 0) tma_store_wait_all<0>();
  }

  // ------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_word) {
    // give copies still in flight time to land before shared memory is released
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    if (threadIdx.x == 0 && p.status != nullptr) atomicExch(p.status, kStatusBarrierTimeout);
  }
  // neither CTA leaves while the other may still signal one of its barriers or feed its tensor cores
  cluster_sync_all();
  if (warp == 2) {
    tc_fence_after();
    tmem2_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace b200
