// Persistent, warp-specialised bf16 GEMM for sm_100a.
//
//   C[M,N] = alpha * op(A)[M,K] * op(B)[N,K]^T  (+ epilogue)
//
// * operands are staged by TMA (never multicast) into a 4-stage ring of 128B-swizzled
//   shared-memory tiles (128 x 64 for A, 256 x 64 for B),
// * one elected thread issues tcgen05.mma (M=128, N=256, K=16, kind::f16, bf16 in /
//   fp32 out) into one of two 256-column TMEM accumulators, so the epilogue of tile i
//   overlaps the main loop of tile i+1,
// * four epilogue warps read the accumulator with tcgen05.ld, apply the epilogue and
//   hand 32-row x 64-column slabs to TMA stores through a swizzled staging buffer.
//
// Either operand can be K-major (row-major [rows, K]) or MN-major (row-major
// [K, rows]); this covers y = x W^T, dx = dy W and dW = dy^T x without a transpose.
//
// Epilogues:
//   PLAIN   C = alpha*acc (+ bias[n]) (+ beta*Cin)
//   SWIGLU  B tile rows 0..127 come from B (gate weights), rows 128..255 from B2 (up
//           weights); writes H = silu(g)*u and, when asked, G and U.
//   STATS   C = bf16(alpha*acc) and per (row, n-tile) softmax partials (max, sum exp)
//           of the rounded values, for the fused linear + cross-entropy.
//   SYMM    M == N and the product is symmetric: only tiles that touch the upper
//           triangle are computed and every tile is also stored transposed
//           (C = alpha*acc + beta*Cin); used by the Newton-Schulz chain of Muon.
//
// Behavioural counterpart in the reference: cuBLAS through nn.Linear everywhere, the
// Triton X*X^T kernel of src/lmms_engine/utils/muon_utils.py:28-126 and Liger's
// chunked logits GEMM (src/lmms_engine/models/qwen2/qwen2_liger.py:142-143).
#include "common.cuh"

#include <stdio.h>

namespace b200 {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int kStages = 4;
constexpr int kATileBytes = BM * BK * 2;  // 16 KB
constexpr int kBTileBytes = BN * BK * 2;  // 32 KB
constexpr int kStageBytes = kATileBytes + kBTileBytes;
constexpr int kEpiWarps = 4;
constexpr int kEpiSlabBytes = 32 * 64 * 2;                       // 32 rows x 64 bf16
constexpr int kEpiBytes = kEpiWarps * 2 * kEpiSlabBytes;         // double-buffered, 32 KB
constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 1024 /*align*/ + 256 /*barriers*/;
constexpr int kThreads = 256;
constexpr int kTmemCols = 512;

enum Epilogue : int { EPI_PLAIN = 0, EPI_SWIGLU = 1, EPI_STATS = 2, EPI_SYMM = 3 };

struct GemmParams {
  int M, N, K;
  int a_mn_major, b_mn_major;
  int a_mn3d, b_mn3d;          // MN-major operand fetched with ONE 3-D TMA box (all 64-wide chunks at once)
  float alpha, beta;
  const __nv_bfloat16* bias;   // [N] or null (PLAIN)
  const __nv_bfloat16* cin;    // [M, ldcin] or null (PLAIN / SYMM)
  int ldcin;
  float2* stats;               // [M, n_tiles] (STATS)
  int n_tiles_n;               // tiles along N of the output problem
  int n_tiles_m;
  int store_gu;                // SWIGLU: also store gate / up pre-activations
  __nv_bfloat16* cmirror;      // SYMM: base of C for the transposed stores
  int ldc;
  // grouped (mixture-of-experts) modes; all tables live in device memory
  const int* tile_expert;      // grouped-M: expert of every 128-row tile of A / C (-1: unused tile)
  int up_row_offset;           // grouped SWIGLU: row of the first "up" weight inside an expert's [2I, K] block
  const int* expert_start;     // grouped-K: row range [start[e], start[e+1]) of expert e in A and B
  int group_k;                 // 1: C[e] = A[rows_e]^T B[rows_e] (both operands MN-major)
  int n_experts;
  int* status;
};

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }

// Map a linear tile index to (m_block, n_block).  Sixteen m-blocks share each sweep
// over N so that concurrently resident CTAs reuse the same B panels out of L2.
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& mb, int& nb) {
  constexpr int kGroup = 16;
  int per_group = kGroup * tiles_n;
  int g = t / per_group;
  int first_m = g * kGroup;
  int gsz = min(kGroup, tiles_m - first_m);
  int r = t - g * per_group;
  mb = first_m + r % gsz;
  nb = r / gsz;
}

template <int EPI>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmB2, const __grid_constant__ CUtensorMap tmC,
                 const __grid_constant__ CUtensorMap tmC2, const __grid_constant__ CUtensorMap tmC3,
                 const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_smem = smem + kStages * kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + kEpiBytes);
  uint64_t* full_bar = bars;                 // [kStages]
  uint64_t* empty_bar = bars + kStages;      // [kStages]
  uint64_t* tfull_bar = bars + 2 * kStages;  // [2]
  uint64_t* tempty_bar = tfull_bar + 2;      // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = p.n_tiles_m, tiles_n = p.n_tiles_n;
  const int n_tiles = tiles_m * tiles_n;
  const int n_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], kEpiWarps);
    }
    *abort_word = 0;
    fence_barrier_init();
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // SYMM skips tiles that lie entirely below the diagonal.
  auto tile_active = [&](int mb, int nb) -> bool {
    if (p.tile_expert != nullptr && p.tile_expert[mb] < 0) return false;
    if (EPI != EPI_SYMM) return true;
    return (nb + 1) * BN > mb * BM;
  };
  // grouped-K: tile t = (expert, m-block, n-block); K runs over the expert's own rows
  const int tiles_per_expert = tiles_m * tiles_n;
  const int total_tiles = p.group_k ? n_tiles * p.n_experts : n_tiles;
  auto decode = [&](int t, int& e, int& mb, int& nb, int& kb_lo, int& kb_n) {
    if (p.group_k) {
      e = t / tiles_per_expert;
      tile_coords(t - e * tiles_per_expert, tiles_m, tiles_n, mb, nb);
      const int r0 = p.expert_start[e], r1 = p.expert_start[e + 1];
      kb_lo = r0 / BK;
      kb_n = (r1 - r0) / BK;
    } else {
      tile_coords(t, tiles_m, tiles_n, mb, nb);
      e = p.tile_expert != nullptr ? p.tile_expert[mb] : 0;
      kb_lo = 0;
      kb_n = n_kb;
    }
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int ex, mb, nb, kb_lo, kb_n;
        decode(t, ex, mb, nb, kb_lo, kb_n);
        if (!tile_active(mb, nb)) continue;
        const int m0 = mb * BM;
        const int n0 = (EPI == EPI_SWIGLU) ? nb * (BN / 2) : nb * BN;
        const bool grouped_b = p.tile_expert != nullptr;  // B is a 3-D map indexed by expert
        for (int kb = 0; kb < kb_n; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_word)) { ok = false; break; }
          uint8_t* sa = smem + s * kStageBytes;
          uint8_t* sb = sa + kATileBytes;
          mbar_expect_tx(&full_bar[s], kStageBytes);
          const int k0 = (kb_lo + kb) * BK;
          if (!p.a_mn_major) {
            tma_load_2d(sa, &tmA, &full_bar[s], k0, m0);
          } else if (p.a_mn3d) {
            tma_load_3d(sa, &tmA, &full_bar[s], 0, k0, m0 / 64);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d(sa + c * 8192, &tmA, &full_bar[s], m0 + c * 64, k0);
          }
          if (EPI == EPI_SWIGLU && grouped_b) {
            tma_load_3d(sb, &tmB, &full_bar[s], k0, n0, ex);
            tma_load_3d(sb + 128 * 128, &tmB, &full_bar[s], k0, p.up_row_offset + n0, ex);
          } else if (EPI == EPI_SWIGLU) {
            // gate rows then up rows, 128 each (K-major only)
            tma_load_2d(sb, &tmB, &full_bar[s], k0, n0);
            tma_load_2d(sb + 128 * 128, &tmB2, &full_bar[s], k0, n0);
          } else if (grouped_b && !p.b_mn_major) {
            tma_load_3d(sb, &tmB, &full_bar[s], k0, n0, ex);
          } else if (grouped_b) {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_load_3d(sb + c * 8192, &tmB, &full_bar[s], n0 + c * 64, k0, ex);
          } else if (!p.b_mn_major) {
            tma_load_2d(sb, &tmB, &full_bar[s], k0, n0);
          } else if (p.b_mn3d) {
            tma_load_3d(sb, &tmB, &full_bar[s], 0, k0, n0 / 64);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_load_2d(sb + c * 8192, &tmB, &full_bar[s], n0 + c * 64, k0);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16_major(BM, BN, p.a_mn_major, p.b_mn_major);
      uint32_t it = 0, tl = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int ex, mb, nb, kb_lo, kb_n;
        decode(t, ex, mb, nb, kb_lo, kb_n);
        if (!tile_active(mb, nb)) continue;
        const int acc = tl & 1;
        const uint32_t acc_ph = (tl >> 1) & 1;
        if (!mbar_wait(&tempty_bar[acc], acc_ph ^ 1, abort_word)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kb_n; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(&full_bar[s], ph, abort_word)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * kStageBytes);
          const uint32_t sb = sa + kATileBytes;
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
            umma_bf16_ss(d_tmem, ad, bd, idesc, (kb | kk) != 0);
          }
          umma_commit(&empty_bar[s]);  // frees the stage once these MMAs retire
        }
        if (ok) umma_commit(&tfull_bar[acc]);
        ++tl;
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ epilogue (warps 4..7)
    const int q = warp - 4;  // TMEM lane quadrant == warp % 4
    uint8_t* slab0 = epi_smem + q * 2 * kEpiSlabBytes;
    uint32_t tl = 0;
    int buf = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      int ex, mb, nb, kb_lo, kb_n;
      decode(t, ex, mb, nb, kb_lo, kb_n);
      if (!tile_active(mb, nb)) continue;
      const bool empty_k = (kb_n == 0);  // grouped-K expert without rows: the product is zero
      const int acc = tl & 1;
      const uint32_t acc_ph = (tl >> 1) & 1;
      if (!mbar_wait(&tfull_bar[acc], acc_ph, abort_word)) { ok = false; break; }
      tc_fence_after();
      const int m0 = mb * BM;
      const int row = m0 + q * 32 + lane;  // global row owned by this thread
      const uint32_t t_acc = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);

      if (EPI == EPI_PLAIN || EPI == EPI_STATS || EPI == EPI_SYMM) {
        const int n0 = nb * BN;
        float run_max = -INFINITY, run_sum = 0.f;
#pragma unroll 1
        for (int c64 = 0; c64 < BN / 64; ++c64) {
          uint8_t* slab = slab0 + buf * kEpiSlabBytes;
          // make sure the TMA store that last read this slab has finished reading
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
            for (int j = 0; j < 32; ++j) v[j] = empty_k ? 0.f : __uint_as_float(r[j]) * p.alpha;
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
              // statistics of the values as they are stored (bf16-rounded)
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
            // swizzled staging: 16-byte chunk j of row r lands at chunk (j ^ (r & 7))
            uint8_t* srow = slab + lane * 128;
#pragma unroll
            for (int j4 = 0; j4 < 4; ++j4) {
              const int chunk = (h * 4 + j4) ^ (lane & 7);
              *reinterpret_cast<uint4*>(srow + chunk * 16) =
                  make_uint4(pk[j4 * 4], pk[j4 * 4 + 1], pk[j4 * 4 + 2], pk[j4 * 4 + 3]);
            }
            if (EPI == EPI_SYMM) {
              // Mirror C[col, row] = C[row, col] for the strictly-lower part.  For a fixed
              // column the 32 threads of the warp write 32 consecutive bf16 of one output row.
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
            if (p.group_k) tma_store_3d(&tmC, slab, n0 + c64 * 64, m0 + q * 32, ex);
            else tma_store_2d(&tmC, slab, n0 + c64 * 64, m0 + q * 32);
            tma_store_commit();
          }
          buf ^= 1;
        }
        if (EPI == EPI_STATS && row < p.M) p.stats[static_cast<size_t>(row) * tiles_n + nb] = make_float2(run_max, run_sum);
      } else {  // EPI_SWIGLU: accumulator cols [0,128) = gate, [128,256) = up
        const int n0 = nb * (BN / 2);
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
              // round gate/up to bf16 first so that H matches silu(G)*U of the stored tensors
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
      // all TMEM reads of this accumulator are done: hand it back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
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
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
  }
  return fn;
}

// The driver entry points used below need the primary context to be current on the calling
// thread.  Autograd runs backward on its own threads, where no runtime call may have bound
// it yet; cudaSetDevice on the current device does.
static void bind_context() {
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaSetDevice(dev);
}

// 2-D bf16 tensor map over a row-major [rows, cols] matrix with row stride `ld` elements.
static int make_map(CUtensorMap* m, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_cols,
                    uint32_t box_rows, bool swizzle128) {
  bind_context();
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr,
            "[b200 gemm] cuTensorMapEncodeTiled failed (%d): ptr=%p rows=%llu cols=%llu ld=%llu box=(%u,%u) swizzle=%d\n",
            static_cast<int>(r), ptr, static_cast<unsigned long long>(rows), static_cast<unsigned long long>(cols),
            static_cast<unsigned long long>(ld), box_cols, box_rows, static_cast<int>(swizzle128));
    return -2;
  }
  return 0;
}

// MN-major operand stored row-major [K, R] (R % 64 == 0) seen as {64, K, R/64}: one box
// {64, BK, chunks} lands in shared memory chunk-major, which is exactly the layout the
// MN-major UMMA descriptor walks (64-wide chunks BK*128 bytes apart).
static int make_map_mn3d(CUtensorMap* m, const void* ptr, uint64_t k_rows, uint64_t r_cols, uint64_t ld,
                         uint32_t chunks) {
  bind_context();
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[3] = {64, k_rows, r_cols / 64};
  cuuint64_t strides[2] = {ld * 2, 128};
  cuuint32_t box[3] = {64, static_cast<cuuint32_t>(BK), chunks};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "[b200 gemm] 3-D map failed (%d): k=%llu r=%llu ld=%llu\n", static_cast<int>(r),
            (unsigned long long)k_rows, (unsigned long long)r_cols, (unsigned long long)ld);
    return -2;
  }
  return 0;
}

// [E, R, C] bf16, contiguous: 3-D map (c, r, e) with box (box_c, box_r, 1)
static int make_map_e3(CUtensorMap* m, const void* ptr, uint64_t E, uint64_t R, uint64_t C, uint32_t box_c,
                       uint32_t box_r) {
  bind_context();
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[3] = {C, R, E};
  cuuint64_t strides[2] = {C * 2, R * C * 2};
  cuuint32_t box[3] = {box_c, box_r, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "[b200 gemm] expert map failed (%d): E=%llu R=%llu C=%llu\n", static_cast<int>(r),
            (unsigned long long)E, (unsigned long long)R, (unsigned long long)C);
    return -2;
  }
  return 0;
}

static int g_num_sms = 0;

template <int EPI>
static int launch(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tB2, const CUtensorMap& tC,
                  const CUtensorMap& tC2, const CUtensorMap& tC3, const GemmParams& p, int max_ctas,
                  cudaStream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return -3;
    attr_set = true;
  }
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  int ctas = g_num_sms;
  if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
  int tiles = p.n_tiles_m * p.n_tiles_n * (p.group_k ? p.n_experts : 1);
  if (tiles < ctas) ctas = tiles;
  if (ctas <= 0) return 0;
  gemm_bf16_kernel<EPI><<<ctas, kThreads, kSmemBytes, stream>>>(tA, tB, tB2, tC, tC2, tC3, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace b200

using namespace b200;

extern "C" {

// C = alpha * op(A) op(B)^T (+bias) (+beta*Cin).  lda/ldb/ldc/ldcin are row strides in
// elements of the matrices as they are stored.  All pointers must be 16-byte aligned
// and all row strides multiples of 8 elements.  Returns 0 on a successful launch.
int b200_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                   int a_mn_major, int b_mn_major, float alpha, float beta, const void* bias, const void* cin,
                   int ldcin, int symmetric, int max_ctas, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda | ldb | ldc) & 7) return -10;
  CUtensorMap tA, tB, tC;
  int rc = 0;
  int a3d = a_mn_major && (M % 64 == 0) && (lda >= M);
  int b3d = b_mn_major && (N % 64 == 0) && (ldb >= N);
  // the one-box fetch is an optimisation: if the driver rejects the 3-D view, use 2-D boxes
  if (a3d && make_map_mn3d(&tA, A, K, M, lda, BM / 64) != 0) a3d = 0;
  if (b3d && make_map_mn3d(&tB, B, K, N, ldb, BN / 64) != 0) b3d = 0;
  if (!a_mn_major) rc |= make_map(&tA, A, M, K, lda, BK, BM, true);
  else if (!a3d) rc |= make_map(&tA, A, K, M, lda, 64, BK, true);
  if (!b_mn_major) rc |= make_map(&tB, B, N, K, ldb, BK, BN, true);
  else if (!b3d) rc |= make_map(&tB, B, K, N, ldb, 64, BK, true);
  rc |= make_map(&tC, C, M, N, ldc, 64, 32, true);
  if (rc != 0) return rc;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.a_mn_major = a_mn_major; p.b_mn_major = b_mn_major;
  p.a_mn3d = a3d; p.b_mn3d = b3d;
  p.alpha = alpha; p.beta = beta;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.cin = static_cast<const __nv_bfloat16*>(cin);
  p.ldcin = ldcin;
  p.n_tiles_m = (M + BM - 1) / BM;
  p.n_tiles_n = (N + BN - 1) / BN;
  p.status = status;
  if (symmetric) {
    if (M != N) return -11;
    p.bias = nullptr;
    p.cmirror = static_cast<__nv_bfloat16*>(C);
    p.ldc = ldc;
    return launch<EPI_SYMM>(tA, tB, tB, tC, tC, tC, p, max_ctas, stream);
  }
  return launch<EPI_PLAIN>(tA, tB, tB, tC, tC, tC, p, max_ctas, stream);
}

// H = silu(X Wg^T) * (X Wu^T); optionally also writes G and U.  X [M,K], Wg/Wu [I,K].
int b200_gemm_swiglu_bf16(const void* X, const void* Wg, const void* Wu, void* H, void* G, void* U, int M, int I,
                          int K, int ldx, int ldw, int ldh, int store_gu, int* status, cudaStream_t stream) {
  if (M <= 0 || I <= 0 || K <= 0) return 0;
  if ((ldx | ldw | ldh) & 7) return -10;
  CUtensorMap tA, tB, tB2, tC, tC2, tC3;
  int rc = 0;
  rc |= make_map(&tA, X, M, K, ldx, BK, BM, true);
  rc |= make_map(&tB, Wg, I, K, ldw, BK, 128, true);
  rc |= make_map(&tB2, Wu, I, K, ldw, BK, 128, true);
  rc |= make_map(&tC, H, M, I, ldh, 64, 32, true);
  rc |= make_map(&tC2, store_gu ? G : H, M, I, ldh, 64, 32, true);
  rc |= make_map(&tC3, store_gu ? U : H, M, I, ldh, 64, 32, true);
  if (rc != 0) return rc;
  GemmParams p{};
  p.M = M; p.N = I; p.K = K;
  p.alpha = 1.f;
  p.n_tiles_m = (M + BM - 1) / BM;
  p.n_tiles_n = (I + 127) / 128;
  p.store_gu = store_gu;
  p.status = status;
  return launch<EPI_SWIGLU>(tA, tB, tB2, tC, tC2, tC3, p, 0, stream);
}

// logits = bf16(alpha * X W^T) plus per-(row, 256-column tile) softmax partials
// stats[row, tile] = (max, sum exp(v - max)) over the stored bf16 values.
int b200_gemm_stats_bf16(const void* X, const void* W, void* logits, void* stats, int M, int N, int K, int ldx,
                         int ldw, int ldc, float alpha, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((ldx | ldw | ldc) & 7) return -10;
  CUtensorMap tA, tB, tC;
  int rc = 0;
  rc |= make_map(&tA, X, M, K, ldx, BK, BM, true);
  rc |= make_map(&tB, W, N, K, ldw, BK, BN, true);
  rc |= make_map(&tC, logits, M, N, ldc, 64, 32, true);
  if (rc != 0) return rc;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.alpha = alpha;
  p.stats = static_cast<float2*>(stats);
  p.n_tiles_m = (M + BM - 1) / BM;
  p.n_tiles_n = (N + BN - 1) / BN;
  p.status = status;
  return launch<EPI_STATS>(tA, tB, tB, tC, tC, tC, p, 0, stream);
}

// ---- grouped (mixture-of-experts) products ------------------------------------------------
// A rows are grouped by expert in 128-row tiles (tile_expert[i] = expert of tile i, -1 for
// unused tiles); W is [E, N, K] (K-major) or [E, K, N] (w_mn_major).  C[rows, N] = A W[e]^T.
int b200_gemm_grouped_bf16(const void* A, const void* W, void* C, const void* tile_expert, int rows, int N, int K,
                           int E, int lda, int ldc, int w_mn_major, int* status, cudaStream_t stream) {
  if (rows <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda | ldc) & 7) return -10;
  CUtensorMap tA, tB, tC;
  int rc = make_map(&tA, A, rows, K, lda, BK, BM, true);
  if (!w_mn_major) rc |= make_map_e3(&tB, W, E, N, K, BK, BN);
  else rc |= make_map_e3(&tB, W, E, K, N, 64, BK);
  rc |= make_map(&tC, C, rows, N, ldc, 64, 32, true);
  if (rc != 0) return rc;
  GemmParams p{};
  p.M = rows; p.N = N; p.K = K;
  p.b_mn_major = w_mn_major;
  p.alpha = 1.f;
  p.n_tiles_m = (rows + BM - 1) / BM;
  p.n_tiles_n = (N + BN - 1) / BN;
  p.tile_expert = static_cast<const int*>(tile_expert);
  p.n_experts = E;
  p.status = status;
  return launch<EPI_PLAIN>(tA, tB, tB, tC, tC, tC, p, 0, stream);
}

// Grouped gate/up projection with SwiGLU: W is [E, 2I, K] with gate rows first.
// H[rows, I] = silu(g) * u; GU[rows, 2I] = [g | u] (kept for backward).
int b200_gemm_grouped_swiglu_bf16(const void* A, const void* W, void* H, void* GU, const void* tile_expert, int rows,
                                  int I, int K, int E, int lda, int* status, cudaStream_t stream) {
  if (rows <= 0 || I <= 0 || K <= 0) return 0;
  if ((lda & 7) || (I & 7)) return -10;
  CUtensorMap tA, tB, tC, tC2, tC3;
  int rc = make_map(&tA, A, rows, K, lda, BK, BM, true);
  rc |= make_map_e3(&tB, W, E, 2 * I, K, BK, 128);
  rc |= make_map(&tC, H, rows, I, I, 64, 32, true);
  rc |= make_map(&tC2, GU, rows, I, 2 * I, 64, 32, true);
  rc |= make_map(&tC3, static_cast<const __nv_bfloat16*>(GU) + I, rows, I, 2 * I, 64, 32, true);
  if (rc != 0) return rc;
  GemmParams p{};
  p.M = rows; p.N = I; p.K = K;
  p.alpha = 1.f;
  p.n_tiles_m = (rows + BM - 1) / BM;
  p.n_tiles_n = (I + 127) / 128;
  p.store_gu = 1;
  p.tile_expert = static_cast<const int*>(tile_expert);
  p.up_row_offset = I;
  p.n_experts = E;
  p.status = status;
  return launch<EPI_SWIGLU>(tA, tB, tB, tC, tC2, tC3, p, 0, stream);
}

// Per-expert weight gradient: dW[e] [M, N] = A[rows_e, M]^T B[rows_e, N], rows_e =
// [expert_start[e], expert_start[e+1]) (multiples of 128; padding rows must be zero in A or B).
int b200_gemm_grouped_wgrad_bf16(const void* A, const void* B, void* dW, const void* expert_start, int rows, int M,
                                 int N, int E, int lda, int ldb, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || E <= 0) return 0;
  if ((lda | ldb) & 7) return -10;
  CUtensorMap tA, tB, tC;
  int rc = make_map(&tA, A, rows, M, lda, 64, BK, true);
  rc |= make_map(&tB, B, rows, N, ldb, 64, BK, true);
  rc |= make_map_e3(&tC, dW, E, M, N, 64, 32);
  if (rc != 0) return rc;
  GemmParams p{};
  p.M = M; p.N = N; p.K = rows;
  p.a_mn_major = 1; p.b_mn_major = 1;
  p.alpha = 1.f;
  p.n_tiles_m = (M + BM - 1) / BM;
  p.n_tiles_n = (N + BN - 1) / BN;
  p.expert_start = static_cast<const int*>(expert_start);
  p.group_k = 1;
  p.n_experts = E;
  p.status = status;
  return launch<EPI_PLAIN>(tA, tB, tB, tC, tC, tC, p, 0, stream);
}

int b200_gemm_tile_n() { return BN; }

}  // extern "C"
