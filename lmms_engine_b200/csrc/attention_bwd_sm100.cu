// Varlen flash-attention backward for sm_100a, split into two tcgen05 kernels so that no
// gradient needs a cross-CTA reduction (no atomics, no fp32 staging buffer):
//
//   dkdv kernel  one CTA per (document, 128-key block, KV head); loops over the query heads of
//                the group and 64-row query tiles in the transposed formulation
//                S^T = K Q^T, dP^T = V dO^T, dV += P^T dO, dK += dS^T Q.
//   dq kernel    one CTA per (document, 128-query block, query head); loops over 64-key tiles:
//                S = Q K^T, dP = dO V^T, dQ += dS K.
//
// Both keep two TMEM buffers for the score tiles and two shared-memory buffers for the
// probability tiles, so the two score products of tile i+1 are issued while the eight softmax
// warps still work on tile i; accumulators stay in TMEM for the whole loop.  Recomputing S and
// dP in the second kernel costs two extra products per tile pair and buys a reduction-free dQ.
//
// Counterpart in the reference: flash_attn_varlen_func's backward
// (src/lmms_engine/kernels/attention.py:39-51).
#include "common.cuh"

#include <stdio.h>

namespace b200 {

constexpr int kKeys = 128;   // key block of the dkdv kernel / query block of the dq kernel
constexpr int kTile = 64;    // inner tile (queries in dkdv, keys in dq)
constexpr int DP = 128;      // padded head dim (smaller head dims are zero-filled by TMA)
constexpr float kLog2eB = 1.4426950408889634f;

struct BwdP {
  const int* cu_q;
  const int* cu_k;
  int n_docs;
  int Hq, Hkv, D;
  float scale, scale_log2;
  int causal, window_left;
  const float* lse;      // [Hq, Tq]
  const float* delta;    // [Hq, Tq]
  __nv_bfloat16* dQ;     // [Tq, Hq, D]
  __nv_bfloat16* dK;     // [Tk, Hkv, D]
  __nv_bfloat16* dV;
  long lddq, lddk, lddv;
  int Tq, Tk;
  int* status;
};

// Shared memory.  The inner tiles (Q_i, dO_i in the dkdv kernel; K_j, V_j in the dq kernel) go through kStages stages:
// a stage is released only when the accumulating products that read it have retired, and the refill then pays the whole
// TMA latency, so with S stages a tile's period is about (latency + MMA time) / (S - 1).  The dq kernel needs no P
// buffers and spends that room on a fourth stage.
struct Smem {
  static constexpr int kStages = 3;
  static constexpr int kBig = kKeys * DP * 2;     // 32 KB: a 128-row tile
  static constexpr int kSmall = kTile * DP * 2;   // 16 KB: a 64-row tile
  static constexpr int kProb = kKeys * kTile * 2; // 16 KB: a 128 x 64 probability tile
  // dkdv: K, V | kStages x (Q_i, dO_i) | 2 x P^T | 2 x dS^T
  static constexpr int kA0 = 0;
  static constexpr int kA1 = kBig;
  static constexpr int kStage = 2 * kBig;
  static constexpr int kP = kStage + kStages * 2 * kSmall;
  static constexpr int kDS = kP + 2 * kProb;
  static constexpr int kBars = kDS + 2 * kProb;
  static constexpr int kTotal = kBars + 256 + 1024;
};

struct SmemQ {
  static constexpr int kStages = 4;
  // dq: Q, dO | kStages x (K_j, V_j) | 2 x dS
  static constexpr int kStage = 2 * Smem::kBig;
  static constexpr int kDS = kStage + kStages * 2 * Smem::kSmall;
  static constexpr int kBars = kDS + 2 * Smem::kProb;
  static constexpr int kTotal = kBars + 256 + 1024;
};
static_assert(Smem::kTotal <= 227 * 1024 && SmemQ::kTotal <= 227 * 1024, "shared memory of the backward kernels");

__device__ __forceinline__ uint64_t desc_lbo(uint32_t addr, uint32_t lbo_bytes) {
  uint64_t d = umma_desc_sw128(addr);
  return (d & ~(uint64_t(0x3FFF) << 16)) | (uint64_t(lbo_bytes >> 4) << 16);
}

__device__ __forceinline__ bool find_work(const int* cu_a, const int* cu_b, int n_docs, int block, int item,
                                          int* work, int total_a, int total_b, int* status) {
  // work: doc, a0 (offset of the 128-block inside the doc), len_a, len_b, a_start, b_start
  int acc = 0;
  for (int d = 0; d < n_docs; ++d) {
    const int la = cu_a[d + 1] - cu_a[d];
    const int nb = (la + block - 1) / block;
    if (item < acc + nb) {
      work[0] = d;
      work[1] = (item - acc) * block;
      work[2] = la;
      work[3] = cu_b[d + 1] - cu_b[d];
      work[4] = cu_a[d];
      work[5] = cu_b[d];
      if (!doc_in_bounds(work[4], work[2], total_a, status) || !doc_in_bounds(work[5], work[3], total_b, status)) {
        work[0] = -1;
        return false;
      }
      return true;
    }
    acc += nb;
  }
  return false;
}

// ============================================================================ dK / dV
__global__ void __launch_bounds__(384, 1)
attn_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO, const BwdP p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Smem::kBars);
  constexpr int S = Smem::kStages;
  uint64_t* kv_full = bars;                  // 1
  uint64_t* q_full = bars + 1;               // S   a stage holds Q_i and dO_i
  uint64_t* q_empty = bars + 1 + S;          // S   the products that read a stage retired
  uint64_t* s_full = bars + 1 + 2 * S;       // 2   S^T and dP^T of a buffer are in TMEM
  uint64_t* ds_full = bars + 3 + 2 * S;      // 2   P^T / dS^T of a buffer are in shared memory
  uint64_t* pd_free = bars + 5 + 2 * S;      // 2   the dV / dK products that read a smem buffer retired
  uint64_t* all_done = bars + 7 + 2 * S;     // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8 + 2 * S);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* work = reinterpret_cast<int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    work[0] = -1;
    find_work(p.cu_k, p.cu_q, p.n_docs, kKeys, blockIdx.x, work, p.Tk, p.Tq, p.status);
    mbar_init(kv_full, 1);
    for (int i = 0; i < S; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&ds_full[i], 8);
      mbar_init(&pd_free[i], 1);
    }
    mbar_init(all_done, 1);
    *abort_word = 0;
    fence_barrier_init();
  }
  __syncthreads();
  if (work[0] < 0) return;
  if (warp == 2) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tm_ST = tmem_base;         // 2 x 64 columns
  const uint32_t tm_dPT = tmem_base + 128;  // 2 x 64 columns
  const uint32_t tm_dV = tmem_base + 256;   // 128 columns
  const uint32_t tm_dK = tmem_base + 384;   // 128 columns

  // here "a" is the key side: work = doc, k0, len_k, len_q, k_start, q_start
  const int k0 = work[1], len_k = work[2], len_q = work[3], k_start = work[4], q_start = work[5];
  const int kvh = blockIdx.y;
  const int group = p.Hq / p.Hkv;
  const int offset = len_k - len_q;
  int q_lo = 0;
  if (p.causal) q_lo = max(0, k0 - offset);
  int q_hi = len_q;
  if (p.window_left >= 0) q_hi = min(len_q, k0 + kKeys - 1 - offset + p.window_left + 1);
  const int ib_lo = q_lo / kTile;
  const int ib_hi = (max(q_hi, 0) + kTile - 1) / kTile;
  const int n_qt = max(ib_hi - ib_lo, 0);
  const int n_iter = n_qt * group;

  if (warp == 0) {
    if (lane == 0 && n_iter > 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmdO);
      mbar_expect_tx(kv_full, 2 * Smem::kBig);
#pragma unroll
      for (int c = 0; c < DP / 64; ++c) {
        tma_load_3d(smem + Smem::kA0 + c * (kKeys * 128), &tmK, kv_full, c * 64, kvh, k_start + k0);
        tma_load_3d(smem + Smem::kA1 + c * (kKeys * 128), &tmV, kv_full, c * 64, kvh, k_start + k0);
      }
      bool ok = true;
      for (int it = 0; it < n_iter && ok; ++it) {
        const int s = it % S;
        const uint32_t ph = (it / S) & 1;
        const int hq = kvh * group + it / n_qt;
        const int qrow = q_start + (ib_lo + it % n_qt) * kTile;
        if (!mbar_wait(&q_empty[s], ph ^ 1, abort_word)) { ok = false; break; }
        mbar_expect_tx(&q_full[s], 2 * Smem::kSmall);
        uint8_t* dst = smem + Smem::kStage + s * 2 * Smem::kSmall;
#pragma unroll
        for (int c = 0; c < DP / 64; ++c) {
          tma_load_3d(dst + c * (kTile * 128), &tmQ, &q_full[s], c * 64, hq, qrow);
          tma_load_3d(dst + Smem::kSmall + c * (kTile * 128), &tmdO, &q_full[s], c * 64, hq, qrow);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_iter > 0) {
      const uint32_t idesc_s = umma_idesc_bf16(kKeys, kTile);                    // M = keys, N = q, K = d
      const uint32_t sK = smem_u32(smem + Smem::kA0), sV = smem_u32(smem + Smem::kA1);
      bool ok = mbar_wait(kv_full, 0, abort_word);
      auto issue_scores = [&](int it) -> bool {
        const int s = it & 1;            // TMEM buffer of the scores
        const int stg = it % S;          // shared-memory stage of Q_i / dO_i
        if (!mbar_wait(&q_full[stg], (it / S) & 1, abort_word)) return false;
        tc_fence_after();
        const uint32_t sQ = smem_u32(smem + Smem::kStage + stg * 2 * Smem::kSmall);
        const uint32_t sdO = sQ + Smem::kSmall;
#pragma unroll
        for (int kk = 0; kk < DP / 16; ++kk) {
          const uint32_t offA = (kk / 4) * (kKeys * 128) + (kk % 4) * 32;
          const uint32_t offB = (kk / 4) * (kTile * 128) + (kk % 4) * 32;
          umma_bf16_ss(tm_ST + s * 64, umma_desc_sw128(sK + offA), umma_desc_sw128(sQ + offB), idesc_s, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < DP / 16; ++kk) {
          const uint32_t offA = (kk / 4) * (kKeys * 128) + (kk % 4) * 32;
          const uint32_t offB = (kk / 4) * (kTile * 128) + (kk % 4) * 32;
          umma_bf16_ss(tm_dPT + s * 64, umma_desc_sw128(sV + offA), umma_desc_sw128(sdO + offB), idesc_s, kk != 0);
        }
        umma_commit(&s_full[s]);
        return true;
      };
      // the score products of tile it reuse the TMEM buffers of tile it - 2: wait until the softmax warps have read them
      for (int it = 0; it < n_iter && ok; ++it) {
        if (it >= 2 && !mbar_wait(&ds_full[it & 1], ((it - 2) >> 1) & 1, abort_word)) { ok = false; break; }
        if (!issue_scores(it)) { ok = false; break; }
      }
    }
  } else if (warp == 3) {
    // A second issuing thread for the accumulating products: a thread blocks while it issues and pays every commit,
    // fence and barrier hand-off in sequence, so one thread for both kinds left the tensor pipe idle for about a
    // third of a tile's time.
    if (lane == 0 && n_iter > 0) {
      const uint32_t idesc_acc = umma_idesc_bf16_major(kKeys, DP, 0, 1);          // M = keys, N = d, K = q
      bool ok = true;
      for (int it = 0; it < n_iter && ok; ++it) {
        const int s = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(&ds_full[s], ph, abort_word)) { ok = false; break; }
        tc_fence_after();
        const int stg = it % S;
        const uint32_t sQ = smem_u32(smem + Smem::kStage + stg * 2 * Smem::kSmall);
        const uint32_t sdO = sQ + Smem::kSmall;
        const uint32_t sPT = smem_u32(smem + Smem::kP + s * Smem::kProb);
        const uint32_t sDST = smem_u32(smem + Smem::kDS + s * Smem::kProb);
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk) {
          // A = P^T / dS^T [128 keys x 64 q] K-major; B = dO_i / Q_i [q, d] MN-major (64-wide d chunks)
          umma_bf16_ss(tm_dV, umma_desc_sw128(sPT + kk * 32), desc_lbo(sdO + kk * 2048, kTile * 128), idesc_acc,
                       (it | kk) != 0);
          umma_bf16_ss(tm_dK, umma_desc_sw128(sDST + kk * 32), desc_lbo(sQ + kk * 2048, kTile * 128), idesc_acc,
                       (it | kk) != 0);
        }
        umma_commit(&q_empty[stg]);
        umma_commit(&pd_free[s]);
      }
      if (ok) umma_commit(all_done);
    }
  } else if (warp >= 4) {
    const int q = warp & 3;               // TMEM lane quadrant
    const int half = (warp - 4) >> 2;     // which 32 query columns of the 64-wide tile
    const int r = q * 32 + lane;          // key row of this thread
    const int kj = k0 + r;
    const uint32_t lane_sel = static_cast<uint32_t>(q * 32) << 16;
    bool ok = true;
    for (int it = 0; it < n_iter && ok; ++it) {
      const int s = it & 1;
      const uint32_t ph = (it >> 1) & 1;
      const int hq = kvh * group + it / n_qt;
      const int qb0 = (ib_lo + it % n_qt) * kTile + half * 32;
      // the 32 queries of this warp's columns: lane l fetches the statistics of query l before the wait (one coalesced
      // load each, latency hidden behind the score products); the loop below reads them by shuffle
      const bool q_ok = qb0 + lane < len_q;
      const size_t stat = static_cast<size_t>(hq) * p.Tq + q_start + qb0 + lane;
      const float lane_lse = q_ok ? p.lse[stat] * kLog2eB : 0.f;
      const float lane_dl = q_ok ? p.delta[stat] * p.scale : 0.f;  // pre-scaled: dS = P * (dP * scale - delta * scale)
      // visibility of the warp's 32 keys x 32 queries as a whole: interior tiles skip the per-element tests
      const int key_first = k0 + q * 32, key_last = key_first + 31;
      bool full = (qb0 + 31 < len_q) && (key_last < len_k);
      bool none = (qb0 >= len_q) || (key_first >= len_k);
      if (p.causal) {
        full = full && (key_last <= qb0 + offset);
        none = none || (key_first > qb0 + 31 + offset);
      }
      if (p.window_left >= 0) {
        full = full && (key_first >= qb0 + 31 + offset - p.window_left);
        none = none || (key_last < qb0 + offset - p.window_left);
      }
      if (!mbar_wait(&s_full[s], ph, abort_word)) { ok = false; break; }
      tc_fence_after();
      uint32_t ppk[16], dpk[16];
      if (none) {
#pragma unroll
        for (int j = 0; j < 16; ++j) ppk[j] = dpk[j] = 0u;
      } else {
        uint32_t rs[32], rd[32];
        tmem_ld_32x32b_x32(tm_ST + s * 64 + lane_sel + half * 32, rs);
        tmem_ld_32x32b_x32(tm_dPT + s * 64 + lane_sel + half * 32, rd);
        tmem_ld_wait();
        if (full) {
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            float pv[2], dsv[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const float l2 = __shfl_sync(0xffffffffu, lane_lse, j + e);
              const float dl = __shfl_sync(0xffffffffu, lane_dl, j + e);
              pv[e] = fast_exp2(fmaf(__uint_as_float(rs[j + e]), p.scale_log2, -l2));
              dsv[e] = pv[e] * fmaf(__uint_as_float(rd[j + e]), p.scale, -dl);
            }
            ppk[j / 2] = pack_bf16x2(pv[0], pv[1]);
            dpk[j / 2] = pack_bf16x2(dsv[0], dsv[1]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            float pv[2], dsv[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int qi = qb0 + j + e;
              const float l2 = __shfl_sync(0xffffffffu, lane_lse, j + e);
              const float dl = __shfl_sync(0xffffffffu, lane_dl, j + e);
              bool vis = (qi < len_q) && (kj < len_k);
              if (p.causal) vis = vis && (kj <= qi + offset);
              if (p.window_left >= 0) vis = vis && (kj >= qi + offset - p.window_left);
              float pe = 0.f, dse = 0.f;
              if (vis) {
                pe = fast_exp2(fmaf(__uint_as_float(rs[j + e]), p.scale_log2, -l2));
                dse = pe * fmaf(__uint_as_float(rd[j + e]), p.scale, -dl);
              }
              pv[e] = pe;
              dsv[e] = dse;
            }
            ppk[j / 2] = pack_bf16x2(pv[0], pv[1]);
            dpk[j / 2] = pack_bf16x2(dsv[0], dsv[1]);
          }
        }
      }
      if (it >= 2 && !mbar_wait(&pd_free[s], ph ^ 1, abort_word)) { ok = false; break; }
      uint8_t* rp = smem + Smem::kP + s * Smem::kProb + r * 128;
      uint8_t* rdst = smem + Smem::kDS + s * Smem::kProb + r * 128;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int chunk = (half * 4 + c) ^ (r & 7);
        *reinterpret_cast<uint4*>(rp + chunk * 16) = make_uint4(ppk[c * 4], ppk[c * 4 + 1], ppk[c * 4 + 2], ppk[c * 4 + 3]);
        *reinterpret_cast<uint4*>(rdst + chunk * 16) = make_uint4(dpk[c * 4], dpk[c * 4 + 1], dpk[c * 4 + 2], dpk[c * 4 + 3]);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_full[s]);
    }
    // ---- epilogue: this thread writes 64 of the 128 d columns of its key row ----------
    if (ok && n_iter > 0) ok = mbar_wait(all_done, 0, abort_word);
    tc_fence_after();
    const bool row_ok = ok && (kj < len_k);
    __nv_bfloat16* dkrow = p.dK + static_cast<size_t>(k_start + kj) * p.lddk + static_cast<size_t>(kvh) * p.D;
    __nv_bfloat16* dvrow = p.dV + static_cast<size_t>(k_start + kj) * p.lddv + static_cast<size_t>(kvh) * p.D;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int col0 = half * 64 + c * 32;
      uint32_t rk[32], rv[32];
      if (n_iter > 0 && ok) {
        tmem_ld_32x32b_x32(tm_dK + lane_sel + col0, rk);
        tmem_ld_32x32b_x32(tm_dV + lane_sel + col0, rv);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) rk[j] = rv[j] = 0u;
      }
      if (row_ok) {
#pragma unroll
        for (int j8 = 0; j8 < 4; ++j8) {
          const int col = col0 + j8 * 8;
          if (col < p.D) {
            uint4 a, b;
            a.x = pack_bf16x2(__uint_as_float(rk[j8 * 8 + 0]), __uint_as_float(rk[j8 * 8 + 1]));
            a.y = pack_bf16x2(__uint_as_float(rk[j8 * 8 + 2]), __uint_as_float(rk[j8 * 8 + 3]));
            a.z = pack_bf16x2(__uint_as_float(rk[j8 * 8 + 4]), __uint_as_float(rk[j8 * 8 + 5]));
            a.w = pack_bf16x2(__uint_as_float(rk[j8 * 8 + 6]), __uint_as_float(rk[j8 * 8 + 7]));
            b.x = pack_bf16x2(__uint_as_float(rv[j8 * 8 + 0]), __uint_as_float(rv[j8 * 8 + 1]));
            b.y = pack_bf16x2(__uint_as_float(rv[j8 * 8 + 2]), __uint_as_float(rv[j8 * 8 + 3]));
            b.z = pack_bf16x2(__uint_as_float(rv[j8 * 8 + 4]), __uint_as_float(rv[j8 * 8 + 5]));
            b.w = pack_bf16x2(__uint_as_float(rv[j8 * 8 + 6]), __uint_as_float(rv[j8 * 8 + 7]));
            *reinterpret_cast<uint4*>(dkrow + col) = a;
            *reinterpret_cast<uint4*>(dvrow + col) = b;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_word) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    if (threadIdx.x == 0 && p.status != nullptr) atomicExch(p.status, kStatusBarrierTimeout);
  }
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ============================================================================ dQ
__global__ void __launch_bounds__(384, 1)
attn_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO, const BwdP p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SmemQ::kBars);
  constexpr int S = SmemQ::kStages;
  uint64_t* q_full = bars;                   // 1   Q and dO
  uint64_t* kv_full = bars + 1;              // S   a stage holds K_j and V_j
  uint64_t* kv_empty = bars + 1 + S;         // S
  uint64_t* s_full = bars + 1 + 2 * S;       // 2
  uint64_t* ds_full = bars + 3 + 2 * S;      // 2
  uint64_t* ds_free = bars + 5 + 2 * S;      // 2
  uint64_t* all_done = bars + 7 + 2 * S;     // 1
  uint64_t* a_ready = bars + 8 + 2 * S;      // 1   Q and dO sit in TMEM (written by the eight softmax warps)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9 + 2 * S);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* work = reinterpret_cast<int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    // heavy (late, long-context) query blocks first
    int total = 0;
    for (int d = 0; d < p.n_docs; ++d) total += (p.cu_q[d + 1] - p.cu_q[d] + kKeys - 1) / kKeys;
    work[0] = -1;
    const int item = total - 1 - static_cast<int>(blockIdx.x);
    if (item >= 0) find_work(p.cu_q, p.cu_k, p.n_docs, kKeys, item, work, p.Tq, p.Tk, p.status);
    mbar_init(q_full, 1);
    for (int i = 0; i < S; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&ds_full[i], 8);
      mbar_init(&ds_free[i], 1);
    }
    mbar_init(all_done, 1);
    mbar_init(a_ready, 8);
    *abort_word = 0;
    fence_barrier_init();
  }
  __syncthreads();
  if (work[0] < 0) return;
  if (warp == 2) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tm_S = tmem_base;          // 2 x 64
  const uint32_t tm_dP = tmem_base + 128;   // 2 x 64
  const uint32_t tm_dQ = tmem_base + 256;   // 128
  // The A operands of the score products, Q and dO, are the same for every key tile.  From shared memory an
  // M = 128, K = 16 instruction pays about 64 cycles for its 4 KB A slice whatever its N, which halves the rate of the
  // 64-column score products; from TMEM (two bf16 per 32-bit column, row m in lane m) it does not.
  const uint32_t tm_Q = tmem_base + 384;    // 64 columns: Q  [128 rows x 128 d] as bf16 pairs
  const uint32_t tm_dO = tmem_base + 448;   // 64 columns: dO

  const int q0 = work[1], len_q = work[2], len_k = work[3], q_start = work[4], k_start = work[5];
  const int head = blockIdx.y;
  const int kvh = head / (p.Hq / p.Hkv);
  const int offset = len_k - len_q;
  int k_hi = len_k;
  if (p.causal) k_hi = min(len_k, q0 + kKeys + offset);
  int k_lo = 0;
  if (p.window_left >= 0) k_lo = max(0, q0 + offset - p.window_left);
  const int jb_lo = k_lo / kTile;
  const int jb_hi = (max(k_hi, 0) + kTile - 1) / kTile;
  const int n_iter = max(jb_hi - jb_lo, 0);

  if (warp == 0) {
    if (lane == 0 && n_iter > 0) {
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, 2 * Smem::kBig);
#pragma unroll
      for (int c = 0; c < DP / 64; ++c) {
        tma_load_3d(smem + Smem::kA0 + c * (kKeys * 128), &tmQ, q_full, c * 64, head, q_start + q0);
        tma_load_3d(smem + Smem::kA1 + c * (kKeys * 128), &tmdO, q_full, c * 64, head, q_start + q0);
      }
      bool ok = true;
      for (int it = 0; it < n_iter && ok; ++it) {
        const int s = it % S;
        const uint32_t ph = (it / S) & 1;
        const int krow = k_start + (jb_lo + it) * kTile;
        if (!mbar_wait(&kv_empty[s], ph ^ 1, abort_word)) { ok = false; break; }
        mbar_expect_tx(&kv_full[s], 2 * Smem::kSmall);
        uint8_t* dst = smem + SmemQ::kStage + s * 2 * Smem::kSmall;
#pragma unroll
        for (int c = 0; c < DP / 64; ++c) {
          tma_load_3d(dst + c * (kTile * 128), &tmK, &kv_full[s], c * 64, kvh, krow);
          tma_load_3d(dst + Smem::kSmall + c * (kTile * 128), &tmV, &kv_full[s], c * 64, kvh, krow);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_iter > 0) {
      const uint32_t idesc_s = umma_idesc_bf16(kKeys, kTile);                 // M = q, N = keys, K = d
      const uint32_t sQ = smem_u32(smem + Smem::kA0), sdO = smem_u32(smem + Smem::kA1);
      bool ok = mbar_wait(a_ready, 0, abort_word);
      tc_fence_after();
      auto issue_scores = [&](int it) -> bool {
        const int s = it & 1;            // TMEM buffer of the scores
        const int stg = it % S;          // shared-memory stage of K_j / V_j
        if (!mbar_wait(&kv_full[stg], (it / S) & 1, abort_word)) return false;
        tc_fence_after();
        const uint32_t sK = smem_u32(smem + SmemQ::kStage + stg * 2 * Smem::kSmall);
        const uint32_t sV = sK + Smem::kSmall;
#pragma unroll
        for (int kk = 0; kk < DP / 16; ++kk) {
          const uint32_t offB = (kk / 4) * (kTile * 128) + (kk % 4) * 32;
          umma_bf16_ts(tm_S + s * 64, tm_Q + kk * 8, umma_desc_sw128(sK + offB), idesc_s, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < DP / 16; ++kk) {
          const uint32_t offB = (kk / 4) * (kTile * 128) + (kk % 4) * 32;
          umma_bf16_ts(tm_dP + s * 64, tm_dO + kk * 8, umma_desc_sw128(sV + offB), idesc_s, kk != 0);
        }
        umma_commit(&s_full[s]);
        return true;
      };
      for (int it = 0; it < n_iter && ok; ++it) {
        if (it >= 2 && !mbar_wait(&ds_full[it & 1], ((it - 2) >> 1) & 1, abort_word)) { ok = false; break; }
        if (!issue_scores(it)) { ok = false; break; }
      }
    }
  } else if (warp == 3) {
    // second issuing thread: the dQ products (see the dK / dV kernel)
    if (lane == 0 && n_iter > 0) {
      const uint32_t idesc_dq = umma_idesc_bf16_major(kKeys, DP, 0, 1);        // M = q, N = d, K = keys
      bool ok = true;
      for (int it = 0; it < n_iter && ok; ++it) {
        const int s = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(&ds_full[s], ph, abort_word)) { ok = false; break; }
        tc_fence_after();
        const int stg = it % S;
        const uint32_t sK = smem_u32(smem + SmemQ::kStage + stg * 2 * Smem::kSmall);
        const uint32_t sDS = smem_u32(smem + SmemQ::kDS + s * Smem::kProb);
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk) {
          // A = dS [128 q x 64 keys] K-major; B = K_j [keys, d] MN-major (64-wide d chunks 8 KB apart)
          umma_bf16_ss(tm_dQ, umma_desc_sw128(sDS + kk * 32), desc_lbo(sK + kk * 2048, kTile * 128), idesc_dq,
                       (it | kk) != 0);
        }
        umma_commit(&kv_empty[stg]);
        umma_commit(&ds_free[s]);
      }
      if (ok) umma_commit(all_done);
    }
  } else if (warp >= 4) {
    const int q = warp & 3;
    const int half = (warp - 4) >> 2;
    const int r = q * 32 + lane;   // query row of this thread
    const int qi = q0 + r;
    const uint32_t lane_sel = static_cast<uint32_t>(q * 32) << 16;
    const bool row_valid = qi < len_q;
    // ---- Q (warps 4-7) and dO (warps 8-11) from shared memory (128-byte swizzle) into TMEM, one row per thread ----
    if (n_iter > 0) {
      bool okq = mbar_wait(q_full, 0, abort_word);
      if (okq) {
        const uint8_t* src = smem + (half == 0 ? Smem::kA0 : Smem::kA1);
        const uint32_t dst = (half == 0 ? tm_Q : tm_dO) + lane_sel;
#pragma unroll
        for (int c64 = 0; c64 < DP / 64; ++c64) {       // two 64-column (128-byte) chunks of the row
#pragma unroll
          for (int h16 = 0; h16 < 2; ++h16) {           // 16 TMEM columns (64 bytes of the row) per store
            uint32_t wds[16];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const int chunk = (h16 * 4 + c) ^ (r & 7);
              const uint4 v = *reinterpret_cast<const uint4*>(src + c64 * (kKeys * 128) + r * 128 + chunk * 16);
              wds[c * 4 + 0] = v.x; wds[c * 4 + 1] = v.y; wds[c * 4 + 2] = v.z; wds[c * 4 + 3] = v.w;
            }
            tmem_st_32x32b_x16(dst + c64 * 32 + h16 * 16, wds);
          }
        }
        tmem_st_wait();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(a_ready);
    }
    const float my_lse = row_valid ? p.lse[static_cast<size_t>(head) * p.Tq + q_start + qi] * kLog2eB : 0.f;
    const float my_delta = row_valid ? p.delta[static_cast<size_t>(head) * p.Tq + q_start + qi] * p.scale : 0.f;  // pre-scaled
    bool ok = true;
    for (int it = 0; it < n_iter && ok; ++it) {
      const int s = it & 1;
      const uint32_t ph = (it >> 1) & 1;
      const int kb0 = (jb_lo + it) * kTile + half * 32;
      // visibility of the warp's 32 queries x 32 keys as a whole: interior tiles skip the per-element tests,
      // tiles above the diagonal skip the exponentials
      const int row_first = q0 + q * 32, row_last = row_first + 31;
      bool full = (row_last < len_q) && (kb0 + 31 < len_k);
      bool none = (row_first >= len_q) || (kb0 >= len_k);
      if (p.causal) {
        full = full && (kb0 + 31 <= row_first + offset);
        none = none || (kb0 > row_last + offset);
      }
      if (p.window_left >= 0) {
        full = full && (kb0 >= row_last + offset - p.window_left);
        none = none || (kb0 + 31 < row_first + offset - p.window_left);
      }
      if (!mbar_wait(&s_full[s], ph, abort_word)) { ok = false; break; }
      tc_fence_after();
      uint32_t dpk[16];
      if (none) {
#pragma unroll
        for (int j = 0; j < 16; ++j) dpk[j] = 0u;
      } else {
        uint32_t rs[32], rd[32];
        tmem_ld_32x32b_x32(tm_S + s * 64 + lane_sel + half * 32, rs);
        tmem_ld_32x32b_x32(tm_dP + s * 64 + lane_sel + half * 32, rd);
        tmem_ld_wait();
        if (full) {
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            float dsv[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const float pe = fast_exp2(fmaf(__uint_as_float(rs[j + e]), p.scale_log2, -my_lse));
              dsv[e] = pe * fmaf(__uint_as_float(rd[j + e]), p.scale, -my_delta);
            }
            dpk[j / 2] = pack_bf16x2(dsv[0], dsv[1]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            float dsv[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int kj = kb0 + j + e;
              bool vis = row_valid && (kj < len_k);
              if (p.causal) vis = vis && (kj <= qi + offset);
              if (p.window_left >= 0) vis = vis && (kj >= qi + offset - p.window_left);
              float dse = 0.f;
              if (vis) {
                const float pe = fast_exp2(fmaf(__uint_as_float(rs[j + e]), p.scale_log2, -my_lse));
                dse = pe * fmaf(__uint_as_float(rd[j + e]), p.scale, -my_delta);
              }
              dsv[e] = dse;
            }
            dpk[j / 2] = pack_bf16x2(dsv[0], dsv[1]);
          }
        }
      }
      if (it >= 2 && !mbar_wait(&ds_free[s], ph ^ 1, abort_word)) { ok = false; break; }
      uint8_t* rdst = smem + SmemQ::kDS + s * Smem::kProb + r * 128;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int chunk = (half * 4 + c) ^ (r & 7);
        *reinterpret_cast<uint4*>(rdst + chunk * 16) = make_uint4(dpk[c * 4], dpk[c * 4 + 1], dpk[c * 4 + 2], dpk[c * 4 + 3]);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_full[s]);
    }
    if (ok && n_iter > 0) ok = mbar_wait(all_done, 0, abort_word);
    tc_fence_after();
    __nv_bfloat16* dqrow = p.dQ + static_cast<size_t>(q_start + qi) * p.lddq + static_cast<size_t>(head) * p.D;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int col0 = half * 64 + c * 32;
      uint32_t rq[32];
      if (n_iter > 0 && ok) {
        tmem_ld_32x32b_x32(tm_dQ + lane_sel + col0, rq);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) rq[j] = 0u;
      }
      if (row_valid && ok) {
#pragma unroll
        for (int j8 = 0; j8 < 4; ++j8) {
          const int col = col0 + j8 * 8;
          if (col < p.D) {
            uint4 a;
            a.x = pack_bf16x2(__uint_as_float(rq[j8 * 8 + 0]), __uint_as_float(rq[j8 * 8 + 1]));
            a.y = pack_bf16x2(__uint_as_float(rq[j8 * 8 + 2]), __uint_as_float(rq[j8 * 8 + 3]));
            a.z = pack_bf16x2(__uint_as_float(rq[j8 * 8 + 4]), __uint_as_float(rq[j8 * 8 + 5]));
            a.w = pack_bf16x2(__uint_as_float(rq[j8 * 8 + 6]), __uint_as_float(rq[j8 * 8 + 7]));
            *reinterpret_cast<uint4*>(dqrow + col) = a;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_word) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    if (threadIdx.x == 0 && p.status != nullptr) atomicExch(p.status, kStatusBarrierTimeout);
  }
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[h, t] = sum_d O[t,h,d] * dO[t,h,d]
__global__ void attn_delta2_kernel(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO,
                                   float* __restrict__ delta, int T, int H, int D, long ldo, long lddo) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const long total = static_cast<long>(T) * H;
  for (long idx = blockIdx.x * static_cast<long>(wpb) + (threadIdx.x >> 5); idx < total;
       idx += static_cast<long>(gridDim.x) * wpb) {
    const long t = idx / H;
    const int h = idx - t * H;
    const __nv_bfloat16* o = O + t * ldo + static_cast<long>(h) * D;
    const __nv_bfloat16* g = dO + t * lddo + static_cast<long>(h) * D;
    float acc = 0.f;
    for (int d = lane * 2; d < D; d += 64) {
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(o + d));
      const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(g + d));
      acc += a.x * b.x + a.y * b.y;
    }
    acc = warp_sum(acc);
    if (lane == 0) delta[static_cast<size_t>(h) * T + t] = acc;
  }
}

typedef CUresult (*EncodeTiledFn2)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int map3(CUtensorMap* m, const void* ptr, uint64_t T, uint64_t H, uint64_t D, uint64_t ld, uint32_t rows) {
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaSetDevice(dev);  // driver calls need the context bound on this thread
  static EncodeTiledFn2 fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return -1;
    fn = reinterpret_cast<EncodeTiledFn2>(sym);
  }
  cuuint64_t dims[3] = {D, H, T};
  cuuint64_t strides[2] = {D * 2, ld * 2};
  cuuint32_t box[3] = {64, 1, rows};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_attn_bwd_v2(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                                const void* lse, void* delta, void* dq, void* dk, void* dv, const void* cu_q,
                                const void* cu_k, int n_docs, int Tq, int Tk, int Hq, int Hkv, int D, long ldq,
                                long ldk, long ldv, long ldo, long lddo, long lddq, long lddk, long lddv, float scale,
                                int causal, int window_left, int* status, cudaStream_t st) {
  if (Tq <= 0 || n_docs <= 0) return 0;
  if (D % 8 || D > 128 || Hq % Hkv) return -10;
  CUtensorMap tq64, tk128, tv128, tdo64, tq128, tk64, tv64, tdo128;
  int rc = map3(&tq64, q, Tq, Hq, D, ldq, kTile) | map3(&tdo64, d_o, Tq, Hq, D, lddo, kTile) |
           map3(&tk128, k, Tk, Hkv, D, ldk, kKeys) | map3(&tv128, v, Tk, Hkv, D, ldv, kKeys) |
           map3(&tq128, q, Tq, Hq, D, ldq, kKeys) | map3(&tdo128, d_o, Tq, Hq, D, lddo, kKeys) |
           map3(&tk64, k, Tk, Hkv, D, ldk, kTile) | map3(&tv64, v, Tk, Hkv, D, ldv, kTile);
  if (rc) return rc;
  {
    long total_w = static_cast<long>(Tq) * Hq;
    int blocks = static_cast<int>((total_w + 7) / 8);
    if (blocks > 148 * 16) blocks = 148 * 16;
    attn_delta2_kernel<<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(o),
                                               static_cast<const __nv_bfloat16*>(d_o), static_cast<float*>(delta), Tq,
                                               Hq, D, ldo, lddo);
  }
  BwdP p{};
  p.cu_q = static_cast<const int*>(cu_q);
  p.cu_k = static_cast<const int*>(cu_k);
  p.n_docs = n_docs;
  p.Hq = Hq; p.Hkv = Hkv; p.D = D;
  p.scale = scale;
  p.scale_log2 = scale * kLog2eB;
  p.causal = causal;
  p.window_left = window_left;
  p.lse = static_cast<const float*>(lse);
  p.delta = static_cast<const float*>(delta);
  p.dQ = static_cast<__nv_bfloat16*>(dq);
  p.dK = static_cast<__nv_bfloat16*>(dk);
  p.dV = static_cast<__nv_bfloat16*>(dv);
  p.lddq = lddq; p.lddk = lddk; p.lddv = lddv;
  p.Tq = Tq;
  p.Tk = Tk;
  p.status = status;
  static bool set = false;
  if (!set) {
    cudaFuncSetAttribute(attn_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kTotal);
    cudaFuncSetAttribute(attn_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemQ::kTotal);
    set = true;
  }
  dim3 grid_kv((Tk + kKeys - 1) / kKeys + n_docs, Hkv);
  attn_dkdv_kernel<<<grid_kv, 384, Smem::kTotal, st>>>(tq64, tk128, tv128, tdo64, p);
  if (cudaGetLastError() != cudaSuccess) return -4;
  dim3 grid_q((Tq + kKeys - 1) / kKeys + n_docs, Hq);
  attn_dq_kernel<<<grid_q, 384, SmemQ::kTotal, st>>>(tq128, tk64, tv64, tdo128, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
