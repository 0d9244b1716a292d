// Varlen (packed) flash attention for sm_100a on tcgen05 / TMEM.
//
// Forward: one CTA per (document, query block of 128 rows, query head).
//   warp 0   TMA producer: Q once, then K_j / V_j tiles (128 keys) into 2-stage rings
//   warp 1   MMA issuer:   S_j = Q K_j^T into one of two TMEM buffers (so QK^T of block
//                          j+1 overlaps the softmax of block j), then O += P_j V_j
//   warp 2   TMEM allocator
//   warps 4-7 softmax: one thread per query row reads S from TMEM, keeps the running
//            max / sum, writes P (bf16) into swizzled shared memory as the A operand of
//            the PV product, rescales the O accumulator in TMEM only when the running
//            max moved by more than 2^8, and finally normalises and stores O and LSE.
// Supports causal / full attention, a left sliding window, GQA, head_dim <= 128
// (tiles are zero-padded to 64 or 128 by the TMA out-of-bounds fill, which is what the
// 80- and 72-wide vision heads use).
//
// Backward: one CTA per (document, key block of 128, KV head); it loops over the
// query heads of the group and over query tiles of 64 rows in the transposed
// formulation (S^T = K Q^T), so that P^T and dS^T come out of TMEM already in the
// K-major layout the dV / dK products want; dQ^T tiles are reduced into an fp32
// buffer with coalesced red.global.add.
//
// Replaces flash_attn_varlen_func / the SDPA dense-mask fallback of the reference
// (src/lmms_engine/kernels/attention.py:20-182).
#include "common.cuh"

#include <cuda_fp16.h>

#include <stdio.h>

namespace b200 {

constexpr int kBlockQ = 128;
constexpr int kBlockK = 128;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct FwdParams {
  const int* cu_q;
  const int* cu_k;
  int n_docs;
  int Hq, Hkv, D;        // D = true head dim
  float scale_log2;      // softmax scale * log2(e)
  int causal;
  int window_left;       // < 0: unlimited
  __nv_bfloat16* O;      // [T, Hq, D]
  long ldo;              // row stride of O in elements
  float* lse;            // [Hq, Tq]
  int Tq, Tk;
  int* status;
};

// ---- shared memory plan (DP = padded head dim: 64 or 128) ------------------------------
template <int DP>
struct FwdSmem {
  // A K or V stage is released only when the product that read it has retired, and its refill then pays the whole TMA
  // latency (about 2 400 cycles), so with S stages a tile's period is at least that latency / (S - 1): three stages each.
  // The room comes from Q, which is copied once into TMEM (the A operand of every Q K^T product) and only lands in
  // shared memory, in the buffer that the probabilities use afterwards.
  static constexpr int kStages = 3;
  static constexpr int kTile = kBlockQ * DP * 2;  // bytes of one Q / K / V tile
  static constexpr int kK = 0;                     // kStages stages
  static constexpr int kV = kK + kStages * kTile;  // kStages stages
  static constexpr int kP = kV + kStages * kTile;  // 128 x 128 bf16
  static constexpr int kQ = kP;                    // landing area of Q: every thread later writes P only where it read Q
  static constexpr int kBars = kP + kBlockQ * kBlockK * 2;
  static constexpr int kX = kBars + 256;           // 1 KB: row maxima (2 tiles x 2 halves x 128 rows, fp16), then row sums (2 x 128, fp32)
  static constexpr int kTotal = kX + 1024 + 1024;
  static_assert(kTotal <= 227 * 1024, "shared memory of the forward kernel");
};

template <int DP>
__global__ void __launch_bounds__(384, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const FwdParams p) {
  using L = FwdSmem<DP>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
  constexpr int S = L::kStages;
  uint64_t* q_full = bars;                  // 1
  uint64_t* k_full = bars + 1;              // S
  uint64_t* k_empty = bars + 1 + S;         // S
  uint64_t* v_full = bars + 1 + 2 * S;      // S
  uint64_t* v_empty = bars + 1 + 3 * S;     // S
  uint64_t* s_full = bars + 1 + 4 * S;      // 2
  uint64_t* s_empty = bars + 3 + 4 * S;     // 2
  uint64_t* p_full = bars + 5 + 4 * S;      // 1
  uint64_t* pv_done = bars + 6 + 4 * S;     // 1
  uint64_t* pair_bar = bars + 7 + 4 * S;    // 4   the two softmax warps of a TMEM lane quadrant exchange their row maxima
  uint64_t* a_ready = bars + 11 + 4 * S;    // 1   Q sits in TMEM
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12 + 4 * S);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* work = reinterpret_cast<int*>(tmem_slot + 2);  // doc, q0, len_q, len_k, q_start, k_start

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // ---- decode the work item: heavy (late) query blocks are scheduled first ------------
  if (threadIdx.x == 0) {
    int total = 0;
    for (int d = 0; d < p.n_docs; ++d) total += (p.cu_q[d + 1] - p.cu_q[d] + kBlockQ - 1) / kBlockQ;
    int item = total - 1 - static_cast<int>(blockIdx.x);
    work[0] = -1;
    if (item >= 0) {
      int acc = 0;
      for (int d = 0; d < p.n_docs; ++d) {
        const int lq = p.cu_q[d + 1] - p.cu_q[d];
        const int nb = (lq + kBlockQ - 1) / kBlockQ;
        if (item < acc + nb) {
          work[0] = d;
          work[1] = (item - acc) * kBlockQ;
          work[2] = lq;
          work[3] = p.cu_k[d + 1] - p.cu_k[d];
          work[4] = p.cu_q[d];
          work[5] = p.cu_k[d];
          if (!doc_in_bounds(work[4], work[2], p.Tq, p.status) || !doc_in_bounds(work[5], work[3], p.Tk, p.status)) work[0] = -1;
          break;
        }
        acc += nb;
      }
    }
    mbar_init(q_full, 1);
    for (int i = 0; i < S; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 8);
    }
    mbar_init(a_ready, 8);
    for (int i = 0; i < 4; ++i) mbar_init(&pair_bar[i], 2);
    mbar_init(p_full, 8);
    mbar_init(pv_done, 1);
    *abort_word = 0;
    fence_barrier_init();
  }
  __syncthreads();
  if (work[0] < 0) return;  // uniform: nothing allocated yet
  if (warp == 2) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_O = tmem_base;            // 128 columns
  const uint32_t tmem_S0 = tmem_base + 128;     // 2 x 128 columns
  const uint32_t tmem_Q = tmem_base + 384;      // DP / 2 columns: Q as bf16 pairs, row m in lane m

  const int q0 = work[1], len_q = work[2], len_k = work[3], q_start = work[4], k_start = work[5];
  const int head = blockIdx.y;
  const int kv_head = head / (p.Hq / p.Hkv);
  const int offset = len_k - len_q;  // causal alignment (bottom-right)
  // key range visible to this query block
  int k_hi = len_k;
  if (p.causal) k_hi = min(len_k, q0 + kBlockQ + offset);
  int k_lo = 0;
  if (p.window_left >= 0) k_lo = max(0, q0 + offset - p.window_left);
  const int jb_lo = k_lo / kBlockK;
  const int jb_hi = (max(k_hi, 0) + kBlockK - 1) / kBlockK;  // exclusive
  const int n_iter = max(jb_hi - jb_lo, 0);

  if (warp == 0) {
    if (lane == 0 && n_iter > 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, L::kTile);
#pragma unroll
      for (int c = 0; c < DP / 64; ++c)
        tma_load_3d(smem + L::kQ + c * (kBlockQ * 128), &tmQ, q_full, c * 64, head, q_start + q0);
      bool ok = true;
      for (int it = 0; it < n_iter && ok; ++it) {
        const int s = it % S;
        const uint32_t ph = (it / S) & 1;
        const int krow = k_start + (jb_lo + it) * kBlockK;
        if (!mbar_wait(&k_empty[s], ph ^ 1, abort_word)) { ok = false; break; }
        mbar_expect_tx(&k_full[s], L::kTile);
#pragma unroll
        for (int c = 0; c < DP / 64; ++c)
          tma_load_3d(smem + L::kK + s * L::kTile + c * (kBlockK * 128), &tmK, &k_full[s], c * 64, kv_head, krow);
        if (!mbar_wait(&v_empty[s], ph ^ 1, abort_word)) { ok = false; break; }
        mbar_expect_tx(&v_full[s], L::kTile);
#pragma unroll
        for (int c = 0; c < DP / 64; ++c)
          tma_load_3d(smem + L::kV + s * L::kTile + c * (kBlockK * 128), &tmV, &v_full[s], c * 64, kv_head, krow);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_iter > 0) {
      const uint32_t idesc_qk = umma_idesc_bf16(kBlockQ, kBlockK);
      bool ok = mbar_wait(a_ready, 0, abort_word);
      auto issue_qk = [&](int it) -> bool {
        const int s = it & 1;            // TMEM buffer of the scores
        const int stg = it % S;          // shared-memory stage of K
        if (!mbar_wait(&k_full[stg], (it / S) & 1, abort_word)) return false;
        if (!mbar_wait(&s_empty[s], ((it >> 1) & 1) ^ 1, abort_word)) return false;
        tc_fence_after();
        const uint32_t sK = smem_u32(smem + L::kK + stg * L::kTile);
#pragma unroll
        for (int kk = 0; kk < DP / 16; ++kk) {
          const uint32_t off = (kk / 4) * (kBlockQ * 128) + (kk % 4) * 32;
          umma_bf16_ts(tmem_S0 + s * 128, tmem_Q + kk * 8, umma_desc_sw128(sK + off), idesc_qk, kk != 0);
        }
        umma_commit(&k_empty[stg]);
        umma_commit(&s_full[s]);
        return true;
      };
      for (int it = 0; it < n_iter && ok; ++it) ok = issue_qk(it);
    }
  } else if (warp == 3) {
    // A second issuing thread for the P V products: a thread blocks while it issues and pays every commit, fence and
    // barrier hand-off in sequence; with one thread for both products the tensor pipe idled during those.
    if (lane == 0 && n_iter > 0) {
      const uint32_t idesc_pv = umma_idesc_bf16_major(kBlockQ, DP, 0, 1);
      const uint32_t sP = smem_u32(smem + L::kP);
      bool ok = true;
      for (int it = 0; it < n_iter && ok; ++it) {
        const int stg = it % S;
        if (!mbar_wait(p_full, it & 1, abort_word)) { ok = false; break; }
        if (!mbar_wait(&v_full[stg], (it / S) & 1, abort_word)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sV = smem_u32(smem + L::kV + stg * L::kTile);
#pragma unroll
        for (int kk = 0; kk < kBlockK / 16; ++kk) {
          // A = P [128 q x 128 keys], K-major, two 64-key halves; B = V [keys x d], MN-major
          const uint64_t ad = umma_desc_sw128(sP + (kk / 4) * (kBlockQ * 128) + (kk % 4) * 32);
          uint64_t bd = umma_desc_sw128(sV + kk * 2048);
          bd = (bd & ~(uint64_t(0x3FFF) << 16)) | (uint64_t((kBlockK * 128) >> 4) << 16);
          umma_bf16_ss(tmem_O, ad, bd, idesc_pv, (it | kk) != 0);
        }
        umma_commit(&v_empty[stg]);
        umma_commit(pv_done);
      }
    }
  } else if (warp >= 4) {
    // Eight softmax warps: the two warps of a TMEM lane quadrant (warp, warp + 4) share the quadrant's 32 rows and
    // take 64 of a tile's 128 key columns each.  Four warps - one per scheduler, 128 exponentials per thread and
    // tile - were the limit of this kernel; the halves only exchange their row maxima (shared memory + a two-warp
    // barrier per tile) and, once at the end, their row sums.
    const int q = warp & 3;
    const int half = (warp - 4) >> 2;
    constexpr int kHalf = kBlockK / 2;      // key columns of a tile per thread
    constexpr int kOC = DP / 2;             // accumulator columns per thread
    const int r = q * 32 + lane;            // row within the query block
    const int qi = q0 + r;                  // row within the document
    const bool row_valid = qi < len_q;
    const uint32_t lane_sel = static_cast<uint32_t>(q * 32) << 16;
    // exchanged maxima are rounded to fp16 on both sides, so that both halves arrive at the same reference value (any
    // common value near the maximum serves; the row sum and the log-sum-exp stay exact)
    __half* xmax = reinterpret_cast<__half*>(smem + L::kX);          // [2 tiles][2 halves][128 rows]
    float* xsum = reinterpret_cast<float*>(smem + L::kX);            // [2 halves][128 rows], after the loop
    float m_used = -INFINITY;               // max the accumulator is currently scaled by
    float l_run = 0.f;                      // sum over this thread's columns only
    bool ok = true;
    uint8_t* sP = smem + L::kP;
    // ---- Q from its landing area (128-byte swizzle) into TMEM: thread (row r, half h) copies the 64-column chunk h of
    // its row - the bytes it alone overwrites with probabilities later ----
    if (n_iter > 0) {
      const bool okq = mbar_wait(q_full, 0, abort_word);
      if (okq && half < DP / 64) {
        const uint8_t* src = smem + L::kQ + half * (kBlockQ * 128) + r * 128;
#pragma unroll
        for (int h16 = 0; h16 < 2; ++h16) {
          uint32_t wds[16];
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int chunk = (h16 * 4 + c) ^ (r & 7);
            const uint4 v = *reinterpret_cast<const uint4*>(src + chunk * 16);
            wds[c * 4 + 0] = v.x; wds[c * 4 + 1] = v.y; wds[c * 4 + 2] = v.z; wds[c * 4 + 3] = v.w;
          }
          tmem_st_32x32b_x16(tmem_Q + lane_sel + half * 32 + h16 * 16, wds);
        }
        tmem_st_wait();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(a_ready);
    }
    for (int it = 0; it < n_iter && ok; ++it) {
      const int s = it & 1;
      const uint32_t ph = (it >> 1) & 1;
      if (!mbar_wait(&s_full[s], ph, abort_word)) { ok = false; break; }
      tc_fence_after();
      const int kb0 = (jb_lo + it) * kBlockK;
      const int kc0 = kb0 + half * kHalf;   // first key column of this thread
      const bool need_mask = (kb0 + kBlockK > len_k) || (p.causal && kb0 + kBlockK - 1 > q0 + offset) ||
                             (p.window_left >= 0 && kb0 < q0 + kBlockQ - 1 + offset - p.window_left);
      float sv[kHalf];
      {
        // both loads in flight before the one wait (raw scores: the scale rides in the exponent's fma)
        uint32_t ra[32], rb[32];
        tmem_ld_32x32b_x32(tmem_S0 + s * 128 + lane_sel + half * kHalf, ra);
        tmem_ld_32x32b_x32(tmem_S0 + s * 128 + lane_sel + half * kHalf + 32, rb);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          sv[j] = __uint_as_float(ra[j]);
          sv[32 + j] = __uint_as_float(rb[j]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[s]);
      if (need_mask) {
#pragma unroll
        for (int j = 0; j < kHalf; ++j) {
          const int kj = kc0 + j;
          bool vis = kj < len_k;
          if (p.causal) vis = vis && (kj <= qi + offset);
          if (p.window_left >= 0) vis = vis && (kj >= qi + offset - p.window_left);
          if (!vis) sv[j] = -INFINITY;
        }
      }
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < kHalf; ++j) mx = fmaxf(mx, sv[j]);
      mx *= p.scale_log2;  // the scale is positive: the maximum of the scaled scores
      // the row's maximum over both halves
      const __half mx_h = __float2half_rn(fmaxf(mx, -60000.f));
      xmax[(s * 2 + half) * kBlockQ + r] = mx_h;
      __syncwarp();
      if (lane == 0) mbar_arrive(&pair_bar[q]);
      if (!mbar_wait(&pair_bar[q], it & 1, abort_word)) { ok = false; break; }
      mx = fmaxf(__half2float(mx_h), __half2float(xmax[(s * 2 + (half ^ 1)) * kBlockQ + r]));
      if (mx <= -60000.f) mx = -INFINITY;  // a row that sees nothing in this tile
      // lazy rescale: keep the old reference max unless it is stale by more than 2^8 (the same decision in both halves)
      const bool grow = mx > m_used + 8.f;
      const bool any_grow = __any_sync(0xffffffffu, grow);
      float alpha = 1.f;
      float m_new = m_used;
      if (grow) {
        m_new = mx;
        alpha = (m_used == -INFINITY) ? 0.f : fast_exp2(m_used - m_new);
      }
      const float neg_ref = (m_new == -INFINITY) ? 0.f : -m_new;
      // per element: one fma, one ex2, one add, half a convert.  The row sum takes the fp32 values (the bf16 rounding of
      // P averages out below the output's own precision).
      float rs0 = 0.f, rs1 = 0.f;
      uint32_t pk[kHalf / 2];
#pragma unroll
      for (int j = 0; j < kHalf; j += 2) {
        const float p0 = fast_exp2(fmaf(sv[j], p.scale_log2, neg_ref));
        const float p1 = fast_exp2(fmaf(sv[j + 1], p.scale_log2, neg_ref));
        pk[j / 2] = pack_bf16x2(p0, p1);
        rs0 += p0;
        rs1 += p1;
      }
      const float rs = rs0 + rs1;
      l_run = l_run * alpha + rs;
      m_used = m_new;
      // P buffer and the O accumulator are free once the previous PV product retired
      if (it > 0) {
        if (!mbar_wait(pv_done, (it - 1) & 1, abort_word)) { ok = false; break; }
        tc_fence_after();
        if (any_grow) {  // this thread rescales its half of the accumulator's columns
#pragma unroll
          for (int c = 0; c < kOC / 32; ++c) {
            uint32_t rr[32];
            tmem_ld_32x32b_x32(tmem_O + lane_sel + half * kOC + c * 32, rr);
            tmem_ld_wait();
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
              uint32_t w[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) w[j] = __float_as_uint(__uint_as_float(rr[h2 * 16 + j]) * alpha);
              tmem_st_32x32b_x16(tmem_O + lane_sel + half * kOC + c * 32 + h2 * 16, w);
            }
          }
          tmem_st_wait();
        }
      }
      // P -> shared memory: this thread's 64 keys are one 128B-swizzled K-major half of the tile
      {
        uint8_t* rowp = sP + half * (kBlockQ * 128) + r * 128;
#pragma unroll
        for (int c16 = 0; c16 < 8; ++c16) {
          const int chunk = c16 ^ (r & 7);
          const int b = c16 * 4;
          *reinterpret_cast<uint4*>(rowp + chunk * 16) = make_uint4(pk[b], pk[b + 1], pk[b + 2], pk[b + 3]);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // ---- epilogue: O / l, LSE -------------------------------------------------------
    if (ok && n_iter > 0) ok = mbar_wait(pv_done, (n_iter - 1) & 1, abort_word);
    tc_fence_after();
    // the row sum over both halves; the area held the maxima: first make sure the partner has read its last one
    __syncwarp();
    if (lane == 0) mbar_arrive(&pair_bar[q]);
    if (ok) ok = mbar_wait(&pair_bar[q], n_iter & 1, abort_word);
    xsum[half * kBlockQ + r] = l_run;
    __syncwarp();
    if (lane == 0) mbar_arrive(&pair_bar[q]);
    if (ok) ok = mbar_wait(&pair_bar[q], (n_iter + 1) & 1, abort_word);
    const float l_all = l_run + xsum[(half ^ 1) * kBlockQ + r];
    const float inv_l = (l_all > 0.f) ? 1.f / l_all : 0.f;
    if (row_valid && ok && half == 0) {
      p.lse[static_cast<size_t>(head) * p.Tq + q_start + qi] =
          (l_all > 0.f) ? (m_used + log2f(l_all)) * kLn2 : -INFINITY;
    }
    __nv_bfloat16* orow = p.O + static_cast<size_t>(q_start + qi) * p.ldo + static_cast<size_t>(head) * p.D;
#pragma unroll
    for (int c = 0; c < kOC / 32; ++c) {
      const int col0 = half * kOC + c * 32;
      uint32_t rr[32];
      if (n_iter > 0 && ok) {
        tmem_ld_32x32b_x32(tmem_O + lane_sel + col0, rr);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) rr[j] = 0u;
      }
      if (row_valid && ok) {
#pragma unroll
        for (int j8 = 0; j8 < 4; ++j8) {
          const int col = col0 + j8 * 8;
          if (col < p.D) {  // D is a multiple of 8
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(rr[j8 * 8 + 0]) * inv_l, __uint_as_float(rr[j8 * 8 + 1]) * inv_l);
            o.y = pack_bf16x2(__uint_as_float(rr[j8 * 8 + 2]) * inv_l, __uint_as_float(rr[j8 * 8 + 3]) * inv_l);
            o.z = pack_bf16x2(__uint_as_float(rr[j8 * 8 + 4]) * inv_l, __uint_as_float(rr[j8 * 8 + 5]) * inv_l);
            o.w = pack_bf16x2(__uint_as_float(rr[j8 * 8 + 6]) * inv_l, __uint_as_float(rr[j8 * 8 + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + col) = o;
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

// ======================================================================== backward
// delta[h, t] = sum_d O[t,h,d] * dO[t,h,d]
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO,
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

struct BwdParams {
  const int* cu_q;
  const int* cu_k;
  int n_docs;
  int Hq, Hkv, D;
  float scale;           // softmax scale
  float scale_log2;
  int causal;
  int window_left;
  const float* lse;      // [Hq, Tq]
  const float* delta;    // [Hq, Tq]
  float* dQ;             // [Tq, Hq, D] fp32, zero-initialised
  __nv_bfloat16* dK;     // [Tk, Hkv, D]
  __nv_bfloat16* dV;
  long lddk, lddv;
  int Tq, Tk;
  int* status;
};

constexpr int kBwdQ = 64;  // query rows per inner tile

template <int DP>
struct BwdSmem {
  static constexpr int kKV = kBlockK * DP * 2;          // K_j or V_j tile
  static constexpr int kQT = kBwdQ * DP * 2;            // Q_i or dO_i tile
  static constexpr int kK = 0;
  static constexpr int kV = kK + kKV;
  static constexpr int kQ = kV + kKV;                   // 2 stages of (Q_i, dO_i)
  static constexpr int kPT = kQ + 2 * 2 * kQT;          // P^T  [128 keys x 64 q] bf16, 16 KB
  static constexpr int kDST = kPT + kBlockK * kBwdQ * 2;  // dS^T
  static constexpr int kStat = kDST + kBlockK * kBwdQ * 2;  // lse[64], delta[64] x 2 stages
  static constexpr int kBars = kStat + 2 * 2 * kBwdQ * 4;
  static constexpr int kTotal = kBars + 256 + 1024;
};

template <int DP>
__global__ void __launch_bounds__(256, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                const BwdParams p) {
  using L = BwdSmem<DP>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
  uint64_t* kv_full = bars;           // 1
  uint64_t* q_full = bars + 1;        // 2
  uint64_t* q_empty = bars + 3;       // 2
  uint64_t* s_full = bars + 5;        // 1  S^T and dP^T ready
  uint64_t* ds_full = bars + 6;       // 1  P^T / dS^T written to smem
  uint64_t* mma_done = bars + 7;      // 1  dV, dK, dQ^T products retired
  uint64_t* dq_read = bars + 8;       // 1  dQ^T (aliasing S^T) drained
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* work = reinterpret_cast<int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    int item = blockIdx.x;
    work[0] = -1;
    int acc = 0;
    for (int d = 0; d < p.n_docs; ++d) {
      const int lk = p.cu_k[d + 1] - p.cu_k[d];
      const int nb = (lk + kBlockK - 1) / kBlockK;
      if (item < acc + nb) {
        work[0] = d;
        work[1] = (item - acc) * kBlockK;
        work[2] = p.cu_q[d + 1] - p.cu_q[d];
        work[3] = lk;
        work[4] = p.cu_q[d];
        work[5] = p.cu_k[d];
        if (!doc_in_bounds(work[4], work[2], p.Tq, p.status) || !doc_in_bounds(work[5], work[3], p.Tk, p.status)) work[0] = -1;
        break;
      }
      acc += nb;
    }
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(ds_full, 4);
    mbar_init(mma_done, 1);
    mbar_init(dq_read, 4);
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
  const uint32_t tm_ST = tmem_base;          // [128 keys x 64 q] fp32: 64 cols; later dQ^T [128 d x 64 q]
  const uint32_t tm_dPT = tmem_base + 64;    // 64 cols
  const uint32_t tm_dV = tmem_base + 128;    // [128 keys x DP]
  const uint32_t tm_dK = tmem_base + 256;    // [128 keys x DP]

  const int k0 = work[1], len_q = work[2], len_k = work[3], q_start = work[4], k_start = work[5];
  const int kvh = blockIdx.y;
  const int group = p.Hq / p.Hkv;
  const int offset = len_k - len_q;
  // query rows that can see this key block
  int q_lo = 0;
  if (p.causal) q_lo = max(0, k0 - offset);
  int q_hi = len_q;
  if (p.window_left >= 0) q_hi = min(len_q, k0 + kBlockK - 1 - offset + p.window_left + 1);
  const int ib_lo = q_lo / kBwdQ;
  const int ib_hi = (max(q_hi, 0) + kBwdQ - 1) / kBwdQ;
  const int n_qt = max(ib_hi - ib_lo, 0);
  const int n_iter = n_qt * group;

  if (warp == 0) {
    if (lane == 0 && n_iter > 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmdO);
      mbar_expect_tx(kv_full, 2 * L::kKV);
#pragma unroll
      for (int c = 0; c < DP / 64; ++c) {
        tma_load_3d(smem + L::kK + c * (kBlockK * 128), &tmK, kv_full, c * 64, kvh, k_start + k0);
        tma_load_3d(smem + L::kV + c * (kBlockK * 128), &tmV, kv_full, c * 64, kvh, k_start + k0);
      }
      bool ok = true;
      for (int it = 0; it < n_iter && ok; ++it) {
        const int s = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        const int hq = kvh * group + it / n_qt;
        const int qrow = q_start + (ib_lo + it % n_qt) * kBwdQ;
        if (!mbar_wait(&q_empty[s], ph ^ 1, abort_word)) { ok = false; break; }
        mbar_expect_tx(&q_full[s], 2 * L::kQT);
        uint8_t* dst = smem + L::kQ + s * 2 * L::kQT;
#pragma unroll
        for (int c = 0; c < DP / 64; ++c) {
          tma_load_3d(dst + c * (kBwdQ * 128), &tmQ, &q_full[s], c * 64, hq, qrow);
          tma_load_3d(dst + L::kQT + c * (kBwdQ * 128), &tmdO, &q_full[s], c * 64, hq, qrow);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_iter > 0) {
      // S^T = K Q^T, dP^T = V dO^T : M = 128 keys, N = 64 q, K = d; both operands K-major
      const uint32_t idesc_s = umma_idesc_bf16(kBlockK, kBwdQ);
      // dV += P^T dO, dK += dS^T Q : M = 128 keys, N = DP, K = 64 q; A K-major, B MN-major
      const uint32_t idesc_dkv = umma_idesc_bf16_major(kBlockK, DP, 0, 1);
      // dQ^T = K^T dS^T : M = DP (d), N = 64 q, K = 128 keys; A MN-major, B MN-major
      const uint32_t idesc_dq = umma_idesc_bf16_major(DP, kBwdQ, 1, 1);
      const uint32_t sK = smem_u32(smem + L::kK), sV = smem_u32(smem + L::kV);
      const uint32_t sPT = smem_u32(smem + L::kPT), sDST = smem_u32(smem + L::kDST);
      bool ok = mbar_wait(kv_full, 0, abort_word);
      for (int it = 0; it < n_iter && ok; ++it) {
        const int s = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(&q_full[s], ph, abort_word)) { ok = false; break; }
        if (it > 0 && !mbar_wait(dq_read, (it - 1) & 1, abort_word)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sQ = smem_u32(smem + L::kQ + s * 2 * L::kQT);
        const uint32_t sdO = sQ + L::kQT;
#pragma unroll
        for (int kk = 0; kk < DP / 16; ++kk) {
          const uint32_t offA = (kk / 4) * (kBlockK * 128) + (kk % 4) * 32;
          const uint32_t offB = (kk / 4) * (kBwdQ * 128) + (kk % 4) * 32;
          umma_bf16_ss(tm_ST, umma_desc_sw128(sK + offA), umma_desc_sw128(sQ + offB), idesc_s, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < DP / 16; ++kk) {
          const uint32_t offA = (kk / 4) * (kBlockK * 128) + (kk % 4) * 32;
          const uint32_t offB = (kk / 4) * (kBwdQ * 128) + (kk % 4) * 32;
          umma_bf16_ss(tm_dPT, umma_desc_sw128(sV + offA), umma_desc_sw128(sdO + offB), idesc_s, kk != 0);
        }
        umma_commit(s_full);
        if (!mbar_wait(ds_full, it & 1, abort_word)) { ok = false; break; }
        tc_fence_after();
        // B operands Q_i / dO_i as [N = d, K = q]: stored [q, d] -> MN-major, 64-wide d chunks
        // are kBwdQ*128 bytes apart, 16 q rows = 2048 bytes.
#pragma unroll
        for (int kk = 0; kk < kBwdQ / 16; ++kk) {
          const uint64_t aP = umma_desc_sw128(sPT + kk * 32);
          const uint64_t aD = umma_desc_sw128(sDST + kk * 32);
          uint64_t bO = umma_desc_sw128(sdO + kk * 2048);
          bO = (bO & ~(uint64_t(0x3FFF) << 16)) | (uint64_t((kBwdQ * 128) >> 4) << 16);
          uint64_t bQ = umma_desc_sw128(sQ + kk * 2048);
          bQ = (bQ & ~(uint64_t(0x3FFF) << 16)) | (uint64_t((kBwdQ * 128) >> 4) << 16);
          umma_bf16_ss(tm_dV, aP, bO, idesc_dkv, (it | kk) != 0);
          umma_bf16_ss(tm_dK, aD, bQ, idesc_dkv, (it | kk) != 0);
        }
        umma_commit(&q_empty[s]);
        // dQ^T [d x q] = K^T [d x keys] * dS [keys x q]
        //   A = K_j stored [keys, d]  -> MN-major A: 64-wide d chunks kBlockK*128 bytes apart
        //   B = dS^T stored [keys, q] -> MN-major B (N = q contiguous, one 64-wide chunk)
#pragma unroll
        for (int kk = 0; kk < kBlockK / 16; ++kk) {
          uint64_t aK = umma_desc_sw128(sK + kk * 2048);
          aK = (aK & ~(uint64_t(0x3FFF) << 16)) | (uint64_t((kBlockK * 128) >> 4) << 16);
          uint64_t bD = umma_desc_sw128(sDST + kk * 2048);
          bD = (bD & ~(uint64_t(0x3FFF) << 16)) | (uint64_t((kBlockK * 128) >> 4) << 16);
          umma_bf16_ss(tm_ST, aK, bD, idesc_dq, kk != 0);
        }
        umma_commit(mma_done);
      }
    }
  } else if (warp >= 4) {
    const int q = warp - 4;
    const int r = q * 32 + lane;      // key row within the block (S^T) / d index (dQ^T)
    const int kj = k0 + r;
    const uint32_t lane_sel = static_cast<uint32_t>(q * 32) << 16;
    uint8_t* sPT = smem + L::kPT;
    uint8_t* sDST = smem + L::kDST;
    bool ok = true;
    for (int it = 0; it < n_iter && ok; ++it) {
      const int hq = kvh * group + it / n_qt;
      const int qb0 = (ib_lo + it % n_qt) * kBwdQ;
      // per-row statistics of this query tile (read straight from global: 64 floats, L2 hits)
      const float* lse_p = p.lse + static_cast<size_t>(hq) * p.Tq + q_start + qb0;
      const float* dl_p = p.delta + static_cast<size_t>(hq) * p.Tq + q_start + qb0;
      if (!mbar_wait(s_full, it & 1, abort_word)) { ok = false; break; }
      tc_fence_after();
      uint32_t ppk[kBwdQ / 2], dpk[kBwdQ / 2];
#pragma unroll
      for (int c = 0; c < kBwdQ / 32; ++c) {
        uint32_t rs[32], rd[32];
        tmem_ld_32x32b_x32(tm_ST + lane_sel + c * 32, rs);
        tmem_ld_32x32b_x32(tm_dPT + lane_sel + c * 32, rd);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          float pv[2], dsv[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int qi = qb0 + c * 32 + j + e;
            bool vis = (qi < len_q) && (kj < len_k);
            if (p.causal) vis = vis && (kj <= qi + offset);
            if (p.window_left >= 0) vis = vis && (kj >= qi + offset - p.window_left);
            float pe = 0.f, dse = 0.f;
            if (vis) {
              const float l = lse_p[c * 32 + j + e];
              pe = exp2f(__uint_as_float(rs[j + e]) * p.scale_log2 - l * kLog2e);
              dse = pe * (__uint_as_float(rd[j + e]) - dl_p[c * 32 + j + e]) * p.scale;
            }
            pv[e] = pe;
            dsv[e] = dse;
          }
          ppk[(c * 32 + j) / 2] = pack_bf16x2(pv[0], pv[1]);
          dpk[(c * 32 + j) / 2] = pack_bf16x2(dsv[0], dsv[1]);
        }
      }
      // P^T / dS^T rows (64 q = 128 bytes) into swizzled K-major tiles
      {
        uint8_t* rp = sPT + r * 128;
        uint8_t* rd = sDST + r * 128;
#pragma unroll
        for (int c16 = 0; c16 < 8; ++c16) {
          const int chunk = c16 ^ (r & 7);
          *reinterpret_cast<uint4*>(rp + chunk * 16) =
              make_uint4(ppk[c16 * 4], ppk[c16 * 4 + 1], ppk[c16 * 4 + 2], ppk[c16 * 4 + 3]);
          *reinterpret_cast<uint4*>(rd + chunk * 16) =
              make_uint4(dpk[c16 * 4], dpk[c16 * 4 + 1], dpk[c16 * 4 + 2], dpk[c16 * 4 + 3]);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
      // dQ^T tile: lane = d index r, columns = q.  red.add coalesces over d.
      if (!mbar_wait(mma_done, it & 1, abort_word)) { ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < kBwdQ / 32; ++c) {
        uint32_t rq[32];
        tmem_ld_32x32b_x32(tm_ST + lane_sel + c * 32, rq);
        tmem_ld_wait();
        if (r < p.D) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int qi = qb0 + c * 32 + j;
            if (qi < len_q)
              atomicAdd(p.dQ + (static_cast<size_t>(q_start + qi) * p.Hq + hq) * p.D + r, __uint_as_float(rq[j]));
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_read);
    }
    // ---- epilogue: dK, dV of this key block ------------------------------------------
    tc_fence_after();
    const bool row_ok = ok && (kj < len_k);
    __nv_bfloat16* dkrow = p.dK + static_cast<size_t>(k_start + kj) * p.lddk + static_cast<size_t>(kvh) * p.D;
    __nv_bfloat16* dvrow = p.dV + static_cast<size_t>(k_start + kj) * p.lddv + static_cast<size_t>(kvh) * p.D;
#pragma unroll
    for (int c = 0; c < DP / 32; ++c) {
      uint32_t rk[32], rv[32];
      if (n_iter > 0 && ok) {
        tmem_ld_32x32b_x32(tm_dK + lane_sel + c * 32, rk);
        tmem_ld_32x32b_x32(tm_dV + lane_sel + c * 32, rv);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) rk[j] = rv[j] = 0u;
      }
      if (row_ok) {
#pragma unroll
        for (int j8 = 0; j8 < 4; ++j8) {
          const int col = c * 32 + j8 * 8;
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

// fp32 [n] -> bf16 [n]
__global__ void f32_to_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, long n) {
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long>(gridDim.x) * blockDim.x)
    out[i] = __float2bfloat16(in[i]);
}

// ---------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
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

// [T, H, D] bf16 with token stride `ld` elements -> 3-D map (d, head, token), box (64, 1, rows)
static int make_map3(CUtensorMap* m, const void* ptr, uint64_t T, uint64_t H, uint64_t D, uint64_t ld, uint32_t rows) {
  bind_context();
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[3] = {D, H, T};
  cuuint64_t strides[2] = {D * 2, ld * 2};
  cuuint32_t box[3] = {64, 1, rows};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "[b200 attn] cuTensorMapEncodeTiled failed (%d): T=%llu H=%llu D=%llu ld=%llu rows=%u\n",
            static_cast<int>(r), (unsigned long long)T, (unsigned long long)H, (unsigned long long)D,
            (unsigned long long)ld, rows);
    return -2;
  }
  return 0;
}

}  // namespace b200

using namespace b200;

extern "C" {

// q [Tq, Hq, D], k/v [Tk, Hkv, D] (token strides ldq/ldk/ldv elements, heads contiguous),
// o [Tq, Hq, D] (stride ldo), lse fp32 [Hq, Tq].  cu_q / cu_k: int32 [n_docs + 1] on device.
int b200_attn_fwd(const void* q, const void* k, const void* v, void* o, void* lse, const void* cu_q,
                  const void* cu_k, int n_docs, int Tq, int Tk, int Hq, int Hkv, int D, long ldq, long ldk, long ldv,
                  long ldo, float scale, int causal, int window_left, int* status, cudaStream_t st) {
  if (Tq <= 0 || n_docs <= 0) return 0;
  if (D % 8 || D > 128 || Hq % Hkv) return -10;
  const int DP = D <= 64 ? 64 : 128;
  CUtensorMap tq, tk, tv;
  int rc = make_map3(&tq, q, Tq, Hq, D, ldq, kBlockQ) | make_map3(&tk, k, Tk, Hkv, D, ldk, kBlockK) |
           make_map3(&tv, v, Tk, Hkv, D, ldv, kBlockK);
  if (rc) return rc;
  FwdParams p{};
  p.cu_q = static_cast<const int*>(cu_q);
  p.cu_k = static_cast<const int*>(cu_k);
  p.n_docs = n_docs;
  p.Hq = Hq; p.Hkv = Hkv; p.D = D;
  p.scale_log2 = scale * kLog2e;
  p.causal = causal;
  p.window_left = window_left;
  p.O = static_cast<__nv_bfloat16*>(o);
  p.ldo = ldo;
  p.lse = static_cast<float*>(lse);
  p.Tq = Tq;
  p.Tk = Tk;
  p.status = status;
  dim3 grid((Tq + kBlockQ - 1) / kBlockQ + n_docs, Hq);
  if (DP == 64) {
    static bool set = false;
    if (!set) { cudaFuncSetAttribute(attn_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem<64>::kTotal); set = true; }
    attn_fwd_kernel<64><<<grid, 384, FwdSmem<64>::kTotal, st>>>(tq, tk, tv, p);
  } else {
    static bool set = false;
    if (!set) { cudaFuncSetAttribute(attn_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem<128>::kTotal); set = true; }
    attn_fwd_kernel<128><<<grid, 384, FwdSmem<128>::kTotal, st>>>(tq, tk, tv, p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// delta: fp32 [Hq, Tq] scratch; dq_acc: fp32 [Tq, Hq, D] scratch (zeroed here); dq/dk/dv bf16 outputs.
int b200_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const void* lse,
                  void* delta, void* dq_acc, void* dq, void* dk, void* dv, const void* cu_q, const void* cu_k,
                  int n_docs, int Tq, int Tk, int Hq, int Hkv, int D, long ldq, long ldk, long ldv, long ldo,
                  long lddo, long lddq, long lddk, long lddv, float scale, int causal, int window_left, int* status,
                  cudaStream_t st) {
  if (Tq <= 0 || n_docs <= 0) return 0;
  if (D % 8 || D > 128 || Hq % Hkv) return -10;
  if (lddq != static_cast<long>(Hq) * D) return -12;  // dq must be contiguous [Tq, Hq, D]
  CUtensorMap tq, tk, tv, tdo;
  int rc = make_map3(&tq, q, Tq, Hq, D, ldq, kBwdQ) | make_map3(&tk, k, Tk, Hkv, D, ldk, kBlockK) |
           make_map3(&tv, v, Tk, Hkv, D, ldv, kBlockK) | make_map3(&tdo, d_o, Tq, Hq, D, lddo, kBwdQ);
  if (rc) return rc;
  {
    long total_w = static_cast<long>(Tq) * Hq;
    int blocks = static_cast<int>((total_w + 7) / 8);
    if (blocks > 148 * 16) blocks = 148 * 16;
    attn_delta_kernel<<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(o),
                                              static_cast<const __nv_bfloat16*>(d_o), static_cast<float*>(delta), Tq,
                                              Hq, D, ldo, lddo);
  }
  const long nq = static_cast<long>(Tq) * Hq * D;
  cudaMemsetAsync(dq_acc, 0, nq * sizeof(float), st);
  BwdParams p{};
  p.cu_q = static_cast<const int*>(cu_q);
  p.cu_k = static_cast<const int*>(cu_k);
  p.n_docs = n_docs;
  p.Hq = Hq; p.Hkv = Hkv; p.D = D;
  p.scale = scale;
  p.scale_log2 = scale * kLog2e;
  p.causal = causal;
  p.window_left = window_left;
  p.lse = static_cast<const float*>(lse);
  p.delta = static_cast<const float*>(delta);
  p.dQ = static_cast<float*>(dq_acc);
  p.dK = static_cast<__nv_bfloat16*>(dk);
  p.dV = static_cast<__nv_bfloat16*>(dv);
  p.lddk = lddk; p.lddv = lddv;
  p.Tq = Tq;
  p.Tk = Tk;
  p.status = status;
  dim3 grid((Tk + kBlockK - 1) / kBlockK + n_docs, Hkv);
  {
    // Always the 128-wide tile: head dims <= 64 are zero-padded by the TMA fill, which keeps
    // every tcgen05.mma of the backward at M = 128.
    static bool set = false;
    if (!set) { cudaFuncSetAttribute(attn_bwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem<128>::kTotal); set = true; }
    attn_bwd_kernel<128><<<grid, 256, BwdSmem<128>::kTotal, st>>>(tq, tk, tv, tdo, p);
  }
  if (cudaGetLastError() != cudaSuccess) return -4;
  int blocks = static_cast<int>((nq + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  f32_to_bf16_kernel<<<blocks, 256, 0, st>>>(static_cast<const float*>(dq_acc), static_cast<__nv_bfloat16*>(dq), nq);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // extern "C"
