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
  int group_m;                 // m-blocks that share one sweep over N (L2 reuse of the B panels)
  int* status;
};

// Collective work fused into one GEMM launch over peer-mapped buffers (plain peer stores and
// system-scope flags; no multicast).  Three independent parts, each optional:
//  push    : before its tiles, every CTA copies a slice of a local block into every rank's buffer
//            (all-gather of rows, or the sequence<->head all-to-all) and raises arrive_in there;
//  wait    : the TMA producer waits for arrive_in of the rank whose rows (mode 1) or k-range
//            (mode 2) a tile reads, so tiles of blocks that have already landed run first;
//  scatter : the epilogue stores each tile into the destination rank's buffer instead of C:
//            mode 1 = row blocks into per-source slots of the rank that owns the rows; every rank
//            computes its own row blocks last and their epilogue adds the slots that have landed
//            by then (reduce-scatter without a separate pass), mode 2 = 64-column chunks routed
//            by a table (all-to-all by heads).  arrive_out counts stored tiles (mode 1, one per
//            epilogue warp) or finished source CTAs (mode 2).
// Flag block of a buffer on every rank: u32 [3][kMaxRanks] = arrive_in | arrive_out | done.
constexpr int kMaxRanks = 8;
constexpr int kMaxPushSeg = 3;
struct CommParams {
  int rank, world;
  long long wait_cycles;
  // push
  int push, push_rows, push_nseg;
  // the block is made of up to three column segments, each with its own source matrix; the rows for
  // destination r start at row r * push_block_rows of every source (0: the same rows go to all ranks)
  const __nv_bfloat16* seg_src[kMaxPushSeg];
  long long seg_src_ld[kMaxPushSeg];
  long long push_block_rows;
  long long push_dst_ld, push_dst_off;     // element offset of this rank's block inside a destination buffer
  int seg_dst_col[kMaxPushSeg], seg_cols[kMaxPushSeg];
  __nv_bfloat16* push_dst[kMaxRanks];
  uint32_t* pflags[kMaxRanks];
  uint32_t in_target;
  // handshake of a shared gather buffer: a CTA that starts raises done on every rank (whatever read
  // this rank's buffer earlier in the stream has finished) and writes to rank r only once all CTAs
  // of r have started too
  int push_done_wait;
  uint32_t push_done_target;
  // wait
  int wait_mode, rows_per_src, k_per_src, m_rot, k_rot;
  int own_direct;                          // mode 1: tiles of this rank's own rows read the source matrix (map tmB2)
  // > 0: the last push_ctas CTAs of the grid only push (all eight warps) and the others only compute,
  // so the copy neither delays an epilogue nor shares an SM with a main loop; 0: warps 2..7 of every
  // CTA push before their tiles (right when no tile can finish before the blocks have landed)
  int push_ctas;
  // 1: the four epilogue warps join warps 2 and 3 in the copy before their first tile (right when no
  // tile can finish before the blocks have landed); 0: only warps 2 and 3 copy, next to the tiles
  int push_wide;
  int in_inc;                              // > 0: arrive_in grows by this much per call (the copy is made outside the kernel)
  const int* kb_src;                       // mode 2: source rank of every 64-wide k-block (null: k / k_per_src)
  // scatter
  int scatter;
  long long sc_ld, sc_slot_stride;
  const int* chunk_dst;
  const int* chunk_col;
  const int* chunk_ndst;
  int sc_row_off;
  __nv_bfloat16* sc_dst[kMaxRanks];
  uint32_t* sflags[kMaxRanks];
  uint32_t out_target, sc_done_target;
  int out_inc_tiles;                       // mode 1: arrive_out grows by 4 (epilogue warps) per tile sent to a rank
  // optional timeline of CTA 0 in globaltimer nanoseconds: [0] start [1] handshake passed [2] first
  // remote block pushed and flagged [3] all blocks pushed [4] producer saw its last source [5] end
  unsigned long long* trace;
  __nv_bfloat16* reduce_out;
  long long reduce_ld;
};

// Signalling convention of the fused collectives: the data stores of a warp / of the pushing warps
// are ordered before the signalling thread by __syncwarp / a named barrier, and the signal itself is
// a release at system scope (flag_add_release), which is cumulative over that order.
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }

// Map a linear tile index to (m_block, n_block).  Sixteen m-blocks share each sweep
// over N so that concurrently resident CTAs reuse the same B panels out of L2.
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& mb, int& nb, int kGroup) {
  int per_group = kGroup * tiles_n;
  int g = t / per_group;
  int first_m = g * kGroup;
  int gsz = min(kGroup, tiles_m - first_m);
  int r = t - g * per_group;
  mb = first_m + r % gsz;
  nb = r / gsz;
}

template <int EPI, int COMM>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmB2, const __grid_constant__ CUtensorMap tmC,
                 const __grid_constant__ CUtensorMap tmC2, const __grid_constant__ CUtensorMap tmC3,
                 const GemmParams p, const __grid_constant__ CommParams cp) {
  // a fused collective may have to wait for a rank that was launched later: its waits use the
  // caller's limit, every other launch keeps the short default
  const long long wait_limit = COMM ? cp.wait_cycles : kWaitCycleLimit;
  const int n_gemm_ctas = COMM ? static_cast<int>(gridDim.x) - cp.push_ctas : static_cast<int>(gridDim.x);
  const bool push_cta = COMM && static_cast<int>(blockIdx.x) >= n_gemm_ctas;
  const bool tracing = COMM && cp.trace != nullptr && blockIdx.x == (cp.push_ctas > 0 ? n_gemm_ctas : 0);
  if (tracing && threadIdx.x == 0) cp.trace[0] = global_ns();
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
  if (warp == 2 && !push_cta) {
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
      tile_coords(t - e * tiles_per_expert, tiles_m, tiles_n, mb, nb, p.group_m);
      const int r0 = p.expert_start[e], r1 = p.expert_start[e + 1];
      kb_lo = r0 / BK;
      kb_n = (r1 - r0) / BK;
    } else {
      tile_coords(t, tiles_m, tiles_n, mb, nb, p.group_m);
      if (COMM) {
        // start with the row blocks whose data is local (gather) or whose destination is the
        // farthest in the ring (reduce-scatter), so that transfers overlap the remaining tiles
        mb += cp.m_rot;
        if (mb >= tiles_m) mb -= tiles_m;
      }
      e = p.tile_expert != nullptr ? p.tile_expert[mb] : 0;
      kb_lo = 0;
      kb_n = n_kb;
    }
  };

  // Copy this rank's block into every rank's buffer (COMM push).  Runs on warps 2..7 (192 threads):
  // the epilogue warps have nothing to drain before the first accumulator completes.  Every thread
  // executes every iteration, so the named barrier below always gets its full count.
  // In a dedicated push CTA all 256 threads run it instead.
  const int push_threads = push_cta ? kThreads : (cp.push_wide ? 192 : 64);
  const int push_slices = cp.push_ctas > 0 ? cp.push_ctas : static_cast<int>(gridDim.x);
  const int push_slice = cp.push_ctas > 0 ? static_cast<int>(blockIdx.x) - n_gemm_ctas : static_cast<int>(blockIdx.x);
  auto push_blocks = [&](const int ct) {
    const int pw = ct >> 5;
    bool okp = true;
    if (cp.push_done_wait && pw == 0 && lane < cp.world) {
      flag_add_release(cp.pflags[lane] + 2 * kMaxRanks + cp.rank, 1u);
    }
    for (int d = 0; d < cp.world; ++d) {
      // the ranks in the order in which they will need this block; the local copy comes last when
      // this rank's own tiles read the source directly, first otherwise
      const int r = cp.own_direct ? (cp.rank - 1 - d + 2 * cp.world) % cp.world : (cp.rank - d + cp.world) % cp.world;
      if (okp && cp.push_done_wait) {
        int w = 1;
        if (lane == 0) w = flag_wait_ge(cp.pflags[cp.rank] + 2 * kMaxRanks + r, cp.push_done_target, wait_limit, abort_word);
        okp = __shfl_sync(0xffffffffu, w, 0) != 0;
        if (tracing && ct == 0 && d == 0) cp.trace[1] = global_ns();
      }
      if (okp) {
        __nv_bfloat16* dst = cp.push_dst[r] + cp.push_dst_off;
        for (int sg = 0; sg < cp.push_nseg; ++sg) {
          const long long sld = cp.seg_src_ld[sg];
          const int vpr = cp.seg_cols[sg] >> 3;  // 16-byte vectors per row
          const long long total = static_cast<long long>(cp.push_rows) * vpr;
          const long long per = (total + push_slices - 1) / push_slices;
          const long long v_hi = min(total, per * (push_slice + 1));
          const __nv_bfloat16* s0 = cp.seg_src[sg] + r * cp.push_block_rows * sld;
          __nv_bfloat16* d0 = dst + cp.seg_dst_col[sg];
          for (long long v = per * push_slice + ct; v < v_hi; v += push_threads * 8) {
            uint4 val[8];
            long long dof[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const long long vv = v + u * push_threads;
              if (vv < v_hi) {
                const long long row = vv / vpr;
                const int c = static_cast<int>(vv - row * vpr) * 8;
                val[u] = *reinterpret_cast<const uint4*>(s0 + row * sld + c);
                dof[u] = row * cp.push_dst_ld + c;
              }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u)
              if (v + u * push_threads < v_hi) *reinterpret_cast<uint4*>(d0 + dof[u]) = val[u];
          }
        }
      }
      bar_sync_named(1, push_threads);
      if (ct == 0 && okp) {
        flag_add_release(cp.pflags[r] + cp.rank, 1u);
        if (tracing && d == 0) cp.trace[2] = global_ns();
        if (tracing && d == cp.world - 1) cp.trace[3] = global_ns();
      }
    }
  };

  if (push_cta) {
    // ------------------------------------------------------------ dedicated push CTA
    push_blocks(threadIdx.x);
  } else if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t it = 0;
      bool ok = true;
      uint32_t landed = 0;  // COMM: sources whose block is known to have arrived
      auto source_ready = [&](int src) -> bool {
        if ((landed >> src) & 1u) return true;
        if (!flag_wait_ge(cp.pflags[cp.rank] + src, cp.in_target, wait_limit, abort_word)) return false;
        fence_proxy_async_all();  // the block was written by generic stores, TMA reads it next
        landed |= 1u << src;
        if (tracing) cp.trace[4] = global_ns();
        return true;
      };
      for (int t = blockIdx.x; t < total_tiles && ok; t += n_gemm_ctas) {
        int ex, mb, nb, kb_lo, kb_n;
        decode(t, ex, mb, nb, kb_lo, kb_n);
        if (!tile_active(mb, nb)) continue;
        const int m0 = mb * BM;
        const int n0 = (EPI == EPI_SWIGLU) ? nb * (BN / 2) : nb * BN;
        const bool grouped_b = p.tile_expert != nullptr;  // B is a 3-D map indexed by expert
        bool own_rows = false;
        if (COMM && cp.wait_mode == 1) {
          const int src = m0 / cp.rows_per_src;
          own_rows = cp.own_direct && src == cp.rank;
          if (!own_rows && !source_ready(src)) { ok = false; break; }
        }
        for (int kb = 0; kb < kb_n; ++kb, ++it) {
          int kbr = kb_lo + kb;
          if (COMM) {
            kbr += cp.k_rot;  // begin with the k-range that this rank contributed itself
            if (kbr >= n_kb) kbr -= n_kb;
            if (cp.wait_mode == 2) {
              const int src = cp.kb_src != nullptr ? cp.kb_src[kbr] : kbr * BK / cp.k_per_src;
              own_rows = cp.own_direct && src == cp.rank;
              if (!own_rows && !source_ready(src)) { ok = false; break; }
            }
          }
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_word, wait_limit)) { ok = false; break; }
          uint8_t* sa = smem + s * kStageBytes;
          uint8_t* sb = sa + kATileBytes;
          mbar_expect_tx(&full_bar[s], kStageBytes);
          const int k0 = kbr * BK;
          if (COMM && own_rows) {
            // this rank's own block straight from the matrix that is being pushed
            if (cp.wait_mode == 1) tma_load_2d(sa, &tmB2, &full_bar[s], k0, m0 - cp.rank * cp.rows_per_src);
            else tma_load_2d(sa, &tmB2, &full_bar[s], k0 - cp.rank * cp.k_per_src, m0 + cp.rank * static_cast<int>(cp.push_block_rows));
          } else if (!p.a_mn_major) {
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
      for (int t = blockIdx.x; t < total_tiles && ok; t += n_gemm_ctas) {
        int ex, mb, nb, kb_lo, kb_n;
        decode(t, ex, mb, nb, kb_lo, kb_n);
        if (!tile_active(mb, nb)) continue;
        const int acc = tl & 1;
        const uint32_t acc_ph = (tl >> 1) & 1;
        if (!mbar_wait(&tempty_bar[acc], acc_ph ^ 1, abort_word, wait_limit)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kb_n; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(&full_bar[s], ph, abort_word, wait_limit)) { ok = false; break; }
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
  } else if (COMM && warp < 4) {
    // ------------------------------------------------------------ push (warps 2, 3; the epilogue warps help)
    if (cp.push && cp.push_ctas == 0) push_blocks((warp - 2) * 32 + lane);
  } else if (warp >= 4) {
    // ------------------------------------------------------------ epilogue (warps 4..7)
    const int q = warp - 4;  // TMEM lane quadrant == warp % 4
    uint8_t* slab0 = epi_smem + q * 2 * kEpiSlabBytes;
    uint32_t tl = 0;
    int buf = 0;
    bool ok = true;
    uint32_t sc_open = 0;  // COMM scatter: destinations known to have drained their slots
    bool own_ready = false;
    if (COMM && cp.push && cp.push_ctas == 0 && cp.push_wide) push_blocks(64 + q * 32 + lane);
    for (int t = blockIdx.x; t < total_tiles && ok; t += n_gemm_ctas) {
      int ex, mb, nb, kb_lo, kb_n;
      decode(t, ex, mb, nb, kb_lo, kb_n);
      if (!tile_active(mb, nb)) continue;
      const bool empty_k = (kb_n == 0);  // grouped-K expert without rows: the product is zero
      const int acc = tl & 1;
      const uint32_t acc_ph = (tl >> 1) & 1;
      if (!mbar_wait(&tfull_bar[acc], acc_ph, abort_word, wait_limit)) { ok = false; break; }
      tc_fence_after();
      const int m0 = mb * BM;
      const int row = m0 + q * 32 + lane;  // global row owned by this thread
      const uint32_t t_acc = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);

      const bool rs_tile = COMM && cp.scatter == 1;
      const int rs_dst = rs_tile ? m0 / cp.rows_per_src : 0;
      const bool own_tile = rs_tile && rs_dst == cp.rank;
      if (own_tile && !own_ready) {
        // partial products of the other ranks for my rows: they were computed before those ranks' own rows
        int w = 1;
        if (lane < cp.world && lane != cp.rank)
          w = flag_wait_ge(cp.sflags[cp.rank] + kMaxRanks + lane, cp.out_target, wait_limit, abort_word);
        if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
        own_ready = true;
      }
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
            if (COMM && own_tile) {
              const long long lrow = row - static_cast<long long>(cp.rank) * cp.rows_per_src;
              for (int sr = 1; sr < cp.world; ++sr) {
                int src = cp.rank + sr;
                if (src >= cp.world) src -= cp.world;
                const __nv_bfloat16* srow = cp.sc_dst[cp.rank] + src * cp.sc_slot_stride + lrow * cp.sc_ld + col0;
#pragma unroll
                for (int j4 = 0; j4 < 4; ++j4) {
                  if (col0 + j4 * 8 < p.N) {
                    const uint4 u = __ldcg(reinterpret_cast<const uint4*>(srow + j4 * 8));
                    const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z),
                                 f3 = unpack_bf16x2(u.w);
                    v[j4 * 8 + 0] += f0.x; v[j4 * 8 + 1] += f0.y; v[j4 * 8 + 2] += f1.x; v[j4 * 8 + 3] += f1.y;
                    v[j4 * 8 + 4] += f2.x; v[j4 * 8 + 5] += f2.y; v[j4 * 8 + 6] += f3.x; v[j4 * 8 + 7] += f3.y;
                  }
                }
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
          if (COMM && cp.scatter) {
            // peer stores straight from the staged slab: 8 lanes cover one 128-byte row segment
            __syncwarp();
            const int r0 = m0 + q * 32;
            const int ccol = n0 + c64 * 64;
            int dst_lo, ndst, col_base;
            long long row_base, slot_off, dld = cp.sc_ld;
            __nv_bfloat16* own_out = nullptr;
            if (cp.scatter == 1) {
              dst_lo = rs_dst;
              ndst = 1;
              col_base = ccol;
              row_base = r0 - static_cast<long long>(dst_lo) * cp.rows_per_src;
              slot_off = cp.rank * cp.sc_slot_stride;
              if (own_tile) {  // already summed: this is the result
                own_out = cp.reduce_out;
                dld = cp.reduce_ld;
              } else if (!((sc_open >> dst_lo) & 1u)) {
                int w = 1;
                if (lane == 0) w = flag_wait_ge(cp.sflags[cp.rank] + 2 * kMaxRanks + dst_lo, cp.sc_done_target, wait_limit, abort_word);
                if (__shfl_sync(0xffffffffu, w, 0) == 0) { ok = false; break; }
                sc_open |= 1u << dst_lo;
              }
            } else {
              const int chunk = ccol >> 6;
              const bool live = ccol < p.N;  // the last tile may hang over the end of the table
              dst_lo = live ? cp.chunk_dst[chunk] : 0;
              ndst = live ? cp.chunk_ndst[chunk] : 0;
              col_base = live ? cp.chunk_col[chunk] : 0;
              row_base = cp.sc_row_off + r0;
              slot_off = 0;
            }
            for (int dd = 0; dd < ndst; ++dd) {
              __nv_bfloat16* dbase = own_out != nullptr ? own_out + col_base : cp.sc_dst[dst_lo + dd] + slot_off + col_base;
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int rr = i * 4 + (lane >> 3);
                const int ch = lane & 7;
                if (r0 + rr < p.M && ccol + ch * 8 < p.N) {
                  const uint4 val = *reinterpret_cast<const uint4*>(slab + rr * 128 + ((ch ^ (rr & 7)) * 16));
                  *reinterpret_cast<uint4*>(dbase + (row_base + rr) * dld + ch * 8) = val;
                }
              }
            }
            __syncwarp();
          } else {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              if (p.group_k) tma_store_3d(&tmC, slab, n0 + c64 * 64, m0 + q * 32, ex);
              else tma_store_2d(&tmC, slab, n0 + c64 * 64, m0 + q * 32);
              tma_store_commit();
            }
          }
          buf ^= 1;
        }
        if (!ok) break;
        if (rs_tile && !own_tile) {
          // this warp's part of the tile is on its way: count it on the destination
          __syncwarp();
          if (lane == 0) {
            flag_add_release(cp.sflags[rs_dst] + kMaxRanks + cp.rank, 1u);
          }
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
    if (COMM && cp.scatter == 2) {
      // every tile of this CTA has been stored: tell all destinations
      bar_sync_named(2, kEpiWarps * 32);
      if (warp == 4 && lane < cp.world && !*abort_word) {
        flag_add_release(cp.sflags[lane] + kMaxRanks + cp.rank, 1u);
      }
    }
  }

  // ------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (COMM) {
    // wait for what the other ranks sent here
    if (static_cast<int>(threadIdx.x) < cp.world) {
      // (mode 1 counts only what other ranks sent: this rank's own rows never pass through a slot)
      if (cp.scatter == 2 || (cp.scatter == 1 && static_cast<int>(threadIdx.x) != cp.rank))
        flag_wait_ge(cp.sflags[cp.rank] + kMaxRanks + threadIdx.x, cp.out_target, wait_limit, abort_word);
      if (cp.push && cp.wait_mode == 0) flag_wait_ge(cp.pflags[cp.rank] + threadIdx.x, cp.in_target, wait_limit, abort_word);
    }
    __syncthreads();
    __syncthreads();
    if (tracing && threadIdx.x == 0) cp.trace[5] = global_ns();
    // this rank no longer reads its gather buffer / its slots: writers of the next call may proceed
    if (static_cast<int>(threadIdx.x) < cp.world && !*abort_word) {
      __threadfence_system();
      if (cp.scatter == 1) flag_add_release(cp.sflags[threadIdx.x] + 2 * kMaxRanks + cp.rank, 1u);
    }
  }
  if (*abort_word) {
    // give copies still in flight time to land before shared memory is released
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    if (threadIdx.x == 0 && p.status != nullptr) atomicExch(p.status, kStatusBarrierTimeout);
  }
  __syncthreads();
  if (warp == 2 && !push_cta) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace b200

#include "gemm2_sm100.cuh"

namespace b200 {

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
static int g_group_m = 8;

template <int EPI, int COMM = 0>
static int launch(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tB2, const CUtensorMap& tC,
                  const CUtensorMap& tC2, const CUtensorMap& tC3, const GemmParams& p, int max_ctas,
                  cudaStream_t stream, const CommParams* comm = nullptr, int* launched = nullptr) {
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<EPI, COMM>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
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
  CommParams cp{};
  if (comm != nullptr) {
    // arrival counters grow by one per (pushing) CTA and call on every rank (all ranks launch the same grid)
    cp = *comm;
    if (cp.push_ctas > 0) {
      // dedicated push CTAs ride on top of the compute CTAs
      if (cp.push_ctas > g_num_sms / 2) cp.push_ctas = g_num_sms / 2;
      if (ctas > g_num_sms - cp.push_ctas) ctas = g_num_sms - cp.push_ctas;
      ctas += cp.push_ctas;
    }
    cp.in_target += static_cast<uint32_t>(cp.in_inc > 0 ? cp.in_inc : (cp.push_ctas > 0 ? cp.push_ctas : ctas));
    cp.out_target += static_cast<uint32_t>(cp.scatter == 1 ? cp.out_inc_tiles : ctas - cp.push_ctas);
    cp.push_done_target += static_cast<uint32_t>(ctas);
  }
  if (launched != nullptr) *launched = ctas;
  GemmParams pp = p;
  if (pp.group_m <= 0) pp.group_m = g_group_m;
  gemm_bf16_kernel<EPI, COMM><<<ctas, kThreads, kSmemBytes, stream>>>(tA, tB, tB2, tC, tC2, tC3, pp, cp);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// 0: one-CTA tiles only; 1: CTA-pair tiles wherever the shape allows (default)
static int g_pair_mode = 1;
static int g_pair_clusters = -1;

template <int EPI>
static int max_pair_clusters() {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(2, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = kSmem2Bytes;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, gemm2_bf16_kernel<EPI>, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

// One 256 x 256 tile per CTA pair; p.n_tiles_m counts 256-row blocks here.
template <int EPI>
static int launch2(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tB2, const CUtensorMap& tC,
                   const CUtensorMap& tC2, const CUtensorMap& tC3, const GemmParams& p, int max_ctas,
                   cudaStream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm2_bf16_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem2Bytes);
    if (e != cudaSuccess) return -3;
    attr_set = true;
  }
  if (g_pair_clusters < 0) {
    // the pairs are persistent: launch no more than can be resident at once
    g_pair_clusters = max_pair_clusters<EPI>();
    if (g_pair_clusters <= 0) return -5;
  }
  int pairs = g_pair_clusters;
  if (max_ctas > 0 && max_ctas / 2 < pairs) pairs = max_ctas / 2 > 0 ? max_ctas / 2 : 1;
  const int tiles = p.n_tiles_m * p.n_tiles_n;
  if (tiles < pairs) pairs = tiles;
  if (pairs <= 0) return 0;
  GemmParams pp = p;
  if (pp.group_m <= 0) pp.group_m = g_group_m;
  gemm2_bf16_kernel<EPI><<<2 * pairs, kThreads, kSmem2Bytes, stream>>>(tA, tB, tB2, tC, tC2, tC3, pp);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

static bool pair_shape_ok(int M, int N) { return g_pair_mode != 0 && M > 128 && N >= 128; }

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
  if (pair_shape_ok(M, N) && (!symmetric || M == N)) {
    // CTA-pair tiles: every CTA stages 128 rows of each operand
    if (a3d && make_map_mn3d(&tA, A, K, M, lda, 2) != 0) a3d = 0;
    if (b3d && make_map_mn3d(&tB, B, K, N, ldb, 2) != 0) b3d = 0;
    if (!a_mn_major) rc |= make_map(&tA, A, M, K, lda, BK, 128, true);
    else if (!a3d) rc |= make_map(&tA, A, K, M, lda, 64, BK, true);
    if (!b_mn_major) rc |= make_map(&tB, B, N, K, ldb, BK, 128, true);
    else if (!b3d) rc |= make_map(&tB, B, K, N, ldb, 64, BK, true);
    rc |= make_map(&tC, C, M, N, ldc, 64, 32, true);
    if (rc != 0) return rc;
    GemmParams p{};
    p.M = M; p.N = N; p.K = K;
    p.a_mn_major = a_mn_major; p.b_mn_major = b_mn_major;
    p.a_mn3d = a3d; p.b_mn3d = b3d;
    p.alpha = alpha; p.beta = beta;
    p.bias = symmetric ? nullptr : static_cast<const __nv_bfloat16*>(bias);
    p.cin = static_cast<const __nv_bfloat16*>(cin);
    p.ldcin = ldcin;
    p.n_tiles_m = (M + kTile2M - 1) / kTile2M;
    p.n_tiles_n = (N + BN - 1) / BN;
    p.status = status;
    if (symmetric) {
      p.cmirror = static_cast<__nv_bfloat16*>(C);
      p.ldc = ldc;
      return launch2<EPI_SYMM>(tA, tB, tB, tC, tC, tC, p, max_ctas, stream);
    }
    return launch2<EPI_PLAIN>(tA, tB, tB, tC, tC, tC, p, max_ctas, stream);
  }
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

// GEMM with fused collective parts (see CommParams).  `ca` is a flat int64 record:
//  [0] rank [1] world [2] wait limit in ms
//  [3] push [4] k-block source table [6] rows between destination blocks [7] push_dst_ld [8] push_dst_off
//  [9] push_rows [10] segments [11..13] source matrix [14..16] destination column [17..19] columns and
//  [73..75] source row stride of each segment
//  [20] arrive_in counter before this call [21] start handshake on the gather buffer [22] done counter before
//  this call [24..31] destination buffer of every rank [32..39] flag block of every rank
//  [40] wait mode [41] rows per source [42] k per source [43] m rotation (blocks) [44] k rotation (blocks)
//  [45] scatter mode [46] sc_ld [47] slot stride [48] chunk_dst [49] chunk_col [50] chunk_ndst [51] row offset
//  [52] arrive_out counter before this call [53] done counter to wait for [54] reduce_out [55] reduce_ld
//  [56..63] scatter buffer of every rank [64..71] its flag block on every rank [72] max CTAs
//  [76] tiles of this rank's own rows read the pushed matrix itself (all-gather mode)
//  [77] optional device buffer of six u64 for CTA 0's timeline (see CommParams::trace)
//  [80] > 0: the blocks are copied outside the kernel (copy engines) and arrive_in grows by this per call;
//       the segment fields then only describe this rank's own block for [76]
//  [79] epilogue warps join the copy (1) or only warps 2 and 3 copy next to the tiles (0)
//  [78] number of dedicated push CTAs (all-gather and re-gather pushes; 0 = push from warps 2..7 of every CTA)
// A is K-major; B is [N,K] or, with b_mn_major, [K,N].  With a scatter mode C is not written and may be
// null.  Returns the number of CTAs launched (every flag counter of this call grows by that much on
// every rank) or a negative error code.
int b200_gemm_comm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                        int b_mn_major, float alpha, const void* bias, const long long* ca, int* status,
                        cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return -10;
  if ((lda | ldb) & 7) return -10;
  CommParams cp{};
  cp.rank = static_cast<int>(ca[0]);
  cp.world = static_cast<int>(ca[1]);
  if (cp.world < 1 || cp.world > kMaxRanks || cp.rank < 0 || cp.rank >= cp.world) return -12;
  cp.wait_cycles = ca[2] * 1900000LL;
  cp.push = static_cast<int>(ca[3]);
  cp.kb_src = reinterpret_cast<const int*>(ca[4]);
  cp.push_block_rows = ca[6]; cp.push_dst_ld = ca[7]; cp.push_dst_off = ca[8];
  cp.push_rows = static_cast<int>(ca[9]);
  cp.push_nseg = static_cast<int>(ca[10]);
  if (cp.push && (cp.push_nseg < 1 || cp.push_nseg > kMaxPushSeg)) return -12;
  for (int i = 0; i < kMaxPushSeg; ++i) {
    cp.seg_src[i] = reinterpret_cast<const __nv_bfloat16*>(ca[11 + i]);
    cp.seg_dst_col[i] = static_cast<int>(ca[14 + i]);
    cp.seg_cols[i] = static_cast<int>(ca[17 + i]);
    cp.seg_src_ld[i] = ca[73 + i];
    if (cp.push && i < cp.push_nseg &&
        (((cp.seg_dst_col[i] | cp.seg_cols[i] | cp.seg_src_ld[i]) & 7) || (ca[11 + i] & 15))) return -10;
  }
  if (cp.push && ((cp.push_dst_ld | cp.push_dst_off) & 7)) return -10;
  cp.in_target = static_cast<uint32_t>(ca[20]);
  cp.push_done_wait = static_cast<int>(ca[21]);
  cp.push_done_target = static_cast<uint32_t>(ca[22]);
  for (int r = 0; r < kMaxRanks; ++r) {
    cp.push_dst[r] = reinterpret_cast<__nv_bfloat16*>(ca[24 + r]);
    cp.pflags[r] = reinterpret_cast<uint32_t*>(ca[32 + r]);
    cp.sc_dst[r] = reinterpret_cast<__nv_bfloat16*>(ca[56 + r]);
    cp.sflags[r] = reinterpret_cast<uint32_t*>(ca[64 + r]);
  }
  cp.wait_mode = static_cast<int>(ca[40]);
  cp.rows_per_src = static_cast<int>(ca[41]);
  cp.k_per_src = static_cast<int>(ca[42]);
  cp.m_rot = static_cast<int>(ca[43]);
  cp.k_rot = static_cast<int>(ca[44]);
  cp.scatter = static_cast<int>(ca[45]);
  cp.sc_ld = ca[46]; cp.sc_slot_stride = ca[47];
  cp.chunk_dst = reinterpret_cast<const int*>(ca[48]);
  cp.chunk_col = reinterpret_cast<const int*>(ca[49]);
  cp.chunk_ndst = reinterpret_cast<const int*>(ca[50]);
  cp.sc_row_off = static_cast<int>(ca[51]);
  cp.out_target = static_cast<uint32_t>(ca[52]);
  cp.sc_done_target = static_cast<uint32_t>(ca[53]);
  cp.reduce_out = reinterpret_cast<__nv_bfloat16*>(ca[54]);
  cp.reduce_ld = ca[55];
  const int max_ctas = static_cast<int>(ca[72]);
  cp.own_direct = static_cast<int>(ca[76]);
  cp.trace = reinterpret_cast<unsigned long long*>(ca[77]);
  cp.push_ctas = cp.push && cp.wait_mode != 2 ? static_cast<int>(ca[78]) : 0;
  if (cp.push_ctas < 0) cp.push_ctas = 0;
  cp.push_wide = static_cast<int>(ca[79]);
  cp.in_inc = static_cast<int>(ca[80]);
  cp.out_inc_tiles = 4 * (cp.rows_per_src > 0 ? cp.rows_per_src / BM : 0) * ((N + BN - 1) / BN);
  const int tiles_m = (M + BM - 1) / BM, n_kb = (K + BK - 1) / BK;
  // row blocks / k-ranges of one source must be whole tiles, or a tile would mix sources
  if ((cp.wait_mode == 1 || cp.scatter == 1) && (cp.rows_per_src % BM != 0 || cp.rows_per_src * cp.world != M)) return -13;
  if (cp.wait_mode == 2 && cp.kb_src == nullptr && (cp.k_per_src % BK != 0 || cp.k_per_src * cp.world != K)) return -13;
  if (cp.m_rot < 0 || cp.m_rot >= tiles_m || cp.k_rot < 0 || cp.k_rot >= n_kb) return -13;
  if (cp.scatter && ((cp.sc_ld | cp.sc_slot_stride | cp.reduce_ld) & 7 || (N & 7))) return -10;
  if (cp.scatter == 0 && (C == nullptr || (ldc & 7))) return -10;
  CUtensorMap tA, tB, tC, tOwn;
  int rc = make_map(&tA, A, M, K, lda, BK, BM, true);
  if (!b_mn_major) rc |= make_map(&tB, B, N, K, ldb, BK, BN, true);
  else rc |= make_map(&tB, B, K, N, ldb, 64, BK, true);
  if (cp.own_direct) {
    // tiles of this rank's own rows read the matrix that is being pushed, not its copy
    if (!(cp.push_nseg == 1 && (cp.wait_mode == 1 || cp.wait_mode == 2))) return -13;
    if (cp.wait_mode == 1) {
      if (cp.seg_cols[0] != K) return -13;
      rc |= make_map(&tOwn, cp.seg_src[0], cp.push_rows, K, cp.seg_src_ld[0], BK, BM, true);
    } else {
      // source [world * rows, k_per_src]: rows of block r feed rank r; this rank reads its own block
      if (cp.kb_src != nullptr || cp.seg_cols[0] != cp.k_per_src) return -13;
      rc |= make_map(&tOwn, cp.seg_src[0], static_cast<uint64_t>(cp.push_block_rows) * cp.world, cp.k_per_src,
                     cp.seg_src_ld[0], BK, BM, true);
    }
  } else {
    tOwn = tB;
  }
  // the C map is unused by a scattering epilogue; describe A so that the encode still succeeds
  if (cp.scatter) rc |= make_map(&tC, A, M, K, lda, 64, 32, true);
  else rc |= make_map(&tC, C, M, N, ldc, 64, 32, true);
  if (rc != 0) return rc;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.b_mn_major = b_mn_major;
  p.alpha = alpha;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.n_tiles_m = tiles_m;
  p.n_tiles_n = (N + BN - 1) / BN;
  p.status = status;
  int launched = 0;
  rc = launch<EPI_PLAIN, 1>(tA, tB, tOwn, tC, tC, tC, p, max_ctas, stream, &cp, &launched);
  return rc != 0 ? rc : launched;
}

// H = silu(X Wg^T) * (X Wu^T); optionally also writes G and U.  X [M,K], Wg/Wu [I,K].
int b200_gemm_swiglu_bf16(const void* X, const void* Wg, const void* Wu, void* H, void* G, void* U, int M, int I,
                          int K, int ldx, int ldw, int ldh, int store_gu, int* status, cudaStream_t stream) {
  if (M <= 0 || I <= 0 || K <= 0) return 0;
  if ((ldx | ldw | ldh) & 7) return -10;
  CUtensorMap tA, tB, tB2, tC, tC2, tC3;
  int rc = 0;
  const bool pair = pair_shape_ok(M, I);
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
  p.n_tiles_m = pair ? (M + kTile2M - 1) / kTile2M : (M + BM - 1) / BM;
  p.n_tiles_n = (I + 127) / 128;
  p.store_gu = store_gu;
  p.status = status;
  if (pair) return launch2<EPI_SWIGLU>(tA, tB, tB2, tC, tC2, tC3, p, 0, stream);
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
  const bool pair = pair_shape_ok(M, N);
  rc |= make_map(&tA, X, M, K, ldx, BK, BM, true);
  rc |= make_map(&tB, W, N, K, ldw, BK, pair ? 128 : BN, true);
  rc |= make_map(&tC, logits, M, N, ldc, 64, 32, true);
  if (rc != 0) return rc;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.alpha = alpha;
  p.stats = static_cast<float2*>(stats);
  p.n_tiles_m = pair ? (M + kTile2M - 1) / kTile2M : (M + BM - 1) / BM;
  p.n_tiles_n = (N + BN - 1) / BN;
  p.status = status;
  if (pair) return launch2<EPI_STATS>(tA, tB, tB, tC, tC, tC, p, 0, stream);
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

// Tuning knob: how many m-blocks share a sweep over N (default 8).
int b200_gemm_set_group_m(int g) {
  if (g >= 1 && g <= 1024) g_group_m = g;
  return g_group_m;
}

int b200_gemm_tile_n() { return BN; }

// CTA pairs that a pair-kernel launch uses at most (-1 before the first such launch).
int b200_gemm_pair_clusters() { return g_pair_clusters; }

// 1 (default): 256 x 256 tiles on CTA pairs wherever the shape allows; 0: one-CTA 128 x 256 tiles only.
int b200_gemm_set_pair_mode(int on) {
  if (on == 0 || on == 1) g_pair_mode = on;
  return g_pair_mode;
}

}  // extern "C"
