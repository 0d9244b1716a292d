// Mixture-of-experts routing and token movement for sm_100a.
//
//  * router: softmax over experts, top-k, optional renormalisation, per-expert histogram -
//    one warp per token, everything in registers;
//  * sort-free, deterministic permutation: per-expert padded row ranges (multiples of the
//    GEMM's 128-row tile, so every tile of the grouped GEMM belongs to exactly one expert),
//    destination row of every (token, slot) pair in token order, inverse maps, and the
//    tile -> expert table the grouped GEMM's scheduler reads from device memory.  No host
//    round trip: all shapes are worst-case bounded;
//  * combine: out[t] = sum_j w[t,j] * src[row_of[t,j]] (also the backward of the dispatch
//    gather), its gradients, and the SwiGLU backward on the [rows, 2I] gate|up layout.
//
// Reference behaviour: eager softmax/topk/histc/argsort/index_select/scatter_add in
// src/lmms_engine/models/qwen3_moe/qwen3_moe_ops.py:257-296 and the permute helpers of
// src/lmms_engine/parallel/expert_parallel/utils.py:54-77 (both with host syncs).
#include "common.cuh"

namespace b200 {

typedef __nv_bfloat16 bf16;
constexpr int kTileRows = 128;

struct alignas(16) V8 {
  uint32_t w[4];
};

// ---------------------------------------------------------------------------- router
// logits [T, E] bf16 or fp32; E <= 256, E % 32 == 0, k <= 16.
template <typename LT>
__global__ void __launch_bounds__(256) moe_router_kernel(const LT* __restrict__ logits, float* __restrict__ probs,
                                                         int* __restrict__ topk_idx, float* __restrict__ topk_w,
                                                         int* __restrict__ counts, int T, int E, int k, int renorm) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int per = E / 32;  // <= 8 values per lane, expert index = lane + 32*i
  for (int t = blockIdx.x * wpb + (threadIdx.x >> 5); t < T; t += gridDim.x * wpb) {
    float v[8];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      v[i] = (i < per) ? static_cast<float>(logits[static_cast<size_t>(t) * E + lane + 32 * i]) : -INFINITY;
      mx = fmaxf(mx, v[i]);
    }
    mx = warp_max(mx);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      v[i] = (i < per) ? __expf(v[i] - mx) : 0.f;
      s += v[i];
    }
    s = warp_sum(s);
    const float inv = 1.f / s;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      v[i] *= inv;
      if (i < per) probs[static_cast<size_t>(t) * E + lane + 32 * i] = v[i];
      // non-finite logits (an upstream overflow) must not derail the selection below: every round has to find an
      // expert index inside [0, E), the histogram and the permutation index memory with it
      if (!(v[i] >= 0.f)) v[i] = 0.f;
    }
    // k rounds of warp arg-max; ties go to the lower expert index (like torch.topk on CUDA
    // is not guaranteed to; the engine's own reference uses the same rule)
    float sel_sum = 0.f;
    float my_w = 0.f;
    int my_e = 0;
    for (int j = 0; j < k; ++j) {
      float best = -1.f;
      int best_e = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int e = lane + 32 * i;
        if (i < per && (v[i] > best || (v[i] == best && e < best_e))) {
          best = v[i];
          best_e = e;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
        if (ob > best || (ob == best && oe < best_e)) {
          best = ob;
          best_e = oe;
        }
      }
      if ((best_e & 31) == lane) v[best_e >> 5] = -2.f;  // remove from further rounds
      sel_sum += best;
      if (lane == j) {
        my_w = best;
        my_e = best_e;
      }
    }
    if (lane < k) {
      topk_idx[static_cast<size_t>(t) * k + lane] = my_e;
      topk_w[static_cast<size_t>(t) * k + lane] = renorm ? my_w / sel_sum : my_w;
      atomicAdd(&counts[my_e], 1);
    }
  }
}

// ---------------------------------------------------------------------------- permutation
// Single CTA: padded exclusive scan of the counts, tile -> expert table.
// expert_start[e] (e = 0..E) in rows; tile_expert[i] = expert of row tile i or -1.
__global__ void moe_offsets_kernel(const int* __restrict__ counts, int* __restrict__ expert_start,
                                   int* __restrict__ tile_expert, int E, int max_tiles) {
  __shared__ int start[257];
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      start[e] = acc;
      acc += (counts[e] + kTileRows - 1) / kTileRows * kTileRows;
    }
    start[E] = acc;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) expert_start[e] = start[e];
  for (int i = threadIdx.x; i < max_tiles; i += blockDim.x) {
    const int row = i * kTileRows;
    int ex = -1;
    if (row < start[E]) {
      int lo = 0, hi = E;  // last e with start[e] <= row
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (start[mid] <= row) lo = mid; else hi = mid;
      }
      ex = lo;
    }
    tile_expert[i] = ex;
  }
}

// Debug build: rows computed from the counts are checked against the size of the row tables (counts that do not belong
// to these top-k indices would otherwise write past them); the flag is read and cleared by b200_moe_debug_bad_index().
#ifdef B200_DEBUG_BOUNDS
__device__ int g_debug_bad_index = 0;
#define MOE_DBG_STATUS (&g_debug_bad_index)
#else
#define MOE_DBG_STATUS nullptr
#endif

// One CTA per expert: destination rows in token order (stable, deterministic).
__global__ void __launch_bounds__(256) moe_rows_kernel(const int* __restrict__ topk_idx, const float* __restrict__ topk_w,
                                                       const int* __restrict__ expert_start, int* __restrict__ row_of,
                                                       int64_t* __restrict__ token_of_row, float* __restrict__ weight_of_row,
                                                       int T, int k, long max_rows) {
  __shared__ int warp_tot[8];
  __shared__ int base;
  const int e = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) base = expert_start[e];
  __syncthreads();
  for (int t0 = 0; t0 < T; t0 += blockDim.x) {
    const int t = t0 + threadIdx.x;
    int slot = -1;
    if (t < T) {
      for (int j = 0; j < k; ++j)
        if (topk_idx[static_cast<size_t>(t) * k + j] == e) slot = j;
    }
    const unsigned ballot = __ballot_sync(0xffffffffu, slot >= 0);
    const int before = __popc(ballot & ((1u << lane) - 1));
    if (lane == 0) warp_tot[warp] = __popc(ballot);
    __syncthreads();
    int wbase = 0;
    for (int w = 0; w < warp; ++w) wbase += warp_tot[w];
    int total = 0;
    for (int w = 0; w < (blockDim.x >> 5); ++w) total += warp_tot[w];
    if (slot >= 0 && B200_DBG_INDEX(base + wbase + before, max_rows, MOE_DBG_STATUS)) {
      const int row = base + wbase + before;
      row_of[static_cast<size_t>(t) * k + slot] = row;
      token_of_row[row] = t;
      weight_of_row[row] = topk_w[static_cast<size_t>(t) * k + slot];
    }
    __syncthreads();
    if (threadIdx.x == 0) base += total;
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------- combine & friends
// out[t, :] = sum_j (w ? w[t,j] : 1) * src[row_of[t,j], :]
__global__ void moe_combine_kernel(const bf16* __restrict__ src, const int* __restrict__ row_of,
                                   const float* __restrict__ w, bf16* __restrict__ out, int T, int k, int H,
                                   long n_src, int* status) {
  const int vec = H / 8;
  const long total = static_cast<long>(T) * vec;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long t = i / vec;
    const int c = (i - t * vec) * 8;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < k; ++j) {
      const int row = row_of[t * k + j];
      if (row < 0 || !index_in_bounds(row, n_src, status)) continue;
      const float wt = w != nullptr ? w[t * k + j] : 1.f;
      const V8 v = *reinterpret_cast<const V8*>(src + static_cast<size_t>(row) * H + c);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = unpack_bf16x2(v.w[q]);
        acc[2 * q] += wt * f.x;
        acc[2 * q + 1] += wt * f.y;
      }
    }
    V8 o;
#pragma unroll
    for (int q = 0; q < 4; ++q) o.w[q] = pack_bf16x2(acc[2 * q], acc[2 * q + 1]);
    *reinterpret_cast<V8*>(out + t * H + c) = o;
  }
}

// dsrc[row, :] = weight_of_row[row] * dout[token_of_row[row], :]   (zero for padding rows)
__global__ void moe_combine_bwd_src_kernel(const bf16* __restrict__ dout, const int64_t* __restrict__ token_of_row,
                                           const float* __restrict__ weight_of_row, bf16* __restrict__ dsrc,
                                           long rows, int H, long n_tok, int* status) {
  const int vec = H / 8;
  const long total = rows * vec;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long r = i / vec;
    const int c = (i - r * vec) * 8;
    const int64_t t = token_of_row[r];
    V8 o;
    o.w[0] = o.w[1] = o.w[2] = o.w[3] = 0u;
    if (t >= 0 && index_in_bounds(t, n_tok, status)) {
      const float wt = weight_of_row != nullptr ? weight_of_row[r] : 1.f;
      const V8 v = *reinterpret_cast<const V8*>(dout + t * H + c);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = unpack_bf16x2(v.w[q]);
        o.w[q] = pack_bf16x2(wt * f.x, wt * f.y);
      }
    }
    *reinterpret_cast<V8*>(dsrc + r * H + c) = o;
  }
}

// dw[t, j] = <dout[t, :], src[row_of[t, j], :]>   (one warp per (t, j))
__global__ void moe_combine_bwd_w_kernel(const bf16* __restrict__ dout, const bf16* __restrict__ src,
                                         const int* __restrict__ row_of, float* __restrict__ dw, long pairs, int k,
                                         int H, long n_src, int* status) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (long p = blockIdx.x * static_cast<long>(wpb) + (threadIdx.x >> 5); p < pairs;
       p += static_cast<long>(gridDim.x) * wpb) {
    const long t = p / k;
    const int row = row_of[p];
    float acc = 0.f;
    const bool ok = row >= 0 && index_in_bounds(row, n_src, status);  // uniform over the warp
    for (int c = lane * 8; ok && c < H; c += 256) {
      const V8 a = *reinterpret_cast<const V8*>(dout + t * H + c);
      const V8 b = *reinterpret_cast<const V8*>(src + static_cast<size_t>(row) * H + c);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 fa = unpack_bf16x2(a.w[q]), fb = unpack_bf16x2(b.w[q]);
        acc += fa.x * fb.x + fa.y * fb.y;
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) dw[p] = acc;
  }
}

// The expert side of the combine's backward on rows that are already in place (expert parallelism: the gradient rows
// arrived in the staging area together with their router weight):
//   d_y[r, :] = w[r] * g[r, :]      dot[r] = <g[r, :], y[r, :]>      (one warp per row, one pass over g and y)
__global__ void moe_row_scale_dot_kernel(const bf16* __restrict__ g, long ldg, const bf16* __restrict__ y,
                                         const float* __restrict__ w, bf16* __restrict__ d_y, float* __restrict__ dot,
                                         long rows, int H) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (long r = blockIdx.x * static_cast<long>(wpb) + (threadIdx.x >> 5); r < rows;
       r += static_cast<long>(gridDim.x) * wpb) {
    const float wt = w[r];
    float acc = 0.f;
    for (int c = lane * 8; c < H; c += 256) {
      const V8 a = *reinterpret_cast<const V8*>(g + r * ldg + c);
      const V8 b = *reinterpret_cast<const V8*>(y + r * static_cast<long>(H) + c);
      V8 o;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 fa = unpack_bf16x2(a.w[q]), fb = unpack_bf16x2(b.w[q]);
        acc += fa.x * fb.x + fa.y * fb.y;
        o.w[q] = pack_bf16x2(wt * fa.x, wt * fa.y);
      }
      *reinterpret_cast<V8*>(d_y + r * static_cast<long>(H) + c) = o;
    }
    acc = warp_sum(acc);
    if (lane == 0) dot[r] = acc;
  }
}

// SwiGLU on the concatenated layout gu[rows, 2I] = [gate | up]:
// forward h = silu(g) * u; backward overwrites gu with [dg | du] given dh.
__global__ void swiglu_cat_fwd_kernel(const bf16* __restrict__ gu, bf16* __restrict__ h, long rows, int I) {
  const int vec = I / 8;
  const long total = rows * vec;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long r = i / vec;
    const int c = (i - r * vec) * 8;
    const V8 g = *reinterpret_cast<const V8*>(gu + r * 2 * I + c);
    const V8 u = *reinterpret_cast<const V8*>(gu + r * 2 * I + I + c);
    V8 o;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 fg = unpack_bf16x2(g.w[q]), fu = unpack_bf16x2(u.w[q]);
      o.w[q] = pack_bf16x2(fg.x / (1.f + __expf(-fg.x)) * fu.x, fg.y / (1.f + __expf(-fg.y)) * fu.y);
    }
    *reinterpret_cast<V8*>(h + r * I + c) = o;
  }
}
__global__ void swiglu_cat_bwd_kernel(const bf16* __restrict__ dh, bf16* gu, long rows, int I) {
  const int vec = I / 8;
  const long total = rows * vec;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long r = i / vec;
    const int c = (i - r * vec) * 8;
    const V8 g = *reinterpret_cast<const V8*>(gu + r * 2 * I + c);
    const V8 u = *reinterpret_cast<const V8*>(gu + r * 2 * I + I + c);
    const V8 d = *reinterpret_cast<const V8*>(dh + r * I + c);
    V8 og, ou;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 fg = unpack_bf16x2(g.w[q]), fu = unpack_bf16x2(u.w[q]), fd = unpack_bf16x2(d.w[q]);
      const float s0 = 1.f / (1.f + __expf(-fg.x)), s1 = 1.f / (1.f + __expf(-fg.y));
      const float si0 = fg.x * s0, si1 = fg.y * s1;
      ou.w[q] = pack_bf16x2(fd.x * si0, fd.y * si1);
      og.w[q] = pack_bf16x2(fd.x * fu.x * (s0 + si0 * (1.f - s0)), fd.y * fu.y * (s1 + si1 * (1.f - s1)));
    }
    *reinterpret_cast<V8*>(gu + r * 2 * I + c) = og;
    *reinterpret_cast<V8*>(gu + r * 2 * I + I + c) = ou;
  }
}

static int grid_for(long items, int threads) {
  long b = (items + threads - 1) / threads;
  if (b > 148 * 8) b = 148 * 8;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

}  // namespace b200

using namespace b200;
#define CHECK_LAUNCH() (cudaGetLastError() == cudaSuccess ? 0 : -4)

extern "C" {

int b200_moe_tile_rows() { return kTileRows; }

// counts must be zeroed by the caller (or is zeroed here when zero_counts != 0).
int b200_moe_router(const void* logits, int logits_fp32, void* probs, void* topk_idx, void* topk_w, void* counts, int T,
                    int E, int k, int renorm, int zero_counts, cudaStream_t st) {
  if (T <= 0) return 0;
  if (E % 32 || E > 256 || k > 16 || k > E) return -10;
  if (zero_counts) cudaMemsetAsync(counts, 0, sizeof(int) * E, st);
  const int blocks = grid_for(static_cast<long>(T) * 32, 256);
  if (logits_fp32)
    moe_router_kernel<float><<<blocks, 256, 0, st>>>((const float*)logits, (float*)probs, (int*)topk_idx,
                                                     (float*)topk_w, (int*)counts, T, E, k, renorm);
  else
    moe_router_kernel<bf16><<<blocks, 256, 0, st>>>((const bf16*)logits, (float*)probs, (int*)topk_idx, (float*)topk_w,
                                                    (int*)counts, T, E, k, renorm);
  return CHECK_LAUNCH();
}

// expert_start int32 [E+1]; tile_expert int32 [max_tiles]; row_of int32 [T*k];
// token_of_row int64 [max_rows] (set to -1 here); weight_of_row fp32 [max_rows].
int b200_moe_permute(const void* topk_idx, const void* topk_w, const void* counts, void* expert_start, void* tile_expert,
                     void* row_of, void* token_of_row, void* weight_of_row, int T, int E, int k, long max_rows,
                     cudaStream_t st) {
  if (T <= 0) return 0;
  if (E > 256) return -10;
  const int max_tiles = static_cast<int>(max_rows / kTileRows);
  cudaMemsetAsync(token_of_row, 0xFF, sizeof(int64_t) * max_rows, st);
  cudaMemsetAsync(weight_of_row, 0, sizeof(float) * max_rows, st);
  moe_offsets_kernel<<<1, 256, 0, st>>>((const int*)counts, (int*)expert_start, (int*)tile_expert, E, max_tiles);
  moe_rows_kernel<<<E, 256, 0, st>>>((const int*)topk_idx, (const float*)topk_w, (const int*)expert_start, (int*)row_of,
                                     (int64_t*)token_of_row, (float*)weight_of_row, T, k, max_rows);
  return CHECK_LAUNCH();
}

// Debug build: 1 if a computed row left its table since the last call (and clears the flag); -1 in the release build.
int b200_moe_debug_bad_index() {
#ifdef B200_DEBUG_BOUNDS
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_debug_bad_index, sizeof(int)) != cudaSuccess) return -2;
  cudaMemcpyToSymbol(g_debug_bad_index, &zero, sizeof(int));
  return v != 0;
#else
  return -1;
#endif
}

// n_src / n_tok: rows of the tensor that the routing table indexes; entries beyond it raise kStatusBadIndex in *status
// and contribute nothing.
int b200_moe_combine(const void* src, const void* row_of, const void* w, void* out, int T, int k, int H, long n_src,
                     void* status, cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 8) return -10;
  moe_combine_kernel<<<grid_for(static_cast<long>(T) * (H / 8), 256), 256, 0, st>>>(
      (const bf16*)src, (const int*)row_of, (const float*)w, (bf16*)out, T, k, H, n_src, (int*)status);
  return CHECK_LAUNCH();
}
int b200_moe_combine_bwd_src(const void* dout, const void* token_of_row, const void* weight_of_row, void* dsrc, long rows,
                             int H, long n_tok, void* status, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (H % 8) return -10;
  moe_combine_bwd_src_kernel<<<grid_for(rows * (H / 8), 256), 256, 0, st>>>(
      (const bf16*)dout, (const int64_t*)token_of_row, (const float*)weight_of_row, (bf16*)dsrc, rows, H, n_tok,
      (int*)status);
  return CHECK_LAUNCH();
}
int b200_moe_combine_bwd_w(const void* dout, const void* src, const void* row_of, void* dw, long pairs, int k, int H,
                           long n_src, void* status, cudaStream_t st) {
  if (pairs <= 0) return 0;
  if (H % 8) return -10;
  moe_combine_bwd_w_kernel<<<grid_for(pairs * 32, 256), 256, 0, st>>>((const bf16*)dout, (const bf16*)src,
                                                                      (const int*)row_of, (float*)dw, pairs, k, H, n_src,
                                                                      (int*)status);
  return CHECK_LAUNCH();
}
int b200_moe_row_scale_dot(const void* g, long ldg, const void* y, const void* w, void* d_y, void* dot, long rows, int H,
                           cudaStream_t st) {
  if (rows <= 0) return 0;
  if (H % 8 || ldg % 8) return -10;
  moe_row_scale_dot_kernel<<<grid_for(rows * 32, 256), 256, 0, st>>>((const bf16*)g, ldg, (const bf16*)y, (const float*)w,
                                                                     (bf16*)d_y, (float*)dot, rows, H);
  return CHECK_LAUNCH();
}
int b200_swiglu_cat_fwd(const void* gu, void* h, long rows, int I, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (I % 8) return -10;
  swiglu_cat_fwd_kernel<<<grid_for(rows * (I / 8), 256), 256, 0, st>>>((const bf16*)gu, (bf16*)h, rows, I);
  return CHECK_LAUNCH();
}
int b200_swiglu_cat_bwd(const void* dh, void* gu, long rows, int I, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (I % 8) return -10;
  swiglu_cat_bwd_kernel<<<grid_for(rows * (I / 8), 256), 256, 0, st>>>((const bf16*)dh, (bf16*)gu, rows, I);
  return CHECK_LAUNCH();
}

}  // extern "C"
