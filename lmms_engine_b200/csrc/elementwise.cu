// Bandwidth-bound kernels of the training step, written for sm_100a:
// RMSNorm / LayerNorm (+ residual add) forward and backward, rotary embedding
// (plain, multimodal-sectioned, multimodal-interleaved, vision 2-D all reduce to a
// per-token cos/sin table plus one apply kernel), SwiGLU, flat-buffer AdamW, Muon
// momentum / scale / update, EMA, gradient norm + clip, index gather/scatter for packed
// sequences, and the cross-entropy passes that follow the logits GEMM.
//
// All kernels use 16-byte vector accesses, grid-stride loops sized to the SM count and
// fp32 arithmetic on bf16 storage.  Reference behaviour: Liger RMSNorm / RoPE / SwiGLU
// (src/lmms_engine/models/qwen2/monkey_patch.py:47-118), torch.optim.AdamW
// (src/lmms_engine/train/fsdp2/fsdp2_trainer.py:202-209), the Muon update
// (src/lmms_engine/utils/muon_utils.py:159-183, 273-275), EMA
// (src/lmms_engine/utils/ema_utils.py:97-101) and foreach grad clipping
// (src/lmms_engine/utils/fsdp2_utils.py:250-289).
#include "common.cuh"

#include <cstdlib>

namespace b200 {

typedef __nv_bfloat16 bf16;

struct alignas(16) bf16x8 {
  uint32_t w[4];
};

__device__ __forceinline__ void load8(const bf16* p, float (&v)[8]) {
  bf16x8 u = *reinterpret_cast<const bf16x8*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = unpack_bf16x2(u.w[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void store8(bf16* p, const float (&v)[8]) {
  bf16x8 u;
#pragma unroll
  for (int i = 0; i < 4; ++i) u.w[i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<bf16x8*>(p) = u;
}

template <int kThreads>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < kThreads / 32) ? red[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

// ------------------------------------------------------------------ RMSNorm / LayerNorm forward
// One CTA per row (H >= 1024) keeps the row in registers: H <= kThreads * 8 * kVecPerThread.
// y = (x [+ res]) * rstd * (w + w_offset);  optional res_out = x + res;  LayerNorm when `ln`.
template <int kThreads, int kVec>
__global__ void __launch_bounds__(kThreads) norm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ res,
                                                            const bf16* __restrict__ w, const bf16* __restrict__ b,
                                                            bf16* __restrict__ y, bf16* __restrict__ res_out,
                                                            float* __restrict__ rstd_out, float* __restrict__ mean_out,
                                                            int rows, int H, float eps, float w_offset, int ln) {
  __shared__ float red[32];
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t base = static_cast<size_t>(row) * H;
    float v[kVec][8];
    float s = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
      const int c = (i * kThreads + threadIdx.x) * 8;
      if (c < H) {
        load8(x + base + c, v[i]);
        if (res != nullptr) {
          float r[8];
          load8(res + base + c, r);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] += r[j];
          // round the sum to bf16 so that the normalised row matches the stored residual stream
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] = __bfloat162float(__float2bfloat16(v[i][j]));
          if (res_out != nullptr) store8(res_out + base + c, v[i]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          s += v[i][j];
          s2 += v[i][j] * v[i][j];
        }
      }
    }
    float mean = 0.f;
    if (ln) {
      mean = block_sum<kThreads>(s, red) / H;
      float var = 0.f;
#pragma unroll
      for (int i = 0; i < kVec; ++i) {
        const int c = (i * kThreads + threadIdx.x) * 8;
        if (c < H) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float d = v[i][j] - mean;
            var += d * d;
          }
        }
      }
      s2 = block_sum<kThreads>(var, red);
    } else {
      s2 = block_sum<kThreads>(s2, red);
    }
    const float rstd = rsqrtf(s2 / H + eps);
    if (threadIdx.x == 0) {
      rstd_out[row] = rstd;
      if (ln && mean_out != nullptr) mean_out[row] = mean;
    }
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
      const int c = (i * kThreads + threadIdx.x) * 8;
      if (c < H) {
        float wv[8], o[8];
        load8(w + c, wv);
        float bv[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (b != nullptr) load8(b + c, bv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (v[i][j] - mean) * rstd * (wv[j] + w_offset) + bv[j];
        store8(y + base + c, o);
      }
    }
  }
}

// One warp per row for short rows (per-head QK-norm: H = 64..512, multiple of 8).
__global__ void __launch_bounds__(256) norm_fwd_warp_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                            bf16* __restrict__ y, float* __restrict__ rstd_out, int rows,
                                                            int H, float eps, float w_offset) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (int row = blockIdx.x * wpb + (threadIdx.x >> 5); row < rows; row += gridDim.x * wpb) {
    const size_t base = static_cast<size_t>(row) * H;
    float v[2][8];
    float s2 = 0.f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int c = (i * 32 + lane) * 8;
      if (c < H) {
        load8(x + base + c, v[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) s2 += v[i][j] * v[i][j];
      }
    }
    s2 = warp_sum(s2);
    const float rstd = rsqrtf(s2 / H + eps);
    if (lane == 0) rstd_out[row] = rstd;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int c = (i * 32 + lane) * 8;
      if (c < H) {
        float wv[8], o[8];
        load8(w + c, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = v[i][j] * rstd * (wv[j] + w_offset);
        store8(y + base + c, o);
      }
    }
  }
}

// ------------------------------------------------------------------ RMSNorm / LayerNorm backward
// dx = rstd * (g - xhat * mean(g * xhat) [- mean(g) for LN]) [+ dres_in], g = dy * (w + off)
// Partial dw (and db) are accumulated per CTA in registers over its rows and written to
// dw_part[blockIdx.x, H]; a second kernel reduces the partials.
template <int kThreads, int kVec>
__global__ void __launch_bounds__(kThreads)
norm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ w,
                const float* __restrict__ rstd_in, const float* __restrict__ mean_in, const bf16* __restrict__ dres_in,
                bf16* __restrict__ dx, float* __restrict__ dw_part, float* __restrict__ db_part, int rows, int H,
                float w_offset, int ln) {
  __shared__ float red[32];
  float dw[kVec][8], db[kVec][8];
#pragma unroll
  for (int i = 0; i < kVec; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dw[i][j] = 0.f, db[i][j] = 0.f;

  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t base = static_cast<size_t>(row) * H;
    const float rstd = rstd_in[row];
    const float mean = (ln && mean_in != nullptr) ? mean_in[row] : 0.f;
    float g[kVec][8], xh[kVec][8];
    float dot = 0.f, gsum = 0.f;
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
      const int c = (i * kThreads + threadIdx.x) * 8;
      if (c < H) {
        float dyv[8], xv[8], wv[8];
        load8(dy + base + c, dyv);
        load8(x + base + c, xv);
        load8(w + c, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xv[j] - mean) * rstd;
          g[i][j] = dyv[j] * (wv[j] + w_offset);
          dw[i][j] += dyv[j] * xh[i][j];
          db[i][j] += dyv[j];
          dot += g[i][j] * xh[i][j];
          gsum += g[i][j];
        }
      }
    }
    dot = block_sum<kThreads>(dot, red) / H;
    if (ln) gsum = block_sum<kThreads>(gsum, red) / H;
    else gsum = 0.f;
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
      const int c = (i * kThreads + threadIdx.x) * 8;
      if (c < H) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (g[i][j] - xh[i][j] * dot - gsum);
        if (dres_in != nullptr) {
          float r[8];
          load8(dres_in + base + c, r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        store8(dx + base + c, o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kVec; ++i) {
    const int c = (i * kThreads + threadIdx.x) * 8;
    if (c < H) {
      float* o = dw_part + static_cast<size_t>(blockIdx.x) * H + c;
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = dw[i][j];
      if (db_part != nullptr) {
        float* ob = db_part + static_cast<size_t>(blockIdx.x) * H + c;
#pragma unroll
        for (int j = 0; j < 8; ++j) ob[j] = db[i][j];
      }
    }
  }
}

__global__ void norm_bwd_warp_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                     const bf16* __restrict__ w, const float* __restrict__ rstd_in,
                                     bf16* __restrict__ dx, float* __restrict__ dw_part, int rows, int H,
                                     float w_offset) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int gw = blockIdx.x * wpb + (threadIdx.x >> 5);
  float dw[2][8];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dw[i][j] = 0.f;
  for (int row = gw; row < rows; row += gridDim.x * wpb) {
    const size_t base = static_cast<size_t>(row) * H;
    const float rstd = rstd_in[row];
    float g[2][8], xh[2][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int c = (i * 32 + lane) * 8;
      if (c < H) {
        float dyv[8], xv[8], wv[8];
        load8(dy + base + c, dyv);
        load8(x + base + c, xv);
        load8(w + c, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = xv[j] * rstd;
          g[i][j] = dyv[j] * (wv[j] + w_offset);
          dw[i][j] += dyv[j] * xh[i][j];
          dot += g[i][j] * xh[i][j];
        }
      }
    }
    dot = warp_sum(dot) / H;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int c = (i * 32 + lane) * 8;
      if (c < H) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (g[i][j] - xh[i][j] * dot);
        store8(dx + base + c, o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int c = (i * 32 + lane) * 8;
    if (c < H) {
      float* o = dw_part + static_cast<size_t>(gw) * H + c;
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = dw[i][j];
    }
  }
}

// RMSNorm backward for narrow rows (per-head norms: H = 64 / 128 / 256): LPR = H / 8 lanes hold a row, a warp works on
// 32 / LPR rows at once, a block of sixteen warps leaves ONE row of dw partials (summed over its warps in shared memory),
// so the grid can fill the machine within the same partials scratch.
template <int LPR>
__global__ void norm_bwd_narrow_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ w,
                                       const float* __restrict__ rstd_in, bf16* __restrict__ dx,
                                       float* __restrict__ dw_part, int rows, float w_offset) {
  constexpr int H = LPR * 8;
  constexpr int RPW = 32 / LPR;  // rows per warp and iteration
  __shared__ float red[16][H];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane / LPR, col = (lane % LPR) * 8;
  const int wpb = blockDim.x >> 5;
  float wv[8], dw[8];
  load8(w + col, wv);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    wv[j] += w_offset;
    dw[j] = 0.f;
  }
  for (long row0 = (static_cast<long>(blockIdx.x) * wpb + warp) * RPW; row0 < rows;
       row0 += static_cast<long>(gridDim.x) * wpb * RPW) {
    const long row = row0 + sub;
    const bool live = row < rows;
    float dyv[8], xv[8], g[8], xh[8];
    float dot = 0.f, rstd = 0.f;
    if (live) {
      const size_t base = static_cast<size_t>(row) * H + col;
      rstd = rstd_in[row];
      load8(dy + base, dyv);
      load8(x + base, xv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        xh[j] = xv[j] * rstd;
        g[j] = dyv[j] * wv[j];
        dw[j] += dyv[j] * xh[j];
        dot += g[j] * xh[j];
      }
    }
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    dot /= H;
    if (live) {
      float o8[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o8[j] = rstd * (g[j] - xh[j] * dot);
      store8(dx + static_cast<size_t>(row) * H + col, o8);
    }
  }
  // lanes that hold the same columns (one per row of the warp's group), then the block's warps
#pragma unroll
  for (int o = LPR; o < 32; o <<= 1)
#pragma unroll
    for (int j = 0; j < 8; ++j) dw[j] += __shfl_xor_sync(0xffffffffu, dw[j], o);
  if (sub == 0) {
#pragma unroll
    for (int j = 0; j < 8; ++j) red[warp][col + j] = dw[j];
  }
  __syncthreads();
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float acc = 0.f;
    for (int q = 0; q < wpb; ++q) acc += red[q][c];
    dw_part[static_cast<size_t>(blockIdx.x) * H + c] = acc;
  }
}

// out[c] = sum_p part[p, c]  (fp32 -> fp32, optionally accumulating into out)
__global__ void colsum_kernel(const float* __restrict__ part, float* __restrict__ out, int parts, int H,
                              int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float s = 0.f;
  for (int p = 0; p < parts; ++p) s += part[static_cast<size_t>(p) * H + c];
  out[c] = accumulate ? out[c] + s : s;
}

// ------------------------------------------------------------------ rotary embedding
// cos/sin tables [T, D] (fp32) from up to three position streams.
// mode 0: plain (pos[0]);  mode 1: sectioned M-RoPE (frequency i uses stream by section
// boundaries s0, s0+s1);   mode 2: interleaved M-RoPE (Qwen3-VL: frequency i uses stream
// i % 3 while i < 3*section[i % 3] for streams 1, 2; stream 0 otherwise).
__global__ void rope_table_kernel(const int64_t* __restrict__ pos, const float* __restrict__ inv_freq,
                                  float* __restrict__ cos_out, float* __restrict__ sin_out, int T, int half,
                                  int mode, int s0, int s1, int s2, float scaling) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= T * half) return;
  const int t = idx / half, i = idx - t * half;
  int stream = 0;
  if (mode == 1) {
    stream = (i < s0) ? 0 : (i < s0 + s1 ? 1 : 2);
  } else if (mode == 2) {
    const int m = i % 3;
    if (m == 1 && i < 3 * s1) stream = 1;
    else if (m == 2 && i < 3 * s2) stream = 2;
    else stream = 0;
  }
  const float ang = static_cast<float>(pos[static_cast<size_t>(stream) * T + t]) * inv_freq[i];
  float sn, cs;
  sincosf(ang, &sn, &cs);
  cs *= scaling;
  sn *= scaling;
  const size_t o = static_cast<size_t>(t) * 2 * half;
  cos_out[o + i] = cs;
  cos_out[o + half + i] = cs;
  sin_out[o + i] = sn;
  sin_out[o + half + i] = sn;
}

// x: [T, Hn, D] (row stride ldx elements between tokens), rotate-half convention:
// y[:half] = x1*c1 - x2*s1 ; y[half:] = x2*c2 + x1*s2.  `conj` applies the transpose
// (backward).  rot_dim <= D: dims beyond rot_dim are copied.
__global__ void rope_apply_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, const float* __restrict__ cosb,
                                  const float* __restrict__ sinb, int T, int Hn, int D, int rot_dim, long ldx,
                                  long ldy, int conj) {
  const int half = rot_dim / 2;
  const int per_head = half / 8;  // vectors of 8 pairs
  const long total = static_cast<long>(T) * Hn * per_head;
  for (long idx = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long>(gridDim.x) * blockDim.x) {
    const int v = idx % per_head;
    const long th = idx / per_head;
    const int h = th % Hn;
    const long t = th / Hn;
    const bf16* xp = x + t * ldx + static_cast<long>(h) * D;
    bf16* yp = y + t * ldy + static_cast<long>(h) * D;
    float x1[8], x2[8], o1[8], o2[8];
    load8(xp + v * 8, x1);
    load8(xp + half + v * 8, x2);
    const float* c = cosb + t * rot_dim;
    const float* s = sinb + t * rot_dim;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float c1 = c[v * 8 + j], c2 = c[half + v * 8 + j];
      const float s1 = s[v * 8 + j], s2 = s[half + v * 8 + j];
      if (!conj) {
        o1[j] = x1[j] * c1 - x2[j] * s1;
        o2[j] = x2[j] * c2 + x1[j] * s2;
      } else {
        o1[j] = x1[j] * c1 + x2[j] * s2;
        o2[j] = x2[j] * c2 - x1[j] * s1;
      }
    }
    store8(yp + v * 8, o1);
    store8(yp + half + v * 8, o2);
  }
}

// ------------------------------------------------------------------ SwiGLU
__global__ void swiglu_fwd_kernel(const bf16* __restrict__ g, const bf16* __restrict__ u, bf16* __restrict__ h,
                                  long n8) {
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float gv[8], uv[8], o[8];
    load8(g + i * 8, gv);
    load8(u + i * 8, uv);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = gv[j] / (1.f + __expf(-gv[j])) * uv[j];
    store8(h + i * 8, o);
  }
}
// dg, du may alias g, u (in place).
__global__ void swiglu_bwd_kernel(const bf16* __restrict__ dh, const bf16* g, const bf16* u, bf16* dg, bf16* du,
                                  long n8) {
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float dv[8], gv[8], uv[8], og[8], ou[8];
    load8(dh + i * 8, dv);
    load8(g + i * 8, gv);
    load8(u + i * 8, uv);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sig = 1.f / (1.f + __expf(-gv[j]));
      const float silu = gv[j] * sig;
      ou[j] = dv[j] * silu;
      og[j] = dv[j] * uv[j] * (sig + silu * (1.f - sig));
    }
    store8(dg + i * 8, og);
    store8(du + i * 8, ou);
  }
}

// ------------------------------------------------------------------ optimizers on flat buffers
// AdamW with fp32 master weights and moments; gradient bf16 or fp32.  `gscale` (device
// scalar, may be null) multiplies the gradient (clip coefficient); `skip` (device int,
// may be null) suppresses the whole update when non-zero (non-finite gradient norm).
template <typename GT>
__global__ void adamw_kernel(float* __restrict__ p32, bf16* __restrict__ p16, float* __restrict__ m,
                             float* __restrict__ v, const GT* __restrict__ g, long n, float lr, float beta1,
                             float beta2, float eps, float wd, float bc1, float bc2, const float* gscale,
                             const int* skip) {
  if (skip != nullptr && *skip) return;
  const float gs = gscale != nullptr ? *gscale : 1.f;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const float gi = static_cast<float>(g[i]) * gs;
    float pi = p32[i];
    const float mi = beta1 * m[i] + (1.f - beta1) * gi;
    const float vi = beta2 * v[i] + (1.f - beta2) * gi * gi;
    m[i] = mi;
    v[i] = vi;
    pi *= (1.f - lr * wd);
    pi -= lr * (mi / bc1) / (sqrtf(vi / bc2) + eps);
    p32[i] = pi;
    if (p16 != nullptr) p16[i] = __float2bfloat16(pi);
  }
}

// Muon step 1: momentum and the Newton-Schulz input.
//   mom = beta*mom + (1-beta)*g ; u = nesterov ? g + beta*(mom - g) : mom ; out = bf16(u)
// plus the sum of squares of u into sumsq[0] (one atomic per CTA) for the Frobenius norm.
template <typename GT>
__global__ void muon_momentum_kernel(float* __restrict__ mom, const GT* __restrict__ g, bf16* __restrict__ out,
                                     float* __restrict__ sumsq, long n, float beta, int nesterov,
                                     const float* gscale) {
  __shared__ float red[32];
  const float gs = gscale != nullptr ? *gscale : 1.f;
  float acc = 0.f;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const float gi = static_cast<float>(g[i]) * gs;
    const float mi = beta * mom[i] + (1.f - beta) * gi;
    mom[i] = mi;
    const float u = nesterov ? gi + beta * (mi - gi) : mi;
    out[i] = __float2bfloat16(u);
    acc += u * u;
  }
  acc = block_sum<256>(acc, red);
  if (threadIdx.x == 0) atomicAdd(sumsq, acc);
}
// x *= 1 / (sqrt(sumsq) + eps)   (bf16 in place)
__global__ void scale_by_norm_kernel(bf16* __restrict__ x, const float* __restrict__ sumsq, long n, float eps) {
  const float s = 1.f / (sqrtf(*sumsq) + eps);
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long>(gridDim.x) * blockDim.x)
    x[i] = __float2bfloat16(__bfloat162float(x[i]) * s);
}
// Muon step 3: p = p*(1 - lr*wd) - lr*scale*o ; bf16 copy refreshed.
__global__ void muon_update_kernel(float* __restrict__ p32, bf16* __restrict__ p16, const bf16* __restrict__ o,
                                   long n, float lr, float wd, float scale, const int* skip) {
  if (skip != nullptr && *skip) return;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float pi = p32[i] * (1.f - lr * wd) - lr * scale * __bfloat162float(o[i]);
    p32[i] = pi;
    if (p16 != nullptr) p16[i] = __float2bfloat16(pi);
  }
}

// ema = decay*ema + (1-decay)*p
template <typename PT>
__global__ void ema_kernel(float* __restrict__ ema, const PT* __restrict__ p, long n, float decay) {
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long>(gridDim.x) * blockDim.x)
    ema[i] = decay * ema[i] + (1.f - decay) * static_cast<float>(p[i]);
}

// ---- 16-byte versions of the optimizer passes ---------------------------------------------------------------
// The passes above move 2 or 4 bytes per thread and iteration, which keeps too few bytes in flight to fill HBM
// (1.3 - 3.5 TB/s measured).  These take four elements per thread and iteration (float4 / 4 x bf16); the launchers use
// them when every pointer is 16-byte aligned (8 for the bf16 arrays) and hand the last n % 4 elements to the scalar
// kernels.  Element-wise results are bit-identical to the scalar kernels; the sums of squares add in another order.
struct alignas(8) bf16x4 {
  uint32_t lo, hi;
};
__device__ __forceinline__ bf16x4 to_bf16x4(float a, float b, float c, float d) {
  bf16x4 r;
  r.lo = pack_bf16x2(a, b);
  r.hi = pack_bf16x2(c, d);
  return r;
}

__global__ void adamw_vec_kernel(float4* __restrict__ p32, bf16x4* __restrict__ p16, float4* __restrict__ m,
                                 float4* __restrict__ v, const float4* __restrict__ g, long nv, float lr, float beta1,
                                 float beta2, float eps, float wd, float bc1, float bc2, const float* gscale,
                                 const int* skip) {
  if (skip != nullptr && *skip) return;
  const float gs = gscale != nullptr ? *gscale : 1.f;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const float4 g4 = g[i];
    float4 p4 = p32[i], m4 = m[i], v4 = v[i];
    const float gi[4] = {g4.x * gs, g4.y * gs, g4.z * gs, g4.w * gs};
    float pi[4] = {p4.x, p4.y, p4.z, p4.w}, mi[4] = {m4.x, m4.y, m4.z, m4.w}, vi[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      mi[e] = beta1 * mi[e] + (1.f - beta1) * gi[e];
      vi[e] = beta2 * vi[e] + (1.f - beta2) * gi[e] * gi[e];
      pi[e] *= (1.f - lr * wd);
      pi[e] -= lr * (mi[e] / bc1) / (sqrtf(vi[e] / bc2) + eps);
    }
    m[i] = make_float4(mi[0], mi[1], mi[2], mi[3]);
    v[i] = make_float4(vi[0], vi[1], vi[2], vi[3]);
    p32[i] = make_float4(pi[0], pi[1], pi[2], pi[3]);
    if (p16 != nullptr) p16[i] = to_bf16x4(pi[0], pi[1], pi[2], pi[3]);
  }
}

__global__ void muon_momentum_vec_kernel(float4* __restrict__ mom, const float4* __restrict__ g, bf16x4* __restrict__ out,
                                         float* __restrict__ sumsq, long nv, float beta, int nesterov,
                                         const float* gscale) {
  __shared__ float red[32];
  const float gs = gscale != nullptr ? *gscale : 1.f;
  float acc = 0.f;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const float4 g4 = g[i];
    const float4 m4 = mom[i];
    const float gi[4] = {g4.x * gs, g4.y * gs, g4.z * gs, g4.w * gs};
    float mi[4] = {m4.x, m4.y, m4.z, m4.w}, u[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      mi[e] = beta * mi[e] + (1.f - beta) * gi[e];
      u[e] = nesterov ? gi[e] + beta * (mi[e] - gi[e]) : mi[e];
      acc += u[e] * u[e];
    }
    mom[i] = make_float4(mi[0], mi[1], mi[2], mi[3]);
    out[i] = to_bf16x4(u[0], u[1], u[2], u[3]);
  }
  acc = block_sum<256>(acc, red);
  if (threadIdx.x == 0) atomicAdd(sumsq, acc);
}

__global__ void scale_by_norm_vec_kernel(uint4* __restrict__ x, const float* __restrict__ sumsq, long nv8, float eps) {
  const float s = 1.f / (sqrtf(*sumsq) + eps);
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < nv8;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    uint4 w = x[i];
    float2 a = unpack_bf16x2(w.x), b = unpack_bf16x2(w.y), c = unpack_bf16x2(w.z), d = unpack_bf16x2(w.w);
    // the same rounding as the scalar kernel: bf16(float(x) * s)
    w.x = pack_bf16x2(a.x * s, a.y * s);
    w.y = pack_bf16x2(b.x * s, b.y * s);
    w.z = pack_bf16x2(c.x * s, c.y * s);
    w.w = pack_bf16x2(d.x * s, d.y * s);
    x[i] = w;
  }
}

__global__ void muon_update_vec_kernel(float4* __restrict__ p32, bf16x4* __restrict__ p16, const bf16x4* __restrict__ o,
                                       long nv, float lr, float wd, float scale, const int* skip) {
  if (skip != nullptr && *skip) return;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const float4 p4 = p32[i];
    const bf16x4 o4 = o[i];
    const float2 oa = unpack_bf16x2(o4.lo), ob = unpack_bf16x2(o4.hi);
    const float r0 = p4.x * (1.f - lr * wd) - lr * scale * oa.x;
    const float r1 = p4.y * (1.f - lr * wd) - lr * scale * oa.y;
    const float r2 = p4.z * (1.f - lr * wd) - lr * scale * ob.x;
    const float r3 = p4.w * (1.f - lr * wd) - lr * scale * ob.y;
    p32[i] = make_float4(r0, r1, r2, r3);
    if (p16 != nullptr) p16[i] = to_bf16x4(r0, r1, r2, r3);
  }
}

__global__ void sumsq_part_vec_kernel(const float4* __restrict__ g, float* __restrict__ part, long nv, const float* tail,
                                      int n_tail) {
  __shared__ float red[32];
  float acc = 0.f;
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x;
  // four independent 16-byte loads per thread and iteration: the grid is capped at the size of the partials scratch
  for (; i + 3 * stride < nv; i += 4 * stride) {
    const float4 a = g[i], b = g[i + stride], c = g[i + 2 * stride], d = g[i + 3 * stride];
    acc += (a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w) + (b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w) +
           (c.x * c.x + c.y * c.y + c.z * c.z + c.w * c.w) + (d.x * d.x + d.y * d.y + d.z * d.z + d.w * d.w);
  }
  for (; i < nv; i += stride) {
    const float4 v = g[i];
    acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (blockIdx.x == 0 && threadIdx.x < n_tail) acc += tail[threadIdx.x] * tail[threadIdx.x];
  acc = block_sum<256>(acc, red);
  if (threadIdx.x == 0) part[blockIdx.x] = acc;
}

// LMMS_B200_SCALAR_OPTIM=1 keeps the scalar passes (the A/B of profiles/optimizer_passes_microbench.md)
static inline bool aligned_to(const void* p, uintptr_t a) {
  static const bool scalar_only = [] {
    const char* e = getenv("LMMS_B200_SCALAR_OPTIM");
    return e != nullptr && e[0] == '1';
  }();
  return !scalar_only && (p == nullptr || (reinterpret_cast<uintptr_t>(p) % a) == 0);
}

// Deterministic two-stage sum of squares: part[blockIdx.x] then a single-CTA finish.
template <typename GT>
__global__ void sumsq_part_kernel(const GT* __restrict__ g, float* __restrict__ part, long n) {
  __shared__ float red[32];
  float acc = 0.f;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const float gi = static_cast<float>(g[i]);
    acc += gi * gi;
  }
  acc = block_sum<256>(acc, red);
  if (threadIdx.x == 0) part[blockIdx.x] = acc;
}
// out[0] (+)= sum(part)
__global__ void sumsq_finish_kernel(const float* __restrict__ part, float* __restrict__ out, int parts,
                                    int accumulate) {
  __shared__ float red[32];
  float acc = 0.f;
  for (int i = threadIdx.x; i < parts; i += blockDim.x) acc += part[i];
  acc = block_sum<256>(acc, red);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + acc : acc;
}
// From the global sum of squares: norm, clip coefficient min(1, max_norm/(norm+1e-6)),
// and a skip flag when the norm is not finite or a kernel of this device has raised the status
// word (a bounded wait that ran out: the gradients of this step may be incomplete).  No host
// round trip.
__global__ void clip_coef_kernel(const float* __restrict__ sumsq, float* __restrict__ norm_out,
                                 float* __restrict__ coef_out, int* __restrict__ skip_out, float max_norm,
                                 const int* __restrict__ status) {
  const float norm = sqrtf(*sumsq);
  *norm_out = norm;
  const bool finite = isfinite(norm);
  const bool faulted = status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0;
  *skip_out = (finite && !faulted) ? 0 : 1;
  float c = 1.f;
  if (max_norm > 0.f && finite) c = fminf(1.f, max_norm / (norm + 1e-6f));
  *coef_out = c;
}
template <typename GT>
__global__ void scale_kernel(GT* __restrict__ g, long n, const float* __restrict__ coef) {
  const float c = *coef;
  if (c == 1.f) return;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long>(gridDim.x) * blockDim.x)
    g[i] = static_cast<GT>(static_cast<float>(g[i]) * c);
}

// ------------------------------------------------------------------ packed-sequence index kernels
// out[i, :] = src[idx[i], :]  (idx < 0 writes zeros) and the scatter inverse (optionally adding).
__global__ void gather_rows_kernel(const bf16* __restrict__ src, const int64_t* __restrict__ idx,
                                   bf16* __restrict__ out, long n_out, int H, long n_src, int* status) {
  const int vec = H / 8;
  const long total = n_out * vec;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long r = i / vec;
    const int c = (i - r * vec) * 8;
    const int64_t s = idx[r];
    bf16x8 v;
    v.w[0] = v.w[1] = v.w[2] = v.w[3] = 0u;
    if (s >= 0 && index_in_bounds(s, n_src, status)) v = *reinterpret_cast<const bf16x8*>(src + s * H + c);
    *reinterpret_cast<bf16x8*>(out + r * H + c) = v;
  }
}
__global__ void scatter_rows_kernel(const bf16* __restrict__ src, const int64_t* __restrict__ idx,
                                    bf16* __restrict__ out, long n_src, int H, int add, long n_out, int* status) {
  const int vec = H / 8;
  const long total = n_src * vec;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long r = i / vec;
    const int c = (i - r * vec) * 8;
    const int64_t d = idx[r];
    if (d < 0 || !index_in_bounds(d, n_out, status)) continue;
    float v[8];
    load8(src + r * H + c, v);
    if (add) {
      float o[8];
      load8(out + d * H + c, o);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += o[j];
    }
    store8(out + d * H + c, v);
  }
}

// ------------------------------------------------------------------ cross-entropy passes
// After the logits GEMM with the statistics epilogue: combine the per-tile partials into
// lse, pick the target logit, emit per-row loss (0 for ignored rows).
__global__ void ce_finalize_kernel(const float2* __restrict__ stats, const bf16* __restrict__ logits,
                                   const int64_t* __restrict__ labels, float* __restrict__ lse_out,
                                   float* __restrict__ loss_out, int rows, int n_tiles, long ld, int V,
                                   int ignore_index) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (int row = blockIdx.x * wpb + (threadIdx.x >> 5); row < rows; row += gridDim.x * wpb) {
    float mx = -INFINITY;
    for (int i = lane; i < n_tiles; i += 32) mx = fmaxf(mx, stats[static_cast<size_t>(row) * n_tiles + i].x);
    mx = warp_max(mx);
    float s = 0.f;
    for (int i = lane; i < n_tiles; i += 32) {
      const float2 st = stats[static_cast<size_t>(row) * n_tiles + i];
      if (st.x > -INFINITY) s += st.y * __expf(st.x - mx);
    }
    s = warp_sum(s);
    if (lane == 0) {
      const float lse = mx + logf(s);
      lse_out[row] = lse;
      const int64_t y = labels[row];
      float l = 0.f;
      if (y != ignore_index && y >= 0 && y < V) l = lse - __bfloat162float(logits[static_cast<size_t>(row) * ld + y]);
      loss_out[row] = l;
    }
  }
}
// In place: logits[r, c] <- gscale[0]*row_w * (exp(logits - lse) - [c == label]); ignored rows -> 0.
__global__ void ce_dlogits_kernel(bf16* __restrict__ logits, const float* __restrict__ lse,
                                  const int64_t* __restrict__ labels, const float* __restrict__ gscale, int rows,
                                  long ld, int V, int ignore_index) {
  const int vec = V / 8;
  const float gs = *gscale;
  for (int row = blockIdx.y; row < rows; row += gridDim.y) {
    const int64_t y = labels[row];
    const bool ign = (y == ignore_index);
    const float l = lse[row];
    bf16* base = logits + static_cast<size_t>(row) * ld;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < vec; i += gridDim.x * blockDim.x) {
      float v[8];
      if (ign) {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = 0.f;
      } else {
        load8(base + i * 8, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float pr = __expf(v[j] - l);
          if (i * 8 + j == y) pr -= 1.f;
          v[j] = pr * gs;
        }
      }
      store8(base + i * 8, v);
    }
  }
}

static int g_sms = 0;
static int num_sms() {
  if (g_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return g_sms;
}
static int grid_for(long work_items, int threads, int per_sm = 8) {
  long blocks = (work_items + threads - 1) / threads;
  long cap = static_cast<long>(num_sms()) * per_sm;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

}  // namespace b200

using namespace b200;

#define CHECK_LAUNCH() (cudaGetLastError() == cudaSuccess ? 0 : -4)

extern "C" {

int b200_num_partials() { return num_sms() * 2; }

// rows x H bf16.  ln = 0: RMSNorm, 1: LayerNorm (b may be null).  res/res_out may be null.
int b200_norm_fwd(const void* x, const void* res, const void* w, const void* b, void* y, void* res_out, void* rstd,
                  void* mean, int rows, int H, float eps, float w_offset, int ln, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (H % 8) return -10;
  if (H <= 512 && !ln && res == nullptr) {
    int blocks = grid_for(static_cast<long>(rows) * 32, 256, 8);
    norm_fwd_warp_kernel<<<blocks, 256, 0, st>>>((const bf16*)x, (const bf16*)w, (bf16*)y, (float*)rstd, rows, H, eps,
                                                 w_offset);
    return CHECK_LAUNCH();
  }
  int blocks = rows < num_sms() * 8 ? rows : num_sms() * 8;
#define NORM_FWD(T, V)                                                                                              \
  norm_fwd_kernel<T, V><<<blocks, T, 0, st>>>((const bf16*)x, (const bf16*)res, (const bf16*)w, (const bf16*)b,     \
                                              (bf16*)y, (bf16*)res_out, (float*)rstd, (float*)mean, rows, H, eps, \
                                              w_offset, ln)
  if (H <= 1024) NORM_FWD(128, 1);
  else if (H <= 2048) NORM_FWD(256, 1);
  else if (H <= 4096) NORM_FWD(256, 2);
  else if (H <= 8192) NORM_FWD(512, 2);
  else if (H <= 16384) NORM_FWD(512, 4);
  else return -11;
#undef NORM_FWD
  return CHECK_LAUNCH();
}

// dw_part / db_part: fp32 [b200_num_partials(), H] scratch.  dw/db fp32 [H] (accumulate flag).
int b200_norm_bwd(const void* dy, const void* x, const void* w, const void* rstd, const void* mean,
                  const void* dres_in, void* dx, void* dw_part, void* db_part, void* dw, void* db, int rows, int H,
                  float w_offset, int ln, int accumulate, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (H % 8) return -10;
  int parts;
  if (H <= 512 && !ln && dres_in == nullptr) {
    if (H == 64 || H == 128 || H == 256) {
      const int lpr = H / 8, rows_per_block = 16 * (32 / lpr);
      long want = (static_cast<long>(rows) + rows_per_block - 1) / rows_per_block;
      parts = static_cast<int>(want < num_sms() * 2 ? want : num_sms() * 2);  // one partials row per block
      if (parts < 1) parts = 1;
      if (H == 64)
        norm_bwd_narrow_kernel<8><<<parts, 512, 0, st>>>((const bf16*)dy, (const bf16*)x, (const bf16*)w, (const float*)rstd,
                                                         (bf16*)dx, (float*)dw_part, rows, w_offset);
      else if (H == 128)
        norm_bwd_narrow_kernel<16><<<parts, 512, 0, st>>>((const bf16*)dy, (const bf16*)x, (const bf16*)w, (const float*)rstd,
                                                          (bf16*)dx, (float*)dw_part, rows, w_offset);
      else
        norm_bwd_narrow_kernel<32><<<parts, 512, 0, st>>>((const bf16*)dy, (const bf16*)x, (const bf16*)w, (const float*)rstd,
                                                          (bf16*)dx, (float*)dw_part, rows, w_offset);
      if (cudaGetLastError() != cudaSuccess) return -4;
      colsum_kernel<<<(H + 255) / 256, 256, 0, st>>>((const float*)dw_part, (float*)dw, parts, H, accumulate);
      return CHECK_LAUNCH();
    }
    int blocks = num_sms() * 2 / 8;
    if (blocks < 1) blocks = 1;
    parts = blocks * 8;
    norm_bwd_warp_kernel<<<blocks, 256, 0, st>>>((const bf16*)dy, (const bf16*)x, (const bf16*)w, (const float*)rstd,
                                                 (bf16*)dx, (float*)dw_part, rows, H, w_offset);
  } else {
    parts = num_sms() * 2;
    if (parts > rows) parts = rows;
#define NORM_BWD(T, V)                                                                                            \
  norm_bwd_kernel<T, V><<<parts, T, 0, st>>>((const bf16*)dy, (const bf16*)x, (const bf16*)w, (const float*)rstd, \
                                             (const float*)mean, (const bf16*)dres_in, (bf16*)dx, (float*)dw_part, \
                                             (float*)db_part, rows, H, w_offset, ln)
    if (H <= 1024) NORM_BWD(128, 1);
    else if (H <= 2048) NORM_BWD(256, 1);
    else if (H <= 4096) NORM_BWD(256, 2);
    else if (H <= 8192) NORM_BWD(512, 2);
    else if (H <= 16384) NORM_BWD(512, 4);
    else return -11;
#undef NORM_BWD
  }
  if (cudaGetLastError() != cudaSuccess) return -4;
  colsum_kernel<<<(H + 255) / 256, 256, 0, st>>>((const float*)dw_part, (float*)dw, parts, H, accumulate);
  if (db != nullptr && db_part != nullptr)
    colsum_kernel<<<(H + 255) / 256, 256, 0, st>>>((const float*)db_part, (float*)db, parts, H, accumulate);
  return CHECK_LAUNCH();
}

int b200_rope_table(const void* pos, const void* inv_freq, void* cos_out, void* sin_out, int T, int half, int mode,
                    int s0, int s1, int s2, float scaling, cudaStream_t st) {
  long n = static_cast<long>(T) * half;
  if (n <= 0) return 0;
  rope_table_kernel<<<(n + 255) / 256, 256, 0, st>>>((const int64_t*)pos, (const float*)inv_freq, (float*)cos_out,
                                                     (float*)sin_out, T, half, mode, s0, s1, s2, scaling);
  return CHECK_LAUNCH();
}

int b200_rope_apply(const void* x, void* y, const void* cosb, const void* sinb, int T, int Hn, int D, int rot_dim,
                    long ldx, long ldy, int conj, cudaStream_t st) {
  if (T <= 0) return 0;
  if (rot_dim % 16 || D % 8 || ldx % 8 || ldy % 8) return -10;
  long total = static_cast<long>(T) * Hn * (rot_dim / 16);
  rope_apply_kernel<<<grid_for(total, 256), 256, 0, st>>>((const bf16*)x, (bf16*)y, (const float*)cosb,
                                                          (const float*)sinb, T, Hn, D, rot_dim, ldx, ldy, conj);
  return CHECK_LAUNCH();
}

int b200_swiglu_fwd(const void* g, const void* u, void* h, long n, cudaStream_t st) {
  if (n <= 0) return 0;
  if (n % 8) return -10;
  swiglu_fwd_kernel<<<grid_for(n / 8, 256), 256, 0, st>>>((const bf16*)g, (const bf16*)u, (bf16*)h, n / 8);
  return CHECK_LAUNCH();
}
int b200_swiglu_bwd(const void* dh, const void* g, const void* u, void* dg, void* du, long n, cudaStream_t st) {
  if (n <= 0) return 0;
  if (n % 8) return -10;
  swiglu_bwd_kernel<<<grid_for(n / 8, 256), 256, 0, st>>>((const bf16*)dh, (const bf16*)g, (const bf16*)u, (bf16*)dg,
                                                          (bf16*)du, n / 8);
  return CHECK_LAUNCH();
}

int b200_adamw(void* p32, void* p16, void* m, void* v, const void* g, int g_is_fp32, long n, float lr, float beta1,
               float beta2, float eps, float wd, float bc1, float bc2, const void* gscale, const void* skip,
               cudaStream_t st) {
  if (n <= 0) return 0;
  if (g_is_fp32 && n >= 4 && aligned_to(p32, 16) && aligned_to(p16, 8) && aligned_to(m, 16) && aligned_to(v, 16) && aligned_to(g, 16)) {
    const long nv = n / 4, done = nv * 4;
    adamw_vec_kernel<<<grid_for(nv, 256), 256, 0, st>>>((float4*)p32, (bf16x4*)p16, (float4*)m, (float4*)v, (const float4*)g, nv, lr,
                                                        beta1, beta2, eps, wd, bc1, bc2, (const float*)gscale, (const int*)skip);
    if (done < n)
      adamw_kernel<float><<<1, 32, 0, st>>>((float*)p32 + done, p16 ? (bf16*)p16 + done : nullptr, (float*)m + done, (float*)v + done,
                                            (const float*)g + done, n - done, lr, beta1, beta2, eps, wd, bc1, bc2,
                                            (const float*)gscale, (const int*)skip);
    return CHECK_LAUNCH();
  }
  int blocks = grid_for(n, 256);
  if (g_is_fp32)
    adamw_kernel<float><<<blocks, 256, 0, st>>>((float*)p32, (bf16*)p16, (float*)m, (float*)v, (const float*)g, n, lr,
                                                beta1, beta2, eps, wd, bc1, bc2, (const float*)gscale,
                                                (const int*)skip);
  else
    adamw_kernel<bf16><<<blocks, 256, 0, st>>>((float*)p32, (bf16*)p16, (float*)m, (float*)v, (const bf16*)g, n, lr,
                                               beta1, beta2, eps, wd, bc1, bc2, (const float*)gscale, (const int*)skip);
  return CHECK_LAUNCH();
}

int b200_muon_momentum(void* mom, const void* g, int g_is_fp32, void* out, void* sumsq, long n, float beta,
                       int nesterov, const void* gscale, float eps, cudaStream_t st) {
  if (n <= 0) return 0;
  cudaMemsetAsync(sumsq, 0, sizeof(float), st);
  if (g_is_fp32 && n % 8 == 0 && aligned_to(mom, 16) && aligned_to(g, 16) && aligned_to(out, 16)) {
    // whole matrices: their element counts are multiples of 8 in every supported layout
    muon_momentum_vec_kernel<<<grid_for(n / 4, 256, 4), 256, 0, st>>>((float4*)mom, (const float4*)g, (bf16x4*)out, (float*)sumsq,
                                                                     n / 4, beta, nesterov, (const float*)gscale);
    scale_by_norm_vec_kernel<<<grid_for(n / 8, 256, 4), 256, 0, st>>>((uint4*)out, (const float*)sumsq, n / 8, eps);
    return CHECK_LAUNCH();
  }
  int blocks = grid_for(n, 256, 4);
  if (g_is_fp32)
    muon_momentum_kernel<float><<<blocks, 256, 0, st>>>((float*)mom, (const float*)g, (bf16*)out, (float*)sumsq, n,
                                                        beta, nesterov, (const float*)gscale);
  else
    muon_momentum_kernel<bf16><<<blocks, 256, 0, st>>>((float*)mom, (const bf16*)g, (bf16*)out, (float*)sumsq, n, beta,
                                                       nesterov, (const float*)gscale);
  scale_by_norm_kernel<<<blocks, 256, 0, st>>>((bf16*)out, (const float*)sumsq, n, eps);
  return CHECK_LAUNCH();
}

int b200_muon_update(void* p32, void* p16, const void* o, long n, float lr, float wd, float scale, const void* skip,
                     cudaStream_t st) {
  if (n <= 0) return 0;
  if (n % 4 == 0 && aligned_to(p32, 16) && aligned_to(p16, 8) && aligned_to(o, 8)) {
    muon_update_vec_kernel<<<grid_for(n / 4, 256), 256, 0, st>>>((float4*)p32, (bf16x4*)p16, (const bf16x4*)o, n / 4, lr, wd, scale,
                                                                 (const int*)skip);
    return CHECK_LAUNCH();
  }
  muon_update_kernel<<<grid_for(n, 256), 256, 0, st>>>((float*)p32, (bf16*)p16, (const bf16*)o, n, lr, wd, scale,
                                                       (const int*)skip);
  return CHECK_LAUNCH();
}

int b200_ema(void* ema, const void* p, int p_is_fp32, long n, float decay, cudaStream_t st) {
  if (n <= 0) return 0;
  if (p_is_fp32) ema_kernel<float><<<grid_for(n, 256), 256, 0, st>>>((float*)ema, (const float*)p, n, decay);
  else ema_kernel<bf16><<<grid_for(n, 256), 256, 0, st>>>((float*)ema, (const bf16*)p, n, decay);
  return CHECK_LAUNCH();
}

// part: fp32 scratch of b200_num_partials() floats.  out[0] (+)= sum g^2.
int b200_sumsq(const void* g, int g_is_fp32, long n, void* part, void* out, int accumulate, cudaStream_t st) {
  int blocks = grid_for(n > 0 ? n : 1, 256, 2);
  if (g_is_fp32 && n >= 4 && aligned_to(g, 16)) {
    const long nv = n / 4;
    blocks = grid_for(nv, 256, 2);  // the partials scratch holds b200_num_partials() = 2 per SM
    sumsq_part_vec_kernel<<<blocks, 256, 0, st>>>((const float4*)g, (float*)part, nv, (const float*)g + nv * 4,
                                                  static_cast<int>(n - nv * 4));
    sumsq_finish_kernel<<<1, 256, 0, st>>>((const float*)part, (float*)out, blocks, accumulate);
    return CHECK_LAUNCH();
  }
  if (g_is_fp32) sumsq_part_kernel<float><<<blocks, 256, 0, st>>>((const float*)g, (float*)part, n);
  else sumsq_part_kernel<bf16><<<blocks, 256, 0, st>>>((const bf16*)g, (float*)part, n);
  sumsq_finish_kernel<<<1, 256, 0, st>>>((const float*)part, (float*)out, blocks, accumulate);
  return CHECK_LAUNCH();
}
int b200_clip_coef(const void* sumsq, void* norm_out, void* coef_out, void* skip_out, float max_norm,
                   const void* status, cudaStream_t st) {
  clip_coef_kernel<<<1, 1, 0, st>>>((const float*)sumsq, (float*)norm_out, (float*)coef_out, (int*)skip_out,
                                    max_norm, (const int*)status);
  return CHECK_LAUNCH();
}
int b200_scale(void* g, int g_is_fp32, long n, const void* coef, cudaStream_t st) {
  if (n <= 0) return 0;
  if (g_is_fp32) scale_kernel<float><<<grid_for(n, 256), 256, 0, st>>>((float*)g, n, (const float*)coef);
  else scale_kernel<bf16><<<grid_for(n, 256), 256, 0, st>>>((bf16*)g, n, (const float*)coef);
  return CHECK_LAUNCH();
}

// n_src / n_out: rows of the indexed tensor; an index beyond it raises kStatusBadIndex in *status and is skipped.
int b200_gather_rows(const void* src, const void* idx, void* out, long n_out, int H, long n_src, void* status,
                     cudaStream_t st) {
  if (n_out <= 0) return 0;
  if (H % 8) return -10;
  gather_rows_kernel<<<grid_for(n_out * (H / 8), 256), 256, 0, st>>>((const bf16*)src, (const int64_t*)idx, (bf16*)out,
                                                                     n_out, H, n_src, (int*)status);
  return CHECK_LAUNCH();
}
int b200_scatter_rows(const void* src, const void* idx, void* out, long n_src, int H, int add, long n_out, void* status,
                      cudaStream_t st) {
  if (n_src <= 0) return 0;
  if (H % 8) return -10;
  scatter_rows_kernel<<<grid_for(n_src * (H / 8), 256), 256, 0, st>>>((const bf16*)src, (const int64_t*)idx,
                                                                      (bf16*)out, n_src, H, add, n_out, (int*)status);
  return CHECK_LAUNCH();
}

int b200_ce_finalize(const void* stats, const void* logits, const void* labels, void* lse, void* loss, int rows,
                     int n_tiles, long ld, int V, int ignore_index, cudaStream_t st) {
  if (rows <= 0) return 0;
  ce_finalize_kernel<<<grid_for(static_cast<long>(rows) * 32, 256), 256, 0, st>>>(
      (const float2*)stats, (const bf16*)logits, (const int64_t*)labels, (float*)lse, (float*)loss, rows, n_tiles, ld,
      V, ignore_index);
  return CHECK_LAUNCH();
}
int b200_ce_dlogits(void* logits, const void* lse, const void* labels, const void* gscale, int rows, long ld, int V,
                    int ignore_index, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (V % 8) return -10;
  int bx = (V / 8 + 255) / 256;
  if (bx > 16) bx = 16;
  int by = rows < 65535 ? rows : 65535;
  ce_dlogits_kernel<<<dim3(bx, by), 256, 0, st>>>((bf16*)logits, (const float*)lse, (const int64_t*)labels,
                                                  (const float*)gscale, rows, ld, V, ignore_index);
  return CHECK_LAUNCH();
}

}  // extern "C"

// ====================================================================================
// Allocation-free RMSNorm backward (see no_alloc.h for who needs it and for its limits).
// ====================================================================================
#include "no_alloc.h"

#include <mutex>

namespace b200 {

// Scratch for the per-CTA partial sums of dw.  File scope, device memory, part of the
// library image: no allocation at run time.  In host code this name is only a handle for
// cudaGetSymbolAddress, never a pointer a kernel could use.
static __device__ __align__(256) float g_noalloc_dw_part[B200_NOALLOC_MAX_PARTS * B200_NOALLOC_MAX_H];

constexpr int kNoAllocMaxDevices = 64;
static float* g_noalloc_ptr[kNoAllocMaxDevices] = {nullptr};
static std::mutex g_noalloc_mutex;

// Device address of the scratch array on the current device, resolved once per device.
static float* noalloc_scratch_for_current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_dw_part) != cudaSuccess || p == nullptr) return nullptr;
    g_noalloc_ptr[dev] = static_cast<float*>(p);
  }
  return g_noalloc_ptr[dev];
}

}  // namespace b200

extern "C" int b200_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const void* rstd, void* dx,
                                        void* dw, int rows, int H, float w_offset, cudaStream_t st) {
  using namespace b200;
  if (rows <= 0) return 0;
  if (H % 8) return -10;
  if (H > B200_NOALLOC_MAX_H) return B200_NOALLOC_ERR_TOO_LARGE;
  float* part = noalloc_scratch_for_current_device();
  if (part == nullptr) return B200_NOALLOC_ERR_SETUP;
  int parts;
  if (H <= 512) {
    int blocks = num_sms() * 2 / 8;
    if (blocks < 1) blocks = 1;
    parts = blocks * 8;
    if (parts > B200_NOALLOC_MAX_PARTS) return B200_NOALLOC_ERR_TOO_LARGE;
    norm_bwd_warp_kernel<<<blocks, 256, 0, st>>>((const bf16*)dy, (const bf16*)x, (const bf16*)w, (const float*)rstd,
                                                 (bf16*)dx, part, rows, H, w_offset);
  } else {
    parts = num_sms() * 2;
    if (parts > rows) parts = rows;
    if (parts > B200_NOALLOC_MAX_PARTS) parts = B200_NOALLOC_MAX_PARTS;
#define NOALLOC_BWD(T, V)                                                                                          \
  norm_bwd_kernel<T, V><<<parts, T, 0, st>>>((const bf16*)dy, (const bf16*)x, (const bf16*)w, (const float*)rstd, \
                                             nullptr, nullptr, (bf16*)dx, part, nullptr, rows, H, w_offset, 0)
    if (H <= 1024) NOALLOC_BWD(128, 1);
    else if (H <= 2048) NOALLOC_BWD(256, 1);
    else NOALLOC_BWD(256, 2);
#undef NOALLOC_BWD
  }
  if (cudaGetLastError() != cudaSuccess) return -4;
  // every partial row that is summed here was written by the launch above
  colsum_kernel<<<(H + 255) / 256, 256, 0, st>>>(part, (float*)dw, parts, H, 0);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
