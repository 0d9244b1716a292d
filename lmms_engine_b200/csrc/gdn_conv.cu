// Short causal depthwise convolution + SiLU over a packed token stream, forward and backward, one pass each.
//
//     pre[t, c] = sum_{j = 0 .. K-1, j <= pos[t]} w[c, K-1-j] * x[t-j, c]        y = pre * sigmoid(pre)
//
// `pos[t]` is the token's position inside its document, so the window never reaches into the previous
// document.  One thread owns two neighbouring channels (neighbouring threads neighbouring pairs: coalesced rows of
// 4-byte accesses) and walks a tile of tokens with the last K inputs in registers, so x and y cross HBM once.
// The backward pass recomputes `pre`, forms d pre = dy * (s + pre * s * (1 - s)) for the tile plus K-1 tokens of look-ahead, emits
// dx[t] = sum_j w[c, K-1-j] * d pre[t+j] (while t+j stays inside the document) and accumulates dw per tile in
// registers before one atomic add per (channel, tap).
//
// Role in the reference: the `causal_conv1d` package / FLA `ShortConvolution` used by the Gated-DeltaNet layers
// (src/lmms_engine/models/qwen3_5/qwen3_5_ops.py:138-298).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace b200 {

constexpr int FWD_TILE = 64;    // tokens walked by one thread, forward
constexpr int BWD_TILE = 128;   // backward: also the span of one atomic add per (channel, tap)
constexpr int V = 2;            // neighbouring channels per thread (one 4-byte bf16x2 or 8-byte float2 access)

__device__ __forceinline__ void load2(const float* p, float o[2]) {
  const float2 v = *reinterpret_cast<const float2*>(p);
  o[0] = v.x; o[1] = v.y;
}
__device__ __forceinline__ void load2(const __nv_bfloat16* p, float o[2]) {
  const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
  o[0] = v.x; o[1] = v.y;
}
__device__ __forceinline__ void store2(float* p, const float o[2]) { *reinterpret_cast<float2*>(p) = make_float2(o[0], o[1]); }
__device__ __forceinline__ void store2(__nv_bfloat16* p, const float o[2]) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(o[0], o[1]);
}

template <typename T, int K>
__global__ void __launch_bounds__(128) conv_silu_fwd_kernel(const T* __restrict__ x, const float* __restrict__ w,
                                                            const int* __restrict__ pos, T* __restrict__ y, long tokens,
                                                            int channels) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * V;
  if (c >= channels) return;
  const long t0 = static_cast<long>(blockIdx.y) * FWD_TILE;
  float wk[K][V], win[K][V];  // win[j] = x[t-j]
#pragma unroll
  for (int j = 0; j < K; ++j)
#pragma unroll
    for (int v = 0; v < V; ++v) wk[j][v] = w[static_cast<long>(c + v) * K + (K - 1 - j)];
#pragma unroll
  for (int j = 1; j < K; ++j) {
    if (t0 - j >= 0) load2(x + (t0 - j) * channels + c, win[j]);
    else win[j][0] = win[j][1] = 0.f;
  }
  const long t1 = min(t0 + FWD_TILE, tokens);
#pragma unroll 4
  for (long t = t0; t < t1; ++t) {
    load2(x + t * channels + c, win[0]);
    const int p = pos[t];
    float pre[V] = {0.f, 0.f}, out[V];
#pragma unroll
    for (int j = 0; j < K; ++j)
      if (j <= p) {
#pragma unroll
        for (int v = 0; v < V; ++v) pre[v] += wk[j][v] * win[j][v];
      }
#pragma unroll
    for (int v = 0; v < V; ++v) out[v] = pre[v] / (1.f + __expf(-pre[v]));
    store2(y + t * channels + c, out);
#pragma unroll
    for (int j = K - 1; j > 0; --j)
#pragma unroll
      for (int v = 0; v < V; ++v) win[j][v] = win[j - 1][v];
  }
}

template <typename T, int K>
__global__ void __launch_bounds__(128) conv_silu_bwd_kernel(const T* __restrict__ x, const float* __restrict__ w,
                                                            const int* __restrict__ pos, const T* __restrict__ dy,
                                                            T* __restrict__ dx, float* __restrict__ dw, long tokens,
                                                            int channels) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * V;
  if (c >= channels) return;
  const long t0 = static_cast<long>(blockIdx.y) * BWD_TILE;
  const long t1 = min(t0 + BWD_TILE, tokens);
  float wk[K][V], win[K][V], dpre[K][V], dwk[K][V];  // dpre[j] = d pre[u-j] of the token u being visited
  int pos_ring[K];                                   // pos_ring[j] = pos[u-j]
#pragma unroll
  for (int j = 0; j < K; ++j) {
    pos_ring[j] = 0;
#pragma unroll
    for (int v = 0; v < V; ++v) {
      wk[j][v] = w[static_cast<long>(c + v) * K + (K - 1 - j)];
      dpre[j][v] = 0.f;
      dwk[j][v] = 0.f;
    }
  }
#pragma unroll
  for (int j = 1; j < K; ++j) {
    if (t0 - j >= 0) load2(x + (t0 - j) * channels + c, win[j]);
    else win[j][0] = win[j][1] = 0.f;
  }
  // visit the tile and K-1 tokens after it: token u closes the window of dx[u-K+1]
#pragma unroll 2
  for (long u = t0; u < t1 + K - 1; ++u) {
#pragma unroll
    for (int j = K - 1; j > 0; --j) {
      pos_ring[j] = pos_ring[j - 1];
#pragma unroll
      for (int v = 0; v < V; ++v) dpre[j][v] = dpre[j - 1][v];
    }
    if (u < tokens) {
      float g[V];
      load2(x + u * channels + c, win[0]);
      load2(dy + u * channels + c, g);
      const int p = pos[u];
      pos_ring[0] = p;
#pragma unroll
      for (int v = 0; v < V; ++v) {
        float pre = 0.f;
#pragma unroll
        for (int j = 0; j < K; ++j)
          if (j <= p) pre += wk[j][v] * win[j][v];
        const float s = 1.f / (1.f + __expf(-pre));
        const float d = g[v] * (s + pre * s * (1.f - s));
        dpre[0][v] = d;
        if (u < t1) {  // every token's weight gradient is counted by the tile that owns it
#pragma unroll
          for (int j = 0; j < K; ++j)
            if (j <= p) dwk[j][v] += d * win[j][v];
        }
      }
#pragma unroll
      for (int j = K - 1; j > 0; --j)
#pragma unroll
        for (int v = 0; v < V; ++v) win[j][v] = win[j - 1][v];
    } else {
      dpre[0][0] = dpre[0][1] = 0.f;
      pos_ring[0] = -1;  // past the end of the stream: contributes nothing
    }
    const long t = u - (K - 1);
    if (t >= t0 && t < t1) {
      // dx[t] = sum_j wk[j] * d pre[t+j] for the t+j that see t, i.e. pos[t+j] >= j; t+j = u-(K-1-j) -> ring index K-1-j
      float acc[V] = {0.f, 0.f};
#pragma unroll
      for (int j = 0; j < K; ++j)
        if (pos_ring[K - 1 - j] >= j) {
#pragma unroll
          for (int v = 0; v < V; ++v) acc[v] += wk[j][v] * dpre[K - 1 - j][v];
        }
      store2(dx + t * channels + c, acc);
    }
  }
#pragma unroll
  for (int j = 0; j < K; ++j)
#pragma unroll
    for (int v = 0; v < V; ++v) atomicAdd(dw + static_cast<long>(c + v) * K + (K - 1 - j), dwk[j][v]);
}

template <typename T>
int launch_fwd(const void* x, const void* w, const void* pos, void* y, long tokens, int channels, int K, cudaStream_t st) {
  const dim3 grid((channels / V + 127) / 128, static_cast<unsigned>((tokens + FWD_TILE - 1) / FWD_TILE));
#define B200_CONV_FWD(KK)                                                                                          \
  conv_silu_fwd_kernel<T, KK><<<grid, 128, 0, st>>>(static_cast<const T*>(x), static_cast<const float*>(w),         \
                                                     static_cast<const int*>(pos), static_cast<T*>(y), tokens, channels)
  if (K == 2) B200_CONV_FWD(2);
  else if (K == 3) B200_CONV_FWD(3);
  else if (K == 4) B200_CONV_FWD(4);
  else return -2;
#undef B200_CONV_FWD
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

template <typename T>
int launch_bwd(const void* x, const void* w, const void* pos, const void* dy, void* dx, void* dw, long tokens,
               int channels, int K, cudaStream_t st) {
  const dim3 grid((channels / V + 127) / 128, static_cast<unsigned>((tokens + BWD_TILE - 1) / BWD_TILE));
#define B200_CONV_BWD(KK)                                                                                          \
  conv_silu_bwd_kernel<T, KK><<<grid, 128, 0, st>>>(static_cast<const T*>(x), static_cast<const float*>(w),         \
                                                     static_cast<const int*>(pos), static_cast<const T*>(dy),       \
                                                     static_cast<T*>(dx), static_cast<float*>(dw), tokens, channels)
  if (K == 2) B200_CONV_BWD(2);
  else if (K == 3) B200_CONV_BWD(3);
  else if (K == 4) B200_CONV_BWD(4);
  else return -2;
#undef B200_CONV_BWD
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace b200

// x, y, dy, dx: [tokens, channels] contiguous, bf16 (is_bf16 = 1) or fp32, channels even and the base pointers 8-byte
// aligned (two channels move per access); w, dw: [channels, K] fp32 (dw zeroed by the caller); pos: [tokens] int32
// position inside the document.  K in {2, 3, 4}.
extern "C" int b200_conv_silu_fwd(const void* x, const void* w, const void* pos, void* y, long tokens, int channels,
                                  int K, int is_bf16, cudaStream_t st) {
  if (tokens <= 0 || channels <= 0) return 0;
  if (tokens > 65535L * b200::FWD_TILE || channels % b200::V) return -3;
  return is_bf16 ? b200::launch_fwd<__nv_bfloat16>(x, w, pos, y, tokens, channels, K, st)
                 : b200::launch_fwd<float>(x, w, pos, y, tokens, channels, K, st);
}

extern "C" int b200_conv_silu_bwd(const void* x, const void* w, const void* pos, const void* dy, void* dx, void* dw,
                                  long tokens, int channels, int K, int is_bf16, cudaStream_t st) {
  if (tokens <= 0 || channels <= 0) return 0;
  if (tokens > 65535L * b200::BWD_TILE || channels % b200::V) return -3;
  return is_bf16 ? b200::launch_bwd<__nv_bfloat16>(x, w, pos, dy, dx, dw, tokens, channels, K, st)
                 : b200::launch_bwd<float>(x, w, pos, dy, dx, dw, tokens, channels, K, st);
}
