// Short causal depthwise convolution + SiLU over a packed token stream, forward and backward, one pass each.
//
//     pre[t, c] = sum_{j = 0 .. K-1, j <= pos[t]} w[c, K-1-j] * x[t-j, c]        y = pre * sigmoid(pre)
//
// `pos[t]` is the token's position inside its document, so the window never reaches into the previous
// document.  One thread owns a channel (neighbouring threads neighbouring channels: coalesced rows) and walks a
// tile of tokens with the last K inputs in registers, so x and y cross HBM once.  The backward pass recomputes
// `pre`, forms d pre = dy * (s + pre * s * (1 - s)) for the tile plus K-1 tokens of look-ahead, emits
// dx[t] = sum_j w[c, K-1-j] * d pre[t+j] (while t+j stays inside the document) and accumulates dw per tile in
// registers before one atomic add per (channel, tap).
//
// Role in the reference: the `causal_conv1d` package / FLA `ShortConvolution` used by the Gated-DeltaNet layers
// (src/lmms_engine/models/qwen3_5/qwen3_5_ops.py:138-298).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace b200 {

constexpr int TOKENS_PER_TILE = 32;

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

template <typename T, int K>
__global__ void conv_silu_fwd_kernel(const T* __restrict__ x, const float* __restrict__ w, const int* __restrict__ pos,
                                     T* __restrict__ y, long tokens, int channels) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const long t0 = static_cast<long>(blockIdx.y) * TOKENS_PER_TILE;
  float wk[K], win[K];  // win[j] = x[t-j]
#pragma unroll
  for (int j = 0; j < K; ++j) wk[j] = w[static_cast<long>(c) * K + (K - 1 - j)];
#pragma unroll
  for (int j = 1; j < K; ++j) win[j] = (t0 - j >= 0) ? to_f(x[(t0 - j) * channels + c]) : 0.f;
  const long t1 = min(t0 + TOKENS_PER_TILE, tokens);
  for (long t = t0; t < t1; ++t) {
    win[0] = to_f(x[t * channels + c]);
    const int p = pos[t];
    float pre = 0.f;
#pragma unroll
    for (int j = 0; j < K; ++j)
      if (j <= p) pre += wk[j] * win[j];
    y[t * channels + c] = from_f<T>(pre / (1.f + __expf(-pre)));
#pragma unroll
    for (int j = K - 1; j > 0; --j) win[j] = win[j - 1];
  }
}

template <typename T, int K>
__global__ void conv_silu_bwd_kernel(const T* __restrict__ x, const float* __restrict__ w, const int* __restrict__ pos,
                                     const T* __restrict__ dy, T* __restrict__ dx, float* __restrict__ dw, long tokens,
                                     int channels) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const long t0 = static_cast<long>(blockIdx.y) * TOKENS_PER_TILE;
  const long t1 = min(t0 + TOKENS_PER_TILE, tokens);
  float wk[K], win[K], dpre[K], dwk[K];  // dpre[j] = d pre[u-j] of the token u being visited
#pragma unroll
  for (int j = 0; j < K; ++j) {
    wk[j] = w[static_cast<long>(c) * K + (K - 1 - j)];
    dpre[j] = 0.f;
    dwk[j] = 0.f;
  }
#pragma unroll
  for (int j = 1; j < K; ++j) win[j] = (t0 - j >= 0) ? to_f(x[(t0 - j) * channels + c]) : 0.f;
  int pos_ring[K];  // pos_ring[j] = pos[u-j]
#pragma unroll
  for (int j = 0; j < K; ++j) pos_ring[j] = 0;
  // visit the tile and K-1 tokens after it: token u closes the window of dx[u-K+1]
  for (long u = t0; u < t1 + K - 1; ++u) {
#pragma unroll
    for (int j = K - 1; j > 0; --j) {
      dpre[j] = dpre[j - 1];
      pos_ring[j] = pos_ring[j - 1];
    }
    if (u < tokens) {
      win[0] = to_f(x[u * channels + c]);
      const int p = pos[u];
      float pre = 0.f;
#pragma unroll
      for (int j = 0; j < K; ++j)
        if (j <= p) pre += wk[j] * win[j];
      const float s = 1.f / (1.f + __expf(-pre));
      const float d = to_f(dy[u * channels + c]) * (s + pre * s * (1.f - s));
      dpre[0] = d;
      pos_ring[0] = p;
      if (u < t1) {  // every token's weight gradient is counted by the tile that owns it
#pragma unroll
        for (int j = 0; j < K; ++j)
          if (j <= p) dwk[j] += d * win[j];
      }
#pragma unroll
      for (int j = K - 1; j > 0; --j) win[j] = win[j - 1];
    } else {
      dpre[0] = 0.f;
      pos_ring[0] = -1;  // past the end of the stream: contributes nothing
    }
    const long t = u - (K - 1);
    if (t >= t0 && t < t1) {
      // dx[t] = sum_j wk[j] * d pre[t+j] for the t+j that see t, i.e. pos[t+j] >= j; t+j = u-(K-1-j) -> ring index K-1-j
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < K; ++j)
        if (pos_ring[K - 1 - j] >= j) acc += wk[j] * dpre[K - 1 - j];
      dx[t * channels + c] = from_f<T>(acc);
    }
  }
#pragma unroll
  for (int j = 0; j < K; ++j) atomicAdd(dw + static_cast<long>(c) * K + (K - 1 - j), dwk[j]);
}

template <typename T>
int launch_fwd(const void* x, const void* w, const void* pos, void* y, long tokens, int channels, int K, cudaStream_t st) {
  const dim3 grid((channels + 127) / 128, static_cast<unsigned>((tokens + TOKENS_PER_TILE - 1) / TOKENS_PER_TILE));
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
  const dim3 grid((channels + 127) / 128, static_cast<unsigned>((tokens + TOKENS_PER_TILE - 1) / TOKENS_PER_TILE));
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

// x, y, dy, dx: [tokens, channels] contiguous, bf16 (is_bf16 = 1) or fp32; w, dw: [channels, K] fp32 (dw zeroed by the
// caller); pos: [tokens] int32 position inside the document.  K in {2, 3, 4}.
extern "C" int b200_conv_silu_fwd(const void* x, const void* w, const void* pos, void* y, long tokens, int channels,
                                  int K, int is_bf16, cudaStream_t st) {
  if (tokens <= 0 || channels <= 0) return 0;
  if (tokens > 65535L * b200::TOKENS_PER_TILE) return -3;
  return is_bf16 ? b200::launch_fwd<__nv_bfloat16>(x, w, pos, y, tokens, channels, K, st)
                 : b200::launch_fwd<float>(x, w, pos, y, tokens, channels, K, st);
}

extern "C" int b200_conv_silu_bwd(const void* x, const void* w, const void* pos, const void* dy, void* dx, void* dw,
                                  long tokens, int channels, int K, int is_bf16, cudaStream_t st) {
  if (tokens <= 0 || channels <= 0) return 0;
  if (tokens > 65535L * b200::TOKENS_PER_TILE) return -3;
  return is_bf16 ? b200::launch_bwd<__nv_bfloat16>(x, w, pos, dy, dx, dw, tokens, channels, K, st)
                 : b200::launch_bwd<float>(x, w, pos, dy, dx, dw, tokens, channels, K, st);
}
