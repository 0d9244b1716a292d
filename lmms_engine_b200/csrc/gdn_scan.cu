// Sequential part of the chunked gated delta rule (Gated-DeltaNet linear attention), forward and backward.
//
// Per head the rule carries a state S [DK, dv] across chunks of C = 64 tokens:
//
//     v_new_i = u_i - w_i S_i          o_i = q~_i S_i          S_{i+1} = gamma_i S_i + k~_i^T v_new_i
//
// with S = 0 at the first chunk of every document (reset flag).  w, u (in-chunk corrected keys / values),
// q~ = q exp(g), k~ = k exp(g_last - g) and gamma = exp(g_last) are produced by batched PyTorch ops over
// all chunks at once; only this recurrence is inherently sequential, and as separate framework ops it costs
// about ten launches per chunk.  Here one CTA owns (head, 32 columns of dv): the state slice lives in shared
// memory for the whole sequence, every chunk's operands are staged in shared memory once, and all products
// run as register-tiled fp32 FMAs (the rule is evaluated in fp32 end to end).
//
// The backward kernel walks the chunks in reverse with dS in shared memory, reading the forward's state
// history; sums over dv (dw, dq~, dk~, dgamma) are written as one partial per dv slice and added by the caller,
// which keeps the result independent of scheduling.
//
// Role in the reference: the `chunk_gated_delta_rule` Triton kernels of the FLA package used by
// src/lmms_engine/models/qwen3_5/qwen3_5_ops.py (gated delta net forward of the patched layers).
#include <cuda_runtime.h>

namespace b200 {

constexpr int DK = 128;   // key head dim
constexpr int C = 64;     // chunk length
constexpr int DVT = 32;   // dv columns per CTA
constexpr int LDK = DK + 4;   // padded rows: conflict-free column reads, 16-byte aligned float4 rows
constexpr int LDV = DVT + 4;
constexpr int THREADS = 256;

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }

__device__ __forceinline__ void cp_async16(float* dst_smem, const float* src) {
  const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(dst_smem));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// stage a [C, DK] fp32 block (contiguous in global memory) into padded shared memory with asynchronous 16-byte
// copies: the caller commits the group and waits for it before the block is read
__device__ __forceinline__ void stage_ck(float* dst, const float* __restrict__ src) {
  for (int idx = threadIdx.x; idx < C * DK / 4; idx += THREADS) {
    const int r = idx / (DK / 4), c4 = idx - r * (DK / 4);
    cp_async16(dst + r * LDK + c4 * 4, src + r * DK + c4 * 4);
  }
}

// stage the [rows, DVT] slice of a [rows, dv] block
__device__ __forceinline__ void stage_slice(float* dst, const float* __restrict__ src, int rows, int dv) {
  for (int idx = threadIdx.x; idx < rows * DVT / 4; idx += THREADS) {
    const int r = idx / (DVT / 4), c4 = idx - r * (DVT / 4);
    st4(dst + r * LDV + c4 * 4, ld4(src + static_cast<long>(r) * dv + c4 * 4));
  }
}

// acc[2][4] += A[r0..r0+1][:] * B[:][c0..c0+3]   (A [C, DK] padded, B [DK, DVT] padded)
__device__ __forceinline__ void rows_times_state(const float* A, const float* B, int r0, int c0, float acc[2][4]) {
#pragma unroll 8
  for (int kk = 0; kk < DK; ++kk) {
    const float4 b = ld4(B + kk * LDV + c0);
    const float a0 = A[r0 * LDK + kk], a1 = A[(r0 + 1) * LDK + kk];
    acc[0][0] += a0 * b.x; acc[0][1] += a0 * b.y; acc[0][2] += a0 * b.z; acc[0][3] += a0 * b.w;
    acc[1][0] += a1 * b.x; acc[1][1] += a1 * b.y; acc[1][2] += a1 * b.z; acc[1][3] += a1 * b.w;
  }
}

// the same for two left operands that share B (one pass over the state)
__device__ __forceinline__ void rows_times_state2(const float* A1, const float* A2, const float* B, int r0, int c0,
                                                  float acc1[2][4], float acc2[2][4]) {
#pragma unroll 8
  for (int kk = 0; kk < DK; ++kk) {
    const float4 b = ld4(B + kk * LDV + c0);
    const float a0 = A1[r0 * LDK + kk], a1 = A1[(r0 + 1) * LDK + kk];
    const float q0 = A2[r0 * LDK + kk], q1 = A2[(r0 + 1) * LDK + kk];
    acc1[0][0] += a0 * b.x; acc1[0][1] += a0 * b.y; acc1[0][2] += a0 * b.z; acc1[0][3] += a0 * b.w;
    acc1[1][0] += a1 * b.x; acc1[1][1] += a1 * b.y; acc1[1][2] += a1 * b.z; acc1[1][3] += a1 * b.w;
    acc2[0][0] += q0 * b.x; acc2[0][1] += q0 * b.y; acc2[0][2] += q0 * b.z; acc2[0][3] += q0 * b.w;
    acc2[1][0] += q1 * b.x; acc2[1][1] += q1 * b.y; acc2[1][2] += q1 * b.z; acc2[1][3] += q1 * b.w;
  }
}

// acc[4][4] += sign * A[:, k0..k0+3]^T * V[:, c0..c0+3]   (A [C, DK] padded, V [C, DVT] padded)
__device__ __forceinline__ void transposed_times_rows(const float* A, const float* V, int k0, int c0, float sign,
                                                      float acc[4][4]) {
#pragma unroll 4
  for (int r = 0; r < C; ++r) {
    const float4 a = ld4(A + r * LDK + k0);
    float4 v = ld4(V + r * LDV + c0);
    v.x *= sign; v.y *= sign; v.z *= sign; v.w *= sign;
    acc[0][0] += a.x * v.x; acc[0][1] += a.x * v.y; acc[0][2] += a.x * v.z; acc[0][3] += a.x * v.w;
    acc[1][0] += a.y * v.x; acc[1][1] += a.y * v.y; acc[1][2] += a.y * v.z; acc[1][3] += a.y * v.w;
    acc[2][0] += a.z * v.x; acc[2][1] += a.z * v.y; acc[2][2] += a.z * v.z; acc[2][3] += a.z * v.w;
    acc[3][0] += a.w * v.x; acc[3][1] += a.w * v.y; acc[3][2] += a.w * v.z; acc[3][3] += a.w * v.w;
  }
}

__global__ void __launch_bounds__(THREADS, 1)
gdn_scan_fwd_kernel(const float* __restrict__ w, const float* __restrict__ u, const float* __restrict__ qt,
                    const float* __restrict__ kt, const float* __restrict__ gamma, const int* __restrict__ reset,
                    float* __restrict__ vnew, float* __restrict__ o, float* __restrict__ hist, int n, int dv) {
  extern __shared__ __align__(16) float smem[];
  float* sW = smem;
  float* sQ = sW + C * LDK;
  float* sK = sQ + C * LDK;
  float* sS = sK + C * LDK;    // [DK][LDV]
  float* sV = sS + DK * LDV;   // [C][LDV]
  const int h = blockIdx.x, slice = blockIdx.y, tid = threadIdx.x;
  const int ty = tid >> 3, tx = tid & 7;
  const int r0 = 2 * ty, k0 = 4 * ty, c0 = 4 * tx;
  for (int idx = tid; idx < DK * LDV; idx += THREADS) sS[idx] = 0.f;
  // operands of chunk 0; inside the loop the next chunk's w / q~ load while the state update runs, and the
  // chunk's k~ loads while the two products with the state run
  stage_ck(sW, w + static_cast<long>(h) * n * C * DK);
  stage_ck(sQ, qt + static_cast<long>(h) * n * C * DK);
  cp_async_commit();
  for (int i = 0; i < n; ++i) {
    const long chunk = static_cast<long>(h) * n + i;
    if (reset[i]) {
#pragma unroll
      for (int j = 0; j < 4; ++j) st4(sS + (k0 + j) * LDV + c0, make_float4(0.f, 0.f, 0.f, 0.f));
    }
    cp_async_wait_all();
    __syncthreads();
    stage_ck(sK, kt + chunk * C * DK);
    cp_async_commit();
    // state before this chunk, for the backward pass
    float* hrow = hist + chunk * DK * dv + static_cast<long>(slice) * DVT;
#pragma unroll
    for (int j = 0; j < 4; ++j) st4(hrow + static_cast<long>(k0 + j) * dv + c0, ld4(sS + (k0 + j) * LDV + c0));
    float p[2][4] = {}, oo[2][4] = {};
    rows_times_state2(sW, sQ, sS, r0, c0, p, oo);
    const long tok = chunk * C;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const long off = (tok + r0 + j) * dv + static_cast<long>(slice) * DVT + c0;
      const float4 uu = ld4(u + off);
      const float4 vn = make_float4(uu.x - p[j][0], uu.y - p[j][1], uu.z - p[j][2], uu.w - p[j][3]);
      st4(vnew + off, vn);
      st4(o + off, make_float4(oo[j][0], oo[j][1], oo[j][2], oo[j][3]));
      st4(sV + (r0 + j) * LDV + c0, vn);
    }
    cp_async_wait_all();
    __syncthreads();   // k~ and v_new are in shared memory; nobody reads w / q~ of this chunk any more
    if (i + 1 < n) {
      stage_ck(sW, w + (chunk + 1) * C * DK);
      stage_ck(sQ, qt + (chunk + 1) * C * DK);
    }
    cp_async_commit();
    const float g = gamma[chunk];
    float acc[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 sv = ld4(sS + (k0 + j) * LDV + c0);   // own tile: only this thread rewrites it
      acc[j][0] = g * sv.x; acc[j][1] = g * sv.y; acc[j][2] = g * sv.z; acc[j][3] = g * sv.w;
    }
    transposed_times_rows(sK, sV, k0, c0, 1.f, acc);
#pragma unroll
    for (int j = 0; j < 4; ++j) st4(sS + (k0 + j) * LDV + c0, make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]));
    // the loop-top barrier orders these writes (and the reads of k~ / v_new) before the next chunk's use
  }
  cp_async_wait_all();
}

// out[r][kk] = sign * sum_c A[r][c] * B[kk][c] for r in 4*ry..+3, kk = kx + 16 j (j < 8); A [C][LDV], B [DK][LDV]
__device__ __forceinline__ void rows_times_state_t(const float* A, const float* B, float sign, float* __restrict__ out,
                                                   int ry, int kx) {
  float acc[4][8] = {};
#pragma unroll 2
  for (int c4 = 0; c4 < DVT; c4 += 4) {
    float4 a[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = ld4(A + (4 * ry + i) * LDV + c4);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float4 b = ld4(B + (kx + 16 * j) * LDV + c4);
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[i][j] += a[i].x * b.x + a[i].y * b.y + a[i].z * b.z + a[i].w * b.w;
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) out[(4 * ry + i) * DK + kx + 16 * j] = sign * acc[i][j];
}

__global__ void __launch_bounds__(THREADS, 1)
gdn_scan_bwd_kernel(const float* __restrict__ w, const float* __restrict__ qt, const float* __restrict__ kt,
                    const float* __restrict__ gamma, const int* __restrict__ reset, const float* __restrict__ vnew,
                    const float* __restrict__ hist, const float* __restrict__ d_vnew, const float* __restrict__ d_o,
                    float* __restrict__ du, float* __restrict__ dw_p, float* __restrict__ dq_p, float* __restrict__ dk_p,
                    float* __restrict__ dgamma_p, int n, int dv, int H) {
  extern __shared__ __align__(16) float smem[];
  float* sW = smem;
  float* sQ = sW + C * LDK;
  float* sK = sQ + C * LDK;
  float* sS = sK + C * LDK;    // state before the chunk
  float* sD = sS + DK * LDV;   // gradient of the state after the chunk
  float* sV = sD + DK * LDV;   // v_new
  float* sO = sV + C * LDV;    // d_o
  float* sT = sO + C * LDV;    // total gradient of v_new
  __shared__ float red[THREADS / 32];
  const int h = blockIdx.x, slice = blockIdx.y, tid = threadIdx.x;
  const int ty = tid >> 3, tx = tid & 7;
  const int r0 = 2 * ty, k0 = 4 * ty, c0 = 4 * tx;
  const int ry = tid >> 4, kx = tid & 15;
  for (int idx = tid; idx < DK * LDV; idx += THREADS) sD[idx] = 0.f;
  for (int i = n - 1; i >= 0; --i) {
    const long chunk = static_cast<long>(h) * n + i;
    const long tok = chunk * C;
    const long col = static_cast<long>(slice) * DVT;
    stage_ck(sW, w + chunk * C * DK);     // asynchronous copies, in flight while the slices below are loaded
    stage_ck(sQ, qt + chunk * C * DK);
    stage_ck(sK, kt + chunk * C * DK);
    cp_async_commit();
    stage_slice(sS, hist + chunk * DK * dv + col, DK, dv);
    stage_slice(sV, vnew + tok * dv + col, C, dv);
    stage_slice(sO, d_o + tok * dv + col, C, dv);
    cp_async_wait_all();
    __syncthreads();
    // total gradient of v_new: what the caller saw plus what the state update carried forward
    float t[2][4] = {};
    rows_times_state(sK, sD, r0, c0, t);
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const long off = (tok + r0 + j) * dv + col + c0;
      const float4 e = ld4(d_vnew + off);
      const float4 tv = make_float4(t[j][0] + e.x, t[j][1] + e.y, t[j][2] + e.z, t[j][3] + e.w);
      st4(du + off, tv);
      st4(sT + (r0 + j) * LDV + c0, tv);
    }
    __syncthreads();
    const long part = ((static_cast<long>(slice) * H + h) * n + i) * C * DK;
    rows_times_state_t(sV, sD, 1.f, dk_p + part, ry, kx);    // d k~ = v_new dS^T
    rows_times_state_t(sT, sS, -1.f, dw_p + part, ry, kx);   // d w = -(total d v_new) S^T
    rows_times_state_t(sO, sS, 1.f, dq_p + part, ry, kx);    // d q~ = d_o S^T
    // d gamma = <dS, S>
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 d = ld4(sD + (k0 + j) * LDV + c0);
      const float4 s = ld4(sS + (k0 + j) * LDV + c0);
      dot += d.x * s.x + d.y * s.y + d.z * s.z + d.w * s.w;
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, m);
    if ((tid & 31) == 0) red[tid >> 5] = dot;
    __syncthreads();   // every read of the old dS is done; each thread rewrites only its own tile below
    if (tid == 0) {
      float s = 0.f;
#pragma unroll
      for (int m = 0; m < THREADS / 32; ++m) s += red[m];
      dgamma_p[(static_cast<long>(slice) * H + h) * n + i] = s;
    }
    // dS before the chunk = gamma dS + q~^T d_o - w^T (total d v_new); nothing flows into the previous document
    const float g = gamma[chunk];
    float acc[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 d = ld4(sD + (k0 + j) * LDV + c0);
      acc[j][0] = g * d.x; acc[j][1] = g * d.y; acc[j][2] = g * d.z; acc[j][3] = g * d.w;
    }
    transposed_times_rows(sQ, sO, k0, c0, 1.f, acc);
    transposed_times_rows(sW, sT, k0, c0, -1.f, acc);
    const bool cut = reset[i] != 0;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      st4(sD + (k0 + j) * LDV + c0, cut ? make_float4(0.f, 0.f, 0.f, 0.f)
                                        : make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]));
    __syncthreads();
  }
}

constexpr int kFwdSmem = (3 * C * LDK + DK * LDV + C * LDV) * 4;
constexpr int kBwdSmem = (3 * C * LDK + 2 * DK * LDV + 3 * C * LDV) * 4;

}  // namespace b200

// All tensors fp32 and contiguous: w, qt, kt [H, n, 64, 128]; u, vnew, o, d_* [H, n, 64, dv]; gamma [H, n];
// reset [n] int32; hist [H, n, 128, dv].  dv must be a multiple of 32.  Returns 0, or a negative code.
extern "C" int b200_gdn_scan_fwd(const void* w, const void* u, const void* qt, const void* kt, const void* gamma,
                                 const void* reset, void* vnew, void* o, void* hist, int H, int n, int dk, int dv,
                                 cudaStream_t st) {
  using namespace b200;
  if (dk != DK || dv % DVT != 0 || dv <= 0) return -2;
  if (H <= 0 || n <= 0) return 0;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(gdn_scan_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFwdSmem) != cudaSuccess) return -3;
    attr = true;
  }
  gdn_scan_fwd_kernel<<<dim3(H, dv / DVT), THREADS, kFwdSmem, st>>>(
      static_cast<const float*>(w), static_cast<const float*>(u), static_cast<const float*>(qt),
      static_cast<const float*>(kt), static_cast<const float*>(gamma), static_cast<const int*>(reset),
      static_cast<float*>(vnew), static_cast<float*>(o), static_cast<float*>(hist), n, dv);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// dw_p, dq_p, dk_p [dv/32, H, n, 64, 128] and dgamma_p [dv/32, H, n] are per-slice partial sums.
extern "C" int b200_gdn_scan_bwd(const void* w, const void* qt, const void* kt, const void* gamma, const void* reset,
                                 const void* vnew, const void* hist, const void* d_vnew, const void* d_o, void* du,
                                 void* dw_p, void* dq_p, void* dk_p, void* dgamma_p, int H, int n, int dk, int dv,
                                 cudaStream_t st) {
  using namespace b200;
  if (dk != DK || dv % DVT != 0 || dv <= 0) return -2;
  if (H <= 0 || n <= 0) return 0;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(gdn_scan_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwdSmem) != cudaSuccess) return -3;
    attr = true;
  }
  gdn_scan_bwd_kernel<<<dim3(H, dv / DVT), THREADS, kBwdSmem, st>>>(
      static_cast<const float*>(w), static_cast<const float*>(qt), static_cast<const float*>(kt),
      static_cast<const float*>(gamma), static_cast<const int*>(reset), static_cast<const float*>(vnew),
      static_cast<const float*>(hist), static_cast<const float*>(d_vnew), static_cast<const float*>(d_o),
      static_cast<float*>(du), static_cast<float*>(dw_p), static_cast<float*>(dq_p), static_cast<float*>(dk_p),
      static_cast<float*>(dgamma_p), n, dv, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
