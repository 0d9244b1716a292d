// Expert-parallel token exchange over peer-mapped memory: the dispatch and combine all-to-alls of a
// mixture-of-experts layer as row-mapped peer copies issued by this GPU's own warps.
//
//   push : row p of the local expert-sorted layout (token token_of_row[p] of x, optionally with a
//          per-row scalar) is stored straight into row dest_row[p] of rank dest_rank[p]'s
//          expert-major staging buffer; padding rows are stored as zeros.  The last CTA to finish
//          publishes this rank's epoch on every peer and waits for theirs, so when the kernel ends
//          everything destined to this rank has landed.
//   pull : out[t] = sum_i w[t,i] * peer(dest_rank[p]).buf[dest_row[p]], p = row_of[t,i]: the combine
//          all-to-all and the weighted scatter-add in one pass of peer loads.  The kernel starts
//          with an epoch handshake (every rank's staging buffer is ready).
//   pull_scalar : the same gather for one fp32 per row (router-weight gradients).
//
// Plain ld/st.global on peer addresses and system-scope flags only (no TMA, no multicast); every
// wait is bounded and raises the status word when it gives up.  Every index that addresses another
// rank's buffer is checked against the buffer's row capacity (and token indices against the token
// count): a bad entry is skipped and reported through the status word instead of being dereferenced.
//
// The reference moves these rows with all_to_all_single around a python expert loop
// (src/lmms_engine/parallel/expert_parallel/utils.py:11-77,
// src/lmms_engine/models/qwen3_moe/qwen3_moe_ops.py:257-296).
#include "common.cuh"

namespace b200 {

constexpr int kEpMaxRanks = 8;
struct EpPeers {
  void* buf[kEpMaxRanks];        // row staging buffer of every rank
  float* scalar[kEpMaxRanks];    // scalar staging buffer of every rank (may be null)
  uint32_t* flags[kEpMaxRanks];  // u32 [4][16] on every rank: push_arrive | pull_ready | scalar_ready | spare
};

__device__ __forceinline__ bool ep_wait_epoch(const uint32_t* flag, uint32_t epoch, long long limit, int* status) {
  const long long t0 = clock64();
  for (;;) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (static_cast<int>(v - epoch) >= 0) return true;
    if (clock64() - t0 > limit) {
      if (status != nullptr) atomicExch(status, kStatusPeerTimeout);
      return false;
    }
    __nanosleep(100);
  }
}

// one warp per row
__global__ void ep_push_kernel(const __nv_bfloat16* __restrict__ x, long ldx, const long long* __restrict__ token_of_row,
                               const float* __restrict__ scalar_of_row, const int* __restrict__ dest_rank,
                               const int* __restrict__ dest_row, long n_rows, int H, long ld_dst, EpPeers peers,
                               int world, int rank, uint32_t epoch, unsigned int* block_counter, int* status,
                               long long limit, long n_tokens, long cap_rows) {
  const int lane = threadIdx.x & 31;
  const long warp0 = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long n_warps = (static_cast<long>(gridDim.x) * blockDim.x) >> 5;
  const int vecs = H >> 3;
  for (long p = warp0; p < n_rows; p += n_warps) {
    const int r = dest_rank[p];
    if (r < 0) continue;  // row of an unused tile
    const long long tok = token_of_row[p];
    if (r >= world || dest_row[p] < 0 || dest_row[p] >= cap_rows || tok >= n_tokens) {
      if (lane == 0 && status != nullptr) atomicExch(status, kStatusOverflow);
      continue;
    }
    uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(peers.buf[r]) + static_cast<long>(dest_row[p]) * ld_dst);
    if (tok >= 0) {
      const uint4* src = reinterpret_cast<const uint4*>(x + tok * ldx);
      for (int v = lane; v < vecs; v += 32) dst[v] = src[v];
    } else {
      const uint4 z = make_uint4(0u, 0u, 0u, 0u);
      for (int v = lane; v < vecs; v += 32) dst[v] = z;
    }
    if (scalar_of_row != nullptr && lane == 0) peers.scalar[r][dest_row[p]] = tok >= 0 ? scalar_of_row[p] : 0.f;
  }
  // last CTA out: publish, then wait for every source
  __syncthreads();
  __shared__ bool last;
  if (threadIdx.x == 0) {
    __threadfence_system();
    last = atomicAdd(block_counter, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!last) return;
  if (threadIdx.x == 0) *block_counter = 0;
  if (static_cast<int>(threadIdx.x) < world) {
    const int r = threadIdx.x;
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peers.flags[r] + rank), "r"(epoch) : "memory");
    ep_wait_epoch(peers.flags[rank] + r, epoch, limit, status);
  }
}

// Epoch handshake at kernel start: CTA 0 publishes, every CTA waits (slot: 16 = pull, 32 = scalar).
__device__ __forceinline__ bool ep_start_handshake(const EpPeers& peers, int world, int rank, uint32_t epoch, int slot,
                                                    int* status, long long limit) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (static_cast<int>(threadIdx.x) < world) {
    const int r = threadIdx.x;
    if (blockIdx.x == 0) {
      __threadfence_system();
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peers.flags[r] + slot + rank), "r"(epoch) : "memory");
    }
    if (!ep_wait_epoch(peers.flags[rank] + slot + r, epoch, limit, status)) ok_s = 0;
  }
  __syncthreads();
  return ok_s != 0;
}

// one warp per token
__global__ void ep_pull_kernel(__nv_bfloat16* __restrict__ out, long ldo, const int* __restrict__ row_of,
                               const float* __restrict__ w, const int* __restrict__ dest_rank,
                               const int* __restrict__ dest_row, long T, int k, int H, long ld_src, EpPeers peers,
                               int world, int rank, uint32_t epoch, int* status, long long limit, long n_rows, long cap_rows) {
  if (!ep_start_handshake(peers, world, rank, epoch, 16, status, limit)) return;
  const int lane = threadIdx.x & 31;
  const long warp0 = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long n_warps = (static_cast<long>(gridDim.x) * blockDim.x) >> 5;
  const int vecs = H >> 3;
  for (long t = warp0; t < T; t += n_warps) {
    for (int v = lane; v < vecs; v += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int i = 0; i < k; ++i) {
        const int p = row_of[t * k + i];
        if (p < 0 || p >= n_rows || dest_rank[p] < 0 || dest_rank[p] >= world || dest_row[p] < 0 || dest_row[p] >= cap_rows) {
          if (status != nullptr) atomicExch(status, kStatusOverflow);
          continue;
        }
        const float wi = w != nullptr ? w[t * k + i] : 1.f;
        const uint4 u = *(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(peers.buf[dest_rank[p]]) +
                                                         static_cast<long>(dest_row[p]) * ld_src) + v);
        const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
        acc[0] += wi * f0.x; acc[1] += wi * f0.y; acc[2] += wi * f1.x; acc[3] += wi * f1.y;
        acc[4] += wi * f2.x; acc[5] += wi * f2.y; acc[6] += wi * f3.x; acc[7] += wi * f3.y;
      }
      reinterpret_cast<uint4*>(out + t * ldo)[v] =
          make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                     pack_bf16x2(acc[6], acc[7]));
    }
  }
}

__global__ void ep_pull_scalar_kernel(float* __restrict__ out, const int* __restrict__ row_of,
                                      const int* __restrict__ dest_rank, const int* __restrict__ dest_row, long n,
                                      EpPeers peers, int world, int rank, uint32_t epoch, int* status, long long limit,
                                      long n_rows, long cap_rows) {
  if (!ep_start_handshake(peers, world, rank, epoch, 32, status, limit)) return;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<long>(gridDim.x) * blockDim.x) {
    const int p = row_of[i];
    if (p < 0 || p >= n_rows || dest_rank[p] < 0 || dest_rank[p] >= world || dest_row[p] < 0 || dest_row[p] >= cap_rows) {
      if (status != nullptr) atomicExch(status, kStatusOverflow);
      out[i] = 0.f;
      continue;
    }
    out[i] = peers.scalar[dest_rank[p]][dest_row[p]];
  }
}

static int fill_peers(EpPeers& pp, const void* const* bufs, const void* const* scalars, const void* const* flags, int world) {
  if (world < 1 || world > kEpMaxRanks) return -10;
  for (int r = 0; r < world; ++r) {
    pp.buf[r] = const_cast<void*>(bufs[r]);
    pp.scalar[r] = scalars != nullptr ? static_cast<float*>(const_cast<void*>(scalars[r])) : nullptr;
    pp.flags[r] = static_cast<uint32_t*>(const_cast<void*>(flags[r]));
  }
  return 0;
}

}  // namespace b200

using namespace b200;

extern "C" {

// timeout_ms bounds every wait (converted with a nominal 1.9 GHz clock).
int b200_ep_push(const void* x, long ldx, const void* token_of_row, const void* scalar_of_row, const void* dest_rank,
                 const void* dest_row, long n_rows, int H, long ld_dst, const void* const* peer_bufs,
                 const void* const* peer_scalars, const void* const* peer_flags, int world, int rank, unsigned int epoch,
                 void* block_counter, int* status, int timeout_ms, long n_tokens, long cap_rows, cudaStream_t st) {
  if ((H & 7) || (ldx & 7) || (ld_dst & 7)) return -10;
  EpPeers pp{};
  if (fill_peers(pp, peer_bufs, scalar_of_row != nullptr ? peer_scalars : nullptr, peer_flags, world) != 0) return -10;
  long blocks = (n_rows * 32 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  ep_push_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(x), ldx, static_cast<const long long*>(token_of_row),
      static_cast<const float*>(scalar_of_row), static_cast<const int*>(dest_rank), static_cast<const int*>(dest_row), n_rows,
      H, ld_dst, pp, world, rank, epoch, static_cast<unsigned int*>(block_counter), status,
      static_cast<long long>(timeout_ms) * 1900000LL, n_tokens, cap_rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

int b200_ep_pull(void* out, long ldo, const void* row_of, const void* w, const void* dest_rank, const void* dest_row, long T,
                 int k, int H, long ld_src, const void* const* peer_bufs, const void* const* peer_flags, int world, int rank,
                 unsigned int epoch, int* status, int timeout_ms, long n_rows, long cap_rows, cudaStream_t st) {
  if (T <= 0) T = 0;
  if ((H & 7) || (ldo & 7) || (ld_src & 7)) return -10;
  EpPeers pp{};
  if (fill_peers(pp, peer_bufs, nullptr, peer_flags, world) != 0) return -10;
  long blocks = (T * 32 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;  // a rank without tokens still takes part in the handshake
  ep_pull_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(
      static_cast<__nv_bfloat16*>(out), ldo, static_cast<const int*>(row_of), static_cast<const float*>(w),
      static_cast<const int*>(dest_rank), static_cast<const int*>(dest_row), T, k, H, ld_src, pp, world, rank, epoch, status,
      static_cast<long long>(timeout_ms) * 1900000LL, n_rows, cap_rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

int b200_ep_pull_scalar(void* out, const void* row_of, const void* dest_rank, const void* dest_row, long n,
                        const void* const* peer_bufs, const void* const* peer_scalars, const void* const* peer_flags,
                        int world, int rank, unsigned int epoch, int* status, int timeout_ms, long n_rows, long cap_rows,
                        cudaStream_t st) {
  EpPeers pp{};
  if (fill_peers(pp, peer_bufs, peer_scalars, peer_flags, world) != 0) return -10;
  long blocks = (n + 255) / 256;
  if (blocks > 148 * 4) blocks = 148 * 4;
  if (blocks < 1) blocks = 1;
  ep_pull_scalar_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(
      static_cast<float*>(out), static_cast<const int*>(row_of), static_cast<const int*>(dest_rank),
      static_cast<const int*>(dest_row), n, pp, world, rank, epoch, status, static_cast<long long>(timeout_ms) * 1900000LL,
      n_rows, cap_rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // extern "C"
