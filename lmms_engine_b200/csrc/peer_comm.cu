// Device-initiated collectives over peer-mapped (symmetric) memory for the owner-sharded
// runtime: every rank maps the flat gradient and parameter buffers of all ranks of its
// NVSwitch domain, so "reduce to owner" is the owner pulling its range from every peer and
// "publish" is the owner pushing its updated range into every replica.  Only plain
// ld/st.global on peer addresses are used (no TMA, no multicast), plus an epoch barrier
// on a small symmetric flag pad whose waits are bounded: a rank that gives up raises the
// status word and returns instead of spinning forever.
//
// The reference moves the same bytes with NCCL reduce-scatter / all-gather inside FSDP2
// and gather/scatter inside its Muon (src/lmms_engine/utils/muon_utils.py:234-272).
#include "common.cuh"

namespace b200 {

constexpr int kMaxPeers = 16;
struct PeerPtrs {
  void* p[kMaxPeers];
};

struct alignas(16) V8 {
  uint32_t w[4];
};

// out_local[lo + i] = scale * sum_r peer_r[lo + i]   (bf16 storage, fp32 sum), i in [0, count)
__global__ void peer_reduce_bf16_kernel(PeerPtrs peers, int n, int self, long lo, long count8, float scale) {
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < count8;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll 4
    for (int r = 0; r < n; ++r) {
      // start with a different peer on every rank so that the links are loaded evenly
      const int src = (self + r) % n;
      const V8 v = *(reinterpret_cast<const V8*>(static_cast<const __nv_bfloat16*>(peers.p[src]) + lo) + i);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(v.w[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    V8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) o.w[j] = pack_bf16x2(acc[2 * j] * scale, acc[2 * j + 1] * scale);
    *(reinterpret_cast<V8*>(static_cast<__nv_bfloat16*>(peers.p[self]) + lo) + i) = o;
  }
}

// peer_r[lo + i] = local[lo + i] for every r != self   (16-byte vectors; element size given in bytes)
__global__ void peer_publish_kernel(PeerPtrs peers, int n, int self, long lo_bytes, long count16) {
  const uint4* src = reinterpret_cast<const uint4*>(static_cast<const char*>(peers.p[self]) + lo_bytes);
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < count16;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const uint4 v = src[i];
    for (int r = 1; r < n; ++r) {
      const int dst = (self + r) % n;
      reinterpret_cast<uint4*>(static_cast<char*>(peers.p[dst]) + lo_bytes)[i] = v;
    }
  }
}

// Epoch barrier: rank `self` stores `epoch` into slot [self] of every peer's pad, then waits
// until all n slots of its own pad reached `epoch`.  Epochs only grow, so no reset is needed.
__global__ void peer_barrier_kernel(PeerPtrs pads, int n, int self, unsigned int epoch, int* status,
                                    long long cycle_limit) {
  const int t = threadIdx.x;
  if (t < n) {
    unsigned int* remote = static_cast<unsigned int*>(pads.p[t]) + self;
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
    const unsigned int* mine = static_cast<const unsigned int*>(pads.p[self]) + t;
    const long long t0 = clock64();
    unsigned int v = 0;
    for (;;) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if (static_cast<int>(v - epoch) >= 0) break;
      if (clock64() - t0 > cycle_limit) {
        if (status != nullptr) atomicExch(status, kStatusPeerTimeout);
        break;
      }
      __nanosleep(200);
    }
  }
}

// flags[i] += 1 with release semantics at system scope, one lane per flag: publishes what earlier
// operations of the stream (copy-engine transfers included) wrote into the peers' memory
__global__ void peer_signal_kernel(PeerPtrs flags, int n) {
  const int t = threadIdx.x;
  if (t < n) {
    __threadfence_system();
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(static_cast<unsigned int*>(flags.p[t])), "r"(1u) : "memory");
  }
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_peer_reduce_bf16(const void* const* peer_ptrs, int n, int self, long lo, long count, float scale,
                          cudaStream_t st) {
  if (count <= 0) return 0;
  if (n > kMaxPeers || (lo % 8) || (count % 8)) return -10;
  PeerPtrs pp{};
  for (int i = 0; i < n; ++i) pp.p[i] = const_cast<void*>(peer_ptrs[i]);
  const long c8 = count / 8;
  long blocks = (c8 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  peer_reduce_bf16_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(pp, n, self, lo, c8, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

int b200_peer_publish(const void* const* peer_ptrs, int n, int self, long lo_bytes, long n_bytes, cudaStream_t st) {
  if (n_bytes <= 0 || n <= 1) return 0;
  if (n > kMaxPeers || (lo_bytes % 16) || (n_bytes % 16)) return -10;
  PeerPtrs pp{};
  for (int i = 0; i < n; ++i) pp.p[i] = const_cast<void*>(peer_ptrs[i]);
  const long c16 = n_bytes / 16;
  long blocks = (c16 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  peer_publish_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(pp, n, self, lo_bytes, c16);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// timeout_ms bounds the wait (converted with a nominal 1.9 GHz clock).
int b200_peer_barrier(const void* const* pad_ptrs, int n, int self, unsigned int epoch, int* status, int timeout_ms,
                      cudaStream_t st) {
  if (n <= 1) return 0;
  if (n > kMaxPeers) return -10;
  PeerPtrs pp{};
  for (int i = 0; i < n; ++i) pp.p[i] = const_cast<void*>(pad_ptrs[i]);
  const long long limit = static_cast<long long>(timeout_ms) * 1900000LL;
  peer_barrier_kernel<<<1, 32, 0, st>>>(pp, n, self, epoch, status, limit);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// One device-to-device copy on the stream (copy engines; the destination may be a peer-mapped address).
int b200_peer_memcpy(void* dst, const void* src, long n_bytes, cudaStream_t st) {
  if (n_bytes <= 0) return 0;
  return cudaMemcpyAsync(dst, src, static_cast<size_t>(n_bytes), cudaMemcpyDeviceToDevice, st) == cudaSuccess ? 0 : -4;
}

// Pitched device-to-device copy (a column block of a matrix) on the stream.
int b200_peer_memcpy2d(void* dst, long dpitch, const void* src, long spitch, long width_bytes, long height, cudaStream_t st) {
  if (width_bytes <= 0 || height <= 0) return 0;
  return cudaMemcpy2DAsync(dst, static_cast<size_t>(dpitch), src, static_cast<size_t>(spitch), static_cast<size_t>(width_bytes),
                           static_cast<size_t>(height), cudaMemcpyDeviceToDevice, st) == cudaSuccess ? 0 : -4;
}

// Add one to each of the n flags (peer-mapped addresses), ordered after everything queued on the stream.
int b200_peer_signal(const void* const* flag_ptrs, int n, cudaStream_t st) {
  if (n <= 0) return 0;
  if (n > kMaxPeers) return -10;
  PeerPtrs pp{};
  for (int i = 0; i < n; ++i) pp.p[i] = const_cast<void*>(flag_ptrs[i]);
  peer_signal_kernel<<<1, 32, 0, st>>>(pp, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // extern "C"
