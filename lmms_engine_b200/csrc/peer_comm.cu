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

// ---------------------------------------------------------------- bucketed reduce-to-owner
// The gradients of one bucket (the parameters of one decoder layer) are final on this rank as soon
// as its backward has passed the layer.  One launch on a side stream then
//   1. tells every peer so: pad_r[flag_off + self] = epoch                       (block 0)
//   2. waits, bounded, until every peer has said the same about this bucket      (every block)
//   3. pulls the ranges of the bucket that this rank owns from all peers, sums them in fp32 and
//      writes the sum over its own copy.
// The backward of the remaining layers keeps running on the main stream meanwhile, so only the
// last bucket's transfer is exposed.  A rank that owns nothing in a bucket still launches (steps 1-2
// with an empty range list).  A wait that runs out raises the status word and the kernel carries on
// with what is there: the optimizer's skip flag reads the same word, so such a step changes nothing.
constexpr int kMaxRanges = 8;
struct RangeList {
  long lo[kMaxRanges];    // first element of the range in the flat buffer
  long nvec[kMaxRanges];  // 16-byte vectors in the range
  int n;
};

template <typename T>
struct Vec16;
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int kElems = 8;
  static __device__ __forceinline__ void add(const uint4& v, float* acc) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(w[j]);
      acc[2 * j] += f.x;
      acc[2 * j + 1] += f.y;
    }
  }
  static __device__ __forceinline__ uint4 pack(const float* acc, float scale) {
    return make_uint4(pack_bf16x2(acc[0] * scale, acc[1] * scale), pack_bf16x2(acc[2] * scale, acc[3] * scale),
                      pack_bf16x2(acc[4] * scale, acc[5] * scale), pack_bf16x2(acc[6] * scale, acc[7] * scale));
  }
};
template <>
struct Vec16<float> {
  static constexpr int kElems = 4;
  static __device__ __forceinline__ void add(const uint4& v, float* acc) {
    acc[0] += __uint_as_float(v.x);
    acc[1] += __uint_as_float(v.y);
    acc[2] += __uint_as_float(v.z);
    acc[3] += __uint_as_float(v.w);
  }
  static __device__ __forceinline__ uint4 pack(const float* acc, float scale) {
    return make_uint4(__float_as_uint(acc[0] * scale), __float_as_uint(acc[1] * scale), __float_as_uint(acc[2] * scale),
                      __float_as_uint(acc[3] * scale));
  }
};

template <typename T>
__global__ void peer_bucket_reduce_kernel(PeerPtrs grads, PeerPtrs pads, int n, int self, int flag_off,
                                          unsigned int epoch, RangeList rl, float scale, int* status,
                                          long long cycle_limit) {
  const int t = threadIdx.x;
  if (blockIdx.x == 0 && t < n) {
    __threadfence_system();
    unsigned int* remote = static_cast<unsigned int*>(pads.p[t]) + flag_off + self;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
  }
  if (rl.n == 0) return;
  if (t < n) {
    const unsigned int* mine = static_cast<const unsigned int*>(pads.p[self]) + flag_off + t;
    const long long t0 = clock64();
    unsigned int v = 0;
    for (;;) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if (static_cast<int>(v - epoch) >= 0) break;
      if (clock64() - t0 > cycle_limit) {
        if (status != nullptr) atomicExch(status, kStatusPeerTimeout);
        break;
      }
      __nanosleep(500);
    }
  }
  __syncthreads();
  long total = 0;
  for (int r = 0; r < rl.n; ++r) total += rl.nvec[r];
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + t; i < total; i += static_cast<long>(gridDim.x) * blockDim.x) {
    long j = i;
    int r = 0;
    while (j >= rl.nvec[r]) {
      j -= rl.nvec[r];
      ++r;
    }
    const long off = rl.lo[r] + j * Vec16<T>::kElems;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    uint4 v[kMaxPeers > 8 ? 8 : kMaxPeers];
    // issue the loads of up to eight peers before the first add: eight 16-byte requests in flight per thread
    for (int r0 = 0; r0 < n; r0 += 8) {
      const int m = min(8, n - r0);
#pragma unroll
      for (int q = 0; q < 8; ++q)
        if (q < m) {
          const int src = (self + r0 + q) % n;  // a different first peer on every rank spreads the load over the links
          v[q] = *reinterpret_cast<const uint4*>(static_cast<const T*>(grads.p[src]) + off);
        }
#pragma unroll
      for (int q = 0; q < 8; ++q)
        if (q < m) Vec16<T>::add(v[q], acc);
    }
    *reinterpret_cast<uint4*>(static_cast<T*>(grads.p[self]) + off) = Vec16<T>::pack(acc, scale);
  }
}

// ---------------------------------------------------------------- gradient slots of the parameter-sharded runtime
// Every rank has written the gradients of one block into the same peer-mapped slot.  The owner of a
// parameter pulls it from all ranks' slots, sums in fp32 and ADDS the sum to its own gradient range
// (fp32 or bf16).  Flags: `ready` (this rank's slot content is final: raised on every peer, waited for
// before the pull) and `ack` (this rank no longer reads the peers' slots: raised on every peer by the
// last block to finish; a rank rewrites a slot only after all acknowledgements of its previous use).
constexpr int kMaxItems = 16;
struct ItemList {
  long slot_off[kMaxItems];  // first element in the slot
  long own_off[kMaxItems];   // first element in the owner's gradient range
  long nvec[kMaxItems];      // 16-byte vectors of the slot's dtype
  int n;
};
__device__ unsigned int g_slot_done[64];

template <typename ST, typename OT>
__global__ void peer_slot_reduce_kernel(PeerPtrs slots, PeerPtrs pads, int n, int self, int ready_off, unsigned int epoch,
                                        int do_signal, ItemList il, OT* __restrict__ g_own, int* status,
                                        long long cycle_limit, int do_ack, int ack_off, unsigned int ack_value) {
  const int t = threadIdx.x;
  if (do_signal && blockIdx.x == 0 && t < n) {
    __threadfence_system();
    unsigned int* remote = static_cast<unsigned int*>(pads.p[t]) + ready_off + self;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
  }
  if (il.n > 0) {
    if (t < n) {
      const unsigned int* mine = static_cast<const unsigned int*>(pads.p[self]) + ready_off + t;
      const long long t0 = clock64();
      unsigned int v = 0;
      for (;;) {
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
        if (static_cast<int>(v - epoch) >= 0) break;
        if (clock64() - t0 > cycle_limit) {
          if (status != nullptr) atomicExch(status, kStatusPeerTimeout);
          break;
        }
        __nanosleep(500);
      }
    }
    __syncthreads();
    long total = 0;
    for (int r = 0; r < il.n; ++r) total += il.nvec[r];
    constexpr int E = Vec16<ST>::kElems;
    for (long i = blockIdx.x * static_cast<long>(blockDim.x) + t; i < total; i += static_cast<long>(gridDim.x) * blockDim.x) {
      long j = i;
      int r = 0;
      while (j >= il.nvec[r]) {
        j -= il.nvec[r];
        ++r;
      }
      const long soff = il.slot_off[r] + j * E;
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      uint4 v[8];
      for (int r0 = 0; r0 < n; r0 += 8) {
        const int m = min(8, n - r0);
#pragma unroll
        for (int q = 0; q < 8; ++q)
          if (q < m) v[q] = *reinterpret_cast<const uint4*>(static_cast<const ST*>(slots.p[(self + r0 + q) % n]) + soff);
#pragma unroll
        for (int q = 0; q < 8; ++q)
          if (q < m) Vec16<ST>::add(v[q], acc);
      }
      OT* out = g_own + il.own_off[r] + j * E;
#pragma unroll
      for (int e = 0; e < E; ++e) out[e] = static_cast<OT>(static_cast<float>(out[e]) + acc[e]);
    }
  }
  if (do_ack) {
    // the last block to get here has seen every other block finish its loads
    __shared__ unsigned int last;
    __threadfence();
    __syncthreads();
    unsigned int* counter = &g_slot_done[(ack_off >> 5) & 63];
    if (t == 0) last = (atomicAdd(counter, 1u) == gridDim.x - 1) ? 1u : 0u;
    __syncthreads();
    if (last) {
      if (t == 0) *counter = 0;
      if (t < n) {
        __threadfence_system();
        unsigned int* remote = static_cast<unsigned int*>(pads.p[t]) + ack_off + self;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(ack_value) : "memory");
      }
    }
  }
}

// Wait (bounded) until the n flags pad_self[off .. off + n) have all reached `value`.
__global__ void peer_wait_flags_kernel(PeerPtrs pads, int n, int self, int off, unsigned int value, int* status,
                                       long long cycle_limit) {
  const int t = threadIdx.x;
  if (t < n) {
    const unsigned int* mine = static_cast<const unsigned int*>(pads.p[self]) + off + t;
    const long long t0 = clock64();
    unsigned int v = 0;
    for (;;) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if (static_cast<int>(v - value) >= 0) break;
      if (clock64() - t0 > cycle_limit) {
        if (status != nullptr) atomicExch(status, kStatusPeerTimeout);
        break;
      }
      __nanosleep(500);
    }
  }
}

// ---------------------------------------------------------------- owner update + publish in one pass
// AdamW on the slice of the flat buffers that this rank owns; the new bf16 value of every element is
// stored into ALL replicas (this rank's included) from the same registers, so no separate publish
// pass reads the parameters again.  `p32`, `m`, `v` are the owner's fp32 slices (element 0 = flat
// element `lo`); `g` is the reduced gradient at flat element `lo`.  n % 8 == 0, lo % 8 == 0.
template <typename GT>
__global__ void peer_adamw_kernel(PeerPtrs params, int n_ranks, int self, long lo, float* __restrict__ p32,
                                  float* __restrict__ m, float* __restrict__ v, const GT* __restrict__ g, long n8,
                                  float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                                  const float* gscale, const int* skip) {
  if (skip != nullptr && *skip) return;
  const float gs = gscale != nullptr ? *gscale : 1.f;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float gi[8], out[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) gi[j] = static_cast<float>(g[i * 8 + j]) * gs;
    float4 pa = reinterpret_cast<float4*>(p32)[2 * i], pb = reinterpret_cast<float4*>(p32)[2 * i + 1];
    float4 ma = reinterpret_cast<float4*>(m)[2 * i], mb = reinterpret_cast<float4*>(m)[2 * i + 1];
    float4 va = reinterpret_cast<float4*>(v)[2 * i], vb = reinterpret_cast<float4*>(v)[2 * i + 1];
    float pv[8] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
    float mv[8] = {ma.x, ma.y, ma.z, ma.w, mb.x, mb.y, mb.z, mb.w};
    float vv[8] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      mv[j] = beta1 * mv[j] + (1.f - beta1) * gi[j];
      vv[j] = beta2 * vv[j] + (1.f - beta2) * gi[j] * gi[j];
      float pi = pv[j] * (1.f - lr * wd);
      pi -= lr * (mv[j] / bc1) / (sqrtf(vv[j] / bc2) + eps);
      pv[j] = pi;
      out[j] = pi;
    }
    reinterpret_cast<float4*>(p32)[2 * i] = make_float4(pv[0], pv[1], pv[2], pv[3]);
    reinterpret_cast<float4*>(p32)[2 * i + 1] = make_float4(pv[4], pv[5], pv[6], pv[7]);
    reinterpret_cast<float4*>(m)[2 * i] = make_float4(mv[0], mv[1], mv[2], mv[3]);
    reinterpret_cast<float4*>(m)[2 * i + 1] = make_float4(mv[4], mv[5], mv[6], mv[7]);
    reinterpret_cast<float4*>(v)[2 * i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    reinterpret_cast<float4*>(v)[2 * i + 1] = make_float4(vv[4], vv[5], vv[6], vv[7]);
    const uint4 pk = make_uint4(pack_bf16x2(out[0], out[1]), pack_bf16x2(out[2], out[3]), pack_bf16x2(out[4], out[5]),
                                pack_bf16x2(out[6], out[7]));
    for (int r = 0; r < n_ranks; ++r) {
      const int dst = (self + r) % n_ranks;
      *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(params.p[dst]) + lo + i * 8) = pk;
    }
  }
}

// Muon: p = p*(1 - lr*wd) - lr*scale*o on the owner's fp32 master, new bf16 value into all replicas.
__global__ void peer_muon_update_kernel(PeerPtrs params, int n_ranks, int self, long lo, float* __restrict__ p32,
                                        const __nv_bfloat16* __restrict__ o, long n8, float lr, float wd, float scale,
                                        const int* skip) {
  if (skip != nullptr && *skip) return;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const uint4 ov = reinterpret_cast<const uint4*>(o)[i];
    const float2 o0 = unpack_bf16x2(ov.x), o1 = unpack_bf16x2(ov.y), o2 = unpack_bf16x2(ov.z), o3 = unpack_bf16x2(ov.w);
    const float od[8] = {o0.x, o0.y, o1.x, o1.y, o2.x, o2.y, o3.x, o3.y};
    float4 pa = reinterpret_cast<float4*>(p32)[2 * i], pb = reinterpret_cast<float4*>(p32)[2 * i + 1];
    float pv[8] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) pv[j] = pv[j] * (1.f - lr * wd) - lr * scale * od[j];
    reinterpret_cast<float4*>(p32)[2 * i] = make_float4(pv[0], pv[1], pv[2], pv[3]);
    reinterpret_cast<float4*>(p32)[2 * i + 1] = make_float4(pv[4], pv[5], pv[6], pv[7]);
    const uint4 pk = make_uint4(pack_bf16x2(pv[0], pv[1]), pack_bf16x2(pv[2], pv[3]), pack_bf16x2(pv[4], pv[5]),
                                pack_bf16x2(pv[6], pv[7]));
    for (int r = 0; r < n_ranks; ++r) {
      const int dst = (self + r) % n_ranks;
      *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(params.p[dst]) + lo + i * 8) = pk;
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

// One bucket of the overlapped reduce-to-owner (see peer_bucket_reduce_kernel).  `ranges` holds n_ranges
// pairs (first element, element count) of the flat buffer, each a multiple of 16 bytes; `max_blocks`
// bounds the grid so that the transfer shares the GPU with the backward pass.
int b200_peer_bucket_reduce(const void* const* grad_ptrs, const void* const* pad_ptrs, int n, int self, int is_fp32,
                            int flag_off, unsigned int epoch, const long* ranges, int n_ranges, float scale, int* status,
                            int timeout_ms, int max_blocks, cudaStream_t st) {
  if (n <= 1) return 0;
  if (n > kMaxPeers || n_ranges < 0) return -10;
  PeerPtrs gp{}, pp{};
  for (int i = 0; i < n; ++i) {
    gp.p[i] = const_cast<void*>(grad_ptrs[i]);
    pp.p[i] = const_cast<void*>(pad_ptrs[i]);
  }
  const long long limit = static_cast<long long>(timeout_ms) * 1900000LL;
  const int epv = is_fp32 ? 4 : 8;
  int done = 0;
  bool first = true;
  while (first || done < n_ranges) {
    RangeList rl{};
    long total = 0;
    for (; done < n_ranges && rl.n < kMaxRanges; ++done) {
      const long lo = ranges[2 * done], cnt = ranges[2 * done + 1];
      if (cnt <= 0) continue;
      if ((lo % epv) || (cnt % epv)) return -10;
      rl.lo[rl.n] = lo;
      rl.nvec[rl.n] = cnt / epv;
      total += cnt / epv;
      ++rl.n;
    }
    long blocks = (total + 255) / 256;
    if (blocks < 1) blocks = 1;
    if (max_blocks > 0 && blocks > max_blocks) blocks = max_blocks;
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (is_fp32)
      peer_bucket_reduce_kernel<float><<<static_cast<int>(blocks), 256, 0, st>>>(gp, pp, n, self, flag_off, epoch, rl, scale,
                                                                                status, limit);
    else
      peer_bucket_reduce_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 256, 0, st>>>(gp, pp, n, self, flag_off, epoch, rl,
                                                                                        scale, status, limit);
    first = false;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Gradient slot of the parameter-sharded runtime (see peer_slot_reduce_kernel).  `items` holds n_items
// triples (first element in the slot, first element in g_own, element count); counts are multiples of
// 8 elements.  Always raises this rank's ready flag and, when done, its acknowledgement.
int b200_peer_slot_reduce(const void* const* slot_ptrs, const void* const* pad_ptrs, int n, void* g_own, int self,
                          int slot_is_fp32, int own_is_fp32, int ready_off, const long* items, int n_items,
                          unsigned int epoch, int* status, int ack_off, unsigned int ack_value, int timeout_ms,
                          cudaStream_t st) {
  if (n <= 1) return 0;
  if (n > kMaxPeers || n_items < 0) return -10;
  PeerPtrs sp{}, pp{};
  for (int i = 0; i < n; ++i) {
    sp.p[i] = const_cast<void*>(slot_ptrs[i]);
    pp.p[i] = const_cast<void*>(pad_ptrs[i]);
  }
  const long long limit = static_cast<long long>(timeout_ms) * 1900000LL;
  const int epv = slot_is_fp32 ? 4 : 8;
  int done = 0;
  bool first = true;
  while (first || done < n_items) {
    ItemList il{};
    long total = 0;
    for (; done < n_items && il.n < kMaxItems; ++done) {
      const long so = items[3 * done], oo = items[3 * done + 1], cnt = items[3 * done + 2];
      if (cnt <= 0) continue;
      if ((so % epv) || (oo % 4) || (cnt % epv)) return -10;
      il.slot_off[il.n] = so;
      il.own_off[il.n] = oo;
      il.nvec[il.n] = cnt / epv;
      total += cnt / epv;
      ++il.n;
    }
    const int do_ack = done >= n_items;
    long blocks = (total + 255) / 256;
    if (blocks < 1) blocks = 1;
    if (blocks > 148 * 4) blocks = 148 * 4;
    const int sig = first ? 1 : 0;
#define LAUNCH_SLOT(ST, OT)                                                                                             \
  peer_slot_reduce_kernel<ST, OT><<<static_cast<int>(blocks), 256, 0, st>>>(sp, pp, n, self, ready_off, epoch, sig, il, \
                                                                            static_cast<OT*>(g_own), status, limit,     \
                                                                            do_ack, ack_off, ack_value)
    if (slot_is_fp32 && own_is_fp32) LAUNCH_SLOT(float, float);
    else if (!slot_is_fp32 && own_is_fp32) LAUNCH_SLOT(__nv_bfloat16, float);
    else if (!slot_is_fp32 && !own_is_fp32) LAUNCH_SLOT(__nv_bfloat16, __nv_bfloat16);
    else return -10;
#undef LAUNCH_SLOT
    first = false;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

int b200_peer_wait_flags(const void* const* pad_ptrs, int n, int self, int off, unsigned int value, int* status,
                         int timeout_ms, cudaStream_t st) {
  if (n <= 1) return 0;
  if (n > kMaxPeers) return -10;
  PeerPtrs pp{};
  for (int i = 0; i < n; ++i) pp.p[i] = const_cast<void*>(pad_ptrs[i]);
  peer_wait_flags_kernel<<<1, 32, 0, st>>>(pp, n, self, off, value, status, static_cast<long long>(timeout_ms) * 1900000LL);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

int b200_peer_adamw(const void* const* param_ptrs, int n, int self, long lo, void* p32, void* m, void* v, const void* g,
                    int g_is_fp32, long count, float lr, float beta1, float beta2, float eps, float wd, float bc1,
                    float bc2, const void* gscale, const void* skip, int max_blocks, cudaStream_t st) {
  if (count <= 0) return 0;
  if (n > kMaxPeers || (lo % 8) || (count % 8)) return -10;
  PeerPtrs pp{};
  for (int i = 0; i < n; ++i) pp.p[i] = const_cast<void*>(param_ptrs[i]);
  const long n8 = count / 8;
  long blocks = (n8 + 255) / 256;
  if (max_blocks > 0 && blocks > max_blocks) blocks = max_blocks;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (g_is_fp32)
    peer_adamw_kernel<float><<<static_cast<int>(blocks), 256, 0, st>>>(pp, n, self, lo, (float*)p32, (float*)m, (float*)v,
                                                                       (const float*)g, n8, lr, beta1, beta2, eps, wd, bc1,
                                                                       bc2, (const float*)gscale, (const int*)skip);
  else
    peer_adamw_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 256, 0, st>>>(
        pp, n, self, lo, (float*)p32, (float*)m, (float*)v, (const __nv_bfloat16*)g, n8, lr, beta1, beta2, eps, wd, bc1, bc2,
        (const float*)gscale, (const int*)skip);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

int b200_peer_muon_update(const void* const* param_ptrs, int n, int self, long lo, void* p32, const void* o, long count,
                          float lr, float wd, float scale, const void* skip, int max_blocks, cudaStream_t st) {
  if (count <= 0) return 0;
  if (n > kMaxPeers || (lo % 8) || (count % 8)) return -10;
  PeerPtrs pp{};
  for (int i = 0; i < n; ++i) pp.p[i] = const_cast<void*>(param_ptrs[i]);
  const long n8 = count / 8;
  long blocks = (n8 + 255) / 256;
  if (max_blocks > 0 && blocks > max_blocks) blocks = max_blocks;
  if (blocks > 148 * 8) blocks = 148 * 8;
  peer_muon_update_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(pp, n, self, lo, (float*)p32, (const __nv_bfloat16*)o, n8,
                                                                    lr, wd, scale, (const int*)skip);
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
