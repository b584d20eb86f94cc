// Expert-parallel exchange over peer memory: the dispatch ("push") and the cross-GPU barrier.
//
// The reference has no multi-GPU code.  Experts are independent units, so every rank owns E/G experts
// and a 1/G slice of the tokens; what has to cross NVLink per layer is (a) every token's row to the
// ranks that own one of its experts, with its routes, and (b) one partial-sum row back per (token,
// rank) pair that did some work.  (a) is ep_push_kernel below, (b) is the combine kernel of route.cu
// writing through SegmentedOut; both use plain stores on addresses of buffers the peers mapped for each
// other.  Nothing here issues a TMA or multicast operation on peer memory.
#include "common.cuh"
#include "grouped.cuh"

namespace umaq {
namespace {

struct PushArgs {
  const __nv_bfloat16* x;
  const void* idx;
  int idx64;
  const float* w;
  int tokens, top_k, hidden, per_rank, placement, flags;
  umaq_ep_peers peers;
  size_t rows_offset, ids_offset, weights_offset;
  int* present;
};

__device__ __forceinline__ int owner_of(int e, int ranks, int per_rank, int placement) {
  if (e < 0 || e >= ranks * per_rank) return -1;
  return placement == 0 ? e % ranks : e / per_rank;
}

// One warp per (token, destination rank).  blockIdx.y walks the destinations starting after this rank,
// so that at any moment the ranks write to different peers.
constexpr int kPushWarps = 8;
__global__ void __launch_bounds__(kPushWarps * 32) ep_push_kernel(const PushArgs a) {
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * kPushWarps + (threadIdx.x >> 5);
  if (i >= a.tokens) return;
  const int G = a.peers.ranks, me = a.peers.rank;
  const int p = (me + 1 + (int)blockIdx.y) % G;
  uint8_t* base = static_cast<uint8_t*>(a.peers.base[p]);
  const size_t row = (size_t)me * a.tokens + i;
  // routes: ids as int32 and weights, always
  int e = -1;
  if (lane < a.top_k) {
    e = a.idx64 ? (int)reinterpret_cast<const long long*>(a.idx)[(size_t)i * a.top_k + lane]
                : reinterpret_cast<const int*>(a.idx)[(size_t)i * a.top_k + lane];
    // with UMAQ_EP_LOCAL_IDS the destination gets the id it would compute itself: local to it, or -1
    int id = e;
    if (a.flags & 1) {
      const bool theirs = owner_of(e, G, a.per_rank, a.placement) == p;
      id = !theirs ? -1 : (a.placement == 0 ? e / G : e - p * a.per_rank);
    }
    reinterpret_cast<int*>(base + a.ids_offset)[row * a.top_k + lane] = id;
    reinterpret_cast<float*>(base + a.weights_offset)[row * a.top_k + lane] = a.w[(size_t)i * a.top_k + lane];
  }
  const bool mine = lane < a.top_k && owner_of(e, G, a.per_rank, a.placement) == p;
  const bool wanted = __any_sync(0xffffffffu, mine);
  if (lane == 0) a.present[(size_t)i * G + p] = wanted ? p : -1;
  if (!wanted) return;
  const uint4* src = reinterpret_cast<const uint4*>(a.x + (size_t)i * a.hidden);
  uint4* dst = reinterpret_cast<uint4*>(base + a.rows_offset + row * a.hidden * 2);
  const int words = a.hidden >> 3;
  for (int b = 0; b < words; b += 256) {
    uint4 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (b + j * 32 + lane < words) v[j] = src[b + j * 32 + lane];
    if (a.flags & 2) {
      // k order of the quantised GEMMs: (k0,k1)(k2,k3)(k4,k5)(k6,k7) -> (k0,k4)(k1,k5)(k2,k6)(k3,k7) per run of 8
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint4 n = v[j];
        v[j] = make_uint4(prmt(n.x, n.z, 0x5410), prmt(n.x, n.z, 0x7632), prmt(n.y, n.w, 0x5410), prmt(n.y, n.w, 0x7632));
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (b + j * 32 + lane < words) dst[b + j * 32 + lane] = v[j];
  }
}

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Thread p signals rank p and waits for rank p.  Everything this rank wrote to peer memory in earlier
// kernels of the stream happens before the release store; everything the peers wrote before their
// signal is visible after the acquire load.
constexpr long long kBarrierWaitCycles = 4ll * 1000 * 1000 * 1000;      // ~2 s of SM clock
__global__ void ep_barrier_kernel(const umaq_ep_peers peers, size_t flags_offset, unsigned* epoch, unsigned* status) {
  const int p = threadIdx.x;
  const unsigned next = *epoch + 1;
  __syncthreads();
  if (p < peers.ranks) {
    unsigned* theirs = reinterpret_cast<unsigned*>(static_cast<uint8_t*>(peers.base[p]) + flags_offset);
    const unsigned* mine = reinterpret_cast<const unsigned*>(static_cast<uint8_t*>(peers.base[peers.rank]) + flags_offset);
    __threadfence_system();
    st_release_sys(theirs + peers.rank, next);
    const long long t0 = clock64();
    bool ok = false;
    for (;;) {
      if ((int)(ld_acquire_sys(mine + p) - next) >= 0) { ok = true; break; }
      if (clock64() - t0 > kBarrierWaitCycles) break;
      __nanosleep(64);
    }
    if (!ok) atomicExch(status, (unsigned)ERR_DEVICE_TIMEOUT);
  }
  __syncthreads();
  if (p == 0) *epoch = next;
}

}  // namespace

int launch_ep_push(const __nv_bfloat16* x, const void* indices, int idx64, const float* weights, int tokens, int top_k,
                   int hidden, int per_rank, int placement, int flags, const umaq_ep_peers& peers, size_t rows_offset,
                   size_t ids_offset, size_t weights_offset, int* present, cudaStream_t stream) {
  if (tokens <= 0 || top_k < 1 || top_k > 32 || hidden % 8 || per_rank < 1 || (placement != 0 && placement != 1) || (flags & ~3) ||
      peers.ranks < 1 || peers.ranks > kMaxPeers || peers.rank < 0 || peers.rank >= peers.ranks ||
      (rows_offset & 15) || (ids_offset & 3) || (weights_offset & 3)) {
    set_error("ep push: unsupported shape or peer table");
    return ERR_BAD_ARGUMENT;
  }
  for (int p = 0; p < peers.ranks; ++p)
    if (!peers.base[p]) { set_error("ep push: null peer buffer"); return ERR_BAD_ARGUMENT; }
  PushArgs a{x, indices, idx64, weights, tokens, top_k, hidden, per_rank, placement, flags, peers, rows_offset, ids_offset,
             weights_offset, present};
  ep_push_kernel<<<dim3((tokens + kPushWarps - 1) / kPushWarps, peers.ranks), kPushWarps * 32, 0, stream>>>(a);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("ep push: launch failed: %s", cudaGetErrorString(e)); return ERR_LAUNCH; }
  return ERR_NONE;
}

int launch_ep_barrier(const umaq_ep_peers& peers, size_t flags_offset, unsigned* epoch, unsigned* status,
                      cudaStream_t stream) {
  if (peers.ranks < 1 || peers.ranks > kMaxPeers || peers.rank < 0 || peers.rank >= peers.ranks || (flags_offset & 3)) {
    set_error("ep barrier: bad peer table");
    return ERR_BAD_ARGUMENT;
  }
  for (int p = 0; p < peers.ranks; ++p)
    if (!peers.base[p]) { set_error("ep barrier: null peer buffer"); return ERR_BAD_ARGUMENT; }
  ep_barrier_kernel<<<1, 32, 0, stream>>>(peers, flags_offset, epoch, status);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("ep barrier: launch failed: %s", cudaGetErrorString(e)); return ERR_LAUNCH; }
  return ERR_NONE;
}

}  // namespace umaq
