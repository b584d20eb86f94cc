// Streaming probes: kernels that only read a buffer, as a measured floor for the batch-1 decode call
// (how fast can one launch pull 27 MB or 105 MB out of HBM on this part, with nothing else to do).
// Two ways of reading, matching the two ways a decode kernel could be built:
//   mode 0: many CTAs, 16-byte ld.global.nc loads into registers, four in flight per thread;
//   mode 1: one persistent CTA per SM, cp.async.bulk copies of 8 KiB into a shared-memory ring issued by all
//           warps, completion on mbarriers, nothing consumes the bytes.
// Not part of the operator; the benchmark calls them through umaq_probe_stream.
#include "common.cuh"
#include "umaq_b200.h"

namespace umaq {
namespace {

constexpr int kProbeThreads = 256;
constexpr int kCopyBytes = 8192;
constexpr int kRingSlots = 24;                       // 192 KiB in flight per SM
constexpr long long kProbeWaitCycles = 200ll * 1000 * 1000;

__global__ void __launch_bounds__(kProbeThreads) probe_loads_kernel(const uint4* __restrict__ src, size_t n16,
                                                                    unsigned* __restrict__ sink) {
  const size_t stride = (size_t)gridDim.x * kProbeThreads;
  size_t i = (size_t)blockIdx.x * kProbeThreads + threadIdx.x;
  unsigned acc = 0;
  for (; i + 3 * stride < n16; i += 4 * stride) {
    uint4 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                   : "=r"(v[j].x), "=r"(v[j].y), "=r"(v[j].z), "=r"(v[j].w)
                   : "l"(src + i + j * stride));
#pragma unroll
    for (int j = 0; j < 4; ++j) acc ^= v[j].x ^ v[j].y ^ v[j].z ^ v[j].w;
  }
  for (; i < n16; i += stride) {
    const uint4 v = __ldg(src + i);
    acc ^= v.x ^ v.y ^ v.z ^ v.w;
  }
  if (acc == 0x9e3779b9u && sink) atomicAdd(sink, 1u);      // keeps the loads alive; practically never taken
}

__global__ void __launch_bounds__(kProbeThreads) probe_bulk_kernel(const uint8_t* __restrict__ src, size_t bytes,
                                                                   unsigned* __restrict__ status) {
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ uint64_t full[kRingSlots];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, warps = kProbeThreads / 32;
  if (tid == 0) {
    for (int s = 0; s < kRingSlots; ++s) mbar_init(full + s, 1);
    fence_barrier_init();
  }
  __syncthreads();
  // this CTA's share, in copies of 8 KiB (the last one of the buffer may be shorter, still a multiple of 16)
  const size_t copies = (bytes + kCopyBytes - 1) / kCopyBytes;
  const size_t c0 = copies * blockIdx.x / gridDim.x, c1 = copies * (blockIdx.x + 1) / gridDim.x;
  // Slot s of the ring belongs to warp s % warps: that warp issues the copy and is the only one that waits for
  // it, so a slot is free again as soon as its own barrier has flipped.
  const long long t0 = clock64();
  bool ok = true;
  for (size_t c = c0 + warp, n = 0; c < c1 && ok; c += warps, ++n) {
    const int slot = warp + (int)(n % (kRingSlots / warps)) * warps;
    const unsigned round = (unsigned)(n / (kRingSlots / warps));
    if (round > 0) {                                 // the copy that used this slot last must have landed
      while (!mbar_try_wait(full + slot, (round - 1) & 1)) {
        if (clock64() - t0 > kProbeWaitCycles) { ok = false; break; }
      }
      if (!ok) break;
    }
    if (lane == 0) {
      const size_t off = c * kCopyBytes;
      const uint32_t len = (uint32_t)(bytes - off < (size_t)kCopyBytes ? bytes - off : (size_t)kCopyBytes);
      mbar_expect_tx(full + slot, len);
      bulk_g2s(ring + (size_t)slot * kCopyBytes, src + off, len, full + slot);
    }
    __syncwarp();
  }
  // drain: every slot this warp used must have flipped for its last round
  const size_t mine = c1 > c0 + warp ? (c1 - c0 - warp + warps - 1) / warps : 0;
  for (size_t n = mine > (size_t)(kRingSlots / warps) ? mine - kRingSlots / warps : 0; n < mine && ok; ++n) {
    const int slot = warp + (int)(n % (kRingSlots / warps)) * warps;
    const unsigned round = (unsigned)(n / (kRingSlots / warps));
    while (!mbar_try_wait(full + slot, round & 1)) {
      if (clock64() - t0 > kProbeWaitCycles) { ok = false; break; }
    }
  }
  if (!ok && lane == 0 && status) atomicExch(status, (unsigned)ERR_DEVICE_TIMEOUT);
  if (!ok) __nanosleep(100000);                      // copies in flight land before the shared memory is given back
}

}  // namespace
}  // namespace umaq

extern "C" int umaq_probe_stream(const void* src, size_t bytes, int mode, void* status_u32, void* stream) {
  using namespace umaq;
  if (!src || bytes == 0 || bytes % 16 || (reinterpret_cast<uintptr_t>(src) & 15) || mode < 0 || mode > 1) {
    set_error("probe: needs a 16-byte aligned buffer, a size that is a multiple of 16 and mode 0 or 1");
    return ERR_BAD_ARGUMENT;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int sms = sm_count();
  if (mode == 0) {
    probe_loads_kernel<<<sms * 8, kProbeThreads, 0, st>>>(static_cast<const uint4*>(src), bytes / 16,
                                                          static_cast<unsigned*>(status_u32));
  } else {
    static thread_local int configured = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured != dev) {
      cudaError_t e = cudaFuncSetAttribute(probe_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kRingSlots * kCopyBytes);
      if (e != cudaSuccess) { set_error("probe: cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return ERR_LAUNCH; }
      configured = dev;
    }
    probe_bulk_kernel<<<sms, kProbeThreads, kRingSlots * kCopyBytes, st>>>(static_cast<const uint8_t*>(src), bytes,
                                                                          static_cast<unsigned*>(status_u32));
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("probe: launch: %s", cudaGetErrorString(e)); return ERR_LAUNCH; }
  return ERR_NONE;
}
