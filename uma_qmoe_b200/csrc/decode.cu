// Batch-1 decode: two kernels chained by programmatic dependent launch.
//
//   out = sum_slot w_slot * Down_e( SiLU(Gate_e x) * Up_e x )   (+ Qwen shared expert)
//
// replaces the reference's two-launch decode
// (src/uma_qmoe/native/packed_q4_kernel.cu:156-231 gate/up+SwiGLU, :1369-1426 down+route sum,
// launched from :1486-1533; Q8 twins :781-892) and the per-expert Python GEMV loops for Qwen
// (src/uma_qmoe/native_backend.py:319-372, :722-753).  Numerics follow the reference's CPU
// correctness path (src/uma_qmoe/custom_op.py:301-340, :465-506): float32 accumulation, one BF16
// rounding of every expert contribution and of the running sum, experts in ascending order; the
// intermediate SiLU(gate) * up travels between the kernels rounded once to BF16, as in the
// reference's own CUDA kernels (packed_q4_kernel.cu:228).
//
// The layer is ~27 MB (OLMoE Q4) to ~105 MB (Qwen Q8 + BF16 shared expert) of weights read exactly
// once: a pure HBM stream of a few microseconds, so everything is organised around keeping that
// stream busy from the first cycle.
//
//  * One CTA per SM per kernel.  A producer warp moves the CTA's weight rows and their group scales
//    into a shared-memory ring (cp.async.bulk for the rows, cp.async for the scales, one mbarrier per
//    stage); with the OLMoE shape a CTA's whole share (~120 KB gate/up, ~60 KB down) is in flight at
//    once.  Eight consumer warps split K: each takes 64-byte columns ("items") of the 16 MMA rows of
//    a stage, so no warp waits for another until the partial sums meet in shared memory.
//  * Both kernels carry the programmatic-stream-serialisation attribute.  The gate/up kernel waits
//    for its predecessor (the routes come from it), then lets the down kernel start: the down CTAs
//    become resident beside the gate/up CTAs (the two kernels' shared memory and registers fit one
//    SM together), stream their weights while gate/up computes, and only then wait for the
//    intermediate.  The down kernel in turn lets the next kernel of the stream start early.
//  * Dequantisation costs no per-weight arithmetic: a nibble becomes the exact BF16 value
//    128 + (code + 8) with one LOP3 per two weights (0x4300 | nibble) and goes straight into
//    m16n8k16 BF16 warp MMAs whose B operand is the activation vector, exact in BF16 as it is; the
//    constant 136 is removed by starting every accumulator at -136 * sum(x) of its 128-wide group,
//    and the group scale is applied once per group in float32.  Q8 bytes are split into two nibbles
//    that meet x and 16 x in the B operand, so they run through the same instructions.  On B200 the
//    HBM-to-issue-rate ratio leaves < 3 instructions per 4-bit weight, which rules out per-weight
//    FMA on the CUDA cores; the warp MMA does the multiply-add and the CUDA cores only unpack.
//  * Gate/up tile = 8 gate rows + 8 up rows of 8 features (column 0 of the MMA).  Down tile = 2
//    output rows x up to 8 routed slots: MMA row g holds slot g's weight row, MMA column g slot g's
//    intermediate, the diagonal of the product is what is kept -- all slots of an output row meet in
//    one CTA, which therefore does the ordered BF16 combine itself.  The BF16 shared expert enters
//    the same tiles with its K dimension cut into 8 segments in place of the slots.
#include "../../include/umaq_b200.h"
#include "common.cuh"
#include "decode.cuh"

#include <algorithm>
#include <cstdlib>
#include <mutex>

namespace umaq {
namespace {

constexpr int kNW = 8;                        // consumer warps; warp kNW is the producer
constexpr int kConsumers = kNW * 32;
constexpr int kThreadsD = (kNW + 1) * 32;
constexpr int kMaxSlots = 8;
// The two kernels share an SM: their dynamic shared memory together stays under kPairSmemBudget (228 KB per SM
// minus 1 KB reserve and the static arrays of each CTA).  The down kernel is planned first and takes what its
// whole share needs, up to kDownSmemMax; the gate/up kernel gets the rest.
constexpr int kPairSmemBudget = 224 * 1024;
constexpr int kDownSmemMax = 112 * 1024;
constexpr long long kDecodeWaitCycles = 40ll * 1000 * 1000;     // ~20 ms of SM clock: far beyond any healthy wait

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async8(void* dst_smem, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
// The barrier receives one arrival when all cp.async copies this thread issued so far have landed
// (the arrival is part of the barrier's initial count).
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Bounded wait that also gives up when another warp of the CTA has already failed.
__device__ __forceinline__ bool wait_or_fail(uint64_t* bar, uint32_t parity, volatile int* fail) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();                 // the SM's own counter: cheap to read inside a spin
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*fail || clock64() - t0 > kDecodeWaitCycles) { *fail = 1; return false; }
  }
}

// Measurement aid (debug bit 4): CTA 0 leaves %globaltimer stamps in the workspace header, 8 bytes each
// from byte 128 on.
__device__ __forceinline__ void stamp(const DecodeParams& p, int slot, int tid_wanted) {
  if ((p.debug & 4) && blockIdx.x == 0 && (int)threadIdx.x == tid_wanted)
    reinterpret_cast<unsigned long long*>(p.sync)[16 + slot] = global_ns();
}

__device__ __forceinline__ long long load_index(const void* idx, int idx64, int i) {
  return idx64 ? reinterpret_cast<const long long*>(idx)[i] : (long long)reinterpret_cast<const int*>(idx)[i];
}

// ---- shared-memory loads by 32-bit shared address ------------------------------------------------------
__device__ __forceinline__ uint4 lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a) : "memory");
  return v;
}
__device__ __forceinline__ float lds32(uint32_t a) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a) : "memory");
  return v;
}
__device__ __forceinline__ float2 lds64(uint32_t a) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a) : "memory");
  return v;
}

// ---- activation fragments ----------------------------------------------------------------------------
// An "item" is 64 bytes of each of the 16 MMA rows of a stage: 128 (Q4), 64 (Q8) or 32 (BF16)
// activations.  Byte offset of activation k of slot `vs` in a fragment buffer laid out
// [item][chunk r][slot][t] x 16 bytes: lane (g, t) of a warp reads, for item i and chunk r, the 16 bytes
// at ((i*R + r)*ng + slot)*64 + t*16 and uses them as the B registers of two MMAs (R = 4 chunks per item
// for Q4 / Q8, 1 for BF16).  Where a value sits inside its 16 bytes follows from how the weight codes
// leave their 32-bit words:
//   Q4   a lane's word holds 8 nibbles k0..k7; (w >> 4p) & 0x000F000F yields the pair (k_p, k_{p+4}),
//        so the 8 values are stored [k0,k4,k1,k5,k2,k6,k3,k7];
//   Q8   a word holds 4 bytes = nibbles (l0,h0,l1,h1,l2,h2,l3,h3); the same four extractions yield
//        (l0,l2), (h0,h2), (l1,l3), (h1,h3), which meet [x0,x2,16x0,16x2,x1,x3,16x1,16x3];
//   BF16 natural order.
// hi selects the 16 x copy of a Q8 value.
__host__ __device__ __forceinline__ int frag_offset(int enc, int ng, int vs, int k, int hi) {
  int item, r, t, e, nr;
  if (enc == ENC_Q4) {
    item = k >> 7; t = (k >> 5) & 3; r = (k >> 3) & 3; nr = 4;
    const int i = k & 7;
    e = 2 * (i & 3) + (i >> 2);
  } else if (enc == ENC_Q8) {
    item = k >> 6; t = (k >> 4) & 3; r = (k >> 2) & 3; nr = 4;
    const int b = k & 3, n = 2 * b + hi;
    e = 2 * (n & 3) + (b >> 1);
  } else {
    item = k >> 5; r = 0; t = (k >> 3) & 3; nr = 1;
    e = k & 7;
  }
  return ((((item * nr + r) * ng + vs) * 4 + t) << 4) + e * 2;
}

// x[0..n) -> fragments (one slot) and, for quantised rows, the sum of every item's activations.
// Called by the kConsumers consumer threads; n is a multiple of 256.
__device__ __forceinline__ void build_x_fragments(int enc, const __nv_bfloat16* __restrict__ x, int n, uint8_t* xf,
                                                  float* gsum, int tid) {
  for (int k0 = tid * 8; k0 < n; k0 += kConsumers * 8) {
    const uint4 raw = *reinterpret_cast<const uint4*>(x + k0);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint16_t bits = (uint16_t)(j & 1 ? w[j >> 1] >> 16 : w[j >> 1] & 0xffffu);
      const float v = __uint_as_float((uint32_t)bits << 16);
      sum += v;
      *reinterpret_cast<uint16_t*>(xf + frag_offset(enc, 1, 0, k0 + j, 0)) = bits;
      if (enc == ENC_Q8)
        *reinterpret_cast<__nv_bfloat16*>(xf + frag_offset(enc, 1, 0, k0 + j, 1)) = __float2bfloat16_rn(v * 16.f);
    }
    if (enc != ENC_BF16) {
      // an item is 128 (Q4) or 64 (Q8) activations = 16 or 8 neighbouring threads
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      sum += __shfl_xor_sync(0xffffffffu, sum, 4);
      if (enc == ENC_Q4) {
        sum += __shfl_xor_sync(0xffffffffu, sum, 8);
        if ((k0 & 127) == 0) gsum[k0 >> 7] = sum;
      } else if ((k0 & 63) == 0) {
        gsum[k0 >> 6] = sum;
      }
    }
  }
}

// ---- N items at once: 16 MMA rows x 64 bytes of weights each, against the fragments ---------------------
// a0[n]: shared address of this lane's 16 bytes of MMA row g of item n, a8off bytes further those of row
// g + 8; bp[n]: its fragment chunk 0, bstep bytes between chunks (SHARE_B: all items use bp[0]);
// i0 / i1: start values of the accumulator columns 2t and 2t+1 (-bias * activation sum).
// c[n][0], c[n][1] = row g, columns 2t, 2t+1; c[n][2], c[n][3] = row g + 8.  The items' MMA chains are
// independent and issued round-robin, so no warp MMA waits for the one before it.
template <uint32_t K>
__device__ __forceinline__ uint32_t nib_bf16(uint32_t w) { return lop3<0x6A>(w, 0x000F000Fu, K); }   // (w & m) ^ K

template <int ENC, int N, bool SHARE_B>
__device__ __forceinline__ void items_mma(const uint32_t (&a0)[N], uint32_t a8off, const uint32_t (&bp)[N], uint32_t bstep,
                                          const float (&i0)[N], const float (&i1)[N], float (&c)[N][4]) {
  uint4 wa[N], wb[N];
#pragma unroll
  for (int n = 0; n < N; ++n) { wa[n] = lds128(a0[n]); wb[n] = lds128(a0[n] + a8off); }
  if (ENC == ENC_BF16) {
    float acc[N][2][4];
#pragma unroll
    for (int n = 0; n < N; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[n][0][e] = acc[n][1][e] = 0.f;
    uint4 b = lds128(bp[0]);
#pragma unroll
    for (int n = 0; n < N; ++n) {
      if (!SHARE_B && n > 0) b = lds128(bp[n]);
      mma_bf16_16816(acc[n][0], wa[n].x, wb[n].x, wa[n].y, wb[n].y, b.x, b.y);
      mma_bf16_16816(acc[n][1], wa[n].z, wb[n].z, wa[n].w, wb[n].w, b.z, b.w);
    }
#pragma unroll
    for (int n = 0; n < N; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) c[n][e] = acc[n][0][e] + acc[n][1][e];
  } else {
    // BF16 128 + n: Q4 n = code + 8 (two's complement nibble ^ 8); Q8 low nibble as is, high nibble ^ 8
    constexpr uint32_t kLo = ENC == ENC_Q4 ? 0x43084308u : 0x43004300u, kHi = 0x43084308u;
    float acc[N][4][4];
#pragma unroll
    for (int n = 0; n < N; ++n) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[n][j][e] = 0.f;
      acc[n][0][0] = i0[n]; acc[n][0][1] = i1[n]; acc[n][0][2] = i0[n]; acc[n][0][3] = i1[n];
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint4 b = lds128(bp[0] + j * bstep);
#pragma unroll
      for (int n = 0; n < N; ++n) {
        if (!SHARE_B && n > 0) b = lds128(bp[n] + j * bstep);
        const uint32_t a = j == 0 ? wa[n].x : j == 1 ? wa[n].y : j == 2 ? wa[n].z : wa[n].w;
        const uint32_t a8 = j == 0 ? wb[n].x : j == 1 ? wb[n].y : j == 2 ? wb[n].z : wb[n].w;
        mma_bf16_16816(acc[n][j], nib_bf16<kLo>(a), nib_bf16<kLo>(a8), nib_bf16<kHi>(a >> 4), nib_bf16<kHi>(a8 >> 4), b.x, b.y);
        mma_bf16_16816(acc[n][j], nib_bf16<kLo>(a >> 8), nib_bf16<kLo>(a8 >> 8), nib_bf16<kHi>(a >> 12),
                       nib_bf16<kHi>(a8 >> 12), b.z, b.w);
      }
    }
#pragma unroll
    for (int n = 0; n < N; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) c[n][e] = (acc[n][0][e] + acc[n][1][e]) + (acc[n][2][e] + acc[n][3][e]);
  }
}

// First work unit of gate/up CTA c: units are weighted by their bytes, routed units first, and a CTA
// owns the units whose cost range starts inside [c, c+1) * total / grid.
__host__ __device__ __forceinline__ int first_unit(const DecodeKernelPlan& P, int c) {
  const long long x = ((long long)c * P.total_cost + P.grid - 1) / P.grid;
  const long long routed = (long long)P.kind[0].units * P.cost[0];
  if (x <= routed || P.kind[1].units == 0) return (int)min((long long)P.kind[0].units, (x + P.cost[0] - 1) / P.cost[0]);
  return P.kind[0].units + (int)min((long long)P.kind[1].units, (x - routed + P.cost[1] - 1) / P.cost[1]);
}

// Position of a warp in the ring of stages.
struct Ring {
  int slot, round, qbase;
  __device__ __forceinline__ void advance(int stages) { if (++slot == stages) { slot = 0; ++round; } }
};

// ---- gate/up: the units [u0, u1) of one kind (compile-time encoding) -----------------------------------
// A warp takes the items i0, i0 + 8, ... of every stage, two at a time; i0 rotates with the running item
// count so that stages whose item count is no multiple of 8 still load the warps evenly.
template <int ENC>
__device__ __forceinline__ void gateup_units(const DecodeKernelPlan& P, const DecodeKind& K, int u0, int u1, int ub,
                                             uint32_t smem_base, uint64_t* full, uint64_t* empty, float* red, Ring& ring,
                                             volatile int* fail, int warp, int lane, bool skip) {
  const int g = lane >> 2, t = lane & 3;
  const uint32_t lane_a = g * K.mstride + t * 16, a8off = 8 * K.mstride;
  const uint32_t xf = smem_base + K.frag_off + t * 16, gs = smem_base + K.gsum_off;
  constexpr uint32_t kFragItem = ENC == ENC_BF16 ? 64 : 256;        // fragment bytes per item (one slot)
  const uint32_t sc_g = (uint32_t)g * K.groups * 4, sc_g8 = (uint32_t)(8 + g) * K.groups * 4;
  const float nbias = -K.bias;
  for (int u = u0; u < u1; ++u) {
    float acc0 = 0.f, acc8 = 0.f;
    for (int ch = 0; ch < K.nch; ++ch) {
      const int i0 = (warp - ring.qbase) & (kNW - 1);
      if (i0 < K.ips && wait_or_fail(full + ring.slot, ring.round & 1, fail) && !skip) {
        const uint32_t st = smem_base + ring.slot * P.stage_bytes, sc = st + P.scale_off;
        int i = i0;
        for (; i + kNW < K.ips; i += 2 * kNW) {
          const int gi = ch * K.ips + i;
          const uint32_t a0[2] = {st + lane_a + i * 64, st + lane_a + (i + kNW) * 64};
          const uint32_t bp[2] = {xf + gi * kFragItem, xf + (gi + kNW) * kFragItem};
          float in0[2] = {0.f, 0.f}, s0[2], s8[2];
          if (ENC != ENC_BF16) {
            in0[0] = nbias * lds32(gs + gi * 4); in0[1] = nbias * lds32(gs + (gi + kNW) * 4);
            const int grp0 = ENC == ENC_Q4 ? gi : gi >> 1, grp1 = ENC == ENC_Q4 ? gi + kNW : (gi + kNW) >> 1;
            s0[0] = lds32(sc + sc_g + grp0 * 4); s8[0] = lds32(sc + sc_g8 + grp0 * 4);
            s0[1] = lds32(sc + sc_g + grp1 * 4); s8[1] = lds32(sc + sc_g8 + grp1 * 4);
          }
          float c[2][4];
          items_mma<ENC, 2, false>(a0, a8off, bp, 64, in0, in0, c);
          if (ENC != ENC_BF16) {
            acc0 = fmaf(s0[0], c[0][0], acc0); acc8 = fmaf(s8[0], c[0][2], acc8);
            acc0 = fmaf(s0[1], c[1][0], acc0); acc8 = fmaf(s8[1], c[1][2], acc8);
          } else { acc0 += c[0][0] + c[1][0]; acc8 += c[0][2] + c[1][2]; }
        }
        if (i < K.ips) {
          const int gi = ch * K.ips + i;
          const uint32_t a0[1] = {st + lane_a + i * 64};
          const uint32_t bp[1] = {xf + gi * kFragItem};
          float in0[1] = {0.f}, s0 = 0.f, s8 = 0.f;
          if (ENC != ENC_BF16) {
            in0[0] = nbias * lds32(gs + gi * 4);
            const int grp = ENC == ENC_Q4 ? gi : gi >> 1;
            s0 = lds32(sc + sc_g + grp * 4); s8 = lds32(sc + sc_g8 + grp * 4);
          }
          float c[1][4];
          items_mma<ENC, 1, false>(a0, a8off, bp, 64, in0, in0, c);
          if (ENC != ENC_BF16) { acc0 = fmaf(s0, c[0][0], acc0); acc8 = fmaf(s8, c[0][2], acc8); }
          else { acc0 += c[0][0]; acc8 += c[0][2]; }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty + ring.slot);
      ring.qbase = (ring.qbase + K.ips) & (kNW - 1);
      ring.advance(P.stages);
    }
    if (t == 0) {
      float* r = red + ((size_t)(u - ub) * kNW + warp) * 16;
      r[g] = acc0; r[8 + g] = acc8;
    }
  }
}

// =====================================================================================================
// Kernel A: gate/up + SwiGLU.  Work unit = 8 features of one slot: MMA rows 0..7 their gate rows,
// 8..15 their up rows, all of K = hidden, in nch ring stages of 16 rows x ch bytes.
// =====================================================================================================
__global__ void __launch_bounds__(kThreadsD, 2) decode_gateup_kernel(const DecodeParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ int s_expert[kMaxSlots];
  __shared__ int s_fail;
  const DecodeKernelPlan& P = p.g;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + P.bar_off);
  uint64_t* empty = full + P.stages;
  if (tid == 0) {
    for (int s = 0; s < P.stages; ++s) { mbar_init(full + s, 1 + 32); mbar_init(empty + s, kNW); }
    s_fail = 0;
    fence_barrier_init();
  }
  stamp(p, 0, 0);
  pdl_wait();                    // the routes and the activation vector come from the kernels before this one
  stamp(p, 1, 0);
  pdl_launch_dependents();       // the down kernel may become resident and stream its weights from here on
  if (tid < p.top_k) {
    long long e = load_index(p.idx, p.idx64, tid);
    if (e < 0 || e >= p.experts) {          // the reference skips such a route; here its weight becomes 0 in the
      atomicExch(p.sync + 2, (unsigned)ERR_BAD_ARGUMENT);     // down kernel and the status word records it
      e = 0;
    }
    s_expert[tid] = (int)e;
  }
  __syncthreads();

  stamp(p, 2, 0);
  const int H = p.hidden;
  const int U0 = P.kind[0].units, upr = p.inter >> 3;
  const int ub = first_unit(P, blockIdx.x), ue = first_unit(P, blockIdx.x + 1);
  volatile int* fail = &s_fail;

  if (warp == kNW) {
    // ---- producer: rows and scales of every stage, in order ------------------------------------------------
    int slot = 0, round = 0;
    for (int u = ub; u < ue && !*fail; ++u) {
      const int k = u < U0 ? 0 : 1;
      const DecodeKind& K = P.kind[k];
      const uint8_t *gsrc, *usrc;
      const float *gs = nullptr, *us = nullptr;
      if (k == 0) {
        const int sl = u / upr, f0 = (u - sl * upr) << 3;
        const size_t row = (size_t)s_expert[sl] * p.inter + f0;
        gsrc = p.gate + row * K.row_bytes; usrc = p.up + row * K.row_bytes;
        if (K.groups) { gs = p.gate_s + row * K.groups; us = p.up_s + row * K.groups; }
      } else {
        const size_t row = (size_t)(u - U0) << 3;
        gsrc = reinterpret_cast<const uint8_t*>(p.sh_gate) + row * K.row_bytes;
        usrc = reinterpret_cast<const uint8_t*>(p.sh_up) + row * K.row_bytes;
      }
      for (int ch = 0; ch < K.nch; ++ch) {
        if (round > 0 && !wait_or_fail(empty + slot, (round - 1) & 1, fail)) break;
        uint8_t* st = smem + (size_t)slot * P.stage_bytes;
        if (lane == 0) mbar_expect_tx(full + slot, (p.debug & 2) ? 0u : 16u * K.ch);
        __syncwarp();
        if (lane < 16 && !(p.debug & 2))
          bulk_g2s(st + lane * K.mstride, (lane < 8 ? gsrc : usrc) + (size_t)(lane & 7) * K.row_bytes + (size_t)ch * K.ch,
                   K.ch, full + slot);
        if (K.groups) {              // [16 MMA rows][groups] floats: 8 gate rows then 8 up rows, 16-byte pieces
          const int pieces = 2 * K.groups;
          for (int i = lane; i < 2 * pieces; i += 32) {
            const int up_half = i >= pieces, j = i - up_half * pieces;
            cp_async16(st + P.scale_off + (size_t)i * 16, (up_half ? us : gs) + j * 4);
          }
        }
        cp_async_arrive(full + slot);
        if (++slot == P.stages) { slot = 0; ++round; }
      }
    }
    stamp(p, 8, kNW * 32);
  } else {
    // ---- consumers ---------------------------------------------------------------------------------------------
    build_x_fragments(P.kind[0].enc, p.x, H, smem + P.kind[0].frag_off, reinterpret_cast<float*>(smem + P.kind[0].gsum_off), tid);
    if (P.kind[1].units && P.kind[1].frag_off != P.kind[0].frag_off)
      build_x_fragments(ENC_BF16, p.x, H, smem + P.kind[1].frag_off, nullptr, tid);
    named_bar_sync(1, kConsumers);
    stamp(p, 3, 0);
    if (warp == 0) { wait_or_fail(full, 0, fail); stamp(p, 4, 0); }
    float* red = reinterpret_cast<float*>(smem + P.red_off);
    const uint32_t smem_base = smem_u32(smem);
    Ring ring{0, 0, 0};
    const int um = min(max(ub, U0), ue);        // routed units [ub, um), shared-expert units [um, ue)
    if (ub < um) {
      if (P.kind[0].enc == ENC_Q4) gateup_units<ENC_Q4>(P, P.kind[0], ub, um, ub, smem_base, full, empty, red, ring, fail, warp, lane, (p.debug & 1) != 0);
      else if (P.kind[0].enc == ENC_Q8) gateup_units<ENC_Q8>(P, P.kind[0], ub, um, ub, smem_base, full, empty, red, ring, fail, warp, lane, (p.debug & 1) != 0);
      else gateup_units<ENC_BF16>(P, P.kind[0], ub, um, ub, smem_base, full, empty, red, ring, fail, warp, lane, (p.debug & 1) != 0);
    }
    if (um < ue) gateup_units<ENC_BF16>(P, P.kind[1], um, ue, ub, smem_base, full, empty, red, ring, fail, warp, lane, (p.debug & 1) != 0);
    stamp(p, 5, 0);
  }
  __syncthreads();
  stamp(p, 6, 0);
  if (s_fail) {
    if (tid == 0) atomicExch(p.sync + 2, (unsigned)ERR_DEVICE_TIMEOUT);
    __nanosleep(100000);           // copies still in flight land before the shared memory is given back
    return;
  }

  // ---- SwiGLU; every value goes where the down kernel's fragments expect it ----------------------------------
  if (tid < (ue - ub) * 8) {
    const int ul = tid >> 3, f = tid & 7, u = ub + ul;
    const float* r = reinterpret_cast<const float*>(smem + P.red_off) + (size_t)ul * kNW * 16;
    float gv = 0.f, uv = 0.f;
#pragma unroll
    for (int w = 0; w < kNW; ++w) { gv += r[w * 16 + f]; uv += r[w * 16 + 8 + f]; }
    if (u < U0) {
      const int sl = u / upr, k = ((u - sl * upr) << 3) + f;
      const DecodeKind& D = p.d.kind[0];
      const float v = silu_f32(gv) * uv;
      uint8_t* dst = p.inter_buf + D.ws_off;
      *reinterpret_cast<__nv_bfloat16*>(dst + frag_offset(D.enc, D.ng, sl, k, 0)) = __float2bfloat16_rn(v);
      if (D.enc == ENC_Q8)
        *reinterpret_cast<__nv_bfloat16*>(dst + frag_offset(D.enc, D.ng, sl, k, 1)) =
            __float2bfloat16_rn(bf16_round(v) * 16.f);
    } else {
      // Qwen2MoeMLP in BF16: every linear / activation output is rounded
      const DecodeKind& D = p.d.kind[1];
      gv = bf16_round(gv); uv = bf16_round(uv);
      const float v = bf16_round(bf16_round(silu_f32(gv)) * uv);
      const int k = ((u - U0) << 3) + f, kseg = p.shared_inter / D.nvs, seg = k / kseg;
      *reinterpret_cast<__nv_bfloat16*>(p.inter_buf + D.ws_off + frag_offset(ENC_BF16, D.ng, seg, k - seg * kseg, 0)) =
          __float2bfloat16_rn(v);
    }
  }
  stamp(p, 7, 0);
}

// ---- down: the stages of one kind (compile-time encoding), two row pairs at a time --------------------
// The two stages of a round hold the same columns of different output rows, so they share the fragments
// and the start values; a warp takes the items i0, i0 + 8, ... of both.
template <int ENC>
__device__ __forceinline__ void down_stages(const DecodeKernelPlan& P, const DecodeKind& K, int npairs, uint32_t smem_base,
                                            uint64_t* full, uint64_t* empty, float* red, Ring& ring, volatile int* fail,
                                            int warp, int lane, bool skip) {
  const int g = lane >> 2, t = lane & 3;
  const int ga = g < K.nvs ? g : 0, gb = g & (K.ng - 1), c0 = (2 * t) & (K.ng - 1);
  const uint32_t lane_a = ga * K.mstride + t * 16, a8off = K.row_bytes;
  constexpr uint32_t kChunks = ENC == ENC_BF16 ? 1 : 4;
  const uint32_t frag_item = kChunks * K.ng * 64, bstep = K.ng * 64;
  const uint32_t fr = smem_base + K.frag_off + (gb * 4 + t) * 16;
  const uint32_t gs = smem_base + K.gsum_off + c0 * 4;
  const uint32_t sc_lane = P.scale_off + (uint32_t)ga * 2 * K.groups * 4;
  const bool odd = g & 1, diag = t == (g >> 1);
  const float nbias = -K.bias;
  for (int ul = 0; ul < npairs; ul += 2) {
    const bool two = ul + 1 < npairs;
    const int slot_a = ring.slot, round_a = ring.round;
    ring.advance(P.stages);
    const int slot_b = two ? ring.slot : slot_a, round_b = two ? ring.round : round_a;
    if (two) ring.advance(P.stages);
    float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    const int i0 = (warp - ring.qbase) & (kNW - 1);
    if (i0 < K.ips && wait_or_fail(full + slot_a, round_a & 1, fail) && wait_or_fail(full + slot_b, round_b & 1, fail) && !skip) {
      const uint32_t st_a = smem_base + slot_a * P.stage_bytes, st_b = smem_base + slot_b * P.stage_bytes;
      for (int i = i0; i < K.ips; i += kNW) {
        const uint32_t a0[2] = {st_a + lane_a + i * 64, st_b + lane_a + i * 64};
        const uint32_t bp[2] = {fr + i * frag_item, fr + i * frag_item};
        float in0[2] = {0.f, 0.f}, in1[2] = {0.f, 0.f}, s[2][2];
        if (ENC != ENC_BF16) {
          const float2 sums = lds64(gs + i * K.ng * 4);
          in0[0] = in0[1] = nbias * sums.x; in1[0] = in1[1] = nbias * sums.y;
          const int grp = ENC == ENC_Q4 ? i : i >> 1;
          s[0][0] = lds32(st_a + sc_lane + grp * 4); s[0][1] = lds32(st_a + sc_lane + (K.groups + grp) * 4);
          s[1][0] = lds32(st_b + sc_lane + grp * 4); s[1][1] = lds32(st_b + sc_lane + (K.groups + grp) * 4);
        }
        float c[2][4];
        items_mma<ENC, 2, true>(a0, a8off, bp, bstep, in0, in1, c);
#pragma unroll
        for (int n = 0; n < 2; ++n) {
          const float v0 = odd ? c[n][1] : c[n][0], v8 = odd ? c[n][3] : c[n][2];     // column g of rows g, g + 8
          if (ENC != ENC_BF16) { acc[n][0] = fmaf(s[n][0], v0, acc[n][0]); acc[n][1] = fmaf(s[n][1], v8, acc[n][1]); }
          else { acc[n][0] += v0; acc[n][1] += v8; }
        }
      }
    }
    __syncwarp();
    if (lane == 0) { mbar_arrive(empty + slot_a); if (two) mbar_arrive(empty + slot_b); }
    ring.qbase = (ring.qbase + K.ips) & (kNW - 1);
    if (diag) {                      // the lane that holds column g
      float* r = red + ((size_t)ul * kNW + warp) * 16;
      r[2 * g] = acc[0][0]; r[2 * g + 1] = acc[0][1];
      if (two) { r[kNW * 16 + 2 * g] = acc[1][0]; r[kNW * 16 + 2 * g + 1] = acc[1][1]; }
    }
  }
}

// =====================================================================================================
// Kernel B: down + ordered combine.  Work unit = a pair of output rows (n, n+1): one ring stage holds,
// per routed slot, those two rows of the slot's expert (MMA rows g and g + 8 for slot g); with a shared
// expert a second series of stages holds the two rows cut into K segments.
// =====================================================================================================
__global__ void __launch_bounds__(kThreadsD, 2) decode_down_kernel(const DecodeParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ int s_expert[kMaxSlots], s_order[kMaxSlots];
  __shared__ float s_weight[kMaxSlots];
  __shared__ float s_tmp[kNW];
  __shared__ float s_gate;
  __shared__ int s_fail, s_present;
  const DecodeKernelPlan& P = p.d;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int H = p.hidden, S = P.kind[1].nvs ? p.shared_inter : 0;
  const int kinds = S ? 2 : 1;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + P.bar_off);
  uint64_t* empty = full + P.stages;
  uint64_t* inter_bar = empty + P.stages;
  if (tid == 0) {
    for (int s = 0; s < P.stages; ++s) { mbar_init(full + s, 1 + 32); mbar_init(empty + s, kNW); }
    mbar_init(inter_bar, 1);
    s_fail = 0;
    fence_barrier_init();
  }
  // Every gate/up CTA has passed its own dependency wait before this kernel could start, so the routes and
  // the activation vector are final; only the intermediate must be waited for.
  stamp(p, 16, 0);
  pdl_launch_dependents();
  if (tid < kMaxSlots) {
    long long e = -1;
    float w = 0.f;
    if (tid < p.top_k) { e = load_index(p.idx, p.idx64, tid); w = p.w[tid]; }
    const bool ok = e >= 0 && e < p.experts;
    s_expert[tid] = ok ? (int)e : 0;            // invalid routes read expert 0's rows and contribute nothing
    s_weight[tid] = ok ? w : 0.f;
    const unsigned present = __ballot_sync(0xffu, ok);
    // rank among the valid routes by (expert, slot): the accumulation order of the reference's CPU path
    int rank = 0;
    for (int j = 0; j < p.top_k; ++j) {
      const long long ej = load_index(p.idx, p.idx64, j);
      rank += ((present >> j) & 1u) && (ej < e || (ej == e && j < tid));
    }
    if (ok) s_order[rank] = tid;
    if (tid == 0) s_present = __popc(present);
  }
  __syncthreads();

  const int pairs = H >> 1;
  const int rp0 = (int)((long long)blockIdx.x * pairs / gridDim.x), rp1 = (int)((long long)(blockIdx.x + 1) * pairs / gridDim.x);
  const int npairs = rp1 - rp0;
  volatile int* fail = &s_fail;
  stamp(p, 17, 0);

  if (warp == kNW) {
    // ---- producer: the routed stages of every row pair, then the shared expert's ----------------------------
    if (p.down_delay_ns > 0) {                 // lets the gate/up kernel's own loads go first
      const uint64_t t0 = global_ns();
      while (global_ns() - t0 < (uint64_t)p.down_delay_ns) __nanosleep(200);
    }
    int slot = 0, round = 0;
    for (int k = 0; k < kinds && !*fail; ++k) {
      const DecodeKind& K = P.kind[k];
      for (int rp = rp0; rp < rp1; ++rp) {
        if (round > 0 && !wait_or_fail(empty + slot, (round - 1) & 1, fail)) break;
        uint8_t* st = smem + (size_t)slot * P.stage_bytes;
        if (lane == 0) mbar_expect_tx(full + slot, (p.debug & 2) ? 0u : (uint32_t)(K.nvs * 2 * K.row_bytes));
        __syncwarp();
        if (k == 0) {
          if (lane < K.nvs && !(p.debug & 2))          // rows n and n+1 of the slot's expert are adjacent: one copy
            bulk_g2s(st + lane * K.mstride, p.down + ((size_t)s_expert[lane] * H + 2 * rp) * K.row_bytes,
                     2u * K.row_bytes, full + slot);
          if (K.groups) {            // [slot][2 rows][groups] floats in 8-byte pieces
            for (int i = lane; i < K.nvs * K.groups; i += 32) {
              const int vs = i / K.groups, j = i - vs * K.groups;
              cp_async8(st + P.scale_off + (size_t)i * 8,
                        p.down_s + ((size_t)s_expert[vs] * H + 2 * rp) * K.groups + 2 * j);
            }
          }
        } else if (lane < 2 * K.nvs && !(p.debug & 2)) {   // segment `seg` of rows n, n+1 of the shared expert's down matrix
          const int seg = lane >> 1, row = lane & 1;
          bulk_g2s(st + seg * K.mstride + row * K.row_bytes,
                   reinterpret_cast<const uint8_t*>(p.sh_down) + ((size_t)(2 * rp + row) * K.nvs + seg) * K.row_bytes,
                   (uint32_t)K.row_bytes, full + slot);
        }
        cp_async_arrive(full + slot);
        if (++slot == P.stages) { slot = 0; ++round; }
      }
    }
    stamp(p, 25, kNW * 32);
  } else {
    // ---- consumers ---------------------------------------------------------------------------------------------
    if (S) {                       // sigmoid gate of the shared expert: bf16(sigmoid(bf16(x . wg)))
      float acc = 0.f;
      for (int k = tid * 2; k < H; k += kConsumers * 2) {
        const __nv_bfloat162 xv = *reinterpret_cast<const __nv_bfloat162*>(p.x + k);
        const __nv_bfloat162 gv = *reinterpret_cast<const __nv_bfloat162*>(p.sh_gatevec + k);
        acc += __low2float(xv) * __low2float(gv) + __high2float(xv) * __high2float(gv);
      }
#pragma unroll
      for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (lane == 0) s_tmp[warp] = acc;
      named_bar_sync(1, kConsumers);
      if (tid == 0) {
        float sum = 0.f;
        for (int i = 0; i < kNW; ++i) sum += s_tmp[i];
        sum = bf16_round(sum);
        s_gate = bf16_round(1.f / (1.f + expf(-sum)));
      }
    }
    stamp(p, 18, 0);
    pdl_wait();                    // the gate/up kernel's intermediate is complete and visible from here on
    stamp(p, 19, 0);
    if (tid == 0) {
      mbar_expect_tx(inter_bar, (uint32_t)(P.kind[0].frag_bytes + (S ? P.kind[1].frag_bytes : 0)));
      bulk_g2s(smem + P.kind[0].frag_off, p.inter_buf + P.kind[0].ws_off, (uint32_t)P.kind[0].frag_bytes, inter_bar);
      if (S) bulk_g2s(smem + P.kind[1].frag_off, p.inter_buf + P.kind[1].ws_off, (uint32_t)P.kind[1].frag_bytes, inter_bar);
    }
    const bool have_inter = wait_or_fail(inter_bar, 0, fail);
    stamp(p, 20, 0);
    // activation sums per (item, slot) of the quantised rows: the bias every accumulator starts from
    if (have_inter && P.kind[0].groups) {
      const DecodeKind& K = P.kind[0];
      float* gsum = reinterpret_cast<float*>(smem + K.gsum_off);
      const int total = K.ips * K.ng * 4;
      for (int base = 0; base < total; base += kConsumers) {
        const int idx = base + tid;
        float sum = 0.f;
        if (idx < total) {
          const int tt = idx & 3, vs = (idx >> 2) & (K.ng - 1), item = idx / (4 * K.ng);
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const uint4 v = *reinterpret_cast<const uint4*>(smem + K.frag_off + ((((item * 4 + r) * K.ng + vs) * 4 + tt) << 4));
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int q = 0; q < 4; ++q)       // Q8 fragments hold x in words 0 and 2 and 16 x in words 1 and 3
              if (K.enc == ENC_Q4 || !(q & 1)) sum += __uint_as_float(w[q] << 16) + __uint_as_float(w[q] & 0xffff0000u);
          }
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if (idx < total && (idx & 3) == 0) gsum[idx >> 2] = sum;
      }
    }
    named_bar_sync(1, kConsumers);
    stamp(p, 21, 0);

    const uint32_t smem_base = smem_u32(smem);
    Ring ring{0, 0, 0};
    float* red = reinterpret_cast<float*>(smem + P.red_off);
    if (P.kind[0].enc == ENC_Q4) down_stages<ENC_Q4>(P, P.kind[0], npairs, smem_base, full, empty, red, ring, fail, warp, lane, (p.debug & 1) != 0);
    else if (P.kind[0].enc == ENC_Q8) down_stages<ENC_Q8>(P, P.kind[0], npairs, smem_base, full, empty, red, ring, fail, warp, lane, (p.debug & 1) != 0);
    else down_stages<ENC_BF16>(P, P.kind[0], npairs, smem_base, full, empty, red, ring, fail, warp, lane, (p.debug & 1) != 0);
    if (S) down_stages<ENC_BF16>(P, P.kind[1], npairs, smem_base, full, empty, reinterpret_cast<float*>(smem + P.red2_off), ring, fail, warp, lane, (p.debug & 1) != 0);
    stamp(p, 22, 0);
  }
  __syncthreads();
  stamp(p, 23, 0);
  if (s_fail) {
    if (tid == 0) atomicExch(p.sync + 2, (unsigned)ERR_DEVICE_TIMEOUT);
    __nanosleep(100000);
    return;
  }

  // ---- sums over the warps, then the ordered combine: ascending expert, BF16 rounding of every
  //      contribution and partial sum ----------------------------------------------------------------------------
  float* ysum = reinterpret_cast<float*>(smem + P.ysum_off);
  for (int idx = tid; idx < npairs * kinds * 16; idx += kThreadsD) {
    const int e = idx & 15, k = (idx >> 4) % kinds, ul = idx / (16 * kinds);
    const float* r = reinterpret_cast<const float*>(smem + (k ? P.red2_off : P.red_off)) + (size_t)ul * kNW * 16 + e;
    float y = 0.f;
#pragma unroll
    for (int w = 0; w < kNW; ++w) y += r[w * 16];
    ysum[(ul * 2 + k) * 16 + e] = y;
  }
  __syncthreads();
  if (tid < npairs * 2) {
    const int ul = tid >> 1, row = tid & 1;
    const float* y = ysum + (size_t)ul * 32;
    float run = 0.f;
    for (int r = 0; r < s_present; ++r) {
      const int slot = s_order[r];
      run = bf16_round(run + bf16_round(y[2 * slot + row] * s_weight[slot]));
    }
    if (S) {
      float ys = 0.f;
      for (int seg = 0; seg < P.kind[1].nvs; ++seg) ys += y[16 + 2 * seg + row];
      run = bf16_round(run + bf16_round(s_gate * bf16_round(ys)));
    }
    p.out[2 * (rp0 + ul) + row] = __float2bfloat16_rn(run);
  }
  stamp(p, 24, 0);
}

// ---- host: plans -------------------------------------------------------------------------------------------
int pow2_at_least(int v) { int n = 1; while (n < v) n <<= 1; return n; }
int align_up(int v, int a) { return (v + a - 1) / a * a; }

void describe_kind(DecodeKind& K, int enc, int k) {
  K.enc = enc;
  K.row_bytes = row_bytes(enc, k);
  K.item_bytes = 64;
  K.r16 = enc == ENC_BF16 ? 1 : 4;
  K.groups = enc == ENC_BF16 ? 0 : k / 128;
  K.bias = enc == ENC_Q4 ? 136.f : (enc == ENC_Q8 ? 2304.f : 0.f);
}

bool plan_gateup(DecodeParams& p, int sms, int budget) {
  DecodeKernelPlan& P = p.g;
  P = DecodeKernelPlan{};
  const int H = p.hidden;
  const int S = p.sh_gate ? p.shared_inter : 0;
  int cursor = 0;
  for (int k = 0; k < 2; ++k) {
    DecodeKind& K = P.kind[k];
    if (k == 1 && !S) break;
    describe_kind(K, k ? ENC_BF16 : p.enc, H);
    K.units = k ? S / 8 : p.top_k * (p.inter / 8);
    // the largest part of a row that is a whole number of items, divides the row and stays <= 1 KB
    K.ch = 0;
    for (int c = std::min(K.row_bytes, 1024) / K.item_bytes * K.item_bytes; c >= K.item_bytes; c -= K.item_bytes)
      if (K.row_bytes % c == 0) { K.ch = c; break; }
    if (!K.ch) return false;
    K.nch = K.row_bytes / K.ch;
    K.ips = K.ch / K.item_bytes;
    K.mstride = K.ch + 64;
    P.cost[k] = K.row_bytes;
  }
  P.total_cost = (long long)P.kind[0].units * P.cost[0] + (long long)P.kind[1].units * P.cost[1];
  P.grid = std::min(sms, P.kind[0].units + P.kind[1].units);
  // fragments: one buffer per encoding
  for (int k = 0; k < 2; ++k) {
    DecodeKind& K = P.kind[k];
    if (k == 1 && !S) break;
    if (k == 1 && P.kind[0].enc == ENC_BF16) { K.frag_off = P.kind[0].frag_off; K.gsum_off = P.kind[0].gsum_off; K.frag_bytes = P.kind[0].frag_bytes; continue; }
    K.frag_bytes = K.enc == ENC_Q8 ? H * 4 : H * 2;        // items x chunks x 4 lanes x 16 bytes
    K.frag_off = cursor; cursor += align_up(K.frag_bytes, 128);
    K.gsum_off = cursor; cursor += align_up((H / 64) * 4, 128);
  }
  int max_units = 0, max_stages = 0;
  for (int c = 0; c < P.grid; ++c) {
    const int ub = first_unit(P, c), ue = first_unit(P, c + 1);
    max_units = std::max(max_units, ue - ub);
    int st = 0;
    for (int u = ub; u < ue; ++u) st += P.kind[u < P.kind[0].units ? 0 : 1].nch;
    max_stages = std::max(max_stages, st);
  }
  P.max_units = max_units;
  P.red_off = cursor; cursor += align_up(max_units * kNW * 16 * 4, 128);
  const int fixed = cursor;
  const int mmax = std::max(P.kind[0].mstride, P.kind[1].mstride);
  P.scale_off = 16 * mmax;
  P.stage_bytes = align_up(P.scale_off + 16 * P.kind[0].groups * 4, 128);
  const int room = budget - fixed - 256;
  P.stages = std::min(max_stages, room / (P.stage_bytes + 16));
  if (P.stages < 2 && max_stages >= 2) return false;
  if (P.stages < 1) return false;
  // stages first (128-byte aligned), then the fixed part, then the barriers
  const int stage_total = P.stages * P.stage_bytes;
  for (int k = 0; k < 2; ++k) { P.kind[k].frag_off += stage_total; P.kind[k].gsum_off += stage_total; }
  P.red_off += stage_total;
  P.bar_off = stage_total + fixed;
  P.smem_bytes = P.bar_off + 2 * P.stages * 8 + 16;
  return P.smem_bytes <= budget;
}

bool plan_down(DecodeParams& p, int sms) {
  DecodeKernelPlan& P = p.d;
  P = DecodeKernelPlan{};
  const int H = p.hidden, I = p.inter;
  const int S = p.sh_gate ? p.shared_inter : 0;
  int cursor = 0, ws = 0;
  {
    DecodeKind& K = P.kind[0];
    describe_kind(K, p.enc, I);
    K.nvs = p.top_k;
    K.ng = pow2_at_least(std::max(2, p.top_k));
    if (K.row_bytes > 4096) return false;
    K.ips = K.row_bytes / K.item_bytes;
    K.mstride = 2 * K.row_bytes + 64;
    K.frag_bytes = K.ips * K.r16 * K.ng * 64;
    K.ws_off = ws; ws += align_up(K.frag_bytes, 256);
    K.frag_off = cursor; cursor += align_up(K.frag_bytes, 128);
    K.gsum_off = cursor; cursor += align_up(K.ips * K.ng * 4, 128);
  }
  if (S) {
    DecodeKind& K = P.kind[1];
    int nseg = 0;
    for (int n = 8; n >= 1; n >>= 1)
      if (S % (n * 32) == 0 && 2 * (S / n) <= 4096) { nseg = n; break; }
    if (!nseg) return false;
    describe_kind(K, ENC_BF16, S / nseg);
    K.nvs = nseg; K.ng = nseg;
    K.ips = K.row_bytes / K.item_bytes;
    K.mstride = 2 * K.row_bytes + 64;
    K.frag_bytes = K.ips * K.r16 * K.ng * 64;
    K.ws_off = ws; ws += align_up(K.frag_bytes, 256);
    K.frag_off = cursor; cursor += align_up(K.frag_bytes, 128);
    K.gsum_off = cursor;
  }
  const int pairs = H / 2;
  P.grid = std::min(sms, pairs);
  P.max_units = (pairs + P.grid - 1) / P.grid;
  P.red_off = cursor; cursor += align_up(P.max_units * kNW * 16 * 4, 128);
  P.red2_off = cursor; if (S) cursor += align_up(P.max_units * kNW * 16 * 4, 128);
  P.ysum_off = cursor; cursor += align_up(P.max_units * 32 * 4, 128);
  const int fixed = cursor;
  const int body = std::max(P.kind[0].nvs * P.kind[0].mstride, P.kind[1].nvs * P.kind[1].mstride);
  P.scale_off = align_up(body, 16);
  P.stage_bytes = align_up(P.scale_off + P.kind[0].nvs * 2 * P.kind[0].groups * 4, 128);
  const int want = P.max_units * (S ? 2 : 1);
  const int room = kDownSmemMax - fixed - 256;
  P.stages = std::min(want, room / (P.stage_bytes + 16));
  if (P.stages < 1 || (P.stages < 2 && want >= 2)) return false;
  const int stage_total = P.stages * P.stage_bytes;
  for (int k = 0; k < 2; ++k) { P.kind[k].frag_off += stage_total; P.kind[k].gsum_off += stage_total; }
  P.red_off += stage_total; P.red2_off += stage_total; P.ysum_off += stage_total;
  P.bar_off = stage_total + fixed;
  P.smem_bytes = P.bar_off + (2 * P.stages + 1) * 8 + 16;
  return P.smem_bytes <= kDownSmemMax;
}

bool plan_both(DecodeParams& p, int sms) {
  if (!plan_down(p, sms)) return false;
  return plan_gateup(p, sms, kPairSmemBudget - align_up(p.d.smem_bytes, 1024));
}

int down_delay_from_env() {
  static const int value = [] {
    const char* s = std::getenv("UMAQ_DECODE_DOWN_DELAY_NS");
    return s ? std::max(0, std::atoi(s)) : 0;
  }();
  return value;
}

int debug_from_env() {
  static const int value = [] {
    const char* s = std::getenv("UMAQ_DECODE_DEBUG");
    return s ? std::atoi(s) : 0;
  }();
  return value;
}

}  // namespace

size_t decode_workspace_bytes(int top_k, int inter, int shared_inter) {
  // four bytes per intermediate value cover every encoding's fragments (Q8 keeps x and 16 x); the slot
  // dimension of the routed fragments is top_k rounded up to a power of two
  const size_t slots = (size_t)pow2_at_least(std::max(2, top_k));
  return kDecodeWsHeader + (slots * (size_t)std::max(inter, 0) + (size_t)std::max(shared_inter, 0)) * sizeof(float) + 512;
}

int launch_moe_decode(DecodeParams p, cudaStream_t stream) {
  const int S = p.sh_gate ? p.shared_inter : 0;
  if (p.top_k < 1 || p.top_k > kMaxSlots || p.hidden % 256 || p.inter % 128 || p.hidden < 256 || p.inter < 128 ||
      p.hidden > 8192 || p.inter > 8192 || (S && (S % 64 || S < 64 || S > 32768)) || p.enc < 0 || p.enc > 2) {
    set_error("decode: unsupported shape (hidden %d, intermediate %d, top_k %d, shared %d, encoding %d)", p.hidden,
              p.inter, p.top_k, p.shared_inter, p.enc);
    return ERR_BAD_ARGUMENT;
  }
  if (p.enc != ENC_BF16 && (!p.gate_s || !p.up_s || !p.down_s)) {
    set_error("decode: quantised layer without scales");
    return ERR_BAD_ARGUMENT;
  }
  const uintptr_t all = reinterpret_cast<uintptr_t>(p.gate) | reinterpret_cast<uintptr_t>(p.up) |
                        reinterpret_cast<uintptr_t>(p.down) | reinterpret_cast<uintptr_t>(p.gate_s) |
                        reinterpret_cast<uintptr_t>(p.up_s) | reinterpret_cast<uintptr_t>(p.down_s) |
                        reinterpret_cast<uintptr_t>(p.x) | reinterpret_cast<uintptr_t>(p.sh_gate) |
                        reinterpret_cast<uintptr_t>(p.sh_up) | reinterpret_cast<uintptr_t>(p.sh_down) |
                        reinterpret_cast<uintptr_t>(p.inter_buf);
  if (all & 15) {
    set_error("decode: weight, scale, activation and workspace pointers must be 16-byte aligned");
    return ERR_BAD_ARGUMENT;
  }
  const int sms = sm_count();
  if (sms <= 0) { set_error("decode: no CUDA device"); return ERR_LAUNCH; }
  if (!plan_both(p, sms)) {
    set_error("decode: shape needs more shared memory than an SM has (hidden %d, intermediate %d, top_k %d, shared %d, "
              "encoding %d)", p.hidden, p.inter, p.top_k, p.shared_inter, p.enc);
    return ERR_UNSUPPORTED;
  }
  p.down_delay_ns = down_delay_from_env();
  p.debug = debug_from_env();
  static thread_local int configured_device = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_device != dev) {
    cudaError_t e = cudaFuncSetAttribute(decode_gateup_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBudget);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(decode_down_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDownSmemMax);
    // both kernels live on an SM at the same time: ask for the largest shared-memory carve-out
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(decode_gateup_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(decode_down_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    if (e != cudaSuccess) { set_error("decode: cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return ERR_LAUNCH; }
    configured_device = dev;
  }
  // Both kernels are chained to their predecessor by programmatic stream serialisation: their CTAs may
  // become resident while the kernel before them drains, and wait on the device before they read what
  // it wrote.
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg{};
  cfg.blockDim = dim3(kThreadsD);
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cfg.gridDim = dim3(p.g.grid);
  cfg.dynamicSmemBytes = p.g.smem_bytes;
  cudaError_t e = cudaLaunchKernelEx(&cfg, decode_gateup_kernel, p);
  if (e != cudaSuccess) { set_error("decode: gate/up launch failed: %s", cudaGetErrorString(e)); return ERR_LAUNCH; }
  cfg.gridDim = dim3(p.d.grid);
  cfg.dynamicSmemBytes = p.d.smem_bytes;
  e = cudaLaunchKernelEx(&cfg, decode_down_kernel, p);
  if (e != cudaSuccess) { set_error("decode: down launch failed: %s", cudaGetErrorString(e)); return ERR_LAUNCH; }
  return ERR_NONE;
}

}  // namespace umaq

// Launch geometry of the two decode kernels for a shape, without launching anything (host arithmetic only).
extern "C" int umaq_decode_plan(int encoding, int hidden, int intermediate, int top_k, int shared_intermediate, int sms,
                                int* out, int out_len) {
  using namespace umaq;
  if (!out || out_len < 12 || sms < 1) { set_error("umaq_decode_plan: bad argument"); return ERR_BAD_ARGUMENT; }
  DecodeParams p{};
  p.enc = encoding; p.hidden = hidden; p.inter = intermediate; p.top_k = top_k;
  p.shared_inter = shared_intermediate;
  p.sh_gate = shared_intermediate ? reinterpret_cast<const __nv_bfloat16*>(uintptr_t(16)) : nullptr;   // presence flag only
  if (top_k < 1 || top_k > kMaxSlots || hidden % 256 || intermediate % 128 || hidden < 256 || intermediate < 128 ||
      encoding < 0 || encoding > 2 || (shared_intermediate && shared_intermediate % 64)) {
    set_error("umaq_decode_plan: unsupported shape");
    return ERR_BAD_ARGUMENT;
  }
  if (!plan_both(p, sms)) { set_error("umaq_decode_plan: shape does not fit an SM"); return ERR_UNSUPPORTED; }
  const int v[12] = {p.g.grid, p.g.stages, p.g.stage_bytes, p.g.smem_bytes, p.g.max_units, p.g.kind[0].ips,
                     p.d.grid, p.d.stages, p.d.stage_bytes, p.d.smem_bytes, p.d.max_units, p.d.kind[0].ips};
  for (int i = 0; i < 12; ++i) out[i] = v[i];
  return ERR_NONE;
}

// ---- decode without a caller-provided workspace ---------------------------------------------------
// Scratch of the entry point below: one fixed block per device that loads this library, held until
// the process exits.  It has the layout of the decode workspace (control words, then the intermediate
// fragments) and therefore bounds the shapes the entry point accepts.
namespace {
constexpr size_t kStaticScratchBytes = 64 * 1024;
}
static __device__ __align__(256) unsigned char g_decode_static_scratch[kStaticScratchBytes];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_scratch_mutex;
void* g_scratch_ptr[kMaxDevices] = {};

// Device address of the scratch block on the current device.  The name of a __device__ array is only
// a host-side stand-in for the symbol; the address a kernel can use has to be asked for, once per
// device, with that device current.
int static_scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    umaq::set_error("umaq_moe_decode_static: cannot identify the current device (%s)", cudaGetErrorString(e));
    return umaq::ERR_LAUNCH;
  }
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_ptr[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_decode_static_scratch);
    if (e != cudaSuccess || !ptr) {
      umaq::set_error("umaq_moe_decode_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return umaq::ERR_LAUNCH;
    }
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return umaq::ERR_NONE;
}
}  // namespace

extern "C" int umaq_moe_decode_static(const umaq_layer* layer, const umaq_shared_expert* shared, const void* hidden_bf16,
                                      const void* expert_indices, int indices_are_int64, const float* routing_weights,
                                      int top_k, void* out_bf16, void* stream) {
  using namespace umaq;
  if (!layer || !hidden_bf16 || !expert_indices || !routing_weights || !out_bf16) {
    set_error("umaq_moe_decode_static: null argument");
    return ERR_BAD_ARGUMENT;
  }
  const int s_inter = shared ? shared->intermediate : 0;
  if (top_k < 1 || top_k > 8 || layer->intermediate < 1 || s_inter < 0) {
    set_error("umaq_moe_decode_static: unsupported shape");
    return ERR_BAD_ARGUMENT;
  }
  const size_t need = decode_workspace_bytes(top_k, layer->intermediate, s_inter);
  if (need > kStaticScratchBytes) {
    set_error("umaq_moe_decode_static: top_k (rounded up to a power of two) * intermediate + shared intermediate = "
              "%lld float32 values need %zu bytes of scratch, the built-in block holds %zu; use umaq_moe_decode with a "
              "caller workspace",
              (long long)pow2_at_least(std::max(2, top_k)) * layer->intermediate + s_inter, need, kStaticScratchBytes);
    return ERR_WORKSPACE;
  }
  void* scratch = nullptr;
  const int rc = static_scratch_for_current_device(&scratch);
  if (rc != ERR_NONE) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The block keeps whatever the previous call left.  The control words (status) must start from
  // zero; the intermediate area is fully rewritten before it is read.
  cudaError_t e = cudaMemsetAsync(scratch, 0, 64, st);
  if (e != cudaSuccess) { set_error("umaq_moe_decode_static: cudaMemsetAsync: %s", cudaGetErrorString(e)); return ERR_LAUNCH; }
  DecodeParams p{};
  p.gate = static_cast<const uint8_t*>(layer->gate);
  p.up = static_cast<const uint8_t*>(layer->up);
  p.down = static_cast<const uint8_t*>(layer->down);
  p.gate_s = layer->gate_scales; p.up_s = layer->up_scales; p.down_s = layer->down_scales;
  p.enc = layer->encoding; p.experts = layer->num_experts; p.hidden = layer->hidden; p.inter = layer->intermediate;
  p.top_k = top_k;
  p.x = static_cast<const __nv_bfloat16*>(hidden_bf16);
  p.idx = expert_indices; p.idx64 = indices_are_int64; p.w = routing_weights;
  if (shared) {
    p.sh_gate = static_cast<const __nv_bfloat16*>(shared->gate);
    p.sh_up = static_cast<const __nv_bfloat16*>(shared->up);
    p.sh_down = static_cast<const __nv_bfloat16*>(shared->down);
    p.sh_gatevec = static_cast<const __nv_bfloat16*>(shared->gate_vec);
    p.shared_inter = shared->intermediate;
    if (!p.sh_gate || !p.sh_up || !p.sh_down || !p.sh_gatevec) {
      set_error("umaq_moe_decode_static: shared expert with a null tensor");
      return ERR_BAD_ARGUMENT;
    }
  }
  p.out = static_cast<__nv_bfloat16*>(out_bf16);
  uint8_t* ws = static_cast<uint8_t*>(scratch);
  p.sync = reinterpret_cast<unsigned*>(ws);
  p.inter_buf = ws + kDecodeWsHeader;
  return launch_moe_decode(p, st);
}
