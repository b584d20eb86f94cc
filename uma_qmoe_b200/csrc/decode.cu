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
// once: a pure HBM stream of a few microseconds.  What limits such a call is not bandwidth but the
// chain of dependent latencies around it (routes -> weight addresses -> first bytes; intermediate ->
// second projection; kernel boundaries), so everything is organised to keep that chain short and the
// stream busy beside it.
//
//  * One CTA per SM per kernel.  A producer warp brings the CTA's weight rows and their group scales
//    into shared memory with a handful of large cp.async.bulk copies (8 KB blocks of 8 rows; the TMA
//    unit takes about a microsecond per ten requests, so many small copies starve the math), one
//    mbarrier per stage; with the OLMoE shape a CTA's whole share (~120 KB gate/up, ~60 KB down) is in
//    flight at once.  Eight consumer warps split K: each takes 64-byte columns ("items") of the 16 MMA
//    rows of a stage, two items at a time, so no warp waits for another until the partial sums meet.
//  * Both kernels carry the programmatic-stream-serialisation attribute.  The gate/up kernel waits
//    for its predecessor (the routes come from it), then lets the down kernel start: the down CTAs
//    become resident beside the gate/up CTAs (the two kernels' shared memory and registers fit one
//    SM together) and stream their weights while gate/up computes.  They learn that the intermediate
//    is complete from a counter every gate/up CTA bumps when it has written its part -- the gate/up
//    kernel never waits for the down kernel and all its CTAs run before the first down CTA starts, so
//    the wait cannot deadlock, and it is bounded.  The down kernel lets the next kernel start early.
//  * Dequantisation costs no per-weight arithmetic: a nibble becomes the exact BF16 value
//    128 + (code + 8) with one LOP3 per two weights (0x4300 | nibble) and goes straight into
//    m16n8k16 BF16 warp MMAs whose B operand is the activation vector, exact in BF16 as it is; the
//    constant 136 is removed by starting every accumulator at -136 * sum(x) of its 128-wide group,
//    and the group scale is applied once per group in float32.  Q8 bytes are split into two nibbles
//    that meet x and 16 x in the B operand, so they run through the same instructions.  On B200 the
//    HBM-to-issue-rate ratio leaves < 3 instructions per 4-bit weight, which rules out per-weight
//    FMA on the CUDA cores; the warp MMA does the multiply-add and the CUDA cores only unpack.
//  * Gate/up tile = 8 gate rows + 8 up rows of 8 features (column 0 of the MMA), gate and up rows
//    alternating over the MMA rows so that the 8 lanes of a shared-memory access phase read one
//    128-byte line of the gate block and one of the up block (64 bytes apart modulo 128): no bank
//    conflicts without padding every row.  Down tile = 2 output rows x up to 8 routed slots: MMA row g
//    holds slot g's weight row, MMA column g slot g's intermediate, the diagonal of the product is
//    what is kept -- all slots of an output row meet in one CTA, which therefore does the ordered BF16
//    combine itself.  The BF16 shared expert enters the same tiles with its K dimension cut into 8
//    segments in place of the slots.
#include "../../include/umaq_b200.h"
#include "common.cuh"
#include "decode.cuh"

#include <algorithm>
#include <cstdlib>
#include <mutex>

namespace umaq {
namespace {

// Warps per CTA.  The gate/up kernel is bound by dependency latency (shared-memory loads -> unpacking -> MMA ->
// scaling), not by any pipe, so it runs 16 warps of at most 64 registers; the down kernel 8 warps of at most 96.
// Registers are split over the SM's four schedulers, 16384 each: 4 x 2048 + 2 x 3072 fits, one warp more of
// either kernel on a scheduler does not, and then the two kernels cannot share the SM.  So there is no extra
// producer warp: when a CTA's whole share fits its shared memory (OLMoE) all warps issue the copies up front
// and all of them compute; otherwise the last warps produce (issuing a bulk copy costs its warp about 100 ns
// and a ring stage of row pieces takes up to 18 of them, so the stages go round several producer warps) and
// the others compute.
constexpr int kNW = 8;                        // down kernel
constexpr int kThreadsD = kNW * 32;
constexpr int kGW = 16;                       // gate/up kernel
constexpr int kGProducers = 4;                // warps that feed the ring when a CTA's share does not fit it at once
constexpr int kDProducers = 2;
constexpr int kThreadsG = kGW * 32;
constexpr int kMaxSlots = 8;
// The two kernels share an SM: their dynamic shared memory together stays under kPairSmemBudget (228 KB per SM
// minus 1 KB reserve and the static arrays of each CTA).  The down kernel is planned first and takes what its
// whole share needs, up to kDownSmemMax; the gate/up kernel gets the rest.
constexpr int kPairSmemBudget = 224 * 1024;
constexpr int kDownSmemMax = 112 * 1024;
constexpr int kDownSmemCeiling = 160 * 1024;      // what the kernel is allowed to ask for (UMAQ_DECODE_DOWN_SMEM)
constexpr long long kDecodeWaitCycles = 40ll * 1000 * 1000;     // ~20 ms of SM clock: far beyond any healthy wait
constexpr int kSyncStatus = 2, kSyncGateUpDone = 4, kSyncTarget = 6;

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void red_release_add_u32(unsigned* p, unsigned v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void cp_async8(void* dst_smem, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
// The barrier receives one arrival when all cp.async copies this thread issued so far have landed
// (the arrival is part of the barrier's initial count).
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// try_wait with a suspend-time hint: the warp sleeps in hardware until the phase completes (or the hint
// runs out) instead of re-issuing the test -- waiting warps must not take issue slots and shared-memory
// pipe cycles from the producer warp that shares their scheduler.
__device__ __forceinline__ bool mbar_try_wait_suspended(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
// Bounded wait that also gives up when another warp of the CTA has already failed.
__device__ __forceinline__ bool wait_or_fail(uint64_t* bar, uint32_t parity, volatile int* fail) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();                 // the SM's own counter: cheap to read
  for (;;) {
    if (mbar_try_wait_suspended(bar, parity, 100000u)) return true;
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

// Eight consecutive activations (raw, starting at k0, a multiple of 8) -> their fragment chunks (one
// slot), as whole 16-byte stores; returns their float32 sum.
__device__ __forceinline__ float store_x_fragments(int enc, uint4 raw, int k0, uint8_t* xf) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) sum += __uint_as_float(w[j] << 16) + __uint_as_float(w[j] & 0xffff0000u);
  if (enc == ENC_Q4) {
    // (e0,e1)(e2,e3)(e4,e5)(e6,e7) -> (e0,e4)(e1,e5)(e2,e6)(e3,e7)
    uint4 q;
    q.x = prmt(raw.x, raw.z, 0x5410); q.y = prmt(raw.x, raw.z, 0x7632);
    q.z = prmt(raw.y, raw.w, 0x5410); q.w = prmt(raw.y, raw.w, 0x7632);
    *reinterpret_cast<uint4*>(xf + frag_offset(ENC_Q4, 1, 0, k0, 0)) = q;
  } else if (enc == ENC_Q8) {
    const __nv_bfloat162 sixteen = __float2bfloat162_rn(16.f);
#pragma unroll
    for (int h = 0; h < 2; ++h) {          // four activations per chunk: [x0,x2,16x0,16x2,x1,x3,16x1,16x3]
      const uint32_t lo = h ? raw.z : raw.x, hi = h ? raw.w : raw.y;
      uint4 q;
      q.x = prmt(lo, hi, 0x5410); q.z = prmt(lo, hi, 0x7632);
      __nv_bfloat162 a = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&q.x), sixteen);
      __nv_bfloat162 b = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&q.z), sixteen);
      q.y = *reinterpret_cast<uint32_t*>(&a); q.w = *reinterpret_cast<uint32_t*>(&b);
      *reinterpret_cast<uint4*>(xf + frag_offset(ENC_Q8, 1, 0, k0 + 4 * h, 0)) = q;
    }
  } else {
    *reinterpret_cast<uint4*>(xf + frag_offset(ENC_BF16, 1, 0, k0, 0)) = raw;
  }
  return sum;
}

// Sum of every item's activations from the per-thread sums of 8 (an item is 16 (Q4) or 8 (Q8) neighbouring threads).
__device__ __forceinline__ void store_item_sums(int enc, float sum, int k0, float* gsum) {
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
    // Two words (j, j+1) of every item at a time: first the MMAs on their low nibble pairs, then the ones on
    // the high pairs, so that the two MMAs of an accumulator are 2N - 1 other MMAs apart.
#pragma unroll
    for (int jp = 0; jp < 4; jp += 2) {
      uint4 b[2][SHARE_B ? 1 : N];
#pragma unroll
      for (int jj = 0; jj < 2; ++jj)
#pragma unroll
        for (int n = 0; n < (SHARE_B ? 1 : N); ++n) b[jj][n] = lds128(bp[n] + (jp + jj) * bstep);
      uint32_t a[2][N], a8[2][N];
#pragma unroll
      for (int jj = 0; jj < 2; ++jj)
#pragma unroll
        for (int n = 0; n < N; ++n) {
          const int j = jp + jj;
          a[jj][n] = j == 0 ? wa[n].x : j == 1 ? wa[n].y : j == 2 ? wa[n].z : wa[n].w;
          a8[jj][n] = j == 0 ? wb[n].x : j == 1 ? wb[n].y : j == 2 ? wb[n].z : wb[n].w;
        }
#pragma unroll
      for (int jj = 0; jj < 2; ++jj)
#pragma unroll
        for (int n = 0; n < N; ++n) {
          const uint4& bb = b[jj][SHARE_B ? 0 : n];
          mma_bf16_16816(acc[n][jp + jj], nib_bf16<kLo>(a[jj][n]), nib_bf16<kLo>(a8[jj][n]), nib_bf16<kHi>(a[jj][n] >> 4),
                         nib_bf16<kHi>(a8[jj][n] >> 4), bb.x, bb.y);
        }
#pragma unroll
      for (int jj = 0; jj < 2; ++jj)
#pragma unroll
        for (int n = 0; n < N; ++n) {
          const uint4& bb = b[jj][SHARE_B ? 0 : n];
          mma_bf16_16816(acc[n][jp + jj], nib_bf16<kLo>(a[jj][n] >> 8), nib_bf16<kLo>(a8[jj][n] >> 8),
                         nib_bf16<kHi>(a[jj][n] >> 12), nib_bf16<kHi>(a8[jj][n] >> 12), bb.z, bb.w);
        }
    }
#pragma unroll
    for (int n = 0; n < N; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) c[n][e] = (acc[n][0][e] + acc[n][1][e]) + (acc[n][2][e] + acc[n][3][e]);
  }
}

// ---- integer path of the gate/up kernel (Q4 / Q8 rows) ---------------------------------------------------
// The activation vector becomes 24-bit fixed point, x * 2^s rounded to an integer v with |v| < 2^23 (s from the
// vector's largest magnitude; a BF16 value within 2^-15 of that magnitude is represented exactly), split into
// three signed base-256 digits v = d2 * 65536 + d1 * 256 + d0.  The digits are the B operand of int8 warp MMAs
// (m16n8k32, int32 accumulation: exact), one digit per MMA column: column 0 = d2, 1 = d1, 2 = d0, column 3
// zero.  The A operand needs next to no unpacking: a Q4 word of 8 nibbles gives (w << 4) & 0xF0F0F0F0 -- the
// even nibbles as the signed bytes 16 * code -- and w & 0xF0F0F0F0 -- the odd ones --, three instructions per
// 8 weights and no bias to remove; a Q8 word is four int8 codes as it stands.
//
// Fragment layout [item][column 0..3][t]: 32 bytes per entry for Q4 (MMA j of the item, j = 0..3, takes bytes
// 8j..8j+7: the digits of x[base + 0,2,4,6] then of x[base + 1,3,5,7], base = item*128 + 32t + 8j), 16 bytes
// for Q8 (MMA h = 0,1 takes bytes 8h..8h+7: x[base..base+3], x[base+4..base+7], base = item*64 + 16t + 8h).
__device__ __forceinline__ void mma_s8_16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                             uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Power of two that puts the magnitude `am` into [2^21, 2^22) -- the fixed-point scale of one item's
// activations -- and its reciprocal.  (v + 0x808080 then lies inside [0, 2^24) and its three bytes, each
// xor 0x80, are the signed base-256 digits of v.)
__device__ __forceinline__ void item_scale(float am, float& scale, float& inv) {
  const int eb = (int)((__float_as_uint(am) >> 23) & 0xff);          // am = 1.m * 2^(eb - 127)
  const int shift = (eb == 0 || eb == 255) ? 0 : 21 - (eb - 127);
  const int sb = min(max(shift + 127, 1), 253);
  scale = __uint_as_float((unsigned)sb << 23);
  inv = __uint_as_float((unsigned)(254 - sb) << 23);
}
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
// byte `idx` of a, b, c, d packed into one word
__device__ __forceinline__ uint32_t pack_bytes(uint32_t a, uint32_t b, uint32_t c, uint32_t d, int idx) {
  const uint32_t sel = (uint32_t)((4 + idx) << 4 | idx);
  return prmt(prmt(a, b, sel), prmt(c, d, sel), 0x5410);
}

// Eight consecutive activations (raw BF16, starting at k0) -> their digit bytes in the four columns, with the
// fixed-point scale of their own item (128 activations for Q4, 64 for Q8: the 16 / 8 neighbouring threads of a
// warp agree on it by shuffle); the thread of the item's first activations stores the reciprocal (for Q4 with
// the 1/16 of the byte trick) into xinv[item].  All 32 lanes of a warp call it together.
template <int ENC>
__device__ __forceinline__ void store_x_digits(uint4 raw, int k0, uint8_t* xf, float* xinv) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  float am = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) am = fmaxf(am, fmaxf(fabsf(bf16_lo(w[j])), fabsf(bf16_hi(w[j]))));
  am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));
  am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 2));
  am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 4));
  if (ENC == ENC_Q4) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 8));
  float scale, inv;
  item_scale(am, scale, inv);
  uint32_t u[8];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    u[2 * j] = (uint32_t)(__float2int_rn(bf16_lo(w[j]) * scale) + 0x808080);
    u[2 * j + 1] = (uint32_t)(__float2int_rn(bf16_hi(w[j]) * scale) + 0x808080);
  }
  int item, t, off, entry;
  if (ENC == ENC_Q4) { item = k0 >> 7; t = (k0 >> 5) & 3; off = ((k0 >> 3) & 3) * 8; entry = 32; }
  else { item = k0 >> 6; t = (k0 >> 4) & 3; off = ((k0 >> 3) & 1) * 8; entry = 16; }
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint2 q = make_uint2(0u, 0u);
    if (c < 3) {          // column c holds byte 2 - c; Q4: b0 = activations 0,2,4,6, b1 = 1,3,5,7; Q8: b0 = 0..3, b1 = 4..7
      if (ENC == ENC_Q4) { q.x = pack_bytes(u[0], u[2], u[4], u[6], 2 - c); q.y = pack_bytes(u[1], u[3], u[5], u[7], 2 - c); }
      else { q.x = pack_bytes(u[0], u[1], u[2], u[3], 2 - c); q.y = pack_bytes(u[4], u[5], u[6], u[7], 2 - c); }
      q.x ^= 0x80808080u; q.y ^= 0x80808080u;
    }
    *reinterpret_cast<uint2*>(xf + ((item * 4 + c) * 4 + t) * entry + off) = q;
  }
  if ((k0 & (ENC == ENC_Q4 ? 127 : 63)) == 0) xinv[item] = ENC == ENC_Q4 ? inv * 0.0625f : inv;
}

// N items: int32 sums of 16 MMA rows x 64 bytes of codes against the digit columns.  c[n][0], c[n][1] = row g,
// columns 2t, 2t+1; c[n][2], c[n][3] = row g + 8.  For Q4 the sums carry the factor 16 of the byte trick.
template <int ENC, int N>
__device__ __forceinline__ void items_imma(const uint32_t (&a0)[N], uint32_t a8off, const uint32_t (&bp)[N], int (&c)[N][4]) {
  uint4 wa[N], wb[N];
#pragma unroll
  for (int n = 0; n < N; ++n) { wa[n] = lds128(a0[n]); wb[n] = lds128(a0[n] + a8off); }
  int acc[N][2][4];
#pragma unroll
  for (int n = 0; n < N; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[n][0][e] = acc[n][1][e] = 0;
  if (ENC == ENC_Q4) {
    uint4 b[N][2];
#pragma unroll
    for (int n = 0; n < N; ++n) { b[n][0] = lds128(bp[n]); b[n][1] = lds128(bp[n] + 16); }
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int n = 0; n < N; ++n) {
        const uint32_t a = j == 0 ? wa[n].x : j == 1 ? wa[n].y : j == 2 ? wa[n].z : wa[n].w;
        const uint32_t a8 = j == 0 ? wb[n].x : j == 1 ? wb[n].y : j == 2 ? wb[n].z : wb[n].w;
        const uint32_t b0 = j == 0 ? b[n][0].x : j == 1 ? b[n][0].z : j == 2 ? b[n][1].x : b[n][1].z;
        const uint32_t b1 = j == 0 ? b[n][0].y : j == 1 ? b[n][0].w : j == 2 ? b[n][1].y : b[n][1].w;
        mma_s8_16832(acc[n][j & 1], (a << 4) & 0xF0F0F0F0u, (a8 << 4) & 0xF0F0F0F0u, a & 0xF0F0F0F0u, a8 & 0xF0F0F0F0u, b0, b1);
      }
  } else {
#pragma unroll
    for (int n = 0; n < N; ++n) {
      const uint4 b = lds128(bp[n]);
      mma_s8_16832(acc[n][0], wa[n].x, wb[n].x, wa[n].y, wb[n].y, b.x, b.y);
      mma_s8_16832(acc[n][1], wa[n].z, wb[n].z, wa[n].w, wb[n].w, b.z, b.w);
    }
  }
#pragma unroll
  for (int n = 0; n < N; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) c[n][e] = acc[n][0][e] + acc[n][1][e];
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
// Stage layout: gate block (8 rows x ch bytes), 64 bytes further than its end the up block, then the
// scales [16][groups] (gate rows, then up rows).  MMA row m holds, for m even, gate row m/2 (+4 for
// m >= 8), for m odd the up row of the same feature.  A warp takes the items i0, i0 + 8, ... of every
// stage, two at a time; i0 rotates with the running item count so that stages whose item count is no
// multiple of 8 still load the warps evenly.
template <int ENC>
__device__ __forceinline__ void gateup_units(const DecodeKernelPlan& P, const DecodeKind& K, int u0, int u1, int ub,
                                             uint32_t smem_base, uint64_t* full, uint64_t* empty, float* red, Ring& ring,
                                             volatile int* fail, int warp, int lane, bool skip, int ncons,
                                             unsigned* dbg_stamps = nullptr) {
  const int g = lane >> 2, t = lane & 3;
  const uint32_t lane_a = (g & 1) * K.mstride + (g >> 1) * K.ch + t * 16, a8off = 4 * K.ch;
  // fragments: BF16 rows [item][t] x 16 bytes; quantised rows the digit columns [item][column][t] x 32 / 16 bytes
  constexpr uint32_t kEntry = ENC == ENC_Q4 ? 32 : 16;
  constexpr uint32_t kFragItem = ENC == ENC_BF16 ? 64 : 16 * kEntry;
  const uint32_t xf = smem_base + K.frag_off + (ENC == ENC_BF16 ? t * 16 : ((g < 3 ? g : 3) * 4 + t) * kEntry);
  const uint32_t xinv = smem_base + K.gsum_off;
  const int srow = (g & 1) * 8 + (g >> 1);                           // row of MMA row g in the scale block / the sums
  const uint32_t sc_g = (uint32_t)srow * K.groups * 4, sc_g8 = (uint32_t)(srow + 4) * K.groups * 4;
  // weight of this lane's two columns in the digit sum: lane t = 0 holds d2 and d1, t = 1 holds d0
  const float k0w = t == 0 ? 65536.f : (t == 1 ? 1.f : 0.f), k1w = t == 0 ? 256.f : 0.f;
  for (int u = u0; u < u1; ++u) {
    float acc0 = 0.f, acc8 = 0.f;
    for (int ch = 0; ch < K.nch; ++ch) {
      int i0 = warp - ring.qbase;                                  // a stage has at most 16 items: with 16
      if (i0 < 0) i0 += ncons;                                      // consumers one per warp
      if (dbg_stamps && (u - ub) < 8 && threadIdx.x == 0 && blockIdx.x == 0)
        reinterpret_cast<unsigned long long*>(dbg_stamps)[48 + 2 * (u - ub)] = global_ns();
      if (i0 < K.ips && wait_or_fail(full + ring.slot, ring.round & 1, fail) && !skip) {
        if (dbg_stamps && (u - ub) < 8 && threadIdx.x == 0 && blockIdx.x == 0)
          reinterpret_cast<unsigned long long*>(dbg_stamps)[49 + 2 * (u - ub)] = global_ns();
        const uint32_t st = smem_base + ring.slot * P.stage_bytes, sc = st + P.scale_off;
        for (int i = i0; i < K.ips; i += ncons) {
        const int gi = ch * K.ips + i;
        const uint32_t a0[1] = {st + lane_a + i * 64};
        const uint32_t bp[1] = {xf + gi * kFragItem};
        if (ENC == ENC_BF16) {
          const float zero[1] = {0.f};
          float c[1][4];
          items_mma<ENC_BF16, 1, false>(a0, a8off, bp, 64, zero, zero, c);
          acc0 += c[0][0]; acc8 += c[0][2];
        } else {
          const int grp = ENC == ENC_Q4 ? gi : gi >> 1;
          const float xi = lds32(xinv + gi * 4);                    // undoes the item's fixed-point scale
          const float s0 = lds32(sc + sc_g + grp * 4) * xi, s8 = lds32(sc + sc_g8 + grp * 4) * xi;
          int c[1][4];
          items_imma<ENC, 1>(a0, a8off, bp, c);
          acc0 = fmaf(s0, fmaf((float)c[0][0], k0w, (float)c[0][1] * k1w), acc0);
          acc8 = fmaf(s8, fmaf((float)c[0][2], k0w, (float)c[0][3] * k1w), acc8);
        }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty + ring.slot);
      ring.qbase = (ring.qbase + K.ips) % ncons;
      ring.advance(P.stages);
    }
    if (ENC != ENC_BF16) {            // the lane of column 2 hands its share to the lane of columns 0 and 1
      acc0 += __shfl_down_sync(0xffffffffu, acc0, 1);
      acc8 += __shfl_down_sync(0xffffffffu, acc8, 1);
    }
    if (t == 0) {                     // [0..7] gate sums of the unit's 8 features, [8..15] up sums
      float* r = red + ((size_t)(u - ub) * kGW + warp) * 16;
      r[srow] = acc0; r[srow + 4] = acc8;
    }
  }
}

// ---- gate/up, Q4, whole share resident (the OLMoE shape): warp w owns item w of every stage ------------
// The item body is bound by shared-memory wavefronts (128 bytes per cycle and SM), and the weights alone
// need 8 of them per item.  So everything else stays out of shared memory: the warp's digit columns are
// loop-invariant and live in registers, and its group scales (row r of stage s, group w) were fetched
// from global memory into sreg[] at kernel start -- value v = 16 s + r in register v >> 5 of lane v & 31 --
// and reach the lanes that need them by shuffle.
__device__ __forceinline__ void gateup_q4_resident(const DecodeKernelPlan& P, const DecodeKind& K, int units,
                                                   uint32_t smem_base, uint64_t* full, float* red, volatile int* fail,
                                                   int warp, int lane, bool skip, const float (&sreg)[4],
                                                   const __nv_bfloat16* __restrict__ x, uint8_t* smem) {
  const int g = lane >> 2, t = lane & 3;
  const uint32_t lane_a = (g & 1) * K.mstride + (g >> 1) * K.ch + t * 16 + warp * 64, a8off = 4 * K.ch;
  const uint32_t xf = smem_base + K.frag_off + warp * 512 + ((g < 3 ? g : 3) * 4 + t) * 32;
  const int srow = (g & 1) * 8 + (g >> 1);
  // The warp converts its own item's 128 activations (four per lane) to digits, through its own 512 bytes of
  // shared memory: nothing here waits for another warp.
  float xi;
  {
    const uint2 raw = *reinterpret_cast<const uint2*>(x + warp * 128 + lane * 4);
    float am = fmaxf(fmaxf(fabsf(bf16_lo(raw.x)), fabsf(bf16_hi(raw.x))), fmaxf(fabsf(bf16_lo(raw.y)), fabsf(bf16_hi(raw.y))));
#pragma unroll
    for (int o = 16; o; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
    float scale;
    item_scale(am, scale, xi);
    xi *= 0.0625f;                                       // the 16 of the byte trick
    const uint32_t u0 = (uint32_t)(__float2int_rn(bf16_lo(raw.x) * scale) + 0x808080);
    const uint32_t u1 = (uint32_t)(__float2int_rn(bf16_hi(raw.x) * scale) + 0x808080);
    const uint32_t u2 = (uint32_t)(__float2int_rn(bf16_lo(raw.y) * scale) + 0x808080);
    const uint32_t u3 = (uint32_t)(__float2int_rn(bf16_hi(raw.y) * scale) + 0x808080);
    // activations 4 lane .. 4 lane + 3 of the item: word j = (lane >> 1) & 3 of lane-quarter t' = lane >> 3; inside
    // the word nibbles 4 (lane & 1) + {0,1,2,3}: the even ones are bytes 2 (lane & 1) + {0,1} of b0, the odd ones of b1
    uint8_t* entry0 = smem + K.frag_off + warp * 512 + (lane >> 3) * 32 + ((lane >> 1) & 3) * 8 + (lane & 1) * 2;
#pragma unroll
    for (int c = 0; c < 3; ++c) {
      const uint32_t sel = (uint32_t)((4 + (2 - c)) << 4 | (2 - c));
      *reinterpret_cast<uint16_t*>(entry0 + c * 128) = (uint16_t)((prmt(u0, u2, sel) & 0xffffu) ^ 0x8080u);
      *reinterpret_cast<uint16_t*>(entry0 + c * 128 + 4) = (uint16_t)((prmt(u1, u3, sel) & 0xffffu) ^ 0x8080u);
    }
    *reinterpret_cast<uint32_t*>(smem + K.frag_off + warp * 512 + 3 * 128 + lane * 4) = 0u;       // column 3: zeros
    __syncwarp();
  }
  const float k0w = (t == 0 ? 65536.f : (t == 1 ? 1.f : 0.f)) * xi, k1w = (t == 0 ? 256.f : 0.f) * xi;
  const uint4 b0 = lds128(xf), b1 = lds128(xf + 16);
  const uint32_t bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
  for (int s = 0; s < units; ++s) {
    float acc0 = 0.f, acc8 = 0.f;
    if (wait_or_fail(full + s, 0, fail) && !skip) {
      const uint32_t st = smem_base + s * P.stage_bytes + lane_a;
      const uint4 wa = lds128(st), wb = lds128(st + a8off);
      const float sv = (s >> 1) == 0 ? sreg[0] : (s >> 1) == 1 ? sreg[1] : (s >> 1) == 2 ? sreg[2] : sreg[3];
      const float s0 = __shfl_sync(0xffffffffu, sv, ((s & 1) << 4) + srow);
      const float s8 = __shfl_sync(0xffffffffu, sv, ((s & 1) << 4) + srow + 4);
      const uint32_t ra[4] = {wa.x, wa.y, wa.z, wa.w}, rb[4] = {wb.x, wb.y, wb.z, wb.w};
      int acc[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
#pragma unroll
      for (int j = 0; j < 4; ++j)
        mma_s8_16832(acc[j & 1], (ra[j] << 4) & 0xF0F0F0F0u, (rb[j] << 4) & 0xF0F0F0F0u, ra[j] & 0xF0F0F0F0u,
                     rb[j] & 0xF0F0F0F0u, bb[2 * j], bb[2 * j + 1]);
      acc0 = s0 * fmaf((float)(acc[0][0] + acc[1][0]), k0w, (float)(acc[0][1] + acc[1][1]) * k1w);
      acc8 = s8 * fmaf((float)(acc[0][2] + acc[1][2]), k0w, (float)(acc[0][3] + acc[1][3]) * k1w);
    }
    acc0 += __shfl_down_sync(0xffffffffu, acc0, 1);      // the lane of column 2 hands its share to the lane of 0 and 1
    acc8 += __shfl_down_sync(0xffffffffu, acc8, 1);
    if (t == 0) {
      float* r = red + ((size_t)s * kGW + warp) * 16;
      r[srow] = acc0; r[srow + 4] = acc8;
    }
  }
}

// =====================================================================================================
// Kernel A: gate/up + SwiGLU.  Work unit = 8 features of one slot: 8 gate rows and 8 up rows, all of
// K = hidden, in nch ring stages of 16 rows x ch bytes.
// =====================================================================================================
__global__ void __maxnreg__(64) decode_gateup_kernel(const DecodeParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ int s_expert[kMaxSlots];
  __shared__ int s_fail;
  const DecodeKernelPlan& P = p.g;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + P.bar_off);
  uint64_t* empty = full + P.stages;
  const int H = p.hidden;
  const int U0 = P.kind[0].units, upr = p.inter >> 3;
  const int ub = first_unit(P, blockIdx.x), ue = first_unit(P, blockIdx.x + 1);
  // all_at_once: the CTA's whole share fits the ring, every warp issues copies and computes; otherwise the
  // last kGProducers warps produce and the others compute
  const bool whole_rows = P.kind[0].nch == 1 && (P.kind[1].units == 0 || P.kind[1].nch == 1);
  const bool all_at_once = whole_rows && ue - ub <= P.stages;
  const int nprod = P.producers;
  const int ncons = all_at_once ? kGW : kGW - nprod;
  const bool consumer = warp < ncons;
  // resident Q4 fast path: every unit of this CTA is a routed one, a stage has one item per warp
  const bool fast = all_at_once && P.kind[0].enc == ENC_Q4 && P.kind[0].ips == kGW && ue <= U0 && ue - ub <= 8;
  if (tid == 0) {
    for (int s = 0; s < P.stages; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, ncons); }
    s_fail = 0;
    fence_barrier_init();
  }
  stamp(p, 0, 0);
  pdl_wait();                    // the routes and the activation vector come from the kernels before this one
  stamp(p, 1, 0);
  if (blockIdx.x == 0 && tid == 0) {
    // the count of finished gate/up CTAs the down kernel of this call waits for: the counter never goes
    // back, every call adds its grid to the target (published before this CTA lets the down kernel start)
    asm volatile("red.relaxed.gpu.global.add.u32 [%0], %1;" ::"l"(p.sync + kSyncTarget), "r"(gridDim.x) : "memory");
    __threadfence();              // (no load to wait for: the fence overlaps the other threads' routes load)
  }
  // the activation vector is on its way while the routes are read
  uint4 x_first = make_uint4(0, 0, 0, 0);
  if (consumer && !fast && tid * 8 < H) x_first = *reinterpret_cast<const uint4*>(p.x + tid * 8);
  if (tid < p.top_k) {
    long long e = load_index(p.idx, p.idx64, tid);
    if (e < 0 || e >= p.experts) {          // the reference skips such a route; here its weight becomes 0 in the
      atomicExch(p.sync + kSyncStatus, (unsigned)ERR_BAD_ARGUMENT);   // down kernel and the status word records it
      e = 0;
    }
    s_expert[tid] = (int)e;
  }
  __syncthreads();
  pdl_launch_dependents();       // the down kernel may become resident and stream its weights from here on
  stamp(p, 2, 0);

  volatile int* fail = &s_fail;

  float sreg[4] = {0.f, 0.f, 0.f, 0.f};
  if (fast) {                    // this warp's group scales for every stage, straight into registers
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int v = 32 * q + lane, u = ub + (v >> 4), r = v & 15;
      if (u < ue) {
        const int sl = u / upr;
        const size_t row = (size_t)s_expert[sl] * p.inter + ((u - sl * upr) << 3) + (r & 7);
        sreg[q] = __ldg((r < 8 ? p.gate_s : p.up_s) + row * P.kind[0].groups + warp);
      }
    }
  }

  if (all_at_once) {
    // Everything fits the ring at once.  Issuing a bulk copy costs a warp about 100 ns, so the stages are
    // spread over all warps: lanes 0..3 of warp w issue the four copies of stages w, w + 16, ...
    for (int st_i = warp; st_i < ue - ub; st_i += kGW) {
      const int u = ub + st_i, c = lane, k = u >= U0 ? 1 : 0;
      const DecodeKind& K = P.kind[k];
      const uint32_t scale_bytes = 8u * K.groups * 4;
      if (lane < 4) {
        size_t row;
        if (k == 0) {
          const int sl = u / upr;
          row = (size_t)s_expert[sl] * p.inter + ((u - sl * upr) << 3);
        } else {
          row = (size_t)(u - U0) << 3;
        }
        const uint8_t* src = nullptr;
        uint32_t bytes = 0, dst = 0;
        if (c < 2) {
          const uint8_t* base_w = k == 0 ? (c ? p.up : p.gate) : reinterpret_cast<const uint8_t*>(c ? p.sh_up : p.sh_gate);
          src = base_w + row * K.row_bytes; bytes = (p.debug & 2) ? 0u : 8u * K.ch; dst = c * K.mstride;
        } else if (K.groups && !fast) {
          src = reinterpret_cast<const uint8_t*>((c == 2 ? p.gate_s : p.up_s) + row * K.groups);
          bytes = scale_bytes; dst = P.scale_off + (c - 2) * scale_bytes;
        }
        if (c == 0) mbar_expect_tx(full + st_i, ((p.debug & 2) ? 0u : 16u * K.ch) + (fast ? 0u : 2 * scale_bytes));
        if (bytes) bulk_g2s(smem + (size_t)st_i * P.stage_bytes + dst, src, bytes, full + st_i);
      }
    }
    stamp(p, 8, 32);
  }

  if (!consumer) {
    // ---- producer (when the CTA's share does not fit the ring at once): one stage = 8 gate rows, 8 up rows
    //      (one bulk copy each when the stage takes whole rows) and their scales ----------------------------
    if (!all_at_once) {
    // Issuing a bulk copy costs a warp about 100 ns, so the stages go round the producer warps.
    const int pj = warp - ncons;
    int n = 0;                                 // running stage number: slot n % stages, round n / stages
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
      const uint32_t scale_bytes = 8u * K.groups * 4;              // per projection
      for (int ch = 0; ch < K.nch; ++ch, ++n) {
        if (n % nprod != pj) continue;
        const int slot = n % P.stages, round = n / P.stages;
        if (round > 0 && !wait_or_fail(empty + slot, (round - 1) & 1, fail)) break;
        uint8_t* st = smem + (size_t)slot * P.stage_bytes;
        if (lane == 0) mbar_expect_tx(full + slot, ((p.debug & 2) ? 0u : 16u * K.ch) + 2 * scale_bytes);
        __syncwarp();
        if (!(p.debug & 2)) {
          if (K.nch == 1) {            // whole rows: the 8 rows of a projection are one contiguous block
            if (lane < 2) bulk_g2s(st + lane * K.mstride, lane ? usrc : gsrc, 8u * K.ch, full + slot);
          } else if (lane < 16) {
            bulk_g2s(st + (lane >> 3) * K.mstride + (lane & 7) * K.ch,
                     (lane < 8 ? gsrc : usrc) + (size_t)(lane & 7) * K.row_bytes + (size_t)ch * K.ch, K.ch, full + slot);
          }
        }
        if (K.groups && lane >= 16 && lane < 18)
          bulk_g2s(st + P.scale_off + (lane - 16) * scale_bytes, lane == 16 ? gs : us, scale_bytes, full + slot);
      }
    }
    }
    stamp(p, 8, (kGW - 1) * 32);
  } else {
    // ---- consumers ---------------------------------------------------------------------------------------------
    if (!fast) {
      const int e0 = P.kind[0].enc;
      const bool second = P.kind[1].units && P.kind[1].frag_off != P.kind[0].frag_off;
      uint8_t* xf0 = smem + P.kind[0].frag_off;
      float* xinv = reinterpret_cast<float*>(smem + P.kind[0].gsum_off);
      for (int k0 = tid * 8; k0 < H; k0 += ncons * 256) {
        const uint4 raw = k0 == tid * 8 ? x_first : *reinterpret_cast<const uint4*>(p.x + k0);
        if (e0 == ENC_BF16) store_x_fragments(ENC_BF16, raw, k0, xf0);
        else if (e0 == ENC_Q4) store_x_digits<ENC_Q4>(raw, k0, xf0, xinv);
        else store_x_digits<ENC_Q8>(raw, k0, xf0, xinv);
        if (second) store_x_fragments(ENC_BF16, raw, k0, smem + P.kind[1].frag_off);
      }
      named_bar_sync(1, ncons * 32);
    }
    stamp(p, 3, 0);
    float* red = reinterpret_cast<float*>(smem + P.red_off);
    const uint32_t smem_base = smem_u32(smem);
    Ring ring{0, 0, 0};
    const int um = min(max(ub, U0), ue);        // routed units [ub, um), shared-expert units [um, ue)
    const bool skip = (p.debug & 1) != 0;
    if (fast) gateup_q4_resident(P, P.kind[0], ue - ub, smem_base, full, red, fail, warp, lane, skip, sreg, p.x, smem);
    else if (ub < um) {
      if (P.kind[0].enc == ENC_Q4) gateup_units<ENC_Q4>(P, P.kind[0], ub, um, ub, smem_base, full, empty, red, ring, fail, warp, lane, skip, ncons, (p.debug & 4) ? p.sync : nullptr);
      else if (P.kind[0].enc == ENC_Q8) gateup_units<ENC_Q8>(P, P.kind[0], ub, um, ub, smem_base, full, empty, red, ring, fail, warp, lane, skip, ncons);
      else gateup_units<ENC_BF16>(P, P.kind[0], ub, um, ub, smem_base, full, empty, red, ring, fail, warp, lane, skip, ncons);
    }
    if (!fast && um < ue) gateup_units<ENC_BF16>(P, P.kind[1], um, ue, ub, smem_base, full, empty, red, ring, fail, warp, lane, skip, ncons);
    stamp(p, 5, 0);
  }
  __syncthreads();
  stamp(p, 6, 0);
  if (s_fail) {
    if (tid == 0) atomicExch(p.sync + kSyncStatus, (unsigned)ERR_DEVICE_TIMEOUT);
    __nanosleep(100000);           // copies still in flight land before the shared memory is given back
    return;
  }

  // ---- SwiGLU; every value goes where the down kernel's fragments expect it ----------------------------------
  if (tid < (ue - ub) * 8) {
    const int ul = tid >> 3, f = tid & 7, u = ub + ul;
    const float* r = reinterpret_cast<const float*>(smem + P.red_off) + (size_t)ul * kGW * 16;
    float gv = 0.f, uv = 0.f;
    for (int w = 0; w < ncons; ++w) { gv += r[w * 16 + f]; uv += r[w * 16 + 8 + f]; }
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
  __syncthreads();
  // Count this CTA as finished.  The release makes the intermediate values its threads stored above (ordered
  // before this point by the barrier) visible to whoever reads the counter with an acquire.
  if (tid == 0) red_release_add_u32(p.sync + kSyncGateUpDone, 1u);
  stamp(p, 7, 0);
}

// ---- down: the row pairs of one kind (compile-time encoding), two at a time ----------------------------
// The two row pairs of a round hold the same columns of different output rows, so they share the
// fragments and the start values; a warp takes the items i0, i0 + 8, ... of both.  Row pair s of the
// ring (or of the CTA's share, when it is resident) has its weights at s * pair_stride, slot g at
// g * mstride inside them, and its scales at sc_base + s * sc_pair_stride + g * sc_slot_stride.
template <int ENC>
__device__ __forceinline__ void down_pairs(const DecodeKernelPlan& P, const DecodeKind& K, int npairs, uint32_t smem_base,
                                           uint64_t* full, uint64_t* empty, float* red, Ring& ring, volatile int* fail,
                                           int warp, int lane, bool skip, int ncons) {
  const int g = lane >> 2, t = lane & 3;
  const int ga = g < K.nvs ? g : 0, gb = g & (K.ng - 1), c0 = (2 * t) & (K.ng - 1);
  const uint32_t lane_a = ga * K.mstride + t * 16, a8off = K.row_bytes;
  constexpr uint32_t kChunks = ENC == ENC_BF16 ? 1 : 4;
  const uint32_t frag_item = kChunks * K.ng * 64, bstep = K.ng * 64;
  const uint32_t fr = smem_base + K.frag_off + (gb * 4 + t) * 16;
  const uint32_t gs = smem_base + K.gsum_off + c0 * 4;
  const uint32_t sc_lane = smem_base + P.sc_base + (uint32_t)ga * P.sc_slot_stride;
  const bool odd = g & 1, diag = t == (g >> 1);
  const float nbias = -K.bias;
  if (P.resident && !wait_or_fail(full, 0, fail)) return;
  const int step = P.resident ? 2 : P.pair_step;
  for (int ul = 0; ul < npairs; ul += step) {
    const bool two = step == 2 && ul + 1 < npairs;
    int sa = ul, sb = two ? ul + 1 : ul;
    bool ready = true;
    int slot_a = 0, slot_b = 0;
    int i0 = warp - ring.qbase;
    if (i0 < 0) i0 += ncons;
    if (!P.resident) {
      slot_a = ring.slot; const int round_a = ring.round;
      ring.advance(P.stages);
      slot_b = two ? ring.slot : slot_a; const int round_b = two ? ring.round : round_a;
      if (two) ring.advance(P.stages);
      sa = slot_a; sb = slot_b;
      if (i0 < K.ips) ready = wait_or_fail(full + slot_a, round_a & 1, fail) && wait_or_fail(full + slot_b, round_b & 1, fail);
    }
    float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    if (i0 < K.ips && ready && !skip) {
      const uint32_t st_a = smem_base + sa * P.pair_stride + lane_a, st_b = smem_base + sb * P.pair_stride + lane_a;
      const uint32_t sc_a = sc_lane + sa * P.sc_pair_stride, sc_b = sc_lane + sb * P.sc_pair_stride;
      for (int i = i0; i < K.ips; i += ncons) {
        const uint32_t a0[2] = {st_a + i * 64, st_b + i * 64};
        const uint32_t bp[2] = {fr + i * frag_item, fr + i * frag_item};
        float in0[2] = {0.f, 0.f}, in1[2] = {0.f, 0.f}, s[2][2];
        if (ENC != ENC_BF16) {
          const float2 sums = lds64(gs + i * K.ng * 4);
          in0[0] = in0[1] = nbias * sums.x; in1[0] = in1[1] = nbias * sums.y;
          const int grp = ENC == ENC_Q4 ? i : i >> 1;
          s[0][0] = lds32(sc_a + grp * 4); s[0][1] = lds32(sc_a + (K.groups + grp) * 4);
          s[1][0] = lds32(sc_b + grp * 4); s[1][1] = lds32(sc_b + (K.groups + grp) * 4);
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
    if (!P.resident) {
      __syncwarp();
      if (lane == 0) { mbar_arrive(empty + slot_a); if (two) mbar_arrive(empty + slot_b); }
    }
    ring.qbase = (ring.qbase + K.ips) % ncons;
    if (diag) {                      // the lane that holds column g
      float* r = red + ((size_t)ul * kNW + warp) * 16;
      r[2 * g] = acc[0][0]; r[2 * g + 1] = acc[0][1];
      if (two) { r[kNW * 16 + 2 * g] = acc[1][0]; r[kNW * 16 + 2 * g + 1] = acc[1][1]; }
    }
  }
}

// ---- down, quantised rows, whole share resident (the OLMoE shape): warp w owns item w of every row pair ---
// As in the gate/up kernel the weights' own 8 shared-memory wavefronts per item are the floor, so the
// loop-invariant intermediate fragments and their sums live in registers and the group scales come from
// global memory: value v = 8 j + slot (j = row of the CTA's share, 0 .. 2 npairs - 1) sits in register
// v >> 5 of lane v & 31 and reaches the lane that needs it by shuffle.
template <int ENC>
__device__ __forceinline__ void down_resident(const DecodeKernelPlan& P, const DecodeKind& K, int npairs, uint32_t smem_base,
                                              uint64_t* full, float* red, volatile int* fail, int warp, int lane, bool skip,
                                              const float (&sreg)[4]) {
  const int g = lane >> 2, t = lane & 3;
  const int ga = g < K.nvs ? g : 0, gb = g & (K.ng - 1), c0 = (2 * t) & (K.ng - 1);
  const uint32_t lane_a = smem_base + ga * K.mstride + t * 16 + warp * 64, a8off = K.row_bytes;
  const uint32_t bstep = K.ng * 64;
  const uint32_t fr = smem_base + K.frag_off + warp * 4 * bstep + (gb * 4 + t) * 16;
  const bool odd = g & 1, diag = t == (g >> 1);
  constexpr uint32_t kLo = ENC == ENC_Q4 ? 0x43084308u : 0x43004300u, kHi = 0x43084308u;
  uint4 b[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) b[j] = lds128(fr + j * bstep);
  const float2 sums = lds64(smem_base + K.gsum_off + (warp * K.ng + c0) * 4);
  const float in0 = -K.bias * sums.x, in1 = -K.bias * sums.y;
  const bool ready = wait_or_fail(full, 0, fail);
  for (int ul = 0; ul < npairs; ul += 2) {
    const bool two = ul + 1 < npairs;
    float res[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    // scales of rows 2 ul .. 2 ul + 3 for slot ga
    float sc[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int j = 2 * ul + r, q = j >> 2;
      const float sv = q == 0 ? sreg[0] : q == 1 ? sreg[1] : q == 2 ? sreg[2] : sreg[3];
      sc[r] = __shfl_sync(0xffffffffu, sv, ((j & 3) << 3) + ga);
    }
    if (ready && !skip) {
      uint4 wa[2], wb[2];
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        const uint32_t a = lane_a + (ul + (two ? n : 0)) * P.pair_stride;
        wa[n] = lds128(a); wb[n] = lds128(a + a8off);
      }
      float acc[2][4][4];
#pragma unroll
      for (int n = 0; n < 2; ++n) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) acc[n][j][e] = 0.f;
        acc[n][0][0] = in0; acc[n][0][1] = in1; acc[n][0][2] = in0; acc[n][0][3] = in1;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int n = 0; n < 2; ++n) {
          const uint32_t a = j == 0 ? wa[n].x : j == 1 ? wa[n].y : j == 2 ? wa[n].z : wa[n].w;
          const uint32_t a8 = j == 0 ? wb[n].x : j == 1 ? wb[n].y : j == 2 ? wb[n].z : wb[n].w;
          mma_bf16_16816(acc[n][j], nib_bf16<kLo>(a), nib_bf16<kLo>(a8), nib_bf16<kHi>(a >> 4), nib_bf16<kHi>(a8 >> 4), b[j].x, b[j].y);
          mma_bf16_16816(acc[n][j], nib_bf16<kLo>(a >> 8), nib_bf16<kLo>(a8 >> 8), nib_bf16<kHi>(a >> 12),
                         nib_bf16<kHi>(a8 >> 12), b[j].z, b[j].w);
        }
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        float sum[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) sum[e] = (acc[n][0][e] + acc[n][1][e]) + (acc[n][2][e] + acc[n][3][e]);
        const float v0 = odd ? sum[1] : sum[0], v8 = odd ? sum[3] : sum[2];     // column g of rows g, g + 8
        res[n][0] = sc[2 * n] * v0; res[n][1] = sc[2 * n + 1] * v8;
      }
    }
    if (diag) {                      // the lane that holds column g
      float* r = red + ((size_t)ul * kNW + warp) * 16;
      r[2 * g] = res[0][0]; r[2 * g + 1] = res[0][1];
      if (two) { r[kNW * 16 + 2 * g] = res[1][0]; r[kNW * 16 + 2 * g + 1] = res[1][1]; }
    }
  }
}

// =====================================================================================================
// Kernel B: down + ordered combine.  Work unit = a pair of output rows (n, n+1): per routed slot those
// two rows of the slot's expert (MMA rows g and g + 8 for slot g); with a shared expert a second series
// of stages holds the two rows cut into K segments.
// =====================================================================================================
__global__ void __maxnreg__(96) decode_down_kernel(const DecodeParams p) {
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
  const uint32_t full_count = P.bulk_scales ? 1 : 1 + 32;
  // with the whole share issued up front by all warps every warp computes; otherwise the last kDProducers produce
  const bool all_at_once = P.resident && P.bulk_scales;
  const int nprod = P.producers;
  const int ncons = all_at_once ? kNW : kNW - nprod;
  const bool consumer = warp < ncons;
  // resident fast path: quantised rows, one item per warp
  const bool fast = all_at_once && P.kind[0].groups && P.kind[0].ips == kNW && !P.kind[1].nvs && P.max_units <= 8;
  if (tid == 0) {
    for (int s = 0; s < P.stages; ++s) { mbar_init(full + s, full_count); mbar_init(empty + s, ncons); }
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
      const long long ej = __shfl_sync(0xffu, e, j);
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

  if (all_at_once) {
    // The CTA's rows of a slot are contiguous in the expert's matrix: one copy per slot and one for its scales,
    // loading the whole share at once.  Warp g issues slot g's two copies (a bulk copy costs its warp ~100 ns).
    const DecodeKind& K0 = P.kind[0];
    const uint32_t wbytes = (uint32_t)npairs * 2 * K0.row_bytes, sbytes = fast ? 0u : (uint32_t)npairs * 2 * K0.groups * 4;
    if (tid == 0) mbar_expect_tx(full, K0.nvs * (((p.debug & 2) ? 0u : wbytes) + sbytes));
    if (warp < K0.nvs && lane < 2) {
      const size_t row = (size_t)s_expert[warp] * H + 2 * rp0;
      if (lane == 0 && !(p.debug & 2)) bulk_g2s(smem + warp * K0.mstride, p.down + row * K0.row_bytes, wbytes, full);
      if (lane == 1 && sbytes) bulk_g2s(smem + P.sc_base + warp * P.sc_slot_stride, p.down_s + row * K0.groups, sbytes, full);
    }
    stamp(p, 25, 0);
  }

  float sreg[4] = {0.f, 0.f, 0.f, 0.f};
  if (fast) {                    // this warp's group scales of every (row, slot) of the share, straight into registers
    const DecodeKind& K0 = P.kind[0];
    const int grp = K0.enc == ENC_Q4 ? warp : warp >> 1;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int v = 32 * q + lane, j = v >> 3, slot = v & 7;
      if (j < 2 * npairs && slot < K0.nvs)
        sreg[q] = __ldg(p.down_s + ((size_t)s_expert[slot] * H + 2 * rp0 + j) * K0.groups + grp);
    }
  }

  if (!consumer) {
    // ---- producer ----------------------------------------------------------------------------------------------
    const DecodeKind& K0 = P.kind[0];
    const int pj = warp - ncons;
    if (P.resident) {
      // (with 16-byte scale rows the copies were issued above by all warps)
      if (!P.bulk_scales && pj == 0) {
        const uint32_t wbytes = (uint32_t)npairs * 2 * K0.row_bytes;
        if (lane == 0) mbar_expect_tx(full, (p.debug & 2) ? 0u : K0.nvs * wbytes);
        __syncwarp();
        if (lane < K0.nvs && !(p.debug & 2))
          bulk_g2s(smem + lane * K0.mstride, p.down + ((size_t)s_expert[lane] * H + 2 * rp0) * K0.row_bytes, wbytes, full);
        const int per_slot = npairs * K0.groups;       // 8-byte pieces
        for (int i = lane; i < K0.nvs * per_slot; i += 32) {
          const int vs = i / per_slot, j = i - vs * per_slot;
          cp_async8(smem + P.sc_base + vs * P.sc_slot_stride + (size_t)j * 8,
                    p.down_s + ((size_t)s_expert[vs] * H + 2 * rp0) * K0.groups + 2 * j);
        }
        cp_async_arrive(full);
      }
    } else {
      int n = 0;                               // running stage number; the stages go round the producer warps
      for (int k = 0; k < kinds && !*fail; ++k) {
        const DecodeKind& K = P.kind[k];
        const uint32_t sbytes = 2u * K.groups * 4;
        for (int rp = rp0; rp < rp1; ++rp, ++n) {
          if (n % nprod != pj) continue;
          const int slot = n % P.stages, round = n / P.stages;
          if (round > 0 && !wait_or_fail(empty + slot, (round - 1) & 1, fail)) break;
          uint8_t* st = smem + (size_t)slot * P.stage_bytes;
          if (lane == 0)
            mbar_expect_tx(full + slot, ((p.debug & 2) ? 0u : (uint32_t)(K.nvs * 2 * K.row_bytes)) +
                                            (P.bulk_scales ? K.nvs * sbytes : 0u));
          __syncwarp();
          if (k == 0) {
            if (lane < K.nvs) {        // rows n and n+1 of the slot's expert are adjacent: one copy
              const size_t row = (size_t)s_expert[lane] * H + 2 * rp;
              if (!(p.debug & 2)) bulk_g2s(st + lane * K.mstride, p.down + row * K.row_bytes, 2u * K.row_bytes, full + slot);
              if (K.groups && P.bulk_scales)
                bulk_g2s(st + P.sc_base + lane * P.sc_slot_stride, p.down_s + row * K.groups, sbytes, full + slot);
            }
            if (K.groups && !P.bulk_scales) {     // [slot][2 rows][groups] floats in 8-byte pieces
              for (int i = lane; i < K.nvs * K.groups; i += 32) {
                const int vs = i / K.groups, j = i - vs * K.groups;
                cp_async8(st + P.sc_base + vs * P.sc_slot_stride + (size_t)j * 8,
                          p.down_s + ((size_t)s_expert[vs] * H + 2 * rp) * K.groups + 2 * j);
              }
            }
          } else if (lane < 2 * K.nvs && !(p.debug & 2)) {   // segment `seg` of rows n, n+1 of the shared expert's down matrix
            const int seg = lane >> 1, row = lane & 1;
            bulk_g2s(st + seg * K.mstride + row * K.row_bytes,
                     reinterpret_cast<const uint8_t*>(p.sh_down) + ((size_t)(2 * rp + row) * K.nvs + seg) * K.row_bytes,
                     (uint32_t)K.row_bytes, full + slot);
          }
          if (!P.bulk_scales) cp_async_arrive(full + slot);
        }
      }
    }
    stamp(p, 25, (kNW - 1) * 32);
  } else {
    // ---- consumers ---------------------------------------------------------------------------------------------
    if (S) {                       // sigmoid gate of the shared expert: bf16(sigmoid(bf16(x . wg)))
      float acc = 0.f;
      for (int k = tid * 2; k < H; k += ncons * 64) {
        const __nv_bfloat162 xv = *reinterpret_cast<const __nv_bfloat162*>(p.x + k);
        const __nv_bfloat162 gv = *reinterpret_cast<const __nv_bfloat162*>(p.sh_gatevec + k);
        acc += __low2float(xv) * __low2float(gv) + __high2float(xv) * __high2float(gv);
      }
#pragma unroll
      for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (lane == 0) s_tmp[warp] = acc;
      named_bar_sync(1, ncons * 32);
      if (tid == 0) {
        float sum = 0.f;
        for (int i = 0; i < ncons; ++i) sum += s_tmp[i];
        sum = bf16_round(sum);
        s_gate = bf16_round(1.f / (1.f + expf(-sum)));
      }
    }
    stamp(p, 18, 0);
    // The intermediate is complete when every gate/up CTA has counted itself in.  They all started before
    // this kernel and never wait for it, so the count always arrives; the wait is bounded all the same.
    if (tid == 0) {
      const unsigned want = ld_acquire_u32(p.sync + kSyncTarget);     // published before this kernel could start
      const long long t0 = clock64();
      while ((int)(ld_acquire_u32(p.sync + kSyncGateUpDone) - want) < 0) {
        if (clock64() - t0 > kDecodeWaitCycles) { s_fail = 1; break; }
      }
    }
    named_bar_sync(1, ncons * 32);
    stamp(p, 19, 0);
    // intermediate fragments: global (L2) -> shared memory; for quantised rows the activation sum of every
    // (item, slot), the bias every accumulator starts from, is formed on the way
    {
      const DecodeKind& K = P.kind[0];
      const uint8_t* src = p.inter_buf + K.ws_off;
      uint8_t* dst = smem + K.frag_off;
      if (K.groups) {
        float* gsum = reinterpret_cast<float*>(smem + K.gsum_off);
        const int total = K.ips * K.ng * 4;
        for (int base = 0; base < total; base += ncons * 32) {
          const int idx = base + tid;
          float sum = 0.f;
          if (idx < total) {
            const int tt = idx & 3, vs = (idx >> 2) & (K.ng - 1), item = idx / (4 * K.ng);
            uint4 v[4];
#pragma unroll
            for (int r = 0; r < 4; ++r)
              v[r] = __ldcg(reinterpret_cast<const uint4*>(src + ((((item * 4 + r) * K.ng + vs) * 4 + tt) << 4)));
#pragma unroll
            for (int r = 0; r < 4; ++r) {
              *reinterpret_cast<uint4*>(dst + ((((item * 4 + r) * K.ng + vs) * 4 + tt) << 4)) = v[r];
              const uint32_t w[4] = {v[r].x, v[r].y, v[r].z, v[r].w};
#pragma unroll
              for (int q = 0; q < 4; ++q)     // Q8 fragments hold x in words 0 and 2 and 16 x in words 1 and 3
                if (K.enc == ENC_Q4 || !(q & 1)) sum += __uint_as_float(w[q] << 16) + __uint_as_float(w[q] & 0xffff0000u);
            }
          }
          sum += __shfl_xor_sync(0xffffffffu, sum, 1);
          sum += __shfl_xor_sync(0xffffffffu, sum, 2);
          if (idx < total && (idx & 3) == 0) gsum[idx >> 2] = sum;
        }
      } else {
        for (int i = tid; i < (K.frag_bytes >> 4); i += ncons * 32)
          reinterpret_cast<uint4*>(dst)[i] = __ldcg(reinterpret_cast<const uint4*>(src) + i);
      }
      if (S) {
        const uint4* s2 = reinterpret_cast<const uint4*>(p.inter_buf + P.kind[1].ws_off);
        uint4* d2 = reinterpret_cast<uint4*>(smem + P.kind[1].frag_off);
        for (int i = tid; i < (P.kind[1].frag_bytes >> 4); i += ncons * 32) d2[i] = __ldcg(s2 + i);
      }
    }
    named_bar_sync(1, ncons * 32);
    stamp(p, 21, 0);

    const uint32_t smem_base = smem_u32(smem);
    Ring ring{0, 0, 0};
    float* red = reinterpret_cast<float*>(smem + P.red_off);
    const bool skip = (p.debug & 1) != 0;
    if (!s_fail && fast) {
      if (P.kind[0].enc == ENC_Q4) down_resident<ENC_Q4>(P, P.kind[0], npairs, smem_base, full, red, fail, warp, lane, skip, sreg);
      else down_resident<ENC_Q8>(P, P.kind[0], npairs, smem_base, full, red, fail, warp, lane, skip, sreg);
    } else if (!s_fail) {
      if (P.kind[0].enc == ENC_Q4) down_pairs<ENC_Q4>(P, P.kind[0], npairs, smem_base, full, empty, red, ring, fail, warp, lane, skip, ncons);
      else if (P.kind[0].enc == ENC_Q8) down_pairs<ENC_Q8>(P, P.kind[0], npairs, smem_base, full, empty, red, ring, fail, warp, lane, skip, ncons);
      else down_pairs<ENC_BF16>(P, P.kind[0], npairs, smem_base, full, empty, red, ring, fail, warp, lane, skip, ncons);
      if (S) down_pairs<ENC_BF16>(P, P.kind[1], npairs, smem_base, full, empty, reinterpret_cast<float*>(smem + P.red2_off), ring, fail, warp, lane, skip, ncons);
    }
    stamp(p, 22, 0);
  }
  __syncthreads();
  stamp(p, 23, 0);
  if (!s_fail) {
    // ---- sums over the warps, then the ordered combine: ascending expert, BF16 rounding of every
    //      contribution and partial sum.  Thread ul*16 + 2*slot + row holds the (row pair, slot, row) sum; the
    //      16 lanes of a row pair exchange them by shuffle, lanes 0 and 1 of the group write the two rows. -----
    for (int base = 0; base < npairs * 16; base += kThreadsD) {
      const int idx = base + tid;
      const bool live = idx < npairs * 16;
      const int e = idx & 15, ul = idx >> 4, row = e & 1;
      float y = 0.f, y2 = 0.f;
      if (live) {
        const float* r = reinterpret_cast<const float*>(smem + P.red_off) + (size_t)ul * kNW * 16 + e;
        for (int w = 0; w < ncons; ++w) y += r[w * 16];
        if (S) {
          const float* r2 = reinterpret_cast<const float*>(smem + P.red2_off) + (size_t)ul * kNW * 16 + e;
          for (int w = 0; w < ncons; ++w) y2 += r2[w * 16];
        }
      }
      const int group0 = lane & 16;              // first lane of this row pair's 16 lanes
      float run = 0.f;
      for (int r = 0; r < s_present; ++r) {
        const int slot = s_order[r];
        const float v = __shfl_sync(0xffffffffu, y, group0 + 2 * slot + row);
        run = bf16_round(run + bf16_round(v * s_weight[slot]));
      }
      if (S) {
        float ys = 0.f;
        for (int seg = 0; seg < P.kind[1].nvs; ++seg) ys += __shfl_sync(0xffffffffu, y2, group0 + 2 * seg + row);
        run = bf16_round(run + bf16_round(s_gate * bf16_round(ys)));
      }
      if (live && e < 2) p.out[2 * (rp0 + ul) + row] = __float2bfloat16_rn(run);
    }
  } else if (tid == 0) {
    atomicExch(p.sync + kSyncStatus, (unsigned)ERR_DEVICE_TIMEOUT);
    __nanosleep(100000);
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

int env_int(const char* name, int fallback) {
  const char* s = std::getenv(name);
  return s ? std::atoi(s) : fallback;
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
    for (int c = std::min(K.row_bytes, 1024) / 64 * 64; c >= 64; c -= 64)
      if (K.row_bytes % c == 0) { K.ch = c; break; }
    if (!K.ch) return false;
    K.nch = K.row_bytes / K.ch;
    K.ips = K.ch / 64;
    K.mstride = 8 * K.ch + 64;             // gate block, 64 bytes, up block
    P.cost[k] = K.row_bytes;
  }
  static const int g_producers = std::max(1, std::min(kGProducers, env_int("UMAQ_DECODE_GATEUP_PRODUCERS", kGProducers)));
  P.producers = g_producers;
  P.total_cost = (long long)P.kind[0].units * P.cost[0] + (long long)P.kind[1].units * P.cost[1];
  P.grid = std::min(sms, P.kind[0].units + P.kind[1].units);
  P.bulk_scales = 1;
  // fragments: one buffer per encoding
  for (int k = 0; k < 2; ++k) {
    DecodeKind& K = P.kind[k];
    if (k == 1 && !S) break;
    if (k == 1 && P.kind[0].enc == ENC_BF16) { K.frag_off = P.kind[0].frag_off; K.gsum_off = P.kind[0].gsum_off; K.frag_bytes = P.kind[0].frag_bytes; continue; }
    K.frag_bytes = K.enc == ENC_BF16 ? H * 2 : H * 4;      // BF16 as is; quantised rows: four digit columns
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
  P.red_off = cursor; cursor += align_up(max_units * kGW * 16 * 4, 128);
  const int fixed = cursor;
  const int body = std::max(P.kind[0].mstride + 8 * P.kind[0].ch, S ? P.kind[1].mstride + 8 * P.kind[1].ch : 0);
  P.scale_off = align_up(body, 128);
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
  static const int down_cap = std::min(kDownSmemCeiling, std::max(64 * 1024, env_int("UMAQ_DECODE_DOWN_SMEM", kDownSmemMax)));
  static const int step_override = env_int("UMAQ_DECODE_DOWN_STEP", 0);
  const int H = p.hidden, I = p.inter;
  const int S = p.sh_gate ? p.shared_inter : 0;
  int cursor = 0, ws = 0;
  {
    DecodeKind& K = P.kind[0];
    describe_kind(K, p.enc, I);
    K.nvs = p.top_k;
    K.ng = pow2_at_least(std::max(2, p.top_k));
    if (K.row_bytes > 4096) return false;
    K.ips = K.row_bytes / 64;
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
    K.ips = K.row_bytes / 64;
    K.mstride = 2 * K.row_bytes + 64;
    K.frag_bytes = K.ips * K.r16 * K.ng * 64;
    K.ws_off = ws; ws += align_up(K.frag_bytes, 256);
    K.frag_off = cursor; cursor += align_up(K.frag_bytes, 128);
    K.gsum_off = cursor;
  }
  DecodeKind& K0 = P.kind[0];
  const int pairs = H / 2;
  // With a shared expert the kernel runs a ring with few consumer warps per CTA; two CTAs per SM (the second one
  // becomes resident when the gate/up CTA of that SM has left) double the warps that do the arithmetic.
  static const int ring_ctas_per_sm = std::max(1, std::min(4, env_int("UMAQ_DECODE_DOWN_CTAS_PER_SM", 2)));
  P.grid = std::min(sms * (S ? ring_ctas_per_sm : 1), pairs);
  P.max_units = (pairs + P.grid - 1) / P.grid;
  P.red_off = cursor; cursor += align_up(P.max_units * kNW * 16 * 4, 128);
  P.red2_off = cursor; if (S) cursor += align_up(P.max_units * kNW * 16 * 4, 128);
  P.ysum_off = cursor; cursor += align_up(P.max_units * 32 * 4, 128);
  const int fixed = cursor;
  // scales as bulk copies need 16-byte sizes and offsets: an even number of groups per row
  P.bulk_scales = K0.groups % 2 == 0;
  const int room = down_cap - fixed - 256;
  P.pair_step = 2;
  static const int d_producers = std::max(1, std::min(3, env_int("UMAQ_DECODE_DOWN_PRODUCERS", kDProducers)));
  P.producers = d_producers;
  // resident: the CTA's rows of every slot in one block per slot (64 bytes apart modulo 128), then the scales
  const int slot_block = P.max_units * 2 * K0.row_bytes + 64;
  const int sc_slot = P.max_units * 2 * K0.groups * 4;
  const int resident_bytes = align_up(K0.nvs * slot_block, 128) + align_up(K0.nvs * sc_slot, 128);
  if (!S && resident_bytes + 16 <= room) {
    P.resident = 1;
    P.stages = 1;
    K0.mstride = slot_block;
    P.pair_stride = 2 * K0.row_bytes;
    P.sc_base = align_up(K0.nvs * slot_block, 128);
    P.sc_pair_stride = 2 * K0.groups * 4;
    P.sc_slot_stride = sc_slot;
    P.stage_bytes = resident_bytes;
  } else {
    K0.mstride = 2 * K0.row_bytes + 64;
    const int body = std::max(K0.nvs * K0.mstride, P.kind[1].nvs * P.kind[1].mstride);
    P.scale_off = align_up(body, 16);
    P.stage_bytes = align_up(P.scale_off + K0.nvs * 2 * K0.groups * 4, 128);
    P.pair_stride = P.stage_bytes;
    P.sc_base = P.scale_off;
    P.sc_pair_stride = P.stage_bytes;
    P.sc_slot_stride = 2 * K0.groups * 4;
    const int want = P.max_units * (S ? 2 : 1);
    P.stages = std::min(want, room / (P.stage_bytes + 16));
    if (P.stages < 1 || (P.stages < 2 && want >= 2)) return false;
    // (measured on the Qwen layer with its three-stage ring: one row pair per round 44.2 us, two 41.2 us -- sharing
    // the fragments between two row pairs is worth more than the extra stage in flight)
    if (step_override == 1 || step_override == 2) P.pair_step = step_override;
  }
  const int stage_total = P.stages * P.stage_bytes;
  for (int k = 0; k < 2; ++k) { P.kind[k].frag_off += stage_total; P.kind[k].gsum_off += stage_total; }
  P.red_off += stage_total; P.red2_off += stage_total; P.ysum_off += stage_total;
  P.bar_off = stage_total + fixed;
  P.smem_bytes = P.bar_off + 2 * P.stages * 8 + 16;
  return P.smem_bytes <= down_cap;
}

bool plan_both(DecodeParams& p, int sms) {
  if (!plan_down(p, sms)) return false;
  return plan_gateup(p, sms, kPairSmemBudget - align_up(p.d.smem_bytes, 1024));
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
  p.debug = debug_from_env();
  static thread_local int configured_device = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_device != dev) {
    cudaError_t e = cudaFuncSetAttribute(decode_gateup_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBudget);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(decode_down_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDownSmemCeiling);
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
  cfg.blockDim = dim3(kThreadsG);
  cfg.dynamicSmemBytes = p.g.smem_bytes;
  cudaError_t e = cudaLaunchKernelEx(&cfg, decode_gateup_kernel, p);
  if (e != cudaSuccess) { set_error("decode: gate/up launch failed: %s", cudaGetErrorString(e)); return ERR_LAUNCH; }
  cfg.gridDim = dim3(p.d.grid);
  cfg.blockDim = dim3(kThreadsD);
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
