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
// intermediate travels between the kernels as power-of-two-prescaled fp16 (BF16 for BF16 rows).
//
// The layer is ~27 MB (OLMoE Q4) to ~105 MB (Qwen Q8 + BF16 shared expert) of weights read exactly
// once: a pure HBM stream of a few microseconds, during which nothing may serialise.  Kernel A
// (gate/up + SwiGLU) gives every 32 features of a selected expert a 256-thread CTA: four 16-row
// warp-MMA tiles (8 gate rows + 8 up rows each, all of K), two warps per tile, the activation
// fragments built once per CTA; kernel B (down + ordered combine) gives every 8 output rows a CTA
// that walks the selected experts in pairs.  Weight blocks stream through register buffers that are
// refilled as soon as they have been multiplied; no CTA waits for another.  Kernel B is launched with
// programmatic stream serialisation: its CTAs start while kernel A drains, issue their first weight
// loads, and only then wait for A's records.
//
// Dequantisation is free of per-weight arithmetic: nibbles become exact integer-valued fp16
// ((w ^ 8) & 0xF | 0x6400 = 1024 + code + 8, one LOP3 per two weights) and go straight into
// m16n8k16 warp MMAs whose B operand is the activation vector; the group scale and the constant
// bias (1032 * sum x etc.) are applied once per 128-wide group in float32.  On B200 the
// HBM-to-issue-rate ratio leaves < 3 instructions per 4-bit weight, which rules out per-weight FMA
// on the CUDA cores; the warp MMA does the multiply-add and the CUDA cores only unpack.
#include "../../include/umaq_b200.h"
#include "common.cuh"
#include "decode.cuh"

#include <algorithm>
#include <mutex>

namespace umaq {
namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kMaxSlots = 9;                    // top-k <= 8 routed + 1 shared

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- block arithmetic: 16 tile rows x one 64-byte block of each row ---------------------------------
// lane = 4*q + c supplies tile rows q and q+8.  Every block runs two accumulator chains; d[] returns
// the four accumulator elements of the lane summed over the chains: d[0], d[1] = row q, MMA columns
// 2c, 2c+1; d[2], d[3] = row q+8.
#define UMAQ_Q4_LO(w) lop3<0x6A>((w), 0x000F000Fu, 0x64086408u)   /* fp16 1024 + (code + 8)      */
#define UMAQ_Q4_HI(w) lop3<0x6A>((w), 0x00F000F0u, 0x64806480u)   /* fp16 1024 + 16 * (code + 8) */

// bytes of activation fragments per 64-byte weight block: Q4 128 k, Q8 64 k, BF16 32 k, 2 bytes each
__device__ __forceinline__ int frag_block_bytes(int enc) { return enc == ENC_Q4 ? 256 : (enc == ENC_Q8 ? 128 : 64); }

// ---- activation fragments in shared memory -------------------------------------------------------------
// fp16 fragments for Q4 rows: each run of 8 activations k0..k7 is stored as
// [k0, k4, k1/16, k5/16, k2, k6, k3/16, k7/16] (the nibble pairs one LOP3 extracts and the 1/16 that
// undoes the in-place high nibble).  Q8 and BF16 rows use natural order.  v[] = four consecutive
// activations starting at k0 (a multiple of 4), already multiplied by the prescale.
__device__ __forceinline__ void store_frag4(int enc, uint8_t* xf, int k0, const float (&v)[4]) {
  if (enc == ENC_Q4) {
    __half* o = reinterpret_cast<__half*>(xf) + (k0 & ~7) + ((k0 >> 2) & 1);
    o[0] = __float2half_rn(v[0]); o[2] = __float2half_rn(v[1] * 0.0625f);
    o[4] = __float2half_rn(v[2]); o[6] = __float2half_rn(v[3] * 0.0625f);
    return;
  }
  uint2 w;
  if (enc == ENC_BF16) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
    w.x = *reinterpret_cast<uint32_t*>(&lo);
    w.y = *reinterpret_cast<uint32_t*>(&hi);
  } else {
    __half2 lo = __floats2half2_rn(v[0], v[1]), hi = __floats2half2_rn(v[2], v[3]);
    w.x = *reinterpret_cast<uint32_t*>(&lo);
    w.y = *reinterpret_cast<uint32_t*>(&hi);
  }
  *reinterpret_cast<uint2*>(xf + (size_t)k0 * 2) = w;
}

// Bias sums of the 64-byte weight blocks of an n-activation fragment vector, read back from shared
// memory: every thread sums 32 stored halves with their coefficients, 4 (Q4) or 2 (Q8) neighbouring
// lanes combine.  Q4: run positions 0,1,4,5 hold x (coefficient 1032), 2,3,6,7 hold x/16 (72 * 16);
// Q8: every position holds x (1152).
template <int NT = kThreads>
__device__ __forceinline__ void build_bias(int enc, const uint8_t* xf, float* bias, int n, int tid) {
  const int chunks = n >> 5;
  for (int ch = tid; ch < ((chunks + 31) & ~31); ch += NT) {
    float sum = 0.f;
    if (ch < chunks) {
      const uint4* src = reinterpret_cast<const uint4*>(xf + (size_t)ch * 64);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 w = src[i];
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&w.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&w.y));
        const float2 c2 = __half22float2(*reinterpret_cast<const __half2*>(&w.z));
        const float2 d = __half22float2(*reinterpret_cast<const __half2*>(&w.w));
        if (enc == ENC_Q4) sum += (a.x + a.y + c2.x + c2.y) * 1032.f + (b.x + b.y + d.x + d.y) * (72.f * 16.f);
        else sum += (a.x + a.y + b.x + b.y + c2.x + c2.y + d.x + d.y) * 1152.f;
      }
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    if (enc == ENC_Q4) {
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      if (ch < chunks && (ch & 3) == 0) bias[ch >> 2] = sum;
    } else if (ch < chunks && (ch & 1) == 0) {
      bias[ch >> 1] = sum;
    }
  }
}

// Power of two s with amax * s in [2^13, 2^14), built from the exponent bits; 1 when amax is zero,
// tiny or not finite.  Keeps every activation inside fp16's range whatever its magnitude.
__device__ __forceinline__ float prescale_for(float amax) {
  const int eb = (__float_as_uint(amax) >> 23) & 0xff;      // amax = m * 2^(eb-126), m in [0.5, 1)
  if (eb < 32 || eb > 240) return 1.f;
  return __uint_as_float((unsigned)(267 - eb) << 23);        // 2^(14 - (eb - 126))
}

// max over the CTA; `red` has NW floats
template <int NW = kWarps>
__device__ __forceinline__ float block_max(float v, float* red, int tid) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((tid & 31) == 0) red[tid >> 5] = v;
  __syncthreads();
  float m = red[0];
#pragma unroll
  for (int i = 1; i < NW; ++i) m = fmaxf(m, red[i]);
  __syncthreads();
  return m;
}

__device__ __forceinline__ long long load_index(const void* idx, int idx64, int i) {
  return idx64 ? reinterpret_cast<const long long*>(idx)[i] : (long long)reinterpret_cast<const int*>(idx)[i];
}

// Four blocks at once: eight accumulator chains issued round-robin, so no MMA waits for the one
// before it (a dependent warp MMA on this architecture takes ~130 cycles to issue).  n = valid blocks;
// d[i] as in mma_block().
// XG: the fragments are in global memory and were written by the preceding kernel of the chain:
// they are read through L2 (ld.global.cg), never through a cache that may predate that kernel.
template <bool XG>
__device__ __forceinline__ uint4 load_frag(const uint8_t* p) {
  return XG ? __ldcg(reinterpret_cast<const uint4*>(p)) : *reinterpret_cast<const uint4*>(p);
}
template <bool XG, int N = 4>
__device__ __forceinline__ void mma_blocks4(int enc, int n, const uint4 (&ra)[N], const uint4 (&rb)[N],
                                            const uint8_t* const (&xf_lane)[N], bool xvalid, float (&d)[N][4]) {
  float d0[N][4], d1[N][4];
#pragma unroll
  for (int i = 0; i < N; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) d0[i][e] = d1[i][e] = 0.f;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  if (enc == ENC_Q4) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int i = 0; i < N; ++i) {
        if (i < n) {
          const uint4 x = xvalid ? load_frag<XG>(xf_lane[i] + 16 * j) : zero;
          const uint32_t a = j == 0 ? ra[i].x : j == 1 ? ra[i].y : j == 2 ? ra[i].z : ra[i].w;
          const uint32_t b = j == 0 ? rb[i].x : j == 1 ? rb[i].y : j == 2 ? rb[i].z : rb[i].w;
          const uint32_t ah = a >> 8, bh = b >> 8;
          mma_f16_16816(d0[i], UMAQ_Q4_LO(a), UMAQ_Q4_LO(b), UMAQ_Q4_HI(a), UMAQ_Q4_HI(b), x.x, x.y);
          mma_f16_16816(d1[i], UMAQ_Q4_LO(ah), UMAQ_Q4_LO(bh), UMAQ_Q4_HI(ah), UMAQ_Q4_HI(bh), x.z, x.w);
        }
      }
    }
  } else if (enc == ENC_Q8) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
      for (int i = 0; i < N; ++i) {
        if (i < n) {
          const uint4 x = xvalid ? load_frag<XG>(xf_lane[i] + 16 * j) : zero;
          const uint32_t a0 = (j == 0 ? ra[i].x : ra[i].z) ^ 0x80808080u, a1 = (j == 0 ? ra[i].y : ra[i].w) ^ 0x80808080u;
          const uint32_t b0 = (j == 0 ? rb[i].x : rb[i].z) ^ 0x80808080u, b1 = (j == 0 ? rb[i].y : rb[i].w) ^ 0x80808080u;
          mma_f16_16816(d0[i], prmt(a0, 0x64646464u, 0x4140), prmt(b0, 0x64646464u, 0x4140),
                        prmt(a0, 0x64646464u, 0x4342), prmt(b0, 0x64646464u, 0x4342), x.x, x.y);
          mma_f16_16816(d1[i], prmt(a1, 0x64646464u, 0x4140), prmt(b1, 0x64646464u, 0x4140),
                        prmt(a1, 0x64646464u, 0x4342), prmt(b1, 0x64646464u, 0x4342), x.z, x.w);
        }
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) {
      if (i < n) {
        const uint4 x = xvalid ? load_frag<XG>(xf_lane[i]) : zero;
        mma_bf16_16816(d0[i], ra[i].x, rb[i].x, ra[i].y, rb[i].y, x.x, x.y);
        mma_bf16_16816(d1[i], ra[i].z, rb[i].z, ra[i].w, rb[i].w, x.z, x.w);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < N; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) d[i][e] = d0[i][e] + d1[i][e];
}

// The same for N complete blocks with the encoding fixed at compile time: no per-block predicates, so the
// compiler emits straight-line LOP3 / HMMA code without convergence barriers around every warp MMA.
// Two accumulator elements are returned: lo[i] = tile row q, MMA column 2c; hi[i] = tile row q + 8, column 2c
// (HI = 2) or 2c + 1 (HI = 3).
template <int ENC, int N, int HI = 2>
__device__ __forceinline__ void mma_full(const uint4 (&ra)[N], const uint4 (&rb)[N], const uint8_t* const (&xf_lane)[N],
                                         float (&lo)[N], float (&hi)[N]) {
  float d0[N][4], d1[N][4];
#pragma unroll
  for (int i = 0; i < N; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) d0[i][e] = d1[i][e] = 0.f;
  if (ENC == ENC_Q4) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int i = 0; i < N; ++i) {
        const uint4 x = *reinterpret_cast<const uint4*>(xf_lane[i] + 16 * j);
        const uint32_t a = j == 0 ? ra[i].x : j == 1 ? ra[i].y : j == 2 ? ra[i].z : ra[i].w;
        const uint32_t b = j == 0 ? rb[i].x : j == 1 ? rb[i].y : j == 2 ? rb[i].z : rb[i].w;
        const uint32_t ah = a >> 8, bh = b >> 8;
        mma_f16_16816(d0[i], UMAQ_Q4_LO(a), UMAQ_Q4_LO(b), UMAQ_Q4_HI(a), UMAQ_Q4_HI(b), x.x, x.y);
        mma_f16_16816(d1[i], UMAQ_Q4_LO(ah), UMAQ_Q4_LO(bh), UMAQ_Q4_HI(ah), UMAQ_Q4_HI(bh), x.z, x.w);
      }
    }
  } else if (ENC == ENC_Q8) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
      for (int i = 0; i < N; ++i) {
        const uint4 x = *reinterpret_cast<const uint4*>(xf_lane[i] + 16 * j);
        const uint32_t a0 = (j == 0 ? ra[i].x : ra[i].z) ^ 0x80808080u, a1 = (j == 0 ? ra[i].y : ra[i].w) ^ 0x80808080u;
        const uint32_t b0 = (j == 0 ? rb[i].x : rb[i].z) ^ 0x80808080u, b1 = (j == 0 ? rb[i].y : rb[i].w) ^ 0x80808080u;
        mma_f16_16816(d0[i], prmt(a0, 0x64646464u, 0x4140), prmt(b0, 0x64646464u, 0x4140),
                      prmt(a0, 0x64646464u, 0x4342), prmt(b0, 0x64646464u, 0x4342), x.x, x.y);
        mma_f16_16816(d1[i], prmt(a1, 0x64646464u, 0x4140), prmt(b1, 0x64646464u, 0x4140),
                      prmt(a1, 0x64646464u, 0x4342), prmt(b1, 0x64646464u, 0x4342), x.z, x.w);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) {
      const uint4 x = *reinterpret_cast<const uint4*>(xf_lane[i]);
      mma_bf16_16816(d0[i], ra[i].x, rb[i].x, ra[i].y, rb[i].y, x.x, x.y);
      mma_bf16_16816(d1[i], ra[i].z, rb[i].z, ra[i].w, rb[i].w, x.z, x.w);
    }
  }
#pragma unroll
  for (int i = 0; i < N; ++i) { lo[i] = d0[i][0] + d1[i][0]; hi[i] = d0[i][HI] + d1[i][HI]; }
}

// ---- activation fragments ------------------------------------------------------------------------------------
// Shared memory the gate/up kernel needs for an n-long activation vector: n fp16 fragments (2n bytes) and the
// bias sums of its 64-byte weight blocks (n/64 floats, padded to a multiple of four).
__host__ __device__ __forceinline__ int frag_body_bytes(int n) { return n * 2 + (((n >> 6) + 3) & ~3) * 4; }
// The record the gate/up kernel leaves for quantised down rows: n fp16 fragments in 32-value chunks, each chunk
// multiplied by its own power-of-two prescale, then the n/32 prescales and the n/32 chunk bias sums (float32).
__host__ __device__ __forceinline__ int chunk_record_bytes(int n) { return n * 2 + (n >> 5) * 8; }

// =====================================================================================================
// Kernel A: one CTA = 32 features of one slot = four 16-row tiles (rows 0..7 gate rows, 8..15 up rows
// of 8 features), all of K = H.  Two warps split the 64-byte blocks of a tile's rows; SwiGLU after the
// cross-warp sum.  The activation fragments are built once per CTA and serve all four tiles (building
// them costs about as many instructions as one tile's arithmetic, so a CTA per tile spent three
// quarters of its instructions there).  Weight blocks stream through two register buffers of two
// blocks each: the loads of group g + 2 are issued as soon as group g has been multiplied.  Every CTA
// writes its 32 intermediates into the slot's record itself (chunk_record_bytes below).
// =====================================================================================================
constexpr int kWarpsA = 8, kThreadsA = kWarpsA * 32, kTilesA = 4, kSplitA = kWarpsA / kTilesA;

struct BlockPair {
  uint4 wa[2], wb[2];
  float sa[2], sb[2];
};

__global__ void __launch_bounds__(kThreadsA, 2) decode_gateup_kernel(const DecodeParams p) {
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ float red[kWarpsA * 16];
  __shared__ float red2[kWarpsA];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, q = lane >> 2, c = lane & 3;
  const int H = p.hidden;
  pdl_launch_dependents();

  constexpr int kFeat = 8 * kTilesA;                           // features per CTA
  const int ctas_r = (p.inter + kFeat - 1) / kFeat, routed = p.top_k * ctas_r;
  const bool shared_tile = (int)blockIdx.x >= routed;
  const int slot = shared_tile ? p.top_k : (int)blockIdx.x / ctas_r;
  const int islot = shared_tile ? p.shared_inter : p.inter;
  const int f0 = (shared_tile ? (int)blockIdx.x - routed : (int)blockIdx.x % ctas_r) * kFeat;
  const int tile = warp / kSplitA, ws = warp % kSplitA;       // this warp: tile `tile`, blocks ws, ws + kSplitA, ...
  const int ft = f0 + 8 * tile;                                // first feature of the warp's tile
  const bool live = ft < islot;                                // the last CTA of a slot may have fewer tiles
  const int enc = shared_tile ? ENC_BF16 : p.enc;
  const int rb = row_bytes(enc, H), nblk = rb >> 6, gk = H >> 7;
  const uint8_t *gate = nullptr, *up = nullptr;
  const float *gate_s = nullptr, *up_s = nullptr;
  if (shared_tile) {
    gate = reinterpret_cast<const uint8_t*>(p.sh_gate) + (size_t)ft * rb;
    up = reinterpret_cast<const uint8_t*>(p.sh_up) + (size_t)ft * rb;
  } else {
    long long e = load_index(p.idx, p.idx64, slot);
    if (e < 0 || e >= p.experts) {
      if (tid == 0) atomicExch(p.sync + 2, (unsigned)ERR_BAD_ARGUMENT);
      return;
    }
    const size_t row = (size_t)e * p.inter + ft;
    gate = p.gate + row * rb; up = p.up + row * rb;
    if (enc != ENC_BF16) { gate_s = p.gate_s + row * gk; up_s = p.up_s + row * gk; }
  }

  const int bpw = live ? (nblk - ws + kSplitA - 1) / kSplitA : 0;
  auto issue = [&](BlockPair& b, int first) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int kb = ws + (first + i) * kSplitA;
      if (first + i < bpw) {
        b.wa[i] = ldg_stream(gate + (size_t)q * rb + ((size_t)kb << 6) + (c << 4));
        b.wb[i] = ldg_stream(up + (size_t)q * rb + ((size_t)kb << 6) + (c << 4));
        if (enc != ENC_BF16) {
          const int g = enc == ENC_Q4 ? kb : (kb >> 1);
          b.sa[i] = gate_s[q * gk + g];
          b.sb[i] = up_s[q * gk + g];
        }
      }
    }
  };
  BlockPair b0, b1;
  issue(b0, 0);                         // weights are in flight while the activation fragments are built
  issue(b1, 2);

  // ---- x -> fragments in shared memory (quantised rows: prescaled fp16 + bias sums; BF16 rows: x as is) ---
  uint8_t* xf = smem;
  float* bias = reinterpret_cast<float*>(smem + (size_t)H * 2);
  float x_inv = 1.f;
  {
    constexpr int kMaxV = 2;                                 // hidden <= 2 * 256 * 4 in one pass
    for (int base = 0; base < H; base += kMaxV * kThreadsA * 4) {
      float vals[kMaxV][4];
      float am = 0.f;
#pragma unroll
      for (int j = 0; j < kMaxV; ++j) {
        const int k0 = base + tid * 4 + j * kThreadsA * 4;
        vals[j][0] = vals[j][1] = vals[j][2] = vals[j][3] = 0.f;
        if (k0 < H) {
          const uint2 raw = *reinterpret_cast<const uint2*>(p.x + k0);
          vals[j][0] = __uint_as_float(raw.x << 16); vals[j][1] = __uint_as_float(raw.x & 0xffff0000u);
          vals[j][2] = __uint_as_float(raw.y << 16); vals[j][3] = __uint_as_float(raw.y & 0xffff0000u);
          am = fmaxf(am, fmaxf(fmaxf(fabsf(vals[j][0]), fabsf(vals[j][1])), fmaxf(fabsf(vals[j][2]), fabsf(vals[j][3]))));
        }
      }
      float sx = 1.f;
      if (enc != ENC_BF16) {
        // hidden sizes up to 2048 are one pass, so the block maximum is the vector maximum; wider
        // vectors would need the maximum over all passes first
        sx = prescale_for(block_max<kWarpsA>(am < 3.0e38f ? am : 0.f, red2, tid));
        x_inv = 1.f / sx;
      }
#pragma unroll
      for (int j = 0; j < kMaxV; ++j) {
        const int k0 = base + tid * 4 + j * kThreadsA * 4;
        if (k0 < H) {
          const float v[4] = {vals[j][0] * sx, vals[j][1] * sx, vals[j][2] * sx, vals[j][3] * sx};
          store_frag4(enc, xf, k0, v);
        }
      }
    }
    __syncthreads();
    if (enc != ENC_BF16) { build_bias<kThreadsA>(enc, xf, bias, H, tid); __syncthreads(); }
  }
  const int fb = frag_block_bytes(enc);
  float acc_lo = 0.f, acc_hi = 0.f;
  auto multiply = [&](const BlockPair& b, int first) {
    const int n = min(2, bpw - first);
    const uint8_t* xp[2];
    float bs[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int kb = ws + (first + min(i, n - 1)) * kSplitA;
      xp[i] = xf + (size_t)kb * fb + c * (fb >> 2);
      bs[i] = enc == ENC_BF16 ? 0.f : bias[kb];
    }
    if (n == 2) {                        // complete pair: straight-line code per encoding
      float lo[2], hi[2];
      if (enc == ENC_Q4) mma_full<ENC_Q4, 2>(b.wa, b.wb, xp, lo, hi);
      else if (enc == ENC_Q8) mma_full<ENC_Q8, 2>(b.wa, b.wb, xp, lo, hi);
      else mma_full<ENC_BF16, 2>(b.wa, b.wb, xp, lo, hi);
      if (enc == ENC_BF16) { acc_lo += lo[0] + lo[1]; acc_hi += hi[0] + hi[1]; }
      else {
        acc_lo = fmaf(b.sa[0], lo[0] - bs[0], acc_lo); acc_hi = fmaf(b.sb[0], hi[0] - bs[0], acc_hi);
        acc_lo = fmaf(b.sa[1], lo[1] - bs[1], acc_lo); acc_hi = fmaf(b.sb[1], hi[1] - bs[1], acc_hi);
      }
      return;
    }
    float d[2][4];
    mma_blocks4<false, 2>(enc, n, b.wa, b.wb, xp, true, d);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      if (i < n) {
        if (enc == ENC_BF16) { acc_lo += d[i][0]; acc_hi += d[i][2]; }
        else { acc_lo = fmaf(b.sa[i], d[i][0] - bs[i], acc_lo); acc_hi = fmaf(b.sb[i], d[i][2] - bs[i], acc_hi); }
      }
    }
  };
  for (int first = 0; first < bpw; first += 4) {
    multiply(b0, first);
    if (first + 4 < bpw) issue(b0, first + 4);
    if (first + 2 < bpw) {
      multiply(b1, first + 2);
      if (first + 6 < bpw) issue(b1, first + 6);
    }
  }
  if (c == 0) { red[warp * 16 + q] = acc_lo; red[warp * 16 + 8 + q] = acc_hi; }
  __syncthreads();
  // ---- SwiGLU, then this CTA's 32 intermediates go straight into the slot's record for the down kernel ------
  // Quantised down rows: fp16 fragments of the chunk with the chunk's own power-of-two prescale, the prescale
  // and the chunk's bias sum (the down kernel brings the chunks of one weight block to a common scale).
  // BF16 down rows: the BF16 values.  No CTA waits for another one.
  const int ioff = shared_tile ? p.top_k * p.inter : slot * p.inter;
  if (warp == 0 && f0 + lane < islot) {           // islot is a multiple of 32: the whole warp or none of it
    const int t = lane >> 3, j = lane & 7;
    float g = 0.f, u = 0.f;
#pragma unroll
    for (int w = 0; w < kSplitA; ++w) { g += red[(t * kSplitA + w) * 16 + j]; u += red[(t * kSplitA + w) * 16 + 8 + j]; }
    float v;
    if (shared_tile) {                  // Qwen2MoeMLP in BF16: every linear / activation output is rounded
      g = bf16_round(g); u = bf16_round(u);
      v = bf16_round(bf16_round(silu_f32(g)) * u);
    } else {
      g *= x_inv; u *= x_inv;
      v = silu_f32(g) * u;
    }
    const int enc_b = shared_tile ? ENC_BF16 : p.enc;          // encoding of the down rows that read it
    uint8_t* recp = reinterpret_cast<uint8_t*>(p.inter_buf + ioff);
    const int k = f0 + lane;
    if (enc_b == ENC_BF16) {
      reinterpret_cast<__nv_bfloat16*>(recp)[k] = __float2bfloat16_rn(v);
    } else {
      float am = fabsf(v);
      am = am < 3.0e38f ? am : 0.f;
#pragma unroll
      for (int o = 16; o; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
      const float sc = prescale_for(am);
      const int r = k & 7;
      int pos = k;
      float val = v * sc, coef = 1152.f;
      if (enc_b == ENC_Q4) {            // run order [k0,k4,k1/16,k5/16,k2,k6,k3/16,k7/16], see store_frag4
        pos = (k & ~7) + (r < 4 ? 2 * r : 2 * (r - 4) + 1);
        if (r & 1) val *= 0.0625f; else coef = 1032.f;
      }
      const __half h = __float2half_rn(val);
      reinterpret_cast<__half*>(recp)[pos] = h;
      float bsum = coef * __half2float(h);
#pragma unroll
      for (int o = 16; o; o >>= 1) bsum += __shfl_xor_sync(0xffffffffu, bsum, o);
      if (lane == 0) {
        float* tail = reinterpret_cast<float*>(recp + (size_t)islot * 2);
        tail[k >> 5] = sc;
        tail[(islot >> 5) + (k >> 5)] = bsum;
      }
    }
  }
  (void)x_inv;
}

// =====================================================================================================
// Kernel B: one CTA = 8 output rows.  Slots are walked in ascending expert order, two per MMA tile
// (tile rows 0..7: row n0+q of the first slot, rows 8..15: the same row of the second; the slots'
// intermediate vectors are MMA columns 0 and 1).  The Qwen shared expert is a last, half-filled tile.
// A warp owns the 64-byte blocks warp, warp + 4, ... of every tile and walks (tile, pair of blocks)
// through four register buffers: their loads go out before griddepcontrol.wait, and every buffer is
// refilled as soon as it has been multiplied.
// =====================================================================================================
struct DownTile {
  const uint8_t* wa; const uint8_t* wb;        // row n0 + q of the two slots' experts (wb null: no second slot)
  const float* sa; const float* sb;            // their scale rows
  int rec_a, rec_b;                            // byte offsets of the slots' records in shared memory
  int slot_a, slot_b;
};

__global__ void __launch_bounds__(kThreads) decode_down_kernel(const DecodeParams p) {
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ int s_order[kMaxSlots];
  __shared__ int s_expert[kMaxSlots];
  __shared__ float s_weight[kMaxSlots];
  __shared__ float s_red[5][kWarps][16];
  __shared__ float s_tmp[kWarps];
  __shared__ float s_gate;
  __shared__ int s_bad;
  __shared__ __align__(16) uint8_t s_zero[256];         // fragment block of the lanes that feed no MMA column
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, q = lane >> 2, c = lane & 3;
  const int H = p.hidden, I = p.inter, S = p.sh_gate ? p.shared_inter : 0;
  const int n0 = blockIdx.x * 8;
  // shared memory: the published records of the routed slots (fragments + bias), then the shared
  // expert's BF16 vector
  const int enc = p.enc;
  const int rec = enc == ENC_BF16 ? I * 2 : chunk_record_bytes(I);     // bytes copied per routed slot
  uint8_t* recs = smem;
  uint8_t* xs = smem + (size_t)p.top_k * rec;
  // per (slot, 64-byte weight block): bias sum and inverse of the common prescale of the block's chunks
  const int nblk_all = row_bytes(enc, I) >> 6;
  float* s_bbias = reinterpret_cast<float*>(xs + (size_t)(p.sh_gate ? p.shared_inter : 0) * 2);
  float* s_binv = s_bbias + (size_t)p.top_k * nblk_all;

  // ---- routes: order by expert (stable), shared expert last ----------------------------------------------
  if (tid == 0) s_bad = 0;
  if (tid < 64) reinterpret_cast<uint32_t*>(s_zero)[tid] = 0u;
  __syncthreads();
  if (tid < p.top_k) {
    const long long e = load_index(p.idx, p.idx64, tid);
    if (e < 0 || e >= p.experts) s_bad = 1;
    s_expert[tid] = (int)e;
    s_weight[tid] = p.w[tid];
  }
  __syncthreads();
  if (s_bad) {
    if (tid == 0) atomicExch(p.sync + 2, (unsigned)ERR_BAD_ARGUMENT);
    return;
  }
  if (tid < p.top_k) {
    int rank = 0;
    for (int j = 0; j < p.top_k; ++j) rank += (s_expert[j] < s_expert[tid]) || (s_expert[j] == s_expert[tid] && j < tid);
    s_order[rank] = tid;
  }
  __syncthreads();

  const int rb = row_bytes(enc, I), nblk = rb >> 6, gk = I >> 7;
  const int rtiles = (p.top_k + 1) >> 1;
  const int bpw = (nblk - warp + kWarps - 1) / kWarps;           // blocks of a routed tile this warp owns
  const int ppw = (bpw + 1) >> 1;                                // pairs of blocks per tile
  const int npairs = rtiles * ppw;
  const int fb = frag_block_bytes(enc);
  auto tile_of = [&](int t) {
    DownTile d;
    const int a = s_order[2 * t], b = 2 * t + 1 < p.top_k ? s_order[2 * t + 1] : -1;
    const size_t ra = (size_t)s_expert[a] * H + n0 + q;
    d.wa = p.down + ra * rb + (c << 4);
    d.sa = enc != ENC_BF16 ? p.down_s + ra * gk : nullptr;
    d.rec_a = a * rec; d.slot_a = a;
    if (b >= 0) {
      const size_t rbw = (size_t)s_expert[b] * H + n0 + q;
      d.wb = p.down + rbw * rb + (c << 4);
      d.sb = enc != ENC_BF16 ? p.down_s + rbw * gk : nullptr;
      d.rec_b = b * rec; d.slot_b = b;
    } else { d.wb = nullptr; d.sb = nullptr; d.rec_b = d.rec_a; d.slot_b = a; }
    return d;
  };
  // (tile, first block of the pair) walked in order; one iterator for the loads, one for the arithmetic
  struct Walk { int t, first, left; };
  auto advance = [&](Walk& w) { w.first += 2; if (w.first >= bpw) { w.first = 0; ++w.t; } --w.left; };
  auto issue = [&](BlockPair& b, const Walk& w) {
    if (w.left <= 0) return;
    const DownTile d = tile_of(w.t);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      if (w.first + i < bpw) {
        const int kb = warp + (w.first + i) * kWarps;
        const int g = enc == ENC_Q4 ? kb : (kb >> 1);
        b.wa[i] = ldg_stream(d.wa + ((size_t)kb << 6));
        if (enc != ENC_BF16) b.sa[i] = d.sa[g];
        if (d.wb) {
          b.wb[i] = ldg_stream(d.wb + ((size_t)kb << 6));
          if (enc != ENC_BF16) b.sb[i] = d.sb[g];
        } else { b.wb[i] = make_uint4(0, 0, 0, 0); b.sb[i] = 0.f; }
      }
    }
  };
  float acc_lo = 0.f, acc_hi = 0.f;
  auto multiply = [&](const BlockPair& b, const Walk& w) {
    const DownTile d = tile_of(w.t);
    const int n = min(2, bpw - w.first);
    const uint8_t* xp[2];
    float bsa[2], bsb[2], iva[2], ivb[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int kb = warp + (w.first + min(i, n - 1)) * kWarps;
      // MMA column 0 <- first slot's vector (lanes of quad 0), column 1 <- second slot's (quad 1), others zero
      const uint8_t* base = q == 0 ? recs + d.rec_a : recs + d.rec_b;
      xp[i] = q < 2 ? base + (size_t)kb * fb + c * (fb >> 2) : s_zero + c * (fb >> 2);
      if (enc != ENC_BF16) {
        bsa[i] = s_bbias[d.slot_a * nblk_all + kb]; bsb[i] = s_bbias[d.slot_b * nblk_all + kb];
        iva[i] = s_binv[d.slot_a * nblk_all + kb]; ivb[i] = s_binv[d.slot_b * nblk_all + kb];
      } else { bsa[i] = bsb[i] = 0.f; iva[i] = ivb[i] = 1.f; }
    }
    float lo[2], hi[2];
    if (n == 2) {
      if (enc == ENC_Q4) mma_full<ENC_Q4, 2, 3>(b.wa, b.wb, xp, lo, hi);
      else if (enc == ENC_Q8) mma_full<ENC_Q8, 2, 3>(b.wa, b.wb, xp, lo, hi);
      else mma_full<ENC_BF16, 2, 3>(b.wa, b.wb, xp, lo, hi);
    } else {
      float dd[2][4];
      mma_blocks4<false, 2>(enc, n, b.wa, b.wb, xp, true, dd);
      lo[0] = dd[0][0]; hi[0] = dd[0][3]; lo[1] = hi[1] = 0.f;
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      if (i < n) {
        if (enc == ENC_BF16) { acc_lo += lo[i]; acc_hi += hi[i]; }
        else {
          acc_lo = fmaf(b.sa[i] * iva[i], lo[i] - bsa[i], acc_lo);
          acc_hi = fmaf(b.sb[i] * ivb[i], hi[i] - bsb[i], acc_hi);
        }
      }
    }
    if (w.first + 2 >= bpw) {              // last pair of the tile for this warp: park the partial sums
      if (c == 0) { s_red[w.t][warp][q] = acc_lo; s_red[w.t][warp][8 + q] = acc_hi; }
      acc_lo = acc_hi = 0.f;
    }
  };
  Walk wi{0, 0, npairs}, wm{0, 0, npairs};
  BlockPair b0, b1, b2, b3;
  issue(b0, wi); advance(wi);            // weights do not depend on kernel A: in flight before the wait
  issue(b1, wi); advance(wi);
  issue(b2, wi); advance(wi);
  issue(b3, wi); advance(wi);

  // sigmoid gate of the shared expert: bf16(sigmoid(bf16(x . wg)))
  if (S) {
    float acc = 0.f;
    for (int k = tid * 2; k < H; k += kThreads * 2) {
      const __nv_bfloat162 xv = *reinterpret_cast<const __nv_bfloat162*>(p.x + k);
      const __nv_bfloat162 gv = *reinterpret_cast<const __nv_bfloat162*>(p.sh_gatevec + k);
      acc += __low2float(xv) * __low2float(gv) + __high2float(xv) * __high2float(gv);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) s_tmp[warp] = acc;
    __syncthreads();
    if (tid == 0) {
      float t = 0.f;
      for (int i = 0; i < kWarps; ++i) t += s_tmp[i];
      t = bf16_round(t);
      s_gate = bf16_round(1.f / (1.f + expf(-t)));
    }
    __syncthreads();
  }

  pdl_wait();                           // kernel A's records are complete and visible from here on

  // ---- copy the records into shared memory -------------------------------------------------------------------
  // Quantised rows: first the chunk prescales and bias sums; every weight block then gets the smallest prescale
  // of its chunks (powers of two, so rescaling a chunk is exact), its bias sum and the inverse prescale; the
  // fragments are copied with their chunk's ratio applied.  BF16 rows: straight 16-byte copies.
  if (enc != ENC_BF16) {
    const int chunks = I >> 5, cpb = enc == ENC_Q4 ? 4 : 2;           // 32-value chunks; chunks per weight block
    const int tailw = (chunks * 8) >> 4;                              // 16-byte words of {prescales, bias sums}
    const int fragw = (I * 2) >> 4;                                   // 16-byte words of fragments per slot
    // all loads of this thread go out together (one L2 round trip): its words of the chunk tables and its
    // first kHold fragment words, which wait in registers until the ratios are known
    constexpr int kHold = 8;
    uint4 held[kHold];
#pragma unroll
    for (int j = 0; j < kHold; ++j) {
      const int w = tid + j * kThreads;                               // word index over all slots
      if (w < p.top_k * fragw) {
        const int s = w / fragw, i = w - s * fragw;
        held[j] = __ldcg(reinterpret_cast<const uint4*>(p.inter_buf + (size_t)s * I) + i);
      }
    }
    for (int w = tid; w < p.top_k * tailw; w += kThreads) {
      const int s = w / tailw, i = w - s * tailw;
      const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(p.inter_buf + (size_t)s * I) + (size_t)I * 2);
      reinterpret_cast<uint4*>(recs + (size_t)s * rec + (size_t)I * 2)[i] = __ldcg(src + i);
    }
    __syncthreads();
    for (int it = tid; it < p.top_k * nblk_all; it += kThreads) {
      const int s = it / nblk_all, kb = it - s * nblk_all;
      float* sc = reinterpret_cast<float*>(recs + (size_t)s * rec + (size_t)I * 2);
      const float* cb = sc + chunks;
      float m = sc[kb * cpb];
      for (int c2 = 1; c2 < cpb; ++c2) m = fminf(m, sc[kb * cpb + c2]);
      float bsum = 0.f;
      for (int c2 = 0; c2 < cpb; ++c2) {
        const float ratio = m / sc[kb * cpb + c2];                    // a power of two <= 1
        bsum += cb[kb * cpb + c2] * ratio;
        sc[kb * cpb + c2] = ratio;                                    // the fragment copy below reads the ratio
      }
      s_bbias[it] = bsum;
      s_binv[it] = 1.f / m;
    }
    __syncthreads();
    auto scaled_store = [&](uint4 w, int s, int i) {
      const float* ratio = reinterpret_cast<const float*>(recs + (size_t)s * rec + (size_t)I * 2);
      const __half2 r2 = __float2half2_rn(ratio[i >> 2]);             // 8 values per word, 32 per chunk
      __half2* h = reinterpret_cast<__half2*>(&w);
      h[0] = __hmul2(h[0], r2); h[1] = __hmul2(h[1], r2); h[2] = __hmul2(h[2], r2); h[3] = __hmul2(h[3], r2);
      reinterpret_cast<uint4*>(recs + (size_t)s * rec)[i] = w;
    };
#pragma unroll
    for (int j = 0; j < kHold; ++j) {
      const int w = tid + j * kThreads;
      if (w < p.top_k * fragw) { const int s = w / fragw; scaled_store(held[j], s, w - s * fragw); }
    }
    for (int w = tid + kHold * kThreads; w < p.top_k * fragw; w += kThreads) {     // shapes with more words
      const int s = w / fragw, i = w - s * fragw;
      scaled_store(__ldcg(reinterpret_cast<const uint4*>(p.inter_buf + (size_t)s * I) + i), s, i);
    }
  } else {
    for (int s = 0; s < p.top_k; ++s) {
      const uint4* src = reinterpret_cast<const uint4*>(p.inter_buf + (size_t)s * I);
      uint4* dst = reinterpret_cast<uint4*>(recs + (size_t)s * rec);
      for (int i = tid; i < (rec >> 4); i += kThreads) dst[i] = __ldcg(src + i);
    }
  }
  if (S) {
    const uint4* src = reinterpret_cast<const uint4*>(p.inter_buf + (size_t)p.top_k * I);
    uint4* dst = reinterpret_cast<uint4*>(xs);
    for (int i = tid; i < (S * 2) >> 4; i += kThreads) dst[i] = __ldcg(src + i);
  }
  __syncthreads();

  // ---- routed tiles: pairs of blocks through the four buffers, four MMA chains per pair ---------------------
  while (wm.left > 0) {
    multiply(b0, wm); advance(wm); issue(b0, wi); advance(wi);
    if (wm.left > 0) { multiply(b1, wm); advance(wm); issue(b1, wi); advance(wi); }
    if (wm.left > 0) { multiply(b2, wm); advance(wm); issue(b2, wi); advance(wi); }
    if (wm.left > 0) { multiply(b3, wm); advance(wm); issue(b3, wi); advance(wi); }
  }
  if (bpw == 0 && c == 0)
    for (int t = 0; t < rtiles; ++t) { s_red[t][warp][q] = 0.f; s_red[t][warp][8 + q] = 0.f; }

  // ---- shared expert: one half-filled BF16 tile, K = S, blocks split over the warps in groups of four ------
  if (S) {
    const int rbs = 2 * S, nb = rbs >> 6;
    const uint8_t* rowp = reinterpret_cast<const uint8_t*>(p.sh_down) + (size_t)(n0 + q) * rbs;
    const uint4 zero4[4] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
    float acc = 0.f;
    for (int first = warp; first < nb; first += kWarps * 4) {
      uint4 w[4];
      const uint8_t* xp[4];
      int n = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int kb = first + i * kWarps;
        if (kb < nb) { w[i] = ldg_stream(rowp + ((size_t)kb << 6) + (c << 4)); n = i + 1; }
        else w[i] = make_uint4(0, 0, 0, 0);
        xp[i] = xs + (size_t)min(kb, nb - 1) * 64 + c * 16;
      }
      float d[4][4];
      mma_blocks4<false>(ENC_BF16, n, w, zero4, xp, true, d);
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (i < n) acc += d[i][0];
    }
    if (c == 0) { s_red[4][warp][q] = acc; s_red[4][warp][8 + q] = 0.f; }
  }
  __syncthreads();

  // ---- ordered combine: ascending expert, BF16 rounding of every contribution and partial sum --------------
  if (tid < 8 && n0 + tid < H) {
    float run = 0.f;
    for (int r = 0; r < p.top_k; ++r) {
      const int t = r >> 1, half = r & 1, slot = s_order[r];
      float y = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) y += s_red[t][w][half * 8 + tid];
      run = bf16_round(run + bf16_round(y * s_weight[slot]));
    }
    if (S) {
      float y = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) y += s_red[4][w][tid];
      run = bf16_round(run + bf16_round(s_gate * bf16_round(y)));
    }
    p.out[n0 + tid] = __float2bfloat16_rn(run);
  }
}

size_t gateup_smem(const DecodeParams& p) {
  return (size_t)frag_body_bytes(p.hidden) + 64;                 // x fragments and their bias sums
}
size_t down_smem(const DecodeParams& p) {
  const size_t rec = p.enc == ENC_BF16 ? (size_t)p.inter * 2 : (size_t)chunk_record_bytes(p.inter);
  const size_t blocks = (size_t)p.top_k * (row_bytes(p.enc, p.inter) >> 6);
  return (size_t)p.top_k * rec + (p.sh_gate ? (size_t)p.shared_inter * 2 : 0) + blocks * 8 + 64;
}

}  // namespace

size_t decode_workspace_bytes(int top_k, int inter, int shared_inter) {
  return kDecodeWsHeader + ((size_t)top_k * inter + shared_inter) * sizeof(float);
}

int launch_moe_decode(DecodeParams p, cudaStream_t stream) {
  if (p.top_k < 1 || p.top_k > 8 || p.hidden % 512 || p.inter % 128 || p.hidden < 512 || p.inter < 128 ||
      p.hidden > 2048 || p.inter > 6144 || (p.sh_gate && (p.shared_inter % 128 || p.shared_inter < 128 || p.shared_inter > 6144)) ||
      p.enc < 0 || p.enc > 2) {
    set_error("decode: unsupported shape (hidden %d, intermediate %d, top_k %d, shared %d, encoding %d)", p.hidden,
              p.inter, p.top_k, p.shared_inter, p.enc);
    return ERR_BAD_ARGUMENT;
  }
  if (p.enc != ENC_BF16 && (!p.gate_s || !p.up_s || !p.down_s)) {
    set_error("decode: quantised layer without scales");
    return ERR_BAD_ARGUMENT;
  }
  const size_t smem_a = gateup_smem(p), smem_b = down_smem(p);
  static thread_local int configured_device = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_device != dev) {
    cudaError_t e = cudaFuncSetAttribute(decode_down_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
    if (e != cudaSuccess) { set_error("decode: cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return ERR_LAUNCH; }
    configured_device = dev;
  }
  if (smem_b > 100 * 1024 || smem_a > 48 * 1024) {
    set_error("decode: shape needs more shared memory than planned");
    return ERR_UNSUPPORTED;
  }
  cudaLaunchConfig_t cfg{};
  cfg.blockDim = dim3(kThreadsA);
  cfg.stream = stream;
  constexpr int kFeat = 8 * kTilesA;
  cfg.gridDim = dim3(p.top_k * ((p.inter + kFeat - 1) / kFeat) + (p.sh_gate ? (p.shared_inter + kFeat - 1) / kFeat : 0));
  cfg.dynamicSmemBytes = smem_a;
  cudaError_t e = cudaLaunchKernelEx(&cfg, decode_gateup_kernel, p);
  if (e != cudaSuccess) { set_error("decode: gate/up launch failed: %s", cudaGetErrorString(e)); return ERR_LAUNCH; }
  // The down kernel is chained by programmatic stream serialisation: its CTAs may start while the
  // gate/up kernel drains, issue their weight loads, and wait on-device before reading its records.
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cfg.blockDim = dim3(kThreads);
  cfg.gridDim = dim3((p.hidden + 7) / 8);
  cfg.dynamicSmemBytes = smem_b;
  e = cudaLaunchKernelEx(&cfg, decode_down_kernel, p);
  if (e != cudaSuccess) { set_error("decode: down launch failed: %s", cudaGetErrorString(e)); return ERR_LAUNCH; }
  return ERR_NONE;
}

}  // namespace umaq

// ---- decode without a caller-provided workspace ---------------------------------------------------
// Scratch of the entry point below: one fixed block per device that loads this library, held until
// the process exits.  It has the layout of the decode workspace (control words, diagnostics, float32
// intermediate) and therefore bounds the shapes the entry point accepts.
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
    set_error("umaq_moe_decode_static: top_k * intermediate + shared intermediate = %lld float32 values need %zu bytes "
              "of scratch, the built-in block holds %zu; use umaq_moe_decode with a caller workspace",
              (long long)top_k * layer->intermediate + s_inter, need, kStaticScratchBytes);
    return ERR_WORKSPACE;
  }
  void* scratch = nullptr;
  const int rc = static_scratch_for_current_device(&scratch);
  if (rc != ERR_NONE) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The block keeps whatever the previous call left.  The control words (status, barrier counter)
  // must start from zero; the intermediate area is fully rewritten before it is read.
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
  p.inter_buf = reinterpret_cast<float*>(ws + kDecodeWsHeader);
  return launch_moe_decode(p, st);
}
