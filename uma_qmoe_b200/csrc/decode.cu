// Batch-1 decode: one persistent cooperative kernel per MoE layer call.
//
//   out = sum_slot w_slot * Down_e( SiLU(Gate_e x) * Up_e x )   (+ Qwen shared expert)
//
// replaces the reference's two-launch decode
// (src/uma_qmoe/native/packed_q4_kernel.cu:156-231 gate/up+SwiGLU, :1369-1426 down+route sum,
// launched from :1486-1533; Q8 twins :781-892) and the per-expert Python GEMV loops for Qwen
// (src/uma_qmoe/native_backend.py:319-372, :722-753).  Numerics follow the reference's CPU
// correctness path (src/uma_qmoe/custom_op.py:301-340, :465-506): float32 intermediate, one BF16
// rounding of every expert contribution and of the running sum, experts in ascending order.
//
// Shape of the work.  The layer is ~27 MB (OLMoE Q4) to ~105 MB (Qwen Q8 + BF16 shared expert) of
// weights read exactly once, i.e. a pure HBM stream of a few microseconds.  One CTA per SM; every
// CTA owns a byte-balanced, contiguous range of gate/up feature rows (phase A) and of output rows
// (phase B).  A producer warp streams the CTA's rows with untiled bulk async copies into a ring of
// shared-memory stages guarded by mbarriers; it never waits for the phase boundary, so the down
// projection rows are already in flight or resident while phase A computes.  Eight consumer warps
// dequantise 64-byte row blocks in registers into exact integer-valued fp16
// (nibble | 0x6400 = 1024 + code, no per-weight arithmetic) and feed m16n8k16 warp MMAs whose B
// operand is the activation vector; the group scale and the constant code bias are applied once
// per 128-wide group in float32.  On B200 the HBM-to-issue-rate ratio leaves < 3 instructions per
// 4-bit weight, which rules out per-weight FMA on the CUDA cores; the warp MMA does the multiply-add
// and the CUDA cores only unpack.  The two phases are separated by one bounded grid barrier.
//
// Latency discipline: a CTA runs each path once, so everything on the critical path is kept to a
// handful of instructions: the stage list is computed once, in parallel, into shared memory; the
// routes are fetched with one round of loads; partial sums are parked and reduced once per phase.
#include "../../include/umaq_b200.h"
#include "common.cuh"
#include "decode.cuh"

#include <mutex>

#include <algorithm>

namespace umaq {
namespace {

constexpr int kGroupWarps = 8;                  // warps that split the K blocks of one stage
constexpr int kConsumerWarps = 16;              // two groups: consecutive tiles go to alternate groups
constexpr int kConsumers = kConsumerWarps * 32;
constexpr int kThreads = kConsumers + 32;       // + one producer warp
constexpr int kMaxSlots = 9;                    // top-k <= 8 routed + 1 shared
constexpr int kScaleArea = 1152;                // bytes of scale staging per ring stage
constexpr int kMaxRing = 16;                    // ring stages
constexpr int kMaxList = 128;                   // stages one CTA may have to process
constexpr int kRedTiles = 24;                   // tiles parked before a cross-warp reduction
constexpr int kMaxUnitsX = 32;                  // hidden size <= 32 * 128
constexpr int kMaxUnitsB = 96;                  // sum of intermediate sizes <= 96 * 128

struct Slot {
  const uint8_t* gate;
  const uint8_t* up;
  const uint8_t* down;
  const float* gate_s;
  const float* up_s;
  const float* down_s;
  float weight;
  int expert;         // sort key (shared expert: INT_MAX)
  int bad;            // expert index out of range
};

// One ring stage: 16 tile rows x nkb 64-byte blocks.
//  kind 0: features [r0, r0+nr) of a slot: gate rows in tile rows 0..7, up rows in 8..15 (nr <= 8)
//  kind 1: output rows [r0, r0+nr) of a slot's down projection (nr <= 16)
struct alignas(16) Stage {
  int flags;     // bit0 kind, bit1 last slice of its tile, bit2 owned by one warp pair, bit3 warp group,
                 // bits 4-7 slot position (phase A: slot; phase B: index into order[]), bits 8-12 nr,
                 // bits 16-19 owner pair (warps 2*owner and 2*owner+1)
  int r0;
  int kb0;       // first 64-byte block of the row covered by this stage
  int nkb;       // blocks covered
  __device__ int kind() const { return flags & 1; }
  __device__ int last() const { return (flags >> 1) & 1; }
  __device__ int owned() const { return (flags >> 2) & 1; }
  __device__ int group() const { return (flags >> 3) & 1; }
  __device__ int pos() const { return (flags >> 4) & 15; }
  __device__ int nr() const { return (flags >> 8) & 31; }
  __device__ int owner() const { return (flags >> 16) & 15; }
};

struct Shared {
  Slot slots[kMaxSlots];
  int order[kMaxSlots];        // phase-B slot order: ascending expert, shared last
  int nlist;                   // stages in list[]
  int first_b;                 // index of the first phase-B stage (== nlist if none)
  int abort_flag;
  float scale_x_inv;           // undoes the power-of-two prescale of x
  float scaleB;                // prescale of the quantised slots' intermediate vectors, and its inverse
  float scaleB_inv;
  float contrib[kMaxSlots][16];
  float sig_gate;              // bf16(sigmoid(bf16(x . wg)))
  float wred[kConsumerWarps];
  float wred2[kConsumerWarps];
  unsigned long long bar_target;   // grid barrier: counter value that releases this launch
  unsigned amaxB;              // max |intermediate| over the quantised slots (float bits)
  float red[kRedTiles][kGroupWarps][16];      // parked partial sums: [tile][warp of the group][tile row]
  Stage tdesc[kRedTiles];
  Stage list[kMaxList];
  uint64_t full[kMaxRing];
  uint64_t empty[kMaxRing];
};

// ---- per-slot shape: depends on the launch parameters only, not on the routes --------------------
struct Shape {
  int H, top_k, enc, inter, shared_inter, nslots, max_kb;
  __device__ int enc_of(int slot) const { return slot < top_k ? enc : ENC_BF16; }
  __device__ int inter_of(int slot) const { return slot < top_k ? inter : shared_inter; }
  __device__ int inter_off(int slot) const { return slot < top_k ? slot * inter : top_k * inter; }
  __device__ int bias_off(int slot) const { return slot * ((row_bytes(enc, inter) >> 6) + 1); }
  __device__ int kbA(int slot) const { return row_bytes(enc_of(slot), H) >> 6; }               // blocks per gate/up row
  __device__ int kbB(int slot) const { return row_bytes(enc_of(slot), inter_of(slot)) >> 6; }  // per down row
  __device__ int slices(int kb) const { return (kb + max_kb - 1) / max_kb; }
};

// Builds the CTA's stage list, one lane per stage.  Phase A: the CTA's byte-balanced range of
// (slot, feature) pairs in tiles of 8 features; phase B: its range of output rows in groups of 16,
// every slot (in order[] position; position s has slot s's shape since the shared expert is last
// in both) per group.
__device__ void build_stage_list(Shared& sh, const Shape& S, int G, int cta, int lane) {
  const unsigned long long costR = 2ull * row_bytes(S.enc, S.H), costS = 4ull * S.H;
  const unsigned long long bytesR = costR * S.inter * S.top_k;
  const unsigned long long total = bytesR + (S.nslots > S.top_k ? costS * S.shared_inter : 0ull);
  auto locate = [&](unsigned long long pos, int& si, int& fi) {
    if (pos >= total) { si = S.nslots; fi = 0; return; }
    if (pos < bytesR) {
      const unsigned long long f = pos / costR;
      si = (int)(f / S.inter); fi = (int)(f % S.inter);
    } else { si = S.top_k; fi = (int)((pos - bytesR) / costS); }
  };
  int s0, f0, s1, f1;
  locate(total * (unsigned long long)cta / G, s0, f0);
  locate(total * (unsigned long long)(cta + 1) / G, s1, f1);
  int startA[kMaxSlots];       // first stage index of each slot's segment
  int totalA = 0;
#pragma unroll
  for (int s = 0; s < kMaxSlots; ++s) {
    int n = 0;
    if (s < S.nslots && s >= s0 && s <= s1) {
      const int lo = s == s0 ? f0 : 0, hi = s == s1 ? f1 : S.inter_of(s);
      if (hi > lo) n = ((hi - lo + 7) >> 3) * S.slices(S.kbA(s));
    }
    startA[s] = totalA;
    totalA += n;
  }
  const int n0 = (int)((long long)S.H * cta / G), n1 = (int)((long long)S.H * (cta + 1) / G);
  const int groups = (n1 - n0 + 15) >> 4;
  int startB[kMaxSlots];
  int perGroup = 0;
#pragma unroll
  for (int s = 0; s < kMaxSlots; ++s) {
    startB[s] = perGroup;
    if (s < S.nslots) perGroup += S.slices(S.kbB(s));
  }
  const int total_stages = totalA + groups * perGroup;
  if (lane == 0) {
    sh.nlist = total_stages;
    sh.first_b = totalA;
  }
  for (int j = lane; j < total_stages && j < kMaxList; j += 32) {
    Stage st;
    if (j < totalA) {
      int s = 0, base = 0;
#pragma unroll
      for (int t = 1; t < kMaxSlots; ++t)
        if (j >= startA[t]) { s = t; base = startA[t]; }
      const int rem = j - base;
      const int nsl = S.slices(S.kbA(s));
      const int tile = rem / nsl, slice = rem - tile * nsl;
      const int lo = s == s0 ? f0 : 0, hi = s == s1 ? f1 : S.inter_of(s);
      const int r0 = lo + tile * 8;
      const int nr = min(8, hi - r0);
      st.kb0 = slice * S.max_kb;
      st.nkb = min(S.max_kb, S.kbA(s) - st.kb0);
      const int tile_id = (base / nsl) + tile + s;      // any numbering that alternates along the list
      st.flags = 0 | ((slice == nsl - 1) << 1) | ((tile_id & 1) << 3) | (s << 4) | (nr << 8);
      st.r0 = r0;
    } else {
      const int jb = j - totalA;
      const int g = jb / perGroup, rem = jb - g * perGroup;
      int pos = 0, base = 0;
#pragma unroll
      for (int t = 1; t < kMaxSlots; ++t)
        if (t < S.nslots && rem >= startB[t]) { pos = t; base = startB[t]; }
      const int slice = rem - base;
      const int nsl = S.slices(S.kbB(pos));
      const int r0 = n0 + g * 16;
      const int nr = min(16, n1 - r0);
      st.kb0 = slice * S.max_kb;
      st.nkb = min(S.max_kb, S.kbB(pos) - st.kb0);
      // an unsliced tile is computed by one warp on its own (all slots of a group in parallel)
      const int own = nsl == 1;
      st.flags = 1 | ((slice == nsl - 1) << 1) | (own << 2) | (((g + pos) & 1) << 3) | (pos << 4) | (nr << 8) |
                 ((pos & 7) << 16);
      st.r0 = r0;
    }
    sh.list[j] = st;
  }
}

// ---- producer ------------------------------------------------------------------------------------
__device__ __forceinline__ void scale_span(int r0, int nr, int K, int& first_byte, int& bytes) {
  // contiguous rows [r0, r0+nr) x (K/128) floats, widened to 16-byte boundaries
  const int gk4 = (K >> 7) * 4;
  const int b0 = r0 * gk4, b1 = (r0 + nr) * gk4;
  first_byte = b0 & ~15;
  bytes = ((b1 + 15) & ~15) - first_byte;
}

__device__ void issue_stage(const Shared& sh, const Shape& S, const Stage& st, uint8_t* buf, uint64_t* bar, int lane) {
  const int kind = st.kind();
  const int slot = kind ? sh.order[st.pos()] : st.pos();
  const Slot& sl = sh.slots[slot];
  const int enc = S.enc_of(slot);
  const int K = kind == 0 ? S.H : S.inter_of(slot);
  const int rb = row_bytes(enc, K);
  const int sb = st.nkb << 6;
  const int nr = st.nr();
  const bool whole = (sb == rb);
  const bool has_scales = enc != ENC_BF16 && st.kb0 == 0;
  const int gk4 = (K >> 7) * 4;
  uint32_t tx;
  int fb = 0, nb = 0;
  if (kind == 0) {
    tx = 2u * nr * sb + (has_scales ? 2u * nr * gk4 : 0u);
  } else {
    scale_span(st.r0, nr, K, fb, nb);
    tx = (uint32_t)nr * sb + (has_scales ? (uint32_t)nb : 0u);
  }
  if (lane == 0) mbar_expect_tx(bar, tx);
  __syncwarp();
  uint8_t* sc = buf + 16 * sb;   // scale staging follows the 16 row slots
  const size_t base = (size_t)st.r0 * rb + ((size_t)st.kb0 << 6);
  if (kind == 0) {
    if (whole) {
      if (lane == 0) bulk_g2s(buf, sl.gate + base, (uint32_t)nr * rb, bar);
      if (lane == 1) bulk_g2s(buf + 8 * sb, sl.up + base, (uint32_t)nr * rb, bar);
    } else if (lane < 16) {
      const int i = lane & 7;
      if (i < nr) bulk_g2s(buf + (lane < 8 ? i : 8 + i) * sb, (lane < 8 ? sl.gate : sl.up) + base + (size_t)i * rb,
                           (uint32_t)sb, bar);
    }
    if (has_scales) {
      if (lane == 2) bulk_g2s(sc, sl.gate_s + (size_t)st.r0 * (K >> 7), (uint32_t)nr * gk4, bar);
      if (lane == 3) bulk_g2s(sc + 8 * gk4, sl.up_s + (size_t)st.r0 * (K >> 7), (uint32_t)nr * gk4, bar);
    }
  } else {
    if (whole) {
      if (lane == 0) bulk_g2s(buf, sl.down + base, (uint32_t)nr * rb, bar);
    } else if (lane < nr) {
      bulk_g2s(buf + lane * sb, sl.down + base + (size_t)lane * rb, (uint32_t)sb, bar);
    }
    if (has_scales && lane == 16) bulk_g2s(sc, reinterpret_cast<const uint8_t*>(sl.down_s) + fb, (uint32_t)nb, bar);
  }
}

// ---- block processors: 16 tile rows x 64-byte blocks of each row ---------------------------------
// lane = 4*q + c supplies tile rows q and q+8; the raw dot products come back in element 0 (row q)
// and element 2 (row q+8) of the accumulators -- every MMA column carries the same activation
// vector.  Each block feeds two independent accumulator chains so that consecutive warp MMAs do
// not wait on each other.

// Q4: a[] / b[] = 16 bytes (32 codes) of rows q / q+8, x[] = 64 bytes of fragments (8 MMAs).
#define UMAQ_Q4_LO(w) lop3<0x6A>((w), 0x000F000Fu, 0x64086408u)   /* fp16 1024 + (code + 8)      */
#define UMAQ_Q4_HI(w) lop3<0x6A>((w), 0x00F000F0u, 0x64806480u)   /* fp16 1024 + 16 * (code + 8) */
__device__ __forceinline__ void mma_block_q4(const uint32_t (&a)[4], const uint32_t (&b)[4], const uint4 (&x)[4],
                                             float (&d0)[4], float (&d1)[4]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t ah = a[j] >> 8, bh = b[j] >> 8;
    mma_f16_16816(d0, UMAQ_Q4_LO(a[j]), UMAQ_Q4_LO(b[j]), UMAQ_Q4_HI(a[j]), UMAQ_Q4_HI(b[j]), x[j].x, x[j].y);
    mma_f16_16816(d1, UMAQ_Q4_LO(ah), UMAQ_Q4_LO(bh), UMAQ_Q4_HI(ah), UMAQ_Q4_HI(bh), x[j].z, x[j].w);
  }
}

// Two Q4 blocks at once, sixteen MMAs over eight accumulator chains issued round-robin, so that
// no MMA has to wait for the one before it; sums come back in s0 (first block) and s1 (second).
__device__ __forceinline__ void mma_pair_q4(const uint32_t (&a0)[4], const uint32_t (&b0)[4], const uint4 (&x0)[4],
                                            const uint32_t (&a1)[4], const uint32_t (&b1)[4], const uint4 (&x1)[4],
                                            float (&s0)[2], float (&s1)[2]) {
  float d[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i) d[i][0] = d[i][1] = d[i][2] = d[i][3] = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int ch = (j & 1) * 4;
    const uint32_t ah = a0[j] >> 8, bh = b0[j] >> 8, ch1 = a1[j] >> 8, dh = b1[j] >> 8;
    mma_f16_16816(d[ch + 0], UMAQ_Q4_LO(a0[j]), UMAQ_Q4_LO(b0[j]), UMAQ_Q4_HI(a0[j]), UMAQ_Q4_HI(b0[j]), x0[j].x, x0[j].y);
    mma_f16_16816(d[ch + 1], UMAQ_Q4_LO(a1[j]), UMAQ_Q4_LO(b1[j]), UMAQ_Q4_HI(a1[j]), UMAQ_Q4_HI(b1[j]), x1[j].x, x1[j].y);
    mma_f16_16816(d[ch + 2], UMAQ_Q4_LO(ah), UMAQ_Q4_LO(bh), UMAQ_Q4_HI(ah), UMAQ_Q4_HI(bh), x0[j].z, x0[j].w);
    mma_f16_16816(d[ch + 3], UMAQ_Q4_LO(ch1), UMAQ_Q4_LO(dh), UMAQ_Q4_HI(ch1), UMAQ_Q4_HI(dh), x1[j].z, x1[j].w);
  }
  s0[0] = (d[0][0] + d[2][0]) + (d[4][0] + d[6][0]);
  s0[1] = (d[0][2] + d[2][2]) + (d[4][2] + d[6][2]);
  s1[0] = (d[1][0] + d[3][0]) + (d[5][0] + d[7][0]);
  s1[1] = (d[1][2] + d[3][2]) + (d[5][2] + d[7][2]);
}

// Q8: 16 codes of rows q / q+8, x[] = 32 bytes of fragments (4 MMAs).
__device__ __forceinline__ void mma_block_q8(const uint32_t (&a)[4], const uint32_t (&b)[4], const uint4 (&x)[2],
                                             float (&d0)[4], float (&d1)[4]) {
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const uint32_t a0 = a[2 * j] ^ 0x80808080u, a1 = a[2 * j + 1] ^ 0x80808080u;
    const uint32_t b0 = b[2 * j] ^ 0x80808080u, b1 = b[2 * j + 1] ^ 0x80808080u;
    // byte | 0x6400 -> fp16 1024 + (code + 128)
    mma_f16_16816(d0, prmt(a0, 0x64646464u, 0x4140), prmt(b0, 0x64646464u, 0x4140),
                  prmt(a0, 0x64646464u, 0x4342), prmt(b0, 0x64646464u, 0x4342), x[j].x, x[j].y);
    mma_f16_16816(d1, prmt(a1, 0x64646464u, 0x4140), prmt(b1, 0x64646464u, 0x4140),
                  prmt(a1, 0x64646464u, 0x4342), prmt(b1, 0x64646464u, 0x4342), x[j].z, x[j].w);
  }
}

__device__ __forceinline__ void mma_block_bf16(const uint32_t (&a)[4], const uint32_t (&b)[4], const uint4& x,
                                               float (&d0)[4], float (&d1)[4]) {
  mma_bf16_16816(d0, a[0], b[0], a[1], b[1], x.x, x.y);
  mma_bf16_16816(d1, a[2], b[2], a[3], b[3], x.z, x.w);
}

__device__ __forceinline__ void lds16(const uint8_t* p, uint32_t (&r)[4]) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  r[0] = v.x; r[1] = v.y; r[2] = v.z; r[3] = v.w;
}

// What one warp needs to know about a stage to process blocks of it.
struct StageView {
  const uint8_t* buf;   // 16 row slots of `sb` bytes
  int sb;
  int nkb, kb0;
  int enc;
  const uint8_t* xf;    // fragments of the activation vector, block 0 of the row
  const float* bias;    // bias sums per block (Q4 / Q8)
  const float* sc;      // staged scales
  int sc_lo, sc_hi;     // element offsets of rows q / q+8 (group 0)
};

// One block (local index blk); fragments, bias and scales come from shared memory and are fetched
// before the MMA chain starts.
__device__ __forceinline__ void block_from_smem(const StageView& v, int blk, int q, int c, float& acc_lo, float& acc_hi) {
  uint32_t a[4], b[4];
  lds16(v.buf + q * v.sb + (blk << 6) + (c << 4), a);
  lds16(v.buf + (q + 8) * v.sb + (blk << 6) + (c << 4), b);
  const int kb = v.kb0 + blk;
  float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};
  if (v.enc == ENC_Q4) {
    const uint4* xp = reinterpret_cast<const uint4*>(v.xf + ((size_t)kb << 8) + (c << 6));
    const uint4 x[4] = {xp[0], xp[1], xp[2], xp[3]};
    const float bs = v.bias[kb], s_lo = v.sc[v.sc_lo + kb], s_hi = v.sc[v.sc_hi + kb];
    mma_block_q4(a, b, x, d0, d1);
    acc_lo = fmaf(s_lo, d0[0] + d1[0] - bs, acc_lo);
    acc_hi = fmaf(s_hi, d0[2] + d1[2] - bs, acc_hi);
  } else if (v.enc == ENC_Q8) {
    const uint4* xp = reinterpret_cast<const uint4*>(v.xf + ((size_t)kb << 7) + (c << 5));
    const uint4 x[2] = {xp[0], xp[1]};
    const float bs = v.bias[kb], s_lo = v.sc[v.sc_lo + (kb >> 1)], s_hi = v.sc[v.sc_hi + (kb >> 1)];
    mma_block_q8(a, b, x, d0, d1);
    acc_lo = fmaf(s_lo, d0[0] + d1[0] - bs, acc_lo);
    acc_hi = fmaf(s_hi, d0[2] + d1[2] - bs, acc_hi);
  } else {
    const uint4 x = *reinterpret_cast<const uint4*>(v.xf + ((size_t)kb << 6) + (c << 4));
    mma_block_bf16(a, b, x, d0, d1);
    acc_lo += d0[0] + d1[0];
    acc_hi += d0[2] + d1[2];
  }
}

// Two adjacent blocks (pb, pb+1).  With row strides that are a multiple of 128 bytes, rows q and q+1
// of a quarter-warp hit the same banks; odd rows therefore read the pair in the opposite order,
// which makes both 16-byte loads conflict-free.  XREG: the Q4 fragments of the pair are passed in
// registers (they do not change while a warp keeps the same pair of a 2048-wide row).
template <bool XREG>
__device__ __forceinline__ void pair_from_smem(const StageView& v, int pb, int q, int c, const uint4 (&xr)[8],
                                               float& acc_lo, float& acc_hi) {
  const bool swap = ((v.sb >> 6) & 1) == 0 && (q & 1);
  const int first = swap ? pb + 1 : pb, second = swap ? pb : pb + 1;
  uint32_t r1a[4], r1b[4], r2a[4], r2b[4];
  lds16(v.buf + q * v.sb + (first << 6) + (c << 4), r1a);
  lds16(v.buf + (q + 8) * v.sb + (first << 6) + (c << 4), r1b);
  lds16(v.buf + q * v.sb + (second << 6) + (c << 4), r2a);
  lds16(v.buf + (q + 8) * v.sb + (second << 6) + (c << 4), r2b);
  const int kb = v.kb0 + pb;
  float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};
  float e0[4] = {0.f, 0.f, 0.f, 0.f}, e1[4] = {0.f, 0.f, 0.f, 0.f};
  uint32_t a0[4], b0[4], a1[4], b1[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    a0[i] = swap ? r2a[i] : r1a[i]; b0[i] = swap ? r2b[i] : r1b[i];
    a1[i] = swap ? r1a[i] : r2a[i]; b1[i] = swap ? r1b[i] : r2b[i];
  }
  if (XREG || v.enc == ENC_Q4) {
    const float bs0 = v.bias[kb], bs1 = v.bias[kb + 1];
    const float sl0 = v.sc[v.sc_lo + kb], sh0 = v.sc[v.sc_hi + kb];
    const float sl1 = v.sc[v.sc_lo + kb + 1], sh1 = v.sc[v.sc_hi + kb + 1];
    float s0[2], s1[2];
    if (XREG) {
      const uint4 x0[4] = {xr[0], xr[1], xr[2], xr[3]};
      const uint4 x1[4] = {xr[4], xr[5], xr[6], xr[7]};
      mma_pair_q4(a0, b0, x0, a1, b1, x1, s0, s1);
    } else {
      const uint4* xp = reinterpret_cast<const uint4*>(v.xf + ((size_t)kb << 8) + (c << 6));
      const uint4 x0[4] = {xp[0], xp[1], xp[2], xp[3]};
      const uint4 x1[4] = {xp[16], xp[17], xp[18], xp[19]};
      mma_pair_q4(a0, b0, x0, a1, b1, x1, s0, s1);
    }
    acc_lo = fmaf(sl0, s0[0] - bs0, acc_lo);
    acc_hi = fmaf(sh0, s0[1] - bs0, acc_hi);
    acc_lo = fmaf(sl1, s1[0] - bs1, acc_lo);
    acc_hi = fmaf(sh1, s1[1] - bs1, acc_hi);
  } else if (v.enc == ENC_Q8) {
    const float bs0 = v.bias[kb], bs1 = v.bias[kb + 1];
    const float sl0 = v.sc[v.sc_lo + (kb >> 1)], sh0 = v.sc[v.sc_hi + (kb >> 1)];   // kb is even: one group
    const uint4* xp = reinterpret_cast<const uint4*>(v.xf + ((size_t)kb << 7) + (c << 5));
    const uint4 x0[2] = {xp[0], xp[1]};
    const uint4 x1[2] = {xp[8], xp[9]};
    mma_block_q8(a0, b0, x0, d0, d1);
    mma_block_q8(a1, b1, x1, e0, e1);
    acc_lo = fmaf(sl0, (d0[0] + d1[0] - bs0) + (e0[0] + e1[0] - bs1), acc_lo);
    acc_hi = fmaf(sh0, (d0[2] + d1[2] - bs0) + (e0[2] + e1[2] - bs1), acc_hi);
  } else {
    const uint4* xp = reinterpret_cast<const uint4*>(v.xf + ((size_t)kb << 6) + (c << 4));
    mma_block_bf16(a0, b0, xp[0], d0, d1);
    mma_block_bf16(a1, b1, xp[4], e0, e1);
    acc_lo += (d0[0] + d1[0]) + (e0[0] + e1[0]);
    acc_hi += (d0[2] + d1[2]) + (e0[2] + e1[2]);
  }
}

// ---- activation fragments --------------------------------------------------------------------
// fp16 fragments for Q4 rows: each run of 8 activations k0..k7 is stored as
// [k0, k4, k1/16, k5/16, k2, k6, k3/16, k7/16] (the nibble pairs one LOP3 extracts and the 1/16 that
// undoes the in-place high nibble).  Q8 and BF16 rows use natural order.
//
// store_unit() stores the fragments of one 128-activation unit (lane owns k = 128*unit + 4*lane +
// 0..3, values already multiplied by the prescale) and, for Q4/Q8, the bias sums of its 64-byte
// weight blocks: sum of 1032*x (even k) + 72*x (odd k) for Q4, 1152*x for Q8, taken from the
// rounded fp16 values.
__device__ __forceinline__ void store_unit(int enc, uint8_t* xf, int unit, const float (&v)[4], int lane) {
  const int k0 = unit * 128 + lane * 4;
  if (enc == ENC_Q4) {
    // the lane's activations k0..k0+3 are elements 0..3 (even lane) or 4..7 (odd lane) of an 8-run:
    // run positions 0,2,4,6 resp. 1,3,5,7
    __half* o = reinterpret_cast<__half*>(xf) + (k0 & ~7) + (lane & 1);
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
// lanes combine.  Q4: run positions 0,1,4,5 hold x (coefficient 1032), 2,3,6,7 hold x/16 (72 * 16).
__device__ __forceinline__ void build_bias(int enc, const uint8_t* xf, float* bias, int n, int tid) {
  const int chunks = n >> 5;
  for (int ch = tid; ch < ((chunks + 31) & ~31); ch += kConsumers) {
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

__global__ void __launch_bounds__(kThreads, 1) moe_decode_kernel(const DecodeParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  Shared& sh = *reinterpret_cast<Shared*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int H = p.hidden;
  const int G = gridDim.x;
  Shape S;
  S.H = H; S.top_k = p.top_k; S.enc = p.enc; S.inter = p.inter; S.shared_inter = p.shared_inter;
  S.nslots = p.top_k + (p.sh_gate ? 1 : 0);
  S.max_kb = p.stage_bytes >> 10;          // a stage holds 16 rows x (max_kb * 64) bytes

  // ---- carve shared memory (same arithmetic as decode_smem_layout() on the host) --------------
  uint8_t* cur = smem_raw + ((sizeof(Shared) + 127) & ~127);
  uint8_t* xfA = cur;                 cur += H * 2;           // routed-encoding fragments of x
  uint8_t* xfA_bf = cur;              cur += H * 2;           // bf16 x (shared expert / bf16 layers)
  float* biasA = reinterpret_cast<float*>(cur); cur += (H >> 6) * 4;
  uint8_t* xfB = cur;                 cur += p.inter_total * 2;
  float* biasB = reinterpret_cast<float*>(cur); cur += ((p.inter_total >> 6) + kMaxSlots) * 4;
  uint8_t* ring = smem_raw + (((cur - smem_raw) + 1023) & ~1023);
  const int stage_bytes = p.stage_bytes + kScaleArea;
  const int nstages = p.nstages;
  volatile int* abort_flag = &sh.abort_flag;
  // CTA 0 leaves cycle stamps of its phases in the diagnostic area of the workspace
  long long* stamps = (blockIdx.x == 0 && tid == 0) ? reinterpret_cast<long long*>(p.sync) + 24 : nullptr;
  const long long t_start = clock64();
#define UMAQ_STAMP(i) do { if (stamps) stamps[i] = clock64() - t_start; } while (0)

  // The activation vector is needed first and is a cold read: every consumer warp fetches its
  // 128-activation units before anything else so the latency overlaps the set-up.
  constexpr int kMaxUX = kMaxUnitsX / kConsumerWarps;
  float xv[kMaxUX][4];
  float gdot = 0.f;
#pragma unroll
  for (int j = 0; j < kMaxUX; ++j) {
    const int u = warp + j * kConsumerWarps;
    xv[j][0] = xv[j][1] = xv[j][2] = xv[j][3] = 0.f;
    if (warp < kConsumerWarps && u * 128 < H) {
      const uint2 raw = *reinterpret_cast<const uint2*>(p.x + u * 128 + lane * 4);
      xv[j][0] = __uint_as_float(raw.x << 16); xv[j][1] = __uint_as_float(raw.x & 0xffff0000u);
      xv[j][2] = __uint_as_float(raw.y << 16); xv[j][3] = __uint_as_float(raw.y & 0xffff0000u);
      if (p.sh_gatevec) {
        const uint2 g = *reinterpret_cast<const uint2*>(p.sh_gatevec + u * 128 + lane * 4);
        gdot += xv[j][0] * __uint_as_float(g.x << 16) + xv[j][1] * __uint_as_float(g.x & 0xffff0000u) +
                xv[j][2] * __uint_as_float(g.y << 16) + xv[j][3] * __uint_as_float(g.y & 0xffff0000u);
      }
    }
  }

  // ---- set-up: routes (one round of global loads), stage list, barriers --------------------------
  if (warp == 0) {
    if (lane == 30) sh.abort_flag = 0;
    if (lane < p.top_k) {
      long long e = p.idx64 ? reinterpret_cast<const long long*>(p.idx)[lane]
                            : (long long)reinterpret_cast<const int*>(p.idx)[lane];
      const float wt = p.w[lane];
      Slot& sl = sh.slots[lane];
      sl.bad = (e < 0 || e >= p.experts);
      if (sl.bad) e = 0;
      const size_t wgu = (size_t)p.inter * row_bytes(p.enc, H), wd = (size_t)H * row_bytes(p.enc, p.inter);
      sl.gate = p.gate + e * wgu; sl.up = p.up + e * wgu; sl.down = p.down + e * wd;
      sl.gate_s = p.gate_s ? p.gate_s + e * (size_t)p.inter * (H >> 7) : nullptr;
      sl.up_s = p.up_s ? p.up_s + e * (size_t)p.inter * (H >> 7) : nullptr;
      sl.down_s = p.down_s ? p.down_s + e * (size_t)H * (p.inter >> 7) : nullptr;
      sl.expert = (int)e; sl.weight = wt;
    } else if (lane == p.top_k && p.sh_gate) {
      Slot& sl = sh.slots[lane];
      sl.gate = reinterpret_cast<const uint8_t*>(p.sh_gate); sl.up = reinterpret_cast<const uint8_t*>(p.sh_up);
      sl.down = reinterpret_cast<const uint8_t*>(p.sh_down);
      sl.gate_s = sl.up_s = sl.down_s = nullptr;
      sl.expert = 0x7fffffff; sl.weight = 1.f; sl.bad = 0;
    }
    __syncwarp();
    // phase-B order: ascending expert number, stable in slot order (rank by counting); shared last
    if (lane < S.nslots) {
      const int mine = sh.slots[lane].expert;
      int rank = 0;
      for (int j = 0; j < S.nslots; ++j) {
        const int other = sh.slots[j].expert;
        rank += (other < mine) || (other == mine && j < lane);
      }
      sh.order[rank] = lane;
      if (sh.slots[lane].bad) {          // every CTA sees the same routes and takes the same exit
        atomicExch(p.sync + 2, (unsigned)ERR_BAD_ARGUMENT);
        sh.abort_flag = 1;
      }
    }
  } else if (warp == 1) {
    build_stage_list(sh, S, G, blockIdx.x, lane);
  } else if (warp == 2) {
    if (lane < nstages) { mbar_init(&sh.full[lane], 1); mbar_init(&sh.empty[lane], kGroupWarps); }
    __syncwarp();
    if (lane == 0) fence_barrier_init();
  } else if (warp == 3) {
    // grid barrier: the counter only ever grows by G per launch; whatever has arrived already,
    // this launch is released at the next multiple of G above the value seen now
    if (lane == 0) {
      const unsigned long long seen = ld_acquire_u64(reinterpret_cast<const unsigned long long*>(p.sync + 4));
      sh.bar_target = (seen / G + 1) * G;
    }
  }
  __syncthreads();
  UMAQ_STAMP(0);
  const int nlist = min(sh.nlist, kMaxList);
  const int first_b = min(sh.first_b, nlist);
  if (sh.nlist > kMaxList && tid == 0) { atomicExch(p.sync + 2, (unsigned)ERR_UNSUPPORTED); *abort_flag = 1; }

  if (warp == kConsumerWarps) {
    // ======================= producer warp ===================================================
    int n = 0;
    for (; n < nlist && !*abort_flag; ++n) {
      const int s = n % nstages;
      if (n >= nstages && !mbar_wait(&sh.empty[s], ((n / nstages) - 1) & 1)) {
        if (lane == 0) { atomicExch(p.sync + 2, (unsigned)ERR_DEVICE_TIMEOUT); *abort_flag = 1; }
        __syncwarp();
        break;
      }
      if (*abort_flag) break;
      issue_stage(sh, S, sh.list[n], ring + (size_t)s * stage_bytes, &sh.full[s], lane);
    }
    // After an abort the consumers skip their waits: drain what was issued so that no copy is
    // still writing this CTA's shared memory when it retires.
    if (*abort_flag) {
      const int first = n > nstages ? n - nstages : 0;
      for (int i = first; i < n; ++i) mbar_wait(&sh.full[i % nstages], (i / nstages) & 1);
    }
    return;
  }

  // ========================= consumer warps =====================================================
  const int q = lane >> 2, c = lane & 3;
  const int grp = warp >> 3, w8 = warp & 7;     // K-split group and position inside it

  // x -> fragments (routed encoding: prescaled fp16; bf16 copy), sigmoid gate of the shared expert.
  // Warp w owns the 128-activation units w, w+16, ... (loaded at kernel entry).
  {
    float am = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxUX; ++j)
      am = fmaxf(am, fmaxf(fmaxf(fabsf(xv[j][0]), fabsf(xv[j][1])), fmaxf(fabsf(xv[j][2]), fabsf(xv[j][3]))));
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
      gdot += __shfl_xor_sync(0xffffffffu, gdot, o);
    }
    if (lane == 0) { sh.wred[warp] = am; sh.wred2[warp] = gdot; }
    named_bar_sync(1, kConsumers);
    float m = 0.f, t = 0.f;
#pragma unroll
    for (int i = 0; i < kConsumerWarps; ++i) { m = fmaxf(m, sh.wred[i]); t += sh.wred2[i]; }
    const float sx = prescale_for(m);
    if (tid == 0) {
      sh.scale_x_inv = 1.f / sx;
      t = bf16_round(t);                                   // nn.Linear output in BF16
      sh.sig_gate = bf16_round(1.f / (1.f + expf(-t)));    // sigmoid of a BF16 tensor
    }
#pragma unroll
    for (int j = 0; j < kMaxUX; ++j) {
      const int u = warp + j * kConsumerWarps;
      if (u * 128 < H) {
        store_unit(ENC_BF16, xfA_bf, u, xv[j], lane);
        if (p.enc != ENC_BF16) {
          const float sv[4] = {xv[j][0] * sx, xv[j][1] * sx, xv[j][2] * sx, xv[j][3] * sx};
          store_unit(p.enc, xfA, u, sv, lane);
        }
      }
    }
    named_bar_sync(1, kConsumers);
    if (p.enc != ENC_BF16) build_bias(p.enc, xfA, biasA, H, tid);
    named_bar_sync(1, kConsumers);
  }
  UMAQ_STAMP(1);

  // Q4 rows of 16 blocks: this warp's two blocks of x stay in registers during phase A.
  const bool xreg = p.enc == ENC_Q4 && (H >> 7) == 16;
  uint4 xr[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) xr[i] = make_uint4(0, 0, 0, 0);
  if (xreg) {
    const uint4* xp = reinterpret_cast<const uint4*>(xfA + ((size_t)(2 * w8) << 8) + (c << 6));
#pragma unroll
    for (int i = 0; i < 4; ++i) { xr[i] = xp[i]; xr[4 + i] = xp[16 + i]; }
  }

  int pend = 0;                  // tiles whose partial sums sit in sh.red, not yet reduced
  float acc_lo = 0.f, acc_hi = 0.f;

  // Reduces the parked tiles and finishes them.  Phase A: sum of the eight K-slices, SwiGLU, float32
  // intermediate.  Phase B: the ordered BF16 running sum over the slots of one 16-row group.
  auto flush = [&]() {
    named_bar_sync(1, kConsumers);
    // `go` only guards work; the barriers below are reached by every thread whatever it reads
    const bool go = !*abort_flag;
    if (pend && sh.tdesc[0].kind() == 0) {
      for (int i = tid; go && i < pend * 8; i += kConsumers) {
        const int t = i >> 3, f = i & 7;
        const Stage td = sh.tdesc[t];
        if (f < td.nr()) {
          const int slot = td.pos();
          float g = 0.f, u = 0.f;
#pragma unroll
          for (int w = 0; w < kGroupWarps; ++w) { g += sh.red[t][w][f]; u += sh.red[t][w][8 + f]; }
          float v;
          if (slot >= S.top_k) {      // Qwen2MoeMLP in BF16: every linear / activation output is rounded
            g = bf16_round(g); u = bf16_round(u);
            v = bf16_round(bf16_round(silu_f32(g)) * u);
          } else {
            if (S.enc != ENC_BF16) { g *= sh.scale_x_inv; u *= sh.scale_x_inv; }
            v = silu_f32(g) * u;
          }
          p.inter_buf[S.inter_off(slot) + td.r0 + f] = v;
        }
      }
    } else if (pend) {
      // the parked tiles are the slots of one row group in phase-B order: every (slot, row)
      // contribution in parallel, then the ordered BF16 running sum per row
      const int nr = sh.tdesc[0].nr();
      for (int i = tid; go && i < pend * 16; i += kConsumers) {
        const int t = i >> 4, r = i & 15;
        const Stage td = sh.tdesc[t];
        const int slot = sh.order[td.pos()];
        float y = 0.f;
        if (td.owned()) {
          y = sh.red[t][0][r] + sh.red[t][1][r];
        } else {
#pragma unroll
          for (int w = 0; w < kGroupWarps; ++w) y += sh.red[t][w][r];
        }
        if (S.enc_of(slot) != ENC_BF16) y *= sh.scaleB_inv;
        sh.contrib[t][r] = slot >= S.top_k ? bf16_round(sh.sig_gate * bf16_round(y))
                                           : bf16_round(y * sh.slots[slot].weight);
      }
      named_bar_sync(1, kConsumers);
      if (go && tid < nr) {
        float run = 0.f;
        for (int t = 0; t < pend; ++t) run = bf16_round(run + sh.contrib[t][tid]);
        p.out[sh.tdesc[0].r0 + tid] = __float2bfloat16_rn(run);
      }
    }
    pend = 0;
    named_bar_sync(1, kConsumers);
  };

  for (int n = 0;; ++n) {
    if (n == first_b) {
      // ---- phase boundary: grid barrier, then phase-B fragments from the float32 intermediates --
      UMAQ_STAMP(2);
      flush();
      if (tid == 0) {
        sh.amaxB = 0u;
        // one monotonic counter; this launch is released at the next multiple of G
        __threadfence();
        red_release_add_u64(reinterpret_cast<unsigned long long*>(p.sync + 4), 1ull);
        if (!*abort_flag) {
          const unsigned long long target = sh.bar_target;
          const uint64_t t0 = global_ns();
          while (ld_acquire_u64(reinterpret_cast<const unsigned long long*>(p.sync + 4)) < target) {
            if (global_ns() - t0 > kWaitBudgetNs) {
              atomicExch(p.sync + 2, (unsigned)ERR_DEVICE_TIMEOUT);
              *abort_flag = 1;
              break;
            }
          }
        }
        __threadfence();
      }
      named_bar_sync(1, kConsumers);
      UMAQ_STAMP(3);
      if (n < nlist && !*abort_flag) {
        // every CTA needs every slot's whole intermediate vector: one batch of L2 loads per warp
        constexpr int kMaxU = kMaxUnitsB / kConsumerWarps;
        float iv[kMaxU][4];
        const int nunits = p.inter_total >> 7;
        const int qunits = S.enc == ENC_BF16 ? 0 : (S.top_k * p.inter) >> 7;   // units that get the prescale
        float a = 0.f;
#pragma unroll
        for (int j = 0; j < kMaxU; ++j) {
          const int u = warp + j * kConsumerWarps;
          iv[j][0] = iv[j][1] = iv[j][2] = iv[j][3] = 0.f;
          if (u < nunits) {
            const float4 f = __ldcg(reinterpret_cast<const float4*>(p.inter_buf + u * 128 + lane * 4));
            iv[j][0] = f.x; iv[j][1] = f.y; iv[j][2] = f.z; iv[j][3] = f.w;
          }
        }
#pragma unroll
        for (int j = 0; j < kMaxU; ++j)
          if (warp + j * kConsumerWarps < qunits)
            a = fmaxf(a, fmaxf(fmaxf(fabsf(iv[j][0]), fabsf(iv[j][1])), fmaxf(fabsf(iv[j][2]), fabsf(iv[j][3]))));
#pragma unroll
        for (int o = 16; o; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
        if (lane == 0 && a < 3.0e38f) atomicMax(&sh.amaxB, __float_as_uint(a));
        named_bar_sync(1, kConsumers);
        const float sc = prescale_for(__uint_as_float(sh.amaxB));
        if (tid == 0) { sh.scaleB = sc; sh.scaleB_inv = 1.f / sc; }
#pragma unroll
        for (int j = 0; j < kMaxU; ++j) {
          const int u = warp + j * kConsumerWarps;
          if (u < nunits) {
            if (u < qunits) {
              const float sv[4] = {iv[j][0] * sc, iv[j][1] * sc, iv[j][2] * sc, iv[j][3] * sc};
              store_unit(S.enc, xfB, u, sv, lane);
            } else {
              store_unit(ENC_BF16, xfB, u, iv[j], lane);
            }
          }
        }
        named_bar_sync(1, kConsumers);
        // bias sums of the quantised slots: slot s's blocks start at bias_off(s)
        if (qunits) {
          const int per = row_bytes(S.enc, p.inter) >> 6;       // 64-byte weight blocks per down row
          for (int sl = 0; sl < S.top_k; ++sl)
            build_bias(S.enc, xfB + (size_t)S.inter_off(sl) * 2, biasB + S.bias_off(sl), p.inter, tid);
          (void)per;
        }
      }
      named_bar_sync(1, kConsumers);
      UMAQ_STAMP(4);
    }
    if (n >= nlist) break;

    const Stage st = sh.list[n];
    const int s = n % nstages;
    const int half = warp & 1;
    const bool mine = st.owned() ? ((warp >> 1) == st.owner()) : (grp == st.group());
    if (mine) {
      const bool live = !*abort_flag && mbar_wait(&sh.full[s], (n / nstages) & 1);
      if (!live && !*abort_flag && lane == 0) { atomicExch(p.sync + 2, (unsigned)ERR_DEVICE_TIMEOUT); *abort_flag = 1; }
      if (live) {
        const int kind = st.kind();
        const int slot = kind ? sh.order[st.pos()] : st.pos();
        StageView v;
        v.buf = ring + (size_t)s * stage_bytes;
        v.sb = st.nkb << 6;
        v.nkb = st.nkb; v.kb0 = st.kb0; v.enc = S.enc_of(slot);
        const int gk = (kind == 0 ? H : S.inter_of(slot)) >> 7;
        v.sc = reinterpret_cast<const float*>(v.buf + 16 * v.sb);
        if (kind == 0) {
          v.sc_lo = q * gk; v.sc_hi = (8 + q) * gk;
          v.xf = v.enc == ENC_BF16 ? xfA_bf : xfA; v.bias = biasA;
        } else {
          const int off = ((st.r0 * gk * 4) & 15) >> 2;
          v.sc_lo = off + q * gk; v.sc_hi = off + (q + 8) * gk;
          v.xf = xfB + (size_t)S.inter_off(slot) * 2; v.bias = biasB + S.bias_off(slot);
        }
        if (xreg && kind == 0 && v.enc == ENC_Q4) {
          pair_from_smem<true>(v, 2 * w8, q, c, xr, acc_lo, acc_hi);
        } else {
          // owned tile: the two warps of the pair take alternate block pairs; K-split stage: the
          // group's eight warps take block pairs (rows of >= 16 blocks) or single blocks
          const bool pairs = st.owned() || v.nkb >= 16;
          const int step = st.owned() ? 4 : (pairs ? 2 * kGroupWarps : kGroupWarps);
          for (int b = st.owned() ? 2 * half : (pairs ? 2 * w8 : w8); b < v.nkb; b += step) {
            if (pairs && b + 1 < v.nkb) pair_from_smem<false>(v, b, q, c, xr, acc_lo, acc_hi);
            else block_from_smem(v, b, q, c, acc_lo, acc_hi);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive_n(&sh.empty[s], st.owned() ? kGroupWarps / 2 : 1);
      }
    }
    if (!st.last()) continue;

    // ---- tile done: park this warp's partial sums; reduce them in batches ------------------------
    if (mine && c == 0) {
      const int wslot = st.owned() ? half : w8;
      sh.red[pend][wslot][q] = acc_lo; sh.red[pend][wslot][q + 8] = acc_hi;
    }
    if (tid == 0) sh.tdesc[pend] = st;
    if (mine) acc_lo = acc_hi = 0.f;
    ++pend;
    // phase B: a row group is complete once its last slot is parked; phase A: when the buffer is full
    if (st.kind() ? (st.pos() == S.nslots - 1) : (pend == kRedTiles)) flush();
  }
  UMAQ_STAMP(5);
#undef UMAQ_STAMP
}

struct SmemPlan { size_t fixed; int stage_bytes; int nstages; size_t total; };

SmemPlan decode_smem_layout(const DecodeParams& p) {
  SmemPlan s{};
  size_t cur = (sizeof(Shared) + 127) & ~size_t(127);
  cur += (size_t)p.hidden * 2 * 2 + (size_t)(p.hidden >> 6) * 4;
  cur += (size_t)p.inter_total * 2 + ((size_t)(p.inter_total >> 6) + kMaxSlots) * 4;
  s.fixed = (cur + 1023) & ~size_t(1023);
  int kb = 16;   // BF16 rows are sliced to 1 KiB; quantised rows are staged whole
  if (p.enc != ENC_BF16) {
    kb = std::max(kb, row_bytes(p.enc, p.hidden) >> 6);
    kb = std::max(kb, (row_bytes(p.enc, p.inter) + 63) >> 6);
  }
  s.stage_bytes = kb << 10;
  const size_t limit = 227 * 1024;
  const size_t per = (size_t)s.stage_bytes + kScaleArea;
  s.nstages = s.fixed + per > limit ? 0 : (int)std::min<size_t>(kMaxRing, (limit - s.fixed) / per);
  s.total = s.fixed + per * s.nstages;
  return s;
}

}  // namespace

size_t decode_workspace_bytes(int top_k, int inter, int shared_inter) {
  return kDecodeWsHeader + ((size_t)top_k * inter + shared_inter) * sizeof(float);
}

int launch_moe_decode(DecodeParams p, cudaStream_t stream) {
  if (p.top_k < 1 || p.top_k > 8 || p.hidden % 128 || p.inter % 128 || p.hidden < 128 || p.inter < 128 ||
      (p.sh_gate && (p.shared_inter % 128 || p.shared_inter < 128)) || p.enc < 0 || p.enc > 2) {
    set_error("decode: unsupported shape (hidden %d, intermediate %d, top_k %d, shared %d, encoding %d)", p.hidden,
              p.inter, p.top_k, p.shared_inter, p.enc);
    return ERR_BAD_ARGUMENT;
  }
  if (p.enc != ENC_BF16 && (!p.gate_s || !p.up_s || !p.down_s)) {
    set_error("decode: quantised layer without scales");
    return ERR_BAD_ARGUMENT;
  }
  p.inter_total = p.top_k * p.inter + (p.sh_gate ? p.shared_inter : 0);
  if (p.hidden > kMaxUnitsX * 128 || p.inter_total > kMaxUnitsB * 128) {
    set_error("decode: hidden size %d or summed intermediate size %d beyond the register plan", p.hidden, p.inter_total);
    return ERR_UNSUPPORTED;
  }
  const SmemPlan plan = decode_smem_layout(p);
  const int grid = sm_count();
  if (plan.nstages < 2 || grid < 1) {
    set_error("decode: shape does not fit the shared-memory plan (fixed %zu B, stage %d B)", plan.fixed,
              plan.stage_bytes);
    return ERR_UNSUPPORTED;
  }
  p.stage_bytes = plan.stage_bytes;
  p.nstages = plan.nstages;
  static thread_local int configured_device = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_device != dev) {
    cudaError_t e = cudaFuncSetAttribute(moe_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) { set_error("decode: cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return ERR_LAUNCH; }
    configured_device = dev;
  }
  void* args[] = {&p};
  cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(moe_decode_kernel), dim3(grid), dim3(kThreads),
                                              args, plan.total, stream);
  if (e != cudaSuccess) { set_error("decode: launch failed: %s", cudaGetErrorString(e)); return ERR_LAUNCH; }
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
  p.amax = reinterpret_cast<unsigned*>(ws + 64);
  p.inter_buf = reinterpret_cast<float*>(ws + kDecodeWsHeader);
  return launch_moe_decode(p, st);
}
