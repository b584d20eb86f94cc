// Prefill / batched path: grouped-expert GEMMs on the 5th-generation tensor cores.
//
//   gate/up:  inter[r, f] = SiLU(x_r . Gate_e[f]) * (x_r . Up_e[f])        (GEMM 1, SwiGLU epilogue)
//   down:     y[r, n]     = w_r * (inter_r . Down_e[n])                    (GEMM 2, weighted epilogue)
//
// over the routes r sorted by expert e.  Replaces the reference's scalar-FMA prefill kernels
// (src/uma_qmoe/native/packed_q4_kernel.cu:560-776 Q4, :894-1099 Q8, launched from :1535-1641 and
// :1691-1762) and its torch._grouped_mm path for BF16 layers (src/uma_qmoe/native_backend.py:958-1005).
//
// One CTA computes one tile of up to 256 routes x 256 columns: two M = 128, N = 256 accumulators
// (all 512 tensor-memory columns) that share every converted weight tile.  The wide tile is what keeps
// the activation traffic from L2 below the tensor rate: a 128-column tile re-reads the activations
// 16 times per layer and is L2-bound at 40 % of the tensor peak.  Warp 0 drives TMA:
// activation tiles (2 x 128 rows x 64 k, 128-byte swizzle) and the packed weight rows of the same k
// range.  Eight warps
// turn the packed codes into BF16 (code * scale) and write the canonical K-major 128-byte-swizzled
// B tile the tensor core reads; warp 1 issues tcgen05.mma (M = 128, N = 256, K = 16) with the FP32
// accumulator in tensor memory and signals buffers free with tcgen05.commit.  The same eight warps
// then read the accumulator with tcgen05.ld and run the epilogue.  BF16 layers skip the conversion:
// TMA writes the swizzled B tile directly.
//
// K order.  Inside every run of 8 consecutive k the quantised paths use the order
// [k0,k4,k1,k5,k2,k6,k3,k7] for BOTH operands: it is what one LOP3 per nibble pair produces, and a
// consistent permutation of K leaves the contraction unchanged.  The gather kernel writes the
// activations in that order and the SwiGLU epilogue writes the intermediate in it.
#include "grouped.cuh"

#include <cuda.h>

#include "common.cuh"

namespace umaq {
namespace {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int kInStages = 3;          // TMA ring of activation tiles (2 x 128 rows x 64 k each)
constexpr int kBStages = 2;           // converted B tiles (256 rows x 64 k)
constexpr int kConvertWarps = 8;
constexpr int kGemmThreads = (3 + kConvertWarps) * 32;   // + activation TMA, MMA issuer, weight TMA
constexpr int kWeightWarp = 2 + kConvertWarps;
constexpr int kHalves = 2;            // M = 128 accumulators per tile
constexpr int kTmemCols = BN * kHalves;   // 512: the whole tensor memory of the SM
constexpr int kMaxGroups = 16;        // quantised K <= 2048

// ---- tcgen05 / TMA wrappers ---------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major, 128-byte-swizzled operand tile whose rows are 128 bytes (64 bf16) and whose 8-row groups
// are 1024 bytes apart; `addr` must be 1024-byte aligned plus a multiple of 32 bytes along K.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);          // start address, 16-byte units
  d |= (uint64_t)1 << 16;                          // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;                // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                          // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                          // SWIZZLE_128B
  return d;
}
// kind::f16, BF16 x BF16 -> FP32, both operands K-major, M = 128, N = BN
constexpr uint32_t kInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

constexpr int kMaxPStages = 4;        // packed-weight ring (8 KiB stages for Q4)
struct GemmShared {
  uint64_t in_full[kInStages];
  uint64_t in_empty[kInStages];
  uint64_t p_full[kMaxPStages];
  uint64_t p_empty[kMaxPStages];
  uint64_t b_full[kBStages];
  uint64_t b_empty[kBStages];
  uint64_t scales_full;
  uint64_t acc_full;
  uint32_t tmem_base;
  int abort_flag;
};

struct TileInfo {
  int expert, row0, nrows;
};

// ---- conversion of one thread's 32 codes (row r, half h of the 64-wide k chunk) ------------------
// Q4: 16 bytes -> 16 bf16x2 words in the permuted order, value = code * scale rounded to BF16.
__device__ __forceinline__ void convert_q4(const uint4 raw, float scale, uint32_t (&out)[16]) {
  const __nv_bfloat162 s2 = __float2bfloat162_rn(scale);
  const __nv_bfloat162 off = __float2bfloat162_rn(136.f);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      // ((w >> 4i) ^ 8) & 0xF | 0x4300 : bf16 128 + (code + 8) for nibbles i and i + 4
      const uint32_t m = lop3<0x6A>(w[j] >> (4 * i), 0x000F000Fu, 0x43084308u);
      __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&m);
      v = __hmul2(__hsub2(v, off), s2);
      out[j * 4 + i] = *reinterpret_cast<uint32_t*>(&v);
    }
  }
}
// Q8: 32 bytes -> 16 bf16x2 words in the permuted order; code * scale in float32, one rounding.
__device__ __forceinline__ void convert_q8(const uint4 r0, const uint4 r1, float scale, uint32_t (&out)[16]) {
  const uint32_t w[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {       // 8 codes: words 2j (k0..k3) and 2j+1 (k4..k7)
    const uint32_t a = w[2 * j] ^ 0x80808080u, b = w[2 * j + 1] ^ 0x80808080u;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      // 0x4B0000xx = float 2^23 + (code + 128)
      const float lo = __uint_as_float(prmt(a, 0x4B000000u, 0x7650 + i)) - 8388736.f;   // k_i
      const float hi = __uint_as_float(prmt(b, 0x4B000000u, 0x7650 + i)) - 8388736.f;   // k_{i+4}
      const __nv_bfloat162 v = __floats2bfloat162_rn(lo * scale, hi * scale);
      out[j * 4 + i] = *reinterpret_cast<const uint32_t*>(&v);
    }
  }
}

template <int ENC, int MODE>
__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b0,
                    const __grid_constant__ CUtensorMap map_b1, const GroupedParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // layout: [A stages][packed stages][B stages][scales][control]
  constexpr int kPackedRow = ENC == ENC_Q4 ? BK / 2 : BK;               // bytes of codes per row and k chunk
  constexpr int kPackedBytes = ENC == ENC_BF16 ? 0 : BN * kPackedRow;
  constexpr int kAHalf = BM * BK * 2, kATile = kHalves * kAHalf, kBTile = BN * BK * 2;
  constexpr int kPStages = ENC == ENC_Q4 ? 4 : 2;
  uint8_t* sA = smem_raw;
  uint8_t* sP = sA + kInStages * kATile;
  uint8_t* sB = sP + kPStages * kPackedBytes;
  constexpr int kNumB = ENC == ENC_BF16 ? kInStages : kBStages;
  float* sScales = reinterpret_cast<float*>(sB + kNumB * kBTile);
  GemmShared& sh = *reinterpret_cast<GemmShared*>(reinterpret_cast<uint8_t*>(sScales) + BN * kMaxGroups * 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile_m = blockIdx.y, tile_n = blockIdx.x;
  if (tile_m >= *p.num_tiles) return;
  const int expert = p.tile_expert[tile_m], row0 = p.tile_row0[tile_m], nrows = p.tile_rows[tile_m];
  const int K = p.k;
  const int nk = K / BK;
  const int groups = K >> 7;
  const bool two = nrows > BM;             // the tile has a second 128-route half
  volatile int* abort_flag = &sh.abort_flag;

  if (tid == 0) {
    for (int s = 0; s < kInStages; ++s) { mbar_init(&sh.in_full[s], 1); mbar_init(&sh.in_empty[s], 1); }
    for (int s = 0; s < kMaxPStages; ++s) { mbar_init(&sh.p_full[s], 1); mbar_init(&sh.p_empty[s], kConvertWarps); }
    for (int s = 0; s < kBStages; ++s) { mbar_init(&sh.b_full[s], kConvertWarps); mbar_init(&sh.b_empty[s], 1); }
    mbar_init(&sh.scales_full, 1);
    mbar_init(&sh.acc_full, 1);
    sh.abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&sh.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh.tmem_base;

  // first weight row of this tile inside the concatenated projection, per half of the tile
  // MODE 0: columns [0,64) = gate rows f0.., [64,128) = up rows f0..;  MODE 1: 128 down rows n0..
  const int f0 = tile_n * (MODE == 0 ? BN / 2 : BN);
  const long long wrow0 = (long long)expert * p.n_rows + f0;

  if (warp == 0) {
    // ===================== TMA producer: activation tiles (and BF16 weight tiles) ==================
    if (lane == 0) {
      int issued = 0;
      for (int kc = 0; kc < nk && !*abort_flag; ++kc) {
        const int s = kc % kInStages;
        if (kc >= kInStages && !mbar_wait(&sh.in_empty[s], ((kc / kInStages) - 1) & 1)) {
          atomicExch(p.status, (unsigned)ERR_DEVICE_TIMEOUT); *abort_flag = 1; break;
        }
        const uint32_t bytes = (two ? kATile : kAHalf) + (ENC == ENC_BF16 ? kBTile : 0);
        mbar_expect_tx(&sh.in_full[s], bytes);
        tma_load_2d(sA + s * kATile, &map_a, kc * BK, row0, &sh.in_full[s]);
        if (two) tma_load_2d(sA + s * kATile + kAHalf, &map_a, kc * BK, row0 + BM, &sh.in_full[s]);
        if (ENC == ENC_BF16) {
          uint8_t* dst = sB + s * kBTile;
          if (MODE == 0) {
            tma_load_2d(dst, &map_b0, kc * BK, (int)wrow0, &sh.in_full[s]);
            tma_load_2d(dst + (BN / 2) * BK * 2, &map_b1, kc * BK, (int)wrow0, &sh.in_full[s]);
          } else {
            tma_load_2d(dst, &map_b0, kc * BK, (int)wrow0, &sh.in_full[s]);
          }
        }
        issued = kc + 1;
      }
      // after an abort nobody consumes: wait (bounded) for the copies still in flight
      if (*abort_flag)
        for (int kc = issued > kInStages ? issued - kInStages : 0; kc < issued; ++kc)
          mbar_wait(&sh.in_full[kc % kInStages], (kc / kInStages) & 1);
    }
  } else if (warp == kWeightWarp) {
    // ===================== TMA producer: scales and packed weight rows, on their own deeper ring ====
    if (lane == 0 && ENC != ENC_BF16) {
      const uint32_t half_bytes = (uint32_t)(MODE == 0 ? BN / 2 : BN) * groups * 4;
      mbar_expect_tx(&sh.scales_full, MODE == 0 ? 2 * half_bytes : half_bytes);
      bulk_g2s(sScales, p.scales0 + wrow0 * groups, half_bytes, &sh.scales_full);
      if (MODE == 0) bulk_g2s(sScales + (BN / 2) * groups, p.scales1 + wrow0 * groups, half_bytes, &sh.scales_full);
      int issued = 0;
      for (int kc = 0; kc < nk && !*abort_flag; ++kc) {
        const int s = kc % kPStages;
        if (kc >= kPStages && !mbar_wait(&sh.p_empty[s], ((kc / kPStages) - 1) & 1)) {
          atomicExch(p.status, (unsigned)ERR_DEVICE_TIMEOUT); *abort_flag = 1; break;
        }
        mbar_expect_tx(&sh.p_full[s], kPackedBytes);
        uint8_t* dst = sP + s * kPackedBytes;
        if (MODE == 0) {
          tma_load_2d(dst, &map_b0, kc * kPackedRow, (int)wrow0, &sh.p_full[s]);
          tma_load_2d(dst + (BN / 2) * kPackedRow, &map_b1, kc * kPackedRow, (int)wrow0, &sh.p_full[s]);
        } else {
          tma_load_2d(dst, &map_b0, kc * kPackedRow, (int)wrow0, &sh.p_full[s]);
        }
        issued = kc + 1;
      }
      if (*abort_flag) {
        mbar_wait(&sh.scales_full, 0);
        for (int kc = issued > kPStages ? issued - kPStages : 0; kc < issued; ++kc)
          mbar_wait(&sh.p_full[kc % kPStages], (kc / kPStages) & 1);
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer ============================================================
    if (lane == 0) {
      for (int kc = 0; kc < nk && !*abort_flag; ++kc) {
        const int s = kc % kInStages;
        const int sb = ENC == ENC_BF16 ? s : kc % kBStages;
        bool ok = mbar_wait(&sh.in_full[s], (kc / kInStages) & 1);
        if (ok && ENC != ENC_BF16) ok = mbar_wait(&sh.b_full[sb], (kc / kBStages) & 1);
        if (!ok) { atomicExch(p.status, (unsigned)ERR_DEVICE_TIMEOUT); *abort_flag = 1; break; }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(sA + s * kATile), b_addr = smem_u32(sB + sb * kBTile);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) {
          const uint64_t bdesc = smem_desc_sw128(b_addr + k * 32);
          tc_mma_bf16(tmem, smem_desc_sw128(a_addr + k * 32), bdesc, kInstrDesc, (kc | k) ? 1u : 0u);
          if (two) tc_mma_bf16(tmem + BN, smem_desc_sw128(a_addr + kAHalf + k * 32), bdesc, kInstrDesc, (kc | k) ? 1u : 0u);
        }
        tc_commit(&sh.in_empty[s]);                 // A tile (and a BF16 B tile) may be overwritten
        if (ENC != ENC_BF16) tc_commit(&sh.b_empty[sb]);
      }
      tc_commit(&sh.acc_full);
    }
  } else if (warp >= 2) {
    // ===================== conversion warps, then epilogue =======================================
    const int ct = tid - 64;                         // 0..255
    if (ENC != ENC_BF16) {
      const int r = ct;                               // B-tile row of this thread (256 rows, 256 threads)
      bool ok = mbar_wait(&sh.scales_full, 0);
      if (!ok && lane == 0) { atomicExch(p.status, (unsigned)ERR_DEVICE_TIMEOUT); *abort_flag = 1; }
      for (int kc = 0; kc < nk && !*abort_flag; ++kc) {
        const int s = kc % kPStages, sb = kc % kBStages;
        ok = mbar_wait(&sh.p_full[s], (kc / kPStages) & 1);
        if (ok && kc >= kBStages) ok = mbar_wait(&sh.b_empty[sb], ((kc / kBStages) - 1) & 1);
        if (!ok) { if (lane == 0) { atomicExch(p.status, (unsigned)ERR_DEVICE_TIMEOUT); *abort_flag = 1; } break; }
        const float scale = sScales[r * groups + (kc >> 1)];
        const uint8_t* src = sP + s * kPackedBytes + r * kPackedRow;
        uint8_t* dstrow = sB + sb * kBTile + r * 128;
#pragma unroll
        for (int h = 0; h < 2; ++h) {                 // the two 32-wide halves of the k chunk
          uint32_t out[16];
          if (ENC == ENC_Q4) {
            convert_q4(*reinterpret_cast<const uint4*>(src + h * 16), scale, out);
          } else {
            convert_q8(*reinterpret_cast<const uint4*>(src + h * 32), *reinterpret_cast<const uint4*>(src + h * 32 + 16),
                       scale, out);
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int chunk = (h * 4 + i) ^ (r & 7);
            *reinterpret_cast<uint4*>(dstrow + chunk * 16) = make_uint4(out[4 * i], out[4 * i + 1], out[4 * i + 2], out[4 * i + 3]);
          }
        }
        fence_proxy_async();                         // generic-proxy writes -> visible to the tensor core
        __syncwarp();
        if (lane == 0) { mbar_arrive(&sh.b_full[sb]); mbar_arrive(&sh.p_empty[s]); }
      }
    }
    // ---- epilogue: warp quarter = warp % 4 (its 32 accumulator lanes), column half = (warp-2)/4 ---
    bool ok = !*abort_flag && mbar_wait(&sh.acc_full, 0);
    if (!ok && !*abort_flag && lane == 0) { atomicExch(p.status, (unsigned)ERR_DEVICE_TIMEOUT); *abort_flag = 1; }
    if (ok) {
      tc_fence_after();
      const int quarter = warp & 3, ch = (warp - 2) >> 2;
      for (int half = 0; half < (two ? 2 : 1); ++half) {
      const int row = half * BM + quarter * 32 + lane;   // route row inside the tile
      const uint32_t tbase = tmem + half * BN + ((uint32_t)(quarter * 32) << 16);
      const bool valid = row < nrows;
      const long long grow = (long long)row0 + row;
      if (MODE == 0) {
        // columns [0, BN/2) gate, [BN/2, BN) up; this warp: features ch*64 .. ch*64+63 in two parts
#pragma unroll
        for (int part = 0; part < 2; ++part) {
          uint32_t g[32], u[32];
          const int c0 = ch * 64 + part * 32;
          tmem_ld32(tbase + c0, g);
          tmem_ld32(tbase + BN / 2 + c0, u);
          tmem_ld_wait();
          if (valid) {
            __nv_bfloat16* dst = p.out + grow * p.out_stride + f0 + c0;
            uint32_t o[16];
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              const float a = silu_f32(__uint_as_float(g[j])) * __uint_as_float(u[j]);
              const float b = silu_f32(__uint_as_float(g[j + 1])) * __uint_as_float(u[j + 1]);
              const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
              o[j >> 1] = *reinterpret_cast<const uint32_t*>(&v);
            }
            if (p.permute_out) {
              // natural pairs (f0,f1)(f2,f3)(f4,f5)(f6,f7) -> (f0,f4)(f1,f5)(f2,f6)(f3,f7) per run of 8
#pragma unroll
              for (int q8 = 0; q8 < 4; ++q8) {
                const uint32_t a = o[4 * q8], b = o[4 * q8 + 1], c = o[4 * q8 + 2], d = o[4 * q8 + 3];
                o[4 * q8] = prmt(a, c, 0x5410); o[4 * q8 + 1] = prmt(a, c, 0x7632);
                o[4 * q8 + 2] = prmt(b, d, 0x5410); o[4 * q8 + 3] = prmt(b, d, 0x7632);
              }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
              reinterpret_cast<uint4*>(dst)[i] = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
          }
        }
      } else {
        const float wr = !valid ? 0.f : (p.route_weight ? p.route_weight[grow] : 1.f);
#pragma unroll
        for (int part = 0; part < 4; ++part) {
          uint32_t a[32];
          const int c0 = ch * 128 + part * 32;
          tmem_ld32(tbase + c0, a);
          tmem_ld_wait();
          if (valid) {
            __nv_bfloat16* dst = p.out + grow * p.out_stride + f0 + c0;
            uint32_t o[16];
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              const __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(a[j]) * wr, __uint_as_float(a[j + 1]) * wr);
              o[j >> 1] = *reinterpret_cast<const uint32_t*>(&v);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
              reinterpret_cast<uint4*>(dst)[i] = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
          }
        }
      }
      }
      tc_fence_before();
    }
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

template <int ENC>
constexpr size_t gemm_smem_bytes() {
  constexpr int packed = ENC == ENC_BF16 ? 0 : BN * (ENC == ENC_Q4 ? BK / 2 : BK);
  constexpr int nb = ENC == ENC_BF16 ? kInStages : kBStages;
  constexpr int np = ENC == ENC_Q4 ? 4 : 2;
  return (size_t)kInStages * (kHalves * BM * BK * 2) + (size_t)np * packed + (size_t)nb * BN * BK * 2 + BN * kMaxGroups * 4 + sizeof(GemmShared) + 1024;
}

// ---- tensor maps ----------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

bool make_map(CUtensorMap* map, CUtensorMapDataType type, int elem_bytes, const void* base, uint64_t inner,
              uint64_t rows, uint32_t box_inner, uint32_t box_rows, CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) { set_error("grouped: cuTensorMapEncodeTiled is not available"); return false; }
  const cuuint64_t dims[2] = {inner, rows};
  const cuuint64_t strides[1] = {inner * (uint64_t)elem_bytes};
  const cuuint32_t box[2] = {box_inner, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, type, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("grouped: cuTensorMapEncodeTiled failed with code %d", (int)r); return false; }
  return true;
}

template <int ENC, int MODE>
int launch_one(const GroupedParams& p, const CUtensorMap& ma, const CUtensorMap& mb0, const CUtensorMap& mb1,
               int n_tiles, cudaStream_t stream) {
  auto kernel = grouped_gemm_kernel<ENC, MODE>;
  constexpr size_t smem = gemm_smem_bytes<ENC>();
  static thread_local int configured = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured != dev) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { set_error("grouped: cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return ERR_LAUNCH; }
    configured = dev;
  }
  kernel<<<dim3(n_tiles, p.max_tiles), kGemmThreads, smem, stream>>>(ma, mb0, mb1, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("grouped: launch failed: %s", cudaGetErrorString(e)); return ERR_LAUNCH; }
  return ERR_NONE;
}

}  // namespace

int launch_grouped_gemm(const GroupedGemmArgs& a, cudaStream_t stream) {
  const int K = a.k;
  if (K % 128 || a.n_rows % (a.mode == 0 ? BN / 2 : BN) || a.total_rows <= 0 || a.max_tiles <= 0 ||
      (a.enc != ENC_BF16 && K > kMaxGroups * 128)) {
    set_error("grouped: unsupported shape (k %d, rows per expert %d)", K, a.n_rows);
    return ERR_BAD_ARGUMENT;
  }
  CUtensorMap ma, mb0, mb1;
  if (!make_map(&ma, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.act, (uint64_t)K, (uint64_t)a.total_rows, BK, BM,
                CU_TENSOR_MAP_SWIZZLE_128B))
    return ERR_LAUNCH;
  const uint64_t wrows = (uint64_t)a.num_experts * a.n_rows;
  const uint32_t box_rows = a.mode == 0 ? BN / 2 : BN;
  bool ok;
  if (a.enc == ENC_BF16) {
    ok = make_map(&mb0, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.w0, (uint64_t)K, wrows, BK, box_rows, CU_TENSOR_MAP_SWIZZLE_128B) &&
         make_map(&mb1, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.mode == 0 ? a.w1 : a.w0, (uint64_t)K, wrows, BK, box_rows,
                  CU_TENSOR_MAP_SWIZZLE_128B);
  } else {
    const uint64_t rowb = a.enc == ENC_Q4 ? K / 2 : K;
    const uint32_t boxb = a.enc == ENC_Q4 ? BK / 2 : BK;
    ok = make_map(&mb0, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.w0, rowb, wrows, boxb, box_rows, CU_TENSOR_MAP_SWIZZLE_NONE) &&
         make_map(&mb1, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.mode == 0 ? a.w1 : a.w0, rowb, wrows, boxb, box_rows,
                  CU_TENSOR_MAP_SWIZZLE_NONE);
  }
  if (!ok) return ERR_LAUNCH;
  GroupedParams p{};
  p.k = K; p.n_rows = a.n_rows;
  p.scales0 = a.s0; p.scales1 = a.s1;
  p.num_tiles = a.num_tiles; p.tile_expert = a.tile_expert; p.tile_row0 = a.tile_row0; p.tile_rows = a.tile_rows;
  p.max_tiles = a.max_tiles;
  p.out = a.out; p.out_stride = a.out_stride; p.route_weight = a.route_weight; p.permute_out = a.permute_out;
  p.status = a.status;
  const int n_tiles = a.n_rows / (a.mode == 0 ? BN / 2 : BN);
#define UMAQ_DISPATCH(E)                                                                       \
  return a.mode == 0 ? launch_one<E, 0>(p, ma, mb0, mb1, n_tiles, stream) : launch_one<E, 1>(p, ma, mb0, mb1, n_tiles, stream)
  if (a.enc == ENC_Q4) { UMAQ_DISPATCH(ENC_Q4); }
  if (a.enc == ENC_Q8) { UMAQ_DISPATCH(ENC_Q8); }
  if (a.enc == ENC_BF16) { UMAQ_DISPATCH(ENC_BF16); }
#undef UMAQ_DISPATCH
  set_error("grouped: unknown encoding %d", a.enc);
  return ERR_BAD_ARGUMENT;
}

}  // namespace umaq
