// Prefill / batched path: grouped-expert GEMMs on the 5th-generation tensor cores.
//
//   gate/up:  inter[r, f] = SiLU(x_r . Gate_e[f]) * (x_r . Up_e[f])        (GEMM 1, SwiGLU epilogue)
//   down:     y[r, n]     = w_r * (inter_r . Down_e[n])                    (GEMM 2, weighted epilogue)
//
// over the routes r sorted by expert e.  Replaces the reference's scalar-FMA prefill kernels
// (src/uma_qmoe/native/packed_q4_kernel.cu:560-776 Q4, :894-1099 Q8, launched from :1535-1641 and
// :1691-1762) and its torch._grouped_mm path for BF16 layers (src/uma_qmoe/native_backend.py:958-1005).
//
// Persistent CTAs (one per SM) walk the tile list; each tile is up to 256 routes x 256 columns: two M = 128, N = 256 accumulators
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
#include "tc.cuh"

namespace umaq {
namespace {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int kInStages = 3;          // TMA ring of activation tiles (2 x 128 rows x 64 k each)
constexpr int kBStages = 2;           // converted B tiles (256 rows x 64 k)
constexpr int kConvertWarps = 8;
constexpr int kGemmThreads = (3 + kConvertWarps) * 32;   // + activation TMA, MMA issuer, weight TMA
constexpr int kWeightWarp = 2 + kConvertWarps;
constexpr int kGatherWarps = 4;       // launched only when the kernel fetches its activation rows by index
constexpr int kGatherThreads = kGatherWarps * 32;
constexpr int kGatherAhead = 2;       // a gather thread hands a stage over two steps after issuing it (< kInStages)
constexpr int kHalves = 2;            // M = 128 accumulators per tile
constexpr int kTmemCols = BN * kHalves;   // 512: the whole tensor memory of the SM
constexpr int kMaxGroups = 16;        // quantised K <= 2048

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
  uint64_t sc_full[2];      // scales of the current / next tile
  uint64_t sc_empty[2];
  uint64_t acc_full;        // all MMAs of the tile are done
  uint64_t acc_empty;       // the epilogue has read the accumulators
  uint32_t tmem_base;
  int abort_flag;
  int gather_token[2 * BM];   // gather mode: token of every row of the current tile
};

struct TileInfo {
  int tile_n, expert, row0, nrows;
};

// Persistent: one CTA per SM walks the (row tile, column tile) list, column tile fastest, so that the
// CTAs running at the same time share activation rows in L2.  The TMA rings run ahead across tile
// boundaries: while the eight conversion warps drain the accumulators of tile i, the activation and
// packed-weight stages and the scales of tile i + 1 are already landing.
template <int ENC, int MODE>
__global__ void __launch_bounds__(kGemmThreads + kGatherThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b0,
                    const __grid_constant__ CUtensorMap map_b1, const __grid_constant__ CUtensorMap map_out,
                    const GroupedParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // layout: [A stages][packed stages][B stages][2 x scales][control]
  constexpr int kPackedRow = ENC == ENC_Q4 ? BK / 2 : BK;               // bytes of codes per row and k chunk
  constexpr int kPackedBytes = ENC == ENC_BF16 ? 0 : BN * kPackedRow;
  constexpr int kAHalf = BM * BK * 2, kATile = kHalves * kAHalf, kBTile = BN * BK * 2;
  constexpr int kPStages = ENC == ENC_Q4 ? 4 : 2;
  uint8_t* sA = smem_raw;
  uint8_t* sP = sA + kInStages * kATile;
  uint8_t* sB = sP + kPStages * kPackedBytes;
  constexpr int kNumB = ENC == ENC_BF16 ? kInStages : kBStages;
  float* sScales = reinterpret_cast<float*>(sB + kNumB * kBTile);
  GemmShared& sh = *reinterpret_cast<GemmShared*>(reinterpret_cast<uint8_t*>(sScales) + 2 * BN * kMaxGroups * 4);
  // The down GEMM of a quantised layer stages its results in shared memory (BF16 weight stages are TMA-fed across
  // tiles and never idle; the gate/up GEMM writes half as much per tile and measured slower staged, with plain
  // stores out of the staging area (0.495 against 0.485 ms) and with tensor stores (0.499)).
  constexpr bool kStaged = ENC != ENC_BF16 && MODE == 1;
  static_assert(kBStages >= 2 && kBTile >= kConvertWarps * 4096, "epilogue staging lives in two converted stages");

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int K = p.k;
  const int nk = K / BK;
  const int groups = K >> 7;
  const int n_col = p.n_rows / (MODE == 0 ? BN / 2 : BN);
  const int total = *p.num_tiles * n_col;
  const int first = blockIdx.x, step = gridDim.x;
  volatile int* abort_flag = &sh.abort_flag;
  // Gather mode (gate/up GEMM only): the activation tile of a stage is written by kGatherThreads threads with
  // 16-byte cp.async copies, row by row from wherever the row's token lives, in the same swizzled layout the TMA
  // produces; the stage's barrier then counts those threads (plus the TMA warp for a BF16 weight tile).
  const bool gather = MODE == 0 && p.gather_route != nullptr;

  if (tid == 0) {
    const uint32_t in_count = gather ? kGatherThreads + (ENC == ENC_BF16 ? 1 : 0) : 1;
    for (int s = 0; s < kInStages; ++s) { mbar_init(&sh.in_full[s], in_count); mbar_init(&sh.in_empty[s], 1); }
    for (int s = 0; s < kMaxPStages; ++s) { mbar_init(&sh.p_full[s], 1); mbar_init(&sh.p_empty[s], kConvertWarps); }
    for (int s = 0; s < kBStages; ++s) { mbar_init(&sh.b_full[s], kConvertWarps); mbar_init(&sh.b_empty[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&sh.sc_full[s], 1); mbar_init(&sh.sc_empty[s], kConvertWarps); }
    mbar_init(&sh.acc_full, 1);
    mbar_init(&sh.acc_empty, kConvertWarps);
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

  auto tile_of = [&](int it) {
    TileInfo t;
    const int tile_m = it / n_col;
    t.tile_n = it - tile_m * n_col;
    t.expert = p.tile_expert[tile_m]; t.row0 = p.tile_row0[tile_m]; t.nrows = p.tile_rows[tile_m];
    return t;
  };
  // first weight row of the tile inside the concatenated projection
  // MODE 0: columns [0,128) = gate rows f0.., [128,256) = up rows f0..;  MODE 1: 256 down rows n0..
  auto weight_row = [&](const TileInfo& t) {
    return (long long)t.expert * p.n_rows + t.tile_n * (MODE == 0 ? BN / 2 : BN);
  };
  auto fail = [&]() { atomicExch(p.status, (unsigned)ERR_DEVICE_TIMEOUT); *abort_flag = 1; };

  if (warp == 0) {
    // ===================== TMA producer: activation tiles (and BF16 weight tiles) ==================
    if (lane == 0 && !(gather && ENC != ENC_BF16)) {
      uint32_t kidx = 0;
      int inflight_from = 0;
      for (int it = first; it < total && !*abort_flag; it += step) {
        const TileInfo t = tile_of(it);
        const bool two = t.nrows > BM;
        const long long wrow0 = weight_row(t);
        bool ok = true;
        for (int kc = 0; kc < nk; ++kc, ++kidx) {
          const uint32_t s = kidx % kInStages, use = kidx / kInStages;
          if (use > 0 && !mbar_wait(&sh.in_empty[s], (use - 1) & 1)) { ok = false; break; }
          const uint32_t bytes = (gather ? 0 : (two ? kATile : kAHalf)) + (ENC == ENC_BF16 ? kBTile : 0);
          mbar_expect_tx(&sh.in_full[s], bytes);
          if (!gather) {
            tma_load_2d(sA + s * kATile, &map_a, kc * BK, t.row0, &sh.in_full[s]);
            if (two) tma_load_2d(sA + s * kATile + kAHalf, &map_a, kc * BK, t.row0 + BM, &sh.in_full[s]);
          }
          if (ENC == ENC_BF16) {
            uint8_t* dst = sB + s * kBTile;
            if (MODE == 0) {
              tma_load_2d(dst, &map_b0, kc * BK, (int)wrow0, &sh.in_full[s]);
              tma_load_2d(dst + (BN / 2) * BK * 2, &map_b1, kc * BK, (int)wrow0, &sh.in_full[s]);
            } else {
              tma_load_2d(dst, &map_b0, kc * BK, (int)wrow0, &sh.in_full[s]);
            }
          }
        }
        if (!ok) { fail(); break; }
      }
      // after an abort nobody consumes: wait (bounded) for the copies still in flight
      if (*abort_flag) {
        inflight_from = kidx > (uint32_t)kInStages ? (int)kidx - kInStages : 0;
        for (uint32_t k2 = inflight_from; k2 < kidx; ++k2) mbar_wait(&sh.in_full[k2 % kInStages], (k2 / kInStages) & 1);
      }
    }
  } else if (warp == kWeightWarp) {
    // ===================== TMA producer: scales and packed weight rows, on their own deeper ring ====
    if (lane == 0 && ENC != ENC_BF16) {
      uint32_t kidx = 0;
      int seq = 0;
      for (int it = first; it < total && !*abort_flag; it += step, ++seq) {
        const TileInfo t = tile_of(it);
        const long long wrow0 = weight_row(t);
        const int sb = seq & 1;
        if (seq >= 2 && !mbar_wait(&sh.sc_empty[sb], ((seq >> 1) - 1) & 1)) { fail(); break; }
        float* dst_sc = sScales + sb * BN * kMaxGroups;
        const uint32_t half_bytes = (uint32_t)(MODE == 0 ? BN / 2 : BN) * groups * 4;
        mbar_expect_tx(&sh.sc_full[sb], MODE == 0 ? 2 * half_bytes : half_bytes);
        bulk_g2s(dst_sc, p.scales0 + wrow0 * groups, half_bytes, &sh.sc_full[sb]);
        if (MODE == 0) bulk_g2s(dst_sc + (BN / 2) * groups, p.scales1 + wrow0 * groups, half_bytes, &sh.sc_full[sb]);
        bool ok = true;
        for (int kc = 0; kc < nk; ++kc, ++kidx) {
          const uint32_t s = kidx % kPStages, use = kidx / kPStages;
          if (use > 0 && !mbar_wait(&sh.p_empty[s], (use - 1) & 1)) { ok = false; break; }
          mbar_expect_tx(&sh.p_full[s], kPackedBytes);
          uint8_t* dst = sP + s * kPackedBytes;
          if (MODE == 0) {
            tma_load_2d(dst, &map_b0, kc * kPackedRow, (int)wrow0, &sh.p_full[s]);
            tma_load_2d(dst + (BN / 2) * kPackedRow, &map_b1, kc * kPackedRow, (int)wrow0, &sh.p_full[s]);
          } else {
            tma_load_2d(dst, &map_b0, kc * kPackedRow, (int)wrow0, &sh.p_full[s]);
          }
        }
        if (!ok) { fail(); break; }
      }
      if (*abort_flag) {
        for (int sb = 0; sb < 2; ++sb) mbar_wait(&sh.sc_full[sb], 0);   // bounded; a barrier never armed just times out
        const uint32_t from = kidx > (uint32_t)kPStages ? kidx - kPStages : 0;
        for (uint32_t k2 = from; k2 < kidx; ++k2) mbar_wait(&sh.p_full[k2 % kPStages], (k2 / kPStages) & 1);
      }
    }
  } else if (warp > kWeightWarp) {
    // ===================== gather producers: 128 threads write every activation tile =========================
    // A row of a stage is 64 k = 128 bytes = eight 16-byte chunks; chunk c of row r lands at r * 128 +
    // ((c ^ (r & 7)) << 4), the 128-byte swizzle the MMA descriptors expect.  Thread j copies chunk j & 7 of
    // rows (j >> 3) + 16 i: eight neighbouring lanes read one row's 128 contiguous bytes, so every copy
    // instruction of a warp covers four whole lines.  Rows past the tile's end are zero-filled.  cp.async writes
    // go through the generic proxy: a thread waits for its own copies of a stage (the younger stages stay in
    // flight), fences them towards the async proxy and arrives.
    const int pt = tid - (kWeightWarp + 1) * 32;          // 0 .. 127
    const int c = pt & 7, rbase = pt >> 3;                // rows rbase, rbase + 16, ...: all have r & 7 == rbase & 7
    const uint32_t dst_off = (uint32_t)rbase * 128 + (uint32_t)((c ^ (rbase & 7)) << 4);
    uint32_t kidx = 0, published = 0;
    bool ok = true;
    auto publish = [&]() {
      fence_proxy_async();
      mbar_arrive(&sh.in_full[published % kInStages]);
      ++published;
    };
    for (int it = first; it < total; it += step) {
      // Everybody has read the previous tile's table; and the threads agree whether to go on (a thread that gave up
      // on a wait, or saw the abort flag, must not leave the others waiting at this barrier).
      if (named_bar_or(1, kGatherThreads, !ok || *abort_flag != 0)) break;
      const TileInfo t = tile_of(it);
      const bool two = t.nrows > BM;
      // the tile's token of every row, shared by the gather threads (-1: no such row)
      sh.gather_token[pt] = pt < t.nrows ? p.gather_route[t.row0 + pt] / p.gather_top_k : -1;
      sh.gather_token[pt + BM] = pt + BM < t.nrows ? p.gather_route[t.row0 + BM + pt] / p.gather_top_k : -1;
      named_bar_sync(1, kGatherThreads);
      int tok[2 * BM / 16];
#pragma unroll
      for (int i = 0; i < 2 * BM / 16; ++i) tok[i] = sh.gather_token[rbase + 16 * i];
      const uint8_t* base = reinterpret_cast<const uint8_t*>(p.gather_src) + c * 16;
      for (int kc = 0; kc < nk; ++kc, ++kidx) {
        // first hand over the stage issued two steps ago (its copies have had two steps to land), so that the
        // MMA issuer never waits for this thread's wait on a free slot below
        if (kidx >= (uint32_t)kGatherAhead) { cp_async_wait<kGatherAhead - 1>(); publish(); }
        const uint32_t s = kidx % kInStages, use = kidx / kInStages;
        if (use > 0 && !mbar_wait(&sh.in_empty[s], (use - 1) & 1)) { ok = false; break; }
        uint8_t* dst = sA + s * kATile + dst_off;
        const uint8_t* col = base + kc * 128;
#pragma unroll
        for (int i = 0; i < BM / 16; ++i)
          cp_async16(dst + i * 2048, col + (size_t)(tok[i] < 0 ? 0 : tok[i]) * K * 2, tok[i] >= 0);
        if (two) {
#pragma unroll
          for (int i = BM / 16; i < 2 * BM / 16; ++i)
            cp_async16(dst + i * 2048, col + (size_t)(tok[i] < 0 ? 0 : tok[i]) * K * 2, tok[i] >= 0);
        }
        cp_async_commit();
      }
    }
    if (!ok && lane == 0) fail();
    cp_async_wait<0>();                                  // also on the abort path: nothing of this thread stays in flight
    if (ok && !*abort_flag)
      while (published < kidx) publish();
  } else if (warp == 1) {
    // ===================== MMA issuer ============================================================
    if (lane == 0) {
      uint32_t kidx = 0;
      int seq = 0;
      for (int it = first; it < total && !*abort_flag; it += step, ++seq) {
        const bool two = p.tile_rows[it / n_col] > BM;
        if (seq >= 1 && !mbar_wait(&sh.acc_empty, (seq - 1) & 1)) { fail(); break; }
        tc_fence_after();
        bool ok = true;
        for (int kc = 0; kc < nk; ++kc, ++kidx) {
          const uint32_t s = kidx % kInStages;
          const uint32_t sb = ENC == ENC_BF16 ? s : kidx % kBStages;
          ok = mbar_wait(&sh.in_full[s], (kidx / kInStages) & 1);
          if (ok && ENC != ENC_BF16) ok = mbar_wait(&sh.b_full[sb], (kidx / kBStages) & 1);
          if (!ok) break;
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
        if (!ok) { fail(); break; }
        tc_commit(&sh.acc_full);
      }
    }
  } else if (warp >= 2) {
    // ===================== conversion warps, then epilogue, tile after tile =========================
    const int ct = tid - 64;                         // 0..255
    const int r = ct;                                 // B-tile row of this thread (256 rows, 256 threads)
    uint32_t kidx = 0;
    int seq = 0;
    for (int it = first; it < total && !*abort_flag; it += step, ++seq) {
      const TileInfo t = tile_of(it);
      const bool two = t.nrows > BM;
      const int f0 = t.tile_n * (MODE == 0 ? BN / 2 : BN);
      bool ok = true;
      if (ENC != ENC_BF16) {
        const int sbuf = seq & 1;
        ok = mbar_wait(&sh.sc_full[sbuf], (seq >> 1) & 1);
        const float* sc = sScales + sbuf * BN * kMaxGroups + r * groups;
        for (int kc = 0; kc < nk && ok; ++kc, ++kidx) {
          const uint32_t s = kidx % kPStages, sb = kidx % kBStages, use = kidx / kBStages;
          ok = mbar_wait(&sh.p_full[s], (kidx / kPStages) & 1);
          if (ok && use > 0) ok = mbar_wait(&sh.b_empty[sb], (use - 1) & 1);
          if (!ok) break;
          const float scale = sc[kc >> 1];
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
        if (ok) {
          __syncwarp();
          if (lane == 0) mbar_arrive(&sh.sc_empty[sbuf]);
        }
      }
      // ---- epilogue: warp quarter = warp % 4 (its 32 accumulator lanes), column half = (warp-2)/4 ---
      if (ok) ok = mbar_wait(&sh.acc_full, seq & 1);
      if (!ok) { if (lane == 0) fail(); break; }
      tc_fence_after();
      // The accumulator reads are software-pipelined: the tcgen05.ld of chunk c + 1 is in flight while chunk c
      // is converted and stored, and the accumulators are handed back to the MMA issuer as soon as the last
      // chunk is in registers, before its arithmetic and stores.
      const int quarter = warp & 3, ch = (warp - 2) >> 2;
      const int nchunks = two ? 8 : 4;                   // per warp: {half 0, half 1} x 4 chunks
      const uint32_t tq = tmem + ((uint32_t)(quarter * 32) << 16);
      // Staged results leave through shared memory so that a warp's store instruction covers whole 128-byte
      // lines (one row per lane costs 32 partly written lines per instruction).  The staging bytes are
      // the rows this warp itself writes in the two converted-weight stages, idle between the tile's last MMA and
      // this warp's next conversion: no other warp and no TMA touches them.
      uint8_t* const stage0 = sB + (warp - 2) * 4096;
      auto stage_piece_of = [&](int i) { return stage0 + i * kBTile; };
      auto release = [&]() {
        tc_fence_before();                               // every tcgen05.ld of this tile is complete (wait::ld)
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh.acc_empty);
      };
      if (MODE == 0) {
        // columns [0, BN/2) gate, [BN/2, BN) up; this warp: features ch*64 .. ch*64+63, 16 per chunk
        uint32_t g[2][16], u[2][16];
        tmem_ld16(tq + ch * 64, g[0]);
        tmem_ld16(tq + BN / 2 + ch * 64, u[0]);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          if (c < nchunks) {
            tmem_ld_wait();
            if (c + 1 < nchunks) {
              const uint32_t nb = tq + ((c + 1) >> 2) * BN + ch * 64 + ((c + 1) & 3) * 16;
              tmem_ld16(nb, g[(c + 1) & 1]);
              tmem_ld16(nb + BN / 2, u[(c + 1) & 1]);
            } else {
              release();
            }
            const int row = (c >> 2) * BM + quarter * 32 + lane;   // route row inside the tile
            if (row < t.nrows && !(p.debug & 2)) {
              const uint32_t (&gg)[16] = g[c & 1];
              const uint32_t (&uu)[16] = u[c & 1];
              __nv_bfloat16* dst = p.out + ((long long)t.row0 + row) * p.out_stride + f0 + ch * 64 + (c & 3) * 16;
              uint32_t o[8];
#pragma unroll
              for (int j = 0; j < 16; j += 2) {
                const float a = silu_f32(__uint_as_float(gg[j])) * __uint_as_float(uu[j]);
                const float b = silu_f32(__uint_as_float(gg[j + 1])) * __uint_as_float(uu[j + 1]);
                const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
                o[j >> 1] = *reinterpret_cast<const uint32_t*>(&v);
              }
              if (p.permute_out) {
                // natural pairs (f0,f1)(f2,f3)(f4,f5)(f6,f7) -> (f0,f4)(f1,f5)(f2,f6)(f3,f7) per run of 8
#pragma unroll
                for (int q8 = 0; q8 < 2; ++q8) {
                  const uint32_t a = o[4 * q8], b = o[4 * q8 + 1], c2 = o[4 * q8 + 2], d = o[4 * q8 + 3];
                  o[4 * q8] = prmt(a, c2, 0x5410); o[4 * q8 + 1] = prmt(a, c2, 0x7632);
                  o[4 * q8 + 2] = prmt(b, d, 0x5410); o[4 * q8 + 3] = prmt(b, d, 0x7632);
                }
              }
              if (!(p.debug & 1)) {
                reinterpret_cast<uint4*>(dst)[0] = make_uint4(o[0], o[1], o[2], o[3]);
                reinterpret_cast<uint4*>(dst)[1] = make_uint4(o[4], o[5], o[6], o[7]);
              }
            }
          }
        }
      } else {
        // this warp: columns ch*128 .. ch*128+127, 32 per chunk
        uint32_t acc[2][32];
        tmem_ld32(tq + ch * 128, acc[0]);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          if (c < nchunks) {
            tmem_ld_wait();
            if (c + 1 < nchunks) tmem_ld32(tq + ((c + 1) >> 2) * BN + ch * 128 + ((c + 1) & 3) * 32, acc[(c + 1) & 1]);
            else release();
            const int row = (c >> 2) * BM + quarter * 32 + lane;
            if ((kStaged || row < t.nrows) && !(p.debug & 2)) {
              const long long grow = (long long)t.row0 + row;
              const float wr = row < t.nrows && p.route_weight ? p.route_weight[grow] : 1.f;
              const uint32_t (&a)[32] = acc[c & 1];
              uint32_t o[16];
#pragma unroll
              for (int j = 0; j < 32; j += 2) {
                const __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(a[j]) * wr, __uint_as_float(a[j + 1]) * wr);
                o[j >> 1] = *reinterpret_cast<const uint32_t*>(&v);
              }
              if (kStaged) {
                // two chunks = 32 rows x 128 B per piece, pieces in turn: 16-byte slot q of row r at r*128 + ((q ^ r&7) << 4)
                if (!(c & 1)) {                              // the piece's previous tensor store has read it
                  if (lane == 0) bulk_wait_read<1>();
                  __syncwarp();
                }
                uint8_t* piece = stage_piece_of((c >> 1) & 1) + lane * 128;
#pragma unroll
                for (int i = 0; i < 4; ++i)
                  *reinterpret_cast<uint4*>(piece + ((((c & 1) * 4 + i) ^ (lane & 7)) << 4)) =
                      make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
              } else if (!(p.debug & 1)) {
                __nv_bfloat16* dst = p.out + grow * p.out_stride + f0 + ch * 128 + (c & 3) * 32;
#pragma unroll
                for (int i = 0; i < 4; ++i)
                  reinterpret_cast<uint4*>(dst)[i] = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
              }
            }
            if (kStaged && (c & 1)) {
              // A piece is full.  A whole group of 32 rows leaves by one tensor store (asynchronous: the warp goes on
              // with the next chunks while the copy engine reads the piece); a ragged group by plain stores, eight
              // lanes writing one row's 128 contiguous bytes, four rows per instruction.  One bulk group per piece
              // either way, so that "at most one group pending" always means the piece about to be written is free.
              const int group_row = (c >> 2) * BM + quarter * 32;
              const bool by_tma = p.tma_out && group_row + 32 <= t.nrows && !(p.debug & 4);
              if (by_tma) fence_proxy_async();               // this lane's staging writes -> visible to the copy engine
              __syncwarp();
              if (by_tma) {
                if (lane == 0) {
                  if (!(p.debug & 3))
                    tma_store_2d(&map_out, f0 + ch * 128 + ((c & 3) >> 1) * 64, t.row0 + group_row, stage_piece_of((c >> 1) & 1));
                  bulk_commit();
                }
              } else if (lane == 0) {
                bulk_commit();
              }
              if (!by_tma && !(p.debug & 3)) {
                const int q = lane & 7;
                const uint8_t* piece = stage_piece_of((c >> 1) & 1);
                __nv_bfloat16* dst = p.out + f0 + ch * 128 + ((c & 3) >> 1) * 64 + q * 8;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  const int lr = 4 * j + (lane >> 3);
                  const int orow = (c >> 2) * BM + quarter * 32 + lr;
                  if (orow < t.nrows) {
                    const uint4 v = *reinterpret_cast<const uint4*>(piece + lr * 128 + ((q ^ (lr & 7)) << 4));
                    *reinterpret_cast<uint4*>(dst + ((long long)t.row0 + orow) * p.out_stride) = v;
                  }
                }
              }
            }
          }
        }
        if (kStaged) {                                       // before this warp's next conversion overwrites its rows
          if (lane == 0) bulk_wait_read<0>();                // (waiting for the last store one k step later measured the same)
          __syncwarp();
        }
      }
    }
  }
  if (kStaged && warp >= 2 && warp < 2 + kConvertWarps && lane == 0) bulk_wait_all();   // this thread's tensor stores
  tc_fence_before();
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
  return (size_t)kInStages * (kHalves * BM * BK * 2) + (size_t)np * packed + (size_t)nb * BN * BK * 2 + 2 * BN * kMaxGroups * 4 + sizeof(GemmShared) + 1024;
}

template <int ENC, int MODE>
int launch_one(const GroupedParams& p, const CUtensorMap& ma, const CUtensorMap& mb0, const CUtensorMap& mb1,
               const CUtensorMap& mo, int n_tiles, cudaStream_t stream) {
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
  (void)n_tiles;
  kernel<<<dim3(sm_count()), kGemmThreads + (MODE == 0 && p.gather_route ? kGatherThreads : 0), smem, stream>>>(ma, mb0, mb1, mo, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("grouped: launch failed: %s", cudaGetErrorString(e)); return ERR_LAUNCH; }
  return ERR_NONE;
}

}  // namespace

// Which kernel a caller gets that does not ask for one (variant 0), from measurements on B200.  Quantised
// encodings: this file's kernel at every size (the CTA-pair kernel's barrier hops between two CTAs need a deeper
// pipeline than shared memory holds next to the conversion ring: 0.66 against 0.48 ms for the OLMoE Q4 gate/up
// GEMM at 8192 tokens).  BF16 weights need no conversion ring, and there the pair kernel, which drains one
// accumulator while the next tile is multiplied, wins on large batches: Qwen shape, 8192 tokens, both GEMMs 0.510
// against 0.530 ms; OLMoE shape 0.687 against 0.725 ms; at 128 tokens it loses 1.5 %.
constexpr long long kPairMinRows = 16384;
static bool takes_pair_kernel(const GroupedGemmArgs& a) {
  return a.variant == 2 || (a.variant == 0 && a.enc == ENC_BF16 && a.total_rows >= kPairMinRows);
}
bool grouped_gemm_can_gather(const GroupedGemmArgs& a) { return a.mode == 0 && !takes_pair_kernel(a); }
int launch_grouped_gemm(const GroupedGemmArgs& a, cudaStream_t stream) {
  if (takes_pair_kernel(a)) {
    if (a.gather_route) { set_error("grouped: the CTA-pair kernel takes gathered activation rows"); return ERR_BAD_ARGUMENT; }
    return launch_grouped_gemm_pair(a, stream);
  }
  return launch_grouped_gemm_single(a, stream);
}

int launch_grouped_gemm_single(const GroupedGemmArgs& a, cudaStream_t stream) {
  const int K = a.k;
  if (K % 128 || a.n_rows % (a.mode == 0 ? BN / 2 : BN) || a.total_rows <= 0 || a.max_tiles <= 0 ||
      (a.enc != ENC_BF16 && K > kMaxGroups * 128)) {
    set_error("grouped: unsupported shape (k %d, rows per expert %d)", K, a.n_rows);
    return ERR_BAD_ARGUMENT;
  }
  if (a.gather_route && (a.mode != 0 || a.gather_top_k < 1)) { set_error("grouped: rows are fetched by index only for the gate/up GEMM"); return ERR_BAD_ARGUMENT; }
  // with rows fetched by index `act` is [tokens, k] and the kernel never uses the activation map: any valid map will do
  CUtensorMap ma, mb0, mb1, mo;
  if (!make_map(&ma, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.act, (uint64_t)K, (uint64_t)(a.gather_route ? BM : a.total_rows), BK, BM,
                CU_TENSOR_MAP_SWIZZLE_128B))
    return ERR_LAUNCH;
  const uint64_t wrows = (uint64_t)a.num_experts * a.n_rows;
  const uint32_t box_rows = a.mode == 0 ? BN / 2 : BN;
  bool ok, tma_out = false;
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
    // the epilogue's tensor stores of 32 rows x 64 columns need a dense [total_rows, n_rows] BF16 output at a 16-byte
    // boundary; any other output is written with plain stores
    tma_out = a.mode == 1 && a.out_stride == a.n_rows && !(reinterpret_cast<uintptr_t>(a.out) & 15);
    if (ok && tma_out)
      ok = make_map(&mo, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.out, (uint64_t)a.n_rows, (uint64_t)a.total_rows, 64, 32,
                    CU_TENSOR_MAP_SWIZZLE_128B);
  }
  if (!tma_out) mo = ma;                                   // never used: any valid map
  if (!ok) return ERR_LAUNCH;
  GroupedParams p{};
  p.k = K; p.n_rows = a.n_rows;
  p.scales0 = a.s0; p.scales1 = a.s1;
  p.num_tiles = a.num_tiles; p.tile_expert = a.tile_expert; p.tile_row0 = a.tile_row0; p.tile_rows = a.tile_rows;
  p.max_tiles = a.max_tiles;
  p.out = a.out; p.out_stride = a.out_stride; p.route_weight = a.route_weight; p.permute_out = a.permute_out;
  { static const int dbg = [] { const char* v = std::getenv("UMAQ_GEMM_DEBUG"); return v ? std::atoi(v) : 0; }(); p.debug = dbg; }
  p.tma_out = tma_out;
  p.status = a.status;
  p.gather_route = a.gather_route; p.gather_top_k = a.gather_top_k; p.gather_src = static_cast<const __nv_bfloat16*>(a.act);
  const int n_tiles = a.n_rows / (a.mode == 0 ? BN / 2 : BN);
#define UMAQ_DISPATCH(E)                                                                       \
  return a.mode == 0 ? launch_one<E, 0>(p, ma, mb0, mb1, mo, n_tiles, stream) : launch_one<E, 1>(p, ma, mb0, mb1, mo, n_tiles, stream)
  if (a.enc == ENC_Q4) { UMAQ_DISPATCH(ENC_Q4); }
  if (a.enc == ENC_Q8) { UMAQ_DISPATCH(ENC_Q8); }
  if (a.enc == ENC_BF16) { UMAQ_DISPATCH(ENC_BF16); }
#undef UMAQ_DISPATCH
  set_error("grouped: unknown encoding %d", a.enc);
  return ERR_BAD_ARGUMENT;
}

}  // namespace umaq
