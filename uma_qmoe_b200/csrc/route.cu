// Routing side of the prefill path: the fused router, the stable expert sort that replaces the
// reference's host-side argsort / bincount / cumsum (src/uma_qmoe/native_backend.py:531-543), the
// row gather that feeds the grouped GEMM and the ordered top-k combine that replaces
// reduce_topk_route_output_kernel (src/uma_qmoe/native/packed_q4_kernel.cu:1349-1365) with the
// accumulation order of the reference's CPU path (src/uma_qmoe/custom_op.py:312-338).
#include "grouped.cuh"

#include <cstdlib>

#include "common.cuh"

namespace umaq {
namespace {

// ---- router: logits = bf16(x . Wr^T), softmax in float32, top-k, optional renormalisation ----------
// The arithmetic of the Hugging Face OlmoeTopKRouter / Qwen2MoeTopKRouter the reference calls at
// src/uma_qmoe/compressed_loader.py:59 and src/uma_qmoe/qwen_compressed_loader.py:73.  One warp per
// token; ties go to the lowest expert index.
constexpr int kRouterWarps = 8;

__global__ void __launch_bounds__(kRouterWarps * 32)
router_topk_kernel(const RouterArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  float* probs = reinterpret_cast<float*>(smem) + (threadIdx.x >> 5) * a.experts;   // per-warp scratch
  const int lane = threadIdx.x & 31;
  const int token = blockIdx.x * kRouterWarps + (threadIdx.x >> 5);
  if (token >= a.tokens) return;
  const int H = a.hidden, E = a.experts;
  const __nv_bfloat16* xr = a.x + (size_t)token * H;
  // logits: BF16 products are exact in float32; they are summed in float64 so that the BF16
  // rounding of the logit matches an exactly rounded dot product (a float32 sum is off by one BF16
  // ulp on ~0.2 % of the logits, which moves near-tied experts across the top-k boundary)
  for (int e = 0; e < E; ++e) {
    const __nv_bfloat16* wr = a.weight + (size_t)e * H;
    double acc = 0.0;
    for (int k = lane * 8; k < H; k += 256) {
      const uint4 xv = *reinterpret_cast<const uint4*>(xr + k);
      const uint4 wv = *reinterpret_cast<const uint4*>(wr + k);
      const uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w}, ws[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc += (double)(__uint_as_float(xs[i] << 16) * __uint_as_float(ws[i] << 16));
        acc += (double)(__uint_as_float(xs[i] & 0xffff0000u) * __uint_as_float(ws[i] & 0xffff0000u));
      }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) {
      const float l = bf16_round((float)acc);       // F.linear output in BF16
      probs[e] = l;
      if (a.out_logits) a.out_logits[(size_t)token * E + e] = __float2bfloat16_rn(l);
    }
  }
  __syncwarp();
  // softmax over the experts in float32
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, probs[e]);
#pragma unroll
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) {
    const float v = expf(probs[e] - mx);
    probs[e] = v;
    sum += v;
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  __syncwarp();
  for (int e = lane; e < E; e += 32) probs[e] = probs[e] / sum;
  __syncwarp();
  // top-k by repeated arg-max (value descending, index ascending)
  float topsum = 0.f;
  float myval = 0.f;
  long long myidx = 0;
  for (int j = 0; j < a.top_k; ++j) {
    float best = -1.f;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = probs[e];
      if (v > best) { best = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == j) { myval = best; myidx = bi; }
    topsum += best;
    if (lane == 0) probs[bi] = -2.f;
    __syncwarp();
  }
  if (lane < a.top_k) {
    a.out_weights[(size_t)token * a.top_k + lane] = a.renormalize ? myval / topsum : myval;
    a.out_indices[(size_t)token * a.top_k + lane] = myidx;
  }
}

// Softmax over the experts in float32, top-k by repeated arg-max (value descending, index ascending),
// optional renormalisation; `probs` holds the BF16-rounded logits of one token on entry.  One warp.
__device__ __forceinline__ void softmax_topk_warp(float* probs, int E, int top_k, int renormalize, int lane,
                                                  float* out_w, long long* out_i) {
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, probs[e]);
#pragma unroll
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) {
    const float v = expf(probs[e] - mx);
    probs[e] = v;
    sum += v;
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  __syncwarp();
  for (int e = lane; e < E; e += 32) probs[e] = probs[e] / sum;
  __syncwarp();
  float topsum = 0.f, myval = 0.f;
  long long myidx = 0;
  for (int j = 0; j < top_k; ++j) {
    float best = -1.f;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = probs[e];
      if (v > best) { best = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == j) { myval = best; myidx = bi; }
    topsum += best;
    if (lane == 0) probs[bi] = -2.f;
    __syncwarp();
  }
  if (lane < top_k) {
    out_w[lane] = renormalize ? myval / topsum : myval;
    out_i[lane] = myidx;
  }
}

// The same softmax / top-k for E <= 64 and top_k <= 8 with eight lanes per token, so that a warp handles four
// tokens at once: lane s of a token's group keeps experts s, s + 8, ... in registers.  Ties go to the lower expert.
__device__ __forceinline__ void softmax_topk_oct(const float* logits, bool live, int E, int top_k, int renormalize, int lane,
                                                 float* out_w, long long* out_i) {
  const int s = lane & 7;
  float v[8];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int e = s + 8 * j;
    v[j] = (live && e < E) ? logits[e] : -INFINITY;
    mx = fmaxf(mx, v[j]);
  }
#pragma unroll
  for (int o = 4; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    v[j] = (s + 8 * j < E) ? expf(v[j] - mx) : 0.f;
    sum += v[j];
  }
#pragma unroll
  for (int o = 4; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = (s + 8 * j < E) ? v[j] / sum : -2.f;
  float topsum = 0.f, myval = 0.f;
  int myidx = 0;
  for (int it = 0; it < top_k; ++it) {
    float best = -1.f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (v[j] > best) { best = v[j]; bi = s + 8 * j; }
#pragma unroll
    for (int o = 4; o; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (s == it) { myval = best; myidx = bi; }
    topsum += best;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (bi == s + 8 * j) v[j] = -2.f;
  }
  if (live && s < top_k) {
    out_w[s] = renormalize ? myval / topsum : myval;
    out_i[s] = myidx;
  }
}

// Tiled router for E <= 64: a CTA takes 32 tokens and all experts, stages 128-wide k chunks of x and
// Wr in shared memory (rows padded by 16 bytes against bank conflicts); thread (ty, tx) accumulates
// tokens {ty, ty+16} x experts {tx, tx+16, tx+32, tx+48}.  The BF16 products are exact in float32;
// runs of 32 are summed in float32 and the runs in float64, which keeps the BF16 rounding of the
// logit equal to that of an exactly rounded dot product in all but ~1 logit in 10^4.
constexpr int kRtTokens = 32, kRtExperts = 64, kRtChunk = 128, kRtPitch = kRtChunk + 8;

__global__ void __launch_bounds__(256) router_tiled_kernel(const RouterArgs a) {
  __shared__ __align__(16) __nv_bfloat16 xs[kRtTokens][kRtPitch];
  __shared__ __align__(16) __nv_bfloat16 ws[kRtExperts][kRtPitch];
  __shared__ float logit[kRtTokens][kRtExperts];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int token0 = blockIdx.x * kRtTokens;
  const int H = a.hidden, E = a.experts;
  double acc[2][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0;
  for (int kc = 0; kc < H; kc += kRtChunk) {
    __syncthreads();
    for (int v = tid; v < kRtTokens * (kRtChunk / 8); v += 256) {
      const int r = v >> 4, c = v & 15;
      uint4 w = make_uint4(0, 0, 0, 0);
      if (token0 + r < a.tokens) w = *reinterpret_cast<const uint4*>(a.x + (size_t)(token0 + r) * H + kc + c * 8);
      *reinterpret_cast<uint4*>(&xs[r][c * 8]) = w;
    }
    for (int v = tid; v < kRtExperts * (kRtChunk / 8); v += 256) {
      const int r = v >> 4, c = v & 15;
      uint4 w = make_uint4(0, 0, 0, 0);
      if (r < E) w = *reinterpret_cast<const uint4*>(a.weight + (size_t)r * H + kc + c * 8);
      *reinterpret_cast<uint4*>(&ws[r][c * 8]) = w;
    }
    __syncthreads();
#pragma unroll
    for (int run = 0; run < kRtChunk / 32; ++run) {
      float part[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) part[i][j] = 0.f;
#pragma unroll
      for (int kk = 0; kk < 32; kk += 8) {
        uint4 xv[2], wv[4];
#pragma unroll
        for (int i = 0; i < 2; ++i) xv[i] = *reinterpret_cast<const uint4*>(&xs[ty + 16 * i][run * 32 + kk]);
#pragma unroll
        for (int j = 0; j < 4; ++j) wv[j] = *reinterpret_cast<const uint4*>(&ws[tx + 16 * j][run * 32 + kk]);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const uint32_t xw[4] = {xv[i].x, xv[i].y, xv[i].z, xv[i].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t ww[4] = {wv[j].x, wv[j].y, wv[j].z, wv[j].w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              part[i][j] = fmaf(__uint_as_float(xw[q] << 16), __uint_as_float(ww[q] << 16), part[i][j]);
              part[i][j] = fmaf(__uint_as_float(xw[q] & 0xffff0000u), __uint_as_float(ww[q] & 0xffff0000u), part[i][j]);
            }
          }
        }
      }
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += (double)part[i][j];
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float l = bf16_round((float)acc[i][j]);            // F.linear output in BF16
      logit[ty + 16 * i][tx + 16 * j] = l;
      const int t = token0 + ty + 16 * i, e = tx + 16 * j;
      if (a.out_logits && t < a.tokens && e < E) a.out_logits[(size_t)t * E + e] = __float2bfloat16_rn(l);
    }
  __syncthreads();
  const int warp = tid >> 5, lane = tid & 31;
  for (int r = warp; r < kRtTokens; r += 8) {
    const int t = token0 + r;
    if (t < a.tokens)
      softmax_topk_warp(logit[r], E, a.top_k, a.renormalize, lane, a.out_weights + (size_t)t * a.top_k,
                        a.out_indices + (size_t)t * a.top_k);
  }
}

// Router for a handful of tokens (decode steps, short prompts; E <= 64): latency is everything here -- at one token
// the tiled kernel above is a single CTA walking 16 k-chunks with two barriers each and takes 65 us, more than the
// expert kernels of the same layer.  Here a cluster of eight CTAs takes four tokens: CTA r of the cluster owns
// experts 8 r .. 8 r + 7, a warp takes half of one expert's row for all four tokens (every load of the router
// matrix is in flight at once: one round trip to L2 per CTA), the two halves meet in shared memory, and the logits
// go to CTA 0 of the cluster through distributed shared memory, which runs the softmax / top-k after a cluster
// barrier.  Products of BF16 values are exact in float32; eight of them are summed in float32 and the runs in
// float64, which makes the BF16 rounding of the logit that of the exact dot product (the other router kernels'
// bound, with shorter runs).
constexpr int kRsTokens = 4, kRsWarps = 16, kRsCluster = 8, kRsExperts = 8;      // experts per CTA
// Most tokens this kernel takes (UMAQ_ROUTER_SMALL_MAX overrides).  Measured on B200, 64 experts: 6 us up to 32
// tokens, 8 us at 128, 16 us at 256, 26 us at 512 against a constant 12.7 us of the tensor-core kernel with
// 32 tokens per CTA.
constexpr int kRouterSmallMax = 192;
// From this many tokens on the tensor-core router takes 64 tokens per CTA instead of 32 (UMAQ_ROUTER_WIDE_MIN
// overrides).  Measured: 32 per CTA 12.7 us up to 4096 tokens and 24 us once its CTAs need a second wave
// (148 SMs x 32 tokens), 64 per CTA 19.4 to 20 us at any size up to 9472 tokens.
constexpr int kRouterWideMin = 4737;

__device__ __forceinline__ float dot8_bf16(const uint4& x, const uint4& w) {
  const uint32_t xs[4] = {x.x, x.y, x.z, x.w}, ws[4] = {w.x, w.y, w.z, w.w};
  float run = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    run = fmaf(__uint_as_float(xs[i] << 16), __uint_as_float(ws[i] << 16), run);
    run = fmaf(__uint_as_float(xs[i] & 0xffff0000u), __uint_as_float(ws[i] & 0xffff0000u), run);
  }
  return run;
}

__global__ void __cluster_dims__(kRsCluster, 1, 1) __launch_bounds__(kRsWarps * 32)
router_small_kernel(const RouterArgs a) {
  extern __shared__ __align__(16) uint8_t rs_smem[];
  __shared__ float logit[kRsTokens][kRtExperts + 1];                      // used in CTA 0 of the cluster
  __shared__ double part[kRsWarps][kRsTokens];
  const int H = a.hidden, E = a.experts, chunks = H >> 3, half_chunks = chunks >> 1;   // 16-byte chunks
  uint4* xs = reinterpret_cast<uint4*>(rs_smem);                          // [kRsTokens][chunks]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint32_t cr;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(cr));
  // A kernel launched behind this one with programmatic stream serialisation (the decode kernels are) may become
  // resident now and run its prologue; it still waits for this grid to finish before it reads the routes.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // a CTA may write into another CTA's shared memory only once that CTA runs: arrive now, wait before the stores
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  const int token0 = (blockIdx.x / kRsCluster) * kRsTokens, nt = min(kRsTokens, a.tokens - token0);
  const uint4* xg = reinterpret_cast<const uint4*>(a.x + (size_t)token0 * H);     // consecutive token rows
  for (int v = tid; v < nt * chunks; v += kRsWarps * 32) xs[v] = xg[v];
  __syncthreads();
  const int e = (int)cr * kRsExperts + (warp & 7), half = warp >> 3;
  double acc[kRsTokens];
#pragma unroll
  for (int t = 0; t < kRsTokens; ++t) acc[t] = 0.0;
  if (e < E) {
    const uint4* wr = reinterpret_cast<const uint4*>(a.weight + (size_t)e * H);
    const int end = (half + 1) * half_chunks;
    for (int base = half * half_chunks; base < end; base += 256) {        // up to 8 chunks per lane and pass
      uint4 wv[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int c = base + j * 32 + lane;
        wv[j] = c < end ? __ldg(wr + c) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int c = base + j * 32 + lane;
        if (c < end) {
#pragma unroll
          for (int t = 0; t < kRsTokens; ++t)
            if (t < nt) acc[t] += (double)dot8_bf16(xs[t * chunks + c], wv[j]);
        }
      }
    }
  }
#pragma unroll
  for (int t = 0; t < kRsTokens; ++t) {
#pragma unroll
    for (int o = 16; o; o >>= 1) acc[t] += __shfl_xor_sync(0xffffffffu, acc[t], o);
    if (lane == 0) part[warp][t] = acc[t];
  }
  __syncthreads();
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  if (tid < kRsExperts * kRsTokens) {                                      // both halves of (expert, token) -> logit
    const int ee = tid & 7, t = tid >> 3, ge = (int)cr * kRsExperts + ee;
    if (ge < E && t < nt) {
      const float l = bf16_round((float)(part[ee][t] + part[ee + 8][t]));  // F.linear output in BF16
      uint32_t remote;
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(&logit[t][ge])), "r"(0));
      asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(l) : "memory");
      if (a.out_logits) a.out_logits[(size_t)(token0 + t) * E + ge] = __float2bfloat16_rn(l);
    }
  }
  // every CTA's logits are in CTA 0's shared memory after this barrier; CTA 0 outlives the others' stores
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  if (cr != 0) return;
  if (a.top_k <= 8) {
    if (warp == 0) {                                                       // eight lanes per token, four tokens
      const int r = lane >> 3;
      const bool live = r < nt;
      const int t = token0 + (live ? r : 0);
      softmax_topk_oct(logit[live ? r : 0], live, E, a.top_k, a.renormalize, lane, a.out_weights + (size_t)t * a.top_k,
                       a.out_indices + (size_t)t * a.top_k);
    }
  } else if (warp < nt) {
    const int t = token0 + warp;
    softmax_topk_warp(logit[warp], E, a.top_k, a.renormalize, lane, a.out_weights + (size_t)t * a.top_k,
                      a.out_indices + (size_t)t * a.top_k);
  }
}

// Tensor-core router for batches (E <= 64): a CTA takes MT = 32 or 64 tokens and all experts.
// x and Wr stream through a 6-stage cp.async ring of 128-wide k chunks (16-byte chunks XOR-swizzled by
// row against bank conflicts); warp (g, h) = (token group of 16, expert half or quarter) runs
// mma.sync.m16n8k16 BF16 with ldmatrix fragments.  The BF16 products are exact in the FP32 accumulator;
// a chunk's 128 products are summed by the tensor core in float32, the chunk sums in float64, so the
// BF16 rounding of the logit equals that of an exactly rounded dot product in all but about one logit
// in 10^4 (the same bound as the tiled kernel).  The logits then go through the same softmax / top-k.
// MT = tokens per CTA: 64 for the largest batches (every CTA re-reads the router matrix from L2), 32 below: the loop
// is one CTA's dependent chain whose length goes with MT, so more and shorter CTAs finish sooner.
constexpr int kRmChunk = 128, kRmStages = 6;
constexpr int kRmTile = 64 * kRmChunk * 2;                 // 16 KiB: 64 rows x 256 bytes (the router matrix's chunk)
constexpr int rm_smem_bytes(int mt) { return kRmStages * (mt * kRmChunk * 2 + kRmTile); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}

template <int MT>
__global__ void __launch_bounds__(256) router_mma_kernel(const RouterArgs a) {
  extern __shared__ __align__(128) uint8_t rm_smem[];
  constexpr int kGroups = MT / 16;                         // token groups of 16
  constexpr int kPerGroup = 8 / kGroups;                   // warps sharing a token group
  constexpr int kWarpExperts = 64 / kPerGroup;             // experts of a warp: 32 (MT 64) or 16 (MT 32)
  constexpr int NJ = kWarpExperts / 8;                     // n-tiles of a warp
  constexpr int kXTile = MT * kRmChunk * 2, kStage = kXTile + kRmTile;
  constexpr int kXPieces = MT * 16 / 256;                  // 16-byte pieces of the token tile per thread and chunk
  static_assert(MT == 64 || MT == 32, "token tile");
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int token0 = blockIdx.x * MT;
  const int H = a.hidden, E = a.experts, nchunks = H / kRmChunk;
  const int g = warp / kPerGroup, h = warp % kPerGroup;    // tokens 16g.., experts kWarpExperts*h..

  // per thread: four 16-byte pieces of the token tile and of the router matrix per chunk; everything that does not
  // depend on the chunk is computed once (the loop is one CTA's dependent chain, every instruction in it counts)
  const uint8_t* x_src[4];
  const uint8_t* w_src[4];
  uint32_t piece_dst[4];
  bool x_ok[4], w_ok[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int v = tid + i * 256, r = v >> 4, c = v & 15;
    const int t = token0 + r;
    x_ok[i] = t < a.tokens;
    w_ok[i] = r < E;
    x_ok[i] = x_ok[i] && i < kXPieces;
    x_src[i] = reinterpret_cast<const uint8_t*>(a.x + (size_t)(x_ok[i] ? t : 0) * H + c * 8);
    w_src[i] = reinterpret_cast<const uint8_t*>(a.weight + (size_t)(w_ok[i] ? r : 0) * H + c * 8);
    piece_dst[i] = (uint32_t)(r * 256 + ((c ^ (r & 7)) << 4));
  }
  auto load_chunk = [&](int kc, int stage) {
    uint8_t* xs = rm_smem + stage * kStage;
    uint8_t* ws = xs + kXTile;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (i < kXPieces) cp_async16(xs + piece_dst[i], x_src[i] + kc * (kRmChunk * 2), x_ok[i]);
      cp_async16(ws + piece_dst[i], w_src[i] + kc * (kRmChunk * 2), w_ok[i]);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  double acc[NJ][4];
#pragma unroll
  for (int j = 0; j < NJ; ++j)
#pragma unroll
    for (int q = 0; q < 4; ++q) acc[j][q] = 0.0;

  for (int s = 0; s < kRmStages - 1; ++s) {
    if (s < nchunks) load_chunk(s, s); else asm volatile("cp.async.commit_group;" ::: "memory");
  }
  // ldmatrix row / chunk of this lane: A = 16 tokens x 16 k, B = 2 n-tiles (16 experts) x 16 k
  const int a_row = g * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, a_sel = lane >> 4;
  const int b_row = h * kWarpExperts + (lane & 7) + ((lane >> 4) & 1) * 8, b_sel = (lane >> 3) & 1;
  uint32_t a_off[kRmChunk / 16], b_off[kRmChunk / 16];   // swizzled offsets of this lane's ldmatrix rows, per k step
#pragma unroll
  for (int k16 = 0; k16 < kRmChunk / 16; ++k16) {
    a_off[k16] = (uint32_t)(a_row * 256 + (((k16 * 2 + a_sel) ^ (a_row & 7)) << 4));
    b_off[k16] = (uint32_t)(kXTile + b_row * 256 + (((k16 * 2 + b_sel) ^ (b_row & 7)) << 4));
  }
  for (int kc = 0; kc < nchunks; ++kc) {
    asm volatile("cp.async.wait_group %0;" ::"n"(kRmStages - 2) : "memory");
    __syncthreads();                                       // chunk kc has landed; chunk kc - 1's buffer is free
    if (kc + kRmStages - 1 < nchunks) load_chunk(kc + kRmStages - 1, (kc + kRmStages - 1) % kRmStages);
    else asm volatile("cp.async.commit_group;" ::: "memory");
    const uint32_t xs = smem_u32(rm_smem + (kc % kRmStages) * kStage);
    float part[NJ][4];
#pragma unroll
    for (int j = 0; j < NJ; ++j)
#pragma unroll
      for (int q = 0; q < 4; ++q) part[j][q] = 0.f;
#pragma unroll
    for (int k16 = 0; k16 < kRmChunk / 16; ++k16) {
      uint32_t a0, a1, a2, a3, b[8];
      ldmatrix_x4(xs + a_off[k16], a0, a1, a2, a3);
      ldmatrix_x4(xs + b_off[k16], b[0], b[1], b[2], b[3]);
      if (NJ == 4) ldmatrix_x4(xs + b_off[k16] + 16 * 256, b[4], b[5], b[6], b[7]);
#pragma unroll
      for (int j = 0; j < NJ; ++j) mma_bf16_16816(part[j], a0, a1, a2, a3, b[2 * j], b[2 * j + 1]);
    }
#pragma unroll
    for (int j = 0; j < NJ; ++j)
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[j][q] += (double)part[j][q];
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();                                         // every warp is done with the ring: reuse it for logits
  float (*logit)[kRtExperts + 1] = reinterpret_cast<float (*)[kRtExperts + 1]>(rm_smem);
#pragma unroll
  for (int j = 0; j < NJ; ++j)
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int r = g * 16 + (lane >> 2) + (q >> 1) * 8, e = h * kWarpExperts + j * 8 + (lane & 3) * 2 + (q & 1);
      const float l = bf16_round((float)acc[j][q]);        // F.linear output in BF16
      logit[r][e] = l;
      const int t = token0 + r;
      if (a.out_logits && t < a.tokens && e < E) a.out_logits[(size_t)t * E + e] = __float2bfloat16_rn(l);
    }
  __syncthreads();
  if (a.top_k <= 8) {
    for (int r = warp * 4 + (lane >> 3); r < MT; r += 32) {            // the loop count is the same for every lane
      const int t = token0 + r;
      const bool live = t < a.tokens;
      softmax_topk_oct(logit[r], live, E, a.top_k, a.renormalize, lane, a.out_weights + (size_t)(live ? t : 0) * a.top_k,
                       a.out_indices + (size_t)(live ? t : 0) * a.top_k);
    }
    return;
  }
  for (int r = warp; r < MT; r += 8) {
    const int t = token0 + r;
    if (t < a.tokens)
      softmax_topk_warp(logit[r], E, a.top_k, a.renormalize, lane, a.out_weights + (size_t)t * a.top_k,
                        a.out_indices + (size_t)t * a.top_k);
  }
}

// ---- stable expert sort of the routes, one CTA --------------------------------------------------------
// Route i = token * top_k + slot.  Warp w owns a contiguous chunk of routes; a per-warp histogram and
// a scan over (expert, warp) give every warp its first position inside each expert's run, and ranks
// inside a 32-route batch come from __match_any_sync, so equal experts keep their route order.
constexpr int kSortThreads = 1024;
constexpr int kTileRows = 256;       // routes per grouped-GEMM tile (two M = 128 accumulators)
constexpr int kMaxSortExperts = 128;

__device__ __forceinline__ int load_expert(const void* idx, int idx64, long long i) {
  return idx64 ? (int)reinterpret_cast<const long long*>(idx)[i] : reinterpret_cast<const int*>(idx)[i];
}

// Offsets and the tile list from the per-expert counts in count[] (shared memory).  Thread 0 scans the counts
// in shared memory only; the global stores (offsets, a few tiles per expert) are then spread over the threads.
// start[e] receives the first sorted position of expert e.  All threads of the CTA call it.
__device__ __forceinline__ void emit_offsets_and_tiles(const SortArgs& a, const int* count, int* start, int* tile_base,
                                                       bool write, int tid, int nthreads) {
  const int E = a.experts;
  if (tid == 0) {
    int run = 0, tiles = 0;
    for (int e = 0; e < E; ++e) {
      const int c = count[e];
      start[e] = run;
      tile_base[e] = tiles;
      run += c;
      tiles += (c + kTileRows - 1) / kTileRows;
    }
    start[E] = run;
    tile_base[E] = tiles;
  }
  __syncthreads();
  if (write) {
    for (int e = tid; e <= E; e += nthreads) a.offsets[e] = start[e];
    for (int e = tid; e < E; e += nthreads) {
      const int c = start[e + 1] - start[e];
      int t = tile_base[e];
      for (int r = 0; r < c && t < a.max_tiles; r += kTileRows, ++t) {
        a.tile_expert[t] = e; a.tile_row0[t] = start[e] + r; a.tile_rows[t] = min(kTileRows, c - r);
      }
    }
    if (tid == 0) *a.num_tiles = min(tile_base[E], a.max_tiles);
  }
}

__global__ void __launch_bounds__(kSortThreads) route_sort_kernel(const SortArgs a) {
  __shared__ int hist[32][kMaxSortExperts];     // per-warp counts, then per-warp running positions
  __shared__ int total[kMaxSortExperts + 1];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int E = a.experts;
  const long long routes = (long long)a.tokens * a.top_k;
  const long long chunk = ((routes + 31) / 32 + 31) / 32 * 32;     // routes per warp, multiple of 32
  const long long begin = min(routes, warp * chunk), end = min(routes, begin + chunk);
  for (int i = tid; i < 32 * kMaxSortExperts; i += kSortThreads) (&hist[0][0])[i] = 0;
  __syncthreads();
  bool bad = false;
  for (long long i = begin + lane; i < end; i += 32) {
    const int e = load_expert(a.indices, a.idx64, i);
    if (e == -1) continue;                       // an absent route (padding of a fixed-capacity exchange)
    if (e < 0 || e >= E) bad = true; else atomicAdd(&hist[warp][e], 1);
  }
  if (bad) atomicExch(a.status, (unsigned)ERR_BAD_ARGUMENT);
  __syncthreads();
  // per expert: exclusive scan over the warps; totals
  if (tid < E) {
    int run = 0;
    for (int w = 0; w < 32; ++w) { const int c = hist[w][tid]; hist[w][tid] = run; run += c; }
    total[tid] = run;
    a.counts[tid] = run;
  }
  __syncthreads();
  __shared__ int start[kMaxSortExperts + 1], tile_base[kMaxSortExperts + 1];
  emit_offsets_and_tiles(a, total, start, tile_base, true, tid, kSortThreads);
  __syncthreads();
  if (tid < E) total[tid] = start[tid];
  __syncthreads();
  for (long long base = begin; base < end; base += 32) {
    const long long i = base + lane;
    const bool live = i < end;
    int e = live ? load_expert(a.indices, a.idx64, i) : -1 - lane;     // distinct keys for idle lanes
    if (live && (e < 0 || e >= E)) { e = -1 - lane; }
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    if (e >= 0) {
      const int pos = total[e] + hist[warp][e] + rank;
      a.sorted_route[pos] = (int)i;
      a.route_pos[i] = pos;
      a.sorted_weight[pos] = a.weights[i];
    } else if (live) {
      a.route_pos[i] = -1;                       // absent or invalid route: no row, the combine skips it
    }
    __syncwarp();
    if (e >= 0 && rank == 0) hist[warp][e] += __popc(peers);
    __syncwarp();
  }
}

// ---- the same sort over several CTAs (large route counts) ------------------------------------------------
// Pass 1: every CTA histograms its contiguous chunk of kChunk routes.  Pass 2: every CTA rebuilds the
// per-expert totals and its own starting positions from the chunk histograms (a few thousand loads),
// then places its routes exactly like the single-CTA kernel.  CTA 0 also writes counts, offsets and
// the tile list.
constexpr int kChunk = 2048;

__global__ void __launch_bounds__(kSortThreads) route_hist_kernel(const SortArgs a, int* __restrict__ chunk_hist) {
  __shared__ int hist[kMaxSortExperts];
  const int tid = threadIdx.x, E = a.experts;
  const long long routes = (long long)a.tokens * a.top_k;
  const long long begin = (long long)blockIdx.x * kChunk, end = min(routes, begin + kChunk);
  if (tid < kMaxSortExperts) hist[tid] = 0;
  __syncthreads();
  bool bad = false;
  for (long long i = begin + tid; i < end; i += kSortThreads) {
    const int e = load_expert(a.indices, a.idx64, i);
    if (e == -1) continue;
    if (e < 0 || e >= E) bad = true; else atomicAdd(&hist[e], 1);
  }
  if (bad) atomicExch(a.status, (unsigned)ERR_BAD_ARGUMENT);
  __syncthreads();
  if (tid < E) chunk_hist[(size_t)blockIdx.x * E + tid] = hist[tid];
}

__global__ void __launch_bounds__(kSortThreads) route_place_kernel(const SortArgs a, const int* __restrict__ chunk_hist,
                                                                   int chunks) {
  __shared__ int hist[32][kMaxSortExperts];     // per-warp counts of this chunk, then running positions
  __shared__ int total[kMaxSortExperts + 1];    // per-expert totals, then first position of this chunk
  __shared__ int before[kMaxSortExperts];       // routes of the expert in earlier chunks
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, E = a.experts;
  const long long routes = (long long)a.tokens * a.top_k;
  const long long cbegin = (long long)blockIdx.x * kChunk, cend = min(routes, cbegin + kChunk);
  const long long per_warp = kChunk / 32;
  const long long begin = min(cend, cbegin + warp * per_warp), end = min(cend, begin + per_warp);
  for (int i = tid; i < 32 * kMaxSortExperts; i += kSortThreads) (&hist[0][0])[i] = 0;
  if (tid < E) {
    int all = 0, prev = 0;
    for (int c2 = 0; c2 < chunks; ++c2) {
      const int v = chunk_hist[(size_t)c2 * E + tid];
      if (c2 < (int)blockIdx.x) prev += v;
      all += v;
    }
    total[tid] = all;
    before[tid] = prev;
    if (blockIdx.x == 0) a.counts[tid] = all;
  }
  __syncthreads();
  for (long long i = begin + lane; i < end; i += 32) {
    const int e = load_expert(a.indices, a.idx64, i);
    if (e >= 0 && e < E) atomicAdd(&hist[warp][e], 1);
  }
  __syncthreads();
  if (tid < E) {
    int run = 0;
    for (int w = 0; w < 32; ++w) { const int c2 = hist[w][tid]; hist[w][tid] = run; run += c2; }
  }
  __syncthreads();
  __shared__ int start[kMaxSortExperts + 1], tile_base[kMaxSortExperts + 1];
  emit_offsets_and_tiles(a, total, start, tile_base, blockIdx.x == 0, tid, kSortThreads);
  __syncthreads();
  if (tid < E) total[tid] = start[tid] + before[tid];
  __syncthreads();
  for (long long base = begin; base < end; base += 32) {
    const long long i = base + lane;
    const bool live = i < end;
    int e = live ? load_expert(a.indices, a.idx64, i) : -1 - lane;
    if (live && (e < 0 || e >= E)) e = -1 - lane;
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    if (e >= 0) {
      const int pos = total[e] + hist[warp][e] + rank;
      a.sorted_route[pos] = (int)i;
      a.route_pos[i] = pos;
      a.sorted_weight[pos] = a.weights[i];
    } else if (live) {
      a.route_pos[i] = -1;                       // absent or invalid route: no row, the combine skips it
    }
    __syncwarp();
    if (e >= 0 && rank == 0) hist[warp][e] += __popc(peers);
    __syncwarp();
  }
}

// ---- gather: sorted_x[i] = x[sorted_route[i] / top_k], optionally in the permuted K order ------------------
// One warp per row, eight rows per CTA; a lane keeps up to eight 16-byte loads in flight before it stores.
constexpr int kGatherRows = 8;
__global__ void __launch_bounds__(kGatherRows * 32)
gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ sorted_route, int top_k,
                   long long routes, int hidden, int permute, __nv_bfloat16* __restrict__ out,
                   const int* __restrict__ valid_rows) {
  const long long i = (long long)blockIdx.x * kGatherRows + (threadIdx.x >> 5);
  if (i >= routes || (valid_rows && i >= *valid_rows)) return;     // fewer present routes than the launch covers
  const int lane = threadIdx.x & 31;
  const int token = sorted_route ? sorted_route[i] / top_k : (int)i;
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)token * hidden);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)i * hidden);
  const int words = hidden / 8;
  for (int base = 0; base < words; base += 256) {
    uint4 w[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int v = base + j * 32 + lane;
      if (v < words) w[j] = src[v];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int v = base + j * 32 + lane;
      if (v < words) {
        uint4 q = w[j];
        if (permute) {
          // (e0,e1)(e2,e3)(e4,e5)(e6,e7) -> (e0,e4)(e1,e5)(e2,e6)(e3,e7)
          const uint32_t a = q.x, b = q.y, c = q.z, d = q.w;
          q.x = prmt(a, c, 0x5410); q.y = prmt(a, c, 0x7632);
          q.z = prmt(b, d, 0x5410); q.w = prmt(b, d, 0x7632);
        }
        dst[v] = q;
      }
    }
  }
}

// ---- expert-parallel dispatch: rows into fixed-capacity per-destination segments ---------------------------
// Sorted route s (key = owner * experts_per_rank + local expert) goes to slot owner * capacity + j, j its
// rank among the routes for that owner.  Slot gets the activation row, meta = {local expert, weight bits};
// the route remembers its slot for the combine.  Routes beyond the capacity get slot -1 and raise *overflow.
// The caller pre-fills meta with -1 so that unused slots read as absent routes on the receiving rank.
__global__ void ep_pack_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ sorted_route,
                               const int* __restrict__ sorted_key, const float* __restrict__ sorted_weight,
                               const int* __restrict__ offsets, int top_k, int hidden, int per_rank, int capacity,
                               __nv_bfloat16* __restrict__ send_rows, int* __restrict__ send_meta,
                               int* __restrict__ route_slot, int* __restrict__ overflow) {
  const int s = blockIdx.x;
  const int key = sorted_key[s], owner = key / per_rank;
  const int j = s - offsets[owner * per_rank];
  const int route = sorted_route[s];
  if (j >= capacity) {
    if (threadIdx.x == 0) { route_slot[route] = -1; atomicOr(overflow, 1); }
    return;
  }
  const long long slot = (long long)owner * capacity + j;
  if (threadIdx.x == 0) {
    send_meta[2 * slot] = key - owner * per_rank;
    send_meta[2 * slot + 1] = __float_as_int(sorted_weight[s]);
    route_slot[route] = (int)slot;
  }
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(route / top_k) * hidden);
  uint4* dst = reinterpret_cast<uint4*>(send_rows + (size_t)slot * hidden);
  for (int v = threadIdx.x; v < hidden / 8; v += blockDim.x) dst[v] = src[v];
}

// ---- combine: ordered BF16 running sum over a token's routes, then the Qwen shared branch -----------------
// out[t] = (((0 + c_e1) + c_e2) + ...) with e1 < e2 < ... and every partial sum rounded to BF16; the
// contributions are already BF16 (GEMM 2 epilogue).  With a shared expert: + bf16(sigmoid(bf16(x . wg))
// * shared_out[t]), as QuantizedQwenMoEBlock does after the operator
// (src/uma_qmoe/qwen_compressed_loader.py:82-85).
__global__ void __launch_bounds__(256, 4)
combine_kernel(const __nv_bfloat16* __restrict__ weighted, const void* __restrict__ indices, int idx64,
               const int* __restrict__ route_pos, int top_k, int hidden, int experts,
               const __nv_bfloat16* __restrict__ shared_out, const __nv_bfloat16* __restrict__ x,
               const __nv_bfloat16* __restrict__ gate_vec, __nv_bfloat16* __restrict__ out, const __grid_constant__ SegmentedOut seg) {
  __shared__ int order_pos[8];
  __shared__ int present;
  __shared__ float red[8];
  __shared__ float gate;
  const int t = blockIdx.x, tid = threadIdx.x;
  __shared__ int raw_e[8], raw_q[8];
  if (tid < top_k) {                               // eight independent loads instead of a serial chain
    raw_e[tid] = load_expert(indices, idx64, (long long)t * top_k + tid);
    raw_q[tid] = route_pos[(long long)t * top_k + tid];
  }
  __syncthreads();
  if (tid < 8) {
    // rank of every present route among the present ones by (expert, slot): a stable sort by counting.
    // Absent routes (expert -1), expert ids outside [0, experts) and routes without a row (position -1)
    // contribute nothing, as in the reference's kernels (src/uma_qmoe/native/packed_q4_kernel.cu:176).
    const bool valid = tid < top_k && raw_e[tid] >= 0 && raw_e[tid] < experts && raw_q[tid] >= 0;
    int rank = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const bool vj = j < top_k && raw_e[j] >= 0 && raw_e[j] < experts && raw_q[j] >= 0;
      rank += vj && (raw_e[j] < raw_e[tid] || (raw_e[j] == raw_e[tid] && j < tid));
    }
    if (valid) order_pos[rank] = raw_q[tid];
    const unsigned m = __ballot_sync(0xffu, valid);
    if (tid == 0) present = __popc(m);
  }
  if (shared_out) {
    float acc = 0.f;
    for (int k = tid; k < hidden; k += 256)
      acc += __bfloat162float(x[(size_t)t * hidden + k]) * __bfloat162float(gate_vec[k]);
#pragma unroll
    for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((tid & 31) == 0) red[tid >> 5] = acc;
  }
  __syncthreads();
  if (shared_out && tid == 0) {
    float s = 0.f;
    for (int i = 0; i < 8; ++i) s += red[i];
    s = bf16_round(s);
    gate = bf16_round(1.f / (1.f + expf(-s)));
  }
  __syncthreads();
  // all of a column pair's contributions are loaded first (independent loads), then summed in order
  const int n = present;
  __nv_bfloat16* dst = out + (size_t)t * hidden;
  if (seg.rows > 0) {                              // segmented output, possibly in a peer GPU's memory
    if (seg.skip_empty && n == 0) return;
    dst = seg.ptr[t / seg.rows] + (size_t)(seg.row0 + t % seg.rows) * hidden;
  }
  unsigned rows[8];                               // row starts in 16-byte words (fewer registers than pointers)
#pragma unroll
  for (int s = 0; s < 8; ++s) rows[s] = (unsigned)(((size_t)order_pos[s < n ? s : 0] * hidden) >> 3);
  const uint4* wbase = reinterpret_cast<const uint4*>(weighted);
  for (int c = tid * 8; c < hidden; c += 2048) {        // 16 bytes per thread and row (hidden % 8 == 0)
    uint4 v[8];
#pragma unroll
    for (int s = 0; s < 8; ++s)
      if (s < n) v[s] = wbase[rows[s] + (c >> 3)];
    float r[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) r[e] = 0.f;
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      if (s < n) {
        const uint32_t w[4] = {v[s].x, v[s].y, v[s].z, v[s].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          r[2 * e] = bf16_round(r[2 * e] + __uint_as_float(w[e] << 16));
          r[2 * e + 1] = bf16_round(r[2 * e + 1] + __uint_as_float(w[e] & 0xffff0000u));
        }
      }
    }
    if (shared_out) {
      const uint4 sv = *reinterpret_cast<const uint4*>(shared_out + (size_t)t * hidden + c);
      const uint32_t w[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        r[2 * e] = bf16_round(r[2 * e] + bf16_round(gate * __uint_as_float(w[e] << 16)));
        r[2 * e + 1] = bf16_round(r[2 * e + 1] + bf16_round(gate * __uint_as_float(w[e] & 0xffff0000u)));
      }
    }
    uint4 o;
    __nv_bfloat162 p0 = __floats2bfloat162_rn(r[0], r[1]), p1 = __floats2bfloat162_rn(r[2], r[3]);
    __nv_bfloat162 p2 = __floats2bfloat162_rn(r[4], r[5]), p3 = __floats2bfloat162_rn(r[6], r[7]);
    o.x = *reinterpret_cast<uint32_t*>(&p0); o.y = *reinterpret_cast<uint32_t*>(&p1);
    o.z = *reinterpret_cast<uint32_t*>(&p2); o.w = *reinterpret_cast<uint32_t*>(&p3);
    *reinterpret_cast<uint4*>(dst + c) = o;
  }
}

// The same ordered sum without a shared expert, one warp per token: no shared memory and no block barrier, the
// order of the routes found with shuffles.  A token with one or two present routes (an expert-parallel rank's
// share) costs a warp a few hundred cycles instead of a block three barriers.
constexpr int kCombineWarps = 8;
__global__ void __launch_bounds__(kCombineWarps * 32)
combine_warp_kernel(const __nv_bfloat16* __restrict__ weighted, const void* __restrict__ indices, int idx64,
                    const int* __restrict__ route_pos, int tokens, int top_k, int hidden, int experts,
                    __nv_bfloat16* __restrict__ out, const __grid_constant__ SegmentedOut seg) {
  const int lane = threadIdx.x & 31;
  const long long t = (long long)blockIdx.x * kCombineWarps + (threadIdx.x >> 5);
  if (t >= tokens) return;                                   // the whole warp
  int e = -1, q = -1;
  if (lane < top_k) {
    e = load_expert(indices, idx64, t * top_k + lane);
    q = route_pos[t * top_k + lane];
  }
  const bool valid = lane < top_k && e >= 0 && e < experts && q >= 0;
  int rank = 0;                                               // among the present routes, by (expert, slot)
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int ej = __shfl_sync(0xffffffffu, e, j);
    const bool vj = __shfl_sync(0xffffffffu, (int)valid, j);
    rank += vj && (ej < e || (ej == e && j < lane));
  }
  const int n = __popc(__ballot_sync(0xffffffffu, valid));
  __nv_bfloat16* dst = out + (size_t)t * hidden;
  if (seg.rows > 0) {                                         // segmented output, possibly in a peer GPU's memory
    if (seg.skip_empty && n == 0) return;
    dst = seg.ptr[t / seg.rows] + (size_t)(seg.row0 + t % seg.rows) * hidden;
  }
  unsigned rows[8];                                           // row starts in 16-byte words
#pragma unroll
  for (int s = 0; s < 8; ++s) {
    const unsigned m = __ballot_sync(0xffffffffu, valid && rank == s);
    const int qs = __shfl_sync(0xffffffffu, q, m ? __ffs(m) - 1 : 0);
    rows[s] = s < n ? (unsigned)(((size_t)qs * hidden) >> 3) : 0u;
  }
  const uint4* wbase = reinterpret_cast<const uint4*>(weighted);
  for (int c = lane; c < (hidden >> 3); c += 32) {            // 16 bytes per lane and row
    uint4 v[8];
#pragma unroll
    for (int s = 0; s < 8; ++s)
      if (s < n) v[s] = wbase[rows[s] + c];
    float r[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) r[i] = 0.f;
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      if (s < n) {
        const uint32_t w[4] = {v[s].x, v[s].y, v[s].z, v[s].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          r[2 * i] = bf16_round(r[2 * i] + __uint_as_float(w[i] << 16));
          r[2 * i + 1] = bf16_round(r[2 * i + 1] + __uint_as_float(w[i] & 0xffff0000u));
        }
      }
    }
    uint4 o;
    __nv_bfloat162 p0 = __floats2bfloat162_rn(r[0], r[1]), p1 = __floats2bfloat162_rn(r[2], r[3]);
    __nv_bfloat162 p2 = __floats2bfloat162_rn(r[4], r[5]), p3 = __floats2bfloat162_rn(r[6], r[7]);
    o.x = *reinterpret_cast<uint32_t*>(&p0); o.y = *reinterpret_cast<uint32_t*>(&p1);
    o.z = *reinterpret_cast<uint32_t*>(&p2); o.w = *reinterpret_cast<uint32_t*>(&p3);
    reinterpret_cast<uint4*>(dst)[c] = o;
  }
}

// tile table of a dense [rows, k] matrix treated as one expert (the Qwen shared expert in prefill)
__global__ void dense_tiles_kernel(int rows, int* num_tiles, int* tile_expert, int* tile_row0, int* tile_rows) {
  const int tiles = (rows + 255) / 256;
  for (int t = threadIdx.x; t < tiles; t += blockDim.x) {
    tile_expert[t] = 0; tile_row0[t] = t * 256; tile_rows[t] = min(256, rows - t * 256);
  }
  if (threadIdx.x == 0) *num_tiles = tiles;
}

int check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("%s: launch failed: %s", what, cudaGetErrorString(e)); return ERR_LAUNCH; }
  return ERR_NONE;
}

}  // namespace

int launch_dense_tiles(int rows, int* num_tiles, int* tile_expert, int* tile_row0, int* tile_rows, cudaStream_t stream) {
  dense_tiles_kernel<<<1, 256, 0, stream>>>(rows, num_tiles, tile_expert, tile_row0, tile_rows);
  return check_launch("dense tiles");
}

int launch_router_topk(const RouterArgs& a, cudaStream_t stream) {
  if (a.tokens <= 0 || a.hidden % 256 || a.experts < a.top_k || a.top_k < 1 || a.top_k > 32 || a.experts > 1024) {
    set_error("router: unsupported shape (tokens %d, hidden %d, experts %d, top_k %d)", a.tokens, a.hidden, a.experts, a.top_k);
    return ERR_BAD_ARGUMENT;
  }
  static const int small_max = [] { const char* v = std::getenv("UMAQ_ROUTER_SMALL_MAX"); return v ? std::atoi(v) : kRouterSmallMax; }();
  if (a.experts <= kRtExperts && a.hidden % kRmChunk == 0 && a.tokens > small_max) {
    static thread_local int configured = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured != dev) {
      cudaError_t e = cudaFuncSetAttribute(router_mma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, rm_smem_bytes(64));
      if (e == cudaSuccess)
        e = cudaFuncSetAttribute(router_mma_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, rm_smem_bytes(32));
      if (e != cudaSuccess) { set_error("router: cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return ERR_LAUNCH; }
      configured = dev;
    }
    static const int wide_min = [] { const char* v = std::getenv("UMAQ_ROUTER_WIDE_MIN"); return v ? std::atoi(v) : kRouterWideMin; }();
    if (a.tokens >= wide_min)
      router_mma_kernel<64><<<(a.tokens + 63) / 64, 256, rm_smem_bytes(64), stream>>>(a);
    else
      router_mma_kernel<32><<<(a.tokens + 31) / 32, 256, rm_smem_bytes(32), stream>>>(a);
    return check_launch("router");
  }
  const size_t small_smem = (size_t)kRsTokens * a.hidden * 2;
  if (a.experts <= kRtExperts && a.tokens <= small_max && small_smem <= 200 * 1024) {
    static thread_local int small_configured = -1, small_bytes = 0;
    int dev = 0;
    cudaGetDevice(&dev);
    if (small_smem > 48 * 1024 && (small_configured != dev || small_bytes < (int)small_smem)) {
      cudaError_t e = cudaFuncSetAttribute(router_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)small_smem);
      if (e != cudaSuccess) { set_error("router: cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return ERR_LAUNCH; }
      small_configured = dev; small_bytes = (int)small_smem;
    }
    router_small_kernel<<<kRsCluster * ((a.tokens + kRsTokens - 1) / kRsTokens), kRsWarps * 32, small_smem, stream>>>(a);
    return check_launch("router");
  }
  if (a.experts <= kRtExperts && a.hidden % kRtChunk == 0 && a.top_k <= 32) {
    router_tiled_kernel<<<(a.tokens + kRtTokens - 1) / kRtTokens, 256, 0, stream>>>(a);
    return check_launch("router");
  }
  const int blocks = (a.tokens + kRouterWarps - 1) / kRouterWarps;
  router_topk_kernel<<<blocks, kRouterWarps * 32, kRouterWarps * a.experts * sizeof(float), stream>>>(a);
  return check_launch("router");
}

int launch_route_sort(const SortArgs& a, cudaStream_t stream) {
  if (a.experts > kMaxSortExperts || a.tokens <= 0 || a.top_k < 1 || (long long)a.tokens * a.top_k > 0x7fffffffLL) {
    set_error("route sort: unsupported shape (tokens %d, top_k %d, experts %d)", a.tokens, a.top_k, a.experts);
    return ERR_BAD_ARGUMENT;
  }
  const long long routes = (long long)a.tokens * a.top_k;
  const int chunks = (int)((routes + kChunk - 1) / kChunk);
  if (chunks <= 2 || !a.scratch || a.scratch_ints < (long long)chunks * a.experts) {
    route_sort_kernel<<<1, kSortThreads, 0, stream>>>(a);
    return check_launch("route sort");
  }
  route_hist_kernel<<<chunks, kSortThreads, 0, stream>>>(a, a.scratch);
  route_place_kernel<<<chunks, kSortThreads, 0, stream>>>(a, a.scratch, chunks);
  return check_launch("route sort");
}

int launch_gather_rows(const __nv_bfloat16* x, const int* sorted_route, int top_k, long long routes, int hidden,
                       int permute, __nv_bfloat16* out, const int* valid_rows, cudaStream_t stream) {
  if (routes <= 0 || hidden % 8 || routes > 0x7fffffffLL) { set_error("gather: unsupported shape"); return ERR_BAD_ARGUMENT; }
  gather_rows_kernel<<<(unsigned)((routes + kGatherRows - 1) / kGatherRows), kGatherRows * 32, 0, stream>>>(
      x, sorted_route, top_k, routes, hidden, permute, out, valid_rows);
  return check_launch("gather");
}

int launch_combine(const __nv_bfloat16* weighted, const void* indices, int idx64, const int* route_pos, int tokens,
                   int top_k, int hidden, int experts, const __nv_bfloat16* shared_out, const __nv_bfloat16* x,
                   const __nv_bfloat16* gate_vec, __nv_bfloat16* out, cudaStream_t stream,
                   const SegmentedOut* segments) {
  if (tokens <= 0 || top_k < 1 || top_k > 8 || hidden % 8) { set_error("combine: unsupported shape"); return ERR_BAD_ARGUMENT; }
  SegmentedOut seg{};
  if (segments) seg = *segments;
  static const int warp_path = [] { const char* v = std::getenv("UMAQ_COMBINE_WARP"); return v ? std::atoi(v) : 1; }();
  if (!shared_out && warp_path) {
    combine_warp_kernel<<<(tokens + kCombineWarps - 1) / kCombineWarps, kCombineWarps * 32, 0, stream>>>(
        weighted, indices, idx64, route_pos, tokens, top_k, hidden, experts, out, seg);
    return check_launch("combine");
  }
  combine_kernel<<<tokens, 256, 0, stream>>>(weighted, indices, idx64, route_pos, top_k, hidden, experts, shared_out, x, gate_vec, out, seg);
  return check_launch("combine");
}

// ---- expert-parallel routing: global expert id -> this rank's local id, or -1 (absent) --------------------------
// placement 0: expert e lives on rank e % ranks as local expert e / ranks; 1: rank e / per_rank, local e % per_rank.
__global__ void ep_local_ids_kernel(const void* __restrict__ indices, int idx64, long long n, int ranks, int rank,
                                    int per_rank, int placement, int* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int e = load_expert(indices, idx64, i);
  int local = -1;
  if (e >= 0 && e < ranks * per_rank) {
    if (placement == 0) { if (e % ranks == rank) local = e / ranks; }
    else if (e / per_rank == rank) local = e % per_rank;
  }
  out[i] = local;
}

int launch_ep_local_ids(const void* indices, int idx64, long long n, int ranks, int rank, int per_rank, int placement,
                        int* out, cudaStream_t stream) {
  if (n <= 0 || ranks < 1 || rank < 0 || rank >= ranks || per_rank < 1 || (placement != 0 && placement != 1)) {
    set_error("ep local ids: bad argument");
    return ERR_BAD_ARGUMENT;
  }
  ep_local_ids_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(indices, idx64, n, ranks, rank, per_rank, placement, out);
  return check_launch("ep local ids");
}

int launch_ep_pack(const __nv_bfloat16* x, const int* sorted_route, const int* sorted_key, const float* sorted_weight,
                   const int* offsets, int routes, int top_k, int hidden, int ranks, int per_rank, int capacity,
                   __nv_bfloat16* send_rows, int* send_meta, int* route_slot, int* overflow, cudaStream_t stream) {
  if (routes <= 0 || hidden % 8 || ranks < 1 || per_rank < 1 || capacity < 1) {
    set_error("ep pack: unsupported shape");
    return ERR_BAD_ARGUMENT;
  }
  cudaError_t e = cudaMemsetAsync(send_meta, 0xFF, (size_t)ranks * capacity * 8, stream);
  if (e != cudaSuccess) { set_error("ep pack: memset: %s", cudaGetErrorString(e)); return ERR_LAUNCH; }
  ep_pack_kernel<<<routes, 128, 0, stream>>>(x, sorted_route, sorted_key, sorted_weight, offsets, top_k, hidden, per_rank,
                                             capacity, send_rows, send_meta, route_slot, overflow);
  return check_launch("ep pack");
}

}  // namespace umaq
