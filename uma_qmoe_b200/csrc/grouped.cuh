// Parameter blocks and host launchers of the prefill path (grouped.cu, route.cu).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/umaq_b200.h"

namespace umaq {

// Device-side view handed to the grouped GEMM kernel.
struct GroupedParams {
  int k;                      // contraction length
  int n_rows;                 // weight rows per expert in this projection
  const float* scales0;       // [E * n_rows, k/128] (gate or down)
  const float* scales1;       // up (mode 0)
  const int* num_tiles;       // device: number of valid 128-route tiles
  const int* tile_expert;     // device [max_tiles]
  const int* tile_row0;       // first sorted route row of the tile
  const int* tile_rows;       // valid rows (<= 128)
  int max_tiles;
  __nv_bfloat16* out;         // mode 0: intermediate [routes, n_rows]; mode 1: weighted outputs [routes, n_rows]
  long long out_stride;       // elements
  const float* route_weight;  // mode 1: routing weight per sorted route
  int permute_out;            // mode 0: write the [k0,k4,k1,k5,k2,k6,k3,k7] order a quantised GEMM 2 expects
  unsigned* status;           // sticky error word
  // mode 0, optional: fetch the activation rows by index instead of reading pre-gathered rows.  Sorted route r
  // is row gather_route[r] / gather_top_k of gather_src ([tokens, k] BF16, k already in the order the encoding wants)
  const int* gather_route;
  int gather_top_k;
  const __nv_bfloat16* gather_src;
  int debug;
  int tma_out;                // mode 1, staged results: map_b1 describes `out` and whole 32-row groups leave by tensor store
};

struct GroupedGemmArgs {
  int mode;                   // 0 gate/up + SwiGLU, 1 down + routing weight
  int enc;
  int num_experts;
  int n_rows;                 // I (mode 0) or H (mode 1)
  int k;                      // H (mode 0) or I (mode 1)
  const void* act;            // bf16 [total_rows, k], sorted by expert
  long long total_rows;
  const void* w0; const float* s0;   // gate or down
  const void* w1; const float* s1;   // up
  const int* num_tiles; const int* tile_expert; const int* tile_row0; const int* tile_rows;
  int max_tiles;
  __nv_bfloat16* out; long long out_stride;
  const float* route_weight;
  int permute_out;
  unsigned* status;
  int variant;                // 0: by size; 1: one CTA per tile (grouped.cu); 2: persistent CTA pairs (grouped_pair.cu)
  // mode 0 on the one-CTA kernel, optional: act = [tokens, k] and the kernel fetches row sorted_route[r] / top_k
  // for sorted route r itself (no gathered copy of the activations)
  const int* gather_route;
  int gather_top_k;
};

// true if launch_grouped_gemm would run the kernel that can fetch its activation rows by index
bool grouped_gemm_can_gather(const GroupedGemmArgs& a);

int launch_grouped_gemm(const GroupedGemmArgs& a, cudaStream_t stream);        // picks the variant
int launch_grouped_gemm_single(const GroupedGemmArgs& a, cudaStream_t stream);
int launch_grouped_gemm_pair(const GroupedGemmArgs& a, cudaStream_t stream);

// ---- routing (route.cu) ---------------------------------------------------------------------------
struct RouterArgs {
  const __nv_bfloat16* x;        // [tokens, hidden]
  const __nv_bfloat16* weight;   // [experts, hidden]
  int tokens, hidden, experts, top_k, renormalize;
  float* out_weights;            // [tokens, top_k] float32
  long long* out_indices;        // [tokens, top_k] int64
  __nv_bfloat16* out_logits;     // optional [tokens, experts]
};
int launch_router_topk(const RouterArgs& a, cudaStream_t stream);

struct SortArgs {
  const void* indices; int idx64;  // [tokens, top_k]
  const float* weights;            // [tokens, top_k]
  int tokens, top_k, experts;
  int* counts;                     // [experts]
  int* offsets;                    // [experts + 1]
  int* sorted_route;               // [routes] token * top_k + slot, stable by expert
  int* route_pos;                  // [routes] inverse permutation
  float* sorted_weight;            // [routes]
  int* num_tiles; int* tile_expert; int* tile_row0; int* tile_rows;   // 128-route tiles
  int max_tiles;
  unsigned* status;
  int* scratch;                    // optional: ceil(routes / 2048) * experts ints let the sort use many CTAs
  long long scratch_ints;
};
int launch_route_sort(const SortArgs& a, cudaStream_t stream);

int launch_dense_tiles(int rows, int* num_tiles, int* tile_expert, int* tile_row0, int* tile_rows, cudaStream_t stream);

// rows of x gathered into sorted order; `permute` writes each run of 8 as [0,4,1,5,2,6,3,7]
// valid_rows (device, may be null): only the first *valid_rows sorted routes exist
int launch_gather_rows(const __nv_bfloat16* x, const int* sorted_route, int top_k, long long routes, int hidden,
                       int permute, __nv_bfloat16* out, const int* valid_rows, cudaStream_t stream);
int launch_ep_local_ids(const void* indices, int idx64, long long n, int ranks, int rank, int per_rank, int placement,
                        int* out, cudaStream_t stream);
// expert-parallel exchange over peer memory (ep_peer.cu)
int launch_ep_push(const __nv_bfloat16* x, const void* indices, int idx64, const float* weights, int tokens, int top_k,
                   int hidden, int per_rank, int placement, int flags, const umaq_ep_peers& peers, size_t rows_offset,
                   size_t ids_offset, size_t weights_offset, int* present, cudaStream_t stream);
int launch_ep_barrier(const umaq_ep_peers& peers, size_t flags_offset, unsigned* epoch, unsigned* status,
                      cudaStream_t stream);
int launch_ep_pack(const __nv_bfloat16* x, const int* sorted_route, const int* sorted_key, const float* sorted_weight,
                   const int* offsets, int routes, int top_k, int hidden, int ranks, int per_rank, int capacity,
                   __nv_bfloat16* send_rows, int* send_meta, int* route_slot, int* overflow, cudaStream_t stream);
// Where the combine writes: by default row t of `out`.  With rows > 0 the tokens come in segments of `rows`
// (one per source rank of an expert-parallel exchange) and token t goes to row row0 + t % rows of
// ptr[t / rows] -- a buffer that may live on another GPU (plain peer stores); skip_empty leaves the rows
// of tokens without any present route unwritten.
constexpr int kMaxPeers = 8;
struct SegmentedOut {
  __nv_bfloat16* ptr[kMaxPeers];
  int rows;
  int row0;
  int skip_empty;
};
// experts: ids outside [0, experts) are treated as absent routes
int launch_combine(const __nv_bfloat16* weighted, const void* indices, int idx64, const int* route_pos, int tokens,
                   int top_k, int hidden, int experts, const __nv_bfloat16* shared_out, const __nv_bfloat16* x,
                   const __nv_bfloat16* gate_vec, __nv_bfloat16* out, cudaStream_t stream,
                   const SegmentedOut* segments = nullptr);

}  // namespace umaq
