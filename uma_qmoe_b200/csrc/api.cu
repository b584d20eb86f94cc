// extern "C" surface of libumaq_b200.so (declared in include/umaq_b200.h) plus the few host
// utilities the kernels' launchers share.
#include "../../include/umaq_b200.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "common.cuh"
#include "aux.cuh"
#include "decode.cuh"
#include "grouped.cuh"

namespace umaq {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int sm_count() {
  static thread_local int cached_dev = -1, cached = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (dev != cached_dev) {
    cudaDeviceGetAttribute(&cached, cudaDevAttrMultiProcessorCount, dev);
    cached_dev = dev;
  }
  return cached;
}

}  // namespace umaq

using namespace umaq;

extern "C" {

int umaq_build_info(char* buf, int len) {
  static const char info[] = "sm_100a;libumaq_b200;" __DATE__ " " __TIME__;
  if (buf && len > 0) {
    strncpy(buf, info, (size_t)len - 1);
    buf[len - 1] = 0;
  }
  return (int)sizeof(info);
}

const char* umaq_last_error(void) { return g_error; }

int umaq_sm_count(void) { return sm_count(); }

size_t umaq_decode_workspace_bytes(int top_k, int intermediate, int shared_intermediate) {
  return decode_workspace_bytes(top_k, intermediate, shared_intermediate);
}

int umaq_moe_decode(const umaq_layer* layer, const umaq_shared_expert* shared, const void* hidden_bf16,
                    const void* expert_indices, int indices_are_int64, const float* routing_weights, int top_k,
                    void* out_bf16, void* workspace, size_t workspace_bytes, void* stream) {
  if (!layer || !hidden_bf16 || !expert_indices || !routing_weights || !out_bf16 || !workspace) {
    set_error("umaq_moe_decode: null argument");
    return ERR_BAD_ARGUMENT;
  }
  const int s_inter = shared ? shared->intermediate : 0;
  if (workspace_bytes < decode_workspace_bytes(top_k, layer->intermediate, s_inter) ||
      (reinterpret_cast<uintptr_t>(workspace) & 255)) {
    set_error("umaq_moe_decode: workspace too small or not 256-byte aligned");
    return ERR_WORKSPACE;
  }
  DecodeParams p{};
  p.gate = static_cast<const uint8_t*>(layer->gate);
  p.up = static_cast<const uint8_t*>(layer->up);
  p.down = static_cast<const uint8_t*>(layer->down);
  p.gate_s = layer->gate_scales;
  p.up_s = layer->up_scales;
  p.down_s = layer->down_scales;
  p.enc = layer->encoding;
  p.experts = layer->num_experts;
  p.hidden = layer->hidden;
  p.inter = layer->intermediate;
  p.top_k = top_k;
  p.x = static_cast<const __nv_bfloat16*>(hidden_bf16);
  p.idx = expert_indices;
  p.idx64 = indices_are_int64;
  p.w = routing_weights;
  if (shared) {
    p.sh_gate = static_cast<const __nv_bfloat16*>(shared->gate);
    p.sh_up = static_cast<const __nv_bfloat16*>(shared->up);
    p.sh_down = static_cast<const __nv_bfloat16*>(shared->down);
    p.sh_gatevec = static_cast<const __nv_bfloat16*>(shared->gate_vec);
    p.shared_inter = shared->intermediate;
    if (!p.sh_gate || !p.sh_up || !p.sh_down || !p.sh_gatevec) {
      set_error("umaq_moe_decode: shared expert with a null tensor");
      return ERR_BAD_ARGUMENT;
    }
  }
  p.out = static_cast<__nv_bfloat16*>(out_bf16);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  p.sync = reinterpret_cast<unsigned*>(ws);
  p.inter_buf = ws + kDecodeWsHeader;
  return launch_moe_decode(p, static_cast<cudaStream_t>(stream));
}

int umaq_quantize_groups(const void* src_bf16, long long elements, int encoding, void* codes, float* scales,
                         void* stream) {
  return launch_quantize_groups(src_bf16, elements, encoding, codes, scales, static_cast<cudaStream_t>(stream));
}

int umaq_route_topk(const void* hidden_bf16, const void* router_weight_bf16, int tokens, int hidden, int experts,
                    int top_k, int renormalize, float* out_weights, long long* out_indices, void* out_logits_bf16,
                    void* stream) {
  if (!hidden_bf16 || !router_weight_bf16 || !out_weights || !out_indices) {
    set_error("umaq_route_topk: null argument");
    return ERR_BAD_ARGUMENT;
  }
  RouterArgs a{};
  a.x = static_cast<const __nv_bfloat16*>(hidden_bf16);
  a.weight = static_cast<const __nv_bfloat16*>(router_weight_bf16);
  a.tokens = tokens; a.hidden = hidden; a.experts = experts; a.top_k = top_k; a.renormalize = renormalize;
  a.out_weights = out_weights; a.out_indices = out_indices;
  a.out_logits = static_cast<__nv_bfloat16*>(out_logits_bf16);
  return launch_router_topk(a, static_cast<cudaStream_t>(stream));
}

int umaq_route_sort(const void* expert_indices, int indices_are_int64, const float* routing_weights, int tokens, int top_k,
                    int num_experts, int* counts, int* offsets, int* sorted_route, int* route_pos, float* sorted_weight,
                    int* num_tiles, int* tile_table, int max_tiles, unsigned* status, int* scratch, long long scratch_ints,
                    void* stream) {
  if (!expert_indices || !routing_weights || !counts || !offsets || !sorted_route || !route_pos || !sorted_weight ||
      !num_tiles || !tile_table || !status || max_tiles <= 0) {
    set_error("umaq_route_sort: null argument");
    return ERR_BAD_ARGUMENT;
  }
  SortArgs a{};
  a.indices = expert_indices; a.idx64 = indices_are_int64; a.weights = routing_weights;
  a.tokens = tokens; a.top_k = top_k; a.experts = num_experts;
  a.counts = counts; a.offsets = offsets; a.sorted_route = sorted_route; a.route_pos = route_pos;
  a.sorted_weight = sorted_weight; a.num_tiles = num_tiles;
  a.tile_expert = tile_table; a.tile_row0 = tile_table + max_tiles; a.tile_rows = tile_table + 2 * max_tiles;
  a.max_tiles = max_tiles; a.status = status;
  a.scratch = scratch; a.scratch_ints = scratch ? scratch_ints : 0;
  return launch_route_sort(a, static_cast<cudaStream_t>(stream));
}

int umaq_gather_rows(const void* hidden_bf16, const int* sorted_route, int top_k, long long routes, int hidden,
                     int permute, void* out_bf16, void* stream) {
  if (!hidden_bf16 || !out_bf16) { set_error("umaq_gather_rows: null argument"); return ERR_BAD_ARGUMENT; }
  return launch_gather_rows(static_cast<const __nv_bfloat16*>(hidden_bf16), sorted_route, top_k, routes, hidden, permute,
                            static_cast<__nv_bfloat16*>(out_bf16), nullptr, static_cast<cudaStream_t>(stream));
}

int umaq_grouped_gemm(const umaq_layer* layer, int mode, const void* act_bf16, long long total_rows, const int* num_tiles,
                      const int* tile_table, int max_tiles, const float* route_weight, int permute_out, void* out_bf16,
                      unsigned* status, int variant, void* stream) {
  if (!layer || !act_bf16 || !num_tiles || !tile_table || !out_bf16 || !status || (mode != 0 && mode != 1) ||
      variant < 0 || variant > 2) {
    set_error("umaq_grouped_gemm: bad argument");
    return ERR_BAD_ARGUMENT;
  }
  GroupedGemmArgs g{};
  g.mode = mode; g.enc = layer->encoding; g.num_experts = layer->num_experts;
  g.n_rows = mode == 0 ? layer->intermediate : layer->hidden;
  g.k = mode == 0 ? layer->hidden : layer->intermediate;
  g.act = act_bf16; g.total_rows = total_rows;
  if (mode == 0) { g.w0 = layer->gate; g.s0 = layer->gate_scales; g.w1 = layer->up; g.s1 = layer->up_scales; }
  else { g.w0 = layer->down; g.s0 = layer->down_scales; }
  g.num_tiles = num_tiles; g.tile_expert = tile_table; g.tile_row0 = tile_table + max_tiles;
  g.tile_rows = tile_table + 2 * max_tiles; g.max_tiles = max_tiles;
  g.out = static_cast<__nv_bfloat16*>(out_bf16); g.out_stride = g.n_rows;
  g.route_weight = route_weight; g.permute_out = permute_out; g.status = status; g.variant = variant;
  return launch_grouped_gemm(g, static_cast<cudaStream_t>(stream));
}

int umaq_grouped_gemm_by_index(const umaq_layer* layer, const void* hidden_bf16, const int* sorted_route, int top_k,
                               long long routes, const int* num_tiles, const int* tile_table, int max_tiles,
                               int permute_out, void* out_bf16, unsigned* status, void* stream) {
  if (!layer || !hidden_bf16 || !sorted_route || !num_tiles || !tile_table || !out_bf16 || !status || top_k < 1 || routes <= 0) {
    set_error("umaq_grouped_gemm_by_index: bad argument");
    return ERR_BAD_ARGUMENT;
  }
  GroupedGemmArgs g{};
  g.mode = 0; g.enc = layer->encoding; g.num_experts = layer->num_experts;
  g.n_rows = layer->intermediate; g.k = layer->hidden;
  g.act = hidden_bf16; g.total_rows = routes;
  g.w0 = layer->gate; g.s0 = layer->gate_scales; g.w1 = layer->up; g.s1 = layer->up_scales;
  g.num_tiles = num_tiles; g.tile_expert = tile_table; g.tile_row0 = tile_table + max_tiles;
  g.tile_rows = tile_table + 2 * max_tiles; g.max_tiles = max_tiles;
  g.out = static_cast<__nv_bfloat16*>(out_bf16); g.out_stride = g.n_rows;
  g.permute_out = permute_out; g.status = status; g.variant = 1;
  g.gather_route = sorted_route; g.gather_top_k = top_k;
  return launch_grouped_gemm(g, static_cast<cudaStream_t>(stream));
}

int umaq_ep_local_ids(const void* expert_indices, int indices_are_int64, long long count, int ranks, int rank,
                       int experts_per_rank, int placement, int* local_ids, void* stream) {
  if (!expert_indices || !local_ids) { set_error("umaq_ep_local_ids: null argument"); return ERR_BAD_ARGUMENT; }
  return launch_ep_local_ids(expert_indices, indices_are_int64, count, ranks, rank, experts_per_rank, placement, local_ids,
                             static_cast<cudaStream_t>(stream));
}

int umaq_ep_push(const void* hidden_bf16, const void* expert_indices, int indices_are_int64, const float* routing_weights,
                 int tokens, int top_k, int hidden, int experts_per_rank, int placement, int flags,
                 const umaq_ep_peers* peers, size_t rows_offset, size_t ids_offset, size_t weights_offset, int* present,
                 void* stream) {
  if (!hidden_bf16 || !expert_indices || !routing_weights || !peers || !present) {
    set_error("umaq_ep_push: null argument");
    return ERR_BAD_ARGUMENT;
  }
  return launch_ep_push(static_cast<const __nv_bfloat16*>(hidden_bf16), expert_indices, indices_are_int64, routing_weights,
                        tokens, top_k, hidden, experts_per_rank, placement, flags, *peers, rows_offset, ids_offset, weights_offset,
                        present, static_cast<cudaStream_t>(stream));
}

int umaq_ep_barrier(const umaq_ep_peers* peers, size_t flags_offset, unsigned* epoch, unsigned* status, void* stream) {
  if (!peers || !epoch || !status) { set_error("umaq_ep_barrier: null argument"); return ERR_BAD_ARGUMENT; }
  return launch_ep_barrier(*peers, flags_offset, epoch, status, static_cast<cudaStream_t>(stream));
}

int umaq_ep_pack(const void* hidden_bf16, const int* sorted_route, const int* sorted_key, const float* sorted_weight,
                 const int* offsets, int routes, int top_k, int hidden, int ranks, int experts_per_rank, int capacity,
                 void* send_rows_bf16, int* send_meta, int* route_slot, int* overflow, void* stream) {
  if (!hidden_bf16 || !sorted_route || !sorted_key || !sorted_weight || !offsets || !send_rows_bf16 || !send_meta ||
      !route_slot || !overflow) {
    set_error("umaq_ep_pack: null argument");
    return ERR_BAD_ARGUMENT;
  }
  return launch_ep_pack(static_cast<const __nv_bfloat16*>(hidden_bf16), sorted_route, sorted_key, sorted_weight, offsets,
                        routes, top_k, hidden, ranks, experts_per_rank, capacity,
                        static_cast<__nv_bfloat16*>(send_rows_bf16), send_meta, route_slot, overflow,
                        static_cast<cudaStream_t>(stream));
}

int umaq_combine_routes(const void* weighted_bf16, const void* expert_indices, int indices_are_int64, const int* route_pos,
                        int tokens, int top_k, int hidden, void* out_bf16, void* stream) {
  if (!weighted_bf16 || !expert_indices || !route_pos || !out_bf16) {
    set_error("umaq_combine_routes: null argument");
    return ERR_BAD_ARGUMENT;
  }
  return launch_combine(static_cast<const __nv_bfloat16*>(weighted_bf16), expert_indices, indices_are_int64, route_pos,
                        tokens, top_k, hidden, 0x7fffffff, nullptr, nullptr, nullptr, static_cast<__nv_bfloat16*>(out_bf16),
                        static_cast<cudaStream_t>(stream));
}

namespace {
struct PrefillPlan {
  size_t status, counts, offsets, num_tiles, tiles, sort_scratch, sorted_route, route_pos, sorted_weight, xs, inter, yw;
  long long sort_ints;
  size_t s_num_tiles, s_tiles, s_inter, s_out, total;
  int max_tiles, s_max_tiles;
};
size_t align256(size_t v) { return (v + 255) & ~size_t(255); }
PrefillPlan prefill_plan(long long tokens, int top_k, int experts, int hidden, int inter, int shared_inter) {
  PrefillPlan p{};
  const size_t routes = (size_t)tokens * top_k;
  p.max_tiles = (int)((routes + 127) / 128) + experts;
  p.s_max_tiles = (int)((tokens + 127) / 128);
  size_t cur = 0;
  auto take = [&](size_t bytes) { const size_t at = cur; cur = align256(cur + bytes); return at; };
  p.status = take(256);
  p.counts = take((size_t)experts * 4);
  p.offsets = take((size_t)(experts + 1) * 4);
  p.num_tiles = take(4);
  p.tiles = take((size_t)p.max_tiles * 12);
  p.sort_ints = (long long)((routes + 2047) / 2048) * experts;
  p.sort_scratch = take((size_t)p.sort_ints * 4);
  p.sorted_route = take(routes * 4);
  p.route_pos = take(routes * 4);
  p.sorted_weight = take(routes * 4);
  p.xs = take(routes * hidden * 2);
  p.inter = take(routes * inter * 2);
  p.yw = take(routes * hidden * 2);
  if (shared_inter) {
    p.s_num_tiles = take(4);
    p.s_tiles = take((size_t)p.s_max_tiles * 12);
    p.s_inter = take((size_t)tokens * shared_inter * 2);
    p.s_out = take((size_t)tokens * hidden * 2);
  }
  p.total = cur;
  return p;
}
}  // namespace

size_t umaq_prefill_workspace_bytes(long long tokens, int top_k, int num_experts, int hidden, int intermediate,
                                    int shared_intermediate) {
  return prefill_plan(tokens, top_k, num_experts, hidden, intermediate, shared_intermediate).total;
}

static int prefill_impl(const umaq_layer* layer, const umaq_shared_expert* shared, const void* hidden_bf16,
                        const void* expert_indices, int indices_are_int64, const float* routing_weights, long long tokens,
                        int top_k, void* out_bf16, void* workspace, size_t workspace_bytes, void* stream_,
                        const SegmentedOut* segments, bool rows_k_permuted = false) {
  if (!layer || !hidden_bf16 || !expert_indices || !routing_weights || (!out_bf16 && !segments) || !workspace || tokens <= 0) {
    set_error("umaq_moe_prefill: null argument");
    return ERR_BAD_ARGUMENT;
  }
  const int H = layer->hidden, I = layer->intermediate, E = layer->num_experts;
  const int S = shared ? shared->intermediate : 0;
  if (tokens * (long long)top_k > 0x7fffffffLL || top_k < 1 || top_k > 8) {
    set_error("umaq_moe_prefill: unsupported route count");
    return ERR_BAD_ARGUMENT;
  }
  const PrefillPlan pl = prefill_plan(tokens, top_k, E, H, I, S);
  if (workspace_bytes < pl.total || (reinterpret_cast<uintptr_t>(workspace) & 255)) {
    set_error("umaq_moe_prefill: workspace too small or not 256-byte aligned");
    return ERR_WORKSPACE;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  auto at = [&](size_t off) { return ws + off; };
  unsigned* status = reinterpret_cast<unsigned*>(at(pl.status));
  int* tiles = reinterpret_cast<int*>(at(pl.tiles));
  const long long routes = tokens * top_k;
  const int quant = layer->encoding != ENC_BF16;

  SortArgs sa{};
  sa.indices = expert_indices; sa.idx64 = indices_are_int64; sa.weights = routing_weights;
  sa.tokens = (int)tokens; sa.top_k = top_k; sa.experts = E;
  sa.counts = reinterpret_cast<int*>(at(pl.counts)); sa.offsets = reinterpret_cast<int*>(at(pl.offsets));
  sa.sorted_route = reinterpret_cast<int*>(at(pl.sorted_route)); sa.route_pos = reinterpret_cast<int*>(at(pl.route_pos));
  sa.sorted_weight = reinterpret_cast<float*>(at(pl.sorted_weight));
  sa.num_tiles = reinterpret_cast<int*>(at(pl.num_tiles));
  sa.tile_expert = tiles; sa.tile_row0 = tiles + pl.max_tiles; sa.tile_rows = tiles + 2 * pl.max_tiles;
  sa.max_tiles = pl.max_tiles; sa.status = status;
  sa.scratch = reinterpret_cast<int*>(at(pl.sort_scratch)); sa.scratch_ints = pl.sort_ints;
  int rc = launch_route_sort(sa, stream);
  if (rc) return rc;
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(at(pl.xs));
  GroupedGemmArgs g{};
  g.mode = 0; g.enc = layer->encoding; g.num_experts = E; g.n_rows = I; g.k = H;
  g.total_rows = routes;
  g.w0 = layer->gate; g.s0 = layer->gate_scales; g.w1 = layer->up; g.s1 = layer->up_scales;
  g.num_tiles = sa.num_tiles; g.tile_expert = sa.tile_expert; g.tile_row0 = sa.tile_row0; g.tile_rows = sa.tile_rows;
  g.max_tiles = pl.max_tiles;
  g.out = reinterpret_cast<__nv_bfloat16*>(at(pl.inter)); g.out_stride = I; g.permute_out = quant; g.status = status;
  if (grouped_gemm_can_gather(g)) {
    // The gate/up GEMM fetches its activation rows by index: no [routes, H] copy of the activations exists.  The
    // quantised kernels want k in the order their conversion produces, so x is permuted once (tokens rows, not routes).
    const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(hidden_bf16);
    if (quant && !rows_k_permuted) {
      rc = launch_gather_rows(src, nullptr, 1, tokens, H, 1, xs, nullptr, stream);
      if (rc) return rc;
      src = xs;
    }
    g.act = src; g.gather_route = sa.sorted_route; g.gather_top_k = top_k;
  } else {
    // routes with expert id -1 are absent: only the first offsets[E] sorted rows exist
    rc = launch_gather_rows(static_cast<const __nv_bfloat16*>(hidden_bf16), sa.sorted_route, top_k, routes, H, quant, xs,
                            sa.offsets + E, stream);
    if (rc) return rc;
    g.act = xs;
  }
  rc = launch_grouped_gemm(g, stream);
  if (rc) return rc;
  g.mode = 1; g.n_rows = H; g.k = I; g.act = g.out; g.gather_route = nullptr;
  g.w0 = layer->down; g.s0 = layer->down_scales; g.w1 = nullptr; g.s1 = nullptr;
  g.out = reinterpret_cast<__nv_bfloat16*>(at(pl.yw)); g.out_stride = H; g.route_weight = sa.sorted_weight; g.permute_out = 0;
  rc = launch_grouped_gemm(g, stream);
  if (rc) return rc;

  const __nv_bfloat16* shared_out = nullptr;
  if (shared) {
    int* st = reinterpret_cast<int*>(at(pl.s_tiles));
    int* snt = reinterpret_cast<int*>(at(pl.s_num_tiles));
    rc = launch_dense_tiles((int)tokens, snt, st, st + pl.s_max_tiles, st + 2 * pl.s_max_tiles, stream);
    if (rc) return rc;
    GroupedGemmArgs d{};
    d.mode = 0; d.enc = ENC_BF16; d.num_experts = 1; d.n_rows = S; d.k = H;
    d.act = hidden_bf16; d.total_rows = tokens;
    d.w0 = shared->gate; d.w1 = shared->up;
    d.num_tiles = snt; d.tile_expert = st; d.tile_row0 = st + pl.s_max_tiles; d.tile_rows = st + 2 * pl.s_max_tiles;
    d.max_tiles = pl.s_max_tiles;
    d.out = reinterpret_cast<__nv_bfloat16*>(at(pl.s_inter)); d.out_stride = S; d.status = status;
    rc = launch_grouped_gemm(d, stream);
    if (rc) return rc;
    d.mode = 1; d.n_rows = H; d.k = S; d.act = d.out; d.w0 = shared->down; d.w1 = nullptr;
    d.out = reinterpret_cast<__nv_bfloat16*>(at(pl.s_out)); d.out_stride = H; d.route_weight = nullptr;
    rc = launch_grouped_gemm(d, stream);
    if (rc) return rc;
    shared_out = d.out;
  }
  return launch_combine(reinterpret_cast<const __nv_bfloat16*>(at(pl.yw)), expert_indices, indices_are_int64, sa.route_pos,
                        (int)tokens, top_k, H, E, shared_out, static_cast<const __nv_bfloat16*>(hidden_bf16),
                        shared ? static_cast<const __nv_bfloat16*>(shared->gate_vec) : nullptr,
                        static_cast<__nv_bfloat16*>(out_bf16), stream, segments);
}

int umaq_moe_prefill(const umaq_layer* layer, const umaq_shared_expert* shared, const void* hidden_bf16,
                     const void* expert_indices, int indices_are_int64, const float* routing_weights, long long tokens,
                     int top_k, void* out_bf16, void* workspace, size_t workspace_bytes, void* stream_) {
  return prefill_impl(layer, shared, hidden_bf16, expert_indices, indices_are_int64, routing_weights, tokens, top_k,
                      out_bf16, workspace, workspace_bytes, stream_, nullptr);
}

int umaq_moe_prefill_to_peers(const umaq_layer* layer, const void* hidden_bf16, const void* expert_indices,
                              int indices_are_int64, const float* routing_weights, long long tokens, int top_k,
                              const umaq_ep_peers* peers, size_t parts_offset, int segment_rows, int rows_k_permuted,
                              void* workspace, size_t workspace_bytes, void* stream_) {
  if (!peers || peers->ranks < 1 || peers->ranks > kMaxPeers || peers->rank < 0 || peers->rank >= peers->ranks ||
      segment_rows < 1 || tokens != (long long)segment_rows * peers->ranks || !layer) {
    set_error("umaq_moe_prefill_to_peers: bad peer table or segment size");
    return ERR_BAD_ARGUMENT;
  }
  SegmentedOut seg{};
  for (int p = 0; p < peers->ranks; ++p) {
    if (!peers->base[p]) { set_error("umaq_moe_prefill_to_peers: null peer buffer"); return ERR_BAD_ARGUMENT; }
    seg.ptr[p] = reinterpret_cast<__nv_bfloat16*>(static_cast<uint8_t*>(peers->base[p]) + parts_offset);
  }
  seg.rows = segment_rows;
  seg.row0 = peers->rank * segment_rows;
  seg.skip_empty = 1;
  if (rows_k_permuted) {
    // only the by-index gate/up GEMM of a quantised layer reads its rows in that order
    GroupedGemmArgs g{};
    g.mode = 0; g.enc = layer->encoding; g.num_experts = layer->num_experts; g.n_rows = layer->intermediate; g.k = layer->hidden;
    g.total_rows = tokens * top_k;
    if (layer->encoding == ENC_BF16 || !grouped_gemm_can_gather(g)) {
      set_error("umaq_moe_prefill_to_peers: rows_k_permuted needs a quantised layer the gate/up GEMM reads by index");
      return ERR_BAD_ARGUMENT;
    }
  }
  return prefill_impl(layer, nullptr, hidden_bf16, expert_indices, indices_are_int64, routing_weights, tokens, top_k,
                      nullptr, workspace, workspace_bytes, stream_, &seg, rows_k_permuted != 0);
}

int umaq_ep_layer(const umaq_layer* layer, const void* hidden_bf16, const void* expert_indices, int indices_are_int64,
                  const float* routing_weights, int tokens, int top_k, int experts_per_rank, int placement,
                  const umaq_ep_peers* peers, size_t rows_offset, size_t ids_offset, size_t weights_offset,
                  size_t parts_offset, size_t flags_offset, int* present, const int* part_pos, unsigned* epoch,
                  unsigned* status, void* workspace, size_t workspace_bytes, void* out_bf16, void* stream) {
  if (!layer || !peers || !part_pos || !epoch || !status || !out_bf16) {
    set_error("umaq_ep_layer: null argument");
    return ERR_BAD_ARGUMENT;
  }
  if (peers->ranks < 1 || peers->ranks > kMaxPeers || peers->rank < 0 || peers->rank >= peers->ranks ||
      !peers->base[peers->rank]) {
    set_error("umaq_ep_layer: bad peer table");
    return ERR_BAD_ARGUMENT;
  }
  const int quant = layer->encoding != ENC_BF16;
  int rc = umaq_ep_push(hidden_bf16, expert_indices, indices_are_int64, routing_weights, tokens, top_k, layer->hidden,
                        experts_per_rank, placement, UMAQ_EP_LOCAL_IDS | (quant ? UMAQ_EP_K_PERMUTED : 0), peers,
                        rows_offset, ids_offset, weights_offset, present, stream);
  if (rc) return rc;
  rc = umaq_ep_barrier(peers, flags_offset, epoch, status, stream);
  if (rc) return rc;
  uint8_t* mine = static_cast<uint8_t*>(peers->base[peers->rank]);
  rc = umaq_moe_prefill_to_peers(layer, mine + rows_offset, mine + ids_offset, 0,
                                 reinterpret_cast<const float*>(mine + weights_offset), (long long)tokens * peers->ranks,
                                 top_k, peers, parts_offset, tokens, quant, workspace, workspace_bytes, stream);
  if (rc) return rc;
  rc = umaq_ep_barrier(peers, flags_offset, epoch, status, stream);
  if (rc) return rc;
  return umaq_combine_routes(mine + parts_offset, present, 0, part_pos, tokens, peers->ranks, layer->hidden, out_bf16, stream);
}

}  // extern "C"
