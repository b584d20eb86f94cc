/* C ABI of the B200 (sm_100a) routed-expert MoE kernels.
 *
 * Plain pointers and sizes only.  Every pointer named "device" is a CUDA device
 * pointer valid on the current device; `stream` is a cudaStream_t passed as
 * void*.  Calls enqueue work on `stream` and return without synchronising;
 * they allocate nothing and own nothing: inputs, outputs and workspaces belong
 * to the caller.  Return value: 0 on success, a negative UMAQ_ERR_* code
 * otherwise (umaq_last_error() then holds a message for the calling thread).
 *
 * The entry points are what a host binding of the UMA-QMoE reference calls in
 * place of its pybind11 extension (src/uma_qmoe/native/packed_q4_binding.cpp:490-515
 * in the reference: q4_linear, q8_linear, q4_moe_forward, q4_moe_prefill,
 * q8_moe_forward, q8_moe_prefill).
 */
#ifndef UMAQ_B200_H
#define UMAQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { UMAQ_ENC_Q4 = 0, UMAQ_ENC_Q8 = 1, UMAQ_ENC_BF16 = 2 };

enum {
  UMAQ_OK = 0,
  UMAQ_ERR_BAD_ARGUMENT = -1,
  UMAQ_ERR_WORKSPACE = -2,
  UMAQ_ERR_LAUNCH = -3,
  UMAQ_ERR_DEVICE_TIMEOUT = -4,
  UMAQ_ERR_UNSUPPORTED = -5
};

/* One staged MoE layer: all experts of a projection concatenated in expert
 * order, each expert's tensor in its canonical pack bytes (row-major [rows, K],
 * K contiguous; Q4: K/2 bytes per row, low nibble first; Q8: K int8; BF16: 2K
 * bytes) and, for Q4/Q8, float32 scales [rows, K/128].  This is the device
 * layout the reference's backend builds in
 * src/uma_qmoe/native_backend.py:374-455 (Q4), :769-842 (Q8), :876-956 (BF16,
 * there as one stacked gate_up tensor; here gate and up stay separate). */
typedef struct umaq_layer {
  const void* gate;          /* device [E, I, K=H] codes */
  const void* up;            /* device [E, I, K=H] codes */
  const void* down;          /* device [E, H, K=I] codes */
  const float* gate_scales;  /* device [E, I, H/128] or NULL for BF16 */
  const float* up_scales;
  const float* down_scales;  /* device [E, H, I/128] or NULL for BF16 */
  int32_t encoding;          /* UMAQ_ENC_* */
  int32_t num_experts;       /* E */
  int32_t hidden;            /* H */
  int32_t intermediate;      /* I */
} umaq_layer;

/* Qwen shared expert (BF16 nn.Linear weights) and its sigmoid gate vector:
 * src/uma_qmoe/qwen_compressed_loader.py:72,82-85. */
typedef struct umaq_shared_expert {
  const void* gate;       /* device bf16 [S, H] */
  const void* up;         /* device bf16 [S, H] */
  const void* down;       /* device bf16 [H, S] */
  const void* gate_vec;   /* device bf16 [H] (shared_expert_gate.weight) */
  int32_t intermediate;   /* S */
} umaq_shared_expert;

/* "sm_100a;<git-independent build id>" into buf; returns bytes needed. */
int umaq_build_info(char* buf, int len);
/* Message of the last failing call made by this thread ("" if none). */
const char* umaq_last_error(void);
/* Number of SMs of the current device (the grid of the persistent kernels). */
int umaq_sm_count(void);

/* ---- batch-1 decode --------------------------------------------------------
 * out[H] = sum over the top_k routes of w * Down_e(SiLU(Gate_e x) * Up_e x),
 * accumulated like the reference's CPU correctness path (ascending expert
 * number, BF16 running sum); with `shared` != NULL additionally
 * + sigmoid(x . gate_vec) * SharedExpert(x) with BF16 nn.Linear roundings.
 * Replaces q4_moe_forward / q8_moe_forward
 * (src/uma_qmoe/native/packed_q4_binding.cpp:197-265, :407-440) and the Qwen
 * per-expert q4_linear / q8_linear loops (src/uma_qmoe/native_backend.py:319-372,
 * :722-753).
 *
 * workspace: umaq_decode_workspace_bytes() bytes, 256-byte aligned, zeroed once
 * by the caller before its first use; calls sharing a workspace must not overlap
 * on the device.  Word 2 (uint32 at byte offset 8) is a sticky device-side
 * status: 0, or a UMAQ_ERR_* code if a bounded wait gave up or an expert index
 * was out of range.  A route with an out-of-range index contributes nothing, as
 * in the reference's kernels (src/uma_qmoe/native/packed_q4_kernel.cu:176), and
 * the output is still complete; after a timeout the output is undefined and the
 * first 1024 bytes of the workspace must be zeroed again (once all work on it
 * has drained) before the next call: the arrival counters in it are then stale. */
size_t umaq_decode_workspace_bytes(int top_k, int intermediate, int shared_intermediate);
int umaq_moe_decode(const umaq_layer* layer, const umaq_shared_expert* shared /* may be NULL */,
                    const void* hidden_bf16 /* device [H] */,
                    const void* expert_indices /* device [top_k] */, int indices_are_int64,
                    const float* routing_weights /* device [top_k] */, int top_k,
                    void* out_bf16 /* device [H] */, void* workspace, size_t workspace_bytes,
                    void* stream);

/* Launch geometry umaq_moe_decode would use for a shape on a device with `sms` SMs; nothing is launched
 * and no device is touched (no counterpart in the reference).  out[0..5]: gate/up kernel CTAs, ring
 * stages, bytes per stage, dynamic shared memory, most work units of a CTA, 64-byte items per stage;
 * out[6..11]: the same for the down kernel.  UMAQ_ERR_UNSUPPORTED when a shape does not fit an SM. */
int umaq_decode_plan(int encoding, int hidden, int intermediate, int top_k, int shared_intermediate, int sms,
                     int* out /* host [12] */, int out_len);

/* Decode for callers that cannot allocate device memory.  It has no counterpart in the
 * reference.  Same computation and result as umaq_moe_decode, but the scratch the kernel
 * needs (control words and the intermediate of the selected experts) lives in a
 * 64 KiB block built into the library instead of a caller workspace.  It is meant for
 * hosts that are handed only their input and output buffers: code running inside another
 * framework's stream callback or custom-call hook, or a plug-in whose memory is owned by
 * the embedding runtime, where calling cudaMalloc (or any allocator) is not allowed or
 * would serialise the device.  The call itself allocates nothing.
 *
 * Limits and rules:
 *  - top_k (rounded up to a power of two) * intermediate + shared intermediate must fit:
 *    at most 15,744 values of four bytes (OLMoE 8 x 1024 and Qwen 4 x 1408 + 5632 fit);
 *    larger shapes are refused with UMAQ_ERR_WORKSPACE and a message, use umaq_moe_decode then.
 *  - The status word of the built-in block cannot be read by the caller and is cleared by
 *    the next call: a route with an out-of-range expert index contributes nothing (as in
 *    umaq_moe_decode) but is not reported.  Validate indices first if that matters.
 *  - Every device that loads the library holds its own 64 KiB block until the process
 *    exits.  The first call on a device looks up the block's device address; make that
 *    first call outside any stream capture.
 *  - All calls on a device share the block, and it keeps what the last call left; each
 *    call clears the control words it needs on `stream` before it launches.  Two calls
 *    that can overlap on the device (different streams without an ordering between
 *    them) race on it: order them. */
int umaq_moe_decode_static(const umaq_layer* layer, const umaq_shared_expert* shared /* may be NULL */,
                           const void* hidden_bf16 /* device [H] */,
                           const void* expert_indices /* device [top_k] */, int indices_are_int64,
                           const float* routing_weights /* device [top_k] */, int top_k,
                           void* out_bf16 /* device [H] */, void* stream);

/* ---- router ---------------------------------------------------------------------
 * logits = bf16(x . Wr^T), softmax over the experts in float32, top-k (ties to the
 * lowest expert index), optional division by the top-k sum: the arithmetic of the
 * Hugging Face OlmoeTopKRouter / Qwen2MoeTopKRouter modules the reference calls
 * before the operator (src/uma_qmoe/compressed_loader.py:59,
 * src/uma_qmoe/qwen_compressed_loader.py:73; restated in
 * benchmarks/runners/capture_qwen_route_trace.py:46-66).  out_logits may be NULL. */
int umaq_route_topk(const void* hidden_bf16 /* device [tokens, hidden] */,
                    const void* router_weight_bf16 /* device [experts, hidden] */, int tokens, int hidden,
                    int experts, int top_k, int renormalize, float* out_weights /* device [tokens, top_k] */,
                    long long* out_indices /* device [tokens, top_k] */,
                    void* out_logits_bf16 /* device [tokens, experts] or NULL */, void* stream);

/* ---- prefill / batched tokens ----------------------------------------------------
 * Same result contract as umaq_moe_decode for `tokens` rows: stable sort of the
 * routes by expert (replaces the host-side argsort / bincount / cumsum of
 * src/uma_qmoe/native_backend.py:531-543), grouped gate/up GEMM with SwiGLU,
 * grouped down GEMM with the routing weight, ordered BF16 top-k combine; with
 * `shared` != NULL the Qwen shared expert and its sigmoid gate are added.
 * Replaces q4_moe_prefill / q8_moe_prefill
 * (src/uma_qmoe/native/packed_q4_binding.cpp:267-347, :442-488) and the BF16
 * torch._grouped_mm path (src/uma_qmoe/native_backend.py:958-1005).
 * workspace: umaq_prefill_workspace_bytes() bytes, 256-byte aligned; its first
 * uint32 is a sticky device-side status (zero it before the first call). */
size_t umaq_prefill_workspace_bytes(long long tokens, int top_k, int num_experts, int hidden, int intermediate,
                                    int shared_intermediate);
int umaq_moe_prefill(const umaq_layer* layer, const umaq_shared_expert* shared /* may be NULL */,
                     const void* hidden_bf16 /* device [tokens, H] */,
                     const void* expert_indices /* device [tokens, top_k] */, int indices_are_int64,
                     const float* routing_weights /* device [tokens, top_k] */, long long tokens, int top_k,
                     void* out_bf16 /* device [tokens, H] */, void* workspace, size_t workspace_bytes, void* stream);

/* ---- building blocks of the prefill path ---------------------------------------------
 * The pieces umaq_moe_prefill chains, exported for hosts that place a collective
 * between them (expert parallelism) and for per-kernel measurement.  They have no
 * single counterpart in the reference; each cites what it replaces.
 *
 * umaq_route_sort: stable sort of the tokens*top_k routes by expert id, replacing
 * torch.argsort(stable) / bincount / cumsum at src/uma_qmoe/native_backend.py:531-543.
 * Route i = token * top_k + slot.  Outputs (all device): counts[E], offsets[E+1],
 * sorted_route[routes] (route ids in expert order), route_pos[routes] (its inverse),
 * sorted_weight[routes], and the tile list of the grouped GEMM (up to 256 routes of one expert each):
 * *num_tiles and tile_table = int[3 * max_tiles] holding expert, first row, row count.
 * max_tiles >= ceil(routes / 128) + E.  *status: sticky error word, zero it first.
 * scratch (device, may be NULL): ceil(routes / 2048) * E ints let large sorts run on many CTAs. */
int umaq_route_sort(const void* expert_indices, int indices_are_int64, const float* routing_weights, int tokens,
                    int top_k, int num_experts, int* counts, int* offsets, int* sorted_route, int* route_pos,
                    float* sorted_weight, int* num_tiles, int* tile_table, int max_tiles, unsigned* status,
                    int* scratch, long long scratch_ints, void* stream);
/* out[i] = hidden[sorted_route[i] / top_k] (sorted_route == NULL: out[i] = hidden[i]);
 * permute != 0 writes every run of 8 elements as [0,4,1,5,2,6,3,7], the K order the
 * quantised grouped GEMM expects of its activations. */
int umaq_gather_rows(const void* hidden_bf16, const int* sorted_route, int top_k, long long routes, int hidden,
                     int permute, void* out_bf16, void* stream);
/* One grouped GEMM over the tile list.  mode 0: out[r, :I] = SiLU(act_r . Gate_e) * (act_r . Up_e)
 * (permute_out != 0 writes the permuted K order for a quantised mode-1 GEMM); mode 1:
 * out[r, :H] = route_weight[r] * (act_r . Down_e) (route_weight NULL = 1).  Replaces the
 * tile kernels at src/uma_qmoe/native/packed_q4_kernel.cu:560-776 and :894-1099.
 * variant: 0 = the library picks (CTA pairs for BF16 weights on 16,384 routes or more, one-CTA tiles
 * otherwise), 1 = persistent one-CTA tiles, 2 = persistent CTA pairs (tcgen05 cta_group::2; same tiles,
 * slower on B200 for the quantised encodings).  out is a dense [total_rows, I or H] BF16 matrix; the
 * mode-1 kernel of a quantised layer writes it with tensor stores when it starts on a 16-byte boundary,
 * with plain stores otherwise (same bytes either way). */
int umaq_grouped_gemm(const umaq_layer* layer, int mode, const void* act_bf16, long long total_rows,
                      const int* num_tiles, const int* tile_table, int max_tiles, const float* route_weight,
                      int permute_out, void* out_bf16, unsigned* status, int variant, void* stream);
/* The gate/up GEMM (mode 0) as umaq_moe_prefill runs it on the one-CTA kernel: no gathered copy of the
 * activations; sorted route r reads row sorted_route[r] / top_k of hidden_bf16 ([tokens, H]; for a quantised
 * layer already in the permuted k order, i.e. umaq_gather_rows with sorted_route NULL and permute != 0). */
int umaq_grouped_gemm_by_index(const umaq_layer* layer, const void* hidden_bf16, const int* sorted_route, int top_k,
                               long long routes, const int* num_tiles, const int* tile_table, int max_tiles,
                               int permute_out, void* out_bf16, unsigned* status, void* stream);
/* Expert-parallel routing table (no counterpart in the reference): local_ids[i] = local expert id of
 * expert_indices[i] on rank `rank`, or -1 (absent route) when another rank owns the expert.
 * placement 0: expert e on rank e % ranks as local e / ranks; 1: rank e / experts_per_rank, local e % experts_per_rank. */
int umaq_ep_local_ids(const void* expert_indices, int indices_are_int64, long long count, int ranks, int rank,
                      int experts_per_rank, int placement, int* local_ids, void* stream);
/* Expert-parallel dispatch into fixed-capacity segments, so that the exchange needs no row counts
 * on the host (no counterpart in the reference, which is single-device).  The routes were sorted by
 * key = owner_rank * experts_per_rank + local_expert (umaq_route_sort over the keys; offsets is its
 * [ranks*experts_per_rank + 1] output, sorted_key[s] the key of sorted route s).  Sorted route s of
 * owner d and rank j among d's routes is written to slot d*capacity + j: its activation row to
 * send_rows[slot], {local expert, weight bits} to send_meta[slot], slot to route_slot[route].  Unused
 * slots keep meta -1, which every kernel of this library treats as an absent route; routes beyond
 * the capacity get route_slot -1 and set *overflow (device int, sticky; the caller then repeats the
 * layer with exact counts). */
int umaq_ep_pack(const void* hidden_bf16, const int* sorted_route, const int* sorted_key, const float* sorted_weight,
                 const int* offsets, int routes, int top_k, int hidden, int ranks, int experts_per_rank, int capacity,
                 void* send_rows_bf16, int* send_meta, int* route_slot, int* overflow, void* stream);

/* ---- expert-parallel exchange over peer memory (no counterpart in the reference) -----------------
 * One process per GPU; every rank holds a buffer of the same layout that all ranks have mapped
 * (torch.distributed._symmetric_memory or any other peer mapping).  base[p] is rank p's buffer as seen
 * from this process.  The kernels use plain loads and stores on those addresses (no multicast, no TMA
 * on peer memory, no library call that is handed a peer pointer). */
typedef struct umaq_ep_peers {
  void* base[8];
  int32_t ranks;
  int32_t rank;
} umaq_ep_peers;
/* Dispatch: for every local token i and every rank p, the token's top_k expert ids (as int32) and routing
 * weights go to rows rank*tokens + i of p's id / weight tables (at ids_offset / weights_offset in p's
 * buffer); the activation row goes to the same row of p's row table (rows_offset) only when p owns at
 * least one of the token's experts (placement as in umaq_ep_local_ids).  present[i*ranks + p] = p if the
 * row was sent, else -1: the table the final combine uses to skip ranks that hold none of a token's
 * experts.  Replaces an all-gather of rows, ids and weights.  flags: UMAQ_EP_LOCAL_IDS writes into p's id table
 * what umaq_ep_local_ids would compute there (the id local to p, -1 for routes of other ranks), so that p needs no
 * pass of its own; UMAQ_EP_K_PERMUTED writes the rows in the k order the quantised GEMMs read
 * ([k0,k4,k1,k5,k2,k6,k3,k7] per run of 8; see umaq_moe_prefill_to_peers' rows_k_permuted). */
#define UMAQ_EP_LOCAL_IDS 1
#define UMAQ_EP_K_PERMUTED 2
int umaq_ep_push(const void* hidden_bf16 /* device [tokens, hidden] */, const void* expert_indices, int indices_are_int64,
                 const float* routing_weights, int tokens, int top_k, int hidden, int experts_per_rank, int placement,
                 int flags, const umaq_ep_peers* peers, size_t rows_offset, size_t ids_offset, size_t weights_offset,
                 int* present /* device [tokens, ranks] */, void* stream);
/* Barrier across the ranks' streams: writes the next epoch number into every peer's flag word for this
 * rank (at flags_offset, one uint32 per rank, zero at start) and waits until every peer's word for this
 * rank has reached it.  *epoch (device, this rank's own, zero at start) counts the barriers.  The wait is
 * bounded (about two seconds); if it gives up, *status becomes UMAQ_ERR_DEVICE_TIMEOUT and the kernel
 * returns, so a missing peer costs an error, not a hang. */
int umaq_ep_barrier(const umaq_ep_peers* peers, size_t flags_offset, unsigned* epoch /* device */,
                    unsigned* status /* device */, void* stream);
/* umaq_moe_prefill over the rows every rank pushed (tokens = ranks * segment_rows, expert ids local to
 * this rank, -1 for routes other ranks own), with the combine writing token (p, i)'s ordered partial sum
 * straight into row rank*segment_rows + i of rank p's parts table (parts_offset) instead of a local
 * tensor followed by an all-to-all.  Tokens without a route on this rank are not written; the reader
 * skips them through the `present` table of umaq_ep_push.  rows_k_permuted != 0: the rows were pushed with
 * UMAQ_EP_K_PERMUTED and the operator's own permutation pass is skipped (quantised layers only). */
int umaq_moe_prefill_to_peers(const umaq_layer* layer, const void* hidden_bf16, const void* expert_indices,
                              int indices_are_int64, const float* routing_weights, long long tokens, int top_k,
                              const umaq_ep_peers* peers, size_t parts_offset, int segment_rows, int rows_k_permuted,
                              void* workspace, size_t workspace_bytes, void* stream);
/* One expert-parallel layer over this rank's tokens from a single host call: umaq_ep_push (with both flags) ->
 * umaq_ep_barrier -> umaq_moe_prefill_to_peers over the rows that arrived -> umaq_ep_barrier ->
 * umaq_combine_routes over the partial sums (part_pos[i*ranks + p] = p*tokens + i), the five launches' arguments
 * being the ones documented above (offsets inside every rank's buffer; present [tokens, ranks]; epoch and status
 * device words, zero at start).  The workspace is umaq_prefill_workspace_bytes(tokens*ranks, top_k, local experts, ...).
 * A host whose launch calls are slow (an interpreter, several ranks sharing the cores) spends one call, not five. */
int umaq_ep_layer(const umaq_layer* layer, const void* hidden_bf16, const void* expert_indices, int indices_are_int64,
                  const float* routing_weights, int tokens, int top_k, int experts_per_rank, int placement,
                  const umaq_ep_peers* peers, size_t rows_offset, size_t ids_offset, size_t weights_offset,
                  size_t parts_offset, size_t flags_offset, int* present, const int* part_pos, unsigned* epoch,
                  unsigned* status, void* workspace, size_t workspace_bytes, void* out_bf16 /* [tokens, hidden] */,
                  void* stream);
/* out[t] = BF16 running sum of weighted[route_pos[t*top_k+s]] over the token's routes in
 * ascending expert order: the accumulation order of the reference's CPU path
 * (src/uma_qmoe/custom_op.py:312-338), in place of
 * reduce_topk_route_output_kernel (src/uma_qmoe/native/packed_q4_kernel.cu:1349-1365).
 * Routes with expert index -1 or route_pos -1 are absent and contribute nothing. */
int umaq_combine_routes(const void* weighted_bf16, const void* expert_indices, int indices_are_int64,
                        const int* route_pos, int tokens, int top_k, int hidden, void* out_bf16, void* stream);

/* ---- device-side packer -------------------------------------------------------
 * Quantises `elements` (a multiple of 128) BF16 values, row-major, into the
 * canonical Q4 (elements/2 bytes) or Q8 (elements bytes) codes and elements/128
 * float32 scales, bit-identical to the reference's host packer
 * (src/uma_qmoe/q4.py:136-165, src/uma_qmoe/target_pack.py:92-112). */
int umaq_quantize_groups(const void* src_bf16 /* device */, long long elements, int encoding,
                         void* codes /* device */, float* scales /* device */, void* stream);

/* ---- native pack reader and asynchronous staging --------------------------------------------------
 * Counterpart of the reference's Python readers (src/uma_qmoe/expert_pack.py:317-556 ExpertPackReader,
 * src/uma_qmoe/target_pack.py:493-812 TargetPackReader) and of the blocking per-layer staging in
 * src/uma_qmoe/native_backend.py:374-455.  umaq_pack_open maps the file read-only once and checks every
 * rule of the container before it returns a handle (prefix, SHA-256 of header, payload and every tensor,
 * canonical header JSON, model and policy identities, tensor layout, zero gaps, Q4 reserved code, scales);
 * the first violation fails the call with UMAQ_ERR_BAD_ARGUMENT and umaq_last_error() holds the same
 * message the Python readers raise.  kind: 0 = ExpertPack (UQMOEPK1), 1 = TargetPack (UQMOTPK1).
 * The expected_* strings may be NULL (not checked).  Views point into the mapping and stay valid until
 * umaq_pack_close. */
typedef struct umaq_pack umaq_pack;
typedef struct umaq_stage_ticket umaq_stage_ticket;
typedef struct umaq_pack_tensor {
  const char* name;
  const void* data;          /* canonical codes */
  size_t data_bytes;
  const void* scales;        /* float32 group scales, scale_bytes == 0 for bf16_le */
  size_t scale_bytes;
  int32_t encoding;          /* UMAQ_ENC_* */
  int32_t rank;
  long long shape[4];
  int32_t layer, expert, projection;   /* projection: 0 gate, 1 up, 2 down; -1 where the name is no expert tensor */
} umaq_pack_tensor;
int umaq_pack_open(const char* path, int kind, const char* expected_model_id, const char* expected_model_revision,
                   const char* expected_model_manifest_sha256, const char* expected_policy_id, umaq_pack** out);
void umaq_pack_close(umaq_pack* pack);
long long umaq_pack_tensor_count(const umaq_pack* pack);
const char* umaq_pack_header_json(const umaq_pack* pack, size_t* length);   /* the header bytes as stored (canonical JSON) */
int umaq_pack_layer_encoding(const umaq_pack* pack, int layer);             /* UMAQ_ENC_* or a negative error */
int umaq_pack_tensor_view(const umaq_pack* pack, const char* name, umaq_pack_tensor* view);
int umaq_pack_tensor_at(const umaq_pack* pack, long long index, umaq_pack_tensor* view);   /* file order */
/* SHA-256 of a host buffer with the reader's implementation (scalar_only != 0: without the CPU's SHA extensions). */
int umaq_sha256(const void* data, size_t bytes, int scalar_only, unsigned char digest[32]);
/* Stages layer `layer_index` of the pack into the caller's device tensors `dst` (the umaq_layer layout: per
 * projection all experts concatenated; dst->encoding / num_experts / hidden / intermediate say what is expected
 * and must match the pack).  Returns at once: a worker thread copies the tensors from the mapping into two
 * pinned 32 MiB buffers in turn (several threads per chunk) and issues one cudaMemcpyAsync per piece on a stream
 * of its own.  umaq_stage_wait blocks the host until everything is enqueued (not until it is copied), makes
 * `stream` wait for the copies, frees the ticket and reports the worker's host time.  One layer is staged at a
 * time per pack; close the pack only after every ticket has been waited for. */
int umaq_stage_layer_async(umaq_pack* pack, int layer_index, const umaq_layer* dst, int device, umaq_stage_ticket** ticket);
int umaq_stage_wait(umaq_stage_ticket* ticket, void* stream, double* host_seconds /* may be NULL */);

/* Measurement aid (no counterpart in the reference, not used by the operator): one launch that only reads
 * `bytes` bytes (a multiple of 16, 16-byte aligned) from device memory and throws them away.  mode 0: 16-byte
 * loads from many CTAs; mode 1: one persistent CTA per SM, cp.async.bulk copies into a shared-memory ring.
 * status_u32 (device, may be NULL) receives UMAQ_ERR_DEVICE_TIMEOUT if a bounded wait gave up.  Gives the floor
 * a batch-1 decode call of the same size can be compared with. */
int umaq_probe_stream(const void* src, size_t bytes, int mode, void* status_u32, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* UMAQ_B200_H */
