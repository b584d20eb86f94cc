// Parameter block and host launcher of the batch-1 decode kernels (decode.cu).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace umaq {

// Workspace layout (bytes): [0,1024) header -- the uint32 at byte 8 is the sticky status word;
// [1024,...) 4 * intermediate bytes per slot (routed slots in route order, then the shared expert) that
// hold the record the gate/up kernel leaves for the down kernel (fp16 fragments in 32-value chunks with
// their prescales and bias sums, or the BF16 vector for BF16 rows).  The header must be zero before the
// first use.
constexpr size_t kDecodeWsHeader = 1024;

struct DecodeParams {
  // routed experts of one layer, all experts concatenated per projection (expert stride =
  // rows * row_bytes for the codes, rows * K/128 floats for the scales)
  const uint8_t* gate;
  const uint8_t* up;
  const uint8_t* down;
  const float* gate_s;
  const float* up_s;
  const float* down_s;
  int enc;
  int experts;
  int hidden;
  int inter;
  int top_k;
  const __nv_bfloat16* x;     // [hidden]
  const void* idx;            // [top_k] int32 or int64
  int idx64;
  const float* w;             // [top_k]
  // optional Qwen shared expert (BF16) and its sigmoid gate vector
  const __nv_bfloat16* sh_gate;
  const __nv_bfloat16* sh_up;
  const __nv_bfloat16* sh_down;
  const __nv_bfloat16* sh_gatevec;
  int shared_inter;
  __nv_bfloat16* out;         // [hidden]
  // workspace
  unsigned* sync;             // header words; sync[2] is the status word
  float* inter_buf;           // the slots' records (4 * intermediate bytes apart)
};

size_t decode_workspace_bytes(int top_k, int inter, int shared_inter);
// Checks the shapes and launches the two kernels on `stream`.
int launch_moe_decode(DecodeParams p, cudaStream_t stream);

}  // namespace umaq
