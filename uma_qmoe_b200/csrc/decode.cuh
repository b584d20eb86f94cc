// Parameter block and host launcher of the batch-1 decode kernel (decode.cu).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace umaq {

// Workspace layout (bytes): [0,1024) header -- the uint32 at byte 8 is the sticky status word, the
// uint32 words from byte 64 count finished gate/up tiles per slot (self-resetting); [1024,...) one run
// per slot (routed slots in route order, then the shared expert) that first holds the float32
// intermediate and then, in place, its fragment record.
// Must be zero before its first use.
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
  unsigned* sync;             // control words
  unsigned* amax;             // [2][16]
  float* inter_buf;
  // derived by the launcher
  int inter_total;            // sum of intermediate sizes over slots
  int stage_bytes;            // weight bytes per ring stage (16 rows x slice)
  int nstages;
};

size_t decode_workspace_bytes(int top_k, int inter, int shared_inter);
// Fills the derived fields, checks shapes and launches cooperatively on `stream`.
int launch_moe_decode(DecodeParams p, cudaStream_t stream);

}  // namespace umaq
