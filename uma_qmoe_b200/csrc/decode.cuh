// Parameter block, launch plan and host launcher of the batch-1 decode kernels (decode.cu).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace umaq {

// Workspace layout (bytes): [0,1024) header -- the uint32 at byte 8 is the sticky status word;
// [1024,...) the intermediate vectors the gate/up kernel leaves for the down kernel, already in the
// order of the down kernel's MMA fragments (BF16; Q8 rows hold every value twice, as x and 16 x).
// The header must be zero before the first use.
constexpr size_t kDecodeWsHeader = 1024;

// One kind of weight rows a decode kernel streams: the routed experts of the layer, or the Qwen
// shared expert (always BF16).
struct DecodeKind {
  int enc;          // ENC_*
  int units;        // gate/up kernel: work units of 8 features (8 gate rows + 8 up rows)
  int row_bytes;    // gate/up: bytes of a weight row; down: bytes of one slot's part of a row
  int ch;           // gate/up: row bytes per ring stage (row_bytes = nch * ch)
  int nch;          // gate/up: ring stages per unit
  int ips;          // items per stage; an item = 64 bytes of each of the 16 MMA rows
  int item_bytes;   // 64
  int r16;          // 16-byte activation-fragment chunks per lane and item: 4 (Q4, Q8) or 1 (BF16)
  int groups;       // float32 scales per weight row (K / 128); 0 for BF16
  int nvs;          // down: slots of an MMA tile (top_k routed slots, or K segments of the shared expert)
  int ng;           // down: slot dimension of the fragment layout (power of two >= nvs)
  int mstride;      // shared-memory stride: gate/up from the gate block to the up block of a stage (8 ch + 64);
                    // down between the slots' row blocks
  int frag_off;     // shared-memory offset of the activation fragments
  int gsum_off;     // shared-memory offset of the per-item activation sums (bias correction)
  int frag_bytes;   // bytes of the activation fragments
  int ws_off;       // byte offset (after the header) of this kind's intermediate fragments in the workspace
  float bias;       // the constant every decoded code carries: 136 (Q4), 2304 (Q8), 0 (BF16)
};

struct DecodeKernelPlan {
  DecodeKind kind[2];       // [0] routed experts, [1] shared expert (units / nvs 0 when absent)
  long long cost[2];        // gate/up: bytes per unit and MMA row, the weight of a unit when CTAs split the work
  long long total_cost;
  int grid;                 // CTAs (<= one per SM)
  int stages;               // ring depth
  int stage_bytes;
  int scale_off;            // offset of the scale area inside a stage
  int red_off;              // per-warp partial sums [unit][warp][16]
  int red2_off;             // down: the same for the shared expert
  int ysum_off;             // down: per (row pair, kind, row, slot) sums over the warps
  int bar_off;              // mbarriers: full[stages], empty[stages]
  int bulk_scales;          // scales travel as bulk copies (sizes and offsets are multiples of 16 bytes), else as 8-byte cp.async
  int resident;             // down: the CTA's whole share is loaded at once, slot by slot (no ring)
  int pair_stride;          // down: bytes from one row pair's weights to the next (ring: stage_bytes)
  int sc_base;              // down: offset of the scales (ring: inside a stage)
  int sc_pair_stride;       // down: bytes from one row pair's scales to the next
  int sc_slot_stride;       // down: bytes from one slot's scales to the next
  int smem_bytes;
  int max_units;            // most units (gate/up) or row pairs (down) any CTA gets
  int producers;            // warps that feed the ring when a CTA's share does not fit it at once
  int pair_step;            // down: row pairs a consumer round takes together (2 shares the fragments; 1 when the ring
                            // is too short to hold two rounds)
};

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
  unsigned* sync;             // header words; sync[2] is the status word, sync[4] counts the gate/up CTAs that have
                              // finished, over all calls, and sync[6] is the count the current call's down kernel
                              // waits for (every call adds its grid size; the words are never reset)
  uint8_t* inter_buf;         // intermediate fragments (after the header)
  // launch plans, filled by launch_moe_decode
  DecodeKernelPlan g;         // gate/up + SwiGLU kernel
  DecodeKernelPlan d;         // down + combine kernel
  int debug;                  // measurement switches: 1 = consumers skip the arithmetic, 2 = producers skip the weight
                              // copies, 4 = CTA 0 writes %globaltimer stamps into the header (bytes 128 and up)
};

size_t decode_workspace_bytes(int top_k, int inter, int shared_inter);
// Checks the shapes, plans both kernels and launches them on `stream`.
int launch_moe_decode(DecodeParams p, cudaStream_t stream);

}  // namespace umaq
