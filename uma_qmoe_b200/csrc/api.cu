// extern "C" surface of libumaq_b200.so (declared in include/umaq_b200.h) plus the few host
// utilities the kernels' launchers share.
#include "../../include/umaq_b200.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "common.cuh"
#include "aux.cuh"
#include "decode.cuh"

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
  p.amax = reinterpret_cast<unsigned*>(ws + 64);
  p.inter_buf = reinterpret_cast<float*>(ws + kDecodeWsHeader);
  return launch_moe_decode(p, static_cast<cudaStream_t>(stream));
}

int umaq_quantize_groups(const void* src_bf16, long long elements, int encoding, void* codes, float* scales,
                         void* stream) {
  return launch_quantize_groups(src_bf16, elements, encoding, codes, scales, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
