// Small supporting kernels: the device-side packer that writes the canonical Q4 / Q8 bytes.
#include "common.cuh"
#include "aux.cuh"

namespace umaq {
namespace {

// One warp per 128-element group; lane l owns elements 4l..4l+3.
// Bit-identical to the reference's host packer: scale = max|g| / qmax in float32 (1.0 for an
// all-zero group), code = clip(rint(g / scale), -qmax, qmax)
// (src/uma_qmoe/q4.py:136-165, src/uma_qmoe/target_pack.py:92-112 in the reference).
template <int QMAX, bool NIBBLES>
__global__ void quantize_groups_kernel(const __nv_bfloat16* __restrict__ src, long long groups,
                                       uint8_t* __restrict__ codes, float* __restrict__ scales) {
  const long long g = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (g >= groups) return;
  const int lane = threadIdx.x & 31;
  const uint2 raw = *reinterpret_cast<const uint2*>(src + g * 128 + lane * 4);
  float v[4];
  v[0] = __uint_as_float(raw.x << 16);
  v[1] = __uint_as_float(raw.x & 0xffff0000u);
  v[2] = __uint_as_float(raw.y << 16);
  v[3] = __uint_as_float(raw.y & 0xffff0000u);
  float am = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int o = 16; o; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
  float scale = __fdiv_rn(am, (float)QMAX);
  if (scale == 0.f) scale = 1.f;
  int q[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float r = rintf(__fdiv_rn(v[i], scale));
    r = fminf(fmaxf(r, (float)-QMAX), (float)QMAX);
    q[i] = (int)r;
  }
  if (NIBBLES) {
    const uint32_t w = (q[0] & 0xF) | ((q[1] & 0xF) << 4) | ((q[2] & 0xF) << 8) | ((q[3] & 0xF) << 12);
    reinterpret_cast<uint16_t*>(codes)[g * 32 + lane] = (uint16_t)w;
  } else {
    const uint32_t w = (q[0] & 0xFF) | ((q[1] & 0xFF) << 8) | ((q[2] & 0xFF) << 16) | ((uint32_t)(q[3] & 0xFF) << 24);
    reinterpret_cast<uint32_t*>(codes)[g * 32 + lane] = w;
  }
  if (lane == 0) scales[g] = scale;
}

}  // namespace

int launch_quantize_groups(const void* src_bf16, long long elements, int enc, void* codes, float* scales,
                           cudaStream_t stream) {
  if (!src_bf16 || !codes || !scales || elements <= 0 || elements % 128) {
    set_error("quantize: element count must be a positive multiple of 128");
    return ERR_BAD_ARGUMENT;
  }
  const long long groups = elements / 128;
  const int wpb = 8;
  const long long blocks = (groups + wpb - 1) / wpb;
  if (blocks > 0x7fffffffLL) { set_error("quantize: tensor too large"); return ERR_BAD_ARGUMENT; }
  const __nv_bfloat16* s = static_cast<const __nv_bfloat16*>(src_bf16);
  if (enc == ENC_Q4)
    quantize_groups_kernel<7, true><<<(unsigned)blocks, wpb * 32, 0, stream>>>(s, groups, static_cast<uint8_t*>(codes), scales);
  else if (enc == ENC_Q8)
    quantize_groups_kernel<127, false><<<(unsigned)blocks, wpb * 32, 0, stream>>>(s, groups, static_cast<uint8_t*>(codes), scales);
  else { set_error("quantize: encoding must be Q4 or Q8"); return ERR_BAD_ARGUMENT; }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("quantize: launch failed: %s", cudaGetErrorString(e)); return ERR_LAUNCH; }
  return ERR_NONE;
}

}  // namespace umaq
