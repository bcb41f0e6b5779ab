// uint8 pixels -> normalised bf16 planes: y[b,c,:,:] = (x[b,c,:,:] - mean[c]) / std[c].
// 16 pixels per thread (one 16-byte load, two 16-byte stores).
#include "common.cuh"

namespace samb {
namespace {

__global__ void __launch_bounds__(256)
normalize_u8_kernel(const uint8_t* __restrict__ x, __nv_bfloat16* __restrict__ y, long long nvec, int plane_vecs,
                    int C, float m0, float m1, float m2, float s0, float s1, float s2) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const int c = int((i / plane_vecs) % C);
    const float mean = c == 0 ? m0 : (c == 1 ? m1 : m2);
    const float stdv = c == 0 ? s0 : (c == 1 ? s1 : s2);
    const uint4 v = reinterpret_cast<const uint4*>(x)[i];
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint32_t word = w[k >> 1] >> ((k & 1) * 16);
      const float a = __fdiv_rn(float(word & 0xffu) - mean, stdv);
      const float b = __fdiv_rn(float((word >> 8) & 0xffu) - mean, stdv);
      __nv_bfloat162 p = __floats2bfloat162_rn(a, b);
      o[k] = *reinterpret_cast<uint32_t*>(&p);
    }
    reinterpret_cast<uint4*>(y)[2 * i] = make_uint4(o[0], o[1], o[2], o[3]);
    reinterpret_cast<uint4*>(y)[2 * i + 1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

}  // namespace
}  // namespace samb

extern "C" int samb_normalize_u8(const uint8_t* x, void* y, int B, int C, int H, int W, const float* mean_host,
                                 const float* std_host, void* stream) {
  if (!x || !y || !mean_host || !std_host || B <= 0 || H <= 0 || W <= 0) return SAMB_E_BADARG;
  if (C != 3 || (H * (long long)W) % 16) return SAMB_E_SHAPE;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15u) return SAMB_E_ALIGN;
  const int plane_vecs = int(H * (long long)W / 16);
  const long long nvec = (long long)B * C * plane_vecs;
  long long blocks = (nvec + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  samb::normalize_u8_kernel<<<unsigned(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      x, static_cast<__nv_bfloat16*>(y), nvec, plane_vecs, C, mean_host[0], mean_host[1], mean_host[2], std_host[0],
      std_host[1], std_host[2]);
  return samb::launch_status();
}
