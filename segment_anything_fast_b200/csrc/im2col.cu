// Gather kernels that turn the two convolutions of the encoder into GEMM operands.
//  * patch embedding: non-overlapping P x P patches of an NCHW image become rows [c][ky][kx]
//    (the order of the flattened Conv2d weight), one row per patch, raster order.
//  * neck 3x3, padding 1, on token-major (NHWC) activations: each token's row is the 9 neighbouring
//    channel vectors [ky][kx][c], zeros outside the raster.
// Both move 16 bytes per thread per access and are pure bandwidth.
#include "common.cuh"

namespace samb {
namespace {

// x: [B, Cin, S, S] bf16 (S = grid*P) -> a: [B*grid*grid, Cin*P*P].  One thread copies 8 pixels of one
// image row segment; consecutive threads walk along the image row, so reads are contiguous.
__global__ void __launch_bounds__(256)
patch_rows_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ a, int B, int Cin, int grid, int P) {
  const int S = grid * P;
  const int vec_per_row = S / 8;
  const long long total = (long long)B * Cin * S * vec_per_row;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int vx = int(idx % vec_per_row);
    long long r = idx / vec_per_row;
    const int y = int(r % S);
    r /= S;
    const int c = int(r % Cin);
    const int b = int(r / Cin);
    const int x0 = vx * 8;
    const int px = x0 / P, kx = x0 - px * P;
    const int py = y / P, ky = y - py * P;
    const uint4 v = *reinterpret_cast<const uint4*>(x + ((((long long)b * Cin + c) * S + y) * S + x0));
    const long long row = ((long long)b * grid + py) * grid + px;
    *reinterpret_cast<uint4*>(a + row * ((long long)Cin * P * P) + (c * P + ky) * P + kx) = v;
  }
}

// The same gather straight from the uint8 pixels, with Sam.preprocess' normalisation applied on the way:
// a[row, (c, ky, kx)] = bf16((x[b, c, y, x] - mean[c]) / std[c]).  One thread turns 16 pixels (one 16-byte load)
// into 32 bytes of a patch row, so neither a normalised copy of the image nor a second pass over it exists.
__global__ void __launch_bounds__(256)
patch_rows_u8_kernel(const uint8_t* __restrict__ x, __nv_bfloat16* __restrict__ a, int B, int Cin, int grid, int P,
                     float m0, float m1, float m2, float s0, float s1, float s2) {
  const int S = grid * P;
  const int vec_per_row = S / 16;
  const long long total = (long long)B * Cin * S * vec_per_row;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int vx = int(idx % vec_per_row);
    long long r = idx / vec_per_row;
    const int y = int(r % S);
    r /= S;
    const int c = int(r % Cin);
    const int b = int(r / Cin);
    const int x0 = vx * 16;
    const int px = x0 / P, kx = x0 - px * P;
    const int py = y / P, ky = y - py * P;
    const float mean = c == 0 ? m0 : (c == 1 ? m1 : m2);
    const float stdv = c == 0 ? s0 : (c == 1 ? s1 : s2);
    const uint4 v = __ldcs(reinterpret_cast<const uint4*>(x + ((((long long)b * Cin + c) * S + y) * S + x0)));
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint32_t word = w[k >> 1] >> ((k & 1) * 16);
      const float lo = __fdiv_rn(float(word & 0xffu) - mean, stdv);
      const float hi = __fdiv_rn(float((word >> 8) & 0xffu) - mean, stdv);
      o[k] = pack_bf16x2(lo, hi);
    }
    const long long row = ((long long)b * grid + py) * grid + px;
    uint4* dst = reinterpret_cast<uint4*>(a + row * ((long long)Cin * P * P) + (c * P + ky) * P + kx);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

// x: [B*grid*grid, C] bf16 -> a: [B*grid*grid, 9*C]; one warp per (token, tap).
__global__ void __launch_bounds__(256)
conv3x3_rows_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ a, long long tokens, int grid,
                    int C) {
  const int lane = threadIdx.x & 31;
  const long long wid = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (wid >= tokens * 9) return;
  const long long t = wid / 9;
  const int tap = int(wid - t * 9);
  const int ky = tap / 3, kx = tap - ky * 3;
  const int px = int(t % grid);
  const int py = int((t / grid) % grid);
  const int sy = py + ky - 1, sx = px + kx - 1;
  const bool inside = sy >= 0 && sy < grid && sx >= 0 && sx < grid;
  const uint4* src = reinterpret_cast<const uint4*>(x + (t + (long long)(ky - 1) * grid + (kx - 1)) * C);
  uint4* dst = reinterpret_cast<uint4*>(a + t * (9LL * C) + (long long)tap * C);
  for (int v = lane; v < C / 8; v += 32) dst[v] = inside ? src[v] : make_uint4(0u, 0u, 0u, 0u);
}

}  // namespace
}  // namespace samb

extern "C" {

int samb_patch_rows(const void* x, void* a, int B, int Cin, int grid, int patch, void* stream) {
  if (!x || !a || B <= 0 || Cin <= 0 || grid <= 0 || patch <= 0) return SAMB_E_BADARG;
  if (patch % 8) return SAMB_E_SHAPE;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(a)) & 15u) return SAMB_E_ALIGN;
  const long long total = (long long)B * Cin * grid * patch * (grid * patch / 8);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 64) blocks = 148 * 64;
  samb::patch_rows_kernel<<<unsigned(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(a), B, Cin, grid, patch);
  return samb::launch_status();
}

int samb_patch_rows_u8(const uint8_t* x, void* a, int B, int Cin, int grid, int patch, const float* mean_host,
                       const float* std_host, void* stream) {
  if (!x || !a || !mean_host || !std_host || B <= 0 || grid <= 0 || patch <= 0) return SAMB_E_BADARG;
  if (Cin != 3 || patch % 16) return SAMB_E_SHAPE;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(a)) & 15u) return SAMB_E_ALIGN;
  const long long total = (long long)B * Cin * grid * patch * (grid * patch / 16);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 64) blocks = 148 * 64;
  samb::patch_rows_u8_kernel<<<unsigned(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      x, static_cast<__nv_bfloat16*>(a), B, Cin, grid, patch, mean_host[0], mean_host[1], mean_host[2], std_host[0],
      std_host[1], std_host[2]);
  return samb::launch_status();
}

int samb_conv3x3_rows(const void* x, void* a, int64_t tokens, int grid, int C, void* stream) {
  if (!x || !a || tokens < 0 || grid <= 0 || C <= 0) return SAMB_E_BADARG;
  if (C % 8 || tokens % ((int64_t)grid * grid)) return SAMB_E_SHAPE;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(a)) & 15u) return SAMB_E_ALIGN;
  if (tokens == 0) return SAMB_OK;
  const long long blocks = (tokens * 9 + 7) / 8;
  if (blocks > 0x7fffffffLL) return SAMB_E_SHAPE;
  samb::conv3x3_rows_kernel<<<unsigned(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(a), tokens, grid, C);
  return samb::launch_status();
}

}  // extern "C"
