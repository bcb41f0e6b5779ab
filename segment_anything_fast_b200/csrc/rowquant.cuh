// Per-row symmetric int8 quantisation building blocks shared by the row kernels (LayerNorm + quantise, plain
// quantise) and by the re-quantising Linear: bf16 unpack / pack, running |max| on packed bf16 pairs, and the exact
// rounding of x / scale without a division per element.
#pragma once

#include "common.cuh"

namespace samb {

constexpr float kAbsmaxFloor = 1e-5f;     // scale = max(absmax, floor) / 127: an all-zero row quantises to zeros

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {   // one shift or mask per element
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    f[2 * j] = __uint_as_float(w[j] << 16);
    f[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
  }
}
// Running maximum of |x| over packed bf16 pairs, kept as a packed pair (max and abs are exact in bf16).
__device__ __forceinline__ __nv_bfloat162 absmax8(__nv_bfloat162 m, const uint4& u) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int j = 0; j < 4; ++j) m = __hmax2(m, __habs2(p[j]));
  return m;
}
__device__ __forceinline__ float absmax_fold(__nv_bfloat162 m) {
  const float2 t = __bfloat1622float2(m);
  return fmaxf(t.x, t.y);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int j = 0; j < 4; ++j) p[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
  return u;
}

// Eight values -> eight int8 (two words), each rint(x / sc) bit-identical to the IEEE quotient, without a division
// or a conversion instruction per element.  x * (1/sc) is within 2^-23 relative (1.5e-5 absolute for |x/sc| <= 127.5)
// of the true quotient, so rounding it can only disagree with rounding the quotient next to a half-integer; only
// there is the real division evaluated.  fma(x, 1/sc, 1.5 * 2^23) rounds the exact product to the nearest (even)
// integer and leaves it, in two's complement, in the low mantissa bits, so its low byte is the int8; a second fma
// gives the distance of the product from that integer.  |x / sc| <= 127 (1 + 2^-24) because sc is the row's
// absmax / 127 (or larger), so nothing needs clamping.
__device__ __forceinline__ uint2 quant8(const uint4& raw, float sc, float inv_sc) {
  constexpr float kMagic = 12582912.0f;
  const f32x2 magic2 = pack2(kMagic, kMagic), inv2 = pack2(inv_sc, inv_sc);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  uint32_t b[8];
  float worst = 0.f;                 // largest distance of a product from the integer it rounded to: 0.5 = a tie
#pragma unroll
  for (int j = 0; j < 4; ++j) {      // two elements per packed fp32 instruction
    const f32x2 x2 = bf16x2_to_f32x2(w[j]);
    const f32x2 y2 = ffma2(x2, inv2, magic2);                    // the exact products, rounded to integers once
    const f32x2 e2 = ffma2(x2, inv2, fsub2(magic2, y2));         // products minus those integers (magic - y is exact)
    float y0, y1, e0, e1;
    unpack2(y2, y0, y1);
    unpack2(e2, e0, e1);
    worst = fmaxf(fmaxf(worst, fabsf(e0)), fabsf(e1));
    b[2 * j] = __float_as_uint(y0);
    b[2 * j + 1] = __float_as_uint(y1);
  }
  if (worst > 0.49996f) {            // rare: some element sits next to a half-integer; redo the eight exactly
    float f[8];
    unpack8(raw, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) b[j] = __float_as_uint(__fadd_rn(rintf(__fdiv_rn(f[j], sc)), kMagic));
  }
  const uint32_t b01 = __byte_perm(b[0], b[1], 0x0040), b23 = __byte_perm(b[2], b[3], 0x0040);
  const uint32_t b45 = __byte_perm(b[4], b[5], 0x0040), b67 = __byte_perm(b[6], b[7], 0x0040);
  return make_uint2(__byte_perm(b01, b23, 0x5410), __byte_perm(b45, b67, 0x5410));
}


// scale and its reciprocal for a row whose |max| is amax
__device__ __forceinline__ void row_scale(float amax, float& sc, float& inv_sc) {
  sc = __fdiv_rn(fmaxf(amax, kAbsmaxFloor), 127.0f);
  inv_sc = __frcp_rn(sc);
}

}  // namespace samb
