// Bandwidth kernels: row LayerNorm (optionally scattering into the zero-padded window order and/or
// quantising each row to int8), plain per-row int8 quantisation, and the neck's channel LayerNorm
// with an NHWC -> NCHW transposing store.  One warp owns one row; a lane holds up to 8 vectors of
// 8 bf16 (C <= 2048), so every row is read once and written once with 16-byte accesses.
#include <cstdlib>

#include "common.cuh"
#include "rowquant.cuh"

namespace samb {
namespace {

constexpr int kMaxVec = 8;          // 16-byte vectors per lane
constexpr int kWarpsPerBlock = 8;

struct RowMap {
  // Output row -> input row for the window-partitioned order; window == 0 means identity.
  int grid, window, nw;
  __device__ __forceinline__ long long src_row(long long out_row) const {
    if (window == 0) return out_row;
    const int ww = window * window;
    const long long win = out_row / ww;
    const int l = int(out_row - win * ww);
    const int ly = l / window, lx = l - ly * window;
    const long long img = win / (nw * nw);
    const int wi = int(win - img * nw * nw);
    const int wy = wi / nw, wx = wi - wy * nw;
    const int y = wy * window + ly, x = wx * window + lx;
    if (y >= grid || x >= grid) return -1;      // zero padding
    return (img * grid + y) * grid + x;
  }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// kNorm: apply LayerNorm; kQuant: emit int8 + scale instead of bf16.
template <bool kNorm, bool kQuant>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
row_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
           __nv_bfloat16* __restrict__ y, int8_t* __restrict__ yq, float* __restrict__ scale, long long out_rows,
           int C, float eps, RowMap map) {
  const int lane = threadIdx.x & 31;
  const long long orow = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (orow >= out_rows) return;
  const int nvec = C >> 3;
  const long long irow = map.src_row(orow);

  if (irow < 0) {  // padded window token: zeros (and the floor scale)
    for (int i = lane; i < nvec; i += 32) {
      if (kQuant) reinterpret_cast<uint2*>(yq + orow * C)[i] = make_uint2(0u, 0u);
      else reinterpret_cast<uint4*>(y + orow * C)[i] = make_uint4(0u, 0u, 0u, 0u);
    }
    if (kQuant && lane == 0) scale[orow] = kAbsmaxFloor / 127.0f;
    return;
  }

  // The row stays in registers as raw 16-byte vectors (few registers -> many rows in flight per SM);
  // each pass unpacks on the fly.
  uint4 raw[kMaxVec];
  const uint4* xr = reinterpret_cast<const uint4*>(x + irow * C);
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int vi = i * 32 + lane;
    if (vi < nvec) raw[i] = xr[vi];
  }

  // Statistics with one accumulator for the even and one for the odd elements of the lane: the same additions, in
  // the same order, as the packed-pair arithmetic of rows_stream_kernel, so both kernels give the same bits.
  float mean = 0.f, rstd = 1.f;
  if (kNorm) {
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i)
      if (i * 32 + lane < nvec) {
        float f[8];
        unpack8(raw[i], f);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          s0 = __fadd_rn(s0, f[2 * j]);
          s1 = __fadd_rn(s1, f[2 * j + 1]);
        }
      }
    mean = warp_sum(__fadd_rn(s0, s1)) / float(C);
    float q0 = 0.f, q1 = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i)
      if (i * 32 + lane < nvec) {
        float f[8];
        unpack8(raw[i], f);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float d0 = __fsub_rn(f[2 * j], mean), d1 = __fsub_rn(f[2 * j + 1], mean);
          q0 = fmaf(d0, d0, q0);
          q1 = fmaf(d1, d1, q1);
        }
      }
    rstd = rsqrtf(warp_sum(__fadd_rn(q0, q1)) / float(C) + eps);
  }

  // normalised (bf16-rounded) values of vector i
  auto values = [&](int i, int vi, float (&f)[8]) {
    unpack8(raw[i], f);
    if (kNorm) {
      const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * vi), g1 = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * vi + 1);
      const float4 b0 = __ldg(reinterpret_cast<const float4*>(beta) + 2 * vi), b1 = __ldg(reinterpret_cast<const float4*>(beta) + 2 * vi + 1);
      const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
      const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = fmaf(__fmul_rn(__fsub_rn(f[j], mean), rstd), g[j], b[j]);
    }
  };

  if (!kQuant) {
    uint4* yr = reinterpret_cast<uint4*>(y + orow * C);
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int vi = i * 32 + lane;
      if (vi < nvec) {
        float f[8];
        values(i, vi, f);
        yr[vi] = pack8(f);
      }
    }
    return;
  }

  // int8: quantise the bf16-rounded value, as a quantised Linear fed a bf16 tensor would see it.
  // The normalised row replaces the raw one in the same registers (as bf16).
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int vi = i * 32 + lane;
    if (vi < nvec) {
      float f[8];
      values(i, vi, f);
      raw[i] = pack8(f);
      unpack8(raw[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
    }
  }
  amax = warp_max(amax);
  const float sc = __fdiv_rn(fmaxf(amax, kAbsmaxFloor), 127.0f);
  const float inv_sc = __frcp_rn(sc);
  if (lane == 0) scale[orow] = sc;
  uint2* qr = reinterpret_cast<uint2*>(yq + orow * C);
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int vi = i * 32 + lane;
    if (vi < nvec) {
      qr[vi] = quant8(raw[i], sc, inv_sc);
    }
  }
}

// LayerNorm of raster-order rows of exactly NV * 256 elements, bf16 out, with the affine parameters in registers.
// In row_kernel every row re-reads its gamma / beta (8 bytes per 2-byte element, through L1), which is what holds
// that kernel at 0.80 of the copy bandwidth.  Here a warp loads its 2 * NV * 8 parameter values once, then walks
// rows (row = warp + k * all warps) with the loads of the next DEPTH rows already in flight.  Arithmetic and its order
// are row_kernel's: same bits out.
constexpr int kPersistWarps = 4;
template <int NV, int DEPTH>
__global__ void __launch_bounds__(kPersistWarps * 32, 3)
ln_rows_persist_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ gamma,
                       const float* __restrict__ beta, __nv_bfloat16* __restrict__ y, long long rows, float eps) {
  constexpr int C = NV * 256;
  const int lane = threadIdx.x & 31;
  const long long step = (long long)gridDim.x * kPersistWarps;
  long long row = (long long)blockIdx.x * kPersistWarps + (threadIdx.x >> 5);
  float g[NV][8], b[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = i * 32 + lane;
    const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * vi), g1 = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * vi + 1);
    const float4 b0 = __ldg(reinterpret_cast<const float4*>(beta) + 2 * vi), b1 = __ldg(reinterpret_cast<const float4*>(beta) + 2 * vi + 1);
    g[i][0] = g0.x; g[i][1] = g0.y; g[i][2] = g0.z; g[i][3] = g0.w; g[i][4] = g1.x; g[i][5] = g1.y; g[i][6] = g1.z; g[i][7] = g1.w;
    b[i][0] = b0.x; b[i][1] = b0.y; b[i][2] = b0.z; b[i][3] = b0.w; b[i][4] = b1.x; b[i][5] = b1.y; b[i][6] = b1.z; b[i][7] = b1.w;
  }
  uint4 ahead[DEPTH][NV];                                 // rows row, row + step, ... (slot 0 = the next to be worked on)
#pragma unroll
  for (int d = 0; d < DEPTH; ++d) {
    const long long r = row + d * step;
#pragma unroll
    for (int i = 0; i < NV; ++i)
      ahead[d][i] = r < rows ? __ldcs(reinterpret_cast<const uint4*>(x + r * C) + i * 32 + lane) : make_uint4(0u, 0u, 0u, 0u);
  }
  for (; row < rows; row += step) {
    uint4 raw[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) raw[i] = ahead[0][i];
#pragma unroll
    for (int d = 0; d + 1 < DEPTH; ++d)
#pragma unroll
      for (int i = 0; i < NV; ++i) ahead[d][i] = ahead[d + 1][i];
    {
      const long long r = row + DEPTH * step;
      if (r < rows) {
#pragma unroll
        for (int i = 0; i < NV; ++i) ahead[DEPTH - 1][i] = __ldcs(reinterpret_cast<const uint4*>(x + r * C) + i * 32 + lane);
      }
    }
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float f[8];
      unpack8(raw[i], f);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        s0 = __fadd_rn(s0, f[2 * j]);
        s1 = __fadd_rn(s1, f[2 * j + 1]);
      }
    }
    const float mean = warp_sum(__fadd_rn(s0, s1)) / float(C);
    float q0 = 0.f, q1 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float f[8];
      unpack8(raw[i], f);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float d0 = __fsub_rn(f[2 * j], mean), d1 = __fsub_rn(f[2 * j + 1], mean);
        q0 = fmaf(d0, d0, q0);
        q1 = fmaf(d1, d1, q1);
      }
    }
    const float rstd = rsqrtf(warp_sum(__fadd_rn(q0, q1)) / float(C) + eps);
    uint4* yr = reinterpret_cast<uint4*>(y + row * C);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float f[8];
      unpack8(raw[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = fmaf(__fmul_rn(__fsub_rn(f[j], mean), rstd), g[i][j], b[i][j]);
      yr[i * 32 + lane] = pack8(f);
    }
  }
}

template <int NV>
int launch_ln_persist(const __nv_bfloat16* x, const float* gamma, const float* beta, __nv_bfloat16* y, long long rows,
                      float eps, cudaStream_t st) {
  long long blocks = (long long)sm_count() * 3;
  const long long need = (rows + kPersistWarps - 1) / kPersistWarps;
  if (blocks > need) blocks = need;
  // one row ahead: two ahead costs registers (spills at NV = 5) and measured slower (0.120 against 0.117 ms)
  ln_rows_persist_kernel<NV, 1><<<unsigned(blocks), kPersistWarps * 32, 0, st>>>(x, gamma, beta, y, rows, eps);
  return launch_status();
}

__device__ __forceinline__ void cp_async_16(uint32_t smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Persistent, prefetching form of the row kernels for raster-order rows of up to NV * 256 elements: a warp owns
// every G-th row (G = warps in the grid) and keeps the next STAGES - 1 of its rows in flight as 16-byte cp.async
// copies into a private shared-memory ring (each lane later reads back exactly the pieces it copied, so no
// barrier is involved and nothing can hang), which decouples the bytes in flight per SM from the register
// budget.  The arithmetic, and its order, are those of row_kernel / quant_rows_kernel: same bits out.
template <bool kNorm, bool kQuant, bool kGelu, int NV, int STAGES>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
rows_stream_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                   __nv_bfloat16* __restrict__ y, int8_t* __restrict__ yq, float* __restrict__ scale, long long rows,
                   int C, float eps) {
  extern __shared__ uint4 ring[];                         // [warp][stage][vector i][lane]
  constexpr bool kDirect = STAGES == 0;                   // no ring: plain loads, many vectors per lane in flight
  constexpr int kRing = kDirect ? 1 : STAGES;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long G = (long long)gridDim.x * kWarpsPerBlock;
  const int nvec = C >> 3;
  uint4* mine = ring + (size_t)warp * kRing * NV * 32 + lane;
  auto issue = [&](long long row, int st) {
    if (kDirect) return;
    if (row < rows) {
      const uint4* xr = reinterpret_cast<const uint4*>(x + row * C);
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int vi = i * 32 + lane;
        if (vi < nvec) cp_async_16(smem_u32(mine + (st * NV + i) * 32), xr + vi);
      }
    }
    cp_async_commit();                                    // an empty group past the last row keeps the count uniform
  };
  const long long row0 = (long long)blockIdx.x * kWarpsPerBlock + warp;
#pragma unroll
  for (int st = 0; st < kRing - 1; ++st) issue(row0 + st * G, st);
  int it = 0;
  for (long long row = row0; row < rows; row += G, ++it) {
    uint4 raw[NV];
    if (kDirect) {
      const uint4* xr = reinterpret_cast<const uint4*>(x + row * C);
#pragma unroll
      for (int i = 0; i < NV; ++i)
        if (i * 32 + lane < nvec) raw[i] = __ldcs(xr + i * 32 + lane);     // read once: streaming
    } else {
      issue(row + (kRing - 1) * G, (it + kRing - 1) % kRing);
      cp_async_wait<kRing - 1>();                         // this row's copies have landed
      const int st = it % kRing;
#pragma unroll
      for (int i = 0; i < NV; ++i)
        if (i * 32 + lane < nvec) raw[i] = mine[(st * NV + i) * 32];
    }

    __nv_bfloat162 m2 = __floats2bfloat162_rn(0.f, 0.f);       // running |max| of the (bf16) values to quantise
    if (kNorm) {
      // the row is unpacked once and stays in registers as fp32 pairs through the three passes
      f32x2 v[NV][4];
      f32x2 s2 = pack2(0.f, 0.f);
#pragma unroll
      for (int i = 0; i < NV; ++i)
        if (i * 32 + lane < nvec) {
          const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            v[i][j] = bf16x2_to_f32x2(w[j]);
            s2 = fadd2(s2, v[i][j]);
          }
        }
      float s_lo, s_hi;
      unpack2(s2, s_lo, s_hi);
      const float mean = warp_sum(s_lo + s_hi) / float(C);
      const f32x2 mean2 = pack2(mean, mean);
      f32x2 q2 = pack2(0.f, 0.f);
#pragma unroll
      for (int i = 0; i < NV; ++i)
        if (i * 32 + lane < nvec) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            v[i][j] = fsub2(v[i][j], mean2);
            q2 = ffma2(v[i][j], v[i][j], q2);
          }
        }
      float q_lo, q_hi;
      unpack2(q2, q_lo, q_hi);
      const float rstd = rsqrtf(warp_sum(q_lo + q_hi) / float(C) + eps);
      const f32x2 rstd2 = pack2(rstd, rstd);
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int vi = i * 32 + lane;
        if (vi < nvec) {
          // eight gains and eight offsets as four fp32 pairs each
          const ulonglong2 g0 = __ldg(reinterpret_cast<const ulonglong2*>(gamma) + 2 * vi), g1 = __ldg(reinterpret_cast<const ulonglong2*>(gamma) + 2 * vi + 1);
          const ulonglong2 b0 = __ldg(reinterpret_cast<const ulonglong2*>(beta) + 2 * vi), b1 = __ldg(reinterpret_cast<const ulonglong2*>(beta) + 2 * vi + 1);
          const f32x2 g[4] = {g0.x, g0.y, g1.x, g1.y}, b[4] = {b0.x, b0.y, b1.x, b1.y};
          uint32_t o[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float lo, hi;
            unpack2(ffma2(fmul2(v[i][j], rstd2), g[j], b[j]), lo, hi);
            o[j] = pack_bf16x2(lo, hi);
          }
          raw[i] = make_uint4(o[0], o[1], o[2], o[3]);
          if (kQuant) m2 = absmax8(m2, raw[i]);
          else reinterpret_cast<uint4*>(y + row * C)[vi] = raw[i];
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < NV; ++i)
        if (i * 32 + lane < nvec) {
          if (kGelu) {                                    // bf16(gelu(x)) is what gets quantised
            float f[8];
            unpack8(raw[i], f);
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = gelu_erf(f[j]);
            raw[i] = pack8(f);
          }
          m2 = absmax8(m2, raw[i]);
        }
    }
    if (kQuant) {
      const float amax = warp_max(absmax_fold(m2));
      const float sc = __fdiv_rn(fmaxf(amax, kAbsmaxFloor), 127.0f);
      const float inv_sc = __frcp_rn(sc);
      if (lane == 0) scale[row] = sc;
      uint2* qr = reinterpret_cast<uint2*>(yq + row * C);
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int vi = i * 32 + lane;
        if (vi < nvec) {
          qr[vi] = quant8(raw[i], sc, inv_sc);
        }
      }
    }
  }
  if (!kDirect) cp_async_wait<0>();
}

// Host side of rows_stream_kernel: picks the vector count, sizes the ring and the persistent grid.
template <bool kNorm, bool kQuant, bool kGelu, int NV, int STAGES>
int launch_stream_nv(const __nv_bfloat16* x, const float* gamma, const float* beta, __nv_bfloat16* y, int8_t* yq,
                     float* scale, long long rows, int C, float eps, cudaStream_t st) {
  auto kern = rows_stream_kernel<kNorm, kQuant, kGelu, NV, STAGES>;
  constexpr int kSmem = kWarpsPerBlock * STAGES * NV * 32 * 16;
  long long blocks = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
  if (STAGES > 0) {                     // persistent: exactly one resident wave
    static int per_sm = 0;              // resident blocks per SM of this instantiation (a device fact, asked once)
    if (per_sm == 0) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess) return SAMB_E_LAUNCH;
      int n = 0;
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, kWarpsPerBlock * 32, kSmem) != cudaSuccess || n < 1)
        return SAMB_E_LAUNCH;
      per_sm = n;
    }
    const long long cap = (long long)sm_count() * per_sm;
    if (blocks > cap) blocks = cap;
  } else if (blocks > 0x7fffffffLL) {
    return SAMB_E_SHAPE;
  }
  kern<<<unsigned(blocks), kWarpsPerBlock * 32, kSmem, st>>>(x, gamma, beta, y, yq, scale, rows, C, eps);
  return launch_status();
}
// SAMB_ROWS_DIRECT=1 in the environment (a tuning switch) makes the narrow-row kernels use plain loads, one
// row per warp and a block per eight rows, instead of the persistent prefetching form.
inline bool rows_direct() {
  static int v = -1;
  if (v < 0) v = getenv("SAMB_ROWS_DIRECT") != nullptr ? 1 : 0;
  return v == 1;
}
template <bool kNorm, bool kQuant, bool kGelu>
int launch_stream(const __nv_bfloat16* x, const float* gamma, const float* beta, __nv_bfloat16* y, int8_t* yq,
                  float* scale, long long rows, int C, float eps, cudaStream_t st) {
  const int nv = (C / 8 + 31) / 32;
  // measured on 131072 x 1280: quantise-only rows are fastest with plain loads (0.099 against 0.104 ms), LayerNorm
  // + quantise with the prefetch ring (0.172 against 0.230 ms)
#define SAMB_NV(NV, ST)                                                                                          \
  return (rows_direct() || !kNorm) ? launch_stream_nv<kNorm, kQuant, kGelu, NV, 0>(x, gamma, beta, y, yq, scale, rows, C, eps, st) \
                       : launch_stream_nv<kNorm, kQuant, kGelu, NV, ST>(x, gamma, beta, y, yq, scale, rows, C, eps, st)
  if (nv <= 1) SAMB_NV(1, 4);
  if (nv <= 3) SAMB_NV(3, 4);
  if (nv <= 5) SAMB_NV(5, 4);
  SAMB_NV(8, 3);
#undef SAMB_NV
}

// Wide rows (C up to 3 * 256 * 8 = 6144): a 256-thread block per row, up to three 16-byte vectors per thread,
// absmax through shared memory.  Persistent blocks walk every gridDim-th row and keep their next STAGES - 1 rows
// in flight as cp.async copies into a per-thread ring (each thread reads back its own pieces).
// kGelu: the row first goes through the exact-erf GELU and is rounded back to bf16 (the activation tensor
// the reference materialises between lin1 and lin2), then quantised.
template <bool kGelu, int STAGES>
__global__ void __launch_bounds__(256)
quant_rows_wide_kernel(const __nv_bfloat16* __restrict__ x, int8_t* __restrict__ yq, float* __restrict__ scale,
                       long long rows, int C) {
  extern __shared__ uint4 ring[];                         // [stage][vector i][thread]
  __shared__ float s_max[2][8];
  const int nvec = C >> 3;
  uint4* mine = ring + threadIdx.x;
  auto issue = [&](long long row, int st) {
    if (row < rows) {
      const uint4* xr = reinterpret_cast<const uint4*>(x + row * C);
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        const int vi = i * 256 + threadIdx.x;
        if (vi < nvec) cp_async_16(smem_u32(mine + (st * 3 + i) * 256), xr + vi);
      }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) issue((long long)blockIdx.x + (long long)st * gridDim.x, st);
  int it = 0;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x, ++it) {
    issue(row + (long long)(STAGES - 1) * gridDim.x, (it + STAGES - 1) % STAGES);
    cp_async_wait<STAGES - 1>();
    const int st = it % STAGES;
    uint4 raw[3];
    __nv_bfloat162 m2 = __floats2bfloat162_rn(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      const int vi = i * 256 + threadIdx.x;
      if (vi < nvec) {
        raw[i] = mine[(st * 3 + i) * 256];
        if (kGelu) {
          float f[8];
          unpack8(raw[i], f);
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] = gelu_erf(f[j]);
          raw[i] = pack8(f);
        }
        m2 = absmax8(m2, raw[i]);
      }
    }
    float amax = absmax_fold(m2);
    amax = warp_max(amax);
    float* sm = s_max[it & 1];                            // two buffers: one barrier per row is enough
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = sm[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) amax = fmaxf(amax, sm[w]);
    const float sc = __fdiv_rn(fmaxf(amax, kAbsmaxFloor), 127.0f);
    const float inv_sc = __frcp_rn(sc);
    if (threadIdx.x == 0) scale[row] = sc;
    uint2* qr = reinterpret_cast<uint2*>(yq + row * C);
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      const int vi = i * 256 + threadIdx.x;
      if (vi < nvec) {
        qr[vi] = quant8(raw[i], sc, inv_sc);
      }
    }
  }
  cp_async_wait<0>();
}

// Channel LayerNorm of x[tokens, C] (NHWC rows) written as out[img, C, hw] (NCHW).  One block
// normalises 32 consecutive tokens (one warp per token, 4 rounds of 8) into shared memory, then
// writes 32-token runs per channel.
template <bool kTranspose>
__global__ void __launch_bounds__(256)
ln2d_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
            __nv_bfloat16* __restrict__ out, long long tokens, int C, int hw, float eps) {
  extern __shared__ __nv_bfloat16 tile[];   // [32][C + 2]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long t0 = (long long)blockIdx.x * 32;
  const int pitch = C + 2;
  for (int r = warp; r < 32; r += 8) {
    const long long t = t0 + r;
    if (t >= tokens) break;
    const __nv_bfloat16* xr = x + t * C;
    float s = 0.f;
    for (int c = lane; c < C; c += 32) s += __bfloat162float(xr[c]);
    const float mean = warp_sum(s) / float(C);
    float q = 0.f;
    for (int c = lane; c < C; c += 32) {
      const float d = __bfloat162float(xr[c]) - mean;
      q += d * d;
    }
    const float rstd = rsqrtf(warp_sum(q) / float(C) + eps);
    for (int c = lane; c < C; c += 32) {
      const float o = (__bfloat162float(xr[c]) - mean) * rstd * gamma[c] + beta[c];
      if (kTranspose) tile[r * pitch + c] = __float2bfloat16_rn(o);
      else out[t * C + c] = __float2bfloat16_rn(o);
    }
  }
  if (!kTranspose) return;
  __syncthreads();
  // hw is a multiple of 32 (checked on the host), so a 32-token run never straddles two images.
  const long long img = t0 / hw;
  const int p0 = int(t0 - img * hw);
  for (int c = warp; c < C; c += 8) {
    if (t0 + lane < tokens) out[(img * C + c) * hw + p0 + lane] = tile[lane * pitch + c];
  }
}

int check_rows(const void* x, long long rows, int C) {
  if (x == nullptr || rows < 0 || C <= 0) return SAMB_E_BADARG;
  if (C % 8 || C > kMaxVec * 32 * 8) return SAMB_E_SHAPE;
  if (reinterpret_cast<uintptr_t>(x) & 15u) return SAMB_E_ALIGN;
  return SAMB_OK;
}

int make_map(RowMap* m, long long rows, int grid, int window, long long* out_rows) {
  m->grid = grid;
  m->window = window;
  m->nw = 0;
  *out_rows = rows;
  if (window < 0 || grid < 0) return SAMB_E_BADARG;
  if (window == 0) return SAMB_OK;
  if (grid <= 0 || rows % ((long long)grid * grid)) return SAMB_E_SHAPE;
  m->nw = (grid + window - 1) / window;
  *out_rows = rows / ((long long)grid * grid) * m->nw * m->nw * window * window;
  return SAMB_OK;
}

template <bool kNorm, bool kQuant>
int launch_rows(const void* x, const float* gamma, const float* beta, void* y, int8_t* yq, float* scale,
                int64_t rows, int C, float eps, int grid, int window, void* stream) {
  if (int e = check_rows(x, rows, C)) return e;
  if (kNorm && (gamma == nullptr || beta == nullptr)) return SAMB_E_BADARG;
  if (kQuant ? (yq == nullptr || scale == nullptr) : (y == nullptr)) return SAMB_E_BADARG;
  RowMap map;
  long long out_rows;
  if (int e = make_map(&map, rows, grid, window, &out_rows)) return e;
  if (out_rows == 0) return SAMB_OK;
  const long long blocks = (out_rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
  if (blocks > 0x7fffffffLL) return SAMB_E_SHAPE;
  // Raster order + int8 output: the persistent prefetching kernel (0.172 against 0.204 ms for 131072 x 1280).
  // The bf16 form does not gain from that kernel (0.149 against 0.141 ms for row_kernel); it has its own below.
  if (window == 0 && (kQuant || getenv("SAMB_ROWS_STREAM") != nullptr))
    return launch_stream<kNorm, kQuant, false>(static_cast<const __nv_bfloat16*>(x), gamma, beta,
                                               static_cast<__nv_bfloat16*>(y), yq, scale, out_rows, C, eps,
                                               static_cast<cudaStream_t>(stream));
  // Raster order + bf16 output + a row of 3, 4 or 5 x 256 elements (ViT-B / L / H): parameters in registers.
  if constexpr (kNorm && !kQuant) {
    if (window == 0 && C % 256 == 0 && C / 256 >= 3 && C / 256 <= 5 && getenv("SAMB_LN_ROWKERNEL") == nullptr &&
        !((reinterpret_cast<uintptr_t>(gamma) | reinterpret_cast<uintptr_t>(beta)) & 15u)) {
      const auto* xb = static_cast<const __nv_bfloat16*>(x);
      auto* yb = static_cast<__nv_bfloat16*>(y);
      auto st = static_cast<cudaStream_t>(stream);
      switch (C / 256) {
        case 3: return launch_ln_persist<3>(xb, gamma, beta, yb, out_rows, eps, st);
        case 4: return launch_ln_persist<4>(xb, gamma, beta, yb, out_rows, eps, st);
        default: return launch_ln_persist<5>(xb, gamma, beta, yb, out_rows, eps, st);
      }
    }
  }
  row_kernel<kNorm, kQuant><<<unsigned(blocks), kWarpsPerBlock * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), gamma, beta, static_cast<__nv_bfloat16*>(y), yq, scale, out_rows, C, eps,
      map);
  return launch_status();
}

}  // namespace
}  // namespace samb

namespace samb {
namespace {
int launch_quant_rows(const void* x, int8_t* yq, float* scale, int64_t rows, int C, bool gelu, void* stream) {
  if (x == nullptr || yq == nullptr || scale == nullptr || rows < 0 || C <= 0) return SAMB_E_BADARG;
  if (C % 8 || C > 24 * 256) return SAMB_E_SHAPE;
  if ((reinterpret_cast<uintptr_t>(x) & 15u) || (reinterpret_cast<uintptr_t>(yq) & 7u)) return SAMB_E_ALIGN;
  if (rows == 0) return SAMB_OK;
  const long long blocks = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
  if (blocks > 0x7fffffffLL) return SAMB_E_SHAPE;
  auto st = static_cast<cudaStream_t>(stream);
  auto xb = static_cast<const __nv_bfloat16*>(x);
  if (C <= 8 * 256) {
    if (gelu) return launch_stream<false, true, true>(xb, nullptr, nullptr, nullptr, yq, scale, rows, C, 0.f, st);
    return launch_stream<false, true, false>(xb, nullptr, nullptr, nullptr, yq, scale, rows, C, 0.f, st);
  } else if (getenv("SAMB_WIDE_WARP") != nullptr) {
    // tuning switch: a warp per row with 20 (24) 16-byte vectors per lane in flight (0.53 ms for 131072 x 5120
    // against 0.43 ms for the block-per-row form below, which is the default)
    if (C <= 20 * 256) {
      if (gelu) return launch_stream_nv<false, true, true, 20, 0>(xb, nullptr, nullptr, nullptr, yq, scale, rows, C, 0.f, st);
      return launch_stream_nv<false, true, false, 20, 0>(xb, nullptr, nullptr, nullptr, yq, scale, rows, C, 0.f, st);
    }
    if (gelu) return launch_stream_nv<false, true, true, 24, 0>(xb, nullptr, nullptr, nullptr, yq, scale, rows, C, 0.f, st);
    return launch_stream_nv<false, true, false, 24, 0>(xb, nullptr, nullptr, nullptr, yq, scale, rows, C, 0.f, st);
  } else {
    constexpr int kStages = 3, kSmem = kStages * 3 * 256 * 16;
    static int per_sm[2] = {0, 0};      // resident blocks per SM (a device fact, asked once per variant)
    if (per_sm[gelu] == 0) {
      int n = 0;
      const cudaError_t e = gelu ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, quant_rows_wide_kernel<true, kStages>, 256, kSmem)
                                 : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, quant_rows_wide_kernel<false, kStages>, 256, kSmem);
      if (e != cudaSuccess || n < 1) return SAMB_E_LAUNCH;
      per_sm[gelu] = n;
    }
    const long long cap = (long long)sm_count() * per_sm[gelu];
    const long long nb = rows < cap ? rows : cap;
    if (gelu) quant_rows_wide_kernel<true, kStages><<<unsigned(nb), 256, kSmem, st>>>(xb, yq, scale, rows, C);
    else quant_rows_wide_kernel<false, kStages><<<unsigned(nb), 256, kSmem, st>>>(xb, yq, scale, rows, C);
  }
  return launch_status();
}
}  // namespace
}  // namespace samb

extern "C" {

int samb_layernorm_bf16(const void* x, const float* gamma, const float* beta, void* y, int64_t rows, int C, float eps,
                        int grid, int window, void* stream) {
  return samb::launch_rows<true, false>(x, gamma, beta, y, nullptr, nullptr, rows, C, eps, grid, window, stream);
}

int samb_layernorm_quant_i8(const void* x, const float* gamma, const float* beta, int8_t* yq, float* scale,
                            int64_t rows, int C, float eps, int grid, int window, void* stream) {
  return samb::launch_rows<true, true>(x, gamma, beta, nullptr, yq, scale, rows, C, eps, grid, window, stream);
}

int samb_quant_rows_i8(const void* x, int8_t* yq, float* scale, int64_t rows, int C, void* stream) {
  return samb::launch_quant_rows(x, yq, scale, rows, C, false, stream);
}

int samb_gelu_quant_rows_i8(const void* x, int8_t* yq, float* scale, int64_t rows, int C, void* stream) {
  return samb::launch_quant_rows(x, yq, scale, rows, C, true, stream);
}

int samb_layernorm2d_nchw(const void* x, const float* gamma, const float* beta, void* out, int64_t tokens, int C,
                          int hw, float eps, int to_nchw, void* stream) {
  if (x == nullptr || gamma == nullptr || beta == nullptr || out == nullptr || tokens < 0 || C <= 0 || hw <= 0)
    return SAMB_E_BADARG;
  if (C > 4096 || (to_nchw && (hw % 32 || tokens % hw))) return SAMB_E_SHAPE;
  if (tokens == 0) return SAMB_OK;
  const long long blocks = (tokens + 31) / 32;
  const size_t smem = to_nchw ? size_t(32) * (C + 2) * sizeof(__nv_bfloat16) : 0;
  if (smem > 48 * 1024) return SAMB_E_SHAPE;
  auto st = static_cast<cudaStream_t>(stream);
  if (to_nchw)
    samb::ln2d_kernel<true><<<unsigned(blocks), 256, smem, st>>>(static_cast<const __nv_bfloat16*>(x), gamma, beta,
                                                                 static_cast<__nv_bfloat16*>(out), tokens, C, hw, eps);
  else
    samb::ln2d_kernel<false><<<unsigned(blocks), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), gamma, beta,
                                                               static_cast<__nv_bfloat16*>(out), tokens, C, hw, eps);
  return samb::launch_status();
}

}  // extern "C"
