// Tensor-pipe rate probe: every CTA issues back-to-back tcgen05.mma (M 128, N 256) on operands that stay in its
// shared memory, so nothing but the tensor pipe (and the power budget) limits it.  The number it gives is the
// denominator for roofline fractions of the int8 GEMMs, for which no library figure is at hand; the bf16 form is
// there to cross-check the probe against a library GEMM's measured rate.
#include "common.cuh"

namespace samb {
namespace {

constexpr int SLABS = 4;                       // K slabs of 128 bytes per row resident in shared memory
constexpr int A_BYTES = 128 * 128;             // one slab of A: 128 rows x 128 B (128B swizzle atoms of 8 rows)
constexpr int B_BYTES = 256 * 128;             // one slab of B: 256 rows x 128 B
constexpr int SMEM_BYTES = SLABS * (A_BYTES + B_BYTES) + 1024;
constexpr int MMAS_PER_ROUND = SLABS * 4;      // 4 MMAs of 32 B of K per slab

template <bool kInt8>
__global__ void __launch_bounds__(128, 1) mma_rate_kernel(int rounds, uint32_t seed, int32_t* status, int32_t* sink) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar[2];
  __shared__ uint32_t tmem_base;
  __shared__ int abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5;

  // operands: pseudo-random small integers / bf16 values in (-1, 1), so that the multipliers toggle as they do on data
  uint32_t s = seed ^ (blockIdx.x * 0x9E3779B9u) ^ (tid * 0x85EBCA6Bu);
  uint32_t* w = reinterpret_cast<uint32_t*>(smem);
  for (int i = tid; i < SLABS * (A_BYTES + B_BYTES) / 4; i += 128) {
    s = s * 1664525u + 1013904223u;
    uint32_t v = s ^ (s >> 15);
    if (!kInt8) v = (v & 0x807F807Fu) | 0x3F003F00u;     // two bf16 with exponent 126: magnitudes in [0.5, 1)
    w[i] = v;
  }
  if (tid == 0) {
    mbar_init(&bar[0], 1);
    mbar_init(&bar[1], 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base, 512);
    tmem_relinquish();
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  if (warp == 1 && elect_one()) {
    const uint32_t a0 = smem_u32(smem), b0 = a0 + SLABS * A_BYTES;
    const uint32_t idesc = kInt8 ? make_idesc(kAccS32, kFmtS8, kFmtS8, 128, 256) : make_idesc(kAccF32, kFmtBF16, kFmtBF16, 128, 256);
    uint32_t phase[2] = {0, 0};
    bool ok = true;
    for (int r = 0; r < rounds && ok; ++r) {
      const int buf = r & 1;
      if (r >= 2) {                                        // at most two rounds of MMAs in flight
        ok = mbar_wait(&bar[buf], phase[buf], &abort_flag, status, 0x51);
        phase[buf] ^= 1;
        tc_fence_after();
      }
      if (!ok) break;
#pragma unroll
      for (int sl = 0; sl < SLABS; ++sl) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint64_t ad = make_smem_desc(a0 + sl * A_BYTES + k * 32, 16, 1024, kSwizzle128B);
          const uint64_t bd = make_smem_desc(b0 + sl * B_BYTES + k * 32, 16, 1024, kSwizzle128B);
          if (kInt8) umma_i8_ss(tmem_base + buf * 256, ad, bd, idesc, (sl | k) ? 1u : 0u);
          else umma_f16_ss(tmem_base + buf * 256, ad, bd, idesc, (sl | k) ? 1u : 0u);
        }
      }
      tc_commit(&bar[buf]);
    }
    for (int i = 0; i < 2 && ok; ++i) {                    // drain what is still in flight
      const int r = rounds - 2 + i;
      if (r < 0) continue;
      ok = mbar_wait(&bar[r & 1], phase[r & 1], &abort_flag, status, 0x52);
      phase[r & 1] ^= 1;
    }
    tc_fence_after();
  }
  __syncthreads();
  tc_fence_after();
  if (warp == 0) {
    uint32_t v[16];
    tmem_ld_32x32b_x16(tmem_base, v);                      // keep the accumulators observable
    tmem_ld_wait();
    if (sink != nullptr && v[0] == 0x12345678u && v[5] == 0x9ABCDEF0u) sink[0] = int(v[1]);
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 512);
}

}  // namespace
}  // namespace samb

extern "C" int samb_selftest_mma_rate(int int8, int rounds, int ctas, int32_t* status, int32_t* sink, double* ops_out,
                                      void* stream) {
  using namespace samb;
  if (rounds <= 0 || ctas <= 0 || status == nullptr) return SAMB_E_BADARG;
  if (int rc = check_device_arch()) return rc;
  if (ctas > 4 * sm_count()) return SAMB_E_SHAPE;
  auto st = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (int8) {
    e = cudaFuncSetAttribute(mma_rate_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return SAMB_E_LAUNCH;
    mma_rate_kernel<true><<<ctas, 128, SMEM_BYTES, st>>>(rounds, 0x1234567u, status, sink);
  } else {
    e = cudaFuncSetAttribute(mma_rate_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return SAMB_E_LAUNCH;
    mma_rate_kernel<false><<<ctas, 128, SMEM_BYTES, st>>>(rounds, 0x1234567u, status, sink);
  }
  if (ops_out != nullptr)      // multiply-adds counted as 2 operations; K per MMA: 32 (int8) or 16 (bf16)
    *ops_out = double(ctas) * rounds * MMAS_PER_ROUND * 2.0 * 128.0 * 256.0 * (int8 ? 32.0 : 16.0);
  return launch_status();
}
