// Persistent warp-specialised GEMM on the 5th-generation tensor cores:
//   out[M,N] = epilogue( A[M,K] * W[N,K]^T )
// One CTA per SM walks 128x256 output tiles.  Warp 0 streams A/W k-slabs (128 bytes of K per row,
// 128B-swizzled) into a 4-deep shared-memory ring with TMA; warp 1 issues tcgen05.mma into one of two
// 256-column fp32/int32 accumulators in tensor memory; warps 2..5 drain the other accumulator
// (tcgen05.ld -> scale/bias/GELU/residual -> bf16 -> global) while the next tile is being multiplied.
// The bf16 (kind::f16) and int8 (kind::i8) variants share every byte offset: 128 bytes of K are
// 64 bf16 (4 MMAs of K=16) or 128 int8 (4 MMAs of K=32).
#include "common.cuh"

namespace samb {

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int SLAB_BYTES = 128;                 // K bytes per row per stage (one swizzle atom)
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * SLAB_BYTES;  // 16 KiB
constexpr int B_STAGE_BYTES = BN * SLAB_BYTES;  // 32 KiB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int NUM_ACC = 2;
constexpr int TMEM_COLS = NUM_ACC * BN;         // 512: all of tensor memory, one CTA per SM
constexpr int NUM_THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;

struct GemmParams {
  void* out;
  const float* bias;
  const __nv_bfloat16* residual;
  const float* a_scale;
  const float* w_scale;
  int* status;
  long long M;
  long long ldo, ldr, res_rows;
  int N, K;
  int k_slabs;
  int tiles_n;
  long long num_tiles;
  int epilogue;
};

__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f)); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <bool kInt8>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;
  uint64_t* acc_empty = acc_full + NUM_ACC;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + NUM_ACC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < NUM_ACC; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 128);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int slab_elems = kInt8 ? SLAB_BYTES : SLAB_BYTES / 2;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (long long tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
        const int m0 = int(tile / p.tiles_n) * BM;
        const int n0 = int(tile % p.tiles_n) * BN;
        for (int ks = 0; ks < p.k_slabs; ++ks) {
          if (!(ok = mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, 1))) break;
          uint8_t* sa = smem + stage * STAGE_BYTES;
          mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
          tma_load_2d(sa, &tmA, &full_bar[stage], ks * slab_elems, m0);
          tma_load_2d(sa + A_STAGE_BYTES, &tmB, &full_bar[stage], ks * slab_elems, n0);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = kInt8 ? make_idesc(kAccS32, kFmtS8, kFmtS8, BM, BN)
                                       : make_idesc(kAccF32, kFmtBF16, kFmtBF16, BM, BN);
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (long long tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
        if (!(ok = mbar_wait(&acc_empty[acc], acc_phase ^ 1u, abort_flag, p.status, 2))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int ks = 0; ks < p.k_slabs; ++ks) {
          if (!(ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.status, 3))) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_STAGE_BYTES;
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            // K-major, 128B swizzle: 8-row groups 1024 B apart; 32 bytes of K per MMA.
            const uint64_t adesc = make_smem_desc(a_addr + k4 * 32, 16, 1024, kSwizzle128B);
            const uint64_t bdesc = make_smem_desc(b_addr + k4 * 32, 16, 1024, kSwizzle128B);
            const uint32_t accumulate = (ks | k4) != 0 ? 1u : 0u;
            if (kInt8) umma_i8_ss(d_tmem, adesc, bdesc, idesc, accumulate);
            else umma_f16_ss(d_tmem, adesc, bdesc, idesc, accumulate);
          }
          tc_commit(&empty_bar[stage]);   // stage reusable once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit(&acc_full[acc]);        // accumulator complete
        if (++acc == NUM_ACC) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const uint32_t lane_base = uint32_t(warp & 3) * 32u;   // the TMEM lane quarter this warp may read
    uint32_t acc = 0, acc_phase = 0;
    bool ok = true;
    const bool raw = (p.epilogue & SAMB_EPI_RAW) != 0;
    const bool has_bias = (p.epilogue & SAMB_EPI_BIAS) != 0;
    const bool has_gelu = (p.epilogue & SAMB_EPI_GELU) != 0;
    const bool has_res = (p.epilogue & SAMB_EPI_RESIDUAL) != 0;
    for (long long tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
      const int m0 = int(tile / p.tiles_n) * BM;
      const int n0 = int(tile % p.tiles_n) * BN;
      if (!(ok = mbar_wait(&acc_full[acc], acc_phase, abort_flag, p.status, 4))) break;
      tc_fence_after();
      const long long row = (long long)m0 + lane_base + lane;
      const bool row_ok = row < p.M;
      const long long res_row = (has_res && row_ok) ? row % p.res_rows : 0;
      float a_scale = 1.0f;
      if (kInt8 && !raw && row_ok) a_scale = p.a_scale[row];
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) break;                       // uniform across the CTA
        uint32_t r[32];
        __syncwarp();
        tmem_ld_32x32b_x32(tmem_base + (lane_base << 16) + acc * BN + c * 32, r);
        tmem_ld_wait();
        if (!row_ok) continue;                        // lanes past M only take part in the load
        if (raw) {
          uint32_t* o = reinterpret_cast<uint32_t*>(p.out) + row * p.ldo + col0;
#pragma unroll
          for (int g = 0; g < 8; ++g)
            if (col0 + g * 4 < p.N)
              *reinterpret_cast<uint4*>(o + g * 4) = make_uint4(r[g * 4], r[g * 4 + 1], r[g * 4 + 2], r[g * 4 + 3]);
          continue;
        }
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + row * p.ldo + col0;
        const __nv_bfloat16* res = has_res ? p.residual + res_row * p.ldr + col0 : nullptr;
#pragma unroll
        for (int g = 0; g < 4; ++g) {                // groups of 8 columns = one 16-byte store
          if (col0 + g * 8 >= p.N) break;
          float v[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int n = col0 + g * 8 + j;
            float x;
            if (kInt8) {
              x = __fmul_rn(__fmul_rn(float(int(r[g * 8 + j])), a_scale), __ldg(p.w_scale + n));
            } else {
              x = __uint_as_float(r[g * 8 + j]);
            }
            if (has_bias) x = __fadd_rn(x, __ldg(p.bias + n));
            if (has_gelu) x = gelu_erf(x);
            v[j] = x;
          }
          if (has_res) {
            const uint4 rv = *reinterpret_cast<const uint4*>(res + g * 8);
            const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 f = __bfloat1622float2(rp[j]);
              v[2 * j] += f.x;
              v[2 * j + 1] += f.y;
            }
          }
          *reinterpret_cast<uint4*>(o + g * 8) = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]),
                                                            pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
        }
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[acc]);
      if (++acc == NUM_ACC) { acc = 0; acc_phase ^= 1u; }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

int launch_gemm(bool int8, const void* A, int64_t lda, const void* W, int64_t ldw, const float* a_scale,
                const float* w_scale, const float* bias, const void* residual, int64_t ldr, int64_t res_rows,
                void* out, int64_t ldo, int64_t M, int N, int K, int epilogue, int32_t* status, void* stream) {
  if (A == nullptr || W == nullptr || out == nullptr || status == nullptr) return SAMB_E_BADARG;
  if (M < 0 || N <= 0 || K <= 0) return SAMB_E_BADARG;
  if (epilogue & ~(SAMB_EPI_BIAS | SAMB_EPI_GELU | SAMB_EPI_RESIDUAL | SAMB_EPI_RAW)) return SAMB_E_BADARG;
  const bool raw = (epilogue & SAMB_EPI_RAW) != 0;
  if (raw && epilogue != SAMB_EPI_RAW) return SAMB_E_BADARG;
  if ((epilogue & SAMB_EPI_BIAS) && bias == nullptr) return SAMB_E_BADARG;
  if ((epilogue & SAMB_EPI_RESIDUAL) && residual == nullptr) return SAMB_E_BADARG;
  if (int8 && !raw && (a_scale == nullptr || w_scale == nullptr)) return SAMB_E_BADARG;
  const int esz = int8 ? 1 : 2;
  const int kmul = 16 / esz;                       // K and leading dims: 16-byte multiples
  if (K % kmul || lda % kmul || ldw % kmul || lda < K || ldw < K) return SAMB_E_SHAPE;
  const int out_mul = raw ? 4 : 8;
  if (N % 8 || ldo % out_mul || ldo < N) return SAMB_E_SHAPE;
  if ((epilogue & SAMB_EPI_RESIDUAL) && (ldr % 8 || ldr < N || res_rows <= 0)) return SAMB_E_SHAPE;
  if (M > (int64_t(1) << 31) - BM) return SAMB_E_SHAPE;
  if ((reinterpret_cast<uintptr_t>(out) & 15u) || (residual && (reinterpret_cast<uintptr_t>(residual) & 15u)))
    return SAMB_E_ALIGN;
  if (int e = check_device_arch()) return e;
  if (M == 0) return SAMB_OK;

  const CUtensorMapDataType dt = int8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const uint32_t slab_elems = uint32_t(SLAB_BYTES / esz);
  CUtensorMap tmA, tmB;
  {
    const uint64_t dims[2] = {uint64_t(K), uint64_t(M)};
    const uint64_t strides[2] = {uint64_t(esz), uint64_t(lda) * esz};
    const uint32_t box[2] = {slab_elems, uint32_t(BM)};
    if (int e = make_tensor_map(&tmA, dt, 2, const_cast<void*>(A), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return e;
  }
  {
    const uint64_t dims[2] = {uint64_t(K), uint64_t(N)};
    const uint64_t strides[2] = {uint64_t(esz), uint64_t(ldw) * esz};
    const uint32_t box[2] = {slab_elems, uint32_t(BN)};
    if (int e = make_tensor_map(&tmB, dt, 2, const_cast<void*>(W), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return e;
  }

  GemmParams p;
  p.out = out;
  p.bias = bias;
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.a_scale = a_scale;
  p.w_scale = w_scale;
  p.status = status;
  p.M = M;
  p.ldo = ldo;
  p.ldr = ldr;
  p.res_rows = res_rows > 0 ? res_rows : 1;
  p.N = N;
  p.K = K;
  p.k_slabs = (K * esz + SLAB_BYTES - 1) / SLAB_BYTES;
  p.tiles_n = (N + BN - 1) / BN;
  p.num_tiles = ((M + BM - 1) / BM) * p.tiles_n;
  p.epilogue = epilogue;

  auto kern = int8 ? gemm_tc_kernel<true> : gemm_tc_kernel<false>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
    return SAMB_E_LAUNCH;
  const long long grid = p.num_tiles < sm_count() ? p.num_tiles : sm_count();
  kern<<<dim3(unsigned(grid)), dim3(NUM_THREADS), SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(tmA, tmB, p);
  return launch_status();
}

}  // namespace
}  // namespace samb

extern "C" {

int samb_gemm_bf16(const void* A, int64_t lda, const void* W, int64_t ldw, const float* bias, const void* residual,
                   int64_t ldr, int64_t res_rows, void* out, int64_t ldo, int64_t M, int N, int K, int epilogue,
                   int32_t* status, void* stream) {
  return samb::launch_gemm(false, A, lda, W, ldw, nullptr, nullptr, bias, residual, ldr, res_rows, out, ldo, M, N, K,
                           epilogue, status, stream);
}

int samb_gemm_i8(const int8_t* Aq, int64_t lda, const float* a_scale, const int8_t* Wq, int64_t ldw,
                 const float* w_scale, const float* bias, const void* residual, int64_t ldr, int64_t res_rows,
                 void* out, int64_t ldo, int64_t M, int N, int K, int epilogue, int32_t* status, void* stream) {
  return samb::launch_gemm(true, Aq, lda, Wq, ldw, a_scale, w_scale, bias, residual, ldr, res_rows, out, ldo, M, N, K,
                           epilogue, status, stream);
}

}  // extern "C"
