// Persistent warp-specialised GEMM on the 5th-generation tensor cores:
//   out[M,N] = epilogue( A[M,K] * W[N,K]^T )
// One CTA per SM walks 128x256 output tiles.  Warp 0 streams A/W k-slabs (128 bytes of K per row,
// 128B-swizzled) into a 4-deep shared-memory ring with TMA; warp 1 issues tcgen05.mma into one of two
// 256-column fp32/int32 accumulators in tensor memory; warps 2..9 drain the other accumulator
// (tcgen05.ld -> scale/bias/GELU/residual -> bf16 -> swizzled staging tile -> TMA store) while the
// next tile is being multiplied.
// The bf16 (kind::f16) and int8 (kind::i8) variants share every byte offset: 128 bytes of K are
// 64 bf16 (4 MMAs of K=16) or 128 int8 (4 MMAs of K=32).
#include <cstdlib>

#include "common.cuh"
#include "rowquant.cuh"

namespace samb {

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int SLAB_BYTES = 128;                 // K bytes per row per stage (one swizzle atom)
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * SLAB_BYTES;  // 16 KiB
constexpr int B_STAGE_BYTES = BN * SLAB_BYTES;  // 32 KiB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int K2_A1_OFF = 32 * 1024;            // k2 mode: [128][16] bf16 tail of A inside the stage
constexpr int K2_B1_OFF = 36 * 1024;            //          [tg_bn][16] bf16 tail of W
constexpr int EPI_COLSCALE = 16;                // internal epilogue flag: out = acc * w_scale[n] (bf16 operands)
constexpr int NUM_ACC = 2;
constexpr int TMEM_COLS = NUM_ACC * BN;         // 512: all of tensor memory, one CTA per SM
constexpr int NUM_THREADS = 320;                // TMA warp, MMA warp, 8 epilogue warps
constexpr int EPI_THREADS = 256;
constexpr int OUT_STAGE_BYTES = BM * 128;        // 64 bf16 columns of the tile, 128B-swizzled rows
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + OUT_STAGE_BYTES + 2 * BN * 4 + 1024 /*alignment slack*/ + 256 /*barriers*/;

struct GemmParams {
  void* out;
  const float* bias;
  const __nv_bfloat16* residual;
  const float* a_scale;
  const float* w_scale;
  float* row_absmax;             // optional: atomic maximum of |bf16(out[m, :])| per row (see launch_gemm_i8_rowmax)
  int* status;
  long long M;
  long long ldo, ldr, res_rows;
  int N, K;
  int k_slabs;
  int last_ksteps;               // MMAs (of 32 K-bytes) that the last slab really holds, 1..4
  int tiles_n;
  int bn;                        // output-tile width actually used: 64, 128 or 256 (narrow N)
  long long num_tiles;
  long long tiles_per_batch;     // tiles of one column batch (== num_tiles when not batched)
  int a_col_stride;              // batch b reads A columns [b*a_col_stride, +K)
  int o_col_stride;              // and writes out columns [b*o_col_stride, +N)
  int a_row_stride;              // batch b reads A rows [b*a_row_stride + m, ...) (head-major operand planes)
  int tg, tg_bn;                 // tg > 1: a tile is tg independent products of tg_bn columns each (consecutive
                                 // batches sharing W), so narrow batched outputs still fill a 256-column tile
  int b_resident;                // one column tile and few K slabs: W is fetched with the CTA's first tile only and
                                 // slab ks stays in stage ks (later fills of those stages bring only A)
  int k2;                        // grouped tiles with K = 80 bf16: a stage holds a whole product (64 + 16 columns of K)
  int nstages;                   // pipeline stages in use: STAGES, or STAGES - 1 when the last stage's shared memory
                                 // serves as three more output staging tiles (out_ring)
  int out_ring;                  // 1: every 64-column chunk of a tile has its own staging tile (short-K products, whose
                                 // epilogue would otherwise wait for each chunk's store to be read before the next)
  int hm_group;                  // > 0: head-major output, hm_group 16-column pieces per head (see launch_gemm)
  int epilogue;
};

// Named barrier over the 256 epilogue threads that also AND-reduces a predicate, so that all of
// them take the same decision to continue or to drain.
__device__ __forceinline__ bool epi_all(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\t"
      "bar.red.and.pred p, 1, 256, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"(uint32_t(pred))
      : "memory");
  return r != 0;
}
__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// kEpi: compile-time SAMB_EPI_* flags.  SAMB_EPI_RAW stores the accumulator words directly; every
// other combination goes registers -> 128B-swizzled staging tile -> TMA store, 64 columns at a time.
template <bool kInt8, int kEpi>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmOut, const __grid_constant__ CUtensorMap tmA2,
               const __grid_constant__ CUtensorMap tmB2, const GemmParams p) {
  constexpr bool kRaw = (kEpi & SAMB_EPI_RAW) != 0;
  constexpr bool kBias = (kEpi & SAMB_EPI_BIAS) != 0;
  constexpr bool kGelu = (kEpi & SAMB_EPI_GELU) != 0;
  constexpr bool kRes = (kEpi & SAMB_EPI_RESIDUAL) != 0;
  constexpr bool kColScale = kInt8 || (kEpi & EPI_COLSCALE) != 0;   // multiply by w_scale[n]
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_out = smem + STAGES * STAGE_BYTES;                      // [128][64] bf16, 128B swizzle
  float* s_bias = reinterpret_cast<float*>(stage_out + OUT_STAGE_BYTES);  // [256]
  float* s_wscale = s_bias + BN;                                          // [256]
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(s_wscale + BN);
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
      mbar_init(&acc_empty[a], EPI_THREADS / 32);   // one arrival per epilogue warp
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (p.k2) {
      tma_prefetch_desc(&tmA2);
      tma_prefetch_desc(&tmB2);
    }
    if (!kRaw) tma_prefetch_desc(&tmOut);
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
      bool ok = true, b_loaded = false;
      for (long long tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
        const int bt = int(tile / p.tiles_per_batch);
        const long long tb = tile - bt * p.tiles_per_batch;
        const int m0 = int(tb / p.tiles_n) * BM;
        const int n0 = int(tb % p.tiles_n) * p.bn;
        const int a_col0 = bt * p.a_col_stride;
        if (p.k2) {
          // whole product per stage: K columns 0..63 as 128-byte rows (128B swizzle), 64..79 as 32-byte rows
          // (32B swizzle), so four independent products are in flight per CTA
          for (int g = 0; ok && g < p.tg; ++g) {
            if (!(ok = mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, 1))) break;
            uint8_t* sa = smem + stage * STAGE_BYTES;
            const int arow = m0 + (bt * p.tg + g) * p.a_row_stride;
            // every product multiplies by the same tables: they are fetched once, with the CTA's first product,
            // into stage 0, and stay there (later fills of stage 0 bring only the A parts)
            const bool with_b = !b_loaded;
            mbar_expect_tx(&full_bar[stage], A_STAGE_BYTES + BM * 32 + (with_b ? p.tg_bn * SLAB_BYTES + p.tg_bn * 32 : 0));
            tma_load_2d(sa, &tmA, &full_bar[stage], 0, arow);
            tma_load_2d(sa + K2_A1_OFF, &tmA2, &full_bar[stage], 64, arow);
            if (with_b) {
              tma_load_2d(sa + A_STAGE_BYTES, &tmB, &full_bar[stage], 0, 0);
              tma_load_2d(sa + K2_B1_OFF, &tmB2, &full_bar[stage], 64, 0);
              b_loaded = true;
            }
            if (++stage == uint32_t(p.nstages)) { stage = 0; phase ^= 1u; }
          }
          continue;
        }
        for (int gk = 0; gk < p.tg * p.k_slabs; ++gk) {
          const int g = gk / p.k_slabs, ks = gk - g * p.k_slabs;       // product inside the tile, K slab
          if (!(ok = mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, 1))) break;
          uint8_t* sa = smem + stage * STAGE_BYTES;
          const bool with_b = !(p.b_resident && b_loaded);
          mbar_expect_tx(&full_bar[stage], A_STAGE_BYTES + (with_b ? p.tg_bn * SLAB_BYTES : 0));
          tma_load_2d(sa, &tmA, &full_bar[stage], a_col0 + ks * slab_elems, m0 + (bt * p.tg + g) * p.a_row_stride);
          if (with_b) tma_load_2d(sa + A_STAGE_BYTES, &tmB, &full_bar[stage], ks * slab_elems, p.tg > 1 ? 0 : n0);
          if (++stage == uint32_t(p.nstages)) { stage = 0; phase ^= 1u; }
        }
        b_loaded = true;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp walks the loop (warp-uniform waits and descriptors); one elected lane issues.
    {
      const uint32_t idesc = kInt8 ? make_idesc(kAccS32, kFmtS8, kFmtS8, BM, p.tg_bn)
                                   : make_idesc(kAccF32, kFmtBF16, kFmtBF16, BM, p.tg_bn);
      // K-major, 128B swizzle: 8-row groups 1024 B apart; the start address moves in 16-byte units.
      const uint64_t desc0 = make_smem_desc(smem_u32(smem), 16, 1024, kSwizzle128B);
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (long long tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
        if (!(ok = mbar_wait(&acc_empty[acc], acc_phase ^ 1u, abort_flag, p.status, 2))) break;
        tc_fence_after();
        if (p.k2) {
          const uint64_t desc1 = make_smem_desc(smem_u32(smem), 16, 256, kSwizzle32B);
          for (int g = 0; g < p.tg; ++g) {
            const uint32_t d_tmem = tmem_base + acc * BN + g * p.tg_bn;
            if (!(ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.status, 3))) break;
            tc_fence_after();
            if (elect_one()) {
              const uint64_t adesc = desc0 + stage * (STAGE_BYTES / 16);
              const uint64_t bdesc = desc0 + A_STAGE_BYTES / 16;      // the tables live in stage 0
#pragma unroll
              for (int k4 = 0; k4 < 4; ++k4) umma_f16_ss(d_tmem, adesc + k4 * 2, bdesc + k4 * 2, idesc, k4 != 0 ? 1u : 0u);
              umma_f16_ss(d_tmem, desc1 + (stage * STAGE_BYTES + K2_A1_OFF) / 16, desc1 + K2_B1_OFF / 16, idesc, 1u);
              tc_commit(&empty_bar[stage]);
            }
            __syncwarp();
            if (++stage == uint32_t(p.nstages)) { stage = 0; phase ^= 1u; }
          }
        } else
        for (int gk = 0; gk < p.tg * p.k_slabs; ++gk) {
          const int g = gk / p.k_slabs, ks = gk - g * p.k_slabs;
          const uint32_t d_tmem = tmem_base + acc * BN + g * p.tg_bn;
          if (!(ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.status, 3))) break;
          tc_fence_after();
          if (elect_one()) {
            const uint64_t adesc = desc0 + stage * (STAGE_BYTES / 16);
            const uint64_t bdesc = desc0 + (p.b_resident ? ks : int(stage)) * (STAGE_BYTES / 16) + A_STAGE_BYTES / 16;
            const int nsteps = ks == p.k_slabs - 1 ? p.last_ksteps : 4;
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {         // 32 bytes of K per MMA
              if (k4 >= nsteps) break;
              const uint32_t accumulate = (ks | k4) != 0 ? 1u : 0u;
              if (kInt8) umma_i8_ss(d_tmem, adesc + k4 * 2, bdesc + k4 * 2, idesc, accumulate);
              else umma_f16_ss(d_tmem, adesc + k4 * 2, bdesc + k4 * 2, idesc, accumulate);
            }
            tc_commit(&empty_bar[stage]);             // stage reusable once these MMAs have read it
          }
          __syncwarp();
          if (++stage == uint32_t(p.nstages)) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if (elect_one()) tc_commit(&acc_full[acc]);   // accumulator complete
        __syncwarp();
        if (++acc == NUM_ACC) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    // Two warps share each TMEM lane quarter (a warp may only touch lanes 32*(warp%4)..+31) and split
    // every 64-column chunk between them: `half` selects the 32-column side.
    const uint32_t lane_base = uint32_t(warp & 3) * 32u;
    const int half = (warp - 2) >> 2;
    const int erow = int(lane_base) + lane;                // row inside the tile
    const int et = int(threadIdx.x) - 64;                  // 0..255
    uint32_t acc = 0, acc_phase = 0;
    for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
      const int bt = int(tile / p.tiles_per_batch);
      const long long tb = tile - bt * p.tiles_per_batch;
      const int m0 = int(tb / p.tiles_n) * BM;
      const int n0 = int(tb % p.tiles_n) * p.bn;
      const long long row = (long long)m0 + erow;
      const bool row_ok = row < p.M;
      if (!kRaw) {
        // per-column vectors of this tile; the barrier inside epi_all() publishes them
        const int n = n0 + et;
        if (kBias) s_bias[et] = n < p.N ? __ldg(p.bias + n) : 0.f;
        if (kColScale) {
          const int ns = p.tg > 1 ? et % p.tg_bn : n;       // grouped tiles: every product uses the same W rows
          s_wscale[et] = ns < p.N ? __ldg(p.w_scale + ns) : 0.f;
        }
      }
      const bool got = mbar_wait(&acc_full[acc], acc_phase, abort_flag, p.status, 4);
      if (!epi_all(got)) break;
      tc_fence_after();
      const uint32_t t_addr = tmem_base + (lane_base << 16) + acc * BN + half * 32;
      if (kRaw) {
#pragma unroll 1
        for (int c = 0; c < p.bn / 64; ++c) {
          const int col0 = n0 + c * 64 + half * 32;
          if (col0 >= p.N) break;                       // uniform across the warp
          uint32_t r[32];
          __syncwarp();
          tmem_ld_32x32b_x32(t_addr + c * 64, r);
          tmem_ld_wait();
          if (!row_ok) continue;                        // lanes past M only take part in the load
          uint32_t* o = reinterpret_cast<uint32_t*>(p.out) + row * p.ldo + col0;
#pragma unroll
          for (int g = 0; g < 8; ++g)
            if (col0 + g * 4 < p.N)
              *reinterpret_cast<uint4*>(o + g * 4) = make_uint4(r[g * 4], r[g * 4 + 1], r[g * 4 + 2], r[g * 4 + 3]);
        }
      } else {
        float a_scale = 1.0f;
        if (kInt8 && row_ok) a_scale = __ldg(p.a_scale + row);
        __nv_bfloat162 m2 = __floats2bfloat162_rn(0.f, 0.f);   // running |max| of this row's outputs in this tile
        const __nv_bfloat16* res_row = nullptr;
        if (kRes && row_ok) res_row = p.residual + (row % p.res_rows) * p.ldr + n0 + half * 32;
#pragma unroll 1
        for (int c = 0; c < p.bn / 64; ++c) {
          const int col0 = n0 + c * 64;                 // first column of the chunk
          if (col0 >= p.N) break;                       // uniform across the CTA
          const int colh = col0 + half * 32;            // first column of this warp's side
          uint4 rv[4];
          if (kRes) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              rv[u] = make_uint4(0u, 0u, 0u, 0u);
              if (row_ok && colh + u * 8 < p.N) rv[u] = __ldg(reinterpret_cast<const uint4*>(res_row + c * 64) + u);
            }
          }
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_addr + c * 64, r);
          tmem_ld_wait();
          uint4 packed[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            float v[8];
            const int ct0 = c * 64 + half * 32 + u * 8;   // first of these eight columns inside the tile
            epilogue8<kInt8, kInt8 || kColScale, kBias, kGelu>(r + u * 8, a_scale, s_wscale + ct0, s_bias + ct0, v);
            if (kRes) {
              const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&rv[u]);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(rp[j]);
                v[2 * j] += f.x;
                v[2 * j + 1] += f.y;
              }
            }
            packed[u] = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]),
                                   pack_bf16x2(v[6], v[7]));
            if (p.row_absmax != nullptr) m2 = absmax8(m2, packed[u]);
          }
          // staging tile of this chunk: the one after the ring, or (out_ring) one of four, the last three carved
          // out of the unused last pipeline stage; then only the tile's first chunk waits for earlier stores
          uint8_t* so = stage_out;
          if (p.out_ring && c > 0) so = smem + (STAGES - 1) * STAGE_BYTES + (c - 1) * OUT_STAGE_BYTES;
          if (!p.out_ring || c == 0) {
            if (et == 0) tma_store_wait_read<0>();      // the staging tile(s) are free again
            epi_sync();
          }
          if (p.hm_group == 0) {
            uint8_t* srow = so + erow * 128;
#pragma unroll
            for (int u = 0; u < 4; ++u)
              *reinterpret_cast<uint4*>(srow + (((half * 4 + u) ^ (erow & 7)) << 4)) = packed[u];
          } else {
            // head-major: four [128][16-column] pieces (32-byte rows, 32B swizzle), one TMA store each
            uint8_t* srow = stage_out + erow * 32;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int unit = half * 4 + u;             // 16-byte unit inside the 64-column chunk
              *reinterpret_cast<uint4*>(srow + (unit >> 1) * 4096 + (((unit & 1) ^ ((erow >> 2) & 1)) << 4)) = packed[u];
            }
          }
          fence_proxy_async_smem();
          epi_sync();
          if (et == 0) {
            if (p.hm_group == 0) {
              tma_store_2d(&tmOut, so, bt * p.tg * p.o_col_stride + col0, m0);  // clipped at M and at the row end
            } else {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const int col = col0 + q * 16;
                if (col < p.N) {
                  const int g = col >> 4;                // 16-column piece index: plane g / group, piece g % group
                  tma_store_4d(&tmOut, stage_out + q * 4096, 0, g % p.hm_group, m0, g / p.hm_group);
                }
              }
            }
            tma_store_commit();
          }
        }
        // non-negative floats order like their bit patterns: one integer atomic per row and tile
        if (p.row_absmax != nullptr && row_ok)
          atomicMax(reinterpret_cast<int*>(p.row_absmax + row), __float_as_int(absmax_fold(m2)));
      }
      tc_fence_before();
      mbar_arrive_warp(&acc_empty[acc]);
      if (++acc == NUM_ACC) { acc = 0; acc_phase ^= 1u; }
    }
    if (!kRaw && et == 0) tma_store_wait_all<0>();
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <bool kInt8>
using KernelFn = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap,
                          const GemmParams);

template <bool kInt8>
KernelFn<kInt8> pick_kernel(int epi) {
  switch (epi) {
    case 0: return gemm_tc_kernel<kInt8, 0>;
    case 1: return gemm_tc_kernel<kInt8, 1>;
    case 2: return gemm_tc_kernel<kInt8, 2>;
    case 3: return gemm_tc_kernel<kInt8, 3>;
    case 4: return gemm_tc_kernel<kInt8, 4>;
    case 5: return gemm_tc_kernel<kInt8, 5>;
    case 6: return gemm_tc_kernel<kInt8, 6>;
    case 7: return gemm_tc_kernel<kInt8, 7>;
    case EPI_COLSCALE: return gemm_tc_kernel<kInt8, EPI_COLSCALE>;
    default: return gemm_tc_kernel<kInt8, SAMB_EPI_RAW>;
  }
}

inline int kmul_of(bool int8) { return int8 ? 16 : 8; }

int launch_gemm(bool int8, const void* A, int64_t lda, const void* W, int64_t ldw, const float* a_scale,
                const float* w_scale, const float* bias, const void* residual, int64_t ldr, int64_t res_rows,
                void* out, int64_t ldo, int64_t M, int N, int K, int epilogue, int32_t* status, void* stream,
                int batch = 1, int a_col_stride = 0, int o_col_stride = 0, int64_t a_row_stride = 0, int head_dim = 0,
                float* row_absmax = nullptr) {
  if (A == nullptr || W == nullptr || out == nullptr || status == nullptr) return SAMB_E_BADARG;
  if (M < 0 || N <= 0 || K <= 0 || batch <= 0) return SAMB_E_BADARG;
  if (epilogue == EPI_COLSCALE) {
    if (int8 || w_scale == nullptr) return SAMB_E_BADARG;
  } else if (epilogue & ~(SAMB_EPI_BIAS | SAMB_EPI_GELU | SAMB_EPI_RESIDUAL | SAMB_EPI_RAW)) {
    return SAMB_E_BADARG;
  }
  if (batch > 1 && (N % 64 || a_col_stride % kmul_of(int8) || o_col_stride % 8 || (epilogue & SAMB_EPI_RAW)))
    return SAMB_E_SHAPE;
  const bool raw = (epilogue & SAMB_EPI_RAW) != 0;
  if (raw && epilogue != SAMB_EPI_RAW) return SAMB_E_BADARG;
  if ((epilogue & SAMB_EPI_BIAS) && bias == nullptr) return SAMB_E_BADARG;
  if ((epilogue & SAMB_EPI_RESIDUAL) && residual == nullptr) return SAMB_E_BADARG;
  if (int8 && !raw && (a_scale == nullptr || w_scale == nullptr)) return SAMB_E_BADARG;
  const int esz = int8 ? 1 : 2;
  const int kmul = 16 / esz;                       // K and leading dims: 16-byte multiples
  const long long a_cols = (long long)(batch - 1) * a_col_stride + K;   // columns of A that are read
  const long long o_cols = (long long)(batch - 1) * o_col_stride + N;   // columns of out that are written
  if (K % kmul || lda % kmul || ldw % kmul || lda < a_cols || ldw < K) return SAMB_E_SHAPE;
  const int out_mul = raw ? 4 : 8;
  if (N % 8 || (!head_dim && (ldo % out_mul || ldo < o_cols))) return SAMB_E_SHAPE;
  if ((epilogue & SAMB_EPI_RESIDUAL) && (ldr % 8 || ldr < N || res_rows <= 0)) return SAMB_E_SHAPE;
  if (M > (int64_t(1) << 31) - BM || (a_row_stride * batch) > (int64_t(1) << 31) - BM) return SAMB_E_SHAPE;
  if (head_dim && (head_dim % 16 || N % head_dim || (epilogue & SAMB_EPI_RAW) || batch != 1)) return SAMB_E_SHAPE;
  if ((reinterpret_cast<uintptr_t>(out) & 15u) || (residual && (reinterpret_cast<uintptr_t>(residual) & 15u)))
    return SAMB_E_ALIGN;
  if (int e = check_device_arch()) return e;
  if (M == 0) return SAMB_OK;
  // Large plain products run on CTA pairs; SAMB_GEMM_SINGLE_CTA=1 keeps them on this file's kernel (A/B timing).
  // An int8 product with a short K and the GELU epilogue is bound by that epilogue; the pair's shared
  // accumulator hand-off only couples it more tightly, so it stays on this file's kernel.
  const bool epi_bound = int8 && K < 2048 && (epilogue & SAMB_EPI_GELU) && getenv("SAMB_GELU_SINGLE_CTA") != nullptr;
  if (!raw && batch == 1 && epilogue != EPI_COLSCALE && !epi_bound && getenv("SAMB_GEMM_SINGLE_CTA") == nullptr) {
    const int e = launch_gemm_pair(int8, A, lda, W, ldw, a_scale, w_scale, bias, residual, ldr, res_rows, out, ldo, M, N, K,
                                   epilogue, head_dim, status, stream, row_absmax);
    if (e != SAMB_E_SHAPE) return e;
  }

  const CUtensorMapDataType dt = int8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const uint32_t slab_elems = uint32_t(SLAB_BYTES / esz);
  CUtensorMap tmA, tmB;
  {
    // batched: columns past a batch's K belong to the next batch; W's zero fill beyond K cancels them
    const uint64_t dims[2] = {uint64_t(batch > 1 && a_col_stride ? lda : K), uint64_t(a_row_stride ? a_row_stride * batch : M)};
    const uint64_t strides[2] = {uint64_t(esz), uint64_t(lda) * esz};
    const uint32_t box[2] = {slab_elems, uint32_t(BM)};
    if (int e = make_tensor_map(&tmA, dt, 2, const_cast<void*>(A), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return e;
  }
  {
    const uint64_t dims[2] = {uint64_t(K), uint64_t(N)};
    const uint64_t strides[2] = {uint64_t(esz), uint64_t(ldw) * esz};
    const uint32_t box[2] = {slab_elems, uint32_t(N <= 64 ? 64 : (N <= 128 ? 128 : BN))};   // == tg_bn
    if (int e = make_tensor_map(&tmB, dt, 2, const_cast<void*>(W), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return e;
  }

  GemmParams p;
  p.out = out;
  p.bias = bias;
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.a_scale = a_scale;
  p.w_scale = w_scale;
  p.row_absmax = row_absmax;
  p.status = status;
  p.M = M;
  p.ldo = ldo;
  p.ldr = ldr;
  p.res_rows = res_rows > 0 ? res_rows : 1;
  p.N = N;
  p.K = K;
  p.k_slabs = (K * esz + SLAB_BYTES - 1) / SLAB_BYTES;
  p.last_ksteps = (K * esz - (p.k_slabs - 1) * SLAB_BYTES + 31) / 32;
  p.bn = N <= 64 ? 64 : (N <= 128 ? 128 : BN);
  p.tg = 1;
  p.tg_bn = p.bn;
  if (batch > 1 && a_row_stride && N == 64 && o_col_stride == N && epilogue == EPI_COLSCALE) {
    p.tg = batch % 4 == 0 ? 4 : (batch % 2 == 0 ? 2 : 1);        // tg narrow products share one tile
    p.bn = p.tg * N;
  }
  p.k2 = (p.tg > 1 && !int8 && K == 80) ? 1 : 0;
  p.b_resident = (p.tg == 1 && N <= p.bn && p.k_slabs <= STAGES - 1 && batch > 1 && a_row_stride != 0) ? 1 : 0;
  // one staging tile per chunk where the epilogue binds: grouped short-K products, and the int8 GELU epilogue
  p.out_ring = (((p.tg > 1 || (p.b_resident && p.bn == BN && !raw)) && head_dim == 0) ||
                (epi_bound && head_dim == 0 && !raw && p.bn == BN)) ? 1 : 0;
  p.nstages = p.out_ring ? STAGES - 1 : STAGES;
  p.tiles_n = p.tg > 1 ? 1 : (N + p.bn - 1) / p.bn;
  if (p.tg > 1) p.N = p.tg * N;                                  // logical width of a grouped tile
  p.tiles_per_batch = ((M + BM - 1) / BM) * p.tiles_n;
  p.num_tiles = p.tiles_per_batch * (batch / p.tg);
  p.a_col_stride = a_col_stride;
  p.o_col_stride = o_col_stride;
  p.a_row_stride = int(a_row_stride);
  p.hm_group = head_dim / 16;
  p.epilogue = epilogue;

  CUtensorMap tmOut = tmA;   // unused by the raw-accumulator variant
  if (!raw && head_dim) {
    // out is [N / head_dim planes][M rows][head_dim]: a 64-column chunk leaves as 16-column pieces
    const uint64_t dims[4] = {16, uint64_t(head_dim / 16), uint64_t(M), uint64_t(N / head_dim)};
    const uint64_t strides[4] = {2, 32, uint64_t(head_dim) * 2, uint64_t(M) * head_dim * 2};
    const uint32_t box[4] = {16, 1, uint32_t(BM), 1};
    if (int e = make_tensor_map(&tmOut, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, out, dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_32B))
      return e;
  } else if (!raw) {
    const uint64_t dims[2] = {uint64_t(o_cols), uint64_t(M)};
    const uint64_t strides[2] = {2, uint64_t(ldo) * 2};
    const uint32_t box[2] = {64, uint32_t(BM)};
    if (int e = make_tensor_map(&tmOut, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, out, dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_128B))
      return e;
  }
  CUtensorMap tmA2 = tmA, tmB2 = tmB;
  if (p.k2) {
    const uint64_t dimsA[2] = {uint64_t(K), uint64_t(a_row_stride * batch)};
    const uint64_t stridesA[2] = {2, uint64_t(lda) * 2};
    const uint32_t boxA[2] = {16, uint32_t(BM)};
    if (int e = make_tensor_map(&tmA2, dt, 2, const_cast<void*>(A), dimsA, stridesA, boxA, CU_TENSOR_MAP_SWIZZLE_32B))
      return e;
    const uint64_t dimsB[2] = {uint64_t(K), uint64_t(N)};
    const uint64_t stridesB[2] = {2, uint64_t(ldw) * 2};
    const uint32_t boxB[2] = {16, 64};
    if (int e = make_tensor_map(&tmB2, dt, 2, const_cast<void*>(W), dimsB, stridesB, boxB, CU_TENSOR_MAP_SWIZZLE_32B))
      return e;
  }
  auto kern = int8 ? pick_kernel<true>(epilogue) : pick_kernel<false>(epilogue);
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
    return SAMB_E_LAUNCH;
  const long long grid = p.num_tiles < sm_count() ? p.num_tiles : sm_count();
  kern<<<dim3(unsigned(grid)), dim3(NUM_THREADS), SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(tmA, tmB, tmOut, tmA2, tmB2, p);
  return launch_status();
}

}  // namespace

int launch_gemm_i8_rowmax(const int8_t* Aq, int64_t lda, const float* a_scale, const int8_t* Wq, int64_t ldw,
                          const float* w_scale, const float* bias, const void* residual, int64_t ldr, int64_t res_rows,
                          void* out, int64_t ldo, int64_t M, int N, int K, int epilogue, int32_t* status, void* stream,
                          float* row_absmax) {
  if (epilogue & SAMB_EPI_RAW) return SAMB_E_BADARG;
  return launch_gemm(true, Aq, lda, Wq, ldw, a_scale, w_scale, bias, residual, ldr, res_rows, out, ldo, M, N, K, epilogue,
                     status, stream, 1, 0, 0, 0, 0, row_absmax);
}
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

int samb_relpos_table_products(const void* q_planes, const void* tables, const float* col_scale, void* tab,
                               int64_t ldt, int64_t rows, int H, int d, int t_head_stride, int32_t* status,
                               void* stream) {
  if (H <= 0 || d <= 0 || t_head_stride <= 0) return SAMB_E_BADARG;
  return samb::launch_gemm(false, q_planes, d, tables, d, nullptr, col_scale, nullptr, nullptr, 0, 0, tab, ldt, rows,
                           t_head_stride, d, samb::EPI_COLSCALE, status, stream, H, 0, t_head_stride, rows);
}

int samb_gemm_bf16_heads(const void* A, int64_t lda, const void* W, int64_t ldw, const float* bias, void* out,
                         int64_t M, int N, int K, int head_dim, int32_t* status, void* stream) {
  if (head_dim <= 0) return SAMB_E_BADARG;
  return samb::launch_gemm(false, A, lda, W, ldw, nullptr, nullptr, bias, nullptr, 0, 0, out, 0, M, N, K,
                           bias ? SAMB_EPI_BIAS : 0, status, stream, 1, 0, 0, 0, head_dim);
}

int samb_gemm_i8_heads(const int8_t* Aq, int64_t lda, const float* a_scale, const int8_t* Wq, int64_t ldw,
                       const float* w_scale, const float* bias, void* out, int64_t M, int N, int K, int head_dim,
                       int32_t* status, void* stream) {
  if (head_dim <= 0) return SAMB_E_BADARG;
  return samb::launch_gemm(true, Aq, lda, Wq, ldw, a_scale, w_scale, bias, nullptr, 0, 0, out, 0, M, N, K,
                           bias ? SAMB_EPI_BIAS : 0, status, stream, 1, 0, 0, 0, head_dim);
}

}  // extern "C"
