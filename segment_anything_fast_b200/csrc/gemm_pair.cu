// The Linear-layer GEMM on CTA pairs (thread-block clusters of two, tcgen05 cta_group::2):
//   out[M,N] = epilogue( A[M,K] * W[N,K]^T ),  N a multiple of 256.
// A pair owns a 256 x 256 output tile.  Each CTA streams its own 128 rows of A and its own half (128 rows)
// of the W tile; one MMA issued by the pair's leader (M = 256, N = 256) reads A and half of W from each
// CTA's shared memory and accumulates into both CTAs' tensor memory (128 rows each).  Against the
// single-CTA kernel this halves the W bytes every CTA loads and reads per MMA (8 instead of 12 KB of
// operands per 128 tensor-pipe cycles), which is what the single-CTA kernel is bound by, and leaves room
// for a 6-deep ring.  Roles per CTA: warp 0 TMA producer, warp 1 MMA issue (leader CTA only), warps 2..17
// epilogue of the CTA's own 128 rows (four warps per tensor-memory lane quarter, 16 of every 64 columns each:
// the int8 epilogues are issue-bound with fewer), and one more warp whose only job is the output: it waits
// for a staged 64-column chunk, issues its TMA store, waits until the store has read the staging tile and
// hands the tile back (with a residual: has the TMA unit fill it with the residual of a later chunk), so
// that no epilogue thread ever waits for a store.
// Barriers: `full` lives in the leader (both CTAs' copies are counted there), `empty` and `acc_full`
// exist in both CTAs and receive one commit each from the leader, `acc_empty` lives in the leader and
// counts the epilogue warps of both CTAs.  No copy is multicast.
#include "common.cuh"
#include "rowquant.cuh"

namespace samb {

namespace {

constexpr int BM = 128;                        // rows per CTA (256 per pair)
constexpr int BN = 256;
constexpr int SLAB_BYTES = 128;
constexpr int A_STAGE_BYTES = BM * SLAB_BYTES;          // 16 KiB: this CTA's rows of A
constexpr int B_STAGE_BYTES = (BN / 2) * SLAB_BYTES;    // 16 KiB: this CTA's half of the W tile
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int NUM_ACC = 2;
constexpr int TMEM_COLS = NUM_ACC * BN;
constexpr int OUT_STAGE_BYTES = BM * 128;
// Operand ring and output staging share the shared memory.  bf16: 6 stages + 1 staging tile (a 256-wide tile
// takes 2 x as many tensor-pipe cycles per output byte as in int8, the store is never the hold-up).  int8: a
// stage holds twice the K depth, 5 are plenty, and the room goes to three staging tiles that rotate per
// 64-column chunk, so that a chunk never waits for the previous chunk's store to drain.  With a residual the
// staging tiles also receive the residual tile (TMA load, two chunks ahead of its use), which takes three of them.
#ifndef SAMB_PAIR_RES_STAGES_BF16
#define SAMB_PAIR_RES_STAGES_BF16 5
#endif
__host__ __device__ constexpr int pair_stages(bool int8, bool res) {
  return int8 ? 5 : (res ? SAMB_PAIR_RES_STAGES_BF16 : 6);
}
__host__ __device__ constexpr int pair_out_bufs(bool int8, bool res) {
  return int8 ? 3 : (res ? (SAMB_PAIR_RES_STAGES_BF16 == 5 ? 3 : 2) : 1);
}
__host__ __device__ constexpr int pair_smem_bytes(bool int8, bool res) {
  return pair_stages(int8, res) * STAGE_BYTES + pair_out_bufs(int8, res) * OUT_STAGE_BYTES + 1024 + 256;
}

struct PairParams {
  void* out;
  const float* bias;
  const float* a_scale;
  const float* w_scale;
  float* row_absmax;             // optional: atomic maximum of |bf16(out[m, :])| per row (see launch_gemm_i8_rowmax)
  int* status;
  long long M;
  int res_rows;                  // the residual row of output row m is m % res_rows (a multiple of 128, or >= M)
  int N, K;
  int k_slabs, last_ksteps;
  int tiles_n;
  int num_tiles;                 // < 2^31 (checked by the launcher): tile arithmetic stays in 32 bits
  int hm_group;
};

// kEpiWarps: 8 (two warps per tensor-memory lane quarter, 32 of every 64 columns each) or 16 (four per
// quarter, 16 columns each).  The cheap int8 epilogues are issue-latency bound and gain from 16; the
// bf16 ones are hidden behind the longer bf16 products either way and save barrier traffic with 8.
template <bool kInt8, int kEpi, int kEpiWarps>
__global__ void __launch_bounds__(96 + 32 * kEpiWarps, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmOut, const __grid_constant__ CUtensorMap tmRes,
                 const PairParams p) {
  constexpr bool kBias = (kEpi & SAMB_EPI_BIAS) != 0;
  constexpr bool kGelu = (kEpi & SAMB_EPI_GELU) != 0;
  constexpr bool kRes = (kEpi & SAMB_EPI_RESIDUAL) != 0;
  constexpr int EPI_THREADS = 32 * kEpiWarps;
  constexpr int CW = 64 / (kEpiWarps / 4);               // columns of a 64-column chunk per warp: 32 or 16
  constexpr int NV = CW / 8;                             // 16-byte output pieces per thread and chunk
  constexpr int STAGES = pair_stages(kInt8, kRes);
  constexpr int OUT_BUFS = pair_out_bufs(kInt8, kRes);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_out0 = smem + STAGES * STAGE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(stage_out0 + OUT_BUFS * OUT_STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;
  uint64_t* acc_empty = acc_full + NUM_ACC;
  uint64_t* res_full = acc_empty + NUM_ACC;              // residual tile landed, per staging tile
  uint64_t* stage_full = res_full + 3;                   // chunk staged by every epilogue warp, per staging tile
  uint64_t* stage_free = stage_full + 3;                 // the chunk's store has read the staging tile
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(stage_free + 3);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();               // 0 = leader of the pair
  const int pair = int(blockIdx.x >> 1), num_pairs = int(gridDim.x >> 1);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < NUM_ACC; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 2 * EPI_THREADS / 32);    // the epilogue warps of both CTAs
    }
    for (int b = 0; b < 3; ++b) {
      mbar_init(&res_full[b], 1);
      mbar_init(&stage_full[b], kEpiWarps);
      mbar_init(&stage_free[b], 1);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmOut);
    if (kRes) tma_prefetch_desc(&tmRes);
  }
  cluster_sync_all();                                    // both CTAs' barriers exist before any remote use
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int slab_elems = kInt8 ? SLAB_BYTES : SLAB_BYTES / 2;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      const uint32_t full0 = map_to_cta(&full_bar[0], 0);            // the leader's barriers
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < p.num_tiles; tile += num_pairs) {
        const int m0 = (tile / p.tiles_n) * (2 * BM) + int(rank) * BM;
        const int n0 = (tile % p.tiles_n) * BN + int(rank) * (BN / 2);
        for (int ks = 0; ks < p.k_slabs; ++ks) {
          if (!(ok = mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, 1))) break;
          uint8_t* sa = smem + stage * STAGE_BYTES;
          if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * STAGE_BYTES);   // both CTAs' copies
          tma_load_2d_pair(sa, &tmA, full0 + stage * 8, ks * slab_elems, m0);
          tma_load_2d_pair(sa + A_STAGE_BYTES, &tmB, full0 + stage * 8, ks * slab_elems, n0);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issue (leader CTA only)
    if (rank == 0) {
      const uint32_t idesc = kInt8 ? make_idesc(kAccS32, kFmtS8, kFmtS8, 2 * BM, BN)
                                   : make_idesc(kAccF32, kFmtBF16, kFmtBF16, 2 * BM, BN);
      const uint64_t desc0 = make_smem_desc(smem_u32(smem), 16, 1024, kSwizzle128B);
      const uint32_t empty_own = map_to_cta(&empty_bar[0], 0), empty_peer = map_to_cta(&empty_bar[0], 1);
      const uint32_t accf_own = map_to_cta(&acc_full[0], 0), accf_peer = map_to_cta(&acc_full[0], 1);
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < p.num_tiles; tile += num_pairs) {
        if (!(ok = mbar_wait(&acc_empty[acc], acc_phase ^ 1u, abort_flag, p.status, 2))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int ks = 0; ks < p.k_slabs; ++ks) {
          if (!(ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.status, 3))) break;
          tc_fence_after();
          if (elect_one()) {
            const uint64_t adesc = desc0 + stage * (STAGE_BYTES / 16);
            const uint64_t bdesc = adesc + A_STAGE_BYTES / 16;
            const int nsteps = ks == p.k_slabs - 1 ? p.last_ksteps : 4;
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {
              if (k4 >= nsteps) break;
              const uint32_t accumulate = (ks | k4) != 0 ? 1u : 0u;
              if (kInt8) umma_i8_ss_pair(d_tmem, adesc + k4 * 2, bdesc + k4 * 2, idesc, accumulate);
              else umma_f16_ss_pair(d_tmem, adesc + k4 * 2, bdesc + k4 * 2, idesc, accumulate);
            }
            tc_commit_pair(empty_own + stage * 8);        // the stage is reusable in both CTAs
            tc_commit_pair(empty_peer + stage * 8);
          }
          __syncwarp();
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if (elect_one()) {
          tc_commit_pair(accf_own + acc * 8);             // accumulator complete in both CTAs
          tc_commit_pair(accf_peer + acc * 8);
        }
        __syncwarp();
        if (++acc == NUM_ACC) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else if (warp == 2 + kEpiWarps) {
    // ------------------------------------------------------------------ output warp: stores, residual loads
    // One thread.  Chunk n of this CTA (64 columns of one of its tiles, in the order the epilogue works through them)
    // lives in staging tile n % OUT_BUFS.  With a residual the TMA unit copies the residual's [128 x 64] tile of a
    // chunk into that staging tile as soon as the store of the chunk that used the tile before has read it; the
    // epilogue threads read their 16-byte pieces from where they are about to write.  (Reading the residual from
    // global memory with a row per lane takes 32 cache lines per request, which made the epilogue the bottleneck
    // of the K = 1280 products.)
    if (lane == 0) {
      const uint32_t my_chunks = uint32_t((p.num_tiles - pair + num_pairs - 1) / num_pairs) * (BN / 64);
      auto chunk_coords = [&](uint32_t n, int& m0, int& col0) {
        const int t = pair + int(n / (BN / 64)) * num_pairs;
        m0 = (t / p.tiles_n) * (2 * BM) + int(rank) * BM;
        col0 = (t % p.tiles_n) * BN + int(n % (BN / 64)) * 64;
      };
      auto fetch_residual = [&](uint32_t n) {
        if (n >= my_chunks) return;
        int m0, col0;
        chunk_coords(n, m0, col0);
        const int b = int(n % OUT_BUFS);
        mbar_expect_tx(&res_full[b], OUT_STAGE_BYTES);
        tma_load_2d(stage_out0 + b * OUT_STAGE_BYTES, &tmRes, &res_full[b], col0, m0 % p.res_rows);
      };
      if (kRes)
        for (int n = 0; n < OUT_BUFS; ++n) fetch_residual(uint32_t(n));      // every staging tile starts out free
      for (uint32_t n = 0; n < my_chunks; ++n) {
        const int b = int(n % OUT_BUFS);
        if (!mbar_wait(&stage_full[b], (n / OUT_BUFS) & 1u, abort_flag, p.status, 6)) break;
        uint8_t* stage_out = stage_out0 + b * OUT_STAGE_BYTES;
        int m0, col0;
        chunk_coords(n, m0, col0);
        if (p.hm_group == 0) {
          tma_store_2d(&tmOut, stage_out, col0, m0);
        } else {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int g = (col0 + q * 16) >> 4;
            tma_store_4d(&tmOut, stage_out + q * 4096, 0, g % p.hm_group, m0, g / p.hm_group);
          }
        }
        tma_store_commit();
        // with several staging tiles, let this store run and hand back the tile of the one before it
        tma_store_wait_read<(OUT_BUFS > 1 ? 1 : 0)>();
        if (OUT_BUFS > 1 && n == 0) continue;
        const uint32_t freed = OUT_BUFS > 1 ? n - 1 : n;
        if (kRes) fetch_residual(freed + OUT_BUFS);
        else mbar_arrive(&stage_free[freed % OUT_BUFS]);
      }
      tma_store_wait_all<0>();
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps, own 128 rows
    const uint32_t lane_base = uint32_t(warp & 3) * 32u;
    const int qc = (warp - 2) >> 2;                      // which CW columns of every 64-column chunk
    const int erow = int(lane_base) + lane;
    const uint32_t acc_empty0 = map_to_cta(&acc_empty[0], 0);        // the leader's barrier
    uint32_t acc = 0, acc_phase = 0, chunk_no = 0;
    // Per-column bias and weight scale are read from global memory where they are used (every lane of a warp reads
    // the same 32 bytes, which stay in L1); the per-row activation scale of the next tile is fetched a tile ahead.
    float next_ascale = 1.0f;
    auto fetch_ascale = [&](int t) {
      next_ascale = 1.0f;
      if (!kInt8 || t >= p.num_tiles) return;
      const long long row = (long long)(t / p.tiles_n) * (2 * BM) + int(rank) * BM + erow;
      if (row < p.M) next_ascale = __ldg(p.a_scale + row);
    };
    fetch_ascale(pair);
    for (int tile = pair; tile < p.num_tiles; tile += num_pairs) {
      const int m0 = (tile / p.tiles_n) * (2 * BM) + int(rank) * BM;
      const int n0 = (tile % p.tiles_n) * BN;
      const long long row = (long long)m0 + erow;
      const bool row_ok = row < p.M;
      const float* g_bias = p.bias + n0;
      const float* g_wscale = p.w_scale + n0;
      const float a_scale = next_ascale;
      fetch_ascale(tile + num_pairs);
      // a wait that gives up ends the loop for the whole warp (its lanes meet again in __syncwarp below)
      if (!__all_sync(0xffffffffu, mbar_wait(&acc_full[acc], acc_phase, abort_flag, p.status, 4))) break;
      tc_fence_after();
      const uint32_t t_addr = tmem_base + (lane_base << 16) + acc * BN + qc * CW;
      // The chunk loop is software-pipelined: the tensor-memory load of chunk c + 1 is in flight while chunk c goes
      // through the arithmetic, and the accumulator is handed back to the MMA warp as soon as its last chunk has
      // been read (before that chunk's arithmetic and staging).
      __nv_bfloat162 m2 = __floats2bfloat162_rn(0.f, 0.f);   // running |max| of this row's outputs in this tile
      uint32_t rbuf[2][CW];
      if constexpr (CW == 32) tmem_ld_32x32b_x32(t_addr, rbuf[0]);
      else tmem_ld_32x32b_x16(t_addr, rbuf[0]);
#pragma unroll
      for (int c = 0; c < BN / 64; ++c) {
        tmem_ld_wait();                                  // chunk c is in rbuf[c & 1]
        if (c + 1 < BN / 64) {
          if constexpr (CW == 32) tmem_ld_32x32b_x32(t_addr + (c + 1) * 64, rbuf[(c + 1) & 1]);
          else tmem_ld_32x32b_x16(t_addr + (c + 1) * 64, rbuf[(c + 1) & 1]);
        } else {
          // Every column of this accumulator is in registers (the wait above).  The arrival is relaxed: a release
          // at cluster scope here stalled the warp for some 1.5 k cycles per tile, and there is nothing to publish;
          // the loads it must not overtake have completed.
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster_relaxed(acc_empty0 + acc * 8);
        }
        const uint32_t(&r)[CW] = rbuf[c & 1];
        const uint32_t sbuf = chunk_no % OUT_BUFS, suse = chunk_no / OUT_BUFS;
        uint8_t* stage_out = stage_out0 + sbuf * OUT_STAGE_BYTES;
        // Is the staging tile ready (the residual has landed / the store of the chunk that used it before has read
        // it)?  Asked before the arithmetic, without blocking, so that the answer costs nothing when it is yes.
        bool ready = true;
        if (kRes) ready = mbar_test_wait(&res_full[sbuf], suse & 1u);
        else if (suse > 0) ready = mbar_test_wait(&stage_free[sbuf], (suse - 1u) & 1u);
        float v[NV][8];
#pragma unroll
        for (int u = 0; u < NV; ++u) {
          const int ct0 = c * 64 + qc * CW + u * 8;      // first of these eight columns inside the tile
          epilogue8<kInt8, kInt8, kBias, kGelu>(r + u * 8, a_scale, g_wscale + ct0, g_bias + ct0, v[u]);
        }
        // a wait that gives up has raised the abort flag and the status word; the next accumulator wait ends the loop
        if (!ready) {
          if (kRes) mbar_wait(&res_full[sbuf], suse & 1u, abort_flag, p.status, 5);
          else mbar_wait(&stage_free[sbuf], (suse - 1u) & 1u, abort_flag, p.status, 7);
        }
        uint4 packed[NV];
#pragma unroll
        for (int u = 0; u < NV; ++u) {
          if (kRes) {
            const uint4 rv = *reinterpret_cast<const uint4*>(stage_out + erow * 128 + (((qc * NV + u) ^ (erow & 7)) << 4));
            const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 f = __bfloat1622float2(rp[j]);
              v[u][2 * j] += f.x;
              v[u][2 * j + 1] += f.y;
            }
          }
          packed[u] = make_uint4(pack_bf16x2(v[u][0], v[u][1]), pack_bf16x2(v[u][2], v[u][3]),
                                 pack_bf16x2(v[u][4], v[u][5]), pack_bf16x2(v[u][6], v[u][7]));
          if (p.row_absmax != nullptr) m2 = absmax8(m2, packed[u]);
        }
        if (p.hm_group == 0) {
          uint8_t* srow = stage_out + erow * 128;
#pragma unroll
          for (int u = 0; u < NV; ++u)
            *reinterpret_cast<uint4*>(srow + (((qc * NV + u) ^ (erow & 7)) << 4)) = packed[u];
        } else {
          // head-major: four [128][16-column] pieces (32-byte rows, 32B swizzle), one TMA store each
          uint8_t* srow = stage_out + erow * 32;
#pragma unroll
          for (int u = 0; u < NV; ++u) {
            const int unit = qc * NV + u;                // 16-byte unit inside the 64-column chunk
            *reinterpret_cast<uint4*>(srow + (unit >> 1) * 4096 + (((unit & 1) ^ ((erow >> 2) & 1)) << 4)) = packed[u];
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&stage_full[sbuf]);   // the output warp stores the chunk once every warp has arrived
        ++chunk_no;
      }
      // non-negative floats order like their bit patterns: one integer atomic per row and tile
      if (p.row_absmax != nullptr && row_ok)
        atomicMax(reinterpret_cast<int*>(p.row_absmax + row), __float_as_int(absmax_fold(m2)));
      if (++acc == NUM_ACC) { acc = 0; acc_phase ^= 1u; }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                    // no CTA leaves while its peer may still signal it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

using PairFn = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap, const PairParams);

template <bool kInt8>
PairFn pick_pair(int epi) {
  constexpr int W = kInt8 ? 16 : 8;
  switch (epi) {
    case 0: return gemm_pair_kernel<kInt8, 0, W>;
    case 1: return gemm_pair_kernel<kInt8, 1, W>;
    case 3: return gemm_pair_kernel<kInt8, 3, W>;
    case 5: return gemm_pair_kernel<kInt8, 5, W>;
    default: return nullptr;
  }
}

}  // namespace

// Returns SAMB_E_SHAPE when the problem is outside what the pair kernel covers (the caller then uses the
// single-CTA kernel); argument validity has been checked by the caller.
int launch_gemm_pair(bool int8, const void* A, int64_t lda, const void* W, int64_t ldw, const float* a_scale,
                     const float* w_scale, const float* bias, const void* residual, int64_t ldr, int64_t res_rows,
                     void* out, int64_t ldo, int64_t M, int N, int K, int epilogue, int head_dim, int32_t* status,
                     void* stream, float* row_absmax) {
  if (N % BN || M < 8 * 2 * BM) return SAMB_E_SHAPE;
  const bool res = (epilogue & SAMB_EPI_RESIDUAL) != 0;
  if (res_rows <= 0) res_rows = M;
  // the residual comes in [128 x 64] boxes: a CTA's 128 rows may not wrap around the residual's rows, and the
  // box wants 16-byte aligned rows
  if (res && ((res_rows < M && res_rows % BM) || (ldr * 2) % 16 || (reinterpret_cast<uintptr_t>(residual) & 15u)))
    return SAMB_E_SHAPE;
  // the epilogue reads bias and weight scale in 16-byte pieces; tile arithmetic is 32-bit
  if ((reinterpret_cast<uintptr_t>(bias) | reinterpret_cast<uintptr_t>(w_scale)) & 15u) return SAMB_E_SHAPE;
  if (((M + 2 * BM - 1) / (2 * BM)) * (N / BN) >= (1ll << 31) || M >= (1ll << 31)) return SAMB_E_SHAPE;
  auto kern = int8 ? pick_pair<true>(epilogue) : pick_pair<false>(epilogue);
  if (kern == nullptr) return SAMB_E_SHAPE;
  const int esz = int8 ? 1 : 2;
  const CUtensorMapDataType dt = int8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const uint32_t slab_elems = uint32_t(SLAB_BYTES / esz);
  CUtensorMap tmA, tmB, tmOut;
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
    const uint32_t box[2] = {slab_elems, uint32_t(BN / 2)};
    if (int e = make_tensor_map(&tmB, dt, 2, const_cast<void*>(W), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return e;
  }
  if (head_dim) {
    const uint64_t dims[4] = {16, uint64_t(head_dim / 16), uint64_t(M), uint64_t(N / head_dim)};
    const uint64_t strides[4] = {2, 32, uint64_t(head_dim) * 2, uint64_t(M) * head_dim * 2};
    const uint32_t box[4] = {16, 1, uint32_t(BM), 1};
    if (int e = make_tensor_map(&tmOut, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, out, dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_32B))
      return e;
  } else {
    const uint64_t dims[2] = {uint64_t(N), uint64_t(M)};
    const uint64_t strides[2] = {2, uint64_t(ldo) * 2};
    const uint32_t box[2] = {64, uint32_t(BM)};
    if (int e = make_tensor_map(&tmOut, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, out, dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_128B))
      return e;
  }
  CUtensorMap tmRes = tmOut;
  if (res) {
    const uint64_t dims[2] = {uint64_t(N), uint64_t(res_rows < M ? res_rows : M)};
    const uint64_t strides[2] = {2, uint64_t(ldr) * 2};
    const uint32_t box[2] = {64, uint32_t(BM)};
    if (int e = make_tensor_map(&tmRes, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(residual), dims, strides,
                                box, CU_TENSOR_MAP_SWIZZLE_128B))
      return e;
  }
  PairParams p;
  p.out = out;
  p.bias = bias;
  p.a_scale = a_scale;
  p.w_scale = w_scale;
  p.row_absmax = row_absmax;
  p.status = status;
  p.M = M;
  p.res_rows = int(res_rows < M ? res_rows : M);
  p.N = N;
  p.K = K;
  p.k_slabs = (K * esz + SLAB_BYTES - 1) / SLAB_BYTES;
  p.last_ksteps = (K * esz - (p.k_slabs - 1) * SLAB_BYTES + 31) / 32;
  p.tiles_n = N / BN;
  p.num_tiles = int(((M + 2 * BM - 1) / (2 * BM)) * p.tiles_n);
  p.hm_group = head_dim / 16;

  const int smem_bytes = pair_smem_bytes(int8, res);
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess)
    return SAMB_E_LAUNCH;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cfg.blockDim = dim3(int8 ? 96 + 32 * 16 : 96 + 32 * 8);   // producer, MMA, epilogue warps, output warp
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cfg.gridDim = dim3(unsigned(sm_count() & ~1));
  static int cached_clusters[2][8] = {};                  // co-resident pairs per kernel variant (0 = not asked yet)
  int& max_clusters = cached_clusters[int8 ? 1 : 0][epilogue & 7];
  if (max_clusters == 0 &&
      (cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg) != cudaSuccess || max_clusters < 1)) {
    cudaGetLastError();
    max_clusters = -1;
  }
  if (max_clusters < 1) return SAMB_E_SHAPE;              // pairs cannot be placed: single-CTA kernel
  long long pairs = max_clusters < sm_count() / 2 ? max_clusters : sm_count() / 2;
  if (p.num_tiles < pairs) pairs = p.num_tiles;
  cfg.gridDim = dim3(unsigned(2 * pairs));
  if (cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmOut, tmRes, p) != cudaSuccess) {
    cudaGetLastError();
    return SAMB_E_LAUNCH;
  }
  return launch_status();
}

}  // namespace samb
