// int8 GEMM with a 2:4-sparse weight on the sparse tensor-core path:
//   out[T, N] = epilogue( Xq[T, K] * Wsparse[N, K]^T )
// tcgen05.mma.sp takes the sparse matrix as its A operand, so the roles are swapped with respect to
// the dense kernel: a tile is 128 output channels (MMA M, rows of the compressed weight) by 208
// tokens (MMA N, rows of the activation), and the accumulator holds the tile transposed (TMEM lane =
// channel, column = token).  Per 128 logical K the producer warp brings in 64 compressed weight bytes
// per channel (64B swizzle), 128 activation bytes per token (128B swizzle) and 16 bytes of position
// codes per channel; the MMA warp copies the codes to tensor memory (tcgen05.cp) and issues two MMAs
// of logical K = 64; eight epilogue warps drain the other accumulator through one of two token-major
// staging tiles (the residual, when there is one, is brought into the same tile by TMA beforehand)
// and two TMA stores.
// kPair: the same on CTA pairs (cluster of two, cta_group::2): a pair owns 256 channels x 224 tokens, each CTA
// holds its 128 channels of the weight (values + codes) and half of the token tile, one MMA (M = 256) issued
// by the leader accumulates into both CTAs' tensor memory, so the activation operand is streamed once per
// 256 channels and its shared-memory reads per CTA are halved.  Barrier scheme as in the dense pair kernel.
#include <cstdlib>

#include "common.cuh"
#include "rowquant.cuh"

namespace samb {

namespace {

constexpr int TC = 128;                        // channels per tile
constexpr int TT = 208;                        // tokens per tile: 2 accumulators + code ring fit 512 columns
constexpr int KB = 128;                        // logical K per stage
constexpr int A_BYTES = TC * KB / 2;           // 8 KiB
constexpr int B_BYTES = TT * KB;               // 26 KiB
constexpr int E_BYTES = TC * 16;               // 2 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES + E_BYTES;   // 36 KiB, a multiple of 1024
constexpr int STAGES = 3;
constexpr int OUT_HALF_BYTES = TT * 128;       // 64 channels of every token row, 128B-swizzled
constexpr int OUT_BYTES = 2 * OUT_HALF_BYTES;   // one staging tile; there are two
constexpr int NUM_ACC = 2;
constexpr int E_COL = NUM_ACC * TT;            // 416: first column of the code ring (4 columns per stage)
constexpr int TMEM_COLS = 512;
constexpr int NUM_THREADS = 320;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 2 * OUT_BYTES + TT * 4 + 1024 + 256;
// pair mode
constexpr int TT_P = 224;                      // tokens per pair tile (112 streamed by each CTA)
constexpr int B_BYTES_P = (TT_P / 2) * KB;     // 14 KiB
constexpr int STAGE_BYTES_P = A_BYTES + B_BYTES_P + E_BYTES;   // 24 KiB
constexpr int STAGES_P = 6;                    // 144 KiB of operands in flight: a stage is only ~220 tensor cycles of work
constexpr int OUT_BUFS_P = 1;                  // one staging tile (the pair products have no GELU: the epilogue has slack)
constexpr int OUT_HALF_BYTES_P = TT_P * 128;
constexpr int SMEM_BYTES_P = STAGES_P * STAGE_BYTES_P + OUT_BUFS_P * 2 * OUT_HALF_BYTES_P + TT_P * 4 + 1024 + 256;

struct SpParams {
  void* out;
  const float* bias;
  const __nv_bfloat16* residual;
  const float* a_scale;
  const float* w_scale;
  float* row_absmax;            // optional: atomic maximum of |bf16(out[t, :])| per token row
  int* status;
  long long T;                  // tokens
  long long ldo, ldr, res_rows;
  int N, K;
  int k_blocks;
  int tiles_c;
  long long num_tiles;
};

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

template <int kEpi, bool kPair>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_sp24_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                 const __grid_constant__ CUtensorMap tmE, const __grid_constant__ CUtensorMap tmOut,
                 const __grid_constant__ CUtensorMap tmRes, const SpParams p) {
  constexpr bool kRaw = (kEpi & SAMB_EPI_RAW) != 0;
  constexpr bool kBias = (kEpi & SAMB_EPI_BIAS) != 0;
  constexpr bool kGelu = (kEpi & SAMB_EPI_GELU) != 0;
  constexpr bool kRes = (kEpi & SAMB_EPI_RESIDUAL) != 0;
  // geometry of this variant (the names shadow the single-CTA constants of the namespace)
  constexpr int TT = kPair ? TT_P : samb::TT;
  constexpr int TB = kPair ? TT_P / 2 : samb::TT;                          // token rows this CTA streams per stage
  constexpr int B_BYTES = TB * KB;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES + E_BYTES;
  constexpr int STAGES = kPair ? STAGES_P : samb::STAGES;
  constexpr int OUT_HALF_BYTES = TT * 128;
  constexpr int OUT_BYTES = 2 * OUT_HALF_BYTES;
  constexpr int OUT_BUFS = kPair ? OUT_BUFS_P : 2;                         // staging tiles
  constexpr int E_COL = NUM_ACC * TT;
  constexpr int kChunks = TT / 16;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_out = smem + STAGES * STAGE_BYTES;
  float* s_tok = reinterpret_cast<float*>(stage_out + OUT_BUFS * OUT_BYTES);      // [TT] per-token scales
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(s_tok + TT);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;
  uint64_t* acc_empty = acc_full + NUM_ACC;
  uint64_t* res_bar = acc_empty + NUM_ACC;                                 // residual tile landed, per staging tile
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(res_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = kPair ? cluster_ctarank() : 0u;                    // 0 = leader of the pair
  const long long first_tile = kPair ? (blockIdx.x >> 1) : blockIdx.x;
  const long long tile_step = kPair ? (gridDim.x >> 1) : gridDim.x;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < NUM_ACC; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], kPair ? 16 : 8);                            // the epilogue warps of the CTA / of both CTAs
      mbar_init(&res_bar[a], 1);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmE);
    if (!kRaw) tma_prefetch_desc(&tmOut);
    if (kRes) tma_prefetch_desc(&tmRes);
  }
  if (kPair) cluster_sync_all();                         // both CTAs' barriers exist before any remote use
  if (warp == 1) {
    if (kPair) { tmem_alloc_pair(tmem_slot, TMEM_COLS); tmem_relinquish_pair(); }
    else { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const uint32_t full0 = kPair ? map_to_cta(&full_bar[0], 0) : 0u;     // pair: bytes are counted by the leader
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (long long tile = first_tile; ok && tile < p.num_tiles; tile += tile_step) {
        const int ct = int(tile % p.tiles_c) * (kPair ? 2 : 1) + int(rank);   // this CTA's 128-channel tile
        const int t0 = int(tile / p.tiles_c) * TT + int(rank) * TB;           // first token row this CTA streams
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!(ok = mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, 1))) break;
          uint8_t* sa = smem + stage * STAGE_BYTES;
          if (kPair) {
            if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * STAGE_BYTES);
            tma_load_2d_pair(sa, &tmW, full0 + stage * 8, kb * (KB / 2), ct * TC);
            tma_load_2d_pair(sa + A_BYTES, &tmX, full0 + stage * 8, kb * KB, t0);
            tma_load_2d_pair(sa + A_BYTES + B_BYTES, &tmE, full0 + stage * 8, 0, (ct * p.k_blocks + kb) * TC);
          } else {
            mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
            tma_load_2d(sa, &tmW, &full_bar[stage], kb * (KB / 2), ct * TC);
            tma_load_2d(sa + A_BYTES, &tmX, &full_bar[stage], kb * KB, t0);
            tma_load_2d(sa + A_BYTES + B_BYTES, &tmE, &full_bar[stage], 0, (ct * p.k_blocks + kb) * TC);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (pair: the leader CTA only)
    if (rank == 0) {
      const uint32_t idesc = make_idesc(kAccS32, kFmtS8, kFmtS8, kPair ? 2 * TC : TC, TT) | (1u << 2);   // bit 2: sparse A
      const uint64_t adesc0 = make_smem_desc(smem_u32(smem), 16, 512, kSwizzle64B);
      const uint64_t bdesc0 = make_smem_desc(smem_u32(smem) + A_BYTES, 16, 1024, kSwizzle128B);
      const uint64_t edesc0 = make_smem_desc(smem_u32(smem) + A_BYTES + B_BYTES, 128, 128, kSwizzleNone);
      uint32_t empty_own = 0, empty_peer = 0, accf_own = 0, accf_peer = 0;
      if (kPair) {
        empty_own = map_to_cta(&empty_bar[0], 0); empty_peer = map_to_cta(&empty_bar[0], 1);
        accf_own = map_to_cta(&acc_full[0], 0); accf_peer = map_to_cta(&acc_full[0], 1);
      }
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (long long tile = first_tile; ok && tile < p.num_tiles; tile += tile_step) {
        if (!(ok = mbar_wait(&acc_empty[acc], acc_phase ^ 1u, abort_flag, p.status, 2))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * TT;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!(ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.status, 3))) break;
          tc_fence_after();
          if (elect_one()) {
            const uint32_t e_tmem = tmem_base + E_COL + stage * 4;
            const uint64_t so = uint64_t(stage) * (STAGE_BYTES / 16);
            if (kPair) tmem_cp_128x128b_pair(e_tmem, edesc0 + so);
            else tmem_cp_128x128b(e_tmem, edesc0 + so);
#pragma unroll
            for (int k2 = 0; k2 < 2; ++k2) {        // logical K 64: 32 compressed bytes of A, 64 bytes of X
              const uint32_t accumulate = (kb | k2) != 0 ? 1u : 0u;
              if (kPair) umma_i8_sp_ss_pair(d_tmem, adesc0 + so + k2 * 2, bdesc0 + so + k2 * 4, e_tmem + k2 * 2, idesc, accumulate);
              else umma_i8_sp_ss(d_tmem, adesc0 + so + k2 * 2, bdesc0 + so + k2 * 4, e_tmem + k2 * 2, idesc, accumulate);
            }
            if (kPair) { tc_commit_pair(empty_own + stage * 8); tc_commit_pair(empty_peer + stage * 8); }
            else tc_commit(&empty_bar[stage]);
          }
          __syncwarp();
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if (elect_one()) {
          if (kPair) { tc_commit_pair(accf_own + acc * 8); tc_commit_pair(accf_peer + acc * 8); }
          else tc_commit(&acc_full[acc]);
        }
        __syncwarp();
        if (++acc == NUM_ACC) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    // Thread = one channel of the tile (TMEM lane); two warps share a lane quarter and split the
    // 16-token chunks (13 or, on pairs, 14): the first takes chunks 0..6, the second the rest.
    const uint32_t lane_base = uint32_t(warp & 3) * 32u;
    const int half = (warp - 2) >> 2;
    const int ch = int(lane_base) + lane;                  // channel inside the tile
    const int et = int(threadIdx.x) - 64;                  // 0..255
    const int chunk_begin = half * 7;
    const int n_chunks = half == 0 ? 7 : kChunks - 7;
    const int unit = (ch & 63) >> 3, sub = (ch & 7) * 2;
    const uint32_t acc_empty0 = kPair ? map_to_cta(&acc_empty[0], 0) : 0u;   // pair: the leader's barrier
    uint32_t acc = 0, acc_phase = 0, it = 0;
    // The residual tile of the first tile is requested here; that of tile i+1 after tile i's stores.
    if (kRes && et == 0 && first_tile < p.num_tiles) {
      const int ct = int(first_tile % p.tiles_c) * (kPair ? 2 : 1) + int(rank);
      const int t0 = int(first_tile / p.tiles_c) * TT;
      mbar_expect_tx(&res_bar[0], OUT_BYTES);
      tma_load_2d(stage_out, &tmRes, &res_bar[0], ct * TC, t0);
      tma_load_2d(stage_out + OUT_HALF_BYTES, &tmRes, &res_bar[0], ct * TC + 64, t0);
    }
    for (long long tile = first_tile; tile < p.num_tiles; tile += tile_step, ++it) {
      const int ct = int(tile % p.tiles_c) * (kPair ? 2 : 1) + int(rank);   // this CTA's 128-channel tile
      const long long t0 = (tile / p.tiles_c) * TT;
      const int n = ct * TC + ch;
      const bool ch_ok = n < p.N;
      const uint32_t buf = OUT_BUFS == 2 ? (it & 1u) : 0u;
      // staging: [channel half][token][64 channels] bf16, 128-byte rows, 16-byte units XOR (token & 7)
      uint8_t* s_tile = stage_out + buf * OUT_BYTES;
      uint8_t* s_half = s_tile + (ch >> 6) * OUT_HALF_BYTES;
      if (!kRaw && et < TT) s_tok[et] = t0 + et < p.T ? __ldg(p.a_scale + t0 + et) : 0.f;
      float w_scale = 0.f, bias = 0.f;
      if (!kRaw && ch_ok) {
        w_scale = __ldg(p.w_scale + n);
        if (kBias) bias = __ldg(p.bias + n);
      }
      // the stores of the tile before last (same staging tile) have been read: et == 0 waited for
      // them right after it issued the previous tile's stores, before the barrier below
      bool got = mbar_wait(&acc_full[acc], acc_phase, abort_flag, p.status, 4);
      if (kRes && got) got = mbar_wait(&res_bar[buf], (it / OUT_BUFS) & 1u, abort_flag, p.status, 5);
      if (!epi_all(got)) break;                            // also publishes s_tok
      tc_fence_after();
      const uint32_t t_addr = tmem_base + (lane_base << 16) + acc * TT;
#pragma unroll 1
      for (int c = 0; c < n_chunks; ++c) {
        const int tk0 = (chunk_begin + c) * 16;            // first token of the chunk inside the tile
        uint32_t r[16];
        tmem_ld_32x32b_x16(t_addr + tk0, r);
        tmem_ld_wait();
        if (kRaw) {
          if (ch_ok) {
            int32_t* o = reinterpret_cast<int32_t*>(p.out) + n;
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (t0 + tk0 + j < p.T) o[(t0 + tk0 + j) * p.ldo] = int32_t(r[j]);
          }
        } else {
          // loads, arithmetic and stores in separate passes: shared-memory stores in between would
          // order the sixteen independent chains one after the other
          float sc[16], v[16];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float4 f = *reinterpret_cast<const float4*>(s_tok + tk0 + q * 4);
            sc[q * 4] = f.x; sc[q * 4 + 1] = f.y; sc[q * 4 + 2] = f.z; sc[q * 4 + 3] = f.w;
          }
          uint8_t* cell0 = s_half + tk0 * 128 + sub;       // (tk0 + j) & 7 == j & 7
          if (kRes) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              v[j] = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(cell0 + j * 128 + ((unit ^ (j & 7)) << 4)));
          }
          const f32x2 ws2 = pack2(w_scale, w_scale), bias2 = pack2(bias, bias);
#pragma unroll
          for (int j = 0; j < 16; j += 2) {              // two tokens per packed fp32 instruction
            f32x2 x = fmul2(fmul2(pack2(float(int(r[j])), float(int(r[j + 1]))), pack2(sc[j], sc[j + 1])), ws2);
            if (kBias) x = fadd2(x, bias2);
            if (kGelu) x = gelu_erf2(x);
            if (kRes) x = fadd2(x, pack2(v[j], v[j + 1]));
            unpack2(x, v[j], v[j + 1]);
          }
#pragma unroll
          for (int j = 0; j < 16; ++j)
            *reinterpret_cast<__nv_bfloat16*>(cell0 + j * 128 + ((unit ^ (j & 7)) << 4)) = __float2bfloat16_rn(v[j]);
        }
      }
      if (!kRaw) {
        fence_proxy_async_smem();
        epi_sync();
        if (p.row_absmax != nullptr && et < TT && t0 + et < p.T) {
          // the staged tile is token-major: thread et takes token row et of both 64-channel halves (channels past
          // N were computed from zero weights and a zero bias: they hold 0) and leaves its |max| with one atomic
          __nv_bfloat162 m2 = __floats2bfloat162_rn(0.f, 0.f);
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            const uint8_t* rowp = s_tile + hf * OUT_HALF_BYTES + et * 128;
#pragma unroll
            for (int u = 0; u < 8; ++u)      // physical unit order follows the row's swizzle: bank-conflict free
              m2 = absmax8(m2, *reinterpret_cast<const uint4*>(rowp + ((u ^ (et & 7)) << 4)));
          }
          atomicMax(reinterpret_cast<int*>(p.row_absmax + t0 + et), __float_as_int(absmax_fold(m2)));
        }
        if (et == 0) {
          tma_store_2d(&tmOut, s_tile, ct * TC, int(t0));                          // clipped at T and N
          if (ct * TC + 64 < p.N) tma_store_2d(&tmOut, s_tile + OUT_HALF_BYTES, ct * TC + 64, int(t0));
          tma_store_commit();
          tma_store_wait_read<OUT_BUFS - 1>();             // the staging tile of the next tile is free again
          const long long next = tile + tile_step;
          if (kRes && next < p.num_tiles) {
            const int nct = int(next % p.tiles_c) * (kPair ? 2 : 1) + int(rank);
            const int nt0 = int(next / p.tiles_c) * TT;
            const uint32_t nbuf = OUT_BUFS == 2 ? (buf ^ 1u) : 0u;
            uint8_t* dst = stage_out + nbuf * OUT_BYTES;
            mbar_expect_tx(&res_bar[nbuf], OUT_BYTES);
            tma_load_2d(dst, &tmRes, &res_bar[nbuf], nct * TC, nt0);
            tma_load_2d(dst + OUT_HALF_BYTES, &tmRes, &res_bar[nbuf], nct * TC + 64, nt0);
          }
        }
      }
      tc_fence_before();
      if (kPair) {
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster_relaxed(acc_empty0 + acc * 8);   // nothing to publish: the loads have completed
      } else {
        mbar_arrive_warp(&acc_empty[acc]);
      }
      if (++acc == NUM_ACC) { acc = 0; acc_phase ^= 1u; }
    }
    if (!kRaw && et == 0) tma_store_wait_all<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (kPair) cluster_sync_all();                         // no CTA leaves while its peer may still signal it
  if (warp == 1) {
    tc_fence_after();
    if (kPair) tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// One thread per (weight row, block of 128 logical K): keeps the non-zero entries of every group of
// four (padding with the lowest unused positions when fewer than two are non-zero), writes the 64 kept
// bytes and the 16 bytes of position codes (group g of the block in bits 4g..4g+3: first kept position
// in the low two bits, second in the high two).  Rows and K beyond the matrix get the code 0x4.
__global__ void pack_sp24_kernel(const int8_t* __restrict__ W, long long ldw, int N, int K, int8_t* __restrict__ Wc,
                                 long long ldc, uint8_t* __restrict__ meta, int k_blocks, int rows_padded,
                                 int* status) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)rows_padded * k_blocks) return;
  const int row = int(idx / k_blocks), kb = int(idx % k_blocks);
  uint8_t* mrow = meta + (((long long)(row / TC) * k_blocks + kb) * TC + row % TC) * 16;
  bool bad = false;
  for (int b = 0; b < 16; ++b) {
    uint32_t code = 0;
    for (int h = 0; h < 2; ++h) {
      const int k = kb * KB + (b * 2 + h) * 4;
      uint32_t nib = 0x4;                         // positions 0 and 1
      if (row < N && k < K) {
        int8_t v[4];
        *reinterpret_cast<uint32_t*>(v) = *reinterpret_cast<const uint32_t*>(W + row * ldw + k);
        int pos[2], cnt = 0, nz = 0;
        for (int i = 0; i < 4; ++i) nz += v[i] != 0;
        bad |= nz > 2;
        for (int i = 0; i < 4 && cnt < 2; ++i)
          if (v[i] != 0) pos[cnt++] = i;
        for (int i = 0; i < 4 && cnt < 2; ++i) {  // fewer than two non-zeros: fill with unused zeros
          bool used = false;
          for (int j = 0; j < cnt; ++j) used |= pos[j] == i;
          if (!used && v[i] == 0) pos[cnt++] = i;
        }
        if (pos[0] > pos[1]) { const int t = pos[0]; pos[0] = pos[1]; pos[1] = t; }
        nib = uint32_t(pos[0]) | (uint32_t(pos[1]) << 2);
        int8_t* o = Wc + row * ldc + k / 2;
        o[0] = v[pos[0]];
        o[1] = v[pos[1]];
      }
      code |= nib << (4 * h);
    }
    mrow[b] = uint8_t(code);
  }
  if (bad) atomicCAS(status, 0, int((kDevNot24 << 24) | (uint32_t(row) & 0xFFFFFFu)));
}

using SpKernelFn = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap,
                            const CUtensorMap, const SpParams);

SpKernelFn pick_sp_kernel(int epi, bool pair) {
  if (pair) {
    switch (epi) {
      case 1: return gemm_sp24_kernel<1, true>;
      case 5: return gemm_sp24_kernel<5, true>;
      case SAMB_EPI_RAW: return gemm_sp24_kernel<SAMB_EPI_RAW, true>;
      default: return nullptr;
    }
  }
  switch (epi) {
    case 0: return gemm_sp24_kernel<0, false>;
    case 1: return gemm_sp24_kernel<1, false>;
    case 2: return gemm_sp24_kernel<2, false>;
    case 3: return gemm_sp24_kernel<3, false>;
    case 4: return gemm_sp24_kernel<4, false>;
    case 5: return gemm_sp24_kernel<5, false>;
    case 6: return gemm_sp24_kernel<6, false>;
    case 7: return gemm_sp24_kernel<7, false>;
    default: return gemm_sp24_kernel<SAMB_EPI_RAW, false>;
  }
}

}  // namespace
}  // namespace samb

extern "C" {

int64_t samb_sp24_meta_bytes(int N, int K) {
  if (N <= 0 || K <= 0) return 0;
  const int64_t tiles_c = (N + samb::TC - 1) / samb::TC, k_blocks = (K + samb::KB - 1) / samb::KB;
  return tiles_c * k_blocks * samb::TC * 16;
}

int samb_pack_sp24(const int8_t* Wq, int64_t ldw, int N, int K, int8_t* Wc, int64_t ldc, uint8_t* meta,
                   int32_t* status, void* stream) {
  if (Wq == nullptr || Wc == nullptr || meta == nullptr || status == nullptr) return SAMB_E_BADARG;
  if (N <= 0 || K <= 0) return SAMB_E_BADARG;
  if (K % 32 || ldw % 4 || ldw < K || ldc % 16 || ldc < K / 2) return SAMB_E_SHAPE;
  if ((reinterpret_cast<uintptr_t>(Wq) & 3u) || (reinterpret_cast<uintptr_t>(meta) & 15u)) return SAMB_E_ALIGN;
  const int k_blocks = (K + samb::KB - 1) / samb::KB;
  const int rows_padded = (N + samb::TC - 1) / samb::TC * samb::TC;
  const long long threads = (long long)rows_padded * k_blocks;
  samb::pack_sp24_kernel<<<unsigned((threads + 127) / 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      Wq, ldw, N, K, Wc, ldc, meta, k_blocks, rows_padded, status);
  return samb::launch_status();
}

}  // extern "C"

namespace samb {
int launch_gemm_i8_sp24(const int8_t* Xq, int64_t ldx, const float* x_scale, const int8_t* Wc, int64_t ldc,
                        const uint8_t* meta, const float* w_scale, const float* bias, const void* residual,
                        int64_t ldr, int64_t res_rows, void* out, int64_t ldo, int64_t T, int N, int K, int epilogue,
                        int32_t* status, void* stream, float* row_absmax) {
  if (Xq == nullptr || Wc == nullptr || meta == nullptr || out == nullptr || status == nullptr) return SAMB_E_BADARG;
  if (T < 0 || N <= 0 || K <= 0) return SAMB_E_BADARG;
  if (epilogue & ~(SAMB_EPI_BIAS | SAMB_EPI_GELU | SAMB_EPI_RESIDUAL | SAMB_EPI_RAW)) return SAMB_E_BADARG;
  const bool raw = (epilogue & SAMB_EPI_RAW) != 0;
  if (raw && epilogue != SAMB_EPI_RAW) return SAMB_E_BADARG;
  if ((epilogue & SAMB_EPI_BIAS) && bias == nullptr) return SAMB_E_BADARG;
  if ((epilogue & SAMB_EPI_RESIDUAL) && residual == nullptr) return SAMB_E_BADARG;
  if (!raw && (x_scale == nullptr || w_scale == nullptr)) return SAMB_E_BADARG;
  if (K % 32 || ldx % 16 || ldx < K || ldc % 16 || ldc < K / 2) return SAMB_E_SHAPE;
  if (N % 8 || ldo < N || (!raw && ldo % 8)) return SAMB_E_SHAPE;
  // the residual tile is fetched by TMA: no row broadcast here, 16-byte row pitch and base
  if ((epilogue & SAMB_EPI_RESIDUAL) && (ldr < N || ldr % 8 || res_rows != T)) return SAMB_E_SHAPE;
  if ((epilogue & SAMB_EPI_RESIDUAL) && (reinterpret_cast<uintptr_t>(residual) & 15u)) return SAMB_E_ALIGN;
  if (T > (int64_t(1) << 31) - TT) return SAMB_E_SHAPE;
  if ((reinterpret_cast<uintptr_t>(out) & 15u) || (reinterpret_cast<uintptr_t>(meta) & 15u)) return SAMB_E_ALIGN;
  if (int e = check_device_arch()) return e;
  if (T == 0) return SAMB_OK;

  SpParams p;
  p.out = out;
  p.bias = bias;
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.a_scale = x_scale;
  p.w_scale = w_scale;
  p.row_absmax = row_absmax;
  p.status = status;
  p.T = T;
  p.ldo = ldo;
  p.ldr = ldr;
  p.res_rows = res_rows > 0 ? res_rows : 1;
  p.N = N;
  p.K = K;
  p.k_blocks = (K + KB - 1) / KB;
  // CTA pairs for the products without the GELU epilogue (that one is bound by its epilogue either way)
  auto pair_kern = pick_sp_kernel(epilogue, true);
  const bool pair = pair_kern != nullptr && N % (2 * TC) == 0 && T >= 2048 && getenv("SAMB_GEMM_SINGLE_CTA") == nullptr;
  const int tt = pair ? TT_P : TT;                       // tokens per tile
  const int tiles128 = (N + TC - 1) / TC;                // 128-channel tiles of the weight (layout of `meta`)
  p.tiles_c = pair ? N / (2 * TC) : tiles128;
  p.num_tiles = ((T + tt - 1) / tt) * p.tiles_c;

  CUtensorMap tmW, tmX, tmE, tmOut;
  {
    const uint64_t dims[2] = {uint64_t(K / 2), uint64_t(N)};
    const uint64_t strides[2] = {1, uint64_t(ldc)};
    const uint32_t box[2] = {uint32_t(KB / 2), uint32_t(TC)};
    if (int e = make_tensor_map(&tmW, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(Wc), dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_64B))
      return e;
  }
  {
    const uint64_t dims[2] = {uint64_t(K), uint64_t(T)};
    const uint64_t strides[2] = {1, uint64_t(ldx)};
    const uint32_t box[2] = {uint32_t(KB), uint32_t(pair ? TT_P / 2 : TT)};
    if (int e = make_tensor_map(&tmX, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(Xq), dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_128B))
      return e;
  }
  {
    const uint64_t dims[2] = {16, uint64_t(tiles128) * p.k_blocks * TC};
    const uint64_t strides[2] = {1, 16};
    const uint32_t box[2] = {16, uint32_t(TC)};
    if (int e = make_tensor_map(&tmE, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(meta), dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_NONE))
      return e;
  }
  tmOut = tmX;
  if (!raw) {
    const uint64_t dims[2] = {uint64_t(N), uint64_t(T)};
    const uint64_t strides[2] = {2, uint64_t(ldo) * 2};
    const uint32_t box[2] = {64, uint32_t(tt)};
    if (int e = make_tensor_map(&tmOut, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, out, dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_128B))
      return e;
  }
  CUtensorMap tmRes = tmOut;
  if (epilogue & SAMB_EPI_RESIDUAL) {
    const uint64_t dims[2] = {uint64_t(N), uint64_t(T)};
    const uint64_t strides[2] = {2, uint64_t(ldr) * 2};
    const uint32_t box[2] = {64, uint32_t(tt)};
    if (int e = make_tensor_map(&tmRes, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(residual), dims, strides,
                                box, CU_TENSOR_MAP_SWIZZLE_128B))
      return e;
  }
  if (pair) {
    if (cudaFuncSetAttribute(pair_kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES_P) != cudaSuccess)
      return SAMB_E_LAUNCH;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES_P;
    cfg.stream = static_cast<cudaStream_t>(stream);
    long long pairs = sm_count() / 2;
    if (p.num_tiles < pairs) pairs = p.num_tiles;
    cfg.gridDim = dim3(unsigned(2 * pairs));
    if (cudaLaunchKernelEx(&cfg, pair_kern, tmW, tmX, tmE, tmOut, tmRes, p) != cudaSuccess) {
      cudaGetLastError();
      return SAMB_E_LAUNCH;
    }
    return launch_status();
  }
  auto kern = pick_sp_kernel(epilogue, false);
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
    return SAMB_E_LAUNCH;
  const long long grid = p.num_tiles < sm_count() ? p.num_tiles : sm_count();
  kern<<<dim3(unsigned(grid)), dim3(NUM_THREADS), SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(tmW, tmX, tmE, tmOut, tmRes, p);
  return launch_status();
}
}  // namespace samb

extern "C" {

int samb_gemm_i8_sp24(const int8_t* Xq, int64_t ldx, const float* x_scale, const int8_t* Wc, int64_t ldc,
                      const uint8_t* meta, const float* w_scale, const float* bias, const void* residual,
                      int64_t ldr, int64_t res_rows, void* out, int64_t ldo, int64_t T, int N, int K, int epilogue,
                      int32_t* status, void* stream) {
  return samb::launch_gemm_i8_sp24(Xq, ldx, x_scale, Wc, ldc, meta, w_scale, bias, residual, ldr, res_rows, out, ldo, T,
                                   N, K, epilogue, status, stream, nullptr);
}

}  // extern "C"
