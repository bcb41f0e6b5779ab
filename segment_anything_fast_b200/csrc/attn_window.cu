// Attention with the decomposed relative-position bias for the windowed blocks: every window is
// WS x WS = N tokens (14 x 14 = 196) attending to themselves,
//   O = softmax(scale * Q K^T + rel_h[i, j / WS] + rel_w[i, j % WS]) V.
//
// The work items are (window, head) pairs: ~107 KB of q/k/v in, 31 KB out, 39 MFLOP — a memory-bound
// stream.  One persistent CTA per SM walks its items with a two-deep TMA ring (the loads of item
// k+1 fly while item k is being computed):
//   warp 0      TMA producer: Q (two 128-row tiles), K and V (N rounded up to 208 rows) per item
//   warps 1, 7  tcgen05.mma issue, one warp per query tile: Q K^T into tensor memory, later P V
//   warps 2..6, 8, 9  softmax, one thread per query row (warps 2..5 rows 0..127; warps 8, 9, 6 rows 128..223 of
//               tile 1: its fourth lane quarter, rows 224..255, lies beyond the window and the key padding, so the
//               warp that would own it issues tile 1's products instead)
//  * The logits of a tile occupy 208 TMEM columns.  The threads read them twice (row maximum, then
//    exponentials) and write P back as packed bf16 pairs over the columns already consumed, so P V
//    takes its A operand from tensor memory and P never touches shared memory.  The product lands in
//    columns [112, 192) of the same tile.
//  * rel_w rides on the tensor core: A = [Q | rel_w/scale (16 columns)], B = [K | E], E[j, j % WS] = 1.
//  * rel_h is constant over runs of WS keys and is folded into the exp2 FMA addend.
//  * The bias values of item k+1 are fetched into registers before the softmax of item k starts (tensor / stored
//    product sources).  With the tables themselves as the source (what the encoder uses), the tile's MMA warp first
//    multiplies the tile's Q rows by the resident [64 x d] block [rel_pos_h | rel_pos_w] (N = 64, into the logit
//    columns, which are idle then); every thread reads its 2 x 27 products from tensor memory and shifts out its
//    2 x 14 values rel[k] = T[pos + 13 - k] in registers, so no product tensor exists in global memory.
// Padded layouts (qkv_fused 0 / 1): zero-padded window tokens are ordinary rows of the padded qkv buffer;
// rows N..207 of the K/V box belong to the next window and their probabilities are written as zero.
// Raster layout (qkv_fused 2): q/k/v stay in raster token order and never hold pad tokens.  A window is
// gathered by WS x WS TMA boxes whose out-of-range part (border windows) is zero-filled.  A pad token's
// key and value are the projection biases (its LayerNorm output is zero), so for border windows the
// softmax warps overwrite the pad rows of the K and V tiles with k_bias / v_bias of the head before they
// release their tile's first product; from there on a pad key is
// an ordinary key, exactly as in the padded layouts.
#include <cuda_fp16.h>

#include "common.cuh"

namespace samb {
namespace {

constexpr int NUM_THREADS = 320;   // TMA warp, tile-0 MMA warp, 4 + 3 softmax warps, tile-1 MMA warp (warp 7: the
                                   // lane quarter of tile 1 whose rows 224..255 lie beyond the window and the key padding)
constexpr int TMEM_COLS = 512;   // tile 0 at column 0, tile 1 at column 256
constexpr int kOCol = 112;       // P V result inside a tile's columns (P uses [0, 104))
constexpr int kTCol = 192;       // mode 2: products with the table block, 64 columns (free once an item's P is complete)
constexpr int STAGES = 2;
constexpr float kLog2e = 1.4426950408889634f;

struct WinParams {
  const __nv_bfloat16* rel_h;    // mode 0: [W*H, N, WS]
  const __nv_bfloat16* rel_w;
  const __nv_bfloat16* tab;      // mode 1: table products [W*N, ldt]
  long long ldt;
  int t_head_stride, t_w_off, rel_mode;   // rel_mode: 0 tensors, 1 stored table products, 2 products computed here
  __nv_bfloat16* o;
  long long o_pitch;
  int qkv_fused;                 // 0: q/k/v/o are [W*H*N, d]; 1: head-major qkv [3H][W*N][d], o rows are raster tokens
  int H, grid, nw;               // raster side and windows per side (fused modes)
  int B, vlast;                  // raster mode: images, valid extent of the last window of a row / column
  const __nv_bfloat16* kv_bias;  // raster mode: qkv projection bias [3H * D] (keys / values of pad tokens)
  int items;                     // number of (window, head) pairs
  unsigned long long mH, mWW, mNW;   // ceil(2^40 / d) for d = H, nw * nw, nw (0: divide the slow way; see fdiv)
  float scale;
  int* status;
};

template <int D, int WS>
struct WinSmem {
  static constexpr int N = WS * WS;
  static constexpr int NK = (N + 15) / 16 * 16;      // keys rounded up to the MMA granule (208)
  static constexpr int CH = D / 16;
  static constexpr int KSTEPS = NK / 16;
  static constexpr int Q_CHUNK = NK * 32;            // query rows per 16-column chunk; tile 1's product reads up to
                                                     // row 255, i.e. past the chunk: rows >= N are never stored
  static constexpr int KV_CHUNK = NK * 32;
  static constexpr int STAGE = CH * (Q_CHUNK + 2 * KV_CHUNK);   // Q | K | V of one item
  static constexpr int OFF_K = CH * Q_CHUNK;         // inside a stage
  static constexpr int OFF_V = OFF_K + CH * KV_CHUNK;
  static constexpr int OFF_RELW = STAGES * STAGE;    // [256][16] bf16, 32B swizzle (per item)
  static constexpr int OFF_E = OFF_RELW + 256 * 32;  // [NK][16] bf16 one-hot (constant)
  static constexpr int OFF_TAB = OFF_E + KV_CHUNK;   // [CH][64][16] bf16 table block [rel_pos_h | rel_pos_w], 32B swizzle
  static constexpr int TAB_CHUNK = 64 * 32;
  static constexpr int OFF_BAR = OFF_TAB + CH * TAB_CHUNK;
  static constexpr int OFF_PADTAB = OFF_BAR + 256;   // [3][N] key index of the i-th pad token per border-window kind
  static constexpr int BYTES = OFF_PADTAB + 3 * 256 + 1024;
  static_assert(N <= 256 && NK <= 256 && WS <= 16, "window too large for this kernel");
  static_assert(STAGE % 256 == 0 && Q_CHUNK % 256 == 0 && NK / 2 <= kOCol && kOCol + D <= 256, "layout");
  static_assert(CH * Q_CHUNK >= N * D * 2, "the output rows are staged in the Q region");
  static_assert(BYTES <= 227 * 1024, "shared memory");
};

// x / d for 0 <= x < 2^20 with m = ceil(2^40 / d): a multiplication instead of the ~100-instruction division, which
// sits on every item's critical path (the border-window test of the bias prologue).  m == 0: plain division.
__device__ __forceinline__ int fdiv(int x, int d, unsigned long long m) {
  return m ? int((static_cast<unsigned long long>(static_cast<unsigned int>(x)) * m) >> 40) : x / d;
}
__host__ inline unsigned long long fdiv_magic(long long items, int d) {
  if (items >= (1ll << 20) || d <= 0) return 0ull;
  return ((1ull << 40) + static_cast<unsigned long long>(d) - 1) / static_cast<unsigned long long>(d);
}
// two 16-bit elements of the tensors' type (bfloat16, or float16 when kHalf) in one word
template <bool kHalf>
__device__ __forceinline__ uint32_t wpack2(float lo, float hi) {
  if constexpr (kHalf) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float wexp2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
template <bool kHalf>
__device__ __forceinline__ float bits_to_float(uint32_t bits16) {      // low 16 bits hold one element
  if constexpr (kHalf) return __half2float(__ushort_as_half(static_cast<unsigned short>(bits16)));
  return __uint_as_float(bits16 << 16);
}

// out[e] = v[s + WS - 1 - e], e < WS: the WS consecutive products T[pos .. pos + WS - 1] of a row, in key order
// (rel[k] = T[pos + WS - 1 - k]).  A four-stage shifter on registers; s < 16.
template <int WS>
__device__ __forceinline__ void select_shifted(const uint32_t (&v)[32], int s, float (&out)[WS]) {
  uint32_t a[24], b[20], c[18];
  const bool s8 = s & 8, s4 = s & 4, s2 = s & 2, s1 = s & 1;
#pragma unroll
  for (int q = 0; q < 24; ++q) a[q] = s8 ? v[q + 8] : v[q];
#pragma unroll
  for (int q = 0; q < 20; ++q) b[q] = s4 ? a[q + 4] : a[q];
#pragma unroll
  for (int q = 0; q < 18; ++q) c[q] = s2 ? b[q + 2] : b[q];
#pragma unroll
  for (int e = 0; e < WS; ++e) {
    const int q = WS - 1 - e;
    out[e] = __uint_as_float(s1 ? c[q + 1] : c[q]);
  }
}
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// kHalf: q, k, v, the bias tensors and the output are float16 (bias-tensor mode only; the table modes are bf16).
template <int D, int WS, bool kHalf>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_window_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                   const __grid_constant__ CUtensorMap tmT, const WinParams p) {
  using L = WinSmem<D, WS>;
  constexpr int N = L::N, NK = L::NK, CH = L::CH;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* full = bars + 0;        // [STAGES] k/v of an item have landed
  uint64_t* empty = bars + 2;       // [STAGES] every MMA reading the stage has finished and its output store was read
  uint64_t* pro_done = bars + 4;    // [2]      this item's rel_w rows of tile t are in shared memory
  uint64_t* s_full = bars + 6;      // [2]      logits of tile t are in TMEM
  uint64_t* p_full = bars + 8;      // [2]      P of tile t is in TMEM
  uint64_t* o_full = bars + 10;     // [2]      P V of tile t is in TMEM
  uint64_t* t_free = bars + 12;     // [2]      tile t's TMEM columns may be overwritten (O has been read)
  uint64_t* s_done = bars + 14;     // [2][2]   logits product of tile t for items of parity k & 1 has read its Q rows:
                                    //          what the OTHER tile waits for before it stages output over them.  Two
                                    //          barriers per tile because a tile may be a whole item ahead of the other.
  uint64_t* t_full = bars + 18;     // [2]      mode 2: the table products of tile t are in TMEM
  uint64_t* tab_full = bars + 20;   //          mode 2: the table block is in shared memory
  uint64_t* q_full = bars + 21;     // [STAGES] q of an item has landed (ahead of k/v: the table products only need q)
  uint64_t* out_ready = bars + 23;  // [STAGES] every softmax warp has staged its output rows of the item in the stage
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 25);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    // a stage is free when both tiles' MMAs that read it have finished AND the output store staged in it has been read
    // (the producer sends that store itself before it waits for `empty`)
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1); mbar_init(&q_full[s], 1); mbar_init(&empty[s], 2); mbar_init(&out_ready[s], 7);
    }
    for (int t = 0; t < 2; ++t) {
      const int nw_t = t == 0 ? 4 : 3;          // softmax warps of the tile (tile 1 has real rows in three lane quarters)
      mbar_init(&pro_done[t], nw_t);
      mbar_init(&s_done[t * 2], 1); mbar_init(&s_done[t * 2 + 1], 1);
      mbar_init(&s_full[t], 1); mbar_init(&p_full[t], nw_t); mbar_init(&o_full[t], 1); mbar_init(&t_free[t], nw_t);
      mbar_init(&t_full[t], 1);
    }
    mbar_init(tab_full, 1);
    fence_mbar_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmO);
    if (p.rel_mode == 2) tma_prefetch_desc(&tmT);
  }
  if (p.qkv_fused == 2) {
    // rows N..NK-1 of every K / V chunk are never written by a copy in this mode: zero them once (their
    // probabilities are zero, but 0 x stale bits must not be a NaN)
    // pad-token lists: kind 0 = right border (columns >= vlast), 1 = bottom border (rows >= vlast), 2 = corner
    for (int idx = threadIdx.x; idx < 3 * N; idx += NUM_THREADS) {
      const int kind = idx / N, pi = idx - kind * N;
      const int vy = kind == 0 ? WS : p.vlast, vx = kind == 1 ? WS : p.vlast;
      const int n_right = vy * (WS - vx), n_pad = n_right + (WS - vy) * WS;
      int r = 0;
      if (pi < n_pad) {
        if (pi < n_right) r = (pi / (WS - vx)) * WS + vx + pi % (WS - vx);
        else r = (vy + (pi - n_right) / WS) * WS + (pi - n_right) % WS;
      }
      smem[L::OFF_PADTAB + kind * 256 + pi] = uint8_t(r);
    }
    constexpr int kTail = NK - N;
    for (int idx = threadIdx.x; idx < STAGES * 2 * CH * kTail * 2; idx += NUM_THREADS) {
      const int half = idx & 1, r = (idx >> 1) % kTail, c = (idx >> 1) / kTail % CH, kv = (idx >> 1) / (kTail * CH) % 2,
                st = (idx >> 1) / (kTail * CH * 2);
      uint8_t* row = smem + st * L::STAGE + (kv ? L::OFF_V : L::OFF_K) + c * L::KV_CHUNK + (N + r) * 32;
      *reinterpret_cast<uint4*>(row + half * 16) = make_uint4(0u, 0u, 0u, 0u);
    }
    fence_proxy_async_smem();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      if (p.rel_mode == 2) {                         // the table block, once per CTA
        mbar_expect_tx(tab_full, CH * L::TAB_CHUNK);
        tma_load_3d(smem + L::OFF_TAB, &tmT, tab_full, 0, 0, 0);
      }
      // The item's output is staged in the Q region of its stage by the softmax warps; this thread sends it (one
      // TMA store: a WS x WS x D box of the output tensor, which drops the pad tokens of border windows by clipping)
      // when it comes back to the stage for the load of the item after next, so no softmax warp waits for a store.
      auto send_output = [&](int it_o, uint32_t st_o, uint32_t use_parity) -> bool {
        if (!mbar_wait(&out_ready[st_o], use_parity, abort_flag, p.status, 14)) return false;
        int cx = 0, cy = 0, cz = 0, cw = it_o;
        if (p.qkv_fused) {
          const int w = fdiv(it_o, p.H, p.mH), h = it_o - w * p.H;
          const int ww = p.nw * p.nw;
          const int b = fdiv(w, ww, p.mWW), wi = w - b * ww;
          const int wy = fdiv(wi, p.nw, p.mNW), wx = wi - wy * p.nw;
          cx = h * D; cy = wx * WS; cz = wy * WS; cw = b;
        }
        tma_store_4d(&tmO, smem + st_o * L::STAGE, cx, cy, cz, cw);
        tma_store_commit();
        tma_store_wait_read<0>();                                // the staging rows have been read
        return true;
      };
      uint32_t stage = 0, phase = 0;
      int j = 0;
      bool ok = true;
      for (int it = blockIdx.x; it < p.items; it += gridDim.x, ++j) {
        const int w = fdiv(it, p.H, p.mH), h = it - w * p.H;
        int rq, rk, rv;                              // first row of this item in the q, k, v operands
        if (p.qkv_fused) {                           // head-major buffer: planes [q heads | k heads | v heads]
          const int R = (p.items / p.H) * N;         // rows per plane
          rq = h * R + w * N; rk = (p.H + h) * R + w * N; rv = (2 * p.H + h) * R + w * N;
        } else {
          rq = rk = rv = it * N;
        }
        if (j >= STAGES && !(ok = send_output(it - STAGES * int(gridDim.x), stage, phase ^ 1u))) break;
        if (!(ok = mbar_wait(&empty[stage], phase ^ 1u, abort_flag, p.status, 1))) break;
        uint8_t* st = smem + stage * L::STAGE;
        if (p.qkv_fused == 2) {
          const int ww = p.nw * p.nw;
          const int b = fdiv(w, ww, p.mWW), wi = w - b * ww;
          const int wy = fdiv(wi, p.nw, p.mNW), wx = wi - wy * p.nw;
          mbar_expect_tx(&q_full[stage], CH * N * 32);
          mbar_expect_tx(&full[stage], 2 * CH * N * 32);
#pragma unroll
          for (int c = 0; c < CH; ++c)             // one WS x WS box per 16-column chunk; q first
            tma_load_4d(st + c * L::Q_CHUNK, &tmQ, &q_full[stage], c * 16, wx * WS, wy * WS, h * p.B + b);
#pragma unroll
          for (int c = 0; c < CH; ++c)
            tma_load_4d(st + L::OFF_K + c * L::KV_CHUNK, &tmQ, &full[stage], c * 16, wx * WS, wy * WS, (p.H + h) * p.B + b);
#pragma unroll
          for (int c = 0; c < CH; ++c)
            tma_load_4d(st + L::OFF_V + c * L::KV_CHUNK, &tmQ, &full[stage], c * 16, wx * WS, wy * WS, (2 * p.H + h) * p.B + b);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          continue;
        }
        mbar_expect_tx(&q_full[stage], CH * L::Q_CHUNK);
        mbar_expect_tx(&full[stage], 2 * CH * L::KV_CHUNK);
        tma_load_3d(st, &tmQ, &q_full[stage], 0, rq, 0);
        tma_load_3d(st + L::OFF_K, &tmK, &full[stage], 0, rk, 0);
        tma_load_3d(st + L::OFF_V, &tmV, &full[stage], 0, rv, 0);
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
      // the outputs of the last items (those no later load came back for)
      for (int r = j > STAGES ? j - STAGES : 0; ok && r < j; ++r)
        ok = send_output(int(blockIdx.x) + r * int(gridDim.x), uint32_t(r % STAGES), uint32_t(r / STAGES) & 1u);
      tma_store_wait_all<0>();
    }
  } else if (warp == 1 || warp == 7) {
    // ---------------------------------------------------------------- MMA issue, one warp per query tile
    // (whole warp, one elected lane issues).  Issuing holds the thread until the tensor pipe has taken the
    // instructions, and each tile's chain S -> softmax -> P V -> output is serial: with a warp per tile the
    // two chains only meet in the tensor pipe, one tile's softmax overlapping the other tile's products.
    const int t = warp == 1 ? 0 : 1;
    constexpr uint32_t kFmt = kHalf ? kFmtF16 : kFmtBF16;
    constexpr uint32_t idesc_s = make_idesc(kAccF32, kFmt, kFmt, 128, NK);
    constexpr uint32_t idesc_o = make_idesc(kAccF32, kFmt, kFmt, 128, D, false, /*B MN-major*/ true);
    // K-major, 32B swizzle (8-row groups 256 B apart); start addresses move in 16-byte units
    const uint64_t dq0 = make_smem_desc(smem_u32(smem), 16, 256, kSwizzle32B);
    const uint64_t drw = make_smem_desc(smem_u32(smem + L::OFF_RELW), 16, 256, kSwizzle32B);
    const uint64_t de = make_smem_desc(smem_u32(smem + L::OFF_E), 16, 256, kSwizzle32B);
    // V: MN-major, column chunks KV_CHUNK apart (LBO), 8-key groups 256 B apart (SBO)
    const uint64_t dv0 = make_smem_desc(smem_u32(smem + L::OFF_V), L::KV_CHUNK, 256, kSwizzle32B);
    const uint32_t d_tmem = tmem_base + t * 256;
    constexpr uint32_t idesc_t = make_idesc(kAccF32, kFmtBF16, kFmtBF16, 128, 64);
    const uint64_t dtab = make_smem_desc(smem_u32(smem + L::OFF_TAB), 16, 256, kSwizzle32B);
    uint32_t stage = 0, phase = 0, k = 0;
    bool ok = true;
    // Mode 2: the products of an item's queries with the table block go to columns kTCol.. of the tile, which
    // are free from the moment the previous item's probabilities are complete (its logits are consumed, its P and O
    // sit below kTCol).  They are issued one item ahead, in front of the previous item's P V, so that the softmax
    // threads can pick an item's bias values while that P V runs instead of at the head of the item's own chain.
    const bool ahead = p.rel_mode == 2;
    auto issue_tables = [&](uint32_t st) {
      tc_fence_after();
      if (elect_one()) {
        const uint64_t dq = dq0 + st * (L::STAGE / 16);
#pragma unroll
        for (int c = 0; c < CH; ++c)
          umma_f16_ss(d_tmem + kTCol, dq + (c * L::Q_CHUNK + t * 4096) / 16, dtab + c * (L::TAB_CHUNK / 16), idesc_t, c != 0);
        tc_commit(&t_full[t]);
      }
      __syncwarp();
    };
    if (ahead && int(blockIdx.x) < p.items) {
      ok = mbar_wait(tab_full, 0, abort_flag, p.status, 11) && mbar_wait(&q_full[0], 0, abort_flag, p.status, 13);
      if (ok) issue_tables(0);
    }
    for (int it = blockIdx.x; ok && it < p.items; it += gridDim.x, ++k) {
      const uint32_t par = k & 1u;
      if (!(ok = mbar_wait(&q_full[stage], phase, abort_flag, p.status, 2))) break;
      if (!(ok = mbar_wait(&full[stage], phase, abort_flag, p.status, 2))) break;
      if (!(ok = mbar_wait(&pro_done[t], par, abort_flag, p.status, 3))) break;
      if (!(ok = mbar_wait(&t_free[t], par ^ 1u, abort_flag, p.status, 4))) break;
      tc_fence_after();
      if (elect_one()) {                           // logits of this tile
        const uint64_t dq = dq0 + stage * (L::STAGE / 16);
        const uint64_t dk = dq + L::OFF_K / 16;
#pragma unroll
        for (int c = 0; c < CH; ++c)
          umma_f16_ss(d_tmem, dq + (c * L::Q_CHUNK + t * 4096) / 16, dk + c * (L::KV_CHUNK / 16), idesc_s, c != 0);
        umma_f16_ss(d_tmem, drw + t * (4096 / 16), de, idesc_s, 1u);
        tc_commit(&s_full[t]);
        tc_commit(&s_done[t * 2 + par]);
      }
      __syncwarp();
      if (!(ok = mbar_wait(&p_full[t], par, abort_flag, p.status, 5))) break;
      // the next item's table products go first when its queries have landed (they normally have), else after P V
      const uint32_t nstage = stage + 1 == STAGES ? 0u : stage + 1, nphase = nstage == 0 ? phase ^ 1u : phase;
      bool tables_due = ahead && it + int(gridDim.x) < p.items;
      if (tables_due && mbar_test_wait(&q_full[nstage], nphase)) {
        issue_tables(nstage);
        tables_due = false;
      }
      tc_fence_after();
      if (elect_one()) {                           // P V of this tile: A = P from TMEM, B = V
        const uint64_t dv = dv0 + stage * (L::STAGE / 16);
#pragma unroll
        for (int kk = 0; kk < L::KSTEPS; ++kk)
          umma_f16_ts(d_tmem + kOCol, d_tmem + kk * 8, dv + kk * (512 / 16), idesc_o, kk != 0);
        tc_commit(&o_full[t]);
        tc_commit(&empty[stage]);                  // this tile has issued everything that reads the stage
      }
      __syncwarp();
      if (tables_due) {
        if (!(ok = mbar_wait(&q_full[nstage], nphase, abort_flag, p.status, 13))) break;
        issue_tables(nstage);
      }
      stage = nstage;
      phase = nphase;
    }
  } else {
    // ---------------------------------------------------------------- softmax (one thread = one query row)
    const int t = (warp - 2) >> 2;                               // query tile of this warp
    const int i = (warp & 3) * 32 + lane;                        // row in the tile == TMEM lane
    const int n = t * 128 + i;                                   // token inside the window
    const bool valid = n < N;
    const uint32_t lane_addr = tmem_base + (uint32_t((warp & 3) * 32) << 16) + t * 256;
    const int qh = n / WS, qw = n - qh * WS;
    const int sw = (n >> 2) & 1;                                 // 32B swizzle: 16-byte halves swap every 4 rows
    const float inv_scale = p.rel_mode == 0 ? 1.0f / p.scale : 1.0f;   // table products arrive pre-divided
    const float c2 = p.scale * kLog2e;

    if (n < NK) {                                                // constant one-hot row of key n
      constexpr uint32_t kOne = kHalf ? 0x3C00u : 0x3F80u;       // 1.0 in the operands' type
      uint32_t e[8];
#pragma unroll
      for (int q = 0; q < 8; ++q)
        e[q] = (valid && qw == 2 * q ? kOne : 0u) | (valid && qw == 2 * q + 1 ? (kOne << 16) : 0u);
      uint8_t* erow = smem + L::OFF_E + n * 32;
      *reinterpret_cast<uint4*>(erow + ((0 ^ sw) << 4)) = make_uint4(e[0], e[1], e[2], e[3]);
      *reinterpret_cast<uint4*>(erow + ((1 ^ sw) << 4)) = make_uint4(e[4], e[5], e[6], e[7]);
    }

    // Raw bf16 bias values of one item, [rel_h | rel_w] x 12 words; nothing touches them until the item
    // starts, so the loads issued for item k+1 have the whole of item k to land.
    //  * tensors (mode 0): 14 values = 7 aligned words per part, in key order.
    //  * table products (mode 1): the 14 values rel[k] = T[pos + 13 - k] are contiguous in T in reverse
    //    key order, starting at element `pos` of a 128-byte-aligned slice: three 16-byte loads from the
    //    aligned address below it, shifted down by (pos % 8) elements when the item starts.
    uint32_t rawv[2][12];
    const int rev = p.rel_mode != 0;
    const int sh_h = rev ? (qh & 7) : 0, sh_w = rev ? (qw & 7) : 0;
    auto fetch_bias = [&](int it) {
      if (!valid) return;
      if (!rev) {
        const uint32_t* s_h = reinterpret_cast<const uint32_t*>(p.rel_h + ((long long)it * N + n) * WS);
        const uint32_t* s_w = reinterpret_cast<const uint32_t*>(p.rel_w + ((long long)it * N + n) * WS);
#pragma unroll
        for (int q = 0; q < WS / 2; ++q) { rawv[0][q] = __ldg(s_h + q); rawv[1][q] = __ldg(s_w + q); }
      } else {
        const int w = it / p.H, h = it - w * p.H;
        long long trow = (long long)w * N + n;
        if (p.qkv_fused == 2) {                    // raster rows; pad queries of border windows have none
          const int ww = p.nw * p.nw;
          const int b = w / ww, wi = w - b * ww;
          const int wy = wi / p.nw, wx = wi - wy * p.nw;
          const int y = wy * WS + qh, x = wx * WS + qw;
          if (y >= p.grid || x >= p.grid) return;
          trow = ((long long)b * p.grid + y) * p.grid + x;
        }
        const __nv_bfloat16* tb = p.tab + trow * p.ldt + h * p.t_head_stride;
        const uint4* s_h = reinterpret_cast<const uint4*>(tb + (qh - sh_h));
        const uint4* s_w = reinterpret_cast<const uint4*>(tb + p.t_w_off + (qw - sh_w));
#pragma unroll
        for (int q = 0; q < 3; ++q) {
          const uint4 a = __ldg(s_h + q), c = __ldg(s_w + q);
          rawv[0][4 * q] = a.x; rawv[0][4 * q + 1] = a.y; rawv[0][4 * q + 2] = a.z; rawv[0][4 * q + 3] = a.w;
          rawv[1][4 * q] = c.x; rawv[1][4 * q + 1] = c.y; rawv[1][4 * q + 2] = c.z; rawv[1][4 * q + 3] = c.w;
        }
      }
    };
    // element e (0..13) of part x in key order, after undoing the alignment shift and the reversal
    auto bias_elems = [&](int x, int sh, uint32_t (&out)[WS]) {
      uint32_t v[12];
#pragma unroll
      for (int q = 0; q < 12; ++q) v[q] = rawv[x][q];
#pragma unroll
      for (int q = 0; q < 10; ++q) v[q] = (sh & 4) ? v[q + 2] : v[q];      // 4 elements = 2 words
#pragma unroll
      for (int q = 0; q < 9; ++q) v[q] = (sh & 2) ? v[q + 1] : v[q];       // 2 elements = 1 word
#pragma unroll
      for (int q = 0; q < 7; ++q) v[q] = (sh & 1) ? __funnelshift_r(v[q], v[q + 1], 16) : v[q];
#pragma unroll
      for (int e = 0; e < WS; ++e) {
        const int f = WS - 1 - e;
        const uint32_t fwd = (v[e >> 1] >> ((e & 1) * 16)) & 0xffffu, bwd = (v[f >> 1] >> ((f & 1) * 16)) & 0xffffu;
        out[e] = rev ? bwd : fwd;
      }
    };
#pragma unroll
    for (int q = 0; q < 12; ++q) rawv[0][q] = rawv[1][q] = 0u;

    // ---- an item's bias: rel_h (bf16 pairs, kept in registers until the item's softmax), rel_w/scale into the
    // A-operand tile, and for border windows the pad rows of the item's K / V tiles.  `kp` is the item's position in
    // this CTA's sequence (stage and barrier parities follow from it).
    auto prologue = [&](int it_p, uint32_t kp, uint32_t (&bhp)[WS / 2]) -> bool {
      bool good = true;
      // border window (raster layout): this thread's 16-byte piece of the projection bias, requested first
      int vy = WS, vx = WS;
      uint4 bk = make_uint4(0u, 0u, 0u, 0u), bv = bk;
      const int ptid = (warp & 3) * 32 + lane, piece = ptid % (2 * CH);
      const int sweep = (t == 0 ? 128 : 96) / (2 * CH);      // pad rows patched per sweep by the tile's threads
      if (p.qkv_fused == 2) {
        const int w = fdiv(it_p, p.H, p.mH), h = it_p - w * p.H, ww = p.nw * p.nw;
        const int wi = w - fdiv(w, ww, p.mWW) * ww;
        const int wy = fdiv(wi, p.nw, p.mNW), wx = wi - wy * p.nw;
        if (wy == p.nw - 1) vy = p.vlast;
        if (wx == p.nw - 1) vx = p.vlast;
        if ((vy < WS || vx < WS) && ptid < sweep * 2 * CH) {
          bk = __ldg(reinterpret_cast<const uint4*>(p.kv_bias + (size_t)(p.H + h) * D) + piece);
          bv = __ldg(reinterpret_cast<const uint4*>(p.kv_bias + (size_t)(2 * p.H + h) * D) + piece);
        }
      }
      float rw[16];
      if (p.rel_mode == 2) {
        // this row's products with the tables are in columns kTCol.. of the tile (rel_pos_h first, rel_pos_w 32
        // columns on); rounded to bf16 as a stored product tensor would be, so that both sources give the same bits
        good = mbar_wait(&t_full[t], kp & 1u, abort_flag, p.status, 12);
        tc_fence_after();
        uint32_t th[32], tw[32];
        tmem_ld_32x32b_x32(lane_addr + kTCol, th);
        tmem_ld_32x32b_x32(lane_addr + kTCol + 32, tw);
        tmem_ld_wait();
        tc_fence_before();                                       // the next logits product overwrites part of these columns
        float sel[WS];
        select_shifted<WS>(th, qh & 15, sel);
#pragma unroll
        for (int q = 0; q < WS / 2; ++q) bhp[q] = wpack2<kHalf>(sel[2 * q], sel[2 * q + 1]);
        select_shifted<WS>(tw, qw, sel);
        const float inv_s = 1.0f / p.scale;
#pragma unroll
        for (int q = 0; q < 16; ++q) rw[q] = q < WS ? round_bf16(sel[q < WS ? q : 0] * inv_s) : 0.f;
      } else {
        uint32_t eh[WS], ew[WS];
        bias_elems(0, sh_h, eh);
        bias_elems(1, sh_w, ew);
#pragma unroll
        for (int q = 0; q < 16; ++q) rw[q] = q < WS ? bits_to_float<kHalf>(ew[q < WS ? q : 0]) * inv_scale : 0.f;
#pragma unroll
        for (int q = 0; q < WS / 2; ++q) bhp[q] = eh[2 * q] | (eh[2 * q + 1] << 16);
      }
      uint8_t* rrow = smem + L::OFF_RELW + n * 32;
      *reinterpret_cast<uint4*>(rrow + ((0 ^ sw) << 4)) =
          make_uint4(wpack2<kHalf>(rw[0], rw[1]), wpack2<kHalf>(rw[2], rw[3]), wpack2<kHalf>(rw[4], rw[5]), wpack2<kHalf>(rw[6], rw[7]));
      *reinterpret_cast<uint4*>(rrow + ((1 ^ sw) << 4)) =
          make_uint4(wpack2<kHalf>(rw[8], rw[9]), wpack2<kHalf>(rw[10], rw[11]), wpack2<kHalf>(rw[12], rw[13]), wpack2<kHalf>(rw[14], rw[15]));
      if (vy < WS || vx < WS) {
        // border window: pad tokens' K and V rows <- projection bias.  Both tile groups write both (the same
        // values), so neither tile's products depend on the other group's progress.
        good = good && mbar_wait(&full[kp % STAGES], (kp / STAGES) & 1u, abort_flag, p.status, 9);   // the zero fill has landed
        const int n_pad = vy * (WS - vx) + (WS - vy) * WS;
        const uint8_t* tabp = smem + L::OFF_PADTAB + (vy == WS ? 0 : (vx == WS ? 1 : 2)) * 256;
        uint8_t* stage_base = smem + (kp % STAGES) * L::STAGE;
        // thread = one 16-byte piece (of the 2 * CH per row) for every `sweep`-th pad row
        const int c = piece >> 1, hf = piece & 1;
        if (good && ptid < sweep * 2 * CH) {
          for (int pi = ptid / (2 * CH); pi < n_pad; pi += sweep) {
            const int r = tabp[pi];
            const int off = c * L::KV_CHUNK + r * 32 + ((hf ^ ((r >> 2) & 1)) << 4);
            *reinterpret_cast<uint4*>(stage_base + L::OFF_K + off) = bk;
            *reinterpret_cast<uint4*>(stage_base + L::OFF_V + off) = bv;
          }
        }
      }
      fence_proxy_async_smem();
      mbar_arrive_warp(&pro_done[t]);
      return good;
    };

    // Order of work per thread.  Mode 2: softmax of item k, then the bias of item k + 1 (its table products were issued
    // ahead of item k's P V and land while that runs), then item k's output; the logits product of item k + 1 can
    // start as soon as the output accumulator has been read.  Modes 0 / 1 (bias from global memory): the bias of an
    // item at the head of the item, from values requested during the previous item's P V.
    const bool ahead = p.rel_mode == 2;
    int it = blockIdx.x;
    bool ok = true;
    uint32_t bhp[WS / 2];
#pragma unroll
    for (int q = 0; q < WS / 2; ++q) bhp[q] = 0u;
    if (it < p.items) {
      if (!ahead) fetch_bias(it);
      ok = prologue(it, 0u, bhp);
    }
    for (uint32_t k = 0; ok && it < p.items; it += gridDim.x, ++k) {
      const uint32_t par = k & 1u;
      float bh[WS];
#pragma unroll
      for (int q = 0; q < WS / 2; ++q) {
        bh[2 * q] = bits_to_float<kHalf>(bhp[q] & 0xffffu) * kLog2e;
        bh[2 * q + 1] = bits_to_float<kHalf>(bhp[q] >> 16) * kLog2e;
      }
      if (!(ok = mbar_wait(&s_full[t], par, abort_flag, p.status, 6))) break;
      tc_fence_after();
      // pass 1: per key-row maxima of the raw logits, then the row maximum of the biased logits
      float mx[WS];
#pragma unroll
      for (int q = 0; q < WS; ++q) mx[q] = -INFINITY;
      uint32_t rbuf[2][16];
      tmem_ld_32x32b_x16(lane_addr, rbuf[0]);
#pragma unroll
      for (int c = 0; c < NK / 16; ++c) {
        tmem_ld_wait();                                          // chunk c has landed
        if (c + 1 < NK / 16) tmem_ld_32x32b_x16(lane_addr + (c + 1) * 16, rbuf[(c + 1) & 1]);   // next chunk in flight
        const uint32_t(&r)[16] = rbuf[c & 1];
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          const int j = c * 16 + u;
          if (j < N) mx[j / WS] = fmaxf(mx[j / WS], __uint_as_float(r[u]));
        }
      }
      float m = -INFINITY;
#pragma unroll
      for (int q = 0; q < WS; ++q) m = fmaxf(m, fmaf(mx[q], c2, bh[q]));
#pragma unroll
      for (int q = 0; q < WS; ++q) bh[q] -= m;
      // pass 2: probabilities -> packed bf16 P over the logit columns already consumed
      float l = 0.f;
      tmem_ld_32x32b_x16(lane_addr, rbuf[0]);
#pragma unroll
      for (int c = 0; c < NK / 16; ++c) {
        tmem_ld_wait();                                          // chunk c has landed
        if (c + 1 < NK / 16) tmem_ld_32x32b_x16(lane_addr + (c + 1) * 16, rbuf[(c + 1) & 1]);   // next chunk in flight
        const uint32_t(&r)[16] = rbuf[c & 1];
        float e[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          const int j = c * 16 + u;
          e[u] = 0.f;
          if (j < N) {
            e[u] = wexp2(fmaf(__uint_as_float(r[u]), c2, bh[j / WS]));
            l += e[u];
          }
        }
        const uint32_t pk[8] = {wpack2<kHalf>(e[0], e[1]), wpack2<kHalf>(e[2], e[3]), wpack2<kHalf>(e[4], e[5]), wpack2<kHalf>(e[6], e[7]),
                                wpack2<kHalf>(e[8], e[9]), wpack2<kHalf>(e[10], e[11]), wpack2<kHalf>(e[12], e[13]), wpack2<kHalf>(e[14], e[15])};
        // columns [8c, 8c+8) hold logits 16..31 of chunk c/2, consumed in an earlier iteration (for c = 0:
        // chunk 0 itself, already in registers; chunk 1, in flight, starts at column 16)
        tmem_st_32x32b_x8(lane_addr + c * 8, pk);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive_warp(&p_full[t]);
      // The next item's bias values are requested here, where few registers are live: they land during the
      // P V product and the output staging.  (Requested before the softmax they had to be spilled, and the spill
      // waited for the loads.)  Mode 2 picks them from the table products right away.
      const int it_next = it + gridDim.x;
      if (it_next < p.items) {
        if (ahead) ok = prologue(it_next, k + 1u, bhp);
        else fetch_bias(it_next);
      }

      if (!(ok = mbar_wait(&o_full[t], par, abort_flag, p.status, 7))) break;
      tc_fence_after();
      const float inv_l = 1.0f / l;
      uint32_t ro[D / 16][16];
#pragma unroll
      for (int c = 0; c < D / 16; ++c) tmem_ld_32x32b_x16(lane_addr + kOCol + c * 16, ro[c]);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive_warp(&t_free[t]);                              // O is in registers: the tile's columns are free
      // The item's output goes through shared memory (the Q region of this stage is dead once the logits
      // exist) as [token][D] rows and leaves with one TMA store: a WS x WS x D box of the output tensor,
      // which drops the zero-padded tokens of border windows by clipping.
      uint8_t* stg = smem + (k % STAGES) * L::STAGE;
      // the staging rows overlap the other tile's Q rows: its logits product must have read them
      if (!(ok = mbar_wait(&s_done[(t ^ 1) * 2 + par], (k >> 1) & 1u, abort_flag, p.status, 10))) break;
      if (valid) {
#pragma unroll
        for (int c = 0; c < D / 16; ++c) {
          float f[16];
#pragma unroll
          for (int u = 0; u < 16; ++u) f[u] = __uint_as_float(ro[c][u]) * inv_l;
          uint4* dst = reinterpret_cast<uint4*>(stg + n * (D * 2) + c * 32);
          dst[0] = make_uint4(wpack2<kHalf>(f[0], f[1]), wpack2<kHalf>(f[2], f[3]), wpack2<kHalf>(f[4], f[5]), wpack2<kHalf>(f[6], f[7]));
          dst[1] = make_uint4(wpack2<kHalf>(f[8], f[9]), wpack2<kHalf>(f[10], f[11]), wpack2<kHalf>(f[12], f[13]), wpack2<kHalf>(f[14], f[15]));
        }
      }
      fence_proxy_async_smem();
      mbar_arrive_warp(&out_ready[k % STAGES]);                   // the producer thread sends the item's store
      if (!ahead && it_next < p.items) ok = prologue(it_next, k + 1u, bhp);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int D, int WS, bool kHalf = false>
int launch_window(const void* q, const void* k, const void* v, long long rows, long long cols, WinParams p,
                  long long items, void* stream, const void* tables = nullptr) {
  using L = WinSmem<D, WS>;
  CUtensorMap tmQ, tmK, tmV, tmT;
  if (p.qkv_fused == 2) {
    // raster planes [3H * B][grid][grid][D]: one WS x WS box of 16 columns per copy
    const uint64_t g = uint64_t(p.grid);
    const uint64_t dims[4] = {uint64_t(D), g, g, uint64_t(3) * p.H * p.B};
    const uint64_t strides[4] = {2, uint64_t(D) * 2, g * D * 2, g * g * D * 2};
    const uint32_t box[4] = {16, uint32_t(WS), uint32_t(WS), 1};
    if (int e = make_tensor_map(&tmQ, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(q), dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_32B))
      return e;
    tmK = tmV = tmQ;
  } else {
  const uint64_t dims[3] = {16, uint64_t(rows), uint64_t(cols / 16)};
  const uint64_t strides[3] = {2, uint64_t(cols) * 2, 32};
  const uint32_t box_q[3] = {16, uint32_t(L::NK), uint32_t(D / 16)};
  const uint32_t box_kv[3] = {16, uint32_t(L::NK), uint32_t(D / 16)};
  if (int e = make_tensor_map(&tmQ, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box_q,
                              CU_TENSOR_MAP_SWIZZLE_32B))
    return e;
  if (int e = make_tensor_map(&tmK, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(k), dims, strides, box_kv,
                              CU_TENSOR_MAP_SWIZZLE_32B))
    return e;
  if (int e = make_tensor_map(&tmV, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(v), dims, strides, box_kv,
                              CU_TENSOR_MAP_SWIZZLE_32B))
    return e;
  }
  CUtensorMap tmO;
  {
    const uint64_t pitch = uint64_t(p.o_pitch) * 2;
    uint64_t dims[4], strides[4];
    if (p.qkv_fused) {   // o[b][y][x][channels]
      const uint64_t g = uint64_t(p.grid);
      dims[0] = uint64_t(p.H) * D; dims[1] = g; dims[2] = g; dims[3] = uint64_t(items / p.H) / (uint64_t(p.nw) * p.nw);
      strides[0] = 2; strides[1] = pitch; strides[2] = g * pitch; strides[3] = g * g * pitch;
    } else {             // o[item][WS][WS][D]
      dims[0] = D; dims[1] = WS; dims[2] = WS; dims[3] = uint64_t(items);
      strides[0] = 2; strides[1] = pitch; strides[2] = WS * pitch; strides[3] = uint64_t(WS) * WS * pitch;
    }
    const uint32_t box[4] = {uint32_t(D), uint32_t(WS), uint32_t(WS), 1};
    if (int e = make_tensor_map(&tmO, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, p.o, dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_NONE))
      return e;
  }
  tmT = tmQ;
  if (tables != nullptr) {                         // [64 rows][D]: rel_pos_h from row 0, rel_pos_w from row 32
    const uint64_t dims[3] = {16, 64, uint64_t(D / 16)};
    const uint64_t strides[3] = {2, uint64_t(D) * 2, 32};
    const uint32_t box[3] = {16, 64u, uint32_t(D / 16)};
    if (int e = make_tensor_map(&tmT, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(tables), dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_32B))
      return e;
  }
  auto kern = attn_window_kernel<D, WS, kHalf>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::BYTES) != cudaSuccess)
    return SAMB_E_LAUNCH;
  if (items > 0x7fffffffLL) return SAMB_E_SHAPE;
  p.items = int(items);
  p.mH = fdiv_magic(items, p.H);
  p.mWW = fdiv_magic(items, p.nw * p.nw);
  p.mNW = fdiv_magic(items, p.nw);
  const long long grid = items < sm_count() ? items : sm_count();
  kern<<<unsigned(grid), NUM_THREADS, L::BYTES, static_cast<cudaStream_t>(stream)>>>(tmQ, tmK, tmV, tmO, tmT, p);
  return launch_status();
}

}  // namespace
}  // namespace samb

extern "C" {

static int attn_relpos_window_any(bool half, const void* q, const void* k, const void* v, const void* rel_h,
                                  const void* rel_w, void* o, int B, int H, int window, int d, float scale,
                                  int32_t* status, void* stream) {
  using namespace samb;
  if (!q || !k || !v || !rel_h || !rel_w || !o || !status) return SAMB_E_BADARG;
  if (B <= 0 || H <= 0) return SAMB_E_BADARG;
  if (window != 14 || (d != 64 && d != 80)) return SAMB_E_SHAPE;
  const long long rows = (long long)B * H * window * window;
  if (rows > 0x7fffffffLL) return SAMB_E_SHAPE;
  if (reinterpret_cast<uintptr_t>(o) & 15u) return SAMB_E_ALIGN;
  if (int e = check_device_arch()) return e;
  WinParams p{};
  p.rel_h = static_cast<const __nv_bfloat16*>(rel_h);
  p.rel_w = static_cast<const __nv_bfloat16*>(rel_w);
  p.rel_mode = 0;
  p.o = static_cast<__nv_bfloat16*>(o);
  p.o_pitch = d;
  p.qkv_fused = 0;
  p.H = H;
  p.scale = scale;
  p.status = status;
  if (half)
    return d == 80 ? launch_window<80, 14, true>(q, k, v, rows, d, p, (long long)B * H, stream)
                   : launch_window<64, 14, true>(q, k, v, rows, d, p, (long long)B * H, stream);
  return d == 80 ? launch_window<80, 14>(q, k, v, rows, d, p, (long long)B * H, stream)
                 : launch_window<64, 14>(q, k, v, rows, d, p, (long long)B * H, stream);
}

int samb_attn_relpos_window(const void* q, const void* k, const void* v, const void* rel_h, const void* rel_w, void* o,
                            int B, int H, int window, int d, float scale, int32_t* status, void* stream) {
  return attn_relpos_window_any(false, q, k, v, rel_h, rel_w, o, B, H, window, d, scale, status, stream);
}

int samb_attn_relpos_window_f16(const void* q, const void* k, const void* v, const void* rel_h, const void* rel_w,
                                void* o, int B, int H, int window, int d, float scale, int32_t* status, void* stream) {
  return attn_relpos_window_any(true, q, k, v, rel_h, rel_w, o, B, H, window, d, scale, status, stream);
}

int samb_attn_relpos_window_qkv(const void* qkv, const void* tab, int64_t ldt, int t_head_stride, int t_w_off, void* o,
                                int64_t o_pitch, int B, int H, int grid, int window, int d, float scale,
                                int32_t* status, void* stream) {
  using namespace samb;
  if (!qkv || !tab || !o || !status) return SAMB_E_BADARG;
  if (B <= 0 || H <= 0 || grid <= 0) return SAMB_E_BADARG;
  if (window != 14 || (d != 64 && d != 80)) return SAMB_E_SHAPE;
  const int nw = (grid + window - 1) / window;
  const long long W = (long long)B * nw * nw;
  if (3LL * H * W * window * window > 0x7fffffffLL || o_pitch % 8 || o_pitch < (int64_t)H * d) return SAMB_E_SHAPE;
  if (ldt < (int64_t)H * t_head_stride || t_w_off + 2 * window - 1 > t_head_stride || 2 * window - 1 > t_w_off)
    return SAMB_E_SHAPE;
  // the bias prologue reads 16-byte vectors below each needed element and up to the end of a head's slice
  if (ldt % 8 || t_head_stride % 64 || t_w_off % 8 || t_head_stride - t_w_off < 32 || t_w_off < 32) return SAMB_E_SHAPE;
  if ((reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(tab)) & 15u) return SAMB_E_ALIGN;
  if (int e = check_device_arch()) return e;
  WinParams p{};
  p.tab = static_cast<const __nv_bfloat16*>(tab);
  p.ldt = ldt; p.t_head_stride = t_head_stride; p.t_w_off = t_w_off; p.rel_mode = 1;
  p.o = static_cast<__nv_bfloat16*>(o);
  p.o_pitch = o_pitch;
  p.qkv_fused = 1;
  p.H = H; p.grid = grid; p.nw = nw;
  p.scale = scale;
  p.status = status;
  const long long rows = 3LL * H * W * window * window;
  return d == 80 ? launch_window<80, 14>(qkv, qkv, qkv, rows, d, p, W * H, stream)
                 : launch_window<64, 14>(qkv, qkv, qkv, rows, d, p, W * H, stream);
}

int samb_attn_relpos_window_raster(const void* qkv, const void* qkv_bias, const void* tab, int64_t ldt,
                                   int t_head_stride, int t_w_off, void* o, int64_t o_pitch, int B, int H, int grid,
                                   int window, int d, float scale, int32_t* status, void* stream) {
  using namespace samb;
  if (!qkv || !qkv_bias || !tab || !o || !status) return SAMB_E_BADARG;
  if (B <= 0 || H <= 0 || grid <= 0) return SAMB_E_BADARG;
  if (window != 14 || (d != 64 && d != 80)) return SAMB_E_SHAPE;
  const int nw = (grid + window - 1) / window;
  const long long W = (long long)B * nw * nw;
  if (3LL * H * B * grid * grid > 0x7fffffffLL || W * H > 0x7fffffffLL || o_pitch % 8 || o_pitch < (int64_t)H * d)
    return SAMB_E_SHAPE;
  if (ldt < (int64_t)H * t_head_stride || t_w_off + 2 * window - 1 > t_head_stride || 2 * window - 1 > t_w_off)
    return SAMB_E_SHAPE;
  if (ldt % 8 || t_head_stride % 64 || t_w_off % 8 || t_head_stride - t_w_off < 32 || t_w_off < 32) return SAMB_E_SHAPE;
  if ((reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(tab) | reinterpret_cast<uintptr_t>(qkv) |
       reinterpret_cast<uintptr_t>(qkv_bias)) & 15u)
    return SAMB_E_ALIGN;
  if (int e = check_device_arch()) return e;
  WinParams p{};
  p.tab = static_cast<const __nv_bfloat16*>(tab);
  p.ldt = ldt; p.t_head_stride = t_head_stride; p.t_w_off = t_w_off; p.rel_mode = 1;
  p.o = static_cast<__nv_bfloat16*>(o);
  p.o_pitch = o_pitch;
  p.qkv_fused = 2;
  p.H = H; p.grid = grid; p.nw = nw; p.B = B; p.vlast = grid - (nw - 1) * window;
  p.kv_bias = static_cast<const __nv_bfloat16*>(qkv_bias);
  p.scale = scale;
  p.status = status;
  return d == 80 ? launch_window<80, 14>(qkv, qkv, qkv, 0, d, p, W * H, stream)
                 : launch_window<64, 14>(qkv, qkv, qkv, 0, d, p, W * H, stream);
}

int samb_attn_relpos_window_tables(const void* qkv, const void* qkv_bias, const void* tables, void* o, int64_t o_pitch,
                                   int B, int H, int grid, int window, int d, float scale, int32_t* status,
                                   void* stream) {
  using namespace samb;
  if (!qkv || !qkv_bias || !tables || !o || !status) return SAMB_E_BADARG;
  if (B <= 0 || H <= 0 || grid <= 0) return SAMB_E_BADARG;
  if (window != 14 || (d != 64 && d != 80)) return SAMB_E_SHAPE;
  const int nw = (grid + window - 1) / window;
  const long long W = (long long)B * nw * nw;
  if (3LL * H * B * grid * grid > 0x7fffffffLL || W * H > 0x7fffffffLL || o_pitch % 8 || o_pitch < (int64_t)H * d)
    return SAMB_E_SHAPE;
  if ((reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(tables) | reinterpret_cast<uintptr_t>(qkv) |
       reinterpret_cast<uintptr_t>(qkv_bias)) & 15u)
    return SAMB_E_ALIGN;
  if (int e = check_device_arch()) return e;
  WinParams p{};
  p.rel_mode = 2;
  p.o = static_cast<__nv_bfloat16*>(o);
  p.o_pitch = o_pitch;
  p.qkv_fused = 2;
  p.H = H; p.grid = grid; p.nw = nw; p.B = B; p.vlast = grid - (nw - 1) * window;
  p.kv_bias = static_cast<const __nv_bfloat16*>(qkv_bias);
  p.scale = scale;
  p.status = status;
  return d == 80 ? launch_window<80, 14>(qkv, qkv, qkv, 0, d, p, W * H, stream, tables)
                 : launch_window<64, 14>(qkv, qkv, qkv, 0, d, p, W * H, stream, tables);
}

}  // extern "C"
