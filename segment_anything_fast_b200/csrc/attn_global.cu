// Flash attention with the decomposed relative-position bias, for the global blocks
// (keys on an Sh x 64 raster, N = 64*Sh <= 4096 a multiple of 256, head dim d in {64, 80}):
//   O = softmax(scale * Q K^T + rel_h[i, kh(j)] + rel_w[i, kw(j)]) V
//
// One CTA owns 256 query rows (two 128-row tiles A and B) of one (image, head) and walks the keys
// 128 at a time (two raster rows).  Warp 0 feeds K/V tiles through a TMA ring, warp 1 issues
// tcgen05.mma, warps 4..7 run the softmax of tile A and warps 8..11 that of tile B (one thread per
// query row).  While one tile's threads are busy in the exponentials, the tensor core works on the
// other tile's Q K^T / P V, so neither pipe waits on a single chain.
//
// Where the bias goes:
//  * rel_w depends on the key column kw = j % 64, the same pattern in every key tile.  It rides on
//    the tensor core (adding it per element in the softmax threads was measured 20% slower): the A operand is [Q | rel_w/scale] (K = d + 64) and the B operand is
//    [K_tile | E] with E a constant one-hot matrix (E[j, kw(j)] = 1), so Q K^T + rel_w/scale comes
//    out of one accumulation and the softmax multiplies everything by scale.  The rel_w/scale part of A sits in
//    tensor memory (32 columns per tile), E in shared memory as one [128 x 64] block: four products of N = 128
//    per key tile (issuing a tcgen05.mma costs the issuing thread about as much whatever its size).
//  * rel_h depends on the key row kh: two values per query row and key tile.  They are folded into
//    the addend of the exp2 FMA, which costs nothing per element.
// Where the bias comes from: as rel_h / rel_w tensors (mode 0), as table products computed by a separate GEMM
// (mode 1), or (mode 2, what the encoder uses) from the relative-position tables themselves: the CTA multiplies
// its 256 query rows by the [256 x d] table block [rel_pos_h | rel_pos_w] on the tensor core before the key loop
// (two products of N = 256 into the logit / output columns, which are idle then), every thread rounds its row of
// products to bf16 into shared memory (the P buffers, idle as well) and picks its 2 x 64 values
// rel[k] = T[pos + S - 1 - k] from there, so neither the products nor get_rel_pos' gathered tables ever exist
// in global memory.
// Per tile: the 128x128 logits live in one TMEM buffer and are pulled into registers in one pass
// (the buffer is handed back to the tensor core right away); P returns through shared memory in the
// 128B-swizzled K-major layout; O accumulates in TMEM across key tiles.  The running maximum is only
// raised when it would grow by more than 2^8 (probabilities stay below 256, exact enough in fp32 /
// bf16); only then is O rescaled in place, which after the first few key tiles almost never happens.
#include <cuda_fp16.h>

#include "common.cuh"

namespace samb {
namespace {

constexpr int BM = 128;          // query rows per tile
constexpr int BK = 128;          // keys per tile
constexpr int SW = 64;           // raster width the kernel is specialised for
constexpr int KV_STAGES = 2;
constexpr int NUM_THREADS = 384;   // warpgroup 0: TMA + MMA warps (2 idle); warpgroups 1, 2: softmax of tiles A, B
constexpr int TMEM_COLS = 512;   // S_A @0, S_B @128, O_A @256, O_B @384; rel_w/scale (bf16 pairs) A @336, B @464
__host__ __device__ constexpr int relw_col(int t) { return t == 0 ? 336 : 464; }
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;   // log2 domain

struct AttnParams {
  // bias sources: mode 0 = rel_h [BH, N, Sh] / rel_w [BH, N, 64] tensors; mode 1 = table products T[row, ldt]
  const __nv_bfloat16* rel_h;
  const __nv_bfloat16* rel_w;
  const __nv_bfloat16* tab;
  long long ldt;                 // elements per token row of T
  int t_head_stride;             // columns per head in T
  int t_w_off;                   // column offset of the rel_pos_w products inside a head's slice
  int rel_mode;                  // 0 tensors, 1 table products in global memory, 2 products computed by this kernel
  __nv_bfloat16* o;
  long long o_pitch;             // elements between consecutive output rows
  int o_head_stride;             // column offset per head in the output row
  int qkv_fused;                 // 0: q/k/v are [BH*N, d] tensors; 1: one head-major buffer [3H][B*N][d]
  int H, N, Sh;
  float scale;
  int* status;
};

template <int D>
struct Smem {
  static constexpr int CH = D / 16;                 // 16-element (32-byte) column chunks
  static constexpr int Q_CHUNK = 256 * 32;          // 256 query rows of one chunk
  static constexpr int KV_TILE = 128 * 32 * CH;     // one 128-row K or V tile, chunk major
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_E = OFF_Q + CH * Q_CHUNK;            // [128][64] bf16 one-hot (key j -> column j % 64), 128B swizzle
  static constexpr int OFF_P = OFF_E + 128 * 128;               // 2 tiles x 2 x [128][64] bf16, 128B swizzle
  static constexpr int OFF_KV = OFF_P + 2 * 2 * 128 * 128;      // ring of (K tile, V tile)
  static constexpr int OFF_BAR = OFF_KV + KV_STAGES * 2 * KV_TILE;
  static constexpr int BYTES = OFF_BAR + 256 + 1024;
};

__device__ __forceinline__ uint32_t bfpack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// Two 16-bit elements of the tensors' type (bfloat16, or float16 when kHalf) in one word.
template <bool kHalf>
__device__ __forceinline__ uint32_t pack_pair(float lo, float hi) {
  if constexpr (kHalf) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    return bfpack2(lo, hi);
  }
}
template <bool kHalf>
__device__ __forceinline__ float2 unpack_pair(uint32_t w) {
  if constexpr (kHalf) return __half22float2(*reinterpret_cast<const __half2*>(&w));
  else return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// kHalf: q, k, v, the bias tensors and the output are float16 instead of bfloat16 (bias tensors only: the table
// modes belong to the bf16 encoder).  Logits, softmax statistics and the output accumulator are fp32 either way.
template <int D, bool kHalf>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_global_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmT,
                   const AttnParams p) {
  using L = Smem<D>;
  constexpr int CH = L::CH;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* q_full = bars + 0;
  uint64_t* pro_done = bars + 1;
  uint64_t* k_full = bars + 2;                  // [KV_STAGES] K and V tiles travel through separate rings:
  uint64_t* k_empty = k_full + KV_STAGES;       //   a K tile is free as soon as both Q K^T products have
  uint64_t* v_full = k_empty + KV_STAGES;       //   read it, a V tile one key tile later, so the next K
  uint64_t* v_empty = v_full + KV_STAGES;       //   load gets a whole key tile of lead time
  uint64_t* s_full = v_empty + KV_STAGES;       // [2] logits of tile t are in TMEM
  uint64_t* s_free = s_full + 2;                // [2] tile t's threads hold the logits in registers
  uint64_t* p_full = s_free + 2;                // [2] P of tile t is in shared memory (and O rescaled)
  uint64_t* pv_done = p_full + 2;               // [2] P V of tile t finished: P buffer free, O stable
  uint64_t* t_full = pv_done + 2;               // mode 2: both tiles' table products are in TMEM
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(t_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles_q = p.N / (2 * BM);
  const int bh = blockIdx.x / n_tiles_q;
  const int n0 = (blockIdx.x - bh * n_tiles_q) * (2 * BM);
  const int b = bh / p.H, h = bh - b * p.H;
  const int nblk = p.N / BK;

  // rows of token 0 of this (image, head) in the q, k, v operands.  Head-major qkv buffer: planes
  // [q heads | k heads | v heads], each [B*N, d]; separate tensors: [B*H*N, d] each.
  int rq, rk, rv;
  if (p.qkv_fused) {
    const int R = (gridDim.x / (p.H * n_tiles_q)) * p.N;     // rows per plane = B*N
    rq = h * R + b * p.N;
    rk = (p.H + h) * R + b * p.N;
    rv = (2 * p.H + h) * R + b * p.N;
  } else {
    rq = rk = rv = bh * p.N;
  }

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    mbar_init(t_full, 1);
    mbar_init(pro_done, 8);                     // one arrival per softmax warp
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&s_full[t], 1); mbar_init(&s_free[t], 4);
      mbar_init(&p_full[t], 4); mbar_init(&pv_done[t], 1);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
    if (p.rel_mode == 2) tma_prefetch_desc(&tmT);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Register budget: the launch gives every thread 168; the data-movement warpgroup hands most of its
  // share to the two softmax warpgroups, which hold a whole 128-wide logit row per thread.
  if (warp < 4) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 104;");
  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      mbar_expect_tx(q_full, (p.rel_mode == 2 ? 2 : 1) * CH * L::Q_CHUNK);
      tma_load_3d(smem + L::OFF_Q, &tmQ, q_full, 0, rq + n0, 0);
      // the [256 x d] table block, laid out like a 256-row Q block, parked in the (still idle) P buffers
      if (p.rel_mode == 2) tma_load_3d(smem + L::OFF_P, &tmT, q_full, 0, 0, 0);
      uint32_t stage = 0, phase = 0;
      for (int j = 0; j < nblk; ++j) {
        uint8_t* sk = smem + L::OFF_KV + stage * 2 * L::KV_TILE;
        if (!mbar_wait(&k_empty[stage], phase ^ 1u, abort_flag, p.status, 1)) break;
        mbar_expect_tx(&k_full[stage], L::KV_TILE);
        tma_load_3d(sk, &tmK, &k_full[stage], 0, rk + j * BK, 0);
        if (!mbar_wait(&v_empty[stage], phase ^ 1u, abort_flag, p.status, 11)) break;
        mbar_expect_tx(&v_full[stage], L::KV_TILE);
        tma_load_3d(sk + L::KV_TILE, &tmV, &v_full[stage], 0, rv + j * BK, 0);
        if (++stage == KV_STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    // The whole warp runs the loop (warp-uniform control flow and descriptors); one elected lane
    // issues the tensor-core instructions and their commits.
    {
      constexpr uint32_t kFmt = kHalf ? kFmtF16 : kFmtBF16;
      constexpr uint32_t idesc_s = make_idesc(kAccF32, kFmt, kFmt, BM, BK);
      constexpr uint32_t idesc_o = make_idesc(kAccF32, kFmt, kFmt, BM, D, false, /*B MN-major*/ true);
      // Base descriptors; the start-address field counts 16-byte units, so "+ bytes / 16" moves a tile.
      const uint64_t dq = make_smem_desc(smem_u32(smem + L::OFF_Q), 16, 256, kSwizzle32B);        // K-major, 32B swizzle
      const uint64_t dk = make_smem_desc(smem_u32(smem + L::OFF_KV), 16, 256, kSwizzle32B);
      const uint64_t de = make_smem_desc(smem_u32(smem + L::OFF_E), 16, 1024, kSwizzle128B);
      const uint64_t dp = make_smem_desc(smem_u32(smem + L::OFF_P), 16, 1024, kSwizzle128B);
      // V: MN-major 32B swizzle, column chunks 4096 B apart (LBO), 8-key groups 256 B apart (SBO)
      const uint64_t dv = make_smem_desc(smem_u32(smem + L::OFF_KV + L::KV_TILE), 4096, 256, kSwizzle32B);
      constexpr uint32_t kStageUnits = 2 * L::KV_TILE / 16;
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, 2);
      if (ok && p.rel_mode == 2) {
        // T_t = Q_t * [rel_pos_h | rel_pos_w]^T, N = 256: tile A into columns 0..255, tile B into 256..511
        tc_fence_after();
        if (elect_one()) {
          constexpr uint32_t idesc_t = make_idesc(kAccF32, kFmtBF16, kFmtBF16, BM, 256);
          const uint64_t dt = make_smem_desc(smem_u32(smem + L::OFF_P), 16, 256, kSwizzle32B);
#pragma unroll
          for (int t = 0; t < 2; ++t)
#pragma unroll
            for (int c = 0; c < CH; ++c)
              umma_f16_ss(tmem_base + t * 256, dq + t * (4096 / 16) + c * (L::Q_CHUNK / 16), dt + c * (L::Q_CHUNK / 16),
                          idesc_t, c != 0);
          tc_commit(t_full);
        }
        __syncwarp();
      }
      ok = ok && mbar_wait(pro_done, 0, abort_flag, p.status, 3);

      auto issue_s = [&](int t, int j) {         // S_t = [Q_t | relw_t] * [K_j | E]^T
        if (elect_one()) {
          const uint32_t d_tmem = tmem_base + t * 128;
          const uint64_t dkj = dk + uint32_t(j % KV_STAGES) * kStageUnits;
          const uint64_t dqt = dq + t * (4096 / 16);
#pragma unroll
          for (int c = 0; c < CH; ++c)
            umma_f16_ss(d_tmem, dqt + c * (L::Q_CHUNK / 16), dkj + c * (4096 / 16), idesc_s, c != 0);
#pragma unroll
          for (int c = 0; c < 4; ++c)            // + (rel_w/scale)[128 x 64] (from tensor memory) * E^T: 16 columns per product
            umma_f16_ts(d_tmem, tmem_base + relw_col(t) + c * 8, de + c * 2, idesc_s, 1u);
          tc_commit(&s_full[t]);
        }
        __syncwarp();
      };

      // Event-driven issue: each tile advances on its own (logits of key tile js[t], P V of key tile
      // jp[t]) as soon as its operands are ready, so a tile that is still in its exponentials never
      // holds up the other tile's products.  Every condition is polled without blocking; the idle
      // poll count is bounded.
      int js[2] = {0, 0}, jp[2] = {0, 0};
      int k_released = 0, v_released = 0;        // key tiles whose K / V buffers have been handed back
      uint32_t idle = 0;
      while (ok && (jp[0] < nblk || jp[1] < nblk)) {
        bool progress = false;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          const int j = js[t];
          if (j < nblk && mbar_test_wait(&k_full[j % KV_STAGES], uint32_t(j / KV_STAGES) & 1u) &&
              (j == 0 || mbar_test_wait(&s_free[t], uint32_t(j - 1) & 1u))) {
            tc_fence_after();
            issue_s(t, j);
            js[t] = j + 1;
            progress = true;
          }
          const int jv = jp[t];
          if (jv < nblk && jv < js[t] && mbar_test_wait(&p_full[t], uint32_t(jv) & 1u) &&
              mbar_test_wait(&v_full[jv % KV_STAGES], uint32_t(jv / KV_STAGES) & 1u)) {
            tc_fence_after();
            if (elect_one()) {
              const uint64_t dvj = dv + uint32_t(jv % KV_STAGES) * kStageUnits;
              const uint64_t dpt = dp + t * (32768 / 16);
              const uint32_t d_tmem = tmem_base + 256 + t * 128;
#pragma unroll
              for (int kk = 0; kk < BK / 16; ++kk)   // 16 keys per step: 32 B of a P row, 512 B of V
                umma_f16_ss(d_tmem, dpt + (kk >> 2) * (16384 / 16) + (kk & 3) * 2, dvj + kk * (512 / 16), idesc_o,
                            (jv | kk) != 0);
              tc_commit(&pv_done[t]);
            }
            __syncwarp();
            jp[t] = jv + 1;
            progress = true;
          }
        }
        // hand buffers back once both tiles have issued everything that reads them
        const int s_min = js[0] < js[1] ? js[0] : js[1];
        const int p_min = jp[0] < jp[1] ? jp[0] : jp[1];
        while (k_released < s_min) {
          if (elect_one()) tc_commit(&k_empty[k_released % KV_STAGES]);
          __syncwarp();
          ++k_released;
        }
        while (v_released < p_min) {
          if (elect_one()) tc_commit(&v_empty[v_released % KV_STAGES]);
          __syncwarp();
          ++v_released;
        }
        if (progress) {
          idle = 0;
        } else if (++idle > kSpinLimit || (idle > 2048u && *abort_flag)) {
          *abort_flag = 1;
          if (p.status != nullptr) atomicCAS(p.status, 0, int((kDevTimeout << 24) | (13u << 16) | (blockIdx.x & 0xffffu)));
          ok = false;
        } else if (idle > 4096u) {
          __nanosleep(32);
        }
      }
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 200;");
    // ---------------------------------------------------------------- softmax (one thread = one row)
    const int t = (warp - 4) >> 2;                         // query tile
    const int i = (warp & 3) * 32 + lane;                  // row in the tile == TMEM lane
    const uint32_t lane_addr = tmem_base + (uint32_t((warp & 3) * 32) << 16);
    const int n = n0 + t * BM + i;                         // token index inside the image
    const int qh = n / SW, qw = n - qh * SW;
    // rel_w tensors are divided by scale here; table products arrive already divided
    const float inv_scale = p.rel_mode == 0 ? 1.0f / p.scale : 1.0f;
    // ---- prologue: this row's bias values, fetched with 16-byte loads.
    //  * tensors (mode 0): rel_h [Sh] and rel_w [64] rows, in key order.
    //  * table products (mode 1): rel[k] = T[pos + S - 1 - k] is contiguous in T in reverse key order starting
    //    at element `pos` (qh resp. qw) of a 128-byte-aligned slice: load from the aligned address below,
    //    shift down by pos % 8 elements, read backwards.
    // rel_w/scale goes to tensor memory as the A operand of the one-hot products; rel_h stays in a per-thread array indexed by the key
    // tile at run time (local memory: one coalesced word per thread and key tile).
    uint32_t relh_loc[32];                                 // word j = (rel_h[2j], rel_h[2j+1]) as bf16 bits
    {
      const int rev = p.rel_mode != 0;
      auto load_row = [&](const __nv_bfloat16* base, int pos, int count, uint32_t (&out)[32]) {
        // out[e >> 1] halves e = 0..count-1 in key order (count <= 64, multiple of 2)
        uint32_t v[36];
        const int sh = rev ? (pos & 7) : 0;
        const uint4* src = reinterpret_cast<const uint4*>(base + (rev ? pos - sh : 0));
        const int nvec = rev ? (count + 8 + 7) / 8 : count / 8;
        if (!rev && (count & 7)) {                       // short rel_h rows (small rasters): plain 4-byte loads
          const uint32_t* s32 = reinterpret_cast<const uint32_t*>(base);
#pragma unroll
          for (int q = 0; q < 36; ++q) v[q] = q < count / 2 ? __ldg(s32 + q) : 0u;
        } else {
#pragma unroll
          for (int q = 0; q < 9; ++q) {
            uint4 a = make_uint4(0u, 0u, 0u, 0u);
            if (q < nvec) a = __ldg(src + q);
            v[4 * q] = a.x; v[4 * q + 1] = a.y; v[4 * q + 2] = a.z; v[4 * q + 3] = a.w;
          }
        }
#pragma unroll
        for (int q = 0; q < 34; ++q) v[q] = (sh & 4) ? v[q + 2] : v[q];
#pragma unroll
        for (int q = 0; q < 33; ++q) v[q] = (sh & 2) ? v[q + 1] : v[q];
#pragma unroll
        for (int q = 0; q < 32; ++q) v[q] = (sh & 1) ? __funnelshift_r(v[q], v[q + 1], 16) : v[q];
        // key order: forward as is; reversed: element e = v-element (count - 1 - e), i.e. swap halves and words
#pragma unroll
        for (int q = 0; q < 32; ++q) {
          const int qq = count / 2 - 1 - q;
          const uint32_t r = v[qq >= 0 ? qq : 0];
          out[q] = rev ? ((r >> 16) | (r << 16)) : v[q];
        }
      };
      const __nv_bfloat16 *base_h, *base_w;
      if (p.rel_mode == 2) {
        base_h = base_w = nullptr;
      } else if (!rev) {
        base_h = p.rel_h + ((long long)bh * p.N + n) * p.Sh;
        base_w = p.rel_w + ((long long)bh * p.N + n) * SW;
      } else {
        base_h = p.tab + ((long long)b * p.N + n) * p.ldt + h * p.t_head_stride;
        base_w = base_h + p.t_w_off;
      }
      uint32_t rw[32];
      if (p.rel_mode == 2) {
        // This row's 256 products sit in TMEM (tile A: columns 0..255, tile B: 256..511).  One half at a time
        // (rel_pos_h, then rel_pos_w divided by scale): round to bf16, park the 128 values in this row's 256 bytes
        // of its tile's P buffer (16-byte units XOR-swizzled by the row, so a warp's stores spread over the banks),
        // and read rel[k] = T[pos + S - 1 - k] back two bytes at a time.
        bool got = mbar_wait(t_full, 0, abort_flag, p.status, 12);
        tc_fence_after();
        uint8_t* srow = smem + L::OFF_P + (t * BM + i) * 256;
        const float inv_s = 1.0f / p.scale;
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
          uint32_t tv[128];
          const uint32_t ta = lane_addr + t * 256 + half * 128;
          tmem_ld_32x32b_x32(ta, *reinterpret_cast<uint32_t(*)[32]>(&tv[0]));
          tmem_ld_32x32b_x32(ta + 32, *reinterpret_cast<uint32_t(*)[32]>(&tv[32]));
          tmem_ld_32x32b_x32(ta + 64, *reinterpret_cast<uint32_t(*)[32]>(&tv[64]));
          tmem_ld_32x32b_x32(ta + 96, *reinterpret_cast<uint32_t(*)[32]>(&tv[96]));
          tmem_ld_wait();
          const float mul = half ? inv_s : 1.0f;
#pragma unroll
          for (int u = 0; u < 16; ++u) {
            uint32_t w4[4];
#pragma unroll
            for (int q = 0; q < 4; ++q)
              w4[q] = bfpack2(__uint_as_float(tv[u * 8 + 2 * q]) * mul, __uint_as_float(tv[u * 8 + 2 * q + 1]) * mul);
            *reinterpret_cast<uint4*>(srow + ((u ^ (i & 15)) << 4)) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
          }
          const int pos = half ? qw : qh, count = half ? SW : p.Sh;
          auto elem = [&](int k) -> uint32_t {            // rel[k], k < count, as bf16 bits
            const int e = pos + count - 1 - k;
            return *reinterpret_cast<const uint16_t*>(srow + (((e >> 3) ^ (i & 15)) << 4) + (e & 7) * 2);
          };
#pragma unroll
          for (int q = 0; q < 32; ++q) {
            uint32_t w = 0u;
            if (2 * q < count && got) w = elem(2 * q) | (elem(2 * q + 1) << 16);
            if (half) rw[q] = w;
            else relh_loc[q] = w;
          }
        }
        // tile A's rel_w operand columns (336..) lie inside tile B's product columns: nobody stores to tensor
        // memory before every softmax thread has read its products
        tc_fence_before();
        asm volatile("bar.sync 1, 256;" ::: "memory");
        tc_fence_after();
      } else {
      load_row(base_w, qw, SW, rw);
      load_row(base_h, qh, p.Sh, relh_loc);
      }
      uint8_t* e_row = smem + L::OFF_E + i * 128;
      uint32_t wpk[32];                                    // (rel_w[2k], rel_w[2k+1]) / scale as bf16 pairs: the A operand row
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        uint32_t e[4];
#pragma unroll
        for (int tt = 0; tt < 4; ++tt) {
          const int k0 = u * 8 + 2 * tt;
          const uint32_t pr = rw[u * 4 + tt];
          const float2 prf = unpack_pair<kHalf>(pr);
          wpk[u * 4 + tt] = pack_pair<kHalf>(prf.x * inv_scale, prf.y * inv_scale);
          constexpr uint32_t kOne = kHalf ? 0x3C00u : 0x3F80u;            // 1.0 in the operands' type
          e[tt] = ((i & 63) == k0 ? kOne : 0u) | ((i & 63) == k0 + 1 ? (kOne << 16) : 0u);
        }
        const int phys = (u ^ (i & 7)) << 4;
        if (t == 0) *reinterpret_cast<uint4*>(e_row + phys) = make_uint4(e[0], e[1], e[2], e[3]);
      }
      tmem_st_32x32b_x16(lane_addr + relw_col(t), *reinterpret_cast<uint32_t(*)[16]>(&wpk[0]));
      tmem_st_32x32b_x16(lane_addr + relw_col(t) + 16, *reinterpret_cast<uint32_t(*)[16]>(&wpk[16]));
      tmem_st_wait();
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive_warp(pro_done);
    }
    const float c2 = p.scale * kLog2e;
    float m_used = -INFINITY, l_run = 0.f;
    const uint32_t s_addr = lane_addr + t * 128;
    const uint32_t o_addr = lane_addr + 256 + t * 128;
    uint8_t* p_tile = smem + L::OFF_P + t * 32768 + i * 128;
    bool ok = true;

    for (int j = 0; j < nblk; ++j) {
      const uint32_t par = uint32_t(j) & 1u;
      // rel_h of this key tile's two raster rows
      const uint32_t hpair = relh_loc[j];
      const float2 hpf = unpack_pair<kHalf>(hpair);
      const float bh0 = hpf.x * kLog2e, bh1 = hpf.y * kLog2e;
      if (!(ok = mbar_wait(&s_full[t], par, abort_flag, p.status, 8))) break;
      tc_fence_after();
      uint32_t s[128];
      tmem_ld_32x32b_x32(s_addr, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
      tmem_ld_32x32b_x32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
      tmem_ld_32x32b_x32(s_addr + 64, *reinterpret_cast<uint32_t(*)[32]>(&s[64]));
      tmem_ld_32x32b_x32(s_addr + 96, *reinterpret_cast<uint32_t(*)[32]>(&s[96]));
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive_warp(&s_free[t]);                              // the tensor core may overwrite the logits
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int c = 0; c < 64; ++c) {
        mx0 = fmaxf(mx0, __uint_as_float(s[c]));
        mx1 = fmaxf(mx1, __uint_as_float(s[64 + c]));
      }
      const float m_blk = fmaxf(fmaf(mx0, c2, bh0), fmaf(mx1, c2, bh1));
      // P V of the previous key tile must be done: the P buffer is free and O is stable
      if (!(ok = mbar_wait(&pv_done[t], par ^ 1u, abort_flag, p.status, 9))) break;
      if (j == 0) {
        m_used = m_blk;
      } else if (__any_sync(0xffffffffu, m_blk > m_used + kRescaleThreshold)) {
        const float m_new = fmaxf(m_used, m_blk);
        const float alpha = fast_exp2(m_used - m_new);
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < D / 16; ++c) {
          uint32_t r[16];
          tmem_ld_32x32b_x16(o_addr + c * 16, r);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 16; ++q) r[q] = __float_as_uint(__uint_as_float(r[q]) * alpha);
          tmem_st_32x32b_x16(o_addr + c * 16, r);
        }
        tmem_st_wait();
        l_run *= alpha;
        m_used = m_new;
      }
      const float add0 = bh0 - m_used, add1 = bh1 - m_used;
      float l_blk = 0.f;
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        float e[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          e[q] = fast_exp2(fmaf(__uint_as_float(s[u * 8 + q]), c2, u < 8 ? add0 : add1));
          l_blk += e[q];
        }
        *reinterpret_cast<uint4*>(p_tile + (u >> 3) * 16384 + (((u & 7) ^ (i & 7)) << 4)) =
            make_uint4(pack_pair<kHalf>(e[0], e[1]), pack_pair<kHalf>(e[2], e[3]), pack_pair<kHalf>(e[4], e[5]),
                       pack_pair<kHalf>(e[6], e[7]));
      }
      l_run += l_blk;
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive_warp(&p_full[t]);
    }
    if (ok) ok = mbar_wait(&pv_done[t], uint32_t(nblk - 1) & 1u, abort_flag, p.status, 10);
    if (ok) {
      tc_fence_after();
      const float inv_l = 1.0f / l_run;
      __nv_bfloat16* orow = p.qkv_fused ? p.o + ((long long)b * p.N + n) * p.o_pitch + h * p.o_head_stride
                                        : p.o + ((long long)bh * p.N + n) * p.o_pitch;
#pragma unroll
      for (int c = 0; c < D / 16; ++c) {
        uint32_t r[16];
        tmem_ld_32x32b_x16(o_addr + c * 16, r);
        tmem_ld_wait();
        float f[16];
#pragma unroll
        for (int q = 0; q < 16; ++q) f[q] = __uint_as_float(r[q]) * inv_l;
        *reinterpret_cast<uint4*>(orow + c * 16) =
            make_uint4(pack_pair<kHalf>(f[0], f[1]), pack_pair<kHalf>(f[2], f[3]), pack_pair<kHalf>(f[4], f[5]),
                       pack_pair<kHalf>(f[6], f[7]));
        *reinterpret_cast<uint4*>(orow + c * 16 + 8) =
            make_uint4(pack_pair<kHalf>(f[8], f[9]), pack_pair<kHalf>(f[10], f[11]), pack_pair<kHalf>(f[12], f[13]),
                       pack_pair<kHalf>(f[14], f[15]));
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int D, bool kHalf = false>
int launch_d(const void* q, const void* k, const void* v, long long rows, long long cols, long long pitch_elems,
             const AttnParams& p, int BH, void* stream, const void* tables = nullptr) {
  CUtensorMap tm[4];
  const void* base[3] = {q, k, v};
  for (int t = 0; t < 3; ++t) {
    const uint64_t dims[3] = {16, uint64_t(rows), uint64_t(cols / 16)};
    const uint64_t strides[3] = {2, uint64_t(pitch_elems) * 2, 32};
    const uint32_t box[3] = {16, t == 0 ? 256u : 128u, uint32_t(D / 16)};
    if (int e = make_tensor_map(&tm[t], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base[t]), dims, strides,
                                box, CU_TENSOR_MAP_SWIZZLE_32B))
      return e;
  }
  tm[3] = tm[0];
  if (tables != nullptr) {                       // [256 rows][D] table block, fetched like a 256-row Q block
    const uint64_t dims[3] = {16, 256, uint64_t(D / 16)};
    const uint64_t strides[3] = {2, uint64_t(D) * 2, 32};
    const uint32_t box[3] = {16, 256u, uint32_t(D / 16)};
    if (int e = make_tensor_map(&tm[3], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(tables), dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_32B))
      return e;
  }
  auto kern = attn_global_kernel<D, kHalf>;   // the copies move 2-byte elements: one tensor-map type serves both
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<D>::BYTES) != cudaSuccess)
    return SAMB_E_LAUNCH;
  const long long grid = (long long)BH * (p.N / (2 * BM));
  if (grid > 0x7fffffffLL) return SAMB_E_SHAPE;
  kern<<<unsigned(grid), NUM_THREADS, Smem<D>::BYTES, static_cast<cudaStream_t>(stream)>>>(tm[0], tm[1], tm[2], tm[3], p);
  return launch_status();
}

}  // namespace
}  // namespace samb

extern "C" {

static int attn_relpos_global_any(bool half, const void* q, const void* k, const void* v, const void* rel_h,
                                  const void* rel_w, void* o, int B, int H, int N, int d, float scale, int32_t* status,
                                  void* stream) {
  using namespace samb;
  if (!q || !k || !v || !rel_h || !rel_w || !o || !status) return SAMB_E_BADARG;
  if (B <= 0 || H <= 0 || N <= 0) return SAMB_E_BADARG;
  if ((d != 64 && d != 80) || N % 256 || N > 4096) return SAMB_E_SHAPE;
  if ((long long)B * H * N > 0x7fffffffLL) return SAMB_E_SHAPE;
  if ((reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(rel_h) | reinterpret_cast<uintptr_t>(rel_w)) & 15u)
    return SAMB_E_ALIGN;
  if (int e = check_device_arch()) return e;
  AttnParams p{};
  p.rel_h = static_cast<const __nv_bfloat16*>(rel_h);
  p.rel_w = static_cast<const __nv_bfloat16*>(rel_w);
  p.rel_mode = 0;
  p.o = static_cast<__nv_bfloat16*>(o);
  p.o_pitch = d;
  p.o_head_stride = 0;
  p.qkv_fused = 0;
  p.H = H; p.N = N; p.Sh = N / 64;
  p.scale = scale;
  p.status = status;
  const long long rows = (long long)B * H * N;
  if (half)
    return d == 80 ? launch_d<80, true>(q, k, v, rows, d, d, p, B * H, stream)
                   : launch_d<64, true>(q, k, v, rows, d, d, p, B * H, stream);
  return d == 80 ? launch_d<80>(q, k, v, rows, d, d, p, B * H, stream) : launch_d<64>(q, k, v, rows, d, d, p, B * H, stream);
}

int samb_attn_relpos_global(const void* q, const void* k, const void* v, const void* rel_h, const void* rel_w,
                            void* o, int B, int H, int N, int d, float scale, int32_t* status, void* stream) {
  return attn_relpos_global_any(false, q, k, v, rel_h, rel_w, o, B, H, N, d, scale, status, stream);
}

int samb_attn_relpos_global_f16(const void* q, const void* k, const void* v, const void* rel_h, const void* rel_w,
                                void* o, int B, int H, int N, int d, float scale, int32_t* status, void* stream) {
  return attn_relpos_global_any(true, q, k, v, rel_h, rel_w, o, B, H, N, d, scale, status, stream);
}

int samb_attn_relpos_global_qkv(const void* qkv, const void* tab, int64_t ldt, int t_head_stride, int t_w_off, void* o,
                                int64_t o_pitch, int B, int H, int N, int d, float scale, int32_t* status,
                                void* stream) {
  using namespace samb;
  if (!qkv || !tab || !o || !status) return SAMB_E_BADARG;
  if (B <= 0 || H <= 0 || N <= 0) return SAMB_E_BADARG;
  if ((d != 64 && d != 80) || N % 256 || N > 4096) return SAMB_E_SHAPE;
  if (3LL * H * B * N > 0x7fffffffLL || o_pitch % 8 || o_pitch < (int64_t)H * d) return SAMB_E_SHAPE;
  if (ldt < (int64_t)H * t_head_stride || t_w_off + 127 > t_head_stride || N / 64 * 2 - 1 > t_w_off) return SAMB_E_SHAPE;
  // the bias prologue reads 16-byte vectors from 128-byte-aligned slices: [0, 128) and [t_w_off, t_w_off + 128)
  if (ldt % 64 || t_head_stride % 64 || t_w_off % 64 || t_w_off < 128 || t_head_stride - t_w_off < 128) return SAMB_E_SHAPE;
  if ((reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(tab)) & 15u) return SAMB_E_ALIGN;
  if (int e = check_device_arch()) return e;
  AttnParams p{};
  p.tab = static_cast<const __nv_bfloat16*>(tab);
  p.ldt = ldt;
  p.t_head_stride = t_head_stride;
  p.t_w_off = t_w_off;
  p.rel_mode = 1;
  p.o = static_cast<__nv_bfloat16*>(o);
  p.o_pitch = o_pitch;
  p.o_head_stride = d;
  p.qkv_fused = 1;
  p.H = H; p.N = N; p.Sh = N / 64;
  p.scale = scale;
  p.status = status;
  const long long rows = 3LL * H * B * N;
  return d == 80 ? launch_d<80>(qkv, qkv, qkv, rows, d, d, p, B * H, stream)
                 : launch_d<64>(qkv, qkv, qkv, rows, d, d, p, B * H, stream);
}

int samb_attn_relpos_global_tables(const void* qkv, const void* tables, void* o, int64_t o_pitch, int B, int H, int N,
                                   int d, float scale, int32_t* status, void* stream) {
  using namespace samb;
  if (!qkv || !tables || !o || !status) return SAMB_E_BADARG;
  if (B <= 0 || H <= 0 || N <= 0) return SAMB_E_BADARG;
  if ((d != 64 && d != 80) || N % 256 || N > 4096) return SAMB_E_SHAPE;
  if (3LL * H * B * N > 0x7fffffffLL || o_pitch % 8 || o_pitch < (int64_t)H * d) return SAMB_E_SHAPE;
  if ((reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(tables) | reinterpret_cast<uintptr_t>(qkv)) & 15u)
    return SAMB_E_ALIGN;
  if (int e = check_device_arch()) return e;
  AttnParams p{};
  p.rel_mode = 2;
  p.o = static_cast<__nv_bfloat16*>(o);
  p.o_pitch = o_pitch;
  p.o_head_stride = d;
  p.qkv_fused = 1;
  p.H = H; p.N = N; p.Sh = N / 64;
  p.scale = scale;
  p.status = status;
  const long long rows = 3LL * H * B * N;
  return d == 80 ? launch_d<80>(qkv, qkv, qkv, rows, d, d, p, B * H, stream, tables)
                 : launch_d<64>(qkv, qkv, qkv, rows, d, d, p, B * H, stream, tables);
}

}  // extern "C"
