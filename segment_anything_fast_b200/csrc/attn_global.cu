// Flash attention with the decomposed relative-position bias, for the global blocks
// (keys on an Sh x 64 raster, N = 64*Sh <= 4096, head dim d in {64, 80}):
//   O = softmax(scale * Q K^T + rel_h[i, kh(j)] + rel_w[i, kw(j)]) V
//
// One CTA owns 128 query rows of one (image, head) and walks the keys 128 at a time (two raster
// rows).  Warp 0 feeds K/V tiles through a 3-deep TMA ring, warp 1 issues tcgen05.mma, warps 2..5
// (one thread per query row) run the online softmax out of tensor memory.
//
// Where the bias goes:
//  * rel_w depends on the key column kw = j % 64, the same pattern in every key tile.  It rides on
//    the tensor core: the A operand is [Q | rel_w/scale] (K = d + 64) and the B operand is
//    [K_tile | E] with E a constant one-hot matrix (E[j, kw(j)] = 1), so Q K^T + rel_w/scale comes
//    out of one accumulation and the softmax multiplies everything by scale.
//  * rel_h depends on the key row kh: two values per query row and key tile.  They are folded into
//    the addend of the exp2 FMA, which costs nothing per element.
// The 128x128 logits live in two TMEM buffers (QK^T of tile j+1 overlaps the softmax of tile j), P
// goes back to the tensor core through shared memory in the 128B-swizzled K-major layout, P V lands
// in a fresh TMEM buffer per tile and is folded into fp32 register accumulators with the usual
// running-max rescale.
#include "common.cuh"

namespace samb {
namespace {

constexpr int BM = 128;          // query rows per CTA
constexpr int BK = 128;          // keys per tile
constexpr int SW = 64;           // raster width the kernel is specialised for
constexpr int KV_STAGES = 3;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;   // S0 @0, S1 @128, O0 @256, O1 @384
constexpr float kLog2e = 1.4426950408889634f;

struct AttnParams {
  // bias sources: mode 0 = rel_h/rel_w tensors [BH, N, 64]; mode 1 = table products T[row, ldt]
  const __nv_bfloat16* rel_h;
  const __nv_bfloat16* rel_w;
  const __nv_bfloat16* tab;
  long long ldt;                 // elements per token row of T
  int t_head_stride;             // columns per head in T
  int t_w_off;                   // column offset of the rel_pos_w products inside a head's slice
  int rel_mode;
  __nv_bfloat16* o;
  long long o_pitch;             // elements between consecutive output rows
  int o_head_stride;             // column offset per head in the output row
  int qkv_fused;                 // 0: q/k/v are [BH*N, d]; 1: [B*N, 3*H*d] (q | k | v, head major)
  int H, N, Sh;
  float scale;
  int* status;
};

template <int D>
struct Smem {
  static constexpr int CH = D / 16;                 // 16-element (32-byte) column chunks
  static constexpr int TILE = 128 * 32 * CH;        // one 128-row tile of D columns, chunk major
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_RELW = OFF_Q + TILE;                 // [128][64] bf16, 128B swizzle
  static constexpr int OFF_E = OFF_RELW + 128 * 128;            // [128][64] bf16 one-hot, 128B swizzle
  static constexpr int OFF_RELH = OFF_E + 128 * 128;            // [64][128] bf16 (key row major)
  static constexpr int OFF_P = OFF_RELH + 64 * 128 * 2;         // 2 x [128][64] bf16, 128B swizzle
  static constexpr int OFF_KV = OFF_P + 2 * 128 * 128;          // ring of (K tile, V tile)
  static constexpr int OFF_BAR = OFF_KV + KV_STAGES * 2 * TILE;
  static constexpr int BYTES = OFF_BAR + 256 + 1024;
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_global_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  using L = Smem<D>;
  constexpr int CH = L::CH;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* q_full = bars + 0;
  uint64_t* pro_done = bars + 1;
  uint64_t* kv_full = bars + 2;                 // [KV_STAGES]
  uint64_t* kv_empty = kv_full + KV_STAGES;     // [KV_STAGES]
  uint64_t* s_full = kv_empty + KV_STAGES;      // [2]
  uint64_t* s_empty = s_full + 2;               // [2]
  uint64_t* p_full = s_empty + 2;
  uint64_t* p_empty = p_full + 1;
  uint64_t* o_full = p_empty + 1;               // [2]
  uint64_t* o_empty = o_full + 2;               // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles_q = p.N / BM;
  const int bh = blockIdx.x / n_tiles_q;
  const int n0 = (blockIdx.x - bh * n_tiles_q) * BM;
  const int b = bh / p.H, h = bh - b * p.H;
  const int nblk = p.N / BK;

  // tensor-map coordinates of this (image, head): row of token 0, 16-element column chunk of q/k/v
  int row_base, cq, ck, cv;
  if (p.qkv_fused) {
    row_base = b * p.N;
    cq = (h * D) / 16;
    ck = (p.H * D + h * D) / 16;
    cv = (2 * p.H * D + h * D) / 16;
  } else {
    row_base = bh * p.N;
    cq = ck = cv = 0;
  }

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    mbar_init(pro_done, 128);
    for (int s = 0; s < KV_STAGES; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 128);
      mbar_init(&o_full[i], 1); mbar_init(&o_empty[i], 128);
    }
    mbar_init(p_full, 128);
    mbar_init(p_empty, 1);
    fence_mbar_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      mbar_expect_tx(q_full, L::TILE);
      tma_load_3d(smem + L::OFF_Q, &tmQ, q_full, 0, row_base + n0, cq);
      uint32_t stage = 0, phase = 0;
      for (int j = 0; j < nblk; ++j) {
        if (!mbar_wait(&kv_empty[stage], phase ^ 1u, abort_flag, p.status, 1)) break;
        uint8_t* sk = smem + L::OFF_KV + stage * 2 * L::TILE;
        mbar_expect_tx(&kv_full[stage], 2 * L::TILE);
        tma_load_3d(sk, &tmK, &kv_full[stage], 0, row_base + j * BK, ck);
        tma_load_3d(sk + L::TILE, &tmV, &kv_full[stage], 0, row_base + j * BK, cv);
        if (++stage == KV_STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(kAccF32, kFmtBF16, kFmtBF16, BM, BK);
      constexpr uint32_t idesc_o = make_idesc(kAccF32, kFmtBF16, kFmtBF16, BM, D, false, /*B MN-major*/ true);
      const uint32_t q_addr = smem_u32(smem + L::OFF_Q);
      const uint32_t relw_addr = smem_u32(smem + L::OFF_RELW);
      const uint32_t e_addr = smem_u32(smem + L::OFF_E);
      const uint32_t p_addr = smem_u32(smem + L::OFF_P);
      const uint32_t kv_addr = smem_u32(smem + L::OFF_KV);
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, 2) && mbar_wait(pro_done, 0, abort_flag, p.status, 3);

      auto issue_s = [&](int j) -> bool {        // S[j%2] = [Q | relw] * [K_j | E]^T
        const uint32_t st = uint32_t(j % KV_STAGES), sb = uint32_t(j & 1);
        if (!mbar_wait(&kv_full[st], uint32_t(j / KV_STAGES) & 1u, abort_flag, p.status, 4)) return false;
        if (!mbar_wait(&s_empty[sb], (uint32_t(j >> 1) & 1u) ^ 1u, abort_flag, p.status, 5)) return false;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + sb * 128;
        const uint32_t k_addr = kv_addr + st * 2 * L::TILE;
#pragma unroll
        for (int c = 0; c < CH; ++c) {           // K-major, 32B swizzle: 8-row groups 256 B apart
          umma_f16_ss(d_tmem, make_smem_desc(q_addr + c * 4096, 16, 256, kSwizzle32B),
                      make_smem_desc(k_addr + c * 4096, 16, 256, kSwizzle32B), idesc_s, c != 0);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {            // K-major, 128B swizzle
          umma_f16_ss(d_tmem, make_smem_desc(relw_addr + c * 32, 16, 1024, kSwizzle128B),
                      make_smem_desc(e_addr + c * 32, 16, 1024, kSwizzle128B), idesc_s, 1u);
        }
        tc_commit(&s_full[sb]);
        return true;
      };

      if (ok) ok = issue_s(0);
      for (int j = 0; ok && j < nblk; ++j) {
        if (j + 1 < nblk) { if (!(ok = issue_s(j + 1))) break; }
        const uint32_t st = uint32_t(j % KV_STAGES), ob = uint32_t(j & 1);
        if (!(ok = mbar_wait(p_full, uint32_t(j) & 1u, abort_flag, p.status, 6))) break;
        if (!(ok = mbar_wait(&o_empty[ob], (uint32_t(j >> 1) & 1u) ^ 1u, abort_flag, p.status, 7))) break;
        tc_fence_after();
        const uint32_t v_addr = kv_addr + st * 2 * L::TILE + L::TILE;
        const uint32_t d_tmem = tmem_base + 256 + ob * 128;
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk) {
          // A = P: K-major 128B swizzle, two [128][64] tiles.  B = V: MN-major 32B swizzle, 16 keys
          // (512 B) per step, column chunks 4096 B apart (LBO), 8-key groups 256 B apart (SBO).
          umma_f16_ss(d_tmem,
                      make_smem_desc(p_addr + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024, kSwizzle128B),
                      make_smem_desc(v_addr + kk * 512, 4096, 256, kSwizzle32B), idesc_o, kk != 0);
        }
        tc_commit(&o_full[ob]);
        tc_commit(&kv_empty[st]);
        tc_commit(p_empty);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax (one thread = one row)
    const int i = (warp & 3) * 32 + lane;                 // row in the tile == TMEM lane
    const uint32_t lane_addr = tmem_base + (uint32_t((warp & 3) * 32) << 16);
    const int n = n0 + i;                                  // token index inside the image
    const int qh = n / SW, qw = n - qh * SW;
    // rel_w tensors are divided by scale here; table products arrive already divided (see the ABI header)
    const float inv_scale = p.rel_mode == 0 ? 1.0f / p.scale : 1.0f;
    // ---- prologue: rel_w/scale -> swizzled A tile, one-hot E row, rel_h column
    {
      const __nv_bfloat16* src_h;
      const __nv_bfloat16* src_w;
      int step;                                            // +1: src[k]; -1: src[-k] (table products)
      if (p.rel_mode == 0) {
        src_h = p.rel_h + ((long long)bh * p.N + n) * p.Sh;
        src_w = p.rel_w + ((long long)bh * p.N + n) * SW;
        step = 1;
      } else {
        const __nv_bfloat16* t = p.tab + ((long long)b * p.N + n) * p.ldt + h * p.t_head_stride;
        src_h = t + (qh + p.Sh - 1);
        src_w = t + p.t_w_off + (qw + SW - 1);
        step = -1;
      }
      uint8_t* relw_row = smem + L::OFF_RELW + i * 128;
      uint8_t* e_row = smem + L::OFF_E + i * 128;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        uint32_t w[4], e[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int k0 = u * 8 + 2 * t;
          const float a = __bfloat162float(src_w[step * k0]) * inv_scale;
          const float c = __bfloat162float(src_w[step * (k0 + 1)]) * inv_scale;
          w[t] = pack2(a, c);
          e[t] = ((i & 63) == k0 ? 0x3F80u : 0u) | ((i & 63) == k0 + 1 ? 0x3F800000u : 0u);
        }
        const int phys = (u ^ (i & 7)) << 4;
        *reinterpret_cast<uint4*>(relw_row + phys) = make_uint4(w[0], w[1], w[2], w[3]);
        *reinterpret_cast<uint4*>(e_row + phys) = make_uint4(e[0], e[1], e[2], e[3]);
      }
      __nv_bfloat16* relh = reinterpret_cast<__nv_bfloat16*>(smem + L::OFF_RELH);
      for (int kh = 0; kh < p.Sh; ++kh) relh[kh * 128 + i] = src_h[step * kh];
      fence_proxy_async_smem();
      mbar_arrive(pro_done);
    }
    const __nv_bfloat16* relh = reinterpret_cast<const __nv_bfloat16*>(smem + L::OFF_RELH);
    const float c2 = p.scale * kLog2e;
    float m_run = -INFINITY, l_run = 0.f, alpha_prev = 1.f;
    float acc[D];
#pragma unroll
    for (int c = 0; c < D; ++c) acc[c] = 0.f;
    bool ok = true;

    auto fold_o = [&](int j, float alpha) -> bool {       // acc = acc * alpha + (P_j V_j)
      const uint32_t ob = uint32_t(j & 1);
      if (!mbar_wait(&o_full[ob], uint32_t(j >> 1) & 1u, abort_flag, p.status, 8)) return false;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < D / 16; ++c) {
        uint32_t r[16];
        tmem_ld_32x32b_x16(lane_addr + 256 + ob * 128 + c * 16, r);
        tmem_ld_wait();
#pragma unroll
        for (int t = 0; t < 16; ++t) acc[c * 16 + t] = fmaf(acc[c * 16 + t], alpha, __uint_as_float(r[t]));
      }
      tc_fence_before();
      mbar_arrive(&o_empty[ob]);
      return true;
    };

    for (int j = 0; j < nblk; ++j) {
      const uint32_t sb = uint32_t(j & 1);
      if (!(ok = mbar_wait(&s_full[sb], uint32_t(j >> 1) & 1u, abort_flag, p.status, 9))) break;
      tc_fence_after();
      const uint32_t s_addr = lane_addr + sb * 128;
      // pass 1: row maximum, separately for the two key rows of this tile
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(s_addr + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int t = 0; t < 32; ++t) mx[c >> 1] = fmaxf(mx[c >> 1], __uint_as_float(r[t]));
      }
      const float bh0 = __bfloat162float(relh[(2 * j) * 128 + i]) * kLog2e;
      const float bh1 = __bfloat162float(relh[(2 * j + 1) * 128 + i]) * kLog2e;
      const float m_new = fmaxf(m_run, fmaxf(fmaf(mx[0], c2, bh0), fmaf(mx[1], c2, bh1)));
      const float alpha = fast_exp2(m_run - m_new);
      const float add[2] = {bh0 - m_new, bh1 - m_new};
      // P buffer must have been consumed by the previous P V
      if (!(ok = mbar_wait(p_empty, (uint32_t(j) & 1u) ^ 1u, abort_flag, p.status, 10))) break;
      // pass 2: p = exp2(s * c2 + add), row sum, bf16 P into the swizzled A tile
      float l_blk = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(s_addr + c * 32, r);
        tmem_ld_wait();
        uint8_t* prow = smem + L::OFF_P + (c >> 1) * 16384 + i * 128;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          float e[8];
#pragma unroll
          for (int t = 0; t < 8; ++t) {
            e[t] = fast_exp2(fmaf(__uint_as_float(r[u * 8 + t]), c2, add[c >> 1]));
            l_blk += e[t];
          }
          const int unit = (c & 1) * 4 + u;
          *reinterpret_cast<uint4*>(prow + ((unit ^ (i & 7)) << 4)) =
              make_uint4(pack2(e[0], e[1]), pack2(e[2], e[3]), pack2(e[4], e[5]), pack2(e[6], e[7]));
        }
      }
      tc_fence_before();
      mbar_arrive(&s_empty[sb]);
      fence_proxy_async_smem();
      mbar_arrive(p_full);
      // fold the previous tile's P V while the tensor core works on this one
      if (j > 0) { if (!(ok = fold_o(j - 1, alpha_prev))) break; }
      l_run = fmaf(l_run, alpha, l_blk);
      m_run = m_new;
      alpha_prev = alpha;
    }
    if (ok) ok = fold_o(nblk - 1, alpha_prev);
    if (ok) {
      const float inv_l = 1.0f / l_run;
      // output row: [BH*N, d] rows for the op layout, token rows with a per-head column slice otherwise
      __nv_bfloat16* orow = p.qkv_fused ? p.o + ((long long)b * p.N + n) * p.o_pitch + h * p.o_head_stride
                                        : p.o + ((long long)bh * p.N + n) * p.o_pitch;
#pragma unroll
      for (int u = 0; u < D / 8; ++u) {
        *reinterpret_cast<uint4*>(orow + u * 8) =
            make_uint4(pack2(acc[u * 8] * inv_l, acc[u * 8 + 1] * inv_l), pack2(acc[u * 8 + 2] * inv_l, acc[u * 8 + 3] * inv_l),
                       pack2(acc[u * 8 + 4] * inv_l, acc[u * 8 + 5] * inv_l), pack2(acc[u * 8 + 6] * inv_l, acc[u * 8 + 7] * inv_l));
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

}  // namespace

template <int D>
static int launch_d(const void* q, const void* k, const void* v, long long rows, long long cols, long long pitch_elems,
                    const AttnParams& p, int BH, void* stream) {
  CUtensorMap tm[3];
  const void* base[3] = {q, k, v};
  for (int t = 0; t < 3; ++t) {
    const uint64_t dims[3] = {16, uint64_t(rows), uint64_t(cols / 16)};
    const uint64_t strides[3] = {2, uint64_t(pitch_elems) * 2, 32};
    const uint32_t box[3] = {16, 128, uint32_t(D / 16)};
    if (int e = make_tensor_map(&tm[t], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base[t]), dims, strides,
                                box, CU_TENSOR_MAP_SWIZZLE_32B))
      return e;
  }
  auto kern = attn_global_kernel<D>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<D>::BYTES) != cudaSuccess)
    return SAMB_E_LAUNCH;
  const long long grid = (long long)BH * (p.N / BM);
  if (grid > 0x7fffffffLL) return SAMB_E_SHAPE;
  kern<<<unsigned(grid), NUM_THREADS, Smem<D>::BYTES, static_cast<cudaStream_t>(stream)>>>(tm[0], tm[1], tm[2], p);
  return launch_status();
}

}  // namespace samb

extern "C" {

int samb_attn_relpos_global(const void* q, const void* k, const void* v, const void* rel_h, const void* rel_w,
                            void* o, int B, int H, int N, int d, float scale, int32_t* status, void* stream) {
  using namespace samb;
  if (!q || !k || !v || !rel_h || !rel_w || !o || !status) return SAMB_E_BADARG;
  if (B <= 0 || H <= 0 || N <= 0) return SAMB_E_BADARG;
  if ((d != 64 && d != 80) || N % 128 || N > 4096) return SAMB_E_SHAPE;
  if ((long long)B * H * N > 0x7fffffffLL) return SAMB_E_SHAPE;
  if (reinterpret_cast<uintptr_t>(o) & 15u) return SAMB_E_ALIGN;
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
  return d == 80 ? launch_d<80>(q, k, v, rows, d, d, p, B * H, stream) : launch_d<64>(q, k, v, rows, d, d, p, B * H, stream);
}

int samb_attn_relpos_global_qkv(const void* qkv, const void* tab, int64_t ldt, int t_head_stride, int t_w_off, void* o,
                                int64_t o_pitch, int B, int H, int N, int d, float scale, int32_t* status,
                                void* stream) {
  using namespace samb;
  if (!qkv || !tab || !o || !status) return SAMB_E_BADARG;
  if (B <= 0 || H <= 0 || N <= 0) return SAMB_E_BADARG;
  if ((d != 64 && d != 80) || N % 128 || N > 4096) return SAMB_E_SHAPE;
  if ((long long)B * N > 0x7fffffffLL || o_pitch % 8 || o_pitch < (int64_t)H * d) return SAMB_E_SHAPE;
  if (ldt < (int64_t)H * t_head_stride || t_w_off + 127 > t_head_stride || N / 64 * 2 - 1 > t_w_off) return SAMB_E_SHAPE;
  if (reinterpret_cast<uintptr_t>(o) & 15u) return SAMB_E_ALIGN;
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
  const long long rows = (long long)B * N, cols = 3LL * H * d;
  return d == 80 ? launch_d<80>(qkv, qkv, qkv, rows, cols, cols, p, B * H, stream)
                 : launch_d<64>(qkv, qkv, qkv, rows, cols, cols, p, B * H, stream);
}

}  // extern "C"
