/*
 * samb200 — C ABI of the B200 (sm_100a) SAM image-encoder kernels.
 *
 * Conventions
 *   - Every entry point returns SAMB_OK (0) or a negative SAMB_E_* code; argument errors are
 *     detected on the host before anything is launched.  No C++ exception crosses this boundary.
 *   - All pointers are DEVICE pointers owned by the caller unless the comment says "host".
 *     The library allocates nothing, frees nothing, keeps no pointer after returning and never
 *     synchronises: work is enqueued on `stream` (a cudaStream_t passed as void*).
 *   - `status` is a caller-owned 4-byte device word, zero-initialised by the caller.  Kernels that
 *     wait on hardware barriers bound every wait; a wait that runs out stores
 *     (0x7E << 24) | (site << 16) | (cta & 0xffff) there and the kernel drains and returns.
 *   - bf16 tensors are row-major, 16-byte aligned, with row lengths that are multiples of 8
 *     elements (16 for int8).  Small vectors (bias, LayerNorm gain/offset, scales) are float32.
 *   - Threading: no entry point keeps per-call state, so calls from different host threads do not disturb
 *     one another's results.  The library does keep a few process-wide caches of device facts (architecture
 *     check and SM count per device ordinal, how many CTA pairs fit on a GPU, the driver entry point used to
 *     build TMA tensor maps).  They are filled on first use without locking: concurrent first calls write the
 *     same values, the occupancy figure assumes that every GPU of the process is the same model, and none of
 *     them holds a caller pointer.  One process per GPU, calls from one thread, is the tested arrangement.
 *   - Citations "ref:" name the file:line of pytorch-labs/segment-anything-fast that the entry
 *     point replaces on the image-encoder path.
 */
#ifndef SAMB200_H_
#define SAMB200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SAMB_ABI_VERSION 1

enum {
  SAMB_OK = 0,
  SAMB_E_BADARG = -1,  /* null pointer / negative size / unknown enum value */
  SAMB_E_SHAPE = -2,   /* size outside what the kernel supports */
  SAMB_E_ALIGN = -3,   /* pointer or stride not 16-byte aligned */
  SAMB_E_ARCH = -4,    /* current device is not sm_100 */
  SAMB_E_LAUNCH = -5,  /* CUDA reported an error at launch or tensor-map creation */
  SAMB_E_TIMEOUT = -6, /* reported by samb_decode_status for a device-side bounded-wait expiry */
  SAMB_E_NOT24 = -7    /* reported by samb_decode_status: samb_pack_sp24 met a group of four with > 2 non-zeros */
};

/* GEMM epilogues (bit flags) */
enum {
  SAMB_EPI_BIAS = 1,      /* + bias[n]                                         */
  SAMB_EPI_GELU = 2,      /* exact (erf) GELU after the bias                   */
  SAMB_EPI_RESIDUAL = 4,  /* + residual[m, n] (bf16) after bias / GELU          */
  SAMB_EPI_RAW = 8        /* store the raw accumulator (fp32 / int32), no other flag allowed */
};

int samb_abi_version(void);
const char* samb_error_string(int code);
/* Host helper: maps a status word read back from the device to SAMB_OK / SAMB_E_TIMEOUT / SAMB_E_NOT24. */
int samb_decode_status(int32_t status_word);
/* Waits (bounded, ~`limit_polls` polls) on a barrier that nothing signals; the kernel must come
 * back with the timeout code in *status.  Exercises the give-up path without faulting anything. */
int samb_selftest_bounded_wait(int32_t* status, uint32_t limit_polls, void* stream);
/* Tensor-pipe rate probe (measurement aid, no counterpart in the reference): `ctas` CTAs each issue
 * `rounds` x 16 back-to-back tcgen05.mma (M 128, N 256; kind::i8 when int8 != 0, else kind::f16 on bf16) on
 * operands resident in shared memory.  *ops_out (host, optional) receives the operations launched (2 per
 * multiply-add); the caller times the launch with events.  `sink` (device, optional) is never written in
 * practice; it keeps the accumulators observable.  Gives the measured int8 / bf16 peak that roofline
 * fractions of the GEMMs are quoted against. */
int samb_selftest_mma_rate(int int8, int rounds, int ctas, int32_t* status, int32_t* sink, double* ops_out,
                           void* stream);

/* ---------------------------------------------------------------------------------------------
 * LayerNorm over the last dim of x[rows, C] (bf16 in, fp32 statistics, bf16 out).
 * ref: nn.LayerNorm in Block.forward, modeling/image_encoder.py:152,162,169,181 (eps 1e-6 from
 * build_sam.py:112).
 * If window > 0 the rows are tokens of `rows / (grid*grid)` images on a grid x grid raster and the
 * output is written in the window-partitioned, zero-padded order of window_partition
 * (modeling/image_encoder.py:256-277): y[(img*nw*nw + wy*nw + wx)*window*window + ly*window + lx, :],
 * nw = ceil(grid/window), pad rows are written as zeros.  y then has
 * images*nw*nw*window*window rows.  With window == 0, y has `rows` rows in the input order.
 * ------------------------------------------------------------------------------------------- */
int samb_layernorm_bf16(const void* x, const float* gamma, const float* beta, void* y, int64_t rows, int C,
                        float eps, int grid, int window, void* stream);

/* Same, fused with per-row symmetric int8 quantisation of the bf16-rounded LayerNorm output:
 * scale[r] = max(absmax_r, 1e-5) / 127, yq = clamp(rint(y / scale), -127, 127).
 * ref: torchao apply_dynamic_quant at experiments/eval_combo.py:357-360 (activation side). */
int samb_layernorm_quant_i8(const void* x, const float* gamma, const float* beta, int8_t* yq, float* scale,
                            int64_t rows, int C, float eps, int grid, int window, void* stream);

/* Per-row symmetric int8 quantisation of x[rows, C] (bf16), same formula. */
int samb_quant_rows_i8(const void* x, int8_t* yq, float* scale, int64_t rows, int C, void* stream);
/* The same after the exact (erf) GELU: yq, scale = quantise(bf16(gelu(x))): the MLP's activation
 * (modeling/common.py:25-26, act between lin1 and lin2) applied to a bf16 lin1 output that was produced
 * without the GELU epilogue. */
int samb_gelu_quant_rows_i8(const void* x, int8_t* yq, float* scale, int64_t rows, int C, void* stream);

/* ---------------------------------------------------------------------------------------------
 * out[M, N] = epilogue(A[M, K] * W[N, K]^T), bf16 operands, fp32 accumulation on tcgen05 tensor
 * cores (TMA-fed, accumulators in tensor memory).  A, W, out, residual row-major bf16 with leading
 * dimensions lda, ldw, ldo, ldr (elements, multiples of 8).  With SAMB_EPI_RAW `out` is float32.
 * The residual has res_rows rows and row m adds residual[m % res_rows] (res_rows == M for a plain
 * residual; res_rows == tokens per image broadcasts one positional table over the batch).
 * ref: nn.Linear qkv/proj (modeling/image_encoder.py:213-214,228,251), MLPBlock lin1/GELU/lin2
 * (modeling/common.py:21-26), the residual adds (image_encoder.py:180-181), PatchEmbed conv as a
 * GEMM (:398-406) and the neck's convolutions (:89-105).
 * ------------------------------------------------------------------------------------------- */
int samb_gemm_bf16(const void* A, int64_t lda, const void* W, int64_t ldw, const float* bias, const void* residual,
                   int64_t ldr, int64_t res_rows, void* out, int64_t ldo, int64_t M, int N, int K, int epilogue,
                   int32_t* status, void* stream);

/* out[M, N] = epilogue(float(int32(Aq[M,K]) * int32(Wq[N,K])^T) * a_scale[m] * w_scale[n]),
 * int8 operands, exact int32 accumulation on tcgen05 kind::i8.  With SAMB_EPI_RAW `out` is int32
 * and the scales are ignored.  K multiple of 16.
 * ref: torchao dynamically-quantised Linear swapped in at experiments/eval_combo.py:357-360. */
int samb_gemm_i8(const int8_t* Aq, int64_t lda, const float* a_scale, const int8_t* Wq, int64_t ldw,
                 const float* w_scale, const float* bias, const void* residual, int64_t ldr, int64_t res_rows,
                 void* out, int64_t ldo, int64_t M, int N, int K, int epilogue, int32_t* status, void* stream);

/* The int8 Linear of samb_gemm_i8 (epilogue: SAMB_EPI_BIAS and / or SAMB_EPI_GELU only) that also hands its
 * output on as the next int8 Linear's input: out[M, N] (bf16, as samb_gemm_i8 writes it) plus its per-row symmetric
 * int8 quantisation yq[M, N] (contiguous rows of N), y_scale[M] = max(absmax_m, 1e-5) / 127, the same values
 * samb_quant_rows_i8 gives on `out`.  The GEMM epilogue leaves every row's |max| in row_absmax_scratch (M floats of
 * caller-owned scratch memory, any contents on entry: it is cleared first) through atomic maxima, so the
 * quantisation is a streaming pass with no reduction.  Two calls sharing one scratch array must not overlap.
 * ref: lin1 -> act -> lin2 of MLPBlock with torchao's dynamically quantised Linears, modeling/common.py:21-26,
 * experiments/eval_combo.py:357-360 (lin2's activation-side quantisation of lin1's output). */
int samb_gemm_i8_requant(const int8_t* Aq, int64_t lda, const float* a_scale, const int8_t* Wq, int64_t ldw,
                         const float* w_scale, const float* bias, void* out, int64_t ldo, int8_t* yq, float* y_scale,
                         float* row_absmax_scratch, int64_t M, int N, int K, int epilogue, int32_t* status,
                         void* stream);

/* The same for a 2:4-compressed weight (samb_pack_sp24 output; arguments as samb_gemm_i8_sp24): the sparse kernel's
 * epilogue stages its tile token-major, and one thread per token row leaves that row's |max| in the scratch.
 * ref: as above, for the pruned mlp.lin1 of sparse.py:28-32. */
int samb_gemm_i8_sp24_requant(const int8_t* Xq, int64_t ldx, const float* x_scale, const int8_t* Wc, int64_t ldc,
                              const uint8_t* meta, const float* w_scale, const float* bias, void* out, int64_t ldo,
                              int8_t* yq, float* y_scale, float* row_absmax_scratch, int64_t T, int N, int K,
                              int epilogue, int32_t* status, void* stream);

/* samb_gemm_i8_requant for callers that cannot allocate device memory (no counterpart in the reference).
 * Some hosts of this library have nowhere to get scratch from: a plug-in running inside an inference server whose
 * memory pool is closed to it, a process whose device memory was handed out in full at start-up, a real-time loop
 * that must keep away from the allocator (cudaMalloc synchronises the device).  They pass only inputs and
 * outputs; the one-float-per-row scratch is an array inside the library's own device image instead
 * (1 MiB, held by every GPU that loads the library until the process exits).
 *  - At most samb_gemm_i8_requant_static_max_rows() rows (262144); more returns SAMB_E_SHAPE.
 *  - The first call on a device looks up the array's device address (with that device current).  Make that first
 *    call outside any stream capture.
 *  - Every call on a device uses the same array (it is cleared at the start of each call), so two calls that may
 *    overlap on the GPU (different streams) race; serialise them.
 *  - Nothing is allocated or freed, by this entry point or by anything it calls. */
int64_t samb_gemm_i8_requant_static_max_rows(void);
int samb_gemm_i8_requant_static(const int8_t* Aq, int64_t lda, const float* a_scale, const int8_t* Wq, int64_t ldw,
                                const float* w_scale, const float* bias, void* out, int64_t ldo, int8_t* yq,
                                float* y_scale, int64_t M, int N, int K, int epilogue, int32_t* status, void* stream);

/* Channel LayerNorm of x[tokens, C] (token-major rows, bf16): each row is normalised over its C
 * channels in fp32.  With to_nchw != 0 the result is stored as out[tokens/hw, C, hw] (hw multiple
 * of 32), else in the input layout.
 * ref: LayerNorm2d, modeling/common.py:31-43, used by the neck (modeling/image_encoder.py:96,104). */
int samb_layernorm2d_nchw(const void* x, const float* gamma, const float* beta, void* out, int64_t tokens, int C,
                          int hw, float eps, int to_nchw, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Attention with the decomposed relative-position bias, global blocks:
 *   o = softmax(scale * q k^T + rel_h[..., i, kh(j)] + rel_w[..., i, kw(j)]) v,  key j = kh*64 + kw.
 * q, k, v, o: contiguous bf16 [B, H, N, d]; rel_h: [B, H, N, N/64]; rel_w: [B, H, N, 64] (bf16).
 * N a multiple of 256, N <= 4096, d in {64, 80}.  tcgen05 flash attention: logits and P·V in tensor
 * memory, K/V tiles by TMA, rel_w added on the tensor core through a one-hot operand, rel_h folded
 * into the exponent's FMA.
 * ref: _attention_rel_h_rel_w and the Triton kernel it dispatches to, flash_4.py:30-145,335-370
 * (called at modeling/image_encoder.py:245).
 * ------------------------------------------------------------------------------------------- */
int samb_attn_relpos_global(const void* q, const void* k, const void* v, const void* rel_h, const void* rel_w,
                            void* o, int B, int H, int N, int d, float scale, int32_t* status, void* stream);

/* The same operator on float16 tensors (q, k, v, rel_h, rel_w, o all float16): the tensor core multiplies
 * float16 operands, the probabilities are rounded to float16, everything else (logits, softmax statistics, output
 * accumulator) is fp32 as above.  ref: the float16 half of the reference's own test of the operator,
 * test/test_flash_4.py:10-43 (dtype sweep). */
int samb_attn_relpos_global_f16(const void* q, const void* k, const void* v, const void* rel_h, const void* rel_w,
                                void* o, int B, int H, int N, int d, float scale, int32_t* status, void* stream);

/* Same attention reading q/k/v from the head-major qkv buffer qkv[3*H][B*N][d] written by
 * samb_gemm_*_heads (planes: q heads, k heads, v heads) and writing o[B*N, o_pitch]
 * with head h at columns [h*d, (h+1)*d) (the layout proj consumes, image_encoder.py:249).  The bias
 * comes from table products tab[B*N, ldt]: for head h, tab[t, h*t_head_stride + m] = q_t,h . rel_pos_h[m]
 * (m < 2*N/64-1) and tab[t, h*t_head_stride + t_w_off + m] = (q_t,h . rel_pos_w[m]) / scale (m < 127),
 * i.e. the width products are stored already divided by the softmax scale; the kernel
 * reads rel_h[i, kh] = tab[.., qh(i) - kh + N/64 - 1] and rel_w[i, kw] = tab[.., t_w_off + qw(i) - kw + 63]
 * (get_rel_pos / add_decomposed_rel_pos, modeling/image_encoder.py:305-372). */
int samb_attn_relpos_global_qkv(const void* qkv, const void* tab, int64_t ldt, int t_head_stride, int t_w_off, void* o,
                                int64_t o_pitch, int B, int H, int N, int d, float scale, int32_t* status,
                                void* stream);

/* The same attention with the bias computed inside the kernel from the relative-position tables themselves:
 * tables is bf16 [256, d] holding rel_pos_h (2*N/64 - 1 rows) from row 0 and rel_pos_w (127 rows) from row 128,
 * zeros elsewhere.  Every CTA multiplies its 256 query rows by the table block on the tensor core before the key
 * loop (q . rel_pos_h[m] and (q . rel_pos_w[m]) / scale, rounded to bf16 as a separately stored product would be)
 * and reads rel_h[i, kh] = T_h[qh(i) - kh + N/64 - 1], rel_w[i, kw] = T_w[qw(i) - kw + 63] from shared memory, so
 * no product tensor exists in global memory.  qkv / o as in samb_attn_relpos_global_qkv.
 * ref: add_decomposed_rel_pos + get_rel_pos fused into the attention, modeling/image_encoder.py:305-372, 238-245. */
int samb_attn_relpos_global_tables(const void* qkv, const void* tables, void* o, int64_t o_pitch, int B, int H, int N,
                                   int d, float scale, int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Attention with the decomposed relative-position bias, windowed blocks: B independent windows of
 * window x window = N tokens (window must be 14), key j = kh*window + kw.
 * q, k, v, o: contiguous bf16 [B, H, N, d]; rel_h, rel_w: [B, H, N, window] (bf16); d in {64, 80}.
 * ref: the SDPA composite _attention_rel_h_rel_w falls back to for N = 196, flash_4.py:368-370.
 * ------------------------------------------------------------------------------------------- */
int samb_attn_relpos_window(const void* q, const void* k, const void* v, const void* rel_h, const void* rel_w, void* o,
                            int B, int H, int window, int d, float scale, int32_t* status, void* stream);

/* The same operator on float16 tensors (q, k, v, rel_h, rel_w, o all float16); logits, softmax statistics and the
 * output accumulator stay fp32.  The reference sends this shape to SDPA, which takes either type
 * (flash_4.py:368-370). */
int samb_attn_relpos_window_f16(const void* q, const void* k, const void* v, const void* rel_h, const void* rel_w, void* o,
                            int B, int H, int window, int d, float scale, int32_t* status, void* stream);

/* Windowed attention over the head-major qkv projection of the window-partitioned, zero-padded token
 * order (the row order samb_layernorm_bf16 writes with window > 0): qkv[3*H][B*nw*nw*N][d].  The output goes
 * straight back to raster order, o[(b*grid + y)*grid + x, h*d ...] with pad tokens dropped, i.e.
 * window_unpartition (modeling/image_encoder.py:280-302) is folded into the store.  Bias from table
 * products as in samb_attn_relpos_global_qkv with 2*window-1 entries per table. */
int samb_attn_relpos_window_qkv(const void* qkv, const void* tab, int64_t ldt, int t_head_stride, int t_w_off, void* o,
                                int64_t o_pitch, int B, int H, int grid, int window, int d, float scale,
                                int32_t* status, void* stream);

/* Windowed attention straight from raster-order head-major qkv [3H][B*grid*grid][d]: no window-partitioned
 * copy of the tokens exists.  Each (window, head) gathers its window x window tokens with TMA boxes; the part of
 * a border window beyond the raster is the reference's zero padding (F.pad in window_partition,
 * modeling/image_encoder.py:268-271), whose keys / values are the projection biases: qkv_bias is the qkv
 * Linear's bias as bf16 [3H*d] (zeros for a bias-free projection).  tab [B*grid*grid, ldt] holds the table
 * products of samb_relpos_table_products in raster row order.  o as in samb_attn_relpos_window_qkv. */
int samb_attn_relpos_window_raster(const void* qkv, const void* qkv_bias, const void* tab, int64_t ldt,
                                   int t_head_stride, int t_w_off, void* o, int64_t o_pitch, int B, int H, int grid,
                                   int window, int d, float scale, int32_t* status, void* stream);

/* The same with the bias computed inside the kernel from the relative-position tables: tables is bf16 [64, d]
 * holding rel_pos_h (2*window - 1 rows) from row 0 and rel_pos_w from row 32, zeros elsewhere.  For every
 * (window, head) the kernel multiplies the queries by the table block on the tensor core (q . rel_pos_h[m] and
 * (q . rel_pos_w[m]) / scale, rounded to bf16 as a stored product would be) and every query row shifts its
 * 2 x window values rel[k] = T[pos + window - 1 - k] out of the products in registers; no product tensor exists
 * in global memory.  ref: add_decomposed_rel_pos + get_rel_pos, modeling/image_encoder.py:305-372, inside the
 * windowed attention of :238-245. */
int samb_attn_relpos_window_tables(const void* qkv, const void* qkv_bias, const void* tables, void* o, int64_t o_pitch,
                                   int B, int H, int grid, int window, int d, float scale, int32_t* status,
                                   void* stream);

/* Head-major variants of the qkv projection: out is [N / head_dim][M][head_dim] (bf16), i.e. one
 * contiguous [M, head_dim] plane per (q|k|v, head) instead of M rows of N columns, so that the
 * attention kernels stream whole contiguous tiles.  Epilogue: + bias (may be NULL).  head_dim a
 * multiple of 16 that divides N.
 * ref: the reshape/permute/unbind of the qkv output, modeling/image_encoder.py:228-230. */
int samb_gemm_bf16_heads(const void* A, int64_t lda, const void* W, int64_t ldw, const float* bias, void* out,
                         int64_t M, int N, int K, int head_dim, int32_t* status, void* stream);
int samb_gemm_i8_heads(const int8_t* Aq, int64_t lda, const float* a_scale, const int8_t* Wq, int64_t ldw,
                       const float* w_scale, const float* bias, void* out, int64_t M, int N, int K, int head_dim,
                       int32_t* status, void* stream);

/* 2:4 semi-structured sparse int8 weights on the sparse tensor-core path (tcgen05.mma.sp).
 * ref: apply_sparse / to_sparse_semi_structured, segment_anything_fast/sparse.py:28-32 (the reference
 * compresses every nn.Linear weight and lets torch's cuSPARSELt/CUTLASS sparse matmul run it); the
 * int8 + 2:4 combination for mlp.lin1 / mlp.lin2 is the one experiments/eval_combo.py:374-376 names.
 *
 * samb_pack_sp24: Wq[N, K] int8 row-major with at most two non-zeros in every aligned group of four
 * along K (K % 32 == 0) -> Wc[N, K/2] int8 (the kept entries in order; ldc % 16 == 0) and `meta`
 * (samb_sp24_meta_bytes(N, K) bytes, 16-byte aligned): the 2-bit positions of the kept entries, tiled
 * for the kernel ([ceil(N/128)][ceil(K/128)][128 rows][16 bytes]).  A group with more than two
 * non-zeros sets *status (samb_decode_status -> SAMB_E_NOT24).
 * samb_gemm_i8_sp24: out[T, N] = epilogue((Xq[T, K] . Wsparse[N, K]^T) * x_scale[t] * w_scale[n]) with
 * the epilogue flags and SAMB_EPI_RAW (int32 out) of samb_gemm_i8; the residual is [T, N] (res_rows
 * must equal T: no row broadcast; ldr % 8 == 0, 16-byte aligned base).  The int32 accumulators equal those of the dense product with the uncompressed Wq bit for bit. */
int64_t samb_sp24_meta_bytes(int N, int K);
int samb_pack_sp24(const int8_t* Wq, int64_t ldw, int N, int K, int8_t* Wc, int64_t ldc, uint8_t* meta,
                   int32_t* status, void* stream);
int samb_gemm_i8_sp24(const int8_t* Xq, int64_t ldx, const float* x_scale, const int8_t* Wc, int64_t ldc,
                      const uint8_t* meta, const float* w_scale, const float* bias, const void* residual,
                      int64_t ldr, int64_t res_rows, void* out, int64_t ldo, int64_t T, int N, int K, int epilogue,
                      int32_t* status, void* stream);

/* Products of every head's queries with the relative-position tables, for the *_qkv attention
 * entry points:  tab[t, h*t_head_stride + m] = (q_planes[h][t, :] . tables[m, :]) * col_scale[m]
 * for m < t_head_stride (a multiple of 64).  q_planes is the head-major qkv buffer (its first H
 * planes are the queries); tables is bf16 [t_head_stride, d] holding rel_pos_h at rows [0, 2S-1),
 * rel_pos_w at rows [t_w_off, t_w_off + 2S-1) and zeros elsewhere; col_scale is 1 for the rel_pos_h
 * rows and 1/scale for the rel_pos_w rows.  One batched tcgen05 GEMM over heads.
 * ref: the two einsums of add_decomposed_rel_pos, modeling/image_encoder.py:365-366. */
int samb_relpos_table_products(const void* q_planes, const void* tables, const float* col_scale, void* tab,
                               int64_t ldt, int64_t rows, int H, int d, int t_head_stride, int32_t* status,
                               void* stream);

/* x[B, Cin, grid*patch, grid*patch] (bf16, NCHW) -> a[B*grid*grid, Cin*patch*patch]: one row per
 * patch in raster order, columns ordered [c][ky][kx] like the flattened Conv2d weight, so that
 * PatchEmbed's strided convolution is a[.] * weight^T.  patch multiple of 8.
 * ref: PatchEmbed.forward, modeling/image_encoder.py:398-406. */
int samb_patch_rows(const void* x, void* a, int B, int Cin, int grid, int patch, void* stream);

/* samb_patch_rows on the raw pixels: x[B, 3, grid*patch, grid*patch] uint8 -> the same patch rows holding
 * bf16((x - mean[c]) / std[c]) (mean / std: HOST arrays of 3 floats), i.e. Sam.preprocess' normalisation, the cast to
 * the model dtype and the im2col of the patch embedding in one pass; no normalised copy of the image exists.
 * patch multiple of 16.  ref: modeling/sam.py:164-168, predictor.py:88-90, modeling/image_encoder.py:398-406. */
int samb_patch_rows_u8(const uint8_t* x, void* a, int B, int Cin, int grid, int patch, const float* mean_host,
                       const float* std_host, void* stream);

/* x[tokens, C] (token-major raster of grid x grid per image) -> a[tokens, 9*C]: the 3x3 neighbourhood
 * [ky][kx][c] of every token with zeros outside the raster (padding 1), the GEMM operand of the
 * neck's second convolution.  ref: nn.Conv2d(256, 256, 3, padding=1), modeling/image_encoder.py:97-103. */
int samb_conv3x3_rows(const void* x, void* a, int64_t tokens, int grid, int C, void* stream);

/* y[b,c,h,w] = bf16((x[b,c,h,w] - mean[c]) / std[c]) for uint8 x[B,3,H,W]; mean/std are HOST arrays of
 * 3 floats.  H*W multiple of 16.  ref: Sam.preprocess normalisation, modeling/sam.py:164-168, and the
 * cast to the model dtype at predictor.py:88-90. */
int samb_normalize_u8(const uint8_t* x, void* y, int B, int C, int H, int W, const float* mean_host,
                      const float* std_host, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Mask filters of the automatic mask generator in one pass over the predicted logits [N, H, W]
 * (fp32, or bf16 when is_bf16): inter[n] / uni[n] = pixels above thr + offset / above thr - offset,
 * boxes[n] = XYXY bounds of (logit > thr) or zeros when empty, binary (optional, may be NULL) =
 * (logit > thr) as bytes.
 * ref: calculate_stability_score (utils/amg.py:193-213, stability = inter / uni), the thresholding and
 * batched_mask_to_box (utils/amg.py:340-383) at automatic_mask_generator.py:335-345. */
int samb_mask_stats(const void* logits, int is_bf16, int64_t N, int H, int W, float thr, float offset,
                    int32_t* inter, int32_t* uni, int32_t* boxes, uint8_t* binary, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Uncompressed run-length encoding of boolean masks [N, H, W] (bytes 0 / 1; W <= 4096) in column-major
 * pixel order, the layout pycocotools reads: row n of counts [N, cap] receives the run lengths (the
 * leading run is of zeros and has length 0 when pixel (0,0) is set) and n_counts[n] how many there are.
 * A mask with more than cap runs still reports its n_counts; its row of counts is then unspecified and
 * the caller repeats the call with a larger cap.
 * ref: mask_to_rle_pytorch (utils/amg.py:144-170) and mask_to_rle_pytorch_2 (utils/amg.py:106-141), called
 * at automatic_mask_generator.py:257. */
int samb_mask_rle(const uint8_t* masks, int64_t N, int H, int W, int32_t* counts, int32_t* n_counts, int cap,
                  void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SAMB200_H_ */
