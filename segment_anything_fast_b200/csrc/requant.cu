// int8 Linear whose bf16 output is re-quantised per row for the next int8 Linear, without a reduction pass over
// the output: the GEMM epilogue leaves every row's |max| in a scratch array through atomic maxima, and a purely
// streaming kernel then turns the bf16 rows into int8 with the scale that maximum gives (the arithmetic of
// quant_rows_kernel, bit for bit).  Used for mlp.lin1 -> GELU -> quantise -> mlp.lin2 in the int8 encoder.
//
// The scratch is one float per output row.  samb_gemm_i8_requant takes it from the caller;
// samb_gemm_i8_requant_static keeps it in an array that is part of this library's device image, for callers that
// have no way to allocate device memory.
#include "common.cuh"
#include "rowquant.cuh"

namespace samb {
namespace {

constexpr int kWarps = 8;

__global__ void zero_floats_kernel(float* __restrict__ p, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    p[i] = 0.f;
}

// One warp per row; the row's scale comes from absmax[row], so nothing is reduced and no lane waits for another:
// every lane streams 16-byte pieces in, 8-byte pieces out, five loads in flight at a time.
__global__ void __launch_bounds__(kWarps * 32)
quant_given_absmax_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const float* __restrict__ absmax,
                          int8_t* __restrict__ yq, float* __restrict__ scale, long long rows, int C) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * kWarps + (threadIdx.x >> 5);
  if (row >= rows) return;
  float sc, inv_sc;
  row_scale(__ldg(absmax + row), sc, inv_sc);
  if (lane == 0) scale[row] = sc;
  const int nvec = C >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * ldx);
  uint2* qr = reinterpret_cast<uint2*>(yq + row * (long long)C);
  int i = lane;
  for (; i + 4 * 32 < nvec; i += 5 * 32) {
    uint4 v[5];
#pragma unroll
    for (int u = 0; u < 5; ++u) v[u] = __ldcs(xr + i + u * 32);
#pragma unroll
    for (int u = 0; u < 5; ++u) qr[i + u * 32] = quant8(v[u], sc, inv_sc);
  }
  for (; i < nvec; i += 32) qr[i] = quant8(__ldcs(xr + i), sc, inv_sc);
}

// ---- scratch that needs no allocation --------------------------------------------------------------------------
// One float per output row, for products of up to kStaticRows rows (1 MiB).  The array belongs to the library's
// device image: every GPU on which the library's kernels get loaded holds it until the process exits.
constexpr long long kStaticRows = 262144;
static __device__ __align__(256) float g_row_absmax_static[kStaticRows];

// Device address of the array on the current device.  In host code the array's name is only a handle for the
// runtime, not an address a kernel could use, so the address is asked for once per device, with that device
// current, and kept.  cudaGetSymbolAddress allocates nothing; it may have to load this library's device code on
// the device first, which is why the first call per device belongs before any stream capture.
int static_scratch(float** out) {
  static float* addr[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return SAMB_E_LAUNCH;
  if (addr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_row_absmax_static) != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return SAMB_E_LAUNCH;
    }
    addr[dev] = static_cast<float*>(p);
  }
  *out = addr[dev];
  return SAMB_OK;
}

// Wc / meta null: dense weight Wq [N, K]; else the 2:4-compressed weight of samb_pack_sp24.
int requant(const int8_t* Aq, int64_t lda, const float* a_scale, const int8_t* Wq, int64_t ldw, const uint8_t* meta,
            const float* w_scale, const float* bias, void* out, int64_t ldo, int8_t* yq, float* y_scale,
            float* row_absmax, int64_t M, int N, int K, int epilogue, int32_t* status, void* stream) {
  if (!Aq || !Wq || !out || !yq || !y_scale || !row_absmax || !status) return SAMB_E_BADARG;
  if (M < 0 || N <= 0 || K <= 0) return SAMB_E_BADARG;
  if (epilogue & ~(SAMB_EPI_BIAS | SAMB_EPI_GELU)) return SAMB_E_BADARG;     // no residual, no raw accumulators
  if (N % 8) return SAMB_E_SHAPE;
  if (reinterpret_cast<uintptr_t>(yq) & 7u) return SAMB_E_ALIGN;
  if (M == 0) return SAMB_OK;
  auto st = static_cast<cudaStream_t>(stream);
  // the maxima accumulate with atomics, so the array starts at zero on every call
  const long long zb = (M + 255) / 256;
  zero_floats_kernel<<<unsigned(zb < 1184 ? zb : 1184), 256, 0, st>>>(row_absmax, M);
  if (int e = launch_status()) return e;
  const int e = meta == nullptr
                    ? launch_gemm_i8_rowmax(Aq, lda, a_scale, Wq, ldw, w_scale, bias, nullptr, 0, 0, out, ldo, M, N, K,
                                            epilogue, status, stream, row_absmax)
                    : launch_gemm_i8_sp24(Aq, lda, a_scale, Wq, ldw, meta, w_scale, bias, nullptr, 0, 0, out, ldo, M, N, K,
                                          epilogue, status, stream, row_absmax);
  if (e) return e;
  const long long blocks = (M + kWarps - 1) / kWarps;
  if (blocks > 0x7fffffffLL) return SAMB_E_SHAPE;
  quant_given_absmax_kernel<<<unsigned(blocks), kWarps * 32, 0, st>>>(static_cast<const __nv_bfloat16*>(out), ldo,
                                                                     row_absmax, yq, y_scale, M, N);
  return launch_status();
}

}  // namespace
}  // namespace samb

extern "C" {

int samb_gemm_i8_requant(const int8_t* Aq, int64_t lda, const float* a_scale, const int8_t* Wq, int64_t ldw,
                         const float* w_scale, const float* bias, void* out, int64_t ldo, int8_t* yq, float* y_scale,
                         float* row_absmax_scratch, int64_t M, int N, int K, int epilogue, int32_t* status,
                         void* stream) {
  return samb::requant(Aq, lda, a_scale, Wq, ldw, nullptr, w_scale, bias, out, ldo, yq, y_scale, row_absmax_scratch, M,
                       N, K, epilogue, status, stream);
}

int samb_gemm_i8_sp24_requant(const int8_t* Xq, int64_t ldx, const float* x_scale, const int8_t* Wc, int64_t ldc,
                              const uint8_t* meta, const float* w_scale, const float* bias, void* out, int64_t ldo,
                              int8_t* yq, float* y_scale, float* row_absmax_scratch, int64_t T, int N, int K,
                              int epilogue, int32_t* status, void* stream) {
  if (meta == nullptr) return SAMB_E_BADARG;
  return samb::requant(Xq, ldx, x_scale, Wc, ldc, meta, w_scale, bias, out, ldo, yq, y_scale, row_absmax_scratch, T, N, K,
                       epilogue, status, stream);
}

int64_t samb_gemm_i8_requant_static_max_rows(void) { return samb::kStaticRows; }

int samb_gemm_i8_requant_static(const int8_t* Aq, int64_t lda, const float* a_scale, const int8_t* Wq, int64_t ldw,
                                const float* w_scale, const float* bias, void* out, int64_t ldo, int8_t* yq,
                                float* y_scale, int64_t M, int N, int K, int epilogue, int32_t* status, void* stream) {
  if (M > samb::kStaticRows) return SAMB_E_SHAPE;       // more rows than the built-in scratch holds
  float* scratch = nullptr;
  if (int e = samb::static_scratch(&scratch)) return e;
  return samb::requant(Aq, lda, a_scale, Wq, ldw, nullptr, w_scale, bias, out, ldo, yq, y_scale, scratch, M, N, K,
                       epilogue, status, stream);
}

}  // extern "C"
