// One pass over predicted mask logits [N, H, W] for the automatic mask generator's filters:
//   inter[n] = #(logit > thr + offset), uni[n] = #(logit > thr - offset)    (stability score = inter / uni)
//   box[n]   = XYXY bounds of (logit > thr), [0,0,0,0] for an empty mask
//   binary   = (logit > thr) as bytes (optional)
// One 512-thread block per mask (several resident per SM) streams its H*W logits with 16-byte loads (scalar loads when a mask does
// not start on a 16-byte boundary), keeps counts and bounds in registers, and reduces them through warp
// shuffles and shared memory: no atomics, every output written once.
#include "common.cuh"

namespace samb {
namespace {

constexpr int kThreads = 512;

struct Acc {
  int inter, uni, x0, y0, x1, y1;
};

__device__ __forceinline__ void visit(float v, long long idx, int W, float hi, float lo, float thr, Acc& a, int& y,
                                      int& x) {
  // (y, x) of idx is maintained by the caller for consecutive elements
  a.inter += v > hi;
  a.uni += v > lo;
  if (v > thr) {
    a.x0 = min(a.x0, x); a.x1 = max(a.x1, x);
    a.y0 = min(a.y0, y); a.y1 = max(a.y1, y);
  }
  if (++x == W) { x = 0; ++y; }
}

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__global__ void __launch_bounds__(kThreads)
mask_stats_kernel(const T* __restrict__ logits, int H, int W, float thr, float offset, int* __restrict__ inter,
                  int* __restrict__ uni, int* __restrict__ boxes, uint8_t* __restrict__ binary) {
  constexpr int V = 16 / sizeof(T);                       // elements per 16-byte load
  const long long n = blockIdx.x;
  const long long count = (long long)H * W;
  const T* m = logits + n * count;
  uint8_t* bout = binary != nullptr ? binary + n * count : nullptr;
  const float hi = thr + offset, lo = thr - offset;
  Acc a{0, 0, W, H, -1, -1};
  const bool vec = (reinterpret_cast<uintptr_t>(m) & 15u) == 0 && (bout == nullptr || (reinterpret_cast<uintptr_t>(bout) % V) == 0);
  const long long nvec = vec ? count / V : 0;
#pragma unroll 2
  for (long long i = threadIdx.x; i < nvec; i += kThreads) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(m) + i);
    const T* e = reinterpret_cast<const T*>(&raw);
    const long long idx = i * V;
    int y = int(idx / W), x = int(idx - (long long)y * W);
    uint32_t bits[V / 4 > 0 ? V / 4 : 1] = {};
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float v = to_float<T>(e[j]);
      if (bout != nullptr && v > thr) bits[j / 4] |= 1u << ((j & 3) * 8);
      visit(v, idx + j, W, hi, lo, thr, a, y, x);
    }
    if (bout != nullptr) {
      if (V == 4) *reinterpret_cast<uint32_t*>(bout + idx) = bits[0];
      else *reinterpret_cast<uint2*>(bout + idx) = make_uint2(bits[0], bits[V / 4 > 1 ? 1 : 0]);
    }
  }
  for (long long idx = nvec * V + threadIdx.x; idx < count; idx += kThreads) {     // tail, or everything when unaligned
    const float v = to_float<T>(m[idx]);
    int y = int(idx / W), x = int(idx - (long long)y * W);
    if (bout != nullptr) bout[idx] = v > thr;
    visit(v, idx, W, hi, lo, thr, a, y, x);
  }
  // block reduction
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    a.inter += __shfl_xor_sync(0xffffffffu, a.inter, o);
    a.uni += __shfl_xor_sync(0xffffffffu, a.uni, o);
    a.x0 = min(a.x0, __shfl_xor_sync(0xffffffffu, a.x0, o));
    a.y0 = min(a.y0, __shfl_xor_sync(0xffffffffu, a.y0, o));
    a.x1 = max(a.x1, __shfl_xor_sync(0xffffffffu, a.x1, o));
    a.y1 = max(a.y1, __shfl_xor_sync(0xffffffffu, a.y1, o));
  }
  __shared__ Acc part[kThreads / 32];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = a;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < kThreads / 32; ++w) {
      a.inter += part[w].inter; a.uni += part[w].uni;
      a.x0 = min(a.x0, part[w].x0); a.y0 = min(a.y0, part[w].y0);
      a.x1 = max(a.x1, part[w].x1); a.y1 = max(a.y1, part[w].y1);
    }
    inter[n] = a.inter;
    uni[n] = a.uni;
    const bool empty = a.x1 < a.x0 || a.y1 < a.y0;
    boxes[n * 4 + 0] = empty ? 0 : a.x0;
    boxes[n * 4 + 1] = empty ? 0 : a.y0;
    boxes[n * 4 + 2] = empty ? 0 : a.x1;
    boxes[n * 4 + 3] = empty ? 0 : a.y1;
  }
}

}  // namespace
}  // namespace samb

extern "C" int samb_mask_stats(const void* logits, int is_bf16, int64_t N, int H, int W, float thr, float offset,
                               int32_t* inter, int32_t* uni, int32_t* boxes, uint8_t* binary, void* stream) {
  using namespace samb;
  if (logits == nullptr || inter == nullptr || uni == nullptr || boxes == nullptr) return SAMB_E_BADARG;
  if (N < 0 || H <= 0 || W <= 0) return SAMB_E_BADARG;
  if (N > 0x7fffffffLL || (long long)H * W > 0x7fffffffLL) return SAMB_E_SHAPE;
  if (reinterpret_cast<uintptr_t>(logits) & (is_bf16 ? 1u : 3u)) return SAMB_E_ALIGN;
  if (N == 0) return SAMB_OK;
  auto st = static_cast<cudaStream_t>(stream);
  if (is_bf16)
    mask_stats_kernel<__nv_bfloat16><<<unsigned(N), kThreads, 0, st>>>(static_cast<const __nv_bfloat16*>(logits), H, W, thr,
                                                                     offset, inter, uni, boxes, binary);
  else
    mask_stats_kernel<float><<<unsigned(N), kThreads, 0, st>>>(static_cast<const float*>(logits), H, W, thr, offset, inter,
                                                              uni, boxes, binary);
  return launch_status();
}
