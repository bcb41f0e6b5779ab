// Host-side plumbing shared by every entry point: tensor-map construction through the driver
// entry point (no link-time dependency on libcuda), device checks, error strings, and the
// bounded-wait self test.
#include <mutex>

#include "common.cuh"

namespace samb {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int make_tensor_map(CUtensorMap* out, CUtensorMapDataType dtype, int rank, void* base, const uint64_t* dims,
                    const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return SAMB_E_LAUNCH;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) return SAMB_E_ALIGN;
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t bx[5], estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    estr[i] = 1;
    if (i > 0) {
      if (strides_bytes[i] % 16) return SAMB_E_ALIGN;
      gstr[i - 1] = strides_bytes[i];
    }
  }
  CUresult r = fn(out, dtype, cuuint32_t(rank), base, gdim, gstr, bx, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? SAMB_OK : SAMB_E_LAUNCH;
}

int check_device_arch() {
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return SAMB_E_LAUNCH;
  if (dev < 64 && cached[dev] != 0) return cached[dev] > 0 ? SAMB_OK : SAMB_E_ARCH;
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return SAMB_E_LAUNCH;
  if (dev < 64) cached[dev] = (major == 10) ? 1 : -1;
  return major == 10 ? SAMB_OK : SAMB_E_ARCH;
}

int sm_count() {
  static int cached[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && cached[dev] > 0) return cached[dev];
  int n = 148;
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  if (dev < 64) cached[dev] = n;
  return n;
}

__global__ void bounded_wait_selftest_kernel(int* status, uint32_t limit) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&bar, 1);
    fence_mbar_init();
  }
  __syncthreads();
  // Nothing ever arrives on `bar`: the wait must give up, record site 0x55 and return false.
  if (threadIdx.x == 0) (void)mbar_wait(&bar, 0, &abort_flag, status, 0x55u, limit);
  __syncthreads();
}

}  // namespace samb

extern "C" {

int samb_abi_version(void) { return SAMB_ABI_VERSION; }

const char* samb_error_string(int code) {
  switch (code) {
    case SAMB_OK: return "ok";
    case SAMB_E_BADARG: return "bad argument";
    case SAMB_E_SHAPE: return "unsupported shape";
    case SAMB_E_ALIGN: return "pointer or stride not 16-byte aligned";
    case SAMB_E_ARCH: return "device is not sm_100";
    case SAMB_E_LAUNCH: return "CUDA launch / tensor-map error";
    case SAMB_E_TIMEOUT: return "device-side bounded wait expired";
    case SAMB_E_NOT24: return "weight is not 2:4 sparse (a group of four holds more than two non-zeros)";
    default: return "unknown error";
  }
}

int samb_decode_status(int32_t w) {
  if (w == 0) return SAMB_OK;
  if ((uint32_t(w) >> 24) == samb::kDevNot24) return SAMB_E_NOT24;
  return ((uint32_t(w) >> 24) == samb::kDevTimeout) ? SAMB_E_TIMEOUT : SAMB_E_LAUNCH;
}

int samb_selftest_bounded_wait(int32_t* status, uint32_t limit_polls, void* stream) {
  if (status == nullptr || limit_polls == 0 || limit_polls > samb::kSpinLimit) return SAMB_E_BADARG;
  if (int e = samb::check_device_arch()) return e;
  samb::bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status, limit_polls);
  return samb::launch_status();
}

}  // extern "C"
