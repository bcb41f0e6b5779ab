// Uncompressed run-length encoding of boolean masks [N, H, W] (bytes 0 / 1) in column-major pixel order, the
// layout pycocotools reads: counts[0] is the length of the leading run of zeros (0 when pixel (0,0) is set), then
// runs of ones and zeros alternate until H*W pixels are covered.
//
// One block per mask.  A thread owns four adjacent columns of one band of rows (up to 1024 threads: column groups x
// row bands), so a warp reads 128 contiguous bytes of a row while every thread walks down its own columns.  In
// column-major order the pixel before (y, x) is (y-1, x), or (H-1, x-1) at the top of a column.  Pass 1 counts the
// value changes of each (column, band) and notes the rows that had one in a short per-thread list in shared memory
// (row, which of the four columns changed); a block-wide exclusive scan in (column, band) order gives each
// (column, band) its rank; pass 2 stores the column-major index of every change at its rank, from the list, or by
// walking the band again when a thread saw more changed rows than its list holds (noise-like masks); pass 3 turns
// consecutive indices into run lengths (staged in shared memory when the mask has at most 8192 of them, else in
// place).  The mask is read once for blob-like masks.  No atomics, no scratch memory: a mask with more runs than
// `cap` reports the count it needs and leaves its row of `counts` unspecified.
#include "common.cuh"

namespace samb {
namespace {

constexpr int kPosLen = 8192;                        // boundaries a block can stage in shared memory (4 bytes each)
constexpr int kListLen = 48;                         // changed rows a thread can note (2 bytes each)
constexpr uint32_t kNibbleMul = (1u << 24) | (1u << 17) | (1u << 10) | (1u << 3);   // bytes 0/1 -> bits 24..27

// bytes of columns c0..c0+3 of one row (0 for columns past W)
template <bool kVec>
__device__ __forceinline__ uint32_t load_cols(const uint8_t* __restrict__ row, int c0, int W) {
  if (kVec) return __ldg(reinterpret_cast<const uint32_t*>(row + c0));
  uint32_t w = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (c0 + j < W) w |= uint32_t(__ldg(row + c0 + j)) << (8 * j);
  return w;
}

// col_threads (a multiple of 32) column groups x bands row bands = blockDim.x <= kMaxThreads; thread = band *
// col_threads + group.  Masks up to 2048 columns run 512-thread blocks (two per SM, 16 rows in flight per thread);
// wider ones 1024-thread blocks with 8 rows in flight.
template <bool kVec, int kMaxThreads>
__global__ void __launch_bounds__(kMaxThreads, kMaxThreads <= 512 ? 2 : 1)
mask_rle_kernel(const uint8_t* __restrict__ masks, int H, int W, int32_t* __restrict__ counts,
                int32_t* __restrict__ n_counts, int cap, int col_threads, int bands, int band_rows, int list_len) {
  constexpr int kRowsPerBatch = kMaxThreads <= 512 ? 16 : 8;
  __shared__ int s_cnt[4 * kMaxThreads];             // [column][band] change counts, then their exclusive prefix
  extern __shared__ uint16_t s_list[];               // [list_len][blockDim.x]: (row in band) << 4 | changed columns
  int* s_pos = reinterpret_cast<int*>(s_list + size_t(kListLen) * blockDim.x);   // [kPosLen] staged boundaries
  __shared__ int warp_tot[32];
  __shared__ int s_total;
  const long long n = blockIdx.x;
  const uint8_t* m = masks + n * (long long)H * W;
  int32_t* out = counts + n * (long long)cap;
  const int band = int(threadIdx.x) / col_threads;
  const int c0 = (int(threadIdx.x) - band * col_threads) * 4;
  const int y_begin = band * band_rows, y_end = min(H, y_begin + band_rows);
  const bool live = c0 < W && y_begin < H;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  // value before the first pixel of each of this thread's columns: the row above, or for the top band the bottom
  // of the column to the left; pixel (0,0) has no predecessor (its own value stands in: no change is seen there)
  uint32_t prev0 = 0;
  if (live) {
    if (band > 0) {
      prev0 = load_cols<kVec>(m + (long long)(y_begin - 1) * W, c0, W);
    } else {
      const uint8_t* last = m + (long long)(H - 1) * W;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = c0 + j;
        if (c < W) prev0 |= uint32_t(c == 0 ? __ldg(m) : __ldg(last + c - 1)) << (8 * j);
      }
    }
  }

  // ---- pass 1: changes per (column, band)
  int cnt[4] = {0, 0, 0, 0};
  int noted = 0;                                     // changed rows seen (may exceed list_len: then pass 2 walks again)
  if (live) {
    uint32_t prev = prev0, packed = 0;               // packed: four byte counters, flushed before they can wrap
    int since_flush = 0;
    for (int y0 = y_begin; y0 < y_end; y0 += kRowsPerBatch) {
      uint32_t cur[kRowsPerBatch];
#pragma unroll
      for (int r = 0; r < kRowsPerBatch; ++r)
        cur[r] = y0 + r < y_end ? load_cols<kVec>(m + (long long)(y0 + r) * W, c0, W) : 0u;
#pragma unroll
      for (int r = 0; r < kRowsPerBatch; ++r) {
        if (y0 + r < y_end) {
          const uint32_t chg = cur[r] ^ prev;
          packed += chg;
          if (chg != 0) {
            if (noted < list_len)
              s_list[noted * blockDim.x + threadIdx.x] = uint16_t(((y0 + r - y_begin) << 4) | ((chg * kNibbleMul) >> 24));
            ++noted;
          }
          prev = cur[r];
        }
      }
      since_flush += kRowsPerBatch;
      if (since_flush > 255 - kRowsPerBatch || y0 + kRowsPerBatch >= y_end) {
#pragma unroll
        for (int j = 0; j < 4; ++j) cnt[j] += (packed >> (8 * j)) & 0xffu;
        packed = 0;
        since_flush = 0;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) s_cnt[(c0 + j) * bands + band] = cnt[j];
  __syncthreads();

  // ---- exclusive scan of s_cnt (4 * blockDim.x entries, four consecutive ones per thread)
  int e[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) e[j] = s_cnt[4 * threadIdx.x + j];
  const int mine = e[0] + e[1] + e[2] + e[3];
  int incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    const int t = lane < nw ? warp_tot[lane] : 0;
    int ti = t;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, ti, o);
      if (lane >= o) ti += v;
    }
    warp_tot[lane] = ti - t;                         // exclusive warp offsets
    if (lane == 31) s_total = ti;
  }
  __syncthreads();
  {
    int run = warp_tot[warp] + incl - mine;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      s_cnt[4 * threadIdx.x + j] = run;
      run += e[j];
    }
  }
  __syncthreads();
  const int nchg = s_total;
  const int first = __ldg(m) != 0 ? 1 : 0;

  // ---- pass 2: column-major index of every change, at slot first + 1 + rank (slot `first` is index 0).
  // Masks with few enough boundaries stage them in shared memory (boundary k at s_pos[k]) and pass 3 writes the run
  // lengths in one coalesced sweep; the others go through the `counts` row itself.
  const bool staged = nchg + 1 <= kPosLen;
  if (threadIdx.x == 0) {
    if (first && cap > 0) out[0] = 0;
    if (staged) s_pos[0] = 0;
    else if (first < cap) out[first] = 0;
    n_counts[n] = first + nchg + 1;
  }
  if (live && noted != 0) {
    int slot[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) slot[j] = first + 1 + s_cnt[(c0 + j) * bands + band];
    if (noted <= list_len) {
      for (int i = 0; i < noted; ++i) {
        const uint32_t ent = s_list[i * blockDim.x + threadIdx.x];
        const int idx = c0 * H + y_begin + int(ent >> 4);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if ((ent >> j) & 1u) {
            if (staged) s_pos[slot[j] - first] = idx + j * H;
            else if (slot[j] < cap) out[slot[j]] = idx + j * H;
            ++slot[j];
          }
        }
      }
    } else {
      uint32_t prev = prev0;
      for (int y0 = y_begin; y0 < y_end; y0 += kRowsPerBatch) {
        uint32_t cur[kRowsPerBatch];
#pragma unroll
        for (int r = 0; r < kRowsPerBatch; ++r)
          cur[r] = y0 + r < y_end ? load_cols<kVec>(m + (long long)(y0 + r) * W, c0, W) : 0u;
#pragma unroll
        for (int r = 0; r < kRowsPerBatch; ++r) {
          if (y0 + r < y_end) {
            const uint32_t chg = cur[r] ^ prev;
            if (chg != 0) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                if ((chg >> (8 * j)) & 0xffu) {
                  if (staged) s_pos[slot[j] - first] = (c0 + j) * H + y0 + r;
                  else if (slot[j] < cap) out[slot[j]] = (c0 + j) * H + y0 + r;
                  ++slot[j];
                }
              }
            }
            prev = cur[r];
          }
        }
      }
    }
  }
  __syncthreads();

  // ---- pass 3: boundaries -> run lengths
  const int hw = H * W;
  if (staged) {
    for (int k = int(threadIdx.x); k <= nchg; k += int(blockDim.x))
      if (first + k < cap) out[first + k] = (k < nchg ? s_pos[k + 1] : hw) - s_pos[k];
    return;
  }
  // in place, a block-wide chunk at a time
  for (int base = 0; base <= nchg; base += int(blockDim.x)) {
    const int k = base + int(threadIdx.x);
    const bool ok = k <= nchg && first + k < cap;
    int a = 0, b = hw;
    if (ok) {
      a = out[first + k];
      if (k < nchg && first + k + 1 < cap) b = out[first + k + 1];
    }
    __syncthreads();
    if (ok) out[first + k] = b - a;
    __syncthreads();
  }
}

}  // namespace
}  // namespace samb

extern "C" int samb_mask_rle(const uint8_t* masks, int64_t N, int H, int W, int32_t* counts, int32_t* n_counts,
                             int cap, void* stream) {
  using namespace samb;
  if (masks == nullptr || counts == nullptr || n_counts == nullptr || N < 0 || H <= 0 || W <= 0 || cap < 0)
    return SAMB_E_BADARG;
  if (N > 0x7fffffffLL || (long long)H * W > 0x7fffffffLL || W > 4096) return SAMB_E_SHAPE;
  if (N == 0) return SAMB_OK;
  const int col_threads = (((W + 3) / 4) + 31) / 32 * 32;
  const int max_threads = col_threads <= 512 ? 512 : 1024;
  int bands = max_threads / col_threads;                       // row bands: fill the block, at least 32 rows each
  if (bands > (H + 31) / 32) bands = (H + 31) / 32;
  const int band_rows = (H + bands - 1) / bands;
  const int threads = col_threads * bands;
  auto st = static_cast<cudaStream_t>(stream);
  const bool vec = W % 4 == 0 && (reinterpret_cast<uintptr_t>(masks) & 3u) == 0;
  const int list_len = band_rows <= 4096 ? kListLen : 0;       // a list entry keeps 12 bits of row
  const size_t list_bytes = size_t(kListLen) * threads * sizeof(uint16_t) + size_t(kPosLen) * sizeof(int);
  auto kern = vec ? (max_threads == 512 ? mask_rle_kernel<true, 512> : mask_rle_kernel<true, 1024>)
                  : (max_threads == 512 ? mask_rle_kernel<false, 512> : mask_rle_kernel<false, 1024>);
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(size_t(kListLen) * 1024 * sizeof(uint16_t) + size_t(kPosLen) * sizeof(int))) !=
      cudaSuccess)
    return SAMB_E_LAUNCH;
  kern<<<unsigned(N), threads, list_bytes, st>>>(masks, H, W, counts, n_counts, cap, col_threads, bands, band_rows, list_len);
  return launch_status();
}
