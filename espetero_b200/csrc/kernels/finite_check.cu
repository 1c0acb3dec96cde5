// NaN / Inf / outlier detector over a region, for debugging (sm_100a).
//
// The reference adds a finite_check dispatch after chosen dispatches when ESPETERO_CHECK_FINITE is
// set (src/model/impl/finite_check.h:4-18; kernel kernels/05_finite_check.metal; the attention
// output is the site "attn_out", src/model/impl/forest.h:4019-4047). Same record here - the number
// of offending elements, the smallest offending index (row * cols + col), a block counter and the
// first offender's value as fp32 bits - and the same rule: |x| bits >= thr_bits offend, so NaN and
// Inf always do (0x7F800000 = only those). Bit tests, not float compares.
#include "common.cuh"
#include "../launch.h"

namespace esp {
namespace {

__device__ __forceinline__ uint32_t element_bits(const uint8_t* x, size_t o, int dtype) {
  if (dtype == ESP_FINITE_F32) return reinterpret_cast<const uint32_t*>(x)[o];
  const uint32_t h = reinterpret_cast<const uint16_t*>(x)[o];
  if (dtype == ESP_FINITE_BF16) return h << 16;
  return __float_as_uint(__half2float(__ushort_as_half(uint16_t(h))));  // fp16: Inf / NaN widen to Inf / NaN
}

__global__ void finite_init_kernel(uint32_t* rec) {
  rec[0] = 0u, rec[1] = 0xFFFFFFFFu, rec[2] = 0u, rec[3] = 0u;
}

__global__ void __launch_bounds__(256) finite_check_kernel(const uint8_t* x, uint32_t* rec, uint32_t rows, uint32_t cols, uint64_t ld,
                                                            int dtype, uint32_t thr_bits) {
  const uint64_t n = uint64_t(rows) * cols;
  uint32_t first = 0xFFFFFFFFu, cnt = 0;
  for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += uint64_t(gridDim.x) * blockDim.x) {
    const uint32_t r = uint32_t(i / cols), c = uint32_t(i - uint64_t(r) * cols);
    const uint32_t b = element_bits(x, size_t(r) * ld + c, dtype) & 0x7FFFFFFFu;
    if (b >= thr_bits) {
      first = min(first, uint32_t(i));
      ++cnt;
    }
  }
  first = __reduce_min_sync(0xffffffffu, first);
  cnt = __reduce_add_sync(0xffffffffu, cnt);
  __shared__ uint32_t tf[8], tc[8];
  __shared__ bool last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) tf[warp] = first, tc[warp] = cnt;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t f = 0xFFFFFFFFu, k = 0;
    for (int s = 0; s < 8; ++s) f = min(f, tf[s]), k += tc[s];
    if (k) {
      atomicAdd(rec + 0, k);
      atomicMin(rec + 1, f);
    }
    __threadfence();
    last = atomicAdd(rec + 2, 1u) == gridDim.x - 1;
    if (last) {  // the last block: the first offender's value
      __threadfence();
      const uint32_t i = atomicAdd(rec + 1, 0u);
      if (i != 0xFFFFFFFFu) {
        const uint32_t r = i / cols, c = i - r * cols;
        rec[3] = element_bits(x, size_t(r) * ld + c, dtype);
      }
    }
  }
}

}  // namespace

cudaError_t launch_finite_check(const void* x, uint32_t rows, uint32_t cols, uint64_t ld, int dtype, uint32_t thr_bits, uint32_t* rec,
                                cudaStream_t stream, uint64_t* launches) {
  finite_init_kernel<<<1, 1, 0, stream>>>(rec);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const uint64_t n = uint64_t(rows) * cols;
  const unsigned grid = unsigned(std::min<uint64_t>(148 * 8, (n + 255) / 256));
  finite_check_kernel<<<std::max(1u, grid), 256, 0, stream>>>(static_cast<const uint8_t*>(x), rec, rows, cols, ld, dtype, thr_bits);
  e = cudaGetLastError();
  if (e == cudaSuccess && launches) *launches += 2;
  return e;
}

}  // namespace esp
