// Qwen sparse attention, selection side (sm_100a): the top-512 blocks of every sparse row and the union
// lists of the 8-row tiles. Replaces qsa_select and qsa_tiles of the reference
// (kernels/45_qsa.metal:281-364, :366-450; host dispatch src/model/impl/forest.h:1586-1644). The
// attention over the lists is the general kernel (flash_general.cu: tiles with pad0 = 1).
//
// A query row at sequence index s sees n = s + 1 tokens; with nb = n / 4 complete blocks of 4 tokens it
// is sparse once nb > 512: it then attends the 512 blocks whose indexer scores are highest plus its tail
// (the tokens past 4 nb). Scores are fp32 >= 0, so their bit patterns order like the values: a 4-pass
// 8-bit radix select finds the 512th largest pattern; every block above it is taken, then the lowest-
// numbered blocks equal to it. All of this is integer work and bit-exact against the reference.
#include "common.cuh"
#include "../launch.h"

namespace esp {
namespace {

constexpr int kTopK = 512;  // blocks per sparse row (QSA_TOPK)

// Exclusive prefix sum of one value per thread over the CTA (threads in index order); *total = the sum.
template <int NT>
__device__ __forceinline__ uint32_t cta_exclusive_sum(uint32_t v, uint32_t* warp_sums, uint32_t* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  __syncthreads();  // warp_sums of the previous round have been read
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    const uint32_t t = lane < NT / 32 ? warp_sums[lane] : 0u;
    uint32_t in2 = t;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t n = __shfl_up_sync(0xffffffffu, in2, o);
      if (lane >= o) in2 += n;
    }
    if (lane < NT / 32) warp_sums[lane] = in2 - t;
    if (lane == 31) *total = in2;
  }
  __syncthreads();
  return warp_sums[warp] + incl - v;
}

// grid (sparse rows), 1024 threads. scores: [n_sparse][nbmax] fp32 >= 0; rinfo: int4 per pass row (s, nb, sparse row, tree);
// srows: the pass row of every sparse row; sel: [n_sparse][nbw] bitmap out.
__global__ void __launch_bounds__(1024) qsa_select_kernel(const float* scores, const int32_t* srows, const int32_t* rinfo, uint32_t* sel,
                                                           int nbmax, int nbw) {
  constexpr int NT = 1024;
  __shared__ uint32_t hist[256];
  __shared__ uint32_t sh[2];
  __shared__ uint32_t warp_sums[32];
  __shared__ uint32_t total;
  const int sr = blockIdx.x, tid = threadIdx.x;
  const int nb = min(max(rinfo[4 * size_t(srows[sr]) + 1], 0), nbmax);  // a bad record cannot run away
  const uint32_t* u = reinterpret_cast<const uint32_t*>(scores + size_t(sr) * nbmax);
  uint32_t prefix = 0, mask = 0, k = kTopK;
  for (int shift = 24; shift >= 0; shift -= 8) {
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    for (int b = tid; b < nb; b += NT) {
      const uint32_t v = u[b];
      if ((v & mask) == prefix) atomicAdd(&hist[(v >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      uint32_t cum = 0, bin = 0;
      for (int j = 255; j >= 0; --j) {
        const uint32_t h = hist[j];
        if (cum + h >= k) {
          bin = uint32_t(j);
          break;
        }
        cum += h;
      }
      sh[0] = prefix | (bin << shift);
      sh[1] = k - cum;
    }
    __syncthreads();
    prefix = sh[0], k = sh[1];
    mask |= 255u << shift;
    __syncthreads();
  }
  // every block above the threshold, then the lowest blocks equal to it until k are taken
  const int nw = (nb + 31) / 32;
  uint32_t running = 0;
  for (int w0 = 0; w0 < nbw; w0 += NT) {
    const int w = w0 + tid;
    uint32_t gt = 0, eq = 0;
    if (w < nw) {
      for (int bit = 0; bit < 32; ++bit) {
        const int b = w * 32 + bit;
        if (b >= nb) break;
        const uint32_t v = u[b];
        gt |= uint32_t(v > prefix) << bit;
        eq |= uint32_t(v == prefix) << bit;
      }
    }
    const uint32_t c = __popc(eq);
    const uint32_t before = running + cta_exclusive_sum<NT>(c, warp_sums, &total);
    uint32_t take = before >= k ? 0u : min(c, k - before);
    uint32_t word = gt;
    while (take > 0) {
      const uint32_t lo = eq & (~eq + 1u);
      word |= lo;
      eq ^= lo;
      --take;
    }
    if (w < nbw) sel[size_t(sr) * nbw + w] = word;
    running += total;
  }
}

// grid (tiles), 256 threads. Per tile the blocks holding cached tokens (b < ceil(P / 4)) that any of its rows reads,
// ascending, as (block << 8) | 8-bit row mask; tcount = entries (capped at lmax).
__global__ void __launch_bounds__(256) qsa_tiles_kernel(const uint32_t* sel, const esp_attn_tree* trees, const int32_t* rinfo, const esp_qsa_tile* qtiles,
                                                         uint32_t* tlist, uint32_t* tcount, int nbmax, int nbw, int lmax) {
  constexpr int NT = 256;
  __shared__ uint32_t warp_sums[32];
  __shared__ uint32_t total;
  const int tid = threadIdx.x;
  const esp_qsa_tile qt = qtiles[blockIdx.x];
  const esp_attn_tree T = trees[qt.tree];
  const int nbc = min(max((T.P + 3) / 4, 0), nbmax + 1);
  int srow[8], nbr[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    srow[k] = -2, nbr[k] = 0;  // no row
    if (k < qt.rows) {
      srow[k] = rinfo[4 * size_t(qt.r0 + k) + 2];
      nbr[k] = rinfo[4 * size_t(qt.r0 + k) + 1];
    }
  }
  const int nw = (nbc + 31) / 32;
  uint32_t running = 0;
  uint32_t* out = tlist + size_t(blockIdx.x) * lmax;
  for (int w0 = 0; w0 < nw; w0 += NT) {
    const int w = w0 + tid;
    uint32_t rw[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      uint32_t x = 0;
      if (w < nw) {
        if (srow[k] == -1) {
          x = 0xFFFFFFFFu;  // a row still dense reads every cached block
        } else if (srow[k] >= 0) {
          x = w < nbw ? sel[size_t(srow[k]) * nbw + w] : 0u;
          if (nbr[k] / 32 == w) x |= 1u << (nbr[k] % 32);  // the tail's block
        }
      }
      rw[k] = x;
    }
    const int lim = nbc - w * 32;
    const uint32_t vmask = w < nw ? (lim >= 32 ? 0xFFFFFFFFu : ((1u << uint32_t(max(lim, 0))) - 1u)) : 0u;
    uint32_t any = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) any |= rw[k];
    any &= vmask;
    const uint32_t c = __popc(any);
    uint32_t at = running + cta_exclusive_sum<NT>(c, warp_sums, &total);
    uint32_t a = any;
    while (a) {
      const int bit = __ffs(a) - 1;
      a &= a - 1u;
      uint32_t m8 = 0;
#pragma unroll
      for (int k = 0; k < 8; ++k) m8 |= ((rw[k] >> uint32_t(bit)) & 1u) << uint32_t(k);
      if (at < uint32_t(lmax)) out[at] = (uint32_t(w * 32 + bit) << 8) | m8;
      ++at;
    }
    running += total;
  }
  if (tid == 0) tcount[blockIdx.x] = min(running, uint32_t(lmax));
}

}  // namespace

cudaError_t launch_qsa_select(const float* scores, const int32_t* srows, const int32_t* rinfo, uint32_t* sel, int32_t n_sparse, int32_t nbmax,
                              int32_t nbw, cudaStream_t stream, uint64_t* launches) {
  if (n_sparse <= 0) return cudaSuccess;
  qsa_select_kernel<<<unsigned(n_sparse), 1024, 0, stream>>>(scores, srows, rinfo, sel, nbmax, nbw);
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess && launches) ++*launches;
  return e;
}

cudaError_t launch_qsa_tiles(const uint32_t* sel, const esp_attn_tree* trees, const int32_t* rinfo, const esp_qsa_tile* qtiles, int32_t n_qtiles,
                             uint32_t* tlist, uint32_t* tcount, int32_t nbmax, int32_t nbw, cudaStream_t stream, uint64_t* launches) {
  if (n_qtiles <= 0) return cudaSuccess;
  qsa_tiles_kernel<<<unsigned(n_qtiles), 256, 0, stream>>>(sel, trees, rinfo, qtiles, tlist, tcount, nbmax, nbw, ESP_QSA_LMAX);
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess && launches) ++*launches;
  return e;
}

}  // namespace esp
