// attention_combine, kv_save and kv_copy_blocks for sm_100a.
//
// attention_combine (kernels/40_attention.metal:811-864 of the reference; generic head
// dim kernels/80_gemma.metal:568-601): merges the split-K partial records of a row group,
// O = sum_s e^(m_s - M) O_s / sum_s e^(m_s - M) l_s, records summed in split order (no
// atomics: the result does not depend on scheduling), then the output gate.
// kv_save (:875-889) copies batch K/V rows into (block, pos) of the paged pool;
// kv_copy_blocks (:894-905) copies whole blocks in every layer region (copy-on-write).
#include "common.cuh"
#include "../launch.h"

#include "merge.cuh"

namespace esp {
namespace {

template <int QDT>
__global__ void __launch_bounds__(kCombineThreads) combine_kernel(const CombineArgs a) {
  __shared__ MergeScratch scratch;
  const esp_attn_params& p = a.p;
  const int HD = a.HD, G = a.G, TR = a.tile_rows;
  const int tpd = HD / 4, tph = tpd * a.n_slices;
  const int job_i = blockIdx.x / a.rows_max, r = blockIdx.x % a.rows_max;
  const int h = blockIdx.y * (kCombineThreads / tph) + threadIdx.x / tph;
  // The records are written by the attention kernel launched just before on the same stream:
  // with programmatic dependent launch this grid may start early and waits here for them.
  pdl_wait();
  pdl_launch_dependents();  // short CTAs: the next pass's grid may queue up behind them right away
  const esp_attn_combine job = a.n_inline ? a.inline_jobs[job_i] : a.jobs[job_i];
  if (r >= job.rows) return;
  const bool live = h < p.H;  // the last CTA of a row may reach past the heads
  const int d4 = threadIdx.x % tpd, kvh = live ? h / G : 0, hg = live ? h % G : 0;
  const size_t stride = size_t(p.Hkv) * TR * G * (HD + 2);
  const size_t rec_off = ((size_t(kvh) * TR + size_t(r)) * G + hg) * (HD + 2);
  const Merged m = merge_records(a.parts + size_t(job.part0) * stride + rec_off, live ? job.nparts : 0, stride, HD, a.n_slices, scratch);
  if (!m.owner || !live) return;
  if (a.out_parts) {
    // Reduce mode: the merged, still unnormalised record [O | M | L] of the job, for a second
    // merge level (records of other GPUs).
    store_record(a.out_parts + size_t(a.out_part0 + job_i) * stride + rec_off, m, HD, d4);
    return;
  }
  finish_row<QDT>(m, a.X, a.O, a.lse, p, HD, job.r0 + r, h, d4);
}

// 16 bytes per thread; grid (entries, ceil(kv_ld * 2 / 16 / 128)).
__global__ void kv_save_kernel16(const uint4* Kb, const uint4* Vb, uint4* kv, const esp_kv_save_entry* entries,
                                 const esp_attn_params p) {
  const int c = blockIdx.y * blockDim.x + threadIdx.x;  // 16-byte chunk of the row
  const int row_chunks = p.kv_ld / 8;
  if (c >= row_chunks) return;
  const esp_kv_save_entry e = entries[blockIdx.x];
  const size_t src = size_t(e.src_row) * row_chunks + c;
  const size_t blk = size_t(p.bt) * row_chunks;
  const size_t dst = p.kv_base / 8 + size_t(e.block) * 2 * blk + size_t(e.pos) * row_chunks + c;
  kv[dst] = Kb[src];
  kv[dst + blk] = Vb[src];
}

// E4M3 pool: 8 elements per thread, quantised with the destination block's scales.
template <int QDT>
__global__ void kv_save_kernel_e4m3(const uint4* Kb, const uint4* Vb, uint8_t* kv, const float* kv_scales,
                                    const esp_kv_save_entry* entries, const esp_attn_params p, int HD) {
  using QE = Elem16<QDT>;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;  // 8-element chunk of the row
  const int row_chunks = p.kv_ld / 8;
  if (c >= row_chunks) return;
  const esp_kv_save_entry e = entries[blockIdx.x];
  const int kvh = (c * 8) / HD;
  const size_t blk = size_t(p.bt) * p.kv_ld;
  const size_t dst = p.kv_base + size_t(e.block) * 2 * blk + size_t(e.pos) * p.kv_ld + size_t(c) * 8;
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    const uint4 v = (which ? Vb : Kb)[size_t(e.src_row) * row_chunks + c];
    const float sc = kv_scales[(size_t(e.block) * 2 + which) * p.Hkv + kvh];
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint8_t out[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = QE::unpack2(w[i]);
      // division, not multiplication by the reciprocal, so that the codes match a host
      // quantiser that divides
      out[2 * i] = f32_to_e4m3(__fdiv_rn(f.x, sc));
      out[2 * i + 1] = f32_to_e4m3(__fdiv_rn(f.y, sc));
    }
    *reinterpret_cast<uint2*>(kv + dst + which * blk) = *reinterpret_cast<const uint2*>(out);
  }
}

// One thread widens 8 codes: grid (8-element chunks of a block's K + V rows / 256, entries).
template <int QDT>
__global__ void kv_dequant_kernel(const uint8_t* kv, const float* kv_scales, const int32_t* blocks, uint4* out, int32_t* identity,
                                  const esp_attn_params p, int HD, int n_blocks) {
  using QE = Elem16<QDT>;
  const int e = blockIdx.y;
  const size_t row_chunks = size_t(p.kv_ld) / 8, half_chunks = size_t(p.bt) * row_chunks;  // K rows, then V rows
  const size_t c = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (c == 0) identity[e] = e;
  if (c >= 2 * half_chunks) return;
  const int b = blocks[e];
  if (b < 0 || b >= n_blocks) return;  // an entry no tile reads (validated plans never name it)
  const int which = c >= half_chunks;
  const int col = int(c % row_chunks) * 8, kvh = col / HD;
  const float sc = kv_scales[(size_t(b) * 2 + which) * p.Hkv + kvh];
  const uint2 codes = *reinterpret_cast<const uint2*>(kv + p.kv_base + size_t(b) * 2 * half_chunks * 8 + c * 8);
  const uint32_t w[2] = {codes.x, codes.y};
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t pair = (w[i >> 1] >> (16 * (i & 1))) & 0xFFFFu;
    const uint32_t h2 = e4m3x2_to_f16x2(uint16_t(pair));  // exact
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h2));
    o[i] = QE::pack2(f.x * sc, f.y * sc);
  }
  out[size_t(e) * 2 * half_chunks + c] = make_uint4(o[0], o[1], o[2], o[3]);
}

// grid (chunks of a block pair, pairs, layers); 16 bytes per thread.
__global__ void kv_copy_blocks_kernel(uint4* kv, const int2* pairs, size_t blk2_chunks, size_t region_chunks) {
  const size_t c = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (c >= blk2_chunks) return;
  const int2 pr = pairs[blockIdx.y];
  uint4* base = kv + size_t(blockIdx.z) * region_chunks;
  base[size_t(pr.y) * blk2_chunks + c] = base[size_t(pr.x) * blk2_chunks + c];
}

}  // namespace

cudaError_t launch_combine(const CombineArgs& a, cudaStream_t stream, uint64_t* launches) {
  if (a.n_jobs <= 0) return cudaSuccess;
  // Programmatic dependent launch: the grid may be scheduled while the attention kernel before
  // it drains; griddepcontrol.wait in the kernel orders it after that kernel's writes.
  cudaLaunchConfig_t cfg{};
  const int hpb = kCombineThreads / ((a.HD / 4) * a.n_slices);  // heads per CTA
  cfg.gridDim = dim3(unsigned(a.n_jobs) * unsigned(a.rows_max), unsigned((a.p.H + hpb - 1) / hpb));
  cfg.blockDim = dim3(kCombineThreads);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = a.q_dtype == ESP_F16 ? cudaLaunchKernelEx(&cfg, combine_kernel<ESP_F16>, a)
                                       : cudaLaunchKernelEx(&cfg, combine_kernel<ESP_BF16>, a);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e == cudaSuccess) ++*launches;
  return e;
}

cudaError_t launch_kv_save(const void* Kb, const void* Vb, void* kv, const float* kv_scales, const esp_kv_save_entry* entries,
                           int32_t n, const esp_attn_params& p, int32_t HD, int32_t q_dtype, int32_t kv_dtype,
                           cudaStream_t stream, uint64_t* launches) {
  if (n <= 0) return cudaSuccess;
  const int row_chunks = p.kv_ld / 8;
  const dim3 block(128), grid(unsigned(n), unsigned((row_chunks + 127) / 128));
  if (kv_dtype == ESP_E4M3) {
    if (q_dtype == ESP_F16)
      kv_save_kernel_e4m3<ESP_F16><<<grid, block, 0, stream>>>(static_cast<const uint4*>(Kb), static_cast<const uint4*>(Vb),
                                                             static_cast<uint8_t*>(kv), kv_scales, entries, p, HD);
    else
      kv_save_kernel_e4m3<ESP_BF16><<<grid, block, 0, stream>>>(static_cast<const uint4*>(Kb), static_cast<const uint4*>(Vb),
                                                              static_cast<uint8_t*>(kv), kv_scales, entries, p, HD);
  } else {
    kv_save_kernel16<<<grid, block, 0, stream>>>(static_cast<const uint4*>(Kb), static_cast<const uint4*>(Vb),
                                                 static_cast<uint4*>(kv), entries, p);
  }
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) ++*launches;
  return e;
}

cudaError_t launch_kv_dequant(const void* kv, const float* kv_scales, const int32_t* blocks, int32_t n_entries, void* out,
                              int32_t* identity, const esp_attn_params& p, int32_t HD, int32_t n_blocks, int32_t q_dtype,
                              cudaStream_t stream, uint64_t* launches) {
  if (n_entries <= 0) return cudaSuccess;
  const size_t chunks = 2 * size_t(p.bt) * size_t(p.kv_ld) / 8;
  const dim3 grid(unsigned((chunks + 255) / 256), unsigned(n_entries));
  if (q_dtype == ESP_F16)
    kv_dequant_kernel<ESP_F16><<<grid, 256, 0, stream>>>(static_cast<const uint8_t*>(kv), kv_scales, blocks, static_cast<uint4*>(out), identity, p, HD, n_blocks);
  else
    kv_dequant_kernel<ESP_BF16><<<grid, 256, 0, stream>>>(static_cast<const uint8_t*>(kv), kv_scales, blocks, static_cast<uint4*>(out), identity, p, HD, n_blocks);
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) ++*launches;
  return e;
}

cudaError_t launch_kv_copy_blocks(void* kv, const int32_t* pairs, int32_t n_pairs, const esp_attn_params& p,
                                  uint64_t region_elems, int32_t n_layers, int32_t elem_bytes, cudaStream_t stream,
                                  uint64_t* launches) {
  if (n_pairs <= 0 || n_layers <= 0) return cudaSuccess;
  const size_t blk2_chunks = 2 * size_t(p.bt) * p.kv_ld * elem_bytes / 16;
  const size_t region_chunks = size_t(region_elems) * elem_bytes / 16;
  const dim3 block(128), grid(unsigned((blk2_chunks + 127) / 128), unsigned(n_pairs), unsigned(n_layers));
  kv_copy_blocks_kernel<<<grid, block, 0, stream>>>(static_cast<uint4*>(kv), reinterpret_cast<const int2*>(pairs), blk2_chunks,
                                                    region_chunks);
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) ++*launches;
  return e;
}

}  // namespace esp
