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

namespace esp {
namespace {

// One CTA of 256 threads per (job row, group of heads). A head is served by HD / 4 threads (4 dims
// each) times n_slices record slices: slice k takes the records k, k + n_slices, ... so that many
// record loads are in flight at once (a single sequential walk over 64 records is latency-bound);
// passes with few records per job use fewer slices and put more heads in a CTA. The maximum M is
// found first by all threads of the head, so every slice weighs its records with the final
// e^(m_s - M); the slices' sums are then added in slice order through shared memory: no atomics,
// the result does not depend on scheduling. The grid covers only rows_max rows per job (1 for
// decode passes). A record is HD + 2 floats long, so records are only 8-byte aligned: float2 loads.
__device__ __forceinline__ float4 ld_rec4(const float* p) {
  const float2 a = *reinterpret_cast<const float2*>(p), b = *reinterpret_cast<const float2*>(p + 2);
  return make_float4(a.x, a.y, b.x, b.y);
}

constexpr int kCombineThreads = 256;

template <int QDT>
__global__ void __launch_bounds__(kCombineThreads) combine_kernel(const CombineArgs a) {
  using QE = Elem16<QDT>;
  __shared__ float red_m[kCombineThreads / 32];
  __shared__ float red_acc[kCombineThreads][5];
  const esp_attn_params& p = a.p;
  const int HD = a.HD, G = a.G, TR = a.tile_rows;
  const int tpd = HD / 4, nsl = a.n_slices;  // threads per record, record slices per head
  const int tph = tpd * nsl;                 // threads per head (a multiple of 32)
  const int job_i = blockIdx.x / a.rows_max, r = blockIdx.x % a.rows_max;
  const int hb = threadIdx.x / tph;          // head within the CTA
  const int h = blockIdx.y * (kCombineThreads / tph) + hb;
  // The records are written by the attention kernel launched just before on the same stream:
  // with programmatic dependent launch this grid may start early and waits here for them.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const esp_attn_combine job = a.jobs[job_i];
  if (r >= job.rows) return;
  const int tid = threadIdx.x, sl = (tid % tph) / tpd, d4 = tid % tpd;
  const int kvh = h / G, hg = h % G;
  const size_t stride = size_t(p.Hkv) * TR * G * (HD + 2);
  const float* rec0 = a.parts + ((size_t(job.part0) * p.Hkv + kvh) * TR * G + size_t(r) * G + hg) * (HD + 2);
  const int n = job.nparts;
  float M = -INFINITY;
  for (int s = tid % tph; s < n; s += tph) M = fmaxf(M, rec0[size_t(s) * stride + HD]);
#pragma unroll
  for (int o = 16; o; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
  if ((tid & 31) == 0) red_m[tid >> 5] = M;
  __syncthreads();
  M = -INFINITY;
  for (int w = hb * (tph / 32); w < (hb + 1) * (tph / 32); ++w) M = fmaxf(M, red_m[w]);
  float L = 0.0f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  int s = sl;
  for (; s + 3 * nsl < n; s += 4 * nsl) {
    float m4[4], l4[4];
    float4 o4[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float* rec = rec0 + size_t(s + i * nsl) * stride;
      m4[i] = rec[HD], l4[i] = rec[HD + 1];
      o4[i] = ld_rec4(rec + 4 * d4);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float w = (m4[i] == -INFINITY) ? 0.0f : __expf(m4[i] - M);
      L += w * l4[i];
      acc.x += w * o4[i].x, acc.y += w * o4[i].y, acc.z += w * o4[i].z, acc.w += w * o4[i].w;
    }
  }
  for (; s < n; s += nsl) {
    const float* rec = rec0 + size_t(s) * stride;
    const float w = (rec[HD] == -INFINITY) ? 0.0f : __expf(rec[HD] - M);
    const float4 o = ld_rec4(rec + 4 * d4);
    L += w * rec[HD + 1];
    acc.x += w * o.x, acc.y += w * o.y, acc.z += w * o.z, acc.w += w * o.w;
  }
  red_acc[tid][0] = acc.x, red_acc[tid][1] = acc.y, red_acc[tid][2] = acc.z, red_acc[tid][3] = acc.w, red_acc[tid][4] = L;
  __syncthreads();
  if (sl != 0) return;
  for (int k = 1; k < nsl; ++k) {  // fixed order
    const float* q = red_acc[hb * tph + k * tpd + d4];
    acc.x += q[0], acc.y += q[1], acc.z += q[2], acc.w += q[3], L += q[4];
  }
  if (a.out_parts) {
    // Reduce mode: the merged, still unnormalised record [O | M | L] of the job, for a second
    // merge level (records of other GPUs).
    float* rec = a.out_parts + ((size_t(a.out_part0 + job_i) * p.Hkv + kvh) * TR * G + size_t(r) * G + hg) * (HD + 2);
    *reinterpret_cast<float2*>(rec + 4 * d4) = make_float2(acc.x, acc.y);
    *reinterpret_cast<float2*>(rec + 4 * d4 + 2) = make_float2(acc.z, acc.w);
    if (d4 == 0) {
      rec[HD] = M;
      rec[HD + 1] = L;
    }
    return;
  }
  const int row = job.r0 + r;
  const float inv = L > 0.0f ? 1.0f / L : 0.0f;
  float o[4] = {acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv};
  if (a.X) {
    const float4 gt = *reinterpret_cast<const float4*>(a.X + size_t(row) * p.g_ld + size_t(h) * 2 * HD + HD + 4 * d4);
    o[0] *= sigmoid_gate(gt.x), o[1] *= sigmoid_gate(gt.y), o[2] *= sigmoid_gate(gt.z), o[3] *= sigmoid_gate(gt.w);
  }
  uint2 packed;
  packed.x = QE::pack2(o[0], o[1]);
  packed.y = QE::pack2(o[2], o[3]);
  *reinterpret_cast<uint2*>(static_cast<typename QE::T*>(a.O) + size_t(row) * p.q_ld + size_t(h) * HD + 4 * d4) = packed;
  if (a.lse && d4 == 0) a.lse[size_t(row) * p.H + h] = L > 0.0f ? M + __logf(L) : -INFINITY;
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
