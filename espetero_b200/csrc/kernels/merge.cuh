// The merge of split-K partial records, shared by attention_combine and the peer exchange kernel.
//
// A CTA of 256 threads serves a group of heads of one (job, row). A head is served by HD / 4
// threads (4 dims each) times n_slices record slices: slice k takes the records k, k + n_slices,
// ... so that many record loads are in flight at once (a single sequential walk over 64 records is
// latency-bound); passes with few records per job use fewer slices and put more heads in a CTA.
// The maximum M is found first by all threads of the head, so every slice weighs its records with
// the final e^(m_s - M); the slices' sums are then added in slice order through shared memory: no
// atomics, the result does not depend on scheduling. A record is HD + 2 floats long, so records
// are only 8-byte aligned: float2 accesses.
#pragma once

#include "common.cuh"

namespace esp {

constexpr int kCombineThreads = 256;

struct MergeScratch {
  float m[kCombineThreads / 32];
  float acc[kCombineThreads][5];
};

struct Merged {
  float4 acc;  // sum_s e^(m_s - M) O_s, this thread's 4 dims
  float M, L;
  bool owner;  // true on the threads of slice 0, which hold the result
};

__device__ __forceinline__ float4 ld_rec4(const float* p) {
  const float2 a = *reinterpret_cast<const float2*>(p), b = *reinterpret_cast<const float2*>(p + 2);
  return make_float4(a.x, a.y, b.x, b.y);
}

// rec0: record 0 of this thread's (row, head); records `stride` floats apart. Every thread of the
// CTA must call this (it synchronises the CTA twice), heads past H included (give them n = 0).
__device__ __forceinline__ Merged merge_records(const float* rec0, int n, size_t stride, int HD, int nsl, MergeScratch& sh) {
  const int tpd = HD / 4, tph = tpd * nsl;
  const int tid = threadIdx.x, hb = tid / tph, sl = (tid % tph) / tpd, d4 = tid % tpd;
  float M = -INFINITY;
  for (int s = tid % tph; s < n; s += tph) M = fmaxf(M, rec0[size_t(s) * stride + HD]);
#pragma unroll
  for (int o = 16; o; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
  if ((tid & 31) == 0) sh.m[tid >> 5] = M;
  __syncthreads();
  M = -INFINITY;
  for (int w = hb * (tph / 32); w < (hb + 1) * (tph / 32); ++w) M = fmaxf(M, sh.m[w]);
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
  float* mine = sh.acc[tid];
  mine[0] = acc.x, mine[1] = acc.y, mine[2] = acc.z, mine[3] = acc.w, mine[4] = L;
  __syncthreads();
  Merged out;
  out.owner = sl == 0;
  if (out.owner) {
    for (int k = 1; k < nsl; ++k) {  // fixed order
      const float* q = sh.acc[hb * tph + k * tpd + d4];
      acc.x += q[0], acc.y += q[1], acc.z += q[2], acc.w += q[3], L += q[4];
    }
  }
  out.acc = acc, out.M = M, out.L = L;
  return out;
}

// The unnormalised record [O | M | L] of a merge, written by the owner threads.
__device__ __forceinline__ void store_record(float* rec, const Merged& m, int HD, int d4) {
  *reinterpret_cast<float2*>(rec + 4 * d4) = make_float2(m.acc.x, m.acc.y);
  *reinterpret_cast<float2*>(rec + 4 * d4 + 2) = make_float2(m.acc.z, m.acc.w);
  if (d4 == 0) *reinterpret_cast<float2*>(rec + HD) = make_float2(m.M, m.L);
}

// Normalise, apply the output gate, convert and store one row's head; lse if asked for.
template <int QDT>
__device__ __forceinline__ void finish_row(const Merged& m, const float* X, void* O, float* lse, const esp_attn_params& p, int HD,
                                           int row, int h, int d4) {
  using QE = Elem16<QDT>;
  const float inv = m.L > 0.0f ? 1.0f / m.L : 0.0f;
  float o[4] = {m.acc.x * inv, m.acc.y * inv, m.acc.z * inv, m.acc.w * inv};
  if (X) {
    const float4 gt = *reinterpret_cast<const float4*>(X + size_t(row) * p.g_ld + size_t(h) * 2 * HD + HD + 4 * d4);
    o[0] *= sigmoid_gate(gt.x), o[1] *= sigmoid_gate(gt.y), o[2] *= sigmoid_gate(gt.z), o[3] *= sigmoid_gate(gt.w);
  }
  uint2 packed;
  packed.x = QE::pack2(o[0], o[1]);
  packed.y = QE::pack2(o[2], o[3]);
  *reinterpret_cast<uint2*>(static_cast<typename QE::T*>(O) + size_t(row) * p.q_ld + size_t(h) * HD + 4 * d4) = packed;
  if (lse && d4 == 0) lse[size_t(row) * p.H + h] = m.L > 0.0f ? m.M + __logf(m.L) : -INFINITY;
}

}  // namespace esp
