// The merge of split-K partial records, shared by attention_combine and the peer exchange kernel.
//
// A CTA of 256 threads serves a group of heads of one (job, row). A head is served by HD / 4
// threads (4 dims each) times n_slices record slices: slice k takes the records k, k + n_slices,
// ... so that many record loads are in flight at once (a single sequential walk over 64 records is
// latency-bound); passes with few records per job use fewer slices and put more heads in a CTA.
// Every slice folds its records into a running (M, L, acc); the slices' results are then folded in
// slice order through shared memory: no atomics, the result does not depend on scheduling. A record is HD + 2 floats long, so records
// are only 8-byte aligned: float2 accesses.
#pragma once

#include "common.cuh"

namespace esp {

constexpr int kCombineThreads = 256;

struct MergeScratch {
  float acc[kCombineThreads][6];  // per thread: its slice's 4 dims, L and M
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
// CTA must call this (it synchronises the CTA once), heads past H included (give them n = 0).
// One pass: a slice loads up to eight of its records at once (one round trip to L2 for most
// passes), folds them into a running (M, L, acc) with the batch's maximum, and the slices are
// folded the same way in slice order by the threads of slice 0.
__device__ __forceinline__ Merged merge_records(const float* rec0, int n, size_t stride, int HD, int nsl, MergeScratch& sh) {
  const int tpd = HD / 4, tph = tpd * nsl;
  const int tid = threadIdx.x, hb = tid / tph, sl = (tid % tph) / tpd, d4 = tid % tpd;
  float M = -INFINITY, L = 0.0f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s = sl; s < n; s += 8 * nsl) {
    float2 ml[8];
    float4 o4[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int idx = s + i * nsl;
      ml[i] = make_float2(-INFINITY, 0.0f);
      o4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (idx < n) {
        const float* rec = rec0 + size_t(idx) * stride;
        ml[i] = *reinterpret_cast<const float2*>(rec + HD);
        o4[i] = ld_rec4(rec + 4 * d4);
      }
    }
    float bm = ml[0].x;
#pragma unroll
    for (int i = 1; i < 8; ++i) bm = fmaxf(bm, ml[i].x);
    if (bm > M) {  // rescale what has been summed so far (factor 0 the first time)
      const float f = __expf(M - bm);
      L *= f, acc.x *= f, acc.y *= f, acc.z *= f, acc.w *= f;
      M = bm;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float w = (ml[i].x == -INFINITY) ? 0.0f : __expf(ml[i].x - M);
      L += w * ml[i].y;
      acc.x += w * o4[i].x, acc.y += w * o4[i].y, acc.z += w * o4[i].z, acc.w += w * o4[i].w;
    }
  }
  Merged out;
  out.owner = sl == 0;
  if (nsl > 1) {
    float* mine = sh.acc[tid];
    mine[0] = acc.x, mine[1] = acc.y, mine[2] = acc.z, mine[3] = acc.w, mine[4] = L, mine[5] = M;
    __syncthreads();
    if (out.owner) {
      for (int k = 1; k < nsl; ++k) {  // fixed order
        const float* q = sh.acc[hb * tph + k * tpd + d4];
        const float mk = q[5];
        if (mk == -INFINITY) continue;
        if (mk > M) {
          const float f = __expf(M - mk);
          L *= f, acc.x *= f, acc.y *= f, acc.z *= f, acc.w *= f;
          M = mk;
        }
        const float w = __expf(mk - M);
        acc.x += w * q[0], acc.y += w * q[1], acc.z += w * q[2], acc.w += w * q[3], L += w * q[4];
      }
    }
  } else {
    __syncthreads();  // callers rely on one CTA-wide barrier inside
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
