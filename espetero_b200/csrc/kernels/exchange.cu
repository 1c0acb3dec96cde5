// exchange_parts: the split-KV merge across the GPUs of one box in one kernel per rank.
//
// The reference runs on one GPU and ends a split-K pass with attention_combine
// (kernels/40_attention.metal:811-864). With one long sequence cut by KV range over several
// GPUs that merge has two levels; this kernel does both and the exchange between them:
//   step 1  merge this rank's records of a (job, row, head) into one unnormalised record
//   step 2  store it into slot `rank` of every rank's exchange buffer (plain stores through
//           peer mappings: NVLink), fence, publish flag (job, row, head) of this rank on every peer
//   step 3  wait until all ranks' flags of this CTA's heads carry the epoch, then merge the
//           `world` records in rank order from the local exchange buffer and finish the row.
// A CTA waits only for the CTAs that serve the same heads on the other GPUs; nothing waits on
// another CTA of its own GPU, and the whole grid is resident, so the wait cannot starve the
// publisher. The wait is bounded by a timer: on expiry the CTA writes the status word and returns
// without touching O.
#include "merge.cuh"
#include "../launch.h"

namespace esp {
namespace {

__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
// Records in the exchange buffer are written by other GPUs: read them past L1.
__device__ __forceinline__ float2 ld_cg2(const float* p) {
  float2 v;
  asm volatile("ld.global.cg.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "l"(p) : "memory");
  return v;
}

template <int QDT>
__global__ void __launch_bounds__(kCombineThreads) exchange_kernel(const ExchangeArgs x) {
  __shared__ MergeScratch scratch;
  __shared__ int all_here;
  const CombineArgs& a = x.c;
  const esp_attn_params& p = a.p;
  const int HD = a.HD, G = a.G, TR = a.tile_rows, H = p.H;
  const int tpd = HD / 4, tph = tpd * a.n_slices, hpb = kCombineThreads / tph;
  const int job_i = blockIdx.x / a.rows_max, r = blockIdx.x % a.rows_max;
  const int h0 = blockIdx.y * hpb, h = h0 + threadIdx.x / tph;
  const bool live_head = h < H;
  const int d4 = threadIdx.x % tpd, kvh = live_head ? h / G : 0, hg = live_head ? h % G : 0;
  const size_t stride = size_t(p.Hkv) * TR * G * (HD + 2);              // one record slot of all (kv head, row, head)
  const size_t rec_off = ((size_t(kvh) * TR + size_t(r)) * G + hg) * (HD + 2);
  const size_t rank_floats = size_t(a.n_jobs) * stride;                   // one rank's records in a buffer
  const size_t epoch_off = size_t(x.epoch & 1) * size_t(x.world) * rank_floats;
  const size_t flags_per_rank = size_t(a.n_jobs) * a.rows_max * H;
  const size_t flag0 = (size_t(job_i) * a.rows_max + r) * H;             // + head

  asm volatile("griddepcontrol.wait;" ::: "memory");
  const esp_attn_combine job = a.jobs[job_i];
  const bool live = live_head && r < job.rows;

  if (x.phases & 1) {
    const Merged m = merge_records(a.parts + size_t(job.part0) * stride + rec_off, live ? job.nparts : 0, stride, HD, a.n_slices, scratch);
    if (m.owner && live) {
      const size_t off = epoch_off + size_t(x.rank) * rank_floats + size_t(job_i) * stride + rec_off;
      for (int q = 0; q < x.world; ++q) store_record(x.records[q] + off, m, HD, d4);
    }
    __syncthreads();  // all record stores of the CTA are ordered before the fence below
    if (threadIdx.x < hpb * x.world) {
      const int q = threadIdx.x / hpb, hh = h0 + threadIdx.x % hpb;
      if (hh < H) {
        __threadfence_system();
        st_release_sys(x.flags[q] + size_t(x.rank) * flags_per_rank + flag0 + hh, x.epoch);
      }
    }
  }

  if (x.phases & 2) {
    if (threadIdx.x == 0) all_here = 1;
    __syncthreads();
    if (threadIdx.x < hpb * x.world) {
      const int q = threadIdx.x / hpb, hh = h0 + threadIdx.x % hpb;
      if (hh < H) {
        const unsigned long long* f = x.flags[x.rank] + size_t(q) * flags_per_rank + flag0 + hh;
        const uint64_t t0 = global_timer_ns();
        const uint64_t limit = uint64_t(x.wait_ms) * 1000000ull;
        bool ok = ld_acquire_sys(f) >= x.epoch;
        while (!ok) {
          __nanosleep(64);
          ok = ld_acquire_sys(f) >= x.epoch;
          if (!ok && global_timer_ns() - t0 > limit) break;
        }
        if (!ok) all_here = 0;
      }
    }
    __syncthreads();
    if (!all_here) {
      if (threadIdx.x == 0) atomicCAS(x.status, kStatusOk, kStatusPeerTimeout);
      return;
    }
    if (!live || (threadIdx.x % tph) / tpd != 0) return;
    // Second level: `world` records in rank order, one thread per 4 dims (at most 8 records).
    const float* rec0 = x.records[x.rank] + epoch_off + size_t(job_i) * stride + rec_off;
    float M = -INFINITY;
    for (int q = 0; q < x.world; ++q) M = fmaxf(M, ld_cg2(rec0 + size_t(q) * rank_floats + HD).x);
    Merged m;
    m.acc = make_float4(0.f, 0.f, 0.f, 0.f), m.M = M, m.L = 0.0f, m.owner = true;
    for (int q = 0; q < x.world; ++q) {
      const float* rec = rec0 + size_t(q) * rank_floats;
      const float2 ml = ld_cg2(rec + HD);
      const float w = (ml.x == -INFINITY) ? 0.0f : __expf(ml.x - M);
      const float2 o01 = ld_cg2(rec + 4 * d4), o23 = ld_cg2(rec + 4 * d4 + 2);
      m.L += w * ml.y;
      m.acc.x += w * o01.x, m.acc.y += w * o01.y, m.acc.z += w * o23.x, m.acc.w += w * o23.y;
    }
    finish_row<QDT>(m, a.X, a.O, a.lse, p, HD, job.r0 + r, h, d4);
  }
}

}  // namespace

cudaError_t launch_exchange(const ExchangeArgs& x, cudaStream_t stream, uint64_t* launches) {
  const CombineArgs& a = x.c;
  if (a.n_jobs <= 0) return cudaSuccess;
  cudaLaunchConfig_t cfg{};
  const int hpb = kCombineThreads / ((a.HD / 4) * a.n_slices);
  cfg.gridDim = dim3(unsigned(a.n_jobs) * unsigned(a.rows_max), unsigned((a.p.H + hpb - 1) / hpb));
  cfg.blockDim = dim3(kCombineThreads);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = a.q_dtype == ESP_F16 ? cudaLaunchKernelEx(&cfg, exchange_kernel<ESP_F16>, x)
                                       : cudaLaunchKernelEx(&cfg, exchange_kernel<ESP_BF16>, x);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e == cudaSuccess) ++*launches;
  return e;
}

// CTAs of the exchange grid; the caller refuses grids that cannot be resident at once.
int64_t exchange_grid_ctas(const CombineArgs& a) {
  const int hpb = kCombineThreads / ((a.HD / 4) * a.n_slices);
  return int64_t(a.n_jobs) * a.rows_max * ((a.p.H + hpb - 1) / hpb);
}

}  // namespace esp
