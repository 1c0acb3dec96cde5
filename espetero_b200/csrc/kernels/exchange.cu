// exchange_parts: the split-KV merge across the GPUs of one box in one kernel per rank.
//
// The reference runs on one GPU and ends a split-K pass with attention_combine
// (kernels/40_attention.metal:811-864). With one long sequence cut by KV range over several
// GPUs that merge has two levels; this kernel does both and the exchange between them:
//   step 1  merge this rank's records of a (job, row, head) into one unnormalised record
//   step 2  store it into slot `rank` of every rank's exchange buffer through peer mappings
//           (NVLink) as 8-byte words {value, tag}: the tag is the call's epoch, so every word
//           says by itself whether it has arrived - no fence, no separate flag, one hop
//   step 3  read the `world` records from the local exchange buffer, polling the words (of all ranks
//           still missing at once) until they carry the tag, merge them in rank order and finish the row.
// A thread waits only for words that the same head's CTA on another GPU stores; nothing waits on
// another CTA of its own GPU, and the whole grid is resident, so the wait cannot starve the
// sender. The wait is bounded by a timer: on expiry the CTA writes the status word and returns
// without touching O.
#include "merge.cuh"
#include "../launch.h"

namespace esp {
namespace {

constexpr int kMaxRanks = ESP_ATTN_MAX_PEERS;  // slots of ExchangeArgs::records

template <int QDT>
__global__ void __launch_bounds__(kCombineThreads) exchange_kernel(const ExchangeArgs x) {
  __shared__ MergeScratch scratch;
  const CombineArgs& a = x.c;
  const esp_attn_params& p = a.p;
  const int HD = a.HD, G = a.G, TR = a.tile_rows, H = p.H;
  const int tpd = HD / 4, tph = tpd * a.n_slices, hpb = kCombineThreads / tph;
  const int job_i = blockIdx.x / a.rows_max, r = blockIdx.x % a.rows_max;
  const int h = blockIdx.y * hpb + threadIdx.x / tph;
  const bool live_head = h < H;
  const int d4 = threadIdx.x % tpd, kvh = live_head ? h / G : 0, hg = live_head ? h % G : 0;
  const size_t stride = size_t(p.Hkv) * TR * G * (HD + 2);              // one record slot of all (kv head, row, head)
  const size_t rec_off = ((size_t(kvh) * TR + size_t(r)) * G + hg) * (HD + 2);
  const size_t rank_words = size_t(a.n_jobs) * stride;                    // one rank's records in a buffer
  const size_t epoch_off = size_t(x.epoch & 1) * size_t(x.world) * rank_words;
  const uint32_t tag = uint32_t(x.epoch);

  const bool tracing = x.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0;
  if (tracing) x.trace[0] = global_timer_ns();  // CTA running (the attention kernel may still be draining)
  pdl_wait();
  if (tracing) x.trace[1] = global_timer_ns();  // the local records are complete
  const esp_attn_combine job = a.n_inline ? a.inline_jobs[job_i] : a.jobs[job_i];
  const bool live = live_head && r < job.rows;

  if (x.phases & 1) {
    const Merged m = merge_records(a.parts + size_t(job.part0) * stride + rec_off, live ? job.nparts : 0, stride, HD, a.n_slices, scratch);
    if (m.owner && live) {
      const size_t off = epoch_off + size_t(x.rank) * rank_words + size_t(job_i) * stride + rec_off;
      for (int q = 0; q < x.world; ++q) {
        uint2* dst = x.records[q] + off;
        st_word(dst + 4 * d4, m.acc.x, tag), st_word(dst + 4 * d4 + 1, m.acc.y, tag);
        st_word(dst + 4 * d4 + 2, m.acc.z, tag), st_word(dst + 4 * d4 + 3, m.acc.w, tag);
        if (d4 == 0) st_word(dst + HD, m.M, tag), st_word(dst + HD + 1, m.L, tag);
      }
    }
    if (tracing) x.trace[2] = global_timer_ns();  // merged and on its way to the peers
  }

  if (x.phases & 2) {
    // Second level: `world` records in rank order, one thread per 4 dims. Every word is polled
    // until it carries this call's tag (or the time runs out).
    const bool owner = live && (threadIdx.x % tph) / tpd == 0;
    bool ok = true;
    Merged m;
    m.acc = make_float4(0.f, 0.f, 0.f, 0.f), m.M = -INFINITY, m.L = 0.0f, m.owner = true;
    if (owner) {
      const uint2* rec0 = x.records[x.rank] + epoch_off + size_t(job_i) * stride + rec_off;
      const uint64_t t0 = global_timer_ns();
      const uint64_t limit = uint64_t(x.wait_ms) * 1000000ull;
      // Every look asks for the words of ALL ranks that are still missing at once (one trip to memory per look,
      // not one per rank); what has arrived is kept, and the merge below runs over the ranks in order.
      float v[kMaxRanks][6];
      uint32_t have = 0;
      const uint32_t every = x.world >= 32 ? ~0u : (1u << x.world) - 1u;
      for (;;) {
#pragma unroll
        for (int q = 0; q < kMaxRanks; ++q) {
          if (q < x.world && !((have >> q) & 1u)) {
            const uint2* rec = rec0 + size_t(q) * rank_words;
            uint2 w[6];
#pragma unroll
            for (int i = 0; i < 4; ++i) w[i] = ld_word(rec + 4 * d4 + i);
            w[4] = ld_word(rec + HD), w[5] = ld_word(rec + HD + 1);
            bool all = true;
#pragma unroll
            for (int i = 0; i < 6; ++i) all = all && w[i].y == tag;
            if (all) {
              have |= 1u << q;
#pragma unroll
              for (int i = 0; i < 6; ++i) v[q][i] = __uint_as_float(w[i].x);
            }
          }
        }
        if (have == every) break;
        if (global_timer_ns() - t0 > limit) {
          ok = false;
          break;
        }
        __nanosleep(32);
      }
#pragma unroll
      for (int q = 0; q < kMaxRanks; ++q) {
        if (!ok || q >= x.world) continue;
        const float m_q = v[q][4];
        if (m_q == -INFINITY) continue;  // an empty record adds nothing
        if (m_q > m.M) {                  // rescale what has been summed so far
          const float f = __expf(m.M - m_q);  // 0 for the first record
          m.L *= f, m.acc.x *= f, m.acc.y *= f, m.acc.z *= f, m.acc.w *= f;
          m.M = m_q;
        }
        const float wq = __expf(m_q - m.M);
        m.L += wq * v[q][5];
        m.acc.x += wq * v[q][0], m.acc.y += wq * v[q][1];
        m.acc.z += wq * v[q][2], m.acc.w += wq * v[q][3];
      }
    }
    if (tracing) x.trace[3] = global_timer_ns();  // every rank's records are here
    // Nobody writes O unless every thread of the CTA has all its words.
    if (!__syncthreads_and(ok)) {
      if (threadIdx.x == 0) atomicCAS(x.status, kStatusOk, kStatusPeerTimeout);
      return;
    }
    if (!owner) return;
    finish_row<QDT>(m, a.X, a.O, a.lse, p, HD, job.r0 + r, h, d4);
    if (tracing) x.trace[4] = global_timer_ns();
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
