// esp_attn_decode_static: split-K decode for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc at the point where they run
// attention: an engine that hands the whole GPU to one pre-sized arena at start-up and
// forbids later allocations, a plugin loaded into a process whose allocator owns all of
// device memory, a real-time serving loop that treats any allocation (and the implicit
// device synchronisation cudaFree brings) as a latency fault. The regular path asks two
// things of them that they may not be able to give: a context (esp_attn_create allocates
// its status word) and a `parts` buffer for the split-K records. This entry point needs
// neither. The partial records live in a fixed array inside the library's device image,
// so the memory exists from the moment the library is loaded on a GPU until the process
// exits, on every GPU that loads it.
//
// It runs the same kernels as esp_attn_forward does for single-row trees (decode_gqa, then
// attention_combine) and gives bit-identical results; only the home of the records differs.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <climits>
#include <mutex>

#include "../host_util.h"
#include "../launch.h"

namespace {

// Capacity of the record array: 4 Mi floats = 16 MiB per GPU. A pass needs
// n_parts * Hkv * tile_rows * G * (HD + 2) floats (e.g. 32 records of the long-context
// FP8 decode, H32/Hkv8/HD256: 2.1 M floats).
constexpr size_t kStaticPartsFloats = size_t(ESP_ATTN_STATIC_PARTS_FLOATS);

static __device__ __align__(256) float g_static_parts[kStaticPartsFloats];
static __device__ __align__(256) int g_static_status[64] = {0};
// Arrival counters of the in-kernel merge; every pass leaves them at zero again.
static __device__ __align__(256) int g_static_counters[esp::kFixupCounters] = {0};

// In host code the two names above are only handles of the symbols, not device addresses;
// the addresses a kernel can use are looked up once per device and kept here.
struct DeviceSlot {
  std::atomic<bool> ready{false};
  float* parts = nullptr;
  int* status = nullptr;
  int* counters = nullptr;
  void* encode_tiled = nullptr;
};
constexpr int kMaxDevices = 64;
DeviceSlot g_slots[kMaxDevices];

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int cuda_fail(cudaError_t e, const char* what) {
  return esp::fail(ESP_ERR_CUDA, "esp_attn_decode_static: %s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
}

// First call on a device, with that device current: resolve the device addresses of the
// arrays, the tensor-map encoder, and raise the kernels' shared-memory limits. None of
// these calls allocates device memory.
int setup_device(int dev) {
  DeviceSlot& s = g_slots[dev];
  cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&s.parts), g_static_parts);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(records)");
  e = cudaGetSymbolAddress(reinterpret_cast<void**>(&s.status), g_static_status);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(status)");
  e = cudaGetSymbolAddress(reinterpret_cast<void**>(&s.counters), g_static_counters);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(counters)");
  cudaDriverEntryPointQueryResult q{};
  e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &s.encode_tiled, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !s.encode_tiled)
    return esp::fail(ESP_ERR_CUDA, "esp_attn_decode_static: cuTensorMapEncodeTiled not available from the driver");
  if ((e = esp::decode_gqa_setup()) != cudaSuccess) return cuda_fail(e, "decode kernel setup");
  s.ready.store(true, std::memory_order_release);
  return ESP_OK;
}

// Host threads may race to make the first call on a device: the set-up runs once, under a lock.
std::mutex g_setup_lock;
int ensure_device(int dev) {
  if (g_slots[dev].ready.load(std::memory_order_acquire)) return ESP_OK;
  std::lock_guard<std::mutex> hold(g_setup_lock);
  if (g_slots[dev].ready.load(std::memory_order_relaxed)) return ESP_OK;
  return setup_device(dev);
}

}  // namespace

extern "C" int esp_attn_decode_static(const esp_attn_shape* shape, void* stream_v, const esp_attn_args* args) {
  if (!shape || !args) return esp::fail(ESP_ERR_INVALID, "esp_attn_decode_static: null argument");
  const esp_attn_shape& s = *shape;
  const esp_attn_args& a = *args;
  const int TR = s.tile_rows > 0 ? s.tile_rows : 8;
  if (s.H <= 0 || s.Hkv <= 0 || s.H % s.Hkv) return esp::fail(ESP_ERR_INVALID, "esp_attn_decode_static: H=%d, Hkv=%d", s.H, s.Hkv);
  const int G = s.H / s.Hkv;
  const int esz = s.kv_dtype == ESP_E4M3 ? 1 : 2;
  if (!esp::decode_gqa_supports(s.HD, G, s.bt, s.q_dtype, s.kv_dtype) || !(s.scale > 0.0f))
    return esp::fail(ESP_ERR_UNSUPPORTED, "esp_attn_decode_static: shape outside the decode kernel (HD 64/128/256/512, G <= 8, bt %% 16 == 0)");
  if (a.n_tiles <= 0) return ESP_OK;
  if (!a.Q || !a.Kb || !a.Vb || !a.O || !a.kv || !a.blocks || !a.tiles || !a.trees || !a.tiles_host || !a.trees_host || a.n_blocks <= 0)
    return esp::fail(ESP_ERR_INVALID, "esp_attn_decode_static: null input / output / plan pointer");
  if (a.n_jobs > 0 && !a.jobs) return esp::fail(ESP_ERR_INVALID, "esp_attn_decode_static: combine jobs without a jobs array");
  if (s.kv_dtype == ESP_E4M3 && !a.kv_scales) return esp::fail(ESP_ERR_INVALID, "esp_attn_decode_static: E4M3 pool needs kv_scales");
  if ((s.flags & ESP_ATTN_FLAG_GATE) && !a.X) return esp::fail(ESP_ERR_INVALID, "esp_attn_decode_static: gate flag set but X is null");
  if (a.p.H != s.H || a.p.Hkv != s.Hkv || a.p.bt != s.bt || a.p.q_ld < s.H * s.HD || a.p.kv_ld < s.Hkv * s.HD ||
      (size_t(a.p.kv_ld) * esz) % 128 || (a.p.kv_base * esz) % 128)
    return esp::fail(ESP_ERR_INVALID, "esp_attn_decode_static: params do not match the shape");
  if (a.n_jobs > 0 && !a.jobs_host)
    return esp::fail(ESP_ERR_INVALID, "esp_attn_decode_static: combine jobs need their host copy (jobs_host): the records they name cannot be checked against the built-in array otherwise");
  for (int i = 0; i < a.n_trees; ++i)
    if (a.trees_host[i].M != 1) return esp::fail(ESP_ERR_UNSUPPORTED, "esp_attn_decode_static: tree %d has %d rows (decode only)", i, a.trees_host[i].M);
  // Records the pass touches: the largest one a tile writes or a combine job reads.
  int64_t top_part = 0;
  for (int i = 0; i < a.n_tiles; ++i) top_part = std::max<int64_t>(top_part, int64_t(a.tiles_host[i].part) + 1);
  for (int i = 0; i < a.n_jobs; ++i) {
    const esp_attn_combine& j = a.jobs_host[i];
    if (j.part0 < 0 || j.nparts < 1) return esp::fail(ESP_ERR_INVALID, "esp_attn_decode_static: job %d: records [%d, +%d)", i, j.part0, j.nparts);
    top_part = std::max<int64_t>(top_part, int64_t(j.part0) + j.nparts);
  }
  const size_t rec_floats = size_t(s.Hkv) * size_t(TR) * size_t(G) * size_t(s.HD + 2);
  const size_t need = size_t(top_part) * rec_floats;
  if (need > kStaticPartsFloats)
    return esp::fail(ESP_ERR_CAPACITY, "esp_attn_decode_static: the pass needs %zu floats of records, the built-in array holds %zu; use esp_attn_forward with a caller-owned parts buffer",
                     need, kStaticPartsFloats);

  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices) return esp::fail(ESP_ERR_UNSUPPORTED, "esp_attn_decode_static: device index %d", dev);
  if (int rc = ensure_device(dev)) return rc;
  const DeviceSlot& slot = g_slots[dev];

  // The same host checks esp_attn_forward makes (trees, tiles and jobs against the row, block-table
  // and record counts), with the built-in array standing in for the caller's parts buffer.
  {
    esp_attn_args chk = a;
    chk.parts = slot.parts;
    chk.n_parts = int32_t(std::min<size_t>(kStaticPartsFloats / rec_floats, size_t(INT32_MAX)));
    chk.anc_mask = nullptr;
    esp_attn_shape cs = s;
    cs.flags &= ~ESP_ATTN_FLAG_ANC_MASK;  // single-row trees have no batch keys to mask: desc is what the kernel gets
    if (!a.desc) chk.desc = reinterpret_cast<const int32_t*>(a.Q);  // never dereferenced by the decode kernel; only its presence is checked
    if (int rc = esp::validate_pass(cs, TR, true, chk)) return rc;
  }

  CUtensorMap map;
  {
    const cuuint64_t line_elems = 128 / esz;
    const cuuint64_t gdim[3] = {line_elems, cuuint64_t(a.n_blocks) * 2 * cuuint64_t(a.p.bt), cuuint64_t(a.p.kv_ld) * esz / 128};
    const cuuint64_t gstride[2] = {cuuint64_t(a.p.kv_ld) * esz, 128};
    const cuuint32_t box[3] = {cuuint32_t(line_elems), cuuint32_t(esp::kDecodeKeyBlock), cuuint32_t(s.HD * esz / 128)};
    const cuuint32_t estr[3] = {1, 1, 1};
    void* base = const_cast<uint8_t*>(static_cast<const uint8_t*>(a.kv)) + a.p.kv_base * esz;
    const CUresult r = reinterpret_cast<EncodeTiledFn>(slot.encode_tiled)(
        &map, esz == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, base, gdim, gstride, box, estr,
        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return esp::fail(ESP_ERR_CUDA, "esp_attn_decode_static: cuTensorMapEncodeTiled failed with CUresult %d", int(r));
  }

  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  uint64_t launches = 0;
  esp::KernelArgs k{};
  k.Q = a.Q, k.Kb = a.Kb, k.Vb = a.Vb, k.kv = a.kv, k.kv_scales = a.kv_scales, k.blocks = a.blocks;
  k.desc = a.desc, k.anc_mask = nullptr;
  k.X = (s.flags & ESP_ATTN_FLAG_GATE) ? a.X : nullptr;
  k.O = a.O, k.lse = a.lse, k.parts = slot.parts, k.tiles = a.tiles, k.trees = a.trees, k.status = slot.status;
  k.p = a.p, k.HD = s.HD, k.G = G, k.tile_rows = TR, k.n_tiles = a.n_tiles;
  k.q_dtype = s.q_dtype, k.kv_dtype = s.kv_dtype, k.n_blocks = a.n_blocks, k.scale = s.scale;
  k.n_trees = a.n_trees, k.n_block_entries = a.n_block_entries;
  k.pos = a.pos, k.window = a.window, k.ring = a.ring, k.bidi = a.bidi;
  // Nothing in the array has to be cleared first: every record the merge reads below is
  // written in full by the attention kernel of this same call.
  // Same choice as esp_attn_forward (identical bits): plans whose split tiles name their jobs are
  // merged by the attention kernel itself, others by the combine kernel.
  k.counters = slot.counters, k.jobs = a.jobs;
  k.fuse = esp::decode_fuse_small(a.n_tiles, s.Hkv, a.n_jobs, s.HD == 64 || (s.kv_dtype == ESP_E4M3 && s.HD == 128)) && G % 2 == 0 && a.n_jobs > 0 && a.jobs && esp::plan_fusable(a.tiles_host, a.n_tiles, a.jobs_host, a.n_jobs, s.Hkv);
  if ((e = esp::launch_decode_gqa(k, map, stream, &launches)) != cudaSuccess) return cuda_fail(e, "decode_gqa");
  if (a.n_jobs > 0 && !k.fuse) {
    esp::CombineArgs c{};
    c.parts = slot.parts, c.X = k.X, c.O = a.O, c.lse = a.lse, c.jobs = a.jobs, c.p = a.p;
    c.HD = s.HD, c.G = G, c.tile_rows = TR, c.n_jobs = a.n_jobs, c.q_dtype = s.q_dtype;
    c.rows_max = 1;  // decode: one row per job
    c.out_parts = nullptr, c.out_part0 = 0;
    int parts_max = 64;  // same slicing as esp_attn_forward, so that the two give identical bits
    if (a.jobs_host) {
      parts_max = 1;
      for (int i = 0; i < a.n_jobs; ++i) parts_max = a.jobs_host[i].nparts > parts_max ? a.jobs_host[i].nparts : parts_max;
    }
    c.n_slices = esp::combine_slices(s.HD, parts_max);
    if (a.jobs_host && a.n_jobs <= esp::kInlineJobsMax) {
      c.n_inline = a.n_jobs;
      for (int i = 0; i < a.n_jobs; ++i) c.inline_jobs[i] = a.jobs_host[i];
    }
    if ((e = esp::launch_combine(c, stream, &launches)) != cudaSuccess) return cuda_fail(e, "attention_combine");
  }
  return ESP_OK;
}

// Reads and clears the status word of the current device's built-in arrays: a bounded wait of the
// decode kernel that ran out (a TMA or bulk copy that never landed) leaves a code there, and the
// output of that pass is then not to be trusted. Also zeroes the merge's arrival counters, which a
// kernel that gave up may have left half counted. Synchronises the stream; allocates nothing.
extern "C" int esp_attn_decode_static_status(void* stream_v) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices) return esp::fail(ESP_ERR_UNSUPPORTED, "esp_attn_decode_static_status: device index %d", dev);
  if (!g_slots[dev].ready.load(std::memory_order_acquire)) return ESP_OK;  // nothing has run here yet
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  int st = 0;
  e = cudaMemcpyFromSymbolAsync(&st, g_static_status, sizeof(int), 0, cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return cuda_fail(e, "reading the status word");
  if (st == 0) return ESP_OK;
  cudaMemsetAsync(g_slots[dev].status, 0, sizeof(int) * 64, stream);
  cudaMemsetAsync(g_slots[dev].counters, 0, sizeof(int) * esp::kFixupCounters, stream);
  return esp::fail(ESP_ERR_CUDA, "esp_attn_decode_static: a kernel gave up a bounded wait (status %d: %s); the outputs of passes since the last check are not valid",
                   st, st == esp::kStatusTmaTimeout ? "a TMA or bulk copy never completed" : "unexpected code");
}
