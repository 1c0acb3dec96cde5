// Checkpoint files of a sequence's KV blocks, in the reference's layout.
//
// Reference: slot_save / slot_load, src/model/model.mm:604-740. A file is a CkptHeader
// (magic "CPKU", version 4) followed by the sequence's KV blocks layer-major (for every layer,
// the blocks in the order of the sequence's block list, each `block_bytes` long: K rows then V
// rows), then the sections of other subsystems (linear-layer state, MTP rows, n-gram state,
// sparse-attention index blocks, sliding-window rings). This path owns only the KV blocks: it
// writes the other sections with zero counts and refuses files that carry them.
//
// E4M3 pools (an extension: the reference has no FP8 KV cache) need the blocks' scales as well,
// or a loaded sequence would decode with the scales of whatever used its new blocks before. Such a
// file carries one more section behind the blocks - for every layer, for every block of the list,
// its 2 * Hkv fp32 scales (K row, V row) - and announces it in the header word the reference leaves
// at zero (`pad` = scale bytes per block and layer). The reference refuses such a file by its size.
//
// On the GPU the blocks of a layer are scattered over the pool: a kernel gathers them into a
// contiguous staging buffer (or scatters them from it), the staging buffer crosses PCIe in one
// copy per chunk of up to 64 MB, and the host reads / writes the file sequentially.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

#include "../../include/espetero_attn.h"
#include "host_util.h"

namespace {

// Byte layout of the reference's header (model.mm:604-614); 120 bytes.
struct CkptHeader {
  uint32_t magic, version;
  int32_t len, next_pos, mtp_ok, n_lh, mh_pos[3];
  int32_t n_blocks, n_layers, n_linear;
  uint64_t block_bytes, conv_bytes, st_bytes, mtp_bytes, ple_bytes;
  int32_t i_layers, pad;
  uint64_t iblock_bytes;
  int32_t r_layers, r_blocks;
  uint64_t rblock_bytes;
};
static_assert(sizeof(CkptHeader) == 120, "checkpoint header layout");
constexpr uint32_t kMagic = 0x554b5043u;
constexpr uint32_t kVersion = 4;
constexpr size_t kChunkBytes = size_t(64) << 20;

// grid (16-byte chunks of a block / 256, blocks of the chunk); to_staging: pool -> staging, else back.
__global__ void gather_blocks_kernel(uint4* pool_layer, uint4* staging, const int32_t* blocks, size_t block_chunks, int to_staging) {
  const size_t c = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (c >= block_chunks) return;
  uint4* in_pool = pool_layer + size_t(blocks[blockIdx.y]) * block_chunks + c;
  uint4* in_stage = staging + size_t(blockIdx.y) * block_chunks + c;
  if (to_staging) *in_stage = *in_pool;
  else *in_pool = *in_stage;
}

// grid (blocks); thread t copies float t of the block's 2 * Hkv scales.
__global__ void gather_scales_kernel(float* table_layer, float* staging, const int32_t* blocks, int per_block, int to_staging) {
  float* in_table = table_layer + size_t(blocks[blockIdx.x]) * per_block;
  float* in_stage = staging + size_t(blockIdx.x) * per_block;
  for (int i = threadIdx.x; i < per_block; i += blockDim.x) {
    if (to_staging) in_stage[i] = in_table[i];
    else in_table[i] = in_stage[i];
  }
}

struct Staging {
  void* dev = nullptr;
  void* host = nullptr;
  int32_t* dev_blocks = nullptr;
  ~Staging() {
    if (dev) cudaFree(dev);
    if (host) cudaFreeHost(host);
    if (dev_blocks) cudaFree(dev_blocks);
  }
};

int cuda_fail(cudaError_t e, const char* what) {
  return esp::fail(ESP_ERR_CUDA, "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
}

// Moves the blocks of every layer between the pool and the file, a chunk of blocks at a time.
int move_blocks(FILE* f, bool save, cudaStream_t stream, void* kv, const int32_t* blocks, int32_t nb, int32_t n_layers,
                uint64_t region_bytes, uint64_t block_bytes) {
  if (nb == 0 || n_layers == 0) return ESP_OK;
  const int32_t per_chunk = int32_t(std::max<uint64_t>(1, std::min<uint64_t>(uint64_t(nb), kChunkBytes / block_bytes)));
  Staging st;
  cudaError_t e = cudaMalloc(&st.dev, size_t(per_chunk) * block_bytes);
  if (e == cudaSuccess) e = cudaMallocHost(&st.host, size_t(per_chunk) * block_bytes);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&st.dev_blocks), sizeof(int32_t) * size_t(nb));
  if (e == cudaSuccess) e = cudaMemcpyAsync(st.dev_blocks, blocks, sizeof(int32_t) * size_t(nb), cudaMemcpyHostToDevice, stream);
  if (e != cudaSuccess) return cuda_fail(e, "checkpoint staging buffers");
  const size_t block_chunks = block_bytes / 16;
  for (int32_t l = 0; l < n_layers; ++l) {
    uint4* layer = reinterpret_cast<uint4*>(static_cast<uint8_t*>(kv) + uint64_t(l) * region_bytes);
    for (int32_t b0 = 0; b0 < nb; b0 += per_chunk) {
      const int32_t n = std::min(per_chunk, nb - b0);
      const size_t bytes = size_t(n) * block_bytes;
      const dim3 grid(unsigned((block_chunks + 255) / 256), unsigned(n));
      if (save) {
        gather_blocks_kernel<<<grid, 256, 0, stream>>>(layer, static_cast<uint4*>(st.dev), st.dev_blocks + b0, block_chunks, 1);
        if ((e = cudaGetLastError()) == cudaSuccess) e = cudaMemcpyAsync(st.host, st.dev, bytes, cudaMemcpyDeviceToHost, stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
        if (e != cudaSuccess) return cuda_fail(e, "checkpoint gather");
        if (std::fwrite(st.host, 1, bytes, f) != bytes) return esp::fail(ESP_ERR_INVALID, "checkpoint: short write");
      } else {
        if (std::fread(st.host, 1, bytes, f) != bytes) return esp::fail(ESP_ERR_INVALID, "checkpoint: short read");
        e = cudaMemcpyAsync(st.dev, st.host, bytes, cudaMemcpyHostToDevice, stream);
        if (e == cudaSuccess) {
          gather_blocks_kernel<<<grid, 256, 0, stream>>>(layer, static_cast<uint4*>(st.dev), st.dev_blocks + b0, block_chunks, 0);
          e = cudaGetLastError();
        }
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream);  // the staging buffers are reused by the next chunk
        if (e != cudaSuccess) return cuda_fail(e, "checkpoint scatter");
      }
    }
  }
  return ESP_OK;
}

// The scale rows of an E4M3 pool's blocks, layer-major, behind the blocks.
int move_scales(FILE* f, bool save, cudaStream_t stream, float* scales, const int32_t* blocks, int32_t nb, int32_t n_layers,
                uint64_t region_floats, int32_t per_block) {
  if (nb == 0 || n_layers == 0) return ESP_OK;
  Staging st;
  const size_t bytes = size_t(nb) * per_block * sizeof(float);
  cudaError_t e = cudaMalloc(&st.dev, bytes);
  if (e == cudaSuccess) e = cudaMallocHost(&st.host, bytes);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&st.dev_blocks), sizeof(int32_t) * size_t(nb));
  if (e == cudaSuccess) e = cudaMemcpyAsync(st.dev_blocks, blocks, sizeof(int32_t) * size_t(nb), cudaMemcpyHostToDevice, stream);
  if (e != cudaSuccess) return cuda_fail(e, "checkpoint staging buffers (scales)");
  for (int32_t l = 0; l < n_layers; ++l) {
    float* layer = scales + uint64_t(l) * region_floats;
    if (save) {
      gather_scales_kernel<<<unsigned(nb), 64, 0, stream>>>(layer, static_cast<float*>(st.dev), st.dev_blocks, per_block, 1);
      if ((e = cudaGetLastError()) == cudaSuccess) e = cudaMemcpyAsync(st.host, st.dev, bytes, cudaMemcpyDeviceToHost, stream);
      if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
      if (e != cudaSuccess) return cuda_fail(e, "checkpoint gather (scales)");
      if (std::fwrite(st.host, 1, bytes, f) != bytes) return esp::fail(ESP_ERR_INVALID, "checkpoint: short write");
    } else {
      if (std::fread(st.host, 1, bytes, f) != bytes) return esp::fail(ESP_ERR_INVALID, "checkpoint: short read");
      e = cudaMemcpyAsync(st.dev, st.host, bytes, cudaMemcpyHostToDevice, stream);
      if (e == cudaSuccess) {
        gather_scales_kernel<<<unsigned(nb), 64, 0, stream>>>(layer, static_cast<float*>(st.dev), st.dev_blocks, per_block, 0);
        e = cudaGetLastError();
      }
      if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
      if (e != cudaSuccess) return cuda_fail(e, "checkpoint scatter (scales)");
    }
  }
  return ESP_OK;
}

}  // namespace

extern "C" {

int esp_kv_slot_save(const char* path, void* stream, const void* kv, const int32_t* blocks_host, int32_t len, int32_t next_pos,
                     int32_t bt, int32_t n_layers, uint64_t region_bytes, uint64_t block_bytes, const float* kv_scales, int32_t Hkv,
                     uint64_t scales_region_floats) {
  if (!path || !kv || len < 0 || bt <= 0 || n_layers <= 0 || block_bytes == 0 || block_bytes % 16 || region_bytes % 16)
    return esp::fail(ESP_ERR_INVALID, "esp_kv_slot_save: bad argument (block and region sizes are multiples of 16 bytes)");
  if (kv_scales && (Hkv <= 0 || Hkv > (1 << 20))) return esp::fail(ESP_ERR_INVALID, "esp_kv_slot_save: scales given but Hkv=%d", Hkv);
  if (kv_scales)
    for (int32_t i = 0; i < (len + bt - 1) / bt; ++i)
      if (blocks_host && blocks_host[i] >= 0 && uint64_t(blocks_host[i] + 1) * 2 * uint64_t(Hkv) > scales_region_floats)
        return esp::fail(ESP_ERR_INVALID, "esp_kv_slot_save: block %d has no row in a scale table of %llu floats per layer", blocks_host[i],
                         (unsigned long long)scales_region_floats);
  const int32_t nb = (len + bt - 1) / bt;
  if (nb > 0 && !blocks_host) return esp::fail(ESP_ERR_INVALID, "esp_kv_slot_save: null block list");
  for (int32_t i = 0; i < nb; ++i)
    if (blocks_host[i] < 0 || uint64_t(blocks_host[i] + 1) * block_bytes > region_bytes)
      return esp::fail(ESP_ERR_INVALID, "esp_kv_slot_save: block %d (entry %d) outside the layer region", blocks_host[i], i);
  CkptHeader h{};
  h.magic = kMagic, h.version = kVersion, h.len = len, h.next_pos = next_pos;
  h.n_blocks = nb, h.n_layers = n_layers, h.block_bytes = block_bytes;
  h.pad = kv_scales ? int32_t(2 * Hkv * sizeof(float)) : 0;  // E4M3 pools: a scale section follows the blocks
  FILE* f = std::fopen(path, "wb");
  if (!f) return esp::fail(ESP_ERR_INVALID, "esp_kv_slot_save: cannot open %s for writing", path);
  int rc = std::fwrite(&h, 1, sizeof(h), f) == sizeof(h) ? ESP_OK : esp::fail(ESP_ERR_INVALID, "esp_kv_slot_save: short write");
  if (rc == ESP_OK)
    rc = move_blocks(f, true, static_cast<cudaStream_t>(stream), const_cast<void*>(kv), blocks_host, nb, n_layers, region_bytes, block_bytes);
  if (rc == ESP_OK && kv_scales)
    rc = move_scales(f, true, static_cast<cudaStream_t>(stream), const_cast<float*>(kv_scales), blocks_host, nb, n_layers, scales_region_floats, 2 * Hkv);
  if (std::fclose(f) != 0 && rc == ESP_OK) rc = esp::fail(ESP_ERR_INVALID, "esp_kv_slot_save: close failed");
  return rc;
}

int esp_kv_slot_load(const char* path, void* stream, void* kv, esp_kv_pool* pool, int32_t* blocks_out, int32_t blocks_cap,
                     int32_t* n_blocks, int32_t* len, int32_t* next_pos, int32_t bt, int32_t n_layers, uint64_t region_bytes,
                     uint64_t block_bytes, float* kv_scales, int32_t Hkv, uint64_t scales_region_floats) {
  if (!path || !kv || !pool || !n_blocks || !len || !next_pos || bt <= 0 || n_layers <= 0 || block_bytes == 0 || block_bytes % 16 || region_bytes % 16)
    return esp::fail(ESP_ERR_INVALID, "esp_kv_slot_load: bad argument");
  FILE* f = std::fopen(path, "rb");
  if (!f) return esp::fail(ESP_ERR_INVALID, "esp_kv_slot_load: cannot open %s", path);
  struct Closer {
    FILE* f;
    ~Closer() { std::fclose(f); }
  } closer{f};
  CkptHeader h;
  if (std::fread(&h, 1, sizeof(h), f) != sizeof(h)) return esp::fail(ESP_ERR_INVALID, "esp_kv_slot_load: no header");
  // The reference's checks (model.mm:668-676), for the sections this path owns; the others must be empty.
  if (h.magic != kMagic || h.version != kVersion) return esp::fail(ESP_ERR_INVALID, "esp_kv_slot_load: not a version-%u checkpoint", kVersion);
  if (h.n_layers != n_layers || h.block_bytes != block_bytes)
    return esp::fail(ESP_ERR_INVALID, "esp_kv_slot_load: the file holds %d layers of %llu-byte blocks, the pool %d of %llu", h.n_layers,
                     (unsigned long long)h.block_bytes, n_layers, (unsigned long long)block_bytes);
  if (h.n_linear || h.conv_bytes || h.st_bytes || h.mtp_bytes || h.ple_bytes || h.i_layers || h.iblock_bytes || h.r_layers || h.r_blocks ||
      h.rblock_bytes)
    return esp::fail(ESP_ERR_UNSUPPORTED, "esp_kv_slot_load: the file carries state of other subsystems (linear layers, MTP, index blocks or rings)");
  if (h.n_blocks < 0 || h.len < 0 || int64_t(h.len) > int64_t(h.n_blocks) * bt) return esp::fail(ESP_ERR_INVALID, "esp_kv_slot_load: inconsistent lengths");
  // The scale section of an E4M3 pool: file and pool must agree on having one, and on its row size.
  const int32_t want_pad = kv_scales ? int32_t(2 * Hkv * sizeof(float)) : 0;
  if (kv_scales && Hkv <= 0) return esp::fail(ESP_ERR_INVALID, "esp_kv_slot_load: scales given but Hkv=%d", Hkv);
  if (h.pad != want_pad)
    return esp::fail(ESP_ERR_INVALID, "esp_kv_slot_load: the file carries %d bytes of block scales per block and layer, the pool expects %d (E4M3 pools have them, 16-bit pools do not)",
                     h.pad, want_pad);
  const uint64_t need = sizeof(h) + uint64_t(h.n_blocks) * uint64_t(h.n_layers) * (h.block_bytes + uint64_t(h.pad));
  if (std::fseek(f, 0, SEEK_END) != 0 || uint64_t(std::ftell(f)) != need) return esp::fail(ESP_ERR_INVALID, "esp_kv_slot_load: file size does not match its header");
  std::fseek(f, long(sizeof(h)), SEEK_SET);
  if (h.n_blocks > blocks_cap || (h.n_blocks > 0 && !blocks_out)) return esp::fail(ESP_ERR_CAPACITY, "esp_kv_slot_load: %d blocks, room for %d", h.n_blocks, blocks_cap);
  if (esp_kv_free_count(pool) < h.n_blocks) return esp::fail(ESP_ERR_CAPACITY, "KV cache full: the checkpoint needs %d blocks", h.n_blocks);
  for (int32_t i = 0; i < h.n_blocks; ++i) {
    if (int rc = esp_kv_alloc(pool, &blocks_out[i])) return rc;
    if (uint64_t(blocks_out[i] + 1) * block_bytes > region_bytes ||
        (kv_scales && uint64_t(blocks_out[i] + 1) * 2 * uint64_t(Hkv) > scales_region_floats)) {
      for (int32_t k = 0; k <= i; ++k) esp_kv_release(pool, blocks_out[k]);
      return esp::fail(ESP_ERR_INVALID, "esp_kv_slot_load: the pool's blocks do not fit the layer region");
    }
  }
  int rc = move_blocks(f, false, static_cast<cudaStream_t>(stream), kv, blocks_out, h.n_blocks, n_layers, region_bytes, block_bytes);
  if (rc == ESP_OK && kv_scales)
    rc = move_scales(f, false, static_cast<cudaStream_t>(stream), kv_scales, blocks_out, h.n_blocks, n_layers, scales_region_floats, 2 * Hkv);
  if (rc != ESP_OK) {
    for (int32_t i = 0; i < h.n_blocks; ++i) esp_kv_release(pool, blocks_out[i]);
    return rc;
  }
  *n_blocks = h.n_blocks, *len = h.len, *next_pos = h.next_pos;
  return ESP_OK;
}

}  // extern "C"
