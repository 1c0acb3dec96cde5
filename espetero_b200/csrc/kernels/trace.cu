// esp_attn_stamp: a one-thread kernel that stores %globaltimer, the clock the per-CTA trace
// stamps use. Enqueued before and after a pass it brackets the pass in the same time base, so that
// the part of a kernel's duration that lies before its first CTA starts and after its last CTA
// exits can be read off (the reference's set_profile, src/model/model.mm:1041-1054, times whole
// dispatches from the host; this is its device-side counterpart).
#include "common.cuh"
#include "../host_util.h"
#include "../launch.h"

namespace {
__global__ void stamp_kernel(unsigned long long* dst) { *dst = esp::global_timer_ns(); }
}  // namespace

extern "C" int esp_attn_stamp(void* stream, uint64_t* device_slot) {
  if (!device_slot) return esp::fail(ESP_ERR_INVALID, "esp_attn_stamp: null slot");
  stamp_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(reinterpret_cast<unsigned long long*>(device_slot));
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return esp::fail(ESP_ERR_CUDA, "esp_attn_stamp: %s", cudaGetErrorString(e));
  return ESP_OK;
}
