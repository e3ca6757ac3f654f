// ma_b200_forward_static_scratch: the generic-kernel forward pass for callers that cannot
// provide a workspace because they cannot allocate device memory at all.
//
// Some hosts of this library have no way to obtain scratch memory at call time: a serving
// process whose device memory was handed in full to another component's pool at start-up,
// a plug-in that is forbidden to touch the CUDA allocator, or a latency-critical loop in
// which an allocator call (which may synchronise the whole device) is not acceptable.  For
// them the stage-to-stage state lives in a fixed array that is part of the library image
// on every GPU that loads it, and this entry point never allocates or frees anything.
#include <mutex>
#include <string>

#include "ma_common.cuh"

namespace {

// 8 MiB per GPU, resident from library load until process exit.
constexpr size_t kStaticScratchBytes = MA_B200_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_ptr[kMaxDevices] = {};  // device address of g_static_scratch, per device ordinal

// In host code the array's name is only a handle for the runtime, not an address a kernel can
// use; the device address has to be asked for, once per device, with that device current.
int scratch_address(void** out, std::string* err) {
  int dev = -1;
  cudaError_t ce = cudaGetDevice(&dev);
  if (ce != cudaSuccess) {
    *err = std::string("cudaGetDevice: ") + cudaGetErrorString(ce);
    return MA_B200_CUDA_ERROR;
  }
  if (dev < 0 || dev >= kMaxDevices) {
    *err = "device ordinal out of range for the static scratch table";
    return MA_B200_UNSUPPORTED;
  }
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    ce = cudaGetSymbolAddress(&p, g_static_scratch);
    if (ce != cudaSuccess || p == nullptr) {
      *err = std::string("cudaGetSymbolAddress(static scratch): ") + cudaGetErrorString(ce);
      return MA_B200_CUDA_ERROR;
    }
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return MA_B200_OK;
}

thread_local std::string g_static_error;

}  // namespace

extern "C" {

MA_B200_API size_t ma_b200_static_scratch_bytes(void) { return kStaticScratchBytes; }

MA_B200_API const char* ma_b200_static_scratch_last_error(void) { return g_static_error.c_str(); }

MA_B200_API int ma_b200_forward_static_scratch(const ma_b200_problem* p, void* stream) {
  g_static_error.clear();
  if (p == nullptr) {
    g_static_error = "problem is NULL";
    return MA_B200_INVALID_ARGUMENT;
  }
  // Always the generic kernel family: it needs nothing beyond the scratch (no tensor maps, no
  // host-side plan), so nothing is allocated on either side of the bus.
  ma_b200_problem q = *p;
  q.kernel = MA_B200_KERNEL_GENERIC;
  ma_b200_workspace_layout L;
  int rc = ma_b200_workspace_layout_of(&q, &L);
  if (rc != MA_B200_OK) {
    g_static_error = ma_b200_last_error();
    return rc;
  }
  if (L.total > kStaticScratchBytes) {
    g_static_error = "problem needs " + std::to_string(L.total) + " bytes of scratch but the static scratch holds " +
                     std::to_string(kStaticScratchBytes) + " bytes; use ma_b200_forward with a caller-owned workspace";
    return MA_B200_WORKSPACE_TOO_SMALL;
  }
  void* scratch = nullptr;
  rc = scratch_address(&scratch, &g_static_error);
  if (rc != MA_B200_OK) return rc;
  // ma_b200_forward clears the status word at the head of the scratch itself; every other byte a
  // stage reads was written by an earlier stage of the same call, so stale contents are harmless.
  rc = ma_b200_forward(&q, scratch, kStaticScratchBytes, stream);
  if (rc != MA_B200_OK) g_static_error = ma_b200_last_error();
  return rc;
}

}  // extern "C"
