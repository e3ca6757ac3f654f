// Shared definitions for the MonarchAttention kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/monarch_attention_b200.h"

namespace ma {

constexpr float kEps = 1e-12f;            // eps of the right-factor stages (reference: ma/ma_torch.py:10)
constexpr float kTiny = 1.17549435e-38f;  // smallest normal fp32: floor of the right-factor entries (:18)

// A strided (E,H,N,W) view; strides in elements, innermost stride 1.
struct View4 {
  const void* ptr;
  long long se, sh, sn;
};

// Everything a stage kernel needs to know about one forward call.
struct Geometry {
  int E, H, N, D, Dv;
  int B, M;        // block size, number of blocks
  int pad_off;     // padded position p = m*B + j maps to token p - pad_off
  int T;
  float sm_scale;  // (float)(1/sqrt(D))
  View4 q, k, v, out;
  const uint8_t* mask;  // (E,N) bytes, non-zero = valid; or nullptr
  long long mask_se;
  // stage-to-stage state (workspace)
  void* ar;   // (EH, M, B, D)  qk dtype
  float* cr;  // (EH, M, B)
  void* al;   // (EH, B, M, D)  qk dtype
  float* cl;  // (EH, B, M)
  void* y;    // (EH, B, M, Dv) v dtype
  int* status;  // device flag, 0 = fine
};

enum StageKind { kStageRight = 0, kStageRightWithV = 1, kStageLeft = 2, kStageOutput = 3 };

template <typename T>
struct Cvt;
template <>
struct Cvt<float> {
  static __device__ __forceinline__ float to_f(float x) { return x; }
  static __device__ __forceinline__ float from_f(float x) { return x; }
};
template <>
struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float x) { return __float2bfloat16_rn(x); }
};
template <>
struct Cvt<__half> {
  static __device__ __forceinline__ float to_f(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half from_f(float x) { return __float2half_rn(x); }
};

// Round an fp32 value through storage type T and back (the reference rounds every
// contraction result to the storage dtype before the fp32 softmax arithmetic).
template <typename T>
__device__ __forceinline__ float round_through(float x) {
  return Cvt<T>::to_f(Cvt<T>::from_f(x));
}

// Host-side launchers implemented by the kernel translation units.
// Each returns cudaSuccess or the launch error.
// Test hook: 1 = the generic family always runs its general (warp-per-row) form.
void generic_set_general_form_only(int on);
cudaError_t launch_generic_stage(const Geometry& g, int qk_dtype, int v_dtype, StageKind kind, bool first,
                                 cudaStream_t stream);
size_t generic_stage_smem_bytes(const Geometry& g, StageKind kind);

// Warp-level tensor-core stage kernels (16-bit, block size and count <= 128, D <= 80).
bool warp_supported(const Geometry& g, int qk_dtype, int v_dtype, const char** why);
cudaError_t launch_warp_stage(const Geometry& g, int qk_dtype, StageKind kind, bool first, cudaStream_t stream);
// Whole head per CTA, both stages of a one-iteration call in one launch (state in shared memory).
bool head_fused_supported(const Geometry& g, int qk_dtype, int v_dtype, const char** why);
cudaError_t launch_head_fused(const Geometry& g, int qk_dtype, cudaStream_t stream);

// Tensor-core (tcgen05) path.
bool tc_supported(const Geometry& g, int qk_dtype, int v_dtype, const char** why);
// The TMA tensor maps of one call.  tc_plan_get copies them into *plan, from a cache when the same
// pointers, strides and sizes were seen before; tc_plan_create always encodes (heap object).
struct TcPlan;
int tc_plan_get(const Geometry& g, int qk_dtype, TcPlan* plan, const char** err);
int tc_plan_create(const Geometry& g, int qk_dtype, TcPlan** plan, const char** err);
void tc_plan_destroy(TcPlan* plan);
// Persistent fused kernel: stages [stage_begin, stage_end) of the 2T stages in one cooperative launch.
size_t fused_counter_bytes(const Geometry& g);
cudaError_t launch_fused(const TcPlan* plan, const Geometry& g, int* counters, int stage_begin, int stage_end,
                         int wait_deps, cudaStream_t stream);
// Code of a bounded device-side wait that gave up on `device` since the last poll (0 = none); reads a mapped
// host word, so it needs no synchronisation.
int fused_poll_status(int device);
// Iterations of the producer's dependency wait before it gives up (0 = default); for the wait-expiry self-test.
void fused_set_spin_limit(int iterations);

}  // namespace ma
