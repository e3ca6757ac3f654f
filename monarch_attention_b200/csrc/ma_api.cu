// C ABI of the library: argument validation, workspace layout, kernel selection and the
// stage driver  (T-1) x [right-factor, left-factor], right-factor-with-V, output
// (reference: ma/ma_torch.py:100-105).
#include <math.h>
#include <stdio.h>
#include <string.h>

#include <string>

#include "ma_common.cuh"
#include "ma_tc_plan.cuh"

namespace {

thread_local std::string g_last_error;

int fail(int code, const std::string& msg) {
  g_last_error = msg;
  return code;
}

size_t dtype_size(int dt) {
  switch (dt) {
    case MA_B200_F32: return 4;
    case MA_B200_BF16: return 2;
    case MA_B200_F16: return 2;
    default: return 0;
  }
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

int validate(const ma_b200_problem* p, bool need_pointers) {
  if (p == nullptr) return fail(MA_B200_INVALID_ARGUMENT, "problem is NULL");
  if (p->abi_version != MA_B200_ABI_VERSION)
    return fail(MA_B200_INVALID_ARGUMENT, "abi_version mismatch: got " + std::to_string(p->abi_version));
  if (p->E <= 0 || p->H <= 0 || p->N <= 0 || p->D <= 0 || p->Dv <= 0)
    return fail(MA_B200_INVALID_ARGUMENT, "E, H, N, D, Dv must be positive");
  if (p->block_size <= 0) return fail(MA_B200_INVALID_ARGUMENT, "block_size must be positive");
  if (p->num_steps <= 0) return fail(MA_B200_INVALID_ARGUMENT, "num_steps must be positive");
  if (dtype_size(p->qk_dtype) == 0 || dtype_size(p->v_dtype) == 0)
    return fail(MA_B200_INVALID_ARGUMENT, "unknown dtype");
  if (!(p->qk_dtype == p->v_dtype || p->v_dtype == MA_B200_F32))
    return fail(MA_B200_UNSUPPORTED, "v_dtype must equal qk_dtype or be f32");
  if (p->kernel < MA_B200_KERNEL_AUTO || p->kernel > MA_B200_KERNEL_HEAD_FUSED || p->kernel == 4)
    return fail(MA_B200_INVALID_ARGUMENT, "unknown kernel family");
  if ((long long)p->E * p->H > 0x7fffffffLL / 2) return fail(MA_B200_INVALID_ARGUMENT, "E*H too large");
  if (need_pointers) {
    if (!p->q.ptr || !p->k.ptr || !p->v.ptr || !p->out.ptr)
      return fail(MA_B200_INVALID_ARGUMENT, "q, k, v and out must be non-NULL");
    const ma_b200_tensor* ts[4] = {&p->q, &p->k, &p->v, &p->out};
    const char* names[4] = {"q", "k", "v", "out"};
    for (int i = 0; i < 4; ++i) {
      if (ts[i]->stride_e < 0 || ts[i]->stride_h < 0 || ts[i]->stride_n < 0)
        return fail(MA_B200_INVALID_ARGUMENT, std::string(names[i]) + ": negative stride");
      const size_t es = dtype_size(i < 2 ? p->qk_dtype : p->v_dtype);
      if (reinterpret_cast<uintptr_t>(ts[i]->ptr) % es != 0)
        return fail(MA_B200_INVALID_ARGUMENT, std::string(names[i]) + ": pointer not aligned to its element size");
    }
    const int W = p->Dv;
    if (p->out.stride_n < W && p->N > 1) return fail(MA_B200_INVALID_ARGUMENT, "out rows overlap (stride_n < Dv)");
    if (p->mask != nullptr && p->mask_stride_e < 0) return fail(MA_B200_INVALID_ARGUMENT, "mask: negative stride");
  }
  return MA_B200_OK;
}

ma::Geometry make_geometry(const ma_b200_problem* p) {
  ma::Geometry g;
  memset(&g, 0, sizeof(g));
  g.E = p->E; g.H = p->H; g.N = p->N; g.D = p->D; g.Dv = p->Dv;
  g.B = p->block_size;
  g.M = (p->N + p->block_size - 1) / p->block_size;
  g.pad_off = p->pre_pad ? g.M * g.B - g.N : 0;
  g.T = p->num_steps;
  g.sm_scale = (float)(1.0 / sqrt((double)p->D));
  auto view = [](const ma_b200_tensor& t) {
    ma::View4 v;
    v.ptr = t.ptr; v.se = t.stride_e; v.sh = t.stride_h; v.sn = t.stride_n;
    return v;
  };
  g.q = view(p->q); g.k = view(p->k); g.v = view(p->v); g.out = view(p->out);
  g.mask = p->mask;
  g.mask_se = p->mask_stride_e;
  return g;
}

int resolve_kernel(const ma_b200_problem* p, const ma::Geometry& g, int* kernel) {
  const char* why = "";
  const bool tc_ok = ma::tc_supported(g, p->qk_dtype, p->v_dtype, &why);
  const bool wants_tc = p->kernel == MA_B200_KERNEL_TCGEN05 || p->kernel == MA_B200_KERNEL_TCGEN05_STAGED;
  if (wants_tc && !tc_ok)
    return fail(MA_B200_UNSUPPORTED, std::string("tcgen05 path cannot run this problem: ") + why);
  const char* why_w = "";
  const bool warp_ok = ma::warp_supported(g, p->qk_dtype, p->v_dtype, &why_w);
  if (p->kernel == MA_B200_KERNEL_WARP_MMA && !warp_ok)
    return fail(MA_B200_UNSUPPORTED, std::string("warp-level tensor-core path cannot run this problem: ") + why_w);
  const char* why_h = "";
  const bool head_ok = ma::head_fused_supported(g, p->qk_dtype, p->v_dtype, &why_h);
  if (p->kernel == MA_B200_KERNEL_HEAD_FUSED && !head_ok)
    return fail(MA_B200_UNSUPPORTED, std::string("one-CTA-per-head kernel cannot run this problem: ") + why_h);
  if (p->kernel == MA_B200_KERNEL_AUTO)
    // (the one-CTA-per-head kernel is selectable but not preferred: on the ViT / RoBERTa shapes it
    // measured slower than the two staged launches - these tiny tiles are instruction-bound)
    *kernel = tc_ok ? MA_B200_KERNEL_TCGEN05 : (warp_ok ? MA_B200_KERNEL_WARP_MMA : MA_B200_KERNEL_GENERIC);
  else *kernel = p->kernel;
  if (*kernel == MA_B200_KERNEL_GENERIC) {
    const size_t need = ma::generic_stage_smem_bytes(g, g.B > g.M ? ma::kStageRight : ma::kStageLeft);
    if (need > 200 * 1024)
      return fail(MA_B200_UNSUPPORTED, "generic path: block size or block count too large for shared memory");
    if (g.M > 65535 || g.B > 65535)  // gridDim.y; E*H sits on gridDim.x (limit 2^31 - 1, checked in validate)
      return fail(MA_B200_UNSUPPORTED, "generic path: grid too large");
  }
  return MA_B200_OK;
}

int layout_of(const ma_b200_problem* p, ma_b200_workspace_layout* L) {
  int rc = validate(p, false);
  if (rc != MA_B200_OK) return rc;
  ma::Geometry g = make_geometry(p);
  int kernel = 0;
  rc = resolve_kernel(p, g, &kernel);
  if (rc != MA_B200_OK) return rc;
  const size_t EH = (size_t)p->E * p->H, MB = (size_t)g.M * g.B;
  const size_t qs = dtype_size(p->qk_dtype), vs = dtype_size(p->v_dtype);
  size_t off = 0;
  L->status = off; off = align_up(off + 256, 256);
  L->counters = off; off = align_up(off + EH * 2 * (size_t)p->num_steps * sizeof(int), 256);
  L->ar = off;     off = align_up(off + (p->num_steps > 1 ? EH * MB * p->D * qs : 0), 256);
  L->cr = off;     off = align_up(off + (p->num_steps > 1 ? EH * MB * sizeof(float) : 0), 256);
  L->al = off;     off = align_up(off + EH * MB * p->D * qs, 256);
  L->cl = off;     off = align_up(off + EH * MB * sizeof(float), 256);
  L->y = off;      off = align_up(off + EH * MB * p->Dv * vs, 256);
  L->total = off;
  L->M = g.M;
  L->kernel = kernel;
  return MA_B200_OK;
}

int run_forward(const ma_b200_problem* p, void* workspace, size_t workspace_bytes, void* stream_v, float* stage_ms,
                int n_stage_ms) {
  int rc = validate(p, true);
  if (rc != MA_B200_OK) return rc;
  ma_b200_workspace_layout L;
  rc = layout_of(p, &L);
  if (rc != MA_B200_OK) return rc;
  if (workspace == nullptr) return fail(MA_B200_INVALID_ARGUMENT, "workspace is NULL");
  if (reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
    return fail(MA_B200_INVALID_ARGUMENT, "workspace must be 256-byte aligned");
  if (workspace_bytes < L.total)
    return fail(MA_B200_WORKSPACE_TOO_SMALL, "workspace has " + std::to_string(workspace_bytes) + " bytes, need " +
                                                 std::to_string(L.total));
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  ma::Geometry g = make_geometry(p);
  char* ws = reinterpret_cast<char*>(workspace);
  g.status = reinterpret_cast<int*>(ws + L.status);
  g.ar = ws + L.ar;
  g.cr = reinterpret_cast<float*>(ws + L.cr);
  g.al = ws + L.al;
  g.cl = reinterpret_cast<float*>(ws + L.cl);
  g.y = ws + L.y;

  auto cuda_fail = [&](cudaError_t e, const char* what) {
    return fail(MA_B200_CUDA_ERROR, std::string(what) + ": " + cudaGetErrorString(e));
  };
  // status word and the stage-completion counters start at zero
  cudaError_t ce = cudaMemsetAsync(ws + L.status, 0, L.ar - L.status, stream);
  if (ce != cudaSuccess) return cuda_fail(ce, "cudaMemsetAsync(status, counters)");
  int* counters = reinterpret_cast<int*>(ws + L.counters);

  ma::TcPlan plan_store;
  const ma::TcPlan* plan = nullptr;
  if (L.kernel == MA_B200_KERNEL_TCGEN05 || L.kernel == MA_B200_KERNEL_TCGEN05_STAGED) {
    const char* err = "";
    rc = ma::tc_plan_get(g, p->qk_dtype, &plan_store, &err);
    if (rc != MA_B200_OK) return fail(rc, std::string("tcgen05 plan: ") + err);
    plan = &plan_store;
  }

  const int n_stages = 2 * p->num_steps;
  cudaEvent_t* ev = nullptr;
  if (stage_ms != nullptr) {
    ev = new cudaEvent_t[n_stages + 1];
    for (int i = 0; i <= n_stages; ++i) cudaEventCreate(&ev[i]);
    cudaEventRecord(ev[0], stream);
  }
  int stage_idx = 0;
  auto launch = [&](ma::StageKind kind, bool first) -> cudaError_t {
    cudaError_t e;
    if (L.kernel == MA_B200_KERNEL_TCGEN05_STAGED)
      e = ma::launch_fused(plan, g, counters, stage_idx, stage_idx + 1, 0, stream);
    else if (L.kernel == MA_B200_KERNEL_WARP_MMA) e = ma::launch_warp_stage(g, p->qk_dtype, kind, first, stream);
    else e = ma::launch_generic_stage(g, p->qk_dtype, p->v_dtype, kind, first, stream);
    ++stage_idx;
    if (ev != nullptr) cudaEventRecord(ev[stage_idx], stream);
    return e;
  };

  rc = MA_B200_OK;
  bool first = true;
  if (L.kernel == MA_B200_KERNEL_HEAD_FUSED) {
    ce = ma::launch_head_fused(g, p->qk_dtype, stream);
    if (ce != cudaSuccess) rc = cuda_fail(ce, "one-CTA-per-head kernel");
    if (ev != nullptr)
      for (int i = 1; i <= n_stages; ++i) cudaEventRecord(ev[i], stream);
  } else if (L.kernel == MA_B200_KERNEL_TCGEN05) {
    // every stage in one persistent launch
    ce = ma::launch_fused(plan, g, counters, 0, n_stages, 1, stream);
    if (ce != cudaSuccess) rc = cuda_fail(ce, "fused kernel");
    if (ev != nullptr) {
      cudaEventRecord(ev[1], stream);
      for (int i = 2; i <= n_stages; ++i) cudaEventRecord(ev[i], stream);
    }
  } else {
  for (int t = 0; t + 1 < p->num_steps && rc == MA_B200_OK; ++t) {
    if ((ce = launch(ma::kStageRight, first)) != cudaSuccess) { rc = cuda_fail(ce, "right-factor stage"); break; }
    first = false;
    if ((ce = launch(ma::kStageLeft, false)) != cudaSuccess) { rc = cuda_fail(ce, "left-factor stage"); break; }
  }
  if (rc == MA_B200_OK && (ce = launch(ma::kStageRightWithV, first)) != cudaSuccess)
    rc = cuda_fail(ce, "right-factor stage with V");
  if (rc == MA_B200_OK && (ce = launch(ma::kStageOutput, false)) != cudaSuccess) rc = cuda_fail(ce, "output stage");
  }

  if (ev != nullptr) {
    if (rc == MA_B200_OK) {
      ce = cudaStreamSynchronize(stream);
      if (ce != cudaSuccess) rc = cuda_fail(ce, "cudaStreamSynchronize");
      for (int i = 0; i < n_stages && i < n_stage_ms && rc == MA_B200_OK; ++i)
        cudaEventElapsedTime(&stage_ms[i], ev[i], ev[i + 1]);
    }
    for (int i = 0; i <= n_stages; ++i) cudaEventDestroy(ev[i]);
    delete[] ev;
  }
  return rc;
}

}  // namespace

extern "C" {

size_t ma_b200_workspace_bytes(const ma_b200_problem* p) {
  ma_b200_workspace_layout L;
  if (layout_of(p, &L) != MA_B200_OK) return 0;
  return L.total;
}

int ma_b200_workspace_layout_of(const ma_b200_problem* p, ma_b200_workspace_layout* layout) {
  if (layout == nullptr) return fail(MA_B200_INVALID_ARGUMENT, "layout is NULL");
  return layout_of(p, layout);
}

int ma_b200_forward(const ma_b200_problem* p, void* workspace, size_t workspace_bytes, void* stream) {
  return run_forward(p, workspace, workspace_bytes, stream, nullptr, 0);
}

int ma_b200_forward_timed(const ma_b200_problem* p, void* workspace, size_t workspace_bytes, void* stream,
                          float* stage_ms, int32_t n_stage_ms) {
  if (stage_ms == nullptr || n_stage_ms <= 0) return fail(MA_B200_INVALID_ARGUMENT, "stage_ms is NULL or empty");
  return run_forward(p, workspace, workspace_bytes, stream, stage_ms, n_stage_ms);
}

int ma_b200_device_status(void* workspace, void* stream) {
  if (workspace == nullptr) return fail(MA_B200_INVALID_ARGUMENT, "workspace is NULL");
  int flag = 0;
  cudaError_t ce = cudaMemcpyAsync(&flag, workspace, sizeof(int), cudaMemcpyDeviceToHost,
                                   reinterpret_cast<cudaStream_t>(stream));
  if (ce == cudaSuccess) ce = cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(stream));
  if (ce != cudaSuccess) return fail(MA_B200_CUDA_ERROR, std::string("device_status: ") + cudaGetErrorString(ce));
  if (flag != 0)
    return fail(MA_B200_DEVICE_WAIT_EXPIRED, "device flag = " + std::to_string(flag) + " (a bounded wait expired)");
  return MA_B200_OK;
}

int ma_b200_poll_device_status(int device) {
  const int code = ma::fused_poll_status(device);
  if (code != 0)
    return fail(MA_B200_DEVICE_WAIT_EXPIRED, "device " + std::to_string(device) + ": wait " + std::to_string(code) +
                                                 " of the fused kernel gave up; the output of that call is undefined");
  return MA_B200_OK;
}

void ma_b200_selftest_generic_general_form(int on) { ma::generic_set_general_form_only(on); }

int ma_b200_selftest_wait_expiry(const ma_b200_problem* p, void* workspace, size_t workspace_bytes, void* stream_v) {
  int rc = validate(p, true);
  if (rc != MA_B200_OK) return rc;
  ma_b200_problem q = *p;
  q.kernel = MA_B200_KERNEL_TCGEN05;
  ma_b200_workspace_layout L;
  rc = layout_of(&q, &L);
  if (rc != MA_B200_OK) return rc;
  if (workspace == nullptr || reinterpret_cast<uintptr_t>(workspace) % 256 != 0 || workspace_bytes < L.total)
    return fail(MA_B200_INVALID_ARGUMENT, "workspace is NULL, misaligned or too small");
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  ma::Geometry g = make_geometry(&q);
  char* ws = reinterpret_cast<char*>(workspace);
  g.status = reinterpret_cast<int*>(ws + L.status);
  g.ar = ws + L.ar; g.cr = reinterpret_cast<float*>(ws + L.cr);
  g.al = ws + L.al; g.cl = reinterpret_cast<float*>(ws + L.cl);
  g.y = ws + L.y;
  cudaError_t ce = cudaMemsetAsync(ws + L.status, 0, L.ar - L.status, stream);
  if (ce != cudaSuccess) return fail(MA_B200_CUDA_ERROR, cudaGetErrorString(ce));
  ma::TcPlan plan;
  const char* err = "";
  rc = ma::tc_plan_get(g, q.qk_dtype, &plan, &err);
  if (rc != MA_B200_OK) return fail(rc, std::string("tcgen05 plan: ") + err);
  // Stage 1 alone, waiting on completion counters of stage 0 that nothing will ever raise: every
  // producer runs out of patience after a few hundred microseconds and the CTAs return.
  ma::fused_set_spin_limit(4096);
  ce = ma::launch_fused(&plan, g, reinterpret_cast<int*>(ws + L.counters), 1, 2, 1, stream);
  ma::fused_set_spin_limit(0);
  if (ce != cudaSuccess) return fail(MA_B200_CUDA_ERROR, std::string("fused kernel: ") + cudaGetErrorString(ce));
  return MA_B200_OK;
}

const char* ma_b200_status_string(int status) {
  switch (status) {
    case MA_B200_OK: return "ok";
    case MA_B200_INVALID_ARGUMENT: return "invalid argument";
    case MA_B200_UNSUPPORTED: return "unsupported configuration";
    case MA_B200_CUDA_ERROR: return "CUDA error";
    case MA_B200_DEVICE_WAIT_EXPIRED: return "device-side bounded wait expired";
    case MA_B200_WORKSPACE_TOO_SMALL: return "workspace too small";
    default: return "unknown status";
  }
}

const char* ma_b200_last_error(void) { return g_last_error.c_str(); }

int32_t ma_b200_abi_version(void) { return MA_B200_ABI_VERSION; }

}  // extern "C"
