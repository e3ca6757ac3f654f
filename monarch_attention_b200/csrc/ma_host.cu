// ma_b200_forward_host: the forward pass for q, k, v and the result in HOST memory.
//
// For the long-sequence workloads the PCIe copies around a call cost far more than the kernels
// (134 MB against 0.14 ms of compute for N = 16384 and 16 heads).  Every (batch, head) pair is
// independent in every stage, so the call is cut into chunks of a few heads and pipelined over
// three streams owned by the library -
//     copy-in : H2D q, k, v of chunk i+1
//     compute : ma_b200_forward on chunk i (device staging buffers, E = 1, H = heads of the chunk)
//     copy-out: D2H result of chunk i-1
// - with three staging slots in caller-provided device memory and events between the streams.
// PCIe is full duplex, so the steady state is bound by the larger copy direction alone; the chunks of
// the last batch element shrink towards the end so that little is left exposed after the last copy-in.
// The whole pipeline is queued from one host thread without waiting for the GPU; on return the
// caller's stream has been made to wait for the last copy.
#include <mutex>
#include <string>

#include "ma_common.cuh"

namespace {

constexpr int kSlots = 3;
constexpr int kMaxDevices = 64;
constexpr size_t kAlign = 256;

struct Pipes {
  bool ready = false;
  cudaStream_t in = nullptr, comp = nullptr, out = nullptr;
  cudaEvent_t start = nullptr, loaded[kSlots] = {}, computed[kSlots] = {}, stored[kSlots] = {}, done_comp = nullptr,
              done_out = nullptr;
  // what the previous call on this device laid out in the scratch (a streamed call may only overlap a
  // previous call that used the same slots)
  const void* last_scratch = nullptr;
  size_t last_slot_bytes = 0, last_total = 0;
};
Pipes g_pipes[kMaxDevices];
std::mutex g_pipes_mutex;
thread_local std::string g_host_error;

size_t round_up(size_t x) { return (x + kAlign - 1) / kAlign * kAlign; }
size_t elem_size(int dtype) { return dtype == MA_B200_F32 ? 4 : 2; }

struct HostLayout {
  int hc;                                // heads per chunk (clamped to H)
  size_t qk_bytes, v_bytes;              // one staging tensor of a slot
  size_t slot_bytes, mask_off, mask_bytes, ws_off, ws_bytes, total;
};

// 0 on success; fills the layout of the device scratch for this problem.
int host_layout(const ma_b200_problem* p, int heads_per_chunk, HostLayout* L, std::string* err) {
  if (p == nullptr) { *err = "problem is null"; return MA_B200_INVALID_ARGUMENT; }
  if (heads_per_chunk < 1) { *err = "heads_per_chunk must be at least 1"; return MA_B200_INVALID_ARGUMENT; }
  if (p->E < 1 || p->H < 1 || p->N < 1 || p->D < 1 || p->Dv < 1) { *err = "E, H, N, D, Dv must be positive"; return MA_B200_INVALID_ARGUMENT; }
  L->hc = heads_per_chunk < p->H ? heads_per_chunk : p->H;
  L->qk_bytes = round_up((size_t)L->hc * p->N * p->D * elem_size(p->qk_dtype));
  L->v_bytes = round_up((size_t)L->hc * p->N * p->Dv * elem_size(p->v_dtype));
  L->slot_bytes = 2 * L->qk_bytes + 2 * L->v_bytes;  // q, k, v, result
  L->mask_off = kSlots * L->slot_bytes;
  L->mask_bytes = p->mask != nullptr ? round_up((size_t)p->E * p->N) : 0;
  L->ws_off = L->mask_off + L->mask_bytes;
  // workspace of the largest chunk problem (pointers are not looked at by the size query)
  ma_b200_problem sub = *p;
  sub.E = 1;
  sub.H = L->hc;
  sub.q.ptr = sub.k.ptr = sub.v.ptr = sub.out.ptr = nullptr;
  sub.q.stride_e = sub.k.stride_e = (int64_t)L->hc * p->N * p->D;
  sub.q.stride_h = sub.k.stride_h = (int64_t)p->N * p->D;
  sub.q.stride_n = sub.k.stride_n = p->D;
  sub.v.stride_e = sub.out.stride_e = (int64_t)L->hc * p->N * p->Dv;
  sub.v.stride_h = sub.out.stride_h = (int64_t)p->N * p->Dv;
  sub.v.stride_n = sub.out.stride_n = p->Dv;
  sub.mask = nullptr;
  sub.mask_stride_e = 0;
  L->ws_bytes = ma_b200_workspace_bytes(&sub);
  if (L->ws_bytes == 0) { *err = std::string("chunk problem rejected: ") + ma_b200_last_error(); return MA_B200_INVALID_ARGUMENT; }
  L->ws_bytes = round_up(L->ws_bytes);
  L->total = L->ws_off + L->ws_bytes;
  return MA_B200_OK;
}

int get_pipes(Pipes** out, std::string* err) {
  int dev = -1;
  cudaError_t ce = cudaGetDevice(&dev);
  if (ce != cudaSuccess) { *err = std::string("cudaGetDevice: ") + cudaGetErrorString(ce); return MA_B200_CUDA_ERROR; }
  if (dev < 0 || dev >= kMaxDevices) { *err = "device ordinal out of range"; return MA_B200_UNSUPPORTED; }
  std::lock_guard<std::mutex> lock(g_pipes_mutex);
  Pipes& P = g_pipes[dev];
  if (!P.ready) {
    auto ev = [&](cudaEvent_t* e) { return cudaEventCreateWithFlags(e, cudaEventDisableTiming); };
    bool ok = cudaStreamCreateWithFlags(&P.in, cudaStreamNonBlocking) == cudaSuccess &&
              cudaStreamCreateWithFlags(&P.comp, cudaStreamNonBlocking) == cudaSuccess &&
              cudaStreamCreateWithFlags(&P.out, cudaStreamNonBlocking) == cudaSuccess && ev(&P.start) == cudaSuccess &&
              ev(&P.done_comp) == cudaSuccess && ev(&P.done_out) == cudaSuccess;
    for (int i = 0; i < kSlots && ok; ++i)
      ok = ev(&P.loaded[i]) == cudaSuccess && ev(&P.computed[i]) == cudaSuccess && ev(&P.stored[i]) == cudaSuccess;
    if (!ok) { *err = std::string("creating streams / events: ") + cudaGetErrorString(cudaGetLastError()); return MA_B200_CUDA_ERROR; }
    P.ready = true;
  }
  *out = &P;
  return MA_B200_OK;
}

// Copies `heads` heads of one batch element between a strided host tensor and a dense staging
// buffer (heads, N, W).  One copy when the heads are dense in host memory, one (pitched) copy per
// head otherwise.
cudaError_t copy_heads(void* dev, const ma_b200_tensor& host, int e, int h0, int heads, int N, int W, size_t es,
                       bool to_device, cudaStream_t s) {
  char* hbase = static_cast<char*>(const_cast<void*>(host.ptr)) + ((int64_t)e * host.stride_e + (int64_t)h0 * host.stride_h) * (int64_t)es;
  const bool rows_dense = host.stride_n == W;
  const bool heads_dense = rows_dense && (heads == 1 || host.stride_h == (int64_t)N * W);
  const cudaMemcpyKind kind = to_device ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost;
  if (heads_dense) {
    const size_t bytes = (size_t)heads * N * W * es;
    return to_device ? cudaMemcpyAsync(dev, hbase, bytes, kind, s) : cudaMemcpyAsync(hbase, dev, bytes, kind, s);
  }
  for (int h = 0; h < heads; ++h) {
    char* hp = hbase + (int64_t)h * host.stride_h * (int64_t)es;
    char* dp = static_cast<char*>(dev) + (size_t)h * N * W * es;
    cudaError_t ce;
    if (rows_dense) {
      ce = to_device ? cudaMemcpyAsync(dp, hp, (size_t)N * W * es, kind, s) : cudaMemcpyAsync(hp, dp, (size_t)N * W * es, kind, s);
    } else {
      ce = to_device ? cudaMemcpy2DAsync(dp, (size_t)W * es, hp, (size_t)host.stride_n * es, (size_t)W * es, N, kind, s)
                     : cudaMemcpy2DAsync(hp, (size_t)host.stride_n * es, dp, (size_t)W * es, (size_t)W * es, N, kind, s);
    }
    if (ce != cudaSuccess) return ce;
  }
  return cudaSuccess;
}

}  // namespace

extern "C" {

MA_B200_API const char* ma_b200_host_last_error(void) { return g_host_error.c_str(); }

MA_B200_API size_t ma_b200_host_scratch_bytes(const ma_b200_problem* p, int heads_per_chunk) {
  HostLayout L;
  g_host_error.clear();
  if (host_layout(p, heads_per_chunk, &L, &g_host_error) != MA_B200_OK) return 0;
  return L.total;
}

static int forward_host_impl(const ma_b200_problem* p, int heads_per_chunk, void* device_scratch, size_t scratch_bytes,
                             void* stream_v, bool streamed) {
  g_host_error.clear();
  HostLayout L;
  int rc = host_layout(p, heads_per_chunk, &L, &g_host_error);
  if (rc != MA_B200_OK) return rc;
  if (p->q.ptr == nullptr || p->k.ptr == nullptr || p->v.ptr == nullptr || p->out.ptr == nullptr) {
    g_host_error = "q, k, v and out must be host pointers";
    return MA_B200_INVALID_ARGUMENT;
  }
  if (device_scratch == nullptr || scratch_bytes < L.total) {
    g_host_error = "device scratch too small: need " + std::to_string(L.total) + " bytes";
    return MA_B200_WORKSPACE_TOO_SMALL;
  }
  if (reinterpret_cast<uintptr_t>(device_scratch) % kAlign != 0) {
    g_host_error = "device scratch must be 256-byte aligned";
    return MA_B200_INVALID_ARGUMENT;
  }
  Pipes* P = nullptr;
  rc = get_pipes(&P, &g_host_error);
  if (rc != MA_B200_OK) return rc;
  cudaStream_t caller = reinterpret_cast<cudaStream_t>(stream_v);
  char* base = static_cast<char*>(device_scratch);
  const size_t es_qk = elem_size(p->qk_dtype), es_v = elem_size(p->v_dtype);
  auto fail = [&](cudaError_t ce, const char* what) {
    g_host_error = std::string(what) + ": " + cudaGetErrorString(ce);
    return MA_B200_CUDA_ERROR;
  };
  cudaError_t ce;
#define MA_TRY(call, what) \
  if ((ce = (call)) != cudaSuccess) return fail(ce, what)

  // A streamed call may start copying in while the previous call on this device is still computing and
  // copying out, provided that call used the scratch in the same way (same slots: the per-slot events then
  // order every reuse); anything else is ordered after what the caller has already queued on its stream,
  // which includes the end of the previous call.
  const bool overlap = streamed && P->last_scratch == device_scratch && P->last_slot_bytes == L.slot_bytes &&
                       P->last_total == L.total;
  P->last_scratch = device_scratch;
  P->last_slot_bytes = L.slot_bytes;
  P->last_total = L.total;
  if (!overlap) {
    MA_TRY(cudaEventRecord(P->start, caller), "cudaEventRecord(start)");
    MA_TRY(cudaStreamWaitEvent(P->in, P->start, 0), "cudaStreamWaitEvent(in, start)");
    MA_TRY(cudaStreamWaitEvent(P->comp, P->start, 0), "cudaStreamWaitEvent(comp, start)");
    MA_TRY(cudaStreamWaitEvent(P->out, P->start, 0), "cudaStreamWaitEvent(out, start)");
  } else if (p->mask != nullptr) {
    // the mask has one place in the scratch: the previous call's kernels must have read theirs
    MA_TRY(cudaStreamWaitEvent(P->in, P->done_comp, 0), "cudaStreamWaitEvent(in, done_comp)");
  }
  unsigned char* mask_dev = nullptr;
  if (p->mask != nullptr) {
    mask_dev = reinterpret_cast<unsigned char*>(base + L.mask_off);
    const size_t pitch = (size_t)p->mask_stride_e;
    if (pitch == (size_t)p->N || p->E == 1) {
      MA_TRY(cudaMemcpyAsync(mask_dev, p->mask, (size_t)p->E * p->N, cudaMemcpyHostToDevice, P->in), "mask upload");
    } else {
      MA_TRY(cudaMemcpy2DAsync(mask_dev, p->N, p->mask, pitch, p->N, p->E, cudaMemcpyHostToDevice, P->in), "mask upload");
    }
  }

  int i = 0;
  for (int e = 0; e < p->E; ++e) {
    int nh = 0;
    for (int h0 = 0; h0 < p->H; h0 += nh, ++i) {
      // Chunks of hc heads, except that the last batch element tapers off (each chunk at most half of
      // what is left): once the last copy-in has landed, only the kernels and the copy-out of the last
      // chunk are still to come, and nothing overlaps them.
      const int left = p->H - h0;
      nh = left < L.hc ? left : L.hc;
      if (e == p->E - 1 && nh > 1 && nh > left / 2) nh = left / 2 > 1 ? left / 2 : 1;
      const int slot = i % kSlots;
      char* sq = base + (size_t)slot * L.slot_bytes;
      char* sk = sq + L.qk_bytes;
      char* sv = sk + L.qk_bytes;
      char* so = sv + L.v_bytes;
      // copy in: the kernels of the chunk that used this slot last have read q, k, v
      if (i >= kSlots || overlap) MA_TRY(cudaStreamWaitEvent(P->in, P->computed[slot], 0), "wait(in, computed)");
      MA_TRY(copy_heads(sq, p->q, e, h0, nh, p->N, p->D, es_qk, true, P->in), "H2D q");
      MA_TRY(copy_heads(sk, p->k, e, h0, nh, p->N, p->D, es_qk, true, P->in), "H2D k");
      MA_TRY(copy_heads(sv, p->v, e, h0, nh, p->N, p->Dv, es_v, true, P->in), "H2D v");
      MA_TRY(cudaEventRecord(P->loaded[slot], P->in), "record(loaded)");
      // compute: inputs landed, and the previous result of this slot has left it
      MA_TRY(cudaStreamWaitEvent(P->comp, P->loaded[slot], 0), "wait(comp, loaded)");
      if (i >= kSlots || overlap) MA_TRY(cudaStreamWaitEvent(P->comp, P->stored[slot], 0), "wait(comp, stored)");
      ma_b200_problem sub = *p;
      sub.E = 1;
      sub.H = nh;
      sub.q = {sq, (int64_t)nh * p->N * p->D, (int64_t)p->N * p->D, p->D};
      sub.k = {sk, (int64_t)nh * p->N * p->D, (int64_t)p->N * p->D, p->D};
      sub.v = {sv, (int64_t)nh * p->N * p->Dv, (int64_t)p->N * p->Dv, p->Dv};
      sub.out = {so, (int64_t)nh * p->N * p->Dv, (int64_t)p->N * p->Dv, p->Dv};
      sub.mask = mask_dev != nullptr ? mask_dev + (size_t)e * p->N : nullptr;
      sub.mask_stride_e = mask_dev != nullptr ? p->N : 0;
      rc = ma_b200_forward(&sub, base + L.ws_off, L.ws_bytes, P->comp);
      if (rc != MA_B200_OK) {
        g_host_error = std::string("chunk forward: ") + ma_b200_last_error();
        return rc;
      }
      MA_TRY(cudaEventRecord(P->computed[slot], P->comp), "record(computed)");
      // copy out
      MA_TRY(cudaStreamWaitEvent(P->out, P->computed[slot], 0), "wait(out, computed)");
      MA_TRY(copy_heads(so, p->out, e, h0, nh, p->N, p->Dv, es_v, false, P->out), "D2H result");
      MA_TRY(cudaEventRecord(P->stored[slot], P->out), "record(stored)");
    }
  }
  // the caller's stream continues once the last kernel and the last copy are done
  MA_TRY(cudaEventRecord(P->done_comp, P->comp), "record(done_comp)");
  MA_TRY(cudaEventRecord(P->done_out, P->out), "record(done_out)");
  MA_TRY(cudaStreamWaitEvent(caller, P->done_comp, 0), "wait(caller, done_comp)");
  MA_TRY(cudaStreamWaitEvent(caller, P->done_out, 0), "wait(caller, done_out)");
#undef MA_TRY
  return MA_B200_OK;
}

MA_B200_API int ma_b200_forward_host(const ma_b200_problem* p, int heads_per_chunk, void* device_scratch,
                                     size_t scratch_bytes, void* stream_v) {
  return forward_host_impl(p, heads_per_chunk, device_scratch, scratch_bytes, stream_v, false);
}

MA_B200_API int ma_b200_forward_host_streamed(const ma_b200_problem* p, int heads_per_chunk, void* device_scratch,
                                              size_t scratch_bytes, void* stream_v) {
  return forward_host_impl(p, heads_per_chunk, device_scratch, scratch_bytes, stream_v, true);
}

}  // extern "C"
