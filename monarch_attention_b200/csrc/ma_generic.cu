// Generic SIMT stage kernels: any block size, block count, head width, value width,
// fp32 / bf16 / fp16 storage, key/query mask, front or back padding.
//
// This is the correctness anchor of the library and the path for fp32 inputs.  It
// follows the reference's rounding points exactly: every contraction result is
// rounded to the storage dtype before the fp32 softmax arithmetic, factor entries
// are rounded to the storage dtype before the second contraction
// (reference: ma/ma_torch.py:10-62).
//
// Work decomposition: one CTA per (head, key block m) for the right-factor stages and
// per (head, column j) for the left-factor and output stages; one warp per row of the
// small attention problem; lanes run over keys for the logits and over the feature
// axis for the weighted sums.  Operand rows are read straight from global memory
// (they are L1/L2 resident for the tile a CTA works on).
#include <math.h>

#include "ma_common.cuh"

namespace ma {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// <a, row> with a in shared memory (fp32) and row in global memory (storage dtype),
// accumulated in fp32 in increasing feature order.
template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ a, const T* __restrict__ row, int D) {
  float acc = 0.f;
  for (int d = 0; d < D; ++d) acc = fmaf(a[d], Cvt<T>::to_f(row[d]), acc);
  return acc;
}

// Token row of a (E,H,N,W) view for padded position p, or nullptr when p is padding.
template <typename T>
__device__ __forceinline__ const T* token_row(const View4& t, int e, int h, int p, int pad_off, int N) {
  int n = p - pad_off;
  if (n < 0 || n >= N) return nullptr;
  return reinterpret_cast<const T*>(t.ptr) + (long long)e * t.se + (long long)h * t.sh + (long long)n * t.sn;
}

__device__ __forceinline__ bool token_valid(const Geometry& g, int e, int p) {
  int n = p - g.pad_off;
  if (n < 0 || n >= g.N) return false;
  return g.mask == nullptr || g.mask[(long long)e * g.mask_se + n] != 0;
}

// ---------------------------------------------------------------------------------
// Right-factor stage (reference: ma/ma_torch.py:10-23 and, WITH_V, :38-52).
// grid = (M, E*H).  Shared memory: kWarps*(D + B) floats.
// ---------------------------------------------------------------------------------
template <typename TQ, typename TV, bool WITH_V>
__global__ void __launch_bounds__(kThreads) right_stage_kernel(const Geometry g, const int first) {
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m = blockIdx.x, eh = blockIdx.y;
  const int e = eh / g.H, h = eh % g.H;
  const int B = g.B, D = g.D, Dv = g.Dv, M = g.M;
  float* avec = smem + warp * (D + B);
  float* rbuf = avec + D;

  const TQ* ar = reinterpret_cast<const TQ*>(g.ar) + ((long long)eh * M + m) * B * D;
  TQ* al = reinterpret_cast<TQ*>(g.al) + (long long)eh * B * M * D;
  TV* y = reinterpret_cast<TV*>(g.y) + (long long)eh * B * M * Dv;
  float* cl = g.cl + (long long)eh * B * M;
  const float* cr = g.cr + ((long long)eh * M + m) * B;

  for (int j = warp; j < B; j += kWarps) {
    // aggregated query of row j (the query itself on the first pass: left factor = identity)
    float crj = 1.0f;
    if (first) {
      const TQ* qrow = token_row<TQ>(g.q, e, h, m * B + j, g.pad_off, g.N);
      for (int d = lane; d < D; d += 32) avec[d] = qrow ? Cvt<TQ>::to_f(qrow[d]) : 0.f;
    } else {
      for (int d = lane; d < D; d += 32) avec[d] = Cvt<TQ>::to_f(ar[(long long)j * D + d]);
      crj = cr[j];
    }
    __syncwarp();
    const float denom_c = crj + kEps;

    float vmax = -INFINITY;
    for (int i = lane; i < B; i += 32) {
      const TQ* krow = token_row<TQ>(g.k, e, h, m * B + i, g.pad_off, g.N);
      float dot = krow ? dot_row<TQ>(avec, krow, D) : 0.f;
      float x = (g.sm_scale * round_through<TQ>(dot)) / denom_c;
      if (!token_valid(g, e, m * B + i)) x = -INFINITY;
      rbuf[i] = x;
      vmax = fmaxf(vmax, x);
    }
    vmax = fmaxf(warp_max(vmax), kEps);  // the row maximum is clamped from below (:14-16)
    float vsum = 0.f;
    for (int i = lane; i < B; i += 32) {
      float ex = expf(rbuf[i] - vmax);
      rbuf[i] = ex;
      vsum += ex;
    }
    vsum = warp_sum(vsum) + kEps;
    float ent = 0.f;
    for (int i = lane; i < B; i += 32) {
      float r = fmaxf(rbuf[i] / vsum, kTiny);
      ent += r * logf(r);
      rbuf[i] = r;
    }
    ent = warp_sum(ent);
    if (lane == 0) cl[(long long)j * M + m] = ent;
    __syncwarp();

    for (int d = lane; d < D; d += 32) {
      float acc = 0.f;
      for (int i = 0; i < B; ++i) {
        const TQ* krow = token_row<TQ>(g.k, e, h, m * B + i, g.pad_off, g.N);
        if (krow) acc = fmaf(round_through<TQ>(rbuf[i]), Cvt<TQ>::to_f(krow[d]), acc);
      }
      // sm_scale * (r @ k): the product is rounded to storage, scaled, rounded again (:21)
      al[((long long)j * M + m) * D + d] = Cvt<TQ>::from_f(g.sm_scale * round_through<TQ>(acc));
    }
    if (WITH_V) {
      for (int d = lane; d < Dv; d += 32) {
        float acc = 0.f;
        for (int i = 0; i < B; ++i) {
          const TV* vrow = token_row<TV>(g.v, e, h, m * B + i, g.pad_off, g.N);
          if (vrow) acc = fmaf(round_through<TV>(rbuf[i]), Cvt<TV>::to_f(vrow[d]), acc);
        }
        y[((long long)j * M + m) * Dv + d] = Cvt<TV>::from_f(acc);
      }
    }
    __syncwarp();
  }
}

// ---------------------------------------------------------------------------------
// Left-factor stage (reference: ma/ma_torch.py:26-35).  grid = (B, E*H).
// Pass 1: per query l, maximum and sum over m of exp(w[l,m]).  Pass 2: per m, the
// normalised column, its sum (cr) and the weighted sum of queries (ar); the logits are
// recomputed with the same operand order, so they are bit-identical to pass 1.
// Shared memory: kWarps*(D + M) + 3*M floats.
// ---------------------------------------------------------------------------------
template <typename TQ>
__global__ void __launch_bounds__(kThreads) left_stage_kernel(const Geometry g) {
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = blockIdx.x, eh = blockIdx.y;
  const int e = eh / g.H, h = eh % g.H;
  const int B = g.B, D = g.D, M = g.M;
  float* avec = smem + warp * (D + M);
  float* rbuf = avec + D;
  float* s_max = smem + kWarps * (D + M);
  float* s_sum = s_max + M;
  float* s_ok = s_sum + M;

  const TQ* al = reinterpret_cast<const TQ*>(g.al) + ((long long)eh * B + j) * M * D;
  const float* cl = g.cl + ((long long)eh * B + j) * M;
  TQ* ar = reinterpret_cast<TQ*>(g.ar) + (long long)eh * M * B * D;
  float* cr = g.cr + (long long)eh * M * B;

  for (int l = warp; l < M; l += kWarps) {
    const TQ* qrow = token_row<TQ>(g.q, e, h, l * B + j, g.pad_off, g.N);
    for (int d = lane; d < D; d += 32) avec[d] = qrow ? Cvt<TQ>::to_f(qrow[d]) : 0.f;
    __syncwarp();
    float vmax = -INFINITY;
    for (int mm = lane; mm < M; mm += 32) {
      float w = round_through<TQ>(dot_row<TQ>(avec, al + (long long)mm * D, D)) - cl[mm];
      rbuf[mm] = w;
      vmax = fmaxf(vmax, w);
    }
    vmax = warp_max(vmax);
    float vsum = 0.f;
    for (int mm = lane; mm < M; mm += 32) vsum += expf(rbuf[mm] - vmax);
    vsum = warp_sum(vsum);
    if (lane == 0) {
      s_max[l] = vmax;
      s_sum[l] = vsum;
      s_ok[l] = token_valid(g, e, l * B + j) ? 1.f : 0.f;
    }
    __syncwarp();
  }
  __syncthreads();

  for (int mm = warp; mm < M; mm += kWarps) {
    for (int d = lane; d < D; d += 32) avec[d] = Cvt<TQ>::to_f(al[(long long)mm * D + d]);
    __syncwarp();
    const float c = cl[mm];
    float colsum = 0.f;
    for (int l = lane; l < M; l += 32) {
      const TQ* qrow = token_row<TQ>(g.q, e, h, l * B + j, g.pad_off, g.N);
      float dot = 0.f;
      if (qrow) {
        // same products in the same order as pass 1 (fmaf(a, b, acc) with a, b swapped is identical)
        for (int d = 0; d < D; ++d) dot = fmaf(Cvt<TQ>::to_f(qrow[d]), avec[d], dot);
      }
      float w = round_through<TQ>(dot) - c;
      float p = s_ok[l] * (expf(w - s_max[l]) / s_sum[l]);
      rbuf[l] = p;
      colsum += p;
    }
    colsum = warp_sum(colsum);
    if (lane == 0) cr[(long long)mm * B + j] = colsum;
    __syncwarp();
    for (int d = lane; d < D; d += 32) {
      float acc = 0.f;
      for (int l = 0; l < M; ++l) {
        const TQ* qrow = token_row<TQ>(g.q, e, h, l * B + j, g.pad_off, g.N);
        if (qrow) acc = fmaf(round_through<TQ>(rbuf[l]), Cvt<TQ>::to_f(qrow[d]), acc);
      }
      ar[((long long)mm * B + j) * D + d] = Cvt<TQ>::from_f(acc);
    }
    __syncwarp();
  }
}

// ---------------------------------------------------------------------------------
// Output stage (reference: ma/ma_torch.py:55-62).  grid = (B, E*H).  No query mask:
// every real token gets an output row.  Shared memory: kWarps*(D + M) floats.
// ---------------------------------------------------------------------------------
template <typename TQ, typename TV>
__global__ void __launch_bounds__(kThreads) output_stage_kernel(const Geometry g) {
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = blockIdx.x, eh = blockIdx.y;
  const int e = eh / g.H, h = eh % g.H;
  const int B = g.B, D = g.D, Dv = g.Dv, M = g.M;
  float* avec = smem + warp * (D + M);
  float* rbuf = avec + D;

  const TQ* al = reinterpret_cast<const TQ*>(g.al) + ((long long)eh * B + j) * M * D;
  const float* cl = g.cl + ((long long)eh * B + j) * M;
  const TV* y = reinterpret_cast<const TV*>(g.y) + ((long long)eh * B + j) * M * Dv;

  for (int l = warp; l < M; l += kWarps) {
    const int n = l * B + j - g.pad_off;
    if (n < 0 || n >= g.N) continue;  // padding rows are dropped from the output (:108)
    const TQ* qrow = token_row<TQ>(g.q, e, h, l * B + j, g.pad_off, g.N);
    for (int d = lane; d < D; d += 32) avec[d] = Cvt<TQ>::to_f(qrow[d]);
    __syncwarp();
    float vmax = -INFINITY;
    for (int mm = lane; mm < M; mm += 32) {
      float w = round_through<TQ>(dot_row<TQ>(avec, al + (long long)mm * D, D)) - cl[mm];
      rbuf[mm] = w;
      vmax = fmaxf(vmax, w);
    }
    vmax = warp_max(vmax);
    float vsum = 0.f;
    for (int mm = lane; mm < M; mm += 32) {
      float ex = expf(rbuf[mm] - vmax);
      rbuf[mm] = ex;
      vsum += ex;
    }
    vsum = warp_sum(vsum);
    __syncwarp();
    TV* orow = reinterpret_cast<TV*>(const_cast<void*>(g.out.ptr)) + (long long)e * g.out.se +
               (long long)h * g.out.sh + (long long)n * g.out.sn;
    for (int d = lane; d < Dv; d += 32) {
      float acc = 0.f;
      for (int mm = 0; mm < M; ++mm)
        acc = fmaf(round_through<TV>(rbuf[mm] / vsum), Cvt<TV>::to_f(y[(long long)mm * Dv + d]), acc);
      orow[d] = Cvt<TV>::from_f(acc);
    }
    __syncwarp();
  }
}

template <typename TQ, typename TV>
cudaError_t launch_typed(const Geometry& g, StageKind kind, bool first, cudaStream_t stream) {
  const size_t smem = generic_stage_smem_bytes(g, kind);
  const dim3 block(kThreads);
  const int EH = g.E * g.H;
  auto raise = [&](const void* fn) -> cudaError_t {
    if (smem > 48 * 1024) return cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return cudaSuccess;
  };
  cudaError_t err = cudaSuccess;
  switch (kind) {
    case kStageRight:
      if ((err = raise((const void*)right_stage_kernel<TQ, TV, false>)) != cudaSuccess) return err;
      right_stage_kernel<TQ, TV, false><<<dim3(g.M, EH), block, smem, stream>>>(g, first ? 1 : 0);
      break;
    case kStageRightWithV:
      if ((err = raise((const void*)right_stage_kernel<TQ, TV, true>)) != cudaSuccess) return err;
      right_stage_kernel<TQ, TV, true><<<dim3(g.M, EH), block, smem, stream>>>(g, first ? 1 : 0);
      break;
    case kStageLeft:
      if ((err = raise((const void*)left_stage_kernel<TQ>)) != cudaSuccess) return err;
      left_stage_kernel<TQ><<<dim3(g.B, EH), block, smem, stream>>>(g);
      break;
    case kStageOutput:
      if ((err = raise((const void*)output_stage_kernel<TQ, TV>)) != cudaSuccess) return err;
      output_stage_kernel<TQ, TV><<<dim3(g.B, EH), block, smem, stream>>>(g);
      break;
  }
  return cudaGetLastError();
}

}  // namespace

size_t generic_stage_smem_bytes(const Geometry& g, StageKind kind) {
  const size_t keys = (kind == kStageRight || kind == kStageRightWithV) ? g.B : g.M;
  size_t floats = (size_t)kWarps * (g.D + keys);
  if (kind == kStageLeft) floats += 3 * (size_t)g.M;
  return floats * sizeof(float);
}

cudaError_t launch_generic_stage(const Geometry& g, int qk_dtype, int v_dtype, StageKind kind, bool first,
                                 cudaStream_t stream) {
  if (qk_dtype == MA_B200_F32 && v_dtype == MA_B200_F32) return launch_typed<float, float>(g, kind, first, stream);
  if (qk_dtype == MA_B200_BF16 && v_dtype == MA_B200_BF16)
    return launch_typed<__nv_bfloat16, __nv_bfloat16>(g, kind, first, stream);
  if (qk_dtype == MA_B200_F16 && v_dtype == MA_B200_F16) return launch_typed<__half, __half>(g, kind, first, stream);
  if (qk_dtype == MA_B200_BF16 && v_dtype == MA_B200_F32)
    return launch_typed<__nv_bfloat16, float>(g, kind, first, stream);
  if (qk_dtype == MA_B200_F16 && v_dtype == MA_B200_F32) return launch_typed<__half, float>(g, kind, first, stream);
  return cudaErrorInvalidValue;
}

}  // namespace ma
