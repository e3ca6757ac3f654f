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
// axis for the weighted sums.  The operand tiles of a CTA are converted to fp32 and kept in shared
// memory when they fit (see "Operand tiles in shared memory" below); otherwise their rows are read
// straight from global memory.
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
#pragma unroll 8
  for (int d = 0; d < D; ++d) acc = fmaf(a[d], Cvt<T>::to_f(row[d]), acc);
  return acc;
}

// The same dot product with the row already converted to fp32 in shared memory.
__device__ __forceinline__ float dot_smem(const float* __restrict__ a, const float* __restrict__ row, int D) {
  float acc = 0.f;
#pragma unroll 8
  for (int d = 0; d < D; ++d) acc = fmaf(a[d], row[d], acc);
  return acc;
}

// Token row of a (E,H,N,W) view for padded position p, or nullptr when p is padding.
template <typename T>
__device__ __forceinline__ const T* token_row(const View4& t, int e, int h, int p, int pad_off, int N) {
  int n = p - pad_off;
  if (n < 0 || n >= N) return nullptr;
  return reinterpret_cast<const T*>(t.ptr) + (long long)e * t.se + (long long)h * t.sh + (long long)n * t.sn;
}

// Operand tiles in shared memory.  When they fit, the rows a CTA works on are converted to fp32 once and
// kept in shared memory with a row pitch of W + 1 floats (lanes that walk down a column of rows then hit
// 32 different banks); rows that do not exist (padding) are zero, which gives the same sums as skipping
// them.  Every product and every sum is formed in the same order as on the path that reads the rows from
// global memory, so the two paths return the same bits; the staged one just does not issue one
// uncoalesced global load per multiply.
enum { kStageKeys = 1, kStageValues = 2, kStageQueries = 4 };

// rows `r` = 0..rows-1 of a user tensor at padded positions p0 + r * pstep
template <typename T>
__device__ __forceinline__ void stage_token_rows(float* dst, const View4& t, int e, int h, int p0, int pstep, int rows,
                                                 int W, const Geometry& g) {
  for (int idx = threadIdx.x; idx < rows * W; idx += blockDim.x) {
    const int r = idx / W, d = idx - r * W;
    const T* row = token_row<T>(t, e, h, p0 + r * pstep, g.pad_off, g.N);
    dst[r * (W + 1) + d] = row ? Cvt<T>::to_f(row[d]) : 0.f;
  }
}
// rows of a dense (rows, W) state tensor
template <typename T>
__device__ __forceinline__ void stage_dense_rows(float* dst, const T* src, int rows, int W) {
  for (int idx = threadIdx.x; idx < rows * W; idx += blockDim.x) {
    const int r = idx / W, d = idx - r * W;
    dst[r * (W + 1) + d] = Cvt<T>::to_f(src[idx]);
  }
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
__global__ void __launch_bounds__(kThreads) right_stage_kernel(const Geometry g, const int first, const int staged) {
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m = blockIdx.y, eh = blockIdx.x;  // E*H on x: no 65535 limit
  const int e = eh / g.H, h = eh % g.H;
  const int B = g.B, D = g.D, Dv = g.Dv, M = g.M;
  float* avec = smem + warp * (D + B);
  float* rbuf = avec + D;
  float* sK = nullptr;
  float* sV = nullptr;
  {
    float* next = smem + kWarps * (D + B);
    if (staged & kStageKeys) { sK = next; next += (size_t)B * (D + 1); }
    if (WITH_V && (staged & kStageValues)) sV = next;
    if (sK) stage_token_rows<TQ>(sK, g.k, e, h, m * B, 1, B, D, g);
    if (sV) stage_token_rows<TV>(sV, g.v, e, h, m * B, 1, B, Dv, g);
    if (sK || sV) __syncthreads();
  }

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
      float dot;
      if (sK) {
        dot = dot_smem(avec, sK + (size_t)i * (D + 1), D);
      } else {
        const TQ* krow = token_row<TQ>(g.k, e, h, m * B + i, g.pad_off, g.N);
        dot = krow ? dot_row<TQ>(avec, krow, D) : 0.f;
      }
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
      if (sK) {
#pragma unroll 8
        for (int i = 0; i < B; ++i) acc = fmaf(round_through<TQ>(rbuf[i]), sK[(size_t)i * (D + 1) + d], acc);
      } else {
        for (int i = 0; i < B; ++i) {
          const TQ* krow = token_row<TQ>(g.k, e, h, m * B + i, g.pad_off, g.N);
          if (krow) acc = fmaf(round_through<TQ>(rbuf[i]), Cvt<TQ>::to_f(krow[d]), acc);
        }
      }
      // sm_scale * (r @ k): the product is rounded to storage, scaled, rounded again (:21)
      al[((long long)j * M + m) * D + d] = Cvt<TQ>::from_f(g.sm_scale * round_through<TQ>(acc));
    }
    if (WITH_V) {
      for (int d = lane; d < Dv; d += 32) {
        float acc = 0.f;
        if (sV) {
#pragma unroll 8
          for (int i = 0; i < B; ++i) acc = fmaf(round_through<TV>(rbuf[i]), sV[(size_t)i * (Dv + 1) + d], acc);
        } else {
          for (int i = 0; i < B; ++i) {
            const TV* vrow = token_row<TV>(g.v, e, h, m * B + i, g.pad_off, g.N);
            if (vrow) acc = fmaf(round_through<TV>(rbuf[i]), Cvt<TV>::to_f(vrow[d]), acc);
          }
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
__global__ void __launch_bounds__(kThreads) left_stage_kernel(const Geometry g, const int staged) {
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = blockIdx.y, eh = blockIdx.x;
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
  float* sAL = nullptr;  // al[j]: (M, D)
  float* sQ = nullptr;   // q column j: rows l = 0..M-1
  {
    float* next = s_ok + M;
    if (staged & kStageKeys) { sAL = next; next += (size_t)M * (D + 1); }
    if (staged & kStageQueries) sQ = next;
    if (sAL) stage_dense_rows<TQ>(sAL, al, M, D);
    if (sQ) stage_token_rows<TQ>(sQ, g.q, e, h, j, B, M, D, g);
    if (sAL || sQ) __syncthreads();
  }

  for (int l = warp; l < M; l += kWarps) {
    const TQ* qrow = token_row<TQ>(g.q, e, h, l * B + j, g.pad_off, g.N);
    for (int d = lane; d < D; d += 32) avec[d] = qrow ? Cvt<TQ>::to_f(qrow[d]) : 0.f;
    __syncwarp();
    float vmax = -INFINITY;
    for (int mm = lane; mm < M; mm += 32) {
      const float dot = sAL ? dot_smem(avec, sAL + (size_t)mm * (D + 1), D) : dot_row<TQ>(avec, al + (long long)mm * D, D);
      float w = round_through<TQ>(dot) - cl[mm];
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
    for (int d = lane; d < D; d += 32) avec[d] = sAL ? sAL[(size_t)mm * (D + 1) + d] : Cvt<TQ>::to_f(al[(long long)mm * D + d]);
    __syncwarp();
    const float c = cl[mm];
    float colsum = 0.f;
    for (int l = lane; l < M; l += 32) {
      float dot = 0.f;
      // same products in the same order as pass 1 (fmaf(a, b, acc) with a, b swapped is identical)
      if (sQ) {
        const float* qs = sQ + (size_t)l * (D + 1);
#pragma unroll 8
        for (int d = 0; d < D; ++d) dot = fmaf(qs[d], avec[d], dot);
      } else {
        const TQ* qrow = token_row<TQ>(g.q, e, h, l * B + j, g.pad_off, g.N);
        if (qrow)
#pragma unroll 8
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
      if (sQ) {
#pragma unroll 8
        for (int l = 0; l < M; ++l) acc = fmaf(round_through<TQ>(rbuf[l]), sQ[(size_t)l * (D + 1) + d], acc);
      } else {
        for (int l = 0; l < M; ++l) {
          const TQ* qrow = token_row<TQ>(g.q, e, h, l * B + j, g.pad_off, g.N);
          if (qrow) acc = fmaf(round_through<TQ>(rbuf[l]), Cvt<TQ>::to_f(qrow[d]), acc);
        }
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
__global__ void __launch_bounds__(kThreads) output_stage_kernel(const Geometry g, const int staged) {
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = blockIdx.y, eh = blockIdx.x;
  const int e = eh / g.H, h = eh % g.H;
  const int B = g.B, D = g.D, Dv = g.Dv, M = g.M;
  float* avec = smem + warp * (D + M);
  float* rbuf = avec + D;

  const TQ* al = reinterpret_cast<const TQ*>(g.al) + ((long long)eh * B + j) * M * D;
  const float* cl = g.cl + ((long long)eh * B + j) * M;
  const TV* y = reinterpret_cast<const TV*>(g.y) + ((long long)eh * B + j) * M * Dv;
  float* sAL = nullptr;  // al[j]: (M, D)
  float* sY = nullptr;   // y[j]: (M, Dv)
  {
    float* next = smem + kWarps * (D + M);
    if (staged & kStageKeys) { sAL = next; next += (size_t)M * (D + 1); }
    if (staged & kStageValues) sY = next;
    if (sAL) stage_dense_rows<TQ>(sAL, al, M, D);
    if (sY) stage_dense_rows<TV>(sY, y, M, Dv);
    if (sAL || sY) __syncthreads();
  }

  for (int l = warp; l < M; l += kWarps) {
    const int n = l * B + j - g.pad_off;
    if (n < 0 || n >= g.N) continue;  // padding rows are dropped from the output (:108)
    const TQ* qrow = token_row<TQ>(g.q, e, h, l * B + j, g.pad_off, g.N);
    for (int d = lane; d < D; d += 32) avec[d] = Cvt<TQ>::to_f(qrow[d]);
    __syncwarp();
    float vmax = -INFINITY;
    for (int mm = lane; mm < M; mm += 32) {
      const float dot = sAL ? dot_smem(avec, sAL + (size_t)mm * (D + 1), D) : dot_row<TQ>(avec, al + (long long)mm * D, D);
      float w = round_through<TQ>(dot) - cl[mm];
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
    // the factor is normalised and rounded to the value type once per row (:59-61)
    for (int mm = lane; mm < M; mm += 32) rbuf[mm] = round_through<TV>(rbuf[mm] / vsum);
    __syncwarp();
    TV* orow = reinterpret_cast<TV*>(const_cast<void*>(g.out.ptr)) + (long long)e * g.out.se +
               (long long)h * g.out.sh + (long long)n * g.out.sn;
    for (int d = lane; d < Dv; d += 32) {
      float acc = 0.f;
      if (sY) {
#pragma unroll 8
        for (int mm = 0; mm < M; ++mm) acc = fmaf(rbuf[mm], sY[(size_t)mm * (Dv + 1) + d], acc);
      } else {
#pragma unroll 4
        for (int mm = 0; mm < M; ++mm) acc = fmaf(rbuf[mm], Cvt<TV>::to_f(y[(long long)mm * Dv + d]), acc);
      }
      orow[d] = Cvt<TV>::from_f(acc);
    }
    __syncwarp();
  }
}

// ---------------------------------------------------------------------------------
// Small tiles: block size and block count up to 16 (the reference's own CPU-sized configuration,
// 16 x 16 blocks of fp32).  Same arithmetic, same rounding points and the same order of every sum as the
// kernels above - the results are bit-identical - but one THREAD per logit instead of one warp per row:
// thread t of the 256 owns (row t / 16, key t % 16) of the 16 x 16 tile, a row's softmax is a reduction
// over a half-warp, and the weighted sums are taken by the same thread grid as (row, 16 features at a
// time).  A row-per-warp kernel leaves half of its lanes idle on such tiles and spends most of its
// instructions on loop and address arithmetic.
// ---------------------------------------------------------------------------------
constexpr int kSmallMax = 16;

__device__ __forceinline__ float half_max(float v) {  // over the 16 lanes that share a row
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float half_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// rows r = 0..15 (zero beyond `rows`) of a user tensor at padded positions p0 + r * pstep, pitch W + 1
template <typename T>
__device__ __forceinline__ void small_token_rows(float* dst, const View4& t, int e, int h, int p0, int pstep, int rows,
                                                 int W, const Geometry& g) {
  const int r = threadIdx.x >> 4, c = threadIdx.x & 15;
  const T* row = r < rows ? token_row<T>(t, e, h, p0 + r * pstep, g.pad_off, g.N) : nullptr;
  for (int d = c; d < W; d += 16) dst[r * (W + 1) + d] = row ? Cvt<T>::to_f(row[d]) : 0.f;
}
template <typename T>
__device__ __forceinline__ void small_dense_rows(float* dst, const T* src, int rows, int W) {
  const int r = threadIdx.x >> 4, c = threadIdx.x & 15;
  for (int d = c; d < W; d += 16) dst[r * (W + 1) + d] = r < rows ? Cvt<T>::to_f(src[(long long)r * W + d]) : 0.f;
}
// sum_i w[i] * rows[i][d] in increasing i, for this thread's row weights and the features d = c, c + 16, ...
template <typename TR, typename F>
__device__ __forceinline__ void small_weighted_sums(const float* w, const float* rows, int n, int W, int c, F&& emit) {
  for (int d = c; d < W; d += 16) {
    float acc = 0.f;
#pragma unroll 8
    for (int i = 0; i < n; ++i) acc = fmaf(round_through<TR>(w[i]), rows[i * (W + 1) + d], acc);
    emit(d, acc);
  }
}

template <typename TQ, typename TV, bool WITH_V>
__global__ void __launch_bounds__(256) small_right_kernel(const Geometry g, const int first) {
  extern __shared__ float smem[];
  const int m = blockIdx.y, eh = blockIdx.x, e = eh / g.H, h = eh % g.H;
  const int B = g.B, D = g.D, Dv = g.Dv, M = g.M;
  const int j = threadIdx.x >> 4, i = threadIdx.x & 15;
  float* sA = smem;                       // ar (or q) rows of the block
  float* sK = sA + kSmallMax * (D + 1);
  float* sV = sK + kSmallMax * (D + 1);
  float* sR = sV + (WITH_V ? kSmallMax * (Dv + 1) : 0);  // [16][17] factor rows
  if (first) small_token_rows<TQ>(sA, g.q, e, h, m * B, 1, B, D, g);
  else small_dense_rows<TQ>(sA, reinterpret_cast<const TQ*>(g.ar) + ((long long)eh * M + m) * B * D, B, D);
  small_token_rows<TQ>(sK, g.k, e, h, m * B, 1, B, D, g);
  if (WITH_V) small_token_rows<TV>(sV, g.v, e, h, m * B, 1, B, Dv, g);
  __syncthreads();

  const bool live = j < B && i < B;
  float x = -INFINITY;
  if (live) {
    const float crj = first ? 1.0f : g.cr[((long long)eh * M + m) * B + j];
    const float dot = dot_smem(sA + j * (D + 1), sK + i * (D + 1), D);
    x = (g.sm_scale * round_through<TQ>(dot)) / (crj + kEps);
    if (!token_valid(g, e, m * B + i)) x = -INFINITY;
  }
  const float vmax = fmaxf(half_max(x), kEps);
  const float ex = live ? expf(x - vmax) : 0.f;
  const float vsum = half_sum(ex) + kEps;
  const float r = fmaxf(ex / vsum, kTiny);
  const float ent = half_sum(live ? r * logf(r) : 0.f);
  if (live && i == 0) g.cl[((long long)eh * B + j) * M + m] = ent;
  sR[j * 17 + i] = live ? r : 0.f;
  __syncthreads();
  if (j < B) {
    TQ* al = reinterpret_cast<TQ*>(g.al) + (((long long)eh * B + j) * M + m) * D;
    // sm_scale * (r @ k): the product is rounded to storage, scaled, rounded again (:21)
    small_weighted_sums<TQ>(sR + j * 17, sK, B, D, i,
                            [&](int d, float acc) { al[d] = Cvt<TQ>::from_f(g.sm_scale * round_through<TQ>(acc)); });
    if (WITH_V) {
      TV* y = reinterpret_cast<TV*>(g.y) + (((long long)eh * B + j) * M + m) * Dv;
      small_weighted_sums<TV>(sR + j * 17, sV, B, Dv, i, [&](int d, float acc) { y[d] = Cvt<TV>::from_f(acc); });
    }
  }
}

template <typename TQ>
__global__ void __launch_bounds__(256) small_left_kernel(const Geometry g) {
  extern __shared__ float smem[];
  const int j = blockIdx.y, eh = blockIdx.x, e = eh / g.H, h = eh % g.H;
  const int B = g.B, D = g.D, M = g.M;
  const int l = threadIdx.x >> 4, mm = threadIdx.x & 15;
  float* sQ = smem;                        // query column j: rows l
  float* sAL = sQ + kSmallMax * (D + 1);   // al[j]: rows m
  float* sP = sAL + kSmallMax * (D + 1);   // [m][17]: factor, transposed for the sums over l
  small_token_rows<TQ>(sQ, g.q, e, h, j, B, M, D, g);
  small_dense_rows<TQ>(sAL, reinterpret_cast<const TQ*>(g.al) + ((long long)eh * B + j) * M * D, M, D);
  __syncthreads();
  const bool live = l < M && mm < M;
  float w = -INFINITY;
  if (live) {
    const float dot = dot_smem(sQ + l * (D + 1), sAL + mm * (D + 1), D);
    w = round_through<TQ>(dot) - g.cl[((long long)eh * B + j) * M + mm];
  }
  const float vmax = half_max(w);
  const float vsum = half_sum(live ? expf(w - vmax) : 0.f);
  float p = 0.f;
  if (live) p = (token_valid(g, e, l * B + j) ? 1.f : 0.f) * (expf(w - vmax) / vsum);
  sP[mm * 17 + l] = p;
  __syncthreads();
  if (l < M) {  // this thread group now works on block row m = l
    const int m = l, c = mm;
    const float* prow = sP + m * 17;
    if (c == 0) {
      // the sum over l in the order of a butterfly reduction over 32 lanes of which the upper 16 hold zeros
      float t[16];
#pragma unroll
      for (int q = 0; q < 16; ++q) t[q] = q < M ? prow[q] : 0.f;
#pragma unroll
      for (int o = 8; o > 0; o >>= 1)
#pragma unroll
        for (int q = 0; q < o; ++q) t[q] = t[q] + t[q + o];
      g.cr[((long long)eh * M + m) * B + j] = t[0];
    }
    TQ* ar = reinterpret_cast<TQ*>(g.ar) + (((long long)eh * M + m) * B + j) * D;
    small_weighted_sums<TQ>(prow, sQ, M, D, c, [&](int d, float acc) { ar[d] = Cvt<TQ>::from_f(acc); });
  }
}

template <typename TQ, typename TV>
__global__ void __launch_bounds__(256) small_output_kernel(const Geometry g) {
  extern __shared__ float smem[];
  const int j = blockIdx.y, eh = blockIdx.x, e = eh / g.H, h = eh % g.H;
  const int B = g.B, D = g.D, Dv = g.Dv, M = g.M;
  const int l = threadIdx.x >> 4, mm = threadIdx.x & 15;
  float* sQ = smem;
  float* sAL = sQ + kSmallMax * (D + 1);
  float* sY = sAL + kSmallMax * (D + 1);
  float* sP = sY + kSmallMax * (Dv + 1);  // [l][17]
  small_token_rows<TQ>(sQ, g.q, e, h, j, B, M, D, g);
  small_dense_rows<TQ>(sAL, reinterpret_cast<const TQ*>(g.al) + ((long long)eh * B + j) * M * D, M, D);
  small_dense_rows<TV>(sY, reinterpret_cast<const TV*>(g.y) + ((long long)eh * B + j) * M * Dv, M, Dv);
  __syncthreads();
  const bool live = l < M && mm < M;
  float w = -INFINITY;
  if (live) {
    const float dot = dot_smem(sQ + l * (D + 1), sAL + mm * (D + 1), D);
    w = round_through<TQ>(dot) - g.cl[((long long)eh * B + j) * M + mm];
  }
  const float vmax = half_max(w);
  const float ex = live ? expf(w - vmax) : 0.f;
  const float vsum = half_sum(ex);
  sP[l * 17 + mm] = live ? round_through<TV>(ex / vsum) : 0.f;
  __syncthreads();
  const int n = l * B + j - g.pad_off;
  if (l < M && n >= 0 && n < g.N) {  // padding rows are dropped from the output (:108)
    TV* orow = reinterpret_cast<TV*>(const_cast<void*>(g.out.ptr)) + (long long)e * g.out.se + (long long)h * g.out.sh +
               (long long)n * g.out.sn;
    small_weighted_sums<float>(sP + l * 17, sY, M, Dv, mm, [&](int d, float acc) { orow[d] = Cvt<TV>::from_f(acc); });
  }
}

size_t small_smem_bytes(const Geometry& g) {
  return ((size_t)kSmallMax * (2 * (g.D + 1) + (g.Dv + 1)) + kSmallMax * 17) * sizeof(float);
}
int g_general_form_only = 0;  // test hook: 1 = never take the small-tile kernels
bool small_tiles(const Geometry& g) {
  if (g_general_form_only) return false;
  return g.B <= kSmallMax && g.M <= kSmallMax && small_smem_bytes(g) <= 48 * 1024;
}

// Which operand tiles go to shared memory (kStage* bits) and the bytes that takes on top of `base`.
// Tiles are added while the total stays within 160 KB; a tile that does not fit is read from global
// memory as before (the explicit-matrix case, whose value rows are N wide, is the usual one).
int staging_plan(const Geometry& g, StageKind kind, size_t base, size_t* total) {
  const size_t limit = 160 * 1024;
  int flags = 0;
  size_t bytes = base;
  auto add = [&](int bit, size_t rows, size_t width) {
    const size_t need = rows * (width + 1) * sizeof(float);
    if (bytes + need <= limit) { flags |= bit; bytes += need; }
  };
  switch (kind) {
    case kStageRight: add(kStageKeys, g.B, g.D); break;
    case kStageRightWithV: add(kStageKeys, g.B, g.D); add(kStageValues, g.B, g.Dv); break;
    case kStageLeft: add(kStageKeys, g.M, g.D); add(kStageQueries, g.M, g.D); break;
    case kStageOutput: add(kStageKeys, g.M, g.D); add(kStageValues, g.M, g.Dv); break;
  }
  *total = bytes;
  return flags;
}

template <typename TQ, typename TV>
cudaError_t launch_typed(const Geometry& g, StageKind kind, bool first, cudaStream_t stream) {
  size_t smem = 0;
  const int staged = staging_plan(g, kind, generic_stage_smem_bytes(g, kind), &smem);
  const dim3 block(kThreads);
  const int EH = g.E * g.H;
  auto raise = [&](const void* fn) -> cudaError_t {
    if (smem > 48 * 1024) return cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return cudaSuccess;
  };
  cudaError_t err = cudaSuccess;
  if (small_tiles(g)) {
    const size_t sm = small_smem_bytes(g);
    switch (kind) {
      case kStageRight: small_right_kernel<TQ, TV, false><<<dim3(EH, g.M), 256, sm, stream>>>(g, first ? 1 : 0); break;
      case kStageRightWithV: small_right_kernel<TQ, TV, true><<<dim3(EH, g.M), 256, sm, stream>>>(g, first ? 1 : 0); break;
      case kStageLeft: small_left_kernel<TQ><<<dim3(EH, g.B), 256, sm, stream>>>(g); break;
      case kStageOutput: small_output_kernel<TQ, TV><<<dim3(EH, g.B), 256, sm, stream>>>(g); break;
    }
    return cudaGetLastError();
  }
  switch (kind) {
    case kStageRight:
      if ((err = raise((const void*)right_stage_kernel<TQ, TV, false>)) != cudaSuccess) return err;
      right_stage_kernel<TQ, TV, false><<<dim3(EH, g.M), block, smem, stream>>>(g, first ? 1 : 0, staged);
      break;
    case kStageRightWithV:
      if ((err = raise((const void*)right_stage_kernel<TQ, TV, true>)) != cudaSuccess) return err;
      right_stage_kernel<TQ, TV, true><<<dim3(EH, g.M), block, smem, stream>>>(g, first ? 1 : 0, staged);
      break;
    case kStageLeft:
      if ((err = raise((const void*)left_stage_kernel<TQ>)) != cudaSuccess) return err;
      left_stage_kernel<TQ><<<dim3(EH, g.B), block, smem, stream>>>(g, staged);
      break;
    case kStageOutput:
      if ((err = raise((const void*)output_stage_kernel<TQ, TV>)) != cudaSuccess) return err;
      output_stage_kernel<TQ, TV><<<dim3(EH, g.B), block, smem, stream>>>(g, staged);
      break;
  }
  return cudaGetLastError();
}

}  // namespace

void generic_set_general_form_only(int on) { g_general_form_only = on ? 1 : 0; }

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
