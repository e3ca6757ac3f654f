// Tensor-core stage kernels for sm_100a: TMA tile loads into 128B-swizzled shared
// memory, tcgen05.mma block contractions with fp32 accumulators in tensor memory, a
// fused row softmax that reads the accumulator with tcgen05.ld (one row per thread),
// and TMA stores of the stage result.
//
// Shapes served by the one-tile-per-CTA kernels of this file: 16-bit storage (bf16 / fp16), D = Dv = 64,
// block size = block count = 128, N = 128*128, no mask and no padding.  (The tensor maps built here also
// serve the fused kernel, which takes block size = block count = 64 as well.)
//
// One CTA works on one 128-row tile:
//   right-factor stages (reference: ma/ma_torch.py:10-23, :38-52): rows j of key block m
//       S[j,i]  = <ar[m,j], k[m,i]>                       (tcgen05, K-major x K-major)
//       P[j,i]  = exp(x - max(rowmax x, eps)),  x = sm_scale*S/(cr+eps)
//       O[j,:]  = P @ [k[m] | v[m]]                        (tcgen05, P from shared memory)
//       al = sm_scale*O_k/(sum+eps), y = O_v/(sum+eps), cl from the sums (see below)
//   left-factor stage (:26-35): column j, rows l (one token per block)
//       S[l,m]  = <q[l,j], al[j,m]>,  P[l,m] = exp(S - cl[m] - rowmax)
//       O[m,:]  = P^T @ [q'[.,j] | s],  q'[l] = q[l]/rowsum[l], s[l] = 1/rowsum[l]
//       ar = O[:, :64], cr = O[:, 64]
//   output stage (:55-62): S, P as in the left-factor stage, O[l,:] = P @ y[j], z = O/rowsum.
//
// The negative entropy cl = sum_i r_i log r_i is evaluated without a logarithm per
// element: with e_i = exp(t_i), t_i = x_i - s, S' = sum e + eps and r_i = e_i/S',
//   sum_i r_i log r_i = (sum_i e_i t_i)/S' - log(S') * (sum_i e_i)/S'.
//
// Every wait on an mbarrier is bounded; on expiry the CTA raises the device status flag,
// drains its own copies, frees its tensor memory and returns.
#include <cuda.h>

#include <mutex>
#include <type_traits>

#include "ma_common.cuh"
#include "ma_sm100.cuh"
#include "ma_tc_plan.cuh"

namespace ma {

// ---------------------------------------------------------------------------------
// Host side: tensor maps
// ---------------------------------------------------------------------------------
namespace {

constexpr int kTile = 128;    // rows per tile = keys per tile
constexpr int kHead = 64;     // head width (elements)
constexpr int kTileBytes = kTile * kHead * 2;
constexpr int kTcThreads = 128;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// 5-D map over 16-bit elements: dims (64, d1, d2, d3, d4), byte strides s1..s4, box (64, b1, b2, 1, 1).
bool encode5(CUtensorMap* map, int dtype, const void* base, const cuuint64_t dims[5], const cuuint64_t strides_bytes[4],
             cuuint32_t b1, cuuint32_t b2) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t gdim[5], gstr[4];
  for (int i = 0; i < 5; ++i) gdim[i] = dims[i];
  for (int i = 0; i < 4; ++i) {
    gstr[i] = strides_bytes[i];
    // a size-1 dimension may carry any stride; give the encoder a legal one
    if (gdim[i + 1] == 1 && (gstr[i] == 0 || gstr[i] % 16 != 0)) gstr[i] = 128;
  }
  const cuuint32_t box[5] = {(cuuint32_t)kHead, b1, b2, 1, 1};
  const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  const CUtensorMapDataType dt = dtype == MA_B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = fn(map, dt, 5, const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

bool view_ok(const View4& t, int E, int H) {
  if (reinterpret_cast<uintptr_t>(t.ptr) % 16 != 0) return false;
  if (t.sn % 8 != 0 || t.sn < kHead) return false;
  if (H > 1 && (t.sh % 8 != 0 || t.sh == 0)) return false;
  if (E > 1 && (t.se % 8 != 0 || t.se == 0)) return false;
  return true;
}

}  // namespace

bool tc_supported(const Geometry& g, int qk_dtype, int v_dtype, const char** why) {
  auto no = [&](const char* w) { *why = w; return false; };
  if (qk_dtype != v_dtype || (qk_dtype != MA_B200_BF16 && qk_dtype != MA_B200_F16))
    return no("needs bf16 or f16 for q, k and v");
  if (g.D != kHead || g.Dv != kHead) return no("needs D = Dv = 64");
  if (!((g.B == kTile && g.M == kTile) || (g.B == kTile / 2 && g.M == kTile / 2)))
    return no("needs block size = block count = 128 (or 64: two blocks per 128-row tile)");
  if (g.N != g.B * g.M) return no("needs N = block size * block count (no padding)");
  if (g.mask != nullptr) return no("mask not handled on this path");
  if ((long long)g.E * g.H > 65535) return no("E*H too large for the grid");
  if (g.q.ptr != nullptr) {  // layout queries pass no pointers
    if (!view_ok(g.q, g.E, g.H) || !view_ok(g.k, g.E, g.H) || !view_ok(g.v, g.E, g.H) || !view_ok(g.out, g.E, g.H))
      return no("q, k, v, out need 16-byte aligned bases and strides that are non-zero multiples of 8 elements");
  }
  if (encode_fn() == nullptr) return no("driver entry point cuTensorMapEncodeTiled not available");
  return true;
}

int tc_plan_create(const Geometry& g, int qk_dtype, TcPlan** out, const char** err) {
  TcPlan* plan = new TcPlan;
  plan->qk_dtype = qk_dtype;
  const cuuint64_t B = g.B, M = g.M, EH = (cuuint64_t)g.E * g.H;
  bool ok = true;
  // A tile is 128 rows.  With block size 128 that is one key block (or one column j: every 128th token);
  // with block size 64 it is two consecutive key blocks (128 consecutive tokens), or two consecutive
  // columns j, j+1 (two boxes of 64 tokens each, rows jj*64 + l).  per = blocks / columns per tile.
  const cuuint64_t per = kTile / B;
  auto user = [&](const View4& t, CUtensorMap* blk, CUtensorMap* col) {
    const cuuint64_t str[4] = {(cuuint64_t)t.sn * 2, (cuuint64_t)t.sn * 2 * B, (cuuint64_t)t.sh * 2,
                               (cuuint64_t)t.se * 2};
    if (blk) {  // tokens as (128, N/128)
      const cuuint64_t bdims[5] = {(cuuint64_t)kHead, (cuuint64_t)kTile, B * M / kTile, (cuuint64_t)g.H, (cuuint64_t)g.E};
      const cuuint64_t bstr[4] = {(cuuint64_t)t.sn * 2, (cuuint64_t)t.sn * 2 * kTile, (cuuint64_t)t.sh * 2,
                                  (cuuint64_t)t.se * 2};
      ok = ok && encode5(blk, qk_dtype, t.ptr, bdims, bstr, kTile, 1);
    }
    if (col) {  // tokens as (B, M): one column j, 128 / per blocks (a tile takes `per` such boxes)
      const cuuint64_t dims[5] = {(cuuint64_t)kHead, B, M, (cuuint64_t)g.H, (cuuint64_t)g.E};
      ok = ok && encode5(col, qk_dtype, t.ptr, dims, str, 1, (cuuint32_t)(kTile / per));
    }
  };
  user(g.q, &plan->maps.q_blk, &plan->maps.q_col);
  user(g.k, &plan->maps.k_blk, nullptr);
  user(g.v, &plan->maps.v_blk, nullptr);
  user(g.out, nullptr, &plan->maps.out_col);
  // workspace tensors (EH, outer, inner, 64), contiguous
  auto scratch = [&](const void* base, cuuint64_t inner, cuuint64_t outer, CUtensorMap* blk, CUtensorMap* col) {
    const cuuint64_t dims[5] = {(cuuint64_t)kHead, inner, outer, EH, 1};
    const cuuint64_t str[4] = {(cuuint64_t)kHead * 2, (cuuint64_t)kHead * 2 * inner,
                               (cuuint64_t)kHead * 2 * inner * outer, (cuuint64_t)kHead * 2 * inner * outer * EH};
    // rows of a head as (128, inner*outer/128): a tile is 128 consecutive rows whatever the block size
    const cuuint64_t bdims[5] = {(cuuint64_t)kHead, (cuuint64_t)kTile, inner * outer / kTile, EH, 1};
    const cuuint64_t bstr[4] = {(cuuint64_t)kHead * 2, (cuuint64_t)kHead * 2 * kTile,
                                (cuuint64_t)kHead * 2 * inner * outer, (cuuint64_t)kHead * 2 * inner * outer * EH};
    ok = ok && encode5(blk, qk_dtype, base, bdims, bstr, kTile, 1);
    ok = ok && encode5(col, qk_dtype, base, dims, str, 1, (cuuint32_t)(kTile / per));
  };
  if (g.T > 1) scratch(g.ar, B, M, &plan->maps.ar_blk, &plan->maps.ar_col);
  else { plan->maps.ar_blk = plan->maps.q_blk; plan->maps.ar_col = plan->maps.q_col; }
  scratch(g.al, M, B, &plan->maps.al_blk, &plan->maps.al_col);
  scratch(g.y, M, B, &plan->maps.y_blk, &plan->maps.y_col);
  if (!ok) {
    delete plan;
    *err = "cuTensorMapEncodeTiled rejected a tensor map";
    return MA_B200_CUDA_ERROR;
  }
  *out = plan;
  return MA_B200_OK;
}

void tc_plan_destroy(TcPlan* plan) { delete plan; }

// ---------------------------------------------------------------------------------
// Device side
// ---------------------------------------------------------------------------------
namespace {

using namespace sm100;

// Shared-memory map (offsets from a 1024-byte aligned base).
constexpr uint32_t kOffA = 0;                    // GEMM1 A operand: ar / q block, or column of q
constexpr uint32_t kOffB = kOffA + kTileBytes;   // GEMM1 B operand: k block, or al[j]
constexpr uint32_t kOffV = kOffB + kTileBytes;   // v block / y[j] / scaled q column (directly after B)
constexpr uint32_t kOffP = kOffV + kTileBytes;   // P or P^T, 128 x 128 16-bit
constexpr uint32_t kOffS = kOffP + 2 * kTileBytes;  // 16 x 128 K-major operand holding 1/rowsum (left stage)
constexpr uint32_t kOffVec = kOffS + 4096;       // 128 floats: log2e * cl[j, :]
constexpr uint32_t kOffBar = kOffVec + 512;      // 3 mbarriers + tensor-memory base
constexpr uint32_t kSmemUsed = kOffBar + 64;
constexpr uint32_t kSmemBytes = kSmemUsed + 1024;  // slack for manual 1024-byte alignment

constexpr uint32_t kTmemCols = 256;  // S: columns 0..127, O: columns 128..255

template <int KIND, typename T>
__global__ void __launch_bounds__(kTcThreads) tc_stage_kernel(const __grid_constant__ TcMaps maps, const Geometry g,
                                                              const int first) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t sA = base + kOffA, sB = base + kOffB, sV = base + kOffV, sP = base + kOffP, sS = base + kOffS;
  float* vec = reinterpret_cast<float*>(base_ptr + kOffVec);
  const uint32_t bar_load = base + kOffBar, bar_mma1 = bar_load + 8, bar_mma2 = bar_load + 16;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + kOffBar + 24);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int tile = blockIdx.x;  // key block m (right stages) or column j (left / output stages)
  const int eh = blockIdx.y, e = eh / g.H, h = eh % g.H;
  constexpr bool kRight = (KIND == kStageRight || KIND == kStageRightWithV);
  constexpr int kFmt = sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? 1 : 0;

  if (tid == 0) {
    mbar_init(bar_load, 1);
    mbar_init(bar_mma1, 1);
    mbar_init(bar_mma2, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(base + kOffBar + 24),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (KIND == kStageLeft) {  // zero the 16 x 128 operand that will carry 1/rowsum in its first row
    uint32_t* z = reinterpret_cast<uint32_t*>(base_ptr + kOffS);
    for (int i = tid; i < 1024; i += kTcThreads) z[i] = 0u;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_row = tmem + ((uint32_t)(warp * 32) << 16);  // this warp's lane quarter

  // ---- loads -------------------------------------------------------------------
  if (tid == 0) {
    if (kRight) {
      mbar_expect_tx(bar_load, (KIND == kStageRightWithV ? 3 : 2) * kTileBytes);
      if (first) tma_load_5d(sA, &maps.q_blk, bar_load, 0, 0, tile, h, e);
      else tma_load_5d(sA, &maps.ar_blk, bar_load, 0, 0, tile, eh, 0);
      tma_load_5d(sB, &maps.k_blk, bar_load, 0, 0, tile, h, e);
      if (KIND == kStageRightWithV) tma_load_5d(sV, &maps.v_blk, bar_load, 0, 0, tile, h, e);
    } else {
      mbar_expect_tx(bar_load, (KIND == kStageOutput ? 3 : 2) * kTileBytes);
      tma_load_5d(sA, &maps.q_col, bar_load, 0, tile, 0, h, e);
      tma_load_5d(sB, &maps.al_blk, bar_load, 0, 0, tile, eh, 0);
      if (KIND == kStageOutput) tma_load_5d(sV, &maps.y_blk, bar_load, 0, 0, tile, eh, 0);
    }
  }
  float row_scale = 0.f;  // right stages: sm_scale / (cr + eps) for this thread's row
  if (kRight) {
    const float crj = first ? 1.0f : g.cr[((long long)eh * g.M + tile) * g.B + tid];
    row_scale = g.sm_scale / (crj + kEps);
  } else {
    vec[tid] = kLog2e * g.cl[((long long)eh * g.B + tile) * g.M + tid];
  }

  bool ok = mbar_wait(bar_load, 0);
  int failed = __syncthreads_or(ok ? 0 : 1);  // also publishes vec[]

  // ---- GEMM 1: S = A * B^T (both K-major, K = 64) ------------------------------------
  if (!failed && tid == 0) {
    tc_fence_after();
    constexpr uint32_t idesc = instr_desc(kFmt, 0, 0, kTile, kTile);
#pragma unroll
    for (int kk = 0; kk < kHead / 16; ++kk)
      mma_f16(tmem, smem_desc(sA + kk * 32, 16), smem_desc(sB + kk * 32, 16), idesc, kk > 0);
    mma_commit(bar_mma1);
  }
  if (!failed) {
    ok = mbar_wait(bar_mma1, 0);
    failed = __syncthreads_or(ok ? 0 : 2);
  }

  float row_sum = 0.f, row_ent = 0.f;
  if (!failed) {
    tc_fence_after();
    // ---- softmax pass 1: row maximum -------------------------------------------------
    float vmax = -INFINITY;
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      float s[32];
      tmem_ld32(tmem_row + c * 32, s);
      if (kRight) {
#pragma unroll
        for (int i = 0; i < 32; ++i) vmax = fmaxf(vmax, s[i]);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) vmax = fmaxf(vmax, fmaf(s[i], kLog2e, -vec[c * 32 + i]));
      }
    }
    // log2-domain multiplier and offset: u = s*mul - off, e = 2^u
    float mul, off;
    if (kRight) {
      const float top = fmaxf(vmax * row_scale, kEps);  // lower clamp on the row maximum
      mul = row_scale * kLog2e;
      off = top * kLog2e;
    } else {
      mul = kLog2e;
      off = vmax;
    }
    // ---- softmax pass 2: exponentials, sums, P to shared memory --------------------------
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      float s[32];
      tmem_ld32(tmem_row + c * 32, s);
      uint32_t packed[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        float u0, u1;
        if (kRight) {
          u0 = fmaf(s[i], mul, -off);
          u1 = fmaf(s[i + 1], mul, -off);
        } else {
          u0 = fmaf(s[i], mul, -vec[c * 32 + i]) - off;
          u1 = fmaf(s[i + 1], mul, -vec[c * 32 + i + 1]) - off;
        }
        const float e0 = ex2(u0), e1 = ex2(u1);
        row_sum += e0 + e1;
        if (kRight) row_ent = fmaf(e0, u0, fmaf(e1, u1, row_ent));
        packed[i >> 1] = pack2<T>(e0, e1);
      }
      // Columns [32c, 32c+32) of row tid.  The bytes land in the same place for both uses of the
      // buffer: as a K-major operand (row = M index, 64-column halves = K blocks) in the right-factor
      // and output stages, and as an MN-major operand holding P^T (row = K index, 64-column halves =
      // M atoms) in the left-factor stage.
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const uint32_t col = c * 32 + q4 * 8;
        const uint32_t addr = sP + (col >> 6) * kTileBytes + swz(tid, (col & 63) >> 3);
        st_shared_v4(addr, packed[q4 * 4], packed[q4 * 4 + 1], packed[q4 * 4 + 2], packed[q4 * 4 + 3]);
      }
    }
    if (KIND == kStageLeft) {
      // scale this thread's query row by 1/rowsum into the second operand buffer, and publish 1/rowsum
      const float inv = 1.0f / row_sum;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        const uint4 v = ld_shared_v4(sA + swz(tid, ch));
        float2 a = unpack2<T>(v.x), b = unpack2<T>(v.y), c2 = unpack2<T>(v.z), d = unpack2<T>(v.w);
        st_shared_v4(sV + swz(tid, ch), pack2<T>(a.x * inv, a.y * inv), pack2<T>(b.x * inv, b.y * inv),
                     pack2<T>(c2.x * inv, c2.y * inv), pack2<T>(d.x * inv, d.y * inv));
      }
      // row 0 of the 16 x 128 K-major operand: element k = tid lives in K-block tid/64
      T* srow = reinterpret_cast<T*>(base_ptr + kOffS + (tid >> 6) * 2048);
      srow[tid & 63] = Cvt<T>::from_f(inv);
    }
    fence_async_smem();
    tc_fence_before();
  }
  __syncthreads();

  // ---- GEMM 2 ------------------------------------------------------------------------
  if (!failed && tid == 0) {
    tc_fence_after();
    const uint32_t tmem_o = tmem + 128;
    if (KIND == kStageRight) {
      // O[j, 0:64] = P[j, :] @ k  (A K-major, B = k tile read MN-major)
      constexpr uint32_t idesc = instr_desc(kFmt, 0, 1, kHead, kTile);
#pragma unroll
      for (int kk = 0; kk < kTile / 16; ++kk)
        mma_f16(tmem_o, smem_desc(sP + (kk >> 2) * kTileBytes + (kk & 3) * 32, 16),
                smem_desc(sB + kk * 2048, kTileBytes), idesc, kk > 0);
    } else if (KIND == kStageRightWithV) {
      // O[j, 0:128] = P[j, :] @ [k | v]  (the v tile follows the k tile: second 64-column atom)
      constexpr uint32_t idesc = instr_desc(kFmt, 0, 1, 2 * kHead, kTile);
#pragma unroll
      for (int kk = 0; kk < kTile / 16; ++kk)
        mma_f16(tmem_o, smem_desc(sP + (kk >> 2) * kTileBytes + (kk & 3) * 32, 16),
                smem_desc(sB + kk * 2048, kTileBytes), idesc, kk > 0);
    } else if (KIND == kStageLeft) {
      // O[m, 0:64] = P^T[m, :] @ q',  O[m, 64:80] = P^T[m, :] @ s
      constexpr uint32_t idesc_q = instr_desc(kFmt, 1, 1, kHead, kTile);
      constexpr uint32_t idesc_s = instr_desc(kFmt, 1, 0, 16, kTile);
#pragma unroll
      for (int kk = 0; kk < kTile / 16; ++kk) {
        const uint64_t a = smem_desc(sP + kk * 2048, kTileBytes);
        mma_f16(tmem_o, a, smem_desc(sV + kk * 2048, kTileBytes), idesc_q, kk > 0);
        mma_f16(tmem_o + kHead, a, smem_desc(sS + (kk >> 2) * 2048 + (kk & 3) * 32, 16), idesc_s, kk > 0);
      }
    } else {
      // O[l, 0:64] = P[l, :] @ y[j]
      constexpr uint32_t idesc = instr_desc(kFmt, 0, 1, kHead, kTile);
#pragma unroll
      for (int kk = 0; kk < kTile / 16; ++kk)
        mma_f16(tmem_o, smem_desc(sP + (kk >> 2) * kTileBytes + (kk & 3) * 32, 16),
                smem_desc(sV + kk * 2048, kTileBytes), idesc, kk > 0);
    }
    mma_commit(bar_mma2);
  }
  if (!failed) {
    ok = mbar_wait(bar_mma2, 0);
    failed = __syncthreads_or(ok ? 0 : 3);
  }

  // ---- epilogue ------------------------------------------------------------------------
  if (!failed) {
    tc_fence_after();
    const uint32_t tmem_o = tmem_row + 128;
    float scale0, scale1 = 0.f;
    if (kRight) {
      const float denom = row_sum + kEps;
      scale0 = g.sm_scale / denom;
      scale1 = 1.0f / denom;
      const float cl = (kLn2 * row_ent) / denom - logf(denom) * (row_sum / denom);
      g.cl[((long long)eh * g.B + tid) * g.M + tile] = cl;
    } else if (KIND == kStageLeft) {
      scale0 = 1.0f;
    } else {
      scale0 = 1.0f / row_sum;
    }
    // first 64 output columns -> staging tile in the A buffer (free: GEMM 1 has completed)
#pragma unroll 1
    for (int c = 0; c < 2; ++c) {
      float o[32];
      tmem_ld32(tmem_o + c * 32, o);
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const float* p = o + q4 * 8;
        st_shared_v4(sA + swz(tid, c * 4 + q4), pack2<T>(p[0] * scale0, p[1] * scale0),
                     pack2<T>(p[2] * scale0, p[3] * scale0), pack2<T>(p[4] * scale0, p[5] * scale0),
                     pack2<T>(p[6] * scale0, p[7] * scale0));
      }
    }
    if (KIND == kStageRightWithV) {  // y -> staging tile in the P buffer (free: GEMM 2 has completed)
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        float o[32];
        tmem_ld32(tmem_o + kHead + c * 32, o);
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const float* p = o + q4 * 8;
          st_shared_v4(sP + swz(tid, c * 4 + q4), pack2<T>(p[0] * scale1, p[1] * scale1),
                       pack2<T>(p[2] * scale1, p[3] * scale1), pack2<T>(p[4] * scale1, p[5] * scale1),
                       pack2<T>(p[6] * scale1, p[7] * scale1));
        }
      }
    }
    if (KIND == kStageLeft) {  // cr[m, j] = O[m, 64]
      float o[32];
      tmem_ld32(tmem_o + kHead, o);
      g.cr[((long long)eh * g.M + tid) * g.B + tile] = o[0];
    }
    fence_async_smem();
    tc_fence_before();
  }
  __syncthreads();
  if (!failed && tid == 0) {
    if (kRight) {
      tma_store_5d(&maps.al_col, sA, 0, tile, 0, eh, 0);
      if (KIND == kStageRightWithV) tma_store_5d(&maps.y_col, sP, 0, tile, 0, eh, 0);
    } else if (KIND == kStageLeft) {
      tma_store_5d(&maps.ar_col, sA, 0, tile, 0, eh, 0);
    } else {
      tma_store_5d(&maps.out_col, sA, 0, tile, 0, h, e);
    }
    tma_store_commit_and_wait();
  }
  if (failed && tid == 0) {
    atomicExch(g.status, 100 + failed);
    // if the tile loads were what timed out, give the copies one more bounded chance to land
    // before this CTA's shared memory is released
    if (failed == 1) (void)mbar_wait(bar_load, 0);
  }

  // ---- teardown --------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

template <int KIND, typename T>
cudaError_t launch_kind(const TcPlan* plan, const Geometry& g, bool first, cudaStream_t stream) {
  auto fn = tc_stage_kernel<KIND, T>;
  cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
  if (e != cudaSuccess) return e;
  fn<<<dim3(kTile, g.E * g.H), kTcThreads, kSmemBytes, stream>>>(plan->maps, g, first ? 1 : 0);
  return cudaGetLastError();
}

template <typename T>
cudaError_t launch_dtype(const TcPlan* plan, const Geometry& g, StageKind kind, bool first, cudaStream_t stream) {
  switch (kind) {
    case kStageRight: return launch_kind<kStageRight, T>(plan, g, first, stream);
    case kStageRightWithV: return launch_kind<kStageRightWithV, T>(plan, g, first, stream);
    case kStageLeft: return launch_kind<kStageLeft, T>(plan, g, first, stream);
    case kStageOutput: return launch_kind<kStageOutput, T>(plan, g, first, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace

cudaError_t launch_tc_stage(const TcPlan* plan, const Geometry& g, StageKind kind, bool first, cudaStream_t stream) {
  if (plan->qk_dtype == MA_B200_BF16) return launch_dtype<__nv_bfloat16>(plan, g, kind, first, stream);
  return launch_dtype<__half>(plan, g, kind, first, stream);
}

}  // namespace ma
