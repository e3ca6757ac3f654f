// Host side of the tensor-core (tcgen05) path: which problems it takes, and the TMA tensor maps of
// one forward call (5-D maps over the caller's strided q, k, v, out views and over the stage-to-stage
// state in the workspace).  Encoding eleven maps costs more host time than a short kernel runs, so
// finished plans are kept in a small mutex-guarded cache keyed by every pointer, stride and size
// that enters a map.
//
// Shapes served: 16-bit storage (bf16 / fp16), D = Dv = 64, block size = block count = 128 or 64
// (two blocks per 128-row tile), N = block size * block count, no mask and no padding.
#include <cuda.h>
#include <string.h>

#include <mutex>

#include "ma_common.cuh"
#include "ma_tc_plan.cuh"

namespace ma {

// ---------------------------------------------------------------------------------
// Host side: tensor maps
// ---------------------------------------------------------------------------------
namespace {

constexpr int kTile = 128;    // rows per tile = keys per tile
constexpr int kHead = 64;     // head width (elements)

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
  if (g.T > 2047) return no("more than 2047 iterations (the stage index of an item descriptor has twelve bits)");
  if (g.q.ptr != nullptr) {  // layout queries pass no pointers
    if (!view_ok(g.q, g.E, g.H) || !view_ok(g.k, g.E, g.H) || !view_ok(g.v, g.E, g.H) || !view_ok(g.out, g.E, g.H))
      return no("q, k, v, out need 16-byte aligned bases and strides that are non-zero multiples of 8 elements");
  }
  if (encode_fn() == nullptr) return no("driver entry point cuTensorMapEncodeTiled not available");
  return true;
}

namespace {

struct PlanKey {
  const void *q, *k, *v, *out, *ar, *al, *y;
  long long qs[3], ks[3], vs[3], os[3];
  int E, H, N, B, T, dtype, device;
  bool operator==(const PlanKey& o) const { return memcmp(this, &o, sizeof(PlanKey)) == 0; }
};
struct CacheEntry {
  PlanKey key;
  TcPlan plan;
  unsigned long long stamp;
  bool used;
};
constexpr int kPlanCache = 16;
CacheEntry g_cache[kPlanCache];
unsigned long long g_stamp = 0;
std::mutex g_cache_mutex;

PlanKey make_key(const Geometry& g, int qk_dtype) {
  PlanKey k;
  memset(&k, 0, sizeof(k));  // padding bytes take part in the comparison
  k.q = g.q.ptr; k.k = g.k.ptr; k.v = g.v.ptr; k.out = g.out.ptr;
  k.ar = g.ar; k.al = g.al; k.y = g.y;
  const View4* vs[4] = {&g.q, &g.k, &g.v, &g.out};
  long long* ss[4] = {k.qs, k.ks, k.vs, k.os};
  for (int i = 0; i < 4; ++i) { ss[i][0] = vs[i]->se; ss[i][1] = vs[i]->sh; ss[i][2] = vs[i]->sn; }
  k.E = g.E; k.H = g.H; k.N = g.N; k.B = g.B; k.T = g.T; k.dtype = qk_dtype;
  cudaGetDevice(&k.device);
  return k;
}

}  // namespace

// Copies the plan of this call into *out: from the cache when the same pointers, strides and sizes
// were seen before, otherwise freshly encoded (and remembered, replacing the least recently used entry).
int tc_plan_get(const Geometry& g, int qk_dtype, TcPlan* out, const char** err) {
  const PlanKey key = make_key(g, qk_dtype);
  {
    std::lock_guard<std::mutex> lock(g_cache_mutex);
    for (int i = 0; i < kPlanCache; ++i)
      if (g_cache[i].used && g_cache[i].key == key) {
        g_cache[i].stamp = ++g_stamp;
        *out = g_cache[i].plan;
        return MA_B200_OK;
      }
  }
  TcPlan* plan = nullptr;
  const int rc = tc_plan_create(g, qk_dtype, &plan, err);
  if (rc != MA_B200_OK) return rc;
  *out = *plan;
  delete plan;
  std::lock_guard<std::mutex> lock(g_cache_mutex);
  int victim = 0;
  for (int i = 0; i < kPlanCache; ++i) {
    if (!g_cache[i].used) { victim = i; break; }
    if (g_cache[i].stamp < g_cache[victim].stamp) victim = i;
  }
  g_cache[victim].key = key;
  g_cache[victim].plan = *out;
  g_cache[victim].stamp = ++g_stamp;
  g_cache[victim].used = true;
  return MA_B200_OK;
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

}  // namespace ma
