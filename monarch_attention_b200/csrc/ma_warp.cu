// Warp-level tensor-core stage kernels for 16-bit inputs with block size and block count up to 128:
// the ViT / RoBERTa / DiT shapes (b = 14..32, N <= 1024, D = 64 or 72) and the b = 64 op sweep.
//
// By bytes these shapes are HBM-bound (intensity ~1.25*b FLOP/B) and their blocks are far smaller than
// a tcgen05 tile, so the job here is to move each operand once, with every row masked / zero-padded in
// flight, and to keep the small contractions on tensor cores: mma.sync m16n8k16 with fp32
// accumulation, fragments read from padded shared-memory tiles with ldmatrix.  Measured, the tiles
// are so small that instruction issue (address arithmetic, softmax, staging) is what bounds them.  One CTA works on one
// tile - (head, key block m) for the right-factor stages, (head, column j) for the left-factor and
// output stages - with one warp per 16 rows.  The row softmax runs on the accumulator fragments
// (a row lives in one quad of lanes), and the normalised factor goes back into the second
// contraction straight from registers (right-factor / output) or through a shared-memory tile that
// is read transposed (left-factor, which contracts over the rows).
//
// Semantics follow the reference stage for stage (reference: ma/ma_torch.py:10-62): invalid keys at
// -inf, row maximum clamped from below at eps, eps in the denominator, floor at FLT_MIN, fully
// masked key blocks give ~0 factors and logit 0, invalid queries zeroed in the left-factor stage
// only, padding rows dropped on output.
#include <math.h>

#include "ma_common.cuh"

namespace ma {
namespace {

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2(uint32_t addr, uint32_t (&r)[2]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2_trans(uint32_t addr, uint32_t (&r)[2]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]);
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
template <>
__device__ __forceinline__ void mma16816<__half>(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <typename T>
__device__ __forceinline__ uint32_t pack_pair(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack_pair<__half>(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

// Copies `rows` rows of `width` 16-bit elements (width a multiple of 8) into a shared tile with row
// pitch `pitch` elements, zero-filling rows that do not exist, columns [width, 8*CHUNKS) and rows
// [rows, rpad).  Threads tid of nthreads cooperate.  The copies are asynchronous (cp.async, 16 bytes
// each, zero-fill by giving a source size of 0): a thread queues all of its pieces without waiting;
// tiles_commit_and_wait() must be called before the tile is read.
// Every source these kernels have is an arithmetic progression of rows: row r comes from element
// offset (n0 + r*nstep)*row_stride of `base` and exists iff r < rows and 0 <= n0 + r*nstep < n_limit
// (token index inside the sequence; for the dense state tensors n0 = 0, nstep = 1, n_limit = rows).
// Row, column chunk, token index and source offset are carried from one 16-byte piece to the next
// with additions only.
template <typename T, int CHUNKS>
__device__ __forceinline__ void load_rows(T* tile, int pitch, int rows, int rpad, int width, const T* base, int n0,
                                          int nstep, int n_limit, long long row_stride, int tid, int nthreads,
                                          const void* any_valid_global) {
  int r = tid / CHUNKS, c = tid - r * CHUNKS;
  const int dr = nthreads / CHUNKS, dc = nthreads - dr * CHUNKS;
  int n = n0 + r * nstep;
  const T* src = base + (long long)n * row_stride;
  uint32_t dst = smem_addr(tile + r * pitch);
  const int dn = dr * nstep;
  const long long dsrc = (long long)dn * row_stride, step1 = (long long)nstep * row_stride;
  const uint32_t ddst = (uint32_t)(dr * pitch) * (uint32_t)sizeof(T), dst1 = (uint32_t)pitch * (uint32_t)sizeof(T);
  while (r < rpad) {
    const bool ok = r < rows && (c << 3) < width && (unsigned)n < (unsigned)n_limit;
    const void* gsrc = ok ? static_cast<const void*>(src + (c << 3)) : any_valid_global;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst + (uint32_t)(c << 4)), "l"(gsrc),
                 "r"(ok ? 16u : 0u)
                 : "memory");
    c += dc; r += dr; n += dn; src += dsrc; dst += ddst;
    if (c >= CHUNKS) { c -= CHUNKS; ++r; n += nstep; src += step1; dst += dst1; }
  }
}
__device__ __forceinline__ void tiles_commit_and_wait() {
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

__device__ __forceinline__ bool pos_valid(const Geometry& g, int e, int p) {
  const int n = p - g.pad_off;
  if (n < 0 || n >= g.N) return false;
  return g.mask == nullptr || g.mask[(long long)e * g.mask_se + n] != 0;
}
// Row of a user tensor for padded position p, given the (e, h) base pointer: nullptr for padding.
template <typename T>
__device__ __forceinline__ const T* head_base(const View4& t, int e, int h) {
  return reinterpret_cast<const T*>(t.ptr) + (long long)e * t.se + (long long)h * t.sh;
}
template <typename T>
__device__ __forceinline__ const T* user_row(const T* base, long long sn, int p, const Geometry& g) {
  const int n = p - g.pad_off;
  if (n < 0 || n >= g.N) return nullptr;
  return base + (long long)n * sn;
}

}  // namespace
}  // namespace ma

// Explicit launcher templates are declared before use in ma_warp_kernels.inc and defined in
// ma_warp_wide.inc, so the public entry points have to come last.
#include "ma_warp_kernels.inc"
#include "ma_warp_wide.inc"
