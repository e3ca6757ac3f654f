// Persistent, warp-specialised tcgen05 kernel that runs every stage of the forward pass
// in ONE launch.
//
// Work items are 128-row tiles: (stage, head, tile index).  Stage s of the 2T stages is
//   right-factor (s even, s < 2T-2), left-factor (s odd, s < 2T-2),
//   right-factor with V (s = 2T-2), output (s = 2T-1)          (reference: ma/ma_torch.py:100-105).
// Items are laid out head-group-major: for each group of up to G heads, for each stage, for each
// head of the group, for each tile.  CTA c of the persistent grid takes items c, c+grid, ... in
// that order.  A stage-s item of a head may start once all items of stage s-1 of that head are
// done; completion is counted in global memory (one counter per head and stage).  Because the
// heads of a group are interleaved, the items a stage depends on were issued (G-1)*tiles items
// earlier, so the bounded wait in the producer rarely spins.  The stage-to-stage state (ar, cr, al,
// cl, y) of a head lives in one of G state slots; the next group reuses the slots (its first stage
// waits for the last stage of the head that had the slot), so only G heads of state are ever live,
// they stay in L2, and lines are overwritten there instead of being written back to HBM.
// The launch is cooperative so that every CTA of the grid is resident, which the in-order
// item schedule needs for forward progress.
//
// Numerics follow the reference's rounding points (ma/ma_torch.py:10-62): the fp32 accumulator of
// the first contraction is rounded to the storage type before the softmax arithmetic, the factor is
// normalised in fp32 and then rounded to the storage type before the second contraction, and the
// column sums cr of the left factor are taken from the factor before that rounding.
//
// Inside a CTA (512 threads, one CTA per SM, all 512 tensor-memory columns):
//   warps 0-3, 4-7   two softmax groups on alternating items, one tile row per thread: the whole row
//              of S is read from tensor memory into registers once (tcgen05.ld), maximum, exponentials,
//              row sum and negative entropy are formed there (packed fp32 pairs), the normalised
//              factor P is rounded to 16 bits and written back over S with tcgen05.st, from where the
//              second contraction reads it as its A operand.  Only the left-factor stage, which needs
//              P^T, goes through shared memory: P as a 16-bit value plus a 16-bit remainder, so that
//              the column sums come out of the tensor core in fp32 precision.
//   warps 8-11 epilogue group: waits for O, rounds it and stores rows to global memory with 32-byte
//              stores
//   warp 12    TMA producer: waits for the item's dependency, loads the 2-3 operand tiles and the
//              512-byte row vector (cr or cl) of the item into a ring of thirteen 16 KB tiles
//   warp 13    MMA issuer 1: S = A B^T for item n (tcgen05.mma, fp32 accumulator S[n%3] in tensor memory)
//   warp 14    MMA issuer 2: the second contraction of item n into O
//   warp 15    publisher: device-scope fence and one increment of the item's completion counter
// All hand-offs are mbarriers; every wait is bounded and abortable (see ma_sm100.cuh).
#include <cuda.h>

#include <mutex>
#include <type_traits>

#include "ma_common.cuh"
#include "ma_sm100.cuh"
#include "ma_tc_plan.cuh"

namespace ma {
namespace {

using namespace sm100;

constexpr int kTile = 128;
constexpr int kHead = 64;
constexpr uint32_t kTileBytes = kTile * kHead * 2;  // 16 KB

constexpr int kEpilogueWarp0 = 8;   // warps 8..11
constexpr int kProducerWarp = 12;
constexpr int kMma1Warp = 13;
constexpr int kMma2Warp = 14;
constexpr int kThreads = 16 * 32;

// Operand tiles live in a ring of thirteen 16 KB tiles.  An item takes two consecutive tiles (A, B) or
// three (A, B, V) - never wrapping: if the tail of the ring is too short it is skipped and charged to
// the item.  Tiles 9..12 double as the P region of the left-factor stage (P and its remainder,
// 2 x 32 KB): while a left-factor item is in flight the ring ends at tile 9.
constexpr int kRingTiles = 13;
constexpr int kRingLeft = 9;
constexpr int kSlots = 8;  // items in flight: depth of the per-item barrier / row-vector rings
// Tensor memory: three S accumulators (columns 0, 128, 256); P (16-bit pairs) is written over the
// first 64 columns of its S.  One O accumulator (column 384): the epilogue empties it much faster
// than items arrive.
constexpr int kSBuffers = 3;
constexpr uint32_t kTmemO = 384;
constexpr uint32_t kOffSlots = 0;
constexpr uint32_t kOffPreg = kRingLeft * kTileBytes;             // P region = ring tiles 9..12
constexpr uint32_t kOffOnes = kRingTiles * kTileBytes;            // 16 x 128 K-major operand of ones (4 KB)
constexpr uint32_t kOffVec = kOffOnes + 4096;                     // kSlots x 512 B (cr or cl of the item)
constexpr uint32_t kOffStats = kOffVec + kSlots * 512;            // 4 x 128 floats (cl of the item's rows)
constexpr uint32_t kOffBar = kOffStats + 4 * 128 * 4;
constexpr int kNumBarsConst = 48;
constexpr int kDescRing = 16;  // item descriptors; deeper than the producer can run ahead (kSlots)
constexpr uint32_t kOffDesc = kOffBar + 8 * kNumBarsConst + 16;
constexpr uint32_t kSmemUsed = kOffDesc + 16 * kDescRing;
constexpr uint32_t kSmemBytes = kSmemUsed + 1024;
static_assert(kOffPreg % 1024 == 0 && kOffOnes % 1024 == 0, "swizzled operands need 1024-byte alignment");
static_assert(kSmemBytes <= 232448, "shared memory per CTA");

// mbarrier indices (8 bytes each)
enum {
  kBarInFull = 0,     // [8] operand tiles of an item filled by TMA
  kBarInEmpty = 8,    // [8] operand tiles of an item released by the second contraction
  kBarSFull = 16,     // [3] S accumulator ready
  kBarSEmpty = 19,    // [3] S / P released by the second contraction
  kBarPFull = 22,     // [3] P written (tensor memory, or shared memory in the left-factor stage)
  kBarOFull = 25,     // [1] O accumulator ready
  kBarOEmpty = 26,    // [1] O accumulator read by the epilogue group
  kBarDone = 28,      // [4] item stored to global memory by all 128 epilogue threads
  kBarPubFree = 32,   // [4] completion of that item published
  kBarStat = 36,      // [4] row statistics of the item written by its softmax group
  kNumBars = 40
};
static_assert(kNumBars <= kNumBarsConst, "barrier count");

struct FusedArgs {
  int stage_begin, stage_end;  // stages [begin, end) of the 2T stages run in this launch
  int group;                   // heads interleaved per group
  int wait_deps;               // wait on the completion counters of the previous stage
  int reuse_slots;             // state of head (group g, position p) lives in slot p (needs wait_deps)
  int spin_limit;              // iterations of the producer's dependency wait before it gives up
  int* counters;               // (E*H, 2T) ints, zeroed before the first launch of a call
  int* host_status;            // mapped host word that receives the code of a wait that gave up, or nullptr
};

struct Item {
  int kind, first, stage, eh, tile, hs;  // hs: state slot of the head
};

// Walks the items of one CTA (global indices blockIdx.x, blockIdx.x + grid, ...) without a division
// per item: the position (group, stage, head in group, tile) is carried along.
struct ItemCursor {
  int gi, sl, hh, tile, gh;  // group, stage within the launch, head within the group, tile, heads in this group
  int idx, total, stride, nst, group, EH, stage_begin, last_stage, reuse;
  int tph;  // tiles per head and stage: N / 128

  __device__ __forceinline__ void init(int first_idx, int stride_, const Geometry& g, const FusedArgs& a) {
    EH = g.E * g.H;
    nst = a.stage_end - a.stage_begin;
    group = a.group;
    reuse = a.reuse_slots;
    stage_begin = a.stage_begin;
    last_stage = 2 * g.T - 1;
    tph = g.N / kTile;
    total = nst * tph * EH;
    stride = stride_;
    idx = first_idx;
    const int per_group = nst * group * tph;
    gi = idx / per_group;
    int r = idx - gi * per_group;
    gh = min(group, EH - gi * group);
    if (gh < 1) gh = 1;
    sl = r / (gh * tph);
    r -= sl * gh * tph;
    hh = r / tph;
    tile = r - hh * tph;
  }
  __device__ __forceinline__ bool valid() const { return idx < total; }
  __device__ __forceinline__ void next() {
    idx += stride;
    tile += stride;
    while (tile >= tph) {
      tile -= tph;
      if (++hh == gh) {
        hh = 0;
        if (++sl == nst) {
          sl = 0;
          ++gi;
          gh = min(group, EH - gi * group);
          if (gh < 1) gh = 1;
        }
      }
    }
  }
  __device__ __forceinline__ Item get() const {
    Item it;
    it.tile = tile;
    it.eh = gi * group + hh;
    it.hs = reuse ? hh : it.eh;
    it.stage = stage_begin + sl;
    it.kind = it.stage == last_stage
                  ? kStageOutput
                  : (it.stage == last_stage - 1 ? kStageRightWithV : ((it.stage & 1) ? kStageLeft : kStageRight));
    it.first = it.stage == 0;
    return it;
  }
};

// Round an fp32 pair through the 16-bit storage type (the reference rounds every contraction result to
// the storage type before the fp32 softmax arithmetic, ma/ma_torch.py:11, :27, :56).
template <typename T>
__device__ __forceinline__ float2 round2(float2 x) {
  return unpack2<T>(pack2<T>(x.x, x.y));
}

template <typename T, int PER>  // PER: key blocks (or columns j) per 128-row tile: 1 (block size 128) or 2 (64)
__global__ void __launch_bounds__(kThreads, 1) fused_kernel(const __grid_constant__ TcMaps maps, const Geometry g,
                                                            const FusedArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + kOffBar;
  auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + kOffBar + 8 * kNumBarsConst);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + kOffBar + 8 * kNumBarsConst + 8);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr int kFmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
  const int tph = g.N / kTile;  // tiles per head and stage
  constexpr int per = PER;
  constexpr int kRowsPer = kTile / PER;  // rows of one block (or column) inside a tile = block size = block count
  constexpr int kCols = kTile / PER;     // columns of S that belong to a row
  const int total = (args.stage_end - args.stage_begin) * tph * g.E * g.H;
  const int nst_all = 2 * g.T;

  if (tid == 0) {
    for (int i = 0; i < kSlots; ++i) { mbar_init(bar(kBarInFull + i), 1); mbar_init(bar(kBarInEmpty + i), 1); }
    for (int i = 0; i < kSBuffers; ++i) {
      mbar_init(bar(kBarSFull + i), 1);
      mbar_init(bar(kBarSEmpty + i), 1);
      mbar_init(bar(kBarPFull + i), 128);
    }
    mbar_init(bar(kBarOFull), 1);
    mbar_init(bar(kBarOEmpty), 128);
    for (int i = 0; i < 4; ++i) {
      mbar_init(bar(kBarDone + i), 128);
      mbar_init(bar(kBarStat + i), 128);
      mbar_init(bar(kBarPubFree + i), 1);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kMma1Warp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     base + kOffBar + 8 * kNumBarsConst),
                 "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  {  // the 16 x 128 operand of ones that turns the second contraction of the left-factor stage into column sums
    uint32_t* z = reinterpret_cast<uint32_t*>(base_ptr + kOffOnes);
    const uint32_t one2 = pack2<T>(1.0f, 1.0f);
    for (int i = tid; i < 1024; i += kThreads) z[i] = one2;
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  // Only the producer walks the item schedule.  It leaves a four-word descriptor per item in a small
  // ring (written before the arrive that opens the item's operand barrier, so every later hand-off
  // carries it); the other roles read it once their first wait for the item has returned.
  const int n_items = total > (int)blockIdx.x ? (total - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  auto read_item = [&](int n, int* first_tile, int* p_dist) {
    const int4 d = *reinterpret_cast<const int4*>(base_ptr + kOffDesc + (n & (kDescRing - 1)) * 16);
    Item it;
    it.kind = d.x & 3;
    it.first = (d.x >> 2) & 1;
    *first_tile = (d.x >> 3) & 15;
    it.tile = (d.x >> 8) & 255;
    it.stage = d.x >> 16;
    it.eh = d.y;
    it.hs = d.z;
    *p_dist = d.w;
    return it;
  };
  auto give_up = [&](int code) {
    *abort_flag = 1;
    if (atomicCAS(g.status, 0, code) == 0 && args.host_status != nullptr) {
      *reinterpret_cast<volatile int*>(args.host_status) = code;
      __threadfence_system();
    }
  };

  // Registers per warpgroup (the launch gives every thread 128): the two softmax groups hold a
  // whole accumulator row each, the epilogue group half a row, the single-thread roles little.
  // 256 x 192 + 128 x 80 + 128 x 48 = 65536 = 512 x 128, so the increase can always be granted.
  // (What setmaxnreg redistributes is the allocation the CTA was launched with - threads x registers
  // per thread - not the whole register file: a request beyond that pool blocks for ever.)
  if (warp >= kProducerWarp) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 48;");
  if (warp == kProducerWarp) {
    // =========================== TMA producer ===========================================
    if (lane == 0) {
      int n = 0, issued = 0;
      int free_tiles = kRingTiles, oldest = 0, ring_pos = 0;  // ring accounting: items [oldest, n) hold tiles
      int lefts = 0;                                          // left-factor items among them
      // per in-flight item, at index m % kSlots, packed: tiles held (incl. skipped tail) | left-factor item << 8 |
      // holds a tile of the P region << 9
      int held[kSlots];
#pragma unroll
      for (int i = 0; i < kSlots; ++i) held[i] = 0;
      auto held_at = [&](int m) {
        int v = 0;
#pragma unroll
        for (int i = 0; i < kSlots; ++i) v = (m % kSlots) == i ? held[i] : v;
        return v;
      };
      auto retire_oldest = [&]() {
        const int v = held_at(oldest);
        free_tiles += v & 255;
        lefts -= (v >> 8) & 1;
        ++oldest;
      };
      ItemCursor cur;
      bool ok = true;
      for (cur.init(blockIdx.x, gridDim.x, g, args); cur.valid() && ok; cur.next(), ++n) {
        const Item it = cur.get();
        const int e = it.eh / g.H, h = it.eh - e * g.H;
        const int slot = n % kSlots;
        if (args.wait_deps) {
          const int* ctr = nullptr;
          if (it.stage > 0) ctr = args.counters + it.eh * nst_all + (it.stage - 1);
          else if (args.reuse_slots && cur.gi > 0) ctr = args.counters + (it.eh - args.group) * nst_all + (nst_all - 1);
          if (ctr != nullptr) {
            bool ready = false;
            for (int spin = 0; spin < args.spin_limit; ++spin) {
              if (ld_acquire_gpu(ctr) >= tph) { ready = true; break; }
              if ((spin & 255) == 255 && *abort_flag) break;
              __nanosleep(32);
            }
            if (!ready) { give_up(201); break; }
            fence_proxy_async_all();  // the state was written with ordinary stores; the loads below are TMA
          }
        }
        // items whose second contraction has completed give their tiles back (in order)
        while (oldest < n && mbar_test(bar(kBarInEmpty + oldest % kSlots), (uint32_t)(oldest / kSlots) & 1u))
          retire_oldest();
        const bool left = it.kind == kStageLeft;
        const int ntiles = (it.kind == kStageRightWithV || it.kind == kStageOutput) ? 3 : 2;
        int t0 = 0, charged = 0;
        for (;;) {
          const int limit = (left || lefts > 0) ? kRingLeft : kRingTiles;
          int pos = ring_pos, sk = 0;
          if (pos + ntiles > limit) { sk = kRingTiles - pos; pos = 0; }
          if (free_tiles >= ntiles + sk && n - oldest < kSlots) { t0 = pos; charged = ntiles + sk; break; }
          if (!mbar_wait_abortable(bar(kBarInEmpty + oldest % kSlots), (uint32_t)(oldest / kSlots) & 1u, abort_flag)) {
            give_up(202);
            ok = false;
            break;
          }
          retire_oldest();
        }
        if (!ok) break;
        // A left-factor item writes P into the P region: it has to wait for the newest older item that
        // is a left-factor item itself or holds one of those tiles (items complete in order).
        int p_dist = 0;
        if (left) {
          for (int m = oldest; m < n; ++m)
            if (held_at(m) >> 8) p_dist = n - m;
        }
        ring_pos = t0 + ntiles;
        const int uses_p = (ring_pos > kRingLeft || charged > ntiles) ? 1 : 0;
        if (ring_pos == kRingTiles) ring_pos = 0;
        {
          const int v = charged | ((left ? 1 : 0) << 8) | (uses_p << 9);
#pragma unroll
          for (int i = 0; i < kSlots; ++i)
            if (slot == i) held[i] = v;
        }
        free_tiles -= charged;
        lefts += left ? 1 : 0;
        const uint32_t sA = base + kOffSlots + t0 * kTileBytes, sB = sA + kTileBytes, sV = sB + kTileBytes;
        const uint32_t vec = base + kOffVec + slot * 512;
        const uint32_t full = bar(kBarInFull + slot);
        const bool right = it.kind == kStageRight || it.kind == kStageRightWithV;
        const bool three = ntiles == 3;
        const bool has_vec = !(right && it.first);
        *reinterpret_cast<int4*>(base_ptr + kOffDesc + (n & (kDescRing - 1)) * 16) =
            make_int4(it.kind | (it.first << 2) | (t0 << 3) | (it.tile << 8) | (it.stage << 16), it.eh, it.hs, p_dist);
        mbar_expect_tx(full, (three ? 3u : 2u) * kTileBytes + (has_vec ? 512u : 0u));
        if (right) {
          if (it.first) tma_load_5d(sA, &maps.q_blk, full, 0, 0, it.tile, h, e);
          else tma_load_5d(sA, &maps.ar_blk, full, 0, 0, it.tile, it.hs, 0);
          tma_load_5d(sB, &maps.k_blk, full, 0, 0, it.tile, h, e);
          if (three) tma_load_5d(sV, &maps.v_blk, full, 0, 0, it.tile, h, e);
          if (has_vec) bulk_load(vec, g.cr + ((long long)it.hs * g.M + it.tile * per) * g.B, 512, full);
        } else {
          // one box per column j of the tile: rows jj*(128/per) + l, the same row order as the blocks of
          // a right-factor tile (a row's own columns are then the same for every lane of a warp, which
          // the warp-wide tensor-memory loads of the softmax need)
          for (int jj = 0; jj < per; ++jj)
            tma_load_5d(sA + jj * (kTileBytes / per), &maps.q_col, full, 0, it.tile * per + jj, 0, h, e);
          tma_load_5d(sB, &maps.al_blk, full, 0, 0, it.tile, it.hs, 0);
          if (three) tma_load_5d(sV, &maps.y_blk, full, 0, 0, it.tile, it.hs, 0);
          bulk_load(vec, g.cl + ((long long)it.hs * g.B + it.tile * per) * g.M, 512, full);
        }
        issued = n + 1;
      }
      // Drain: make sure every copy this thread started has landed before the CTA may exit.
      for (int m = max(0, issued - kSlots); m < issued; ++m)
        (void)mbar_wait(bar(kBarInFull + m % kSlots), (uint32_t)(m / kSlots) & 1u);
    }
  } else if (warp == kMma1Warp) {
    // =========================== MMA issuer 1: S = A B^T ====================================
    // Two single-thread issuers with blocking waits (a polling issuer would take issue slots from the
    // softmax warps that share its scheduler).  They are independent on purpose: the operands of item
    // n+1 may depend on the completion of item n of this same CTA, so the second contraction of item n
    // must never queue behind a wait for item n+1.
    if (lane == 0) {
      const uint32_t dA0 = smem_desc_lo(base + kOffSlots, 16);  // ring tile 0 as a K-major operand; B follows A
      constexpr uint32_t kTileStep = kTileBytes >> 4;
      constexpr uint32_t idesc1 = instr_desc(kFmt, 0, 0, kTile, kTile);
      for (int n = 0; n < n_items; ++n) {
        const int slot = n % kSlots, sb = n % kSBuffers;
        if (!mbar_wait_abortable(bar(kBarInFull + slot), (uint32_t)(n / kSlots) & 1u, abort_flag)) { give_up(301); break; }
        int t0, pd;
        (void)read_item(n, &t0, &pd);
        if (!mbar_wait_abortable(bar(kBarSEmpty + sb), ((uint32_t)(n / kSBuffers) & 1u) ^ 1u, abort_flag)) { give_up(302); break; }
        tc_fence_after();
        const uint32_t dA = dA0 + t0 * kTileStep, dB = dA + kTileStep;
#pragma unroll
        for (int kk = 0; kk < kHead / 16; ++kk) mma_f16_lo(tmem + sb * 128, dA + kk * 2, dB + kk * 2, idesc1, kk > 0);
        mma_commit(bar(kBarSFull + sb));
      }
    }
  } else if (warp == kMma2Warp) {
    // =========================== MMA issuer 2: O = P [B | V] =================================
    if (lane == 0) {
      const uint32_t dP_mn0 = smem_desc_lo(base + kOffPreg, kTileBytes);   // P^T as MN-major A operand (left stage)
      const uint32_t dOnes = smem_desc_lo(base + kOffOnes, 16);            // 16 x 128 K-major operand of ones
      const uint32_t dTmn0 = smem_desc_lo(base + kOffSlots, kTileBytes);   // ring tile 0 as an MN-major operand
      constexpr uint32_t kTileStep = kTileBytes >> 4;
      for (int n = 0; n < n_items; ++n) {
        const int sb = n % kSBuffers, slot = n % kSlots;
        if (!mbar_wait_abortable(bar(kBarPFull + sb), (uint32_t)(n / kSBuffers) & 1u, abort_flag)) { give_up(303); break; }
        int t0, pd;
        const int kind = read_item(n, &t0, &pd).kind;
        if (!mbar_wait_abortable(bar(kBarOEmpty), ((uint32_t)n & 1u) ^ 1u, abort_flag)) { give_up(304); break; }
        tc_fence_after();
        // tiles of the item: A, B, V
        const uint32_t dA = dTmn0 + t0 * kTileStep, dB = dA + kTileStep, dV = dB + kTileStep;
        const uint32_t tmem_o = tmem + kTmemO, tmem_p = tmem + sb * 128;
        if (kind == kStageRight) {
          constexpr uint32_t idesc = instr_desc(kFmt, 0, 1, kHead, kTile);
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk) mma_f16_ts(tmem_o, tmem_p + kk * 8, dB + kk * 128, idesc, kk > 0);
        } else if (kind == kStageRightWithV) {
          // the V tile follows the B tile in the ring: second 64-column atom of a 128-wide operand
          constexpr uint32_t idesc = instr_desc(kFmt, 0, 1, 2 * kHead, kTile);
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk) mma_f16_ts(tmem_o, tmem_p + kk * 8, dB + kk * 128, idesc, kk > 0);
        } else if (kind == kStageLeft) {
          // O[m, :64] = sum_l P[l, m] q[l, :]; O[m, 64] = sum_l (P + remainder)[l, m]
          constexpr uint32_t idesc_q = instr_desc(kFmt, 1, 1, kHead, kTile);
          constexpr uint32_t idesc_s = instr_desc(kFmt, 1, 0, 16, kTile);
          const uint32_t dPlo = dP_mn0 + 2 * kTileStep;
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk) {
            const uint32_t ones = dOnes + ((kk >> 2) * 128 + (kk & 3) * 2);
            mma_f16_lo(tmem_o, dP_mn0 + kk * 128, dA + kk * 128, idesc_q, kk > 0);
            mma_f16_lo(tmem_o + kHead, dP_mn0 + kk * 128, ones, idesc_s, kk > 0);
            mma_f16_lo(tmem_o + kHead, dPlo + kk * 128, ones, idesc_s, 1);
          }
        } else {
          constexpr uint32_t idesc = instr_desc(kFmt, 0, 1, kHead, kTile);
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk) mma_f16_ts(tmem_o, tmem_p + kk * 8, dV + kk * 128, idesc, kk > 0);
        }
        mma_commit(bar(kBarOFull));
        mma_commit(bar(kBarSEmpty + sb));
        mma_commit(bar(kBarInEmpty + slot));
      }
    }
  } else {
    // =========================== publisher =====================================================
    // Makes the stores of every finished item visible device-wide and counts the item in its
    // (head, stage) completion counter, off the critical path of the epilogue group.
    if (lane == 0 && args.wait_deps) {
      for (int n = 0; n < n_items; ++n) {
        if (!mbar_wait_abortable(bar(kBarDone + (n & 3)), (uint32_t)(n >> 2) & 1u, abort_flag)) { give_up(601); break; }
        int t0, pd;
        const Item it = read_item(n, &t0, &pd);
        // the output stage is consumed only when state slots are reused (by the next head in the slot)
        if (it.stage != nst_all - 1 || args.reuse_slots) {
          __threadfence();
          atomicAdd(args.counters + it.eh * nst_all + it.stage, 1);
        }
        mbar_arrive(bar(kBarPubFree + (n & 3)));
      }
    }
  }
  } else if (warp >= kEpilogueWarp0) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 80;");
    // =========================== epilogue group =================================================
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    for (int n = 0; n < n_items; ++n) {
      if (!mbar_wait_abortable(bar(kBarStat + (n & 3)), (uint32_t)(n >> 2) & 1u, abort_flag) ||
          !mbar_wait_abortable(bar(kBarOFull), (uint32_t)n & 1u, abort_flag)) {
        give_up(501);
        break;
      }
      tc_fence_after();
      int t0_unused, pd_unused;
      const Item it = read_item(n, &t0_unused, &pd_unused);
      const float stat = reinterpret_cast<const float*>(base_ptr + kOffStats)[(n & 3) * 128 + row];
      const uint32_t tmem_o = tmem + lane_base + kTmemO;
      T* dst0;
      // Row of the tile -> (row within its block or column, which of the tile's `per` blocks / columns).
      // Right-factor tiles hold blocks one after the other (row = blk*B + j); the accumulator of the
      // left-factor stage (row = jj*M + m) and the column tiles of the output stage (row = jj*M + l) are
      // indexed the same way.
      const int rin = row & (kRowsPer - 1), rblk = row / kRowsPer;
      long long row_y = 0;
      float scale = 1.0f;
      if (it.kind == kStageRight || it.kind == kStageRightWithV) {
        const long long rr = ((long long)it.hs * g.B + rin) * g.M + it.tile * per + rblk;
        dst0 = reinterpret_cast<T*>(g.al) + rr * kHead;
        g.cl[rr] = stat;
        row_y = rr;
        scale = g.sm_scale;  // a power of two for D = 64: scaling before or after the rounding is the same
      } else if (it.kind == kStageLeft) {
        dst0 = reinterpret_cast<T*>(g.ar) + (((long long)it.hs * g.M + rin) * g.B + it.tile * per + rblk) * kHead;
      } else {
        const int e = it.eh / g.H, h = it.eh - e * g.H;
        dst0 = reinterpret_cast<T*>(const_cast<void*>(g.out.ptr)) + (long long)e * g.out.se + (long long)h * g.out.sh +
               ((long long)rin * g.B + it.tile * per + rblk) * g.out.sn;
      }
      // 64 accumulator columns -> one 128-byte row: both chunk loads in flight, then 4 x 32-byte stores
      // (every touched sector is written whole)
      auto store_row = [&](T* dst, uint32_t taddr, float sc) {
        float o0[32], o1[32];
        tmem_ld32_nowait(taddr, o0);
        tmem_ld32_nowait(taddr + 32, o1);
        tmem_wait_ld(o0);
        tmem_wait_ld(o1);
#pragma unroll
        for (int h8 = 0; h8 < 4; ++h8) {
          const float* p = (h8 < 2 ? o0 : o1) + (h8 & 1) * 16;
          uint32_t w[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) w[i] = pack2<T>(p[2 * i] * sc, p[2 * i + 1] * sc);
          st_global_v8(dst + h8 * 16, w);
        }
      };
      store_row(dst0, tmem_o, scale);
      if (it.kind == kStageRightWithV) {
        store_row(reinterpret_cast<T*>(g.y) + row_y * kHead, tmem_o + kHead, 1.0f);
      } else if (it.kind == kStageLeft) {
        float o[32];
        tmem_ld32(tmem_o + kHead, o);
        g.cr[((long long)it.hs * g.M + rin) * g.B + it.tile * per + rblk] = o[0];
      }
      tc_fence_before();
      mbar_arrive(bar(kBarOEmpty));
      if (args.wait_deps) {
        // hand the item to the publisher warp (4-deep ring)
        if (!mbar_wait_abortable(bar(kBarPubFree + (n & 3)), ((uint32_t)(n >> 2) & 1u) ^ 1u, abort_flag)) {
          give_up(502);
          break;
        }
        mbar_arrive(bar(kBarDone + (n & 3)));
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 192;");
    // =========================== softmax groups ==========================================
    const int grp = warp >> 2;                      // items with local index n = grp (mod 2)
    const int row = (warp & 3) * 32 + lane;         // tensor-memory lane = tile row
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    // 64-column halves of the row this thread works on: both, or - with two blocks per tile - only the
    // half that belongs to the row's own block or column (rows are blk*64 + j in the right-factor
    // tiles and jj*64 + l in the column tiles; columns are blk*64 + i, or jj*64 + m); the other half of
    // P is zero.
    const int h0 = per > 1 ? (row >> 6) : 0;  // uniform within a warp
    for (int n = grp; n < n_items; n += 2) {
      const int slot = n % kSlots, sb = n % kSBuffers;
      const float* vec = reinterpret_cast<const float*>(base_ptr + kOffVec + slot * 512) + (per > 1 ? 64 * h0 : 0);
      if (!mbar_wait_abortable(bar(kBarInFull + slot), (uint32_t)(n / kSlots) & 1u, abort_flag)) { give_up(401); break; }
      int tile0, p_dist;
      const Item it = read_item(n, &tile0, &p_dist);
      const bool right = it.kind == kStageRight || it.kind == kStageRightWithV;
      if (!mbar_wait_abortable(bar(kBarSFull + sb), (uint32_t)(n / kSBuffers) & 1u, abort_flag)) { give_up(402); break; }
      tc_fence_after();
      const uint32_t tmem_s = tmem + lane_base + sb * 128;

      // The row's own columns of S, read once and kept in registers.
      float s[kCols];
#pragma unroll
      for (int c = 0; c < kCols / 32; ++c)
        tmem_ld32_nowait(tmem_s + 64 * h0 + 32 * c, *reinterpret_cast<float(*)[32]>(&s[32 * c]));
#pragma unroll
      for (int c = 0; c < kCols / 32; ++c) tmem_wait_ld(*reinterpret_cast<float(*)[32]>(&s[32 * c]));

      float stat = 0.f, inv;
      if (right) {
        // x = sm_scale * round(S) / (cr + eps); the maximum of the rounded values is the rounded maximum
        const float row_scale = g.sm_scale / ((it.first ? 1.0f : vec[row & (kRowsPer - 1)]) + kEps);
        float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
        for (int i = 0; i < kCols; i += 8) {
          m0 = max3(m0, s[i], s[i + 1]);
          m1 = max3(m1, s[i + 2], s[i + 3]);
          m2 = max3(m2, s[i + 4], s[i + 5]);
          m3 = max3(m3, s[i + 6], s[i + 7]);
        }
        const float vmax = round_through<T>(fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)));
        const float top = fmaxf(vmax * row_scale, kEps);  // lower clamp on the row maximum
        const float mul = row_scale * kLog2e, noff = -top * kLog2e;
        const float2 mulv = make_float2(mul, mul), noffv = make_float2(noff, noff);
        float2 sum_a = make_float2(0.f, 0.f), sum_b = sum_a, ent_a = sum_a, ent_b = sum_a;
#pragma unroll
        for (int i = 0; i < kCols; i += 4) {
          const float2 ua = fma2(round2<T>(make_float2(s[i], s[i + 1])), mulv, noffv);
          const float2 ub = fma2(round2<T>(make_float2(s[i + 2], s[i + 3])), mulv, noffv);
          const float2 ea = make_float2(ex2(ua.x), ex2(ua.y)), eb = make_float2(ex2(ub.x), ex2(ub.y));
          sum_a = add2(sum_a, ea);
          sum_b = add2(sum_b, eb);
          ent_a = fma2(ea, ua, ent_a);
          ent_b = fma2(eb, ub, ent_b);
          s[i] = ea.x; s[i + 1] = ea.y; s[i + 2] = eb.x; s[i + 3] = eb.y;
        }
        const float row_sum = (sum_a.x + sum_a.y) + (sum_b.x + sum_b.y);
        const float row_ent = (ent_a.x + ent_a.y) + (ent_b.x + ent_b.y);
        const float denom = row_sum + kEps;
        inv = __frcp_rn(denom);
        // sum_i r_i ln r_i with r_i = e_i / denom and ln e_i = ln2 * u_i
        stat = (kLn2 * row_ent - __logf(denom) * row_sum) * inv;
      } else {
        // w = round(S) - cl[m], softmax over m
        float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
        for (int i = 0; i < kCols; i += 8) {
          const float4 c0 = *reinterpret_cast<const float4*>(vec + i);
          const float4 c1 = *reinterpret_cast<const float4*>(vec + i + 4);
          const float2 a = sub2(round2<T>(make_float2(s[i], s[i + 1])), make_float2(c0.x, c0.y));
          const float2 b = sub2(round2<T>(make_float2(s[i + 2], s[i + 3])), make_float2(c0.z, c0.w));
          const float2 c = sub2(round2<T>(make_float2(s[i + 4], s[i + 5])), make_float2(c1.x, c1.y));
          const float2 d = sub2(round2<T>(make_float2(s[i + 6], s[i + 7])), make_float2(c1.z, c1.w));
          m0 = max3(m0, a.x, a.y);
          m1 = max3(m1, b.x, b.y);
          m2 = max3(m2, c.x, c.y);
          m3 = max3(m3, d.x, d.y);
          s[i] = a.x; s[i + 1] = a.y; s[i + 2] = b.x; s[i + 3] = b.y;
          s[i + 4] = c.x; s[i + 5] = c.y; s[i + 6] = d.x; s[i + 7] = d.y;
        }
        const float noff = -fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)) * kLog2e;
        const float2 mulv = make_float2(kLog2e, kLog2e), noffv = make_float2(noff, noff);
        float2 sum_a = make_float2(0.f, 0.f), sum_b = sum_a;
#pragma unroll
        for (int i = 0; i < kCols; i += 4) {
          const float2 ua = fma2(make_float2(s[i], s[i + 1]), mulv, noffv);
          const float2 ub = fma2(make_float2(s[i + 2], s[i + 3]), mulv, noffv);
          const float2 ea = make_float2(ex2(ua.x), ex2(ua.y)), eb = make_float2(ex2(ub.x), ex2(ub.y));
          sum_a = add2(sum_a, ea);
          sum_b = add2(sum_b, eb);
          s[i] = ea.x; s[i + 1] = ea.y; s[i + 2] = eb.x; s[i + 3] = eb.y;
        }
        inv = __frcp_rn((sum_a.x + sum_a.y) + (sum_b.x + sum_b.y));
      }
      // cl of the row for the epilogue group.  The 4-deep ring cannot be overrun: the first contraction
      // of item n+4 needs the S buffer of item n+1, which its second contraction frees, which needs O
      // free, i.e. the epilogue of item n past its read of this entry.
      reinterpret_cast<float*>(base_ptr + kOffStats)[(n & 3) * 128 + row] = stat;
      mbar_arrive(bar(kBarStat + (n & 3)));

      const float2 invv = make_float2(inv, inv);
      if (it.kind != kStageLeft) {
        // P = round(e / sum) over S in tensor memory: A operand of the second contraction
        uint32_t pk[32];
#pragma unroll
        for (int c = 0; c < kCols / 64; ++c) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float2 r = mul2(make_float2(s[64 * c + 2 * i], s[64 * c + 2 * i + 1]), invv);
            pk[i] = pack2<T>(r.x, r.y);
          }
          tmem_st32(tmem_s + 32 * (h0 + c), pk);
        }
        if (per > 1) {
#pragma unroll
          for (int i = 0; i < 32; ++i) pk[i] = 0u;
          tmem_st32(tmem_s + 32 * (1 - h0), pk);
        }
        tmem_wait_st();
        tc_fence_before();
      } else {
        // P^T goes through shared memory (MN-major A operand): rounded P in tiles 9, 10 of the ring, the
        // rounded remainder P - round(P) in tiles 11, 12.  Wait until the item that used the region last
        // has completed its second contraction.
        if (p_dist > 0) {
          const int m = n - p_dist;
          if (!mbar_wait_abortable(bar(kBarInEmpty + m % kSlots), (uint32_t)(m / kSlots) & 1u, abort_flag)) { give_up(403); break; }
        }
        const uint32_t sP = base + kOffPreg;
#pragma unroll
        for (int c8 = 0; c8 < kCols / 8; ++c8) {
          uint32_t hi[4], lo[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 r = mul2(make_float2(s[8 * c8 + 2 * i], s[8 * c8 + 2 * i + 1]), invv);
            hi[i] = pack2<T>(r.x, r.y);
            const float2 d = sub2(r, unpack2<T>(hi[i]));
            lo[i] = pack2<T>(d.x, d.y);
          }
          const uint32_t off = (uint32_t)(h0 + (c8 >> 3)) * kTileBytes + swz(row, c8 & 7);
          st_shared_v4(sP + off, hi[0], hi[1], hi[2], hi[3]);
          st_shared_v4(sP + 2 * kTileBytes + off, lo[0], lo[1], lo[2], lo[3]);
        }
        if (per > 1) {
#pragma unroll
          for (int c8 = 0; c8 < 8; ++c8) {
            const uint32_t off = (uint32_t)(1 - h0) * kTileBytes + swz(row, c8);
            st_shared_v4(sP + off, 0u, 0u, 0u, 0u);
            st_shared_v4(sP + 2 * kTileBytes + off, 0u, 0u, 0u, 0u);
          }
        }
        fence_async_smem();
      }
      mbar_arrive(bar(kBarPFull + sb));
    }
  }

  // ---- teardown ------------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == kMma1Warp) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
  }
}

// One mapped, pinned host word per device: a CTA that gives up on a bounded wait stores its code there, so
// the host can notice without a synchronisation (ma_b200_poll_status).
struct HostStatus {
  int* host = nullptr;
  int* dev = nullptr;
  bool tried = false;
};
HostStatus g_host_status[64];
std::mutex g_host_status_mutex;
bool g_attr_done[64][4];
int g_sm_count[64];

}  // namespace

size_t fused_counter_bytes(const Geometry& g) { return (size_t)g.E * g.H * 2 * g.T * sizeof(int); }

int fused_poll_status(int device) {
  if (device < 0 || device >= 64) return 0;
  std::lock_guard<std::mutex> lock(g_host_status_mutex);
  HostStatus& hs = g_host_status[device];
  if (hs.host == nullptr) return 0;
  const int code = *reinterpret_cast<volatile int*>(hs.host);
  if (code != 0) *reinterpret_cast<volatile int*>(hs.host) = 0;
  return code;
}

static int g_spin_limit_override = 0;
void fused_set_spin_limit(int iterations) { g_spin_limit_override = iterations; }

// Runs stages [stage_begin, stage_end) in one cooperative launch.
cudaError_t launch_fused(const TcPlan* plan, const Geometry& g, int* counters, int stage_begin, int stage_end,
                         int wait_deps, cudaStream_t stream) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  const bool bf = plan->qk_dtype == MA_B200_BF16;
  const int variant = (g.B == kTile ? 0 : 2) + (bf ? 0 : 1);
  const void* fn = g.B == kTile ? (bf ? (const void*)fused_kernel<__nv_bfloat16, 1> : (const void*)fused_kernel<__half, 1>)
                                : (bf ? (const void*)fused_kernel<__nv_bfloat16, 2> : (const void*)fused_kernel<__half, 2>);
  int* host_status_dev = nullptr;
  {
    // once per device and kernel variant: shared-memory opt-in, SM count, the mapped status word
    std::lock_guard<std::mutex> lock(g_host_status_mutex);
    if (!g_attr_done[dev][variant]) {
      e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
      if (e != cudaSuccess) return e;
      e = cudaDeviceGetAttribute(&g_sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
      if (e != cudaSuccess) return e;
      g_attr_done[dev][variant] = true;
    }
    HostStatus& hs = g_host_status[dev];
    if (!hs.tried) {
      hs.tried = true;
      void* hp = nullptr;
      if (cudaHostAlloc(&hp, 64, cudaHostAllocMapped) == cudaSuccess) {
        *reinterpret_cast<int*>(hp) = 0;
        void* dp = nullptr;
        if (cudaHostGetDevicePointer(&dp, hp, 0) == cudaSuccess) {
          hs.host = reinterpret_cast<int*>(hp);
          hs.dev = reinterpret_cast<int*>(dp);
        } else {
          cudaFreeHost(hp);
        }
      }
      (void)cudaGetLastError();
    }
    host_status_dev = hs.dev;
  }
  const int sms = g_sm_count[dev];
  FusedArgs a;
  a.stage_begin = stage_begin;
  a.stage_end = stage_end;
  // Heads interleaved per group.  A stage-s item waits for the stage-(s-1) items of its head, which were
  // issued (group-1)*tiles items earlier; that distance has to cover the items a CTA keeps in flight, or
  // the producer spends its time waiting on completion counters (measured on 16 heads of N = 16384 with
  // four items in flight: 365 us with 1 head per group, 225 with 2, 155 with 4, 136 with 8).  With fewer
  // tiles per head (N = 4096: 32) the same distance in items needs more heads per group.
  {
    const int tiles = g.N / kTile;
    int want = 1 + (7 * kTile + tiles - 1) / tiles;  // (want - 1) * tiles >= 7 * 128 items
    if (want < 8) want = 8;
    a.group = g.E * g.H < want ? g.E * g.H : want;
  }
  a.wait_deps = wait_deps;
  a.reuse_slots = wait_deps && (stage_begin == 0 && stage_end == 2 * g.T) ? 1 : 0;
  a.spin_limit = g_spin_limit_override > 0 ? g_spin_limit_override : (1 << 24);
  a.counters = counters;
  a.host_status = host_status_dev;
  const int total = (stage_end - stage_begin) * (g.N / kTile) * g.E * g.H;
  const int grid = total < sms ? total : sms;
  void* params[] = {(void*)&plan->maps, (void*)&g, (void*)&a};
  return cudaLaunchCooperativeKernel(fn, dim3(grid), dim3(kThreads), params, kSmemBytes, stream);
}

}  // namespace ma
