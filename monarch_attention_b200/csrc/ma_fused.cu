// Persistent, warp-specialised tcgen05 kernel that runs every stage of the forward pass
// in ONE launch.
//
// Work items are 128-row tiles: (stage, head, tile index).  Stage s of the 2T stages is
//   right-factor (s even, s < 2T-2), left-factor (s odd, s < 2T-2),
//   right-factor with V (s = 2T-2), output (s = 2T-1)          (reference: ma/ma_torch.py:100-105).
// Items are laid out head-group-major: for each group of up to G heads, for each stage, for each
// head of the group, for each tile.  CTA c of the persistent grid takes items c, c+grid, ... in
// that order.  A stage-s item of a head may start once all 128 items of stage s-1 of that head are
// done; completion is counted in global memory (one counter per head and stage).  Because the
// heads of a group are interleaved, the items a stage depends on were issued (G-1)*128 items
// earlier, so the bounded wait in the producer rarely spins, while the state of only ~G heads
// (a few MB each) is live at a time and stays in L2: the factors never round-trip to HBM.
// The launch is cooperative so that every CTA of the grid is resident, which the in-order
// item schedule needs for forward progress.
//
// Inside a CTA (512 threads, one CTA per SM, all 512 tensor-memory columns):
//   warps 0-3, 4-7   two softmax groups on alternating items, one tile row per thread: two passes
//              over the row of S (max; exp, sums, entropy) in short loops that read 32-column
//              chunks with tcgen05.ld one chunk ahead of the arithmetic, P (16-bit) to swizzled
//              shared memory, row statistics to a small ring for the epilogue
//   warps 8-11 epilogue group: waits for O[n%2], scales it by the row statistics and stores rows to
//              global memory with 32-byte stores (it absorbs the latency of the second contraction so
//              that the softmax groups never wait for it)
//   warp 12    TMA producer: waits for the item's dependency, loads the 2-3 operand tiles and the
//              512-byte row vector (cr or cl) of the item into a 3-deep ring of 48 KB slots
//   warp 13    MMA issuer 1: S = A B^T for item n (tcgen05.mma, fp32 accumulator S[n%2] in tensor memory)
//   warp 14    MMA issuer 2: the second contraction of item n from P[n%2] into O[n%2]
//   warp 15    publisher: device-scope fence and one increment of the item's completion counter
// All hand-offs are mbarriers; every wait is bounded and abortable (see ma_sm100.cuh).
#include <cuda.h>

#include <stdio.h>
#include <stdlib.h>

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

constexpr int kSoftmaxWarps = 8;    // two groups of four
constexpr int kEpilogueWarp0 = 8;   // warps 8..11
constexpr int kProducerWarp = 12;
constexpr int kMma1Warp = 13;
constexpr int kMma2Warp = 14;
constexpr int kPublishWarp = 15;
constexpr int kThreads = 16 * 32;

// Operand tiles live in a ring of nine 16 KB tiles.  An item takes two consecutive tiles (A, B) or
// three (A, B, V) - never wrapping: if the tail of the ring is too short it is skipped - so up to four
// items of the two-tile kinds are in flight, which is what hides the latency of their loads.
constexpr int kNumBarsConst = 32;
// Tensor memory: three S accumulators (columns 0, 128, 256) so that S = A B^T of a group's next item
// can run while the group is still reading its current one, and one O accumulator (column 384): the
// epilogue empties it much faster than items arrive.
constexpr int kSBuffers = 3;
constexpr uint32_t kTmemO = 384;
constexpr int kRingTiles = 9;
constexpr int kItemsInFlight = 4;  // depth of the per-item barrier / row-vector rings
constexpr uint32_t kOffSlots = 0;
constexpr uint32_t kOffP = kOffSlots + kRingTiles * kTileBytes;  // 2 x 32 KB
constexpr uint32_t kOffSv = kOffP + 2 * 2 * kTileBytes;          // 2 x 4 KB (per P buffer; left stage)
constexpr uint32_t kOffVec = kOffSv + 2 * 4096;                  // 4 x 512 B (per item in flight)
static_assert(kOffP % 1024 == 0 && kOffSv % 1024 == 0, "swizzled operands need 1024-byte alignment");
constexpr uint32_t kOffStats = kOffVec + kItemsInFlight * 512;   // 4 x 128 x 3 floats of row statistics
constexpr uint32_t kOffBar = kOffStats + 4 * 128 * 12;
constexpr int kDescRing = 16;  // item descriptors; deeper than the producer can run ahead of the publisher (9)
constexpr uint32_t kOffDesc = kOffBar + 8 * kNumBarsConst + 16;
constexpr uint32_t kSmemUsed = kOffDesc + 8 * kDescRing;
constexpr uint32_t kSmemBytes = kSmemUsed + 1024;

// mbarrier indices (8 bytes each)
enum {
  kBarInFull = 0,    // [4] operand tiles of an item filled by TMA
  kBarInEmpty = 4,   // [4] operand tiles of an item released by the second contraction
  kBarSFull = 8,     // [3] S accumulator ready
  kBarSEmpty = 11,   // [3] S accumulator read by the softmax group
  kBarPFull = 14,    // [2] P written
  kBarPEmpty = 16,   // [2] P consumed by the second contraction
  kBarOFull = 18,    // [1] O accumulator ready
  kBarOEmpty = 19,   // [1] O accumulator read by the epilogue group
  kBarDone = 20,     // [4] item stored to global memory by all 128 epilogue threads
  kBarPubFree = 24,  // [4] completion of that item published
  kBarStat = 28,     // [4] row statistics of the item written by its softmax group
  kNumBars = 32
};

struct FusedArgs {
  int stage_begin, stage_end;  // stages [begin, end) of the 2T stages run in this launch
  int group;                   // heads interleaved per group
  int wait_deps;               // wait on the completion counters of the previous stage
  int* counters;               // (E*H, 2T) ints, zeroed before the first launch of a call
  int dbg;                     // ablation switches, read only by diagnostic builds (-DMA_DIAG)
};

struct Item {
  int kind, first, stage, eh, tile;
};

// Walks the items of one CTA (global indices blockIdx.x, blockIdx.x + grid, ...) without a division
// per item: the position (group, stage, head in group, tile) is carried along.
struct ItemCursor {
  int gi, sl, hh, tile, gh;  // group, stage within the launch, head within the group, tile, heads in this group
  int idx, total, stride, nst, group, EH, stage_begin, last_stage;
  int tph;       // tiles per head and stage: N / 128
  int ring_pos;  // next free tile of the operand ring (advanced by take())

  __device__ __forceinline__ void init(int first_idx, int stride_, const Geometry& g, const FusedArgs& a) {
    EH = g.E * g.H;
    nst = a.stage_end - a.stage_begin;
    group = a.group;
    stage_begin = a.stage_begin;
    last_stage = 2 * g.T - 1;
    tph = g.N / kTile;
#ifdef MA_DIAG
    total = (a.dbg & 32) ? 0 : nst * tph * EH;
#else
    total = nst * tph * EH;
#endif
    stride = stride_;
    idx = first_idx;
    ring_pos = 0;
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
    it.stage = stage_begin + sl;
    it.kind = it.stage == last_stage
                  ? kStageOutput
                  : (it.stage == last_stage - 1 ? kStageRightWithV : ((it.stage & 1) ? kStageLeft : kStageRight));
    it.first = it.stage == 0;
    return it;
  }
  // The current item plus its place in the operand ring; call exactly once per item, in item order.
  // first_tile: index of the item's A tile (B and V follow it); skipped: tiles wasted at the ring's tail.
  __device__ __forceinline__ Item take(int* first_tile, int* tiles, int* skipped) {
    const Item it = get();
    const int k = (it.kind == kStageRightWithV || it.kind == kStageOutput) ? 3 : 2;
    int sk = 0;
    if (ring_pos + k > kRingTiles) {
      sk = kRingTiles - ring_pos;
      ring_pos = 0;
    }
    *first_tile = ring_pos;
    *tiles = k;
    *skipped = sk;
    ring_pos += k;
    if (ring_pos == kRingTiles) ring_pos = 0;
    return it;
  }
};

template <typename T, int PER>  // PER: key blocks (or columns j) per 128-row tile: 1 (block size 128) or 2 (64)
__global__ void __launch_bounds__(kThreads, 1) fused_kernel(const __grid_constant__ TcMaps maps, const Geometry g,
                                                            const FusedArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + kOffBar;
  auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + kOffBar + 8 * kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + kOffBar + 8 * kNumBars + 8);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef MA_DIAG
  const int dbg_flags = args.dbg;  // ablation switches for timing experiments (diagnostic builds only)
#else
  constexpr int dbg_flags = 0;
#endif
  constexpr int kFmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
  const int tph = g.N / kTile;        // tiles per head and stage
  constexpr int per = PER;
  constexpr int kRowsPer = kTile / PER;  // rows of one block (or column) inside a tile = block size = block count
  const int total = (dbg_flags & 32) ? 0 : (args.stage_end - args.stage_begin) * tph * g.E * g.H;
  const int nst_all = 2 * g.T;


  if (tid == 0) {
    static_assert(kNumBars == kNumBarsConst, "barrier count");
    for (int i = 0; i < kItemsInFlight; ++i) { mbar_init(bar(kBarInFull + i), 1); mbar_init(bar(kBarInEmpty + i), 1); }
    for (int i = 0; i < 2; ++i) {

      mbar_init(bar(kBarPFull + i), 128);
      mbar_init(bar(kBarPEmpty + i), 1);

    }
    for (int i = 0; i < kSBuffers; ++i) {
      mbar_init(bar(kBarSFull + i), 1);
      mbar_init(bar(kBarSEmpty + i), 128);
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
                     base + kOffBar + 8 * kNumBars),
                 "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  {  // zero both 16 x 128 operands that will carry 1/rowsum in their first row (left-factor stage)
    uint32_t* z = reinterpret_cast<uint32_t*>(base_ptr + kOffSv);
    for (int i = tid; i < 2 * 1024; i += kThreads) z[i] = 0u;
    // With two blocks per tile every row of P has entries only in the 64 columns of its own block; the
    // other 64 are never written and have to read as zero in the second contraction.
    if (per > 1) {
      uint4* zp = reinterpret_cast<uint4*>(base_ptr + kOffP);
      for (int i = tid; i < (int)(2 * 2 * kTileBytes / 16); i += kThreads) zp[i] = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  // Only the producer walks the item schedule.  It leaves a two-word descriptor per item in a small
  // ring (written before the arrive that opens the item's operand barrier, so every later hand-off
  // carries it); the other roles read it once their first wait for the item has returned.
  const int n_items = total > (int)blockIdx.x ? (total - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  auto read_item = [&](int n, int* first_tile) {
    const int2 d = *reinterpret_cast<const int2*>(base_ptr + kOffDesc + (n & (kDescRing - 1)) * 8);
    Item it;
    it.kind = d.x & 3;
    it.first = (d.x >> 2) & 1;
    *first_tile = (d.x >> 3) & 15;
    it.tile = (d.x >> 8) & 255;
    it.stage = d.x >> 16;
    it.eh = d.y;
    return it;
  };
  auto give_up = [&](int code) {
    *abort_flag = 1;
    atomicCAS(g.status, 0, code);
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
      int free_tiles = kRingTiles, oldest = 0;     // ring accounting: items [oldest, n) hold tiles
      int held[kItemsInFlight] = {0, 0, 0, 0};     // tiles (incl. skipped tail) held by item m, at m % 4
      ItemCursor cur;
      bool ok = true;
      for (cur.init(blockIdx.x, gridDim.x, g, args); cur.valid() && ok; cur.next(), ++n) {
        int t0, ntiles, skipped;
        const Item it = cur.take(&t0, &ntiles, &skipped);
        const int e = it.eh / g.H, h = it.eh - e * g.H;
        const int slot = n % kItemsInFlight;
        if (args.wait_deps && it.stage > 0) {
          const int* ctr = args.counters + it.eh * nst_all + (it.stage - 1);
          bool ready = false;
          for (int spin = 0; spin < (1 << 24); ++spin) {
            if (ld_acquire_gpu(ctr) >= tph) { ready = true; break; }
            if ((spin & 255) == 255 && *abort_flag) break;
            __nanosleep(32);
          }
          if (!ready) { give_up(201); break; }
          fence_proxy_async_all();  // the state was written with ordinary stores; the loads below are TMA
        }
        // make room: items release their tiles in order (second contraction of item m done)
        while (free_tiles < ntiles + skipped || n - oldest >= kItemsInFlight) {
          if (!mbar_wait_abortable(bar(kBarInEmpty + oldest % kItemsInFlight), (uint32_t)(oldest / kItemsInFlight) & 1u,
                                   abort_flag)) {
            give_up(202);
            ok = false;
            break;
          }
          free_tiles += held[oldest % kItemsInFlight];
          ++oldest;
        }
        if (!ok) break;
        held[slot] = ntiles + skipped;
        free_tiles -= ntiles + skipped;
        const uint32_t sA = base + kOffSlots + t0 * kTileBytes, sB = sA + kTileBytes, sV = sB + kTileBytes;
        const uint32_t vec = base + kOffVec + slot * 512;
        const uint32_t full = bar(kBarInFull + slot);
        const bool right = it.kind == kStageRight || it.kind == kStageRightWithV;
        const bool three = ntiles == 3;
        const bool has_vec = !(right && it.first);
        *reinterpret_cast<int2*>(base_ptr + kOffDesc + (n & (kDescRing - 1)) * 8) =
            make_int2(it.kind | (it.first << 2) | (t0 << 3) | (it.tile << 8) | (it.stage << 16), it.eh);
        mbar_expect_tx(full, (three ? 3u : 2u) * kTileBytes + (has_vec ? 512u : 0u));
        if (right) {
          if (it.first) tma_load_5d(sA, &maps.q_blk, full, 0, 0, it.tile, h, e);
          else tma_load_5d(sA, &maps.ar_blk, full, 0, 0, it.tile, it.eh, 0);
          tma_load_5d(sB, &maps.k_blk, full, 0, 0, it.tile, h, e);
          if (three) tma_load_5d(sV, &maps.v_blk, full, 0, 0, it.tile, h, e);
          if (has_vec) bulk_load(vec, g.cr + ((long long)it.eh * g.M + it.tile * per) * g.B, 512, full);
        } else {
          // one box per column j of the tile: rows jj*(128/per) + l, the same row order as the blocks of
          // a right-factor tile (a row's own columns are then the same for every lane of a warp, which
          // the warp-wide tensor-memory loads of the softmax need)
          for (int jj = 0; jj < per; ++jj)
            tma_load_5d(sA + jj * (kTileBytes / per), &maps.q_col, full, 0, it.tile * per + jj, 0, h, e);
          tma_load_5d(sB, &maps.al_blk, full, 0, 0, it.tile, it.eh, 0);
          if (three) tma_load_5d(sV, &maps.y_blk, full, 0, 0, it.tile, it.eh, 0);
          bulk_load(vec, g.cl + ((long long)it.eh * g.B + it.tile * per) * g.M, 512, full);
        }
        issued = n + 1;
      }
      // Drain: make sure every copy this thread started has landed before the CTA may exit.
      for (int m = max(0, issued - kItemsInFlight); m < issued; ++m)
        (void)mbar_wait(bar(kBarInFull + m % kItemsInFlight), (uint32_t)(m / kItemsInFlight) & 1u);
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
        const int slot = n % kItemsInFlight, sb = n % kSBuffers;
        if (!mbar_wait_abortable(bar(kBarInFull + slot), (uint32_t)(n / kItemsInFlight) & 1u, abort_flag)) { give_up(301); break; }
        int t0;
        (void)read_item(n, &t0);
        if (!mbar_wait_abortable(bar(kBarSEmpty + sb), ((uint32_t)(n / kSBuffers) & 1u) ^ 1u, abort_flag)) { give_up(302); break; }
        tc_fence_after();
        if (!(dbg_flags & 8)) {
          const uint32_t dA = dA0 + t0 * kTileStep, dB = dA + kTileStep;
#pragma unroll
          for (int kk = 0; kk < kHead / 16; ++kk) mma_f16_lo(tmem + sb * 128, dA + kk * 2, dB + kk * 2, idesc1, kk > 0);
        }
        mma_commit(bar(kBarSFull + sb));
      }
    }
  } else if (warp == kMma2Warp) {
    // =========================== MMA issuer 2: O = P [B | V] =================================
    if (lane == 0) {
      const uint32_t dP_k0 = smem_desc_lo(base + kOffP, 16);           // P as K-major A operand
      const uint32_t dP_mn0 = smem_desc_lo(base + kOffP, kTileBytes);   // P^T as MN-major A operand
      const uint32_t dS0 = smem_desc_lo(base + kOffSv, 16);             // 16 x 128 K-major operand (1/rowsum)
      const uint32_t dTmn0 = smem_desc_lo(base + kOffSlots, kTileBytes);  // ring tile 0 as an MN-major operand
      constexpr uint32_t kTileStep = kTileBytes >> 4, kPStep = (2 * kTileBytes) >> 4;
      for (int n = 0; n < n_items; ++n) {
        const int pb = n & 1, slot = n % kItemsInFlight;
        const uint32_t ph2 = (uint32_t)(n >> 1) & 1u;
        if (!mbar_wait_abortable(bar(kBarPFull + pb), ph2, abort_flag)) { give_up(303); break; }
        int t0;
        const int kind = read_item(n, &t0).kind;
        if (!mbar_wait_abortable(bar(kBarOEmpty), ((uint32_t)n & 1u) ^ 1u, abort_flag)) { give_up(304); break; }
        tc_fence_after();
        if (!(dbg_flags & 8)) {
          const uint32_t dPk = dP_k0 + pb * kPStep, dPmn = dP_mn0 + pb * kPStep;
          // tiles of the item: A (left stage: q' written over it), B, V
          const uint32_t dA = dTmn0 + t0 * kTileStep, dB = dA + kTileStep, dV = dB + kTileStep;
          const uint32_t tmem_o = tmem + kTmemO;
          if (kind == kStageRight) {
            constexpr uint32_t idesc = instr_desc(kFmt, 0, 1, kHead, kTile);
#pragma unroll
            for (int kk = 0; kk < kTile / 16; ++kk)
              mma_f16_lo(tmem_o, dPk + ((kk >> 2) * kTileStep + (kk & 3) * 2), dB + kk * 128, idesc, kk > 0);
          } else if (kind == kStageRightWithV) {
            // the V tile follows the B tile in the ring: second 64-column atom of a 128-wide operand
            constexpr uint32_t idesc = instr_desc(kFmt, 0, 1, 2 * kHead, kTile);
#pragma unroll
            for (int kk = 0; kk < kTile / 16; ++kk)
              mma_f16_lo(tmem_o, dPk + ((kk >> 2) * kTileStep + (kk & 3) * 2), dB + kk * 128, idesc, kk > 0);
          } else if (kind == kStageLeft) {
            constexpr uint32_t idesc_q = instr_desc(kFmt, 1, 1, kHead, kTile);
            constexpr uint32_t idesc_s = instr_desc(kFmt, 1, 0, 16, kTile);
            const uint32_t dS = dS0 + pb * (4096 >> 4);
#pragma unroll
            for (int kk = 0; kk < kTile / 16; ++kk) {
              mma_f16_lo(tmem_o, dPmn + kk * 128, dA + kk * 128, idesc_q, kk > 0);
              mma_f16_lo(tmem_o + kHead, dPmn + kk * 128, dS + ((kk >> 2) * 128 + (kk & 3) * 2), idesc_s, kk > 0);
            }
          } else {
            constexpr uint32_t idesc = instr_desc(kFmt, 0, 1, kHead, kTile);
#pragma unroll
            for (int kk = 0; kk < kTile / 16; ++kk)
              mma_f16_lo(tmem_o, dPk + ((kk >> 2) * kTileStep + (kk & 3) * 2), dV + kk * 128, idesc, kk > 0);
          }
        }
        mma_commit(bar(kBarOFull));
        mma_commit(bar(kBarPEmpty + pb));
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
        int t0;
        const Item it = read_item(n, &t0);
        if (it.stage != nst_all - 1) {  // nothing consumes the output stage
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
      int t0_unused;
      const Item it = read_item(n, &t0_unused);
      const float* stp = reinterpret_cast<const float*>(base_ptr + kOffStats) + ((n & 3) * 128 + row) * 3;
      const float4 st = make_float4(stp[0], stp[1], stp[2], 0.f);
      const uint32_t tmem_o = tmem + lane_base + kTmemO;
      T* dst0;
      // Row of the tile -> (row within its block or column, which of the tile's `per` blocks / columns).
      // Right-factor tiles hold blocks one after the other (row = blk*B + j); the accumulator of the
      // left-factor stage (row = jj*M + m) and the column tiles of the output stage (row = jj*M + l) are
      // indexed the same way.
      const int rin = row & (kRowsPer - 1), rblk = row / kRowsPer;
      long long row_y = 0;
      if (it.kind == kStageRight || it.kind == kStageRightWithV) {
        const long long rr = ((long long)it.eh * g.B + rin) * g.M + it.tile * per + rblk;
        dst0 = reinterpret_cast<T*>(g.al) + rr * kHead;
        g.cl[rr] = st.z;
        row_y = rr;
      } else if (it.kind == kStageLeft) {
        dst0 = reinterpret_cast<T*>(g.ar) + (((long long)it.eh * g.M + rin) * g.B + it.tile * per + rblk) * kHead;
      } else {
        const int e = it.eh / g.H, h = it.eh - e * g.H;
        dst0 = reinterpret_cast<T*>(const_cast<void*>(g.out.ptr)) + (long long)e * g.out.se + (long long)h * g.out.sh +
               ((long long)rin * g.B + it.tile * per + rblk) * g.out.sn;
      }
      // 64 accumulator columns -> one 128-byte row: both chunk loads in flight, then 4 x 32-byte stores
      // (every touched sector is written whole)
      auto store_row = [&](T* dst, uint32_t taddr, float scale) {
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
          for (int i = 0; i < 8; ++i) w[i] = pack2<T>(p[2 * i] * scale, p[2 * i + 1] * scale);
          st_global_v8(dst + h8 * 16, w);
        }
      };
      if (!(dbg_flags & 4)) {
        store_row(dst0, tmem_o, st.x);
        if (it.kind == kStageRightWithV) {
          store_row(reinterpret_cast<T*>(g.y) + row_y * kHead, tmem_o + kHead, st.y);
        } else if (it.kind == kStageLeft) {
          float o[32];
          tmem_ld32(tmem_o + kHead, o);
          g.cr[((long long)it.eh * g.M + rin) * g.B + it.tile * per + rblk] = o[0] + o[1];
        }
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
    bool alive = true;
#if defined(MA_DIAG) && defined(MA_TRACE)
    long long tr[8][8];
    const bool tracer = (dbg_flags & 64) && (blockIdx.x == 0 || blockIdx.x == 77) && (tid & 127) == 0;
    const long long t_loop = clock64();
#define MA_TR(i) if (tracer && (n >> 1) < 8) tr[n >> 1][i] = clock64() - t_loop;
#else
#define MA_TR(i)
#endif
    int n = grp;
    for (; n < n_items; n += 2) {
      MA_TR(0)
      const int slot = n % kItemsInFlight, sb = n & 1, s3 = n % kSBuffers;  // P buffer / S accumulator of the item
      const uint32_t ph2 = (uint32_t)(n >> 1) & 1u;
      const uint32_t sP = base + kOffP + sb * 2 * kTileBytes;
      const float* vec = reinterpret_cast<const float*>(base_ptr + kOffVec + slot * 512);

      if (!mbar_wait_abortable(bar(kBarInFull + slot), (uint32_t)(n / kItemsInFlight) & 1u, abort_flag)) { give_up(401); alive = false; break; }
      int tile0;
      const Item it = read_item(n, &tile0);
      const bool right = it.kind == kStageRight || it.kind == kStageRightWithV;
      const uint32_t sA = base + kOffSlots + tile0 * kTileBytes;
      if (!mbar_wait_abortable(bar(kBarSFull + s3), (uint32_t)(n / kSBuffers) & 1u, abort_flag)) { give_up(402); alive = false; break; }
      tc_fence_after();
      MA_TR(1)
      const uint32_t tmem_s = tmem + lane_base + s3 * 128;

      // Two passes over the row of S, each a short loop over 64-column halves whose body handles two
      // 32-column chunks in two register buffers: the tensor-memory load of the next chunk is in flight
      // while the current one is processed, and the loop body stays small enough to sit in the
      // instruction cache (a fully unrolled 128-column pass starves the schedulers of instructions).
      float row_scale = 0.f;
      if (right) row_scale = g.sm_scale / ((it.first ? 1.0f : vec[row]) + kEps);
      float ca[32], cb[32];
      float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
      float s0 = 0.f, s1 = 0.f, t0 = 0.f, t1 = 0.f;
      float mul, off;
      // P row `row`, columns [col0, col0+32): K-major operand (row = M index) for the right-factor and
      // output stages, MN-major operand holding P^T (row = K index) for the left-factor stage - the
      // bytes land in the same place either way.
      auto store_p = [&](const uint32_t (&packed)[16], int col0) {
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const uint32_t col = col0 + q4 * 8;
          st_shared_v4(sP + (col >> 6) * kTileBytes + swz(row, (col & 63) >> 3), packed[q4 * 4], packed[q4 * 4 + 1],
                       packed[q4 * 4 + 2], packed[q4 * 4 + 3]);
        }
      };
      // 64-column halves of the row this thread works on: both, or - with two blocks per tile - only the
      // half that belongs to the row's own block or column (rows are blk*64 + j in the right-factor
      // tiles and jj*64 + l in the column tiles; columns are blk*64 + i, or jj*64 + m); the other half of
      // P stays zero from the start of the launch.
      const int h0 = per > 1 ? (row >> 6) : 0, h1 = per > 1 ? h0 + 1 : 2;  // uniform within a warp
      tmem_ld32_nowait(tmem_s + 64 * h0, ca);
      if (right) {
        auto max_chunk = [&](const float (&s)[32]) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            m0 = max3(m0, s[i], s[i + 1]);
            m1 = max3(m1, s[i + 2], s[i + 3]);
            m2 = max3(m2, s[i + 4], s[i + 5]);
            m3 = max3(m3, s[i + 6], s[i + 7]);
          }
        };
#pragma unroll 1
        for (int h = h0; h < h1; ++h) {
          tmem_wait_ld(ca); tmem_ld32_nowait(tmem_s + 64 * h + 32, cb); max_chunk(ca);
          tmem_wait_ld(cb); tmem_ld32_nowait(tmem_s + 64 * (h + 1 < h1 ? h + 1 : h0), ca); max_chunk(cb);
        }
        MA_TR(2)
        const float vmax = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
        const float top = fmaxf(vmax * row_scale, kEps);  // lower clamp on the row maximum
        mul = row_scale * kLog2e;
        off = top * kLog2e;
        MA_TR(3)
        if (!mbar_wait_abortable(bar(kBarPEmpty + sb), ph2 ^ 1u, abort_flag)) { tmem_wait_ld(ca); give_up(403); alive = false; break; }
        MA_TR(4)
        auto exp_chunk = [&](const float (&s)[32], int col0) {
          uint32_t packed[16];
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float u0 = fmaf(s[i], mul, -off), u1 = fmaf(s[i + 1], mul, -off);
            const float u2 = fmaf(s[i + 2], mul, -off), u3 = fmaf(s[i + 3], mul, -off);
            const float e0 = ex2(u0), e1 = ex2(u1), e2 = ex2(u2), e3 = ex2(u3);
            s0 += e0 + e1;
            s1 += e2 + e3;
            t0 = fmaf(e0, u0, fmaf(e1, u1, t0));
            t1 = fmaf(e2, u2, fmaf(e3, u3, t1));
            packed[i >> 1] = pack2<T>(e0, e1);
            packed[(i >> 1) + 1] = pack2<T>(e2, e3);
          }
          store_p(packed, col0);
        };
#pragma unroll 1
        for (int h = h0; h < h1; ++h) {
          tmem_wait_ld(ca); tmem_ld32_nowait(tmem_s + 64 * h + 32, cb); exp_chunk(ca, 64 * h);
          tmem_wait_ld(cb);
          if (h + 1 < h1) tmem_ld32_nowait(tmem_s + 64 * (h + 1), ca);
          else { tc_fence_before(); mbar_arrive(bar(kBarSEmpty + s3)); }  // S has been read in full
          exp_chunk(cb, 64 * h + 32);
        }
      } else {
        auto max_chunk = [&](const float (&s)[32], const float* c) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            const float4 x = *reinterpret_cast<const float4*>(c + i);
            const float4 y = *reinterpret_cast<const float4*>(c + i + 4);
            m0 = max3(m0, s[i] - x.x, s[i + 1] - x.y);
            m1 = max3(m1, s[i + 2] - x.z, s[i + 3] - x.w);
            m2 = max3(m2, s[i + 4] - y.x, s[i + 5] - y.y);
            m3 = max3(m3, s[i + 6] - y.z, s[i + 7] - y.w);
          }
        };
#pragma unroll 1
        for (int h = h0; h < h1; ++h) {
          tmem_wait_ld(ca); tmem_ld32_nowait(tmem_s + 64 * h + 32, cb); max_chunk(ca, vec + 64 * h);
          tmem_wait_ld(cb); tmem_ld32_nowait(tmem_s + 64 * (h + 1 < h1 ? h + 1 : h0), ca); max_chunk(cb, vec + 64 * h + 32);
        }
        MA_TR(2)
        const float vmax = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
        mul = kLog2e;
        off = vmax * kLog2e;
        MA_TR(3)
        if (!mbar_wait_abortable(bar(kBarPEmpty + sb), ph2 ^ 1u, abort_flag)) { tmem_wait_ld(ca); give_up(403); alive = false; break; }
        MA_TR(4)
        auto exp_chunk = [&](const float (&s)[32], const float* c, int col0) {
          uint32_t packed[16];
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float4 x = *reinterpret_cast<const float4*>(c + i);
            const float e0 = ex2(fmaf(s[i] - x.x, mul, -off)), e1 = ex2(fmaf(s[i + 1] - x.y, mul, -off));
            const float e2 = ex2(fmaf(s[i + 2] - x.z, mul, -off)), e3 = ex2(fmaf(s[i + 3] - x.w, mul, -off));
            s0 += e0 + e1;
            s1 += e2 + e3;
            packed[i >> 1] = pack2<T>(e0, e1);
            packed[(i >> 1) + 1] = pack2<T>(e2, e3);
          }
          store_p(packed, col0);
        };
#pragma unroll 1
        for (int h = h0; h < h1; ++h) {
          tmem_wait_ld(ca); tmem_ld32_nowait(tmem_s + 64 * h + 32, cb); exp_chunk(ca, vec + 64 * h, 64 * h);
          tmem_wait_ld(cb);
          if (h + 1 < h1) tmem_ld32_nowait(tmem_s + 64 * (h + 1), ca);
          else { tc_fence_before(); mbar_arrive(bar(kBarSEmpty + s3)); }  // S has been read in full
          exp_chunk(cb, vec + 64 * h + 32, 64 * h + 32);
        }
      }
      const float row_sum = s0 + s1, row_ent = t0 + t1;
      MA_TR(5)

      float4 st = make_float4(0.f, 0.f, 0.f, 0.f);  // scale of O[:, :64], scale of O[:, 64:], cl, unused
      if (right) {
        const float denom = row_sum + kEps;
        const float rden = __frcp_rn(denom);
        st.x = g.sm_scale * rden;
        st.y = rden;
        st.z = kLn2 * (row_ent - __log2f(denom) * row_sum) * rden;
      } else if (it.kind == kStageLeft) {
        const float inv = __frcp_rn(row_sum);
        st.x = 1.0f;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {  // q' = q / rowsum, in place (S = A B^T has consumed the tile)
          const uint4 v = ld_shared_v4(sA + swz(row, ch));
          const float2 a = unpack2<T>(v.x), b = unpack2<T>(v.y), c2 = unpack2<T>(v.z), d = unpack2<T>(v.w);
          st_shared_v4(sA + swz(row, ch), pack2<T>(a.x * inv, a.y * inv), pack2<T>(b.x * inv, b.y * inv),
                       pack2<T>(c2.x * inv, c2.y * inv), pack2<T>(d.x * inv, d.y * inv));
        }
        // 1/rowsum as a 16-bit value plus its 16-bit remainder, in rows 0 and 1 of the 16 x 128 operand
        // (row r, column c of a swizzled 64-column atom: r*128 + ((c/8) ^ r)*16 + (c%8)*2 bytes): the
        // column sums cr = sum_l P[l, m] / rowsum_l then carry the rounding of P only.
        uint8_t* atom = base_ptr + kOffSv + sb * 4096 + (row >> 6) * 2048;
        const int c = row & 63;
        const T hi = Cvt<T>::from_f(inv);
        reinterpret_cast<T*>(atom)[c] = hi;
        *reinterpret_cast<T*>(atom + 128 + (((c >> 3) ^ 1) << 4) + ((c & 7) << 1)) = Cvt<T>::from_f(inv - Cvt<T>::to_f(hi));
      } else {
        st.x = __frcp_rn(row_sum);
      }
      // Row statistics for the epilogue group.  The 4-deep ring cannot be overrun: item n+4 of this
      // group needs P[n%2] free twice over, i.e. the second contraction of item n+2, which needs
      // O[n%2] free, i.e. the epilogue of item n finished.
      {
        float* stp = reinterpret_cast<float*>(base_ptr + kOffStats) + ((n & 3) * 128 + row) * 3;
        stp[0] = st.x;
        stp[1] = st.y;
        stp[2] = st.z;
      }
      mbar_arrive(bar(kBarStat + (n & 3)));
      MA_TR(6)
      fence_async_smem();
      mbar_arrive(bar(kBarPFull + sb));
      MA_TR(7)
    }
    (void)alive;
#if defined(MA_DIAG) && defined(MA_TRACE)
    if (tracer)
      for (int i = 0; i < 8 && (2 * i + grp) < n; ++i)
        printf("kind %d cta %d grp %d item %d: start %lld | S ready +%lld | ld+max +%lld | - +%lld | P free +%lld | exp +%lld | stats +%lld | arrive +%lld\n",
               dbg_flags >> 8, (int)blockIdx.x, grp, 2 * i + grp, tr[i][0], tr[i][1] - tr[i][0], tr[i][2] - tr[i][1], tr[i][3] - tr[i][2],
               tr[i][4] - tr[i][3], tr[i][5] - tr[i][4], tr[i][6] - tr[i][5], tr[i][7] - tr[i][6]);
#endif


  }

  // ---- teardown ------------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == kMma1Warp) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
  }
}

}  // namespace

size_t fused_counter_bytes(const Geometry& g) { return (size_t)g.E * g.H * 2 * g.T * sizeof(int); }

// Runs stages [stage_begin, stage_end) in one cooperative launch.
cudaError_t launch_fused(const TcPlan* plan, const Geometry& g, int* counters, int stage_begin, int stage_end,
                         int wait_deps, cudaStream_t stream) {
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return e;
  FusedArgs a;
  a.stage_begin = stage_begin;
  a.stage_end = stage_end;
  // Heads interleaved per group.  A stage-s item waits for the 128 stage-(s-1) items of its head, which
  // were issued (group-1)*128 items earlier: measured on 16 heads of N = 16384, one launch takes 365 us
  // with 1 head per group, 225 with 2, 155 with 4, 136 with 8 and 134 with 16 - below 8 the producer
  // spends its time waiting on completion counters.  8 keeps ~100 MB of state live, which still fits L2.
  // With fewer tiles per head (N = 4096: 32) the same distance in items needs more heads per group.
  {
    const int tiles = g.N / kTile;
    int want = 1 + (7 * kTile + tiles - 1) / tiles;  // (want - 1) * tiles >= 7 * 128 items
    if (want < 8) want = 8;
    a.group = g.E * g.H < want ? g.E * g.H : want;
  }
  a.wait_deps = wait_deps;
  a.counters = counters;
  a.dbg = 0;
#ifdef MA_DIAG
  if (const char* d = getenv("MA_B200_DEBUG")) a.dbg = atoi(d);
  if (const char* d = getenv("MA_B200_GROUP")) a.group = atoi(d) < g.E * g.H ? atoi(d) : g.E * g.H;
#endif
  const int total = (stage_end - stage_begin) * (g.N / kTile) * g.E * g.H;
  const int grid = total < sms ? total : sms;
  const bool bf = plan->qk_dtype == MA_B200_BF16;
  const void* fn = g.B == kTile ? (bf ? (const void*)fused_kernel<__nv_bfloat16, 1> : (const void*)fused_kernel<__half, 1>)
                                : (bf ? (const void*)fused_kernel<__nv_bfloat16, 2> : (const void*)fused_kernel<__half, 2>);
  e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
  if (e != cudaSuccess) return e;
  void* params[] = {(void*)&plan->maps, (void*)&g, (void*)&a};
  return cudaLaunchCooperativeKernel(fn, dim3(grid), dim3(kThreads), params, kSmemBytes, stream);
}

}  // namespace ma
