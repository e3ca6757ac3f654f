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
// earlier, so the bounded wait in the planner rarely spins.  The stage-to-stage state (ar, cr, al,
// cl, y) of a head lives in one of G state slots; the next group reuses the slots (its first stage
// waits for the last stage of the head that had the slot).  Every state tile is written once and read
// once; its reader drops the tile's lines from L2 (discard.global.L2), so the state is never written
// back to HBM, and q, k, v tiles are marked evict-first on their last use: HBM sees q, k, v once and the
// result once.
// The launch is cooperative so that every CTA of the grid is resident, which the in-order
// item schedule needs for forward progress.
//
// Numerics follow the reference's rounding points (ma/ma_torch.py:10-62): the fp32 accumulator of
// the first contraction is rounded to the storage type before the softmax arithmetic, the factor is
// normalised in fp32 and then rounded to the storage type before the second contraction, and the
// column sums cr of the left factor are taken from the factor before that rounding.
//
// Inside a CTA (768 threads, one CTA per SM, all 512 tensor-memory columns):
//   warps 0-15 softmax: four groups of four warps, all on the SAME item.  A tile row is split between
//              the four threads `row` of the groups (32 columns each; warps w, w+4, w+8, w+12 reach the
//              same tensor-memory lanes and share a scheduler).  Each thread reads its columns of S into
//              registers once (tcgen05.ld), takes their maximum, exponentiates against it (packed fp32
//              pairs), and the four parts of a row exchange (shift, sum, entropy sum) through shared
//              memory once and rescale.  The normalised factor P is rounded to 16 bits and written to the
//              item's P buffer in tensor memory (tcgen05.st), from where the second contraction reads it
//              as its A operand.  Only the left-factor stage, which needs P^T, goes through shared
//              memory: P as a 16-bit value plus a 16-bit remainder, so that the column sums come out of
//              the tensor core in fp32 precision.
//   warps 16-19 epilogue group: waits for O, rounds it and stores rows to global memory with 32-byte
//              stores and drops the state tiles the item read from L2
//   warp 20    planner: works out the item schedule, waits for each item's dependency, keeps the
//              accounts of the operand ring (twelve 16 KB tiles) and leaves a descriptor per item
//   warp 23    issuer: issues the item's TMA loads (2-3 operand tiles and the 512-byte row vector cr
//              or cl); each of these instructions blocks for as long as the TMA unit is busy, which is
//              why nothing else is in this warp
//   warp 21    MMA issuer 1: S = A B^T for item n (tcgen05.mma, fp32 accumulator in buffer n%3 of tensor
//              memory); its second thread is the publisher: device-scope fence and one increment of the
//              item's (head, stage) completion counter
//   warp 22    MMA issuer 2: the second contraction of item n, O written over the item's S
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

constexpr int kGroups = 4;          // softmax warpgroups: threads per tile row
constexpr int kEpilogueWarp0 = 4 * kGroups;   // four warps
constexpr int kPlannerWarp = kEpilogueWarp0 + 4;
constexpr int kMma1Warp = kPlannerWarp + 1;
constexpr int kMma2Warp = kPlannerWarp + 2;
constexpr int kIssuerWarp = kPlannerWarp + 3;
constexpr int kThreads = (kIssuerWarp + 1) * 32;
// Registers per thread after setmaxnreg, by role.  What setmaxnreg redistributes is the allocation the CTA
// was launched with (threads x registers per thread at launch), not the whole register file: a request
// beyond that pool blocks for ever, so the host checks the sum against the compiled kernel before it launches.
constexpr int kRegsSoftmax = 72, kRegsEpilogue = 96, kRegsSingle = 40;
constexpr int kRegPool = 4 * kGroups * 32 * kRegsSoftmax + 128 * kRegsEpilogue + 128 * kRegsSingle;

// Operand tiles live in a ring of twelve 16 KB tiles.  An item takes two consecutive tiles (A, B) or
// three (A, B, V) - never wrapping: if the tail of the ring is too short it is skipped and charged to
// the item.  Tiles 8..11 double as the P region of the left-factor stage (P and its remainder,
// 2 x 32 KB): while a left-factor item is in flight the ring ends at tile 8.
constexpr int kRingTiles = 12;
constexpr int kRingLeft = 8;
constexpr int kSlots = 8;  // items in flight: depth of the per-item barrier / row-vector rings
// Tensor memory: three 128-column accumulator buffers (columns 0, 128, 256): item n's S = A B^T goes to
// buffer n % 3, the softmax reads it, and the second contraction writes the item's O over it, so that S
// and O of an item share a buffer and three items can be between the first contraction and the
// epilogue.  P (16-bit pairs, 64 columns) has two buffers of its own (columns 384, 448), one per softmax
// group.
constexpr int kSBuffers = 3;
constexpr uint32_t kTmemP = 384;
constexpr uint32_t kOffSlots = 0;
constexpr uint32_t kOffPreg = kRingLeft * kTileBytes;             // P region = ring tiles 8..11
constexpr uint32_t kOffOnes = kRingTiles * kTileBytes;            // 16 x 128 K-major operand of ones (4 KB)
constexpr uint32_t kOffVec = kOffOnes + 4096;                     // kSlots x 512 B (cr or cl of the item)
constexpr uint32_t kOffStats = kOffVec + kSlots * 512;            // 4 x 128 floats (cl of the item's rows)
constexpr uint32_t kOffXch = kOffStats + 4 * 128 * 4;              // 2 x 3 x kGroups x 128 floats exchanged between the parts of a row
constexpr uint32_t kOffBar = kOffXch + 2 * 3 * kGroups * 128 * 4;
constexpr int kNumBarsConst = 56;
constexpr int kDescRing = 16;  // item descriptors; deeper than the planner can run ahead (kSlots)
constexpr uint32_t kOffDesc = kOffBar + 8 * kNumBarsConst + 16;
constexpr uint32_t kSmemUsed = kOffDesc + 16 * kDescRing;
constexpr uint32_t kSmemBytes = kSmemUsed + 1024;
static_assert(kOffPreg % 1024 == 0 && kOffOnes % 1024 == 0, "swizzled operands need 1024-byte alignment");
static_assert(kSmemBytes <= 232448, "shared memory per CTA");

// mbarrier indices (8 bytes each)
enum {
  kBarInFull = 0,     // [8] operand tiles of an item filled by TMA
  kBarInEmpty = 8,    // [8] operand tiles of an item released by the second contraction
  kBarPlan = 16,      // [8] descriptor of an item written by the planner
  kBarSFull = 24,     // [3] S accumulator ready
  kBarSEmpty = 27,    // [3] accumulator buffer (S, then O) read by the epilogue group
  kBarOFull = 30,     // [3] O accumulator ready
  kBarPFull = 33,     // [2] P written (tensor memory, or shared memory in the left-factor stage)
  kBarPEmpty = 35,    // [2] P consumed by the second contraction
  kBarStat = 37,      // [4] row statistics of the item written by its softmax group      // [4] row statistics of the item written by its softmax group
  kBarDone = 41,      // [4] item stored to global memory by all 128 epilogue threads
  kBarPubFree = 45,   // [4] completion of that item published
  kNumBars = 49
};
static_assert(kNumBars <= kNumBarsConst, "barrier count");
constexpr int kEpilogueBarrier = 1;  // named barrier of the 128 epilogue threads
constexpr int kSoftmaxBarrier = 3;   // named barriers 3..6: one per set of softmax warps that share rows

struct FusedArgs {
  int stage_begin, stage_end;  // stages [begin, end) of the 2T stages run in this launch
  int group;                   // heads interleaved per group
  int wait_deps;               // wait on the completion counters of the previous stage
  int reuse_slots;             // state of head (group g, position p) lives in slot p (needs wait_deps)
  int spin_limit;              // iterations of the planner's dependency wait before it gives up
  int* counters;               // (E*H, 2T) ints, zeroed before the first launch of a call
  int* host_status;            // mapped host word that receives the code of a wait that gave up, or nullptr
};

struct Item {
  int kind, first, stage, eh, tile, hs, e, h, t0, p_dist;  // hs: state slot of the head; t0: first ring tile
};

// Round an fp32 pair through the 16-bit storage type (the reference rounds every contraction result to
// the storage type before the fp32 softmax arithmetic, ma/ma_torch.py:11, :27, :56).
// Done on the FMA pipe (Veltkamp split with the constant 2^(24-p) + 1 for a p-bit significand: the high
// part is x rounded to nearest at p bits), because the conversion instructions share a pipe with the
// exponentials, which is the busiest one of this kernel.  The product is formed with scalar mul.rn: the
// packed form was contracted with the subtraction into one fused multiply-add, which undoes the rounding.
__device__ __forceinline__ float mul_rn(float a, float b) {
  float d;
  asm("mul.rn.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
  return d;
}
template <typename T>
__device__ __forceinline__ float2 round2(float2 x) {
  constexpr float c = std::is_same<T, __nv_bfloat16>::value ? 65537.0f : 8193.0f;
  const float2 big = make_float2(mul_rn(x.x, c), mul_rn(x.y, c));
  return add2(big, sub2(x, big));
}
// 16-bit pair -> fp32 pair without a conversion instruction where the format allows it
template <typename T>
__device__ __forceinline__ float2 widen2(uint32_t u) {
  return unpack2<T>(u);
}
template <>
__device__ __forceinline__ float2 widen2<__nv_bfloat16>(uint32_t u) {
  return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
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
    for (int i = 0; i < kSlots; ++i) {
      mbar_init(bar(kBarInFull + i), 1);
      mbar_init(bar(kBarInEmpty + i), 1);
      mbar_init(bar(kBarPlan + i), 1);
    }
    for (int i = 0; i < kSBuffers; ++i) {
      mbar_init(bar(kBarSFull + i), 1);
      mbar_init(bar(kBarSEmpty + i), 128);
      mbar_init(bar(kBarOFull + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(kBarPFull + i), 128 * kGroups);
      mbar_init(bar(kBarPEmpty + i), 1);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(bar(kBarStat + i), 128);
      mbar_init(bar(kBarDone + i), 128);
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

  // Only the planner walks the item schedule.  It leaves a four-word descriptor per item in a small
  // ring (written before the arrive that hands the item to the issuer, whose arrive on the item's
  // operand barrier carries it on to every later hand-off); the other roles read it once their first
  // wait for the item has returned.
  const int n_items = total > (int)blockIdx.x ? (total - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  auto read_item = [&](int n) {
    const int4 d = *reinterpret_cast<const int4*>(base_ptr + kOffDesc + (n & (kDescRing - 1)) * 16);
    Item it;
    it.kind = d.x & 3;
    it.first = (d.x >> 2) & 1;
    it.t0 = (d.x >> 3) & 15;
    it.tile = (d.x >> 8) & 255;
    it.stage = (d.x >> 16) & 4095;
    it.p_dist = (d.x >> 28) & 7;
    it.eh = d.y;
    it.hs = d.z;
    it.e = (int)((unsigned)d.w >> 16);
    it.h = d.w & 0xffff;
    return it;
  };
  auto give_up = [&](int code) {
    *abort_flag = 1;
    if (atomicCAS(g.status, 0, code) == 0 && args.host_status != nullptr) {
      *reinterpret_cast<volatile int*>(args.host_status) = code;
      __threadfence_system();
    }
  };

  // Registers per role (kRegsSoftmax / kRegsEpilogue / kRegsSingle; the launch gives every thread 80): a
  // softmax thread holds 32 accumulator columns, an epilogue thread a 64-column row of O, the single-thread
  // roles little.
#define ROLE_WAIT(b_, p_) mbar_wait_abortable(b_, p_, abort_flag)
  if (warp >= kPlannerWarp) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsSingle));
  if (warp == kPlannerWarp) {
    // =========================== planner =================================================
    // The warp works in batches of kBatch items: lane L < kBatch works out item n0 + L of this CTA (the
    // divisions of the schedule) and reads the completion counter it depends on, so that the latency of
    // those loads is paid once per batch (a longer batch would look further ahead than dependencies are
    // complete).  Then lane 0 takes the items one by one: ring accounts, descriptor, hand-off to the
    // issuer.  (Prefetching the q, k, v tiles of the next batch into L2 from here was measured: the
    // prefetch instructions queue in the TMA unit ahead of the loads that matter, and cost 1 - 8 %.)
    constexpr int kBatch = 4;
    int free_tiles = kRingTiles, oldest = 0, ring_pos = 0;  // ring accounting (lane 0): items [oldest, n) hold tiles
    int lefts = 0;                                          // left-factor items among them
    int last_p = -1;  // newest item that is a left-factor item or holds a tile of the P region
    // per in-flight item m, six bits at 6*(m % kSlots): tiles held (incl. skipped tail, <= 15) | left-factor item << 4
    unsigned long long held = 0ull;
    bool ok = true;
    const int EH = g.E * g.H, nst = args.stage_end - args.stage_begin, last_stage = nst_all - 1;
    const int per_group = nst * args.group * tph;
    for (int n0 = 0; n0 < n_items && ok; n0 += kBatch) {
      const int my_n = n0 + lane;
      const int idx = (int)blockIdx.x + my_n * (int)gridDim.x;
      int w0 = 0, my_eh = 0, my_hs = 0, my_eh_hi = 0, dep_ok = 1;
      if (lane < kBatch && my_n < n_items) {
        const int gi = idx / per_group;
        int r = idx - gi * per_group;
        int gh = min(args.group, EH - gi * args.group);
        if (gh < 1) gh = 1;
        const int sl = r / (gh * tph);
        r -= sl * gh * tph;
        const int hh = r / tph, tile = r - hh * tph;
        my_eh = gi * args.group + hh;
        my_hs = args.reuse_slots ? hh : my_eh;
        const int stage = args.stage_begin + sl;
        const int kind = stage == last_stage
                             ? kStageOutput
                             : (stage == last_stage - 1 ? kStageRightWithV : ((stage & 1) ? kStageLeft : kStageRight));
        w0 = kind | ((stage == 0 ? 1 : 0) << 2) | (tile << 8) | (stage << 16);
        const int e = my_eh / g.H;
        my_eh_hi = (e << 16) | (my_eh - e * g.H);  // (batch element, head) of the user tensors
        if (args.wait_deps) {
          const int* ctr = nullptr;
          if (stage > 0) ctr = args.counters + my_eh * nst_all + (stage - 1);
          else if (args.reuse_slots && gi > 0) ctr = args.counters + (my_eh - args.group) * nst_all + (nst_all - 1);
          if (ctr != nullptr) dep_ok = ld_acquire_gpu(ctr) >= tph ? 1 : 0;
        }
      }
      __syncwarp();
      const int batch = min(kBatch, n_items - n0);
      for (int i = 0; i < batch && ok; ++i) {
        const int n = n0 + i, slot = n % kSlots;
        const int d0 = __shfl_sync(0xffffffffu, w0, i), eh = __shfl_sync(0xffffffffu, my_eh, i);
        const int hs = __shfl_sync(0xffffffffu, my_hs, i), ehh = __shfl_sync(0xffffffffu, my_eh_hi, i);
        const int dok = __shfl_sync(0xffffffffu, dep_ok, i);
        if (lane == 0) {
          const int kind = d0 & 3, stage = d0 >> 16;
          const bool left = kind == kStageLeft;
          const int ntiles = (kind == kStageRightWithV || kind == kStageOutput) ? 3 : 2;
          if (!dok) {  // not yet complete when the batch was prepared: wait here
            const int* ctr = stage > 0 ? args.counters + eh * nst_all + (stage - 1)
                                       : args.counters + (eh - args.group) * nst_all + (nst_all - 1);
            bool ready = false;
            for (int spin = 0; spin < args.spin_limit; ++spin) {
              if (ld_acquire_gpu(ctr) >= tph) { ready = true; break; }
              if ((spin & 255) == 255 && *abort_flag) break;
              __nanosleep(32);
            }
            if (!ready) { give_up(201); ok = false; }
          }
          int t0 = 0, charged = 0;
          while (ok) {
            const int limit = (left || lefts > 0) ? kRingLeft : kRingTiles;
            int pos = ring_pos, sk = 0;
            if (pos + ntiles > limit) { sk = kRingTiles - pos; pos = 0; }
            if (free_tiles >= ntiles + sk && n - oldest < kSlots) { t0 = pos; charged = ntiles + sk; break; }
            // items whose second contraction has completed give their tiles back (in order)
            if (!ROLE_WAIT(bar(kBarInEmpty + oldest % kSlots), (uint32_t)(oldest / kSlots) & 1u)) {
              give_up(202);
              ok = false;
              break;
            }
            const int v = (int)(held >> (6 * (oldest % kSlots))) & 63;
            free_tiles += v & 15;
            lefts -= (v >> 4) & 1;
            ++oldest;
          }
          if (ok) {
            // A left-factor item writes P into the P region: it has to wait for the newest older item that
            // is a left-factor item itself or holds one of those tiles (items complete in order).
            const int p_dist = (left && last_p >= oldest) ? n - last_p : 0;
            ring_pos = t0 + ntiles;
            if (left || ring_pos > kRingLeft || charged > ntiles) last_p = n;
            if (ring_pos == kRingTiles) ring_pos = 0;
            held = (held & ~(63ull << (6 * slot))) | ((unsigned long long)(charged | ((left ? 1 : 0) << 4)) << (6 * slot));
            free_tiles -= charged;
            lefts += left ? 1 : 0;
            *reinterpret_cast<int4*>(base_ptr + kOffDesc + (n & (kDescRing - 1)) * 16) =
                make_int4((d0 & 0x0fffff07) | (t0 << 3) | (p_dist << 28), eh, hs, ehh);
            mbar_arrive(bar(kBarPlan + slot));
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      }
    }
  } else if (warp == kIssuerWarp) {
    // =========================== issuer: TMA loads ========================================
    if (lane == 0) {
      const unsigned long long pol_first = l2_policy_evict_first();
      int issued = 0;
      for (int n = 0; n < n_items; ++n) {
        const int slot = n % kSlots;
        if (!ROLE_WAIT(bar(kBarPlan + slot), (uint32_t)(n / kSlots) & 1u)) break;  // the planner gave up
        const Item it = read_item(n);
        const bool right = it.kind == kStageRight || it.kind == kStageRightWithV;
        const bool three = it.kind == kStageRightWithV || it.kind == kStageOutput;
        const bool has_vec = !(right && it.first);
        const uint32_t sA = base + kOffSlots + it.t0 * kTileBytes, sB = sA + kTileBytes, sV = sB + kTileBytes;
        const uint32_t vec = base + kOffVec + slot * 512;
        const uint32_t full = bar(kBarInFull + slot);
        mbar_expect_tx(full, (three ? 3u : 2u) * kTileBytes + (has_vec ? 512u : 0u));
        issued = n + 1;
        // q, k, v tiles that no later stage reads again are marked to leave L2 first
        if (right) {
          if (it.first) tma_load_5d(sA, &maps.q_blk, full, 0, 0, it.tile, it.h, it.e);
          else tma_load_5d(sA, &maps.ar_blk, full, 0, 0, it.tile, it.hs, 0);
          if (three) {
            tma_load_5d_hint(sB, &maps.k_blk, full, 0, 0, it.tile, it.h, it.e, pol_first);
            tma_load_5d_hint(sV, &maps.v_blk, full, 0, 0, it.tile, it.h, it.e, pol_first);
          } else {
            tma_load_5d(sB, &maps.k_blk, full, 0, 0, it.tile, it.h, it.e);
          }
          if (has_vec) bulk_load(vec, g.cr + ((long long)it.hs * g.M + it.tile * per) * g.B, 512, full);
        } else {
          // one box per column j of the tile: rows jj*(128/per) + l, the same row order as the blocks of
          // a right-factor tile (a row's own columns are then the same for every lane of a warp, which
          // the warp-wide tensor-memory loads of the softmax need)
          for (int jj = 0; jj < per; ++jj) {
            if (three) tma_load_5d_hint(sA + jj * (kTileBytes / per), &maps.q_col, full, 0, it.tile * per + jj, 0, it.h, it.e, pol_first);
            else tma_load_5d(sA + jj * (kTileBytes / per), &maps.q_col, full, 0, it.tile * per + jj, 0, it.h, it.e);
          }
          tma_load_5d(sB, &maps.al_blk, full, 0, 0, it.tile, it.hs, 0);
          if (three) tma_load_5d(sV, &maps.y_blk, full, 0, 0, it.tile, it.hs, 0);
          bulk_load(vec, g.cl + ((long long)it.hs * g.B + it.tile * per) * g.M, 512, full);
        }
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
        if (!ROLE_WAIT(bar(kBarInFull + slot), (uint32_t)(n / kSlots) & 1u)) { give_up(301); break; }
        const int t0 = read_item(n).t0;
        if (!ROLE_WAIT(bar(kBarSEmpty + sb), ((uint32_t)(n / kSBuffers) & 1u) ^ 1u)) { give_up(302); break; }
        tc_fence_after();
        const uint32_t dA = dA0 + t0 * kTileStep, dB = dA + kTileStep;
#pragma unroll
        for (int kk = 0; kk < kHead / 16; ++kk) mma_f16_lo(tmem + sb * 128, dA + kk * 2, dB + kk * 2, idesc1, kk > 0);
        mma_commit(bar(kBarSFull + sb));
      }
    } else if (lane == 1 && args.wait_deps) {
      // =========================== publisher (second thread of this warp) ====================
      // Makes the stores of every finished item visible device-wide and counts the item in its (head,
      // stage) completion counter.  The fence waits for the group's stores to be acknowledged, which
      // takes about a microsecond: a thread of its own keeps that off the epilogue group's path.  (The
      // output stage is consumed only when state slots are reused, by the next head in the slot.)
      for (int n = 0; n < n_items; ++n) {
        if (!ROLE_WAIT(bar(kBarDone + (n & 3)), (uint32_t)(n >> 2) & 1u)) { give_up(601); break; }
        const Item it = read_item(n);
        if (it.stage != nst_all - 1 || args.reuse_slots) {
          __threadfence();
          atomicAdd(args.counters + it.eh * nst_all + it.stage, 1);
        }
        mbar_arrive(bar(kBarPubFree + (n & 3)));
      }
    }
  } else {
    // =========================== MMA issuer 2: O = P [B | V] =================================
    if (lane == 0) {
      const uint32_t dP_mn0 = smem_desc_lo(base + kOffPreg, kTileBytes);   // P^T as MN-major A operand (left stage)
      const uint32_t dOnes = smem_desc_lo(base + kOffOnes, 16);            // 16 x 128 K-major operand of ones
      const uint32_t dTmn0 = smem_desc_lo(base + kOffSlots, kTileBytes);   // ring tile 0 as an MN-major operand
      constexpr uint32_t kTileStep = kTileBytes >> 4;
      for (int n = 0; n < n_items; ++n) {
        const int sb = n % kSBuffers, slot = n % kSlots, pb = n & 1;
        if (!ROLE_WAIT(bar(kBarPFull + pb), (uint32_t)(n >> 1) & 1u)) { give_up(303); break; }
        const Item it = read_item(n);
        const int kind = it.kind;
        tc_fence_after();
        // tiles of the item: A, B, V
        const uint32_t dA = dTmn0 + it.t0 * kTileStep, dB = dA + kTileStep, dV = dB + kTileStep;
        const uint32_t tmem_o = tmem + sb * 128, tmem_p = tmem + kTmemP + pb * 64;  // O goes over the item's S
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
        mma_commit(bar(kBarOFull + sb));
        mma_commit(bar(kBarPEmpty + pb));
        mma_commit(bar(kBarInEmpty + slot));
      }
    }
  }
  } else if (warp >= kEpilogueWarp0) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsEpilogue));
    // =========================== epilogue group =================================================
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const unsigned long long pol_first = l2_policy_evict_first();
    for (int n = 0; n < n_items; ++n) {
      const int sb = n % kSBuffers;
      const bool got = ROLE_WAIT(bar(kBarStat + (n & 3)), (uint32_t)(n >> 2) & 1u) &&
                       ROLE_WAIT(bar(kBarOFull + sb), (uint32_t)(n / kSBuffers) & 1u);
      // all 128 threads leave together or not at all (a thread that went on alone would strand the
      // others at the group barrier below)
      if (named_barrier_or(kEpilogueBarrier, 128, !got)) {
        if (!got) give_up(501);
        break;
      }
      tc_fence_after();
      const Item it = read_item(n);
      const float stat = reinterpret_cast<const float*>(base_ptr + kOffStats)[(n & 3) * 128 + row];
      const uint32_t tmem_o = tmem + lane_base + sb * 128;
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
        // sm_scale is a power of two for D = 64, so scaling before or after the rounding is the same: the
        // plain right-factor stage has it folded into P already, the stage with V applies it here
        if (it.kind == kStageRightWithV) scale = g.sm_scale;
      } else if (it.kind == kStageLeft) {
        dst0 = reinterpret_cast<T*>(g.ar) + (((long long)it.hs * g.M + rin) * g.B + it.tile * per + rblk) * kHead;
      } else {
        dst0 = reinterpret_cast<T*>(const_cast<void*>(g.out.ptr)) + (long long)it.e * g.out.se + (long long)it.h * g.out.sh +
               ((long long)rin * g.B + it.tile * per + rblk) * g.out.sn;
      }
      // 64 accumulator columns -> one 128-byte row: both chunk loads in flight, then 4 x 32-byte stores
      // (every touched sector is written whole); the result rows are not read again and leave L2 first
      auto store_row = [&](T* dst, uint32_t taddr, float sc, bool streaming) {
        float o0[32], o1[32];
        tmem_ld32_nowait(taddr, o0);
        tmem_ld32_nowait(taddr + 32, o1);
        tmem_wait_ld(o0);
        tmem_wait_ld(o1);
#pragma unroll
        for (int h8 = 0; h8 < 4; ++h8) {
          const float* p = (h8 < 2 ? o0 : o1) + (h8 & 1) * 16;
          uint32_t w[8];
          if (sc != 1.0f) {
            const float2 scv = make_float2(sc, sc);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float2 t = mul2(make_float2(p[2 * i], p[2 * i + 1]), scv);
              w[i] = pack2<T>(t.x, t.y);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) w[i] = pack2<T>(p[2 * i], p[2 * i + 1]);
          }
          if (streaming) st_global_v8_hint(dst + h8 * 16, w, pol_first);
          else st_global_v8(dst + h8 * 16, w);
        }
      };
      store_row(dst0, tmem_o, scale, it.kind == kStageOutput);
      if (it.kind == kStageRightWithV) {
        store_row(reinterpret_cast<T*>(g.y) + row_y * kHead, tmem_o + kHead, 1.0f, false);
      } else if (it.kind == kStageLeft) {
        float o[32];
        tmem_ld32(tmem_o + kHead, o);
        g.cr[((long long)it.hs * g.M + rin) * g.B + it.tile * per + rblk] = o[0];
      }
      tc_fence_before();
      mbar_arrive(bar(kBarSEmpty + sb));  // the accumulator buffer may take the S of item n + 3
      if (args.wait_deps) {
        // The state tiles this item read (each is written once and read once) are dead: drop their lines
        // from L2 so that they are never written back to HBM and make room at once.  One 128-byte row per
        // thread; a tile is 128 consecutive rows.
        const long long trow = ((long long)it.hs * kTile * tph + (long long)it.tile * kTile + row) * kHead;
        if (it.kind == kStageLeft || it.kind == kStageOutput) {
          l2_discard_line(reinterpret_cast<const T*>(g.al) + trow);
          if (it.kind == kStageOutput) l2_discard_line(reinterpret_cast<const T*>(g.y) + trow);
        } else if (!it.first) {
          l2_discard_line(reinterpret_cast<const T*>(g.ar) + trow);
        }
        // The rows stored above are read by other CTAs with TMA, i.e. through the async proxy: the
        // writer orders its generic-proxy stores before it (a fence on the reading side would make the
        // issuer wait for its own copies in flight, which serialises the loads of consecutive items).
        asm volatile("fence.proxy.async.global;" ::: "memory");
        // hand the item to the publisher (4-deep ring)
        if (!ROLE_WAIT(bar(kBarPubFree + (n & 3)), ((uint32_t)(n >> 2) & 1u) ^ 1u)) give_up(502);
        mbar_arrive(bar(kBarDone + (n & 3)));
      }
    }
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
    // =========================== softmax warps ===========================================
    // All kGroups groups of four warps work on the SAME item: a row's columns are split between the
    // threads `row` of the groups (warps w, w + 4, w + 8, ... reach the same tensor-memory lanes and
    // share a scheduler).  Every warp then runs the same short instruction sequence at the same time,
    // and a scheduler has kGroups of them to hide one another's latencies - with two groups of one
    // thread per row on alternating items, every scheduler had two copies of a four times longer
    // sequence in flight at different places, and the warps spent more time waiting for instructions
    // than issuing them.  Each part of a row is exponentiated against its OWN maximum; the parts then
    // exchange (shift, sum, entropy sum) through shared memory once and rescale.
    const int grp = warp >> 2;
    const int row = (warp & 3) * 32 + lane;         // tensor-memory lane = tile row
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    // With two blocks per tile only the 64-column half that belongs to the row's own block or column
    // means anything (rows are blk*64 + j in the right-factor tiles and jj*64 + l in the column tiles;
    // columns are blk*64 + i, or jj*64 + m); the other half of P is zero.
    const int h0 = per > 1 ? (row >> 6) : 0;    // uniform within a warp
    constexpr int kOwn = 128 / PER;             // columns of the row that mean anything
    constexpr int kMine = kOwn / kGroups;       // columns this thread works on
    static_assert(kMine == 32 || kMine == 16, "tensor-memory access shapes below");
    const int col0 = (per > 1 ? 64 * h0 : 0) + kMine * grp;  // first of them
    float* xch_base = reinterpret_cast<float*>(base_ptr + kOffXch);  // [2][3][kGroups][128]: shift, sum, entropy sum per part
    for (int n = 0; n < n_items; ++n) {
      // by item parity: a fast thread's next item must not overwrite what a slow one still reads
      float* xch = xch_base + (n & 1) * (3 * kGroups * 128);
      const int slot = n % kSlots, sb = n % kSBuffers, pb = n & 1;
      const float* vec = reinterpret_cast<const float*>(base_ptr + kOffVec + slot * 512);
      bool ok = mbar_wait_abortable(bar(kBarInFull + slot), (uint32_t)(n / kSlots) & 1u, abort_flag);
      ok = ok && mbar_wait_abortable(bar(kBarSFull + sb), (uint32_t)(n / kSBuffers) & 1u, abort_flag);
      Item it;
      it.kind = kStageRight; it.first = 1; it.p_dist = 0;
      if (ok) it = read_item(n);
      const bool right = it.kind == kStageRight || it.kind == kStageRightWithV;
      tc_fence_after();
      const uint32_t tmem_s = tmem + lane_base + sb * 128;

      // This thread's columns of S, read once and kept in registers.
      float s[kMine];
      if (ok) {
        if (kMine == 32) {
          tmem_ld32_nowait(tmem_s + col0, *reinterpret_cast<float(*)[32]>(&s[0]));
          tmem_wait_ld(*reinterpret_cast<float(*)[32]>(&s[0]));
        } else {
          tmem_ld16_nowait(tmem_s + col0, *reinterpret_cast<float(*)[16]>(&s[0]));
          tmem_wait_ld16(*reinterpret_cast<float(*)[16]>(&s[0]));
        }
      } else {
#pragma unroll
        for (int i = 0; i < kMine; ++i) s[i] = 0.f;
      }

      // Pass 1: maximum of this part of the row.  Right-factor stages: of S itself (rounding is
      // monotonic, so the maximum of the rounded logits is the rounded maximum).  Left-factor / output
      // stages: the logits round(S) - cl[m] are formed in place first.
      float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
      if (right) {
#pragma unroll
        for (int i = 0; i < kMine; i += 8) {
          m0 = max3(m0, s[i], s[i + 1]);
          m1 = max3(m1, s[i + 2], s[i + 3]);
          m2 = max3(m2, s[i + 4], s[i + 5]);
          m3 = max3(m3, s[i + 6], s[i + 7]);
        }
      } else {
        const float* cl = vec + col0;
#pragma unroll
        for (int i = 0; i < kMine; i += 8) {
          const float4 c0 = *reinterpret_cast<const float4*>(cl + i);
          const float4 c1 = *reinterpret_cast<const float4*>(cl + i + 4);
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
      }
      // With top the shift of the whole row (the largest of the parts': max(max(a, eps), max(b, eps)) =
      // max(max(a, b), eps)) and c = 2^(shift_part - top) <= 1:
      //   e_i = c e'_i,   sum e_i log2 e_i = c (sum e'_i u'_i + log2(c) sum e'_i).
      const float hmax = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
      float my_off, part_sum, part_ent = 0.f;  // my_off: this part's shift in log2 units
      if (right) {
        // x = sm_scale * round(S) / (cr + eps), clamp on the maximum from below
        const float row_scale = g.sm_scale / ((it.first ? 1.0f : vec[row]) + kEps);
        const float mul = row_scale * kLog2e;
        my_off = fmaxf(round_through<T>(hmax) * row_scale, kEps) * kLog2e;
        // Pass 2: e' = 2^(mul * round(S) - off) in place, sum, sum of e' * log2(e')
        const float2 mulv = make_float2(mul, mul), noffv = make_float2(-my_off, -my_off);
        float2 sum_a = make_float2(0.f, 0.f), sum_b = sum_a, ent_a = sum_a, ent_b = sum_a;
#pragma unroll
        for (int i = 0; i < kMine; i += 4) {
          const float2 ua = fma2(round2<T>(make_float2(s[i], s[i + 1])), mulv, noffv);
          const float2 ub = fma2(round2<T>(make_float2(s[i + 2], s[i + 3])), mulv, noffv);
          const float2 ea = make_float2(ex2(ua.x), ex2(ua.y)), eb = make_float2(ex2(ub.x), ex2(ub.y));
          sum_a = add2(sum_a, ea);
          sum_b = add2(sum_b, eb);
          ent_a = fma2(ea, ua, ent_a);
          ent_b = fma2(eb, ub, ent_b);
          s[i] = ea.x; s[i + 1] = ea.y; s[i + 2] = eb.x; s[i + 3] = eb.y;
        }
        part_sum = (sum_a.x + sum_a.y) + (sum_b.x + sum_b.y);
        part_ent = (ent_a.x + ent_a.y) + (ent_b.x + ent_b.y);
      } else {
        my_off = hmax * kLog2e;
        // Pass 2: e' = 2^(log2e * w - off) in place, sum
        const float2 mulv = make_float2(kLog2e, kLog2e), noffv = make_float2(-my_off, -my_off);
        float2 sum_a = make_float2(0.f, 0.f), sum_b = sum_a;
#pragma unroll
        for (int i = 0; i < kMine; i += 4) {
          const float2 ua = fma2(make_float2(s[i], s[i + 1]), mulv, noffv);
          const float2 ub = fma2(make_float2(s[i + 2], s[i + 3]), mulv, noffv);
          const float2 ea = make_float2(ex2(ua.x), ex2(ua.y)), eb = make_float2(ex2(ub.x), ex2(ub.y));
          sum_a = add2(sum_a, ea);
          sum_b = add2(sum_b, eb);
          s[i] = ea.x; s[i + 1] = ea.y; s[i + 2] = eb.x; s[i + 3] = eb.y;
        }
        part_sum = (sum_a.x + sum_a.y) + (sum_b.x + sum_b.y);
      }
      xch[grp * 128 + row] = my_off;
      xch[(kGroups + grp) * 128 + row] = part_sum;
      xch[(2 * kGroups + grp) * 128 + row] = part_ent;
      // the exchange, between the warps that share the rows (they also share a scheduler, so they get here
      // together); also the one place where they agree to leave (a thread that went on or left alone
      // would strand its partners at the barrier)
      if (named_barrier_or(kSoftmaxBarrier + (warp & 3), 32 * kGroups, !ok)) {
        if (!ok) give_up(401);
        break;
      }
      // (all parts evaluate the same expressions on the same numbers, so they get the same bits)
      float offs[kGroups], sums[kGroups];
      float top = -INFINITY;
#pragma unroll
      for (int q = 0; q < kGroups; ++q) {
        offs[q] = xch[q * 128 + row];
        sums[q] = xch[(kGroups + q) * 128 + row];
        top = fmaxf(top, offs[q]);
      }
      float row_sum = 0.f, my_c = 1.f;
#pragma unroll
      for (int q = 0; q < kGroups; ++q) {
        offs[q] -= top;                 // log2 of the part's factor c
        const float c = ex2(offs[q]);
        if (q == grp) my_c = c;
        sums[q] *= c;
        row_sum += sums[q];
      }
      // 1 / sum by the approximate reciprocal (1 ulp; the quotient is rounded to 16 bits right after) - the
      // exact one is a long dependent sequence on the path of every item
      const float denom = right ? row_sum + kEps : row_sum;
      float rden;
      asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rden) : "f"(denom));
      // this part's exponentials were taken against its own shift.  al = sm_scale * (P k): the scale is a
      // power of two (D = 64), so it can ride on P exactly; the stage with V keeps P unscaled (y = P v)
      // and scales the al half in the epilogue
      float inv = rden * my_c;
      if (it.kind == kStageRight) inv *= g.sm_scale;

      const float2 invv = make_float2(inv, inv);
      if (it.kind != kStageLeft) {
        // Pass 3: P = round(e / sum) into the item's P buffer in tensor memory: A operand of the second
        // contraction.  (The buffer is free once the second contraction of item n - 2 has completed - long
        // ago, as a rule.  A wait that runs out is reported and noticed at the next item's barrier.)
        if (!mbar_wait_abortable(bar(kBarPEmpty + pb), ((uint32_t)(n >> 1) & 1u) ^ 1u, abort_flag)) give_up(404);
        tc_fence_after();
        const uint32_t tmem_p = tmem + lane_base + kTmemP + pb * 64;
        uint32_t pk[kMine / 2];
#pragma unroll
        for (int i = 0; i < kMine / 2; ++i) {
          const float2 r = mul2(make_float2(s[2 * i], s[2 * i + 1]), invv);
          pk[i] = pack2<T>(r.x, r.y);
        }
        // cells (two columns each) of this thread's columns; with two blocks per tile, zeros in the
        // matching cells of the other half
        const uint32_t cell0 = (uint32_t)(col0 >> 1);
        if (kMine == 32) {
          tmem_st16(tmem_p + cell0, *reinterpret_cast<uint32_t(*)[16]>(&pk[0]));
        } else {
          tmem_st8(tmem_p + cell0, *reinterpret_cast<uint32_t(*)[8]>(&pk[0]));
          if (per > 1) {
#pragma unroll
            for (int i = 0; i < 8; ++i) pk[i] = 0u;
            tmem_st8(tmem_p + (cell0 ^ 32u), *reinterpret_cast<uint32_t(*)[8]>(&pk[0]));
          }
        }
        tmem_wait_st();
        tc_fence_before();
      } else {
        // P^T goes through shared memory (MN-major A operand): rounded P in the first two tiles of the P
        // region, the rounded remainder P - round(P) in the other two.  Wait until the item that used the
        // region last has completed its second contraction.
        if (it.p_dist > 0) {
          const int m = n - it.p_dist;
          if (!mbar_wait_abortable(bar(kBarInEmpty + m % kSlots), (uint32_t)(m / kSlots) & 1u, abort_flag)) give_up(403);
        }
        const uint32_t sP = base + kOffPreg;
        // 16-byte groups (8 columns) of this thread's columns: 64-column atom and group within it
        const uint32_t atom = (uint32_t)col0 >> 6, g0 = ((uint32_t)col0 & 63u) >> 3;
#pragma unroll
        for (int c8 = 0; c8 < kMine / 8; ++c8) {
          uint32_t hi[4], lo[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 r = mul2(make_float2(s[8 * c8 + 2 * i], s[8 * c8 + 2 * i + 1]), invv);
            hi[i] = pack2<T>(r.x, r.y);
            const float2 d = sub2(r, widen2<T>(hi[i]));
            lo[i] = pack2<T>(d.x, d.y);
          }
          const uint32_t off = atom * kTileBytes + swz(row, g0 + c8);
          st_shared_v4(sP + off, hi[0], hi[1], hi[2], hi[3]);
          st_shared_v4(sP + 2 * kTileBytes + off, lo[0], lo[1], lo[2], lo[3]);
        }
        if (per > 1) {
#pragma unroll
          for (int c8 = 0; c8 < kMine / 8; ++c8) {
            const uint32_t off = (atom ^ 1u) * kTileBytes + swz(row, g0 + c8);
            st_shared_v4(sP + off, 0u, 0u, 0u, 0u);
            st_shared_v4(sP + 2 * kTileBytes + off, 0u, 0u, 0u, 0u);
          }
        }
        fence_async_smem();
      }
      mbar_arrive(bar(kBarPFull + pb));
      // cl of the row for the epilogue group, off the path to P: sum_i r_i ln r_i with r_i = e_i / denom and
      // ln e_i = ln2 * u_i.  The 4-deep ring cannot be overrun: the first contraction of item n+4 needs the
      // accumulator buffer of item n+1 back from the epilogue, which takes the items in order.
      if (grp == 0) {
        if (right) {
          float row_ent = 0.f;
#pragma unroll
          for (int q = 0; q < kGroups; ++q) {
            // sums[q] = c s', offs[q] = log2 c:  c (E' + log2(c) s') = c E' + log2(c) (c s')
            const float c = ex2(offs[q]);
            row_ent += c * xch[(2 * kGroups + q) * 128 + row] + offs[q] * sums[q];
          }
          reinterpret_cast<float*>(base_ptr + kOffStats)[(n & 3) * 128 + row] = (kLn2 * row_ent - __logf(denom) * row_sum) * rden;
        }
        mbar_arrive(bar(kBarStat + (n & 3)));
      }
    }
  }

  // ---- teardown ------------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == kMma1Warp) {
    __syncwarp();
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
      cudaFuncAttributes fa;
      e = cudaFuncGetAttributes(&fa, fn);
      if (e != cudaSuccess) return e;
      // a build whose launch allocation cannot cover the roles' requests must not start: setmaxnreg would block
      // (and the decreases must really be decreases, the increase an increase)
      if (fa.numRegs * kThreads < kRegPool || fa.numRegs < kRegsSoftmax || fa.numRegs < kRegsSingle || fa.numRegs > kRegsEpilogue)
        return cudaErrorLaunchOutOfResources;
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
