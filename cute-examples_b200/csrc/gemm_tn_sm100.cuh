// Persistent, warp-specialised TN GEMM for sm_100a:
//   C[M,N] = A[M,K] * B[N,K]^T, 16-bit inputs (bf16 or fp16), fp32 accumulation in
//   tensor memory, same-dtype output rounded to nearest even.
//
// It replaces the reference's Hopper kernel test::gemm_kernel
// (kernels/gemm_kernels/sm90a/gemm.cuh:246-418, 452-462): same math and the same
// "both operands K-major" layout contract, but none of its structure.  Roles per CTA
// (64 + 32 x kEpiWarps threads):
//   warp 0      TMA producer   : global -> smem ring of kStages (A tile + B tile(s)), mbarrier tx-count
//   warp 1      MMA issuer     : tcgen05.mma from smem descriptors into TMEM; tcgen05.commit frees
//                                 ring slots and publishes finished accumulators
//   warps 2..   epilogue       : tcgen05.ld TMEM -> registers -> 16-bit -> swizzled smem -> TMA store
// Warps 0 and 1 run their loops with all 32 lanes and warp-uniform waits; one elected lane
// issues.  (TMA and MMA instructions take uniform-register operands: a loop run by a single
// diverged lane pays a register move per operand and was measured at 0.74 of the tensor rate.)
//
// Two accumulator slots live in TMEM (2 x kMmaN fp32 columns).  Either consecutive tiles
// alternate between them, so the epilogue of tile i runs under the mainloop of tile i+1
// (the reference's single register-resident accumulator idles the tensor pipe during every
// epilogue, gemm.cuh:368-395), or one double-width tile owns both (see GemmConfig).
//
// kCtaGroup == 2 pairs two CTAs (a 2-CTA cluster) on one 256 x kBlockN tile: each CTA
// loads its own 128 rows of A and its own share of the B rows with plain TMA loads, and
// the leader CTA issues cta_group::2 MMAs that read both CTAs' shared memory.  This gives
// the operand sharing that the reference gets from a cluster-broadcast load of B
// (gemm_test.cu:60-64) without any broadcast load.
//
// Work is handed out as segments (WorkIter): whole tiles in a static persistent order, or, for
// the K-split schedule, equal runs of K blocks with fp32 partial tiles for the tiles a run
// boundary cuts.  The finished tile can be stored through several output tensor maps
// (gemm_tn_fanout_kernel): that is how the column-sharded multi-GPU GEMM writes every GPU's C.
//
// The columns of a tile row need not be cut into equal tiles: tile widths are launch parameters in
// steps of 64 columns (TileParams::bal_*), so the host can give a tile row the number of tiles that
// fills the SMs evenly; the MMA's N, the B rows loaded and the epilogue's chunk count follow.
//
// Launch overlap: the kernel lets the next kernel of the stream be scheduled as soon as it starts
// (griddepcontrol.launch_dependents), and itself waits for the previous kernel
// (griddepcontrol.wait) only after its set-up, before its first access to global memory.
//
// Every wait is bounded: when one runs out the CTA (and its pair peer) is flagged, all roles
// fall through to the common tear-down, TMEM is released and the launcher reports the status
// word.  The reference's waits are unbounded (gemm.cuh:75-78, 91-94).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ptx_sm100.cuh"

namespace gemm_sm100 {

using namespace sm100;

// Device status codes (first failure wins); 0 means success.
enum : uint32_t {
  kStatusOk = 0,
  kStatusTimeoutProducer = 0x100,   // + barrier stage
  kStatusTimeoutMma = 0x200,
  kStatusTimeoutMmaAcc = 0x300,
  kStatusTimeoutEpilogue = 0x400,
  kStatusTimeoutPartial = 0x500,    // a split tile's partial sums never arrived
};

struct TileParams {
  int M, N, K;
  int m_tiles;   // ceil(M / (128 * kCtaGroup))
  int n_tiles;   // ceil(N / kBlockN)
  int k_blocks;  // ceil(K / 64)
  int group_m;   // tiles along M per rasterisation group
  // Column tiling.  The N / 64 chunks of 64 columns are dealt to the n_tiles tiles of a tile row:
  // every tile covers bal_q chunks, the bal_rem tiles from index bal_start on one more.
  // Uniform tiles of kBlockN columns are bal_q = kBlockN / 64, bal_rem = 0 (the last tile hangs
  // over the edge: loads are zero-filled, stores clipped).  A balanced tiling gives the tile row
  // the number of tiles that fills the SMs evenly and makes the tiles as wide as that allows,
  // e.g. 4096 columns as 8 x 448 + 1 x 512 instead of 8 x 512.  Widths are at most kBlockN and,
  // for double-width configurations, more than kMmaN (both halves non-empty).
  int bal_q, bal_rem, bal_start;
  int b_box_rows;  // rows per TMA box of B: kBRows for uniform tiles, 64 / kCtaGroup for balanced ones
  // > 0: before waiting for the previous kernel of the stream (programmatic dependent launch), the
  // producer asks L2 for the operand boxes of its first two stages.  A prefetch is only a hint
  // and L2 is where this GPU's writes become visible, so it is safe whatever that kernel still
  // writes; it puts the DRAM reads of this launch's first stages under that kernel's tail.
  int early_prefetch;
  unsigned int* status;            // device word, 0 = ok
  unsigned long long timeout_ns;   // bound of every device-side wait
  unsigned long long* trace;       // optional: kTraceWords counters per CTA (nullptr = off)
  unsigned int debug_flags;        // experiments only; 0 in normal use (see kDebug*)
  // K-split schedule only: one arrival counter and one fp32 partial tile per CTA of the grid.
  unsigned int* sk_flags;          // zeroed before the launch
  float* sk_partials;              // grid x (sk_rows x kBlockN) floats
  int sk_rows;                     // rows kept per partial tile: 128, or M rounded up to 32 when M < 128
  int sk_factor;                   // <= 1: contiguous ranges; > 1: every tile cut into this many equal K ranges
                                   // (then one partial tile per unit and CTA of the pair, one counter per tile and CTA)
  // > 0 (even split with sk_factor 2 or 4, launched in clusters of sk_factor CTA (pair)s, one unit
  // per CTA (pair)): the contributors of a tile sit in one cluster and exchange their partial sums
  // through distributed shared memory instead of the workspace, which is then not used at all.
  int sk_cluster;
  // Order in which a tile's K blocks are loaded (the sum does not depend on it beyond rounding):
  // 0 ascending.  1 ("rotate"): every tile starts at a different K block and wraps around, so CTAs
  // that each stream their own B tile hit different column offsets at any moment.  2
  // ("serpentine"): every other tile of a CTA runs K backwards, so the operand panel that
  // consecutive tiles of the rasterisation share is re-read most-recently-loaded first, while
  // its tail end is still in L2.
  int k_rotate;
  // Optional epilogue scaling (kernels instantiated with kScaled only): C = alpha * acc + beta * C.
  float alpha, beta;
  void* c_ptr;                     // C as the caller passed it: read when beta != 0, and written with
  long long ldc;                   // plain stores in its last N % 8 columns; row pitch in elements
};

// Experiment switches (results are garbage with any of them set).
enum : unsigned int {
  kDebugSkipLoads = 1u,   // no TMA loads, MMA does not wait for operands: pure MMA issue/execute rate
  kDebugSkipStores = 2u,  // epilogue reads TMEM but stores nothing
  kDebugSkipMma = 4u,     // operands are loaded and released, no MMA is issued: pure load rate
};

// Per-CTA trace record (cycles are clock64 of the CTA's SM).
enum : int {
  kTraceEntry = 0,        // kernel entry
  kTraceSetupDone = 1,    // barriers initialised, TMEM allocated
  kTraceMmaFirst = 2,     // first operand stage landed
  kTraceMmaStallFull = 3, // cycles the MMA thread waited for operand stages
  kTraceMmaStallAcc = 4,  // cycles the MMA thread waited for a free accumulator
  kTraceMmaEnd = 5,       // last MMA issued
  kTraceProdStall = 6,    // cycles the producer waited for free ring slots
  kTraceProdEnd = 7,      // last load issued
  kTraceEpiStall = 8,     // cycles epilogue warp 2 waited for accumulators
  kTraceEpiEnd = 9,       // epilogue warp 2 done
  kTraceExit = 10,        // after tear-down barrier
  kTraceTiles = 11,       // tiles this CTA processed
  kTraceTimeEntryNs = 12, // %globaltimer at entry
  kTraceTimeExitNs = 13,  // %globaltimer at exit
  kTraceRxReady = 14,     // cluster K-split: every contributor's ring is idle (epilogue warp 2)
  kTraceRxDone = 15,      // cluster K-split: every contributor's partial sums have arrived (epilogue warp 2)
  kTraceWords = 16,
};

template <int kCtaGroup_, int kMmaN_, int kHalves_, int kStages_, int kEpiWarps_, bool kIsBf16_, int kARows_ = 128,
          int kEpiBufs_ = 0, int kKSub_ = 1>
struct GemmConfig {
  static constexpr int kCtaGroup = kCtaGroup_;
  static constexpr int kBlockM = 128;              // rows of the accumulator (and of the MMA's A operand) per CTA
  // Rows of A that are actually loaded per stage.  Less than 128 only in the configurations for
  // problems of at most that many rows (M <= kARows): the MMA still reads a 128-row operand from
  // the stage's address, and what lies behind the loaded rows (later stages of the ring) is
  // multiplied into accumulator rows >= M, which nothing ever reads.  The shared memory saved
  // goes into more stages: for the memory-bound few-row shapes, more of B in flight per SM.
  static constexpr int kARows = kARows_;
  static constexpr int kMmaN = kMmaN_;             // N of one MMA instruction (whole pair)
  // kHalves == 1: the tile is kMmaN wide and the two accumulator slots in TMEM alternate
  //               between consecutive tiles (the epilogue of one runs under the next mainloop).
  // kHalves == 2: the tile is 2 x kMmaN wide and occupies both slots; every A stage feeds two
  //               MMAs, so shared memory receives 25 % fewer bytes per flop, at the price of
  //               an epilogue that is only partly hidden.
  static constexpr int kHalves = kHalves_;
  static constexpr int kBlockN = kMmaN * kHalves;  // columns of C per tile (whole pair)
  // K elements per stage: kKSub blocks of 64 (64 x 16 bit = one 128-byte swizzle row).  With two, a
  // stage's operand tiles are each loaded by ONE TMA instruction (a 3-D box: 64 elements x rows x 2 K
  // blocks, landing as two ordinary K-major tiles one after the other): an SM's TMA takes about 130
  // cycles per instruction on top of 7 cycles per KB, so tiles whose boxes are small (the 256 x 128
  // pair tile: 16 KB + 8 KB per K block) load 1.5x as many bytes per clock that way.
  static constexpr int kKSub = kKSub_;
  static constexpr int kBlockK = 64 * kKSub;
  static constexpr int kStages = kStages_;
  static constexpr int kEpiWarps = kEpiWarps_;     // 4 or 8
  static constexpr bool kIsBf16 = kIsBf16_;
  static constexpr int kUmmaK = 16;
  static constexpr int kBRows = kMmaN / kCtaGroup;              // rows of B this CTA loads per half
  static constexpr int kABytes = kARows * kBlockK * 2;
  static constexpr int kBHalfBytes = kBRows * kBlockK * 2;
  static constexpr int kBBytes = kHalves * kBHalfBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kEpiCols = 64;                           // columns per TMA-store chunk
  static constexpr int kEpiWarpBuf = 32 * kEpiCols * 2;         // one warp, one chunk: 4 KiB
  static constexpr int kEpiBufs = kEpiBufs_ > 0 ? kEpiBufs_ : 8 / kEpiWarps;   // staging buffers per warp
  static constexpr int kEpiBytes = kEpiWarps * kEpiBufs * kEpiWarpBuf;   // 32 KiB
  // Two accumulator slots.  TMEM is allocated in powers of two (32..512 columns); the slots sit
  // half an allocation apart, so a 192-column accumulator leaves 64 unused columns behind it.
  static constexpr int kTmemCols = 2 * kMmaN <= 128 ? 128 : (2 * kMmaN <= 256 ? 256 : 512);
  static constexpr int kSlotCols = kTmemCols / 2;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kEpiBytes + kBarrierBytes;
  static constexpr int kThreads = 64 + 32 * kEpiWarps;
  static_assert(kKSub == 1 || kKSub == 2 || kKSub == 4, "K blocks per stage");
  static_assert(kHalves == 1 || kHalves == 2, "halves");
  static_assert(kEpiWarps == 4 || kEpiWarps == 8, "epilogue warps");
  static_assert(kMmaN % 64 == 0 && kMmaN >= 64 && kMmaN <= 256, "MMA N");
  static_assert(kMmaN <= kSlotCols, "an accumulator must fit its slot");
  static_assert(kCtaGroup == 1 || kMmaN % 32 == 0, "pair MMA: each CTA supplies N / 2 rows of B, a multiple of 16");
  static_assert(kBHalfBytes % 1024 == 0, "B tile must keep 1024-byte swizzle alignment");
  static_assert(kARows % 8 == 0 && kARows >= 8 && kARows <= kBlockM, "A rows: whole 8-row swizzle groups");
  static_assert(kARows == kBlockM || kCtaGroup == 1, "short A tiles: single-CTA configurations only");
  static_assert(kEpiBufs == 1 || kEpiBufs == 2, "staging buffers per epilogue warp");
  // the MMA reads 128 rows from every A stage: the last stage's read must stay inside the ring
  static_assert(kStages * kABytes + kBlockM * kBlockK * 2 - kABytes <= kStages * kStageBytes, "A over-read leaves the ring");
  static_assert(kSmemBytes <= 232448, "shared memory budget");
};

// A run of consecutive K blocks of one output tile.
struct Segment {
  int tile, kb0, kb1;
  int part;   // even split only: which of the tile's `factor` equal K ranges this is
};

// What one CTA (pair) works on, as a sequence of segments.
//  kSplitK == false: whole tiles `first, first + step, ...` (static persistent schedule).
//  kSplitK == true : the flattened (tile, K block) space is cut into equal contiguous ranges,
//    one per CTA (pair), so every SM streams the same number of K blocks whatever the tile
//    count; a tile cut by a range boundary is summed by the owner of its first K block from
//    fp32 partial tiles the other owners leave in global memory.
//  kSplitK == true with factor > 1 ("even split", single-width tiles): every tile is cut into
//    `factor` equal K ranges, range j of tile t is unit t * factor + j, units go round-robin over
//    the CTA (pair)s; every contributor writes an fp32 partial tile and then, once the tile's
//    arrival counter is full, reduces and stores its own share of the tile, so the reduction is
//    spread over the contributors instead of falling to one owner.
template <bool kSplitK>
struct WorkIter {
  int tile, step, num_tiles, k_blocks, factor;
  long long u, u_end;

  __device__ __forceinline__ static long long range_start(int cluster, int clusters, long long units) {
    return (long long)cluster * units / clusters;
  }
  __device__ __forceinline__ WorkIter(int cluster, int clusters, int num_tiles_, int k_blocks_, int factor_ = 0)
      : tile(cluster), step(clusters), num_tiles(num_tiles_), k_blocks(k_blocks_), factor(factor_) {
    const long long units = (long long)num_tiles_ * k_blocks_;
    u = range_start(cluster, clusters, units);
    u_end = range_start(cluster + 1, clusters, units);
  }
  __device__ __forceinline__ bool next(Segment& s) {
    if constexpr (!kSplitK) {
      if (tile >= num_tiles) return false;
      s.tile = tile;
      s.kb0 = 0;
      s.kb1 = k_blocks;
      tile += step;
      return true;
    } else {
      if (factor > 1) {
        // even split: `tile` walks the units
        if (tile >= num_tiles * factor) return false;
        const int t_ = tile / factor, j_ = tile - t_ * factor;
        s.tile = __reduce_max_sync(0xffffffffu, t_);
        s.part = __reduce_max_sync(0xffffffffu, j_);
        s.kb0 = __reduce_max_sync(0xffffffffu, (int)((long long)j_ * k_blocks / factor));
        s.kb1 = __reduce_max_sync(0xffffffffu, (int)((long long)(j_ + 1) * k_blocks / factor));
        tile += step;
        return true;
      }
      if (u >= u_end) return false;
      int tile_ = (int)(u / k_blocks);
      int kb0_ = (int)(u - (long long)tile_ * k_blocks);
      const long long left = u_end - u;
      int kb1_ = (left < (long long)(k_blocks - kb0_)) ? kb0_ + (int)left : k_blocks;
      // Every lane holds the same values, but they come out of a 64-bit division in the vector
      // datapath; a warp reduction hands them back as warp-uniform values, which the loops built
      // on them (barrier waits, TMA and MMA issue) need to stay in uniform registers.
      s.tile = __reduce_max_sync(0xffffffffu, tile_);
      s.kb0 = __reduce_max_sync(0xffffffffu, kb0_);
      s.kb1 = __reduce_max_sync(0xffffffffu, kb1_);
      u += s.kb1 - s.kb0;
      return true;
    }
  }
};

struct WaitCtx {
  volatile uint32_t* abort_flag;   // this CTA's flag in shared memory
  uint32_t peer_abort_addr;        // shared::cluster address of the pair peer's flag (or own)
  unsigned int* status;
  unsigned long long timeout_ns;
};

// Every wait below is executed by a whole, converged warp and returns a warp-uniform result:
// the single-issuer roles keep all their values in uniform registers that way (TMA and MMA
// instructions take uniform operands; a loop run by one diverged lane pays a register move
// per operand).
//
// Cold path of a bounded mbarrier wait: polls until the phase completes, the CTA is flagged,
// or the time limit passes (then flags this CTA and its pair peer and records `code`).
__device__ __noinline__ bool wait_slow(uint32_t bar, uint32_t parity, const WaitCtx& ctx, uint32_t code) {
  bool done = false;
  // try_wait suspends the thread for a hardware-defined while; normal waits end inside this
  // first batch, without a read of the (slow) global timer.
  if (__all_sync(0xffffffffu, mbar_wait_spin(bar, parity, 1024))) return true;
  const uint64_t t0 = global_timer_ns();
#pragma unroll 1
  while (true) {
    done = __all_sync(0xffffffffu, mbar_wait_spin(bar, parity, 64));
    if (done) return true;
    const bool flagged = *ctx.abort_flag != 0;
    const bool late = global_timer_ns() - t0 > ctx.timeout_ns;
    if (__any_sync(0xffffffffu, flagged || late)) {
      if (!flagged) {
        *ctx.abort_flag = 1;
        st_cluster_u32(ctx.peer_abort_addr, 1);
        atomicCAS(ctx.status, 0u, code);
      }
      return false;
    }
  }
}

// Bounded mbarrier wait (whole warp).  Returns false if the CTA was flagged or the wait ran out.
__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity, const WaitCtx& ctx,
                                             uint32_t code) {
  if (__all_sync(0xffffffffu, mbar_wait_spin(bar, parity, 8))) return true;
  return wait_slow(bar, parity, ctx, code);
}

// Bounded wait (whole warp) until a global arrival counter reaches `want`.  Arrivals are counted in
// the low 16 bits; the high bits count the warps that are done with the partial tiles (see the even
// K-split below).
__device__ __noinline__ bool wait_counter(const unsigned int* counter, unsigned int want, const WaitCtx& ctx,
                                          uint32_t code) {
  const volatile unsigned int* c = counter;
  uint64_t t0 = 0;
#pragma unroll 1
  for (unsigned int spin = 0;; ++spin) {
    if (__all_sync(0xffffffffu, (*c & 0xffffu) >= want)) {
      __threadfence();   // acquire: the partial sums written before the arrivals are visible now
      return true;
    }
    __nanosleep(100);
    if ((spin & 255u) == 255u) {
      if (t0 == 0) t0 = global_timer_ns();
      const bool flagged = *ctx.abort_flag != 0;
      const bool late = global_timer_ns() - t0 > ctx.timeout_ns;
      if (__any_sync(0xffffffffu, flagged || late)) {
        if (!flagged) {
          *ctx.abort_flag = 1;
          st_cluster_u32(ctx.peer_abort_addr, 1);
          atomicCAS(ctx.status, 0u, code);
        }
        return false;
      }
    }
  }
}

__device__ __forceinline__ void tile_coords(int tile, const TileParams& p, int& m_tile, int& n_tile) {
  // Groups of `group_m` tile-rows; inside a group M runs fastest, so the CTAs working at
  // the same time share few distinct A and B panels (L2 reuse).
  const int per_group = p.group_m * p.n_tiles;
  const int group = tile / per_group;
  const int in_group = tile - group * per_group;
  const int first_m = group * p.group_m;
  const int rows = min(p.group_m, p.m_tiles - first_m);
  m_tile = first_m + in_group % rows;
  n_tile = in_group / rows;
}

// Columns of tile `n_tile` of a tile row: first column, width of the first accumulator half and of
// the second one (0 for single-width configurations).
struct TileCols {
  int col0, w0, w1;
};
template <class Cfg>
__device__ __forceinline__ TileCols tile_columns(int n_tile, const TileParams& p) {
  const int d = n_tile - p.bal_start;                      // wide tiles: d in [0, bal_rem)
  const bool wide = d >= 0 && d < p.bal_rem;
  const int wide_before = d <= 0 ? 0 : (d < p.bal_rem ? d : p.bal_rem);
  const int width = (p.bal_q + (wide ? 1 : 0)) * Cfg::kEpiCols;
  TileCols t;
  t.col0 = (n_tile * p.bal_q + wide_before) * Cfg::kEpiCols;
  t.w0 = (Cfg::kHalves == 1 || width < Cfg::kMmaN) ? width : Cfg::kMmaN;
  t.w1 = width - t.w0;
  return t;
}

template <bool kIsBf16>
__device__ __forceinline__ uint32_t pack2(uint32_t lo_bits, uint32_t hi_bits) {
  const float lo = __uint_as_float(lo_bits), hi = __uint_as_float(hi_bits);
  if constexpr (kIsBf16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

// kDebug compiles the per-role trace counters and the experiment switches in; the product
// instantiation (kDebug == false) carries none of it in its loops.
//
// `tmap_c` points at `num_c` tensor maps of the output: the finished tile is stored through
// every one of them (one for the plain GEMM; the column-sharded multi-GPU path passes one map
// per GPU, each describing this rank's column slab inside that GPU's C, so the all-gather of C
// happens in the epilogue as TMA stores over NVLink).
//
// kBIsKN: B is given as [K, N] (N contiguous, the "NN" product A * B) instead of [N, K].  Only the
// B loads and the B descriptors change: a stage then holds B as 64-column blocks of 64 K rows
// (one TMA box each), described to the tensor core as an MN-major operand.
// kAIsKM: likewise A given as [K, M] (M contiguous), i.e. the product A^T * B.
// kScaled: the epilogue applies alpha and beta (the reference has neither: gemm.cuh:368-377 only
// converts the accumulator).
template <class Cfg, bool kDebug, bool kSplitK, bool kBIsKN = false, bool kAIsKM = false, bool kScaled = false>
__device__ __forceinline__ void gemm_tn_body(const CUtensorMap& tmap_a, const CUtensorMap& tmap_b,
                                             const CUtensorMap* tmap_c, const int num_c, const TileParams& p) {
  constexpr int G = Cfg::kCtaGroup;
  constexpr int kStages = Cfg::kStages;
  static_assert(!kBIsKN || Cfg::kBRows % 64 == 0, "B[K,N] tiles are loaded in blocks of 64 columns");
  unsigned long long* trace = nullptr;
  unsigned int dbg = 0;
  if constexpr (kDebug) {
    trace = p.trace ? p.trace + (size_t)blockIdx.x * kTraceWords : nullptr;
    dbg = p.debug_flags;
    if (trace && threadIdx.x == 0) {
      trace[kTraceEntry] = clock64();
      trace[kTraceTimeEntryNs] = global_timer_ns();
    }
  }

  // The next kernel in the stream (if it was launched for it) may be scheduled from now on: its
  // CTAs take the SMs this grid leaves idle or frees, set themselves up and wait below.
  grid_launch_dependents();

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;          // 128B-swizzle atoms need 1024 B
  uint8_t* smem = smem_raw + (base - raw_addr);

  const uint32_t smem_a = base;
  const uint32_t smem_b = base + kStages * Cfg::kABytes;
  const uint32_t smem_epi = smem_b + kStages * Cfg::kBBytes;
  uint8_t* bar_mem = smem + kStages * Cfg::kStageBytes + Cfg::kEpiBytes;
  // barrier block: full[kStages], empty[kStages], tfull[2], tempty[2], tmem_ready, then two words
  const uint32_t bar_base = smem_u32(bar_mem);
  constexpr uint32_t kFullOff = 0, kEmptyOff = 8u * kStages, kTFullOff = 16u * kStages,
                     kTEmptyOff = 16u * kStages + 16u, kTmemReadyOff = 16u * kStages + 32u;
  // cluster K-split: "every contributor's operand ring is idle" and "every contributor's partial sums are here"
  constexpr uint32_t kRxReadyOff = Cfg::kBarrierBytes - 16, kRxDoneOff = Cfg::kBarrierBytes - 8;
  static_assert(8 * (2 * kStages + 5) + 8 <= Cfg::kBarrierBytes - 16, "barrier block too small");
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_mem + 8 * (2 * kStages + 5));
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const uint32_t lane = lane_id();
  // A pair is two CTAs of the cluster whose ranks differ in the last bit.  Clusters are pairs,
  // except for the cluster K-split, where a cluster holds all contributors of a tile.
  const uint32_t cluster_rank = cluster_ctarank();
  const uint32_t cta_rank = (G == 2) ? (cluster_rank & 1u) : 0u;
  const uint32_t pair_base = cluster_rank - cta_rank;        // cluster rank of this pair's leader
  const bool is_leader = cta_rank == 0;
  const bool cluster_split = kSplitK && Cfg::kHalves == 1 && p.sk_cluster > 0;

  WaitCtx ctx;
  ctx.abort_flag = abort_flag;
  ctx.peer_abort_addr = (G == 2) ? map_to_cta(smem_u32((const void*)abort_flag), pair_base + (cta_rank ^ 1u))
                                 : smem_u32((const void*)abort_flag);
  ctx.status = p.status;
  ctx.timeout_ns = p.timeout_ns;

  if (threadIdx.x < 32) {
    if (threadIdx.x == 0) {
      *abort_flag = 0;
      prefetch_tensormap(&tmap_a);
      prefetch_tensormap(&tmap_b);
      for (int d = 0; d < num_c; ++d) prefetch_tensormap(tmap_c + d);
      if constexpr (kSplitK) {
        // every epilogue warp of every contributor to this CTA's rows arrives once on each
        const uint32_t arrivals = (uint32_t)(Cfg::kEpiWarps * (p.sk_cluster > 0 ? p.sk_factor : 1));
        mbar_init(bar_base + kRxReadyOff, arrivals);
        // the other contributors' copies into this CTA's receive area are counted in bytes
        mbar_init(bar_base + kRxDoneOff, 1);
      }
    }
    // One barrier per lane (they sit 8 bytes apart in the order full[], empty[], tfull[2], tempty[2],
    // tmem_ready).  full: the leader's producer arrives once and posts the byte count; empty and
    // tfull: one tcgen05.commit per use; tempty: every epilogue warp of the pair arrives once;
    // tmem_ready (pair mode): the peer's TMEM allocation is done.
    for (uint32_t b = threadIdx.x; b < 2u * kStages + 5u; b += 32u)
      mbar_init(bar_base + 8u * b, (b == 2u * kStages + 2u || b == 2u * kStages + 3u) ? Cfg::kEpiWarps * G : 1);
    fence_mbar_init();
    if constexpr (kSplitK) {
      if (threadIdx.x == 0 && p.sk_cluster > 0) {
        // What the other contributors will send: for every epilogue warp whose 32 rows exist (rows
        // past M are not exchanged), the chunks of this CTA's share, 8 KB each.
        // More contributors than 64-column chunks (four for a 128-column tile): a share is one chunk
        // of one half of the rows, so only the warps of that half send to this CTA.
        constexpr int kTileChunks = Cfg::kBlockN / 64;
        const int unit = (int)(blockIdx.x / G);
        int m_tile, n_tile;
        tile_coords(unit / p.sk_factor, p, m_tile, n_tile);
        const int rows = p.M - (m_tile * G + (int)cta_rank) * Cfg::kBlockM;
        const int row_groups = p.sk_factor > kTileChunks ? p.sk_factor / kTileChunks : 1;
        const int warps = 4 / row_groups;                       // epilogue warps (32 rows each) per share
        const int first_row = ((unit % p.sk_factor) % row_groups) * warps * 32;
        const int mine = rows - first_row;                      // rows of this CTA's share that exist
        const int live_warps = mine <= 0 ? 0 : (mine >= warps * 32 ? warps : (mine + 31) / 32);
        const int chunks = row_groups > 1 ? 1 : kTileChunks / p.sk_factor;
        mbar_arrive_expect_tx(bar_base + kRxDoneOff, (uint32_t)(live_warps * (p.sk_factor - 1) * chunks * 8192));
      }
    }
  }
  // Barriers are initialised: let the producer go.  The TMEM allocation (slow for a CTA pair)
  // happens after this point, off the path of the first operand loads.
  __syncthreads();
  if (G == 2 || cluster_split) {
    cluster_arrive();
    cluster_wait();
  }
  if constexpr (kDebug)
    if (trace && threadIdx.x == 0) trace[kTraceSetupDone] = clock64();
  uint32_t tmem_base = 0;
  if (warp >= 1) {
    // TMEM address hand-over between the allocating warp and the epilogue warps only.
    if (warp == 1) {
      tmem_alloc<G>(smem_u32(tmem_slot), Cfg::kTmemCols);
      tmem_relinquish<G>();
      tc_fence_before_sync();
    }
    named_barrier_sync(1, Cfg::kThreads - 32);
    tc_fence_after_sync();
    tmem_base = *tmem_slot;
    if constexpr (G == 2) {
      // The leader's MMAs write both CTAs' TMEM: it must know the peer's allocation is done.
      if (warp == 1 && !is_leader && lane == 0) mbar_arrive_cluster(map_to_cta(bar_base + kTmemReadyOff, pair_base));
    }
  }

  const int num_tiles = p.m_tiles * p.n_tiles;
  const int cluster_id = blockIdx.x / G;
  const int num_clusters = gridDim.x / G;
  const int k_blocks = p.k_blocks;
  const int sk_factor = (kSplitK && Cfg::kHalves == 1) ? p.sk_factor : 0;   // even split: single-width tiles only

  if constexpr (!kSplitK && !kBIsKN && !kAIsKM && Cfg::kKSub == 1) {
    if (warp == 0 && p.early_prefetch > 0 && cluster_id < num_tiles) {
      // L2 prefetch of the first tile's first kStages K blocks (the boxes the producer loads first)
      if (elect_one()) {
        int m_tile, n_tile;
        tile_coords(cluster_id, p, m_tile, n_tile);
        const TileCols tc = tile_columns<Cfg>(n_tile, p);
        const int row_a = (m_tile * G + (int)cta_rank) * Cfg::kBlockM;
        const int rot = p.k_rotate == 1 ? (int)(((long long)cluster_id * k_blocks) / num_tiles) : 0;
        // two stages' worth: every prefetch is a TMA instruction of its own (about 130 cycles each), and
        // they sit in front of the first loads when there is no previous kernel to hide them under
        const int stages = k_blocks < 2 ? k_blocks : 2;
        for (int kb = 0; kb < stages; ++kb) {
          int kb_phys = kb + rot;
          if (kb_phys >= k_blocks) kb_phys -= k_blocks;
          const int x = kb_phys * Cfg::kBlockK;
          if (row_a < p.M) tma_prefetch_2d(&tmap_a, x, row_a);
#pragma unroll
          for (int h = 0; h < Cfg::kHalves; ++h) {
            const int rows = (h ? tc.w1 : tc.w0) / G;
            const int row0 = tc.col0 + (h ? tc.w0 : 0) + (int)cta_rank * rows;
            for (int j = 0; j < rows; j += p.b_box_rows)
              if (row0 + j < p.N) tma_prefetch_2d(&tmap_b, x, row0 + j);
          }
        }
      }
      __syncwarp();
    }
  }

  // Everything up to here used only this CTA's own resources (and hints to L2).  Global memory
  // (operands that the previous kernel in the stream may have written, C that it may still be
  // writing) comes next.
  grid_dependency_wait();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    // The whole warp runs the loop, one elected lane issues.  The loop is flattened over
    // (tile, k-block) and unrolled over the ring so that every barrier and shared-memory
    // address is the ring base plus a constant.
    if (!(kDebug && (dbg & kDebugSkipLoads))) {
      const bool issuer = elect_one();
      const uint64_t pol = policy_evict_normal();
      // Both CTAs of a pair complete their bytes on the LEADER's barrier: the leader's MMA
      // thread is the only consumer of the ring.
      const uint32_t full_leader = (G == 2) ? map_to_cta(bar_base + kFullOff, pair_base) : bar_base + kFullOff;
      uint32_t phase = 0;
      WorkIter<kSplitK> work(cluster_id, num_clusters, num_tiles, k_blocks, sk_factor);
      Segment seg;
      bool have = work.next(seg);
      int kb = seg.kb0, row_a = 0, rot = 0, tiles_done = 0;
      int row_b[2] = {0, 0}, rows_b[2] = {0, 0};          // this CTA's first row and row count of B per half
      uint32_t tx_bytes = 0;
      const int b_box = p.b_box_rows;
      bool seg_start = true, backwards = false;
      bool ok = true;
      long long stall = 0;
      while (have && ok) {
#pragma unroll
        for (int s = 0; s < kStages; ++s) {
          if (!have) break;
          if (seg_start) {
            int m_tile, n_tile;
            tile_coords(seg.tile, p, m_tile, n_tile);
            row_a = (m_tile * G + (int)cta_rank) * Cfg::kBlockM;
            const TileCols tc = tile_columns<Cfg>(n_tile, p);
            rows_b[0] = tc.w0 / G;
            rows_b[1] = tc.w1 / G;
            row_b[0] = tc.col0 + (int)cta_rank * rows_b[0];
            row_b[1] = tc.col0 + tc.w0 + (int)cta_rank * rows_b[1];
            tx_bytes = (uint32_t)(Cfg::kABytes + (rows_b[0] + rows_b[1]) * Cfg::kBlockK * 2) * G;
            rot = p.k_rotate == 1 ? (int)(((long long)seg.tile * k_blocks) / num_tiles) : 0;
            backwards = !kSplitK && p.k_rotate == 2 && (tiles_done & 1);
            ++tiles_done;
            seg_start = false;
          }
          long long t0 = 0;
          if constexpr (kDebug) t0 = trace ? clock64() : 0;
          if (!wait_bounded(bar_base + kEmptyOff + 8u * s, phase ^ 1u, ctx, kStatusTimeoutProducer + s)) {
            ok = false;
            break;
          }
          if constexpr (kDebug)
            if (trace) stall += clock64() - t0;
          int kb_phys = kb + rot;                  // which K block this step loads (order is free)
          if (kb_phys >= k_blocks) kb_phys -= k_blocks;
          if (backwards) kb_phys = k_blocks - 1 - kb;
          const int x = kb_phys * Cfg::kBlockK;
          if (issuer) {
            if (is_leader) mbar_arrive_expect_tx(bar_base + kFullOff + 8u * s, tx_bytes);
            if constexpr (Cfg::kKSub > 1) {
              // one box per operand tile: all K blocks of the stage (uniform tiles only)
              tma_load_3d<G>(smem_a + s * Cfg::kABytes, &tmap_a, full_leader + 8u * s, 0, row_a, kb_phys * Cfg::kKSub, pol);
            } else if constexpr (!kAIsKM) {
              tma_load_2d<G>(smem_a + s * Cfg::kABytes, &tmap_a, full_leader + 8u * s, x, row_a, pol);
            } else {
              // A[K, M]: coordinates are (row of C, K); two 64 x 64 boxes cover the CTA's 128 rows
#pragma unroll
              for (int j = 0; j < Cfg::kBlockM / 64; ++j)
                tma_load_2d<G>(smem_a + s * Cfg::kABytes + j * 8192, &tmap_a, full_leader + 8u * s,
                               row_a + j * 64, x, pol);
            }
#pragma unroll
            for (int h = 0; h < Cfg::kHalves; ++h) {
              if constexpr (Cfg::kKSub > 1) {
                tma_load_3d<G>(smem_b + s * Cfg::kBBytes + h * Cfg::kBHalfBytes, &tmap_b, full_leader + 8u * s, 0,
                               row_b[h], kb_phys * Cfg::kKSub, pol);
              } else if constexpr (!kBIsKN) {
                // one box of b_box rows at a time (a single box for uniform tiles)
#pragma unroll 1
                for (int j = 0; j < rows_b[h]; j += b_box)
                  tma_load_2d<G>(smem_b + s * Cfg::kBBytes + h * Cfg::kBHalfBytes + j * (Cfg::kBlockK * 2), &tmap_b,
                                 full_leader + 8u * s, x, row_b[h] + j, pol);
              } else {
                // B[K, N] (uniform tiles only): coordinates are (column of B, K); one 64 x 64 box per
                // block of 64 columns
#pragma unroll
                for (int j = 0; j < Cfg::kBRows / 64; ++j)
                  tma_load_2d<G>(smem_b + s * Cfg::kBBytes + h * Cfg::kBHalfBytes + j * 8192, &tmap_b,
                                 full_leader + 8u * s, row_b[h] + j * 64, x, pol);
              }
            }
          }
          if (++kb == seg.kb1) {
            have = work.next(seg);
            kb = seg.kb0;
            seg_start = true;
          }
        }
        phase ^= 1u;
      }
      if constexpr (kDebug)
        if (trace && issuer) {
          trace[kTraceProdStall] = stall;
          trace[kTraceProdEnd] = clock64();
        }
    }
    __syncwarp();
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    // The leader CTA's warp runs the loop, one elected lane issues.  Same flattening /
    // unrolling as the producer: per ring slot the operand descriptors are the slot-0
    // descriptors plus a constant.
    if (is_leader) {
      const bool issuer = elect_one();
      bool peer_ready = true;
      if constexpr (G == 2) peer_ready = wait_bounded(bar_base + kTmemReadyOff, 0u, ctx, kStatusTimeoutMmaAcc + 0xf);
      // instruction descriptor without N: the width of each half is a property of the tile
      constexpr uint32_t idesc_base =
          make_idesc_f16(Cfg::kIsBf16 ? 1u : 0u, Cfg::kBlockM * G, 0, kBIsKN ? 1u : 0u, kAIsKM ? 1u : 0u);
      uint32_t idesc_h[2] = {idesc_base, idesc_base};
      const uint64_t da0 = kAIsKM ? make_smem_desc_sw128_mn(smem_a, 8192) : make_smem_desc_sw128(smem_a);
      constexpr uint32_t kAStepK = kAIsKM ? 128u : 2u;
      const uint64_t db0 = kBIsKN ? make_smem_desc_sw128_mn(smem_b, 8192) : make_smem_desc_sw128(smem_b);
      // start-address step (16-byte units) of B per 16-element K step: 32 bytes along a K-major row,
      // two 8-row groups of 1024 bytes for the MN-major layout
      constexpr uint32_t kBStepK = kBIsKN ? 128u : 2u;
      const uint32_t bar_peer = (G == 2) ? map_to_cta(bar_base, pair_base + 1u) : bar_base;
      uint32_t phase = 0;
      WorkIter<kSplitK> work(cluster_id, num_clusters, num_tiles, k_blocks, sk_factor);
      Segment seg;
      bool have = work.next(seg);
      int kb = seg.kb0, iter = 0;          // iter counts segments: it selects the accumulator slot
      bool ok = peer_ready;
      long long stall_full = 0, stall_acc = 0;
      const bool skip_mma = kDebug && (dbg & kDebugSkipMma);
      while (have && ok) {
#pragma unroll
        for (int s = 0; s < kStages; ++s) {
          if (!have) break;
          long long tf = 0;
          if constexpr (kDebug) tf = trace ? clock64() : 0;
          if (!(kDebug && (dbg & kDebugSkipLoads)) &&
              !wait_bounded(bar_base + kFullOff + 8u * s, phase, ctx, kStatusTimeoutMma + s)) {
            ok = false;
            break;
          }
          if constexpr (kDebug)
            if (trace) {
              const long long now = clock64();
              if (iter == 0 && kb == seg.kb0) {
                if (issuer) trace[kTraceMmaFirst] = now;
              } else {
                stall_full += now - tf;
              }
            }
          tc_fence_after_sync();
          const bool first_kb = kb == seg.kb0;
          const bool last_kb = kb == seg.kb1 - 1;
          if (first_kb) {
            int m_tile, n_tile;
            tile_coords(seg.tile, p, m_tile, n_tile);
            const TileCols tc = tile_columns<Cfg>(n_tile, p);
            idesc_h[0] = idesc_base | ((uint32_t)(tc.w0 >> 3) << 17);
            idesc_h[1] = idesc_base | ((uint32_t)(tc.w1 >> 3) << 17);
          }
#pragma unroll
          for (int h = 0; h < Cfg::kHalves; ++h) {
            // accumulator slot of this half, and the parity of its hand-over barriers
            const int slot = Cfg::kHalves == 1 ? (iter & 1) : h;
            const uint32_t slot_phase = Cfg::kHalves == 1 ? ((iter >> 1) & 1u) : (iter & 1u);
            if (first_kb) {
              long long ta = 0;
              if constexpr (kDebug) ta = trace ? clock64() : 0;
              if (!wait_bounded(bar_base + kTEmptyOff + 8u * slot, slot_phase ^ 1u, ctx,
                                kStatusTimeoutMmaAcc + slot)) {
                ok = false;
                break;
              }
              if constexpr (kDebug)
                if (trace) stall_acc += clock64() - ta;
              tc_fence_after_sync();
            }
            const uint32_t tmem_d = tmem_base + slot * Cfg::kSlotCols;
            // descriptor address fields are in 16-byte units; +2 per 16-element K step (32 bytes
            // inside the 128-byte swizzle row)
            const uint64_t da = da0 + (uint64_t)((s * Cfg::kABytes) >> 4);
            const uint64_t db = db0 + (uint64_t)((s * Cfg::kBBytes + h * Cfg::kBHalfBytes) >> 4);
            if (issuer) {
              if (!skip_mma) {
                umma_f16<G>(tmem_d, da, db, idesc_h[h], first_kb ? 0u : 1u);   // first K step of a segment overwrites
#pragma unroll
                for (int k = 1; k < Cfg::kBlockK / Cfg::kUmmaK; ++k) {
                  // four steps inside a 64-element K block, then on to the stage's next K block (its own
                  // K-major tile, right behind the first)
                  constexpr uint32_t kASub = (uint32_t)(Cfg::kABytes / Cfg::kKSub) >> 4;
                  constexpr uint32_t kBSub = (uint32_t)(Cfg::kBHalfBytes / Cfg::kKSub) >> 4;
                  umma_f16<G>(tmem_d, da + kASub * (k >> 2) + kAStepK * (k & 3), db + kBSub * (k >> 2) + kBStepK * (k & 3),
                              idesc_h[h], 1u);
                }
              }
              if (last_kb) {                                             // this half's accumulator is complete
                if (skip_mma) {
                  mbar_arrive_cluster_relaxed(bar_base + kTFullOff + 8u * slot);
                  if constexpr (G == 2) mbar_arrive_cluster_relaxed(bar_peer + kTFullOff + 8u * slot);
                } else {
                  umma_commit<G>(bar_base + kTFullOff + 8u * slot);
                  if constexpr (G == 2) umma_commit<G>(bar_peer + kTFullOff + 8u * slot);
                }
              }
            }
          }
          if (!ok) break;
          if (issuer) {
            if (skip_mma) {
              mbar_arrive_cluster_relaxed(bar_base + kEmptyOff + 8u * s);
              if constexpr (G == 2) mbar_arrive_cluster_relaxed(bar_peer + kEmptyOff + 8u * s);
            } else {
              umma_commit<G>(bar_base + kEmptyOff + 8u * s);               // slot reusable once its MMAs retire
              if constexpr (G == 2) umma_commit<G>(bar_peer + kEmptyOff + 8u * s);
            }
          }
          if (++kb == seg.kb1) {
            have = work.next(seg);
            kb = seg.kb0;
            ++iter;
          }
        }
        phase ^= 1u;
      }
      if constexpr (kDebug)
        if (trace && issuer) {
          trace[kTraceMmaStallFull] = stall_full;
          trace[kTraceMmaStallAcc] = stall_acc;
          trace[kTraceMmaEnd] = clock64();
          trace[kTraceTiles] = iter;
        }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;                                  // TMEM lane quarter this warp may read
    const int e = warp - 2;                                  // epilogue warp index
    constexpr int kColGroups = Cfg::kEpiWarps / 4;           // warps sharing a lane quarter split the chunks
    const int cg = e >> 2;
    constexpr int kChunks = Cfg::kMmaN / Cfg::kEpiCols;      // 64-column chunks per accumulator slot
    const uint32_t stage_buf = smem_epi + (uint32_t)e * Cfg::kEpiBufs * Cfg::kEpiWarpBuf;
    const uint32_t tempty_leader = ((G == 2) ? map_to_cta(bar_base, pair_base) : bar_base) + kTEmptyOff;
    int iter = 0;
    uint32_t buf = 0;
    bool ok = true;
    long long stall = 0;
    WorkIter<kSplitK> work(cluster_id, num_clusters, num_tiles, k_blocks, sk_factor);
    Segment seg;
    // K-split schedule: 16-byte pieces of a partial tile are laid out [piece][row][4 floats], so
    // the 32 rows a warp owns are 512 contiguous bytes per piece.  Only rows below M exist.
    const int sk_rows = kSplitK ? p.sk_rows : Cfg::kBlockM;
    const size_t partial_floats = (size_t)sk_rows * Cfg::kBlockN;
    const int my_row = q * 32 + (int)lane;                   // row of the CTA's 128 x kBlockN tile
    // cluster K-split: a contributor's share of the tile's 16-byte pieces (kBlockN / 4 of them) is
    // 2^rx_share_shift pieces wide
    int rx_share_shift = 0;
    int rx_row_groups = 1;
    int remote_chunks = 0;                                   // chunks this warp has sent to other CTAs so far
    constexpr uint32_t kRxBytes = Cfg::kBlockM * Cfg::kBlockN * 4;   // receive area: one fp32 partial tile, at the start of the ring
    if constexpr (kSplitK && Cfg::kHalves == 1) {
      static_assert(Cfg::kEpiWarps != 4 || kStages * Cfg::kStageBytes + Cfg::kEpiBytes >= (int)kRxBytes + 4 * 3 * 8192,
                    "ring + epilogue staging must hold the receive area and three staging slots per warp");
      if (cluster_split) {
        while (((Cfg::kBlockN / 4) >> rx_share_shift) > sk_factor) ++rx_share_shift;
        if (sk_factor > Cfg::kBlockN / 64) {                   // a share is one chunk of one group of row quarters
          rx_row_groups = sk_factor / (Cfg::kBlockN / 64);
          rx_share_shift = 4;
        }
      }
    }
    const int rx_warps = 4 / rx_row_groups;                  // row quarters (epilogue warps) per share
    for (; ok && work.next(seg); ++iter) {
      int m_tile, n_tile;
      tile_coords(seg.tile, p, m_tile, n_tile);
      const int row0 = (m_tile * G + (int)cta_rank) * Cfg::kBlockM + q * 32;
      const TileCols tcols = tile_columns<Cfg>(n_tile, p);
      const bool row_live = row0 + (int)lane < p.M;          // rows past M hold zeros: never moved
      // Contiguous ranges: a segment that does not start its tile leaves a partial tile for the
      // tile's owner.  Even split: every contributor leaves one, nobody owns the tile.
      const bool even = kSplitK && sk_factor > 1;
      const bool writes_partial = kSplitK && (even || seg.kb0 != 0);
      const bool reduces = kSplitK && !even && seg.kb0 == 0 && seg.kb1 != k_blocks;
      // this segment's partial tile: one per CTA, or one per unit and CTA of the pair
      const size_t my_partial = even ? ((size_t)(seg.tile * sk_factor + seg.part) * G + cta_rank) : (size_t)blockIdx.x;
      int writer_first = 0, writer_count = 0;
      if constexpr (kSplitK) {
        if (reduces) {
          // The tile's later K blocks belong to the next CTA (pair)s in range order.
          const long long units = (long long)num_tiles * k_blocks;
          const long long tile_end = (long long)(seg.tile + 1) * k_blocks;
          writer_first = cluster_id + 1;
          while (writer_first + writer_count < num_clusters &&
                 WorkIter<true>::range_start(writer_first + writer_count, num_clusters, units) < tile_end)
            ++writer_count;
          for (int w = 0; ok && w < writer_count; ++w)
            ok = wait_counter(p.sk_flags + (size_t)(writer_first + w) * G + cta_rank, Cfg::kEpiWarps, ctx,
                              kStatusTimeoutPartial);
          if (!ok) break;
        }
      }
#pragma unroll 1
      for (int h = 0; ok && h < Cfg::kHalves; ++h) {
        const int slot = Cfg::kHalves == 1 ? (iter & 1) : h;
        const uint32_t slot_phase = Cfg::kHalves == 1 ? ((iter >> 1) & 1u) : (iter & 1u);
        const int col0 = tcols.col0 + (h ? tcols.w0 : 0);
        const int chunks_h = (h ? tcols.w1 : tcols.w0) / Cfg::kEpiCols;    // 64-column chunks of this half
        long long te = 0;
        if constexpr (kDebug) te = trace ? clock64() : 0;
        if (!wait_bounded(bar_base + kTFullOff + 8u * slot, slot_phase, ctx, kStatusTimeoutEpilogue + slot)) {
          ok = false;
          break;
        }
        if constexpr (kDebug)
          if (trace) stall += clock64() - te;
        tc_fence_after_sync();
        if constexpr (kSplitK) {
          if (cluster_split) {
            // This CTA's accumulator is complete, so its operand ring is idle: it becomes the place
            // where the tile's contributors leave their partial sums of this CTA's share.  Tell
            // every contributor, and wait until all of them have said the same.
            __syncwarp();
            if ((int)lane < sk_factor)
              mbar_arrive_cluster_release(map_to_cta(bar_base + kRxReadyOff, lane * G + cta_rank));
            if (!wait_bounded(bar_base + kRxReadyOff, 0u, ctx, kStatusTimeoutPartial + 1)) {
              ok = false;
              break;
            }
            fence_acq_rel_cluster();
            if constexpr (kDebug)
              if (trace && warp == 2 && lane == 0) trace[kTraceRxReady] = clock64();
          }
        }
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + slot * Cfg::kSlotCols;
        // Everything that happens to one 32-row x 64-column chunk once it sits in registers.
        auto finish_chunk = [&](const int c, uint32_t (&v0)[32], uint32_t (&v1)[32]) {
          if constexpr (kSplitK) {
            const int piece0 = (h * kChunks + c) * 16;       // first 16-byte piece of this chunk
            if (cluster_split) {
              // The chunk belongs to the share of contributor `owner`.  Its receive area is laid out
              // [sender][row quarter][piece of the share][row][16 bytes], so what one warp sends
              // for one chunk is 8 KB in one piece: written to a staging slot of its own (every
              // chunk that leaves the CTA has one, nothing is reused) and moved by one asynchronous
              // copy that is counted on the owner's barrier.  The own share goes straight into place.
              if (row0 >= p.M) return;                          // none of this warp's rows exist: nothing to exchange
              // owner of this warp's chunk: by columns, and (more contributors than chunks) by row group
              const int by_cols = piece0 >> rx_share_shift;
              const int owner = by_cols * rx_row_groups + q / rx_warps;
              const int local0 = piece0 - (by_cols << rx_share_shift);
              const uint32_t rx_off =
                  (uint32_t)((((seg.part * rx_warps + q % rx_warps) << rx_share_shift) + local0) * 512);
              uint32_t dst = smem_a + rx_off;
              if (owner != seg.part) dst = smem_a + kRxBytes + (uint32_t)(q * 3 + remote_chunks) * 8192u;
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const uint32_t* v = (j < 8) ? &v0[4 * j] : &v1[4 * (j - 8)];
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + j * 512u + lane * 16u), "r"(v[0]),
                             "r"(v[1]), "r"(v[2]), "r"(v[3])
                             : "memory");
              }
              if (owner != seg.part) {
                ++remote_chunks;
                fence_proxy_async_smem();
                __syncwarp();
                const uint32_t to = (uint32_t)owner * G + cta_rank;
                if (lane == 0)
                  bulk_copy_smem_to_cluster(map_to_cta(smem_a + rx_off, to), dst, 8192u,
                                            map_to_cta(bar_base + kRxDoneOff, to));
              }
              return;
            }
            if (writes_partial) {
              if (row_live) {
                float4* dst = reinterpret_cast<float4*>(p.sk_partials + my_partial * partial_floats) +
                              (size_t)piece0 * sk_rows + my_row;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  const uint32_t* v = (j < 8) ? &v0[4 * j] : &v1[4 * (j - 8)];
                  dst[(size_t)j * sk_rows] = make_float4(__uint_as_float(v[0]), __uint_as_float(v[1]),
                                                               __uint_as_float(v[2]), __uint_as_float(v[3]));
                }
              }
              return;                                          // nothing goes to C from this segment
            }
            if (reduces && row_live) {
              for (int w = 0; w < writer_count; ++w) {
                const float4* src = reinterpret_cast<const float4*>(
                                        p.sk_partials + ((size_t)(writer_first + w) * G + cta_rank) * partial_floats) +
                                    (size_t)piece0 * sk_rows + my_row;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  uint32_t* v = (j < 8) ? &v0[4 * j] : &v1[4 * (j - 8)];
                  const float4 t = __ldcg(src + (size_t)j * sk_rows);
                  v[0] = __float_as_uint(__uint_as_float(v[0]) + t.x);
                  v[1] = __float_as_uint(__uint_as_float(v[1]) + t.y);
                  v[2] = __float_as_uint(__uint_as_float(v[2]) + t.z);
                  v[3] = __float_as_uint(__uint_as_float(v[3]) + t.w);
                }
              }
            }
          }
          if constexpr (kScaled) {
            const int col = col0 + c * Cfg::kEpiCols;
            if ((p.alpha != 1.0f || p.beta != 0.0f) && row0 + (int)lane < p.M && col < p.N) {
              const float alpha = p.alpha, beta = p.beta;
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                v0[i] = __float_as_uint(__uint_as_float(v0[i]) * alpha);
                v1[i] = __float_as_uint(__uint_as_float(v1[i]) * alpha);
              }
              if (beta != 0.0f) {
                // Old C of this thread's row in 16-byte pieces; the piece that straddles N (N not a
                // multiple of 8) is read element by element, so nothing past C[row, N-1] is touched.
                const uint16_t* crow = reinterpret_cast<const uint16_t*>(p.c_ptr) +
                                       (long long)(row0 + (int)lane) * p.ldc + col;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  if (col + 8 * j < p.N) {
                    uint32_t w[4] = {0u, 0u, 0u, 0u};
                    if (col + 8 * j + 8 <= p.N) {
                      const uint4 old = *reinterpret_cast<const uint4*>(crow + 8 * j);
                      w[0] = old.x, w[1] = old.y, w[2] = old.z, w[3] = old.w;
                    } else {
#pragma unroll
                      for (int t = 0; t < 8; ++t)
                        if (col + 8 * j + t < p.N) w[t >> 1] |= (uint32_t)crow[8 * j + t] << (16 * (t & 1));
                    }
                    uint32_t* v = (j < 4) ? &v0[8 * j] : &v1[8 * (j - 4)];
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                      float lo, hi;
                      if constexpr (Cfg::kIsBf16) {
                        lo = __uint_as_float(w[t] << 16);
                        hi = __uint_as_float(w[t] & 0xffff0000u);
                      } else {
                        const __half2 h2 = *reinterpret_cast<const __half2*>(&w[t]);
                        lo = __low2float(h2);
                        hi = __high2float(h2);
                      }
                      v[2 * t] = __float_as_uint(fmaf(beta, lo, __uint_as_float(v[2 * t])));
                      v[2 * t + 1] = __float_as_uint(fmaf(beta, hi, __uint_as_float(v[2 * t + 1])));
                    }
                  }
                }
              }
            }
          }
          const bool live = (row0 < p.M) && (c < chunks_h) && (col0 + c * Cfg::kEpiCols < p.N) &&
                            !(kDebug && (dbg & kDebugSkipStores));
          if (live) {
            // The staging buffer about to be rewritten must have been read by its store.
            if (lane == 0) tma_store_wait_read<Cfg::kEpiBufs - 1>();
            __syncwarp();
            const uint32_t dst = stage_buf + buf * Cfg::kEpiWarpBuf + lane * 128u;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint32_t* v = (j < 4) ? &v0[8 * j] : &v1[8 * (j - 4)];
              const uint32_t w0 = pack2<Cfg::kIsBf16>(v[0], v[1]);
              const uint32_t w1 = pack2<Cfg::kIsBf16>(v[2], v[3]);
              const uint32_t w2 = pack2<Cfg::kIsBf16>(v[4], v[5]);
              const uint32_t w3 = pack2<Cfg::kIsBf16>(v[6], v[7]);
              // 16-byte chunk j of row `lane` lands at chunk j ^ (row % 8): the 128-byte swizzle
              const uint32_t addr = dst + (((uint32_t)j ^ (lane & 7u)) << 4);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w0), "r"(w1),
                           "r"(w2), "r"(w3)
                           : "memory");
            }
            fence_proxy_async_smem();
            __syncwarp();
            // The output's tensor map ends at the last whole 16-byte piece of a row (a TMA store
            // that crosses the end of the tensor inside a piece was seen to write the whole piece,
            // zeroing up to 7 elements of the caller's memory past column N-1).  The N % 8 columns
            // after it go out as 2-byte stores, each thread re-reading its own staged piece.
            const int n_floor = p.N & ~7;
            const int colc = col0 + c * Cfg::kEpiCols;
            if (p.N != n_floor && colc <= n_floor && n_floor < colc + Cfg::kEpiCols && row_live) {
              const uint32_t j = (uint32_t)(n_floor - colc) >> 3;
              uint32_t w[4];
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3])
                           : "r"(dst + ((j ^ (lane & 7u)) << 4))
                           : "memory");
              uint16_t* crow = reinterpret_cast<uint16_t*>(p.c_ptr) + (long long)(row0 + (int)lane) * p.ldc + n_floor;
#pragma unroll
              for (int t = 0; t < 7; ++t)
                if (t < p.N - n_floor) crow[t] = (uint16_t)(w[t >> 1] >> (16 * (t & 1)));
            }
            if (lane == 0) {
              if (colc < n_floor)
                for (int d = 0; d < num_c; ++d)
                  tma_store_2d(tmap_c + d, stage_buf + buf * Cfg::kEpiWarpBuf, colc, row0);
              tma_store_commit();                              // also when empty: one group per buffer use
            }
            if constexpr (Cfg::kEpiBufs == 2) buf ^= 1u;
          }
        };
        constexpr int kPerWarp = kChunks / kColGroups;       // chunks of one slot this warp drains
        if constexpr (kPerWarp == 2 && !kSplitK) {
          // Drain both chunks into registers first and hand the slot back at once: the MMA
          // issuer restarts ~2 chunk-stores earlier (the double-width tile has no spare slot).
          uint32_t a0[32], a1[32], b0[32], b1[32];
          tmem_ld_32x32(taddr + cg * Cfg::kEpiCols, a0);
          tmem_ld_32x32(taddr + cg * Cfg::kEpiCols + 32, a1);
          tmem_ld_32x32(taddr + (cg + kColGroups) * Cfg::kEpiCols, b0);
          tmem_ld_32x32(taddr + (cg + kColGroups) * Cfg::kEpiCols + 32, b1);
          tmem_ld_wait();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(tempty_leader + 8u * slot);
          finish_chunk(cg, a0, a1);
          finish_chunk(cg + kColGroups, b0, b1);
        } else {
          if (cg >= chunks_h) {
            // a narrow tile leaves this warp without a chunk: it only hands the slot back
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty_leader + 8u * slot);
          }
#pragma unroll 1
          for (int c = cg; c < chunks_h; c += kColGroups) {
            uint32_t v0[32], v1[32];
            tmem_ld_32x32(taddr + c * Cfg::kEpiCols, v0);
            tmem_ld_32x32(taddr + c * Cfg::kEpiCols + 32, v1);
            tmem_ld_wait();
            if (c + kColGroups >= chunks_h) {
              // All of this warp's reads of the slot are done: hand it back to the MMA issuer.
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive_cluster(tempty_leader + 8u * slot);
            }
            finish_chunk(c, v0, v1);
          }
        }
      }
      if constexpr (kSplitK) {
        if (ok && cluster_split) {
          if constexpr (Cfg::kHalves == 1) {
            // Wait for the other contributors' copies (counted in bytes), then sum this CTA's share
            // in contributor order and store it.
            ok = wait_bounded(bar_base + kRxDoneOff, 0u, ctx, kStatusTimeoutPartial + 2);
            if (!ok) break;
            if constexpr (kDebug)
              if (trace && warp == 2 && lane == 0) trace[kTraceRxDone] = clock64();
            const int share = 1 << rx_share_shift;                // pieces (of 4 columns) in this CTA's share
            const int row = (m_tile * G + (int)cta_rank) * Cfg::kBlockM + my_row;
            const int col_first = n_tile * Cfg::kBlockN + (seg.part / rx_row_groups) * share * 4;
            const bool my_rows = q / rx_warps == seg.part % rx_row_groups;   // this warp's rows are in the share
            if (row < p.M && my_rows && !(kDebug && (dbg & kDebugSkipStores))) {
              uint16_t* crow = reinterpret_cast<uint16_t*>(p.c_ptr) + (long long)row * p.ldc + col_first;
              // [sender][row quarter of the share][piece][row]: this thread's row of piece l from sender i
              const float4* rx = reinterpret_cast<const float4*>(smem) + ((size_t)((q % rx_warps) * share) * 32 + lane);
              const size_t sender_stride = (size_t)rx_warps * share * 32;
#pragma unroll 1
              for (int l = 0; l < share; l += 2) {                 // two pieces = 8 columns = 16 bytes of C
                const int col = col_first + l * 4;
                if (col >= p.N) break;
                const float4* r0 = rx + (size_t)l * 32;
                const float4* r1 = r0 + 32;
                float4 s0 = r0[0], s1 = r1[0];
                {
                  const float4 a0 = r0[sender_stride], a1 = r1[sender_stride];
                  s0.x += a0.x, s0.y += a0.y, s0.z += a0.z, s0.w += a0.w;
                  s1.x += a1.x, s1.y += a1.y, s1.z += a1.z, s1.w += a1.w;
                }
                if (sk_factor == 4) {
                  const float4 b0 = r0[2 * sender_stride], b1 = r1[2 * sender_stride];
                  const float4 c0 = r0[3 * sender_stride], c1 = r1[3 * sender_stride];
                  s0.x += b0.x, s0.y += b0.y, s0.z += b0.z, s0.w += b0.w;
                  s1.x += b1.x, s1.y += b1.y, s1.z += b1.z, s1.w += b1.w;
                  s0.x += c0.x, s0.y += c0.y, s0.z += c0.z, s0.w += c0.w;
                  s1.x += c1.x, s1.y += c1.y, s1.z += c1.z, s1.w += c1.w;
                }
                const uint32_t w0 = pack2<Cfg::kIsBf16>(__float_as_uint(s0.x), __float_as_uint(s0.y));
                const uint32_t w1 = pack2<Cfg::kIsBf16>(__float_as_uint(s0.z), __float_as_uint(s0.w));
                const uint32_t w2 = pack2<Cfg::kIsBf16>(__float_as_uint(s1.x), __float_as_uint(s1.y));
                const uint32_t w3 = pack2<Cfg::kIsBf16>(__float_as_uint(s1.z), __float_as_uint(s1.w));
                if (col + 8 <= p.N) {
                  *reinterpret_cast<uint4*>(crow + l * 4) = make_uint4(w0, w1, w2, w3);
                } else {
                  const uint32_t w[4] = {w0, w1, w2, w3};
#pragma unroll
                  for (int t2 = 0; t2 < 8; ++t2)
                    if (col + t2 < p.N) crow[l * 4 + t2] = (uint16_t)(w[t2 >> 1] >> (16 * (t2 & 1)));
                }
              }
            }
          }
        } else if (ok && writes_partial) {
          // Publish this warp's share of the partial tile: writes, fence, then one arrival.
          __threadfence();
          __syncwarp();
          if (lane == 0) atomicAdd(p.sk_flags + (even ? (size_t)seg.tile * G + cta_rank : (size_t)blockIdx.x), 1u);
        }
        if constexpr (Cfg::kHalves == 1) {
          if (ok && even && !cluster_split) {
            // Every contributor of the tile has arrived once all their epilogue warps have: then this
            // one reduces and stores its share, the 32-row x 64-column blocks b with b % factor == part,
            // adding the partial tiles in range order.  Plain 16-byte stores from registers.
            ok = wait_counter(p.sk_flags + (size_t)seg.tile * G + cta_rank, Cfg::kEpiWarps * sk_factor, ctx,
                              kStatusTimeoutPartial);
            if (!ok) break;
            constexpr int kBlocks = 4 * kChunks;                   // 4 row quarters x 64-column chunks
            // Every warp works on every block of this contributor's share, each on its own 16 / kEpiWarps
            // pieces (of 4 columns) of the block's 64 columns, with the loads of up to eight
            // contributors in flight at once: the reduction is a chain of L2 round trips, and dealing
            // whole blocks to single warps that read one contributor at a time made it eight times
            // as long.
            constexpr int kPieces = 16 / Cfg::kEpiWarps;
            constexpr int kInFlight = 8;
#pragma unroll 1
            for (int b = seg.part; b < kBlocks; b += sk_factor) {
              const int bq = b & 3, bc = b >> 2;                  // row quarter, chunk of the tile
              const int row = (m_tile * G + (int)cta_rank) * Cfg::kBlockM + bq * 32 + (int)lane;
              const int colc = n_tile * Cfg::kBlockN + bc * Cfg::kEpiCols + e * kPieces * 4;   // this warp's columns
              if (row >= p.M || colc >= p.N || (kDebug && (dbg & kDebugSkipStores))) continue;
              uint16_t* crow = reinterpret_cast<uint16_t*>(p.c_ptr) + (long long)row * p.ldc + colc;
              const size_t piece_off = (size_t)(bc * 16 + e * kPieces) * sk_rows + bq * 32 + lane;
              float4 acc[kPieces];
#pragma unroll 1
              for (int i0 = 0; i0 < sk_factor; i0 += kInFlight) {
                float4 t[kInFlight][kPieces];
#pragma unroll
                for (int ii = 0; ii < kInFlight; ++ii) {
                  if (i0 + ii < sk_factor) {
                    const float4* src = reinterpret_cast<const float4*>(
                                            p.sk_partials +
                                            ((size_t)(seg.tile * sk_factor + i0 + ii) * G + cta_rank) * partial_floats) +
                                        piece_off;
#pragma unroll
                    for (int j = 0; j < kPieces; ++j) t[ii][j] = __ldcg(src + (size_t)j * sk_rows);
                  }
                }
#pragma unroll
                for (int ii = 0; ii < kInFlight; ++ii) {           // added in range order: the result is
                  if (i0 + ii < sk_factor) {                       // independent of who arrived when
#pragma unroll
                    for (int j = 0; j < kPieces; ++j) {
                      if (i0 + ii == 0) {
                        acc[j] = t[ii][j];
                      } else {
                        acc[j].x += t[ii][j].x;
                        acc[j].y += t[ii][j].y;
                        acc[j].z += t[ii][j].z;
                        acc[j].w += t[ii][j].w;
                      }
                    }
                  }
                }
              }
#pragma unroll
              for (int j = 0; j < kPieces / 2; ++j) {             // 8 columns = 16 bytes of C per step
                const int col = colc + j * 8;
                const uint32_t w0 = pack2<Cfg::kIsBf16>(__float_as_uint(acc[2 * j].x), __float_as_uint(acc[2 * j].y));
                const uint32_t w1 = pack2<Cfg::kIsBf16>(__float_as_uint(acc[2 * j].z), __float_as_uint(acc[2 * j].w));
                const uint32_t w2 = pack2<Cfg::kIsBf16>(__float_as_uint(acc[2 * j + 1].x), __float_as_uint(acc[2 * j + 1].y));
                const uint32_t w3 = pack2<Cfg::kIsBf16>(__float_as_uint(acc[2 * j + 1].z), __float_as_uint(acc[2 * j + 1].w));
                if (col + 8 <= p.N) {
                  *reinterpret_cast<uint4*>(crow + j * 8) = make_uint4(w0, w1, w2, w3);
                } else {
                  const uint32_t w[4] = {w0, w1, w2, w3};
#pragma unroll
                  for (int t2 = 0; t2 < 8; ++t2)
                    if (col + t2 < p.N) crow[j * 8 + t2] = (uint16_t)(w[t2 >> 1] >> (16 * (t2 & 1)));
                }
              }
            }
            // Done with the tile's partial sums.  The last of the tile's warps to say so puts the
            // counter back to zero, so a workspace that starts out zeroed is zeroed again when the
            // launch completes and the next launch needs no memset in front of it.
            __syncwarp();
            if (lane == 0) {
              unsigned int* counter = p.sk_flags + (size_t)seg.tile * G + cta_rank;
              const unsigned int before = atomicAdd(counter, 0x10000u);
              if ((before >> 16) == (unsigned int)(Cfg::kEpiWarps * sk_factor) - 1u) atomicExch(counter, 0u);
            }
          }
        }
      }
    }
    if (lane == 0) tma_store_wait_read<0>();   // smem may go once it has been read; the writes finish on their own
    __syncwarp();
    if constexpr (kDebug)
      if (trace && warp == 2 && lane == 0) {
        trace[kTraceEpiStall] = stall;
        trace[kTraceEpiEnd] = clock64();
      }
  }

  // ------------------------------------------------------------------ tear-down
  if (*abort_flag != 0) {
    // A wait gave up: loads this CTA issued may still be in flight towards its shared memory.
    // Give them time to land (they take microseconds) before the memory is handed back.
#pragma unroll 1
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (G == 2 || cluster_split) {
    // The peer's shared memory and barriers are MMA / commit targets until both are here; in the
    // cluster K-split every CTA's shared memory is a store target of the whole cluster.
    cluster_arrive();
    cluster_wait();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<G>(tmem_base, Cfg::kTmemCols);
  }
  if constexpr (kDebug)
    if (trace && threadIdx.x == 0) {
      trace[kTraceExit] = clock64();
      trace[kTraceTimeExitNs] = global_timer_ns();
    }
}

template <class Cfg, bool kDebug, bool kSplitK = false>
__global__ void __launch_bounds__(Cfg::kThreads, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_c, const TileParams p) {
  gemm_tn_body<Cfg, kDebug, kSplitK>(tmap_a, tmap_b, &tmap_c, 1, p);
}

// The other operand layouts: same kernel, B given as [K,N] and / or A given as [K,M], loaded and
// described as MN-major operands.
// These instantiations also carry the alpha / beta epilogue (a run-time test per chunk).
template <class Cfg, bool kAIsKM, bool kBIsKN>
__global__ void __launch_bounds__(Cfg::kThreads, 1)
gemm_layout_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                   const __grid_constant__ CUtensorMap tmap_c, const TileParams p) {
  gemm_tn_body<Cfg, false, false, kBIsKN, kAIsKM, true>(tmap_a, tmap_b, &tmap_c, 1, p);
}

// Self-test of the bounded wait: one warp waits on a barrier that nothing ever arrives on.  The
// wait must give up after the time limit, record kStatusSelfTest and let the kernel return.
constexpr uint32_t kStatusSelfTest = 0x7e57;
__global__ void __launch_bounds__(32, 1) wait_timeout_selftest_kernel(unsigned int* status, unsigned long long timeout_ns) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    fence_mbar_init();
  }
  __syncwarp();
  WaitCtx ctx;
  ctx.abort_flag = &abort_flag;
  ctx.peer_abort_addr = smem_u32(&abort_flag);
  ctx.status = status;
  ctx.timeout_ns = timeout_ns;
  (void)wait_bounded(smem_u32(&bar), 0u, ctx, kStatusSelfTest);
}

// Output tensor maps of the store-to-every-GPU variant.
constexpr int kMaxOutputs = 8;
struct OutputMaps {
  CUtensorMap maps[kMaxOutputs];
};

template <class Cfg, bool kDebug = false>
__global__ void __launch_bounds__(Cfg::kThreads, 1)
gemm_tn_fanout_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const __grid_constant__ OutputMaps outputs, const int num_outputs, const TileParams p) {
  gemm_tn_body<Cfg, kDebug, false>(tmap_a, tmap_b, outputs.maps, num_outputs, p);
}

}  // namespace gemm_sm100
