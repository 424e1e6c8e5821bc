// Persistent, warp-specialised TN GEMM for sm_100a:
//   C[M,N] = A[M,K] * B[N,K]^T, 16-bit inputs (bf16 or fp16), fp32 accumulation in
//   tensor memory, same-dtype output rounded to nearest even.
//
// It replaces the reference's Hopper kernel test::gemm_kernel
// (kernels/gemm_kernels/sm90a/gemm.cuh:246-418, 452-462): same math and the same
// "both operands K-major" layout contract, but none of its structure.  Roles per CTA
// (192 threads):
//   warp 0      TMA producer   : global -> smem ring of kStages (A tile + B tile), mbarrier tx-count
//   warp 1      MMA issuer     : one thread issues tcgen05.mma from smem descriptors into TMEM;
//                                 tcgen05.commit frees ring slots and publishes finished accumulators
//   warps 2..5  epilogue       : tcgen05.ld TMEM -> registers -> 16-bit -> swizzled smem -> TMA store
// Two accumulator buffers live in TMEM (2 x kBlockN fp32 columns), so the epilogue of
// tile i runs under the mainloop of tile i+1 (the reference's single register-resident
// accumulator idles the tensor pipe during every epilogue, gemm.cuh:368-395).
//
// kCtaGroup == 2 pairs two CTAs (a 2-CTA cluster) on one 256 x kBlockN tile: each CTA
// loads its own 128 rows of A and its own kBlockN/2 rows of B with plain TMA loads, and
// the leader CTA issues cta_group::2 MMAs that read both CTAs' shared memory.  This gives
// the operand sharing that the reference gets from a cluster-broadcast load of B
// (gemm_test.cu:60-64) without any broadcast load.
//
// Every wait on an mbarrier is bounded: when a wait runs out the CTA (and its pair
// peer) is flagged, all roles fall through to the common tear-down, TMEM is released and
// the launcher reports the status word.  The reference's waits are unbounded
// (gemm.cuh:75-78, 91-94).
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
};

struct TileParams {
  int M, N, K;
  int m_tiles;   // ceil(M / (128 * kCtaGroup))
  int n_tiles;   // ceil(N / kBlockN)
  int k_blocks;  // ceil(K / 64)
  int group_m;   // tiles along M per rasterisation group
  unsigned int* status;            // device word, 0 = ok
  unsigned long long timeout_ns;   // bound of every device-side wait
};

template <int kCtaGroup_, int kBlockN_, int kStages_, bool kIsBf16_>
struct GemmConfig {
  static constexpr int kCtaGroup = kCtaGroup_;
  static constexpr int kBlockM = 128;              // rows of A (and of the accumulator) per CTA
  static constexpr int kBlockN = kBlockN_;         // MMA N: columns of C per tile (whole pair)
  static constexpr int kBlockK = 64;               // 64 x 16 bit = one 128-byte swizzle row
  static constexpr int kStages = kStages_;
  static constexpr bool kIsBf16 = kIsBf16_;
  static constexpr int kUmmaK = 16;
  static constexpr int kBRows = kBlockN / kCtaGroup;            // rows of B this CTA loads
  static constexpr int kABytes = kBlockM * kBlockK * 2;
  static constexpr int kBBytes = kBRows * kBlockK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kEpiCols = 64;                           // columns per TMA-store chunk
  static constexpr int kEpiWarpBuf = 32 * kEpiCols * 2;         // one warp, one chunk: 4 KiB
  static constexpr int kEpiBytes = 4 * 2 * kEpiWarpBuf;         // 4 warps, double buffered
  static constexpr int kTmemCols = 2 * kBlockN;                 // two accumulator buffers
  static constexpr int kBarrierBytes = 256;
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kEpiBytes + kBarrierBytes;
  static constexpr int kThreads = 192;
  static_assert(kBlockN % 64 == 0 && kBlockN >= 64 && kBlockN <= 256, "tile N");
  static_assert(kTmemCols == 128 || kTmemCols == 256 || kTmemCols == 512, "TMEM columns: power of two");
  static_assert(kBBytes % 1024 == 0, "B tile must keep 1024-byte swizzle alignment");
  static_assert(kSmemBytes <= 232448, "shared memory budget");
};

struct WaitCtx {
  volatile uint32_t* abort_flag;   // this CTA's flag in shared memory
  uint32_t peer_abort_addr;        // shared::cluster address of the pair peer's flag (or own)
  unsigned int* status;
  unsigned long long timeout_ns;
};

// Bounded mbarrier wait.  Returns false if the CTA was flagged or the wait ran out.
__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity, const WaitCtx& ctx,
                                             uint32_t code) {
#pragma unroll 1
  for (int i = 0; i < 64; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
#pragma unroll 1
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*ctx.abort_flag != 0) return false;
    if (global_timer_ns() - t0 > ctx.timeout_ns) {
      *ctx.abort_flag = 1;
      st_cluster_u32(ctx.peer_abort_addr, 1);
      atomicCAS(ctx.status, 0u, code);
      return false;
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

template <class Cfg>
__global__ void __launch_bounds__(Cfg::kThreads, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_c, const TileParams p) {
  constexpr int G = Cfg::kCtaGroup;
  constexpr int kStages = Cfg::kStages;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;          // 128B-swizzle atoms need 1024 B
  uint8_t* smem = smem_raw + (base - raw_addr);

  const uint32_t smem_a = base;
  const uint32_t smem_b = base + kStages * Cfg::kABytes;
  const uint32_t smem_epi = smem_b + kStages * Cfg::kBBytes;
  uint8_t* bar_mem = smem + kStages * Cfg::kStageBytes + Cfg::kEpiBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(bar_mem);
  // barrier indices
  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  static_assert(8 * (2 * kStages + 4) + 8 <= Cfg::kBarrierBytes, "barrier block too small");
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_mem + 8 * (2 * kStages + 4));
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const uint32_t lane = lane_id();
  const uint32_t cta_rank = (G == 2) ? cluster_ctarank() : 0u;
  const bool is_leader = cta_rank == 0;

  WaitCtx ctx;
  ctx.abort_flag = abort_flag;
  ctx.peer_abort_addr = (G == 2) ? map_to_cta(smem_u32((const void*)abort_flag), cta_rank ^ 1u)
                                 : smem_u32((const void*)abort_flag);
  ctx.status = p.status;
  ctx.timeout_ns = p.timeout_ns;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
    prefetch_tensormap(&tmap_c);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);    // leader's producer arrives once and posts the byte count
      mbar_init(empty_bar(s), 1);   // one tcgen05.commit per use
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);          // one tcgen05.commit per tile
      mbar_init(tempty_bar(a), 4 * G);     // every epilogue warp of the pair arrives once
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc<G>(smem_u32(tmem_slot), Cfg::kTmemCols);
    tmem_relinquish<G>();
  }
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (G == 2) {
    cluster_arrive();
    cluster_wait();
  }
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = p.m_tiles * p.n_tiles;
  const int first_tile = blockIdx.x / G;
  const int tile_step = gridDim.x / G;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const uint64_t pol = policy_evict_normal();
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = first_tile; ok && tile < num_tiles; tile += tile_step) {
        int m_tile, n_tile;
        tile_coords(tile, p, m_tile, n_tile);
        const int row_a = (m_tile * G + (int)cta_rank) * Cfg::kBlockM;
        const int row_b = n_tile * Cfg::kBlockN + (int)cta_rank * Cfg::kBRows;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!wait_bounded(empty_bar(stage), phase ^ 1u, ctx, kStatusTimeoutProducer + stage)) {
            ok = false;
            break;
          }
          // Both CTAs of a pair complete their bytes on the LEADER's barrier: the
          // leader's MMA thread is the only consumer of the ring.
          const uint32_t fb = (G == 2) ? map_to_cta(full_bar(stage), 0u) : full_bar(stage);
          if (is_leader) mbar_arrive_expect_tx(full_bar(stage), Cfg::kStageBytes * G);
          tma_load_2d<G>(smem_a + stage * Cfg::kABytes, &tmap_a, fb, kb * Cfg::kBlockK, row_a, pol);
          tma_load_2d<G>(smem_b + stage * Cfg::kBBytes, &tmap_b, fb, kb * Cfg::kBlockK, row_b, pol);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0 && is_leader) {
      constexpr uint32_t idesc =
          make_idesc_f16(Cfg::kIsBf16 ? 1u : 0u, Cfg::kBlockM * G, Cfg::kBlockN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int iter = 0;
      for (int tile = first_tile; ok && tile < num_tiles; tile += tile_step, ++iter) {
        const int acc = iter & 1;
        const uint32_t acc_phase = (iter >> 1) & 1u;
        if (!wait_bounded(tempty_bar(acc), acc_phase ^ 1u, ctx, kStatusTimeoutMmaAcc + acc)) break;
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * Cfg::kBlockN;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!wait_bounded(full_bar(stage), phase, ctx, kStatusTimeoutMma + stage)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint64_t da = make_smem_desc_sw128(smem_a + stage * Cfg::kABytes);
          const uint64_t db = make_smem_desc_sw128(smem_b + stage * Cfg::kBBytes);
#pragma unroll
          for (int k = 0; k < Cfg::kBlockK / Cfg::kUmmaK; ++k) {
            // +32 bytes per 16-element K step inside the 128-byte swizzle row (>>4 encoded)
            umma_f16<G>(tmem_d, da + 2u * k, db + 2u * k, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit<G>(empty_bar(stage));                       // slot reusable once MMAs retire
          if constexpr (G == 2) umma_commit<G>(map_to_cta(empty_bar(stage), 1u));
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit<G>(tfull_bar(acc));                           // accumulator ready
        if constexpr (G == 2) umma_commit<G>(map_to_cta(tfull_bar(acc), 1u));
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;                                  // TMEM lane quarter this warp may read
    const uint32_t stage_buf = smem_epi + (uint32_t)(warp - 2) * 2u * Cfg::kEpiWarpBuf;
    const uint32_t tempty_leader0 = (G == 2) ? map_to_cta(tempty_bar(0), 0u) : tempty_bar(0);
    const uint32_t tempty_leader1 = (G == 2) ? map_to_cta(tempty_bar(1), 0u) : tempty_bar(1);
    int iter = 0;
    uint32_t buf = 0;
    bool ok = true;
    for (int tile = first_tile; ok && tile < num_tiles; tile += tile_step, ++iter) {
      int m_tile, n_tile;
      tile_coords(tile, p, m_tile, n_tile);
      const int acc = iter & 1;
      const uint32_t acc_phase = (iter >> 1) & 1u;
      const int row0 = (m_tile * G + (int)cta_rank) * Cfg::kBlockM + q * 32;
      const int col0 = n_tile * Cfg::kBlockN;
      if (!wait_bounded(tfull_bar(acc), acc_phase, ctx, kStatusTimeoutEpilogue + acc)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * Cfg::kBlockN;
#pragma unroll 1
      for (int c = 0; c < Cfg::kBlockN / Cfg::kEpiCols; ++c) {
        uint32_t v0[32], v1[32];
        tmem_ld_32x32(taddr + c * Cfg::kEpiCols, v0);
        tmem_ld_32x32(taddr + c * Cfg::kEpiCols + 32, v1);
        tmem_ld_wait();
        if (c == Cfg::kBlockN / Cfg::kEpiCols - 1) {
          // All of this warp's reads of the accumulator are done: hand the buffer back.
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(acc ? tempty_leader1 : tempty_leader0);
        }
        const bool live = (row0 < p.M) && (col0 + c * Cfg::kEpiCols < p.N);
        if (live) {
          // The staging buffer written two chunks ago must have been read by its store.
          if (lane == 0) tma_store_wait_read<1>();
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
          if (lane == 0) {
            tma_store_2d(&tmap_c, stage_buf + buf * Cfg::kEpiWarpBuf, col0 + c * Cfg::kEpiCols, row0);
            tma_store_commit();
          }
          buf ^= 1u;
        }
      }
    }
    if (lane == 0) tma_store_wait_all<0>();
    __syncwarp();
  }

  // ------------------------------------------------------------------ tear-down
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (G == 2) {
    // The peer's shared memory and barriers are MMA / commit targets until both are here.
    cluster_arrive();
    cluster_wait();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<G>(tmem_base, Cfg::kTmemCols);
  }
}

}  // namespace gemm_sm100
