// Host launcher and C ABI (include/gemm_sm100.h) of the sm_100a TN GEMM.
// Compiled by nvcc alone: no torch headers in this translation unit (the reference's
// launcher sm90a/gemm_test.cu:9-10 pulls torch/extension.h into its .cu file).
//
// What the reference does per call in test::gemm_tn_test (gemm_test.cu:12-92) and where
// it is here:  argument checks :15-41 -> validate();  CuTe tensor-map construction
// :56-68 -> encode_2d() through the driver entry point;  grid = min(132, tiles) :70-72 ->
// persistent grid from the device's SM count and cluster occupancy;  cluster launch
// :82-85 -> cudaLaunchKernelEx on the caller's stream;  sync + exit on error :86 ->
// asynchronous, errors returned.
#include <cuda.h>
#include <cmath>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <atomic>
#include <mutex>
#include <utility>
#include <vector>
#include <cstdint>

#include "../../include/gemm_sm100.h"
#include "gemm_tn_sm100.cuh"

namespace {

using namespace gemm_sm100;

// One status word per device (a __device__ variable exists once per device).
__device__ unsigned int g_status_word;

// Scratch of gemm_sm100_tn_static_scratch: arrival counters (first kStaticFlagBytes) followed by
// fp32 partial tiles.  Every device that loads this library holds one copy until exit.
constexpr size_t kStaticFlagBytes = 1024;
constexpr size_t kStaticScratchBytes = kStaticFlagBytes + 5u * 1024u * 1024u;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
constexpr int kNumConfigs = 16;

struct ConfigInfo {
  int cta_group, mma_n, halves, stages, epi_warps;
  int a_rows = 128;    // rows of A loaded per stage: the configuration only takes problems of at most that many rows
  int epi_bufs = 0;    // staging buffers per epilogue warp (0: 8 / epi_warps)
  int k_sub = 1;       // 64-element K blocks per stage (2: one 3-D TMA box per operand tile and stage)
};
constexpr ConfigInfo kConfigs[kNumConfigs] = {
    {2, 256, 1, 6, 4},   // 256 x 256 pair tile, alternating accumulator slots
    {2, 256, 2, 4, 8},   // 256 x 512 pair tile, both slots, 8 epilogue warps
    {1, 256, 1, 4, 4},   // 128 x 256 single-CTA tile
    {1, 128, 1, 4, 4},   // 128 x 128 single-CTA tile
    {2, 256, 2, 4, 4},
    {2, 256, 1, 6, 8},
    {1, 256, 1, 4, 8},
    // 256 x 128 pair tile: fewest operand bytes per SM among the small tiles.  Five stages: with
    // operand boxes this small the ring delivers FEWER bytes per clock the more loads it keeps in
    // flight (trace counters with the MMAs switched off, 8192 x 4096 x 4096: 0.48 of the MMA rate
    // with 4 stages, 0.47 with 5, 0.44 with 6, 0.35 with 8), and few-tile problems ran 13-20 % faster
    // with 5 stages than with 8.
    {2, 128, 1, 5, 4},
    {2, 192, 1, 6, 4},   // 256 x 192 pair tile: for tile counts that quantise badly with 256 columns
    // 128 x 256 tiles for problems of at most 16 / 64 rows: only those rows of A are loaded, and the
    // shared memory saved holds more stages (6 / 5 x 32 KiB of B in flight per SM instead of 4)
    {1, 256, 1, 6, 4, 16, 1},
    {1, 256, 1, 5, 4, 64, 1},
    // 256 x 128 pair tile with two K blocks per stage (K % 64 == 0 only): half as many, twice as
    // large TMA boxes as configuration 7
    {2, 128, 1, 4, 4, 128, 0, 2},
    // 128 x 128 single-CTA tile with two K blocks per stage, for problems of at most 128 rows whose
    // columns give too few 256-wide tiles: twice the tiles of configuration 2, half-size partial tiles
    {1, 128, 1, 3, 4, 128, 0, 2},
    // 128 x 64 tiles for problems of at most 16 / 64 rows and several thousand columns: four K blocks
    // (512 bytes of every row) per TMA box, short A
    {1, 64, 1, 5, 4, 16, 1, 4},
    {1, 64, 1, 3, 4, 64, 1, 4},
    // configuration 9 with two K blocks per box (K % 64 == 0): 16 x 28672 x 8192 74.5 against 75.6 us
    {1, 256, 1, 3, 4, 16, 1, 2},
};

template <int kIndex, bool kIsBf16>
using ConfigOf = GemmConfig<kConfigs[kIndex].cta_group, kConfigs[kIndex].mma_n, kConfigs[kIndex].halves,
                            kConfigs[kIndex].stages, kConfigs[kIndex].epi_warps, kIsBf16, kConfigs[kIndex].a_rows,
                            kConfigs[kIndex].epi_bufs, kConfigs[kIndex].k_sub>;

struct DeviceState {
  bool ready = false;
  int device = 0;
  int sm_count = 0;
  int cc_major = 0;
  unsigned int* status_ptr = nullptr;
  void* static_scratch = nullptr;      // device address of g_static_scratch on this device
  int max_ctas[kNumConfigs][2] = {};   // persistent grid limit per config and dtype
  bool attr_set[kNumConfigs][2] = {};
};

std::mutex g_mutex;
DeviceState g_dev[kMaxDevices];
// Process-wide knobs.  Written by gemm_sm100_set_option / gemm_sm100_set_trace_buffer, read by
// launches on any thread: atomics, so a concurrent change is seen whole or not at all.
std::atomic<long> g_opt_tile_config{-1};
std::atomic<long> g_opt_timeout_ms{2000};
std::atomic<long> g_opt_max_ctas{0};
std::atomic<long> g_opt_debug_flags{0};
std::atomic<long> g_opt_group_m{0};
std::atomic<long> g_opt_k_rotate{-1};   // 0 never, 1 always, -1 (default) when there is a single tile row: 3 % on the few-row shapes, 2 = serpentine
std::atomic<long> g_opt_sk_cluster{-1};  // cluster K-split (partial sums through distributed shared memory): -1 planner, 0 never, 1 always where an even split of 2 or 4 is made
std::atomic<long> g_opt_pdl{1};        // 1: launch with programmatic stream serialization (overlap with the previous kernel's tail)
std::atomic<long> g_opt_early_prefetch{1};   // with pdl: L2 prefetch of the first stages before waiting for the previous kernel
std::atomic<long> g_opt_tiles_n{0};    // > 0: force this many tiles per tile row (tests), when the configuration allows the widths
std::atomic<long> g_opt_balance{1};    // 1: the planner may choose a balanced column tiling; 0: uniform tiles only
std::atomic<long> g_opt_split_k{-1};   // -1 automatic, 0 never, 1 whenever the configuration allows it
// Clusters of 2, 4 and 8 CTAs (one CTA per SM) the device holds at once, from the occupancy query.
std::atomic<int> g_held_clusters[3] = {};
// Bumped by every gemm_sm100_set_option: cached plans of an older generation are stale.
std::atomic<unsigned> g_opt_generation{1};

// Workspaces registered with gemm_sm100_workspace_register: the library zero-fills the start once
// and from then on knows how long a prefix the launches queued so far leave zeroed.
struct KeptWorkspace {
  void* ptr;
  size_t clean_bytes;   // this prefix is zero once the work queued so far has run
};
constexpr size_t kKeptWorkspaceZeroBytes = 4096;   // more than any plan's counter area
std::mutex g_kept_mutex;
std::vector<KeptWorkspace> g_kept_workspaces;

// Whether the counter area (the first `flag_bytes` of `workspace`) has to be zero-filled before a
// K-split launch.  `self_resetting`: the launch leaves its counters at zero (the even split does,
// the contiguous one does not).  The partial tiles follow the counters, so after the launch nothing
// beyond `flag_bytes` is known to be zero.
bool kept_workspace_needs_zeroing(void* workspace, size_t flag_bytes, bool self_resetting) {
  std::lock_guard<std::mutex> lock(g_kept_mutex);
  for (KeptWorkspace& w : g_kept_workspaces) {
    if (w.ptr != workspace) continue;
    const bool zero_already = flag_bytes <= w.clean_bytes;
    w.clean_bytes = self_resetting ? flag_bytes : 0;
    return !zero_already;
  }
  return true;
}

void kept_workspaces_mark_dirty() {
  std::lock_guard<std::mutex> lock(g_kept_mutex);
  for (KeptWorkspace& w : g_kept_workspaces) w.clean_bytes = 0;
}
// Trace buffer (gemm_sm100_set_trace_buffer): pointer, size and the device that owns the memory,
// kept together under g_mutex so that a launch reads a consistent triple.  Launches on any other
// device ignore the buffer (its address means nothing there).
struct TraceBuffer {
  unsigned long long* ptr = nullptr;
  size_t bytes = 0;
  int device = -1;
};
TraceBuffer g_trace;
std::atomic<bool> g_trace_on{false};   // fast check outside the mutex

TraceBuffer trace_for_device(int device) {
  if (!g_trace_on.load(std::memory_order_acquire)) return TraceBuffer{};
  std::lock_guard<std::mutex> lock(g_mutex);
  return g_trace.device == device ? g_trace : TraceBuffer{};
}

// Optional overrides from the environment, read once when the library is loaded:
// GEMM_SM100_TILE_CONFIG, GEMM_SM100_SPLIT_K, GEMM_SM100_GROUP_M, GEMM_SM100_MAX_CTAS,
// GEMM_SM100_TIMEOUT_MS (same meaning and ranges as gemm_sm100_set_option; bad values are ignored).
struct EnvOverrides {
  static void read(const char* name, std::atomic<long>& target, long lo, long hi) {
    const char* text = std::getenv(name);
    if (!text || !*text) return;
    char* end = nullptr;
    const long v = std::strtol(text, &end, 10);
    if (end && *end == '\0' && v >= lo && v <= hi) target = v;
  }
  EnvOverrides() {
    read("GEMM_SM100_TILE_CONFIG", g_opt_tile_config, -1, kNumConfigs - 1);
    read("GEMM_SM100_SPLIT_K", g_opt_split_k, -1, 16);
    read("GEMM_SM100_GROUP_M", g_opt_group_m, 0, 4096);
    read("GEMM_SM100_MAX_CTAS", g_opt_max_ctas, 0, 1 << 20);
    read("GEMM_SM100_TIMEOUT_MS", g_opt_timeout_ms, 1, 60000);
    read("GEMM_SM100_PDL", g_opt_pdl, 0, 1);
  }
};
const EnvOverrides g_env_overrides;

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

int set_cuda_error(int* out, cudaError_t e) {
  if (out) *out = static_cast<int>(e);
  return GEMM_SM100_ERR_CUDA;
}

// Looks the driver's tensor-map encoder up once (no link-time dependency on libcuda).
int get_encoder(int* cuda_error_out) {
  if (g_encode) return GEMM_SM100_OK;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess) return set_cuda_error(cuda_error_out, e);
  if (qres != cudaDriverEntryPointSuccess || fn == nullptr)
    return set_cuda_error(cuda_error_out, cudaErrorSymbolNotFound);
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return GEMM_SM100_OK;
}

// Columns of C the TMA stores cover: whole 16-byte pieces only (the kernel writes the last N % 8
// columns with plain stores); never 0, which is not a valid extent (the map is unused then).
inline long tma_store_cols(long n) { return n >= 8 ? (n & ~7L) : 8; }

// Tensor map of a row-major 2-D array of 16-bit elements: `rows` x `cols`, pitch `ld`
// elements, box `box_rows` x 64 columns, 128-byte swizzle (64 x 2 B = one swizzle row).
// With k_sub > 1 (cols a multiple of 64) the same array is described as 3-D: 64 elements x rows x
// 64-element K blocks (128 bytes apart), box 64 x box_rows x k_sub, so that one copy brings k_sub K
// blocks of the rows, each as its own K-major tile.
int encode_2d(CUtensorMap* map, const void* base, int dtype, long rows, long cols, long ld,
              int box_rows, int* cuda_error_out, int k_sub = 1) {
  const bool blocks = k_sub > 1;
  const cuuint64_t dims[3] = {blocks ? 64u : static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows),
                              static_cast<cuuint64_t>(cols / 64)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * 2u, 128u};
  const cuuint32_t box[3] = {64u, static_cast<cuuint32_t>(box_rows), static_cast<cuuint32_t>(k_sub)};
  const cuuint32_t elem_strides[3] = {1u, 1u, 1u};
  const CUtensorMapDataType dt =
      dtype == GEMM_SM100_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = g_encode(map, dt, blocks ? 3 : 2, const_cast<void*>(base), dims, strides, box, elem_strides,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_cuda_error(cuda_error_out, cudaErrorInvalidValue);
  return GEMM_SM100_OK;
}

// Per-thread cache of encoded tensor maps.  The encoding depends only on the arguments below, so
// a caller that multiplies the same buffers again (a layer of a model, a benchmark loop) skips the
// driver's encoder: three calls of roughly a microsecond each per launch, which is most of the host
// cost of a small GEMM (the reference rebuilds all three maps on every call, gemm_test.cu:56-68).
struct MapKey {
  const void* base;
  long rows, cols, ld;
  int box_rows, dtype, k_sub;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows &&
           dtype == o.dtype && k_sub == o.k_sub;
  }
};
struct MapCache {
  static constexpr int kEntries = 32;
  MapKey keys[kEntries] = {};
  CUtensorMap maps[kEntries];
  bool used[kEntries] = {};
  unsigned next = 0;
};
thread_local MapCache t_map_cache;

int encode_2d_cached(CUtensorMap* map, const void* base, int dtype, long rows, long cols, long ld, int box_rows,
                     int* cuda_error_out, int k_sub = 1) {
  MapCache& c = t_map_cache;
  const MapKey key{base, rows, cols, ld, box_rows, dtype, k_sub};
  for (int i = 0; i < MapCache::kEntries; ++i)
    if (c.used[i] && c.keys[i] == key) {
      std::memcpy(map, &c.maps[i], sizeof(CUtensorMap));
      return GEMM_SM100_OK;
    }
  const int rc = encode_2d(map, base, dtype, rows, cols, ld, box_rows, cuda_error_out, k_sub);
  if (rc != GEMM_SM100_OK) return rc;
  const unsigned slot = c.next++ % MapCache::kEntries;
  c.keys[slot] = key;
  std::memcpy(&c.maps[slot], map, sizeof(CUtensorMap));
  c.used[slot] = true;
  return GEMM_SM100_OK;
}

int device_state(DeviceState** out, int* cuda_error_out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return set_cuda_error(cuda_error_out, e);
  if (dev < 0 || dev >= kMaxDevices) return set_cuda_error(cuda_error_out, cudaErrorInvalidDevice);
  DeviceState& st = g_dev[dev];
  if (!st.ready) {
    e = cudaDeviceGetAttribute(&st.sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return set_cuda_error(cuda_error_out, e);
    e = cudaDeviceGetAttribute(&st.cc_major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return set_cuda_error(cuda_error_out, e);
    if (st.cc_major != 10) return GEMM_SM100_ERR_UNSUPPORTED_DEVICE;
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_status_word);
    if (e != cudaSuccess) return set_cuda_error(cuda_error_out, e);
    st.status_ptr = static_cast<unsigned int*>(p);
    st.device = dev;
    // How many clusters of 2, 4 and 8 one-CTA-per-SM blocks the device holds at once (host-side
    // occupancy queries): the planner's wave count for the cluster K-split.
    {
      using Cfg = ConfigOf<2, true>;
      auto kernel = gemm_tn_kernel<Cfg, false, true>;
      if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) == cudaSuccess) {
        for (int i = 0; i < 3; ++i) {
          const unsigned size = 2u << i;
          cudaLaunchConfig_t qc = {};
          qc.gridDim = dim3(static_cast<unsigned>(st.sm_count) / size * size);
          qc.blockDim = dim3(Cfg::kThreads);
          qc.dynamicSmemBytes = Cfg::kSmemBytes;
          cudaLaunchAttribute qa[1];
          qa[0].id = cudaLaunchAttributeClusterDimension;
          qa[0].val.clusterDim.x = size;
          qa[0].val.clusterDim.y = 1;
          qa[0].val.clusterDim.z = 1;
          qc.attrs = qa;
          qc.numAttrs = 1;
          int clusters = 0;
          if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &qc) == cudaSuccess && clusters > 0)
            g_held_clusters[i] = clusters;
        }
      }
      (void)cudaGetLastError();
    }
    // No memset: a __device__ variable without an initialiser starts at zero when its module is
    // loaded, so the first call on a device issues no synchronous work (it may come while another
    // stream is being captured).
    st.ready = true;
  }
  *out = &st;
  return GEMM_SM100_OK;
}

struct Problem {
  const void* A;
  const void* B;
  void* C;
  int M, N, K;
  long lda, ldb, ldc;
  int dtype;
  bool b_is_kn = false;   // B given as [K, N] (pitch ldb >= N) instead of [N, K]
  bool a_is_km = false;   // A given as [K, M] (pitch lda >= M) instead of [M, K]
  float alpha = 1.0f;     // C = alpha * op(A) op(B) + beta * C (only the layout kernels apply them)
  float beta = 0.0f;
};

int validate(const Problem& p) {
  if (p.M < 0 || p.N < 0 || p.K < 0) return GEMM_SM100_ERR_BAD_SHAPE;
  if (p.dtype != GEMM_SM100_BF16 && p.dtype != GEMM_SM100_FP16) return GEMM_SM100_ERR_UNSUPPORTED_DTYPE;
  if (p.M == 0 || p.N == 0) return GEMM_SM100_OK;
  if (!p.C || (p.K > 0 && (!p.A || !p.B))) return GEMM_SM100_ERR_NULL_POINTER;
  if (p.K % 8 != 0) return GEMM_SM100_ERR_BAD_SHAPE;
  if (p.lda < (p.a_is_km ? p.M : p.K) || p.ldb < (p.b_is_kn ? p.N : p.K) || p.ldc < p.N)
    return GEMM_SM100_ERR_BAD_SHAPE;
  if (p.lda % 8 != 0 || p.ldb % 8 != 0 || p.ldc % 8 != 0) return GEMM_SM100_ERR_BAD_ALIGNMENT;
  if ((reinterpret_cast<uintptr_t>(p.A) | reinterpret_cast<uintptr_t>(p.B) |
       reinterpret_cast<uintptr_t>(p.C)) & 15u)
    return GEMM_SM100_ERR_BAD_ALIGNMENT;
  return GEMM_SM100_OK;
}

inline long ceil_div(long a, long b) { return (a + b - 1) / b; }

// Cost model used to choose a tile configuration: time ~ longest chain of tiles on one CTA (pair) x
// (K blocks of a tile + what a tile boundary costs) / (relative rate of the configuration).
// Fitted to interleaved timings of the configurations on B200 (tests/gemm_bench.py --ab, variants
// in rotating order; 8192^3, 8192 x 8192 x 4096, 16384^2 x 4096, 4096^3, 5120^3, the two MLP shapes):
//  * The 256 x 512 tile, whose accumulator fills TMEM, loses about 2.5 K blocks per tile because its
//    next tile cannot start before the accumulator is drained.
//  * The 256 x 256 tile loads operands only 1.04x as fast as it computes (trace counters with the
//    MMAs switched off; 1.27x for the 256 x 512 tile).  After an idle period, at the higher SM clock
//    a GPU starts with, that margin is gone: 8192^3 in bursts of 20 launches took 790 us against
//    718 us with the wide tile; in the power-capped steady state (lower SM clock, same L2) it was
//    2-4 % faster than the wide tile.  The rate below sits between the two regimes.
// So short K and chains that come out more than a few per cent longer go to the 256 x 256 tile, the
// rest to the wider one.
// Per configuration; rate 0 = not a candidate of the automatic choice (test / experiment variants).
// The 256 x 128 pair tile (7) only matters when a problem has too few tiles for anything wider:
// it moves 24 KB per K block and SM where the 128 x 128 tile moves 32 (8 % faster there).  The
// 256 x 192 tile (8) is load-bound (0.80x) and is kept for tests: balanced tilings of the two
// 256-column configurations cover its use.  Configuration 11 is 7 with two K blocks per TMA box:
// 17-25 % faster on the few-tile shapes, K % 64 == 0 only (its rate is refined in make_plan).
constexpr double kConfigRate[kNumConfigs] = {0.95, 1.0, 0.72, 0.5, 0.0, 0.0, 0.0, 0.63, 0.70, 0.80, 0.76, 0.77, 0.71, 0.62, 0.55, 0.815};
constexpr double kTileBoundaryKBlocks[kNumConfigs] = {0.0, 2.5, 0.0, 0.0, 2.5, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0};
// Store-to-every-output kernel, 256 x 512 tile: exposed epilogue time per output beyond the first,
// in K blocks of that tile.  Trace counters with all outputs in local memory (32768 x 4096 x 8192):
// the MMA issuer's wait for a free accumulator grows from 2.6 % of the loop with one output to 6.4 %
// with four and 10.8 % with eight, about 1.5 K blocks per output; with seven of eight outputs across
// NVLink (two GPUs emulating the stores of an eight-GPU run, K = 32768) the wide tile lost 8-10 % against
// the plain kernel and the 256 x 256 tile 2-5 %, about 6.5 K blocks per remote output.
constexpr double kFanoutKBlocksPerOutput = 6.5;
constexpr int kSplitKConfig = 2;                      // K-split configuration of the static-scratch entry point
// Configurations that have a K-split variant: the 256 x 512 pair tile and the 128 x 256 tile.
constexpr bool has_split_k(int config) { return config == 0 || config == 1 || config == 2 || config == 11 || config == 12; }
// Configurations whose K-split kernel also has the even split (single-width tiles).
constexpr bool has_even_split(int config) { return config == 0 || config == 2 || config == 11 || config == 12; }
// Largest even split: a tile has 16 blocks of 32 rows x 64 columns to share out among its contributors.
constexpr int kMaxEvenSplit = 16;
// Configurations with a store-to-every-output kernel (the pair tiles of the multi-GPU path).
constexpr bool has_fanout(int config) { return config == 0 || config == 1; }
// Configurations the planner may give a balanced column tiling (256-column MMAs; the others are
// special-purpose small tiles).
constexpr bool has_balanced(int config) { return config == 0 || config == 1 || config == 2; }
// Configurations with kernels for the other operand layouts and alpha / beta.
constexpr bool has_layouts(int config) { return config >= 0 && config <= 3; }
// Even split: what cutting costs per wave of units on top of the K blocks, in K blocks of the
// configuration's tile, as  fixed + per_range / ranges : measured on B200 about 6 us + 25 us / ranges
// for the 256-column tiles (partial tiles written, the wait for the other contributors, a share of the
// tile read back from every contributor and stored: the more contributors, the smaller the share) and
// 6.5 us for the 128-column tile, whose partial tiles are half as large.
constexpr double kEvenSplitFixedKBlocks[kNumConfigs] = {21.0, 0.0, 16.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 44.0, 35.0, 0.0, 0.0, 0.0};
constexpr double kEvenSplitPerRangeKBlocks[kNumConfigs] = {89.0, 0.0, 68.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0};
// The exchange's cost for the cluster K-split (2 or 4 ranges per tile, the contributors of a tile
// in one cluster, partial sums exchanged through distributed shared memory: no workspace, no
// counters, no trip through L2): 8 - 8.5 us for the 256-column tiles, 5.6 us for the 128-column one.
constexpr double kClusterSplitFixupKBlocks[kNumConfigs] = {29.0, 0.0, 23.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 38.0, 30.0, 0.0, 0.0, 0.0};

// Clusters of `cluster_ctas` CTAs (one CTA per SM) the device holds at once: a cluster sits inside
// one GPC, and a GPC of this generation has about 18 SMs.
inline long resident_clusters(int sm_count, int cluster_ctas) {
  // what the occupancy query said for this process's device (filled with the device state)
  const int index = cluster_ctas == 2 ? 0 : (cluster_ctas == 4 ? 1 : (cluster_ctas == 8 ? 2 : -1));
  if (index >= 0 && g_held_clusters[index].load() > 0) return g_held_clusters[index].load();
  const int gpcs = sm_count >= 36 ? sm_count / 18 : 1;
  const int per_gpc = sm_count / gpcs;
  const long n = static_cast<long>(gpcs) * (per_gpc / cluster_ctas);
  return n > 0 ? n : 1;
}

struct Plan {
  int config = 0;
  // Column tiling (TileParams::bal_q / bal_rem): tiles_n tiles per tile row; 0 = uniform tiles.
  int tiles_n = 0, bal_q = 0, bal_rem = 0, bal_start = 0;
  bool split_k = false;
  int ctas = 0;              // grid size
  size_t flag_bytes = 0;     // K-split: arrival counters (one per CTA), padded to 256 bytes
  size_t partial_bytes = 0;  // K-split: one fp32 partial tile per CTA
  int partial_rows = 128;    // K-split: rows kept per partial tile
  int split_factor = 0;      // K-split: > 1 = every tile cut into this many equal K ranges
  bool cluster = false;      // even split whose contributors form a cluster and exchange partial sums in shared memory
};

inline int grid_cap(const ConfigInfo& c, int sm_count) {
  long cap = sm_count - sm_count % c.cta_group;
  if (g_opt_max_ctas > 0 && g_opt_max_ctas < cap) cap = g_opt_max_ctas - g_opt_max_ctas % c.cta_group;
  if (cap < c.cta_group) cap = c.cta_group;
  return static_cast<int>(cap);
}

// Host mirror of the kernel's tile_coords(): column-tile index of tile `t`.
inline int n_tile_of(long t, int m_tiles, int n_tiles, int group_m) {
  const long per_group = static_cast<long>(group_m) * n_tiles;
  const long group = t / per_group;
  const long in_group = t - group * per_group;
  const long first_m = group * group_m;
  const long rows = (m_tiles - first_m) < group_m ? (m_tiles - first_m) : group_m;
  return static_cast<int>(in_group / rows);
}

inline int default_group_m(int m_tiles) {
  return g_opt_group_m.load() > 0 ? static_cast<int>(g_opt_group_m.load()) : (m_tiles >= 16 ? 16 : 8);
}

// What one K block of a tile of `width` columns costs, in columns of a full-rate tile: the MMAs
// take time in proportion to the width, the operand loads (A tile + this CTA's share of B) in
// proportion to their bytes, and the SM gets about 63 bytes per clock from L2 when every SM is
// pulling (trace counters with the MMAs switched off: the 256 x 256 pair tile loads 1.04x as fast
// as it computes, the 256 x 192 tile only 0.80x).  Normalised so that the configuration's full
// tile costs its own width (its measured rate is in kConfigRate).
double effective_width(const ConfigInfo& c, int width) {
  const int full = c.mma_n * c.halves;
  auto cycles = [&](int w) {
    const double mma = 2.0 * w;                                              // 4 MMAs of w / 2 cycles
    const double load = (128.0 * 64 * 2 + static_cast<double>(w) / c.cta_group * 64 * 2) / 63.0;
    return mma > load ? mma : load;
  };
  return cycles(width) / cycles(full) * full;
}

// Longest chain of work any CTA (pair) gets under the static persistent schedule, for `tiles_n`
// tiles per tile row dealt as the kernel deals them; in effective columns.
double schedule_cost(const ConfigInfo& c, int m_tiles, int tiles_n, int q, int rem, int start, long slots) {
  const long tiles = static_cast<long>(m_tiles) * tiles_n;
  const long clusters = tiles < slots ? tiles : slots;
  const int group_m = default_group_m(m_tiles);
  const double wide = effective_width(c, (q + 1) * 64), narrow = effective_width(c, q * 64);
  double worst = 0.0;
  for (long cl = 0; cl < clusters; ++cl) {
    double sum = 0.0;
    for (long t = cl; t < tiles; t += clusters)
    {
      const int d = n_tile_of(t, m_tiles, tiles_n, group_m) - start;
      sum += (d >= 0 && d < rem) ? wide : narrow;
    }
    if (sum > worst) worst = sum;
  }
  return worst;
}

// The K-split schedule gives every CTA the same number of K blocks; it pays when whole tiles
// quantise badly over the SMs (few tiles, as in the memory-bound small-M shapes) and K is long.
Plan make_plan(int M, int N, int K, int sm_count, bool allow_split = true, int config_limit = kNumConfigs,
               bool allow_balance = true) {
  Plan best;
  double best_cost = 1e300;
  const long k_blocks = ceil_div(K, 64);
  // A forced configuration that cannot take this problem (more rows than its A tile holds) is
  // ignored: the automatic choice runs instead.
  const long forced_index = g_opt_tile_config.load();
  const bool forced_config = forced_index >= 0 && forced_index < kNumConfigs && forced_index < config_limit &&
                             (kConfigs[forced_index].a_rows >= 128 || M <= kConfigs[forced_index].a_rows) &&
                             (kConfigs[forced_index].k_sub == 1 || K % 64 == 0);
  const int first = forced_config ? static_cast<int>(forced_index) : 0;
  const int last = forced_config ? first + 1 : config_limit;   // config_limit: callers whose kernels exist for the first few configurations only
  for (int i = first; i < last; ++i) {
    const ConfigInfo& c = kConfigs[i];
    if (c.a_rows < 128 && M > c.a_rows) continue;        // few-row configurations: only what their A tile holds
    if (c.k_sub > 1 && K % 64 != 0) continue;           // whole 64-element K blocks only (nothing bounds K inside a block)
    const int block_n = c.mma_n * c.halves;
    const long tiles = ceil_div(M, 128L * c.cta_group) * ceil_div(N, block_n);
    // The 64-column few-row tiles stream B well only when most SMs have one (16 x 8192 x 8192: 27.5 us
    // against 29.8 for the wider tile cut along K; 64 x 6144 x 4096: 14.2 against 18.6; but 16 x 4096 x 8192,
    // 64 tiles: 24.0 against 18.2).
    if (c.k_sub == 4 && !forced_config && tiles < 96) continue;
    const int cap = grid_cap(c, sm_count);
    const long slots = cap / c.cta_group;
    const long waves = ceil_div(tiles, slots);
    if (!forced_config && kConfigRate[i] <= 0.0) continue;
    double rate = kConfigRate[i] > 0.0 ? kConfigRate[i] : 1.0;
    // The 256 x 128 tile with two K blocks per box: 1.2x configuration 7 when every SM is pulling
    // operands (64 tiles), 1.33x with 32 tiles or fewer (1024 x 1024 x 4096: 15.6 against 20.7 us).
    if (c.k_sub == 2 && c.cta_group == 2 && tiles <= 32) rate = 0.88;
    // A pair tile spends its second CTA on rows that do not exist when M <= 128 (and streams B in
    // boxes of 64 rows): 128 x 8192 x 8192 took 43 us that way, 34.5 us with the 128-row tile cut along K.
    if (c.cta_group == 2 && c.mma_n == 128 && M <= 128) rate *= 0.6;
    // The 128 x 128 tile with two K blocks per box pays for problems of 65-128 rows (128 x 4096 x 8192: 19.7 us
    // cut in four against 22.3 us for the 128 x 256 tile cut in nine); with fewer rows the wider tile's
    // smaller partial tiles win (64 x 4096 x 8192: 20.5 against 19.8 us, 16 x 4096 x 8192: 20.7 against 18.2).
    if (c.cta_group == 1 && c.k_sub == 2 && c.mma_n == 128 && M <= 64) rate *= 0.65;
    Plan cand;
    cand.config = i;
    cand.ctas = static_cast<int>((tiles < slots ? tiles : slots) * c.cta_group);
    // costs in units of (one K block of one tile column) per CTA
    const double boundary = kTileBoundaryKBlocks[i];
    double cost = static_cast<double>(waves) * block_n * (k_blocks + boundary) / rate;
    // Balanced column tiling (whole tiles only): another number of tiles per tile row, the
    // chunks of 64 columns dealt evenly, when the static schedule's longest chain gets shorter
    // by more than 2 %.  Skipped for problems of many waves, where quantisation costs little.
    if (allow_balance && g_opt_balance.load() != 0 && has_balanced(i) && (waves <= 24 || g_opt_tiles_n.load() > 0) && N >= 64) {
      const int m_tiles = static_cast<int>(ceil_div(M, 128L * c.cta_group));
      const int chunks = static_cast<int>(ceil_div(N, 64));
      const int q_full = block_n / 64;
      // No MMA narrower than 192 columns: the 192-wide pair MMA still runs at the full tensor rate
      // (0.99 in the trace counters with loads switched off), the 128-wide one does not, and
      // few-tile problems are better off with the small-tile configurations and their deeper rings.
      // So single-width tiles are 192 or 256 wide, double-width ones 448 or 512.
      const int q_min = c.halves == 2 ? c.mma_n / 64 + 3 : 3;
      const int t_uniform = static_cast<int>(ceil_div(chunks, q_full));
      int t_last = chunks / q_min;
      if (t_last > 2 * t_uniform + 2) t_last = 2 * t_uniform + 2;
      double best_chain = static_cast<double>(waves) * block_n;
      // A single tile row (the memory-bound few-row shapes) keeps uniform tiles unless forced: 148
      // tiles of 192 columns on 148 SMs measured 14 % slower than 112 tiles of 256 on 112 SMs
      // (more, narrower row streams; the loop of the 112 is already at the DRAM's read rate).
      const bool single_row = m_tiles == 1;
      const int forced_t = static_cast<int>(g_opt_tiles_n.load());
      for (int t_n = t_uniform; (t_n <= t_last && !single_row) || forced_t > 0; ++t_n) {
        if (forced_t > 0) t_n = forced_t;
        const int q = chunks / t_n, rem = chunks % t_n;
        if (forced_t > 0) {
          if (t_n <= chunks && q >= q_min && q + (rem ? 1 : 0) <= q_full) {
            best_chain = schedule_cost(c, m_tiles, t_n, q, rem, 0, slots);
            cand.tiles_n = t_n, cand.bal_q = q, cand.bal_rem = rem, cand.bal_start = 0;
          }
          break;
        }
        if (q < q_min || q + (rem ? 1 : 0) > q_full) continue;
        if (static_cast<long>(m_tiles) * t_n > 40000) break;
        // where in the tile row the wider tiles sit decides which CTAs get two of them: first,
        // middle or last, whichever leaves the shortest chain
        const int starts[3] = {0, (t_n - rem) / 2, t_n - rem};
        for (int si = 0; si < (rem ? 3 : 1); ++si) {
          const double chain = schedule_cost(c, m_tiles, t_n, q, rem, starts[si], slots);
          if (chain < best_chain * 0.98) {
            best_chain = chain;
            cand.tiles_n = t_n;
            cand.bal_q = q;
            cand.bal_rem = rem;
            cand.bal_start = starts[si];
          }
        }
      }
      if (cand.tiles_n > 0) {
        const long bal_tiles = static_cast<long>(m_tiles) * cand.tiles_n;
        cand.ctas = static_cast<int>((bal_tiles < slots ? bal_tiles : slots) * c.cta_group);
        cost = best_chain * (k_blocks + boundary) / rate;
      }
    }
    const long units = tiles * k_blocks;
    // K-split.  Forced (split_k = 1): as many ranges as CTA (pair)s.  Automatic: the 128 x 256
    // tile only, when whole tiles would leave more than half of the SMs idle, with the number of
    // ranges that minimises   K blocks per range / rate + 7 x ranges per tile + 20   (in K blocks
    // of this tile).  The terms, fitted to timings of 128..1024 x 256..4096 x 4096..65536 on B200:
    // the owner of a cut tile sums its contributors' fp32 partial tiles alone (about 7 K blocks'
    // worth of time each), and a cut launch costs about 20 K blocks more than a whole one (counters
    // zeroed by a memset node, partial tiles written, accumulator drains).  CTAs that work on the
    // same operand panel at different K offsets no longer fetch it together, so operands beyond
    // what L2 holds are charged as DRAM traffic (2048 x 2048 x 8192 with the 256 x 512 tile: 92 us
    // cut against 53 us whole).  For 4096^3 (1.73 waves) cutting took 111 us against 95 us: a bad
    // wave count alone never selects it.
    const bool forced_split = g_opt_split_k > 0;
    long ranges = units < slots ? units : slots;
    double split_cost = static_cast<double>(units) / ranges * block_n / rate + 9.0 * block_n;
    bool auto_split = false;
    if (!forced_split && g_opt_split_k < 0 && i == kSplitKConfig && tiles * 2 <= slots) {
      long r = static_cast<long>(std::sqrt(static_cast<double>(units) * tiles / 5.0) + 0.5);
      if (r > slots) r = slots;
      if (r > units / 4) r = units / 4;                      // at least four K blocks per range
      if (r >= 2 * tiles) {
        const double operand_bytes = 2.0 * (static_cast<double>(M) + N) * K;
        const double miss = operand_bytes > 48e6 ? 1.0 - 48e6 / operand_bytes : 0.0;
        double stream = static_cast<double>(units) / r / rate;
        const double dram = static_cast<double>(units) * 0.0204 * miss;
        if (dram > stream) stream = dram;
        ranges = r;
        split_cost = (stream + 7.0 * r / tiles + 20.0) * block_n;
        auto_split = split_cost < cost;
        split_cost *= 1.15;                                  // the fit is good to about 10 %: ties go to whole tiles
      }
    }
    const bool can_split = allow_split && has_split_k(i) && units >= 2 && c.k_sub == 1;   // contiguous ranges: 64-element K blocks only
    // Even split: every tile cut into s equal K ranges, the reduction spread over the contributors.
    // Forced with split_k = s (2..16); automatic when it beats whole tiles and the contiguous ranges.
    int even_s = 0;
    bool even_cluster = false;
    double even_cost = 1e300;
    if (allow_split && has_even_split(i) && g_opt_split_k != 0 && g_opt_split_k != 1) {
      const long sk_cluster = g_opt_sk_cluster.load();
      double best_score = 1e300;
      auto consider = [&](int f, bool cluster, long waves_f, double fixup) {
        const double c_f = static_cast<double>(waves_f) * (static_cast<double>(k_blocks) / f + boundary + fixup) * block_n / rate;
        if (c_f < best_score) {
          best_score = c_f;
          even_cost = c_f;
          even_s = f;
          even_cluster = cluster;
        }
      };
      for (int f = 2; f <= kMaxEvenSplit; ++f) {
        if (g_opt_split_k > 1 && f != g_opt_split_k) continue;
        if (f > slots || k_blocks < 8L * f || tiles * f > 0x3fffffff / 64) continue;
        if (f > 4 * (c.mma_n / 64)) continue;               // a contributor's share is at least one 32 x 64 block
        // in a cluster a share is made of whole 64-column chunks, or (twice as many contributors as
        // chunks) of one chunk of one half of the rows
        const int chunks = c.mma_n / 64;
        const bool cluster_ok = (f == 2 || f == 4) && (chunks % f == 0 || f == 2 * chunks);
        if (sk_cluster != 1 || !cluster_ok)
          consider(f, false, ceil_div(tiles * f, slots), kEvenSplitFixedKBlocks[i] + kEvenSplitPerRangeKBlocks[i] / f);
        // 2 or 4 contributors per tile: clusters of up to 8 CTAs, and every chunk that leaves a CTA has
        // a staging slot of its own in shared memory; one unit per CTA (pair), as many waves of
        // clusters as that takes
        if (sk_cluster != 0 && cluster_ok && tiles * f * c.cta_group <= 65535) {
          // only the 32-row groups that exist are exchanged: with few rows the exchange is mostly its
          // fixed part (16 x 8192 x 8192 cut in four: 29.4 us, 33.6 us when all 128 rows were sent)
          const double live = M >= 128 ? 1.0 : 0.4 + 0.15 * static_cast<double>(ceil_div(M, 32));
          consider(f, true, ceil_div(tiles, resident_clusters(sm_count, f * c.cta_group)), kClusterSplitFixupKBlocks[i] * live);
        }
      }
    }
    const double best_other = (can_split && auto_split) ? split_cost : cost;
    if (even_s > 0 && (g_opt_split_k > 1 || even_cost < best_other)) {
      const long even_units = tiles * even_s;
      cost = even_cost * 1.1;                                // ties go to the simpler schedule
      cand.tiles_n = cand.bal_q = cand.bal_rem = 0;          // cut tiles are uniform
      cand.split_k = true;
      cand.split_factor = even_s;
      cand.ctas = static_cast<int>((even_units < slots ? even_units : slots) * c.cta_group);
      cand.partial_rows = M < 128 ? static_cast<int>((M + 31) / 32 * 32) : 128;
      cand.flag_bytes = (static_cast<size_t>(tiles) * c.cta_group * sizeof(unsigned int) + 255) / 256 * 256;
      cand.partial_bytes = static_cast<size_t>(even_units) * c.cta_group * cand.partial_rows * block_n * sizeof(float);
      if (even_cluster) {
        cand.cluster = true;
        cand.ctas = static_cast<int>(even_units * c.cta_group);
        cand.flag_bytes = cand.partial_bytes = 0;            // nothing goes through global memory
      }
    } else if (can_split && (g_opt_split_k == 1 || auto_split)) {
      cost = split_cost;
      cand.tiles_n = cand.bal_q = cand.bal_rem = 0;
      cand.split_k = true;
      cand.ctas = static_cast<int>(ranges * c.cta_group);
      cand.partial_rows = M < 128 ? static_cast<int>((M + 31) / 32 * 32) : 128;
      cand.flag_bytes = (static_cast<size_t>(cand.ctas) * sizeof(unsigned int) + 255) / 256 * 256;
      cand.partial_bytes = static_cast<size_t>(cand.ctas) * cand.partial_rows * block_n * sizeof(float);
    }
    if (cost < best_cost) {
      best_cost = cost;
      best = cand;
    }
  }
  return best;
}

// Per-thread cache of plans: the binding asks for the workspace size and then launches, and callers
// repeat shapes, so the cost model runs once per (shape, option state).
Plan plan_for(int M, int N, int K, int sm_count, bool allow_split = true, int config_limit = kNumConfigs,
              bool allow_balance = true) {
  struct Entry {
    int M = -1, N = 0, K = 0, sm = 0, limit = 0;
    bool allow = false, balance = false;
    unsigned generation = 0;
    Plan plan;
  };
  constexpr int kEntries = 16;
  thread_local Entry cache[kEntries];
  thread_local unsigned next = 0;
  const unsigned generation = g_opt_generation.load(std::memory_order_acquire);
  for (int i = 0; i < kEntries; ++i) {
    const Entry& e = cache[i];
    if (e.M == M && e.N == N && e.K == K && e.sm == sm_count && e.limit == config_limit && e.allow == allow_split &&
        e.balance == allow_balance && e.generation == generation)
      return e.plan;
  }
  Entry& e = cache[next++ % kEntries];
  e.M = M, e.N = N, e.K = K, e.sm = sm_count, e.limit = config_limit, e.allow = allow_split;
  e.balance = allow_balance;
  e.generation = generation;
  e.plan = make_plan(M, N, K, sm_count, allow_split, config_limit, allow_balance);
  return e.plan;
}

// Tile counts, rasterisation and wait limit of one launch (everything that does not depend on
// the schedule variant).
template <class Cfg>
TileParams base_tile_params(const Problem& p, const DeviceState& st) {
  TileParams tp;
  tp.M = p.M;
  tp.N = p.N;
  tp.K = p.K;
  tp.m_tiles = static_cast<int>(ceil_div(p.M, 128L * Cfg::kCtaGroup));
  tp.n_tiles = static_cast<int>(ceil_div(p.N, Cfg::kBlockN));
  tp.k_blocks = static_cast<int>(ceil_div(p.K, Cfg::kBlockK));
  // Rasterisation group: 16 tile rows when the problem has that many (measured best from 8192
  // to 32768 rows: the A panel of a group is reused by more B tiles), else 8.
  tp.group_m = default_group_m(tp.m_tiles);
  tp.bal_q = Cfg::kBlockN / 64;
  tp.bal_rem = 0;
  tp.bal_start = 0;
  tp.b_box_rows = Cfg::kBRows;
  tp.early_prefetch = (g_opt_pdl.load() != 0 && g_opt_early_prefetch.load() != 0) ? 1 : 0;
  tp.status = st.status_ptr;
  tp.timeout_ns = static_cast<unsigned long long>(g_opt_timeout_ms.load()) * 1000000ull;
  tp.trace = nullptr;
  tp.debug_flags = 0;
  tp.sk_flags = nullptr;
  tp.sk_partials = nullptr;
  tp.sk_rows = 128;
  tp.sk_factor = 0;
  tp.sk_cluster = 0;
  tp.k_rotate = 0;
  tp.alpha = p.alpha;
  tp.beta = p.beta;
  tp.c_ptr = p.C;
  tp.ldc = p.ldc;
  return tp;
}

// Order of a tile's K blocks (TileParams::k_rotate) for this problem under the "k_rotate" option.
// Automatic (-1): rotation only in the memory-bound few-row regime (at most 128 rows, thousands of
// columns).  Other problems keep K ascending, so that the same rows give the same bits whether
// they are computed in one call or in row panels, and in every operand layout.
int k_order_for(const Problem& p, bool split_k) {
  const long k_order = g_opt_k_rotate.load();
  const bool few_rows = p.M <= 128 && p.N >= 2048 && !split_k;
  return k_order == 2 ? 2 : ((k_order == 1 || (k_order < 0 && few_rows)) ? 1 : 0);
}

// Cluster launch of `kernel` on `ctas` CTAs of Cfg::kThreads threads.
template <class Cfg, class Kernel, class... Args>
cudaError_t launch_kernel(Kernel kernel, long ctas, int cluster_ctas, cudaStream_t stream, const Args&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(ctas));
  cfg.blockDim = dim3(Cfg::kThreads);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  unsigned n = 0;
  if (cluster_ctas > 1) {                              // single-CTA tiles are launched without a cluster
    attrs[n].id = cudaLaunchAttributeClusterDimension;
    attrs[n].val.clusterDim.x = static_cast<unsigned>(cluster_ctas);
    attrs[n].val.clusterDim.y = 1;
    attrs[n].val.clusterDim.z = 1;
    ++n;
  }
  if (g_opt_pdl.load() != 0) {
    // Programmatic dependent launch: this kernel's CTAs may be scheduled while the previous kernel
    // of the stream drains (if that kernel allows it, as these kernels do at their start); they
    // set up barriers and tensor memory and then wait for it to complete before touching global
    // memory.  Back-to-back GEMMs lose a few microseconds less between launches.
    attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// One-time set-up of a tile configuration on a device: the dynamic shared-memory limit of every
// instantiation that can be launched for it, and how many CTAs of it are co-resident.
template <int kCfgIndex, bool kIsBf16>
int ensure_config(DeviceState& st, int* cuda_error_out) {
  constexpr ConfigInfo ci = kConfigs[kCfgIndex];
  using Cfg = ConfigOf<kCfgIndex, kIsBf16>;
  constexpr int dt = kIsBf16 ? 0 : 1;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (st.attr_set[kCfgIndex][dt]) return GEMM_SM100_OK;
  cudaError_t e = cudaFuncSetAttribute(gemm_tn_kernel<Cfg, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       Cfg::kSmemBytes);
  if (e != cudaSuccess) return set_cuda_error(cuda_error_out, e);
  e = cudaFuncSetAttribute(gemm_tn_kernel<Cfg, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
  if (e != cudaSuccess) return set_cuda_error(cuda_error_out, e);
  if constexpr (has_split_k(kCfgIndex)) {
    e = cudaFuncSetAttribute(gemm_tn_kernel<Cfg, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg::kSmemBytes);
    if (e != cudaSuccess) return set_cuda_error(cuda_error_out, e);
    e = cudaFuncSetAttribute(gemm_tn_kernel<Cfg, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg::kSmemBytes);
    if (e != cudaSuccess) return set_cuda_error(cuda_error_out, e);
  }
  if constexpr (has_fanout(kCfgIndex)) {
    e = cudaFuncSetAttribute(gemm_tn_fanout_kernel<Cfg, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg::kSmemBytes);
    if (e != cudaSuccess) return set_cuda_error(cuda_error_out, e);
    e = cudaFuncSetAttribute(gemm_tn_fanout_kernel<Cfg, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg::kSmemBytes);
    if (e != cudaSuccess) return set_cuda_error(cuda_error_out, e);
  }
  if constexpr (has_layouts(kCfgIndex)) {
    for (auto k : {gemm_layout_kernel<Cfg, true, true>, gemm_layout_kernel<Cfg, true, false>,
                   gemm_layout_kernel<Cfg, false, true>, gemm_layout_kernel<Cfg, false, false>}) {
      e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
      if (e != cudaSuccess) return set_cuda_error(cuda_error_out, e);
    }
  }
  int max_ctas = st.sm_count;
  if (Cfg::kCtaGroup == 1) {
    // Persistent grid of single CTAs: what the device can hold at once (one CTA per SM with this
    // much shared memory).  The K-split schedules rely on the whole grid being resident.
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemm_tn_kernel<Cfg, false>, Cfg::kThreads,
                                                      Cfg::kSmemBytes);
    if (e != cudaSuccess) return set_cuda_error(cuda_error_out, e);
    if (per_sm < 1) return set_cuda_error(cuda_error_out, cudaErrorLaunchOutOfResources);
    const long resident = static_cast<long>(per_sm) * st.sm_count;
    if (resident < max_ctas) max_ctas = static_cast<int>(resident);
  }
  if (Cfg::kCtaGroup == 2) {
    cudaLaunchConfig_t qc = {};
    qc.gridDim = dim3(st.sm_count - st.sm_count % 2);
    qc.blockDim = dim3(Cfg::kThreads);
    qc.dynamicSmemBytes = Cfg::kSmemBytes;
    cudaLaunchAttribute qa[1];
    qa[0].id = cudaLaunchAttributeClusterDimension;
    qa[0].val.clusterDim.x = 2;
    qa[0].val.clusterDim.y = 1;
    qa[0].val.clusterDim.z = 1;
    qc.attrs = qa;
    qc.numAttrs = 1;
    int clusters = 0;
    e = cudaOccupancyMaxActiveClusters(&clusters, gemm_tn_kernel<Cfg, false>, &qc);
    if (e != cudaSuccess) return set_cuda_error(cuda_error_out, e);
    if (clusters < 1) return set_cuda_error(cuda_error_out, cudaErrorLaunchOutOfResources);
    max_ctas = 2 * clusters;
    if (max_ctas > st.sm_count) max_ctas = st.sm_count - st.sm_count % 2;
  }
  st.max_ctas[kCfgIndex][dt] = max_ctas;
  st.attr_set[kCfgIndex][dt] = true;
  return GEMM_SM100_OK;
}

template <int kCfgIndex, bool kIsBf16>
int launch_config(const Problem& p, const Plan& plan, void* workspace, DeviceState& st, cudaStream_t stream,
                  int* cuda_error_out) {
  constexpr ConfigInfo ci = kConfigs[kCfgIndex];
  using Cfg = ConfigOf<kCfgIndex, kIsBf16>;
  constexpr int dt = kIsBf16 ? 0 : 1;
  int rc = ensure_config<kCfgIndex, kIsBf16>(st, cuda_error_out);
  if (rc) return rc;
  // The instrumented instantiation runs only while a trace buffer (of this device) or an
  // experiment flag is set.
  const TraceBuffer trace = trace_for_device(st.device);
  const bool debug = trace.ptr != nullptr || g_opt_debug_flags.load() != 0;
  auto kernel = debug ? gemm_tn_kernel<Cfg, true> : gemm_tn_kernel<Cfg, false>;
  if constexpr (has_split_k(kCfgIndex)) {
    if (plan.split_k) kernel = (trace.ptr && plan.cluster) ? gemm_tn_kernel<Cfg, true, true> : gemm_tn_kernel<Cfg, false, true>;
  }
  cudaError_t e;

  TileParams tp = base_tile_params<Cfg>(p, st);
  int b_box = Cfg::kBRows;
  if (plan.tiles_n > 0) {
    tp.n_tiles = plan.tiles_n;
    tp.bal_q = plan.bal_q;
    tp.bal_rem = plan.bal_rem;
    tp.bal_start = plan.bal_start;
    b_box = 64 / Cfg::kCtaGroup;          // tile widths are multiples of 64 columns: this CTA's share of them
    tp.b_box_rows = b_box;
  }
  tp.debug_flags = static_cast<unsigned int>(g_opt_debug_flags.load());
  tp.k_rotate = k_order_for(p, plan.split_k);
  if (plan.split_k && plan.cluster) {
    tp.sk_factor = plan.split_factor;
    tp.sk_cluster = 1;
  } else if (plan.split_k) {
    tp.sk_flags = static_cast<unsigned int*>(workspace);
    tp.sk_partials = reinterpret_cast<float*>(static_cast<char*>(workspace) + plan.flag_bytes);
    tp.sk_rows = plan.partial_rows;
    tp.sk_factor = plan.split_factor;
    // The even split's counters return to zero by themselves; a registered workspace that was left
    // by such a launch needs no memset (and the kernel can then overlap the previous one's tail).
    if (kept_workspace_needs_zeroing(workspace, plan.flag_bytes, plan.split_factor > 1)) {
      e = cudaMemsetAsync(tp.sk_flags, 0, plan.flag_bytes, stream);
      if (e != cudaSuccess) return set_cuda_error(cuda_error_out, e);
    }
  }

  CUtensorMap map_a, map_b, map_c;
  rc = encode_2d_cached(&map_a, p.A, p.dtype, p.M, p.K, p.lda, Cfg::kARows, cuda_error_out, Cfg::kKSub);
  if (rc) return rc;
  rc = encode_2d_cached(&map_b, p.B, p.dtype, p.N, p.K, p.ldb, b_box, cuda_error_out, Cfg::kKSub);
  if (rc) return rc;
  rc = encode_2d_cached(&map_c, p.C, p.dtype, p.M, tma_store_cols(p.N), p.ldc, 32, cuda_error_out);
  if (rc) return rc;

  long ctas = plan.ctas;
  if (ctas > st.max_ctas[kCfgIndex][dt] && !plan.cluster) {   // (the cluster split runs in as many waves as it takes)
    // Fewer co-resident CTAs than SMs (never seen on B200).  The K-split schedule needs the
    // grid it was planned for, because the workspace is indexed by CTA.
    if (plan.split_k) return set_cuda_error(cuda_error_out, cudaErrorLaunchOutOfResources);
    ctas = st.max_ctas[kCfgIndex][dt];
  }
  if (trace.ptr && trace.bytes >= static_cast<size_t>(ctas) * kTraceWords * sizeof(unsigned long long))
    tp.trace = trace.ptr;

  e = launch_kernel<Cfg>(kernel, ctas, plan.cluster ? plan.split_factor * Cfg::kCtaGroup : Cfg::kCtaGroup, stream, map_a, map_b,
                          map_c, tp);
  if (e != cudaSuccess) return set_cuda_error(cuda_error_out, e);
  return GEMM_SM100_OK;
}

// Launch of the store-to-every-output variant (pair-tile configurations 0 and 1 only).
template <int kCfgIndex, bool kIsBf16>
int launch_fanout(const Problem& p, void* const* outputs, int num_outputs, DeviceState& st, cudaStream_t stream,
                  int* cuda_error_out) {
  constexpr ConfigInfo ci = kConfigs[kCfgIndex];
  using Cfg = ConfigOf<kCfgIndex, kIsBf16>;
  static_assert(has_fanout(kCfgIndex), "no store-to-every-output variant of this configuration");
  constexpr int dt = kIsBf16 ? 0 : 1;
  int rc = ensure_config<kCfgIndex, kIsBf16>(st, cuda_error_out);
  if (rc) return rc;
  const TraceBuffer trace = trace_for_device(st.device);
  auto kernel = trace.ptr ? gemm_tn_fanout_kernel<Cfg, true> : gemm_tn_fanout_kernel<Cfg, false>;
  TileParams tp = base_tile_params<Cfg>(p, st);

  CUtensorMap map_a, map_b;
  OutputMaps out;
  std::memset(&out, 0, sizeof(out));
  rc = encode_2d_cached(&map_a, p.A, p.dtype, p.M, p.K, p.lda, Cfg::kBlockM, cuda_error_out);
  if (rc) return rc;
  rc = encode_2d_cached(&map_b, p.B, p.dtype, p.N, p.K, p.ldb, Cfg::kBRows, cuda_error_out);
  if (rc) return rc;
  for (int d = 0; d < num_outputs; ++d) {
    rc = encode_2d_cached(&out.maps[d], outputs[d], p.dtype, p.M, p.N, p.ldc, 32, cuda_error_out);
    if (rc) return rc;
  }
  long ctas = static_cast<long>(tp.m_tiles) * tp.n_tiles * Cfg::kCtaGroup;
  const long cap = grid_cap(ci, st.sm_count);
  if (ctas > cap) ctas = cap;
  if (ctas > st.max_ctas[kCfgIndex][dt]) ctas = st.max_ctas[kCfgIndex][dt];
  if (trace.ptr && trace.bytes >= static_cast<size_t>(ctas) * kTraceWords * sizeof(unsigned long long))
    tp.trace = trace.ptr;

  cudaError_t e = launch_kernel<Cfg>(kernel, ctas, Cfg::kCtaGroup, stream, map_a, map_b, out, num_outputs, tp);
  if (e != cudaSuccess) return set_cuda_error(cuda_error_out, e);
  return GEMM_SM100_OK;
}

// Launch of the variants with B as [K,N] and / or A as [K,M] (whole tiles only: no K-split, no
// trace instantiation).
template <int kCfgIndex, bool kIsBf16>
int launch_nn(const Problem& p, const Plan& plan, DeviceState& st, cudaStream_t stream, int* cuda_error_out) {
  constexpr ConfigInfo ci = kConfigs[kCfgIndex];
  using Cfg = ConfigOf<kCfgIndex, kIsBf16>;
  static_assert(has_layouts(kCfgIndex), "no layout variants of this configuration");
  auto kernel = p.a_is_km ? (p.b_is_kn ? gemm_layout_kernel<Cfg, true, true> : gemm_layout_kernel<Cfg, true, false>)
                          : (p.b_is_kn ? gemm_layout_kernel<Cfg, false, true> : gemm_layout_kernel<Cfg, false, false>);
  int rc = ensure_config<kCfgIndex, kIsBf16>(st, cuda_error_out);
  if (rc) return rc;
  TileParams tp = base_tile_params<Cfg>(p, st);
  tp.k_rotate = k_order_for(p, false);
  CUtensorMap map_a, map_b, map_c;
  rc = p.a_is_km ? encode_2d_cached(&map_a, p.A, p.dtype, p.K, p.M, p.lda, 64, cuda_error_out)   // K rows of M columns
                 : encode_2d_cached(&map_a, p.A, p.dtype, p.M, p.K, p.lda, Cfg::kBlockM, cuda_error_out);
  if (rc) return rc;
  rc = p.b_is_kn ? encode_2d_cached(&map_b, p.B, p.dtype, p.K, p.N, p.ldb, 64, cuda_error_out)   // K rows of N columns
                 : encode_2d_cached(&map_b, p.B, p.dtype, p.N, p.K, p.ldb, Cfg::kBRows, cuda_error_out);
  if (rc) return rc;
  rc = encode_2d_cached(&map_c, p.C, p.dtype, p.M, tma_store_cols(p.N), p.ldc, 32, cuda_error_out);
  if (rc) return rc;
  const cudaError_t e = launch_kernel<Cfg>(kernel, plan.ctas, Cfg::kCtaGroup, stream, map_a, map_b, map_c, tp);
  if (e != cudaSuccess) return set_cuda_error(cuda_error_out, e);
  return GEMM_SM100_OK;
}

template <bool kIsBf16>
int dispatch_nn(const Plan& plan, const Problem& p, DeviceState& st, cudaStream_t stream, int* cuda_error_out) {
  switch (plan.config) {
    case 0: return launch_nn<0, kIsBf16>(p, plan, st, stream, cuda_error_out);
    case 1: return launch_nn<1, kIsBf16>(p, plan, st, stream, cuda_error_out);
    case 2: return launch_nn<2, kIsBf16>(p, plan, st, stream, cuda_error_out);
    case 3: return launch_nn<3, kIsBf16>(p, plan, st, stream, cuda_error_out);
    default: return GEMM_SM100_ERR_BAD_OPTION;
  }
}

template <bool kIsBf16>
int dispatch(const Plan& plan, const Problem& p, void* ws, DeviceState& st, cudaStream_t stream, int* cuda_error_out) {
  switch (plan.config) {
    case 0: return launch_config<0, kIsBf16>(p, plan, ws, st, stream, cuda_error_out);
    case 1: return launch_config<1, kIsBf16>(p, plan, ws, st, stream, cuda_error_out);
    case 2: return launch_config<2, kIsBf16>(p, plan, ws, st, stream, cuda_error_out);
    case 3: return launch_config<3, kIsBf16>(p, plan, ws, st, stream, cuda_error_out);
    case 4: return launch_config<4, kIsBf16>(p, plan, ws, st, stream, cuda_error_out);
    case 5: return launch_config<5, kIsBf16>(p, plan, ws, st, stream, cuda_error_out);
    case 6: return launch_config<6, kIsBf16>(p, plan, ws, st, stream, cuda_error_out);
    case 7: return launch_config<7, kIsBf16>(p, plan, ws, st, stream, cuda_error_out);
    case 8: return launch_config<8, kIsBf16>(p, plan, ws, st, stream, cuda_error_out);
    case 9: return launch_config<9, kIsBf16>(p, plan, ws, st, stream, cuda_error_out);
    case 10: return launch_config<10, kIsBf16>(p, plan, ws, st, stream, cuda_error_out);
    case 11: return launch_config<11, kIsBf16>(p, plan, ws, st, stream, cuda_error_out);
    case 12: return launch_config<12, kIsBf16>(p, plan, ws, st, stream, cuda_error_out);
    case 13: return launch_config<13, kIsBf16>(p, plan, ws, st, stream, cuda_error_out);
    case 14: return launch_config<14, kIsBf16>(p, plan, ws, st, stream, cuda_error_out);
    case 15: return launch_config<15, kIsBf16>(p, plan, ws, st, stream, cuda_error_out);
    default: return GEMM_SM100_ERR_BAD_OPTION;
  }
}

int current_sm_count() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev >= 0 && dev < kMaxDevices && g_dev[dev].ready) return g_dev[dev].sm_count;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
  return n;
}

}  // namespace

extern "C" {

int gemm_sm100_tn(const void* A, const void* B, void* C, int M, int N, int K, long lda, long ldb,
                  long ldc, int dtype, void* workspace, size_t workspace_bytes, void* cuda_stream,
                  int* cuda_error_out) {
  if (cuda_error_out) *cuda_error_out = 0;
  Problem p{A, B, C, M, N, K, lda, ldb, ldc, dtype};
  int rc = validate(p);
  if (rc != GEMM_SM100_OK) return rc;
  if (M == 0 || N == 0) return GEMM_SM100_OK;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (K == 0) {
    cudaError_t e = cudaMemset2DAsync(C, static_cast<size_t>(ldc) * 2, 0, static_cast<size_t>(N) * 2,
                                      static_cast<size_t>(M), stream);
    return e == cudaSuccess ? GEMM_SM100_OK : set_cuda_error(cuda_error_out, e);
  }
  DeviceState* st = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    rc = device_state(&st, cuda_error_out);
    if (rc != GEMM_SM100_OK) return rc;
    rc = get_encoder(cuda_error_out);
    if (rc != GEMM_SM100_OK) return rc;
  }
  Plan plan = plan_for(M, N, K, st->sm_count);
  if (plan.split_k && !plan.cluster) {
    if (workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & 255u) ||
        workspace_bytes < plan.flag_bytes + plan.partial_bytes) {
      // A K-split the caller asked for needs its workspace; one the planner chose by itself is
      // only an optimisation: without the memory the problem runs as whole tiles.
      if (g_opt_split_k > 0) return GEMM_SM100_ERR_WORKSPACE;
      plan = plan_for(M, N, K, st->sm_count, /*allow_split=*/false);
    }
  }
  if (dtype == GEMM_SM100_BF16) return dispatch<true>(plan, p, workspace, *st, stream, cuda_error_out);
  return dispatch<false>(plan, p, workspace, *st, stream, cuda_error_out);
}

int gemm_sm100_tn_static_scratch(const void* A, const void* B, void* C, int M, int N, int K, long lda,
                                 long ldb, long ldc, int dtype, void* cuda_stream, int* cuda_error_out) {
  if (cuda_error_out) *cuda_error_out = 0;
  Problem p{A, B, C, M, N, K, lda, ldb, ldc, dtype};
  int rc = validate(p);
  if (rc != GEMM_SM100_OK) return rc;
  if (M == 0 || N == 0) return GEMM_SM100_OK;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (K == 0) {
    cudaError_t e = cudaMemset2DAsync(C, static_cast<size_t>(ldc) * 2, 0, static_cast<size_t>(N) * 2,
                                      static_cast<size_t>(M), stream);
    return e == cudaSuccess ? GEMM_SM100_OK : set_cuda_error(cuda_error_out, e);
  }
  DeviceState* st = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    rc = device_state(&st, cuda_error_out);
    if (rc != GEMM_SM100_OK) return rc;
    rc = get_encoder(cuda_error_out);
    if (rc != GEMM_SM100_OK) return rc;
    if (st->static_scratch == nullptr) {
      // Once per device, with that device current.  In host code the array's name is only a
      // handle for this lookup; the kernel must be given the address the runtime returns.
      void* ptr = nullptr;
      cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
      if (e != cudaSuccess) return set_cuda_error(cuda_error_out, e);
      st->static_scratch = ptr;
    }
  }
  // The 128 x 256 single-CTA configuration with the K-split schedule whenever the problem has
  // at least two K blocks of work to divide (otherwise one whole tile, which needs no scratch).
  const ConfigInfo& c = kConfigs[kSplitKConfig];
  const int block_n = c.mma_n * c.halves;
  const long tiles = ceil_div(M, 128L) * ceil_div(N, block_n);
  const long units = tiles * ceil_div(K, 64);
  const long slots = grid_cap(c, st->sm_count);
  Plan plan;
  plan.config = kSplitKConfig;
  if (units >= 2) {
    const long ranges = units < slots ? units : slots;
    plan.split_k = true;
    plan.ctas = static_cast<int>(ranges);
    plan.partial_rows = M < 128 ? static_cast<int>((M + 31) / 32 * 32) : 128;
    plan.flag_bytes = kStaticFlagBytes;
    plan.partial_bytes = static_cast<size_t>(plan.ctas) * plan.partial_rows * block_n * sizeof(float);
    if (static_cast<size_t>(plan.ctas) * sizeof(unsigned int) > kStaticFlagBytes ||
        plan.flag_bytes + plan.partial_bytes > kStaticScratchBytes)
      return GEMM_SM100_ERR_STATIC_SCRATCH;
  } else {
    plan.ctas = static_cast<int>(tiles < slots ? tiles : slots);
  }
  if (dtype == GEMM_SM100_BF16) return dispatch<true>(plan, p, st->static_scratch, *st, stream, cuda_error_out);
  return dispatch<false>(plan, p, st->static_scratch, *st, stream, cuda_error_out);
}

int gemm_sm100_tn_fanout(const void* A, const void* B, void* const* outputs, int num_outputs, int M, int N,
                         int K, long lda, long ldb, long ldc, int dtype, void* cuda_stream, int* cuda_error_out) {
  if (cuda_error_out) *cuda_error_out = 0;
  if (outputs == nullptr) return GEMM_SM100_ERR_NULL_POINTER;
  if (num_outputs < 1 || num_outputs > kMaxOutputs) return GEMM_SM100_ERR_BAD_SHAPE;
  for (int d = 0; d < num_outputs; ++d) {
    Problem pd{A, B, outputs[d], M, N, K, lda, ldb, ldc, dtype};
    const int rc = validate(pd);
    if (rc != GEMM_SM100_OK) return rc;
  }
  if (M == 0 || N == 0) return GEMM_SM100_OK;
  if (K == 0 || N % 8 != 0) return GEMM_SM100_ERR_BAD_SHAPE;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  DeviceState* st = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    int rc = device_state(&st, cuda_error_out);
    if (rc != GEMM_SM100_OK) return rc;
    rc = get_encoder(cuda_error_out);
    if (rc != GEMM_SM100_OK) return rc;
  }
  Problem p{A, B, outputs[0], M, N, K, lda, ldb, ldc, dtype};
  // Pair-tile configurations only.  The wave model of the plain GEMM, with what the epilogue's
  // extra stores cost added to the tile boundary: the 256 x 512 tile fills TMEM, so the time its
  // epilogue needs to push every 64-column chunk through one staging buffer per warp to
  // `num_outputs` destinations (all but one of them across NVLink in the multi-GPU use) is
  // exposed before the next tile's first MMA; the 256 x 256 tile drains one accumulator slot
  // while the tensor pipe fills the other, with two staging buffers per warp, and hides it.
  // See kFanoutKBlocksPerOutput for the measurements behind the constant.
  const long slots = st->sm_count / 2;
  const double k_blocks = static_cast<double>(ceil_div(K, 64L));
  const double cost0 = static_cast<double>(ceil_div(ceil_div(M, 256L) * ceil_div(N, 256L), slots)) * 256 *
                       (k_blocks + kTileBoundaryKBlocks[0]) / kConfigRate[0];
  const double cost1 = static_cast<double>(ceil_div(ceil_div(M, 256L) * ceil_div(N, 512L), slots)) * 512 *
                       (k_blocks + kTileBoundaryKBlocks[1] + kFanoutKBlocksPerOutput * (num_outputs - 1)) /
                       kConfigRate[1];
  const bool wide = g_opt_tile_config == 1 || (g_opt_tile_config != 0 && cost1 <= cost0);
  if (dtype == GEMM_SM100_BF16)
    return wide ? launch_fanout<1, true>(p, outputs, num_outputs, *st, stream, cuda_error_out)
                : launch_fanout<0, true>(p, outputs, num_outputs, *st, stream, cuda_error_out);
  return wide ? launch_fanout<1, false>(p, outputs, num_outputs, *st, stream, cuda_error_out)
              : launch_fanout<0, false>(p, outputs, num_outputs, *st, stream, cuda_error_out);
}

int gemm_sm100_nn(const void* A, const void* B, void* C, int M, int N, int K, long lda, long ldb, long ldc,
                  int dtype, void* cuda_stream, int* cuda_error_out) {
  return gemm_sm100_gemm(A, B, C, M, N, K, lda, ldb, ldc, dtype, 0, 1, cuda_stream, cuda_error_out);
}

int gemm_sm100_gemm(const void* A, const void* B, void* C, int M, int N, int K, long lda, long ldb, long ldc,
                    int dtype, int a_is_km, int b_is_kn, void* cuda_stream, int* cuda_error_out) {
  return gemm_sm100_gemm_scaled(A, B, C, M, N, K, lda, ldb, ldc, dtype, a_is_km, b_is_kn, 1.0f, 0.0f, cuda_stream,
                                cuda_error_out);
}

int gemm_sm100_gemm_scaled(const void* A, const void* B, void* C, int M, int N, int K, long lda, long ldb,
                           long ldc, int dtype, int a_is_km, int b_is_kn, float alpha, float beta,
                           void* cuda_stream, int* cuda_error_out) {
  if (cuda_error_out) *cuda_error_out = 0;
  if (!a_is_km && !b_is_kn && alpha == 1.0f && beta == 0.0f)
    return gemm_sm100_tn(A, B, C, M, N, K, lda, ldb, ldc, dtype, nullptr, 0, cuda_stream, cuda_error_out);
  Problem p{A, B, C, M, N, K, lda, ldb, ldc, dtype, b_is_kn != 0, a_is_km != 0, alpha, beta};
  int rc = validate(p);
  if (rc != GEMM_SM100_OK) return rc;
  if (M == 0 || N == 0) return GEMM_SM100_OK;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (K == 0 && beta != 0.0f) return GEMM_SM100_ERR_BAD_SHAPE;   // beta * C alone is not a GEMM
  if (K == 0) {
    cudaError_t e = cudaMemset2DAsync(C, static_cast<size_t>(ldc) * 2, 0, static_cast<size_t>(N) * 2,
                                      static_cast<size_t>(M), stream);
    return e == cudaSuccess ? GEMM_SM100_OK : set_cuda_error(cuda_error_out, e);
  }
  DeviceState* st = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    rc = device_state(&st, cuda_error_out);
    if (rc != GEMM_SM100_OK) return rc;
    rc = get_encoder(cuda_error_out);
    if (rc != GEMM_SM100_OK) return rc;
  }
  Plan plan = plan_for(M, N, K, st->sm_count, /*allow_split=*/false, /*config_limit=*/4, /*allow_balance=*/false);
  if (plan.config > 3) plan = Plan{};       // (a forced configuration without such a variant)
  if (plan.ctas == 0) {
    const long tiles = ceil_div(M, 256L) * ceil_div(N, 256L);
    const long slots = st->sm_count / 2;
    plan.config = 0;
    plan.ctas = static_cast<int>((tiles < slots ? tiles : slots) * 2);
  }
  if (dtype == GEMM_SM100_BF16) return dispatch_nn<true>(plan, p, *st, stream, cuda_error_out);
  return dispatch_nn<false>(plan, p, *st, stream, cuda_error_out);
}

int gemm_sm100_selftest_wait_timeout(void* cuda_stream, int* cuda_error_out) {
  if (cuda_error_out) *cuda_error_out = 0;
  DeviceState* st = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    const int rc = device_state(&st, cuda_error_out);
    if (rc != GEMM_SM100_OK) return rc;
  }
  wait_timeout_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      st->status_ptr, static_cast<unsigned long long>(g_opt_timeout_ms.load()) * 1000000ull);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? GEMM_SM100_OK : set_cuda_error(cuda_error_out, e);
}

size_t gemm_sm100_static_scratch_capacity(void) { return kStaticScratchBytes; }

size_t gemm_sm100_workspace_bytes(int M, int N, int K, int dtype) {
  (void)dtype;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const Plan plan = plan_for(M, N, K, current_sm_count());
  return plan.split_k ? plan.flag_bytes + plan.partial_bytes : 0;
}

int gemm_sm100_num_sms(void) {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
  return n;
}

int gemm_sm100_device_status(unsigned int* status_out, int* cuda_error_out) {
  if (cuda_error_out) *cuda_error_out = 0;
  if (status_out) *status_out = 0;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return set_cuda_error(cuda_error_out, e);
  DeviceState* st = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    int rc = device_state(&st, cuda_error_out);
    if (rc != GEMM_SM100_OK) return rc;
  }
  unsigned int word = 0;
  e = cudaMemcpy(&word, st->status_ptr, sizeof(word), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return set_cuda_error(cuda_error_out, e);
  if (status_out) *status_out = word;
  if (word != 0) {
    kept_workspaces_mark_dirty();   // a kernel that gave up may have left arrival counters behind
    e = cudaMemset(st->status_ptr, 0, sizeof(word));
    if (e != cudaSuccess) return set_cuda_error(cuda_error_out, e);
    return GEMM_SM100_ERR_DEVICE_TIMEOUT;
  }
  return GEMM_SM100_OK;
}

int gemm_sm100_workspace_register(void* workspace, size_t workspace_bytes, void* stream, int* cuda_error_out) {
  if (cuda_error_out) *cuda_error_out = 0;
  if (!workspace) return GEMM_SM100_ERR_NULL_POINTER;
  if (workspace_bytes < 256 || (reinterpret_cast<uintptr_t>(workspace) & 255u)) return GEMM_SM100_ERR_WORKSPACE;
  const size_t bytes = workspace_bytes < kKeptWorkspaceZeroBytes ? workspace_bytes / 256 * 256 : kKeptWorkspaceZeroBytes;
  cudaError_t e = cudaMemsetAsync(workspace, 0, bytes, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return set_cuda_error(cuda_error_out, e);
  std::lock_guard<std::mutex> lock(g_kept_mutex);
  for (KeptWorkspace& w : g_kept_workspaces)
    if (w.ptr == workspace) {
      w.clean_bytes = bytes;
      return GEMM_SM100_OK;
    }
  g_kept_workspaces.push_back({workspace, bytes});
  return GEMM_SM100_OK;
}

int gemm_sm100_workspace_unregister(void* workspace) {
  std::lock_guard<std::mutex> lock(g_kept_mutex);
  for (size_t i = 0; i < g_kept_workspaces.size(); ++i)
    if (g_kept_workspaces[i].ptr == workspace) {
      g_kept_workspaces.erase(g_kept_workspaces.begin() + static_cast<long>(i));
      return GEMM_SM100_OK;
    }
  return GEMM_SM100_ERR_WORKSPACE;
}

int gemm_sm100_resident_clusters(int cluster_ctas) {
  DeviceState* st = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (device_state(&st, nullptr) != GEMM_SM100_OK) return -1;
  }
  if (cluster_ctas != 2 && cluster_ctas != 4 && cluster_ctas != 8) return -1;
  return static_cast<int>(resident_clusters(st->sm_count, cluster_ctas));
}

int gemm_sm100_set_option(const char* name, long value) {
  if (!name) return GEMM_SM100_ERR_NULL_POINTER;
  std::lock_guard<std::mutex> lock(g_mutex);
  g_opt_generation.fetch_add(1, std::memory_order_acq_rel);   // cached plans depend on the options
  if (std::strcmp(name, "tile_config") == 0) {
    if (value < -1 || value >= kNumConfigs) return GEMM_SM100_ERR_BAD_OPTION;
    g_opt_tile_config = value;
    return GEMM_SM100_OK;
  }
  if (std::strcmp(name, "timeout_ms") == 0) {
    if (value < 1 || value > 60000) return GEMM_SM100_ERR_BAD_OPTION;
    g_opt_timeout_ms = value;
    return GEMM_SM100_OK;
  }
  if (std::strcmp(name, "debug_flags") == 0) {
    if (value < 0 || value > 7) return GEMM_SM100_ERR_BAD_OPTION;
    g_opt_debug_flags = value;
    return GEMM_SM100_OK;
  }
  if (std::strcmp(name, "k_rotate") == 0) {
    if (value < -1 || value > 2) return GEMM_SM100_ERR_BAD_OPTION;
    g_opt_k_rotate = value;
    return GEMM_SM100_OK;
  }
  if (std::strcmp(name, "split_k") == 0) {
    if (value < -1 || value > kMaxEvenSplit) return GEMM_SM100_ERR_BAD_OPTION;
    g_opt_split_k = value;
    return GEMM_SM100_OK;
  }
  if (std::strcmp(name, "sk_cluster") == 0) {
    if (value < -1 || value > 1) return GEMM_SM100_ERR_BAD_OPTION;
    g_opt_sk_cluster = value;
    return GEMM_SM100_OK;
  }
  if (std::strcmp(name, "pdl") == 0) {
    if (value < 0 || value > 1) return GEMM_SM100_ERR_BAD_OPTION;
    g_opt_pdl = value;
    return GEMM_SM100_OK;
  }
  if (std::strcmp(name, "early_prefetch") == 0) {
    if (value < 0 || value > 1) return GEMM_SM100_ERR_BAD_OPTION;
    g_opt_early_prefetch = value;
    return GEMM_SM100_OK;
  }
  if (std::strcmp(name, "tiles_n") == 0) {
    if (value < 0 || value > (1 << 20)) return GEMM_SM100_ERR_BAD_OPTION;
    g_opt_tiles_n = value;
    return GEMM_SM100_OK;
  }
  if (std::strcmp(name, "balance") == 0) {
    if (value < 0 || value > 1) return GEMM_SM100_ERR_BAD_OPTION;
    g_opt_balance = value;
    return GEMM_SM100_OK;
  }
  if (std::strcmp(name, "group_m") == 0) {
    if (value < 0 || value > 4096) return GEMM_SM100_ERR_BAD_OPTION;
    g_opt_group_m = value;
    return GEMM_SM100_OK;
  }
  if (std::strcmp(name, "max_ctas") == 0) {
    if (value < 0) return GEMM_SM100_ERR_BAD_OPTION;
    g_opt_max_ctas = value;
    return GEMM_SM100_OK;
  }
  return GEMM_SM100_ERR_BAD_OPTION;
}

int gemm_sm100_set_trace_buffer(void* device_buffer, size_t bytes) {
  if (device_buffer != nullptr && (reinterpret_cast<uintptr_t>(device_buffer) & 7u)) return GEMM_SM100_ERR_BAD_ALIGNMENT;
  int device = -1;
  if (device_buffer != nullptr) {
    // The buffer belongs to one device: only launches on that device may write to it.
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, device_buffer) != cudaSuccess || attr.type != cudaMemoryTypeDevice) {
      (void)cudaGetLastError();
      return GEMM_SM100_ERR_BAD_OPTION;
    }
    device = attr.device;
  }
  std::lock_guard<std::mutex> lock(g_mutex);
  g_trace.ptr = static_cast<unsigned long long*>(device_buffer);
  g_trace.bytes = device_buffer ? bytes : 0;
  g_trace.device = device;
  g_trace_on.store(device_buffer != nullptr, std::memory_order_release);
  return GEMM_SM100_OK;
}

int gemm_sm100_describe_config(int index, char* buf, size_t buf_bytes) {
  if (!buf || buf_bytes == 0) return GEMM_SM100_ERR_NULL_POINTER;
  if (index < 0 || index >= kNumConfigs) return GEMM_SM100_ERR_BAD_OPTION;
  const ConfigInfo& c = kConfigs[index];
  const int tmem_cols = 2 * c.mma_n <= 128 ? 128 : (2 * c.mma_n <= 256 ? 256 : 512);
  int n = std::snprintf(buf, buf_bytes, "cta_group=%d tile=%dx%dx%d stages=%d tmem_cols=%d epilogue_warps=%d",
                        c.cta_group, 128 * c.cta_group, c.mma_n * c.halves, 64 * c.k_sub, c.stages, tmem_cols, c.epi_warps);
  if (c.a_rows != 128 && n > 0 && static_cast<size_t>(n) < buf_bytes)
    std::snprintf(buf + n, buf_bytes - n, " a_rows=%d", c.a_rows);
  return GEMM_SM100_OK;
}

int gemm_sm100_describe_plan(int M, int N, int K, int dtype, char* buf, size_t buf_bytes) {
  (void)dtype;
  if (!buf || buf_bytes == 0) return GEMM_SM100_ERR_NULL_POINTER;
  if (M <= 0 || N <= 0 || K <= 0) return GEMM_SM100_ERR_BAD_SHAPE;
  const Plan plan = plan_for(M, N, K, current_sm_count());
  const ConfigInfo& c = kConfigs[plan.config];
  const int block_n = c.mma_n * c.halves;
  char tiling[128];
  if (plan.tiles_n > 0)
    std::snprintf(tiling, sizeof(tiling), "balanced: %d tiles per row, %d x %d + %d x %d columns (wide from %d)",
                  plan.tiles_n, plan.bal_rem, (plan.bal_q + 1) * 64, plan.tiles_n - plan.bal_rem, plan.bal_q * 64,
                  plan.bal_start);
  else
    std::snprintf(tiling, sizeof(tiling), "uniform: %ld tiles per row of %d columns", ceil_div(N, block_n), block_n);
  char split[96];
  if (!plan.split_k)
    std::snprintf(split, sizeof(split), "whole tiles");
  else if (plan.split_factor > 1)
    std::snprintf(split, sizeof(split), "every tile cut into %d K ranges%s", plan.split_factor,
                  plan.cluster ? " (one cluster per tile)" : "");
  else
    std::snprintf(split, sizeof(split), "contiguous K ranges");
  std::snprintf(buf, buf_bytes, "config=%d tile=%dx%dx64 %s; %s; ctas=%d workspace=%zu", plan.config, 128 * c.cta_group,
                block_n, tiling, split, plan.ctas, plan.split_k ? plan.flag_bytes + plan.partial_bytes : size_t{0});
  return GEMM_SM100_OK;
}

int gemm_sm100_select_config(int M, int N, int K, int dtype) {
  (void)dtype;
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  return plan_for(M, N, K, current_sm_count()).config;
}

const char* gemm_sm100_error_string(int code) {
  switch (code) {
    case GEMM_SM100_OK: return "ok";
    case GEMM_SM100_ERR_NULL_POINTER: return "null pointer";
    case GEMM_SM100_ERR_BAD_SHAPE: return "bad shape (negative extent, K not a multiple of 8, or leading dimension too small)";
    case GEMM_SM100_ERR_BAD_ALIGNMENT: return "pointer or row pitch not 16-byte aligned";
    case GEMM_SM100_ERR_UNSUPPORTED_DTYPE: return "unsupported dtype (bf16 = 0, fp16 = 1)";
    case GEMM_SM100_ERR_CUDA: return "CUDA error";
    case GEMM_SM100_ERR_DEVICE_TIMEOUT: return "device-side wait timed out";
    case GEMM_SM100_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
    case GEMM_SM100_ERR_UNSUPPORTED_DEVICE: return "device is not sm_100";
    case GEMM_SM100_ERR_BAD_OPTION: return "unknown option or value out of range";
    case GEMM_SM100_ERR_STATIC_SCRATCH:
      return "problem needs more scratch than the built-in array of gemm_sm100_tn_static_scratch holds "
             "(M above 32 on a full-size GPU); use gemm_sm100_tn with a caller workspace";
    default: return "unknown error code";
  }
}

}  // extern "C"

namespace {

template <int kCfgIndex>
int ensure_both_dtypes(DeviceState& st, int* cuda_error_out) {
  const int rc = ensure_config<kCfgIndex, true>(st, cuda_error_out);
  return rc ? rc : ensure_config<kCfgIndex, false>(st, cuda_error_out);
}

template <int... kIndices>
int ensure_all(DeviceState& st, int* cuda_error_out, std::integer_sequence<int, kIndices...>) {
  int rc = GEMM_SM100_OK;
  (void)((rc = ensure_both_dtypes<kIndices>(st, cuda_error_out), rc == GEMM_SM100_OK) && ...);
  return rc;
}

}  // namespace

extern "C" int gemm_sm100_init(int* cuda_error_out) {
  if (cuda_error_out) *cuda_error_out = 0;
  DeviceState* st = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    int rc = device_state(&st, cuda_error_out);
    if (rc != GEMM_SM100_OK) return rc;
    rc = get_encoder(cuda_error_out);
    if (rc != GEMM_SM100_OK) return rc;
    if (st->static_scratch == nullptr) {
      void* ptr = nullptr;
      const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
      if (e != cudaSuccess) return set_cuda_error(cuda_error_out, e);
      st->static_scratch = ptr;
    }
  }
  return ensure_all(*st, cuda_error_out, std::make_integer_sequence<int, kNumConfigs>{});
}
