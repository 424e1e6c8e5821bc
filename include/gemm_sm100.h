/* C ABI of the B200 (sm_100a) TN GEMM:  C[M,N] = A[M,K] * B[N,K]^T,
 * 16-bit inputs (bf16 or fp16), fp32 accumulation, same-dtype output (round to nearest even).
 *
 * This is the native boundary underneath the Python entry point
 * gemm_kernels._C.gemm_tn_test(A, B, C).  The reference has no C ABI: its native entry
 * is the C++ function test::gemm_tn_test(torch::Tensor, torch::Tensor, torch::Tensor)
 * (kernels/gemm_kernels/sm90a/gemm_test.cu:12-92), bound by pybind11 in
 * kernels/gemm_kernels/__init__.cpp:6-9.  The functions below carry that function's
 * contract with plain pointers and sizes; the library is compiled without torch.
 *
 * All pointers are device pointers on the CURRENT CUDA device unless stated otherwise.
 * Nothing here allocates device memory and nothing calls exit(): every failure is a
 * return code (the reference prints and exits on a CUDA error, gemm_test.cu:78,86).
 *
 * First use and stream capture.  The first launch of a tile configuration on a device sets
 * function attributes and queries occupancy (host-side calls, no device work and no
 * synchronisation).  A host that captures CUDA graphs should call gemm_sm100_init() once per
 * device before its first capture, which does all of that up front.
 *
 * Co-residency.  The K-split schedules that use a workspace (gemm_sm100_workspace_bytes() > 0, or the "split_k"
 * option, or gemm_sm100_tn_static_scratch) let CTAs wait for partial sums of other CTAs of the
 * same grid, so the whole grid must be resident at once.  The grid is sized from the device's SM
 * count; a host that gives this library only part of the SMs (an SM-limited or "green" context,
 * a long-running kernel on another stream) should set the option "split_k" to 0, or "max_ctas"
 * to the SMs it really has.  If such a wait runs out ("timeout_ms") the kernel returns with C
 * partly unwritten and the only signal is the status word: read it with
 * gemm_sm100_device_status().
 */
#ifndef GEMM_SM100_H_
#define GEMM_SM100_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Return codes. */
#define GEMM_SM100_OK 0
#define GEMM_SM100_ERR_NULL_POINTER 1
#define GEMM_SM100_ERR_BAD_SHAPE 2        /* negative extent, K not a multiple of 8, ld too small */
#define GEMM_SM100_ERR_BAD_ALIGNMENT 3    /* base pointer or row pitch not 16-byte aligned */
#define GEMM_SM100_ERR_UNSUPPORTED_DTYPE 4
#define GEMM_SM100_ERR_CUDA 5             /* a CUDA call failed; *cuda_error_out holds the cudaError_t */
#define GEMM_SM100_ERR_DEVICE_TIMEOUT 6   /* a bounded device-side wait ran out (see gemm_sm100_device_status) */
#define GEMM_SM100_ERR_WORKSPACE 7        /* workspace missing, misaligned or too small */
#define GEMM_SM100_ERR_UNSUPPORTED_DEVICE 8 /* current device is not compute capability 10.x */
#define GEMM_SM100_ERR_BAD_OPTION 9
#define GEMM_SM100_ERR_STATIC_SCRATCH 10  /* problem too large for gemm_sm100_tn_static_scratch */

/* Element types of A, B and C. */
#define GEMM_SM100_BF16 0
#define GEMM_SM100_FP16 1

/* Enqueues C = A * B^T on `cuda_stream` (a cudaStream_t; NULL = legacy default stream)
 * and returns without waiting for the GPU.
 *   A: M rows of K elements, row pitch lda (elements);  B: N rows of K elements, pitch ldb;
 *   C: M rows of N elements, pitch ldc.  "TN": both operands have K contiguous.
 * Requirements: K % 8 == 0, lda/ldb/ldc % 8 == 0, all three base pointers 16-byte aligned,
 * lda, ldb >= K, ldc >= N.  M and N are arbitrary (the reference requires M % 256 == 0,
 * N % 256 == 0, K % 64 == 0: gemm_test.cu:32-41).  M == 0 or N == 0 is a no-op; K == 0 zero-fills C.
 * `workspace` should hold gemm_sm100_workspace_bytes(M, N, K, dtype) bytes (256-byte aligned)
 * when that is non-zero; it may be NULL otherwise.  Without it a K-split schedule that the
 * library chose by itself falls back to whole tiles (slower for few-tile, long-K problems); one
 * forced through the "split_k" option returns GEMM_SM100_ERR_WORKSPACE.
 * Replaces: test::gemm_tn_test, gemm_test.cu:12-92 (argument checks :15-41, tensor-map
 * construction :56-68, launch :70-85).  Differences by design: asynchronous on the caller's
 * stream (the reference uses the legacy default stream and then cudaDeviceSynchronize, :82-86).
 */
int gemm_sm100_tn(const void* A, const void* B, void* C, int M, int N, int K, long lda, long ldb,
                  long ldc, int dtype, void* workspace, size_t workspace_bytes, void* cuda_stream,
                  int* cuda_error_out);

/* C[M,N] = A[M,K] * B[K,N]: the same kernels with B given row-major as [K, N] (N contiguous,
 * pitch ldb >= N elements), i.e. without the transposed copy of B that the reference's callers
 * make to reach its [N, K] contract (kernels/tests/gemm_bench.py:278-295,
 * `B.t().contiguous()`).  B is loaded as 64-column blocks and handed to the tensor core as an
 * MN-major operand.  Requirements as for gemm_sm100_tn with ldb % 8 == 0; needs no workspace
 * (whole tiles only).  No reference counterpart: the reference implements the TN contract only. */
int gemm_sm100_nn(const void* A, const void* B, void* C, int M, int N, int K, long lda, long ldb, long ldc,
                  int dtype, void* cuda_stream, int* cuda_error_out);

/* All four operand layouts behind one call: A as [M,K] (a_is_km = 0) or [K,M] (1, pitch
 * lda >= M), B as [N,K] (b_is_kn = 0) or [K,N] (1, pitch ldb >= N).  (0,0) is gemm_sm100_tn
 * without a workspace: a K-split the library would have chosen by itself then runs as whole
 * tiles (call gemm_sm100_tn with a workspace to get the split); (0,1) is gemm_sm100_nn.  The
 * [K,*] forms are loaded as MN-major operands; whole tiles only.  No reference counterpart (TN
 * only). */
int gemm_sm100_gemm(const void* A, const void* B, void* C, int M, int N, int K, long lda, long ldb, long ldc,
                    int dtype, int a_is_km, int b_is_kn, void* cuda_stream, int* cuda_error_out);

/* C = alpha * op(A) op(B) + beta * C for any of the four layouts of gemm_sm100_gemm.  alpha and
 * beta are applied in fp32 in the epilogue, before the single rounding to the output type; with
 * beta != 0 the old C is read (16-bit, same pitch).  K == 0 is only accepted with beta == 0.
 * No reference counterpart: its epilogue only converts the accumulator (gemm.cuh:368-377). */
int gemm_sm100_gemm_scaled(const void* A, const void* B, void* C, int M, int N, int K, long lda, long ldb,
                           long ldc, int dtype, int a_is_km, int b_is_kn, float alpha, float beta,
                           void* cuda_stream, int* cuda_error_out);

/* C = A * B^T stored into `num_outputs` (1..8) output matrices at once: the epilogue issues one
 * TMA store per output for every finished tile.  All outputs share M, N, ldc and dtype; each
 * pointer must be 16-byte aligned and writable from the current device (its own memory, or a
 * peer GPU's memory mapped into this process, e.g. a symmetric-memory buffer).  This is the
 * building block of the column-sharded multi-GPU GEMM: rank g passes, for every GPU r,
 * `C_r + g * N_shard` with ldc = N_total, and the all-gather of C happens inside the GEMM as
 * stores over NVLink (no staging buffer, no separate collective; the caller still needs a
 * cross-GPU barrier before reading C).  K must be > 0 and N a multiple of 8.  Needs no workspace.
 * No reference counterpart: the reference is single-GPU (one store per tile, gemm.cuh:388-394). */
int gemm_sm100_tn_fanout(const void* A, const void* B, void* const* outputs, int num_outputs, int M, int N,
                         int K, long lda, long ldb, long ldc, int dtype, void* cuda_stream, int* cuda_error_out);

/* Same product C = A * B^T as gemm_sm100_tn, for hosts that have no way to hand this library
 * scratch memory and must not see it allocate any: an operator plugged into a serving stack
 * that owns the whole device through its own pool and passes only input and output buffers, a
 * binding whose call signature has no workspace slot, or a latency-critical loop where a
 * cudaMalloc (which synchronises the device) is not acceptable.  It has no counterpart in the
 * reference, whose kernel needs no scratch at all.
 *
 * It always runs the 128 x 256-tile kernel with the K-split schedule (every CTA gets an equal
 * run of K blocks; tiles cut by a range boundary are summed from fp32 partial tiles), and keeps
 * the arrival counters and partial tiles in an array built into the library
 * (gemm_sm100_static_scratch_capacity() bytes, 5 MiB + 1 KiB, resident on every GPU that loads
 * the library until the process exits).  One partial tile of round_up(min(M,128), 32) x 256
 * floats per CTA must fit: on a 148-SM GPU that means M <= 32 (the few-rows, long-K shapes the
 * schedule is meant for); anything larger is refused with GEMM_SM100_ERR_STATIC_SCRATCH and
 * nothing is launched.  Arguments, requirements and the other return codes are those of
 * gemm_sm100_tn.
 *
 * The call allocates nothing (no cudaMalloc, no cudaFree, no allocating library routine); it
 * zeroes the counters on `cuda_stream` before the kernel.  The first call on each device looks
 * up the array's device address (cudaGetSymbolAddress, with that device current): make that
 * first call before starting any stream capture.  All calls on a device share the one array,
 * which keeps whatever the previous call left in it: two calls whose GPU work can overlap
 * (different streams without an ordering between them) race on it and give wrong results;
 * calls on one stream, or otherwise ordered, are safe. */
int gemm_sm100_tn_static_scratch(const void* A, const void* B, void* C, int M, int N, int K, long lda,
                                 long ldb, long ldc, int dtype, void* cuda_stream, int* cuda_error_out);

/* Size in bytes of the array gemm_sm100_tn_static_scratch works in. */
size_t gemm_sm100_static_scratch_capacity(void);

/* Bytes of scratch memory gemm_sm100_tn needs for this problem on the current device: 0 for
 * most shapes; non-zero when the K-split schedule is chosen (few tiles and long K, e.g. the
 * memory-bound small-M shapes), which keeps one arrival counter and one fp32 partial tile per
 * CTA there.  The contents need no initialisation.  No reference counterpart: the reference
 * kernel needs no workspace (gemm_test.cu:70-85). */
size_t gemm_sm100_workspace_bytes(int M, int N, int K, int dtype);

/* Optional: hands a workspace to the library for keeping.  The first 4 KiB (the arrival counters of
 * any plan) are zero-filled once, on `cuda_stream`; from then on a K-split launch that is given this
 * pointer skips the memset in front of the kernel whenever the previous launch on it left the
 * counters at zero, which the even K-split does by itself.  Without the memset node the kernel is a
 * programmatic dependent of the previous one like the unsplit kernels are.  The caller promises
 * that nothing else writes the workspace while it is registered, that launches using it are ordered
 * one after another (one stream, or events), and calls gemm_sm100_workspace_unregister before
 * freeing it.  After gemm_sm100_device_status has reported a time-out every registered workspace is
 * zero-filled again before its next use.  `workspace`: 256-byte aligned, at least 256 bytes.
 * Returns GEMM_SM100_OK, GEMM_SM100_ERR_WORKSPACE, GEMM_SM100_ERR_NULL_POINTER or
 * GEMM_SM100_ERR_CUDA.  No reference counterpart (the reference needs no workspace). */
int gemm_sm100_workspace_register(void* workspace, size_t workspace_bytes, void* cuda_stream,
                                  int* cuda_error_out);

/* Forgets a registered workspace (GEMM_SM100_ERR_WORKSPACE if it was not registered). */
int gemm_sm100_workspace_unregister(void* workspace);

/* How many thread-block clusters of `cluster_ctas` (2, 4 or 8) CTAs of this library's kernels
 * (one CTA per SM) the current device holds at once, from the CUDA occupancy query; what the
 * planner divides by when it counts the waves of a cluster K-split.  Negative on error.  No
 * reference counterpart. */
int gemm_sm100_resident_clusters(int cluster_ctas);

/* Number of SMs of the current device (the persistent grid is sized from it; the
 * reference hard-codes 132, gemm_test.cu:72).  Returns a negative value on error. */
int gemm_sm100_num_sms(void);

/* Waits for the current device to finish, then reads and clears the device status word
 * that the kernels set when a bounded wait runs out.  *status_out receives the raw word
 * (0 = no failure).  Returns GEMM_SM100_OK, GEMM_SM100_ERR_DEVICE_TIMEOUT or
 * GEMM_SM100_ERR_CUDA.  Replaces the reference's CUTE_CHECK_LAST() after the launch
 * (gemm_test.cu:86), which synchronises and exits the process on error. */
int gemm_sm100_device_status(unsigned int* status_out, int* cuda_error_out);

/* Tuning / test knobs, process-wide.  Set them before asking gemm_sm100_workspace_bytes, which
 * depends on them.
 *   "tile_config"  -1 = choose automatically (default), otherwise an index reported by
 *                  gemm_sm100_describe_config.  A configuration that cannot take the problem
 *                  (more rows than its A tile holds; K not a multiple of 64 for the one that
 *                  loads two K blocks per TMA box) is ignored and the automatic choice runs.
 *   "timeout_ms"   bound of each device-side wait, 1..60000, default 2000.
 *   "max_ctas"     0 = all SMs (default); otherwise caps the persistent grid.
 *   "split_k"      -1 = automatic (default); 0 = never; 1 = contiguous K ranges, one per CTA or
 *                  pair, whenever the chosen configuration has a K-split variant; 2..16 = every
 *                  tile cut into that many equal K ranges with the reduction spread over the
 *                  contributors (256 x 256 and 128 x 256 tiles; 2..8 for the 256 x 128 tile with
 *                  two K blocks per TMA box).  A forced value the chosen configuration cannot
 *                  take is ignored.
 *   "sk_cluster"   how the contributors of a tile cut into 2 or 4 K ranges exchange their partial
 *                  sums: 1 = always inside a thread-block cluster (one cluster per tile, one range
 *                  per CTA or pair, partial tiles moved between the CTAs' shared memories by
 *                  asynchronous bulk copies; needs no workspace and no co-residency of the grid);
 *                  0 = always through the workspace; -1 = the planner decides (default).
 *   "balance"      1 = the planner may give a tile row a number of tiles that fills the SMs evenly,
 *                  with tile widths in steps of 64 columns (default); 0 = uniform tiles only.
 *   "pdl"          1 = launch with the programmatic-stream-serialization attribute (default): when
 *                  the previous kernel in the stream is one of this library's, the new kernel's
 *                  CTAs are scheduled while it drains, set up their barriers and tensor memory,
 *                  and wait for its completion before they touch global memory; after any other
 *                  kernel the launch is an ordinary one.  0 = ordinary launches only.
 *   "early_prefetch" 1 = with "pdl", every CTA asks L2 for the operand boxes of its first two
 *                  stages before it waits for the previous kernel (default; a hint only: L2 is
 *                  where this GPU's writes become visible, so nothing stale can be read later);
 *                  0 = off.
 *   "tiles_n"      0 = the planner's choice (default); > 0 forces that many tiles per tile row
 *                  (tests; ignored where the configuration cannot make tiles of the resulting widths).
 *   "group_m"      0 = default; tile rows per rasterisation group.
 *   "k_rotate"     order of a tile's K blocks: 0 = ascending; 1 = every tile starts at a different K
 *                  block and wraps; -1 = that, for problems of at most 128 rows and at least 2048
 *                  columns only (default: the CTAs of these memory-bound shapes then stream
 *                  different column offsets of B at any moment; every other problem sums K in
 *                  ascending order, so a row's result does not depend on how the caller cuts M); 2 = every other tile of a CTA runs K backwards (re-reads the
 *                  shared operand panel newest-first).
 *   "debug_flags"  EXPERIMENTS ONLY, results are garbage while it is non-zero: bit 0 skips the
 *                  operand loads, bit 1 the stores of C, bit 2 the MMAs (pure issue-rate and
 *                  load-rate measurements of tests/trace_report.py).  Default 0.
 * The environment variables GEMM_SM100_TILE_CONFIG, GEMM_SM100_SPLIT_K, GEMM_SM100_GROUP_M,
 * GEMM_SM100_MAX_CTAS, GEMM_SM100_TIMEOUT_MS and GEMM_SM100_PDL give the initial values when the library is
 * loaded ("debug_flags" has no variable on purpose).
 * The reference's equivalents are compile-time constants (gemm.cuh:420-451). */
int gemm_sm100_set_option(const char* name, long value);

/* Writes a short description of tile configuration `index` ("cta_group=2 tile=256x256x64
 * stages=6 ...") into buf; returns GEMM_SM100_ERR_BAD_OPTION past the last index. */
int gemm_sm100_describe_config(int index, char* buf, size_t buf_bytes);

/* Writes what gemm_sm100_tn would do for this problem on the current device, in words: tile
 * configuration, column tiling (uniform, or balanced with the tile widths), K-split schedule,
 * grid size and workspace bytes.  For logs and benchmark records. */
int gemm_sm100_describe_plan(int M, int N, int K, int dtype, char* buf, size_t buf_bytes);

/* Index of the tile configuration gemm_sm100_tn would pick for this problem on the current
 * device (negative on error). */
int gemm_sm100_select_config(int M, int N, int K, int dtype);

/* One-time set-up of the current device, optional: looks up the driver's tensor-map encoder and
 * the library's device variables, sets the shared-memory limit of every kernel instantiation
 * and queries how many CTAs of each are co-resident.  Idempotent and thread-safe; issues no
 * device work.  Every launching entry point does the part it needs on first use; call this
 * once per device before capturing a stream.  No reference counterpart (the reference sets
 * its one kernel's attribute on every call, gemm_test.cu:74-78). */
int gemm_sm100_init(int* cuda_error_out);

/* Profiling aid.  While a device buffer is registered, every launch ON THE DEVICE THAT OWNS THE
 * BUFFER whose grid fits
 * (grid CTAs x 16 x 8 bytes <= bytes) writes one 16-word record per CTA: clock64 stamps of
 * kernel entry, set-up done, first operand stage, last MMA issued, last load issued, epilogue
 * done, exit; cycles each role spent waiting (MMA on operand stages [3] and on a free
 * accumulator [4], producer on free ring slots [6], epilogue on accumulators [8]); tiles
 * processed [11]; %globaltimer at entry [12] and exit [13].  NULL switches tracing off.
 * Launches on other devices ignore the buffer.  The caller keeps the memory alive until it
 * has switched tracing off; a pointer that is not device memory is refused.
 * The reference has no tracing in code; its profiler.py is a bare launch for Nsight
 * (kernels/tests/profiler.py:1-12). */
int gemm_sm100_set_trace_buffer(void* device_buffer, size_t bytes);

/* Self-test of the failure path, safe to run on a shared GPU: launches one warp that waits, with
 * the same bounded wait the GEMM kernels use, on a barrier nothing ever arrives on.  After the
 * "timeout_ms" limit the wait gives up, the kernel records status word 0x7e57 and returns;
 * gemm_sm100_device_status then reports GEMM_SM100_ERR_DEVICE_TIMEOUT and the context stays
 * usable.  (The reference's waits are unbounded, gemm.cuh:75-78, 91-94: a lost arrival hangs the
 * GPU.) */
int gemm_sm100_selftest_wait_timeout(void* cuda_stream, int* cuda_error_out);

/* Static, human-readable name of a return code. */
const char* gemm_sm100_error_string(int code);

#ifdef __cplusplus
}
#endif
#endif /* GEMM_SM100_H_ */
