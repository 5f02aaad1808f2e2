/* C ABI of the B200 (sm_100a) dense GEMM:  C[M,N] = A[M,K] * B[N,K]^T, bf16 in, fp32 accumulate,
 * bf16 out. A and B are both K-contiguous ("K-major"); C is row-major unless stated otherwise.
 *
 * This header is the drop-in boundary for the host launchers of Faraz9877/H100_GEMM. Each entry
 * point names the reference interface it replaces (paths are relative to that project).
 * Plain pointers and sizes only; no C++ or framework types. Every function returns a
 * b200_status code (0 = success) instead of calling exit()/assert() as the reference does
 * (common.h:29-37, tma.cuh:95-178). Nothing here falls back to a CPU implementation: without a
 * CUDA device the compute entry points return B200_ERR_CUDA.
 *
 * All pointers are device pointers unless the parameter name starts with `h`.
 * `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream, as the
 * reference launches on, matmul_h100.cu.jinja:970).
 */
#ifndef B200_GEMM_H_
#define B200_GEMM_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum b200_status {
  B200_OK = 0,
  B200_ERR_INVALID_ARG = 1,     /* NULL pointer, non-positive size, bad enum value          */
  B200_ERR_UNSUPPORTED_CFG = 2, /* tile/cluster/stage combination that has no kernel        */
  B200_ERR_SMEM = 3,            /* configuration needs more shared memory than an SM has    */
  B200_ERR_WORKSPACE = 4,       /* workspace missing or smaller than b200_gemm_workspace_bytes */
  B200_ERR_CUDA = 5,            /* a CUDA runtime/driver call failed (see b200_gemm_last_cuda_error) */
  B200_ERR_DEVICE_TIMEOUT = 6,  /* a bounded wait inside the kernel gave up                 */
  B200_ERR_ALPHA_BETA = 7,      /* reserved                                                 */
  B200_ERR_STATIC_SCRATCH = 8   /* b200_gemm_bf16_fixed_scratch: shape needs more than its fixed scratch */
} b200_status;

/* Tunable surface. The first six fields are the template variables of the reference's
 * matmul_h100.cu.jinja:9-14 / gemm_tuner.py:17-24 and keep their meaning:
 *   block_m   rows of C per CTA: 128 (one tcgen05 accumulator of 128 TMEM lanes) or 256 (two of
 *             them, sharing every B tile). 16, 32 or 64 select the few-rows plan for decode-like
 *             shapes: a block_m x 128 tile computed with the operands swapped inside (128 rows of B
 *             on the MMA's M dimension, block_m rows of A on its N dimension) and stored
 *             transposed; see swap_ab below for its variants.
 *   block_n   columns of C per tile: 64, 128, 192 or 256; 224 with block_m = 128, cluster_m = 1 and
 *             whole tiles (sched = 0) only.
 *   block_k   K-tile staged per pipeline stage: 64 (one 128-byte swizzle row).
 *   stages    shared-memory ring depth; 0 = as many as fit.
 *   cluster_m CTAs along M that share one B tile. 1 = single-CTA MMA. 2 = a CTA pair driving one
 *             tcgen05.mma.cta_group::2 (256 x block_n per pair; each CTA stages half of B). Larger
 *             powers of two keep the pair and only widen the raster group (no multicast loads).
 *   cluster_n must be 1 (the reference's tuner rejects anything else, gemm_tuner.py:77-78).
 * The rest are additions with neutral defaults (all zero):
 *   sched     0 data-parallel tiles, 1 split-K, 2 stream-K, 3 hybrid (full waves of tiles
 *             data-parallel, the last partly filled wave stream-K), 4 hybrid over two waves (the
 *             last full wave is cut stream-K style together with the partly filled one).
 *   split_k   K-slices per tile for sched 1 (0/1 = none).
 *   raster    0 group tiles along M, 1 along N.
 *   group     raster group width in tiles; 0 = default (8).
 *   c_col_major  0: C row-major [M,N] (matmul_h100.cu.jinja:696); 1: column-major, leading
 *             dimension M (matmul_utils.cuh:529,545).
 *   max_ctas  cap on the persistent grid; 0 = every SM.
 *   epilogue  how C is written: 0 = library default, 1 = bf16 tiles staged in shared memory and
 *             written with TMA tile stores, 2 = 16-byte global stores straight from registers
 *             (leaves the staging memory to the operand ring), 3 = transposed through a small
 *             shared-memory slab per warp and written with coalesced 16-byte stores. C rows that are not 16-byte aligned
 *             are always written with 2-byte stores (the reference's epilogue,
 *             matmul_h100.cu.jinja:689-698).
 *   swap_ab   1 selects the few-rows plan explicitly (block_m = 16, 32 or 64 imply it): block_m
 *             (16, 32, 64 or 128) rows of A ride the MMA's N dimension; block_n (128 or 256) is the
 *             number of rows of B each CTA puts on the MMA's M dimension per tile; cluster_m = 2 runs
 *             a CTA pair in which each CTA stages only half of the block_m rows of A. No split-K.
 */
typedef struct b200_gemm_cfg {
  int block_m;
  int block_n;
  int block_k;
  int stages;
  int cluster_m;
  int cluster_n;
  int sched;
  int split_k;
  int raster;
  int group;
  int c_col_major;
  int max_ctas;
  int epilogue;
  int swap_ab;
} b200_gemm_cfg;

/* Replaces gpu_gemm<AType,BType,CType,AccumType,CLUSTER_M,CLUSTER_N,BLOCKM,BLOCKN,BLOCKK,STAGES>
 * (GemmParams) — matmul_h100.cu.jinja:927-985 — for bf16. cfg == NULL picks a configuration from
 * the shape. The result is (bf16)(acc * alpha + beta): beta is added as a SCALAR, which is what
 * the reference's own GEMMs define (reference.h:40,72); alpha = 1, beta = 0 is the fast path the
 * reference's kernels hard-wire (matmul_h100.cu.jinja:696).
 * `workspace` may be NULL when b200_gemm_workspace_bytes() returns 0 for the same arguments.
 * Asynchronous on `stream`; no host synchronisation, no allocation. The kernel is launched with
 * programmatic stream serialization: its set-up may overlap the tail of the kernel before it in
 * the stream, and it waits for that kernel to complete before it reads or writes global memory
 * (environment variable B200_GEMM_NO_PDL=1 turns this off). */
int b200_gemm_bf16(int M, int N, int K, const void* A, const void* B, void* C, float alpha,
                   float beta, const b200_gemm_cfg* cfg, void* workspace, size_t workspace_bytes,
                   void* stream);

/* The same GEMM for IEEE fp16 inputs and output (fp32 accumulation): the data type of the
 * reference's tunable template, whose only instantiation is half_t (matmul_h100.cu.jinja:1010-1013,
 * WgMMA<half_t,half_t,float> at :291-292). Same arguments and rules as b200_gemm_bf16. */
int b200_gemm_f16(int M, int N, int K, const void* A, const void* B, void* C, float alpha, float beta,
                  const b200_gemm_cfg* cfg, void* workspace, size_t workspace_bytes, void* stream);

/* `batch` independent GEMMs of one shape; stride* are element distances between consecutive
 * problems. No counterpart function in the reference; it covers the batched configuration its
 * rank-3 tensor maps are built for (tma.cuh:83-181 with TmaDim = 3). */
int b200_gemm_batched_bf16(int batch, int M, int N, int K, const void* A, long long strideA,
                           const void* B, long long strideB, void* C, long long strideC,
                           float alpha, float beta, const b200_gemm_cfg* cfg, void* workspace,
                           size_t workspace_bytes, void* stream);

/* Bytes of device workspace the two functions above need for these arguments: fp32 partial
 * tiles for split-K / stream-K, and re-pitched copies of A and B when K is not a multiple of 8
 * elements (TMA needs a 16-byte row pitch — the reference asserts it, tma.cuh:109). */
size_t b200_gemm_workspace_bytes(int batch, int M, int N, int K, const b200_gemm_cfg* cfg);

/* Fills *cfg with the configuration cfg == NULL would use for this shape. */
int b200_gemm_default_cfg(int batch, int M, int N, int K, b200_gemm_cfg* cfg);

/* Tuning table: measured configurations fed back into the cfg == NULL dispatch. The reference's
 * tuner searches one shape and leaves its result in a JSON file and a rendered source
 * (gemm_tuner.py:126-145); nothing consumes it. Here a table of (batch, M, N, K) -> configuration
 * is looked up before the built-in heuristic: the exact shape if present, otherwise the entry of
 * the same class (batched or not; ceil(log2) of M, N and K) nearest in log2 distance.
 *   b200_gemm_tuning_load   reads a text file — one entry per line,
 *       batch M N K block_m block_n cluster_m stages sched split_k raster group epilogue [swap_ab]
 *     ('#' starts a comment; the last column may be left out) — and returns the number of entries added, or -B200_ERR_* when the
 *     file cannot be read, a line is malformed or names a configuration without a kernel (then
 *     nothing is added). Before the first use of the table the library loads the file the
 *     environment variable B200_GEMM_TUNING_TABLE names or, when the variable is not set, the
 *     measured table shipped beside it (<directory of the shared object>/../tuner/
 *     b200_measured.table); an empty value of the variable starts with an empty table.
 *     h100_gemm_b200/tuner/gemm_tuner.py --table writes the format.
 *   b200_gemm_tuning_add    adds or replaces one entry (c_col_major and max_ctas must be 0: they
 *     are per-call choices).
 *   b200_gemm_tuning_clear / _size   empty the table / number of entries.
 *   b200_gemm_heuristic_cfg the built-in choice, ignoring the table.
 * b200_gemm_bf16_fixed_scratch and b200_gemm_bf16_gather never consult the table.
 *
 * Stream-K and the hybrid schedules (sched 2, 3, 4 — the default for M <= 128 with many tiles)
 * assume that the whole grid is resident at once: a worker that finishes a split tile waits, with a
 * bound of about 0.1 s, for partial tiles of workers launched after it. The grid is sized for an
 * otherwise idle device. When other kernels hold SMs at the same time (another stream of the same
 * process, MPS), pass sched = 0 or cap the grid with max_ctas; a serving loop should also poll
 * b200_gemm_last_device_status(), which reports a wait that gave up (the results of that launch are
 * then not valid). */
int b200_gemm_tuning_load(const char* path);
int b200_gemm_tuning_add(int batch, int M, int N, int K, const b200_gemm_cfg* cfg);
void b200_gemm_tuning_clear(void);
int b200_gemm_tuning_size(void);
int b200_gemm_heuristic_cfg(int batch, int M, int N, int K, b200_gemm_cfg* cfg);
/* The same choice for a device with `sm_count` multiprocessors (the built-in heuristic counts waves
 * of tiles over the SMs of the current device; 148 when there is none). No reference counterpart:
 * its launcher hard-codes the SM count (matmul_h100_optimal.cu:40). */
int b200_gemm_heuristic_cfg_for_sms(int batch, int M, int N, int K, int sm_count, b200_gemm_cfg* cfg);

/* Replaces runKernel(int M,int N,int K,bf16* A,bf16* B,bf16* C,int* DB) —
 * matmul_h100_optimal.cu:32-59: default configuration, COLUMN-major C (ld = M), default stream.
 * DB is accepted and ignored, as in the reference (matmul_h100_optimal.cu:32,58). */
int b200_run_kernel(int M, int N, int K, void* A, void* B, void* C, int* DB);

/* Same GEMM with HOST buffers (pageable or pinned): copies A and B to the device in row bands, runs
 * one kernel per block of C as soon as its two bands have arrived and copies that block back, so
 * that kernels and device -> host copies hide behind the host -> device copies. Synchronous. It keeps device
 * staging buffers between calls (released by b200_gemm_host_release). This is the call a
 * harness like the reference's main() makes around its copy_to_gpu / gpu_gemm / copy_to_cpu
 * sequence (matmul_h100.cu.jinja:1036-1054). */
int b200_gemm_bf16_host(int M, int N, int K, const void* hA, const void* hB, void* hC, float alpha,
                        float beta, const b200_gemm_cfg* cfg);
/* The copies of b200_gemm_bf16_host without the kernels, in the same order on the same streams: what
 * the host links alone allow for this shape (hC receives whatever the device buffer holds). A
 * benchmark divides the two to see how much of the end-to-end time is the copies. State is kept
 * per device; calls from several host threads are serialised; on any error the call returns only
 * after its copies in flight have finished with the caller's buffers. */
int b200_gemm_bf16_host_copies_only(int M, int N, int K, const void* hA, const void* hB, void* hC);
/* Frees the staging buffers, streams and events of every device. */
void b200_gemm_host_release(void);

/* The few-rows GEMM (M <= 128, the decode shapes that run stream-K) for callers that cannot
 * allocate or pass device memory beyond the operands: a serving loop that fixes its device memory
 * plan at start-up and bans cudaMalloc afterwards, or a plug-in API with no workspace argument.
 * This entry point has no counterpart in the reference. It computes what b200_gemm_bf16 does with
 * the configuration b200_gemm_fixed_scratch_cfg returns (single-CTA stream-K tiles of 128 columns;
 * never the tuning table, whatever it holds), but keeps the stream-K partial tiles and flags in a
 * 10 MiB array inside the library image (so every GPU that loads the library holds that memory
 * until exit) and calls no cudaMalloc/cudaFree itself.
 *   Limits: M <= 128, K % 8 == 0, A and B 16-byte aligned; anything else returns
 *     B200_ERR_STATIC_SCRATCH (use b200_gemm_bf16 with a workspace instead).
 *   First call on a device: looks up the array's device address (cudaGetSymbolAddress) and does
 *     the library's other one-time set-up; make that first call outside any stream capture.
 *   Sharing: all calls use the same array and it keeps the previous call's contents (the kernel
 *     does not depend on them). Two calls whose kernels can overlap on the GPU — different
 *     streams, or different host threads — race on it: serialise them on one stream. */
int b200_gemm_bf16_fixed_scratch(int M, int N, int K, const void* A, const void* B, void* C, float alpha,
                                 float beta, void* stream);
/* The configuration b200_gemm_bf16_fixed_scratch runs for this shape (B200_ERR_STATIC_SCRATCH when
 * M > 128); passing it to b200_gemm_bf16 with a workspace gives bit-identical results. */
int b200_gemm_fixed_scratch_cfg(int M, int N, int K, b200_gemm_cfg* cfg);

/* Row-sharded GEMM fused with the all-gather of C. Rank `rank` of `world` (<= 8) ranks on one node
 * holds M rows of A; C_all[p] is the base of rank p's copy of the FULL C ([world * M, N], bf16,
 * row-major) as addressable from this device — its own allocation for p == rank, peer-mapped
 * memory (b200_peer_import) for the others. The kernel's epilogue writes every finished tile into
 * all `world` copies with TMA stores over NVLink, so when every rank's launch has completed each
 * rank holds the whole C; no separate collective runs. The caller must order "all launches
 * complete" before anyone reads C (a barrier between the ranks, e.g. a one-element all-reduce on
 * the same stream). Needs N % 8 == 0 and 16-byte aligned copies. cfg == NULL picks the pair-tile
 * configuration the fused epilogue is built for (256 rows per CTA for two or three ranks, 128 rows
 * per CTA from four ranks on, as measured); other tile shapes return
 * B200_ERR_UNSUPPORTED_CFG. The reference has no multi-GPU path; this is the M-sharded
 * configuration with the collective that follows the kernel folded into it. */
int b200_gemm_bf16_gather(int M, int N, int K, const void* A, const void* B, void* const* C_all, int world,
                          int rank, const b200_gemm_cfg* cfg, void* stream);

/* Device memory that other processes on the node can map (CUDA IPC): allocate, export a 64-byte
 * handle, import a peer's handle (enables peer access lazily), close an imported mapping, free. */
int b200_peer_alloc(size_t bytes, void** ptr);
int b200_peer_free(void* ptr);
int b200_peer_export(void* ptr, unsigned char handle[64]);
int b200_peer_import(const unsigned char handle[64], void** ptr);
int b200_peer_close(void* ptr);

/* Several GPUs of one node from ONE process: the row-sharded GEMM behind a handle, for a C or C++
 * harness in the style of the reference's second main (matmul_h100_optimal.cu:115-229: allocate,
 * fill, launch in a loop, time). Rank p of `world` (<= 8) runs on devices[p] (NULL: device p) and
 * owns device buffers A [M_shard, K], B [N, K] and C; the caller fills A and B (b200_mgemm_buffers
 * hands the pointers out) and reads C.
 *   gather = 0  C is [M_shard, N] per rank; the ranks exchange nothing.
 *   gather = 1  C is the full [world * M_shard, N] on every rank, written by every rank's kernel
 *               through peer access (the fused epilogue of b200_gemm_bf16_gather); needs N % 8 == 0
 *               and peer access between the devices (B200_ERR_UNSUPPORTED_CFG otherwise).
 * b200_mgemm_run enqueues one launch per device on the handle's own streams and returns;
 * b200_mgemm_sync waits for all of them — after it, with gather = 1, every copy of C is complete —
 * and reports the slowest device's time for the last run, from CUDA events on the launching
 * streams. The current device is left as it was. A gather over NCCL instead of the fused epilogue is
 * offered by the Python layer only (h100_gemm_b200/sharding.py), so that this library does not
 * link a collective library. The reference has no multi-GPU path. */
typedef struct b200_mgemm b200_mgemm;
int b200_mgemm_create(b200_mgemm** handle, int world, const int* devices, int M_shard, int N, int K, int gather);
int b200_mgemm_buffers(b200_mgemm* handle, int rank, void** A, void** B, void** C);
int b200_mgemm_run(b200_mgemm* handle);
int b200_mgemm_sync(b200_mgemm* handle, float* ms_max);
int b200_mgemm_destroy(b200_mgemm* handle);

/* Replaces reference_gpu_gemm(GemmParams) — reference.h:49-90: a plain SIMT GEMM (one thread per
 * 4x4 outputs, k ascending, fp32) used as an on-device cross-check for shapes too large for the
 * CPU oracle. */
int b200_reference_gpu_gemm_bf16(int M, int N, int K, const void* A, const void* B, void* C,
                                 float alpha, float beta, void* stream);

/* fp16 counterpart of b200_reference_gpu_gemm_bf16 (reference_gpu_gemm<half_t,...>, the check the
 * reference's template main runs, matmul_h100.cu.jinja:1043-1044). */
int b200_reference_gpu_gemm_f16(int M, int N, int K, const void* A, const void* B, void* C, float alpha,
                                float beta, void* stream);

/* Synchronises the current device and reports the device-side status word: out[0] = 0 when no
 * bounded wait has given up since the last call; otherwise out[0] = role code, out[1] = block,
 * out[2] = tile, out[3] = detail. Returns B200_OK or B200_ERR_DEVICE_TIMEOUT; the word is
 * cleared. (The reference's waits are unbounded, barrier.cuh:47-62.) */
int b200_gemm_last_device_status(unsigned int out[4]);

/* Optional tracing. While a device buffer of at least 8 * (number of CTAs) 64-bit words is
 * registered, every bf16 launch (b200_gemm_bf16_gather included) runs the tracing build of the kernel (a few percent slower) and
 * writes eight cycle counters per CTA: [0] total, [1] producer wait, [2] MMA wait for operands,
 * [3] MMA wait for an accumulator buffer, [4] epilogue wait, [5] accumulator drain, [6] epilogue
 * busy, [7] tiles ([4]-[7] are those of the first epilogue warp). buffer == NULL switches it off. This is the working version of the debug
 * buffer `DB` the reference allocates for per-SM load/compute/store cycle sums but never fills
 * (matmul_h100_optimal.cu:132-139,167-198). */
int b200_gemm_set_profile_buffer(void* buffer, size_t bytes);

/* Failure-detection self-test: launches a one-block kernel that waits, for at most
 * `budget_cycles` SM cycles (<= 2^31), on an mbarrier nothing arrives on. The wait gives up, the
 * kernel returns normally and b200_gemm_last_device_status() then reports out[0] == 9. No
 * counterpart in the reference, whose waits cannot give up (barrier.cuh:47-62,
 * matmul_utils.cuh:279-293). */
int b200_gemm_selftest_bounded_wait(long long budget_cycles);

const char* b200_gemm_strerror(int status);
/* cudaError_t / CUresult value of the most recent failing CUDA call on this thread. */
int b200_gemm_last_cuda_error(void);
/* Multiprocessor count of the current device (get_sm_count, common.h:43-60); <= 0 on error. */
int b200_gemm_sm_count(void);

#ifdef __cplusplus
}
#endif
#endif /* B200_GEMM_H_ */
