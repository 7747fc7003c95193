/* beam_b200 — C ABI of the B200 (sm_100a) kernels behind BEAM's fp16 "rc" GEMM registry.
 *
 * rc GEMM:  C[M,N] (fp16, row-major) = A[M,K] (fp16, row-major) x B[N,K]^T (B stored [N,K], i.e.
 * column-major KxN), fp32 accumulation, one round-to-nearest-even to fp16 at the end, alpha = 1,
 * beta = 0.  (Reference semantics: cuda/cute_kernels/main.cc:29-40, cute_gemm_128x128.cu:89-92,183,
 * cuda/cutlass_kernels/cutlass_gemmrc.cu:22-30.)
 *
 * Conventions for every entry point:
 *   - all pointers are DEVICE pointers on the CUDA device current on the calling thread, unless a
 *     parameter is documented as host memory; A, B, C and workspace must be 16-byte aligned;
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream); calls are
 *     asynchronous with respect to the host and re-entrant across streams;
 *   - the return value is a BEAM_* status; nothing here ever calls exit() or throws.  The reference's
 *     entry functions return void and exit(-1) / std::terminate / silently do nothing on error
 *     (cuda/include/cuda_utils.h:7-23, torch_utils.h:7-37, cutlass_gemmrc.cu:33-37);
 *   - shapes: K % 8 == 0 and N % 8 == 0 (16-byte rows for TMA); M, N, K need not be tile multiples
 *     (out-of-range tile parts are zero-filled on load and masked on store).
 *   - device-pointer entry points allocate nothing after the first call on a device (that call
 *     creates a small fault word); split-K and LayerNorm scratch is caller-provided.
 */
#ifndef BEAM_B200_H_
#define BEAM_B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define BEAM_API __attribute__((visibility("default")))
#else
#define BEAM_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define BEAM_OK 0
#define BEAM_ERR_INVALID_ARG 1     /* null pointer, non-positive size, bad enum */
#define BEAM_ERR_UNSUPPORTED 2     /* shape / tile / split factor this build cannot run */
#define BEAM_ERR_ALIGNMENT 3       /* pointer not 16-byte aligned or K, N not multiples of 8 */
#define BEAM_ERR_WORKSPACE 4       /* workspace missing or too small */
#define BEAM_ERR_CUDA 5            /* a CUDA runtime call failed (see beam_last_cuda_error) */
#define BEAM_ERR_TENSORMAP 6       /* the driver refused a TMA descriptor */
#define BEAM_ERR_DEVICE_TIMEOUT 7  /* a kernel's bounded wait ran out (see beam_device_status) */
#define BEAM_ERR_NO_DEVICE 8       /* no sm_100 device is current */

/* Blackwell tuning knobs; zero in any field means "library default".  This is what replaces the
 * reference's shape_threadblock / shape_warp vectors (cuda/cutlass_kernels/main.cc:129-141) in
 * the auto-tuner's search space. */
typedef struct beam_gemm_cfg {
  int tile_n;         /* output tile N: 64, 128, 256, or 512 (two UMMA N = 256 halves, pair only)   */
  int cta_pair;       /* 1 = one CTA per 128-row tile; 2 = cta_group::2 pair on a 256-row tile */
  int stages;         /* depth of the TMA->UMMA shared-memory ring (2..8)                      */
  int group_m;        /* tile rasterisation: M-tiles per L2 group                              */
  int split_k_slices; /* split-K only: number of K slices (0 = heuristic)                      */
  int max_ctas;       /* cap on the persistent grid (0 = all SMs); -1 with tile_n = 512: one tile per
                         CTA pair instead of a persistent grid                                  */
  int l2_hints;       /* L2 eviction policy, three decimal digits: hundreds = C stores, tens = A loads,
                         ones = B loads; 0 none (default: loads without a policy stay eligible for
                         merging by the L2 request coalescer), 1 evict-first, 2 evict-last         */
  int flags;          /* BEAM_FLAG_* bits                                                       */
  int tile_m;         /* 0 = 128 rows per CTA; 512 (with tile_n = 256, cta_pair = 2) = 512 x 256 tile per
                         CTA pair: two 256-row accumulators that multiply by the same B operand       */
  int tiles_in_flight; /* tile_n = 128 with stages = 0 only: 0 or 2 = the CTA (pair) works on two neighbouring tiles at
                         once and alternates its UMMAs between their accumulators (a UMMA of N = 128 is shorter than
                         the wait for its predecessor's result); 1 = one tile at a time                     */
} beam_gemm_cfg;

/* Split-K only.  The caller guarantees that A and B are not outputs of the kernel that immediately precedes
 * this call on the stream (they were complete before that kernel started).  The first kernel of the call is
 * a programmatic dependent launch; with this flag it starts streaming A and B while the preceding kernel
 * (typically the previous split-K call's reduction) is still finishing, and only its writes wait for that
 * kernel to complete.  Without the flag it waits before its first global read, which is always safe. */
#define BEAM_FLAG_INPUTS_STABLE 1
/* beam_gemmrc_fp16 only: A, B and C hold bf16 instead of fp16 (same kernels; fp32 accumulation, one rounding to
 * bf16).  The reference reaches bf16 only through its cuBLAS comparator (cuda/cublas.cc:106-108). */
#define BEAM_FLAG_BF16 2
/* Split-K only.  Run the call as two kernels (partials, then a reduction kernel) even where the one-kernel form
 * applies.  Both forms add the partials in the same order and agree bit for bit; this flag exists for comparison
 * and for callers that must not launch cooperative grids. */
#define BEAM_FLAG_SPLITK_TWO_KERNELS 4
/* Split-K only.  Run the call as one kernel wherever that form applies, including calls that carry
 * BEAM_FLAG_INPUTS_STABLE (which run as two kernels by default). */
#define BEAM_FLAG_SPLITK_ONE_KERNEL 8
/* beam_gemmrc_fp16 with 256 x 256 tiles on CTA pairs only.  By default, when the tiles of the persistent grid's last
 * wave occupy at most half of the CTA pairs, each of them is computed as two 128-column halves by two pairs, and a
 * half tile adds up the even and the odd 64-wide blocks of K separately before adding the two sums (two UMMA chains
 * keep the tensor pipe busy where one chain of N = 128 instructions cannot).  The order is fixed, so results are
 * reproducible run to run, but an element of a cut tile can differ in its last bit from the same element computed in
 * a whole tile.  This flag keeps every tile whole: one summation order everywhere, for comparison and for callers
 * that compare bits across different shapes. */
#define BEAM_FLAG_WHOLE_TILES 16

BEAM_API const char* beam_status_string(int status);
/* Text of the last CUDA runtime error seen by this thread inside the library ("" if none). */
BEAM_API const char* beam_last_cuda_error(void);
/* Library build tag, e.g. "beam_b200 sm_100a". */
BEAM_API const char* beam_version(void);

/* Reads the current device's fault word (synchronises the device). 0 = healthy.  Non-zero values
 * are DeviceFault codes written by a kernel whose bounded wait expired. `clear` != 0 resets it. */
BEAM_API int beam_device_status(int clear, int* fault_word_out);

/* ---- large rc GEMM -------------------------------------------------------------------------- */

/* Generic entry: persistent warp-specialised TMA + tcgen05 kernel, configuration from cfg (NULL =
 * defaults).  Everything below is a named preset of this. */
BEAM_API int beam_gemmrc_fp16(const void* A, const void* B, void* C, int m, int n, int k, const beam_gemm_cfg* cfg,
                     void* stream);

/* Row-sharded GEMM fused with the all-gather of C (no counterpart in the reference, which is single-GPU).
 * Rank `rank` of `world` (<= 8, one process per GPU) multiplies its m_local rows of A by all of B and stores
 * every finished tile of C straight into row block `rank` of each GPU's gathered C[world * m_local, N]:
 * C_gathered[d] is the device pointer, valid in THIS process, of rank d's gathered buffer (its own for
 * d == rank, peer-mapped memory for the others: CUDA IPC / VMM / torch symmetric memory).  The epilogue issues
 * one plain TMA store per destination over NVLink, so the gather overlaps the main loop tile by tile.
 * The call returns after the launch; the gathered buffers are complete once every rank's kernel has
 * finished (a host- or stream-level barrier across the ranks after it).  m_local must be the same on all ranks. */
BEAM_API int beam_gemmrc_fp16_allgather(const void* A_local, const void* B, void* const* C_gathered, int world,
                                        int rank, int m_local, int n, int k, const beam_gemm_cfg* cfg, void* stream);

/* Registry name `custom_gemmrc_128x128` — replaces entry_custom_gemmrc_128x128
 * (cuda/cute_kernels/cute_gemm_128x128.cu:193-205, declared cuda/cute_kernels/main.cc:13-14):
 * 128x128 output tile per CTA. */
BEAM_API int beam_custom_gemmrc_128x128(const void* A, const void* B, void* C, int m, int n, int k, void* stream);

/* Registry name `custom_gemmrc_128x256` — replaces entry_custom_gemmrc_128x256
 * (cuda/cute_kernels/cute_gemm_128x256.cu:196-208, declared cuda/cute_kernels/main.cc:15-16):
 * 128x256 output tile per CTA. */
BEAM_API int beam_custom_gemmrc_128x256(const void* A, const void* B, void* C, int m, int n, int k, void* stream);

/* Registry name `cutlass_gemmrc` — replaces entry_cutlass_gemmrc (cuda/cutlass_kernels/
 * cutlass_gemmrc.cu:21-40): the library's best default: CTA pairs on 256x512 tiles when the problem has
 * at least four waves of them, 256x256 tiles otherwise. */
BEAM_API int beam_cutlass_gemmrc(const void* A, const void* B, void* C, int m, int n, int k, void* stream);

/* Registry name `cutlass_gemmrc_spec` — replaces entry_cutlass_gemmrc_spec (cuda/cutlass_kernels/
 * cutlass_gemmrc.cu:55-111).  shape_threadblock = {tb_m, tb_n} selects the tile family:
 * {128,128}, {128,256} -> one CTA per tile; {256,128}, {256,256}, {256,512} -> CTA pair.  shape_warp is accepted
 * for signature compatibility and ignored (a UMMA has no warp tile).  Unlike the reference, an
 * unknown shape returns BEAM_ERR_UNSUPPORTED instead of silently doing nothing (:73-80). */
BEAM_API int beam_cutlass_gemmrc_spec(const void* A, const void* B, void* C, int m, int n, int k, int tb_m, int tb_n,
                             int warp_m, int warp_n, void* stream);

/* ---- split-K rc GEMM for small M, N and huge K ------------------------------------------------ */

/* Scratch bytes the split-K entry points need: fp32 partials [slices][M][N] (the layout of the
 * reference's CUTLASS workspace).  tile_n = 0 and split_k_slices = 0 mean "what the library would
 * pick"; pass the same values as to the entry point. */
BEAM_API size_t beam_gemmrc_splitk_workspace_bytes(int m, int n, int k, int tile_n, int split_k_slices);

/* The split factor the heuristic picks for this tile_n (0 = default tile) for a plain call on the current device:
 * work items for about two thirds of the SMs (seven eighths for folded problems, M and N <= 64), at least 256 of K
 * per slice; values measured on B200 with chains of dependent calls.  Replaces get_slice_heuristic
 * (cuda/cutlass_kernels/cutlass_gemmrc_splitk.cu:44-57), which models the 108 SMs of an A100. */
BEAM_API int beam_gemmrc_splitk_heuristic(int m, int n, int k, int tile_n);

/* How a split-K call with these arguments runs on the current device: info[0] = tile N, info[1] = K slices,
 * info[2] = 1 if the problem runs folded (M, N <= 64: two k-blocks per UMMA), info[3] = kernels per call (1 or 2),
 * info[4] = 1 if the call's first kernel is a programmatic dependent launch.  info must hold 5 ints. */
BEAM_API int beam_gemmrc_splitk_describe(int m, int n, int k, int tile_n, int split_k_slices, int flags, int* info);

/* Generic split-K entry: cfg->tile_n (0 = default), cfg->split_k_slices (0 = heuristic) and cfg->flags
 * (BEAM_FLAG_INPUTS_STABLE, BEAM_FLAG_SPLITK_TWO_KERNELS, BEAM_FLAG_SPLITK_ONE_KERNEL) are honoured; cfg may be NULL.  The two registry names
 * below are presets. */
BEAM_API int beam_gemmrc_splitk_fp16(const void* A, const void* B, void* C, int m, int n, int k,
                                     const beam_gemm_cfg* cfg, void* workspace, size_t workspace_bytes,
                                     void* stream);

/* Registry name `cutlass_gemmrc_splitk` — replaces entry_cutlass_gemmrc_splitk (cuda/cutlass_kernels/
 * cutlass_gemmrc_splitk.cu:59-105).  K is cut into `split_k_slices` contiguous runs of 64-wide
 * k-blocks; each CTA accumulates one slice of one tile in TMEM and writes an fp32 partial to
 * `workspace`; the partials of every output are then added in a fixed order that depends only on the
 * slice count (bitwise reproducible) and rounded once to fp16.  When every (tile, slice) fits on the
 * device at once (tiles x slices <= SM count, which the heuristic guarantees) this is ONE cooperative
 * kernel: after a grid-wide barrier each CTA sums its share of the output; otherwise a second kernel does
 * the sum.  The reference always launches two kernels (gemm_splitk_parallel + reduce).  A split factor outside
 * [1, K/64] falls back to the heuristic, as the reference does for values outside (0, K/32) (:77-94).
 * The reference keeps a hidden grow-only cudaMalloc'd buffer (:31-42); here the caller owns it. */
BEAM_API int beam_cutlass_gemmrc_splitk(const void* A, const void* B, void* C, int m, int n, int k, int split_k_slices,
                               void* workspace, size_t workspace_bytes, void* stream);

/* Registry name `cutlass_gemmrc_splitk_spec` — replaces entry_cutlass_gemmrc_splitk_spec
 * (cuda/cutlass_kernels/cutlass_gemmrc_splitk.cu:107-195).  tb_n selects the UMMA N of the tile
 * (64, 128 or 256); tb_m and shape_warp are accepted and ignored (tiles are always 128 rows, rows
 * beyond M are zero-filled). */
BEAM_API int beam_cutlass_gemmrc_splitk_spec(const void* A, const void* B, void* C, int m, int n, int k, int tb_m,
                                    int tb_n, int warp_m, int warp_n, int split_k_slices, void* workspace,
                                    size_t workspace_bytes, void* stream);

/* Split-K for callers that must not allocate (no counterpart in the reference, whose split-K grows a
 * hidden cudaMalloc'd buffer on demand).  Same arithmetic and kernels as beam_cutlass_gemmrc_splitk, but
 * the fp32 partials live in a 16 MiB array that is part of the library's device image, so the caller passes
 * only inputs and outputs: for host threads in latency-critical loops (cudaMalloc/cudaFree serialise on the
 * driver's allocator and cudaFree synchronises the device), for processes that gave all device memory to
 * another allocator at start-up, and for runtimes that forbid allocation after initialisation.
 *   - limit: slices * M * N * 4 bytes <= 16 MiB, otherwise BEAM_ERR_WORKSPACE (use the workspace entry);
 *     the array occupies 16 MiB on every GPU that loads the library until the process exits;
 *   - the first call on a device does a one-time set-up (symbol address, kernel attributes) and is
 *     therefore slower than the calls after it;
 *   - calls no cudaMalloc / cudaFree / allocating routine and does not touch the library's per-device
 *     context, so beam_device_status() does not see its kernels: pass `device_fault_word` (a zeroed
 *     4-byte device int of your own, or NULL) to receive a DeviceFault code if a bounded wait expires;
 *   - all calls on a device share the array, which keeps the previous call's contents (nothing in it needs
 *     to start at zero; each call overwrites what it reads).  Calls that overlap on the GPU race. */
BEAM_API int beam_gemmrc_splitk_noalloc(const void* A, const void* B, void* C, int m, int n, int k,
                                        int split_k_slices, int* device_fault_word, void* stream);

/* ---- fused GEMM + LayerNorm --------------------------------------------------------------------- */

/* Scratch bytes for beam_gemmrc_layernorm on the current device: row statistics exchanged between the N tiles
 * (8 bytes per row per 256 columns) and tickets; when N needs more 256-wide tiles than the device has CTA pairs
 * (N > 18944 on 148 SMs) also an fp32 panel of M x N. */
BEAM_API size_t beam_gemmrc_layernorm_workspace_bytes(int m, int n, int k);

/* Registry slot `cutlass_parallel_gemmrc_lnr` (cuda/cute_kernels/main.cc:55-76,87; the reference
 * kernel behind it, cute_gemm_ln.cu:24-245, is a GEMM next to an unrelated SiLU and has no LayerNorm).
 * out[M,N] = LayerNorm_row( X[M,K] x W[N,K]^T ) * gamma[N] + beta[N]: mean and population variance per
 * output row in fp32 from the fp32 accumulators, rstd = rsqrt(var + eps), result rounded once to fp16. */
BEAM_API int beam_gemmrc_layernorm(const void* X, const void* W, void* out, const void* gamma, const void* beta, float eps,
                          int m, int n, int k, void* workspace, size_t workspace_bytes, void* stream);

/* ---- GEMM with a co-scheduled element-wise SiLU ------------------------------------------------- */

/* What the reference kernel behind `cutlass_parallel_gemmrc_lnr` really computes (cuda/cute_kernels/
 * cute_gemm_ln.cu:24-245, entry :230-245): C = A x B^T and, independently, y[i] = x[i] / (1 + exp(-x[i])) for
 * `count` halves of a second tensor (fp32 math, fp16 in and out).  The reference parks the element-wise work on
 * a quarter of its CTAs; here the epilogue warps of the persistent GEMM work through it, 1024 elements at a time,
 * while they wait for their next accumulator.  x, y: 16-byte aligned device pointers; x may equal y. */
BEAM_API int beam_gemmrc_silu(const void* A, const void* B, void* C, int m, int n, int k, const void* x, void* y,
                              long long count, void* stream);

/* ---- host-buffer convenience (what a caller with pageable or pinned HOST arrays uses) ---------- */

/* A, B, C are HOST pointers (pinned memory for full PCIe speed).  A and B go to the device in alternating row
 * blocks; after every arrival the strip of C that has become computable is multiplied and copied back, so both
 * directions of the link are busy from the second block on; blocks until C is complete.  Device staging buffers
 * are allocated on the first call on a device and reused while they fit; calls on one device run one at a time. */
BEAM_API int beam_gemmrc_fp16_host(const void* A_host, const void* B_host, void* C_host, int m, int n, int k);

/* The same with B already resident on the device (B_dev: device pointer, [N,K] fp16, 16-byte aligned): only A goes
 * up and only C comes back.  For the ranks of a row-sharded job (no counterpart in the reference, which is
 * single-GPU): each rank uploads 1/world of B, the ranks all-gather B over NVLink, and every step then moves just
 * the rank's own rows of A and C over PCIe. */
BEAM_API int beam_gemmrc_fp16_host_rows(const void* A_host, const void* B_dev, void* C_host, int m, int n, int k);

#ifdef __cplusplus
}
#endif
#endif /* BEAM_B200_H_ */
