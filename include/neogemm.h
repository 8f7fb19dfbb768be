/* neogemm.h - C ABI of the B200 (sm_100a) BF16 GEMM library, libneogemm.so.
 *
 * One operation:  C = A * B^T  with bf16 A[M,K] (row-major), bf16 B[N,K] (row-major, i.e. K-major),
 * fp32 accumulation and a bf16 (round-to-nearest-even) result.  This is the operation of the
 * reference's PyTorch-extension function neoGemmV1(A, B, C) (nemgemmV03.cu:343-391; older name
 * neogemm(), neogemmV02.cu:262-303), driven by benchmark.py:24.
 *
 * Plain pointers and sizes only: no torch or C++ types cross this boundary.  All device pointers
 * must belong to the CUDA device that is current on the calling thread.  Calls are asynchronous
 * with respect to the host unless stated otherwise; `stream` is a cudaStream_t passed as void*
 * (NULL = the legacy default stream, which is what the reference launches on,
 * nemgemmV03.cu:383).
 *
 * There is no CPU fallback.  Every function that needs a GPU fails with an error code when no
 * usable sm_100 device is current.
 */
#ifndef NEOGEMM_H_
#define NEOGEMM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Return codes.  0 is success; everything else leaves C unspecified. */
enum neogemm_status {
  NEOGEMM_OK = 0,
  NEOGEMM_ERR_BAD_ARG = 1,        /* null pointer, negative size, bad leading dimension */
  NEOGEMM_ERR_UNSUPPORTED = 2,    /* K % 8 != 0, lda/ldb % 8 != 0, misaligned A/B, or not sm_100 */
  NEOGEMM_ERR_DESCRIPTOR = 3,     /* cuTensorMapEncodeTiled failed or is unavailable */
  NEOGEMM_ERR_LAUNCH = 4,         /* cudaLaunchKernelEx / attribute set-up failed */
  NEOGEMM_ERR_DEVICE_TIMEOUT = 5, /* an earlier launch on this device reported a bounded wait that
                                     expired; see neogemm_device_status() */
  NEOGEMM_ERR_WORKSPACE = 6,      /* caller's workspace too small, or internal allocation failed */
  NEOGEMM_ERR_CUDA = 7            /* any other CUDA runtime error (copy, allocation, sync) */
};

/* C = A * B^T on device memory.
 *
 * Replaces the body of neoGemmV1 (nemgemmV03.cu:343-391): that function reads M = A.size(0),
 * K = A.size(1), N = B.size(0) (:344-346), builds two tensor maps and launches one 64x64 tile per
 * CTA.  Here the same three sizes arrive explicitly, with leading dimensions in ELEMENTS.
 *
 *   A   [M,K] bf16, element (i,k) at A[i*lda + k]          lda >= K, lda % 8 == 0, 16-B aligned
 *   B   [N,K] bf16, element (j,k) at B[j*ldb + k]          ldb >= K, ldb % 8 == 0, 16-B aligned
 *   C   bf16 result.
 *       c_col_major == 0: element (i,j) at C[i*ldc + j], ldc >= N   (row-major [M,N])
 *       c_col_major != 0: element (i,j) at C[j*ldc + i], ldc >= M   (column-major, which is what
 *                         the reference writes, neogemmV02.cu:236,242, and why benchmark.py:25
 *                         transposes the view afterwards)
 *   M, N >= 0 (0 is a no-op), K >= 0 with K % 8 == 0 (K == 0 writes zeros).
 *       The reference requires multiples of 64 in all three (nemgemmV03.cu:375); edges are
 *       handled here by TMA zero-fill and clipped stores.
 *   workspace / workspace_bytes: scratch for the stream-K schedule used on skinny shapes
 *       (neogemm_workspace_bytes() says how much).  NULL selects a library-owned per-device
 *       buffer that is allocated on first use; that buffer is shared by all calls on the device,
 *       so concurrent launches on different streams must pass their own workspaces.  A caller's
 *       workspace must be zero-filled once before its first use; the kernel leaves it reusable.
 *   stream: cudaStream_t.
 */
int neogemm_bf16_nt(const void* A, const void* B, void* C,
                    int64_t M, int64_t N, int64_t K,
                    int64_t lda, int64_t ldb, int64_t ldc,
                    int c_col_major,
                    void* workspace, size_t workspace_bytes,
                    void* stream);

/* Fused epilogue:  C = act(alpha * A * B^T + beta * C + bias), computed in fp32 on the
 * accumulator before the single rounding to bf16.
 *   alpha, beta : fp32 scalars; with beta != 0 the previous contents of C are read (same layout)
 *   bias        : NULL, or N bf16 values, bias[j] added to column j of C = A * B^T (the bias of a
 *                 linear layer whose weight is B)
 *   activation  : 0 none, 1 ReLU, 2 GELU (tanh form)
 * Everything else as neogemm_bf16_nt(); K must be > 0.  The reference declares alpha and beta as
 * kernel parameters and comments the intent but never implements it (neogemmv4.cu:166,266). */
int neogemm_bf16_nt_fused(const void* A, const void* B, void* C,
                          int64_t M, int64_t N, int64_t K,
                          int64_t lda, int64_t ldb, int64_t ldc, int c_col_major,
                          float alpha, float beta, const void* bias, int activation,
                          void* workspace, size_t workspace_bytes, void* stream);

/* The fused product with an fp32 result: C holds 4-byte floats and receives
 * act(alpha * A * B^T + beta * C + bias) unrounded (the fp32 accumulator after the epilogue
 * arithmetic), so a caller that goes on computing in fp32 - a loss, a reduction over several
 * products - does not pay a bf16 rounding in between.  With beta != 0 the previous fp32 contents
 * of C are read.  ldc is in ELEMENTS (floats); C must be 4-byte aligned; the TMA-store kernels
 * are used when ldc % 4 == 0 and C is 16-byte aligned, the direct-store kernels otherwise.
 * Everything else as neogemm_bf16_nt_fused().  This is the other half of the intent the reference
 * only sketches (alpha/beta parameters and an unfinished epilogue, neogemmv4.cu:166,266-267). */
int neogemm_bf16_nt_fused_f32(const void* A, const void* B, void* C,
                              int64_t M, int64_t N, int64_t K,
                              int64_t lda, int64_t ldb, int64_t ldc, int c_col_major,
                              float alpha, float beta, const void* bias, int activation,
                              void* workspace, size_t workspace_bytes, void* stream);

/* The same product for callers that must not allocate: it calls no cudaMalloc, cudaFree,
 * cudaHostAlloc or any other allocating routine, on any call.  (No counterpart in the reference.)
 *
 * Meant for code that cannot ask the CUDA allocator for memory when it multiplies: a serving
 * loop whose own pool already holds the whole device, a latency-critical path that cannot afford
 * an allocation or its failure, a plugin that may not touch the host process's allocator.
 * neogemm_bf16_nt() can allocate (a pinned status word on its first call per device, and a
 * library-owned workspace when a skinny shape takes the stream-K schedule); this one uses a fixed
 * 32 MiB array compiled into the library as its stream-K scratch, which every GPU that loads
 * libneogemm.so holds until the process exits.
 *
 * Arguments as for neogemm_bf16_nt(), without the workspace pair.  Differences:
 *   - a shape whose stream-K scratch (256 KiB of counters + one fp32 partial tile per contributor
 *     of every cut tile) would exceed the 32 MiB returns NEOGEMM_ERR_WORKSPACE.  That is not only
 *     very long skinny shapes: a large result that cannot take the TMA-store kernels (packed
 *     row-major C with N % 8 != 0, e.g. 8192 x 1001) is planned as cut 128 x 128 tiles and is
 *     refused as well - use neogemm_bf16_nt() for those.  The benchmark's decode shapes
 *     (M <= 128, N = 28672, K = 8192) run as one wave of whole tiles and need no scratch at all;
 *     64 x 3584 x 2048 uses 3.8 MiB of it, 16 x 40960 x 4096 (cut tiles plus run-time claimed
 *     pieces) 7.8 MiB;
 *   - the first call on each device looks up the device address of the array
 *     (cudaGetSymbolAddress) and the driver's tensor-map encoder; make that first call - or
 *     neogemm_noalloc_init() - before starting any stream capture;
 *   - the CUDA driver loads a library's code and static data onto a device lazily, on first use.
 *     That first use (32 MiB plus the kernels) needs device memory that this library never asks
 *     for but the driver does: call neogemm_noalloc_init() BEFORE the pool takes the device.  A
 *     set-up that failed is retried on the next call, it is not remembered;
 *   - all calls on a device share the one array: calls whose kernels may overlap on the GPU
 *     (different streams) race on it - serialise them, or use neogemm_bf16_nt() with separate
 *     workspaces.  The part that must start at zero is cleared in stream order by every call;
 *   - device-side errors (an expired bounded wait, an index that failed the kernel's own bounds
 *     check) are recorded in a word in DEVICE memory, which neogemm_device_status() does not
 *     show: read it with neogemm_noalloc_status().  Once that has seen an error, this entry point
 *     returns NEOGEMM_ERR_DEVICE_TIMEOUT until neogemm_noalloc_clear_status();
 *   - thread-local overrides and tuning knobs are ignored; neogemm_last_config() reports the
 *     plan of the most recent call as usual.
 */
int neogemm_bf16_nt_noalloc(const void* A, const void* B, void* C,
                            int64_t M, int64_t N, int64_t K,
                            int64_t lda, int64_t ldb, int64_t ldc,
                            int c_col_major, void* stream);

/* Companions of neogemm_bf16_nt_noalloc(); none of them allocates.  (No counterpart in the
 * reference.)
 *
 * neogemm_noalloc_init(): makes the driver load everything the entry point can ever launch on the
 *   current device - the fixed scratch array, its status word and every kernel variant - and
 *   zeroes the status word.  Call it once per device while device memory is still available
 *   (before the caller's pool claims it) and before any stream capture; afterwards no shape can
 *   meet a kernel that still has to be placed on the device.  Synchronous.  Safe to repeat.
 * neogemm_noalloc_status(out, stream): waits for `stream`, then copies the device-side error
 *   record of the entry point into out[4] (same fields as neogemm_device_status()).  Synchronous;
 *   meant for the end of a batch or a health check, not for every call.
 * neogemm_noalloc_clear_status(): waits for the device, clears the record, re-opens the entry
 *   point after an error. */
int neogemm_noalloc_init(void);
int neogemm_noalloc_status(int out[4], void* stream);
int neogemm_noalloc_clear_status(void);

/* Upper bound on the workspace neogemm_bf16_nt() may need for this shape on the current device
 * (0 when the data-parallel schedule would be chosen).  No counterpart in the reference, which
 * has no split-K. */
size_t neogemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int c_col_major);

/* Same product with HOST buffers: copies A and B to the device, runs the kernel and copies C
 * back, then waits.  The work is ordered after what is already queued on `stream`; internally
 * the operand that indexes the stored rows of C goes up in row chunks on a copy queue of the
 * library's own, each chunk's product is launched on `stream` as it lands and its rows of C
 * return on a second copy queue, so that both PCIe directions and the GPU overlap (pinned host
 * memory is needed for that; pageable memory works but serialises).  Packed layouts (lda = ldb = K; ldc = N, or
 * M when c_col_major).  Device staging buffers are owned by the library and reused across calls.
 * This is the call a host program without device memory of its own makes; the reference's
 * counterpart is the cublass/matmul.cu flow (host malloc -> cudaMemcpy -> kernel -> cudaMemcpy,
 * matmul.cu:95-120,146-149). */
int neogemm_bf16_nt_host(const void* A_host, const void* B_host, void* C_host,
                         int64_t M, int64_t N, int64_t K,
                         int c_col_major, void* stream);

/* Device-side error record of the current device: out[0] = code (0 none; 1 producer wait expired,
 * 2 MMA operand wait, 3 MMA accumulator wait, 4 epilogue wait, 5 tensor-memory address,
 * 6 an index failed the kernel's own bounds check and the access was skipped, 7 a wait on the
 * run-time work queue expired),
 * out[1] = CTA index, out[2] = segment index, out[3] = ring stage or accumulator.  Meaningful once
 * the stream of the launch has been synchronised.  The reference only prints cudaGetLastError
 * (nemgemmV03.cu:387-390). */
int neogemm_device_status(int out[4]);

/* Clears the device-side error record of the current device. */
int neogemm_clear_device_status(void);

/* Human-readable text for a return code. */
const char* neogemm_status_str(int status);

/* Kernel configuration chosen by the most recent neogemm_bf16_nt() on this thread:
 * out[0] = CTAs per tile (1 or 2), out[1] = tile columns (UMMA N), out[2] = ring stages,
 * out[3] = 1 if operands were swapped (B rows on the 128-lane axis), out[4] = 1 if stream-K
 * (all tiles for skinny shapes, the last partly filled wave for large ones),
 * out[5] = CTAs launched, out[6] = tiles, out[7] = raster group height. */
int neogemm_last_config(int out[8]);

/* How the tiles of the most recent neogemm_bf16_nt*() call on this thread left the SMs:
 * 0 the kernel's regular epilogue (TMA-store boxes of 32 rows, or stores from registers),
 * 1 a tall tile staged whole in the idle operand ring and stored as one TMA box,
 * 2 the same with the operands' roles exchanged in the MMA (pairs of 128-column tall tiles).
 * For tests and benchmarks; no counterpart in the reference. */
int neogemm_last_store_path(void);

/* Tuning / test override for the calling thread; -1 leaves a field to the heuristic.
 *   cta_group: 1 or 2;  block_n: 16,32,64,128,256;  swap: 0/1;  stream_k: 0/1;
 *   group_m: raster group height in tiles;  max_ctas: cap on launched CTAs. */
int neogemm_set_override(int cta_group, int block_n, int swap, int stream_k, int group_m,
                         int max_ctas);

/* Tuning knobs of the calling thread; value -1 restores the library default.
 *   key 0: L2 eviction hints of the TMA copies.  Bit 0: loads of the operand on the 128-lane axis
 *          are evict-last; bit 1: loads of the other operand are evict-first; bit 2: stores of C
 *          are evict-first; bit 3: 128-lane operand evict-first; bit 4: other operand evict-last.
 *   key 1: nanoseconds the epilogue warps may stay suspended in one mbarrier.try_wait while they
 *          wait for a finished accumulator (0 = plain try_wait).
 *   key 2: the same for the TMA producer's and the MMA warp's waits on the operand ring.
 *   key 3: the 256 x 512 pair tile (two UMMA-N halves sharing one operand): 0 never, 1 whenever
 *          the shape allows, -1 chosen by estimated time.
 *   key 5: L2 promotion of the TMA loads: 0 none, 1 64 B, 2 128 B, 3 256 B (default).
 *   key 4: pieces (of 16 k-blocks) per tile that the stream-K schedule of skinny shapes leaves to
 *          be claimed at run time instead of assigning them statically (0 = none, up to 4).
 *   key 6: two-half tiles: k-blocks (1..3) issued for the first half alone at the start of a tile,
 *          while the epilogue still reads the second half of the previous tile.
 *   key 7: skinny shapes that need between one and two 128-row tiles per SM run as ONE wave of
 *          whole tiles (no cut tiles, no closing sums): -1 with tall tiles (256 rows per CTA
 *          sharing the small operand, one CTA per SM), 0 not at all (stream-K instead),
 *          1 with 128-row tiles, two CTAs per SM and half-size rings, whenever such a kernel
 *          exists and all tiles fit at once, 2 with tall tiles whenever they fit in one wave,
 *          3 and 4 as -1 with another way out for a tall tile's result (the default stages the
 *          tile in the idle operand ring and stores it as one TMA box; pairs of 128-column tall
 *          tiles also exchange the operands' roles in the MMA, so that no tensor work is spent
 *          on rows past the tile's height): 4 keeps the usual roles, 3 also stores from
 *          registers.
 *   key 8: wave pacing of launches with many waves of whole tiles (workers wait, briefly and
 *          without obligation, for each other at the start of every wave so that tiles sharing
 *          operand panels keep sharing them in L2): -1 from 8 waves on, 0 off, 1 from 2 waves on.
 *   key 9: whole tiles of odd waves walk K backwards, so that the k-slices of a row panel used
 *          last by one wave are asked for first by the next (fewer DRAM reads: 838 -> 752 MB at
 *          8192^3, which under the power cap is worth 0.5-0.8 % of time; the sums of those tiles
 *          then round like a reversed k loop - results stay reproducible launch to launch, the
 *          order is a fixed property of the tile's place in the schedule): -1 on for plain
 *          round-robin schedules of the TMA-store kernels with more than one wave, 0 off, 1 on
 *          for every schedule.
 *   key 10: set-up overlap.  Launches carry the programmatic-stream-serialization attribute, so
 *          a launch's CTAs are placed and initialise barriers and tensor memory while the previous
 *          kernel of the stream drains; the kernel still waits for that kernel's completion before
 *          it touches global memory.  1 or -1 on, 0 off (plain stream order).
 *   key 11: two-pass split-K.  When a launch has fewer tiles than SMs (or SM pairs) and K is
 *          long, every tile is cut into 2..8 equal k-chunks, one per CTA; -1 or 1: the GEMM kernel
 *          only publishes fp32 partials and a reduction kernel launched right behind it sums
 *          them, applies the epilogue and stores C; 0: wide tiles are not cut at all and the
 *          last contributor of a cut narrow tile sums it alone (the earlier behaviour).
 *   key 12: 128 x 64 tiles for small problems (twice as many CTAs as 128 x 128 tiles): -1 when
 *          the 128 x 128 tiles would occupy at most half of the SMs, 0 never, 1 whenever the
 *          single-CTA 128 x 128 TMA-store kernel would be used.
 * No counterpart in the reference (its maps only set L2 promotion, nemgemmV03.cu:52). */
int neogemm_set_tuning(int key, int value);

/* Profiling aid.  While a device buffer is registered on the calling thread, every launch records
 * into it, 16 int64 per CTA.  Clock-cycle sums (added to what is there): [0] producer waiting for
 * a ring slot, [1] producer loop, [2] MMA waiting for operand bytes, [3] MMA waiting for a drained
 * accumulator, [4] MMA loop, [5] first epilogue warp waiting for an accumulator, [6] its loop,
 * [7] segments processed.  Timestamps in %globaltimer nanoseconds (overwritten): [8] CTA start,
 * [9] MMA loop start, [10] MMA loop end, [11] epilogue loop end, [12] CTA end.
 * The buffer must hold 128 bytes per launched CTA and be zeroed by the caller; NULL switches the
 * timers off (the default; the timed paths then cost one predicated branch).  This is the filled-in
 * version of the per-CTA load/compute/store cycle records the reference's harness only reserves
 * (cublass/matmul.cu:99-106,151-165). */
int neogemm_set_phase_timers(void* device_buffer, size_t bytes);

/* Host-only view of the launcher's decisions, for tests and reports; needs no GPU.  Plans the
 * product for a device with `sm_count` SMs and an output pitch `ldc` (16-byte aligned C assumed)
 * and walks the kernel's own work iterator on the host.
 *   plan_out[16]: CTAs per tile, tile columns, stages, swap, stream-K, CTAs, tiles, raster group,
 *                 epilogue (0 TMA store, 1 direct), Md, Nd, tile rows, tile columns, k-blocks,
 *                 partial slots per tile, first tile of the stream-K region.
 *   segments: up to max_segments records of 8 ints {worker, tile, first k-block, k-blocks,
 *                 contributor index, contributors, tile row, tile column} (may be NULL).
 * Returns the number of segments, or minus a neogemm_status code.  No counterpart in the
 * reference, whose schedule is one 64x64 tile per CTA (neogemmV02.cu:190-191). */
int neogemm_debug_plan(int64_t M, int64_t N, int64_t K, int64_t ldc, int c_col_major, int sm_count,
                       int* plan_out, int* segments, int max_segments);

/* Self-test of the bounded device-side waits.  Launches one warp that waits, for at most
 * `limit_us` microseconds (1..100000), on a barrier nothing will ever complete.  The warp must
 * give up when the limit expires, record the error exactly as the GEMM's roles do (code 4, CTA 0,
 * segment -1) and exit normally: afterwards neogemm_device_status() shows that record, every
 * neogemm_bf16_nt* call returns NEOGEMM_ERR_DEVICE_TIMEOUT, and neogemm_clear_device_status()
 * makes the library usable again - the CUDA context is unaffected throughout.  `waited_ns_out`
 * (nullable) receives the time the warp actually waited.  Synchronous.  The reference has no
 * error path to test (nemgemmV03.cu:387-390 prints cudaGetLastError). */
int neogemm_debug_wait_expiry(unsigned int limit_us, unsigned long long* waited_ns_out);

/* The same self-test aimed at the error record of neogemm_bf16_nt_noalloc(): afterwards
 * neogemm_noalloc_status() shows code 4 and that entry point returns NEOGEMM_ERR_DEVICE_TIMEOUT
 * until neogemm_noalloc_clear_status().  Allocates nothing.  Synchronous. */
int neogemm_debug_wait_expiry_noalloc(unsigned int limit_us);

/* Library version, e.g. 100 = 1.0.0. */
int neogemm_version(void);

#ifdef __cplusplus
}
#endif

#endif /* NEOGEMM_H_ */
