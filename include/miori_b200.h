/*
 * miori_b200 -- C ABI of the B200 (sm_100a) backend for Miori's quantized-matmul path.
 *
 * This is the boundary a host program binds (C++, cgo, ctypes, ...).  Every entry
 * returns 0 on success and a negative MIORI_E_* code on failure; the message for the
 * calling thread's last failure is miori_last_error().  Nothing here allocates behind
 * the caller's back except the buffer functions, and every launch entry only ENQUEUES
 * work on the given CUDA stream (void* stream is a cudaStream_t; NULL is the legacy
 * default stream), exactly as the reference's operators only encode dispatches
 * (reference src/ops.cpp: every op ends in dispatchThreadgroups and returns void).
 *
 * Data formats (reference shaders/ops.metal:5-6,45 and src/cpu_ref.h:25-45):
 *   q4  [N][K/8] uint32, eight 4-bit codes per word, low nibble first
 *   q8  [N][K/4] uint32, four 8-bit codes per word, low byte first
 *   s,b [N][K/group] bf16 scale and bias, weight = float(code)*scale + bias
 *   x   [M][K] bf16 activations, y [M][N] fp32 (or bf16 with MIORI_OUT_BF16)
 * group is 32 (what the reference hard-codes, config/m6.h:48) or 64.
 *
 * All pointers passed to launch entries are DEVICE pointers (or pointers the device
 * can dereference, e.g. managed memory from miori_buffer_alloc(shared=1)).
 */
#ifndef MIORI_B200_H_
#define MIORI_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MIORI_OK 0
#define MIORI_E_INVALID (-1)  /* bad argument: null pointer, unsupported shape, alignment */
#define MIORI_E_CUDA (-2)     /* a CUDA runtime or driver call failed */
#define MIORI_E_NOMEM (-3)    /* allocation failed */
#define MIORI_E_STATE (-4)    /* call made in the wrong state */
#define MIORI_E_DEVICE (-5)   /* a kernel reported an internal error (bounded wait expired) */

/* launch flags */
#define MIORI_OUT_F32 0u       /* y / C written as fp32 (what the reference's kernels write) */
#define MIORI_OUT_BF16 1u      /* y / C rounded to bf16 (RNE) in the epilogue */
#define MIORI_LAUNCH_PDL 2u    /* programmatic dependent launch: the kernel may start while its
                                  predecessor on the stream drains; it prefetches weights (which
                                  must be immutable while in flight) and waits for the
                                  predecessor before touching x / A or writing y / C */
#define MIORI_GEMV_EXACT 4u    /* force the fp32-dequant GEMV path for every M (default: M<=4) */
const char* miori_last_error(void);
/* Library version string, e.g. "miori_b200 0.1 sm_100a". */
const char* miori_version(void);

/* ---- device runtime: replaces reference src/metal.h:10-22 / src/metal.cpp ---------- */

typedef struct miori_device miori_device; /* one GPU + one in-order queue (a CUDA stream) */
typedef struct miori_buffer miori_buffer;

/* Metal::init (src/metal.cpp:10-24): open GPU `ordinal`, create its queue. */
int miori_device_open(int ordinal, miori_device** out);
int miori_device_close(miori_device* dev);
/* The queue's cudaStream_t, for passing to the launch entries. */
void* miori_device_stream(miori_device* dev);
int miori_device_ordinal(miori_device* dev);

/* Metal::new_buffer (src/metal.cpp:42-48).  shared!=0: host-visible storage the host can
 * read and write through miori_buffer_contents() with no explicit copy (CUDA managed
 * memory, the counterpart of MTLResourceStorageModeShared); shared==0: device-only. */
int miori_buffer_alloc(miori_device* dev, size_t bytes, int shared, miori_buffer** out);
int miori_buffer_free(miori_buffer* buf);
void* miori_buffer_contents(miori_buffer* buf);   /* MTL::Buffer::contents(); NULL if device-only */
void* miori_buffer_device_ptr(miori_buffer* buf); /* pointer for launch entries */
size_t miori_buffer_length(miori_buffer* buf);    /* MTL::Buffer::length() */
/* Hint that the buffer will next be used by the GPU (1) or the host (0); optional. */
int miori_buffer_prefetch(miori_buffer* buf, int to_device);

/* Metal::begin / Metal::submit (src/metal.cpp:50-59).  begin opens a command scope on
 * the queue; submit closes it and, when wait!=0, blocks until the queue drains and
 * reports any asynchronous error. */
int miori_begin(miori_device* dev);
int miori_submit(miori_device* dev, int wait);

/* Pinned host staging for callers that keep their own host buffers. */
int miori_host_alloc(size_t bytes, void** out);
int miori_host_free(void* p);
/* Asynchronous copies on `stream` (host memory should be pinned). */
int miori_memcpy_h2d(void* dst_dev, const void* src_host, size_t bytes, void* stream);
int miori_memcpy_d2h(void* dst_host, const void* src_dev, size_t bytes, void* stream);
int miori_stream_sync(void* stream);

/* ---- GEMV: replaces shaders/ops.metal:6-42 (gemv4), :46-82 (gemv8),
 *      shaders/batch.metal:145-188 (gemv4_b), :192-236 (gemv8_b) and the tuning variants
 *      ops.metal:563-602 (gemv4x4), :711-751 (gemv4x2).  Bound by src/ops.cpp:7-37,
 *      347-360, 376-390, 424-454, 524-574. ----------------------------------------- */

/* y[m][n] = sum_k (code[n][k]*s[n][k/group] + b[n][k/group]) * x[m][k], 1 <= M <= 32.
 * The result of a row m does not depend on M (reference shaders/batch.metal:142-144)
 * within the same numeric path: M <= 4 dequantizes in fp32 (as gemv4 / gemv4_b do; at
 * group 64 the 4-bit kernel sums a group's two halves in a different order for M = 3, 4
 * than for M <= 2, so those agree to fp32 rounding rather than bit for bit, while group
 * 32 is bit-identical for all M <= 4); M > 4 multiplies bf16-rounded weights on the
 * tensor cores (as the reference does for wide batches through its bf16 cache,
 * src/batch.cpp:223-230) unless MIORI_GEMV_EXACT is set.  Requires K % group == 0, group in {32,64}; q,s,b,x 16-byte
 * aligned.  Only M rows of x are read and M rows of y written (the reference's
 * gemv4_b always touches four, shaders/batch.metal:178-179). */
int miori_gemv4(const void* q, const void* s, const void* b, const void* x, void* y,
                uint32_t N, uint32_t K, uint32_t M, uint32_t group, uint32_t flags,
                void* stream);
int miori_gemv8(const void* q, const void* s, const void* b, const void* x, void* y,
                uint32_t N, uint32_t K, uint32_t M, uint32_t group, uint32_t flags,
                void* stream);

/* ---- bf16 weight cache: replaces shaders/ops.metal:142-166 (dequant4), :754-779
 *      (dequant8), shaders/gemm_mpp.metal:9-34 (dequant_tile).  Bound by
 *      src/ops.cpp:74-87, 310-322, 624-637. ------------------------------------------ */

/* out[n][k] = bf16(float(code)*scale + bias), row-major [N][K], bit-exact with
 * src/cpu_ref.h:16-23,25-45. */
int miori_dequant4_rowmajor(const void* q, const void* s, const void* b, void* out,
                            uint32_t N, uint32_t K, uint32_t group, void* stream);
int miori_dequant8_rowmajor(const void* q, const void* s, const void* b, void* out,
                            uint32_t N, uint32_t K, uint32_t group, void* stream);
/* The cache consumed by miori_gemm_bf16_cache.  Its layout is private to this library
 * (as [N/64][K][64] is private to the reference's dequant_tile / gemm_mpp pair);
 * miori_cache_bytes gives its size and miori_cache_to_rowmajor undoes the layout.  One promise
 * is public: weight rows are stored one after the other, so bytes [miori_cache_bytes(r0, K),
 * miori_cache_bytes(r0 + n, K)) of a cache are the cache of its rows r0 .. r0 + n - 1, and a
 * row shard of a projection needs no copy. */
size_t miori_cache_bytes(uint32_t N, uint32_t K);
int miori_dequant4_cache(const void* q, const void* s, const void* b, void* cache,
                         uint32_t N, uint32_t K, uint32_t group, void* stream);
int miori_cache_to_rowmajor(const void* cache, void* out, uint32_t N, uint32_t K,
                            void* stream);

/* ---- prefill GEMM: replaces shaders/gemm_mpp.metal:36-54 (gemm_mpp) and :57-73
 *      (gemm_mpp32).  Bound by src/ops.cpp:324-345, 639-651. -------------------------- */

/* C[M][N] = A[M][K] (bf16, contiguous) x cache(N,K)^T, fp32 accumulation on the
 * tcgen05 tensor cores; C contiguous fp32 (or bf16 with MIORI_OUT_BF16).  One entry
 * serves both reference tile shapes: a row of C does not depend on M
 * (reference src/main.cpp:1403-1443).  Requires K % 64 == 0, N % 8 == 0, A and cache
 * 16-byte aligned. */
int miori_gemm_bf16_cache(const void* A, const void* cache, void* C, uint32_t M, uint32_t N,
                          uint32_t K, uint32_t flags, void* stream);

/* Host-only: what the planner would launch for this shape with `workspace_bytes` of workspace --
 * the tile's width in output columns (128 or 256; a tile is 128 rows, 256 when two CTAs share it),
 * the CTAs per tile (1, or 2 for the cta_group::2 kernel) and the number of K slices (1 = no
 * split).  For tests and for hosts that want to log the choice; no device is touched beyond the
 * SM count. */
int miori_gemm_plan(uint32_t M, uint32_t N, uint32_t K, size_t workspace_bytes, uint32_t* tile_n,
                    uint32_t* ctas_per_tile, uint32_t* splits);
/* Same product with a caller-provided scratch area that lets problems with few output tiles
 * (small M or N, long K) split K across SMs: partial tiles go to `workspace` (fp32) and a
 * second kernel sums them in a fixed order, so results stay reproducible and independent of
 * M.  miori_gemm_workspace_bytes gives the size worth passing (0: the shape does not
 * split); a smaller or NULL workspace only reduces or disables the splitting.  The workspace
 * contents are scratch; two launches in flight at once must not share it.  (The reference
 * has no counterpart: its GEMM is a library call, shaders/gemm_mpp.metal:47-53.) */
size_t miori_gemm_workspace_bytes(uint32_t M, uint32_t N, uint32_t K);
int miori_gemm_bf16_cache_ws(const void* A, const void* cache, void* C, uint32_t M, uint32_t N,
                             uint32_t K, uint32_t flags, void* workspace, size_t workspace_bytes,
                             void* stream);

/* The split-K GEMM for callers that cannot supply a workspace because they cannot allocate
 * device memory when they call: e.g. a decode loop that divided up the GPU's memory once at
 * start-up, or a plug-in in a process where another runtime owns the allocator.  (No
 * counterpart in the reference, whose GEMM is a closed library call.)  The K-split partials go
 * to a 16 MiB array built into the library (miori_gemm_static_scratch_bytes); every GPU that
 * loads the library holds that array until the process exits.  The call allocates nothing --
 * no cudaMalloc / cudaFree, no allocating library routine.  Shapes whose preferred split needs
 * more than the array are refused with MIORI_E_INVALID and a message that names the sizes
 * (miori_gemm_bf16_cache still runs them, unsplit and without scratch; compare
 * miori_gemm_workspace_bytes with miori_gemm_static_scratch_bytes to know beforehand);
 * shapes that do not split at all run without touching it.  The first call on a device looks
 * up the array's device address, so make that call before starting any stream capture.  All
 * calls share the one array: it keeps whatever the last call left (nothing needs clearing,
 * every partial is overwritten before it is read), and two calls whose kernels overlap on the
 * GPU -- different streams, or different host threads -- race on it; keep them in one stream. */
size_t miori_gemm_static_scratch_bytes(void);
int miori_gemm_bf16_cache_static(const void* A, const void* cache, void* C, uint32_t M, uint32_t N,
                                 uint32_t K, uint32_t flags, void* stream);

/* ---- strided bf16 GEMM: replaces gemm_naive (shaders/ops.metal:199-251, bound by
 *      src/ops.cpp:89-106), which carries the N=16 gate projection on every GEMM path
 *      (src/engine.cpp:516, src/batch.cpp:237,435) and the wide-batch LM head against the bf16
 *      embedding (src/batch.cpp:741). ------------------------------------------------------------ */

/* C[M][N] (fp32, or bf16 with MIORI_OUT_BF16; rows ldc elements apart) = A[M][K] (bf16, rows lda
 * apart) x B[N][K]^T (bf16, rows ldb apart), fp32 accumulation; any M, N, K >= 1.  Byte offsets
 * of the reference's signature are folded into the pointers.  Operands whose bases and row
 * pitches are 16-byte multiples (lda % 8 == 0, ldb % 8 == 0, ldc * element size % 16 == 0) run on
 * the tcgen05 kernels of miori_gemm_bf16_cache; anything else runs on a plain fp32-FMA kernel. */
int miori_gemm_bf16_strided(const void* A, uint32_t lda, const void* B, uint32_t ldb, void* C,
                            uint32_t ldc, uint32_t M, uint32_t N, uint32_t K, uint32_t flags,
                            void* stream);

/* ---- projection dispatch: replaces BatchEngine::linear / linear_p and Engine::p_gemm
 *      (reference src/batch.cpp:223-230, 429-431, src/engine.cpp:508-518), which route a
 *      projection to gemv4_b for narrow batches and to the bf16-cache GEMM otherwise. ------ */

/* y[M][N] = x[M][K] (bf16) x cache[N][K]^T for 1 <= M <= 32: the cache of miori_dequant4_cache
 * streamed once in 16-row tiles on mma.sync tensor cores, fp32 accumulation, fp32 or bf16 output,
 * no workspace.  What the reference's wide-batch path (gemm_mpp on the bf16 cache) computes for
 * the batch sizes of a decode step; a row's value depends neither on the grid nor on M within a
 * class of batch sizes (1..8, 9..16, 17..32 rows).  Every
 * warp keeps its share of the activations in registers (K <= 2048 for 17..32 rows, K <= 4096 for
 * 9..16 rows, K <= 8192 up to 8 rows) or, for longer rows up to K = 8192, streams it from L2 a few
 * k-slabs ahead of its use; beyond K = 8192 MIORI_E_INVALID: use miori_gemm_bf16_cache there. */
int miori_gemv_bf16_cache(const void* x, const void* cache, void* y, uint32_t M, uint32_t N, uint32_t K,
                          uint32_t flags, void* stream);

/* y[M][N] (fp32) = x[M][K] (bf16) x W^T.  Up to four rows stream the packed 4-bit weights with
 * fp32 dequantization (miori_gemv4), the reference's own cut-over.  Wider batches multiply the bf16
 * cache when `cache` is given -- with the narrow-batch kernel (miori_gemv_bf16_cache) while the
 * projection is short and for 9..16 rows, with the tensor-core GEMM (miori_gemm_bf16_cache_ws) for
 * long rows or wide outputs at more than 16 rows -- and otherwise stay on the packed weights (wide
 * outputs up to 8 rows, and everything when no cache is given, M <= 32).  miori_linear4_route tells which: 0 packed GEMV, 1 narrow-batch
 * cache kernel, 2 tensor-core GEMM (host-only; for logs and tests). */
int miori_linear4_route(uint32_t M, uint32_t N, uint32_t K, int has_cache);
int miori_linear4(const void* q, const void* s, const void* b, const void* cache, const void* x,
                  void* y, uint32_t N, uint32_t K, uint32_t M, uint32_t group, uint32_t flags,
                  void* workspace, size_t workspace_bytes, void* stream);

/* ---- multi-GPU: N-sharded GEMV with the all-gather of y fused into the kernel.  The reference
 *      runs on one GPU and has no counterpart; the partition follows its operand layout (rows of
 *      q, s, b are independent: shaders/ops.metal:6-42), so rank r multiplies rows
 *      [row0, row0 + n_local) and every rank ends up with the whole y. --------------------------- */

/* One per rank (one process per GPU).  Each rank allocates an arena of device memory that every
 * other rank maps through CUDA IPC; outputs live at the same offset in every arena.  create
 * allocates and zeroes the arena on the current device (nine times arena_bytes: the user area
 * plus two inboxes in which the peers' rows arrive as 8-byte packets); handle exports the 64-byte token
 * (miori_peers_handle_bytes) the host passes to the other ranks by any channel; connect takes the
 * tokens of all ranks in rank order (`world` x 64 bytes, this rank's own entry ignored). */
typedef struct miori_peers miori_peers;
int miori_peers_create(int rank, int world, size_t arena_bytes, miori_peers** out);
size_t miori_peers_handle_bytes(void);
int miori_peers_handle(miori_peers* g, void* handle_out);
int miori_peers_connect(miori_peers* g, const void* handles);
void* miori_peers_arena(miori_peers* g);        /* local arena (device pointer), offset 0 */
size_t miori_peers_arena_bytes(miori_peers* g);
/* MIORI_E_DEVICE if a kernel on this rank gave up waiting for a peer; the group is unusable
 * afterwards.  Every wait for a peer is bounded: about a second unless miori_peers_set_wait_us
 * gives another limit (1 us .. 10 s; call it with no kernel of the group in flight).  The limit
 * also bounds how far apart in time the ranks may ENQUEUE the same launch: a rank whose launch
 * comes later than that after its peers' (first-use module load, graph instantiation, a paused
 * host thread) makes them give up, so put a host barrier between set-up and the first launch. */
int miori_peers_status(miori_peers* g);
int miori_peers_set_wait_us(miori_peers* g, uint32_t microseconds);
/* Call only when no rank has kernels in flight that store into this rank's arena. */
int miori_peers_destroy(miori_peers* g);

/* miori_gemv4 / miori_gemv8 on this rank's n_local rows of an n_total-row weight matrix (q, s, b
 * point at the shard), delivering y[m][row0 + n] to y_offset of EVERY rank's arena: the epilogue
 * stores the rows locally and sends them to the peers over NVLink, and collects the peers' rows
 * before the kernel ends.  When the kernel completes on a rank, all ranks' rows are there.
 * Every rank must enqueue the same sequence of *_allgather / miori_allgather calls on its
 * group; x may be any device pointer, also one inside the arena.  y is fp32 [M][n_total] (bf16
 * with MIORI_OUT_BF16).  Requires (K / group) % 8 == 0; other shapes get MIORI_E_INVALID. */
int miori_gemv4_allgather(miori_peers* g, const void* q, const void* s, const void* b, const void* x,
                          size_t y_offset, uint32_t n_local, uint32_t row0, uint32_t n_total,
                          uint32_t K, uint32_t M, uint32_t group, uint32_t flags, void* stream);
int miori_gemv8_allgather(miori_peers* g, const void* q, const void* s, const void* b, const void* x,
                          size_t y_offset, uint32_t n_local, uint32_t row0, uint32_t n_total,
                          uint32_t K, uint32_t M, uint32_t group, uint32_t flags, void* stream);
/* All-gather for outputs of other kernels (e.g. the cache GEMM on an N-sharded cache): copies this
 * rank's block src[M][n_local] (contiguous rows, elements of elem_bytes = 2 or 4) into columns
 * [row0, row0 + n_local) of y[M][n_total] at y_offset of every rank's arena, its own included.
 * Same ordering guarantees as above. */
int miori_allgather(miori_peers* g, const void* src, size_t y_offset, uint32_t M, uint32_t n_local,
                    uint32_t row0, uint32_t n_total, uint32_t elem_bytes, uint32_t flags,
                    void* stream);

/* Greedy sampling over an N-sharded head without gathering the logits (the reference's host
 * loop over 128000 logits, src/engine.cpp:740-747, ties to the lowest index): every rank passes
 * the logits of its own rows (fp32, or bf16 with MIORI_OUT_BF16) and the index of its first row;
 * the ranks exchange (value, index) pairs, two 8-byte packets per rank.  Afterwards the arena of
 * every rank holds, at y_offset, `world` pairs [value fp32, index u32] and then the winning pair.
 * Same launch-order contract as the *_allgather entries. */
int miori_argmax_allreduce(miori_peers* g, const void* v, uint32_t n_local, uint32_t index0,
                           size_t y_offset, uint32_t flags, void* stream);
/* The head of a greedy decode step in one launch: this rank's rows of y = W x (one activation row)
 * go to y_offset of its own arena only, every thread keeps the best (value, index) of what it
 * stores, and the CTA that finishes last exchanges the rank's best with the peers, so that when
 * the kernel completes the winning token is on every rank and nothing but 16 bytes per peer has
 * crossed NVLink.  At best_offset (16-byte aligned, miori_gemv_argmax_bytes(world) bytes, zero
 * before the first use -- a fresh arena is) lie 16 bytes of scratch, then [rank][value, index]
 * and the winner [value, index] as 32-bit words: the winner sits 16 + 8 * world bytes in.  With
 * bf16 output the rounded logits are compared, so the result equals the arg-max of the gathered
 * bf16 vector; ties go to the lowest index, NaN never wins.  A world of one rank works too (no
 * exchange): the single-GPU form of "LM head, then pick".  Replaces the reference's gemv8 on the
 * head followed by the host loop of src/engine.cpp:740-747. */
size_t miori_gemv_argmax_bytes(int world);
int miori_gemv4_argmax(miori_peers* g, const void* q, const void* s, const void* b, const void* x,
                       size_t y_offset, size_t best_offset, uint32_t n_local, uint32_t row0,
                       uint32_t n_total, uint32_t K, uint32_t group, uint32_t flags, void* stream);
int miori_gemv8_argmax(miori_peers* g, const void* q, const void* s, const void* b, const void* x,
                       size_t y_offset, size_t best_offset, uint32_t n_local, uint32_t row0,
                       uint32_t n_total, uint32_t K, uint32_t group, uint32_t flags, void* stream);

/* ---- the steps either side of a projection (reference src/engine.cpp:389-413, 484-502) and the
 *      8-bit embedding gather that shares its table with the LM head. -------------------------- */

/* rmsnorm (shaders/ops.metal:86-115, src/ops.h:16-18): y[r][i] = bf16(x[r][i] * rsqrt(mean_i
 * x[r][i]^2 + eps) * gamma[i]); x fp32 [rows][n], gamma bf16 [n], y bf16 [rows][n]. */
int miori_rmsnorm(const void* x, const void* gamma, void* y, uint32_t rows, uint32_t n, float eps,
                  uint32_t flags, void* stream);
/* post_norm_add (shaders/ops.metal:605-631): out = x + src * rsqrt(mean src^2 + eps) * gamma, all
 * fp32 [rows][n] but gamma (bf16 [n]). */
int miori_post_norm_add(const void* x, const void* src, const void* gamma, void* out, uint32_t rows,
                        uint32_t n, float eps, uint32_t flags, void* stream);
/* silu_mul (shaders/ops.metal:129-139, src/ops.h:23-24): out[i] = bf16(gate[i] / (1 + exp(-gate[i]))
 * * up[i]); gate, up fp32, out bf16. */
int miori_silu_mul(const void* gate, const void* up, void* out, size_t n, uint32_t flags, void* stream);
/* embed8 (shaders/ops.metal:170-197, src/ops.h:35-37): out[t] = bf16 dequantization of row
 * tokens[t] of the 8-bit table q/s/b [rows][K]; bit-exact with src/cpu_ref.h:36-45.  An id
 * outside the table leaves its output row untouched. */
int miori_embed8(const void* q, const void* s, const void* b, const void* tokens, void* out, uint32_t T,
                 uint32_t rows, uint32_t K, uint32_t group, uint32_t flags, void* stream);
/* Index (u32) and, if out_value is not NULL, value (fp32) of the largest of n elements (fp32, or
 * bf16 with MIORI_OUT_BF16); ties go to the lowest index (src/engine.cpp:740-747). */
int miori_argmax(const void* v, uint32_t n, uint32_t flags, void* out_index, void* out_value, void* stream);
/* miori_gemv4 over the fused gate + up weights (w1 rows [0, N/2), then w3 rows [N/2, N)) with
 * silu_mul (shaders/ops.metal:129-139) as its epilogue: y bf16 [M][N/2], y[m][i] = bf16(silu(g) * u)
 * for g, u the fp32 results of rows i and N/2 + i, bit for bit what miori_gemv4 followed by
 * miori_silu_mul gives.  Saves the activation's launch and the fp32 round trip of 2 N values per
 * row (docs/MILESTONES.md:87, "SiLU x up epilogue").  N a multiple of 16, M <= 16 (wider batches
 * go through the bf16 cache, whose GEMM has no such epilogue); runs on the TMA + mma.sync kernel,
 * shapes it does not take get MIORI_E_INVALID. */
int miori_gemv4_silu(const void* q, const void* s, const void* b, const void* x, void* y, uint32_t N,
                     uint32_t K, uint32_t M, uint32_t group, uint32_t flags, void* stream);
/* The gate + up projection with both neighbours: y = bf16(silu(g) * u) of W * bf16(rmsnorm(x)), x fp32
 * [M][K], gamma bf16 [K], y bf16 [M][N/2]; M <= 4.  One launch for rmsnorm, w1, w3 and silu_mul. */
int miori_gemv4_rmsnorm_silu(const void* q, const void* s, const void* b, const void* x, const void* gamma,
                             float eps, void* y, uint32_t N, uint32_t K, uint32_t M, uint32_t group,
                             uint32_t flags, void* stream);
/* miori_gemv4 with post_norm_add (shaders/ops.metal:605-631) as its epilogue, for the o and w2
 * projections of a decode step: out = residual + v * rsqrt(mean(v^2) + eps) * gamma over each
 * output row v = W x; residual and out fp32 [M][N] (distinct), gamma bf16 [N], M <= 4.  Every CTA
 * stores its rows of v into out; the one that finishes last runs the stand-alone kernel's row pass
 * over out in place, so the result is bit for bit that of miori_gemv4 followed by
 * miori_post_norm_add.  `counter` is one 32-bit word of device memory that is zero before the first
 * launch; the kernel leaves it zero.  Launches that may run concurrently need counters of their
 * own.  Shapes the TMA + mma.sync kernel does not take get MIORI_E_INVALID. */
int miori_gemv4_post_norm_add(const void* q, const void* s, const void* b, const void* x,
                              const void* residual, const void* gamma, float eps, void* counter,
                              void* out, uint32_t N, uint32_t K, uint32_t M, uint32_t group,
                              uint32_t flags, void* stream);
/* miori_gemv4 / miori_gemv8 with the RMSNorm of the activations fused into their staging:
 * y = W * bf16(rmsnorm(x)), x fp32 [M][K], gamma bf16 [K].  Saves the norm's launch and the
 * round trip of its output (the fusion the reference planned, docs/MILESTONES.md:87).  4-bit
 * weights with up to four rows of K <= 2048 and fp32 out run on the TMA + mma.sync kernel (every CTA
 * sums the rows' squares for itself, then normalises while it stages), everything else on the tcgen05
 * kernel; shapes
 * neither takes get MIORI_E_INVALID.  The result is the unfused pair's up to the fp32 order of the sum
 * of squares. */
int miori_gemv4_rmsnorm(const void* q, const void* s, const void* b, const void* x, const void* gamma,
                        float eps, void* y, uint32_t N, uint32_t K, uint32_t M, uint32_t group,
                        uint32_t flags, void* stream);
int miori_gemv8_rmsnorm(const void* q, const void* s, const void* b, const void* x, const void* gamma,
                        float eps, void* y, uint32_t N, uint32_t K, uint32_t M, uint32_t group,
                        uint32_t flags, void* stream);

/* Non-zero if a kernel of this library recorded an internal error on the current
 * device since the last call (bounded wait expired); clears the record. */
int miori_device_error_poll(void);

#ifdef __cplusplus
}
#endif
#endif /* MIORI_B200_H_ */
