/*
 * lce_b200 -- C ABI of the B200 (sm_100a) fused linear + cross-entropy library.
 *
 * This is the operator boundary of the hot path
 *     loss = cross_entropy(logit_scale * (x @ W), y) + z_regularization * mean(logsumexp^2)
 * computed N_chunk rows at a time, with both gradients produced during the forward pass.
 * It replaces the two Triton launches and the host-side torch reductions that the reference
 * performs once per row chunk (linear_cross_entropy/ops.py:721-791 in the reference project).
 *
 * Conventions
 *   - Plain C: pointers, sizes, PODs. No C++/torch types cross this boundary.
 *   - Every pointer named dev_* / x / weight / labels / workspace ... is a DEVICE pointer.
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued on it, nothing synchronises
 *     (except lce_read_status, which is a debugging call).
 *   - The library never allocates device memory: the caller passes one workspace blob sized by
 *     lce_workspace_bytes().
 *   - Every entry point returns an int status: LCE_OK or a negative LCE_ERR_* code;
 *     lce_status_string() maps it to text.  No exception crosses the ABI.
 *   - W is stored (hidden, vocab) with the vocab index contiguous, like the reference's
 *     transposed nn.Linear weight (ops.py:913).
 *
 * Shapes: any number of rows and any vocabulary size; hidden % 8 == 0; chunk_rows % 128 == 0. The rows of x, W and
 * dW must start on 16-byte boundaries (LCE_ERR_MISALIGNED otherwise): for a vocabulary size that is not a multiple
 * of 8 give W and dW a row stride rounded up to 8 elements. The kernels work on 128 x 256 tiles: what hangs over
 * the edges is zero-filled on load and masked on store. (The reference asserts N % 512, V % 4096, H % 256: ops.py:689-691.)
 */
#ifndef LCE_B200_H
#define LCE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LCE_OK 0
#define LCE_ERR_INVALID_ARGUMENT (-1)
#define LCE_ERR_UNSUPPORTED_SHAPE (-2)
#define LCE_ERR_MISALIGNED (-3)
#define LCE_ERR_UNSUPPORTED_DEVICE (-4)
#define LCE_ERR_CUDA (-5)
#define LCE_ERR_DEVICE_TIMEOUT (-6)
#define LCE_ERR_DRIVER (-7)
#define LCE_ERR_TOO_LARGE (-8)

/* element types of x / W (and of the exp slab the forward writes) */
#define LCE_DTYPE_F16 0
#define LCE_DTYPE_BF16 1
#define LCE_DTYPE_F32 2 /* multiplied as TF32, like tl.dot on fp32 inputs in the reference */

/* One problem description shared by all calls of one forward+backward pass. */
typedef struct lce_problem {
  int64_t n_rows_total;   /* N = B*S, all chunks                                  */
  int64_t chunk_rows;     /* rows per chunk: min(N, N_chunk_size) (ops.py:687) rounded up to a multiple of 128 */
  int64_t hidden;         /* H = in_features                                       */
  int64_t vocab_local;    /* columns of W held by this rank (V when not sharded)  */
  int64_t vocab_offset;   /* class id of local column 0 (0 when not sharded)      */
  int64_t ignore_index;   /* rows with this label do not count (ops.py:705)       */
  int32_t world;          /* number of vocab shards whose row statistics are combined */
  int32_t dtype;          /* LCE_DTYPE_* of x and W                                */
  int32_t monitoring;     /* 1: also produce logit max / entropy / norm            */
  int32_t want_grad;      /* 0: forward only (no slab is written)                  */
  float logit_scale;      /* z = logit_scale * (x @ W)  (ops.py:200)               */
  float z_regularization; /* weight of mean(lse^2)       (ops.py:756-761)          */
  int32_t slab_mode;      /* LCE_SLAB_* : how the exponentials kept between forward and backward are normalised */
  int32_t chunk_buffers;  /* 0 or 1: one set of per-chunk buffers (slab, statistics) in the workspace; 2: two sets,
                             used alternately by consecutive chunks, so that lce_forward_chunk of chunk c + 1 may
                             be enqueued before the combine / backward calls of chunk c (see lce_combine_chunk_peer) */
} lce_problem;

/* slab_mode. The forward keeps exp(z - b) of the chunk in the element type of the inputs (the "slab").
 * LCE_SLAB_DEFAULT: bf16 / fp32 use ONE base b per row, found from a two-tile probe, which makes the backward a
 *   plain contraction with a per-row factor; a row group whose logits fall outside the window around its base
 *   (row max - base outside about [-60, +72]) is recomputed. fp16 uses LCE_SLAB_PER_TILE (its exponent range
 *   is too narrow for one base per row).
 * LCE_SLAB_PER_TILE: b = the maximum of each (row, 256-column tile); lce_dz_chunk then rewrites the slab in
 *   place once. Never recomputes; the better choice for bf16 / fp32 when the logits of a row spread over more
 *   than about 100 units, where the default mode would recompute most chunks. All calls of a pass must use the
 *   same mode. */
#define LCE_SLAB_DEFAULT 0
#define LCE_SLAB_PER_TILE 1

/* Number of per-row partial statistics a rank exports per chunk (base b of the sums, sum exp(z - b),
 * target logit, sum exp(z - b) z, sum z^2, max z); lce_forward_chunk writes LCE_ROW_PARTS * chunk_rows floats. */
#define LCE_ROW_PARTS 6

/* ---- housekeeping ------------------------------------------------------------------------- */
int lce_version(void);
const char* lce_status_string(int status);
/* Kernels launched by this library in this process so far (all threads). */
long long lce_launch_count(void);

/* Bytes of workspace one pass needs for `p` (slab + statistics + split-K partials + scalars).
 * Replaces the per-call torch allocations of ops.py:697-703. */
int lce_workspace_bytes(const lce_problem* p, size_t* bytes);

/* ---- the pass, in call order ------------------------------------------------------------------
 * lce_begin            once:      counts valid labels (ops.py:705), clears the loss accumulators
 * per chunk:
 *   lce_forward_chunk             logit GEMM + softmax statistics + exp slab (ops.py:722-752)
 *   [sharded: all-gather the row partials of all ranks]
 *   lce_combine_chunk             log-sum-exp per row, loss / metric sums (ops.py:753-761)
 *   lce_backward_chunk            dZ, dx rows of the chunk, dW accumulation (ops.py:763-791)
 *                                 (= lce_dz_chunk + lce_dx_chunk + lce_dw_chunk)
 *   [sharded: all-reduce the chunk's dx rows]
 * lce_finalize         once:      5 scalars (ops.py:793-802)
 */
int lce_begin(const lce_problem* p, const int64_t* labels, void* workspace, void* stream);

/* x: [n_rows_total, hidden] with row stride x_ld elements; weight: [hidden, vocab_local] with row
 * stride w_ld elements; labels: [n_rows_total]. Processes rows [row0, row0 + rows), which must lie
 * inside one chunk (chunks start at multiples of chunk_rows); row0 % 128 == 0, and rows % 128 == 0 unless
 * the call ends with the last row of the problem.
 * row_parts_local: float[LCE_ROW_PARTS * chunk_rows] output (this rank's per-row partials). */
int lce_forward_chunk(const lce_problem* p, const void* x, int64_t x_ld, const void* weight, int64_t w_ld,
                      const int64_t* labels, int64_t row0, int64_t rows, void* workspace,
                      float* row_parts_local, void* stream);

/* row_parts_all: float[world * LCE_ROW_PARTS * chunk_rows], rank-major (for world == 1 this is
 * row_parts_local). */
int lce_combine_chunk(const lce_problem* p, const float* row_parts_all, const int64_t* labels, int64_t row0,
                      int64_t rows, void* workspace, void* stream);

/* The backward half of a chunk, in three steps that may also be called one by one (each on rows
 * [row0, row0 + rows) of one chunk; a call may cover a 128-aligned part of a chunk, which is how the
 * host overlaps the slab transform of one half chunk with the tensor-core work of the other):
 *
 * lce_dz_chunk   prepares dZ = softmax*(1 + 2 z_reg lse) - onehot (ops.py:309-314) from the slab the forward
 *                wrote. fp16: the slab holds exp(z - tile max) and is rewritten in place (one pass over it).
 *                bf16 / fp32: the slab holds exp(z - b_i) with one base b_i per row, so dZ is the slab times a
 *                per-row factor c_i = exp(b_i - lse_i)(1 + 2 z_reg lse_i) minus the one-hot; only the label
 *                entry of each row is touched (slab[i, y_i] -= 1/c_i), c_i goes into the epilogue of dx and
 *                into a scaled copy c_i * x_i of the chunk's x rows that dW is computed from.
 *                Needs lce_combine_chunk of the same rows.
 * lce_dx_chunk   dx rows = dZ W^T * logit_scale / n_valid (ops.py:317,332). dx: [n_rows_total, hidden]
 *                with row stride dx_ld and element type dx_dtype (LCE_DTYPE_*).
 * lce_dw_chunk   dW (+)= x^T dZ * logit_scale / n_valid (ops.py:424,443), summed over the chunks of the pass in
 *                more precision than the result has. dweight: [hidden, vocab_local] in the element type of
 *                x / W (row stride dw_ld elements), overwritten by the call with first != 0 and complete after
 *                the call with last != 0. For the 16-bit types the running sum is carried as the PAIR
 *                dweight + dweight_residual, both in the element type: each call rounds the new sum to dweight and
 *                the rounding error to dweight_residual (about 16 significant bits together; the reference
 *                accumulates fp16 gradients in fp16 and bf16 gradients in an fp32 buffer the size of W, ops.py:
 *                440-444, 693). dweight_residual: scratch of the same shape and row stride (dwr_ld == dw_ld), only
 *                meaningful between the calls of one pass; may be null for a pass of a single call (first and
 *                last) and for fp32, where dweight is its own accumulator. No buffer of hidden x vocab fp32
 *                values and no conversion pass exist.
 * lce_backward_chunk = the three in sequence. */
int lce_dz_chunk(const lce_problem* p, const void* x, int64_t x_ld, const int64_t* labels, int64_t row0,
                 int64_t rows, void* workspace, void* stream);
int lce_dx_chunk(const lce_problem* p, const void* weight, int64_t w_ld, int64_t row0, int64_t rows, void* workspace,
                 void* dx, int64_t dx_ld, int32_t dx_dtype, void* stream);
int lce_dw_chunk(const lce_problem* p, const void* x, int64_t x_ld, int64_t row0, int64_t rows, void* workspace,
                 void* dweight, int64_t dw_ld, void* dweight_residual, int64_t dwr_ld, int32_t first, int32_t last,
                 void* stream);
int lce_backward_chunk(const lce_problem* p, const void* x, int64_t x_ld, const void* weight, int64_t w_ld,
                       const int64_t* labels, int64_t row0, int64_t rows, void* workspace, void* dx,
                       int64_t dx_ld, int32_t dx_dtype, void* dweight, int64_t dw_ld, void* dweight_residual,
                       int64_t dwr_ld, int32_t first, int32_t last, void* stream);

/* ---- dx exchange between the ranks of a vocabulary-sharded run, over peer-mapped memory -------------------
 * No counterpart in the reference (it has no multi-GPU path). These three calls replace lce_dx_chunk plus the
 * all-reduce of the chunk's dx rows that a sharded caller would otherwise issue: the dx contraction itself
 * stores its fp32 output tiles into the memory of the rank that owns the rows (rank o owns chunk rows
 * [o * chunk_rows / world, (o + 1) * chunk_rows / world)), the owner sums all ranks' tiles in a fixed order,
 * rounds once and stores the finished rows into every rank's staging area, from where they are copied into dx.
 * Only stores and 32-bit flags cross the links. dx comes out bitwise identical on all ranks.
 *
 * lce_peer_table: world / rank of the caller and, for every rank, the address AS SEEN FROM THE CALLING GPU of
 * that rank's exchange buffer (base[rank] is the caller's own). Each buffer holds lce_peer_bytes() bytes, is
 * 256-byte aligned, must be zero before its first use and is owned by the caller (the library allocates
 * nothing); all ranks must use the same problem, dx_dtype and sequence of epochs.
 * epoch: a counter the caller increases by one for every lce_dx_chunk_peer call on this set of buffers
 * (starting at 1, same value on all ranks); it selects one of two buffer halves and is the value the flags
 * are compared against.
 * Requires chunk_rows % (128 * world) == 0 (LCE_ERR_UNSUPPORTED_SHAPE otherwise) and world <= LCE_MAX_PEERS.
 * Waits on other ranks are bounded by wait_ms (<= 0: 10 s); when one runs out the device status word is set,
 * nothing is copied and the loss of the pass becomes NaN.
 *
 * lce_dx_chunk_peer   contraction + scatter into the owners' buffers, then flag A. Stream-ordered after
 *                     lce_dz_chunk like lce_dx_chunk.
 * lce_dx_reduce_peer  waits for flag A of all ranks; sums and broadcasts the rows this rank owns; flag B.
 * lce_dx_finish_peer  waits for flag B of all ranks; copies the chunk's rows from the staging area into dx.
 * The last two may run on another stream than the first (ordered after it by an event); at most two epochs
 * may be in flight: lce_dx_chunk_peer(epoch e) must be ordered after lce_dx_finish_peer(epoch e - 2). */
#define LCE_MAX_PEERS 8
typedef struct lce_peer_table {
  int32_t world;
  int32_t rank;
  void* base[LCE_MAX_PEERS];
} lce_peer_table;
int lce_peer_bytes(const lce_problem* p, int32_t dx_dtype, size_t* bytes);
int lce_dx_chunk_peer(const lce_problem* p, const void* weight, int64_t w_ld, int64_t row0, int64_t rows,
                      void* workspace, const lce_peer_table* peers, int32_t dx_dtype, uint32_t epoch, void* stream);
int lce_dx_reduce_peer(const lce_problem* p, int64_t row0, int64_t rows, void* workspace, const lce_peer_table* peers,
                       int32_t dx_dtype, uint32_t epoch, int32_t wait_ms, void* stream);
int lce_dx_finish_peer(const lce_problem* p, int64_t row0, int64_t rows, void* workspace, const lce_peer_table* peers,
                       uint32_t epoch, void* dx, int64_t dx_ld, int32_t dx_dtype, int32_t wait_ms, void* stream);

/* The whole pass of an UNSHARDED problem (world == 1) in one call: lce_begin, then per chunk lce_forward_chunk,
 * lce_combine_chunk and -- with want_grad -- lce_dz_chunk, lce_dx_chunk (dx != NULL) and lce_dw_chunk
 * (dweight != NULL), then lce_finalize; everything on `stream`, nothing synchronises. This is the reference's whole
 * LinearXentImplementation.forward (ops.py:665-802) behind one entry point, and what makes small problems cheap:
 * their cost is the host time per call, not the kernels. row_parts: LCE_ROW_PARTS * chunk_rows floats of scratch.
 * dx / dweight: either may be NULL when that gradient is not wanted (not both, with want_grad); dweight_residual as
 * for lce_dw_chunk (needed for 16-bit types when the pass has more than one chunk). */
int lce_fused_pass(const lce_problem* p, const void* x, int64_t x_ld, const void* weight, int64_t w_ld,
                   const int64_t* labels, void* workspace, float* row_parts, void* dx, int64_t dx_ld, int32_t dx_dtype,
                   void* dweight, int64_t dw_ld, void* dweight_residual, int64_t dwr_ld, float* out5, void* stream);

/* ---- row statistics exchange between the ranks of a vocabulary-sharded run, over peer-mapped memory -------
 * No counterpart in the reference (it has no multi-GPU path). These calls replace the all-gather of the per-row
 * partials that a sharded caller would otherwise issue between lce_forward_chunk and lce_combine_chunk: each rank
 * STORES its LCE_ROW_PARTS x rows partials into every rank's exchange buffer and publishes a 32-bit flag; the
 * combine step waits (bounded) for the flags of all ranks and merges the partials in rank order, so every rank
 * computes bitwise the same log-sum-exp. Only stores and flags cross the links.
 *
 * Used with chunk_buffers == 2 this takes the exchange off the critical path: the caller enqueues
 *     forward(c + 1), push(c + 1), combine_peer(c), backward(c)
 * so the partials of a chunk have been travelling for a whole backward step before anyone waits for them.
 *
 * Buffers: one per rank, lce_parts_bytes() bytes, 256-byte aligned, zero before first use, owned by the caller,
 * addressed through an lce_peer_table (as for the dx exchange; a separate buffer). It holds four slots, selected by
 * epoch % 4. epoch: a counter the caller increases by one per lce_parts_push on this set of buffers (from 1, same
 * sequence on all ranks). A push for epoch e must be ordered (stream order on each rank is enough) after that rank's
 * lce_combine_chunk_peer of epoch e - 2 or later; the four slots then make it impossible to overwrite partials
 * that some rank has not merged yet.
 *
 * lce_parts_push          row_parts_local as written by lce_forward_chunk for rows [row0, row0 + rows).
 * lce_combine_chunk_peer  lce_combine_chunk reading all ranks' partials of `epoch` from this rank's buffer. When the
 *                         wait for a flag runs out (wait_ms, <= 0: 10 s) the status word is set and the loss
 *                         of the pass becomes NaN. */
int lce_parts_bytes(const lce_problem* p, size_t* bytes);
int lce_parts_push(const lce_problem* p, const float* row_parts_local, int64_t row0, int64_t rows,
                   const lce_peer_table* peers, uint32_t epoch, void* stream);
int lce_combine_chunk_peer(const lce_problem* p, const lce_peer_table* peers, uint32_t epoch, const int64_t* labels,
                           int64_t row0, int64_t rows, void* workspace, int32_t wait_ms, void* stream);

/* out5: float[5] = loss, z_value, logit_max, logit_entropy, logit_norm (the reference's return
 * tuple, ops.py:802). The last three are only meaningful with monitoring. If any kernel of the pass
 * reported a device-side error the loss is NaN. */
int lce_finalize(const lce_problem* p, void* workspace, float* out5, void* stream);

/* How often the default slab mode had to recompute in the pass that used `workspace`: copies two int32
 * {256-row groups recomputed, 256-row groups processed} to host_out2, asynchronously on `stream` when host_out2 is
 * pinned memory (valid once the stream has passed this point; nothing synchronises). A caller that sees a large
 * fraction should run its next passes of that shape with LCE_SLAB_PER_TILE. No counterpart in the reference. */
int lce_rerun_stats_async(void* workspace, int32_t* host_out2, void* stream);

/* dst[r, c] = src[r, c] * (*dev_factor), converting element type (the reference's
 * x_grad.mul_(grad_output), ops.py:810). cols % 8 == 0. src == dst is allowed when the types match, and
 * then a factor of exactly 1 (the plain loss.backward() case) leaves the data untouched. */
int lce_grad_scale_cast(const void* src, int32_t src_dtype, int64_t src_ld, void* dst, int32_t dst_dtype,
                        int64_t dst_ld, int64_t rows, int64_t cols, const float* dev_factor, void* stream);

/* Synchronises `stream` and returns the pass's device status word translated to an LCE_* code
 * (LCE_ERR_DEVICE_TIMEOUT if a bounded in-kernel wait ran out). Debugging / tests. */
int lce_read_status(void* workspace, void* stream);

/* ---- evaluation without a workspace ---------------------------------------------------------------
 * lce_eval_loss_static computes the five output scalars of a forward-only pass (out5 as in lce_finalize)
 * for callers that cannot hand the library a workspace because they cannot allocate device memory at the
 * point of the call: a latency-critical loop that must not pay cudaMalloc's implicit device
 * synchronisation, an inference-server plugin that is only given its input and output buffers, an
 * evaluation hook running after the framework's memory pool has claimed all device memory. Its scratch (per-tile softmax statistics, per-row partials, accumulators)
 * is a fixed LCE_STATIC_SCRATCH_BYTES array inside the library's device image: every GPU that loads the
 * library holds it until the process exits, and the entry point calls no cudaMalloc, cudaFree or other
 * allocating routine. The caller still passes x, weight, labels and out5 (device pointers).
 *   - p: n_rows_total, hidden, vocab_local, dtype, ignore_index, logit_scale, z_regularization and
 *     monitoring are used; chunk_rows, world, vocab_offset and want_grad are ignored (forward only,
 *     unsharded; rows are processed in the largest chunks whose statistics fit the scratch).
 *   - LCE_ERR_TOO_LARGE if not even 128 rows fit (vocab_local beyond about 2 million columns without monitoring, 1 million with); the other
 *     shape rules are those of lce_forward_chunk.
 *   - The first call on each device resolves the scratch array's device address (cudaGetSymbolAddress) and
 *     sets kernel attributes; make that first call outside of any stream capture.
 *   - All calls share the one array, which keeps the previous call's contents: every accumulator is cleared
 *     at the start of a call, everything else is rewritten before it is read. Two calls that overlap on the
 *     GPU (different streams, or different host threads on one device) race on it; serialise them.
 * It has no counterpart in the reference. */
#define LCE_STATIC_SCRATCH_BYTES (8u << 20)
int lce_eval_loss_static(const lce_problem* p, const void* x, int64_t x_ld, const void* weight, int64_t w_ld,
                         const int64_t* labels, float* out5, void* stream);

/* ---- measurement ------------------------------------------------------------------------------
 * With profiling enabled, a CUDA event pair is recorded on the launching stream around each of the
 * three tensor-core contractions (0: logits z = x W, 1: dx = dZ W^T, 2: dW = x^T dZ).
 * lce_profile_read waits for the recorded events, returns per contraction the summed device time in
 * milliseconds and the number of launches since the previous read, and resets both.
 * Plays the part of the reference benchmark's do_bench timing (bench_fusions.py:280-281), per kernel. */
int lce_profile_enable(int32_t enable);
int lce_profile_read(double* ms3, long long* launches3);

/* ---- diagnostics ------------------------------------------------------------------------------
 * Not part of the pass: stateless, changes nothing the other entry points see.
 *
 * Runs the GEMM engine alone: out[s][M, N] = A * B^T over K-split s (fp32, row stride N).
 * a_mn_major == 0: a is [M, K] (K contiguous, row stride a_ld); != 0: a is [K, M] (row stride a_ld).
 * Same for b with N. M % 128 == 0, N % 256 == 0, K % (splits * 128 bytes) == 0.
 * single_cta != 0: use the single-CTA kernel (128 x 256 tiles) even where the pass would use CTA pairs
 * (cta_group::2, 256 x 256 tiles; the pass falls back to the single-CTA kernel for an odd number of 128-row tiles).
 * raster_group, n_fastest: the order in which the persistent CTAs walk the tile grid. n_fastest != 0: along N first
 * (the dx contraction), else along M first (logits, dW). raster_group 0: as in the pass (bands of at most 4096
 * rows when the fast dimension is longer, unless the environment variable LCE_RASTER_GROUP says otherwise),
 * -1: no bands, -2: chosen from the shape whatever the environment says, G > 0: bands of G tiles. The result does
 * not depend on either.
 * dev_status: int[8] device words, 8-byte aligned: [0] status (0 = ok); [2..3] int64 SM cycles and [4..5] int64
 * nanoseconds that CTA 0 spent in the kernel (their ratio is the SM clock the kernel ran at).
 * No counterpart in the reference. */
int lce_debug_gemm(int32_t dtype, int32_t a_mn_major, int32_t b_mn_major, const void* a, int64_t a_ld,
                   const void* b, int64_t b_ld, float* out, int64_t m, int64_t n, int64_t k, int32_t splits,
                   int32_t single_cta, int32_t raster_group, int32_t n_fastest, int* dev_status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LCE_B200_H */
