/*
 * blksprs_b200 — C ABI of the B200 (sm_100a) block-sparse matmul path.
 *
 * Every entry point is `extern "C"`, takes plain device pointers, sizes and a
 * CUDA stream handle (`void*`, a `cudaStream_t`), returns an `int` status
 * (0 = BSP_OK) and never throws.  Unless stated otherwise nothing here
 * allocates or frees device memory: the caller owns every buffer (inputs,
 * outputs and the small workspaces whose sizes the `*_bytes` helpers report).
 *
 * Data model (identical to the blksprs library this path replaces):
 *   compressed tensor   contiguous (n_blocks, bs, bs), fp16 / bf16 / fp32;
 *                       block p is the p-th non-zero of the layout in
 *                       row-major (batch, row, col) order.
 *   sparsity layout     contiguous (B, rows/bs, cols/bs) of 0/1 in any real
 *                       dtype (bool, integers, floats).
 *   LUT                 int64 (n, 3) rows (batch, row, col) of the non-zeros
 *                       (blksprs/utils/tools.py:33-35, build_layout_indices).
 *   reverse LUT         int64 (B*R*C,): rank of the block among the non-zeros
 *                       or -1 (blksprs/utils/tools.py:38-57,
 *                       build_packed_indices).
 */
#ifndef BLKSPRS_B200_H
#define BLKSPRS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------ */
enum {
    BSP_OK = 0,
    BSP_ERR_INVALID_ARG = 1,   /* null pointer, negative size, bad enum          */
    BSP_ERR_UNSUPPORTED = 2,   /* dtype / block size not handled by this build   */
    BSP_ERR_WORKSPACE = 3,     /* workspace smaller than the *_bytes helper says */
    BSP_ERR_CUDA = 4,          /* a CUDA runtime / driver call failed            */
    BSP_ERR_DEVICE_RANGE = 5,  /* status word: a LUT / pair index out of range   */
    BSP_ERR_DEVICE_TIMEOUT = 6,/* status word: a bounded device wait ran out     */
    BSP_ERR_TOO_LARGE = 7      /* input larger than a built-in scratch array     */
};

/* element type of a sparsity layout */
enum {
    BSP_L_BOOL = 0, /* torch.bool / uint8 */
    BSP_L_I8 = 1,
    BSP_L_I16 = 2,
    BSP_L_I32 = 3,
    BSP_L_I64 = 4,
    BSP_L_F16 = 5,
    BSP_L_BF16 = 6,
    BSP_L_F32 = 7,
    BSP_L_F64 = 8
};

/* element type of a compressed tensor */
enum { BSP_F16 = 0, BSP_BF16 = 1, BSP_F32 = 2 };

/* which block product a launch computes; A, B, O are compressed tensors */
enum {
    BSP_OP_NN = 0, /* O(r,c) = sum_t A(r,t)   * B(t,c)    forward  O  = X * Y    */
    BSP_OP_NT = 1, /* O(r,c) = sum_t A(r,t)   * B(c,t)^T  backward dX = dO * Y^T */
    BSP_OP_TN = 2  /* O(r,c) = sum_t A(t,r)^T * B(t,c)    backward dY = X^T * dO */
};

/* output-layout inference rule */
enum { BSP_LAYOUT_EXACT = 0, BSP_LAYOUT_FAST = 1, BSP_LAYOUT_OUTER = 2 };

/* Library version (major*10000 + minor*100 + patch). No reference counterpart. */
int bsp_version(void);

/* Text for a status code. No reference counterpart (the reference raises
 * Python exceptions only; the host shim maps codes to those exceptions). */
const char* bsp_status_string(int status);

/* Text of the last CUDA error seen by the calling thread ("" if none). */
const char* bsp_last_cuda_error(void);

/* ---- LUT construction -------------------------------------------------- */

/* Bytes of scratch the two LUT builders need for a layout of `numel` entries. */
size_t bsp_lut_workspace_bytes(int64_t numel);

/* Reverse LUT.  Replaces build_packed_indices, blksprs/utils/tools.py:38-57:
 *   flat = layout.reshape(-1).to(int64)
 *   packed[e] = (flat[e] == 1) ? cumsum(flat)[e] - 1 : -1
 * `total_out` (device, int64[1], may be null) receives cumsum(flat)[-1]
 * (0 for an empty layout). */
int bsp_build_packed_indices(const void* layout, int layout_dtype, int64_t numel,
                             int64_t* packed_out, int64_t* total_out,
                             void* workspace, size_t workspace_bytes, void* stream);

/* Reverse LUT for callers that may not allocate device memory.  No counterpart
 * in the reference (which allocates freely through torch); same result as
 * bsp_build_packed_indices, bit for bit.
 *
 * Who needs it: hosts that hand out all device memory once at start-up from
 * their own arena (an inference server that reserves the whole HBM for weights
 * and KV cache, an embedded pipeline with a fixed memory map) and therefore
 * have no allocator to ask for the scan's scratch buffer, and hosts for which
 * the implicit device-wide synchronisation of cudaMalloc / cudaFree in the
 * middle of a step is not acceptable.  Here the scratch is a fixed array inside
 * the library image: 16 KiB + 8 B on every GPU that loads the library, held
 * until the process exits.  The call itself, and everything it calls, performs
 * no cudaMalloc, cudaFree or other allocating routine; `layout`, `packed_out`
 * and `total_out` are still the caller's buffers.
 *
 * Limits and rules:
 *  - numel <= bsp_static_scratch_max_numel() (4 194 304 layout entries);
 *    larger layouts are refused with BSP_ERR_TOO_LARGE and nothing is launched.
 *  - The first call on each device looks up the array's device address (with
 *    that device current) and caches it; make that first call during set-up,
 *    before any stream capture begins.
 *  - All calls on a device share the one array, which keeps the previous call's
 *    contents (nothing in it needs clearing: each call overwrites what it later
 *    reads).  Two calls whose kernels can overlap on the GPU (different streams
 *    without an ordering between them) race on it; keep calls on one stream or
 *    order them with events. */
int bsp_build_packed_indices_static(const void* layout, int layout_dtype, int64_t numel,
                                    int64_t* packed_out, int64_t* total_out, void* stream);

/* Largest `numel` bsp_build_packed_indices_static accepts.  No reference counterpart. */
int64_t bsp_static_scratch_max_numel(void);

/* Number of non-zero layout entries, written to `count_out` (device int64[1]).
 * Replaces the count in matmul_build_layout_cache, blksprs/ops/matmul.py:270-273
 * (`torch.sum(layout.to(torch.int)).item()`), minus the host read, which the
 * caller does.  Leaves per-chunk partial counts in `workspace` for
 * bsp_build_layout_indices. */
int bsp_count_nonzero(const void* layout, int layout_dtype, int64_t numel,
                      int64_t* count_out, void* workspace, size_t workspace_bytes,
                      void* stream);

/* LUT.  Replaces build_layout_indices, blksprs/utils/tools.py:33-35
 * (`torch.nonzero(layout).contiguous()`): row p of `lut_out` (int64, (n,3)) is
 * the (batch,row,col) of the p-th non-zero in row-major order.  Must follow
 * bsp_count_nonzero on the same layout, stream and workspace; `capacity_rows`
 * is the number of rows `lut_out` can hold (rows beyond it are dropped). */
int bsp_build_layout_indices(const void* layout, int layout_dtype,
                             int64_t B, int64_t R, int64_t C,
                             int64_t* lut_out, int64_t capacity_rows,
                             void* workspace, size_t workspace_bytes, void* stream);

/* Output-layout inference.  Replaces build_sparsity_layout_matmul (exact),
 * _fast and _outer, blksprs/layouting/sparsity_layout.py:244-309.
 * lx is (B,R,K), ly is (B,K,C), out is uint8/bool (B,R,C).
 *   exact: out = any_k(lx[b,r,k] != 0 && ly[b,k,c] != 0)
 *   fast : out = any_k(lx[b,r,k]) && any_k(ly[b,k,c])
 *   outer: out = any_k(lx[b,r,k]) || any_k(ly[b,k,c])            */
int bsp_layout_matmul(const void* lx, int lx_dtype, const void* ly, int ly_dtype,
                      int64_t B, int64_t R, int64_t K, int64_t C, int mode,
                      uint8_t* out, void* stream);

/* ---- pair plan ---------------------------------------------------------
 * The reference kernel walks all K/T segments of every output block and
 * tests two reverse-LUT entries per step (blksprs/ops/matmul.py:191-226).
 * Here that walk is done once per layout triple: for every output block p
 * the plan stores the list of (a_block, b_block) index pairs it contracts.
 *
 * Indexing: for output block (b, r, c) and inner index t in [0, T)
 *   a = packed_a[b*a_sb + r*a_sr + t*a_st],  b = packed_b[b*b_sb + t*b_st + c*b_sc]
 * and the pair is kept iff both are >= 0.
 */

/* counts_out[p] (int32, n_out) = number of pairs of output block p. */
int bsp_plan_count(const int64_t* lut_out, int64_t n_out,
                   const int64_t* packed_a, int64_t a_sb, int64_t a_sr, int64_t a_st,
                   const int64_t* packed_b, int64_t b_sb, int64_t b_st, int64_t b_sc,
                   int64_t T, int32_t* counts_out, void* stream);

/* Bytes of scratch bsp_plan_offsets needs. */
size_t bsp_plan_workspace_bytes(int64_t n_out);

/* offsets_out (int32, n_out+1) = exclusive prefix sum of counts; the last
 * entry is the total pair count.  `total_out` (device int64[1], may be null)
 * receives the same total in 64 bits so the caller can reject plans whose
 * pair count does not fit int32. */
int bsp_plan_offsets(const int32_t* counts, int64_t n_out, int32_t* offsets_out,
                     int64_t* total_out, void* workspace, size_t workspace_bytes,
                     void* stream);

/* pairs_out (int32, (total,2)) filled in output-block order, t ascending:
 * pairs_out[2p] = a_block index, with bit 30 set on the last pair of its output
 * block; pairs_out[2p+1] = b_block index.  Block indices must be below 2^30. */
int bsp_plan_fill(const int64_t* lut_out, int64_t n_out,
                  const int64_t* packed_a, int64_t a_sb, int64_t a_sr, int64_t a_st,
                  const int64_t* packed_b, int64_t b_sb, int64_t b_st, int64_t b_sc,
                  int64_t T, const int32_t* offsets, int32_t* pairs_out, void* stream);

/* Splits n_out items (output blocks or panels, with CSR `offsets` of their pairs
 * or steps) into `n_chunks` contiguous ranges of nearly equal cost (cost of an
 * item = its count + `block_cost`); chunk_begin_out is int32 (n_chunks+1). */
int bsp_plan_schedule(const int32_t* offsets, int64_t n_out, int32_t block_cost,
                      int32_t n_chunks, int32_t* chunk_begin_out, void* stream);

/* ---- block-sparse matmul ---------------------------------------------- */

/* Block-sparse product on a pair plan with warp-level mma.sync instructions:
 * any block size >= 16, fp16 / bf16 / fp32 (TF32).  Replaces matmul_forward +
 * matmul_kernel, blksprs/ops/matmul.py:70-127,148-253 (op = BSP_OP_NN), and the
 * two products of matmul_wrapper_backward, blksprs/ops/matmul.py:130-145
 * (BSP_OP_NT, BSP_OP_TN), without materialising the transposes of
 * ops/transpose.py.
 *   a, b       compressed operands (n_a, bs, bs), (n_b, bs, bs) of `dtype`
 *   out        compressed result (n_out, bs, bs) of `dtype`; every block is
 *              written (zeros where a block has no pair); fp32 accumulation.
 *              a, b and out must be 16-byte aligned (BSP_ERR_INVALID_ARG)
 *   offsets    int32 (n_out+1), pairs int32 (total,2)
 *   status_word device int32[1] or null: receives BSP_ERR_DEVICE_* when a
 *              kernel meets an out-of-range index or a wait limit; never
 *              cleared by the kernel. */
int bsp_matmul_mma(const void* a, int64_t n_a, const void* b, int64_t n_b,
                   void* out, int64_t n_out,
                   const int32_t* offsets, const int32_t* pairs,
                   int bs, int dtype, int op, int32_t* status_word, void* stream);

/* ---- tcgen05 kernel and its step plan ------------------------------------
 * For fp16 / bf16 / fp32 (as TF32) and bs 64 / 128 the same products run on tcgen05 tensor
 * cores from a step plan.  A panel is a run of up to `width` (1 or 2) output
 * blocks, consecutive in the output LUT and in the same (batch, row) of the
 * output layout.  The reference kernel (blksprs/ops/matmul.py:148-253) re-loads
 * the x tile for every output tile of a row; here one staged A block serves the
 * whole panel and the panel's B blocks are multiplied by one wide MMA. */

/* Largest panel width for this (dtype, bs); 0 if the tcgen05 kernel does not apply. */
int bsp_umma_max_width(int dtype, int bs);

/* Number of persistent CTAs the tcgen05 kernel launches at most for this shape
 * on the current device (callers size their unit schedule as a multiple of it). */
int bsp_umma_num_ctas(int dtype, int bs, int width);

/* counts_out[p] (int32) = number of steps of panel p (inner indices t whose A
 * block exists and that hit at least one B block of the panel); touched_out[p]
 * (int32) = bit mask of the panel columns hit by any step.  panel_first is
 * int32 (n_panels+1): first output block of each panel (any grouping of
 * consecutive output blocks, up to four per panel; blocks of a panel that lie
 * in different layout rows are walked row by row).  stats (int64[3], zeroed by
 * the caller, or null) receives the largest counts_out value, the number of
 * (A block, B block) pairs all steps stand for and, with block_counts_out, the
 * largest entry of that.  block_counts_out (int32 per output block, or null)
 * receives the pairs of every single output block: the counts of the plan with
 * one block per panel, which then needs no walk of its own.  Strides as in
 * bsp_plan_count. */
int bsp_panel_count(const int64_t* lut_out, const int32_t* panel_first, int64_t n_panels,
                    const int64_t* packed_a, int64_t a_sb, int64_t a_sr, int64_t a_st,
                    const int64_t* packed_b, int64_t b_sb, int64_t b_st, int64_t b_sc,
                    int64_t T, int32_t* counts_out, int32_t* touched_out, int64_t* stats,
                    int32_t* block_counts_out, void* stream);

/* steps_out (int32, (total_steps, 8)): [0] a_block, [1..4] b_block per panel
 * column or -1, [5] control word (bits 0-3 present columns, bits 4-7 columns
 * touched for the first time, bit 8 last step of the panel, bits 12-14 panel
 * size), [6..7] zero.  step_offsets = exclusive prefix sum of the counts
 * (bsp_plan_offsets). */
int bsp_panel_fill(const int64_t* lut_out, const int32_t* panel_first, int64_t n_panels,
                   const int64_t* packed_a, int64_t a_sb, int64_t a_sr, int64_t a_st,
                   const int64_t* packed_b, int64_t b_sb, int64_t b_st, int64_t b_sc,
                   int64_t T, const int32_t* step_offsets, int32_t* steps_out, void* stream);

/* Block-sparse product on a step plan.  Same result contract as bsp_matmul_mma.
 *   unit_panel  int32 (n_units+1): the panels split into contiguous units of
 *               about equal cost (bsp_plan_schedule on step_offsets); CTA c of
 *               the launch works on units c, c + n_ctas, ...
 *   unit_step   int32 (n_units+1): step_offsets[unit_panel[u]]
 *   sched       NULL: every CTA takes the units c, c + n_ctas, ... (static).
 *               Otherwise device int32[2], zero before the first launch: after
 *               its first unit a CTA draws its next units from this counter, so
 *               slower CTAs take fewer; the kernel leaves both words zero again.
 *               One launch at a time per `sched` buffer: a launch recorded
 *               into a CUDA graph needs a buffer of its own (a replay can
 *               overlap later launches of the capture stream), and such a
 *               graph must not be replayed concurrently with itself.
 *   bias        NULL, or one element of the data dtype per output column
 *               (16-byte aligned): out[p, r, c] additionally gets
 *               bias[out_lut[p][2] * bs + c], added to the fp32 accumulator
 *               before the single rounding — the bias branch of
 *               apply_torch_linear, blksprs/utils/processing.py:72-84, fused
 *               into the product's epilogue
 *   out_lut     the output LUT (int64 (n_out, 3)); read only with a bias */
int bsp_matmul_umma(const void* a, int64_t n_a, const void* b, int64_t n_b,
                    void* out, int64_t n_out, const void* bias, const int64_t* out_lut,
                    const int32_t* panel_first, int64_t n_panels,
                    const int32_t* step_offsets, const int32_t* steps, const int32_t* touched,
                    const int32_t* unit_panel, const int32_t* unit_step, int32_t n_units,
                    int32_t* sched, int width, int bs, int dtype, int op,
                    int32_t* status_word, void* stream);

/* Self test of the bounded device wait (no reference counterpart): launches one
 * thread that waits at most `limit_us` (1..100000) microseconds on a barrier
 * nothing arrives on; the kernel must return and leave BSP_ERR_DEVICE_TIMEOUT
 * in `status_word` (device int32[1]).  The matmul kernels use the same wait
 * with a limit of about one second. */
int bsp_selftest_wait_limit(uint32_t limit_us, int32_t* status_word, void* stream);

/* Compressed transpose.  Replaces transpose_forward + flow_pull_kernel,
 * blksprs/ops/transpose.py:45-51, blksprs/ops/flow.py:64-111:
 *   out[p] = x[src_index[p]]^T  for p in [0, n_out), where src_index (int64,
 * n_out) is packed_indices(layout) gathered at the transposed coordinates of
 * the p-th non-zero of the transposed layout; out[p] = 0 when src_index[p] < 0.
 * elem_bytes is 1, 2, 4 or 8. */
int bsp_transpose_blocks(const void* x, int64_t n_x, void* out, int64_t n_out,
                         const int64_t* src_index, int bs, int elem_bytes,
                         void* stream);

/* ---- dense <-> compressed conversion ------------------------------------ */

/* Dense -> compressed.  Replaces to_sparse_forward + to_sparse_kernel,
 * blksprs/ops/conversion.py:191-276: out[p] = block (b, r, c) of the dense
 * (B, rows, cols) tensor for the p-th row (b, r, c) of `lut` (int64 (n,3)).
 * elem_bytes is 1, 2, 4 or 8. */
int bsp_to_sparse(const void* dense, int64_t B, int64_t rows, int64_t cols,
                  const int64_t* lut, int64_t n, int bs, int elem_bytes,
                  void* out, void* stream);

/* Compressed -> dense.  Replaces to_dense_forward + to_dense_kernel,
 * blksprs/ops/conversion.py:463-557, in one pass: block (b, r, c) of the dense
 * (B, R*bs, C*bs) result is x[packed[b,r,c]] where the reverse LUT entry is
 * >= 0 and is filled with `fill_bits` (the bit pattern of one element, low
 * bytes first) elsewhere. */
int bsp_to_dense(const void* x, int64_t n_x, const int64_t* packed,
                 int64_t B, int64_t R, int64_t C, int bs, int elem_bytes,
                 uint64_t fill_bits, void* dense, void* stream);

/* ---- row-wise block-sparse softmax (fp32) ------------------------------- */

/* out = softmax over every matrix row of the block-sparse tensor, taken over
 * the row's active blocks only (inactive blocks count as -inf).  Replaces
 * softmax_forward, blksprs/ops/softmax.py:93-144 (row_wise_max, row_wise_sub,
 * exp, row_wise_sum, softmax_kernel) and the fused variant :438-466 with one
 * kernel.  `packed` is the reverse LUT of the (B, R, C) layout. */
int bsp_softmax_fwd(const float* x, int64_t n_x, const int64_t* packed,
                    int64_t B, int64_t R, int64_t C, int bs, float* out, void* stream);

/* softmax(scale * x) over the active blocks of every row, with x of any of the
 * data types and the result in `out_dtype` (fp32 arithmetic): the scale, the
 * casts and the softmax of the reference's attention-by-parts chain
 * (test/cases/test_blocksparse.py:1517-1529: matmul, * scale, softmax,
 * blksprs/ops/softmax.py:23-144) in one pass, used behind the mma.sync matmul
 * kernels (block size 16 / 32).  BSP_ERR_UNSUPPORTED for layouts with more
 * than 8192 block columns. */
int bsp_softmax_fwd_scaled(const void* x, int in_dtype, int64_t n_x, const int64_t* packed,
                           int64_t B, int64_t R, int64_t C, int bs, float scale,
                           void* out, int out_dtype, void* stream);

/* Gradient of softmax(scale * x) with respect to x from the probabilities `o`
 * and their gradient `grad_out`: grad_x = scale * o * (grad_out - sum over the
 * row of grad_out * o), each tensor in its own data type (fp32 arithmetic): the
 * casts, blksprs/ops/softmax.py:157-208 and the scale of the backward of the
 * attention-by-parts chain in one pass.  BSP_ERR_UNSUPPORTED for layouts with
 * more than 8192 block columns. */
int bsp_softmax_bwd_scaled(const void* grad_out, int g_dtype, const void* o, int o_dtype, int64_t n_x,
                           const int64_t* packed, int64_t B, int64_t R, int64_t C, int bs,
                           float scale, void* grad_x, int x_dtype, void* stream);

/* grad_x = o * (grad_out - sum_row(grad_out * o)).  Replaces softmax_backward,
 * blksprs/ops/softmax.py:157-208 and :479-520. */
int bsp_softmax_bwd(const float* grad_out, const float* o, int64_t n_x, const int64_t* packed,
                    int64_t B, int64_t R, int64_t C, int bs, float* grad_x, void* stream);

/* Matmul + scale + softmax, first half: the forward product of bsp_matmul_umma
 * (same plan arguments, BSP_OP_NN) whose epilogue turns the fp32 accumulators
 * into s = scale * acc, takes the maximum m of every matrix row inside the
 * block, and writes exp(s - m) to `out` (dtype of the operands) and
 * (m, sum of exp) to stats[block][row] (fp32 pairs, (n_out, bs, 2)).  Blocks
 * without a pair hold scores of zero: exp = 1, stats (0, bs).  Together with
 * bsp_softmax_normalize this replaces the chain matmul -> multiply by a scale
 * -> softmax of the reference (blksprs/ops/matmul.py:17-67,
 * blksprs/ops/softmax.py:23-144, as used in test/cases/test_blocksparse.py:
 * 1517-1529) without the score tensor ever being written or re-read as such. */
int bsp_matmul_umma_softmax(const void* a, int64_t n_a, const void* b, int64_t n_b, void* out,
                            int64_t n_out, float* stats, float scale,
                            const int32_t* panel_first, int64_t n_panels, const int32_t* step_offsets,
                            const int32_t* steps, const int32_t* touched, const int32_t* unit_panel,
                            const int32_t* unit_step, int32_t n_units, int32_t* sched, int width,
                            int bs, int dtype, int32_t* status_word, void* stream);

/* Second half: with M = max over the blocks of a block row of m and
 * L = sum over them of l * exp(m - M), out = e * exp(m - M) / L, converted to
 * `out_dtype` (BSP_F16 / BSP_BF16 / BSP_F32).  row_first: int32
 * (n_block_rows + 1), index of the first compressed block of every block row
 * of the layout (a block row's blocks are consecutive in the compressed
 * tensor).  Same result as softmax_forward, blksprs/ops/softmax.py:93-144, on
 * the scaled scores, followed by a cast. */
int bsp_softmax_normalize(const void* e, int in_dtype, const float* stats, int64_t n_blocks,
                          const int32_t* row_first, int64_t n_block_rows, int bs, void* out,
                          int out_dtype, void* stream);

/* ---- the sparse linear helper (bias and chunked weight gradient) -------- */

/* out[p, r, c] = x[p, r, c] + bias[lut[p][2] * bs + c] for the n_blocks rows
 * (batch, row, column) of the output LUT `lut` (int64 (n,3)); `bias` holds
 * n_cols elements of the data dtype.  x and out may be the same buffer.
 * Replaces the bias branch of apply_torch_linear[_cached],
 * blksprs/utils/processing.py:72-84 and :170-198 (to_sparse of a repeated
 * bias slice, `repeat` over the output layout, elementwise add), in one pass
 * without materialising the bias per block. */
int bsp_bias_add(const void* x, const int64_t* lut, int64_t n_blocks, int bs,
                 const void* bias, int64_t n_cols, int dtype, void* out, void* stream);

/* grad_bias[lut[p][2] * bs + c] += sum over r of grad_out[p, r, c], in fp32
 * (the caller zeroes grad_bias).  Replaces what autograd derives for the same
 * branch: the backward of the add, of `repeat` and of to_sparse
 * (blksprs/utils/processing.py:72-84). */
int bsp_bias_grad(const void* grad_out, const int64_t* lut, int64_t n_blocks, int bs,
                  int dtype, float* grad_bias, int64_t n_cols, void* stream);

/* out[i] = sum over s < n_chunks of parts[s * numel + i], accumulated in fp32
 * and rounded once; numel is a multiple of 8.  Folds the per-chunk weight
 * gradients of the linear helper; the reference gets the same sum from the
 * backward of `w.repeat(batch, 1, 1)` (blksprs/utils/processing.py:52). */
int bsp_sum_chunks(const void* parts, int64_t n_chunks, int64_t numel, int dtype,
                   void* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BLKSPRS_B200_H */
