/*
 * bsp.h -- C ABI of the B200-native block-sparse hot path.
 *
 * Every entry point is extern "C", takes plain pointers / sizes / strides and
 * returns an int status (BSP_OK == 0).  After a non-zero status,
 * bsp_last_error() returns a thread-local, human readable message.
 *
 * Conventions
 *   layout   int64 host array [H, Mb, Nb]; an entry != 0 means "block present".
 *            Never modified by the library.
 *   block    edge of a square block: 16, 32, 64 or 128.
 *   block format  a sparse tensor is stored as [Z, nnz, block, block]; block b is
 *            the b-th nonzero of the layout in (h, i, j) row-major order.
 *   dtype    BSP_F32 / BSP_F16 / BSP_BF16; all operands of a call share it.
 *            16-bit types accumulate in FP32.
 *   strides  always in ELEMENTS.
 *   stream   a cudaStream_t passed as void*; launches are asynchronous on it.
 *   memory   the library never allocates device memory; every buffer (inputs,
 *            outputs, tables, scratch) is owned by the caller.
 *   meta     device copy of the buffer written by bsp_meta_build; meta_hdr is a
 *            HOST pointer to (a copy of) its first BSP_META_HEADER ints, from
 *            which the launch code reads the layout dimensions.
 *
 * The table builders run on the host and write host memory.  They are called
 * twice: first with out == NULL to learn *total (number of int32 entries),
 * then with a buffer of at least that capacity.
 */
#ifndef BSP_B200_H
#define BSP_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BSP_OK               0
#define BSP_ERR_INVALID      1  /* bad argument (maps to ValueError)            */
#define BSP_ERR_UNSUPPORTED  2  /* maps to NotImplementedError                  */
#define BSP_ERR_CAPACITY     3  /* output buffer too small; *total says how big */
#define BSP_ERR_CUDA         4  /* CUDA runtime error (maps to RuntimeError)    */
#define BSP_ERR_EMPTY_HEAD   5  /* a head of the layout has no nonzero block    */
#define BSP_ERR_TIMEOUT      6  /* a bounded device-side wait expired           */

#define BSP_F32  0
#define BSP_F16  1
#define BSP_BF16 2

#define BSP_MAX_PACKS 8

/* Message for the last non-zero status returned on this thread. */
const char* bsp_last_error(void);

/* ABI version; bumped on any signature change. */
int bsp_abi_version(void);

/* ------------------------------------------------------------------------ */
/* Layout -> table builders (host)                                          */
/* ------------------------------------------------------------------------ */

/*
 * SDD table.  Replaces _sparse_matmul.make_sdd_lut (torch_blocksparse/matmul.py:281-297)
 * together with the native sdd_segment / segment_blocks it calls
 * (csrc/utils.cpp:11-120).  Bit-identical output: nonzero blocks greedily packed
 * into w x w super-blocks for w = 64/block, w/2, ..., 1; four int32 per entry
 * (head, row, col, block id).  The tables of the successive pack sizes are
 * written back to back into `out`; packs[p], widths[p] (number of super-blocks)
 * and offsets[p] (first int of that table inside `out`) describe them, *n_packs
 * says how many there are (empty passes are omitted, as in the reference).
 * block == 128 has start width 0 in the reference and yields no table at all;
 * that behaviour is kept (n_packs == 0).
 */
int bsp_sdd_lut_build(const int64_t* layout, int H, int Mb, int Nb, int block,
                      int32_t* out, int64_t out_cap,
                      int32_t* packs, int64_t* widths, int64_t* offsets,
                      int* n_packs, int64_t* total);

/*
 * DSD / DDS table.  Replaces _sparse_matmul.load_balance + make_dxx_lut
 * (torch_blocksparse/matmul.py:221-267, 372-458).  Bit-identical output: six
 * int32 of header per segment (offset, K extent, column, head, lock id, max id),
 * then interleaved (dense increment, sparse increment) pairs and two trailing
 * zeros.  `step` is 8 for FP32 and 16 otherwise (matmul.py:617); `trans`
 * selects per-row (1) or per-column (0) reductions.  A head without any
 * nonzero block is an error (BSP_ERR_EMPTY_HEAD), as in the reference.
 */
int bsp_dxx_lut_build(const int64_t* layout, int H, int Mb, int Nb, int block,
                      int step, int trans,
                      int32_t* out, int64_t out_cap, int64_t* total,
                      int* num_locks, int* width);

/*
 * Softmax table.  Replaces _sparse_softmax.make_lut (torch_blocksparse/softmax.py:201-221).
 * Bit-identical output: (size, offset) per (head, block-row), then
 * (block id, column, row, head) per nonzero block.  *maxlut = largest number of
 * nonzero blocks in any block-row.
 */
int bsp_softmax_lut_build(const int64_t* layout, int H, int Mb, int Nb,
                          int32_t* out, int64_t out_cap, int64_t* total, int* maxlut);

/*
 * "fixed" sparse-transformer layout.  Replaces
 * DeepSpeedSparseSelfAttention._make_layout
 * (torch_blocksparse/deepspeedsparseselfattention.py:33-65).  mode: 0 dense,
 * 1 fixed.  Writes int64 [num_heads, num_blocks, num_blocks] into `out`.
 */
int bsp_fixed_layout_build(int num_heads, int num_blocks, int mode, int block_stride,
                           int unidirectional, int numverts, int vertsize, int64_t* out);

/*
 * Sliding-window layouts: block-row i sees block-columns [i - below, i + above],
 * the first `global_cols` block-columns and, per head, the `num_random`
 * block-columns listed for it in random_cols [num_heads, num_blocks, num_random]
 * (the caller draws them, so that any seeded generator can be used); the first
 * `global_rows` block-rows see everything.  below = band - 1, above = 0 gives a
 * causal band; below = above = window / 2 with random and global blocks a
 * BigBird-style layout.  Writes int64 [num_heads, num_blocks, num_blocks].
 * No counterpart in the reference (its SparsityConfig only knows "dense" and
 * "fixed", deepspeedsparseselfattention.py:16-17).
 */
int bsp_window_layout_build(int num_heads, int num_blocks, int below, int above, int global_rows, int global_cols,
                            const int32_t* random_cols, int num_random, int64_t* out);

/*
 * Execution metadata consumed by the compute kernels (no counterpart in the
 * reference, whose kernels read the tables above; those tables can contain
 * duplicate / out-of-layout entries and are therefore never executed from).
 * int32 layout of `out`:
 *   [0] magic  [1] H  [2] Mb  [3] Nb  [4] nnz  [5] max nnz per block-row
 *   [6] max nnz per block-column  [7] reserved
 *   row_ptr [H*Mb+1]   CSR offsets; the canonical block id is the CSR position
 *   blk_row [nnz]      block-row of every block
 *   blk_col [nnz]      block-column of every block
 *   blk_head[nnz]      head of every block
 *   col_ptr [H*Nb+1]   CSC offsets
 *   col_row [nnz]      block-row of every block in CSC order
 *   col_bid [nnz]      canonical block id of every block in CSC order
 *   row_order [H*Mb]   (head*Mb + row) sorted by descending nnz (stable)
 *   col_order [H*Nb]   (head*Nb + col) sorted by descending nnz (stable)
 */
#define BSP_META_MAGIC 0x42535031
#define BSP_META_HEADER 8
int bsp_meta_build(const int64_t* layout, int H, int Mb, int Nb,
                   int32_t* out, int64_t out_cap, int64_t* total);

/*
 * bsp_meta_build on the device: `layout` is a DEVICE pointer to [H, Mb, Nb]
 * elements of elem_bytes (1, 4 or 8) bytes, nonzero = present; `out` a DEVICE
 * buffer of at least bsp_meta_device_capacity(H, Mb, Nb) ints (the worst case:
 * the number of nonzero blocks is only known once the kernels have counted
 * them).  The buffer's leading ints are bit-identical to what bsp_meta_build
 * writes for the same layout.  Runs on `stream`; when hdr_host is not NULL the
 * BSP_META_HEADER header ints are copied to it and the stream is synchronised
 * (the launch code and the caller need the block count): those 32 bytes are the
 * only host traffic.  Replaces, for the execution metadata, the reference's
 * host-side table rebuild and upload per (dtype, device)
 * (torch_blocksparse/matmul.py:611-641, 293, 455; softmax.py:220).
 */
int64_t bsp_meta_device_capacity(int H, int Mb, int Nb);
int bsp_meta_build_device(const void* layout, int elem_bytes, int H, int Mb, int Nb,
                          int32_t* out, int64_t out_cap, int32_t* hdr_host, void* stream);

/*
 * The table of bsp_softmax_lut_build written on the device from the device copy
 * of the execution metadata (bsp_meta_build or bsp_meta_build_device) of the same
 * layout: `meta_hdr` the HOST copy of its header, `meta` and `out` DEVICE
 * pointers.  Same two calls as the host builders (out == NULL: *total and
 * *maxlut only); bit-identical contents; runs on `stream`, does not
 * synchronise.  With bsp_meta_build_device a layout that lives in device memory
 * gets its softmax table without a copy to the host (replaces the host-side
 * build and `.to(device)` of torch_blocksparse/softmax.py:201-221).
 */
int bsp_softmax_lut_from_meta(const int32_t* meta_hdr, const int32_t* meta, int32_t* out, int64_t out_cap,
                              int64_t* total, int* maxlut, void* stream);

/*
 * Tile lists of the tcgen05 attention kernels (no counterpart in the
 * reference).  Those kernels work on tiles of 128 query rows (forward, dQ) or
 * 128 key rows (dK, dV), made of two 64-row chunks, and walk 64-row chunks of
 * the other operand.  With block 128 a tile is one block-row; with block 64 it
 * is a pair of block-rows (block-columns) of one head, chosen by similarity of
 * their nonzero sets: its list is the union of their positions plus a 2-bit
 * mask telling which half of the tile owns the block.  int32 layout of `out`:
 *   [0] magic [1] H [2] L/block [3] block [4] tiles per head [5] row entries
 *   [6] column entries [7] block of the layout the lists were built from
 *   (blocks 16 and 32 are turned into 64-wide lists on the coarsened layout:
 *   [2] and [3] then describe those)
 *   then twice (row tiles, column tiles), n = H * tiles per head:
 *   c01 [2n] (the tile's two 64-row chunk ids, -1: none)  ptr [n+1]
 *   chunk [E]  mask [E]  sub [E]  order [n] (tiles sorted longest first)
 *   sub: per half of the tile 16 bits saying which 16 x 16 pieces of the 64 x
 *   64 position lie in a nonzero block (all ones for blocks 64 and 128).
 * block must be 16, 32, 64 or 128, and L a multiple of 64 (else
 * BSP_ERR_UNSUPPORTED).
 */
#define BSP_TILES_MAGIC 0x42535054
#define BSP_TILES_HEADER 8
int bsp_attn_tiles_build(const int64_t* layout, int H, int nb, int block,
                         int32_t* out, int64_t out_cap, int64_t* total);

/*
 * bsp_attn_tiles_build on the device, for at most 512 positions of 64 x 64 (128
 * x 128 for block 128) per side (BSP_ERR_UNSUPPORTED otherwise: build on the
 * host); blocks 16 and 32 are coarsened on the device as well: `layout`
 * is a DEVICE pointer to [H, nb, nb] elements of elem_bytes (1, 4 or 8) bytes,
 * `out` a DEVICE buffer of at least bsp_attn_tiles_device_capacity(H, nb, block)
 * ints.  Its leading ints are bit-identical to the host builder's output; the
 * BSP_TILES_HEADER header ints are copied to hdr_host when it is not NULL (the
 * stream is then synchronised).  No counterpart in the reference.
 */
int64_t bsp_attn_tiles_device_capacity(int H, int nb, int block);
int bsp_attn_tiles_build_device(const void* layout, int elem_bytes, int H, int nb, int block,
                                int32_t* out, int64_t out_cap, int32_t* hdr_host, void* stream);

/* ------------------------------------------------------------------------ */
/* Softmax (device)                                                         */
/* ------------------------------------------------------------------------ */

/*
 * In-place block-sparse row softmax.  Replaces the softmax_fwd kernel and its
 * launch code (torch_blocksparse/softmax.py:7-138, 253-313):
 *   y = softmax_row(x*scale + rpe + kpm + attn_mask), stored over x.
 * x      [Z, nnz, block, block], z-stride x_sz.
 * lut    device copy of the table written by bsp_softmax_lut_build.
 * rpe    optional [Z, H, M, N] (strides rpe_sz, rpe_sh, rpe_sr; unit column
 *        stride; rpe_sz may be 0 for a broadcast), added after the scale.
 * kpm    optional key-padding mask [Z, N] (stride kpm_sz).
 * am     optional attention mask [M, N] (row stride am_sr).
 * *_mul  0: the mask is added; 1: 'mul' mode, mask == 0 -> -inf, else 0
 *        (softmax.py:104-110).
 * Rows longer than 32767 elements are rejected with BSP_ERR_UNSUPPORTED
 * (softmax.py:225-227).
 */
int bsp_softmax_fwd(void* x, int dtype, int Z, int64_t x_sz, int block,
                    int H, int Mb, const int32_t* lut, int maxlut, float scale,
                    const void* rpe, int64_t rpe_sz, int64_t rpe_sh, int64_t rpe_sr,
                    const void* kpm, int64_t kpm_sz, int kpm_mul,
                    const void* am, int64_t am_sr, int am_mul,
                    void* stream);

/*
 * Softmax backward, in place over dy.  Replaces softmax_bwd
 * (torch_blocksparse/softmax.py:144-194, 315-326):
 *   dx = y * (dy - sum_row(y*dy)) * scale.
 */
int bsp_softmax_bwd(const void* y, void* dy, int dtype, int Z, int64_t y_sz, int64_t dy_sz,
                    int block, int H, int Mb, const int32_t* lut, int maxlut, float scale,
                    void* stream);

/* ------------------------------------------------------------------------ */
/* MatMul (device)                                                          */
/* ------------------------------------------------------------------------ */

/*
 * SDD: C_sparse = A . B sampled on the layout.  Replaces the SDD variant of the
 * reference kernel and _sdd_matmul (torch_blocksparse/matmul.py:30-54, 299-364).
 * A is the logical [Z, H, Mb*block, K] operand and B the logical
 * [Z, H, K, Nb*block] operand, both addressed through element strides, which is
 * how trans_a / trans_b / trans_c of the reference are expressed (one of the
 * two inner strides of each operand must be 1).  C is written in block format
 * (z-stride c_sz), every block completely.  K must be a multiple of 16
 * (matmul.py:318-319), else BSP_ERR_INVALID.
 */
int bsp_sdd(const void* a, const void* b, void* c, int dtype, int block,
            int Z, int H, int K,
            int64_t a_sz, int64_t a_sh, int64_t a_sm, int64_t a_sk,
            int64_t b_sz, int64_t b_sh, int64_t b_sk, int64_t b_sn,
            int64_t c_sz, const int32_t* meta_hdr, const int32_t* meta, void* stream);

/*
 * DSD: C_dense = op(S) . B.  Replaces the DSD variant and _dsd_matmul
 * (torch_blocksparse/matmul.py:66-82, 507-552).  S is in block format (z-stride
 * s_sz); trans_s != 0 uses S transposed.  B is the logical [Z, H, K, N] operand,
 * C the logical [Z, H, M, N] result, both through element strides (trans_b and
 * trans_c of the reference).  Every element of C is written, zeros where a
 * block-row of op(S) is empty.
 */
int bsp_dsd(const void* s, const void* b, void* c, int dtype, int block,
            int Z, int H, int N, int64_t s_sz, int trans_s,
            int64_t b_sz, int64_t b_sh, int64_t b_sk, int64_t b_sn,
            int64_t c_sz, int64_t c_sh, int64_t c_sm, int64_t c_sn,
            const int32_t* meta_hdr, const int32_t* meta, void* stream);

/*
 * DDS: C_dense = A . op(S).  Replaces the DDS variant and _dds_matmul
 * (torch_blocksparse/matmul.py:83-99, 460-505).  A is the logical [Z, H, M, K]
 * operand, C the logical [Z, H, M, N] result.
 */
int bsp_dds(const void* a, const void* s, void* c, int dtype, int block,
            int Z, int H, int M,
            int64_t a_sz, int64_t a_sh, int64_t a_sm, int64_t a_sk,
            int64_t s_sz, int trans_s,
            int64_t c_sz, int64_t c_sh, int64_t c_sm, int64_t c_sn,
            const int32_t* meta_hdr, const int32_t* meta, void* stream);

/*
 * Debug aids (no counterpart in the reference): check every index the compute
 * kernels will derive from a DEVICE metadata buffer (bsp_meta_build /
 * bsp_meta_build_device) or from DEVICE attention tile lists
 * (bsp_attn_tiles_build) of `len` ints against the sizes in the buffer's own
 * header - pointers monotone and in range, block ids below the block count,
 * rows / columns / heads / chunk ids inside the layout, orders inside their
 * range.  Returns BSP_OK, or BSP_ERR_INVALID with the number of the failed check
 * in *code and the offending entry in *pos.  Synchronises `stream`.  The Python
 * layer runs them on every buffer it uploads when BSP_DEBUG=1 is set in the
 * environment; they stand in for a device memory checker on systems where none
 * can be run.
 */
int bsp_meta_validate(const int32_t* meta, int64_t len, int* code, int* pos, void* stream);
int bsp_attn_tiles_validate(const int32_t* tiles, int64_t len, int* code, int* pos, void* stream);

/* ------------------------------------------------------------------------ */
/* Fused sparse self-attention (device)                                     */
/* ------------------------------------------------------------------------ */

/*
 * O = softmax(scale * Q K^T + rpe + kpm + attn_mask on the layout) . V in one
 * kernel.  Replaces the three-launch chain of
 * DeepSpeedSparseSelfAttention.forward
 * (torch_blocksparse/deepspeedsparseselfattention.py:157-166) without writing
 * the score tensor to memory.  q, k, v, o are [Z, H, L, D] with unit stride on
 * D and the given z / h / row strides; lse is FP32 [Z, H, L]: per row
 * log2(sum_j exp(f_j)) of the pre-softmax values f, consumed by the backward.  D is 64 or 128; dtype F16 or BF16.
 * tiles / tiles_hdr: optional device copy of the buffer written by
 * bsp_attn_tiles_build and a HOST pointer to its first BSP_TILES_HEADER ints.
 * When given (lists built for this block size; q, k, v with positive strides;
 * rpe, key-padding mask and attention mask, where present, with 16-byte
 * aligned bases and strides that are multiples of 8 elements) the tcgen05 +
 * tensor-memory + TMA kernels run; otherwise, or with NULL, the mma.sync
 * kernels do.  Both give the
 * same result within rounding.  A query row whose keys are all masked out gets
 * zeros (the reference's softmax gives NaN there).
 * am_mul = 2: the caller vouches that `am` is the lower-triangular causal mask
 * in 'mul' form (am[i][j] != 0 exactly for j <= i); kernels that can do so
 * derive it from the indices instead of reading it, the others read it as with
 * am_mul = 1.
 */
int bsp_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                 int dtype, int block, int Z, int H, int L, int D,
                 int64_t q_sz, int64_t q_sh, int64_t q_sr,
                 int64_t k_sz, int64_t k_sh, int64_t k_sr,
                 int64_t v_sz, int64_t v_sh, int64_t v_sr,
                 int64_t o_sz, int64_t o_sh, int64_t o_sr,
                 const int32_t* meta_hdr, const int32_t* meta,
                 const int32_t* tiles_hdr, const int32_t* tiles, float scale,
                 const void* rpe, int64_t rpe_sz, int64_t rpe_sh, int64_t rpe_sr,
                 const void* kpm, int64_t kpm_sz, int kpm_mul,
                 const void* am, int64_t am_sr, int am_mul,
                 void* stream);

/*
 * Backward of bsp_attn_fwd: dq, dk, dv from q, k, v, o, do and lse, recomputing
 * the probabilities block by block.  `delta` is caller-provided FP32 scratch of
 * Z*H*L elements (row sums of o*do).  dq/dk/dv are contiguous [Z, H, L, D].
 * On the tcgen05 kernels the dQ kernel is launched on a second stream that the
 * library keeps per calling thread and device (created on first use), forked
 * from and joined to `stream` by events: work queued on `stream` after the call
 * sees all three gradients.
 */
int bsp_attn_bwd(const void* q, const void* k, const void* v, const void* o,
                 const void* dout, const float* lse, float* delta,
                 void* dq, void* dk, void* dv,
                 int dtype, int block, int Z, int H, int L, int D,
                 int64_t q_sz, int64_t q_sh, int64_t q_sr,
                 int64_t k_sz, int64_t k_sh, int64_t k_sr,
                 int64_t v_sz, int64_t v_sh, int64_t v_sr,
                 int64_t o_sz, int64_t o_sh, int64_t o_sr,
                 int64_t do_sz, int64_t do_sh, int64_t do_sr,
                 const int32_t* meta_hdr, const int32_t* meta,
                 const int32_t* tiles_hdr, const int32_t* tiles, float scale,
                 const void* rpe, int64_t rpe_sz, int64_t rpe_sh, int64_t rpe_sr,
                 const void* kpm, int64_t kpm_sz, int kpm_mul,
                 const void* am, int64_t am_sr, int am_mul,
                 void* stream);

/*
 * The same backward, restricted to the steps selected by the bit mask `parts`
 * (1: delta = rowsum(o*do), 2: dk and dv, 4: dq), so that a caller can time or
 * schedule the three launches separately.  Step 2 and 4 read the delta written
 * by step 1.  bsp_attn_bwd is parts == 7.  No counterpart in the reference.
 */
int bsp_attn_bwd_parts(const void* q, const void* k, const void* v, const void* o,
                       const void* dout, const float* lse, float* delta,
                       void* dq, void* dk, void* dv,
                       int dtype, int block, int Z, int H, int L, int D,
                       int64_t q_sz, int64_t q_sh, int64_t q_sr,
                       int64_t k_sz, int64_t k_sh, int64_t k_sr,
                       int64_t v_sz, int64_t v_sh, int64_t v_sr,
                       int64_t o_sz, int64_t o_sh, int64_t o_sr,
                       int64_t do_sz, int64_t do_sh, int64_t do_sr,
                       const int32_t* meta_hdr, const int32_t* meta,
                 const int32_t* tiles_hdr, const int32_t* tiles, float scale,
                       const void* rpe, int64_t rpe_sz, int64_t rpe_sh, int64_t rpe_sr,
                       const void* kpm, int64_t kpm_sz, int kpm_mul,
                       const void* am, int64_t am_sr, int am_mul,
                       int parts, void* stream);

/*
 * Backward of bsp_attn_fwd for callers that cannot allocate device memory.
 * (No counterpart in the reference.)  Some hosts of this library have no
 * allocator to hand: a runtime that pre-plans all of its device memory and
 * forbids cudaMalloc once it is running, a plug-in that only receives the
 * tensors of its inputs and outputs, code that runs inside a region where the
 * driver's allocator must not be entered.  bsp_attn_bwd asks such a caller for
 * Z*H*L floats of scratch it has no way to provide.  This variant takes the
 * same arguments minus `delta` and keeps that scratch in an array built into
 * the library image instead (BSP_ATTN_STATIC_ROWS floats = 4 MiB, resident on
 * every GPU that loads the library until the process exits).  It calls no
 * allocating routine of any kind.
 *
 *   limit     Z*H*L <= BSP_ATTN_STATIC_ROWS, else BSP_ERR_UNSUPPORTED.
 *   set-up    the first call on each device looks up the device address of the
 *             array (cudaGetSymbolAddress, with that device current) and caches
 *             it; make that first call outside any stream capture.  The device
 *             that `stream` belongs to must be the current device of the calling
 *             thread.  That first call may also be the moment the driver loads
 *             the library's device code and reserves the 4 MiB, so a caller that
 *             forbids allocation after start-up should make one warm-up call
 *             during start-up.  The cached address does not survive
 *             cudaDeviceReset.
 *   sharing   every call on a device uses the same array, which keeps whatever
 *             the previous call left in it.  Nothing in it has to start at
 *             zero: the first kernel of the call overwrites the Z*H*L entries
 *             the later ones read.  Two calls that overlap on the GPU (different
 *             streams, or different threads) race on it; serialise them.
 * Results are identical to bsp_attn_bwd.
 */
#define BSP_ATTN_STATIC_ROWS (1 << 20)
int bsp_attn_bwd_static(const void* q, const void* k, const void* v, const void* o,
                        const void* dout, const float* lse,
                        void* dq, void* dk, void* dv,
                        int dtype, int block, int Z, int H, int L, int D,
                        int64_t q_sz, int64_t q_sh, int64_t q_sr,
                        int64_t k_sz, int64_t k_sh, int64_t k_sr,
                        int64_t v_sz, int64_t v_sh, int64_t v_sr,
                        int64_t o_sz, int64_t o_sh, int64_t o_sr,
                        int64_t do_sz, int64_t do_sh, int64_t do_sr,
                        const int32_t* meta_hdr, const int32_t* meta,
                 const int32_t* tiles_hdr, const int32_t* tiles, float scale,
                        const void* rpe, int64_t rpe_sz, int64_t rpe_sh, int64_t rpe_sr,
                        const void* kpm, int64_t kpm_sz, int kpm_mul,
                        const void* am, int64_t am_sr, int am_mul,
                        void* stream);

/*
 * Reads and clears the device-side status words (synchronises the device).
 * *status = 0 and BSP_OK when no bounded wait inside a tcgen05 kernel has expired
 * since the last read; otherwise *status = 1 (attention forward), 2 (attention
 * dQ), 3 (attention dK/dV), 4 (dsd / dds) or 5 (sdd), the return value is
 * BSP_ERR_TIMEOUT and the outputs of the launch that set it are not valid.  A
 * caller checks it where it synchronises anyway.  No counterpart in the
 * reference.
 */
int bsp_device_status(int* status);

/*
 * Test hook of the bounded waits (no counterpart in the reference): the number
 * of attempts a wait inside the tcgen05 attention kernels may make
 * (wait_budget <= 0: the default, 2^21) and, with skip_chunk >= 0, the loads of
 * that chunk of every tile are withheld, so that the waits for it run out and
 * the kernels return with the status word set instead of waiting for ever.
 * Process-wide; applies to launches made afterwards.
 */
int bsp_debug_attn_wait(int wait_budget, int skip_chunk);

/*
 * Kernel family of bsp_sdd / bsp_dsd / bsp_dds for block 32 / 64 / 128 with
 * FP16 / BF16 operands (no counterpart in the reference): non-zero (the default)
 * lets the cases the tcgen05 kernels cover (sdd: K a multiple of 64; dsd / dds:
 * dense width a multiple of 128 and at most 1024 blocks on the reduction side;
 * TMA-friendly strides) run on them; zero keeps every product on the mma.sync
 * kernels.  Process-wide.  At block 32 / 64 the tcgen05 dsd / dds kernel fills
 * the places of absent blocks with zeros instead of skipping them, so a
 * non-finite value of the dense operand can turn into NaN in output rows whose
 * own blocks do not touch it.
 */
int bsp_matmul_use_tcgen05(int enable);

#ifdef __cplusplus
}
#endif
#endif /* BSP_B200_H */
