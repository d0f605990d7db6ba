// Block-sparse dsd (and, through the transposed problem, dds) on the Blackwell tensor
// path for block 64 and 128: tcgen05.mma with the accumulator in tensor memory,
// operands brought in by TMA.
//
// Same contract as the mma.sync kernel of dsd_impl.cuh (which replaces the launch of
// torch_blocksparse/matmul.py:498-504, 545-551): C[rows of a block-row] = sum over the
// nonzero blocks (i, j) of that block-row of op(S)(i, j) . B[rows of block j].  The sparse
// operand is used as stored (K-major A tiles) or transposed (MN-major A tiles, lists from the
// CSC side of the metadata).
//
// Geometry: every MMA has M = 128.  A CTA owns 128 rows of C (one block-row for block 128,
// block-rows 2i and 2i + 1 for block 64) and 128 columns, and walks "stages" of K = 64:
//   block 128  the two halves of every nonzero block of the row;
//   block 64   the union of the two rows' column blocks, in column order; the half of the
//              A tile whose row has no block there is filled with zeros by an out-of-range
//              TMA box.
// A stage is 16 KB of A (128 rows x 64 k, K-major) and 16 KB of the dense operand (64 k x
// 128 n), one N = 128 MMA per K-step: n contiguous -> MN-major B (two 64-wide groups, 8 KB
// apart, in one descriptor); k contiguous -> K-major B.
//
// Warps: 0-3 write the result back (tensor memory -> registers -> global), 4 issues the TMA
// loads (one thread), 5 issues the MMAs (one thread).  mbarriers only; every wait is bounded
// (tc.cuh) and a wait that expires sets the device status word of the tcgen05 kernels.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "common.h"
#include "tc.cuh"
#include "mm_tc.cuh"

namespace bsp {

// Set by a kernel whose bounded wait expired; read through dsd_tc_device_status().
static __device__ int g_dsd_status;

namespace {

using namespace tc;
using namespace mmtc;

constexpr int kTN = 128;          // columns of C per CTA
constexpr int kStages = 3;
constexpr int kStageBytes = 32768;
constexpr int kSmem = kStages * kStageBytes + 1024;
constexpr int kThreads = 192;

struct DsdTcArgs {
  void* c;
  int64_t c_sz, c_sh, c_sm, c_sn;
  int H, Mb, block, rows_total, nnz_rows;   // rows_total = Mb * block; nnz_rows = nnz * block (first out-of-range row of S)
  int tiles_per_head;
  const int32_t *row_ptr, *blk_col;          // lists of a block-row of op(S): CSR of the layout, or (transposed use) its CSC
  const int32_t* blk_id;                     // storage index of every list entry (NULL: the entry's own position)
};

// B_KMAJOR: the dense operand has k contiguous ([n][k] in memory); else n contiguous ([k][n]).
// C_ROWS: the result has unit stride along n (a thread writes its row with 16-byte stores);
// else unit stride along m (the transposed problem of dds: lanes write neighbouring addresses).
// A_MN: the sparse operand is used transposed: a stored block [k][m] is an MN-major A tile, two
// groups of 64 m each holding 64 k-rows of 128 bytes (the second group 8 KB after the first).
template <typename T, bool A_MN, bool B_KMAJOR, bool C_ROWS>
__global__ void __launch_bounds__(kThreads, 2)
dsd_tc_kernel(const __grid_constant__ CUtensorMap m_s, const __grid_constant__ CUtensorMap m_b, DsdTcArgs a) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024 - (saddr(smem_raw) & 1023)) & 1023);
  __shared__ uint64_t bar_full[kStages], bar_empty[kStages], bar_done;
  __shared__ uint32_t tmem_slot;
  __shared__ int n_stages, failed[2];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = blockIdx.x, n0 = blockIdx.y * kTN, z = blockIdx.z;
  const int h = tile / a.tiles_per_head, tr = tile % a.tiles_per_head;
  const int block = a.block;
  // block-rows of this tile and their nonzero lists (CSR order = storage order of the blocks)
  const int r0 = block == 128 ? tr : 2 * tr;
  const int r1 = (block == 64 && 2 * tr + 1 < a.Mb) ? 2 * tr + 1 : -1;
  const int p0 = a.row_ptr[h * a.Mb + r0], e0 = a.row_ptr[h * a.Mb + r0 + 1];
  const int p1 = r1 >= 0 ? a.row_ptr[h * a.Mb + r1] : 0, e1 = r1 >= 0 ? a.row_ptr[h * a.Mb + r1 + 1] : 0;

  if (tid == 0) {
    failed[0] = 0;
    failed[1] = kWaitBudget;
    for (int s = 0; s < kStages; ++s) { mbar_init(&bar_full[s], 1); mbar_init(&bar_empty[s], 1); }
    mbar_init(&bar_done, 1);
    mbar_init_fence();
    int n = 0;
    if (block == 128) {
      n = 2 * (e0 - p0);
    } else {                                   // size of the union of the two column lists
      int i = p0, j = p1;
      while (i < e0 || j < e1) {
        const int ci = i < e0 ? a.blk_col[i] : 0x7fffffff, cj = j < e1 ? a.blk_col[j] : 0x7fffffff;
        if (ci <= cj) ++i;
        if (cj <= ci) ++j;
        ++n;
      }
    }
    n_stages = n;
  }
  if (warp == 1) { tmem_alloc(&tmem_slot, kTN); tmem_relinquish(); }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem = tmem_slot;
  const int ns = n_stages;
  volatile int* fl = failed;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && ns > 0) {
      prefetch_map(&m_s); prefetch_map(&m_b);
      int i = p0, j = p1;
      for (int it = 0; it < ns; ++it) {
        const int s = it % kStages;
        if (it >= kStages && !mbar_wait(&bar_empty[s], ((it / kStages) - 1) & 1, fl)) break;
        unsigned char* sp = smem + s * kStageBytes;
        int krow;                               // first row of the dense operand for this stage
        mbar_expect_tx(&bar_full[s], kStageBytes);
        if (block == 128) {
          const int e = p0 + (it >> 1), kh = it & 1;
          const int bid = a.blk_id ? a.blk_id[e] : e;
          if (A_MN) {                               // rows kh * 64 .. of the stored block, its two halves of 64 columns
            tma_load_3d(sp, &m_s, &bar_full[s], 0, bid * 128 + kh * 64, z);
            tma_load_3d(sp + 8192, &m_s, &bar_full[s], 64, bid * 128 + kh * 64, z);
          } else {
            tma_load_3d(sp, &m_s, &bar_full[s], kh * 64, bid * 128, z);
          }
          krow = a.blk_col[e] * 128 + kh * 64;
        } else {
          const int ci = i < e0 ? a.blk_col[i] : 0x7fffffff, cj = j < e1 ? a.blk_col[j] : 0x7fffffff;
          const int col = ci < cj ? ci : cj;
          // a row without a block in this column gets zeros: the box lies past the last block
          tma_load_3d(sp, &m_s, &bar_full[s], 0, ci == col ? (a.blk_id ? a.blk_id[i] : i) * 64 : a.nnz_rows, z);
          tma_load_3d(sp + 8192, &m_s, &bar_full[s], 0, cj == col ? (a.blk_id ? a.blk_id[j] : j) * 64 : a.nnz_rows, z);
          if (ci == col) ++i;
          if (cj == col) ++j;
          krow = col * 64;
        }
        if (B_KMAJOR) {
          tma_load_4d(sp + 16384, &m_b, &bar_full[s], krow, n0, h, z);
        } else {
          tma_load_4d(sp + 16384, &m_b, &bar_full[s], n0, krow, h, z);
          tma_load_4d(sp + 16384 + 8192, &m_b, &bar_full[s], n0 + 64, krow, h, z);
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && ns > 0) {
      const uint32_t idesc = instr_desc(128, 128, B_KMAJOR ? 0 : 1, Bf<T>::v) | (A_MN ? 1u << 15 : 0u);
      bool ok = true;
      for (int it = 0; ok && it < ns; ++it) {
        const int s = it % kStages;
        // (MN-major A: 8 KB between its two groups of 64 rows, in the leading-offset field)
        const uint32_t a_lo = A_MN ? (((saddr(smem + s * kStageBytes) & 0x3FFFF) >> 4) | (512u << 16))
                                   : desc_lo(saddr(smem + s * kStageBytes));
        // (MN-major B: 8 KB between its two groups of 64 columns, in the leading-offset field)
        const uint32_t b_lo = B_KMAJOR ? desc_lo(saddr(smem + s * kStageBytes + 16384))
                                       : (((saddr(smem + s * kStageBytes + 16384) & 0x3FFFF) >> 4) | (512u << 16));
        ok = mbar_wait(&bar_full[s], (it / kStages) & 1, fl);
        if (!ok) break;
        fence_after();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          const uint32_t acc = (it > 0 || ks > 0) ? 1u : 0u;
          const uint64_t da = desc_from_lo(a_lo + ks * (A_MN ? 128 : 2));   // per K-step: 32 bytes (K-major), 16 rows (MN-major)
          // per K-step: 32 bytes (K-major) or 16 rows = 2048 bytes (MN-major)
          mma_ss(tmem, da, desc_from_lo(b_lo + ks * (B_KMAJOR ? 2 : 128)), idesc, acc);
        }
        commit(&bar_empty[s]);                                      // the stage is free once these MMAs have read it
      }
      if (ok) commit(&bar_done);
    }
  } else {
    // ------------------------------------------------------------------ write-back
    const int row = warp * 32 + lane;
    const int grow = (block == 128 ? r0 * 128 : r0 * 64) + row;
    const bool row_ok = grow < a.rows_total && (block == 128 || row < 64 || r1 >= 0);
    T* crow = reinterpret_cast<T*>(a.c) + z * a.c_sz + h * a.c_sh + (int64_t)grow * a.c_sm + (int64_t)n0 * a.c_sn;
    bool ok = true;
    if (ns > 0) ok = mbar_wait_warp(&bar_done, 0, fl);
    if (ok) {
      fence_after();
      const uint32_t ta = tmem + ((uint32_t)(warp * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < kTN; c += 32) {
        uint32_t r[32];
        if (ns > 0) {
          tmem_ld32(ta + c, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;                   // a block-row without blocks: zeros, as the reference gives
        }
        if (row_ok) {
          if (C_ROWS) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 v;
              v.x = pack2<T>(__uint_as_float(r[i]), __uint_as_float(r[i + 1]));
              v.y = pack2<T>(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
              v.z = pack2<T>(__uint_as_float(r[i + 4]), __uint_as_float(r[i + 5]));
              v.w = pack2<T>(__uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]));
              *reinterpret_cast<uint4*>(crow + c + i) = v;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) crow[(int64_t)(c + i) * a.c_sn] = cvt1<T>(__uint_as_float(r[i]));
          }
        }
      }
    }
  }
  fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, kTN);
  if (tid == 0 && failed[0]) atomicExch(&g_dsd_status, 4);
}

template <typename T, bool AM, bool BK, bool CR>
int launch(const CUtensorMap& ms, const CUtensorMap& mb, const DsdTcArgs& a, dim3 grid, cudaStream_t st) {
  auto kern = dsd_tc_kernel<T, AM, BK, CR>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
  if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "dsd (tcgen05): cannot reserve shared memory: %s", cudaGetErrorString(e));
  kern<<<grid, kThreads, kSmem, st>>>(ms, mb, a);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "dsd (tcgen05) launch failed: %s", cudaGetErrorString(e));
  return BSP_OK;
}

template <typename T, bool AM>
int launch_a(bool bk, bool cr, const CUtensorMap& ms, const CUtensorMap& mb, const DsdTcArgs& a, dim3 grid, cudaStream_t st) {
  if (bk) return cr ? launch<T, AM, true, true>(ms, mb, a, grid, st) : launch<T, AM, true, false>(ms, mb, a, grid, st);
  return cr ? launch<T, AM, false, true>(ms, mb, a, grid, st) : launch<T, AM, false, false>(ms, mb, a, grid, st);
}

template <typename T>
int launch_t(bool am, bool bk, bool cr, const CUtensorMap& ms, const CUtensorMap& mb, const DsdTcArgs& a, dim3 grid, cudaStream_t st) {
  return am ? launch_a<T, true>(bk, cr, ms, mb, a, grid, st) : launch_a<T, false>(bk, cr, ms, mb, a, grid, st);
}

}  // namespace

// True when dsd_tc covers the case: FP16 / BF16, block 64 / 128, N a multiple of 128, both dense tensors with one unit inner stride and 16-byte friendly
// addresses and strides.
bool dsd_tc_eligible(const void* s, const void* b, const void* c, int dtype, int block, int N, int trans_s, int64_t s_sz,
                     int64_t b_sz, int64_t b_sh, int64_t b_sk, int64_t b_sn,
                     int64_t c_sz, int64_t c_sh, int64_t c_sm, int64_t c_sn) {
  if (dtype != BSP_F16 && dtype != BSP_BF16) return false;
  if ((block != 64 && block != 128) || N % kTN) return false;
  if ((b_sk != 1) == (b_sn != 1) || (c_sm != 1) == (c_sn != 1)) return false;
  const int64_t b_outer = b_sk == 1 ? b_sn : b_sk;
  if ((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15) return false;
  if ((s_sz | b_sz | b_sh | b_outer) & 7) return false;
  if (s_sz <= 0 || b_sz <= 0 || b_sh <= 0 || b_outer <= 0) return false;     // TMA strides: no broadcast
  if (c_sn == 1 && ((c_sz | c_sh | c_sm) & 7)) return false;
  return true;
}

int dsd_tc(const void* s, const void* b, void* c, int dtype, int block, int Z, int N, int64_t s_sz, int trans_s,
           int64_t b_sz, int64_t b_sh, int64_t b_sk, int64_t b_sn,
           int64_t c_sz, int64_t c_sh, int64_t c_sm, int64_t c_sn, const Meta& m, cudaStream_t st) {
  const bool bk = b_sk == 1, cr = c_sn == 1;
  // op(S) has the layout's rows (and walks its CSR) or, transposed, its columns (CSC)
  const int out_b = trans_s ? m.Nb : m.Mb, red_b = trans_s ? m.Mb : m.Nb;
  const int64_t ktot = (int64_t)red_b * block;
  CUtensorMap ms, mb;
  {
    cuuint64_t dims[3] = {(cuuint64_t)block, (cuuint64_t)m.nnz * block, (cuuint64_t)Z};
    cuuint64_t strides[2] = {(cuuint64_t)block * 2, (cuuint64_t)(Z > 1 ? s_sz : (int64_t)m.nnz * block * block) * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)((block == 128 && !trans_s) ? 128 : 64), 1};
    if (int rc = encode(&ms, s, dtype, 3, dims, strides, box)) return rc;
  }
  {
    const int64_t inner = bk ? ktot : N, outer = bk ? N : ktot, outer_stride = bk ? b_sn : b_sk;
    cuuint64_t dims[4] = {(cuuint64_t)inner, (cuuint64_t)outer, (cuuint64_t)m.H, (cuuint64_t)Z};
    cuuint64_t strides[3] = {(cuuint64_t)outer_stride * 2, (cuuint64_t)(m.H > 1 ? b_sh : outer * outer_stride) * 2,
                             (cuuint64_t)(Z > 1 ? b_sz : (int64_t)m.H * outer * outer_stride) * 2};
    cuuint32_t box[4] = {64, (cuuint32_t)(bk ? 128 : 64), 1, 1};
    if (int rc = encode(&mb, b, dtype, 4, dims, strides, box)) return rc;
  }
  DsdTcArgs a = {};
  a.c = c; a.c_sz = c_sz; a.c_sh = c_sh; a.c_sm = c_sm; a.c_sn = c_sn;
  a.H = m.H; a.Mb = out_b; a.block = block; a.rows_total = out_b * block; a.nnz_rows = m.nnz * block;
  a.tiles_per_head = (out_b * block + 127) / 128;
  if (trans_s) { a.row_ptr = m.col_ptr; a.blk_col = m.col_row; a.blk_id = m.col_bid; }
  else { a.row_ptr = m.row_ptr; a.blk_col = m.blk_col; a.blk_id = nullptr; }
  dim3 grid(m.H * a.tiles_per_head, N / kTN, Z);
  if (dtype == BSP_F16) return launch_t<__half>(trans_s != 0, bk, cr, ms, mb, a, grid, st);
  return launch_t<__nv_bfloat16>(trans_s != 0, bk, cr, ms, mb, a, grid, st);
}

// 0, or non-zero when a bounded wait inside the kernel above expired (synchronises the device).
int dsd_tc_device_status(int* out) {
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_dsd_status, sizeof(int));
  if (e == cudaSuccess && v != 0) { const int zero = 0; e = cudaMemcpyToSymbol(g_dsd_status, &zero, sizeof(int)); }   // reading clears
  if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "device status: %s", cudaGetErrorString(e));
  *out = v;
  return BSP_OK;
}

}  // namespace bsp
