// Block-sparse sdd on the Blackwell tensor path for block 32, 64 and 128: tcgen05.mma with the
// accumulator in tensor memory, operands brought in by TMA.
//
// Same contract as the mma.sync kernel of sdd_impl.cuh (which replaces the launch of
// torch_blocksparse/matmul.py:354-360): every nonzero block (i, j) of the layout receives
// op(A)[rows of block-row i, :] . op(B)[:, columns of block-column j].
//
// Geometry: every MMA has M = 128 and the CTA's accumulator is 128 x 128.
//   block 128  a CTA computes one nonzero block;
//   block 64   a CTA takes block-rows 2i and 2i + 1 and two consecutive entries of the union
//              of their column lists: four blocks, of which those the layout holds are stored;
//   block 32   four block-rows and four consecutive entries of the union of their column
//              lists: sixteen blocks, of which those the layout holds are stored.
// The reduction runs over K in stages of 64: 16 KB of A (128 m x 64 k, two TMA boxes of 64 x
// 64) and 16 KB of B (64 k x 128 n, one box per column block).  Either operand may have k or
// its other dimension contiguous: k contiguous gives K-major tiles, the other case MN-major
// tiles (groups of 64 rows or columns, 8 KB apart, in one descriptor; the 32 columns of a
// block-32 column block form groups of 4 KB in the 64-byte swizzle); every K-step is one
// 128 x 128 x 16 MMA.  A box that lies outside the tensor (block-rows past the last one,
// missing columns at the end of the union) is filled with zeros.
//
// Warps: 0-3 write the blocks back, 4 issues the TMA loads, 5 the MMAs (one thread each).
// mbarriers only; every wait is bounded and a wait that expires sets a device status word.
#include <algorithm>
#include "mm_tc.cuh"

namespace bsp {

// Set by a kernel whose bounded wait expired; read through sdd_tc_device_status().
static __device__ int g_sdd_status;

namespace {

using namespace tc;
using namespace mmtc;

constexpr int kStages = 3;
constexpr int kStageBytes = 32768;
constexpr int kSmem = kStages * kStageBytes + 1024;
constexpr int kThreads = 192;

struct SddTcArgs {
  void* c;
  int64_t c_sz;
  int H, Mb, Nb, block, K, nnz;
  int tiles_per_head;                          // block 64: pairs of block-rows per head
  const int32_t *row_ptr, *blk_row, *blk_col, *blk_head;
};

constexpr int kNone = 0x7fffffff;

template <typename T, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kThreads, 2)
sdd_tc_kernel(const __grid_constant__ CUtensorMap m_a, const __grid_constant__ CUtensorMap m_b, SddTcArgs a) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024 - (saddr(smem_raw) & 1023)) & 1023);
  __shared__ uint64_t bar_full[kStages], bar_empty[kStages], bar_done;
  __shared__ uint32_t tmem_slot;
  __shared__ int failed[2];
  // work of this CTA: head, first row of A, its column blocks (first column of B, or -1; two of
  // 64 columns or four of 32) and the ids of the blocks to store ([block-row][column block], -1: none)
  __shared__ int w_h, w_m0, w_n[4], w_id[4][4];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int z = blockIdx.z, block = a.block;

  if (tid == 0) {
    failed[0] = 0;
    failed[1] = kWaitBudget;
    for (int i = 0; i < 4; ++i) {
      w_n[i] = -1;
      for (int j = 0; j < 4; ++j) w_id[i][j] = -1;
    }
    if (block == 128) {
      const int e = blockIdx.x;
      w_h = a.blk_head[e];
      w_m0 = a.blk_row[e] * 128;
      w_n[0] = a.blk_col[e] * 128;
      w_n[1] = w_n[0] + 64;
      w_id[0][0] = e;
    } else {
      const int tile = blockIdx.y, g = blockIdx.x;   // the groups of a tile are neighbours in the launch: they share A in L2
      const int R = 128 / block;                      // block-rows of a tile = column blocks of a group
      const int h = tile / a.tiles_per_head, r0 = R * (tile % a.tiles_per_head);
      w_h = h;
      w_m0 = r0 * block;
      int i[4], e[4], c[4];
      for (int r = 0; r < 4; ++r) {
        i[r] = e[r] = 0;
        if (r < R && r0 + r < a.Mb) { i[r] = a.row_ptr[h * a.Mb + r0 + r]; e[r] = a.row_ptr[h * a.Mb + r0 + r + 1]; }
        c[r] = i[r] < e[r] ? a.blk_col[i[r]] : kNone;
      }
      // entries R g .. R g + R - 1 of the union of the column lists (each in column order)
      for (int n = 0; n < R * g + R; ++n) {
        const int col = min(min(c[0], c[1]), min(c[2], c[3]));
        if (col == kNone) break;
        if (n >= R * g) w_n[n - R * g] = col * block;
        for (int r = 0; r < 4; ++r)
          if (c[r] == col) {
            if (n >= R * g) w_id[r][n - R * g] = i[r];
            ++i[r];
            c[r] = i[r] < e[r] ? a.blk_col[i[r]] : kNone;
          }
      }
    }
    for (int s = 0; s < kStages; ++s) { mbar_init(&bar_full[s], 1); mbar_init(&bar_empty[s], 1); }
    mbar_init(&bar_done, 1);
    mbar_init_fence();
  }
  __syncthreads();
  if (w_n[0] < 0) return;                      // this group of columns does not exist (uniform)
  if (warp == 1) { tmem_alloc(&tmem_slot, 128); tmem_relinquish(); }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem = tmem_slot;
  const int ns = a.K / 64;
  const int h = w_h, m0 = w_m0;
  volatile int* fl = failed;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_map(&m_a); prefetch_map(&m_b);
      // a missing column block: a box past the end of B, filled with zeros
      int nb[4];
      for (int j = 0; j < 4; ++j) nb[j] = w_n[j] >= 0 ? w_n[j] : a.Nb * block;
      for (int it = 0; it < ns; ++it) {
        const int s = it % kStages, k0 = it * 64;
        if (it >= kStages && !mbar_wait(&bar_empty[s], ((it / kStages) - 1) & 1, fl)) break;
        unsigned char* sp = smem + s * kStageBytes;
        mbar_expect_tx(&bar_full[s], kStageBytes);
        if (A_MN) {                               // [k][m] in memory: 64 m x 64 k-rows per box
          tma_load_4d(sp, &m_a, &bar_full[s], m0, k0, h, z);
          tma_load_4d(sp + 8192, &m_a, &bar_full[s], m0 + 64, k0, h, z);
        } else {                                  // [m][k]: 64 k x 64 m-rows per box
          tma_load_4d(sp, &m_a, &bar_full[s], k0, m0, h, z);
          tma_load_4d(sp + 8192, &m_a, &bar_full[s], k0, m0 + 64, h, z);
        }
        if (block == 32) {                        // four column blocks of 32: 4 KB each in either form
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (B_MN) tma_load_4d(sp + 16384 + j * 4096, &m_b, &bar_full[s], nb[j], k0, h, z);
            else tma_load_4d(sp + 16384 + j * 4096, &m_b, &bar_full[s], k0, nb[j], h, z);
          }
        } else if (B_MN) {                        // [k][n]: 64 n x 64 k-rows per box
          tma_load_4d(sp + 16384, &m_b, &bar_full[s], nb[0], k0, h, z);
          tma_load_4d(sp + 16384 + 8192, &m_b, &bar_full[s], nb[1], k0, h, z);
        } else {                                  // [n][k]: 64 k x 64 n-rows per box
          tma_load_4d(sp + 16384, &m_b, &bar_full[s], k0, nb[0], h, z);
          tma_load_4d(sp + 16384 + 8192, &m_b, &bar_full[s], k0, nb[1], h, z);
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = instr_desc(128, 128, B_MN ? 1 : 0, Bf<T>::v) | (A_MN ? 1u << 15 : 0u);
      bool ok = true;
      for (int it = 0; ok && it < ns; ++it) {
        const int s = it % kStages;
        // (MN-major A: 8 KB between its two groups of 64 rows, in the leading-offset field)
        const uint32_t a_lo = A_MN ? (((saddr(smem + s * kStageBytes) & 0x3FFFF) >> 4) | (512u << 16))
                                   : desc_lo(saddr(smem + s * kStageBytes));
        // (block 32, MN-major B: groups of 32 columns in the 64-byte swizzle, 64 k-rows of 64 bytes
        // = 4 KB apart, 8-row groups of 512 bytes, 16 rows = 1 KB per K-step)
        const bool b64s = B_MN && block == 32;
        const uint32_t b_lo = B_MN ? (((saddr(smem + s * kStageBytes + 16384) & 0x3FFFF) >> 4) | ((b64s ? 256u : 512u) << 16))
                                   : desc_lo(saddr(smem + s * kStageBytes + 16384));
        const uint32_t b_hi = b64s ? ((512u >> 4) | (1u << 14) | (4u << 29)) : kDescHi;
        ok = mbar_wait(&bar_full[s], (it / kStages) & 1, fl);
        if (!ok) break;
        fence_after();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          const uint32_t acc = (it > 0 || ks > 0) ? 1u : 0u;
          const uint64_t da = desc_from_lo(a_lo + ks * (A_MN ? 128 : 2));   // per K-step: 16 rows (MN-major), 32 bytes (K-major)
          const uint64_t db = (static_cast<uint64_t>(b_hi) << 32) | (b_lo + ks * (B_MN ? (b64s ? 64 : 128) : 2));
          mma_ss(tmem, da, db, idesc, acc);
        }
        commit(&bar_empty[s]);
      }
      if (ok) commit(&bar_done);
    }
  } else {
    // ------------------------------------------------------------------ write-back
    const int row = warp * 32 + lane;
    const int rh = block == 32 ? row >> 5 : row >> 6;
    if (mbar_wait_warp(&bar_done, 0, fl)) {
      fence_after();
      const uint32_t ta = tmem + ((uint32_t)(warp * 32) << 16);
      T* cz = reinterpret_cast<T*>(a.c) + z * a.c_sz;
#pragma unroll 1
      for (int c = 0; c < 128; c += 32) {
        // block 128: one block, this thread's row of 128 columns; block 64: block [rh][c / 64];
        // block 32: block [rh][c / 32], a whole row of it
        const int id = block == 128 ? w_id[0][0] : block == 64 ? w_id[rh][c >> 6] : w_id[rh][c >> 5];
        if (id < 0) continue;                                        // uniform per warp
        uint32_t r[32];
        tmem_ld32(ta + c, r);
        tmem_ld_wait();
        T* dst = block == 128 ? cz + (int64_t)id * 16384 + row * 128 + c
                 : block == 64 ? cz + (int64_t)id * 4096 + (row & 63) * 64 + (c & 63)
                               : cz + (int64_t)id * 1024 + (row & 31) * 32;
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint4 v;
          v.x = pack2<T>(__uint_as_float(r[i]), __uint_as_float(r[i + 1]));
          v.y = pack2<T>(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
          v.z = pack2<T>(__uint_as_float(r[i + 4]), __uint_as_float(r[i + 5]));
          v.w = pack2<T>(__uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]));
          *reinterpret_cast<uint4*>(dst + i) = v;
        }
      }
    }
  }
  fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 128);
  if (tid == 0 && failed[0]) atomicExch(&g_sdd_status, 5);
}

template <typename T, bool AM, bool BM>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const SddTcArgs& a, dim3 grid, cudaStream_t st) {
  auto kern = sdd_tc_kernel<T, AM, BM>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
  if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "sdd (tcgen05): cannot reserve shared memory: %s", cudaGetErrorString(e));
  kern<<<grid, kThreads, kSmem, st>>>(ma, mb, a);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "sdd (tcgen05) launch failed: %s", cudaGetErrorString(e));
  return BSP_OK;
}

template <typename T>
int launch_t(bool am, bool bm, const CUtensorMap& ma, const CUtensorMap& mb, const SddTcArgs& a, dim3 grid, cudaStream_t st) {
  if (am) return bm ? launch<T, true, true>(ma, mb, a, grid, st) : launch<T, true, false>(ma, mb, a, grid, st);
  return bm ? launch<T, false, true>(ma, mb, a, grid, st) : launch<T, false, false>(ma, mb, a, grid, st);
}

// [Z, H, outer, inner] dense operand with unit stride on `inner`: boxes of 64 x 64, or of the
// extents given (an inner extent of 32 elements goes with the 64-byte swizzle).
int dense_map(CUtensorMap* m, const void* p, int dtype, int Z, int H, int64_t inner, int64_t outer,
              int64_t outer_stride, int64_t sh, int64_t sz, int box_inner = 64, int box_outer = 64) {
  cuuint64_t dims[4] = {(cuuint64_t)inner, (cuuint64_t)outer, (cuuint64_t)H, (cuuint64_t)Z};
  cuuint64_t strides[3] = {(cuuint64_t)outer_stride * 2, (cuuint64_t)(H > 1 ? sh : outer * outer_stride) * 2,
                           (cuuint64_t)(Z > 1 ? sz : (int64_t)H * outer * outer_stride) * 2};
  cuuint32_t box[4] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer, 1, 1};
  return encode(m, p, dtype, 4, dims, strides, box, box_inner == 32 ? 64 : 128);
}

}  // namespace

// True when sdd_tc covers the case: FP16 / BF16, block 32 / 64 / 128, K a multiple of 64, dense
// operands with one unit inner stride and 16-byte friendly addresses and strides.
bool sdd_tc_eligible(const void* a, const void* b, const void* c, int dtype, int block, int K,
                     int64_t a_sz, int64_t a_sh, int64_t a_sm, int64_t a_sk,
                     int64_t b_sz, int64_t b_sh, int64_t b_sk, int64_t b_sn, int64_t c_sz) {
  if (dtype != BSP_F16 && dtype != BSP_BF16) return false;
  if ((block != 32 && block != 64 && block != 128) || K % 64) return false;
  if ((a_sm != 1) == (a_sk != 1) || (b_sk != 1) == (b_sn != 1)) return false;
  const int64_t a_outer = a_sk == 1 ? a_sm : a_sk, b_outer = b_sk == 1 ? b_sn : b_sk;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15) return false;
  if ((a_sz | a_sh | a_outer | b_sz | b_sh | b_outer | c_sz) & 7) return false;
  if (a_sz <= 0 || a_sh <= 0 || a_outer <= 0 || b_sz <= 0 || b_sh <= 0 || b_outer <= 0) return false;   // TMA strides: no broadcast
  return true;
}

int sdd_tc(const void* a, const void* b, void* c, int dtype, int block, int Z, int K,
           int64_t a_sz, int64_t a_sh, int64_t a_sm, int64_t a_sk,
           int64_t b_sz, int64_t b_sh, int64_t b_sk, int64_t b_sn, int64_t c_sz, const Meta& m, cudaStream_t st) {
  const bool am = a_sm == 1, bm = b_sn == 1;       // MN-major: the non-k dimension is contiguous
  const int64_t M = (int64_t)m.Mb * block, N = (int64_t)m.Nb * block;
  CUtensorMap ma, mb;
  if (int rc = am ? dense_map(&ma, a, dtype, Z, m.H, M, K, a_sk, a_sh, a_sz) : dense_map(&ma, a, dtype, Z, m.H, K, M, a_sm, a_sh, a_sz)) return rc;
  // (block 32: one box per column block, 32 columns of 64 k)
  const int bn = block == 32 ? 32 : 64;
  if (int rc = bm ? dense_map(&mb, b, dtype, Z, m.H, N, K, b_sk, b_sh, b_sz, bn, 64)
                  : dense_map(&mb, b, dtype, Z, m.H, K, N, b_sn, b_sh, b_sz, 64, bn)) return rc;
  SddTcArgs p = {};
  p.c = c; p.c_sz = c_sz; p.H = m.H; p.Mb = m.Mb; p.Nb = m.Nb; p.block = block; p.K = K; p.nnz = m.nnz;
  const int R = 128 / block;                        // block-rows per tile and column blocks per group (block 32 / 64)
  p.tiles_per_head = (m.Mb + R - 1) / R;
  p.row_ptr = m.row_ptr; p.blk_row = m.blk_row; p.blk_col = m.blk_col; p.blk_head = m.blk_head;
  dim3 grid;
  if (block == 128) {
    grid = dim3(m.nnz, 1, Z);
  } else {
    // the union of R column lists has at most R * max_row entries, and never more than Nb
    const int groups = (std::min(m.Nb, R * std::max(m.max_row, 1)) + R - 1) / R;
    grid = dim3(groups, m.H * p.tiles_per_head, Z);
  }
  if (dtype == BSP_F16) return launch_t<__half>(am, bm, ma, mb, p, grid, st);
  return launch_t<__nv_bfloat16>(am, bm, ma, mb, p, grid, st);
}

// 0, or non-zero when a bounded wait inside the kernel above expired (synchronises the device).
int sdd_tc_device_status(int* out) {
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_sdd_status, sizeof(int));
  if (e == cudaSuccess && v != 0) { const int zero = 0; e = cudaMemcpyToSymbol(g_sdd_status, &zero, sizeof(int)); }   // reading clears
  if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "device status: %s", cudaGetErrorString(e));
  *out = v;
  return BSP_OK;
}

}  // namespace bsp
