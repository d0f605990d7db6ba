// Block-sparse sdd on the Blackwell tensor path for block 32, 64 and 128: tcgen05.mma with the
// accumulator in tensor memory, operands brought in by TMA.
//
// Same contract as the mma.sync kernel of sdd_impl.cuh (which replaces the launch of
// torch_blocksparse/matmul.py:354-360): every nonzero block (i, j) of the layout receives
// op(A)[rows of block-row i, :] . op(B)[:, columns of block-column j].
//
// Geometry: every MMA has M = 128 and a CTA's accumulator is 128 x 256: R = 128 / block
// block-rows by 2 R consecutive entries of the union of their column lists (block 128: two
// blocks of one row, block 64: 2 x 4, block 32: 4 x 8 candidate blocks), of which those the
// layout holds are stored.  A group whose entries fill at most half of the 256 columns runs
// with N = 128.  The reduction runs over K in stages of 64: 16 KB of A (128 m x 64 k, two TMA
// boxes of 64 x 64) and up to 32 KB of B (64 k x 256 n, one box per column block, two for a
// block of 128 with n contiguous).  Either operand may have k or its other dimension
// contiguous: k contiguous gives K-major tiles, the other case MN-major tiles (groups of 64
// rows or columns, 8 KB apart, in one descriptor; the 32 columns of a block-32 column block
// form groups of 4 KB in the 64-byte swizzle); every K-step is one 128 x N x 16 MMA.  A box
// that lies outside the tensor (block-rows past the last one) is filled with zeros; column
// blocks past the end of the union are neither loaded nor computed (N = 128) or computed on
// whatever the ring holds and not stored.
//
// Warps: 0-3 write the blocks back, 4 issues the TMA loads (one lane per box), 5 the MMAs
// (one thread).  Two CTAs per SM, two stages each.  mbarriers only; every wait is bounded
// and a wait that expires sets a device status word.
#include <algorithm>
#include "mm_tc.cuh"

namespace bsp {

// Set by a kernel whose bounded wait expired; read through sdd_tc_device_status().
static __device__ int g_sdd_status;

namespace {

using namespace tc;
using namespace mmtc;

constexpr int kStages = 2;
constexpr int kStageA = 16384, kStageB = 32768;
constexpr int kStageBytes = kStageA + kStageB;
constexpr int kSmem = kStages * kStageBytes + 1024;
constexpr int kThreads = 192;
constexpr int kTN = 256;

struct SddTcArgs {
  void* c;
  int64_t c_sz;
  int H, Mb, Nb, block, K, nnz;
  int tiles_per_head;                          // groups of R block-rows per head
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
  // work of this CTA: head, first row of A, its column blocks (first column of B, or -1), how
  // many there are, and the ids of the blocks to store ([block-row][column block], -1: none)
  __shared__ int w_h, w_m0, w_cols, w_n[8], w_id[4][8];
  __shared__ uint32_t row_mask[4][32];          // set-up: block-row r has a block in column 32 * word + bit

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int z = blockIdx.z, block = a.block;
  const int R = 128 / block, NC = 2 * R;        // block-rows of a tile, column blocks of a group

  if (tid == 0) {
    failed[0] = 0;
    failed[1] = kWaitBudget;
    for (int s = 0; s < kStages; ++s) { mbar_init(&bar_full[s], 1); mbar_init(&bar_empty[s], 1); }
    mbar_init(&bar_done, 1);
    mbar_init_fence();
  }
  if (warp == 0) {
    // The work of this CTA, found by the whole warp: entries NC g .. NC g + NC - 1 of the union
    // of the tile's column lists.  Up to 1024 block-columns the lists become bit masks (lane w
    // holds columns 32 w .. 32 w + 31 of every block-row) and positions are prefix counts of
    // set bits; beyond that lane 0 merges the lists.
    const uint32_t full = 0xffffffffu;
    if (lane < 8) {
      w_n[lane] = -1;
      for (int i = 0; i < 4; ++i) w_id[i][lane] = -1;
    }
    const int tile = blockIdx.y, g = blockIdx.x;     // the groups of a tile are neighbours in the launch: they share A in L2
    const int h = tile / a.tiles_per_head, r0 = R * (tile % a.tiles_per_head);
    if (lane == 0) { w_h = h; w_m0 = r0 * block; w_cols = 0; }
    int rs = 0, re = 0;
    if (lane < R && r0 + lane < a.Mb) { rs = a.row_ptr[h * a.Mb + r0 + lane]; re = a.row_ptr[h * a.Mb + r0 + lane + 1]; }
    __syncwarp();
    if (R == 1) {                                     // one list: its entries directly
      const int first = __shfl_sync(full, rs, 0) + NC * g, end = __shfl_sync(full, re, 0);
      if (lane < NC && first + lane < end) {
        w_n[lane] = a.blk_col[first + lane] * block;
        w_id[0][lane] = first + lane;
      }
      if (lane == 0) w_cols = max(0, min(NC, end - first));
    } else if (a.Nb <= 1024) {
#pragma unroll
      for (int r = 0; r < 4; ++r) row_mask[r][lane] = 0;
      __syncwarp();
      int start[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        start[r] = __shfl_sync(full, rs, r);
        const int end = __shfl_sync(full, re, r);
        for (int j = start[r] + lane; j < end; j += 32) {
          const int c = a.blk_col[j];
          atomicOr(&row_mask[r][c >> 5], 1u << (c & 31));
        }
      }
      __syncwarp();
      uint32_t m[4], u = 0;
      int rank0[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        m[r] = row_mask[r][lane];
        u |= m[r];
        int x = __popc(m[r]);
        const int v = x;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const int y = __shfl_up_sync(full, x, d);
          if (lane >= d) x += y;
        }
        rank0[r] = x - v;
      }
      int x = __popc(u);
      const int v = x;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int y = __shfl_up_sync(full, x, d);
        if (lane >= d) x += y;
      }
      const int total = __shfl_sync(full, x, 31);
      int q = x - v;                                  // position in the union of this lane's first column
      for (uint32_t bits = u; bits; ++q) {
        const int bit = __ffs(bits) - 1;
        bits &= bits - 1;
        const int j = q - NC * g;
        if (j < 0 || j >= NC) continue;
        w_n[j] = (lane * 32 + bit) * block;
#pragma unroll
        for (int r = 0; r < 4; ++r)
          if ((m[r] >> bit) & 1u) w_id[r][j] = start[r] + rank0[r] + __popc(m[r] & ((1u << bit) - 1u));
      }
      if (lane == 0) w_cols = max(0, min(NC, total - NC * g));
    } else if (lane == 0) {
      int i[4], e[4], c[4];
      for (int r = 0; r < 4; ++r) {
        i[r] = e[r] = 0;
        if (r < R && r0 + r < a.Mb) { i[r] = a.row_ptr[h * a.Mb + r0 + r]; e[r] = a.row_ptr[h * a.Mb + r0 + r + 1]; }
        c[r] = i[r] < e[r] ? a.blk_col[i[r]] : kNone;
      }
      int cols = 0;
      for (int n = 0; n < NC * g + NC; ++n) {
        const int col = min(min(c[0], c[1]), min(c[2], c[3]));
        if (col == kNone) break;
        if (n >= NC * g) { w_n[n - NC * g] = col * block; cols = n - NC * g + 1; }
        for (int r = 0; r < 4; ++r)
          if (c[r] == col) {
            if (n >= NC * g) w_id[r][n - NC * g] = i[r];
            ++i[r];
            c[r] = i[r] < e[r] ? a.blk_col[i[r]] : kNone;
          }
      }
      w_cols = cols;
    }
  }
  __syncthreads();
  if (w_cols == 0) return;                     // this group of columns does not exist (uniform)
  if (warp == 1) { tmem_alloc(&tmem_slot, kTN); tmem_relinquish(); }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem = tmem_slot;
  const int ns = a.K / 64;
  const int h = w_h, m0 = w_m0;
  // columns computed: 128 when the group's column blocks fill at most half of the accumulator
  const int ncomp = w_cols * block <= 128 ? 128 : 256;
  volatile int* fl = failed;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    // lanes 0-7: the boxes of B (block 128 with n contiguous: two per column block; else one per
    // column block), lanes 8 and 9: the two boxes of A
    if (lane < 10) {
      const uint32_t m10 = 0x3ffu;
      if (lane == 0) { prefetch_map(&m_a); prefetch_map(&m_b); }
      const bool split = block == 128 && B_MN;                    // a column block of 128 n-contiguous columns takes two boxes of 64
      const int nbox = split ? 2 * w_cols : w_cols;               // boxes of B that exist
      const int box_bytes = split ? 8192 : block * 128;
      const int cj = split ? lane >> 1 : lane;                    // column block of this lane's box
      const bool mine = lane < 8 && lane < nbox && (split ? lane < 4 : true);
      const int n_first = mine ? w_n[cj] + (split ? (lane & 1) * 64 : 0) : 0;
      const uint32_t tx = kStageA + nbox * box_bytes;
      int ok = 1;
      for (int it = 0; it < ns; ++it) {
        const int s = it % kStages, k0 = it * 64;
        if (it >= kStages) {
          if (lane == 0) ok = mbar_wait(&bar_empty[s], ((it / kStages) - 1) & 1, fl) ? 1 : 0;
          ok = __shfl_sync(m10, ok, 0);
          if (!ok) break;
        }
        unsigned char* sp = smem + s * kStageBytes;
        if (lane == 0) mbar_expect_tx(&bar_full[s], tx);
        __syncwarp(m10);
        if (lane >= 8) {
          const int half = lane - 8;
          if (A_MN) tma_load_4d(sp + half * 8192, &m_a, &bar_full[s], m0 + half * 64, k0, h, z);   // [k][m]: 64 m x 64 k-rows
          else tma_load_4d(sp + half * 8192, &m_a, &bar_full[s], k0, m0 + half * 64, h, z);        // [m][k]: 64 k x 64 m-rows
        } else if (mine) {
          unsigned char* bp = sp + kStageA + lane * box_bytes;
          if (B_MN) tma_load_4d(bp, &m_b, &bar_full[s], n_first, k0, h, z);                        // [k][n]
          else tma_load_4d(bp, &m_b, &bar_full[s], k0, n_first, h, z);                             // [n][k]
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = instr_desc(128, ncomp, B_MN ? 1 : 0, Bf<T>::v) | (A_MN ? 1u << 15 : 0u);
      bool ok = true;
      for (int it = 0; ok && it < ns; ++it) {
        const int s = it % kStages;
        // (MN-major A: 8 KB between its two groups of 64 rows, in the leading-offset field)
        const uint32_t a_lo = A_MN ? (((saddr(smem + s * kStageBytes) & 0x3FFFF) >> 4) | (512u << 16))
                                   : desc_lo(saddr(smem + s * kStageBytes));
        // (block 32, MN-major B: groups of 32 columns in the 64-byte swizzle, 64 k-rows of 64 bytes
        // = 4 KB apart, 8-row groups of 512 bytes, 16 rows = 1 KB per K-step)
        const bool b64s = B_MN && block == 32;
        const uint32_t b_lo = B_MN ? (((saddr(smem + s * kStageBytes + kStageA) & 0x3FFFF) >> 4) | ((b64s ? 256u : 512u) << 16))
                                   : desc_lo(saddr(smem + s * kStageBytes + kStageA));
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
    const int rh = block == 128 ? 0 : block == 64 ? row >> 6 : row >> 5;
    if (mbar_wait_warp_idle(&bar_done, 0, fl, lane)) {
      fence_after();
      const uint32_t ta = tmem + ((uint32_t)(warp * 32) << 16);
      T* cz = reinterpret_cast<T*>(a.c) + z * a.c_sz;
#pragma unroll 1
      for (int c = 0; c < ncomp; c += 32) {
        // the block this thread's 32 columns belong to: [rh][c / block]
        const int id = block == 128 ? w_id[0][c >> 7] : block == 64 ? w_id[rh][c >> 6] : w_id[rh][c >> 5];
        if (id < 0) continue;                                        // uniform per warp
        uint32_t r[32];
        tmem_ld32(ta + c, r);
        tmem_ld_wait();
        T* dst = block == 128 ? cz + (int64_t)id * 16384 + row * 128 + (c & 127)
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
  if (warp == 1) tmem_dealloc(tmem, kTN);
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
  // (one box per column block: 32, 64 or 128 columns of 64 k; with n contiguous a box holds 64
  // columns at most, so a block of 128 takes two)
  const int bn = block == 32 ? 32 : (bm || block == 64) ? 64 : 128;
  if (int rc = bm ? dense_map(&mb, b, dtype, Z, m.H, N, K, b_sk, b_sh, b_sz, bn, 64)
                  : dense_map(&mb, b, dtype, Z, m.H, K, N, b_sn, b_sh, b_sz, 64, bn)) return rc;
  SddTcArgs p = {};
  p.c = c; p.c_sz = c_sz; p.H = m.H; p.Mb = m.Mb; p.Nb = m.Nb; p.block = block; p.K = K; p.nnz = m.nnz;
  const int R = 128 / block, NC = 2 * R;            // block-rows per tile, column blocks per group
  p.tiles_per_head = (m.Mb + R - 1) / R;
  p.row_ptr = m.row_ptr; p.blk_row = m.blk_row; p.blk_col = m.blk_col; p.blk_head = m.blk_head;
  // the union of R column lists has at most R * max_row entries, and never more than Nb
  const int groups = (std::min(m.Nb, R * std::max(m.max_row, 1)) + NC - 1) / NC;
  dim3 grid(groups, m.H * p.tiles_per_head, Z);
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
