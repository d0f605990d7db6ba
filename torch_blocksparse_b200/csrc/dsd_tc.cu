// Block-sparse dsd (and, through the transposed problem, dds) on the Blackwell tensor
// path for block 32, 64 and 128: tcgen05.mma with the accumulator in tensor memory,
// operands brought in by TMA, persistent CTAs.
//
// Same contract as the mma.sync kernel of dsd_impl.cuh (which replaces the launch of
// torch_blocksparse/matmul.py:498-504, 545-551): C[rows of a block-row] = sum over the
// nonzero blocks (i, j) of that block-row of op(S)(i, j) . B[rows of block j].  The sparse
// operand is used as stored (K-major A tiles) or transposed (MN-major A tiles, lists from the
// CSC side of the metadata).
//
// Geometry: every MMA has M = 128.  A tile is 128 rows of C (one block-row for block 128, two
// for block 64, four for block 32) by TN = 256 columns (128 when the width is no multiple of
// 256).  The block-rows of a tile are walked together, in
// column order, over the UNION of their column lists; the piece of the A tile whose row has no
// block in a column is zero (a non-finite value of the dense operand in such a place turns
// into NaN where the mma.sync kernels, which skip absent blocks, give a finite result).  A
// "stage" of the operand ring covers K = 64:
//   block 128  one half of a nonzero block;
//   block 64   one column of the union;
//   block 32   two columns of the union (two sub-tiles of K = 32, 64-byte swizzle; the second
//              may be absent at the end of a tile).
// A stage holds 16 KB of A and 64 x TN elements of the dense operand.  Pieces of A that are
// zero are not loaded when the stage's piece already holds zeros (the ring is cleared once at
// the start and the loading lanes track which pieces hold a block); otherwise a TMA box that
// lies past the last block fills them with zeros.
//
// Persistent CTAs: each walks tiles blockIdx.x, blockIdx.x + gridDim.x, ... (row
// tiles fastest, so that the CTAs that run together share the dense panel in L2) with an
// operand ring that runs on across tile boundaries.  The hand-offs between the loading, issuing
// and write-back threads cost several hundred cycles per stage whatever the ring's depth (a
// kernel with every load, MMA and store taken out ran at 800-950 cycles per stage with one
// CTA per SM).  For blocks 32 and 64 two CTAs per SM, each with one accumulator and a ring of
// two stages, hide them (configuration 2: 0.89 -> 0.72 ms, block 64 on the 4096^3 case 0.97 ->
// 0.87 ms).  Block 128 is bound by the traffic from L2 into shared memory (its loads alone
// take 0.50 of its 0.65 ms) and keeps one CTA per SM with two accumulators and four stages,
// whose write-back overlaps the next tile (with unit stride along the rows of the result, the
// dds case, 0.59 against 0.71 ms).
//
// Warps: 0-3 write the result back (tensor memory -> registers -> global), 4 loads the sparse
// operand, 5 issues the MMAs (one thread), 6 loads the dense operand, 7 plans:
// it turns the tile's column lists into bit masks (the reduction side may have 1024 blocks at
// most), forms their union and writes one entry per stage (rows of the sparse operand, block
// columns of the dense one) into a double-buffered plan in shared memory, so that the loading
// threads do nothing per stage but wait, announce the bytes and issue.  mbarriers only; every
// wait is bounded (tc.cuh) and a wait that expires sets the device status word.
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

constexpr int kThreads = 256;
constexpr int kStageA = 16384;
constexpr int kFirst = 1, kLast = 2, kEnd = 4, kHalf = 8;   // stage flags
constexpr int kNone = 0x7fffffff;

// CTAS: CTAs per SM.  Two (blocks 32 and 64) have one accumulator and a short ring each; one
// (block 128) has two accumulators, so that the write-back of a tile overlaps the products of the
// next one, and a ring twice as deep.
template <int TN, int CTAS> struct Geo {
  static constexpr int kAcc = CTAS == 2 ? 1 : 2;
  static constexpr int kStageB = 64 * TN * 2;
  static constexpr int kStage = kStageA + kStageB;
  static constexpr int kStages = CTAS == 2 ? (TN == 256 ? 2 : 3) : (TN == 256 ? 4 : 6);
  static constexpr int kSmem = kStages * kStage + 1024;
};

struct DsdTcArgs {
  void* c;
  int64_t c_sz, c_sh, c_sm, c_sn;
  int H, Mb, block, rows_total, nnz_rows;   // rows_total = Mb * block; nnz_rows = nnz * block (first out-of-range row of S)
  int tiles_per_head, n_tiles, total_tiles;
  const int32_t *row_ptr, *blk_col;          // lists of a block-row of op(S): CSR of the layout, or (transposed use) its CSC
  const int32_t* blk_id;                     // storage index of every list entry (NULL: the entry's own position)
};

// D[tmem] (+)= A[smem] * B[smem] with the descriptors given as their two 32-bit words.
BSP_DEVI void mma_desc(uint32_t d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\t"
               "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
               ::"r"(d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
}
BSP_DEVI void mma_desc_acc(uint32_t d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi, uint32_t idesc) {
  asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.eq.b32 p, 0, 0;\n\t"
               "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
               ::"r"(d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc) : "memory");
}

struct Tile { int tr, nt, h, z; };
BSP_DEVI Tile tile_of(const DsdTcArgs& a, int t) {
  Tile c;
  c.tr = t % a.tiles_per_head; t /= a.tiles_per_head;
  c.nt = t % a.n_tiles; t /= a.n_tiles;
  c.h = t % a.H;
  c.z = t / a.H;
  return c;
}

// The load plan of a tile, written by the planning warp and read by the two loading warps.  One
// entry per stage (block 128: per nonzero block, i.e. two stages): words 0-7 the first row of the
// sparse operand's block for every piece of the stage's A part (piece = 4 * sub-tile + block-row;
// -1: the block-row has no block in that column), words 8 and 9 the block-column of sub-tile 0 / 1
// (-1: block 32 with an odd number of columns, last entry).  A tile with more than kChunk
// entries takes several buffers in a row.
constexpr int kChunk = 64;
struct Plan {
  int n, last;                 // entries in this buffer; 1 if the tile ends with it
  int e[kChunk][12];
};

BSP_DEVI int warp_exclusive_sum(int v, int lane, int* total) {
  int x = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int y = __shfl_up_sync(0xffffffffu, x, d);
    if (lane >= d) x += y;
  }
  *total = __shfl_sync(0xffffffffu, x, 31);
  return x - v;
}

// B_KMAJOR: the dense operand has k contiguous ([n][k] in memory); else n contiguous ([k][n]).
// C_ROWS: the result has unit stride along n (a thread writes its row with 16-byte stores);
// else unit stride along m (the transposed problem of dds: lanes write neighbouring addresses).
// A_MN: the sparse operand is used transposed: a stored block [k][m] is an MN-major A tile.
template <typename T, int TN, int CTAS, bool A_MN, bool B_KMAJOR, bool C_ROWS>
__global__ void __launch_bounds__(kThreads, CTAS)
dsd_tc_kernel(const __grid_constant__ CUtensorMap m_s, const __grid_constant__ CUtensorMap m_b, DsdTcArgs a) {
  using G = Geo<TN, CTAS>;
  constexpr int S = G::kStages;
  constexpr int kAcc = G::kAcc;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024 - (saddr(smem_raw) & 1023)) & 1023);
  __shared__ uint64_t bar_full[S], bar_empty[S], bar_acc_full[2], bar_acc_empty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int failed[2];
  __shared__ volatile int stage_flags[S];
  __shared__ Plan plan[2];
  __shared__ uint64_t bar_plan_full[2], bar_plan_empty[2];
  __shared__ uint32_t row_mask[4][32];           // planning warp: block-row r has a block in column 32 * word + bit

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int block = a.block;
  const int R = 128 / block;

  if (tid == 0) {
    failed[0] = 0;
    failed[1] = kWaitBudget;
    for (int s = 0; s < S; ++s) { mbar_init(&bar_full[s], 2); mbar_init(&bar_empty[s], 1); }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bar_acc_full[b], 1); mbar_init(&bar_acc_empty[b], 4);
      mbar_init(&bar_plan_full[b], 1); mbar_init(&bar_plan_empty[b], 2);
    }
    mbar_init_fence();
  }
  if (warp == 1) { tmem_alloc(&tmem_slot, kAcc * TN); tmem_relinquish(); }
  // the A part of every stage starts as zeros (see the loading thread)
  for (int i = tid; i < S * (kStageA / 16); i += kThreads)
    reinterpret_cast<uint4*>(smem + (i / (kStageA / 16)) * G::kStage)[i % (kStageA / 16)] = make_uint4(0, 0, 0, 0);
  fence_async_smem();
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem = tmem_slot;
  volatile int* fl = failed;

  if (warp == 7) {
    // ------------------------------------------------------------------ planning
    // The union of the tile's column lists as bit masks: lane w holds columns 32 w .. 32 w + 31
    // of every block-row (the reduction side has at most 1024 blocks).  Every lane then writes
    // the entries of its own columns: the position of a column in the union and of a block in
    // its row's list are prefix counts of set bits.
    const uint32_t full = 0xffffffffu;
    int cb = 0;
    bool ok = true;
    for (int t = blockIdx.x; ok && t < a.total_tiles; t += gridDim.x) {
      const Tile tc_ = tile_of(a, t);
      int rs = 0, re = 0;
      {
        const int br = tc_.tr * R + lane;
        if (lane < R && br < a.Mb) { rs = a.row_ptr[tc_.h * a.Mb + br]; re = a.row_ptr[tc_.h * a.Mb + br + 1]; }
      }
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
      uint32_t m[4];
      int rank0[4];                               // blocks of row r in the columns before this lane's
      uint32_t u = 0;
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        m[r] = row_mask[r][lane];
        u |= m[r];
        int tot;
        rank0[r] = warp_exclusive_sum(__popc(m[r]), lane, &tot);
      }
      int total;
      const int off = warp_exclusive_sum(__popc(u), lane, &total);
      const int n_ent = block == 32 ? (total + 1) >> 1 : total;
      const int chunks = n_ent > kChunk ? (n_ent + kChunk - 1) / kChunk : 1;
      for (int c = 0; ok && c < chunks; ++c, ++cb) {
        const int buf = cb & 1;
        if (cb >= 2) {
          int k = 1;
          if (lane == 0) k = mbar_wait(&bar_plan_empty[buf], ((cb >> 1) - 1) & 1, fl) ? 1 : 0;
          if (!__shfl_sync(full, k, 0)) { ok = false; break; }
        }
        const int lo = c * kChunk, hi = min(n_ent, lo + kChunk);
        uint32_t bits = u;
        for (int q = off; bits; ++q) {
          const int bit = __ffs(bits) - 1;
          bits &= bits - 1;
          const int e = block == 32 ? q >> 1 : q, sub = block == 32 ? q & 1 : 0;
          if (e < lo || e >= hi) continue;
          int* E = plan[buf].e[e - lo];
          E[8 + sub] = lane * 32 + bit;
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            int v = -1;
            if ((m[r] >> bit) & 1u) {
              const int idx = start[r] + rank0[r] + __popc(m[r] & ((1u << bit) - 1u));
              v = (a.blk_id ? a.blk_id[idx] : idx) * block;
            }
            E[sub * 4 + r] = v;
          }
        }
        if (lane == 0) {
          if (block == 32 && (total & 1) && hi == n_ent && hi > lo) {     // the last entry has one column only
            int* E = plan[buf].e[hi - 1 - lo];
            E[9] = -1;
            E[4] = E[5] = E[6] = E[7] = -1;
          }
          plan[buf].n = hi > lo ? hi - lo : 0;
          plan[buf].last = c == chunks - 1;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_plan_full[buf]);
      }
    }
  } else if (warp == 4) {
    // ------------------------------------------------------------------ sparse operand
    // Lanes 0-7, one per piece of a stage's A part (block 64: two pieces of 8 KB, block 32: two
    // sub-tiles of four pieces of 2 KB; block 128: lane 0, or lanes 0 and 1 for the two halves of
    // a transposed block).  A piece without a block is loaded (as zeros, from past the last
    // block) only if it held one.
    if (lane < 8) {
      const uint32_t m8 = 0xffu;
      if (lane == 0) prefetch_map(&m_s);
      uint32_t dirty = 0;                          // bit s: this lane's piece of ring slot s holds a block
      int it = 0, cb = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < a.total_tiles; t += gridDim.x) {
        const Tile tc_ = tile_of(a, t);
        int flags = kFirst, last_chunk = 0;
        do {
          const int buf = cb & 1;
          int k = 1;
          if (lane == 0) k = mbar_wait(&bar_plan_full[buf], (cb >> 1) & 1, fl) ? 1 : 0;
          if (!__shfl_sync(m8, k, 0)) { ok = false; break; }
          __syncwarp(m8);                              // lane 0 has acquired the plan; the other lanes read it after this
          const int n = plan[buf].n;
          last_chunk = plan[buf].last;
          for (int e = 0; ok && e < n; ++e) {
            const int* E = plan[buf].e[e];
            const int mine = E[lane];
            const bool half = block == 32 && E[9] < 0;
            const bool last = last_chunk && e == n - 1;
            const int reps = block == 128 ? 2 : 1;
            for (int kh = 0; kh < reps; ++kh) {
              const int s = it % S;
              if (it >= S) {
                // (every lane waits itself: cheaper than one waiting lane and a shuffle)
                if (!__all_sync(m8, mbar_wait(&bar_empty[s], ((it / S) - 1) & 1, fl))) { ok = false; break; }
              }
              unsigned char* sp = smem + s * G::kStage;
              if (block == 128) {
                if (lane == 0) {
                  stage_flags[s] = flags | ((last && kh) ? kLast : 0);
                  mbar_expect_tx(&bar_full[s], kStageA);
                }
                __syncwarp(m8);
                const int row = __shfl_sync(m8, mine, 0);
                if (A_MN) {                          // rows kh * 64 .. of the stored block, its two halves of 64 columns
                  if (lane < 2) tma_load_3d(sp + lane * 8192, &m_s, &bar_full[s], lane * 64, row + kh * 64, tc_.z);
                } else if (lane == 0) {
                  tma_load_3d(sp, &m_s, &bar_full[s], kh * 64, row, tc_.z);
                }
              } else {
                const bool exists = block == 64 ? lane < 2 : !(half && lane >= 4);
                bool ld = false;
                if (exists) {
                  if (mine >= 0) { ld = true; dirty |= 1u << s; }
                  else if (dirty & (1u << s)) { ld = true; dirty &= ~(1u << s); }
                }
                const int piece = block == 64 ? 8192 : 2048;
                const int nld = __popc(__ballot_sync(m8, ld));
                if (lane == 0) {
                  stage_flags[s] = flags | (last ? kLast : 0) | (half ? kHalf : 0);
                  mbar_expect_tx(&bar_full[s], nld * piece);
                }
                __syncwarp(m8);
                if (ld)
                  tma_load_3d(sp + (block == 64 ? lane * 8192 : (lane >> 2) * 8192 + (lane & 3) * 2048), &m_s, &bar_full[s], 0,
                              mine >= 0 ? mine : a.nnz_rows, tc_.z);
              }
              flags = 0;
              ++it;
            }
          }
          __syncwarp(m8);
          if (lane == 0) mbar_arrive(&bar_plan_empty[buf]);
          ++cb;
        } while (ok && !last_chunk);
      }
      if (ok && lane == 0) {                                     // tells the issuing thread that nothing follows
        const int s = it % S;
        if (it < S || mbar_wait(&bar_empty[s], ((it / S) - 1) & 1, fl)) {
          stage_flags[s] = kEnd;
          mbar_arrive(&bar_full[s]);
        }
      }
    }
  } else if (warp == 6) {
    // ------------------------------------------------------------------ dense operand
    // k contiguous: one box of TN rows; n contiguous: one box of 64 columns per lane (the groups
    // of 64 columns of the MN-major tile), issued together.  Lane 0 announces the bytes.
    constexpr int NG = B_KMAJOR ? 1 : TN / 64;
    if (lane < NG) {
      constexpr uint32_t mg = (1u << NG) - 1u;
      if (lane == 0) prefetch_map(&m_b);
      int it = 0, cb = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < a.total_tiles; t += gridDim.x) {
        const Tile tc_ = tile_of(a, t);
        const int n0 = tc_.nt * TN;
        int last_chunk = 0;
        do {
          const int buf = cb & 1;
          int k = 1;
          if (lane == 0) k = mbar_wait(&bar_plan_full[buf], (cb >> 1) & 1, fl) ? 1 : 0;
          if (NG > 1) { k = __shfl_sync(mg, k, 0); __syncwarp(mg); }
          if (!k) { ok = false; break; }
          const int n = plan[buf].n;
          last_chunk = plan[buf].last;
          for (int e = 0; ok && e < n; ++e) {
            const int c0 = plan[buf].e[e][8], c1 = plan[buf].e[e][9];
            const int reps = block == 128 ? 2 : 1;
            for (int kh = 0; kh < reps; ++kh) {
              const int s = it % S;
              if (it >= S) {
                k = mbar_wait(&bar_empty[s], ((it / S) - 1) & 1, fl) ? 1 : 0;
                if (NG > 1) k = __all_sync(mg, k);
                if (!k) { ok = false; break; }
              }
              unsigned char* bp = smem + s * G::kStage + kStageA;
              const bool two = block == 32 && c1 >= 0;
              if (lane == 0) mbar_expect_tx(&bar_full[s], (block == 32 && !two) ? G::kStageB / 2 : G::kStageB);
              if (NG > 1) __syncwarp(mg);
              if (block == 32) {
                if (B_KMAJOR) {
                  tma_load_4d(bp, &m_b, &bar_full[s], c0 * 32, n0, tc_.h, tc_.z);
                  if (two) tma_load_4d(bp + G::kStageB / 2, &m_b, &bar_full[s], c1 * 32, n0, tc_.h, tc_.z);
                } else {                                  // groups of 32 k-rows x 128 bytes: 4 KB apart
                  tma_load_4d(bp + lane * 4096, &m_b, &bar_full[s], n0 + lane * 64, c0 * 32, tc_.h, tc_.z);
                  if (two) tma_load_4d(bp + G::kStageB / 2 + lane * 4096, &m_b, &bar_full[s], n0 + lane * 64, c1 * 32, tc_.h, tc_.z);
                }
              } else {
                const int krow = block == 128 ? c0 * 128 + kh * 64 : c0 * 64;
                if (B_KMAJOR) tma_load_4d(bp, &m_b, &bar_full[s], krow, n0, tc_.h, tc_.z);
                else tma_load_4d(bp + lane * 8192, &m_b, &bar_full[s], n0 + lane * 64, krow, tc_.h, tc_.z);
              }
              ++it;
            }
          }
          if (NG > 1) __syncwarp(mg);
          if (lane == 0) mbar_arrive(&bar_plan_empty[buf]);
          ++cb;
        } while (ok && !last_chunk);
      }
      if (ok && lane == 0) {
        const int s = it % S;
        if (it < S || mbar_wait(&bar_empty[s], ((it / S) - 1) & 1, fl)) mbar_arrive(&bar_full[s]);
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = instr_desc(128, TN, B_KMAJOR ? 0 : 1, Bf<T>::v) | (A_MN ? 1u << 15 : 0u);
      // Descriptors.  Blocks 64 / 128: 128-byte swizzle, K-major operands advance 32 bytes per
      // K-step, MN-major ones 16 rows of 128 bytes; the groups of 64 columns (rows of A) of an
      // MN-major operand lie 8 KB apart.  Block 32: the sparse operand and a K-major dense
      // operand use the 64-byte swizzle (8-row groups of 512 bytes; an MN-major A has its
      // groups of 32 rows 2 KB apart and advances 16 rows of 64 bytes per K-step); an MN-major
      // dense sub-tile has 32 k-rows, so its groups of 64 columns lie 4 KB apart.
      constexpr uint32_t kHi64 = (512u >> 4) | (1u << 14) | (4u << 29);
      const bool b32 = block == 32;
      const uint32_t a_hi = b32 ? kHi64 : kDescHi;
      const uint32_t b_hi = (b32 && B_KMAJOR) ? kHi64 : kDescHi;
      const uint32_t a_lbo = A_MN ? ((b32 ? 2048u : 8192u) >> 4) << 16 : 1u << 16;
      const uint32_t b_lbo = B_KMAJOR ? 1u << 16 : ((b32 ? 4096u : 8192u) >> 4) << 16;
      const uint32_t a_step = A_MN ? (b32 ? 64u : 128u) : 2u;
      const uint32_t b_step = B_KMAJOR ? 2u : 128u;
      const uint32_t sb = saddr(smem) >> 4;
      int tiles = 0;
      uint32_t d = tmem, ph = 0;
      bool run = true;
      // one pass of the loop body per ring slot, so that every descriptor is a constant offset from `sb`
      while (run) {
#pragma unroll
        for (int s = 0; s < S; ++s) {
          if (!mbar_wait(&bar_full[s], ph, fl)) { run = false; break; }
          fence_after();
          const int f = stage_flags[s];
          if (f & kEnd) { run = false; break; }
          if (f & kFirst) {
            const int buf = tiles % kAcc;
            if (tiles >= kAcc && !mbar_wait(&bar_acc_empty[buf], ((tiles / kAcc) - 1) & 1, fl)) { run = false; break; }
            fence_after();
            d = tmem + buf * TN;
            ++tiles;
          }
          const uint32_t a0 = ((sb + ((s * G::kStage) >> 4)) & 0x3FFFu) | a_lbo;
          const uint32_t b0 = ((sb + ((s * G::kStage + kStageA) >> 4)) & 0x3FFFu) | b_lbo;
          {
            if (!b32) {
              mma_desc(d, a0, a_hi, b0, b_hi, idesc, (f & kFirst) ? 0u : 1u);
              mma_desc_acc(d, a0 + a_step, a_hi, b0 + b_step, b_hi, idesc);
              mma_desc_acc(d, a0 + 2 * a_step, a_hi, b0 + 2 * b_step, b_hi, idesc);
              mma_desc_acc(d, a0 + 3 * a_step, a_hi, b0 + 3 * b_step, b_hi, idesc);
            } else {
              // K-steps 2, 3 belong to the second sub-tile (8 KB further in A, half a stage further in B)
              mma_desc(d, a0, a_hi, b0, b_hi, idesc, (f & kFirst) ? 0u : 1u);
              mma_desc_acc(d, a0 + a_step, a_hi, b0 + b_step, b_hi, idesc);
              if (!(f & kHalf)) {
                const uint32_t a1 = a0 + (8192u >> 4), b1 = b0 + ((uint32_t)(G::kStageB / 2) >> 4);
                mma_desc_acc(d, a1, a_hi, b1, b_hi, idesc);
                mma_desc_acc(d, a1 + a_step, a_hi, b1 + b_step, b_hi, idesc);
              }
            }
          }
          commit(&bar_empty[s]);                                    // the stage is free once these MMAs have read it
          if (f & kLast) commit(&bar_acc_full[(tiles - 1) % kAcc]);
        }
        ph ^= 1;
      }
    }
  } else if (warp < 4) {
    // ------------------------------------------------------------------ write-back
    const int row = warp * 32 + lane;
    int tiles = 0;
    bool ok = true;
    for (int t = blockIdx.x; ok && t < a.total_tiles; t += gridDim.x) {
      const Tile tc_ = tile_of(a, t);
      const int br0 = tc_.tr * R;
      const int br1 = min(br0 + R, a.Mb);
      const bool any = a.row_ptr[tc_.h * a.Mb + br1] > a.row_ptr[tc_.h * a.Mb + br0];
      const int grow = tc_.tr * 128 + row;
      const bool row_ok = grow < a.rows_total;
      T* crow = reinterpret_cast<T*>(a.c) + tc_.z * a.c_sz + tc_.h * a.c_sh + (int64_t)grow * a.c_sm +
                (int64_t)(tc_.nt * TN) * a.c_sn;
      const int buf = tiles % kAcc;
      if (any) {
        ok = mbar_wait_warp_idle(&bar_acc_full[buf], (tiles / kAcc) & 1, fl, lane);
        if (!ok) break;
        fence_after();
      }
      const uint32_t ta = tmem + buf * TN + ((uint32_t)(warp * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < TN; c += 32) {
        uint32_t r[32];
        if (any) {
          tmem_ld32(ta + c, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;                   // block-rows without blocks: zeros, as the reference gives
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
      if (any) {
        fence_before();
        warp_arrive(&bar_acc_empty[buf], lane);
        ++tiles;
      }
    }
  }
  fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, kAcc * TN);
  if (tid == 0 && failed[0]) atomicExch(&g_dsd_status, 4);
}

template <typename T, int TN, int CTAS, bool AM, bool BK, bool CR>
int launch(const CUtensorMap& ms, const CUtensorMap& mb, const DsdTcArgs& a, int sms, cudaStream_t st) {
  auto kern = dsd_tc_kernel<T, TN, CTAS, AM, BK, CR>;
  constexpr int smem = Geo<TN, CTAS>::kSmem;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "dsd (tcgen05): cannot reserve shared memory: %s", cudaGetErrorString(e));
  const int grid = a.total_tiles < CTAS * sms ? a.total_tiles : CTAS * sms;
  kern<<<grid, kThreads, smem, st>>>(ms, mb, a);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "dsd (tcgen05) launch failed: %s", cudaGetErrorString(e));
  return BSP_OK;
}

template <typename T, int TN, int CTAS, bool AM>
int launch_a(bool bk, bool cr, const CUtensorMap& ms, const CUtensorMap& mb, const DsdTcArgs& a, int sms, cudaStream_t st) {
  if (bk) return cr ? launch<T, TN, CTAS, AM, true, true>(ms, mb, a, sms, st) : launch<T, TN, CTAS, AM, true, false>(ms, mb, a, sms, st);
  return cr ? launch<T, TN, CTAS, AM, false, true>(ms, mb, a, sms, st) : launch<T, TN, CTAS, AM, false, false>(ms, mb, a, sms, st);
}

template <typename T, int TN>
int launch_t(bool am, bool bk, bool cr, const CUtensorMap& ms, const CUtensorMap& mb, const DsdTcArgs& a, int sms, cudaStream_t st) {
  if (a.block == 128)
    return am ? launch_a<T, TN, 1, true>(bk, cr, ms, mb, a, sms, st) : launch_a<T, TN, 1, false>(bk, cr, ms, mb, a, sms, st);
  return am ? launch_a<T, TN, 2, true>(bk, cr, ms, mb, a, sms, st) : launch_a<T, TN, 2, false>(bk, cr, ms, mb, a, sms, st);
}

// Number of SMs of the current device (one persistent CTA each).
int sm_count() {
  static thread_local int cached_dev = -1, cached = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (dev != cached_dev) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    cached = n;
    cached_dev = dev;
  }
  return cached;
}

}  // namespace

// True when dsd_tc covers the case: FP16 / BF16, block 32 / 64 / 128, N a multiple of 128, both dense tensors with
// one unit inner stride and 16-byte friendly addresses and strides.
bool dsd_tc_eligible(const void* s, const void* b, const void* c, int dtype, int block, int N, int trans_s, int64_t s_sz,
                     int64_t b_sz, int64_t b_sh, int64_t b_sk, int64_t b_sn,
                     int64_t c_sz, int64_t c_sh, int64_t c_sm, int64_t c_sn) {
  if (dtype != BSP_F16 && dtype != BSP_BF16) return false;
  if ((block != 32 && block != 64 && block != 128) || N % 128) return false;
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
  const int TN = N % 256 == 0 ? 256 : 128;
  // op(S) has the layout's rows (and walks its CSR) or, transposed, its columns (CSC)
  const int out_b = trans_s ? m.Nb : m.Mb, red_b = trans_s ? m.Mb : m.Nb;
  const int64_t ktot = (int64_t)red_b * block;
  const int kbox = block == 32 ? 32 : 64;                  // k extent of one load of the dense operand
  const int swz = block == 32 ? 64 : 128;
  CUtensorMap ms, mb;
  {
    cuuint64_t dims[3] = {(cuuint64_t)block, (cuuint64_t)m.nnz * block, (cuuint64_t)Z};
    cuuint64_t strides[2] = {(cuuint64_t)block * 2, (cuuint64_t)(Z > 1 ? s_sz : (int64_t)m.nnz * block * block) * 2};
    cuuint32_t box[3] = {(cuuint32_t)(block == 32 ? 32 : 64),
                         (cuuint32_t)(block == 32 ? 32 : (block == 128 && !trans_s) ? 128 : 64), 1};
    if (int rc = encode(&ms, s, dtype, 3, dims, strides, box, swz)) return rc;
  }
  const int64_t outer_n = bk ? b_sn : b_sk;                // stride between rows of the dense operand in memory
  const int64_t sh = m.H > 1 ? b_sh : (bk ? N : ktot) * outer_n;
  if (bk) {                                                // [n][k]: boxes of TN rows of kbox elements
    cuuint64_t dims[4] = {(cuuint64_t)ktot, (cuuint64_t)N, (cuuint64_t)m.H, (cuuint64_t)Z};
    cuuint64_t strides[3] = {(cuuint64_t)outer_n * 2, (cuuint64_t)sh * 2, (cuuint64_t)(Z > 1 ? b_sz : (int64_t)m.H * sh) * 2};
    cuuint32_t box[4] = {(cuuint32_t)kbox, (cuuint32_t)TN, 1, 1};
    if (int rc = encode(&mb, b, dtype, 4, dims, strides, box, swz)) return rc;
  } else {                                                 // [k][n]: boxes of 64 columns x kbox rows, one per group of 64 columns
    cuuint64_t dims[4] = {(cuuint64_t)N, (cuuint64_t)ktot, (cuuint64_t)m.H, (cuuint64_t)Z};
    cuuint64_t strides[3] = {(cuuint64_t)outer_n * 2, (cuuint64_t)sh * 2, (cuuint64_t)(Z > 1 ? b_sz : (int64_t)m.H * sh) * 2};
    cuuint32_t box[4] = {64, (cuuint32_t)kbox, 1, 1};
    if (int rc = encode(&mb, b, dtype, 4, dims, strides, box, 128)) return rc;
  }
  DsdTcArgs a = {};
  a.c = c; a.c_sz = c_sz; a.c_sh = c_sh; a.c_sm = c_sm; a.c_sn = c_sn;
  a.H = m.H; a.Mb = out_b; a.block = block; a.rows_total = out_b * block; a.nnz_rows = m.nnz * block;
  a.tiles_per_head = (out_b * block + 127) / 128;
  a.n_tiles = N / TN;
  const int64_t total = (int64_t)Z * m.H * a.tiles_per_head * a.n_tiles;
  if (total > 0x7fffffff) return fail(BSP_ERR_INVALID, "dsd: too many tiles");
  a.total_tiles = (int)total;
  if (trans_s) { a.row_ptr = m.col_ptr; a.blk_col = m.col_row; a.blk_id = m.col_bid; }
  else { a.row_ptr = m.row_ptr; a.blk_col = m.blk_col; a.blk_id = nullptr; }
  const int sms = sm_count();
  if (sms <= 0) return fail(BSP_ERR_CUDA, "dsd (tcgen05): cannot query the device");
  if (dtype == BSP_F16)
    return TN == 256 ? launch_t<__half, 256>(trans_s != 0, bk, cr, ms, mb, a, sms, st)
                     : launch_t<__half, 128>(trans_s != 0, bk, cr, ms, mb, a, sms, st);
  return TN == 256 ? launch_t<__nv_bfloat16, 256>(trans_s != 0, bk, cr, ms, mb, a, sms, st)
                   : launch_t<__nv_bfloat16, 128>(trans_s != 0, bk, cr, ms, mb, a, sms, st);
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
