// Fused block-sparse self-attention on the Blackwell tensor path: tcgen05.mma
// with accumulators in tensor memory, operands brought in by TMA.
//
// Same contract as the mma.sync kernels of attn_impl.cuh (which replace the
// sdd -> softmax -> dsd chain of
// torch_blocksparse/deepspeedsparseselfattention.py:157-166 and its backward);
// this path covers head dimension 64 and 128, FP16 / BF16, without rpe and
// attention mask; a key-padding mask is a per-key bias here.  Blocks 64 and
// 128 map onto its tiles directly; blocks 16 and 32 run on the lists of the
// layout coarsened to 64, with the 16 x 16 pieces that no block covers masked
// out of the scores.
//
// Geometry: every MMA has M = 128.  A CTA owns a tile of 128 rows of the
// "outer" operand(s), resident in shared memory, made of two 64-row chunks (one
// block-row when block = 128, a pair of block-rows when block = 64, see
// bsp_attn_tiles_build), and walks the tile's list of 64-row "inner" chunks:
//
//   forward   outer Q            inner K, V     S = Q K^T;  P = 2^(S c - m);  O += P V
//   dQ        outer Q, dO        inner K, V     S = Q K^T, dP = dO V^T;  dS = P (dP - delta) scale;  dQ += dS K
//   dK / dV   outer K, V         inner Q, dO    S^T = K Q^T, dP^T = V dO^T;  dV += P^T dO,  dK += dS^T Q
//
// Scores live in tensor memory, in two buffers where the columns allow it (the
// tensor core then computes the scores of chunk t+1 while the compute warps turn
// chunk t into P / dS); P / dS are written back (16-bit, packed) over the scores
// they came from and feed the accumulating products as the A operand straight
// from tensor memory.  Two threads share a tile row, 32 columns of a chunk each;
// in the forward each keeps its own running maximum, sum and O accumulator (the
// two halves of a chunk are two K-slices of the P V product) and the halves are
// merged when the tile is done.  For block = 64 a 2-bit mask per chunk says
// which half of the tile owns the block; the other half contributes zeros.
// Where tensor memory has columns to spare the packed operands get columns of
// their own, so that the score columns are free again as soon as they have been
// read (Cfg::ER, Cfg::ER2).
//
// Warp roles: eight compute warps and two issuing warps (one thread each): one
// issues the score products, the other the accumulating products and the TMA
// loads of the ring of inner chunks.  They talk through mbarriers only (one
// arrival per warp); every wait is bounded (tc.cuh) and a wait that expires
// sets the device status word.
#include <atomic>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "common.h"
#include "tc.cuh"
#include "tile.cuh"

namespace bsp {

// Relative position bias [Z or 1, H, L, L] (rpe_sz == 0: no batch dimension) and attention mask
// [L, L] of a call, as the tcgen05 kernels take them: am_mode 1 = added, 2 = 'mul'.
struct XtHost { const void* rpe; int64_t rpe_sz, rpe_sh, rpe_sr; const void* am; int64_t am_sr; int am_mode; };

// Set by a kernel whose bounded wait expired; read by bsp_device_status().
static __device__ int g_tc_status;


namespace {

using namespace tc;

constexpr float kLog2eT = 1.4426950408889634f;
constexpr float kNegInfT = -__builtin_huge_valf();
constexpr int FWD = 0, DQ = 1, DKV = 2;

struct TcArgs {
  void* out0; void* out1;             // FWD: O | DQ: dQ | DKV: dK, dV
  float* lse_out;                     // FWD
  const float* lse; const float* delta;   // backward
  int64_t o_sz, o_sh, o_sr;           // strides of O (FWD); gradients are contiguous [Z, H, L, D]
  int Z, H, L, tiles_per_head;
  float scale, scale_log2;
  const int32_t *c01, *ptr, *chunk, *mask, *sub, *order;
  int fine;                            // the layout's blocks are smaller than 64: pieces of a position may be absent
  int causal;                          // key j is visible to query i only for j <= i (handled by the FINE instantiation)
  const void* kpm; int64_t kpm_sz; int kpm_mul;   // key-padding mask [Z, L] (KPM variants), 'mul' mode flag
  int has_rpe, rpe_z, am_mode;         // XT variants: rpe present, rpe has a batch dimension, attention mask absent (0) / added (1) / 'mul' (2)
  int wait_budget;                     // attempts a bounded wait may make
  int skip_chunk;                      // test hook: the loads of this chunk of every tile are not issued (-1: none)
};

template <typename T> BSP_DEVI uint32_t pack16(float a, float b);
template <> BSP_DEVI uint32_t pack16<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> BSP_DEVI uint32_t pack16<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <typename T> BSP_DEVI float2 unpack16(uint32_t v);
template <> BSP_DEVI float2 unpack16<__half>(uint32_t v) { return __half22float2(*reinterpret_cast<__half2*>(&v)); }
template <> BSP_DEVI float2 unpack16<__nv_bfloat16>(uint32_t v) {
  return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}
// Key-padding mask values -> additive terms in the base-2 domain: 'add' mode adds the value,
// 'mul' mode turns a zero into -inf and anything else into 0 (softmax.py:104-110 of the reference).
BSP_DEVI float kpm_term(float v, int mul) { return mul ? (v == 0.f ? kNegInfT : 0.f) : v * kLog2eT; }
template <typename T>
BSP_DEVI void kpm_terms8(const unsigned char* p, int mul, float (&b)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = unpack16<T>(w[i]);
    b[2 * i] = kpm_term(f.x, mul);
    b[2 * i + 1] = kpm_term(f.y, mul);
  }
}
// Relative position bias and attention mask (XT variants).  Their 64 x 64 pieces for a chunk
// travel with it: per half of the tile one box of rpe at `xt` and one of the mask 16 KB further
// (at `xt` itself when there is no rpe),
// rows of 128 bytes, 16-byte units swizzled by the row as TMA writes them.  Rows of a box are
// query rows, columns key columns.  The terms are added in the base-2 domain; a 'mul' mask
// turns a zero into -inf and anything else into 0 (softmax.py:104-110 of the reference).
BSP_DEVI uint32_t xt_off(int half, int row, int col) {
  return (uint32_t)(half * 8192 + row * 128 + ((((col >> 3) ^ (row & 7)) << 4) | ((col & 7) << 1)));
}
// Eight consecutive columns (one 16-byte unit `unit`) of query row `row`: b[i] += terms.
template <typename T>
BSP_DEVI void xt_add8(const unsigned char* xt, const int has_rpe, const int am_mode, int half, int row, int unit, float (&b)[8]) {
  const uint32_t off = (uint32_t)(half * 8192 + row * 128 + ((unit ^ (row & 7)) << 4));
  if (has_rpe) {
    const uint4 raw = *reinterpret_cast<const uint4*>(xt + off);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = unpack16<T>(w[i]);
      b[2 * i] = fmaf(f.x, kLog2eT, b[2 * i]);
      b[2 * i + 1] = fmaf(f.y, kLog2eT, b[2 * i + 1]);
    }
  }
  if (am_mode) {
    const uint4 raw = *reinterpret_cast<const uint4*>(xt + (has_rpe ? 16384 : 0) + off);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = unpack16<T>(w[i]);
      if (am_mode == 2) {
        if (f.x == 0.f) b[2 * i] = kNegInfT;
        if (f.y == 0.f) b[2 * i + 1] = kNegInfT;
      } else {
        b[2 * i] = fmaf(f.x, kLog2eT, b[2 * i]);
        b[2 * i + 1] = fmaf(f.y, kLog2eT, b[2 * i + 1]);
      }
    }
  }
}
// The term of one element (query row `row`, key column `col` of the box of `half`).
template <typename T>
BSP_DEVI float xt_term(const unsigned char* xt, const int has_rpe, const int am_mode, int half, int row, int col) {
  const uint32_t off = xt_off(half, row, col);
  float t = 0.f;
  if (has_rpe) t = static_cast<float>(*reinterpret_cast<const T*>(xt + off)) * kLog2eT;
  if (am_mode) {
    const float m = static_cast<float>(*reinterpret_cast<const T*>(xt + (has_rpe ? 16384 : 0) + off));
    t = am_mode == 2 ? (m == 0.f ? kNegInfT : t) : fmaf(m, kLog2eT, t);
  }
  return t;
}
// Which of this thread's two groups of 16 columns of a chunk exist (bit 0, bit 1)?  `sub` holds,
// per half of the tile, 16 bits: bit 4 a + b for the piece of row group a and column group b (of
// 16 each) of the 64 x 64 position; all ones for blocks 64 and 128, partly zero for smaller
// blocks.  0 when the half's block is absent.
BSP_DEVI int chunk_pieces(int mask, int sub, int half, int trow, int chalf) {
  if (!((mask >> half) & 1)) return 0;
  return (sub >> (16 * half + 4 * ((trow & 63) >> 4) + 2 * chalf)) & 3;
}
constexpr uint32_t kNegInfBits = 0xff800000u;
// Scores of absent pieces become -inf: their probabilities are exactly zero.
BSP_DEVI void mask_pieces(uint32_t (&s)[32], int pieces) {
  if (!(pieces & 1)) {
#pragma unroll
    for (int i = 0; i < 16; ++i) s[i] = kNegInfBits;
  }
  if (!(pieces & 2)) {
#pragma unroll
    for (int i = 16; i < 32; ++i) s[i] = kNegInfBits;
  }
}
// Causal mask on N score registers: column col0 + i against this thread's row.  Forward and dQ
// (rows are queries, columns keys): a key after the query is hidden; dK / dV (rows are keys,
// columns queries): a query before the key does not see it.
template <int N, bool ROWS_ARE_KEYS>
BSP_DEVI void mask_causal(uint32_t (&s)[N], int col0, int row) {
  if (ROWS_ARE_KEYS ? (col0 >= row) : (col0 + N - 1 <= row)) return;   // nothing hidden in this stretch
#pragma unroll
  for (int i = 0; i < N; ++i)
    if (ROWS_ARE_KEYS ? (col0 + i < row) : (col0 + i > row)) s[i] = kNegInfBits;
}
// ---- packed FP32 arithmetic (two values per instruction on sm_100)
BSP_DEVI float2 f2(float a, float b) { return make_float2(a, b); }
BSP_DEVI float2 u2f(uint32_t a, uint32_t b) { return make_float2(__uint_as_float(a), __uint_as_float(b)); }
BSP_DEVI float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
// Maximum of 32 score registers with three-input maxima.
BSP_DEVI float max32(const uint32_t (&s)[32]) {
  float m0 = max3(__uint_as_float(s[0]), __uint_as_float(s[1]), __uint_as_float(s[2]));
  float m1 = max3(__uint_as_float(s[3]), __uint_as_float(s[4]), __uint_as_float(s[5]));
  float m2 = max3(__uint_as_float(s[6]), __uint_as_float(s[7]), __uint_as_float(s[8]));
  float m3 = max3(__uint_as_float(s[9]), __uint_as_float(s[10]), __uint_as_float(s[11]));
#pragma unroll
  for (int i = 12; i < 28; i += 8) {
    m0 = max3(m0, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
    m1 = max3(m1, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
    m2 = max3(m2, __uint_as_float(s[i + 4]), __uint_as_float(s[i + 5]));
    m3 = max3(m3, __uint_as_float(s[i + 6]), __uint_as_float(s[i + 7]));
  }
  m0 = max3(m0, __uint_as_float(s[28]), __uint_as_float(s[29]));
  m1 = max3(m1, __uint_as_float(s[30]), __uint_as_float(s[31]));
  return fmaxf(max3(m0, m1, m2), m3);
}
// The exponentials of a pair on the special-function unit; y is the exponent (SIGN = 1) or its
// negative (SIGN = -1: the negation folds into the instruction's operand).  A cubic on the FMA
// pipe for a share of the pairs was measured and lost: in an isolated loop the best mix gave
// 17.0 instead of 13.9 exponentials per clock and SM, inside these kernels every share was slower.
template <int SIGN>
BSP_DEVI float2 exp2_pair(float2 y) {
  return f2(fast_exp2(SIGN > 0 ? y.x : -y.x), fast_exp2(SIGN > 0 ? y.y : -y.y));
}

template <typename T> struct IsBf16 { static constexpr int v = 0; };
template <> struct IsBf16<__nv_bfloat16> { static constexpr int v = 1; };

template <int D, int MODE, bool KPM = false, int XT = 0> struct Cfg {
  static constexpr int ATOMS = D / 64;                         // 64-element (128-byte) column groups
  static constexpr int NRES = MODE == FWD ? 1 : 2;             // resident 128-row operands
  static constexpr int NC = 8;                                 // compute warps: two threads per tile row
  static constexpr int NT = (NC + 2) * 32;                     // + loader / score issuer, accumulate issuer
  static constexpr int RES_BYTES = ATOMS * 128 * 128;
  static constexpr int CH_BYTES = ATOMS * 64 * 128;
  // A key-padding mask is a bias per key: per column of the scores in the forward and in dQ
  // (64 values travel with every chunk), per row in dK/dV (read once per tile).
  static constexpr bool BIAS = KPM && MODE != DKV;
  // XT: how many of {relative position bias, attention mask} are read (0, 1, 2); their 64 x 64
  // pieces for the chunk (one box per half of the tile and tensor) travel with it, 16 KB per
  // stage and tensor.  With both the kernel runs with one CTA per SM; with one, the forward and
  // dQ run two CTAs per SM with two stages each at head dimension 64 (forward 0.80 -> 0.50 ms,
  // dQ 0.78 -> 0.54 ms on configuration 4 at Z=4 with rpe), dK/dV stays with one CTA and four
  // stages (0.97 against 1.02 ms).
  static constexpr int XT_OFF = 2 * CH_BYTES + 1024;
  static constexpr int STAGE = 2 * CH_BYTES + ((MODE == DKV || BIAS || XT) ? 1024 : 0) + XT * 2 * 8192;   // + lse / delta, or the bias, of the chunk
  static constexpr int TAIL_BYTES = MODE == DKV ? 512 : (BIAS ? 128 : 0);
  // score buffers in tensor memory: two (scores of the next chunk are computed while this
  // one is consumed) where the columns allow it with two CTAs per SM, else one
  static constexpr int NBUF = MODE == FWD ? 2 : (D == 64 ? 1 : 2);
  static constexpr bool XT1_PAIR = XT == 1 && D == 64 && MODE != DKV;
  static constexpr int NSTAGE = XT == 2 ? (D == 64 ? (MODE == FWD ? 4 : 3) : 2)
                                : XT == 1 ? (D == 64 ? (XT1_PAIR ? 2 : 4) : 3)
                                          : ((MODE != FWD && D == 128) ? 3 : 4);
  static constexpr int SMEM = NRES * RES_BYTES + NSTAGE * STAGE + 1024;
  static constexpr int SCORE_COLS = MODE == FWD ? 64 : 128;    // per buffer: S (and dP)
  // Early release (dQ at head_dim 64): the packed dS operand of the accumulating product gets
  // its own double-buffered columns instead of overwriting the scores, so the score buffer is
  // free as soon as the compute threads have read it and the scores of the next chunk are
  // computed during the exponentials of this one.
  static constexpr bool ER = MODE == DQ && D == 64;
  // dK/dV at head_dim 64 has no spare columns.  There the packed P^T and dS^T both go over
  // dP^T's columns (a thread's 32 columns of dP^T hold its 16 + 16 packed columns), so S^T's
  // columns are released after the read and only dP^T waits for the accumulation.
  static constexpr bool ER2 = MODE == DKV && D == 64;
  static constexpr int PK_BASE = NBUF * SCORE_COLS;
  static constexpr int ACC_BASE = PK_BASE + (ER ? 64 : 0);
  // forward: one O accumulator per half of the key chunk (the two threads of a row keep
  // independent running maxima); dK/dV: dV and dK
  static constexpr int ACC_COLS = MODE == DQ ? D : 2 * D;
  // Resident operands that are the A side of the score products are copied to tensor memory
  // once per tile where the columns allow it: an MMA whose A comes from shared memory reads
  // 4 KB of A and 2 KB of B per K-step and is bound by that traffic (48 cycles at N = 64
  // instead of 32 with two CTAs issuing).
  static constexpr bool RES_T = (MODE == DQ || MODE == FWD) && D == 128;
  static constexpr int RES_BASE = ACC_BASE + ACC_COLS;
  static constexpr int RES_COLS = RES_T ? NRES * (D / 2) : 0;
  static constexpr int TMEM = RES_BASE + RES_COLS <= 256 ? 256 : 512;
  static constexpr int CTAS = (D == 64 && (XT == 0 || XT1_PAIR)) ? 2 : 1;
};

// Writes accumulator columns [c0, c0 + n) of this thread's tensor-memory lane to dst[c0 .. c0 + n) as 16-bit values.
template <typename T>
BSP_DEVI void store_acc(T* dst, uint32_t taddr, int c0, int n, float mul) {
  for (int c = c0; c < c0 + n; c += 32) {
    uint32_t r[32];
    tmem_ld32(taddr + c, r);
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
      uint4 v;
      v.x = pack16<T>(__uint_as_float(r[i]) * mul, __uint_as_float(r[i + 1]) * mul);
      v.y = pack16<T>(__uint_as_float(r[i + 2]) * mul, __uint_as_float(r[i + 3]) * mul);
      v.z = pack16<T>(__uint_as_float(r[i + 4]) * mul, __uint_as_float(r[i + 5]) * mul);
      v.w = pack16<T>(__uint_as_float(r[i + 6]) * mul, __uint_as_float(r[i + 7]) * mul);
      *reinterpret_cast<uint4*>(dst + c + i) = v;
    }
  }
}

// FINE: the lists come from a layout with blocks smaller than 64 (pieces of a position may be
// absent); a separate instantiation keeps the other case free of that bookkeeping.
template <typename T, int D, int MODE, bool KPM, bool FINE, int XT>
__global__ void __launch_bounds__(Cfg<D, MODE, KPM, XT>::NT, Cfg<D, MODE, KPM, XT>::CTAS)
attn_tc_kernel(const __grid_constant__ CUtensorMap m_res0, const __grid_constant__ CUtensorMap m_res1,
               const __grid_constant__ CUtensorMap m_ch0, const __grid_constant__ CUtensorMap m_ch1,
               const __grid_constant__ CUtensorMap m_rpe, const __grid_constant__ CUtensorMap m_am, TcArgs a) {
  using C = Cfg<D, MODE, KPM, XT>;
  static_assert(!XT || FINE, "the variants with rpe / attention mask use the masked code path");
  constexpr int ATOMS = C::ATOMS, ST = C::NSTAGE, NC = C::NC, NBUF = C::NBUF;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024 - (saddr(smem_raw) & 1023)) & 1023);
  unsigned char* res = smem;                                   // [NRES][ATOMS][128 rows][128 B]
  unsigned char* stg = res + C::NRES * C::RES_BYTES;           // [ST][ch0 | ch1 | lse, delta]
  __shared__ uint64_t bar_res, bar_rt, bar_rd, bar_full[ST], bar_s[4], bar_p[4], bar_acc[4], bar_done;
  __shared__ float xch[2][2][128];                           // forward: (max, sum) of the two halves of every row
  __shared__ uint32_t tmem_slot;
  __shared__ int failed[2];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // One-dimensional grid, batch entries of a tile adjacent: CTAs start in the order of the
  // tiles' lengths (longest first) over the whole launch, not per batch entry.
  const int z = blockIdx.x % a.Z;
  const int ti = a.order[blockIdx.x / a.Z];
  const int h = ti / a.tiles_per_head;
  const int first = a.ptr[ti], ntiles = a.ptr[ti + 1] - first;
  const int c0 = a.c01[2 * ti], c1 = a.c01[2 * ti + 1];
  const int64_t zh = (int64_t)(z * a.H + h) * a.L;

  // row of the tile this thread works on (compute warps), its global row and whether it exists
  const int quarter = warp & 3, chalf = (warp < NC) ? (warp >> 2) : 0;   // chalf: which 32 columns of a chunk
  const int trow = quarter * 32 + lane;
  const int mychunk = trow < 64 ? c0 : c1;
  const int64_t grow = (int64_t)(mychunk < 0 ? 0 : mychunk) * 64 + (trow & 63);
  const bool row_ok = mychunk >= 0 && warp < NC;

  if (ntiles == 0) {                                          // nothing in this tile: zeros, as the reference's products give
    if (row_ok && chalf == 0) {
      T* o0 = MODE == FWD ? reinterpret_cast<T*>(a.out0) + z * a.o_sz + h * a.o_sh + grow * a.o_sr
                          : reinterpret_cast<T*>(a.out0) + (zh + grow) * D;
      for (int c = 0; c < D; c += 8) {
        *reinterpret_cast<uint4*>(o0 + c) = make_uint4(0, 0, 0, 0);
        if (MODE == DKV) *reinterpret_cast<uint4*>(reinterpret_cast<T*>(a.out1) + (zh + grow) * D + c) = make_uint4(0, 0, 0, 0);
      }
      if (MODE == FWD) a.lse_out[zh + grow] = kNegInfT;
    }
    return;
  }
  // One chunk of the other operand (and what travels with it) into its stage of the ring.
  auto load_chunk = [&](int t, int crow) {
    const int stage = t % ST;
    unsigned char* sp = stg + stage * C::STAGE;
    uint32_t bytes = 2 * C::CH_BYTES + C::TAIL_BYTES;
    if constexpr (XT) bytes += (uint32_t)((c1 < 0 ? 1 : 2) * 8192 * ((a.has_rpe ? 1 : 0) + (a.am_mode ? 1 : 0)));
    mbar_expect_tx(&bar_full[stage], bytes);
    if (t == a.skip_chunk) return;                             // (test hook: this stage never fills, its consumers' waits run out)
    for (int at = 0; at < ATOMS; ++at) {
      tma_load_4d(sp + at * 8192, &m_ch0, &bar_full[stage], at * 64, crow, h, z);
      tma_load_4d(sp + C::CH_BYTES + at * 8192, &m_ch1, &bar_full[stage], at * 64, crow, h, z);
    }
    if (MODE == DKV) {
      bulk_load(sp + 2 * C::CH_BYTES, a.lse + zh + crow, 256, &bar_full[stage]);
      bulk_load(sp + 2 * C::CH_BYTES + 256, a.delta + zh + crow, 256, &bar_full[stage]);
    }
    if (C::BIAS) bulk_load(sp + 2 * C::CH_BYTES, reinterpret_cast<const T*>(a.kpm) + z * a.kpm_sz + crow, 128, &bar_full[stage]);
    if constexpr (XT) {
      // rows of rpe / the mask are queries, columns keys: the tile's rows are queries in the
      // forward and in dQ (the chunk brings keys), keys in dK / dV (the chunk brings queries)
      for (int hf = 0; hf < (c1 < 0 ? 1 : 2); ++hf) {
        const int outer = (hf == 0 ? c0 : c1) * 64;
        const int col = MODE == DKV ? outer : crow, row = MODE == DKV ? crow : outer;
        if (a.has_rpe) tma_load_4d(sp + C::XT_OFF + hf * 8192, &m_rpe, &bar_full[stage], col, row, h, a.rpe_z ? z : 0);
        if (a.am_mode) tma_load_4d(sp + C::XT_OFF + (a.has_rpe ? 16384 : 0) + hf * 8192, &m_am, &bar_full[stage], col, row, 0, 0);
      }
    }
  };
  // The thread that issues the loads sets up their barriers itself and starts the resident
  // operands and the first chunks at once: their latency overlaps the rest of the set-up
  // (other barriers, tensor-memory allocation, the block-wide synchronisation).
  if (tid == NC * 32) {
    mbar_init(&bar_res, 1);
    for (int s = 0; s < ST; ++s) mbar_init(&bar_full[s], 1);
    mbar_init_fence();
    prefetch_map(&m_res0); prefetch_map(&m_ch0); prefetch_map(&m_ch1);
    if constexpr (XT) { if (a.has_rpe) prefetch_map(&m_rpe); if (a.am_mode) prefetch_map(&m_am); }
    mbar_expect_tx(&bar_res, C::NRES * C::RES_BYTES);
    for (int hf = 0; hf < 2; ++hf) {
      const int crow = (hf == 0 || c1 < 0 ? c0 : c1) * 64;
      for (int at = 0; at < ATOMS; ++at) {
        tma_load_4d(res + at * 16384 + hf * 8192, &m_res0, &bar_res, at * 64, crow, h, z);
        if (C::NRES == 2) tma_load_4d(res + C::RES_BYTES + at * 16384 + hf * 8192, &m_res1, &bar_res, at * 64, crow, h, z);
      }
    }
    for (int t = 0; t < ST && t < ntiles; ++t) load_chunk(t, a.chunk[first + t] * 64);
  }
  if (tid == 0) {
    failed[0] = 0;
    failed[1] = a.wait_budget;
    mbar_init(&bar_rt, NC);
    mbar_init(&bar_rd, NC);
    if (C::ER) mbar_init(&bar_p[1], NC);
    if (C::ER2) mbar_init(&bar_s[2], 1);
    for (int b = 0; b < 4; ++b) mbar_init(&bar_acc[b], 1);
    for (int b = 0; b < NBUF; ++b) { mbar_init(&bar_s[b], 1); mbar_init(&bar_p[b], NC); }
    mbar_init(&bar_done, 1);
    mbar_init_fence();
  }
  if (warp == 1) { tmem_alloc(&tmem_slot, C::TMEM); tmem_relinquish(); }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem = tmem_slot;
  volatile int* fl = failed;

  if (warp >= NC) {
    // ------------------------------------------------------------------ loader and MMA issuers
    if (lane == 0) {
      const uint32_t idesc_kk = instr_desc(128, 64, 0, IsBf16<T>::v);   // A, B K-major
      const uint32_t idesc_mn = instr_desc(128, 64, 1, IsBf16<T>::v);   // B MN-major
      // Descriptor low words: a K-step advances a K-major operand by 32 bytes (2 units of 16
      // bytes) inside a 64-column group and an MN-major operand by 16 rows (128 units); the
      // next group of 64 columns lies 128 rows (resident) or 64 rows (chunk) further.
      // The issuing thread executes its instructions one after the other, and every
      // instruction between two MMAs delays the tensor core: all descriptors of a chunk are
      // therefore built first (while the barriers are still pending) and the MMAs of a
      // product are issued back to back.  A K-step advances a K-major operand by 32 bytes (2
      // units of 16 bytes) inside a 64-column group and an MN-major operand by 16 rows (128
      // units); the next group of 64 columns lies 128 rows (resident) or 64 rows (chunk) on.
      constexpr int KS = D / 16;
      const uint32_t res_lo = desc_lo(saddr(res));
      const uint32_t stg_lo = desc_lo(saddr(stg));
      uint64_t a0[KS], a1[MODE == FWD ? 1 : KS];            // resident operands: the same for every chunk
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        a0[ks] = desc_from_lo(res_lo + (ks / 4) * 1024 + (ks % 4) * 2);
        if (MODE != FWD) a1[ks] = desc_from_lo(res_lo + C::RES_BYTES / 16 + (ks / 4) * 1024 + (ks % 4) * 2);
      }
      uint64_t sb0[KS], sb1[MODE == FWD ? 1 : KS];          // chunk operands of the scores being prepared
      auto prep_scores = [&](int t) {
        const uint32_t sp_lo = stg_lo + (t % ST) * (C::STAGE / 16);
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          sb0[ks] = desc_from_lo(sp_lo + (ks / 4) * 512 + (ks % 4) * 2);
          if (MODE != FWD) sb1[ks] = desc_from_lo(sp_lo + C::CH_BYTES / 16 + (ks / 4) * 512 + (ks % 4) * 2);
        }
      };
      // part: 1 = first product (S), 2 = second (dP), 3 = both, one commit each call
      auto scores = [&](int t, int part, uint64_t* bar) {
        const uint32_t ts = tmem + (t % NBUF) * C::SCORE_COLS;
        if (C::RES_T) {
          const uint32_t tq = tmem + C::RES_BASE;
          if (part & 1) {
            mma_ts(ts, tq, sb0[0], idesc_kk, 0u);
#pragma unroll
            for (int ks = 1; ks < KS; ++ks) mma_ts_acc(ts, tq + ks * 8, sb0[ks], idesc_kk);
          }
          if (MODE != FWD && (part & 2)) {
            mma_ts(ts + 64, tq + D / 2, sb1[0], idesc_kk, 0u);
#pragma unroll
            for (int ks = 1; ks < KS; ++ks) mma_ts_acc(ts + 64, tq + D / 2 + ks * 8, sb1[ks], idesc_kk);
          }
        } else {
          if (part & 1) {
            mma_ss(ts, a0[0], sb0[0], idesc_kk, 0u);
#pragma unroll
            for (int ks = 1; ks < KS; ++ks) mma_ss_acc(ts, a0[ks], sb0[ks], idesc_kk);
          }
          if (MODE != FWD && (part & 2)) {
            mma_ss(ts + 64, a1[0], sb1[0], idesc_kk, 0u);
#pragma unroll
            for (int ks = 1; ks < KS; ++ks) mma_ss_acc(ts + 64, a1[ks], sb1[ks], idesc_kk);
          }
        }
        commit(bar);
      };
      uint64_t vb0[ATOMS * 4], vb1[ATOMS * 4];              // chunk operands of the accumulation being prepared
      auto prep_acc = [&](int t) {
        const uint32_t sp_lo = stg_lo + (t % ST) * (C::STAGE / 16);
#pragma unroll
        for (int at = 0; at < ATOMS; ++at)
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            vb0[at * 4 + ks] = desc_from_lo(sp_lo + at * 512 + ks * 128);
            vb1[at * 4 + ks] = desc_from_lo(sp_lo + C::CH_BYTES / 16 + at * 512 + ks * 128);
          }
      };
      // head_dim 128: the chunk operand of an accumulating product has two groups of 64 columns,
      // 8 KB apart; with that distance in the leading-offset field one N = 128 MMA covers both
      // (64 cycles instead of 2 x 48)
      constexpr bool WIDE = ATOMS == 2;
      const uint32_t idesc_acc = WIDE ? instr_desc(128, 128, 1, IsBf16<T>::v) : idesc_mn;
      auto wide = [](uint64_t d) { return WIDE ? ((d & ~0x3FFF0000ull) | (512ull << 16)) : d; };
      auto accumulate = [&](int t) {
        const uint32_t ts = tmem + (t % NBUF) * C::SCORE_COLS;
        const uint32_t ta = tmem + C::ACC_BASE;
        const uint32_t later = t > 0 ? 1u : 0u;
#pragma unroll
        for (int at = 0; at < (WIDE ? 1 : ATOMS); ++at)
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            // packed 16-bit operand of K-step ks (16 rows of the chunk): 8 columns inside the
            // 32-column slice of the compute thread that produced it
            const uint32_t pa = ts + (ks >> 1) * 32 + (ks & 1) * 8;
            if (MODE == FWD) {          // O_half += P_half . V_half: one accumulator per half of the chunk
              if (ks & 1) mma_ts_acc(ta + (ks >> 1) * D + at * 64, pa, wide(vb1[at * 4 + ks]), idesc_acc);
              else mma_ts(ta + (ks >> 1) * D + at * 64, pa, wide(vb1[at * 4 + ks]), idesc_acc, later);
            } else if (MODE == DQ) {    // dQ += dS . K
              const uint32_t da = C::ER ? tmem + C::PK_BASE + (t & 1) * 32 + ks * 8 : pa + 64;
              if (ks > 0) mma_ts_acc(ta + at * 64, da, wide(vb0[at * 4 + ks]), idesc_acc);
              else mma_ts(ta + at * 64, da, wide(vb0[at * 4 + ks]), idesc_acc, later);
            } else {                    // dV += P^T . dO,  dK += dS^T . Q
              const uint32_t pp = C::ER2 ? ts + 64 + (ks >> 1) * 32 + (ks & 1) * 16 : pa;
              const uint32_t pd = C::ER2 ? pp + 8 : pa + 64;
              if (ks > 0) {
                mma_ts_acc(ta + at * 64, pp, wide(vb1[at * 4 + ks]), idesc_acc);
                mma_ts_acc(ta + D + at * 64, pd, wide(vb0[at * 4 + ks]), idesc_acc);
              } else {
                mma_ts(ta + at * 64, pp, wide(vb1[at * 4 + ks]), idesc_acc, later);
                mma_ts(ta + D + at * 64, pd, wide(vb0[at * 4 + ks]), idesc_acc, later);
              }
            }
          }
        commit(&bar_acc[t & 3]);      // chunk t fully consumed: its score buffer and its stage are free
      };
      // Two issuing threads, one per kind of product, each in its own warp: the scores of chunk
      // t only wait for their operands and for the score buffer, the accumulation of chunk t
      // only for the compute warps; neither queues behind the other's barrier.  The accumulate
      // issuer, which has less to issue, also refills the ring of chunk operands.
      if (warp == NC) {
        bool ok = mbar_wait(C::RES_T ? &bar_rt : &bar_res, 0, fl);
        for (int t = 0; ok && t < ntiles; ++t) {
          prep_scores(t);
          ok = mbar_wait(&bar_full[t % ST], (t / ST) & 1, fl);
          if (C::ER || C::ER2) {
            if (ok && t >= 1) ok = mbar_wait(&bar_rd, (t - 1) & 1, fl);     // scores of chunk t - 1 are in registers
          } else {
            if (ok && t >= NBUF) ok = mbar_wait(&bar_acc[(t - NBUF) & 3], ((t - NBUF) >> 2) & 1, fl);
          }
          if (!ok) break;
          fence_after();
          if (C::ER2) {
            scores(t, 1, &bar_s[0]);
            if (t >= 1) {                                   // dP^T's columns still hold the operands of chunk t - 1
              ok = mbar_wait(&bar_acc[(t - 1) & 3], ((t - 1) >> 2) & 1, fl);
              if (!ok) break;
              fence_after();
            }
            scores(t, 2, &bar_s[2]);
          } else {
            scores(t, 3, &bar_s[t % NBUF]);
          }
        }
      } else {
        bool ok = true;
        for (int t = 0; ok && t < ntiles; ++t) {
          // first the stage of chunk t - 1 is refilled: its accumulation, issued one iteration
          // ago, completes while the compute warps are still busy with chunk t
          const int tn = t - 1 + ST;
          if (t >= 1 && tn < ntiles) {
            const int crow_n = a.chunk[first + tn] * 64;
            ok = mbar_wait(&bar_acc[(t - 1) & 3], ((t - 1) >> 2) & 1, fl);
            if (!ok) break;
            load_chunk(tn, crow_n);
          }
          prep_acc(t);
          ok = mbar_wait(&bar_full[t % ST], (t / ST) & 1, fl) &&
               (C::ER ? mbar_wait(&bar_p[t & 1], (t >> 1) & 1, fl) : mbar_wait(&bar_p[t % NBUF], (t / NBUF) & 1, fl));
          if (!ok) break;
          fence_after();
          accumulate(t);
        }
        if (ok) commit(&bar_done);
      }
    }
  } else {
    // ------------------------------------------------------------------ compute warps
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const int half = trow >> 6;                               // which 64-row chunk of the tile
    bool ok = true;
    if (C::RES_T) {
      // this thread's share of its row of the resident operands: shared memory (128-byte
      // rows, 16-byte units swizzled by the row) -> tensor memory, two 16-bit values per column
      ok = mbar_wait_warp(&bar_res, 0, fl);
      if (ok) {
        constexpr int UNITS = D / 16;                            // 16-byte units per thread and operand
#pragma unroll
        for (int r = 0; r < C::NRES; ++r) {
          const unsigned char* row = res + r * C::RES_BYTES + (D == 128 ? chalf * 16384 : 0) + trow * 128;
          uint32_t w[UNITS * 4];
#pragma unroll
          for (int u = 0; u < UNITS; ++u) {
            const int unit = (D == 128 ? u : chalf * UNITS + u) ^ (trow & 7);
            const uint4 v = *reinterpret_cast<const uint4*>(row + unit * 16);
            w[4 * u] = v.x; w[4 * u + 1] = v.y; w[4 * u + 2] = v.z; w[4 * u + 3] = v.w;
          }
          const uint32_t tq = tmem + C::RES_BASE + r * (D / 2) + chalf * (D / 4) + lane_base;
          if constexpr (D == 128) tmem_st32(tq, w); else tmem_st16(tq, w);
        }
        tmem_st_wait();
        fence_before();
        warp_arrive(&bar_rt, lane);
      }
    }
    if (MODE == FWD) {
      // this thread owns 32 of the 64 key columns of its row, with its own running
      // maximum, sum and O accumulator; the two halves are merged at the end
      const uint32_t t_acc = tmem + C::ACC_BASE + chalf * D + lane_base;
      float m_ref = kNegInfT, l = 0.f;
      for (int t = 0; ok && t < ntiles; ++t) {
        const uint32_t ts = tmem + (t % NBUF) * C::SCORE_COLS + lane_base + chalf * 32;
        int pieces = 3;
        bool valid, partial = false;
        if constexpr (FINE) {
          pieces = chunk_pieces(a.mask[first + t], a.sub[first + t], half, trow, chalf);
          valid = __any_sync(0xffffffffu, pieces != 0);               // per warp: something to compute
          partial = __any_sync(0xffffffffu, pieces != 3);
        } else {
          valid = (a.mask[first + t] >> half) & 1;                    // uniform per warp
        }
        ok = mbar_wait_warp(&bar_s[t % NBUF], (t / NBUF) & 1, fl);
        if (!ok) break;
        fence_after();
        uint32_t sr[32];
        tmem_ld32(ts, sr);
        tmem_ld_wait();
        if (partial) mask_pieces(sr, pieces);
        if (FINE && a.causal) mask_causal<32, false>(sr, a.chunk[first + t] * 64 + chalf * 32, (int)grow);
        float mt = kNegInfT;
        if (valid) {
          if constexpr (KPM || XT) {                         // scores become s * scale + bias (base 2) in place
            const unsigned char* bp = stg + (t % ST) * C::STAGE + 2 * C::CH_BYTES + chalf * 64;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              float b[8];
              if constexpr (KPM) kpm_terms8<T>(bp + g * 16, a.kpm_mul, b);
              else {
#pragma unroll
                for (int i = 0; i < 8; ++i) b[i] = 0.f;
              }
              if constexpr (XT) xt_add8<T>(stg + (t % ST) * C::STAGE + C::XT_OFF, a.has_rpe, a.am_mode, half, trow & 63, chalf * 4 + g, b);
#pragma unroll
              for (int i = 0; i < 8; i += 2) {
                const float2 y = __ffma2_rn(u2f(sr[8 * g + i], sr[8 * g + i + 1]), f2(a.scale_log2, a.scale_log2), f2(b[i], b[i + 1]));
                sr[8 * g + i] = __float_as_uint(y.x); sr[8 * g + i + 1] = __float_as_uint(y.y);
              }
            }
          }
          mt = max32(sr) * ((KPM || XT) ? 1.f : a.scale_log2);
        }
        // the reference maximum is only raised when the row maximum outgrows it by 2^8
        const bool grow_m = mt > m_ref + 8.f;
        if (__any_sync(0xffffffffu, grow_m)) {
          const float m_new = grow_m ? mt : m_ref;
          const float alpha = grow_m ? fast_exp2(m_ref - m_new) : 1.f;      // 0 while m_ref is still -inf
          l *= alpha;
          if (t > 0) {                                      // the accumulator must be complete up to chunk t-1
            ok = mbar_wait_warp(&bar_acc[(t - 1) & 3], ((t - 1) >> 2) & 1, fl);
            if (!ok) break;
            fence_after();
            for (int c = 0; c < D; c += 16) {               // (16 at a time: the scores stay in registers)
              uint32_t orr[16];
              tmem_ld16(t_acc + c, orr);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 16; ++i) orr[i] = __float_as_uint(__uint_as_float(orr[i]) * alpha);
              tmem_st16(t_acc + c, orr);
            }
            tmem_st_wait();
          }
          m_ref = m_new;
        }
        // exponentials in two halves of 16 columns: eight packed registers live at a time
        if (valid) {
          float2 s2[2] = {f2(0.f, 0.f), f2(0.f, 0.f)};
          // (with a mask or absent pieces a row may still have seen -inf only: its reference stays 0 then)
          const float m_use = ((KPM || FINE) && m_ref == kNegInfT) ? 0.f : m_ref;
          const float2 nm2 = f2(-m_use, -m_use), sl2 = f2(a.scale_log2, a.scale_log2);
#pragma unroll
          for (int hp = 0; hp < 2; ++hp) {
            uint32_t ph[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float2 s01 = u2f(sr[16 * hp + 2 * i], sr[16 * hp + 2 * i + 1]);
              const float2 y = (KPM || XT) ? __fadd2_rn(s01, nm2) : __ffma2_rn(s01, sl2, nm2);
              const float2 p = exp2_pair<1>(y);
              s2[i & 1] = __fadd2_rn(s2[i & 1], p);
              ph[i] = pack16<T>(p.x, p.y);
            }
            tmem_st8(ts + hp * 8, ph);
          }
          l += (s2[0].x + s2[0].y) + (s2[1].x + s2[1].y);
        } else {
          uint32_t pz[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) pz[i] = 0u;
          tmem_st16(ts, pz);
        }
        tmem_st_wait();
        fence_before();
        warp_arrive(&bar_p[t % NBUF], lane);
      }
      // merge the two halves of every row: O = (O_a 2^(m_a - m) + O_b 2^(m_b - m)) / l
      xch[chalf][0][trow] = m_ref;
      xch[chalf][1][trow] = l;
      asm volatile("bar.sync 1, 256;" ::: "memory");          // the eight compute warps, always executed
      if (ok && mbar_wait_warp(&bar_done, 0, fl)) {
        fence_after();
        if (mychunk >= 0) {                                   // uniform per warp: a warp lies inside one chunk
          const float ma = xch[0][0][trow], mb = xch[1][0][trow], la = xch[0][1][trow], lb = xch[1][1][trow];
          const float m = fmaxf(ma, mb);
          const float wa = ma == kNegInfT ? 0.f : fast_exp2(ma - m), wb = mb == kNegInfT ? 0.f : fast_exp2(mb - m);
          const float lsum = la * wa + lb * wb;
          const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
          T* orow = reinterpret_cast<T*>(a.out0) + z * a.o_sz + h * a.o_sh + grow * a.o_sr;
          const uint32_t ta = tmem + C::ACC_BASE + lane_base;
          for (int c = chalf * (D / 2); c < (chalf + 1) * (D / 2); c += 32) {
            uint32_t ra[32], rb[32];
            tmem_ld32(ta + c, ra);
            tmem_ld32(ta + D + c, rb);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              float o[8];
#pragma unroll
              for (int j = 0; j < 8; ++j)
                o[j] = (__uint_as_float(ra[i + j]) * wa + __uint_as_float(rb[i + j]) * wb) * inv;
              uint4 v;
              v.x = pack16<T>(o[0], o[1]); v.y = pack16<T>(o[2], o[3]);
              v.z = pack16<T>(o[4], o[5]); v.w = pack16<T>(o[6], o[7]);
              *reinterpret_cast<uint4*>(orow + c + i) = v;
            }
          }
          if (chalf == 0) a.lse_out[zh + grow] = lsum > 0.f ? m + log2f(lsum) : kNegInfT;
        }
      }
    } else {
      // (a fully masked query row has lse = -inf: +inf makes its probabilities 0, not NaN)
      float my_lse = (MODE == DQ && row_ok) ? a.lse[zh + grow] : 0.f;
      if ((KPM || FINE) && my_lse == kNegInfT) my_lse = -kNegInfT;
      // dK/dV: the bias of this thread's key row
      const float my_b = (KPM && MODE == DKV && row_ok)
          ? kpm_term(static_cast<float>(reinterpret_cast<const T*>(a.kpm)[z * a.kpm_sz + grow]), a.kpm_mul) : 0.f;
      const float my_d = (MODE == DQ && row_ok) ? a.delta[zh + grow] : 0.f;
      const float2 nd2 = f2(-my_d, -my_d), sl2 = f2(a.scale_log2, a.scale_log2);
      for (int t = 0; ok && t < ntiles; ++t) {
        const uint32_t ts = tmem + (t % NBUF) * C::SCORE_COLS + lane_base + chalf * 32;
        int pieces = 3;
        bool valid, partial = false;
        if constexpr (FINE) {
          pieces = chunk_pieces(a.mask[first + t], a.sub[first + t], half, trow, chalf);
          valid = __any_sync(0xffffffffu, pieces != 0);               // per warp: something to compute
          partial = __any_sync(0xffffffffu, pieces != 3);
        } else {
          valid = (a.mask[first + t] >> half) & 1;                    // uniform per warp
        }
        const float4* vec = reinterpret_cast<const float4*>(stg + (t % ST) * C::STAGE + 2 * C::CH_BYTES) + chalf * 8;
        ok = mbar_wait_warp(&bar_s[t % NBUF], (t / NBUF) & 1, fl);
        if (!ok) break;
        fence_after();
        if constexpr (C::ER) {
          // S and dP of this thread's 32 columns go to registers at once; the score buffer is
          // then handed back, and the next scores are computed during the arithmetic below
          uint32_t sr[32], qr[32], dr[16];
          tmem_ld32(ts, sr);
          tmem_ld32(ts + 64, qr);
          tmem_ld_wait();
          fence_before();
          warp_arrive(&bar_rd, lane);
          if (partial) mask_pieces(sr, pieces);
          if (FINE && a.causal) mask_causal<32, false>(sr, a.chunk[first + t] * 64 + chalf * 32, (int)grow);
          if (valid) {
            const unsigned char* bp = stg + (t % ST) * C::STAGE + 2 * C::CH_BYTES + chalf * 64;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              float b[8];
              if constexpr (KPM || XT) {
                if constexpr (KPM) kpm_terms8<T>(bp + g * 16, a.kpm_mul, b);
                else {
#pragma unroll
                  for (int i = 0; i < 8; ++i) b[i] = 0.f;
                }
                if constexpr (XT) xt_add8<T>(stg + (t % ST) * C::STAGE + C::XT_OFF, a.has_rpe, a.am_mode, half, trow & 63, chalf * 4 + g, b);
#pragma unroll
                for (int i = 0; i < 8; ++i) b[i] -= my_lse;
              } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) b[i] = -my_lse;
              }
#pragma unroll
              for (int i = 8 * g; i < 8 * g + 8; i += 2) {
                const float2 y = __ffma2_rn(u2f(sr[i], sr[i + 1]), sl2, f2(b[i - 8 * g], b[i + 1 - 8 * g]));
                const float2 p = exp2_pair<1>(y);
                const float2 d = __fmul2_rn(p, __fadd2_rn(u2f(qr[i], qr[i + 1]), nd2));   // P (dP - delta); the scale is applied to dQ
                dr[i / 2] = pack16<T>(d.x, d.y);
              }
            }
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) dr[i] = 0u;
          }
          if (t >= 2) {                                     // the accumulation of chunk t - 2 has read its operand
            ok = mbar_wait_warp(&bar_acc[(t - 2) & 3], ((t - 2) >> 2) & 1, fl);
            if (!ok) break;
            fence_after();
          }
          tmem_st16(tmem + C::PK_BASE + (t & 1) * 32 + chalf * 16 + lane_base, dr);
          tmem_st_wait();
          fence_before();
          warp_arrive(&bar_p[t & 1], lane);
          continue;
        }
        if constexpr (C::ER2) {
          // First all of S^T: read, handed back, exponentials, P^T packed to 16 bits; this runs
          // while dP^T is still being computed.  Then dP^T in two passes of 16 columns; pass
          // hv leaves its part of the packed P^T in columns [16 hv, 16 hv + 8) and its packed
          // dS^T in the next 8 columns of this thread's 32 columns of dP^T, all read before.
          // dS is formed with P as the accumulating product sees it (rounded to 16 bits),
          // which is also how a stored softmax output would enter the product.
          float pf[32];                                        // P^T of this thread's 32 columns
          if (valid) {
            uint32_t sr[32];
            tmem_ld32(ts, sr);
            tmem_ld_wait();
            fence_before();
            warp_arrive(&bar_rd, lane);
            if (partial) mask_pieces(sr, pieces);
            if (FINE && a.causal) mask_causal<32, true>(sr, a.chunk[first + t] * 64 + chalf * 32, (int)grow);
            const float2 nsl2 = f2(-a.scale_log2, -a.scale_log2);
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              float4 lv = vec[i / 4];                           // per-query lse of this chunk
              if (KPM || FINE) {                              // own bias; a query row without any key counts as +inf
                lv.x = lv.x == kNegInfT ? -kNegInfT : lv.x - my_b; lv.y = lv.y == kNegInfT ? -kNegInfT : lv.y - my_b;
                lv.z = lv.z == kNegInfT ? -kNegInfT : lv.z - my_b; lv.w = lv.w == kNegInfT ? -kNegInfT : lv.w - my_b;
              }
              if constexpr (XT) {                             // rpe / mask of (query chalf * 32 + i .. + 3, this key)
                const unsigned char* xt = stg + (t % ST) * C::STAGE + C::XT_OFF;
                lv.x -= xt_term<T>(xt, a.has_rpe, a.am_mode, half, chalf * 32 + i, trow & 63);
                lv.y -= xt_term<T>(xt, a.has_rpe, a.am_mode, half, chalf * 32 + i + 1, trow & 63);
                lv.z -= xt_term<T>(xt, a.has_rpe, a.am_mode, half, chalf * 32 + i + 2, trow & 63);
                lv.w -= xt_term<T>(xt, a.has_rpe, a.am_mode, half, chalf * 32 + i + 3, trow & 63);
              }
              // the negated exponent lse - s c: the lse comes from shared memory as it is
              const float2 z0 = __ffma2_rn(u2f(sr[i], sr[i + 1]), nsl2, f2(lv.x, lv.y));
              const float2 z1 = __ffma2_rn(u2f(sr[i + 2], sr[i + 3]), nsl2, f2(lv.z, lv.w));
              const float2 p0 = exp2_pair<-1>(z0);
              const float2 p1 = exp2_pair<-1>(z1);
              pf[i] = p0.x; pf[i + 1] = p0.y; pf[i + 2] = p1.x; pf[i + 3] = p1.y;
            }
          } else {
            fence_before();
            warp_arrive(&bar_rd, lane);
#pragma unroll
            for (int i = 0; i < 32; ++i) pf[i] = 0.f;
          }
          ok = mbar_wait_warp(&bar_s[2], t & 1, fl);
          if (!ok) break;
          fence_after();
#pragma unroll
          for (int hv = 0; hv < 2; ++hv) {
            uint32_t qr[16], dr[8], ph[8];
            if (valid) {
              tmem_ld16(ts + 64 + hv * 16, qr);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 16; i += 4) {
                const float4 ev = vec[16 + hv * 4 + i / 4];     // per-query delta of this chunk
                const float2 pa = f2(pf[hv * 16 + i], pf[hv * 16 + i + 1]), pb = f2(pf[hv * 16 + i + 2], pf[hv * 16 + i + 3]);
                // P (dP - delta); the score scale is applied to dK when it is stored
                const float2 d0 = __fmul2_rn(pa, __ffma2_rn(f2(ev.x, ev.y), f2(-1.f, -1.f), u2f(qr[i], qr[i + 1])));
                const float2 d1 = __fmul2_rn(pb, __ffma2_rn(f2(ev.z, ev.w), f2(-1.f, -1.f), u2f(qr[i + 2], qr[i + 3])));
                dr[i / 2] = pack16<T>(d0.x, d0.y); dr[i / 2 + 1] = pack16<T>(d1.x, d1.y);
                ph[i / 2] = pack16<T>(pa.x, pa.y); ph[i / 2 + 1] = pack16<T>(pb.x, pb.y);
              }
            } else {
#pragma unroll
              for (int i = 0; i < 8; ++i) { dr[i] = 0u; ph[i] = 0u; }
            }
            tmem_st8(ts + 64 + hv * 16, ph);
            tmem_st8(ts + 64 + hv * 16 + 8, dr);
          }
          tmem_st_wait();
          fence_before();
          warp_arrive(&bar_p[0], lane);
          continue;
        }
        // Two passes of 16 columns keep the live registers of a pass at 48.  The packed
        // 16-bit results of pass hv go to columns [8 hv, 8 hv + 8) of this thread's own
        // 32-column slice: pass 0 only overwrites columns it has already read.
#pragma unroll
        for (int hv = 0; hv < 2; ++hv) {
          uint32_t sr[16], qr[16], pr[8], dr[8];
          if (valid) {
            tmem_ld16(ts + hv * 16, sr);
            tmem_ld16(ts + 64 + hv * 16, qr);
            tmem_ld_wait();
            if (partial && !((pieces >> hv) & 1)) {             // this pass is one group of 16 columns
#pragma unroll
              for (int i = 0; i < 16; ++i) sr[i] = kNegInfBits;
            }
            if (FINE && a.causal) mask_causal<16, MODE == DKV>(sr, a.chunk[first + t] * 64 + chalf * 32 + hv * 16, (int)grow);
#pragma unroll
            for (int i = 0; i < 16; i += 4) {
              float ls[4], es[4];
              if (MODE == DKV) {                            // per-query lse and delta * scale of this chunk
                const float4 lv = vec[hv * 4 + i / 4], ev = vec[16 + hv * 4 + i / 4];
                ls[0] = lv.x; ls[1] = lv.y; ls[2] = lv.z; ls[3] = lv.w;
                es[0] = ev.x; es[1] = ev.y; es[2] = ev.z; es[3] = ev.w;
                if (KPM || FINE) {
#pragma unroll
                  for (int j = 0; j < 4; ++j) ls[j] = ls[j] == kNegInfT ? -kNegInfT : ls[j] - my_b;
                }
              } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) { ls[j] = my_lse; es[j] = my_d; }
                if constexpr (KPM) {                        // bias of the four keys
                  const uint2 raw = *reinterpret_cast<const uint2*>(stg + (t % ST) * C::STAGE + 2 * C::CH_BYTES + chalf * 64 + (hv * 16 + i) * 2);
                  const float2 b01 = unpack16<T>(raw.x), b23 = unpack16<T>(raw.y);
                  ls[0] -= kpm_term(b01.x, a.kpm_mul); ls[1] -= kpm_term(b01.y, a.kpm_mul);
                  ls[2] -= kpm_term(b23.x, a.kpm_mul); ls[3] -= kpm_term(b23.y, a.kpm_mul);
                }
              }
              if constexpr (XT) {                             // rpe / mask of the four (query, key) pairs
                const unsigned char* xt = stg + (t % ST) * C::STAGE + C::XT_OFF;
                const int cc = chalf * 32 + hv * 16 + i;        // column of the chunk: a key (dQ) or a query (dK / dV)
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  ls[j] -= MODE == DKV ? xt_term<T>(xt, a.has_rpe, a.am_mode, half, cc + j, trow & 63)
                                       : xt_term<T>(xt, a.has_rpe, a.am_mode, half, trow & 63, cc + j);
              }
              // two elements per instruction: the negated exponent lse - s c, P = 2^-(that), and
              // dS = P (dP - delta); the score scale is applied when dQ / dK are written
              const float2 nsl2 = f2(-a.scale_log2, -a.scale_log2), m1 = f2(-1.f, -1.f);
              const float2 p0 = exp2_pair<-1>(__ffma2_rn(u2f(sr[i], sr[i + 1]), nsl2, f2(ls[0], ls[1])));
              const float2 p1 = exp2_pair<-1>(__ffma2_rn(u2f(sr[i + 2], sr[i + 3]), nsl2, f2(ls[2], ls[3])));
              const float2 d0 = __fmul2_rn(p0, __ffma2_rn(f2(es[0], es[1]), m1, u2f(qr[i], qr[i + 1])));
              const float2 d1 = __fmul2_rn(p1, __ffma2_rn(f2(es[2], es[3]), m1, u2f(qr[i + 2], qr[i + 3])));
              pr[i / 2] = pack16<T>(p0.x, p0.y); pr[i / 2 + 1] = pack16<T>(p1.x, p1.y);
              dr[i / 2] = pack16<T>(d0.x, d0.y); dr[i / 2 + 1] = pack16<T>(d1.x, d1.y);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) { pr[i] = 0u; dr[i] = 0u; }
          }
          if (MODE == DKV) tmem_st8(ts + hv * 8, pr);
          tmem_st8(ts + 64 + hv * 8, dr);
        }
        tmem_st_wait();
        fence_before();
        warp_arrive(&bar_p[t % NBUF], lane);
      }
      if (ok && mbar_wait_warp(&bar_done, 0, fl)) {
        fence_after();
        if (mychunk >= 0) {                                   // uniform per warp
          // the two threads of a row split the D output columns
          const uint32_t ta = tmem + C::ACC_BASE + lane_base;
          T* o0 = reinterpret_cast<T*>(a.out0) + (zh + grow) * D;
          // (dS is formed without the score scale, which is applied here)
          const float ds_scale = a.scale;
          if (MODE == DQ) {
            store_acc<T>(o0, ta, chalf * (D / 2), D / 2, ds_scale);
          } else {
            T* o1 = reinterpret_cast<T*>(a.out1) + (zh + grow) * D;
            store_acc<T>(o1, ta, chalf * (D / 2), D / 2, 1.f);            // dV: accumulator columns [0, D)
            store_acc<T>(o0 - D, ta, D + chalf * (D / 2), D / 2, ds_scale);    // dK: accumulator columns [D, 2D)
          }
        }
      }
    }
  }
  fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, C::TMEM);
  if (tid == 0 && failed[0]) atomicExch(&g_tc_status, 1 + MODE);
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    cudaDriverEntryPointQueryResult q;
    void* p = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess) fn = (EncodeTiledFn)p;
  }
  return fn;
}

// [Z, H, L, D] operand with unit stride on D: boxes of 64 columns x 64 rows, 128-byte swizzle.
int encode_map(CUtensorMap* m, const void* ptr, int dtype, int Z, int H, int L, int D,
             int64_t sz, int64_t sh, int64_t sr) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(BSP_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  // The encoder is a driver call and needs the primary context bound to this thread; a thread
  // that has made no runtime call yet (a worker thread of the caller) has none.
  static thread_local bool bound = false;
  if (!bound) { cudaFree(nullptr); bound = true; }
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)L, (cuuint64_t)H, (cuuint64_t)Z};
  cuuint64_t strides[3] = {(cuuint64_t)sr * 2, (cuuint64_t)(H > 1 ? sh : (int64_t)L * sr) * 2,
                           (cuuint64_t)(Z > 1 ? sz : (int64_t)H * L * sr) * 2};
  cuuint32_t box[4] = {64, 64, 1, 1};
  cuuint32_t es[4] = {1, 1, 1, 1};
  CUresult r = fn(m, dtype == BSP_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                  const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(BSP_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return BSP_OK;
}

// A tensor map is a pure function of the address, the type, the shape and the strides: a training
// loop presents the same few operands step after step, so the last maps of every calling thread
// are kept and an encoder call is only made for an operand not seen recently.
struct MapKey {
  const void* ptr; int dtype, Z, H, L, D; int64_t sz, sh, sr;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && dtype == o.dtype && Z == o.Z && H == o.H && L == o.L && D == o.D && sz == o.sz && sh == o.sh && sr == o.sr;
  }
};
constexpr int kMapCache = 16;
struct MapCache { MapKey key[kMapCache]; CUtensorMap map[kMapCache]; int used = 0, next = 0; };

int make_map(CUtensorMap* m, const void* ptr, int dtype, int Z, int H, int L, int D,
             int64_t sz, int64_t sh, int64_t sr) {
  static thread_local MapCache cache;
  const MapKey k = {ptr, dtype, Z, H, L, D, sz, sh, sr};
  for (int i = 0; i < cache.used; ++i)
    if (cache.key[i] == k) { *m = cache.map[i]; return BSP_OK; }
  if (int rc = encode_map(m, ptr, dtype, Z, H, L, D, sz, sh, sr)) return rc;
  const int slot = cache.used < kMapCache ? cache.used++ : (cache.next++ % kMapCache);
  cache.key[slot] = k;
  cache.map[slot] = *m;
  return BSP_OK;
}

// Test hooks (bsp_debug_attn_wait): the budget of the bounded waits and a chunk whose loads are withheld.
std::atomic<int> g_wait_budget{kWaitBudget}, g_skip_chunk{-1};

struct TileSet { const int32_t *c01, *ptr, *chunk, *mask, *sub, *order; };
struct TilesView { int H, nb, block, tiles_per_head, fine; TileSet rt, ct; };

int decode_tiles(const int32_t* hdr, const int32_t* dev, TilesView& v) {
  if (hdr[0] != BSP_TILES_MAGIC) return fail(BSP_ERR_INVALID, "attention tile lists: bad magic");
  v.H = hdr[1]; v.nb = hdr[2]; v.block = hdr[3]; v.tiles_per_head = hdr[4]; v.fine = hdr[7] < 64 ? 1 : 0;
  const int64_t n = (int64_t)v.H * v.tiles_per_head;
  const int32_t* p = dev + BSP_TILES_HEADER;
  auto take = [&](TileSet& s, int64_t entries) {
    s.c01 = p; p += 2 * n; s.ptr = p; p += n + 1; s.chunk = p; p += entries; s.mask = p; p += entries; s.sub = p; p += entries; s.order = p; p += n;
  };
  take(v.rt, hdr[5]);
  take(v.ct, hdr[6]);
  return BSP_OK;
}

// The maps a launch needs: resident operands, chunk operands and (XT variants) rpe / attention mask.
struct Maps { CUtensorMap r0, r1, c0, c1, rpe, am; };

template <typename T, int D, int MODE, bool KPM, bool FINE, int XT>
int launch(const Maps& m, const TcArgs& a, int n_tiles, int Z, cudaStream_t st, const char* what) {
  using C = Cfg<D, MODE, KPM, XT>;
  auto kern = attn_tc_kernel<T, D, MODE, KPM, FINE, XT>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
  if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "attention (tcgen05 %s): cannot reserve shared memory: %s", what, cudaGetErrorString(e));
  TcArgs b = a;
  b.Z = Z;
  b.wait_budget = g_wait_budget.load();
  b.skip_chunk = g_skip_chunk.load();
  kern<<<(unsigned)((int64_t)n_tiles * Z), C::NT, C::SMEM, st>>>(m.r0, m.r1, m.c0, m.c1, m.rpe, m.am, b);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "attention (tcgen05 %s) launch failed: %s", what, cudaGetErrorString(e));
  return BSP_OK;
}

template <int MODE, bool KPM, bool FINE, int XT>
int launch_dt(int dtype, int D, const Maps& m, const TcArgs& a, int n_tiles, int Z, cudaStream_t st, const char* what) {
  if (dtype == BSP_F16) {
    if (D == 64) return launch<__half, 64, MODE, KPM, FINE, XT>(m, a, n_tiles, Z, st, what);
    return launch<__half, 128, MODE, KPM, FINE, XT>(m, a, n_tiles, Z, st, what);
  }
  if (D == 64) return launch<__nv_bfloat16, 64, MODE, KPM, FINE, XT>(m, a, n_tiles, Z, st, what);
  return launch<__nv_bfloat16, 128, MODE, KPM, FINE, XT>(m, a, n_tiles, Z, st, what);
}
template <int MODE>
int launch_any(int dtype, int D, const Maps& m, const TcArgs& a, int n_tiles, int Z, cudaStream_t st, const char* what) {
  if (a.has_rpe && a.am_mode) {           // rpe and an attention mask that is read: the masked code path
    if (a.kpm) return launch_dt<MODE, true, true, 2>(dtype, D, m, a, n_tiles, Z, st, what);
    return launch_dt<MODE, false, true, 2>(dtype, D, m, a, n_tiles, Z, st, what);
  }
  if (a.has_rpe || a.am_mode) {           // one of them
    if (a.kpm) return launch_dt<MODE, true, true, 1>(dtype, D, m, a, n_tiles, Z, st, what);
    return launch_dt<MODE, false, true, 1>(dtype, D, m, a, n_tiles, Z, st, what);
  }
  if (a.kpm) {
    if (a.fine || a.causal) return launch_dt<MODE, true, true, 0>(dtype, D, m, a, n_tiles, Z, st, what);
    return launch_dt<MODE, true, false, 0>(dtype, D, m, a, n_tiles, Z, st, what);
  }
  if (a.fine || a.causal) return launch_dt<MODE, false, true, 0>(dtype, D, m, a, n_tiles, Z, st, what);
  return launch_dt<MODE, false, false, 0>(dtype, D, m, a, n_tiles, Z, st, what);
}

// rpe [Z or 1, H, L, L] and the attention mask [L, L] as maps of 64 x 64 boxes; an absent one gets
// a copy of `any` (never dereferenced).
int xt_maps(Maps& m, TcArgs& a, const XtHost* xt, const CUtensorMap& any, int dtype, int Z, int H, int L) {
  m.rpe = any; m.am = any;
  a.has_rpe = 0; a.rpe_z = 0; a.am_mode = 0;
  if (!xt) return BSP_OK;
  if (xt->rpe) {
    a.has_rpe = 1; a.rpe_z = xt->rpe_sz != 0 ? 1 : 0;
    if (int rc = make_map(&m.rpe, xt->rpe, dtype, a.rpe_z ? Z : 1, H, L, L, xt->rpe_sz, xt->rpe_sh, xt->rpe_sr)) return rc;
  }
  if (xt->am) {
    a.am_mode = xt->am_mode;
    if (int rc = make_map(&m.am, xt->am, dtype, 1, 1, L, L, 0, 0, xt->am_sr)) return rc;
  }
  return BSP_OK;
}

// A second stream per calling thread and device, on which the dQ kernel of a backward runs
// beside the dK / dV kernel (they are independent): the CTAs of the one fill the SMs the other
// leaves idle in its last wave, which is most of the time when a shard is small.
struct SideStream { cudaStream_t stream = nullptr; cudaEvent_t fork = nullptr, join = nullptr; };

int side_stream(SideStream** out) {
  constexpr int kMaxDev = 64;
  static thread_local SideStream table[kMaxDev];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return fail(BSP_ERR_CUDA, "attention: cannot tell the current device");
  SideStream& s = table[dev];
  if (!s.stream) {
    cudaError_t e = cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&s.join, cudaEventDisableTiming);
    if (e != cudaSuccess) { s = SideStream(); return fail(BSP_ERR_CUDA, "attention: cannot create the second stream: %s", cudaGetErrorString(e)); }
  }
  *out = &s;
  return BSP_OK;
}

void fill_tiles(TcArgs& a, const TilesView& tv, const TileSet& s) {
  a.tiles_per_head = tv.tiles_per_head;
  a.c01 = s.c01; a.ptr = s.ptr; a.chunk = s.chunk; a.mask = s.mask; a.sub = s.sub; a.order = s.order;
  a.fine = tv.fine;
}

}  // namespace

// Forward on the tcgen05 path.  Preconditions (checked by the caller): dtype F16 / BF16,
// D in {64, 128}, block in {64, 128}, no rpe / attention mask, unit stride on D; kpm (optional)
// is the key-padding mask [Z, L] in the operands' type with 16-byte aligned rows.
int attn_fwd_tc(const void* q, const void* k, const void* v, void* o, float* lse,
                int dtype, int Z, int H, int L, int D,
                int64_t q_sz, int64_t q_sh, int64_t q_sr, int64_t k_sz, int64_t k_sh, int64_t k_sr,
                int64_t v_sz, int64_t v_sh, int64_t v_sr, int64_t o_sz, int64_t o_sh, int64_t o_sr,
                const int32_t* tiles_hdr, const int32_t* tiles, float scale,
                const void* kpm, int64_t kpm_sz, int kpm_mul, int causal, const XtHost* xt, cudaStream_t st) {
  TilesView tv;
  if (int rc = decode_tiles(tiles_hdr, tiles, tv)) return rc;
  if (tv.H != H || tv.nb * tv.block != L) return fail(BSP_ERR_INVALID, "attention tile lists do not fit %d heads of length %d", H, L);
  CUtensorMap mq, mk, mv;
  if (int rc = make_map(&mq, q, dtype, Z, H, L, D, q_sz, q_sh, q_sr)) return rc;
  if (int rc = make_map(&mk, k, dtype, Z, H, L, D, k_sz, k_sh, k_sr)) return rc;
  if (int rc = make_map(&mv, v, dtype, Z, H, L, D, v_sz, v_sh, v_sr)) return rc;
  Maps m;
  m.r0 = mq; m.r1 = mq; m.c0 = mk; m.c1 = mv;
  TcArgs a = {};
  if (int rc = xt_maps(m, a, xt, mq, dtype, Z, H, L)) return rc;
  a.out0 = o; a.lse_out = lse; a.o_sz = o_sz; a.o_sh = o_sh; a.o_sr = o_sr;
  a.H = H; a.L = L; a.scale = scale; a.scale_log2 = scale * kLog2eT;
  a.kpm = kpm; a.kpm_sz = kpm_sz; a.kpm_mul = kpm_mul; a.causal = causal;
  fill_tiles(a, tv, tv.rt);
  return launch_any<FWD>(dtype, D, m, a, H * tv.tiles_per_head, Z, st, "forward");
}

// dK/dV (parts & 2) and dQ (parts & 4) on the tcgen05 path; `delta` must already hold rowsum(o * do).
int attn_bwd_tc(const void* q, const void* k, const void* v, const void* dout, const float* lse, const float* delta,
                void* dq, void* dk, void* dv, int dtype, int Z, int H, int L, int D,
                int64_t q_sz, int64_t q_sh, int64_t q_sr, int64_t k_sz, int64_t k_sh, int64_t k_sr,
                int64_t v_sz, int64_t v_sh, int64_t v_sr, int64_t do_sz, int64_t do_sh, int64_t do_sr,
                const int32_t* tiles_hdr, const int32_t* tiles, float scale,
                const void* kpm, int64_t kpm_sz, int kpm_mul, int causal, int parts, const XtHost* xt, int overlap,
                cudaStream_t st) {
  TilesView tv;
  if (int rc = decode_tiles(tiles_hdr, tiles, tv)) return rc;
  if (tv.H != H || tv.nb * tv.block != L) return fail(BSP_ERR_INVALID, "attention tile lists do not fit %d heads of length %d", H, L);
  CUtensorMap mq, mk, mv, md;
  if (int rc = make_map(&mq, q, dtype, Z, H, L, D, q_sz, q_sh, q_sr)) return rc;
  if (int rc = make_map(&mk, k, dtype, Z, H, L, D, k_sz, k_sh, k_sr)) return rc;
  if (int rc = make_map(&mv, v, dtype, Z, H, L, D, v_sz, v_sh, v_sr)) return rc;
  if (int rc = make_map(&md, dout, dtype, Z, H, L, D, do_sz, do_sh, do_sr)) return rc;
  Maps m;
  TcArgs a = {};
  if (int rc = xt_maps(m, a, xt, mq, dtype, Z, H, L)) return rc;
  a.lse = lse; a.delta = delta; a.H = H; a.L = L; a.scale = scale; a.scale_log2 = scale * kLog2eT;
  a.kpm = kpm; a.kpm_sz = kpm_sz; a.kpm_mul = kpm_mul; a.causal = causal;
  const int n_tiles = H * tv.tiles_per_head;
  // dK / dV on the caller's stream; dQ beside it on the thread's second stream when both are
  // asked for and the caller allows it (fork and join by events, so the caller's stream order,
  // and a stream capture, see one backward)
  SideStream* side = nullptr;
  if (overlap && (parts & 6) == 6) {
    if (int rc = side_stream(&side)) return rc;
    cudaError_t e = cudaEventRecord(side->fork, st);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(side->stream, side->fork, 0);
    if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "attention: forking to the second stream failed: %s", cudaGetErrorString(e));
  }
  if (parts & 2) {
    a.out0 = dk; a.out1 = dv;
    fill_tiles(a, tv, tv.ct);
    m.r0 = mk; m.r1 = mv; m.c0 = mq; m.c1 = md;
    if (int rc = launch_any<DKV>(dtype, D, m, a, n_tiles, Z, st, "dK/dV")) return rc;
  }
  if (parts & 4) {
    a.out0 = dq; a.out1 = nullptr;
    fill_tiles(a, tv, tv.rt);
    m.r0 = mq; m.r1 = md; m.c0 = mk; m.c1 = mv;
    if (int rc = launch_any<DQ>(dtype, D, m, a, n_tiles, Z, side ? side->stream : st, "dQ")) return rc;
  }
  if (side) {
    cudaError_t e = cudaEventRecord(side->join, side->stream);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(st, side->join, 0);
    if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "attention: joining the second stream failed: %s", cudaGetErrorString(e));
  }
  return BSP_OK;
}


// Test hook: wait_budget <= 0 restores the default; skip_chunk < 0 withholds nothing.
int tc_debug_wait(int wait_budget, int skip_chunk) {
  g_wait_budget.store(wait_budget > 0 ? wait_budget : kWaitBudget);
  g_skip_chunk.store(skip_chunk < 0 ? -1 : skip_chunk);
  return BSP_OK;
}

int tc_device_status(int* out) {
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int));
  if (e == cudaSuccess && v != 0) { const int zero = 0; e = cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int)); }   // reading clears
  if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "reading the device status failed: %s", cudaGetErrorString(e));
  *out = v;
  return BSP_OK;
}

}  // namespace bsp
