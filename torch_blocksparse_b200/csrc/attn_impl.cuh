// Fused block-sparse self-attention, forward and backward (mma.sync path).
//
// Replaces the three-launch chain sdd(Q, K^T) -> softmax -> dsd(P, V) of
// DeepSpeedSparseSelfAttention.forward
// (torch_blocksparse/deepspeedsparseselfattention.py:157-166) and the five
// launches of its autograd backward, without ever writing the score tensor
// [Z, nnz, block, block] to memory.
//
//   forward   one CTA per block-row of the layout: walks the row's nonzero
//             blocks (CSR), S = Q K^T on tensor cores, online softmax in FP32
//             registers (scale, rpe, key-padding and attention masks applied to
//             S exactly as the softmax kernel applies them), O += P V.  Also
//             writes the row-wise base-2 log-sum-exp for the backward.
//   backward  (1) delta = rowsum(O * dO);
//             (2) one CTA per block-column (CSC): recomputes P^T from the
//                 log-sum-exp, accumulates dV += P^T dO and dK += dS^T Q;
//             (3) one CTA per block-row (CSR): recomputes P, dQ += dS K.
//             Every output element is produced by exactly one CTA in a fixed
//             order: no atomics, bitwise reproducible.
//
// Each warp owns 16 rows of its CTA's tile; K/V (or Q/dO) tiles stream through
// a double-buffered cp.async pipeline.
#pragma once
#include "common.h"
#include "tile.cuh"

namespace bsp {
namespace {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kNegInfA = -__builtin_huge_valf();

struct MaskArgs {
  const void* rpe; int64_t rpe_sz, rpe_sh, rpe_sr;
  const void* kpm; int64_t kpm_sz; int kpm_mul;
  const void* am; int64_t am_sr; int am_mul;
};

struct AttnArgs {
  const void *q, *k, *v, *o, *dout;
  void *o_w, *dq, *dk, *dv;
  float* lse; float* delta;
  int64_t q_sz, q_sh, q_sr, k_sz, k_sh, k_sr, v_sz, v_sh, v_sr, o_sz, o_sh, o_sr, do_sz, do_sh, do_sr;
  int H, L, nb;                 // nb = L / block
  float scale;
  const int32_t *row_ptr, *blk_col, *row_order, *col_ptr, *col_row, *col_order;
  MaskArgs m;
};

template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <typename T> __device__ __forceinline__ float ldf(const T* p) { return static_cast<float>(*p); }

template <int B, int D> struct AttnCfg {
  static constexpr int NW = B / 16;                 // warps; each owns 16 rows of the CTA tile
  static constexpr int NT = NW * 32;
  static constexpr int BN = B < 64 ? B : 64;        // width of the streamed tile
  static constexpr int SUBS = B / BN;
  static constexpr int PD = D + 8;                  // shared-memory pitch (elements)
  static constexpr int KD = D / 16;                 // k-steps over the head dimension
  static constexpr int NI = BN / 8;                 // n-tiles of a score tile
  static constexpr int DI = D / 8;                  // n-tiles over the head dimension
};

// S (16 x BN per warp) = A_frag (16 x D, registers) . Xs^T, Xs stored [BN][PD].
template <typename T, int BN, int D, int PD>
__device__ __forceinline__ void qk_tile(float (&s)[BN / 8][4], const uint32_t (&af)[D / 16][4], const T* Xs, int lane) {
  const int l7 = lane & 7, mi4 = lane >> 3;
#pragma unroll
  for (int j = 0; j < BN / 8; ++j)
#pragma unroll
    for (int r = 0; r < 4; ++r) s[j][r] = 0.f;
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk)
#pragma unroll
    for (int j = 0; j < BN / 8; j += 2) {
      uint32_t b[4];
      ldsm_x4(b, smem_u32(Xs + (j * 8 + (mi4 >> 1) * 8 + l7) * PD + kk * 16 + (mi4 & 1) * 8));
      mma16816<T>(s[j], af[kk], b[0], b[1]);
      mma16816<T>(s[j + 1], af[kk], b[2], b[3]);
    }
}

// acc (16 x D per warp) += P (16 x BN, packed A fragments) . Xs, Xs stored [BN][PD].
template <typename T, int BN, int D, int PD>
__device__ __forceinline__ void pv_tile(float (&acc)[D / 8][4], const uint32_t (&pf)[BN / 16][4], const T* Xs, int lane) {
  const int l7 = lane & 7, mi4 = lane >> 3;
#pragma unroll
  for (int kk = 0; kk < BN / 16; ++kk)
#pragma unroll
    for (int j = 0; j < D / 8; j += 2) {
      uint32_t b[4];
      ldsm_x4_t(b, smem_u32(Xs + (kk * 16 + (mi4 & 1) * 8 + l7) * PD + j * 8 + (mi4 >> 1) * 8));
      mma16816<T>(acc[j], pf[kk], b[0], b[1]);
      mma16816<T>(acc[j + 1], pf[kk], b[2], b[3]);
    }
}

// Loads the 16 x D A-fragments of rows [r0, r0+16) of a tile stored [rows][PD].
template <typename T, int D, int PD>
__device__ __forceinline__ void load_a_frags(uint32_t (&af)[D / 16][4], const T* Xs, int r0, int lane) {
  const int l7 = lane & 7, mi4 = lane >> 3;
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk)
    ldsm_x4(af[kk], smem_u32(Xs + (r0 + (mi4 & 1) * 8 + l7) * PD + kk * 16 + (mi4 >> 1) * 8));
}

// Score -> pre-softmax value for element (grow, gcol): s*scale + rpe + kpm + am.
template <typename T>
__device__ __forceinline__ float apply_masks(float s, const AttnArgs& p, int z, int h, int grow, int gcol) {
  float f = s * p.scale;
  if (p.m.rpe) f += ldf(reinterpret_cast<const T*>(p.m.rpe) + z * p.m.rpe_sz + h * p.m.rpe_sh + (int64_t)grow * p.m.rpe_sr + gcol);
  if (p.m.kpm) {
    const float r = ldf(reinterpret_cast<const T*>(p.m.kpm) + z * p.m.kpm_sz + gcol);
    f += p.m.kpm_mul ? (r == 0.f ? kNegInfA : 0.f) : r;
  }
  if (p.m.am) {
    const float r = ldf(reinterpret_cast<const T*>(p.m.am) + (int64_t)grow * p.m.am_sr + gcol);
    f += p.m.am_mul ? (r == 0.f ? kNegInfA : 0.f) : r;
  }
  return f;
}

// ---------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------
template <typename T, int B, int D>
__global__ void __launch_bounds__(AttnCfg<B, D>::NT) attn_fwd_kernel(AttnArgs p) {
  using C = AttnCfg<B, D>;
  constexpr int BN = C::BN, PD = C::PD, NT = C::NT, NI = C::NI, DI = C::DI;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* Qs = reinterpret_cast<T*>(smem_raw);
  T* Ks = Qs + B * PD;                   // [2][BN][PD]
  T* Vs = Ks + 2 * BN * PD;              // [2][BN][PD]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const int z = blockIdx.y;
  const int ho = p.row_order[blockIdx.x];
  const int h = ho / p.nb, i = ho % p.nb;
  const int first = p.row_ptr[ho], count = p.row_ptr[ho + 1] - first;
  const bool has_mask = p.m.rpe || p.m.kpm || p.m.am;

  T* orow = reinterpret_cast<T*>(p.o_w) + z * p.o_sz + h * p.o_sh + ((int64_t)i * B + warp * 16) * p.o_sr;
  float* lrow = p.lse + ((int64_t)(z * p.H + h) * p.L + i * B + warp * 16);
  if (count == 0) {                      // block-row without any nonzero block: zeros, as the dsd product gives
    for (int e = lane; e < 16 * D; e += 32) orow[(e / D) * p.o_sr + e % D] = cvt_out<T>(0.f);
    if (lane < 16) lrow[lane] = kNegInfA;
    return;
  }
  const T* qg = reinterpret_cast<const T*>(p.q) + z * p.q_sz + h * p.q_sh + (int64_t)i * B * p.q_sr;
  const T* kg = reinterpret_cast<const T*>(p.k) + z * p.k_sz + h * p.k_sh;
  const T* vg = reinterpret_cast<const T*>(p.v) + z * p.v_sz + h * p.v_sh;

  auto issue = [&](int t, int stage) {
    const int j = p.blk_col[first + t / C::SUBS];
    const int64_t r0 = (int64_t)j * B + (t % C::SUBS) * BN;
    load_tile<T, BN, D, PD, NT>(Ks + stage * BN * PD, kg + r0 * p.k_sr, p.k_sr, tid, BN, D);
    load_tile<T, BN, D, PD, NT>(Vs + stage * BN * PD, vg + r0 * p.v_sr, p.v_sr, tid, BN, D);
  };

  load_tile<T, B, D, PD, NT>(Qs, qg, p.q_sr, tid, B, D);
  cp_async_commit();
  issue(0, 0);
  cp_async_commit();
  cp_async_wait<1>();
  __syncthreads();
  uint32_t qf[C::KD][4];
  load_a_frags<T, D, PD>(qf, Qs, warp * 16, lane);

  float oacc[DI][4];
#pragma unroll
  for (int j = 0; j < DI; ++j)
#pragma unroll
    for (int r = 0; r < 4; ++r) oacc[j][r] = 0.f;
  float mrow[2] = {kNegInfA, kNegInfA}, lsum[2] = {0.f, 0.f};
  const float sl2 = p.scale * kLog2e;
  const int grow0 = i * B + warp * 16 + g;

  const int ntiles = count * C::SUBS;
  for (int t = 0; t < ntiles; ++t) {
    if (t + 1 < ntiles) { issue(t + 1, (t + 1) & 1); cp_async_commit(); cp_async_wait<1>(); }
    else cp_async_wait<0>();
    __syncthreads();
    const T* ks = Ks + (t & 1) * BN * PD;
    const T* vs = Vs + (t & 1) * BN * PD;
    float s[NI][4];
    qk_tile<T, BN, D, PD>(s, qf, ks, lane);
    // values in the log2 domain: f * log2(e)
    if (has_mask) {
      const int gcol0 = p.blk_col[first + t / C::SUBS] * B + (t % C::SUBS) * BN + 2 * t4;
#pragma unroll
      for (int j = 0; j < NI; ++j)
#pragma unroll
        for (int r = 0; r < 4; ++r)
          s[j][r] = apply_masks<T>(s[j][r], p, z, h, grow0 + 8 * (r >> 1), gcol0 + j * 8 + (r & 1)) * kLog2e;
    } else {
#pragma unroll
      for (int j = 0; j < NI; ++j)
#pragma unroll
        for (int r = 0; r < 4; ++r) s[j][r] *= sl2;
    }
    float alpha[2];
#pragma unroll
    for (int hr = 0; hr < 2; ++hr) {
      float mx = mrow[hr];
#pragma unroll
      for (int j = 0; j < NI; ++j) mx = fmaxf(mx, fmaxf(s[j][2 * hr], s[j][2 * hr + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float msafe = mx == kNegInfA ? 0.f : mx;
      alpha[hr] = fast_exp2(mrow[hr] - msafe);     // 0 while the running max is still -inf
      mrow[hr] = mx;
      float rs = 0.f;
#pragma unroll
      for (int j = 0; j < NI; ++j) {
        s[j][2 * hr] = fast_exp2(s[j][2 * hr] - msafe);
        s[j][2 * hr + 1] = fast_exp2(s[j][2 * hr + 1] - msafe);
        rs += s[j][2 * hr] + s[j][2 * hr + 1];
      }
      lsum[hr] = lsum[hr] * alpha[hr] + rs;
    }
#pragma unroll
    for (int j = 0; j < DI; ++j) {
      oacc[j][0] *= alpha[0]; oacc[j][1] *= alpha[0];
      oacc[j][2] *= alpha[1]; oacc[j][3] *= alpha[1];
    }
    uint32_t pf[BN / 16][4];
#pragma unroll
    for (int kk = 0; kk < BN / 16; ++kk) {
      pf[kk][0] = pack2<T>(s[2 * kk][0], s[2 * kk][1]);
      pf[kk][1] = pack2<T>(s[2 * kk][2], s[2 * kk][3]);
      pf[kk][2] = pack2<T>(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pf[kk][3] = pack2<T>(s[2 * kk + 1][2], s[2 * kk + 1][3]);
    }
    pv_tile<T, BN, D, PD>(oacc, pf, vs, lane);
    __syncthreads();
  }
#pragma unroll
  for (int hr = 0; hr < 2; ++hr) {
    lsum[hr] += __shfl_xor_sync(0xffffffffu, lsum[hr], 1);
    lsum[hr] += __shfl_xor_sync(0xffffffffu, lsum[hr], 2);
  }
  // a row whose every entry is masked has l == 0: its output is zero and its log-sum-exp -inf
  // (the reference's softmax gives NaN there; the tcgen05 kernels agree with this choice)
  const float inv[2] = {lsum[0] > 0.f ? 1.f / lsum[0] : 0.f, lsum[1] > 0.f ? 1.f / lsum[1] : 0.f};
#pragma unroll
  for (int j = 0; j < DI; ++j) {
    *reinterpret_cast<uint32_t*>(orow + (int64_t)g * p.o_sr + j * 8 + 2 * t4) = pack2<T>(oacc[j][0] * inv[0], oacc[j][1] * inv[0]);
    *reinterpret_cast<uint32_t*>(orow + (int64_t)(g + 8) * p.o_sr + j * 8 + 2 * t4) = pack2<T>(oacc[j][2] * inv[1], oacc[j][3] * inv[1]);
  }
  if (t4 == 0) {
    // base-2 units, the domain the row maximum is tracked in: log2(sum_j 2^(f_j * log2 e))
    lrow[g] = lsum[0] > 0.f ? mrow[0] + log2f(lsum[0]) : kNegInfA;
    lrow[g + 8] = lsum[1] > 0.f ? mrow[1] + log2f(lsum[1]) : kNegInfA;
  }
}

// ---------------------------------------------------------------------------
// backward (1): delta[z, h, row] = sum_d O * dO
// ---------------------------------------------------------------------------
template <typename T, int D>
__global__ void attn_delta_kernel(AttnArgs p, int rows_total) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows_total) return;
  const int lane = threadIdx.x & 31;
  const int r = row % p.L, zh = row / p.L, h = zh % p.H, z = zh / p.H;
  const T* o = reinterpret_cast<const T*>(p.o) + z * p.o_sz + h * p.o_sh + (int64_t)r * p.o_sr;
  const T* d = reinterpret_cast<const T*>(p.dout) + z * p.do_sz + h * p.do_sh + (int64_t)r * p.do_sr;
  float acc = 0.f;
  for (int c = lane * 2; c < D; c += 64) {
    acc += ldf(o + c) * ldf(d + c) + ldf(o + c + 1) * ldf(d + c + 1);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) p.delta[row] = acc;
}

// The same with 16-byte loads: D / 8 lanes per row, several rows per warp.  Needs 16-byte
// aligned rows of O and dO (checked by the launcher).
template <typename T, int D>
__global__ void __launch_bounds__(256) attn_delta_vec_kernel(AttnArgs p, int rows_total) {
  constexpr int LPR = D / 8, RPW = 32 / LPR;
  const int lane = threadIdx.x & 31;
  const int row = (blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * RPW + lane / LPR;
  float acc = 0.f;
  if (row < rows_total) {
    const int r = row % p.L, zh = row / p.L, h = zh % p.H, z = zh / p.H;
    const T* o = reinterpret_cast<const T*>(p.o) + z * p.o_sz + h * p.o_sh + (int64_t)r * p.o_sr + (lane % LPR) * 8;
    const T* d = reinterpret_cast<const T*>(p.dout) + z * p.do_sz + h * p.do_sh + (int64_t)r * p.do_sr + (lane % LPR) * 8;
    const uint4 ov = __ldg(reinterpret_cast<const uint4*>(o)), dv = __ldg(reinterpret_cast<const uint4*>(d));
    const T* oe = reinterpret_cast<const T*>(&ov);
    const T* de = reinterpret_cast<const T*>(&dv);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc += ldf(oe + i) * ldf(de + i);
  }
#pragma unroll
  for (int off = LPR / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (row < rows_total && lane % LPR == 0) p.delta[row] = acc;
}

// ---------------------------------------------------------------------------
// backward (2): dK, dV of one block-column
// ---------------------------------------------------------------------------
template <typename T, int B, int D>
__global__ void __launch_bounds__(AttnCfg<B, D>::NT) attn_bwd_kv_kernel(AttnArgs p) {
  using C = AttnCfg<B, D>;
  // the streamed tile holds BM query rows; narrower for D = 128 to bound registers
  constexpr int BM = (D > 64 && B > 32) ? 32 : C::BN;
  constexpr int SUBS = B / BM, PD = C::PD, NT = C::NT, MI = BM / 8, DI = C::DI;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* Ks = reinterpret_cast<T*>(smem_raw);      // [B][PD]
  T* Vs = Ks + B * PD;                         // [B][PD]
  T* Qs = Vs + B * PD;                         // [2][BM][PD]
  T* Ds = Qs + 2 * BM * PD;                    // [2][BM][PD]
  float* Ls = reinterpret_cast<float*>(Ds + 2 * BM * PD);   // [2][BM] log-sum-exp
  float* Es = Ls + 2 * BM;                     // [2][BM] delta
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const int z = blockIdx.y;
  const int ho = p.col_order[blockIdx.x];
  const int h = ho / p.nb, j = ho % p.nb;
  const int first = p.col_ptr[ho], count = p.col_ptr[ho + 1] - first;
  const bool has_mask = p.m.rpe || p.m.kpm || p.m.am;
  const float sl2 = p.scale * kLog2e;

  T* dkrow = reinterpret_cast<T*>(p.dk) + ((int64_t)(z * p.H + h) * p.L + (int64_t)j * B + warp * 16) * D;
  T* dvrow = reinterpret_cast<T*>(p.dv) + ((int64_t)(z * p.H + h) * p.L + (int64_t)j * B + warp * 16) * D;
  if (count == 0) {
    for (int e = lane; e < 16 * D; e += 32) { dkrow[e] = cvt_out<T>(0.f); dvrow[e] = cvt_out<T>(0.f); }
    return;
  }
  const T* kg = reinterpret_cast<const T*>(p.k) + z * p.k_sz + h * p.k_sh + (int64_t)j * B * p.k_sr;
  const T* vg = reinterpret_cast<const T*>(p.v) + z * p.v_sz + h * p.v_sh + (int64_t)j * B * p.v_sr;
  const T* qg = reinterpret_cast<const T*>(p.q) + z * p.q_sz + h * p.q_sh;
  const T* dg = reinterpret_cast<const T*>(p.dout) + z * p.do_sz + h * p.do_sh;
  const float* lg = p.lse + (int64_t)(z * p.H + h) * p.L;
  const float* eg = p.delta + (int64_t)(z * p.H + h) * p.L;

  auto issue = [&](int t, int stage) {
    const int i = p.col_row[first + t / SUBS];
    const int64_t r0 = (int64_t)i * B + (t % SUBS) * BM;
    load_tile<T, BM, D, PD, NT>(Qs + stage * BM * PD, qg + r0 * p.q_sr, p.q_sr, tid, BM, D);
    load_tile<T, BM, D, PD, NT>(Ds + stage * BM * PD, dg + r0 * p.do_sr, p.do_sr, tid, BM, D);
    for (int e = tid; e < BM / 4; e += NT) {
      cp_async16(Ls + stage * BM + e * 4, lg + r0 + e * 4, true);
      cp_async16(Es + stage * BM + e * 4, eg + r0 + e * 4, true);
    }
  };

  load_tile<T, B, D, PD, NT>(Ks, kg, p.k_sr, tid, B, D);
  load_tile<T, B, D, PD, NT>(Vs, vg, p.v_sr, tid, B, D);
  cp_async_commit();
  issue(0, 0);
  cp_async_commit();
  cp_async_wait<1>();
  __syncthreads();
  uint32_t kf[C::KD][4], vf[C::KD][4];
  load_a_frags<T, D, PD>(kf, Ks, warp * 16, lane);
  load_a_frags<T, D, PD>(vf, Vs, warp * 16, lane);

  float dk[DI][4], dv[DI][4];
#pragma unroll
  for (int c = 0; c < DI; ++c)
#pragma unroll
    for (int r = 0; r < 4; ++r) { dk[c][r] = 0.f; dv[c][r] = 0.f; }
  const int gcol0 = j * B + warp * 16 + g;       // key index of this thread's rows (g, g + 8)

  const int ntiles = count * SUBS;
  for (int t = 0; t < ntiles; ++t) {
    if (t + 1 < ntiles) { issue(t + 1, (t + 1) & 1); cp_async_commit(); cp_async_wait<1>(); }
    else cp_async_wait<0>();
    __syncthreads();
    const T* qs = Qs + (t & 1) * BM * PD;
    const T* ds = Ds + (t & 1) * BM * PD;
    const float* ls = Ls + (t & 1) * BM;
    const float* es = Es + (t & 1) * BM;
    // S^T (16 keys x BM queries) and dP^T
    float st[MI][4], dp[MI][4];
    qk_tile<T, BM, D, PD>(st, kf, qs, lane);
    qk_tile<T, BM, D, PD>(dp, vf, ds, lane);
    const int grow0 = p.col_row[first + t / SUBS] * B + (t % SUBS) * BM + 2 * t4;
#pragma unroll
    for (int c = 0; c < MI; ++c)
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int m = c * 8 + 2 * t4 + (r & 1);            // query row inside the tile
        float pr;                                          // P = 2^(f * log2 e - lse)
        // (a query row without any visible key has lse = -inf: +inf makes its probabilities 0, not NaN)
        if (has_mask) pr = fast_exp2(fmaf(apply_masks<T>(st[c][r], p, z, h, grow0 + c * 8 + (r & 1), gcol0 + 8 * (r >> 1)), kLog2e,
                                          ls[m] == kNegInfA ? kNegInfA : -ls[m]));
        else pr = fast_exp2(fmaf(st[c][r], sl2, -ls[m]));
        st[c][r] = pr;
        dp[c][r] = pr * (dp[c][r] - es[m]) * p.scale;
      }
    uint32_t pf[BM / 16][4], sf[BM / 16][4];
#pragma unroll
    for (int kk = 0; kk < BM / 16; ++kk) {
      pf[kk][0] = pack2<T>(st[2 * kk][0], st[2 * kk][1]);
      pf[kk][1] = pack2<T>(st[2 * kk][2], st[2 * kk][3]);
      pf[kk][2] = pack2<T>(st[2 * kk + 1][0], st[2 * kk + 1][1]);
      pf[kk][3] = pack2<T>(st[2 * kk + 1][2], st[2 * kk + 1][3]);
      sf[kk][0] = pack2<T>(dp[2 * kk][0], dp[2 * kk][1]);
      sf[kk][1] = pack2<T>(dp[2 * kk][2], dp[2 * kk][3]);
      sf[kk][2] = pack2<T>(dp[2 * kk + 1][0], dp[2 * kk + 1][1]);
      sf[kk][3] = pack2<T>(dp[2 * kk + 1][2], dp[2 * kk + 1][3]);
    }
    pv_tile<T, BM, D, PD>(dv, pf, ds, lane);      // dV += P^T dO
    pv_tile<T, BM, D, PD>(dk, sf, qs, lane);      // dK += dS^T Q
    __syncthreads();
  }
#pragma unroll
  for (int c = 0; c < DI; ++c) {
    *reinterpret_cast<uint32_t*>(dkrow + g * D + c * 8 + 2 * t4) = pack2<T>(dk[c][0], dk[c][1]);
    *reinterpret_cast<uint32_t*>(dkrow + (g + 8) * D + c * 8 + 2 * t4) = pack2<T>(dk[c][2], dk[c][3]);
    *reinterpret_cast<uint32_t*>(dvrow + g * D + c * 8 + 2 * t4) = pack2<T>(dv[c][0], dv[c][1]);
    *reinterpret_cast<uint32_t*>(dvrow + (g + 8) * D + c * 8 + 2 * t4) = pack2<T>(dv[c][2], dv[c][3]);
  }
}

// ---------------------------------------------------------------------------
// backward (3): dQ of one block-row
// ---------------------------------------------------------------------------
template <typename T, int B, int D>
__global__ void __launch_bounds__(AttnCfg<B, D>::NT) attn_bwd_q_kernel(AttnArgs p) {
  using C = AttnCfg<B, D>;
  constexpr int BN = (D > 64 && B > 32) ? 32 : C::BN;
  constexpr int SUBS = B / BN, PD = C::PD, NT = C::NT, NI = BN / 8, DI = C::DI;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* Qs = reinterpret_cast<T*>(smem_raw);      // [B][PD]
  T* Ds = Qs + B * PD;                         // [B][PD]
  T* Ks = Ds + B * PD;                         // [2][BN][PD]
  T* Vs = Ks + 2 * BN * PD;                    // [2][BN][PD]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const int z = blockIdx.y;
  const int ho = p.row_order[blockIdx.x];
  const int h = ho / p.nb, i = ho % p.nb;
  const int first = p.row_ptr[ho], count = p.row_ptr[ho + 1] - first;
  const bool has_mask = p.m.rpe || p.m.kpm || p.m.am;

  const float sl2 = p.scale * kLog2e;
  T* dqrow = reinterpret_cast<T*>(p.dq) + ((int64_t)(z * p.H + h) * p.L + (int64_t)i * B + warp * 16) * D;
  if (count == 0) {
    for (int e = lane; e < 16 * D; e += 32) dqrow[e] = cvt_out<T>(0.f);
    return;
  }
  const T* qg = reinterpret_cast<const T*>(p.q) + z * p.q_sz + h * p.q_sh + (int64_t)i * B * p.q_sr;
  const T* dg = reinterpret_cast<const T*>(p.dout) + z * p.do_sz + h * p.do_sh + (int64_t)i * B * p.do_sr;
  const T* kg = reinterpret_cast<const T*>(p.k) + z * p.k_sz + h * p.k_sh;
  const T* vg = reinterpret_cast<const T*>(p.v) + z * p.v_sz + h * p.v_sh;

  auto issue = [&](int t, int stage) {
    const int j = p.blk_col[first + t / SUBS];
    const int64_t r0 = (int64_t)j * B + (t % SUBS) * BN;
    load_tile<T, BN, D, PD, NT>(Ks + stage * BN * PD, kg + r0 * p.k_sr, p.k_sr, tid, BN, D);
    load_tile<T, BN, D, PD, NT>(Vs + stage * BN * PD, vg + r0 * p.v_sr, p.v_sr, tid, BN, D);
  };
  load_tile<T, B, D, PD, NT>(Qs, qg, p.q_sr, tid, B, D);
  load_tile<T, B, D, PD, NT>(Ds, dg, p.do_sr, tid, B, D);
  cp_async_commit();
  issue(0, 0);
  cp_async_commit();
  cp_async_wait<1>();
  __syncthreads();
  uint32_t qf[C::KD][4], df[C::KD][4];
  load_a_frags<T, D, PD>(qf, Qs, warp * 16, lane);
  load_a_frags<T, D, PD>(df, Ds, warp * 16, lane);
  const int grow0 = i * B + warp * 16 + g;
  const int64_t zhl = (int64_t)(z * p.H + h) * p.L;
  float lse[2] = {p.lse[zhl + grow0], p.lse[zhl + grow0 + 8]};
  // (a query row without any visible key has lse = -inf: +inf makes its probabilities 0, not NaN)
  if (lse[0] == kNegInfA) lse[0] = -kNegInfA;
  if (lse[1] == kNegInfA) lse[1] = -kNegInfA;
  const float dlt[2] = {p.delta[zhl + grow0], p.delta[zhl + grow0 + 8]};

  float dq[DI][4];
#pragma unroll
  for (int c = 0; c < DI; ++c)
#pragma unroll
    for (int r = 0; r < 4; ++r) dq[c][r] = 0.f;

  const int ntiles = count * SUBS;
  for (int t = 0; t < ntiles; ++t) {
    if (t + 1 < ntiles) { issue(t + 1, (t + 1) & 1); cp_async_commit(); cp_async_wait<1>(); }
    else cp_async_wait<0>();
    __syncthreads();
    const T* ks = Ks + (t & 1) * BN * PD;
    const T* vs = Vs + (t & 1) * BN * PD;
    float s[NI][4], dp[NI][4];
    qk_tile<T, BN, D, PD>(s, qf, ks, lane);
    qk_tile<T, BN, D, PD>(dp, df, vs, lane);
    const int gcol0 = p.blk_col[first + t / SUBS] * B + (t % SUBS) * BN + 2 * t4;
#pragma unroll
    for (int c = 0; c < NI; ++c)
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        float pr;                                          // P = 2^(f * log2 e - lse)
        if (has_mask) pr = fast_exp2(fmaf(apply_masks<T>(s[c][r], p, z, h, grow0 + 8 * (r >> 1), gcol0 + c * 8 + (r & 1)), kLog2e, -lse[r >> 1]));
        else pr = fast_exp2(fmaf(s[c][r], sl2, -lse[r >> 1]));
        dp[c][r] = pr * (dp[c][r] - dlt[r >> 1]) * p.scale;
      }
    uint32_t sf[BN / 16][4];
#pragma unroll
    for (int kk = 0; kk < BN / 16; ++kk) {
      sf[kk][0] = pack2<T>(dp[2 * kk][0], dp[2 * kk][1]);
      sf[kk][1] = pack2<T>(dp[2 * kk][2], dp[2 * kk][3]);
      sf[kk][2] = pack2<T>(dp[2 * kk + 1][0], dp[2 * kk + 1][1]);
      sf[kk][3] = pack2<T>(dp[2 * kk + 1][2], dp[2 * kk + 1][3]);
    }
    pv_tile<T, BN, D, PD>(dq, sf, ks, lane);      // dQ += dS K
    __syncthreads();
  }
#pragma unroll
  for (int c = 0; c < DI; ++c) {
    *reinterpret_cast<uint32_t*>(dqrow + g * D + c * 8 + 2 * t4) = pack2<T>(dq[c][0], dq[c][1]);
    *reinterpret_cast<uint32_t*>(dqrow + (g + 8) * D + c * 8 + 2 * t4) = pack2<T>(dq[c][2], dq[c][3]);
  }
}

// ---------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------
template <typename K>
int set_smem(K kern, int bytes, const char* what) {
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "%s: cannot reserve %d bytes of shared memory: %s", what, bytes, cudaGetErrorString(e));
  }
  return BSP_OK;
}

inline int launched(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "%s launch failed: %s", what, cudaGetErrorString(e));
  return BSP_OK;
}

template <typename T, int B, int D>
int attn_fwd_launch(const AttnArgs& p, int Z, cudaStream_t st) {
  using C = AttnCfg<B, D>;
  const int bytes = (B + 4 * C::BN) * C::PD * int(sizeof(T));
  auto kern = attn_fwd_kernel<T, B, D>;
  if (int rc = set_smem(kern, bytes, "attention forward")) return rc;
  kern<<<dim3(p.H * p.nb, Z), C::NT, bytes, st>>>(p);
  return launched("attention forward");
}

template <typename T, int B, int D>
int attn_bwd_launch(const AttnArgs& p, int Z, int parts, cudaStream_t st) {
  using C = AttnCfg<B, D>;
  const int rows = Z * p.H * p.L;
  if (parts & 1) {
    const bool vec = ((reinterpret_cast<uintptr_t>(p.o) | reinterpret_cast<uintptr_t>(p.dout)) & 15) == 0 &&
                     ((p.o_sz | p.o_sh | p.o_sr | p.do_sz | p.do_sh | p.do_sr) & 7) == 0;
    constexpr int RPC = 8 * (32 / (D / 8));               // rows per CTA of the vector kernel
    if (vec) attn_delta_vec_kernel<T, D><<<(rows + RPC - 1) / RPC, 256, 0, st>>>(p, rows);
    else attn_delta_kernel<T, D><<<(rows + 7) / 8, 256, 0, st>>>(p, rows);
    if (int rc = launched("attention delta")) return rc;
  }
  constexpr int BT = (D > 64 && B > 32) ? 32 : C::BN;
  if (parts & 2) {
    const int bytes = (2 * B + 4 * BT) * C::PD * int(sizeof(T)) + 4 * BT * int(sizeof(float));
    auto kern = attn_bwd_kv_kernel<T, B, D>;
    if (int rc = set_smem(kern, bytes, "attention backward (dK, dV)")) return rc;
    kern<<<dim3(p.H * p.nb, Z), C::NT, bytes, st>>>(p);
    if (int rc = launched("attention backward (dK, dV)")) return rc;
  }
  if (parts & 4) {
    const int bytes = (2 * B + 4 * BT) * C::PD * int(sizeof(T));
    auto kern = attn_bwd_q_kernel<T, B, D>;
    if (int rc = set_smem(kern, bytes, "attention backward (dQ)")) return rc;
    kern<<<dim3(p.H * p.nb, Z), C::NT, bytes, st>>>(p);
    if (int rc = launched("attention backward (dQ)")) return rc;
  }
  return BSP_OK;
}

}  // namespace

template <typename T>
int attn_fwd_t(const AttnArgs& p, int block, int D, int Z, cudaStream_t st) {
#define BSP_ATTN_CASE(BB, DD) if (block == BB && D == DD) return attn_fwd_launch<T, BB, DD>(p, Z, st);
  BSP_ATTN_CASE(16, 64) BSP_ATTN_CASE(32, 64) BSP_ATTN_CASE(64, 64) BSP_ATTN_CASE(128, 64)
  BSP_ATTN_CASE(16, 128) BSP_ATTN_CASE(32, 128) BSP_ATTN_CASE(64, 128) BSP_ATTN_CASE(128, 128)
#undef BSP_ATTN_CASE
  return fail(BSP_ERR_UNSUPPORTED, "fused attention supports head dimensions 64 and 128 (got %d)", D);
}

template <typename T>
int attn_bwd_t(const AttnArgs& p, int block, int D, int Z, int parts, cudaStream_t st) {
#define BSP_ATTN_CASE(BB, DD) if (block == BB && D == DD) return attn_bwd_launch<T, BB, DD>(p, Z, parts, st);
  BSP_ATTN_CASE(16, 64) BSP_ATTN_CASE(32, 64) BSP_ATTN_CASE(64, 64) BSP_ATTN_CASE(128, 64)
  BSP_ATTN_CASE(16, 128) BSP_ATTN_CASE(32, 128) BSP_ATTN_CASE(64, 128) BSP_ATTN_CASE(128, 128)
#undef BSP_ATTN_CASE
  return fail(BSP_ERR_UNSUPPORTED, "fused attention supports head dimensions 64 and 128 (got %d)", D);
}

}  // namespace bsp
