// Fused block-sparse self-attention on the Blackwell tensor path: tcgen05.mma
// with accumulators in tensor memory, operands brought in by TMA.
//
// Same contract as the mma.sync kernels of attn_impl.cuh (which replace the
// sdd -> softmax -> dsd chain of
// torch_blocksparse/deepspeedsparseselfattention.py:157-166); this path covers
// block 64 and 128, head dimension 64 and 128, FP16 / BF16, without rpe / masks.
//
// Geometry: every MMA has M = 128.  A CTA owns a tile of 128 query rows (two
// block-rows of the layout when block = 64, see bsp_attn_tiles_build) and walks
// the tile's list of 64-row key chunks:
//     S[128 x 64]  = Q . K_chunk^T          (A, B from shared memory, K-major)
//     P            = 2^(S*c - m)            (registers; one thread per query row)
//     O[128 x D]  += P . V_chunk            (A = P from tensor memory, B MN-major)
// S, P and O live in tensor memory (S: 64 columns, P packed over the first 32
// of them, O: D columns).  Because P reuses the columns of S, the next S is
// only issued once the product that reads P has completed.  The running maximum is only raised when it grows by
// more than 2^8 ("lazy rescale"), so O is almost never read back before the end.
// For block = 64 a 2-bit mask per chunk says which half of the tile owns the
// block; the other half sees -inf.
//
// 128 threads per CTA (thread r = query row r = TMEM lane r); thread 0 also
// issues the TMA loads and the MMAs.  Several CTAs per SM overlap one CTA's
// exponentials with another's MMAs.  All waits are bounded (tc.cuh).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "common.h"
#include "tc.cuh"
#include "tile.cuh"

namespace bsp {

// Set by a kernel whose bounded wait expired; read by bsp_device_status().
static __device__ int g_tc_status;

namespace {

using namespace tc;

constexpr float kLog2eT = 1.4426950408889634f;
constexpr float kNegInfT = -__builtin_huge_valf();
constexpr int kStagesFwd = 3;

struct TcFwdArgs {
  void* o; float* lse;
  int64_t o_sz, o_sh, o_sr;
  int H, L, tiles_per_head;
  float scale_log2;
  const int32_t *ptr, *chunk, *mask, *order;
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
template <typename T> struct IsBf16 { static constexpr int v = 0; };
template <> struct IsBf16<__nv_bfloat16> { static constexpr int v = 1; };

template <int D> struct FwdSmem {
  static constexpr int ATOMS = D / 64;                  // 64-element (128-byte) column groups
  static constexpr int Q_BYTES = ATOMS * 128 * 128;     // 128 rows
  static constexpr int KV_BYTES = ATOMS * 64 * 128;     // 64 rows
  static constexpr int TOTAL = Q_BYTES + kStagesFwd * 2 * KV_BYTES + 1024;   // + alignment slack
  static constexpr int TMEM_COLS = D == 64 ? 128 : 256; // S (64) + O (D), rounded to a power of two
};

template <typename T, int D>
__global__ void __launch_bounds__(128, 3) attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap mq,
                                                          const __grid_constant__ CUtensorMap mk,
                                                          const __grid_constant__ CUtensorMap mv, TcFwdArgs a) {
  using SM = FwdSmem<D>;
  constexpr int ATOMS = SM::ATOMS, ST = kStagesFwd;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024 - (saddr(smem_raw) & 1023)) & 1023);
  unsigned char* q_s = smem;
  unsigned char* k_s = q_s + SM::Q_BYTES;               // [ST][ATOMS][64 rows][128 B]
  unsigned char* v_s = k_s + ST * SM::KV_BYTES;
  __shared__ uint64_t bar_q, bar_kv[ST], bar_s, bar_pv;
  __shared__ uint32_t tmem_slot;
  __shared__ int failed;

  const int tid = threadIdx.x, warp = tid >> 5;
  const int z = blockIdx.y;
  const int ti = a.order[blockIdx.x];
  const int h = ti / a.tiles_per_head, t128 = ti % a.tiles_per_head;
  const int first = a.ptr[ti], ntiles = a.ptr[ti + 1] - first;
  const int row = t128 * 128 + tid;
  T* orow = reinterpret_cast<T*>(a.o) + z * a.o_sz + h * a.o_sh + (int64_t)row * a.o_sr;
  float* lse = a.lse + ((int64_t)(z * a.H + h) * a.L + row);
  if (ntiles == 0) {                                    // nothing attends: zeros, as the dsd product gives
#pragma unroll
    for (int c = 0; c < D; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(0, 0, 0, 0);
    *lse = kNegInfT;
    return;
  }
  if (tid == 0) {
    failed = 0;
    mbar_init(&bar_q, 1);
    for (int s = 0; s < ST; ++s) mbar_init(&bar_kv[s], 1);
    mbar_init(&bar_s, 1);
    mbar_init(&bar_pv, 1);
    mbar_init_fence();
    prefetch_map(&mq); prefetch_map(&mk); prefetch_map(&mv);
  }
  if (warp == 0) { tmem_alloc(&tmem_slot, SM::TMEM_COLS); tmem_relinquish(); }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t t_s = tmem, t_p = tmem, t_o = tmem + 64;
  const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
  volatile int* fl = &failed;

  auto load_kv = [&](int t) {                           // thread 0 only
    const int stage = t % ST;
    const int krow = a.chunk[first + t] * 64;
    mbar_expect_tx(&bar_kv[stage], 2 * SM::KV_BYTES);
#pragma unroll
    for (int at = 0; at < ATOMS; ++at) {
      tma_load_4d(k_s + stage * SM::KV_BYTES + at * 8192, &mk, &bar_kv[stage], at * 64, krow, h, z);
      tma_load_4d(v_s + stage * SM::KV_BYTES + at * 8192, &mv, &bar_kv[stage], at * 64, krow, h, z);
    }
  };
  const uint32_t idesc_qk = instr_desc(128, 64, 0, IsBf16<T>::v);
  const uint32_t idesc_pv = instr_desc(128, 64, 1, IsBf16<T>::v);
  auto issue_qk = [&](int t) {                          // thread 0 only: S = Q . K^T
    const int stage = t % ST;
    mbar_wait(&bar_kv[stage], (t / ST) & 1, fl);
    fence_after();
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const uint32_t off = (ks % 4) * 32;
      const uint64_t da = smem_desc(saddr(q_s + (ks / 4) * 16384) + off, 1024);
      const uint64_t db = smem_desc(saddr(k_s + stage * SM::KV_BYTES + (ks / 4) * 8192) + off, 1024);
      mma_ss(t_s, da, db, idesc_qk, ks > 0);
    }
    commit(&bar_s);
  };
  auto issue_pv = [&](int t) {                          // thread 0 only: O += P . V
    const int stage = t % ST;
#pragma unroll
    for (int at = 0; at < ATOMS; ++at)
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        const uint64_t db = smem_desc(saddr(v_s + stage * SM::KV_BYTES + at * 8192) + ks * 2048, 1024);
        mma_ts(t_o + at * 64, t_p + ks * 8, db, idesc_pv, (t > 0 || ks > 0) ? 1u : 0u);
      }
    commit(&bar_pv);
  };

  if (tid == 0) {
    mbar_expect_tx(&bar_q, SM::Q_BYTES);
#pragma unroll
    for (int at = 0; at < ATOMS; ++at) tma_load_4d(q_s + at * 16384, &mq, &bar_q, at * 64, t128 * 128, h, z);
    for (int t = 0; t < ST && t < ntiles; ++t) load_kv(t);
    mbar_wait(&bar_q, 0, fl);
    issue_qk(0);
  }

  float m_ref = kNegInfT, l = 0.f;
  const int half = warp >> 1;                           // which 64 rows of the tile this warp holds
  for (int t = 0; t < ntiles; ++t) {
    const bool valid = (a.mask[first + t] >> half) & 1;
    mbar_wait(&bar_s, t & 1, fl);
    fence_after();
    uint32_t sr[2][32];
    tmem_ld32(t_s + lane_base, sr[0]);
    tmem_ld32(t_s + lane_base + 32, sr[1]);
    tmem_ld_wait();
    float mt = kNegInfT;
    if (valid) {
#pragma unroll
      for (int i = 0; i < 64; ++i) mt = fmaxf(mt, __uint_as_float(sr[i >> 5][i & 31]));
      mt *= a.scale_log2;
    }
    // raise the reference maximum only when the row maximum outgrows it by 2^8
    const bool grow = mt > m_ref + 8.f;
    if (__any_sync(0xffffffffu, grow)) {
      const float m_new = grow ? mt : m_ref;
      const float alpha = grow ? fast_exp2(m_ref - m_new) : 1.f;   // 0 while m_ref is still -inf
      l *= alpha;
      if (t > 0) {
        // S(t) is complete, hence so is the earlier PV(t-1): O is stable
#pragma unroll
        for (int c = 0; c < D; c += 32) {
          uint32_t orr[32];
          tmem_ld32(t_o + lane_base + c, orr);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) orr[i] = __float_as_uint(__uint_as_float(orr[i]) * alpha);
          tmem_st32(t_o + lane_base + c, orr);
        }
        tmem_st_wait();
      }
      m_ref = m_new;
    }
    uint32_t pr[32];
    if (valid) {
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float p0 = fast_exp2(fmaf(__uint_as_float(sr[(2 * i) >> 5][(2 * i) & 31]), a.scale_log2, -m_ref));
        const float p1 = fast_exp2(fmaf(__uint_as_float(sr[(2 * i + 1) >> 5][(2 * i + 1) & 31]), a.scale_log2, -m_ref));
        sum += p0 + p1;
        pr[i] = pack16<T>(p0, p1);
      }
      l += sum;
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) pr[i] = 0u;
    }
    tmem_st32(t_p + lane_base, pr);
    tmem_st_wait();
    fence_before();
    __syncthreads();
    if (tid == 0) {
      fence_after();
      issue_pv(t);
      if (t + 1 < ntiles) {
        mbar_wait(&bar_pv, t & 1, fl);                  // P(t) shares its columns with S(t+1)
        issue_qk(t + 1);
      }
      // the stage of chunk t-1 is free (PV(t-1) completed before S(t) did): refill it
      if (t >= 1 && t - 1 + ST < ntiles) load_kv(t - 1 + ST);
    }
  }
  mbar_wait(&bar_pv, (ntiles - 1) & 1, fl);
  fence_after();
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int c = 0; c < D; c += 32) {
    uint32_t orr[32];
    tmem_ld32(t_o + lane_base + c, orr);
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
      uint4 v;
      v.x = pack16<T>(__uint_as_float(orr[i]) * inv, __uint_as_float(orr[i + 1]) * inv);
      v.y = pack16<T>(__uint_as_float(orr[i + 2]) * inv, __uint_as_float(orr[i + 3]) * inv);
      v.z = pack16<T>(__uint_as_float(orr[i + 4]) * inv, __uint_as_float(orr[i + 5]) * inv);
      v.w = pack16<T>(__uint_as_float(orr[i + 6]) * inv, __uint_as_float(orr[i + 7]) * inv);
      *reinterpret_cast<uint4*>(orow + c + i) = v;
    }
  }
  *lse = l > 0.f ? m_ref + log2f(l) : kNegInfT;
  fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, SM::TMEM_COLS);
  if (tid == 0 && failed) atomicExch(&g_tc_status, 1);
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

// [Z, H, L, D] operand with unit stride on D: box of 64 columns x `rows` rows.
int make_map_4d(CUtensorMap* m, const void* ptr, int dtype, int Z, int H, int L, int D,
                int64_t sz, int64_t sh, int64_t sr, int rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(BSP_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)L, (cuuint64_t)H, (cuuint64_t)Z};
  cuuint64_t strides[3] = {(cuuint64_t)sr * 2, (cuuint64_t)(H > 1 ? sh : (int64_t)L * sr) * 2,
                           (cuuint64_t)(Z > 1 ? sz : (int64_t)H * L * sr) * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)rows, 1, 1};
  cuuint32_t es[4] = {1, 1, 1, 1};
  CUresult r = fn(m, dtype == BSP_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                  const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(BSP_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return BSP_OK;
}

struct TilesView {
  int H, nb, block, tiles_per_head;
  const int32_t *rt_ptr, *rt_chunk, *rt_mask, *rt_order, *ct_ptr, *ct_chunk, *ct_mask, *ct_order;
};

int decode_tiles(const int32_t* hdr, const int32_t* dev, TilesView& v) {
  if (hdr[0] != BSP_TILES_MAGIC) return fail(BSP_ERR_INVALID, "attention tile lists: bad magic");
  v.H = hdr[1]; v.nb = hdr[2]; v.block = hdr[3]; v.tiles_per_head = hdr[4];
  const int64_t n = (int64_t)v.H * v.tiles_per_head, er = hdr[5], ec = hdr[6];
  const int32_t* p = dev + BSP_TILES_HEADER;
  v.rt_ptr = p; p += n + 1; v.rt_chunk = p; p += er; v.rt_mask = p; p += er; v.rt_order = p; p += n;
  v.ct_ptr = p; p += n + 1; v.ct_chunk = p; p += ec; v.ct_mask = p; p += ec; v.ct_order = p;
  return BSP_OK;
}

template <typename T, int D>
int launch_fwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const TcFwdArgs& a,
               int n_tiles, int Z, cudaStream_t st) {
  auto kern = attn_fwd_tc_kernel<T, D>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem<D>::TOTAL);
  if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "attention (tcgen05 forward): cannot reserve shared memory: %s", cudaGetErrorString(e));
  kern<<<dim3(n_tiles, Z), 128, FwdSmem<D>::TOTAL, st>>>(mq, mk, mv, a);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "attention (tcgen05 forward) launch failed: %s", cudaGetErrorString(e));
  return BSP_OK;
}

}  // namespace

// Forward on the tcgen05 path.  Preconditions (checked by the caller): dtype F16 / BF16,
// D in {64, 128}, block in {64, 128}, L multiple of 128, no rpe / masks, unit stride on D.
int attn_fwd_tc(const void* q, const void* k, const void* v, void* o, float* lse,
                int dtype, int Z, int H, int L, int D,
                int64_t q_sz, int64_t q_sh, int64_t q_sr, int64_t k_sz, int64_t k_sh, int64_t k_sr,
                int64_t v_sz, int64_t v_sh, int64_t v_sr, int64_t o_sz, int64_t o_sh, int64_t o_sr,
                const int32_t* tiles_hdr, const int32_t* tiles, float scale, cudaStream_t st) {
  TilesView tv;
  if (int rc = decode_tiles(tiles_hdr, tiles, tv)) return rc;
  if (tv.H != H || tv.nb * tv.block != L) return fail(BSP_ERR_INVALID, "attention tile lists do not fit %d heads of length %d", H, L);
  CUtensorMap mq, mk, mv;
  if (int rc = make_map_4d(&mq, q, dtype, Z, H, L, D, q_sz, q_sh, q_sr, 128)) return rc;
  if (int rc = make_map_4d(&mk, k, dtype, Z, H, L, D, k_sz, k_sh, k_sr, 64)) return rc;
  if (int rc = make_map_4d(&mv, v, dtype, Z, H, L, D, v_sz, v_sh, v_sr, 64)) return rc;
  TcFwdArgs a;
  a.o = o; a.lse = lse; a.o_sz = o_sz; a.o_sh = o_sh; a.o_sr = o_sr;
  a.H = H; a.L = L; a.tiles_per_head = tv.tiles_per_head; a.scale_log2 = scale * kLog2eT;
  a.ptr = tv.rt_ptr; a.chunk = tv.rt_chunk; a.mask = tv.rt_mask; a.order = tv.rt_order;
  const int n_tiles = H * tv.tiles_per_head;
  if (dtype == BSP_F16) {
    if (D == 64) return launch_fwd<__half, 64>(mq, mk, mv, a, n_tiles, Z, st);
    return launch_fwd<__half, 128>(mq, mk, mv, a, n_tiles, Z, st);
  }
  if (D == 64) return launch_fwd<__nv_bfloat16, 64>(mq, mk, mv, a, n_tiles, Z, st);
  return launch_fwd<__nv_bfloat16, 128>(mq, mk, mv, a, n_tiles, Z, st);
}

int tc_device_status(int* out) {
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int));
  if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "reading the device status failed: %s", cudaGetErrorString(e));
  *out = v;
  return BSP_OK;
}

}  // namespace bsp
