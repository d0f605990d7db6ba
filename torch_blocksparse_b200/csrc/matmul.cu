// C-ABI entry points of the block-sparse matrix products: argument checks,
// metadata decoding and kernel family selection.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <atomic>
#include "common.h"

namespace bsp {

template <typename T>
int sdd_mma_t(const void* a, const void* b, void* c, int block, int Z, int K,
              int64_t a_sz, int64_t a_sh, int64_t a_sm, int64_t a_sk,
              int64_t b_sz, int64_t b_sh, int64_t b_sk, int64_t b_sn,
              int64_t c_sz, const Meta& m, cudaStream_t st);
template <typename T>
int dsd_mma_t(const void* s, const void* b, void* c, int block, int Z, int N,
              int64_t s_sz, int trans_s,
              int64_t b_sz, int64_t b_sh, int64_t b_sk, int64_t b_sn,
              int64_t c_sz, int64_t c_sh, int64_t c_sm, int64_t c_sn,
              const Meta& m, cudaStream_t st);

bool dsd_tc_eligible(const void* s, const void* b, const void* c, int dtype, int block, int N, int trans_s, int64_t s_sz,
                     int64_t b_sz, int64_t b_sh, int64_t b_sk, int64_t b_sn,
                     int64_t c_sz, int64_t c_sh, int64_t c_sm, int64_t c_sn);
int dsd_tc(const void* s, const void* b, void* c, int dtype, int block, int Z, int N, int64_t s_sz, int trans_s,
           int64_t b_sz, int64_t b_sh, int64_t b_sk, int64_t b_sn,
           int64_t c_sz, int64_t c_sh, int64_t c_sm, int64_t c_sn, const Meta& m, cudaStream_t st);

bool sdd_tc_eligible(const void* a, const void* b, const void* c, int dtype, int block, int K,
                     int64_t a_sz, int64_t a_sh, int64_t a_sm, int64_t a_sk,
                     int64_t b_sz, int64_t b_sh, int64_t b_sk, int64_t b_sn, int64_t c_sz);
int sdd_tc(const void* a, const void* b, void* c, int dtype, int block, int Z, int K,
           int64_t a_sz, int64_t a_sh, int64_t a_sm, int64_t a_sk,
           int64_t b_sz, int64_t b_sh, int64_t b_sk, int64_t b_sn, int64_t c_sz, const Meta& m, cudaStream_t st);

namespace {

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int decode_meta(const int32_t* hdr, const int32_t* dev, Meta& m) {
  if (!hdr || !dev) return fail(BSP_ERR_INVALID, "metadata pointer is NULL");
  if (hdr[0] != BSP_META_MAGIC) return fail(BSP_ERR_INVALID, "metadata header is corrupt (bad magic)");
  if (hdr[1] <= 0 || hdr[2] <= 0 || hdr[3] <= 0 || hdr[4] < 0) return fail(BSP_ERR_INVALID, "metadata header is corrupt");
  m = meta_view(dev, hdr[1], hdr[2], hdr[3], hdr[4], hdr[5], hdr[6]);
  return BSP_OK;
}

int check_basic(const char* op, int dtype, int block, int Z, int H, const Meta& m) {
  if (!valid_dtype(dtype)) return fail(BSP_ERR_INVALID, "%s: unknown dtype %d", op, dtype);
  if (!valid_block(block)) return fail(BSP_ERR_INVALID, "%s: block must be 16, 32, 64 or 128 (got %d)", op, block);
  if (Z <= 0 || Z > 65535) return fail(BSP_ERR_INVALID, "%s: batch %d outside [1, 65535]", op, Z);
  if (H != m.H) return fail(BSP_ERR_INVALID, "%s: operand has %d heads, layout has %d", op, H, m.H);
  return BSP_OK;
}

// A dense operand must have one unit inner stride; everything else has to keep
// 16-byte alignment for the vector copies.
int check_dense(const char* op, const char* name, const void* p, int dtype, int64_t sz, int64_t sh,
                int64_t s0, int64_t s1) {
  const int vec = dtype == BSP_F32 ? 4 : 8;
  if (!p) return fail(BSP_ERR_INVALID, "%s: %s is NULL", op, name);
  if (!aligned16(p)) return fail(BSP_ERR_INVALID, "%s: %s must be 16-byte aligned", op, name);
  if (s0 != 1 && s1 != 1) return fail(BSP_ERR_INVALID, "%s: %s needs a unit stride on one of its two inner dimensions", op, name);
  const int64_t other = s0 == 1 ? s1 : s0;
  if (sz % vec || sh % vec || (other != 1 && other % vec))
    return fail(BSP_ERR_INVALID, "%s: strides of %s must be multiples of %d elements", op, name, vec);
  return BSP_OK;
}

int check_sparse(const char* op, const char* name, const void* p, int dtype, int64_t sz) {
  const int vec = dtype == BSP_F32 ? 4 : 8;
  if (!p) return fail(BSP_ERR_INVALID, "%s: %s is NULL", op, name);
  if (!aligned16(p)) return fail(BSP_ERR_INVALID, "%s: %s must be 16-byte aligned", op, name);
  if (sz % vec) return fail(BSP_ERR_INVALID, "%s: batch stride of %s must be a multiple of %d elements", op, name, vec);
  return BSP_OK;
}

// Switch of the tcgen05 kernels for MatMul (on by default); see bsp_matmul_use_tcgen05.
std::atomic<int> g_matmul_tc{1};

int run_dsd(const void* s, const void* b, void* c, int dtype, int block, int Z, int N,
            int64_t s_sz, int trans_s,
            int64_t b_sz, int64_t b_sh, int64_t b_sk, int64_t b_sn,
            int64_t c_sz, int64_t c_sh, int64_t c_sm, int64_t c_sn,
            const Meta& m, cudaStream_t st) {
  // (a layout without any block has no sparse tensor to describe to the tensor-map encoder: the
  // mma.sync kernel writes the zeros)
  // (the tcgen05 kernel plans a tile with one bit per block of the reduction side, 1024 at most)
  if (g_matmul_tc.load() && m.nnz > 0 && (trans_s ? m.Mb : m.Nb) <= 1024 &&
      dsd_tc_eligible(s, b, c, dtype, block, N, trans_s, s_sz, b_sz, b_sh, b_sk, b_sn, c_sz, c_sh, c_sm, c_sn))
    return dsd_tc(s, b, c, dtype, block, Z, N, s_sz, trans_s, b_sz, b_sh, b_sk, b_sn, c_sz, c_sh, c_sm, c_sn, m, st);
  if (dtype == BSP_F32)
    return dsd_mma_t<float>(s, b, c, block, Z, N, s_sz, trans_s, b_sz, b_sh, b_sk, b_sn, c_sz, c_sh, c_sm, c_sn, m, st);
  if (dtype == BSP_F16)
    return dsd_mma_t<__half>(s, b, c, block, Z, N, s_sz, trans_s, b_sz, b_sh, b_sk, b_sn, c_sz, c_sh, c_sm, c_sn, m, st);
  return dsd_mma_t<__nv_bfloat16>(s, b, c, block, Z, N, s_sz, trans_s, b_sz, b_sh, b_sk, b_sn, c_sz, c_sh, c_sm, c_sn, m, st);
}

}  // namespace
}  // namespace bsp

using namespace bsp;

extern "C" int bsp_sdd(const void* a, const void* b, void* c, int dtype, int block,
                       int Z, int H, int K,
                       int64_t a_sz, int64_t a_sh, int64_t a_sm, int64_t a_sk,
                       int64_t b_sz, int64_t b_sh, int64_t b_sk, int64_t b_sn,
                       int64_t c_sz, const int32_t* meta_hdr, const int32_t* meta, void* stream) {
  Meta m;
  if (int rc = decode_meta(meta_hdr, meta, m)) return rc;
  if (int rc = check_basic("sdd", dtype, block, Z, H, m)) return rc;
  if (K <= 0 || K % 16) return fail(BSP_ERR_INVALID, "Reduction size for SDD must be a multiple of 16");
  if (int rc = check_dense("sdd", "a", a, dtype, a_sz, a_sh, a_sm, a_sk)) return rc;
  if (int rc = check_dense("sdd", "b", b, dtype, b_sz, b_sh, b_sk, b_sn)) return rc;
  if (int rc = check_sparse("sdd", "c", c, dtype, c_sz)) return rc;
  if (m.nnz == 0) return BSP_OK;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // (the tcgen05 kernel's grid: groups of 128 rows per head in y, the batch in z)
  if (g_matmul_tc.load() && Z <= 65535 && (int64_t)m.H * ((m.Mb * block + 127) / 128) <= 65535 &&
      sdd_tc_eligible(a, b, c, dtype, block, K, a_sz, a_sh, a_sm, a_sk, b_sz, b_sh, b_sk, b_sn, c_sz))
    return sdd_tc(a, b, c, dtype, block, Z, K, a_sz, a_sh, a_sm, a_sk, b_sz, b_sh, b_sk, b_sn, c_sz, m, st);
  if (dtype == BSP_F32)
    return sdd_mma_t<float>(a, b, c, block, Z, K, a_sz, a_sh, a_sm, a_sk, b_sz, b_sh, b_sk, b_sn, c_sz, m, st);
  if (dtype == BSP_F16)
    return sdd_mma_t<__half>(a, b, c, block, Z, K, a_sz, a_sh, a_sm, a_sk, b_sz, b_sh, b_sk, b_sn, c_sz, m, st);
  return sdd_mma_t<__nv_bfloat16>(a, b, c, block, Z, K, a_sz, a_sh, a_sm, a_sk, b_sz, b_sh, b_sk, b_sn, c_sz, m, st);
}

extern "C" int bsp_dsd(const void* s, const void* b, void* c, int dtype, int block,
                       int Z, int H, int N, int64_t s_sz, int trans_s,
                       int64_t b_sz, int64_t b_sh, int64_t b_sk, int64_t b_sn,
                       int64_t c_sz, int64_t c_sh, int64_t c_sm, int64_t c_sn,
                       const int32_t* meta_hdr, const int32_t* meta, void* stream) {
  Meta m;
  if (int rc = decode_meta(meta_hdr, meta, m)) return rc;
  if (int rc = check_basic("dsd", dtype, block, Z, H, m)) return rc;
  const int vec = dtype == BSP_F32 ? 4 : 8;
  if (N <= 0 || N % vec) return fail(BSP_ERR_INVALID, "dsd: dense width %d must be a positive multiple of %d", N, vec);
  if (m.nnz > 0)                 // (a layout without blocks has an empty sparse operand, never dereferenced)
    if (int rc = check_sparse("dsd", "a", s, dtype, s_sz)) return rc;
  if (int rc = check_dense("dsd", "b", b, dtype, b_sz, b_sh, b_sk, b_sn)) return rc;
  if (!c) return fail(BSP_ERR_INVALID, "dsd: c is NULL");
  return run_dsd(s, b, c, dtype, block, Z, N, s_sz, trans_s, b_sz, b_sh, b_sk, b_sn, c_sz, c_sh, c_sm, c_sn, m,
                 reinterpret_cast<cudaStream_t>(stream));
}

// C = A . op(S) is computed as C^T = op(S)^T . A^T: the sparse operand is used
// with the opposite transposition and the dense operand / result swap the
// roles of their two inner strides.
extern "C" int bsp_dds(const void* a, const void* s, void* c, int dtype, int block,
                       int Z, int H, int M,
                       int64_t a_sz, int64_t a_sh, int64_t a_sm, int64_t a_sk,
                       int64_t s_sz, int trans_s,
                       int64_t c_sz, int64_t c_sh, int64_t c_sm, int64_t c_sn,
                       const int32_t* meta_hdr, const int32_t* meta, void* stream) {
  Meta m;
  if (int rc = decode_meta(meta_hdr, meta, m)) return rc;
  if (int rc = check_basic("dds", dtype, block, Z, H, m)) return rc;
  const int vec = dtype == BSP_F32 ? 4 : 8;
  if (M <= 0 || M % vec) return fail(BSP_ERR_INVALID, "dds: dense height %d must be a positive multiple of %d", M, vec);
  if (int rc = check_dense("dds", "a", a, dtype, a_sz, a_sh, a_sm, a_sk)) return rc;
  if (m.nnz > 0)
    if (int rc = check_sparse("dds", "b", s, dtype, s_sz)) return rc;
  if (!c) return fail(BSP_ERR_INVALID, "dds: c is NULL");
  return run_dsd(s, a, c, dtype, block, Z, M, s_sz, !trans_s, a_sz, a_sh, a_sk, a_sm, c_sz, c_sh, c_sn, c_sm, m,
                 reinterpret_cast<cudaStream_t>(stream));
}

// Chooses the kernel family of MatMul for block 64 / 128 with FP16 / BF16 operands: non-zero
// (default) lets the eligible cases run on the tcgen05 kernels, zero keeps everything on the
// mma.sync kernels.  Process-wide; meant for comparisons and tests.
extern "C" int bsp_matmul_use_tcgen05(int enable) {
  g_matmul_tc.store(enable ? 1 : 0);
  return BSP_OK;
}
