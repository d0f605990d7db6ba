// C-ABI entry points of the fused block-sparse self-attention.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <mutex>
#include "attn_impl.cuh"

// Scratch of the allocation-free backward (bsp_attn_bwd_static): one FP32 value
// per attention row.  It is part of the library image, so every GPU that loads
// the library holds these 4 MiB until the process exits.
static __device__ __align__(256) float g_static_delta[BSP_ATTN_STATIC_ROWS];

namespace bsp {

struct XtHost { const void* rpe; int64_t rpe_sz, rpe_sh, rpe_sr; const void* am; int64_t am_sr; int am_mode; };
int attn_fwd_tc(const void* q, const void* k, const void* v, void* o, float* lse,
                int dtype, int Z, int H, int L, int D,
                int64_t q_sz, int64_t q_sh, int64_t q_sr, int64_t k_sz, int64_t k_sh, int64_t k_sr,
                int64_t v_sz, int64_t v_sh, int64_t v_sr, int64_t o_sz, int64_t o_sh, int64_t o_sr,
                const int32_t* tiles_hdr, const int32_t* tiles, float scale,
                const void* kpm, int64_t kpm_sz, int kpm_mul, int causal, const XtHost* xt, cudaStream_t st);
int attn_bwd_tc(const void* q, const void* k, const void* v, const void* dout, const float* lse, const float* delta,
                void* dq, void* dk, void* dv, int dtype, int Z, int H, int L, int D,
                int64_t q_sz, int64_t q_sh, int64_t q_sr, int64_t k_sz, int64_t k_sh, int64_t k_sr,
                int64_t v_sz, int64_t v_sh, int64_t v_sr, int64_t do_sz, int64_t do_sh, int64_t do_sr,
                const int32_t* tiles_hdr, const int32_t* tiles, float scale,
                const void* kpm, int64_t kpm_sz, int kpm_mul, int causal, int parts, const XtHost* xt, int overlap,
                cudaStream_t st);
int tc_device_status(int* out);
int tc_debug_wait(int wait_budget, int skip_chunk);
int dsd_tc_device_status(int* out);
int sdd_tc_device_status(int* out);

namespace {

// The tcgen05 kernels cover FP16 / BF16 on 128-row tiles.  A key-padding mask, a relative
// position bias and an attention mask are taken when they can be fetched in 16-byte pieces
// (aligned base, strides that are multiples of 8 elements); an attention mask the caller vouches
// to be the causal one (flag 2) is derived from the indices instead of being read.
bool tc_eligible(const int32_t* tiles_hdr, const int32_t* tiles, int block, int L, int D,
                 const void* rpe, int64_t rpe_sz, int64_t rpe_sh, int64_t rpe_sr,
                 const void* kpm, int64_t kpm_sz, const void* am, int64_t am_sr) {
  if (!(tiles_hdr && tiles && (D == 64 || D == 128))) return false;
  // the lists were built for this block size (blocks 16 and 32 run on 64-wide lists with masks of 16 x 16 pieces)
  if (!((block == 16 || block == 32 || block == 64 || block == 128) && tiles_hdr[7] == block)) return false;
  if (kpm && ((reinterpret_cast<uintptr_t>(kpm) & 15) || (kpm_sz & 7))) return false;
  if (rpe && ((reinterpret_cast<uintptr_t>(rpe) & 15) || (rpe_sz & 7) || (rpe_sh & 7) || (rpe_sr & 7) ||
              rpe_sz < 0 || rpe_sh <= 0 || rpe_sr <= 0)) return false;
  if (am && ((reinterpret_cast<uintptr_t>(am) & 15) || (am_sr & 7) || am_sr <= 0)) return false;
  return true;
}

// rpe / attention mask of a call in the form the tcgen05 launchers take (a causal-flagged mask is not read).
XtHost xt_of(const void* rpe, int64_t rpe_sz, int64_t rpe_sh, int64_t rpe_sr, const void* am, int64_t am_sr, int am_mul) {
  XtHost x = {rpe, rpe_sz, rpe_sh, rpe_sr, nullptr, 0, 0};
  if (am && am_mul != 2) { x.am = am; x.am_sr = am_sr; x.am_mode = am_mul ? 2 : 1; }
  return x;
}

// Strides the tensor-map encoder takes: positive (an operand expanded over the batch or the heads
// has stride 0 and stays on the mma.sync kernels).
bool tma_strides(int Z, int H, int64_t sz, int64_t sh, int64_t sr) {
  return sr > 0 && (H == 1 || sh > 0) && (Z == 1 || sz > 0);
}

// Whether a backward may put its dQ kernel on a second stream (off inside bsp_attn_bwd_static).
thread_local int g_allow_overlap = 1;
struct NoOverlap {
  int saved;
  NoOverlap() : saved(g_allow_overlap) { g_allow_overlap = 0; }
  ~NoOverlap() { g_allow_overlap = saved; }
};

constexpr int kMaxDevices = 64;
std::mutex g_static_mutex;
float* g_static_delta_ptr[kMaxDevices] = {};   // device address of g_static_delta, per device

// Device address of the scratch array on the current device.  In host code the
// array's name is only a handle; the address a kernel can use comes from
// cudaGetSymbolAddress, looked up once per device with that device current.
int static_delta_address(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "attention (static scratch): cudaGetDevice failed: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(BSP_ERR_UNSUPPORTED, "attention (static scratch): device index %d is outside [0, %d)", dev, kMaxDevices);
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (!g_static_delta_ptr[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_delta);
    if (e != cudaSuccess || !ptr)
      return fail(BSP_ERR_CUDA, "attention (static scratch): cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    g_static_delta_ptr[dev] = static_cast<float*>(ptr);
  }
  *out = g_static_delta_ptr[dev];
  return BSP_OK;
}

bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int check_qkv(const char* name, const void* p, int64_t sz, int64_t sh, int64_t sr) {
  if (!p) return fail(BSP_ERR_INVALID, "attention: %s is NULL", name);
  if (!al16(p) || sz % 8 || sh % 8 || sr % 8)
    return fail(BSP_ERR_INVALID, "attention: %s must be 16-byte aligned with strides that are multiples of 8 elements", name);
  return BSP_OK;
}

int fill_common(AttnArgs& p, int dtype, int block, int Z, int H, int L, int D,
                const int32_t* hdr, const int32_t* meta, float scale,
                const void* rpe, int64_t rpe_sz, int64_t rpe_sh, int64_t rpe_sr,
                const void* kpm, int64_t kpm_sz, int kpm_mul,
                const void* am, int64_t am_sr, int am_mul) {
  if (dtype != BSP_F16 && dtype != BSP_BF16)
    return fail(BSP_ERR_UNSUPPORTED, "fused attention supports FP16 and BF16 (use the three-op chain for FP32)");
  if (!valid_block(block)) return fail(BSP_ERR_INVALID, "attention: block must be 16, 32, 64 or 128 (got %d)", block);
  if (D != 64 && D != 128) return fail(BSP_ERR_UNSUPPORTED, "fused attention supports head dimensions 64 and 128 (got %d)", D);
  if (Z <= 0 || Z > 65535) return fail(BSP_ERR_INVALID, "attention: batch %d outside [1, 65535]", Z);
  if (!hdr || !meta) return fail(BSP_ERR_INVALID, "attention: metadata pointer is NULL");
  if (hdr[0] != BSP_META_MAGIC) return fail(BSP_ERR_INVALID, "attention: metadata header is corrupt (bad magic)");
  if (hdr[1] != H || hdr[2] != hdr[3] || hdr[2] * block != L)
    return fail(BSP_ERR_INVALID, "attention: layout [%d,%d,%d] with block %d does not fit %d heads of length %d",
                hdr[1], hdr[2], hdr[3], block, H, L);
  Meta m = meta_view(meta, hdr[1], hdr[2], hdr[3], hdr[4], hdr[5], hdr[6]);
  p.H = H; p.L = L; p.nb = L / block; p.scale = scale;
  p.row_ptr = m.row_ptr; p.blk_col = m.blk_col; p.row_order = m.row_order;
  p.col_ptr = m.col_ptr; p.col_row = m.col_row; p.col_order = m.col_order;
  p.m.rpe = rpe; p.m.rpe_sz = rpe_sz; p.m.rpe_sh = rpe_sh; p.m.rpe_sr = rpe_sr;
  p.m.kpm = kpm; p.m.kpm_sz = kpm_sz; p.m.kpm_mul = kpm_mul;
  p.m.am = am; p.m.am_sr = am_sr; p.m.am_mul = am_mul;
  return BSP_OK;
}

}  // namespace
}  // namespace bsp

using namespace bsp;

extern "C" int bsp_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                            int dtype, int block, int Z, int H, int L, int D,
                            int64_t q_sz, int64_t q_sh, int64_t q_sr,
                            int64_t k_sz, int64_t k_sh, int64_t k_sr,
                            int64_t v_sz, int64_t v_sh, int64_t v_sr,
                            int64_t o_sz, int64_t o_sh, int64_t o_sr,
                            const int32_t* meta_hdr, const int32_t* meta,
                            const int32_t* tiles_hdr, const int32_t* tiles, float scale,
                            const void* rpe, int64_t rpe_sz, int64_t rpe_sh, int64_t rpe_sr,
                            const void* kpm, int64_t kpm_sz, int kpm_mul,
                            const void* am, int64_t am_sr, int am_mul, void* stream) {
  AttnArgs p = {};
  if (int rc = fill_common(p, dtype, block, Z, H, L, D, meta_hdr, meta, scale, rpe, rpe_sz, rpe_sh, rpe_sr,
                           kpm, kpm_sz, kpm_mul, am, am_sr, am_mul)) return rc;
  if (int rc = check_qkv("q", q, q_sz, q_sh, q_sr)) return rc;
  if (int rc = check_qkv("k", k, k_sz, k_sh, k_sr)) return rc;
  if (int rc = check_qkv("v", v, v_sz, v_sh, v_sr)) return rc;
  if (int rc = check_qkv("o", o, o_sz, o_sh, o_sr)) return rc;
  if (!lse) return fail(BSP_ERR_INVALID, "attention: lse is NULL");
  p.q = q; p.k = k; p.v = v; p.o_w = o; p.lse = lse;
  p.q_sz = q_sz; p.q_sh = q_sh; p.q_sr = q_sr; p.k_sz = k_sz; p.k_sh = k_sh; p.k_sr = k_sr;
  p.v_sz = v_sz; p.v_sh = v_sh; p.v_sr = v_sr; p.o_sz = o_sz; p.o_sh = o_sh; p.o_sr = o_sr;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (tc_eligible(tiles_hdr, tiles, block, L, D, rpe, rpe_sz, rpe_sh, rpe_sr, kpm, kpm_sz, am, am_sr) &&
      tma_strides(Z, H, q_sz, q_sh, q_sr) && tma_strides(Z, H, k_sz, k_sh, k_sr) && tma_strides(Z, H, v_sz, v_sh, v_sr)) {
    const XtHost xt = xt_of(rpe, rpe_sz, rpe_sh, rpe_sr, am, am_sr, am_mul);
    return attn_fwd_tc(q, k, v, o, lse, dtype, Z, H, L, D, q_sz, q_sh, q_sr, k_sz, k_sh, k_sr, v_sz, v_sh, v_sr,
                       o_sz, o_sh, o_sr, tiles_hdr, tiles, scale, kpm, kpm_sz, kpm_mul, am != nullptr && am_mul == 2, &xt, st);
  }
  if (dtype == BSP_F16) return attn_fwd_t<__half>(p, block, D, Z, st);
  return attn_fwd_t<__nv_bfloat16>(p, block, D, Z, st);
}

extern "C" int bsp_attn_bwd_parts(const void* q, const void* k, const void* v, const void* o,
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
                            const void* am, int64_t am_sr, int am_mul, int parts, void* stream) {
  if (parts <= 0 || parts > 7) return fail(BSP_ERR_INVALID, "attention: parts must be a bit mask in [1, 7]");
  AttnArgs p = {};
  if (int rc = fill_common(p, dtype, block, Z, H, L, D, meta_hdr, meta, scale, rpe, rpe_sz, rpe_sh, rpe_sr,
                           kpm, kpm_sz, kpm_mul, am, am_sr, am_mul)) return rc;
  if (int rc = check_qkv("q", q, q_sz, q_sh, q_sr)) return rc;
  if (int rc = check_qkv("k", k, k_sz, k_sh, k_sr)) return rc;
  if (int rc = check_qkv("v", v, v_sz, v_sh, v_sr)) return rc;
  if (int rc = check_qkv("o", o, o_sz, o_sh, o_sr)) return rc;
  if (int rc = check_qkv("do", dout, do_sz, do_sh, do_sr)) return rc;
  if (!lse || !delta) return fail(BSP_ERR_INVALID, "attention: lse or delta is NULL");
  if (!al16(lse) || !al16(delta)) return fail(BSP_ERR_INVALID, "attention: lse and delta must be 16-byte aligned");
  if (!dq || !dk || !dv || !al16(dq) || !al16(dk) || !al16(dv))
    return fail(BSP_ERR_INVALID, "attention: dq, dk, dv must be non-NULL and 16-byte aligned");
  p.q = q; p.k = k; p.v = v; p.o = o; p.dout = dout;
  p.lse = const_cast<float*>(lse); p.delta = delta; p.dq = dq; p.dk = dk; p.dv = dv;
  p.q_sz = q_sz; p.q_sh = q_sh; p.q_sr = q_sr; p.k_sz = k_sz; p.k_sh = k_sh; p.k_sr = k_sr;
  p.v_sz = v_sz; p.v_sh = v_sh; p.v_sr = v_sr; p.o_sz = o_sz; p.o_sh = o_sh; p.o_sr = o_sr;
  p.do_sz = do_sz; p.do_sh = do_sh; p.do_sr = do_sr;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (tc_eligible(tiles_hdr, tiles, block, L, D, rpe, rpe_sz, rpe_sh, rpe_sr, kpm, kpm_sz, am, am_sr) &&
      tma_strides(Z, H, q_sz, q_sh, q_sr) && tma_strides(Z, H, k_sz, k_sh, k_sr) && tma_strides(Z, H, v_sz, v_sh, v_sr) &&
      tma_strides(Z, H, do_sz, do_sh, do_sr)) {
    // delta = rowsum(o * do) by the streaming kernel, the two matrix kernels on tcgen05
    if (parts & 1) {
      const int rc = dtype == BSP_F16 ? attn_bwd_t<__half>(p, block, D, Z, 1, st) : attn_bwd_t<__nv_bfloat16>(p, block, D, Z, 1, st);
      if (rc) return rc;
    }
    if (!(parts & 6)) return BSP_OK;
    const XtHost xt = xt_of(rpe, rpe_sz, rpe_sh, rpe_sr, am, am_sr, am_mul);
    return attn_bwd_tc(q, k, v, dout, lse, delta, dq, dk, dv, dtype, Z, H, L, D, q_sz, q_sh, q_sr, k_sz, k_sh, k_sr,
                       v_sz, v_sh, v_sr, do_sz, do_sh, do_sr, tiles_hdr, tiles, scale, kpm, kpm_sz, kpm_mul,
                       am != nullptr && am_mul == 2, parts & 6, &xt, g_allow_overlap, st);
  }
  if (dtype == BSP_F16) return attn_bwd_t<__half>(p, block, D, Z, parts, st);
  return attn_bwd_t<__nv_bfloat16>(p, block, D, Z, parts, st);
}

extern "C" int bsp_attn_bwd(const void* q, const void* k, const void* v, const void* o,
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
                            const void* am, int64_t am_sr, int am_mul, void* stream) {
  return bsp_attn_bwd_parts(q, k, v, o, dout, lse, delta, dq, dk, dv, dtype, block, Z, H, L, D,
                            q_sz, q_sh, q_sr, k_sz, k_sh, k_sr, v_sz, v_sh, v_sr, o_sz, o_sh, o_sr,
                            do_sz, do_sh, do_sr, meta_hdr, meta, tiles_hdr, tiles, scale, rpe, rpe_sz, rpe_sh, rpe_sr,
                            kpm, kpm_sz, kpm_mul, am, am_sr, am_mul, 7, stream);
}

extern "C" int bsp_attn_bwd_static(const void* q, const void* k, const void* v, const void* o,
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
                                   const void* am, int64_t am_sr, int am_mul, void* stream) {
  if (Z <= 0 || H <= 0 || L <= 0) return fail(BSP_ERR_INVALID, "attention (static scratch): non-positive size");
  const int64_t rows = (int64_t)Z * H * L;
  if (rows > BSP_ATTN_STATIC_ROWS)
    return fail(BSP_ERR_UNSUPPORTED,
                "attention (static scratch): Z*H*L = %lld rows exceed the built-in scratch of %d rows; "
                "use bsp_attn_bwd with caller-provided scratch", (long long)rows, BSP_ATTN_STATIC_ROWS);
  float* delta = nullptr;
  if (int rc = static_delta_address(&delta)) return rc;
  // (one stream only: creating the second stream of bsp_attn_bwd would allocate)
  NoOverlap guard;
  return bsp_attn_bwd_parts(q, k, v, o, dout, lse, delta, dq, dk, dv, dtype, block, Z, H, L, D,
                            q_sz, q_sh, q_sr, k_sz, k_sh, k_sr, v_sz, v_sh, v_sr, o_sz, o_sh, o_sr,
                            do_sz, do_sh, do_sr, meta_hdr, meta, tiles_hdr, tiles, scale, rpe, rpe_sz, rpe_sh, rpe_sr,
                            kpm, kpm_sz, kpm_mul, am, am_sr, am_mul, 7, stream);
}

extern "C" int bsp_device_status(int* status) {
  if (!status) return fail(BSP_ERR_INVALID, "status is NULL");
  int attn = 0, dsd = 0, sdd = 0;
  if (int rc = tc_device_status(&attn)) return rc;
  if (int rc = dsd_tc_device_status(&dsd)) return rc;
  if (int rc = sdd_tc_device_status(&sdd)) return rc;
  *status = attn ? attn : (dsd ? dsd : sdd);
  if (*status)
    return fail(BSP_ERR_TIMEOUT, "a bounded wait expired inside a tcgen05 kernel (%s): the outputs of that launch are not valid",
                attn == 1 ? "attention forward" : attn == 2 ? "attention dQ" : attn == 3 ? "attention dK/dV" : dsd ? "dsd / dds" : "sdd");
  return BSP_OK;
}

extern "C" int bsp_debug_attn_wait(int wait_budget, int skip_chunk) { return tc_debug_wait(wait_budget, skip_chunk); }
