// Thin wrappers over the Blackwell (sm_100a) instructions the tcgen05 kernels
// use: mbarrier, TMA tile loads (cp.async.bulk.tensor), tensor-memory
// allocation / load / store, tcgen05.mma and its descriptors.
//
// Every wait is bounded: a wait that does not complete within its budget
// returns false, the caller records the failure in a status word and keeps its
// control flow (barriers included) intact, so a protocol error shows up as an
// error code, never as a hung GPU.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace bsp {
namespace tc {

#define BSP_DEVI __device__ __forceinline__

BSP_DEVI uint32_t saddr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// ---- mbarrier ---------------------------------------------------------------
BSP_DEVI void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(saddr(bar)), "r"(count));
}
BSP_DEVI void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
BSP_DEVI void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(saddr(bar)), "r"(bytes) : "memory");
}
BSP_DEVI bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(saddr(bar)), "r"(parity) : "memory");
  return ok != 0;
}
BSP_DEVI void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(saddr(bar)) : "memory");
}
// One arrival per warp, after all its lanes have finished (and fenced) their part: 32 lanes
// arriving on one barrier serialise in the shared-memory atomic unit.  The whole warp must call it.
BSP_DEVI void warp_arrive(uint64_t* bar, int lane) {
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
}
constexpr int kWaitBudget = 1 << 21;   // default number of try_wait attempts before a wait is declared failed
// `failed` points at two ints of the CTA's shared memory: [0] is set once a wait of the CTA has
// expired, [1] holds the number of attempts a wait may make (kWaitBudget unless the launch says
// otherwise).  Returns false when the phase did not complete in time, or soon after the CTA
// has failed (failed[0] != 0), so that a failed CTA drains quickly.
BSP_DEVI bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* failed) {
  if (mbar_try_wait(bar, parity)) return true;          // (the common case pays for nothing else)
  const int budget = failed[1];
  for (int i = 1; i < budget; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 1023) == 1023 && failed[0]) return false;
  }
  failed[0] = 1;
  return false;
}

// mbar_wait for a whole warp: the outcome is made uniform, so that a warp leaves its loop as one.
// (Every lane waits itself: with lane 0 waiting and a shuffle handing the outcome to the others the
// attention step was 9 % slower, dK/dV 16 %.)
BSP_DEVI bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile int* failed) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, failed));
}

// A whole warp waiting for something that takes long (a write-back warp waiting for a tile's
// products): lane 0 alone polls, with a pause between attempts, and shares the outcome, so
// that the waiting warps leave the shared-memory pipe and the issue slots to the others.
BSP_DEVI bool mbar_wait_warp_idle(uint64_t* bar, uint32_t parity, volatile int* failed, int lane) {
  int ok = 1;
  if (lane == 0) {
    ok = 0;
    const int budget = failed[1];
    for (int i = 0; i < budget; ++i) {
      if (mbar_try_wait(bar, parity)) { ok = 1; break; }
      if ((i & 63) == 63 && failed[0]) break;
      __nanosleep(128);
    }
    if (!ok) failed[0] = 1;
  }
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// ---- TMA ----------------------------------------------------------------------
BSP_DEVI void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
               ::"r"(saddr(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(saddr(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
// Plain (untiled) bulk copy global -> shared; both addresses 16-byte aligned, size a multiple of 16.
BSP_DEVI void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(saddr(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(saddr(bar)) : "memory");
}
// Makes this thread's earlier writes to shared memory visible to the asynchronous proxy (the
// tensor core reads MMA operands through it).
BSP_DEVI void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// Four consecutive FP32 values added to global memory in one reduction (16-byte aligned).
BSP_DEVI void red_add4(float* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
               ::"l"(p), "f"(__uint_as_float(a)), "f"(__uint_as_float(b)), "f"(__uint_as_float(c)), "f"(__uint_as_float(d)) : "memory");
}
BSP_DEVI void prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---- tensor memory ---------------------------------------------------------------
BSP_DEVI void tmem_alloc(uint32_t* slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(saddr(slot)), "r"(ncols) : "memory");
}
BSP_DEVI void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
BSP_DEVI void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
BSP_DEVI void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
BSP_DEVI void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
BSP_DEVI void commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(saddr(bar)) : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns; the warp reads its own quarter of the lanes
BSP_DEVI void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
               "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                 "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                 "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr) : "memory");
}
BSP_DEVI void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
               "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr) : "memory");
}
BSP_DEVI void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}
BSP_DEVI void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
               "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                 "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
BSP_DEVI void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
BSP_DEVI void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
               "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                 "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                 "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                 "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
}
BSP_DEVI void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---- tcgen05.mma ---------------------------------------------------------------
// High word of every shared-memory descriptor used here: 1024 bytes between 8-row
// groups (bits 32-45), descriptor version 1 (bit 46), 128-byte swizzle (bits 61-63).
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
// Low word: start address (bits 0-13, in 16-byte units) and the unused leading offset.
BSP_DEVI uint32_t desc_lo(uint32_t addr) { return ((addr & 0x3FFFF) >> 4) | (1u << 16); }

// D[tmem] (+)= A[smem] * B[smem]
BSP_DEVI void mma_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]; A holds two 16-bit values per 32-bit column
BSP_DEVI void mma_ts(uint32_t d, uint32_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
               ::"r"(d), "r"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}

// The same two products with the operand descriptors given as their low 32-bit
// words (see desc_lo): the high word is the same for every descriptor of these
// kernels, so an issue costs one add per operand instead of a 64-bit rebuild.
BSP_DEVI void mma_ss_lo(uint32_t d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "mov.b64 da, {%1, %5};\n\tmov.b64 db, {%2, %5};\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t}"
               ::"r"(d), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHi) : "memory");
}
BSP_DEVI void mma_ts_lo(uint32_t d, uint32_t a, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "mov.b64 db, {%2, %5};\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %3, p;\n\t}"
               ::"r"(d), "r"(a), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHi) : "memory");
}

// Issue forms for back-to-back issue with descriptors prepared in advance: nothing
// but the MMA itself sits between two issues.
BSP_DEVI void mma_ss_acc(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.eq.b32 p, 0, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d), "l"(a), "l"(b), "r"(idesc) : "memory");
}
BSP_DEVI void mma_ts_acc(uint32_t d, uint32_t a, uint64_t b, uint32_t idesc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.eq.b32 p, 0, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
               ::"r"(d), "r"(a), "l"(b), "r"(idesc) : "memory");
}
BSP_DEVI uint64_t desc_from_lo(uint32_t lo) { return (static_cast<uint64_t>(kDescHi) << 32) | lo; }

// Variants that always accumulate (no predicate set-up between back-to-back issues).
BSP_DEVI void mma_ss_lo_acc(uint32_t d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc) {
  asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.eq.b32 p, 0, 0;\n\t"
               "mov.b64 da, {%1, %4};\n\tmov.b64 db, {%2, %4};\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t}"
               ::"r"(d), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(kDescHi) : "memory");
}
BSP_DEVI void mma_ts_lo_acc(uint32_t d, uint32_t a, uint32_t b_lo, uint32_t idesc) {
  asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.eq.b32 p, 0, 0;\n\t"
               "mov.b64 db, {%2, %4};\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %3, p;\n\t}"
               ::"r"(d), "r"(a), "r"(b_lo), "r"(idesc), "r"(kDescHi) : "memory");
}

// Shared-memory operand descriptor for tiles in the 128-byte-swizzled layout TMA
// writes (rows of 128 bytes, groups of 8 rows = 1024 bytes).  `sbo` is the
// distance between consecutive 8-row groups.  For a K-major operand a row is an
// M/N index and holds 64 K-elements: one MMA (K = 16) reads 32 bytes of each
// row, so successive K-steps advance the start address by 32 bytes.  For an
// MN-major operand a row is a K index and holds 64 M/N-elements: one MMA reads
// 16 rows, successive K-steps advance the start address by 2048 bytes.
BSP_DEVI uint64_t smem_desc(uint32_t addr, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(1) << 16;                       // leading-dimension offset: unused for these layouts
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= static_cast<uint64_t>(1) << 46;                       // descriptor version of sm_100
  d |= static_cast<uint64_t>(2) << 61;                       // 128-byte swizzle
  return d;
}
// Instruction descriptor, kind::f16: FP16 (0) or BF16 (1) operands, FP32 accumulator.
BSP_DEVI uint32_t instr_desc(int M, int N, int b_mn_major, int bf16) {
  uint32_t d = 0;
  d |= 1u << 4;                                  // accumulator format: F32
  d |= static_cast<uint32_t>(bf16) << 7;         // A format
  d |= static_cast<uint32_t>(bf16) << 10;        // B format
  d |= static_cast<uint32_t>(b_mn_major) << 16;  // B is MN-major (A stays K-major)
  d |= static_cast<uint32_t>(N >> 3) << 17;
  d |= static_cast<uint32_t>(M >> 4) << 24;
  return d;
}

}  // namespace tc
}  // namespace bsp
