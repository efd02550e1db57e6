// PTX wrappers for the Blackwell (sm_100a) data path used by the large-M kernels: mbarriers with
// bounded waits, TMA tile loads, tensor-memory allocation, tcgen05.mma / commit / ld, and the
// shared-memory and instruction descriptors those take.
//
// Every wait here is bounded.  When a wait gives up, the kernel records a code in the device status word
// (read by zt_poll_device_status) and unwinds: roles stop issuing work, tensor memory is released
// and the kernel returns, so the context stays usable.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace zt {

// Address (device pointer) of the per-device status word kernels write when a wait expires:
// 0 = fine; else the code of the first wait that gave up.  Kernels get it as a parameter.
int *device_status_ptr();

enum DeviceStatus : int {
  kStatusOk = 0,
  kStatusProducerTimeout = 101,  // TMA producer waited for a free stage
  kStatusMmaTimeout = 102,       // MMA issuer waited for data
  kStatusEpilogueTimeout = 103,  // epilogue waited for the accumulator
  kStatusConvertTimeout = 104,   // dequant warps waited for a stage
  kStatusSelfTest = 199          // zt_selftest_expire_wait: the deliberately unanswered wait gave up
};

namespace tc {

constexpr uint32_t kSpinLimit = 1u << 20;  // try_wait polls before giving up (each poll may block ~us)

__device__ __forceinline__ void report_timeout(int *status, int code) {
  if (status) atomicCAS(status, 0, code);
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b32 r;\n\telect.sync r|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ---- mbarrier ---------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Returns false when the phase did not complete within the poll limit.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t limit = kSpinLimit) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t i = 0; i < limit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if (i > 64) __nanosleep(64);
  }
  return false;
}

// Variants that take the barrier's shared-window address (computed once outside a hot loop).
__device__ __forceinline__ bool mbar_wait_addr(uint32_t addr, uint32_t parity, uint32_t limit = kSpinLimit) {
  for (uint32_t i = 0; i < limit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if (i > 64) __nanosleep(64);
  }
  return false;
}
__device__ __forceinline__ bool mbar_test_addr(uint32_t addr, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(addr), "r"(parity)
      : "memory");
  return done != 0;
}
__device__ __forceinline__ void mbar_expect_tx_addr(uint32_t addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(addr), "r"(bytes) : "memory");
}

// Same with non-blocking polls (mbarrier.test_wait): the waiter notices the completed phase within a few tens of
// cycles instead of when a suspended try_wait returns, at the price of issue slots while it spins.  For single
// threads on the critical path of a pipeline.
__device__ __forceinline__ bool mbar_wait_spin(uint64_t *bar, uint32_t parity, uint32_t limit = kSpinLimit << 4) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t i = 0; i < limit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

// Same, for waits that are expected to last: each poll may suspend the warp for up to `hint_ns`
// (it wakes when the phase completes), so a waiting warp takes almost no issue slots.
__device__ __forceinline__ bool mbar_wait_suspend(uint64_t *bar, uint32_t parity, uint32_t sleep_ns = 100,
                                                  uint32_t hint_ns = 2000) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t i = 0; i < (kSpinLimit >> 3); ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity), "r"(hint_ns)
        : "memory");
    if (done) return true;
    if (i >= 2) __nanosleep(sleep_ns);   // a failed poll returns early more often than not: keep pollers off the issue slots
  }
  return false;
}

// ---- TMA ----------------------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

// 3-D tile load global -> shared (c0 innermost).
__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *m, uint64_t *bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// 2-D tile load global -> shared, completion counted in bytes on `bar`.  c0 is the innermost
// coordinate (must be a multiple of 16 bytes worth of elements), c1 the row.
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *m, uint64_t *bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void tma_load_2d_addr(uint32_t dst, const CUtensorMap *m, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

// ---- tensor memory ------------------------------------------------------------------------------
// Whole-warp calls.  `cols` is a power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t *slot_in_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot_in_smem)),
               "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Makes generic-proxy writes to shared memory visible to the async proxy (TMA / tcgen05 reads).
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- descriptors --------------------------------------------------------------------------------
// Shared-memory matrix descriptor for a K-major operand tile stored as rows of 128 bytes with the
// 128-byte swizzle (what a TMA load with CU_TENSOR_MAP_SWIZZLE_128B writes): 8-row groups are 1024
// bytes apart.  The tile base must be 1024-byte aligned; stepping along K inside the 128-byte row
// is done by adding the byte offset (>> 4) to the low word.
__device__ __forceinline__ uint64_t smem_desc_k_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);  // start address, bits [0,14)
  d |= (uint64_t)1 << 16;                       // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;             // stride byte offset: next 8-row group
  d |= (uint64_t)1 << 46;                       // descriptor version of sm_100
  d |= (uint64_t)2 << 61;                       // layout type: 128-byte swizzle
  return d;
}

// Instruction descriptor (dense, no negate, both operands K-major).
//   c_format: 1 = f32, 2 = s32.   a/b_format: kind::f16 -> 0 f16, 1 bf16;  kind::i8 -> 0 u8, 1 s8.
__host__ __device__ constexpr uint32_t instr_desc(uint32_t c_format, uint32_t a_format, uint32_t b_format, uint32_t m,
                                                  uint32_t n) {
  return (c_format << 4) | (a_format << 7) | (b_format << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// ---- MMA ------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on `bar` once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void mma_commit_addr(uint32_t bar_addr) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_addr) : "memory");
}
// The descriptor of smem_desc_k_sw128 put together from its constant high word and the start-address field.
__device__ __forceinline__ uint64_t smem_desc_from_words(uint32_t lo, uint32_t hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}

// ---- accumulator read-back ------------------------------------------------------------------------
// Each lane reads 32 consecutive 32-bit columns of its own TMEM lane (row).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

}  // namespace tc

// ---- host side: tensor maps ---------------------------------------------------------------------
// Encodes a 2-D row-major tensor map (inner extent `inner` elements of `elem_bytes`, `rows` rows,
// row pitch `pitch_bytes`) with a box of box_inner x box_rows and the 128-byte swizzle.  Returns
// ZT_SUCCESS or an error (message set).
// General form: `rank` dimensions (innermost first), `strides_bytes` for dimensions 1..rank-1 (multiples
// of 16), a box per dimension, with or without the 128-byte swizzle.  Out-of-bounds elements read as zero.
int make_tensor_map(CUtensorMap *out, const void *base, CUtensorMapDataType dtype, int rank, const uint64_t *dims,
                    const uint64_t *strides_bytes, const uint32_t *box, bool swizzle128);

int make_tensor_map_2d(CUtensorMap *out, const void *base, CUtensorMapDataType dtype, uint32_t elem_bytes,
                       uint64_t inner, uint64_t rows, uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_rows);

}  // namespace zt
