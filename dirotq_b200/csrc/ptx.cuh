// Thin inline-PTX layer for sm_100a: mbarrier, TMA (no cluster broadcast forms), tcgen05
// (TMEM allocation, UMMA issue/commit, TMEM loads, smem->TMEM copies) and descriptor builders.
// Every wait in this file is bounded: a wait that runs out records a code and returns false so
// the kernel can unwind (drain its copies, free TMEM) instead of spinning forever.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include <cuda_bf16.h>

namespace dq {

// ---- error codes written to the status word (first error wins) -------------------------------
enum : int {
  ERR_NONE = 0,
  ERR_WAIT_FULL = 1,      // consumer waited for a filled smem stage
  ERR_WAIT_EMPTY = 2,     // producer waited for a free smem stage
  ERR_WAIT_ACC_FULL = 3,  // epilogue waited for an accumulator
  ERR_WAIT_ACC_EMPTY = 4, // MMA issuer waited for a drained accumulator
  ERR_WAIT_DRAIN = 5,     // teardown waited for copies in flight
  ERR_WAIT_SF = 6,        // scale factors: mover waited for the tiles, or the issuer for the movers
};

// ~1.5 s at the boost clock; clock64() ticks at the SM clock.
constexpr long long kWaitLimitCycles = 3000000000LL;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier ----------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// adds to the pending byte count without arriving
__device__ __forceinline__ void mbar_expect_tx_only(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// One poll.  `suspend_ns` is the hardware suspend-time hint: the thread sleeps inside the instruction
// (no issue slots used) until the phase completes or roughly that long has passed.
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity, uint32_t suspend_ns = 0) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(suspend_ns)
      : "memory");
  return ok != 0;
}
// Four phase tests issued back to back, so that their latencies overlap (a test costs about a hundred
// cycles even when the phase has long completed).  Bit i of the result: barrier i's phase is complete.
__device__ __forceinline__ uint32_t mbar_test4(uint32_t b0, uint32_t p0, uint32_t b1, uint32_t p1, uint32_t b2, uint32_t p2,
                                               uint32_t b3, uint32_t p3) {
  uint32_t m;
  asm volatile(
      "{\n\t.reg .pred q0, q1, q2, q3;\n\t.reg .u32 t0, t1, t2, t3;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 q0, [%1], %2;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 q1, [%3], %4;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 q2, [%5], %6;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 q3, [%7], %8;\n\t"
      "selp.u32 t0, 1, 0, q0;\n\t"
      "selp.u32 t1, 2, 0, q1;\n\t"
      "selp.u32 t2, 4, 0, q2;\n\t"
      "selp.u32 t3, 8, 0, q3;\n\t"
      "or.b32 t0, t0, t1;\n\t"
      "or.b32 t2, t2, t3;\n\t"
      "or.b32 %0, t0, t2;\n\t}"
      : "=r"(m)
      : "r"(b0), "r"(p0), "r"(b1), "r"(p1), "r"(b2), "r"(p2), "r"(b3), "r"(p3)
      : "memory");
  return m;
}

// Bounded wait.  Waiters sleep in hardware (20 us per poll) instead of spinning, so they do not
// compete with the working warps for issue slots; between polls the shared abort flag and the clock
// are checked.  `abort_flag` lives in shared memory: once any role gave up, all later waits of the
// CTA return at once.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int code) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
    if (mbar_try(bar, parity, 20000u)) return true;
    __nanosleep(128);            // keep pollers off the issue ports of the working warps
    if (*abort_flag) return false;
    // abort_flag[1]: the launch's wait limit in units of 1024 cycles (0 = the default above)
    const long long limit = abort_flag[1] > 0 ? ((long long)abort_flag[1] << 10) : kWaitLimitCycles;
    if (clock64() - t0 > limit) {
      *abort_flag = 1;
      if (status) atomicCAS(status, 0, code);
      return false;
    }
  }
}

// Bounded wait for roles on the critical path (a stage hand-off every few hundred cycles): polls
// back to back for a while -- a suspended waiter wakes up too late for such short intervals -- and
// only then falls into the sleeping loop of mbar_wait.
__device__ __forceinline__ bool mbar_wait_hot(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                              int* status, int code) {
#pragma unroll 1
  for (int i = 0; i < 4096; ++i)
    if (mbar_try(bar, parity)) return true;
  return mbar_wait(bar, parity, abort_flag, status, code);
}

// GELU, tanh form (torch.nn.functional.gelu(approximate="tanh")), applied to a value that was first rounded
// to bf16 -- the tensor the reference's activation module sees -- with the hardware tanh (relative error about
// 2^-11, below the bf16 rounding of the result).
__device__ __forceinline__ float gelu_tanh_bf16(float x) {
  x = __bfloat162float(__float2bfloat16_rn(x));
  const float u = 0.7978845608028654f * __fmaf_rn(0.044715f * x * x, x, x);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  return 0.5f * x * (1.f + t);
}

// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute may start
// (and run its prologue: barrier init, TMEM allocation, descriptor prefetch) while the previous kernel of the
// stream is still finishing.  pdl_wait() returns once that kernel has completed and its writes are visible;
// nothing may touch global memory before it.  pdl_launch_dependents() lets the NEXT kernel start early.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// generic-proxy writes to smem -> visible to the async proxy (UMMA / TMA reads)
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- TMA ---------------------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tmap(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}
// 2-D tiled load, completion on an mbarrier of this CTA.  x = innermost coordinate (elements).
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(tmap), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
// TMA store smem -> global (box clipped at the tensor's edges); completion is tracked per thread in bulk groups
__device__ __forceinline__ void tma_store_2d(const void* tmap, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(tmap), "r"(src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all of this thread's groups have finished READING their shared-memory source (it may be overwritten)
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// all but the most recent of this thread's groups have finished reading their shared-memory source
__device__ __forceinline__ void bulk_wait_read1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
// all of this thread's groups are complete (the global writes are done)
__device__ __forceinline__ void bulk_wait_all0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// untiled bulk copy global -> smem (16-byte aligned addresses, size multiple of 16)
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

// ---- TMEM --------------------------------------------------------------------------------------
// One full warp calls these.  ncols: power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// completion of all UMMAs issued so far by this thread -> one arrival on `bar`
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---- descriptors -------------------------------------------------------------------------------
// Shared-memory matrix descriptor, K-major operand stored as rows of 128 bytes with the 128-byte
// swizzle (what a TMA box of 128 bytes x rows with SWIZZLE_128B writes): 8-row groups are 1024
// bytes apart.  The tile base must be 1024-byte aligned; advancing along K inside the 128-byte
// row is done by adding the byte offset (>>4) to the start-address field.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);   // start address, bits [0,14)
  d |= (uint64_t)1 << 16;                   // leading byte offset (ignored for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;         // stride byte offset: 8 rows * 128 B
  d |= (uint64_t)1 << 46;                   // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                   // SWIZZLE_128B
  return d;
}
// Unswizzled K-major, rows of 16 bytes, 8-row groups 128 bytes apart (scale-factor tiles).
__device__ __forceinline__ uint64_t smem_desc_rows16(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);
  d |= (uint64_t)(128 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  return d;
}

enum : uint32_t { FMT_F16 = 0, FMT_BF16 = 1, FMT_U8 = 0, FMT_S8 = 1, FMT_E2M1_MX = 1 };
enum : uint32_t { ACC_F16 = 0, ACC_F32 = 1, ACC_S32 = 2 };

// Instruction descriptor for kind::f16 / kind::i8 (dense, both operands K-major).
__host__ __device__ constexpr uint32_t idesc_dense(uint32_t acc, uint32_t afmt, uint32_t bfmt, uint32_t M, uint32_t N) {
  return (acc << 4) | (afmt << 7) | (bfmt << 10) | ((N >> 3) << 17) | ((M >> 4) << 24);
}
// Instruction descriptor for kind::mxf4nvf4 with UE4M3 scale factors (scale_format bit 23 = 0),
// scale-factor ids 0 (a whole 32-bit TMEM column holds the four factors of one row).
__host__ __device__ constexpr uint32_t idesc_nvf4(uint32_t M, uint32_t N) {
  return (FMT_E2M1_MX << 7) | (FMT_E2M1_MX << 10) | ((N >> 3) << 17) | ((M >> 4) << 24);
}

// ---- UMMA issue (one thread) -------------------------------------------------------------------
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum)
      : "memory");
}
// A operand from tensor memory (lane = row, 32-bit columns hold two 16-bit K elements), B from smem.
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accum)
      : "memory");
}
// The four K = 16 UMMAs of one 64-wide operand stage in one block: A from tensor memory (8 columns per step), B through a
// shared-memory descriptor whose low word advances by 2 (32 bytes) per step; `accum0` = 0 clears the accumulator first.
__device__ __forceinline__ void umma_f16_ts_x4(uint32_t d_tmem, uint32_t a_tmem, uint32_t bdesc_lo, uint32_t bdesc_hi,
                                               uint32_t idesc, uint32_t accum0) {
  asm volatile(
      "{\n\t.reg .pred p, t;\n\t.reg .b64 d0, d1, d2, d3;\n\t.reg .b32 l1, l2, l3, a1, a2, a3;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "setp.eq.b32 t, 0, 0;\n\t"
      "add.u32 l1, %2, 2;\n\tadd.u32 l2, %2, 4;\n\tadd.u32 l3, %2, 6;\n\t"
      "add.u32 a1, %1, 8;\n\tadd.u32 a2, %1, 16;\n\tadd.u32 a3, %1, 24;\n\t"
      "mov.b64 d0, {%2, %3};\n\tmov.b64 d1, {l1, %3};\n\tmov.b64 d2, {l2, %3};\n\tmov.b64 d3, {l3, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], d0, %4, p;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], d1, %4, t;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a2], d2, %4, t;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a3], d3, %4, t;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(bdesc_lo), "r"(bdesc_hi), "r"(idesc), "r"(accum0)
      : "memory");
}
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum)
      : "memory");
}
// E2M1 x E2M1, one UE4M3 scale factor per 16 elements along K, K = 64 per instruction.
__device__ __forceinline__ void umma_nvf4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum,
                                          uint32_t sfa_tmem, uint32_t sfb_tmem) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
// The four K = 16 UMMAs of one 64-wide operand stage, both operands through shared-memory descriptors given as low words
// (address >> 4, advancing by 2 = 32 bytes per step) and one common high word; `accum0` = 0 clears the accumulator first.
__device__ __forceinline__ void umma_f16_ss_x4(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc,
                                               uint32_t accum0) {
  asm volatile(
      "{\n\t.reg .pred p, t;\n\t.reg .b64 da, db;\n\t.reg .b32 x, y;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "setp.eq.b32 t, 0, 0;\n\t"
      "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t"
      "add.u32 x, %1, 2;\n\tadd.u32 y, %2, 2;\n\tmov.b64 da, {x, %3};\n\tmov.b64 db, {y, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, t;\n\t"
      "add.u32 x, %1, 4;\n\tadd.u32 y, %2, 4;\n\tmov.b64 da, {x, %3};\n\tmov.b64 db, {y, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, t;\n\t"
      "add.u32 x, %1, 6;\n\tadd.u32 y, %2, 6;\n\tmov.b64 da, {x, %3};\n\tmov.b64 db, {y, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, t;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accum0)
      : "memory");
}
// One whole NVFP4 operand stage (four 64-element k-blocks) in one block: eight scale-factor copies shared memory ->
// tensor memory (4 columns per k-block and operand), then four block-scaled UMMAs.  Descriptors are given as low
// words (address >> 4, advancing by 2 per k-block for the operands and by 32 for the 512-byte scale tiles) with the
// two constant high words; `accum0` = 0 clears the accumulator first.
__device__ __forceinline__ void umma_nvf4_stage4(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi_op, uint32_t idesc,
                                                 uint32_t accum0, uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t sfa_lo,
                                                 uint32_t sfb_lo, uint32_t hi_sf) {
  asm volatile(
      "{\n\t.reg .pred p, t;\n\t.reg .b64 da, db;\n\t.reg .b32 x, y, u, v;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "setp.eq.b32 t, 0, 0;\n\t"
      // scale factors of the four k-blocks
      "mov.b64 da, {%8, %10};\n\tmov.b64 db, {%9, %10};\n\t"
      "tcgen05.cp.cta_group::1.32x128b.warpx4 [%6], da;\n\ttcgen05.cp.cta_group::1.32x128b.warpx4 [%7], db;\n\t"
      "add.u32 x, %8, 32;\n\tadd.u32 y, %9, 32;\n\tadd.u32 u, %6, 4;\n\tadd.u32 v, %7, 4;\n\t"
      "mov.b64 da, {x, %10};\n\tmov.b64 db, {y, %10};\n\t"
      "tcgen05.cp.cta_group::1.32x128b.warpx4 [u], da;\n\ttcgen05.cp.cta_group::1.32x128b.warpx4 [v], db;\n\t"
      "add.u32 x, %8, 64;\n\tadd.u32 y, %9, 64;\n\tadd.u32 u, %6, 8;\n\tadd.u32 v, %7, 8;\n\t"
      "mov.b64 da, {x, %10};\n\tmov.b64 db, {y, %10};\n\t"
      "tcgen05.cp.cta_group::1.32x128b.warpx4 [u], da;\n\ttcgen05.cp.cta_group::1.32x128b.warpx4 [v], db;\n\t"
      "add.u32 x, %8, 96;\n\tadd.u32 y, %9, 96;\n\tadd.u32 u, %6, 12;\n\tadd.u32 v, %7, 12;\n\t"
      "mov.b64 da, {x, %10};\n\tmov.b64 db, {y, %10};\n\t"
      "tcgen05.cp.cta_group::1.32x128b.warpx4 [u], da;\n\ttcgen05.cp.cta_group::1.32x128b.warpx4 [v], db;\n\t"
      // the four UMMAs
      "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], da, db, %4, [%6], [%7], p;\n\t"
      "add.u32 x, %1, 2;\n\tadd.u32 y, %2, 2;\n\tadd.u32 u, %6, 4;\n\tadd.u32 v, %7, 4;\n\t"
      "mov.b64 da, {x, %3};\n\tmov.b64 db, {y, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], da, db, %4, [u], [v], t;\n\t"
      "add.u32 x, %1, 4;\n\tadd.u32 y, %2, 4;\n\tadd.u32 u, %6, 8;\n\tadd.u32 v, %7, 8;\n\t"
      "mov.b64 da, {x, %3};\n\tmov.b64 db, {y, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], da, db, %4, [u], [v], t;\n\t"
      "add.u32 x, %1, 6;\n\tadd.u32 y, %2, 6;\n\tadd.u32 u, %6, 12;\n\tadd.u32 v, %7, 12;\n\t"
      "mov.b64 da, {x, %3};\n\tmov.b64 db, {y, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], da, db, %4, [u], [v], t;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(hi_op), "r"(idesc), "r"(accum0), "r"(sfa_tmem), "r"(sfb_tmem), "r"(sfa_lo),
        "r"(sfb_lo), "r"(hi_sf)
      : "memory");
}
// 32 rows x 16 bytes of smem -> TMEM lanes 0..31 (4 columns), replicated to all four lane quarters.
__device__ __forceinline__ void tmem_cp_32x128b_x4(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

// ---- TMEM -> registers: warp w of a warpgroup reads lanes 32*(w%4).. ; thread i gets lane i ----
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// registers -> TMEM: 32 consecutive 32-bit columns of this thread's lane
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
// registers -> TMEM: 16 consecutive 32-bit columns of this thread's lane
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(pred)::"memory");
  return pred != 0;
}

}  // namespace dq
