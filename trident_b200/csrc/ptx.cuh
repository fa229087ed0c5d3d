// Inline-PTX wrappers for the Blackwell (sm_100a) primitives the tensor-core kernels use:
// mbarrier, bulk tensor copies (TMA), tcgen05 tensor-memory allocation / MMA / commit /
// load / store, plus the shared-memory matrix descriptor and instruction descriptor
// encodings. Single-CTA forms only (cta_group::1, plain per-CTA bulk loads).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tb200 {
namespace ptx {

__device__ inline uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ------------------------------------------------------------------ mbarrier
__device__ inline void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
// Makes freshly initialised barriers visible to the async proxy (TMA, tcgen05.commit).
__device__ inline void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// Orders generic-proxy shared-memory writes before async-proxy reads (tcgen05.mma operands
// written with ordinary stores).
__device__ inline void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ inline void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ inline void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ inline bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Every wait in the tensor-core kernels is bounded. `abort_flag` points at two words of the
// CTA's shared memory: [0] the abort flag, [1] the wait limit in units of 65536 clock cycles
// (set by the kernel from its parameters; WAIT_LIMIT_UNITS unless a test shortens it). After
// that many cycles the waiting thread raises the abort flag and records `code` in the library's
// device status word. Once the flag is up every later wait of the CTA returns after at most
// 1024 polls, so the kernel runs to its normal end (its roles then drain what they have in
// flight and tensor memory is released) with an invalid result instead of hanging.
constexpr uint32_t WAIT_LIMIT_UNITS = 61035;  // x 65536 cycles: about two seconds of SM clock

__device__ inline void mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                                 int* status, int code) {
  if (mbar_try_wait(bar, parity)) return;
  const long long start = clock64();
  uint32_t polls = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++polls & 1023u) == 0) {
      if (abort_flag[0]) return;
      if (clock64() - start > (static_cast<long long>(abort_flag[1]) << 16)) {
        abort_flag[0] = 1;
        if (status) atomicCAS(status, 0, code);
        return;
      }
    }
  }
}
// The same wait for a role's last act, draining what it put in flight (bulk copies into the
// CTA's shared memory, tcgen05.mma writing tensor memory) before the CTA releases both: it
// does not return early when the abort flag is up, only when the barrier completes or the
// time limit passes.
__device__ inline void mbar_wait_drain(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                                       int* status, int code) {
  if (mbar_try_wait(bar, parity)) return;
  const long long start = clock64();
  uint32_t polls = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++polls & 1023u) == 0 && clock64() - start > (static_cast<long long>(abort_flag[1]) << 16)) {
      abort_flag[0] = 1;
      if (status) atomicCAS(status, 0, code);
      return;
    }
  }
}

// ------------------------------------------------------------------ TMA
// 2-D tiled bulk load global -> shared, completion on an mbarrier. x is the innermost
// coordinate: x * element size must be a multiple of 16 bytes.
__device__ inline void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ inline void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// L2 eviction priorities for bulk tensor loads: a tile that only one CTA ever reads (its own Q
// tiles in the attention forward, its K/V tile in the backward) is marked as the first to go.
__device__ inline uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ inline uint64_t l2_policy_evict_normal() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(p));
  return p;
}
// 0 = normal, 1 = first to go. (A "kept" priority is not offered: lines marked so outlive the
// kernel and crowd the next kernel's working set out of L2.)
__device__ inline uint64_t l2_policy(int kind) {
  return kind == 1 ? l2_policy_evict_first() : l2_policy_evict_normal();
}
__device__ inline void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ------------------------------------------------------------------ tensor memory
// One full warp allocates `ncols` (power of two >= 32) columns; the base address is written
// to shared memory.
__device__ inline void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ inline void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ inline void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ inline void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ inline void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// True in exactly one lane of a (converged) warp. A role that issues tcgen05.mma runs its loop
// with the whole warp and predicates the instruction on this: address arithmetic then stays
// warp-uniform. Measured with two arithmetic-bound warps on the same scheduler, a loop entered by
// lane 0 alone issued one tcgen05.mma per 187 cycles, the warp-uniform loop one per 89-99.
__device__ inline bool elect_one() {
  uint32_t pe;
  asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.b32 %0, 1, 0, P;\n\t}" : "=r"(pe));
  return pe != 0;
}

// D[tmem] (+)= A[smem] * B[smem]; one thread issues.
__device__ inline void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ inline void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives once on `bar` when every tcgen05.mma issued so far by this thread has completed.
__device__ inline void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// 32 lanes x 32-bit, N consecutive columns per thread: thread t of warp w reads lane
// 32*(w%4)+t of the tensor-memory address `taddr` (lane in bits 31..16, column in 15..0).
__device__ inline void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
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
__device__ inline void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ inline void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ inline void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31};"
      ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]),
        "r"(taddr)
      : "memory");
}
__device__ inline void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15};"
      ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(taddr)
      : "memory");
}
__device__ inline void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ------------------------------------------------------------------ descriptors
// Shared-memory matrix descriptor for a 128-byte-swizzled operand tile whose base is
// 1024-byte aligned. Fields (64 bits): start address >> 4 in [0,14); leading byte offset
// >> 4 in [16,30); stride byte offset >> 4 in [32,46); descriptor version 1 in [46,48);
// swizzle mode in [61,64) with 2 = 128-byte swizzle.
//   K-major tile  (rows of 64 16-bit elements = 128 B; 8-row groups of 1024 B):
//       lbo is not used by the hardware for swizzled K-major tiles (16 is passed),
//       sbo = 1024 = distance between 8-row groups; advance 32 B per K=16 step.
//   MN-major tile (64 MN elements contiguous = 128 B per reduction row; 8 reduction rows
//       form a 1024 B group): lbo = distance between blocks of 64 MN elements,
//       sbo = 1024 = distance between 8-row groups; advance 2048 B per K=16 step.
__device__ inline uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Instruction descriptor of tcgen05.mma.kind::f16 with fp32 accumulation. Bits: D format
// (1 = f32) in [4,6); A format in [7,10) and B format in [10,13) (0 = f16, 1 = bf16); A
// major in bit 15 and B major in bit 16 (0 = K-major, 1 = MN-major); N >> 3 in [17,23);
// M >> 4 in [24,29).
__host__ __device__ constexpr uint32_t make_idesc(bool bf16, bool a_mn_major, bool b_mn_major, int M, int N) {
  return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((a_mn_major ? 1u : 0u) << 15) |
         ((b_mn_major ? 1u : 0u) << 16) | (static_cast<uint32_t>(N >> 3) << 17) |
         (static_cast<uint32_t>(M >> 4) << 24);
}

}  // namespace ptx

// ------------------------------------------------------------------ host: tensor maps
// 2-D tensor map over a row-major [rows, cols] 16-bit matrix with leading dimension `ld`
// (elements), box [box_rows, box_cols] and 128-byte swizzle (box_cols * 2 bytes == 128).
// Returns false with the error text set when the driver rejects the encoding.
bool make_tensor_map_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                        uint32_t box_rows, uint32_t box_cols);
// 3-D variant: [batch, rows, cols] with strides (batch_stride, ld, 1) in elements.
bool make_tensor_map_3d(CUtensorMap* map, const void* base, uint64_t batch, uint64_t rows, uint64_t cols,
                        uint64_t batch_stride, uint64_t ld, uint32_t box_rows, uint32_t box_cols);

// Device status word of the tensor-core kernels (0 = no bounded wait has ever expired).
int* device_status_ptr();
// Test hook of the calling thread (tb200_test_wait_fault): 0 = normal operation.
int test_wait_fault_mode();

}  // namespace tb200
