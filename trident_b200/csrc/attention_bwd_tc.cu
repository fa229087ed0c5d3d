// tcgen05 attention backward for 16-bit q/k/v with head size 64 or 128 and a sequence length
// that is a multiple of 128.
//
// A CTA owns one 128-row key/value tile of one (batch, head), keeps K_j and V_j resident in
// shared memory and walks the query tiles i (all of them, or i >= j under the causal mask).
// Everything is computed transposed, with the key index on the tensor-memory lanes, so that
// the two probabilities-shaped operands never leave tensor memory:
//
//   S^T  = K_j Q_i^T            (A = K_j, B = Q_i, both K-major)         -> TMEM [kv][q]
//   dP^T = V_j dO_i^T           (A = V_j, B = dO_i, both K-major)        -> TMEM [kv][q]
//   compute warps (one thread per key row), in two stages per query tile:
//     A: P^T  = exp2(S^T * scale*log2e - lse_q*log2e)  -> 16-bit, written over S^T
//     B: dS^T = P^T (dP^T - delta_q)                   -> 16-bit, over dP^T and to smem
//   dV  += P^T  dO_i            (A from TMEM, B = dO_i read MN-major)    -> TMEM [kv][d]
//   dK  += dS^T Q_i             (A from TMEM, B = Q_i  read MN-major)    -> TMEM [kv][d]
//   dQ_i, in the columns dP^T occupied, by head size:
//     D = 128: dQ_i^T = K_j^T dS^T (A = K_j, B = dS^T in smem, both MN-major) -> TMEM [d][q]; the
//              drain warps (one thread per feature d) add it to an fp32 accumulator in global
//              memory with red.global.add.f32, a warp covering 128 contiguous bytes of one dQ
//              row per instruction. Three of the four 32-column blocks are loaded before the
//              first reductions, so 32 of the 128 reductions per thread precede the release of
//              the tensor memory (the next dP^T needs those columns).
//     D = 64:  dQ_i = dS K_j (A = dS^T in smem, B = K_j, both MN-major) -> TMEM [q][d]; the drain
//              warps (one thread per query row) copy it into a staging tile of its own in shared
//              memory and one thread adds that to the accumulator with bulk tensor reduce-add
//              copies. (Per-thread 16-byte reductions of this layout were bound by half-used
//              L2 sectors; M = 64 products for a transposed dQ are not used.)
//   A last small kernel scales and rounds the accumulator. (Letting the CTA that adds the last
//   part of a dQ tile convert it, behind a fence and a counter per tile, was measured: the fence
//   after every tile's 16 K reductions cost the drain warps more than the pass it saved, 1.95 ms
//   against 1.65 ms for the configuration [4,32,4096,128].)
//
// The MMA thread issues, per query tile s:  dP^T(s) | dV(s) | S^T(s+1) | dK(s) dQ(s), so the
// tensor pipe always has the neighbouring tile's products to run while the compute warps are
// in stage A or B (Q_i and dO_i are double-buffered in shared memory for that). The softmax
// scale is applied once to dK in the epilogue and to dQ in the final conversion.
//
// A row kernel that runs first provides -delta_q = -sum_d O dO and -lse_q*log2e, and clears the
// fp32 dQ accumulator (no separate memset). The order
// in which key tiles add into dQ is not fixed, so dQ can differ in the last bits from run to
// run; dK and dV are deterministic.
#include <mutex>
#include <type_traits>

#include "attention.cuh"
#include "attn_math.cuh"
#include "common.cuh"
#include "ptx.cuh"

namespace tb200 {

bool make_tensor_map_bhsd(CUtensorMap* map, const void* base, int64_t B, int64_t H, int64_t S, int64_t D,
                          const int64_t* st, uint32_t box_rows);

namespace {

// Warps: 0 producer, 1 MMA issuer, 2 tensor-memory allocation, 3 idle, then 4 * CG compute
// warps (a key row is shared by CG threads, each taking 128 / CG query columns) and four drain
// warps. CG is 2, except for the masked kernel at D = 64, where the compute warps are the
// critical path (one shared-memory load per mask element) and CG = 4 halves their work.
__host__ __device__ constexpr int cgroups_for(int D, bool masked) { return (masked && D == 64) ? 4 : 2; }
__host__ __device__ constexpr int bwd_threads_for(int D, bool masked) { return (4 + 4 * cgroups_for(D, masked) + 4) * 32; }
constexpr float LOG2E = 1.4426950408889634f;
// Register allowances at D = 128 (512 threads, launched with 128 registers each): the drain warps
// take the whole dQ tile into registers (128 values a thread) so that tensor memory is released
// before the first reduction is issued; the service and compute warps give registers back.
constexpr int BWD_REGS_LAUNCH = 128, BWD_REGS_SERVICE = 96, BWD_REGS_COMPUTE = 120, BWD_REGS_DRAIN = 168;
static_assert(4 * 32 * BWD_REGS_SERVICE + 8 * 32 * BWD_REGS_COMPUTE + 4 * 32 * BWD_REGS_DRAIN <= BWD_REGS_LAUNCH * 512,
              "register pool of the CTA exceeded: setmaxnreg.inc would never return");

// Tensor-memory column (relative to the tile's first column) of the packed 16-bit copy of 32-bit
// chunk c (32 query columns) of a P^T or dS^T row: each compute thread packs into the columns it
// has just read itself (its NCH chunks), so no thread overwrites columns another thread still
// has to read and no barrier between the owners of a row is needed.
__host__ __device__ constexpr uint32_t packed_col(int c, int nch) {
  return static_cast<uint32_t>((c / nch) * (32 * nch) + (c % nch) * 16);
}

struct BwdParams {
  AttnArgs a;
  void* dk;
  void* dv;
  float* dq_acc;        // [B,H,S,D] fp32, zeroed by the row kernel
  const float* nlse2;   // [B,H,S]  -lse * log2(e)
  const float* ndelta;  // [B,H,S]  -sum_d out*dout
  const void* mask;
  void* dmask;          // null, or the dense [B,H,S,S] gradient of the additive mask (= dS)
  int mask_tma;         // the mask tile is staged in shared memory by bulk tensor copies
  int mask_has_b, mask_has_h;  // 0 when that mask dimension is broadcast
  int* status;
  float scale_log2;
  int nq;
};

__device__ inline void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z,
                                   int w, uint64_t l2_policy) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%3, %4, %5, %6}], [%2], %7;" ::"r"(ptx::smem_u32(smem_dst)),
      "l"(map), "r"(ptx::smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w), "l"(l2_policy)
      : "memory");
}
// 1-D bulk copy global -> shared (16-byte aligned, size a multiple of 16).
__device__ inline void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   ptx::smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(ptx::smem_u32(bar))
               : "memory");
}
// Adds a [128 rows][32 floats] shared-memory box (128-byte swizzled) into a 2-D fp32 tensor.
__device__ inline void tma_reduce_add_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map),
               "r"(x), "r"(y), "r"(ptx::smem_u32(smem_src))
               : "memory");
}
__device__ inline void red_add_f32(float* addr, float v) {
  asm volatile("red.global.add.f32 [%0], %1;" ::"l"(addr), "f"(v) : "memory");
}
__device__ inline void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ inline void bulk_wait_group_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ inline void bulk_wait_group0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
template <typename T>
__device__ inline void unpack_pair(uint32_t v, float& lo, float& hi);
template <>
__device__ inline void unpack_pair<__nv_bfloat16>(uint32_t v, float& lo, float& hi) {
  lo = __uint_as_float(v << 16);
  hi = __uint_as_float(v & 0xffff0000u);
}
template <>
__device__ inline void unpack_pair<__half>(uint32_t v, float& lo, float& hi) {
  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&v));
  lo = f.x;
  hi = f.y;
}

// DMASK: the kernel also writes dS as the dense gradient of the additive mask (a variant of its
// own: as a run-time branch in stage B it cost the masked kernel 8 %)
template <typename T, int D, bool CAUSAL, bool MASKED, bool DMASK = false>
__global__ void __launch_bounds__(bwd_threads_for(D, MASKED), 1)
    attn_bwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                       const __grid_constant__ CUtensorMap map_dq, const __grid_constant__ CUtensorMap map_mask,
                       const BwdParams p) {
  constexpr int CGROUPS = cgroups_for(D, MASKED);
  constexpr int NCH = 4 / CGROUPS;  // 32-column chunks per compute thread
  constexpr int COMPUTE_WARPS = 4 * CGROUPS;
  constexpr int DRAIN_WARP0 = 4 + COMPUTE_WARPS;
  constexpr int TILE_BYTES = 128 * D * 2;
  constexpr int NBOX = D / 64;
  constexpr int BOX_BYTES = 128 * 64 * 2;
  constexpr int DS_BYTES = 128 * 128 * 2;
  constexpr bool IS_BF16 = std::is_same<T, __nv_bfloat16>::value;
  constexpr uint32_t IDESC_ST = ptx::make_idesc(IS_BF16, false, false, 128, 128);   // K-major x K-major
  constexpr uint32_t IDESC_DKV = ptx::make_idesc(IS_BF16, false, true, 128, D);     // TMEM A, MN-major B
  constexpr uint32_t IDESC_DQ = ptx::make_idesc(IS_BF16, true, true, 128, D);       // MN-major x MN-major
  // At D = 128 dQ_i is produced transposed, dQ^T = K_j^T dS^T (the same two descriptors with
  // their roles swapped), so that a drain thread owns one feature d and a warp-level scalar
  // reduction covers 128 contiguous bytes of one dQ row. At D = 64 (M = 64 is not used) dQ_i
  // keeps the query index on the lanes and goes out through shared memory and a bulk
  // tensor reduce-add.
  constexpr bool DQ_T = (D == 128);
  constexpr uint32_t IDESC_DQT = ptx::make_idesc(IS_BF16, true, true, 128, 128);
  // At D = 64 there is shared memory left for a double-buffered [128 q][128 kv] mask tile,
  // fetched with the Q/dO tile; the compute threads then read their key column from shared
  // memory instead of issuing one global load per query row.
  constexpr bool MASK_SMEM = MASKED && D == 64;
  constexpr int MASK_TILE_BYTES = 128 * 128 * 2;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t COL_ST = 0, COL_DPT = 128, COL_DV = 256, COL_DK = 256 + D;
  constexpr uint32_t COL_DQ = COL_DPT;  // dQ_i reuses the dP^T columns once dS^T has been consumed

  // The dynamic shared memory of this kernel starts at the CTA's shared window (no static
  // shared memory is declared), which is 1024-byte aligned; checked below.
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* k_smem = smem;
  uint8_t* v_smem = smem + TILE_BYTES;
  uint8_t* q_smem = smem + 2 * TILE_BYTES;    // [2]
  uint8_t* do_smem = smem + 4 * TILE_BYTES;   // [2]
  uint8_t* ds_smem = smem + 6 * TILE_BYTES;
  uint8_t* mask_smem = smem + 6 * TILE_BYTES + DS_BYTES;  // [2][MASK_TILE_BYTES] when MASK_SMEM
  constexpr int STAGE_BYTES = DQ_T ? 0 : 128 * D * 4;  // dQ staging tile (fp32), D = 64 only
  uint8_t* dq_stage = smem + 6 * TILE_BYTES + DS_BYTES + (MASK_SMEM ? 2 * MASK_TILE_BYTES : 0);
  float* nlse_smem = reinterpret_cast<float*>(dq_stage + STAGE_BYTES);  // [2][128]
  float* ndelta_smem = nlse_smem + 256;                                           // [2][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(ndelta_smem + 256);
  uint64_t* kv_full = bars + 0;
  uint64_t* qdo_full = bars + 1;     // [2]
  uint64_t* qdo_empty = bars + 3;    // [2]
  uint64_t* st_ready = bars + 5;     // S^T(s) computed
  uint64_t* p1_ready = bars + 6;     // P^T(s) written            (256 arrivals)
  uint64_t* dpt_ready = bars + 7;    // dP^T(s) computed
  uint64_t* p2_ready = bars + 8;     // dS^T(s) written           (256 arrivals)
  uint64_t* dq_ready = bars + 9;     // dQ(s) computed
  uint64_t* dq_drained = bars + 10;  // dQ(s) read out            (128 arrivals)
  uint64_t* all_done = bars + 11;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  volatile uint32_t* abort_flag = tmem_slot + 1;  // [0] abort flag, [1] wait limit (ptx::mbar_wait)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int jt = blockIdx.x;
  int bh = blockIdx.y;
  if (MASKED && p.a.ms[1] == 0 && p.a.H > 1) {
    const int lin = (int)blockIdx.x + (int)gridDim.x * (int)blockIdx.y;
    const int rest = lin / (int)p.a.H;
    jt = rest % (int)gridDim.x;
    bh = (rest / (int)gridDim.x) * (int)p.a.H + lin % (int)p.a.H;
  }
  if constexpr (CAUSAL) {
    // Under the causal mask a CTA walks nq - jt query tiles. Numbering the CTAs head by head leaves
    // 32-tile CTAs of the last heads to start when little other work is left (a long tail); numbering
    // them over groups of 16 (batch, head) slices, key tile first inside a group, starts every long
    // CTA at least 16 * nq CTAs before the end, while the Q and dO tiles that the CTAs running at one
    // time share (16 slices) still fit in L2.
    constexpr int GROUP = 16;  // measured: 4, 8 and 16 equal (1.63 ms), 1 and 32 3 % slower, 64 10 % slower
    const int nbh = (int)gridDim.y, nx = (int)gridDim.x;
    const int lin = (int)blockIdx.x + nx * (int)blockIdx.y;
    const int group = lin / (GROUP * nx);
    const int in_group = min(GROUP, nbh - group * GROUP);
    const int rem = lin - group * GROUP * nx;
    jt = rem / in_group;
    bh = group * GROUP + rem % in_group;
  }
  const int b = bh / (int)p.a.H, h = bh % (int)p.a.H;
  const int i_begin = CAUSAL ? jt : 0;
  const int steps = p.nq - i_begin;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 12; ++i) ptx::mbar_init(&bars[i], (i == 6 || i == 8) ? COMPUTE_WARPS * 32 : (i == 10 ? 128 : 1));
    abort_flag[0] = 0;
    abort_flag[1] = ptx::WAIT_LIMIT_UNITS;
    if ((ptx::smem_u32(smem) & 1023u) != 0) {  // swizzled tiles need a 1024-byte aligned base
      abort_flag[0] = 1;
      atomicCAS(p.status, 0, 40);
    }
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&map_q);
    ptx::prefetch_tensormap(&map_k);
    ptx::prefetch_tensormap(&map_v);
    ptx::prefetch_tensormap(&map_do);
    ptx::prefetch_tensormap(&map_dq);
  }
  if (warp == 2) {
    ptx::tmem_alloc(tmem_slot, TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // (warpgroups: warps 0-3 service, 4-11 compute, 12-15 drain; an increase waits until the
  // CTA's own pool holds the request, which the static_assert above and the host's check of the
  // compiled register count guarantee)
  constexpr bool REBALANCE = DQ_T && !MASKED;
  static_assert(!REBALANCE || bwd_threads_for(D, MASKED) == 512, "allowances are written for 16 warps");

  if (warp < 4) {
  if constexpr (REBALANCE) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(BWD_REGS_SERVICE));
  if (warp == 0 && lane == 0) {
    // ---------------------------------------------------------------- producer
    // L2 priorities (0 normal, 1 first to go): this CTA's K/V tile is read by no one else
    const uint64_t keep = ptx::l2_policy(0), once = ptx::l2_policy(1);
    const uint64_t mask_policy = ptx::l2_policy(0);
    ptx::mbar_expect_tx(kv_full, 2 * TILE_BYTES);
#pragma unroll
    for (int c = 0; c < NBOX; ++c) {
      tma_load_4d(k_smem + c * BOX_BYTES, &map_k, kv_full, c * 64, jt * 128, h, b, once);
      tma_load_4d(v_smem + c * BOX_BYTES, &map_v, kv_full, c * 64, jt * 128, h, b, once);
    }
    for (int s = 0; s < steps; ++s) {
      const int it = i_begin + (s + jt) % steps;  // staggered start: CTAs of one head add into different dQ tiles
      const int st = s & 1;
      ptx::mbar_wait(&qdo_empty[st], ((s >> 1) & 1) ^ 1, abort_flag, p.status, 41);
      const bool stage_mask = MASK_SMEM && p.mask_tma;
      ptx::mbar_expect_tx(&qdo_full[st], 2 * TILE_BYTES + 2 * 512 + (stage_mask ? MASK_TILE_BYTES : 0));
      if (stage_mask) {
#pragma unroll
        for (int bx = 0; bx < 2; ++bx)
          tma_load_4d(mask_smem + st * MASK_TILE_BYTES + bx * BOX_BYTES, &map_mask, &qdo_full[st],
                      jt * 128 + 64 * bx, it * 128, p.mask_has_h ? h : 0, p.mask_has_b ? b : 0, mask_policy);
      }
#pragma unroll
      for (int c = 0; c < NBOX; ++c) {
        tma_load_4d(q_smem + st * TILE_BYTES + c * BOX_BYTES, &map_q, &qdo_full[st], c * 64, it * 128, h, b, keep);
        tma_load_4d(do_smem + st * TILE_BYTES + c * BOX_BYTES, &map_do, &qdo_full[st], c * 64, it * 128, h, b, keep);
      }
      const long long row0 = ((long long)b * p.a.H + h) * p.a.S + (long long)it * 128;
      bulk_load(nlse_smem + st * 128, p.nlse2 + row0, 512, &qdo_full[st]);
      bulk_load(ndelta_smem + st * 128, p.ndelta + row0, 512, &qdo_full[st]);
    }
    // Drain: every copy issued above has landed before the CTA gives up its shared memory (on the
    // normal path the consumers have waited for all of them already).
    ptx::mbar_wait_drain(kv_full, 0, abort_flag, p.status, 54);
    for (int s = steps > 2 ? steps - 2 : 0; s < steps; ++s)
      ptx::mbar_wait_drain(&qdo_full[s & 1], (s >> 1) & 1, abort_flag, p.status, 54);
  } else if (warp == 1 && lane == 0) {
    // ---------------------------------------------------------------- MMA issuer
    const uint32_t ka = ptx::smem_u32(k_smem), va = ptx::smem_u32(v_smem);
    const uint32_t sa = ptx::smem_u32(ds_smem);
    auto issue_st = [&](int st) {  // S^T = K_j Q^T
      const uint32_t qa = ptx::smem_u32(q_smem + st * TILE_BYTES);
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const uint32_t off = (ks >> 2) * BOX_BYTES + (ks & 3) * 32;
        ptx::umma_ss(tmem_base + COL_ST, ptx::make_smem_desc(ka + off, 16, 1024),
                     ptx::make_smem_desc(qa + off, 16, 1024), IDESC_ST, ks != 0);
      }
    };
    ptx::mbar_wait(kv_full, 0, abort_flag, p.status, 42);
    ptx::mbar_wait(&qdo_full[0], 0, abort_flag, p.status, 43);
    ptx::tc_fence_after();
    issue_st(0);
    ptx::umma_commit(st_ready);
    for (int s = 0; s < steps; ++s) {
      const int st = s & 1;
      const uint32_t ph = s & 1;
      const uint32_t qa = ptx::smem_u32(q_smem + st * TILE_BYTES);
      const uint32_t da = ptx::smem_u32(do_smem + st * TILE_BYTES);
      // dP^T(s) = V_j dO^T: its columns still hold dQ(s-1) until the drain warps are done
      if (s > 0) ptx::mbar_wait(dq_drained, ph ^ 1, abort_flag, p.status, 44);
      ptx::tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const uint32_t off = (ks >> 2) * BOX_BYTES + (ks & 3) * 32;
        ptx::umma_ss(tmem_base + COL_DPT, ptx::make_smem_desc(va + off, 16, 1024),
                     ptx::make_smem_desc(da + off, 16, 1024), IDESC_ST, ks != 0);
      }
      ptx::umma_commit(dpt_ready);
      // dV += P^T dO (reduction over the 128 query rows of the tile)
      ptx::mbar_wait(p1_ready, ph, abort_flag, p.status, 45);
      ptx::tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)  // (16 query columns per step: half of a packed chunk)
        ptx::umma_ts(tmem_base + COL_DV, tmem_base + COL_ST + packed_col(ks >> 1, NCH) + (ks & 1) * 8,
                     ptx::make_smem_desc(da + ks * 2048, BOX_BYTES, 1024), IDESC_DKV, (s | ks) != 0);
      // S^T(s+1): overwrites P^T(s), which the dV products above read first (in-order pipe)
      if (s + 1 < steps) {
        ptx::mbar_wait(&qdo_full[st ^ 1], ((s + 1) >> 1) & 1, abort_flag, p.status, 46);
        ptx::tc_fence_after();
        issue_st(st ^ 1);
        ptx::umma_commit(st_ready);
      }
      // dK += dS^T Q (dS^T from tensor memory), then dQ = dS K into the dP^T columns. (dK with dS^T
      // taken from shared memory, which would let dQ go first, was measured: with both operands
      // of four of the five products coming from shared memory the tensor pipe waits for
      // operands, 133 cycles per instruction on average instead of 75.)
      ptx::mbar_wait(p2_ready, ph, abort_flag, p.status, 47);
      ptx::tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        ptx::umma_ts(tmem_base + COL_DK, tmem_base + COL_DPT + packed_col(ks >> 1, NCH) + (ks & 1) * 8,
                     ptx::make_smem_desc(qa + ks * 2048, BOX_BYTES, 1024), IDESC_DKV, (s | ks) != 0);
      ptx::umma_commit(&qdo_empty[st]);  // Q_s and dO_s are dead once dK(s) has run
      if constexpr (DQ_T) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)  // dQ^T = K_j^T dS^T, reduction over the 128 key rows
          ptx::umma_ss(tmem_base + COL_DQ, ptx::make_smem_desc(ka + ks * 2048, BOX_BYTES, 1024),
                       ptx::make_smem_desc(sa + ks * 2048, BOX_BYTES, 1024), IDESC_DQT, ks != 0);
      } else {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)  // reduction over the 128 key rows of the tile
          ptx::umma_ss(tmem_base + COL_DQ, ptx::make_smem_desc(sa + ks * 2048, BOX_BYTES, 1024),
                       ptx::make_smem_desc(ka + ks * 2048, BOX_BYTES, 1024), IDESC_DQ, ks != 0);
      }
      ptx::umma_commit(dq_ready);
    }
    ptx::umma_commit(all_done);
    // Tensor memory is freed after the CTA-wide barrier at the end: the issuer itself waits until
    // everything it issued has completed (the compute warps wait for the same barrier, but after
    // an aborted wait they may pass it early).
    ptx::mbar_wait_drain(all_done, 0, abort_flag, p.status, 53);
  }
  } else if (warp < DRAIN_WARP0) {
    // ---------------------------------------------------------------- P^T / dS^T (lane = key row)
    if constexpr (REBALANCE) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(BWD_REGS_COMPUTE));
    // warps 4-7 take the first 128 / CGROUPS query columns of their rows, warps 8-11 the next, ...
    const int quarter = warp & 3;
    const int cgrp = (warp - 4) >> 2;
    const int c0 = NCH * cgrp;  // first 32-column chunk of this thread
    const int r = quarter * 32 + lane;
    const int kv_g = jt * 128 + r;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t st_addr = tmem_base + lane_off + COL_ST;
    const uint32_t dp_addr = tmem_base + lane_off + COL_DPT;
    const uint64_t scale2 = am::pack2f(p.scale_log2, p.scale_log2);
    const T* mask_col = nullptr;
    if constexpr (MASKED)
      mask_col = reinterpret_cast<const T*>(p.mask) + (long long)b * p.a.ms[0] + (long long)h * p.a.ms[1] +
                 (long long)kv_g * p.a.ms[3];
    for (int s = 0; s < steps; ++s) {
      const int it = i_begin + (s + jt) % steps;  // staggered start: CTAs of one head add into different dQ tiles
      const int st = s & 1;
      const float4* nlse4 = reinterpret_cast<const float4*>(nlse_smem + st * 128);
      const float4* ndel4 = reinterpret_cast<const float4*>(ndelta_smem + st * 128);
      uint32_t pp[NCH * 16];  // this thread's part of a P^T row, packed pairs along the query index
      ptx::mbar_wait(&qdo_full[st], (s >> 1) & 1, abort_flag, p.status, 48);  // -lse, -delta of the tile
      ptx::mbar_wait(st_ready, s & 1, abort_flag, p.status, 49);
      ptx::tc_fence_after();
      const bool diag = CAUSAL && (it == jt);
      // ---- stage A: P^T = exp2(S^T * scale*log2e - lse*log2e)
      {
        uint32_t ra[32];
        [[maybe_unused]] uint32_t rb[32];
        // `diag_tag` is a compile-time flag: only the tile on the diagonal pays for the per-element
        // comparison (with a run-time flag every tile of the causal kernel carried it)
        auto stage_a = [&](const uint32_t (&sv)[32], int c, int lc, auto diag_tag) {
          constexpr bool DIAG = decltype(diag_tag)::value;
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const float4 nl = nlse4[c * 8 + g];
            float x0, x1, x2, x3;
            am::unpack2f(am::fma2(am::pack2u(sv[g * 4], sv[g * 4 + 1]), scale2, am::pack2f(nl.x, nl.y)), x0, x1);
            am::unpack2f(am::fma2(am::pack2u(sv[g * 4 + 2], sv[g * 4 + 3]), scale2, am::pack2f(nl.z, nl.w)), x2, x3);
            if constexpr (MASKED) {
              if (MASK_SMEM && p.mask_tma) {
                // element (q, kv = r) of the 128-byte swizzled [128 q][64 kv] boxes
                const int qc = c * 32 + g * 4;
                const uint8_t* mt = mask_smem + st * MASK_TILE_BYTES + (r >> 6) * BOX_BYTES + (r & 7) * 2;
                const int kchunk = (r & 63) >> 3;
                x0 += Traits<T>::to_f(*reinterpret_cast<const T*>(mt + (qc + 0) * 128 + ((kchunk ^ ((qc + 0) & 7)) << 4))) * LOG2E;
                x1 += Traits<T>::to_f(*reinterpret_cast<const T*>(mt + (qc + 1) * 128 + ((kchunk ^ ((qc + 1) & 7)) << 4))) * LOG2E;
                x2 += Traits<T>::to_f(*reinterpret_cast<const T*>(mt + (qc + 2) * 128 + ((kchunk ^ ((qc + 2) & 7)) << 4))) * LOG2E;
                x3 += Traits<T>::to_f(*reinterpret_cast<const T*>(mt + (qc + 3) * 128 + ((kchunk ^ ((qc + 3) & 7)) << 4))) * LOG2E;
              } else {
                const long long q0 = (long long)it * 128 + c * 32 + g * 4;
                x0 += Traits<T>::to_f(mask_col[(q0 + 0) * p.a.ms[2]]) * LOG2E;
                x1 += Traits<T>::to_f(mask_col[(q0 + 1) * p.a.ms[2]]) * LOG2E;
                x2 += Traits<T>::to_f(mask_col[(q0 + 2) * p.a.ms[2]]) * LOG2E;
                x3 += Traits<T>::to_f(mask_col[(q0 + 3) * p.a.ms[2]]) * LOG2E;
              }
            }
            float p0 = am::ex2(x0), p1 = am::ex2(x1), p2 = am::ex2(x2), p3 = am::ex2(x3);
            if constexpr (DIAG) {  // query index below the key index contributes nothing
              const int col = c * 32 + g * 4;
              if (col + 0 < r) p0 = 0.f;
              if (col + 1 < r) p1 = 0.f;
              if (col + 2 < r) p2 = 0.f;
              if (col + 3 < r) p3 = 0.f;
            }
            pp[lc * 16 + g * 2] = am::cvt_pair<T>(p0, p1);
            pp[lc * 16 + g * 2 + 1] = am::cvt_pair<T>(p2, p3);
          }
        };
        ptx::tmem_ld32(st_addr + c0 * 32, ra);
        am::tmem_ld_wait_dep(ra);
        if constexpr (NCH == 2) ptx::tmem_ld32(st_addr + c0 * 32 + 32, rb);
        if (diag) stage_a(ra, c0, 0, std::true_type{});
        else stage_a(ra, c0, 0, std::false_type{});
        if constexpr (NCH == 2) {
          am::tmem_ld_wait_dep(rb);
          if (diag) stage_a(rb, c0 + 1, 1, std::true_type{});
          else stage_a(rb, c0 + 1, 1, std::false_type{});
        }
        // packed P^T goes over this thread's own S^T columns (see packed_col)
#pragma unroll
        for (int lc = 0; lc < NCH; ++lc) {
          uint32_t chunk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) chunk[i] = pp[lc * 16 + i];
          ptx::tmem_st16(st_addr + packed_col(c0 + lc, NCH), chunk);
        }
        ptx::tmem_st_wait();
        ptx::tc_fence_before();
        ptx::mbar_arrive(p1_ready);
      }
      // ---- stage B: dS^T = P^T (dP^T - delta)
      ptx::mbar_wait(dpt_ready, s & 1, abort_flag, p.status, 50);
      ptx::tc_fence_after();
      {
        uint32_t ra[32];
        [[maybe_unused]] uint32_t rb[32];
        auto stage_b = [&](const uint32_t (&dv)[32], int c, int lc) {
          uint32_t dd[16];
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const float4 nd = ndel4[c * 8 + g];
            float pa, pb, pc, pd;
            unpack_pair<T>(pp[lc * 16 + g * 2], pa, pb);
            unpack_pair<T>(pp[lc * 16 + g * 2 + 1], pc, pd);
            float d0, d1, d2, d3;
            am::unpack2f(am::mul2(am::pack2f(pa, pb),
                                  am::add2(am::pack2u(dv[g * 4], dv[g * 4 + 1]), am::pack2f(nd.x, nd.y))),
                         d0, d1);
            am::unpack2f(am::mul2(am::pack2f(pc, pd),
                                  am::add2(am::pack2u(dv[g * 4 + 2], dv[g * 4 + 3]), am::pack2f(nd.z, nd.w))),
                         d2, d3);
            dd[g * 2] = am::cvt_pair<T>(d0, d1);
            dd[g * 2 + 1] = am::cvt_pair<T>(d2, d3);
            if constexpr (DMASK) {
              // the additive mask enters the scores after the scale: its gradient is dS itself.
              // (a warp's lanes are 32 adjacent keys of one query row: 64-byte segments)
              {
                T* dm = reinterpret_cast<T*>(p.dmask) +
                        (((long long)b * p.a.H + h) * p.a.S + ((long long)it * 128 + c * 32 + g * 4)) * p.a.S + kv_g;
                dm[0] = Traits<T>::from_f(d0);
                dm[p.a.S] = Traits<T>::from_f(d1);
                dm[2 * p.a.S] = Traits<T>::from_f(d2);
                dm[3 * p.a.S] = Traits<T>::from_f(d3);
              }
            }
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) pp[lc * 16 + i] = dd[i];  // P^T is no longer needed
          // dS^T tile in shared memory: [key row][query], 64-query blocks of 16 KB, 128-byte
          // rows whose 16-byte chunks are XOR-swizzled with the row index (the layout a
          // 128-byte-swizzled tensor copy of a [128][64] box would produce)
          uint8_t* blk = ds_smem + (c >> 1) * BOX_BYTES + r * 128;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int chunk = ((c & 1) * 4 + g) ^ (r & 7);
            *reinterpret_cast<uint4*>(blk + chunk * 16) =
                make_uint4(dd[g * 4 + 0], dd[g * 4 + 1], dd[g * 4 + 2], dd[g * 4 + 3]);
          }
        };
        ptx::tmem_ld32(dp_addr + c0 * 32, ra);
        am::tmem_ld_wait_dep(ra);
        if constexpr (NCH == 2) ptx::tmem_ld32(dp_addr + c0 * 32 + 32, rb);
        stage_b(ra, c0, 0);
        if constexpr (NCH == 2) {
          am::tmem_ld_wait_dep(rb);
          stage_b(rb, c0 + 1, 1);
        }
        // packed dS^T over this thread's own dP^T columns (for dK) besides the shared-memory copy (for dQ)
#pragma unroll
        for (int lc = 0; lc < NCH; ++lc) {
          uint32_t chunk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) chunk[i] = pp[lc * 16 + i];
          ptx::tmem_st16(dp_addr + packed_col(c0 + lc, NCH), chunk);
        }
        ptx::tmem_st_wait();
        ptx::fence_proxy_async_smem();
        ptx::tc_fence_before();
        ptx::mbar_arrive(p2_ready);
      }
    }
    // epilogue: dV and dK rows of this key tile
    ptx::mbar_wait(all_done, 0, abort_flag, p.status, 51);
    ptx::tc_fence_after();
    const long long out_row = (((long long)b * p.a.H + h) * p.a.S + kv_g) * D;
    T* dv_row = reinterpret_cast<T*>(p.dv) + out_row;
    T* dk_row = reinterpret_cast<T*>(p.dk) + out_row;
    // the first half of the column groups writes dV, the second half dK; a group takes
    // D * 2 / CGROUPS feature columns of its matrix
    constexpr int EPI_CHUNKS = D / 32 * 2 / CGROUPS;
#pragma unroll 1
    for (int ci = 0; ci < EPI_CHUNKS; ++ci) {
      const bool is_k = cgrp >= CGROUPS / 2;
      const int cc = (cgrp % (CGROUPS / 2)) * EPI_CHUNKS + ci;
      const float mul = is_k ? p.a.scale : 1.f;
      uint32_t rr[32];
      ptx::tmem_ld32(tmem_base + lane_off + (is_k ? COL_DK : COL_DV) + cc * 32, rr);
      ptx::tmem_ld_wait();
      T* dst = (is_k ? dk_row : dv_row) + cc * 32;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint4 o;
        o.x = am::cvt_pair<T>(__uint_as_float(rr[g * 8 + 0]) * mul, __uint_as_float(rr[g * 8 + 1]) * mul);
        o.y = am::cvt_pair<T>(__uint_as_float(rr[g * 8 + 2]) * mul, __uint_as_float(rr[g * 8 + 3]) * mul);
        o.z = am::cvt_pair<T>(__uint_as_float(rr[g * 8 + 4]) * mul, __uint_as_float(rr[g * 8 + 5]) * mul);
        o.w = am::cvt_pair<T>(__uint_as_float(rr[g * 8 + 6]) * mul, __uint_as_float(rr[g * 8 + 7]) * mul);
        *reinterpret_cast<uint4*>(dst + g * 8) = o;
      }
    }
  } else {
    // ---------------------------------------------------------------- dQ drain
    if constexpr (REBALANCE) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(BWD_REGS_DRAIN));
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t dq_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + COL_DQ;
    const long long row_base = ((long long)b * p.a.H + h) * p.a.S;
    for (int s = 0; s < steps; ++s) {
      const int it = i_begin + (s + jt) % steps;  // staggered start: CTAs of one head add into different dQ tiles
      ptx::mbar_wait(dq_ready, s & 1, abort_flag, p.status, 52);
      ptx::tc_fence_after();
      if constexpr (DQ_T) {
        // lane = feature d: this thread owns feature d = r of the tile's 128 query rows
        float* dst = p.dq_acc + (row_base + (long long)it * 128) * D + r;
        if constexpr (REBALANCE) {
          // the whole tile goes to registers, tensor memory is released, then the 128 reductions
          uint32_t r0[32], r1[32], r2[32], r3[32];
          ptx::tmem_ld32(dq_addr, r0);
          ptx::tmem_ld32(dq_addr + 32, r1);
          ptx::tmem_ld32(dq_addr + 64, r2);
          ptx::tmem_ld32(dq_addr + 96, r3);
          am::tmem_ld_wait_dep(r0);
          am::tmem_ld_wait_dep(r1);
          am::tmem_ld_wait_dep(r2);
          am::tmem_ld_wait_dep(r3);
          ptx::tc_fence_before();
          ptx::mbar_arrive(dq_drained);
#pragma unroll
          for (int i = 0; i < 32; ++i) red_add_f32(dst + (long long)i * D, __uint_as_float(r0[i]));
#pragma unroll
          for (int i = 0; i < 32; ++i) red_add_f32(dst + (long long)(32 + i) * D, __uint_as_float(r1[i]));
#pragma unroll
          for (int i = 0; i < 32; ++i) red_add_f32(dst + (long long)(64 + i) * D, __uint_as_float(r2[i]));
#pragma unroll
          for (int i = 0; i < 32; ++i) red_add_f32(dst + (long long)(96 + i) * D, __uint_as_float(r3[i]));
        } else {
          // Three of the four 32-column blocks are loaded at once; the fourth reuses the
          // registers of the first after its reductions are issued, so that only 32 of the
          // 128 reductions stand between the product and the release of the tensor memory.
          uint32_t r0[32], r1[32], r2[32];
          ptx::tmem_ld32(dq_addr, r0);
          ptx::tmem_ld32(dq_addr + 32, r1);
          ptx::tmem_ld32(dq_addr + 64, r2);
          am::tmem_ld_wait_dep(r0);
          am::tmem_ld_wait_dep(r1);
          am::tmem_ld_wait_dep(r2);
#pragma unroll
          for (int i = 0; i < 32; ++i) red_add_f32(dst + (long long)i * D, __uint_as_float(r0[i]));
          ptx::tmem_ld32(dq_addr + 96, r0);
          am::tmem_ld_wait_dep(r0);
          ptx::tc_fence_before();
          ptx::mbar_arrive(dq_drained);  // tensor memory released as soon as its values sit in registers
#pragma unroll
          for (int i = 0; i < 32; ++i) red_add_f32(dst + (long long)(32 + i) * D, __uint_as_float(r1[i]));
#pragma unroll
          for (int i = 0; i < 32; ++i) red_add_f32(dst + (long long)(64 + i) * D, __uint_as_float(r2[i]));
#pragma unroll
          for (int i = 0; i < 32; ++i) red_add_f32(dst + (long long)(96 + i) * D, __uint_as_float(r0[i]));
        }
      } else {
        // lane = query row; dQ_i leaves through a staging tile of D/32 boxes of [128 rows][32
        // floats] (16 KB each) and bulk tensor reduce-add copies
        static_assert(D == 64, "the staging path is written for two boxes");
        uint32_t r0[32], r1[32];
        ptx::tmem_ld32(dq_addr, r0);
        ptx::tmem_ld32(dq_addr + 32, r1);
        am::tmem_ld_wait_dep(r0);
        am::tmem_ld_wait_dep(r1);
        ptx::tc_fence_before();
        ptx::mbar_arrive(dq_drained);  // tensor memory released as soon as its values sit in registers
        // the copies of the previous tile must have read the staging tile before it is rewritten
        if (threadIdx.x == DRAIN_WARP0 * 32) bulk_wait_group_read0();
        asm volatile("bar.sync 2, 128;" ::: "memory");
        uint8_t* row0 = dq_stage + r * 128;
        uint8_t* row1 = dq_stage + 16384 + r * 128;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int chunk = (k ^ (r & 7)) * 16;  // 128-byte swizzle: conflict-free and what the copy expects
          *reinterpret_cast<uint4*>(row0 + chunk) = make_uint4(r0[k * 4], r0[k * 4 + 1], r0[k * 4 + 2], r0[k * 4 + 3]);
          *reinterpret_cast<uint4*>(row1 + chunk) = make_uint4(r1[k * 4], r1[k * 4 + 1], r1[k * 4 + 2], r1[k * 4 + 3]);
        }
        ptx::fence_proxy_async_smem();
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (threadIdx.x == DRAIN_WARP0 * 32) {
          const int y = (int)(row_base + (long long)it * 128);
          tma_reduce_add_2d(&map_dq, dq_stage, 0, y);
          tma_reduce_add_2d(&map_dq, dq_stage + 16384, 32, y);
          bulk_commit_group();
        }
      }
    }
    if (threadIdx.x == DRAIN_WARP0 * 32) bulk_wait_group0();  // every reduce-add has landed before the CTA ends
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ndelta = -sum_d out*dout (out strided over b, h, s; dout contiguous) and nlse2 = -lse * log2(e).
// D / 8 threads share a (b, h, s) row, each with one 16-byte load of out and of dout, so a warp
// covers 256 / D rows and moves 1 KB per pair of load instructions.
// The same threads clear the row's D floats of the fp32 dQ accumulator (32 bytes each).
template <typename T, int D>
__global__ void __launch_bounds__(256)
    attn_bwd_prep_kernel(float* __restrict__ ndelta, float* __restrict__ nlse2, const T* __restrict__ out,
                         const T* __restrict__ dout, const float* __restrict__ lse, float* __restrict__ dq_acc,
                         AttnArgs a) {
  constexpr int TPR = D / 8;           // threads per row
  constexpr int ROWS_PER_CTA = 256 / TPR;
  const int sub = threadIdx.x % TPR;
  const int64_t r = (int64_t)blockIdx.x * ROWS_PER_CTA + threadIdx.x / TPR;
  const int64_t total = a.B * a.H * a.S;
  const bool live = r < total;
  float acc = 0.f;
  if (live) {
    const int64_t s = r % a.S, h = (r / a.S) % a.H, b = r / (a.S * a.H);
    const T* orow = out + b * a.os[0] + h * a.os[1] + s * a.os[2] + sub * 8;
    const T* drow = dout + r * D + sub * 8;
    float o[8], g[8];
    unpack<T>(ld_stream(orow), o);
    unpack<T>(ld_stream(drow), g);
    float4* acc_row = reinterpret_cast<float4*>(dq_acc + r * D + sub * 8);
    acc_row[0] = make_float4(0.f, 0.f, 0.f, 0.f);
    acc_row[1] = make_float4(0.f, 0.f, 0.f, 0.f);

#pragma unroll
    for (int i = 0; i < 8; ++i) acc = fmaf(o[i], g[i], acc);
  }
#pragma unroll
  for (int off = TPR / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (live && sub == 0) {
    ndelta[r] = -acc;
    nlse2[r] = -lse[r] * LOG2E;
  }
}

template <typename T>
__global__ void dq_convert_kernel(T* __restrict__ dq, const float* __restrict__ acc, long long n, float scale) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= n) return;
  // streamed once: kept out of L1
  const uint4 ra = ld_stream(acc + i), rc = ld_stream(acc + i + 4);
  const float v[8] = {__uint_as_float(ra.x) * scale, __uint_as_float(ra.y) * scale, __uint_as_float(ra.z) * scale,
                      __uint_as_float(ra.w) * scale, __uint_as_float(rc.x) * scale, __uint_as_float(rc.y) * scale,
                      __uint_as_float(rc.z) * scale, __uint_as_float(rc.w) * scale};
  st_stream(dq + i, pack<T>(v));
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// 2-D map over the fp32 dq accumulator [rows, D], box [128 rows][32 floats], 128-byte swizzle.
static bool make_dq_map(CUtensorMap* map, float* base, uint64_t rows, uint64_t D) {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(sym);
    else
      cudaGetLastError();
  });
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from the driver");
    return false;
  }
  bind_primary_context();
  cuuint64_t dims[2] = {D, rows};
  cuuint64_t strides[1] = {D * 4};
  cuuint32_t box[2] = {32, 128};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base, dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled (dq accumulator) failed with CUresult %d", (int)r);
    return false;
  }
  return true;
}

template <typename T, int D, bool CAUSAL, bool MASKED, bool DMASK = false>
static int launch_bwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& md,
                      const CUtensorMap& mdq, const CUtensorMap& mmask, const BwdParams& p, cudaStream_t st) {
  constexpr int SMEM = 6 * 128 * D * 2 + 128 * 128 * 2 + 2048 + 128 + ((MASKED && D == 64) ? 2 * 128 * 128 * 2 : 0) +
                       (D == 64 ? 128 * D * 4 : 0);
  static_assert(MASKED || !DMASK, "a mask gradient needs a mask");
  auto kern = attn_bwd_tc_kernel<T, D, CAUSAL, MASKED, DMASK>;
  static std::atomic<unsigned long long> optin_done{0};
  const cudaError_t attr_err = smem_optin_per_device(optin_done, reinterpret_cast<const void*>(kern), SMEM);
  if (attr_err != cudaSuccess) {
    set_error("attention_bwd: cudaFuncSetAttribute failed: %s", cudaGetErrorString(attr_err));
    return (int)attr_err;
  }
  if constexpr (D == 128 && !MASKED) {
    // the kernel's setmaxnreg.inc has no bound on its wait: refuse to launch a build whose register
    // pool (registers per thread at launch x threads) cannot hold the allowances it will ask for
    static std::atomic<int> regs_cached{0};
    int regs = regs_cached.load(std::memory_order_relaxed);
    if (regs == 0) {
      cudaFuncAttributes fa;
      const cudaError_t e = cudaFuncGetAttributes(&fa, kern);
      if (e != cudaSuccess) {
        set_error("attention_bwd: cudaFuncGetAttributes failed: %s", cudaGetErrorString(e));
        return (int)e;
      }
      regs = fa.numRegs;
      regs_cached.store(regs, std::memory_order_relaxed);
    }
    if (regs * 512 < 4 * 32 * BWD_REGS_SERVICE + 8 * 32 * BWD_REGS_COMPUTE + 4 * 32 * BWD_REGS_DRAIN ||
        regs < BWD_REGS_COMPUTE) {
      set_error("attention_bwd: kernel compiled with %d registers per thread, the register rebalancing needs %d",
                regs, BWD_REGS_LAUNCH);
      return TB200_ERR_UNSUPPORTED;
    }
  }
  dim3 grid((unsigned)p.nq, (unsigned)(p.a.B * p.a.H));
  kern<<<grid, bwd_threads_for(D, MASKED), SMEM, st>>>(mq, mk, mv, md, mdq, mmask, p);
  return launch_status("attn_bwd_tc");
}

}  // namespace

// scratch: [ndelta | nlse2] (2 * B*H*S floats, 256-byte aligned) followed by the fp32 dq
// accumulator (B*H*S*D floats). Launches: row kernel (which also clears the accumulator), main
// kernel, dq conversion.
int launch_attn_bwd_tc(void* dq, void* dk, void* dv, void* dmask, const void* dout, const void* q, const void* k,
                       const void* v, const void* out, const float* lse, float* row_scratch, float* dq_acc,
                       const void* mask, const AttnArgs& a, int dtype, cudaStream_t st) {
  CUtensorMap mq, mk, mv, md, mdq;
  const int64_t ds[4] = {a.H * a.S * a.D, a.S * a.D, a.D, 1};  // dout is contiguous
  if (!make_tensor_map_bhsd(&mq, q, a.B, a.H, a.S, a.D, a.qs, 128) ||
      !make_tensor_map_bhsd(&mk, k, a.B, a.H, a.S, a.D, a.ks, 128) ||
      !make_tensor_map_bhsd(&mv, v, a.B, a.H, a.S, a.D, a.vs, 128) ||
      !make_tensor_map_bhsd(&md, dout, a.B, a.H, a.S, a.D, ds, 128) ||
      !make_dq_map(&mdq, dq_acc, (uint64_t)(a.B * a.H * a.S), (uint64_t)a.D))
    return TB200_ERR_UNSUPPORTED;
  const long long rows = (long long)a.B * a.H * a.S;
  const long long n = rows * a.D;
  float* ndelta = row_scratch;
  float* nlse2 = row_scratch + rows;
  BwdParams p;
  CUtensorMap mmask = mq;  // placeholder when no mask tile is staged
  p.mask_tma = 0;
  p.mask_has_b = mask && a.ms[0] != 0;
  p.mask_has_h = mask && a.ms[1] != 0;
  if (mask && a.D == 64 && a.ms[3] == 1 && aligned16(mask) && a.ms[2] > 0 && a.ms[2] % 8 == 0 &&
      (!p.mask_has_h || (a.ms[1] > 0 && a.ms[1] % 8 == 0)) && (!p.mask_has_b || (a.ms[0] > 0 && a.ms[0] % 8 == 0))) {
    // the mask seen as [Bm, Hm, S(query), S(key)] with its broadcast dimensions collapsed to 1
    // (a mask broadcast over the query rows, or one the driver refuses a tensor map for, is read
    // with plain loads instead)
    const int64_t mst[4] = {a.ms[0], a.ms[1], a.ms[2], 1};
    if (make_tensor_map_bhsd(&mmask, mask, p.mask_has_b ? a.B : 1, p.mask_has_h ? a.H : 1, a.S, a.S, mst, 128))
      p.mask_tma = 1;
    else
      mmask = mq;
  }
  p.a = a;
  p.dk = dk;
  p.dv = dv;
  p.dq_acc = dq_acc;
  p.nlse2 = nlse2;
  p.ndelta = ndelta;
  p.mask = mask;
  p.dmask = mask ? dmask : nullptr;
  p.status = device_status_ptr();
  p.scale_log2 = a.scale * LOG2E;
  p.nq = (int)(a.S / 128);
  auto go = [&](auto tag, auto dsel) -> int {
    using T = decltype(tag);
    constexpr int D = decltype(dsel)::value;
    attn_bwd_prep_kernel<T, D><<<(unsigned)ceil_div(rows, 256 / (D / 8)), 256, 0, st>>>(
        ndelta, nlse2, (const T*)out, (const T*)dout, lse, dq_acc, a);
    int rc = launch_status("attn_bwd_prep");
    if (rc) return rc;
    if (a.causal)
      rc = launch_bwd<T, D, true, false>(mq, mk, mv, md, mdq, mmask, p, st);
    else if (mask && p.dmask)
      rc = launch_bwd<T, D, false, true, true>(mq, mk, mv, md, mdq, mmask, p, st);
    else if (mask)
      rc = launch_bwd<T, D, false, true>(mq, mk, mv, md, mdq, mmask, p, st);
    else
      rc = launch_bwd<T, D, false, false>(mq, mk, mv, md, mdq, mmask, p, st);
    if (rc) return rc;
    dq_convert_kernel<T><<<(unsigned)ceil_div(n, 8 * 256), 256, 0, st>>>((T*)dq, dq_acc, n, a.scale);
    return launch_status("dq_convert");
  };
  if (dtype == TB200_BF16)
    return a.D == 128 ? go(__nv_bfloat16{}, IntD<128>{}) : go(__nv_bfloat16{}, IntD<64>{});
  return a.D == 128 ? go(__half{}, IntD<128>{}) : go(__half{}, IntD<64>{});
}

}  // namespace tb200
