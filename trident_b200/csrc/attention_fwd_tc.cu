// tcgen05 attention forward for 16-bit q/k/v with head size 64 or 128 and a sequence
// length that is a multiple of 128.
//
// A CTA owns two adjacent 128-row query tiles of one (batch, head) and walks the key/value
// sequence in 128-row tiles. Both score tiles and both output accumulators live in tensor
// memory (S0, S1: 128 fp32 columns each; O0, O1: D columns each: 512 columns at D = 128),
// so that the tensor pipe works on one query tile while the softmax warps work on the other:
//
//   warp 0      TMA producer: Q0, Q1 once, then a 2-stage ring of K tiles and one of V tiles
//   warp 1      MMA issuer (the warp walks the loop, one elected lane issues):
//               S_t = Q_t K_j^T  (both operands K-major in smem),
//               O_t += P_t V_j (P_t read from tensor memory, V_j MN-major in smem)
//   warp 2      tensor-memory allocation
//   warp 3      at D = 64 with a mask: producer of the [128 q][128 kv] mask tiles (a two-stage ring of
//               shared-memory buffers per query tile; a softmax thread reads its row segment from the
//               buffer while it scales the scores and hands the stage back after the last use)
//   warps 4-7   softmax of query tile 0, warps 8-11 of query tile 1: one thread per score
//               row; row maximum and sum need no shuffles. The 128 scores of the row are read
//               from tensor memory once and stay in registers between the maximum and the
//               exponentials (the softmax warps raise their register allowance with setmaxnreg,
//               the four service warps lower theirs). exp2 with the softmax scale and log2(e)
//               folded in; P is written back as packed 16-bit values: over S at D = 128 (tensor
//               memory is full), to columns of its own at D = 64, where the next score product of
//               the tile is issued as soon as the scores are in registers instead of after P V.
//
// The running maximum used for the exponent is only advanced when the true maximum has
// moved by more than 8 (in log2 units); only then is the accumulator O_t rescaled in tensor
// memory. The final division by the row sum undoes the stale maximum exactly.
//
// Causal tiles above the diagonal are skipped, the diagonal tile is masked per element, and
// CTAs are ordered longest first. An additive mask is read by the softmax threads (each
// thread its own row segment) with broadcast strides honoured.
//
// log-sum-exp saved for backward: lse = ln(2) * m + ln(l) per query row (natural log).
#include <mutex>
#include <type_traits>

#include "attention.cuh"
#include "attn_math.cuh"
#include "common.cuh"
#include "ptx.cuh"

namespace tb200 {
namespace {

constexpr int TQ = 128;       // query rows per tile
constexpr int TK = 128;        // key/value rows per tile
constexpr int FWD_THREADS = 384;
// Register allowances of the kernel's warps (see the setmaxnreg calls): the kernel must be launched
// with REGS_LAUNCH registers per thread for the totals to fit the CTA's pool; the host checks the
// compiled kernel's register count before the first launch.
constexpr int REGS_LAUNCH = 168, REGS_SERVICE = 56, REGS_SOFTMAX = 224;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;
constexpr float RESCALE_THRESHOLD = 8.f;

struct FwdParams {
  AttnArgs a;
  void* out;
  float* lse;
  const void* mask;
  int mask_vec;       // mask rows can be read with 16-byte loads
  int mask_tma;       // the [128 q][128 kv] mask tiles are staged in shared memory by bulk tensor copies
  int mask_has_b, mask_has_h;  // 0 when that mask dimension is broadcast
  int* status;
  float scale_log2;   // softmax scale * log2(e)
  int nq;             // query tiles per (batch, head)
  uint32_t wait_units;  // limit of every bounded wait, in units of 65536 cycles
  int skip_k_tile;      // -1; a test sets the key tile whose copy CTA (0, 0) leaves out
};

template <typename T>
__device__ inline uint32_t pack_pair(float a, float b);
template <>
__device__ inline uint32_t pack_pair<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <>
__device__ inline uint32_t pack_pair<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ inline void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z,
                                   int w, uint64_t l2_policy) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%3, %4, %5, %6}], [%2], %7;" ::"r"(ptx::smem_u32(smem_dst)),
      "l"(map), "r"(ptx::smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w), "l"(l2_policy)
      : "memory");
}

// Eight 16-bit values as four fp32 pairs (for the two-lane fp32 instructions).
template <typename T>
__device__ inline void pairs8(const uint4& raw, uint64_t (&out)[4]) {
  const uint32_t* w = reinterpret_cast<const uint32_t*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
      out[i] = am::pack2u(w[i] << 16, w[i] & 0xffff0000u);
    } else {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      out[i] = am::pack2f(f.x, f.y);
    }
  }
}

// 32 additive-mask values of one row, pre-multiplied by log2(e).
template <typename T>
__device__ inline void load_mask32(float (&mv)[32], const T* row, long long col, long long stride, bool vec) {
  if (vec) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float f[8];
      unpack<T>(__ldg(reinterpret_cast<const uint4*>(row + col + j * 8)), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) mv[j * 8 + i] = f[i] * LOG2E;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) mv[i] = Traits<T>::to_f(row[(col + i) * stride]) * LOG2E;
  }
}

template <typename T, int D, bool CAUSAL, bool MASKED>
__global__ void __launch_bounds__(FWD_THREADS, 1)
    attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_mask,
                       const FwdParams p) {
  constexpr int TILE_BYTES = 128 * D * 2;
  // At D = 64 there is shared memory left for two [128 q][128 kv] mask tiles per query tile: a
  // thread's row segment then comes from shared memory (conflict-free 16-byte reads of the
  // 128-byte swizzled boxes) instead of 16 global loads that each touch 32 different lines per warp.
  constexpr bool MASK_SMEM = MASKED && D == 64;
  constexpr int MASK_TILE_BYTES = 128 * 128 * 2;
  constexpr int NBOX = D / 64;
  constexpr int BOX_BYTES = 128 * 64 * 2;
  constexpr bool IS_BF16 = std::is_same<T, __nv_bfloat16>::value;
  constexpr uint32_t IDESC_QK = ptx::make_idesc(IS_BF16, false, false, TQ, TK);
  constexpr uint32_t IDESC_PV = ptx::make_idesc(IS_BF16, false, true, TQ, D);
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t COL_S = 0, COL_O = 256;
  // At D = 64 the output accumulators leave 128 columns free: P gets columns of its own instead of
  // overwriting S, so the next score product of a query tile is issued as soon as the softmax
  // threads hold the current scores in registers (it no longer has to follow the P V product).
  constexpr bool P_SPLIT = D == 64;
  constexpr uint32_t COL_P = 384;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_smem = smem;                       // [2][TILE_BYTES]
  uint8_t* k_smem = smem + 2 * TILE_BYTES;      // [2][TILE_BYTES]
  uint8_t* v_smem = smem + 4 * TILE_BYTES;      // [2][TILE_BYTES]
  uint8_t* mask_smem = smem + 6 * TILE_BYTES;   // [2 query tiles][2 stages][MASK_TILE_BYTES] when MASK_SMEM
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * TILE_BYTES + (MASK_SMEM ? 4 * MASK_TILE_BYTES : 0));
  // Hand-overs (j = key tile, t = query tile; every barrier completes once per j, so a waiter of
  // phase j passes parity j & 1 and no barrier can run two phases ahead of its waiter):
  //   barrier     arriver, after                                waiter, before                      ordering
  //   k/v_full    bulk copy (complete_tx)                       MMA: QK^T / P V read the stage      async proxy on both sides
  //   k/v_empty   tcgen05.commit after the last product that    producer: next copy into the stage  commit = products done reading
  //               reads the stage
  //   s_full[t]   tcgen05.commit after Q_t K_j^T                softmax: tcgen05.ld of S_t          fence::after_thread_sync
  //   s_free[t]   128 softmax threads after wait::ld of S_t(j)  MMA: Q_t K_{j+1}^T over S_t         fence::before / ::after
  //               (D = 64 only; at D = 128 the product follows P V(j) on the in-order pipe)
  //   p_full[t]   128 softmax threads after wait::st of P_t(j)  MMA: P_t V_j                        fence::before / ::after
  //               (and of the rescaled O_t)
  //   o_done[t]   tcgen05.commit after P_t V_j                  softmax: rescale of O_t, P_t(j+1)   fence::after_thread_sync
  //               over P_t(j) (D = 64), final read of O_t
  //   mask_full   bulk copy (complete_tx)                       softmax: ld.shared of its row       mbarrier acquire
  //   mask_empty  128 softmax threads after the values were     mask producer: next copy            fence.proxy.async + release
  //               consumed
  uint64_t* q_full = bars;         // [2]
  uint64_t* k_full = bars + 2;     // [2]
  uint64_t* k_empty = bars + 4;    // [2]
  uint64_t* v_full = bars + 6;     // [2]
  uint64_t* v_empty = bars + 8;    // [2]
  uint64_t* s_full = bars + 10;    // [2]  MMA -> softmax: scores ready
  uint64_t* p_full = bars + 12;    // [2]  softmax -> MMA: probabilities written
  uint64_t* o_done = bars + 14;    // [2]  MMA -> softmax: P V accumulated
  uint64_t* s_free = bars + 16;      // [2]  softmax -> MMA: scores read into registers (P_SPLIT)
  uint64_t* mask_full = bars + 18;   // [2 tiles][2 stages]  mask producer -> softmax of query tile t
  uint64_t* mask_empty = bars + 22;  // [2 tiles][2 stages]  softmax -> mask producer: last read done
  uint64_t* mma_drained = bars + 26; // MMA issuer: every product it issued has completed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 27);
  volatile uint32_t* abort_flag = tmem_slot + 1;  // [0] abort flag, [1] wait limit (ptx::mbar_wait)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // CTAs are numbered x-fastest. With a mask that is broadcast over heads the head index is
  // made the fastest one instead, so that the H CTAs that read the same mask tiles run at the
  // same time and all but one of them find the tiles in L2.
  int bx = blockIdx.x, bh = blockIdx.y;
  if (MASKED && p.a.ms[1] == 0 && p.a.H > 1) {
    const int lin = (int)blockIdx.x + (int)gridDim.x * (int)blockIdx.y;
    const int rest = lin / (int)p.a.H;
    bx = rest % (int)gridDim.x;
    bh = (rest / (int)gridDim.x) * (int)p.a.H + lin % (int)p.a.H;
  }
  const int pair = (int)gridDim.x - 1 - bx;  // longest (causal) work first
  const int b = bh / (int)p.a.H, h = bh % (int)p.a.H;
  const int qt0 = 2 * pair, qt1 = 2 * pair + 1;
  const bool active1 = qt1 < p.nq;
  const int nkv = (int)(p.a.S / TK);
  const int n0 = CAUSAL ? qt0 + 1 : nkv;
  const int n1 = active1 ? (CAUSAL ? qt1 + 1 : nkv) : 0;
  const int nmax = n0 > n1 ? n0 : n1;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 12; ++i) ptx::mbar_init(&bars[i], 1);
    ptx::mbar_init(&p_full[0], 128);
    ptx::mbar_init(&p_full[1], 128);
    ptx::mbar_init(&o_done[0], 1);
    ptx::mbar_init(&o_done[1], 1);
    for (int i = 0; i < 4; ++i) {
      ptx::mbar_init(&mask_full[i], 1);
      ptx::mbar_init(&mask_empty[i], 128);
    }
    ptx::mbar_init(&s_free[0], 128);
    ptx::mbar_init(&s_free[1], 128);
    ptx::mbar_init(mma_drained, 1);
    abort_flag[0] = 0;
    abort_flag[1] = p.wait_units;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&map_q);
    ptx::prefetch_tensormap(&map_k);
    ptx::prefetch_tensormap(&map_v);
    if (MASK_SMEM && p.mask_tma) ptx::prefetch_tensormap(&map_mask);
  }
  if (warp == 2) {
    ptx::tmem_alloc(tmem_slot, TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Register allowance: the four service warps give registers back and the eight softmax warps
  // (two warpgroups) take them. An increase waits, without a bound, until the CTA's own pool
  // (the registers it was launched with) holds enough, so the totals are checked at compile
  // time: a sum above the launch allocation would block the softmax warps for ever.
  static_assert(FWD_THREADS == 384 && REGS_LAUNCH * FWD_THREADS <= 65536, "launch allocation");
  static_assert(4 * 32 * REGS_SERVICE + 8 * 32 * REGS_SOFTMAX <= REGS_LAUNCH * FWD_THREADS,
                "register pool of the CTA exceeded: setmaxnreg.inc would never return");
  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS_SERVICE));
  if (warp == 0 && lane == 0) {
    // ---------------------------------------------------------------- producer
    // L2 priorities (0 normal, 1 first to go, 2 kept): only a CTA's own query tiles, which no other
    // CTA reads, are marked. Keeping K and V (2) cut the forward's DRAM reads of the masked
    // configuration by a quarter, but lines marked that way outlive the kernel and crowd out
    // whatever runs next (the backward's traffic doubled), so nothing is marked "kept".
    const uint64_t keep = ptx::l2_policy(0), once = ptx::l2_policy(1);
    ptx::mbar_expect_tx(&q_full[0], TILE_BYTES);
#pragma unroll
    for (int c = 0; c < NBOX; ++c)
      tma_load_4d(q_smem + c * BOX_BYTES, &map_q, &q_full[0], c * 64, qt0 * TQ, h, b, once);
    if (active1) {
      ptx::mbar_expect_tx(&q_full[1], TILE_BYTES);
#pragma unroll
      for (int c = 0; c < NBOX; ++c)
        tma_load_4d(q_smem + TILE_BYTES + c * BOX_BYTES, &map_q, &q_full[1], c * 64, qt1 * TQ, h, b, once);
    }
    for (int j = 0; j < nmax; ++j) {
      const int st = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      ptx::mbar_wait(&k_empty[st], ph ^ 1, abort_flag, p.status, 11);
      if (!(j == p.skip_k_tile && blockIdx.x == 0 && blockIdx.y == 0)) {  // (test hook: see FwdParams)
        ptx::mbar_expect_tx(&k_full[st], TILE_BYTES);
#pragma unroll
        for (int c = 0; c < NBOX; ++c)
          tma_load_4d(k_smem + st * TILE_BYTES + c * BOX_BYTES, &map_k, &k_full[st], c * 64, j * TK, h, b, keep);
      }
      ptx::mbar_wait(&v_empty[st], ph ^ 1, abort_flag, p.status, 12);
      ptx::mbar_expect_tx(&v_full[st], TILE_BYTES);
#pragma unroll
      for (int c = 0; c < NBOX; ++c)
        tma_load_4d(v_smem + st * TILE_BYTES + c * BOX_BYTES, &map_v, &v_full[st], c * 64, j * TK, h, b, keep);
    }
    // Drain: the CTA's shared memory is given up when the CTA ends, so every copy issued above
    // must have landed by then. On the normal path the MMA issuer has consumed them all; after an
    // aborted wait it may have run ahead, so the last copy into each stage is waited for here.
    ptx::mbar_wait_drain(&q_full[0], 0, abort_flag, p.status, 15);
    if (active1) ptx::mbar_wait_drain(&q_full[1], 0, abort_flag, p.status, 15);
    for (int j = nmax > 2 ? nmax - 2 : 0; j < nmax; ++j) {
      ptx::mbar_wait_drain(&k_full[j & 1], (j >> 1) & 1, abort_flag, p.status, 16);
      ptx::mbar_wait_drain(&v_full[j & 1], (j >> 1) & 1, abort_flag, p.status, 17);
    }
  } else if (MASK_SMEM && warp == 3 && lane == 0) {
    // ---------------------------------------------------------------- mask producer
    // Two stages per query tile: the copy of key tile j + 1 is in flight while the softmax
    // threads of the tile read key tile j's stage. Stage j & 1 holds key tile j; its k-th use
    // (k = j >> 1) is phase k of both of its barriers.
    //   mask_empty -> this thread: 128 softmax threads arrived after their last ld.shared of the
    //     stage had returned its value (the arrive follows instructions that consume it) and after a
    //     fence.proxy.async, since the next access to the stage is this bulk copy (async proxy).
    //   mask_full -> softmax threads: completes when the copy's bytes have landed (complete_tx).
    if (p.mask_tma) {
      const uint64_t once = ptx::l2_policy(0);
      for (int j = 0; j < nmax; ++j) {
        const int stg = j & 1;
        const uint32_t ph = (j >> 1) & 1;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (j < (t == 0 ? n0 : n1)) {
            uint64_t* full = &mask_full[t * 2 + stg];
            uint8_t* dst = mask_smem + (t * 2 + stg) * MASK_TILE_BYTES;
            ptx::mbar_wait(&mask_empty[t * 2 + stg], ph ^ 1, abort_flag, p.status, 13 + t);
            ptx::mbar_expect_tx(full, MASK_TILE_BYTES);
#pragma unroll
            for (int c = 0; c < 2; ++c)
              tma_load_4d(dst + c * BOX_BYTES, &map_mask, full, j * TK + c * 64, (t == 0 ? qt0 : qt1) * TQ,
                          p.mask_has_h ? h : 0, p.mask_has_b ? b : 0, once);
          }
        }
      }
      // drain (see the K/V producer): the last copy into each stage has landed
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const int nt = t == 0 ? n0 : n1;
        for (int j = nt > 2 ? nt - 2 : 0; j < nt; ++j)
          ptx::mbar_wait_drain(&mask_full[t * 2 + (j & 1)], (j >> 1) & 1, abort_flag, p.status, 18);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    // The whole warp walks the loop; one elected lane waits, issues and commits.
    const bool elected = ptx::elect_one();
    auto wait_ = [&](uint64_t* bar, uint32_t parity, int code) {
      if (elected) ptx::mbar_wait(bar, parity, abort_flag, p.status, code);
      __syncwarp();
    };
    auto commit_ = [&](uint64_t* bar) {
      if (elected) ptx::umma_commit(bar);
    };
    // Shared-memory descriptors are built once: per product only the 14-bit address field moves,
    // by a compile-time constant per K step. (The issuing warp shares its scheduler with two
    // softmax warps that issue almost every cycle; with the descriptors rebuilt per instruction the
    // issue of one tcgen05.mma took about 80 cycles, more than the 64 the instruction needs on the
    // tensor pipe.)
    const uint64_t dq0 = ptx::make_smem_desc(ptx::smem_u32(q_smem), 16, 1024);
    const uint64_t dk0 = ptx::make_smem_desc(ptx::smem_u32(k_smem), 16, 1024);
    const uint64_t dv0 = ptx::make_smem_desc(ptx::smem_u32(v_smem), BOX_BYTES, 1024);
    constexpr uint64_t NEXT_TILE = static_cast<uint64_t>(TILE_BYTES >> 4);  // second query tile / second stage
    auto issue_qk = [&](int t, int st) {
      const uint64_t qd = dq0 + (t ? NEXT_TILE : 0), kd = dk0 + (st ? NEXT_TILE : 0);
      const uint32_t d_tmem = tmem_base + COL_S + t * 128;
      // (every lane walks the unrolled loop and the elected one issues: with the eight
      // instructions inside one `if (elected)` block the unpaired last query tile of an odd
      // tile count came out wrong in some runs; the cause was not found, this form is the one
      // that has always been correct)
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const uint64_t off = static_cast<uint64_t>(((ks >> 2) * BOX_BYTES + (ks & 3) * 32) >> 4);
        if (elected) ptx::umma_ss(d_tmem, qd + off, kd + off, IDESC_QK, ks != 0);
      }
    };
    auto issue_pv = [&](int t, int st, bool accumulate) {
      const uint64_t vd = dv0 + (st ? NEXT_TILE : 0);
      const uint32_t d_tmem = tmem_base + COL_O + t * D;
      const uint32_t p_tmem = tmem_base + (P_SPLIT ? COL_P + t * 64 : COL_S + t * 128);
#pragma unroll
      for (int ks = 0; ks < TK / 16; ++ks) {
        if (elected)
          ptx::umma_ts(d_tmem, p_tmem + ks * 8, vd + static_cast<uint64_t>((ks * 2048) >> 4), IDESC_PV,
                       accumulate || ks != 0);
      }
    };
    wait_(&q_full[0], 0, 21);
    if (active1) wait_(&q_full[1], 0, 22);
    wait_(&k_full[0], 0, 23);
    ptx::tc_fence_after();
    issue_qk(0, 0);
    commit_(&s_full[0]);
    if (n1 > 0) {
      issue_qk(1, 0);
      commit_(&s_full[1]);
    }
    commit_(&k_empty[0]);
    if constexpr (P_SPLIT) {
      for (int j = 0; j < nmax; ++j) {
        const int st = j & 1, nst = (j + 1) & 1;
        const uint32_t ph = (j >> 1) & 1, nph = ((j + 1) >> 1) & 1;
        const uint32_t jp = j & 1;
        bool k_next_ready = false;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          const int nt = t == 0 ? n0 : n1, no = t == 0 ? n1 : n0;
          // the last user of a K or V stage releases it: tile 1 when it takes part, else tile 0
          const bool last_k = t == 1 || j + 1 >= no, last_v = t == 1 || j >= no;
          if (j + 1 < nt) {
            wait_(&s_free[t], jp, 35 + t);
            if (!k_next_ready) wait_(&k_full[nst], nph, 26);
            k_next_ready = true;
            ptx::tc_fence_after();
            issue_qk(t, nst);
            commit_(&s_full[t]);
            if (last_k) commit_(&k_empty[nst]);
          }
          if (j < nt) {
            wait_(&p_full[t], jp, 24 + 3 * t);
            wait_(&v_full[st], ph, 25 + 3 * t);
            ptx::tc_fence_after();
            issue_pv(t, st, j > 0);
            commit_(&o_done[t]);
            if (last_v) commit_(&v_empty[st]);
          }
        }
      }
    } else {
    for (int j = 0; j < nmax; ++j) {
      const int st = j & 1, nst = (j + 1) & 1;
      const uint32_t ph = (j >> 1) & 1, nph = ((j + 1) >> 1) & 1;
      const uint32_t jp = j & 1;
      bool k_next_ready = false;
      if (j < n0) {
        wait_(&p_full[0], jp, 24);
        wait_(&v_full[st], ph, 25);
        ptx::tc_fence_after();
        issue_pv(0, st, j > 0);
        commit_(&o_done[0]);
        if (j >= n1) commit_(&v_empty[st]);
      }
      if (j + 1 < n0) {
        wait_(&k_full[nst], nph, 26);
        k_next_ready = true;
        ptx::tc_fence_after();
        issue_qk(0, nst);
        commit_(&s_full[0]);
        if (j + 1 >= n1) commit_(&k_empty[nst]);
      }
      if (j < n1) {
        wait_(&p_full[1], jp, 27);
        wait_(&v_full[st], ph, 28);
        ptx::tc_fence_after();
        issue_pv(1, st, j > 0);
        commit_(&o_done[1]);
        commit_(&v_empty[st]);
      }
      if (j + 1 < n1) {
        if (!k_next_ready) wait_(&k_full[nst], nph, 29);
        ptx::tc_fence_after();
        issue_qk(1, nst);
        commit_(&s_full[1]);
        commit_(&k_empty[nst]);
      }
    }
    }
    // Tensor memory is freed after the CTA-wide barrier at the end. On the normal path the softmax
    // warps have waited for the last product; after an aborted wait they may not have, so the
    // issuer itself waits until everything it issued has completed.
    commit_(mma_drained);
    if (elected) ptx::mbar_wait_drain(mma_drained, 0, abort_flag, p.status, 19);
    __syncwarp();
  }
  } else {
    // ---------------------------------------------------------------- softmax + epilogue
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS_SOFTMAX));
    const int t = (warp - 4) >> 2;
    const int quarter = warp & 3;
    const int n = t == 0 ? n0 : n1;
    const int qt = t == 0 ? qt0 : qt1;
    const int row_in_tile = quarter * 32 + lane;
    const long long row_g = (long long)qt * TQ + row_in_tile;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_off + COL_S + t * 128;
    const uint32_t o_addr = tmem_base + lane_off + COL_O + t * D;
    const uint32_t p_addr = tmem_base + lane_off + (P_SPLIT ? COL_P + t * 64 : COL_S + t * 128);
    const T* mask_row = nullptr;
    if constexpr (MASKED)
      mask_row = reinterpret_cast<const T*>(p.mask) + (long long)b * p.a.ms[0] + (long long)h * p.a.ms[1] +
                 row_g * p.a.ms[2];
    float m_used = -INFINITY, l = 0.f;
    for (int j = 0; j < n; ++j) {
      const long long kv0 = (long long)j * TK;
      // Mask values of this row and key tile. Staged tiles (D = 64) are read from shared memory
      // chunk by chunk while the scores are scaled; otherwise the row's 128 values are requested
      // from global memory before the scores are waited for, so that their latency hides behind
      // the QK^T product (16-byte loads, kept packed).
      uint4 mraw[(MASKED && !MASK_SMEM) ? 16 : 1];
      const bool mask_staged = MASK_SMEM && p.mask_tma;
      uint32_t mask_row_addr = 0;
      if constexpr (MASKED) {
        if (mask_staged) {
          ptx::mbar_wait(&mask_full[t * 2 + (j & 1)], (j >> 1) & 1, abort_flag, p.status, 30);
          mask_row_addr = ptx::smem_u32(mask_smem + (t * 2 + (j & 1)) * MASK_TILE_BYTES) + row_in_tile * 128;
        } else if constexpr (!MASK_SMEM) {
          if (p.mask_vec) {
#pragma unroll
            for (int c = 0; c < 16; ++c) mraw[c] = __ldg(reinterpret_cast<const uint4*>(mask_row + kv0 + c * 8));
          }
        }
      }
      // 16-byte group g (0..15) of the row's 128 mask values (mask_vec paths)
      auto mask_group = [&](int g) -> uint4 {
        if constexpr (MASK_SMEM) {
          if (mask_staged) {
            // chunk g & 7 of row r sits at r * 128 + (((g & 7) ^ (r & 7)) << 4) of box g >> 3
            uint4 v;
            const uint32_t addr = mask_row_addr + (g >> 3) * BOX_BYTES + (((g & 7) ^ (row_in_tile & 7)) << 4);
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                         : "r"(addr)
                         : "memory");
            return v;
          }
          return __ldg(reinterpret_cast<const uint4*>(mask_row + kv0 + g * 8));
        } else if constexpr (MASKED) {
          return mraw[g];
        } else {
          return make_uint4(0, 0, 0, 0);
        }
      };
      auto mask32 = [&](float (&mv)[32], int c) {
        if (p.mask_vec) {  // (implied by mask_tma)
#pragma unroll
          for (int jv = 0; jv < 4; ++jv) {
            float f[8];
            unpack<T>(mask_group(c * 4 + jv), f);
#pragma unroll
            for (int i = 0; i < 8; ++i) mv[jv * 8 + i] = f[i] * LOG2E;
          }
        } else {
          load_mask32<T>(mv, mask_row, kv0 + c * 32, p.a.ms[3], false);
        }
      };
      ptx::mbar_wait(&s_full[t], j & 1, abort_flag, p.status, 31);
      ptx::tc_fence_after();
      const bool diag = CAUSAL && (j == n - 1);
      // The row's 128 scores are read from tensor memory once and stay in registers between
      // the maximum and the exponentials (the softmax warps raise their register allowance
      // for that): raw accumulator bits on the plain path, scaled and masked values otherwise.
      uint32_t sr[4][32];
      // pass 1: row maximum of the scaled (and masked) scores, in log2 units
      float mx = -INFINITY;
      const bool plain = !MASKED && !diag;  // uniform over the CTA's softmax warps of this tile
      if (plain) {
        // raw maximum (the scale is positive), two elements per three-input max, the load of
        // the next 32 columns in flight while the current ones are reduced
        float m0 = -INFINITY, m1 = -INFINITY;
        auto reduce32 = [&](const uint32_t (&r)[32]) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            m0 = am::max3(m0, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
            m1 = am::max3(m1, __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
          }
        };
        ptx::tmem_ld32(s_addr, sr[0]);
        am::tmem_ld_wait_dep(sr[0]);
        ptx::tmem_ld32(s_addr + 32, sr[1]);
        reduce32(sr[0]);
        am::tmem_ld_wait_dep(sr[1]);
        ptx::tmem_ld32(s_addr + 64, sr[2]);
        reduce32(sr[1]);
        am::tmem_ld_wait_dep(sr[2]);
        ptx::tmem_ld32(s_addr + 96, sr[3]);
        reduce32(sr[2]);
        am::tmem_ld_wait_dep(sr[3]);
        reduce32(sr[3]);
        mx = fmaxf(m0, m1) * p.scale_log2;
      } else {
        const int lim = CAUSAL ? row_in_tile : 1 << 30;  // columns above `lim` are masked (diagonal tile)
        auto scale32 = [&](uint32_t (&r)[32], int c) {
          if constexpr (MASKED && !CAUSAL) {
            if (p.mask_vec) {
              // packed path: score * scale + mask on fp32 pairs (natural units; log2(e) is applied
              // with the subtraction of the maximum in pass 2), two values per maximum
              const uint64_t scale2 = am::pack2f(p.a.scale, p.a.scale);
              float mx1 = -INFINITY;
#pragma unroll
              for (int jv = 0; jv < 4; ++jv) {
                uint64_t m2[4];
                pairs8<T>(mask_group(c * 4 + jv), m2);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const int idx = jv * 8 + i * 2;
                  const uint64_t sc = am::fma2(am::pack2u(r[idx], r[idx + 1]), scale2, m2[i]);
                  float a, b;
                  am::unpack2f(sc, a, b);
                  if (i & 1) mx1 = am::max3(mx1, a, b);
                  else mx = am::max3(mx, a, b);
                  r[idx] = __float_as_uint(a);
                  r[idx + 1] = __float_as_uint(b);
                }
              }
              mx = fmaxf(mx, mx1);
              return;
            }
          }
          float mv[32];
          if constexpr (MASKED) mask32(mv, c);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float sc = __uint_as_float(r[i]) * p.scale_log2;
            if constexpr (MASKED) sc += mv[i];
            if (c * 32 + i > lim) sc = -INFINITY;
            mx = fmaxf(mx, sc);
            r[i] = __float_as_uint(sc);
          }
        };
        ptx::tmem_ld32(s_addr, sr[0]);
        am::tmem_ld_wait_dep(sr[0]);
        ptx::tmem_ld32(s_addr + 32, sr[1]);
        scale32(sr[0], 0);
        am::tmem_ld_wait_dep(sr[1]);
        ptx::tmem_ld32(s_addr + 64, sr[2]);
        scale32(sr[1], 1);
        am::tmem_ld_wait_dep(sr[2]);
        ptx::tmem_ld32(s_addr + 96, sr[3]);
        scale32(sr[2], 2);
        am::tmem_ld_wait_dep(sr[3]);
        scale32(sr[3], 3);
        if constexpr (MASKED) {
          if (p.mask_vec) mx *= LOG2E;  // the packed path works in natural units
        }
        if constexpr (MASK_SMEM) {
          if (mask_staged) {
            // Last read of the mask stage: every ld.shared above has returned its value (the
            // arithmetic of scale32 consumed it) before this arrive is issued. The stage's next
            // access is a bulk tensor copy, hence the proxy fence ahead of the release.
            ptx::fence_proxy_async_smem();
            ptx::mbar_arrive(&mask_empty[t * 2 + (j & 1)]);
          }
        }
      }
      if constexpr (P_SPLIT) {
        // the scores are in registers: the score columns may take the next product
        ptx::tc_fence_before();
        ptx::mbar_arrive(&s_free[t]);
      }
      const float m_new = fmaxf(m_used, mx);
      if (j == 0) {
        m_used = m_new;
      } else {
        const bool need = m_new > m_used + RESCALE_THRESHOLD;
        if (__any_sync(0xffffffffu, need)) {
          // the previous P V must have landed before O is touched
          ptx::mbar_wait(&o_done[t], (j - 1) & 1, abort_flag, p.status, 32);
          ptx::tc_fence_after();
          const float factor = m_new == -INFINITY ? 1.f : exp2f(m_used - m_new);
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t r[32];
            ptx::tmem_ld32(o_addr + c * 32, r);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * factor);
            ptx::tmem_st32(o_addr + c * 32, r);
          }
          ptx::tmem_st_wait();
          l *= factor;
          m_used = m_new;
        }
      }
      const float m_safe = m_used == -INFINITY ? 0.f : m_used;
      // pass 2: probabilities, row sum, P written as packed 16-bit pairs (over S, or to its own columns)
      {
        // registers hold raw products (plain), natural-unit masked scores (packed mask path) or
        // log2-unit scores (diagonal tiles, strided masks)
        const float to_log2 = plain ? p.scale_log2 : ((MASKED && p.mask_vec) ? LOG2E : 1.f);
        const uint64_t scale2 = am::pack2f(to_log2, to_log2);
        const uint64_t negm2 = am::pack2f(-m_safe, -m_safe);
        uint64_t lsum = am::pack2f(0.f, 0.f);
        // The exponentials of a block of 32 columns are written as three passes over the block
        // (arguments, exponentials, sums and packing) so that the 32 independent exp2 of a thread
        // are issued back to back instead of each one being followed by its dependants.
        uint64_t lsum_b = am::pack2f(0.f, 0.f);
        auto exp32 = [&](const uint32_t (&r)[32], int c) {
          float x[32];
#pragma unroll
          for (int i = 0; i < 32; i += 2)
            am::unpack2f(am::fma2(am::pack2u(r[i], r[i + 1]), scale2, negm2), x[i], x[i + 1]);
#pragma unroll
          for (int i = 0; i < 32; ++i) x[i] = am::ex2(x[i]);
          uint32_t packed[16];
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            lsum = am::add2(lsum, am::pack2f(x[i], x[i + 1]));
            lsum_b = am::add2(lsum_b, am::pack2f(x[i + 2], x[i + 3]));
            packed[i >> 1] = am::cvt_pair<T>(x[i], x[i + 1]);
            packed[(i >> 1) + 1] = am::cvt_pair<T>(x[i + 2], x[i + 3]);
          }
          ptx::tmem_st16(p_addr + c * 16, packed);
        };
        if constexpr (P_SPLIT) {
          // P(j) goes over P(j-1): the product that read it must have completed (it has, as a rule:
          // it was issued a whole pass ago)
          if (j > 0) {
            ptx::mbar_wait(&o_done[t], (j - 1) & 1, abort_flag, p.status, 34);
            ptx::tc_fence_after();
          }
        }
        exp32(sr[0], 0);
        exp32(sr[1], 1);
        exp32(sr[2], 2);
        exp32(sr[3], 3);
        float l0, l1;
        am::unpack2f(am::add2(lsum, lsum_b), l0, l1);
        l += l0 + l1;
      }
      ptx::tmem_st_wait();
      ptx::tc_fence_before();
      ptx::mbar_arrive(&p_full[t]);
    }
    if (n > 0) {
      ptx::mbar_wait(&o_done[t], (n - 1) & 1, abort_flag, p.status, 33);
      ptx::tc_fence_after();
      const float inv = 1.f / l;
      T* orow = reinterpret_cast<T*>(p.out) + (long long)b * p.a.os[0] + (long long)h * p.a.os[1] +
                row_g * p.a.os[2];
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        ptx::tmem_ld32(o_addr + c * 32, r);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int jv = 0; jv < 4; ++jv) {
          uint4 o;
          o.x = pack_pair<T>(__uint_as_float(r[jv * 8 + 0]) * inv, __uint_as_float(r[jv * 8 + 1]) * inv);
          o.y = pack_pair<T>(__uint_as_float(r[jv * 8 + 2]) * inv, __uint_as_float(r[jv * 8 + 3]) * inv);
          o.z = pack_pair<T>(__uint_as_float(r[jv * 8 + 4]) * inv, __uint_as_float(r[jv * 8 + 5]) * inv);
          o.w = pack_pair<T>(__uint_as_float(r[jv * 8 + 6]) * inv, __uint_as_float(r[jv * 8 + 7]) * inv);
          *reinterpret_cast<uint4*>(orow + c * 32 + jv * 8) = o;
        }
      }
      const float m_safe = m_used == -INFINITY ? 0.f : m_used;
      p.lse[((long long)b * p.a.H + h) * p.a.S + row_g] = m_safe * LN2 + logf(l);
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn4() {
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
  return fn;
}

}  // namespace

// 4-D tensor map over a [B,H,S,D] 16-bit tensor with element strides st[0..3] (st[3] == 1),
// box [1,1,box_rows,64], 128-byte swizzle.
bool make_tensor_map_bhsd(CUtensorMap* map, const void* base, int64_t B, int64_t H, int64_t S, int64_t D,
                          const int64_t* st, uint32_t box_rows) {
  EncodeFn fn = encode_fn4();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from the driver");
    return false;
  }
  bind_primary_context();
  // a dimension of extent 1 may carry any stride in torch; give it a well-formed one
  int64_t ss = st[2], sh = st[1], sb = st[0];
  if (S == 1) ss = D;
  if (H == 1) sh = ss * S;
  if (B == 1) sb = sh * H;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)ss * 2, (cuuint64_t)sh * 2, (cuuint64_t)sb * 2};
  cuuint32_t box[4] = {64, box_rows, 1, 1};
  cuuint32_t elem[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled (4-D) failed with CUresult %d", (int)r);
    return false;
  }
  return true;
}

static bool strides_ok(const void* ptr, const int64_t* st, int64_t B, int64_t H, int64_t S) {
  if (!aligned16(ptr) || st[3] != 1) return false;
  if (S > 1 && (st[2] % 8 || st[2] <= 0)) return false;
  if (H > 1 && (st[1] % 8 || st[1] <= 0)) return false;
  if (B > 1 && (st[0] % 8 || st[0] <= 0)) return false;
  return true;
}

bool attn_tc_supported(const AttnArgs& a, int dtype, const void* q, const void* k, const void* v,
                       const void* out) {
  if (dtype != TB200_F16 && dtype != TB200_BF16) return false;
  if (a.D != 64 && a.D != 128) return false;
  if (a.S % 128 != 0 || a.S <= 0) return false;
  if (a.B * a.H > 65535 || a.S >= (1ll << 30)) return false;
  if (!strides_ok(q, a.qs, a.B, a.H, a.S) || !strides_ok(k, a.ks, a.B, a.H, a.S) ||
      !strides_ok(v, a.vs, a.B, a.H, a.S) || !strides_ok(out, a.os, a.B, a.H, a.S))
    return false;
  return encode_fn4() != nullptr;
}

template <typename T, int D, bool CAUSAL, bool MASKED>
static int launch_fwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mmask,
                      const FwdParams& p, cudaStream_t st) {
  constexpr int SMEM = 6 * 128 * D * 2 + ((MASKED && D == 64) ? 4 * 128 * 128 * 2 : 0) + 1024 + 256;
  static_assert(SMEM <= 227 * 1024, "shared memory of one CTA");
  auto kern = attn_fwd_tc_kernel<T, D, CAUSAL, MASKED>;
  static std::atomic<unsigned long long> optin_done{0};
  static std::atomic<int> launch_regs_cached{0};  // a property of the compiled code, the same on every device
  cudaError_t attr_err = smem_optin_per_device(optin_done, reinterpret_cast<const void*>(kern), SMEM);
  int launch_regs = launch_regs_cached.load(std::memory_order_relaxed);
  if (attr_err == cudaSuccess && launch_regs == 0) {
    cudaFuncAttributes fa;
    if ((attr_err = cudaFuncGetAttributes(&fa, kern)) == cudaSuccess) {
      launch_regs = fa.numRegs;
      launch_regs_cached.store(launch_regs, std::memory_order_relaxed);
    }
  }
  if (attr_err != cudaSuccess) {
    set_error("attention_fwd: cudaFuncSetAttribute failed: %s", cudaGetErrorString(attr_err));
    return (int)attr_err;
  }
  // The kernel's setmaxnreg.inc has no bound on its wait: refuse to launch a build whose register
  // pool (registers per thread at launch x threads) cannot hold the allowances it will ask for.
  if (launch_regs * FWD_THREADS < 4 * 32 * REGS_SERVICE + 8 * 32 * REGS_SOFTMAX) {
    set_error("attention_fwd: kernel compiled with %d registers per thread, the register rebalancing needs %d",
              launch_regs, REGS_LAUNCH);
    return TB200_ERR_UNSUPPORTED;
  }
  dim3 grid((unsigned)((p.nq + 1) / 2), (unsigned)(p.a.B * p.a.H));
  kern<<<grid, FWD_THREADS, SMEM, st>>>(mq, mk, mv, mmask, p);
  return launch_status("attn_fwd_tc");
}

int launch_attn_fwd_tc(void* out, float* lse, const void* q, const void* k, const void* v, const void* mask,
                       const AttnArgs& a, int dtype, cudaStream_t st) {
  CUtensorMap mq, mk, mv;
  if (!make_tensor_map_bhsd(&mq, q, a.B, a.H, a.S, a.D, a.qs, 128) ||
      !make_tensor_map_bhsd(&mk, k, a.B, a.H, a.S, a.D, a.ks, 128) ||
      !make_tensor_map_bhsd(&mv, v, a.B, a.H, a.S, a.D, a.vs, 128))
    return TB200_ERR_UNSUPPORTED;
  FwdParams p;
  p.a = a;
  p.out = out;
  p.lse = lse;
  p.mask = mask;
  p.mask_vec = mask && a.ms[3] == 1 && aligned16(mask) && a.ms[2] % 8 == 0 && a.ms[1] % 8 == 0 && a.ms[0] % 8 == 0;
  p.status = device_status_ptr();
  p.scale_log2 = a.scale * LOG2E;
  p.nq = (int)(a.S / TQ);
  const bool fault_test = test_wait_fault_mode() == 1;
  p.wait_units = fault_test ? 30u : ptx::WAIT_LIMIT_UNITS;  // 30 x 65536 cycles: about a millisecond
  p.skip_k_tile = fault_test ? 1 : -1;
  CUtensorMap mmask = mq;  // placeholder when no mask tile is staged
  p.mask_tma = 0;
  p.mask_has_b = mask && a.ms[0] != 0;
  p.mask_has_h = mask && a.ms[1] != 0;
  if (mask && !a.causal && a.D == 64 && p.mask_vec && a.ms[2] > 0 && (!p.mask_has_h || a.ms[1] > 0) &&
      (!p.mask_has_b || a.ms[0] > 0)) {
    // the mask seen as [Bm, Hm, S(query), S(key)] with its broadcast dimensions collapsed to 1
    // (a mask broadcast over the query rows, or one the driver refuses a tensor map for, is read
    // with plain loads instead)
    const int64_t mst[4] = {a.ms[0], a.ms[1], a.ms[2], 1};
    if (make_tensor_map_bhsd(&mmask, mask, p.mask_has_b ? a.B : 1, p.mask_has_h ? a.H : 1, a.S, a.S, mst, 128))
      p.mask_tma = 1;
    else
      mmask = mq;
  }
  auto go = [&](auto tag, auto dsel) -> int {
    using T = decltype(tag);
    constexpr int D = decltype(dsel)::value;
    if (a.causal) return launch_fwd<T, D, true, false>(mq, mk, mv, mmask, p, st);
    if (mask) return launch_fwd<T, D, false, true>(mq, mk, mv, mmask, p, st);
    return launch_fwd<T, D, false, false>(mq, mk, mv, mmask, p, st);
  };
  if (dtype == TB200_BF16)
    return a.D == 128 ? go(__nv_bfloat16{}, IntD<128>{}) : go(__nv_bfloat16{}, IntD<64>{});
  return a.D == 128 ? go(__half{}, IntD<128>{}) : go(__half{}, IntD<64>{});
}

}  // namespace tb200
