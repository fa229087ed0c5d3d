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
//   dQ_i = dS K_j               (A = dS^T in smem read MN-major, B = K_j MN-major)
//                               -> TMEM [q][d], in the columns dP^T occupied
//   drain warps (one thread per query row) add dQ_i into an fp32 accumulator in global
//   memory with vector reductions; a last small kernel scales and rounds it.
//
// The MMA thread issues, per query tile s:  dP^T(s) | dV(s) | S^T(s+1) | dK(s) dQ(s), so the
// tensor pipe always has the neighbouring tile's products to run while the compute warps are
// in stage A or B (Q_i and dO_i are double-buffered in shared memory for that). The softmax
// scale is applied once to dK in the epilogue and to dQ in the final conversion.
//
// A row kernel that runs first provides -delta_q = -sum_d O dO and -lse_q*log2e. The order
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

constexpr int BWD_THREADS = 384;
constexpr float LOG2E = 1.4426950408889634f;

struct BwdParams {
  AttnArgs a;
  void* dk;
  void* dv;
  float* dq_acc;        // [B,H,S,D] fp32, zeroed before the launch
  const float* nlse2;   // [B,H,S]  -lse * log2(e)
  const float* ndelta;  // [B,H,S]  -sum_d out*dout
  const void* mask;
  int* status;
  float scale_log2;
  int nq;
};

__device__ inline void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z,
                                   int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], "
      "[%2];" ::"r"(ptx::smem_u32(smem_dst)),
      "l"(map), "r"(ptx::smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
// 1-D bulk copy global -> shared (16-byte aligned, size a multiple of 16).
__device__ inline void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   ptx::smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(ptx::smem_u32(bar))
               : "memory");
}
__device__ inline void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}
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

template <typename T, int D, bool CAUSAL, bool MASKED>
__global__ void __launch_bounds__(BWD_THREADS, 1)
    attn_bwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                       const BwdParams p) {
  constexpr int TILE_BYTES = 128 * D * 2;
  constexpr int NBOX = D / 64;
  constexpr int BOX_BYTES = 128 * 64 * 2;
  constexpr int DS_BYTES = 128 * 128 * 2;
  constexpr bool IS_BF16 = std::is_same<T, __nv_bfloat16>::value;
  constexpr uint32_t IDESC_ST = ptx::make_idesc(IS_BF16, false, false, 128, 128);   // K-major x K-major
  constexpr uint32_t IDESC_DKV = ptx::make_idesc(IS_BF16, false, true, 128, D);     // TMEM A, MN-major B
  constexpr uint32_t IDESC_DQ = ptx::make_idesc(IS_BF16, true, true, 128, D);       // MN-major x MN-major
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
  float* nlse_smem = reinterpret_cast<float*>(smem + 6 * TILE_BYTES + DS_BYTES);  // [2][128]
  float* ndelta_smem = nlse_smem + 256;                                           // [2][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(ndelta_smem + 256);
  uint64_t* kv_full = bars + 0;
  uint64_t* qdo_full = bars + 1;     // [2]
  uint64_t* qdo_empty = bars + 3;    // [2]
  uint64_t* st_ready = bars + 5;     // S^T(s) computed
  uint64_t* p1_ready = bars + 6;     // P^T(s) written            (128 arrivals)
  uint64_t* dpt_ready = bars + 7;    // dP^T(s) computed
  uint64_t* p2_ready = bars + 8;     // dS^T(s) written           (128 arrivals)
  uint64_t* dq_ready = bars + 9;     // dQ(s) computed
  uint64_t* dq_drained = bars + 10;  // dQ(s) read out            (128 arrivals)
  uint64_t* all_done = bars + 11;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int jt = blockIdx.x;  // key/value tile; under the causal mask the first tiles do most work
  const int bh = blockIdx.y;
  const int b = bh / (int)p.a.H, h = bh % (int)p.a.H;
  const int i_begin = CAUSAL ? jt : 0;
  const int steps = p.nq - i_begin;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 12; ++i) ptx::mbar_init(&bars[i], (i == 6 || i == 8 || i == 10) ? 128 : 1);
    *abort_flag = 0;
    if ((ptx::smem_u32(smem) & 1023u) != 0) {  // swizzled tiles need a 1024-byte aligned base
      *abort_flag = 1;
      atomicCAS(p.status, 0, 40);
    }
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&map_q);
    ptx::prefetch_tensormap(&map_k);
    ptx::prefetch_tensormap(&map_v);
    ptx::prefetch_tensormap(&map_do);
  }
  if (warp == 2) {
    ptx::tmem_alloc(tmem_slot, TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 && lane == 0) {
    // ---------------------------------------------------------------- producer
    ptx::mbar_expect_tx(kv_full, 2 * TILE_BYTES);
#pragma unroll
    for (int c = 0; c < NBOX; ++c) {
      tma_load_4d(k_smem + c * BOX_BYTES, &map_k, kv_full, c * 64, jt * 128, h, b);
      tma_load_4d(v_smem + c * BOX_BYTES, &map_v, kv_full, c * 64, jt * 128, h, b);
    }
    for (int s = 0; s < steps; ++s) {
      const int it = i_begin + s;
      const int st = s & 1;
      ptx::mbar_wait(&qdo_empty[st], ((s >> 1) & 1) ^ 1, abort_flag, p.status, 41);
      ptx::mbar_expect_tx(&qdo_full[st], 2 * TILE_BYTES + 2 * 512);
#pragma unroll
      for (int c = 0; c < NBOX; ++c) {
        tma_load_4d(q_smem + st * TILE_BYTES + c * BOX_BYTES, &map_q, &qdo_full[st], c * 64, it * 128, h, b);
        tma_load_4d(do_smem + st * TILE_BYTES + c * BOX_BYTES, &map_do, &qdo_full[st], c * 64, it * 128, h, b);
      }
      const long long row0 = ((long long)b * p.a.H + h) * p.a.S + (long long)it * 128;
      bulk_load(nlse_smem + st * 128, p.nlse2 + row0, 512, &qdo_full[st]);
      bulk_load(ndelta_smem + st * 128, p.ndelta + row0, 512, &qdo_full[st]);
    }
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
      for (int ks = 0; ks < 8; ++ks)
        ptx::umma_ts(tmem_base + COL_DV, tmem_base + COL_ST + ks * 8,
                     ptx::make_smem_desc(da + ks * 2048, BOX_BYTES, 1024), IDESC_DKV, (s | ks) != 0);
      // S^T(s+1): overwrites P^T(s), which the dV products above read first (in-order pipe)
      if (s + 1 < steps) {
        ptx::mbar_wait(&qdo_full[st ^ 1], ((s + 1) >> 1) & 1, abort_flag, p.status, 46);
        ptx::tc_fence_after();
        issue_st(st ^ 1);
        ptx::umma_commit(st_ready);
      }
      // dK += dS^T Q, then dQ = dS K into the dP^T columns
      ptx::mbar_wait(p2_ready, ph, abort_flag, p.status, 47);
      ptx::tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        ptx::umma_ts(tmem_base + COL_DK, tmem_base + COL_DPT + ks * 8,
                     ptx::make_smem_desc(qa + ks * 2048, BOX_BYTES, 1024), IDESC_DKV, (s | ks) != 0);
      ptx::umma_commit(&qdo_empty[st]);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)  // reduction over the 128 key rows of the tile
        ptx::umma_ss(tmem_base + COL_DQ, ptx::make_smem_desc(sa + ks * 2048, BOX_BYTES, 1024),
                     ptx::make_smem_desc(ka + ks * 2048, BOX_BYTES, 1024), IDESC_DQ, ks != 0);
      ptx::umma_commit(dq_ready);
    }
    ptx::umma_commit(all_done);
  } else if (warp >= 4 && warp < 8) {
    // ---------------------------------------------------------------- P^T / dS^T (lane = key row)
    const int quarter = warp & 3;
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
      const int it = i_begin + s;
      const int st = s & 1;
      const float4* nlse4 = reinterpret_cast<const float4*>(nlse_smem + st * 128);
      const float4* ndel4 = reinterpret_cast<const float4*>(ndelta_smem + st * 128);
      uint32_t pp[64];  // P^T row of this thread, packed pairs along the query index
      ptx::mbar_wait(&qdo_full[st], (s >> 1) & 1, abort_flag, p.status, 48);  // -lse, -delta of the tile
      ptx::mbar_wait(st_ready, s & 1, abort_flag, p.status, 49);
      ptx::tc_fence_after();
      const bool diag = CAUSAL && (it == jt);
      // ---- stage A: P^T = exp2(S^T * scale*log2e - lse*log2e)
      {
        uint32_t ra[32], rb[32];
        auto stage_a = [&](const uint32_t (&sv)[32], int c) {
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const float4 nl = nlse4[c * 8 + g];
            float x0, x1, x2, x3;
            am::unpack2f(am::fma2(am::pack2u(sv[g * 4], sv[g * 4 + 1]), scale2, am::pack2f(nl.x, nl.y)), x0, x1);
            am::unpack2f(am::fma2(am::pack2u(sv[g * 4 + 2], sv[g * 4 + 3]), scale2, am::pack2f(nl.z, nl.w)), x2, x3);
            if constexpr (MASKED) {
              const long long q0 = (long long)it * 128 + c * 32 + g * 4;
              x0 += Traits<T>::to_f(mask_col[(q0 + 0) * p.a.ms[2]]) * LOG2E;
              x1 += Traits<T>::to_f(mask_col[(q0 + 1) * p.a.ms[2]]) * LOG2E;
              x2 += Traits<T>::to_f(mask_col[(q0 + 2) * p.a.ms[2]]) * LOG2E;
              x3 += Traits<T>::to_f(mask_col[(q0 + 3) * p.a.ms[2]]) * LOG2E;
            }
            float p0 = am::ex2(x0), p1 = am::ex2(x1), p2 = am::ex2(x2), p3 = am::ex2(x3);
            if (diag) {  // query index below the key index contributes nothing
              const int col = c * 32 + g * 4;
              if (col + 0 < r) p0 = 0.f;
              if (col + 1 < r) p1 = 0.f;
              if (col + 2 < r) p2 = 0.f;
              if (col + 3 < r) p3 = 0.f;
            }
            pp[c * 16 + g * 2] = am::cvt_pair<T>(p0, p1);
            pp[c * 16 + g * 2 + 1] = am::cvt_pair<T>(p2, p3);
          }
        };
        ptx::tmem_ld32(st_addr, ra);
        am::tmem_ld_wait_dep(ra);
        ptx::tmem_ld32(st_addr + 32, rb);
        stage_a(ra, 0);
        am::tmem_ld_wait_dep(rb);
        ptx::tmem_ld32(st_addr + 64, ra);
        stage_a(rb, 1);
        am::tmem_ld_wait_dep(ra);
        ptx::tmem_ld32(st_addr + 96, rb);
        stage_a(ra, 2);
        am::tmem_ld_wait_dep(rb);
        stage_a(rb, 3);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t chunk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) chunk[i] = pp[c * 16 + i];
          ptx::tmem_st16(st_addr + c * 16, chunk);
        }
        ptx::tmem_st_wait();
        ptx::tc_fence_before();
        ptx::mbar_arrive(p1_ready);
      }
      // ---- stage B: dS^T = P^T (dP^T - delta)
      ptx::mbar_wait(dpt_ready, s & 1, abort_flag, p.status, 50);
      ptx::tc_fence_after();
      {
        uint32_t ra[32], rb[32];
        auto stage_b = [&](const uint32_t (&dv)[32], int c) {
          uint32_t dd[16];
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const float4 nd = ndel4[c * 8 + g];
            float pa, pb, pc, pd;
            unpack_pair<T>(pp[c * 16 + g * 2], pa, pb);
            unpack_pair<T>(pp[c * 16 + g * 2 + 1], pc, pd);
            float d0, d1, d2, d3;
            am::unpack2f(am::mul2(am::pack2f(pa, pb),
                                  am::add2(am::pack2u(dv[g * 4], dv[g * 4 + 1]), am::pack2f(nd.x, nd.y))),
                         d0, d1);
            am::unpack2f(am::mul2(am::pack2f(pc, pd),
                                  am::add2(am::pack2u(dv[g * 4 + 2], dv[g * 4 + 3]), am::pack2f(nd.z, nd.w))),
                         d2, d3);
            dd[g * 2] = am::cvt_pair<T>(d0, d1);
            dd[g * 2 + 1] = am::cvt_pair<T>(d2, d3);
          }
          ptx::tmem_st16(dp_addr + c * 16, dd);
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
        ptx::tmem_ld32(dp_addr, ra);
        am::tmem_ld_wait_dep(ra);
        ptx::tmem_ld32(dp_addr + 32, rb);
        stage_b(ra, 0);
        am::tmem_ld_wait_dep(rb);
        ptx::tmem_ld32(dp_addr + 64, ra);
        stage_b(rb, 1);
        am::tmem_ld_wait_dep(ra);
        ptx::tmem_ld32(dp_addr + 96, rb);
        stage_b(ra, 2);
        am::tmem_ld_wait_dep(rb);
        stage_b(rb, 3);
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
#pragma unroll 1
    for (int c = 0; c < 2 * D / 32; ++c) {
      const bool is_k = c >= D / 32;
      const int cc = is_k ? c - D / 32 : c;
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
  } else if (warp >= 8) {
    // ---------------------------------------------------------------- dQ drain (lane = query row)
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t dq_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + COL_DQ;
    for (int s = 0; s < steps; ++s) {
      const int it = i_begin + s;
      ptx::mbar_wait(dq_ready, s & 1, abort_flag, p.status, 52);
      ptx::tc_fence_after();
      float* dst = p.dq_acc + ((((long long)b * p.a.H + h) * p.a.S) + (long long)it * 128 + r) * D;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t rr[32];
        ptx::tmem_ld32(dq_addr + c * 32, rr);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 8; ++g)
          red_add_v4(dst + c * 32 + g * 4, __uint_as_float(rr[g * 4 + 0]), __uint_as_float(rr[g * 4 + 1]),
                     __uint_as_float(rr[g * 4 + 2]), __uint_as_float(rr[g * 4 + 3]));
      }
      ptx::tc_fence_before();
      ptx::mbar_arrive(dq_drained);
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// One warp per (b, h, s) row: ndelta = -sum_d out*dout (out strided, dout contiguous) and
// nlse2 = -lse * log2(e).
template <typename T>
__global__ void attn_bwd_prep_kernel(float* __restrict__ ndelta, float* __restrict__ nlse2,
                                     const T* __restrict__ out, const T* __restrict__ dout,
                                     const float* __restrict__ lse, AttnArgs a) {
  const int lane = threadIdx.x & 31;
  const int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t total = a.B * a.H * a.S;
  if (r >= total) return;
  const int64_t s = r % a.S, h = (r / a.S) % a.H, b = r / (a.S * a.H);
  const T* orow = out + b * a.os[0] + h * a.os[1] + s * a.os[2];
  const T* drow = dout + r * a.D;
  float acc = 0.f;
  for (int d = lane * 2; d < a.D; d += 64) {
    float o0, o1, g0, g1;
    unpack_pair<T>(*reinterpret_cast<const uint32_t*>(orow + d), o0, o1);
    unpack_pair<T>(*reinterpret_cast<const uint32_t*>(drow + d), g0, g1);
    acc += o0 * g0 + o1 * g1;
  }
  acc = warp_sum(acc);
  if (lane == 0) {
    ndelta[r] = -acc;
    nlse2[r] = -lse[r] * LOG2E;
  }
}

template <typename T>
__global__ void dq_convert_kernel(T* __restrict__ dq, const float* __restrict__ acc, long long n, float scale) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= n) return;
  const float4 a = *reinterpret_cast<const float4*>(acc + i);
  const float4 c = *reinterpret_cast<const float4*>(acc + i + 4);
  const float v[8] = {a.x * scale, a.y * scale, a.z * scale, a.w * scale,
                      c.x * scale, c.y * scale, c.z * scale, c.w * scale};
  *reinterpret_cast<uint4*>(dq + i) = pack<T>(v);
}

template <typename T, int D, bool CAUSAL, bool MASKED>
static int launch_bwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& md,
                      const BwdParams& p, cudaStream_t st) {
  constexpr int SMEM = 6 * 128 * D * 2 + 128 * 128 * 2 + 2048 + 128;
  auto kern = attn_bwd_tc_kernel<T, D, CAUSAL, MASKED>;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [&] { attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM); });
  if (attr_err != cudaSuccess) {
    set_error("attention_bwd: cudaFuncSetAttribute failed: %s", cudaGetErrorString(attr_err));
    return (int)attr_err;
  }
  dim3 grid((unsigned)p.nq, (unsigned)(p.a.B * p.a.H));
  kern<<<grid, BWD_THREADS, SMEM, st>>>(mq, mk, mv, md, p);
  return launch_status("attn_bwd_tc");
}

}  // namespace

// scratch: [ndelta | nlse2] (2 * B*H*S floats, 256-byte aligned) followed by the fp32 dq
// accumulator (B*H*S*D floats). Launches: prep, memset, main kernel, dq convert.
int launch_attn_bwd_tc(void* dq, void* dk, void* dv, const void* dout, const void* q, const void* k,
                       const void* v, const void* out, const float* lse, float* row_scratch, float* dq_acc,
                       const void* mask, const AttnArgs& a, int dtype, cudaStream_t st) {
  CUtensorMap mq, mk, mv, md;
  const int64_t ds[4] = {a.H * a.S * a.D, a.S * a.D, a.D, 1};  // dout is contiguous
  if (!make_tensor_map_bhsd(&mq, q, a.B, a.H, a.S, a.D, a.qs, 128) ||
      !make_tensor_map_bhsd(&mk, k, a.B, a.H, a.S, a.D, a.ks, 128) ||
      !make_tensor_map_bhsd(&mv, v, a.B, a.H, a.S, a.D, a.vs, 128) ||
      !make_tensor_map_bhsd(&md, dout, a.B, a.H, a.S, a.D, ds, 128))
    return TB200_ERR_UNSUPPORTED;
  const long long rows = (long long)a.B * a.H * a.S;
  const long long n = rows * a.D;
  float* ndelta = row_scratch;
  float* nlse2 = row_scratch + rows;
  cudaError_t e = cudaMemsetAsync(dq_acc, 0, (size_t)n * sizeof(float), st);
  if (e != cudaSuccess) {
    set_error("attention_bwd: memset of the dq accumulator failed: %s", cudaGetErrorString(e));
    return (int)e;
  }
  BwdParams p;
  p.a = a;
  p.dk = dk;
  p.dv = dv;
  p.dq_acc = dq_acc;
  p.nlse2 = nlse2;
  p.ndelta = ndelta;
  p.mask = mask;
  p.status = device_status_ptr();
  p.scale_log2 = a.scale * LOG2E;
  p.nq = (int)(a.S / 128);
  auto go = [&](auto tag, auto dsel) -> int {
    using T = decltype(tag);
    constexpr int D = decltype(dsel)::value;
    attn_bwd_prep_kernel<T><<<(unsigned)ceil_div(rows, 8), 256, 0, st>>>(ndelta, nlse2, (const T*)out,
                                                                        (const T*)dout, lse, a);
    int rc = launch_status("attn_bwd_prep");
    if (rc) return rc;
    if (a.causal)
      rc = launch_bwd<T, D, true, false>(mq, mk, mv, md, p, st);
    else if (mask)
      rc = launch_bwd<T, D, false, true>(mq, mk, mv, md, p, st);
    else
      rc = launch_bwd<T, D, false, false>(mq, mk, mv, md, p, st);
    if (rc) return rc;
    dq_convert_kernel<T><<<(unsigned)ceil_div(n, 8 * 256), 256, 0, st>>>((T*)dq, dq_acc, n, a.scale);
    return launch_status("dq_convert");
  };
  if (dtype == TB200_BF16)
    return a.D == 128 ? go(__nv_bfloat16{}, IntD<128>{}) : go(__nv_bfloat16{}, IntD<64>{});
  return a.D == 128 ? go(__half{}, IntD<128>{}) : go(__half{}, IntD<64>{});
}

}  // namespace tb200
