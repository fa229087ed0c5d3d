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
//   softmax warps (one thread per key row):
//        P^T  = exp2(S^T * scale*log2e - lse_q * log2e)   -> 16-bit, written over S^T
//        dS^T = P^T (dP^T - delta_q) * scale              -> 16-bit, over dP^T and to smem
//   dV  += P^T  dO_i            (A from TMEM, B = dO_i read MN-major)    -> TMEM [kv][d]
//   dK  += dS^T Q_i             (A from TMEM, B = Q_i  read MN-major)    -> TMEM [kv][d]
//   dQ_i = dS K_j               (A = dS^T in smem read MN-major, B = K_j MN-major)
//                                                                         -> TMEM [q][d]
//   drain warps (one thread per query row) add dQ_i into an fp32 accumulator in global
//   memory with vector reductions; a last small kernel rounds it to the output type.
//
// delta_q = sum_d O dO comes from a row kernel that runs first. The order in which key
// tiles add into dQ is not fixed, so dQ can differ in the last bits from run to run; dK
// and dV are deterministic.
#include <mutex>
#include <type_traits>

#include "attention.cuh"
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
  float* dq_acc;       // [B,H,S,D] fp32, zeroed before the launch
  const float* lse;    // [B,H,S]
  const float* delta;  // [B,H,S]
  const void* mask;
  int* status;
  float scale_log2;
  int nq;
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
  constexpr uint32_t COL_DQ = COL_ST;  // dQ_i reuses the S^T columns once P^T has been consumed

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* k_smem = smem;
  uint8_t* v_smem = smem + TILE_BYTES;
  uint8_t* q_smem = smem + 2 * TILE_BYTES;
  uint8_t* do_smem = smem + 3 * TILE_BYTES;
  uint8_t* ds_smem = smem + 4 * TILE_BYTES;
  float* lse_smem = reinterpret_cast<float*>(smem + 4 * TILE_BYTES + DS_BYTES);
  float* delta_smem = lse_smem + 128;
  uint64_t* bars = reinterpret_cast<uint64_t*>(delta_smem + 128);
  uint64_t* kv_full = bars + 0;
  uint64_t* qdo_full = bars + 1;
  uint64_t* qdo_empty = bars + 2;
  uint64_t* s_ready = bars + 3;
  uint64_t* p_ready = bars + 4;      // 128 arrivals
  uint64_t* dq_ready = bars + 5;
  uint64_t* dq_drained = bars + 6;   // 128 arrivals
  uint64_t* all_done = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int jt = blockIdx.x;  // key/value tile; under the causal mask the first tiles do most work
  const int bh = blockIdx.y;
  const int b = bh / (int)p.a.H, h = bh % (int)p.a.H;
  const int i_begin = CAUSAL ? jt : 0;
  const int steps = p.nq - i_begin;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 8; ++i) ptx::mbar_init(&bars[i], (i == 4 || i == 6) ? 128 : 1);
    *abort_flag = 0;
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
      ptx::mbar_wait(qdo_empty, (s & 1) ^ 1, abort_flag, p.status, 41);
      ptx::mbar_expect_tx(qdo_full, 2 * TILE_BYTES + 2 * 512);
#pragma unroll
      for (int c = 0; c < NBOX; ++c) {
        tma_load_4d(q_smem + c * BOX_BYTES, &map_q, qdo_full, c * 64, it * 128, h, b);
        tma_load_4d(do_smem + c * BOX_BYTES, &map_do, qdo_full, c * 64, it * 128, h, b);
      }
      const long long row0 = ((long long)b * p.a.H + h) * p.a.S + (long long)it * 128;
      bulk_load(lse_smem, p.lse + row0, 512, qdo_full);
      bulk_load(delta_smem, p.delta + row0, 512, qdo_full);
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------------------------------------------------------- MMA issuer
    const uint32_t ka = ptx::smem_u32(k_smem), va = ptx::smem_u32(v_smem);
    const uint32_t qa = ptx::smem_u32(q_smem), da = ptx::smem_u32(do_smem), sa = ptx::smem_u32(ds_smem);
    ptx::mbar_wait(kv_full, 0, abort_flag, p.status, 42);
    for (int s = 0; s < steps; ++s) {
      const uint32_t ph = s & 1;
      ptx::mbar_wait(qdo_full, ph, abort_flag, p.status, 43);
      if (s > 0) ptx::mbar_wait(dq_drained, ph ^ 1, abort_flag, p.status, 44);
      ptx::tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const uint32_t off = (ks >> 2) * BOX_BYTES + (ks & 3) * 32;
        ptx::umma_ss(tmem_base + COL_ST, ptx::make_smem_desc(ka + off, 16, 1024),
                     ptx::make_smem_desc(qa + off, 16, 1024), IDESC_ST, ks != 0);
      }
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const uint32_t off = (ks >> 2) * BOX_BYTES + (ks & 3) * 32;
        ptx::umma_ss(tmem_base + COL_DPT, ptx::make_smem_desc(va + off, 16, 1024),
                     ptx::make_smem_desc(da + off, 16, 1024), IDESC_ST, ks != 0);
      }
      ptx::umma_commit(s_ready);
      ptx::mbar_wait(p_ready, ph, abort_flag, p.status, 45);
      ptx::tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)  // reduction over the 128 query rows of the tile
        ptx::umma_ts(tmem_base + COL_DV, tmem_base + COL_ST + ks * 8,
                     ptx::make_smem_desc(da + ks * 2048, BOX_BYTES, 1024), IDESC_DKV, (s | ks) != 0);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        ptx::umma_ts(tmem_base + COL_DK, tmem_base + COL_DPT + ks * 8,
                     ptx::make_smem_desc(qa + ks * 2048, BOX_BYTES, 1024), IDESC_DKV, (s | ks) != 0);
      ptx::umma_commit(qdo_empty);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)  // reduction over the 128 key rows of the tile
        ptx::umma_ss(tmem_base + COL_DQ, ptx::make_smem_desc(sa + ks * 2048, BOX_BYTES, 1024),
                     ptx::make_smem_desc(ka + ks * 2048, BOX_BYTES, 1024), IDESC_DQ, ks != 0);
      ptx::umma_commit(dq_ready);
    }
    ptx::umma_commit(all_done);
  } else if (warp >= 4 && warp < 8) {
    // ---------------------------------------------------------------- softmax / dS (lane = key row)
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int kv_g = jt * 128 + r;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t st_addr = tmem_base + lane_off + COL_ST;
    const uint32_t dp_addr = tmem_base + lane_off + COL_DPT;
    const T* mask_col = nullptr;
    if constexpr (MASKED)
      mask_col = reinterpret_cast<const T*>(p.mask) + (long long)b * p.a.ms[0] + (long long)h * p.a.ms[1] +
                 (long long)kv_g * p.a.ms[3];
    for (int s = 0; s < steps; ++s) {
      const int it = i_begin + s;
      ptx::mbar_wait(qdo_full, s & 1, abort_flag, p.status, 46);   // lse / delta of this tile
      ptx::mbar_wait(s_ready, s & 1, abort_flag, p.status, 47);
      ptx::tc_fence_after();
      const bool diag = CAUSAL && (it == jt);
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t sv[32], dv[32];
        ptx::tmem_ld32(st_addr + c * 32, sv);
        ptx::tmem_ld32(dp_addr + c * 32, dv);
        ptx::tmem_ld_wait();
        uint32_t pp[16], dd[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float pv[2], dsv[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int col = c * 32 + i + u;  // query row inside the tile
            float x = fmaf(__uint_as_float(sv[i + u]), p.scale_log2, -lse_smem[col] * LOG2E);
            if constexpr (MASKED)
              x += Traits<T>::to_f(mask_col[((long long)it * 128 + col) * p.a.ms[2]]) * LOG2E;
            float pr = exp2f(x);
            if (diag && col < r) pr = 0.f;  // query index below the key index
            pv[u] = pr;
            dsv[u] = pr * (__uint_as_float(dv[i + u]) - delta_smem[col]) * p.a.scale;
          }
          pp[i >> 1] = pack_pair<T>(pv[0], pv[1]);
          dd[i >> 1] = pack_pair<T>(dsv[0], dsv[1]);
        }
        ptx::tmem_st16(st_addr + c * 16, pp);
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
      }
      ptx::tmem_st_wait();
      ptx::fence_proxy_async_smem();
      ptx::tc_fence_before();
      ptx::mbar_arrive(p_ready);
    }
    // epilogue: dV and dK rows of this key tile
    ptx::mbar_wait(all_done, 0, abort_flag, p.status, 48);
    ptx::tc_fence_after();
    const long long out_row = (((long long)b * p.a.H + h) * p.a.S + kv_g) * D;
    T* dv_row = reinterpret_cast<T*>(p.dv) + out_row;
    T* dk_row = reinterpret_cast<T*>(p.dk) + out_row;
#pragma unroll 1
    for (int c = 0; c < 2 * D / 32; ++c) {
      const bool is_k = c >= D / 32;
      const int cc = is_k ? c - D / 32 : c;
      uint32_t rr[32];
      ptx::tmem_ld32(tmem_base + lane_off + (is_k ? COL_DK : COL_DV) + cc * 32, rr);
      ptx::tmem_ld_wait();
      T* dst = (is_k ? dk_row : dv_row) + cc * 32;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint4 o;
        o.x = pack_pair<T>(__uint_as_float(rr[g * 8 + 0]), __uint_as_float(rr[g * 8 + 1]));
        o.y = pack_pair<T>(__uint_as_float(rr[g * 8 + 2]), __uint_as_float(rr[g * 8 + 3]));
        o.z = pack_pair<T>(__uint_as_float(rr[g * 8 + 4]), __uint_as_float(rr[g * 8 + 5]));
        o.w = pack_pair<T>(__uint_as_float(rr[g * 8 + 6]), __uint_as_float(rr[g * 8 + 7]));
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
      ptx::mbar_wait(dq_ready, s & 1, abort_flag, p.status, 49);
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

template <typename T>
__global__ void dq_convert_kernel(T* __restrict__ dq, const float* __restrict__ acc, long long n) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= n) return;
  const float4 a = *reinterpret_cast<const float4*>(acc + i);
  const float4 c = *reinterpret_cast<const float4*>(acc + i + 4);
  const float v[8] = {a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w};
  *reinterpret_cast<uint4*>(dq + i) = pack<T>(v);
}

template <typename T, int D, bool CAUSAL, bool MASKED>
static int launch_bwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& md,
                      const BwdParams& p, cudaStream_t st) {
  constexpr int SMEM = 4 * 128 * D * 2 + 128 * 128 * 2 + 1024 + 1024 + 256;
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

// delta must already hold sum_d out*dout. dq_acc is scratch of B*H*S*D floats.
int launch_attn_bwd_tc(void* dq, void* dk, void* dv, const void* dout, const void* q, const void* k,
                       const void* v, const float* lse, const float* delta, float* dq_acc, const void* mask,
                       const AttnArgs& a, int dtype, cudaStream_t st) {
  CUtensorMap mq, mk, mv, md;
  const int64_t ds[4] = {a.H * a.S * a.D, a.S * a.D, a.D, 1};  // dout is contiguous
  if (!make_tensor_map_bhsd(&mq, q, a.B, a.H, a.S, a.D, a.qs, 128) ||
      !make_tensor_map_bhsd(&mk, k, a.B, a.H, a.S, a.D, a.ks, 128) ||
      !make_tensor_map_bhsd(&mv, v, a.B, a.H, a.S, a.D, a.vs, 128) ||
      !make_tensor_map_bhsd(&md, dout, a.B, a.H, a.S, a.D, ds, 128))
    return TB200_ERR_UNSUPPORTED;
  const long long n = (long long)a.B * a.H * a.S * a.D;
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
  p.lse = lse;
  p.delta = delta;
  p.mask = mask;
  p.status = device_status_ptr();
  p.scale_log2 = a.scale * LOG2E;
  p.nq = (int)(a.S / 128);
  auto go = [&](auto tag, auto dsel) -> int {
    using T = decltype(tag);
    constexpr int D = decltype(dsel)::value;
    int rc;
    if (a.causal)
      rc = launch_bwd<T, D, true, false>(mq, mk, mv, md, p, st);
    else if (mask)
      rc = launch_bwd<T, D, false, true>(mq, mk, mv, md, p, st);
    else
      rc = launch_bwd<T, D, false, false>(mq, mk, mv, md, p, st);
    if (rc) return rc;
    dq_convert_kernel<T><<<(unsigned)ceil_div(n, 8 * 256), 256, 0, st>>>((T*)dq, dq_acc, n);
    return launch_status("dq_convert");
  };
  if (dtype == TB200_BF16)
    return a.D == 128 ? go(__nv_bfloat16{}, IntD<128>{}) : go(__nv_bfloat16{}, IntD<64>{});
  return a.D == 128 ? go(__half{}, IntD<128>{}) : go(__half{}, IntD<64>{});
}

}  // namespace tb200
