// tcgen05 GEMM for Linear and GEGLU: C[m,n] = sum_k A(m,k) B(n,k) (+ bias), 16-bit operands,
// fp32 accumulation in tensor memory.
//
// One persistent CTA per SM walks 128 x 256 output tiles. Warp roles:
//   warp 0   TMA producer: per 64-deep K block, one A tile (16 KB) and one B tile (32 KB)
//            into a 4-stage shared-memory ring (128-byte swizzle), signalled through
//            full/empty mbarriers;
//   warp 1   MMA issuer: one thread issues four tcgen05.mma (M128 N256 K16) per stage into one
//            of two 256-column fp32 accumulators in tensor memory, commits the stage back to
//            the producer and, after the last K block, the accumulator to the epilogue;
//   warp 2   allocates and frees the 512 tensor-memory columns;
//   warps 4-7 epilogue: each thread owns one accumulator row (tensor-memory lane), reads it 32
//            columns at a time, applies bias / GEGLU, rounds once and stores 64-byte row
//            segments. The second accumulator lets tile i's epilogue overlap tile i+1's MMAs.
//
// Operand majorness is a property of the shared-memory descriptors, so the three Linear
// GEMMs need no transposes: forward (A, B K-major), input gradient (B = w read MN-major),
// weight gradient (A = dy and B = x both read MN-major).
//
// GEGLU forward stacks the `state` rows [n0, n0+128) and the `gate` rows [N/2+n0, ...) of the
// weight in one B tile, so state and gate of the same output column land in one accumulator
// and the epilogue writes state_gate and out = state * gelu(gate) from a single K loop.
#include "gemm_tc.cuh"

#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"

namespace tb200 {

__device__ int g_device_status = 0;

int* device_status_ptr() {
  int* p = nullptr;
  cudaGetSymbolAddress((void**)&p, g_device_status);
  return p;
}

static thread_local int g_test_wait_fault = 0;
int test_wait_fault_mode() { return g_test_wait_fault; }

namespace {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_TILE_BYTES = BM * BK * 2;          // 16 KB
constexpr int B_TILE_BYTES = BN * BK * 2;          // 32 KB
constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr int TMEM_COLS = 512;
constexpr int NUM_THREADS = 256;

struct GemmParams {
  int M, N, K;          // C is [M, N]; in GEGLU mode N is the full state_gate width
  int num_m_tiles, num_n_tiles, num_k_blocks;
  void* c;
  long long c_ld;
  const void* bias;
  void* geglu_out;      // [M, N/2] or null
  int gelu_tanh;
  int* status;
  const float* row_scale;  // nullable: per-row factor applied to the accumulator (fused RMSNorm)
};

template <typename T>
__device__ inline uint32_t pack2(float a, float b);
template <>
__device__ inline uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <>
__device__ inline uint32_t pack2<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <typename T>
__device__ inline float round_to(float v) { return Traits<T>::to_f(Traits<T>::from_f(v)); }

__device__ inline float gelu_erf(float g) { return 0.5f * g * (1.f + erff(g * 0.7071067811865476f)); }
__device__ inline float gelu_tanh_f(float g) {
  return 0.5f * g * (1.f + tanhf(0.7978845608028654f * g * (1.f + 0.044715f * g * g)));
}

// Stores 32 consecutive columns of one row; `valid` columns are in range (multiple of 8).
template <typename T>
__device__ inline void store_row32(T* dst, const float* v, int valid) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (j * 8 < valid) {
      uint4 o;
      o.x = pack2<T>(v[j * 8 + 0], v[j * 8 + 1]);
      o.y = pack2<T>(v[j * 8 + 2], v[j * 8 + 3]);
      o.z = pack2<T>(v[j * 8 + 4], v[j * 8 + 5]);
      o.w = pack2<T>(v[j * 8 + 6], v[j * 8 + 7]);
      *reinterpret_cast<uint4*>(dst + j * 8) = o;
    }
  }
}

// Order of the output tiles. The CTAs of the persistent grid work on consecutive tile numbers at
// the same time, so a "wave" of them should touch as few distinct A row blocks and B column
// blocks as possible: tiles are numbered m-fastest inside groups of RASTER_GROUP row blocks, which
// makes a wave of 148 tiles cover about 16 row blocks x 9 column blocks (instead of 148 x 1, which
// re-read the whole A operand from HBM once per column block).
constexpr int RASTER_GROUP = 16;
__device__ inline void tile_coords(int tile, int num_m, int num_n, int& m_tile, int& n_tile) {
  const int per_group = RASTER_GROUP * num_n;
  const int group = tile / per_group;
  const int first_m = group * RASTER_GROUP;
  const int rows = min(RASTER_GROUP, num_m - first_m);
  const int in_group = tile - group * per_group;
  m_tile = first_m + in_group % rows;
  n_tile = in_group / rows;
}

template <typename T, bool A_KMAJOR, bool B_KMAJOR, bool GEGLU>
__global__ void __launch_bounds__(NUM_THREADS, 1)
    gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;                 // [STAGES]  TMA -> MMA
  uint64_t* empty_bar = bars + STAGES;       // [STAGES]  MMA -> TMA
  uint64_t* acc_full = bars + 2 * STAGES;    // [2]       MMA -> epilogue
  uint64_t* acc_empty = bars + 2 * STAGES + 2;  // [2]    epilogue -> MMA
  uint64_t* mma_drained = bars + 2 * STAGES + 4;  // MMA issuer: every product it issued has completed
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 5);
  volatile uint32_t* abort_flag = tmem_base_slot + 1;  // [0] abort flag, [1] wait limit (ptx::mbar_wait)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = p.num_m_tiles * p.num_n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(&acc_full[s], 1);
      ptx::mbar_init(&acc_empty[s], 4);
    }
    ptx::mbar_init(mma_drained, 1);
    abort_flag[0] = 0;
    abort_flag[1] = ptx::WAIT_LIMIT_UNITS;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_b);
  }
  if (warp == 2) {
    ptx::tmem_alloc(tmem_base_slot, TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------ producer
    int stage = 0;
    uint32_t phase = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      int m_tile, n_tile;
      tile_coords(tile, p.num_m_tiles, p.num_n_tiles, m_tile, n_tile);
      const int m0 = m_tile * BM;
      const int n0 = GEGLU ? n_tile * (BN / 2) : n_tile * BN;
      for (int kb = 0; kb < p.num_k_blocks; ++kb) {
        ptx::mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, 1);
        uint8_t* a_dst = smem + stage * STAGE_BYTES;
        uint8_t* b_dst = a_dst + A_TILE_BYTES;
        ptx::mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
        const int k0 = kb * BK;
        if constexpr (A_KMAJOR) {
          ptx::tma_load_2d(a_dst, &map_a, &full_bar[stage], k0, m0);  // box [128 rows][64 k]
        } else {
          // operand stored [k][m]: two boxes of [64 k][64 m]
          ptx::tma_load_2d(a_dst, &map_a, &full_bar[stage], m0, k0);
          ptx::tma_load_2d(a_dst + 8192, &map_a, &full_bar[stage], m0 + 64, k0);
        }
        if constexpr (B_KMAJOR) {
          // two boxes of [128 rows][64 k]; in GEGLU mode the second holds the gate rows
          const int second = GEGLU ? p.N / 2 + n0 : n0 + 128;
          ptx::tma_load_2d(b_dst, &map_b, &full_bar[stage], k0, n0);
          ptx::tma_load_2d(b_dst + 16384, &map_b, &full_bar[stage], k0, second);
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            ptx::tma_load_2d(b_dst + j * 8192, &map_b, &full_bar[stage], n0 + 64 * j, k0);
        }
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ------------------------------------------------------------ MMA issuer
    constexpr bool IS_BF16 = std::is_same<T, __nv_bfloat16>::value;
    constexpr uint32_t idesc = ptx::make_idesc(IS_BF16, !A_KMAJOR, !B_KMAJOR, BM, BN);
    constexpr uint32_t A_LBO = A_KMAJOR ? 16 : 8192, B_LBO = B_KMAJOR ? 16 : 8192;
    constexpr uint32_t A_STEP = (A_KMAJOR ? 32 : 2048) >> 4, B_STEP = (B_KMAJOR ? 32 : 2048) >> 4;
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      ptx::mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, p.status, 2);
      ptx::tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * BN;
      for (int kb = 0; kb < p.num_k_blocks; ++kb) {
        ptx::mbar_wait(&full_bar[stage], phase, abort_flag, p.status, 3);
        ptx::tc_fence_after();
        const uint32_t a_addr = ptx::smem_u32(smem + stage * STAGE_BYTES);
        const uint64_t a_desc = ptx::make_smem_desc(a_addr, A_LBO, 1024);
        const uint64_t b_desc = ptx::make_smem_desc(a_addr + A_TILE_BYTES, B_LBO, 1024);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)
          ptx::umma_ss(d_tmem, a_desc + k * A_STEP, b_desc + k * B_STEP, idesc, (kb | k) != 0);
        ptx::umma_commit(&empty_bar[stage]);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      ptx::umma_commit(&acc_full[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    // Tensor memory is freed after the CTA-wide barrier below. On the normal path the epilogue has
    // waited for every accumulator; after an aborted wait it may not have, so the issuer itself
    // waits until the products it issued have completed.
    ptx::umma_commit(mma_drained);
    ptx::mbar_wait_drain(mma_drained, 0, abort_flag, p.status, 5);
  } else if (warp >= 4) {
    // ------------------------------------------------------------ epilogue
    const int quarter = warp & 3;  // tensor-memory lanes [32*quarter, 32*quarter+32)
    int acc = 0;
    uint32_t acc_phase = 0;
    T* C = reinterpret_cast<T*>(p.c);
    const T* bias = reinterpret_cast<const T*>(p.bias);
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      int m_tile, n_tile;
      tile_coords(tile, p.num_m_tiles, p.num_n_tiles, m_tile, n_tile);
      const int m0 = m_tile * BM;
      ptx::mbar_wait(&acc_full[acc], acc_phase, abort_flag, p.status, 4);
      ptx::tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      const float rs = (p.row_scale && row < p.M) ? __ldg(p.row_scale + row) : 1.f;
      if constexpr (!GEGLU) {
        const int n0 = n_tile * BN;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col = n0 + c * 32;
          if (col >= p.N) break;  // uniform across the CTA
          uint32_t r[32];
          ptx::tmem_ld32(t_row + c * 32, r);
          ptx::tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * rs;
          const int valid = min(32, p.N - col);
          if (bias) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i < valid) v[i] += Traits<T>::to_f(__ldg(bias + col + i));
          }
          if (row < p.M) store_row32<T>(C + (long long)row * p.c_ld + col, v, valid);
        }
      } else {
        const int X = p.N / 2;
        const int n0 = n_tile * (BN / 2);
        T* OUT = reinterpret_cast<T*>(p.geglu_out);
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          const int col = n0 + c * 32;
          if (col >= X) break;
          uint32_t rs_[32], rg[32];
          ptx::tmem_ld32(t_row + c * 32, rs_);
          ptx::tmem_ld32(t_row + BN / 2 + c * 32, rg);
          ptx::tmem_ld_wait();
          float s[32], g[32];
          const int valid = min(32, X - col);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            s[i] = __uint_as_float(rs_[i]) * rs;
            g[i] = __uint_as_float(rg[i]) * rs;
            if (bias && i < valid) {
              s[i] += Traits<T>::to_f(__ldg(bias + col + i));
              g[i] += Traits<T>::to_f(__ldg(bias + X + col + i));
            }
            // the saved state_gate is what backward sees: compute from its rounded values
            s[i] = round_to<T>(s[i]);
            g[i] = round_to<T>(g[i]);
          }
          if (row < p.M) {
            T* sg_row = C + (long long)row * p.c_ld;
            store_row32<T>(sg_row + col, s, valid);
            store_row32<T>(sg_row + X + col, g, valid);
          }
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float ge = round_to<T>(p.gelu_tanh ? gelu_tanh_f(g[i]) : gelu_erf(g[i]));
            s[i] *= ge;
          }
          if (row < p.M) store_row32<T>(OUT + (long long)row * X + col, s, valid);
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&acc_empty[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
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

EncodeFn encode_fn() {
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

bool make_tensor_map_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                        uint32_t box_rows, uint32_t box_cols) {
  EncodeFn fn = encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from the driver");
    return false;
  }
  bind_primary_context();
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (rows=%llu cols=%llu ld=%llu)", (int)r,
              (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)ld);
    return false;
  }
  return true;
}

bool make_tensor_map_3d(CUtensorMap* map, const void* base, uint64_t batch, uint64_t rows, uint64_t cols,
                        uint64_t batch_stride, uint64_t ld, uint32_t box_rows, uint32_t box_cols) {
  EncodeFn fn = encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from the driver");
    return false;
  }
  bind_primary_context();
  cuuint64_t dims[3] = {cols, rows, batch};
  cuuint64_t strides[2] = {ld * 2, batch_stride * 2};
  cuuint32_t box[3] = {box_cols, box_rows, 1};
  cuuint32_t elem[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled (3-D) failed with CUresult %d", (int)r);
    return false;
  }
  return true;
}

bool tc_gemm_supported(const TcGemmArgs& g, int dtype) {
  if (dtype != TB200_F16 && dtype != TB200_BF16) return false;
  if (g.M <= 0 || g.N <= 0 || g.K <= 0) return false;
  if (g.M >= (1ll << 31) || g.N >= (1ll << 31) || g.K >= (1ll << 31)) return false;
  if (!aligned16(g.a) || !aligned16(g.b) || !aligned16(g.c)) return false;
  if (g.a_ld % 8 || g.b_ld % 8 || g.c_ld % 8 || g.N % 8) return false;
  if (g.a_ld < (g.a_kmajor ? g.K : g.M) || g.b_ld < (g.b_kmajor ? g.K : g.N) || g.c_ld < g.N) return false;
  if (g.geglu_out) {
    if (!aligned16(g.geglu_out) || (g.N / 2) % 8 || !g.a_kmajor || !g.b_kmajor) return false;
    if (g.bias && (reinterpret_cast<uintptr_t>(g.bias) & 1)) return false;
  }
  return encode_fn() != nullptr;
}

template <typename T, bool AK, bool BK_, bool GEGLU>
static int launch_variant(const TcGemmArgs& g, const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p,
                          cudaStream_t st) {
  auto kern = gemm_tc_kernel<T, AK, BK_, GEGLU>;
  static std::atomic<unsigned long long> optin_done{0};
  const cudaError_t attr_err = smem_optin_per_device(optin_done, reinterpret_cast<const void*>(kern), SMEM_BYTES);
  if (attr_err != cudaSuccess) {
    set_error("gemm_tc: cudaFuncSetAttribute failed: %s", cudaGetErrorString(attr_err));
    return (int)attr_err;
  }
  const int tiles = p.num_m_tiles * p.num_n_tiles;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kern<<<grid, NUM_THREADS, SMEM_BYTES, st>>>(ma, mb, p);
  return launch_status("gemm_tc");
}

int launch_gemm_tc(const TcGemmArgs& g, int dtype, cudaStream_t st) {
  CUtensorMap ma, mb;
  bool ok;
  if (g.a_kmajor)
    ok = make_tensor_map_2d(&ma, g.a, (uint64_t)g.M, (uint64_t)g.K, (uint64_t)g.a_ld, 128, 64);
  else
    ok = make_tensor_map_2d(&ma, g.a, (uint64_t)g.K, (uint64_t)g.M, (uint64_t)g.a_ld, 64, 64);
  if (!ok) return TB200_ERR_UNSUPPORTED;
  if (g.b_kmajor)
    ok = make_tensor_map_2d(&mb, g.b, (uint64_t)g.N, (uint64_t)g.K, (uint64_t)g.b_ld, 128, 64);
  else
    ok = make_tensor_map_2d(&mb, g.b, (uint64_t)g.K, (uint64_t)g.N, (uint64_t)g.b_ld, 64, 64);
  if (!ok) return TB200_ERR_UNSUPPORTED;

  GemmParams p;
  p.M = (int)g.M;
  p.N = (int)g.N;
  p.K = (int)g.K;
  p.num_m_tiles = (int)ceil_div(g.M, BM);
  p.num_n_tiles = g.geglu_out ? (int)ceil_div(g.N / 2, BN / 2) : (int)ceil_div(g.N, BN);
  p.num_k_blocks = (int)ceil_div(g.K, BK);
  p.c = g.c;
  p.c_ld = g.c_ld;
  p.bias = g.bias;
  p.geglu_out = g.geglu_out;
  p.gelu_tanh = g.gelu_tanh;
  p.row_scale = g.row_scale;
  p.status = device_status_ptr();

  const bool bf = dtype == TB200_BF16;
  if (g.geglu_out)
    return bf ? launch_variant<__nv_bfloat16, true, true, true>(g, ma, mb, p, st)
              : launch_variant<__half, true, true, true>(g, ma, mb, p, st);
  if (g.a_kmajor && g.b_kmajor)
    return bf ? launch_variant<__nv_bfloat16, true, true, false>(g, ma, mb, p, st)
              : launch_variant<__half, true, true, false>(g, ma, mb, p, st);
  if (g.a_kmajor && !g.b_kmajor)
    return bf ? launch_variant<__nv_bfloat16, true, false, false>(g, ma, mb, p, st)
              : launch_variant<__half, true, false, false>(g, ma, mb, p, st);
  if (!g.a_kmajor && !g.b_kmajor)
    return bf ? launch_variant<__nv_bfloat16, false, false, false>(g, ma, mb, p, st)
              : launch_variant<__half, false, false, false>(g, ma, mb, p, st);
  set_error("gemm_tc: operand layout (A MN-major, B K-major) is not instantiated");
  return TB200_ERR_UNSUPPORTED;
}

}  // namespace tb200

// Reads the device status word (synchronises the device): 0 when no bounded wait of a
// tensor-core kernel has expired since the library was loaded, otherwise the code of the
// first wait that gave up. `reset` != 0 clears it afterwards.
extern "C" int tb200_device_status(int reset) {
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, tb200::g_device_status, sizeof(int));
  if (e != cudaSuccess) {
    tb200::set_error("device_status: %s", cudaGetErrorString(e));
    return -(int)e - 1000;
  }
  if (reset && v != 0) {
    int zero = 0;
    cudaMemcpyToSymbol(tb200::g_device_status, &zero, sizeof(int));
  }
  return v;
}

// Test hook of the calling thread. mode 1: the next attention forward launches of this thread run
// with a wait limit of about one millisecond, and the producer of CTA (0, 0) leaves out the bulk
// copy of its second key tile (it touches no memory it would not otherwise touch), so that the
// MMA issuer's wait for that tile runs out: the kernel must still end, free its tensor memory
// and leave a non-zero code in the device status word. mode 0: normal operation. Returns the
// old mode.
extern "C" int tb200_test_wait_fault(int mode) {
  const int old = tb200::g_test_wait_fault;
  tb200::g_test_wait_fault = mode;
  return old;
}
