// Measuring device, not part of the library: cycles per tcgen05.mma instruction (M = 128, K = 16, bf16,
// fp32 accumulation) as a function of N, of the A operand's source (shared or tensor memory), of the
// layout of B (K-major or MN-major), of what the other warps of the CTA do meanwhile (nothing, tensor
// memory loads, or arithmetic that saturates the schedulers) and of how the issuing loop is entered
// (lane 0 alone, the whole warp with one elected lane, or two warps on two schedulers).
// One CTA per SM; operands hold pseudo-random values in [-2, 2); every wait is bounded.
//   python -m trident_b200.umma_probe            (compiles this file and runs it)
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <algorithm>
#include <cuda_runtime.h>
#include <cuda.h>
#include "ptx.cuh"

using namespace tb200;

constexpr bool RANDOM_DATA = true;
template <int N, int NACC, int TS, int BMN, int LD, int ISSUE>
__global__ void __launch_bounds__(320, 1)
    probe(long long* out, int iters, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* a_smem = smem;           // [128][64] bf16, 16 KB
  uint8_t* b_smem = smem + 16384;   // [256][64] bf16, 32 KB
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + 49152);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  for (int i = threadIdx.x; i < 49152 / 4; i += blockDim.x) {
    uint32_t h = (uint32_t)i * 2654435761u + 12345u + blockIdx.x * 7919u;
    h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
    // two bf16 values in [-2, 2): random sign and mantissa, exponent 0x3f (1..2) or 0x3e
    const uint32_t lo = (h & 0x807fu) | (((h >> 7) & 1u) ? 0x3f80u : 0x3f00u);
    const uint32_t hi = ((h >> 16) & 0x807fu) | (((h >> 23) & 1u) ? 0x3f80u : 0x3f00u);
    reinterpret_cast<uint32_t*>(smem)[i] = RANDOM_DATA ? (lo | (hi << 16)) : 0u;
  }
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    ptx::mbar_init(bar, ISSUE == 2 ? 2 : 1);
    *abort_flag = 0;
    ptx::fence_barrier_init();
  }
  ptx::fence_proxy_async_smem();
  if (warp == 0) {
    ptx::tmem_alloc(tmem_slot, 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (RANDOM_DATA && warp < 4) {
    uint32_t r[16];
    for (int i = 0; i < 16; ++i) {
      uint32_t h = (threadIdx.x * 16 + i) * 2654435761u + 777u;
      h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
      r[i] = (h & 0x807f807fu) | 0x3f803f00u;
    }
    ptx::tmem_st16(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + 496, r);
    ptx::tmem_st_wait();
    // zero the accumulators' columns 0..255
    uint32_t z[32];
    for (int i = 0; i < 32; ++i) z[i] = 0;
    for (int c = 0; c < 8; ++c) ptx::tmem_st32(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + c * 32, z);
    ptx::tmem_st_wait();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  {
    constexpr uint32_t idesc = ptx::make_idesc(true, false, BMN != 0, 128, N);
    const uint32_t aa = ptx::smem_u32(a_smem), ba = ptx::smem_u32(b_smem);
    const uint32_t a_tmem = tmem_base + 496;  // 8 columns of packed bf16 = a [128][16] A operand
    const int lane = threadIdx.x & 31;
    bool issuer = false, timer = false;
    uint32_t acc_col = 0;
    int my_iters = iters;
    if (ISSUE == 0) { issuer = timer = threadIdx.x == 256; }
    if (ISSUE == 1) { issuer = warp == 8; }
    if (ISSUE == 2) { issuer = (warp == 8 || warp == 9) && lane == 0; timer = threadIdx.x == 256; acc_col = (warp - 8) * N; my_iters = iters / 2; }
    if (issuer) {
      bool elected = true;
      if (ISSUE == 1) {
        uint32_t pe;
        asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.b32 %0, 1, 0, P;\n\t}" : "=r"(pe));
        elected = pe != 0;
        timer = elected;
      }
      uint64_t da[4], db[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        da[k] = ptx::make_smem_desc(aa + k * 32, 16, 1024);
        db[k] = BMN ? ptx::make_smem_desc(ba + k * 2048, 16384, 1024) : ptx::make_smem_desc(ba + k * 32, 16, 1024);
      }
      const long long t0 = clock64();
      for (int i = 0; i < my_iters; i += 4) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (elected) {
            if (TS)
              ptx::umma_ts(tmem_base + acc_col, a_tmem, db[k], idesc, 1);
            else
              ptx::umma_ss(tmem_base + acc_col, da[k], db[k], idesc, 1);
          }
        }
      }
      if (elected) ptx::umma_commit(bar);
      const long long t1 = clock64();
      if (timer) {
        ptx::mbar_wait(bar, 0, abort_flag, status, 1);
        const long long t2 = clock64();
        out[blockIdx.x * 2] = t1 - t0;
        out[blockIdx.x * 2 + 1] = t2 - t0;
      }
    }
  }
  if (LD < 0 && warp < 8) {  // ALU-busy warps, two per scheduler
    float x0 = threadIdx.x, x1 = x0 + 1, x2 = x0 + 2, x3 = x0 + 3;
    for (int n = 0; n < -LD; ++n) {
      x0 = fmaf(x0, 1.0001f, 0.5f); x1 = fmaf(x1, 1.0001f, 0.5f); x2 = fmaf(x2, 1.0001f, 0.5f); x3 = fmaf(x3, 1.0001f, 0.5f);
    }
    if (x0 + x1 + x2 + x3 == 12345.f) out[1] = 1;
  }
  if (LD > 0 && warp < 8) {
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    uint32_t acc = 0;
    for (int n = 0; n < LD; ++n) {
      uint32_t r[32];
      ptx::tmem_ld32(tmem_base + lane_off + 256 + ((n + warp) & 3) * 32, r);
      ptx::tmem_ld_wait();
      acc ^= r[n & 31];
    }
    if (acc == 0x12345) out[0] = acc;
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, 512);
  }
}

template <int N, int NACC, int TS, int BMN = 0, int LD = 0, int ISSUE = 0>
void run(int grid, long long* out, int* status, int iters, int SMEM, int reps) {
  cudaFuncSetAttribute(probe<N, NACC, TS, BMN, LD, ISSUE>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0); cudaEventCreate(&e1);
  cudaEventRecord(e0);
  for (int rep = 0; rep < reps; ++rep) probe<N, NACC, TS, BMN, LD, ISSUE><<<grid, 320, SMEM>>>(out, iters, status);
  cudaEventRecord(e1);
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) { printf("error %s\n", cudaGetErrorString(e)); exit(1); }
  float ms; cudaEventElapsedTime(&ms, e0, e1);
  printf("  %d launches in %.1f ms: %.0f TFLOP/s over the whole run\n", reps, ms, 2.0 * 128 * N * 16 * iters * grid * reps / ms / 1e9);
  std::vector<long long> h(grid * 2);
  cudaMemcpy(h.data(), out, grid * 2 * sizeof(long long), cudaMemcpyDeviceToHost);
  std::vector<long long> tot, iss;
  for (int i = 0; i < grid; ++i) { tot.push_back(h[i * 2 + 1]); iss.push_back(h[i * 2]); }
  std::sort(tot.begin(), tot.end());
  std::sort(iss.begin(), iss.end());
  int st;
  cudaMemcpy(&st, status, sizeof(int), cudaMemcpyDeviceToHost);
  const double cyc = (double)tot[tot.size() / 2] / iters;
  printf("grid %3d  N=%3d acc=%d A=%s Bmn=%d ld=%d issue=%d: %.1f cycles/instr (ideal %d; issue loop alone %.1f) -> %.0f flop/clk/SM, status %d\n",
         grid, N, NACC, TS ? "tmem" : "smem", BMN, LD, ISSUE, cyc, N / 2, (double)iss[iss.size() / 2] / iters, 2.0 * 128 * N * 16 / cyc, st);
}

int main(int argc, char** argv) {
  const int grid = 148;
  long long* out;
  int* status;
  cudaMalloc(&out, grid * 2 * sizeof(long long));
  cudaMalloc(&status, sizeof(int));
  cudaMemset(status, 0, sizeof(int));
  const int SMEM = 49152 + 1024 + 64;
  const int iters = 48000;
  const int reps = argc > 1 ? atoi(argv[1]) : 3;  // e.g. 1500 for a seconds-long run (watch the clocks beside it)
  // N, accumulators (unused), A from tensor memory, B MN-major, other warps (0 idle, > 0 tensor-memory
  // loads, < 0 arithmetic), issue structure (0 lane 0 alone, 1 elected lane of the whole warp, 2 two warps)
  run<256, 1, 0, 0, 0, 0>(grid, out, status, iters, SMEM, reps);
  run<128, 1, 0, 0, 0, 0>(grid, out, status, iters, SMEM, reps);
  run<128, 1, 1, 1, 0, 0>(grid, out, status, iters, SMEM, reps);
  run<64, 1, 0, 0, 0, 0>(grid, out, status, iters, SMEM, reps);
  run<64, 1, 1, 1, 0, 0>(grid, out, status, iters, SMEM, reps);
  run<128, 1, 1, 1, 3000, 0>(grid, out, status, iters, SMEM, reps);
  run<128, 1, 0, 0, -800000, 0>(grid, out, status, iters, SMEM, reps);
  run<128, 1, 0, 0, -800000, 1>(grid, out, status, iters, SMEM, reps);
  run<128, 1, 0, 0, -800000, 2>(grid, out, status, iters, SMEM, reps);
  run<128, 1, 1, 1, -800000, 0>(grid, out, status, iters, SMEM, reps);
  run<128, 1, 1, 1, -800000, 1>(grid, out, status, iters, SMEM, reps);
  return 0;
}
