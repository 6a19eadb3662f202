// Micro-benchmark: issue-to-completion rate of tcgen05.mma (kind::f16, bf16) from one thread of one CTA per SM.
// Timing only; operands are zeros.  Variants chosen by argv[1].
#include "../csrc/ca_common.cuh"
#include <cstdio>
#include <cstdlib>
using namespace ca;

__device__ long long g_cycles[160];
__device__ int g_status;

struct P { int variant; int n_mma; int N; int use_elect; };

__global__ void __launch_bounds__(128, 1) mma_rate_kernel(P p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    ptx::mbar_init(ptx::smem_u32(&bar), 1);
    ptx::mbar_fence_init();
    ptx::fence_proxy_async_smem();
  }
  // zero the operand tiles (96 KB)
  for (int i = threadIdx.x; i < 96 * 1024 / 16; i += blockDim.x)
    reinterpret_cast<uint4*>(smem_raw + (base - ptx::smem_u32(smem_raw)))[i] = make_uint4(0, 0, 0, 0);
  ptx::fence_proxy_async_smem();
  if (warp == 0) {
    ptx::tmem_alloc(ptx::smem_u32(&tmem_base), 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = tmem_base;
  bool leader = false;
  if (warp == 1) {
    if (p.use_elect) {
      uint32_t pred;
      asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(pred));
      leader = pred != 0;
    } else {
      leader = lane == 0;
    }
  }
  if (leader && p.variant < 5) {
    const uint32_t idesc_ss = ptx::make_idesc_f16(1, 128, p.N, 0, 0);
    const uint32_t idesc_pv = ptx::make_idesc_f16(1, 128, 128, 0, 1);
    const uint64_t a0 = ptx::make_smem_desc_sw128(base, 0, 1024);
    const uint64_t b0 = ptx::make_smem_desc_sw128(base + 32768, 0, 1024);
    const uint64_t v0 = ptx::make_smem_desc_sw128(base + 32768, 16384, 1024);
    long long t0 = clock64();
    const int groups = p.n_mma / 8;
    for (int g = 0; g < groups; ++g) {
      const uint32_t d = tmem + (g & 1) * 128u + ((p.variant == 3 && (g & 2)) ? 256u : 0u);
      if (p.variant == 0 || p.variant == 2) {        // SS, like Q.K^T (variant 2: N = 256)
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint64_t o = static_cast<uint64_t>(((k >> 2) * 16384 + (k & 3) * 32) >> 4);
          ptx::mma_ss(d, a0 + o, b0 + o, idesc_ss, k > 0 ? 1u : 0u);
        }
      } else if (p.variant == 1) {                    // TS, like P.V (A = 64 TMEM columns, B MN-major)
#pragma unroll
        for (int k = 0; k < 8; ++k)
          ptx::mma_ts(tmem + 256u + (g & 1) * 128u, tmem + (g & 1) * 128u + k * 8, v0 + static_cast<uint64_t>(k * (2048 >> 4)), idesc_pv, k > 0 ? 1u : 0u);
      } else if (p.variant == 3) {                    // alternate SS and TS groups like the attention loop
        if (g & 1) {
#pragma unroll
          for (int k = 0; k < 8; ++k)
            ptx::mma_ts(tmem + 256u + (g & 2) * 64u, tmem + (g & 2) * 64u + k * 8, v0 + static_cast<uint64_t>(k * (2048 >> 4)), idesc_pv, k > 0 ? 1u : 0u);
        } else {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint64_t o = static_cast<uint64_t>(((k >> 2) * 16384 + (k & 3) * 32) >> 4);
            ptx::mma_ss(tmem + (g & 2) * 64u, a0 + o, b0 + o, idesc_ss, k > 0 ? 1u : 0u);
          }
        }
      }
    }
    ptx::tc_commit(ptx::smem_u32(&bar));
    const bool ok = ptx::mbar_wait_bounded(ptx::smem_u32(&bar), 0, &abort_flag, 2000000000ull);
    long long t1 = clock64();
    g_cycles[blockIdx.x] = t1 - t0;
    if (!ok) atomicOr(&g_status, 1);
  }
  if (warp == 2 && (p.variant == 5 || p.variant == 6)) {
    // the attention kernel's issue pattern: slot-dependent descriptors, S then PV groups
    const uint32_t idesc_ss = ptx::make_idesc_f16(1, 128, 128, 0, 0);
    const uint32_t idesc_pv = ptx::make_idesc_f16(1, 128, 128, 0, 1);
    const uint64_t q_desc[2] = {ptx::make_smem_desc_sw128(base, 0, 1024), ptx::make_smem_desc_sw128(base + 32768, 0, 1024)};
    const uint64_t k_desc0 = ptx::make_smem_desc_sw128(base + 65536, 0, 1024);
    const uint64_t v_desc0 = ptx::make_smem_desc_sw128(base + 65536, 16384, 1024);
    const uint32_t tS[2] = {tmem, tmem + 128u};
    const uint32_t tO[2] = {tmem + 256u, tmem + 384u};
    const int groups = p.n_mma / 8;
    long long t0 = clock64();
    if (p.variant == 5) {
      if (lane == 0) {
        int ring = 0;
        for (int g = 0; g < groups; ++g) {
          const int tile = (g >> 1) & 1;
          const int slot = (ring * p.use_elect) & 0;  // runtime value (always slot 0: 32 KB of operands exist)
          ring += 1;
          if (g & 1) {
            const uint64_t vd = v_desc0 + static_cast<uint64_t>(slot * (32768 >> 4));
#pragma unroll
            for (int k = 0; k < 8; ++k) ptx::mma_ts(tO[tile], tS[tile] + k * 8, vd + static_cast<uint64_t>(k * (2048 >> 4)), idesc_pv, k > 0 ? 1u : 0u);
          } else {
            const uint64_t qd = q_desc[tile];
            const uint64_t kd = k_desc0 + static_cast<uint64_t>(slot * (32768 >> 4));
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const uint64_t o = static_cast<uint64_t>(((k >> 2) * 16384 + (k & 3) * 32) >> 4);
              ptx::mma_ss(tS[tile], qd + o, kd + o, idesc_ss, k > 0 ? 1u : 0u);
            }
          }
        }
        ptx::tc_commit(ptx::smem_u32(&bar));
      }
    } else {
      int ring = 0;
      for (int g = 0; g < groups; ++g) {
        const int tile = (g >> 1) & 1;
        const int slot = (ring * p.use_elect) & 0;
        ring += 1;
        if (g & 1) {
          const uint64_t vd = v_desc0 + static_cast<uint64_t>(slot * (32768 >> 4));
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            uint32_t pred;
            asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(pred));
            if (pred) ptx::mma_ts(tO[tile], tS[tile] + k * 8, vd + static_cast<uint64_t>(k * (2048 >> 4)), idesc_pv, k > 0 ? 1u : 0u);
          }
        } else {
          const uint64_t qd = q_desc[tile];
          const uint64_t kd = k_desc0 + static_cast<uint64_t>(slot * (32768 >> 4));
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint64_t o = static_cast<uint64_t>(((k >> 2) * 16384 + (k & 3) * 32) >> 4);
            uint32_t pred;
            asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(pred));
            if (pred) ptx::mma_ss(tS[tile], qd + o, kd + o, idesc_ss, k > 0 ? 1u : 0u);
          }
        }
      }
      if (lane == 0) ptx::tc_commit(ptx::smem_u32(&bar));
    }
    if (lane == 0) {
      const bool ok = ptx::mbar_wait_bounded(ptx::smem_u32(&bar), 0, &abort_flag, 2000000000ull);
      long long t1 = clock64();
      g_cycles[blockIdx.x] = t1 - t0;
      if (!ok) atomicOr(&g_status, 1);
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, 512);
  }
}

int main(int argc, char** argv) {
  P p;
  p.variant = argc > 1 ? atoi(argv[1]) : 0;
  p.n_mma = argc > 2 ? atoi(argv[2]) : 4096;
  p.N = p.variant == 2 ? 256 : 128;
  if (getenv("MMA_N")) p.N = atoi(getenv("MMA_N"));
  p.use_elect = argc > 3 ? atoi(argv[3]) : 0;
  int grid = argc > 4 ? atoi(argv[4]) : 148;
  const int smem = 97 * 1024 + 1024;
  cudaFuncSetAttribute(mma_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0); cudaEventCreate(&e1);
  for (int rep = 0; rep < 3; ++rep) {
    cudaEventRecord(e0);
    mma_rate_kernel<<<grid, 128, smem>>>(p);
    cudaEventRecord(e1);
    cudaError_t err = cudaDeviceSynchronize();
    if (err != cudaSuccess) { printf("error %s\n", cudaGetErrorString(err)); return 1; }
    float ms; cudaEventElapsedTime(&ms, e0, e1);
    long long cyc[160]; int st;
    cudaMemcpyFromSymbol(cyc, g_cycles, sizeof(cyc));
    cudaMemcpyFromSymbol(&st, g_status, sizeof(int));
    double flops = 2.0 * 128 * p.N * 16 * p.n_mma * grid;
    printf("variant %d N %d elect %d grid %d: %lld cycles for %d MMAs = %.1f cycles/MMA (CTA 0), kernel %.1f us -> %.0f TFLOP/s, eff clock %.2f GHz, status %d\n",
           p.variant, p.N, p.use_elect, grid, cyc[0], p.n_mma, (double)cyc[0] / p.n_mma, ms * 1e3, flops / (ms * 1e-3) / 1e12,
           cyc[0] / (ms * 1e-3) / 1e9, st);
  }
  return 0;
}
