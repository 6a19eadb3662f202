// Micro-benchmark of the S -> softmax -> P hand-off: issuer thread issues 8 MMAs + commit(bar_s); 128 worker threads wait
// bar_s and arrive on bar_p; issuer waits bar_p.  Reports cycles per round trip beyond the 512 cycles of MMA work.
#include "../csrc/ca_common.cuh"
#include <cstdio>
#include <cstdlib>
using namespace ca;
__device__ long long g_cycles[160];
__device__ int g_status;
struct P { int mode; int iters; int n_mma; };

__global__ void __launch_bounds__(256, 1) handoff_kernel(P p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  __shared__ uint64_t bar_s, bar_p;
  __shared__ uint32_t tmem_base;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int arrivals = p.mode == 0 ? 128 : (p.mode == 1 ? 4 : 128);
  if (threadIdx.x == 0) {
    abort_flag = 0;
    ptx::mbar_init(ptx::smem_u32(&bar_s), 1);
    ptx::mbar_init(ptx::smem_u32(&bar_p), arrivals);
    ptx::mbar_fence_init();
    ptx::fence_proxy_async_smem();
  }
  for (int i = threadIdx.x; i < 64 * 1024 / 16; i += blockDim.x)
    reinterpret_cast<uint4*>(smem_raw + (base - ptx::smem_u32(smem_raw)))[i] = make_uint4(0, 0, 0, 0);
  ptx::fence_proxy_async_smem();
  if (warp == 4) { ptx::tmem_alloc(ptx::smem_u32(&tmem_base), 512); ptx::tmem_relinquish(); }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = tmem_base;
  volatile int* af = &abort_flag;
  if (warp < 4) {                       // workers ("softmax" threads)
    for (int it = 0; it < p.iters; ++it) {
      bool ok = ptx::mbar_wait_bounded(ptx::smem_u32(&bar_s), it & 1, af, 1000000000ull);
      if (!__all_sync(0xffffffffu, ok)) break;
      ptx::tc_fence_after();
      if (p.mode == 2) {                // also read 32 columns of S from TMEM like a real consumer would
        uint32_t v[32];
        ptx::tmem_ld32(tmem + (static_cast<uint32_t>(warp * 32) << 16), v);
        ptx::tc_wait_ld();
        if (v[0] == 0x12345678u) g_status = 2;
      }
      ptx::tc_fence_before();
      if (p.mode == 1) { __syncwarp(); if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&bar_p)); }
      else ptx::mbar_arrive(ptx::smem_u32(&bar_p));
    }
  } else if (warp == 5 && lane == 0) {  // issuer
    const uint32_t idesc = ptx::make_idesc_f16(1, 128, 128, 0, 0);
    const uint64_t a0 = ptx::make_smem_desc_sw128(base, 0, 1024);
    const uint64_t b0 = ptx::make_smem_desc_sw128(base + 32768, 0, 1024);
    long long t0 = clock64();
    bool ok = true;
    for (int it = 0; it < p.iters && ok; ++it) {
      for (int k = 0; k < p.n_mma; ++k) {
        const uint64_t o = static_cast<uint64_t>((((k & 7) >> 2) * 16384 + (k & 3) * 32) >> 4);
        ptx::mma_ss(tmem, a0 + o, b0 + o, idesc, k > 0 ? 1u : 0u);
      }
      ptx::tc_commit(ptx::smem_u32(&bar_s));
      ok = ptx::mbar_wait_bounded(ptx::smem_u32(&bar_p), it & 1, af, 1000000000ull);
      ptx::tc_fence_after();
    }
    long long t1 = clock64();
    g_cycles[blockIdx.x] = t1 - t0;
    if (!ok) atomicOr(&g_status, 1);
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 4) { ptx::tc_fence_after(); ptx::tmem_dealloc(tmem, 512); }
}

int main(int argc, char** argv) {
  P p; p.mode = argc > 1 ? atoi(argv[1]) : 0; p.iters = argc > 2 ? atoi(argv[2]) : 2000; p.n_mma = argc > 3 ? atoi(argv[3]) : 8;
  const int smem = 66 * 1024;
  cudaFuncSetAttribute(handoff_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  for (int rep = 0; rep < 2; ++rep) {
    handoff_kernel<<<148, 256, smem>>>(p);
    cudaError_t err = cudaDeviceSynchronize();
    if (err != cudaSuccess) { printf("error %s\n", cudaGetErrorString(err)); return 1; }
    long long cyc[160]; int st;
    cudaMemcpyFromSymbol(cyc, g_cycles, sizeof(cyc)); cudaMemcpyFromSymbol(&st, g_status, sizeof(int));
    printf("mode %d (%s), %d MMAs per round: %.1f cycles per round trip, %.1f beyond the MMA work, status %d\n", p.mode,
           p.mode == 0 ? "128 arrivals" : p.mode == 1 ? "4 elected arrivals" : "128 arrivals + TMEM load", p.n_mma,
           (double)cyc[0] / p.iters, (double)cyc[0] / p.iters - 64.0 * p.n_mma, st);
  }
  return 0;
}
