// Developer micro-benchmark: cycles per tcgen05.mma (M = 128, K = 16, bf16) for N = 64 / 128 / 256 and every combination of
// K-major / MN-major shared-memory operands; one CTA, one issuing thread, all-zero operands.  Not part of the library.
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 --expt-relaxed-constexpr mma_timing.cu -o mma_timing -lcuda && ./mma_timing 256
#include <cstdio>
#include <cstdlib>
#include "ua_ptx.cuh"
using namespace ua::ptx;

__global__ void __launch_bounds__(128, 1) bench_kernel(long long* out, int reps) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ uint32_t misc[4];
  __shared__ __align__(8) unsigned long long bar_mem[2];
  for (int x = threadIdx.x; x < 160 * 1024 / 16; x += 128) reinterpret_cast<uint4*>(smem)[x] = make_uint4(0, 0, 0, 0);
  const uint32_t bar = smem_u32(&bar_mem[0]);
  if (threadIdx.x == 0) { misc[1] = 0; misc[2] = 0; mbar_init(bar, 1); mbar_init_fence(); }
  if (threadIdx.x < 32) { tmem_alloc(smem_u32(misc), 512); tmem_relinquish(); }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = misc[0];
  volatile int* abort_flag = reinterpret_cast<volatile int*>(misc + 1);
  if (threadIdx.x == 0) {
    const uint32_t sb = smem_u32(smem);
    int phase = 0, slot = 0;
    for (int variant = 0; variant < 4; ++variant) {
      const int a_mn = variant >> 1, b_mn = variant & 1;
      for (int n = 64; n <= 256; n *= 2) {
        for (int mode = 0; mode < 2; ++mode) {   // mode 0: all into one accumulator; mode 1: alternate two accumulators
          const uint32_t idesc = idesc_bf16(128, n, a_mn, b_mn);
          const uint64_t a0 = desc_from_lo(desc_lo(sb, a_mn ? 16384 : 16));
          const uint64_t b0 = desc_from_lo(desc_lo(sb + 65536, b_mn ? 16384 : 16));
          const uint64_t sa = a_mn ? 128 : 2, sbb = b_mn ? 128 : 2;
          long long t0 = clock64();
          for (int r = 0; r < reps; ++r) {
            const int k = r & 3;
            const uint32_t d = tmem + ((mode && (r & 4)) ? 256 : 0);
            mma_ss(d, a0 + k * sa, b0 + k * sbb, idesc, r > 7);
          }
          tc_commit(bar);
          long long t1 = clock64();
          if (!mbar_wait(bar, phase & 1, abort_flag)) { out[63] = -1; break; }
          long long t2 = clock64();
          ++phase;
          out[slot * 2] = t1 - t0;
          out[slot * 2 + 1] = t2 - t0;
          ++slot;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) tmem_dealloc(tmem, 512);
}

int main(int argc, char** argv) {
  const int reps = argc > 1 ? atoi(argv[1]) : 256;
  long long* d;
  cudaMalloc(&d, 64 * sizeof(long long));
  cudaMemset(d, 0, 64 * sizeof(long long));
  const int smem = 161 * 1024 + 1024;
  cudaFuncSetAttribute(bench_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  for (int it = 0; it < 2; ++it) {
    bench_kernel<<<1, 128, smem>>>(d, reps);
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { printf("error %s\n", cudaGetErrorString(e)); return 1; }
  }
  long long h[64];
  cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost);
  int slot = 0;
  for (int variant = 0; variant < 4; ++variant)
    for (int n = 64; n <= 256; n *= 2)
      for (int mode = 0; mode < 2; ++mode, ++slot)
        printf("a_mn=%d b_mn=%d N=%3d mode=%d: issue %.1f cyc/mma, complete %.1f cyc/mma\n", variant >> 1, variant & 1, n, mode,
               (double)h[slot * 2] / reps, (double)h[slot * 2 + 1] / reps);
  printf("flag %lld\n", h[63]);
  return 0;
}
