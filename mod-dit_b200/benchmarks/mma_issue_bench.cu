// Microbenchmark: what a tcgen05.mma instruction costs the thread that issues it, on sm_100a.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -I mod-dit_b200/csrc -I include \
//        -o mma_issue_bench mod-dit_b200/benchmarks/mma_issue_bench.cu && ./mma_issue_bench
//
// One CTA per SM.  One thread (or one thread in each of two warps) issues groups of eight M128 x N x K16 bf16 MMAs
// back to back on constant shared-memory / tensor-memory operands and the elapsed SM clocks per MMA are printed,
// for N = 64 / 128 / 256, both operands in shared memory (SS) or A in tensor memory (TS), with and without a
// tcgen05.commit after every group, with extra (already complete) mbarrier waits per group, and with the other
// warps of the CTA busy on the FMA / special-function pipes.  It explains the ceiling of the sparse forward's
// single issuing thread: the pipe needs 64 clocks for an N = 128 product, the issuing warp can hand one over
// only every ~84.  Every wait is bounded (ptx::mbar_wait).
#include <cstdio>
#include <cstdint>
#include <cuda_bf16.h>
#include "ptx.cuh"
using namespace moddit;

struct Res { long long clks; int err; };

// KIND: 0 SS N128, 1 SS N256, 2 TS N128, 3 SS N64, 4 TS N64, 5 TS N256
template <int KIND>
__global__ void __launch_bounds__(384, 1) bench(Res* res, int reps, int commit_every, int issuers, int noise, int waits_per_group) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ unsigned long long bars[4];
  __shared__ uint32_t tmem_base;
  __shared__ int abort_flag;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  constexpr int N = (KIND == 1 || KIND == 5) ? 256 : ((KIND == 3 || KIND == 4) ? 64 : 128);
  constexpr bool TS = (KIND == 2 || KIND == 4 || KIND == 5);
  const uint32_t sA = ptx::smem_u32(smem);              // 128 x 128 bf16 = 32 KB
  const uint32_t sB = sA + 32768;                       // 256 x 128 bf16 = 64 KB
  for (int i = threadIdx.x; i < (96 * 1024) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0x3c003c00u;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 4; ++i) ptx::mbar_init(ptx::smem_u32(&bars[i]), 1);
    abort_flag = 0;
    ptx::fence_barrier_init();
  }
  ptx::fence_proxy_async_smem();
  if (warp == 2) { ptx::tmem_alloc(ptx::smem_u32(&tmem_base), 512); ptx::tmem_relinquish(); ptx::tc_fence_before(); }
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = tmem_base;
  volatile int* af = &abort_flag;
  if (warp < issuers && lane == 0) {
    const uint32_t idesc = ptx::idesc_f16(128, N, true, false);
    const uint64_t da = ptx::smem_desc_sw128(sA, 16, 1024);
    const uint64_t db = ptx::smem_desc_sw128(sB, 16, 1024);
    auto adv = [](uint64_t d, uint32_t bytes) { return (d & 0xffffffff00000000ull) | (uint32_t)((uint32_t)d + (bytes >> 4)); };
    const uint32_t dcol = tmem + warp * 256;            // accumulator (<= 256 columns per issuer)
    const uint32_t acol = tmem + (issuers == 1 ? 256 : (warp * 256 + 128));   // TS: A operand columns (garbage)
    const uint32_t bar_c = ptx::smem_u32(&bars[warp]);
    const uint32_t bar_w = ptx::smem_u32(&bars[2]);     // a barrier that is always "ready" for parity 1
    uint32_t par = 0;
    bool ok = true;
    const long long t0 = clock64();
    for (int r = 0; r < reps && ok; ++r) {
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint32_t off = (kk / 4) * (N * 128) + (kk % 4) * 32;
        const uint32_t offa = (kk / 4) * (128 * 128) + (kk % 4) * 32;
        if (TS) ptx::mma_ts(dcol, acol + kk * 8, adv(db, off), idesc, kk > 0);
        else ptx::mma_ss(dcol, adv(da, offa), adv(db, off), idesc, kk > 0);
      }
      for (int w = 0; w < waits_per_group; ++w) ok = ok && ptx::mbar_wait(bar_w, 1, af);
      if (commit_every && (r % commit_every) == commit_every - 1) {
        ptx::tc_commit(bar_c);
        if (commit_every >= 1000) { ok = ptx::mbar_wait(bar_c, par, af); par ^= 1; }
      }
    }
    ptx::tc_commit(ptx::smem_u32(&bars[3 - warp]) );
    // final: wait for everything
    const uint32_t fb = ptx::smem_u32(&bars[3 - warp]);
    ok = ptx::mbar_wait(fb, 0, af) && ok;
    const long long t1 = clock64();
    if (blockIdx.x == 0) { res[warp].clks = t1 - t0; res[warp].err = ok ? 0 : 1; }
  } else if (warp >= 4 && noise) {
    // softmax-like load: MUFU + FMA on registers, runs until the issuers are done (bounded)
    float x = threadIdx.x * 1e-3f, y = 0.f;
    for (int i = 0; i < reps * noise; ++i) {
#pragma unroll
      for (int j = 0; j < 16; ++j) { x = x * 1.0001f + 0.5f; y += ptx::ex2(-x); }
    }
    if (y == 12345.f) res[3].err = 7;
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 2) { ptx::tc_fence_after(); ptx::tmem_dealloc(tmem, 512); }
}

template <int KIND>
void run(const char* name, Res* d, int reps, int commit_every, int issuers, int noise, int waits) {
  cudaFuncSetAttribute(bench<KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
  cudaMemset(d, 0, sizeof(Res) * 4);
  bench<KIND><<<148, 384, 100 * 1024>>>(d, reps, commit_every, issuers, noise, waits);
  cudaError_t e = cudaDeviceSynchronize();
  Res h[4];
  cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost);
  printf("%-10s commit_every=%-5d issuers=%d noise=%d waits=%d : %.1f clk/MMA (issuer0) %.1f (issuer1) err=%d/%d cuda=%s\n", name, commit_every,
         issuers, noise, waits, (double)h[0].clks / (8.0 * reps), (double)h[1].clks / (8.0 * reps), h[0].err, h[1].err, cudaGetErrorString(e));
}

int main() {
  Res* d; cudaMalloc(&d, sizeof(Res) * 4);
  const int R = 2000;
  for (int ce : {0, 1}) {
    run<0>("SS N128", d, R, ce, 1, 0, 0);
    run<1>("SS N256", d, R, ce, 1, 0, 0);
    run<3>("SS N64", d, R, ce, 1, 0, 0);
    run<2>("TS N128", d, R, ce, 1, 0, 0);
    run<5>("TS N256", d, R, ce, 1, 0, 0);
    run<4>("TS N64", d, R, ce, 1, 0, 0);
  }
  run<0>("SS N128", d, R, 1, 2, 0, 0);
  run<2>("TS N128", d, R, 1, 2, 0, 0);
  run<0>("SS N128", d, R, 1, 1, 4, 0);
  run<2>("TS N128", d, R, 1, 1, 4, 0);
  run<0>("SS N128", d, R, 1, 1, 0, 1);
  run<0>("SS N128", d, R, 1, 1, 0, 2);
  run<2>("TS N128", d, R, 1, 1, 0, 2);
  run<0>("SS N128", d, R, 1, 1, 4, 2);
  return 0;
}
