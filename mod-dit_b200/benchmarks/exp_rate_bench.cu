// Microbenchmark: clocks a softmax warp needs for the exponentials of 64 columns of one row (P = exp2(S * scale -
// ref), packed to bfloat16, row sum), as a function of the warps per scheduler and of how the loop is written.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -I mod-dit_b200/csrc -I include \
//        -o exp_rate_bench mod-dit_b200/benchmarks/exp_rate_bench.cu && ./exp_rate_bench
//
// One CTA per SM with 1 to 4 warps per scheduler, inputs in registers, no memory traffic.  The exponential unit
// does 16 results per clock and SM, so 64 columns cost a scheduler 512 clocks of unit time whatever else happens.
// Measured on a B200: the bare ex2 instructions reach that with two warps (517) and 576 with one; the loop as the
// sparse forward has it needs 1069 clocks with one warp per scheduler, 594 per half row with two, 533 with four.
// In this kernel the one-warp figure depends on the row-sum chains (no sums: 652; four packed chains: 584; eight:
// 988; staging or skewing the loop in the source changes nothing), but inside the forward kernels the same change
// of chains moved nothing (two, three and four chains within 1.5 % of each other on every workload).
#include <cstdio>
#include <cstdint>
#include <cuda_bf16.h>
#include "ptx.cuh"
using namespace moddit;
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ void exp_half(const float* v, float scale_log2, float ref, uint32_t* pk, uint64_t& sum2a, uint64_t& sum2b) {
  const uint64_t scale2 = ptx::pack_f32x2(scale_log2, scale_log2);
  const uint64_t nref2 = ptx::pack_f32x2(-ref, -ref);
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const uint64_t x2 = ptx::fma_f32x2(ptx::pack_f32x2(v[2 * i], v[2 * i + 1]), scale2, nref2);
    float x0, x1;
    ptx::unpack_f32x2(x2, x0, x1);
    float p0 = ptx::ex2(x0), p1 = ptx::ex2(x1);
    const uint64_t p2 = ptx::pack_f32x2(p0, p1);
    if (i & 1) sum2b = ptx::add_f32x2(sum2b, p2); else sum2a = ptx::add_f32x2(sum2a, p2);
    pk[i] = pack2(p0, p1);
  }
}
// all FMAs, then all exponentials, then the packing: in place
__device__ __forceinline__ void exp_half_staged(float* v, float scale_log2, float ref, uint32_t* pk, uint64_t& sum2a, uint64_t& sum2b) {
  const uint64_t scale2 = ptx::pack_f32x2(scale_log2, scale_log2);
  const uint64_t nref2 = ptx::pack_f32x2(-ref, -ref);
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const uint64_t x2 = ptx::fma_f32x2(ptx::pack_f32x2(v[2 * i], v[2 * i + 1]), scale2, nref2);
    ptx::unpack_f32x2(x2, v[2 * i], v[2 * i + 1]);
  }
#pragma unroll
  for (int i = 0; i < 64; ++i) v[i] = ptx::ex2(v[i]);
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const uint64_t p2 = ptx::pack_f32x2(v[2 * i], v[2 * i + 1]);
    if (i & 1) sum2b = ptx::add_f32x2(sum2b, p2); else sum2a = ptx::add_f32x2(sum2a, p2);
    pk[i] = pack2(v[2 * i], v[2 * i + 1]);
  }
}
// blocks of 8 pairs, skewed: exponentials of block b are issued before the packing of block b - 1
template <int BP>
__device__ __forceinline__ void exp_half_skew(const float* v, float scale_log2, float ref, uint32_t* pk, uint64_t& sum2a, uint64_t& sum2b) {
  const uint64_t scale2 = ptx::pack_f32x2(scale_log2, scale_log2);
  const uint64_t nref2 = ptx::pack_f32x2(-ref, -ref);
  float p[2][2 * BP];
#pragma unroll
  for (int b = 0; b <= 32 / BP; ++b) {
    if (b < 32 / BP) {
#pragma unroll
      for (int i = 0; i < BP; ++i) {
        const int c = b * BP + i;
        const uint64_t x2 = ptx::fma_f32x2(ptx::pack_f32x2(v[2 * c], v[2 * c + 1]), scale2, nref2);
        float x0, x1;
        ptx::unpack_f32x2(x2, x0, x1);
        p[b & 1][2 * i] = ptx::ex2(x0);
        p[b & 1][2 * i + 1] = ptx::ex2(x1);
      }
    }
    if (b > 0) {
#pragma unroll
      for (int i = 0; i < BP; ++i) {
        const int c = (b - 1) * BP + i;
        const float p0 = p[(b - 1) & 1][2 * i], p1 = p[(b - 1) & 1][2 * i + 1];
        const uint64_t p2 = ptx::pack_f32x2(p0, p1);
        if (c & 1) sum2b = ptx::add_f32x2(sum2b, p2); else sum2a = ptx::add_f32x2(sum2a, p2);
        pk[c] = pack2(p0, p1);
      }
    }
  }
}
// as exp_half, without the sums / without the 16-bit conversion
template <bool SUM, bool CVT>
__device__ __forceinline__ void exp_half_part(const float* v, float scale_log2, float ref, uint32_t* pk, uint64_t& sum2a, uint64_t& sum2b) {
  const uint64_t scale2 = ptx::pack_f32x2(scale_log2, scale_log2);
  const uint64_t nref2 = ptx::pack_f32x2(-ref, -ref);
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const uint64_t x2 = ptx::fma_f32x2(ptx::pack_f32x2(v[2 * i], v[2 * i + 1]), scale2, nref2);
    float x0, x1;
    ptx::unpack_f32x2(x2, x0, x1);
    float p0 = ptx::ex2(x0), p1 = ptx::ex2(x1);
    if (SUM) {
      const uint64_t p2 = ptx::pack_f32x2(p0, p1);
      if (i & 1) sum2b = ptx::add_f32x2(sum2b, p2); else sum2a = ptx::add_f32x2(sum2a, p2);
    }
    pk[i] = CVT ? pack2(p0, p1) : (__float_as_uint(p0) ^ __float_as_uint(p1));
  }
}
// NA packed accumulators (NA > 0) or -NA scalar ones
template <int NA>
__device__ __forceinline__ void exp_half_acc(const float* v, float scale_log2, float ref, uint32_t* pk, uint64_t& sum2a, uint64_t& sum2b) {
  const uint64_t scale2 = ptx::pack_f32x2(scale_log2, scale_log2);
  const uint64_t nref2 = ptx::pack_f32x2(-ref, -ref);
  constexpr int N = NA > 0 ? NA : -NA;
  uint64_t a2[N];
  float a1[N];
#pragma unroll
  for (int j = 0; j < N; ++j) { a2[j] = 0; a1[j] = 0.f; }
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const uint64_t x2 = ptx::fma_f32x2(ptx::pack_f32x2(v[2 * i], v[2 * i + 1]), scale2, nref2);
    float x0, x1;
    ptx::unpack_f32x2(x2, x0, x1);
    float p0 = ptx::ex2(x0), p1 = ptx::ex2(x1);
    if (NA > 0) a2[i % N] = ptx::add_f32x2(a2[i % N], ptx::pack_f32x2(p0, p1));
    else { a1[(2 * i) % N] += p0; a1[(2 * i + 1) % N] += p1; }
    pk[i] = pack2(p0, p1);
  }
  if (NA > 0) {
#pragma unroll
    for (int j = 0; j < N; ++j) { if (j & 1) sum2b = ptx::add_f32x2(sum2b, a2[j]); else sum2a = ptx::add_f32x2(sum2a, a2[j]); }
  } else {
    float t = 0.f;
#pragma unroll
    for (int j = 0; j < N; ++j) t += a1[j];
    sum2a = ptx::add_f32x2(sum2a, ptx::pack_f32x2(t, 0.f));
  }
}
template <int MODE>
__global__ void k(float* out, long long* clk, int iters, float sc) {
  float v[64];
  for (int i = 0; i < 64; ++i) v[i] = (threadIdx.x * 64 + i) * 1e-4f;
  uint64_t sa = 0, sb = 0;
  uint32_t acc = 0;
  __syncthreads();
  long long t0 = clock64();
  for (int it = 0; it < iters; ++it) {
    uint32_t pk[32];
    if (MODE != 1) {
      float w[64];
#pragma unroll
      for (int i = 0; i < 64; ++i) w[i] = v[i];
      if (MODE == 0) exp_half(w, sc, (float)it * 1e-3f, pk, sa, sb);
      if (MODE == 2) exp_half_staged(w, sc, (float)it * 1e-3f, pk, sa, sb);
      if (MODE == 3) exp_half_skew<8>(w, sc, (float)it * 1e-3f, pk, sa, sb);
      if (MODE == 4) exp_half_skew<4>(w, sc, (float)it * 1e-3f, pk, sa, sb);
      if (MODE == 5) exp_half_part<false, true>(w, sc, (float)it * 1e-3f, pk, sa, sb);
      if (MODE == 6) exp_half_part<true, false>(w, sc, (float)it * 1e-3f, pk, sa, sb);
      if (MODE == 7) exp_half_skew<16>(w, sc, (float)it * 1e-3f, pk, sa, sb);
      if (MODE == 8) exp_half_acc<4>(w, sc, (float)it * 1e-3f, pk, sa, sb);
      if (MODE == 9) exp_half_acc<8>(w, sc, (float)it * 1e-3f, pk, sa, sb);
      if (MODE == 10) exp_half_acc<-4>(w, sc, (float)it * 1e-3f, pk, sa, sb);
      if (MODE == 11) exp_half_acc<-8>(w, sc, (float)it * 1e-3f, pk, sa, sb);
      if (MODE == 12) exp_half_acc<-2>(w, sc, (float)it * 1e-3f, pk, sa, sb);
#pragma unroll
      for (int i = 0; i < 32; ++i) acc ^= pk[i];
    } else {
      // exponentials only
#pragma unroll
      for (int i = 0; i < 64; ++i) acc ^= __float_as_uint(ptx::ex2(v[i] + (float)it));
    }
  }
  long long t1 = clock64();
  float a, b; ptx::unpack_f32x2(sa, a, b); float c, d; ptx::unpack_f32x2(sb, c, d);
  out[blockIdx.x * blockDim.x + threadIdx.x] = a + b + c + d + __uint_as_float(acc);
  if (threadIdx.x == 0 && blockIdx.x == 0) clk[0] = t1 - t0;
}
int main() {
  float* out; long long* clk;
  cudaMalloc(&out, 148 * 1024 * 4); cudaMalloc(&clk, 8);
  const int iters = 2000;
  const char* names[] = {"exp_half as shipped", "ex2 only", "staged in place", "skew 8 pairs", "skew 4 pairs", "no sums", "no 16-bit conversion", "skew 16 pairs", "4 packed accumulators", "8 packed accumulators", "4 scalar accumulators", "8 scalar accumulators", "2 scalar accumulators"};
  for (int mode = 0; mode < 13; ++mode)
    for (int w = 1; w <= 4; ++w) {
      for (int rep = 0; rep < 2; ++rep) {
        switch (mode) {
          case 0: k<0><<<148, 128 * w>>>(out, clk, iters, 0.1f); break;
          case 1: k<1><<<148, 128 * w>>>(out, clk, iters, 0.1f); break;
          case 2: k<2><<<148, 128 * w>>>(out, clk, iters, 0.1f); break;
          case 3: k<3><<<148, 128 * w>>>(out, clk, iters, 0.1f); break;
          case 4: k<4><<<148, 128 * w>>>(out, clk, iters, 0.1f); break;
          case 5: k<5><<<148, 128 * w>>>(out, clk, iters, 0.1f); break;
          case 6: k<6><<<148, 128 * w>>>(out, clk, iters, 0.1f); break;
          case 7: k<7><<<148, 128 * w>>>(out, clk, iters, 0.1f); break;
          case 8: k<8><<<148, 128 * w>>>(out, clk, iters, 0.1f); break;
          case 9: k<9><<<148, 128 * w>>>(out, clk, iters, 0.1f); break;
          case 10: k<10><<<148, 128 * w>>>(out, clk, iters, 0.1f); break;
          case 11: k<11><<<148, 128 * w>>>(out, clk, iters, 0.1f); break;
          case 12: k<12><<<148, 128 * w>>>(out, clk, iters, 0.1f); break;
        }
        cudaDeviceSynchronize();
      }
      long long h; cudaMemcpy(&h, clk, 8, cudaMemcpyDeviceToHost);
      printf("mode %d (%s) warps/scheduler %d: %.1f clocks per 64-column half row per warp, %.1f per half row per scheduler\n", mode,
             names[mode], w, (double)h / iters, (double)h / iters / w);
    }
  printf("err %s\n", cudaGetErrorString(cudaGetLastError()));
  return 0;
}
