// Block mean-pooling of Q/K and the pooled darkness map (HBM-bound and latency-bound stages).
//
// pool_blocks: one CTA per (block, head) streams the block's rows with 128-bit loads; every thread
// keeps eight fp32 column sums, row groups are combined through shared memory in a fixed order.
// Algorithmic traffic: N*D*2 bytes read + ceil(N/bs)*D*4 bytes written per head.
//
// pooled_map: one CTA per (32 query blocks, head): fp32 logits against all key blocks (warp-level tensor-core
// products of the means split into two bfloat16 terms) are kept in shared memory, then each warp normalises its rows and
// writes 1 - exp(logit - row maximum) as float16 (0 at the brightest block of a row, 1 where there is nothing;
// relative to the row maximum so that the float16 grid resolves the bright blocks).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace moddit {
namespace {

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]);

template <>
__device__ __forceinline__ void unpack8<__nv_bfloat16>(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

template <>
__device__ __forceinline__ void unpack8<__half>(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
    const float2 p = __half22float2(h);
    f[2 * i] = p.x;
    f[2 * i + 1] = p.y;
  }
}

constexpr int kPoolThreads = 256;

// Sequence-shard form of the pooling (kShard): the rows of a head are `halo_rows` rows of a halo buffer (the
// part of the first block that the previous rank holds) followed by this rank's `N` rows, and the mean of
// block `blk` goes to the rank that owns the head, at block `block_base + blk` of its (heads_per_peer,
// nb_total, D) buffer - plain peer stores.  Row order and reduction order are those of the plain form, so a
// block pooled from a shard equals the block pooled from the whole sequence bit for bit.
constexpr int kMaxPoolPeers = 8;
struct PoolShard {
  const void* halo;          // (heads, halo_cap, D) rows received from the previous rank
  int halo_rows;
  int halo_cap;
  float* peer[kMaxPoolPeers];
  int heads_per_peer;
  int nb_total;
  int block_base;
};

// D is 64 or 128: D/8 threads cover one row with one 16-byte load each.
template <typename T, int D, bool kShard>
__global__ void __launch_bounds__(kPoolThreads) pool_blocks_kernel(const T* __restrict__ x, int N, int bs,
                                                                   float* __restrict__ out,
                                                                   const __grid_constant__ PoolShard shard) {
  constexpr int kTpr = D / 8;                   // threads per row
  constexpr int kRpp = kPoolThreads / kTpr;     // rows per pass
  __shared__ float red[kRpp][D];

  const int blk = blockIdx.x;
  const int bh = blockIdx.y;
  const int nb = gridDim.x;
  const int row0 = blk * bs;
  const int halo_rows = kShard ? shard.halo_rows : 0;
  const int rows = min(bs, halo_rows + N - row0);
  const int cg = threadIdx.x % kTpr;
  const int rg = threadIdx.x / kTpr;
  // row r of the block: in the halo while row0 + r < halo_rows, in x afterwards
  const uint4* base = reinterpret_cast<const uint4*>(x + (static_cast<int64_t>(bh) * N + (row0 - halo_rows)) * D) + cg;
  const uint4* hbase = nullptr;
  if constexpr (kShard)
    hbase = reinterpret_cast<const uint4*>(static_cast<const T*>(shard.halo) +
                                           (static_cast<int64_t>(bh) * shard.halo_cap + row0) * D) + cg;

  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  // rows/kRpp is at most 8 (bs=128, D=128): issue the loads of up to eight rows before using any.
  for (int r0 = rg; r0 < rows; r0 += 8 * kRpp) {
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int r = r0 + u * kRpp;
      if (r >= rows) {
        v[u] = make_uint4(0, 0, 0, 0);
      } else if (kShard && row0 + r < halo_rows) {
        v[u] = __ldg(hbase + static_cast<int64_t>(r) * kTpr);
      } else {
        v[u] = __ldg(base + static_cast<int64_t>(r) * kTpr);
      }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      float f[8];
      unpack8<T>(v[u], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) red[rg][cg * 8 + i] = acc[i];
  __syncthreads();
  if (threadIdx.x < D) {
    float s = 0.f;
#pragma unroll 8
    for (int g = 0; g < kRpp; ++g) s += red[g][threadIdx.x];
    float* dst;
    if constexpr (kShard) {
      const int owner = bh / shard.heads_per_peer;
      dst = shard.peer[owner] + (static_cast<int64_t>(bh - owner * shard.heads_per_peer) * shard.nb_total +
                                 shard.block_base + blk) * D;
    } else {
      dst = out + (static_cast<int64_t>(bh) * nb + blk) * D;
    }
    dst[threadIdx.x] = s / static_cast<float>(rows);
  }
}

// Self-similarity of a block of rows: the mean cosine similarity over all pairs of its rows (a row paired with
// itself included), which equals |sum of the rows scaled to unit length|^2 / rows^2.  `center` (one vector of D
// floats per head, may be null) is subtracted from every row first.  One CTA per (block, head), rows laid over
// the threads as in pool_blocks_kernel; sums in a fixed order.  A block of nearly parallel rows gives ~1, rows
// pointing anywhere give ~1/rows.  Traffic: N*D*2 bytes read per head.
template <typename T, int D>
__global__ void __launch_bounds__(kPoolThreads) block_similarity_kernel(const T* __restrict__ x, int N, int bs,
                                                                        const float* __restrict__ center,
                                                                        float* __restrict__ out) {
  constexpr int kTpr = D / 8;
  constexpr int kRpp = kPoolThreads / kTpr;
  __shared__ float red[kRpp][D];
  __shared__ float part[D / 32];

  const int blk = blockIdx.x;
  const int bh = blockIdx.y;
  const int row0 = blk * bs;
  const int rows = min(bs, N - row0);
  const int cg = threadIdx.x % kTpr;
  const int rg = threadIdx.x / kTpr;
  const uint4* base = reinterpret_cast<const uint4*>(x + (static_cast<int64_t>(bh) * N + row0) * D) + cg;
  float c[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (center != nullptr) {
    const float4* cp = reinterpret_cast<const float4*>(center + static_cast<int64_t>(bh) * D + cg * 8);
    const float4 c0 = __ldg(cp), c1 = __ldg(cp + 1);
    c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w; c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
  }
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int b0 = 0; b0 < rows; b0 += 8 * kRpp) {       // uniform trip count: the shuffles need every lane
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int r = b0 + rg + u * kRpp;
      v[u] = r < rows ? __ldg(base + static_cast<int64_t>(r) * kTpr) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const bool valid = b0 + rg + u * kRpp < rows;
      float f[8];
      unpack8<T>(v[u], f);
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        f[i] -= c[i];
        ss = fmaf(f[i], f[i], ss);
      }
#pragma unroll
      for (int o = kTpr / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float inv = (valid && ss > 0.f) ? rsqrtf(ss) : 0.f;     // a zero row contributes nothing
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = fmaf(f[i], inv, acc[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) red[rg][cg * 8 + i] = acc[i];
  __syncthreads();
  if (threadIdx.x < D) {
    float s = 0.f;
#pragma unroll 8
    for (int g = 0; g < kRpp; ++g) s += red[g][threadIdx.x];
    s *= s;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (threadIdx.x % 32 == 0) part[threadIdx.x / 32] = s;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < D / 32; ++w) s += part[w];
    out[static_cast<int64_t>(bh) * gridDim.x + blk] = s / (static_cast<float>(rows) * static_cast<float>(rows));
  }
}

template <bool kShard>
void launch_pool(const void* x, int dtype, int D, int N, int bs, float* out, const PoolShard& shard, dim3 grid,
                 cudaStream_t st) {
  if (dtype == MODDIT_BF16) {
    if (D == 64)
      pool_blocks_kernel<__nv_bfloat16, 64, kShard><<<grid, kPoolThreads, 0, st>>>(
          static_cast<const __nv_bfloat16*>(x), N, bs, out, shard);
    else
      pool_blocks_kernel<__nv_bfloat16, 128, kShard><<<grid, kPoolThreads, 0, st>>>(
          static_cast<const __nv_bfloat16*>(x), N, bs, out, shard);
  } else {
    if (D == 64)
      pool_blocks_kernel<__half, 64, kShard><<<grid, kPoolThreads, 0, st>>>(static_cast<const __half*>(x), N, bs, out,
                                                                           shard);
    else
      pool_blocks_kernel<__half, 128, kShard><<<grid, kPoolThreads, 0, st>>>(static_cast<const __half*>(x), N, bs, out,
                                                                            shard);
  }
}

constexpr int kMapThreads = 256;
constexpr int kMapRows = 32;    // query blocks per CTA
constexpr int kMapCols = 128;   // key blocks per staged tile

// Logits on the tensor cores (warp-level mma.sync m16n8k16: the contraction is 5 GFLOP at the largest shape, far too
// small to pay for a tcgen05 pipeline).  The float32 block means are split into two bfloat16 terms, x = hi + lo,
// and a product is hi*hi + hi*lo + lo*hi with float32 accumulation: 16 mantissa bits per factor, a relative error
// of about 2^-16 per product, well inside the float16 grid of the map.  Both operands sit in shared memory as
// bfloat16 rows padded by 16 bytes (ldmatrix reads eight rows of 16 bytes at a time: odd multiples of 16 bytes
// between rows keep them on different banks).  Warp w owns key columns [16w, 16w+16) of every staged key tile for
// all 32 query rows of the CTA.
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// four floats -> their bfloat16 heads and the bfloat16 of what the heads leave over
__device__ __forceinline__ void split4(const float4& v, uint2& hi, uint2& lo) {
  const __nv_bfloat162 h0 = __floats2bfloat162_rn(v.x, v.y), h1 = __floats2bfloat162_rn(v.z, v.w);
  const float2 f0 = __bfloat1622float2(h0), f1 = __bfloat1622float2(h1);
  const __nv_bfloat162 l0 = __floats2bfloat162_rn(v.x - f0.x, v.y - f0.y);
  const __nv_bfloat162 l1 = __floats2bfloat162_rn(v.z - f1.x, v.w - f1.y);
  hi = make_uint2(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1));
  lo = make_uint2(*reinterpret_cast<const uint32_t*>(&l0), *reinterpret_cast<const uint32_t*>(&l1));
}

__global__ void __launch_bounds__(kMapThreads) pooled_map_kernel(const float* __restrict__ qbar,
                                                                 const float* __restrict__ kbar, int nb, int D,
                                                                 int q_off, int k_off, int n, float scale,
                                                                 __half* __restrict__ map) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int ld = D + 8;                          // bfloat16 elements per staged row (16 bytes of padding)
  __nv_bfloat16* qhi = reinterpret_cast<__nv_bfloat16*>(smem_raw);       // [kMapRows][ld]
  __nv_bfloat16* qlo = qhi + kMapRows * ld;
  __nv_bfloat16* khi = qlo + kMapRows * ld;                              // [kMapCols][ld]
  __nv_bfloat16* klo = khi + kMapCols * ld;
  float* lg = reinterpret_cast<float*>(klo + kMapCols * ld);             // [kMapRows][n]

  const int bh = blockIdx.y;
  const int i0 = blockIdx.x * kMapRows;
  const int tid = threadIdx.x;
  const int warp = tid / 32, lane = tid % 32;
  const float* qh = qbar + (static_cast<int64_t>(bh) * nb + q_off) * D;
  const float* kh = kbar + (static_cast<int64_t>(bh) * nb + k_off) * D;
  const int d4 = D / 4;

  for (int e = tid; e < kMapRows * d4; e += kMapThreads) {
    const int r = e / d4, c = e - r * d4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i0 + r < n) v = __ldg(reinterpret_cast<const float4*>(qh + static_cast<int64_t>(i0 + r) * D) + c);
    v.x *= scale; v.y *= scale; v.z *= scale; v.w *= scale;
    uint2 hi, lo;
    split4(v, hi, lo);
    *reinterpret_cast<uint2*>(qhi + r * ld + 4 * c) = hi;
    *reinterpret_cast<uint2*>(qlo + r * ld + 4 * c) = lo;
  }
  // ldmatrix addresses of this lane: A = 16 x 16 tile of the query rows (matrices: rows 0-7 / 8-15 x k 0-7 / 8-15),
  // B = two 8-column tiles of the key rows x 16 k (matrices: (tile 0, k 0-7), (tile 0, k 8-15), (tile 1, ...))
  const uint32_t a_off = static_cast<uint32_t>(((lane % 16) * ld + (lane / 16) * 8) * 2);
  const uint32_t b_off = static_cast<uint32_t>(((16 * warp + (lane / 16) * 8 + (lane % 8)) * ld + ((lane / 8) % 2) * 8) * 2);
  const uint32_t s_qhi = static_cast<uint32_t>(__cvta_generic_to_shared(qhi));
  const uint32_t s_qlo = static_cast<uint32_t>(__cvta_generic_to_shared(qlo));
  const uint32_t s_khi = static_cast<uint32_t>(__cvta_generic_to_shared(khi));
  const uint32_t s_klo = static_cast<uint32_t>(__cvta_generic_to_shared(klo));
  const int g = lane / 4, t2 = 2 * (lane % 4);
  for (int j0 = 0; j0 < n; j0 += kMapCols) {
    __syncthreads();
    // stage the key tile: eight independent 16-byte loads in flight per thread before any is used (one load at a
    // time, each waiting for the memory system, was most of this kernel's time)
    for (int e0 = tid; e0 < kMapCols * d4; e0 += 8 * kMapThreads) {
      float4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int e = e0 + u * kMapThreads;
        const int r = e / d4, c = e - r * d4;
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (e < kMapCols * d4 && j0 + r < n)
          v[u] = __ldg(reinterpret_cast<const float4*>(kh + static_cast<int64_t>(j0 + r) * D) + c);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int e = e0 + u * kMapThreads;
        if (e >= kMapCols * d4) break;
        const int r = e / d4, c = e - r * d4;
        uint2 hi, lo;
        split4(v[u], hi, lo);
        *reinterpret_cast<uint2*>(khi + r * ld + 4 * c) = hi;
        *reinterpret_cast<uint2*>(klo + r * ld + 4 * c) = lo;
      }
    }
    __syncthreads();
    float acc[2][2][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mt][nt][i] = 0.f;
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t bh_[4], bl_[4];
      ldmatrix_x4(bh_, s_khi + b_off + ks * 32);
      ldmatrix_x4(bl_, s_klo + b_off + ks * 32);
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        uint32_t ah[4], al[4];
        ldmatrix_x4(ah, s_qhi + a_off + (mt * 16 * ld + ks * 16) * 2);
        ldmatrix_x4(al, s_qlo + a_off + (mt * 16 * ld + ks * 16) * 2);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          mma_bf16(acc[mt][nt], al, bh_[2 * nt], bh_[2 * nt + 1]);      // small terms first
          mma_bf16(acc[mt][nt], ah, bl_[2 * nt], bl_[2 * nt + 1]);
          mma_bf16(acc[mt][nt], ah, bh_[2 * nt], bh_[2 * nt + 1]);
        }
      }
    }
    // accumulator element i of a 16 x 8 tile: row g + 8 * (i / 2), column t2 + (i % 2)
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int j = j0 + 16 * warp + 8 * nt + t2 + (i % 2);
          if (j < n) lg[(mt * 16 + g + 8 * (i / 2)) * n + j] = acc[mt][nt][i];
        }
  }
  __syncthreads();
  // per row: darkness = 1 - exp(logit - row maximum); warp w handles rows w, w+8, ...
  for (int r = warp; r < kMapRows; r += kMapThreads / 32) {
    const int i = i0 + r;
    if (i >= n) break;
    const float* row = lg + r * n;
    float m = -INFINITY;
    for (int j = lane; j < n; j += 32) m = fmaxf(m, row[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    __half* dst = map + (static_cast<int64_t>(bh) * n + i) * n;
    for (int j = lane; j < n; j += 32) dst[j] = __float2half_rn(1.f - expf(row[j] - m));
  }
}

// ---- the same map in three small launches, through a workspace ------------------------------------------------------
// The kernel above keeps a CTA's 32 x n logits in shared memory so that one launch can take the row maxima: one CTA
// per SM, every CTA walking all n key blocks tile by tile behind block-wide barriers - 45 us per CTA at n = 900,
// 4.7 waves of them at 24 heads, and the same 45 us when a rank holds three heads and the grid is less than a wave.
// With a workspace the logits are a plain batched matrix product with no dependence between tiles:
//   1. the scaled query means and the key means of the video region are split into bfloat16 head / remainder rows
//      once (every logit tile would otherwise redo the split of the rows it stages),
//   2. one CTA per 64 x 128 logit tile (two per SM) copies its rows with cp.async - all of a CTA's copies in
//      flight at once, no registers in between - and writes float32 logits,
//   3. a warp per row takes the maximum and writes the float16 map (the logits are still in the L2).
// Fragments, split and accumulation order are those of the kernel above, so the two routes give the same bits.
constexpr int kLgRows = 64;     // query blocks per CTA
constexpr int kLgCols = 128;    // key blocks per CTA

// (BH, nb, D) float32 -> rows [off, off + n) as (BH, n, 2, D) bfloat16: head row, then remainder row
__global__ void __launch_bounds__(256) split_means_kernel(const float* __restrict__ qbar, const float* __restrict__ kbar,
                                                          int nb, int D, int q_off, int k_off, int n, float scale,
                                                          int64_t total4, __nv_bfloat16* __restrict__ qs,
                                                          __nv_bfloat16* __restrict__ ks) {
  const int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= total4) return;
  const bool is_k = blockIdx.y != 0;
  const int d4 = D / 4;
  const int c = static_cast<int>(e % d4);
  const int64_t row = e / d4;                    // bh * n + r
  const int64_t bh = row / n;
  const int r = static_cast<int>(row - bh * n);
  const float* src = (is_k ? kbar : qbar) + ((bh * nb + (is_k ? k_off : q_off) + r) * D);
  float4 v = __ldg(reinterpret_cast<const float4*>(src) + c);
  if (!is_k) { v.x *= scale; v.y *= scale; v.z *= scale; v.w *= scale; }
  uint2 hi, lo;
  split4(v, hi, lo);
  __nv_bfloat16* dst = (is_k ? ks : qs) + row * 2 * D;
  *reinterpret_cast<uint2*>(dst + 4 * c) = hi;
  *reinterpret_cast<uint2*>(dst + D + 4 * c) = lo;
}

__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(src) : "memory");
}

// rows [row0, row0 + kRows) of a split matrix (rows past n - 1 repeat row n - 1: their logits are never stored)
template <int kRows>
__device__ __forceinline__ void stage_split_rows(const __nv_bfloat16* __restrict__ src, int row0, int n, int D,
                                                 uint32_t s_hi, uint32_t s_lo, int ld, int tid) {
  const int cpr = D / 8;                          // 16-byte chunks per row half
  for (int e = tid; e < kRows * 2 * cpr; e += kMapThreads) {
    const int r = e / (2 * cpr), w = e - r * 2 * cpr;
    const int part = w / cpr, c = w - part * cpr;
    const __nv_bfloat16* g = src + (static_cast<int64_t>(min(row0 + r, n - 1)) * 2 + part) * D + 8 * c;
    cp_async16((part ? s_lo : s_hi) + static_cast<uint32_t>((r * ld + 8 * c) * 2), g);
  }
}

__global__ void __launch_bounds__(kMapThreads, 2) pooled_logits_kernel(const __nv_bfloat16* __restrict__ qs,
                                                                       const __nv_bfloat16* __restrict__ ks, int D,
                                                                       int n, float* __restrict__ lg) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int ld = D + 8;
  __nv_bfloat16* qhi = reinterpret_cast<__nv_bfloat16*>(smem_raw);       // [kLgRows][ld]
  __nv_bfloat16* qlo = qhi + kLgRows * ld;
  __nv_bfloat16* khi = qlo + kLgRows * ld;                               // [kLgCols][ld]
  __nv_bfloat16* klo = khi + kLgCols * ld;
  const int bh = blockIdx.z;
  const int i0 = blockIdx.y * kLgRows;
  const int j0 = blockIdx.x * kLgCols;
  const int tid = threadIdx.x;
  const int warp = tid / 32, lane = tid % 32;
  const uint32_t s_qhi = static_cast<uint32_t>(__cvta_generic_to_shared(qhi));
  const uint32_t s_qlo = static_cast<uint32_t>(__cvta_generic_to_shared(qlo));
  const uint32_t s_khi = static_cast<uint32_t>(__cvta_generic_to_shared(khi));
  const uint32_t s_klo = static_cast<uint32_t>(__cvta_generic_to_shared(klo));
  stage_split_rows<kLgRows>(qs + static_cast<int64_t>(bh) * n * 2 * D, i0, n, D, s_qhi, s_qlo, ld, tid);
  stage_split_rows<kLgCols>(ks + static_cast<int64_t>(bh) * n * 2 * D, j0, n, D, s_khi, s_klo, ld, tid);
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();
  const uint32_t a_off = static_cast<uint32_t>(((lane % 16) * ld + (lane / 16) * 8) * 2);
  const uint32_t b_off = static_cast<uint32_t>(((16 * warp + (lane / 16) * 8 + (lane % 8)) * ld + ((lane / 8) % 2) * 8) * 2);
  const int g = lane / 4, t2 = 2 * (lane % 4);
  constexpr int kMT = kLgRows / 16;
  float acc[kMT][2][4];
#pragma unroll
  for (int mt = 0; mt < kMT; ++mt)
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[mt][nt][i] = 0.f;
  for (int ks_ = 0; ks_ < D / 16; ++ks_) {
    uint32_t bh_[4], bl_[4];
    ldmatrix_x4(bh_, s_khi + b_off + ks_ * 32);
    ldmatrix_x4(bl_, s_klo + b_off + ks_ * 32);
#pragma unroll
    for (int mt = 0; mt < kMT; ++mt) {
      uint32_t ah[4], al[4];
      ldmatrix_x4(ah, s_qhi + a_off + (mt * 16 * ld + ks_ * 16) * 2);
      ldmatrix_x4(al, s_qlo + a_off + (mt * 16 * ld + ks_ * 16) * 2);
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        mma_bf16(acc[mt][nt], al, bh_[2 * nt], bh_[2 * nt + 1]);      // small terms first
        mma_bf16(acc[mt][nt], ah, bl_[2 * nt], bl_[2 * nt + 1]);
        mma_bf16(acc[mt][nt], ah, bh_[2 * nt], bh_[2 * nt + 1]);
      }
    }
  }
  float* dst = lg + static_cast<int64_t>(bh) * n * n;
#pragma unroll
  for (int mt = 0; mt < kMT; ++mt)
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = i0 + mt * 16 + g + 8 * (i / 2);
        const int j = j0 + 16 * warp + 8 * nt + t2 + (i % 2);
        if (r < n && j < n) dst[static_cast<int64_t>(r) * n + j] = acc[mt][nt][i];
      }
}

// darkness = 1 - exp(logit - row maximum), a warp per row of the workspace
__global__ void __launch_bounds__(kMapThreads) pooled_darkness_kernel(const float* __restrict__ lg, int64_t rows, int n,
                                                                      __half* __restrict__ map) {
  const int lane = threadIdx.x % 32;
  const int64_t r = static_cast<int64_t>(blockIdx.x) * (kMapThreads / 32) + threadIdx.x / 32;
  if (r >= rows) return;
  const float* row = lg + r * n;
  float m = -INFINITY;
  for (int j = lane; j < n; j += 32) m = fmaxf(m, row[j]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  __half* dst = map + r * n;
  for (int j = lane; j < n; j += 32) dst[j] = __float2half_rn(1.f - expf(row[j] - m));
}

size_t pooled_logits_smem(int D) {
  return sizeof(__nv_bfloat16) * static_cast<size_t>(2 * (kLgRows + kLgCols)) * (D + 8);
}
// workspace: float32 logits | split query means | split key means (each part a multiple of 16 bytes)
size_t pooled_ws_logits_bytes(int BH, int n) {
  return (sizeof(float) * static_cast<size_t>(BH) * n * n + 15) / 16 * 16;
}
size_t pooled_ws_split_bytes(int BH, int n, int D) {
  return sizeof(__nv_bfloat16) * static_cast<size_t>(BH) * n * 2 * D;
}

size_t pooled_map_smem(int D, int n) {
  return sizeof(__nv_bfloat16) * (static_cast<size_t>(2 * (kMapRows + kMapCols)) * (D + 8)) +
         sizeof(float) * static_cast<size_t>(kMapRows) * n;
}

}  // namespace
}  // namespace moddit

using namespace moddit;

extern "C" int moddit_pool_blocks(const void* x, int dtype, int BH, int N, int D, int block_size, float* out,
                                  void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(x && out, "pool_blocks: null pointer");
  MODDIT_CHECK_ARG(BH > 0 && N > 0, "pool_blocks: BH=%d N=%d must be positive", BH, N);
  if (D != 64 && D != 128) return fail(MODDIT_E_UNSUPPORTED, "pool_blocks: head_dim must be 64 or 128, got %d", D);
  if (block_size != 64 && block_size != 128)
    return fail(MODDIT_E_UNSUPPORTED, "pool_blocks: block_size must be 64 or 128, got %d", block_size);
  if (dtype != MODDIT_BF16 && dtype != MODDIT_FP16) return fail(MODDIT_E_ARG, "pool_blocks: unknown dtype %d", dtype);
  if (!aligned16(x)) return fail(MODDIT_E_ALIGN, "pool_blocks: input must be 16-byte aligned");
  if (BH > 65535) return fail(MODDIT_E_UNSUPPORTED, "pool_blocks: BH=%d exceeds 65535", BH);
  if (int rc = require_sm100()) return rc;
  const dim3 grid(ceil_div(N, block_size), BH);
  const PoolShard none = {};
  launch_pool<false>(x, dtype, D, N, block_size, out, none, grid, as_stream(stream));
  MODDIT_CHECK_LAUNCH("pool_blocks_kernel");
  return MODDIT_OK;
}

extern "C" int moddit_block_similarity(const void* x, int dtype, int BH, int N, int D, int block_size,
                                       const float* center, float* out, void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(x && out, "block_similarity: null pointer");
  MODDIT_CHECK_ARG(BH > 0 && N > 0, "block_similarity: BH=%d N=%d must be positive", BH, N);
  if (D != 64 && D != 128) return fail(MODDIT_E_UNSUPPORTED, "block_similarity: head_dim must be 64 or 128, got %d", D);
  if (block_size != 64 && block_size != 128)
    return fail(MODDIT_E_UNSUPPORTED, "block_similarity: block_size must be 64 or 128, got %d", block_size);
  if (dtype != MODDIT_BF16 && dtype != MODDIT_FP16) return fail(MODDIT_E_ARG, "block_similarity: unknown dtype %d", dtype);
  if (!aligned16(x) || !aligned16(center))
    return fail(MODDIT_E_ALIGN, "block_similarity: input and center must be 16-byte aligned");
  if (BH > 65535) return fail(MODDIT_E_UNSUPPORTED, "block_similarity: BH=%d exceeds 65535", BH);
  if (int rc = require_sm100()) return rc;
  const dim3 grid(ceil_div(N, block_size), BH);
  cudaStream_t st = as_stream(stream);
  if (dtype == MODDIT_BF16) {
    if (D == 64)
      block_similarity_kernel<__nv_bfloat16, 64><<<grid, kPoolThreads, 0, st>>>(static_cast<const __nv_bfloat16*>(x), N,
                                                                              block_size, center, out);
    else
      block_similarity_kernel<__nv_bfloat16, 128><<<grid, kPoolThreads, 0, st>>>(static_cast<const __nv_bfloat16*>(x), N,
                                                                               block_size, center, out);
  } else {
    if (D == 64)
      block_similarity_kernel<__half, 64><<<grid, kPoolThreads, 0, st>>>(static_cast<const __half*>(x), N, block_size,
                                                                       center, out);
    else
      block_similarity_kernel<__half, 128><<<grid, kPoolThreads, 0, st>>>(static_cast<const __half*>(x), N, block_size,
                                                                        center, out);
  }
  MODDIT_CHECK_LAUNCH("block_similarity_kernel");
  return MODDIT_OK;
}

extern "C" int moddit_pool_blocks_shard(const void* x, const void* halo, int dtype, int heads, int rows_local,
                                        int halo_rows, int halo_capacity, int D, int block_size, int n_blocks,
                                        float* const* peer_out, int n_peers, int heads_per_peer, int total_blocks,
                                        int block_base, void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(x && peer_out, "pool_blocks_shard: null pointer");
  MODDIT_CHECK_ARG(heads > 0 && heads <= 65535 && rows_local > 0 && n_blocks > 0,
                   "pool_blocks_shard: heads=%d rows=%d blocks=%d out of range", heads, rows_local, n_blocks);
  if (D != 64 && D != 128) return fail(MODDIT_E_UNSUPPORTED, "pool_blocks_shard: head_dim must be 64 or 128, got %d", D);
  if (block_size != 64 && block_size != 128)
    return fail(MODDIT_E_UNSUPPORTED, "pool_blocks_shard: block_size must be 64 or 128, got %d", block_size);
  if (dtype != MODDIT_BF16 && dtype != MODDIT_FP16)
    return fail(MODDIT_E_ARG, "pool_blocks_shard: unknown dtype %d", dtype);
  MODDIT_CHECK_ARG(n_peers >= 1 && n_peers <= kMaxPoolPeers && heads_per_peer > 0 && heads == n_peers * heads_per_peer,
                   "pool_blocks_shard: %d heads do not split into %d peers x %d heads", heads, n_peers, heads_per_peer);
  MODDIT_CHECK_ARG(halo_rows >= 0 && halo_rows < block_size && halo_rows <= halo_capacity,
                   "pool_blocks_shard: halo_rows=%d outside [0, min(block_size, capacity=%d))", halo_rows, halo_capacity);
  MODDIT_CHECK_ARG(halo_rows == 0 || halo, "pool_blocks_shard: halo rows without a halo buffer");
  MODDIT_CHECK_ARG(static_cast<long long>(n_blocks - 1) * block_size < static_cast<long long>(halo_rows) + rows_local,
                   "pool_blocks_shard: %d blocks exceed the %d + %d rows at hand", n_blocks, halo_rows, rows_local);
  MODDIT_CHECK_ARG(block_base >= 0 && block_base + n_blocks <= total_blocks,
                   "pool_blocks_shard: blocks [%d, %d) outside [0, %d)", block_base, block_base + n_blocks, total_blocks);
  if (!aligned16(x) || (halo && !aligned16(halo)))
    return fail(MODDIT_E_ALIGN, "pool_blocks_shard: inputs must be 16-byte aligned");
  if (int rc = require_sm100()) return rc;
  PoolShard shard = {};
  shard.halo = halo;
  shard.halo_rows = halo_rows;
  shard.halo_cap = halo_capacity;
  for (int i = 0; i < n_peers; ++i) {
    MODDIT_CHECK_ARG(peer_out[i] && aligned16(peer_out[i]), "pool_blocks_shard: peer buffer %d null or unaligned", i);
    shard.peer[i] = peer_out[i];
  }
  shard.heads_per_peer = heads_per_peer;
  shard.nb_total = total_blocks;
  shard.block_base = block_base;
  launch_pool<true>(x, dtype, D, rows_local, block_size, nullptr, shard, dim3(n_blocks, heads), as_stream(stream));
  MODDIT_CHECK_LAUNCH("pool_blocks_kernel (shard)");
  return MODDIT_OK;
}

extern "C" int moddit_pooled_map(const float* qbar, const float* kbar, int BH, int nb, int D, int q_block_offset,
                                 int k_block_offset, int n, float scale, void* map_f16, void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(qbar && kbar && map_f16, "pooled_map: null pointer");
  MODDIT_CHECK_ARG(BH > 0 && nb > 0 && n > 0 && D > 0, "pooled_map: sizes must be positive");
  MODDIT_CHECK_ARG(q_block_offset >= 0 && k_block_offset >= 0 && q_block_offset + n <= nb && k_block_offset + n <= nb,
                   "pooled_map: video region [%d+%d) / [%d+%d) exceeds %d blocks", q_block_offset, n, k_block_offset,
                   n, nb);
  if (BH > 65535) return fail(MODDIT_E_UNSUPPORTED, "pooled_map: BH=%d exceeds 65535", BH);
  if (int rc = require_sm100()) return rc;
  cudaStream_t st = as_stream(stream);
  __half* map = static_cast<__half*>(map_f16);
  const size_t sm = pooled_map_smem(D, n);
  if ((D & 15) != 0 || !aligned16(qbar) || !aligned16(kbar))
    return fail(MODDIT_E_ALIGN, "pooled_map: head_dim must be a multiple of 16 and the inputs 16-byte aligned");
  if (sm > 227 * 1024)
    return fail(MODDIT_E_UNSUPPORTED, "pooled_map: n=%d video blocks do not fit the shared-memory row buffer", n);
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(pooled_map_kernel), sm)) return rc;
  pooled_map_kernel<<<dim3(ceil_div(n, kMapRows), BH), kMapThreads, sm, st>>>(qbar, kbar, nb, D, q_block_offset,
                                                                               k_block_offset, n, scale, map);
  MODDIT_CHECK_LAUNCH("pooled_map_kernel");
  return MODDIT_OK;
}

extern "C" size_t moddit_pooled_map_workspace_bytes(int BH, int n, int D) {
  if (BH <= 0 || n <= 0 || D <= 0) return 0;
  return pooled_ws_logits_bytes(BH, n) + 2 * pooled_ws_split_bytes(BH, n, D);
}

extern "C" int moddit_pooled_map_ws(const float* qbar, const float* kbar, int BH, int nb, int D, int q_block_offset,
                                    int k_block_offset, int n, float scale, void* map_f16, void* workspace,
                                    size_t workspace_bytes, void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(qbar && kbar && map_f16 && workspace, "pooled_map_ws: null pointer");
  MODDIT_CHECK_ARG(BH > 0 && nb > 0 && n > 0 && D > 0, "pooled_map_ws: sizes must be positive");
  MODDIT_CHECK_ARG(q_block_offset >= 0 && k_block_offset >= 0 && q_block_offset + n <= nb && k_block_offset + n <= nb,
                   "pooled_map_ws: video region [%d+%d) / [%d+%d) exceeds %d blocks", q_block_offset, n,
                   k_block_offset, n, nb);
  MODDIT_CHECK_ARG(workspace_bytes >= moddit_pooled_map_workspace_bytes(BH, n, D),
                   "pooled_map_ws: workspace of %zu bytes, %zu needed", workspace_bytes,
                   moddit_pooled_map_workspace_bytes(BH, n, D));
  if (BH > 65535) return fail(MODDIT_E_UNSUPPORTED, "pooled_map_ws: BH=%d exceeds 65535", BH);
  if ((D & 15) != 0 || D > 256 || !aligned16(qbar) || !aligned16(kbar) || !aligned16(workspace))
    return fail(MODDIT_E_ALIGN,
                "pooled_map_ws: head_dim must be a multiple of 16 (at most 256), inputs and workspace 16-byte aligned");
  if (int rc = require_sm100()) return rc;
  cudaStream_t st = as_stream(stream);
  const size_t sm = pooled_logits_smem(D);
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(pooled_logits_kernel), sm)) return rc;
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  float* lg = reinterpret_cast<float*>(ws);
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(ws + pooled_ws_logits_bytes(BH, n));
  __nv_bfloat16* ks = reinterpret_cast<__nv_bfloat16*>(ws + pooled_ws_logits_bytes(BH, n) + pooled_ws_split_bytes(BH, n, D));
  const int64_t total4 = static_cast<int64_t>(BH) * n * (D / 4);
  split_means_kernel<<<dim3(static_cast<unsigned>((total4 + 255) / 256), 2), 256, 0, st>>>(
      qbar, kbar, nb, D, q_block_offset, k_block_offset, n, scale, total4, qs, ks);
  MODDIT_CHECK_LAUNCH("split_means_kernel");
  pooled_logits_kernel<<<dim3(ceil_div(n, kLgCols), ceil_div(n, kLgRows), BH), kMapThreads, sm, st>>>(qs, ks, D, n, lg);
  MODDIT_CHECK_LAUNCH("pooled_logits_kernel");
  const int64_t rows = static_cast<int64_t>(BH) * n;
  pooled_darkness_kernel<<<static_cast<unsigned>((rows + kMapThreads / 32 - 1) / (kMapThreads / 32)), kMapThreads, 0, st>>>(
      lg, rows, n, static_cast<__half*>(map_f16));
  MODDIT_CHECK_LAUNCH("pooled_darkness_kernel");
  return MODDIT_OK;
}

// ---- strided row copy (used to place sequence/head shards directly into a peer GPU's buffer) ---------
namespace moddit {
namespace {

// rows x width_bytes, 16 bytes per thread per step; plain loads from `src`, plain stores to `dst`
// (which may be peer memory mapped into this process: ordinary P2P stores, no TMA, no multicast).
__global__ void __launch_bounds__(256) copy_rows_kernel(const unsigned char* __restrict__ src,
                                                        unsigned char* __restrict__ dst, int64_t src_pitch,
                                                        int64_t dst_pitch, int64_t width16) {
  const uint4* s = reinterpret_cast<const uint4*>(src + static_cast<int64_t>(blockIdx.y) * src_pitch);
  uint4* d = reinterpret_cast<uint4*>(dst + static_cast<int64_t>(blockIdx.y) * dst_pitch);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < width16; i += 4 * stride) {
    const uint4 a = __ldg(s + i), b = __ldg(s + i + stride), c = __ldg(s + i + 2 * stride), e = __ldg(s + i + 3 * stride);
    d[i] = a;
    d[i + stride] = b;
    d[i + 2 * stride] = c;
    d[i + 3 * stride] = e;
  }
  for (; i < width16; i += stride) d[i] = __ldg(s + i);
}

constexpr int kMaxCopyJobs = 24;
struct CopyJobs {
  const unsigned char* src[kMaxCopyJobs];
  unsigned char* dst[kMaxCopyJobs];
};

// Same copy for up to 24 (source, destination) pairs in one launch: blockIdx.z selects the pair.
__global__ void __launch_bounds__(256) copy_rows_multi_kernel(const __grid_constant__ CopyJobs jobs, int64_t src_pitch,
                                                              int64_t dst_pitch, int64_t width16) {
  const uint4* s = reinterpret_cast<const uint4*>(jobs.src[blockIdx.z] + static_cast<int64_t>(blockIdx.y) * src_pitch);
  uint4* d = reinterpret_cast<uint4*>(jobs.dst[blockIdx.z] + static_cast<int64_t>(blockIdx.y) * dst_pitch);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < width16; i += 4 * stride) {
    const uint4 a = __ldg(s + i), b = __ldg(s + i + stride), c = __ldg(s + i + 2 * stride), e = __ldg(s + i + 3 * stride);
    d[i] = a;
    d[i + stride] = b;
    d[i + 2 * stride] = c;
    d[i + 3 * stride] = e;
  }
  for (; i < width16; i += stride) d[i] = __ldg(s + i);
}

// The same jobs on a fixed, small number of CTAs: segments of 64 KB are dealt round-robin to the CTAs, eight
// 16-byte loads in flight per thread.  Meant for an exchange that runs beside other kernels: a grid that fills
// the GPU would make them queue behind the copy, this one leaves them most of the SMs.
constexpr int kCopySegment16 = 4096;     // 16-byte words per segment
__global__ void __launch_bounds__(256) copy_rows_narrow_kernel(const __grid_constant__ CopyJobs jobs, int n_jobs,
                                                               int rows, int64_t src_pitch, int64_t dst_pitch,
                                                               int64_t width16) {
  const int64_t segs_per_row = (width16 + kCopySegment16 - 1) / kCopySegment16;
  const int64_t total = static_cast<int64_t>(n_jobs) * rows * segs_per_row;
  for (int64_t t = blockIdx.x; t < total; t += gridDim.x) {
    const int64_t jr = t / segs_per_row, sg = t - jr * segs_per_row;
    const int job = static_cast<int>(jr / rows), row = static_cast<int>(jr - static_cast<int64_t>(job) * rows);
    const uint4* s = reinterpret_cast<const uint4*>(jobs.src[job] + row * src_pitch) + sg * kCopySegment16;
    uint4* d = reinterpret_cast<uint4*>(jobs.dst[job] + row * dst_pitch) + sg * kCopySegment16;
    const int n16 = static_cast<int>(min(static_cast<int64_t>(kCopySegment16), width16 - sg * kCopySegment16));
    int i = threadIdx.x;
    for (; i + 7 * 256 < n16; i += 8 * 256) {
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = __ldg(s + i + u * 256);
#pragma unroll
      for (int u = 0; u < 8; ++u) d[i + u * 256] = v[u];
    }
    for (; i < n16; i += 256) d[i] = __ldg(s + i);
  }
}

}  // namespace
}  // namespace moddit

extern "C" int moddit_copy_rows_narrow(const void* const* src, void* const* dst, int n_jobs, int64_t src_pitch,
                                       int64_t dst_pitch, int64_t width_bytes, int rows, int max_ctas, void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(src && dst, "copy_rows_narrow: null pointer table");
  MODDIT_CHECK_ARG(n_jobs >= 1 && n_jobs <= kMaxCopyJobs, "copy_rows_narrow: n_jobs=%d outside [1, %d]", n_jobs, kMaxCopyJobs);
  MODDIT_CHECK_ARG(rows > 0 && rows <= 65535 && width_bytes > 0, "copy_rows_narrow: rows=%d width=%lld out of range", rows,
                   static_cast<long long>(width_bytes));
  MODDIT_CHECK_ARG(max_ctas >= 1 && max_ctas <= 4096, "copy_rows_narrow: max_ctas=%d outside [1, 4096]", max_ctas);
  if ((src_pitch & 15) || (dst_pitch & 15) || (width_bytes & 15))
    return fail(MODDIT_E_ALIGN, "copy_rows_narrow: pitches and width must be multiples of 16 bytes");
  CopyJobs jobs = {};
  for (int i = 0; i < n_jobs; ++i) {
    if (!src[i] || !dst[i] || !aligned16(src[i]) || !aligned16(dst[i]))
      return fail(MODDIT_E_ALIGN, "copy_rows_narrow: job %d has a null or unaligned pointer", i);
    jobs.src[i] = static_cast<const unsigned char*>(src[i]);
    jobs.dst[i] = static_cast<unsigned char*>(dst[i]);
  }
  const int64_t width16 = width_bytes / 16;
  const int64_t total = static_cast<int64_t>(n_jobs) * rows * ((width16 + kCopySegment16 - 1) / kCopySegment16);
  const unsigned grid = static_cast<unsigned>(total < max_ctas ? total : max_ctas);
  copy_rows_narrow_kernel<<<grid, 256, 0, as_stream(stream)>>>(jobs, n_jobs, rows, src_pitch, dst_pitch, width16);
  MODDIT_CHECK_LAUNCH("copy_rows_narrow_kernel");
  return MODDIT_OK;
}

extern "C" int moddit_copy_rows_multi(const void* const* src, void* const* dst, int n_jobs, int64_t src_pitch,
                                      int64_t dst_pitch, int64_t width_bytes, int rows, void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(src && dst, "copy_rows_multi: null pointer table");
  MODDIT_CHECK_ARG(n_jobs >= 1 && n_jobs <= kMaxCopyJobs, "copy_rows_multi: n_jobs=%d outside [1, %d]", n_jobs, kMaxCopyJobs);
  MODDIT_CHECK_ARG(rows > 0 && rows <= 65535 && width_bytes > 0, "copy_rows_multi: rows=%d width=%lld out of range", rows,
                   static_cast<long long>(width_bytes));
  if ((src_pitch & 15) || (dst_pitch & 15) || (width_bytes & 15))
    return fail(MODDIT_E_ALIGN, "copy_rows_multi: pitches and width must be multiples of 16 bytes");
  CopyJobs jobs = {};
  for (int i = 0; i < n_jobs; ++i) {
    if (!src[i] || !dst[i] || !aligned16(src[i]) || !aligned16(dst[i]))
      return fail(MODDIT_E_ALIGN, "copy_rows_multi: job %d has a null or unaligned pointer", i);
    jobs.src[i] = static_cast<const unsigned char*>(src[i]);
    jobs.dst[i] = static_cast<unsigned char*>(dst[i]);
  }
  const int64_t width16 = width_bytes / 16;
  int64_t bx = (width16 + 256 * 4 - 1) / (256 * 4);
  const int64_t cap = (148 * 8 + static_cast<int64_t>(rows) * n_jobs - 1) / (static_cast<int64_t>(rows) * n_jobs);
  if (bx > cap) bx = cap;
  if (bx < 1) bx = 1;
  copy_rows_multi_kernel<<<dim3(static_cast<unsigned>(bx), rows, n_jobs), 256, 0, as_stream(stream)>>>(
      jobs, src_pitch, dst_pitch, width16);
  MODDIT_CHECK_LAUNCH("copy_rows_multi_kernel");
  return MODDIT_OK;
}

// The same strided copy on the copy engines (no SM is used): one 2-D asynchronous copy.  On an NVLink node a
// peer destination gets the full link bandwidth and the SMs stay free for the kernels of the step.
extern "C" int moddit_copy_rows_dma(const void* src, void* dst, int64_t src_pitch, int64_t dst_pitch,
                                    int64_t width_bytes, int rows, void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(src && dst, "copy_rows_dma: null pointer");
  MODDIT_CHECK_ARG(rows > 0 && width_bytes > 0 && src_pitch >= width_bytes && dst_pitch >= width_bytes,
                   "copy_rows_dma: rows=%d width=%lld pitches %lld/%lld out of range", rows,
                   static_cast<long long>(width_bytes), static_cast<long long>(src_pitch),
                   static_cast<long long>(dst_pitch));
  MODDIT_CHECK_CUDA(cudaMemcpy2DAsync(dst, static_cast<size_t>(dst_pitch), src, static_cast<size_t>(src_pitch),
                                      static_cast<size_t>(width_bytes), static_cast<size_t>(rows), cudaMemcpyDefault,
                                      as_stream(stream)));
  return MODDIT_OK;
}

extern "C" int moddit_copy_rows(const void* src, void* dst, int64_t src_pitch, int64_t dst_pitch, int64_t width_bytes,
                                int rows, void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(src && dst, "copy_rows: null pointer");
  MODDIT_CHECK_ARG(rows > 0 && rows <= 65535 && width_bytes > 0, "copy_rows: rows=%d width=%lld out of range", rows,
                   static_cast<long long>(width_bytes));
  if (!aligned16(src) || !aligned16(dst) || (src_pitch & 15) || (dst_pitch & 15) || (width_bytes & 15))
    return fail(MODDIT_E_ALIGN, "copy_rows: pointers, pitches and width must be multiples of 16 bytes");
  const int64_t width16 = width_bytes / 16;
  int64_t bx = (width16 + 256 * 4 - 1) / (256 * 4);
  const int64_t cap = (148 * 8 + rows - 1) / rows;      // about eight CTAs per SM in total
  if (bx > cap) bx = cap;
  if (bx < 1) bx = 1;
  copy_rows_kernel<<<dim3(static_cast<unsigned>(bx), rows), 256, 0, as_stream(stream)>>>(
      static_cast<const unsigned char*>(src), static_cast<unsigned char*>(dst), src_pitch, dst_pitch, width16);
  MODDIT_CHECK_LAUNCH("copy_rows_kernel");
  return MODDIT_OK;
}
