// Second, independently written path for the exact sparsity-map replay: warp-level tensor-core products
// (mma.sync m16n8k16) with register fragments, no TMA, no tensor memory, no mbarriers.
//
// It exists so that the cross-check the reference's own test makes between its two kernels
// (tests/test_flash_sparsity.py:61-104, CUDA replay against the Triton replay) still compares two code paths here:
// `moddit_replay_map` (tcgen05, N = 256 instructions, accumulators in tensor memory) and this one share nothing
// but the definition  count(S[r,c] < lse[r] + log_thr) / bs^2,  S = round_dtype(q * scale) k^T in float32.
// The two differ only in the order of the float32 additions inside a dot product, i.e. in a handful of
// comparisons that sit within rounding of the threshold.
//
// One CTA (8 warps) owns 128 video query rows; warp w keeps rows [16w, 16w+16) as A fragments (scaled and rounded
// once) and walks the key blocks 64 keys at a time: the key tile is staged in shared memory (rows padded by 16 bytes
// for ldmatrix), each warp forms its 16 x 64 scores and counts the ones below its rows' lines.  Counts per
// (64-row half, 64-key block) are added up in shared memory and written once at the end.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace moddit {
namespace {

constexpr int kRmThreads = 256;
constexpr int kRmRows = 128;      // query rows per CTA
constexpr int kRmKeys = 64;       // keys per staged tile

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

template <bool kBF16>
__device__ __forceinline__ void mma16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (kBF16) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

// two neighbouring 16-bit elements, each multiplied by `scale` in float32 and rounded back to the 16-bit type
template <bool kBF16>
__device__ __forceinline__ uint32_t scale_round2(uint32_t two, float scale) {
  if constexpr (kBF16) {
    const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&two);
    const __nv_bfloat162 o = __halves2bfloat162(__float2bfloat16_rn(__bfloat162float(h.x) * scale),
                                                __float2bfloat16_rn(__bfloat162float(h.y) * scale));
    return *reinterpret_cast<const uint32_t*>(&o);
  } else {
    const __half2 h = *reinterpret_cast<const __half2*>(&two);
    const __half2 o = __halves2half2(__float2half_rn(__half2float(h.x) * scale), __float2half_rn(__half2float(h.y) * scale));
    return *reinterpret_cast<const uint32_t*>(&o);
  }
}

template <int D, bool kBF16>
__global__ void __launch_bounds__(kRmThreads) replay_map_mma_kernel(
    const uint16_t* __restrict__ q, const uint16_t* __restrict__ k, const float* __restrict__ lse, int N, int bs,
    float scale, float log_thr, int q_off, int k_off, int n, __half* __restrict__ map) {
  constexpr int kLd = D + 8;                     // 16-bit elements per staged key row
  constexpr int kSteps = D / 16;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint16_t* ks = reinterpret_cast<uint16_t*>(smem_raw);                       // [kRmKeys][kLd]
  int* cnt = reinterpret_cast<int*>(ks + kRmKeys * kLd);                      // [2 row halves][key blocks of 64]

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int g = lane / 4, t2 = 2 * (lane % 4);
  const int bh = blockIdx.y;
  const int vtok = n * bs;
  const int row0 = blockIdx.x * kRmRows;         // first video row of the CTA
  const int nkb = (vtok + kRmKeys - 1) / kRmKeys;
  for (int i = threadIdx.x; i < 2 * nkb; i += kRmThreads) cnt[i] = 0;

  // A fragments of this warp's 16 rows: element pairs (row g / g + 8, columns 16 ks + t2 (+ 8))
  uint32_t a[kSteps][4];
  float line[2];
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int vr = row0 + 16 * warp + g + 8 * half;          // row inside the video region
    const bool ok = vr < vtok && q_off + vr < N;
    line[half] = ok ? lse[static_cast<int64_t>(bh) * N + q_off + vr] + log_thr : -INFINITY;
    const uint16_t* src = q + (static_cast<int64_t>(bh) * N + q_off + (ok ? vr : 0)) * D;
#pragma unroll
    for (int s = 0; s < kSteps; ++s) {
      const uint32_t lo = ok ? *reinterpret_cast<const uint32_t*>(src + 16 * s + t2) : 0u;
      const uint32_t hi = ok ? *reinterpret_cast<const uint32_t*>(src + 16 * s + t2 + 8) : 0u;
      a[s][half] = scale_round2<kBF16>(lo, scale);
      a[s][2 + half] = scale_round2<kBF16>(hi, scale);
    }
  }
  const uint32_t s_ks = static_cast<uint32_t>(__cvta_generic_to_shared(ks));
  // ldmatrix addresses: two 8-key tiles x 16 elements of the head dimension per instruction
  const uint32_t b_off = static_cast<uint32_t>((((lane / 16) * 8 + (lane % 8)) * kLd + ((lane / 8) % 2) * 8) * 2);
  const int rh = (16 * warp) / 64;               // 64-row half of the CTA's rows this warp belongs to

  for (int kb = 0; kb < nkb; ++kb) {
    __syncthreads();
    // stage 64 keys x D: 16-byte pieces, rows beyond the video region are zero
    for (int e = threadIdx.x; e < kRmKeys * (D / 8); e += kRmThreads) {
      const int r = e / (D / 8), c = e - r * (D / 8);
      const int vk = kb * kRmKeys + r;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (vk < vtok && k_off + vk < N)
        v = __ldg(reinterpret_cast<const uint4*>(k + (static_cast<int64_t>(bh) * N + k_off + vk) * D) + c);
      *reinterpret_cast<uint4*>(ks + r * kLd + 8 * c) = v;
    }
    __syncthreads();
    const int valid = min(kRmKeys, vtok - kb * kRmKeys);     // keys of this tile inside the video region
    int below = 0;
#pragma unroll
    for (int np = 0; np < kRmKeys / 16; ++np) {              // pairs of 8-key tiles
      float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int s = 0; s < kSteps; ++s) {
        uint32_t b[4];
        ldmatrix_x4(b, s_ks + b_off + static_cast<uint32_t>((np * 16 * kLd + s * 16) * 2));
        mma16<kBF16>(acc[0], a[s], b[0], b[1]);
        mma16<kBF16>(acc[1], a[s], b[2], b[3]);
      }
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int col = np * 16 + nt * 8 + t2 + (i % 2);
          below += (col < valid && acc[nt][i] < line[i / 2]) ? 1 : 0;
        }
    }
    below = __reduce_add_sync(0xffffffffu, below);
    if (lane == 0 && below) atomicAdd(&cnt[rh * nkb + kb], below);
  }
  __syncthreads();
  // block (bi, bj) of the map: bs = 64 -> one counter; bs = 128 -> both row halves x two key blocks
  const float inv_area = 1.0f / static_cast<float>(bs * bs);
  if (bs == 64) {
    for (int half = 0; half < 2; ++half) {
      const int bi = (row0 / 64) + half;
      if (bi >= n) break;
      __half* dst = map + (static_cast<int64_t>(bh) * n + bi) * n;
      for (int bj = threadIdx.x; bj < n; bj += kRmThreads)
        dst[bj] = __float2half_rn(static_cast<float>(cnt[half * nkb + bj]) * inv_area);
    }
  } else {
    const int bi = row0 / 128;
    if (bi < n) {
      __half* dst = map + (static_cast<int64_t>(bh) * n + bi) * n;
      for (int bj = threadIdx.x; bj < n; bj += kRmThreads) {
        const int c = cnt[2 * bj] + cnt[2 * bj + 1] + cnt[nkb + 2 * bj] + cnt[nkb + 2 * bj + 1];
        dst[bj] = __float2half_rn(static_cast<float>(c) * inv_area);
      }
    }
  }
}

template <int D, bool kBF16>
int launch_mma(const void* q, const void* k, const float* lse, int BH, int N, int bs, float scale, float log_thr,
               int q_off, int k_off, int n, void* map, cudaStream_t st) {
  const int vtok = n * bs;
  const int nkb = ceil_div(vtok, kRmKeys);
  const size_t smem = sizeof(uint16_t) * kRmKeys * (D + 8) + sizeof(int) * 2 * nkb;
  auto kernel = replay_map_mma_kernel<D, kBF16>;
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem)) return rc;
  kernel<<<dim3(ceil_div(vtok, kRmRows), BH), kRmThreads, smem, st>>>(
      static_cast<const uint16_t*>(q), static_cast<const uint16_t*>(k), lse, N, bs, scale, log_thr, q_off, k_off, n,
      static_cast<__half*>(map));
  MODDIT_CHECK_LAUNCH("replay_map_mma_kernel");
  return MODDIT_OK;
}

}  // namespace
}  // namespace moddit

using namespace moddit;

extern "C" int moddit_replay_map_mma(const void* q, const void* k, const float* lse, int dtype, int BH, int N, int D,
                                     int block_size, float softmax_scale, float log_threshold, int q_video_offset,
                                     int k_video_offset, int video_blocks, void* map_f16, void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(q && k && lse && map_f16, "replay_map_mma: null pointer");
  MODDIT_CHECK_ARG(BH > 0 && BH <= 65535 && N > 0, "replay_map_mma: BH=%d N=%d out of range", BH, N);
  MODDIT_CHECK_ARG(video_blocks > 0, "replay_map_mma: video_blocks must be positive");
  MODDIT_CHECK_ARG(q_video_offset >= 0 && k_video_offset >= 0, "replay_map_mma: video offsets must be non-negative");
  if (block_size != 64 && block_size != 128)
    return fail(MODDIT_E_UNSUPPORTED, "replay_map_mma: block_size must be 64 or 128, got %d", block_size);
  if (D != 64 && D != 128) return fail(MODDIT_E_UNSUPPORTED, "replay_map_mma: head_dim must be 64 or 128, got %d", D);
  if (dtype != MODDIT_BF16 && dtype != MODDIT_FP16) return fail(MODDIT_E_ARG, "replay_map_mma: unknown dtype %d", dtype);
  const long long vt = static_cast<long long>(video_blocks) * block_size;
  MODDIT_CHECK_ARG(q_video_offset + vt <= N, "replay_map_mma: Q video region exceeds sequence length");
  MODDIT_CHECK_ARG(k_video_offset + vt <= N, "replay_map_mma: K video region exceeds sequence length");
  if (!aligned16(q) || !aligned16(k)) return fail(MODDIT_E_ALIGN, "replay_map_mma: q and k must be 16-byte aligned");
  if (int rc = require_sm100()) return rc;
  cudaStream_t st = as_stream(stream);
  if (D == 128) {
    return dtype == MODDIT_BF16
               ? launch_mma<128, true>(q, k, lse, BH, N, block_size, softmax_scale, log_threshold, q_video_offset,
                                       k_video_offset, video_blocks, map_f16, st)
               : launch_mma<128, false>(q, k, lse, BH, N, block_size, softmax_scale, log_threshold, q_video_offset,
                                        k_video_offset, video_blocks, map_f16, st);
  }
  return dtype == MODDIT_BF16
             ? launch_mma<64, true>(q, k, lse, BH, N, block_size, softmax_scale, log_threshold, q_video_offset,
                                    k_video_offset, video_blocks, map_f16, st)
             : launch_mma<64, false>(q, k, lse, BH, N, block_size, softmax_scale, log_threshold, q_video_offset,
                                     k_video_offset, video_blocks, map_f16, st);
}
