// Exact sparsity-map replay for sm_100a: S = round(q*scale) k^T on the tcgen05 tensor pipe, then a
// compare-and-count epilogue straight out of tensor memory.
//
// One CTA owns 128 consecutive video query rows of one head and sweeps all video key tiles.
//   warp 0      TMA producer: Q tile once, K tiles through a 4-stage ring
//   warp 1      MMA issuer: two key tiles per instruction (N = 256: the instruction-issue cost of the one
//               issuing thread, not the tensor pipe, limits this kernel), into one of two 256-column
//               accumulators
//   warp 2      tensor-memory allocation / release
//   warps 4-7   count group 0 (even key tiles = first 128 columns of an accumulator); thread r owns row r
//   warps 8-11  count group 1 (odd key tiles = second 128 columns)
// The Q tile is scaled and rounded to the input dtype in shared memory before the first MMA (the
// reference rounds the scaled query the same way).  Counts of the four 64x64 quarters of every
// 128x128 tile are accumulated in shared memory and the finished map rows are written once, coalesced.
// Tensor-pipe work: 2*128*128*D flop per tile; memory traffic: one K tile (128*D*2 bytes) per tile,
// served from L2 for all but the first query tile of a head.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "ptx.cuh"
#include "tmap.cuh"

namespace moddit {
namespace {

constexpr int kThreads = 384;
constexpr int kTile = 128;
constexpr int kStages = 4;
constexpr int kPairStages = kStages / 2;

enum BarrierIndex {
  kQFull = 0,
  kQReady,
  kKFull0,                          // kPairStages: both key tiles of a pair have landed
  kKEmpty0 = kKFull0 + kPairStages, // kPairStages
  kSFull0 = kKEmpty0 + kPairStages, // 2: accumulator b holds the scores of key tiles 2*pj, 2*pj+1
  kSFree0 = kSFull0 + 2,        // 2
  kNumBarriers = kSFree0 + 2
};

struct __align__(8) Control {
  unsigned long long bars[kNumBarriers];
  uint32_t tmem_base;
  int abort_flag;
};

template <int D>
constexpr size_t fixed_smem_bytes() {
  return static_cast<size_t>(1 + kStages) * kTile * D * 2 + 1024 + sizeof(Control);
}

__device__ __forceinline__ void report(int32_t* status, int code, int role, int where) {
  if (atomicCAS(status, 0, code) == 0) {
    status[1] = static_cast<int32_t>(blockIdx.y * gridDim.x + blockIdx.x);
    status[2] = role;
    status[3] = where;
  }
}

template <int D, bool kBF16>
__global__ void __launch_bounds__(kThreads, 1) replay_map_kernel(
    const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
    const float* __restrict__ lse, int N, int bs, float scale, float log_thr, int q_off, int k_off, int n,
    __half* __restrict__ map, int32_t* __restrict__ status) {
  constexpr int kTileBytes = kTile * D * 2;
  constexpr int kChunks = D / 64;
  constexpr int kChunkBytes = kTile * 128;
  constexpr uint32_t kIdesc256 = ptx::idesc_f16(128, 256, kBF16, false);
  constexpr uint32_t kIdesc128 = ptx::idesc_f16(128, 128, kBF16, false);
  // K ring, chunk-major: [64-column chunk][stage][128 rows x 128 B], so the rows of two consecutive stages are
  // contiguous inside a chunk and one N = 256 operand covers both tiles
  constexpr int kRingChunkBytes = kStages * kChunkBytes;

  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Control* ctl = reinterpret_cast<Control*>(smem + (1 + kStages) * kTileBytes);
  int* quarter = reinterpret_cast<int*>(ctl + 1);           // [ntk][4] counts of the 64x64 quarters
  const uint32_t sQ = ptx::smem_u32(smem);
  const uint32_t sK = sQ + kTileBytes;
  const uint32_t bar0 = ptx::smem_u32(&ctl->bars[0]);
  auto bar = [&](int i) { return bar0 + 8u * static_cast<uint32_t>(i); };
  volatile int* abort_flag = &ctl->abort_flag;

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  const int qt = blockIdx.x;
  const int bh = blockIdx.y;
  const int vtok = n * bs;                                  // video tokens
  const int ntk = (vtok + kTile - 1) / kTile;
  const int qrow0 = q_off + qt * kTile;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kNumBarriers; ++i) {
      uint32_t c = 1;
      if (i == kQReady) c = 256;
      if (i >= kSFree0) c = 256;
      ptx::mbar_init(bar(i), c);
    }
    ctl->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&tm_q);
    ptx::prefetch_tensormap(&tm_k);
  }
  for (int i = threadIdx.x; i < ntk * 4; i += kThreads) quarter[i] = 0;
  if (warp == 2) {
    ptx::tmem_alloc(ptx::smem_u32(&ctl->tmem_base), 512);
    ptx::tmem_relinquish();
    ptx::tc_fence_before();
  }
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      ptx::mbar_expect_tx(bar(kQFull), kTileBytes);
      for (int c = 0; c < kChunks; ++c) ptx::tma_load_3d(sQ + c * kChunkBytes, &tm_q, bar(kQFull), c * 64, qrow0, bh);
      // two key tiles (one N = 256 operand) share a barrier pair: the issuing thread pays one wait and one
      // commit per MMA group for its operands
      bool ok = true;
      int issued = 0;
      for (int j = 0; j < ntk; j += 2) {
        const int pj = j / 2;
        const int ps = pj % kPairStages;
        const bool two = (j + 1) < ntk;
        ok = ptx::mbar_wait(bar(kKEmpty0 + ps), ((pj / kPairStages) & 1) ^ 1, abort_flag);
        if (!ok) { report(status, 1, 0, j); break; }
        ptx::mbar_expect_tx(bar(kKFull0 + ps), (two ? 2u : 1u) * kTileBytes);
        for (int t = 0; t < (two ? 2 : 1); ++t)
          for (int c = 0; c < kChunks; ++c)
            ptx::tma_load_3d(sK + c * kRingChunkBytes + (2 * ps + t) * kChunkBytes, &tm_k, bar(kKFull0 + ps), c * 64,
                             k_off + (j + t) * kTile, bh);
        issued = pj + 1;
      }
      if (!ok) {
        for (int pj = max(0, issued - kPairStages); pj < issued; ++pj)
          for (int i = 0; i < 4096 && !ptx::mbar_try_wait(bar(kKFull0 + pj % kPairStages), (pj / kPairStages) & 1); ++i) {}
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = ptx::mbar_wait(bar(kQReady), 0, abort_flag);
      if (!ok) report(status, 2, 1, -1);
      const uint64_t dq0 = ptx::smem_desc_sw128(sQ, 16, 1024);
      const uint64_t dk0 = ptx::smem_desc_sw128(sK, 16, 1024);
      auto advance = [](uint64_t desc, uint32_t bytes) -> uint64_t {
        // the start-address field (units of 16 bytes) never carries out for shared-memory addresses
        return (desc & 0xffffffff00000000ull) | static_cast<uint32_t>(static_cast<uint32_t>(desc) + (bytes >> 4));
      };
      for (int j = 0; j < ntk && ok; j += 2) {
        const int pj = j / 2;
        const int ps = pj % kPairStages;
        const int b = pj & 1;
        const bool two = (j + 1) < ntk;
        ok = ptx::mbar_wait(bar(kKFull0 + ps), (pj / kPairStages) & 1, abort_flag);
        if (ok) ok = ptx::mbar_wait(bar(kSFree0 + b), ((pj >> 1) & 1) ^ 1, abort_flag);
        if (!ok) { report(status, 2, 1, j); break; }
        ptx::tc_fence_after();
        const uint64_t dk = advance(dk0, static_cast<uint32_t>(2 * ps) * kChunkBytes);
        const uint32_t idesc = two ? kIdesc256 : kIdesc128;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          ptx::mma_ss(tmem + b * 256, advance(dq0, (kk / 4) * kChunkBytes + (kk % 4) * 32),
                      advance(dk, (kk / 4) * kRingChunkBytes + (kk % 4) * 32), idesc, kk > 0 ? 1u : 0u);
        ptx::tc_commit(bar(kSFull0 + b));
        ptx::tc_commit(bar(kKEmpty0 + ps));
      }
    }
  } else if (warp >= 4) {
    const int g = (warp - 4) / 4;
    const int wq = warp % 4;
    const int r = wq * 32 + lane;
    const int t256 = threadIdx.x - 128;                     // 0..255 over both count groups
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;

    // scale + round the Q tile in place (element-wise, so the swizzled order does not matter)
    bool ok = ptx::mbar_wait(bar(kQFull), 0, abort_flag);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      uint4* q4 = reinterpret_cast<uint4*>(smem);
      for (int i = t256; i < kTileBytes / 16; i += 256) {
        uint4 w = q4[i];
        uint32_t* p = reinterpret_cast<uint32_t*>(&w);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if constexpr (kBF16) {
            const __nv_bfloat162 h2 = *reinterpret_cast<const __nv_bfloat162*>(&p[u]);
            const __nv_bfloat162 o2 = __halves2bfloat162(__float2bfloat16_rn(__bfloat162float(h2.x) * scale),
                                                         __float2bfloat16_rn(__bfloat162float(h2.y) * scale));
            p[u] = *reinterpret_cast<const uint32_t*>(&o2);
          } else {
            const __half2 h2 = *reinterpret_cast<const __half2*>(&p[u]);
            const __half2 o2 = __halves2half2(__float2half_rn(__half2float(h2.x) * scale),
                                              __float2half_rn(__half2float(h2.y) * scale));
            p[u] = *reinterpret_cast<const uint32_t*>(&o2);
          }
        }
        q4[i] = w;
      }
      ptx::fence_proxy_async_smem();
      ptx::mbar_arrive(bar(kQReady));
    } else if (lane == 0) {
      report(status, 4, 2 + g, -1);
    }

    const int grow = qrow0 + r;
    const bool row_ok = (qt * kTile + r) < vtok && grow < N;
    const float line = row_ok ? (lse[static_cast<int64_t>(bh) * N + grow] + log_thr) : -INFINITY;
    const int rh = r >> 6;
    for (int j = g; j < ntk && ok; j += 2) {
      const int pj = j / 2;
      const int b = pj & 1;
      ok = ptx::mbar_wait(bar(kSFull0 + b), (pj >> 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { if (lane == 0) report(status, 5, 2 + g, j); break; }
      ptx::tc_fence_after();
      float v[kTile];
#pragma unroll
      for (int c = 0; c < 4; ++c) ptx::tmem_ld32(tmem + lane_base + b * 256 + g * 128 + c * 32, reinterpret_cast<uint32_t*>(v) + c * 32);
      ptx::tmem_ld_wait();
      ptx::tc_fence_before();
      ptx::mbar_arrive(bar(kSFree0 + b));
      int c_lo = 0, c_hi = 0;
#pragma unroll
      for (int c = 0; c < 64; ++c) c_lo += (v[c] < line) ? 1 : 0;
#pragma unroll
      for (int c = 64; c < 128; ++c) c_hi += (v[c] < line) ? 1 : 0;
      c_lo = __reduce_add_sync(0xffffffffu, c_lo);
      c_hi = __reduce_add_sync(0xffffffffu, c_hi);
      if (lane == 0) {
        atomicAdd(&quarter[j * 4 + rh * 2 + 0], c_lo);
        atomicAdd(&quarter[j * 4 + rh * 2 + 1], c_hi);
      }
    }
    // all 256 counting threads meet, then write the finished map rows
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (!*abort_flag) {
      const float inv_area = 1.0f / static_cast<float>(bs * bs);
      if (bs == 128) {
        if (qt < n) {
          __half* dst = map + (static_cast<int64_t>(bh) * n + qt) * n;
          for (int j = t256; j < n; j += 256) {
            const int cnt = quarter[j * 4] + quarter[j * 4 + 1] + quarter[j * 4 + 2] + quarter[j * 4 + 3];
            dst[j] = __float2half_rn(static_cast<float>(cnt) * inv_area);
          }
        }
      } else {
        for (int h2 = 0; h2 < 2; ++h2) {
          const int bi = qt * 2 + h2;
          if (bi >= n) break;
          __half* dst = map + (static_cast<int64_t>(bh) * n + bi) * n;
          for (int bj = t256; bj < n; bj += 256)
            dst[bj] = __float2half_rn(static_cast<float>(quarter[(bj >> 1) * 4 + h2 * 2 + (bj & 1)]) * inv_area);
        }
      }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, 512);
  }
}

template <int D, bool kBF16>
int launch(const void* q, const void* k, const float* lse, int dtype, int BH, int N, int bs, float scale,
           float log_thr, int q_off, int k_off, int n, void* map, int32_t* status, cudaStream_t st) {
  CUtensorMap tq, tk;
  if (int rc = make_tmap_rows(&tq, q, dtype, BH, N, D, kTile)) return rc;
  if (int rc = make_tmap_rows(&tk, k, dtype, BH, N, D, kTile)) return rc;
  const int ntk = ceil_div(n * bs, kTile);
  const size_t smem = fixed_smem_bytes<D>() + static_cast<size_t>(ntk) * 4 * sizeof(int);
  if (smem > 227 * 1024) return fail(MODDIT_E_UNSUPPORTED, "replay_map: %d key tiles do not fit the shared-memory counters", ntk);
  auto kernel = replay_map_kernel<D, kBF16>;
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem)) return rc;
  kernel<<<dim3(ntk, BH), kThreads, smem, st>>>(tq, tk, lse, N, bs, scale, log_thr, q_off, k_off, n,
                                                static_cast<__half*>(map), status);
  MODDIT_CHECK_LAUNCH("replay_map_kernel");
  return MODDIT_OK;
}

}  // namespace
}  // namespace moddit

using namespace moddit;

// The status words live in a small device buffer owned by the library user only for the sparse
// forward; the replay entry point keeps the reference's signature (no status argument), so it uses a
// per-device static word that the kernel only ever writes when a bounded wait expires.
static __device__ int32_t g_replay_status[4];

extern "C" int moddit_replay_map(const void* q, const void* k, const float* lse, int dtype, int BH, int N, int D,
                                 int block_size, float softmax_scale, float log_threshold, int q_video_offset,
                                 int k_video_offset, int video_blocks, void* map_f16, void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(q && k && lse && map_f16, "replay_map: null pointer");
  MODDIT_CHECK_ARG(BH > 0 && BH <= 65535 && N > 0, "replay_map: BH=%d N=%d out of range", BH, N);
  MODDIT_CHECK_ARG(video_blocks > 0, "replay_map: video_blocks must be positive");
  MODDIT_CHECK_ARG(q_video_offset >= 0 && k_video_offset >= 0, "replay_map: video offsets must be non-negative");
  if (block_size != 64 && block_size != 128)
    return fail(MODDIT_E_UNSUPPORTED, "replay_map: block_size must be 64 or 128, got %d", block_size);
  if (D != 64 && D != 128) return fail(MODDIT_E_UNSUPPORTED, "replay_map: head_dim must be 64 or 128, got %d", D);
  if (dtype != MODDIT_BF16 && dtype != MODDIT_FP16) return fail(MODDIT_E_ARG, "replay_map: unknown dtype %d", dtype);
  const long long vt = static_cast<long long>(video_blocks) * block_size;
  MODDIT_CHECK_ARG(q_video_offset + vt <= N, "replay_map: Q video region exceeds sequence length");
  MODDIT_CHECK_ARG(k_video_offset + vt <= N, "replay_map: K video region exceeds sequence length");
  if (!aligned16(q) || !aligned16(k)) return fail(MODDIT_E_ALIGN, "replay_map: q and k must be 16-byte aligned");
  if (int rc = require_sm100()) return rc;
  int32_t* status = nullptr;
  MODDIT_CHECK_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_replay_status));
  cudaStream_t st = as_stream(stream);
  if (D == 128) {
    return dtype == MODDIT_BF16 ? launch<128, true>(q, k, lse, dtype, BH, N, block_size, softmax_scale, log_threshold,
                                                    q_video_offset, k_video_offset, video_blocks, map_f16, status, st)
                                : launch<128, false>(q, k, lse, dtype, BH, N, block_size, softmax_scale, log_threshold,
                                                     q_video_offset, k_video_offset, video_blocks, map_f16, status, st);
  }
  return dtype == MODDIT_BF16 ? launch<64, true>(q, k, lse, dtype, BH, N, block_size, softmax_scale, log_threshold,
                                                 q_video_offset, k_video_offset, video_blocks, map_f16, status, st)
                              : launch<64, false>(q, k, lse, dtype, BH, N, block_size, softmax_scale, log_threshold,
                                                  q_video_offset, k_video_offset, video_blocks, map_f16, status, st);
}

// Reads (and clears) the replay kernel's status words; non-zero code means a bounded wait expired in
// some earlier replay launch on the current device.  Synchronises `stream`.
extern "C" int moddit_replay_status(int32_t* host_status4, void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(host_status4, "replay_status: null pointer");
  int32_t* status = nullptr;
  MODDIT_CHECK_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_replay_status));
  cudaStream_t st = as_stream(stream);
  MODDIT_CHECK_CUDA(cudaMemcpyAsync(host_status4, status, 4 * sizeof(int32_t), cudaMemcpyDeviceToHost, st));
  MODDIT_CHECK_CUDA(cudaMemsetAsync(status, 0, 4 * sizeof(int32_t), st));
  MODDIT_CHECK_CUDA(cudaStreamSynchronize(st));
  return MODDIT_OK;
}
