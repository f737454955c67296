// Block-sparse flash-attention forward for sm_100a: tcgen05 MMAs with accumulators in tensor memory,
// K/V tiles fetched by TMA from a compacted work list (a skipped block costs no memory traffic),
// warp-specialised online softmax.
//
// One CTA owns a PAIR of adjacent 128-row query tiles (A, B) of one head and walks the union of
// their key-tile lists, so a K/V tile needed by both is fetched once.  Roles (12 warps):
//   warp 0      TMA producer: Q tiles once, then K and V tiles through two 2-stage rings (V of entry e and K
//               of entry e + 1 share their barriers: they are consumed together)
//   warp 1      MMA issuer: S_X = Q_X K^T (SS form), O_X += P_X V (P read from tensor memory)
//   warp 2      tensor-memory allocation / release
//   warps 4-7   softmax of tile A: thread r owns row r (tensor-memory lane r)
//   warps 8-11  softmax of tile B
// Tensor memory (512 columns): S_A [0,128) S_B [128,256) O_A [256,256+D) O_B [256+D,256+2D); P_X
// (16-bit) overwrites the first 64 columns of S_X.  MMAs issued by one thread execute in order, which
// is what makes the aliasing and the "S ready implies the previous P V finished" reasoning valid.
// The issue order  PV(A,e) QK(A,e+1) PV(B,e) QK(B,e+1)  lets the softmax of one tile overlap the MMAs
// of the other.
//
// Every wait is bounded (ptx::mbar_wait); on expiry the CTA records a status word, lets its copies
// land, releases tensor memory and returns.
//
// Tensor-pipe work per kept 128x128 tile: 4*128*128*D flop (QK^T and PV); memory traffic per fetched
// key tile: 2*128*D*2 bytes (K and V), shared by both query tiles.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "ptx.cuh"
#include "tmap.cuh"

namespace moddit {
namespace {

constexpr int kThreads = 384;
constexpr int kTile = 128;
constexpr float kRescaleThreshold = 8.0f;   // log2 domain: rescale O only when the row max grew by more than this

enum BarrierIndex {
  kQFull = 0,
  kKFirst,                      // K tile of entry 0
  kFull0, kFull1,               // entry e (index e & 1): V tile of e and K tile of e + 1 have landed
  kEmpty0, kEmpty1,             // entry e: its V stage and the K stage of e + 1 may be overwritten
  kSFullA, kSFullB,
  kPLoA, kPHiA, kPLoB, kPHiB,   // first / second half row of P stored, per query tile
  kOFinal,
  kNumBarriers
};

// Optional destination of the output rows on a multi-GPU run: instead of one local (BH, N, D) tensor the
// rows of sequence shard r (rows [r*rows_per_peer, (r+1)*rows_per_peer)) are stored straight into rank r's
// (total_heads, rows_per_peer, D) buffer at head `head_base + bh` - the output re-shard is fused into the
// epilogue as plain peer stores.
constexpr int kMaxPeers = 8;
struct OutScatter {
  void* peer[kMaxPeers];
  int n_peers;          // 0: write `out` locally
  int rows_per_peer;
  int head_base;
};

struct __align__(8) Control {
  unsigned long long bars[kNumBarriers];
  uint32_t tmem_base;
  int abort_flag;
};

template <int D>
constexpr size_t smem_bytes() {
  // 2 Q tiles + 2 K stages + 2 V stages, 1024-byte alignment slack, control block
  return static_cast<size_t>(6) * kTile * D * 2 + 1024 + sizeof(Control);
}

__device__ __forceinline__ void report(int32_t* status, int code, int role, int where) {
  if (atomicCAS(status, 0, code) == 0) {
    status[1] = static_cast<int32_t>(blockIdx.y * gridDim.x + blockIdx.x);
    status[2] = role;
    status[3] = where;
  }
}

template <bool kBF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (kBF16) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
  } else {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
}

template <int D, bool kBF16>
__global__ void __launch_bounds__(kThreads, 1) sparse_attn_fwd_kernel(
    const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
    const __grid_constant__ CUtensorMap tm_v, const int32_t* __restrict__ counts,
    const int32_t* __restrict__ entries, const int32_t* __restrict__ order, int Hm, int ntk, int N, float scale_log2, int q_split, int kvl_lo,
    int kvl_hi, void* __restrict__ out_raw, float* __restrict__ lse, int32_t* __restrict__ status,
    const __grid_constant__ OutScatter scatter) {
  constexpr int kTileBytes = kTile * D * 2;       // one Q, K or V tile
  constexpr int kChunks = D / 64;                 // 64-element (128-byte) column chunks per tile
  constexpr int kChunkBytes = kTile * 128;
  constexpr uint32_t kIdescQK = ptx::idesc_f16(128, 128, kBF16, false);
  constexpr uint32_t kIdescPV = ptx::idesc_f16(128, D, kBF16, true);

  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Control* ctl = reinterpret_cast<Control*>(smem + 6 * kTileBytes);
  const uint32_t sQ = ptx::smem_u32(smem);
  const uint32_t sK = sQ + 2 * kTileBytes;
  const uint32_t sV = sQ + 4 * kTileBytes;
  const uint32_t bar0 = ptx::smem_u32(&ctl->bars[0]);
  auto bar = [&](int i) { return bar0 + 8u * static_cast<uint32_t>(i); };
  volatile int* abort_flag = &ctl->abort_flag;

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  // grid: x = work item (mask head, query-tile pair), y = batch.  Blocks start in increasing blockIdx.x;
  // `order` (from the work-list builder) puts long lists first, otherwise items run head by head.
  const int npairs = static_cast<int>(gridDim.x) / Hm;
  const int item = order ? order[blockIdx.x] : static_cast<int>(blockIdx.x);
  const int mh = item / npairs;
  const int pair = item - mh * npairs;
  const int bh = blockIdx.y * Hm + mh;
  const int ntq = (N + kTile - 1) / kTile;
  const bool has_b = (2 * pair + 1) < ntq;
  const int cnt = counts[static_cast<int64_t>(mh) * npairs + pair];
  const int32_t* ent = entries + (static_cast<int64_t>(mh) * npairs + pair) * ntk;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kNumBarriers; ++i) ptx::mbar_init(bar(i), (i >= kPLoA && i <= kPHiB) ? 128u : 1u);
    ctl->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&tm_q);
    ptx::prefetch_tensormap(&tm_k);
    ptx::prefetch_tensormap(&tm_v);
  }
  if (warp == 2) {
    ptx::tmem_alloc(ptx::smem_u32(&ctl->tmem_base), 512);
    ptx::tmem_relinquish();
    ptx::tc_fence_before();
  }
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;

  // Register budget: the softmax warpgroups hold a 128-value row per thread, the control warps need little
  // (128 control threads give up what 256 softmax threads take: 168 -> 72 / 216 at D = 128 and 56 / 224 at
  // D = 64, the splits that leave each instantiation without a single spill).
  // The control branch and the softmax branch are disjoint in the control-flow graph so that each gets
  // its own register allocation.
  if (warp < 4) {
  if constexpr (D == 128) asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
  else asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      ptx::mbar_expect_tx(bar(kQFull), (has_b ? 2u : 1u) * kTileBytes);
      for (int x = 0; x < (has_b ? 2 : 1); ++x)
        for (int c = 0; c < kChunks; ++c)
          ptx::tma_load_3d(sQ + x * kTileBytes + c * kChunkBytes, &tm_q, bar(kQFull), c * 64, (2 * pair + x) * kTile,
                           bh);
      // Entry e consumes V(e) and K(e+1) together (P V of e, then Q K^T of e + 1), so the two tiles share one
      // pair of barriers: the MMA-issuing thread pays one wait and one commit per entry for its operands.
      bool ok = true;
      int issued = 0;
      if (cnt > 0) {
        ptx::mbar_expect_tx(bar(kKFirst), kTileBytes);
        for (int c = 0; c < kChunks; ++c)
          ptx::tma_load_3d(sK + c * kChunkBytes, &tm_k, bar(kKFirst), c * 64, (ent[0] >> 8) * kTile, bh);
      }
      for (int e = 0; e < cnt && ok; ++e) {
        const int s = e & 1;
        // kEmpty1 also completes once before the loop (the first K tile's stage), hence the shifted parity
        const uint32_t par = ((e >> 1) & 1) ^ (s ? 0u : 1u);
        const bool next = (e + 1) < cnt;
        ok = ptx::mbar_wait(bar(kEmpty0 + s), par, abort_flag);
        if (!ok) { report(status, 1, 0, e); break; }
        ptx::mbar_expect_tx(bar(kFull0 + s), (next ? 2u : 1u) * kTileBytes);
        const int row0 = (ent[e] >> 8) * kTile;
        for (int c = 0; c < kChunks; ++c)
          ptx::tma_load_3d(sV + s * kTileBytes + c * kChunkBytes, &tm_v, bar(kFull0 + s), c * 64, row0, bh);
        if (next) {
          const int row1 = (ent[e + 1] >> 8) * kTile;
          for (int c = 0; c < kChunks; ++c)
            ptx::tma_load_3d(sK + (s ^ 1) * kTileBytes + c * kChunkBytes, &tm_k, bar(kFull0 + s), c * 64, row1, bh);
        }
        issued = e + 1;
      }
      if (!ok) {
        // give copies in flight a bounded time to land (their barriers may never be consumed)
        for (int i = 0; i < 4096 && cnt > 0 && !ptx::mbar_try_wait(bar(kKFirst), 0); ++i) {}
        for (int e = max(0, issued - 2); e < issued; ++e)
          for (int i = 0; i < 4096 && !ptx::mbar_try_wait(bar(kFull0 + (e & 1)), (e >> 1) & 1); ++i) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // Descriptor bases are built once; inside the loops an MMA costs one 32-bit add per operand (the
      // issuing thread shares its scheduler with two busy softmax warps, so every instruction counts).
      const uint64_t dq[2] = {ptx::smem_desc_sw128(sQ, 16, 1024), ptx::smem_desc_sw128(sQ + kTileBytes, 16, 1024)};
      const uint64_t dk[2] = {ptx::smem_desc_sw128(sK, 16, 1024), ptx::smem_desc_sw128(sK + kTileBytes, 16, 1024)};
      const uint64_t dv[2] = {ptx::smem_desc_sw128(sV, kChunkBytes, 1024),
                              ptx::smem_desc_sw128(sV + kTileBytes, kChunkBytes, 1024)};
      auto advance = [](uint64_t desc, uint32_t bytes) -> uint64_t {
        // the start-address field (bits 0-13, units of 16 bytes) never carries out for shared-memory addresses
        return (desc & 0xffffffff00000000ull) | static_cast<uint32_t>(static_cast<uint32_t>(desc) + (bytes >> 4));
      };
      auto issue_qk = [&](int x, int s) {
        const uint64_t a0 = dq[x], b0 = dk[s];
        const uint32_t d = tmem + x * 128;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * kChunkBytes + (kk % 4) * 32;
          ptx::mma_ss(d, advance(a0, off), advance(b0, off), kIdescQK, kk > 0 ? 1u : 0u);
        }
        ptx::tc_commit(bar(kSFullA + x));
      };
      // P*V for one half of the key tile (keys [64*half, 64*half+64))
      auto issue_pv_half = [&](int x, int s, int half, uint32_t acc) {
        const uint64_t b0 = dv[s];
        const uint32_t d = tmem + 256 + x * D, a = tmem + x * 128;
#pragma unroll
        for (int kq = 0; kq < kTile / 32; ++kq) {
          const int kk = half * (kTile / 32) + kq;
          ptx::mma_ts(d, a + kk * 8, advance(b0, kk * 2048), kIdescPV, (acc || kq > 0) ? 1u : 0u);
        }
      };
      // waits for the two half rows of P in turn; returns false if a wait gave up
      auto pv_when_ready = [&](int x, int s, uint32_t acc, uint32_t parity) -> bool {
        if (!ptx::mbar_wait(bar(kPLoA + 2 * x), parity, abort_flag)) return false;
        ptx::tc_fence_after();
        issue_pv_half(x, s, 0, acc);
        if (!ptx::mbar_wait(bar(kPHiA + 2 * x), parity, abort_flag)) return false;
        ptx::tc_fence_after();
        issue_pv_half(x, s, 1, 1u);
        return true;
      };
      bool ok = ptx::mbar_wait(bar(kQFull), 0, abort_flag);
      if (!ok) report(status, 2, 1, -1);
      uint32_t par_p[2] = {0, 0};
      uint32_t acc[2] = {0, 0};
      if (ok && cnt > 0) {
        ok = ptx::mbar_wait(bar(kKFirst), 0, abort_flag);
        if (!ok) report(status, 2, 1, 0);
        if (ok) {
          ptx::tc_fence_after();
          const int fl = ent[0] & 0xff;
          if (fl & 0x0f) issue_qk(0, 0);
          if (fl & 0xf0) issue_qk(1, 0);
          ptx::tc_commit(bar(kEmpty1));     // K stage 0 is free for the K tile of entry 2 (loaded with V of entry 1)
        }
      }
      int fl_carry = (cnt > 0) ? (ent[0] & 0xff) : 0;
      for (int e = 0; e < cnt && ok; ++e) {
        const int s = e & 1;
        const int fl = fl_carry;
        const bool next = (e + 1) < cnt;
        const int fln = next ? (ent[e + 1] & 0xff) : 0;   // issued here, first used after the P V of tile A
        fl_carry = fln;
        ok = ptx::mbar_wait(bar(kFull0 + s), (e >> 1) & 1, abort_flag);
        if (!ok) { report(status, 2, 1, e); break; }
        if (fl & 0x0f) {
          ok = pv_when_ready(0, s, acc[0], par_p[0]);
          if (!ok) { report(status, 3, 1, e); break; }
          par_p[0] ^= 1;
          acc[0] = 1;
        }
        if (fln & 0x0f) issue_qk(0, s ^ 1);
        if (fl & 0xf0) {
          ok = pv_when_ready(1, s, acc[1], par_p[1]);
          if (!ok) { report(status, 3, 1, e); break; }
          par_p[1] ^= 1;
          acc[1] = 1;
        }
        if (fln & 0xf0) issue_qk(1, s ^ 1);
        ptx::tc_commit(bar(kEmpty0 + s));
      }
      ptx::tc_commit(bar(kOFinal));
    }
  }
  } else {
    if constexpr (D == 128) asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    else asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    // ------------------------------------------------------------------ softmax + epilogue
    const int x = (warp - 4) / 4;                 // 0: tile A, 1: tile B
    const int wq = warp % 4;                      // tensor-memory lane quarter of this warp
    const int r = wq * 32 + lane;                 // row inside the tile
    const int tile = 2 * pair + x;
    const int grow = tile * kTile + r;            // global query row
    const int kvl = (grow < q_split) ? kvl_lo : kvl_hi;
    const int kvl_min = min(kvl_lo, kvl_hi);
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
    const uint32_t tS = tmem + lane_base + x * 128;
    const uint32_t tO = tmem + lane_base + 256 + x * D;
    const int rh = r >> 6;

    float m = -INFINITY, l = 0.f;
    uint32_t par_s = 0;
    int done = 0;
    bool ok = true;
    for (int e = 0; e < cnt; ++e) {
      const int en = ent[e];
      const int sub = (en >> (4 * x)) & 0xf;
      if (!sub) continue;
      const int col0 = (en >> 8) * kTile;
      ok = ptx::mbar_wait(bar(kSFullA + x), par_s, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { if (lane == 0) report(status, 4, 2 + x, e); break; }
      par_s ^= 1;
      ptx::tc_fence_after();

      float v[kTile];
#pragma unroll
      for (int c = 0; c < 4; ++c) ptx::tmem_ld32(tS + c * 32, reinterpret_cast<uint32_t*>(v) + c * 32);
      ptx::tmem_ld_wait();

      if (sub != 0xf || col0 + kTile > kvl_min) {
        const int lim = kvl - col0;               // columns >= lim are beyond the valid keys
        const bool keep_lo = (sub >> (2 * rh)) & 1;
        const bool keep_hi = (sub >> (2 * rh + 1)) & 1;
#pragma unroll
        for (int c = 0; c < kTile; ++c) {
          const bool valid = (c < 64 ? keep_lo : keep_hi) && (c < lim);
          v[c] = valid ? v[c] : -INFINITY;
        }
      }
      // P = exp2(S*scale - ref) for the whole row, packed to 16 bits and stored over the first 64 columns
      // of S; returns the row sum.
      // row maximum: eight independent chains of three-input max
      float mxa[8];
#pragma unroll
      for (int a = 0; a < 8; ++a) mxa[a] = ptx::max3(v[a], v[a + 8], v[a + 16]);
#pragma unroll
      for (int c = 24; c + 16 <= kTile; c += 16)
#pragma unroll
        for (int a = 0; a < 8; ++a) mxa[a] = ptx::max3(mxa[a], v[c + a], v[c + a + 8]);
#pragma unroll
      for (int a = 0; a < 8; ++a) mxa[a] = fmaxf(mxa[a], v[kTile - 8 + a]);
      const float mx = fmaxf(ptx::max3(mxa[0], mxa[1], mxa[2]), ptx::max3(mxa[3], mxa[4], mxa[5]));
      const float m_new = fmaxf(m, ptx::max3(mx, mxa[6], mxa[7]) * scale_log2);
      if (done == 0) {
        m = m_new;
      } else if (__any_sync(0xffffffffu, m_new > m + kRescaleThreshold)) {
        const float alpha = (m == -INFINITY) ? 0.f : ptx::ex2(m - m_new);
        l *= alpha;
        m = m_new;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          float o[32];
          ptx::tmem_ld32(tO + c * 32, reinterpret_cast<uint32_t*>(o));
          ptx::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] *= alpha;
          ptx::tmem_st32(tO + c * 32, reinterpret_cast<const uint32_t*>(o));
        }
      }
      // P = exp2(S*scale - m), two fp32 lanes per instruction where the hardware has packed forms; each
      // half row is handed to the MMA warp as soon as it is stored, so P*V starts while the other half
      // is still being computed.
      const float ref = (m == -INFINITY) ? 0.f : m;
      const uint64_t scale2 = ptx::pack_f32x2(scale_log2, scale_log2);
      const uint64_t nref2 = ptx::pack_f32x2(-ref, -ref);
      uint64_t sum2a = 0, sum2b = 0;    // bit pattern of (0.f, 0.f)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const uint64_t x2 = ptx::fma_f32x2(ptx::pack_f32x2(v[half * 64 + 2 * i], v[half * 64 + 2 * i + 1]), scale2, nref2);
          float x0, x1;
          ptx::unpack_f32x2(x2, x0, x1);
          const float p0 = ptx::ex2(x0), p1 = ptx::ex2(x1);
          const uint64_t p2 = ptx::pack_f32x2(p0, p1);
          if (i & 1) sum2b = ptx::add_f32x2(sum2b, p2); else sum2a = ptx::add_f32x2(sum2a, p2);
          pk[i] = pack2<kBF16>(p0, p1);
        }
        ptx::tmem_st32(tS + half * 32, pk);
        ptx::tmem_st_wait();
        ptx::tc_fence_before();
        ptx::mbar_arrive(bar(kPLoA + 2 * x + half));
      }
      float s0, s1, s2, s3;
      ptx::unpack_f32x2(sum2a, s0, s1);
      ptx::unpack_f32x2(sum2b, s2, s3);
      const float sum = (s0 + s1) + (s2 + s3);
      l += sum;
      ++done;
    }

    if (lane == 0 && wq == 0) {
    }
    if (ok) {
      ok = ptx::mbar_wait(bar(kOFinal), 0, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok && lane == 0) report(status, 5, 2 + x, -1);
    }
    if (ok && tile < ntq) {
      ptx::tc_fence_after();
      const float inv = (done > 0 && l > 0.f) ? 1.f / l : 0.f;
      uint4* dst;
      if (scatter.n_peers > 0) {
        const int r = min(grow / scatter.rows_per_peer, scatter.n_peers - 1);
        dst = reinterpret_cast<uint4*>(
            static_cast<unsigned char*>(scatter.peer[r]) +
            (static_cast<int64_t>(scatter.head_base + bh) * scatter.rows_per_peer + (grow - r * scatter.rows_per_peer)) * D * 2);
      } else {
        dst = reinterpret_cast<uint4*>(static_cast<unsigned char*>(out_raw) +
                                       (static_cast<int64_t>(bh) * N + grow) * D * 2);
      }
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        float o[32];
        if (done > 0) {
          ptx::tmem_ld32(tO + c * 32, reinterpret_cast<uint32_t*>(o));
          ptx::tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0.f;
        }
        if (grow < N) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 w;
            w.x = pack2<kBF16>(o[q4 * 8 + 0] * inv, o[q4 * 8 + 1] * inv);
            w.y = pack2<kBF16>(o[q4 * 8 + 2] * inv, o[q4 * 8 + 3] * inv);
            w.z = pack2<kBF16>(o[q4 * 8 + 4] * inv, o[q4 * 8 + 5] * inv);
            w.w = pack2<kBF16>(o[q4 * 8 + 6] * inv, o[q4 * 8 + 7] * inv);
            dst[c * 4 + q4] = w;
          }
        }
      }
      if (lse != nullptr && grow < N) {
        lse[static_cast<int64_t>(bh) * N + grow] =
            (done > 0 && l > 0.f) ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
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

// ====================================================================================================
// Head dimension 64.
//
// At D = 64 a 128 x 128 tile carries half the tensor work of the D = 128 tile for the same 16,384 exponentials, so
// the kernel above - in which a tile's chain Q K^T -> softmax -> P V is strictly serial because P overwrites S -
// spends most of a key-tile slot waiting on that chain.  Here tensor memory has room to break the chain:
//   S_A [0,128)  S_B [128,256)  O_A [256,320)  O_B [320,384)  P_A [384,448)  P_B [448,512)
// P has columns of its own, so Q K^T of the NEXT entry is issued as soon as the softmax has read S of the current
// one into registers (barrier kSFree), and a tile's softmax runs back to back while its products run beside it.
// With the chain gone the two query tiles no longer need one thread to hold them in anti-phase, and each tile gets
// its own issuing thread (warps 1 and 3: a warp can hand over one tcgen05.mma per ~84 clocks, and the twelve
// instructions of a tile-entry at this size keep the pipe busy for half of that).
// What P V(X, e) must not overlap is (1) the softmax overwriting P_X with the next entry's values and (2) the softmax
// rescaling O_X; both wait for tile X's issuer to have finished slot e (kDone_X, committed after the issuer's last
// MMA of the slot), which is also what tells the producer that the slot's K/V stages are free (it waits for both
// tiles').  The barrier is per tile on purpose: one barrier for both would release the two tiles' exponentials at
// the same instant, and they share the special-function unit.
// ====================================================================================================
constexpr int kStages64 = 4;      // K and V tiles in flight (16 KB each at D = 64: shared memory has room, and a tile
                                  // requested only one slot ahead does not always arrive within that slot)
enum BarrierIndex64 {
  k6QFull = 0,
  k6KFirst,
  k6Full0,                                       // [kStages64] V(e) and K(e + 1) have landed (index e % kStages64)
  k6DoneA0 = k6Full0 + kStages64,                // [kStages64] tile A's issuer has finished all its MMAs of slot e
  k6DoneB0 = k6DoneA0 + kStages64,               // [kStages64] the same for tile B
  k6SFullA = k6DoneB0 + kStages64, k6SFullB,
  k6SFreeA, k6SFreeB,            // the softmax warpgroup has read S_X into registers (128 arrivals)
  k6PLoA, k6PHiA, k6PLoB, k6PHiB,
  k6OFinalA, k6OFinalB,
  k6NumBarriers
};

struct __align__(8) Control64 {
  unsigned long long bars[k6NumBarriers];
  uint32_t tmem_base;
  int abort_flag;
};

constexpr size_t smem_bytes_d64() {
  return static_cast<size_t>(2 + 2 * kStages64) * kTile * 64 * 2 + 1024 + sizeof(Control64);
}

// Maximum of 64 values: eight independent chains of three-input max.
__device__ __forceinline__ float row_max64(const float* v) {
  float a[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) a[i] = ptx::max3(v[i], v[i + 8], v[i + 16]);
#pragma unroll
  for (int c = 24; c + 16 <= 64; c += 16)
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] = ptx::max3(a[i], v[c + i], v[c + i + 8]);
#pragma unroll
  for (int i = 0; i < 8; ++i) a[i] = fmaxf(a[i], v[56 + i]);
  return fmaxf(ptx::max3(a[0], a[1], a[2]), ptx::max3(ptx::max3(a[3], a[4], a[5]), a[6], a[7]));
}

// P = exp2(S * scale - ref) for 64 columns of one row: pk[32] = 16-bit pairs; the row sum goes into the packed sums.
//
// The exponential unit does 16 results per clock and SM: a 128 x 128 tile of P costs it 1024 clocks, twice what the
// tensor pipe needs for the tile's two products at D = 64, and with the chain between the products broken it is
// the unit this kernel waits for.  kPoly of every 8 column pairs are therefore computed on the FMA pipe instead:
//   2^x = 2^n * p(f),  n = round(x),  f = x - n in [-1/2, 1/2],  p a cubic with relative error 7.5e-5 (a sixth of
// the rounding step of a bfloat16 P, a sixth of a float16 one's), 2^n added into the exponent field.  x is first
// clamped to [-120, 8] by a saturating FMA ((x + 120) / 128 in [0, 1]); the upper end is the most the lazily
// updated row maximum can trail by, and 2^-120 stands in for anything smaller - rows that must give exact zeros
// (masked columns) use kPoly = 0.
#ifndef MODDIT_D64_POLY_PAIRS
#define MODDIT_D64_POLY_PAIRS 0
#endif
constexpr int kPolyPairs64 = MODDIT_D64_POLY_PAIRS;

template <bool kBF16, int kPoly>
__device__ __forceinline__ void exp_half(const float* v, float scale_log2, float ref, uint32_t* pk, uint64_t& sum2a,
                                         uint64_t& sum2b) {
  const uint64_t scale2 = ptx::pack_f32x2(scale_log2, scale_log2);
  const uint64_t nref2 = ptx::pack_f32x2(-ref, -ref);
  const float pa = scale_log2 * 0.0078125f;
  const float pb = (120.f - ref) * 0.0078125f;
  constexpr float kMagic = 12582912.f - 120.f;            // 1.5 * 2^23 - 120: adding it rounds to an integer
  const uint64_t k128 = ptx::pack_f32x2(128.f, 128.f);
  const uint64_t kmag = ptx::pack_f32x2(kMagic, kMagic);
  const uint64_t kneg = ptx::pack_f32x2(-1.f, -1.f);
  const uint64_t c3 = ptx::pack_f32x2(0.05517167f, 0.05517167f);
  const uint64_t c2 = ptx::pack_f32x2(0.24261113f, 0.24261113f);
  const uint64_t c1 = ptx::pack_f32x2(0.69326097f, 0.69326097f);
  const uint64_t c0 = ptx::pack_f32x2(0.99992806f, 0.99992806f);
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    float p0, p1;
    if (((i % 8) * kPoly) % 8 < kPoly) {
      const uint64_t y2 = ptx::pack_f32x2(ptx::fma_sat(v[2 * i], pa, pb), ptx::fma_sat(v[2 * i + 1], pa, pb));
      const uint64_t r2 = ptx::fma_f32x2(y2, k128, kmag);         // x + 1.5 * 2^23: the integer n sits in the low bits
      const uint64_t f2 = ptx::fma_f32x2(y2, k128, ptx::fma_f32x2(r2, kneg, kmag));   // x - n
      uint64_t q2 = ptx::fma_f32x2(f2, c3, c2);
      q2 = ptx::fma_f32x2(q2, f2, c1);
      q2 = ptx::fma_f32x2(q2, f2, c0);
      float r0, r1, q0, q1;
      ptx::unpack_f32x2(r2, r0, r1);
      ptx::unpack_f32x2(q2, q0, q1);
      p0 = __uint_as_float(__float_as_uint(q0) + (__float_as_uint(r0) << 23));
      p1 = __uint_as_float(__float_as_uint(q1) + (__float_as_uint(r1) << 23));
    } else {
      const uint64_t x2 = ptx::fma_f32x2(ptx::pack_f32x2(v[2 * i], v[2 * i + 1]), scale2, nref2);
      float x0, x1;
      ptx::unpack_f32x2(x2, x0, x1);
      p0 = ptx::ex2(x0);
      p1 = ptx::ex2(x1);
    }
    const uint64_t p2 = ptx::pack_f32x2(p0, p1);
    if (i & 1) sum2b = ptx::add_f32x2(sum2b, p2); else sum2a = ptx::add_f32x2(sum2a, p2);
    pk[i] = pack2<kBF16>(p0, p1);
  }
}

template <bool kBF16>
__global__ void __launch_bounds__(kThreads, 1) sparse_attn_fwd_d64_kernel(
    const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
    const __grid_constant__ CUtensorMap tm_v, const int32_t* __restrict__ counts,
    const int32_t* __restrict__ entries, const int32_t* __restrict__ order, int Hm, int ntk, int N, float scale_log2,
    int q_split, int kvl_lo, int kvl_hi, void* __restrict__ out_raw, float* __restrict__ lse,
    int32_t* __restrict__ status, const __grid_constant__ OutScatter scatter) {
  constexpr int D = 64;
  constexpr int kTileBytes = kTile * D * 2;       // one Q, K or V tile: 128 rows x 128 bytes
  constexpr uint32_t kIdescQK = ptx::idesc_f16(128, 128, kBF16, false);
  constexpr uint32_t kIdescPV = ptx::idesc_f16(128, D, kBF16, true);

  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Control64* ctl = reinterpret_cast<Control64*>(smem + (2 + 2 * kStages64) * kTileBytes);
  const uint32_t sQ = ptx::smem_u32(smem);
  const uint32_t sK = sQ + 2 * kTileBytes;
  const uint32_t sV = sK + kStages64 * kTileBytes;
  const uint32_t bar0 = ptx::smem_u32(&ctl->bars[0]);
  auto bar = [&](int i) { return bar0 + 8u * static_cast<uint32_t>(i); };
  volatile int* abort_flag = &ctl->abort_flag;

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  const int npairs = static_cast<int>(gridDim.x) / Hm;
  const int item = order ? order[blockIdx.x] : static_cast<int>(blockIdx.x);
  const int mh = item / npairs;
  const int pair = item - mh * npairs;
  const int bh = blockIdx.y * Hm + mh;
  const int ntq = (N + kTile - 1) / kTile;
  const bool has_b = (2 * pair + 1) < ntq;
  const int cnt = counts[static_cast<int64_t>(mh) * npairs + pair];
  const int32_t* ent = entries + (static_cast<int64_t>(mh) * npairs + pair) * ntk;

  if (threadIdx.x == 0) {
    for (int i = 0; i < k6NumBarriers; ++i) {
      uint32_t c = 1;
      if (i >= k6SFreeA && i <= k6PHiB) c = 128;
      ptx::mbar_init(bar(i), c);
    }
    ctl->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&tm_q);
    ptx::prefetch_tensormap(&tm_k);
    ptx::prefetch_tensormap(&tm_v);
  }
  if (warp == 2) {
    ptx::tmem_alloc(ptx::smem_u32(&ctl->tmem_base), 512);
    ptx::tmem_relinquish();
    ptx::tc_fence_before();
  }
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;

  // Slot j's completion shows on k6Done_X[j % kStages64].  "Slot -1" is the Q K^T of entry 0, issued before the loop:
  // it shares the last index, whose phases are therefore one ahead of the others'.
  auto done_index = [](int j) -> int { return (j + kStages64) % kStages64; };
  auto done_parity = [](int j) -> uint32_t {
    return static_cast<uint32_t>((((j + kStages64) % kStages64 == kStages64 - 1) ? (j + 1) / kStages64 : j / kStages64) & 1);
  };

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (warp == 0) {
      // ------------------------------------------------------------------ TMA producer
      if (lane == 0) {
        ptx::mbar_expect_tx(bar(k6QFull), (has_b ? 2u : 1u) * kTileBytes);
        for (int x = 0; x < (has_b ? 2 : 1); ++x)
          ptx::tma_load_3d(sQ + x * kTileBytes, &tm_q, bar(k6QFull), 0, (2 * pair + x) * kTile, bh);
        bool ok = true;
        int issued = 0;
        if (cnt > 0) {
          ptx::mbar_expect_tx(bar(k6KFirst), kTileBytes);
          ptx::tma_load_3d(sK, &tm_k, bar(k6KFirst), 0, (ent[0] >> 8) * kTile, bh);
        }
        // entry e: V(e) into V stage e % kStages64 and K(e + 1) into K stage (e + 1) % kStages64, once slot
        // e - kStages64 has completed in both tiles (it read both stages last)
        for (int e = 0; e < cnt && ok; ++e) {
          const int s = e % kStages64;
          const bool next = (e + 1) < cnt;
          if (e >= kStages64 - 1) {
            const int j = e - kStages64;
            ok = ptx::mbar_wait(bar(k6DoneA0 + done_index(j)), done_parity(j), abort_flag) &&
                 ptx::mbar_wait(bar(k6DoneB0 + done_index(j)), done_parity(j), abort_flag);
            if (!ok) { report(status, 1, 0, e); break; }
          }
          ptx::mbar_expect_tx(bar(k6Full0 + s), (next ? 2u : 1u) * kTileBytes);
          ptx::tma_load_3d(sV + s * kTileBytes, &tm_v, bar(k6Full0 + s), 0, (ent[e] >> 8) * kTile, bh);
          if (next)
            ptx::tma_load_3d(sK + ((e + 1) % kStages64) * kTileBytes, &tm_k, bar(k6Full0 + s), 0, (ent[e + 1] >> 8) * kTile,
                             bh);
          issued = e + 1;
        }
        if (!ok) {
          // give copies in flight a bounded time to land (their barriers may never be consumed)
          for (int i = 0; i < 4096 && cnt > 0 && !ptx::mbar_try_wait(bar(k6KFirst), 0); ++i) {}
          for (int e = max(0, issued - kStages64); e < issued; ++e)
            for (int i = 0; i < 4096 && !ptx::mbar_try_wait(bar(k6Full0 + e % kStages64), (e / kStages64) & 1); ++i) {}
        }
      }
    } else if (warp == 1 || warp == 3) {
      // ------------------------------------------------------------------ MMA issuers, one per query tile
      if (lane == 0) {
        const int x = warp >> 1;
        const uint64_t dqx = ptx::smem_desc_sw128(sQ + x * kTileBytes, 16, 1024);
        const uint64_t dk0 = ptx::smem_desc_sw128(sK, 16, 1024);
        const uint64_t dv0 = ptx::smem_desc_sw128(sV, kTileBytes, 1024);
        const uint32_t tSx = tmem + x * 128, tOx = tmem + 256 + x * D, tPx = tmem + 384 + x * 64;
        auto advance = [](uint64_t desc, uint32_t bytes) -> uint64_t {
          return (desc & 0xffffffff00000000ull) | static_cast<uint32_t>(static_cast<uint32_t>(desc) + (bytes >> 4));
        };
        auto issue_qk = [&](int s) {          // s: K stage
          const uint64_t b0 = advance(dk0, static_cast<uint32_t>(s) * kTileBytes);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk)
            ptx::mma_ss(tSx, advance(dqx, kk * 32), advance(b0, kk * 32), kIdescQK, kk > 0 ? 1u : 0u);
          ptx::tc_commit(bar(k6SFullA + x));
        };
        auto issue_pv_half = [&](int s, int half, uint32_t acc) {   // s: V stage
          const uint64_t b0 = advance(dv0, static_cast<uint32_t>(s) * kTileBytes);
#pragma unroll
          for (int kq = 0; kq < 4; ++kq) {
            const int kk = half * 4 + kq;
            ptx::mma_ts(tOx, tPx + kk * 8, advance(b0, kk * 2048), kIdescPV, (acc || kq > 0) ? 1u : 0u);
          }
        };
        bool ok = ptx::mbar_wait(bar(k6QFull), 0, abort_flag);
        if (!ok) report(status, 2, 1 + x, -1);
        // flags of entry e, e + 1 and e + 2: each is loaded two slots before the issuer needs it (a load issued
        // where its value is used would put a trip to the L2 on the issuing thread's path every slot)
        int sub = (cnt > 0) ? ((ent[0] >> (4 * x)) & 0xf) : 0;
        int subn = (cnt > 1) ? ((ent[1] >> (4 * x)) & 0xf) : 0;
        int n_qk = 0;                       // Q K^T products issued so far for this tile
        if (ok && cnt > 0) {
          ok = ptx::mbar_wait(bar(k6KFirst), 0, abort_flag);
          if (!ok) report(status, 2, 1 + x, 0);
          if (ok) {
            ptx::tc_fence_after();
            if (sub) { issue_qk(0); ++n_qk; }
            ptx::tc_commit(bar(k6DoneA0 + kStages64 * x + kStages64 - 1));   // "slot -1": K stage 0 is free again
          }
        }
        uint32_t par_p = 0, acc = 0;
        for (int e = 0; e < cnt && ok; ++e) {
          const int s = e % kStages64;
          const int subnn = (e + 2 < cnt) ? ((ent[e + 2] >> (4 * x)) & 0xf) : 0;   // first used in the next slot
          ok = ptx::mbar_wait(bar(k6Full0 + s), (e / kStages64) & 1, abort_flag);
          if (!ok) { report(status, 2, 1 + x, e); break; }
          if (subn) {
            // S_x is free once the softmax has read the scores of the tile's previous entry
            if (n_qk > 0) {
              ok = ptx::mbar_wait(bar(k6SFreeA + x), static_cast<uint32_t>((n_qk - 1) & 1), abort_flag);
              if (!ok) { report(status, 6, 1 + x, e); break; }
            }
            ptx::tc_fence_after();
            issue_qk((e + 1) % kStages64);
            ++n_qk;
          }
          if (sub) {
            ok = ptx::mbar_wait(bar(k6PLoA + 2 * x), par_p, abort_flag);
            if (!ok) { report(status, 3, 1 + x, e); break; }
            ptx::tc_fence_after();
            issue_pv_half(s, 0, acc);
            ok = ptx::mbar_wait(bar(k6PHiA + 2 * x), par_p, abort_flag);
            if (!ok) { report(status, 3, 1 + x, e); break; }
            ptx::tc_fence_after();
            issue_pv_half(s, 1, 1u);
            par_p ^= 1;
            acc = 1u;
          }
          ptx::tc_commit(bar(k6DoneA0 + kStages64 * x + s));  // this tile's MMAs of slot e are done
          sub = subn;
          subn = subnn;
        }
        ptx::tc_commit(bar(k6OFinalA + x));
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    // ------------------------------------------------------------------ softmax + epilogue
    const int x = (warp - 4) / 4;                 // 0: tile A, 1: tile B
    const int wq = warp % 4;                      // tensor-memory lane quarter of this warp
    const int r = wq * 32 + lane;                 // row inside the tile
    const int tile = 2 * pair + x;
    const int grow = tile * kTile + r;            // global query row
    const int kvl = (grow < q_split) ? kvl_lo : kvl_hi;
    const int kvl_min = min(kvl_lo, kvl_hi);
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
    const uint32_t tS = tmem + lane_base + x * 128;
    const uint32_t tO = tmem + lane_base + 256 + x * D;
    const uint32_t tP = tmem + lane_base + 384 + x * 64;
    const int rh = r >> 6;                        // row half of the tile: the same for the whole warp

    float m = -INFINITY, l = 0.f;
    uint32_t par_s = 0;
    int done = 0;
    bool ok = true;
    int en_next = (cnt > 0) ? ent[0] : 0;
    for (int e = 0; e < cnt; ++e) {
      const int en = en_next;
      en_next = (e + 1 < cnt) ? ent[e + 1] : 0;   // in flight while this entry is processed
      const int sub = (en >> (4 * x)) & 0xf;
      if (!sub) continue;
      const int col0 = (en >> 8) * kTile;
      ok = ptx::mbar_wait(bar(k6SFullA + x), par_s, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { if (lane == 0) report(status, 4, 2 + x, e); break; }
      par_s ^= 1;
      ptx::tc_fence_after();
      // per 64-key half (flags are the same for every thread of the warp): keep = the rows of this warp keep it
      const bool keep[2] = {((sub >> (2 * rh)) & 1) != 0, ((sub >> (2 * rh + 1)) & 1) != 0};
      const bool edge = col0 + kTile > kvl_min;   // the tile reaches past the valid keys of some row
      float v[kTile];
#pragma unroll
      for (int half = 0; half < 2; ++half)
        if (keep[half]) {
          ptx::tmem_ld32(tS + half * 64, reinterpret_cast<uint32_t*>(v) + half * 64);
          ptx::tmem_ld32(tS + half * 64 + 32, reinterpret_cast<uint32_t*>(v) + half * 64 + 32);
        }
      ptx::tmem_ld_wait();
      ptx::tc_fence_before();
      ptx::mbar_arrive(bar(k6SFreeA + x));        // the next Q K^T of this tile may overwrite S
      if (edge) {
        const int lim = kvl - col0;               // columns >= lim are beyond the valid keys of this row
#pragma unroll
        for (int c = 0; c < kTile; ++c)
          if (keep[c / 64]) v[c] = (c < lim) ? v[c] : -INFINITY;
      }
      float mx = -INFINITY;
#pragma unroll
      for (int half = 0; half < 2; ++half)
        if (keep[half]) mx = fmaxf(mx, row_max64(v + half * 64));
      const float m_new = fmaxf(m, mx * scale_log2);
      // this tile's products of the previous slot have completed: P_x may be overwritten and O_x may be rescaled
      if (e > 0) {
        ok = ptx::mbar_wait(bar(k6DoneA0 + kStages64 * x + done_index(e - 1)), done_parity(e - 1), abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { if (lane == 0) report(status, 7, 2 + x, e); break; }
        ptx::tc_fence_after();
      }
      if (done == 0) {
        m = m_new;
      } else if (__any_sync(0xffffffffu, m_new > m + kRescaleThreshold)) {
        const float alpha = (m == -INFINITY) ? 0.f : ptx::ex2(m - m_new);
        l *= alpha;
        m = m_new;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          float o[32];
          ptx::tmem_ld32(tO + c * 32, reinterpret_cast<uint32_t*>(o));
          ptx::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] *= alpha;
          ptx::tmem_st32(tO + c * 32, reinterpret_cast<const uint32_t*>(o));
        }
      }
      const float ref = (m == -INFINITY) ? 0.f : m;
      uint64_t sum2a = 0, sum2b = 0;    // bit pattern of (0.f, 0.f)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t pk[32];
        if (keep[half]) {
          if (edge) exp_half<kBF16, 0>(v + half * 64, scale_log2, ref, pk, sum2a, sum2b);   // may hold -inf: exact zeros
          else exp_half<kBF16, kPolyPairs64>(v + half * 64, scale_log2, ref, pk, sum2a, sum2b);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) pk[i] = 0u;   // a half this row half does not keep: no exponentials at all
        }
        ptx::tmem_st32(tP + half * 32, pk);
        ptx::tmem_st_wait();
        ptx::tc_fence_before();
        ptx::mbar_arrive(bar(k6PLoA + 2 * x + half));
      }
      float s0, s1, s2, s3;
      ptx::unpack_f32x2(sum2a, s0, s1);
      ptx::unpack_f32x2(sum2b, s2, s3);
      l += (s0 + s1) + (s2 + s3);
      ++done;
    }

    if (ok) {
      ok = ptx::mbar_wait(bar(k6OFinalA + x), 0, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok && lane == 0) report(status, 5, 2 + x, -1);
    }
    if (ok && tile < ntq) {
      ptx::tc_fence_after();
      const float inv = (done > 0 && l > 0.f) ? 1.f / l : 0.f;
      uint4* dst;
      if (scatter.n_peers > 0) {
        const int pr = min(grow / scatter.rows_per_peer, scatter.n_peers - 1);
        dst = reinterpret_cast<uint4*>(
            static_cast<unsigned char*>(scatter.peer[pr]) +
            (static_cast<int64_t>(scatter.head_base + bh) * scatter.rows_per_peer + (grow - pr * scatter.rows_per_peer)) * D * 2);
      } else {
        dst = reinterpret_cast<uint4*>(static_cast<unsigned char*>(out_raw) + (static_cast<int64_t>(bh) * N + grow) * D * 2);
      }
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        float o[32];
        if (done > 0) {
          ptx::tmem_ld32(tO + c * 32, reinterpret_cast<uint32_t*>(o));
          ptx::tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0.f;
        }
        if (grow < N) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 w;
            w.x = pack2<kBF16>(o[q4 * 8 + 0] * inv, o[q4 * 8 + 1] * inv);
            w.y = pack2<kBF16>(o[q4 * 8 + 2] * inv, o[q4 * 8 + 3] * inv);
            w.z = pack2<kBF16>(o[q4 * 8 + 4] * inv, o[q4 * 8 + 5] * inv);
            w.w = pack2<kBF16>(o[q4 * 8 + 6] * inv, o[q4 * 8 + 7] * inv);
            dst[c * 4 + q4] = w;
          }
        }
      }
      if (lse != nullptr && grow < N) {
        lse[static_cast<int64_t>(bh) * N + grow] =
            (done > 0 && l > 0.f) ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
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

template <bool kBF16>
int launch_d64(const void* q, const void* k, const void* v, int dtype, int BH, int N, const int32_t* counts,
               const int32_t* entries, const int32_t* order, int Hm, float softmax_scale, int q_split, int kvl_lo,
               int kvl_hi, void* out, float* lse, int32_t* status, const OutScatter& scatter, cudaStream_t st) {
  CUtensorMap tq, tk, tv;
  if (int rc = make_tmap_rows(&tq, q, dtype, BH, N, 64, kTile)) return rc;
  if (int rc = make_tmap_rows(&tk, k, dtype, BH, N, 64, kTile)) return rc;
  if (int rc = make_tmap_rows(&tv, v, dtype, BH, N, 64, kTile)) return rc;
  const int ntq = ceil_div(N, kTile);
  const int npairs = (ntq + 1) / 2;
  auto kernel = sparse_attn_fwd_d64_kernel<kBF16>;
  const size_t smem = smem_bytes_d64();
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem)) return rc;
  const float scale_log2 = softmax_scale * 1.4426950408889634f;
  kernel<<<dim3(npairs * Hm, BH / Hm), kThreads, smem, st>>>(tq, tk, tv, counts, entries, order, Hm, ntq, N, scale_log2,
                                                            q_split, kvl_lo, kvl_hi, out, lse, status, scatter);
  MODDIT_CHECK_LAUNCH("sparse_attn_fwd_d64_kernel");
  return MODDIT_OK;
}

template <int D, bool kBF16>
int launch(const void* q, const void* k, const void* v, int dtype, int BH, int N, const int32_t* counts,
           const int32_t* entries, const int32_t* order, int Hm, float softmax_scale, int q_split, int kvl_lo, int kvl_hi, void* out,
           float* lse, int32_t* status, const OutScatter& scatter, cudaStream_t st) {
  CUtensorMap tq, tk, tv;
  if (int rc = make_tmap_rows(&tq, q, dtype, BH, N, D, kTile)) return rc;
  if (int rc = make_tmap_rows(&tk, k, dtype, BH, N, D, kTile)) return rc;
  if (int rc = make_tmap_rows(&tv, v, dtype, BH, N, D, kTile)) return rc;
  const int ntq = ceil_div(N, kTile);
  const int npairs = (ntq + 1) / 2;
  auto kernel = sparse_attn_fwd_kernel<D, kBF16>;
  const size_t smem = smem_bytes<D>();
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem)) return rc;
  const float scale_log2 = softmax_scale * 1.4426950408889634f;
  kernel<<<dim3(npairs * Hm, BH / Hm), kThreads, smem, st>>>(tq, tk, tv, counts, entries, order, Hm, ntq, N, scale_log2, q_split,
                                                   kvl_lo, kvl_hi, out, lse, status, scatter);
  MODDIT_CHECK_LAUNCH("sparse_attn_fwd_kernel");
  return MODDIT_OK;
}

}  // namespace
}  // namespace moddit

using namespace moddit;

static int sparse_attn_dispatch(const void* q, const void* k, const void* v, int dtype, int BH, int N, int D,
                                const int32_t* counts, const int32_t* entries, const int32_t* order, int Hm,
                                float softmax_scale, int q_split, int kv_len_lo, int kv_len_hi, void* out, float* lse,
                                int32_t* status, const OutScatter& scatter, void* stream) {
  MODDIT_CHECK_ARG(q && k && v && counts && entries && status, "sparse_attn_fwd: null pointer");
  MODDIT_CHECK_ARG(out || scatter.n_peers > 0, "sparse_attn_fwd: no output destination");
  MODDIT_CHECK_ARG(BH > 0 && BH <= 65535 && N > 0 && Hm > 0, "sparse_attn_fwd: BH=%d N=%d Hm=%d out of range", BH, N, Hm);
  MODDIT_CHECK_ARG(BH % Hm == 0, "sparse_attn_fwd: BH=%d is not a multiple of the mask heads Hm=%d", BH, Hm);
  MODDIT_CHECK_ARG(softmax_scale > 0.f, "sparse_attn_fwd: softmax_scale must be positive");
  MODDIT_CHECK_ARG(kv_len_lo >= 0 && kv_len_lo <= N && kv_len_hi >= 0 && kv_len_hi <= N,
                   "sparse_attn_fwd: kv_len (%d, %d) outside [0, N=%d]", kv_len_lo, kv_len_hi, N);
  if (D != 64 && D != 128) return fail(MODDIT_E_UNSUPPORTED, "sparse_attn_fwd: head_dim must be 64 or 128, got %d", D);
  if (dtype != MODDIT_BF16 && dtype != MODDIT_FP16) return fail(MODDIT_E_ARG, "sparse_attn_fwd: unknown dtype %d", dtype);
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out))
    return fail(MODDIT_E_ALIGN, "sparse_attn_fwd: q, k, v and out must be 16-byte aligned");
  if (int rc = require_sm100()) return rc;
  cudaStream_t st = as_stream(stream);
  if (D == 128) {
    return dtype == MODDIT_BF16
               ? launch<128, true>(q, k, v, dtype, BH, N, counts, entries, order, Hm, softmax_scale, q_split, kv_len_lo,
                                   kv_len_hi, out, lse, status, scatter, st)
               : launch<128, false>(q, k, v, dtype, BH, N, counts, entries, order, Hm, softmax_scale, q_split, kv_len_lo,
                                    kv_len_hi, out, lse, status, scatter, st);
  }
#ifdef MODDIT_D64_SHARED_KERNEL
  return dtype == MODDIT_BF16 ? launch<64, true>(q, k, v, dtype, BH, N, counts, entries, order, Hm, softmax_scale, q_split,
                                                 kv_len_lo, kv_len_hi, out, lse, status, scatter, st)
                              : launch<64, false>(q, k, v, dtype, BH, N, counts, entries, order, Hm, softmax_scale, q_split,
                                                  kv_len_lo, kv_len_hi, out, lse, status, scatter, st);
#else
  return dtype == MODDIT_BF16 ? launch_d64<true>(q, k, v, dtype, BH, N, counts, entries, order, Hm, softmax_scale, q_split,
                                                 kv_len_lo, kv_len_hi, out, lse, status, scatter, st)
                              : launch_d64<false>(q, k, v, dtype, BH, N, counts, entries, order, Hm, softmax_scale, q_split,
                                                  kv_len_lo, kv_len_hi, out, lse, status, scatter, st);
#endif
}

extern "C" int moddit_sparse_attn_fwd(const void* q, const void* k, const void* v, int dtype, int BH, int N, int D,
                                      const int32_t* counts, const int32_t* entries, const int32_t* order, int Hm,
                                      float softmax_scale, int q_split, int kv_len_lo, int kv_len_hi, void* out,
                                      float* lse, int32_t* status, void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(out, "sparse_attn_fwd: null output pointer");
  OutScatter none = {};
  return sparse_attn_dispatch(q, k, v, dtype, BH, N, D, counts, entries, order, Hm, softmax_scale, q_split, kv_len_lo,
                              kv_len_hi, out, lse, status, none, stream);
}

extern "C" int moddit_sparse_attn_fwd_scatter(const void* q, const void* k, const void* v, int dtype, int BH, int N,
                                              int D, const int32_t* counts, const int32_t* entries,
                                              const int32_t* order, int Hm, float softmax_scale, int q_split,
                                              int kv_len_lo, int kv_len_hi, void* const* peer_out, int n_peers,
                                              int head_base, float* lse, int32_t* status, void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(peer_out, "sparse_attn_fwd_scatter: null peer table");
  MODDIT_CHECK_ARG(n_peers >= 1 && n_peers <= kMaxPeers, "sparse_attn_fwd_scatter: n_peers=%d outside [1, %d]", n_peers,
                   kMaxPeers);
  MODDIT_CHECK_ARG(N % n_peers == 0, "sparse_attn_fwd_scatter: N=%d does not divide over %d peers", N, n_peers);
  MODDIT_CHECK_ARG(head_base >= 0, "sparse_attn_fwd_scatter: head_base must be non-negative");
  OutScatter sc = {};
  for (int i = 0; i < n_peers; ++i) {
    MODDIT_CHECK_ARG(peer_out[i] && aligned16(peer_out[i]), "sparse_attn_fwd_scatter: peer buffer %d null or unaligned", i);
    sc.peer[i] = peer_out[i];
  }
  sc.n_peers = n_peers;
  sc.rows_per_peer = N / n_peers;
  sc.head_base = head_base;
  return sparse_attn_dispatch(q, k, v, dtype, BH, N, D, counts, entries, order, Hm, softmax_scale, q_split, kv_len_lo,
                              kv_len_hi, nullptr, lse, status, sc, stream);
}
