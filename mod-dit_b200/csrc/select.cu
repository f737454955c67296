// Line selection, mask generation, cumulative-mass selection and the work lists of the sparse forward.
// All integer / byte work on small arrays: each kernel is one pass with coalesced reads and writes.
#include <cuda_fp16.h>

#include "common.cuh"

namespace moddit {
namespace {

// Monotone map float -> uint32 (ascending); -0 and +0 coincide, NaN sorts last.
__device__ __forceinline__ uint32_t order_key(float f) {
  if (f != f) return 0xffffffffu;
  if (f == 0.f) f = 0.f;
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Synchronisation after one compare-exchange stage of a shared-memory bitonic sort in which thread t handles the
// pairs t, t + blockDim, ...: with stride <= 32 the 32 pairs of a warp lie inside one aligned run of 64 elements that
// no other warp touches, so a stage only needs a block-wide barrier if it, or the stage after it, reaches further.
__device__ __forceinline__ void bitonic_stage_sync(int stride, int size, int P) {
  const int next = (stride > 1) ? (stride >> 1) : ((size < P) ? size : 0);
  if (stride > 32 || next > 32) __syncthreads();
  else __syncwarp();
}

constexpr int kSelectThreads = 1024;

// One CTA per head: the L = 3n - 1 extrapolated line intensities become 64-bit keys (value order << 32 | index),
// padded to a power of two P with all-ones keys, and are bitonic-sorted ascending in shared memory; the first k
// of the order are the selection (smallest value first, equal values lowest index first - the same total order
// as ranking every element against every other, at L log^2 L instead of L^2 compares).
__global__ void __launch_bounds__(kSelectThreads) select_lines_kernel(
    const float* __restrict__ cur_c, const float* __restrict__ cur_d, const float* __restrict__ last_c,
    const float* __restrict__ last_d, int n, int k, int P, float predict_T, int64_t* __restrict__ selected) {
  extern __shared__ __align__(8) unsigned long long sort_keys[];
  const int h = blockIdx.x;
  const int nd = 2 * n - 1;
  const int L = n + nd;
  for (int i = threadIdx.x; i < P; i += kSelectThreads) {
    if (i >= L) {
      sort_keys[i] = ~0ull;
      continue;
    }
    float cur, last;
    if (i < n) {
      cur = cur_c[static_cast<int64_t>(h) * n + i];
      last = last_c[static_cast<int64_t>(h) * n + i];
    } else {
      cur = cur_d[static_cast<int64_t>(h) * nd + (i - n)];
      last = last_d[static_cast<int64_t>(h) * nd + (i - n)];
    }
    // cur + (cur - last) / predict_T with IEEE operations in this order (no contraction)
    const float pred = __fadd_rn(cur, __fdiv_rn(__fsub_rn(cur, last), predict_T));
    sort_keys[i] = (static_cast<unsigned long long>(order_key(pred)) << 32) | static_cast<uint32_t>(i);
  }
  __syncthreads();
  for (int size = 2; size <= P; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = threadIdx.x; t < P / 2; t += kSelectThreads) {
        const int lo = 2 * t - (t & (stride - 1));
        const int hi = lo + stride;
        const bool up = ((lo & size) == 0);
        const unsigned long long a = sort_keys[lo], b = sort_keys[hi];
        if ((a > b) == up) {
          sort_keys[lo] = b;
          sort_keys[hi] = a;
        }
      }
      bitonic_stage_sync(stride, size, P);
    }
  }
  __syncthreads();
  for (int r = threadIdx.x; r < k; r += kSelectThreads)
    selected[static_cast<int64_t>(h) * k + r] = static_cast<int64_t>(static_cast<uint32_t>(sort_keys[r]));
}

__global__ void head_modes_kernel(const float* __restrict__ b_d, int H, float threshold, int32_t* __restrict__ modes) {
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h < H) modes[h] = (b_d[h] <= threshold) ? MODDIT_MODE_BLOCK_DIAGONAL : MODDIT_MODE_SPARSE;
}

constexpr int kMaskRows = 32;
constexpr int kMaskThreads = 256;

// One CTA per (32 mask rows, head), a warp per row.  Shared memory holds two bit arrays: one bit per mask column
// ("selected column", and every column outside the video region, which is always kept) and one bit per diagonal
// offset, the latter padded with zero bits on both sides so that a row may read 32 bits starting anywhere.  For a
// row, lane l builds the keep bits of columns [32 l, 32 l + 32) of a 1024-column segment with a handful of word
// operations - column word | diagonal bits funnel-shifted to the row's offset | the row's own frame as a bit range -
// and the warp then writes the segment 128 bytes per instruction, every lane expanding four bits it fetches from
// the lane that holds them.  (One byte decided and stored per thread and step made this kernel instruction-bound.)
__device__ __forceinline__ uint32_t low_bits(int x) { return x >= 32 ? 0xffffffffu : ((1u << x) - 1u); }

__global__ void __launch_bounds__(kMaskThreads) mask_from_lines_kernel(
    const int64_t* __restrict__ selected, int k, const int32_t* __restrict__ modes, int n, int bpf, int voff, int nbt,
    int pad_bits, int col_words, int diag_words, uint8_t* __restrict__ mask) {
  extern __shared__ __align__(4) uint32_t bits_s[];
  uint32_t* colw = bits_s;                 // [col_words]  bit C
  uint32_t* dw = bits_s + col_words;       // [diag_words] bit pad_bits + (column - row + n - 1)
  const int h = blockIdx.y;
  const int mode = modes[h];
  const bool frames_on = (mode == MODDIT_MODE_BLOCK_DIAGONAL);
  const bool all = (mode == MODDIT_MODE_FULL);
  for (int w = threadIdx.x; w < col_words; w += kMaskThreads) {
    // columns outside [voff, voff + n) are text (or padding of the word): always kept
    const int c0 = 32 * w;
    const int a = min(max(voff - c0, 0), 32), b = min(max(voff + n - c0, 0), 32);
    colw[w] = ~(low_bits(b) & ~low_bits(a));
  }
  for (int w = threadIdx.x; w < diag_words; w += kMaskThreads) dw[w] = 0u;
  __syncthreads();
  for (int t = threadIdx.x; t < k; t += kMaskThreads) {
    const int64_t idx = selected[static_cast<int64_t>(h) * k + t];   // [0,n): column; n + (offset + n - 1): diagonal
    if (idx >= 0 && idx < n) {
      const int c = static_cast<int>(idx) + voff;
      atomicOr(&colw[c >> 5], 1u << (c & 31));
    } else if (idx >= n && idx < 3 * n - 1) {
      const int d = static_cast<int>(idx) - n + pad_bits;
      atomicOr(&dw[d >> 5], 1u << (d & 31));
    }
  }
  __syncthreads();
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  for (int rr = warp; rr < kMaskRows; rr += kMaskThreads / 32) {
    const int R = blockIdx.x * kMaskRows + rr;
    if (R >= nbt) break;
    const int i = R - voff;
    uint8_t* dst = mask + (static_cast<int64_t>(h) * nbt + R) * nbt;
    const bool whole_row = all || i < 0 || i >= n;              // text rows and 'full' heads keep everything
    int f_lo = 0, f_hi = 0;                                     // the row's own frame as a column range
    if (frames_on && !whole_row) {
      f_lo = voff + (i / bpf) * bpf;
      f_hi = min(f_lo + bpf, voff + n);
    }
    for (int seg = 0; seg < nbt; seg += 1024) {
      const int c0 = seg + 32 * lane;
      uint32_t word = 0xffffffffu;
      if (!whole_row && c0 < nbt) {
        const int b = c0 - R + n - 1 + pad_bits;                // >= 0: pad_bits >= voff
        word = colw[c0 >> 5] | __funnelshift_r(dw[b >> 5], dw[(b >> 5) + 1], b & 31);
        const int fa = min(max(f_lo - c0, 0), 32), fb = min(max(f_hi - c0, 0), 32);
        word |= low_bits(fb) & ~low_bits(fa);
      }
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const uint32_t wv = __shfl_sync(0xffffffffu, word, 4 * r + (lane >> 3));
        const int C = seg + 128 * r + 4 * lane;
        if (C >= nbt) continue;
        const uint32_t x = (wv >> ((lane & 7) * 4)) & 0xfu;
        const uint32_t bytes = (x & 1u) | ((x & 2u) << 7) | ((x & 4u) << 14) | ((x & 8u) << 21);
        uint8_t* p = dst + C;
        const uintptr_t addr = reinterpret_cast<uintptr_t>(p);
        if (C + 3 < nbt && (addr & 3) == 0) {
          *reinterpret_cast<uint32_t*>(p) = bytes;
        } else if (C + 3 < nbt && (addr & 1) == 0) {
          *reinterpret_cast<uint16_t*>(p) = static_cast<uint16_t>(bytes);
          *reinterpret_cast<uint16_t*>(p + 2) = static_cast<uint16_t>(bytes >> 16);
        } else {
          for (int q = 0; q < 4 && C + q < nbt; ++q) p[q] = static_cast<uint8_t>(bytes >> (8 * q));
        }
      }
    }
  }
}

// ---- cumulative-mass selection ------------------------------------------------------------------
constexpr int kMassBits = 24;
constexpr int kMassThreads = 512;

// One CTA per (query block, head).  Keys ((2^24 - w) << 32 | j) are bitonic-sorted ascending, i.e.
// by brightness descending then index ascending; integer prefix sums decide the kept prefix.
// With topk_count > 0 the kept prefix is the first topk_count blocks of that order instead (no forced diagonal);
// row_full[h,i] != 0 keeps the whole row i, col_keep[h,j] != 0 keeps column j in every row (either may be null).
__global__ void __launch_bounds__(kMassThreads) select_mass_kernel(const __half* __restrict__ map, int n, int P,
                                                                   uint32_t tau_fixed, int topk_count,
                                                                   const uint8_t* __restrict__ row_full,
                                                                   const uint8_t* __restrict__ col_keep,
                                                                   uint8_t* __restrict__ keep) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned long long* key = reinterpret_cast<unsigned long long*>(smem_raw);   // [P]
  unsigned long long* pre = key + P;                                           // [P] inclusive prefix of w
  __shared__ unsigned long long carry[kMassThreads];
  const int i = blockIdx.x, h = blockIdx.y;
  const __half* row = map + (static_cast<int64_t>(h) * n + i) * n;
  for (int j = threadIdx.x; j < P; j += kMassThreads) {
    if (j < n) {
      float b = 1.0f - __half2float(row[j]);
      b = fminf(fmaxf(b, 0.f), 1.f);
      const uint32_t w = static_cast<uint32_t>(floorf(b * 16777216.0f));       // exact: b is a multiple of 2^-24
      key[j] = (static_cast<unsigned long long>((1u << kMassBits) - w) << 32) | static_cast<uint32_t>(j);
    } else {
      key[j] = ~0ull;
    }
  }
  __syncthreads();
  for (int size = 2; size <= P; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = threadIdx.x; t < P / 2; t += kMassThreads) {
        const int lo = 2 * t - (t & (stride - 1));
        const int hi = lo + stride;
        const bool up = ((lo & size) == 0);
        const unsigned long long a = key[lo], b = key[hi];
        if ((a > b) == up) {
          key[lo] = b;
          key[hi] = a;
        }
      }
      bitonic_stage_sync(stride, size, P);
    }
  }
  __syncthreads();
  // inclusive prefix of w over the sorted order (padding has w = 2^24 - 0xffffffff wraps; mask it out)
  const int per = (P + kMassThreads - 1) / kMassThreads;
  const int beg = min(P, static_cast<int>(threadIdx.x) * per), end = min(P, beg + per);
  unsigned long long run = 0;
  for (int e = beg; e < end; ++e) {
    const unsigned long long kk = key[e];
    const unsigned long long w = (static_cast<uint32_t>(kk) < static_cast<uint32_t>(n) && kk != ~0ull)
                                     ? (1ull << kMassBits) - (kk >> 32)
                                     : 0ull;
    run += w;
    pre[e] = run;
  }
  carry[threadIdx.x] = run;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long acc = 0;
    for (int t = 0; t < kMassThreads; ++t) {
      const unsigned long long v = carry[t];
      carry[t] = acc;
      acc += v;
    }
  }
  __syncthreads();
  for (int e = beg; e < end; ++e) pre[e] += carry[threadIdx.x];
  __syncthreads();
  const unsigned long long total = pre[P - 1];
  const unsigned long long target = (static_cast<unsigned long long>(tau_fixed) * total + ((1ull << kMassBits) - 1)) >>
                                    kMassBits;
  uint8_t* dst = keep + (static_cast<int64_t>(h) * n + i) * n;
  for (int e = threadIdx.x; e < P; e += kMassThreads) {
    const unsigned long long kk = key[e];
    if (kk == ~0ull) continue;
    const int j = static_cast<int>(static_cast<uint32_t>(kk));
    const unsigned long long excl = (e == 0) ? 0ull : pre[e - 1];
    bool k = topk_count > 0 ? e < topk_count : (excl < target || j == i);
    if (row_full != nullptr && row_full[static_cast<int64_t>(h) * n + i] != 0) k = true;
    if (col_keep != nullptr && col_keep[static_cast<int64_t>(h) * n + j] != 0) k = true;
    dst[j] = k ? 1 : 0;
  }
}

// The same selection without sorting, one warp per (query block, head), for n <= 1024 (32 values per lane in
// registers).  In the sorted order (brightness descending, index ascending) the weight that precedes element e is
//   before(e) = sum of the weights greater than w_e  +  w_e * (equal weights with a lower index),
// and e is kept iff before(e) < target (or, in the count form, iff its rank - the same expression with ones
// instead of weights - is below the count).  The sum over greater weights only depends on the value, so a
// bisection over the 25-bit value range finds t* = the smallest value whose "sum of greater weights" is below the
// target: everything brighter than t* is kept, everything darker is not, and the elements equal to t* are kept in
// index order while the running sum stays below the target.  Bit-identical to the sort kernel.
constexpr int kMassWarpMax = 1024;
constexpr int kMassWarpThreads = 256;

__global__ void __launch_bounds__(kMassWarpThreads) select_mass_warp_kernel(
    const __half* __restrict__ map, int n, int rows_total, uint32_t tau_fixed, int topk_count,
    const uint8_t* __restrict__ row_full, const uint8_t* __restrict__ col_keep, uint8_t* __restrict__ keep) {
  const int lane = threadIdx.x % 32;
  const int rowid = blockIdx.x * (kMassWarpThreads / 32) + threadIdx.x / 32;      // h * n + i
  if (rowid >= rows_total) return;
  const int h = rowid / n, i = rowid - h * n;
  const __half* row = map + static_cast<int64_t>(rowid) * n;
  uint32_t w[32];
#pragma unroll
  for (int u = 0; u < 32; ++u) {
    const int j = lane + 32 * u;
    w[u] = 0xffffffffu;                                     // beyond the row: compares greater than nothing, never kept
    if (j < n) {
      float b = 1.0f - __half2float(row[j]);
      b = fminf(fmaxf(b, 0.f), 1.f);
      w[u] = static_cast<uint32_t>(floorf(b * 16777216.0f));                      // exact: b is a multiple of 2^-24
    }
  }
  const bool by_count = topk_count > 0;
  // amount(u): what element u adds to a sum (its weight, or one in the count form); 0 beyond the row
  auto greater_than = [&](uint32_t t) -> unsigned long long {
    uint32_t part = 0;                                      // at most 32 * 2^24 per lane
#pragma unroll
    for (int u = 0; u < 32; ++u) {
      const bool in = (w[u] != 0xffffffffu) && (w[u] > t);
      part += in ? (by_count ? 1u : w[u]) : 0u;
    }
    unsigned long long tot = part;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
    return tot;
  };
  unsigned long long target;
  if (by_count) {
    target = static_cast<unsigned long long>(topk_count);
  } else {
    uint32_t part = 0;
#pragma unroll
    for (int u = 0; u < 32; ++u) part += (w[u] != 0xffffffffu) ? w[u] : 0u;
    unsigned long long total = part;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
    target = (static_cast<unsigned long long>(tau_fixed) * total + ((1ull << kMassBits) - 1)) >> kMassBits;
  }
  // smallest t in [0, 2^24] with greater_than(t) < target; greater_than(2^24) = 0, so t = 2^24 qualifies unless
  // the target is 0 (then nothing is kept by the rule)
  uint32_t lo = 0, hi = 1u << kMassBits;
  if (target == 0) {
    lo = hi = 0xfffffffeu;                                  // no element reaches it: nothing kept by the rule
  } else {
    while (lo < hi) {
      const uint32_t mid = lo + ((hi - lo) >> 1);
      if (greater_than(mid) < target) hi = mid; else lo = mid + 1;
    }
  }
  const uint32_t tstar = lo;
  const unsigned long long above = (target == 0) ? 0ull : greater_than(tstar);
  const bool whole_row = row_full != nullptr && row_full[rowid] != 0;
  uint8_t* dst = keep + static_cast<int64_t>(rowid) * n;
  unsigned long long ties_before = 0;                       // elements equal to t* in earlier groups of 32
#pragma unroll
  for (int u = 0; u < 32; ++u) {
    const int j = lane + 32 * u;
    const bool tie = (w[u] == tstar);
    const unsigned bal = __ballot_sync(0xffffffffu, tie);
    if (j < n) {
      bool k = false;
      if (target != 0) {
        if (w[u] > tstar) {
          k = true;
        } else if (tie) {
          const unsigned long long prior = ties_before + __popc(bal & ((1u << lane) - 1));
          k = above + prior * (by_count ? 1ull : static_cast<unsigned long long>(tstar)) < target;
        }
      }
      if (!by_count && j == i) k = true;                    // the mass rule always keeps the diagonal block
      if (whole_row) k = true;
      if (col_keep != nullptr && col_keep[static_cast<int64_t>(h) * n + j] != 0) k = true;
      dst[j] = k ? 1 : 0;
    }
    ties_before += __popc(bal);
  }
}

// ---- work lists ---------------------------------------------------------------------------------
constexpr int kListThreads = 256;
constexpr int kListBatch = 4;

// One warp per (pair of 128-row query tiles, mask head): the warp walks the key tiles 32 at a time, a ballot
// marks the tiles some sub-block of the pair keeps, and every kept tile is written at its running position (the
// list stays in increasing key-tile order).  No shared memory, no block-wide synchronisation.
__global__ void __launch_bounds__(kListThreads) tile_lists_kernel(const uint8_t* __restrict__ mask, int nbq, int nbk,
                                                                  int sub, int ntq, int ntk, int kv_block_limit,
                                                                  int npairs, int32_t* __restrict__ counts,
                                                                  int32_t* __restrict__ entries) {
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int p = blockIdx.x * (kListThreads / 32) + warp, h = blockIdx.y;
  if (p >= npairs) return;
  const uint8_t* mh = mask + static_cast<int64_t>(h) * nbq * nbk;
  int32_t* out = entries + (static_cast<int64_t>(h) * npairs + p) * ntk;
  const int lim = min(nbk, kv_block_limit);
  int base = 0;
  // kListBatch steps of 32 key tiles at a time: all their mask bytes are requested before the first ballot, so the
  // warp waits for the memory system once per 128 key tiles instead of once per 32 (16 steps at a time measured
  // slower than 4: 0.083 against 0.060 ms at 24 heads x 902 tiles)
  for (int t0 = 0; t0 < ntk; t0 += 32 * kListBatch) {
    int fls[kListBatch];
#pragma unroll
    for (int u = 0; u < kListBatch; ++u) {
      const int t = t0 + 32 * u + lane;
      int fl = 0;
      if (t < ntk) {
        for (int x = 0; x < 2; ++x) {
          const int qt = 2 * p + x;
          if (qt >= ntq) continue;
          if (sub == 1) {               // block size 128: one mask block is the whole tile, all four flags at once
            const uint8_t m = (qt < nbq && t < lim) ? mh[static_cast<int64_t>(qt) * nbk + t] : uint8_t(0);
            fl |= m ? (0xf << (4 * x)) : 0;
            continue;
          }
          for (int rh = 0; rh < 2; ++rh)
            for (int ch = 0; ch < 2; ++ch) {
              const int bi = qt * 2 + rh, bj = t * 2 + ch;
              const uint8_t m = (bi < nbq && bj < lim) ? mh[static_cast<int64_t>(bi) * nbk + bj] : uint8_t(0);
              fl |= m ? (1 << (4 * x + 2 * rh + ch)) : 0;
            }
        }
      }
      fls[u] = fl;
    }
#pragma unroll
    for (int u = 0; u < kListBatch; ++u) {
      const int t = t0 + 32 * u + lane;
      const unsigned bal = __ballot_sync(0xffffffffu, fls[u] != 0);
      if (fls[u]) out[base + __popc(bal & ((1u << lane) - 1))] = (t << 8) | fls[u];
      base += __popc(bal);
    }
  }
  if (lane == 0) counts[static_cast<int64_t>(h) * npairs + p] = base;
}

// Start order of the (head, query-tile pair) work items of the sparse forward: order[pos] = head * npairs + pair.
// Pairs are ranked by list length inside their head (rank by counting; ties by index, so the result is
// deterministic).  The kLongFirst longest pairs of EVERY head come first (a pair of text rows keeps every key
// tile and runs several times longer than the average pair: started late it would be the tail of the launch),
// then head after head, longest first, so that one head's K and V stay in L2 while its pairs run.
constexpr int kLongFirst = 2;
constexpr int kOrderSplit = 4;      // CTAs per head: each ranks a quarter of the pairs against all of them
// With heads_per_group < Hm the heads are ordered group by group (heads [g * heads_per_group, ...) form group g):
// group g's part of `order` starts at g * heads_per_group * npairs, is laid out like a whole order of that many
// heads and holds indices relative to the group's first head - what a launch over that group's heads alone needs.
__global__ void __launch_bounds__(256) order_pairs_kernel(const int32_t* __restrict__ counts, int npairs,
                                                          int heads_per_group, int32_t* __restrict__ order) {
  extern __shared__ int32_t cnt_s[];
  const int h = blockIdx.x;
  const int g = h / heads_per_group, hl = h - g * heads_per_group;
  const int Hg = min(heads_per_group, static_cast<int>(gridDim.x) - g * heads_per_group);
  int32_t* og = order + static_cast<int64_t>(g) * heads_per_group * npairs;
  const int32_t* c = counts + static_cast<int64_t>(h) * npairs;
  for (int i = threadIdx.x; i < npairs; i += blockDim.x) cnt_s[i] = c[i];
  __syncthreads();
  const int r0 = min(kLongFirst, npairs);
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < npairs; i += kOrderSplit * blockDim.x) {
    const int ci = cnt_s[i];
    int rank = 0;
#pragma unroll 8
    for (int j = 0; j < npairs; ++j) {
      const int cj = cnt_s[j];
      rank += (cj > ci) || (cj == ci && j < i);
    }
    const int64_t pos = (rank < r0) ? static_cast<int64_t>(rank) * Hg + hl
                                    : static_cast<int64_t>(r0) * Hg + static_cast<int64_t>(hl) * (npairs - r0) + (rank - r0);
    og[pos] = hl * npairs + i;
  }
}


// ---- static radial mask (comparison mode `--sparse_type radial`) -----------------------------------------
// The reference builds, for every pair of frames, a token-level band |col - row| <= width(frame distance),
// drops whole frame distances at a distance-dependent stride, places the band in a tile padded to the block
// grid and keeps a block when more than 60 % of its non-empty columns are more than a third full; the
// tiles are OR-ed into the mask and text rows/columns are all true.  A column's fill is the overlap of two
// intervals, so a block is decided in O(block_size) integer operations without any token-level array: one
// thread per block, looping over the frame pairs whose tile covers it.
constexpr int kMaxRadialFrames = 128;
struct RadialTable {
  int width[kMaxRadialFrames];        // band half-width per frame distance (floor of the float32 bound)
  uint8_t kept[kMaxRadialFrames];     // whether that frame distance is kept at all
};

__global__ void __launch_bounds__(256) radial_mask_kernel(const __grid_constant__ RadialTable tab, int tpf, int frames,
                                                          int bs, int nb, int border, int first_col_all,
                                                          uint8_t* __restrict__ mask) {
  const int C = blockIdx.x * blockDim.x + threadIdx.x;
  const int R = blockIdx.y;
  if (C >= nb) return;
  bool keep = (R >= border) || (C >= border);
  if (!keep) {
    const int k = (tpf - 1) / bs + 1;                       // blocks per side of a frame-pair tile
    // frames whose tile covers block row R: (R-k+1)*bs <= i*tpf < (R+1)*bs
    const long long lo_r = static_cast<long long>(R - k + 1) * bs, hi_r = static_cast<long long>(R + 1) * bs;
    const long long lo_c = static_cast<long long>(C - k + 1) * bs, hi_c = static_cast<long long>(C + 1) * bs;
    const int i0 = lo_r <= 0 ? 0 : static_cast<int>((lo_r + tpf - 1) / tpf);
    const int i1 = min(frames - 1, static_cast<int>((hi_r + tpf - 1) / tpf) - 1);
    const int j0 = lo_c <= 0 ? 0 : static_cast<int>((lo_c + tpf - 1) / tpf);
    const int j1 = min(frames - 1, static_cast<int>((hi_c + tpf - 1) / tpf) - 1);
    for (int i = i0; i <= i1 && !keep; ++i) {
      const long long ti = static_cast<long long>(i) * tpf;
      const int lr = R - static_cast<int>(ti / bs), rem_r = static_cast<int>(ti % bs);
      const int ra = max(0, lr * bs - rem_r), rb = min(tpf, (lr + 1) * bs - rem_r);    // local rows [ra, rb)
      if (rb <= ra) continue;
      for (int j = j0; j <= j1 && !keep; ++j) {
        const long long tj = static_cast<long long>(j) * tpf;
        const int lc = C - static_cast<int>(tj / bs), rem_c = static_cast<int>(tj % bs);
        const int ca = max(0, lc * bs - rem_c), cb = min(tpf, (lc + 1) * bs - rem_c);  // local columns [ca, cb)
        if (cb <= ca) continue;
        const int dist = abs(i - j);
        const bool all = first_col_all && j == 0;
        if (!all && !tab.kept[dist]) continue;
        const int W = all ? tpf : tab.width[dist];
        int nonzero = 0, high = 0;
        for (int c = ca; c < cb; ++c) {
          const int cnt = min(rb - 1, c + W) - max(ra, c - W) + 1;
          nonzero += cnt > 0;
          high += 3 * cnt > bs;
        }
        keep = nonzero > 0 && 5 * high > 3 * nonzero;
      }
    }
  }
  mask[static_cast<int64_t>(R) * nb + C] = keep ? 1 : 0;
}

}  // namespace
}  // namespace moddit

using namespace moddit;

extern "C" int moddit_select_lines(const float* cur_c, const float* cur_d, const float* last_c, const float* last_d,
                                   int H, int n, int top_k, float predict_T, int64_t* selected, void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(cur_c && cur_d && last_c && last_d && selected, "select_lines: null pointer");
  MODDIT_CHECK_ARG(H > 0 && n > 0 && top_k > 0, "select_lines: H=%d n=%d top_k=%d must be positive", H, n, top_k);
  MODDIT_CHECK_ARG(predict_T != 0.f, "select_lines: predict_T must be non-zero");
  if (n > 4096) return fail(MODDIT_E_UNSUPPORTED, "select_lines: n=%d exceeds 4096", n);
  if (int rc = require_sm100()) return rc;
  const int L = 3 * n - 1;
  const int k = top_k < L ? top_k : L;
  int P = 2;
  while (P < L) P <<= 1;
  const size_t smem = sizeof(unsigned long long) * P;     // at most 128 KB (n <= 4096)
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(select_lines_kernel), smem)) return rc;
  select_lines_kernel<<<H, kSelectThreads, smem, as_stream(stream)>>>(cur_c, cur_d, last_c, last_d, n, k, P, predict_T,
                                                                      selected);
  MODDIT_CHECK_LAUNCH("select_lines_kernel");
  return MODDIT_OK;
}

extern "C" int moddit_head_modes(const float* b_d, int H, float threshold, int32_t* modes, void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(b_d && modes && H > 0, "head_modes: bad arguments");
  if (int rc = require_sm100()) return rc;
  head_modes_kernel<<<ceil_div(H, 128), 128, 0, as_stream(stream)>>>(b_d, H, threshold, modes);
  MODDIT_CHECK_LAUNCH("head_modes_kernel");
  return MODDIT_OK;
}

extern "C" int moddit_mask_from_lines(const int64_t* selected, int k, const int32_t* modes, int H, int n,
                                      int blocks_per_frame, int layout, int text_blocks, int nbt, uint8_t* mask,
                                      void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(selected && modes && mask, "mask_from_lines: null pointer");
  MODDIT_CHECK_ARG(H > 0 && H <= 65535 && n > 0 && k >= 0 && blocks_per_frame > 0 && text_blocks >= 0,
                   "mask_from_lines: bad sizes");
  if (n > 4096) return fail(MODDIT_E_UNSUPPORTED, "mask_from_lines: n=%d exceeds 4096", n);
  int voff = 0;
  if (layout == MODDIT_LAYOUT_WAN) {
    MODDIT_CHECK_ARG(nbt == n, "mask_from_lines: wan layout needs nbt == n (got %d, %d)", nbt, n);
  } else if (layout == MODDIT_LAYOUT_HUNYUAN) {
    MODDIT_CHECK_ARG(nbt >= n, "mask_from_lines: nbt=%d smaller than n=%d", nbt, n);
  } else if (layout == MODDIT_LAYOUT_COGVIDEOX) {
    MODDIT_CHECK_ARG(nbt == n + text_blocks, "mask_from_lines: cogvideox layout needs nbt == text_blocks + n");
    voff = text_blocks;
  } else {
    return fail(MODDIT_E_ARG, "mask_from_lines: unknown layout %d", layout);
  }
  if (int rc = require_sm100()) return rc;
  // bit arrays: columns padded to the 1024-column segments a warp walks; diagonals with pad_bits zero bits in front
  // (a row's first word starts at offset -row >= -(voff + n - 1) relative to the main diagonal's n - 1) and room for
  // a whole segment behind
  const int col_words = ceil_div(nbt, 1024) * 32;
  const int pad_bits = ceil_div(voff, 32) * 32 + 32;
  const int diag_words = (pad_bits + 32 * col_words + n) / 32 + 2;
  const size_t smem = sizeof(uint32_t) * static_cast<size_t>(col_words + diag_words);
  if (smem > 200 * 1024) return fail(MODDIT_E_UNSUPPORTED, "mask_from_lines: %d blocks exceed the bit arrays", nbt);
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(mask_from_lines_kernel), smem)) return rc;
  mask_from_lines_kernel<<<dim3(ceil_div(nbt, kMaskRows), H), kMaskThreads, smem, as_stream(stream)>>>(
      selected, k, modes, n, blocks_per_frame, voff, nbt, pad_bits, col_words, diag_words, mask);
  MODDIT_CHECK_LAUNCH("mask_from_lines_kernel");
  return MODDIT_OK;
}

extern "C" int moddit_select_mass(const void* map_f16, int H, int n, float tau, uint8_t* keep, void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(map_f16 && keep, "select_mass: null pointer");
  MODDIT_CHECK_ARG(H > 0 && H <= 65535 && n > 0, "select_mass: bad sizes");
  MODDIT_CHECK_ARG(tau >= 0.f && tau <= 1.f, "select_mass: tau=%g outside [0, 1]", tau);
  if (n > 2048) return fail(MODDIT_E_UNSUPPORTED, "select_mass: n=%d exceeds 2048", n);
  if (int rc = require_sm100()) return rc;
  const uint32_t tau_fixed = static_cast<uint32_t>(floorf(tau * 16777216.0f));
  if (n <= kMassWarpMax) {
    const int rows = H * n;
    select_mass_warp_kernel<<<ceil_div(rows, kMassWarpThreads / 32), kMassWarpThreads, 0, as_stream(stream)>>>(
        static_cast<const __half*>(map_f16), n, rows, tau_fixed, 0, nullptr, nullptr, keep);
    MODDIT_CHECK_LAUNCH("select_mass_warp_kernel");
    return MODDIT_OK;
  }
  int P = 2;
  while (P < n) P <<= 1;
  select_mass_kernel<<<dim3(n, H), kMassThreads, 2 * sizeof(unsigned long long) * P, as_stream(stream)>>>(
      static_cast<const __half*>(map_f16), n, P, tau_fixed, 0, nullptr, nullptr, keep);
  MODDIT_CHECK_LAUNCH("select_mass_kernel");
  return MODDIT_OK;
}

extern "C" int moddit_select_topk_blocks(const void* map_f16, int H, int n, int count, const uint8_t* row_full,
                                         const uint8_t* col_keep, uint8_t* keep, void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(map_f16 && keep, "select_topk_blocks: null pointer");
  MODDIT_CHECK_ARG(H > 0 && H <= 65535 && n > 0, "select_topk_blocks: bad sizes");
  MODDIT_CHECK_ARG(count > 0 && count <= n, "select_topk_blocks: count=%d outside 1..%d", count, n);
  if (n > 2048) return fail(MODDIT_E_UNSUPPORTED, "select_topk_blocks: n=%d exceeds 2048", n);
  if (int rc = require_sm100()) return rc;
  if (n <= kMassWarpMax) {
    const int rows = H * n;
    select_mass_warp_kernel<<<ceil_div(rows, kMassWarpThreads / 32), kMassWarpThreads, 0, as_stream(stream)>>>(
        static_cast<const __half*>(map_f16), n, rows, 0u, count, row_full, col_keep, keep);
    MODDIT_CHECK_LAUNCH("select_mass_warp_kernel");
    return MODDIT_OK;
  }
  int P = 2;
  while (P < n) P <<= 1;
  select_mass_kernel<<<dim3(n, H), kMassThreads, 2 * sizeof(unsigned long long) * P, as_stream(stream)>>>(
      static_cast<const __half*>(map_f16), n, P, 0u, count, row_full, col_keep, keep);
  MODDIT_CHECK_LAUNCH("select_mass_kernel");
  return MODDIT_OK;
}

extern "C" int moddit_tile_lists(const uint8_t* mask, int Hm, int nbq, int nbk, int block_size, int N,
                                 int kv_block_limit, int32_t* counts, int32_t* entries, int32_t* order,
                                 void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(mask && counts && entries, "tile_lists: null pointer");
  MODDIT_CHECK_ARG(Hm > 0 && Hm <= 65535 && nbq > 0 && nbk > 0 && N > 0 && kv_block_limit >= 0, "tile_lists: bad sizes");
  if (block_size != 64 && block_size != 128)
    return fail(MODDIT_E_UNSUPPORTED, "tile_lists: block_size must be 64 or 128, got %d", block_size);
  const int ntq = ceil_div(N, 128);
  if (ntq >= (1 << 23)) return fail(MODDIT_E_UNSUPPORTED, "tile_lists: N=%d too large", N);
  if (int rc = require_sm100()) return rc;
  const int npairs = (ntq + 1) / 2;
  tile_lists_kernel<<<dim3(ceil_div(npairs, kListThreads / 32), Hm), kListThreads, 0, as_stream(stream)>>>(
      mask, nbq, nbk, 128 / block_size, ntq, ntq, kv_block_limit, npairs, counts, entries);
  MODDIT_CHECK_LAUNCH("tile_lists_kernel");
  if (order != nullptr) {
    order_pairs_kernel<<<dim3(Hm, kOrderSplit), 256, sizeof(int32_t) * npairs, as_stream(stream)>>>(counts, npairs, Hm, order);
    MODDIT_CHECK_LAUNCH("order_pairs_kernel");
  }
  return MODDIT_OK;
}

extern "C" int moddit_order_pairs(const int32_t* counts, int Hm, int npairs, int heads_per_group, int32_t* order,
                                  void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(counts && order, "order_pairs: null pointer");
  MODDIT_CHECK_ARG(Hm > 0 && Hm <= 65535 && npairs > 0, "order_pairs: Hm=%d npairs=%d out of range", Hm, npairs);
  MODDIT_CHECK_ARG(heads_per_group > 0 && heads_per_group <= Hm, "order_pairs: heads_per_group=%d outside [1, %d]",
                   heads_per_group, Hm);
  if (sizeof(int32_t) * static_cast<size_t>(npairs) > 200 * 1024)
    return fail(MODDIT_E_UNSUPPORTED, "order_pairs: npairs=%d too large", npairs);
  if (int rc = require_sm100()) return rc;
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(order_pairs_kernel), sizeof(int32_t) * npairs)) return rc;
  order_pairs_kernel<<<dim3(Hm, kOrderSplit), 256, sizeof(int32_t) * npairs, as_stream(stream)>>>(counts, npairs,
                                                                                                 heads_per_group, order);
  MODDIT_CHECK_LAUNCH("order_pairs_kernel");
  return MODDIT_OK;
}

extern "C" int moddit_radial_mask(int layout, int video_tokens, int num_frames, int seq_len, int block_size,
                                  float decay_factor, uint8_t* mask, void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(mask, "radial_mask: null pointer");
  MODDIT_CHECK_ARG(video_tokens > 0 && num_frames > 0 && seq_len >= video_tokens && block_size > 0,
                   "radial_mask: video=%d frames=%d seq=%d block=%d out of range", video_tokens, num_frames, seq_len,
                   block_size);
  MODDIT_CHECK_ARG(decay_factor > 0.f, "radial_mask: decay_factor must be positive");
  if (layout != MODDIT_LAYOUT_HUNYUAN && layout != MODDIT_LAYOUT_WAN)
    return fail(MODDIT_E_ARG, "radial_mask: Unknown model type: layout %d (hunyuan and wan only)", layout);
  if (num_frames > kMaxRadialFrames)
    return fail(MODDIT_E_UNSUPPORTED, "radial_mask: %d frames exceed %d", num_frames, kMaxRadialFrames);
  const int tpf = video_tokens / num_frames;
  MODDIT_CHECK_ARG(tpf > 0, "radial_mask: fewer video tokens than frames");
  const int nb = seq_len / block_size;
  MODDIT_CHECK_ARG(nb > 0, "radial_mask: sequence shorter than a block");
  const int k = (tpf - 1) / block_size + 1;
  MODDIT_CHECK_ARG(static_cast<long long>(num_frames - 1) * tpf / block_size + k <= nb,
                   "radial_mask: the last frame's tile does not fit %d blocks", nb);
  if (int rc = require_sm100()) return rc;
  // band half-width and kept flag per frame distance, in the reference's arithmetic: powers of two and the
  // decay factor in double precision, the comparison against token distances in float32
  RadialTable tab = {};
  int bits = 0;
  for (int t = tpf; t > 0; t >>= 1) ++bits;                 // tpf.bit_length()
  const double pow_tpf = ldexp(1.0, bits);
  for (int dist = 0; dist < num_frames; ++dist) {
    int group = 0;
    for (int t = dist; t > 0; t >>= 1) ++group;             // dist.bit_length()
    double width;
    if ((layout == MODDIT_LAYOUT_WAN && dist < 1) || (layout == MODDIT_LAYOUT_HUNYUAN && dist <= 1)) {
      width = tpf;
    } else if (layout == MODDIT_LAYOUT_WAN && dist == 1) {
      width = tpf / 2;
    } else {
      const double decay = pow_tpf / ldexp(1.0, group) * static_cast<double>(decay_factor);
      width = decay >= block_size ? decay : block_size;
    }
    tab.width[dist] = static_cast<int>(floorf(fminf(static_cast<float>(width), 1.0e9f)));
    const double plain = pow_tpf / ldexp(1.0, group);
    tab.kept[dist] = plain >= 128.0 ? 1 : (dist % static_cast<int>(128.0 / plain) == 0);
  }
  radial_mask_kernel<<<dim3(ceil_div(nb, 256), nb), 256, 0, as_stream(stream)>>>(
      tab, tpf, num_frames, block_size, nb, video_tokens / block_size, layout == MODDIT_LAYOUT_WAN ? 1 : 0, mask);
  MODDIT_CHECK_LAUNCH("radial_mask_kernel");
  return MODDIT_OK;
}
