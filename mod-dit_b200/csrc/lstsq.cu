// Least-squares fit of a block map onto the (diagonals | verticals | per-frame block diagonal) basis.
//
// Unknown order everywhere: [2n-1 diagonals, offset -(n-1)..n-1 | n verticals | 1 block], F = 3n.
//
// mts      : one pass over the map.  A CTA stages 32 map rows in shared memory (optionally merging
//            history on the way in), then threads own a column / a diagonal and walk down the rows,
//            so no atomics are needed; per-tile partial sums go to scratch and a second small
//            kernel adds them in a fixed order (deterministic).  Algorithmic traffic: H*n*n*2 bytes.
// mtm      : closed-form Gram matrix (kept for API parity; the solve below never forms it).
// solve    : the Gram matrix is  [[Dd+lI, A, b], [A^T, (n+l)I, c], [b^T, c^T, e+l]]  with Dd diagonal,
//            so the 2n-1 diagonal unknowns are eliminated analytically; products with A and A^T are
//            prefix/suffix/window sums.  What remains is a data-independent (n+1)x(n+1) SPD system
//            whose inverse is computed once per geometry in float64 (solve_prepare); a solve is then
//            two scans, one (n+1)^2 matrix-vector product per head and an elementwise back-substitution.
#include <cuda_fp16.h>

#include <mutex>

#include "common.cuh"

namespace moddit {
namespace {

constexpr int kTileRows = 32;
constexpr int kMtsThreads = 256;

__device__ __forceinline__ double block_sum_double(double v, double* scratch) {
  // scratch: at least 32 doubles of shared memory
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  double t = 0.0;
  if (warp == 0) {
    t = (lane < (blockDim.x + 31) / 32) ? scratch[lane] : 0.0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) scratch[0] = t;
  }
  __syncthreads();
  t = scratch[0];
  __syncthreads();
  return t;
}

// Partial layout per (head, tile): [n + kTileRows - 1 diagonal partials | n column partials], then one double.
__global__ void __launch_bounds__(kMtsThreads) mts_partial_kernel(
    const __half* __restrict__ map, const __half* __restrict__ prev, const uint8_t* __restrict__ keep,
    int64_t mask_head_stride, int64_t mask_row_stride, int mask_off, __half* __restrict__ merged, int n, int bpf,
    float* __restrict__ part_f, double* __restrict__ part_blk) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ double red[32];

  const int h = blockIdx.y;
  const int tiles = gridDim.x;
  const int i0 = blockIdx.x * kTileRows;
  const int rows = min(kTileRows, n - i0);
  const int tid = threadIdx.x;
  const int64_t span0 = (static_cast<int64_t>(h) * n + i0) * n;  // first element of the tile
  const int len = rows * n;

  // The tile [kTileRows][n] starts `mis` halves into the buffer, `mis` being how far the tile's first element in
  // global memory sits past a 16-byte boundary: 16-byte chunks of the source are then 16-byte chunks of the copy.
  const __half* src = map + span0;
  const int mis = static_cast<int>((reinterpret_cast<uintptr_t>(src) >> 1) & 7);
  __half* tile = reinterpret_cast<__half*>(smem_raw) + mis;
  if (prev == nullptr) {
    // contiguous span of rows*n halves: scalar head until 16-byte aligned, 128-bit body, scalar tail
    const int head = min(len, (8 - mis) & 7);
    for (int e = tid; e < head; e += kMtsThreads) tile[e] = src[e];
    const int body = (len - head) / 8;
    const uint4* vsrc = reinterpret_cast<const uint4*>(src + head);
    uint4* vdst = reinterpret_cast<uint4*>(tile + head);
    for (int e = tid; e < body; e += kMtsThreads) vdst[e] = __ldg(vsrc + e);
    for (int e = head + body * 8 + tid; e < len; e += kMtsThreads) tile[e] = src[e];
  } else {
    const uint8_t* kh = keep + static_cast<int64_t>(h) * mask_head_stride;
    for (int e = tid; e < len; e += kMtsThreads) {
      const int r = e / n, j = e - r * n;
      const bool kp = kh[static_cast<int64_t>(i0 + r + mask_off) * mask_row_stride + (j + mask_off)] != 0;
      const __half v = kp ? map[span0 + e] : prev[span0 + e];
      tile[e] = v;
      merged[span0 + e] = v;
    }
  }
  __syncthreads();

  float* pf = part_f + (static_cast<int64_t>(h) * tiles + blockIdx.x) * (2 * n + kTileRows - 1);
  // diagonals of the tile: index dd = (j - r) + kTileRows - 1 in [0, n + kTileRows - 1)
  for (int dd = tid; dd < n + kTileRows - 1; dd += kMtsThreads) {
    const int d = dd - (kTileRows - 1);
    float s = 0.f;
    for (int r = 0; r < rows; ++r) {
      const int j = d + r;
      if (j >= 0 && j < n) s += __half2float(tile[r * n + j]);
    }
    pf[dd] = s;
  }
  for (int j = tid; j < n; j += kMtsThreads) {
    float s = 0.f;
    for (int r = 0; r < rows; ++r) s += __half2float(tile[r * n + j]);
    pf[n + kTileRows - 1 + j] = s;
  }
  // per-frame block-diagonal: rows/cols below cov = (n / bpf) * bpf with row/bpf == col/bpf
  const int cov = (n / bpf) * bpf;
  double bsum = 0.0;
  for (int e = tid; e < rows * bpf; e += kMtsThreads) {
    const int r = e / bpf, c = e - r * bpf;
    const int i = i0 + r;
    if (i < cov) bsum += static_cast<double>(__half2float(tile[r * n + (i / bpf) * bpf + c]));
  }
  bsum = block_sum_double(bsum, red);
  if (tid == 0) part_blk[static_cast<int64_t>(h) * tiles + blockIdx.x] = bsum;
}

__global__ void __launch_bounds__(256) mts_finish_kernel(const float* __restrict__ part_f,
                                                         const double* __restrict__ part_blk, int n, int tiles,
                                                         float* __restrict__ mts) {
  const int h = blockIdx.y;
  const int x = blockIdx.x * blockDim.x + threadIdx.x;
  const int F = 3 * n;
  if (x >= F) return;
  const int stride = 2 * n + kTileRows - 1;
  const float* pf = part_f + static_cast<int64_t>(h) * tiles * stride;
  float out;
  if (x < 2 * n - 1) {
    const int o = x - (n - 1);
    float s = 0.f;
    for (int t = 0; t < tiles; ++t) {
      // tile-local diagonal d = j - r = o + i0
      const int dd = o + t * kTileRows + (kTileRows - 1);
      if (dd >= 0 && dd < n + kTileRows - 1) s += pf[static_cast<int64_t>(t) * stride + dd];
    }
    out = s;
  } else if (x < 3 * n - 1) {
    const int j = x - (2 * n - 1);
    float s = 0.f;
    for (int t = 0; t < tiles; ++t) s += pf[static_cast<int64_t>(t) * stride + n + kTileRows - 1 + j];
    out = s;
  } else {
    double s = 0.0;
    for (int t = 0; t < tiles; ++t) s += part_blk[static_cast<int64_t>(h) * tiles + t];
    out = static_cast<float>(s);
  }
  mts[static_cast<int64_t>(h) * F + x] = out;
}

// Element (a, b) of the structural Gram matrix M^T M + reg * I for unknowns [2n-1 diagonals | n columns | 1 block].
__device__ __forceinline__ float mtm_entry(int a, int b, int n, int bpf, float reg) {
  const bool diag = (a == b);
  if (a > b) {  // symmetric: evaluate the upper triangle
    const int t = a;
    a = b;
    b = t;
  }
  const int nd = 2 * n - 1;
  const int nb = n / bpf, cov = nb * bpf;
  float v = 0.f;
  if (a < nd) {
    const int o = a - (n - 1);
    const int ao = o < 0 ? -o : o;
    if (b < nd) {
      v = diag ? static_cast<float>(n - ao) : 0.f;
    } else if (b < nd + n) {
      const int j = b - nd;
      v = (o >= 0 ? (j >= o) : (j < n + o)) ? 1.f : 0.f;
    } else {
      v = (ao < bpf) ? static_cast<float>(nb * (bpf - ao)) : 0.f;
    }
  } else if (a < nd + n) {
    const int j = a - nd;
    if (b < nd + n) {
      v = diag ? static_cast<float>(n) : 0.f;
    } else {
      v = (j < cov) ? static_cast<float>(bpf) : 0.f;
    }
  } else {
    v = static_cast<float>(nb * bpf * bpf);
  }
  if (diag) v = __fadd_rn(v, reg);
  return v;
}

__global__ void mtm_kernel(int n, int bpf, float reg, float* __restrict__ mtm) {
  const int F = 3 * n;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<int64_t>(F) * F) return;
  mtm[idx] = mtm_entry(static_cast<int>(idx / F), static_cast<int>(idx % F), n, bpf, reg);
}

// ---- small systems: normal equations in shared memory, Cholesky, one warp per head -------------------------------
// For 3n <= kSmallMaxF unknowns the whole Gram matrix fits one CTA's shared memory in float32 (rows padded by one
// word so that column walks do not collide on a bank).  `solve_small_factor_kernel` (once per geometry, like the
// reference's cached factor, MoD/mod/cuda_lstsq.py:153-186) builds it from the closed form and factors it in place
// (right-looking Cholesky, a warp per row of the trailing update); `solve_small_kernel` (per call) brings the
// factor into shared memory and every warp takes the right-hand side of one head: forward and back substitution
// as warp-wide dot products, float32 like the reference's torch.linalg.cholesky / cholesky_solve on this system
// (MoD/mod/cuda_lstsq.py:177,203).
constexpr int kSmallMaxF = 224;
constexpr int kSmallFactorThreads = 1024;
constexpr int kSmallThreads = 256;

__global__ void __launch_bounds__(kSmallFactorThreads) solve_small_factor_kernel(int n, int bpf, float reg,
                                                                                float* __restrict__ L) {
  extern __shared__ __align__(16) float small_smem[];
  const int F = 3 * n;
  const int ld = F + 1;
  float* A = small_smem;                                 // [F][ld], lower triangle becomes L
  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  for (int e = tid; e < F * F; e += kSmallFactorThreads) {
    const int a = e / F, b = e - a * F;
    A[a * ld + b] = mtm_entry(a, b, n, bpf, reg);
  }
  __syncthreads();
  for (int k = 0; k < F; ++k) {
    const float piv = sqrtf(A[k * ld + k]);              // every thread reads the same word; thread 0 writes it below
    __syncthreads();
    if (tid == 0) A[k * ld + k] = piv;
    const float inv = 1.0f / piv;
    for (int i = k + 1 + tid; i < F; i += kSmallFactorThreads) A[i * ld + k] *= inv;
    __syncthreads();
    // trailing update of the lower triangle: A[i][j] -= L[i][k] * L[j][k] for k < j <= i; a warp per row
    for (int i = k + 1 + warp; i < F; i += kSmallFactorThreads / 32) {
      const float lik = A[i * ld + k];
      for (int j = k + 1 + lane; j <= i; j += 32) A[i * ld + j] = fmaf(-lik, A[j * ld + k], A[i * ld + j]);
    }
    __syncthreads();
  }
  for (int e = tid; e < F * F; e += kSmallFactorThreads) {
    const int a = e / F, b = e - a * F;
    L[e] = (b <= a) ? A[a * ld + b] : 0.f;
  }
}

__global__ void __launch_bounds__(kSmallThreads) solve_small_kernel(const float* __restrict__ mts,
                                                                    const float* __restrict__ L, int H, int n,
                                                                    float* __restrict__ X) {
  extern __shared__ __align__(16) float small_smem[];
  const int F = 3 * n;
  const int ld = F + 1;
  float* A = small_smem;                                 // [F][ld]: the factor
  float* ys = A + static_cast<size_t>(F) * ld;           // [warps][F] right-hand sides / solutions
  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  for (int e = tid; e < F * F; e += kSmallThreads) {
    const int a = e / F, b = e - a * F;
    A[a * ld + b] = L[e];
  }
  __syncthreads();
  const int h = blockIdx.x * (kSmallThreads / 32) + warp;
  if (h >= H) return;                                     // no block-wide barrier below this line
  float* y = ys + warp * F;
  for (int i = lane; i < F; i += 32) y[i] = mts[static_cast<int64_t>(h) * F + i];
  __syncwarp();
  for (int i = 0; i < F; ++i) {                           // L y = b
    float acc = 0.f;
    for (int j = lane; j < i; j += 32) acc = fmaf(A[i * ld + j], y[j], acc);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) y[i] = (y[i] - acc) / A[i * ld + i];
    __syncwarp();
  }
  for (int i = F - 1; i >= 0; --i) {                      // L^T x = y
    float acc = 0.f;
    for (int j = i + 1 + lane; j < F; j += 32) acc = fmaf(A[j * ld + i], y[j], acc);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) y[i] = (y[i] - acc) / A[i * ld + i];
    __syncwarp();
  }
  for (int i = lane; i < F; i += 32) X[static_cast<int64_t>(h) * F + i] = y[i];
}

// ---- solve set-up -------------------------------------------------------------------------------
// factor layout (doubles): Sinv[(n+1)^2] | w[2n-1] | wb[2n-1]      (w = 1/(n-|o|+l), wb = w*b)
// workspace (doubles)    : pw[2n] | pwb[2n] | row[n+1] | col[n+1] | scalars[2]

__global__ void solve_vectors_kernel(int n, int bpf, double lam, double* __restrict__ w, double* __restrict__ wb,
                                     double* __restrict__ pw, double* __restrict__ pwb,
                                     double* __restrict__ scalars) {
  // single thread: 2n-1 terms, runs once per geometry
  if (blockIdx.x != 0 || threadIdx.x != 0) return;
  const int nd = 2 * n - 1;
  const int nb = n / bpf;
  double accw = 0.0, accwb = 0.0, bwb = 0.0;
  pw[0] = 0.0;
  pwb[0] = 0.0;
  for (int oi = 0; oi < nd; ++oi) {
    const int o = oi - (n - 1);
    const int ao = o < 0 ? -o : o;
    const double wi = 1.0 / (static_cast<double>(n - ao) + lam);
    const double bi = (ao < bpf) ? static_cast<double>(nb) * (bpf - ao) : 0.0;
    w[oi] = wi;
    wb[oi] = wi * bi;
    accw += wi;
    accwb += wi * bi;
    bwb += wi * bi * bi;
    pw[oi + 1] = accw;      // exclusive prefix at index oi+1
    pwb[oi + 1] = accwb;
  }
  scalars[0] = bwb;
}

__global__ void schur_build_kernel(int n, int bpf, double lam, const double* __restrict__ pw,
                                   const double* __restrict__ pwb, const double* __restrict__ scalars,
                                   double* __restrict__ S) {
  const int m = n + 1;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<int64_t>(m) * m) return;
  const int a = static_cast<int>(idx / m), b = static_cast<int>(idx % m);
  const int nb = n / bpf, cov = nb * bpf;
  double v;
  if (a < n && b < n) {
    const int lo = a < b ? a : b, hi = a < b ? b : a;
    // sum of w over offsets o in [hi-n+1, lo]  ->  prefix indices [hi, lo+n)
    v = -(pw[lo + n] - pw[hi]);
    if (a == b) v += static_cast<double>(n) + lam;
  } else if (a == n && b == n) {
    v = static_cast<double>(nb) * bpf * bpf + lam - scalars[0];
  } else {
    const int j = a < n ? a : b;
    v = ((j < cov) ? static_cast<double>(bpf) : 0.0) - (pwb[j + n] - pwb[j]);
  }
  S[idx] = v;
}

// In-place Gauss-Jordan inversion of an SPD matrix, one pivot per pair of launches.
__global__ void gj_save_kernel(const double* __restrict__ A, int m, int k, double* __restrict__ row,
                               double* __restrict__ col) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= m) return;
  row[i] = A[static_cast<int64_t>(k) * m + i];
  col[i] = A[static_cast<int64_t>(i) * m + k];
}

__global__ void gj_update_kernel(double* __restrict__ A, int m, int k, const double* __restrict__ row,
                                 const double* __restrict__ col) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  const int i = blockIdx.y;
  if (j >= m) return;
  const double p = 1.0 / row[k];
  double v;
  if (i == k) {
    v = (j == k) ? p : row[j] * p;
  } else if (j == k) {
    v = -col[i] * p;
  } else {
    v = A[static_cast<int64_t>(i) * m + j] - col[i] * row[j] * p;
  }
  A[static_cast<int64_t>(i) * m + j] = v;
}

// ---- per-call solve -----------------------------------------------------------------------------
// workspace (doubles): g[H][n+1] | y[kGemvSplit][H][n+1] (partial products per slice of the inner index)

constexpr int kSolveThreads = 512;

// Inclusive block scan of `vals` (length len) in shared memory, in place; every thread takes part.
__device__ void block_scan_inclusive(double* vals, int len, double* carry_smem) {
  // chunked: each thread scans a contiguous chunk, then chunk totals are scanned by thread 0
  const int per = (len + blockDim.x - 1) / blockDim.x;
  const int beg = min(len, static_cast<int>(threadIdx.x) * per);
  const int end = min(len, beg + per);
  double run = 0.0;
  for (int e = beg; e < end; ++e) {
    run += vals[e];
    vals[e] = run;
  }
  carry_smem[threadIdx.x] = run;
  __syncthreads();
  if (threadIdx.x == 0) {
    double acc = 0.0;
    for (int t = 0; t < static_cast<int>(blockDim.x); ++t) {
      const double v = carry_smem[t];
      carry_smem[t] = acc;
      acc += v;
    }
  }
  __syncthreads();
  const double off = carry_smem[threadIdx.x];
  for (int e = beg; e < end; ++e) vals[e] += off;
  __syncthreads();
}

__global__ void __launch_bounds__(kSolveThreads) solve_rhs_kernel(const float* __restrict__ mts,
                                                                  const double* __restrict__ w,
                                                                  const double* __restrict__ wb, int n,
                                                                  double* __restrict__ g) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  double* t = reinterpret_cast<double*>(smem_raw);   // [2n-1] -> inclusive prefix of w*rd
  double* carry = t + (2 * n - 1);                   // [kSolveThreads]
  __shared__ double red[32];
  const int h = blockIdx.x;
  const int nd = 2 * n - 1;
  const float* r = mts + static_cast<int64_t>(h) * 3 * n;
  double dot = 0.0;
  for (int oi = threadIdx.x; oi < nd; oi += kSolveThreads) {
    const double rd = static_cast<double>(r[oi]);
    t[oi] = w[oi] * rd;
    dot += wb[oi] * rd;
  }
  __syncthreads();
  block_scan_inclusive(t, nd, carry);
  dot = block_sum_double(dot, red);
  double* gh = g + static_cast<int64_t>(h) * (n + 1);
  for (int j = threadIdx.x; j < n; j += kSolveThreads) {
    // sum_{o=j-n+1..j} t[o] -> indices oi in [j, j+n-1]
    const double win = t[j + n - 1] - (j > 0 ? t[j - 1] : 0.0);
    gh[j] = static_cast<double>(r[nd + j]) - win;
  }
  if (threadIdx.x == 0) gh[n] = static_cast<double>(r[nd + n]) - dot;
}

// y_slice = Sinv[j0:j1, :]^T * g[j0:j1] for one head and one slice of the inner index (Sinv is symmetric, so
// thread i walks column i and consecutive threads read consecutive addresses).  The inner index is split
// over blockIdx.z so that the whole GPU takes part: a single pass over it is bound by load latency.
constexpr int kGemvSplit = 16;
constexpr int kGemvHeads = 4;     // heads per CTA: an element of Sinv is loaded once for all of them
__global__ void __launch_bounds__(128) solve_gemv_kernel(const double* __restrict__ Sinv,
                                                         const double* __restrict__ g, int m, int H,
                                                         double* __restrict__ y) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  double* gs = reinterpret_cast<double*>(smem_raw);      // [kGemvHeads][per]
  const int h0 = blockIdx.y * kGemvHeads;
  const int per = (m + kGemvSplit - 1) / kGemvSplit;
  const int j0 = blockIdx.z * per;
  const int j1 = min(m, j0 + per);
  for (int e = threadIdx.x; e < kGemvHeads * per; e += blockDim.x) {
    const int hh = e / per, j = j0 + (e - hh * per);
    gs[e] = (h0 + hh < H && j < j1) ? g[static_cast<int64_t>(h0 + hh) * m + j] : 0.0;
  }
  __syncthreads();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= m) return;
  // per head the same four chains, in the same order, as a one-head pass would use
  double a[kGemvHeads][4];
#pragma unroll
  for (int hh = 0; hh < kGemvHeads; ++hh)
#pragma unroll
    for (int c = 0; c < 4; ++c) a[hh][c] = 0.0;
  int j = j0;
  for (; j + 3 < j1; j += 4) {
    double s[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) s[c] = Sinv[static_cast<int64_t>(j + c) * m + i];
#pragma unroll
    for (int hh = 0; hh < kGemvHeads; ++hh)
#pragma unroll
      for (int c = 0; c < 4; ++c) a[hh][c] = fma(s[c], gs[hh * per + (j + c - j0)], a[hh][c]);
  }
  for (; j < j1; ++j) {
    const double s = Sinv[static_cast<int64_t>(j) * m + i];
#pragma unroll
    for (int hh = 0; hh < kGemvHeads; ++hh) a[hh][0] = fma(s, gs[hh * per + (j - j0)], a[hh][0]);
  }
  // slice partial: y is laid out [slice][head][m]; the back-substitution adds the slices in a fixed order
#pragma unroll
  for (int hh = 0; hh < kGemvHeads; ++hh)
    if (h0 + hh < H)
      y[(static_cast<int64_t>(blockIdx.z) * H + (h0 + hh)) * m + i] = (a[hh][0] + a[hh][1]) + (a[hh][2] + a[hh][3]);
}

__global__ void __launch_bounds__(kSolveThreads) solve_back_kernel(const float* __restrict__ mts,
                                                                   const double* __restrict__ w,
                                                                   const double* __restrict__ wb,
                                                                   const double* __restrict__ y, int n,
                                                                   float* __restrict__ X) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  double* pc = reinterpret_cast<double*>(smem_raw);  // [n] inclusive prefix of c
  double* carry = pc + n;                            // [kSolveThreads]
  const int h = blockIdx.x;
  const int H = gridDim.x;
  const int nd = 2 * n - 1;
  const int m = n + 1;
  const float* r = mts + static_cast<int64_t>(h) * 3 * n;
  float* xh = X + static_cast<int64_t>(h) * 3 * n;
  auto y_at = [&](int j) {          // sum of the gemv slices, always in the same order
    double acc = 0.0;
    for (int sl = 0; sl < kGemvSplit; ++sl) acc += y[(static_cast<int64_t>(sl) * H + h) * m + j];
    return acc;
  };
  for (int j = threadIdx.x; j < n; j += kSolveThreads) {
    const double yj = y_at(j);
    pc[j] = yj;
    xh[nd + j] = static_cast<float>(yj);
  }
  const double e = y_at(n);
  if (threadIdx.x == 0) xh[nd + n] = static_cast<float>(e);
  __syncthreads();
  block_scan_inclusive(pc, n, carry);
  const double total = pc[n - 1];
  for (int oi = threadIdx.x; oi < nd; oi += kSolveThreads) {
    const int o = oi - (n - 1);
    // (A c)[o] = sum_{j>=o} c_j for o >= 0 ; sum_{j<n+o} c_j for o < 0
    const double ac = (o >= 0) ? (total - (o > 0 ? pc[o - 1] : 0.0)) : pc[n + o - 1];
    xh[oi] = static_cast<float>(w[oi] * (static_cast<double>(r[oi]) - ac) - wb[oi] * e);
  }
}

}  // namespace
}  // namespace moddit

using namespace moddit;

static int check_n(const char* who, int n) {
  if (n < 1 || n > 4096) return fail(MODDIT_E_UNSUPPORTED, "%s: n=%d video blocks outside [1, 4096]", who, n);
  return MODDIT_OK;
}

extern "C" size_t moddit_mts_workspace_bytes(int H, int n) {
  if (H <= 0 || n <= 0) return 0;
  const size_t tiles = static_cast<size_t>(ceil_div(n, kTileRows));
  const size_t f = static_cast<size_t>(H) * tiles * (2 * static_cast<size_t>(n) + kTileRows - 1) * sizeof(float);
  const size_t fpad = (f + 15) / 16 * 16;
  return fpad + static_cast<size_t>(H) * tiles * sizeof(double);
}

extern "C" int moddit_mts(const void* map_f16, const void* prev_f16, const uint8_t* keep_mask,
                          int64_t mask_head_stride, int64_t mask_row_stride, int mask_off, void* merged_out_f16,
                          int H, int n, int blocks_per_frame, float* mts, void* workspace, size_t workspace_bytes,
                          void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(map_f16 && mts, "mts: null pointer");
  MODDIT_CHECK_ARG(H > 0 && H <= 65535, "mts: H=%d outside [1, 65535]", H);
  if (int rc = check_n("mts", n)) return rc;
  MODDIT_CHECK_ARG(blocks_per_frame > 0, "mts: blocks_per_frame=%d must be positive", blocks_per_frame);
  MODDIT_CHECK_ARG((prev_f16 == nullptr) == (keep_mask == nullptr) && (prev_f16 == nullptr) == (merged_out_f16 == nullptr),
                   "mts: prev, keep_mask and merged_out must be given together");
  if (!workspace || workspace_bytes < moddit_mts_workspace_bytes(H, n))
    return fail(MODDIT_E_WORKSPACE, "mts: workspace of %zu bytes needed, got %zu", moddit_mts_workspace_bytes(H, n),
                workspace_bytes);
  if (!aligned16(workspace)) return fail(MODDIT_E_ALIGN, "mts: workspace must be 16-byte aligned");
  const size_t smem = (static_cast<size_t>(kTileRows) * n + 8) * sizeof(__half);   // + the alignment shift
  if (smem > 200 * 1024) return fail(MODDIT_E_UNSUPPORTED, "mts: n=%d rows do not fit shared memory", n);
  if (int rc = require_sm100()) return rc;
  const int tiles = ceil_div(n, kTileRows);
  const size_t f = static_cast<size_t>(H) * tiles * (2 * static_cast<size_t>(n) + kTileRows - 1) * sizeof(float);
  float* part_f = static_cast<float*>(workspace);
  double* part_blk = reinterpret_cast<double*>(static_cast<unsigned char*>(workspace) + (f + 15) / 16 * 16);
  cudaStream_t st = as_stream(stream);
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(mts_partial_kernel), smem)) return rc;
  mts_partial_kernel<<<dim3(tiles, H), kMtsThreads, smem, st>>>(
      static_cast<const __half*>(map_f16), static_cast<const __half*>(prev_f16), keep_mask, mask_head_stride,
      mask_row_stride, mask_off, static_cast<__half*>(merged_out_f16), n, blocks_per_frame, part_f, part_blk);
  MODDIT_CHECK_LAUNCH("mts_partial_kernel");
  mts_finish_kernel<<<dim3(ceil_div(3 * n, 256), H), 256, 0, st>>>(part_f, part_blk, n, tiles, mts);
  MODDIT_CHECK_LAUNCH("mts_finish_kernel");
  return MODDIT_OK;
}

// ---- variant of moddit_mts whose scratch lives in a static device array ----------------------------
constexpr size_t kStaticScratchBytes = size_t(8) << 20;   // 8 MiB per device that loads the library
static __device__ __align__(256) unsigned char g_mts_static_scratch[kStaticScratchBytes];

// In host code the array's name is only a handle for the runtime's symbol table, not a device address;
// the address the kernels need is looked up once per device (with that device current) and kept here.
static std::mutex g_static_scratch_mutex;
static void* g_static_scratch_addr[64] = {};

extern "C" size_t moddit_mts_noalloc_max_bytes(void) { return kStaticScratchBytes; }

extern "C" int moddit_mts_noalloc(const void* map_f16, int H, int n, int blocks_per_frame, float* mts, void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(map_f16 && mts, "mts_noalloc: null pointer");
  MODDIT_CHECK_ARG(H > 0 && H <= 65535, "mts_noalloc: H=%d outside [1, 65535]", H);
  if (int rc = check_n("mts_noalloc", n)) return rc;
  MODDIT_CHECK_ARG(blocks_per_frame > 0, "mts_noalloc: blocks_per_frame=%d must be positive", blocks_per_frame);
  const size_t need = moddit_mts_workspace_bytes(H, n);
  if (need > kStaticScratchBytes)
    return fail(MODDIT_E_UNSUPPORTED,
                "mts_noalloc: H=%d, n=%d needs %zu bytes of scratch but the built-in array holds %zu; use moddit_mts "
                "with a caller-provided workspace",
                H, n, need, kStaticScratchBytes);
  const size_t smem = (static_cast<size_t>(kTileRows) * n + 8) * sizeof(__half);   // + the alignment shift
  if (smem > 200 * 1024) return fail(MODDIT_E_UNSUPPORTED, "mts_noalloc: n=%d rows do not fit shared memory", n);
  if (int rc = require_sm100()) return rc;
  int dev = 0;
  MODDIT_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(MODDIT_E_UNSUPPORTED, "mts_noalloc: device index %d not supported", dev);
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> guard(g_static_scratch_mutex);
    if (g_static_scratch_addr[dev] == nullptr) {
      void* addr = nullptr;
      MODDIT_CHECK_CUDA(cudaGetSymbolAddress(&addr, g_mts_static_scratch));
      g_static_scratch_addr[dev] = addr;
    }
    scratch = g_static_scratch_addr[dev];
  }
  const int tiles = ceil_div(n, kTileRows);
  const size_t f = static_cast<size_t>(H) * tiles * (2 * static_cast<size_t>(n) + kTileRows - 1) * sizeof(float);
  float* part_f = static_cast<float*>(scratch);
  double* part_blk = reinterpret_cast<double*>(static_cast<unsigned char*>(scratch) + (f + 15) / 16 * 16);
  cudaStream_t st = as_stream(stream);
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(mts_partial_kernel), smem)) return rc;
  // every partial that the second kernel reads is written by the first, so nothing has to start at zero
  mts_partial_kernel<<<dim3(tiles, H), kMtsThreads, smem, st>>>(static_cast<const __half*>(map_f16), nullptr, nullptr,
                                                                 0, 0, 0, nullptr, n, blocks_per_frame, part_f,
                                                                 part_blk);
  MODDIT_CHECK_LAUNCH("mts_partial_kernel");
  mts_finish_kernel<<<dim3(ceil_div(3 * n, 256), H), 256, 0, st>>>(part_f, part_blk, n, tiles, mts);
  MODDIT_CHECK_LAUNCH("mts_finish_kernel");
  return MODDIT_OK;
}

namespace moddit {
namespace {
// The map that fitted line intensities describe: one thread per element, rows of the output contiguous over
// the threads.  Sum in the order diagonal, vertical, block term (float32), as the reference accumulates them.
__global__ void __launch_bounds__(256) reconstruct_map_kernel(const float* __restrict__ d, const float* __restrict__ c,
                                                              const float* __restrict__ b_d, int n, int bpf,
                                                              float* __restrict__ out) {
  const int h = blockIdx.z, i = blockIdx.y;
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= n) return;
  const int covered = (n / bpf) * bpf;          // the block term stops at the last whole frame
  float v = 0.f + __ldg(d + static_cast<int64_t>(h) * (2 * n - 1) + (j - i + n - 1));
  v += 2.f * __ldg(c + static_cast<int64_t>(h) * n + j);
  if (i < covered && j < covered && i / bpf == j / bpf) v += __ldg(b_d + h);
  out[(static_cast<int64_t>(h) * n + i) * n + j] = v;
}
}  // namespace
}  // namespace moddit

extern "C" int moddit_reconstruct_map(const float* d, const float* c, const float* b_d, int H, int n,
                                      int blocks_per_frame, float* out, void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(d && c && b_d && out, "reconstruct_map: null pointer");
  MODDIT_CHECK_ARG(H > 0 && H <= 65535 && n > 0 && n <= 65535 && blocks_per_frame > 0,
                   "reconstruct_map: H=%d n=%d blocks_per_frame=%d out of range", H, n, blocks_per_frame);
  if (int rc = require_sm100()) return rc;
  moddit::reconstruct_map_kernel<<<dim3(ceil_div(n, 256), n, H), 256, 0, as_stream(stream)>>>(d, c, b_d, n,
                                                                                           blocks_per_frame, out);
  MODDIT_CHECK_LAUNCH("reconstruct_map_kernel");
  return MODDIT_OK;
}

extern "C" int moddit_mtm(int n, int blocks_per_frame, float regularization, float* mtm, void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(mtm, "mtm: null pointer");
  if (int rc = check_n("mtm", n)) return rc;
  MODDIT_CHECK_ARG(blocks_per_frame > 0, "mtm: blocks_per_frame=%d must be positive", blocks_per_frame);
  if (int rc = require_sm100()) return rc;
  const int64_t total = static_cast<int64_t>(3 * n) * (3 * n);
  mtm_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, as_stream(stream)>>>(n, blocks_per_frame,
                                                                                         regularization, mtm);
  MODDIT_CHECK_LAUNCH("mtm_kernel");
  return MODDIT_OK;
}

extern "C" size_t moddit_solve_factor_bytes(int n) {
  if (n <= 0) return 0;
  const size_t m = static_cast<size_t>(n) + 1;
  return sizeof(double) * (m * m + 2 * (2 * static_cast<size_t>(n) - 1));
}

extern "C" size_t moddit_solve_prepare_workspace_bytes(int n) {
  if (n <= 0) return 0;
  return sizeof(double) * (2 * 2 * static_cast<size_t>(n) + 2 * (static_cast<size_t>(n) + 1) + 2);
}

extern "C" int moddit_solve_prepare(int n, int blocks_per_frame, double regularization, void* factor,
                                    void* workspace, size_t workspace_bytes, void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(factor, "solve_prepare: null factor pointer");
  if (int rc = check_n("solve_prepare", n)) return rc;
  MODDIT_CHECK_ARG(blocks_per_frame > 0, "solve_prepare: blocks_per_frame=%d must be positive", blocks_per_frame);
  MODDIT_CHECK_ARG(regularization > 0.0,
                   "solve_prepare: regularization=%g must be positive (the basis is rank deficient without it)",
                   regularization);
  if (!workspace || workspace_bytes < moddit_solve_prepare_workspace_bytes(n))
    return fail(MODDIT_E_WORKSPACE, "solve_prepare: workspace of %zu bytes needed, got %zu",
                moddit_solve_prepare_workspace_bytes(n), workspace_bytes);
  if (!aligned16(factor) || !aligned16(workspace))
    return fail(MODDIT_E_ALIGN, "solve_prepare: factor and workspace must be 16-byte aligned");
  if (int rc = require_sm100()) return rc;
  const int m = n + 1;
  double* Sinv = static_cast<double*>(factor);
  double* w = Sinv + static_cast<size_t>(m) * m;
  double* wb = w + (2 * n - 1);
  double* pw = static_cast<double*>(workspace);
  double* pwb = pw + 2 * n;
  double* row = pwb + 2 * n;
  double* col = row + m;
  double* scalars = col + m;
  cudaStream_t st = as_stream(stream);
  solve_vectors_kernel<<<1, 1, 0, st>>>(n, blocks_per_frame, regularization, w, wb, pw, pwb, scalars);
  MODDIT_CHECK_LAUNCH("solve_vectors_kernel");
  const int64_t total = static_cast<int64_t>(m) * m;
  schur_build_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, st>>>(n, blocks_per_frame, regularization,
                                                                                 pw, pwb, scalars, Sinv);
  MODDIT_CHECK_LAUNCH("schur_build_kernel");
  for (int k = 0; k < m; ++k) {
    gj_save_kernel<<<ceil_div(m, 256), 256, 0, st>>>(Sinv, m, k, row, col);
    gj_update_kernel<<<dim3(ceil_div(m, 256), m), 256, 0, st>>>(Sinv, m, k, row, col);
  }
  MODDIT_CHECK_LAUNCH("gauss-jordan kernels");
  return MODDIT_OK;
}

extern "C" size_t moddit_solve_workspace_bytes(int H, int n) {
  if (H <= 0 || n <= 0) return 0;
  return sizeof(double) * (1 + kGemvSplit) * static_cast<size_t>(H) * (static_cast<size_t>(n) + 1);
}

extern "C" int moddit_solve(const float* mts, const void* factor, int H, int n, int blocks_per_frame,
                            double regularization, float* X, void* workspace, size_t workspace_bytes, void* stream) {
  clear_error();
  (void)blocks_per_frame;
  (void)regularization;
  MODDIT_CHECK_ARG(mts && factor && X, "solve: null pointer");
  MODDIT_CHECK_ARG(H > 0 && H <= 65535, "solve: H=%d outside [1, 65535]", H);
  if (int rc = check_n("solve", n)) return rc;
  if (!workspace || workspace_bytes < moddit_solve_workspace_bytes(H, n))
    return fail(MODDIT_E_WORKSPACE, "solve: workspace of %zu bytes needed, got %zu", moddit_solve_workspace_bytes(H, n),
                workspace_bytes);
  if (!aligned16(factor) || !aligned16(workspace))
    return fail(MODDIT_E_ALIGN, "solve: factor and workspace must be 16-byte aligned");
  if (int rc = require_sm100()) return rc;
  const int m = n + 1;
  const double* Sinv = static_cast<const double*>(factor);
  const double* w = Sinv + static_cast<size_t>(m) * m;
  const double* wb = w + (2 * n - 1);
  double* g = static_cast<double*>(workspace);
  double* y = g + static_cast<size_t>(H) * m;
  cudaStream_t st = as_stream(stream);
  const size_t sm_rhs = sizeof(double) * ((2 * n - 1) + kSolveThreads);
  const size_t sm_back = sizeof(double) * (n + kSolveThreads);
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(solve_rhs_kernel), sm_rhs)) return rc;
  solve_rhs_kernel<<<H, kSolveThreads, sm_rhs, st>>>(mts, w, wb, n, g);
  MODDIT_CHECK_LAUNCH("solve_rhs_kernel");
  solve_gemv_kernel<<<dim3(ceil_div(m, 128), ceil_div(H, kGemvHeads), kGemvSplit), 128,
                      sizeof(double) * kGemvHeads * ceil_div(m, kGemvSplit), st>>>(Sinv, g, m, H, y);
  MODDIT_CHECK_LAUNCH("solve_gemv_kernel");
  solve_back_kernel<<<H, kSolveThreads, sm_back, st>>>(mts, w, wb, y, n, X);
  MODDIT_CHECK_LAUNCH("solve_back_kernel");
  return MODDIT_OK;
}

extern "C" int moddit_solve_small_max_n(void) { return kSmallMaxF / 3; }

extern "C" size_t moddit_solve_small_factor_bytes(int n) {
  return (n > 0 && 3 * n <= kSmallMaxF) ? sizeof(float) * static_cast<size_t>(3 * n) * (3 * n) : 0;
}

static int check_small(const char* who, int n) {
  if (n <= 0) return fail(MODDIT_E_ARG, "%s: n=%d must be positive", who, n);
  if (3 * n > kSmallMaxF)
    return fail(MODDIT_E_UNSUPPORTED, "%s: 3n=%d unknowns exceed the %d that fit shared memory; use moddit_solve", who,
                3 * n, kSmallMaxF);
  return MODDIT_OK;
}

extern "C" int moddit_solve_small_prepare(int n, int blocks_per_frame, float regularization, float* factor,
                                          void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(factor, "solve_small_prepare: null pointer");
  MODDIT_CHECK_ARG(blocks_per_frame > 0, "solve_small_prepare: blocks_per_frame must be positive");
  MODDIT_CHECK_ARG(regularization > 0.f, "solve_small_prepare: the system is singular without regularisation");
  if (int rc = check_small("solve_small_prepare", n)) return rc;
  if (int rc = require_sm100()) return rc;
  const int F = 3 * n;
  const size_t smem = sizeof(float) * static_cast<size_t>(F) * (F + 1);
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(solve_small_factor_kernel), smem)) return rc;
  solve_small_factor_kernel<<<1, kSmallFactorThreads, smem, as_stream(stream)>>>(n, blocks_per_frame, regularization,
                                                                                factor);
  MODDIT_CHECK_LAUNCH("solve_small_factor_kernel");
  return MODDIT_OK;
}

extern "C" int moddit_solve_small(const float* mts, const float* factor, int H, int n, float* X, void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(mts && factor && X, "solve_small: null pointer");
  MODDIT_CHECK_ARG(H > 0 && H <= 65535 * (kSmallThreads / 32), "solve_small: H=%d out of range", H);
  if (int rc = check_small("solve_small", n)) return rc;
  if (int rc = require_sm100()) return rc;
  const int F = 3 * n;
  const size_t smem = sizeof(float) * (static_cast<size_t>(F) * (F + 1) + static_cast<size_t>(kSmallThreads / 32) * F);
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(solve_small_kernel), smem)) return rc;
  solve_small_kernel<<<ceil_div(H, kSmallThreads / 32), kSmallThreads, smem, as_stream(stream)>>>(mts, factor, H, n, X);
  MODDIT_CHECK_LAUNCH("solve_small_kernel");
  return MODDIT_OK;
}
