// Attention prologue: what the reference's processors do between the q/k/v projections and the attention call
// (per-head or whole-row normalisation of q and k, rotary embedding of the latent tokens, the move from the
// projections' token-major layout to the head-major layout of the attention kernels), in one pass over
// the data.  Follows MoD/models/hunyuan/attention_processor.py:57-106, MoD/models/wan/attention_processor.py:70-93
// and 123-125, MoD/models/cogvideox/attention_processor.py:113-135.
//
// One CTA = eight rows per thread of one head of one of the three tensors: one token block of 128 rows at
// D = 128, several shorter blocks otherwise.  D/8 threads cover a row with one 16-byte load each (a 2*D-byte
// piece of the token's row), so the row statistics are a shuffle reduction over D/8 lanes and a rotary pair
// never leaves its thread; the head-major store is contiguous over the CTA's rows.  Thread-to-row mapping and
// summation order of the optional block means are those of pool_blocks_kernel, so the means equal the ones
// pooled afterwards from the stored tensor bit for bit.  1/sqrt is the hardware approximation, as in the
// tensor library's own device code.
// Bound: HBM.  Algorithmic bytes per token and tensor: 2*H*D read + 2*H*D written (+ the rotary tables:
// 4*D or 8*D bytes per token, fetched once for all heads and shared through L2).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "common.cuh"

namespace moddit {
namespace {

constexpr int kThreads = 256;

// Arithmetic on a 32-bit word holding two neighbouring elements of the 16-bit type T.
template <typename T>
struct Pair;
template <>
struct Pair<__nv_bfloat16> {
  static __device__ __forceinline__ float lo(uint32_t w) { return __uint_as_float(w << 16); }
  static __device__ __forceinline__ float hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
  static __device__ __forceinline__ uint32_t pack(float a, float b) {   // round to nearest even, a in the low half
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
  // product of two T values rounded once to T (what a tensor product of two T tensors gives)
  static __device__ __forceinline__ uint32_t mul(uint32_t a, uint32_t b) {
    const __nv_bfloat162 v = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&a),
                                     *reinterpret_cast<const __nv_bfloat162*>(&b));
    return *reinterpret_cast<const uint32_t*>(&v);
  }
};
template <>
struct Pair<__half> {
  static __device__ __forceinline__ float lo(uint32_t w) { return __low2float(*reinterpret_cast<const __half2*>(&w)); }
  static __device__ __forceinline__ float hi(uint32_t w) { return __high2float(*reinterpret_cast<const __half2*>(&w)); }
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    const __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
  static __device__ __forceinline__ uint32_t mul(uint32_t a, uint32_t b) {
    const __half2 v = __hmul2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&v);
  }
};

template <typename T>
__device__ __forceinline__ void unpack(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = Pair<T>::lo(w[i]);
    f[2 * i + 1] = Pair<T>::hi(w[i]);
  }
}

// Sum over the kTpr lanes that hold one row (kTpr is 8 or 16: the lanes are an aligned group of a warp).
template <int kTpr>
__device__ __forceinline__ float row_sum(float x) {
#pragma unroll
  for (int o = kTpr / 2; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

struct PrologueArgs {
  const void* in[3];
  void* out[3];
  const void* weight[2];
  const void* bias[2];
  const float* inv_rms[2];
  float* pool[2];
  const float* cos;
  const float* sin;
  int64_t token_stride;   // elements between consecutive tokens of an input
  int S, H, N_out, dst_row0, bs, nb_total, blk_base;
  int group;              // token blocks per CTA (a CTA always has eight rows per thread to load)
  int rope_form, rope_lo, rope_hi;
  float eps;
};

// Grid: x = head + H * tensor (q, k, v), y = token block, z = batch - the CTAs of one token block run together,
// so the rotary table rows of the block are fetched from HBM once and shared through L2.
// kRope is the table form (MODDIT_ROPE_*); whether anything is rotated is decided at run time.
template <typename T, int D, int kNorm, int kRope>
__global__ void __launch_bounds__(kThreads, 4) qkv_prologue_kernel(const __grid_constant__ PrologueArgs a) {
  constexpr int kTpr = D / 8;               // threads per row
  constexpr int kRpp = kThreads / kTpr;     // rows per pass
  constexpr float kInvD = 1.0f / D;         // D is a power of two: the product equals the division
  constexpr int kTabW = kRope == MODDIT_ROPE_PAIR ? D / 2 : D;      // table values per token
  constexpr int kTabC = kRope == MODDIT_ROPE_PAIR ? 4 : 8;          // table values per thread and row
  __shared__ float red[kRpp][D];

  const int which = blockIdx.x / a.H;
  const int h = blockIdx.x - which * a.H;
  const int b = blockIdx.z;
  const T* __restrict__ in = static_cast<const T*>(a.in[which]);
  if (in == nullptr) return;
  T* __restrict__ out = static_cast<T*>(a.out[which]);
  const int blk0 = blockIdx.y * a.group;    // first token block of this CTA
  const int row0 = blk0 * a.bs;
  const int rows = min(a.group * a.bs, a.S - row0);
  const int spb = a.group > 1 ? a.bs / kRpp : 0;   // load slots per block when the CTA holds several blocks
  const int cg = threadIdx.x % kTpr;
  const int rg = threadIdx.x / kTpr;
  const bool normed = kNorm != MODDIT_NORM_NONE && which < 2;
  const bool rope_on = which < 2 && a.cos != nullptr;
  float* pool = which < 2 ? a.pool[which] : nullptr;

  // weight (and bias) of this thread's eight columns
  uint4 w2 = make_uint4(0, 0, 0, 0), b2 = make_uint4(0, 0, 0, 0);
  bool has_w = false;
  if (normed) {
    const int wofs = (kNorm == MODDIT_NORM_RMS_ALL_HEADS ? h * D : 0) + cg * 8;
    has_w = a.weight[which] != nullptr;
    if (has_w) w2 = __ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(a.weight[which]) + wofs));
    if (kNorm == MODDIT_NORM_LAYER && a.bias[which] != nullptr)
      b2 = __ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(a.bias[which]) + wofs));
  }

  const T* src = in + (static_cast<int64_t>(b) * a.S + row0) * a.token_stride + h * D + cg * 8;
  T* dst = out + ((static_cast<int64_t>(b) * a.H + h) * a.N_out + a.dst_row0 + row0) * D + cg * 8;
  // table entries of row r of this CTA start at tab + r * kTabW (32-bit offsets: the host checks the size)
  const int tab = (row0 - a.rope_lo) * kTabW + cg * kTabC;

  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  // Mean of block blk0 + j from the threads' partial sums, in the order pool_blocks_kernel adds them.
  auto flush = [&](int j, int block_rows) {
#pragma unroll
    for (int i = 0; i < 8; ++i) red[rg][cg * 8 + i] = acc[i];
    __syncthreads();
    if (threadIdx.x < D) {
      float t = 0.f;
#pragma unroll 8
      for (int g = 0; g < kRpp; ++g) t += red[g][threadIdx.x];
      pool[((static_cast<int64_t>(b) * a.H + h) * a.nb_total + a.blk_base + blk0 + j) * D + threadIdx.x] =
          t / static_cast<float>(block_rows);
    }
    __syncthreads();
  };

  // kWhole: the CTA has all of its 8 * kRpp rows and they are rotated all or none - no test per row.
  auto run = [&](auto whole_tag) {
    constexpr bool kWhole = decltype(whole_tag)::value;
    const bool rope_all = rope_on && row0 >= a.rope_lo && row0 < a.rope_hi;      // only read when kWhole
    for (int base = 0; base < rows; base += 8 * kRpp) {     // uniform trip count: the shuffles need every lane
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int r = base + rg + u * kRpp;
        v[u] = (kWhole || r < rows) ? __ldg(reinterpret_cast<const uint4*>(src + static_cast<int64_t>(r) * a.token_stride))
                                    : make_uint4(0, 0, 0, 0);
      }
      if (rope_on) {
        // the table rows are needed one after the other below: ask for all of them now
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int r = base + rg + u * kRpp;
          const int s = row0 + r;
          if (kWhole ? rope_all : (r < rows && s >= a.rope_lo && s < a.rope_hi)) {
            asm volatile("prefetch.global.L1 [%0];" ::"l"(a.cos + tab + r * kTabW));
            asm volatile("prefetch.global.L1 [%0];" ::"l"(a.sin + tab + r * kTabW));
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int r = base + rg + u * kRpp;
        const bool valid = kWhole || r < rows;
        const int s = row0 + r;               // token index within the input
        uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
        if (normed) {
          if constexpr (kNorm == MODDIT_NORM_RMS_HEAD || kNorm == MODDIT_NORM_RMS_ALL_HEADS) {
            float rs;
            if constexpr (kNorm == MODDIT_NORM_RMS_HEAD) {
              float ss = 0.f;
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float x0 = Pair<T>::lo(w[i]), x1 = Pair<T>::hi(w[i]);
                ss = fmaf(x0, x0, ss);
                ss = fmaf(x1, x1, ss);
              }
              rs = rsqrtf(__fadd_rn(row_sum<kTpr>(ss) * kInvD, a.eps));
            } else {
              rs = valid ? __ldg(a.inv_rms[which] + static_cast<int64_t>(b) * a.S + s) : 0.f;
            }
            // x * rsqrt in float32 rounded to T, then the product with the weight rounded to T again
            const uint32_t wt[4] = {w2.x, w2.y, w2.z, w2.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              w[i] = Pair<T>::pack(__fmul_rn(Pair<T>::lo(w[i]), rs), __fmul_rn(Pair<T>::hi(w[i]), rs));
              if (has_w) w[i] = Pair<T>::mul(w[i], wt[i]);
            }
          } else if constexpr (kNorm == MODDIT_NORM_LAYER) {
            float f[8], wv[8], bv[8];
            unpack<T>(v[u], f);
            unpack<T>(w2, wv);
            unpack<T>(b2, bv);
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) sum += f[i];
            const float mean = row_sum<kTpr>(sum) * kInvD;
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              f[i] -= mean;
              ss = fmaf(f[i], f[i], ss);
            }
            const float rstd = rsqrtf(__fadd_rn(row_sum<kTpr>(ss) * kInvD, a.eps));
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float y0 = fmaf(f[2 * i] * rstd, has_w ? wv[2 * i] : 1.f, bv[2 * i]);
              const float y1 = fmaf(f[2 * i + 1] * rstd, has_w ? wv[2 * i + 1] : 1.f, bv[2 * i + 1]);
              w[i] = valid ? Pair<T>::pack(y0, y1) : 0u;
            }
          }
        }
        if (kWhole ? rope_all : (rope_on && valid && s >= a.rope_lo && s < a.rope_hi)) {
          float c[kTabC], n[kTabC];
          const float* cp = a.cos + tab + r * kTabW;
          const float* np = a.sin + tab + r * kTabW;
#pragma unroll
          for (int i = 0; i < kTabC; i += 4) {
            *reinterpret_cast<float4*>(c + i) = __ldg(reinterpret_cast<const float4*>(cp + i));
            *reinterpret_cast<float4*>(n + i) = __ldg(reinterpret_cast<const float4*>(np + i));
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            // multipliers of (x0, x1) for the even element (ce, se) and for the odd element (so, co)
            const float ce = kRope == MODDIT_ROPE_PAIR ? c[i] : c[2 * i];
            const float co = kRope == MODDIT_ROPE_PAIR ? c[i] : (kRope == MODDIT_ROPE_ELEMENTWISE ? c[2 * i + 1] : c[2 * i]);
            const float se = kRope == MODDIT_ROPE_PAIR ? n[i] : (kRope == MODDIT_ROPE_ELEMENTWISE ? n[2 * i] : n[2 * i + 1]);
            const float so = kRope == MODDIT_ROPE_PAIR ? n[i] : n[2 * i + 1];
            const float x0 = Pair<T>::lo(w[i]), x1 = Pair<T>::hi(w[i]);
            // products rounded separately, then one add (no fused multiply-add), as a tensor expression does
            w[i] = Pair<T>::pack(__fsub_rn(__fmul_rn(x0, ce), __fmul_rn(x1, se)),
                                 __fadd_rn(__fmul_rn(x0, so), __fmul_rn(x1, co)));
          }
        }
        if (valid) *reinterpret_cast<uint4*>(dst + static_cast<int64_t>(r) * D) = make_uint4(w[0], w[1], w[2], w[3]);
        if (pool != nullptr) {                 // rows past the end hold zeros here
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            acc[2 * i] += Pair<T>::lo(w[i]);
            acc[2 * i + 1] += Pair<T>::hi(w[i]);
          }
          if (spb > 0 && (u + 1) % spb == 0) {  // last slot of a block (the same for every thread)
            const int j = u / spb;
            if (j * a.bs < rows) flush(j, min(a.bs, rows - j * a.bs));
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = 0.f;
          }
        }
      }
    }
  };
  const bool rope_mixed = rope_on && !((row0 >= a.rope_lo && row0 + rows <= a.rope_hi) ||
                                       row0 + rows <= a.rope_lo || row0 >= a.rope_hi);
  if (rows == 8 * kRpp && !rope_mixed)
    run(std::true_type{});
  else
    run(std::false_type{});
  if (pool != nullptr && spb == 0) flush(0, rows);
}

// One warp per token: 1/sqrt(mean of squares over the whole H*D row + eps) for the normalisation that spans
// the heads (Wan: norm_q / norm_k are applied before the split into heads).
template <typename T>
__global__ void __launch_bounds__(kThreads) token_inv_rms_kernel(const T* __restrict__ q, const T* __restrict__ k,
                                                                 int64_t tokens, int64_t token_stride, int width,
                                                                 float eps, float* __restrict__ out_q,
                                                                 float* __restrict__ out_k) {
  const int lane = threadIdx.x % 32;
  const int64_t tok = static_cast<int64_t>(blockIdx.x) * (kThreads / 32) + threadIdx.x / 32;
  if (tok >= tokens) return;
  const T* x = blockIdx.y == 0 ? q : k;
  float* out = blockIdx.y == 0 ? out_q : out_k;
  if (x == nullptr) return;
  const uint4* row = reinterpret_cast<const uint4*>(x + tok * token_stride);
  float ss = 0.f;
  for (int c = lane; c < width / 8; c += 32) {
    float f[8];
    unpack<T>(__ldg(row + c), f);
#pragma unroll
    for (int i = 0; i < 8; ++i) ss = fmaf(f[i], f[i], ss);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (lane == 0) out[tok] = rsqrtf(__fadd_rn(ss / static_cast<float>(width), eps));
}

template <typename T>
int launch_prologue(const PrologueArgs& a, int B, int D, int norm_kind, int64_t token_stride, float* ws,
                    cudaStream_t st) {
  if (norm_kind == MODDIT_NORM_RMS_ALL_HEADS) {
    const int64_t tokens = static_cast<int64_t>(B) * a.S;
    const dim3 grid(static_cast<unsigned>((tokens + kThreads / 32 - 1) / (kThreads / 32)), 2);
    token_inv_rms_kernel<T><<<grid, kThreads, 0, st>>>(static_cast<const T*>(a.in[0]), static_cast<const T*>(a.in[1]),
                                                       tokens, token_stride, a.H * D, a.eps, ws, ws + tokens);
    MODDIT_CHECK_LAUNCH("token_inv_rms_kernel");
  }
  const dim3 grid(3 * a.H, ceil_div(a.S, a.bs * a.group), B);
#define MODDIT_PROLOGUE_ROPE(NORM, ROPE)                                        \
  case ROPE:                                                                    \
    if (D == 64)                                                                \
      qkv_prologue_kernel<T, 64, NORM, ROPE><<<grid, kThreads, 0, st>>>(a);     \
    else                                                                        \
      qkv_prologue_kernel<T, 128, NORM, ROPE><<<grid, kThreads, 0, st>>>(a);    \
    break;
#define MODDIT_PROLOGUE_CASE(NORM)                                              \
  case NORM:                                                                    \
    switch (rope) {                                                             \
      MODDIT_PROLOGUE_ROPE(NORM, MODDIT_ROPE_ELEMENTWISE)                       \
      MODDIT_PROLOGUE_ROPE(NORM, MODDIT_ROPE_EVEN_COS_ODD_SIN)                  \
      default:                                                                  \
        MODDIT_PROLOGUE_ROPE(NORM, MODDIT_ROPE_PAIR)                            \
    }                                                                           \
    break;
  const int rope = a.cos != nullptr ? a.rope_form : MODDIT_ROPE_PAIR;
  switch (norm_kind) {
    MODDIT_PROLOGUE_CASE(MODDIT_NORM_NONE)
    MODDIT_PROLOGUE_CASE(MODDIT_NORM_RMS_HEAD)
    MODDIT_PROLOGUE_CASE(MODDIT_NORM_RMS_ALL_HEADS)
    MODDIT_PROLOGUE_CASE(MODDIT_NORM_LAYER)
    default:
      return fail(MODDIT_E_ARG, "unknown norm_kind %d", norm_kind);
  }
#undef MODDIT_PROLOGUE_ROPE
#undef MODDIT_PROLOGUE_CASE
  MODDIT_CHECK_LAUNCH("qkv_prologue_kernel");
  return MODDIT_OK;
}

}  // namespace
}  // namespace moddit

using namespace moddit;

extern "C" size_t moddit_qkv_prologue_workspace_bytes(int B, int S, int norm_kind) {
  if (norm_kind != MODDIT_NORM_RMS_ALL_HEADS || B <= 0 || S <= 0) return 0;
  return static_cast<size_t>(2) * B * S * sizeof(float);
}

extern "C" int moddit_qkv_prologue(const void* q_in, const void* k_in, const void* v_in, int dtype, int B, int S,
                                   int H, int D, int64_t token_stride, int norm_kind, const void* q_weight,
                                   const void* q_bias, const void* k_weight, const void* k_bias, float eps,
                                   const float* rope_cos, const float* rope_sin, int rope_form, int rope_lo,
                                   int rope_hi, void* q_out, void* k_out, void* v_out, int N_out, int dst_row0,
                                   float* q_pool, float* k_pool, int block_size, void* workspace, size_t ws_bytes,
                                   void* stream) {
  clear_error();
  MODDIT_CHECK_ARG(dtype == MODDIT_BF16 || dtype == MODDIT_FP16, "dtype must be MODDIT_BF16 or MODDIT_FP16");
  MODDIT_CHECK_ARG(D == 64 || D == 128, "head_dim %d not supported (64 or 128)", D);
  MODDIT_CHECK_ARG(B > 0 && S > 0 && H > 0, "B, S and H must be positive (got %d, %d, %d)", B, S, H);
  MODDIT_CHECK_ARG(B <= 65535, "B must fit a grid dimension");
  MODDIT_CHECK_ARG(token_stride >= static_cast<int64_t>(H) * D && token_stride % 8 == 0,
                   "token_stride %lld must be a multiple of 8 elements and at least H*D",
                   static_cast<long long>(token_stride));
  MODDIT_CHECK_ARG(dst_row0 >= 0 && static_cast<int64_t>(dst_row0) + S <= N_out,
                   "rows %d..%d do not fit an output of %d rows", dst_row0, dst_row0 + S, N_out);
  MODDIT_CHECK_ARG(norm_kind >= MODDIT_NORM_NONE && norm_kind <= MODDIT_NORM_LAYER, "unknown norm_kind %d",
                   norm_kind);
  MODDIT_CHECK_ARG(q_in != nullptr || k_in != nullptr || v_in != nullptr, "no input tensor given");
  const void* ins[3] = {q_in, k_in, v_in};
  void* outs[3] = {q_out, k_out, v_out};
  for (int i = 0; i < 3; ++i) {
    if (ins[i] == nullptr) continue;
    MODDIT_CHECK_ARG(outs[i] != nullptr, "input %d has no output buffer", i);
    MODDIT_CHECK_ARG(aligned16(ins[i]) && aligned16(outs[i]), "tensor %d is not 16-byte aligned", i);
  }
  const void* params[4] = {q_weight, q_bias, k_weight, k_bias};
  for (const void* p : params) MODDIT_CHECK_ARG(aligned16(p), "norm parameters must be 16-byte aligned");
  MODDIT_CHECK_ARG((rope_cos == nullptr) == (rope_sin == nullptr), "rope_cos and rope_sin go together");
  if (rope_cos != nullptr) {
    MODDIT_CHECK_ARG(aligned16(rope_cos) && aligned16(rope_sin), "rotary tables must be 16-byte aligned");
    MODDIT_CHECK_ARG(0 <= rope_lo && rope_lo <= rope_hi && rope_hi <= S, "rotary range [%d, %d) outside 0..%d",
                     rope_lo, rope_hi, S);
    MODDIT_CHECK_ARG(rope_form >= MODDIT_ROPE_ELEMENTWISE && rope_form <= MODDIT_ROPE_PAIR, "unknown rope_form %d",
                     rope_form);
    MODDIT_CHECK_ARG(static_cast<int64_t>(S) * D < (1ll << 31), "rotary tables of %d x %d values are too large", S, D);
  }
  const bool pooled = q_pool != nullptr || k_pool != nullptr;
  int bs = 128;
  if (pooled) {
    MODDIT_CHECK_ARG(block_size > 0 && dst_row0 % block_size == 0,
                     "block means need block_size > 0 and dst_row0 (%d) on a block boundary", dst_row0);
    // a short last block is only right at the very end of the output sequence: anywhere else the rows that
    // complete the block come from another call and this call's partial mean would be wrong
    MODDIT_CHECK_ARG(S % block_size == 0 || static_cast<int64_t>(dst_row0) + S == N_out,
                     "block means need S (%d) to be a multiple of block_size (%d) unless the rows end the output "
                     "sequence (dst_row0 + S = %lld, N_out = %d)", S, block_size,
                     static_cast<long long>(dst_row0) + S, N_out);
    bs = block_size;
  }
  MODDIT_CHECK_ARG(ceil_div(S, bs) <= 65535, "S / block_size must fit a grid dimension");
  float* ws = nullptr;
  if (norm_kind == MODDIT_NORM_RMS_ALL_HEADS) {
    MODDIT_CHECK_ARG(workspace != nullptr && ws_bytes >= moddit_qkv_prologue_workspace_bytes(B, S, norm_kind),
                     "workspace too small: %zu bytes needed", moddit_qkv_prologue_workspace_bytes(B, S, norm_kind));
    MODDIT_CHECK_ARG((reinterpret_cast<uintptr_t>(workspace) & 3u) == 0, "workspace must be 4-byte aligned");
    ws = static_cast<float*>(workspace);
  }
  if (int rc = require_sm100()) return rc;

  PrologueArgs a{};
  for (int i = 0; i < 3; ++i) { a.in[i] = ins[i]; a.out[i] = outs[i]; }
  a.weight[0] = q_weight; a.weight[1] = k_weight;
  a.bias[0] = q_bias; a.bias[1] = k_bias;
  a.inv_rms[0] = ws; a.inv_rms[1] = ws ? ws + static_cast<int64_t>(B) * S : nullptr;
  a.pool[0] = q_pool; a.pool[1] = k_pool;
  a.cos = rope_cos; a.sin = rope_sin;
  a.token_stride = token_stride;
  a.S = S; a.H = H; a.N_out = N_out; a.dst_row0 = dst_row0; a.bs = bs;
  a.nb_total = ceil_div(N_out, bs); a.blk_base = dst_row0 / bs;
  const int rows_per_pass = kThreads / (D / 8);      // short blocks: several per CTA, eight rows per thread
  a.group = (bs % rows_per_pass == 0 && (8 * rows_per_pass) % bs == 0) ? 8 * rows_per_pass / bs : 1;
  a.rope_form = rope_form; a.rope_lo = rope_lo; a.rope_hi = rope_hi;
  a.eps = eps;
  return dtype == MODDIT_BF16
             ? launch_prologue<__nv_bfloat16>(a, B, D, norm_kind, token_stride, ws, as_stream(stream))
             : launch_prologue<__half>(a, B, D, norm_kind, token_stride, ws, as_stream(stream));
}
