// Attention prologue: what the reference's processors do between the q/k/v projections and the attention call
// (per-head or whole-row normalisation of q and k, rotary embedding of the latent tokens, the move from the
// projections' token-major layout to the head-major layout of the attention kernels), in one pass over
// the data.  Follows MoD/models/hunyuan/attention_processor.py:57-106, MoD/models/wan/attention_processor.py:70-93
// and 123-125, MoD/models/cogvideox/attention_processor.py:113-135.
//
// One CTA = one block of `block_size` tokens of one head of one of the three tensors.  D/8 threads cover a row
// with one 16-byte load each (a 2*D-byte piece of the token's row), so the row statistics are a shuffle
// reduction over D/8 lanes and a rotary pair never leaves its thread; the head-major store is contiguous
// over the whole block.  Thread-to-row mapping and summation order of the optional block means are those of
// pool_blocks_kernel, so the means equal the ones pooled afterwards from the stored tensor bit for bit.
// Bound: HBM.  Algorithmic bytes per token and tensor: 2*H*D read + 2*H*D written (+ the rotary tables:
// 8*D bytes per token, shared by the heads through L2).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace moddit {
namespace {

constexpr int kThreads = 256;

template <typename T>
struct Cvt;
template <>
struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ float up(uint16_t b) { return __uint_as_float(static_cast<uint32_t>(b) << 16); }
  static __device__ __forceinline__ uint16_t down(float f) { return __bfloat16_as_ushort(__float2bfloat16_rn(f)); }
};
template <>
struct Cvt<__half> {
  static __device__ __forceinline__ float up(uint16_t b) { return __half2float(__ushort_as_half(b)); }
  static __device__ __forceinline__ uint16_t down(float f) { return __half_as_ushort(__float2half_rn(f)); }
};

template <typename T>
__device__ __forceinline__ void unpack(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = Cvt<T>::up(static_cast<uint16_t>(w[i] & 0xffffu));
    f[2 * i + 1] = Cvt<T>::up(static_cast<uint16_t>(w[i] >> 16));
  }
}

// Rounds to T and returns the rounded values in f as well.
template <typename T>
__device__ __forceinline__ uint4 pack_round(float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint16_t lo = Cvt<T>::down(f[2 * i]);
    const uint16_t hi = Cvt<T>::down(f[2 * i + 1]);
    f[2 * i] = Cvt<T>::up(lo);
    f[2 * i + 1] = Cvt<T>::up(hi);
    w[i] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

template <typename T>
__device__ __forceinline__ float round_to(float f) {
  return Cvt<T>::up(Cvt<T>::down(f));
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
  int norm_kind, rope_form, rope_lo, rope_hi;
  float eps;
};

template <typename T, int D>
__global__ void __launch_bounds__(kThreads) qkv_prologue_kernel(const __grid_constant__ PrologueArgs a) {
  constexpr int kTpr = D / 8;               // threads per row
  constexpr int kRpp = kThreads / kTpr;     // rows per pass
  __shared__ float red[kRpp][D];

  const int which = blockIdx.z % 3;
  const int b = blockIdx.z / 3;
  const T* __restrict__ in = static_cast<const T*>(a.in[which]);
  if (in == nullptr) return;
  T* __restrict__ out = static_cast<T*>(a.out[which]);
  const int blk = blockIdx.x;
  const int h = blockIdx.y;
  const int row0 = blk * a.bs;
  const int rows = min(a.bs, a.S - row0);
  const int cg = threadIdx.x % kTpr;
  const int rg = threadIdx.x / kTpr;
  const int norm = which < 2 ? a.norm_kind : MODDIT_NORM_NONE;
  const bool rope_on = which < 2 && a.cos != nullptr;
  float* pool = which < 2 ? a.pool[which] : nullptr;

  // weight and bias of this thread's eight columns, kept as floats
  float wv[8], bv[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) { wv[i] = 1.f; bv[i] = 0.f; }
  if (norm != MODDIT_NORM_NONE) {
    const int wofs = (norm == MODDIT_NORM_RMS_ALL_HEADS ? h * D : 0) + cg * 8;
    if (a.weight[which] != nullptr)
      unpack<T>(__ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(a.weight[which]) + wofs)), wv);
    if (norm == MODDIT_NORM_LAYER && a.bias[which] != nullptr)
      unpack<T>(__ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(a.bias[which]) + wofs)), bv);
  }
  const bool has_w = norm != MODDIT_NORM_NONE && a.weight[which] != nullptr;

  const T* src = in + (static_cast<int64_t>(b) * a.S + row0) * a.token_stride + h * D + cg * 8;
  T* dst = out + ((static_cast<int64_t>(b) * a.H + h) * a.N_out + a.dst_row0 + row0) * D + cg * 8;

  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int base = 0; base < rows; base += 8 * kRpp) {   // uniform trip count: the shuffles below need every lane
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int r = base + rg + u * kRpp;
      v[u] = r < rows ? __ldg(reinterpret_cast<const uint4*>(src + static_cast<int64_t>(r) * a.token_stride))
                      : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int r = base + rg + u * kRpp;
      const bool valid = r < rows;
      const int s = row0 + r;               // token index within the input
      float f[8];
      unpack<T>(v[u], f);
      if (norm == MODDIT_NORM_RMS_HEAD || norm == MODDIT_NORM_RMS_ALL_HEADS) {
        float rs;
        if (norm == MODDIT_NORM_RMS_HEAD) {
          float ss = 0.f;
#pragma unroll
          for (int i = 0; i < 8; ++i) ss = fmaf(f[i], f[i], ss);
          ss = row_sum<kTpr>(ss);
          rs = __frsqrt_rn(__fadd_rn(ss / static_cast<float>(D), a.eps));
        } else {
          rs = valid ? __ldg(a.inv_rms[which] + static_cast<int64_t>(b) * a.S + s) : 0.f;
        }
        // x * rsqrt in float32, rounded to T, then the product with the weight rounded to T again
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          f[i] = __fmul_rn(f[i], rs);
          if (has_w) f[i] = __fmul_rn(round_to<T>(f[i]), wv[i]);
          f[i] = round_to<T>(f[i]);
        }
      } else if (norm == MODDIT_NORM_LAYER) {
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) sum += f[i];
        const float mean = row_sum<kTpr>(sum) / static_cast<float>(D);
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float d = f[i] - mean;
          ss = fmaf(d, d, ss);
        }
        const float rstd = __frsqrt_rn(__fadd_rn(row_sum<kTpr>(ss) / static_cast<float>(D), a.eps));
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = round_to<T>(fmaf((f[i] - mean) * rstd, wv[i], bv[i]));
      }
      if (rope_on && valid && s >= a.rope_lo && s < a.rope_hi) {
        const int64_t t = (static_cast<int64_t>(s - a.rope_lo)) * D + cg * 8;
        float c[8], sn[8];
        *reinterpret_cast<float4*>(c) = __ldg(reinterpret_cast<const float4*>(a.cos + t));
        *reinterpret_cast<float4*>(c + 4) = __ldg(reinterpret_cast<const float4*>(a.cos + t + 4));
        *reinterpret_cast<float4*>(sn) = __ldg(reinterpret_cast<const float4*>(a.sin + t));
        *reinterpret_cast<float4*>(sn + 4) = __ldg(reinterpret_cast<const float4*>(a.sin + t + 4));
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float x0 = f[2 * i], x1 = f[2 * i + 1];
          // products rounded separately, then one add (no fused multiply-add), as a tensor expression does
          const float ce = c[2 * i];
          const float co = a.rope_form == MODDIT_ROPE_EVEN_COS_ODD_SIN ? c[2 * i] : c[2 * i + 1];
          const float se = a.rope_form == MODDIT_ROPE_EVEN_COS_ODD_SIN ? sn[2 * i + 1] : sn[2 * i];
          const float so = sn[2 * i + 1];
          f[2 * i] = __fsub_rn(__fmul_rn(x0, ce), __fmul_rn(x1, se));
          f[2 * i + 1] = __fadd_rn(__fmul_rn(x0, so), __fmul_rn(x1, co));
        }
      }
      const uint4 o = pack_round<T>(f);
      if (valid) *reinterpret_cast<uint4*>(dst + static_cast<int64_t>(r) * D) = o;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += valid ? f[i] : 0.f;
    }
  }
  if (pool == nullptr) return;
#pragma unroll
  for (int i = 0; i < 8; ++i) red[rg][cg * 8 + i] = acc[i];
  __syncthreads();
  if (threadIdx.x < D) {
    float s = 0.f;
#pragma unroll 8
    for (int g = 0; g < kRpp; ++g) s += red[g][threadIdx.x];
    pool[((static_cast<int64_t>(b) * a.H + h) * a.nb_total + a.blk_base + blk) * D + threadIdx.x] =
        s / static_cast<float>(rows);
  }
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
  if (lane == 0) out[tok] = __frsqrt_rn(__fadd_rn(ss / static_cast<float>(width), eps));
}

template <typename T>
int launch_prologue(const PrologueArgs& a, int B, int D, bool across, int64_t token_stride, float* ws,
                    cudaStream_t st) {
  if (across) {
    const int64_t tokens = static_cast<int64_t>(B) * a.S;
    const dim3 grid(static_cast<unsigned>((tokens + kThreads / 32 - 1) / (kThreads / 32)), 2);
    token_inv_rms_kernel<T><<<grid, kThreads, 0, st>>>(static_cast<const T*>(a.in[0]), static_cast<const T*>(a.in[1]),
                                                       tokens, token_stride, a.H * D, a.eps, ws, ws + tokens);
    MODDIT_CHECK_LAUNCH("token_inv_rms_kernel");
  }
  const dim3 grid(ceil_div(a.S, a.bs), a.H, 3 * B);
  if (D == 64)
    qkv_prologue_kernel<T, 64><<<grid, kThreads, 0, st>>>(a);
  else
    qkv_prologue_kernel<T, 128><<<grid, kThreads, 0, st>>>(a);
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
  MODDIT_CHECK_ARG(H <= 65535 && 3 * static_cast<int64_t>(B) <= 65535, "H and 3*B must fit a grid dimension");
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
    MODDIT_CHECK_ARG(rope_form == MODDIT_ROPE_ELEMENTWISE || rope_form == MODDIT_ROPE_EVEN_COS_ODD_SIN,
                     "unknown rope_form %d", rope_form);
  }
  const bool pooled = q_pool != nullptr || k_pool != nullptr;
  int bs = 128;
  if (pooled) {
    MODDIT_CHECK_ARG(block_size > 0 && dst_row0 % block_size == 0,
                     "block means need block_size > 0 and dst_row0 (%d) on a block boundary", dst_row0);
    bs = block_size;
  }
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
  a.norm_kind = norm_kind; a.rope_form = rope_form; a.rope_lo = rope_lo; a.rope_hi = rope_hi;
  a.eps = eps;
  const bool across = norm_kind == MODDIT_NORM_RMS_ALL_HEADS;
  return dtype == MODDIT_BF16
             ? launch_prologue<__nv_bfloat16>(a, B, D, across, token_stride, ws, as_stream(stream))
             : launch_prologue<__half>(a, B, D, across, token_stride, ws, as_stream(stream));
}
