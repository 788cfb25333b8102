// The element-wise steps a linear-attention block runs right before and right after the delta-rule op, each as
// one pass over HBM in the layout the op reads ([B,T,H,D], token-major: no transposes in between):
//
//   short_conv_kernel     y = silu(causal depthwise conv1d(concat(cache, x)))       core/conv.py:13-68 followed by
//                         and the new conv cache                                     gated_deltanet.py:764-783
//   gate_act_kernel       g = -exp(A_log) softplus(a + bias), beta = sigmoid(b)      gated_deltanet.py:804-815,
//                                                                                    kda.py:120-172
//   gated_rmsnorm_kernel  y = o / sqrt(mean(o^2) + eps) * w * sigmoid(gate)          gated_deltanet.py:853-865,
//                         from o in either layout to [B,T,H,V]                       kda.py:664-700, common.py:42-53
//
// All three are bound by HBM: 16-byte accesses, fp32 arithmetic, grids of many small CTAs.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "dr_common.cuh"

namespace dr {
namespace blk {

// 16 bytes of activations as fp32 values: 8 bf16 or 4 fp32
template <int DT> struct Vec;
template <> struct Vec<DR_BF16> {
  static constexpr int N = 8;
  __device__ static void load(const void* base, int64_t idx, float (&f)[8]) {
    const uint4 r = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(base) + idx);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 p = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
      f[2 * i] = p.x; f[2 * i + 1] = p.y;
    }
  }
  __device__ static void store(void* base, int64_t idx, const float (&f)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 p = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&p);
    }
    *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(base) + idx) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <> struct Vec<DR_F32> {
  static constexpr int N = 4;
  __device__ static void load(const void* base, int64_t idx, float (&f)[4]) {
    const float4 r = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + idx);
    f[0] = r.x; f[1] = r.y; f[2] = r.z; f[3] = r.w;
  }
  __device__ static void store(void* base, int64_t idx, const float (&f)[4]) {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + idx) = make_float4(f[0], f[1], f[2], f[3]);
  }
};

__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float sigmoidf(float x) { return 1.f / (1.f + __expf(-x)); }
// log(1 + e^x) without overflow
__device__ __forceinline__ float softplusf(float x) { return fmaxf(x, 0.f) + log1pf(__expf(-fabsf(x))); }

// ---------------------------------------------------------------------------------------------------------
// Causal depthwise convolution over time, then SiLU.
//   xx = concat(cache [B,W-1,C], x [B,T,C]);  y[t] = bias + sum_j w[j] xx[t + j]  (w[W-1] meets x[t]);
//   new cache = the last W-1 rows of xx.  W == 1: y = x + bias, as the reference (its weight is not applied).
// A thread owns 16 bytes of channels and walks kConvTile time steps with the window in registers; consecutive
// threads own consecutive channels, so every access of a warp is one 512-byte row segment.
// ---------------------------------------------------------------------------------------------------------
constexpr int kConvTile = 32;
constexpr int kConvMaxW = 8;

struct ConvParams {
  const void* x; const float* w; const float* bias; const void* cache_in;
  void* y; void* cache_out;
  int B, T, C, W, apply_silu;
};

template <int DT, int MW>   // MW: compiled window bound (4 covers the blocks' kernel size, 8 the rest)
__global__ void __launch_bounds__(128) short_conv_kernel(const ConvParams p) {
  using VT = Vec<DT>;
  constexpr int N = VT::N;
  const int cvecs = p.C / N;
  const int cv = blockIdx.x * blockDim.x + threadIdx.x;
  if (cv >= cvecs) return;
  const int c0 = cv * N;
  const int b = blockIdx.z;
  const int t_begin = blockIdx.y * kConvTile, t_end = min(p.T, t_begin + kConvTile);
  const int W = p.W, H = W - 1;   // H: rows of history
  const int64_t xb = (int64_t)b * p.T * p.C, cb = (int64_t)b * H * p.C;

  float wt[MW][N], bias[N], win[MW][N];   // win[j] = xx[t + j] for the current t
#pragma unroll
  for (int i = 0; i < N; ++i) bias[i] = p.bias ? p.bias[c0 + i] : 0.f;
#pragma unroll
  for (int j = 0; j < MW; ++j)
#pragma unroll
    for (int i = 0; i < N; ++i) wt[j][i] = (j < W && W > 1) ? p.w[(int64_t)j * p.C + c0 + i] : (j == 0 ? 1.f : 0.f);

  // row r of xx (r = 0 .. H + T - 1): cache for r < H, else x[r - H]; missing cache = zeros
  auto load_row = [&](int r, float (&f)[N]) {
    if (r >= H) VT::load(p.x, xb + (int64_t)(r - H) * p.C + c0, f);
    else if (p.cache_in) VT::load(p.cache_in, cb + (int64_t)r * p.C + c0, f);
    else {
#pragma unroll
      for (int i = 0; i < N; ++i) f[i] = 0.f;
    }
  };
  // history of the first step of the tile
#pragma unroll
  for (int j = 0; j < MW - 1; ++j)
    if (j < H) load_row(t_begin + j, win[j]);
  // the last tile also owns the new cache: rows T .. T + H - 1 of xx, read before anything is written so that
  // a one-tile call (decode) may update its cache in place
  float keep[MW - 1][N];
  const bool last = t_end == p.T;
  if (last && p.cache_out) {
#pragma unroll
    for (int j = 0; j < MW - 1; ++j)
      if (j < H) load_row(p.T + j, keep[j]);
  }
  for (int t = t_begin; t < t_end; ++t) {
    float cur[N], acc[N];
    VT::load(p.x, xb + (int64_t)t * p.C + c0, cur);
#pragma unroll
    for (int i = 0; i < N; ++i) acc[i] = bias[i];
#pragma unroll
    for (int j = 0; j < MW - 1; ++j) {
      if (j < H) {
#pragma unroll
        for (int i = 0; i < N; ++i) acc[i] += wt[j][i] * win[j][i];
      }
    }
#pragma unroll
    for (int j = 0; j < MW; ++j) {   // the current step meets w[W-1]
      if (j == H) {
#pragma unroll
        for (int i = 0; i < N; ++i) acc[i] += wt[j][i] * cur[i];
      }
    }
    if (p.apply_silu) {
#pragma unroll
      for (int i = 0; i < N; ++i) acc[i] = silu(acc[i]);
    }
    VT::store(p.y, xb + (int64_t)t * p.C + c0, acc);
    // slide the window
#pragma unroll
    for (int j = 0; j < MW - 2; ++j) {
      if (j + 1 < H) {
#pragma unroll
        for (int i = 0; i < N; ++i) win[j][i] = win[j + 1][i];
      }
    }
#pragma unroll
    for (int j = 0; j < MW - 1; ++j) {
      if (j == H - 1) {
#pragma unroll
        for (int i = 0; i < N; ++i) win[j][i] = cur[i];
      }
    }
  }
  if (last && p.cache_out) {
#pragma unroll
    for (int j = 0; j < MW - 1; ++j)
      if (j < H) VT::store(p.cache_out, cb + (int64_t)j * p.C + c0, keep[j]);
  }
}

inline cudaError_t launch_short_conv(const ConvParams& p, int dt, cudaStream_t stream) {
  const int n = dt == DR_BF16 ? 8 : 4;
  const int cvecs = p.C / n;
  dim3 grid((cvecs + 127) / 128, (p.T + kConvTile - 1) / kConvTile, p.B);
  if (dt == DR_BF16) {
    if (p.W <= 4) short_conv_kernel<DR_BF16, 4><<<grid, 128, 0, stream>>>(p);
    else short_conv_kernel<DR_BF16, kConvMaxW><<<grid, 128, 0, stream>>>(p);
  } else {
    if (p.W <= 4) short_conv_kernel<DR_F32, 4><<<grid, 128, 0, stream>>>(p);
    else short_conv_kernel<DR_F32, kConvMaxW><<<grid, 128, 0, stream>>>(p);
  }
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------------------
// Gate activations.  mode 0 (Gated DeltaNet): a, b [B,T,H] ->
//     g = -exp(A_log[h]) softplus(a + dt_bias[h]),  beta = sigmoid(b) (x2 with allow_neg_eigval)
// mode 1 (KDA, kda_gate): graw [B,T,H*K] (+ g_bias[H*K]) ->
//     g = -exp(A_log[h]) (x > threshold ? x : softplus(x)),  beta = sigmoid(b)
// Outputs fp32, token-major ([B,T,H] / [B,T,H,K]): the layout DR_LAYOUT_BTHD reads.
// ---------------------------------------------------------------------------------------------------------
struct GateParams {
  const void* a; const void* b; const float* A_log; const float* bias;
  float* g; float* beta;
  int64_t n_g, n_beta;   // elements of g and of beta
  int H, K;              // K = 1 in mode 0
  int a_dt, b_dt, mode;
  float beta_scale, threshold;
};

__global__ void __launch_bounds__(256) gate_act_kernel(const GateParams p) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < p.n_g) {
    const int hk = (int)(i % ((int64_t)p.H * p.K));   // position inside a token: h * K + k
    const int h = hk / p.K;
    float x = ld_elem(p.a, i, p.a_dt);
    if (p.bias) x += p.bias[p.mode == 0 ? h : hk];
    const float sp = (p.mode == 1 && x > p.threshold) ? x : softplusf(x);
    p.g[i] = -expf(p.A_log[h]) * sp;
  }
  if (p.beta && i < p.n_beta) p.beta[i] = p.beta_scale * (1.f / (1.f + expf(-ld_elem(p.b, i, p.b_dt))));
}

inline cudaError_t launch_gate_act(const GateParams& p, cudaStream_t stream) {
  const int64_t n = p.n_g > p.n_beta ? p.n_g : p.n_beta;
  gate_act_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(p);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------------------
// Per-head RMSNorm of the op's output with the sigmoid gate, written token-major for the output projection:
//   y[b,t,h,:] = o[b,h,t,:] / sqrt(mean(o^2) + eps) * w * sigmoid(gate[b,t,h,:])      (gate optional)
// One warp per (b,t,h) row; o is read through SeqMap in either layout, so the transpose the reference does
// before the norm costs nothing.  V is a multiple of the 16-byte vector, at most 512.
// ---------------------------------------------------------------------------------------------------------
template <int DT>
__device__ __forceinline__ void ld4(const void* base, int64_t idx, float (&f)[4]) {
  if constexpr (DT == DR_BF16) {
    const uint2 r = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(base) + idx);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
  } else {
    const float4 r = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + idx);
    f[0] = r.x; f[1] = r.y; f[2] = r.z; f[3] = r.w;
  }
}
template <int DT>
__device__ __forceinline__ void st4(void* base, int64_t idx, const float (&f)[4]) {
  if constexpr (DT == DR_BF16) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
    uint2 r;
    r.x = *reinterpret_cast<const uint32_t*>(&a); r.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(base) + idx) = r;
  } else {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + idx) = make_float4(f[0], f[1], f[2], f[3]);
  }
}

struct NormParams {
  const void* o; const void* gate; const float* w; void* y;
  SeqMap map;
  int V; float eps;
};

template <int ODT, int GDT, int YDT>
__global__ void __launch_bounds__(256) gated_rmsnorm_kernel(const NormParams p) {
  constexpr int N = 4;   // every lane owns groups of 4 consecutive columns: 8- or 16-byte accesses
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);   // (b, t, h) flattened
  const int64_t nrows = (int64_t)p.map.B * p.map.T * p.map.H;
  if (row >= nrows) return;
  const int h = (int)(row % p.map.H);
  const int64_t bt = row / p.map.H;
  const int t = (int)(bt % p.map.T), b = (int)(bt / p.map.T);
  const int V = p.V;
  const int64_t src = p.map.base(b, h, V) + (int64_t)t * p.map.tok(V);
  const int64_t dst = row * V;
  float x[4][N];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = N * lane + 128 * i;
#pragma unroll
    for (int e = 0; e < N; ++e) x[i][e] = 0.f;
    if (c < V) {
      ld4<ODT>(p.o, src + c, x[i]);
#pragma unroll
      for (int e = 0; e < N; ++e) ss += x[i][e] * x[i][e];
    }
  }
  ss = warp_sum(ss);
  const float r = 1.f / sqrtf(ss / (float)V + p.eps);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = N * lane + 128 * i;
    if (c < V) {
      const float4 w4 = *reinterpret_cast<const float4*>(p.w + c);
      float gt[N] = {0.f, 0.f, 0.f, 0.f}, yv[N];
      if (p.gate) ld4<GDT>(p.gate, dst + c, gt);
      yv[0] = x[i][0] * r * w4.x; yv[1] = x[i][1] * r * w4.y; yv[2] = x[i][2] * r * w4.z; yv[3] = x[i][3] * r * w4.w;
      if (p.gate) {
#pragma unroll
        for (int e = 0; e < N; ++e) yv[e] *= sigmoidf(gt[e]);
      }
      st4<YDT>(p.y, dst + c, yv);
    }
  }
}

inline cudaError_t launch_gated_rmsnorm(const NormParams& p, int odt, int gdt, int ydt, cudaStream_t stream) {
  const int64_t nrows = (int64_t)p.map.B * p.map.T * p.map.H;
  const unsigned grid = (unsigned)((nrows + 7) / 8);
#define DR_NORM_CASE(O, G, Y) \
  if (odt == O && gdt == G && ydt == Y) { gated_rmsnorm_kernel<O, G, Y><<<grid, 256, 0, stream>>>(p); return cudaGetLastError(); }
  DR_NORM_CASE(DR_BF16, DR_BF16, DR_BF16)
  DR_NORM_CASE(DR_F32, DR_F32, DR_F32)
  DR_NORM_CASE(DR_F32, DR_BF16, DR_BF16)
  DR_NORM_CASE(DR_BF16, DR_F32, DR_BF16)
  DR_NORM_CASE(DR_F32, DR_BF16, DR_F32)
  DR_NORM_CASE(DR_BF16, DR_BF16, DR_F32)
  DR_NORM_CASE(DR_BF16, DR_F32, DR_F32)
  DR_NORM_CASE(DR_F32, DR_F32, DR_BF16)
#undef DR_NORM_CASE
  return cudaErrorInvalidValue;
}

}  // namespace blk
}  // namespace dr
