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
  __device__ static uint4 raw(const void* base, int64_t idx) {
    return *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(base) + idx);
  }
  __device__ static void load(const void* base, int64_t idx, float (&f)[8]) { cvt(raw(base, idx), f); }
  __device__ static void cvt(const uint4 r, float (&f)[8]) {
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
  __device__ static uint4 raw(const void* base, int64_t idx) {
    return *reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(base) + idx);
  }
  __device__ static void load(const void* base, int64_t idx, float (&f)[4]) { cvt(raw(base, idx), f); }
  __device__ static void cvt(const uint4 r, float (&f)[4]) {
    f[0] = __uint_as_float(r.x); f[1] = __uint_as_float(r.y); f[2] = __uint_as_float(r.z); f[3] = __uint_as_float(r.w);
  }
  __device__ static void store(void* base, int64_t idx, const float (&f)[4]) {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + idx) = make_float4(f[0], f[1], f[2], f[3]);
  }
};

__device__ __forceinline__ float silu(float x) { return __fdividef(x, 1.f + __expf(-x)); }
__device__ __forceinline__ float sigmoidf(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }
// log(1 + e^x) without overflow
__device__ __forceinline__ float softplusf(float x) { return fmaxf(x, 0.f) + log1pf(__expf(-fabsf(x))); }

// ---------------------------------------------------------------------------------------------------------
// Causal depthwise convolution over time, then SiLU.
//   xx = concat(cache [B,W-1,C], x [B,T,C]);  y[t] = bias + sum_j w[j] xx[t + j]  (w[W-1] meets x[t]);
//   new cache = the last W-1 rows of xx.  W == 1: y = x + bias, as the reference (its weight is not applied).
// A thread produces kConvSteps consecutive time steps of 16 bytes of channels (8 bf16 / 4 fp32): it fetches the
// kConvSteps + W - 1 rows it needs (all loads issued before the first use; the W - 1 rows shared with the thread
// before it come from L1/L2), so there is no serial walk and the SM holds many small independent threads.
// ---------------------------------------------------------------------------------------------------------
constexpr int kConvSteps = 4;   // time steps per thread (measured best of 2, 3, 4, 8); also the longest T whose cache may be updated in place
constexpr int kConvMaxW = 8;

struct ConvParams {
  const void* x; const float* w; const float* bias; const void* cache_in;
  void* y; void* cache_out;
  int B, T, C, W, apply_silu;
};

// 16 bytes of channels per thread: 8 bf16 or 4 fp32
template <int DT> using ConvVec = Vec<DT>;

template <int DT, int MW, bool EXACT>   // EXACT: the window is MW (compiled for 1..4); else any window up to MW
__global__ void __launch_bounds__(128) short_conv_kernel(const ConvParams p) {
  using Q = ConvVec<DT>;
  using Raw = uint4;
  constexpr int N = Q::N, HW = MW - 1, ROWS = kConvSteps + HW;
  const int cv = blockIdx.x * 32 + (threadIdx.x & 31);
  const int t0 = (blockIdx.y * 4 + (threadIdx.x >> 5)) * kConvSteps;
  if (cv >= p.C / N || t0 >= p.T) return;
  const int c0 = cv * N;
  const int b = blockIdx.z;
  const int W = EXACT ? MW : p.W, H = W - 1;   // H: rows of history
  const int64_t xb = (int64_t)b * p.T * p.C + c0, cb = (int64_t)b * H * p.C + c0;

  // rows t0 .. t0 + kConvSteps - 1 + H of xx = concat(cache, x): cache (zeros if absent) for r < H, else x[r - H]
  Raw raw[ROWS];
#pragma unroll
  for (int w = 0; w < ROWS; ++w) {
    const int r = t0 + w;
    raw[w] = Raw{};
    if (w < kConvSteps + H) {
      if (r >= H) { if (r - H < p.T) raw[w] = Q::raw(p.x, xb + (int64_t)(r - H) * p.C); }
      else if (p.cache_in) raw[w] = Q::raw(p.cache_in, cb + (int64_t)r * p.C);
    }
  }
  float wt[MW][N], bias[N];
  {
#pragma unroll
    for (int q4 = 0; q4 < N; q4 += 4) {
      const float4 b4 = p.bias ? *reinterpret_cast<const float4*>(p.bias + c0 + q4) : make_float4(0.f, 0.f, 0.f, 0.f);
      bias[q4] = b4.x; bias[q4 + 1] = b4.y; bias[q4 + 2] = b4.z; bias[q4 + 3] = b4.w;
    }
  }
#pragma unroll
  for (int j = 0; j < MW; ++j) {
#pragma unroll
    for (int q4 = 0; q4 < N; q4 += 4) {
      float4 w4 = make_float4(j == 0 ? 1.f : 0.f, j == 0 ? 1.f : 0.f, j == 0 ? 1.f : 0.f, j == 0 ? 1.f : 0.f);
      if (j < W && W > 1) w4 = *reinterpret_cast<const float4*>(p.w + (int64_t)j * p.C + c0 + q4);
      wt[j][q4] = w4.x; wt[j][q4 + 1] = w4.y; wt[j][q4 + 2] = w4.z; wt[j][q4 + 3] = w4.w;
    }
  }
  float row[ROWS][N];
#pragma unroll
  for (int w = 0; w < ROWS; ++w) Q::cvt(raw[w], row[w]);
#pragma unroll
  for (int u = 0; u < kConvSteps; ++u) {
    if (t0 + u < p.T) {
      float acc[N];
#pragma unroll
      for (int i = 0; i < N; ++i) acc[i] = bias[i];
#pragma unroll
      for (int j = 0; j < MW; ++j) {
        if (j < W) {
#pragma unroll
          for (int i = 0; i < N; ++i) acc[i] += wt[j][i] * row[u + j][i];
        }
      }
      if (p.apply_silu) {
#pragma unroll
        for (int i = 0; i < N; ++i) acc[i] = silu(acc[i]);
      }
      Q::store(p.y, xb + (int64_t)(t0 + u) * p.C, acc);
    }
  }
  // the thread that holds the end of the sequence also holds the new cache: rows T .. T + H - 1 of xx
  if (p.cache_out && t0 + kConvSteps >= p.T) {
#pragma unroll
    for (int w = 0; w < ROWS; ++w) {
      const int j = t0 + w - p.T;
      if (j >= 0 && j < H) Q::store(p.cache_out, cb + (int64_t)j * p.C, row[w]);
    }
  }
}

inline cudaError_t launch_short_conv(const ConvParams& p, int dt, cudaStream_t stream) {
  const int cvecs = p.C / (dt == DR_BF16 ? 8 : 4);
  dim3 grid((cvecs + 31) / 32, (p.T + 4 * kConvSteps - 1) / (4 * kConvSteps), p.B);
#define DR_CONV_CASE(DT)                                                                        \
  switch (p.W) {                                                                                \
    case 1: short_conv_kernel<DT, 1, true><<<grid, 128, 0, stream>>>(p); break;                 \
    case 2: short_conv_kernel<DT, 2, true><<<grid, 128, 0, stream>>>(p); break;                 \
    case 3: short_conv_kernel<DT, 3, true><<<grid, 128, 0, stream>>>(p); break;                 \
    case 4: short_conv_kernel<DT, 4, true><<<grid, 128, 0, stream>>>(p); break;                 \
    default: short_conv_kernel<DT, kConvMaxW, false><<<grid, 128, 0, stream>>>(p); break;       \
  }
  if (dt == DR_BF16) { DR_CONV_CASE(DR_BF16) } else { DR_CONV_CASE(DR_F32) }
#undef DR_CONV_CASE
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

// V = 128 (the blocks' head size): 16 lanes x 8 columns per row, two rows per warp and pass, two passes with every
// load of both issued before the first reduction (one 16-lane butterfly per row).
template <int DT>
__device__ __forceinline__ void ld8(const void* base, int64_t idx, float (&f)[8]) {
  if constexpr (DT == DR_BF16) {
    Vec<DR_BF16>::load(base, idx, f);
  } else {
    float a[4], b[4];
    Vec<DR_F32>::load(base, idx, a); Vec<DR_F32>::load(base, idx + 4, b);
#pragma unroll
    for (int i = 0; i < 4; ++i) { f[i] = a[i]; f[4 + i] = b[i]; }
  }
}
template <int DT>
__device__ __forceinline__ void st8(void* base, int64_t idx, const float (&f)[8]) {
  if constexpr (DT == DR_BF16) {
    Vec<DR_BF16>::store(base, idx, f);
  } else {
    const float a[4] = {f[0], f[1], f[2], f[3]}, b[4] = {f[4], f[5], f[6], f[7]};
    Vec<DR_F32>::store(base, idx, a); Vec<DR_F32>::store(base, idx + 4, b);
  }
}

constexpr int kNormRowsPerWarp = 4;

template <int ODT, int GDT, int YDT>
__global__ void __launch_bounds__(256) gated_rmsnorm_v128_kernel(const NormParams p) {
  constexpr int V = 128, P = kNormRowsPerWarp / 2;
  const int lane = threadIdx.x & 31, sub = lane >> 4, c = (lane & 15) * 8;
  const int64_t nrows = (int64_t)p.map.B * p.map.T * p.map.H;
  const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const float4 w0 = *reinterpret_cast<const float4*>(p.w + c), w1 = *reinterpret_cast<const float4*>(p.w + c + 4);
  const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
  // a few resident CTAs per SM walk the rows: no CTA start-up per 32 rows
  for (int64_t warp_id = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
       warp_id * kNormRowsPerWarp < nrows; warp_id += nwarps) {
  float x[P][8], gt[P][8];
  int64_t dst[P];
  bool live[P];
  uint32_t h0 = 0, tt0 = 0, b0 = 0;   // (b, t, h) of the warp's first row
  if (!p.map.bthd) {
    const uint32_t r32 = (uint32_t)(warp_id * kNormRowsPerWarp), bt = r32 / (uint32_t)p.map.H;
    h0 = r32 % (uint32_t)p.map.H; tt0 = bt % (uint32_t)p.map.T; b0 = bt / (uint32_t)p.map.T;
  }
#pragma unroll
  for (int i = 0; i < P; ++i) {
    const int64_t row = warp_id * kNormRowsPerWarp + 2 * i + sub;
    live[i] = row < nrows;
    dst[i] = row * V + c;
#pragma unroll
    for (int e = 0; e < 8; ++e) { x[i][e] = 0.f; gt[i][e] = 0.f; }
    if (live[i]) {
      int64_t src = dst[i];   // token-major o: the same place as y
      if (!p.map.bthd) {      // (rows < 2^31, checked by the caller: 32-bit divisions, once per warp and pass)
        const uint32_t H32 = (uint32_t)p.map.H, T32 = (uint32_t)p.map.T;
        uint32_t h = h0 + 2 * i + sub, t = tt0, b = b0;
        while (h >= H32) { h -= H32; ++t; }
        while (t >= T32) { t -= T32; ++b; }
        src = (((int64_t)b * H32 + h) * T32 + t) * V + c;
      }
      ld8<ODT>(p.o, src, x[i]);
      if (p.gate) ld8<GDT>(p.gate, dst[i], gt[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < P; ++i) {
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += x[i][e] * x[i][e];
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float r = 1.f / sqrtf(ss * (1.f / V) + p.eps);
    float y[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      y[e] = x[i][e] * r * wv[e];
      if (p.gate) y[e] *= sigmoidf(gt[i][e]);
    }
    if (live[i]) st8<YDT>(p.y, dst[i], y);
  }
  }
}

inline cudaError_t launch_gated_rmsnorm(const NormParams& p, int odt, int gdt, int ydt, int sms, cudaStream_t stream) {
  const int64_t nrows = (int64_t)p.map.B * p.map.T * p.map.H;
  const unsigned grid = (unsigned)((nrows + 7) / 8);
  const int64_t want128 = (nrows + 8 * kNormRowsPerWarp - 1) / (8 * kNormRowsPerWarp);
  const unsigned grid128 = (unsigned)(want128 < (int64_t)sms * 8 ? want128 : (int64_t)sms * 8);
#define DR_NORM_CASE(O, G, Y)                                                              \
  if (odt == O && gdt == G && ydt == Y) {                                                  \
    if (p.V == 128) gated_rmsnorm_v128_kernel<O, G, Y><<<grid128, 256, 0, stream>>>(p);    \
    else gated_rmsnorm_kernel<O, G, Y><<<grid, 256, 0, stream>>>(p);                       \
    return cudaGetLastError();                                                             \
  }
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
