// Token-by-token scans whose state is a [key, value] matrix with a per-token diagonal decay and rank-one
// writes: the RWKV-7 diagonal-plus-low-rank rule, the RWKV-6 rule with its current-token bonus, and the
// Mamba-2 SSD rule (scalar decay per head and token, B as key, C as query, state stored [value, key]).
//
// Same skeleton as the delta-rule recurrence: one CTA of 128 threads owns 32 value columns of one
// (batch, head) state, four adjacent lanes share a column and split the key axis, so each reduction over
// the key axis is a thread-local sum finished by two warp shuffles; the token vectors are staged in shared
// memory one token ahead (fetch to registers before the arithmetic of the current token, commit after it),
// one __syncthreads per token.  The per-token transforms of the inputs (exp of the log decay, the sigmoid of
// the receptance, softplus and clamp of dt) are applied once per element at the commit.
#pragma once

#include "dr_common.cuh"

namespace dr {

enum { LR_DPLR = 0, LR_RWKV6 = 1, LR_SSD = 2 };

// One per-token vector (or scalar) of a tensor with unit feature stride.
struct LrVec {
  const void* p;
  int64_t sb, sh, st;  // element strides over batch, head, token
  int dt;              // DrDtype
  int hdiv;            // head h reads row h / hdiv (grouped B and C of the SSD)
  __device__ __forceinline__ int64_t at(int b, int h, int t) const {
    return (int64_t)b * sb + (int64_t)(h / hdiv) * sh + (int64_t)t * st;
  }
};

struct LinRecParams {
  LrVec q, k, w, a, b;  // key axis: query / key / log decay / the two low-rank vectors
  LrVec v;              // value axis
  LrVec dt;             // SSD: one scalar per token and head
  void* o;              // output, addressed like v with its own strides
  int64_t o_sb, o_sh, o_st;
  int o_dt;
  const float* u;        // RWKV-6 bonus [H, K]
  const float* A;        // SSD [H]
  const float* D;        // SSD [H]
  const float* dt_bias;  // SSD [H] or null
  const float* h0;       // null: zero state
  float* hT;             // null: not wanted (may alias h0: every thread reads its entries before it writes them)
  int64_t s_k, s_v;      // state entry (key kk, value vv) of unit n at n*K*V + kk*s_k + vv*s_v
  int B, H, T, K, V;
  float scale, dt_lo, dt_hi;
};

constexpr int kLrThreads = 128;
constexpr int kLrCols = 32;

__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }

template <int KIND, int KP>
__global__ void __launch_bounds__(kLrThreads) linrec_kernel(const LinRecParams p) {
  constexpr int NV = KIND == LR_DPLR ? 5 : (KIND == LR_RWKV6 ? 3 : 2);  // staged key-axis vectors: q k [w [a b]]
  constexpr int KPP = KP + 1;
  constexpr int KS = 4 * KPP;
  __shared__ float s_vec[2][NV][KS];
  __shared__ float s_v[2][kLrCols];
  __shared__ float s_sc[2][2];   // SSD: decay exp(A dt), dt

  const int K = p.K, V = p.V, T = p.T;
  const int tid = threadIdx.x;
  const int col = tid >> 2, part = tid & 3;
  const int nvs = (V + kLrCols - 1) / kLrCols;
  const int unit = blockIdx.x / nvs;
  const int v0 = (blockIdx.x % nvs) * kLrCols;
  const int b = unit / p.H, h = unit % p.H;
  const int vcol = v0 + col;
  const bool vok = vcol < V;

  const LrVec* vecs[5] = {&p.q, &p.k, &p.w, &p.a, &p.b};
  int64_t base[NV];
#pragma unroll
  for (int j = 0; j < NV; ++j) base[j] = vecs[j]->at(b, h, 0);
  const int64_t v_base = p.v.at(b, h, 0);
  const int64_t o_base = (int64_t)b * p.o_sb + (int64_t)h * p.o_sh;
  const int64_t dt_base = KIND == LR_SSD ? p.dt.at(b, h, 0) : 0;
  const float A_h = KIND == LR_SSD ? p.A[h] : 0.f;
  const float D_h = KIND == LR_SSD ? p.D[h] : 0.f;
  const float bias_h = (KIND == LR_SSD && p.dt_bias) ? p.dt_bias[h] : 0.f;

  float S[KP], ur[KIND == LR_RWKV6 ? KP : 1];
  const int64_t s_unit = (int64_t)unit * K * V;
#pragma unroll
  for (int i = 0; i < KP; ++i) {
    const int kk = part * KP + i;
    S[i] = (p.h0 && vok && kk < K) ? p.h0[s_unit + kk * p.s_k + vcol * p.s_v] : 0.f;
    if (KIND == LR_RWKV6) ur[i] = kk < K ? p.u[(int64_t)h * K + kk] : 0.f;
  }

  constexpr int NS = (4 * KP + kLrThreads - 1) / kLrThreads;
  float f[NV][NS], f_x = 0.f;
  auto fetch = [&](int t) {
#pragma unroll
    for (int j = 0; j < NV; ++j)
#pragma unroll
      for (int s = 0; s < NS; ++s) {
        const int i = tid + s * kLrThreads;
        f[j][s] = i < K ? ld_elem(vecs[j]->p, base[j] + t * vecs[j]->st + i, vecs[j]->dt) : 0.f;
      }
    if (tid < kLrCols)
      f_x = (v0 + tid < V) ? ld_elem(p.v.p, v_base + t * p.v.st + v0 + tid, p.v.dt) : 0.f;
    else if (KIND == LR_SSD && tid == kLrCols)
      f_x = ld_elem(p.dt.p, dt_base + t * p.dt.st, p.dt.dt);
  };
  auto commit = [&](int buf) {
#pragma unroll
    for (int s = 0; s < NS; ++s) {
      const int i = tid + s * kLrThreads;
      if (i < 4 * KP) {
        const int phys = i + i / KP;
        const bool in = i < K;
        float qv = f[0][s];
        if (KIND == LR_RWKV6) qv = in ? p.scale / (1.f + expf(-qv)) : 0.f;   // sigmoid(r) * scale
        if (KIND == LR_DPLR) qv *= p.scale;
        s_vec[buf][0][phys] = qv;
        s_vec[buf][1][phys] = f[1][s];
        if (KIND == LR_DPLR) {
          s_vec[buf][2][phys] = expf(f[2][s]);
          s_vec[buf][3][phys] = f[3][s];
          s_vec[buf][4][phys] = f[4][s];
        }
        if (KIND == LR_RWKV6) s_vec[buf][2][phys] = expf(-expf(f[2][s]));
      }
    }
    if (tid < kLrCols) {
      s_v[buf][tid] = f_x;
    } else if (KIND == LR_SSD && tid == kLrCols) {
      const float dte = fminf(fmaxf(softplus_f(f_x + bias_h), p.dt_lo), p.dt_hi);
      s_sc[buf][0] = expf(A_h * dte);
      s_sc[buf][1] = dte;
    }
  };
  auto quad_sum = [](float x) {
    x += __shfl_xor_sync(0xffffffffu, x, 1);
    x += __shfl_xor_sync(0xffffffffu, x, 2);
    return x;
  };

  if (T > 0) { fetch(0); commit(0); }
  __syncthreads();
  for (int t = 0; t < T; ++t) {
    const int buf = t & 1;
    if (t + 1 < T) fetch(t + 1);
    const float* sq = &s_vec[buf][0][part * KPP];
    const float* sk = &s_vec[buf][1][part * KPP];
    const float xv = s_v[buf][col];
    float o = 0.f;
    if (KIND == LR_DPLR) {
      const float* sw = &s_vec[buf][2][part * KPP];
      const float* sa = &s_vec[buf][3][part * KPP];
      const float* sb = &s_vec[buf][4][part * KPP];
      float ah = 0.f;
#pragma unroll
      for (int i = 0; i < KP; ++i) ah += sa[i] * S[i];
      ah = quad_sum(ah);
#pragma unroll
      for (int i = 0; i < KP; ++i) {
        S[i] = sw[i] * S[i] + sb[i] * ah + sk[i] * xv;
        o += S[i] * sq[i];
      }
    } else if (KIND == LR_RWKV6) {
      const float* sw = &s_vec[buf][2][part * KPP];
#pragma unroll
      for (int i = 0; i < KP; ++i) {
        const float kv = sk[i] * xv;
        o += (S[i] + ur[i] * kv) * sq[i];
        S[i] = S[i] * sw[i] + kv;
      }
    } else {
      const float dec = s_sc[buf][0], xd = s_sc[buf][1] * xv;
#pragma unroll
      for (int i = 0; i < KP; ++i) {
        S[i] = dec * S[i] + sk[i] * xd;
        o += S[i] * sq[i];
      }
    }
    o = quad_sum(o);
    if (KIND == LR_SSD) o += D_h * xv;
    if (part == 0 && vok) st_elem(p.o, o_base + t * p.o_st + vcol, p.o_dt, o);
    if (t + 1 < T) commit(buf ^ 1);
    __syncthreads();
  }
  if (p.hT && vok) {
#pragma unroll
    for (int i = 0; i < KP; ++i) {
      const int kk = part * KP + i;
      if (kk < K) p.hT[s_unit + kk * p.s_k + vcol * p.s_v] = S[i];
    }
  }
}

template <int KIND>
inline cudaError_t launch_linrec_kind(const LinRecParams& p, cudaStream_t stream) {
  const int nvs = (p.V + kLrCols - 1) / kLrCols;
  const dim3 grid((unsigned)((int64_t)p.B * p.H * nvs)), block(kLrThreads);
  const int kp = (p.K + 3) / 4;
  if (kp <= 4) linrec_kernel<KIND, 4><<<grid, block, 0, stream>>>(p);
  else if (kp <= 8) linrec_kernel<KIND, 8><<<grid, block, 0, stream>>>(p);
  else if (kp <= 16) linrec_kernel<KIND, 16><<<grid, block, 0, stream>>>(p);
  else if (kp <= 32) linrec_kernel<KIND, 32><<<grid, block, 0, stream>>>(p);
  else linrec_kernel<KIND, 64><<<grid, block, 0, stream>>>(p);
  return cudaGetLastError();
}

inline cudaError_t launch_linrec(int kind, const LinRecParams& p, cudaStream_t stream) {
  if (kind == LR_DPLR) return launch_linrec_kind<LR_DPLR>(p, stream);
  if (kind == LR_RWKV6) return launch_linrec_kind<LR_RWKV6>(p, stream);
  return launch_linrec_kind<LR_SSD>(p, stream);
}

}  // namespace dr
