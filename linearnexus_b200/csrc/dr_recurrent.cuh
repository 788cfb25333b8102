// Token-by-token forward: the fp32 state stays in registers for the whole sequence.
//
// One CTA of 128 threads owns 32 value columns of one (batch, head) state.  Four adjacent
// lanes share a column and split the key axis (KP rows each), so both reductions over k
// (v_old = S~^T k, o = S'^T q) are thread-local sums finished by two warp shuffles; no
// shared-memory reduction and one __syncthreads per token (the double-buffered token
// stage).  Works for any K <= 4*KP and any V (tail columns masked).
#pragma once

#include "dr_common.cuh"

namespace dr {

constexpr int kRecThreads = 128;
constexpr int kRecCols = 32;

template <int KP>
__global__ void __launch_bounds__(kRecThreads) recurrent_kernel(const FwdParams p) {
  constexpr int KPP = KP + 1;          // padded partition stride (bank spread)
  constexpr int KS = 4 * KPP;          // floats per staged q / k / gamma vector
  __shared__ float s_q[2][KS], s_k[2][KS], s_gm[2][KS];
  __shared__ float s_v[2][kRecCols];
  __shared__ float s_sc[2][2];  // gamma (scalar), beta

  const int K = p.K, V = p.V, T = p.map.T;
  const int tid = threadIdx.x;
  const int col = tid >> 2, part = tid & 3;
  const int nvs = (V + kRecCols - 1) / kRecCols;
  const int unit = blockIdx.x / nvs;
  const int v0 = (blockIdx.x % nvs) * kRecCols;
  const int b = unit / p.map.H, h = unit % p.map.H;
  const int vcol = v0 + col;
  const bool vok = vcol < V;

  const int64_t qk_base = p.map.base_qk(b, h, K), qk_tok = p.map.tok_qk(K);
  const int64_t gk_base = p.map.base(b, h, K), gk_tok = p.map.tok(K);   // per-channel decay: one row per value head
  const int64_t v_base = p.map.base(b, h, V), v_tok = p.map.tok(V);
  const int64_t s_base = p.map.base(b, h, 1), s_tok = p.map.tok(1);

  float S[KP];
#pragma unroll
  for (int i = 0; i < KP; ++i) {
    const int kk = part * KP + i;
    S[i] = (p.h0 && vok && kk < K) ? p.h0[((int64_t)unit * K + kk) * V + vcol] : 0.f;
  }

  // Token stage, split into a fetch (global -> registers, issued before the arithmetic of
  // the current token) and a commit (registers -> shared, after it) so that the global
  // latency overlaps the recurrence step.
  constexpr int NS = (4 * KP + kRecThreads - 1) / kRecThreads;
  float f_q[NS], f_k[NS], f_g[NS], f_x = 0.f;
  auto fetch = [&](int t) {
#pragma unroll
    for (int s = 0; s < NS; ++s) {
      const int i = tid + s * kRecThreads;
      f_q[s] = 0.f; f_k[s] = 0.f; f_g[s] = 0.f;
      if (i < K) {
        f_q[s] = ld_elem(p.q, qk_base + t * qk_tok + i, p.qkv_dt);
        f_k[s] = ld_elem(p.k, qk_base + t * qk_tok + i, p.qkv_dt);
        if (p.variant == DR_KDA) f_g[s] = ld_elem(p.g, gk_base + t * gk_tok + i, p.g_dt);
      }
    }
    if (tid < kRecCols)
      f_x = (v0 + tid < V) ? ld_elem(p.v, v_base + t * v_tok + v0 + tid, p.qkv_dt) : 0.f;
    else if (tid == kRecCols)
      f_x = (p.variant == DR_GATED) ? ld_elem(p.g, s_base + t * s_tok, p.g_dt) : 0.f;
    else if (tid == kRecCols + 1)
      f_x = p.beta[s_base + t * s_tok];
  };
  auto commit = [&](int buf) {
#pragma unroll
    for (int s = 0; s < NS; ++s) {
      const int i = tid + s * kRecThreads;
      if (i < 4 * KP) {
        const int phys = i + i / KP;
        s_q[buf][phys] = f_q[s];
        s_k[buf][phys] = f_k[s];
        s_gm[buf][phys] = expf(f_g[s]);
      }
    }
    if (tid < kRecCols) s_v[buf][tid] = f_x;
    else if (tid == kRecCols) s_sc[buf][0] = expf(f_x);
    else if (tid == kRecCols + 1) s_sc[buf][1] = f_x;
  };

  if (T > 0) { fetch(0); commit(0); }
  __syncthreads();
  for (int t = 0; t < T; ++t) {
    const int buf = t & 1;
    if (t + 1 < T) fetch(t + 1);

    float qr[KP], kr[KP];
    float nq = 0.f, nk = 0.f;
#pragma unroll
    for (int i = 0; i < KP; ++i) {
      qr[i] = s_q[buf][part * KPP + i];
      kr[i] = s_k[buf][part * KPP + i];
      nq += qr[i] * qr[i];
      nk += kr[i] * kr[i];
    }
    float qmul = p.scale, kmul = 1.f;
    if (p.l2norm) {
      nq += __shfl_xor_sync(0xffffffffu, nq, 1);
      nq += __shfl_xor_sync(0xffffffffu, nq, 2);
      nk += __shfl_xor_sync(0xffffffffu, nk, 1);
      nk += __shfl_xor_sync(0xffffffffu, nk, 2);
      qmul = p.scale / (sqrtf(nq) + 1e-6f);
      kmul = 1.f / (sqrtf(nk) + 1e-6f);
    }
    const float gs = s_sc[buf][0], beta = s_sc[buf][1];
    float vo = 0.f;
#pragma unroll
    for (int i = 0; i < KP; ++i) {
      kr[i] *= kmul;
      float gm = gs;
      if (p.variant == DR_KDA) gm = s_gm[buf][part * KPP + i];
      S[i] *= gm;
      vo += S[i] * kr[i];
    }
    vo += __shfl_xor_sync(0xffffffffu, vo, 1);
    vo += __shfl_xor_sync(0xffffffffu, vo, 2);
    const float d = beta * (s_v[buf][col] - vo);
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < KP; ++i) {
      S[i] += kr[i] * d;
      o += S[i] * qr[i];
    }
    o += __shfl_xor_sync(0xffffffffu, o, 1);
    o += __shfl_xor_sync(0xffffffffu, o, 2);
    if (part == 0 && vok) st_elem(p.o, v_base + t * v_tok + vcol, p.out_dt, o * qmul);
    if (t + 1 < T) commit(buf ^ 1);
    __syncthreads();
  }
  if (p.hT && vok) {
#pragma unroll
    for (int i = 0; i < KP; ++i) {
      const int kk = part * KP + i;
      if (kk < K) p.hT[((int64_t)unit * K + kk) * V + vcol] = S[i];
    }
  }
}

inline cudaError_t launch_recurrent(const FwdParams& p, cudaStream_t stream) {
  const int nvs = (p.V + kRecCols - 1) / kRecCols;
  const dim3 grid((unsigned)((int64_t)p.map.B * p.map.H * nvs)), block(kRecThreads);
  const int kp = (p.K + 3) / 4;
  if (kp <= 4) recurrent_kernel<4><<<grid, block, 0, stream>>>(p);
  else if (kp <= 8) recurrent_kernel<8><<<grid, block, 0, stream>>>(p);
  else if (kp <= 16) recurrent_kernel<16><<<grid, block, 0, stream>>>(p);
  else if (kp <= 32) recurrent_kernel<32><<<grid, block, 0, stream>>>(p);
  else recurrent_kernel<64><<<grid, block, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace dr
