// Token-by-token forward of the delta rule (DeltaNet, Gated DeltaNet, KDA): the fp32 state stays in registers
// for the whole sequence.
//
// Same skeleton as the scans of dr_linrec.cuh.  One CTA of 128 threads owns 64 value columns of one
// (batch, head) state; a thread keeps a KP x 4 tile (KP keys of one of 8 key parts, 4 adjacent columns), so every
// key-axis value read from shared memory feeds four multiply-adds per term.  Token vectors are staged in blocks of
// TB tokens: the loads of block n+1 are issued as raw bits before the arithmetic of block n and committed after
// it (exp of the decay once per element), one __syncthreads per block.  Per token, with S~ the decayed state,
//     v_old = S~^T k^        d = beta (v - v_old)        S = S~ + k^ d^T        o = S^T q^
// only v_old sits on the state's dependency chain: o = q^T S~ + (q^.k^) d reads the decayed state, so its
// products run while the three shuffle rounds of v_old are in flight, and the sums of the squares for the l2
// normalisation depend on the inputs alone.  The output sums of a block are reduced over the eight key parts at
// once (reduce-scatter, lane p ends with the four column sums of token p).  Tokens past the end are staged as
// no-ops (k = 0, beta = 0, decay 1).  Works for any K <= 256 and any V (tail columns masked); writes the state at
// every chunk start when the caller keeps checkpoints for the backward (p.ckpt, chunk size p.C).
#pragma once

#include "dr_common.cuh"
#include "dr_linrec.cuh"

namespace dr {

// Element i of a bf16 / float32 array as raw bits into the register of its width (the other one keeps 0): two
// predicated loads with separate destinations, so a run-time storage type costs neither a branch nor a consumer
// behind the load (either would make the loads of a block complete one after another).
__device__ __forceinline__ void ld_raw_either(const void* p, int64_t i, int dt, bool ok, uint32_t& r16, uint32_t& r32) {
  r16 = 0; r32 = 0;
  const char* a16 = reinterpret_cast<const char*>(p) + 2 * i;
  const char* a32 = reinterpret_cast<const char*>(p) + 4 * i;
  const int mode = ok ? (dt == DR_BF16 ? 1 : 2) : 0;
  asm volatile(
      "{\n\t.reg .pred ph, pf;\n\t"
      "setp.eq.s32 ph, %4, 1;\n\t"
      "setp.eq.s32 pf, %4, 2;\n\t"
      "@ph ld.global.nc.u16 %0, [%2];\n\t"
      "@pf ld.global.nc.u32 %1, [%3];\n\t}"
      : "+r"(r16), "+r"(r32) : "l"(a16), "l"(a32), "r"(mode));
}
__device__ __forceinline__ float raw_either_to_float(uint32_t r16, uint32_t r32, int dt) {
  return __uint_as_float(dt == DR_BF16 ? r16 << 16 : r32);
}

template <int VARIANT, int KP, int TB>
__global__ void __launch_bounds__(kLrThreads) recurrent_kernel(const FwdParams p) {
  constexpr int NV = VARIANT == DR_KDA ? 3 : 2;   // staged key-axis vectors: q, k [, e^g]
  constexpr int KPP = KP + 4;
  constexpr int KS = kLrParts * KPP;
  constexpr int KA = kLrParts * KP;
  constexpr int NS = TB * KA / kLrThreads;
  constexpr int NX = (TB * kLrCols + kLrThreads - 1) / kLrThreads;
  static_assert(TB * KA % kLrThreads == 0 && KP % 4 == 0 && 2 * TB <= kLrThreads, "staging assumes whole rounds");
  __shared__ __align__(16) float s_vec[2][TB][NV][KS];
  __shared__ __align__(16) float s_v[2][TB][kLrCols];
  __shared__ float s_sc[2][TB][2];   // e^g (scalar decay), beta

  const int K = p.K, V = p.V, T = p.map.T;
  const int tid = threadIdx.x;
  const int cg = tid >> 3, part = tid & 7;
  const int nvs = (V + kLrCols - 1) / kLrCols;
  const int unit = blockIdx.x / nvs;
  const int v0 = (blockIdx.x % nvs) * kLrCols;
  const int b = unit / p.map.H, h = unit % p.map.H;
  const int vc0 = v0 + cg * kLrCW;

  const int64_t qk_base = p.map.base_qk(b, h, K), qk_tok = p.map.tok_qk(K);
  const int64_t gk_base = p.map.base(b, h, K), gk_tok = p.map.tok(K);   // per-channel decay: one row per value head
  const int64_t v_base = p.map.base(b, h, V), v_tok = p.map.tok(V);
  const int64_t s_base = p.map.base(b, h, 1), s_tok = p.map.tok(1);

  float S[KP][kLrCW];
  const int64_t s_unit = (int64_t)unit * K * V;
#pragma unroll
  for (int i = 0; i < KP; ++i) {
    const int kk = part * KP + i;
#pragma unroll
    for (int c = 0; c < kLrCW; ++c)
      S[i][c] = (p.h0 && vc0 + c < V && kk < K && in_bounds(p.status, s_unit + (int64_t)kk * V + vc0 + c, p.n_state))
                    ? p.h0[s_unit + (int64_t)kk * V + vc0 + c] : 0.f;
  }

  uint32_t f16[NV][NS], f32[NV][NS], x16[NX], x32[NX], g16 = 0, g32 = 0, braw = 0;
  auto fetch = [&](int t0) {
#pragma unroll
    for (int s = 0; s < NS; ++s) {
      const int e = tid + s * kLrThreads;
      const int tok = e / KA, i = e % KA;
      const bool live = i < K && t0 + tok < T;
      const int64_t at = qk_base + (int64_t)(t0 + tok) * qk_tok + i;
      const bool ok = live && in_bounds(p.status, at, p.n_qk);
      ld_raw_either(p.q, at, p.qkv_dt, ok, f16[0][s], f32[0][s]);
      ld_raw_either(p.k, at, p.qkv_dt, ok, f16[1][s], f32[1][s]);
      if (VARIANT == DR_KDA) {
        const int64_t ga = gk_base + (int64_t)(t0 + tok) * gk_tok + i;
        ld_raw_either(p.g, ga, p.g_dt, live && in_bounds(p.status, ga, p.n_gk), f16[2][s], f32[2][s]);
      }
    }
#pragma unroll
    for (int s = 0; s < NX; ++s) {
      const int e = tid + s * kLrThreads;
      const int tok = e / kLrCols, c = e % kLrCols;
      const int64_t va = v_base + (int64_t)(t0 + tok) * v_tok + v0 + c;
      const bool ok = e < TB * kLrCols && v0 + c < V && t0 + tok < T && in_bounds(p.status, va, p.n_v);
      ld_raw_either(p.v, va, p.qkv_dt, ok, x16[s], x32[s]);
    }
    // threads 0..TB-1: beta of token tid; threads TB..2TB-1: the scalar log decay of token tid - TB
    if (tid < TB) {
      uint32_t unused;
      const int64_t ba = s_base + (int64_t)(t0 + tid) * s_tok;
      ld_raw_either(p.beta, ba, DR_F32, t0 + tid < T && in_bounds(p.status, ba, p.n_tok), unused, braw);
    } else if (VARIANT == DR_GATED && tid < 2 * TB) {
      const int64_t ga = s_base + (int64_t)(t0 + tid - TB) * s_tok;
      ld_raw_either(p.g, ga, p.g_dt, t0 + tid - TB < T && in_bounds(p.status, ga, p.n_tok), g16, g32);
    }
  };
  auto commit = [&](int buf) {
#pragma unroll
    for (int s = 0; s < NS; ++s) {
      const int e = tid + s * kLrThreads;
      const int tok = e / KA, i = e % KA;
      const int phys = i + (i / KP) * 4;
      s_vec[buf][tok][0][phys] = raw_either_to_float(f16[0][s], f32[0][s], p.qkv_dt);
      s_vec[buf][tok][1][phys] = raw_either_to_float(f16[1][s], f32[1][s], p.qkv_dt);
      if (VARIANT == DR_KDA) s_vec[buf][tok][2][phys] = expf(raw_either_to_float(f16[2][s], f32[2][s], p.g_dt));   // raw 0 -> 1
    }
#pragma unroll
    for (int s = 0; s < NX; ++s) {
      const int e = tid + s * kLrThreads;
      if (e < TB * kLrCols) s_v[buf][e / kLrCols][e % kLrCols] = raw_either_to_float(x16[s], x32[s], p.qkv_dt);
    }
    if (tid < TB) s_sc[buf][tid][1] = __uint_as_float(braw);
    else if (tid < 2 * TB) s_sc[buf][tid - TB][0] = VARIANT == DR_GATED ? expf(raw_either_to_float(g16, g32, p.g_dt)) : 1.f;
  };

  if (T > 0) { fetch(0); commit(0); }
  __syncthreads();
  for (int t0 = 0, buf = 0; t0 < T; t0 += TB, buf ^= 1) {
    if (t0 + TB < T) fetch(t0 + TB);
    float ob[TB * kLrCW];
#pragma unroll
    for (int tt = 0; tt < TB; ++tt) {
      const float4* sq = reinterpret_cast<const float4*>(&s_vec[buf][tt][0][part * KPP]);
      const float4* sk = reinterpret_cast<const float4*>(&s_vec[buf][tt][1][part * KPP]);
      const float4 x4 = *reinterpret_cast<const float4*>(&s_v[buf][tt][cg * kLrCW]);
      const float xv[kLrCW] = {x4.x, x4.y, x4.z, x4.w};
      const float gs = s_sc[buf][tt][0], beta = s_sc[buf][tt][1];
      if (p.ckpt && t0 + tt < T && (t0 + tt) % p.C == 0) {   // the state at the start of every chunk, for the backward
        float* ck = p.ckpt + ((int64_t)unit * ((T + p.C - 1) / p.C) + (t0 + tt) / p.C) * K * V;
#pragma unroll
        for (int i = 0; i < KP; ++i) {
          const int kk = part * KP + i;
#pragma unroll
          for (int c = 0; c < kLrCW; ++c)
            if (kk < K && vc0 + c < V && in_bounds(p.status, (ck - p.ckpt) + (int64_t)kk * V + vc0 + c, p.n_ckpt))
              ck[(int64_t)kk * V + vc0 + c] = S[i][c];
        }
      }
      float qr[KP], kr[KP];
      float nq = 0.f, nk = 0.f, qk = 0.f;
#pragma unroll
      for (int i = 0; i < KP / 4; ++i) {
        const float4 qv = sq[i], kv = sk[i];
        qr[4 * i] = qv.x; qr[4 * i + 1] = qv.y; qr[4 * i + 2] = qv.z; qr[4 * i + 3] = qv.w;
        kr[4 * i] = kv.x; kr[4 * i + 1] = kv.y; kr[4 * i + 2] = kv.z; kr[4 * i + 3] = kv.w;
      }
#pragma unroll
      for (int i = 0; i < KP; ++i) {
        nq += qr[i] * qr[i];
        nk += kr[i] * kr[i];
        qk += qr[i] * kr[i];
      }
      float qmul = p.scale, kmul = 1.f;
      if (p.l2norm) {   // x / (||x|| + 1e-6); depends on the inputs only
        qmul = p.scale / (sqrtf(part_sum(nq)) + 1e-6f);
        kmul = 1.f / (sqrtf(part_sum(nk)) + 1e-6f);
      }
      // decay, then this thread's share of S~^T k and of q^T S~
      float vo[kLrCW] = {0.f, 0.f, 0.f, 0.f}, o[kLrCW] = {0.f, 0.f, 0.f, 0.f};
      if (VARIANT == DR_KDA) {
        const float4* sg = reinterpret_cast<const float4*>(&s_vec[buf][tt][2][part * KPP]);
#pragma unroll
        for (int i = 0; i < KP / 4; ++i) {
          const float4 gv = sg[i];
          const float g4[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
          for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int c = 0; c < kLrCW; ++c) S[4 * i + j][c] *= g4[j];
        }
      } else if (VARIANT == DR_GATED) {
#pragma unroll
        for (int i = 0; i < KP; ++i)
#pragma unroll
          for (int c = 0; c < kLrCW; ++c) S[i][c] *= gs;
      }
#pragma unroll
      for (int i = 0; i < KP; ++i)
#pragma unroll
        for (int c = 0; c < kLrCW; ++c) {
          vo[c] += kr[i] * S[i][c];
          o[c] += qr[i] * S[i][c];
        }
      float d[kLrCW];
#pragma unroll
      for (int c = 0; c < kLrCW; ++c) d[c] = kmul * beta * (xv[c] - kmul * part_sum(vo[c]));   // k^ d^T = k (kmul d)^T
#pragma unroll
      for (int i = 0; i < KP; ++i)
#pragma unroll
        for (int c = 0; c < kLrCW; ++c) S[i][c] += kr[i] * d[c];
#pragma unroll
      for (int c = 0; c < kLrCW; ++c) ob[tt * kLrCW + c] = qmul * (o[c] + qk * d[c]);
    }
    {
      int n = TB * kLrCW;
#pragma unroll
      for (int m = 4; m >= 1; m >>= 1) {
        const bool upper = (part & m) != 0;
        if (n > kLrCW) {
          n >>= 1;
#pragma unroll
          for (int i = 0; i < TB * kLrCW / 2; ++i) {
            if (i < n) {
              const float send = upper ? ob[i] : ob[i + n];
              const float keep = upper ? ob[i + n] : ob[i];
              ob[i] = keep + __shfl_xor_sync(0xffffffffu, send, m);
            }
          }
        } else {
#pragma unroll
          for (int c = 0; c < kLrCW; ++c) ob[c] += __shfl_xor_sync(0xffffffffu, ob[c], m);
        }
      }
    }
    {
      constexpr int kShare = kLrParts / TB;
      const int tok = part / kShare;
      if (p.o && part % kShare == 0 && t0 + tok < T) {
        const int64_t at = v_base + (int64_t)(t0 + tok) * v_tok + vc0;
#pragma unroll
        for (int c = 0; c < kLrCW; ++c)
          if (vc0 + c < V && in_bounds(p.status, at + c, p.n_v)) st_elem(p.o, at + c, p.out_dt, ob[c]);
      }
    }
    if (t0 + TB < T) commit(buf ^ 1);
    __syncthreads();
  }
  if (p.hT) {
#pragma unroll
    for (int i = 0; i < KP; ++i) {
      const int kk = part * KP + i;
#pragma unroll
      for (int c = 0; c < kLrCW; ++c)
        if (kk < K && vc0 + c < V && in_bounds(p.status, s_unit + (int64_t)kk * V + vc0 + c, p.n_state))
          p.hT[s_unit + (int64_t)kk * V + vc0 + c] = S[i][c];
    }
  }
}

template <int VARIANT>
inline cudaError_t launch_recurrent_variant(const FwdParams& p, cudaStream_t stream) {
  const int nvs = (p.V + kLrCols - 1) / kLrCols;
  const dim3 grid((unsigned)((int64_t)p.map.B * p.map.H * nvs)), block(kLrThreads);
  const int kp = (p.K + kLrParts - 1) / kLrParts;
  if (kp <= 4) recurrent_kernel<VARIANT, 4, 8><<<grid, block, 0, stream>>>(p);
  else if (kp <= 8) recurrent_kernel<VARIANT, 8, 8><<<grid, block, 0, stream>>>(p);
  else if (kp <= 16) recurrent_kernel<VARIANT, 16, 4><<<grid, block, 0, stream>>>(p);
  else recurrent_kernel<VARIANT, 32, 2><<<grid, block, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_recurrent(const FwdParams& p, cudaStream_t stream) {
  if (p.variant == DR_KDA) return launch_recurrent_variant<DR_KDA>(p, stream);
  if (p.variant == DR_GATED) return launch_recurrent_variant<DR_GATED>(p, stream);
  return launch_recurrent_variant<DR_DELTA>(p, stream);
}

}  // namespace dr
