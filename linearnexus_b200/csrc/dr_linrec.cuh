// Token-by-token scans whose state is a [key, value] matrix with a per-token diagonal decay and rank-one
// writes: the RWKV-7 diagonal-plus-low-rank rule, the RWKV-6 rule with its current-token bonus, and the
// Mamba-2 SSD rule (scalar decay per head and token, B as key, C as query, state stored [value, key]).
//
// One CTA of 128 threads owns 64 value columns of one (batch, head) state, held in registers for the whole
// sequence: a thread keeps a KP x 4 tile (KP keys of one of 8 key parts, 4 adjacent columns).  Eight adjacent
// lanes share a column group and split the key axis, so each reduction over the key axis is a thread-local sum
// finished by three warp shuffles and the arithmetic of a token needs no CTA-wide barrier.  Four columns per
// thread is what keeps the kernel off the shared-memory roof: every key-axis value read from shared memory
// feeds four multiply-adds per rule term (with one column per thread the vector reads alone cost more cycles
// than the arithmetic).  The token vectors are staged through shared memory in blocks of TB tokens: the global
// loads of block n+1 are issued (as raw bits, so none of them waits for another) before the arithmetic of block n
// and committed after it, where the per-element transforms run once (exp of the log decay, sigmoid of the
// receptance, softplus and clamp of dt); one __syncthreads per block.  Tokens past the end of the sequence are
// staged as no-ops (decay 1, nothing written), so the TB tokens of a block run as straight-line code.
//
// What bounds it: 5 K V (DPLR), 4 K V (RWKV-6), 3 K V (SSD) fp32 multiply-adds per token and head on the CUDA
// cores, and one dependent reduce-then-update chain per token.  The tensor cores need the chunked forms.
#pragma once

#include "dr_common.cuh"
#include "dr_scan_launch.h"

namespace dr {

constexpr int kLrThreads = 128;
constexpr int kLrParts = 8;                              // lanes that split the key axis
constexpr int kLrCW = 4;                                 // value columns per thread
constexpr int kLrCols = kLrThreads / kLrParts * kLrCW;   // value columns per CTA (64)

__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }

// Element i of a bf16 (BF) or float32 array as raw bits (0 when !ok), and the bits as a float.  The storage type is
// a template parameter of the kernel: a run-time select between a 16-bit and a 32-bit load puts a consumer (the
// merge of the two arms, or the second of two predicated loads into one register) right behind every load, and
// the loads of a token block then complete one memory round trip after another instead of together.
template <bool BF>
__device__ __forceinline__ uint32_t ld_raw(const void* p, int64_t i, bool ok) {
  // volatile: the load stays where the block prefetch issues it (a plain read-only load may be sunk to its first
  // use, behind the arithmetic it is meant to overlap)
  uint32_t r = 0;
  if (BF) {
    const uint16_t* a = reinterpret_cast<const uint16_t*>(p) + i;
    asm volatile("{\n\t.reg .pred pk;\n\tsetp.ne.s32 pk, %2, 0;\n\t@pk ld.global.nc.u16 %0, [%1];\n\t}" : "+r"(r) : "l"(a), "r"((int)ok));
  } else {
    const uint32_t* a = reinterpret_cast<const uint32_t*>(p) + i;
    asm volatile("{\n\t.reg .pred pk;\n\tsetp.ne.s32 pk, %2, 0;\n\t@pk ld.global.nc.u32 %0, [%1];\n\t}" : "+r"(r) : "l"(a), "r"((int)ok));
  }
  return r;
}
template <bool BF>
__device__ __forceinline__ float raw_to_float(uint32_t r) { return __uint_as_float(BF ? r << 16 : r); }

// sum over the 8 lanes that share a column group
__device__ __forceinline__ float part_sum(float x) {
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  x += __shfl_xor_sync(0xffffffffu, x, 4);
  return x;
}

// KP: keys per thread (the key axis is cut into 8 parts of KP).  TB: tokens staged per block.
template <int KIND, int KP, int TB, bool BF>
__global__ void __launch_bounds__(kLrThreads) linrec_kernel(const LinRecParams p) {
  constexpr int NV = KIND == LR_DPLR ? 5 : (KIND == LR_RWKV6 ? 3 : 2);  // staged key-axis vectors: q k [w [a b]]
  constexpr int KPP = KP + 4;  // part stride: float4 reads stay aligned, the eight parts start on distinct banks
  constexpr int KS = kLrParts * KPP;
  constexpr int KA = kLrParts * KP;                                             // key slots (>= K)
  constexpr int NS = TB * KA / kLrThreads;                                      // key-vector elements per thread and block
  constexpr int NX = (TB * kLrCols + kLrThreads - 1) / kLrThreads;              // value elements per thread and block
  static_assert(TB * KA % kLrThreads == 0 && KP % 4 == 0 && TB <= kLrThreads, "staging assumes whole rounds");
  __shared__ __align__(16) float s_vec[2][TB][NV][KS];
  __shared__ __align__(16) float s_v[2][TB][kLrCols];
  __shared__ float s_sc[2][TB][2];   // SSD: decay exp(A dt), dt

  const int K = p.K, V = p.V, T = p.T;
  const int tid = threadIdx.x;
  const int cg = tid >> 3, part = tid & 7;
  const int nvs = (V + kLrCols - 1) / kLrCols;
  const int unit = blockIdx.x / nvs;
  const int v0 = (blockIdx.x % nvs) * kLrCols;
  const int b = unit / p.H, h = unit % p.H;
  const int vc0 = v0 + cg * kLrCW;   // first of this thread's columns

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

  float S[KP][kLrCW], ur[KIND == LR_RWKV6 ? KP : 1];
  const int64_t s_unit = (int64_t)unit * K * V;
#pragma unroll
  for (int i = 0; i < KP; ++i) {
    const int kk = part * KP + i;
#pragma unroll
    for (int c = 0; c < kLrCW; ++c)
      S[i][c] = (p.h0 && vc0 + c < V && kk < K && in_bounds(p.status, s_unit + kk * p.s_k + (vc0 + c) * p.s_v, p.n_state))
                    ? p.h0[s_unit + kk * p.s_k + (vc0 + c) * p.s_v] : 0.f;
    if (KIND == LR_RWKV6) ur[i] = kk < K ? p.u[(int64_t)h * K + kk] : 0.f;
  }

  uint32_t f[NV][NS], fx[NX], fdt = 0;
  auto fetch = [&](int t0) {
#pragma unroll
    for (int s = 0; s < NS; ++s) {
      const int e = tid + s * kLrThreads;
      const int tok = e / KA, i = e % KA;
      const bool ok = i < K && t0 + tok < T;
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        const int64_t at = base[j] + (int64_t)(t0 + tok) * vecs[j]->st + i;
        f[j][s] = ld_raw<BF>(vecs[j]->p, at, ok && in_bounds(p.status, at, vecs[j]->n));
      }
    }
#pragma unroll
    for (int s = 0; s < NX; ++s) {
      const int e = tid + s * kLrThreads;
      const int tok = e / kLrCols, c = e % kLrCols;
      const bool ok = e < TB * kLrCols && v0 + c < V && t0 + tok < T;
      const int64_t va = v_base + (int64_t)(t0 + tok) * p.v.st + v0 + c;
      fx[s] = ld_raw<BF>(p.v.p, va, ok && in_bounds(p.status, va, p.v.n));
    }
    if (KIND == LR_SSD) {   // dt is float32
      const int64_t da = dt_base + (int64_t)(t0 + tid) * p.dt.st;
      fdt = ld_raw<false>(p.dt.p, da, tid < TB && t0 + tid < T && in_bounds(p.status, da, p.dt.n));
    }
  };
  auto commit = [&](int buf, int t0) {
#pragma unroll
    for (int s = 0; s < NS; ++s) {
      const int e = tid + s * kLrThreads;
      const int tok = e / KA, i = e % KA;
      const int phys = i + (i / KP) * 4;
      const bool live = i < K && t0 + tok < T;   // dead slots and tokens past the end: zero vectors, decay 1
      float qv = raw_to_float<BF>(f[0][s]);
      if (KIND == LR_RWKV6) qv = live ? p.scale / (1.f + __expf(-qv)) : 0.f;   // sigmoid(r) * scale
      if (KIND == LR_DPLR) qv *= p.scale;
      s_vec[buf][tok][0][phys] = qv;
      s_vec[buf][tok][1][phys] = raw_to_float<BF>(f[1][s]);
      if (KIND == LR_DPLR) {
        s_vec[buf][tok][2][phys] = expf(raw_to_float<BF>(f[2][s]));   // raw 0 -> decay 1
        s_vec[buf][tok][3][phys] = raw_to_float<BF>(f[3][s]);
        s_vec[buf][tok][4][phys] = raw_to_float<BF>(f[4][s]);
      }
      if (KIND == LR_RWKV6) s_vec[buf][tok][2][phys] = live ? expf(-expf(raw_to_float<BF>(f[2][s]))) : 1.f;
    }
#pragma unroll
    for (int s = 0; s < NX; ++s) {
      const int e = tid + s * kLrThreads;
      if (e < TB * kLrCols) s_v[buf][e / kLrCols][e % kLrCols] = raw_to_float<BF>(fx[s]);
    }
    if (KIND == LR_SSD && tid < TB) {
      const bool live = t0 + tid < T;
      const float dte = fminf(fmaxf(softplus_f(raw_to_float<false>(fdt) + bias_h), p.dt_lo), p.dt_hi);
      s_sc[buf][tid][0] = live ? expf(A_h * dte) : 1.f;
      s_sc[buf][tid][1] = live ? dte : 0.f;
    }
  };

  if (T > 0) { fetch(0); commit(0, 0); }
  __syncthreads();
  for (int t0 = 0, buf = 0; t0 < T; t0 += TB, buf ^= 1) {
    if (t0 + TB < T) fetch(t0 + TB);
    // this thread's share of every output of the block; summed over the eight key parts after the block
    float ob[TB * kLrCW];
#pragma unroll
    for (int tt = 0; tt < TB; ++tt) {
      const float4* sq = reinterpret_cast<const float4*>(&s_vec[buf][tt][0][part * KPP]);
      const float4* sk = reinterpret_cast<const float4*>(&s_vec[buf][tt][1][part * KPP]);
      const float4 x4 = *reinterpret_cast<const float4*>(&s_v[buf][tt][cg * kLrCW]);
      const float xv[kLrCW] = {x4.x, x4.y, x4.z, x4.w};
      float o[kLrCW] = {0.f, 0.f, 0.f, 0.f};
      if (KIND == LR_DPLR) {
        // h' = w h + k v^T + b (a^T h).  Only the last term waits for the reduction over the key axis: w h + k v^T
        // and its share of the output are computed while the three shuffle rounds of a^T h are in flight, and
        // o = q^T h' = q^T (w h + k v^T) + (q^T b) (a^T h) needs the reduced value once per column.
        const float4* sw = reinterpret_cast<const float4*>(&s_vec[buf][tt][2][part * KPP]);
        const float4* sa = reinterpret_cast<const float4*>(&s_vec[buf][tt][3][part * KPP]);
        const float4* sb = reinterpret_cast<const float4*>(&s_vec[buf][tt][4][part * KPP]);
        float ah[kLrCW] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < KP / 4; ++i) {
          const float4 av = sa[i];
          const float a4[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
          for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int c = 0; c < kLrCW; ++c) ah[c] += a4[j] * S[4 * i + j][c];
        }
#pragma unroll
        for (int c = 0; c < kLrCW; ++c) ah[c] = part_sum(ah[c]);
        float qb = 0.f;
#pragma unroll
        for (int i = 0; i < KP / 4; ++i) {
          const float4 wv = sw[i], kv = sk[i], qv = sq[i], bv = sb[i];
          const float w4[4] = {wv.x, wv.y, wv.z, wv.w}, k4[4] = {kv.x, kv.y, kv.z, kv.w};
          const float q4[4] = {qv.x, qv.y, qv.z, qv.w}, b4[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            qb += q4[j] * b4[j];
#pragma unroll
            for (int c = 0; c < kLrCW; ++c) {
              S[4 * i + j][c] = w4[j] * S[4 * i + j][c] + k4[j] * xv[c];
              o[c] += S[4 * i + j][c] * q4[j];
            }
          }
        }
#pragma unroll
        for (int i = 0; i < KP / 4; ++i) {
          const float4 bv = sb[i];
          const float b4[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
          for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int c = 0; c < kLrCW; ++c) S[4 * i + j][c] += b4[j] * ah[c];
        }
#pragma unroll
        for (int c = 0; c < kLrCW; ++c) o[c] += qb * ah[c];
      } else if (KIND == LR_RWKV6) {
        const float4* sw = reinterpret_cast<const float4*>(&s_vec[buf][tt][2][part * KPP]);
#pragma unroll
        for (int i = 0; i < KP / 4; ++i) {
          const float4 wv = sw[i], kv = sk[i], qv = sq[i];
          const float w4[4] = {wv.x, wv.y, wv.z, wv.w}, k4[4] = {kv.x, kv.y, kv.z, kv.w}, q4[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float uq = ur[4 * i + j] * q4[j];
#pragma unroll
            for (int c = 0; c < kLrCW; ++c) {
              const float kvv = k4[j] * xv[c];
              o[c] += S[4 * i + j][c] * q4[j] + kvv * uq;
              S[4 * i + j][c] = S[4 * i + j][c] * w4[j] + kvv;
            }
          }
        }
      } else {
        const float dec = s_sc[buf][tt][0], dte = s_sc[buf][tt][1];
        float xd[kLrCW];
#pragma unroll
        for (int c = 0; c < kLrCW; ++c) xd[c] = dte * xv[c];
#pragma unroll
        for (int i = 0; i < KP / 4; ++i) {
          const float4 kv = sk[i], qv = sq[i];
          const float k4[4] = {kv.x, kv.y, kv.z, kv.w}, q4[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
          for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int c = 0; c < kLrCW; ++c) {
              S[4 * i + j][c] = dec * S[4 * i + j][c] + k4[j] * xd[c];
              o[c] += S[4 * i + j][c] * q4[j];
            }
        }
        if (part == 0) {   // the skip term D x, counted once per column
#pragma unroll
          for (int c = 0; c < kLrCW; ++c) o[c] += D_h * xv[c];
        }
      }
#pragma unroll
      for (int c = 0; c < kLrCW; ++c) ob[tt * kLrCW + c] = o[c];
    }
    // Sum over the eight key parts, all tokens of the block at once.  While more than one token is left per lane
    // a round halves the list: a lane keeps the half its bit selects and adds the partner's copy of it (reduce-
    // scatter), so lane `part` ends with the four column sums of token part * TB / 8; rounds after that are plain
    // butterflies.  TB * 4 + ... shuffles per block instead of 3 * TB * 4, none of them on the state's chain.
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
      // lanes that hold distinct tokens: the top log2(TB) of the three part bits select the token
      constexpr int kShare = kLrParts / TB;              // lanes holding the same token (1, 2 or 4)
      const int tok = part / kShare;
      if (part % kShare == 0 && t0 + tok < T) {
        const int64_t at = o_base + (int64_t)(t0 + tok) * p.o_st + vc0;
#pragma unroll
        for (int c = 0; c < kLrCW; ++c)
          if (vc0 + c < V && in_bounds(p.status, at + c, p.n_o)) st_elem(p.o, at + c, p.o_dt, ob[c]);
      }
    }
    if (t0 + TB < T) commit(buf ^ 1, t0 + TB);
    __syncthreads();
  }
  if (p.hT) {
#pragma unroll
    for (int i = 0; i < KP; ++i) {
      const int kk = part * KP + i;
#pragma unroll
      for (int c = 0; c < kLrCW; ++c)
        if (kk < K && vc0 + c < V && in_bounds(p.status, s_unit + kk * p.s_k + (vc0 + c) * p.s_v, p.n_state))
          p.hT[s_unit + kk * p.s_k + (vc0 + c) * p.s_v] = S[i][c];
    }
  }
}

template <int KIND, bool BF>
inline cudaError_t launch_linrec_kind(const LinRecParams& p, cudaStream_t stream) {
  const int nvs = (p.V + kLrCols - 1) / kLrCols;
  const dim3 grid((unsigned)((int64_t)p.B * p.H * nvs)), block(kLrThreads);
  const int kp = (p.K + kLrParts - 1) / kLrParts;
  // tokens per block for the small key tiles: the DPLR body is the longest (its eight unrolled tokens overflow the
  // instruction cache: 1.33 -> 1.16 ms with four), the other two rules prefer fewer barriers (RWKV-6 1.16 vs 1.46 ms)
  constexpr int TBS = KIND == LR_DPLR ? 4 : 8;
  if (kp <= 4) linrec_kernel<KIND, 4, TBS, BF><<<grid, block, 0, stream>>>(p);
  else if (kp <= 8) linrec_kernel<KIND, 8, TBS, BF><<<grid, block, 0, stream>>>(p);
  else if (kp <= 16) linrec_kernel<KIND, 16, 4, BF><<<grid, block, 0, stream>>>(p);
  else linrec_kernel<KIND, 32, 2, BF><<<grid, block, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_linrec(int kind, bool io_bf16, const LinRecParams& p, cudaStream_t stream) {
  if (io_bf16) {
    if (kind == LR_DPLR) return launch_linrec_kind<LR_DPLR, true>(p, stream);
    if (kind == LR_RWKV6) return launch_linrec_kind<LR_RWKV6, true>(p, stream);
    return launch_linrec_kind<LR_SSD, true>(p, stream);
  }
  if (kind == LR_DPLR) return launch_linrec_kind<LR_DPLR, false>(p, stream);
  if (kind == LR_RWKV6) return launch_linrec_kind<LR_RWKV6, false>(p, stream);
  return launch_linrec_kind<LR_SSD, false>(p, stream);
}

}  // namespace dr
