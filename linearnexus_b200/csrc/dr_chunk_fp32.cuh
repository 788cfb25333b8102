// Chunkwise (WY / UT transform) forward in full fp32 on the CUDA cores: the exact path.
//
// Serves fp32 parity (max-abs 1e-4 against the reference maths) and every shape the
// tensor-core kernel does not take: any chunk C <= 64, K <= 128 (multiple of 4), any V.
// One CTA of 256 threads owns 32 value columns of one (batch, head) sequence and walks its
// chunks in order with the fp32 state slice S[K][32] resident in shared memory.
// Per chunk (G = within-chunk cumulative log decay, D_ij = exp(G_i - G_j)):
//   A_kk[i][j] = beta_i * sum_k k_ik k_jk D_ijk (i>j)     A_qk[i][j] = sum_k q_ik k_jk D_ijk (i>=j)
//   (I + A_kk) [W | U] = [beta k e^G | beta v]             (forward substitution, one thread per column)
//   V_new = U - W S ;  O = (q e^G) S + A_qk V_new ;  S <- e^{G_last} S + (k e^{G_last-G})^T V_new
// Every exponent that is evaluated is <= 0 (pairwise differences for i >= j, G itself, and
// G_last - G), so nothing can overflow whatever the size of g.
#pragma once

#include "dr_common.cuh"

namespace dr {

constexpr int kCfThreads = 256;
constexpr int kCfCols = 32;

struct ChunkFp32Smem {
  int ldk, lda, ldv;
  size_t off_q, off_k, off_w, off_g, off_akk, off_aqk, off_u, off_vn, off_s, off_gs, off_beta, off_glast;
  size_t total_floats;
};

__host__ __device__ inline ChunkFp32Smem chunk_fp32_layout(int C, int K, bool kda) {
  ChunkFp32Smem L;
  L.ldk = K + 4;
  L.lda = C + 1;
  L.ldv = kCfCols + 1;
  size_t o = 0;
  L.off_q = o; o += (size_t)C * L.ldk;
  L.off_k = o; o += (size_t)C * L.ldk;
  L.off_w = o; o += (size_t)C * L.ldk;
  L.off_g = o; o += kda ? (size_t)C * L.ldk : 0;
  L.off_akk = o; o += (size_t)C * L.lda;
  L.off_aqk = o; o += (size_t)C * L.lda;
  L.off_u = o; o += (size_t)C * L.ldv;
  L.off_vn = o; o += (size_t)C * L.ldv;
  L.off_s = o; o += (size_t)K * L.ldv;
  L.off_gs = o; o += C;
  L.off_beta = o; o += C;
  L.off_glast = o; o += K;
  L.total_floats = (o + 3) & ~(size_t)3;
  return L;
}

__global__ void __launch_bounds__(kCfThreads) chunk_fp32_kernel(const FwdParams p) {
  extern __shared__ __align__(16) float smem[];
  const int K = p.K, V = p.V, C = p.C, T = p.map.T;
  const bool kda = p.variant == DR_KDA, gated = p.variant == DR_GATED;
  const ChunkFp32Smem L = chunk_fp32_layout(C, K, kda);
  float* sQ = smem + L.off_q;
  float* sK = smem + L.off_k;
  float* sW = smem + L.off_w;
  float* sG = smem + L.off_g;       // KDA only: cumulative per-channel log decay [C][ldk]
  float* sAkk = smem + L.off_akk;
  float* sAqk = smem + L.off_aqk;
  float* sU = smem + L.off_u;
  float* sVn = smem + L.off_vn;
  float* sS = smem + L.off_s;
  float* sGs = smem + L.off_gs;     // cumulative scalar log decay [C]
  float* sBeta = smem + L.off_beta;
  float* sGl = smem + L.off_glast;  // exp(G_last) per channel [K]
  const int ldk = L.ldk, lda = L.lda, ldv = L.ldv;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nvs = (V + kCfCols - 1) / kCfCols;
  const int unit = blockIdx.x / nvs;
  const int v0 = (blockIdx.x % nvs) * kCfCols;
  const int b = unit / p.map.H, h = unit % p.map.H;
  const int64_t qk_base = p.map.base_qk(b, h, K), qk_tok = p.map.tok_qk(K);
  const int64_t gk_base = p.map.base(b, h, K), gk_tok = p.map.tok(K);   // per-channel decay: one row per value head
  const int64_t v_base = p.map.base(b, h, V), v_tok = p.map.tok(V);
  const int64_t s_base = p.map.base(b, h, 1), s_tok = p.map.tok(1);

  for (int i = tid; i < K * kCfCols; i += kCfThreads) {
    const int kk = i / kCfCols, vv = i % kCfCols;
    sS[kk * ldv + vv] = (p.h0 && v0 + vv < V && in_bounds(p.status, ((int64_t)unit * K + kk) * V + v0 + vv, p.n_state))
                            ? p.h0[((int64_t)unit * K + kk) * V + v0 + vv] : 0.f;
  }

  const int nchunks = (T + C - 1) / C;
  for (int n = 0; n < nchunks; ++n) {
    const int t0 = n * C;
    const int rows = min(C, T - t0);
    __syncthreads();
    if (p.ckpt) {
      float* ck = p.ckpt + ((int64_t)unit * nchunks + n) * K * V;
      for (int i = tid; i < K * kCfCols; i += kCfThreads) {
        const int kk = i / kCfCols, vv = i % kCfCols;
        if (v0 + vv < V && in_bounds(p.status, (ck - p.ckpt) + (int64_t)kk * V + v0 + vv, p.n_ckpt))
          ck[(int64_t)kk * V + v0 + vv] = sS[kk * ldv + vv];
      }
    }
    // ---- (1) stage q, k (normalised, q scaled), g, beta, beta*v -------------------------
    for (int c = warp; c < C; c += kCfThreads / 32) {
      float nq = 0.f, nk = 0.f;
      const bool live = c < rows;
      for (int i = lane; i < K; i += 32) {
        float qv = 0.f, kv = 0.f, gv = 0.f;
        if (live) {
          if (in_bounds(p.status, qk_base + (t0 + c) * qk_tok + i, p.n_qk)) {
            qv = ld_elem(p.q, qk_base + (t0 + c) * qk_tok + i, p.qkv_dt);
            kv = ld_elem(p.k, qk_base + (t0 + c) * qk_tok + i, p.qkv_dt);
          }
          if (kda && in_bounds(p.status, gk_base + (t0 + c) * gk_tok + i, p.n_gk))
            gv = ld_elem(p.g, gk_base + (t0 + c) * gk_tok + i, p.g_dt);
        }
        sQ[c * ldk + i] = qv;
        sK[c * ldk + i] = kv;
        if (kda) sG[c * ldk + i] = gv;
        nq += qv * qv;
        nk += kv * kv;
      }
      float qmul = p.scale, kmul = 1.f;
      if (p.l2norm) {
        nq = warp_sum(nq);
        nk = warp_sum(nk);
        qmul = p.scale / (sqrtf(nq) + 1e-6f);
        kmul = 1.f / (sqrtf(nk) + 1e-6f);
      }
      __syncwarp();
      for (int i = lane; i < K; i += 32) {
        sQ[c * ldk + i] *= qmul;
        sK[c * ldk + i] *= kmul;
      }
      if (lane == 0) {
        const bool there = live && in_bounds(p.status, s_base + (t0 + c) * s_tok, p.n_tok);
        sBeta[c] = there ? p.beta[s_base + (t0 + c) * s_tok] : 0.f;
        sGs[c] = (there && gated) ? ld_elem(p.g, s_base + (t0 + c) * s_tok, p.g_dt) : 0.f;
      }
    }
    __syncthreads();
    for (int i = tid; i < C * kCfCols; i += kCfThreads) {
      const int c = i / kCfCols, vv = i % kCfCols;
      float x = 0.f;
      if (c < rows && v0 + vv < V && in_bounds(p.status, v_base + (t0 + c) * v_tok + v0 + vv, p.n_v))
        x = ld_elem(p.v, v_base + (t0 + c) * v_tok + v0 + vv, p.qkv_dt);
      sU[c * ldv + vv] = sBeta[c] * x;
    }
    // cumulative sums of the log decay along the chunk
    if (kda) {
      for (int i = tid; i < K; i += kCfThreads) {
        float acc = 0.f;
        for (int c = 0; c < C; ++c) {
          acc += sG[c * ldk + i];
          sG[c * ldk + i] = acc;
        }
        sGl[i] = expf(acc);
      }
    } else {
      if (tid == 0) {
        float acc = 0.f;
        for (int c = 0; c < C; ++c) {
          acc += sGs[c];
          sGs[c] = acc;
        }
      }
    }
    __syncthreads();
    // ---- (2) A_kk, A_qk over the lower triangle ------------------------------------------
    for (int pid = tid; pid < C * C; pid += kCfThreads) {
      const int i = pid / C, j = pid % C;
      float akk = 0.f, aqk = 0.f;
      if (j <= i) {
        const float4* qi = reinterpret_cast<const float4*>(sQ + i * ldk);
        const float4* ki = reinterpret_cast<const float4*>(sK + i * ldk);
        const float4* kj = reinterpret_cast<const float4*>(sK + j * ldk);
        if (kda) {
          const float4* gi = reinterpret_cast<const float4*>(sG + i * ldk);
          const float4* gj = reinterpret_cast<const float4*>(sG + j * ldk);
          for (int x = 0; x < K / 4; ++x) {
            const float4 a = qi[x], bq = ki[x], c4 = kj[x], g1 = gi[x], g2 = gj[x];
            const float e0 = __expf(fminf(g1.x - g2.x, 0.f)), e1 = __expf(fminf(g1.y - g2.y, 0.f));
            const float e2 = __expf(fminf(g1.z - g2.z, 0.f)), e3 = __expf(fminf(g1.w - g2.w, 0.f));
            aqk += a.x * c4.x * e0 + a.y * c4.y * e1 + a.z * c4.z * e2 + a.w * c4.w * e3;
            akk += bq.x * c4.x * e0 + bq.y * c4.y * e1 + bq.z * c4.z * e2 + bq.w * c4.w * e3;
          }
        } else {
          for (int x = 0; x < K / 4; ++x) {
            const float4 a = qi[x], bq = ki[x], c4 = kj[x];
            aqk += a.x * c4.x + a.y * c4.y + a.z * c4.z + a.w * c4.w;
            akk += bq.x * c4.x + bq.y * c4.y + bq.z * c4.z + bq.w * c4.w;
          }
          const float dcy = expf(fminf(sGs[i] - sGs[j], 0.f));
          aqk *= dcy;
          akk *= dcy;
        }
      }
      sAqk[i * lda + j] = aqk;
      sAkk[i * lda + j] = (j < i) ? sBeta[i] * akk : 0.f;
    }
    __syncthreads();
    // ---- (3) operand transforms:  W_rhs = beta k e^G,  Q <- q e^G,  K <- k e^{G_last - G} ----
    for (int i = tid; i < C * K; i += kCfThreads) {
      const int c = i / K, kk = i % K;
      float G, Gl;
      if (kda) {
        G = sG[c * ldk + kk];
        Gl = sG[(C - 1) * ldk + kk];
      } else {
        G = sGs[c];
        Gl = sGs[C - 1];
      }
      const float eg = expf(G);
      const float kv = sK[c * ldk + kk];
      sW[c * ldk + kk] = sBeta[c] * kv * eg;
      sQ[c * ldk + kk] *= eg;
      sK[c * ldk + kk] = kv * expf(fminf(Gl - G, 0.f));
    }
    if (!kda) {
      const float el = expf(sGs[C - 1]);
      for (int i = tid; i < K; i += kCfThreads) sGl[i] = el;
    }
    __syncthreads();
    // ---- (4) forward substitution, one thread per right-hand-side column ------------------
    if (tid < K + kCfCols) {
      float* X = tid < K ? sW + tid : sU + (tid - K);
      const int ld = tid < K ? ldk : ldv;
      for (int i = 1; i < C; ++i) {
        float acc = X[i * ld];
        const float* arow = sAkk + i * lda;
        for (int j = 0; j < i; ++j) acc -= arow[j] * X[j * ld];
        X[i * ld] = acc;
      }
    }
    __syncthreads();
    // ---- (5) V_new = U - W S  and  O_inter = (q e^G) S  (thread: column lane, 8 rows) ------
    float oacc[8];
    {
      float vacc[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) { vacc[r] = 0.f; oacc[r] = 0.f; }
      for (int kk = 0; kk < K; ++kk) {
        const float s = sS[kk * ldv + lane];
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          const int c = warp + 8 * r;
          if (c < C) {
            vacc[r] += sW[c * ldk + kk] * s;
            oacc[r] += sQ[c * ldk + kk] * s;
          }
        }
      }
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const int c = warp + 8 * r;
        if (c < C) sVn[c * ldv + lane] = sU[c * ldv + lane] - vacc[r];
      }
    }
    __syncthreads();
    // ---- (6) O = O_inter + A_qk V_new ------------------------------------------------------
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const int c = warp + 8 * r;
      if (c < rows) {
        float acc = oacc[r];
        for (int j = 0; j <= c; ++j) acc += sAqk[c * lda + j] * sVn[j * ldv + lane];
        if (p.o && v0 + lane < V && in_bounds(p.status, v_base + (t0 + c) * v_tok + v0 + lane, p.n_v))
          st_elem(p.o, v_base + (t0 + c) * v_tok + v0 + lane, p.out_dt, acc);
      }
    }
    // ---- (7) S <- e^{G_last} S + K~^T V_new -------------------------------------------------
    for (int k0 = warp; k0 < K; k0 += 8 * 4) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      for (int c = 0; c < C; ++c) {
        const float vn = sVn[c * ldv + lane];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int kk = k0 + 8 * r;
          if (kk < K) acc[r] += sK[c * ldk + kk] * vn;
        }
      }
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int kk = k0 + 8 * r;
        if (kk < K) sS[kk * ldv + lane] = sGl[kk] * sS[kk * ldv + lane] + acc[r];
      }
    }
  }
  __syncthreads();
  if (p.hT) {
    for (int i = tid; i < K * kCfCols; i += kCfThreads) {
      const int kk = i / kCfCols, vv = i % kCfCols;
      if (v0 + vv < V && in_bounds(p.status, ((int64_t)unit * K + kk) * V + v0 + vv, p.n_state))
        p.hT[((int64_t)unit * K + kk) * V + v0 + vv] = sS[kk * ldv + vv];
    }
  }
}

inline size_t chunk_fp32_smem_bytes(int C, int K, bool kda) {
  return chunk_fp32_layout(C, K, kda).total_floats * sizeof(float);
}

inline cudaError_t launch_chunk_fp32(const FwdParams& p, cudaStream_t stream) {
  const size_t smem = chunk_fp32_smem_bytes(p.C, p.K, p.variant == DR_KDA);
  cudaError_t e = cudaFuncSetAttribute(chunk_fp32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  const int nvs = (p.V + kCfCols - 1) / kCfCols;
  const dim3 grid((unsigned)((int64_t)p.map.B * p.map.H * nvs)), block(kCfThreads);
  chunk_fp32_kernel<<<grid, block, smem, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace dr
