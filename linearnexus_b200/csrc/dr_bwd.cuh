// Backward of the chunkwise delta rule (DeltaNet / Gated DeltaNet / KDA): exact fp32 on the CUDA cores, and for
// bf16 inputs of DeltaNet / Gated DeltaNet the same phases as tf32 mma.sync products (16 warps per CTA).
//
// The reference has no backward function (its gradients are autodiff through the chunk
// functions); this is the hand-derived chunk-form adjoint.  Per chunk, with S0 the state at the
// chunk start, dS1 the incoming state gradient, G the cumulative log decay, E_ij = e^{G_i-G_j}:
//   forward pieces   X = tril(K^K^^T.E,-1)  A = tril(Q^K^^T.E)  M = I + diag(beta) X
//                    R = beta V - (beta K^ e^G) S0      Vn = M^-1 R
//   adjoints         dVn = A^T dO + (K^ e^{G_L-G}) dS1          dR = M^-T dVn
//                    dV = beta dR                               dA = tril(dO Vn^T)
//                    dM = -dR Vn^T -> dX = beta dM (strict)     dbeta = dR.V + dM.X + dKg.K^ e^G
//                    dQg = dO S0^T   dKg = -dR S0^T   dKt = Vn dS1^T
//                    dQ^ = dQg e^G + (dA.E) K^
//                    dK^ = [dKg beta e^G + (dX.E) K^]_row + [dKt e^{G_L-G} + (dA.E)^T Q^ + (dX.E)^T K^]_col
//                    dG  = Q^.dQ^ + K^.(dK^_row - dK^_col);  dG_L += sum_i dKt.Kt + e^{G_L} <dS1,S0>
//                    dS0 = (Q^ e^G)^T dO + e^{G_L} dS1 - (beta K^ e^G)^T dR
//   then dg = reverse cumulative sum of dG inside the chunk, and the l2-norm / scale chain rule.
//
// Launches: (1) a chunk forward that leaves the state at every chunk start (the fused tcgen05 kernel, the
// two-kernel KDA forward or the fp32 kernel, by shape; skipped when the caller ran the saving forward),
// (1b, tensor-core path) a chunk-parallel pre-pass with what does not depend on the value slice (X, A,
// T = M^-1, q^, k^), (2) the adjoint kernel, one CTA per (batch, head, slice of value columns) walking the
// chunks backwards and storing its partial dQ^, dK^ to the slice's own copy (dG, dbeta by atomics; the adjoint
// is linear in them), (3) a finalize kernel (sum of the copies -- over the value heads of a group too when q, k
// have fewer heads --, normalisation chain rule, reverse cumulative sum, casts).
// Workspace: checkpoints [B*H][N][K][V] | dQ^ copies [slices][B*H][N*C][K] | dK^ copies | dG acc | pre-pass
// records [B*H][N][3*64*64 + 2*64*K], all fp32.
#pragma once

#include <mutex>

#include "dr_chunk_fp32.cuh"
#include "dr_scan_launch.h"
#include "dr_chunk_sm100.cuh"
#include "dr_kda_sm100.cuh"
#include "dr_common.cuh"

namespace dr {

constexpr int kBwThreads = 256;
#ifndef DR_BWD_EXACT_THREADS
#define DR_BWD_EXACT_THREADS 512
#endif
constexpr int kBwSlice = 32;   // value columns per adjoint CTA, every variant (KDA at K = 128: 204 KB of shared memory)
// the tensor-core adjoint runs 16 warps: its phases are short dependent chains of mma.sync and shared-memory
// fetches, and four warps per scheduler hide them where two did not
__host__ __device__ constexpr int bwd_threads(bool tc) { return tc ? 512 : DR_BWD_EXACT_THREADS; }

// Row-panel products on the warp-level tensor-core path (mma.sync m16n8k8, tf32 operands, fp32 accumulate);
// a(m, k), b(k, n) are element accessors into fp32 shared memory.  Lane (g = lane/4, t = lane%4) ends up with
// D[m0+g][n0+2t], D[m0+g][n0+2t+1], D[m0+g+8][n0+2t], D[m0+g+8][n0+2t+1] of every tile.
// The warp owns 16 rows (m0..) and NT consecutive 8-column tiles
// (n0..); the A fragment is fetched once per k-step and reused for every tile, and products that share
// their B operand share its fetch too.  Operands are passed as raw fp32 bits (the tensor core ignores the
// low mantissa bits: truncation to tf32).  k runs over [kb, ke) in steps of 8.
template <int NT, class AF, class BF>
__device__ __forceinline__ void rgemm(float (&d)[NT][4], int m0, int n0, int kb, int ke, AF a, BF b, int lane) {
  const int g = lane >> 2, t = lane & 3;
  for (int k0 = kb; k0 < ke; k0 += 8) {
    uint32_t af[4];
    af[0] = __float_as_uint(a(m0 + g, k0 + t));
    af[1] = __float_as_uint(a(m0 + g + 8, k0 + t));
    af[2] = __float_as_uint(a(m0 + g, k0 + t + 4));
    af[3] = __float_as_uint(a(m0 + g + 8, k0 + t + 4));
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      uint32_t bf[2];
      bf[0] = __float_as_uint(b(k0 + t, n0 + 8 * nt + g));
      bf[1] = __float_as_uint(b(k0 + t + 4, n0 + 8 * nt + g));
      sm100::mma_tf32(d[nt], af, bf);
    }
  }
}
template <int NT, class AF1, class AF2, class BF>
__device__ __forceinline__ void rgemm2(float (&d1)[NT][4], float (&d2)[NT][4], int m0, int n0, int kb, int ke, AF1 a1,
                                       AF2 a2, BF b, int lane) {
  const int g = lane >> 2, t = lane & 3;
  for (int k0 = kb; k0 < ke; k0 += 8) {
    uint32_t af1[4], af2[4];
    af1[0] = __float_as_uint(a1(m0 + g, k0 + t));     af2[0] = __float_as_uint(a2(m0 + g, k0 + t));
    af1[1] = __float_as_uint(a1(m0 + g + 8, k0 + t)); af2[1] = __float_as_uint(a2(m0 + g + 8, k0 + t));
    af1[2] = __float_as_uint(a1(m0 + g, k0 + t + 4)); af2[2] = __float_as_uint(a2(m0 + g, k0 + t + 4));
    af1[3] = __float_as_uint(a1(m0 + g + 8, k0 + t + 4)); af2[3] = __float_as_uint(a2(m0 + g + 8, k0 + t + 4));
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      uint32_t bf[2];
      bf[0] = __float_as_uint(b(k0 + t, n0 + 8 * nt + g));
      bf[1] = __float_as_uint(b(k0 + t + 4, n0 + 8 * nt + g));
      sm100::mma_tf32(d1[nt], af1, bf);
      sm100::mma_tf32(d2[nt], af2, bf);
    }
  }
}
// The same row-panel products with the contraction index taken in pairs: lane (g, t) supplies k0 + 2t and
// k0 + 2t + 1 where the natural order has k0 + t and k0 + t + 4 (a sum over k does not care).  The accessors
// return both values at once, a2(m, k) = {A[m][k], A[m][k+1]} and b2(k, n) = {B[k][n], B[k+1][n]}.
template <int NT, class AF, class BF>
__device__ __forceinline__ void rgemm_p(float (&d)[NT][4], int m0, int n0, int kb, int ke, AF a2, BF b2, int lane) {
  const int g = lane >> 2, t = lane & 3;
  for (int k0 = kb; k0 < ke; k0 += 8) {
    const float2 x0 = a2(m0 + g, k0 + 2 * t), x1 = a2(m0 + g + 8, k0 + 2 * t);
    const uint32_t af[4] = {__float_as_uint(x0.x), __float_as_uint(x1.x), __float_as_uint(x0.y), __float_as_uint(x1.y)};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const float2 y = b2(k0 + 2 * t, n0 + 8 * nt + g);
      const uint32_t bf[2] = {__float_as_uint(y.x), __float_as_uint(y.y)};
      sm100::mma_tf32(d[nt], af, bf);
    }
  }
}
template <int NT, class AF1, class AF2, class BF>
__device__ __forceinline__ void rgemm2_p(float (&d1)[NT][4], float (&d2)[NT][4], int m0, int n0, int kb, int ke, AF1 a1,
                                         AF2 a2, BF b2, int lane) {
  const int g = lane >> 2, t = lane & 3;
  for (int k0 = kb; k0 < ke; k0 += 8) {
    const float2 x0 = a1(m0 + g, k0 + 2 * t), x1 = a1(m0 + g + 8, k0 + 2 * t);
    const float2 z0 = a2(m0 + g, k0 + 2 * t), z1 = a2(m0 + g + 8, k0 + 2 * t);
    const uint32_t af1[4] = {__float_as_uint(x0.x), __float_as_uint(x1.x), __float_as_uint(x0.y), __float_as_uint(x1.y)};
    const uint32_t af2[4] = {__float_as_uint(z0.x), __float_as_uint(z1.x), __float_as_uint(z0.y), __float_as_uint(z1.y)};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const float2 y = b2(k0 + 2 * t, n0 + 8 * nt + g);
      const uint32_t bf[2] = {__float_as_uint(y.x), __float_as_uint(y.y)};
      sm100::mma_tf32(d1[nt], af1, bf);
      sm100::mma_tf32(d2[nt], af2, bf);
    }
  }
}

// sum over j < n (n <= 128) of a(j) b(j) where a(j) is the same for all lanes of the warp and costly: lane l
// evaluates a(l), a(l + 32), ... once and a shuffle hands the values round; b(j) is the lane's own operand.
template <class AF, class BF>
__device__ __forceinline__ float bcast_dot(AF a, BF b, int n, int lane) {
  float av[4], acc = 0.f;
#pragma unroll
  for (int ii = 0; ii < 4; ++ii) av[ii] = (lane + 32 * ii < n) ? a(lane + 32 * ii) : 0.f;
#pragma unroll
  for (int ii = 0; ii < 4; ++ii) {
    if (32 * ii < n) {
      const int lim = min(32, n - 32 * ii);
#pragma unroll 8
      for (int l = 0; l < 32; ++l) {
        const float x = __shfl_sync(0xffffffffu, av[ii], l);
        if (l < lim) acc += x * b(32 * ii + l);
      }
    }
  }
  return acc;
}

struct BwdParams {
  const void* q; const void* k; const void* v; const void* g; const float* beta;
  const void* d_o; const float* d_hT;
  void* dv; float* dbeta; float* dh0;
  const float* ckpt; float* dq_acc; float* dk_acc; float* dg_acc;
  float* pre;   // per chunk [3][64][64] X, A, T then [2][64][K] q^, k^ from bwd_pre_kernel (tensor-core path), or null
  SeqMap map;
  int K, V, C, N;
  int variant, qkv_dt, g_dt, l2norm;
  float scale;
};

struct BwdSmem {
  int ldk, ldq, lda, ldt, ldv;
  size_t q, k, g, x, a, t, v, d_o, vn, dr, s0, ds, gs, eg, wd, beta, dbeta, el, total;
};

// tc: the strides decide which tensor-core fragment fetches are free of bank conflicts.  A fragment is read either
// along the rows of its array (array row <- lane / 4, the contraction index k <- lane % 4 along the row) or
// across them (array row <- k <- lane % 4, consecutive words <- lane / 4).  With k in the natural order (lane % 4
// and lane % 4 + 4) a read along the rows wants a stride of 4 mod 32 words and a read across them 8 mod 32; with
// k taken in pairs (2 (lane % 4) and the word after it: one 8-byte load along a row) it is the other way round.
// Every product of the kernel picks the order that suits both of its operands: k^ and T sit at 4 mod 32,
// everything else at 8 mod 32.  Three products keep a two-way conflict on one operand (T^T in dR; k^ in dS0 and
// in the column sums of dX).
__host__ __device__ inline BwdSmem bwd_layout(int C, int K, int VS, bool kda, bool tc = false) {
  BwdSmem L;
  L.ldk = K + 4; L.ldq = tc ? K + 8 : K + 4;
  L.lda = tc ? 72 : kda ? sm100::LDT : C + 1; L.ldt = sm100::LDT; L.ldv = tc ? VS + 8 : VS + 1;
  size_t o = 0;
  L.q = o; o += (size_t)C * L.ldq;
  L.k = o; o += (size_t)C * L.ldk;
  L.g = o; o += kda ? (size_t)C * L.ldk : 0;
  L.x = o; o += (size_t)C * L.lda;
  L.a = o; o += (size_t)C * L.lda;
  L.t = o; o += (tc || kda) ? (size_t)C * L.ldt : 0;
  L.v = o; o += (size_t)C * L.ldv;
  L.d_o = o; o += (size_t)C * L.ldv;
  L.vn = o; o += (size_t)C * L.ldv;
  L.dr = o; o += (size_t)C * L.ldv;
  L.s0 = o; o += (size_t)K * L.ldv;
  L.ds = o; o += (size_t)K * L.ldv;
  L.gs = o; o += C; L.eg = o; o += C; L.wd = o; o += C; L.beta = o; o += C; L.dbeta = o; o += C;
  L.el = o; o += K;
  L.total = (o + 3) & ~(size_t)3;
  return L;
}


// TC: the products run on mma.sync tf32 (bf16 inputs: well inside their 2e-2 tolerance); otherwise exact fp32.
template <int VS, bool KDA, bool TC>
__global__ void __launch_bounds__(bwd_threads(TC)) bwd_chunk_kernel(const BwdParams p) {
  constexpr int NTHR = bwd_threads(TC), NW = NTHR / 32;
  constexpr int NTW = NW / 4;   // tensor-core phases: warps that share one 16-row panel of the chunk
  extern __shared__ __align__(16) float smem[];
  const int K = p.K, V = p.V, C = p.C, T = p.map.T, N = p.N;
  const bool gated = p.variant == DR_GATED;
  const BwdSmem L = bwd_layout(C, K, VS, KDA, TC);
  float* sQ = smem + L.q;      float* sK = smem + L.k;     float* sG = smem + L.g;
  float* sX = smem + L.x;      float* sA = smem + L.a;      float* sT = smem + L.t;
  float* sV = smem + L.v;      float* sdO = smem + L.d_o;  float* sVn = smem + L.vn;  float* sdR = smem + L.dr;
  float* sS0 = smem + L.s0;    float* sdS = smem + L.ds;
  float* sGs = smem + L.gs;    float* sEG = smem + L.eg;   float* sWd = smem + L.wd;
  float* sBeta = smem + L.beta; float* sdBeta = smem + L.dbeta; float* sEL = smem + L.el;
  const int ldk = L.ldk, ldq = L.ldq, lda = L.lda, ldt = L.ldt, ldv = L.ldv;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nvs = (V + VS - 1) / VS;
  const int unit = blockIdx.x / nvs;
  const int v0 = (blockIdx.x % nvs) * VS;
  const int b = unit / p.map.H, h = unit % p.map.H;
  const int64_t qk_base = p.map.base_qk(b, h, K), qk_tok = p.map.tok_qk(K);   // q, k: head h / (H / Hq)
  const int64_t gk_base = p.map.base(b, h, K), gk_tok = p.map.tok(K);          // per-channel decay: per value head
  const int64_t v_base = p.map.base(b, h, V), v_tok = p.map.tok(V);
  const int64_t s_base = p.map.base(b, h, 1), s_tok = p.map.tok(1);
  const int64_t acc_row0 = (int64_t)unit * N * C;  // first row of this unit in the [.., N*C, ..] accumulators
  // dq^, dk^ partials of this value slice go to the slice's own copy of the accumulator (plain stores;
  // the finalize kernel adds the slices), dG and dbeta are few enough for atomics
  const int64_t slice_off = (int64_t)(blockIdx.x % nvs) * ((int64_t)p.map.B * p.map.H * N * C) * K;

  for (int i = tid; i < K * VS; i += NTHR) {
    const int kk = i / VS, vv = i % VS;
    sdS[kk * ldv + vv] = (p.d_hT && v0 + vv < V) ? p.d_hT[((int64_t)unit * K + kk) * V + v0 + vv] : 0.f;
  }

  if constexpr (TC) {
    // blocks above the diagonal of X, A, T: zero once (the copies below skip them, the dA / dX tiles rewrite zeros)
    for (int i = tid; i < 64 * 64; i += NTHR) {
      const int r = i >> 6, c = i & 63;
      if ((c >> 4) > (r >> 4)) { sX[r * lda + c] = 0.f; sA[r * lda + c] = 0.f; sT[r * ldt + c] = 0.f; }
    }
  }
  for (int n = N - 1; n >= 0; --n) {
    const int t0 = n * C;
    const int rows = min(C, T - t0);
    __syncthreads();
    // ---- stage q^, k^ (fp32, normalised / scaled), g, beta, v, dO, S0 --------------------------------
    if constexpr (TC) {
      {
        // X, A, T of this chunk were computed once for all value slices by bwd_pre_kernel: 16-byte async copies
        // into their arrays (and so were the normalised fp32 rows q^, k^)
        // (only the 16x16 blocks on and below the diagonal: the others are zero in all three and stay zero here)
        // Two groups: A, T, k^ are needed from the first product on; X and q^ only by the dA / dX tiles and the
        // per-channel products, so their copies keep running under the phases before those.
        const float* src = p.pre + ((int64_t)unit * N + n) * (3 * 64 * 64 + 2 * 64 * K);
        const float* qsrc = src + 3 * 4096;   // q^, k^: a warp per row, 512 bytes per instruction
        for (int i = tid; i < 2 * 64 * 16; i += NTHR) {
          const int m = 1 + (i >> 10), r = (i >> 4) & 63, c4 = (i & 15) * 4;
          float* dst = (m == 1 ? sA + r * lda : sT + r * ldt) + c4;
          if ((c4 >> 4) <= (r >> 4)) tc::cp_async16(tc::smem_u32(dst), src + m * 4096 + r * 64 + c4, true);
        }
        for (int r = warp; r < 64; r += NW)
          for (int c4 = 4 * lane; c4 < K; c4 += 128) tc::cp_async16(tc::smem_u32(sK + r * ldk + c4), qsrc + (64 + r) * K + c4, true);
        tc::cp_async_commit();
        for (int i = tid; i < 64 * 16; i += NTHR) {
          const int r = i >> 4, c4 = (i & 15) * 4;
          if ((c4 >> 4) <= (r >> 4)) tc::cp_async16(tc::smem_u32(sX + r * lda + c4), src + r * 64 + c4, true);
        }
        for (int r = warp; r < 64; r += NW)
          for (int c4 = 4 * lane; c4 < K; c4 += 128) tc::cp_async16(tc::smem_u32(sQ + r * ldq + c4), qsrc + r * K + c4, true);
        tc::cp_async_commit();
      }
      // beta: row warp + NW * lane of the chunk (C = 64); the last warp takes the decay of all 64 rows (two per
      // lane) and scans it in registers while the other loads are in flight
      constexpr int RPW = 64 / NW;
      float bt = 0.f, g_lo = 0.f, g_hi = 0.f;
      if (lane < RPW && warp + NW * lane < rows) bt = p.beta[s_base + (t0 + warp + NW * lane) * s_tok];
      if (warp == NW - 1 && gated) {
        if (lane < rows) g_lo = ld_elem(p.g, s_base + (t0 + lane) * s_tok, p.g_dt);
        if (lane + 32 < rows) g_hi = ld_elem(p.g, s_base + (t0 + lane + 32) * s_tok, p.g_dt);
      }
      // bf16 v, dO and the fp32 checkpoint slice: 16-byte accesses, every global load issued before the first is used
      uint4 vr = make_uint4(0u, 0u, 0u, 0u), dor = make_uint4(0u, 0u, 0u, 0u);
      const int vrow = tid / (VS / 8), vpc = tid % (VS / 8);
      if (tid < C * (VS / 8) && vrow < rows && v0 + 8 * vpc < V) {
        vr = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.v) + v_base + (t0 + vrow) * v_tok + v0 + 8 * vpc);
        dor = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.d_o) + v_base + (t0 + vrow) * v_tok + v0 + 8 * vpc);
      }
      constexpr int SIT = 2048 / NTHR;   // K <= 256, VS = 32: at most 2048 16-byte pieces of the checkpoint slice
      float4 s0r[SIT];
      {
        const float* ck = p.ckpt + ((int64_t)unit * N + n) * K * V;
#pragma unroll
        for (int it = 0; it < SIT; ++it) {
          const int i = tid + it * NTHR;
          const int kk = i / (VS / 4), j4 = 4 * (i % (VS / 4));
          s0r[it] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (i < K * (VS / 4) && v0 + j4 < V) s0r[it] = *reinterpret_cast<const float4*>(ck + (int64_t)kk * V + v0 + j4);
        }
      }
      if (lane < RPW) {
        const int c = warp + NW * lane;
        sBeta[c] = bt;
        sdBeta[c] = 0.f;
      }
      if (warp == NW - 1) {
        // inclusive prefix sums G of the 64 log-decays, then e^G, e^{G_L - G} and e^{G_L}
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const float a = __shfl_up_sync(0xffffffffu, g_lo, o), b2 = __shfl_up_sync(0xffffffffu, g_hi, o);
          if (lane >= o) { g_lo += a; g_hi += b2; }
        }
        g_hi += __shfl_sync(0xffffffffu, g_lo, 31);
        const float gl = __shfl_sync(0xffffffffu, g_hi, 31);
        sGs[lane] = g_lo; sGs[lane + 32] = g_hi;
        sEG[lane] = expf(g_lo); sEG[lane + 32] = expf(g_hi);
        sWd[lane] = expf(fminf(gl - g_lo, 0.f)); sWd[lane + 32] = expf(fminf(gl - g_hi, 0.f));
        const float egl = expf(gl);
        for (int i = lane; i < K; i += 32) sEL[i] = egl;
      }
#pragma unroll
      for (int it = 0; it < SIT; ++it) {
        const int i = tid + it * NTHR;
        if (i < K * (VS / 4)) *reinterpret_cast<float4*>(sS0 + (i / (VS / 4)) * ldv + 4 * (i % (VS / 4))) = s0r[it];
      }
      if (tid < C * (VS / 8)) {
        const uint32_t* wv = reinterpret_cast<const uint32_t*>(&vr);
        const uint32_t* wo = reinterpret_cast<const uint32_t*>(&dor);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wv[e]));
          const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wo[e]));
          *reinterpret_cast<float2*>(sV + vrow * ldv + 8 * vpc + 2 * e) = x;
          *reinterpret_cast<float2*>(sdO + vrow * ldv + 8 * vpc + 2 * e) = y;
        }
      }
    } else {
    // rows warp, warp + NW, ... of the chunk, four at a time: every global load of the four rows is issued before
    // the first norm (K <= 128: at most four elements per lane, row and array)
    for (int cb = warp; cb < C; cb += 4 * NW) {
      float qv[4][4], kv[4][4], gv[4][4], bt[4], gs[4];
#pragma unroll
      for (int rr = 0; rr < 4; ++rr) {
        const int c = cb + rr * NW;
        const bool live = c < rows;
#pragma unroll
        for (int ii = 0; ii < 4; ++ii) {
          const int i = lane + 32 * ii;
          qv[rr][ii] = kv[rr][ii] = gv[rr][ii] = 0.f;
          if (live && i < K) {
            qv[rr][ii] = ld_elem(p.q, qk_base + (t0 + c) * qk_tok + i, p.qkv_dt);
            kv[rr][ii] = ld_elem(p.k, qk_base + (t0 + c) * qk_tok + i, p.qkv_dt);
            if (KDA) gv[rr][ii] = ld_elem(p.g, gk_base + (t0 + c) * gk_tok + i, p.g_dt);
          }
        }
        bt[rr] = (live && lane == 0) ? p.beta[s_base + (t0 + c) * s_tok] : 0.f;
        gs[rr] = (live && gated && lane == 0) ? ld_elem(p.g, s_base + (t0 + c) * s_tok, p.g_dt) : 0.f;
      }
#pragma unroll
      for (int rr = 0; rr < 4; ++rr) {
        const int c = cb + rr * NW;
        if (c < C) {
          float nq = 0.f, nk = 0.f;
#pragma unroll
          for (int ii = 0; ii < 4; ++ii) { nq += qv[rr][ii] * qv[rr][ii]; nk += kv[rr][ii] * kv[rr][ii]; }
          float qmul = p.scale, kmul = 1.f;
          if (p.l2norm) {
            nq = warp_sum(nq);
            nk = warp_sum(nk);
            qmul = p.scale / (sqrtf(nq) + 1e-6f);
            kmul = 1.f / (sqrtf(nk) + 1e-6f);
          }
#pragma unroll
          for (int ii = 0; ii < 4; ++ii) {
            const int i = lane + 32 * ii;
            if (i < K) {
              sQ[c * ldq + i] = qv[rr][ii] * qmul;
              sK[c * ldk + i] = kv[rr][ii] * kmul;
              if (KDA) sG[c * ldk + i] = gv[rr][ii];
            }
          }
          if (lane == 0) {
            sBeta[c] = bt[rr];
            sGs[c] = gs[rr];
            sdBeta[c] = 0.f;
          }
        }
      }
    }
    for (int i = tid; i < C * VS; i += NTHR) {
      const int c = i / VS, vv = i % VS;
      float x = 0.f, y = 0.f;
      if (c < rows && v0 + vv < V) {
        x = ld_elem(p.v, v_base + (t0 + c) * v_tok + v0 + vv, p.qkv_dt);
        y = ld_elem(p.d_o, v_base + (t0 + c) * v_tok + v0 + vv, p.qkv_dt);
      }
      sV[c * ldv + vv] = x;
      sdO[c * ldv + vv] = y;
    }
    {
      const float* ck = p.ckpt + ((int64_t)unit * N + n) * K * V;
      for (int i = tid; i < K * VS; i += NTHR) {
        const int kk = i / VS, vv = i % VS;
        sS0[kk * ldv + vv] = (v0 + vv < V) ? ck[(int64_t)kk * V + v0 + vv] : 0.f;
      }
    }
    }
    if constexpr (TC) tc::cp_async_wait_1();   // A, T, k^ have landed; X, q^ may still be in flight
    __syncthreads();
    if (KDA) {
      for (int i = tid; i < K; i += NTHR) {
        float acc = 0.f;
        for (int c = 0; c < C; ++c) {
          acc += sG[c * ldk + i];
          sG[c * ldk + i] = acc;
        }
        sEL[i] = expf(acc);
      }
    } else if (!TC && tid == 0) {
      float acc = 0.f;
      for (int c = 0; c < C; ++c) { acc += sGs[c]; sGs[c] = acc; }
    }
    if (!TC) __syncthreads();
    if (!KDA && !TC) {
      const float gl = sGs[C - 1];
      for (int i = tid; i < C; i += NTHR) {
        sEG[i] = expf(sGs[i]);
        sWd[i] = expf(fminf(gl - sGs[i], 0.f));
      }
      for (int i = tid; i < K; i += NTHR) sEL[i] = expf(gl);
    }
    // ---- X = tril(K^K^^T.E,-1) (not yet scaled by beta), A = tril(Q^K^^T.E) ---------------------------
    if constexpr (TC) {
      // X and A (decay folded in) came from the pre-pass
    } else {
    for (int pid = tid; pid < C * C; pid += NTHR) {
      const int i = pid / C, j = pid % C;
      float akk = 0.f, aqk = 0.f;
      if (j <= i) {
        const float4* qi = reinterpret_cast<const float4*>(sQ + i * ldq);
        const float4* ki = reinterpret_cast<const float4*>(sK + i * ldk);
        const float4* kj = reinterpret_cast<const float4*>(sK + j * ldk);
        if (KDA) {
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
        }
      }
      sA[i * lda + j] = aqk;   // GDN/DeltaNet: the decay factor is applied where the entry is used
      sX[i * lda + j] = (j < i) ? akk : 0.f;
    }
    }
    __syncthreads();
    auto ld2 = [](const float* ptr) { return *reinterpret_cast<const float2*>(ptr); };
    // explicit inverse (tf32 merge products) instead of the substitutions: exact-path kernel, bf16 inputs only
    const bool use_inv = KDA && !TC && NW == 16 && C == 64 && p.qkv_dt == DR_BF16;
    auto Eij = [&](int i, int j) -> float { return (KDA || TC) ? 1.f : __expf(fminf(sGs[i] - sGs[j], 0.f)); };
    // ---- R = beta V - (beta K^ e^G) S0  (lane = value column, warp = rows) ----------------------------
    if constexpr (TC) {
      {
        constexpr int NT = VS / 8 / NTW;
        const int m0 = (warp / NTW) * 16, n0 = (warp % NTW) * 8 * NT;
        float d[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) d[nt][0] = d[nt][1] = d[nt][2] = d[nt][3] = 0.f;
        rgemm<NT>(d, m0, n0, 0, K, [&](int m, int k) { return sK[m * ldk + k]; },
                  [&](int k, int nn) { return sS0[k * ldv + nn]; }, lane);
        const int g = lane >> 2, t = lane & 3;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int c = m0 + g + (e >> 1) * 8, vv = n0 + 8 * nt + 2 * t + (e & 1);
            sVn[c * ldv + vv] = sBeta[c] * (sV[c * ldv + vv] - sEG[c] * d[nt][e]);
          }
      }
    } else {
    {
      constexpr int RPW = NW;  // rows per warp pass
      const int vv = lane % VS, sub = lane / VS;  // VS = 16: two row streams per warp
      constexpr int STREAMS = 32 / VS;
      for (int c = warp * STREAMS + sub; c < C; c += RPW * STREAMS) {
        float acc = 0.f;
        const float bc = sBeta[c];
        if constexpr (KDA && VS == 32) {
          // the 32 lanes of a row need the same k^ e^G: each lane forms four of them once, a shuffle hands them round
          acc = bcast_dot([&](int kk) { return sK[c * ldk + kk] * __expf(sG[c * ldk + kk]); },
                          [&](int kk) { return sS0[kk * ldv + vv]; }, K, lane);
        } else {
        for (int kk = 0; kk < K; ++kk) {
          const float eg = KDA ? __expf(sG[c * ldk + kk]) : 1.f;
          acc += sK[c * ldk + kk] * eg * sS0[kk * ldv + vv];
        }
        }
        if (!KDA) acc *= sEG[c];
        sVn[c * ldv + vv] = bc * (sV[c * ldv + vv] - acc);
      }
    }
    }
    __syncthreads();
    // ---- Vn = M^-1 R : forward substitution, 8 lanes per column -----------------------------------------
    if constexpr (TC) {
      // with the explicit inverse T = (I + diag(beta) X)^-1 of the pre-pass, Vn = T R on the tensor cores
      constexpr int NT = VS / 8 / NTW;
      const int m0 = (warp / NTW) * 16, n0 = (warp % NTW) * 8 * NT;
      float d[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) d[nt][0] = d[nt][1] = d[nt][2] = d[nt][3] = 0.f;
      rgemm<NT>(d, m0, n0, 0, m0 + 16, [&](int m, int k) { return k <= m ? sT[m * ldt + k] : 0.f; },
                [&](int k, int nn) { return sVn[k * ldv + nn]; }, lane);
      __syncthreads();
      const int g = lane >> 2, t = lane & 3;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e)
          sVn[(m0 + g + (e >> 1) * 8) * ldv + n0 + 8 * nt + 2 * t + (e & 1)] = d[nt][e];
    } else if (use_inv) {
      // (bf16 inputs of the per-channel variant) the blocked inverse of the forward kernels instead of 63 dependent
      // steps, then Vn = T R with four rows per thread
      if (tid < 256) sm100::block_inverse_64(sX, sBeta, sT, tid);
      __syncthreads();
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      if (lane < VS) {
        for (int j = 0; j < 64; ++j) {
          const float x = sVn[j * ldv + lane];
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const int i = warp + 16 * r;
            acc[r] += (j <= i ? sT[i * ldt + j] : 0.f) * x;
          }
        }
      }
      __syncthreads();
      if (lane < VS) {
#pragma unroll
        for (int r = 0; r < 4; ++r) sVn[(warp + 16 * r) * ldv + lane] = acc[r];
      }
    } else
    if (tid < 8 * VS) {
      const int col = tid >> 3, l8 = tid & 7;
      for (int i = 1; i < C; ++i) {
        float part = 0.f;
        for (int j = l8; j < i; j += 8) part += sX[i * lda + j] * Eij(i, j) * sVn[j * ldv + col];
        part += __shfl_xor_sync(0xffffffffu, part, 1);
        part += __shfl_xor_sync(0xffffffffu, part, 2);
        part += __shfl_xor_sync(0xffffffffu, part, 4);
        if (l8 == 0) sVn[i * ldv + col] -= sBeta[i] * part;
        __syncwarp();
      }
    }
    __syncthreads();
    // ---- dVn = A^T dO + (K^ e^{G_L-G}) dS1 -----------------------------------------------------------------
    if constexpr (TC) {
      {
        constexpr int NT = VS / 8 / NTW;
        const int m0 = (warp / NTW) * 16, n0 = (warp % NTW) * 8 * NT;
        float d1[NT][4], d2[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          d1[nt][0] = d1[nt][1] = d1[nt][2] = d1[nt][3] = 0.f;
          d2[nt][0] = d2[nt][1] = d2[nt][2] = d2[nt][3] = 0.f;
        }
        rgemm<NT>(d1, m0, n0, m0, C, [&](int m, int k) { return sA[k * lda + m]; },   // A^T (lower A, decayed)
                  [&](int k, int nn) { return sdO[k * ldv + nn]; }, lane);
        rgemm<NT>(d2, m0, n0, 0, K, [&](int m, int k) { return sK[m * ldk + k]; },
                  [&](int k, int nn) { return sdS[k * ldv + nn]; }, lane);
        const int g = lane >> 2, t = lane & 3;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int c = m0 + g + (e >> 1) * 8, vv = n0 + 8 * nt + 2 * t + (e & 1);
            sdR[c * ldv + vv] = d1[nt][e] + sWd[c] * d2[nt][e];
          }
      }
    } else {
    {
      const int vv = lane % VS, sub = lane / VS;
      constexpr int STREAMS = 32 / VS;
      for (int c = warp * STREAMS + sub; c < C; c += NW * STREAMS) {
        float acc = 0.f;
        for (int i = c; i < C; ++i) acc += sA[i * lda + c] * Eij(i, c) * sdO[i * ldv + vv];
        float acc2 = 0.f;
        if constexpr (KDA && VS == 32) {
          acc2 = bcast_dot([&](int kk) { return sK[c * ldk + kk] * __expf(fminf(sG[(C - 1) * ldk + kk] - sG[c * ldk + kk], 0.f)); },
                           [&](int kk) { return sdS[kk * ldv + vv]; }, K, lane);
        } else {
        for (int kk = 0; kk < K; ++kk) {
          const float w = KDA ? __expf(fminf(sG[(C - 1) * ldk + kk] - sG[c * ldk + kk], 0.f)) : 1.f;
          acc2 += sK[c * ldk + kk] * w * sdS[kk * ldv + vv];
        }
        }
        if (!KDA) acc2 *= sWd[c];
        sdR[c * ldv + vv] = acc + acc2;
      }
    }
    }
    __syncthreads();
    // ---- dR = M^-T dVn : back substitution ---------------------------------------------------------------------
    if constexpr (TC) {
      constexpr int NT = VS / 8 / NTW;
      const int m0 = (warp / NTW) * 16, n0 = (warp % NTW) * 8 * NT;
      float d[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) d[nt][0] = d[nt][1] = d[nt][2] = d[nt][3] = 0.f;
      rgemm<NT>(d, m0, n0, m0, C, [&](int m, int k) { return k >= m ? sT[k * ldt + m] : 0.f; },
                [&](int k, int nn) { return sdR[k * ldv + nn]; }, lane);
      __syncthreads();
      const int g = lane >> 2, t = lane & 3;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e)
          sdR[(m0 + g + (e >> 1) * 8) * ldv + n0 + 8 * nt + 2 * t + (e & 1)] = d[nt][e];
    } else if (use_inv) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};   // dR = T^T dVn
      if (lane < VS) {
        for (int j = 0; j < 64; ++j) {
          const float x = sdR[j * ldv + lane];
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const int i = warp + 16 * r;
            acc[r] += (j >= i ? sT[j * ldt + i] : 0.f) * x;
          }
        }
      }
      __syncthreads();
      if (lane < VS) {
#pragma unroll
        for (int r = 0; r < 4; ++r) sdR[(warp + 16 * r) * ldv + lane] = acc[r];
      }
    } else
    if (tid < 8 * VS) {
      const int col = tid >> 3, l8 = tid & 7;
      for (int i = C - 2; i >= 0; --i) {
        float part = 0.f;
        for (int j = i + 1 + l8; j < C; j += 8) part += sBeta[j] * sX[j * lda + i] * Eij(j, i) * sdR[j * ldv + col];
        part += __shfl_xor_sync(0xffffffffu, part, 1);
        part += __shfl_xor_sync(0xffffffffu, part, 2);
        part += __shfl_xor_sync(0xffffffffu, part, 4);
        if (l8 == 0) sdR[i * ldv + col] -= part;
        __syncwarp();
      }
    }
    __syncthreads();
    // ---- dV = beta dR ; dbeta += dR.V ; dA = tril(dO Vn^T).E ; dX = beta tril(-dR Vn^T).E ; dbeta += dM.X ------
    for (int i = tid; i < C * VS; i += NTHR) {
      const int c = i / VS, vv = i % VS;
      if (c < rows && v0 + vv < V)
        st_elem(p.dv, v_base + (t0 + c) * v_tok + v0 + vv, p.qkv_dt, sBeta[c] * sdR[c * ldv + vv]);
    }
    for (int c = warp; c < C; c += NW) {
      float acc = 0.f;
      for (int vv = lane; vv < VS; vv += 32) acc += sdR[c * ldv + vv] * sV[c * ldv + vv];
      acc = warp_sum(acc);
      if (lane == 0) sdBeta[c] += acc;
    }
    if constexpr (TC) tc::cp_async_wait_all();   // X, q^
    __syncthreads();
    if constexpr (TC) {
      {
        // warp = 16 rows x 64 / NTW columns; both products share the B operand Vn^T
        constexpr int NA = 8 / NTW;
        const int m0 = (warp / NTW) * 16, n0 = (warp % NTW) * 8 * NA;
        float da[NA][4], dm[NA][4];
#pragma unroll
        for (int nt = 0; nt < NA; ++nt) {
          da[nt][0] = da[nt][1] = da[nt][2] = da[nt][3] = 0.f;
          dm[nt][0] = dm[nt][1] = dm[nt][2] = dm[nt][3] = 0.f;
        }
        if (n0 <= m0 + 15)
          rgemm2_p<NA>(da, dm, m0, n0, 0, VS, [&](int m, int k) { return ld2(sdO + m * ldv + k); },
                       [&](int m, int k) { return ld2(sdR + m * ldv + k); },
                       [&](int k, int nn) { return ld2(sVn + nn * ldv + k); }, lane);
        const int g = lane >> 2, t = lane & 3;
        float dbacc[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < NA; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int i = m0 + g + (e >> 1) * 8, j = n0 + 8 * nt + 2 * t + (e & 1);
            const float ee = (j <= i) ? __expf(fminf(sGs[i] - sGs[j], 0.f)) : 0.f;
            const float dmv = -dm[nt][e];
            if (j < i) dbacc[e >> 1] += dmv * sX[i * lda + j];   // sX already carries the decay factor
            sA[i * lda + j] = (j <= i) ? da[nt][e] * ee : 0.f;
            sX[i * lda + j] = (j < i) ? sBeta[i] * dmv * ee : 0.f;
          }
#pragma unroll
        for (int hr = 0; hr < 2; ++hr) {
          float x = dbacc[hr];
          x += __shfl_xor_sync(0xffffffffu, x, 1);
          x += __shfl_xor_sync(0xffffffffu, x, 2);
          if (t == 0) atomicAdd(&sdBeta[m0 + g + hr * 8], x);
        }
      }
    } else {
    for (int pid = tid; pid < C * C; pid += NTHR) {
      const int i = pid / C, j = pid % C;   // a warp covers 32 consecutive j of one row i
      float da = 0.f, dm = 0.f;
      if (j <= i) {
        for (int vv = 0; vv < VS; ++vv) {
          const float vn = sVn[j * ldv + vv];
          da += sdO[i * ldv + vv] * vn;
          dm -= sdR[i * ldv + vv] * vn;
        }
      }
      const float e = (j <= i) ? Eij(i, j) : 0.f;
      if (j < i) atomicAdd(&sdBeta[i], dm * sX[i * lda + j] * e);
      sA[i * lda + j] = (j <= i) ? da * e : 0.f;
      sX[i * lda + j] = (j < i) ? sBeta[i] * dm * e : 0.f;
    }
    }
    __syncthreads();
    // ---- per (row i, channel k): dQ^, dK^, dG, dbeta; lane = channel, warp = rows ----------------------------------
    if constexpr (TC) {
      // warp w owns rows 16*(w/NTW)..; the channel tiles are dealt to the NTW warps of a row panel in pairs.
      // Seven products per tile; products with the same B operand share its fetch, the A fragments are
      // fetched once per pair of tiles.
      const int g = lane >> 2, t = lane & 3;
      const int m0 = (warp / NTW) * 16;
      float dgrow[2] = {0.f, 0.f}, dbrow[2] = {0.f, 0.f}, extra = 0.f;
      const float row_eg[2] = {sEG[m0 + g], sEG[m0 + g + 8]}, row_el[2] = {sWd[m0 + g], sWd[m0 + g + 8]};
      const float row_beta[2] = {sBeta[m0 + g], sBeta[m0 + g + 8]};
      for (int n0 = (warp % NTW) * 16; n0 < K; n0 += 16 * NTW) {
        float dQg[2][4], dKg[2][4], dKt[2][4], rowA[2][4], rowX[2][4], colA[2][4], colX[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e)
            dQg[nt][e] = dKg[nt][e] = dKt[nt][e] = rowA[nt][e] = rowX[nt][e] = colA[nt][e] = colX[nt][e] = 0.f;
        rgemm2_p<2>(dQg, dKg, m0, n0, 0, VS, [&](int m, int k) { return ld2(sdO + m * ldv + k); },
                    [&](int m, int k) { return ld2(sdR + m * ldv + k); },
                    [&](int k, int nn) { return ld2(sS0 + nn * ldv + k); }, lane);
        rgemm_p<2>(dKt, m0, n0, 0, VS, [&](int m, int k) { return ld2(sVn + m * ldv + k); },
                   [&](int k, int nn) { return ld2(sdS + nn * ldv + k); }, lane);
        auto bK = [&](int k, int nn) { return sK[k * ldk + nn]; };
        // rows of dA, dX (lower: k <= m) ...
        rgemm2_p<2>(rowA, rowX, m0, n0, 0, m0 + 16, [&](int m, int k) { return ld2(sA + m * lda + k); },
                    [&](int m, int k) { return ld2(sX + m * lda + k); },
                    [&](int k, int nn) { return make_float2(sK[k * ldk + nn], sK[(k + 1) * ldk + nn]); }, lane);
        // ... and their columns (k >= m)
        rgemm<2>(colX, m0, n0, m0, C, [&](int m, int k) { return sX[k * lda + m]; }, bK, lane);
        rgemm<2>(colA, m0, n0, m0, C, [&](int m, int k) { return sA[k * lda + m]; },
                 [&](int k, int nn) { return sQ[k * ldq + nn]; }, lane);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int hr = 0; hr < 2; ++hr) {
            // two adjacent channels of one row: 8-byte accesses
            const int i = m0 + g + hr * 8, kk = n0 + 8 * nt + 2 * t;
            const float eg = row_eg[hr], el = row_el[hr], bi = row_beta[hr];
            const float2 qh = ld2(sQ + i * ldq + kk), kh = ld2(sK + i * ldk + kk);
            float2 dq, dk;
            {
              const int e = 2 * hr;
              dq.x = dQg[nt][e] * eg + rowA[nt][e];
              const float dk_row = -dKg[nt][e] * bi * eg + rowX[nt][e];
              const float dk_col = dKt[nt][e] * el + colA[nt][e] + colX[nt][e];
              dbrow[hr] += -dKg[nt][e] * kh.x * eg;
              dgrow[hr] += qh.x * dq.x + kh.x * (dk_row - dk_col);
              extra += dKt[nt][e] * kh.x * el;
              dk.x = dk_row + dk_col;
            }
            {
              const int e = 2 * hr + 1;
              dq.y = dQg[nt][e] * eg + rowA[nt][e];
              const float dk_row = -dKg[nt][e] * bi * eg + rowX[nt][e];
              const float dk_col = dKt[nt][e] * el + colA[nt][e] + colX[nt][e];
              dbrow[hr] += -dKg[nt][e] * kh.y * eg;
              dgrow[hr] += qh.y * dq.y + kh.y * (dk_row - dk_col);
              extra += dKt[nt][e] * kh.y * el;
              dk.y = dk_row + dk_col;
            }
            const int64_t at = slice_off + (acc_row0 + t0 + i) * K + kk;
            *reinterpret_cast<float2*>(p.dq_acc + at) = dq;
            *reinterpret_cast<float2*>(p.dk_acc + at) = dk;
          }
      }
#pragma unroll
      for (int hrow = 0; hrow < 2; ++hrow) {
        float db = dbrow[hrow], dg = dgrow[hrow];
        db += __shfl_xor_sync(0xffffffffu, db, 1); db += __shfl_xor_sync(0xffffffffu, db, 2);
        dg += __shfl_xor_sync(0xffffffffu, dg, 1); dg += __shfl_xor_sync(0xffffffffu, dg, 2);
        if (t == 0) {
          const int i = m0 + g + hrow * 8;
          atomicAdd(&sdBeta[i], db);
          if (p.dg_acc) atomicAdd(p.dg_acc + acc_row0 + t0 + i, dg);
        }
      }
      extra = warp_sum(extra);
      if (lane == 0 && p.dg_acc) atomicAdd(p.dg_acc + acc_row0 + t0 + C - 1, extra);
    } else {
    {
      const int nkk = K / 32 + (K % 32 ? 1 : 0);
      float extraL[4] = {0.f, 0.f, 0.f, 0.f};  // dG_L contribution, per channel slot of this lane (K <= 128)
      for (int i = warp; i < C; i += NW) {
        float dgrow = 0.f, dbrow = 0.f;
        for (int ks = 0; ks < nkk; ++ks) {
          const int kk = lane + 32 * ks;
          if (kk >= K) continue;
          float dQg = 0.f, dKg = 0.f, dKt = 0.f;
          for (int vv = 0; vv < VS; ++vv) {
            const float s0 = sS0[kk * ldv + vv];
            dQg += sdO[i * ldv + vv] * s0;
            dKg -= sdR[i * ldv + vv] * s0;
            dKt += sVn[i * ldv + vv] * sdS[kk * ldv + vv];
          }
          float rowA = 0.f, rowX = 0.f, colA = 0.f, colX = 0.f;
          if (KDA) {
            const float gi = sG[i * ldk + kk];
            for (int j = 0; j <= i; ++j) {
              const float e = __expf(fminf(gi - sG[j * ldk + kk], 0.f)) * sK[j * ldk + kk];
              rowA += sA[i * lda + j] * e;
              rowX += sX[i * lda + j] * e;
            }
            for (int i2 = i; i2 < C; ++i2) {
              const float e = __expf(fminf(sG[i2 * ldk + kk] - gi, 0.f));
              colA += sA[i2 * lda + i] * e * sQ[i2 * ldq + kk];
              colX += sX[i2 * lda + i] * e * sK[i2 * ldk + kk];
            }
          } else {
            for (int j = 0; j <= i; ++j) {
              const float kj = sK[j * ldk + kk];
              rowA += sA[i * lda + j] * kj;
              rowX += sX[i * lda + j] * kj;
            }
            for (int i2 = i; i2 < C; ++i2) {
              colA += sA[i2 * lda + i] * sQ[i2 * ldq + kk];
              colX += sX[i2 * lda + i] * sK[i2 * ldk + kk];
            }
          }
          const float eg = KDA ? __expf(sG[i * ldk + kk]) : sEG[i];
          const float el = KDA ? __expf(fminf(sG[(C - 1) * ldk + kk] - sG[i * ldk + kk], 0.f)) : sWd[i];
          const float qh = sQ[i * ldq + kk], kh = sK[i * ldk + kk];
          const float dq = dQg * eg + rowA;
          const float dk_row = dKg * sBeta[i] * eg + rowX;
          const float dk_col = dKt * el + colA + colX;
          dbrow += dKg * kh * eg;
          const float dG = qh * dq + kh * (dk_row - dk_col);
          extraL[ks] += dKt * kh * el;
          const int64_t arow = acc_row0 + t0 + i;
          p.dq_acc[slice_off + arow * K + kk] = dq;
          p.dk_acc[slice_off + arow * K + kk] = dk_row + dk_col;
          if (KDA) atomicAdd(p.dg_acc + arow * K + kk, dG);
          else dgrow += dG;
        }
        dbrow = warp_sum(dbrow);
        if (lane == 0) atomicAdd(&sdBeta[i], dbrow);
        if (!KDA && p.dg_acc) {
          dgrow = warp_sum(dgrow);
          if (lane == 0) atomicAdd(p.dg_acc + acc_row0 + t0 + i, dgrow);
        }
      }
      if (p.dg_acc) {
        const int64_t lrow = acc_row0 + t0 + C - 1;
        if (KDA) {
          for (int ks = 0; ks < nkk; ++ks)
            if (lane + 32 * ks < K) atomicAdd(p.dg_acc + lrow * K + lane + 32 * ks, extraL[ks]);
        } else {
          float e = extraL[0] + extraL[1] + extraL[2] + extraL[3];
          e = warp_sum(e);
          if (lane == 0) atomicAdd(p.dg_acc + lrow, e);
        }
      }
    }
    }
    // ---- dS0 = (Q^ e^G)^T dO + e^{G_L} dS1 - (beta K^ e^G)^T dR ; dG_L += e^{G_L} <dS1, S0> -------------------------
    if constexpr (TC) {
      // rows = channels k (panels of 16), columns = the VS value columns cut into NTW / 2 parts; the warps of one
      // column part take panels j, j + 8 (K <= 256)
      constexpr int CP = NTW / 2;            // column parts
      constexpr int NT = VS / 8 / CP;
      const int panel = warp / CP, n0 = (warp % CP) * 8 * NT;
      float keep[2][NT][4];
      const int g = lane >> 2, t = lane & 3;
      float tsum = 0.f;
#pragma unroll
      for (int slot = 0; slot < 2; ++slot) {
        const int m0 = (panel + 8 * slot) * 16;
        if (m0 < K) {
          float d[NT][4];
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) d[nt][0] = d[nt][1] = d[nt][2] = d[nt][3] = 0.f;
          rgemm<NT>(d, m0, n0, 0, C, [&](int m, int k) { return sEG[k] * sQ[k * ldq + m]; },
                    [&](int k, int nn) { return sdO[k * ldv + nn]; }, lane);
          rgemm<NT>(d, m0, n0, 0, C, [&](int m, int k) { return -sEG[k] * sBeta[k] * sK[k * ldk + m]; },
                    [&](int k, int nn) { return sdR[k * ldv + nn]; }, lane);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int kk = m0 + g + (e >> 1) * 8, vv = n0 + 8 * nt + 2 * t + (e & 1);
              const float ds1 = sdS[kk * ldv + vv];
              tsum += ds1 * sS0[kk * ldv + vv] * sEL[kk];
              keep[slot][nt][e] = d[nt][e] + sEL[kk] * ds1;
            }
        }
      }
      tsum = warp_sum(tsum);
      if (lane == 0 && p.dg_acc) atomicAdd(p.dg_acc + acc_row0 + t0 + C - 1, tsum);
      __syncthreads();
#pragma unroll
      for (int slot = 0; slot < 2; ++slot) {
        const int m0 = (panel + 8 * slot) * 16;
        if (m0 < K) {
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e)
              sdS[(m0 + g + (e >> 1) * 8) * ldv + n0 + 8 * nt + 2 * t + (e & 1)] = keep[slot][nt][e];
        }
      }
    } else {
    float ds_new[16];
    {
      const int vv = lane % VS, sub = lane / VS;
      constexpr int STREAMS = 32 / VS;
      int slot = 0;
      for (int kk = warp * STREAMS + sub; kk < K; kk += NW * STREAMS, ++slot) {
        float acc = 0.f;
        if constexpr (KDA && VS == 32) {
          acc = bcast_dot([&](int i) { return __expf(sG[i * ldk + kk]) * sQ[i * ldq + kk]; },
                          [&](int i) { return sdO[i * ldv + vv]; }, C, lane) -
                bcast_dot([&](int i) { return __expf(sG[i * ldk + kk]) * sBeta[i] * sK[i * ldk + kk]; },
                          [&](int i) { return sdR[i * ldv + vv]; }, C, lane);
        } else {
        for (int i = 0; i < C; ++i) {
          const float eg = KDA ? __expf(sG[i * ldk + kk]) : sEG[i];
          acc += eg * (sQ[i * ldq + kk] * sdO[i * ldv + vv] - sBeta[i] * sK[i * ldk + kk] * sdR[i * ldv + vv]);
        }
        }
        const float ds1 = sdS[kk * ldv + vv];
        float t = ds1 * sS0[kk * ldv + vv] * sEL[kk];
        // reduce over the VS value columns of this row stream
        for (int o = VS / 2; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (vv == 0 && p.dg_acc) {
          const int64_t lrow = acc_row0 + t0 + C - 1;
          if (KDA) atomicAdd(p.dg_acc + lrow * K + kk, t);
          else atomicAdd(p.dg_acc + lrow, t);
        }
        ds_new[slot] = acc + sEL[kk] * ds1;
      }
    }
    __syncthreads();
    {
      const int vv = lane % VS, sub = lane / VS;
      constexpr int STREAMS = 32 / VS;
      int slot = 0;
      for (int kk = warp * STREAMS + sub; kk < K; kk += NW * STREAMS, ++slot) sdS[kk * ldv + vv] = ds_new[slot];
    }
    }
    for (int c = tid; c < rows; c += NTHR) atomicAdd(p.dbeta + s_base + (t0 + c) * s_tok, sdBeta[c]);
  }
  __syncthreads();
  if (p.dh0) {
    for (int i = tid; i < K * VS; i += NTHR) {
      const int kk = i / VS, vv = i % VS;
      if (v0 + vv < V) p.dh0[((int64_t)unit * K + kk) * V + v0 + vv] = sdS[kk * ldv + vv];
    }
  }
}

// Chunk-parallel pre-pass of the tensor-core adjoint (bf16 inputs, C = 64): the pieces of a chunk that do not
// depend on the value slice -- X = tril(K^K^^T.E,-1), A = tril(Q^K^^T.E) and T = (I + diag(beta) X)^-1 -- computed
// once per chunk instead of once per slice, one CTA per (sequence, chunk), together with the normalised fp32
// rows q^, k^ themselves.  Output per chunk: [3][64][64] then [2][64][K] fp32.
// (T takes the place of A, which is written out before the inverse starts: two CTAs per SM at K = 128)
inline size_t bwd_pre_smem_bytes(int K) { return sizeof(float) * (2 * 64 * (size_t)(K + 4) + 2 * 64 * sm100::LDT + 128); }

__global__ void __launch_bounds__(kBwThreads, 2) bwd_pre_kernel(const BwdParams p) {
  extern __shared__ __align__(16) float smem[];
  const int K = p.K, T = p.map.T, N = p.N;
  constexpr int C = 64;
  const int ldk = K + 4, lda = sm100::LDT;
  float* sQ = smem;
  float* sK = sQ + C * ldk;
  float* sX = sK + C * ldk;
  float* sA = sX + C * lda;
  float* sT = sA;   // A leaves for global memory before the inverse writes T
  float* sGs = sA + C * lda;
  float* sBeta = sGs + 64;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int unit = blockIdx.x / N, n = blockIdx.x % N;
  const int b = unit / p.map.H, h = unit % p.map.H;
  const int64_t qk_base = p.map.base_qk(b, h, K), qk_tok = p.map.tok_qk(K);
  const int64_t s_base = p.map.base(b, h, 1), s_tok = p.map.tok(1);
  const bool gated = p.variant == DR_GATED;
  const int t0 = n * C, rows = min(C, T - t0);
  // ---- stage q^, k^ (fp32, normalised / scaled), g, beta: all global loads of the warp's eight rows first --------
  {
    const __nv_bfloat16* gq = reinterpret_cast<const __nv_bfloat16*>(p.q);
    const __nv_bfloat16* gk = reinterpret_cast<const __nv_bfloat16*>(p.k);
    uint2 qr[8][2], kr[8][2];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int c = warp + 8 * i;
#pragma unroll
      for (int ps = 0; ps < 2; ++ps) {
        const int ch = 128 * ps + 4 * lane;
        qr[i][ps] = make_uint2(0u, 0u); kr[i][ps] = make_uint2(0u, 0u);
        if (c < rows && ch < K) {
          qr[i][ps] = *reinterpret_cast<const uint2*>(gq + qk_base + (t0 + c) * qk_tok + ch);
          kr[i][ps] = *reinterpret_cast<const uint2*>(gk + qk_base + (t0 + c) * qk_tok + ch);
        }
      }
    }
    float bt = 0.f, gt_ = 0.f;
    if (lane < 8 && warp + 8 * lane < rows) {
      bt = p.beta[s_base + (t0 + warp + 8 * lane) * s_tok];
      if (gated) gt_ = ld_elem(p.g, s_base + (t0 + warp + 8 * lane) * s_tok, p.g_dt);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int c = warp + 8 * i;
      float qf[2][4], kf[2][4];
      float nq = 0.f, nk = 0.f;
#pragma unroll
      for (int ps = 0; ps < 2; ++ps) {
        const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qr[i][ps].x));
        const float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qr[i][ps].y));
        const float2 b0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&kr[i][ps].x));
        const float2 b1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&kr[i][ps].y));
        qf[ps][0] = a0.x; qf[ps][1] = a0.y; qf[ps][2] = a1.x; qf[ps][3] = a1.y;
        kf[ps][0] = b0.x; kf[ps][1] = b0.y; kf[ps][2] = b1.x; kf[ps][3] = b1.y;
#pragma unroll
        for (int e = 0; e < 4; ++e) { nq += qf[ps][e] * qf[ps][e]; nk += kf[ps][e] * kf[ps][e]; }
      }
      float qmul = p.scale, kmul = 1.f;
      if (p.l2norm) {
        nq = warp_sum(nq);
        nk = warp_sum(nk);
        qmul = p.scale / (sqrtf(nq) + 1e-6f);
        kmul = 1.f / (sqrtf(nk) + 1e-6f);
      }
#pragma unroll
      for (int ps = 0; ps < 2; ++ps) {
        const int ch = 128 * ps + 4 * lane;
        if (ch < K) {
          *reinterpret_cast<float4*>(sQ + c * ldk + ch) =
              make_float4(qf[ps][0] * qmul, qf[ps][1] * qmul, qf[ps][2] * qmul, qf[ps][3] * qmul);
          *reinterpret_cast<float4*>(sK + c * ldk + ch) =
              make_float4(kf[ps][0] * kmul, kf[ps][1] * kmul, kf[ps][2] * kmul, kf[ps][3] * kmul);
        }
      }
      if (lane == i) { sBeta[c] = bt; sGs[c] = gt_; }
    }
  }
  __syncthreads();
  if (tid == 0) {
    float acc = 0.f;
    for (int c = 0; c < C; ++c) { acc += sGs[c]; sGs[c] = acc; }
  }
  __syncthreads();
  // ---- X, A: the adjoint kernel's balanced triangular tasks (warp w: task w on K^, task 7-w on Q^) ---------------
  {
    const int g = lane >> 2, t = lane & 3;
#pragma unroll 1
    for (int pass = 0; pass < 2; ++pass) {
      const int task = pass ? 7 - warp : warp;
      const int i0 = task < 3 ? 48 : task < 5 ? 32 : task < 7 ? 16 : 0;
      const int nt0 = task < 3 ? 3 * task : task < 5 ? 3 * (task - 3) : task < 7 ? 2 * (task - 5) : 0;
      const int ntn = (task == 2 || task >= 5) ? 2 : 3;
      const float* arows = pass ? sQ : sK;
      float d[3][4];
#pragma unroll
      for (int nt = 0; nt < 3; ++nt) d[nt][0] = d[nt][1] = d[nt][2] = d[nt][3] = 0.f;
      for (int k0 = 0; k0 < K; k0 += 8) {
        uint32_t af[4];
        af[0] = __float_as_uint(arows[(i0 + g) * ldk + k0 + t]);
        af[1] = __float_as_uint(arows[(i0 + g + 8) * ldk + k0 + t]);
        af[2] = __float_as_uint(arows[(i0 + g) * ldk + k0 + t + 4]);
        af[3] = __float_as_uint(arows[(i0 + g + 8) * ldk + k0 + t + 4]);
#pragma unroll
        for (int nt = 0; nt < 3; ++nt) {
          if (nt < ntn) {
            uint32_t bf[2];
            bf[0] = __float_as_uint(sK[(8 * (nt0 + nt) + g) * ldk + k0 + t]);
            bf[1] = __float_as_uint(sK[(8 * (nt0 + nt) + g) * ldk + k0 + t + 4]);
            sm100::mma_tf32(d[nt], af, bf);
          }
        }
      }
#pragma unroll
      for (int nt = 0; nt < 3; ++nt) {
        if (nt < ntn) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int i = i0 + g + (e >> 1) * 8, j = 8 * (nt0 + nt) + 2 * t + (e & 1);
            const float v = d[nt][e] * __expf(fminf(sGs[i] - sGs[j], 0.f));
            if (pass) sA[i * lda + j] = (j <= i) ? v : 0.f;
            else sX[i * lda + j] = (j < i) ? v : 0.f;
          }
        }
      }
    }
    for (int e = tid; e < 64 * 64; e += kBwThreads) {
      const int i = e >> 6, j = e & 63;
      if ((j >> 3) > (i >> 4) * 2 + 1) { sX[i * lda + j] = 0.f; sA[i * lda + j] = 0.f; }
    }
  }
  __syncthreads();
  // ---- X, A, T -> [3][64][64]: A first (its array is reused for T), then the inverse, then X and T -----------------
  float* dst = p.pre + ((int64_t)unit * N + n) * (3 * 64 * 64 + 2 * 64 * K);
  for (int i = tid; i < 64 * 16; i += kBwThreads) {
    const int r = i >> 4, c4 = (i & 15) * 4;
    *reinterpret_cast<float4*>(dst + 4096 + r * 64 + c4) = *reinterpret_cast<const float4*>(sA + r * lda + c4);
  }
  __syncthreads();
  sm100::block_inverse_64(sX, sBeta, sT, tid);   // ends with a barrier of all 256 threads
  for (int i = tid; i < 3 * 64 * 16; i += kBwThreads) {
    const int m = i >> 10, r = (i >> 4) & 63, c4 = (i & 15) * 4;
    if (m == 1) continue;
    const float* src = (m == 0 ? sX : sT) + r * lda + c4;
    float4 v = *reinterpret_cast<const float4*>(src);
    if (m == 2) {   // the inverse leaves scratch above the diagonal: store zeros there
      if (c4 + 0 > r) v.x = 0.f;
      if (c4 + 1 > r) v.y = 0.f;
      if (c4 + 2 > r) v.z = 0.f;
      if (c4 + 3 > r) v.w = 0.f;
    }
    *reinterpret_cast<float4*>(dst + m * 4096 + r * 64 + c4) = v;
  }
  {
    float* qdst = dst + 3 * 4096;
    const int k4 = K >> 2;
    for (int i = tid; i < 2 * 64 * k4; i += kBwThreads) {
      const int m = i / (64 * k4), r = (i / k4) & 63, c4 = (i % k4) * 4;
      *reinterpret_cast<float4*>(qdst + (m * 64 + r) * K + c4) = *reinterpret_cast<const float4*>((m ? sK : sQ) + r * ldk + c4);
    }
  }
}

struct BwdFinalParams {
  const void* q; const void* k;
  void* dq; void* dk; float* dg;
  const float* dq_acc; const float* dk_acc; const float* dg_acc;
  SeqMap map;
  int K, C, N, variant, qkv_dt, l2norm, nvs;
  int64_t slice_stride;  // floats between the per-slice copies of dq_acc / dk_acc
  float scale;
};

// One CTA per (unit, chunk): sum of the partial copies, normalisation/scale chain rule per row, reverse
// cumulative sum of dG.
__global__ void __launch_bounds__(256) bwd_finalize_kernel(const BwdFinalParams p) {
  const int K = p.K, C = p.C, N = p.N, T = p.map.T;
  const int unit = blockIdx.x / N, n = blockIdx.x % N;
  const int b = unit / p.map.H, h = unit % p.map.H;
  const int t0 = n * C, rows = min(C, T - t0);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t qk_base = p.map.base_qk(b, h, K), qk_tok = p.map.tok_qk(K);
  const int64_t gk_base = p.map.base(b, h, K), gk_tok = p.map.tok(K);
  const int64_t s_base = p.map.base(b, h, 1), s_tok = p.map.tok(1);
  const int64_t acc_row0 = (int64_t)unit * N * C + t0;
  // Grouped value attention: the G = H / Hq value heads of a group share one q/k head, whose gradient is the sum
  // over the group.  The CTA of the group's first head adds all G x nvs partial copies (the chain rule of the
  // normalisation is linear in them); the others only have their dg to do.
  const int G = p.map.H / p.map.Hq;
  const int ncopies = G * p.nvs;
  const int64_t head_stride = (int64_t)N * C * K;   // floats between the accumulator rows of consecutive heads
  auto copy_off = [&](int ci) -> int64_t { return (int64_t)(ci / p.nvs) * head_stride + (int64_t)(ci % p.nvs) * p.slice_stride; };
  // lane = four consecutive channels (two groups of 128 channels for K > 128): 16-byte loads of the slice
  // partials, all of a row's loads issued before the first sum
  for (int c = warp; c < ((h % G) == 0 ? rows : 0); c += 8) {
    const float* aq0 = p.dq_acc + (acc_row0 + c) * K;
    const float* ak0 = p.dk_acc + (acc_row0 + c) * K;
    const int64_t grow = qk_base + (t0 + c) * qk_tok;
    float nq = 0.f, nk = 0.f, dq_q = 0.f, dk_k = 0.f;
    float aq[2][4], ak[2][4], qv[2][4], kv[2][4];
#pragma unroll
    for (int s2 = 0; s2 < 2; ++s2) {
      const int i = 4 * lane + 128 * s2;
#pragma unroll
      for (int e = 0; e < 4; ++e) { aq[s2][e] = 0.f; ak[s2][e] = 0.f; qv[s2][e] = 0.f; kv[s2][e] = 0.f; }
      if (i < K) {
        float4 xq[8], xk[8];   // the first eight copies in flight together (V <= 256 in 32-column slices, one head)
#pragma unroll
        for (int sl = 0; sl < 8; ++sl) {
          if (sl < ncopies) {
            xq[sl] = *reinterpret_cast<const float4*>(aq0 + copy_off(sl) + i);
            xk[sl] = *reinterpret_cast<const float4*>(ak0 + copy_off(sl) + i);
          }
        }
        for (int sl = 8; sl < ncopies; ++sl) {   // (head groups)
          const float4 a = *reinterpret_cast<const float4*>(aq0 + copy_off(sl) + i);
          const float4 bq = *reinterpret_cast<const float4*>(ak0 + copy_off(sl) + i);
          aq[s2][0] += a.x; aq[s2][1] += a.y; aq[s2][2] += a.z; aq[s2][3] += a.w;
          ak[s2][0] += bq.x; ak[s2][1] += bq.y; ak[s2][2] += bq.z; ak[s2][3] += bq.w;
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          qv[s2][e] = ld_elem(p.q, grow + i + e, p.qkv_dt);
          kv[s2][e] = ld_elem(p.k, grow + i + e, p.qkv_dt);
        }
#pragma unroll
        for (int sl = 0; sl < 8; ++sl) {
          if (sl < ncopies) {
            aq[s2][0] += xq[sl].x; aq[s2][1] += xq[sl].y; aq[s2][2] += xq[sl].z; aq[s2][3] += xq[sl].w;
            ak[s2][0] += xk[sl].x; ak[s2][1] += xk[sl].y; ak[s2][2] += xk[sl].z; ak[s2][3] += xk[sl].w;
          }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          nq += qv[s2][e] * qv[s2][e]; nk += kv[s2][e] * kv[s2][e];
          dq_q += qv[s2][e] * aq[s2][e]; dk_k += kv[s2][e] * ak[s2][e];
        }
      }
    }
    nq = sqrtf(warp_sum(nq)); nk = sqrtf(warp_sum(nk));
    dq_q = warp_sum(dq_q); dk_k = warp_sum(dk_k);
#pragma unroll
    for (int s2 = 0; s2 < 2; ++s2) {
      const int i = 4 * lane + 128 * s2;
      if (i >= K) continue;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float dq = p.scale * aq[s2][e], dk = ak[s2][e];
        if (p.l2norm) {
          const float rq = 1.f / (nq + 1e-6f), rk = 1.f / (nk + 1e-6f);
          // y = s x / (n + eps):  dx = s [ dy / (n + eps) - x (x.dy) / (n (n + eps)^2) ]
          dq = p.scale * (aq[s2][e] * rq - (nq > 0.f ? qv[s2][e] * dq_q * rq * rq / nq : 0.f));
          dk = ak[s2][e] * rk - (nk > 0.f ? kv[s2][e] * dk_k * rk * rk / nk : 0.f);
        }
        st_elem(p.dq, grow + i + e, p.qkv_dt, dq);
        st_elem(p.dk, grow + i + e, p.qkv_dt, dk);
      }
    }
  }
  if (p.variant == DR_GATED) {
    // dg = reverse cumulative sum of dG inside the chunk: one warp, two rows per lane
    if (warp == 0) {
      float a = lane < C ? p.dg_acc[acc_row0 + lane] : 0.f;
      float bq = lane + 32 < C ? p.dg_acc[acc_row0 + 32 + lane] : 0.f;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {   // inclusive suffix sums within each half
        const float ya = __shfl_down_sync(0xffffffffu, a, o);
        const float yb = __shfl_down_sync(0xffffffffu, bq, o);
        if (lane + o < 32) { a += ya; bq += yb; }
      }
      const float upper = __shfl_sync(0xffffffffu, bq, 0);   // total of rows 32..63
      a += upper;
      if (lane < rows) p.dg[s_base + (t0 + lane) * s_tok] = a;
      if (lane + 32 < rows) p.dg[s_base + (t0 + 32 + lane) * s_tok] = bq;
    }
  } else if (p.variant == DR_KDA) {
    for (int i = threadIdx.x; i < K; i += blockDim.x) {
      float acc = 0.f;
      for (int c = C - 1; c >= 0; --c) {
        acc += p.dg_acc[(acc_row0 + c) * K + i];
        if (c < rows) p.dg[gk_base + (t0 + c) * gk_tok + i] = acc;
      }
    }
  }
}

inline bool bwd_supported(const DrDesc* d) {
  return d->chunk <= 64 && d->K <= 128 && (d->variant != DR_KDA || d->K % 16 == 0);
}

// bf16 inputs with whole 16x8 tiles: the products of the adjoint run on the tensor cores (tf32); fp32 inputs
// stay on the exact CUDA-core path
inline bool bwd_tensor_core_path(const DrDesc* d) {
  return d->variant != DR_KDA && d->qkv_dtype == DR_BF16 && d->chunk == 64 && d->K % 16 == 0 && d->V % 8 == 0;
}

inline int64_t bwd_workspace_bytes(const DrDesc* d) {
  if (!bwd_supported(d)) return DR_ERR_UNSUPPORTED;
  const int64_t N = (d->T + d->chunk - 1) / d->chunk;
  const int64_t units = (int64_t)d->B * d->H;
  const int64_t rows = units * N * d->chunk;
  const int64_t nvs = (d->V + kBwSlice - 1) / kBwSlice;
  int64_t f = units * N * d->K * d->V + 2 * rows * d->K * nvs;
  if (d->variant == DR_GATED) f += rows;
  if (d->variant == DR_KDA) f += rows * d->K;
  if (bwd_tensor_core_path(d)) f += units * N * (3 * 64 * 64 + 2 * 64 * d->K);   // X, A, T, q^, k^ of every chunk
  return f * (int64_t)sizeof(float);
}

// Where the pieces of the backward workspace lie (all fp32): checkpoints | dq^ copies | dk^ copies | dG | pre-pass records.
struct BwdRegions {
  float *ckpt, *dq_acc, *dk_acc, *dg_acc, *pre;
  int64_t N, units, rows, nvs;
  size_t dg_floats;
};
inline BwdRegions bwd_regions(const DrDesc* d, void* workspace) {
  BwdRegions r;
  const int C = d->chunk, K = d->K, V = d->V;
  r.N = (d->T + C - 1) / C; r.units = (int64_t)d->B * d->H; r.rows = r.units * r.N * C;
  r.nvs = (V + kBwSlice - 1) / kBwSlice;
  r.ckpt = reinterpret_cast<float*>(workspace);
  r.dq_acc = r.ckpt + r.units * r.N * K * V;      // [nvs][rows][K], one copy per value slice (fully overwritten)
  r.dk_acc = r.dq_acc + r.nvs * r.rows * K;
  r.dg_floats = d->variant == DR_GATED ? r.rows : d->variant == DR_KDA ? r.rows * K : 0;
  r.dg_acc = d->variant == DR_DELTA ? nullptr : r.dk_acc + r.nvs * r.rows * K;
  r.pre = r.dk_acc + r.nvs * r.rows * K + r.dg_floats;   // [units][N][3][64][64] + q^, k^: tensor-core path only
  return r;
}

// The chunk-parallel pre-pass of the tensor-core adjoint (X, A, T, q^, k^ of every chunk).  It reads q, k, g, beta
// only, so it belongs to the forward half of a training step: launch_bwd_forward runs it beside the checkpointing
// forward, which at training batch sizes (one CTA per sequence) leaves most SMs idle.
inline cudaError_t launch_bwd_pre(const DrDesc* d, const void* q, const void* k, const void* g, const float* beta,
                                  void* workspace, cudaStream_t stream, int* launches) {
  const BwdRegions r = bwd_regions(d, workspace);
  BwdParams p{};
  p.q = q; p.k = k; p.g = g; p.beta = beta; p.pre = r.pre;
  p.map.B = d->B; p.map.H = d->H; p.map.T = d->T; p.map.bthd = d->layout == DR_LAYOUT_BTHD;
  p.map.Hq = d->qk_heads > 0 ? d->qk_heads : d->H;
  p.K = d->K; p.V = d->V; p.C = d->chunk; p.N = (int)r.N;
  p.variant = d->variant; p.qkv_dt = d->qkv_dtype; p.g_dt = d->g_dtype; p.l2norm = d->use_qk_l2norm; p.scale = d->scale;
  const size_t psmem = bwd_pre_smem_bytes(d->K);
  cudaError_t e = cudaFuncSetAttribute(bwd_pre_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)psmem);
  if (e != cudaSuccess) return e;
  bwd_pre_kernel<<<(unsigned)(r.units * r.N), kBwThreads, psmem, stream>>>(p);
  ++*launches;
  return cudaGetLastError();
}

// One non-blocking side stream per device, created on first use (the only stream the library owns).
inline cudaError_t bwd_side_stream(cudaStream_t* out) {
  static std::mutex mu;
  static cudaStream_t streams[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(mu);
  if (!streams[dev]) {
    e = cudaStreamCreateWithFlags(&streams[dev], cudaStreamNonBlocking);
    if (e != cudaSuccess) return e;
  }
  *out = streams[dev];
  return cudaSuccess;
}

// The checkpointing forward of the backward: state at the start of every chunk -> the head of the workspace.
// With o / hT given it is also the forward a training step needs (dr_chunk_fwd_saving), so that step runs one
// forward instead of two.  KDA at the tensor-core shape uses the two-kernel forward with its records parked in the
// accumulator part of the workspace (262 KB per chunk there against 82 KB of records; the adjoint overwrites it).
// own_stream: the pre-pass may run on the library's side stream, forked from and joined to `stream` with events
// (false for callers that must not create streams or events: the pre-pass then runs on `stream` before the forward).
inline cudaError_t launch_bwd_forward(const DrDesc* d, const void* q, const void* k, const void* v, const void* g,
                                      const float* beta, const float* h0, void* o, float* hT, void* workspace,
                                      int32_t* status, cudaStream_t stream, int* launches, bool own_stream = true) {
  const int C = d->chunk, K = d->K, V = d->V;
  cudaEvent_t joined = nullptr;
  if (d->variant != DR_KDA && bwd_tensor_core_path(d)) {
    cudaStream_t side = nullptr;
    cudaEvent_t forked = nullptr;
    if (own_stream && bwd_side_stream(&side) == cudaSuccess &&
        cudaEventCreateWithFlags(&forked, cudaEventDisableTiming) == cudaSuccess &&
        cudaEventCreateWithFlags(&joined, cudaEventDisableTiming) == cudaSuccess) {
      cudaError_t ef = cudaEventRecord(forked, stream);
      if (ef == cudaSuccess) ef = cudaStreamWaitEvent(side, forked, 0);
      if (ef == cudaSuccess) ef = launch_bwd_pre(d, q, k, g, beta, workspace, side, launches);
      if (ef == cudaSuccess) ef = cudaEventRecord(joined, side);
      cudaEventDestroy(forked);   // released once the work recorded in it has completed
      if (ef != cudaSuccess) { cudaEventDestroy(joined); return ef; }
    } else {
      if (forked) cudaEventDestroy(forked);
      if (joined) { cudaEventDestroy(joined); joined = nullptr; }
      const cudaError_t ep = launch_bwd_pre(d, q, k, g, beta, workspace, stream, launches);
      if (ep != cudaSuccess) return ep;
    }
  }
  const int64_t N = (d->T + C - 1) / C, units = (int64_t)d->B * d->H;
  float* ckpt = reinterpret_cast<float*>(workspace);
  FwdParams f;
  f.q = q; f.k = k; f.v = v; f.g = g; f.beta = beta; f.h0 = h0; f.o = o; f.hT = hT; f.status = status;
  f.ckpt = ckpt;
  f.map.B = d->B; f.map.H = d->H; f.map.T = d->T; f.map.bthd = d->layout == DR_LAYOUT_BTHD;
  f.map.Hq = d->qk_heads > 0 ? d->qk_heads : d->H;
  f.K = K; f.V = V; f.C = C;
  f.variant = d->variant; f.qkv_dt = d->qkv_dtype; f.g_dt = d->g_dtype; f.out_dt = o ? d->out_dtype : d->qkv_dtype;
  f.l2norm = d->use_qk_l2norm; f.scale = d->scale;
  f.set_extents();
  const bool tc_shape = sm100::kAvailable && K == 128 && V == 128 && C == 64 && d->qkv_dtype == DR_BF16;
  // the tensor-core forwards write the same checkpoints when the shape qualifies
  const bool fused = tc_shape && (d->variant == DR_DELTA || (d->variant == DR_GATED && d->g_dtype == DR_F32)) &&
                     (!o || d->out_dtype == DR_BF16);
  const bool split = tc_shape && !fused && d->variant == DR_KDA;
  cudaError_t e;
  if (fused) {
    e = sm100::launch_chunk(f, stream);
    ++*launches;
  } else if (split) {
    int n2 = 0;
    e = kda::launch_chunk(f, ckpt + units * N * K * V, stream, &n2);
    *launches += n2;
  } else {
    // every other shape: the token recurrence (the same function of the inputs as the chunk form, and on the CUDA
    // cores 4-11x faster than the fp32 chunk kernel) leaves the state at each chunk start on its way
    e = launch_recurrent(f, stream);
    ++*launches;
  }
  if (joined) {   // what follows on `stream` waits for the pre-pass as well
    const cudaError_t ej = cudaStreamWaitEvent(stream, joined, 0);
    cudaEventDestroy(joined);
    if (e == cudaSuccess) e = ej;
  }
  return e;
}

inline cudaError_t launch_bwd_adjoint(const DrDesc* d, const void* q, const void* k, const void* v, const void* g,
                                      const float* beta, const void* d_o, const float* d_hT, void* dq, void* dk,
                                      void* dv, float* dbeta, float* dg, float* dh0, void* workspace,
                                      cudaStream_t stream, int* launches) {
  const int C = d->chunk, K = d->K, V = d->V;
  const BwdRegions rg = bwd_regions(d, workspace);
  const int64_t N = rg.N, units = rg.units, rows = rg.rows, nvs = rg.nvs;
  float *ckpt = rg.ckpt, *dq_acc = rg.dq_acc, *dk_acc = rg.dk_acc, *dg_acc = rg.dg_acc, *pre = rg.pre;
  const size_t dg_floats = rg.dg_floats;
  cudaError_t e = cudaSuccess;
  if (dg_floats) e = cudaMemsetAsync(dg_acc, 0, dg_floats * sizeof(float), stream);
  if (e != cudaSuccess) return e;
  const size_t nbeta = (size_t)units * d->T;
  e = cudaMemsetAsync(dbeta, 0, nbeta * sizeof(float), stream);
  if (e != cudaSuccess) return e;
  SeqMap map;
  map.B = d->B; map.H = d->H; map.T = d->T; map.bthd = d->layout == DR_LAYOUT_BTHD;
  map.Hq = d->qk_heads > 0 ? d->qk_heads : d->H;
  // (2) adjoint
  BwdParams p;
  p.q = q; p.k = k; p.v = v; p.g = g; p.beta = beta; p.d_o = d_o; p.d_hT = d_hT;
  p.dv = dv; p.dbeta = dbeta; p.dh0 = dh0;
  p.ckpt = ckpt; p.dq_acc = dq_acc; p.dk_acc = dk_acc; p.dg_acc = dg_acc; p.pre = nullptr;
  p.map = map; p.K = K; p.V = V; p.C = C; p.N = (int)N;
  p.variant = d->variant; p.qkv_dt = d->qkv_dtype; p.g_dt = d->g_dtype; p.l2norm = d->use_qk_l2norm; p.scale = d->scale;
  if (d->variant == DR_KDA) {
    constexpr int VS = kBwSlice;
    const size_t smem = bwd_layout(C, K, VS, true).total * sizeof(float);
    e = cudaFuncSetAttribute(bwd_chunk_kernel<VS, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    bwd_chunk_kernel<VS, true, false><<<(unsigned)(units * ((V + VS - 1) / VS)), bwd_threads(false), smem, stream>>>(p);
  } else {
    constexpr int VS = 32;
    // bf16 inputs with whole 16x8 tiles: the products run on the tensor cores (tf32); fp32 inputs stay exact
    const bool tc = bwd_tensor_core_path(d);
    const size_t smem = bwd_layout(C, K, VS, false, tc).total * sizeof(float);
    if (tc) {
      // the slice-independent pieces (X, A, T, q^, k^ of every chunk) were left in the workspace by launch_bwd_forward
      p.pre = pre;
      e = cudaFuncSetAttribute(bwd_chunk_kernel<VS, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
      bwd_chunk_kernel<VS, false, true><<<(unsigned)(units * ((V + VS - 1) / VS)), bwd_threads(true), smem, stream>>>(p);
    } else {
      e = cudaFuncSetAttribute(bwd_chunk_kernel<VS, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
      bwd_chunk_kernel<VS, false, false><<<(unsigned)(units * ((V + VS - 1) / VS)), bwd_threads(false), smem, stream>>>(p);
    }
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  ++*launches;
  // (3) finalize
  BwdFinalParams fp;
  fp.q = q; fp.k = k; fp.dq = dq; fp.dk = dk; fp.dg = dg;
  fp.dq_acc = dq_acc; fp.dk_acc = dk_acc; fp.dg_acc = dg_acc;
  fp.map = map; fp.K = K; fp.C = C; fp.N = (int)N; fp.variant = d->variant; fp.qkv_dt = d->qkv_dtype;
  fp.l2norm = d->use_qk_l2norm; fp.scale = d->scale;
  fp.nvs = (int)nvs; fp.slice_stride = rows * K;
  bwd_finalize_kernel<<<(unsigned)(units * N), 256, 0, stream>>>(fp);
  ++*launches;
  return cudaGetLastError();
}

// forward recomputation + adjoint (dr_chunk_bwd)
inline cudaError_t launch_bwd(const DrDesc* d, const void* q, const void* k, const void* v, const void* g,
                              const float* beta, const float* h0, const void* d_o, const float* d_hT, void* dq,
                              void* dk, void* dv, float* dbeta, float* dg, float* dh0, void* workspace,
                              int32_t* status, cudaStream_t stream, int* launches, bool own_stream = true) {
  // only the forward has bounded waits that can report; the adjoint kernels synchronise with block barriers
  cudaError_t e = launch_bwd_forward(d, q, k, v, g, beta, h0, nullptr, nullptr, workspace, status, stream, launches,
                                     own_stream);
  if (e != cudaSuccess) return e;
  return launch_bwd_adjoint(d, q, k, v, g, beta, d_o, d_hT, dq, dk, dv, dbeta, dg, dh0, workspace, stream, launches);
}

}  // namespace dr
