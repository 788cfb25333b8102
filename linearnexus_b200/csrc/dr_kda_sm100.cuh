// Chunkwise forward with PER-CHANNEL decay (KDA) for Blackwell, as two kernels:
//
//   (1) intra_kernel   one CTA per (sequence, chunk), all chunks in parallel: everything that does not
//                      depend on the running state.  Cumulative log decay G, the decayed chunk-local
//                      products A_kk, A_qk, the unit-lower inverse T = (I + diag(beta) A_kk)^-1 and the
//                      bf16 operand tiles of the state pass, written to a workspace record per chunk in
//                      exactly the 8x8 core-matrix order the tensor cores read, so that the state kernel
//                      fetches each tile with ONE 1-d bulk copy (no tensor map).
//   (2) state_kernel   one CTA per sequence walks the chunks; the fp32 state lives transposed in tensor
//                      memory (lane = value column) and every product is a tcgen05.mma:
//                          U^T      = V^T (T diag(beta))^T                   128x64x64   smem x smem
//                          Vn^T     = U^T - S^T W^T                          128x64x128  tmem x smem
//                          Dq       = S^T Qg^T                               128x64x128
//                          Do       = Vn^T A_qk^T                            128x64x64
//                          S^T      = S^T diag(e^{G_L}) + Vn^T Kd            128x128x64
//                      with W = T diag(beta) (k^ e^G), Qg = scale q^ e^G, Kd = k^ e^{G_L - G}.
//
// Per-channel decay cannot be folded into row/column factors of a plain K K^T product the way a scalar
// decay can, and e^{-G} alone overflows for strong decay.  The chunk-local products therefore use 16-row
// sub-blocks: an off-diagonal block (rows in sub-block bi, columns in an earlier sub-block) is the
// bf16 tensor-core product of  x_i e^{G_i - G_n}  and  k_j e^{G_n - G_j}  with n the first row of bi, so
// both exponents are <= 0; the four diagonal 16x16 blocks are summed exactly in fp32 on the CUDA cores.
//
// Shape: K = V = 128, chunk 64, bf16 q/k/v, g bf16 or fp32 ([.., K] for KDA; the scalar-decay and
// decay-free variants are served too, by broadcasting), fp32 beta/state, bf16 or fp32 output.
#pragma once

#include "dr_chunk_sm100.cuh"

namespace dr {
namespace kda {

using sm100::LDT;
using sm100::RBS;
using sm100::A_RBS;

constexpr int kC = 64, kD = 128;
constexpr int kThreads = 256;

// workspace record of one chunk (bytes); every tile in 8x8 core-matrix order
constexpr int WS_W = 0;                    // W   [64][128] bf16
constexpr int WS_QG = WS_W + 16384;        // Qg  [64][128] bf16
constexpr int WS_KD = WS_QG + 16384;       // Kd  [64][128] bf16
constexpr int WS_V = WS_KD + 16384;        // V   [64][128] bf16 (rows past the end of the sequence zero)
constexpr int WS_TB = WS_V + 16384;        // T diag(beta) [64][64] bf16
constexpr int WS_AQK = WS_TB + 8192;       // A_qk         [64][64] bf16
constexpr int WS_EGL = WS_AQK + 8192;      // e^{G_L}[128] fp32
constexpr int WS_REC = WS_EGL + 512;       // 82432

inline int64_t workspace_bytes(int64_t units, int T) { return units * ((T + kC - 1) / kC) * (int64_t)WS_REC; }

// ---- intra-chunk kernel ------------------------------------------------------------------------------------
constexpr int LDF = 132;   // row stride (floats) of the [64][128] fp32 arrays
constexpr int LDH = 136;   // row stride (bf16) of the [..][128] bf16 operand arrays (conflict-free fragments)
constexpr int IN_G = 0;                          // G      fp32 [64][132]
constexpr int IN_K = IN_G + 64 * LDF * 4;        // k^ (later k^ e^G)
constexpr int IN_Q = IN_K + 64 * LDF * 4;        // scale q^ (later W staging)
constexpr int IN_QP = IN_Q + 64 * LDF * 4;       // q+ bf16 [64][136]
constexpr int IN_KP = IN_QP + 64 * LDH * 2;      // k+ bf16 [64][136]
constexpr int IN_KM = IN_KP + 64 * LDH * 2;      // k- bf16 [96][136]: versions for sub-blocks 1,2,3 (16,32,48 rows)
constexpr int IN_AKK = IN_KM + 96 * LDH * 2;     // A_kk fp32 [64][68]
constexpr int IN_AQK = IN_AKK + 64 * LDT * 4;    // A_qk fp32 [64][68]
constexpr int IN_T = IN_AQK + 64 * LDT * 4;      // T    fp32 [64][68]
constexpr int IN_BETA = IN_T + 64 * LDT * 4;     // beta[64]
constexpr int IN_TOTAL = IN_BETA + 64 * 4;

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// four consecutive elements starting at element index i (a multiple of 4)
__device__ __forceinline__ void ld4(const void* p, int64_t i, int dt, float (&x)[4]) {
  if (dt == DR_BF16) {
    const uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p) + i);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
  } else {
    const float4 f = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
    x[0] = f.x; x[1] = f.y; x[2] = f.z; x[3] = f.w;
  }
}

// 16-byte piece number `piece` of a [64][128] tile in core-matrix order -> (row, first column)
__device__ __forceinline__ void piece128(int piece, int& row, int& col) {
  row = (piece >> 7) * 8 + (piece & 7);
  col = ((piece >> 3) & 15) * 8;
}
// same for a [64][64] tile
__device__ __forceinline__ void piece64(int piece, int& row, int& col) {
  row = (piece >> 6) * 8 + (piece & 7);
  col = ((piece >> 3) & 7) * 8;
}
__device__ __forceinline__ uint4 pack8(const float (&x)[8]) {
  uint4 u;
  u.x = tc::pack_bf16(x[0], x[1]); u.y = tc::pack_bf16(x[2], x[3]);
  u.z = tc::pack_bf16(x[4], x[5]); u.w = tc::pack_bf16(x[6], x[7]);
  return u;
}

__global__ void __launch_bounds__(kThreads, 1) intra_kernel(const FwdParams p, uint8_t* __restrict__ ws) {
  extern __shared__ __align__(1024) uint8_t smem[];
  float* sG = reinterpret_cast<float*>(smem + IN_G);
  float* sK = reinterpret_cast<float*>(smem + IN_K);
  float* sQ = reinterpret_cast<float*>(smem + IN_Q);
  __nv_bfloat16* sQp = reinterpret_cast<__nv_bfloat16*>(smem + IN_QP);
  __nv_bfloat16* sKp = reinterpret_cast<__nv_bfloat16*>(smem + IN_KP);
  __nv_bfloat16* sKm = reinterpret_cast<__nv_bfloat16*>(smem + IN_KM);
  float* sAkk = reinterpret_cast<float*>(smem + IN_AKK);
  float* sAqk = reinterpret_cast<float*>(smem + IN_AQK);
  float* sT = reinterpret_cast<float*>(smem + IN_T);
  float* sBeta = reinterpret_cast<float*>(smem + IN_BETA);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int T = p.map.T;
  const int nchunks = (T + kC - 1) / kC;
  const int unit = blockIdx.x / nchunks, n = blockIdx.x % nchunks;
  const int b = unit / p.map.H, h = unit % p.map.H;
  const int t0 = n * kC, rows = min(kC, T - t0);
  const int64_t qk_base = p.map.base(b, h, kD), qk_tok = p.map.tok(kD);
  const int64_t s_base = p.map.base(b, h, 1), s_tok = p.map.tok(1);
  uint8_t* rec = ws + ((int64_t)unit * nchunks + n) * WS_REC;

  // ---- load: k^ = k / (|k| + eps), scale q^, raw log decay; lane = four channels, warp = rows ------------
  for (int c = warp; c < kC; c += 8) {
    const bool live = c < rows;
    float qv[4] = {0.f, 0.f, 0.f, 0.f}, kv[4] = {0.f, 0.f, 0.f, 0.f}, gv[4] = {0.f, 0.f, 0.f, 0.f};
    if (live) {
      const int64_t at = qk_base + (t0 + c) * qk_tok + 4 * lane;
      ld4(p.q, at, DR_BF16, qv);
      ld4(p.k, at, DR_BF16, kv);
      if (p.variant == DR_KDA) {
        ld4(p.g, at, p.g_dt, gv);
      } else if (p.variant == DR_GATED) {
        const float gs = ld_elem(p.g, s_base + (t0 + c) * s_tok, p.g_dt);
        gv[0] = gv[1] = gv[2] = gv[3] = gs;
      }
    }
    float qmul = p.scale, kmul = 1.f;
    if (p.l2norm) {
      const float nq = warp_sum(qv[0] * qv[0] + qv[1] * qv[1] + qv[2] * qv[2] + qv[3] * qv[3]);
      const float nk = warp_sum(kv[0] * kv[0] + kv[1] * kv[1] + kv[2] * kv[2] + kv[3] * kv[3]);
      qmul = p.scale / (sqrtf(nq) + 1e-6f);
      kmul = 1.f / (sqrtf(nk) + 1e-6f);
    }
    *reinterpret_cast<float4*>(sQ + c * LDF + 4 * lane) = make_float4(qv[0] * qmul, qv[1] * qmul, qv[2] * qmul, qv[3] * qmul);
    *reinterpret_cast<float4*>(sK + c * LDF + 4 * lane) = make_float4(kv[0] * kmul, kv[1] * kmul, kv[2] * kmul, kv[3] * kmul);
    *reinterpret_cast<float4*>(sG + c * LDF + 4 * lane) = make_float4(gv[0], gv[1], gv[2], gv[3]);
    if (lane == 0) sBeta[c] = live ? p.beta[s_base + (t0 + c) * s_tok] : 0.f;
  }
  for (int i = tid; i < 64 * LDT; i += kThreads) { sAkk[i] = 0.f; sAqk[i] = 0.f; }
  // V rows -> the record's tile, 16 bytes per piece (coalesced writes)
  {
    const __nv_bfloat16* gv = reinterpret_cast<const __nv_bfloat16*>(p.v);
    const int64_t v_base = p.map.base(b, h, kD), v_tok = p.map.tok(kD);
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int piece = tid + kThreads * it;
      int row, col;
      piece128(piece, row, col);
      uint4 u = make_uint4(0u, 0u, 0u, 0u);
      if (row < rows) u = *reinterpret_cast<const uint4*>(gv + v_base + (t0 + row) * v_tok + col);
      *reinterpret_cast<uint4*>(rec + WS_V + piece * 16) = u;
    }
  }
  __syncthreads();
  // ---- G = inclusive prefix sum of the log decay over the rows of the chunk, per channel ---------------------
  {
    const int ch = tid & 127, half = tid >> 7;
    float acc = 0.f;
    for (int r = 0; r < 32; ++r) {
      acc += sG[(32 * half + r) * LDF + ch];
      sG[(32 * half + r) * LDF + ch] = acc;
    }
    __syncthreads();
    if (half) {
      const float add = sG[31 * LDF + ch];
      for (int r = 32; r < 64; ++r) sG[r * LDF + ch] += add;
    }
    __syncthreads();
  }
  // ---- bf16 operands of the off-diagonal sub-blocks -----------------------------------------------------------
  //   q+_i = scale q^_i e^{G_i - G_n(i)},  k+_i = k^_i e^{G_i - G_n(i)},  n(i) = first row of i's sub-block
  //   k-_{bi,j} = k^_j e^{G_{16 bi} - G_j}  for j < 16 bi
  for (int idx = tid; idx < 64 * 64; idx += kThreads) {
    const int i = idx >> 6, c2 = (idx & 63) * 2, nrow = i & ~15;
    const float e0 = __expf(sG[i * LDF + c2] - sG[nrow * LDF + c2]);
    const float e1 = __expf(sG[i * LDF + c2 + 1] - sG[nrow * LDF + c2 + 1]);
    *reinterpret_cast<uint32_t*>(sQp + i * LDH + c2) = tc::pack_bf16(sQ[i * LDF + c2] * e0, sQ[i * LDF + c2 + 1] * e1);
    *reinterpret_cast<uint32_t*>(sKp + i * LDH + c2) = tc::pack_bf16(sK[i * LDF + c2] * e0, sK[i * LDF + c2 + 1] * e1);
  }
  for (int idx = tid; idx < 96 * 64; idx += kThreads) {
    const int r = idx >> 6, c2 = (idx & 63) * 2;
    const int bi = r < 16 ? 1 : r < 48 ? 2 : 3;
    const int j = r - (bi == 1 ? 0 : bi == 2 ? 16 : 48);
    const float e0 = __expf(sG[16 * bi * LDF + c2] - sG[j * LDF + c2]);
    const float e1 = __expf(sG[16 * bi * LDF + c2 + 1] - sG[j * LDF + c2 + 1]);
    *reinterpret_cast<uint32_t*>(sKm + r * LDH + c2) = tc::pack_bf16(sK[j * LDF + c2] * e0, sK[j * LDF + c2 + 1] * e1);
  }
  __syncthreads();
  // ---- off-diagonal 16x16 blocks on mma.sync (bf16): 6 blocks x {k,q} x two 8-column halves = 24 tiles --------
  for (int x = 0; x < 3; ++x) {
    const int task = warp * 3 + x;
    const int bp = task >> 2, isq = (task >> 1) & 1, nt = task & 1;
    const int bi = bp == 0 ? 1 : bp < 3 ? 2 : 3;
    const int jb = bp == 0 ? 0 : bp < 3 ? bp - 1 : bp - 3;
    const __nv_bfloat16* arow = (isq ? sQp : sKp) + (16 * bi + g) * LDH;
    const __nv_bfloat16* brow = sKm + ((bi == 1 ? 0 : bi == 2 ? 16 : 48) + 16 * jb + 8 * nt + g) * LDH;
    float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const int k0 = ks * 16 + 2 * t;
      uint32_t a[4], bb[2];
      a[0] = *reinterpret_cast<const uint32_t*>(arow + k0);
      a[1] = *reinterpret_cast<const uint32_t*>(arow + 8 * LDH + k0);
      a[2] = *reinterpret_cast<const uint32_t*>(arow + k0 + 8);
      a[3] = *reinterpret_cast<const uint32_t*>(arow + 8 * LDH + k0 + 8);
      bb[0] = *reinterpret_cast<const uint32_t*>(brow + k0);
      bb[1] = *reinterpret_cast<const uint32_t*>(brow + k0 + 8);
      mma_bf16(d, a, bb);
    }
    float* out = (isq ? sAqk : sAkk) + (16 * bi + g) * LDT + 16 * jb + 8 * nt + 2 * t;
    *reinterpret_cast<float2*>(out) = make_float2(d[0], d[1]);
    *reinterpret_cast<float2*>(out + 8 * LDT) = make_float2(d[2], d[3]);
  }
  // ---- diagonal 16x16 blocks exactly (fp32): warp = two rows of every block, lane = four channels -------------
  for (int blk = 0; blk < 4; ++blk) {
#pragma unroll 1
    for (int sel = 0; sel < 2; ++sel) {
      const int rr = sel ? 15 - warp : warp;
      const int i = 16 * blk + rr;
      const float4 qi = *reinterpret_cast<const float4*>(sQ + i * LDF + 4 * lane);
      const float4 ki = *reinterpret_cast<const float4*>(sK + i * LDF + 4 * lane);
      const float4 gi = *reinterpret_cast<const float4*>(sG + i * LDF + 4 * lane);
      for (int jg = 0; jg <= rr; jg += 4) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          v[u] = 0.f; v[u + 4] = 0.f;
          if (jg + u <= rr) {
            const int j = 16 * blk + jg + u;
            const float4 kj = *reinterpret_cast<const float4*>(sK + j * LDF + 4 * lane);
            const float4 gj = *reinterpret_cast<const float4*>(sG + j * LDF + 4 * lane);
            const float w0 = kj.x * __expf(gi.x - gj.x), w1 = kj.y * __expf(gi.y - gj.y);
            const float w2 = kj.z * __expf(gi.z - gj.z), w3 = kj.w * __expf(gi.w - gj.w);
            v[u] = ki.x * w0 + ki.y * w1 + ki.z * w2 + ki.w * w3;
            v[u + 4] = qi.x * w0 + qi.y * w1 + qi.z * w2 + qi.w * w3;
          }
        }
        // eight sums over the 32 lanes in nine shuffles: each level halves the number of live values
        const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4;
        float x4[4], y2[2];
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
          const float keep = b4 ? v[k4 + 4] : v[k4], send = b4 ? v[k4] : v[k4 + 4];
          x4[k4] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
        }
#pragma unroll
        for (int k2 = 0; k2 < 2; ++k2) {
          const float keep = b3 ? x4[k2 + 2] : x4[k2], send = b3 ? x4[k2] : x4[k2 + 2];
          y2[k2] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
        }
        float z = (b2 ? y2[1] : y2[0]) + __shfl_xor_sync(0xffffffffu, b2 ? y2[0] : y2[1], 4);
        z += __shfl_xor_sync(0xffffffffu, z, 2);
        z += __shfl_xor_sync(0xffffffffu, z, 1);
        if (t == 0) {
          const int idx = (b4 ? 4 : 0) + (b3 ? 2 : 0) + (b2 ? 1 : 0);
          const int jj = jg + (idx & 3);
          if (idx >= 4) { if (jj <= rr) sAqk[i * LDT + 16 * blk + jj] = z; }
          else if (jj < rr) sAkk[i * LDT + 16 * blk + jj] = z;
        }
      }
    }
  }
  __syncthreads();
  // ---- T = (I + diag(beta) A_kk)^-1 -----------------------------------------------------------------------------
  sm100::block_inverse_64(sAkk, sBeta, sT, tid);
  // ---- record tiles: T diag(beta), A_qk, Qg = scale q^ e^G, Kd = k^ e^{G_L - G}, e^{G_L} ------------------------
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    const int piece = tid + kThreads * it;
    int row, col;
    piece64(piece, row, col);
    float a[8], c[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int j = col + e;
      a[e] = j <= row ? sT[row * LDT + j] * sBeta[j] : 0.f;
      c[e] = j <= row ? sAqk[row * LDT + j] : 0.f;
    }
    *reinterpret_cast<uint4*>(rec + WS_TB + piece * 16) = pack8(a);
    *reinterpret_cast<uint4*>(rec + WS_AQK + piece * 16) = pack8(c);
  }
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int piece = tid + kThreads * it;
    int row, col;
    piece128(piece, row, col);
    float a[8], c[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float gg = sG[row * LDF + col + e];
      a[e] = sQ[row * LDF + col + e] * __expf(gg);
      c[e] = sK[row * LDF + col + e] * __expf(sG[63 * LDF + col + e] - gg);
    }
    *reinterpret_cast<uint4*>(rec + WS_QG + piece * 16) = pack8(a);
    *reinterpret_cast<uint4*>(rec + WS_KD + piece * 16) = pack8(c);
  }
  if (tid < kD) reinterpret_cast<float*>(rec + WS_EGL)[tid] = __expf(sG[63 * LDF + tid]);
  __syncthreads();
  for (int idx = tid; idx < 64 * 128; idx += kThreads) {
    const int r = idx >> 7, c = idx & 127;
    sK[r * LDF + c] *= __expf(sG[r * LDF + c]);
  }
  __syncthreads();
  // ---- W = (T diag(beta)) (k^ e^G): 64x128x64 on mma.sync (tf32); warp = 16 rows x 64 channels -------------------
  {
    const int m0 = (warp >> 1) * 16, nb = (warp & 1) * 64;
    float d[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) { d[nt][0] = d[nt][1] = d[nt][2] = d[nt][3] = 0.f; }
    const int r0 = m0 + g, r1 = r0 + 8;
    for (int ks = 0; ks * 8 <= m0 + 15; ++ks) {
      const int k0 = ks * 8 + t, k1 = k0 + 4;
      uint32_t a[4];
      a[0] = sm100::to_tf32(k0 <= r0 ? sT[r0 * LDT + k0] * sBeta[k0] : 0.f);
      a[1] = sm100::to_tf32(k0 <= r1 ? sT[r1 * LDT + k0] * sBeta[k0] : 0.f);
      a[2] = sm100::to_tf32(k1 <= r0 ? sT[r0 * LDT + k1] * sBeta[k1] : 0.f);
      a[3] = sm100::to_tf32(k1 <= r1 ? sT[r1 * LDT + k1] * sBeta[k1] : 0.f);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        uint32_t bb[2];
        bb[0] = sm100::to_tf32(sK[k0 * LDF + nb + nt * 8 + g]);
        bb[1] = sm100::to_tf32(sK[k1 * LDF + nb + nt * 8 + g]);
        sm100::mma_tf32(d[nt], a, bb);
      }
    }
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      *reinterpret_cast<float2*>(sQ + r0 * LDF + nb + nt * 8 + 2 * t) = make_float2(d[nt][0], d[nt][1]);
      *reinterpret_cast<float2*>(sQ + r1 * LDF + nb + nt * 8 + 2 * t) = make_float2(d[nt][2], d[nt][3]);
    }
  }
  __syncthreads();
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int piece = tid + kThreads * it;
    int row, col;
    piece128(piece, row, col);
    float a[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) a[e] = sQ[row * LDF + col + e];
    *reinterpret_cast<uint4*>(rec + WS_W + piece * 16) = pack8(a);
  }
}

// ---- state kernel ----------------------------------------------------------------------------------------------
// tensor-memory columns
constexpr uint32_t TM_S = 0;      // S^T fp32                        128
constexpr uint32_t TM_SB = 128;   // bf16 copy of S^T (A operand)      64
constexpr uint32_t TM_DU = 192;   // 2 x 64: U^T -> Vn^T -> Do
constexpr uint32_t TM_DQ = 320;   // S^T Qg^T                          64
constexpr uint32_t TM_VA = 384;   // Vn^T bf16                         32
constexpr uint32_t TM_COLS = 512;
// shared memory: two record buffers, then the fp32 output staging tile [64][128]
constexpr int ST_O = 2 * WS_REC;
constexpr int ST_TOTAL = ST_O + 64 * 128 * 4;

struct StateCtl {
  uint64_t full[2], bar1, bar2;
  uint32_t tmem_base;
  int abort;
};

__global__ void __launch_bounds__(kThreads, 1) state_kernel(const FwdParams p, const uint8_t* __restrict__ ws) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ __align__(8) StateCtl ctl;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int hs = tid >> 7, l128 = tid & 127;
  const int T = p.map.T, nchunks = (T + kC - 1) / kC;
  const int unit = blockIdx.x;
  const int b = unit / p.map.H, h = unit % p.map.H;
  const int64_t o_base = p.map.base(b, h, kD), o_tok = p.map.tok(kD);
  const uint8_t* recs = ws + (int64_t)unit * nchunks * WS_REC;

  if (warp == 0) {
    tc::tmem_alloc(tc::smem_u32(&ctl.tmem_base), TM_COLS);
    tc::tmem_relinquish();
  }
  if (tid == 0) {
    tc::mbar_init(tc::smem_u32(&ctl.full[0]), 1);
    tc::mbar_init(tc::smem_u32(&ctl.full[1]), 1);
    tc::mbar_init(tc::smem_u32(&ctl.bar1), 1);
    tc::mbar_init(tc::smem_u32(&ctl.bar2), 1);
    tc::fence_mbar_init();
    ctl.abort = 0;
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tbase = ctl.tmem_base;
  const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
  volatile int* abort_p = &ctl.abort;
  auto wait_bar = [&](uint64_t* bar, uint32_t parity) {
    if (!*abort_p) {
      if (!tc::mbar_wait_bounded(tc::smem_u32(bar), parity, sm100::kWaitLimit)) {
        *abort_p = 1;
        if (p.status) atomicOr(p.status, DR_DEV_TIMEOUT);
      }
    }
  };
  // the whole record of chunk m -> buffer m & 1, one bulk copy (the record is contiguous)
  auto issue_load = [&](int m) {
    const uint32_t bar = tc::smem_u32(&ctl.full[m & 1]);
    tc::mbar_arrive_expect_tx(bar, WS_REC);
    const uint32_t dst = tc::smem_u32(smem + (m & 1) * WS_REC);
    const uint8_t* src = recs + (int64_t)m * WS_REC;
    // four copies so that several are in flight
    constexpr int Q4 = WS_REC / 4;   // 20608, a multiple of 16
#pragma unroll
    for (int i = 0; i < 4; ++i) tc::bulk_g2s(dst + i * Q4, src + i * Q4, Q4, bar);
  };
  if (tid == 0) {
    if (nchunks > 0) issue_load(0);
    if (nchunks > 1) issue_load(1);
  }

  const uint32_t id_n64 = tc::idesc_bf16(128, 64, 0, 0);
  const uint32_t id_n64_amn = tc::idesc_bf16(128, 64, 1, 0);
  const uint32_t id_n64_neg = id_n64 | (1u << 13);
  const uint32_t id_n128_bmn = tc::idesc_bf16(128, 128, 0, 1);

  // initial state: S^T[v][k] = h0[k][v]
  {
    const float* h0 = p.h0 ? p.h0 + (int64_t)unit * kD * kD : nullptr;
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
      const int c0 = 64 * hs + 32 * cc;
      uint32_t r[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) r[j] = h0 ? __float_as_uint(h0[(c0 + j) * kD + l128]) : 0u;
      tc::tmem_st32(tbase + TM_S + lane_addr + c0, r);
    }
    tc::tc_wait_st();
  }
  float* sO = reinterpret_cast<float*>(smem + ST_O);
  // O^T of chunk m = Dq + Do -> staging tile -> rows of the output
  auto output_epilogue = [&](int m) {
    const int t0m = m * kC, rowsm = min(kC, T - t0m);
    {
      const int c0 = 32 * hs;
      uint32_t rq[32], ro[32];
      tc::tmem_ld32(tbase + TM_DQ + lane_addr + c0, rq);
      tc::tmem_ld32(tbase + TM_DU + 64 * (m & 1) + lane_addr + c0, ro);
      tc::tc_wait_ld();
#pragma unroll
      for (int j = 0; j < 32; ++j) sO[(c0 + j) * kD + l128] = __uint_as_float(rq[j]) + __uint_as_float(ro[j]);
    }
    tc::tc_fence_before();
    __syncthreads();
    if (p.o) {
      const int r = tid >> 2, qtr = tid & 3;
      if (r < rowsm) {
        const float* src = sO + r * kD + 32 * qtr;
        const int64_t at = o_base + (int64_t)(t0m + r) * o_tok + 32 * qtr;
        if (p.out_dt == DR_BF16) {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.o) + at;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float x[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) x[e] = src[8 * j + e];
            reinterpret_cast<uint4*>(dst)[j] = pack8(x);
          }
        } else {
          float* dst = reinterpret_cast<float*>(p.o) + at;
#pragma unroll
          for (int j = 0; j < 8; ++j) reinterpret_cast<float4*>(dst)[j] = reinterpret_cast<const float4*>(src)[j];
        }
      }
    }
  };

  uint32_t ph1 = 0, ph2 = 0;
  for (int n = 0; n < nchunks; ++n) {
    const int s = n & 1;
    const uint8_t* st = smem + s * WS_REC;
    const uint32_t aW = tc::smem_u32(st + WS_W), aQg = tc::smem_u32(st + WS_QG), aKd = tc::smem_u32(st + WS_KD);
    const uint32_t aV = tc::smem_u32(st + WS_V), aTb = tc::smem_u32(st + WS_TB), aAqk = tc::smem_u32(st + WS_AQK);
    const float* sEGL = reinterpret_cast<const float*>(st + WS_EGL);
    wait_bar(&ctl.full[s], (n >> 1) & 1);
    tc::tc_fence_after();
    // ---- state pass: bf16 copy of S^T for the products; fp32 master decayed per key channel -------------------
    {
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c0 = 64 * hs + 32 * cc;
        uint32_t r[32], pk[16];
        tc::tmem_ld32(tbase + TM_S + lane_addr + c0, r);
        tc::tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j) pk[j] = tc::pack_bf16(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
        if (p.ckpt) {
          float* ck = p.ckpt + ((int64_t)unit * nchunks + n) * kD * kD;
#pragma unroll
          for (int j = 0; j < 32; ++j) ck[(c0 + j) * kD + l128] = __uint_as_float(r[j]);
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * sEGL[c0 + j]);
        tc::tmem_st16(tbase + TM_SB + lane_addr + c0 / 2, pk);
        tc::tmem_st32(tbase + TM_S + lane_addr + c0, r);
      }
      tc::tc_wait_st();
    }
    tc::tc_fence_before();
    __syncthreads();
    // ---- U^T = V^T Tb^T, then Vn^T = U^T - S^T W^T ---------------------------------------------------------------
    if (tid == 0) {
      tc::tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        const uint64_t ad = tc::smem_desc(aV + ks * 2 * RBS, RBS, 128);   // MN-major, 16 chunk rows per step
        const uint64_t bd = tc::smem_desc(aTb + ks * 256, 128, A_RBS);
        tc::mma_ss(tbase + TM_DU + 64 * s, ad, bd, id_n64_amn, ks > 0);
      }
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint64_t bd = tc::smem_desc(aW + ks * 256, 128, RBS);
        tc::mma_ts(tbase + TM_DU + 64 * s, tbase + TM_SB + ks * 8, bd, id_n64_neg, 1);
      }
      tc::mma_commit(tc::smem_u32(&ctl.bar1));
    }
    if (n > 0) output_epilogue(n - 1);   // overlaps the products; frees Dq
    tc::tc_fence_before();
    __syncthreads();
    if (tid == 0) {  // Dq = S^T Qg^T
      tc::tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint64_t bd = tc::smem_desc(aQg + ks * 256, 128, RBS);
        tc::mma_ts(tbase + TM_DQ, tbase + TM_SB + ks * 8, bd, id_n64, ks > 0);
      }
    }
    wait_bar(&ctl.bar1, ph1); ph1 ^= 1;
    tc::tc_fence_after();
    // ---- Vn^T -> bf16 -----------------------------------------------------------------------------------------------
    {
      const int c0 = 32 * hs;
      uint32_t r[32], pa[16];
      tc::tmem_ld32(tbase + TM_DU + 64 * s + lane_addr + c0, r);
      tc::tc_wait_ld();
#pragma unroll
      for (int j = 0; j < 16; ++j) pa[j] = tc::pack_bf16(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
      tc::tmem_st16(tbase + TM_VA + lane_addr + c0 / 2, pa);
    }
    tc::tc_wait_st();
    tc::tc_fence_before();
    __syncthreads();
    // ---- S^T += Vn^T Kd ;  Do = Vn^T A_qk^T ---------------------------------------------------------------------------
    if (tid == 0) {
      tc::tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        const uint64_t bd = tc::smem_desc(aKd + ks * 2 * RBS, RBS, 128);  // Kd MN-major
        tc::mma_ts(tbase + TM_S, tbase + TM_VA + ks * 8, bd, id_n128_bmn, 1);
      }
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        const uint64_t bd = tc::smem_desc(aAqk + ks * 256, 128, A_RBS);
        tc::mma_ts(tbase + TM_DU + 64 * s, tbase + TM_VA + ks * 8, bd, id_n64, ks > 0);
      }
      tc::mma_commit(tc::smem_u32(&ctl.bar2));
    }
    wait_bar(&ctl.bar2, ph2); ph2 ^= 1;
    tc::tc_fence_after();
    // every product that reads this buffer is complete: fetch the record of chunk n + 2 into it
    if (tid == 0 && n + 2 < nchunks) {
      tc::fence_async_smem();
      issue_load(n + 2);
    }
  }
  if (nchunks > 0) output_epilogue(nchunks - 1);
  if (p.hT) {
    float* hT = p.hT + (int64_t)unit * kD * kD;
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
      const int c0 = 64 * hs + 32 * cc;
      uint32_t r[32];
      tc::tmem_ld32(tbase + TM_S + lane_addr + c0, r);
      tc::tc_wait_ld();
#pragma unroll
      for (int j = 0; j < 32; ++j) hT[(c0 + j) * kD + l128] = __uint_as_float(r[j]);
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tbase, TM_COLS);
}

inline cudaError_t launch_chunk(const FwdParams& p, void* workspace, cudaStream_t stream, int* launches) {
  cudaError_t e = cudaFuncSetAttribute(intra_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, IN_TOTAL);
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ST_TOTAL);
  if (e != cudaSuccess) return e;
  const int64_t units = (int64_t)p.map.B * p.map.H;
  const int nchunks = (p.map.T + kC - 1) / kC;
  uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
  intra_kernel<<<(unsigned)(units * nchunks), kThreads, IN_TOTAL, stream>>>(p, ws);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  state_kernel<<<(unsigned)units, kThreads, ST_TOTAL, stream>>>(p, ws);
  *launches = 2;
  return cudaGetLastError();
}

}  // namespace kda
}  // namespace dr

