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
// Shared memory is kept under half an SM's worth so that two CTAs are resident and one chunk's latency
// (global loads, the serial prefix sum, the barriers between phases) hides behind the other's work.  The
// inputs stay as raw bf16 with their l2-norm factors on the side, and the decayed bf16 operands of the
// tensor-core products are formed in registers from them (no scaled copies in shared memory).
constexpr int LDF = 132;   // row stride (floats) of G
constexpr int LDH = 136;   // row stride (bf16) of the raw q, k rows and of the W staging tile
constexpr int LDQ = 72;    // row stride (bf16) of A_qk
constexpr int IN_G = 0;                          // log2(e) G   fp32 [64][132]
constexpr int IN_K = IN_G + 64 * LDF * 4;        // raw k       bf16 [64][136]
constexpr int IN_Q = IN_K + 64 * LDH * 2;        // raw q       bf16 [64][136]
constexpr int IN_AKK = IN_Q + 64 * LDH * 2;      // A_kk fp32 [64][68]; later the W staging tile bf16 [64][136]
constexpr int IN_T = IN_AKK + 64 * LDT * 4;      // T    fp32 [64][68]
constexpr int IN_AQK = IN_T + 64 * LDT * 4;      // A_qk bf16 [64][72]
constexpr int IN_BETA = IN_AQK + 64 * LDQ * 2;   // beta[64], rk[64], rq[64]
constexpr int IN_TOTAL = IN_BETA + 3 * 64 * 4;
static_assert(64 * LDT * 4 == 64 * LDH * 2, "the W staging tile reuses the A_kk array");
static_assert(2 * (IN_TOTAL + 1024) <= 233472, "two CTAs per SM");

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float2 bf2(uint32_t u) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u));
}

// two bf16 products in one instruction (operands and result packed in 32 bits)
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// four consecutive elements starting at element index i (a multiple of 4)
__device__ __forceinline__ void ld4(const void* p, int64_t i, int dt, float (&x)[4]) {
  if (dt == DR_BF16) {
    const uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p) + i);
    const float2 a = bf2(u.x), b = bf2(u.y);
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


__global__ void __launch_bounds__(kThreads, 2) intra_kernel(const FwdParams p, uint8_t* __restrict__ ws, const int copy_v) {
  extern __shared__ __align__(1024) uint8_t smem[];
  float* sG = reinterpret_cast<float*>(smem + IN_G);
  __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(smem + IN_K);
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem + IN_Q);
  float* sAkk = reinterpret_cast<float*>(smem + IN_AKK);
  __nv_bfloat16* sWst = reinterpret_cast<__nv_bfloat16*>(smem + IN_AKK);
  float* sT = reinterpret_cast<float*>(smem + IN_T);
  __nv_bfloat16* sAqk = reinterpret_cast<__nv_bfloat16*>(smem + IN_AQK);
  float* sBeta = reinterpret_cast<float*>(smem + IN_BETA);
  float* sRk = sBeta + 64;
  float* sRq = sBeta + 128;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int T = p.map.T;
  const int nchunks = (T + kC - 1) / kC;
  const int unit = blockIdx.x / nchunks, n = blockIdx.x % nchunks;
  const int b = unit / p.map.H, h = unit % p.map.H;
  const int t0 = n * kC, rows = min(kC, T - t0);
  const int64_t qk_base = p.map.base_qk(b, h, kD), qk_tok = p.map.tok_qk(kD);   // q, k (possibly fewer heads)
  const int64_t gk_base = p.map.base(b, h, kD), gk_tok = p.map.tok(kD);         // per-channel decay: per value head
  const int64_t s_base = p.map.base(b, h, 1), s_tok = p.map.tok(1);
  uint8_t* rec = ws + ((int64_t)unit * nchunks + n) * WS_REC;
  constexpr float kLog2e = 1.4426950408889634f;

  // ---- load: raw k, q rows, their norm factors, the log decay (in log2 units); lane = four channels ---------
  // (all global loads of the warp's eight rows are issued before the first is used)
  {
    uint2 qraw[8], kraw[8];
    float gv[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int c = warp + 8 * i;
      qraw[i] = make_uint2(0u, 0u); kraw[i] = make_uint2(0u, 0u);
      gv[i][0] = gv[i][1] = gv[i][2] = gv[i][3] = 0.f;
      if (c < rows) {
        const int64_t at = qk_base + (t0 + c) * qk_tok + 4 * lane;
        qraw[i] = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p.q) + at);
        kraw[i] = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p.k) + at);
        if (p.variant == DR_KDA) {
          ld4(p.g, gk_base + (t0 + c) * gk_tok + 4 * lane, p.g_dt, gv[i]);
        } else if (p.variant == DR_GATED) {
          const float gs = ld_elem(p.g, s_base + (t0 + c) * s_tok, p.g_dt);
          gv[i][0] = gv[i][1] = gv[i][2] = gv[i][3] = gs;
        }
      }
    }
    float bt = 0.f;
    if (lane < 8 && warp + 8 * lane < rows) bt = p.beta[s_base + (t0 + warp + 8 * lane) * s_tok];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int c = warp + 8 * i;
      *reinterpret_cast<uint2*>(sQ + c * LDH + 4 * lane) = qraw[i];
      *reinterpret_cast<uint2*>(sK + c * LDH + 4 * lane) = kraw[i];
      *reinterpret_cast<float4*>(sG + c * LDF + 4 * lane) =
          make_float4(gv[i][0] * kLog2e, gv[i][1] * kLog2e, gv[i][2] * kLog2e, gv[i][3] * kLog2e);
      float qmul = p.scale, kmul = 1.f;
      if (p.l2norm) {
        const float2 q0 = bf2(qraw[i].x), q1 = bf2(qraw[i].y), k0 = bf2(kraw[i].x), k1 = bf2(kraw[i].y);
        const float nq = warp_sum(q0.x * q0.x + q0.y * q0.y + q1.x * q1.x + q1.y * q1.y);
        const float nk = warp_sum(k0.x * k0.x + k0.y * k0.y + k1.x * k1.x + k1.y * k1.y);
        qmul = p.scale / (sqrtf(nq) + 1e-6f);
        kmul = 1.f / (sqrtf(nk) + 1e-6f);
      }
      if (lane == i) {
        sBeta[c] = bt;
        sRk[c] = kmul;
        sRq[c] = qmul;
      }
    }
  }
  // V rows -> the record's tile, 16 bytes per piece (coalesced writes); skipped when the state kernel can fetch
  // the rows itself through a tensor map
  if (copy_v) {
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
  // thread = (8-row segment, four channels): local scan, then the totals of the earlier segments are added;
  // the segment totals live in the first rows of the (still unused) T array
  {
    const int seg = tid >> 5, c4 = 4 * (tid & 31);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 loc[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const float4 x = *reinterpret_cast<const float4*>(sG + (8 * seg + r) * LDF + c4);
      acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
      loc[r] = acc;
    }
    *reinterpret_cast<float4*>(sT + seg * 128 + c4) = acc;
    __syncthreads();
    float4 pre = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s2 = 0; s2 < seg; ++s2) {
      const float4 x = *reinterpret_cast<const float4*>(sT + s2 * 128 + c4);
      pre.x += x.x; pre.y += x.y; pre.z += x.z; pre.w += x.w;
    }
#pragma unroll
    for (int r = 0; r < 8; ++r)
      *reinterpret_cast<float4*>(sG + (8 * seg + r) * LDF + c4) =
          make_float4(loc[r].x + pre.x, loc[r].y + pre.y, loc[r].z + pre.z, loc[r].w + pre.w);
    __syncthreads();
  }
  // ---- chunk-local products on mma.sync (bf16) -------------------------------------------------------------------
  // Rows of sub-block bi against the columns of blocks 0..bi; operands  x_i e^{G_i - G_n}  and  k_j e^{G_n - G_j}
  // (n = first row of bi) are formed in registers; the k and q rows share their decay factors and the column
  // operand.  For columns of EARLIER blocks both exponents are <= 0.  For the columns of bi itself the second
  // exponent is positive, at most the decay accumulated over the block; when that exceeds 2^64 in some channel
  // (never with trained gates, but legal input) the block is redone exactly below.
  // Eight warp tasks: (bi; 8-column tiles)  3;0-2  3;3-5  3;6-7  2;0-2  2;3-5  1;0-1  1;2-3  0;0-1
  auto block_unsafe = [&](int blk) -> bool {   // warp-uniform
    const float4 ga = *reinterpret_cast<const float4*>(sG + (16 * blk) * LDF + 4 * lane);
    const float4 gb = *reinterpret_cast<const float4*>(sG + (16 * blk + 15) * LDF + 4 * lane);
    float m = fmaxf(fmaxf(ga.x - gb.x, ga.y - gb.y), fmaxf(ga.z - gb.z, ga.w - gb.w));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    return !(m <= 64.f);
  };
  {
    const int bi = warp < 3 ? 3 : warp < 5 ? 2 : warp < 7 ? 1 : 0;
    const int nt0 = warp < 3 ? 3 * warp : warp < 5 ? 3 * (warp - 3) : warp < 7 ? 2 * (warp - 5) : 0;
    const int ntn = (warp == 2 || warp >= 5) ? 2 : 3;
    const bool skip_diag = block_unsafe(bi);
    const int r0 = 16 * bi + g, r1 = r0 + 8, nrow = 16 * bi;
    float dk[3][4], dq[3][4];
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      dk[i][0] = dk[i][1] = dk[i][2] = dk[i][3] = 0.f;
      dq[i][0] = dq[i][1] = dq[i][2] = dq[i][3] = 0.f;
    }
#pragma unroll 2
    for (int ks = 0; ks < 8; ++ks) {
      const int k0 = ks * 16 + 2 * t;
      const float2 gn0 = *reinterpret_cast<const float2*>(sG + nrow * LDF + k0);
      const float2 gn1 = *reinterpret_cast<const float2*>(sG + nrow * LDF + k0 + 8);
      uint32_t ak[4], aq[4];
      {
        const float2 ga = *reinterpret_cast<const float2*>(sG + r0 * LDF + k0);
        const float2 gb = *reinterpret_cast<const float2*>(sG + r1 * LDF + k0);
        const float2 gc = *reinterpret_cast<const float2*>(sG + r0 * LDF + k0 + 8);
        const float2 gd = *reinterpret_cast<const float2*>(sG + r1 * LDF + k0 + 8);
        // decay factors as bf16 pairs, shared by the k and the q row; the products are packed bf16 multiplies (the
        // operands of the tensor-core product are bf16 either way: one rounding of the factor, one of the product)
        const uint32_t ea = tc::pack_bf16(ex2(ga.x - gn0.x), ex2(ga.y - gn0.y)), eb = tc::pack_bf16(ex2(gb.x - gn0.x), ex2(gb.y - gn0.y));
        const uint32_t ec = tc::pack_bf16(ex2(gc.x - gn1.x), ex2(gc.y - gn1.y)), ed = tc::pack_bf16(ex2(gd.x - gn1.x), ex2(gd.y - gn1.y));
        ak[0] = mul_bf16x2(*reinterpret_cast<const uint32_t*>(sK + r0 * LDH + k0), ea);
        ak[1] = mul_bf16x2(*reinterpret_cast<const uint32_t*>(sK + r1 * LDH + k0), eb);
        ak[2] = mul_bf16x2(*reinterpret_cast<const uint32_t*>(sK + r0 * LDH + k0 + 8), ec);
        ak[3] = mul_bf16x2(*reinterpret_cast<const uint32_t*>(sK + r1 * LDH + k0 + 8), ed);
        aq[0] = mul_bf16x2(*reinterpret_cast<const uint32_t*>(sQ + r0 * LDH + k0), ea);
        aq[1] = mul_bf16x2(*reinterpret_cast<const uint32_t*>(sQ + r1 * LDH + k0), eb);
        aq[2] = mul_bf16x2(*reinterpret_cast<const uint32_t*>(sQ + r0 * LDH + k0 + 8), ec);
        aq[3] = mul_bf16x2(*reinterpret_cast<const uint32_t*>(sQ + r1 * LDH + k0 + 8), ed);
      }
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        if (i < ntn && !(skip_diag && nt0 + i >= 2 * bi)) {
          const int j = 8 * (nt0 + i) + g;
          const float2 gj0 = *reinterpret_cast<const float2*>(sG + j * LDF + k0);
          const float2 gj1 = *reinterpret_cast<const float2*>(sG + j * LDF + k0 + 8);
          uint32_t bb[2];
          bb[0] = mul_bf16x2(*reinterpret_cast<const uint32_t*>(sK + j * LDH + k0),
                             tc::pack_bf16(ex2(gn0.x - gj0.x), ex2(gn0.y - gj0.y)));
          bb[1] = mul_bf16x2(*reinterpret_cast<const uint32_t*>(sK + j * LDH + k0 + 8),
                             tc::pack_bf16(ex2(gn1.x - gj1.x), ex2(gn1.y - gj1.y)));
          mma_bf16(dk[i], ak, bb);
          mma_bf16(dq[i], aq, bb);
        }
      }
    }
    const float fk0 = sRk[r0], fk1 = sRk[r1], fq0 = sRq[r0], fq1 = sRq[r1];
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      if (i < ntn) {
        const int c = 8 * (nt0 + i) + 2 * t;
        const float c0 = sRk[c], c1 = sRk[c + 1];
        *reinterpret_cast<uint32_t*>(sAqk + r0 * LDQ + c) = tc::pack_bf16(dq[i][0] * fq0 * c0, dq[i][1] * fq0 * c1);
        *reinterpret_cast<uint32_t*>(sAqk + r1 * LDQ + c) = tc::pack_bf16(dq[i][2] * fq1 * c0, dq[i][3] * fq1 * c1);
        *reinterpret_cast<float2*>(sAkk + r0 * LDT + c) = make_float2(dk[i][0] * fk0 * c0, dk[i][1] * fk0 * c1);
        *reinterpret_cast<float2*>(sAkk + r1 * LDT + c) = make_float2(dk[i][2] * fk1 * c0, dk[i][3] * fk1 * c1);
      }
    }
  }
  // ---- diagonal 16x16 blocks exactly (fp32), only for blocks whose decay range is too wide for the product form ----
  // Two warps per block, 64 channels each, two channels per lane; the 16 rows of k and the per-row decay
  // d_r = e^{G_r - G_{r-1}} stay in registers, so e^{G_i - G_j} is a running product (no exponentials per pair).
  // Partial sums of the two channel halves meet in a scratch array (the T array, not yet in use).
  __syncthreads();   // the tensor-core tasks have written their (possibly non-finite) entries of these blocks
  if (block_unsafe(warp >> 1)) {
    const int blk = warp >> 1, half = warp & 1, ch0 = 64 * half + 2 * lane;
    float2 kr[16], dd[16];
    {
      float2 gprev = make_float2(0.f, 0.f);
#pragma unroll
      for (int r = 0; r < 16; ++r) {
        const int row = 16 * blk + r;
        kr[r] = bf2(*reinterpret_cast<const uint32_t*>(sK + row * LDH + ch0));
        const float2 gg = *reinterpret_cast<const float2*>(sG + row * LDF + ch0);
        dd[r] = make_float2(ex2(gg.x - gprev.x), ex2(gg.y - gprev.y));   // dd[0] is never used
        gprev = gg;
      }
    }
    float* part = sT + (half * 4 + blk) * 512;   // [i][j][kk,qk]
    const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4;
    const int idx = (b4 ? 4 : 0) + (b3 ? 2 : 0) + (b2 ? 1 : 0);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float2 qi = bf2(*reinterpret_cast<const uint32_t*>(sQ + (16 * blk + i) * LDH + ch0));
      const float2 ki = kr[i];
      float2 P = make_float2(1.f, 1.f);
#pragma unroll
      for (int jg = (i & ~3); jg >= 0; jg -= 4) {
        float v[8];
#pragma unroll
        for (int u = 3; u >= 0; --u) {
          const int j = jg + u;
          if (j <= i) {
            const float w0 = kr[j].x * P.x, w1 = kr[j].y * P.y;
            v[u] = ki.x * w0 + ki.y * w1;
            v[u + 4] = qi.x * w0 + qi.y * w1;
            if (j > 0) { P.x *= dd[j].x; P.y *= dd[j].y; }
          } else {
            v[u] = 0.f; v[u + 4] = 0.f;
          }
        }
        // eight sums over the 32 lanes in nine shuffles: each level halves the number of live values
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
          const int j = jg + (idx & 3);
          if (j <= i) part[(i * 16 + j) * 2 + (idx >> 2)] = z;
        }
      }
    }
    asm volatile("bar.sync %0, 64;" ::"r"(2 + blk) : "memory");   // the two warps of this block
    const float* p0 = sT + blk * 512;
    const float* p1 = sT + (4 + blk) * 512;
    for (int e = lane; e < 256; e += 32) {
      const int i = e >> 4, j = e & 15, gi = 16 * blk + i, gj = 16 * blk + j;
      if (half == 0) {
        if (j < i) sAkk[gi * LDT + gj] = (p0[2 * e] + p1[2 * e]) * sRk[gi] * sRk[gj];
      } else if (j <= i) {
        sAqk[gi * LDQ + gj] = __float2bfloat16_rn((p0[2 * e + 1] + p1[2 * e + 1]) * sRq[gi] * sRk[gj]);
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
    float a[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int j = col + e;
      a[e] = j <= row ? sT[row * LDT + j] * sBeta[j] : 0.f;
    }
    *reinterpret_cast<uint4*>(rec + WS_TB + piece * 16) = pack8(a);
    uint4 q = *reinterpret_cast<const uint4*>(sAqk + row * LDQ + col);
    uint32_t* qw = reinterpret_cast<uint32_t*>(&q);
#pragma unroll
    for (int e = 0; e < 4; ++e) {   // keep j <= row
      const int j = col + 2 * e;
      if (j > row) qw[e] = 0u;
      else if (j + 1 > row) qw[e] &= 0x0000ffffu;
    }
    *reinterpret_cast<uint4*>(rec + WS_AQK + piece * 16) = q;
  }
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int piece = tid + kThreads * it;
    int row, col;
    piece128(piece, row, col);
    const uint4 uq = *reinterpret_cast<const uint4*>(sQ + row * LDH + col);
    const uint4 uk = *reinterpret_cast<const uint4*>(sK + row * LDH + col);
    const uint32_t* wq = reinterpret_cast<const uint32_t*>(&uq);
    const uint32_t* wk = reinterpret_cast<const uint32_t*>(&uk);
    const float rq = sRq[row], rk = sRk[row];
    float a[8], c[8], kg[8];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 gg = *reinterpret_cast<const float2*>(sG + row * LDF + col + 2 * e);
      const float2 gl = *reinterpret_cast<const float2*>(sG + 63 * LDF + col + 2 * e);
      const float2 qq = bf2(wq[e]), kk = bf2(wk[e]);
      const float e0 = ex2(gg.x), e1 = ex2(gg.y);
      a[2 * e] = qq.x * rq * e0;
      a[2 * e + 1] = qq.y * rq * e1;
      c[2 * e] = kk.x * rk * ex2(gl.x - gg.x);
      c[2 * e + 1] = kk.y * rk * ex2(gl.y - gg.y);
      kg[2 * e] = kk.x * rk * e0;
      kg[2 * e + 1] = kk.y * rk * e1;
    }
    *reinterpret_cast<uint4*>(rec + WS_QG + piece * 16) = pack8(a);
    *reinterpret_cast<uint4*>(rec + WS_KD + piece * 16) = pack8(c);
    *reinterpret_cast<uint4*>(sQ + row * LDH + col) = pack8(kg);   // k^ e^G for the W product (q is dead)
  }
  if (tid < kD) reinterpret_cast<float*>(rec + WS_EGL)[tid] = ex2(sG[63 * LDF + tid]);
  __syncthreads();
  // ---- W = (T diag(beta)) (k^ e^G): 64x128x64 on mma.sync (tf32); warp = 16 rows x 64 channels ----------------------
  // (A_kk is dead after the inverse: its array takes the bf16 staging tile of W; bf16 -> tf32 is exact)
  {
    const int m0 = (warp >> 1) * 16, nb = (warp & 1) * 64;
    float d[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) { d[nt][0] = d[nt][1] = d[nt][2] = d[nt][3] = 0.f; }
    const int r0 = m0 + g, r1 = r0 + 8;
    for (int ks = 0; ks * 8 <= m0 + 15; ++ks) {
      const int k0 = ks * 8 + t, k1 = k0 + 4;
      const float s0 = sBeta[k0], s1 = sBeta[k1];
      uint32_t a[4];
      a[0] = sm100::to_tf32(k0 <= r0 ? sT[r0 * LDT + k0] * s0 : 0.f);
      a[1] = sm100::to_tf32(k0 <= r1 ? sT[r1 * LDT + k0] * s0 : 0.f);
      a[2] = sm100::to_tf32(k1 <= r0 ? sT[r0 * LDT + k1] * s1 : 0.f);
      a[3] = sm100::to_tf32(k1 <= r1 ? sT[r1 * LDT + k1] * s1 : 0.f);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const int ch = nb + nt * 8 + g;
        uint32_t bb[2];
        bb[0] = (uint32_t)reinterpret_cast<const uint16_t*>(sQ)[k0 * LDH + ch] << 16;
        bb[1] = (uint32_t)reinterpret_cast<const uint16_t*>(sQ)[k1 * LDH + ch] << 16;
        sm100::mma_tf32(d[nt], a, bb);
      }
    }
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      *reinterpret_cast<uint32_t*>(sWst + r0 * LDH + nb + nt * 8 + 2 * t) = tc::pack_bf16(d[nt][0], d[nt][1]);
      *reinterpret_cast<uint32_t*>(sWst + r1 * LDH + nb + nt * 8 + 2 * t) = tc::pack_bf16(d[nt][2], d[nt][3]);
    }
  }
  __syncthreads();
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int piece = tid + kThreads * it;
    int row, col;
    piece128(piece, row, col);
    *reinterpret_cast<uint4*>(rec + WS_W + piece * 16) = *reinterpret_cast<const uint4*>(sWst + row * LDH + col);
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
  uint64_t full[2], go1, go2, go3, bar1, bar2;
  uint32_t tmem_base;
  int abort;
};

// Nine warps.  Warps 0-7 (256 threads; two warps per 32-lane quarter of tensor memory, each taking half of the
// columns) do everything that touches data; warp 8 only issues: the bulk copies of the records and every
// tcgen05.mma.  Issuing one product costs its thread ~100 cycles, 28 products per chunk: on a worker warp that
// time would sit on the serial chain of the chunk, on the issuing warp it overlaps the workers' epilogues.
// Hand-offs are mbarriers: go1 (bf16 state copy written), go2 (the previous chunk's Dq has been read),
// go3 (bf16 V_new written) from the workers; bar1, bar2 (products complete) from tcgen05.commit.
constexpr int kStateThreads = kThreads + 32;

// Kernel parameters of the state pass: the forward parameters plus the output tensor map ({128, T, H, B} view of
// o in its own dtype; one box {128, 64, 1, 1} stores a chunk's rows and clips the ragged tail).
struct StateParams {
  CUtensorMap to;
  CUtensorMap tv;   // 5-d view of v whose box is one 64x128 tile in core-matrix order (see sm100::make_input_map)
  FwdParams p;
  const uint8_t* ws;
  int use_tma_out, use_tma_v;
};

__global__ void __launch_bounds__(kStateThreads, 1) state_kernel(const __grid_constant__ StateParams P) {
  const FwdParams& p = P.p;
  const uint8_t* __restrict__ ws = P.ws;
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ __align__(8) StateCtl ctl;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int hs = (tid >> 7) & 1, l128 = tid & 127;
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
    tc::mbar_init(tc::smem_u32(&ctl.go1), kThreads);
    tc::mbar_init(tc::smem_u32(&ctl.go2), kThreads);
    tc::mbar_init(tc::smem_u32(&ctl.go3), kThreads);
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
  auto wait_bar = [&](uint64_t* bar, uint32_t parity) {
    if (tc::mbar_try(tc::smem_u32(bar), parity)) return;
    sm100::wait_more(tc::smem_u32(bar), parity, p.status, &ctl.abort, (uint32_t)((const char*)bar - (const char*)&ctl),
                     (uint32_t)(warp == 8 ? 1 : 0));
  };
  auto arrive = [&](uint64_t* bar) { sm100::mbar_arrive(tc::smem_u32(bar)); };
  auto workers_sync = [&]() { asm volatile("bar.sync 1, 256;" ::: "memory"); };

  if (warp == 8) {
    // =========================== ISSUING WARP (one thread) ======================================================
    if (tid == kThreads) {
      // the whole record of chunk m -> buffer m & 1 (the record is contiguous; four copies in flight)
      auto issue_load = [&](int m) {
        const uint32_t bar = tc::smem_u32(&ctl.full[m & 1]);
        tc::mbar_arrive_expect_tx(bar, WS_REC);
        const uint32_t dst = tc::smem_u32(smem + (m & 1) * WS_REC);
        const uint8_t* src = recs + (int64_t)m * WS_REC;
        if (P.use_tma_v) {
          // the V rows straight from the input tensor; the record carries the other tiles
          tc::tma_load_5d(dst + WS_V, &P.tv, 0, 0, 0, m * 8, unit, bar);
#pragma unroll
          for (int i = 0; i < 3; ++i) tc::bulk_g2s(dst + i * 16384, src + i * 16384, 16384, bar);   // W, Qg, Kd
          tc::bulk_g2s(dst + WS_TB, src + WS_TB, WS_REC - WS_TB, bar);                                   // Tb, A_qk, e^{G_L}
        } else {
          constexpr int Q4 = WS_REC / 4;   // 20608, a multiple of 16
#pragma unroll
          for (int i = 0; i < 4; ++i) tc::bulk_g2s(dst + i * Q4, src + i * Q4, Q4, bar);
        }
      };
      if (nchunks > 0) issue_load(0);
      if (nchunks > 1) issue_load(1);
      const uint32_t id_n64 = tc::idesc_bf16(128, 64, 0, 0);
      const uint32_t id_n64_amn = tc::idesc_bf16(128, 64, 1, 0);
      const uint32_t id_n64_neg = id_n64 | (1u << 13);
      const uint32_t id_n128_bmn = tc::idesc_bf16(128, 128, 0, 1);
      for (int n = 0; n < nchunks; ++n) {
        const int s = n & 1;
        const uint8_t* st = smem + s * WS_REC;
        const uint32_t aW = tc::smem_u32(st + WS_W), aQg = tc::smem_u32(st + WS_QG), aKd = tc::smem_u32(st + WS_KD);
        const uint32_t aV = tc::smem_u32(st + WS_V), aTb = tc::smem_u32(st + WS_TB), aAqk = tc::smem_u32(st + WS_AQK);
        wait_bar(&ctl.full[s], (n >> 1) & 1);
        // U^T = V^T Tb^T needs no state: issue it before the workers' state pass has finished
        tc::tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          const uint64_t ad = tc::smem_desc(aV + ks * 2 * RBS, RBS, 128);   // MN-major, 16 chunk rows per step
          const uint64_t bd = tc::smem_desc(aTb + ks * 256, 128, A_RBS);
          tc::mma_ss(tbase + TM_DU + 64 * s, ad, bd, id_n64_amn, ks > 0);
        }
        wait_bar(&ctl.go1, n & 1);
        tc::tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {   // Vn^T = U^T - S^T W^T
          const uint64_t bd = tc::smem_desc(aW + ks * 256, 128, RBS);
          tc::mma_ts(tbase + TM_DU + 64 * s, tbase + TM_SB + ks * 8, bd, id_n64_neg, 1);
        }
        tc::mma_commit(tc::smem_u32(&ctl.bar1));
        if (n > 0) wait_bar(&ctl.go2, (n - 1) & 1);   // the previous chunk's Dq has been read
        tc::tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {   // Dq = S^T Qg^T
          const uint64_t bd = tc::smem_desc(aQg + ks * 256, 128, RBS);
          tc::mma_ts(tbase + TM_DQ, tbase + TM_SB + ks * 8, bd, id_n64, ks > 0);
        }
        wait_bar(&ctl.go3, n & 1);
        tc::tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {   // S^T += Vn^T Kd   (Kd MN-major)
          const uint64_t bd = tc::smem_desc(aKd + ks * 2 * RBS, RBS, 128);
          tc::mma_ts(tbase + TM_S, tbase + TM_VA + ks * 8, bd, id_n128_bmn, 1);
        }
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {   // Do = Vn^T A_qk^T
          const uint64_t bd = tc::smem_desc(aAqk + ks * 256, 128, A_RBS);
          tc::mma_ts(tbase + TM_DU + 64 * s, tbase + TM_VA + ks * 8, bd, id_n64, ks > 0);
        }
        tc::mma_commit(tc::smem_u32(&ctl.bar2));
        // every product that reads this buffer has completed once bar2 flips: fetch the record of chunk n + 2
        if (n + 2 < nchunks) {
          wait_bar(&ctl.bar2, n & 1);
          tc::fence_async_smem();
          issue_load(n + 2);
        }
      }
    }
  } else {
    // =========================== WORKERS ===========================================================================
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
    __nv_bfloat16* sOh = reinterpret_cast<__nv_bfloat16*>(smem + ST_O);
    // O^T of chunk m = Dq + Do -> staging tile [64][128] in the output dtype -> one tiled TMA store (or, without a
    // tensor map, row copies by the threads)
    auto output_epilogue = [&](int m) {
      const int t0m = m * kC, rowsm = min(kC, T - t0m);
      if (P.use_tma_out && tid == 0) tc::bulk_wait_read_all();   // the previous store has read the staging tile
      workers_sync();
      {
        const int c0 = 32 * hs;
        uint32_t rq[32], ro[32];
        tc::tmem_ld32(tbase + TM_DQ + lane_addr + c0, rq);
        tc::tmem_ld32(tbase + TM_DU + 64 * (m & 1) + lane_addr + c0, ro);
        tc::tc_wait_ld();
        tc::tc_fence_before();
        arrive(&ctl.go2);   // Dq (and this accumulator) may be overwritten
        if (p.out_dt == DR_BF16) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            sOh[(c0 + j) * kD + l128] = __float2bfloat16_rn(__uint_as_float(rq[j]) + __uint_as_float(ro[j]));
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) sO[(c0 + j) * kD + l128] = __uint_as_float(rq[j]) + __uint_as_float(ro[j]);
        }
      }
      if (!p.o) return;
      if (P.use_tma_out) {
        tc::fence_async_smem();
        workers_sync();
        if (tid == 0) {
          tc::tma_store_4d(&P.to, tc::smem_u32(sO), 0, t0m, h, b);
          tc::bulk_commit();
        }
        return;
      }
      workers_sync();
      const int r = tid >> 2, qtr = tid & 3;
      if (r < rowsm) {
        const int64_t at = o_base + (int64_t)(t0m + r) * o_tok + 32 * qtr;
        if (p.out_dt == DR_BF16) {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.o) + at;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            reinterpret_cast<uint4*>(dst)[j] = reinterpret_cast<const uint4*>(sOh + r * kD + 32 * qtr)[j];
        } else {
          float* dst = reinterpret_cast<float*>(p.o) + at;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            reinterpret_cast<float4*>(dst)[j] = reinterpret_cast<const float4*>(sO + r * kD + 32 * qtr)[j];
        }
      }
    };

    for (int n = 0; n < nchunks; ++n) {
      const int s = n & 1;
      const float* sEGL = reinterpret_cast<const float*>(smem + s * WS_REC + WS_EGL);
      wait_bar(&ctl.full[s], (n >> 1) & 1);
      if (n > 0) {
        wait_bar(&ctl.bar2, (n - 1) & 1);   // the previous chunk's state update and Do have completed
        tc::tc_fence_after();
      }
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
      arrive(&ctl.go1);
      if (n > 0) output_epilogue(n - 1);   // overlaps the products of this chunk
      wait_bar(&ctl.bar1, n & 1);
      tc::tc_fence_after();
      // ---- Vn^T -> bf16 -------------------------------------------------------------------------------------------
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
      arrive(&ctl.go3);
    }
    if (nchunks > 0) {
      wait_bar(&ctl.bar2, (nchunks - 1) & 1);
      tc::tc_fence_after();
      output_epilogue(nchunks - 1);
      if (P.use_tma_out && tid == 0) tc::bulk_wait_all();
    }
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
  StateParams SP;
  memset(&SP, 0, sizeof(SP));
  SP.p = p;
  SP.ws = ws;
  // V rows by TMA need the rows of one sequence contiguous and whole 8-row blocks
  SP.use_tma_v = !p.map.bthd && p.map.T % 8 == 0 && sm100::make_input_map(&SP.tv, p.v, units, p.map.T);
  intra_kernel<<<(unsigned)(units * nchunks), kThreads, IN_TOTAL, stream>>>(p, ws, SP.use_tma_v ? 0 : 1);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  SP.use_tma_out = p.o != nullptr && sm100::make_output_map(&SP.to, p.o, p.map, p.out_dt == DR_BF16 ? 2 : 4);
  state_kernel<<<(unsigned)units, kStateThreads, ST_TOTAL, stream>>>(SP);
  *launches = 2;
  return cudaGetLastError();
}

}  // namespace kda
}  // namespace dr

