// Chunkwise gated delta-rule forward on the Blackwell tensor cores (tcgen05 + TMEM).
//
// Shape: K = V = 128, chunk C = 64, bf16 q/k/v/o, fp32 g/beta/state.  One CTA of 128 threads
// owns one (batch, head) sequence; the fp32 state lives TRANSPOSED in tensor memory
// (S^T: lane = value column v, column = key row k) for the whole sequence, so every product of
// the chunk recurrence has M = 128 = V and the per-thread epilogues own one value column.
//
// Per chunk (G = cumulative log decay inside the chunk, L = its last row):
//   (1) D1 = [K^;Q^] K^^T                       128x64x128   smem x smem
//       A_kk = beta_i D1[i][j] e^{G_i-G_j} (i>j)  ->  T = (I + A_kk)^-1 on the CUDA cores (fp32)
//       A_qk = D1[64+i][j] e^{G_i-G_j} (i>=j)     ->  bf16 operand
//   (2) D2 = S^T [K^;Q^]^T                       128x128x128  tmem(bf16 copy of S^T) x smem
//       R^T[v][c] = beta_c (V[c][v] - D2[v][c] e^{G_c})                        -> bf16 -> tmem
//   (3) D3 = R^T T^T = V_new^T                   128x64x64    tmem x smem
//   (4) D4 = V_new^T A_qk^T                      128x64x64    tmem x smem
//       O^T[v][i] = e^{G_i} D2[v][64+i] + D4[v][i]
//   (5) S^T = e^{G_L} S^T + (V_new^T e^{G_L-G_c}) K^   128x128x64   tmem x smem (K^ read MN-major)
// The shared-memory tile [K^;Q^] is stored once as 8x8 core matrices and serves as the A operand
// of (1), the K-major B operand of (1) and (2), and the MN-major B operand of (5).
#pragma once

#include "dr_common.cuh"
#include "dr_tcgen05.cuh"
#include "dr_umma_selftest.cuh"

namespace dr {
namespace sm100 {

constexpr bool kAvailable = true;
constexpr int kThreads = 128;
constexpr int kC = 64, kD = 128;

// tensor-memory columns (32-bit x 128 lanes each)
constexpr uint32_t TM_S = 0;      // S^T fp32                    128 cols
constexpr uint32_t TM_SB = 128;   // bf16 copy of S^T (A operand)  64 cols
constexpr uint32_t TM_D2 = 192;   // S^T [K^;Q^]^T               128 cols
constexpr uint32_t TM_D3 = 320;   // D1, then V_new^T, then D4     64 cols
constexpr uint32_t TM_RA = 384;   // R^T, then V_new^T (bf16)      32 cols
constexpr uint32_t TM_VB = 416;   // decayed V_new^T (bf16)        32 cols
constexpr uint32_t TM_COLS = 512;

// shared-memory map (bytes)
constexpr int SM_QK = 0;                       // [K^ (64 rows); Q^ (64 rows)] x 128, core-matrix tiled: 32 KB
constexpr int QK_RBS = 16 * 128;               // row-block stride of SM_QK
constexpr int SM_V = SM_QK + 128 * 128 * 2;    // V chunk [64][128] bf16 row-major, reused as the O staging tile: 16 KB
constexpr int SM_T = SM_V + 64 * 128 * 2;      // T [64][64] bf16 core-matrix tiled: 8 KB
constexpr int SM_AQK = SM_T + 64 * 64 * 2;     // A_qk [64][64] bf16 core-matrix tiled: 8 KB
constexpr int A_RBS = 8 * 128;                 // row-block stride of SM_T / SM_AQK
constexpr int SM_AKK = SM_AQK + 64 * 64 * 2;   // A_kk fp32 [64][65]
constexpr int AKK_LD = 65;
constexpr int SM_G = SM_AKK + 64 * AKK_LD * 4; // G[64], beta[64], e^G[64], e^{G_L-G}[64]
constexpr int SM_TOTAL = SM_G + 4 * 64 * 4;

__global__ void __launch_bounds__(kThreads, 1) chunk_sm100_kernel(const FwdParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int T = p.map.T;
  const int unit = blockIdx.x;
  const int b = unit / p.map.H, h = unit % p.map.H;
  const int64_t qk_base = p.map.base(b, h, kD), qk_tok = p.map.tok(kD);
  const int64_t s_base = p.map.base(b, h, 1), s_tok = p.map.tok(1);
  const __nv_bfloat16* gq = reinterpret_cast<const __nv_bfloat16*>(p.q);
  const __nv_bfloat16* gk = reinterpret_cast<const __nv_bfloat16*>(p.k);
  const __nv_bfloat16* gv = reinterpret_cast<const __nv_bfloat16*>(p.v);
  __nv_bfloat16* go = reinterpret_cast<__nv_bfloat16*>(p.o);
  const float* gg = reinterpret_cast<const float*>(p.g);

  uint8_t* sQK = smem + SM_QK;
  __nv_bfloat16* sV = reinterpret_cast<__nv_bfloat16*>(smem + SM_V);
  uint8_t* sT = smem + SM_T;
  uint8_t* sAqk = smem + SM_AQK;
  float* sAkk = reinterpret_cast<float*>(smem + SM_AKK);
  float* sG = reinterpret_cast<float*>(smem + SM_G);
  float* sBeta = sG + 64;
  float* sEG = sG + 128;
  float* sW = sG + 192;

  if (warp == 0) {
    tc::tmem_alloc(tc::smem_u32(&tmem_base_s), TM_COLS);
    tc::tmem_relinquish();
  }
  if (tid == 0) {
    tc::mbar_init(tc::smem_u32(&bar), 1);
    tc::fence_mbar_init();
    abort_s = 0;
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tbase = tmem_base_s;
  const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
  const uint32_t bar_a = tc::smem_u32(&bar);
  uint32_t phase = 0;

  auto wait_mma = [&]() {
    if (!abort_s) {
      if (!tc::mbar_wait_bounded(bar_a, phase, kWaitLimit)) {
        abort_s = 1;
        if (p.status) atomicOr(p.status, DR_DEV_TIMEOUT);
      }
    }
    phase ^= 1;
    tc::tc_fence_after();
  };

  // ---- initial state: S^T[v][k] = h0[k][v] (thread = value column v) -------------------------
  {
    const float* h0 = p.h0 ? p.h0 + (int64_t)unit * kD * kD : nullptr;
    for (int c0 = 0; c0 < kD; c0 += 32) {
      uint32_t r[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) r[j] = h0 ? __float_as_uint(h0[(c0 + j) * kD + tid]) : 0u;
      tc::tmem_st32(tbase + TM_S + lane_addr + c0, r);
    }
    tc::tc_wait_st();
  }

  const uint32_t id_n64 = tc::idesc_bf16(128, 64, 0, 0);
  const uint32_t id_n128 = tc::idesc_bf16(128, 128, 0, 0);
  const uint32_t id_n128_mn = tc::idesc_bf16(128, 128, 0, 1);
  const uint32_t aQK = tc::smem_u32(sQK), aT = tc::smem_u32(sT), aAqk = tc::smem_u32(sAqk);

  const int nchunks = (T + kC - 1) / kC;
  for (int n = 0; n < nchunks; ++n) {
    const int t0 = n * kC;
    const int rows = min(kC, T - t0);
    __syncthreads();  // previous chunk's readers of smem are done
    // ---- P1: stage K^, Q^ (fp32 l2norm, q scaled), V, g, beta --------------------------------
    {
      const int r = tid >> 1, half = tid & 1;  // row r, columns [64*half, 64*half+64)
      const bool live = r < rows;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const __nv_bfloat16* src = (which == 0 ? gk : gq) + qk_base + (int64_t)(t0 + r) * qk_tok + 64 * half;
        uint4 raw[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) raw[j] = live ? reinterpret_cast<const uint4*>(src)[j] : make_uint4(0, 0, 0, 0);
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[j]);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h2[e]);
            ss += f.x * f.x + f.y * f.y;
          }
        }
        float mul = which == 0 ? 1.f : p.scale;
        if (p.l2norm) {
          ss += __shfl_xor_sync(0xffffffffu, ss, 1);
          mul = mul / (sqrtf(ss) + 1e-6f);
        }
        const int row = which == 0 ? r : 64 + r;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[j]);
          uint4 out;
          uint32_t* o32 = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h2[e]);
            o32[e] = tc::pack_bf16(f.x * mul, f.y * mul);
          }
          *reinterpret_cast<uint4*>(sQK + tc::core_off(row, 64 * half + 8 * j, QK_RBS)) = out;
        }
      }
      // V rows: 64 rows x 256 B; thread handles 8 x 16 B of row r, half
      {
        const __nv_bfloat16* src = gv + qk_base + (int64_t)(t0 + r) * qk_tok + 64 * half;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint4 x = live ? reinterpret_cast<const uint4*>(src)[j] : make_uint4(0, 0, 0, 0);
          reinterpret_cast<uint4*>(sV + r * kD + 64 * half)[j] = x;
        }
      }
      if (tid < 64) {
        const bool lv = tid < rows;
        sBeta[tid] = lv ? p.beta[s_base + (int64_t)(t0 + tid) * s_tok] : 0.f;
        sG[tid] = (lv && gg) ? gg[s_base + (int64_t)(t0 + tid) * s_tok] : 0.f;
      }
    }
    __syncthreads();
    if (warp == 0) {  // inclusive scan of g over the 64 rows
      float a = sG[lane], bq = sG[lane + 32];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float x = __shfl_up_sync(0xffffffffu, a, o);
        const float y = __shfl_up_sync(0xffffffffu, bq, o);
        if (lane >= o) { a += x; bq += y; }
      }
      const float tot = __shfl_sync(0xffffffffu, a, 31);
      bq += tot;
      const float last = __shfl_sync(0xffffffffu, bq, 31);
      sG[lane] = a; sG[lane + 32] = bq;
      sEG[lane] = __expf(a); sEG[lane + 32] = __expf(bq);
      sW[lane] = __expf(fminf(last - a, 0.f)); sW[lane + 32] = __expf(fminf(last - bq, 0.f));
    }
    tc::fence_async_smem();
    tc::tc_fence_before();
    __syncthreads();
    // ---- P2: D1 = [K^;Q^] K^^T ------------------------------------------------------------------
    if (tid == 0) {
      tc::tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint64_t ad = tc::smem_desc(aQK + ks * 256, 128, QK_RBS);
        tc::mma_ss(tbase + TM_D3, ad, ad, id_n64, ks > 0);  // B = first 64 rows of the same tile
      }
      tc::mma_commit(bar_a);
    }
    wait_mma();
    // ---- P3: A_kk (fp32, rows 0..63) and A_qk (bf16 operand, rows 64..127) -----------------------
    {
      const int i = tid & 63;
      const float Gi = sG[i], bi = sBeta[i];
#pragma unroll
      for (int c0 = 0; c0 < 64; c0 += 32) {
        uint32_t r[32];
        tc::tmem_ld32(tbase + TM_D3 + lane_addr + c0, r);
        tc::tc_wait_ld();
        if (tid < 64) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int jj = c0 + j;
            const float x = __uint_as_float(r[j]) * __expf(fminf(Gi - sG[jj], 0.f)) * bi;
            sAkk[i * AKK_LD + jj] = jj < i ? x : 0.f;
          }
        } else {
#pragma unroll
          for (int j8 = 0; j8 < 4; ++j8) {
            uint4 out;
            uint32_t* o32 = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int j0 = c0 + 8 * j8 + 2 * e;
              float x0 = __uint_as_float(r[8 * j8 + 2 * e]) * __expf(fminf(Gi - sG[j0], 0.f));
              float x1 = __uint_as_float(r[8 * j8 + 2 * e + 1]) * __expf(fminf(Gi - sG[j0 + 1], 0.f));
              x0 = j0 <= i ? x0 : 0.f;
              x1 = j0 + 1 <= i ? x1 : 0.f;
              o32[e] = tc::pack_bf16(x0, x1);
            }
            *reinterpret_cast<uint4*>(sAqk + tc::core_off(i, c0 + 8 * j8, A_RBS)) = out;
          }
        }
      }
    }
    tc::tc_fence_before();
    __syncthreads();
    // ---- P4: T = (I + A_kk)^-1, one column per thread (threads 0..63); state pass (all) ----------
    if (tid < 64) {
      float x[64];
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        float acc = (i == tid) ? 1.f : 0.f;
        const float* arow = sAkk + i * AKK_LD;
#pragma unroll
        for (int j = 0; j < i; ++j) acc -= arow[j] * x[j];
        x[i] = acc;
      }
#pragma unroll
      for (int i = 0; i < 64; ++i)
        *reinterpret_cast<__nv_bfloat16*>(sT + tc::core_off(i, tid, A_RBS)) = __float2bfloat16_rn(x[i]);
    }
    {
      // S^T: bf16 copy of the undecayed state for (2); fp32 master pre-multiplied by e^{G_L} for (5)
      tc::tc_fence_after();
      const float gl = sEG[63];
#pragma unroll
      for (int c0 = 0; c0 < kD; c0 += 32) {
        uint32_t r[32], pk[16];
        tc::tmem_ld32(tbase + TM_S + lane_addr + c0, r);
        tc::tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j) pk[j] = tc::pack_bf16(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * gl);
        tc::tmem_st16(tbase + TM_SB + lane_addr + c0 / 2, pk);
        tc::tmem_st32(tbase + TM_S + lane_addr + c0, r);
      }
      tc::tc_wait_st();
    }
    tc::fence_async_smem();
    tc::tc_fence_before();
    __syncthreads();
    // ---- P5: D2 = S^T [K^;Q^]^T --------------------------------------------------------------------
    if (tid == 0) {
      tc::tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint64_t bd = tc::smem_desc(aQK + ks * 256, 128, QK_RBS);
        tc::mma_ts(tbase + TM_D2, tbase + TM_SB + ks * 8, bd, id_n128, ks > 0);
      }
      tc::mma_commit(bar_a);
    }
    wait_mma();
    // ---- P6: R^T[v][c] = beta_c (V[c][v] - D2[v][c] e^{G_c}) -> bf16 A operand -----------------------
#pragma unroll
    for (int c0 = 0; c0 < 64; c0 += 32) {
      uint32_t r[32], pk[16];
      tc::tmem_ld32(tbase + TM_D2 + lane_addr + c0, r);
      tc::tc_wait_ld();
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int c = c0 + 2 * j;
        const float a0 = sBeta[c] * (__bfloat162float(sV[c * kD + tid]) - __uint_as_float(r[2 * j]) * sEG[c]);
        const float a1 = sBeta[c + 1] * (__bfloat162float(sV[(c + 1) * kD + tid]) - __uint_as_float(r[2 * j + 1]) * sEG[c + 1]);
        pk[j] = tc::pack_bf16(a0, a1);
      }
      tc::tmem_st16(tbase + TM_RA + lane_addr + c0 / 2, pk);
    }
    tc::tc_wait_st();
    tc::tc_fence_before();
    __syncthreads();
    // ---- P7: D3 = R^T T^T = V_new^T ---------------------------------------------------------------------
    if (tid == 0) {
      tc::tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        const uint64_t bd = tc::smem_desc(aT + ks * 256, 128, A_RBS);
        tc::mma_ts(tbase + TM_D3, tbase + TM_RA + ks * 8, bd, id_n64, ks > 0);
      }
      tc::mma_commit(bar_a);
    }
    wait_mma();
    // ---- P8: V_new^T -> bf16 (plain, and decayed by e^{G_L - G_c}) ----------------------------------------
#pragma unroll
    for (int c0 = 0; c0 < 64; c0 += 32) {
      uint32_t r[32], pa[16], pb[16];
      tc::tmem_ld32(tbase + TM_D3 + lane_addr + c0, r);
      tc::tc_wait_ld();
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float x0 = __uint_as_float(r[2 * j]), x1 = __uint_as_float(r[2 * j + 1]);
        pa[j] = tc::pack_bf16(x0, x1);
        pb[j] = tc::pack_bf16(x0 * sW[c0 + 2 * j], x1 * sW[c0 + 2 * j + 1]);
      }
      tc::tmem_st16(tbase + TM_RA + lane_addr + c0 / 2, pa);
      tc::tmem_st16(tbase + TM_VB + lane_addr + c0 / 2, pb);
    }
    tc::tc_wait_st();
    tc::tc_fence_before();
    __syncthreads();
    // ---- P9: D4 = V_new^T A_qk^T ;  S^T += (decayed V_new^T) K^ ----------------------------------------------
    if (tid == 0) {
      tc::tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        const uint64_t bd = tc::smem_desc(aAqk + ks * 256, 128, A_RBS);
        tc::mma_ts(tbase + TM_D3, tbase + TM_RA + ks * 8, bd, id_n64, ks > 0);
      }
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        // K^ rows (chunk positions) are the contraction axis: MN-major, 16 rows = 2 row blocks per step
        const uint64_t bd = tc::smem_desc(aQK + ks * 2 * QK_RBS, QK_RBS, 128);
        tc::mma_ts(tbase + TM_S, tbase + TM_VB + ks * 8, bd, id_n128_mn, 1);
      }
      tc::mma_commit(bar_a);
    }
    wait_mma();
    // ---- P10: O^T[v][i] = e^{G_i} D2[v][64+i] + D4[v][i]; stage through shared memory ------------------------
#pragma unroll
    for (int c0 = 0; c0 < 64; c0 += 32) {
      uint32_t r2[32], r4[32];
      tc::tmem_ld32(tbase + TM_D2 + lane_addr + 64 + c0, r2);
      tc::tmem_ld32(tbase + TM_D3 + lane_addr + c0, r4);
      tc::tc_wait_ld();
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int i = c0 + j;
        sV[i * kD + tid] = __float2bfloat16_rn(sEG[i] * __uint_as_float(r2[j]) + __uint_as_float(r4[j]));
      }
    }
    tc::tc_fence_before();
    __syncthreads();
    {
      const int r = tid >> 1, half = tid & 1;
      if (r < rows) {
        __nv_bfloat16* dst = go + qk_base + (int64_t)(t0 + r) * qk_tok + 64 * half;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          reinterpret_cast<uint4*>(dst)[j] = reinterpret_cast<const uint4*>(sV + r * kD + 64 * half)[j];
      }
    }
  }
  // ---- final state: hT[k][v] = S^T[v][k] ---------------------------------------------------------------
  tc::tc_fence_after();
  if (p.hT) {
    float* hT = p.hT + (int64_t)unit * kD * kD;
    for (int c0 = 0; c0 < kD; c0 += 32) {
      uint32_t r[32];
      tc::tmem_ld32(tbase + TM_S + lane_addr + c0, r);
      tc::tc_wait_ld();
#pragma unroll
      for (int j = 0; j < 32; ++j) hT[(c0 + j) * kD + tid] = __uint_as_float(r[j]);
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tbase, TM_COLS);
}

inline cudaError_t launch_chunk(const FwdParams& p, cudaStream_t stream) {
  cudaError_t e = cudaFuncSetAttribute(chunk_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_TOTAL);
  if (e != cudaSuccess) return e;
  const dim3 grid((unsigned)((int64_t)p.map.B * p.map.H)), block(kThreads);
  chunk_sm100_kernel<<<grid, block, SM_TOTAL, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace sm100
}  // namespace dr
