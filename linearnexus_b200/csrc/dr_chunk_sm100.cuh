// Chunkwise gated delta-rule forward on the Blackwell tensor cores (tcgen05 + TMEM).
//
// Shape: K = V = 128, chunk C = 64, bf16 q/k/v/o, fp32 g/beta/state.  One CTA of 512 threads
// owns one (batch, head) sequence.  The fp32 state lives TRANSPOSED in tensor memory for the
// whole sequence (S^T: lane = value column v, column = key row k), so every product has
// M = 128 and each epilogue thread owns one value column.
//
// Four groups of four warps (one warp per 32-lane quarter of tensor memory in each group) form a
// pipeline over the chunks of the sequence.  Each group has its own instruction stream, so the short
// dependent phases of one group fill the issue slots the others leave idle.  A tcgen05.mma instruction
// occupies the tensor pipe (and its issuing thread) for about 64 cycles whatever its N <= 128; the 40
// instructions of a chunk are spread over elected threads of three groups so that only products (3) and
// (5) sit on the serial chain.
//
//   PA (warps 0-3)   state-independent, chunk n:
//     K,Q rows land by TMA as one [K;Q] tile already in core-matrix order (4-slot ring; the copy of chunk n+2 is
//     issued as soon as chunk n-2 has left the consumer, before this group waits for chunk n+1's tile).
//     The l2 norms are not applied to the tiles: they are folded into row and column factors (rk from the
//     diagonal of D1, rq from the raw Q rows).
//     (1) D1 = [K;Q] K^T                             128x64x128  smem x smem, issued one chunk ahead
//         X = D1[i][j] e^{G_i-G_j} (i>=j, fp32) -> fp32 matrix;  A_qk = D1[64+i][j] e^{G_i-G_j} (i>=j) -> bf16 tile
//   PB (warps 4-7)   chunk n, one hand-over behind PA:
//         T = (I + diag(beta rk^2) X)^-1 in place: 8x8 blocks by substitution, three merge levels on mma.sync tf32
//         -> Tb = T diag(beta rk), Tw = T diag(beta e^G rk^2)   bf16 tiles
//         rq_i = scale / (||q_i|| + eps) of the next chunk (mma.sync on the raw Q rows)
//   CB (warps 12-15) everything around the chain, as early as its inputs allow; its products are issued by
//         threads of three different warps (0: W^T, 32: U^T and the V copy, 64: Dq):
//     (2) W^T = K^T Tw^T  -> the stage accumulator (still idle) -> bf16 tile W (MN-major B operand: 16-byte stores)
//         U^T = V^T Tb^T  -> the stage accumulator            128x64x64   smem(MN-major) x smem
//         output of the previous chunk: O^T[v][i] = rq_i (e^{G_i} Dq[v][i] + Do[v][i]), from the accumulators
//         to global memory (lane pairs exchange halves: 4-byte stores, 64 contiguous bytes per token row and warp);
//         then  Dq = S^T Q^T of this chunk                                                 128x64x128
//   CA (warps 8-11)  the serial chain over the state:
//         bf16 copy of S^T for the products; fp32 S^T pre-multiplied by e^{G_L}
//     (3) V_new^T = U^T - S^T W^T  (accumulated onto U^T with negate-A)                    128x64x128
//         V_new^T -> bf16, plain and decayed by e^{G_L-G_c}
//     (5) S^T += (V_new^T e^{G_L-G_c}) K   (K read MN-major)                                128x128x64
//     (4) Do = V_new^T A_qk^T                                                              128x64x64
//
// The [K;Q] tile is stored once as 8x8 core matrices and serves as A and B of (1), MN-major
// A of (2), K-major B of Dq and MN-major B of (5).  Hand-overs are mbarriers (arrive counts of a whole
// group, or tcgen05.commit for product completion); every wait is bounded: a wait that runs out sets
// DR_DEV_TIMEOUT in the status word (with the barrier and group that gave up) and the kernel finishes without
// further waiting.  A wait site is one mbarrier.try_wait; the bounded loop, the abort flag and the record live in
// one out-of-line function (the hand-over latency and the size of the four loop bodies are what the step time
// follows).  A barrier whose waiter can lag its producer by more than one completion is doubled (bar2 / bar2b).
#pragma once

#include <cuda.h>

#include <cstring>

#include "dr_common.cuh"
#include "dr_sm100_common.cuh"
#include "dr_tcgen05.cuh"
#include "dr_umma_selftest.cuh"

namespace dr {
namespace sm100 {

constexpr bool kAvailable = true;
constexpr int kThreads = 512;
constexpr int kGrp = 128;

// tensor-memory columns (32-bit x 128 lanes each): 512 in total
constexpr uint32_t TM_S = 0;      // S^T fp32                                   128
constexpr uint32_t TM_SB = 128;   // bf16 copy of S^T (A operand)                 64
constexpr uint32_t TM_D1 = 192;   // D1                                           64
constexpr uint32_t TM_DU = 256;   // 2 stages x 64: W^T, then U^T -> V_new^T -> Do   128
constexpr uint32_t TM_DQ = 384;   // S^T Q^^T                                     64
constexpr uint32_t TM_VA = 448;   // V_new^T bf16                                 32
constexpr uint32_t TM_VB = 480;   // decayed V_new^T bf16                         32
constexpr uint32_t TM_COLS = 512;

// shared-memory map (bytes)
constexpr int QK_TILE = 128 * 128 * 2;        // [K (64 rows); Q (64 rows)] x 128 raw bf16, 32 KB
constexpr int kRing = 4;                      // K,Q tiles in flight: one each in PA, PB, the consumer + one landing
constexpr int SM_QKR = 0;                     // ring of kRing such tiles (chunk n uses tile n % kRing)
constexpr int W_TILE = 128 * 64 * 2;          // W as [128 k][64 c] core matrices, 16 KB
constexpr int SM_W = kRing * QK_TILE;         // one W tile
constexpr int AQK_TILE = 64 * 64 * 2;         // A_qk [64][64] bf16, 8 KB
constexpr int SM_AQK = SM_W + W_TILE;         // three A_qk tiles (chunk n uses n % 3)
constexpr int SM_V = SM_AQK + 3 * AQK_TILE;   // V [64][128] core-matrix tile, 16 KB
constexpr int AKK_BYTES = 64 * LDT * 4;       // X, then T in place (fp32 [64][68]), then the bf16 tiles
constexpr int SM_AKK = SM_V + 64 * 128 * 2;   // two such buffers (chunk n uses n & 1)
constexpr int XB_TB = 0;                      //   T diag(beta rk)         [64][64] bf16 core-matrix tile, 8 KB
constexpr int XB_TW = 64 * 64 * 2;            //   T diag(beta e^G rk^2)   [64][64] bf16, 8 KB
constexpr int SM_TOTAL = SM_AKK + 2 * AKK_BYTES;

struct alignas(16) Ctl {
  uint64_t full[3], empty[3], akk[2], xfree[2], kq[kRing], vb, barP, barW, barUW, wrdy, sbrdy, bar1, bar2s, bar2, barDq;
  alignas(16) float gb[128];         // raw beta (0..63) and g (64..127) of the chunk being scanned
  alignas(16) float rq[4][64];       // scale / (||q_i|| + eps) of chunk m in slot m % 4
  alignas(16) float sc[4][256];      // of chunk m in slot m % 4: e^G, e^{G_L-G}, beta, G log2(e) (64 each)
  alignas(16) float keep[3][128];    // CB-private, chunk m in slot m % 3: rq_i e^{G_i} (0..63) and rq_i (64..127); three
                                     // slots so that a group barrier lies between the last read and the next write of one
  alignas(16) float rk[2][64];       // per X buffer: 1 / (||k_j|| + eps)
  alignas(16) float rs[2][64];       // per X buffer: beta_i rk_i^2, row factor of the unit-lower system
  uint32_t tmem_base;
  int abort;
  uint64_t bar2b;                    // the output products' barrier of the odd chunks (bar2: even chunks); it fills what
                                     // was padding, the block is as large as without it
};

// Kernel parameters: the common forward parameters plus the TMA tensor maps (see make_input_map /
// make_output_map); the map coordinates of a sequence are derived from (b, h) in the kernel.
struct alignas(64) Sm100Params {
  CUtensorMap tk, tq, tv;
  FwdParams p;
};

// A shared-memory descriptor whose start address is `bytes` further on (the address field holds bytes / 16 and
// cannot carry out of its 14 bits for addresses inside one CTA's shared memory).
__device__ __forceinline__ uint64_t desc_adv(uint64_t d, uint32_t bytes) { return d + (uint64_t)(bytes >> 4); }

struct SyncPB { __device__ __forceinline__ void operator()() const { group_sync128(2); } };

template <bool kTma>
__global__ void __launch_bounds__(kThreads, 1) chunk_sm100_kernel(const __grid_constant__ Sm100Params P) {
  const FwdParams& p = P.p;
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ __align__(16) Ctl ctl;   // its float arrays are read with 16-byte loads

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int grp = warp >> 2;             // 0 PA, 1 PB, 2 CA, 3 CB
  const int gt = tid & (kGrp - 1);       // thread index inside its group = tensor-memory lane it owns
  const int wq = warp & 3;
  const int T = p.map.T;
  const int unit = blockIdx.x;
  const int b = unit / p.map.H, h = unit % p.map.H;
  const int hq = p.map.hq(h);
  const int64_t qk_base = p.map.base_qk(b, h, kD), qk_tok = p.map.tok_qk(kD);   // q, k (possibly fewer heads)
  const int64_t vo_base = p.map.base(b, h, kD), vo_tok = p.map.tok(kD);         // v, o
  const int64_t s_base = p.map.base(b, h, 1), s_tok = p.map.tok(1);
  // tensor-map coordinates of this sequence (column-block origin, outermost index)
  const int qc2 = p.map.bthd ? 16 * hq : 0, qc4 = p.map.bthd ? b : b * p.map.Hq + hq;
  const int vc2 = p.map.bthd ? 16 * h : 0, vc4 = p.map.bthd ? b : unit;

  if (warp == 0) {
    tc::tmem_alloc(tc::smem_u32(&ctl.tmem_base), TM_COLS);
    tc::tmem_relinquish();
  }
  if (tid == 0) {
    for (int i = 0; i < 3; ++i) {
      tc::mbar_init(tc::smem_u32(&ctl.full[i]), kGrp);
      tc::mbar_init(tc::smem_u32(&ctl.empty[i]), kGrp);
    }
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(tc::smem_u32(&ctl.akk[i]), kGrp);
      tc::mbar_init(tc::smem_u32(&ctl.xfree[i]), 1);
    }
    for (int i = 0; i < kRing; ++i) tc::mbar_init(tc::smem_u32(&ctl.kq[i]), kTma ? 1 : kGrp);
    tc::mbar_init(tc::smem_u32(&ctl.vb), kTma ? 1 : kGrp);
    tc::mbar_init(tc::smem_u32(&ctl.barP), 1);
    tc::mbar_init(tc::smem_u32(&ctl.barW), 1);
    tc::mbar_init(tc::smem_u32(&ctl.barUW), 1);
    tc::mbar_init(tc::smem_u32(&ctl.wrdy), kGrp);
    tc::mbar_init(tc::smem_u32(&ctl.sbrdy), kGrp);
    tc::mbar_init(tc::smem_u32(&ctl.bar1), 1);
    tc::mbar_init(tc::smem_u32(&ctl.bar2s), 1);
    tc::mbar_init(tc::smem_u32(&ctl.bar2), 1);
    tc::mbar_init(tc::smem_u32(&ctl.bar2b), 1);
    tc::mbar_init(tc::smem_u32(&ctl.barDq), 1);
    tc::fence_mbar_init();
    ctl.abort = 0;
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tbase = ctl.tmem_base;
  const uint32_t lane_addr = (uint32_t)(wq * 32) << 16;

  auto wait_bar = [&](uint64_t* bar, uint32_t parity) {
    if (tc::mbar_try(tc::smem_u32(bar), parity)) return;   // the common case, and all that a call site carries
    wait_more(tc::smem_u32(bar), parity, p.status, &ctl.abort, (uint32_t)((const char*)bar - (const char*)&ctl), (uint32_t)grp);
  };
  auto arrive = [&](uint64_t* bar) { mbar_arrive(tc::smem_u32(bar)); };

  const uint32_t id_n64 = tc::idesc_bf16(128, 64, 0, 0);
  const uint32_t id_n64_amn = tc::idesc_bf16(128, 64, 1, 0);
  const uint32_t id_n64_bmn_neg = tc::idesc_bf16(128, 64, 0, 1) | (1u << 13);
  const uint32_t id_n128_bmn = tc::idesc_bf16(128, 128, 0, 1);
  const int nchunks = (T + kC - 1) / kC;
  float* const sAkk0 = reinterpret_cast<float*>(smem + SM_AKK);

  if (grp == 0) {
    // =========================== PA: K,Q tiles, D1, decay masks ======================================
    const __nv_bfloat16* gq = reinterpret_cast<const __nv_bfloat16*>(p.q);
    const __nv_bfloat16* gk = reinterpret_cast<const __nv_bfloat16*>(p.k);
    const float* gg = p.g ? reinterpret_cast<const float*>(p.g) + s_base : nullptr;
    const float* gbeta = p.beta + s_base;

    // K,Q rows (raw bf16), g and beta of chunk m -> ring tile m % kRing / raw scalars.  The l2 normalisation is
    // NOT applied to the tiles: it is folded into the factors rk, rs, rq.  Warp 0 fetches the scalars (and
    // later scans them); with TMA its first lane also issues the tile copies.
    auto issue_kq = [&](int m) {
      const int t0m = m * kC, rowsm = min(kC, T - t0m);
      uint8_t* dQK = smem + SM_QKR + (m % kRing) * QK_TILE;
      if (kTma) {
        if (gt == 0) {
          const uint32_t bar = tc::smem_u32(&ctl.kq[m % kRing]);
          tc::mbar_arrive_expect_tx(bar, 2u * 64 * 256);
          tc::tma_load_5d(tc::smem_u32(dQK), &P.tk, 0, 0, qc2, m * 8, qc4, bar);
          tc::tma_load_5d(tc::smem_u32(dQK) + 64 * 256, &P.tq, 0, 0, qc2, m * 8, qc4, bar);
        }
      } else {
        const int rin = gt & 7, kb = gt >> 3;
#pragma unroll 2
        for (int rb = 0; rb < 8; ++rb) {
          const int r = rb * 8 + rin;
          const bool live = r < rowsm;
          const int64_t off = qk_base + (int64_t)(t0m + (live ? r : 0)) * qk_tok + kb * 8;
          tc::cp_async16(tc::smem_u32(dQK + tc::core_off(r, kb * 8, RBS)), gk + off, live);
          tc::cp_async16(tc::smem_u32(dQK + tc::core_off(64 + r, kb * 8, RBS)), gq + off, live);
        }
      }
      if (warp == 0) {
        float* dG = ctl.gb;
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const int r = lane + 32 * hf;
          const bool live = r < rowsm;
          const int64_t off = live ? (int64_t)(t0m + r) * s_tok : 0;
          tc::cp_async4(tc::smem_u32(dG + r), gbeta + off, live);                          // beta
          tc::cp_async4(tc::smem_u32(dG + 64 + r), gg ? gg + off : gbeta, live && gg);     // g (0 without decay)
        }
      }
      tc::cp_async_commit();
    };
    // every thread: its copies of chunk m have landed (and, without TMA, are published on the tile's barrier)
    auto land_kq = [&](int m) {
      tc::cp_async_wait_all();
      if (!kTma) {
        tc::fence_async_smem();
        arrive(&ctl.kq[m % kRing]);
      }
    };

    // inclusive scan of the log decay over the 64 rows of a chunk (one warp): G, e^G, e^{G_L - G}, beta and
    // G2 = G log2(e) (the decay mask takes its exponentials in base 2)
    auto scan_stage = [&](int m) {
      constexpr float kLog2e = 1.4426950408889634f;
      float* zG = ctl.sc[m % 4];
      const float* raw = ctl.gb;
      zG[128 + lane] = raw[lane]; zG[160 + lane] = raw[32 + lane];   // beta
      float a = raw[64 + lane], bq = raw[96 + lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float x = __shfl_up_sync(0xffffffffu, a, o);
        const float y = __shfl_up_sync(0xffffffffu, bq, o);
        if (lane >= o) { a += x; bq += y; }
      }
      const float tot = __shfl_sync(0xffffffffu, a, 31);
      bq += tot;
      const float last = __shfl_sync(0xffffffffu, bq, 31);
      zG[lane] = tc::fast_exp2(a * kLog2e); zG[32 + lane] = tc::fast_exp2(bq * kLog2e);
      zG[64 + lane] = tc::fast_exp2(fminf(last - a, 0.f) * kLog2e);
      zG[96 + lane] = tc::fast_exp2(fminf(last - bq, 0.f) * kLog2e);
      zG[192 + lane] = a * kLog2e; zG[224 + lane] = bq * kLog2e;
    };

    // first product of chunk m: D1 = [K;Q] K^T on the raw rows (B = first 64 rows of the same tile)
    auto issue_d1 = [&](int m) {
      wait_bar(&ctl.kq[m % kRing], (m / kRing) & 1);
      tc::tc_fence_after();
      const uint64_t ad0 = tc::smem_desc(tc::smem_u32(smem + SM_QKR + (m % kRing) * QK_TILE), 128, RBS);
#pragma unroll 1
      for (int ks = 0; ks < 8; ++ks) {
        const uint64_t ad = desc_adv(ad0, ks * 256);
        tc::mma_ss(tbase + TM_D1, ad, ad, id_n64, ks > 0);
      }
      tc::mma_commit(tc::smem_u32(&ctl.barP));
    };

    issue_kq(0);
    land_kq(0);
    if (warp == 0) { __syncwarp(); scan_stage(0); }
    if (gt == 64) issue_d1(0);
    if (nchunks > 1) issue_kq(1);   // the copies run two chunks ahead of the masks (see the end of the loop body)
    uint32_t phP = 0;
    for (int n = 0; n < nchunks; ++n) {
      const int s = n & 1;
      uint8_t* sAqk = smem + SM_AQK + (n % 3) * AQK_TILE;
      float* sX = sAkk0 + s * (64 * LDT);
      const float* sG = ctl.sc[n % 4];
      const float* sBeta = sG + 128;
      group_sync128(1);  // the scalars of this chunk (scan) are visible
      // chunk n-2 has left PB and its U^T, W^T products: X buffer s is free.  (Chunk n-3 has left the consumer, so the
      // A_qk tile n % 3 is free: waited for at the end of the previous iteration.)
      if (n >= 2) wait_bar(&ctl.xfree[s], ((n >> 1) - 1) & 1);
      wait_bar(&ctl.barP, phP); phP ^= 1;   // D1 of this chunk was issued during the previous iteration
      tc::tc_fence_after();
      {
        // one pass per 32-column half at or below this warp's diagonal (rows 0..31: one, rows 32..63: two), the same
        // code for both: x = D1 . 2^{min(G2_i - G2_j, 0)}.  X keeps whatever lands above the diagonal (the inverse
        // reads the strict lower triangle only; the diagonal holds ||k_i||^2 until the inverse overwrites it);
        // the A_qk tile is an operand of product (4) and gets exact zeros there.  The row factor beta_i rk_i^2 and
        // the column factors rk_j are applied later (rs in the solve, rk in the Tb/Tw tiles).
        const int i = gt & 63;
        const bool qrow = gt >= 64;        // warps 2,3 hold the Q rows (A_qk); warps 0,1 the K rows (X)
        const int nh = 1 + (wq & 1);
        const float* sG2 = sG + 192;
        const float Gi = sG2[i];
#pragma unroll 1
        for (int c0 = 0; c0 < 32 * nh; c0 += 16) {
          uint32_t r[16];
          tc::tmem_ld16(tbase + TM_D1 + lane_addr + c0, r);
          tc::tc_wait_ld();
#pragma unroll
          for (int j4 = 0; j4 < 4; ++j4) {
            const float4 g4 = *reinterpret_cast<const float4*>(sG2 + c0 + 4 * j4);
            r[4 * j4 + 0] = __float_as_uint(__uint_as_float(r[4 * j4 + 0]) * tc::fast_exp2(fminf(Gi - g4.x, 0.f)));
            r[4 * j4 + 1] = __float_as_uint(__uint_as_float(r[4 * j4 + 1]) * tc::fast_exp2(fminf(Gi - g4.y, 0.f)));
            r[4 * j4 + 2] = __float_as_uint(__uint_as_float(r[4 * j4 + 2]) * tc::fast_exp2(fminf(Gi - g4.z, 0.f)));
            r[4 * j4 + 3] = __float_as_uint(__uint_as_float(r[4 * j4 + 3]) * tc::fast_exp2(fminf(Gi - g4.w, 0.f)));
          }
          if (!qrow) {
#pragma unroll
            for (int j4 = 0; j4 < 4; ++j4)
              *reinterpret_cast<uint4*>(sX + i * LDT + c0 + 4 * j4) = make_uint4(r[4 * j4], r[4 * j4 + 1], r[4 * j4 + 2], r[4 * j4 + 3]);
          } else {
            const int lim = i - c0;   // columns c0 + e with e <= lim are at or below the diagonal
#pragma unroll
            for (int j8 = 0; j8 < 2; ++j8) {
              uint4 out;
              uint32_t* o32 = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int e0 = 8 * j8 + 2 * e;
                const float x0 = e0 <= lim ? __uint_as_float(r[e0]) : 0.f;
                const float x1 = e0 + 1 <= lim ? __uint_as_float(r[e0 + 1]) : 0.f;
                o32[e] = tc::pack_bf16(x0, x1);
              }
              *reinterpret_cast<uint4*>(sAqk + tc::core_off(i, c0 + 8 * j8, A_RBS)) = out;
            }
          }
        }
        if (!qrow) {
          const float d = sX[i * LDT + i];   // this thread's own store
          const float rk = p.l2norm ? 1.f / (sqrtf(d) + 1e-6f) : 1.f;
          ctl.rk[s][i] = rk;
          ctl.rs[s][i] = sBeta[i] * rk * rk;
        } else if (nh == 1) {   // rows 0..31: columns 32..63 lie above the diagonal
#pragma unroll
          for (int j8 = 0; j8 < 4; ++j8)
            *reinterpret_cast<uint4*>(sAqk + tc::core_off(i, 32 + 8 * j8, A_RBS)) = make_uint4(0u, 0u, 0u, 0u);
        }
      }
      tc::fence_async_smem();                // the A_qk tile is read by the tensor cores
      tc::tc_fence_before();
      arrive(&ctl.akk[s]);                   // X, A_qk, rk, rs of chunk n are ready: PB starts
      group_sync128(1);                      // every warp has drained D1 from tensor memory
      // what the NEXT chunk needs from this group, behind the hand-over
      if (n + 1 < nchunks) {
        land_kq(n + 1);                      // the next chunk's beta, g (and, without TMA, its K,Q rows)
        if (gt == 64) issue_d1(n + 1);       // completes behind PB's inverse of this chunk
        if (warp == 0) { __syncwarp(); scan_stage(n + 1); }
      }
      // chunk n-2 has left the consumer: its ring tile and its scalar and rq slots, (n+2) % 4, are free.  The copies of
      // chunk n+2 start here, BEFORE this group waits for chunk n+1's tile at the end of the next iteration: a tile
      // copy (2048 box rows of 16 bytes) takes about as long as a whole iteration, and with the next copy issued only
      // after the previous tile had landed this group's loop was the longest of the four.
      if (n >= 2) wait_bar(&ctl.empty[(n - 2) % 3], ((n - 2) / 3) & 1);
      if (n + 2 < nchunks) issue_kq(n + 2);
    }
  } else if (grp == 1) {
    // =========================== PB: inverse, Tb / Tw tiles ==========================================
    // rq_i = scale / (||q_i|| + eps) of chunk m from the raw rows 64..127 of its tile
    auto q_norms = [&](int m) {
      wait_bar(&ctl.kq[m % kRing], (m / kRing) & 1);
      float* dst = ctl.rq[m % 4];
      const float scale = p.scale;
      const bool l2 = p.l2norm != 0;
      row_sq_norms_64(smem + SM_QKR + (m % kRing) * QK_TILE, 64, wq, lane,
                      [&](int r, float ss) { dst[r] = l2 ? scale / (sqrtf(ss) + 1e-6f) : scale; });
    };
    q_norms(0);
    for (int n = 0; n < nchunks; ++n) {
      const int s = n & 1;
      float* sT = sAkk0 + s * (64 * LDT);
      uint8_t* sTb = reinterpret_cast<uint8_t*>(sT) + XB_TB;
      uint8_t* sTw = reinterpret_cast<uint8_t*>(sT) + XB_TW;
      const float* sEG = ctl.sc[n % 4];
      const float* sBeta = ctl.sc[n % 4] + 128;
      wait_bar(&ctl.akk[s], (n >> 1) & 1);
      block_inverse_64_inplace(sT, ctl.rs[s], gt, SyncPB());
      {
        // Tb = T diag(beta rk), Tw = T diag(beta e^G rk^2) as bf16 tiles IN PLACE of T: every thread takes its 32
        // entries of T into registers, the group synchronises, then the tiles are written over the matrix
        const int rin = gt & 7, jb = (gt >> 3) & 7, rbq = gt >> 6;
        float bj[8], bw[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float rkj = ctl.rk[s][8 * jb + e];
          bj[e] = sBeta[8 * jb + e] * rkj;
          bw[e] = bj[e] * sEG[8 * jb + e] * rkj;
        }
        float4 t0v[4], t1v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int i = 8 * (2 * j + rbq) + rin;
          t0v[j] = *reinterpret_cast<const float4*>(sT + i * LDT + 8 * jb);
          t1v[j] = *reinterpret_cast<const float4*>(sT + i * LDT + 8 * jb + 4);
        }
        group_sync128(2);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int i = 8 * (2 * j + rbq) + rin;
          float t[8] = {t0v[j].x, t0v[j].y, t0v[j].z, t0v[j].w, t1v[j].x, t1v[j].y, t1v[j].z, t1v[j].w};
#pragma unroll
          for (int e = 0; e < 8; ++e) t[e] = (8 * jb + e <= i) ? t[e] : 0.f;
          uint4 ob, ow;
          uint32_t* pb = reinterpret_cast<uint32_t*>(&ob);
          uint32_t* pw = reinterpret_cast<uint32_t*>(&ow);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            pb[e] = tc::pack_bf16(t[2 * e] * bj[2 * e], t[2 * e + 1] * bj[2 * e + 1]);
            pw[e] = tc::pack_bf16(t[2 * e] * bw[2 * e], t[2 * e + 1] * bw[2 * e + 1]);
          }
          const uint32_t off = tc::core_off(i, 8 * jb, A_RBS);
          *reinterpret_cast<uint4*>(sTb + off) = ob;
          *reinterpret_cast<uint4*>(sTw + off) = ow;
        }
      }
      tc::fence_async_smem();
      arrive(&ctl.full[n % 3]);   // A_qk, Tb, Tw and the scalars of chunk n are ready
      if (n + 1 < nchunks) q_norms(n + 1);   // in this group's idle time; published by its next arrival on `full`
    }
  } else if (grp == 2) {
    // =========================== CA: the serial chain over the state =================================
    // initial state: S^T[v][k] = h0[k][v] (thread = value column v)
    {
      const float* h0 = p.h0 ? p.h0 + (int64_t)unit * kD * kD : nullptr;
#pragma unroll 1
      for (int cc = 0; cc < 4; ++cc) {
        const int c0 = 32 * cc;
        uint32_t r[32];
#pragma unroll
        for (int j = 0; j < 32; ++j)
          r[j] = (h0 && in_bounds(p.status, (h0 - p.h0) + (c0 + j) * kD + gt, p.n_state)) ? __float_as_uint(h0[(c0 + j) * kD + gt]) : 0u;
        tc::tmem_st32(tbase + TM_S + lane_addr + c0, r);
      }
      tc::tc_wait_st();
    }
    uint32_t ph1 = 0;
    for (int n = 0; n < nchunks; ++n) {
      const int s = n & 1;
      const uint32_t aQK = tc::smem_u32(smem + SM_QKR + (n % kRing) * QK_TILE);
      const uint32_t aW = tc::smem_u32(smem + SM_W);
      const uint32_t aAqk = tc::smem_u32(smem + SM_AQK + (n % 3) * AQK_TILE);
      const float* sEG = ctl.sc[n % 4];
      const float* sWd = sEG + 64;
      if (n >= 1) {
        wait_bar(&ctl.bar2s, (n - 1) & 1);   // the state update of the previous chunk is complete, and with it
        wait_bar(&ctl.barDq, (n - 1) & 1);   // every earlier product of the chain; Dq has read the bf16 state
      }
      wait_bar(&ctl.full[n % 3], (n / 3) & 1);
      tc::tc_fence_after();
      // ---- state pass: bf16 copy of S^T for the products; fp32 master pre-multiplied by e^{G_L} --------
      {
        const float gl = sEG[63];
#pragma unroll 1
        for (int c0 = 0; c0 < kD; c0 += 16) {
          uint32_t r[16], pk[8];
          tc::tmem_ld16(tbase + TM_S + lane_addr + c0, r);
          tc::tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 8; ++j) pk[j] = tc::pack_bf16(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
          if (p.ckpt) {  // state at the start of this chunk, [K][V] row-major, for the backward
            float* ck = p.ckpt + ((int64_t)unit * nchunks + n) * kD * kD;
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (in_bounds(p.status, (ck - p.ckpt) + (c0 + j) * kD + gt, p.n_ckpt)) ck[(c0 + j) * kD + gt] = __uint_as_float(r[j]);
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * gl);
          tc::tmem_st8(tbase + TM_SB + lane_addr + c0 / 2, pk);
          tc::tmem_st16(tbase + TM_S + lane_addr + c0, r);
        }
        tc::tc_wait_st();
      }
      tc::tc_fence_before();
      arrive(&ctl.sbrdy);        // CB's elected thread issues Dq from the bf16 copy
      if (n >= 1) {
        // Chunk n-1 has left the consumer: its K,Q tile, A_qk tile and scalars are free.  Its last product, Do, was issued
        // behind the state update and reads the A_qk tile: it has its own barrier, and by now (a state pass later) the
        // wait costs nothing, whereas at the top of the iteration it would sit on the chain.
        wait_bar(((n - 1) & 1) ? &ctl.bar2b : &ctl.bar2, ((n - 1) >> 1) & 1);
        arrive(&ctl.empty[(n - 1) % 3]);
      }
      group_sync128(3);
      // ---- (3) V_new^T = U^T - S^T W^T --------------------------------------------------------------------
      if (gt == 0) {
        wait_bar(&ctl.wrdy, n & 1);          // W tile written by CB
        wait_bar(&ctl.barUW, n & 1);         // U^T complete
        tc::tc_fence_after();
        const uint64_t wd0 = tc::smem_desc(aW, A_RBS, 128);   // W MN-major: 16 key rows per step
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          tc::mma_ts(tbase + TM_DU + 64 * s, tbase + TM_SB + ks * 8, desc_adv(wd0, ks * 2 * A_RBS), id_n64_bmn_neg, 1);
        tc::mma_commit(tc::smem_u32(&ctl.bar1));
      }
      wait_bar(&ctl.bar1, ph1); ph1 ^= 1;
      tc::tc_fence_after();
      // ---- V_new^T -> bf16 (plain, and decayed by e^{G_L - G_c}) ---------------------------------------------
#pragma unroll 1
      for (int c0 = 0; c0 < kC; c0 += 16) {
        uint32_t r[16], pa[8], pb[8];
        tc::tmem_ld16(tbase + TM_DU + 64 * s + lane_addr + c0, r);
        tc::tc_wait_ld();
#pragma unroll
        for (int j4 = 0; j4 < 4; ++j4) {
          const float4 w4 = *reinterpret_cast<const float4*>(sWd + c0 + 4 * j4);
          const float x0 = __uint_as_float(r[4 * j4]), x1 = __uint_as_float(r[4 * j4 + 1]);
          const float x2 = __uint_as_float(r[4 * j4 + 2]), x3 = __uint_as_float(r[4 * j4 + 3]);
          pa[2 * j4] = tc::pack_bf16(x0, x1);
          pa[2 * j4 + 1] = tc::pack_bf16(x2, x3);
          pb[2 * j4] = tc::pack_bf16(x0 * w4.x, x1 * w4.y);
          pb[2 * j4 + 1] = tc::pack_bf16(x2 * w4.z, x3 * w4.w);
        }
        tc::tmem_st8(tbase + TM_VA + lane_addr + c0 / 2, pa);
        tc::tmem_st8(tbase + TM_VB + lane_addr + c0 / 2, pb);
      }
      tc::tc_wait_st();
      tc::tc_fence_before();
      group_sync128(3);
      // ---- (5) S^T += (decayed V_new^T) K^ ;  (4) Do = V_new^T A_qk^T -------------------------------------------
      if (gt == 0) {
        tc::tc_fence_after();
        const uint64_t kd0 = tc::smem_desc(aQK, RBS, 128);  // K^ MN-major
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          tc::mma_ts(tbase + TM_S, tbase + TM_VB + ks * 8, desc_adv(kd0, ks * 2 * RBS), id_n128_bmn, 1);
        tc::mma_commit(tc::smem_u32(&ctl.bar2s));
        const uint64_t ad0 = tc::smem_desc(aAqk, 128, A_RBS);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          tc::mma_ts(tbase + TM_DU + 64 * s, tbase + TM_VA + ks * 8, desc_adv(ad0, ks * 256), id_n64, ks > 0);
        tc::mma_commit(tc::smem_u32((n & 1) ? &ctl.bar2b : &ctl.bar2));
      }
    }
    // final state: hT[k][v] = S^T[v][k]
    wait_bar(&ctl.bar2s, (nchunks - 1) & 1);
    tc::tc_fence_after();
    if (p.hT) {
      float* hT = p.hT + (int64_t)unit * kD * kD;
#pragma unroll 1
      for (int cc = 0; cc < 4; ++cc) {
        const int c0 = 32 * cc;
        uint32_t r[32];
        tc::tmem_ld32(tbase + TM_S + lane_addr + c0, r);
        tc::tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (in_bounds(p.status, (hT - p.hT) + (c0 + j) * kD + gt, p.n_state)) hT[(c0 + j) * kD + gt] = __uint_as_float(r[j]);
      }
    }
    wait_bar(((nchunks - 1) & 1) ? &ctl.bar2b : &ctl.bar2, ((nchunks - 1) >> 1) & 1);   // every product has completed before tensor memory is released
  } else {
    // =========================== CB: q norms, W tile, U^T, output, Dq ==================================
    const __nv_bfloat16* gv = reinterpret_cast<const __nv_bfloat16*>(p.v);
    __nv_bfloat16* go = reinterpret_cast<__nv_bfloat16*>(p.o);
    uint8_t* sV = smem + SM_V;
    // The group's three products per chunk are issued by threads of three different warps (a product blocks its issuing
    // thread for 330-540 cycles, and the warps meet again at the group's next barrier): W^T by thread 0, U^T and the V
    // copy by thread 32, Dq by thread 64.  Each commits to its own barrier.
    constexpr int kUThread = 32, kDqThread = 64;
    // V rows of chunk m -> core-matrix tile
    auto issue_v = [&](int m) {
      if (kTma) {
        if (gt == kUThread) {
          const uint32_t bar = tc::smem_u32(&ctl.vb);
          tc::mbar_arrive_expect_tx(bar, 64u * 256);
          tc::tma_load_5d(tc::smem_u32(sV), &P.tv, 0, 0, vc2, m * 8, vc4, bar);
        }
      } else {
        const int t0m = m * kC, rowsm = min(kC, T - t0m);
        const int rin = gt & 7, kb = gt >> 3;
#pragma unroll 2
        for (int rb = 0; rb < 8; ++rb) {
          const int r = rb * 8 + rin;
          const bool live = r < rowsm;
          const __nv_bfloat16* src = gv + vo_base + (int64_t)(t0m + (live ? r : 0)) * vo_tok + kb * 8;
          tc::cp_async16(tc::smem_u32(sV + tc::core_off(r, kb * 8, RBS)), src, live);
        }
        tc::cp_async_commit();
        tc::cp_async_wait_all();
        tc::fence_async_smem();
        arrive(&ctl.vb);
      }
    };
    // Dq = S^T Q^T of chunk m (elected thread): the bf16 state copy of chunk m is ready and the Dq columns
    // have been read by the output epilogue of chunk m-1
    auto issue_dq = [&](int m) {
      wait_bar(&ctl.sbrdy, m & 1);
      tc::tc_fence_after();
      const uint64_t qd0 = tc::smem_desc(tc::smem_u32(smem + SM_QKR + (m % kRing) * QK_TILE) + 8 * RBS, 128, RBS);   // rows 64..127
#pragma unroll 1
      for (int ks = 0; ks < 8; ++ks)
        tc::mma_ts(tbase + TM_DQ, tbase + TM_SB + ks * 8, desc_adv(qd0, ks * 256), id_n64, ks > 0);
      tc::mma_commit(tc::smem_u32(&ctl.barDq));
    };
    // O^T of chunk m: rq_i (e^{G_i} Dq + Do), straight from the accumulators to global memory.  Each thread owns
    // one value column v and 64 tokens; neighbouring lanes swap halves of token pairs so that every lane stores
    // two adjacent columns of one token (a warp writes 64 contiguous bytes of each of two token rows per
    // instruction).  `next` >= 0: Dq of that chunk is issued as soon as every thread has read the Dq columns.
    auto out_epilogue = [&](int m, int next) {
      const int sm_ = m & 1;
      const float* sEGm = ctl.keep[m % 3];        // rq_i e^{G_i}
      const float* sRQm = ctl.keep[m % 3] + 64;   // rq_i
      const int t0m = m * kC;
      const int rowsm = min(kC, T - t0m);
      const bool odd = gt & 1;
      __nv_bfloat16* orow = go ? go + vo_base + (int64_t)(t0m + (odd ? 1 : 0)) * vo_tok + (gt & ~1) : nullptr;
#pragma unroll 1
      for (int c0 = 0; c0 < kC; c0 += 16) {
        uint32_t rq[16], ro[16];
        tc::tmem_ld16(tbase + TM_DQ + lane_addr + c0, rq);
        tc::tmem_ld16(tbase + TM_DU + 64 * sm_ + lane_addr + c0, ro);
        tc::tc_wait_ld();
        if (c0 == kC - 16) {
          tc::tc_fence_before();
          group_sync128(4);      // Dq and this stage's accumulator are in registers, in every thread
          if (next >= 0 && gt == kDqThread) issue_dq(next);
        }
        if (go) {
          // phases kept apart by hand: 8 packed pairs, then 8 exchanges, then 8 stores
          uint32_t mine[8], other[8];
#pragma unroll
          for (int j4 = 0; j4 < 4; ++j4) {
            const float4 e4 = *reinterpret_cast<const float4*>(sEGm + c0 + 4 * j4);
            const float4 q4 = *reinterpret_cast<const float4*>(sRQm + c0 + 4 * j4);
            mine[2 * j4] = tc::pack_bf16(e4.x * __uint_as_float(rq[4 * j4]) + q4.x * __uint_as_float(ro[4 * j4]),
                                         e4.y * __uint_as_float(rq[4 * j4 + 1]) + q4.y * __uint_as_float(ro[4 * j4 + 1]));
            mine[2 * j4 + 1] = tc::pack_bf16(e4.z * __uint_as_float(rq[4 * j4 + 2]) + q4.z * __uint_as_float(ro[4 * j4 + 2]),
                                             e4.w * __uint_as_float(rq[4 * j4 + 3]) + q4.w * __uint_as_float(ro[4 * j4 + 3]));
          }
#pragma unroll
          for (int e = 0; e < 8; ++e) other[e] = __shfl_xor_sync(0xffffffffu, mine[e], 1);
          __nv_bfloat16* op = orow + (int64_t)c0 * vo_tok;
          const int64_t step = 2 * vo_tok;
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            // even lane: token 2e, columns (v, v+1); odd lane: token 2e+1, columns (v-1, v)
            const uint32_t word = odd ? __byte_perm(other[e], mine[e], 0x7632) : __byte_perm(mine[e], other[e], 0x5410);
            if (c0 + 2 * e + (odd ? 1 : 0) < rowsm && in_bounds(p.status, (op - go) + 1, p.n_v))
              *reinterpret_cast<uint32_t*>(op) = word;
            op += step;
          }
        }
      }
    };

    issue_v(0);
    for (int n = 0; n < nchunks; ++n) {
      const int s = n & 1;
      const uint32_t aQK = tc::smem_u32(smem + SM_QKR + (n % kRing) * QK_TILE);
      uint8_t* sWt = smem + SM_W;
      const uint32_t aXB = tc::smem_u32(reinterpret_cast<uint8_t*>(sAkk0 + s * (64 * LDT)));   // Tb, Tw of this chunk
      wait_bar(&ctl.full[n % 3], (n / 3) & 1);
      tc::tc_fence_after();
      // ---- (2a) W^T = K^T Tw^T -> this stage's accumulator, idle until U^T is issued into it ---------------
      if (gt == 0) {
        const uint64_t kd0 = tc::smem_desc(aQK, RBS, 128);   // K MN-major, 16 chunk rows per step
        const uint64_t twd0 = tc::smem_desc(aXB + XB_TW, 128, A_RBS);
#pragma unroll 1
        for (int ks = 0; ks < 4; ++ks)
          tc::mma_ss(tbase + TM_DU + 64 * s, desc_adv(kd0, ks * 2 * RBS), desc_adv(twd0, ks * 256), id_n64_amn, ks > 0);
        tc::mma_commit(tc::smem_u32(&ctl.barW));
      }
      // the scalars this chunk's output epilogue will need, kept where PA cannot overwrite them
      if (gt < 64) {
        const float rqi = ctl.rq[n % 4][gt];
        ctl.keep[n % 3][gt] = ctl.sc[n % 4][gt] * rqi;
        ctl.keep[n % 3][64 + gt] = rqi;
      }
      wait_bar(&ctl.barW, n & 1);
      if (n >= 1) wait_bar(&ctl.bar1, (n - 1) & 1);   // product (3) of the previous chunk has read the W tile
      tc::tc_fence_after();
      // ---- W^T[k][c] (lane = k) -> bf16 tile, key rows x chunk rows in core-matrix order (MN-major B of (3)) ---
#pragma unroll 1
      for (int c0 = 0; c0 < kC; c0 += 16) {
        uint32_t r[16];
        tc::tmem_ld16(tbase + TM_DU + 64 * s + lane_addr + c0, r);
        tc::tc_wait_ld();
#pragma unroll
        for (int cb = 0; cb < 2; ++cb) {
          uint4 out;
          out.x = tc::pack_bf16(__uint_as_float(r[8 * cb + 0]), __uint_as_float(r[8 * cb + 1]));
          out.y = tc::pack_bf16(__uint_as_float(r[8 * cb + 2]), __uint_as_float(r[8 * cb + 3]));
          out.z = tc::pack_bf16(__uint_as_float(r[8 * cb + 4]), __uint_as_float(r[8 * cb + 5]));
          out.w = tc::pack_bf16(__uint_as_float(r[8 * cb + 6]), __uint_as_float(r[8 * cb + 7]));
          *reinterpret_cast<uint4*>(sWt + tc::core_off(gt, c0 + 8 * cb, A_RBS)) = out;
        }
      }
      tc::fence_async_smem();
      tc::tc_fence_before();
      arrive(&ctl.wrdy);
      group_sync128(4);   // W^T has left the accumulator in every thread; the kept scalars are visible
      // ---- (2b) U^T = V^T Tb^T -> the same accumulator ---------------------------------------------------
      if (gt == kUThread) {
        tc::tc_fence_after();
        wait_bar(&ctl.vb, n & 1);
        tc::tc_fence_after();
        const uint64_t vd0 = tc::smem_desc(tc::smem_u32(sV), RBS, 128);
        const uint64_t tbd0 = tc::smem_desc(aXB + XB_TB, 128, A_RBS);
#pragma unroll 1
        for (int ks = 0; ks < 4; ++ks)
          tc::mma_ss(tbase + TM_DU + 64 * s, desc_adv(vd0, ks * 2 * RBS), desc_adv(tbd0, ks * 256), id_n64_amn, ks > 0);
        tc::mma_commit(tc::smem_u32(&ctl.barUW));
        wait_bar(&ctl.barUW, n & 1);   // V, Tb, Tw have been read: release the X buffer, fetch the next chunk's V rows
        arrive(&ctl.xfree[s]);
      }
      if (n + 1 < nchunks) {
        if (!kTma) wait_bar(&ctl.barUW, n & 1);   // every thread copies V rows
        issue_v(n + 1);
      }
      // ---- output of the previous chunk, then Dq of this one ---------------------------------------------
      if (n >= 1) {
        // Do and Dq of chunk n-1 are complete.  Do alternates between two barriers (even / odd chunks): the chain can
        // commit chunk n's Do before this group gets here (it only needs the W tile, released above), and a parity wait
        // on one barrier could not tell that phase from the one before chunk n-1's and would never return.  It cannot
        // commit chunk n+1's: that needs the next W tile, which this group writes after this wait.
        wait_bar(((n - 1) & 1) ? &ctl.bar2b : &ctl.bar2, ((n - 1) >> 1) & 1);
        wait_bar(&ctl.barDq, (n - 1) & 1);
        tc::tc_fence_after();
        out_epilogue(n - 1, n);
      } else if (gt == kDqThread) {
        issue_dq(0);
      }
    }
    wait_bar(((nchunks - 1) & 1) ? &ctl.bar2b : &ctl.bar2, ((nchunks - 1) >> 1) & 1);
    wait_bar(&ctl.barDq, (nchunks - 1) & 1);
    tc::tc_fence_after();
    out_epilogue(nchunks - 1, -1);
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tbase, TM_COLS);
}

inline cudaError_t launch_chunk(const FwdParams& p, cudaStream_t stream) {
  // TMA inputs need whole 8-row blocks; otherwise the per-thread cp.async instantiation loads the tiles
  // (same layout, same results).
  Sm100Params P;
  memset(&P, 0, sizeof(P));
  P.p = p;
  const bool bthd = p.map.bthd != 0;
  const bool tma_in = p.map.T % 8 == 0 && make_input_map(&P.tk, p.k, p.map.B, p.map.Hq, p.map.T, bthd) &&
                      make_input_map(&P.tq, p.q, p.map.B, p.map.Hq, p.map.T, bthd) &&
                      make_input_map(&P.tv, p.v, p.map.B, p.map.H, p.map.T, bthd);
  auto kern = tma_in ? chunk_sm100_kernel<true> : chunk_sm100_kernel<false>;
  thread_local int attr_dev[2] = {-1, -1};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (attr_dev[tma_in] != dev) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_TOTAL);
    if (e != cudaSuccess) return e;
    attr_dev[tma_in] = dev;
  }
  const dim3 grid((unsigned)((int64_t)p.map.B * p.map.H)), block(kThreads);
  kern<<<grid, block, SM_TOTAL, stream>>>(P);
  return cudaGetLastError();
}

}  // namespace sm100
}  // namespace dr
