// Chunkwise gated delta-rule forward on the Blackwell tensor cores (tcgen05 + TMEM).
//
// Shape: K = V = 128, chunk C = 64, bf16 q/k/v/o, fp32 g/beta/state.  One CTA of 512 threads
// owns one (batch, head) sequence.  The fp32 state lives TRANSPOSED in tensor memory for the
// whole sequence (S^T: lane = value column v, column = key row k), so every product has
// M = 128 and each epilogue thread owns one value column.
//
// Two groups of eight warps run as a two-stage pipeline over the chunks of the sequence (two
// warps share each 32-lane quarter of tensor memory and split the columns of every epilogue):
//
//   PRODUCER (warps 0-7): everything that does not depend on the state.
//     Raw K,Q rows of a chunk land by TMA as one [K;Q] tile already in core-matrix order, two chunks
//     ahead (3-deep ring).  The l2 norms are not applied to the tiles: they are folded into row and
//     column factors (rk from the diagonal of (1), rq from the raw Q rows).
//     (1) D1 = [K;Q] K^T                             128x64x128  smem x smem, issued one chunk ahead
//         X = D1[i][j] e^{G_i-G_j} (i>j, fp32);  A_qk = D1[64+i][j] e^{G_i-G_j} (i>=j) -> bf16 tile
//         T = (I + diag(beta rk^2) X)^-1: 8x8 blocks by substitution, three merge levels on mma.sync tf32;
//         the first two levels occupy warps 0-3 while warps 4-7 issue (1) of the next chunk, scan its
//         decay and take the query norms
//         -> Tb = T diag(beta rk), Tw = T diag(beta e^G rk^2)   bf16 tiles
//   CONSUMER (warps 8-15): the serial chain over the state.
//     (2) U^T = V^T Tb^T  -> TMEM (stage accumulator)  128x64x64   smem(MN-major) x smem
//         W^T = K^T Tw^T  -> idle TMEM columns -> bf16 tile W      smem(MN-major) x smem
//         (issued the moment the chunk is handed over; the next chunk's V rows are fetched when they complete)
//         bf16 copy of S^T for the products; fp32 S^T pre-multiplied by e^{G_L}
//     (3) V_new^T = U^T - S^T W^T  (accumulated onto U^T with negate-A)                    128x64x128
//         Dq = S^T Q^T                                                                     128x64x128
//     (4) Do = V_new^T A_qk^T                                                              128x64x64
//     (5) S^T += (V_new^T e^{G_L-G_c}) K   (K read MN-major)                                128x128x64
//         O^T[v][i] = rq_i e^{G_i} Dq[v][i] + rq_i Do[v][i], written one chunk late so that it overlaps (3)
//
// The [K;Q] tile is stored once as 8x8 core matrices and serves as A and B of (1), MN-major
// A of (2), K-major B of (3) and MN-major B of (5).  Every wait on an mbarrier is bounded; a
// wait that runs out sets DR_DEV_TIMEOUT in the status word and the kernel finishes without
// further waiting.
#pragma once

#include <cuda.h>

#include <cstring>

#include "dr_common.cuh"
#include "dr_tcgen05.cuh"
#include "dr_umma_selftest.cuh"

namespace dr {
namespace sm100 {

constexpr bool kAvailable = true;
constexpr int kThreads = 512;
constexpr int kGroup = 256;
constexpr int kC = 64, kD = 128;

// tensor-memory columns (32-bit x 128 lanes each): 512 in total
constexpr uint32_t TM_S = 0;      // S^T fp32                                   128
constexpr uint32_t TM_SB = 128;   // bf16 copy of S^T (A operand)                 64
constexpr uint32_t TM_D1 = 192;   // producer scratch: D1, then W^T               64
constexpr uint32_t TM_DU = 256;   // 2 stages x 64: U^T -> V_new^T -> Do          128
constexpr uint32_t TM_DQ = 384;   // S^T Q^^T                                     64
constexpr uint32_t TM_VA = 448;   // V_new^T bf16                                 32
constexpr uint32_t TM_VB = 480;   // decayed V_new^T bf16                         32
constexpr uint32_t TM_COLS = 512;

// shared-memory map (bytes).  Per stage (two stages):
constexpr int RBS = 16 * 128;                 // row-block stride of the 128-column core-matrix tiles
constexpr int A_RBS = 8 * 128;                // row-block stride of the 64-column tiles
constexpr int QK_TILE = 128 * 128 * 2;        // [K (64 rows); Q (64 rows)] x 128 raw bf16, 32 KB
constexpr int SM_QKR = 0;                     // ring of 3 such tiles (chunk n uses tile n % 3)
constexpr int SM_STAGE = 3 * QK_TILE;         // two stages follow
constexpr int W_KBS = 144;                    // k-block stride of the W tile (padded: conflict-free 2-byte stores)
constexpr int W_RBS = 16 * W_KBS;             // its row-block stride
constexpr int ST_W = 0;                       // W [64][128] (18 KB padded); reused as the O staging tile
constexpr int ST_AQK = ST_W + 8 * W_RBS;       // A_qk [64][64]                           8 KB
constexpr int ST_SC = ST_AQK + 64 * 64 * 2;   // G, e^G, e^{G_L-G}, beta: 4 x 64 floats  1 KB
constexpr int STAGE_BYTES = ST_SC + 4 * 64 * 4;
// Producer-private:
constexpr int SM_V = SM_STAGE + 2 * STAGE_BYTES;  // V [64][128] core-matrix tile       16 KB
constexpr int SM_TB = SM_V + 64 * 128 * 2;    // T diag(beta)        [64][64] bf16
constexpr int SM_TW = SM_TB + 64 * 64 * 2;    // T diag(beta e^G)    [64][64] bf16
constexpr int LDT = 68;                       // row stride (floats) of the fp32 64x64 matrices
constexpr int SM_AKK = SM_TW + 64 * 64 * 2;   // A_kk fp32 [64][68]
constexpr int SM_T32 = SM_AKK + 64 * LDT * 4; // T fp32 [64][68]
constexpr int SM_TOTAL = SM_T32 + 64 * LDT * 4;

// Optional per-phase cycle counters (CTA 0 only), compiled in with -DDR_PROFILE.
#ifdef DR_PROFILE
__device__ unsigned long long g_prof[192];
#define PROF_DECL unsigned long long prof_t0 = clock64(); unsigned long long wt0 = 0; (void)wt0;
#define PROF(idx)                                              \
  do {                                                         \
    if (blockIdx.x == 0 && gt == 0) {                          \
      const unsigned long long prof_t = clock64();             \
      atomicAdd(&g_prof[idx], prof_t - prof_t0);               \
      prof_t0 = prof_t;                                        \
    }                                                          \
  } while (0)
#define WSTART wt0 = clock64()
#define WEND(idx)                                                                   \
  do {                                                                              \
    if (blockIdx.x == 0 && lane == 0) atomicAdd(&g_prof[48 + idx * 8 + (warp & 7)], clock64() - wt0); \
  } while (0)
#define IPROF_DECL unsigned long long ip0 = clock64();
#define IPROF(idx)                                                                           \
  do {                                                                                       \
    if (blockIdx.x == 0 && gt == 0) { const unsigned long long t_ = clock64(); atomicAdd(&g_prof[idx], t_ - ip0); ip0 = t_; } \
  } while (0)
#else
#define IPROF_DECL
#define IPROF(idx)
#define PROF_DECL
#define PROF(idx)
#define WSTART
#define WEND(idx)
#endif

struct Ctl {
  uint64_t full[2], empty[2], barP, barUW, uwfree, bar1, bar2, kq[3], vb;
  float gb[3][128];      // raw beta (0..63) and g (64..127) of chunk m in slot m % 3
  float sc[3][256];      // G, e^G, e^{G_L-G}, beta (64 each) of chunk m in slot m % 3
  float eg_keep[2][64];  // rq_i e^{G_i} of the chunk whose output epilogue is still pending, per stage
  float rq_keep[2][64];  // rq_i of that chunk
  float rq[2][64];       // per stage: scale / (||q_i|| + eps)           (producer -> consumer)
  float rk[64];          // 1 / (||k_j|| + eps)                           (producer-private)
  float rs[64];          // beta_i rk_i^2: row factor of the unit-lower system
  uint32_t tmem_base;
  int abort;
};

__device__ __forceinline__ void group_sync(int id) { asm volatile("bar.sync %0, 256;" ::"r"(id) : "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// T = (I + diag(rs) A)^-1 for a strictly lower-triangular 64x64 A (fp32, row stride LDT).
// 8x8 diagonal blocks by forward substitution on the CUDA cores, then three merge levels
// (block size 8, 16, 32):  T_10 = -T_11 (diag(rs) A_10) T_00, each of the two products on the
// warp-level tensor-core path (mma.sync m16n8k8, tf32 operands, fp32 accumulate) because these
// tiny products are bound by shared-memory wavefronts, not flops, on the CUDA cores.
// sT receives the lower triangle of T; entries above the diagonal are scratch (callers mask them).
__device__ __forceinline__ uint32_t to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

struct SyncGroup256 { __device__ __forceinline__ void operator()() const { group_sync(1); } };
// the first four warps of a group only (barrier 3): the 8- and 16-wide merge levels have work for four warps
struct SyncHalf128 { __device__ __forceinline__ void operator()() const { asm volatile("bar.sync 3, 128;" ::: "memory"); } };

template <int BS, class Sync>
__device__ __forceinline__ void inverse_merge_level(const float* __restrict__ sA, const float* __restrict__ rs,
                                                    float* __restrict__ sT, int warp8, int lane, Sync sync) {
  constexpr int MT = BS >= 16 ? BS / 16 : 1, NT = BS / 8, KS = BS / 8;
  constexpr int TPP = MT * NT, NPAIR = 32 / BS, TILES = NPAIR * TPP;
  const int g = lane >> 2, t = lane & 3;
  const bool work = warp8 < TILES;
  const int pr = work ? warp8 / TPP : 0, rem = warp8 % TPP;
  const int mt = rem / NT, nt = rem % NT;
  const int r0 = 2 * BS * pr + BS, c0 = 2 * BS * pr;   // block row / column origin of this pair
  const int m0 = mt * 16 + g, m1 = m0 + 8;              // rows of this lane inside the block
  const int n0 = nt * 8;
  // step 1: X = diag(rs) A_10 T_00   -> scratch at the mirrored block (rows c0.., columns r0..)
  if (work) {
    float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int k0 = ks * 8 + t, k1 = k0 + 4;
      uint32_t a[4], b[2];
      a[0] = to_tf32(m0 < BS ? sA[(r0 + m0) * LDT + c0 + k0] : 0.f);
      a[1] = to_tf32(m1 < BS ? sA[(r0 + m1) * LDT + c0 + k0] : 0.f);
      a[2] = to_tf32(m0 < BS ? sA[(r0 + m0) * LDT + c0 + k1] : 0.f);
      a[3] = to_tf32(m1 < BS ? sA[(r0 + m1) * LDT + c0 + k1] : 0.f);
      const int n = n0 + g;                              // T_00 is lower triangular: entry (k, n) needs n <= k
      b[0] = to_tf32(n <= k0 ? sT[(c0 + k0) * LDT + c0 + n] : 0.f);
      b[1] = to_tf32(n <= k1 ? sT[(c0 + k1) * LDT + c0 + n] : 0.f);
      mma_tf32(d, a, b);
    }
    if (m0 < BS) {
      const float f = rs[r0 + m0];
      *reinterpret_cast<float2*>(sT + (c0 + m0) * LDT + r0 + n0 + 2 * t) = make_float2(f * d[0], f * d[1]);
    }
    if (m1 < BS) {
      const float f = rs[r0 + m1];
      *reinterpret_cast<float2*>(sT + (c0 + m1) * LDT + r0 + n0 + 2 * t) = make_float2(f * d[2], f * d[3]);
    }
  }
  sync();
  // step 2: T_10 = -T_11 X
  if (work) {
    float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int k0 = ks * 8 + t, k1 = k0 + 4;
      uint32_t a[4], b[2];
      // T_11 is lower triangular: entry (m, k) needs k <= m
      a[0] = to_tf32((m0 < BS && k0 <= m0) ? sT[(r0 + m0) * LDT + r0 + k0] : 0.f);
      a[1] = to_tf32((m1 < BS && k0 <= m1) ? sT[(r0 + m1) * LDT + r0 + k0] : 0.f);
      a[2] = to_tf32((m0 < BS && k1 <= m0) ? sT[(r0 + m0) * LDT + r0 + k1] : 0.f);
      a[3] = to_tf32((m1 < BS && k1 <= m1) ? sT[(r0 + m1) * LDT + r0 + k1] : 0.f);
      b[0] = to_tf32(sT[(c0 + k0) * LDT + r0 + n0 + g]);
      b[1] = to_tf32(sT[(c0 + k1) * LDT + r0 + n0 + g]);
      mma_tf32(d, a, b);
    }
    if (m0 < BS) *reinterpret_cast<float2*>(sT + (r0 + m0) * LDT + c0 + n0 + 2 * t) = make_float2(-d[0], -d[1]);
    if (m1 < BS) *reinterpret_cast<float2*>(sT + (r0 + m1) * LDT + c0 + n0 + 2 * t) = make_float2(-d[2], -d[3]);
  }
  sync();
}

__device__ __forceinline__ void block_inverse_64(const float* __restrict__ sA, const float* __restrict__ rs,
                                                 float* __restrict__ sT, int gt) {
  const int warp8 = gt >> 5, lane = gt & 31;
  // 8x8 diagonal blocks: one thread per column of each block
  if (gt < 64) {
    const int o = (gt >> 3) * 8, c = gt & 7;
    float x[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < i; ++j) acc += sA[(o + i) * LDT + o + j] * x[j];
      x[i] = ((i == c) ? 1.f : 0.f) - rs[o + i] * acc;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) sT[(o + i) * LDT + o + c] = x[i];
  }
  group_sync(1);
  inverse_merge_level<8>(sA, rs, sT, warp8, lane, SyncGroup256());
  inverse_merge_level<16>(sA, rs, sT, warp8, lane, SyncGroup256());
  inverse_merge_level<32>(sA, rs, sT, warp8, lane, SyncGroup256());
}

// The same inverse with the group split for its first part: warps 0-3 run the diagonal blocks and the 8- and
// 16-wide merge levels (which have work for four warps only) while warps 4-7 run `side()`; all eight warps
// join for the 32-wide level.  Every thread of the group must call it.
template <class Side>
__device__ __forceinline__ void block_inverse_64_split(const float* __restrict__ sA, const float* __restrict__ rs,
                                                       float* __restrict__ sT, int gt, Side side) {
  const int warp8 = gt >> 5, lane = gt & 31;
  if (gt < 128) {
    if (gt < 64) {
      const int o = (gt >> 3) * 8, c = gt & 7;
      float x[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < i; ++j) acc += sA[(o + i) * LDT + o + j] * x[j];
        x[i] = ((i == c) ? 1.f : 0.f) - rs[o + i] * acc;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) sT[(o + i) * LDT + o + c] = x[i];
    }
    SyncHalf128()();
    inverse_merge_level<8>(sA, rs, sT, warp8, lane, SyncHalf128());
    inverse_merge_level<16>(sA, rs, sT, warp8, lane, SyncHalf128());
  } else {
    side();
  }
  group_sync(1);
  inverse_merge_level<32>(sA, rs, sT, warp8, lane, SyncGroup256());
}

// Kernel parameters: the common forward parameters plus the TMA tensor maps.
//   tk, tq, tv : 5-d views {8 elements, 8 rows, 16 k-blocks, T/8 row blocks, B*H} of the [B,H,T,128] bf16
//                inputs; one box {8,8,16,8,1} lands a 64x128 chunk in shared memory already in the
//                8x8 core-matrix order the tensor cores read (used when use_tma_in).
//   to         : 4-d view {128, T, H, B} of the output; one box {128,64,1,1} stores a chunk's rows and
//                clips the ragged tail (used when use_tma_out).
struct alignas(64) Sm100Params {
  CUtensorMap tk, tq, tv, to;
  FwdParams p;
  int use_tma_in, use_tma_out;
};

__global__ void __launch_bounds__(kThreads, 1) chunk_sm100_kernel(const __grid_constant__ Sm100Params P) {
  const FwdParams& p = P.p;
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ __align__(8) Ctl ctl;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gt = tid & (kGroup - 1);     // thread index inside its group of eight warps
  const int hs = gt >> 7;                // which of the two warps sharing a tensor-memory lane quarter
  const int l128 = gt & 127;             // tensor-memory lane owned by this thread
  const bool producer = tid < kGroup;
  const int T = p.map.T;
  const int unit = blockIdx.x;
  const int b = unit / p.map.H, h = unit % p.map.H;
  const int64_t qk_base = p.map.base_qk(b, h, kD), qk_tok = p.map.tok_qk(kD);   // q, k (possibly fewer heads)
  const int64_t vo_base = p.map.base(b, h, kD), vo_tok = p.map.tok(kD);         // v, o
  const int unit_qk = b * p.map.Hq + p.map.hq(h);
  const int64_t s_base = p.map.base(b, h, 1), s_tok = p.map.tok(1);

  if (warp == 0) {
    tc::tmem_alloc(tc::smem_u32(&ctl.tmem_base), TM_COLS);
    tc::tmem_relinquish();
  }
  if (tid == 0) {
    tc::mbar_init(tc::smem_u32(&ctl.full[0]), kGroup);
    tc::mbar_init(tc::smem_u32(&ctl.full[1]), kGroup);
    tc::mbar_init(tc::smem_u32(&ctl.empty[0]), kGroup);
    tc::mbar_init(tc::smem_u32(&ctl.empty[1]), kGroup);
    tc::mbar_init(tc::smem_u32(&ctl.barUW), 1);
    tc::mbar_init(tc::smem_u32(&ctl.uwfree), 1);
    tc::mbar_init(tc::smem_u32(&ctl.barP), 1);
    tc::mbar_init(tc::smem_u32(&ctl.bar1), 1);
    tc::mbar_init(tc::smem_u32(&ctl.bar2), 1);
    tc::mbar_init(tc::smem_u32(&ctl.kq[0]), 1);
    tc::mbar_init(tc::smem_u32(&ctl.kq[1]), 1);
    tc::mbar_init(tc::smem_u32(&ctl.kq[2]), 1);
    tc::mbar_init(tc::smem_u32(&ctl.vb), 1);
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
      if (!tc::mbar_wait_bounded(tc::smem_u32(bar), parity, kWaitLimit)) {
        *abort_p = 1;
        if (p.status) atomicOr(p.status, DR_DEV_TIMEOUT);
      }
    }
  };

  // Long waits (a whole group idling until the other group hands a stage over) back off with
  // nanosleep between polls so that the waiting warps leave the issue slots and the shared-memory
  // pipe to the working group.
  auto wait_bar_relaxed = [&](uint64_t* bar, uint32_t parity) {
    if (!*abort_p) {
      if (!tc::mbar_wait_sleepy(tc::smem_u32(bar), parity)) {
        *abort_p = 1;
        if (p.status) atomicOr(p.status, DR_DEV_TIMEOUT);
      }
    }
  };

  const uint32_t id_n64 = tc::idesc_bf16(128, 64, 0, 0);
  const uint32_t id_n64_amn = tc::idesc_bf16(128, 64, 1, 0);
  const uint32_t id_n64_neg = id_n64 | (1u << 13);
  const uint32_t id_n128_bmn = tc::idesc_bf16(128, 128, 0, 1);
  const int nchunks = (T + kC - 1) / kC;

  if (producer) {
    // =========================== PRODUCER ===========================================================
    const __nv_bfloat16* gq = reinterpret_cast<const __nv_bfloat16*>(p.q);
    const __nv_bfloat16* gk = reinterpret_cast<const __nv_bfloat16*>(p.k);
    const __nv_bfloat16* gv = reinterpret_cast<const __nv_bfloat16*>(p.v);
    const float* gg = reinterpret_cast<const float*>(p.g);
    uint8_t* sV = smem + SM_V;
    uint8_t* sTb = smem + SM_TB;
    uint8_t* sTw = smem + SM_TW;
    float* sAkk = reinterpret_cast<float*>(smem + SM_AKK);
    float* sT32 = reinterpret_cast<float*>(smem + SM_T32);
    uint32_t phP = 0;

    // K,Q rows (raw bf16), g and beta of chunk m -> tile / scalars of stage m&1, 16-byte (4-byte)
    // cp.async per thread; thread -> (row in block, k-block).  The l2 normalisation is NOT applied
    // to the tiles: it is folded into the epilogue factors rk, rs, rq.
    auto issue_kq = [&](int m) {
      const int t0m = m * kC, rowsm = min(kC, T - t0m);
      uint8_t* dQK = smem + SM_QKR + (m % 3) * QK_TILE;
      float* dG = ctl.gb[m % 3];
      if (P.use_tma_in) {
        if (gt == 64) {  // a warp other than the one that issues the products
          const uint32_t bar = tc::smem_u32(&ctl.kq[m % 3]);
          tc::mbar_arrive_expect_tx(bar, 2u * 64 * 256);
          tc::tma_load_5d(tc::smem_u32(dQK), &P.tk, 0, 0, 0, m * 8, unit_qk, bar);
          tc::tma_load_5d(tc::smem_u32(dQK) + 64 * 256, &P.tq, 0, 0, 0, m * 8, unit_qk, bar);
        }
      } else {
        const int rin = gt & 7, kb = (gt >> 3) & 15, rbh = gt >> 7;
#pragma unroll
        for (int rb2 = 0; rb2 < 4; ++rb2) {
          const int r = (2 * rb2 + rbh) * 8 + rin;
          const bool live = r < rowsm;
          const int64_t off = qk_base + (int64_t)(t0m + (live ? r : 0)) * qk_tok + kb * 8;
          tc::cp_async16(tc::smem_u32(dQK + tc::core_off(r, kb * 8, RBS)), gk + off, live);
          tc::cp_async16(tc::smem_u32(dQK + tc::core_off(64 + r, kb * 8, RBS)), gq + off, live);
        }
      }
      if (gt >= 128) {
        const int r = gt & 63;
        const bool live = r < rowsm;
        const int64_t off = s_base + (int64_t)(t0m + (live ? r : 0)) * s_tok;
        if (gt < 192) tc::cp_async4(tc::smem_u32(dG + r), p.beta + off, live);                     // beta
        else tc::cp_async4(tc::smem_u32(dG + 64 + r), gg ? gg + off : p.beta + off, live && gg);  // g (0 without decay)
      }
      tc::cp_async_commit();
    };
    // V rows of chunk m -> core-matrix tile
    // (with TMA only chunk 0 is fetched here; the consumer fetches V of chunk m+1 the moment its U^T product
    // of chunk m has completed)
    auto issue_v = [&](int m) {
      const int t0m = m * kC, rowsm = min(kC, T - t0m);
      if (P.use_tma_in) {
        if (gt == 64) {
          const uint32_t bar = tc::smem_u32(&ctl.vb);
          tc::mbar_arrive_expect_tx(bar, 64u * 256);
          tc::tma_load_5d(tc::smem_u32(sV), &P.tv, 0, 0, 0, m * 8, unit, bar);
        }
      } else {
        const int rin = gt & 7, kb = (gt >> 3) & 15, rbh = gt >> 7;
#pragma unroll
        for (int rb2 = 0; rb2 < 4; ++rb2) {
          const int r = (2 * rb2 + rbh) * 8 + rin;
          const bool live = r < rowsm;
          const __nv_bfloat16* src = gv + vo_base + (int64_t)(t0m + (live ? r : 0)) * vo_tok + kb * 8;
          tc::cp_async16(tc::smem_u32(sV + tc::core_off(r, kb * 8, RBS)), src, live);
        }
      }
      tc::cp_async_commit();
    };

    // inclusive scan of the log decay over the 64 rows of a stage (one warp): G, e^G, e^{G_L - G}
    auto scan_stage = [&](int m) {
      float* zG = ctl.sc[m % 3];
      const float* raw = ctl.gb[m % 3];
      zG[192 + lane] = raw[lane]; zG[224 + lane] = raw[32 + lane];   // beta
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
      zG[lane] = a; zG[lane + 32] = bq;
      zG[64 + lane] = __expf(a); zG[96 + lane] = __expf(bq);
      zG[128 + lane] = __expf(fminf(last - a, 0.f)); zG[160 + lane] = __expf(fminf(last - bq, 0.f));
    };

    // first product of chunk m: D1 = [K;Q] K^T on the raw rows (B = first 64 rows of the same tile)
    auto issue_d1 = [&](int m) {
      if (P.use_tma_in) wait_bar(&ctl.kq[m % 3], (m / 3) & 1);
      tc::tc_fence_after();
      const uint32_t aQK = tc::smem_u32(smem + SM_QKR + (m % 3) * QK_TILE);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint64_t ad = tc::smem_desc(aQK + ks * 256, 128, RBS);
        tc::mma_ss(tbase + TM_D1, ad, ad, id_n64, ks > 0);
      }
      tc::mma_commit(tc::smem_u32(&ctl.barP));
    };

    if (nchunks > 0) {
      issue_kq(0);
      issue_v(0);
      tc::cp_async_wait_all();
      if (!P.use_tma_in) tc::fence_async_smem();
      group_sync(1);
      if (warp == 1) scan_stage(0);
      if (gt == 0) issue_d1(0);
    }
    PROF_DECL
    for (int n = 0; n < nchunks; ++n) {
      const int s = n & 1;
      uint8_t* st = smem + SM_STAGE + s * STAGE_BYTES;
      uint8_t* sAqk = st + ST_AQK;
      const uint8_t* sQKp = smem + SM_QKR + (n % 3) * QK_TILE;
      const float* sG = ctl.sc[n % 3];
      const float* sEG = sG + 64;
      const float* sBeta = sG + 192;
      group_sync(1);  // the scalars of this chunk (scan) are visible
      PROF(0);
      // the consumer has finished chunk n-2, so tile (n+1) % 3 and stage s are free: fetch the next chunk's
      // K,Q (and beta, g) a whole iteration before their first use
      // (every thread waits: the first epilogue below overwrites the stage's A_qk tile)
      if (n >= 2) wait_bar(&ctl.empty[s], ((n >> 1) - 1) & 1);
      if (n + 1 < nchunks) issue_kq(n + 1);
      PROF(2);
      // ---- D1 of this chunk was issued during the previous iteration ----------------------------------------
      wait_bar(&ctl.barP, phP); phP ^= 1;
      tc::tc_fence_after();
      PROF(3);
      WSTART;
      {
        const int i = l128 & 63, c0 = 32 * hs;
        const float Gi = sG[i];
        uint32_t r[32];
        tc::tmem_ld32(tbase + TM_D1 + lane_addr + c0, r);
        tc::tc_wait_ld();
        if (l128 < 64) {
          // X = (K K^T) . E on the raw rows, strictly lower; the row factor beta_i rk_i^2 and the column
          // factors rk_j are applied later (rs in the solve, rk in the Tb/Tw tiles)
          if ((i >> 5) == hs) {  // this half holds the diagonal entry ||k_i||^2
            float d = 0.f;
#pragma unroll
            for (int j = 0; j < 32; ++j) d = (c0 + j == i) ? __uint_as_float(r[j]) : d;
            const float rk = p.l2norm ? 1.f / (sqrtf(d) + 1e-6f) : 1.f;
            ctl.rk[i] = rk;
            ctl.rs[i] = sBeta[i] * rk * rk;
          }
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            float4 o4;
            float* o = reinterpret_cast<float*>(&o4);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int jj = c0 + 4 * j4 + e;
              const float x = __uint_as_float(r[4 * j4 + e]) * __expf(fminf(Gi - sG[jj], 0.f));
              o[e] = jj < i ? x : 0.f;
            }
            *reinterpret_cast<float4*>(sAkk + i * LDT + c0 + 4 * j4) = o4;
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
      WEND(1);
      tc::cp_async_wait_all();   // the next chunk's beta, g (and, without TMA, its K,Q rows) have landed
      if (!P.use_tma_in) tc::fence_async_smem();
      tc::tc_fence_before();
      group_sync(1);
      PROF(4);
      // ---- T'' = (I + diag(rs) X)^-1 on warps 0-3 (+ all eight for the last level).  Meanwhile warps 4-7:
      //      D1 of the NEXT chunk (its scratch columns are free now, so it completes behind the inverse), the
      //      decay scan of the next chunk, and this chunk's query norms for the consumer -----------------------
      WSTART;
      block_inverse_64_split(sAkk, ctl.rs, sT32, gt, [&]() {
        if (n + 1 < nchunks) {
          if (gt == 128) issue_d1(n + 1);
          if (warp == 5) scan_stage(n + 1);
        }
        if (gt >= 192) {  // rq_i = scale / (||q_i|| + eps) from the raw rows 64..127 of the tile, one thread per row
          const int row = gt - 192;
          float ss = 0.f;
#pragma unroll
          for (int it = 0; it < 16; ++it) {
            const uint4 c = *reinterpret_cast<const uint4*>(sQKp + tc::core_off(64 + row, it * 8, RBS));
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&c);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = __bfloat1622float2(h2[e]);
              ss += f.x * f.x + f.y * f.y;
            }
          }
          ctl.rq[s][row] = p.l2norm ? p.scale / (sqrtf(ss) + 1e-6f) : p.scale;
        }
      });
      WEND(5);
      PROF(1);
      WSTART;
      // the consumer's U^T, W^T products of the previous chunk have read Tb, Tw (and V)
      if (n >= 1) wait_bar(&ctl.uwfree, (n - 1) & 1);
      if (!P.use_tma_in && n >= 1) issue_v(n);   // (with TMA the consumer fetched it)
      {
        const int rin = gt & 7, jb = (gt >> 3) & 7, rbq = gt >> 6;
        float bj[8], bw[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float rkj = ctl.rk[8 * jb + e];
          bj[e] = sBeta[8 * jb + e] * rkj;
          bw[e] = bj[e] * sEG[8 * jb + e] * rkj;
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int i = 8 * (4 * j + rbq) + rin;
          const float4 t0v = *reinterpret_cast<const float4*>(sT32 + i * LDT + 8 * jb);
          const float4 t1v = *reinterpret_cast<const float4*>(sT32 + i * LDT + 8 * jb + 4);
          float t[8] = {t0v.x, t0v.y, t0v.z, t0v.w, t1v.x, t1v.y, t1v.z, t1v.w};
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
      WEND(6);
      if (!P.use_tma_in) tc::cp_async_wait_all();   // this chunk's V rows
      tc::fence_async_smem();
      mbar_arrive(tc::smem_u32(&ctl.full[s]));   // A_qk, Tb, Tw, the scalars (and V) of chunk n are ready
      PROF(5);
    }
  } else {
    // =========================== CONSUMER ===========================================================
    __nv_bfloat16* go = reinterpret_cast<__nv_bfloat16*>(p.o);
    uint32_t ph1 = 0, ph2 = 0;
    // initial state: S^T[v][k] = h0[k][v] (thread = value column v, half of the key columns)
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
    // O^T of chunk m: e^{G_i} Dq + Do -> staging tile (the stage's W region, no longer needed)
    // -> coalesced store; then releases stage m&1 to the producer.
    auto final_epilogue = [&](int m) {
      const int sm_ = m & 1;
      uint8_t* stm = smem + SM_STAGE + sm_ * STAGE_BYTES;
      const float* sEGm = ctl.eg_keep[sm_];   // rq_i e^{G_i}
      const float* sRQm = ctl.rq_keep[sm_];   // rq_i = scale / (||q_i|| + eps)
      __nv_bfloat16* sO = reinterpret_cast<__nv_bfloat16*>(stm + ST_W);
      const int t0m = m * kC;
      const int rowsm = min(kC, T - t0m);
      {
        const int c0 = 32 * hs;
        uint32_t rq[32], ro[32];
        tc::tmem_ld32(tbase + TM_DQ + lane_addr + c0, rq);
        tc::tmem_ld32(tbase + TM_DU + 64 * sm_ + lane_addr + c0, ro);
        tc::tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int i = c0 + j;
          sO[i * kD + l128] = __float2bfloat16_rn(sEGm[i] * __uint_as_float(rq[j]) + sRQm[i] * __uint_as_float(ro[j]));
        }
      }
      tc::tc_fence_before();
      if (!p.o) {
        group_sync(2);  // output not wanted (checkpoint-only forward of the backward)
      } else if (P.use_tma_out) {
        tc::fence_async_smem();
        group_sync(2);
        if (gt == 0) {  // one tiled store of the whole chunk; rows past T are clipped by the tensor map
          tc::tma_store_4d(&P.to, tc::smem_u32(sO), 0, t0m, h, b);
          tc::bulk_commit();   // its shared-memory reads are awaited before the tile is written again
        }
      } else {
        group_sync(2);
        const int r = gt >> 2, qtr = gt & 3;
        if (r < rowsm) {
          __nv_bfloat16* dst = go + vo_base + (int64_t)(t0m + r) * vo_tok + 32 * qtr;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            reinterpret_cast<uint4*>(dst)[j] = reinterpret_cast<const uint4*>(sO + r * kD + 32 * qtr)[j];
        }
      }
    };

    PROF_DECL
    for (int n = 0; n < nchunks; ++n) {
      const int s = n & 1;
      uint8_t* st = smem + SM_STAGE + s * STAGE_BYTES;
      const uint8_t* sQKc = smem + SM_QKR + (n % 3) * QK_TILE;
      const uint32_t aQK = tc::smem_u32(sQKc), aW = tc::smem_u32(st + ST_W), aAqk = tc::smem_u32(st + ST_AQK);
      const float* sEG = ctl.sc[n % 3] + 64;
      const float* sWd = sEG + 64;
      uint8_t* sWt = st + ST_W;
      wait_bar_relaxed(&ctl.full[s], (n >> 1) & 1);
      tc::tc_fence_after();
      PROF(16);
      // ---- (2) W^T = K^T Tw^T -> the (idle) bf16 V_new columns;  U^T = V^T Tb^T -> stage accumulator ----------
      if (gt == 0) {
        // the output store that read this stage's staging tile (chunk n-2) has finished reading it; every
        // other thread learns that through the completion barrier of the products issued next
        if (P.use_tma_out) tc::bulk_wait_read_all();
        if (P.use_tma_in) wait_bar(&ctl.vb, n & 1);
        const uint32_t aV = tc::smem_u32(smem + SM_V), aTb = tc::smem_u32(smem + SM_TB), aTw = tc::smem_u32(smem + SM_TW);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          const uint64_t ad = tc::smem_desc(aQK + ks * 2 * RBS, RBS, 128);   // K MN-major, 16 chunk rows per step
          const uint64_t bd = tc::smem_desc(aTw + ks * 256, 128, A_RBS);
          tc::mma_ss(tbase + TM_VA, ad, bd, id_n64_amn, ks > 0);
        }
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          const uint64_t ad = tc::smem_desc(aV + ks * 2 * RBS, RBS, 128);
          const uint64_t bd = tc::smem_desc(aTb + ks * 256, 128, A_RBS);
          tc::mma_ss(tbase + TM_DU + 64 * s, ad, bd, id_n64_amn, ks > 0);
        }
        tc::mma_commit(tc::smem_u32(&ctl.barUW));
      }
      // ---- state pass: bf16 copy of S^T for the products; fp32 master pre-multiplied by e^{G_L} --------
      {
        const float gl = sEG[63];
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int c0 = 64 * hs + 32 * cc;
          uint32_t r[32], pk[16];
          tc::tmem_ld32(tbase + TM_S + lane_addr + c0, r);
          tc::tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) pk[j] = tc::pack_bf16(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
          if (p.ckpt) {  // state at the start of this chunk, [K][V] row-major, for the backward
            float* ck = p.ckpt + ((int64_t)unit * nchunks + n) * kD * kD;
#pragma unroll
            for (int j = 0; j < 32; ++j) ck[(c0 + j) * kD + l128] = __uint_as_float(r[j]);
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * gl);
          tc::tmem_st16(tbase + TM_SB + lane_addr + c0 / 2, pk);
          tc::tmem_st32(tbase + TM_S + lane_addr + c0, r);
        }
        tc::tc_wait_st();
      }
      PROF(17);
      // ---- W^T[k][c] (lane = k) -> bf16 tile W[c][k] (K-major B operand of (3)) ----------------------------
      wait_bar(&ctl.barUW, n & 1);
      tc::tc_fence_after();
      if (gt == 0) {
        // Tb, Tw and the V tile are free again: tell the producer, and fetch the next chunk's V rows
        mbar_arrive(tc::smem_u32(&ctl.uwfree));
        if (P.use_tma_in && n + 1 < nchunks) {
          const uint32_t bar = tc::smem_u32(&ctl.vb);
          tc::mbar_arrive_expect_tx(bar, 64u * 256);
          tc::tma_load_5d(tc::smem_u32(smem + SM_V), &P.tv, 0, 0, 0, (n + 1) * 8, unit, bar);
        }
      }
      {
        const int c0 = 32 * hs;
        uint32_t r[32];
        tc::tmem_ld32(tbase + TM_VA + lane_addr + c0, r);
        tc::tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j)
          *reinterpret_cast<__nv_bfloat16*>(sWt + ((c0 + j) >> 3) * W_RBS + (l128 >> 3) * W_KBS + ((c0 + j) & 7) * 16 +
                                            (l128 & 7) * 2) = __float2bfloat16_rn(__uint_as_float(r[j]));
      }
      tc::fence_async_smem();
      tc::tc_fence_before();
      group_sync(2);
      PROF(22);
      // ---- (3) V_new^T = U^T - S^T W^T --------------------------------------------------------------------
      if (gt == 0) {
        tc::tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t bd = tc::smem_desc(aW + ks * 2 * W_KBS, W_KBS, W_RBS);
          tc::mma_ts(tbase + TM_DU + 64 * s, tbase + TM_SB + ks * 8, bd, id_n64_neg, 1);
        }
        tc::mma_commit(tc::smem_u32(&ctl.bar1));
      }
      PROF(23);
      if (n > 0) final_epilogue(n - 1);  // overlaps (3); frees Dq and the other stage
      tc::tc_fence_before();
      group_sync(2);
      PROF(18);
      if (gt == 0) {  // Dq = S^T Q^^T   (Q^ = rows 64..127 of the tile)
        tc::tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t bd = tc::smem_desc(aQK + 8 * RBS + ks * 256, 128, RBS);
          tc::mma_ts(tbase + TM_DQ, tbase + TM_SB + ks * 8, bd, id_n64, ks > 0);
        }
      }
      wait_bar(&ctl.bar1, ph1); ph1 ^= 1;
      tc::tc_fence_after();
      PROF(19);
      // ---- V_new^T -> bf16 (plain, and decayed by e^{G_L - G_c}) ---------------------------------------------
      {
        const int c0 = 32 * hs;
        uint32_t r[32], pa[16], pb[16];
        tc::tmem_ld32(tbase + TM_DU + 64 * s + lane_addr + c0, r);
        tc::tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float x0 = __uint_as_float(r[2 * j]), x1 = __uint_as_float(r[2 * j + 1]);
          pa[j] = tc::pack_bf16(x0, x1);
          pb[j] = tc::pack_bf16(x0 * sWd[c0 + 2 * j], x1 * sWd[c0 + 2 * j + 1]);
        }
        tc::tmem_st16(tbase + TM_VA + lane_addr + c0 / 2, pa);
        tc::tmem_st16(tbase + TM_VB + lane_addr + c0 / 2, pb);
      }
      tc::tc_wait_st();
      tc::tc_fence_before();
      group_sync(2);
      PROF(20);
      // ---- (5) S^T += (decayed V_new^T) K^ ;  (4) Do = V_new^T A_qk^T -------------------------------------------
      if (gt == 0) {
        tc::tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          const uint64_t bd = tc::smem_desc(aQK + ks * 2 * RBS, RBS, 128);  // K^ MN-major
          tc::mma_ts(tbase + TM_S, tbase + TM_VB + ks * 8, bd, id_n128_bmn, 1);
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
      // every product that reads this stage's tiles is complete: hand [K^;Q^], A_qk and the scalars
      // back to the producer now; the accumulator and the W region follow after the output epilogue
      if (gt < 64) {
        const float rqi = ctl.rq[s][gt];
        ctl.eg_keep[s][gt] = sEG[gt] * rqi;
        ctl.rq_keep[s][gt] = rqi;
      }
      mbar_arrive(tc::smem_u32(&ctl.empty[s]));
      PROF(21);
    }
    group_sync(2);  // eg_keep of the last chunk is visible to the whole group
    if (nchunks > 0) final_epilogue(nchunks - 1);
    if (P.use_tma_out && gt == 0) tc::bulk_wait_all();
    // final state: hT[k][v] = S^T[v][k]
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

// cuTensorMapEncodeTiled is fetched from the driver at run time (no link dependency on libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      ptr = nullptr;
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

// 5-d input view of a contiguous [B*H][T][128] bf16 tensor (see Sm100Params).
inline bool make_input_map(CUtensorMap* m, const void* base, int64_t units, int T) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t dims[5] = {8, 8, 16, (cuuint64_t)(T / 8), (cuuint64_t)units};
  const cuuint64_t strides[4] = {256, 16, 2048, (cuuint64_t)T * 256};  // bytes, dims 1..4
  const cuuint32_t box[5] = {8, 8, 16, 8, 1};
  const cuuint32_t es[5] = {1, 1, 1, 1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(base), dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 4-d output view {128, T, H, B} of [B,H,T,128] or [B,T,H,128], bf16 (elem_bytes 2) or fp32 (4).
inline bool make_output_map(CUtensorMap* m, void* base, const SeqMap& sm, int elem_bytes = 2) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t row = 128ull * elem_bytes;
  const cuuint64_t dims[4] = {128, (cuuint64_t)sm.T, (cuuint64_t)sm.H, (cuuint64_t)sm.B};
  cuuint64_t strides[3];
  if (sm.bthd) { strides[0] = (cuuint64_t)sm.H * row; strides[1] = row; strides[2] = (cuuint64_t)sm.T * sm.H * row; }
  else { strides[0] = row; strides[1] = (cuuint64_t)sm.T * row; strides[2] = (cuuint64_t)sm.H * sm.T * row; }
  const cuuint32_t box[4] = {128, 64, 1, 1};
  const cuuint32_t es[4] = {1, 1, 1, 1};
  return fn(m, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, base, dims,
            strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

inline cudaError_t launch_chunk(const FwdParams& p, cudaStream_t stream) {
  cudaError_t e = cudaFuncSetAttribute(chunk_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_TOTAL);
  if (e != cudaSuccess) return e;
  Sm100Params P;
  memset(&P, 0, sizeof(P));
  P.p = p;
  const int64_t units = (int64_t)p.map.B * p.map.H;
  // TMA inputs need the rows of one (batch, head) contiguous and whole 8-row blocks; otherwise the
  // per-thread cp.async path loads the tiles (same layout, same results).
  const int64_t units_qk = (int64_t)p.map.B * p.map.Hq;
  P.use_tma_in = !p.map.bthd && p.map.T % 8 == 0 && make_input_map(&P.tk, p.k, units_qk, p.map.T) &&
                 make_input_map(&P.tq, p.q, units_qk, p.map.T) && make_input_map(&P.tv, p.v, units, p.map.T);
  P.use_tma_out = p.o != nullptr && make_output_map(&P.to, p.o, p.map);
  const dim3 grid((unsigned)units), block(kThreads);
  chunk_sm100_kernel<<<grid, block, SM_TOTAL, stream>>>(P);
  return cudaGetLastError();
}

}  // namespace sm100
}  // namespace dr
