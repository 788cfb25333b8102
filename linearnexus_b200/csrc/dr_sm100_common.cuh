// Pieces shared by the tcgen05 kernels (fused chunk forward, two-kernel forward, backward pre-pass):
// tile geometry, the blocked 64x64 unit-lower-triangular inverse on mma.sync tf32, and the TMA tensor
// maps (encoded once per distinct tensor and kept in a small host-side cache).
#pragma once

#include <cuda.h>

#include <cstring>
#include <mutex>

#include "dr_common.cuh"
#include "dr_tcgen05.cuh"

namespace dr {
namespace sm100 {

constexpr int kC = 64, kD = 128;
constexpr int RBS = 16 * 128;    // row-block stride (bytes) of the 128-column bf16 core-matrix tiles
constexpr int A_RBS = 8 * 128;   // row-block stride of the 64-column tiles
constexpr int LDT = 68;          // row stride (floats) of the fp32 64x64 matrices
constexpr uint32_t kWaitLimit = 4u << 20;

__device__ __forceinline__ void group_sync(int id) { asm volatile("bar.sync %0, 256;" ::"r"(id) : "memory"); }
__device__ __forceinline__ void group_sync128(int id) { asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// The rest of a wait whose first try_wait came back empty, kept out of line (the kernel's speed follows its code size).
// Bounded; when the bound runs out every later wait of the CTA returns at once (abort flag), DR_DEV_TIMEOUT is set, and
// the first such wait of the launch leaves its place in bits 8..15 of the status word (bits 8..13: the barrier's number
// in the control block, 63 for one behind the float arrays; bits 14..15: the warp group).
__device__ __noinline__ void wait_more(uint32_t bar, uint32_t parity, int32_t* status, int* abort_flag, uint32_t bar_offset,
                                       uint32_t grp) {
  volatile int* ab = abort_flag;
  if (*ab) return;
  if (tc::mbar_wait_slow(bar, parity, kWaitLimit)) return;
  *ab = 1;
  if (!status) return;
  const uint32_t num = bar_offset / 8u < 63u ? bar_offset / 8u : 63u;
  atomicCAS(status, 0, DR_DEV_TIMEOUT | (int)((num | (grp << 6)) << 8));
  atomicOr(status, DR_DEV_TIMEOUT);
}

// Test kernel of the record above: one thread waits, with this very routine and its full bound (about a second of SM
// clock), on an mbarrier that nothing arrives on.  The status word gets DR_DEV_TIMEOUT and the site given here; a second
// wait of the same CTA returns at once (abort flag) and leaves the record alone.  The kernel returns normally.
__global__ void wait_site_kernel(int32_t* status, uint32_t barrier_number, uint32_t grp) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    tc::mbar_init(tc::smem_u32(&bar), 1);
    tc::fence_mbar_init();
    if (!tc::mbar_try(tc::smem_u32(&bar), 0)) wait_more(tc::smem_u32(&bar), 0, status, &abort_flag, barrier_number * 8u, grp);
    if (!tc::mbar_try(tc::smem_u32(&bar), 0)) wait_more(tc::smem_u32(&bar), 0, status, &abort_flag, 0u, 0u);
  }
}

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

// ||x_r||^2 for 64 rows of a bf16 core-matrix tile (rows row0 .. row0+63, 128 columns, row-block stride RBS) on
// the warp-level tensor cores: warp w of a four-warp group takes rows 16w .. 16w+15, forms their 16x16 Gram
// block with mma.sync m16n8k16 (the A fragments double as the B fragments) and keeps the diagonal.  A core
// matrix (8 rows x 16 bytes, 128 contiguous bytes) is exactly one ldmatrix 8x8 matrix.
// out(r, value) is called once per row by the lane that holds its diagonal entry.
template <class Out>
__device__ __forceinline__ void row_sq_norms_64(const uint8_t* tile, int row0, int w, int lane, Out out) {
  const int mi = lane >> 3, rin = lane & 7;
  const uint32_t base = tc::smem_u32(tile) + (uint32_t)(((row0 >> 3) + 2 * w + (mi & 1)) * RBS + (mi >> 1) * 128 + rin * 16);
  float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    uint32_t a[4];
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3])
                 : "r"(base + ks * 256));
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d0[0]), "+f"(d0[1]), "+f"(d0[2]), "+f"(d0[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(a[0]), "r"(a[2]));
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d1[0]), "+f"(d1[1]), "+f"(d1[2]), "+f"(d1[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(a[1]), "r"(a[3]));
  }
  const int g = lane >> 2, t = lane & 3;
  if (t == (g >> 1)) {   // this lane holds entries (g, g) of the first and (g+8, g+8) of the second product
    out(16 * w + g, (g & 1) ? d0[1] : d0[0]);
    out(16 * w + 8 + g, (g & 1) ? d1[3] : d1[2]);
  }
}

// ---------------------------------------------------------------------------------------------------
// T = (I + diag(rs) A)^-1 for a strictly lower-triangular 64x64 A (fp32, row stride LDT).
// 8x8 diagonal blocks by forward substitution on the CUDA cores, then three merge levels
// (block size 8, 16, 32):  T_10 = -T_11 (diag(rs) A_10) T_00, each of the two products on the
// warp-level tensor-core path (mma.sync m16n8k8, tf32 operands, fp32 accumulate): these tiny
// products are bound by shared-memory wavefronts, not flops, on the CUDA cores.
// sT receives the lower triangle of T; entries above the diagonal are scratch (callers mask them).
// sA and sT may be the SAME array: every block of A is consumed before the block of T that takes
// its place is written.
// ---------------------------------------------------------------------------------------------------
struct SyncGroup256 { __device__ __forceinline__ void operator()() const { group_sync(1); } };

// One merge level on NW warps (w = index of the calling warp inside its group).
template <int BS, int NW, class Sync>
__device__ __forceinline__ void inverse_merge_level(const float* __restrict__ sA, const float* __restrict__ rs,
                                                    float* __restrict__ sT, int w, int lane, Sync sync) {
  constexpr int MT = BS >= 16 ? BS / 16 : 1, NT = BS / 8, KS = BS / 8;
  constexpr int TPP = MT * NT, NPAIR = 32 / BS, TILES = NPAIR * TPP;
  const int g = lane >> 2, t = lane & 3;
  // step 1: X = diag(rs) A_10 T_00   -> scratch at the mirrored block (rows c0.., columns r0..)
#pragma unroll
  for (int tile = w; tile < TILES; tile += NW) {
    const int pr = tile / TPP, rem = tile % TPP;
    const int mt = rem / NT, nt = rem % NT;
    const int r0 = 2 * BS * pr + BS, c0 = 2 * BS * pr;   // block row / column origin of this pair
    const int m0 = mt * 16 + g, m1 = m0 + 8;              // rows of this lane inside the block
    const int n0 = nt * 8;
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
#pragma unroll
  for (int tile = w; tile < TILES; tile += NW) {
    const int pr = tile / TPP, rem = tile % TPP;
    const int mt = rem / NT, nt = rem % NT;
    const int r0 = 2 * BS * pr + BS, c0 = 2 * BS * pr;
    const int m0 = mt * 16 + g, m1 = m0 + 8;
    const int n0 = nt * 8;
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

// 8x8 diagonal blocks: one thread per column of each block (threads 0..63 of the group, i.e. two full
// warps).  All entries of A's block are read before the first entry of T is written (in-place use).
__device__ __forceinline__ void inverse_diag_blocks(const float* __restrict__ sA, const float* __restrict__ rs,
                                                    float* __restrict__ sT, int gt) {
  if (gt < 64) {
    const int o = (gt >> 3) * 8, c = gt & 7;
    float a[8][8];
#pragma unroll
    for (int i = 1; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < i; ++j) a[i][j] = sA[(o + i) * LDT + o + j];
    float f[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = rs[o + i];
    __syncwarp();
    float x[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < i; ++j) acc += a[i][j] * x[j];
      x[i] = ((i == c) ? 1.f : 0.f) - f[i] * acc;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) sT[(o + i) * LDT + o + c] = x[i];
  }
}

// The inverse on a group of 256 threads synchronised by named barrier 1.
__device__ __forceinline__ void block_inverse_64(const float* __restrict__ sA, const float* __restrict__ rs,
                                                 float* __restrict__ sT, int gt) {
  const int warp8 = gt >> 5, lane = gt & 31;
  inverse_diag_blocks(sA, rs, sT, gt);
  group_sync(1);
  inverse_merge_level<8, 8>(sA, rs, sT, warp8, lane, SyncGroup256());
  inverse_merge_level<16, 8>(sA, rs, sT, warp8, lane, SyncGroup256());
  inverse_merge_level<32, 8>(sA, rs, sT, warp8, lane, SyncGroup256());
}

// The inverse IN PLACE (sT holds A on entry, T on return) on a group of 128 threads synchronised by `sync`.
template <class Sync>
__device__ __forceinline__ void block_inverse_64_inplace(float* __restrict__ sT, const float* __restrict__ rs, int gt,
                                                         Sync sync) {
  const int w = gt >> 5, lane = gt & 31;
  inverse_diag_blocks(sT, rs, sT, gt);
  sync();
  inverse_merge_level<8, 4>(sT, rs, sT, w, lane, sync);
  inverse_merge_level<16, 4>(sT, rs, sT, w, lane, sync);
  inverse_merge_level<32, 4>(sT, rs, sT, w, lane, sync);
}

// ---------------------------------------------------------------------------------------------------
// TMA tensor maps.  cuTensorMapEncodeTiled is fetched from the driver at run time (no link dependency
// on libcuda).  Encoded maps are kept in a small cache keyed by (pointer, geometry): a serving or
// training loop calls with the same buffers over and over.
// ---------------------------------------------------------------------------------------------------
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

struct MapKey {
  const void* base;
  int64_t a, b, c;   // geometry (meaning depends on kind)
  int kind;          // 0: [units][T][128] input, 1: [B][T][heads][128] input, 2: output
  bool operator==(const MapKey& o) const { return base == o.base && a == o.a && b == o.b && c == o.c && kind == o.kind; }
};
struct MapCache {
  static constexpr int kSlots = 32;
  std::mutex mu;
  MapKey key[kSlots];
  CUtensorMap map[kSlots];
  int used = 0, next = 0;
  bool find(const MapKey& k, CUtensorMap* out) {
    std::lock_guard<std::mutex> lock(mu);
    for (int i = 0; i < used; ++i)
      if (key[i] == k) { *out = map[i]; return true; }
    return false;
  }
  void put(const MapKey& k, const CUtensorMap& m) {
    std::lock_guard<std::mutex> lock(mu);
    const int i = used < kSlots ? used++ : (next++ % kSlots);
    key[i] = k; map[i] = m;
  }
};
inline MapCache& map_cache() { static MapCache c; return c; }

// 5-d input view whose box {8,8,16,8,1} lands one 64x128 bf16 chunk in shared memory already in the
// 8x8 core-matrix order the tensor cores read (needs T % 8 == 0).
//   [B*heads, T, 128] storage ([B,H,T,D]): dims {8 elems, 8 rows, 16 column blocks, T/8 row blocks, B*heads};
//     the chunk m of sequence u is at coordinates (0, 0, 0, 8m, u).
//   [B, T, heads, 128] storage ([B,T,H,D]): dims {8 elems, 8 rows (stride heads*256 B), 16*heads column
//     blocks, T/8 row blocks, B}; the chunk m of (b, h) is at coordinates (0, 0, 16h, 8m, b).
// The maps cover this GPU's memory only and are used without multicast.
inline bool make_input_map(CUtensorMap* m, const void* base, int64_t B, int64_t heads, int T, bool bthd) {
  const MapKey key{base, B, heads, T, bthd ? 1 : 0};
  if (map_cache().find(key, m)) return true;
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  cuuint64_t dims[5], strides[4];
  if (bthd) {
    dims[0] = 8; dims[1] = 8; dims[2] = 16 * (cuuint64_t)heads; dims[3] = (cuuint64_t)(T / 8); dims[4] = (cuuint64_t)B;
    strides[0] = (cuuint64_t)heads * 256; strides[1] = 16; strides[2] = 8 * (cuuint64_t)heads * 256;
    strides[3] = (cuuint64_t)T * heads * 256;
  } else {
    dims[0] = 8; dims[1] = 8; dims[2] = 16; dims[3] = (cuuint64_t)(T / 8); dims[4] = (cuuint64_t)(B * heads);
    strides[0] = 256; strides[1] = 16; strides[2] = 2048; strides[3] = (cuuint64_t)T * 256;
  }
  const cuuint32_t box[5] = {8, 8, 16, 8, 1};
  const cuuint32_t es[5] = {1, 1, 1, 1, 1};
  if (fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(base), dims, strides, box, es,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  map_cache().put(key, *m);
  return true;
}
// the [B*heads][T][128] form with the units already flattened
inline bool make_input_map(CUtensorMap* m, const void* base, int64_t units, int T) {
  return make_input_map(m, base, units, 1, T, false);
}

// 4-d output view {128, T, H, B} of [B,H,T,128] or [B,T,H,128], bf16 (elem_bytes 2) or fp32 (4); one box
// {128,64,1,1} stores a chunk's rows and clips the ragged tail.
inline bool make_output_map(CUtensorMap* m, void* base, const SeqMap& sm, int elem_bytes = 2) {
  const MapKey key{base, ((int64_t)sm.B << 32) | (uint32_t)sm.H, sm.T, (sm.bthd ? 1 : 0) | (elem_bytes << 1), 2};
  if (map_cache().find(key, m)) return true;
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t row = 128ull * elem_bytes;
  const cuuint64_t dims[4] = {128, (cuuint64_t)sm.T, (cuuint64_t)sm.H, (cuuint64_t)sm.B};
  cuuint64_t strides[3];
  if (sm.bthd) { strides[0] = (cuuint64_t)sm.H * row; strides[1] = row; strides[2] = (cuuint64_t)sm.T * sm.H * row; }
  else { strides[0] = row; strides[1] = (cuuint64_t)sm.T * row; strides[2] = (cuuint64_t)sm.H * sm.T * row; }
  const cuuint32_t box[4] = {128, 64, 1, 1};
  const cuuint32_t es[4] = {1, 1, 1, 1};
  if (fn(m, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, base, dims,
         strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  map_cache().put(key, *m);
  return true;
}

}  // namespace sm100
}  // namespace dr
