// Self-test of the tcgen05 plumbing: D[128][N] = (+/-)A[128][Kd] * B^T on one CTA, with the operand
// placements the chunk kernel uses (A from shared memory K-major (mode 0), from TMEM (mode 1) or
// from shared memory MN-major (mode 2, source given as [Kd][128]); bit 2 of the mode sets the
// descriptor's negate-A flag; B K-major or MN-major; un-swizzled core-matrix layout).  The GPU
// tests compare D with a float matmul.
#pragma once

#include "dr_common.cuh"
#include "dr_sm100_common.cuh"
#include "dr_tcgen05.cuh"

namespace dr {
namespace sm100 {

__global__ void __launch_bounds__(128) umma_selftest_kernel(const __nv_bfloat16* __restrict__ A,
                                                            const __nv_bfloat16* __restrict__ B,
                                                            float* __restrict__ D, int Kd, int N, int a_tmem,
                                                            int b_mn, int32_t* status) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_base_s;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int neg_a = (a_tmem >> 2) & 1;
  const int M = (a_tmem & 8) ? 64 : 128;  // bit 3: M = 64 (rows land on 16 lanes of each 32-lane quarter)
  a_tmem &= 3;
  const int a_mn = a_tmem == 2;
  uint8_t* sA = smem_raw;
  uint8_t* sB = smem_raw + 128 * 128 * 2;
  const int a_rbs = a_mn ? 16 * 128 : (Kd / 8) * 128;
  const int b_rbs = b_mn ? (N / 8) * 128 : (Kd / 8) * 128;

  if (warp == 0) {
    tc::tmem_alloc(tc::smem_u32(&tmem_base_s), 512);
    tc::tmem_relinquish();
  }
  if (tid == 0) {
    tc::mbar_init(tc::smem_u32(&bar), 1);
    tc::fence_mbar_init();
  }
  // stage A (row m = tid) and B
  if (a_mn) {
    for (int i = tid; i < 128 * Kd; i += 128) {  // source [Kd][128]: rows are k, 16 bytes run along m
      const int kk = i / 128, m = i % 128;
      *reinterpret_cast<__nv_bfloat16*>(sA + tc::core_off(kk, m, a_rbs)) = A[i];
    }
  } else {
    for (int i = tid; i < 128 * Kd; i += 128) {
      const int r = i / Kd, c = i % Kd;
      *reinterpret_cast<__nv_bfloat16*>(sA + tc::core_off(r, c, a_rbs)) = A[i];
    }
  }
  if (b_mn) {
    for (int i = tid; i < Kd * N; i += 128) {  // source [Kd][N]
      const int kk = i / N, n = i % N;
      *reinterpret_cast<__nv_bfloat16*>(sB + tc::core_off(kk, n, b_rbs)) = B[i];
    }
  } else {
    for (int i = tid; i < N * Kd; i += 128) {  // source [N][Kd]
      const int n = i / Kd, kk = i % Kd;
      *reinterpret_cast<__nv_bfloat16*>(sB + tc::core_off(n, kk, b_rbs)) = B[i];
    }
  }
  tc::fence_async_smem();
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tbase = tmem_base_s;
  const uint32_t tD = tbase, tA = tbase + 256;
  const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
  if (a_tmem == 1) {
    for (int c0 = 0; c0 < Kd / 2; c0 += 16) {
      uint32_t r[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int kk = 2 * (c0 + j);
        r[j] = tc::pack_bf16(__bfloat162float(A[tid * Kd + kk]), __bfloat162float(A[tid * Kd + kk + 1]));
      }
      tc::tmem_st16(tA + lane_addr + c0, r);
    }
    tc::tc_wait_st();
  }
  tc::tc_fence_before();
  __syncthreads();
  if (tid == 0) {
    tc::tc_fence_after();
    const uint32_t idesc = tc::idesc_bf16(M, N, a_mn, b_mn) | ((uint32_t)neg_a << 13);
    for (int ks = 0; ks < Kd / 16; ++ks) {
      uint64_t bd;
      if (b_mn)  // MN-major: SBO = 128 (next 8 n), LBO = row-block stride (next 8 k); 16 k per step
        bd = tc::smem_desc(tc::smem_u32(sB) + ks * 2 * b_rbs, b_rbs, 128);
      else       // K-major: LBO = 128 (next 8 k), SBO = row-block stride (next 8 n); 32 bytes of k per step
        bd = tc::smem_desc(tc::smem_u32(sB) + ks * 256, 128, b_rbs);
      if (a_tmem == 1) {
        tc::mma_ts(tD, tA + ks * 8, bd, idesc, ks > 0);
      } else if (a_mn) {
        const uint64_t ad = tc::smem_desc(tc::smem_u32(sA) + ks * 2 * a_rbs, a_rbs, 128);
        tc::mma_ss(tD, ad, bd, idesc, ks > 0);
      } else {
        const uint64_t ad = tc::smem_desc(tc::smem_u32(sA) + ks * 256, 128, a_rbs);
        tc::mma_ss(tD, ad, bd, idesc, ks > 0);
      }
    }
    tc::mma_commit(tc::smem_u32(&bar));
  }
  const bool ok = tc::mbar_wait_bounded(tc::smem_u32(&bar), 0, kWaitLimit);
  if (!ok && status) atomicOr(status, DR_DEV_TIMEOUT);
  tc::tc_fence_after();
  for (int c0 = 0; c0 < N; c0 += 32) {
    uint32_t r[32];
    tc::tmem_ld32(tD + lane_addr + c0, r);
    tc::tc_wait_ld();
    if (M == 128) {
#pragma unroll
      for (int j = 0; j < 32; ++j) D[tid * N + c0 + j] = __uint_as_float(r[j]);
    } else if ((tid & 31) < 16) {  // M = 64: row m sits on lane (m % 16) + 32 * (m / 16)
      const int m = 16 * warp + (tid & 31);
#pragma unroll
      for (int j = 0; j < 32; ++j) D[m * N + c0 + j] = __uint_as_float(r[j]);
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tbase, 512);
}

// One warp waits on an mbarrier that nothing ever arrives on, with the bounded wait the kernels use and a
// small attempt limit: the wait gives up, the status word gets DR_DEV_TIMEOUT, the kernel returns normally.
__global__ void wait_timeout_kernel(int32_t* status, uint32_t attempts) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    tc::mbar_init(tc::smem_u32(&bar), 1);
    tc::fence_mbar_init();
  }
  __syncwarp();
  if (!tc::mbar_wait_bounded(tc::smem_u32(&bar), 0, attempts) && threadIdx.x == 0) atomicOr(status, DR_DEV_TIMEOUT);
}

inline cudaError_t launch_umma_selftest(const void* A, const void* B, float* D, int Kd, int N, int a_tmem,
                                        int b_mn, int32_t* status, cudaStream_t stream) {
  const int smem = 128 * 128 * 2 * 2;
  cudaError_t e = cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  umma_selftest_kernel<<<1, 128, smem, stream>>>(reinterpret_cast<const __nv_bfloat16*>(A),
                                                 reinterpret_cast<const __nv_bfloat16*>(B), D, Kd, N, a_tmem,
                                                 b_mn, status);
  return cudaGetLastError();
}

}  // namespace sm100
}  // namespace dr
