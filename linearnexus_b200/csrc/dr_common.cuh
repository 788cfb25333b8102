// Shared device/host helpers for the delta-rule kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "deltarule_sm100.h"

namespace dr {

// Addressing of one (batch, head) sequence inside a [B,H,T,D] or [B,T,H,D] tensor.
// Element index of token t, feature d is  base(b,h,D) + t * tok(D) + d.
struct SeqMap {
  int B, H, T;
  int bthd;  // 0: [B,H,T,D]   1: [B,T,H,D]
  int Hq;    // heads of q and k (grouped value attention: head h of v, o reads q/k head h / (H / Hq)); Hq == H: none
  __host__ __device__ inline int64_t base(int b, int h, int D) const {
    return bthd ? ((int64_t)b * T * H + h) * D : ((int64_t)b * H + h) * (int64_t)T * D;
  }
  __host__ __device__ inline int64_t tok(int D) const { return bthd ? (int64_t)H * D : D; }
  // the same for q and k
  __host__ __device__ inline int hq(int h) const { return Hq == H ? h : h / (H / Hq); }
  __host__ __device__ inline int64_t base_qk(int b, int h, int D) const {
    return bthd ? ((int64_t)b * T * Hq + hq(h)) * D : ((int64_t)b * Hq + hq(h)) * (int64_t)T * D;
  }
  __host__ __device__ inline int64_t tok_qk(int D) const { return bthd ? (int64_t)Hq * D : D; }
};

__device__ __forceinline__ float ld_elem(const void* p, int64_t i, int dt) {
  return dt == DR_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i])
                       : reinterpret_cast<const float*>(p)[i];
}

__device__ __forceinline__ void st_elem(void* p, int64_t i, int dt, float x) {
  if (dt == DR_BF16)
    reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(x);
  else
    reinterpret_cast<float*>(p)[i] = x;
}

// Index checks of the debug build (-DDR_BOUNDS_CHECK, linearnexus_b200/libdeltarule_sm100_bounds.so): the kernels that
// index global memory by hand ask in_bounds() before an access; an index outside [0, n) sets DR_DEV_BOUNDS in the
// status word and the access is skipped -- never a trap, never a fault.  The release build compiles the checks away.
#ifdef DR_BOUNDS_CHECK
__device__ __forceinline__ bool in_bounds(int32_t* status, int64_t i, int64_t n) {
  if (i >= 0 && i < n) return true;
  if (status) atomicOr(status, DR_DEV_BOUNDS);
  return false;
}
#else
__device__ __forceinline__ bool in_bounds(int32_t*, int64_t, int64_t) { return true; }
#endif

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

// Parameters every forward kernel takes (plain struct passed by value).
struct FwdParams {
  const void* q;
  const void* k;
  const void* v;
  const void* g;      // null for DR_DELTA
  const float* beta;
  const float* h0;    // null: zero state
  void* o;
  float* hT;          // null: not wanted
  int32_t* status;    // device status word or null
  float* ckpt;        // null, or [B*H][N][K][V]: state at the start of every chunk (backward)
  SeqMap map;
  int K, V, C;
  int variant, qkv_dt, g_dt, out_dt, l2norm;
  float scale;
  // element counts of the caller's arrays (what the index checks of the debug build compare against)
  int64_t n_qk, n_v, n_gk, n_tok, n_state, n_ckpt;
  __host__ void set_extents() {
    const int64_t bh = (int64_t)map.B * map.H, bhq = (int64_t)map.B * map.Hq;
    n_qk = bhq * map.T * K;
    n_v = bh * map.T * V;
    n_gk = bh * map.T * K;
    n_tok = bh * map.T;
    n_state = bh * K * V;
    n_ckpt = C > 0 ? bh * ((map.T + C - 1) / C) * K * V : 0;
  }
};

}  // namespace dr
