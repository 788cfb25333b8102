// Parameter blocks and launchers of the token-recurrent scans (kernels: dr_linrec.cuh, dr_recurrent.cuh, compiled
// in their own translation unit, dr_scans.cu, so that the library's units build side by side).
#pragma once

#include "dr_common.cuh"

namespace dr {

enum { LR_DPLR = 0, LR_RWKV6 = 1, LR_SSD = 2 };

// One per-token vector (or scalar) of a tensor with unit feature stride.
struct LrVec {
  const void* p;
  int64_t sb, sh, st;  // element strides over batch, head, token
  int dt;              // DrDtype
  int hdiv;            // head h reads row h / hdiv (grouped B and C of the SSD)
  int64_t n;           // elements in the array (index checks of the debug build)
  __device__ __forceinline__ int64_t at(int b, int h, int t) const {
    return (int64_t)b * sb + (int64_t)(h / hdiv) * sh + (int64_t)t * st;
  }
};

struct LinRecParams {
  LrVec q, k, w, a, b;  // key axis: query / key / log decay / the two low-rank vectors
  LrVec v;              // value axis
  LrVec dt;             // SSD: one scalar per token and head
  void* o;              // output, addressed like v with its own strides
  int64_t o_sb, o_sh, o_st;
  int o_dt;
  const float* u;        // RWKV-6 bonus [H, K]
  const float* A;        // SSD [H]
  const float* D;        // SSD [H]
  const float* dt_bias;  // SSD [H] or null
  const float* h0;       // null: zero state
  float* hT;             // null: not wanted (may alias h0: every thread reads its entries before it writes them)
  int64_t s_k, s_v;      // state entry (key kk, value vv) of unit n at n*K*V + kk*s_k + vv*s_v
  int32_t* status;       // device status word or null
  int64_t n_o, n_state;  // elements of o and of each state array
  int B, H, T, K, V;
  float scale, dt_lo, dt_hi;
};

// io_bf16: the storage type of q, k, w, a, b, v (one type for all of them); dt of the SSD is float32
cudaError_t launch_linrec(int kind, bool io_bf16, const LinRecParams& p, cudaStream_t stream);
// DeltaNet / Gated DeltaNet / KDA token recurrence (p.variant), any K <= 256
cudaError_t launch_recurrent(const FwdParams& p, cudaStream_t stream);

}  // namespace dr
