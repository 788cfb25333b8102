// Single-token decode step: one pass over the fp32 state cache, updated in place.
//
// One CTA of 256 threads owns one (batch, head) state S[K][V] (row-major, v contiguous).
// Thread (ks, vg) holds float4 columns 4*vg..4*vg+3 of rows ks, ks+nks, ... in registers,
// so every warp reads and writes whole 128-bit-wide contiguous row segments exactly once.
// The two reductions over k (v_old = S~^T k and S~^T q) are accumulated per thread,
// combined across the ks groups through shared memory, and the rank-one update is applied
// to the registers before the single store:
//     S~ = gamma * S ; d = beta * (v - S~^T k) ; S' = S~ + k d^T ; o = S~^T q + (q.k) d
#pragma once

#include "dr_common.cuh"

namespace dr {

struct StepParams {
  const void* q;
  const void* k;
  const void* v;
  const void* g;
  const float* beta;
  const float* s_in;
  float* s_out;
  void* o;
  int K, V;
  int H, Hq;   // heads of v/o/state and of q/k (grouped value attention when Hq < H)
  int variant, qkv_dt, g_dt, out_dt, l2norm;
  float scale;
  // unit (b * H + h) -> row of q and k
  __host__ __device__ inline int64_t unit_qk(int64_t unit) const {
    if (Hq == H) return unit;
    const int u = (int)unit, b = u / H, h = u - b * H;   // B * H < 2^24: 32-bit arithmetic
    return b * Hq + h / (H / Hq);
  }
};

constexpr int kStepThreads = 256;

template <int ROWS>
__global__ void __launch_bounds__(kStepThreads) step_kernel(const StepParams p) {
  extern __shared__ float smem[];
  const int K = p.K, V = p.V;
  float* s_q = smem;            // [K] normalised, scaled
  float* s_k = s_q + K;         // [K] normalised
  float* s_gam = s_k + K;       // [K] per-row decay (KDA) / broadcast
  float* s_red = s_gam + K;     // [2][nks][V]
  __shared__ float s_part[3][kStepThreads / 32];
  __shared__ float s_scal[3];

  const int tid = threadIdx.x;
  const int64_t unit = blockIdx.x;
  const int nvg = V >> 2;
  const int nks = kStepThreads / nvg > 0 ? kStepThreads / nvg : 1;
  const int vg = tid % nvg;
  const int ks = tid / nvg;
  const bool active = ks < nks && (tid < nvg * nks);

  const float* S_in = p.s_in + unit * (int64_t)K * V;
  float* S_out = p.s_out + unit * (int64_t)K * V;

  // Issue the state loads first: they are the long-latency, bandwidth-carrying part.
  float4 st[ROWS > 0 ? ROWS : 1];
  if (ROWS > 0) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const int kk = ks + r * nks;
      st[r] = (active && kk < K)
                  ? __ldcs(reinterpret_cast<const float4*>(S_in + (int64_t)kk * V) + vg)
                  : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }

  // q, k -> fp32, optional l2 normalisation; q.k after normalisation.
  float qq = 0.f, kq = 0.f, kk2 = 0.f;
  for (int i = tid; i < K; i += kStepThreads) {
    const float qv = ld_elem(p.q, p.unit_qk(unit) * K + i, p.qkv_dt);
    const float kv = ld_elem(p.k, p.unit_qk(unit) * K + i, p.qkv_dt);
    s_q[i] = qv;
    s_k[i] = kv;
    qq += qv * qv;
    kk2 += kv * kv;
    kq += qv * kv;
    float gam = 1.f;
    if (p.variant == DR_KDA) gam = expf(ld_elem(p.g, unit * K + i, p.g_dt));
    s_gam[i] = gam;
  }
  qq = warp_sum(qq);
  kk2 = warp_sum(kk2);
  kq = warp_sum(kq);
  if ((tid & 31) == 0) {
    s_part[0][tid >> 5] = qq;
    s_part[1][tid >> 5] = kk2;
    s_part[2][tid >> 5] = kq;
  }
  __syncthreads();
  if (tid < 3) {
    float a = 0.f;
    for (int w = 0; w < kStepThreads / 32; ++w) a += s_part[tid][w];
    s_scal[tid] = a;
  }
  __syncthreads();
  float qmul = p.scale, kmul = 1.f;
  if (p.l2norm) {
    qmul = p.scale / (sqrtf(s_scal[0]) + 1e-6f);
    kmul = 1.f / (sqrtf(s_scal[1]) + 1e-6f);
  }
  const float qk = s_scal[2] * qmul * kmul;
  const float gscal = (p.variant == DR_GATED) ? expf(ld_elem(p.g, unit, p.g_dt)) : 1.f;
  const float beta = p.beta[unit];

  float4 a_k = make_float4(0.f, 0.f, 0.f, 0.f);  // sum_k S~[k][v] * k[k]
  float4 a_q = make_float4(0.f, 0.f, 0.f, 0.f);  // sum_k S~[k][v] * q[k]
  if (active) {
    if (ROWS > 0) {
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        const int kk = ks + r * nks;
        if (kk < K) {
          const float gm = gscal * s_gam[kk];
          const float kn = s_k[kk] * kmul, qn = s_q[kk] * qmul;
          st[r].x *= gm; st[r].y *= gm; st[r].z *= gm; st[r].w *= gm;
          a_k.x += st[r].x * kn; a_k.y += st[r].y * kn; a_k.z += st[r].z * kn; a_k.w += st[r].w * kn;
          a_q.x += st[r].x * qn; a_q.y += st[r].y * qn; a_q.z += st[r].z * qn; a_q.w += st[r].w * qn;
        }
      }
    } else {
      for (int kk = ks; kk < K; kk += nks) {
        float4 s = reinterpret_cast<const float4*>(S_in + (int64_t)kk * V)[vg];
        const float gm = gscal * s_gam[kk];
        const float kn = s_k[kk] * kmul, qn = s_q[kk] * qmul;
        s.x *= gm; s.y *= gm; s.z *= gm; s.w *= gm;
        a_k.x += s.x * kn; a_k.y += s.y * kn; a_k.z += s.z * kn; a_k.w += s.w * kn;
        a_q.x += s.x * qn; a_q.y += s.y * qn; a_q.z += s.z * qn; a_q.w += s.w * qn;
      }
    }
    reinterpret_cast<float4*>(s_red + (int64_t)ks * V)[vg] = a_k;
    reinterpret_cast<float4*>(s_red + (int64_t)(nks + ks) * V)[vg] = a_q;
  }
  __syncthreads();
  if (!active) return;
  float4 vo = make_float4(0.f, 0.f, 0.f, 0.f), oq = vo;
  for (int j = 0; j < nks; ++j) {
    const float4 x = reinterpret_cast<const float4*>(s_red + (int64_t)j * V)[vg];
    const float4 y = reinterpret_cast<const float4*>(s_red + (int64_t)(nks + j) * V)[vg];
    vo.x += x.x; vo.y += x.y; vo.z += x.z; vo.w += x.w;
    oq.x += y.x; oq.y += y.y; oq.z += y.z; oq.w += y.w;
  }
  float4 d;
  {
    const int64_t vi = unit * V + 4 * vg;
    d.x = beta * (ld_elem(p.v, vi + 0, p.qkv_dt) - vo.x);
    d.y = beta * (ld_elem(p.v, vi + 1, p.qkv_dt) - vo.y);
    d.z = beta * (ld_elem(p.v, vi + 2, p.qkv_dt) - vo.z);
    d.w = beta * (ld_elem(p.v, vi + 3, p.qkv_dt) - vo.w);
    if (ks == 0) {
      st_elem(p.o, vi + 0, p.out_dt, oq.x + qk * d.x);
      st_elem(p.o, vi + 1, p.out_dt, oq.y + qk * d.y);
      st_elem(p.o, vi + 2, p.out_dt, oq.z + qk * d.z);
      st_elem(p.o, vi + 3, p.out_dt, oq.w + qk * d.w);
    }
  }
  if (ROWS > 0) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const int kk = ks + r * nks;
      if (kk < K) {
        const float kn = s_k[kk] * kmul;
        float4 s = st[r];
        s.x += kn * d.x; s.y += kn * d.y; s.z += kn * d.z; s.w += kn * d.w;
        __stcs(reinterpret_cast<float4*>(S_out + (int64_t)kk * V) + vg, s);
      }
    }
  } else {
    for (int kk = ks; kk < K; kk += nks) {
      float4 s = reinterpret_cast<const float4*>(S_in + (int64_t)kk * V)[vg];
      const float gm = gscal * s_gam[kk];
      const float kn = s_k[kk] * kmul;
      s.x = s.x * gm + kn * d.x; s.y = s.y * gm + kn * d.y;
      s.z = s.z * gm + kn * d.z; s.w = s.w * gm + kn * d.w;
      reinterpret_cast<float4*>(S_out + (int64_t)kk * V)[vg] = s;
    }
  }
}

inline size_t step_smem_bytes(int K, int V) {
  const int nvg = V >> 2;
  const int nks = kStepThreads / nvg > 0 ? kStepThreads / nvg : 1;
  return sizeof(float) * (3 * (size_t)K + 2 * (size_t)nks * V);
}

// Returns rows per thread needed to keep the whole state in registers (0: too large).
inline int step_rows(int K, int V) {
  const int nvg = V >> 2;
  if (nvg > kStepThreads) return 0;
  const int nks = kStepThreads / nvg;
  const int rows = (K + nks - 1) / nks;
  if (rows <= 4) return 4;
  if (rows <= 16) return 16;
  if (rows <= 32) return 32;
  return 0;
}

inline cudaError_t launch_step(const StepParams& p, int64_t units, cudaStream_t stream) {
  const size_t smem = step_smem_bytes(p.K, p.V);
  const dim3 grid((unsigned)units), block(kStepThreads);
  switch (step_rows(p.K, p.V)) {
    case 4: step_kernel<4><<<grid, block, smem, stream>>>(p); break;
    case 16: step_kernel<16><<<grid, block, smem, stream>>>(p); break;
    case 32: step_kernel<32><<<grid, block, smem, stream>>>(p); break;
    default: step_kernel<0><<<grid, block, smem, stream>>>(p); break;
  }
  return cudaGetLastError();
}

}  // namespace dr
