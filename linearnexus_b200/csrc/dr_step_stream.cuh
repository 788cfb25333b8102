// Decode step for K = V = 128 as a persistent, software-pipelined stream over the state cache.
//
// One CTA per SM walks its share of the (batch, head) units.  The 64 KB state of a unit travels by the TMA
// engine in both directions: cp.async.bulk global -> shared one unit ahead (three 64 KB buffers: one being
// loaded, one being worked on, one being written back), cp.async.bulk shared -> global after the update.
// The threads only ever touch shared memory and registers, so the memory system always has a full load and
// a full store of 64 KB in flight per SM, with no phase in which a CTA's loads have drained and its stores
// have not started (what limits the one-CTA-per-unit kernel to two such CTAs per SM).
// Same arithmetic as step_kernel:
//     S~ = gamma * S ; d = beta * (v - S~^T k) ; S' = S~ + k d^T ; o = S~^T q + (q.k) d
#pragma once

#include "dr_step.cuh"
#include "dr_tcgen05.cuh"

namespace dr {

constexpr int kStreamStages = 3;
constexpr int kStreamD = 128;
constexpr int kStreamStateBytes = kStreamD * kStreamD * 4;   // 65536
// three state buffers; q, k, gamma, v [128] each; reduction scratch [2][8][128]
constexpr int kStreamSmem = kStreamStages * kStreamStateBytes + (4 * kStreamD + 2 * 8 * kStreamD) * 4;

__global__ void __launch_bounds__(kStepThreads, 1) step_stream_kernel(const StepParams p, const int64_t units,
                                                                      int32_t* status) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  float* sS = reinterpret_cast<float*>(smem_raw);
  float* s_q = sS + kStreamStages * kStreamD * kStreamD;
  float* s_k = s_q + kStreamD;
  float* s_gam = s_k + kStreamD;
  float* s_v = s_gam + kStreamD;
  float* s_red = s_v + kStreamD;   // [2][8][128]
  __shared__ __align__(8) uint64_t full[kStreamStages];
  __shared__ float s_part[3][4];
  __shared__ int s_abort;   // set once a bounded wait has run out: from then on nothing is written back
  constexpr int K = kStreamD, V = kStreamD;

  const int tid = threadIdx.x;
  const int vg = tid & 31, ks = tid >> 5;   // float4 column group, row group (rows ks, ks + 8, ...)
  const int64_t first = blockIdx.x, stride = gridDim.x;
  if (first >= units) return;
  const int64_t nmine = (units - first + stride - 1) / stride;

  if (tid == 0) {
    for (int i = 0; i < kStreamStages; ++i) tc::mbar_init(tc::smem_u32(&full[i]), 1);
    tc::fence_mbar_init();
    s_abort = 0;
  }
  __syncthreads();
  auto issue_load = [&](int64_t i) {   // thread 0
    const uint32_t bar = tc::smem_u32(&full[i % kStreamStages]);
    tc::mbar_arrive_expect_tx(bar, kStreamStateBytes);
    const uint32_t dst = tc::smem_u32(sS + (i % kStreamStages) * K * V);
    const uint8_t* src = reinterpret_cast<const uint8_t*>(p.s_in + (first + i * stride) * (int64_t)K * V);
#pragma unroll
    for (int c = 0; c < 4; ++c) tc::bulk_g2s(dst + c * 16384, src + c * 16384, 16384, bar);
  };
  if (tid == 0) issue_load(0);

  // raw per-unit vectors of the NEXT unit, fetched one iteration ahead (thread t < 128: channel t)
  float nq = 0.f, nk = 0.f, ng = 0.f, nv = 0.f, nbeta = 0.f, ngs = 0.f;
  auto fetch_small = [&](int64_t unit) {
    if (tid < K) {
      nq = ld_elem(p.q, p.unit_qk(unit) * K + tid, p.qkv_dt);
      nk = ld_elem(p.k, p.unit_qk(unit) * K + tid, p.qkv_dt);
      nv = ld_elem(p.v, unit * V + tid, p.qkv_dt);
      if (p.variant == DR_KDA) ng = ld_elem(p.g, unit * K + tid, p.g_dt);
    }
    nbeta = p.beta[unit];
    if (p.variant == DR_GATED) ngs = ld_elem(p.g, unit, p.g_dt);
  };
  fetch_small(first);

  for (int64_t i = 0; i < nmine; ++i) {
    const int64_t unit = first + i * stride;
    float* S = sS + (i % kStreamStages) * K * V;
    // this unit's vectors -> shared; then the next unit's loads (state by TMA, vectors into registers)
    const float beta = nbeta;
    const float gscal = (p.variant == DR_GATED) ? expf(ngs) : 1.f;
    float qq = 0.f, kk2 = 0.f, kq = 0.f;
    if (tid < K) {
      s_q[tid] = nq;
      s_k[tid] = nk;
      s_v[tid] = nv;
      s_gam[tid] = (p.variant == DR_KDA) ? expf(ng) : 1.f;
      qq = nq * nq; kk2 = nk * nk; kq = nq * nk;
      qq = warp_sum(qq); kk2 = warp_sum(kk2); kq = warp_sum(kq);
      if ((tid & 31) == 0) { s_part[0][tid >> 5] = qq; s_part[1][tid >> 5] = kk2; s_part[2][tid >> 5] = kq; }
    }
    if (i + 1 < nmine) {
      if (tid == 0) {
        tc::bulk_wait_read_1();   // the write-back that last used the target buffer (two units ago) has read it
        issue_load(i + 1);
      }
      fetch_small(unit + stride);
    }
    __syncthreads();
    float qmul = p.scale, kmul = 1.f;
    const float sq = s_part[0][0] + s_part[0][1] + s_part[0][2] + s_part[0][3];
    const float sk = s_part[1][0] + s_part[1][1] + s_part[1][2] + s_part[1][3];
    const float sqk = s_part[2][0] + s_part[2][1] + s_part[2][2] + s_part[2][3];
    if (p.l2norm) {
      qmul = p.scale / (sqrtf(sq) + 1e-6f);
      kmul = 1.f / (sqrtf(sk) + 1e-6f);
    }
    const float qk = sqk * qmul * kmul;

    // the state has landed
    {
      const uint32_t bar = tc::smem_u32(&full[i % kStreamStages]);
      const uint32_t parity = (uint32_t)((i / kStreamStages) & 1);
      if (!tc::mbar_wait_bounded(bar, parity, 4u << 20)) {
        s_abort = 1;   // the state of this unit never arrived: its stale buffer must not reach the cache
        if (status) atomicOr(status, DR_DEV_TIMEOUT);
      }
    }
    float4 st[16];
    float4 a_k = make_float4(0.f, 0.f, 0.f, 0.f), a_q = a_k;
#pragma unroll
    for (int r = 0; r < 16; ++r) {
      const int kk = ks + 8 * r;
      st[r] = reinterpret_cast<const float4*>(S + kk * V)[vg];
      const float gm = gscal * s_gam[kk];
      const float kn = s_k[kk] * kmul, qn = s_q[kk] * qmul;
      st[r].x *= gm; st[r].y *= gm; st[r].z *= gm; st[r].w *= gm;
      a_k.x += st[r].x * kn; a_k.y += st[r].y * kn; a_k.z += st[r].z * kn; a_k.w += st[r].w * kn;
      a_q.x += st[r].x * qn; a_q.y += st[r].y * qn; a_q.z += st[r].z * qn; a_q.w += st[r].w * qn;
    }
    reinterpret_cast<float4*>(s_red + ks * V)[vg] = a_k;
    reinterpret_cast<float4*>(s_red + (8 + ks) * V)[vg] = a_q;
    __syncthreads();
    float4 vo = make_float4(0.f, 0.f, 0.f, 0.f), oq = vo;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float4 x = reinterpret_cast<const float4*>(s_red + j * V)[vg];
      const float4 y = reinterpret_cast<const float4*>(s_red + (8 + j) * V)[vg];
      vo.x += x.x; vo.y += x.y; vo.z += x.z; vo.w += x.w;
      oq.x += y.x; oq.y += y.y; oq.z += y.z; oq.w += y.w;
    }
    const float4 vv = reinterpret_cast<const float4*>(s_v)[vg];
    float4 d;
    d.x = beta * (vv.x - vo.x); d.y = beta * (vv.y - vo.y); d.z = beta * (vv.z - vo.z); d.w = beta * (vv.w - vo.w);
    if (ks == 0) {
      const int64_t vi = unit * V + 4 * vg;
      st_elem(p.o, vi + 0, p.out_dt, oq.x + qk * d.x);
      st_elem(p.o, vi + 1, p.out_dt, oq.y + qk * d.y);
      st_elem(p.o, vi + 2, p.out_dt, oq.z + qk * d.z);
      st_elem(p.o, vi + 3, p.out_dt, oq.w + qk * d.w);
    }
#pragma unroll
    for (int r = 0; r < 16; ++r) {
      const int kk = ks + 8 * r;
      const float kn = s_k[kk] * kmul;
      float4 s = st[r];
      s.x += kn * d.x; s.y += kn * d.y; s.z += kn * d.z; s.w += kn * d.w;
      reinterpret_cast<float4*>(S + kk * V)[vg] = s;
    }
    tc::fence_async_smem();   // the updated state is read by the TMA engine next
    __syncthreads();
    if (tid == 0 && !s_abort) {
      uint8_t* dst = reinterpret_cast<uint8_t*>(p.s_out + unit * (int64_t)K * V);
      const uint32_t src = tc::smem_u32(S);
#pragma unroll
      for (int c = 0; c < 4; ++c) tc::bulk_s2g(dst + c * 16384, src + c * 16384, 16384);
      tc::bulk_commit();
    }
  }
  if (tid == 0) tc::bulk_wait_all();
}

// the streamed kernel serves K = V = 128 once there is more than one unit per SM to pipeline
inline bool step_stream_eligible(const StepParams& p, int64_t units, int sms) {
  return p.K == kStreamD && p.V == kStreamD && units >= 2 * (int64_t)sms;
}

inline cudaError_t launch_step_stream(const StepParams& p, int64_t units, int sms, int32_t* status,
                                      cudaStream_t stream) {
  cudaError_t e = cudaFuncSetAttribute(step_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kStreamSmem);
  if (e != cudaSuccess) return e;
  step_stream_kernel<<<(unsigned)sms, kStepThreads, kStreamSmem, stream>>>(p, units, status);
  return cudaGetLastError();
}

}  // namespace dr
