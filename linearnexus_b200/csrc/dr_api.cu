// C ABI of the delta-rule kernels: argument validation and dispatch.  No device memory is
// allocated here; every launch goes to the caller's stream.
#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "deltarule_sm100.h"
#include "deltarule_sm100_debug.h"
#include "dr_chunk_fp32.cuh"
#include "dr_chunk_sm100.cuh"
#include "dr_kda_sm100.cuh"
#include "dr_step_stream.cuh"
#include "dr_bwd.cuh"
#include "dr_block_ops.cuh"
#include "dr_common.cuh"
#include "dr_scan_launch.h"
#include "dr_step.cuh"

namespace {

std::atomic<uint64_t> g_launches{0};
thread_local int tl_cuda_error = 0;
thread_local int tl_device_status = 0;
thread_local const char* tl_path = "none";

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool dtype_ok(int d) { return d == DR_F32 || d == DR_BF16; }

int check_cuda(cudaError_t e) {
  if (e == cudaSuccess) return DR_OK;
  tl_cuda_error = (int)e;
  return DR_ERR_CUDA;
}

// Checks shared by every entry point.
int validate_common(const DrDesc* d, bool need_chunk) {
  if (!d) return DR_ERR_NULL;
  if (d->variant < DR_DELTA || d->variant > DR_KDA) return DR_ERR_VARIANT;
  if (d->layout != DR_LAYOUT_BHTD && d->layout != DR_LAYOUT_BTHD) return DR_ERR_SHAPE;
  if (d->B < 1 || d->H < 1 || d->T < 1) return DR_ERR_SHAPE;
  if ((int64_t)d->B * d->H > (int64_t)1 << 24) return DR_ERR_SHAPE;
  if (d->K < 4 || d->K > 256 || d->K % 4) return DR_ERR_SHAPE;
  if (d->V < 4 || d->V > 256 || d->V % 4) return DR_ERR_SHAPE;
  if (!dtype_ok(d->qkv_dtype) || !dtype_ok(d->out_dtype)) return DR_ERR_DTYPE;
  if (d->variant != DR_DELTA && !dtype_ok(d->g_dtype)) return DR_ERR_DTYPE;
  if (d->qk_heads < 0 || (d->qk_heads > 0 && (d->qk_heads > d->H || d->H % d->qk_heads))) return DR_ERR_SHAPE;
  if (d->reserved) return DR_ERR_SHAPE;
  if (need_chunk) {
    if (d->chunk < 1) return DR_ERR_CHUNK;
    // The reference raises ValueError when chunk_size % 16 != 0 for Gated DeltaNet and KDA
    // (gated_deltanet.py:318-321, kda.py:438-441); DeltaNet has no such rule.
    if (d->variant != DR_DELTA && d->chunk % 16) return DR_ERR_CHUNK;
    if (d->path < DR_PATH_AUTO || d->path > DR_PATH_SPLIT) return DR_ERR_UNSUPPORTED;
  }
  return DR_OK;
}

dr::FwdParams make_fwd(const DrDesc* d, const void* q, const void* k, const void* v, const void* g,
                       const float* beta, const float* h0, void* o, float* hT, int32_t* status) {
  dr::FwdParams p;
  p.q = q; p.k = k; p.v = v; p.g = g; p.beta = beta; p.h0 = h0; p.o = o; p.hT = hT;
  p.status = status;
  p.ckpt = nullptr;
  p.map.B = d->B; p.map.H = d->H; p.map.T = d->T; p.map.bthd = d->layout == DR_LAYOUT_BTHD;
  p.map.Hq = d->qk_heads > 0 ? d->qk_heads : d->H;
  p.K = d->K; p.V = d->V; p.C = d->chunk;
  p.variant = d->variant; p.qkv_dt = d->qkv_dtype; p.g_dt = d->g_dtype; p.out_dt = d->out_dtype;
  p.l2norm = d->use_qk_l2norm; p.scale = d->scale;
  p.set_extents();
  return p;
}

int validate_fwd_ptrs(const DrDesc* d, const void* q, const void* k, const void* v, const void* g,
                      const float* beta, const float* h0, void* o, float* hT) {
  if (!q || !k || !v || !beta || !o) return DR_ERR_NULL;
  if (d->variant == DR_DELTA ? g != nullptr : g == nullptr) return DR_ERR_VARIANT;
  // rows of q, k, v, o, per-channel g and the states are read with 16-byte accesses; beta and a scalar g are
  // read one element at a time (a sequence of a packed batch may start at any token)
  const bool g_rows = d->variant == DR_KDA;
  const uintptr_t g_mask = g_rows ? 15u : (d->g_dtype == DR_BF16 ? 1u : 3u);
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || (reinterpret_cast<uintptr_t>(beta) & 3u) ||
      (g && (reinterpret_cast<uintptr_t>(g) & g_mask)) || (h0 && !aligned16(h0)) || (hT && !aligned16(hT)))
    return DR_ERR_ALIGN;
  return DR_OK;
}

// SM count of the current device (cached per host thread and device)
int sm_count() {
  thread_local int cached_dev = -1, cached = 0;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (dev != cached_dev) {
    if (cudaDeviceGetAttribute(&cached, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    cached_dev = dev;
  }
  return cached;
}

bool tcgen05_eligible(const DrDesc* d) {
  return dr::sm100::kAvailable && d->K == 128 && d->V == 128 && d->chunk == 64 &&
         d->qkv_dtype == DR_BF16 && d->out_dtype == DR_BF16 && (d->variant == DR_GATED || d->variant == DR_DELTA) &&
         (d->variant == DR_DELTA || d->g_dtype == DR_F32);
}

// the two-kernel form (chunk-parallel intra pass + tcgen05 state pass over a workspace)
bool split_eligible(const DrDesc* d) {
  return dr::sm100::kAvailable && d->K == 128 && d->V == 128 && d->chunk == 64 && d->qkv_dtype == DR_BF16;
}
// AUTO for a shape without a tensor-core kernel: the register-resident token recurrence.  It is the same function of
// the inputs as the chunk form, does fewer multiply-adds (4 K V per token against the chunk form's 6CK + 4CV + 6KV
// over C) and measured 4-11x faster than the fp32 chunk kernel on every fp32 shape tried; DR_PATH_FP32 still asks for
// the literal chunk algorithm on the CUDA cores.
constexpr int kPathRecurrence = 100;
int resolve_chunk_path(const DrDesc* d) {
  if (d->path != DR_PATH_AUTO) return d->path;
  if (tcgen05_eligible(d)) return DR_PATH_TCGEN05;
  if (d->variant == DR_KDA && split_eligible(d)) return DR_PATH_SPLIT;
  return kPathRecurrence;
}

bool fp32_chunk_eligible(const DrDesc* d) { return d->chunk <= 64 && d->K <= 128; }

// A [B,H,T,D] / [B,T,H,D] activation as the strided per-token vector the scans of dr_linrec.cuh read.
dr::LrVec lr_vec(const void* p, int B, int H, int T, int D, int dt, int bthd, int hdiv = 1) {
  dr::LrVec v;
  v.p = p; v.dt = dt; v.hdiv = hdiv;
  v.n = (int64_t)B * H * T * D;
  if (bthd) { v.sb = (int64_t)T * H * D; v.sh = D; v.st = (int64_t)H * D; }
  else { v.sb = (int64_t)H * T * D; v.sh = (int64_t)T * D; v.st = D; }
  return v;
}
bool elem_aligned(const void* p, int dt) { return (reinterpret_cast<uintptr_t>(p) & (dt == DR_BF16 ? 1u : 3u)) == 0; }

int validate_linrec(int B, int H, int T, int K, int V, int io_dtype) {
  if (!dtype_ok(io_dtype)) return DR_ERR_DTYPE;
  if (B < 1 || H < 1 || T < 1 || K < 1 || K > 256 || V < 1 || V > 256) return DR_ERR_SHAPE;
  if ((int64_t)B * H * ((V + 63) / 64) >= ((int64_t)1 << 31)) return DR_ERR_SHAPE;
  return DR_OK;
}

__global__ void bounds_probe_kernel(int32_t* status, int64_t idx, int64_t n, int32_t* in_range) {
  *in_range = dr::in_bounds(status, idx, n) ? 1 : 0;
}

}  // namespace

extern "C" {

const char* dr_version(void) { return "deltarule_sm100 0.1 (sm_100a)"; }

const char* dr_strerror(int s) {
  switch (s) {
    case DR_OK: return "ok";
    case DR_ERR_NULL: return "a required pointer is null";
    case DR_ERR_SHAPE: return "shape out of the supported range (K,V multiples of 4 in [4,256]; B,H,T >= 1)";
    case DR_ERR_DTYPE: return "unknown or unsupported dtype tag";
    case DR_ERR_ALIGN: return "pointer not 16-byte aligned";
    case DR_ERR_WORKSPACE: return "workspace too small";
    case DR_ERR_VARIANT: return "unknown variant, or g given/missing against the variant";
    case DR_ERR_CHUNK: return "chunk size not accepted (Gated DeltaNet / KDA need a multiple of 16)";
    case DR_ERR_CUDA: return "CUDA runtime error";
    case DR_ERR_UNSUPPORTED: return "no kernel of this build covers the request";
    case DR_ERR_DEVICE: return "a kernel reported a device-side problem";
    case DR_ERR_STATIC_LIMIT:
      return "the request needs more scratch than the library's built-in static buffer (DR_STATIC_SCRATCH_BYTES); "
             "use dr_chunk_bwd with a caller-provided workspace";
    default: return "unknown status";
  }
}

int dr_last_cuda_error(void) { return tl_cuda_error; }
uint64_t dr_launch_count(void) { return g_launches.load(); }
const char* dr_last_path(void) { return tl_path; }

int64_t dr_workspace_bytes(const DrDesc* d, int op) {
  int s = validate_common(d, true);
  if (s != DR_OK) return s;
  if (op == 0)
    return (resolve_chunk_path(d) == DR_PATH_SPLIT && split_eligible(d))
               ? dr::kda::workspace_bytes((int64_t)d->B * d->H, d->T) : 0;
  if (op == 1) return dr::bwd_workspace_bytes(d);
  return DR_ERR_UNSUPPORTED;
}

int dr_chunk_fwd(const DrDesc* d, const void* q, const void* k, const void* v, const void* g,
                 const float* beta, const float* h0, void* o, float* hT, void* workspace,
                 size_t workspace_bytes, int32_t* status_dev, void* stream) {
  int s = validate_common(d, true);
  if (s != DR_OK) return s;
  s = validate_fwd_ptrs(d, q, k, v, g, beta, h0, o, hT);
  if (s != DR_OK) return s;
  const dr::FwdParams p = make_fwd(d, q, k, v, g, beta, h0, o, hT, status_dev);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int path = resolve_chunk_path(d);
  if (path == DR_PATH_SPLIT) {
    if (!split_eligible(d)) return DR_ERR_UNSUPPORTED;
    const int64_t need = dr::kda::workspace_bytes((int64_t)d->B * d->H, d->T);
    // no silent downgrade to the (much slower) kernel that needs no scratch: the caller asks for that one
    // with DR_PATH_FP32
    if (workspace && !aligned16(workspace)) return DR_ERR_ALIGN;
    if (!workspace || (int64_t)workspace_bytes < need) return DR_ERR_WORKSPACE;
    tl_path = "chunk_split_tcgen05";
    int launches = 0;
    cudaError_t e = dr::kda::launch_chunk(p, workspace, st, &launches);
    g_launches.fetch_add(launches);
    return check_cuda(e);
  }
  if (path == DR_PATH_TCGEN05) {
    if (!tcgen05_eligible(d)) return DR_ERR_UNSUPPORTED;
    tl_path = "chunk_tcgen05";
    g_launches.fetch_add(1);
    return check_cuda(dr::sm100::launch_chunk(p, st));
  }
  if (path == DR_PATH_FP32 && fp32_chunk_eligible(d)) {
    tl_path = "chunk_fp32";
    g_launches.fetch_add(1);
    return check_cuda(dr::launch_chunk_fp32(p, st));
  }
  // AUTO without a tensor-core kernel for the shape, and DR_PATH_FP32 with chunks longer than 64 or K > 128
  tl_path = "recurrent";
  g_launches.fetch_add(1);
  return check_cuda(dr::launch_recurrent(p, st));
}

int dr_chunk_fwd_varlen(const DrDesc* d, const void* q, const void* k, const void* v, const void* g,
                        const float* beta, const int32_t* cu, int32_t n_seqs, const float* h0, void* o, float* hT,
                        void* workspace, size_t workspace_bytes, int32_t* status_dev, void* stream) {
  if (!d || !cu) return DR_ERR_NULL;
  if (n_seqs < 1 || d->layout != DR_LAYOUT_BTHD || cu[0] != 0) return DR_ERR_SHAPE;
  for (int i = 0; i < n_seqs; ++i)
    if (cu[i + 1] <= cu[i]) return DR_ERR_SHAPE;   // offsets strictly increasing: no empty sequence
  const int Hq = d->qk_heads > 0 ? d->qk_heads : d->H;
  const size_t es = d->qkv_dtype == DR_BF16 ? 2 : 4, eo = d->out_dtype == DR_BF16 ? 2 : 4, eg = d->g_dtype == DR_BF16 ? 2 : 4;
  const size_t g_row = d->variant == DR_KDA ? (size_t)d->H * d->K : (size_t)d->H;
  const size_t state = (size_t)d->H * d->K * d->V;
  for (int i = 0; i < n_seqs; ++i) {
    DrDesc ds = *d;
    ds.B = 1;
    ds.T = cu[i + 1] - cu[i];
    const size_t t0 = (size_t)cu[i];
    const char* qi = static_cast<const char*>(q) + t0 * Hq * d->K * es;
    const char* ki = static_cast<const char*>(k) + t0 * Hq * d->K * es;
    const char* vi = static_cast<const char*>(v) + t0 * d->H * d->V * es;
    const char* gi = g ? static_cast<const char*>(g) + t0 * g_row * eg : nullptr;
    char* oi = static_cast<char*>(o) + t0 * d->H * d->V * eo;
    const int s = dr_chunk_fwd(&ds, qi, ki, vi, gi, beta + t0 * d->H, h0 ? h0 + i * state : nullptr, oi,
                               hT ? hT + i * state : nullptr, workspace, workspace_bytes, status_dev, stream);
    if (s != DR_OK) return s;
  }
  return DR_OK;
}

int dr_recurrent_fwd(const DrDesc* d, const void* q, const void* k, const void* v, const void* g,
                     const float* beta, const float* h0, void* o, float* hT, int32_t* status_dev, void* stream) {
  int s = validate_common(d, false);
  if (s != DR_OK) return s;
  s = validate_fwd_ptrs(d, q, k, v, g, beta, h0, o, hT);
  if (s != DR_OK) return s;
  const dr::FwdParams p = make_fwd(d, q, k, v, g, beta, h0, o, hT, status_dev);
  tl_path = "recurrent";
  g_launches.fetch_add(1);
  return check_cuda(dr::launch_recurrent(p, reinterpret_cast<cudaStream_t>(stream)));
}

int dr_step(const DrDesc* d, const void* q, const void* k, const void* v, const void* g,
            const float* beta, const float* state_in, float* state_out, void* o, int32_t* status_dev, void* stream) {
  int s = validate_common(d, false);
  if (s != DR_OK) return s;
  if (d->T != 1) return DR_ERR_SHAPE;
  if (!q || !k || !v || !beta || !o || !state_in || !state_out) return DR_ERR_NULL;
  if (d->variant == DR_DELTA ? g != nullptr : g == nullptr) return DR_ERR_VARIANT;
  if (!aligned16(state_in) || !aligned16(state_out) || !aligned16(q) || !aligned16(k) ||
      !aligned16(v) || !aligned16(o))
    return DR_ERR_ALIGN;
  dr::StepParams p;
  p.q = q; p.k = k; p.v = v; p.g = g; p.beta = beta; p.s_in = state_in; p.s_out = state_out; p.o = o;
  p.K = d->K; p.V = d->V;
  p.H = d->H; p.Hq = d->qk_heads > 0 ? d->qk_heads : d->H;
  p.variant = d->variant; p.qkv_dt = d->qkv_dtype; p.g_dt = d->g_dtype; p.out_dt = d->out_dtype;
  p.l2norm = d->use_qk_l2norm; p.scale = d->scale;
  g_launches.fetch_add(1);
  const int64_t units = (int64_t)d->B * d->H;
  const int sms = sm_count();
  if (sms > 0 && dr::step_stream_eligible(p, units, sms)) {
    tl_path = "step_stream";
    return check_cuda(dr::launch_step_stream(p, units, sms, status_dev, reinterpret_cast<cudaStream_t>(stream)));
  }
  tl_path = "step";
  return check_cuda(dr::launch_step(p, units, reinterpret_cast<cudaStream_t>(stream)));
}

int dr_check_status(int32_t* status_dev, void* stream) {
  if (!status_dev) return DR_ERR_NULL;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int32_t host = 0;
  cudaError_t e = cudaMemcpyAsync(&host, status_dev, sizeof(host), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return check_cuda(e);
  if (host == DR_DEV_OK) return DR_OK;
  e = cudaMemsetAsync(status_dev, 0, sizeof(host), st);   // reported once: the next check starts clean
  if (e != cudaSuccess) return check_cuda(e);
  tl_device_status = host;
  return DR_ERR_DEVICE;
}

int dr_last_device_status(void) { return tl_device_status; }

int dr_debug_wait_timeout(int32_t* status_dev, uint32_t attempts, void* stream) {
  if (!status_dev) return DR_ERR_NULL;
  if (attempts < 1 || attempts > 4096) return DR_ERR_SHAPE;
  tl_path = "wait_timeout";
  g_launches.fetch_add(1);
  dr::sm100::wait_timeout_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(status_dev, attempts);
  return check_cuda(cudaGetLastError());
}

int dr_debug_wait_site(int32_t* status_dev, uint32_t barrier_number, uint32_t group, void* stream) {
  if (!status_dev) return DR_ERR_NULL;
  if (barrier_number > 63 || group > 3) return DR_ERR_SHAPE;
  tl_path = "wait_site";
  g_launches.fetch_add(1);
  dr::sm100::wait_site_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(status_dev, barrier_number, group);
  return check_cuda(cudaGetLastError());
}

int dr_debug_umma_selftest(const void* a, const void* b, float* d_out, int kd, int n, int a_in_tmem,
                            int b_mn_major, int32_t* status_dev, void* stream) {
  if (!a || !b || !d_out) return DR_ERR_NULL;
  if ((n != 64 && n != 128) || kd < 32 || kd > 128 || kd % 32) return DR_ERR_SHAPE;
  tl_path = "umma_selftest";
  g_launches.fetch_add(1);
  return check_cuda(dr::sm100::launch_umma_selftest(a, b, d_out, kd, n, a_in_tmem, b_mn_major, status_dev,
                                                    reinterpret_cast<cudaStream_t>(stream)));
}

int dr_chunk_bwd(const DrDesc* d, const void* q, const void* k, const void* v, const void* g,
                 const float* beta, const float* h0, const void* d_o, const float* d_hT, void* dq,
                 void* dk, void* dv, float* dbeta, float* dg, float* dh0, void* workspace,
                 size_t workspace_bytes, int32_t* status_dev, void* stream) {
  int s = validate_common(d, true);
  if (s != DR_OK) return s;
  if (!q || !k || !v || !beta || !d_o || !dq || !dk || !dv || !dbeta) return DR_ERR_NULL;
  if (d->variant == DR_DELTA ? (g != nullptr || dg != nullptr) : (g == nullptr || dg == nullptr))
    return DR_ERR_VARIANT;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(d_o) || !aligned16(dq) ||
      !aligned16(dk) || !aligned16(dv) || !aligned16(workspace))
    return DR_ERR_ALIGN;
  const int64_t need = dr::bwd_workspace_bytes(d);
  if (need < 0) return (int)need;
  if ((int64_t)workspace_bytes < need || (need > 0 && !workspace)) return DR_ERR_WORKSPACE;
  tl_path = "bwd";
  int launches = 0;
  cudaError_t e = dr::launch_bwd(d, q, k, v, g, beta, h0, d_o, d_hT, dq, dk, dv, dbeta, dg, dh0,
                                 workspace, status_dev, reinterpret_cast<cudaStream_t>(stream), &launches);
  g_launches.fetch_add(launches);
  return check_cuda(e);
}

int dr_chunk_bwd_varlen(const DrDesc* d, const void* q, const void* k, const void* v, const void* g,
                        const float* beta, const int32_t* cu, int32_t n_seqs, const float* h0, const void* d_o,
                        const float* d_hT, void* dq, void* dk, void* dv, float* dbeta, float* dg, float* dh0,
                        void* workspace, size_t workspace_bytes, int32_t* status_dev, void* stream) {
  if (!d || !cu) return DR_ERR_NULL;
  if (n_seqs < 1 || d->layout != DR_LAYOUT_BTHD || cu[0] != 0) return DR_ERR_SHAPE;
  for (int i = 0; i < n_seqs; ++i)
    if (cu[i + 1] <= cu[i]) return DR_ERR_SHAPE;
  if (!q || !k || !v || !d_o || !dq || !dk || !dv || !beta || !dbeta) return DR_ERR_NULL;
  const int Hq = d->qk_heads > 0 ? d->qk_heads : d->H;
  const size_t es = d->qkv_dtype == DR_BF16 ? 2 : 4, eg = d->g_dtype == DR_BF16 ? 2 : 4;
  const size_t g_row = d->variant == DR_KDA ? (size_t)d->H * d->K : (size_t)d->H;
  const size_t state = (size_t)d->H * d->K * d->V;
  // the sequences run one after another on `stream`, so they can share the workspace
  for (int i = 0; i < n_seqs; ++i) {
    DrDesc ds = *d;
    ds.B = 1;
    ds.T = cu[i + 1] - cu[i];
    const size_t t0 = (size_t)cu[i];
    const size_t oqk = t0 * Hq * d->K * es, ov = t0 * d->H * d->V * es;
    auto at = [](const void* p, size_t off) { return p ? static_cast<const char*>(p) + off : nullptr; };
    auto atw = [](void* p, size_t off) { return p ? static_cast<char*>(p) + off : nullptr; };
    const int s = dr_chunk_bwd(&ds, at(q, oqk), at(k, oqk), at(v, ov), at(g, t0 * g_row * eg), beta + t0 * d->H,
                               h0 ? h0 + i * state : nullptr, at(d_o, ov), d_hT ? d_hT + i * state : nullptr,
                               atw(dq, oqk), atw(dk, oqk), atw(dv, ov), dbeta + t0 * d->H, dg ? dg + t0 * g_row : nullptr,
                               dh0 ? dh0 + i * state : nullptr, workspace, workspace_bytes, status_dev, stream);
    if (s != DR_OK) return s;
  }
  return DR_OK;
}

int dr_chunk_fwd_saving(const DrDesc* d, const void* q, const void* k, const void* v, const void* g,
                        const float* beta, const float* h0, void* o, float* hT, void* workspace,
                        size_t workspace_bytes, int32_t* status_dev, void* stream) {
  int s = validate_common(d, true);
  if (s != DR_OK) return s;
  s = validate_fwd_ptrs(d, q, k, v, g, beta, h0, o, hT);
  if (s != DR_OK) return s;
  const int64_t need = dr::bwd_workspace_bytes(d);
  if (need < 0) return (int)need;
  if (!workspace || (int64_t)workspace_bytes < need) return DR_ERR_WORKSPACE;
  if (!aligned16(workspace)) return DR_ERR_ALIGN;
  tl_path = "fwd_saving";
  int launches = 0;
  cudaError_t e = dr::launch_bwd_forward(d, q, k, v, g, beta, h0, o, hT, workspace, status_dev,
                                         reinterpret_cast<cudaStream_t>(stream), &launches);
  g_launches.fetch_add(launches);
  return check_cuda(e);
}

int dr_chunk_bwd_saved(const DrDesc* d, const void* q, const void* k, const void* v, const void* g,
                       const float* beta, const void* d_o, const float* d_hT, void* dq, void* dk, void* dv,
                       float* dbeta, float* dg, float* dh0, void* workspace, size_t workspace_bytes,
                       int32_t* status_dev, void* stream) {
  (void)status_dev;   // the adjoint kernels have no bounded waits: nothing can be reported here
  int s = validate_common(d, true);
  if (s != DR_OK) return s;
  if (!q || !k || !v || !beta || !d_o || !dq || !dk || !dv || !dbeta) return DR_ERR_NULL;
  if (d->variant == DR_DELTA ? (g != nullptr || dg != nullptr) : (g == nullptr || dg == nullptr))
    return DR_ERR_VARIANT;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(d_o) || !aligned16(dq) ||
      !aligned16(dk) || !aligned16(dv) || !aligned16(workspace))
    return DR_ERR_ALIGN;
  const int64_t need = dr::bwd_workspace_bytes(d);
  if (need < 0) return (int)need;
  if ((int64_t)workspace_bytes < need || !workspace) return DR_ERR_WORKSPACE;
  tl_path = "bwd_saved";
  int launches = 0;
  cudaError_t e = dr::launch_bwd_adjoint(d, q, k, v, g, beta, d_o, d_hT, dq, dk, dv, dbeta, dg, dh0, workspace,
                                         reinterpret_cast<cudaStream_t>(stream), &launches);
  g_launches.fetch_add(launches);
  return check_cuda(e);
}

// ---- backward without any allocation by the caller ------------------------------------------------
// Scratch for dr_chunk_bwd_static lives in the library's own device image: a fixed-size array that
// every GPU which loads the library carries from module load until the process exits.
static __device__ __align__(256) unsigned char g_bwd_static_scratch[DR_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
void* g_static_ptr[kMaxDevices] = {nullptr};

// Device address of the static scratch array on the CURRENT device.  The array's name is only a
// host-side handle; the kernels need the address the runtime resolves for this device's copy.
int static_scratch_address(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return check_cuda(e);
  if (dev < 0 || dev >= kMaxDevices) return DR_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (!g_static_ptr[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_bwd_static_scratch);
    if (e != cudaSuccess) return check_cuda(e);
    g_static_ptr[dev] = ptr;
  }
  *out = g_static_ptr[dev];
  return DR_OK;
}
}  // namespace

int dr_chunk_bwd_static(const DrDesc* d, const void* q, const void* k, const void* v, const void* g,
                        const float* beta, const float* h0, const void* d_o, const float* d_hT, void* dq,
                        void* dk, void* dv, float* dbeta, float* dg, float* dh0, int32_t* status_dev,
                        void* stream) {
  int s = validate_common(d, true);
  if (s != DR_OK) return s;
  if (!q || !k || !v || !beta || !d_o || !dq || !dk || !dv || !dbeta) return DR_ERR_NULL;
  if (d->variant == DR_DELTA ? (g != nullptr || dg != nullptr) : (g == nullptr || dg == nullptr))
    return DR_ERR_VARIANT;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(d_o) || !aligned16(dq) ||
      !aligned16(dk) || !aligned16(dv))
    return DR_ERR_ALIGN;
  const int64_t need = dr::bwd_workspace_bytes(d);
  if (need < 0) return (int)need;
  if (need > (int64_t)DR_STATIC_SCRATCH_BYTES) return DR_ERR_STATIC_LIMIT;
  void* scratch = nullptr;
  s = static_scratch_address(&scratch);  // first call on a device resolves the symbol; later calls reuse it
  if (s != DR_OK) return s;
  tl_path = "bwd_static";
  int launches = 0;
  // launch_bwd zeroes the accumulators it adds into and overwrites the checkpoints before reading them,
  // so whatever an earlier call left in the array is never consumed.
  // own_stream = false: this entry creates nothing, not even a stream or an event (everything runs on `stream`)
  cudaError_t e = dr::launch_bwd(d, q, k, v, g, beta, h0, d_o, d_hT, dq, dk, dv, dbeta, dg, dh0, scratch, status_dev,
                                 reinterpret_cast<cudaStream_t>(stream), &launches, false);
  g_launches.fetch_add(launches);
  return check_cuda(e);
}

int dr_short_conv_silu(const void* x, const float* weight, const float* bias, const void* cache_in, void* y,
                       void* cache_out, int B, int T, int C, int W, int dtype, int apply_silu, void* stream) {
  if (!x || !y || (W > 1 && !weight)) return DR_ERR_NULL;
  if (dtype != DR_F32 && dtype != DR_BF16) return DR_ERR_DTYPE;
  if (B < 1 || T < 1 || C < 1 || W < 1 || W > dr::blk::kConvMaxW || C % 8) return DR_ERR_SHAPE;
  if (B > 65535 || (T + 15) / 16 > 65535) return DR_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(y) || (cache_in && !aligned16(cache_in)) || (cache_out && !aligned16(cache_out)) ||
      (W > 1 && !aligned16(weight)) || (bias && !aligned16(bias)))   // the kernel reads taps and bias as float4
    return DR_ERR_ALIGN;
  if (x == y) return DR_ERR_UNSUPPORTED;   // a tile reads the rows before it: not in place
  if (cache_out && cache_out == cache_in && T > dr::blk::kConvSteps) return DR_ERR_UNSUPPORTED;
  dr::blk::ConvParams p;
  p.x = x; p.w = weight; p.bias = bias; p.cache_in = W > 1 ? cache_in : nullptr; p.y = y;
  p.cache_out = W > 1 ? cache_out : nullptr;
  p.B = B; p.T = T; p.C = C; p.W = W; p.apply_silu = apply_silu;
  tl_path = "short_conv";
  cudaError_t e = dr::blk::launch_short_conv(p, dtype, reinterpret_cast<cudaStream_t>(stream));
  g_launches.fetch_add(1);
  return check_cuda(e);
}

int dr_gate_activations(int mode, const void* a, const void* b, const float* A_log, const float* bias, float* g,
                        float* beta, int B, int T, int H, int K, int a_dtype, int b_dtype, float beta_scale,
                        float threshold, void* stream) {
  if (!a || !A_log || !g || ((b == nullptr) != (beta == nullptr))) return DR_ERR_NULL;
  if (mode != 0 && mode != 1) return DR_ERR_VARIANT;
  if ((a_dtype != DR_F32 && a_dtype != DR_BF16) || (b && b_dtype != DR_F32 && b_dtype != DR_BF16)) return DR_ERR_DTYPE;
  if (B < 1 || T < 1 || H < 1 || K < 1 || (mode == 0 && K != 1)) return DR_ERR_SHAPE;
  dr::blk::GateParams p;
  p.a = a; p.b = b; p.A_log = A_log; p.bias = bias; p.g = g; p.beta = beta;
  p.n_beta = b ? (int64_t)B * T * H : 0;
  p.n_g = (int64_t)B * T * H * K;
  p.H = H; p.K = K; p.a_dt = a_dtype; p.b_dt = b_dtype; p.mode = mode;
  p.beta_scale = beta_scale; p.threshold = threshold;
  tl_path = "gate_activations";
  cudaError_t e = dr::blk::launch_gate_act(p, reinterpret_cast<cudaStream_t>(stream));
  g_launches.fetch_add(1);
  return check_cuda(e);
}

int dr_gated_rmsnorm(const void* o, const void* gate, const float* weight, void* y, int B, int H, int T, int V,
                     int o_layout, int o_dtype, int gate_dtype, int y_dtype, float eps, void* stream) {
  if (!o || !weight || !y) return DR_ERR_NULL;
  if (o_layout != DR_LAYOUT_BHTD && o_layout != DR_LAYOUT_BTHD) return DR_ERR_SHAPE;
  if ((o_dtype != DR_F32 && o_dtype != DR_BF16) || (y_dtype != DR_F32 && y_dtype != DR_BF16) ||
      (gate && gate_dtype != DR_F32 && gate_dtype != DR_BF16))
    return DR_ERR_DTYPE;
  if (B < 1 || H < 1 || T < 1 || V < 4 || V > 512 || V % 4) return DR_ERR_SHAPE;
  if ((int64_t)B * H * T >= ((int64_t)1 << 31)) return DR_ERR_SHAPE;
  if (!aligned16(o) || !aligned16(y) || !aligned16(weight) || (gate && !aligned16(gate))) return DR_ERR_ALIGN;
  if (o == y && o_layout != DR_LAYOUT_BTHD) return DR_ERR_UNSUPPORTED;
  dr::blk::NormParams p;
  p.o = o; p.gate = gate; p.w = weight; p.y = y;
  p.map.B = B; p.map.H = H; p.map.T = T; p.map.bthd = o_layout == DR_LAYOUT_BTHD; p.map.Hq = H;
  p.V = V; p.eps = eps;
  tl_path = "gated_rmsnorm";
  cudaError_t e = dr::blk::launch_gated_rmsnorm(p, o_dtype, gate ? gate_dtype : o_dtype, y_dtype, sm_count(),
                                                reinterpret_cast<cudaStream_t>(stream));
  g_launches.fetch_add(1);
  return check_cuda(e);
}

int dr_dplr_recurrent(const void* q, const void* k, const void* v, const void* a, const void* b, const void* gk,
                      const float* h0, void* o, float* hT, int B, int H, int T, int K, int V, float scale,
                      int io_dtype, int layout, int32_t* status_dev, void* stream) {
  if (!q || !k || !v || !a || !b || !gk || !o) return DR_ERR_NULL;
  if (layout != DR_LAYOUT_BHTD && layout != DR_LAYOUT_BTHD) return DR_ERR_SHAPE;
  int s = validate_linrec(B, H, T, K, V, io_dtype);
  if (s != DR_OK) return s;
  for (const void* ptr : {q, k, v, a, b, gk, (const void*)o})
    if (!elem_aligned(ptr, io_dtype)) return DR_ERR_ALIGN;
  const int bthd = layout == DR_LAYOUT_BTHD;
  dr::LinRecParams p{};
  p.q = lr_vec(q, B, H, T, K, io_dtype, bthd); p.k = lr_vec(k, B, H, T, K, io_dtype, bthd);
  p.w = lr_vec(gk, B, H, T, K, io_dtype, bthd); p.a = lr_vec(a, B, H, T, K, io_dtype, bthd);
  p.b = lr_vec(b, B, H, T, K, io_dtype, bthd); p.v = lr_vec(v, B, H, T, V, io_dtype, bthd);
  const dr::LrVec ov = lr_vec(o, B, H, T, V, io_dtype, bthd);
  p.o = o; p.o_sb = ov.sb; p.o_sh = ov.sh; p.o_st = ov.st; p.o_dt = io_dtype;
  p.h0 = h0; p.hT = hT; p.s_k = V; p.s_v = 1;
  p.B = B; p.H = H; p.T = T; p.K = K; p.V = V; p.scale = scale;
  p.status = status_dev; p.n_o = ov.n; p.n_state = (int64_t)B * H * K * V;
  tl_path = "dplr_recurrent";
  cudaError_t e = dr::launch_linrec(dr::LR_DPLR, io_dtype == DR_BF16, p, reinterpret_cast<cudaStream_t>(stream));
  g_launches.fetch_add(1);
  return check_cuda(e);
}

int dr_rwkv6_recurrent(const void* r, const void* k, const void* v, const void* w, const float* u, const float* h0,
                       void* o, float* hT, int B, int H, int T, int K, int V, float scale, int io_dtype, int layout,
                       int32_t* status_dev, void* stream) {
  if (!r || !k || !v || !w || !u || !o) return DR_ERR_NULL;
  if (layout != DR_LAYOUT_BHTD && layout != DR_LAYOUT_BTHD) return DR_ERR_SHAPE;
  int s = validate_linrec(B, H, T, K, V, io_dtype);
  if (s != DR_OK) return s;
  for (const void* ptr : {r, k, v, w, (const void*)o})
    if (!elem_aligned(ptr, io_dtype)) return DR_ERR_ALIGN;
  const int bthd = layout == DR_LAYOUT_BTHD;
  dr::LinRecParams p{};
  p.q = lr_vec(r, B, H, T, K, io_dtype, bthd); p.k = lr_vec(k, B, H, T, K, io_dtype, bthd);
  p.w = lr_vec(w, B, H, T, K, io_dtype, bthd); p.v = lr_vec(v, B, H, T, V, io_dtype, bthd);
  p.a = p.q; p.b = p.q;
  const dr::LrVec ov = lr_vec(o, B, H, T, V, io_dtype, bthd);
  p.o = o; p.o_sb = ov.sb; p.o_sh = ov.sh; p.o_st = ov.st; p.o_dt = io_dtype;
  p.u = u; p.h0 = h0; p.hT = hT; p.s_k = V; p.s_v = 1;
  p.B = B; p.H = H; p.T = T; p.K = K; p.V = V; p.scale = scale;
  p.status = status_dev; p.n_o = ov.n; p.n_state = (int64_t)B * H * K * V;
  tl_path = "rwkv6_recurrent";
  cudaError_t e = dr::launch_linrec(dr::LR_RWKV6, io_dtype == DR_BF16, p, reinterpret_cast<cudaStream_t>(stream));
  g_launches.fetch_add(1);
  return check_cuda(e);
}

int dr_ssd_scan(const void* x, const void* dt, const float* A, const void* Bm, const void* Cm, const float* D,
                const float* dt_bias, const float* h0, void* y, float* hT, int B, int T, int H, int P, int N,
                int groups, float dt_lo, float dt_hi, int io_dtype, int32_t* status_dev, void* stream) {
  if (!x || !dt || !A || !Bm || !Cm || !D || !y) return DR_ERR_NULL;
  int s = validate_linrec(B, H, T, N, P, io_dtype);
  if (s != DR_OK) return s;
  if (groups < 1 || groups > H || H % groups) return DR_ERR_SHAPE;
  for (const void* ptr : {x, Bm, Cm, (const void*)y})
    if (!elem_aligned(ptr, io_dtype)) return DR_ERR_ALIGN;
  if (!elem_aligned(dt, DR_F32)) return DR_ERR_ALIGN;
  dr::LinRecParams p{};
  // key axis = the N state channels (B writes, C reads), value axis = the P channels of the head
  p.q = lr_vec(Cm, B, groups, T, N, io_dtype, 1, H / groups);
  p.k = lr_vec(Bm, B, groups, T, N, io_dtype, 1, H / groups);
  p.w = p.q; p.a = p.q; p.b = p.q;
  p.v = lr_vec(x, B, H, T, P, io_dtype, 1);
  p.dt = lr_vec(dt, B, H, T, 1, DR_F32, 1);
  const dr::LrVec ov = lr_vec(y, B, H, T, P, io_dtype, 1);
  p.o = y; p.o_sb = ov.sb; p.o_sh = ov.sh; p.o_st = ov.st; p.o_dt = io_dtype;
  p.A = A; p.D = D; p.dt_bias = dt_bias; p.h0 = h0; p.hT = hT;
  p.s_k = 1; p.s_v = N;   // state stored [P, N]
  p.B = B; p.H = H; p.T = T; p.K = N; p.V = P; p.scale = 1.f; p.dt_lo = dt_lo; p.dt_hi = dt_hi;
  p.status = status_dev; p.n_o = ov.n; p.n_state = (int64_t)B * H * P * N;
  tl_path = "ssd_scan";
  cudaError_t e = dr::launch_linrec(dr::LR_SSD, io_dtype == DR_BF16, p, reinterpret_cast<cudaStream_t>(stream));
  g_launches.fetch_add(1);
  return check_cuda(e);
}

int dr_debug_bounds_checked(void) {
#ifdef DR_BOUNDS_CHECK
  return 1;
#else
  return 0;
#endif
}

int dr_debug_bounds_probe(int32_t* status_dev, int64_t idx, int64_t n, int32_t* in_range_dev, void* stream) {
  if (!status_dev || !in_range_dev) return DR_ERR_NULL;
  bounds_probe_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(status_dev, idx, n, in_range_dev);
  g_launches.fetch_add(1);
  return check_cuda(cudaGetLastError());
}

}  // extern "C"
