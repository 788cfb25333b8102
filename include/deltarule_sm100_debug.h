/*
 * deltarule_sm100 -- test and bring-up entry points of the library.  None has a counterpart in the
 * reference; production callers need only deltarule_sm100.h.
 */
#ifndef DELTARULE_SM100_DEBUG_H_
#define DELTARULE_SM100_DEBUG_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/*
 * Runs one 128 x n x kd bf16 product D = A * B^T through the tcgen05/TMEM plumbing the chunk kernels
 * use (A [128][kd] row-major read from shared memory or staged in tensor memory; B given as [n][kd]
 * (K-major) or as [kd][n] (MN-major)), so the GPU tests can pin the descriptor encodings against a
 * plain matmul.  n in {64,128}; kd in {32,64,96,128}.  d_out: float32 [128][n].
 */
int dr_debug_umma_selftest(const void* a, const void* b, float* d_out, int kd, int n, int a_in_tmem,
                           int b_mn_major, int32_t* status_dev, void* stream);

/*
 * Exercises the error path of the bounded waits without faulting anything: one warp waits, with the
 * kernels' own wait routine limited to `attempts` tries (1..4096), on an mbarrier that nothing arrives
 * on.  The wait gives up, DR_DEV_TIMEOUT is ORed into *status_dev and the kernel returns normally; the
 * CUDA context stays usable.
 */
int dr_debug_wait_timeout(int32_t* status_dev, uint32_t attempts, void* stream);

/*
 * The same through the wait routine of the tcgen05 kernels with its full bound (about one second): DR_DEV_TIMEOUT plus,
 * in bits 8..15 of the word (DR_DEV_SITE), the barrier number (0..63) and warp group (0..3) given here, as a kernel
 * would record where its first wait gave up.
 */
int dr_debug_wait_site(int32_t* status_dev, uint32_t barrier_number, uint32_t group, void* stream);

/*
 * The index checks of the debug build.  linearnexus_b200/libdeltarule_sm100_bounds.so is this library compiled with
 * -DDR_BOUNDS_CHECK: the kernels that index global memory by hand (token recurrences and scans, the fp32 chunk kernel,
 * the plain loads and stores of the fused tcgen05 forward) compare every index with the size of the caller's array
 * first; an index outside sets DR_DEV_BOUNDS in *status_dev and the access is skipped (no trap, no fault).
 * dr_debug_bounds_checked() tells which build is loaded (1: checks compiled in).  dr_debug_bounds_probe runs the check
 * routine itself on (idx, n) without touching memory: *in_range_dev = 1 when 0 <= idx < n, else 0 and -- in the debug
 * build only -- the status bit.
 */
int dr_debug_bounds_checked(void);
int dr_debug_bounds_probe(int32_t* status_dev, int64_t idx, int64_t n, int32_t* in_range_dev, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DELTARULE_SM100_DEBUG_H_ */
