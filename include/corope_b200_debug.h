/*
 * corope_b200 -- diagnostics of libcorope_b200.so for tests and A/B timing.  Not part of the drop-in surface:
 * nothing here has a counterpart in the reference (Superposition09m/Co-RoPE), and production callers need none of it.
 * All state behind these functions is process-wide and unsynchronised between threads: with two threads (or two
 * streams driven from two threads) calling the library, "last family" reports whichever call came last.
 */
#ifndef COROPE_B200_DEBUG_H_
#define COROPE_B200_DEBUG_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/*
 * Selects the kernel family for 16-bit inputs.  Returns the previous value.
 *   0 = automatic: tensor-core kernels where the shape allows, fed from rotated fp16 copies of K (forward) / Q
 *       (backward) that a pre-pass writes to the workspace -- the fastest variant;
 *   1 = always the general (CUDA-core, fp32-arithmetic) kernels;
 *   2 = tensor-core kernels that rotate every K / Q tile in shared memory themselves: nothing rotated is ever
 *       written to HBM (the literal form of the fusion; slower, see the forward kernel's header comment).
 */
int corope_set_kernel_policy(int policy);

/* Which kernel family the last call of each op (COROPE_OP_*) used in this process: 0 general, 1 tensor-core. */
int corope_last_kernel_family(int op);

/* Number of GPU kernel launches this library has issued in this process so far. */
uint64_t corope_launch_count(void);

/*
 * Test hook for the bounded-wait path: launches one tiny kernel on `stream` whose single warp waits, with a
 * limit of `max_polls` polls, on an mbarrier that nobody ever arrives at.  The wait runs out, the kernel records
 * COROPE_DEV_WAIT_EXPIRED | 0x7e in *status_word exactly like the production kernels do, and returns normally:
 * nothing traps, faults or spins without bound.  Returns 0 or a cudaError_t.
 */
int corope_debug_expire_wait(int* status_word, unsigned max_polls, void* stream);

/*
 * The table synthesis of corope_rope_attn_fwd_freqs / _bwd_freqs on its own: cos_out / sin_out [N, half_d] fp32 (device)
 * from inv_freq [half_d] (device), angle = float(n) * inv_freq[d].  Lets a test compare the synthesized tables with
 * precompute_freqs_cis element by element.
 */
int corope_debug_synth_tables(const float* inv_freq, float* cos_out, float* sin_out, int N, int half_d, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* COROPE_B200_DEBUG_H_ */
