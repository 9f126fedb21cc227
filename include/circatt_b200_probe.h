/*
 * circatt_b200_probe.h -- measurement helpers exported by libcircatt_b200.so.
 * They have no counterpart in the reference; the benchmark uses them to count
 * the library's own kernel launches and to measure the FP32 FMA peak that the
 * roofline fraction of the windowed kernels is quoted against.
 */
#ifndef CIRCATT_B200_PROBE_H
#define CIRCATT_B200_PROBE_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* Number of kernels this library has launched in the calling process so far. */
int64_t ca_probe_launch_count(void);

/* Of those, the launches of the fused fast-path kernels: the TMA-tiled ones and the sliding-tile kernels for
 * 1-D signals (the tests use the difference around a call to assert that the call ran on that path and not
 * on the generic kernels). */
int64_t ca_probe_tiled_launch_count(void);

/* Launches one kernel of `blocks` x 256 threads; each thread runs `iters`
 * rounds of 16 independent packed FP32 FMAs (fma.rn.f32x2) on registers and
 * stores one value to `sink` (blocks*256 floats).  The kernel executes
 * blocks*256*iters*16*2 FMAs = twice that many flops. */
int ca_probe_ffma(int32_t blocks, int32_t iters, float* sink, void* stream);

/* Self test of the bounded device-side waits: launches one thread block that arms a stage
 * barrier with 64 bytes and issues a 32-byte bulk copy, so the barrier can never complete.  The
 * wait gives up after `max_tries` polls (1..2^20); the block then reports exactly like the tiled
 * kernels (ca_stage_timeouts grows by one, bit 0 of the registered status word is set), writes
 * 1 to `out` (nullable device int32; 0 would mean the wait completed) and returns.  Nothing
 * traps, faults or waits without a limit. */
int ca_probe_stage_timeout(int32_t max_tries, int32_t* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif
