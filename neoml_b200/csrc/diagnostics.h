/* Diagnostic entry points of libneoml_b200.so.  They are exported for the benchmark and the tests of this
 * repository and are NOT part of the product interface (include/neoml_b200.h): they keep process-wide state that
 * changes how every later contraction launch in the process is issued or observed. */
#pragma once

#include "../../include/neoml_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Diagnostic aid: when device_buffer is non-NULL, CTA 0 of every later contraction launch stores clock64() stamps of
 * its pipeline roles at device_buffer[kind * steps + index] (16 stamp kinds, 8-byte words; kinds 0-6 and 15 are indexed
 * by K-block step, 7-14 by tile; indices >= steps are dropped).  options bit 4 (value 16): use the cp.async gather
 * kernel even where TMA applies (results are the same; for timing and testing that path).  options bit 5 (value 32):
 * never split the K loop of a few-tile convolution; bit 6 (64): ordinary launches instead of programmatic dependent
 * ones; bit 7 (128): no short-K kernel variant (resident B, residual ring).  (NULL, 0, 0) = normal. */
NB200_API void nb200_debug_set_contraction_trace(void* device_buffer, int steps, int options);
/* Diagnostic aid for benchmarks: while enabled, every contraction launch (the tensor-core kernel with its split-K
 * finishing pass; not the operand preparation before it) is bracketed by a pair of CUDA events on its stream.  Enabling
 * clears the list.  nb200_debug_contraction_times waits for the recorded launches and writes their durations in
 * milliseconds, in launch order; returns how many it wrote (at most `capacity`), negative on a CUDA error.  The event
 * records keep neighbouring kernels from overlapping, so a timed pass runs a little slower than an untimed one. */
NB200_API void nb200_debug_time_contractions(int enable);
NB200_API int nb200_debug_contraction_times(float* ms, int capacity);
/* The same with, beside each duration, the algorithmic flops (2*M*N*K, counted once, no credit for padding) of the
 * entry-point call the launch belongs to. */
NB200_API int nb200_debug_contraction_records(float* ms, double* flops, int capacity);
/* Launches one warp that waits, with the library's bounded wait, on a barrier nothing completes; after limit_ns
 * (at most one second) the wait gives up, the device status word receives 0x7e01 and the kernel returns.  Lets a test
 * walk the time-out path (status word, NB200_EDEVICE, the engine's report) without hanging anything. */
NB200_API int nb200_debug_wait_probe(void* stream, unsigned long long limit_ns);

#ifdef __cplusplus
}
#endif
