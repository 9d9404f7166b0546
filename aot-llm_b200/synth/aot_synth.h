/* Synthetic weights for tests and benchmarks: host-only helpers, built into their own
 * small library (libaot_synth.so) so that nothing but the forward path lives in
 * libaot_cuda.so. Kind ids and status codes are those of include/aot_cuda.h. */
#ifndef AOT_SYNTH_H
#define AOT_SYNTH_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* ---- synthetic test data (the encoders of crates/aot-kernels/src/quantize.rs) */
/* quantize_row (quantize.rs:16-294): encodes n floats as one row of `kind` into
 * out (row_bytes(kind, n) bytes). Host memory, CPU code: this is data
 * generation for tests and benchmarks, not part of the forward pass. */
int aotcu_synth_quantize_row(int kind, const float* x, size_t n, uint8_t* out);
/* Fills `rows` x `cols` weights drawn uniform in (-amp, amp) from a counter-based
 * generator keyed by `seed`, encoded as `kind`, multi-threaded. */
int aotcu_synth_tensor(int kind, size_t rows, size_t cols, float amp, float offset, uint64_t seed, uint8_t* out);
/* Fills `n_blocks` blocks of `kind` with field-uniform random content (f16
 * scales uniform in [1e-3, 1e-2], quant bytes uniform), as the single-kernel
 * benchmark configurations specify. */
int aotcu_synth_blocks(int kind, size_t n_blocks, uint64_t seed, uint8_t* out);

#ifdef __cplusplus
}
#endif
#endif
