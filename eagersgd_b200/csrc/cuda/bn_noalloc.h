/* Batch-norm forward (+ optional residual add, + optional ReLU) that allocates nothing.
 *
 * This entry point has no counterpart in the reference; it exists for callers of this
 * library that are not able to obtain device memory at the moment they need the op:
 *   - a process that has handed the whole GPU to a memory pool of its own (a serving
 *     stack, another framework's caching allocator), so that a fresh cudaMalloc fails;
 *   - code running at a point where calling into an allocator is forbidden or too slow,
 *     e.g. a latency-critical loop that must not take the driver's allocation lock or the
 *     device-wide synchronisation a cudaMalloc / cudaFree implies;
 *   - plain C callers that link the shared library without PyTorch and therefore have no
 *     tensor allocator at all.
 * The regular path (esgd_bn_stats + esgd_bn_finalize + esgd_bn_apply) needs six per-channel
 * fp32 work arrays that its caller must allocate.  Here those arrays live in a fixed
 * device-resident block inside the library instead.
 *
 * Limits and rules
 *   - C (channels) must be a multiple of 8 and at most ESGD_BN_NOALLOC_MAX_CHANNELS; larger
 *     layers are rejected with ESGD_BN_NOALLOC_TOO_MANY_CHANNELS.  The block costs
 *     6 * 4096 * 4 bytes = 96 KiB on every GPU that loads the library, until the process exits.
 *   - The first call on each device looks up the block's device address (with that device
 *     current).  Make that first call outside of any stream capture.
 *   - Every call uses the same block and finds in it whatever the previous call left; the
 *     function clears the accumulators it needs at zero itself.  Two calls that may overlap on
 *     the GPU (different streams without an ordering between them) race on the block: order
 *     them.
 *   - Inputs and outputs are still the caller's: y, residual (may be NULL) and z are bf16
 *     [M, C] row-major (NHWC activations), gamma / beta fp32 [C]; running_mean / running_var
 *     (fp32 [C]) may be NULL.  momentum is the weight of the new batch statistic.
 *   - y, residual and z must start on a 16-byte boundary (the kernels move eight bf16 values
 *     per access); a pointer that does not is refused with ESGD_BN_NOALLOC_BAD_ARGUMENT, as is
 *     a channel count that is not a multiple of 8.
 * Returns 0 on success, a negative ESGD_BN_NOALLOC_* code, or a positive cudaError_t.
 */
#ifndef ESGD_BN_NOALLOC_H
#define ESGD_BN_NOALLOC_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ESGD_BN_NOALLOC_MAX_CHANNELS 4096
#define ESGD_BN_NOALLOC_BAD_ARGUMENT (-1)
#define ESGD_BN_NOALLOC_TOO_MANY_CHANNELS (-2)
#define ESGD_BN_NOALLOC_SETUP_FAILED (-3)

int esgd_bn_forward_noalloc(const void* y, const void* residual, void* z, const float* gamma, const float* beta,
                            float* running_mean, float* running_var, int64_t M, int C, int relu, float momentum,
                            float eps, void* stream);

/* Human-readable text for a return code of the function above. */
const char* esgd_bn_forward_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
#endif
