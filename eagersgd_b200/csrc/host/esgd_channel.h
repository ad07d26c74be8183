/* Partial allreduce on the CPU for C and C++ programs: solo, majority and synchronous averaging of one vector per
 * "channel" between ranks that share memory (threads of one process, or processes over POSIX shared memory).
 *
 * It stands where a C user of the reference calls ffsolo_allreduce / ffrand_allreduce / ffallreduce and posts and
 * waits on the returned schedule (fflib2 src/ff.h:137-165, evaluation/rsgd.c:77-113).  Here a channel is a set of
 * memory segments, one per rank, that every rank can address; a step of a rank is ONE call that publishes its
 * vector, takes part in the round that is open (or opens one, or learns that it missed it), and returns the
 * averaged vector to apply — there is no progress thread: whoever is in a round does the reduction.
 *
 *   uint64_t bytes = esgd_cpu_segment_bytes(count, ESGD_F32);
 *   for every rank r: bases[r] = <zeroed, 256-byte aligned memory of `bytes` bytes that all ranks can reach>
 *   esgd_cpu_params p = {rank, world, ESGD_MODE_SOLO, 1, ESGD_AVG_CONTRIBUTORS, 0, ESGD_F32, 0, 32, seed,
 *                        timeout_ns, 0, count};
 *   every iteration:  status = esgd_cpu_step(bases, &p, grad, out, &info);     // out: what to apply now
 *   at the end:       esgd_cpu_flush(bases, &p, out, &info);                   // rounds that finished after the last step
 *
 * Link with `pkg-config --cflags --libs esgd_host`.  Every wait inside is bounded by timeout_ns; a non-zero return
 * value is a set of ESGD_ST_* bits (sticky in the rank's segment until esgd_ctl_clear_status).
 */
#ifndef ESGD_CHANNEL_H
#define ESGD_CHANNEL_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { ESGD_F32 = 0, ESGD_F64 = 1, ESGD_I32 = 2, ESGD_I64 = 3 };                  /* element types (integers: sums only) */
enum { ESGD_MODE_SOLO = 0, ESGD_MODE_MAJORITY = 1, ESGD_MODE_SYNC = 2 };
enum { ESGD_AVG_CONTRIBUTORS = 0, ESGD_AVG_WORLD = 1, ESGD_AVG_SUM = 2 };         /* divide by what a round summed / by the world (reference) / not at all */
enum { ESGD_ROLE_ABORT = 0, ESGD_ROLE_PARTICIPANT = 1, ESGD_ROLE_DRAIN = 2, ESGD_ROLE_IDLE = 3 };
#define ESGD_FLAG_ACCUMULATE 1u      /* fold a gradient that no round picked up into the rank's next one */
#define ESGD_FLAG_ADAPTIVE_GRACE 2u  /* the grace window follows the observed spread of arrivals */

typedef struct esgd_cpu_params {
  int32_t rank, world, base_mode, include_stale, average, home, dtype;
  int32_t flags;
  int64_t limiter;                 /* eager rounds between two forced synchronous ones (< 0: never force) */
  uint64_t seed, timeout_ns, grace_ns, count;
} esgd_cpu_params;

typedef struct esgd_step_info {
  int32_t role;                    /* ESGD_ROLE_* of this step */
  int32_t n_contrib;               /* gradients summed by the round applied */
  int32_t n_fresh;                 /* ranks that took part in it */
  int32_t is_sync;                 /* the round waited for everybody */
  uint32_t status;
  float drain_rounds;              /* rounds collected at once by a rank that had missed them */
  uint64_t round;
  uint64_t local_step;
} esgd_step_info;

uint64_t esgd_cpu_segment_bytes(uint64_t count, int dtype);
void esgd_cpu_segment_init(void* base, uint64_t bytes);                      /* zero a segment */
uint32_t esgd_cpu_step(void** bases, const esgd_cpu_params* p, const void* grad, void* out, esgd_step_info* info);
uint32_t esgd_cpu_flush(void** bases, const esgd_cpu_params* p, void* out, esgd_step_info* info);
int32_t esgd_majority_initiator(uint64_t seed, uint64_t round, int32_t world);   /* who opens round `round` in majority mode */
int32_t esgd_limiter_is_sync(uint64_t step, int64_t limiter);                   /* is step `step` a forced synchronous one */
/* stats[0..12]: steps, participated, absent, activated, synchronous rounds, dropped gradients, sum of contributors,
 * nanoseconds waited, last round, last contributors, status, newest round seen, folded gradients (24 words are written) */
void esgd_ctl_stats(const void* base, uint64_t* stats);
int32_t esgd_ctl_trace(const void* base, uint64_t* rows, int32_t max_rows);     /* rows of 10 words, oldest first */
void esgd_ctl_clear_status(void* base);

#ifdef __cplusplus
}
#endif
#endif
