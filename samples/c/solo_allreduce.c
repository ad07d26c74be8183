/* Solo (or majority, or synchronous) averaging from a C program: ranks are pthreads, every rank is skewed by
 * `rank` milliseconds per iteration and times one collective — the loop of the reference's evaluation/rsgd.c
 * (fflib2 evaluation/rsgd.c:77-113), written against esgd_channel.h.
 *
 *   cc solo_allreduce.c $(pkg-config --cflags --libs esgd_host) -o solo_allreduce
 *   ./solo_allreduce [ranks] [count] [iters] [mode: 0 solo, 1 majority, 2 sync]
 */
#include <host/esgd_channel.h>
#include <pthread.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>
#include <unistd.h>

#define MAX_RANKS 16
static int P = 4, ITERS = 10, MODE = ESGD_MODE_SOLO;
static uint64_t COUNT = 1024;
static void* bases[MAX_RANKS];
static double latency_us[MAX_RANKS];
static uint64_t participated[MAX_RANKS], absent[MAX_RANKS];
static double applied[MAX_RANKS];
static pthread_barrier_t barrier;

static double now_us(void) {
  struct timespec t;
  clock_gettime(CLOCK_MONOTONIC, &t);
  return t.tv_sec * 1e6 + t.tv_nsec / 1e3;
}

static void* rank_main(void* arg) {
  const int rank = (int)(intptr_t)arg;
  esgd_cpu_params p;
  memset(&p, 0, sizeof(p));
  p.rank = rank; p.world = P; p.base_mode = MODE; p.include_stale = 1; p.average = ESGD_AVG_SUM; p.dtype = ESGD_F32;
  p.limiter = 1024; p.seed = 6545343; p.timeout_ns = 30ull * 1000000000ull; p.count = COUNT;
  float* grad = malloc(COUNT * sizeof(float));
  float* out = malloc(COUNT * sizeof(float));
  esgd_step_info info;
  double total = 0, sum = 0;
  pthread_barrier_wait(&barrier);
  for (int it = 0; it < ITERS; ++it) {
    for (uint64_t j = 0; j < COUNT; ++j) grad[j] = 1.0f;          /* every rank contributes 1 per step */
    usleep(rank * 1000);
    const double t0 = now_us();
    if (esgd_cpu_step(bases, &p, grad, out, &info) != 0) { fprintf(stderr, "rank %d: status %u\n", rank, info.status); exit(2); }
    total += now_us() - t0;
    sum += out[0];
  }
  pthread_barrier_wait(&barrier);                                  /* everybody has posted its last gradient */
  esgd_cpu_flush(bases, &p, out, &info);
  sum += out[0];
  uint64_t st[24];
  esgd_ctl_stats(bases[rank], st);
  latency_us[rank] = total / ITERS;
  participated[rank] = st[1];
  absent[rank] = st[2];
  applied[rank] = sum;
  free(grad);
  free(out);
  return NULL;
}

int main(int argc, char** argv) {
  if (argc > 1) P = atoi(argv[1]);
  if (argc > 2) COUNT = strtoull(argv[2], NULL, 10);
  if (argc > 3) ITERS = atoi(argv[3]);
  if (argc > 4) MODE = atoi(argv[4]);
  if (P < 1 || P > MAX_RANKS) return 1;
  const uint64_t bytes = esgd_cpu_segment_bytes(COUNT, ESGD_F32);
  for (int r = 0; r < P; ++r) {
    if (posix_memalign(&bases[r], 256, bytes) != 0) return 1;
    esgd_cpu_segment_init(bases[r], bytes);
  }
  pthread_barrier_init(&barrier, NULL, P);
  pthread_t th[MAX_RANKS];
  for (int r = 0; r < P; ++r) pthread_create(&th[r], NULL, rank_main, (void*)(intptr_t)r);
  for (int r = 0; r < P; ++r) pthread_join(th[r], NULL);
  double mean = 0;
  int same = 1;
  for (int r = 0; r < P; ++r) {
    mean += latency_us[r] / P;
    if (applied[r] != applied[0]) same = 0;
    printf("rank %d: %.1f us per collective, took part in %llu rounds, missed %llu, total applied %.0f\n", r, latency_us[r],
           (unsigned long long)participated[r], (unsigned long long)absent[r], applied[r]);
  }
  printf("mode %d, %d ranks, %llu floats: mean latency %.1f us; replicas %s\n", MODE, P, (unsigned long long)COUNT, mean,
         same ? "agree" : "DIFFER");
  /* with sums and nothing dropped every replica must have applied every gradient exactly once */
  const double expect = (double)P * ITERS;
  if (!same) return 3;
  if (MODE == ESGD_MODE_SYNC && applied[0] != expect) return 4;
  printf("%s\n", "PASSED");
  return 0;
}
