/* The solo / majority allreduce schedules of the host operation runtime from a C program.  Ranks are pthreads of one
 * "world"; every rank is late by `rank` milliseconds in every iteration, posts the persistent schedule, waits, and
 * reads the result together with the number of ranks that put something new into the round — the loop of the
 * reference's evaluation/rsgd.c and randomsgd.c (fflib2 evaluation/rsgd.c:66-113), where the calls are
 * ffsolo_allreduce / ffschedule_start / ffschedule_post / ffschedule_wait.
 *
 *   cc rt_partial_allreduce.c $(pkg-config --cflags --libs esgd_host) -lpthread -o rt_partial_allreduce
 *   ./rt_partial_allreduce [ranks] [count] [iters] [mode: 0 solo, 1 majority] [limiter]
 */
#include <host/oprt.h>
#include <pthread.h>
#include <stdio.h>
#include <stdlib.h>
#include <time.h>
#include <unistd.h>

#define MAX_RANKS 16
static int P = 4, ITERS = 12, MODE = 0, LIMITER = 5;
static int64_t COUNT = 1024;
static rt_world* world;
static double wait_us[MAX_RANKS], total[MAX_RANKS];
static int64_t info[MAX_RANKS][9];
static int failed[MAX_RANKS];
static pthread_barrier_t barrier;

static double now_us(void) {
  struct timespec t;
  clock_gettime(CLOCK_MONOTONIC, &t);
  return t.tv_sec * 1e6 + t.tv_nsec / 1e3;
}

/* hung on the schedule's end operation: runs on the rank's progress thread once per round */
typedef struct { rt_rank* c; rt_sched s; float* scratch; double sum; int rounds; } watcher;
static void round_ended(rt_op op, void* arg) {
  watcher* w = (watcher*)arg;
  int64_t contributors = 0, round = 0;
  (void)op;
  if (rt_partial_read(w->c, w->s, w->scratch, &contributors, &round) != RT_SUCCESS) return;
  w->sum += w->scratch[0];                       /* every element of a round's result is the same number */
  w->rounds++;
}

static void* rank_main(void* arg) {
  const int rank = (int)(intptr_t)arg;
  rt_rank* c = rt_world_rank(world, rank);
  float* grad = malloc(COUNT * sizeof(float));
  float* avg = calloc(COUNT, sizeof(float));
  float* scratch = calloc(COUNT, sizeof(float));
  rt_buf bg = rt_buffer_create(c, grad, COUNT, RT_FLOAT), ba = rt_buffer_create(c, avg, COUNT, RT_FLOAT);
  /* RT_PARTIAL_ACCUMULATE: a contribution that no round has taken yet is added to the next one, so nothing is lost */
  rt_sched s = MODE == 0 ? rt_solo_allreduce(c, bg, ba, 7, RT_SUM, LIMITER, RT_PARTIAL_ACCUMULATE)
                         : rt_rand_allreduce(c, bg, ba, 7, RT_SUM, 6545343, LIMITER, RT_PARTIAL_ACCUMULATE);
  watcher w = {c, s, scratch, 0.0, 0};
  rt_op watch = rt_op_callback(c, round_ended, &w, RT_DEP_OR);
  rt_op_hb(c, rt_schedule_end_op(c, s), watch);
  if (s < 0 || rt_schedule_start(c, s) != RT_SUCCESS) failed[rank] = 1;
  pthread_barrier_wait(&barrier);
  for (int it = 0; it < ITERS && !failed[rank]; ++it) {
    usleep(1000 * rank);
    for (int64_t k = 0; k < COUNT; ++k) grad[k] = 1.0f;
    const double t0 = now_us();
    if (rt_schedule_post(c, s) != RT_SUCCESS || rt_schedule_wait(c, s, 30.0) != RT_SUCCESS) failed[rank] = 1;
    wait_us[rank] += now_us() - t0;
    for (int64_t k = 0; k < COUNT; ++k) grad[k] = 0.0f;   /* the contribution was copied inside post */
  }
  for (int spin = 0; spin < 100000 && rt_op_completions(c, watch) < ITERS; ++spin) usleep(100);
  pthread_barrier_wait(&barrier);
  if (w.rounds != ITERS || rt_partial_info(c, s, info[rank]) != RT_SUCCESS) failed[rank] = 1;
  total[rank] = w.sum;
  rt_schedule_delete(c, s);
  rt_op_free(c, watch);
  free(grad); free(avg); free(scratch);
  return NULL;
}

int main(int argc, char** argv) {
  if (argc > 1) P = atoi(argv[1]);
  if (argc > 2) COUNT = atol(argv[2]);
  if (argc > 3) ITERS = atoi(argv[3]);
  if (argc > 4) MODE = atoi(argv[4]);
  if (argc > 5) LIMITER = atoi(argv[5]);
  if (P < 1 || P > MAX_RANKS || COUNT < 1 || LIMITER < 0 || ITERS % (LIMITER + 1) != 0) {
    fprintf(stderr, "ranks 1..%d; iters a multiple of limiter + 1 (the last round is then a synchronous one)\n", MAX_RANKS);
    return 2;
  }
  world = rt_world_create(P);
  pthread_barrier_init(&barrier, NULL, P);
  pthread_t th[MAX_RANKS];
  for (int r = 0; r < P; ++r) pthread_create(&th[r], NULL, rank_main, (void*)(intptr_t)r);
  for (int r = 0; r < P; ++r) pthread_join(th[r], NULL);
  int bad = 0;
  for (int r = 0; r < P; ++r) {
    printf("rank %d: %.1f us per post + wait, activated %ld rounds, found %ld already begun, %ld synchronous\n", r,
           wait_us[r] / ITERS, (long)info[r][2], (long)info[r][3], (long)info[r][4]);
    /* every rank saw every round, and the rounds together hold every post of every rank exactly once */
    if (failed[r] || total[r] != (double)P * ITERS || info[r][1] != ITERS || info[r][8] != 0) bad = 1;
  }
  rt_world_destroy(world);
  printf("%s allreduce, %d ranks x %d posts of %ld floats: sum over all rounds = %.0f on every rank (%d x %d expected) %s\n",
         MODE == 0 ? "solo" : "majority", P, ITERS, (long)COUNT, total[0], P, ITERS, bad ? "FAILED" : "PASSED");
  return bad;
}
