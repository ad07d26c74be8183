// Stress driver for the host control plane, meant to be built with -fsanitize=thread (or address):
//   g++ -std=c++17 -O1 -g -fsanitize=thread stress_main.cpp cpu_channel.cpp oprt.cpp -lpthread -o stress && ./stress
// Part 1 runs the partial-allreduce protocol (the very source the CUDA kernels compile) as threads of
// one process in all three modes with random arrival skew, and checks that every rank applied the same
// total and that no status bit was raised.  Part 2 posts a persistent allreduce schedule of the
// operation runtime many times from every rank.  The reference has no sanitizer or race-detection
// build (fflib2 CMakeLists.txt has only -O3 / -DFFDEBUG); this is the race check of this framework's
// host code, and because the device kernels share step.h, of their protocol logic too.
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <chrono>
#include <thread>
#include <vector>
#include "oprt.h"

extern "C" {
struct esgd_step_info {
  int32_t role, n_contrib, n_fresh, is_sync;
  uint32_t status;
  float drain_rounds;
  uint64_t round, local_step;
};
struct esgd_cpu_params {
  int32_t rank, world, base_mode, include_stale, average, home, dtype, flags;
  int64_t limiter;
  uint64_t seed, timeout_ns, grace_ns, count;
};
uint64_t esgd_cpu_segment_bytes(uint64_t count, int dtype);
uint32_t esgd_cpu_step(void** bases, const esgd_cpu_params* p, const void* grad, void* out, esgd_step_info* info);
uint32_t esgd_cpu_flush(void** bases, const esgd_cpu_params* p, void* out, esgd_step_info* info);
}

static int run_channel(int mode, int world, int steps, uint64_t count, int flags) {
  const uint64_t bytes = esgd_cpu_segment_bytes(count, 0);
  std::vector<void*> bases(world);
  for (int r = 0; r < world; ++r) {
    if (posix_memalign(&bases[r], 256, bytes) != 0) return 1;
    memset(bases[r], 0, bytes);
  }
  std::vector<double> totals(world, 0.0);
  std::vector<uint32_t> status(world, 0);
  std::vector<std::thread> th;
  for (int r = 0; r < world; ++r) {
    th.emplace_back([&, r] {
      esgd_cpu_params p;
      memset(&p, 0, sizeof(p));
      p.rank = r; p.world = world; p.base_mode = mode; p.include_stale = 1; p.average = 2 /* sum */; p.home = 0;
      p.dtype = 0; p.flags = flags; p.limiter = 4; p.seed = 6545343; p.timeout_ns = 20ull * 1000000000ull; p.grace_ns = 0; p.count = count;
      std::vector<float> grad(count), out(count);
      unsigned seed = 1234u + (unsigned)r;
      esgd_step_info info;
      for (int k = 0; k < steps; ++k) {
        if (rand_r(&seed) % 4 == 0) std::this_thread::sleep_for(std::chrono::microseconds(rand_r(&seed) % 300));
        for (uint64_t e = 0; e < count; ++e) grad[e] = 1.0f;
        status[r] |= esgd_cpu_step(bases.data(), &p, grad.data(), out.data(), &info);
        totals[r] += out[0];
        for (uint64_t e = 1; e < count; ++e)
          if (out[e] != out[0]) status[r] |= 0x80000000u;      // a torn result
      }
      status[r] |= esgd_cpu_flush(bases.data(), &p, out.data(), &info);
      totals[r] += out[0];
    });
  }
  for (auto& t : th) t.join();
  int bad = 0;
  for (int r = 0; r < world; ++r) {
    if (status[r] != 0 || totals[r] != totals[0]) {
      fprintf(stderr, "mode %d rank %d: status %x total %.1f (rank 0: %.1f)\n", mode, r, status[r], totals[r], totals[0]);
      bad = 1;
    }
    free(bases[r]);
  }
  printf("channel mode %d: %d ranks x %d steps, total applied %.0f on every rank\n", mode, world, steps, totals[0]);
  return bad;
}

static int run_runtime(int world, int posts) {
  rt_world* w = rt_world_create(world);
  std::vector<int> bad(world, 0);
  std::vector<std::thread> th;
  for (int r = 0; r < world; ++r) {
    th.emplace_back([&, r] {
      rt_rank* c = rt_world_rank(w, r);
      std::vector<int32_t> snd(64), rcv(64);
      rt_buf bs = rt_buffer_create(c, snd.data(), 64, RT_INT32), br = rt_buffer_create(c, rcv.data(), 64, RT_INT32);
      rt_sched s = rt_allreduce(c, bs, br, 3, RT_SUM);
      for (int it = 0; it < posts; ++it) {
        for (int e = 0; e < 64; ++e) snd[e] = e + it + r;
        rt_schedule_post(c, s);
        if (rt_schedule_wait(c, s, 30.0) != RT_SUCCESS) { bad[r] = 1; break; }
        for (int e = 0; e < 64; ++e)
          if (rcv[e] != (e + it) * world + world * (world - 1) / 2) bad[r] = 1;
      }
    });
  }
  for (auto& t : th) t.join();
  rt_world_destroy(w);
  int any = 0;
  for (int r = 0; r < world; ++r) any |= bad[r];
  printf("runtime allreduce: %d ranks x %d posts %s\n", world, posts, any ? "FAILED" : "ok");
  return any;
}

// Fresh schedules every iteration: create, post, wait, delete (handles and temporaries are recycled), and the
// persistent form, through the runtime's own native benchmark; the results are checked inside.
static int run_schedule_cycles(int world) {
  double out[3] = {0, 0, 0};
  int bad = 0;
  for (int fresh = 0; fresh < 2; ++fresh) {
    if (rt_bench_allreduce(world, 96, 48, fresh, out) != RT_SUCCESS || out[2] != 1.0) bad = 1;
  }
  printf("runtime schedule cycles: %d ranks %s\n", world, bad ? "FAILED" : "ok");
  return bad;
}

// Solo and majority allreduce as runtime schedules: ranks arrive with random skew, an observer on the schedule's end
// records every round, schedules are created and deleted in cycles with one tag.  Checked: every rank ran every round,
// the rounds agree across ranks, and with accumulation on and a synchronous last round no post was lost.
struct RoundLog { std::vector<int64_t> value, contributors, scratch; rt_rank* c; rt_sched s; int torn = 0; };
static void observe_round(rt_op, void* arg) {
  RoundLog* log = (RoundLog*)arg;
  int64_t k = 0, rnd = 0;
  if (rt_partial_read(log->c, log->s, log->scratch.data(), &k, &rnd) != RT_SUCCESS) return;
  if (log->scratch.front() != log->scratch.back()) log->torn = 1;
  log->value.push_back(log->scratch[0]);
  log->contributors.push_back(k);
}

static int run_partial(int world, int cycles, int steps, int64_t count) {
  rt_world* w = rt_world_create(world);
  std::vector<int> bad(world, 0);
  std::vector<std::vector<RoundLog>> logs(world, std::vector<RoundLog>(cycles));
  std::vector<std::thread> th;
  const int limiter = 3;                              // steps is a multiple of 4: the last round is synchronous
  for (int r = 0; r < world; ++r) {
    th.emplace_back([&, r] {
      rt_rank* c = rt_world_rank(w, r);
      uint64_t rng = 0x243f6a8885a308d3ULL * (uint64_t)(r + 1);
      for (int cy = 0; cy < cycles && !bad[r]; ++cy) {
        std::vector<int64_t> snd(count, r + 1), rcv(count, 0);
        rt_buf bs = rt_buffer_create(c, snd.data(), count, RT_INT64), br = rt_buffer_create(c, rcv.data(), count, RT_INT64);
        rt_sched s = (cy & 1) ? rt_rand_allreduce(c, bs, br, 11, RT_SUM, cy, limiter, RT_PARTIAL_ACCUMULATE)
                              : rt_solo_allreduce(c, bs, br, 11, RT_SUM, limiter, RT_PARTIAL_ACCUMULATE);
        RoundLog& log = logs[r][cy];
        log.c = c; log.s = s; log.scratch.assign(count, 0);
        rt_op obs = rt_op_callback(c, observe_round, &log, RT_DEP_OR);
        rt_op_hb(c, rt_schedule_end_op(c, s), obs);
        rt_schedule_start(c, s);
        for (int it = 0; it < steps; ++it) {
          rng = rng * 6364136223846793005ULL + 1442695040888963407ULL;
          if (((rng >> 33) & 3) == 0) std::this_thread::sleep_for(std::chrono::microseconds((rng >> 40) & 255));
          if (rt_schedule_post(c, s) != RT_SUCCESS || rt_schedule_wait(c, s, 30.0) != RT_SUCCESS) { bad[r] = 1; break; }
        }
        for (int spin = 0; spin < 200000 && rt_op_completions(c, obs) < steps; ++spin) std::this_thread::yield();
        if (rt_op_completions(c, obs) != steps || log.torn) bad[r] = 1;
        int64_t info[9];
        if (rt_partial_info(c, s, info) != RT_SUCCESS || info[1] != steps || info[7] != 0 || info[8] != 0) bad[r] = 1;
        rt_schedule_delete(c, s);
        rt_op_free(c, obs);
        rt_buffer_delete(c, bs);
        rt_buffer_delete(c, br);
      }
    });
  }
  for (auto& t : th) t.join();
  rt_world_destroy(w);
  int any = 0;
  for (int r = 0; r < world; ++r) any |= bad[r];
  for (int cy = 0; cy < cycles && !any; ++cy) {
    int64_t total = 0;
    for (int it = 0; it < steps; ++it) {
      for (int r = 1; r < world; ++r)
        if (logs[r][cy].value[it] != logs[0][cy].value[it] || logs[r][cy].contributors[it] != logs[0][cy].contributors[it]) any = 1;
      total += logs[0][cy].value[it];
    }
    if (logs[0][cy].contributors[steps - 1] != world) any = 1;
    if (total != (int64_t)steps * world * (world + 1) / 2) any = 1;
  }
  printf("runtime partial allreduce: %d ranks x %d cycles x %d posts of %ld elements %s\n", world, cycles, steps, (long)count,
         any ? "FAILED" : "ok");
  return any;
}

int main(int argc, char** argv) {
  const int world = argc > 1 ? atoi(argv[1]) : 4;
  const int steps = argc > 2 ? atoi(argv[2]) : 200;
  int bad = 0;
  for (int mode = 0; mode < 3; ++mode) bad |= run_channel(mode, world, steps, 1024, 2);
  for (int mode = 0; mode < 2; ++mode) bad |= run_channel(mode, world, steps, 1024, 3);   // folding unconsumed gradients
  bad |= run_runtime(world, steps / 4 + 1);
  bad |= run_schedule_cycles(world);
  bad |= run_partial(world, 6, 16, 8);
  bad |= run_partial(world, 2, 8, 8192);               // bodies large enough to be copied straight into a listening receive
  // vectors long enough for a rank's helper threads (from 256 K elements each), with a ragged length
  bad |= run_channel(2, 2, 3, (1u << 20) + 1234, 0);
  bad |= run_channel(0, 2, 3, (1u << 20) + 1234, 1);
  return bad;
}
