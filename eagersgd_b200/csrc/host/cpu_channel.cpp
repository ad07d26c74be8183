// CPU backend of the partial allreduce: the same control protocol as the CUDA
// kernels (protocol/step.h), instantiated with host atomics over memory shared
// by the ranks (threads of one process, or processes mapping POSIX shared
// memory).  It replaces the reference's host path (fflib2 over MPI:
// src/colls/ffsolo_allreduce.c, ffrand_allreduce.c, ffallreduce.c) for CPU runs
// and is the oracle the GPU kernels are tested against.
//
// Segment of one rank for one channel:  [ChannelCtl | slot 0 | slot 1 | mailbox]
#include <stdint.h>
#include <string.h>
#include <stdlib.h>
#include <thread>
#include <vector>
#include "../protocol/channel.h"
#include "../protocol/step.h"
#include "../protocol/env_host.h"
#include "esgd_channel.h"

using namespace esgd;

namespace {

inline uint64_t align_up(uint64_t x, uint64_t a) { return (x + a - 1) / a * a; }

struct SegLayout {
  uint64_t slot_off[2];
  uint64_t mbox_off;
  uint64_t total;
};

SegLayout layout_for(uint64_t count, int elem_size) {
  SegLayout L;
  uint64_t off = align_up(sizeof(ChannelCtl), 256);
  uint64_t bytes = align_up(count * (uint64_t)elem_size, 256);
  L.slot_off[0] = off; off += bytes;
  L.slot_off[1] = off; off += bytes;
  L.mbox_off = off; off += bytes;
  L.total = off;
  return L;
}

enum DType { DT_F32 = 0, DT_F64 = 1, DT_I32 = 2, DT_I64 = 3 };
int dtype_size(int dt) { return (dt == DT_F32 || dt == DT_I32) ? 4 : 8; }

template <class T> struct IsFloat { static const bool v = false; };
template <> struct IsFloat<float> { static const bool v = true; };
template <> struct IsFloat<double> { static const bool v = true; };

// Large vectors are worked on by a few threads of the rank: one core does not reach the memory bandwidth of the
// host.  ESGD_CPU_THREADS sets the number (default: the cores divided among the ranks of the world, at most 4);
// ranges below 256 K elements per thread stay on the calling thread.
int data_threads(int world) {
  static const int forced = [] { const char* e = getenv("ESGD_CPU_THREADS"); return e ? atoi(e) : 0; }();
  if (forced > 0) return forced;
  int hw = (int)std::thread::hardware_concurrency();
  int t = hw / (world > 0 ? world : 1);
  return t < 1 ? 1 : (t > 4 ? 4 : t);
}

template <class F>
void parallel_ranges(uint64_t lo, uint64_t hi, int world, F fn) {
  const uint64_t n = hi > lo ? hi - lo : 0;
  int t = data_threads(world);
  const uint64_t kMinPerThread = 1u << 18;
  if ((uint64_t)t > n / kMinPerThread) t = (int)(n / kMinPerThread);
  if (t <= 1) { fn(lo, hi); return; }
  const uint64_t per = ((n + t - 1) / t + 1023) / 1024 * 1024;      // whole blocks of the reduction loop
  std::vector<std::thread> th;
  for (int i = 1; i < t; ++i) {
    const uint64_t a = lo + per * i, b = a + per < hi ? a + per : hi;
    if (a < hi) th.emplace_back([=] { fn(a, b); });
  }
  fn(lo, lo + per < hi ? lo + per : hi);
  for (auto& x : th) x.join();
}

// Participant: out = scale * sum(contributor slots); this participant's share of
// the vector is also delivered to the mailbox of every absent rank.
template <class T>
void data_participant(void** bases, const SegLayout& L, const Plan& plan, uint64_t count, T* out, int world) {
  const T* src[kMaxRanks];
  for (int s = 0; s < plan.n_src; ++s)
    src[s] = (const T*)((char*)bases[plan.src_rank[s]] + L.slot_off[plan.src_parity[s]]);
  const T scale = IsFloat<T>::v ? (T)plan.scale : (T)1;
  const int n_src = plan.n_src;
  parallel_ranges(0, count, world, [&](uint64_t lo, uint64_t hi) {
    const uint64_t BLK = 1024;
    for (uint64_t b = lo; b < hi; b += BLK) {      // the same blocks and the same order of additions on any thread count
      uint64_t n = hi - b < BLK ? hi - b : BLK;
      T acc[BLK];
      for (uint64_t e = 0; e < n; ++e) acc[e] = src[0][b + e];
      for (int s = 1; s < n_src; ++s)
        for (uint64_t e = 0; e < n; ++e) acc[e] += src[s][b + e];
      for (uint64_t e = 0; e < n; ++e) out[b + e] = acc[e] * scale;
    }
  });
  if (plan.n_push > 0) {
    uint64_t per = (count + plan.part_count - 1) / plan.part_count;
    uint64_t lo = per * (uint64_t)plan.part_index;
    uint64_t hi = lo + per < count ? lo + per : count;
    for (int n = 0; n < plan.n_push; ++n) {
      T* mb = (T*)((char*)bases[plan.push_rank[n]] + L.mbox_off);
      const bool accum = plan.push_accum[n];
      parallel_ranges(lo, hi, world, [&](uint64_t a, uint64_t b) {
        if (accum) for (uint64_t e = a; e < b; ++e) mb[e] += out[e];
        else for (uint64_t e = a; e < b; ++e) mb[e] = out[e];
      });
    }
  }
}

template <class T>
void fold_into(void* slot, const void* grad, uint64_t count, int world) {
  T* s = (T*)slot;
  const T* g = (const T*)grad;
  parallel_ranges(0, count, world, [&](uint64_t a, uint64_t b) { for (uint64_t e = a; e < b; ++e) s[e] += g[e]; });
}

void parallel_copy(void* dst, const void* src, uint64_t bytes, int world) {
  parallel_ranges(0, bytes / 4, world, [&](uint64_t a, uint64_t b) { memcpy((char*)dst + a * 4, (const char*)src + a * 4, (b - a) * 4); });
  if (bytes % 4) memcpy((char*)dst + bytes / 4 * 4, (const char*)src + bytes / 4 * 4, bytes % 4);
}

template <class T>
void run_data(void** bases, int rank, const SegLayout& L, const Plan& plan, uint64_t count, void* out, int world) {
  T* o = (T*)out;
  if (plan.role == ROLE_PARTICIPANT) data_participant<T>(bases, L, plan, count, o, world);
  else if (plan.role == ROLE_DRAIN) parallel_copy(o, (char*)bases[rank] + L.mbox_off, count * sizeof(T), world);
  else memset(o, 0, count * sizeof(T));
}

}  // namespace

// the public C interface: parameter and result records, enumerations, prototypes
static_assert((int)MODE_SOLO == ESGD_MODE_SOLO && (int)MODE_MAJORITY == ESGD_MODE_MAJORITY && (int)MODE_SYNC == ESGD_MODE_SYNC,
              "modes of the header and of the protocol differ");
static_assert((int)ROLE_ABORT == ESGD_ROLE_ABORT && (int)ROLE_PARTICIPANT == ESGD_ROLE_PARTICIPANT &&
              (int)ROLE_DRAIN == ESGD_ROLE_DRAIN && (int)ROLE_IDLE == ESGD_ROLE_IDLE, "roles differ");
static_assert((int)DT_F32 == ESGD_F32 && (int)DT_F64 == ESGD_F64 && (int)DT_I32 == ESGD_I32 && (int)DT_I64 == ESGD_I64,
              "element types differ");

extern "C" {

uint64_t esgd_ctl_bytes(void) { return sizeof(ChannelCtl); }

uint64_t esgd_cpu_segment_bytes(uint64_t count, int dtype) {
  return layout_for(count, dtype_size(dtype)).total;
}

void esgd_cpu_segment_init(void* base, uint64_t bytes) { memset(base, 0, bytes); }

int32_t esgd_majority_initiator(uint64_t seed, uint64_t round, int32_t world) {
  return majority_initiator(seed, round, world);
}

int32_t esgd_limiter_is_sync(uint64_t step, int64_t limiter) { return limiter_is_sync(step, limiter) ? 1 : 0; }

static void fill_view(ChannelView& v, void** bases, int world) {
  for (int j = 0; j < kMaxRanks; ++j) v.ctl[j] = nullptr;
  for (int j = 0; j < world; ++j) v.ctl[j] = (ChannelCtl*)bases[j];
}

// One complete step: publish `grad`, take part in (or absorb) a round, write the
// gradient to apply into `out`.  Returns the sticky status word (0 = fine).
uint32_t esgd_cpu_step(void** bases, const esgd_cpu_params* p, const void* grad, void* out,
                       esgd_step_info* info) {
  ChannelView v;
  fill_view(v, bases, p->world);
  ChannelCtl* me = v.ctl[p->rank];
  SegLayout L = layout_for(p->count, dtype_size(p->dtype));
  StepConfig cfg;
  cfg.rank = p->rank; cfg.world = p->world; cfg.average_world = p->average; cfg.home = p->home;
  cfg.timeout_ns = p->timeout_ns; cfg.grace_ns = p->grace_ns;
  StepPolicy pol;
  pol.base_mode = p->base_mode; pol.include_stale = p->include_stale; pol.limiter = p->limiter; pol.seed = p->seed;
  pol.accumulate = p->flags & 1; pol.adaptive_grace = (p->flags >> 1) & 1;

  Plan plan;
  memset(&plan, 0, sizeof(plan));
  uint64_t k = me->local_step + 1;
  if (wait_slot_free<HostEnv>(v, cfg, pol, k)) {
    void* slot = (char*)bases[p->rank] + L.slot_off[k % kSlotDepth];
    if (slot_fate<HostEnv>(me, pol, k) == SLOT_FOLD) {
      switch (p->dtype) {   // the gradient of epoch k-2 was never picked up: it rides along with this one
        case DT_F32: fold_into<float>(slot, grad, p->count, p->world); break;
        case DT_F64: fold_into<double>(slot, grad, p->count, p->world); break;
        case DT_I32: fold_into<int32_t>(slot, grad, p->count, p->world); break;
        default: fold_into<int64_t>(slot, grad, p->count, p->world); break;
      }
    } else {
      parallel_copy(slot, grad, p->count * (uint64_t)dtype_size(p->dtype), p->world);
    }
    ctl_step<HostEnv>(v, cfg, pol, &plan);
  } else {
    me->local_step = k;
    plan.role = ROLE_ABORT;
  }
  switch (p->dtype) {
    case DT_F32: run_data<float>(bases, p->rank, L, plan, p->count, out, p->world); break;
    case DT_F64: run_data<double>(bases, p->rank, L, plan, p->count, out, p->world); break;
    case DT_I32: run_data<int32_t>(bases, p->rank, L, plan, p->count, out, p->world); break;
    default: run_data<int64_t>(bases, p->rank, L, plan, p->count, out, p->world); break;
  }
  finish_step<HostEnv>(v, cfg, &plan);
  if (info) {
    info->role = plan.role;
    info->n_contrib = plan.n_src;
    info->n_fresh = plan.part_count;
    info->is_sync = plan.is_sync;
    info->status = me->status;
    info->drain_rounds = plan.drain_rounds;
    info->round = plan.round;
    info->local_step = me->local_step;
  }
  return me->status;
}

// Collect rounds that completed after this rank's last step (end of training).
uint32_t esgd_cpu_flush(void** bases, const esgd_cpu_params* p, void* out, esgd_step_info* info) {
  ChannelView v;
  fill_view(v, bases, p->world);
  ChannelCtl* me = v.ctl[p->rank];
  SegLayout L = layout_for(p->count, dtype_size(p->dtype));
  StepConfig cfg;
  cfg.rank = p->rank; cfg.world = p->world; cfg.average_world = p->average; cfg.home = p->home;
  cfg.timeout_ns = p->timeout_ns; cfg.grace_ns = p->grace_ns;
  Plan plan;
  memset(&plan, 0, sizeof(plan));
  ctl_flush<HostEnv>(v, cfg, &plan);
  switch (p->dtype) {
    case DT_F32: run_data<float>(bases, p->rank, L, plan, p->count, out, p->world); break;
    case DT_F64: run_data<double>(bases, p->rank, L, plan, p->count, out, p->world); break;
    case DT_I32: run_data<int32_t>(bases, p->rank, L, plan, p->count, out, p->world); break;
    default: run_data<int64_t>(bases, p->rank, L, plan, p->count, out, p->world); break;
  }
  finish_step<HostEnv>(v, cfg, &plan);
  if (info) {
    info->role = plan.role; info->n_contrib = 0; info->n_fresh = 0; info->is_sync = 0;
    info->status = me->status; info->drain_rounds = plan.drain_rounds; info->round = plan.round;
    info->local_step = me->local_step;
  }
  return me->status;
}

// stats[0..9]: local_step, participated, absent, activated, sync, dropped,
// contrib_sum, wait_ns, last_round, last_contrib; [10] status; [11] latest_round; [12] folded;
// [16..21] clock of the newest control step (ChannelCtl::ctl_t)
void esgd_ctl_stats(const void* base, uint64_t* stats) {
  const ChannelCtl* c = (const ChannelCtl*)base;
  stats[0] = c->local_step; stats[1] = c->stat_rounds_participated; stats[2] = c->stat_rounds_absent;
  stats[3] = c->stat_rounds_activated; stats[4] = c->stat_sync_rounds; stats[5] = c->stat_dropped_grads;
  stats[6] = c->stat_contrib_sum; stats[7] = c->stat_wait_ns; stats[8] = c->stat_last_round;
  stats[9] = c->stat_last_contrib; stats[10] = c->status; stats[11] = c->latest_round;
  stats[12] = c->stat_folded_grads;
  for (int q = 0; q < 6; ++q) stats[16 + q] = c->ctl_t[q];
}

// Copy the trace ring, oldest first, as rows of 10 uint64: step, round, t_ns, wait_ns, role, activator,
// fresh_mask, contrib_mask, is_sync, drain_rounds.  Returns the number of rows written.
int32_t esgd_ctl_trace(const void* base, uint64_t* rows, int32_t max_rows) {
  const ChannelCtl* c = (const ChannelCtl*)base;
  const uint64_t last = c->local_step;
  const uint64_t first = last > (uint64_t)kTraceRing ? last - kTraceRing + 1 : 1;
  int32_t n = 0;
  for (uint64_t k = first; k <= last && n < max_rows; ++k) {
    const TraceEntry& e = c->trace[k % kTraceRing];
    if (e.step != k) continue;
    uint64_t* r = rows + (size_t)n * 10;
    r[0] = e.step; r[1] = e.round; r[2] = e.t_ns; r[3] = e.wait_ns; r[4] = e.role; r[5] = e.activator;
    r[6] = e.fresh_mask; r[7] = e.contrib_mask; r[8] = e.is_sync; r[9] = e.drain_rounds;
    ++n;
  }
  return n;
}

void esgd_ctl_clear_status(void* base) { ((ChannelCtl*)base)->status = 0; }

}  // extern "C"
