// Control step of the partial allreduce, templated on the execution environment.
//
// Env must provide (all at system scope, i.e. visible to every rank):
//   ld_acq64 / st_rel64 / ld_acq32 / st_rel32, st_rlx64 / st_rlx32 (relaxed stores:
//   a group of them behind ONE fence() is as good as a group of release stores and,
//   over NVLink, costs one round trip instead of one per store), cas64 / cas32 (return the old
//   value), add32 (returns the old value), fence(), fence_sc() (sequentially
//   consistent: orders an earlier store before a later load), now_ns(), pause().
//
// One rank calls, per step and per channel, in this order:
//   wait_slot_free()  -> write (or fold) its gradient into publish slot (epoch % 2)
//   ctl_step()        -> publish, elect / wait for the round, build the Plan
//   <data phase>      -> reduce + update (participant) or apply mailbox (drain)
//   finish()          -> completion signalling, lock release
// Every wait is bounded by StepConfig::timeout_ns; when one runs out the step
// returns ROLE_ABORT and sets a sticky status bit that the host reads.
#pragma once
#include "channel.h"

#if defined(__CUDACC__)
#define ESGD_T __device__ __forceinline__
#else
#define ESGD_T inline
#endif

namespace esgd {

struct ChannelView {
  ChannelCtl* ctl[kMaxRanks];
};

struct StepPolicy {
  int32_t base_mode;       // MODE_SOLO / MODE_MAJORITY / MODE_SYNC
  int32_t include_stale;   // sum unconsumed gradients of ranks that have not arrived
  int64_t limiter;         // eager rounds between synchronous rounds; < 0: never force
  uint64_t seed;           // majority initiator stream
  int32_t accumulate;      // fold an own gradient that no round picked up into the next publish of its slot
  int32_t adaptive_grace;  // the grace window follows the smoothed arrival spread (at most StepConfig::grace_ns)
};

ESGD_HD bool round_is_sync(const StepPolicy& pol, uint64_t round) {
  return pol.base_mode == MODE_SYNC || limiter_is_sync(round, pol.limiter);
}

ESGD_HD uint32_t bit_of(int r) { return 1u << r; }
ESGD_HD int popc32(uint32_t x) {
  int c = 0;
  while (x) { x &= x - 1; ++c; }
  return c;
}

// What happens to the gradient of epoch k-2, which still sits in the slot that epoch k is about to use.
enum SlotFate : int32_t { SLOT_CONSUMED = 0, SLOT_FOLD = 1, SLOT_DROP = 2 };

// Valid once wait_slot_free() has returned true for epoch k: a round that picked epoch k-2 up has
// completed by then, and its activator wrote taken[] before it published the round.
template <class E>
ESGD_T int32_t slot_fate(ChannelCtl* me, const StepPolicy& pol, uint64_t k) {
  if (k < 3) return SLOT_CONSUMED;
  if (E::ld_acq64(&me->taken[k % kSlotDepth]) == k - 2) return SLOT_CONSUMED;
  return pol.accumulate ? SLOT_FOLD : SLOT_DROP;
}

// Before epoch k overwrites publish slot k % 2 (last used for epoch k-2) no round may still read it.
// An activator announces its round in every rank's `snap_round`, then (after a sequentially
// consistent fence) reads every rank's published epoch.  This rank published k-1 a step ago and
// fences before it reads `snap_round`: a round it does not see there yet will find epoch >= k-1 and
// never touch the slot of k-2; a round it does see may have picked k-2 up and must complete first.
// Such a round is past its arrival / grace waits and depends on no rank that is not part of it,
// so this wait cannot deadlock.
template <class E>
ESGD_T bool wait_slot_free(const ChannelView& v, const StepConfig& cfg, const StepPolicy& pol, uint64_t k) {
  (void)pol;
  ChannelCtl* me = v.ctl[cfg.rank];
  const uint64_t t0 = E::now_ns();
  E::fence_sc();
  const uint64_t target = E::ld_acq64(&me->snap_round);
  for (;;) {
    if (E::ld_acq64(&me->round_done) >= target) return true;
    if (E::now_ns() - t0 > cfg.timeout_ns) {
      me->status |= ST_TIMEOUT_SLOT;
      return false;
    }
    E::pause();
  }
}

// Runs on the elected activator of round k.  Returns 0 or a status bit.
template <class E>
ESGD_T uint32_t activate_round(const ChannelView& v, const StepConfig& cfg, const StepPolicy& pol,
                                uint64_t k, bool sync_round, uint64_t t0) {
  const int P = cfg.world, me_r = cfg.rank;
  ChannelCtl* me = v.ctl[me_r];

  // Rounds never overlap: the previous one must have completed everywhere.
  while (E::ld_acq64(&me->round_done) + 1 < k) {
    if (E::now_ns() - t0 > cfg.timeout_ns) return ST_TIMEOUT_DONE;
    E::pause();
  }
  uint64_t consumed_prev[kMaxRanks];
  for (int j = 0; j < P; ++j) consumed_prev[j] = 0;
  if (k > 1) {
    const RoundDesc* dp = &me->desc[(k - 1) % kDescRing];
    if (dp->round != k - 1) return ST_DESC_LAPPED;
    for (int j = 0; j < P; ++j) consumed_prev[j] = dp->consumed[j];
  }

  if (sync_round) {  // full-arrival barrier
    for (int j = 0; j < P; ++j) {
      while (E::ld_acq64(&me->pub_epoch[j]) < k) {
        if (E::now_ns() - t0 > cfg.timeout_ns) return ST_TIMEOUT_ARRIVAL;
        E::pause();
      }
    }
  } else if (cfg.grace_ns > 0) {
    // Ranks that arrive within the grace window of the first one are still fresh: without it,
    // near-simultaneous arrivals would all but one count as absent.  The window follows the arrival
    // spread the activators have seen lately (twice its smoothed value, at most grace_ns); every 16th
    // round waits the full window so that a growing spread is noticed.
    ChannelCtl* hm = v.ctl[cfg.home];
    uint64_t window = cfg.grace_ns, ema = 0;
    if (pol.adaptive_grace) {
      ema = E::ld_acq64(&hm->grace_ema_ns);
      const uint64_t w = 2 * ema + 1000;
      if ((k & 15u) != 0 && w < window) window = w;
    }
    const uint64_t tg = E::now_ns();
    uint64_t last_arrival = 0;
    int seen = 1;
    for (;;) {
      int arrived = 0;
      for (int j = 0; j < P; ++j) arrived += (E::ld_acq64(&me->pub_epoch[j]) >= k) ? 1 : 0;
      const uint64_t dt = E::now_ns() - tg;
      if (arrived > seen) { seen = arrived; last_arrival = dt; }
      if (arrived >= P || dt > window) break;
      E::pause();
    }
    if (pol.adaptive_grace) {   // fast attack, slow decay
      const uint64_t smooth = (7 * ema + last_arrival) / 8;
      E::st_rlx64(&hm->grace_ema_ns, last_arrival > smooth ? last_arrival : smooth);
    }
  }

  // One consistent snapshot of who has what; every reducer honours it.  Announced first, so that a
  // rank about to reuse a publish slot knows that this round may be reading it (wait_slot_free).
  for (int j = 0; j < P; ++j) E::st_rlx64(&v.ctl[j]->snap_round, k);
  E::fence_sc();
  me->ctl_t[3] = E::now_ns();
  RoundDesc d;
  d.round = k;
  d.activator = (uint32_t)me_r;
  d.n_fresh = d.n_contrib = 0;
  d.fresh_mask = d.contrib_mask = d.push_mask = d.accum_mask = 0;
  d.is_sync = sync_round ? 1u : 0u;
  for (int j = 0; j < kMaxRanks; ++j) { d.read_epoch[j] = 0; d.consumed[j] = 0; }
  for (int j = 0; j < P; ++j) {
    uint64_t e = E::ld_acq64(&me->pub_epoch[j]);
    bool fresh = (e >= k) || (j == me_r);
    bool stale = !fresh && pol.include_stale && e > consumed_prev[j];
    d.consumed[j] = consumed_prev[j];
    if (fresh) { d.fresh_mask |= bit_of(j); d.n_fresh++; e = k; }
    else d.push_mask |= bit_of(j);
    if (fresh || stale) {
      d.contrib_mask |= bit_of(j);
      d.n_contrib++;
      d.read_epoch[j] = e;
      d.consumed[j] = e;
    }
  }

  // Lock the mailboxes of the absent ranks on behalf of this round's pushers.
  uint32_t locked = 0, st = 0;
  for (int j = 0; j < P && !st; ++j) {
    if (!(d.push_mask & bit_of(j))) continue;
    ChannelCtl* cj = v.ctl[j];
    while (E::cas32(&cj->mbox_lock, 0u, (uint32_t)(1 + me_r)) != 0u) {
      if (E::now_ns() - t0 > cfg.timeout_ns) { st = ST_TIMEOUT_LOCK; break; }
      E::pause();
    }
    if (st) break;
    locked |= bit_of(j);
    uint32_t cnt = E::ld_acq32(&cj->mbox_count);
    if (cnt > 0) d.accum_mask |= bit_of(j);
    E::st_rlx32(&cj->mbox_count, cnt + 1);   // ordered before the descriptor by the fence below
  }
  if (st) {
    for (int j = 0; j < P; ++j)
      if (locked & bit_of(j)) {
        ChannelCtl* cj = v.ctl[j];
        E::st_rel32(&cj->mbox_count, E::ld_acq32(&cj->mbox_count) - 1);
        E::st_rel32(&cj->mbox_lock, 0u);
      }
    return st;
  }

  // Tell every contributor which of its epochs this round picks up (it decides from this whether a
  // later publish must fold an older gradient in), before the round becomes visible anywhere.
  for (int j = 0; j < P; ++j)
    if (d.contrib_mask & bit_of(j)) E::st_rlx64(&v.ctl[j]->taken[d.read_epoch[j] % kSlotDepth], d.read_epoch[j]);

  // Activation = one descriptor store per peer, then the round number.
  E::st_rlx32(&me->done_count[k % kDescRing], 0u);
  for (int j = 0; j < P; ++j) {
    RoundDesc* dj = &v.ctl[j]->desc[k % kDescRing];
    *dj = d;
  }
  E::fence();
  for (int j = 0; j < P; ++j) E::st_rlx64(&v.ctl[j]->latest_round, k);
  me->ctl_t[4] = E::now_ns();
  me->stat_rounds_activated++;
  return 0;
}

// A rank whose record of round results is complete: any participant of the newest completed round
// (it took part in, or collected, every earlier round before it could post that one).  Called with the
// caller's own mailbox lock held: no round that lacks the caller can start, and the caller takes part in
// none, so nothing is in flight and the descriptor ring is stable.  Different late ranks pick different
// participants.  Returns -1 if the descriptor is gone (protocol error).
template <class E>
ESGD_T int32_t pick_drain_source(ChannelCtl* me, int rank) {
  const uint64_t R = E::ld_acq64(&me->round_done);
  const RoundDesc* dr = &me->desc[R % kDescRing];
  if (dr->round != R || dr->n_fresh == 0) return -1;
  int want = rank % (int)dr->n_fresh;
  for (int j = 0; j < kMaxRanks; ++j)
    if (dr->fresh_mask & bit_of(j)) {
      if (want == 0) return j;
      --want;
    }
  return -1;
}

template <class E>
ESGD_T void ctl_step(const ChannelView& v, const StepConfig& cfg, const StepPolicy& pol, Plan* plan) {
  const int P = cfg.world, i = cfg.rank;
  ChannelCtl* me = v.ctl[i];
  const uint64_t k = me->local_step + 1;
  me->local_step = k;
  const uint64_t t0 = E::now_ns();

  plan->role = ROLE_ABORT;
  plan->n_src = plan->n_push = 0;
  plan->part_index = 0;
  plan->part_count = 1;
  plan->fresh_mask = 0;
  plan->two_shot = 0;
  plan->drain_src = -1;
  plan->activator = i;
  plan->holds_own_lock = 0;
  plan->round = k;
  plan->scale = 1.0f;
  plan->drain_rounds = 0.0f;

  const bool sync_round = round_is_sync(pol, k);
  plan->is_sync = sync_round ? 1 : 0;
  // The gradient of epoch k-2 shared this epoch's slot: picked up by a round, folded in, or superseded
  // (the reference overwrites its send buffer the same way).
  {
    const int32_t fate = slot_fate<E>(me, pol, k);
    if (fate == SLOT_FOLD) me->stat_folded_grads++;
    else if (fate == SLOT_DROP) me->stat_dropped_grads++;
  }
  // Eager solo rounds elect their activator (first arriver wins a compare-and-swap on the home rank);
  // majority rounds and synchronous rounds have a designated one, known to every rank without a message:
  // the shared-seed initiator, and rank (k mod P), which saves the election's round trip.
  bool may_activate = true, elected = false;
  if (sync_round) { may_activate = ((int)(k % (uint64_t)P) == i); elected = may_activate; }
  else if (pol.base_mode == MODE_MAJORITY) may_activate = (majority_initiator(pol.seed, k, P) == i);

  // Publish: the gradient is already in slot (k % 2); make it visible, then the epoch.
  E::fence();
  for (int j = 0; j < P; ++j) E::st_rlx64(&v.ctl[j]->pub_epoch[i], k);
  me->ctl_t[0] = t0;
  me->ctl_t[1] = E::now_ns();
  me->ctl_t[2] = me->ctl_t[3] = me->ctl_t[4] = 0;

  bool tried = false;
  uint64_t lr;
  for (;;) {
    lr = E::ld_acq64(&me->latest_round);
    if (lr >= k) break;
    if (may_activate && !tried) {
      tried = true;
      if (elected) E::st_rlx64(&v.ctl[cfg.home]->owner, k);   // keeps the election word in step for eager rounds
      if (elected || E::cas64(&v.ctl[cfg.home]->owner, k - 1, k) == k - 1) {
        me->ctl_t[2] = E::now_ns();
        uint32_t st = activate_round<E>(v, cfg, pol, k, sync_round, t0);
        if (st) { me->status |= st; me->stat_wait_ns += E::now_ns() - t0; return; }
        continue;
      }
    }
    if (E::now_ns() - t0 > cfg.timeout_ns) {
      me->status |= ST_TIMEOUT_ROUND;
      me->stat_wait_ns += E::now_ns() - t0;
      return;
    }
    E::pause();
  }

  me->ctl_t[5] = E::now_ns();
  const RoundDesc* d = &me->desc[k % kDescRing];
  const bool participant = (lr == k) && (d->round == k) && (d->fresh_mask & bit_of(i));
  if (sync_round) me->stat_sync_rounds++;

  if (participant) {
    if (E::ld_acq32(&me->mbox_count) != 0) me->status |= ST_MBOX_NOT_EMPTY;
    plan->role = ROLE_PARTICIPANT;
    plan->activator = (int32_t)d->activator;
    plan->part_count = (int32_t)d->n_fresh;
    plan->fresh_mask = d->fresh_mask;
    plan->part_index = popc32(d->fresh_mask & (bit_of(i) - 1u));
    plan->scale = cfg.average_world == 1 ? 1.0f / (float)P
                  : cfg.average_world == 2 ? 1.0f : 1.0f / (float)d->n_contrib;
    for (int j = 0; j < P; ++j) {
      if (d->contrib_mask & bit_of(j)) {
        plan->src_rank[plan->n_src] = j;
        plan->src_parity[plan->n_src] = (int32_t)(d->read_epoch[j] % kSlotDepth);
        plan->n_src++;
      }
      if (d->push_mask & bit_of(j)) {
        plan->push_rank[plan->n_push] = j;
        plan->push_accum[plan->n_push] = (d->accum_mask & bit_of(j)) ? 1 : 0;
        plan->n_push++;
      }
    }
    me->stat_rounds_participated++;
    me->stat_contrib_sum += d->n_contrib;
    me->stat_last_round = k;
    me->stat_last_contrib = d->n_contrib;
  } else {
    // Absent from round k (it ran, or is running, without this rank's fresh
    // gradient).  Whatever this rank missed is in its mailbox once round k is done.
    while (E::ld_acq64(&me->round_done) < k) {
      if (E::now_ns() - t0 > cfg.timeout_ns) {
        me->status |= ST_TIMEOUT_DONE;
        me->stat_wait_ns += E::now_ns() - t0;
        return;
      }
      E::pause();
    }
    while (E::cas32(&me->mbox_lock, 0u, (uint32_t)(1 + i)) != 0u) {
      if (E::now_ns() - t0 > cfg.timeout_ns) {
        me->status |= ST_TIMEOUT_LOCK;
        me->stat_wait_ns += E::now_ns() - t0;
        return;
      }
      E::pause();
    }
    uint32_t cnt = E::ld_acq32(&me->mbox_count);
    me->stat_rounds_absent++;
    me->stat_last_round = E::ld_acq64(&me->latest_round);
    me->stat_last_contrib = 0;
    if (cnt == 0) {
      E::st_rel32(&me->mbox_lock, 0u);
      plan->role = ROLE_IDLE;
    } else {
      E::st_rel32(&me->mbox_count, 0u);
      plan->role = ROLE_DRAIN;
      plan->holds_own_lock = 1;
      plan->drain_rounds = (float)cnt;
      plan->drain_src = pick_drain_source<E>(me, i);
    }
  }
  const uint64_t t1 = E::now_ns();
  me->stat_wait_ns += t1 - t0;
  {
    TraceEntry* te = &me->trace[k % kTraceRing];
    te->step = k;
    te->round = participant ? k : me->stat_last_round;
    te->t_ns = t1;
    te->wait_ns = t1 - t0;
    te->role = (uint32_t)plan->role;
    te->activator = participant ? d->activator : 0xffffffffu;
    te->fresh_mask = participant ? d->fresh_mask : 0u;
    te->contrib_mask = participant ? d->contrib_mask : 0u;
    te->is_sync = sync_round ? 1u : 0u;
    te->drain_rounds = (uint32_t)plan->drain_rounds;
  }
}

// Called once per rank after its data phase.
template <class E>
ESGD_T void finish_step(const ChannelView& v, const StepConfig& cfg, const Plan* plan) {
  ChannelCtl* me = v.ctl[cfg.rank];
  if (plan->role == ROLE_PARTICIPANT) {
    ChannelCtl* act = v.ctl[plan->activator];   // the atomic below releases this rank's writes and acquires the others'

    uint32_t old = E::add32(&act->done_count[plan->round % kDescRing], 1u);
    if ((int32_t)old == plan->part_count - 1) {
      E::fence();
      for (int n = 0; n < plan->n_push; ++n) E::st_rlx32(&v.ctl[plan->push_rank[n]]->mbox_lock, 0u);
      for (int j = 0; j < cfg.world; ++j) E::st_rlx64(&v.ctl[j]->round_done, plan->round);
    }
  } else if (plan->role == ROLE_DRAIN && plan->holds_own_lock) {
    E::fence();
    E::st_rel32(&me->mbox_lock, 0u);
  }
}

// End of training: collect whatever is still in the mailbox (no new round).
template <class E>
ESGD_T void ctl_flush(const ChannelView& v, const StepConfig& cfg, Plan* plan) {
  ChannelCtl* me = v.ctl[cfg.rank];
  const uint64_t t0 = E::now_ns();
  plan->role = ROLE_ABORT;
  plan->n_src = plan->n_push = 0;
  plan->holds_own_lock = 0;
  plan->two_shot = 0;
  plan->drain_src = -1;
  plan->fresh_mask = 0;
  plan->round = E::ld_acq64(&me->latest_round);
  while (E::ld_acq64(&me->round_done) < plan->round) {
    if (E::now_ns() - t0 > cfg.timeout_ns) { me->status |= ST_TIMEOUT_DONE; return; }
    E::pause();
  }
  while (E::cas32(&me->mbox_lock, 0u, (uint32_t)(1 + cfg.rank)) != 0u) {
    if (E::now_ns() - t0 > cfg.timeout_ns) { me->status |= ST_TIMEOUT_LOCK; return; }
    E::pause();
  }
  uint32_t cnt = E::ld_acq32(&me->mbox_count);
  if (cnt == 0) {
    E::st_rel32(&me->mbox_lock, 0u);
    plan->role = ROLE_IDLE;
  } else {
    E::st_rel32(&me->mbox_count, 0u);
    plan->role = ROLE_DRAIN;
    plan->holds_own_lock = 1;
    plan->drain_rounds = (float)cnt;
    plan->drain_src = pick_drain_source<E>(me, cfg.rank);
  }
}

}  // namespace esgd
