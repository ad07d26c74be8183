// Partial-allreduce channel protocol: one implementation, compiled twice.
//
// The control plane of the solo / majority / synchronous partial allreduce is
// written once against an "Env" policy (atomics at system scope, a clock, a
// pause) and instantiated for (a) CUDA device code, where the channel memory of
// every rank is peer-mapped over NVLink, and (b) host code, where the ranks are
// threads or processes sharing a POSIX shared-memory segment.  The CPU build is
// both the CPU backend and the oracle for the GPU kernels.
//
// Behaviour reproduced (reference: fflib2 src/colls/ffsolo_allreduce.c:20-148,
// ffrand_allreduce.c:27-150, ffsolo_limiter.c:4-36, ffactivation.c:11-106):
//   * collectives are persistent: created once, then post/wait every step;
//   * round k is opened by the first k-th post of any rank (solo) or by a
//     shared-seed pseudo-random initiator (majority);
//   * ranks that have not arrived contribute nothing fresh; a late k-th post is
//     absorbed and never blocks;
//   * every (limiter+1)-th post is a fully synchronous round (bounded staleness).
// What is deliberately different: no message tree (NVSwitch makes every peer one
// hop, so activation is one descriptor store per peer), a consistent contributor
// snapshot taken by one elected activator, and a locked per-rank mailbox that
// counts the rounds a rank missed, so no round result is lost: the CPU backend
// accumulates the missed results there, the GPU backend lets the late rank pull
// the difference of a participant's running sum of round results and its own.
// A gradient that was published but never picked up by a round can be folded into
// the rank's next publish of the same slot parity instead of being superseded
// (StepPolicy::accumulate; the reference overwrites, opt_esgd_solo_imagenet_imbalance.py:301-314).
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define ESGD_HD __host__ __device__ __forceinline__
#define ESGD_D __device__ __forceinline__
#else
#define ESGD_HD inline
#endif

namespace esgd {

constexpr int kMaxRanks = 16;
constexpr int kDescRing = 4;      // descriptors are only read by the round's own participants
constexpr int kSlotDepth = 2;     // publish slots per rank (double buffered)

enum Mode : int32_t { MODE_SOLO = 0, MODE_MAJORITY = 1, MODE_SYNC = 2 };

enum Role : int32_t {
  ROLE_ABORT = 0,        // a bounded wait ran out; nothing is applied this step
  ROLE_PARTICIPANT = 1,  // reduce the contributors named by the round descriptor
  ROLE_DRAIN = 2,        // apply what the mailbox accumulated (rounds this rank missed)
  ROLE_IDLE = 3          // nothing to apply (mailbox empty)
};

enum StatusBits : uint32_t {
  ST_OK = 0,
  ST_TIMEOUT_ROUND = 1u << 0,     // no round >= k became visible in time
  ST_TIMEOUT_ARRIVAL = 1u << 1,   // sync round: some rank never published
  ST_TIMEOUT_LOCK = 1u << 2,      // mailbox lock not obtained in time
  ST_TIMEOUT_DONE = 1u << 3,      // previous round never completed
  ST_DESC_LAPPED = 1u << 4,       // descriptor ring overwritten before it was read
  ST_MBOX_NOT_EMPTY = 1u << 5,    // participant found data in its own mailbox (protocol error)
  ST_TIMEOUT_SLOT = 1u << 6,      // publish slot still being read
  ST_TIMEOUT_GATHER = 1u << 7,    // two-shot reduction: a participant's share never arrived
  ST_TIMEOUT_BARRIER = 1u << 8    // blocks of one rank's kernel did not meet (device only)
};

struct alignas(128) RoundDesc {
  uint64_t round;                 // written last, with release
  uint32_t activator;
  uint32_t n_fresh;               // participants (ranks that published this round's epoch)
  uint32_t n_contrib;             // slots summed (fresh + stale-unconsumed)
  uint32_t fresh_mask;
  uint32_t contrib_mask;
  uint32_t push_mask;             // absent ranks: result goes to their mailbox
  uint32_t accum_mask;            // subset of push_mask whose mailbox already holds data
  uint32_t is_sync;
  uint64_t read_epoch[kMaxRanks]; // which epoch's slot to read for each contributor
  uint64_t consumed[kMaxRanks];   // last consumed epoch per rank after this round
};

// One entry of the per-rank trace ring (the newest kTraceRing steps of this rank).
constexpr int kTraceRing = 64;
struct TraceEntry {
  uint64_t step;          // local post count
  uint64_t round;         // round applied (participant) or newest round seen (absent)
  uint64_t t_ns;          // clock at the end of the control step
  uint64_t wait_ns;       // time spent in this control step (publish, election, waits)
  uint32_t role;          // Role
  uint32_t activator;
  uint32_t fresh_mask;
  uint32_t contrib_mask;
  uint32_t is_sync;
  uint32_t drain_rounds;  // rounds collected from the mailbox (absent ranks)
};

// One per (channel, rank); lives in that rank's arena; peers read and write it.
struct alignas(128) ChannelCtl {
  uint64_t pub_epoch[kMaxRanks];          // [j] pushed by rank j: its latest published epoch
  alignas(128) uint64_t owner;            // election word; only the home rank's copy is used
  alignas(128) uint64_t snap_round;       // newest round whose activator is past its waits and is taking (or has
                                          // taken) the snapshot of who contributes what; written into every rank
  alignas(128) uint64_t latest_round;     // newest round whose descriptor is visible here
  alignas(128) uint64_t round_done;       // newest round whose data phase has completed
  alignas(128) uint32_t done_count[kDescRing];  // finishers; only the activator's copy is used
  alignas(128) uint32_t mbox_lock;        // 0 free, else 1 + holder
  uint32_t mbox_count;                    // rounds accumulated since the last drain
  alignas(128) uint64_t gather_round[kMaxRanks];  // [j] pushed by participant j: its reduced share of that round is
                                                  // complete in ITS shard buffer and may be pulled (two-shot reduction)
  alignas(128) uint64_t taken[kSlotDepth];        // [e % 2] = e: epoch e of this rank was picked up by a round
                                                  // (written by that round's activator before the descriptor)
  alignas(128) uint64_t grace_ema_ns;     // home rank's copy: smoothed arrival spread seen by activators
  alignas(128) RoundDesc desc[kDescRing];
  // ---- local only (never touched by peers) ----
  alignas(128) uint64_t local_step;       // posts made so far by the owning rank
  uint32_t status;                        // sticky OR of StatusBits
  uint32_t blocks_done;                   // data-phase block counter (device)
  uint64_t stat_rounds_participated;
  uint64_t stat_rounds_absent;
  uint64_t stat_rounds_activated;
  uint64_t stat_sync_rounds;
  uint64_t stat_dropped_grads;            // own published gradients that were superseded unconsumed
  uint64_t stat_contrib_sum;              // sum over participated rounds of n_contrib
  uint64_t stat_wait_ns;                  // time spent in bounded waits
  uint64_t stat_last_round;               // round applied at the last step
  uint64_t stat_last_contrib;
  uint64_t stat_folded_grads;             // own unconsumed gradients folded into a later publish
  uint64_t ctl_t[6];                      // clock of the newest control step: start, published, election decided,
                                          // activation waits over, descriptor out (activator only), round visible
  TraceEntry trace[kTraceRing];           // ring indexed by local_step % kTraceRing
};

// What the control step hands to the data phase of the same rank.
struct alignas(16) Plan {
  int32_t role;
  int32_t n_src;
  int32_t n_push;
  int32_t part_index;             // this rank's index among the participants
  int32_t part_count;
  int32_t activator;
  int32_t holds_own_lock;         // drain: own mailbox lock is held and must be released
  int32_t is_sync;
  uint32_t fresh_mask;            // the participants (bit per rank)
  int32_t two_shot;               // data phase split into reduce-scatter and gather (set by the device front end)
  int32_t drain_src;              // drain: a rank whose running sum of round results is complete (device backend)
  int32_t pad_;
  uint64_t round;
  float scale;                    // 1/contributors or 1/world
  float drain_rounds;             // number of rounds summed in the mailbox (drain)
  int32_t src_rank[kMaxRanks];
  int32_t src_parity[kMaxRanks];
  int32_t push_rank[kMaxRanks];
  int32_t push_accum[kMaxRanks];
};

struct StepConfig {
  int32_t rank;
  int32_t world;
  int32_t average_world;          // 0: 1/contributors, 1: 1/world (reference), 2: plain sum
  int32_t home;                   // rank whose `owner` word elects the activator
  uint64_t timeout_ns;            // bound on every wait
  uint64_t grace_ns;              // activator waits this long for near-simultaneous arrivals
};

// ---------------------------------------------------------------------------
// Shared-seed initiator stream for majority mode: every rank draws the same
// sequence (reference: rand_r(&seed) % P with one seed, ffrand_allreduce.c:88).
// A counter-based generator keeps ranks in lock-step even when one of them
// skips rounds: initiator(k) depends on (seed, k) only.
ESGD_HD uint32_t mix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  x = x ^ (x >> 31);
  return (uint32_t)(x >> 32);
}
ESGD_HD int32_t majority_initiator(uint64_t seed, uint64_t round, int32_t world) {
  return (int32_t)(mix64(seed * 0x100000001B3ull + round) % (uint32_t)world);
}

// Bounded staleness: `limiter` eager rounds, then one synchronous round, counted
// per local post (reference: ffsolo_limiter.c:9-31).  limiter < 0 disables.
ESGD_HD bool limiter_is_sync(uint64_t step, int64_t limiter) {
  if (limiter < 0) return false;
  return (step % (uint64_t)(limiter + 1)) == 0;
}

}  // namespace esgd
