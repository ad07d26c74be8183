// Host operation runtime (see oprt.h).  One progress thread per rank executes posted
// operations, matches messages in the in-process mailbox and fires dependents
// (reference: fflib2 src/ffop.c:59-401, src/ffprogress.c:28-58, src/ffop_scheduler.c,
// src/ffschedule.c:84-237, src/colls/ffallreduce.c:74-177, ffactivation.c:11-106,
// ffsolo_limiter.c:4-36).  Differences by design: every reduction operator is implemented,
// the allreduce is correct for any number of ranks, waits take a timeout, and the transport
// is a mailbox between threads instead of MPI.
#include "oprt.h"

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <initializer_list>
#include <limits>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <tuple>
#include <vector>

namespace {

constexpr size_t kDirectBytes = 16 << 10;         // bodies from this size on are copied straight into a listening receive
constexpr size_t kPooledBodyBytes = 64 << 10;     // message bodies from this size on are recycled
constexpr size_t kMaxSpareBodies = 64;
constexpr size_t kMaxSpareBytes = 512u << 20;
constexpr double kDefaultWaitSeconds = 600.0;   // what "no timeout" means: ten minutes, then RT_TIMEOUT
// How long an idle progress thread / a waiter spins before it sleeps (ESGD_RT_SPIN_US overrides; 0 = sleep at once).
int spin_micros() {
  static const int v = [] { const char* e = getenv("ESGD_RT_SPIN_US"); return e ? atoi(e) : 50; }();
  return v;
}
#define kSpinMicros spin_micros()
constexpr int kBusySpinFactor = 20;   // the window of a thread that has reason to expect an event soon

size_t dtype_size(int dt) { return dt == RT_CHAR ? 1 : (dt == RT_INT32 || dt == RT_FLOAT) ? 4 : 8; }

// Shadow-tagged messages live in a tag space of their own.
int wire_tag(int tag, int options) { return (options & RT_SHADOW_TAG) ? (tag | 0x40000000) : tag; }

enum OpType { T_NOP, T_CALLBACK, T_COMP, T_SEND, T_RECV };

struct Buffer {
  bool alive = true;
  void* ptr = nullptr;
  std::vector<uint8_t> own;
  int64_t count = 0;
  int dtype = RT_FLOAT;
  void* data() { return ptr ? ptr : (void*)own.data(); }
};

// One happens-before edge.  Plain edges (rt_op_hb) fire whenever the parent completes.  Versioned edges
// (rt_op_hb_fallback without RT_DEP_IGNORE_VERSION) follow the reference's version rules
// (fflib2 src/ffop.c:299-401): the parent's n-th completion satisfies the dependent's n-th run only.
struct Edge {
  rt_op child = RT_NONE;
  rt_op fallback = RT_NONE;   // gets the completion when the dependent has already run for this version
  int options = 0;
  int count = 0;              // constrained edge: completions it may still pass on
  int futures = 0;            // completions that arrived ahead of the dependent's version
  rt_op constrains_op = RT_NONE;   // edge (op, index) whose `count` this edge feeds when it passes one on
  int constrains_idx = -1;
};

struct Op {
  OpType type = T_NOP;
  int options = 0;
  rt_buf a = RT_NONE, b = RT_NONE, out = RT_NONE;
  int oper = RT_SUM, peer = -1, tag = 0;
  rt_callback_fn cb = nullptr;
  void* cb_arg = nullptr;
  std::vector<Edge> edges;    // happens-before edges to dependents, in creation order
  std::vector<rt_op> parents; // who points here (needed to unlink on free)
  int num_parents = 0;
  int64_t posted = 0;         // posts so far, explicit or by a parent (the "posted version")
  bool alive = true;
  int dep_left = 0;           // parents still to complete in this round (AND)
  size_t first_rr = 0;        // round-robin cursor for RT_DEP_FIRST
  int64_t executed = 0;       // times started
  std::atomic<int64_t> completed{0};
  std::atomic<int64_t> waited{0};
  bool in_flight = false;     // a recv waiting for its message
};

struct Message {
  std::vector<uint8_t> data;
};

struct Schedule {
  bool alive = true;
  std::vector<rt_op> ops;
  std::vector<rt_buf> owned_bufs;   // temporaries a collective created for itself
  std::vector<rt_sched> parts;      // schedules a composite one is made of (deleted with it)
  rt_op begin = RT_NONE, end = RT_NONE;
  bool finalized = false;
  // overridable behaviour and a state slot (ffschedule_set_*_fun / ffschedule_{set,get}_state)
  rt_sched_fn start_fn = nullptr, post_fn = nullptr, test_fn = nullptr, delete_fn = nullptr;
  rt_sched_wait_fn wait_fn = nullptr;
  rt_sched_print_fn print_fn = nullptr;
  void* state = nullptr;
};

struct Partial;   // state of one solo / majority allreduce (defined with the collectives)

}  // namespace

struct rt_world {
  int n = 0;
  std::vector<std::unique_ptr<rt_rank>> ranks;
  std::mutex mail_mu;
  std::map<std::tuple<int, int, int>, std::deque<Message>> mail;  // (src, dst, tag) -> FIFO
  // Message bodies that have been delivered, kept for the next sends: a fresh allocation of a large body is
  // fresh pages from the kernel every time, which costs more than the copy itself.  Guarded by mail_mu.
  std::vector<std::vector<uint8_t>> spare_bodies;
  size_t spare_bytes = 0;
  std::atomic<int64_t> direct_bodies{0}, queued_bodies{0};   // how message bodies travelled (rt_world_stats)
};

struct rt_rank {
  rt_world* world = nullptr;
  int id = 0;
  std::mutex mu;                       // protects ops / buffers / queues
  std::condition_variable cv;          // completions
  std::condition_variable work_cv;     // progress thread wake-up
  std::deque<std::unique_ptr<Op>> ops;
  std::deque<Buffer> bufs;
  std::deque<Schedule> scheds;
  std::deque<rt_op> posted;
  std::vector<rt_op> pending_recvs;
  std::vector<rt_operator_fn> custom_ops;
  std::vector<rt_op> free_ops;         // recycled handles
  std::vector<rt_buf> free_bufs;
  std::vector<rt_sched> free_scheds;
  std::thread progress;
  std::atomic<bool> stop{false};
  std::atomic<uint64_t> signals{0};    // bumped with every wake-up of the progress thread (a spinning one sees it)
  rt_op in_callback = RT_NONE;         // the callback operation that is running with the lock released
  std::map<rt_sched, Partial*> partials;   // state of the partial allreduces that have not been deleted
  std::map<int, int64_t> partial_generation;   // per tag: how many partial allreduces this rank has created
  ~rt_rank();
};

namespace {

template <class T>
void reduce_typed(const T* a, const T* b, T* o, int64_t n, int oper) {
  switch (oper) {
    case RT_SUM: for (int64_t i = 0; i < n; ++i) o[i] = a[i] + b[i]; break;
    case RT_PROD: for (int64_t i = 0; i < n; ++i) o[i] = a[i] * b[i]; break;
    case RT_MAX: for (int64_t i = 0; i < n; ++i) o[i] = a[i] > b[i] ? a[i] : b[i]; break;
    case RT_MIN: for (int64_t i = 0; i < n; ++i) o[i] = a[i] < b[i] ? a[i] : b[i]; break;
    default: break;
  }
}

void run_comp(rt_rank* c, Op& op) {
  Buffer& A = c->bufs[op.a];
  Buffer& O = c->bufs[op.out];
  if (op.oper == RT_IDENTITY) {
    int64_t n = A.count < O.count ? A.count : O.count;
    if (A.data() != O.data()) memcpy(O.data(), A.data(), (size_t)n * dtype_size(A.dtype));
    return;
  }
  Buffer& B = c->bufs[op.b];
  int64_t n = A.count;
  if (B.count < n) n = B.count;
  if (O.count < n) n = O.count;
  if (op.oper >= RT_CUSTOM0) {
    rt_operator_fn fn = c->custom_ops[op.oper - RT_CUSTOM0];
    if (fn) fn(A.data(), B.data(), O.data(), n, A.dtype);
    return;
  }
  switch (A.dtype) {
    case RT_INT32: reduce_typed((const int32_t*)A.data(), (const int32_t*)B.data(), (int32_t*)O.data(), n, op.oper); break;
    case RT_INT64: reduce_typed((const int64_t*)A.data(), (const int64_t*)B.data(), (int64_t*)O.data(), n, op.oper); break;
    case RT_CHAR: reduce_typed((const signed char*)A.data(), (const signed char*)B.data(), (signed char*)O.data(), n, op.oper); break;
    case RT_FLOAT: reduce_typed((const float*)A.data(), (const float*)B.data(), (float*)O.data(), n, op.oper); break;
    default: reduce_typed((const double*)A.data(), (const double*)B.data(), (double*)O.data(), n, op.oper); break;
  }
}

void trigger(rt_rank* c, rt_op id);
void free_op_locked(rt_rank* c, rt_op id);

void post_locked(rt_rank* c, rt_op id) {
  c->ops[id]->posted++;
  c->posted.push_back(id);
}

// One completion of `op` (its `version`-th) travels along edge `e`.  Called with c->mu held.
void satisfy(rt_rank* c, Op& op, Edge& e, int64_t version) {
  rt_op target = e.child;
  if (target == RT_NONE || !c->ops[target] || !c->ops[target]->alive) return;
  const bool versioned = !(e.options & RT_DEP_IGNORE_VERSION);
  int64_t tv = c->ops[target]->posted;
  if (versioned && version <= tv) {            // the dependent already ran for this version
    if (e.fallback == RT_NONE || !c->ops[e.fallback] || !c->ops[e.fallback]->alive) return;
    target = e.fallback;
    tv = c->ops[target]->posted;
    if (version <= tv) return;
  }
  if (versioned && version > tv + 1) {         // ahead of the dependent: remembered until it catches up
    e.futures++;
    return;
  }
  if (e.options & RT_DEP_NO_AUTOPOST) return;
  if (e.options & RT_DEP_CONSTRAINED) {
    if (e.count == 0) return;
    e.count--;
  }
  if (e.constrains_op != RT_NONE && c->ops[e.constrains_op] && e.constrains_idx >= 0)
    c->ops[e.constrains_op]->edges[e.constrains_idx].count++;
  (void)op;
  trigger(c, target);
}

// Called with c->mu held.
void complete(rt_rank* c, rt_op id) {
  Op& op = *c->ops[id];
  const int64_t version = op.completed.fetch_add(1) + 1;
  c->cv.notify_all();
  if (op.edges.empty()) return;
  if (op.options & RT_DEP_FIRST) {           // satisfy exactly one dependent, in turn
    Edge& e = op.edges[op.first_rr % op.edges.size()];
    op.first_rr++;
    satisfy(c, op, e, version);
  } else {
    for (size_t i = 0; i < op.edges.size(); ++i) satisfy(c, op, op.edges[i], version);
  }
}

// A parent of `id` has completed.  Called with c->mu held.
void trigger(rt_rank* c, rt_op id) {
  Op& op = *c->ops[id];
  if ((op.options & RT_NON_PERSISTENT) && op.posted > 0) return;
  if (op.options & RT_DEP_OR) {
    post_locked(c, id);
  } else {
    if (op.dep_left <= 0) op.dep_left = op.num_parents;
    if (--op.dep_left <= 0) {      // an op that is only ever a fall-back has no parent edge of its own
      op.dep_left = 0;
      post_locked(c, id);
    }
  }
}

// Completions that arrived before the op reached their version count now.  Called with c->mu held.
void consume_futures(rt_rank* c, rt_op id) {
  Op& op = *c->ops[id];
  for (rt_op pid : op.parents) {
    if (!c->ops[pid]) continue;
    for (Edge& e : c->ops[pid]->edges)
      if (e.child == id && e.futures > 0) {
        e.futures--;
        trigger(c, id);
      }
  }
}

// Start one operation.  Called with c->mu held; may release it around user callbacks.
void execute(rt_rank* c, rt_op id, std::unique_lock<std::mutex>& lk) {
  if (!c->ops[id] || !c->ops[id]->alive) return;
  Op& op = *c->ops[id];
  op.executed++;
  consume_futures(c, id);
  switch (op.type) {
    case T_NOP: complete(c, id); break;
    case T_CALLBACK: {
      rt_callback_fn fn = op.cb;
      void* arg = op.cb_arg;
      c->in_callback = id;
      lk.unlock();
      if (fn) fn(id, arg);
      lk.lock();
      c->in_callback = RT_NONE;
      if (!op.alive) {                 // freed while its callback ran
        free_op_locked(c, id);
        c->cv.notify_all();
        break;
      }
      complete(c, id);
      break;
    }
    case T_COMP: run_comp(c, op); complete(c, id); break;
    case T_SEND: {
      Buffer& b = c->bufs[op.a];
      const size_t bytes = (size_t)b.count * dtype_size(b.dtype);
      rt_rank* dst = c->world->ranks[op.peer].get();
      if (bytes >= kDirectBytes && dst != c) {
        // A large body goes straight into the buffer of a receive that is already listening: one copy instead of
        // two.  The sender's own lock is released meanwhile (two partners that send to each other at the same moment,
        // as in every round of the allreduce, would otherwise both find the other's lock taken), and the receiver's
        // is only tried: when it is busy, or no receive is listening yet, the body is queued as usual.
        const void* src = b.data();
        const int key_tag = wire_tag(op.tag, op.options);
        const auto key = std::make_tuple(c->id, op.peer, key_tag);
        bool delivered = false;
        c->in_callback = id;                            // keeps the operation alive while the lock is released
        lk.unlock();
        {
          std::unique_lock<std::mutex> dl(dst->mu, std::try_to_lock);
          if (dl.owns_lock()) {
            bool nothing_queued;                        // an earlier body of this (source, tag) must not be overtaken
            {
              std::lock_guard<std::mutex> g(c->world->mail_mu);
              auto it = c->world->mail.find(key);
              nothing_queued = it == c->world->mail.end() || it->second.empty();
            }
            for (size_t i = 0; nothing_queued && i < dst->pending_recvs.size(); ++i) {
              const rt_op rid = dst->pending_recvs[i];
              if (!dst->ops[rid] || !dst->ops[rid]->alive) continue;
              Op& ro = *dst->ops[rid];
              if (ro.peer != c->id || wire_tag(ro.tag, ro.options) != key_tag) continue;
              Buffer& rb = dst->bufs[ro.a];
              const size_t cap = (size_t)rb.count * dtype_size(rb.dtype);
              memcpy(rb.data(), src, bytes < cap ? bytes : cap);
              ro.in_flight = false;
              dst->pending_recvs.erase(dst->pending_recvs.begin() + i);
              complete(dst, rid);
              delivered = true;
              break;
            }
          }
        }
        if (delivered) {
          dst->signals.fetch_add(1, std::memory_order_release);
          dst->work_cv.notify_all();
        }
        lk.lock();
        c->in_callback = RT_NONE;
        if (!op.alive) {                                // freed meanwhile
          free_op_locked(c, id);
          c->cv.notify_all();
          break;
        }
        if (delivered) { c->world->direct_bodies.fetch_add(1, std::memory_order_relaxed); complete(c, id); break; }
      }
      c->world->queued_bodies.fetch_add(1, std::memory_order_relaxed);
      Message m;
      if (bytes >= kPooledBodyBytes) {                  // take a delivered body of sufficient capacity, if there is one
        std::lock_guard<std::mutex> g(c->world->mail_mu);
        auto& pool = c->world->spare_bodies;
        for (size_t i = 0; i < pool.size(); ++i)
          if (pool[i].capacity() >= bytes) {
            c->world->spare_bytes -= pool[i].capacity();
            m.data = std::move(pool[i]);
            pool[i] = std::move(pool.back());
            pool.pop_back();
            break;
          }
      }
      m.data.resize(bytes);
      memcpy(m.data.data(), b.data(), bytes);
      {
        std::lock_guard<std::mutex> g(c->world->mail_mu);
        c->world->mail[std::make_tuple(c->id, op.peer, wire_tag(op.tag, op.options))].push_back(std::move(m));
      }
      dst->signals.fetch_add(1, std::memory_order_release);
      dst->work_cv.notify_all();
      complete(c, id);
      break;
    }
    case T_RECV: op.in_flight = true; c->pending_recvs.push_back(id); break;
  }
}

// Match pending receives against the mailbox.  Called with c->mu held.
bool poll_recvs(rt_rank* c) {
  bool any = false;
  for (size_t i = 0; i < c->pending_recvs.size();) {
    rt_op id = c->pending_recvs[i];
    if (!c->ops[id] || !c->ops[id]->alive) { c->pending_recvs.erase(c->pending_recvs.begin() + i); continue; }
    Op& op = *c->ops[id];
    Message m;
    bool got = false;
    {
      std::lock_guard<std::mutex> g(c->world->mail_mu);
      auto it = c->world->mail.find(std::make_tuple(op.peer, c->id, wire_tag(op.tag, op.options)));
      if (it != c->world->mail.end() && !it->second.empty()) {
        m = std::move(it->second.front());
        it->second.pop_front();
        got = true;
      }
    }
    if (!got) { ++i; continue; }
    Buffer& b = c->bufs[op.a];
    size_t cap = (size_t)b.count * dtype_size(b.dtype);
    memcpy(b.data(), m.data.data(), m.data.size() < cap ? m.data.size() : cap);
    if (m.data.capacity() >= kPooledBodyBytes) {         // keep the body for a later send
      std::lock_guard<std::mutex> g(c->world->mail_mu);
      if (c->world->spare_bodies.size() < kMaxSpareBodies && c->world->spare_bytes + m.data.capacity() <= kMaxSpareBytes) {
        c->world->spare_bytes += m.data.capacity();
        c->world->spare_bodies.push_back(std::move(m.data));
      }
    }
    op.in_flight = false;
    c->pending_recvs.erase(c->pending_recvs.begin() + i);
    complete(c, id);
    any = true;
  }
  return any;
}

void progress_loop(rt_rank* c) {
  std::unique_lock<std::mutex> lk(c->mu);
  while (!c->stop.load()) {
    bool did = false;
    while (!c->posted.empty()) {
      rt_op id = c->posted.front();
      c->posted.pop_front();
      execute(c, id, lk);
      did = true;
    }
    if (poll_recvs(c)) did = true;
    if (!did) {
      // A dependency chain across ranks is a sequence of wake-ups; a condition variable costs tens of
      // microseconds each.  So the thread first spins for a short while (lock released) on the counter that every
      // waker bumps, and only then goes to sleep.
      const uint64_t seen = c->signals.load(std::memory_order_acquire);
      // a rank that is listening for a message expects one soon (its peer is copying a body right now, which for a
      // large body takes longer than the plain window): it spins longer before it pays for a sleep and a wake-up
      const int window = c->pending_recvs.empty() ? kSpinMicros : kSpinMicros * kBusySpinFactor;
      lk.unlock();
      const auto t0 = std::chrono::steady_clock::now();
      int polls = 0;
      while (c->signals.load(std::memory_order_acquire) == seen && !c->stop.load()) {
        if ((++polls & 63) == 0) {
          if (std::chrono::steady_clock::now() - t0 > std::chrono::microseconds(window)) break;
          std::this_thread::yield();
        }
      }
      lk.lock();
      if (c->signals.load(std::memory_order_acquire) == seen && !c->stop.load())
        c->work_cv.wait_for(lk, std::chrono::microseconds(200));
    }
  }
}

rt_op new_op(rt_rank* c, OpType t, int options) {
  std::lock_guard<std::mutex> g(c->mu);
  rt_op id;
  if (!c->free_ops.empty()) {          // a freed handle is used again
    id = c->free_ops.back();
    c->free_ops.pop_back();
    c->ops[id].reset(new Op());
  } else {
    c->ops.emplace_back(new Op());
    id = (rt_op)c->ops.size() - 1;
  }
  c->ops[id]->type = t;
  c->ops[id]->options = options;
  return id;
}

// Unlink and release one operation.  Called with c->mu held.
void free_op_locked(rt_rank* c, rt_op id) {
  if (id < 0 || id >= (rt_op)c->ops.size() || !c->ops[id]) return;
  Op& op = *c->ops[id];
  if (c->in_callback == id) {          // its callback is running right now: execute() frees it when that returns
    op.alive = false;
    return;
  }
  for (Edge& e : op.edges)
    if (e.child != RT_NONE && e.child != id && c->ops[e.child]) {
      Op& ch = *c->ops[e.child];
      for (size_t i = 0; i < ch.parents.size(); ++i)
        if (ch.parents[i] == id) { ch.parents.erase(ch.parents.begin() + i); ch.num_parents--; break; }
    }
  for (rt_op pid : op.parents)
    if (pid != id && c->ops[pid])
      for (Edge& e : c->ops[pid]->edges) {
        if (e.child == id) e.child = RT_NONE;
        if (e.fallback == id) e.fallback = RT_NONE;
      }
  for (size_t i = 0; i < c->posted.size();)
    if (c->posted[i] == id) c->posted.erase(c->posted.begin() + i); else ++i;
  for (size_t i = 0; i < c->pending_recvs.size();)
    if (c->pending_recvs[i] == id) c->pending_recvs.erase(c->pending_recvs.begin() + i); else ++i;
  c->ops[id].reset();
  c->free_ops.push_back(id);
}

// Handle checks (called with c->mu held): a handle that was never given out, or was given back, is refused with
// RT_ERROR instead of being used as an index.
inline bool ok_buf(rt_rank* c, rt_buf b) { return b >= 0 && b < (rt_buf)c->bufs.size() && c->bufs[b].alive; }
inline bool ok_op(rt_rank* c, rt_op id) { return id >= 0 && id < (rt_op)c->ops.size() && c->ops[id] && c->ops[id]->alive; }
inline bool ok_sched(rt_rank* c, rt_sched s) { return s >= 0 && s < (rt_sched)c->scheds.size() && c->scheds[s].alive; }

}  // namespace

extern "C" {

rt_world* rt_world_create(int nranks) {
  rt_world* w = new rt_world();
  w->n = nranks;
  for (int r = 0; r < nranks; ++r) {
    w->ranks.emplace_back(new rt_rank());
    rt_rank* c = w->ranks.back().get();
    c->world = w;
    c->id = r;
  }
  for (auto& c : w->ranks) c->progress = std::thread(progress_loop, c.get());
  return w;
}

void rt_world_destroy(rt_world* w) {
  for (auto& c : w->ranks) { c->stop.store(true); c->work_cv.notify_all(); }
  for (auto& c : w->ranks) if (c->progress.joinable()) c->progress.join();
  delete w;
}

rt_rank* rt_world_rank(rt_world* w, int r) { return w->ranks[r].get(); }
int rt_world_stats(rt_world* w, int64_t* out) {
  out[0] = w->direct_bodies.load(); out[1] = w->queued_bodies.load();
  return RT_SUCCESS;
}
int rt_rank_id(rt_rank* c) { return c->id; }
int rt_rank_size(rt_rank* c) { return c->world->n; }

rt_buf rt_buffer_create(rt_rank* c, void* user_ptr, int64_t count, int dtype) {
  std::lock_guard<std::mutex> g(c->mu);
  rt_buf id;
  if (!c->free_bufs.empty()) {
    id = c->free_bufs.back();
    c->free_bufs.pop_back();
    c->bufs[id] = Buffer();
  } else {
    c->bufs.emplace_back();
    id = (rt_buf)c->bufs.size() - 1;
  }
  Buffer& b = c->bufs[id];
  b.ptr = user_ptr; b.count = count; b.dtype = dtype;
  if (!user_ptr) b.own.assign((size_t)count * dtype_size(dtype), 0);
  return id;
}

int rt_buffer_delete(rt_rank* c, rt_buf id) {
  std::lock_guard<std::mutex> g(c->mu);
  if (id < 0 || id >= (rt_buf)c->bufs.size() || !c->bufs[id].alive) return RT_ERROR;
  c->bufs[id] = Buffer();
  c->bufs[id].alive = false;
  std::vector<uint8_t>().swap(c->bufs[id].own);
  c->free_bufs.push_back(id);
  return RT_SUCCESS;
}

int rt_buffer_resize(rt_rank* c, rt_buf id, void* user_ptr, int64_t count) {
  std::lock_guard<std::mutex> g(c->mu);
  if (!ok_buf(c, id) || count < 0) return RT_ERROR;
  Buffer& b = c->bufs[id];
  b.count = count;
  if (user_ptr) { b.ptr = user_ptr; b.own.clear(); }
  else if (!b.ptr) b.own.resize((size_t)count * dtype_size(b.dtype), 0);
  return RT_SUCCESS;
}

int64_t rt_buffer_count(rt_rank* c, rt_buf b) { std::lock_guard<std::mutex> g(c->mu); return ok_buf(c, b) ? c->bufs[b].count : RT_ERROR; }
void* rt_buffer_data(rt_rank* c, rt_buf b) { std::lock_guard<std::mutex> g(c->mu); return ok_buf(c, b) ? c->bufs[b].data() : nullptr; }

rt_op rt_op_nop(rt_rank* c, int options) { return new_op(c, T_NOP, options); }

rt_op rt_op_callback(rt_rank* c, rt_callback_fn fn, void* arg, int options) {
  rt_op id = new_op(c, T_CALLBACK, options);
  std::lock_guard<std::mutex> g(c->mu);
  c->ops[id]->cb = fn; c->ops[id]->cb_arg = arg;
  return id;
}

rt_op rt_op_comp(rt_rank* c, rt_buf a, rt_buf b, rt_buf out, int oper, int options) {
  {
    std::lock_guard<std::mutex> g(c->mu);
    if (!ok_buf(c, a) || !ok_buf(c, out) || (oper != RT_IDENTITY && !ok_buf(c, b))) return RT_ERROR;
    if (oper >= RT_CUSTOM0 && (oper - RT_CUSTOM0 >= (int)c->custom_ops.size())) return RT_ERROR;
  }
  rt_op id = new_op(c, T_COMP, options);
  std::lock_guard<std::mutex> g(c->mu);
  Op& op = *c->ops[id];
  op.a = a; op.b = b; op.out = out; op.oper = oper;
  return id;
}

rt_op rt_op_send(rt_rank* c, rt_buf b, int peer, int tag, int options) {
  {
    std::lock_guard<std::mutex> g(c->mu);
    if (!ok_buf(c, b) || peer < 0 || peer >= c->world->n) return RT_ERROR;
  }
  rt_op id = new_op(c, T_SEND, options);
  std::lock_guard<std::mutex> g(c->mu);
  Op& op = *c->ops[id];
  op.a = b; op.peer = peer; op.tag = tag;
  return id;
}

rt_op rt_op_recv(rt_rank* c, rt_buf b, int peer, int tag, int options) {
  {
    std::lock_guard<std::mutex> g(c->mu);
    if (!ok_buf(c, b) || peer < 0 || peer >= c->world->n) return RT_ERROR;
  }
  rt_op id = new_op(c, T_RECV, options);
  std::lock_guard<std::mutex> g(c->mu);
  Op& op = *c->ops[id];
  op.a = b; op.peer = peer; op.tag = tag;
  return id;
}

int rt_operator_create(rt_rank* c, rt_operator_fn fn) {
  std::lock_guard<std::mutex> g(c->mu);
  for (size_t i = 0; i < c->custom_ops.size(); ++i)      // a deleted operator's number is given out again
    if (!c->custom_ops[i]) { c->custom_ops[i] = fn; return RT_CUSTOM0 + (int)i; }
  c->custom_ops.push_back(fn);
  return RT_CUSTOM0 + (int)c->custom_ops.size() - 1;
}

// ffcomp_operator_delete: compute operations that still name the operator must not run afterwards.
int rt_operator_delete(rt_rank* c, int oper) {
  std::lock_guard<std::mutex> g(c->mu);
  const int i = oper - RT_CUSTOM0;
  if (i < 0 || i >= (int)c->custom_ops.size() || !c->custom_ops[i]) return RT_ERROR;
  c->custom_ops[i] = nullptr;
  return RT_SUCCESS;
}

// One line on an operation: what it is, whom it talks to, how often it was posted / started / completed, how many
// dependents it has (ffop_tostring).
int rt_op_tostring(rt_rank* c, rt_op id, char* out, int64_t cap) {
  static const char* names[] = {"nop", "callback", "comp", "send", "recv"};
  std::lock_guard<std::mutex> g(c->mu);
  if (id < 0 || id >= (rt_op)c->ops.size() || !c->ops[id] || cap < 1) return RT_ERROR;
  const Op& op = *c->ops[id];
  std::string t = std::string("[") + std::to_string(id) + "." + std::to_string(c->id) + "] " + names[op.type];
  if (op.type == T_SEND || op.type == T_RECV)
    t += std::string(op.type == T_SEND ? " to " : " from ") + std::to_string(op.peer) + " tag " + std::to_string(op.tag) +
         ((op.options & RT_SHADOW_TAG) ? " (shadow)" : "");
  if (op.type == T_COMP) t += " operator " + std::to_string(op.oper);
  t += std::string(" deps ") + ((op.options & RT_DEP_OR) ? "or" : (op.options & RT_DEP_FIRST) ? "first" : "and");
  if (op.options & RT_NON_PERSISTENT) t += " once";
  t += " posted " + std::to_string(op.posted) + " started " + std::to_string(op.executed) + " completed " +
       std::to_string(op.completed.load()) + " parents " + std::to_string(op.num_parents) + " dependents " +
       std::to_string(op.edges.size()) + (op.in_flight ? " listening" : "");
  if ((int64_t)t.size() + 1 > cap) return RT_ERROR;
  memcpy(out, t.c_str(), t.size() + 1);
  return (int)t.size();
}

int rt_op_hb_fallback(rt_rank* c, rt_op first, rt_op second, rt_op fallback, int options, rt_dep* dep) {
  std::lock_guard<std::mutex> g(c->mu);
  if (first < 0 || second < 0 || !c->ops[first] || !c->ops[second]) return RT_ERROR;
  Edge e;
  e.child = second;
  e.fallback = fallback;
  e.options = options;
  c->ops[first]->edges.push_back(e);
  c->ops[second]->parents.push_back(first);
  c->ops[second]->num_parents++;
  if (fallback != RT_NONE && c->ops[fallback]) c->ops[fallback]->parents.push_back(first);
  if (dep) *dep = (first << 20) | (rt_dep)(c->ops[first]->edges.size() - 1);
  return RT_SUCCESS;
}

int rt_op_hb(rt_rank* c, rt_op first, rt_op second) {
  return rt_op_hb_fallback(c, first, second, RT_NONE, RT_DEP_IGNORE_VERSION, nullptr);
}

// The constrained edge passes a completion on only after the constraining edge has passed one
// (ffdep_set_parent, fflib2 src/ffop.c:208-216).
int rt_dep_set_parent(rt_rank* c, rt_dep constrained, rt_dep constraining) {
  std::lock_guard<std::mutex> g(c->mu);
  const rt_op o1 = constrained >> 20, o2 = constraining >> 20;
  const int i1 = (int)(constrained & 0xfffff), i2 = (int)(constraining & 0xfffff);
  if (!c->ops[o1] || !c->ops[o2] || i1 >= (int)c->ops[o1]->edges.size() || i2 >= (int)c->ops[o2]->edges.size())
    return RT_ERROR;
  c->ops[o1]->edges[i1].options |= RT_DEP_CONSTRAINED;
  c->ops[o2]->edges[i2].constrains_op = o1;
  c->ops[o2]->edges[i2].constrains_idx = i1;
  return RT_SUCCESS;
}

int rt_op_post(rt_rank* c, rt_op op) {
  {
    std::lock_guard<std::mutex> g(c->mu);
    if (op < 0 || op >= (rt_op)c->ops.size() || !c->ops[op]) return RT_ERROR;
    post_locked(c, op);
  }
  c->signals.fetch_add(1, std::memory_order_release);
  c->work_cv.notify_all();
  return RT_SUCCESS;
}

int rt_op_free(rt_rank* c, rt_op op) {
  std::lock_guard<std::mutex> g(c->mu);
  if (op < 0 || op >= (rt_op)c->ops.size() || !c->ops[op]) return RT_ERROR;
  free_op_locked(c, op);
  return RT_SUCCESS;
}

// Withdraw an operation that has been posted but has not completed: it leaves the run queue, a receive
// stops listening, and its dependency count starts afresh (ffop_cancel, fflib2 src/ffop.c:403-408).
int rt_op_cancel(rt_rank* c, rt_op id) {
  std::lock_guard<std::mutex> g(c->mu);
  if (id < 0 || id >= (rt_op)c->ops.size() || !c->ops[id]) return RT_ERROR;
  Op& op = *c->ops[id];
  if (op.options & RT_OP_COMPLETE_BEFORE_CANCELLING) {   // what has been posted runs to completion
    op.dep_left = op.num_parents;
    return RT_SUCCESS;
  }
  for (size_t i = 0; i < c->posted.size();)
    if (c->posted[i] == id) c->posted.erase(c->posted.begin() + i); else ++i;
  for (size_t i = 0; i < c->pending_recvs.size();)
    if (c->pending_recvs[i] == id) c->pending_recvs.erase(c->pending_recvs.begin() + i); else ++i;
  op.in_flight = false;
  op.dep_left = op.num_parents;
  return RT_SUCCESS;
}

int rt_op_wait(rt_rank* c, rt_op id, double timeout_s) {
  std::unique_lock<std::mutex> lk(c->mu);
  if (!ok_op(c, id)) return RT_ERROR;
  Op& op = *c->ops[id];
  const int64_t want = op.waited.load() + 1;
  auto pred = [&] { return op.completed.load() >= want; };
  if (timeout_s <= 0) timeout_s = kDefaultWaitSeconds;    // no wait is unbounded
  if (!pred()) {                                          // spin briefly before sleeping (see progress_loop)
    const int window = (c->pending_recvs.empty() && c->posted.empty()) ? kSpinMicros : kSpinMicros * kBusySpinFactor;
    lk.unlock();
    const auto t0 = std::chrono::steady_clock::now();
    int polls = 0;
    while (!pred()) {
      if ((++polls & 63) == 0) {
        if (std::chrono::steady_clock::now() - t0 > std::chrono::microseconds(window)) break;
        std::this_thread::yield();
      }
    }
    lk.lock();
  }
  if (!c->cv.wait_for(lk, std::chrono::duration<double>(timeout_s), pred)) return RT_TIMEOUT;
  op.waited.store(want);
  return RT_SUCCESS;
}

int rt_op_test(rt_rank* c, rt_op id) {
  std::lock_guard<std::mutex> g(c->mu);
  if (!ok_op(c, id)) return RT_ERROR;
  Op& op = *c->ops[id];
  if (op.completed.load() > op.waited.load()) { op.waited.fetch_add(1); return RT_COMPLETED; }
  return RT_SUCCESS;
}

int64_t rt_op_completions(rt_rank* c, rt_op id) { std::lock_guard<std::mutex> g(c->mu); return ok_op(c, id) ? c->ops[id]->completed.load() : RT_ERROR; }

rt_sched rt_schedule_create(rt_rank* c) {
  rt_op b = rt_op_nop(c, 0), e = rt_op_nop(c, 0);
  std::lock_guard<std::mutex> g(c->mu);
  rt_sched id;
  if (!c->free_scheds.empty()) {
    id = c->free_scheds.back();
    c->free_scheds.pop_back();
    c->scheds[id] = Schedule();
  } else {
    c->scheds.emplace_back();
    id = (rt_sched)c->scheds.size() - 1;
  }
  c->scheds[id].begin = b;
  c->scheds[id].end = e;
  return id;
}

// Release a schedule with everything it owns: its operations, begin / end no-ops, the temporaries a
// collective made for itself and the schedules a composite one is built from (ffschedule_delete).
int rt_schedule_delete(rt_rank* c, rt_sched s) {
  rt_sched_fn custom = nullptr;
  std::vector<rt_sched> parts;
  {
    std::lock_guard<std::mutex> g(c->mu);
    if (s < 0 || s >= (rt_sched)c->scheds.size() || !c->scheds[s].alive) return RT_ERROR;
    custom = c->scheds[s].delete_fn;
    c->scheds[s].delete_fn = nullptr;      // the override may call back into the default
    parts = c->scheds[s].parts;
  }
  if (custom) return custom(c, s);
  for (rt_sched p : parts) rt_schedule_delete(c, p);
  std::lock_guard<std::mutex> g(c->mu);
  Schedule& sc = c->scheds[s];
  for (rt_op id : sc.ops) free_op_locked(c, id);
  free_op_locked(c, sc.begin);
  free_op_locked(c, sc.end);
  for (rt_buf b : sc.owned_bufs)
    if (b >= 0 && b < (rt_buf)c->bufs.size() && c->bufs[b].alive) {
      c->bufs[b] = Buffer();
      c->bufs[b].alive = false;
      c->free_bufs.push_back(b);
    }
  sc = Schedule();
  sc.alive = false;
  c->free_scheds.push_back(s);
  return RT_SUCCESS;
}

int rt_schedule_add_part(rt_rank* c, rt_sched s, rt_sched part) {
  std::lock_guard<std::mutex> g(c->mu);
  if (!ok_sched(c, s) || !ok_sched(c, part) || s == part) return RT_ERROR;
  c->scheds[s].parts.push_back(part);
  return RT_SUCCESS;
}

int rt_schedule_own_buffer(rt_rank* c, rt_sched s, rt_buf b) {
  std::lock_guard<std::mutex> g(c->mu);
  if (!ok_sched(c, s) || !ok_buf(c, b)) return RT_ERROR;
  c->scheds[s].owned_bufs.push_back(b);
  return RT_SUCCESS;
}

int rt_schedule_set_state(rt_rank* c, rt_sched s, void* state) {
  std::lock_guard<std::mutex> g(c->mu);
  if (!ok_sched(c, s)) return RT_ERROR;
  c->scheds[s].state = state;
  return RT_SUCCESS;
}
void* rt_schedule_get_state(rt_rank* c, rt_sched s) { std::lock_guard<std::mutex> g(c->mu); return ok_sched(c, s) ? c->scheds[s].state : nullptr; }

int rt_schedule_set_start_fun(rt_rank* c, rt_sched s, rt_sched_fn f) { std::lock_guard<std::mutex> g(c->mu); if (!ok_sched(c, s)) return RT_ERROR; c->scheds[s].start_fn = f; return RT_SUCCESS; }
int rt_schedule_set_post_fun(rt_rank* c, rt_sched s, rt_sched_fn f) { std::lock_guard<std::mutex> g(c->mu); if (!ok_sched(c, s)) return RT_ERROR; c->scheds[s].post_fn = f; return RT_SUCCESS; }
int rt_schedule_set_test_fun(rt_rank* c, rt_sched s, rt_sched_fn f) { std::lock_guard<std::mutex> g(c->mu); if (!ok_sched(c, s)) return RT_ERROR; c->scheds[s].test_fn = f; return RT_SUCCESS; }
int rt_schedule_set_delete_fun(rt_rank* c, rt_sched s, rt_sched_fn f) { std::lock_guard<std::mutex> g(c->mu); if (!ok_sched(c, s)) return RT_ERROR; c->scheds[s].delete_fn = f; return RT_SUCCESS; }
int rt_schedule_set_wait_fun(rt_rank* c, rt_sched s, rt_sched_wait_fn f) { std::lock_guard<std::mutex> g(c->mu); if (!ok_sched(c, s)) return RT_ERROR; c->scheds[s].wait_fn = f; return RT_SUCCESS; }
int rt_schedule_set_print_fun(rt_rank* c, rt_sched s, rt_sched_print_fn f) { std::lock_guard<std::mutex> g(c->mu); if (!ok_sched(c, s)) return RT_ERROR; c->scheds[s].print_fn = f; return RT_SUCCESS; }

// The default behaviours, callable from an override (ffschedule_default_*).
int rt_schedule_default_post(rt_rank* c, rt_sched s) {
  rt_schedule_finalize(c, s);
  return rt_op_post(c, rt_schedule_begin_op(c, s));
}
int rt_schedule_default_wait(rt_rank* c, rt_sched s, double timeout_s) { return rt_op_wait(c, rt_schedule_end_op(c, s), timeout_s); }
int rt_schedule_default_test(rt_rank* c, rt_sched s) { return rt_op_test(c, rt_schedule_end_op(c, s)); }

// ffschedule_default_delete / ffschedule_default_print: what an override calls for the schedule's own part.
int rt_schedule_default_delete(rt_rank* c, rt_sched s) {
  {
    std::lock_guard<std::mutex> g(c->mu);
    if (s < 0 || s >= (rt_sched)c->scheds.size() || !c->scheds[s].alive) return RT_ERROR;
    c->scheds[s].delete_fn = nullptr;
  }
  return rt_schedule_delete(c, s);
}
int rt_schedule_default_print(rt_rank* c, rt_sched s, char* out, int64_t cap) {
  rt_sched_print_fn custom = nullptr;
  {
    std::lock_guard<std::mutex> g(c->mu);
    if (s < 0 || s >= (rt_sched)c->scheds.size() || !c->scheds[s].alive) return RT_ERROR;
    custom = c->scheds[s].print_fn;
    c->scheds[s].print_fn = nullptr;
  }
  const int n = rt_schedule_print(c, s, out, cap);
  { std::lock_guard<std::mutex> g(c->mu); c->scheds[s].print_fn = custom; }
  return n;
}

// Arm a schedule once before its first post (a composite schedule posts its listening side here:
// ffsolo_allreduce.c:97-101).  The default does nothing.
int rt_schedule_start(rt_rank* c, rt_sched s) {
  rt_sched_fn f;
  { std::lock_guard<std::mutex> g(c->mu); if (!ok_sched(c, s)) return RT_ERROR; f = c->scheds[s].start_fn; }
  rt_schedule_finalize(c, s);
  return f ? f(c, s) : RT_SUCCESS;
}

int rt_schedule_add_op(rt_rank* c, rt_sched s, rt_op op) {
  std::lock_guard<std::mutex> g(c->mu);
  if (!ok_sched(c, s) || !ok_op(c, op)) return RT_ERROR;
  c->scheds[s].ops.push_back(op);
  return RT_SUCCESS;
}

// Root ops (no parent) hang off the begin no-op, leaf ops (no child) feed the end no-op
// (ffschedule.c:217-237 does this linking while ops are added).
int rt_schedule_finalize(rt_rank* c, rt_sched s) {
  std::vector<rt_op> roots, leaves;
  rt_op b, e;
  {
    std::lock_guard<std::mutex> g(c->mu);
    if (!ok_sched(c, s)) return RT_ERROR;
    Schedule& sc = c->scheds[s];
    if (sc.finalized) return RT_SUCCESS;
    sc.finalized = true;
    b = sc.begin; e = sc.end;
    for (rt_op id : sc.ops) {
      if (c->ops[id]->num_parents == 0) roots.push_back(id);
      if (c->ops[id]->edges.empty()) leaves.push_back(id);
    }
  }
  for (rt_op id : roots) rt_op_hb(c, b, id);
  for (rt_op id : leaves) rt_op_hb(c, id, e);
  if (roots.empty()) rt_op_hb(c, b, e);
  return RT_SUCCESS;
}

rt_op rt_schedule_begin_op(rt_rank* c, rt_sched s) { std::lock_guard<std::mutex> g(c->mu); return ok_sched(c, s) ? c->scheds[s].begin : RT_NONE; }
rt_op rt_schedule_end_op(rt_rank* c, rt_sched s) { std::lock_guard<std::mutex> g(c->mu); return ok_sched(c, s) ? c->scheds[s].end : RT_NONE; }

int rt_schedule_post(rt_rank* c, rt_sched s) {
  rt_sched_fn f;
  { std::lock_guard<std::mutex> g(c->mu); if (!ok_sched(c, s)) return RT_ERROR; f = c->scheds[s].post_fn; }
  return f ? f(c, s) : rt_schedule_default_post(c, s);
}
int rt_schedule_wait(rt_rank* c, rt_sched s, double timeout_s) {
  rt_sched_wait_fn f;
  { std::lock_guard<std::mutex> g(c->mu); if (!ok_sched(c, s)) return RT_ERROR; f = c->scheds[s].wait_fn; }
  return f ? f(c, s, timeout_s) : rt_schedule_default_wait(c, s, timeout_s);
}
int rt_schedule_test(rt_rank* c, rt_sched s) {
  rt_sched_fn f;
  { std::lock_guard<std::mutex> g(c->mu); if (!ok_sched(c, s)) return RT_ERROR; f = c->scheds[s].test_fn; }
  return f ? f(c, s) : rt_schedule_default_test(c, s);
}

int rt_schedule_print(rt_rank* c, rt_sched s, char* out, int64_t cap) {
  static const char* names[] = {"nop", "callback", "comp", "send", "recv"};
  {
    rt_sched_print_fn f;
    { std::lock_guard<std::mutex> g(c->mu); if (!ok_sched(c, s)) return RT_ERROR; f = c->scheds[s].print_fn; }
    if (f) return f(c, s, out, cap);
  }
  std::lock_guard<std::mutex> g(c->mu);
  Schedule& sc = c->scheds[s];
  std::string dot = "digraph schedule_" + std::to_string(c->id) + "_" + std::to_string(s) + " {\n";
  std::vector<rt_op> all = sc.ops;
  all.push_back(sc.begin);
  all.push_back(sc.end);
  for (rt_op id : all) {
    Op& op = *c->ops[id];
    dot += "  \"" + std::to_string(id) + "." + std::to_string(c->id) + "\" [label=\"" + names[op.type] +
           (id == sc.begin ? " begin" : id == sc.end ? " end" : "") + "\"];\n";
    for (const Edge& ed : op.edges) {
      const rt_op ch = ed.child;
      if (ch == RT_NONE) continue;
      dot += "  \"" + std::to_string(id) + "." + std::to_string(c->id) + "\" -> \"" + std::to_string(ch) + "." +
             std::to_string(c->id) + "\";\n";
    }
  }
  dot += "}\n";
  if ((int64_t)dot.size() + 1 > cap) return RT_ERROR;
  memcpy(out, dot.c_str(), dot.size() + 1);
  return (int)dot.size();
}

// The same graph as two JSON arrays for vis.js network views (ffschedule.c:111-161 prints both forms):
// {"nodes": [{"id": "7.0", "label": "send"}, ...], "edges": [{"from": "7.0", "to": "9.0"}, ...]}
int rt_schedule_print_visjs(rt_rank* c, rt_sched s, char* out, int64_t cap) {
  static const char* names[] = {"nop", "callback", "comp", "send", "recv"};
  std::lock_guard<std::mutex> g(c->mu);
  if (!ok_sched(c, s)) return RT_ERROR;
  Schedule& sc = c->scheds[s];
  std::vector<rt_op> all = sc.ops;
  all.push_back(sc.begin);
  all.push_back(sc.end);
  const std::string r = "." + std::to_string(c->id);
  std::string nodes, edges;
  for (rt_op id : all) {
    Op& op = *c->ops[id];
    if (!nodes.empty()) nodes += ", ";
    nodes += "{\"id\": \"" + std::to_string(id) + r + "\", \"label\": \"" + names[op.type] +
             (id == sc.begin ? " begin" : id == sc.end ? " end" : "") + "\"}";
    for (const Edge& ed : op.edges) {
      if (ed.child == RT_NONE) continue;
      if (!edges.empty()) edges += ", ";
      edges += "{\"from\": \"" + std::to_string(id) + r + "\", \"to\": \"" + std::to_string(ed.child) + r +
               "\", \"arrows\": \"to\"}";
    }
  }
  const std::string js = "{\"nodes\": [" + nodes + "], \"edges\": [" + edges + "]}\n";
  if ((int64_t)js.size() + 1 > cap) return RT_ERROR;
  memcpy(out, js.c_str(), js.size() + 1);
  return (int)js.size();
}

// Recursive doubling for any P: ranks beyond the largest power of two first fold into a
// partner, the power-of-two core exchanges in log2 rounds, and the result is sent back.
rt_sched rt_allreduce(rt_rank* c, rt_buf snd, rt_buf rcv, int tag, int oper) {
  const int P = c->world->n, me = c->id;
  {
    std::lock_guard<std::mutex> g(c->mu);
    if (!ok_buf(c, rcv) || (snd != RT_INPLACE && !ok_buf(c, snd))) return RT_ERROR;
  }
  rt_sched s = rt_schedule_create(c);
  int p2 = 1;
  while (p2 * 2 <= P) p2 *= 2;
  const int extra = P - p2;
  int64_t count;
  int dtype;
  { std::lock_guard<std::mutex> g(c->mu); count = c->bufs[rcv].count; dtype = c->bufs[rcv].dtype; }
  rt_op last = RT_NONE;
  auto chain = [&](rt_op op) { if (last != RT_NONE) rt_op_hb(c, last, op); rt_schedule_add_op(c, s, op); last = op; };
  if (snd != RT_INPLACE) chain(rt_op_comp(c, snd, RT_NONE, rcv, RT_IDENTITY, 0));
  else chain(rt_op_nop(c, 0));
  if (me >= p2) {                       // fold into the core, then receive the result
    chain(rt_op_send(c, rcv, me - p2, tag, 0));
    chain(rt_op_recv(c, rcv, me - p2, tag, 0));
    rt_schedule_finalize(c, s);
    return s;
  }
  if (me < extra) {
    rt_buf tmp = rt_buffer_create(c, nullptr, count, dtype);
    rt_schedule_own_buffer(c, s, tmp);
    chain(rt_op_recv(c, tmp, me + p2, tag, 0));
    chain(rt_op_comp(c, tmp, rcv, rcv, oper, 0));
  }
  for (int mask = 1; mask < p2; mask <<= 1) {
    const int peer = me ^ mask;
    rt_buf tmp = rt_buffer_create(c, nullptr, count, dtype);
    rt_schedule_own_buffer(c, s, tmp);
    rt_op sd = rt_op_send(c, rcv, peer, tag, 0);
    rt_op rv = rt_op_recv(c, tmp, peer, tag, 0);
    rt_op cp = rt_op_comp(c, tmp, rcv, rcv, oper, 0);
    rt_op_hb(c, last, rv);              // listen first: a partner that sends now can copy straight into tmp ...
    rt_op_hb(c, last, sd);              // ... then send what has been reduced so far
    rt_op_hb(c, sd, cp);
    rt_op_hb(c, rv, cp);
    rt_schedule_add_op(c, s, sd);
    rt_schedule_add_op(c, s, rv);
    rt_schedule_add_op(c, s, cp);
    last = cp;
  }
  if (me < extra) chain(rt_op_send(c, rcv, me + p2, tag, 0));
  rt_schedule_finalize(c, s);
  return s;
}

// The listening side of an activation schedule is armed by rt_schedule_start (or the first rt_schedule_post): the
// caller hangs its dependents on `joined` first, so that an activation from a faster rank cannot pass them by.
// Tokens that arrive earlier wait in the mailbox.
static int activation_arm(rt_rank* c, rt_sched s) {
  std::vector<rt_op> recvs;
  {
    std::lock_guard<std::mutex> g(c->mu);
    Schedule& sc = c->scheds[s];
    if (sc.state) return RT_SUCCESS;                    // armed already
    sc.state = (void*)1;
    for (rt_op id : sc.ops)
      if (c->ops[id] && c->ops[id]->type == T_RECV) recvs.push_back(id);
  }
  for (rt_op rv : recvs) rt_op_post(c, rv);
  return RT_SUCCESS;
}

// Activation from any rank: the activator sends a token to everybody; on every rank the
// `joined` no-op (OR) completes once per activation, whether it was local or remote.
// With an all-to-all fabric there is no need for the reference's forwarding tree.
rt_sched rt_activation(rt_rank* c, int tag, rt_op* activate, rt_op* joined) {
  const int P = c->world->n, me = c->id;
  rt_sched s = rt_schedule_create(c);
  rt_buf token = rt_buffer_create(c, nullptr, 1, RT_INT32);
  rt_schedule_own_buffer(c, s, token);
  rt_op act = rt_op_nop(c, 0);
  rt_op join = rt_op_nop(c, RT_DEP_OR);
  rt_schedule_add_op(c, s, act);
  rt_schedule_add_op(c, s, join);
  rt_op_hb(c, act, join);
  for (int r = 0; r < P; ++r) {
    if (r == me) continue;
    rt_op sd = rt_op_send(c, token, r, tag, 0);
    rt_op_hb(c, act, sd);
    rt_schedule_add_op(c, s, sd);
    // a persistent receive per peer: it re-arms itself after every token
    rt_buf rb = rt_buffer_create(c, nullptr, 1, RT_INT32);
    rt_schedule_own_buffer(c, s, rb);
    rt_op rv = rt_op_recv(c, rb, r, tag, RT_DEP_OR);
    rt_op_hb(c, rv, join);
    rt_op_hb(c, rv, rv);
    rt_schedule_add_op(c, s, rv);
  }
  {
    std::lock_guard<std::mutex> g(c->mu);
    c->scheds[s].finalized = true;                      // wired by hand
    c->scheds[s].start_fn = activation_arm;
    c->scheds[s].post_fn = activation_arm;              // the reference arms it with ffschedule_post
  }
  *activate = act;
  *joined = join;
  return s;
}

int rt_limiter(rt_rank* c, int num_async, rt_op* start, rt_op* async_ops, rt_op* sync_op) {
  rt_op st = rt_op_nop(c, RT_DEP_FIRST);
  for (int i = 0; i < num_async; ++i) {
    async_ops[i] = rt_op_nop(c, RT_DEP_OR);
    rt_op_hb(c, st, async_ops[i]);
  }
  *sync_op = rt_op_nop(c, RT_DEP_OR);
  rt_op_hb(c, st, *sync_op);
  *start = st;
  return RT_SUCCESS;
}

}  // extern "C"

// ---- partial allreduces as schedules of this runtime ------------------------------------------------------------------
// The reference builds its solo and majority allreduces from an activation schedule, two allreduce schedules and a
// limiter, glued by version-checked edges (fflib2 src/colls/ffsolo_allreduce.c:21-148, ffrand_allreduce.c:27-128,
// ffactivation.c:11-106).  Here the rounds are numbered instead: a rank's j-th post belongs to round j, the token
// that activates a round carries its number, and every rank runs every round in order.  A post that finds its round
// already begun (another rank activated it) has nothing left to start; what it staged goes into the next round.
namespace {

struct TokenArg;

struct Partial {
  rt_rank* c = nullptr;
  rt_sched self = RT_NONE, ar_data = RT_NONE, ar_cnt = RT_NONE;
  rt_buf snd = RT_NONE, rcv = RT_NONE, stage = RT_NONE, work = RT_NONE, flag = RT_NONE, tok_out = RT_NONE;
  std::vector<rt_buf> tok_in;
  std::vector<rt_op> sends, recvs, tok_cbs;
  rt_op cb_post = RT_NONE, cb_begin = RT_NONE, cb_end = RT_NONE;
  int mode = 0;            // 0: solo (whoever posts first activates), 1: majority (one drawn rank per round activates)
  int oper = RT_SUM, dtype = RT_FLOAT, tag = 0, options = 0;
  int token_tag = 0;       // tag of the activation tokens: the user's tag and which schedule of that tag this is, so that a
                           // schedule which is about to be deleted never swallows a token meant for its successor
  int64_t count = 0, limiter = -1;
  uint64_t seed = 0;
  bool started_flag = false;
  std::vector<TokenArg*> token_args;
  // everything below is guarded by mu
  std::mutex mu;
  bool fresh = false;      // the stage holds a contribution that no round has taken yet
  int64_t posts = 0, posted_by_user = 0, started = 0, begun = 0, done = 0, queued = 0;
  int64_t token_wish = -1;   // newest round a peer's token has asked for
  bool running = false;
  int64_t activated = 0, late = 0, sync_rounds = 0, overwritten = 0, last_contributors = 0, last_round = -1;

  bool is_sync(int64_t j) const { return limiter >= 0 && (j % (limiter + 1)) == limiter; }
  int activator(int64_t j) const {           // the same draw on every rank (ffrand_allreduce.c:88 uses rand_r)
    uint64_t z = seed + 0x9e3779b97f4a7c15ULL * (uint64_t)(j + 1);
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ULL;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebULL;
    z ^= z >> 31;
    return (int)(z % (uint64_t)c->world->n);
  }
};

struct TokenArg { Partial* st; int peer; };

template <class T>
void fill_typed(T* p, int64_t n, int oper) {
  T v = T(0);
  if (oper == RT_PROD) v = T(1);
  else if (oper == RT_MAX) v = std::numeric_limits<T>::lowest();
  else if (oper == RT_MIN) v = std::numeric_limits<T>::max();
  for (int64_t i = 0; i < n; ++i) p[i] = v;
}

// The neutral element of a built-in operator: what a rank without a fresh contribution puts into a round.
void fill_neutral(void* p, int64_t n, int dtype, int oper) {
  switch (dtype) {
    case RT_INT32: fill_typed((int32_t*)p, n, oper); break;
    case RT_INT64: fill_typed((int64_t*)p, n, oper); break;
    case RT_CHAR: fill_typed((signed char*)p, n, oper); break;
    case RT_FLOAT: fill_typed((float*)p, n, oper); break;
    default: fill_typed((double*)p, n, oper); break;
  }
}

// Ask for every round up to j.  Returns how many times cb_begin has to be posted now (0 or 1).  Called with st->mu held.
// `own_post`: the request comes from this rank's post of round j.  A token from a peer never takes a rank across a
// synchronous round that the rank has not posted itself (a peer that posts ahead without waiting could send one): what
// the token asked for is remembered and granted when the rank's own post has begun that round.
int request_upto_locked(Partial* st, int64_t j, bool own_post) {
  int post_now = 0;
  if (!own_post && j > st->token_wish) st->token_wish = j;
  while (st->started <= j) {
    // a synchronous round begins on a rank with that rank's own post of this very round, and with nothing else
    if (st->is_sync(st->started) && !(own_post && st->started == j)) break;
    st->started++;
    if (st->running) st->queued++;
    else { st->running = true; post_now = 1; }
  }
  if (own_post && st->token_wish >= st->started) post_now |= request_upto_locked(st, st->token_wish, false);
  return post_now;
}

// The user's post has reached the progress thread.
void partial_on_post(rt_op, void* arg) {
  Partial* st = (Partial*)arg;
  bool activate = false;
  int post_now = 0;
  int64_t j;
  {
    std::lock_guard<std::mutex> g(st->mu);
    j = st->posts++;
    const bool sync = st->is_sync(j);
    if (st->started <= j) {
      if (sync) post_now = request_upto_locked(st, j, true);
      else if (st->mode == 0 || st->activator(j) == st->c->id) {
        activate = true;
        st->activated++;
        post_now = request_upto_locked(st, j, true);
      }
    } else if (!sync) {
      st->late++;
    }
  }
  if (activate) {
    *(int64_t*)rt_buffer_data(st->c, st->tok_out) = j;
    for (rt_op sd : st->sends) rt_op_post(st->c, sd);    // they run before the round begins: the queue is FIFO
  }
  if (post_now) rt_op_post(st->c, st->cb_begin);
}

// A token from a peer: it names the newest round that peer has activated.
void partial_on_token(rt_op, void* arg) {
  TokenArg* ta = (TokenArg*)arg;
  Partial* st = ta->st;
  const int64_t t = *(int64_t*)rt_buffer_data(st->c, st->tok_in[ta->peer]);
  int post_now = 0;
  {
    std::lock_guard<std::mutex> g(st->mu);
    if (t >= st->started) post_now = request_upto_locked(st, t, false);
  }
  if (post_now) rt_op_post(st->c, st->cb_begin);
}

// A round begins on this rank: its contribution is what the user staged since the last round, or nothing.
void partial_on_begin(rt_op, void* arg) {
  Partial* st = (Partial*)arg;
  int32_t* flag = (int32_t*)rt_buffer_data(st->c, st->flag);
  const size_t bytes = (size_t)st->count * dtype_size(st->dtype);
  const bool keeps_last = (st->options & RT_PARTIAL_STALE) || st->oper >= RT_CUSTOM0;
  std::lock_guard<std::mutex> g(st->mu);
  const int64_t round = st->begun++;
  if (st->is_sync(round)) st->sync_rounds++;
  if (st->options & RT_PARTIAL_LIVE) {                 // the reference's way: whatever the send buffer holds right now
    memcpy(rt_buffer_data(st->c, st->work), rt_buffer_data(st->c, st->snd), bytes);
    *flag = st->fresh ? 1 : 0;
    st->fresh = false;
    return;
  }
  if (st->fresh && !keeps_last) {
    // the staged contribution becomes the round's working vector by exchanging the two buffers' storage: the
    // stage is rewritten by the next post anyway
    std::lock_guard<std::mutex> gc(st->c->mu);
    std::swap(st->c->bufs[st->stage].own, st->c->bufs[st->work].own);
    st->fresh = false;
    *flag = 1;
    return;
  }
  void* work = rt_buffer_data(st->c, st->work);
  void* stage = rt_buffer_data(st->c, st->stage);
  if (st->fresh) {
    memcpy(work, stage, bytes);
    st->fresh = false;
    *flag = 1;
  } else {
    *flag = 0;
    if (keeps_last) memcpy(work, stage, bytes);          // its last contribution again
    else fill_neutral(work, st->count, st->dtype, st->oper);
  }
}

// The round has ended everywhere it matters for this rank: hand the result over and begin the next one if asked.
void partial_on_end(rt_op, void* arg) {
  Partial* st = (Partial*)arg;
  void* rcv = rt_buffer_data(st->c, st->rcv);
  const int32_t contributors = *(int32_t*)rt_buffer_data(st->c, st->flag);
  int post_now = 0;
  {
    std::lock_guard<std::mutex> g(st->mu);
    const void* work = rt_buffer_data(st->c, st->work);
    memcpy(rcv, work, (size_t)st->count * dtype_size(st->dtype));
    st->last_contributors = contributors;
    st->last_round = st->done++;
    st->running = false;
    if (st->queued > 0) { st->queued--; st->running = true; post_now = 1; }
  }
  if (post_now) rt_op_post(st->c, st->cb_begin);
}

int partial_start(rt_rank* c, rt_sched s) {
  Partial* st = (Partial*)rt_schedule_get_state(c, s);
  if (!st) return RT_ERROR;
  if (st->started_flag) return RT_SUCCESS;
  st->started_flag = true;
  for (rt_op rv : st->recvs) rt_op_post(c, rv);          // listen for tokens from now on
  return RT_SUCCESS;
}

// Runs in the caller's thread: the contribution is taken here, so the caller may reuse its buffer at once.
int partial_post(rt_rank* c, rt_sched s) {
  Partial* st = (Partial*)rt_schedule_get_state(c, s);
  if (!st || !st->started_flag) return RT_ERROR;
  const void* snd = rt_buffer_data(c, st->snd);
  if (st->options & RT_PARTIAL_LIVE) {                   // nothing is copied here: rounds read the send buffer themselves
    { std::lock_guard<std::mutex> g(st->mu); st->fresh = true; st->posted_by_user++; }
    return rt_op_post(c, st->cb_post);
  }
  {
    std::lock_guard<std::mutex> g(st->mu);
    void* stage = rt_buffer_data(c, st->stage);          // under the lock: a round that begins exchanges stage and work
    if (st->fresh && (st->options & RT_PARTIAL_ACCUMULATE) && st->oper < RT_CUSTOM0 && st->oper != RT_IDENTITY) {
      // what no round has taken yet is combined with the new contribution instead of being replaced by it
      switch (st->dtype) {
        case RT_INT32: reduce_typed((const int32_t*)stage, (const int32_t*)snd, (int32_t*)stage, st->count, st->oper); break;
        case RT_INT64: reduce_typed((const int64_t*)stage, (const int64_t*)snd, (int64_t*)stage, st->count, st->oper); break;
        case RT_CHAR: reduce_typed((const signed char*)stage, (const signed char*)snd, (signed char*)stage, st->count, st->oper); break;
        case RT_FLOAT: reduce_typed((const float*)stage, (const float*)snd, (float*)stage, st->count, st->oper); break;
        default: reduce_typed((const double*)stage, (const double*)snd, (double*)stage, st->count, st->oper); break;
      }
    } else {
      if (st->fresh) st->overwritten++;                  // the reference's behaviour: the older contribution is lost
      memcpy(stage, snd, (size_t)st->count * dtype_size(st->dtype));
    }
    st->fresh = true;
    st->posted_by_user++;
  }
  return rt_op_post(c, st->cb_post);
}

int partial_delete(rt_rank* c, rt_sched s) {
  Partial* st = (Partial*)rt_schedule_get_state(c, s);
  if (!st) return RT_ERROR;
  std::vector<rt_op> cbs = st->tok_cbs;
  cbs.push_back(st->cb_post); cbs.push_back(st->cb_begin); cbs.push_back(st->cb_end);
  {                                    // tokens of concurrent activators that nobody will read any more
    std::lock_guard<std::mutex> g(c->world->mail_mu);
    for (int r = 0; r < c->world->n; ++r) c->world->mail.erase(std::make_tuple(r, c->id, wire_tag(st->token_tag, RT_SHADOW_TAG)));
  }
  const int rc = rt_schedule_default_delete(c, s);       // operations, parts, owned buffers
  for (int spins = 0; spins < 2000000; ++spins) {        // a callback of this schedule may still be returning
    {
      std::lock_guard<std::mutex> g(c->mu);
      bool busy = false;
      for (rt_op id : cbs) busy = busy || c->in_callback == id;
      if (!busy) break;
    }
    std::this_thread::yield();
  }
  { std::lock_guard<std::mutex> g(c->mu); c->partials.erase(s); }
  for (TokenArg* ta : st->token_args) delete ta;
  delete st;
  return rc;
}

int partial_print(rt_rank* c, rt_sched s, char* out, int64_t cap) {
  Partial* st = (Partial*)rt_schedule_get_state(c, s);
  if (!st || cap < 1) return RT_ERROR;
  int64_t used = 0;
  for (rt_sched part : {st->ar_data, st->ar_cnt}) {      // the parts first, as ffsolo_allreduce_print does
    const int n = rt_schedule_print(c, part, out + used, cap - used);
    if (n < 0) return RT_ERROR;
    used += n;
  }
  const int n = rt_schedule_default_print(c, s, out + used, cap - used);
  return n < 0 ? RT_ERROR : (int)(used + n);
}

rt_sched make_partial(rt_rank* c, rt_buf snd, rt_buf rcv, int tag, int oper, int mode, uint64_t seed, int limiter,
                      int options) {
  const int P = c->world->n, me = c->id;
  int64_t count;
  int dtype;
  {
    std::lock_guard<std::mutex> g(c->mu);
    if (snd < 0 || rcv < 0 || snd >= (rt_buf)c->bufs.size() || rcv >= (rt_buf)c->bufs.size()) return RT_ERROR;
    count = c->bufs[rcv].count; dtype = c->bufs[rcv].dtype;
    if (c->bufs[snd].count != count || c->bufs[snd].dtype != dtype) return RT_ERROR;
  }
  Partial* st = new Partial();
  st->c = c; st->snd = snd; st->rcv = rcv; st->tag = tag; st->oper = oper; st->mode = mode; st->seed = seed;
  st->limiter = limiter; st->options = options; st->count = count; st->dtype = dtype;
  {
    std::lock_guard<std::mutex> g(c->mu);
    st->token_tag = (tag & 0xffff) | (int)((c->partial_generation[tag]++ & 0x3ff) << 16);
  }
  rt_sched s = rt_schedule_create(c);
  st->self = s;
  auto own = [&](int64_t n, int dt) { rt_buf b = rt_buffer_create(c, nullptr, n, dt); rt_schedule_own_buffer(c, s, b); return b; };
  st->stage = own(count, dtype);
  st->work = own(count, dtype);
  st->flag = own(1, RT_INT32);
  st->tok_out = own(1, RT_INT64);
  if (!(options & RT_PARTIAL_STALE) && oper < RT_CUSTOM0)
    fill_neutral(rt_buffer_data(c, st->stage), count, dtype, oper);
  st->ar_data = rt_allreduce(c, RT_INPLACE, st->work, tag, oper);
  st->ar_cnt = rt_allreduce(c, RT_INPLACE, st->flag, tag, RT_SUM);   // how many ranks put something fresh into the round
  rt_schedule_add_part(c, s, st->ar_data);
  rt_schedule_add_part(c, s, st->ar_cnt);
  auto add = [&](rt_op op) { rt_schedule_add_op(c, s, op); return op; };
  st->cb_post = add(rt_op_callback(c, partial_on_post, st, RT_DEP_OR));
  st->cb_begin = add(rt_op_callback(c, partial_on_begin, st, RT_DEP_OR));
  st->cb_end = add(rt_op_callback(c, partial_on_end, st, RT_DEP_OR));
  rt_op_hb(c, st->cb_begin, rt_schedule_begin_op(c, st->ar_data));
  rt_op_hb(c, rt_schedule_end_op(c, st->ar_data), rt_schedule_begin_op(c, st->ar_cnt));
  rt_op_hb(c, rt_schedule_end_op(c, st->ar_cnt), st->cb_end);
  rt_op_hb(c, st->cb_end, rt_schedule_end_op(c, s));      // the schedule's end completes once per round
  rt_op_hb(c, rt_schedule_begin_op(c, s), st->cb_post);
  st->tok_in.assign(P, RT_NONE);
  for (int r = 0; r < P; ++r) {
    if (r == me) continue;
    st->sends.push_back(add(rt_op_send(c, st->tok_out, r, st->token_tag, RT_SHADOW_TAG | RT_DEP_OR)));
    st->tok_in[r] = own(1, RT_INT64);
    rt_op rv = add(rt_op_recv(c, st->tok_in[r], r, st->token_tag, RT_SHADOW_TAG | RT_DEP_OR));
    TokenArg* ta = new TokenArg{st, r};
    st->token_args.push_back(ta);
    rt_op cb = add(rt_op_callback(c, partial_on_token, ta, RT_DEP_OR));
    rt_op_hb(c, rv, cb);                                  // read the token, then listen again
    rt_op_hb(c, cb, rv);
    st->recvs.push_back(rv);
    st->tok_cbs.push_back(cb);
  }
  {
    std::lock_guard<std::mutex> g(c->mu);
    c->scheds[s].finalized = true;                        // wired by hand: no automatic begin / end links
    c->scheds[s].state = st;
    c->scheds[s].start_fn = partial_start;
    c->scheds[s].post_fn = partial_post;
    c->scheds[s].delete_fn = partial_delete;
    c->scheds[s].print_fn = partial_print;
    c->partials[s] = st;
  }
  return s;
}

}  // namespace

rt_rank::~rt_rank() {                  // partial allreduces that were never deleted
  for (auto& kv : partials) {
    for (TokenArg* ta : kv.second->token_args) delete ta;
    delete kv.second;
  }
}

extern "C" {

rt_sched rt_solo_allreduce(rt_rank* c, rt_buf snd, rt_buf rcv, int tag, int op, int limiter, int options) {
  return make_partial(c, snd, rcv, tag, op, 0, 0, limiter, options);
}

rt_sched rt_rand_allreduce(rt_rank* c, rt_buf snd, rt_buf rcv, int tag, int op, int seed, int limiter, int options) {
  return make_partial(c, snd, rcv, tag, op, 1, (uint64_t)(uint32_t)seed, limiter, options);
}

int rt_partial_info(rt_rank* c, rt_sched s, int64_t* out) {
  Partial* st;
  { std::lock_guard<std::mutex> g(c->mu); auto it = c->partials.find(s); if (it == c->partials.end()) return RT_ERROR; st = it->second; }
  std::lock_guard<std::mutex> g(st->mu);
  out[0] = st->posted_by_user; out[1] = st->done; out[2] = st->activated; out[3] = st->late; out[4] = st->sync_rounds;
  out[5] = st->last_contributors; out[6] = st->last_round; out[7] = st->overwritten; out[8] = st->fresh ? 1 : 0;
  return RT_SUCCESS;
}

int rt_partial_read(rt_rank* c, rt_sched s, void* out, int64_t* contributors, int64_t* round) {
  Partial* st;
  { std::lock_guard<std::mutex> g(c->mu); auto it = c->partials.find(s); if (it == c->partials.end()) return RT_ERROR; st = it->second; }
  const void* rcv = rt_buffer_data(c, st->rcv);
  std::lock_guard<std::mutex> g(st->mu);
  if (out) memcpy(out, rcv, (size_t)st->count * dtype_size(st->dtype));
  if (contributors) *contributors = st->last_contributors;
  if (round) *round = st->last_round;
  return RT_SUCCESS;
}

int rt_partial_activator(rt_rank* c, rt_sched s, int64_t round) {
  Partial* st;
  { std::lock_guard<std::mutex> g(c->mu); auto it = c->partials.find(s); if (it == c->partials.end()) return RT_ERROR; st = it->second; }
  if (st->mode != 1 || st->is_sync(round)) return -1;
  return st->activator(round);
}

// Micro-benchmark of the runtime by itself (no interpreter in the loop): `ranks` native threads run the protocol
// of the reference's allreduce programs on int32 vectors of `count` elements, checked against the closed form.
//   fresh = 1: a new schedule per iteration — create, post, wait, delete (evaluation/allreduce.c:44-72);
//   fresh = 0: one persistent schedule posted `iters` times (evaluation/allreduce_inplace.c, benchmark/allreduce.c).
// out_us[0] = mean microseconds per iteration (slowest rank), out_us[1] = creation of the first schedule,
// out_us[2] = 1.0 if every result was right.
int rt_bench_allreduce(int ranks, int64_t count, int iters, int fresh, double* out_us) {
  if (ranks < 1 || count < 1 || iters < 1) return RT_ERROR;
  rt_world* w = rt_world_create(ranks);
  std::vector<double> per(ranks, 0.0), create(ranks, 0.0);
  std::vector<int> ok(ranks, 1);
  std::atomic<int> arrived{0};
  auto body = [&](int r) {
    rt_rank* c = rt_world_rank(w, r);
    std::vector<int32_t> snd(count), rcv(count);
    rt_buf bs = rt_buffer_create(c, snd.data(), count, RT_INT32), br = rt_buffer_create(c, rcv.data(), count, RT_INT32);
    auto t0 = std::chrono::steady_clock::now();
    rt_sched s = rt_allreduce(c, bs, br, 0, RT_SUM);
    create[r] = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count();
    arrived.fetch_add(1);
    while (arrived.load() < ranks) std::this_thread::yield();
    const int warm = 5;
    std::chrono::steady_clock::time_point start;
    for (int it = 0; it < iters + warm; ++it) {
      if (it == warm) start = std::chrono::steady_clock::now();
      for (int64_t j = 0; j < count; ++j) { snd[j] = (int32_t)(it + j); rcv[j] = 0; }
      if (fresh && it > 0) s = rt_allreduce(c, bs, br, it & 0x7f, RT_SUM);
      rt_schedule_post(c, s);
      if (rt_schedule_wait(c, s, 30.0) != RT_SUCCESS) { ok[r] = 0; break; }
      for (int64_t j = 0; j < count; ++j)
        if (rcv[j] != (int32_t)((it + j) * ranks)) { ok[r] = 0; break; }
      if (fresh) rt_schedule_delete(c, s);
    }
    per[r] = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - start).count() / iters;
  };
  std::vector<std::thread> th;
  for (int r = 0; r < ranks; ++r) th.emplace_back(body, r);
  for (auto& t : th) t.join();
  rt_world_destroy(w);
  double worst = 0, cr = 0, good = 1;
  for (int r = 0; r < ranks; ++r) {
    if (per[r] > worst) worst = per[r];
    if (create[r] > cr) cr = create[r];
    if (!ok[r]) good = 0;
  }
  out_us[0] = worst; out_us[1] = cr; out_us[2] = good;
  return RT_SUCCESS;
}

// The reference's SGD-loop timing programs on this runtime (evaluation/ssgd.c:63-97, rsgd.c:77-113,
// randomsgd.c:78-113): every iteration rank r first sleeps r * skew_us, fills its vector with ones, times post + wait
// of the persistent collective, clears the vector, and meets the others at a barrier.  mode 0: synchronous allreduce,
// 1: solo, 2: majority (limiter 1024 as in those programs).  out[0]: microseconds per post + wait, averaged over
// ranks and over the iterations after the second (the figure those programs print); out[1]: mean number of fresh
// contributors per round as the ranks saw it after their waits; out[2]: 1.0 if every result read was a whole number
// between 0 and the number of ranks.
int rt_bench_partial(int ranks, int64_t count, int iters, int mode, int skew_us, double* out) {
  if (ranks < 1 || count < 1 || iters < 3 || mode < 0 || mode > 2) return RT_ERROR;
  rt_world* w = rt_world_create(ranks);
  std::vector<double> per(ranks, 0.0), contrib(ranks, 0.0);
  std::vector<int> ok(ranks, 1);
  std::atomic<int64_t> arrived{0};
  auto barrier = [&](int64_t generation) {
    arrived.fetch_add(1);
    int polls = 0;
    while (arrived.load() < generation * ranks)
      if ((++polls & 255) == 0) std::this_thread::sleep_for(std::chrono::microseconds(20)); else std::this_thread::yield();
  };
  auto body = [&](int r) {
    rt_rank* c = rt_world_rank(w, r);
    std::vector<float> snd(count, 0.f), rcv(count, 0.f), res(count, 0.f);
    rt_buf bs = rt_buffer_create(c, snd.data(), count, RT_FLOAT), br = rt_buffer_create(c, rcv.data(), count, RT_FLOAT);
    rt_sched s = mode == 0 ? rt_allreduce(c, bs, br, 0, RT_SUM)
               : mode == 1 ? rt_solo_allreduce(c, bs, br, 0, RT_SUM, 1024, 0)
                           : rt_rand_allreduce(c, bs, br, 0, RT_SUM, 1234, 1024, 0);
    rt_schedule_start(c, s);
    barrier(1);
    for (int it = 0; it < iters; ++it) {
      if (skew_us > 0 && r > 0) std::this_thread::sleep_for(std::chrono::microseconds((int64_t)r * skew_us));
      for (int64_t j = 0; j < count; ++j) snd[j] = 1.f;
      const auto t0 = std::chrono::steady_clock::now();
      rt_schedule_post(c, s);
      if (rt_schedule_wait(c, s, 30.0) != RT_SUCCESS) { ok[r] = 0; break; }
      const double us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count();
      int64_t k = ranks, rnd = 0;
      if (mode == 0) { res[0] = rcv[0]; res[count - 1] = rcv[count - 1]; }
      else rt_partial_read(c, s, res.data(), &k, &rnd);
      if (res[0] < 0.f || res[0] > (float)ranks || res[0] != (float)(int)res[0] || res[count - 1] != res[0]) ok[r] = 0;
      if (it >= 2) { per[r] += us; contrib[r] += (double)k; }
      for (int64_t j = 0; j < count; ++j) snd[j] = 0.f;
      barrier(it + 2);
    }
    rt_schedule_delete(c, s);
  };
  std::vector<std::thread> th;
  for (int r = 0; r < ranks; ++r) th.emplace_back(body, r);
  for (auto& t : th) t.join();
  rt_world_destroy(w);
  double us = 0, k = 0, good = 1;
  for (int r = 0; r < ranks; ++r) { us += per[r]; k += contrib[r]; if (!ok[r]) good = 0; }
  out[0] = us / ranks / (iters - 2); out[1] = k / ranks / (iters - 2); out[2] = good;
  return RT_SUCCESS;
}

}  // extern "C"
