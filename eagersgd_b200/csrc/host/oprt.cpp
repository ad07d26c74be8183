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
#include <cstring>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <tuple>
#include <vector>

namespace {

size_t dtype_size(int dt) { return (dt == RT_INT32 || dt == RT_FLOAT) ? 4 : 8; }

enum OpType { T_NOP, T_CALLBACK, T_COMP, T_SEND, T_RECV };

struct Buffer {
  void* ptr = nullptr;
  std::vector<uint8_t> own;
  int64_t count = 0;
  int dtype = RT_FLOAT;
  void* data() { return ptr ? ptr : (void*)own.data(); }
};

struct Op {
  OpType type = T_NOP;
  int options = 0;
  rt_buf a = RT_NONE, b = RT_NONE, out = RT_NONE;
  int oper = RT_SUM, peer = -1, tag = 0;
  rt_callback_fn cb = nullptr;
  void* cb_arg = nullptr;
  std::vector<rt_op> children;
  int num_parents = 0;
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
  std::vector<rt_op> ops;
  rt_op begin = RT_NONE, end = RT_NONE;
  bool finalized = false;
};

}  // namespace

struct rt_world {
  int n = 0;
  std::vector<std::unique_ptr<rt_rank>> ranks;
  std::mutex mail_mu;
  std::map<std::tuple<int, int, int>, std::deque<Message>> mail;  // (src, dst, tag) -> FIFO
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
  std::thread progress;
  std::atomic<bool> stop{false};
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
    c->custom_ops[op.oper - RT_CUSTOM0](A.data(), B.data(), O.data(), n, A.dtype);
    return;
  }
  switch (A.dtype) {
    case RT_INT32: reduce_typed((const int32_t*)A.data(), (const int32_t*)B.data(), (int32_t*)O.data(), n, op.oper); break;
    case RT_INT64: reduce_typed((const int64_t*)A.data(), (const int64_t*)B.data(), (int64_t*)O.data(), n, op.oper); break;
    case RT_FLOAT: reduce_typed((const float*)A.data(), (const float*)B.data(), (float*)O.data(), n, op.oper); break;
    default: reduce_typed((const double*)A.data(), (const double*)B.data(), (double*)O.data(), n, op.oper); break;
  }
}

void trigger(rt_rank* c, rt_op id);

// Called with c->mu held.
void complete(rt_rank* c, rt_op id) {
  Op& op = *c->ops[id];
  op.completed.fetch_add(1);
  c->cv.notify_all();
  if (op.children.empty()) return;
  if (op.options & RT_DEP_FIRST) {           // satisfy exactly one dependent, in turn
    rt_op child = op.children[op.first_rr % op.children.size()];
    op.first_rr++;
    trigger(c, child);
  } else {
    for (rt_op child : op.children) trigger(c, child);
  }
}

// A parent of `id` has completed.  Called with c->mu held.
void trigger(rt_rank* c, rt_op id) {
  Op& op = *c->ops[id];
  if ((op.options & RT_NON_PERSISTENT) && op.executed > 0) return;
  if (op.options & RT_DEP_OR) {
    c->posted.push_back(id);
  } else {
    if (op.dep_left <= 0) op.dep_left = op.num_parents;
    if (--op.dep_left == 0) c->posted.push_back(id);
  }
}

// Start one operation.  Called with c->mu held; may release it around user callbacks.
void execute(rt_rank* c, rt_op id, std::unique_lock<std::mutex>& lk) {
  Op& op = *c->ops[id];
  op.executed++;
  switch (op.type) {
    case T_NOP: complete(c, id); break;
    case T_CALLBACK: {
      rt_callback_fn fn = op.cb;
      void* arg = op.cb_arg;
      lk.unlock();
      if (fn) fn(id, arg);
      lk.lock();
      complete(c, id);
      break;
    }
    case T_COMP: run_comp(c, op); complete(c, id); break;
    case T_SEND: {
      Buffer& b = c->bufs[op.a];
      Message m;
      m.data.assign((uint8_t*)b.data(), (uint8_t*)b.data() + (size_t)b.count * dtype_size(b.dtype));
      {
        std::lock_guard<std::mutex> g(c->world->mail_mu);
        c->world->mail[std::make_tuple(c->id, op.peer, op.tag)].push_back(std::move(m));
      }
      rt_rank* dst = c->world->ranks[op.peer].get();
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
    Op& op = *c->ops[id];
    Message m;
    bool got = false;
    {
      std::lock_guard<std::mutex> g(c->world->mail_mu);
      auto it = c->world->mail.find(std::make_tuple(op.peer, c->id, op.tag));
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
    if (!did) c->work_cv.wait_for(lk, std::chrono::microseconds(200));
  }
}

rt_op new_op(rt_rank* c, OpType t, int options) {
  std::lock_guard<std::mutex> g(c->mu);
  c->ops.emplace_back(new Op());
  Op& op = *c->ops.back();
  op.type = t;
  op.options = options;
  return (rt_op)c->ops.size() - 1;
}

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
int rt_rank_id(rt_rank* c) { return c->id; }
int rt_rank_size(rt_rank* c) { return c->world->n; }

rt_buf rt_buffer_create(rt_rank* c, void* user_ptr, int64_t count, int dtype) {
  std::lock_guard<std::mutex> g(c->mu);
  c->bufs.emplace_back();
  Buffer& b = c->bufs.back();
  b.ptr = user_ptr; b.count = count; b.dtype = dtype;
  if (!user_ptr) b.own.assign((size_t)count * dtype_size(dtype), 0);
  return (rt_buf)c->bufs.size() - 1;
}

int rt_buffer_resize(rt_rank* c, rt_buf id, void* user_ptr, int64_t count) {
  std::lock_guard<std::mutex> g(c->mu);
  Buffer& b = c->bufs[id];
  b.count = count;
  if (user_ptr) { b.ptr = user_ptr; b.own.clear(); }
  else if (!b.ptr) b.own.resize((size_t)count * dtype_size(b.dtype), 0);
  return RT_SUCCESS;
}

int64_t rt_buffer_count(rt_rank* c, rt_buf b) { std::lock_guard<std::mutex> g(c->mu); return c->bufs[b].count; }
void* rt_buffer_data(rt_rank* c, rt_buf b) { std::lock_guard<std::mutex> g(c->mu); return c->bufs[b].data(); }

rt_op rt_op_nop(rt_rank* c, int options) { return new_op(c, T_NOP, options); }

rt_op rt_op_callback(rt_rank* c, rt_callback_fn fn, void* arg, int options) {
  rt_op id = new_op(c, T_CALLBACK, options);
  std::lock_guard<std::mutex> g(c->mu);
  c->ops[id]->cb = fn; c->ops[id]->cb_arg = arg;
  return id;
}

rt_op rt_op_comp(rt_rank* c, rt_buf a, rt_buf b, rt_buf out, int oper, int options) {
  rt_op id = new_op(c, T_COMP, options);
  std::lock_guard<std::mutex> g(c->mu);
  Op& op = *c->ops[id];
  op.a = a; op.b = b; op.out = out; op.oper = oper;
  return id;
}

rt_op rt_op_send(rt_rank* c, rt_buf b, int peer, int tag, int options) {
  rt_op id = new_op(c, T_SEND, options);
  std::lock_guard<std::mutex> g(c->mu);
  Op& op = *c->ops[id];
  op.a = b; op.peer = peer; op.tag = tag;
  return id;
}

rt_op rt_op_recv(rt_rank* c, rt_buf b, int peer, int tag, int options) {
  rt_op id = new_op(c, T_RECV, options);
  std::lock_guard<std::mutex> g(c->mu);
  Op& op = *c->ops[id];
  op.a = b; op.peer = peer; op.tag = tag;
  return id;
}

int rt_operator_create(rt_rank* c, rt_operator_fn fn) {
  std::lock_guard<std::mutex> g(c->mu);
  c->custom_ops.push_back(fn);
  return RT_CUSTOM0 + (int)c->custom_ops.size() - 1;
}

int rt_op_hb(rt_rank* c, rt_op first, rt_op second) {
  std::lock_guard<std::mutex> g(c->mu);
  c->ops[first]->children.push_back(second);
  c->ops[second]->num_parents++;
  return RT_SUCCESS;
}

int rt_op_post(rt_rank* c, rt_op op) {
  { std::lock_guard<std::mutex> g(c->mu); c->posted.push_back(op); }
  c->work_cv.notify_all();
  return RT_SUCCESS;
}

int rt_op_wait(rt_rank* c, rt_op id, double timeout_s) {
  std::unique_lock<std::mutex> lk(c->mu);
  Op& op = *c->ops[id];
  const int64_t want = op.waited.load() + 1;
  auto pred = [&] { return op.completed.load() >= want; };
  if (timeout_s <= 0) c->cv.wait(lk, pred);
  else if (!c->cv.wait_for(lk, std::chrono::duration<double>(timeout_s), pred)) return RT_TIMEOUT;
  op.waited.store(want);
  return RT_SUCCESS;
}

int rt_op_test(rt_rank* c, rt_op id) {
  std::lock_guard<std::mutex> g(c->mu);
  Op& op = *c->ops[id];
  if (op.completed.load() > op.waited.load()) { op.waited.fetch_add(1); return RT_COMPLETED; }
  return RT_SUCCESS;
}

int64_t rt_op_completions(rt_rank* c, rt_op id) { std::lock_guard<std::mutex> g(c->mu); return c->ops[id]->completed.load(); }

rt_sched rt_schedule_create(rt_rank* c) {
  rt_op b = rt_op_nop(c, 0), e = rt_op_nop(c, 0);
  std::lock_guard<std::mutex> g(c->mu);
  c->scheds.emplace_back();
  c->scheds.back().begin = b;
  c->scheds.back().end = e;
  return (rt_sched)c->scheds.size() - 1;
}

int rt_schedule_add_op(rt_rank* c, rt_sched s, rt_op op) {
  std::lock_guard<std::mutex> g(c->mu);
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
    Schedule& sc = c->scheds[s];
    if (sc.finalized) return RT_SUCCESS;
    sc.finalized = true;
    b = sc.begin; e = sc.end;
    for (rt_op id : sc.ops) {
      if (c->ops[id]->num_parents == 0) roots.push_back(id);
      if (c->ops[id]->children.empty()) leaves.push_back(id);
    }
  }
  for (rt_op id : roots) rt_op_hb(c, b, id);
  for (rt_op id : leaves) rt_op_hb(c, id, e);
  if (roots.empty()) rt_op_hb(c, b, e);
  return RT_SUCCESS;
}

rt_op rt_schedule_begin_op(rt_rank* c, rt_sched s) { std::lock_guard<std::mutex> g(c->mu); return c->scheds[s].begin; }
rt_op rt_schedule_end_op(rt_rank* c, rt_sched s) { std::lock_guard<std::mutex> g(c->mu); return c->scheds[s].end; }

int rt_schedule_post(rt_rank* c, rt_sched s) {
  rt_schedule_finalize(c, s);
  return rt_op_post(c, rt_schedule_begin_op(c, s));
}
int rt_schedule_wait(rt_rank* c, rt_sched s, double timeout_s) { return rt_op_wait(c, rt_schedule_end_op(c, s), timeout_s); }
int rt_schedule_test(rt_rank* c, rt_sched s) { return rt_op_test(c, rt_schedule_end_op(c, s)); }

int rt_schedule_print(rt_rank* c, rt_sched s, char* out, int64_t cap) {
  static const char* names[] = {"nop", "callback", "comp", "send", "recv"};
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
    for (rt_op ch : op.children)
      dot += "  \"" + std::to_string(id) + "." + std::to_string(c->id) + "\" -> \"" + std::to_string(ch) + "." +
             std::to_string(c->id) + "\";\n";
  }
  dot += "}\n";
  if ((int64_t)dot.size() + 1 > cap) return RT_ERROR;
  memcpy(out, dot.c_str(), dot.size() + 1);
  return (int)dot.size();
}

// Recursive doubling for any P: ranks beyond the largest power of two first fold into a
// partner, the power-of-two core exchanges in log2 rounds, and the result is sent back.
rt_sched rt_allreduce(rt_rank* c, rt_buf snd, rt_buf rcv, int tag, int oper) {
  const int P = c->world->n, me = c->id;
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
    chain(rt_op_recv(c, tmp, me + p2, tag, 0));
    chain(rt_op_comp(c, tmp, rcv, rcv, oper, 0));
  }
  for (int mask = 1; mask < p2; mask <<= 1) {
    const int peer = me ^ mask;
    rt_buf tmp = rt_buffer_create(c, nullptr, count, dtype);
    rt_op sd = rt_op_send(c, rcv, peer, tag, 0);
    rt_op rv = rt_op_recv(c, tmp, peer, tag, 0);
    rt_op cp = rt_op_comp(c, tmp, rcv, rcv, oper, 0);
    rt_op_hb(c, last, sd);              // send what has been reduced so far ...
    rt_op_hb(c, last, rv);              // ... while the partner's data arrives
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

// Activation from any rank: the activator sends a token to everybody; on every rank the
// `joined` no-op (OR) completes once per activation, whether it was local or remote.
// With an all-to-all fabric there is no need for the reference's forwarding tree.
rt_sched rt_activation(rt_rank* c, int tag, rt_op* activate, rt_op* joined) {
  const int P = c->world->n, me = c->id;
  rt_sched s = rt_schedule_create(c);
  rt_buf token = rt_buffer_create(c, nullptr, 1, RT_INT32);
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
    rt_op rv = rt_op_recv(c, rt_buffer_create(c, nullptr, 1, RT_INT32), r, tag, RT_DEP_OR);
    rt_op_hb(c, rv, join);
    rt_op_hb(c, rv, rv);
    rt_schedule_add_op(c, s, rv);
    rt_op_post(c, rv);
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
