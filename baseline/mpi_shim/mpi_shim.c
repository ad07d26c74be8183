/* Shared-memory implementation of the MPI subset declared in mpi.h (baseline tooling).
 *
 * Ranks are processes started by shimrun; they map one file (MPISHIM_FILE) that holds
 *   - a single-producer / single-consumer byte ring for every ordered pair of ranks,
 *   - arrival counters for barriers,
 *   - a staging area for Allreduce / Reduce.
 * A message is a 16-byte header (tag, byte count) followed by its payload, streamed through
 * the ring of (source, destination); messages larger than the ring flow through it in pieces
 * while both sides make progress.  Matching is by (source, tag) in posting order; a message
 * that arrives before its receive is posted is parked in a private buffer.  Every entry point
 * takes one process-wide lock, so any thread may call (MPI_THREAD_MULTIPLE); barriers and the
 * staging area do not use the lock and never block the progress of point-to-point traffic.
 */
#define _GNU_SOURCE
#include "mpi.h"
#include <fcntl.h>
#include <pthread.h>
#include <sched.h>
#include <stdatomic.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#define SHIM_MAX_RANKS 16
#define SHIM_RING_BYTES (2u << 20)
#define SHIM_COLL_CHUNK (4u << 20)
#define SHIM_BAR_SLOTS 64

typedef struct {
  _Atomic uint64_t head;          /* bytes written so far (producer) */
  char pad0[56];
  _Atomic uint64_t tail;          /* bytes consumed so far (consumer) */
  char pad1[56];
  char data[SHIM_RING_BYTES];
} shim_ring;

typedef struct {
  _Atomic uint64_t bar_arrivals[SHIM_BAR_SLOTS];
  _Atomic uint32_t attached;
  char pad[60];
} shim_header;

typedef struct { int32_t tag; int32_t pad; uint64_t bytes; } msg_header;

enum { REQ_SEND = 1, REQ_RECV = 2, REQ_BARRIER = 3 };

struct shim_request {
  int type, complete, cancelled, peer, tag;
  char* buf;
  uint64_t bytes;        /* send: message size; recv: capacity, then received size */
  uint64_t offset;       /* send: payload bytes already in the ring */
  int header_done;
  uint64_t bar_seq;
  struct shim_request* next;
};

typedef struct unexpected {
  int src, tag, complete;
  uint64_t bytes;
  char* data;
  struct shim_request* claim;     /* a receive posted while the message was still arriving */
  struct unexpected* next;
} unexpected_t;

typedef struct {                  /* the message currently arriving from one source */
  int active;
  uint64_t remaining, padding;
  char* dst;                      /* where the payload goes (null: discard the excess of a truncated message) */
  uint64_t dst_room;
  struct shim_request* req;
  unexpected_t* unx;
} incoming_t;

static int g_rank = -1, g_size = 0, g_init = 0;
static char* g_base = NULL;
static size_t g_map_bytes = 0;
static shim_header* g_hdr = NULL;
static char* g_coll_in = NULL;     /* [size][SHIM_COLL_CHUNK] */
static char* g_coll_out = NULL;    /* [SHIM_COLL_CHUNK] */
static shim_ring* g_rings = NULL;  /* [src * size + dst] */
static pthread_mutex_t g_lock = PTHREAD_MUTEX_INITIALIZER;
static struct shim_request* g_posted_head = NULL;
static struct shim_request* g_posted_tail = NULL;
static unexpected_t* g_unx_head = NULL;
static unexpected_t* g_unx_tail = NULL;
static struct shim_request* g_sendq_head[SHIM_MAX_RANKS];
static struct shim_request* g_sendq_tail[SHIM_MAX_RANKS];
static incoming_t g_in[SHIM_MAX_RANKS];
static _Atomic uint64_t g_bar_seq = 0;

/* completed requests are recycled late: the library keeps copies of handles it has already tested */
#define SHIM_GRAVE 65536
static struct shim_request* g_grave[SHIM_GRAVE];
static uint64_t g_grave_n = 0;

static size_t dt_size(MPI_Datatype dt) {
  switch (dt) {
    case MPI_CHAR: case MPI_BYTE: return 1;
    case MPI_INT: case MPI_FLOAT: return 4;
    case MPI_DOUBLE: case MPI_LONG_LONG: return 8;
    default: return 0;
  }
}

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

static size_t layout(int size, size_t* coll_in, size_t* coll_out, size_t* rings) {
  size_t off = align_up(sizeof(shim_header), 4096);
  *coll_in = off; off += (size_t)size * SHIM_COLL_CHUNK;
  *coll_out = off; off += SHIM_COLL_CHUNK;
  *rings = off; off += (size_t)size * size * align_up(sizeof(shim_ring), 4096);
  return off;
}

static shim_ring* ring_of(int src, int dst) {
  return (shim_ring*)((char*)g_rings + ((size_t)src * g_size + dst) * align_up(sizeof(shim_ring), 4096));
}

static struct shim_request* new_request(int type) {
  struct shim_request* r = (struct shim_request*)calloc(1, sizeof(*r));
  r->type = type;
  return r;
}

static void bury(struct shim_request* r) {
  uint64_t i = g_grave_n++ % SHIM_GRAVE;
  if (g_grave[i]) free(g_grave[i]);
  g_grave[i] = r;
}

/* ---- ring primitives ------------------------------------------------------------------ */
static uint64_t ring_space(shim_ring* r) {
  return SHIM_RING_BYTES - (atomic_load_explicit(&r->head, memory_order_relaxed) -
                            atomic_load_explicit(&r->tail, memory_order_acquire));
}
static uint64_t ring_avail(shim_ring* r) {
  return atomic_load_explicit(&r->head, memory_order_acquire) - atomic_load_explicit(&r->tail, memory_order_relaxed);
}
static void ring_put(shim_ring* r, const void* src, uint64_t n) {      /* n <= ring_space */
  uint64_t h = atomic_load_explicit(&r->head, memory_order_relaxed), pos = h % SHIM_RING_BYTES;
  uint64_t first = n < SHIM_RING_BYTES - pos ? n : SHIM_RING_BYTES - pos;
  memcpy(r->data + pos, src, first);
  if (n > first) memcpy(r->data, (const char*)src + first, n - first);
  atomic_store_explicit(&r->head, h + n, memory_order_release);
}
static void ring_get(shim_ring* r, void* dst, uint64_t n) {            /* n <= ring_avail; dst may be null */
  uint64_t t = atomic_load_explicit(&r->tail, memory_order_relaxed), pos = t % SHIM_RING_BYTES;
  uint64_t first = n < SHIM_RING_BYTES - pos ? n : SHIM_RING_BYTES - pos;
  if (dst) {
    memcpy(dst, r->data + pos, first);
    if (n > first) memcpy((char*)dst + first, r->data, n - first);
  }
  atomic_store_explicit(&r->tail, t + n, memory_order_release);
}

/* ---- matching and progress (all under g_lock) ------------------------------------------ */
static int matches(int want_src, int want_tag, int src, int tag) {
  return (want_src == MPI_ANY_SOURCE || want_src == src) && (want_tag == MPI_ANY_TAG || want_tag == tag);
}

static void posted_remove(struct shim_request* r) {
  struct shim_request* prev = NULL;
  for (struct shim_request* c = g_posted_head; c; prev = c, c = c->next) {
    if (c != r) continue;
    if (prev) prev->next = c->next; else g_posted_head = c->next;
    if (g_posted_tail == c) g_posted_tail = prev;
    c->next = NULL;
    return;
  }
}

static void unexpected_remove(unexpected_t* u) {
  unexpected_t* prev = NULL;
  for (unexpected_t* c = g_unx_head; c; prev = c, c = c->next) {
    if (c != u) continue;
    if (prev) prev->next = c->next; else g_unx_head = c->next;
    if (g_unx_tail == c) g_unx_tail = prev;
    return;
  }
}

static void deliver_unexpected(unexpected_t* u, struct shim_request* r) {
  uint64_t n = u->bytes < r->bytes ? u->bytes : r->bytes;
  memcpy(r->buf, u->data, n);
  r->bytes = n;
  r->peer = u->src;
  r->tag = u->tag;
  r->complete = 1;
  unexpected_remove(u);
  free(u->data);
  free(u);
}

static void progress_sends(void) {
  for (int dst = 0; dst < g_size; ++dst) {
    shim_ring* ring = ring_of(g_rank, dst);
    while (g_sendq_head[dst]) {
      struct shim_request* s = g_sendq_head[dst];
      if (!s->header_done) {
        if (ring_space(ring) < sizeof(msg_header)) break;
        msg_header h = {s->tag, 0, s->bytes};
        ring_put(ring, &h, sizeof(h));
        s->header_done = 1;
      }
      const uint64_t padded = align_up(s->bytes, 16);
      while (s->offset < padded) {
        uint64_t room = ring_space(ring);
        if (room == 0) break;
        if (s->offset < s->bytes) {
          uint64_t n = s->bytes - s->offset < room ? s->bytes - s->offset : room;
          ring_put(ring, s->buf + s->offset, n);
          s->offset += n;
        } else {
          static const char zeros[16] = {0};
          uint64_t n = padded - s->offset < room ? padded - s->offset : room;
          ring_put(ring, zeros, n);
          s->offset += n;
        }
      }
      if (s->offset < padded) break;
      s->complete = 1;
      g_sendq_head[dst] = s->next;
      if (!g_sendq_head[dst]) g_sendq_tail[dst] = NULL;
      s->next = NULL;
    }
  }
}

static void progress_recvs(void) {
  for (int src = 0; src < g_size; ++src) {
    shim_ring* ring = ring_of(src, g_rank);
    incoming_t* in = &g_in[src];
    for (;;) {
      uint64_t avail = ring_avail(ring);
      if (!in->active) {
        if (avail < sizeof(msg_header)) break;
        msg_header h;
        ring_get(ring, &h, sizeof(h));
        avail -= sizeof(h);
        memset(in, 0, sizeof(*in));
        in->active = 1;
        in->remaining = h.bytes;
        in->padding = align_up(h.bytes, 16) - h.bytes;
        struct shim_request* r = g_posted_head;
        while (r && !matches(r->peer, r->tag, src, h.tag)) r = r->next;
        if (r) {
          posted_remove(r);
          in->req = r;
          in->dst = r->buf;
          in->dst_room = r->bytes;
          r->bytes = h.bytes < r->bytes ? h.bytes : r->bytes;
          r->peer = src;
          r->tag = h.tag;
        } else {
          unexpected_t* u = (unexpected_t*)calloc(1, sizeof(*u));
          u->src = src; u->tag = h.tag; u->bytes = h.bytes;
          u->data = (char*)malloc(h.bytes ? h.bytes : 1);
          if (g_unx_tail) g_unx_tail->next = u; else g_unx_head = u;
          g_unx_tail = u;
          in->unx = u;
          in->dst = u->data;
          in->dst_room = h.bytes;
        }
      }
      if (in->remaining > 0) {
        if (avail == 0) break;
        uint64_t n = in->remaining < avail ? in->remaining : avail;
        uint64_t keep = n < in->dst_room ? n : in->dst_room;
        if (keep > 0) { ring_get(ring, in->dst, keep); in->dst += keep; in->dst_room -= keep; }
        if (n > keep) ring_get(ring, NULL, n - keep);
        in->remaining -= n;
        avail -= n;
      }
      if (in->remaining == 0) {
        if (in->padding > 0) {
          if (avail < in->padding) break;
          ring_get(ring, NULL, in->padding);
          in->padding = 0;
        }
        if (in->req) in->req->complete = 1;
        if (in->unx) {
          in->unx->complete = 1;
          if (in->unx->claim) deliver_unexpected(in->unx, in->unx->claim);
        }
        in->active = 0;
      }
    }
  }
}

static void progress(void) {
  progress_sends();
  progress_recvs();
}

static int barrier_reached(uint64_t seq) {
  return atomic_load_explicit(&g_hdr->bar_arrivals[seq % SHIM_BAR_SLOTS], memory_order_acquire) >=
         (uint64_t)g_size * (seq / SHIM_BAR_SLOTS + 1);
}
static uint64_t barrier_arrive(void) {
  uint64_t seq = atomic_fetch_add(&g_bar_seq, 1);
  atomic_fetch_add_explicit(&g_hdr->bar_arrivals[seq % SHIM_BAR_SLOTS], 1, memory_order_acq_rel);
  return seq;
}

static int request_done(struct shim_request* r) {
  if (r->type == REQ_BARRIER && !r->complete && barrier_reached(r->bar_seq)) r->complete = 1;
  return r->complete;
}

static void fill_status(struct shim_request* r, MPI_Status* st) {
  if (!st) return;
  st->MPI_SOURCE = r->peer;
  st->MPI_TAG = r->tag;
  st->MPI_ERROR = MPI_SUCCESS;
  st->_cancelled = r->cancelled;
  st->_ucount = r->bytes;
}

/* ---- environment ----------------------------------------------------------------------- */
int MPI_Init_thread(int* argc, char*** argv, int required, int* provided) {
  (void)argc; (void)argv; (void)required;
  if (provided) *provided = MPI_THREAD_MULTIPLE;
  if (g_init) return MPI_SUCCESS;
  const char* file = getenv("MPISHIM_FILE");
  const char* rank = getenv("MPISHIM_RANK");
  const char* size = getenv("MPISHIM_SIZE");
  if (!file || !rank || !size) {
    fprintf(stderr, "mpi shim: start the program with shimrun -n <ranks> <program> ...\n");
    return MPI_ERR_OTHER;
  }
  g_rank = atoi(rank);
  g_size = atoi(size);
  if (g_size < 1 || g_size > SHIM_MAX_RANKS || g_rank < 0 || g_rank >= g_size) return MPI_ERR_OTHER;
  size_t ci, co, rg;
  g_map_bytes = layout(g_size, &ci, &co, &rg);
  int fd = open(file, O_RDWR);
  if (fd < 0) { perror("mpi shim: open"); return MPI_ERR_OTHER; }
  g_base = (char*)mmap(NULL, g_map_bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (g_base == MAP_FAILED) { perror("mpi shim: mmap"); return MPI_ERR_OTHER; }
  g_hdr = (shim_header*)g_base;
  g_coll_in = g_base + ci;
  g_coll_out = g_base + co;
  g_rings = (shim_ring*)(g_base + rg);
  g_init = 1;
  atomic_fetch_add(&g_hdr->attached, 1);
  return MPI_Barrier(MPI_COMM_WORLD);
}

int MPI_Init(int* argc, char*** argv) { return MPI_Init_thread(argc, argv, MPI_THREAD_MULTIPLE, NULL); }
int MPI_Initialized(int* flag) { *flag = g_init; return MPI_SUCCESS; }

int MPI_Finalize(void) {
  if (!g_init) return MPI_SUCCESS;
  MPI_Barrier(MPI_COMM_WORLD);
  munmap(g_base, g_map_bytes);
  g_init = 0;
  return MPI_SUCCESS;
}

int MPI_Comm_rank(MPI_Comm comm, int* rank) { (void)comm; *rank = g_rank; return MPI_SUCCESS; }
int MPI_Comm_size(MPI_Comm comm, int* size) { (void)comm; *size = g_size; return MPI_SUCCESS; }

int MPI_Comm_get_attr(MPI_Comm comm, int keyval, void* attribute_val, int* flag) {
  (void)comm;
  static MPI_Aint tag_ub = 0x7fffffff;
  if (keyval == MPI_TAG_UB) { *(MPI_Aint**)attribute_val = &tag_ub; *flag = 1; }
  else *flag = 0;
  return MPI_SUCCESS;
}

double MPI_Wtime(void) {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

/* ---- point to point -------------------------------------------------------------------- */
int MPI_Isend(const void* buf, int count, MPI_Datatype dt, int dest, int tag, MPI_Comm comm, MPI_Request* req) {
  (void)comm;
  if (dest < 0 || dest >= g_size || count < 0) return MPI_ERR_OTHER;
  struct shim_request* r = new_request(REQ_SEND);
  r->buf = (char*)buf;
  r->bytes = (uint64_t)count * dt_size(dt);
  r->peer = dest;
  r->tag = tag;
  pthread_mutex_lock(&g_lock);
  if (g_sendq_tail[dest]) g_sendq_tail[dest]->next = r; else g_sendq_head[dest] = r;
  g_sendq_tail[dest] = r;
  progress();
  pthread_mutex_unlock(&g_lock);
  *req = r;
  return MPI_SUCCESS;
}

int MPI_Irecv(void* buf, int count, MPI_Datatype dt, int source, int tag, MPI_Comm comm, MPI_Request* req) {
  (void)comm;
  if (source >= g_size || count < 0) return MPI_ERR_OTHER;
  struct shim_request* r = new_request(REQ_RECV);
  r->buf = (char*)buf;
  r->bytes = (uint64_t)count * dt_size(dt);
  r->peer = source;
  r->tag = tag;
  pthread_mutex_lock(&g_lock);
  progress();
  unexpected_t* u = g_unx_head;
  while (u && !(u->claim == NULL && matches(source, tag, u->src, u->tag))) u = u->next;
  if (u && u->complete) deliver_unexpected(u, r);
  else if (u) u->claim = r;
  else {
    if (g_posted_tail) g_posted_tail->next = r; else g_posted_head = r;
    g_posted_tail = r;
  }
  pthread_mutex_unlock(&g_lock);
  *req = r;
  return MPI_SUCCESS;
}

int MPI_Test(MPI_Request* req, int* flag, MPI_Status* status) {
  *flag = 0;
  if (*req == MPI_REQUEST_NULL) { *flag = 1; return MPI_SUCCESS; }
  pthread_mutex_lock(&g_lock);
  progress();
  if (request_done(*req)) {
    fill_status(*req, status);
    bury(*req);
    *req = MPI_REQUEST_NULL;
    *flag = 1;
  }
  pthread_mutex_unlock(&g_lock);
  return MPI_SUCCESS;
}

int MPI_Wait(MPI_Request* req, MPI_Status* status) {
  int flag = 0;
  for (;;) {
    MPI_Test(req, &flag, status);
    if (flag) return MPI_SUCCESS;
    sched_yield();
  }
}

int MPI_Request_get_status(MPI_Request req, int* flag, MPI_Status* status) {
  *flag = 1;
  if (req == MPI_REQUEST_NULL) return MPI_SUCCESS;
  pthread_mutex_lock(&g_lock);
  progress();
  *flag = request_done(req);
  if (*flag) fill_status(req, status);
  pthread_mutex_unlock(&g_lock);
  return MPI_SUCCESS;
}

int MPI_Testsome(int incount, MPI_Request reqs[], int* outcount, int indices[], MPI_Status statuses[]) {
  int active = 0, done = 0;
  pthread_mutex_lock(&g_lock);
  progress();
  for (int i = 0; i < incount; ++i) {
    if (reqs[i] == MPI_REQUEST_NULL) continue;
    ++active;
    if (!request_done(reqs[i])) continue;
    if (statuses) fill_status(reqs[i], &statuses[done]);
    bury(reqs[i]);
    reqs[i] = MPI_REQUEST_NULL;
    indices[done++] = i;
  }
  pthread_mutex_unlock(&g_lock);
  *outcount = active == 0 ? MPI_UNDEFINED : done;
  return MPI_SUCCESS;
}

int MPI_Waitsome(int incount, MPI_Request reqs[], int* outcount, int indices[], MPI_Status statuses[]) {
  for (;;) {
    MPI_Testsome(incount, reqs, outcount, indices, statuses);
    if (*outcount == MPI_UNDEFINED || *outcount > 0) return MPI_SUCCESS;
    sched_yield();
  }
}

int MPI_Cancel(MPI_Request* req) {
  struct shim_request* r = *req;
  if (r == MPI_REQUEST_NULL) return MPI_SUCCESS;
  pthread_mutex_lock(&g_lock);
  progress();
  if (!r->complete && r->type == REQ_RECV) {
    int still_posted = 0;
    for (struct shim_request* c = g_posted_head; c; c = c->next) still_posted |= (c == r);
    if (still_posted) {            /* no message has been matched to it yet */
      posted_remove(r);
      r->cancelled = 1;
      r->complete = 1;
      r->bytes = 0;
    }
  } else if (!r->complete && r->type == REQ_SEND && !r->header_done) {
    struct shim_request* prev = NULL;
    for (struct shim_request* c = g_sendq_head[r->peer]; c; prev = c, c = c->next) {
      if (c != r) continue;
      if (prev) prev->next = c->next; else g_sendq_head[r->peer] = c->next;
      if (g_sendq_tail[r->peer] == c) g_sendq_tail[r->peer] = prev;
      r->next = NULL;
      r->cancelled = 1;
      r->complete = 1;
      break;
    }
  }
  pthread_mutex_unlock(&g_lock);
  return MPI_SUCCESS;
}

/* ---- collectives (lock-free: arrival counters and the staging area) ----------------------- */
int MPI_Barrier(MPI_Comm comm) {
  (void)comm;
  uint64_t seq = barrier_arrive();
  unsigned spins = 0;
  while (!barrier_reached(seq)) {
    if (++spins % 64 == 0) sched_yield();
  }
  return MPI_SUCCESS;
}

int MPI_Ibarrier(MPI_Comm comm, MPI_Request* req) {
  (void)comm;
  struct shim_request* r = new_request(REQ_BARRIER);
  r->bar_seq = barrier_arrive();
  *req = r;
  return MPI_SUCCESS;
}

#define REDUCE_LOOP(T)                                                              \
  {                                                                                 \
    T* o = (T*)(g_coll_out) + lo;                                                   \
    for (size_t e = 0; e < n; ++e) o[e] = ((const T*)g_coll_in)[lo + e];            \
    for (int r = 1; r < g_size; ++r) {                                              \
      const T* in = (const T*)(g_coll_in + (size_t)r * SHIM_COLL_CHUNK) + lo;       \
      if (op == MPI_SUM) for (size_t e = 0; e < n; ++e) o[e] += in[e];              \
      else if (op == MPI_MAX) for (size_t e = 0; e < n; ++e) o[e] = o[e] > in[e] ? o[e] : in[e]; \
      else for (size_t e = 0; e < n; ++e) o[e] = o[e] < in[e] ? o[e] : in[e];       \
    }                                                                               \
  }

/* Chunk by chunk: every rank stages its part, reduces one slice of the chunk over all ranks into the
 * shared result, and copies the whole result out. */
static int allreduce_impl(const void* sendbuf, void* recvbuf, int count, MPI_Datatype dt, MPI_Op op, int root) {
  const size_t es = dt_size(dt);
  if (es == 0 || count < 0) return MPI_ERR_OTHER;
  const size_t per_chunk = SHIM_COLL_CHUNK / es;
  for (size_t done = 0; done < (size_t)count || (count == 0 && done == 0); done += per_chunk) {
    const size_t elems = (size_t)count - done < per_chunk ? (size_t)count - done : per_chunk;
    memcpy(g_coll_in + (size_t)g_rank * SHIM_COLL_CHUNK, (const char*)sendbuf + done * es, elems * es);
    MPI_Barrier(MPI_COMM_WORLD);
    const size_t slice = (elems + g_size - 1) / g_size;
    const size_t lo = slice * g_rank < elems ? slice * g_rank : elems;
    const size_t n = lo + slice < elems ? slice : elems - lo;
    switch (dt) {
      case MPI_INT: REDUCE_LOOP(int32_t) break;
      case MPI_FLOAT: REDUCE_LOOP(float) break;
      case MPI_DOUBLE: REDUCE_LOOP(double) break;
      case MPI_LONG_LONG: REDUCE_LOOP(long long) break;
      default: REDUCE_LOOP(signed char) break;
    }
    MPI_Barrier(MPI_COMM_WORLD);
    if (root < 0 || root == g_rank) memcpy((char*)recvbuf + done * es, g_coll_out, elems * es);
    MPI_Barrier(MPI_COMM_WORLD);
    if (count == 0) break;
  }
  return MPI_SUCCESS;
}

int MPI_Allreduce(const void* sendbuf, void* recvbuf, int count, MPI_Datatype dt, MPI_Op op, MPI_Comm comm) {
  (void)comm;
  return allreduce_impl(sendbuf, recvbuf, count, dt, op, -1);
}

int MPI_Reduce(const void* sendbuf, void* recvbuf, int count, MPI_Datatype dt, MPI_Op op, int root, MPI_Comm comm) {
  (void)comm;
  return allreduce_impl(sendbuf, recvbuf, count, dt, op, root);
}
