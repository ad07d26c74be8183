/* Host operation runtime: persistent, dependency-triggered operations progressed by one thread
 * per rank, and collectives built from them.
 *
 * It provides what the reference's fflib2 core provides on the host (src/ff.h:100-165,
 * src/ffop.c, src/ffschedule.c, src/ffprogress.c): operations (send, recv, compute, no-op,
 * callback) that are created once and posted many times, happens-before edges with AND / OR /
 * FIRST triggering, schedules with begin / end no-ops, buffers that can be resized between
 * posts, reduction operators (built-in and user-defined) over int32 / int64 / float / double,
 * and a recursive-doubling allreduce, an activation broadcast and a bounded-staleness limiter
 * expressed as schedules.  The transport is an in-process mailbox between the ranks of a
 * "world" (ranks are threads of one process); the GPU and multi-process paths of this
 * framework do not use this runtime — they run the one-sided channel protocol instead.
 */
#ifndef ESGD_OPRT_H
#define ESGD_OPRT_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* return codes (ff.h:4-10) */
#define RT_COMPLETED 1
#define RT_SUCCESS 0
#define RT_ERROR (-1)
#define RT_TIMEOUT (-2)

/* datatypes and operators (ff.h:21-41); every operator is implemented */
enum { RT_INT32 = 0, RT_INT64 = 1, RT_FLOAT = 2, RT_DOUBLE = 3, RT_CHAR = 4 };
enum { RT_SUM = 0, RT_PROD = 1, RT_MAX = 2, RT_MIN = 3, RT_IDENTITY = 4, RT_CUSTOM0 = 16 };

/* option bits */
#define RT_DEP_AND 0x0            /* run when all parents have completed (default) */
#define RT_DEP_OR 0x1             /* run when any parent completes */
#define RT_DEP_FIRST 0x2          /* on completion satisfy only ONE dependent, round-robin */
#define RT_NON_PERSISTENT 0x4     /* runs at most once */
/* options of one happens-before edge (rt_op_hb_fallback; ff.h:50-55) */
#define RT_DEP_IGNORE_VERSION 0x10   /* every completion of the first op counts (what rt_op_hb uses) */
#define RT_DEP_NO_AUTOPOST 0x20      /* the edge never posts the second op; it is posted by hand */
#define RT_DEP_CONSTRAINED 0x40      /* passes a completion on only after its constraining edge has (rt_dep_set_parent) */
#define RT_DEP_SKIP_OLD_VERSIONS 0x80 /* accepted and without effect, as in the reference (its code for the bit is commented
                                         out, ffop.c:347-356): a completion that is ahead of the second op is always kept
                                         as a future */
/* more operation options (ff.h:44-57) */
#define RT_SHADOW_TAG 0x100          /* send / recv: a second tag space, so that control tokens never match data */
#define RT_OP_COMPLETE_BEFORE_CANCELLING 0x200   /* rt_op_cancel lets a posted instance finish instead of withdrawing it */
#define RT_COMP_DEST_ATOMIC 0x400    /* compute op: the destination is updated atomically with respect to other
                                        compute ops of the rank.  Always true here (one progress thread per rank
                                        runs them one at a time); the bit is accepted for source compatibility. */
/* options of the partial allreduces (rt_solo_allreduce, rt_rand_allreduce) */
#define RT_PARTIAL_STALE 0x800       /* a rank with nothing new puts its previous contribution into the round again (what the
                                        reference does when the caller leaves its send buffer alone); default: the operator's
                                        neutral element, so that only fresh contributions count */
#define RT_PARTIAL_ACCUMULATE 0x1000 /* a contribution that no round has taken yet is combined with the next one instead of
                                        being replaced by it: nothing a rank posts is lost */
#define RT_PARTIAL_LIVE 0x2000       /* a round reads the send buffer at the moment it begins on the rank, posted or not, and
                                        post copies nothing: exactly the reference's semantics (the caller must not write the
                                        buffer while a round may begin, and clears it itself if a contribution is to count once) */
/* Buffers are always handles into the rank's table (the reference's FFBUFFER_IDX); a handle made around user memory
 * is its FFBUFFER_PTR, and every collective takes handles, so user-managed buffers (FFCOLL_BUFFERS) are the rule. */
#define RT_INPLACE ((int64_t)-2)
#define RT_NONE ((int64_t)-1)

typedef struct rt_world rt_world;
typedef struct rt_rank rt_rank;
typedef int64_t rt_op;        /* handle within a rank */
typedef int64_t rt_buf;
typedef int64_t rt_sched;
typedef int64_t rt_dep;       /* handle of one happens-before edge */
typedef void (*rt_callback_fn)(rt_op op, void* arg);
typedef int (*rt_sched_fn)(rt_rank* c, rt_sched s);
typedef int (*rt_sched_wait_fn)(rt_rank* c, rt_sched s, double timeout_s);
typedef int (*rt_sched_print_fn)(rt_rank* c, rt_sched s, char* out, int64_t cap);
typedef void (*rt_operator_fn)(const void* a, const void* b, void* out, int64_t count, int dtype);

rt_world* rt_world_create(int nranks);
void rt_world_destroy(rt_world* w);
rt_rank* rt_world_rank(rt_world* w, int r);
/* out[2]: message bodies copied straight into a listening receive, and bodies queued in the mailbox */
int rt_world_stats(rt_world* w, int64_t* out);
int rt_rank_id(rt_rank* c);
int rt_rank_size(rt_rank* c);

/* buffers (ffbuffer_{create,resize,get_size,get_data,delete}) */
rt_buf rt_buffer_create(rt_rank* c, void* user_ptr, int64_t count, int dtype); /* user_ptr NULL: runtime-owned */
int rt_buffer_resize(rt_rank* c, rt_buf b, void* user_ptr, int64_t count);
int64_t rt_buffer_count(rt_rank* c, rt_buf b);
void* rt_buffer_data(rt_rank* c, rt_buf b);
int rt_buffer_delete(rt_rank* c, rt_buf b);

/* operations */
rt_op rt_op_nop(rt_rank* c, int options);
rt_op rt_op_callback(rt_rank* c, rt_callback_fn fn, void* arg, int options);
rt_op rt_op_comp(rt_rank* c, rt_buf a, rt_buf b, rt_buf out, int op, int options);  /* out = a (op) b */
rt_op rt_op_send(rt_rank* c, rt_buf b, int peer, int tag, int options);
rt_op rt_op_recv(rt_rank* c, rt_buf b, int peer, int tag, int options);
int rt_operator_create(rt_rank* c, rt_operator_fn fn);   /* returns an operator id >= RT_CUSTOM0 */
int rt_operator_delete(rt_rank* c, int op);              /* the id may be given out again */
int rt_op_tostring(rt_rank* c, rt_op op, char* out, int64_t cap);   /* one line on an operation; returns its length */
int rt_op_hb(rt_rank* c, rt_op first, rt_op second);     /* first happens before second */
/* Versioned edge: the n-th completion of `first` satisfies the n-th run of `second` only.  A completion that
 * finds `second` already past that version goes to `fallback` (RT_NONE: it is dropped); one that is ahead of
 * `second` is remembered and counts when `second` gets there (ffop_hb_fallback, ffop.c:299-401). */
int rt_op_hb_fallback(rt_rank* c, rt_op first, rt_op second, rt_op fallback, int options, rt_dep* dep);
int rt_dep_set_parent(rt_rank* c, rt_dep constrained, rt_dep constraining);
int rt_op_post(rt_rank* c, rt_op op);
int rt_op_cancel(rt_rank* c, rt_op op);                  /* withdraw a posted, not yet completed operation */
int rt_op_free(rt_rank* c, rt_op op);                    /* unlink and release; the handle may be reused */
/* waits for the next completion not yet waited for; timeout_s <= 0 means the default bound of ten minutes */
int rt_op_wait(rt_rank* c, rt_op op, double timeout_s);
int rt_op_test(rt_rank* c, rt_op op);
int64_t rt_op_completions(rt_rank* c, rt_op op);

/* schedules (ffschedule_*) */
rt_sched rt_schedule_create(rt_rank* c);
int rt_schedule_add_op(rt_rank* c, rt_sched s, rt_op op);
int rt_schedule_finalize(rt_rank* c, rt_sched s);        /* link roots to begin and leaves to end */
rt_op rt_schedule_begin_op(rt_rank* c, rt_sched s);
rt_op rt_schedule_end_op(rt_rank* c, rt_sched s);
int rt_schedule_start(rt_rank* c, rt_sched s);           /* arm once before the first post (default: nothing) */
int rt_schedule_post(rt_rank* c, rt_sched s);
int rt_schedule_wait(rt_rank* c, rt_sched s, double timeout_s);
int rt_schedule_test(rt_rank* c, rt_sched s);
int rt_schedule_delete(rt_rank* c, rt_sched s);          /* releases its operations, temporaries and parts */
int rt_schedule_add_part(rt_rank* c, rt_sched s, rt_sched part);   /* composite schedules: deleted together */
int rt_schedule_own_buffer(rt_rank* c, rt_sched s, rt_buf b);      /* buffer released with the schedule */
/* overridable behaviour and a state slot (ffschedule_set_*_fun, ffschedule_{set,get}_state: ff.h:144-159) */
int rt_schedule_set_start_fun(rt_rank* c, rt_sched s, rt_sched_fn f);
int rt_schedule_set_post_fun(rt_rank* c, rt_sched s, rt_sched_fn f);
int rt_schedule_set_wait_fun(rt_rank* c, rt_sched s, rt_sched_wait_fn f);
int rt_schedule_set_test_fun(rt_rank* c, rt_sched s, rt_sched_fn f);
int rt_schedule_set_delete_fun(rt_rank* c, rt_sched s, rt_sched_fn f);
int rt_schedule_set_print_fun(rt_rank* c, rt_sched s, rt_sched_print_fn f);
int rt_schedule_default_post(rt_rank* c, rt_sched s);
int rt_schedule_default_wait(rt_rank* c, rt_sched s, double timeout_s);
int rt_schedule_default_test(rt_rank* c, rt_sched s);
int rt_schedule_default_delete(rt_rank* c, rt_sched s);
int rt_schedule_default_print(rt_rank* c, rt_sched s, char* out, int64_t cap);
int rt_schedule_set_state(rt_rank* c, rt_sched s, void* state);
void* rt_schedule_get_state(rt_rank* c, rt_sched s);
int rt_schedule_print(rt_rank* c, rt_sched s, char* out, int64_t cap);   /* graphviz DOT */
int rt_schedule_print_visjs(rt_rank* c, rt_sched s, char* out, int64_t cap);   /* {"nodes": [...], "edges": [...]} */

/* collectives */
rt_sched rt_allreduce(rt_rank* c, rt_buf snd, rt_buf rcv, int tag, int op);   /* snd == RT_INPLACE: in place */
/* activation: any rank posts `activate`; every rank's `joined` op completes once per activation.  A rank listens from
 * rt_schedule_start (or rt_schedule_post) of the returned schedule on: hang the dependents on `joined` before that */
rt_sched rt_activation(rt_rank* c, int tag, rt_op* activate, rt_op* joined);
/* limiter: posting `start` fires async[0..n-1] in turn, then sync, round-robin */
int rt_limiter(rt_rank* c, int num_async, rt_op* start, rt_op* async_ops, rt_op* sync_op);

/* Partial allreduces (ffsolo_allreduce / ffrand_allreduce, ff.h:161-165): persistent schedules with start / post / wait /
 * test / delete / print like any other.  A rank's j-th post belongs to round j.  In a solo allreduce the first rank to post j
 * activates the round on every rank; in a majority ("rand") allreduce only the rank drawn for round j (the same draw everywhere,
 * from `seed`) does.  A rank takes part in every round with what it has posted since the previous one, or with nothing; its
 * j-th wait returns when round j has completed, which may be long before its own j-th post.  With limiter L >= 0 every
 * (L+1)-th round is synchronous: it begins on a rank only with that rank's own post (L < 0: never).  The contribution is
 * copied inside post, so the send buffer may be reused at once; the result buffer is rewritten by every round
 * (rt_partial_read copies it together with the number of fresh contributors without tearing).  Every rank creates the
 * schedule with the same arguments and posts it the same number of times.  Tags are 16 bits wide (as the reference's);
 * schedules that reuse a tag must be created in the same order on every rank. */
rt_sched rt_solo_allreduce(rt_rank* c, rt_buf snd, rt_buf rcv, int tag, int op, int limiter, int options);
rt_sched rt_rand_allreduce(rt_rank* c, rt_buf snd, rt_buf rcv, int tag, int op, int seed, int limiter, int options);
/* out[9]: posts, rounds completed, rounds this rank activated, posts that found their round already begun, synchronous
 * rounds, fresh contributors of the newest round, its number, contributions replaced before any round took them,
 * 1 if a contribution is waiting for a round */
int rt_partial_info(rt_rank* c, rt_sched s, int64_t* out);
int rt_partial_read(rt_rank* c, rt_sched s, void* out, int64_t* contributors, int64_t* round);
int rt_partial_activator(rt_rank* c, rt_sched s, int64_t round);   /* majority: the rank drawn for a round (-1: synchronous) */

/* native micro-benchmark (threads of this process as ranks); out_us: per-iteration, first creation, all-correct flag */
int rt_bench_allreduce(int ranks, int64_t count, int iters, int fresh, double* out_us);
/* the skewed SGD loop of the reference's ssgd.c / rsgd.c / randomsgd.c (mode 0 / 1 / 2): rank r sleeps r * skew_us before
 * every post; out[0]: mean microseconds per post + wait, out[1]: mean fresh contributors per round, out[2]: all-sane flag */
int rt_bench_partial(int ranks, int64_t count, int iters, int mode, int skew_us, double* out);

#ifdef __cplusplus
}
#endif
#endif
