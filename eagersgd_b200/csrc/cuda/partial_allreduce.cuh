// Device-side channel object and the data phase of the partial allreduce.
//
// One DevChannel (in the rank's own device memory) holds the peer-mapped
// pointers of every rank's control block, publish slots, shard buffer and
// running sum, the local flat buffers the result is applied to, and the Plan
// the control step produced.
//
// Data phase of a participant.  Small rounds are reduced in ONE shot: for every
// 8-element vector, sum the contributors' slots with 16-byte peer loads (fp32
// accumulate), scale by 1/contributors (or 1/world), round to the slot's
// element type and apply.  Larger rounds take TWO shots, both by peer LOADS:
// each participant reduces only its share of the vector, applies it, and leaves
// the rounded result in its own shard buffer; it then pulls the other
// participants' shares from their shard buffers as they become ready and applies
// those.  A rank moves 2(P-1)/P of the vector over NVLink instead of P-1 times
// the vector, and both forms give the same bits.  "Apply" is the fused
// momentum-SGD / weight-decay update on fp32 master weights with a bf16
// write-back, or a store of the averaged gradient when a generic optimizer is
// wrapped.  No NCCL call and no separate elementwise kernel (replaces fflib2
// gcomp SUM, components/gcomp/ffop_gcomp_operator.c:8-58, plus TF ApplyMomentum
// on the reference path).
//
// When the arenas come from symmetric memory with an NVLink multicast mapping (NVSwitch), a round in which
// every rank is on time takes a third form: each rank reduces its share with peer loads as above and
// broadcasts the rounded result into every rank's shard buffer with multimem.st (one store, replicated by
// the switch); the other shares are then read from LOCAL memory.  The gather half of the exchange costs a
// rank 1/P of the vector outbound instead of (P-1)/P inbound.  (Reducing the share with
// multimem.ld_reduce as well was measured and is slower than peer loads here: 57 vs 87 GB/s of reduced
// output per GPU on eight GPUs at 256 MiB, so the reduction stays on peer loads.)  Rounds that lack
// somebody use the peer-load forms for both halves.
//
// Ranks that miss a round get its result later by a pull, not by a push: in a
// round that lacks somebody every participant adds the round's result to its
// running sum; a late rank, holding its own mailbox lock (so that no round is in
// flight), reads the running sum of one participant of the newest completed
// round, applies the difference to its own running sum as one gradient and
// adopts the peer's sum.  The activator of a round therefore writes nothing to
// the ranks that are not there.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>
#include "../protocol/channel.h"
#include "../protocol/step.h"
#include "../protocol/env_device.cuh"

namespace esgd {

enum HyperIdx { HP_LR = 0, HP_MOMENTUM = 1, HP_WD = 2, HP_NESTEROV = 3, HP_GRAD_SCALE = 4, HP_COUNT = 8 };

struct DevChannel {
  ChannelView view;
  void* slot[kMaxRanks][kSlotDepth];
  void* red[kMaxRanks];      // reduced shares of the running round, slot element type (two-shot form)
  void* mc_slot[kSlotDepth]; // multicast addresses of the publish slots and of the shard buffer (null: none):
  void* mc_red;              // a store to one lands in every rank's copy
  float* rsum[kMaxRanks];    // running sums of the results of rounds that lacked somebody
  StepConfig cfg;
  StepPolicy pol;
  uint64_t count;            // elements; multiple of 8
  int32_t slot_bf16;         // publish-slot element type: 1 bf16, 0 fp32
  int32_t grad_in_bf16;
  void* grad_in;             // flat gradient written by backward (null: the caller fills the publish slot directly)
  float* w32;                // fused update: fp32 master weights (null: plain mode)
  float* mom;                // momentum buffer
  __nv_bfloat16* w16;        // optional bf16 copy of the weights used by the model
  void* out;                 // plain mode: gradient to apply
  int32_t out_bf16;
  int32_t clear_grad;        // zero grad_in once it has been copied into the publish slot
  const float* hyper;        // HP_* values in device memory
  Plan plan;
  uint32_t pack_ticket;      // the first block to take a ticket checks that the publish slot is free
  uint32_t pad1;
  uint64_t pack_word;        // (epoch << 8) | (fate + 2), published by that block for the others
  uint32_t bar_pack;         // blocks that have packed their part (the last one runs the control step)
  uint32_t bar_mid;          // blocks that have reduced their part of this rank's share
  uint32_t bar_end;          // blocks that are done with the data phase
  int32_t applied;           // the last step applied something (participant or drain)
  uint64_t two_shot_min;     // smallest element count that takes the two-shot form
  uint64_t mc_min;           // smallest element count that goes over the switch when it can
  uint64_t t_phase[8];       // clock at: first block packing, control start, control end, first data block,
                             // share reduced (two-shot), data end; for the latency break-down of the benchmarks
};

__device__ __forceinline__ void load8(const __nv_bfloat16* p, uint64_t i, float v[8]) {
  uint4 raw = __ldcg(reinterpret_cast<const uint4*>(p + i));
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    float2 f = __bfloat1622float2(h[q]);
    v[2 * q] = f.x;
    v[2 * q + 1] = f.y;
  }
}
__device__ __forceinline__ void load8(const float* p, uint64_t i, float v[8]) {
  float4 a = __ldcg(reinterpret_cast<const float4*>(p + i));
  float4 b = __ldcg(reinterpret_cast<const float4*>(p + i + 4));
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, uint64_t i, const float v[8]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int q = 0; q < 4; ++q) h[q] = __floats2bfloat162_rn(v[2 * q], v[2 * q + 1]);
  *reinterpret_cast<uint4*>(p + i) = raw;
}
__device__ __forceinline__ void store8(float* p, uint64_t i, const float v[8]) {
  *reinterpret_cast<float4*>(p + i) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + i + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
// The value a round hands out is rounded to the slot's element type, whoever computes it: the one-shot
// form, the owner of a share and the ranks that pull the share all apply the same bits.
__device__ __forceinline__ void round8(const __nv_bfloat16*, float v[8]) {
#pragma unroll
  for (int q = 0; q < 8; ++q) v[q] = __bfloat162float(__float2bfloat16_rn(v[q]));
}
__device__ __forceinline__ void round8(const float*, float[8]) {}

// Apply one 8-vector of the averaged gradient.
__device__ __forceinline__ void apply8(const DevChannel* ch, uint64_t i, float g[8], float lr, float mu, float wd,
                                       float nesterov, float gscale) {
  if (ch->w32 != nullptr) {
    float w[8], m[8];
    load8(ch->w32, i, w);
    load8(ch->mom, i, m);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      float gq = g[q] * gscale + wd * w[q];
      m[q] = mu * m[q] + gq;
      float step = nesterov != 0.0f ? gq + mu * m[q] : m[q];
      w[q] -= lr * step;
    }
    store8(ch->w32, i, w);
    store8(ch->mom, i, m);
    if (ch->w16 != nullptr) store8(ch->w16, i, w);
  } else if (ch->out != nullptr) {
    if (ch->out_bf16) store8(reinterpret_cast<__nv_bfloat16*>(ch->out), i, g);
    else store8(reinterpret_cast<float*>(ch->out), i, g);
  }
}

struct Hyper {
  float lr, mu, wd, nesterov, gscale;
  __device__ __forceinline__ explicit Hyper(const float* h)
      : lr(h[HP_LR]), mu(h[HP_MOMENTUM]), wd(h[HP_WD]), nesterov(h[HP_NESTEROV]), gscale(h[HP_GRAD_SCALE]) {}
};

// The share of the vector that participant `index` of `parts` reduces: [lo, hi) in elements.
__device__ __forceinline__ void share_of(uint64_t count, int parts, int index, uint64_t* lo, uint64_t* hi) {
  const uint64_t vecs = count / 8;
  const uint64_t per = (vecs + parts - 1) / parts;
  const uint64_t a = per * (uint64_t)index * 8;
  *lo = a < count ? a : count;
  *hi = a + per * 8 < count ? a + per * 8 : count;
}

__device__ __forceinline__ void mc_store8(__nv_bfloat16* mc, uint64_t i, const float v[8]);
__device__ __forceinline__ void mc_store8(float* mc, uint64_t i, const float v[8]);

enum ShareMode { SHARE_APPLY = 0, SHARE_KEEP = 1, SHARE_MULTICAST = 2 };

// Sum the contributors' slots over [lo, hi), scale and round.  One-shot form (SHARE_APPLY): apply the result,
// and add it to the running sum in rounds that lack somebody.  Two-shot forms: leave the result in this
// rank's shard buffer (SHARE_KEEP) or store it into every rank's shard buffer through the switch
// (SHARE_MULTICAST); everything is applied from the shard buffers afterwards.
template <typename ST, int kKeepShare>
__device__ void reduce_range(const DevChannel* ch, uint64_t lo, uint64_t hi, uint64_t tid, uint64_t nthreads) {
  const Plan& plan = ch->plan;
  const int n_src = plan.n_src;
  const ST* src[kMaxRanks];
#pragma unroll
  for (int s = 0; s < kMaxRanks; ++s)
    src[s] = s < n_src ? reinterpret_cast<const ST*>(ch->slot[plan.src_rank[s]][plan.src_parity[s]]) : nullptr;
  ST* share = reinterpret_cast<ST*>(kKeepShare == SHARE_MULTICAST ? ch->mc_red : ch->red[ch->cfg.rank]);
  float* rs = plan.n_push > 0 ? ch->rsum[ch->cfg.rank] : nullptr;
  const float scale = plan.scale;
  const Hyper hp(ch->hyper);
  for (uint64_t i = lo + tid * 8; i < hi; i += nthreads * 8) {
    float acc[8], v[8];
    load8(src[0], i, acc);
    for (int s = 1; s < n_src; ++s) {
      load8(src[s], i, v);
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] += v[q];
    }
#pragma unroll
    for (int q = 0; q < 8; ++q) acc[q] *= scale;
    round8(src[0], acc);
    if (kKeepShare == SHARE_KEEP) {
      store8(share, i, acc);
      continue;
    }
    if (kKeepShare == SHARE_MULTICAST) {
      mc_store8(share, i, acc);
      continue;
    }
    if (rs != nullptr) {
      load8(rs, i, v);
#pragma unroll
      for (int q = 0; q < 8; ++q) v[q] += acc[q];
      store8(rs, i, v);
    }
    apply8(ch, i, acc, hp.lr, hp.mu, hp.wd, hp.nesterov, hp.gscale);
  }
}

// Two-shot, second half: fetch one share of the result from the shard buffer of `from_rank` and apply it.
template <typename ST>
__device__ void pull_share(const DevChannel* ch, int from_rank, uint64_t lo, uint64_t hi, uint64_t tid,
                           uint64_t nthreads) {
  const ST* share = reinterpret_cast<const ST*>(ch->red[from_rank]);
  float* rs = ch->plan.n_push > 0 ? ch->rsum[ch->cfg.rank] : nullptr;
  const Hyper hp(ch->hyper);
  constexpr int kUnroll = 4;     // independent loads in flight per thread
  const uint64_t stride = nthreads * 8;
  for (uint64_t base = lo + tid * 8; base < hi; base += stride * kUnroll) {
    float g[kUnroll][8];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint64_t i = base + u * stride;
      if (i < hi) load8(share, i, g[u]);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint64_t i = base + u * stride;
      if (i >= hi) break;
      if (rs != nullptr) {
        float v[8];
        load8(rs, i, v);
#pragma unroll
        for (int q = 0; q < 8; ++q) v[q] += g[u][q];
        store8(rs, i, v);
      }
      apply8(ch, i, g[u], hp.lr, hp.mu, hp.wd, hp.nesterov, hp.gscale);
    }
  }
}

// ---- NVSwitch multicast (multimem) ------------------------------------------------------------------------
__device__ __forceinline__ void mc_store8(__nv_bfloat16* mc, uint64_t i, const float v[8]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int q = 0; q < 4; ++q) h[q] = __floats2bfloat162_rn(v[2 * q], v[2 * q + 1]);
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
               :: "l"(mc + i), "f"(__uint_as_float(raw.x)), "f"(__uint_as_float(raw.y)),
                  "f"(__uint_as_float(raw.z)), "f"(__uint_as_float(raw.w)) : "memory");
}
__device__ __forceinline__ void mc_store8(float* mc, uint64_t i, const float v[8]) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
               :: "l"(mc + i), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]) : "memory");
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
               :: "l"(mc + i + 4), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]) : "memory");
}

// Tell every participant that this rank's share of the round is complete in its shard buffer.
__device__ inline void gather_signal(const DevChannel* ch) {
  const Plan& plan = ch->plan;
  for (int j = 0; j < ch->cfg.world; ++j)
    if (plan.fresh_mask & (1u << j)) DevEnv::st_rel64(&ch->view.ctl[j]->gather_round[ch->cfg.rank], plan.round);
}

// Wait (bounded) until participant `owner` has completed its share of the round.
__device__ inline bool gather_wait(const DevChannel* ch, int owner) {
  ChannelCtl* me = ch->view.ctl[ch->cfg.rank];
  const uint64_t t0 = DevEnv::now_ns();
  while (DevEnv::ld_acq64(&me->gather_round[owner]) < ch->plan.round) {
    if (DevEnv::now_ns() - t0 > ch->cfg.timeout_ns) return false;
    DevEnv::pause();
  }
  return true;
}

// A rank that missed rounds: the difference between a complete running sum and its own is what it missed.
__device__ inline void data_drain(const DevChannel* ch, uint64_t tid, uint64_t nthreads) {
  const int src = ch->plan.drain_src;
  if (src < 0 || src == ch->cfg.rank) return;
  const float* theirs = ch->rsum[src];
  float* mine = ch->rsum[ch->cfg.rank];
  const Hyper hp(ch->hyper);
  for (uint64_t i = tid * 8; i < ch->count; i += nthreads * 8) {
    float a[8], b[8];
    load8(theirs, i, a);
    load8(mine, i, b);
#pragma unroll
    for (int q = 0; q < 8; ++q) b[q] = a[q] - b[q];
    store8(mine, i, a);
    apply8(ch, i, b, hp.lr, hp.mu, hp.wd, hp.nesterov, hp.gscale);
  }
}

__device__ inline void data_zero_out(const DevChannel* ch, uint64_t tid, uint64_t nthreads) {
  if (ch->w32 != nullptr || ch->out == nullptr) return;  // fused mode: nothing to apply
  float z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (uint64_t i = tid * 8; i < ch->count; i += nthreads * 8) {
    if (ch->out_bf16) store8(reinterpret_cast<__nv_bfloat16*>(ch->out), i, z);
    else store8(reinterpret_cast<float*>(ch->out), i, z);
  }
}

// The whole data phase of one rank, run by `nblk` blocks of which this is block `blk`.  `s_flag` is a
// word of shared memory.  The last block to finish signals completion (esgd::finish_step).
template <typename ST>
__device__ void participant_phase(DevChannel* ch, uint32_t blk, uint32_t nblk, int* s_flag) {
  const uint64_t tid = (uint64_t)blk * blockDim.x + threadIdx.x, nth = (uint64_t)nblk * blockDim.x;
  const Plan& plan = ch->plan;
  if (!plan.two_shot) {
    reduce_range<ST, SHARE_APPLY>(ch, 0, ch->count, tid, nth);
    return;
  }
  uint64_t lo, hi;
  share_of(ch->count, plan.part_count, plan.part_index, &lo, &hi);
  const bool over_switch = plan.two_shot == 2;
  if (over_switch) reduce_range<ST, SHARE_MULTICAST>(ch, lo, hi, tid, nth);
  else reduce_range<ST, SHARE_KEEP>(ch, lo, hi, tid, nth);
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(&ch->bar_mid, 1u) == nblk - 1) {   // this rank's share is complete: peers may pull it
      ch->bar_mid = 0;
      ch->t_phase[4] = DevEnv::now_ns();
      __threadfence_system();
      gather_signal(ch);
    }
  }
  // Every share, this rank's own included (its flag is raised by the last of this rank's blocks, so waiting
  // for it is also the barrier between the blocks that wrote the share and the blocks that read it).  All
  // blocks of the grid must be able to run at once: the launcher sizes the grid by the kernel's occupancy.
  int owners[kMaxRanks], n_own = 0;
  for (int j = 0; j < ch->cfg.world; ++j)
    if (plan.fresh_mask & (1u << j)) owners[n_own++] = j;
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int j = 0; j < n_own && ok; ++j) ok = gather_wait(ch, owners[j]) ? 1 : 0;
    *s_flag = ok;
  }
  __syncthreads();
  const int ok = *s_flag;
  __syncthreads();
  if (!ok) {
    if (threadIdx.x == 0) atomicOr(&ch->view.ctl[ch->cfg.rank]->status, (uint32_t)ST_TIMEOUT_GATHER);
    return;
  }
  for (int step = 0; step < n_own; ++step) {       // no barrier between the shares: loads of several are in flight
    const int idx = (plan.part_index + step) % n_own;
    share_of(ch->count, n_own, idx, &lo, &hi);
    // over the switch every owner has stored its share into this rank's own shard buffer
    pull_share<ST>(ch, over_switch ? ch->cfg.rank : owners[idx], lo, hi, tid, nth);
  }
}

__device__ inline void data_phase(DevChannel* ch, uint32_t blk, uint32_t nblk, int* s_flag) {
  const uint64_t tid = (uint64_t)blk * blockDim.x + threadIdx.x, nth = (uint64_t)nblk * blockDim.x;
  const int role = ch->plan.role;
  if (blk == 0 && threadIdx.x == 0) ch->t_phase[3] = DevEnv::now_ns();
  if (role == ROLE_PARTICIPANT) {
    if (ch->slot_bf16) participant_phase<__nv_bfloat16>(ch, blk, nblk, s_flag);
    else participant_phase<float>(ch, blk, nblk, s_flag);
  } else if (role == ROLE_DRAIN) {
    data_drain(ch, tid, nth);
  } else {
    data_zero_out(ch, tid, nth);
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(&ch->bar_end, 1u) == nblk - 1) {
      ch->bar_end = 0;
      // finish_step releases at system scope (an acq_rel atomic for a participant, a fence for a drain)
      if (role == ROLE_DRAIN && ch->plan.drain_src < 0)
        atomicOr(&ch->view.ctl[ch->cfg.rank]->status, (uint32_t)ST_DESC_LAPPED);
      finish_step<DevEnv>(ch->view, ch->cfg, &ch->plan);
      ch->t_phase[5] = DevEnv::now_ns();
    }
  }
}

// Copy (and convert) the flat gradient into publish slot (next epoch % 2), or add it to what the slot
// still holds when the gradient published two epochs ago was never picked up by a round; clear the flat
// gradient for the next backward pass if asked to.  `s_flag` is a word of shared memory.
__device__ inline void pack_phase(DevChannel* ch, uint32_t blk, uint32_t nblk, int* s_flag) {
  const uint64_t tid = (uint64_t)blk * blockDim.x + threadIdx.x, nthreads = (uint64_t)nblk * blockDim.x;
  ChannelCtl* me = ch->view.ctl[ch->cfg.rank];
  const uint64_t k = me->local_step + 1;
  if (threadIdx.x == 0) {
    // One block asks (a sequentially consistent fence and a load from the home rank: costly when
    // hundreds of blocks do it at once); the others read its answer from local memory.  The asking
    // block is the first to get here, so it is running and waits for no other block.
    int fate;
    if (atomicAdd(&ch->pack_ticket, 1u) == 0) {
      ch->t_phase[0] = DevEnv::now_ns();
      fate = wait_slot_free<DevEnv>(ch->view, ch->cfg, ch->pol, k) ? slot_fate<DevEnv>(me, ch->pol, k) : -1;
      __threadfence();
      *reinterpret_cast<volatile uint64_t*>(&ch->pack_word) = (k << 8) | (uint64_t)(fate + 2);
    } else {
      const uint64_t t0 = DevEnv::now_ns();
      uint64_t w;
      while (((w = *reinterpret_cast<volatile uint64_t*>(&ch->pack_word)) >> 8) != k) {
        if (DevEnv::now_ns() - t0 > 2 * ch->cfg.timeout_ns) { w = (k << 8) | 1u; break; }
        __nanosleep(64);
      }
      fate = (int)(w & 0xff) - 2;
    }
    *s_flag = fate;
  }
  __syncthreads();
  const int fate = *s_flag;
  __syncthreads();
  if (fate < 0) return;
  if (ch->grad_in == nullptr) return;      // the caller has written this epoch's gradient into the slot itself
  const bool fold = fate == SLOT_FOLD;
  void* dst = ch->slot[ch->cfg.rank][k % kSlotDepth];
  const float z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  constexpr int kUnroll = 4;     // independent 16-byte loads in flight per thread
  const uint64_t stride = nthreads * 8;
  for (uint64_t base = tid * 8; base < ch->count; base += stride * kUnroll) {
    float v[kUnroll][8];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint64_t i = base + u * stride;
      if (i >= ch->count) break;
      if (ch->grad_in_bf16) load8(reinterpret_cast<const __nv_bfloat16*>(ch->grad_in), i, v[u]);
      else load8(reinterpret_cast<const float*>(ch->grad_in), i, v[u]);
    }
    if (fold) {
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const uint64_t i = base + u * stride;
        if (i >= ch->count) break;
        float w[8];
        if (ch->slot_bf16) load8(reinterpret_cast<const __nv_bfloat16*>(dst), i, w);
        else load8(reinterpret_cast<const float*>(dst), i, w);
#pragma unroll
        for (int q = 0; q < 8; ++q) v[u][q] += w[q];
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint64_t i = base + u * stride;
      if (i >= ch->count) break;
      if (ch->slot_bf16) store8(reinterpret_cast<__nv_bfloat16*>(dst), i, v[u]);
      else store8(reinterpret_cast<float*>(dst), i, v[u]);
      if (ch->clear_grad) {
        if (ch->grad_in_bf16) store8(reinterpret_cast<__nv_bfloat16*>(ch->grad_in), i, z);
        else store8(reinterpret_cast<float*>(ch->grad_in), i, z);
      }
    }
  }
}

// The data phase is split in two when there is enough data and it moves fewer bytes: a participant pulls
// (contributors - 1) vectors in one shot, ((contributors - 1) + (participants - 1)) / participants in two.
// Every participant of a round takes the same decision (same count, same threshold, same descriptor).
__device__ inline void decide_two_shot(DevChannel* ch) {
  const Plan& p = ch->plan;
  ch->plan.two_shot = (p.role == ROLE_PARTICIPANT && p.part_count >= 2 && p.n_src >= 3 &&
                       ch->count >= ch->two_shot_min && ch->red[ch->cfg.rank] != nullptr) ? 1 : 0;
  // Over the switch: everybody takes part, so every rank's shard buffer is a destination of the broadcast
  // (and nobody is absent: the running sums stay untouched).
  // From four ranks up: with two, a rank's share is half the vector and storing it through the switch was
  // measured slower (215 GB/s) than the peer's pulling it (620 GB/s).
  if (p.role == ROLE_PARTICIPANT && ch->mc_red != nullptr && p.part_count == ch->cfg.world && p.part_count >= 4 &&
      ch->count >= ch->mc_min)
    ch->plan.two_shot = 2;
  ch->applied = (p.role == ROLE_PARTICIPANT || p.role == ROLE_DRAIN) ? 1 : 0;
}

}  // namespace esgd
