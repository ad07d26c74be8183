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
  float* rsum[kMaxRanks];    // running sums of the results of rounds that lacked somebody
  StepConfig cfg;
  StepPolicy pol;
  uint64_t count;            // elements; multiple of 8
  int32_t slot_bf16;         // publish-slot element type: 1 bf16, 0 fp32
  int32_t grad_in_bf16;
  void* grad_in;             // flat gradient written by backward
  float* w32;                // fused update: fp32 master weights (null: plain mode)
  float* mom;                // momentum buffer
  __nv_bfloat16* w16;        // optional bf16 copy of the weights used by the model
  void* out;                 // plain mode: gradient to apply
  int32_t out_bf16;
  int32_t clear_grad;        // zero grad_in once it has been copied into the publish slot
  const float* hyper;        // HP_* values in device memory
  Plan plan;
  uint32_t bar_pack;         // blocks that have packed their part (the last one runs the control step)
  uint32_t bar_mid;          // blocks that have reduced their part of this rank's share
  uint32_t bar_end;          // blocks that are done with the data phase
  int32_t applied;           // the last step applied something (participant or drain)
  uint64_t two_shot_min;     // smallest element count that takes the two-shot form
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

// Sum the contributors' slots over [lo, hi), scale, round, apply; optionally keep the result in this
// rank's shard buffer (two-shot form) and add it to the running sum (rounds that lack somebody).
template <typename ST, bool kKeepShare>
__device__ void reduce_range(const DevChannel* ch, uint64_t lo, uint64_t hi, uint64_t tid, uint64_t nthreads) {
  const Plan& plan = ch->plan;
  const int n_src = plan.n_src;
  const ST* src[kMaxRanks];
#pragma unroll
  for (int s = 0; s < kMaxRanks; ++s)
    src[s] = s < n_src ? reinterpret_cast<const ST*>(ch->slot[plan.src_rank[s]][plan.src_parity[s]]) : nullptr;
  ST* share = reinterpret_cast<ST*>(ch->red[ch->cfg.rank]);
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
    if (kKeepShare) store8(share, i, acc);
    if (rs != nullptr) {
      load8(rs, i, v);
#pragma unroll
      for (int q = 0; q < 8; ++q) v[q] += acc[q];
      store8(rs, i, v);
    }
    apply8(ch, i, acc, hp.lr, hp.mu, hp.wd, hp.nesterov, hp.gscale);
  }
}

// Two-shot, second half: fetch the share of participant `owner` from its shard buffer and apply it.
template <typename ST>
__device__ void pull_share(const DevChannel* ch, int owner, uint64_t lo, uint64_t hi, uint64_t tid,
                           uint64_t nthreads) {
  const ST* share = reinterpret_cast<const ST*>(ch->red[owner]);
  float* rs = ch->plan.n_push > 0 ? ch->rsum[ch->cfg.rank] : nullptr;
  const Hyper hp(ch->hyper);
  for (uint64_t i = lo + tid * 8; i < hi; i += nthreads * 8) {
    float g[8], v[8];
    load8(share, i, g);
    if (rs != nullptr) {
      load8(rs, i, v);
#pragma unroll
      for (int q = 0; q < 8; ++q) v[q] += g[q];
      store8(rs, i, v);
    }
    apply8(ch, i, g, hp.lr, hp.mu, hp.wd, hp.nesterov, hp.gscale);
  }
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
    reduce_range<ST, false>(ch, 0, ch->count, tid, nth);
    return;
  }
  uint64_t lo, hi;
  share_of(ch->count, plan.part_count, plan.part_index, &lo, &hi);
  reduce_range<ST, true>(ch, lo, hi, tid, nth);
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(&ch->bar_mid, 1u) == nblk - 1) {   // this rank's share is complete: peers may pull it
      ch->bar_mid = 0;
      __threadfence_system();
      gather_signal(ch);
    }
  }
  // the other shares, in an order that differs from rank to rank
  int owners[kMaxRanks], n_own = 0;
  for (int j = 0; j < ch->cfg.world; ++j)
    if (plan.fresh_mask & (1u << j)) owners[n_own++] = j;
  for (int step = 1; step < n_own; ++step) {
    const int idx = (plan.part_index + step) % n_own;
    if (threadIdx.x == 0) *s_flag = gather_wait(ch, owners[idx]) ? 1 : 0;
    __syncthreads();
    const int ok = *s_flag;
    __syncthreads();
    if (!ok) {
      if (threadIdx.x == 0) atomicOr(&ch->view.ctl[ch->cfg.rank]->status, (uint32_t)ST_TIMEOUT_GATHER);
      continue;
    }
    share_of(ch->count, n_own, idx, &lo, &hi);
    pull_share<ST>(ch, owners[idx], lo, hi, tid, nth);
  }
}

__device__ inline void data_phase(DevChannel* ch, uint32_t blk, uint32_t nblk, int* s_flag) {
  const uint64_t tid = (uint64_t)blk * blockDim.x + threadIdx.x, nth = (uint64_t)nblk * blockDim.x;
  const int role = ch->plan.role;
  if (role == ROLE_PARTICIPANT) {
    if (ch->slot_bf16) participant_phase<__nv_bfloat16>(ch, blk, nblk, s_flag);
    else participant_phase<float>(ch, blk, nblk, s_flag);
  } else if (role == ROLE_DRAIN) {
    data_drain(ch, tid, nth);
  } else {
    data_zero_out(ch, tid, nth);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(&ch->bar_end, 1u) == nblk - 1) {
      ch->bar_end = 0;
      __threadfence_system();
      if (role == ROLE_DRAIN && ch->plan.drain_src < 0)
        atomicOr(&ch->view.ctl[ch->cfg.rank]->status, (uint32_t)ST_DESC_LAPPED);
      finish_step<DevEnv>(ch->view, ch->cfg, &ch->plan);
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
  if (threadIdx.x == 0)
    *s_flag = wait_slot_free<DevEnv>(ch->view, ch->cfg, ch->pol, k) ? slot_fate<DevEnv>(me, ch->pol, k) : -1;
  __syncthreads();
  const int fate = *s_flag;
  __syncthreads();
  if (fate < 0) return;
  const bool fold = fate == SLOT_FOLD;
  void* dst = ch->slot[ch->cfg.rank][k % kSlotDepth];
  const float z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (uint64_t i = tid * 8; i < ch->count; i += nthreads * 8) {
    float v[8], u[8];
    if (ch->grad_in_bf16) load8(reinterpret_cast<const __nv_bfloat16*>(ch->grad_in), i, v);
    else load8(reinterpret_cast<const float*>(ch->grad_in), i, v);
    if (fold) {
      if (ch->slot_bf16) load8(reinterpret_cast<const __nv_bfloat16*>(dst), i, u);
      else load8(reinterpret_cast<const float*>(dst), i, u);
#pragma unroll
      for (int q = 0; q < 8; ++q) v[q] += u[q];
    }
    if (ch->slot_bf16) store8(reinterpret_cast<__nv_bfloat16*>(dst), i, v);
    else store8(reinterpret_cast<float*>(dst), i, v);
    if (ch->clear_grad) {
      if (ch->grad_in_bf16) store8(reinterpret_cast<__nv_bfloat16*>(ch->grad_in), i, z);
      else store8(reinterpret_cast<float*>(ch->grad_in), i, z);
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
  ch->applied = (p.role == ROLE_PARTICIPANT || p.role == ROLE_DRAIN) ? 1 : 0;
}

}  // namespace esgd
