// Device-side channel object and the data phase of the partial allreduce.
//
// One DevChannel (in the rank's own device memory) holds the peer-mapped
// pointers of every rank's control block, publish slots and mailbox, the local
// flat buffers the result is applied to, and the Plan the control step produced.
//
// Data phase, participant: for every 8-element vector, sum the contributors'
// slots with 16-byte peer loads (fp32 accumulate), scale by 1/contributors (or
// 1/world), deliver this participant's share of the vector to the mailbox of
// every absent rank, and apply the fused momentum-SGD / weight-decay update to
// the fp32 master weights with a bf16 write-back — or store the averaged
// gradient when a generic optimizer is wrapped.  No NCCL call and no separate
// elementwise kernel (replaces fflib2 gcomp SUM, components/gcomp/
// ffop_gcomp_operator.c:8-58, plus TF ApplyMomentum on the reference path).
//
// Large vectors with two or more participants use a two-shot form of the same
// reduction: each participant sums only ITS share of the vector (a reduce-scatter
// by peer loads), stores the fp32 result into every participant's gather buffer
// (an all-gather by peer stores) and raises a per-round flag there; a second
// kernel waits (bounded) for all shares and applies the update from the local
// gather buffer.  A rank then moves 2(P-1)/P of the vector over NVLink instead of
// P-1 times the vector, with bit-identical results: the same fp32 sums in the
// same order, transported in fp32.
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
  float* mbox[kMaxRanks];
  float* gath[kMaxRanks];    // gather buffers of the two-shot reduction (null: one-shot only)
  StepConfig cfg;
  StepPolicy pol;
  uint64_t count;            // elements; multiple of 8
  int32_t slot_bf16;         // publish-slot element type: 1 bf16, 0 fp32
  int32_t grad_in_bf16;
  const void* grad_in;       // flat gradient written by backward
  float* w32;                // fused update: fp32 master weights (null: plain mode)
  float* mom;                // momentum buffer
  __nv_bfloat16* w16;        // optional bf16 copy of the weights used by the model
  void* out;                 // plain mode: gradient to apply
  int32_t out_bf16;
  int32_t pad0;
  const float* hyper;        // HP_* values in device memory, refreshed by the host
  Plan plan;
  uint32_t blocks_done;
  uint32_t blocks_done2;     // block counter of the gather kernel
  uint64_t two_shot_min;     // smallest element count that takes the two-shot path
  int32_t two_shot_parts;    // fewest participants for which it pays (peer stores are dearer than peer loads)
  int32_t pad2;
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

template <typename ST>
__device__ void data_participant(const DevChannel* ch, uint64_t tid, uint64_t nthreads) {
  const Plan& plan = ch->plan;
  const int n_src = plan.n_src, n_push = plan.n_push;
  const ST* src[kMaxRanks];
#pragma unroll
  for (int s = 0; s < kMaxRanks; ++s)
    src[s] = s < n_src ? reinterpret_cast<const ST*>(ch->slot[plan.src_rank[s]][plan.src_parity[s]]) : nullptr;
  const uint64_t vecs = ch->count / 8;
  const uint64_t per = (vecs + plan.part_count - 1) / plan.part_count;
  const uint64_t lo = per * (uint64_t)plan.part_index * 8;
  const uint64_t hi = min(lo + per * 8, ch->count);
  const float scale = plan.scale;
  const float lr = ch->hyper[HP_LR], mu = ch->hyper[HP_MOMENTUM], wd = ch->hyper[HP_WD];
  const float nesterov = ch->hyper[HP_NESTEROV], gscale = ch->hyper[HP_GRAD_SCALE];
  for (uint64_t i = tid * 8; i < ch->count; i += nthreads * 8) {
    float acc[8], v[8];
    load8(src[0], i, acc);
    for (int s = 1; s < n_src; ++s) {
      load8(src[s], i, v);
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] += v[q];
    }
#pragma unroll
    for (int q = 0; q < 8; ++q) acc[q] *= scale;
    if (n_push > 0 && i >= lo && i < hi) {
      for (int n = 0; n < n_push; ++n) {
        float* mb = ch->mbox[plan.push_rank[n]];
        if (plan.push_accum[n]) {
          load8(mb, i, v);
#pragma unroll
          for (int q = 0; q < 8; ++q) v[q] += acc[q];
          store8(mb, i, v);
        } else {
          store8(mb, i, acc);
        }
      }
    }
    apply8(ch, i, acc, lr, mu, wd, nesterov, gscale);
  }
}

// Two-shot, first half: reduce this participant's share and deliver it to the gather buffer of every
// participant (its own included) and to the mailbox of every absent rank.
template <typename ST>
__device__ void data_reduce_scatter(const DevChannel* ch, uint64_t tid, uint64_t nthreads) {
  const Plan& plan = ch->plan;
  const int n_src = plan.n_src, n_push = plan.n_push;
  const ST* src[kMaxRanks];
#pragma unroll
  for (int s = 0; s < kMaxRanks; ++s)
    src[s] = s < n_src ? reinterpret_cast<const ST*>(ch->slot[plan.src_rank[s]][plan.src_parity[s]]) : nullptr;
  float* dst[kMaxRanks];
  int n_dst = 0;
  for (int j = 0; j < ch->cfg.world; ++j)
    if (plan.fresh_mask & (1u << j)) dst[n_dst++] = ch->gath[j];
  const uint64_t vecs = ch->count / 8;
  const uint64_t per = (vecs + plan.part_count - 1) / plan.part_count;
  const uint64_t lo = per * (uint64_t)plan.part_index * 8;
  const uint64_t hi = min(lo + per * 8, ch->count);
  const float scale = plan.scale;
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
    for (int n = 0; n < n_push; ++n) {
      float* mb = ch->mbox[plan.push_rank[n]];
      if (plan.push_accum[n]) {
        load8(mb, i, v);
#pragma unroll
        for (int q = 0; q < 8; ++q) v[q] += acc[q];
        store8(mb, i, v);
      } else {
        store8(mb, i, acc);
      }
    }
    for (int d = 0; d < n_dst; ++d) store8(dst[d], i, acc);
  }
}

// Two-shot, second half: every share has landed in the local gather buffer; apply it.
__device__ inline void data_apply_gathered(const DevChannel* ch, uint64_t tid, uint64_t nthreads) {
  const float* g_in = ch->gath[ch->cfg.rank];
  const float lr = ch->hyper[HP_LR], mu = ch->hyper[HP_MOMENTUM], wd = ch->hyper[HP_WD];
  const float nesterov = ch->hyper[HP_NESTEROV], gscale = ch->hyper[HP_GRAD_SCALE];
  for (uint64_t i = tid * 8; i < ch->count; i += nthreads * 8) {
    float g[8];
    load8(g_in, i, g);
    apply8(ch, i, g, lr, mu, wd, nesterov, gscale);
  }
}

// Tell every participant that this rank's share of the round is in its gather buffer.
__device__ inline void gather_signal(const DevChannel* ch) {
  const Plan& plan = ch->plan;
  for (int j = 0; j < ch->cfg.world; ++j)
    if (plan.fresh_mask & (1u << j)) DevEnv::st_rel64(&ch->view.ctl[j]->gather_round[ch->cfg.rank], plan.round);
}

// Wait (bounded) until every participant's share of the round has arrived here.
__device__ inline bool gather_wait(const DevChannel* ch) {
  const Plan& plan = ch->plan;
  ChannelCtl* me = ch->view.ctl[ch->cfg.rank];
  const uint64_t t0 = DevEnv::now_ns();
  for (int j = 0; j < ch->cfg.world; ++j) {
    if (!(plan.fresh_mask & (1u << j))) continue;
    while (DevEnv::ld_acq64(&me->gather_round[j]) < plan.round) {
      if (DevEnv::now_ns() - t0 > ch->cfg.timeout_ns) return false;
      DevEnv::pause();
    }
  }
  return true;
}

__device__ inline void data_drain(const DevChannel* ch, uint64_t tid, uint64_t nthreads) {
  const float* mb = ch->mbox[ch->cfg.rank];
  const float lr = ch->hyper[HP_LR], mu = ch->hyper[HP_MOMENTUM], wd = ch->hyper[HP_WD];
  const float nesterov = ch->hyper[HP_NESTEROV], gscale = ch->hyper[HP_GRAD_SCALE];
  for (uint64_t i = tid * 8; i < ch->count; i += nthreads * 8) {
    float g[8];
    load8(mb, i, g);
    apply8(ch, i, g, lr, mu, wd, nesterov, gscale);
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

__device__ inline void data_phase(const DevChannel* ch, uint64_t tid, uint64_t nthreads) {
  const int role = ch->plan.role;
  if (role == ROLE_PARTICIPANT && ch->plan.two_shot) {
    if (ch->slot_bf16) data_reduce_scatter<__nv_bfloat16>(ch, tid, nthreads);
    else data_reduce_scatter<float>(ch, tid, nthreads);
  } else if (role == ROLE_PARTICIPANT) {
    if (ch->slot_bf16) data_participant<__nv_bfloat16>(ch, tid, nthreads);
    else data_participant<float>(ch, tid, nthreads);
  } else if (role == ROLE_DRAIN) {
    data_drain(ch, tid, nthreads);
  } else {
    data_zero_out(ch, tid, nthreads);
  }
}

// Copy (and convert) the flat gradient into publish slot (next epoch % 2).
__device__ inline void pack_phase(const DevChannel* ch, uint64_t tid, uint64_t nthreads) {
  const ChannelCtl* me = ch->view.ctl[ch->cfg.rank];
  const uint64_t k = me->local_step + 1;
  void* dst = ch->slot[ch->cfg.rank][k % kSlotDepth];
  for (uint64_t i = tid * 8; i < ch->count; i += nthreads * 8) {
    float v[8];
    if (ch->grad_in_bf16) load8(reinterpret_cast<const __nv_bfloat16*>(ch->grad_in), i, v);
    else load8(reinterpret_cast<const float*>(ch->grad_in), i, v);
    if (ch->slot_bf16) store8(reinterpret_cast<__nv_bfloat16*>(dst), i, v);
    else store8(reinterpret_cast<float*>(dst), i, v);
  }
}

}  // namespace esgd
