// Kernels and C entry points of the NVLink partial allreduce (solo / majority /
// synchronous), sm_100a.  Per step and channel, on the communication stream:
//
//   pack kernel   : wait (bounded) until the publish slot is free, copy/convert
//                   the flat gradient into slot (epoch % 2)
//   control kernel: one thread runs esgd::ctl_step — publish the epoch into every
//                   peer's control block, elect the activator, snapshot arrivals,
//                   broadcast the round descriptor, build the Plan
//   data kernel   : reduce over peer memory + mailbox delivery + fused update;
//                   the last block signals completion (esgd::finish_step)
//   gather kernel : large vectors only (two-shot reduction): the data kernel reduced and
//                   distributed this rank's share; wait for the other shares, apply the
//                   update from the local gather buffer, signal completion
//
// All cross-GPU waits are bounded; when one runs out the kernel records a status
// bit and returns, leaving the context usable.
#include <cuda_runtime.h>
#include <stdio.h>
#include <string.h>
#include "partial_allreduce.cuh"
#include "launch_count.cuh"

namespace esgd { std::atomic<uint64_t> g_launches{0}; }

using namespace esgd;

namespace {

__global__ void pack_kernel(DevChannel* ch) {
  __shared__ int ok;
  ChannelCtl* me = ch->view.ctl[ch->cfg.rank];
  if (threadIdx.x == 0) ok = wait_slot_free<DevEnv>(me, ch->cfg.timeout_ns) ? 1 : 0;
  __syncthreads();
  if (!ok) return;
  pack_phase(ch, (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, (uint64_t)gridDim.x * blockDim.x);
}

// The data phase is split in two when there is enough data and more than one reducer.  Every
// participant of a round takes the same decision (same count, same threshold, same descriptor).
__device__ inline void decide_two_shot(DevChannel* ch) {
  const Plan& p = ch->plan;
  ch->plan.two_shot = (p.role == ROLE_PARTICIPANT && p.part_count >= ch->two_shot_parts && p.part_count >= 2 &&
                       ch->count >= ch->two_shot_min &&
                       ch->gath[ch->cfg.rank] != nullptr) ? 1 : 0;
}

__global__ void ctl_kernel(DevChannel* ch) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  ChannelCtl* me = ch->view.ctl[ch->cfg.rank];
  ch->blocks_done = 0;
  ch->blocks_done2 = 0;
  ch->plan.two_shot = 0;
  if (me->status & ST_TIMEOUT_SLOT) {  // nothing valid was packed
    me->local_step += 1;
    ch->plan.role = ROLE_ABORT;
    ch->plan.n_src = ch->plan.n_push = 0;
    ch->plan.holds_own_lock = 0;
    return;
  }
  ctl_step<DevEnv>(ch->view, ch->cfg, ch->pol, &ch->plan);
  decide_two_shot(ch);
}

__global__ void flush_ctl_kernel(DevChannel* ch) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  ch->blocks_done = 0;
  ctl_flush<DevEnv>(ch->view, ch->cfg, &ch->plan);
}

__global__ void data_kernel(DevChannel* ch) {
  data_phase(ch, (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, (uint64_t)gridDim.x * blockDim.x);
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned old = atomicAdd(&ch->blocks_done, 1u);
    if (old == gridDim.x - 1) {
      __threadfence_system();
      if (ch->plan.two_shot) gather_signal(ch);     // completion is signalled by the gather kernel
      else finish_step<DevEnv>(ch->view, ch->cfg, &ch->plan);
    }
  }
}

__global__ void gather_kernel(DevChannel* ch) {
  if (!ch->plan.two_shot) return;
  __shared__ int ok;
  if (threadIdx.x == 0) ok = gather_wait(ch) ? 1 : 0;
  __syncthreads();
  if (ok) data_apply_gathered(ch, (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, (uint64_t)gridDim.x * blockDim.x);
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned old = atomicAdd(&ch->blocks_done2, 1u);
    if (old == gridDim.x - 1) {
      if (!ok) ch->view.ctl[ch->cfg.rank]->status |= ST_TIMEOUT_GATHER;
      __threadfence_system();
      finish_step<DevEnv>(ch->view, ch->cfg, &ch->plan);
    }
  }
}

// All ranks of a (small) world inside ONE launch, one block per rank: used to
// exercise the multi-rank protocol on a single GPU, where separate launches
// that wait on one another are not guaranteed to run concurrently.
__global__ void emulated_step_kernel(DevChannel** chans, const uint64_t* delay_ns, int flush) {
  DevChannel* ch = chans[blockIdx.x];
  ChannelCtl* me = ch->view.ctl[ch->cfg.rank];
  __shared__ int ok;
  if (threadIdx.x == 0) {
    ok = 1;
    if (!flush) {
      uint64_t t0 = DevEnv::now_ns();
      while (DevEnv::now_ns() - t0 < delay_ns[blockIdx.x]) __nanosleep(200);
      ok = wait_slot_free<DevEnv>(me, ch->cfg.timeout_ns) ? 1 : 0;
    }
  }
  __syncthreads();
  if (!flush && ok) pack_phase(ch, threadIdx.x, blockDim.x);
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (flush) ctl_flush<DevEnv>(ch->view, ch->cfg, &ch->plan);
    else if (ok) { ctl_step<DevEnv>(ch->view, ch->cfg, ch->pol, &ch->plan); decide_two_shot(ch); }
    else { me->local_step += 1; ch->plan.role = ROLE_ABORT; ch->plan.holds_own_lock = 0; ch->plan.two_shot = 0; }
  }
  __threadfence();
  __syncthreads();
  data_phase(ch, threadIdx.x, blockDim.x);
  __threadfence_system();
  __syncthreads();
  if (ch->plan.two_shot) {
    __shared__ int got;
    if (threadIdx.x == 0) {
      gather_signal(ch);
      got = gather_wait(ch) ? 1 : 0;
      if (!got) me->status |= ST_TIMEOUT_GATHER;
    }
    __syncthreads();
    if (got) data_apply_gathered(ch, threadIdx.x, blockDim.x);
    __threadfence_system();
    __syncthreads();
  }
  if (threadIdx.x == 0) finish_step<DevEnv>(ch->view, ch->cfg, &ch->plan);
}

// Stand-alone fused momentum-SGD / weight-decay update over flat buffers (no communication):
// the same per-element update the reduce kernel applies, with an optional per-tensor LARS
// trust ratio folded into the learning rate by the caller.
__global__ void fused_sgd_kernel(const void* grad, int grad_bf16, float* w32, float* mom, __nv_bfloat16* w16,
                                 uint64_t count, float lr, float mu, float wd, float nesterov, float gscale) {
  DevChannel ch;
  ch.w32 = w32; ch.mom = mom; ch.w16 = w16; ch.out = nullptr;
  const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = tid * 8; i < count; i += nth * 8) {
    float g[8];
    if (grad_bf16) load8(reinterpret_cast<const __nv_bfloat16*>(grad), i, g);
    else load8(reinterpret_cast<const float*>(grad), i, g);
    apply8(&ch, i, g, lr, mu, wd, nesterov, gscale);
  }
}

// Bounded busy-wait on the launching stream: the seeded load-imbalance injector
// (the reference sleeps on the host: resnet_run_loop_solo_imagenet_300.py:288-298).
__global__ void spin_kernel(uint64_t ns) {
  uint64_t t0 = DevEnv::now_ns();
  const uint64_t cap = ns < 5000000000ull ? ns : 5000000000ull;
  while (DevEnv::now_ns() - t0 < cap) __nanosleep(1000);
}

}  // namespace

extern "C" {

struct esgd_channel_desc {
  void* ctl[kMaxRanks];
  void* slot0[kMaxRanks];
  void* slot1[kMaxRanks];
  void* mbox[kMaxRanks];
  void* gath[kMaxRanks];          // gather buffers (all null: one-shot reduction only)
  int32_t rank, world, base_mode, include_stale, average, home, slot_bf16, grad_in_bf16;
  int64_t limiter;
  uint64_t seed, timeout_ns, grace_ns, count;
  void* grad_in;
  void* w32;
  void* mom;
  void* w16;
  void* out;
  int32_t out_bf16, pad;
  void* hyper;
  uint64_t two_shot_min;          // element count from which the reduction runs in two shots
  int32_t two_shot_parts, pad3;   // ... in rounds with at least this many participants
};

uint64_t esgd_dev_channel_bytes(void) { return sizeof(DevChannel); }
uint64_t esgd_dev_ctl_bytes(void) { return sizeof(ChannelCtl); }

// Fill the device-side channel object (a DevChannel in device memory at `dch`).
int esgd_channel_configure(void* dch, const esgd_channel_desc* d, void* stream) {
  if (d->count % 8 != 0 || d->world > kMaxRanks) return -1;
  DevChannel h;
  memset(&h, 0, sizeof(h));
  for (int j = 0; j < d->world; ++j) {
    h.view.ctl[j] = (ChannelCtl*)d->ctl[j];
    h.slot[j][0] = d->slot0[j];
    h.slot[j][1] = d->slot1[j];
    h.mbox[j] = (float*)d->mbox[j];
    h.gath[j] = (float*)d->gath[j];
  }
  h.two_shot_min = d->two_shot_min;
  h.two_shot_parts = d->two_shot_parts;
  h.cfg.rank = d->rank; h.cfg.world = d->world; h.cfg.average_world = d->average; h.cfg.home = d->home;
  h.cfg.timeout_ns = d->timeout_ns; h.cfg.grace_ns = d->grace_ns;
  h.pol.base_mode = d->base_mode; h.pol.include_stale = d->include_stale; h.pol.limiter = d->limiter;
  h.pol.seed = d->seed;
  h.count = d->count; h.slot_bf16 = d->slot_bf16; h.grad_in_bf16 = d->grad_in_bf16;
  h.grad_in = d->grad_in; h.w32 = (float*)d->w32; h.mom = (float*)d->mom; h.w16 = (__nv_bfloat16*)d->w16;
  h.out = d->out; h.out_bf16 = d->out_bf16; h.hyper = (const float*)d->hyper;
  cudaError_t e = cudaMemcpyAsync(dch, &h, sizeof(h), cudaMemcpyHostToDevice, (cudaStream_t)stream);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaStreamSynchronize((cudaStream_t)stream);
}

static inline int grid_for(uint64_t count, int max_blocks) {
  uint64_t need = (count / 8 + 255) / 256;
  if (need < 1) need = 1;
  return (int)(need < (uint64_t)max_blocks ? need : (uint64_t)max_blocks);
}

// One full step of one channel on `stream`.  `two_shot`: the channel was configured with gather buffers and
// `count` reaches its two-shot threshold, so the gather kernel must follow (it returns at once in rounds
// that were reduced in one shot).
int esgd_channel_step(void* dch, uint64_t count, int max_blocks, int two_shot, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  int g = grid_for(count, max_blocks);
  pack_kernel<<<g, 256, 0, s>>>((DevChannel*)dch);
  ctl_kernel<<<1, 32, 0, s>>>((DevChannel*)dch);
  data_kernel<<<g, 256, 0, s>>>((DevChannel*)dch);
  if (two_shot) gather_kernel<<<g, 256, 0, s>>>((DevChannel*)dch);
  count_launch(two_shot ? 4 : 3);
  return (int)cudaGetLastError();
}

int esgd_channel_flush(void* dch, uint64_t count, int max_blocks, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  int g = grid_for(count, max_blocks);
  flush_ctl_kernel<<<1, 32, 0, s>>>((DevChannel*)dch);
  data_kernel<<<g, 256, 0, s>>>((DevChannel*)dch);
  count_launch(2);
  return (int)cudaGetLastError();
}

// `chans`: device array of `world` DevChannel pointers, `delay_ns`: device array.
int esgd_emulated_step(void* chans, void* delay_ns, int world, int flush, void* stream) {
  void* args[] = {&chans, &delay_ns, &flush};
  cudaError_t e = cudaLaunchCooperativeKernel((void*)emulated_step_kernel, dim3(world), dim3(256), args, 0,
                                              (cudaStream_t)stream);
  count_launch();
  return (int)e;
}

// count must be a multiple of 8; w16 may be null.
int esgd_fused_sgd(const void* grad, int grad_bf16, float* w32, float* mom, void* w16, uint64_t count, float lr,
                   float momentum, float wd, int nesterov, float grad_scale, void* stream) {
  if (count % 8) return -1;
  int g = grid_for(count, 148 * 8);
  fused_sgd_kernel<<<g, 256, 0, (cudaStream_t)stream>>>(grad, grad_bf16, w32, mom, (__nv_bfloat16*)w16, count, lr,
                                                        momentum, wd, nesterov ? 1.0f : 0.0f, grad_scale);
  count_launch();
  return (int)cudaGetLastError();
}

int esgd_spin(uint64_t ns, void* stream) {
  spin_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(ns);
  count_launch();
  return (int)cudaGetLastError();
}

// ---- symmetric arena: cudaMalloc + CUDA IPC handles exchanged by the caller ----
int esgd_arena_alloc(uint64_t bytes, void** ptr, void* handle64) {
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(*ptr, 0, bytes);
  if (e != cudaSuccess) return (int)e;
  if (handle64 != nullptr) {
    cudaIpcMemHandle_t h;
    e = cudaIpcGetMemHandle(&h, *ptr);
    if (e != cudaSuccess) return (int)e;
    memcpy(handle64, &h, sizeof(h));
  }
  return (int)cudaDeviceSynchronize();
}

int esgd_arena_open(const void* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return (int)cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
}

int esgd_arena_close(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }
int esgd_arena_free(void* ptr) { return (int)cudaFree(ptr); }

int esgd_enable_peer(int peer) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (peer == dev) return 0;
  int can = 0;
  cudaDeviceCanAccessPeer(&can, dev, peer);
  if (!can) return -2;
  cudaError_t e = cudaDeviceEnablePeerAccess(peer, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); return 0; }
  return (int)e;
}

int esgd_memcpy_d2h(void* dst, const void* src, uint64_t bytes, void* stream) {
  cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaStreamSynchronize((cudaStream_t)stream);
}

uint64_t esgd_launch_count(void) { return g_launches.load(); }

const char* esgd_cuda_error_string(int code) { return cudaGetErrorString((cudaError_t)code); }

}  // extern "C"
