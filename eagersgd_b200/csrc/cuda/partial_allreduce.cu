// Kernels and C entry points of the NVLink partial allreduce (solo / majority /
// synchronous), sm_100a.  Per step and channel, two launches on the communication stream:
//
//   pack + control: every block waits (bounded) until the publish slot is free and copies / converts
//                   (or folds) its part of the flat gradient into slot (epoch % 2), clearing the flat
//                   gradient behind it; the LAST block to finish then runs esgd::ctl_step in one thread:
//                   publish the epoch into every peer's control block, elect the activator, snapshot
//                   arrivals, broadcast the round descriptor, build the Plan.  No block waits for another.
//   data          : reduce over peer memory (one shot, or reduce-scatter + pull-gather) + fused update,
//                   or collect missed rounds from a participant's running sum; the last block signals
//                   completion (esgd::finish_step)
//
// The kernel boundary is the only grid-wide barrier, so no block ever holds an SM while it waits for
// another block of its own grid, and long waits (a synchronous round, a late initiator) are spent by a
// single thread.  All cross-GPU waits are bounded; when one runs out the kernel records a status bit
// and returns, leaving the context usable.
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdio.h>
#include <string.h>
#include "partial_allreduce.cuh"
#include "launch_count.cuh"

namespace esgd { std::atomic<uint64_t> g_launches{0}; }

using namespace esgd;

namespace {

__device__ inline void control_abort(DevChannel* ch) {
  ChannelCtl* me = ch->view.ctl[ch->cfg.rank];
  me->local_step += 1;
  ch->plan.role = ROLE_ABORT;
  ch->plan.n_src = ch->plan.n_push = 0;
  ch->plan.holds_own_lock = 0;
  ch->plan.two_shot = 0;
  ch->plan.drain_src = -1;
  ch->applied = 0;
}

__device__ inline void control_step(DevChannel* ch, int flush) {
  ChannelCtl* me = ch->view.ctl[ch->cfg.rank];
  ch->t_phase[1] = DevEnv::now_ns();
  if (flush) {
    ctl_flush<DevEnv>(ch->view, ch->cfg, &ch->plan);
  } else if (me->status & ST_TIMEOUT_SLOT) {   // nothing valid was packed
    control_abort(ch);
    return;
  } else {
    ctl_step<DevEnv>(ch->view, ch->cfg, ch->pol, &ch->plan);
  }
  decide_two_shot(ch);
  ch->t_phase[2] = DevEnv::now_ns();
}

__global__ void __launch_bounds__(256, 3) pack_ctl_kernel(DevChannel* ch, int flush) {
  __shared__ int s_flag;
  if (!flush) pack_phase(ch, blockIdx.x, gridDim.x, &s_flag);
  // Device-scope fence per thread, system-scope fence once: the control step fences at system scope before
  // it publishes the epoch, and that fence carries the other blocks' slot writes with it (they are ordered
  // before it through this counter).
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(&ch->bar_pack, 1u) == gridDim.x - 1) {
      ch->bar_pack = 0;
      ch->pack_ticket = 0;
      control_step(ch, flush);
    }
  }
}

__global__ void __launch_bounds__(256, 3) data_kernel(DevChannel* ch) {
  __shared__ int s_flag;
  data_phase(ch, blockIdx.x, gridDim.x, &s_flag);
}

// All ranks of a (small) world inside ONE launch, one block per rank: used to
// exercise the multi-rank protocol on a single GPU, where separate launches
// that wait on one another are not guaranteed to run concurrently.
__global__ void __launch_bounds__(256) emulated_step_kernel(DevChannel** chans, const uint64_t* delay_ns, int flush) {
  DevChannel* ch = chans[blockIdx.x];
  __shared__ int s_flag;
  if (threadIdx.x == 0 && !flush) {
    uint64_t t0 = DevEnv::now_ns();
    while (DevEnv::now_ns() - t0 < delay_ns[blockIdx.x]) __nanosleep(200);
  }
  __syncthreads();
  if (!flush) pack_phase(ch, 0, 1, &s_flag);
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) { ch->pack_ticket = 0; control_step(ch, flush); }
  __threadfence();
  __syncthreads();
  data_phase(ch, 0, 1, &s_flag);
}

__global__ void set_hyper_kernel(float* hyper, float lr, float mu, float wd, float nesterov, float gscale) {
  hyper[HP_LR] = lr; hyper[HP_MOMENTUM] = mu; hyper[HP_WD] = wd; hyper[HP_NESTEROV] = nesterov;
  hyper[HP_GRAD_SCALE] = gscale;
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
  void* red[kMaxRanks];           // shard buffers, slot element type (all null: one-shot reduction only)
  void* rsum[kMaxRanks];          // fp32 running sums of round results
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
  int32_t accumulate;             // fold a gradient that no round picked up into the next publish of its slot
  int32_t adaptive_grace;         // the grace window follows the arrival spread (at most grace_ns)
  int32_t clear_grad;             // zero grad_in behind the copy into the publish slot
  int32_t pad3;
  void* mc_slot0;                 // NVLink multicast addresses of the publish slots and the shard buffer
  void* mc_slot1;                 // (all null: the arenas have no multicast mapping)
  void* mc_red;
  uint64_t mc_min;                // element count from which full rounds go over the switch
};

uint64_t esgd_dev_channel_bytes(void) { return sizeof(DevChannel); }
uint64_t esgd_dev_ctl_bytes(void) { return sizeof(ChannelCtl); }

// Fill the device-side channel object (a DevChannel in device memory at `dch`).
int esgd_channel_configure(void* dch, const esgd_channel_desc* d, void* stream) {
  if (d->count % 8 != 0 || d->world > kMaxRanks || d->world < 1) return -1;
  DevChannel h;
  memset(&h, 0, sizeof(h));
  for (int j = 0; j < d->world; ++j) {
    h.view.ctl[j] = (ChannelCtl*)d->ctl[j];
    h.slot[j][0] = d->slot0[j];
    h.slot[j][1] = d->slot1[j];
    h.red[j] = d->red[j];
    h.rsum[j] = (float*)d->rsum[j];
  }
  h.two_shot_min = d->two_shot_min;
  h.clear_grad = d->clear_grad;
  h.mc_slot[0] = d->mc_slot0; h.mc_slot[1] = d->mc_slot1; h.mc_red = d->mc_red; h.mc_min = d->mc_min;
  h.cfg.rank = d->rank; h.cfg.world = d->world; h.cfg.average_world = d->average; h.cfg.home = d->home;
  h.cfg.timeout_ns = d->timeout_ns; h.cfg.grace_ns = d->grace_ns;
  h.pol.base_mode = d->base_mode; h.pol.include_stale = d->include_stale; h.pol.limiter = d->limiter;
  h.pol.seed = d->seed; h.pol.accumulate = d->accumulate; h.pol.adaptive_grace = d->adaptive_grace;
  h.count = d->count; h.slot_bf16 = d->slot_bf16; h.grad_in_bf16 = d->grad_in_bf16;
  h.grad_in = d->grad_in; h.w32 = (float*)d->w32; h.mom = (float*)d->mom; h.w16 = (__nv_bfloat16*)d->w16;
  h.out = d->out; h.out_bf16 = d->out_bf16; h.hyper = (const float*)d->hyper;
  cudaError_t e = cudaMemcpyAsync(dch, &h, sizeof(h), cudaMemcpyHostToDevice, (cudaStream_t)stream);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaStreamSynchronize((cudaStream_t)stream);
}

// The blocks of the data kernel wait for one another's shares, so all of them must be able to be resident at
// once: the grid never exceeds what the occupancy calculator gives for the current device.
static int resident_cap() {
  static int cap[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  if (cap[dev] == 0) {
    int per_sm = 0, sms = 0;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, data_kernel, 256, 0);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cap[dev] = per_sm > 0 && sms > 0 ? per_sm * sms : 148;
  }
  return cap[dev];
}

static inline int grid_for(uint64_t count, int max_blocks) {
  uint64_t need = (count / 8 + 255) / 256;
  if (need < 1) need = 1;
  const int cap = resident_cap();
  if (max_blocks > cap) max_blocks = cap;
  return (int)(need < (uint64_t)max_blocks ? need : (uint64_t)max_blocks);
}

// One full step of one channel on `stream`: two launches.
int esgd_channel_step(void* dch, uint64_t count, int max_blocks, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  int g = grid_for(count, max_blocks);
  pack_ctl_kernel<<<g, 256, 0, s>>>((DevChannel*)dch, 0);
  data_kernel<<<g, 256, 0, s>>>((DevChannel*)dch);
  count_launch(2);
  return (int)cudaGetLastError();
}

int esgd_channel_flush(void* dch, uint64_t count, int max_blocks, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  int g = grid_for(count, max_blocks);
  pack_ctl_kernel<<<1, 32, 0, s>>>((DevChannel*)dch, 1);
  data_kernel<<<g, 256, 0, s>>>((DevChannel*)dch);
  count_launch(2);
  return (int)cudaGetLastError();
}

// Learning rate, momentum, weight decay, Nesterov flag and gradient scale travel as launch arguments, so
// every step reads the values that were current when it was enqueued, however far the host runs ahead.
int esgd_set_hyper(void* hyper, float lr, float momentum, float wd, int nesterov, float grad_scale, void* stream) {
  set_hyper_kernel<<<1, 1, 0, (cudaStream_t)stream>>>((float*)hyper, lr, momentum, wd, nesterov ? 1.0f : 0.0f, grad_scale);
  count_launch();
  return (int)cudaGetLastError();
}

// Did the newest step apply anything (participant or drain)?  Synchronises with `stream`.
int esgd_channel_applied(const void* dch, int* applied, void* stream) {
  cudaError_t e = cudaMemcpyAsync(applied, (const char*)dch + offsetof(DevChannel, applied), sizeof(int),
                                  cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaStreamSynchronize((cudaStream_t)stream);
}

// Device clock (ns) at the phase boundaries of the newest step: first block packing, control start, control
// end, first data block, own share reduced (two-shot rounds), data end.  Synchronises with `stream`.
int esgd_channel_times(const void* dch, uint64_t* t8, void* stream) {
  cudaError_t e = cudaMemcpyAsync(t8, (const char*)dch + offsetof(DevChannel, t_phase), 8 * sizeof(uint64_t),
                                  cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaStreamSynchronize((cudaStream_t)stream);
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
