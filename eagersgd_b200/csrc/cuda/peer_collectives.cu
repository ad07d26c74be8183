// Classic collectives over peer-mapped memory: broadcast, gather, all-gather, send / receive, barrier,
// all-reduce (sum) and the ring-neighbour reduction, written as ONE exchange primitive.
//
// They are the GPU-native counterpart of the MPI operators of the reference's Caffe2 backend
// (deep500/frameworks/caffe2/custom_operators/mpi/{allreduce,broadcast,gather,allgather,send,recv,barrier}.cpp)
// and of CommunicationNetwork (deep500/lv3/communication.py:14-119).  No message is ever sent: a source copies
// its data into its own stage buffer and raises a counter in every destination; a destination waits for the
// counter, pulls the bytes with 16-byte peer loads over NVLink, and acknowledges in the source's memory so the
// stage can be reused.  Counters are per ordered pair (source, destination) and per class of traffic (collectives /
// point-to-point), so point-to-point traffic between two ranks does not involve the others, a receive from
// "whichever rank sends first" can never pick up a peer's next collective, and matching within a class is by order.
// A rank has one message in flight at a time (one stage buffer): a send returns as soon as the stage holds the data,
// and the next publish of that rank waits until everybody the previous one was meant for has read it.
//
// Every wait is bounded: when it runs out the kernel sets a status bit, skips its copies and returns.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../protocol/env_device.cuh"
#include "launch_count.cuh"

namespace {

using esgd::DevEnv;
using esgd::count_launch;
constexpr int kMaxRanks = 16;

enum Reduce : int { RED_NONE = 0, RED_SUM_F32 = 1, RED_SUM_BF16 = 2 };
enum CollStatus : uint32_t {
  CS_TIMEOUT_ACK = 1u << 0,     // a destination never acknowledged the previous message
  CS_TIMEOUT_READY = 1u << 1,   // a source never published
};

// Peer-visible words of one rank (start of its arena; the stage follows at `stage_off`).
constexpr int kClasses = 2;      // 0: collectives, 1: point-to-point
struct CollCtl {
  uint64_t ready[kClasses][kMaxRanks];   // ready[c][j]: number of class-c messages rank j has published for this rank
  uint64_t ack[kClasses][kMaxRanks];     // ack[c][j]: number of this rank's class-c messages that rank j has read
};

// This rank's private state and its view of the peers (device memory of this GPU).
struct CollRank {
  int32_t rank, world;
  uint64_t timeout_ns;
  CollCtl* ctl[kMaxRanks];
  uint8_t* stage[kMaxRanks];
  uint64_t sent[kClasses][kMaxRanks];    // messages published to j
  uint64_t recvd[kClasses][kMaxRanks];   // messages consumed from j
  uint32_t ticket[2];          // last-block-done counters of the two phases
  uint32_t status;
  int32_t any_src;             // result of a probe for "whichever rank sends first"
};

struct Op {
  uint32_t dst_mask;           // ranks that will read what this rank publishes
  uint32_t src_mask;           // ranks this rank reads from
  int64_t bytes;               // per message
  const uint8_t* in;           // data to publish / own contribution
  uint8_t* out;                // destination of what is read
  int64_t out_stride;          // bytes between the outputs of source j and j+1 (0: all to `out`)
  int32_t reduce;              // Reduce
  int32_t self_slot;           // >= 0: copy / include the own contribution at that slot
  int32_t cls;                 // class of traffic: 0 collective, 1 point-to-point
  int32_t pad_;
};

__device__ __forceinline__ uint4 ld_peer16(const uint8_t* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// Block-wide bounded wait: thread 0 polls, everybody learns the outcome.
template <class F>
__device__ bool wait_block(CollRank* me, uint32_t bit, F done) {
  __shared__ int ok;
  if (threadIdx.x == 0) {
    uint64_t t0 = DevEnv::now_ns();
    int good = 1;
    while (!done()) {
      if (DevEnv::now_ns() - t0 > me->timeout_ns) { good = 0; atomicOr(&me->status, bit); break; }
      DevEnv::pause();
    }
    ok = good;
  }
  __syncthreads();
  bool r = ok != 0;
  __syncthreads();
  return r;
}

__device__ void copy_bytes(uint8_t* dst, const uint8_t* src, int64_t bytes, int blk, int nblk, bool peer) {
  int64_t vecs = bytes >> 4;
  int64_t stride = int64_t(nblk) * blockDim.x;
  bool aligned = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15) == 0;
  if (aligned) {
    for (int64_t i = int64_t(blk) * blockDim.x + threadIdx.x; i < vecs; i += stride) {
      uint4 v = peer ? ld_peer16(src + (i << 4)) : *reinterpret_cast<const uint4*>(src + (i << 4));
      *reinterpret_cast<uint4*>(dst + (i << 4)) = v;
    }
  } else {
    vecs = 0;
  }
  // volatile: a peer's stage must never be served from a stale L1 line of an earlier message
  for (int64_t i = (vecs << 4) + int64_t(blk) * blockDim.x + threadIdx.x; i < bytes; i += stride)
    dst[i] = *reinterpret_cast<const volatile uint8_t*>(src + i);
}

// Last block of a phase to get here returns true (after every block's writes are visible to it).
__device__ bool last_block(uint32_t* ticket, int nblk) {
  __shared__ int last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    uint32_t t = atomicAdd(ticket, 1u);
    last = (t == uint32_t(nblk - 1));
    if (last) *ticket = 0;
  }
  __syncthreads();
  return last != 0;
}

__device__ void publish_phase(CollRank* me, const Op& op, int blk, int nblk) {
  if (op.dst_mask == 0) return;
  // the stage is single-buffered: everything published before must have been read
  bool ok = wait_block(me, CS_TIMEOUT_ACK, [&] {
    for (int c = 0; c < kClasses; ++c)
      for (int d = 0; d < me->world; ++d)
        if (me->sent[c][d] && DevEnv::ld_acq64(&me->ctl[me->rank]->ack[c][d]) < me->sent[c][d]) return false;
    return true;
  });
  if (ok) copy_bytes(me->stage[me->rank], op.in, op.bytes, blk, nblk, false);
  if (last_block(&me->ticket[0], nblk) && threadIdx.x == 0) {
    if (ok) {
      DevEnv::fence();
      for (int d = 0; d < me->world; ++d)
        if (op.dst_mask >> d & 1) {
          me->sent[op.cls][d] += 1;
          DevEnv::st_rlx64(&me->ctl[d]->ready[op.cls][me->rank], me->sent[op.cls][d]);
        }
    }
  }
}

template <int kReduce>
__device__ void reduce_sources(CollRank* me, const Op& op, int blk, int nblk) {
  // out[i] = sum over ranks in rank order (own contribution read from `in`): the same order on every rank,
  // so every rank gets the same bits
  constexpr int kPer = kReduce == RED_SUM_F32 ? 4 : 8;
  int64_t vecs = op.bytes >> 4;
  for (int64_t i = int64_t(blk) * blockDim.x + threadIdx.x; i < vecs; i += int64_t(nblk) * blockDim.x) {
    float acc[kPer];
#pragma unroll
    for (int e = 0; e < kPer; ++e) acc[e] = 0.f;
    for (int j = 0; j < me->world; ++j) {
      bool own = (j == me->rank && op.self_slot >= 0);
      if (!own && !(op.src_mask >> j & 1)) continue;
      uint4 v = own ? *reinterpret_cast<const uint4*>(op.in + (i << 4)) : ld_peer16(me->stage[j] + (i << 4));
      if (kReduce == RED_SUM_F32) {
        const float* f = reinterpret_cast<const float*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[e] += f[e];
      } else {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float2 f = __bfloat1622float2(h[e]);
          acc[2 * e] += f.x;
          acc[2 * e + 1] += f.y;
        }
      }
    }
    uint4 o;
    if (kReduce == RED_SUM_F32) {
      float* f = reinterpret_cast<float*>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e) f[e] = acc[e];
    } else {
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
    }
    *reinterpret_cast<uint4*>(op.out + (i << 4)) = o;
  }
}

__device__ void pull_phase(CollRank* me, const Op& op, int blk, int nblk) {
  if (op.src_mask == 0 && op.self_slot < 0) return;
  bool ok = wait_block(me, CS_TIMEOUT_READY, [&] {
    for (int j = 0; j < me->world; ++j)
      if ((op.src_mask >> j & 1) && DevEnv::ld_acq64(&me->ctl[me->rank]->ready[op.cls][j]) <= me->recvd[op.cls][j])
        return false;
    return true;
  });
  if (ok) {
    if (op.reduce == RED_SUM_F32) {
      reduce_sources<RED_SUM_F32>(me, op, blk, nblk);
    } else if (op.reduce == RED_SUM_BF16) {
      reduce_sources<RED_SUM_BF16>(me, op, blk, nblk);
    } else {
      for (int j = 0; j < me->world; ++j) {
        if (j == me->rank && op.self_slot >= 0) {
          uint8_t* dst = op.out + int64_t(op.self_slot) * op.out_stride;
          if (dst != op.in) copy_bytes(dst, op.in, op.bytes, blk, nblk, false);
        } else if (op.src_mask >> j & 1) {
          copy_bytes(op.out + (op.out_stride ? int64_t(j) * op.out_stride : 0), me->stage[j], op.bytes, blk, nblk, true);
        }
      }
    }
  }
  if (last_block(&me->ticket[1], nblk) && threadIdx.x == 0 && ok) {
    DevEnv::fence();
    for (int j = 0; j < me->world; ++j)
      if (op.src_mask >> j & 1) {
        me->recvd[op.cls][j] += 1;
        DevEnv::st_rlx64(&me->ctl[j]->ack[op.cls][me->rank], me->recvd[op.cls][j]);
      }
  }
}

__global__ void __launch_bounds__(256) coll_publish_kernel(CollRank* me, Op op) { publish_phase(me, op, blockIdx.x, gridDim.x); }
__global__ void __launch_bounds__(256) coll_pull_kernel(CollRank* me, Op op) { pull_phase(me, op, blockIdx.x, gridDim.x); }

// All ranks of a world on ONE GPU, one block per rank in one launch (the blocks wait on one another, so they
// must be resident together: a cooperative launch guarantees it).  For tests on a single GPU.
__global__ void __launch_bounds__(256) coll_emulated_kernel(CollRank** ranks, const Op* ops) {
  CollRank* me = ranks[blockIdx.x];
  Op op = ops[blockIdx.x];
  publish_phase(me, op, 0, 1);
  pull_phase(me, op, 0, 1);
}

// Which rank of `mask` has a point-to-point message waiting (bounded); -1 when the wait runs out.
__global__ void coll_probe_kernel(CollRank* me, uint32_t mask) {
  uint64_t t0 = DevEnv::now_ns();
  me->any_src = -1;
  for (;;) {
    for (int j = 0; j < me->world; ++j)
      if ((mask >> j & 1) && DevEnv::ld_acq64(&me->ctl[me->rank]->ready[1][j]) > me->recvd[1][j]) {
        me->any_src = j;
        return;
      }
    if (DevEnv::now_ns() - t0 > me->timeout_ns) { atomicOr(&me->status, CS_TIMEOUT_READY); return; }
    DevEnv::pause();
  }
}

int grid_for(int64_t bytes) {
  int64_t g = (bytes / 16 + 256 * 8 - 1) / (256 * 8);
  return int(g < 1 ? 1 : (g > 592 ? 592 : g));
}

}  // namespace

extern "C" {

uint64_t esgd_coll_ctl_bytes(void) { return sizeof(CollCtl); }
uint64_t esgd_coll_rank_bytes(void) { return sizeof(CollRank); }

// Fill the device-resident descriptor of one rank.  `bases[j]` is rank j's arena as mapped on this GPU
// (control words first, the stage `stage_off` bytes in).
int esgd_coll_init(void* rank_desc, int rank, int world, const uint64_t* bases, uint64_t stage_off, double timeout_s,
                   cudaStream_t stream) {
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world) return cudaErrorInvalidValue;
  CollRank h = {};
  h.rank = rank;
  h.world = world;
  h.timeout_ns = uint64_t(timeout_s * 1e9);
  h.any_src = -1;
  for (int j = 0; j < world; ++j) {
    h.ctl[j] = reinterpret_cast<CollCtl*>(bases[j]);
    h.stage[j] = reinterpret_cast<uint8_t*>(bases[j] + stage_off);
  }
  cudaError_t e = cudaMemcpyAsync(rank_desc, &h, sizeof(h), cudaMemcpyHostToDevice, stream);
  if (e != cudaSuccess) return e;
  return cudaStreamSynchronize(stream);
}

// One exchange: publish `in` to the ranks of dst_mask, read from the ranks of src_mask.
int esgd_coll_exchange(void* rank_desc, uint32_t dst_mask, uint32_t src_mask, int64_t bytes, const void* in, void* out,
                       int64_t out_stride, int reduce, int self_slot, int cls, cudaStream_t stream) {
  if (bytes < 0 || (reduce != RED_NONE && (bytes & 15)) || cls < 0 || cls >= kClasses) return cudaErrorInvalidValue;
  if (reduce != RED_NONE && ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15))
    return cudaErrorMisalignedAddress;
  Op op = {dst_mask, src_mask, bytes, static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out), out_stride, reduce,
           self_slot, cls, 0};
  CollRank* me = static_cast<CollRank*>(rank_desc);
  int grid = grid_for(bytes);
  if (dst_mask) {
    coll_publish_kernel<<<grid, 256, 0, stream>>>(me, op);
    count_launch();
  }
  if (src_mask || self_slot >= 0) {
    coll_pull_kernel<<<grid, 256, 0, stream>>>(me, op);
    count_launch();
  }
  return cudaGetLastError();
}

// `world` ranks on one GPU in one cooperative launch; ops[r] / descs[r] belong to rank r (device arrays).
int esgd_coll_exchange_emulated(void* const* descs_dev, const void* ops_dev, int world, cudaStream_t stream) {
  void* args[] = {(void*)&descs_dev, (void*)&ops_dev};
  count_launch();
  return cudaLaunchCooperativeKernel((void*)coll_emulated_kernel, dim3(world), dim3(256), args, 0, stream);
}

uint64_t esgd_coll_op_bytes(void) { return sizeof(Op); }

// Host-side packing of one Op record (for the emulated launch, whose ops live in a device array).
void esgd_coll_pack_op(void* dst_host, uint32_t dst_mask, uint32_t src_mask, int64_t bytes, const void* in, void* out,
                       int64_t out_stride, int reduce, int self_slot, int cls) {
  Op op = {dst_mask, src_mask, bytes, static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out), out_stride, reduce,
           self_slot, cls, 0};
  *static_cast<Op*>(dst_host) = op;
}

int esgd_coll_probe(void* rank_desc, uint32_t mask, cudaStream_t stream) {
  coll_probe_kernel<<<1, 1, 0, stream>>>(static_cast<CollRank*>(rank_desc), mask);
  count_launch();
  return cudaGetLastError();
}

// Reads status (sticky) and the last probe result; synchronises the stream.
int esgd_coll_state(void* rank_desc, uint32_t* status, int32_t* any_src, cudaStream_t stream) {
  CollRank h;
  cudaError_t e = cudaMemcpyAsync(&h, rank_desc, sizeof(h), cudaMemcpyDeviceToHost, stream);
  if (e != cudaSuccess) return e;
  e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return e;
  *status = h.status;
  *any_src = h.any_src;
  return cudaSuccess;
}

}  // extern "C"
