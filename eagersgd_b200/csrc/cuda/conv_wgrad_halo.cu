// Weight gradient of stride-1 convolutions with shared input boxes (sm_100a, tcgen05 / TMEM / TMA).
//
//   dw[k, r, s, c] = sum over output pixels p of dy[p, k] * x[p + (r, s) - pad, c]
//
// The per-tap kernel (conv_tcgen05.cu) loads a dy box and an x box for every (tap, 64-pixel block): the
// activations cross L2 -> SM once per tap.  Here a CTA owns a SET of taps (as many as fit in tensor memory as
// separate accumulators) and, for every block of full output rows, loads ONE dy box and ONE x box (the rows plus
// the filter margin); the taps are shifted views of the x box, exactly as in the forward halo mode: both boxes
// are indexed by the x box's pixel pitch PW = Wo + S - 1, dy's margin columns are zero-filled by TMA, and tap
// (r, s) reads x (r * PW + s) rows further on.  Both operands are MN-major (the pixel is the K index), the
// accumulators stay in tensor memory over the CTA's whole pixel range and are added to dw with 16-byte fp32
// reductions at the end.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include "launch_count.cuh"
#include "sm100_primitives.cuh"
#include "tensormap.cuh"

using namespace sm100;

namespace {

constexpr int WG_THREADS = 192;       // warp 0: TMA, warp 1: MMA issue, warps 2-5: epilogue
constexpr int WG_SMEM = 226 * 1024;

struct WgHaloParams {
  CUtensorMap tmDY, tmX;
  int N, Ho, Wo, Cout, Cin, R, S, pad;
  int BH, PW, h_tiles;                 // output rows per box, pixel pitch, boxes per image
  int ksteps;                          // ceil(BH * PW / 16)
  int abox, xbox;                      // bytes of one 64-channel atom of the dy / x box (multiples of 1024)
  int nstages;
  int sets, taps_per_set, m_tiles, n_tiles, splits, boxes_total, boxes_per_split;
  float* dw;                           // [Cout][R*S][Cin] fp32
  int* error_flag;
};

template <int BN>
__global__ void __launch_bounds__(WG_THREADS, 1) conv_wgrad_halo_kernel(const __grid_constant__ WgHaloParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int NA = 2, NB = BN / 64;                  // 64-channel atoms of the dy (128 rows) and x operands
  const int stage_bytes = NA * p.abox + NB * p.xbox;
  uint8_t* bar_area = smem + p.nstages * stage_bytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(bar_area);
  uint64_t* empty = full + 4;
  uint64_t* done = empty + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // work item of this CTA
  int id = blockIdx.x;
  const int set = id % p.sets; id /= p.sets;
  const int n_idx = id % p.n_tiles; id /= p.n_tiles;
  const int m_idx = id % p.m_tiles; id /= p.m_tiles;
  const int split = id;
  const int tap0 = set * p.taps_per_set;
  const int ntaps = min(p.taps_per_set, p.R * p.S - tap0);
  const int box0 = split * p.boxes_per_split;
  const int box1 = min(box0 + p.boxes_per_split, p.boxes_total);
  const int m0 = m_idx * 128, n0 = n_idx * BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.nstages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(done, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&p.tmDY);
    tma_prefetch_desc(&p.tmX);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  {
    // Rows the boxes do not cover are read as K padding (dy) or by the most shifted views (x): they must hold
    // zeros (dy) or at least finite values (x) for ever, so the stages start out cleared.
    uint4* p4 = reinterpret_cast<uint4*>(smem);
    const int n16 = p.nstages * stage_bytes / 16;
    for (int i = threadIdx.x; i < n16; i += WG_THREADS) p4[i] = make_uint4(0, 0, 0, 0);
    fence_proxy_async();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      const uint32_t tx = (uint32_t)(NA * p.BH * p.PW * 128 + NB * (p.BH + p.R - 1) * p.PW * 128);
      for (int b = box0; b < box1; ++b) {
        if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag)) break;
        const int h0 = (b % p.h_tiles) * p.BH, n = b / p.h_tiles;
        uint8_t* sa = smem + stage * stage_bytes;
        uint8_t* sb = sa + NA * p.abox;
        mbar_expect_tx(&full[stage], tx);
#pragma unroll
        for (int i = 0; i < NA; ++i) tma_load_4d(sa + i * p.abox, &p.tmDY, &full[stage], m0 + 64 * i, 0, h0, n);
#pragma unroll
        for (int i = 0; i < NB; ++i)
          tma_load_4d(sb + i * p.xbox, &p.tmX, &full[stage], n0 + 64 * i, -p.pad, h0 - p.pad, n);
        if (++stage == p.nstages) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(128, BN, 1, 1);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t accumulate = 0;
      bool ok = true;
      constexpr uint64_t kstep = 2048 >> 4;                      // 16 pixel rows
      // The issuing lane has nothing to hide its own instruction latency behind, so the loop below is fully
      // unrolled over (tap, K step) with compile-time offsets; the taps' view offsets are computed once.
      constexpr int MAXT = 512 / BN;                             // accumulators that fit in tensor memory
      uint64_t view_off[MAXT];
#pragma unroll
      for (int tl = 0; tl < MAXT; ++tl) {
        const int tap = tap0 + (tl < ntaps ? tl : 0);
        const int r = tap / p.S, s = tap - r * p.S;
        view_off[tl] = (uint64_t)((r * p.PW + s) * 8);           // (r * PW + s) rows of 128 bytes, in 16-byte units
      }
      const int ksteps = p.ksteps;                               // <= 8: a box has at most 128 pixel rows
      for (int b = box0; ok && b < box1; ++b) {
        if (!mbar_wait(&full[stage], phase, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + stage * stage_bytes);
        const uint64_t a_desc = umma_smem_desc(sa, (uint32_t)p.abox, 1024);
        const uint64_t b_desc0 = umma_smem_desc(sa + NA * p.abox, (uint32_t)p.xbox, 1024);
#pragma unroll
        for (int tl = 0; tl < MAXT; ++tl) {
          if (tl < ntaps) {
            const uint64_t b_desc = b_desc0 + view_off[tl];
            const uint32_t d = tmem_base + (uint32_t)(tl * BN);
            umma_bf16(d, a_desc, b_desc, idesc, accumulate);
#pragma unroll
            for (int ks = 1; ks < 8; ++ks)
              if (ks < ksteps) umma_bf16(d, a_desc + ks * kstep, b_desc + ks * kstep, idesc, 1u);
          }
        }
        accumulate = 1;
        umma_commit(&empty[stage]);
        if (++stage == p.nstages) { stage = 0; phase ^= 1u; }
      }
      umma_commit(done);
    }
  } else {
    // ---- epilogue: once, after the CTA's whole pixel range
    const int q = warp & 3, row = q * 32 + lane;
    const bool have = box1 > box0;
    if (mbar_wait(done, 0u, abort_flag) && have) {
      tc_fence_after();
      const int k = m0 + row;
      for (int tl = 0; tl < ntaps; ++tl) {
        float* out_row = k < p.Cout ? p.dw + ((size_t)k * (p.R * p.S) + tap0 + tl) * p.Cin : nullptr;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(tl * BN + c * 32), v);
          tmem_ld_wait();
          const int col0 = n0 + c * 32;
          if (out_row != nullptr) {
#pragma unroll
            for (int j4 = 0; j4 < 8; ++j4)
              if (col0 + j4 * 4 < p.Cin)
                atomicAdd(reinterpret_cast<float4*>(out_row + col0 + j4 * 4),
                          make_float4(__uint_as_float(v[j4 * 4]), __uint_as_float(v[j4 * 4 + 1]),
                                      __uint_as_float(v[j4 * 4 + 2]), __uint_as_float(v[j4 * 4 + 3])));
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    __nanosleep(1000000);
    if (threadIdx.x == 0 && p.error_flag != nullptr) atomicExch(p.error_flag, 1);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

int wg_sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

// Geometry of a launch (host arithmetic only, shared by the launcher and by the plan query that the CPU tests
// sweep): box sizes, stages, tap sets, pixel splits.  Returns -7 when two stages do not fit.
int wg_plan(WgHaloParams& p, int BN, int N, int H, int W, int Cin, int Cout, int R, int S, int pad, int bh, int sms) {
  p.N = N; p.Cout = Cout; p.Cin = Cin; p.R = R; p.S = S; p.pad = pad;
  p.Ho = H + 2 * pad - R + 1;
  p.Wo = W + 2 * pad - S + 1;
  p.BH = bh;
  p.PW = p.Wo + S - 1;
  p.h_tiles = p.Ho / bh;
  p.ksteps = (bh * p.PW + 15) / 16;
  const int off_max = (R - 1) * p.PW + (S - 1);
  p.abox = (p.ksteps * 16 * 128 + 1023) / 1024 * 1024;
  p.xbox = ((p.ksteps * 16 + off_max) * 128 + 1023) / 1024 * 1024;
  const int stage_bytes = 2 * p.abox + (BN / 64) * p.xbox;
  p.nstages = (WG_SMEM - 1024 - 256) / stage_bytes;
  if (p.nstages > 4) p.nstages = 4;
  if (p.nstages < 2) return -7;
  p.taps_per_set = 512 / BN;
  if (p.taps_per_set > R * S) p.taps_per_set = R * S;
  p.sets = (R * S + p.taps_per_set - 1) / p.taps_per_set;
  p.taps_per_set = (R * S + p.sets - 1) / p.sets;            // balanced sets (9 taps: 5 + 4, or 3 + 3 + 3)
  p.m_tiles = (Cout + 127) / 128;
  p.n_tiles = (Cin + BN - 1) / BN;
  p.boxes_total = p.h_tiles * N;
  const int base = p.sets * p.m_tiles * p.n_tiles;
  int splits = (2 * sms + base - 1) / base;                   // two waves of CTAs
  if (splits > p.boxes_total) splits = p.boxes_total;
  if (splits < 1) splits = 1;
  p.boxes_per_split = (p.boxes_total + splits - 1) / splits;
  p.splits = (p.boxes_total + p.boxes_per_split - 1) / p.boxes_per_split;
  return 0;
}

// Largest number of full output rows whose pitched pixels fit one 128-row K range; 0: outside this kernel's range.
int wg_pick_bh(int H, int W, int Cin, int Cout, int R, int S, int pad) {
  if (Cin % 64 || Cout % 8 || R * S < 2) return 0;
  const int Ho = H + 2 * pad - R + 1, Wo = W + 2 * pad - S + 1;
  const int PW = Wo + S - 1;
  if (Ho < 1 || Wo < 1 || PW > 128) return 0;
  int bh = 0;
  for (int d = 1; d * PW <= 128 && d <= Ho; ++d) if (Ho % d == 0) bh = d;
  if (bh == 0 || bh * Wo < 48) return 0;
  if (bh + R - 1 > 256) return 0;
  return bh;
}

template <int BN>
int launch_wgrad_halo(const void* x, const void* dy, float* dw, int N, int H, int W, int Cin, int Cout, int R, int S,
                      int pad, int bh, int* error_flag, cudaStream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(conv_wgrad_halo_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, WG_SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  WgHaloParams p;
  const int pr = wg_plan(p, BN, N, H, W, Cin, Cout, R, S, pad, bh, wg_sm_count());
  if (pr != 0) return pr;
  p.dw = dw;
  p.error_flag = error_flag;
  {
    uint64_t dims[4] = {(uint64_t)Cout, (uint64_t)p.Wo, (uint64_t)p.Ho, (uint64_t)N};
    uint64_t strides[3] = {(uint64_t)Cout * 2, (uint64_t)p.Wo * Cout * 2, (uint64_t)p.Ho * p.Wo * Cout * 2};
    uint32_t box[4] = {64, (uint32_t)p.PW, (uint32_t)bh, 1};
    int r = esgd::make_tensormap_bf16(&p.tmDY, dy, 4, dims, strides, box, nullptr);
    if (r != 0) return 1000 + r;
  }
  {
    uint64_t dims[4] = {(uint64_t)Cin, (uint64_t)W, (uint64_t)H, (uint64_t)N};
    uint64_t strides[3] = {(uint64_t)Cin * 2, (uint64_t)W * Cin * 2, (uint64_t)H * W * Cin * 2};
    uint32_t box[4] = {64, (uint32_t)p.PW, (uint32_t)(bh + R - 1), 1};
    int r = esgd::make_tensormap_bf16(&p.tmX, x, 4, dims, strides, box, nullptr);
    if (r != 0) return 2000 + r;
  }
  const int grid = p.sets * p.m_tiles * p.n_tiles * p.splits;
  conv_wgrad_halo_kernel<BN><<<grid, WG_THREADS, WG_SMEM, stream>>>(p);
  esgd::count_launch();
  return (int)cudaGetLastError();
}

}  // namespace

extern "C" {

// Returns -100 when the shape is outside this kernel's range (the caller then uses the per-tap kernel).
// dw: fp32 [Cout][R][S][Cin], zeroed by the caller.  Stride 1 only; Cin % 64 == 0, Cout % 8 == 0.
int esgd_conv2d_wgrad_halo(const void* x, const void* dy, float* dw, int N, int H, int W, int Cin, int Cout, int R,
                           int S, int pad, int* error_flag, void* stream) {
  {
    const char* e = getenv("ESGD_CONV_HALO");          // the same switch as the forward halo mode
    if (e != nullptr && e[0] == '0') return -100;
  }
  const int bh = wg_pick_bh(H, W, Cin, Cout, R, S, pad);
  if (bh == 0) return -100;
  cudaStream_t s = (cudaStream_t)stream;
  int rc;
  if (Cin <= 64) rc = launch_wgrad_halo<64>(x, dy, dw, N, H, W, Cin, Cout, R, S, pad, bh, error_flag, s);
  else if (Cin <= 128) rc = launch_wgrad_halo<128>(x, dy, dw, N, H, W, Cin, Cout, R, S, pad, bh, error_flag, s);
  else rc = launch_wgrad_halo<256>(x, dy, dw, N, H, W, Cin, Cout, R, S, pad, bh, error_flag, s);
  return rc == -7 ? -100 : rc;          // boxes too large for two stages: the per-tap kernel takes the shape
}

// Host arithmetic of a launch without launching anything (no device needed).  out[0..11]: applicable (0/1), BH, PW,
// ksteps, abox, xbox, nstages, sets, taps_per_set, splits, boxes_per_split, grid; out[12] = BN, out[13] = shared
// memory requested, out[14] = m_tiles, out[15] = n_tiles.
void esgd_conv2d_wgrad_halo_plan(int N, int H, int W, int Cin, int Cout, int R, int S, int pad, int sms, int* out) {
  for (int i = 0; i < 16; ++i) out[i] = 0;
  const int bh = wg_pick_bh(H, W, Cin, Cout, R, S, pad);
  if (bh == 0) return;
  const int BN = Cin <= 64 ? 64 : (Cin <= 128 ? 128 : 256);
  WgHaloParams p;
  if (wg_plan(p, BN, N, H, W, Cin, Cout, R, S, pad, bh, sms) != 0) return;
  out[0] = 1; out[1] = p.BH; out[2] = p.PW; out[3] = p.ksteps; out[4] = p.abox; out[5] = p.xbox; out[6] = p.nstages;
  out[7] = p.sets; out[8] = p.taps_per_set; out[9] = p.splits; out[10] = p.boxes_per_split;
  out[11] = p.sets * p.m_tiles * p.n_tiles * p.splits; out[12] = BN; out[13] = WG_SMEM; out[14] = p.m_tiles;
  out[15] = p.n_tiles;
}

}  // extern "C"
