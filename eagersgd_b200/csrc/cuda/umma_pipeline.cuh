// Persistent warp-specialised tcgen05 pipeline shared by the GEMM and the
// implicit-GEMM convolution kernels.
//
//   warp 0     : TMA producer — the Problem policy issues the loads of one k-block
//   warp 1     : tcgen05.mma issuer (one thread); two TMEM accumulators so the
//                epilogue of tile i overlaps the main loop of tile i+1
//   warps 2..9 : epilogue — tcgen05.ld, bias / ReLU, bf16 tile staged in shared
//                memory in the 128-byte-swizzled layout and written with a TMA
//                store (coalesced, clipped at the tensor edge); per-channel sum and
//                sum of squares of the stored tile are taken from shared memory and
//                flushed with one atomic per column per CTA (batch-norm statistics)
//
// B-resident mode: when a CTA keeps one column range for all of its tiles and the whole K
// extent of B for that range fits beside four A stages, B is loaded ONCE and stays in shared
// memory; the ring then carries A only (up to eight stages).  Short-K, long-M problems (1x1
// convolutions over early feature maps, 3x3 over 64 channels) otherwise re-read B from L2 for
// every tile, which is a quarter of their L2 traffic.
//
// A tile is 128 rows x BN columns; a k-block is 64 bf16 (one 128-byte swizzle row).
// Every mbarrier wait is bounded; on expiry the CTA raises an error flag, lets the
// copies in flight land, frees its tensor memory and returns.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdlib.h>
#include "sm100_primitives.cuh"

namespace umma {

using namespace sm100;

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int A_STAGE_BYTES = BM * BK * 2;   // 16 KB
constexpr int PANEL_BYTES = BM * 64 * 2;     // one 128 x 64 bf16 output panel
constexpr int NUM_EPI_THREADS = 256;         // eight epilogue warps
constexpr int NUM_THREADS = 64 + NUM_EPI_THREADS;
constexpr int NUM_PANEL_BUFS = 4;            // output staging ring (the one-barrier hand-over below needs four)

enum OutMode { OUT_BF16 = 0, OUT_F32 = 1, OUT_F32_ATOMIC = 2 };

struct Epilogue {
  int out_mode;
  int relu;
  int n_total;             // number of valid output columns (channels)
  const float* bias;       // per column, may be null
  float* col_sum;          // optional per-column statistics of the stored bf16 values
  float* col_sqsum;
  int* error_flag;
  uint32_t tx_bytes;       // bytes the loads of one k-block deliver (0: full A and B stage tiles)
  uint32_t tx_bytes_a;     // bytes of the A loads alone (B-resident mode; 0: a full A stage tile)
  const void* residual;    // optional bf16 tensor added to the product before rounding (same shape as the output)
  int ldr;                 // its row stride in elements
};

template <int BN>
struct Cfg {
  static constexpr int B_STAGE_BYTES = BN * BK * 2;
  static constexpr int STAGES = BN == 256 ? 3 : (BN == 128 ? 5 : 6);
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int MAX_STAGES = 8;                 // A-only ring of the B-resident mode
  static constexpr int STAGE_AREA = 161 * 1024;        // operand stages (ring, or A ring + resident B)
  static constexpr int SMEM_BYTES = 1024 + STAGE_AREA + NUM_PANEL_BUFS * PANEL_BYTES + 512;
  static_assert(STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) <= STAGE_AREA, "ring does not fit");
  static_assert(SMEM_BYTES <= 227 * 1024, "over the shared-memory limit of a CTA");
  // k-blocks of B that may stay resident: four A stages must still fit
  static constexpr int MAX_RES_KB = (STAGE_AREA - 4 * A_STAGE_BYTES) / B_STAGE_BYTES;
};

// Halo mode (policies with kHalo): a convolution tile loads, per 64-channel block, ONE box of input pixels
// that covers all filter taps (the output rows of the tile plus the filter's margin, full width), and the
// taps are shifted VIEWS of that box: the A descriptor of tap (r, s) starts (r * PW + s) rows of 128 bytes
// into it (the swizzle is a function of the absolute shared-memory address, so a view that starts in the
// middle of a 1024-byte pattern reads what TMA wrote there; the descriptor's base-offset field stays 0 --
// putting the row phase there gives wrong results, as a test run showed).  GEMM rows then run over the box's pixel pitch PW (the margin columns compute values that are
// never stored), and the input crosses L2 -> SM once instead of once per tap.  The box ring has its own
// barriers; the operand ring carries the filter tiles only (or nothing, when they are resident).
constexpr int HALO_BYTES = 32 * 1024;        // one input box (incl. the rows a shifted view may touch past it)
constexpr int MAX_HALOS = 3;

// ESGD_GEMM_B_RESIDENT=0 in the environment turns the B-resident mode off (for A/B timing).
inline bool resident_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("ESGD_GEMM_B_RESIDENT");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

// 32 accumulator columns of one row -> bf16 -> four 16-byte chunks of the swizzled staging panel.
// kPlain leaves out the bias / ReLU code altogether: as run-time options they would be predicated
// instructions that still take issue slots in the common case that uses neither.
template <bool kPlain>
__device__ __forceinline__ void pack_row_to_panel(const uint32_t* r, uint8_t* panel, int row, int half, int col0,
                                                  const Epilogue& ep, bool has_residual) {
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[g * 8 + j]);
    const int chunk = half * 4 + g;          // 16-byte chunk within the 128-byte row
    uint4* slot = reinterpret_cast<uint4*>(panel + row * 128 + ((chunk ^ (row & 7)) << 4));
    if (!kPlain) {
      if (has_residual) {     // the residual panel was brought into this very buffer by TMA; add in place
        const uint4 rv = *slot;
        const uint32_t* rw = reinterpret_cast<const uint32_t*>(&rv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          v[2 * j] += __uint_as_float(rw[j] << 16);
          v[2 * j + 1] += __uint_as_float(rw[j] & 0xffff0000u);
        }
      }
      if (ep.bias != nullptr) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (col0 + g * 8 + j < ep.n_total) v[j] += __ldg(ep.bias + col0 + g * 8 + j);
      }
      if (ep.relu) {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = fmaxf(v[j], 0.0f);
      }
    }
    uint4 pk;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
    *slot = pk;
  }
}

// Problem policy requirements (all __device__ const):
//   static constexpr int BN; static constexpr bool A_MN, B_MN, kZeroStages;
//   struct Tile { int kb0, kb1, n0; ... };
//   bool tile(int it, Tile&)                       enumerate this CTA's tiles
//   void load(const Tile&, int kb, uint8_t* a, uint8_t* b, uint64_t* bar)
//   void load_a(...a, bar) / load_b(...b, bar)     the two halves of load(); int res_kb (0: B not resident)
//   void store_panel(const Tile&, int panel, const void* smem)   TMA store of a 128x64 bf16 panel
//   bool row_valid(const Tile&, int row)           row is a real output (statistics mask)
//   void load_res_panel(const Tile&, int panel, void* smem, uint64_t* bar)   TMA load of the residual's panel
//   static constexpr bool kHalo; int out_row(int row)   row of the stored tile for a GEMM row (identity unless kHalo)
//   kHalo only: int cblks, R, S, PW; void load_halo(const Tile&, int cb, void* smem, uint64_t* bar)
//   int valid_prefix(const Tile&)                  n if exactly rows [0, n) are real outputs, -1 if irregular
//   void* row_ptr(const Tile&, int row)            fp32 output row pointer (direct modes), or nullptr
template <class P>
__device__ __forceinline__ void run(const P& prob, const Epilogue& ep) {
  constexpr int BN = P::BN;
  using C = Cfg<BN>;
  constexpr int STAGES = C::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int res_kb = prob.res_kb;            // > 0: B-resident mode
  constexpr bool kHalo = P::kHalo;
  const int nhalo = kHalo ? (res_kb > 0 ? 2 : MAX_HALOS) : 0;
  const int nstages = kHalo ? (res_kb > 0 ? 1 : min(C::MAX_STAGES, (C::STAGE_AREA - nhalo * HALO_BYTES) / C::B_STAGE_BYTES))
                            : (res_kb > 0 ? min(C::MAX_STAGES, (C::STAGE_AREA - res_kb * C::B_STAGE_BYTES) / A_STAGE_BYTES)
                                          : STAGES);
  uint8_t* sA = smem;                        // halo mode: the input boxes
  uint8_t* sB = kHalo ? sA + nhalo * HALO_BYTES : sA + nstages * A_STAGE_BYTES;
  uint8_t* sC = smem + C::STAGE_AREA;
  uint64_t* full = reinterpret_cast<uint64_t*>(sC + NUM_PANEL_BUFS * PANEL_BYTES);
  uint64_t* empty = full + C::MAX_STAGES;
  uint64_t* tfull = empty + C::MAX_STAGES;
  uint64_t* tempty = tfull + 2;
  uint64_t* bres = tempty + 2;               // the resident B tiles have landed
  uint64_t* rfull = bres + 1;                // residual panel has landed in staging buffer [NUM_PANEL_BUFS]
  uint64_t* hfull = rfull + NUM_PANEL_BUFS;  // halo mode: input box has landed / has been consumed [MAX_HALOS]
  uint64_t* hempty = hfull + MAX_HALOS;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(hempty + MAX_HALOS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::MAX_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull[a], 1); mbar_init(&tempty[a], NUM_EPI_THREADS / 32); }
    mbar_init(bres, 1);
    for (int b = 0; b < NUM_PANEL_BUFS; ++b) mbar_init(&rfull[b], 1);
    for (int b = 0; b < MAX_HALOS; ++b) { mbar_init(&hfull[b], 1); mbar_init(&hempty[b], 1); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  if (P::kZeroStages) {
    // partial boxes leave the tail rows of a stage untouched: they must read as zeros for ever
    uint4* p4 = reinterpret_cast<uint4*>(sA);
    const int n16 = STAGES * (A_STAGE_BYTES + C::B_STAGE_BYTES) / 16;
    for (int i = threadIdx.x; i < n16; i += NUM_THREADS) p4[i] = make_uint4(0, 0, 0, 0);
    fence_proxy_async();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      typename P::Tile t;
      if (res_kb > 0 && prob.tile(0, t)) {
        mbar_expect_tx(bres, (uint32_t)(res_kb * C::B_STAGE_BYTES));
        for (int kb = 0; kb < res_kb; ++kb) prob.load_b(t, kb, sB + kb * C::B_STAGE_BYTES, bres);
      }
      const uint32_t tx_a = ep.tx_bytes_a ? ep.tx_bytes_a : (uint32_t)A_STAGE_BYTES;
      const uint32_t tx_ab = ep.tx_bytes ? ep.tx_bytes : (uint32_t)(A_STAGE_BYTES + C::B_STAGE_BYTES);
      if constexpr (kHalo) {
        // One input box per (tile, channel block), issued one step ahead of the filter tiles it goes with.
        const int cblks = prob.cblks, taps = prob.R * prob.S;
        typename P::Tile tn;                     // box iterator, one (tile, block) ahead
        int it_n = 0, cb_n = 0, hs_n = 0;
        uint32_t hph_n = 0;
        bool more = prob.tile(0, tn);
        auto issue_box = [&]() -> bool {
          if (!more) return true;
          if (!mbar_wait(&hempty[hs_n], hph_n ^ 1u, abort_flag)) return false;
          mbar_expect_tx(&hfull[hs_n], ep.tx_bytes_a);
          prob.load_halo(tn, cb_n, sA + hs_n * HALO_BYTES, &hfull[hs_n]);
          if (++hs_n == nhalo) { hs_n = 0; hph_n ^= 1u; }
          if (++cb_n == cblks) { cb_n = 0; more = prob.tile(++it_n, tn); }
          return true;
        };
        ok = issue_box();
        for (int it = 0; ok && prob.tile(it, t); ++it) {
          for (int cb = 0; ok && cb < cblks; ++cb) {
            ok = issue_box();                    // the next box travels while this block's filter tiles are fed
            if (res_kb > 0) continue;
            for (int tap = 0; ok && tap < taps; ++tap) {
              if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
              mbar_expect_tx(&full[stage], (uint32_t)C::B_STAGE_BYTES);
              prob.load_b(t, tap * cblks + cb, sB + stage * C::B_STAGE_BYTES, &full[stage]);
              if (++stage == nstages) { stage = 0; phase ^= 1u; }
            }
          }
        }
      } else
      for (int it = 0; ok && prob.tile(it, t); ++it) {
        for (int kb = t.kb0; kb < t.kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          if (res_kb > 0) {
            mbar_expect_tx(&full[stage], tx_a);
            prob.load_a(t, kb, sA + stage * A_STAGE_BYTES, &full[stage]);
          } else {
            mbar_expect_tx(&full[stage], tx_ab);
            prob.load(t, kb, sA + stage * A_STAGE_BYTES, sB + stage * C::B_STAGE_BYTES, &full[stage]);
          }
          if (++stage == nstages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, P::A_MN ? 1 : 0, P::B_MN ? 1 : 0);
      // The issuing thread is one lane with nothing to hide its instruction latency behind: every instruction
      // between two tcgen05.mma widens the gap between them.  (Timestamps taken in this loop: a 128 x 64 x 16
      // MMA goes out every ~115 cycles, a 128 x 256 x 16 one every ~185 -- 32 and 128 cycles of tensor-pipe work
      // plus a fixed cost per instruction; narrow tiles are bound by that cost, not by their operands' traffic.
      // Dealing the K steps to several accumulators did not shorten it.)  Descriptors are therefore built once and advanced
      // by adding to their address field (bits 0-13, in 16-byte units; shared memory is < 256 KB, so no carry).
      constexpr uint64_t kStepA = P::A_MN ? (2048 >> 4) : (32 >> 4);      // K advance of 16 elements
      constexpr uint64_t kStepB = P::B_MN ? (2048 >> 4) : (32 >> 4);
      const uint64_t a_desc0 = P::A_MN ? umma_smem_desc(smem_u32(sA), 8192, 1024) : umma_smem_desc(smem_u32(sA), 16, 1024);
      const uint64_t b_desc0 = P::B_MN ? umma_smem_desc(smem_u32(sB), 8192, 1024) : umma_smem_desc(smem_u32(sB), 16, 1024);
      int stage = 0, acc = 0, hs = 0;
      uint32_t phase = 0, acc_phase = 0, hphase = 0;
      bool ok = true;
      typename P::Tile t;
      if (res_kb > 0 && prob.tile(0, t)) ok = mbar_wait(bres, 0u, abort_flag);
      for (int it = 0; ok && prob.tile(it, t); ++it) {
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1u, abort_flag)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        uint32_t accumulate = 0;                  // the tile's first MMA overwrites the accumulator
        if constexpr (kHalo) {
          const int cblks = prob.cblks, R = prob.R, S = prob.S;
          const uint64_t row_step = (uint64_t)(prob.PW * 8);           // one box row of pixels, in 16-byte units
          for (int cb = 0; ok && cb < cblks; ++cb) {
            if (!mbar_wait(&hfull[hs], hphase, abort_flag)) { ok = false; break; }
            tc_fence_after();
            // the window of tap (r, s): the same box, (r * PW + s) pixel rows (128 bytes each) further on
            uint64_t a_row = a_desc0 + (uint64_t)(hs * (HALO_BYTES >> 4));
            uint64_t b_tap = b_desc0 + (uint64_t)(cb * (C::B_STAGE_BYTES >> 4));       // resident: k-block tap*cblks+cb
            const uint64_t b_tap_step = (uint64_t)(cblks * (C::B_STAGE_BYTES >> 4));
            for (int r = 0; ok && r < R; ++r, a_row += row_step) {
              uint64_t a_tap = a_row;
              for (int sx = 0; sx < S; ++sx, a_tap += 8, b_tap += b_tap_step) {
                uint64_t b_cur = b_tap;
                if (res_kb == 0) {
                  if (!mbar_wait(&full[stage], phase, abort_flag)) { ok = false; break; }
                  tc_fence_after();
                  b_cur = b_desc0 + (uint64_t)(stage * (C::B_STAGE_BYTES >> 4));
                }
#pragma unroll
                for (int j = 0; j < BK / 16; ++j) {
                  umma_bf16(d_tmem, a_tap + j * kStepA, b_cur + j * kStepB, idesc, accumulate);
                  accumulate = 1;
                }
                if (res_kb == 0) {
                  umma_commit(&empty[stage]);
                  if (++stage == nstages) { stage = 0; phase ^= 1u; }
                }
              }
            }
            if (!ok) break;
            umma_commit(&hempty[hs]);
            if (++hs == nhalo) { hs = 0; hphase ^= 1u; }
          }
        } else
        for (int kb = t.kb0; kb < t.kb1; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint64_t a_cur = a_desc0 + (uint64_t)(stage * (A_STAGE_BYTES >> 4));
          const uint64_t b_cur = b_desc0 + (uint64_t)((res_kb > 0 ? kb : stage) * (C::B_STAGE_BYTES >> 4));
#pragma unroll
          for (int j = 0; j < BK / 16; ++j) {
            umma_bf16(d_tmem, a_cur + j * kStepA, b_cur + j * kStepB, idesc, accumulate);
            accumulate = 1;
          }
          umma_commit(&empty[stage]);
          if (++stage == nstages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(&tfull[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (8 warps)
    // A warp may only touch TMEM lanes [32*(warp%4), +32): two warps share each lane quarter and
    // split every 64-column panel into halves.
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;       // which 32 columns of a 64-column panel
    const int et = threadIdx.x - 64;        // 0..255 among the epilogue threads
    const int row = q * 32 + lane;          // tile row owned by this thread
    const int drow = prob.out_row(row);     // its row in the stored tile (halo mode: margin rows have none)
    int acc = 0;
    uint32_t acc_phase = 0;
    int buf = 0;                            // staging panel buffer in use (ring)
    // statistics: thread (cp = et % 32, rg = et / 32) covers columns 2cp, 2cp+1 of each panel, rows 16rg..+16
    float st_sum[BN / 64][2], st_sq[BN / 64][2];
#pragma unroll
    for (int pnl = 0; pnl < BN / 64; ++pnl) { st_sum[pnl][0] = st_sum[pnl][1] = st_sq[pnl][0] = st_sq[pnl][1] = 0.f; }
    int stats_n0 = -1;
    const bool has_res = ep.residual != nullptr;
    const bool plain = ep.bias == nullptr && !ep.relu && !has_res;
    uint32_t gpanel = 0;                    // panels processed so far (all threads count alike)
    // Residual prefetch (thread 0): the residual's panels are brought into the staging ring by TMA two panels
    // ahead of the epilogue, which then adds them in place.
    typename P::Tile pf_t;
    int pf_it = 0, pf_pnl = 0;
    uint32_t pf_g = 0;
    bool pf_valid = false;
    auto prefetch_residual = [&]() {
      if (!pf_valid) return;
      const int b = (int)(pf_g % NUM_PANEL_BUFS);
      mbar_expect_tx(&rfull[b], (uint32_t)PANEL_BYTES);
      prob.load_res_panel(pf_t, pf_pnl, sC + b * PANEL_BYTES, &rfull[b]);
      ++pf_g;
      if (++pf_pnl >= min(BN / 64, (ep.n_total - pf_t.n0 + 63) / 64)) {
        pf_pnl = 0;
        pf_valid = prob.tile(++pf_it, pf_t);
      }
    };
    if (has_res && et == 0) {
      pf_valid = prob.tile(0, pf_t);
      prefetch_residual();
      prefetch_residual();
    }
    bool ok = true;
    typename P::Tile t;
    for (int it = 0; ok && prob.tile(it, t); ++it) {
      if (!mbar_wait(&tfull[acc], acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after();
      stats_n0 = t.n0;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + half * 32);
      if (ep.out_mode == OUT_BF16) {
        const int npan = min(BN / 64, (ep.n_total - t.n0 + 63) / 64);   // uniform across the CTA
        uint32_t row_mask = 0xffffu;          // validity of this thread's 16 statistics rows, once per tile
        if (ep.col_sum != nullptr) {
          const int prefix = prob.valid_prefix(t);      // rows [0, prefix) are the real outputs, or -1
          if (prefix >= 0) {
            const int mine = min(16, max(0, prefix - (et >> 5) * 16));
            row_mask = (1u << mine) - 1u;
          } else {
            row_mask = 0u;
            for (int rr = 0; rr < 16; ++rr)
              if (prob.row_valid(t, (et >> 5) * 16 + rr)) row_mask |= 1u << rr;
          }
        }
        uint32_t rbuf[2][32];
        tmem_ld_32x32b_x32(t_row, rbuf[0]);
#pragma unroll
        for (int pnl = 0; pnl < BN / 64; ++pnl) {
          if (pnl < npan) {
            tmem_ld_wait();
            if (pnl + 1 < npan)   // the next panel's accumulators travel while this one is converted
              tmem_ld_32x32b_x32(t_row + (uint32_t)((pnl + 1) * 64), rbuf[(pnl + 1) & 1]);
            uint8_t* panel = sC + buf * PANEL_BYTES;
            // This buffer was last read by the store issued NUM_PANEL_BUFS panels ago; thread 0 waited for
            // that read before it arrived at the previous panel's barrier (see below), so it is free.
            const int col0 = t.n0 + pnl * 64 + half * 32;
            if (has_res && !mbar_wait(&rfull[buf], (gpanel / NUM_PANEL_BUFS) & 1u, abort_flag)) { ok = false; break; }
            if (drow >= 0) {
              if (plain) pack_row_to_panel<true>(rbuf[pnl & 1], panel, drow, half, col0, ep, false);
              else pack_row_to_panel<false>(rbuf[pnl & 1], panel, drow, half, col0, ep, has_res);
            }
            fence_proxy_async();
            named_barrier_sync(1, NUM_EPI_THREADS);    // the panel is complete and visible to the TMA engine
            if (et == 0) {
              prob.store_panel(t, pnl, panel);
              tma_store_commit();
              // One barrier per panel: before thread 0 reaches the NEXT panel's barrier it makes sure that all
              // but the two newest stores have read their buffers, so after that barrier everyone may overwrite
              // the buffer used three panels ago -- the one the panel after next needs.
              tma_store_wait_read<2>();
              if (has_res) prefetch_residual();       // into the buffer the panel after next will use
            }
            if (ep.col_sum != nullptr) {
              // thread (cp, rg): columns 2cp, 2cp+1 of the panel, rows 16rg .. 16rg+15, read back as stored
              const int cp = et & 31, rg = et >> 5;
              const uint8_t* colp = panel + (cp & 3) * 4;
              const int chunk = cp >> 2;
              float s0 = 0.f, s1 = 0.f, q0 = 0.f, q1 = 0.f;
#pragma unroll
              for (int rr = 0; rr < 16; ++rr) {
                const int r_ = rg * 16 + rr;
                uint32_t w = *reinterpret_cast<const uint32_t*>(colp + r_ * 128 + ((chunk ^ (r_ & 7)) << 4));
                if (!((row_mask >> rr) & 1u)) w = 0u;        // rows outside the tensor count as zeros
                const float f0 = __uint_as_float(w << 16), f1 = __uint_as_float(w & 0xffff0000u);
                s0 += f0; s1 += f1; q0 = fmaf(f0, f0, q0); q1 = fmaf(f1, f1, q1);
              }
              st_sum[pnl][0] += s0; st_sum[pnl][1] += s1; st_sq[pnl][0] += q0; st_sq[pnl][1] += q1;
            }
            buf = (buf + 1) % NUM_PANEL_BUFS;
            ++gpanel;
          }
        }
        if (!ok) break;
      } else {
        // fp32 outputs (logits, split-K weight gradients): direct stores / atomics from registers
        float* out_row = reinterpret_cast<float*>(prob.row_ptr(t, row));
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_row + (uint32_t)(c * 64), r);
          tmem_ld_wait();
          const int col0 = t.n0 + c * 64 + half * 32;
          if (out_row != nullptr) {
            // four columns at a time (rows are 32-byte aligned and N is a multiple of 8): 16-byte stores, and
            // 16-byte reductions for the split-K case, a quarter of the atomic instructions
#pragma unroll
            for (int j4 = 0; j4 < 8; ++j4) {
              if (col0 + j4 * 4 < ep.n_total) {
                float4 v = make_float4(__uint_as_float(r[j4 * 4]), __uint_as_float(r[j4 * 4 + 1]),
                                       __uint_as_float(r[j4 * 4 + 2]), __uint_as_float(r[j4 * 4 + 3]));
                if (ep.bias != nullptr) {
                  const float4 b4 = __ldg(reinterpret_cast<const float4*>(ep.bias + col0 + j4 * 4));
                  v.x += b4.x; v.y += b4.y; v.z += b4.z; v.w += b4.w;
                }
                if (ep.relu) { v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f); }
                float4* dst = reinterpret_cast<float4*>(out_row + col0 + j4 * 4);
                if (ep.out_mode == OUT_F32) *dst = v;
                else atomicAdd(dst, v);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (ep.col_sum != nullptr && stats_n0 >= 0) {   // one flush per CTA: its tiles share the column range
      const int cp = et & 31;
#pragma unroll
      for (int pnl = 0; pnl < BN / 64; ++pnl) {
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int col = stats_n0 + pnl * 64 + cp * 2 + k;
          if (col < ep.n_total) {
            atomicAdd(ep.col_sum + col, st_sum[pnl][k]);
            atomicAdd(ep.col_sqsum + col, st_sq[pnl][k]);
          }
        }
      }
    }
    if (et == 0) tma_store_wait_all();               // shared memory must outlive the bulk stores
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    __nanosleep(1000000);
    if (threadIdx.x == 0 && ep.error_flag != nullptr) atomicExch(ep.error_flag, 1);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

}  // namespace umma
