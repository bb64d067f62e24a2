// W4A16 GEMM for sm_100a:  C[M,N] = A[M,K] * dequant(W[N,K])^T (+ bias)
//
// "Swap-AB" tcgen05 design.  The dequantized weight tile is the UMMA *A*
// operand (128 weight rows = 128 TMEM lanes), the activation tile is the UMMA
// *B* operand (m_tile tokens = UMMA N, 16..256), so the same kernel covers
// decode (M = 1..64, HBM-bound) and prefill (M in the thousands, tensor-bound).
//
//   warp 0        weight producer: 1-D bulk copies of packed codes + group
//                 scales (+ zero points) into a deep shared-memory ring
//   warp 1        activation producer: 2-D TMA boxes (64 K x m_tile rows,
//                 128-byte swizzle) into a second ring
//   warp 2        MMA issuer: tcgen05.mma kind::f16, fp32 accumulators in TMEM
//   warp 3        TMEM allocation / release
//   warps 4..11   dequant: thread = weight row; 32 bytes of codes -> 64 values
//                 of the activation type, written straight into tensor memory
//                 (tcgen05.st) where the MMA reads them as its A operand --
//                 the expanded weights never touch shared memory.  Two groups
//                 of four warps alternate k-blocks.
//   warps 12..15  epilogue: tcgen05.ld -> (+bias) -> cast -> global, or fp32
//                 partials + last-arriver reduction when K is split
//
// Replaces the reference's humming<> kernel
// (humming/include/humming/kernel/humming_ws.cuh:25-176) and its pipelines
// (memory/g2s_pipeline.cuh, memory/s2r_pipeline.cuh, mma/wmma.cuh,
// epilogue/pipeline.cuh).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "dequant.cuh"
#include "ptx.cuh"
#include "sched.cuh"

namespace hm {

constexpr int kTileN = 128;        // weight rows per tile (UMMA M)
constexpr int kBlockK = 64;        // K elements per pipeline stage
constexpr int kCodeBytes = kTileN * kBlockK / 2;  // 4096: packed 4-bit codes of one stage
constexpr int kScaleBytes = kTileN * 2;           // 256: one 16-bit scale per row
constexpr int kZpBytes = kTileN / 2;              // 64: one nibble per row
constexpr int kWStageBytes = 4480;                // 4096 + 256 + 64, padded to a multiple of 128
constexpr int kNumBarrierSlots = 128;
constexpr int kTraceEvents = 128;  // traced k-blocks per role
// Timing experiments (results become wrong; used only to locate bottlenecks).
enum : int { HM_DBG_SKIP_MATH = 1, HM_DBG_SKIP_TMEM_ST = 2, HM_DBG_SKIP_MMA = 4, HM_DBG_SKIP_X_LOAD = 8, HM_DBG_SKIP_W_LOAD = 16 };

struct GemmParams {
  const uint8_t* w;        // prepared codes   [n_tile][kb][2][128][16 B]
  const uint8_t* w_scale;  // prepared scales  [n_tile][group][128] x 16 bit
  const uint8_t* w_zp;     // prepared zero points [n_tile][group][64 B] or null
  const void* bias;        // [N] in the output type, or null
  void* c;                 // [M, ldc] output
  float* partials;         // workspace: [grid*2][m_tile][128] fp32
  int* counters;           // workspace: [tiles*4], zero on entry and on exit
  int* status;             // workspace: [8], written on abort only
  int M, N, K;
  int ldc;
  int groups;              // scale groups along K
  int kb_per_group;        // k-blocks per scale group
  SchedParams sched;
  unsigned long long* trace;  // debug: per-role clock64 timeline of CTA 0, or null
  int dbg;                    // debug: HM_DBG_* experiment switches (0 in production)
};

template <int MT, bool A_TMEM>
struct GemmCfg {
  // Ring depths: SX activation stages (shared memory; deep for small token
  // tiles, where the stage is tiny and L2 latency must be covered), SA operand
  // slots for the dequantized weights (tensor memory, 32 columns each, or 16 KB
  // of shared memory in the cross-check variant), SW packed-weight stages.
  static constexpr int SX = MT <= 16 ? 32 : MT <= 32 ? 24 : MT <= 64 ? 12 : MT <= 128 ? 6 : 4;
  static constexpr int SA = A_TMEM ? 8 : 3;
  static constexpr int SW = MT <= 32 ? 16 : (MT <= 64 ? 12 : 8);
  // Dequant warp groups (4 warps each) taking k-blocks round-robin.
  static constexpr int NGROUPS = MT <= 64 ? 4 : 2;
  static constexpr int EPI_WARP0 = 4 + 4 * NGROUPS;
  static constexpr int THREADS = (EPI_WARP0 + 4) * 32;
  static constexpr int ACC_BUFS = (2 * MT + (A_TMEM ? SA * 32 : 0) <= 512) ? 2 : 1;
  static constexpr int A_COL0 = ACC_BUFS * MT;
  static constexpr int USED_COLS = A_COL0 + (A_TMEM ? SA * 32 : 0);
  static constexpr int TMEM_COLS = USED_COLS <= 32 ? 32 : USED_COLS <= 64 ? 64 : USED_COLS <= 128 ? 128 : USED_COLS <= 256 ? 256 : 512;
  static constexpr int X_STAGE = MT * 128;
  static constexpr int A_STAGE = A_TMEM ? 0 : kTileN * 128;
  static constexpr int SMEM_X = 0;
  static constexpr int SMEM_A = SMEM_X + SX * X_STAGE;
  static constexpr int SMEM_W = SMEM_A + SA * A_STAGE;
  static constexpr int SMEM_BAR = SMEM_W + SW * kWStageBytes;
  static constexpr int SMEM_TOTAL = SMEM_BAR + kNumBarrierSlots * 8 + 64;
  static constexpr int SMEM_ALLOC = SMEM_TOTAL + 1024;  // slack for manual 1024-byte alignment
  static_assert(USED_COLS <= 512, "tensor memory budget");
  static_assert(SMEM_ALLOC <= 232448, "shared memory budget");
  static_assert(2 * SW + 2 * SX + 2 * SA + 5 <= kNumBarrierSlots, "barrier slots");
};

template <bool BF16>
HM_DEVICE void store_out(void* c, size_t idx, float v) {
  if constexpr (BF16) {
    reinterpret_cast<__nv_bfloat16*>(c)[idx] = __float2bfloat16_rn(v);
  } else {
    reinterpret_cast<__half*>(c)[idx] = __float2half_rn(v);
  }
}
template <bool BF16>
HM_DEVICE float load_bias(const void* b, int n) {
  if constexpr (BF16) {
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(b)[n]);
  } else {
    return __half2float(reinterpret_cast<const __half*>(b)[n]);
  }
}

HM_DEVICE void report_abort(int* status, int code, int a, int b) {
  if (atomicCAS(&status[0], 0, code) == 0) {
    status[1] = blockIdx.x;
    status[2] = a;
    status[3] = b;
    __threadfence();
  }
}

template <int MT, bool BF16, bool HAS_ZP, bool A_TMEM>
__global__ void __launch_bounds__(GemmCfg<MT, A_TMEM>::THREADS, 1)
gemm_w4a16_kernel(const GemmParams p, const __grid_constant__ CUtensorMap tmap_x) {
  using Cfg = GemmCfg<MT, A_TMEM>;
  constexpr int SX = Cfg::SX;
  constexpr int SA = Cfg::SA;
  constexpr int SW = Cfg::SW;
  constexpr int NGROUPS = Cfg::NGROUPS;
  constexpr int ACC_BUFS = Cfg::ACC_BUFS;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const uint32_t x_smem = smem_base + Cfg::SMEM_X;
  const uint32_t a_smem = smem_base + Cfg::SMEM_A;
  const uint32_t w_smem = smem_base + Cfg::SMEM_W;
  const uint32_t bar0 = smem_base + Cfg::SMEM_BAR;
  // barrier slots
  auto w_full = [&](int i) { return bar0 + 8u * i; };
  auto w_empty = [&](int i) { return bar0 + 8u * (SW + i); };
  auto x_full = [&](int i) { return bar0 + 8u * (2 * SW + i); };
  auto x_empty = [&](int i) { return bar0 + 8u * (2 * SW + SX + i); };
  auto a_full = [&](int i) { return bar0 + 8u * (2 * SW + 2 * SX + i); };
  auto a_empty = [&](int i) { return bar0 + 8u * (2 * SW + 2 * SX + SA + i); };
  constexpr int kBarAcc = 2 * SW + 2 * SX + 2 * SA;
  auto acc_full = [&](int i) { return bar0 + 8u * (kBarAcc + i); };
  auto acc_empty = [&](int i) { return bar0 + 8u * (kBarAcc + 2 + i); };
  const uint32_t drain_bar = bar0 + 8u * (kBarAcc + 4);
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem_gen + Cfg::SMEM_BAR + kNumBarrierSlots * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + Cfg::SMEM_BAR + kNumBarrierSlots * 8 + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < SW; ++i) {
      mbar_init(w_full(i), 1);
      mbar_init(w_empty(i), 4);
    }
    for (int i = 0; i < SX; ++i) {
      mbar_init(x_full(i), 1);
      mbar_init(x_empty(i), 1);
    }
    for (int i = 0; i < SA; ++i) {
      mbar_init(a_full(i), 4);
      mbar_init(a_empty(i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(acc_full(i), 1);
      mbar_init(acc_empty(i), 4);
    }
    mbar_init(drain_bar, 1);
    abort_flag[0] = 0;  // raised by the first wait that gives up
    abort_flag[1] = 0;  // separate flag for the drain waits of the abort path
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  if (warp == 3) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_holder)), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 1 && lane == 0) tma_prefetch_desc(&tmap_x);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  SegIter iter;
  iter.init(p.sched, blockIdx.x);
  Segment seg;
  const bool tracing = p.trace != nullptr && blockIdx.x == 0;
  auto trace = [&](int role, int idx, int j) {
    if (tracing && idx < kTraceEvents) p.trace[(role * kTraceEvents + idx) * 4 + j] = clock64();
  };

  if (warp == 0) {
    // ------------------------------------------------ weight producer
    if (lane == 0) {
      const uint64_t pol = l2_policy_evict_first();
      int it = 0;
      bool ok = true;
      while (ok && iter.next(seg)) {
        const size_t tile_code0 = static_cast<size_t>(seg.n_tile) * p.sched.kb_per_tile;
        const size_t tile_grp0 = static_cast<size_t>(seg.n_tile) * p.groups;
        for (int kb = seg.kb0; kb < seg.kb1; ++kb, ++it) {
          const int sw = it % SW;
          const uint32_t ph = (it / SW) & 1;
          if (!mbar_wait_bounded(w_empty(sw), ph ^ 1, abort_flag)) {
            report_abort(p.status, HM_ABORT_W_EMPTY, it, sw);
            ok = false;
            break;
          }
          trace(0, it, 0);
          const uint32_t dst = w_smem + sw * kWStageBytes;
          const int g = kb / p.kb_per_group;
          if (p.dbg & HM_DBG_SKIP_W_LOAD) {
            mbar_arrive(w_full(sw));
          } else {
            mbar_arrive_expect_tx(w_full(sw), kCodeBytes + kScaleBytes + (HAS_ZP ? kZpBytes : 0));
            bulk_g2s_hint(dst, p.w + (tile_code0 + kb) * kCodeBytes, kCodeBytes, w_full(sw), pol);
            bulk_g2s(dst + kCodeBytes, p.w_scale + (tile_grp0 + g) * kScaleBytes, kScaleBytes, w_full(sw));
            if constexpr (HAS_ZP) {
              bulk_g2s(dst + kCodeBytes + kScaleBytes, p.w_zp + (tile_grp0 + g) * kZpBytes, kZpBytes, w_full(sw));
            }
          }
          trace(0, it, 1);
        }
      }
      if (!ok) {
        // Abort path: let copies already issued land before the CTA exits.
        for (int j = 0; j < SW && j < it; ++j) {
          const int last_it = it - 1 - j;
          mbar_wait_bounded(w_full(last_it % SW), (last_it / SW) & 1, abort_flag + 1);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ activation producer
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      while (ok && iter.next(seg)) {
        for (int kb = seg.kb0; kb < seg.kb1; ++kb, ++it) {
          const int s = it % SX;
          const uint32_t ph = (it / SX) & 1;
          if (!mbar_wait_bounded(x_empty(s), ph ^ 1, abort_flag)) {
            report_abort(p.status, HM_ABORT_X_EMPTY, it, s);
            ok = false;
            break;
          }
          trace(1, it, 0);
          if (p.dbg & HM_DBG_SKIP_X_LOAD) {
            mbar_arrive(x_full(s));
          } else {
            mbar_arrive_expect_tx(x_full(s), Cfg::X_STAGE);
            tma_load_2d(x_smem + s * Cfg::X_STAGE, &tmap_x, kb * kBlockK, seg.m_tile * MT, x_full(s));
          }
          trace(1, it, 1);
        }
      }
      if (!ok) {
        for (int j = 0; j < SX && j < it; ++j) {
          const int last_it = it - 1 - j;
          mbar_wait_bounded(x_full(last_it % SX), (last_it / SX) & 1, abort_flag + 1);
        }
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(BF16 ? 1 : 0, BF16 ? 1 : 0, kTileN, MT);
      int it = 0;
      int sc = 0;
      bool ok = true;
      while (ok && iter.next(seg)) {
        const int b = sc % ACC_BUFS;
        const uint32_t acc_ph = (sc / ACC_BUFS) & 1;
        if (!mbar_wait_bounded(acc_empty(b), acc_ph ^ 1, abort_flag)) {
          report_abort(p.status, HM_ABORT_MMA_ACC, sc, b);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + b * MT;
        for (int kb = seg.kb0; kb < seg.kb1; ++kb, ++it) {
          const int sx = it % SX;
          const int sa = it % SA;
          trace(2, it, 0);
          const bool a_ok = mbar_wait_bounded(a_full(sa), (it / SA) & 1, abort_flag);
          trace(2, it, 1);
          if (!a_ok || !mbar_wait_bounded(x_full(sx), (it / SX) & 1, abort_flag)) {
            report_abort(p.status, HM_ABORT_MMA_OPERANDS, it, sa);
            ok = false;
            break;
          }
          trace(2, it, 2);
          tc_fence_after();
          const uint32_t xs = x_smem + sx * Cfg::X_STAGE;
#pragma unroll
          for (int k4 = 0; k4 < kBlockK / 16; ++k4) {
            if (p.dbg & HM_DBG_SKIP_MMA) break;
            const uint32_t accumulate = (kb != seg.kb0 || k4 != 0) ? 1u : 0u;
            const uint64_t b_desc = umma_desc_sw128(xs, k4 * 32);
            if constexpr (A_TMEM) {
              mma_f16_ts(d_tmem, tmem_base + Cfg::A_COL0 + sa * 32 + k4 * 8, b_desc, idesc, accumulate);
            } else {
              mma_f16_ss(d_tmem, umma_desc_sw128(a_smem + sa * Cfg::A_STAGE, k4 * 32), b_desc, idesc, accumulate);
            }
          }
          tc_commit(x_empty(sx));
          tc_commit(a_empty(sa));
          trace(2, it, 3);
        }
        if (!ok) break;
        tc_commit(acc_full(b));
        ++sc;
      }
      if (!ok) {
        // Abort path: wait for MMAs already issued before TMEM is released.
        tc_commit(drain_bar);
        mbar_wait_bounded(drain_bar, 0, abort_flag + 1);
      }
    }
  } else if (warp >= 4 && warp < Cfg::EPI_WARP0) {
    // ------------------------------------------------ dequant warps
    const int group = (warp - 4) >> 2;  // groups take k-blocks round-robin
    const int q = warp & 3;             // TMEM lane quarter this warp may access
    const int row = q * 32 + lane;
    int it = 0;
    bool ok = true;
    while (ok && iter.next(seg)) {
      for (int kb = seg.kb0; kb < seg.kb1; ++kb, ++it) {
        if ((it % NGROUPS) != group) continue;
        const int sw = it % SW;
        const int s = it % SA;
        if (!mbar_wait_bounded(w_full(sw), (it / SW) & 1, abort_flag)) {
          if (lane == 0) report_abort(p.status, HM_ABORT_DQ_W_FULL, it, sw);
          ok = false;
          break;
        }
        if (q == 0 && lane == 0) trace(3 + group, it, 0);
        const uint8_t* ws = smem_gen + Cfg::SMEM_W + sw * kWStageBytes;
        const uint4 lo = *reinterpret_cast<const uint4*>(ws + row * 16);
        const uint4 hi = *reinterpret_cast<const uint4*>(ws + 2048 + row * 16);
        const uint32_t sc16 = *reinterpret_cast<const uint16_t*>(ws + kCodeBytes + row * 2);
        const uint32_t scale2 = sc16 | (sc16 << 16);
        uint32_t zp = 8;
        if constexpr (HAS_ZP) {
          zp = (ws[kCodeBytes + kScaleBytes + (row >> 1)] >> ((row & 1) * 4)) & 0xF;
        }
        const uint32_t zpm = zp_magic_pair<BF16>(zp);
        uint32_t out[32];
        if (p.dbg & HM_DBG_SKIP_MATH) {
#pragma unroll
          for (int i = 0; i < 32; ++i) out[i] = lo.x + i;
        } else {
        dequant_word_u4<BF16>(lo.x, zpm, scale2, out + 0);
        dequant_word_u4<BF16>(lo.y, zpm, scale2, out + 4);
        dequant_word_u4<BF16>(lo.z, zpm, scale2, out + 8);
        dequant_word_u4<BF16>(lo.w, zpm, scale2, out + 12);
        dequant_word_u4<BF16>(hi.x, zpm, scale2, out + 16);
        dequant_word_u4<BF16>(hi.y, zpm, scale2, out + 20);
        dequant_word_u4<BF16>(hi.z, zpm, scale2, out + 24);
        dequant_word_u4<BF16>(hi.w, zpm, scale2, out + 28);
        }
        // The packed stage has been consumed into registers: hand it back.
        __syncwarp();
        if (lane == 0) mbar_arrive(w_empty(sw));
        if (q == 0 && lane == 0) trace(3 + group, it, 1);
        // Wait until the MMAs that read this operand slot last time are done.
        if (!mbar_wait_bounded(a_empty(s), ((it / SA) & 1) ^ 1, abort_flag)) {
          if (lane == 0) report_abort(p.status, HM_ABORT_DQ_SLOT, it, s);
          ok = false;
          break;
        }
        if (q == 0 && lane == 0) trace(3 + group, it, 2);
        if constexpr (A_TMEM) {
          tc_fence_after();
          if (!(p.dbg & HM_DBG_SKIP_TMEM_ST)) {
            tmem_st_x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + Cfg::A_COL0 + s * 32, out);
            tc_wait_st();
          } else if (out[5] == 0x12345u) {
            p.status[7] = out[9];  // keep the math alive when the store is skipped
          }
          tc_fence_before();
        } else {
          // 128-byte rows, 16-byte chunk c of row r stored at chunk (c ^ (r & 7)).
          uint8_t* a_row = smem_gen + Cfg::SMEM_A + s * Cfg::A_STAGE + (row >> 3) * 1024 + (row & 7) * 128;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            *reinterpret_cast<uint4*>(a_row + ((c ^ (row & 7)) * 16)) =
                make_uint4(out[4 * c], out[4 * c + 1], out[4 * c + 2], out[4 * c + 3]);
          }
          fence_proxy_async_smem();
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(a_full(s));
        if (q == 0 && lane == 0) trace(3 + group, it, 3);
      }
    }
  } else if (warp >= Cfg::EPI_WARP0) {
    // ------------------------------------------------ epilogue warps
    const int q = warp & 3;
    const int row = q * 32 + lane;
    int sc = 0;
    bool ok = true;
    while (ok && iter.next(seg)) {
      const int b = sc % ACC_BUFS;
      if (!mbar_wait_bounded(acc_full(b), (sc / ACC_BUFS) & 1, abort_flag)) {
        if (lane == 0) report_abort(p.status, HM_ABORT_EPI_ACC, sc, b);
        ok = false;
        break;
      }
      tc_fence_after();
      const int n = seg.n_tile * kTileN + row;
      const int m0 = seg.m_tile * MT;
      const int m_valid = (p.M - m0) < MT ? (p.M - m0) : MT;
      const float bias = (p.bias != nullptr) ? load_bias<BF16>(p.bias, n) : 0.f;
      float* slot = p.partials + static_cast<size_t>(seg.slot) * (MT * kTileN);
      const uint32_t t_acc = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + b * MT;
#pragma unroll 1
      for (int c0 = 0; c0 < MT; c0 += 16) {
        if (c0 >= m_valid) break;  // warp-uniform
        uint32_t v[16];
        tmem_ld_x16(t_acc + c0, v);
        tc_wait_ld();
        if (!seg.partial) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (c0 + j < m_valid) {
              store_out<BF16>(p.c, static_cast<size_t>(m0 + c0 + j) * p.ldc + n, __uint_as_float(v[j]) + bias);
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (c0 + j < m_valid) slot[(c0 + j) * kTileN + row] = __uint_as_float(v[j]);
          }
        }
      }
      // Accumulator drained: the MMA issuer may overwrite it.
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty(b));
      ++sc;

      if (seg.partial) {
        // Publish this warp's quarter of the partial tile, then find out whether
        // every other contributor has already published its own.
        __threadfence();
        __syncwarp();
        int last = 0;
        if (lane == 0) {
          int* ctr = p.counters + seg.tile * 4 + q;
          const int old = atomicAdd(ctr, 1);
          last = (old == seg.nseg - 1) ? 1 : 0;
          if (last) *ctr = 0;  // leave the workspace clean for the next launch
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) {
          __threadfence();
          // Sum the contributors in CTA order (a fixed order, so the result does
          // not depend on who arrived last); 8 columns at a time keeps 8 loads per
          // contributor in flight.
          for (int j0 = 0; j0 < m_valid; j0 += 8) {
            float acc[8];
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) acc[jj] = 0.f;
            for (int cs = 0; cs < seg.nseg; ++cs) {
              const int cta = seg.first_cta + cs;
              const float* src = p.partials + static_cast<size_t>(sched_slot(p.sched, cta, seg.tile)) * (MT * kTileN) +
                                 j0 * kTileN + row;
              float v[8];
#pragma unroll
              for (int jj = 0; jj < 8; ++jj) v[jj] = (j0 + jj < m_valid) ? __ldcg(src + jj * kTileN) : 0.f;
#pragma unroll
              for (int jj = 0; jj < 8; ++jj) acc[jj] += v[jj];
            }
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
              if (j0 + jj < m_valid) store_out<BF16>(p.c, static_cast<size_t>(m0 + j0 + jj) * p.ldc + n, acc[jj] + bias);
            }
          }
        }
      }
    }
  }

  // Every role ends here, also after an abort (all waits are bounded).
  tc_fence_before();
  __syncthreads();
  if (warp == 3) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace hm
