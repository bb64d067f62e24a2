// W4A16 GEMM for 1 to 16 tokens ("decode kernel"): warp-level mma.sync on
// weights decoded in registers; the packed weights stream through a ring of
// shared-memory stages filled by bulk copies (cp.async.bulk + mbarrier), the
// expanded weights are never stored anywhere.
//
// Why not tcgen05 here: one tcgen05.mma covers 128 weight rows x 16 K in >= 52
// cycles whatever the token count (80 measured with the dequant warps running),
// which alone is 87 % of the HBM time of a 4-bit weight stream, and a launch of
// the warp-specialised kernel spends 5-6 us in start-up and barrier hand-offs.
// For a few tokens the work per weight is the decode itself (about two
// instructions per weight); a warp-level m16n8k16 MMA adds one instruction per
// 256 weights and takes the decoded pairs straight from registers.
//
// Mapping.  A CTA of 4 warps owns one 128-row weight tile and a K range; warp w
// owns rows 32w .. 32w+31 as two m16 blocks.  One thread keeps kGemvStages
// stages in flight, each the 8 KB of codes of a 128-K step plus the step's
// scales and zero points (the same blocks the tensor-memory kernel streams).  In
// the prepared layout a 16-byte chunk holds 32 consecutive K of one row, word
// j = K 8j .. 8j+7, and ((word >> 4t) & 0x000F000F) is the pair (K 8j+2t,
// 8j+2t+1): exactly the pair lane (g, t) = (lane / 4, lane % 4) feeds to the
// MMA as A-fragment element for row g (or g+8), so every lane extracts only its
// own pair of every word.  The MMA runs on the raw codes (exact in 16 bits);
// scale and zero point are applied once per scale group on the fp32 group sum
// (y += s * (sum (base+q) x - (base+zp) sum x)), which equals the product with
// weights decoded one by one up to fp32 rounding.  Activations are staged once
// per CTA in shared memory (row pitch padded by 16 bytes: conflict-free
// B-fragment loads), zero rows above M.  K is split over CTAs; partial sums go
// to an fp32 workspace and the last CTA of a tile to arrive (atomic counter, no
// spinning) adds them in split order, so the result does not depend on arrival
// order.  The waits on the stage barriers are bounded like every wait of the
// library: on expiry the CTA records a status code and leaves.
//
// Same role as the reference's smallest M bucket of humming<>
// (humming/layer.py:403-451, humming/include/humming/kernel/humming.cuh); the
// reference has no separate small-M kernel.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "dequant.cuh"
#include "gemm_w4a16.cuh"  // store_out, load_bias
#include "ptx.cuh"

namespace hm {

struct GemvParams {
  const uint8_t* w;        // prepared codes   [n_tile][K/128][4 chunks of 32 K][128 rows][16 B]
  const uint8_t* w_scale;  // prepared scales  [n_tile][group][128] x 16 bit
  const uint8_t* w_zp;     // prepared zero points [n_tile][group][64 B] or null
  const void* bias;        // [N] in the output type, or null
  const void* x;           // [M, lda] activations, 16 bit
  void* c;                 // [M, ldc] output, 16 bit
  float* partials;         // workspace: [splits][M][N] fp32 (splits > 1)
  int* counters;           // workspace: [n_tiles], zero on entry and on exit
  int* status;             // workspace: [8], written on abort only
  int M, N, K;
  int lda, ldc;
  int group_size;          // K elements per scale group (64, or a multiple of 128)
  int groups;              // K / group_size
  int steps_per_group;     // 128-K steps per scale group (>= 1)
  int groups_per_step;     // scale groups per 128-K step (1 or 2)
  int n_tiles;             // N / 128
  int kb_total;            // K / 128
  int steps_per_cta;       // 128-K steps per CTA
  int splits;              // CTAs per tile
};

constexpr int kGemvThreads = 128;
constexpr int kGemvXPad = 8;   // elements of padding per activation row in shared memory
#ifndef HM_GEMV_STAGES
#define HM_GEMV_STAGES 3
#endif
constexpr int kGemvStages = HM_GEMV_STAGES;  // packed-weight stages in flight per CTA (8832 bytes each)
// CTAs that fit an SM with that many stages plus about 16 KB of activations (shared memory is the limit).
constexpr int kGemvCtasPerSm = kGemvStages == 2 ? 7 : kGemvStages == 3 ? 5 : 4;
constexpr int HM_ABORT_GEMV_STAGE = 40;

// D (16x8, fp32) += A (16x16, row) * B (16x8, col), 16-bit inputs.
template <bool BF16>
HM_DEVICE void mma_m16n8k16(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
  if constexpr (BF16) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

// The pair (K 2t, 2t+1 of its 8-K word) this lane decodes: one shift + lop3, exact subtract, one rounding multiply.
template <bool BF16>
HM_DEVICE uint32_t dequant_pair_u4(uint32_t word, int shift, uint32_t zp_magic2, uint32_t scale2) {
  const uint32_t t = lop3_and_or(word >> shift, 0x000F000Fu, Magic<BF16>::kBase);
  return mul2<BF16>(sub2<BF16>(t, zp_magic2), scale2);
}

// After a CTA has written its partial sums: the last CTA of the tile to arrive (atomic counter, no
// spinning) adds the splits in order and writes the outputs of the tile's 128 rows, thread = row.
template <bool BF16>
HM_DEVICE void gemv_sum_splits(const GemvParams& p, int n_tile, int tid, int* is_last_smem) {
  int& is_last = *is_last_smem;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int old = atomicAdd(p.counters + n_tile, 1);
    is_last = old == p.splits - 1;
    if (is_last) p.counters[n_tile] = 0;  // leave the workspace clean for the next launch
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  const int n = n_tile * 128 + tid;
  const float bias = p.bias != nullptr ? load_bias<BF16>(p.bias, n) : 0.f;
  // Four tokens x eight splits = 32 loads in flight per thread; every sum adds its splits in order.
  for (int tok0 = 0; tok0 < p.M; tok0 += 4) {
    float sum[4] = {0.f, 0.f, 0.f, 0.f};
    for (int s0 = 0; s0 < p.splits; s0 += 8) {
      float v[4][8];
#pragma unroll
      for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int j = 0; j < 8; ++j)
          v[q][j] = (tok0 + q < p.M && s0 + j < p.splits)
                        ? __ldcg(p.partials + (static_cast<size_t>(s0 + j) * p.M + tok0 + q) * p.N + n)
                        : 0.f;
#pragma unroll
      for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int j = 0; j < 8; ++j) sum[q] += v[q][j];
    }
#pragma unroll
    for (int q = 0; q < 4; ++q)
      if (tok0 + q < p.M) store_out<BF16>(p.c, static_cast<size_t>(tok0 + q) * p.ldc + n, sum[q] + bias);
  }
}

// One token (the kernel also handles two): plain fp32 multiply-adds, thread = weight row.  (The warp-level MMA runs at about one
// m16n8k16 per 20 cycles and scheduler on this GPU, so a token tile of 8 that is mostly padding costs more
// than the multiply-adds.)  Same stage ring and the same per-group scale / zero-point fold as the kernel
// below; the codes of a pair are widened to fp32 by one shift / mask each.
// Dynamic shared memory: [kGemvStages][kWStageBytes] weight stages, [MT][kc] fp32 activations,
// [MT][2 * steps] activation sums per 64-K half step.
template <int MT, bool BF16, bool HAS_ZP>
__global__ void __launch_bounds__(kGemvThreads) gemv_fma_w4a16_kernel(const GemvParams p) {
  extern __shared__ __align__(128) uint8_t gemv_smem[];
  __shared__ __align__(8) unsigned long long full_bar[kGemvStages];
  __shared__ __align__(8) unsigned long long empty_bar[kGemvStages];  // one arrival per warp
  __shared__ int is_last;
  __shared__ volatile int abort_flag[2];
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int n_tile = blockIdx.x % p.n_tiles;
  const int split = blockIdx.x / p.n_tiles;
  const int kb0 = split * p.steps_per_cta;
  const int kb1 = min(kb0 + p.steps_per_cta, p.kb_total);
  const int steps = kb1 - kb0;
  const int kc = steps * 128;
  float* xf = reinterpret_cast<float*>(gemv_smem + kGemvStages * kWStageBytes);  // [MT][kc]
  float* xsum = xf + MT * kc;                                                    // [MT][2 * steps]
  const uint32_t stage0 = smem_u32(gemv_smem);

  const uint8_t* codes_src = p.w + (static_cast<size_t>(n_tile) * p.kb_total + kb0) * (2 * kCodeBytes);
  const uint32_t scale_bytes = p.groups_per_step * kScaleBytes;
  const uint32_t zp_bytes = HAS_ZP ? p.groups_per_step * kZpBytes : 0;
  const uint64_t policy = l2_policy_evict_first();
  auto group_of_step = [&](int kb) { return p.groups_per_step == 2 ? 2 * kb : kb / p.steps_per_group; };
  auto issue = [&](int i) {  // step kb0 + i into stage i % kGemvStages
    const int s = i % kGemvStages;
    const uint32_t dst = stage0 + s * kWStageBytes;
    const uint32_t bar = smem_u32(&full_bar[s]);
    const size_t grp = static_cast<size_t>(n_tile) * p.groups + group_of_step(kb0 + i);
    mbar_arrive_expect_tx(bar, 2 * kCodeBytes + scale_bytes + zp_bytes);
    bulk_g2s_hint(dst, codes_src + static_cast<size_t>(i) * (2 * kCodeBytes), 2 * kCodeBytes, bar, policy);
    bulk_g2s(dst + kWScaleOff, p.w_scale + grp * kScaleBytes, scale_bytes, bar);
    if constexpr (HAS_ZP) bulk_g2s(dst + kWZpOff, p.w_zp + grp * kZpBytes, zp_bytes, bar);
  };
  if (tid == 0) {
    for (int s = 0; s < kGemvStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), kGemvThreads / 32);
    }
    abort_flag[0] = 0;
    abort_flag[1] = 0;
    mbar_fence_init();
    fence_proxy_async_smem();
    for (int i = 0; i < kGemvStages && i < steps; ++i) issue(i);
  }
  // The weights are constant, so the requests above may overlap the previous kernel of the stream;
  // activations, workspace and outputs are touched only after it has completed.
  grid_dep_launch();
  grid_dep_wait();

  // Activations of this K range as fp32 (token rows above M are zero), then their sums per half step.
  for (int i = tid; i < MT * (kc / 8); i += kGemvThreads) {
    const int m = i / (kc / 8);
    const int j = (i - m * (kc / 8)) * 8;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (m < p.M) v = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.x) + static_cast<size_t>(m) * p.lda + kb0 * 128 + j);
    const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
    float f[8];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if constexpr (BF16) {
        f[2 * e] = __uint_as_float(w4[e] << 16);
        f[2 * e + 1] = __uint_as_float(w4[e] & 0xFFFF0000u);
      } else {
        const float2 t2 = __half22float2(*reinterpret_cast<const __half2*>(&w4[e]));
        f[2 * e] = t2.x;
        f[2 * e + 1] = t2.y;
      }
    }
    *reinterpret_cast<float4*>(xf + m * kc + j) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(xf + m * kc + j + 4) = make_float4(f[4], f[5], f[6], f[7]);
  }
  __syncthreads();
  for (int i = tid; i < MT * 2 * steps; i += kGemvThreads) {
    const int m = i / (2 * steps);
    const int hs = i - m * (2 * steps);
    const float* src = xf + m * kc + hs * 64;
    float acc = 0.f;
#pragma unroll 8
    for (int j = 0; j < 64; ++j) acc += src[j];
    xsum[i] = acc;
  }
  __syncthreads();

  const int row = tid;
  const int n = n_tile * 128 + row;
  const int zp_shift = (row & 1) * 4;
  const bool half_group = p.groups_per_step == 2;
  constexpr float kBaseValue = BF16 ? 128.f : 1024.f;
  float y[MT], tacc[MT][2], xrun[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) y[m] = tacc[m][0] = tacc[m][1] = xrun[m] = 0.f;
  bool ok = true;

  for (int i = 0; i < steps; ++i) {
    const int s = i % kGemvStages;
    if (!mbar_wait_bounded(smem_u32(&full_bar[s]), (i / kGemvStages) & 1, abort_flag)) {
      if (lane == 0) report_abort(p.status, HM_ABORT_GEMV_STAGE, i, s);
      ok = false;
      break;
    }
    const uint8_t* st = gemv_smem + s * kWStageBytes;
    const float* xk = xf + i * 128;
#pragma unroll
    for (int c = 0; c < 4; ++c) {  // 32-K chunk c of this row at byte c * 2048 + row * 16
      const uint4 wq = *reinterpret_cast<const uint4*>(st + c * 2048 + row * 16);
      const uint32_t words[4] = {wq.x, wq.y, wq.z, wq.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {  // word j: K 8j .. 8j+7, pair i2 = (K 8j + 2 i2, + 1)
        float wf[8];
#pragma unroll
        for (int i2 = 0; i2 < 4; ++i2) {
          const uint32_t pr = lop3_and_or(words[j] >> (4 * i2), 0x000F000Fu, Magic<BF16>::kBase);
          if constexpr (BF16) {
            wf[2 * i2] = __uint_as_float(pr << 16);
            wf[2 * i2 + 1] = __uint_as_float(pr & 0xFFFF0000u);
          } else {
            const float2 t2 = __half22float2(*reinterpret_cast<const __half2*>(&pr));
            wf[2 * i2] = t2.x;
            wf[2 * i2 + 1] = t2.y;
          }
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          const float4 x0 = *reinterpret_cast<const float4*>(xk + m * kc + c * 32 + j * 8);
          const float4 x1 = *reinterpret_cast<const float4*>(xk + m * kc + c * 32 + j * 8 + 4);
          tacc[m][0] = fmaf(wf[0], x0.x, tacc[m][0]);
          tacc[m][1] = fmaf(wf[1], x0.y, tacc[m][1]);
          tacc[m][0] = fmaf(wf[2], x0.z, tacc[m][0]);
          tacc[m][1] = fmaf(wf[3], x0.w, tacc[m][1]);
          tacc[m][0] = fmaf(wf[4], x1.x, tacc[m][0]);
          tacc[m][1] = fmaf(wf[5], x1.y, tacc[m][1]);
          tacc[m][0] = fmaf(wf[6], x1.z, tacc[m][0]);
          tacc[m][1] = fmaf(wf[7], x1.w, tacc[m][1]);
        }
      }
      if (c & 1) {  // end of a 64-K half step
#pragma unroll
        for (int m = 0; m < MT; ++m) xrun[m] += xsum[m * (2 * steps) + 2 * i + (c >> 1)];
        const bool group_end = half_group || ((c == 3) && (((kb0 + i + 1) % p.steps_per_group) == 0 || i + 1 == steps));
        if (group_end) {
          const int gi = half_group ? (c >> 1) : 0;
          const uint32_t s16 = *reinterpret_cast<const uint16_t*>(st + kWScaleOff + gi * kScaleBytes + row * 2);
          float sc;
          if constexpr (BF16) sc = __uint_as_float(s16 << 16);
          else sc = __half2float(__ushort_as_half(static_cast<unsigned short>(s16)));
          uint32_t zp = 8;
          if constexpr (HAS_ZP) zp = (st[kWZpOff + gi * kZpBytes + (row >> 1)] >> zp_shift) & 0xFu;
          const float cz = kBaseValue + static_cast<float>(zp);
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            y[m] = fmaf(sc, fmaf(-cz, xrun[m], tacc[m][0] + tacc[m][1]), y[m]);
            tacc[m][0] = tacc[m][1] = xrun[m] = 0.f;
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&empty_bar[s]));
    if (tid == 0 && i >= 1 && i - 1 + kGemvStages < steps) {
      const int sp = (i - 1) % kGemvStages;
      if (!mbar_wait_bounded(smem_u32(&empty_bar[sp]), ((i - 1) / kGemvStages) & 1, abort_flag)) {
        report_abort(p.status, HM_ABORT_GEMV_STAGE, i, 100 + sp);
      } else {
        issue(i - 1 + kGemvStages);
      }
    }
  }
  if (!ok) {
    // Abort path: nothing may land after the CTA has exited.
    __syncthreads();
    if (tid == 0) {
      for (int i = 0; i < steps; ++i) mbar_wait_bounded(smem_u32(&full_bar[i % kGemvStages]), (i / kGemvStages) & 1, abort_flag + 1);
    }
    __syncthreads();
    return;
  }

  if (p.splits == 1) {
    const float bias = p.bias != nullptr ? load_bias<BF16>(p.bias, n) : 0.f;
#pragma unroll
    for (int m = 0; m < MT; ++m)
      if (m < p.M) store_out<BF16>(p.c, static_cast<size_t>(m) * p.ldc + n, y[m] + bias);
    return;
  }
#pragma unroll
  for (int m = 0; m < MT; ++m)
    if (m < p.M) p.partials[(static_cast<size_t>(split) * p.M + m) * p.N + n] = y[m];
  gemv_sum_splits<BF16>(p, n_tile, tid, &is_last);
}

// NT: token tiles of 8 (1: up to 8 tokens, 2: up to 16).
// Dynamic shared memory: [kGemvStages][kWStageBytes] weight stages, then [8 * NT][kc + pad] activations.
template <int NT, bool BF16, bool HAS_ZP>
__global__ void __launch_bounds__(kGemvThreads) gemv_w4a16_kernel(const GemvParams p) {
  extern __shared__ __align__(128) uint8_t gemv_smem[];
  __shared__ __align__(8) unsigned long long full_bar[kGemvStages];
  __shared__ __align__(8) unsigned long long empty_bar[kGemvStages];  // one arrival per warp
  __shared__ int is_last;
  __shared__ volatile int abort_flag[2];
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n_tile = blockIdx.x % p.n_tiles;  // neighbouring CTAs share the activation chunk
  const int split = blockIdx.x / p.n_tiles;
  const int kb0 = split * p.steps_per_cta;
  const int kb1 = min(kb0 + p.steps_per_cta, p.kb_total);
  const int steps = kb1 - kb0;
  const int kc = steps * 128;
  const int pitch = kc + kGemvXPad;
  uint16_t* xs = reinterpret_cast<uint16_t*>(gemv_smem + kGemvStages * kWStageBytes);
  const uint32_t stage0 = smem_u32(gemv_smem);

  // ---- producer state (thread 0): sources of step kb, as in the tensor-memory kernel's producers
  const uint8_t* codes_src = p.w + (static_cast<size_t>(n_tile) * p.kb_total + kb0) * (2 * kCodeBytes);
  const uint32_t scale_bytes = p.groups_per_step * kScaleBytes;
  const uint32_t zp_bytes = HAS_ZP ? p.groups_per_step * kZpBytes : 0;
  const uint64_t policy = l2_policy_evict_first();
  auto group_of_step = [&](int kb) { return p.groups_per_step == 2 ? 2 * kb : kb / p.steps_per_group; };
  auto issue = [&](int i) {  // step kb0 + i into stage i % kGemvStages
    const int s = i % kGemvStages;
    const uint32_t dst = stage0 + s * kWStageBytes;
    const uint32_t bar = smem_u32(&full_bar[s]);
    const size_t grp = static_cast<size_t>(n_tile) * p.groups + group_of_step(kb0 + i);
    mbar_arrive_expect_tx(bar, 2 * kCodeBytes + scale_bytes + zp_bytes);
    bulk_g2s_hint(dst, codes_src + static_cast<size_t>(i) * (2 * kCodeBytes), 2 * kCodeBytes, bar, policy);
    bulk_g2s(dst + kWScaleOff, p.w_scale + grp * kScaleBytes, scale_bytes, bar);
    if constexpr (HAS_ZP) bulk_g2s(dst + kWZpOff, p.w_zp + grp * kZpBytes, zp_bytes, bar);
  };
  if (tid == 0) {
    for (int s = 0; s < kGemvStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), kGemvThreads / 32);
    }
    abort_flag[0] = 0;
    abort_flag[1] = 0;
    mbar_fence_init();
    fence_proxy_async_smem();
    // The first stages are requested before anything else: their latency overlaps the activation staging.
    for (int i = 0; i < kGemvStages && i < steps; ++i) issue(i);
  }
  // The weights are constant, so the requests above may overlap the previous kernel of the stream;
  // activations, workspace and outputs are touched only after it has completed.
  grid_dep_launch();
  grid_dep_wait();

  // Activations of this K range, 8 values per 16-byte copy; token rows above M are zero.
  for (int i = tid; i < 8 * NT * (kc / 8); i += kGemvThreads) {
    const int m = i / (kc / 8);
    const int j = (i - m * (kc / 8)) * 8;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (m < p.M) v = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.x) + static_cast<size_t>(m) * p.lda + kb0 * 128 + j);
    *reinterpret_cast<uint4*>(xs + m * pitch + j) = v;
  }
  __syncthreads();

  // Sum of the activations of every (token row, 64-K half step): the zero point and the magic
  // offset of the codes are taken out of the inner loop, see below.
  float* xsum = reinterpret_cast<float*>(xs + 8 * NT * pitch);  // [8 * NT][2 * steps]
  for (int i = tid; i < 8 * NT * 2 * steps; i += kGemvThreads) {
    const int m = i / (2 * steps);
    const int hs = i - m * (2 * steps);
    const uint32_t* src = reinterpret_cast<const uint32_t*>(xs + m * pitch + hs * 64);
    float acc = 0.f;
#pragma unroll 8
    for (int j = 0; j < 32; ++j) {
      const uint32_t v = src[j];
      if constexpr (BF16) {
        acc += __uint_as_float(v << 16) + __uint_as_float(v & 0xFFFF0000u);
      } else {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&v));
        acc += f.x + f.y;
      }
    }
    xsum[i] = acc;
  }
  __syncthreads();

  const int wrow = warp * 32 + g;            // this lane's first weight row inside the tile (+ 8, 16, 24)
  const int row0 = n_tile * 128 + wrow;
  const int zp_shift = (wrow & 1) * 4;       // rows g + 8k have the parity of g
  const bool half_group = p.groups_per_step == 2;  // a scale group per 64-K half step

  // The inner loop multiplies the raw codes: lop3 places code q of a pair in the mantissa of the
  // 16-bit constant `base` (128 for bf16, 1024 for fp16), which reads as base + q exactly, and the
  // MMA accumulates sum_k (base + q_k) * x_k in fp32 for the K range of one scale group (`tacc`).
  // At the end of the group   y += s * (tacc - (base + zp) * sum_k x_k)   = s * sum_k (q_k - zp) * x_k,
  // the same product as with weights decoded one by one, up to fp32 rounding (the decoded weights
  // themselves are never rounded to 16 bits here).  One shift and one lop3 per weight pair.
  float y[2][NT][4];     // [m16 block][token tile][element]
  float tacc[2][2][NT][4];  // two sets (even / odd k16 blocks) halve the dependent MMA chains
#pragma unroll
  for (int mb = 0; mb < 2; ++mb)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        y[mb][nt][e] = 0.f;
        tacc[0][mb][nt][e] = 0.f;
        tacc[1][mb][nt][e] = 0.f;
      }
  float xrun[NT][2];     // sum of x over the current group for tokens 8 nt + 2t, 2t + 1
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) xrun[nt][0] = xrun[nt][1] = 0.f;
  constexpr float kBaseValue = BF16 ? 128.f : 1024.f;

  const int shift = 4 * t;
  // B fragment of a k16 block: tokens g (+8 for the second tile), K = 2t, 2t+1 and + 8 inside the block.
  const uint16_t* xb = xs + g * pitch + 2 * t;
  bool ok = true;

  // Folds the finished group into y and clears the group accumulators.  `st`: the stage holding the
  // group's scales / zero points, `gi`: its index inside the stage (0, or 1 for the second half step).
  auto fold_group = [&](const uint8_t* st, int gi) {
#pragma unroll
    for (int rb = 0; rb < 4; ++rb) {  // row block rb: rows g + 8 rb = element pair (e >> 1) of m16 block rb >> 1
      const uint32_t s16 = *reinterpret_cast<const uint16_t*>(st + kWScaleOff + gi * kScaleBytes + (wrow + 8 * rb) * 2);
      float sc;
      if constexpr (BF16) sc = __uint_as_float(s16 << 16);
      else sc = __half2float(__ushort_as_half(static_cast<unsigned short>(s16)));
      uint32_t zp = 8;
      if constexpr (HAS_ZP) zp = (st[kWZpOff + gi * kZpBytes + ((wrow + 8 * rb) >> 1)] >> zp_shift) & 0xFu;
      const float cz = kBaseValue + static_cast<float>(zp);
      const int mb = rb >> 1, eh = (rb & 1) * 2;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int el = 0; el < 2; ++el) {
          const float tsum = tacc[0][mb][nt][eh + el] + tacc[1][mb][nt][eh + el];
          y[mb][nt][eh + el] = fmaf(sc, fmaf(-cz, xrun[nt][el], tsum), y[mb][nt][eh + el]);
          tacc[0][mb][nt][eh + el] = 0.f;
          tacc[1][mb][nt][eh + el] = 0.f;
        }
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) xrun[nt][0] = xrun[nt][1] = 0.f;
  };

  for (int i = 0; i < steps; ++i) {
    const int s = i % kGemvStages;
    if (!mbar_wait_bounded(smem_u32(&full_bar[s]), (i / kGemvStages) & 1, abort_flag)) {
      if (lane == 0) report_abort(p.status, HM_ABORT_GEMV_STAGE, i, s);
      ok = false;
      break;
    }
    const uint8_t* st = gemv_smem + s * kWStageBytes;
    const uint16_t* xk = xb + i * 128;
#pragma unroll
    for (int c = 0; c < 4; ++c) {  // 32-K chunk c of row r at byte c * 2048 + r * 16
      uint4 wq[4];
#pragma unroll
      for (int rb = 0; rb < 4; ++rb) wq[rb] = *reinterpret_cast<const uint4*>(st + c * 2048 + (wrow + 8 * rb) * 16);
#pragma unroll
      for (int b = 0; b < 2; ++b) {  // two k16 blocks per chunk: words 2b and 2b+1
        uint32_t bf[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          bf[nt][0] = *reinterpret_cast<const uint32_t*>(xk + nt * 8 * pitch + c * 32 + b * 16);
          bf[nt][1] = *reinterpret_cast<const uint32_t*>(xk + nt * 8 * pitch + c * 32 + b * 16 + 8);
        }
#pragma unroll
        for (int mb = 0; mb < 2; ++mb) {  // rows g, g+8 of m16 block mb = row blocks 2mb, 2mb+1
          const uint4& lo = wq[2 * mb];
          const uint4& hi = wq[2 * mb + 1];
          const uint32_t w_lo0 = b == 0 ? lo.x : lo.z, w_lo1 = b == 0 ? lo.y : lo.w;
          const uint32_t w_hi0 = b == 0 ? hi.x : hi.z, w_hi1 = b == 0 ? hi.y : hi.w;
          uint32_t a[4];
          a[0] = lop3_and_or(w_lo0 >> shift, 0x000F000Fu, Magic<BF16>::kBase);  // row g,   K 2t..
          a[1] = lop3_and_or(w_hi0 >> shift, 0x000F000Fu, Magic<BF16>::kBase);  // row g+8, K 2t..
          a[2] = lop3_and_or(w_lo1 >> shift, 0x000F000Fu, Magic<BF16>::kBase);  // row g,   K 8+2t..
          a[3] = lop3_and_or(w_hi1 >> shift, 0x000F000Fu, Magic<BF16>::kBase);  // row g+8, K 8+2t..
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) mma_m16n8k16<BF16>(tacc[b][mb][nt], a, bf[nt][0], bf[nt][1]);
        }
      }
      if (c & 1) {  // end of a 64-K half step
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          xrun[nt][0] += xsum[(8 * nt + 2 * t) * (2 * steps) + 2 * i + (c >> 1)];
          xrun[nt][1] += xsum[(8 * nt + 2 * t + 1) * (2 * steps) + 2 * i + (c >> 1)];
        }
        // The group ends here if groups are 64 K wide, or at the last half of the group's last
        // step, or with the CTA's K range (the rest of the group belongs to other CTAs).
        const bool group_end = half_group || ((c == 3) && (((kb0 + i + 1) % p.steps_per_group) == 0 || i + 1 == steps));
        if (group_end) fold_group(st, half_group ? (c >> 1) : 0);
      }
    }
    // This warp is done with stage s.  The stage of the step before is refilled one step late, so
    // that the producer thread rarely has to wait for the other warps.
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&empty_bar[s]));
    if (tid == 0 && i >= 1 && i - 1 + kGemvStages < steps) {
      const int sp = (i - 1) % kGemvStages;
      if (!mbar_wait_bounded(smem_u32(&empty_bar[sp]), ((i - 1) / kGemvStages) & 1, abort_flag)) {
        report_abort(p.status, HM_ABORT_GEMV_STAGE, i, 100 + sp);
      } else {
        issue(i - 1 + kGemvStages);
      }
    }
  }
  if (!ok) {
    // Abort path: nothing may land after the CTA has exited.  Stages of steps >= i are in flight at most.
    __syncthreads();
    if (tid == 0) {
      for (int i = 0; i < steps; ++i) mbar_wait_bounded(smem_u32(&full_bar[i % kGemvStages]), (i / kGemvStages) & 1, abort_flag + 1);
    }
    __syncthreads();
    return;
  }

  auto& acc = y;

  // Accumulator element e of (mb, nt): row 16*mb + g + 8*(e >> 1), token 8*nt + 2t + (e & 1).
  if (p.splits == 1) {
#pragma unroll
    for (int mb = 0; mb < 2; ++mb)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int n = row0 + 16 * mb + 8 * (e >> 1);
        const float bias = p.bias != nullptr ? load_bias<BF16>(p.bias, n) : 0.f;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const int tok = 8 * nt + 2 * t + (e & 1);
          if (tok < p.M) store_out<BF16>(p.c, static_cast<size_t>(tok) * p.ldc + n, acc[mb][nt][e] + bias);
        }
      }
    return;
  }
#pragma unroll
  for (int mb = 0; mb < 2; ++mb)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int n = row0 + 16 * mb + 8 * (e >> 1);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int tok = 8 * nt + 2 * t + (e & 1);
        if (tok < p.M) p.partials[(static_cast<size_t>(split) * p.M + tok) * p.N + n] = acc[mb][nt][e];
      }
    }
  gemv_sum_splits<BF16>(p, n_tile, tid, &is_last);
}

}  // namespace hm
