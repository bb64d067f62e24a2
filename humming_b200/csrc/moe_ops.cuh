// Element-wise / per-token kernels around the two MoE GEMMs.  The reference
// stops at the GEMMs (routing, SiLU*mul and the sum over top-k are the
// caller's); the benchmark's MoE layer is route -> align -> up GEMM ->
// silu(gate)*up -> down GEMM (x routing weight) -> sum over top-k.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ptx.cuh"

namespace hm {

template <typename T>
__device__ __forceinline__ float ld_as_float(const T* p);
template <>
__device__ __forceinline__ float ld_as_float<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <>
__device__ __forceinline__ float ld_as_float<__half>(const __half* p) { return __half2float(*p); }
template <>
__device__ __forceinline__ float ld_as_float<float>(const float* p) { return *p; }
template <typename T>
__device__ __forceinline__ void st_from_float(T* p, float v);
template <>
__device__ __forceinline__ void st_from_float<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ void st_from_float<__half>(__half* p, float v) { *p = __float2half_rn(v); }

// One warp per token: softmax over the experts' logits (optional), top-k by
// repeated arg-max (ties -> lowest expert id), optional renormalisation of the
// k weights to sum 1.  logits fp32 [tokens, experts], experts <= 1024.
__global__ void moe_route_kernel(const float* __restrict__ logits, int tokens, int experts, int top_k, int use_softmax,
                                 int renormalize, int* __restrict__ topk_ids, float* __restrict__ topk_weights) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= tokens) return;
  const float* row = logits + static_cast<size_t>(warp) * experts;
  constexpr int kMaxPerLane = 32;  // experts <= 1024
  float v[kMaxPerLane];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int e = i * 32 + lane;
    v[i] = e < experts ? row[e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (use_softmax) {
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      v[i] = (i * 32 + lane) < experts ? __expf(v[i] - mx) : -INFINITY;
      if ((i * 32 + lane) < experts) sum += v[i];
    }
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.f / sum;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i)
      if ((i * 32 + lane) < experts) v[i] *= inv;
  }
  float wsum = 0.f;
  float my_w = 0.f;
  int my_id = 0;
  for (int k = 0; k < top_k; ++k) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      const int e = i * 32 + lane;
      if (e < experts && (v[i] > best)) {
        best = v[i];
        best_e = e;
      }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_e = oe;
      }
    }
    if ((best_e & 31) == lane) {
#pragma unroll
      for (int i = 0; i < kMaxPerLane; ++i)
        if (i == (best_e >> 5)) v[i] = -INFINITY;
    }
    wsum += best;
    if (lane == k) {
      my_w = best;
      my_id = best_e;
    }
  }
  if (lane < top_k) {
    topk_ids[static_cast<size_t>(warp) * top_k + lane] = my_id;
    topk_weights[static_cast<size_t>(warp) * top_k + lane] = renormalize ? my_w / wsum : my_w;
  }
}

// out[r, j] = silu(x[r, j]) * x[r, inter + j], x is [rows, 2*inter] = [gate | up].
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t rows, int inter) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= rows * inter) return;
  const int64_t r = i / inter;
  const int j = static_cast<int>(i - r * inter);
  const float g = ld_as_float<T>(x + r * 2 * inter + j);
  const float u = ld_as_float<T>(x + r * 2 * inter + inter + j);
  st_from_float<T>(out + i, g / (1.f + __expf(-g)) * u);
}

// out[t, j] = sum_k x[t, k, j]   (fp32 accumulation)
template <typename T>
__global__ void topk_sum_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t tokens, int top_k, int width) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= tokens * width) return;
  const int64_t t = i / width;
  const int j = static_cast<int>(i - t * width);
  float acc = 0.f;
  for (int k = 0; k < top_k; ++k) acc += ld_as_float<T>(x + (t * top_k + k) * width + j);
  st_from_float<T>(out + i, acc);
}

}  // namespace hm
