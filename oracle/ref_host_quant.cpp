// Test infrastructure, not product code.
//
// Runs the reference's weight quantizer kernel, quant_weight
// (humming/include/humming/kernel/quant_weight.cuh), on the host CPU so that the
// numpy oracle's quantize_weight_int can be pinned against the reference's code.
// Unlike the pack / decode kernels of ref_host.cpp this kernel is cooperative: one
// warp per quantization group, a warp-shuffle reduction, a __shared__ pair and a
// __syncthreads().  It is therefore executed by 32 host threads, one per lane, that
// meet at a barrier wherever the device code synchronises:
//   __shfl_down_sync  -> every lane publishes its value, barrier, reads lane + offset
//                        (its own value when that lane does not exist), barrier
//   __syncthreads     -> barrier
//   __shared__        -> one static object (blocks run one after another)
// The reference header is included from where it lies (include path given by
// oracle/build_ref.sh); nothing is copied.
#include <algorithm>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <thread>
#include <vector>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

namespace {
class Barrier {
 public:
  explicit Barrier(int n) : n_(n) {}
  void wait() {
    std::unique_lock<std::mutex> lock(m_);
    const unsigned gen = gen_;
    if (++count_ == n_) {
      count_ = 0;
      ++gen_;
      cv_.notify_all();
    } else {
      cv_.wait(lock, [&] { return gen != gen_; });
    }
  }

 private:
  std::mutex m_;
  std::condition_variable cv_;
  int n_, count_ = 0;
  unsigned gen_ = 0;
};
Barrier g_barrier(32);
float g_lane_vals[32];
}  // namespace

struct hm_dim3 { unsigned x, y, z; };
static thread_local hm_dim3 threadIdx, blockIdx, blockDim, gridDim;

static inline float __shfl_down_sync(unsigned, float v, int offset) {
  const unsigned lane = threadIdx.x;
  g_lane_vals[lane] = v;
  g_barrier.wait();
  const float got = lane + offset < 32 ? g_lane_vals[lane + offset] : v;
  g_barrier.wait();
  return got;
}
static inline void __syncthreads() { g_barrier.wait(); }
static inline int __float2int_rn(float v) { return static_cast<int>(std::nearbyintf(v)); }  // default mode: to nearest even
using std::max;

#undef __shared__
#define __shared__ static
#undef __global__
#define __global__

#include <humming/kernel/quant_weight.cuh>

template <class Target, uint32_t G, bool ZP>
static void run_quant(const float* in, int32_t* out, float* scales, uint32_t* zps, unsigned groups) {
  // 32 lanes, each walking over all blocks; every lane passes the same barriers in every block, so the
  // lanes stay in the same block (the static __shared__ pair is reused only after the block's last barrier:
  // its next write comes after the next block's shuffles, which are barriers too).
  std::vector<std::thread> lanes;
  for (unsigned t = 0; t < 32; ++t)
    lanes.emplace_back([=] {
      blockDim = {32, 1, 1};
      gridDim = {groups, 1, 1};
      threadIdx = {t, 0, 0};
      for (unsigned b = 0; b < groups; ++b) {
        blockIdx = {b, 0, 0};
        quant_weight<Float32, Target, G, true, false, ZP>(
            reinterpret_cast<uint4*>(const_cast<float*>(in)), reinterpret_cast<uint4*>(out),
            reinterpret_cast<uint32_t*>(scales), zps);
      }
    });
  for (auto& th : lanes) th.join();
}

extern "C" {
// fp32 weights (groups * group_size values, group_size in {32, 128}) -> int32 codes, one fp32 scale per group and,
// with has_zp, one zero point per group.  bits/is_signed: uint4, int4, uint8 or int8 targets.
int ref_quant_weight_f32(const float* in, int32_t* out, float* scales, uint32_t* zps, long groups, int group_size,
                         int bits, int is_signed, int has_zp) {
  const unsigned g = static_cast<unsigned>(groups);
#define CASE(T, B, S, G, Z)                                                         \
  if (bits == B && is_signed == S && group_size == G && has_zp == Z) {              \
    run_quant<T, G, Z != 0>(in, out, scales, zps, g);                               \
    return 0;                                                                       \
  }
  CASE(UInt4, 4, 0, 128, 0) CASE(UInt4, 4, 0, 128, 1) CASE(UInt4, 4, 0, 32, 0) CASE(UInt4, 4, 0, 32, 1)
  CASE(Int4, 4, 1, 128, 0) CASE(UInt8, 8, 0, 128, 0) CASE(UInt8, 8, 0, 128, 1) CASE(Int8, 8, 1, 128, 0)
#undef CASE
  return -1;
}
}
