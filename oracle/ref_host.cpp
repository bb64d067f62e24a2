// Test infrastructure, not product code.
//
// Runs two of the reference's own CUDA helper kernels on the host CPU so the
// numpy oracle can be pinned against the reference's code instead of a reading
// of it: pack_weight_kernel / unpack_weight_kernel
// (humming/include/humming/kernel/pack_weight.cuh) and dequant_unpacked_fp_type
// (humming/include/humming/kernel/dequant_weight.cuh).  Neither uses shared
// memory, warp shuffles or barriers, so executing the kernel body once per
// (blockIdx, threadIdx) in a loop reproduces the device result exactly.
//
// The reference headers are included from where they lie (the include path is
// given by oracle/build_ref.sh); nothing is copied.  CUDA qualifiers and the
// built-in index variables are defined away below.
#include <cstdint>
#include <cstring>

struct hm_dim3 { unsigned x, y, z; };
static thread_local hm_dim3 threadIdx, blockIdx, blockDim, gridDim;

#define __device__
#define __global__
#define __host__
#define __forceinline__ inline
#define __cvta_generic_to_shared(p) (reinterpret_cast<uintptr_t>(p))
struct uint2 { unsigned x, y; };
struct uint4 { unsigned x, y, z, w; };

#include <humming/kernel/dequant_weight.cuh>
#include <humming/kernel/pack_weight.cuh>

template <uint32_t B>
static void run_pack(const uint32_t* in, uint32_t* out, unsigned blocks) {
  blockDim = {32, 1, 1};
  for (unsigned b = 0; b < blocks; ++b)
    for (unsigned t = 0; t < 32; ++t) {
      blockIdx = {b, 0, 0};
      threadIdx = {t, 0, 0};
      pack_weight_kernel<B>(in, out);
    }
}
template <uint32_t B>
static void run_unpack(const uint32_t* in, uint32_t* out, unsigned blocks) {
  blockDim = {32, 1, 1};
  for (unsigned b = 0; b < blocks; ++b)
    for (unsigned t = 0; t < 32; ++t) {
      blockIdx = {b, 0, 0};
      threadIdx = {t, 0, 0};
      unpack_weight_kernel<B>(in, out);
    }
}

#define FOR_BITS(F, ...)                 \
  switch (bits) {                        \
    case 1: F<1>(__VA_ARGS__); break;    \
    case 2: F<2>(__VA_ARGS__); break;    \
    case 3: F<3>(__VA_ARGS__); break;    \
    case 4: F<4>(__VA_ARGS__); break;    \
    case 5: F<5>(__VA_ARGS__); break;    \
    case 6: F<6>(__VA_ARGS__); break;    \
    case 7: F<7>(__VA_ARGS__); break;    \
    case 8: F<8>(__VA_ARGS__); break;    \
    default: return -1;                  \
  }

extern "C" {
// numel codes (multiple of 1024, the kernel's block granularity) -> numel*bits/32 words
int ref_pack_weight(const uint32_t* codes, uint32_t* packed, long numel, int bits) {
  if (numel % 1024) return -2;
  FOR_BITS(run_pack, codes, packed, static_cast<unsigned>(numel / 1024));
  return 0;
}
int ref_unpack_weight(const uint32_t* packed, uint32_t* codes, long numel, int bits) {
  if (numel % 1024) return -2;
  FOR_BITS(run_unpack, packed, codes, static_cast<unsigned>(numel / 1024));
  return 0;
}
int ref_dequant_fp(const uint32_t* codes, float* out, long numel, int exponent_bits, int mantissa_bits, int is_signed) {
  blockDim = {32, 1, 1};
  const unsigned blocks = static_cast<unsigned>((numel + 1023) / 1024);
  for (unsigned b = 0; b < blocks; ++b)
    for (unsigned t = 0; t < 32; ++t) {
      blockIdx = {b, 0, 0};
      threadIdx = {t, 0, 0};
      dequant_unpacked_fp_type(const_cast<uint32_t*>(codes), reinterpret_cast<uint32_t*>(out),
                               static_cast<uint32_t>(numel), exponent_bits, mantissa_bits, is_signed != 0);
    }
  return 0;
}
}
