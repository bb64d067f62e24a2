// Test infrastructure, not product code.
//
// Runs the reference's register-level dequantization of 16-bit-activation GEMMs on the host CPU:
// dequant_single<UIntN, Float16 | BFloat16, zero point?> and dequant_single_zero_point
// (humming/include/humming/datatype/dequant_single.cuh), followed by the multiplication with the group scale in
// the same 16-bit type that the main loop applies (humming/include/humming/arith/mainloop_arith.cuh:117-161,
// __hmul2), so that the oracle's effective 16-bit weight, rn16(fp32(q - zp) * fp32(s)), can be pinned against the
// reference's own code.  The header is included from where it lies (include path given by oracle/build_ref.sh);
// its one inline-PTX helper, lop3_and_or (humming/include/humming/utils/ptx/logic.cuh: (a & b) | c as one lop3
// instruction), is supplied here in plain C++, and the half-precision subtract / multiply are CUDA's own host
// implementations from cuda_fp16.h / cuda_bf16.h.
#include <cstdint>
#include <cstring>
#include <type_traits>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

static inline uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) { return (a & b) | c; }

#include <humming/datatype/dequant_single.cuh>

template <class Source, class Target, bool ZP>
static void run(const uint32_t* q, const uint32_t* zp, const uint16_t* scale, uint16_t* out, long pairs) {
  using scalar_t2 = typename F16Conversion<Target>::scalar_t2;
  for (long i = 0; i < pairs; ++i) {
    // two codes per 32-bit word, one per 16-bit lane, as the fragment layout presents them to dequant_single
    uint32_t val = (q[2 * i] & 0xFFFFu) | (q[2 * i + 1] << 16);
    uint32_t zp_val = 0;
    if (ZP) {
      // the zero point of a group is broadcast to both lanes (dequant_single_zero_point multiplies by 0x00010001);
      // here the two weights may come from different groups, so each lane is expanded on its own
      uint32_t z0 = zp[2 * i], z1 = zp[2 * i + 1];
      uint32_t lo = dequant_single_zero_point<Source, Target>(z0) & 0xFFFFu;
      uint32_t hi = dequant_single_zero_point<Source, Target>(z1) & 0xFFFF0000u;
      zp_val = lo | hi;
    }
    uint32_t w = dequant_single<Source, Target, ZP>(val, zp_val);
    uint32_t s = static_cast<uint32_t>(scale[2 * i]) | (static_cast<uint32_t>(scale[2 * i + 1]) << 16);
    scalar_t2 w2, s2;
    std::memcpy(&w2, &w, 4);
    std::memcpy(&s2, &s, 4);
    scalar_t2 r = __hmul2(w2, s2);
    uint32_t bits;
    std::memcpy(&bits, &r, 4);
    out[2 * i] = static_cast<uint16_t>(bits & 0xFFFFu);
    out[2 * i + 1] = static_cast<uint16_t>(bits >> 16);
  }
}

extern "C" {
// numel (even) codes of `bits` bits, zero points (ignored without has_zp) and 16-bit scale patterns, one per
// weight -> the 16-bit pattern of the weight the tensor cores multiply by.
int ref_dequant_mul_16(const uint32_t* q, const uint32_t* zp, const uint16_t* scale, uint16_t* out, long numel, int bits,
                       int is_bf16, int has_zp) {
  if (numel % 2) return -2;
#define CASE(B, S)                                                                        \
  if (bits == B) {                                                                        \
    if (is_bf16 && has_zp) run<S, BFloat16, true>(q, zp, scale, out, numel / 2);          \
    else if (is_bf16) run<S, BFloat16, false>(q, zp, scale, out, numel / 2);              \
    else if (has_zp) run<S, Float16, true>(q, zp, scale, out, numel / 2);                 \
    else run<S, Float16, false>(q, zp, scale, out, numel / 2);                            \
    return 0;                                                                             \
  }
  CASE(4, UInt4) CASE(2, UInt2) CASE(3, UInt3) CASE(5, UInt5) CASE(6, UInt6)
#undef CASE
  return -1;
}
}
