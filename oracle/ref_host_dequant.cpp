// Test infrastructure, not product code.
//
// Runs the reference's register-level dequantization on the host CPU.  16-bit activations:
// dequant_single<UIntN, Float16 | BFloat16, zero point?> and dequant_single_zero_point
// (humming/include/humming/datatype/dequant_single.cuh), followed by the multiplication with the group scale in
// the same 16-bit type that the main loop applies (humming/include/humming/arith/mainloop_arith.cuh:117-161,
// __hmul2), so that the oracle's effective 16-bit weight, rn16(fp32(q - zp) * fp32(s)), can be pinned against the
// reference's own code.  FP8 activations: dequant_single<Float4E2M1 | UInt4, Float8E4M3> (codes to e4m3 bit
// patterns that are the weight times a fixed power of two) with get_dtype_dequant_exp_offset.  The header is included from where it lies (include path given by oracle/build_ref.sh);
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

#include <humming/arith/exp_offset.cuh>
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

// FP8-activation paths: codes -> e4m3 bit patterns, four 8-bit lanes per word.
template <int KIND>
static uint32_t to_e4m3_word(uint32_t lanes, uint32_t zp) {
  if constexpr (KIND == 0) return dequant_single<Float4E2M1, Float8E4M3, false>(lanes << 4, zp);  // code in the high nibble
  if constexpr (KIND == 1) return dequant_single<UInt4, Float8E4M3, false>(lanes, zp);
  return dequant_single<UInt4, Float8E4M3, true>(lanes, zp);
}

extern "C" {
// kind 0: float4e2m1 codes; kind 1: uint4 codes, fixed zero point 8; kind 2: uint4 codes with a dynamic zero
// point (one per call: the four lanes of a word share it, as the lanes of a fragment word share their group).
// Integer codes are first rewritten the way the reference's repack kernel stores them for these paths
// (humming/include/humming/kernel/process.cuh:207-219): v >= zp ? v - zp : 15 - v.
// out: one e4m3 byte per code.  Returns the power-of-two exponent the reference folds back afterwards
// (get_dtype_dequant_exp_offset, humming/include/humming/arith/exp_offset.cuh:8-36), or a negative error.
int ref_dequant_to_e4m3(const uint32_t* q, uint32_t zp, uint8_t* out, long numel, int kind) {
  if (numel % 4 || kind < 0 || kind > 2) return -2;
  for (long i = 0; i < numel; i += 4) {
    uint32_t lanes = 0;
    for (int l = 0; l < 4; ++l) {
      uint32_t v = q[i + l] & 15u;
      if (kind != 0) {
        const uint32_t z = kind == 1 ? 8u : zp;
        v = v >= z ? v - z : 15u - v;
      }
      lanes |= v << (8 * l);
    }
    uint32_t w = kind == 0 ? to_e4m3_word<0>(lanes, zp) : (kind == 1 ? to_e4m3_word<1>(lanes, zp) : to_e4m3_word<2>(lanes, zp));
    for (int l = 0; l < 4; ++l) out[i + l] = static_cast<uint8_t>(w >> (8 * l));
  }
  if (kind == 0) return static_cast<int>(get_dtype_dequant_exp_offset<Float8E4M3, Float4E2M1>());
  if (kind == 1) return static_cast<int>(get_dtype_dequant_exp_offset<Float8E4M3, UInt4, false>());
  return static_cast<int>(get_dtype_dequant_exp_offset<Float8E4M3, UInt4, true>());
}

// fp32 -> e4m3 with round-to-nearest-even and saturation to +-448, by CUDA's own host implementation of the
// conversion (cuda_fp8.h, __nv_cvt_float_to_fp8): the instruction the reference's Triton quantizer compiles to
// (tensor.to(tl.float8e4nv), humming/kernel/quant_input.py:36-37).  Checks the cast the oracle uses.
int cuda_float_to_e4m3(const float* x, uint8_t* out, long numel) {
  for (long i = 0; i < numel; ++i) out[i] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(x[i], __NV_SATFINITE, __NV_E4M3));
  return 0;
}

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
