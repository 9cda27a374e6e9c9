// Device helpers shared by the tcgen05 quantizer kernels: operand formats, two-wide arithmetic in the activation
// dtype, nibble packing.
#pragma once

#include "qo_internal.cuh"
#include "sm100_ptx.cuh"

namespace qo {
namespace fq {

constexpr int kAtomBytes = 128 * 128;  // 128 rows of one 128-byte swizzle atom
enum Mode { kInt8 = 0, kPacked = 1, kTransform = 2 };

template <typename T> struct Fmt;
template <> struct Fmt<__half> { static constexpr uint32_t id = 0; };
template <> struct Fmt<__nv_bfloat16> { static constexpr uint32_t id = 1; };

template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Two-wide arithmetic in the activation dtype, used by the quantize pass.  Everything here runs on the ALU / FMA
// pipes (packed converts, packed min / max / add); none of it touches the conversion unit.
//   cvt(lo, hi)      two float32 -> packed pair, round to nearest even
//   lo(p), hi(p)     packed pair -> float32
//   nibbles(q)       clamp both halves to [-8, 7], then add the constant whose spacing is 1 (200 for bf16, 1032 for
//                    fp16): the sum is rint(q) + 8 with ties to even, and it sits in the low 4 bits of each half
//   quot(z0, z1)     round(z / s) for both; bf16 multiplies by 1/s (exact, see the file comment), fp16 refines the
//                    product with two FMAs, which gives the correctly rounded quotient (Markstein)
template <typename T> struct P2;
template <> struct P2<__nv_bfloat16> {
  // |result| = max(|a|, |b|) per half (the sign is the xor of the signs and is ignored by the caller)
  static __device__ __forceinline__ uint32_t absmax(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
  }
  static constexpr uint32_t kByteMask = 0x0F0F0F0Fu;  // the nibble's byte also carries exponent bits
  static __device__ __forceinline__ uint32_t cvt(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
  }
  static __device__ __forceinline__ float lo(uint32_t p) { return __uint_as_float(p << 16); }
  static __device__ __forceinline__ float hi(uint32_t p) { return __uint_as_float(p & 0xFFFF0000u); }
  static __device__ __forceinline__ uint32_t nibbles(uint32_t q) {
    uint32_t d;
    asm("{\n\t.reg .b32 t;\n\t"
        "max.bf16x2 t, %1, %2;\n\t"
        "min.bf16x2 t, t, %3;\n\t"
        "add.rn.bf16x2 %0, t, %4;\n\t}"
        : "=r"(d) : "r"(q), "r"(0xC100C100u), "r"(0x40E040E0u), "r"(0x43484348u));
    return d;
  }
  static __device__ __forceinline__ uint32_t quot(float z0, float z1, float, float inv_s) { return cvt(z0 * inv_s, z1 * inv_s); }
  // 1/s as two bf16 terms (both halves of a word hold the same term): hi = round(1/s), lo = round(1/s - hi)
  static __device__ __forceinline__ void recip2(float inv_s, uint32_t& hi2, uint32_t& lo2) {
    hi2 = cvt(inv_s, inv_s);
    const float rest = inv_s - lo(hi2);  // exact in float32
    lo2 = cvt(rest, rest);
  }
  // round(z / s) for a packed pair with two packed instructions: fma(z, hi, round(z * lo)).  The inner rounding
  // error and the error of hi + lo together stay below the distance from z / s to the nearest rounding boundary of
  // the format; checked exhaustively over all 128 x 128 significand pairs of z and s (both signs), which covers
  // every normal operand because the computation is invariant under scaling by powers of two.
  static __device__ __forceinline__ uint32_t quotp(uint32_t zz, float, float, uint32_t hi2, uint32_t lo2) {
    uint32_t t, d;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(t) : "r"(zz), "r"(lo2));
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(zz), "r"(hi2), "r"(t));
    return d;
  }
  // nibbles() without the clamp, for rows whose quotients cannot leave (-7.5, 7.5)
  static __device__ __forceinline__ uint32_t nibbles_inrange(uint32_t q) {
    uint32_t d;
    asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(q), "r"(0x43484348u));
    return d;
  }
  static constexpr uint32_t kFold = 0x44u;  // see fold_pair
  static constexpr uint32_t kHalfBits = 0x4340u;  // a half out of nibbles() is kHalfBits + nibble (see fold_quad)
};
template <> struct P2<__half> {
  static __device__ __forceinline__ uint32_t absmax(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("max.xorsign.abs.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
  }
  static constexpr uint32_t kByteMask = 0xFFFFFFFFu;
  static __device__ __forceinline__ uint32_t cvt(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
  }
  static __device__ __forceinline__ float lo(uint32_t p) { return __low2float(*reinterpret_cast<__half2*>(&p)); }
  static __device__ __forceinline__ float hi(uint32_t p) { return __high2float(*reinterpret_cast<__half2*>(&p)); }
  static __device__ __forceinline__ uint32_t nibbles(uint32_t q) {
    uint32_t d;
    asm("{\n\t.reg .b32 t;\n\t"
        "max.f16x2 t, %1, %2;\n\t"
        "min.f16x2 t, t, %3;\n\t"
        "add.rn.f16x2 %0, t, %4;\n\t}"
        : "=r"(d) : "r"(q), "r"(0xC800C800u), "r"(0x47004700u), "r"(0x64086408u));
    return d;
  }
  static __device__ __forceinline__ uint32_t quot(float z0, float z1, float s, float inv_s) {
    float q0 = z0 * inv_s, q1 = z1 * inv_s;
    q0 = fmaf(fmaf(-q0, s, z0), inv_s, q0);
    q1 = fmaf(fmaf(-q1, s, z1), inv_s, q1);
    return cvt(q0, q1);
  }
  static __device__ __forceinline__ void recip2(float, uint32_t& hi2, uint32_t& lo2) { hi2 = lo2 = 0; }
  // fp16 keeps the float32 route: 1/s can leave the fp16 range
  static __device__ __forceinline__ uint32_t quotp(uint32_t zz, float s, float inv_s, uint32_t, uint32_t) {
    return quot(lo(zz), hi(zz), s, inv_s);
  }
  static __device__ __forceinline__ uint32_t nibbles_inrange(uint32_t q) {
    uint32_t d;
    asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(q), "r"(0x64086408u));
    return d;
  }
  static constexpr uint32_t kFold = 0x06u;
  static constexpr uint32_t kHalfBits = 0x6400u;
};

// 32 accumulator values of one row -> 32 offset-binary nibbles, as 4 words of 4 bytes-with-a-nibble each pair
// (P = elements 0..3, Q = elements 4..7 of a group of 8; see pack8 / bytes4)
template <typename T>
__device__ __forceinline__ void nibble_bytes(const uint32_t (&v)[32], int base, float s, float inv_s, uint32_t& p, uint32_t& q) {
  uint32_t t[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t zz = P2<T>::cvt(__uint_as_float(v[base + 2 * i]), __uint_as_float(v[base + 2 * i + 1]));  // round z
    t[i] = P2<T>::nibbles(P2<T>::quot(P2<T>::lo(zz), P2<T>::hi(zz), s, inv_s));
  }
  p = __byte_perm(t[0], t[1], 0x6420) & P2<T>::kByteMask;  // bytes: elements 0, 1, 2, 3
  q = __byte_perm(t[2], t[3], 0x6420) & P2<T>::kByteMask;  // bytes: elements 4, 5, 6, 7
}
// the same from 4 packed pairs of already rounded z values (elements base .. base+7 of a row held as pairs)
template <typename T>
__device__ __forceinline__ void nibble_bytes_packed(const uint32_t* zz, float s, float inv_s, uint32_t hi2, uint32_t lo2,
                                                    uint32_t& p, uint32_t& q) {
  uint32_t t[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) t[i] = P2<T>::nibbles(P2<T>::quotp(zz[i], s, inv_s, hi2, lo2));
  p = __byte_perm(t[0], t[1], 0x6420) & P2<T>::kByteMask;
  q = __byte_perm(t[2], t[3], 0x6420) & P2<T>::kByteMask;
}
// One word out of nibbles(): both halves are C + n with the nibble n in the low 4 bits.  Returns a word whose LOW
// BYTE is n_lo + 16 * n_hi: subtracting kFold from the low half makes the constant bits that the shift by 12 folds
// in cancel modulo 256.  Two integer multiply-adds, which run on the FMA pipe rather than the busier ALU pipe.
template <typename T>
__device__ __forceinline__ uint32_t fold_pair(uint32_t t) {
  uint32_t a, u;
  asm("mad.lo.u32 %0, %1, 1, %2;" : "=r"(a) : "r"(t), "r"(0u - P2<T>::kFold));
  asm("mad.hi.u32 %0, %1, %2, %1;" : "=r"(u) : "r"(a), "r"(1u << 20));  // (a >> 12) + a
  return u;
}
// Two words out of nibbles() (elements 0,1 and 2,3) -> their four nibbles in the LOW 16 BITS, element i at bits 4i.
// t1 * 256 + t0 puts the four nibble bytes into four different bytes (order 0, 2, 1, 3) on top of known constant
// bits; after subtracting those, (a >> 12) + a drops elements 1 and 3 between elements 0 and 2.  Three integer
// multiply-adds (FMA pipe) for four elements.
template <typename T>
__device__ __forceinline__ uint32_t fold_quad(uint32_t t0, uint32_t t1) {
  constexpr uint32_t kHalf = P2<T>::kHalfBits * 0x00010001u;
  constexpr uint32_t kConst = kHalf + (kHalf << 8);
  uint32_t v, a, u;
  asm("mad.lo.u32 %0, %1, 256, %2;" : "=r"(v) : "r"(t1), "r"(t0));
  asm("mad.lo.u32 %0, %1, 1, %2;" : "=r"(a) : "r"(v), "r"(0u - kConst));
  asm("mad.hi.u32 %0, %1, %2, %1;" : "=r"(u) : "r"(a), "r"(1u << 20));  // (a >> 12) + a
  return u;
}
// four folded pairs -> the packed word of 8 nibbles
__device__ __forceinline__ uint32_t gather4(uint32_t u0, uint32_t u1, uint32_t u2, uint32_t u3) {
  return __byte_perm(__byte_perm(u0, u1, 0x0040), __byte_perm(u2, u3, 0x0040), 0x5410);
}
// 8 rounded z values held as 4 packed pairs -> packed word; CLAMP = false only when |z / s| < 7.5 is known
template <typename T, bool CLAMP>
__device__ __forceinline__ uint32_t quantize8(const uint32_t* zz, float s, float inv_s, uint32_t hi2, uint32_t lo2) {
  uint32_t t[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t q = P2<T>::quotp(zz[i], s, inv_s, hi2, lo2);
    t[i] = CLAMP ? P2<T>::nibbles(q) : P2<T>::nibbles_inrange(q);
  }
  return __byte_perm(fold_quad<T>(t[0], t[1]), fold_quad<T>(t[2], t[3]), 0x5410);
}
// round one float to the activation dtype through the packed convert (ALU pipe, short latency)
template <typename T>
__device__ __forceinline__ float rnd1(float x) { return P2<T>::lo(P2<T>::cvt(x, x)); }
// 8 nibble-bytes -> one packed word, nibble i at bits 4i
__device__ __forceinline__ uint32_t pack8(uint32_t p, uint32_t q) {
  p |= p >> 4;
  q |= q >> 4;
  return __byte_perm(p, q, 0x6420);
}
// 4 nibble-bytes (offset binary) -> 4 signed bytes
__device__ __forceinline__ uint32_t bytes4(uint32_t p) { return ((p | 0x80808080u) - 0x08080808u) ^ 0x80808080u; }

// the packed words of up to 32 codes (`cols` of them real, a multiple of 16): one 16-byte store when all four words are
// real and the address allows it, else 8 bytes at a time (rows of 16, 48, 80 or 112 codes are only 8-byte aligned)
__device__ __forceinline__ void store_words(uint32_t* dst, const uint32_t (&w)[4], int cols) {
  if (cols == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
    *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
  } else {
    *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
    if (cols == 32) *reinterpret_cast<uint2*>(dst + 2) = make_uint2(w[2], w[3]);
  }
}

}  // namespace fq

// one launch of the batched N = 64 kernel (flatquant_sm100_n64.cu); same contract as launch_flatquant_sm100_mode
bool flatquant_sm100_n64_supported(int m, int n);
int launch_flatquant_sm100_n64(int mode, const void* x_map, const void* left, const void* right, void* out, void* scales,
                               int64_t tokens, int m, int n, float clip, int in_dtype, int scale_dtype, uint32_t* status,
                               cudaStream_t stream);

// one launch of the kernel for right transforms of 80 .. 128 (flatquant_sm100_n128.cu); tiles of
// flatquant_sm100_n128_group(m) tokens
bool flatquant_sm100_n128_supported(int m, int n);
int flatquant_sm100_n128_group(int m);
int launch_flatquant_sm100_n128(int mode, const void* x_map, const void* left, const void* right, void* out, void* scales,
                                int64_t tokens, int m, int n, float clip, int in_dtype, int scale_dtype, uint32_t* status,
                                cudaStream_t stream);

}  // namespace qo
