// Device and host helpers shared by the NVFP4 kernels: counter-based RNG, E4M3 scale codec, E2M1 level arithmetic,
// error reporting of the C ABI.
//
// Arithmetic contract: every kernel that produces codes, scale bytes or phase bytes reproduces the reference's fp32
// operation order bit for bit (bitlattice/reference.py; csrc/common.cuh of the reference). The translation units that
// include this header for such kernels are compiled with --fmad=false, so a*b+c is two roundings unless fmaf is
// written out.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/bitlattice_b200.h"

namespace blb {

// ---------------------------------------------------------------------------------------------- host: errors

void set_error(const char* fmt, ...);

#define BL_REQUIRE(cond, ...)            \
  do {                                   \
    if (!(cond)) {                       \
      ::blb::set_error(__VA_ARGS__);     \
      return 1;                          \
    }                                    \
  } while (0)

#define BL_CUDA(expr)                                                                      \
  do {                                                                                     \
    cudaError_t err__ = (expr);                                                            \
    if (err__ != cudaSuccess) {                                                            \
      ::blb::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(err__), __FILE__, __LINE__); \
      return 2;                                                                            \
    }                                                                                      \
  } while (0)

// Makes `device` current for the lifetime of the object and restores the previous device afterwards.
struct DeviceGuard {
  int prev = -1;
  bool changed = false;
  cudaError_t status = cudaSuccess;
  explicit DeviceGuard(int device) {
    status = cudaGetDevice(&prev);
    if (status == cudaSuccess && prev != device) {
      status = cudaSetDevice(device);
      changed = status == cudaSuccess;
    }
  }
  ~DeviceGuard() {
    if (changed) cudaSetDevice(prev);
  }
};

#define BL_DEVICE(device)                                                          \
  ::blb::DeviceGuard guard__(device);                                              \
  if (guard__.status != cudaSuccess) {                                             \
    ::blb::set_error("cannot select CUDA device %d: %s", device, cudaGetErrorString(guard__.status)); \
    return 2;                                                                      \
  }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int sm_count(int device);

// ---------------------------------------------------------------------------------------------- device: RNG

// u in [0, 1) from (element index, seed, step): bitlattice/reference.py:22-30. idx is truncated to 32 bits.
__device__ __forceinline__ float hash_uniform(uint32_t idx, uint32_t key) {
  uint32_t x = idx * 0x27D4EB2Fu + key;
  x = (x ^ (x >> 16)) * 0x7FEB352Du;
  x = (x ^ (x >> 15)) * 0x846CA68Bu;
  x ^= x >> 16;
  return static_cast<float>(x >> 8) * 5.9604644775390625e-08f;
}

__host__ __device__ __forceinline__ uint32_t hash_key(uint32_t seed, uint32_t step) {
  return seed * 0x9E3779B1u + step * 0x85EBCA77u;
}

// Rounding draw of the lattice projection (bitlattice/reference.py:41-51). For 'strat' key is hash_key(seed, 0).
struct RoundParams {
  int mode;        // BL_ROUND_*
  uint32_t key;
  float strat_j;
  float strat_k;
};

__device__ __forceinline__ float rounding_u(const RoundParams& rp, uint32_t idx) {
  if (rp.mode == BL_ROUND_SR) return hash_uniform(idx, rp.key);
  if (rp.mode == BL_ROUND_STRAT) {
    const float v = (rp.strat_j + hash_uniform(idx, rp.key)) / rp.strat_k;
    return v - truncf(v);
  }
  return 0.5f;
}

// ---------------------------------------------------------------------------------------------- device: E4M3

__device__ __forceinline__ float e4m3_decode(uint32_t byte) {
  __nv_fp8_e4m3 v;
  v.__x = static_cast<__nv_fp8_storage_t>(byte);
  return static_cast<float>(v);
}

// clamp to [2^-9, 448], round to nearest even (bitlattice/reference.py:71-72)
__device__ __forceinline__ uint32_t e4m3_encode(float s) {
  const __nv_fp8_e4m3 v(fminf(fmaxf(s, 0.001953125f), 448.0f));
  return v.__x;
}

// ---------------------------------------------------------------------------------------------- device: E2M1 levels
// The 15 levels of NVFP4 in ascending order have rank 0..14 (-6 ... 0 ... 6); rank 7 is zero.
// bitlattice/formats.py:151-170: code c < 8 -> rank 7 + c; code 8 (-0) reads as rank 7; code c > 8 -> rank 15 - c.

__device__ __forceinline__ int rank_of_code(uint32_t c) { return c < 8u ? 7 + static_cast<int>(c) : (c == 8u ? 7 : 15 - static_cast<int>(c)); }
__device__ __forceinline__ uint32_t code_of_rank(int r) { return r >= 7 ? static_cast<uint32_t>(r - 7) : static_cast<uint32_t>(15 - r); }

// magnitude of E2M1 index k in 0..7: {0, .5, 1, 1.5, 2, 3, 4, 6}, built from two byte tables with PRMT (no memory)
__device__ __forceinline__ float mag_of(uint32_t k) {
  const uint32_t hi = __byte_perm(0x3F3F3F00u, 0x40404040u, k << 12);
  const uint32_t lo = __byte_perm(0xC0800000u, 0xC0804000u, k << 8);
  return __uint_as_float(hi | lo);
}

__device__ __forceinline__ float level_of_rank(int r) {
  const int d = r - 7;
  const float m = mag_of(static_cast<uint32_t>(d < 0 ? -d : d));
  return d < 0 ? -m : m;
}

// rank of the nearest level, ties to the lower level: the number of midpoints strictly below x
// (bitlattice/reference.py:130-135)
__device__ __forceinline__ int nearest_rank(float x) {
  return (x > -5.0f) + (x > -3.5f) + (x > -2.5f) + (x > -1.75f) + (x > -1.25f) + (x > -0.75f) + (x > -0.25f) +
         (x > 0.25f) + (x > 0.75f) + (x > 1.25f) + (x > 1.75f) + (x > 2.5f) + (x > 3.5f) + (x > 5.0f);
}

// E2M1 code of the level nearest to v, ties to the lower value: rank -> canonical code
__device__ __forceinline__ uint32_t e2m1_code_nearest(float v) { return code_of_rank(nearest_rank(v)); }

// stochastic rounding between the two E2M1 neighbours of v (bitlattice/fp4ref.py:71-78)
__device__ __forceinline__ uint32_t e2m1_code_sr(float v, float u) {
  const float a = fminf(fabsf(v), 6.0f);
  uint32_t m = (a >= 0.5f) + (a >= 1.0f) + (a >= 1.5f) + (a >= 2.0f) + (a >= 3.0f) + (a >= 4.0f) + (a >= 6.0f);
  if (m < 7u) {
    const float lo = mag_of(m), hi = mag_of(m + 1u);
    m += u * (hi - lo) < a - lo;
  }
  return (v < 0.0f && m ? 8u : 0u) | m;
}

// ---------------------------------------------------------------------------------------------- device: division
// x / y rounded to nearest, from a correctly rounded reciprocal ry = __frcp_rn(y) that the caller shares between many
// quotients: one product and two residual corrections with fused multiply-adds (the sequence compilers emit for an
// fp32 division, minus the reciprocal and the range checks). The residuals are exact, so the result is the correctly
// rounded quotient whenever no intermediate leaves the normal range; outside it the plain division is used.
static __device__ __noinline__ float div_general(float x, float y) { return x / y; }

__device__ __forceinline__ float div_rn(float x, float y, float ry) {
  const float q0 = x * ry;
  float e = fmaf(-y, q0, x);
  float q = fmaf(e, ry, q0);
  e = fmaf(-y, q, x);
  q = fmaf(e, ry, q);
  const float aq = fabsf(q0);
  // zero, tiny, huge or non-finite: the general path, kept out of line so that it costs nothing when not taken
  if (__builtin_expect(!(aq > 1e-30f && aq < 1e30f), 0)) return div_general(x, y);
  return q;
}

// ---------------------------------------------------------------------------------------------- device: fp32 pairs
// Two independent fp32 operations per instruction, each lane rounded to nearest like the scalar operation (the fused
// multiply-add is written out only where a single rounding is wanted: the residuals of the divisions).

using f32x2 = unsigned long long;

__device__ __forceinline__ f32x2 pk(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void upk(f32x2 p, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(p)); }
__device__ __forceinline__ f32x2 mul2p(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ f32x2 add2p(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ f32x2 sub2p(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ f32x2 fma2p(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
// a * b per lane, rounded once, for products that FEED A SUM: written as a fused multiply-add with a +0 addend, which
// the assembler can neither merge with the following add (it would have to fuse two roundings) nor turn back into a
// plain multiply (the +0 turns a product of -0 into +0). Only for uses where the sign of a zero product cannot matter.
__device__ __forceinline__ f32x2 prod2p(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(0ull));
  return r;
}
// x / y per lane from ny = -y and ry = rcp_rn(y): div_rn without its range check (the caller establishes the range)
__device__ __forceinline__ f32x2 div2p(f32x2 x, f32x2 ny, f32x2 ry) {
  const f32x2 q0 = mul2p(x, ry);
  f32x2 e = fma2p(ny, q0, x);
  f32x2 q = fma2p(e, ry, q0);
  e = fma2p(ny, q, x);
  return fma2p(e, ry, q);
}

// ---------------------------------------------------------------------------------------------- device: fast E2M1
// The hardware conversion cvt.rn.satfinite.e2m1x2.f32 rounds two floats to E2M1 nibbles (ties to even, -0 kept).
// It gives the reference's code (ties to the lower level, +0 only) whenever its input is not at, or within rounding
// error of, a midpoint between two levels; the callers below establish that by converting a lower and an upper bound
// of the exact quotient and comparing, and take the exact ladder otherwise.

// byte with the code of `hi` in the upper and of `lo` in the lower nibble
__device__ __forceinline__ uint32_t cvt_e2m1x2(float hi, float lo) {
  uint32_t r;
  asm("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tcvt.u32.u8 %0, t;\n\t}" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// 8 floats -> 8 nibbles (element i in nibble i)
__device__ __forceinline__ uint32_t cvt_e2m1x8(const float v[8]) {
  return cvt_e2m1x2(v[1], v[0]) | (cvt_e2m1x2(v[3], v[2]) << 8) | (cvt_e2m1x2(v[5], v[4]) << 16) |
         (cvt_e2m1x2(v[7], v[6]) << 24);
}

// clear the sign bit of every nibble whose magnitude is zero (-0 -> +0: the reference never writes code 8)
__device__ __forceinline__ uint32_t e2m1_drop_negative_zero(uint32_t w) {
  const uint32_t m = w & 0x77777777u;
  const uint32_t nz = (m | (m >> 1) | (m >> 2)) & 0x11111111u;
  return m | (w & (nz << 3));
}

// Round-to-nearest codes (ties to the lower level) of v[i] / se for 8 values, se > 0.
// inv_lo / inv_hi: (1/se) scaled by (1 - 2^-20) and (1 + 2^-20): v*inv_lo and v*inv_hi bracket the exact quotient
// (the two roundings of each product are below 2^-22 relative), E2M1 rounding is monotone, so equal conversions of
// the two bounds equal the conversion of the quotient, which then is no tie.
// the exact ladder for 8 values: kept out of line so the common path stays small
static __device__ __noinline__ uint32_t e2m1_nearest_x8_exact(float v0, float v1, float v2, float v3, float v4, float v5,
                                                       float v6, float v7, float se) {
  return e2m1_code_nearest(v0 / se) | (e2m1_code_nearest(v1 / se) << 4) | (e2m1_code_nearest(v2 / se) << 8) |
         (e2m1_code_nearest(v3 / se) << 12) | (e2m1_code_nearest(v4 / se) << 16) | (e2m1_code_nearest(v5 / se) << 20) |
         (e2m1_code_nearest(v6 / se) << 24) | (e2m1_code_nearest(v7 / se) << 28);
}

__device__ __forceinline__ uint32_t e2m1_nearest_x8(const float v[8], float se, float inv_lo, float inv_hi) {
  float a[8], b[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    a[i] = v[i] * inv_lo;
    b[i] = v[i] * inv_hi;
  }
  const uint32_t wa = cvt_e2m1x8(a), wb = cvt_e2m1x8(b);
  if (__builtin_expect(wa == wb, 1)) return e2m1_drop_negative_zero(wa);
  return e2m1_nearest_x8_exact(v[0], v[1], v[2], v[3], v[4], v[5], v[6], v[7], se);   // at or next to a midpoint
}

// Stochastic-rounding codes of x[i] = v[i] * inv (bitlattice/fp4ref.py:71-78) for 8 values; u from hash(idx0 + i).
// lo = largest level <= min(|x|, 6) (the float truncated to one mantissa bit, or 0 / 0.5 below 1), gap to the next.
__device__ __forceinline__ uint32_t e2m1_sr_x8(const float v[8], float inv, uint32_t key, uint32_t idx0) {
  float r[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float x = v[i] * inv;
    const float a = fminf(fabsf(x), 6.0f);
    const uint32_t ab = __float_as_uint(a);
    const float lo = a >= 1.0f ? __uint_as_float(ab & 0xFFC00000u) : (a >= 0.5f ? 0.5f : 0.0f);
    const float gap = a >= 2.0f ? __uint_as_float((ab & 0x7F800000u) - 0x00800000u) : 0.5f;
    const float u = hash_uniform(idx0 + i, key);
    const bool up = lo < 6.0f && u * gap < a - lo;
    r[i] = copysignf(up ? lo + gap : lo, x);
  }
  return e2m1_drop_negative_zero(cvt_e2m1x8(r));
}

// ---------------------------------------------------------------------------------------------- device: blocks of 16
// Whole 16-element blocks in one thread, written for few issue slots per element: packed fp32x2 multiplies, four
// conversions merged into one register, and stochastic rounding decided in 2^-25 fixed point.

// {a * s, b * s}: one packed multiply, each lane rounded to nearest like a scalar multiply
__device__ __forceinline__ void mul2(float a, float b, float s, float& ra, float& rb) {
  asm("{\n\t.reg .b64 p, q;\n\t"
      "mov.b64 p, {%2, %3};\n\t"
      "mov.b64 q, {%4, %4};\n\t"
      "mul.rn.f32x2 p, p, q;\n\t"
      "mov.b64 {%0, %1}, p;\n\t}"
      : "=f"(ra), "=f"(rb)
      : "f"(a), "f"(b), "f"(s));
}

// 8 floats -> 8 nibbles in one register (element i in nibble i), hardware rounding (nearest, ties to even)
__device__ __forceinline__ uint32_t cvt_e2m1x8_merged(const float v[8]) {
  uint32_t w;
  asm("{\n\t.reg .b8 t0, t1, t2, t3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 t0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 t1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 t2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 t3, %8, %7;\n\t"
      "mov.b32 %0, {t0, t1, t2, t3};\n\t}"
      : "=r"(w)
      : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]));
  return w;
}

// Round-to-nearest codes (ties to the lower level) of (v[i] * pre) / se for 16 values, se > 0; pre is 1 or a power of
// two folded into the bracket. inv approximates 1 / se to a few ulps; the bracket (1 -+ 2^-19) around it contains the
// exact quotient, so equal conversions of both ends are the conversion of the quotient, which then is no tie;
// otherwise (at or next to a midpoint) the exact ladder decides.
// exact code of one value, out of line: the per-element repair of e2m1_rtn16
static __device__ __noinline__ uint32_t e2m1_nearest_exact(float v, float se) { return e2m1_code_nearest(v / se); }

__device__ __forceinline__ uint2 e2m1_rtn16(const float v[16], float pre, float se, float inv) {
  const float lo = inv * pre * 0.99999809265136718750f, hi = inv * pre * 1.00000190734863281250f;
  float a[16], b[16];
#pragma unroll
  for (int i = 0; i < 16; i += 2) {
    mul2(v[i], v[i + 1], lo, a[i], a[i + 1]);
    mul2(v[i], v[i + 1], hi, b[i], b[i + 1]);
  }
  uint32_t w[2] = {cvt_e2m1x8_merged(a), cvt_e2m1x8_merged(a + 8)};
  uint32_t d[2] = {w[0] ^ cvt_e2m1x8_merged(b), w[1] ^ cvt_e2m1x8_merged(b + 8)};
  // (the reciprocal is only trusted for scales well inside the normal range)
  if (!(se > 1e-30f && se < 1e30f)) d[0] = d[1] = 0xFFFFFFFFu;
  if (__builtin_expect((d[0] | d[1]) != 0u, 0)) {
    // Values at a midpoint between two levels are common with 8-bit inputs and few-bit scales: repair only the
    // elements whose two conversions differ.
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t m = 0xFu << (4 * (i & 7));
      if (d[i >> 3] & m) w[i >> 3] = (w[i >> 3] & ~m) | (e2m1_nearest_exact(v[i] * pre, se) << (4 * (i & 7)));
    }
  }
  return make_uint2(e2m1_drop_negative_zero(w[0]), e2m1_drop_negative_zero(w[1]));
}

// Stochastic-rounding codes of x[i] = v[i] * inv for 16 values (bitlattice/fp4ref.py:71-78), u from hash(idx0 + i).
// With a = min(|x|, 6) and A = ceil(a * 2^25) (exact for a >= 0.5), shifting A right by t = [a >= 2] + [a >= 4] puts
// the level index below a in the bits above 24 and the position between the two neighbouring levels, as a fraction
// of 2^24, in the bits below. The draw n = hash >> 8 rounds up iff n < that fraction, which is the carry of adding
// (2^24 - 1 - n): so the code is ((A >> t) + (~hash >> 8) >> 24) + 2 t. Identical to comparing u * gap < a - lo in
// real numbers, which is what the reference's fp32 expression evaluates without rounding.
// (Shifts, adds and bit operations issue on the ALU pipe, which bounds this loop -- over 80 % busy with the multiply-add
// pipe at a quarter. The 2 t and the merge of the nibble into the word are therefore integer multiply-adds, with the
// multipliers read from constant memory so that the compiler cannot turn them back into shifts and ors: 7 % off the
// transposed stochastic quantizer. High products and wide multiply-adds in place of the right shifts cost more than
// the two ALU instructions they replace; measured and not kept.)
static __device__ __constant__ uint32_t kPipeMul[9] = {2u, 1u, 1u << 4, 1u << 8, 1u << 12, 1u << 16, 1u << 20, 1u << 24, 1u << 28};

__device__ __forceinline__ uint2 e2m1_sr16(const float v[16], float inv, uint32_t key, uint32_t idx0) {
  uint32_t w[2] = {0u, 0u};
  const uint32_t h0 = idx0 * 0x27D4EB2Fu + key;
  const uint32_t two = kPipeMul[0];
#pragma unroll
  for (int i = 0; i < 16; i += 2) {
    float x[2];
    mul2(v[i], v[i + 1], inv, x[0], x[1]);
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const float a = fminf(fabsf(x[e]), 6.0f);
      const uint32_t A = __float2uint_ru(a * 33554432.0f);
      const uint32_t t = __byte_perm(0x02020100u, 0u, A >> 26);
      uint32_t h = h0 + static_cast<uint32_t>(i + e) * 0x27D4EB2Fu;
      h = (h ^ (h >> 16)) * 0x7FEB352Du;
      h = (h ^ (h >> 15)) * 0x846CA68Bu;
      h = ~(h ^ (h >> 16));
      const uint32_t k = (((A >> t) + (h >> 8)) >> 24) + two * t;
      const uint32_t nib = k | ((__float_as_uint(x[e]) >> 28) & 8u);
      w[(i + e) >> 3] = nib * kPipeMul[1 + ((i + e) & 7)] + w[(i + e) >> 3];   // nibbles do not overlap: + is |
    }
  }
  return make_uint2(e2m1_drop_negative_zero(w[0]), e2m1_drop_negative_zero(w[1]));
}

// ---------------------------------------------------------------------------------------------- device: dense loads

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

// 8 consecutive elements starting at a multiple of 8 (16-byte aligned for 2-byte types, 32 for fp32)
template <typename T>
__device__ __forceinline__ void load8(const T* p, float v[8]) {
  if constexpr (sizeof(T) == 4) {
    const float4 a = reinterpret_cast<const float4*>(p)[0];
    const float4 b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = to_f<T>(e[i]);
  }
}

}  // namespace blb
