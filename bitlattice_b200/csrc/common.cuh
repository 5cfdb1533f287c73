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
