// NVFP4 operand quantizers, dequantization and the blocked scale layout.
//
// Reference semantics (compiled with --fmad=false; codes and scale bytes are bit-exact with these):
//   round to nearest : bitlattice/reference.py:164-235 ('rtn': ties to the lower level, v / (scale*global));
//                      reference kernel csrc/act_quant.cu:16-27,66-86
//   stochastic       : bitlattice/fp4ref.py:71-78,103-150 ('sr': v * (1/(scale*global)), u = hash(flat index, seed, 0))
//   transposed, H16  : csrc/act_quant.cu:100-148 (blocks of 16 along the rows of x, v <- v H summed in input order)
//   W^T              : csrc/act_quant.cu:150-175 (values formed as (level*scale)*global, same per-tensor scale)
//   dequantize       : bitlattice/reference.py:238-245
//   blocked scales   : bitlattice/backend.py:179-188
#include <type_traits>

#include "common.cuh"

namespace blb {

constexpr int kQThreads = 256;

// ------------------------------------------------------------------------------------------------ amax

__device__ __forceinline__ void atomic_max_pos(float* addr, float v) {   // v >= 0: integer order == float order
  atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v));
}

// out[0] = max|x| (out must start at zero); the last block to finish writes out[1] = max(out[0] / 2688, 1e-12) and
// out[3] = max(out[0] / 1536, 1e-12); out[2] is the ticket counter
template <typename T>
__global__ void __launch_bounds__(kQThreads) amax_kernel(const T* __restrict__ x, int64_t n, float* __restrict__ out) {
  constexpr int per = 16 / sizeof(T);
  const int64_t nvec = n / per;
  float m = 0.0f;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const uint4 raw = reinterpret_cast<const uint4*>(x)[i];
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int j = 0; j < per; ++j) m = fmaxf(m, fabsf(to_f<T>(e[j])));
  }
  if (blockIdx.x == 0 && threadIdx.x < n - nvec * per) m = fmaxf(m, fabsf(to_f<T>(x[nvec * per + threadIdx.x])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  __shared__ float warp_max[kQThreads / 32];
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < kQThreads / 32; ++w) m = fmaxf(m, warp_max[w]);
    atomic_max_pos(out, m);
    __threadfence();
    unsigned* ticket = reinterpret_cast<unsigned*>(out + 2);
    if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
      __threadfence();
      const float a = *reinterpret_cast<volatile float*>(out);
      out[1] = fmaxf(a / 2688.0f, 1e-12f);
      out[3] = fmaxf(a / 1536.0f, 1e-12f);      // the four-over-six recipe: amax / (6 * 256)
    }
  }
}

// ------------------------------------------------------------------------------------------------ block quantizer

// 8 of the 16 values of a block held by this lane (the partner lane, xor 1, holds the other 8): returns this
// lane's 8 codes; *scale receives the E4M3 byte of the block.
// SR == false: reference.quantize 'rtn'. SR == true: fp4ref.quantize 'sr' (idx0 = flat index of v[0]).
constexpr float kInv6 = 0.16666667163372039794921875f;   // the float nearest to 1/6

// rg = __frcp_rn(g), shared by all blocks of a kernel
template <bool SR>
__device__ __forceinline__ uint32_t quantize_half_block(const float v[8], float g, float rg, uint32_t key,
                                                        uint32_t idx0, uint32_t* scale) {
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  uint32_t out;
  if constexpr (!SR) {
    const uint32_t sb = e4m3_encode(div_rn(fmaxf(div_rn(amax, 6.0f, kInv6), 1e-12f), g, rg));
    const float se = e4m3_decode(sb) * g;
    const float inv = __frcp_rn(se);
    out = e2m1_nearest_x8(v, se, inv * 0.99999904632568359375f, inv * 1.00000095367431640625f);
    *scale = sb;
  } else {
    const uint32_t sb = e4m3_encode(div_rn(div_rn(amax, 6.0f, kInv6), g, rg));
    const float t = e4m3_decode(sb) * g;
    const float inv = t > 0.0f ? __frcp_rn(t) : 0.0f;
    out = e2m1_sr_x8(v, inv, key, idx0);
    *scale = sb;
  }
  return out;
}

__device__ __forceinline__ int64_t scale_index(int layout, int64_t r, int64_t c16, int64_t cols16) {
  if (layout == BL_SF_ROWMAJOR) return r * cols16 + c16;
  const int64_t nc = (cols16 + 3) >> 2;
  return ((r >> 7) * nc + (c16 >> 2)) * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (c16 & 3);
}

// ------------------------------------------------------------------------------------------------ rows

// x [rows, cols] -> codes [rows, cols/2], scales.

// ---- rows, one thread per block of 16 ---------------------------------------------------------------------------------

__device__ __forceinline__ float rcp_approx(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

// block quantization modes
constexpr int kModeRtn = 0, kModeSr = 1, kModeFosMse = 2, kModeFosMae = 3;

// levels of 8 codes (one register of nibbles) times se, through the hardware E2M1 -> fp16 conversion
__device__ __forceinline__ void e2m1_values8(uint32_t w, float se, float out[8]) {
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    uint32_t h2;
    asm("{\n\t.reg .b8 b;\n\tcvt.u8.u32 b, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, b;\n\t}" : "=r"(h2) : "r"(w >> (8 * k)));
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h2));
    out[2 * k] = f.x * se;
    out[2 * k + 1] = f.y * se;
  }
}

// One candidate of the four-over-six choice: codes of v / se (one reciprocal per block, nearest level with ties to the
// even code: the hardware conversion) and the error of the dequantized block, summed over the elements in ascending
// order (bitlattice/fp4ref.py:117-131; the reference's kernel: csrc/nvfp4.cu:176-195)
template <bool MAE>
__device__ __forceinline__ float fos_candidate(const float v[16], float se, uint2& codes) {
  const float inv = se > 0.0f ? __frcp_rn(se) : 0.0f;
  float q[16];
#pragma unroll
  for (int i = 0; i < 16; i += 2) mul2(v[i], v[i + 1], inv, q[i], q[i + 1]);
  codes = make_uint2(cvt_e2m1x8_merged(q), cvt_e2m1x8_merged(q + 8));
  float d[16];
  e2m1_values8(codes.x, se, d);
  e2m1_values8(codes.y, se, d + 8);
  float err = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float e = d[i] - v[i];
    err = err + (MAE ? fabsf(e) : e * e);
  }
  return err;
}

// One block of 16 values v[i] * pre (pre: 1 or a power of two) -> 16 codes and the scale byte.
// kModeRtn: reference.quantize 'rtn'. kModeSr: fp4ref.quantize 'sr' (idx0 = flat index of v[0]). kModeFosMse /
// kModeFosMae: fp4ref.quantize 'rtn' with four_over_six (pre must be 1).
template <int MODE>
__device__ __forceinline__ uint2 quantize_block(const float v[16], float pre, float g, float rg, uint32_t key,
                                                uint32_t idx0, uint32_t* scale) {
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  amax *= pre;
  if constexpr (MODE == kModeRtn) {
    const uint32_t sb = e4m3_encode(div_rn(fmaxf(div_rn(amax, 6.0f, kInv6), 1e-12f), g, rg));
    const float se = e4m3_decode(sb) * g;
    *scale = sb;
    return e2m1_rtn16(v, pre, se, rcp_approx(se));
  } else if constexpr (MODE == kModeSr) {
    const uint32_t sb = e4m3_encode(div_rn(div_rn(amax, 6.0f, kInv6), g, rg));
    const float t = e4m3_decode(sb) * g;
    const float inv = t > 0.0f ? __frcp_rn(t) : 0.0f;
    *scale = sb;
    return e2m1_sr16(v, inv * pre, key, idx0);
  } else {
    const uint32_t b6 = e4m3_encode(div_rn(div_rn(amax, 6.0f, kInv6), g, rg));
    const uint32_t b4 = e4m3_encode(div_rn(amax * 0.25f, g, rg));
    uint2 c6, c4;
    const float e6 = fos_candidate<MODE == kModeFosMae>(v, e4m3_decode(b6) * g, c6);
    const float e4 = fos_candidate<MODE == kModeFosMae>(v, e4m3_decode(b4) * g, c4);
    const bool pick4 = e4 < e6;
    *scale = pick4 ? b4 : b6;
    const uint2 c = pick4 ? c4 : c6;
    return make_uint2(e2m1_drop_negative_zero(c.x), e2m1_drop_negative_zero(c.y));
  }
}

template <typename T>
struct Raw16 {                                       // 16 elements as loaded
  uint4 q[sizeof(T) * 16 / 16];
};

template <typename T>
__device__ __forceinline__ void load_raw16(const T* p, Raw16<T>& r) {
#pragma unroll
  for (int i = 0; i < static_cast<int>(sizeof(T)); ++i) r.q[i] = __ldcs(reinterpret_cast<const uint4*>(p) + i);
}

template <typename T>
__device__ __forceinline__ void unpack_raw16(const Raw16<T>& r, float v[16]) {
  const uint32_t* w = reinterpret_cast<const uint32_t*>(r.q);
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(w[i]);
  } else if constexpr (std::is_same<T, __nv_bfloat16>::value) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
}

// block (bx, 256/bx): x covers the 16-element blocks of a row, y covers rows; a thread keeps its block column and walks
// down the rows, the next row's block in flight while the current one is quantized.
template <typename T, int MODE>
__global__ void __launch_bounds__(kQThreads, MODE == kModeSr ? 4 : 3)
    quantize_rows16_kernel(const T* __restrict__ x, int64_t rows, int64_t cols, const float* __restrict__ global,
                           uint32_t key, uint8_t* __restrict__ codes, uint8_t* __restrict__ scales, int layout) {
  const float g = global[0];
  const float rg = __frcp_rn(g);
  const int64_t cb = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;   // block column
  const int64_t cols16 = cols / 16;
  if (cb >= cols16) return;
  const int64_t row_step = static_cast<int64_t>(gridDim.y) * blockDim.y;
  // scale position: row-major r * cols16 + cb; blocked ((r >> 7) * nc + (cb >> 2)) * 512 + (r & 31) * 16 +
  // ((r >> 5) & 3) * 4 + (cb & 3)
  const int64_t nc = (cols16 + 3) >> 2;
  const int64_t sf_col = layout == BL_SF_ROWMAJOR ? cb : (cb >> 2) * 512 + (cb & 3);
  // the next row's block is loaded before the current one is worked on: a warp never waits for memory with nothing
  // else to issue
  int64_t r = static_cast<int64_t>(blockIdx.y) * blockDim.y + threadIdx.y;
  Raw16<T> cur;
  if (r < rows) load_raw16(x + r * cols + cb * 16, cur);
  for (; r < rows; r += row_step) {
    Raw16<T> next;
    if (r + row_step < rows) load_raw16(x + (r + row_step) * cols + cb * 16, next);
    float v[16];
    unpack_raw16(cur, v);
    uint32_t sb;
    const uint2 out = quantize_block<MODE>(v, 1.0f, g, rg, key, static_cast<uint32_t>(r * cols + cb * 16), &sb);
    __stcs(reinterpret_cast<uint2*>(codes + r * (cols / 2)) + cb, out);
    const int64_t sf_row = layout == BL_SF_ROWMAJOR ? r * cols16
                                                    : (r >> 7) * nc * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4;
    scales[sf_row + sf_col] = static_cast<uint8_t>(sb);
    cur = next;
  }
}

struct RowGeometry {
  dim3 block, grid;
};

static RowGeometry row_geometry(int64_t rows, int64_t cols, int device) {
  const int64_t cpr = cols / 16;
  int bx = 32;
  while (bx < kQThreads && bx < cpr) bx <<= 1;
  const int by = kQThreads / bx;
  const int64_t gx = (cpr + bx - 1) / bx;
  // whole waves whether an SM holds three or four CTAs (59-62 registers per thread): no partly filled last wave
  int64_t gy = (static_cast<int64_t>(sm_count(device)) * 12) / gx;
  const int64_t max_gy = (rows + by - 1) / by;
  gy = gy < 1 ? 1 : (gy > max_gy ? max_gy : gy);
  if (gy > 65535) gy = 65535;
  RowGeometry g;
  g.block = dim3(bx, by);
  g.grid = dim3(static_cast<unsigned>(gx), static_cast<unsigned>(gy));
  return g;
}

// ------------------------------------------------------------------------------------------------ transposed

constexpr int kTM = 128;   // rows of x per tile (8 blocks of 16)
constexpr int kTK = 64;    // columns of x per tile

// Rotated block column: v[j] = sum over i (ascending) of raw[i] * H[i][j]; this thread computes 8 of the 16 outputs
// (j = 8*half .. 8*half+7) of the block whose 16 inputs are raw[].
__device__ __forceinline__ void rotate_half(const float raw[16], const float* __restrict__ sH, int half, float v[8]) {
#pragma unroll
  for (int jj = 0; jj < 8; ++jj) {
    const int j = half * 8 + jj;
    float a = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) a = a + raw[i] * sH[i * 16 + j];
    v[jj] = a;
  }
}

// amax of the (rotated) transposed tensor; out as for amax_kernel but without the scale
template <typename T>
__global__ void __launch_bounds__(kQThreads) amax_t_kernel(const T* __restrict__ x, int64_t M, int64_t K,
                                                           const float* __restrict__ H, float* __restrict__ out) {
  __shared__ float sH[256];
  if (H != nullptr) sH[threadIdx.x] = H[threadIdx.x];
  __syncthreads();
  const int64_t n = (M / 16) * K;
  float m = 0.0f;
  for (int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < n;
       t += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t k = t % K, mb = t / K;
    float raw[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) raw[i] = to_f<T>(x[(mb * 16 + i) * K + k]);
    if (H == nullptr) {
#pragma unroll
      for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(raw[i]));
    } else {
      float v[8];
      rotate_half(raw, sH, 0, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(v[i]));
      rotate_half(raw, sH, 1, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(v[i]));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) atomic_max_pos(out, m);
}

// global scale of the transposed operand: from a bound (given == 1: in[0] is the bound), from an amax (given == 0),
// or as is (given == 2: in[0] already is the scale). The quantizers evaluate it themselves and their first thread
// publishes it, which saves a launch per operand; the one-thread kernel remains for callers whose output aliases the
// input.
__device__ __forceinline__ float global_t(const float* __restrict__ in, int given) {
  if (given == 2) return in[0];
  const float amax = given ? in[0] * 2688.0f : in[0];
  return fmaxf(amax / 2688.0f, 1e-12f);
}

__global__ void global_t_kernel(const float* __restrict__ in, int given, float* __restrict__ global_out) {
  global_out[0] = global_t(in, given);
}

// x [M, K] -> NVFP4 of x^T. A CTA stages a [128, 64] tile of x in shared memory with coalesced row reads; the work
// item (k, mb, half) quantizes 8 of the 16 rotated values of block mb of column k; lane pairs (half 0/1) share a block.
template <typename T, bool SR>
__global__ void __launch_bounds__(kQThreads) quantize_t_kernel(const T* __restrict__ x, int64_t M, int64_t K,
                                                               const float* __restrict__ H,
                                                               const float* __restrict__ global, int given,
                                                               float* __restrict__ global_out, uint32_t key,
                                                               uint8_t* __restrict__ codes, uint8_t* __restrict__ scales,
                                                               int layout) {
  __shared__ float tile[kTM][kTK + 1];
  __shared__ float sH[256];
  if (H != nullptr) sH[threadIdx.x] = H[threadIdx.x];
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * kTM, k0 = static_cast<int64_t>(blockIdx.x) * kTK;
  for (int i = threadIdx.x; i < kTM * kTK; i += kQThreads) {
    const int rr = i / kTK, cc = i % kTK;
    const int64_t m = m0 + rr, k = k0 + cc;
    tile[rr][cc] = (m < M && k < K) ? to_f<T>(x[m * K + k]) : 0.0f;
  }
  __syncthreads();
  const float g = global_t(global, given);
  if (global_out != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) global_out[0] = g;
  // 64 columns x 8 blocks x 2 halves = 1024 work items, 4 per thread; lanes (2j, 2j+1) = halves of one block
  for (int it = 0; it < 4; ++it) {
    const int w = it * kQThreads + threadIdx.x;
    const int half = w & 1, kk = (w >> 1) & (kTK - 1), mb = w >> 7;
    const int64_t k = k0 + kk, m = m0 + mb * 16;
    const bool active = k < K && m < M;               // M % 16 == 0: a block is inside or outside as a whole
    float raw[16], v[8];
#pragma unroll
    for (int i = 0; i < 16; ++i) raw[i] = tile[mb * 16 + i][kk];
    if (H != nullptr) {
      rotate_half(raw, sH, half, v);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = raw[half * 8 + i];
    }
    uint32_t sb;
    const uint32_t idx0 = static_cast<uint32_t>(static_cast<uint64_t>(k) * static_cast<uint64_t>(M) + m + half * 8);
    const uint32_t out = quantize_half_block<SR>(v, g, __frcp_rn(g), key, idx0, &sb);
    if (!active) continue;
    *reinterpret_cast<uint32_t*>(codes + k * (M / 2) + (m + half * 8) / 2) = out;
    if (half == 0) scales[scale_index(layout, k, m / 16, M / 16)] = static_cast<uint8_t>(sb);
  }
}

// ---- transposed quantizer, one thread per (block of 16 rows, pair of adjacent columns) ------------------------------

template <typename T>
__device__ __forceinline__ void load2(const T* p, float& a, float& b) {
  if constexpr (sizeof(T) == 4) {
    const float2 v = *reinterpret_cast<const float2*>(p);
    a = v.x;
    b = v.y;
  } else if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    const uint32_t v = *reinterpret_cast<const uint32_t*>(p);
    a = __uint_as_float(v << 16);
    b = __uint_as_float(v & 0xFFFF0000u);
  } else {
    const float2 v = __half22float2(*reinterpret_cast<const __half2*>(p));
    a = v.x;
    b = v.y;
  }
}

// v[j] = sum over i (ascending, every partial sum rounded to fp32: the reference's order) of p[i] * (-1)^popc(i & j),
// p[i] = raw[i] * H[i][0], for H = diag(s) * Sylvester-Hadamard / 4. Outputs j and j' share every partial sum over
// i < n when j = j' mod n, so the 16 sequential sums form a tree of 2 + 8 + 32 + 128 = 170 additions instead of 256.
__device__ __forceinline__ void rotate16_tree(const float p[16], float v[16]) {
  v[0] = p[0] + p[1];
  v[1] = p[0] - p[1];
#pragma unroll
  for (int n = 2; n < 16; n <<= 1) {
#pragma unroll
    for (int j = 0; j < n; ++j) {
      float a = v[j], b = v[j];
#pragma unroll
      for (int i = 0; i < n; ++i) {
        if (__popc(i & j) & 1) {
          a = a - p[n + i];
          b = b + p[n + i];
        } else {
          a = a + p[n + i];
          b = b - p[n + i];
        }
      }
      v[j] = a;
      v[n + j] = b;
    }
  }
}

// The same tree for two columns at once, one in each lane of packed fp32 pairs: half the instructions. (p holds
// products by +-1/4, which are exact, so it does not matter that a packed product feeding a packed sum is contracted
// into one fused multiply-add.)
__device__ __forceinline__ void rotate16_tree2(const f32x2 p[16], f32x2 v[16]) {
  v[0] = add2p(p[0], p[1]);
  v[1] = sub2p(p[0], p[1]);
#pragma unroll
  for (int n = 2; n < 16; n <<= 1) {
#pragma unroll
    for (int j = 0; j < n; ++j) {
      f32x2 a = v[j], b = v[j];
#pragma unroll
      for (int i = 0; i < n; ++i) {
        if (__popc(i & j) & 1) {
          a = sub2p(a, p[n + i]);
          b = add2p(b, p[n + i]);
        } else {
          a = add2p(a, p[n + i]);
          b = sub2p(b, p[n + i]);
        }
      }
      v[j] = a;
      v[n + j] = b;
    }
  }
}

// any 16 x 16 matrix: for each output the ascending sum over the inputs
__device__ __forceinline__ void rotate16_generic(const float raw[16], const float* __restrict__ sH, float v[16]) {
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    float a = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) a = a + raw[i] * sH[i * 16 + j];
    v[j] = a;
  }
}

// Transposed quantizer, one thread per (block of 16 rows, pair of adjacent columns); adjacent lanes read adjacent column
// pairs, so every row of the tile is read as full 128-byte lines; codes and scales of the 64 x 128 tile are staged in
// shared memory and written out as rows of the transposed result.
template <typename T, bool SR>
__global__ void __launch_bounds__(kQThreads, 4) quantize_t3_kernel(const T* __restrict__ x, int64_t M, int64_t K,
                                                                const float* __restrict__ H,
                                                                const float* __restrict__ global, int given,
                                                                float* __restrict__ global_out, uint32_t key,
                                                                uint8_t* __restrict__ codes, uint8_t* __restrict__ scales,
                                                                int layout) {
  __shared__ uint2 s_codes[kTK][kTM / 16 + 1];
  __shared__ uint8_t s_scales[kTK][kTM / 16];
  __shared__ float sH[256];
  bool structured = false;
  if (H != nullptr) {
    sH[threadIdx.x] = H[threadIdx.x];
    __syncthreads();
    const int i = threadIdx.x >> 4, j = threadIdx.x & 15;
    const float si = sH[i * 16];
    const float expect = (__popc(i & j) & 1) ? -si : si;
    structured = __syncthreads_and(fabsf(si) == 0.25f && sH[threadIdx.x] == expect) != 0;
  }
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * kTM, k0 = static_cast<int64_t>(blockIdx.x) * kTK;
  const int kp = threadIdx.x & 31, mb = threadIdx.x >> 5;
  const int64_t k = k0 + 2 * kp, m = m0 + mb * 16;
  const bool active = k < K && m < M;                   // K is even and M a multiple of 16
  if (active) {
    float ra[16], rb[16];
    const T* p = x + m * K + k;
#pragma unroll
    for (int i = 0; i < 16; ++i) load2(p + i * K, ra[i], rb[i]);
    const float g = global_t(global, given);
    if (global_out != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) global_out[0] = g;
    const float rg = __frcp_rn(g);
    float va[16], vb[16];
    if (H == nullptr) {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        va[i] = ra[i];
        vb[i] = rb[i];
      }
    } else if (structured) {
      f32x2 p2[16], v2[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) p2[i] = mul2p(pk(ra[i], rb[i]), pk(sH[i * 16], sH[i * 16]));
      rotate16_tree2(p2, v2);
#pragma unroll
      for (int i = 0; i < 16; ++i) upk(v2[i], va[i], vb[i]);
    } else {
      rotate16_generic(ra, sH, va);
      rotate16_generic(rb, sH, vb);
    }
    uint32_t sb;
    s_codes[2 * kp][mb] =
        quantize_block<SR ? kModeSr : kModeRtn>(va, 1.0f, g, rg, key, static_cast<uint32_t>(static_cast<uint64_t>(k) * M + m), &sb);
    s_scales[2 * kp][mb] = static_cast<uint8_t>(sb);
    s_codes[2 * kp + 1][mb] =
        quantize_block<SR ? kModeSr : kModeRtn>(vb, 1.0f, g, rg, key, static_cast<uint32_t>(static_cast<uint64_t>(k + 1) * M + m), &sb);
    s_scales[2 * kp + 1][mb] = static_cast<uint8_t>(sb);
  }
  __syncthreads();
  // write-out: thread -> (row of the transposed tile, two of its eight blocks)
  const int row = threadIdx.x >> 2, b0 = (threadIdx.x & 3) * 2;
  const int64_t kr = k0 + row;
  if (kr < K) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int64_t mm = m0 + (b0 + e) * 16;
      if (mm < M) {
        *reinterpret_cast<uint2*>(codes + kr * (M / 2) + mm / 2) = s_codes[row][b0 + e];
        scales[scale_index(layout, kr, mm / 16, M / 16)] = s_scales[row][b0 + e];
      }
    }
  }
}

// NVFP4 W [N, K] -> NVFP4 of W^T [K, N]; same tiling, the tile holds (level*scale)*global
__global__ void __launch_bounds__(kQThreads) requantize_t_kernel(const uint8_t* __restrict__ wcodes,
                                                                 const uint8_t* __restrict__ wscales,
                                                                 const float* __restrict__ global, int64_t N, int64_t K,
                                                                 uint8_t* __restrict__ codes, uint8_t* __restrict__ scales,
                                                                 float* __restrict__ global_out, int layout) {
  __shared__ float tile[kTM][kTK + 1];
  const float g = global[0];
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) global_out[0] = g;
  const int64_t n0 = static_cast<int64_t>(blockIdx.y) * kTM, k0 = static_cast<int64_t>(blockIdx.x) * kTK;
  // 128 rows x 8 chunks of 8 columns
  for (int i = threadIdx.x; i < kTM * (kTK / 8); i += kQThreads) {
    const int rr = i / (kTK / 8), c8 = i % (kTK / 8);
    const int64_t n = n0 + rr, k = k0 + c8 * 8;
    if (n < N && k < K) {
      const uint32_t word = *reinterpret_cast<const uint32_t*>(wcodes + n * (K / 2) + k / 2);
      const float s = e4m3_decode(wscales[n * (K / 16) + k / 16]);
#pragma unroll
      for (int j = 0; j < 8; ++j) tile[rr][c8 * 8 + j] = level_of_rank(rank_of_code((word >> (4 * j)) & 0xFu)) * s * g;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) tile[rr][c8 * 8 + j] = 0.0f;
    }
  }
  __syncthreads();
  // one thread per (column k of W, block of 16 rows): lanes walk k, so tile reads are conflict-free
  const float rg = __frcp_rn(g);
  for (int it = 0; it < 2; ++it) {
    const int w = it * kQThreads + threadIdx.x;
    const int kk = w & (kTK - 1), nb = w >> 6;
    const int64_t k = k0 + kk, n = n0 + nb * 16;
    if (!(k < K && n < N)) continue;
    float v[16];
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      v[i] = tile[nb * 16 + i][kk];
      amax = fmaxf(amax, fabsf(v[i]));
    }
    // the reference kernel's own block rule for W^T (csrc/act_quant.cu:66-86): scale amax/6/g, s > 0 ? v/s : 0
    const uint32_t sb = e4m3_encode(div_rn(div_rn(amax, 6.0f, kInv6), g, rg));
    const float se = e4m3_decode(sb) * g;
    const uint2 out = se > 0.0f ? e2m1_rtn16(v, 1.0f, se, rcp_approx(se)) : make_uint2(0u, 0u);
    *reinterpret_cast<uint2*>(codes + k * (N / 2) + n / 2) = out;
    scales[scale_index(layout, k, n / 16, N / 16)] = static_cast<uint8_t>(sb);
  }
}


// ------------------------------------------------------------------------------------------------ dequantize, layout

template <typename O>
__global__ void __launch_bounds__(kQThreads) dequantize_kernel(const uint8_t* __restrict__ codes,
                                                               const uint8_t* __restrict__ scales,
                                                               const float* __restrict__ global, int64_t nchunks,
                                                               O* __restrict__ out) {
  const float g = global[0];
  for (int64_t ch = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; ch < nchunks;
       ch += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const uint32_t word = reinterpret_cast<const uint32_t*>(codes)[ch];
    const float s = e4m3_decode(scales[ch >> 1]) * g;
    O o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = from_f<O>(level_of_rank(rank_of_code((word >> (4 * i)) & 0xFu)) * s);
    if constexpr (sizeof(O) == 4) {
      reinterpret_cast<float4*>(out + ch * 8)[0] = *reinterpret_cast<float4*>(&o[0]);
      reinterpret_cast<float4*>(out + ch * 8)[1] = *reinterpret_cast<float4*>(&o[4]);
    } else {
      *reinterpret_cast<uint4*>(out + ch * 8) = *reinterpret_cast<uint4*>(&o[0]);
    }
  }
}

__global__ void to_blocked_kernel(const uint8_t* __restrict__ scales, int64_t rows, int64_t cols16,
                                  uint8_t* __restrict__ out) {
  const int64_t n = rows * cols16;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / cols16, c = i - r * cols16;
    out[scale_index(BL_SF_BLOCKED, r, c, cols16)] = scales[i];
  }
}

// self-test of div_rn against the plain division on pseudo-random operands (magnitudes 2^-40 .. 2^40, both signs)
__global__ void selftest_division_kernel(uint64_t n, uint32_t seed, unsigned long long* mismatches) {
  unsigned long long bad = 0;
  for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
    uint32_t a = static_cast<uint32_t>(i) * 0x9E3779B1u + seed, b = static_cast<uint32_t>(i >> 7) * 0x85EBCA77u + ~seed;
    a = (a ^ (a >> 15)) * 0x2C1B3C6Du;  a ^= a >> 12;
    b = (b ^ (b >> 13)) * 0x297A2D39u;  b ^= b >> 15;
    const uint32_t ea = 87u + (a >> 9) % 81u, eb = 87u + (b >> 9) % 81u;
    const float x = __uint_as_float((a & 0x807FFFFFu) | (ea << 23));
    // every 128 consecutive i share y, as the kernels share one reciprocal between many quotients
    const float y = __uint_as_float((b & 0x807FFFFFu) | (eb << 23));
    const float q = div_rn(x, y, __frcp_rn(y));
    bad += __float_as_uint(q) != __float_as_uint(x / y);
    // the packed sequence (no range check of its own): both lanes, inside the range its callers establish
    const float x2 = __uint_as_float(__float_as_uint(x) ^ 0x00155555u);
    float q0, q1;
    upk(div2p(pk(x, x2), pk(-y, -y), pk(__frcp_rn(y), __frcp_rn(y))), q0, q1);
    const float qa = fabsf(x / y), qb = fabsf(x2 / y);
    if (qa > 3.2e-30f && qa < 3.1e29f && fabsf(x) > 3.2e-30f)
      bad += __float_as_uint(q0) != __float_as_uint(x / y);
    if (qb > 3.2e-30f && qb < 3.1e29f && fabsf(x2) > 3.2e-30f)
      bad += __float_as_uint(q1) != __float_as_uint(x2 / y);
    // packed multiply and add against the scalar operations
    float m0, m1, s0, s1;
    upk(mul2p(pk(x, x2), pk(y, x)), m0, m1);
    upk(add2p(pk(x, x2), pk(y, -x)), s0, s1);
    bad += __float_as_uint(m0) != __float_as_uint(x * y);
    bad += __float_as_uint(m1) != __float_as_uint(x2 * x);
    bad += __float_as_uint(s0) != __float_as_uint(x + y);
    bad += __float_as_uint(s1) != __float_as_uint(x2 - x);
    // A packed product must not feed a packed sum: the assembler contracts that pair into one fused multiply-add
    // even under --fmad=false. Products that feed sums are therefore formed by the scalar round-to-nearest multiply,
    // which is never contracted, and only then packed; that pattern is checked here.
    float c0, c1;
    upk(add2p(pk(__fmul_rn(x, y), __fmul_rn(x2, y)), pk(x2, x)), c0, c1);
    bad += __float_as_uint(c0) != __float_as_uint(__fadd_rn(__fmul_rn(x, y), x2));
    bad += __float_as_uint(c1) != __float_as_uint(__fadd_rn(__fmul_rn(x2, y), x));
    // ... or by prod2p (a fused multiply-add with a +0 addend), which keeps its own rounding as well
    float e0, e1;
    upk(add2p(prod2p(pk(x, x2), pk(y, y)), pk(x2, x)), e0, e1);
    bad += __float_as_uint(e0) != __float_as_uint(__fadd_rn(__fmul_rn(x, y), x2));
    bad += __float_as_uint(e1) != __float_as_uint(__fadd_rn(__fmul_rn(x2, y), x));
    upk(add2p(pk(x2, x), prod2p(pk(x, x2), pk(x, x2))), e0, e1);
    bad += __float_as_uint(e0) != __float_as_uint(__fadd_rn(x2, __fmul_rn(x, x)));
    bad += __float_as_uint(e1) != __float_as_uint(__fadd_rn(x, __fmul_rn(x2, x2)));
  }
  if (bad) atomicAdd(mismatches, bad);
}

static int grid_for(int64_t work, int threads, int device) {
  const int64_t blocks = (work + threads - 1) / threads;
  const int64_t cap = static_cast<int64_t>(sm_count(device)) * 16;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

static bool blocked_needs_padding(int64_t rows, int64_t cols16) { return (rows % 128) != 0 || (cols16 % 4) != 0; }

}  // namespace blb

using namespace blb;

extern "C" size_t bl_blocked_scale_bytes(int64_t rows, int64_t cols16) {
  if (rows <= 0 || cols16 <= 0) return 0;
  return static_cast<size_t>(((rows + 127) / 128) * ((cols16 + 3) / 4) * 512);
}

extern "C" int bl_nvfp4_amax(const void* x, int dtype, int64_t n, float* out, int device, bl_stream_t stream) {
  BL_REQUIRE(x && out && n > 0, "amax: null or empty input");
  BL_REQUIRE(dtype >= BL_F32 && dtype <= BL_F16, "amax: unknown dtype %d", dtype);
  BL_REQUIRE(aligned16(x) && aligned16(out), "amax: buffers must be 16-byte aligned");
  BL_DEVICE(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  BL_CUDA(cudaMemsetAsync(out, 0, 16, st));
  const int per = dtype == BL_F32 ? 4 : 8;
  const int grid = grid_for(n / per + 1, kQThreads, device);
  if (dtype == BL_BF16) amax_kernel<<<grid, kQThreads, 0, st>>>(static_cast<const __nv_bfloat16*>(x), n, out);
  else if (dtype == BL_F16) amax_kernel<<<grid, kQThreads, 0, st>>>(static_cast<const __half*>(x), n, out);
  else amax_kernel<<<grid, kQThreads, 0, st>>>(static_cast<const float*>(x), n, out);
  BL_CUDA(cudaGetLastError());
  return 0;
}

constexpr int64_t kSeedFosMse = -2, kSeedFosMae = -3;   // internal mode selectors of quantize_rows_typed

template <typename T>
static int quantize_rows_typed(const T* x, int64_t rows, int64_t cols, const float* g, int64_t seed, uint32_t step,
                               uint8_t* codes, uint8_t* scales, int layout, int device, cudaStream_t st) {
  const RowGeometry geo = row_geometry(rows, cols, device);
  if (seed == kSeedFosMse)
    quantize_rows16_kernel<T, kModeFosMse><<<geo.grid, geo.block, 0, st>>>(x, rows, cols, g, 0u, codes, scales, layout);
  else if (seed == kSeedFosMae)
    quantize_rows16_kernel<T, kModeFosMae><<<geo.grid, geo.block, 0, st>>>(x, rows, cols, g, 0u, codes, scales, layout);
  else if (seed < 0)
    quantize_rows16_kernel<T, kModeRtn><<<geo.grid, geo.block, 0, st>>>(x, rows, cols, g, 0u, codes, scales, layout);
  else
    quantize_rows16_kernel<T, kModeSr><<<geo.grid, geo.block, 0, st>>>(x, rows, cols, g,
                                                                       hash_key(static_cast<uint32_t>(seed), step),
                                                                       codes, scales, layout);
  BL_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int bl_nvfp4_quantize(const void* x, int dtype, int64_t rows, int64_t cols, const float* global_scale,
                                 int64_t seed, uint32_t step, uint8_t* codes, uint8_t* scales, int sf_layout,
                                 int device, bl_stream_t stream) {
  BL_REQUIRE(x && global_scale && codes && scales, "quantize_nvfp4: null buffer");
  BL_REQUIRE(rows > 0 && cols > 0 && cols % 16 == 0,
             "quantize_nvfp4: last dimension must be a multiple of 16, got %lld x %lld", (long long)rows, (long long)cols);
  BL_REQUIRE(dtype >= BL_F32 && dtype <= BL_F16, "quantize_nvfp4: unknown dtype %d", dtype);
  BL_REQUIRE(sf_layout == BL_SF_ROWMAJOR || sf_layout == BL_SF_BLOCKED, "quantize_nvfp4: unknown scale layout %d", sf_layout);
  BL_REQUIRE(aligned16(x) && aligned16(codes), "quantize_nvfp4: x and codes must be 16-byte aligned");
  BL_DEVICE(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (seed < 0) seed = -1;                              // any negative seed: round to nearest
  if (sf_layout == BL_SF_BLOCKED && blocked_needs_padding(rows, cols / 16))
    BL_CUDA(cudaMemsetAsync(scales, 0, bl_blocked_scale_bytes(rows, cols / 16), st));
  if (dtype == BL_BF16)
    return quantize_rows_typed(static_cast<const __nv_bfloat16*>(x), rows, cols, global_scale, seed, step, codes, scales, sf_layout, device, st);
  if (dtype == BL_F16)
    return quantize_rows_typed(static_cast<const __half*>(x), rows, cols, global_scale, seed, step, codes, scales, sf_layout, device, st);
  return quantize_rows_typed(static_cast<const float*>(x), rows, cols, global_scale, seed, step, codes, scales, sf_layout, device, st);
}

// The amax pass and the row quantizer against the per-tensor scale it finds, enqueued by one call (what
// bitlattice/backend.py:237-244 does with two operators): amax4 as bl_nvfp4_amax's out, the rest as bl_nvfp4_quantize.
extern "C" int bl_nvfp4_amax_quantize(const void* x, int dtype, int64_t rows, int64_t cols, float* amax4, int64_t seed,
                                      uint32_t step, uint8_t* codes, uint8_t* scales, int sf_layout, int device,
                                      bl_stream_t stream) {
  BL_REQUIRE(rows > 0 && cols > 0, "amax_quantize: empty input");
  if (int rc = bl_nvfp4_amax(x, dtype, rows * cols, amax4, device, stream)) return rc;
  return bl_nvfp4_quantize(x, dtype, rows, cols, amax4 + 1, seed, step, codes, scales, sf_layout, device, stream);
}

extern "C" int bl_nvfp4_quantize_4over6(const void* x, int dtype, int64_t rows, int64_t cols, const float* global_scale,
                                        int select, uint8_t* codes, uint8_t* scales, int sf_layout, int device,
                                        bl_stream_t stream) {
  BL_REQUIRE(x && global_scale && codes && scales, "quantize_4over6: null buffer");
  BL_REQUIRE(rows > 0 && cols > 0 && cols % 16 == 0,
             "quantize_4over6: last dimension must be a multiple of 16, got %lld x %lld", (long long)rows, (long long)cols);
  BL_REQUIRE(dtype >= BL_F32 && dtype <= BL_F16, "quantize_4over6: unknown dtype %d", dtype);
  BL_REQUIRE(select == BL_SELECT_MSE || select == BL_SELECT_MAE, "quantize_4over6: unknown selection rule %d", select);
  BL_REQUIRE(sf_layout == BL_SF_ROWMAJOR || sf_layout == BL_SF_BLOCKED, "quantize_4over6: unknown scale layout %d", sf_layout);
  BL_REQUIRE(aligned16(x) && aligned16(codes), "quantize_4over6: x and codes must be 16-byte aligned");
  BL_DEVICE(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (sf_layout == BL_SF_BLOCKED && blocked_needs_padding(rows, cols / 16))
    BL_CUDA(cudaMemsetAsync(scales, 0, bl_blocked_scale_bytes(rows, cols / 16), st));
  const int64_t mode = select == BL_SELECT_MAE ? kSeedFosMae : kSeedFosMse;
  if (dtype == BL_BF16)
    return quantize_rows_typed(static_cast<const __nv_bfloat16*>(x), rows, cols, global_scale, mode, 0u, codes, scales, sf_layout, device, st);
  if (dtype == BL_F16)
    return quantize_rows_typed(static_cast<const __half*>(x), rows, cols, global_scale, mode, 0u, codes, scales, sf_layout, device, st);
  return quantize_rows_typed(static_cast<const float*>(x), rows, cols, global_scale, mode, 0u, codes, scales, sf_layout, device, st);
}

template <typename T>
static int quantize_t_typed(const T* x, int64_t M, int64_t K, const float* H, int64_t seed, uint32_t step,
                            const float* bound, float* amax_scratch, uint8_t* codes, uint8_t* scales, float* gout,
                            int layout, int device, cudaStream_t st) {
  if (bound == nullptr) {
    BL_CUDA(cudaMemsetAsync(amax_scratch, 0, 16, st));
    amax_t_kernel<<<grid_for((M / 16) * K, kQThreads, device), kQThreads, 0, st>>>(x, M, K, H, amax_scratch);
    BL_CUDA(cudaGetLastError());
  }
  const float* src = bound == nullptr ? amax_scratch : bound;
  int given = bound == nullptr ? 0 : 1;
  float* publish = gout;
  if (static_cast<const void*>(gout) == static_cast<const void*>(src)) {     // in-place: settle the scale first
    global_t_kernel<<<1, 1, 0, st>>>(src, given, gout);
    BL_CUDA(cudaGetLastError());
    src = gout;
    given = 2;
    publish = nullptr;
  }
  const dim3 grid(static_cast<unsigned>((K + kTK - 1) / kTK), static_cast<unsigned>((M + kTM - 1) / kTM));
  const uint32_t key = seed < 0 ? 0u : hash_key(static_cast<uint32_t>(seed), step);
  const bool pairs = K % 2 == 0 && (reinterpret_cast<uintptr_t>(x) % (2 * sizeof(T))) == 0;
  if (pairs && seed < 0) quantize_t3_kernel<T, false><<<grid, kQThreads, 0, st>>>(x, M, K, H, src, given, publish, key, codes, scales, layout);
  else if (pairs) quantize_t3_kernel<T, true><<<grid, kQThreads, 0, st>>>(x, M, K, H, src, given, publish, key, codes, scales, layout);
  else if (seed < 0) quantize_t_kernel<T, false><<<grid, kQThreads, 0, st>>>(x, M, K, H, src, given, publish, key, codes, scales, layout);
  else quantize_t_kernel<T, true><<<grid, kQThreads, 0, st>>>(x, M, K, H, src, given, publish, key, codes, scales, layout);
  BL_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int bl_nvfp4_quantize_t(const void* x, int dtype, int64_t M, int64_t K, const float* H, int64_t seed,
                                   uint32_t step, const float* global_bound, float* amax_scratch, uint8_t* codes,
                                   uint8_t* scales, float* global_out, int sf_layout, int device, bl_stream_t stream) {
  BL_REQUIRE(x && codes && scales && global_out, "quantize_nvfp4_t: null buffer");
  BL_REQUIRE(M > 0 && K > 0 && M % 16 == 0, "quantize_nvfp4_t: rows must be a multiple of 16, got %lld x %lld",
             (long long)M, (long long)K);
  BL_REQUIRE((M / 16) <= 65535 * 8, "quantize_nvfp4_t: too many rows (%lld)", (long long)M);
  BL_REQUIRE(global_bound != nullptr || amax_scratch != nullptr,
             "quantize_nvfp4_t: without a scale bound the amax pass needs a 4-float scratch buffer");
  BL_REQUIRE(dtype >= BL_F32 && dtype <= BL_F16, "quantize_nvfp4_t: unknown dtype %d", dtype);
  BL_REQUIRE(sf_layout == BL_SF_ROWMAJOR || sf_layout == BL_SF_BLOCKED, "quantize_nvfp4_t: unknown scale layout %d", sf_layout);
  BL_REQUIRE(aligned16(codes), "quantize_nvfp4_t: codes must be 16-byte aligned");
  BL_DEVICE(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (sf_layout == BL_SF_BLOCKED && blocked_needs_padding(K, M / 16))
    BL_CUDA(cudaMemsetAsync(scales, 0, bl_blocked_scale_bytes(K, M / 16), st));
  if (dtype == BL_BF16)
    return quantize_t_typed(static_cast<const __nv_bfloat16*>(x), M, K, H, seed, step, global_bound, amax_scratch, codes, scales, global_out, sf_layout, device, st);
  if (dtype == BL_F16)
    return quantize_t_typed(static_cast<const __half*>(x), M, K, H, seed, step, global_bound, amax_scratch, codes, scales, global_out, sf_layout, device, st);
  return quantize_t_typed(static_cast<const float*>(x), M, K, H, seed, step, global_bound, amax_scratch, codes, scales, global_out, sf_layout, device, st);
}

extern "C" int bl_nvfp4_requantize_t(const uint8_t* codes, const uint8_t* scales, const float* global_scale, int64_t N,
                                     int64_t K, uint8_t* out_codes, uint8_t* out_scales, float* global_out,
                                     int sf_layout, int device, bl_stream_t stream) {
  BL_REQUIRE(codes && scales && global_scale && out_codes && out_scales && global_out, "requantize_nvfp4_t: null buffer");
  BL_REQUIRE(N > 0 && K > 0 && N % 16 == 0 && K % 16 == 0,
             "requantize_nvfp4_t: both dimensions must be multiples of 16, got %lld x %lld", (long long)N, (long long)K);
  BL_REQUIRE(sf_layout == BL_SF_ROWMAJOR || sf_layout == BL_SF_BLOCKED, "requantize_nvfp4_t: unknown scale layout %d", sf_layout);
  BL_REQUIRE(aligned16(codes) && aligned16(out_codes), "requantize_nvfp4_t: code buffers must be 16-byte aligned");
  BL_DEVICE(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (sf_layout == BL_SF_BLOCKED && blocked_needs_padding(K, N / 16))
    BL_CUDA(cudaMemsetAsync(out_scales, 0, bl_blocked_scale_bytes(K, N / 16), st));
  const dim3 grid(static_cast<unsigned>((K + kTK - 1) / kTK), static_cast<unsigned>((N + kTM - 1) / kTM));
  requantize_t_kernel<<<grid, kQThreads, 0, st>>>(codes, scales, global_scale, N, K, out_codes, out_scales, global_out,
                                                  sf_layout);
  BL_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int bl_nvfp4_dequantize(const uint8_t* codes, const uint8_t* scales, const float* global_scale, int64_t rows,
                                   int64_t cols, void* out, int out_dtype, int device, bl_stream_t stream) {
  BL_REQUIRE(codes && scales && global_scale && out, "dequantize: null buffer");
  BL_REQUIRE(rows > 0 && cols > 0 && cols % 16 == 0, "dequantize: last dimension must be a multiple of 16, got %lld x %lld",
             (long long)rows, (long long)cols);
  BL_REQUIRE(out_dtype >= BL_F32 && out_dtype <= BL_F16, "dequantize: unknown output dtype %d", out_dtype);
  BL_REQUIRE(aligned16(codes) && aligned16(out), "dequantize: codes and output must be 16-byte aligned");
  BL_DEVICE(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int64_t nchunks = rows * cols / 8;
  const int grid = grid_for(nchunks, kQThreads, device);
  if (out_dtype == BL_BF16)
    dequantize_kernel<<<grid, kQThreads, 0, st>>>(codes, scales, global_scale, nchunks, static_cast<__nv_bfloat16*>(out));
  else if (out_dtype == BL_F16)
    dequantize_kernel<<<grid, kQThreads, 0, st>>>(codes, scales, global_scale, nchunks, static_cast<__half*>(out));
  else
    dequantize_kernel<<<grid, kQThreads, 0, st>>>(codes, scales, global_scale, nchunks, static_cast<float*>(out));
  BL_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int bl_nvfp4_scales_to_blocked(const uint8_t* scales, int64_t rows, int64_t cols16, uint8_t* out, int device,
                                          bl_stream_t stream) {
  BL_REQUIRE(scales && out && rows > 0 && cols16 > 0, "scales_to_blocked: null or empty input");
  BL_DEVICE(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (blocked_needs_padding(rows, cols16)) BL_CUDA(cudaMemsetAsync(out, 0, bl_blocked_scale_bytes(rows, cols16), st));
  to_blocked_kernel<<<grid_for(rows * cols16, kQThreads, device), kQThreads, 0, st>>>(scales, rows, cols16, out);
  BL_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int bl_selftest_division(uint64_t n, uint32_t seed, uint64_t* mismatches, int device) {
  BL_REQUIRE(mismatches != nullptr && n > 0, "selftest_division: null output or empty range");
  BL_DEVICE(device);
  unsigned long long* d = nullptr;
  BL_CUDA(cudaMalloc(&d, sizeof(unsigned long long)));
  cudaError_t rc = cudaMemset(d, 0, sizeof(unsigned long long));
  if (rc == cudaSuccess) {
    selftest_division_kernel<<<sm_count(device) * 8, 256>>>(n, seed, d);
    rc = cudaGetLastError();
  }
  unsigned long long h = 0;
  if (rc == cudaSuccess) rc = cudaMemcpy(&h, d, sizeof(h), cudaMemcpyDeviceToHost);
  cudaFree(d);
  BL_CUDA(rc);
  *mismatches = h;
  return 0;
}
