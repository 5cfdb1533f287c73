// The general NVFP4 operand quantizer of the 128-rotation recipes, and the scale folding of deferred weight gradients.
//
// Reference semantics: bitlattice/fp4ref.py:103-150 (round to nearest with ties to the even code, stochastic rounding,
// MS-EDEN, four-over-six block scales, the randomized 128-point Hadamard rotation); the reference's operator is
// torch.ops.bitlattice.nvfp4_quantize (csrc/nvfp4.cu:553-600), its scale folding csrc/fold.cu:12-33 /
// bitlattice/backend.py:665-700. The reference's own test allows 2e-3 of codes and scales to differ between its kernel
// and fp4ref because neither fixes a summation order; this file fixes one (compiled with --fmad=false):
//   rotation   x * signs, fast Walsh-Hadamard butterflies with strides 1, 2, ..., 64, then times fp32(1 / sqrt(128))
//   4/6 error  per block: sequential sums over elements 4q .. 4q + 3, then (s0 + s1) + (s2 + s3)
//   MS-EDEN    <x, x> and <x, x_rtn> per 128: sequential sums over 4 elements, then a pairwise tree (neighbours first)
//
// Thread mapping: a lane owns one 16-element block, eight neighbouring lanes one 128-element segment of an output row,
// a warp four rows' segments at a time. Strides 1 .. 8 of the rotation run in registers, strides 16 .. 64 are shuffles
// over lane distances 1, 2, 4; block scales, four-over-six errors and stochastic draws need no exchange, the MS-EDEN
// sums three shuffle steps. A CTA covers 128 output columns x 64 output rows; for transposed output it first stages
// the 128 x 64 source tile (dense values, or NVFP4 codes decoded as (level * scale) * global) in shared memory.
#include <type_traits>

#include "common.cuh"

namespace blb {

constexpr int kGenThreads = 256;
constexpr int kGenTileRows = 64;
constexpr float kInvSqrt128 = 0.08838834764831845f;

enum { kSrcRows = 0, kSrcTransposed = 1, kSrcPackedTransposed = 2 };

struct GenArgs {
  const void* x;              // dense [R, C], or packed codes [R, C / 2]
  const uint8_t* w_scales;    // packed input: its row-major scale bytes [R, C / 16]
  const float* w_global;      // packed input: its per-tensor scale
  int64_t R, C;               // source shape
  int64_t rows, cols;         // output shape: (R, C) or (C, R)
  int mode, fos, mae, rotate, pow2;
  uint32_t key, eden_key, rot_key;
  const float* given;         // per-tensor scale to use, or null: from amax[0]
  float* amax;                // max |value| after the rotation (pass 0 writes, pass 1 reads)
  float* amax_out;            // or null: receives that maximum also when the per-tensor scale is given (delayed scales)
  float* out_global;
  uint8_t* codes;
  uint8_t* scales;
  int layout;
};

__device__ __forceinline__ float general_global(const GenArgs& A) {
  if (A.given) return A.given[0];
  float g = fmaxf(A.amax[0] / (A.fos ? 1536.0f : 2688.0f), 1e-12f);
  if (A.pow2) {                                            // up to the next power of two (g is a normal number)
    uint32_t b = __float_as_uint(g);
    if (b & 0x007FFFFFu) b = (b & 0x7F800000u) + 0x00800000u;
    g = __uint_as_float(b);
  }
  return g;
}

// levels of the eight codes of w (element i in nibble i)
__device__ __forceinline__ void e2m1_levels8(uint32_t w, float out[8]) {
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    uint32_t h2;
    asm("{\n\t.reg .b8 b;\n\tcvt.u8.u32 b, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, b;\n\t}" : "=r"(h2) : "r"(w >> (8 * k)));
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h2));
    out[2 * k] = f.x;
    out[2 * k + 1] = f.y;
  }
}

// round-to-nearest codes (ties to the even code, saturating) of v[i] * inv for a block of 16
__device__ __forceinline__ uint2 e2m1_nearest16(const float v[16], float inv) {
  float q[16];
#pragma unroll
  for (int i = 0; i < 16; i += 2) mul2(v[i], v[i + 1], inv, q[i], q[i + 1]);
  return make_uint2(cvt_e2m1x8_merged(q), cvt_e2m1x8_merged(q + 8));
}

// error of a candidate: sum over the block of (level * t - v)^2 (or | |), four sequential sums over elements
// 4q .. 4q + 3, then (s0 + s1) + (s2 + s3)
__device__ __forceinline__ float candidate_error(const float v[16], uint2 codes, float t, bool mae) {
  float d[16];
  e2m1_levels8(codes.x, d);
  e2m1_levels8(codes.y, d + 8);
  float s[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    float acc = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float e = d[4 * q + i] * t - v[4 * q + i];
      acc = acc + (mae ? fabsf(e) : e * e);
    }
    s[q] = acc;
  }
  return (s[0] + s[1]) + (s[2] + s[3]);
}

// stochastic rounding to E4M3 of a positive value (bitlattice/fp4ref.py:81-88)
__device__ __forceinline__ uint32_t e4m3_sr(float v, float u) {
  v = fminf(fmaxf(v, 0.001953125f), 448.0f);
  uint32_t b = e4m3_encode(v);
  float lo = e4m3_decode(b);
  if (lo > v) {
    b = b > 1u ? b - 1u : 1u;
    lo = e4m3_decode(b);
  }
  const uint32_t hb = b < 0x7Eu ? b + 1u : 0x7Eu;
  const float hi = e4m3_decode(hb);
  const float p = hi > lo ? (v - lo) / (hi - lo) : 0.0f;
  return u < p ? hb : b;
}

// PASS 0: max |value| of the (rotated) output into A.amax[0] (zeroed by the host). PASS 1: codes and scales.
// A warp works on four output rows at a time: lanes 8c .. 8c + 7 hold the eight 16-element blocks of row c's segment.
template <typename T, int SRC, int PASS>
__global__ void __launch_bounds__(kGenThreads) general_kernel(GenArgs A) {
  __shared__ float tile[SRC == kSrcRows ? 1 : 128 * 65];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane >> 3, blk = lane & 7;               // row of the warp's group of four, block of the segment
  const int64_t col0 = static_cast<int64_t>(blockIdx.x) * 128;         // first output column of the segment
  const int64_t row0 = static_cast<int64_t>(blockIdx.y) * kGenTileRows;  // first output row of the tile

  if constexpr (SRC != kSrcRows) {
    // source rows col0 .. col0 + 127 (output columns), source columns row0 .. row0 + 63 (output rows):
    // thread t stages 32 consecutive source elements of source row t / 2
    const int sr = threadIdx.x >> 1, sc0 = (threadIdx.x & 1) * 32;
    const int64_t src_row = col0 + sr, src_col = row0 + sc0;
    float* dst = tile + sr * 65 + sc0;
    const bool inside = src_row < A.R && src_col + 32 <= A.C;
    if constexpr (SRC == kSrcTransposed) {
      const T* x = static_cast<const T*>(A.x);
      if (inside && (A.C % 8) == 0) {
#pragma unroll
        for (int j = 0; j < 4; ++j) load8(x + src_row * A.C + src_col + 8 * j, dst + 8 * j);
      } else {
        for (int j = 0; j < 32; ++j)
          dst[j] = (src_row < A.R && src_col + j < A.C) ? to_f<T>(x[src_row * A.C + src_col + j]) : 0.0f;
      }
    } else {
      if (inside) {
        const uint8_t* codes = static_cast<const uint8_t*>(A.x);
        const uint4 cw = *reinterpret_cast<const uint4*>(codes + src_row * (A.C / 2) + src_col / 2);
        const uint32_t w[4] = {cw.x, cw.y, cw.z, cw.w};
        const float gw = A.w_global[0];
        const float s0 = e4m3_decode(A.w_scales[src_row * (A.C / 16) + src_col / 16]);
        const float s1 = e4m3_decode(A.w_scales[src_row * (A.C / 16) + src_col / 16 + 1]);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const uint32_t c = (w[j >> 3] >> (4 * (j & 7))) & 15u;
          const float m = mag_of(c & 7u);
          dst[j] = ((c & 8u ? -m : m) * (j < 16 ? s0 : s1)) * gw;
        }
      } else {
        for (int j = 0; j < 32; ++j) dst[j] = 0.0f;
      }
    }
    __syncthreads();
  }

  const bool valid_col = col0 + 16 * blk < A.cols;         // cols is a multiple of 16: a whole block or none
  uint32_t neg = 0;                                        // bit i: the rotation negates element i of this lane
  if (A.rotate) {
#pragma unroll
    for (int i = 0; i < 16; ++i)
      neg |= (hash_uniform(static_cast<uint32_t>(16 * blk + i), A.rot_key) < 0.5f ? 1u : 0u) << i;
  }
  const float g = PASS == 1 ? general_global(A) : 1.0f;
  if (PASS == 1 && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) {
    A.out_global[0] = g;
    if (A.amax_out && !A.given) A.amax_out[0] = A.amax[0];
  }
  const bool observe = PASS == 1 && A.amax_out && A.given;     // no amax pass ran: observe the maximum here
  float wmax = 0.0f;

  for (int j = 0; j < kGenTileRows / 32; ++j) {
    const int rr = 4 * (warp + 8 * j) + sub;
    const int64_t r = row0 + rr;
    if (row0 + 4 * (warp + 8 * j) >= A.rows) break;        // the same for every lane of the warp
    const bool valid = valid_col && r < A.rows;
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = 0.0f;
    if (valid) {
      if constexpr (SRC == kSrcRows) {
        const T* p = static_cast<const T*>(A.x) + r * A.C + col0 + 16 * blk;
        if ((A.C % 8) == 0) {
          load8(p, v);
          load8(p + 8, v + 8);
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = to_f<T>(p[i]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = tile[(16 * blk + i) * 65 + rr];
      }
    }
    if (A.rotate) {
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(__float_as_uint(v[i]) ^ (((neg >> i) & 1u) << 31));
#pragma unroll
      for (int h = 1; h < 16; h <<= 1) {                                               // strides 1 .. 8
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          if ((i & h) == 0) {
            const float a = v[i], b = v[i + h];
            v[i] = a + b;
            v[i + h] = a - b;
          }
        }
      }
#pragma unroll
      for (int m = 1; m < 8; m <<= 1) {                                                // strides 16 .. 64
        const float sgn = (blk & m) ? -1.0f : 1.0f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float p = __shfl_xor_sync(0xffffffffu, v[i], m);
          v[i] = fmaf(v[i], sgn, p);                       // a + b below, a - b above: one rounding either way
        }
      }
#pragma unroll
      for (int i = 0; i < 16; i += 2) mul2(v[i], v[i + 1], kInvSqrt128, v[i], v[i + 1]);
    }
    float am = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) am = fmaxf(am, fabsf(v[i]));
    if constexpr (PASS == 0) {
      wmax = fmaxf(wmax, am);
    } else {
      if (observe) wmax = fmaxf(wmax, am);
      uint32_t sb = e4m3_encode(am / 6.0f / g);
      float t = e4m3_decode(sb) * g;
      float inv = t > 0.0f ? 1.0f / t : 0.0f;
      uint2 codes = e2m1_nearest16(v, inv);
      if (A.fos) {
        const uint32_t sb4 = e4m3_encode(am / 4.0f / g);
        const float t4 = e4m3_decode(sb4) * g;
        const float inv4 = t4 > 0.0f ? 1.0f / t4 : 0.0f;
        const uint2 codes4 = e2m1_nearest16(v, inv4);
        const float e6 = candidate_error(v, codes, t, A.mae != 0), e4 = candidate_error(v, codes4, t4, A.mae != 0);
        if (e4 < e6) {
          sb = sb4;
          t = t4;
          inv = inv4;
          codes = codes4;
        }
      }
      if (A.mode == BL_Q_SR) {
        const uint32_t idx0 = static_cast<uint32_t>(static_cast<uint64_t>(r) * static_cast<uint64_t>(A.cols) +
                                                    static_cast<uint64_t>(col0 + 16 * blk));
        codes = e2m1_sr16(v, inv, A.key, idx0);
      } else if (A.mode == BL_Q_EDEN) {
        float d[16];
        e2m1_levels8(codes.x, d);
        e2m1_levels8(codes.y, d + 8);
        float sx[4], sr[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float ax = 0.0f, ar = 0.0f;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            ax = ax + v[4 * q + i] * v[4 * q + i];
            ar = ar + v[4 * q + i] * (d[4 * q + i] * t);
          }
          sx[q] = ax;
          sr[q] = ar;
        }
        float xx = (sx[0] + sx[1]) + (sx[2] + sx[3]), xr = (sr[0] + sr[1]) + (sr[2] + sr[3]);
#pragma unroll
        for (int m = 1; m < 8; m <<= 1) {
          xx = xx + __shfl_xor_sync(0xffffffffu, xx, m);
          xr = xr + __shfl_xor_sync(0xffffffffu, xr, m);
        }
        const float S = xr != 0.0f ? xx / xr : 1.0f;
        const uint32_t block = static_cast<uint32_t>(static_cast<uint64_t>(r) * static_cast<uint64_t>(A.cols / 16) +
                                                     static_cast<uint64_t>((col0 + 16 * blk) / 16));
        sb = e4m3_sr(e4m3_decode(sb) * S, hash_uniform(block, A.eden_key));
      }
      if (valid) {
        codes.x = e2m1_drop_negative_zero(codes.x);
        codes.y = e2m1_drop_negative_zero(codes.y);
        *reinterpret_cast<uint2*>(A.codes + r * (A.cols / 2) + (col0 + 16 * blk) / 2) = codes;
        const int64_t c16 = (col0 + 16 * blk) / 16, cols16 = A.cols / 16;
        int64_t at = r * cols16 + c16;
        if (A.layout != BL_SF_ROWMAJOR) {
          const int64_t nc = (cols16 + 3) >> 2;
          at = ((r >> 7) * nc + (c16 >> 2)) * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (c16 & 3);
        }
        A.scales[at] = static_cast<uint8_t>(sb);
      }
    }
  }
  if (PASS == 0 || observe) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) wmax = fmaxf(wmax, __shfl_xor_sync(0xffffffffu, wmax, o));
    if (lane == 0 && wmax > 0.0f) atomicMax(reinterpret_cast<int*>(PASS == 0 ? A.amax : A.amax_out), __float_as_int(wmax));
  }
}

// Scales of deferred weight-gradient operands brought to a common per-tensor scale: piece j (one micro-batch) has the
// power-of-two scale g[j]; every scale byte of its 512-byte tiles is multiplied by g[j] / max(g) and rounded to E4M3
// (exact while the product stays a normal number); non-zero products below 2^-6 are counted.
__global__ void __launch_bounds__(256) fold_scales_kernel(uint8_t* __restrict__ scales, int64_t tiles,
                                                          const int* __restrict__ piece, const float* __restrict__ g,
                                                          int pieces, int64_t tiles_per_row, float* __restrict__ g_max,
                                                          unsigned long long* __restrict__ rounded) {
  float top = 0.0f;
  for (int j = 0; j < pieces; ++j) top = fmaxf(top, g[j]);
  if (blockIdx.x == 0 && threadIdx.x == 0) g_max[0] = top;
  unsigned long long count = 0;
  const int64_t total = tiles * 512;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const float f = g[piece[(i / 512) % tiles_per_row]] / top;
    if (f == 1.0f) continue;
    const float v = e4m3_decode(scales[i]) * f;
    if (v > 0.0f && v < 0.015625f) ++count;
    const __nv_fp8_e4m3 q(v);
    scales[i] = q.__x;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) count += __shfl_xor_sync(0xffffffffu, count, o);
  if ((threadIdx.x & 31) == 0 && count) atomicAdd(rounded, count);
}

template <typename T>
static int general_typed(GenArgs A, bool packed, bool transpose, bool need_amax, cudaStream_t st) {
  const dim3 grid(static_cast<unsigned>((A.cols + 127) / 128), static_cast<unsigned>((A.rows + kGenTileRows - 1) / kGenTileRows));
  if (need_amax) {
    BL_CUDA(cudaMemsetAsync(A.amax, 0, sizeof(float), st));
    if (packed) general_kernel<uint8_t, kSrcPackedTransposed, 0><<<grid, kGenThreads, 0, st>>>(A);
    else if (transpose) general_kernel<T, kSrcTransposed, 0><<<grid, kGenThreads, 0, st>>>(A);
    else general_kernel<T, kSrcRows, 0><<<grid, kGenThreads, 0, st>>>(A);
  }
  if (packed) general_kernel<uint8_t, kSrcPackedTransposed, 1><<<grid, kGenThreads, 0, st>>>(A);
  else if (transpose) general_kernel<T, kSrcTransposed, 1><<<grid, kGenThreads, 0, st>>>(A);
  else general_kernel<T, kSrcRows, 1><<<grid, kGenThreads, 0, st>>>(A);
  BL_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace blb

using namespace blb;

extern "C" int bl_nvfp4_quantize_general(const void* x, int dtype, int64_t R, int64_t C, int transpose, int mode,
                                         int four_over_six, int select, int rotate, int64_t seed, int64_t rotate_seed,
                                         const float* given_global, int pow2, const uint8_t* w_scales,
                                         const float* w_global, uint8_t* codes, uint8_t* scales, int sf_layout,
                                         float* out_global, float* scratch, float* amax_out, int device,
                                         bl_stream_t stream) {
  BL_REQUIRE(x && codes && scales && out_global && scratch, "quantize_general: null buffer");
  BL_REQUIRE(R > 0 && C > 0 && R < (1ll << 31) && C < (1ll << 31), "quantize_general: bad shape %lld x %lld",
             (long long)R, (long long)C);
  BL_REQUIRE(mode >= BL_Q_RTN && mode <= BL_Q_EDEN, "quantize_general: unknown mode %d", mode);
  BL_REQUIRE(select == BL_SELECT_MSE || select == BL_SELECT_MAE, "quantize_general: unknown selection %d", select);
  BL_REQUIRE(sf_layout == BL_SF_ROWMAJOR || sf_layout == BL_SF_BLOCKED, "quantize_general: unknown scale layout %d", sf_layout);
  const bool packed = w_scales != nullptr;
  BL_REQUIRE(!packed || (w_global && transpose), "quantize_general: NVFP4 input is re-quantized transposed and needs its "
             "per-tensor scale");
  BL_REQUIRE(!packed || C % 32 == 0, "quantize_general: NVFP4 input needs a multiple of 32 columns, got %lld", (long long)C);
  BL_REQUIRE(packed || (dtype >= BL_F32 && dtype <= BL_F16), "quantize_general: unknown dtype %d", dtype);
  const int64_t rows = transpose ? C : R, cols = transpose ? R : C;
  BL_REQUIRE(cols % 16 == 0, "quantize_general: the quantized dimension %lld is not a multiple of 16", (long long)cols);
  BL_REQUIRE(!rotate || cols % 128 == 0, "quantize_general: the rotation needs a multiple of 128 along the quantized "
             "dimension, got %lld", (long long)cols);
  BL_REQUIRE(mode != BL_Q_EDEN || rotate, "quantize_general: MS-EDEN needs the rotation");
  BL_REQUIRE((rows + kGenTileRows - 1) / kGenTileRows <= 65535, "quantize_general: too many rows (%lld)", (long long)rows);
  BL_REQUIRE(aligned16(x) && aligned16(codes), "quantize_general: input and codes must be 16-byte aligned");
  BL_REQUIRE(packed || transpose || C % 4 == 0, "quantize_general: row length must be a multiple of 4");
  BL_DEVICE(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  GenArgs A;
  A.x = x;
  A.w_scales = w_scales;
  A.w_global = w_global;
  A.R = R;
  A.C = C;
  A.rows = rows;
  A.cols = cols;
  A.mode = mode;
  A.fos = four_over_six ? 1 : 0;
  A.mae = select == BL_SELECT_MAE ? 1 : 0;
  A.rotate = rotate ? 1 : 0;
  A.pow2 = pow2 ? 1 : 0;
  const uint32_t s32 = static_cast<uint32_t>(seed);
  const uint32_t r32 = static_cast<uint32_t>(rotate_seed < 0 ? seed : rotate_seed);
  A.key = hash_key(s32, 0u);
  A.eden_key = hash_key(s32 ^ 0x9E3779B9u, 0u);
  A.rot_key = hash_key(r32, 0x5151u);
  A.given = given_global;
  A.amax = scratch;
  A.amax_out = amax_out;
  A.out_global = out_global;
  A.codes = codes;
  A.scales = scales;
  A.layout = sf_layout;
  if (sf_layout == BL_SF_BLOCKED && ((rows % 128) != 0 || ((cols / 16) % 4) != 0))
    BL_CUDA(cudaMemsetAsync(scales, 0, bl_blocked_scale_bytes(rows, cols / 16), st));
  const bool need_amax = given_global == nullptr;
  if (amax_out && !need_amax) BL_CUDA(cudaMemsetAsync(amax_out, 0, sizeof(float), st));
  if (packed || dtype == BL_BF16) return general_typed<__nv_bfloat16>(A, packed, transpose != 0, need_amax, st);
  if (dtype == BL_F16) return general_typed<__half>(A, packed, transpose != 0, need_amax, st);
  return general_typed<float>(A, packed, transpose != 0, need_amax, st);
}

extern "C" int bl_fp4_fold_scales(uint8_t* scales, int64_t row_tiles, int64_t tiles_per_row, const int* piece,
                                  const float* g, int pieces, float* g_max, unsigned long long* rounded, int device,
                                  bl_stream_t stream) {
  BL_REQUIRE(scales && piece && g && g_max && rounded, "fold_scales: null buffer");
  BL_REQUIRE(row_tiles > 0 && tiles_per_row > 0 && pieces > 0, "fold_scales: empty input");
  BL_DEVICE(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int64_t tiles = row_tiles * tiles_per_row;
  const int64_t want = (tiles * 512 + 255) / 256;
  const unsigned grid = static_cast<unsigned>(want < 4096 ? want : 4096);
  fold_scales_kernel<<<grid, 256, 0, st>>>(scales, tiles, piece, g, pieces, tiles_per_row, g_max, rounded);
  BL_CUDA(cudaGetLastError());
  return 0;
}
