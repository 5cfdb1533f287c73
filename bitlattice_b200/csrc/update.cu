// Lattice optimizer update of NVFP4 weights: phase accumulation, group-scale refit inside the trust region and
// stochastic projection back to (code, phase), with the update direction (raw / sign / colnorm + RMS clip) computed
// from the gradient inside the same kernel, so the fp32 direction never exists in memory.
//
// Reference semantics: bitlattice/reference.py:250-335 (lattice_step_quantized, _project, latent),
// bitlattice/_ops.py:135-144 and bitlattice/reference.py:488-490 (directions); the reference's kernels are
// csrc/lattice.cu:56-175 and csrc/directions.cpp:145-191. Compiled with --fmad=false: every fp32 operation rounds
// on its own, in the reference's order.
//
// Data layout in HBM (all row-major over the weight's [rows, cols] view, cols % 16 == 0):
//   codes  [rows, cols/2] bytes, phase [rows, cols*cb/8] bytes, scales [rows, cols/16] bytes, grad [rows, cols].
// One thread owns one 16-element scale group of a row (two 32-bit code words, 2 cb bytes of phase, 32 or 64 bytes of
// gradient, one scale byte) and needs no communication with other threads. A thread keeps its 16 columns while it
// walks down the rows, so per-column statistics (colnorm) stay in registers.
#include <mutex>

#include "common.cuh"

namespace blb {

constexpr int kPanelRows = 128;   // rows summed sequentially into one partial column sum
constexpr int kThreads = 256;

// scratch layout (bytes), see bl_update_scratch_bytes
struct Scratch {
  float* partial;   // [npanels, cols] partial column sums of U0^2
  float* denom;     // [cols]          colnorm denominators
  double* chunk;    // [nchunks]       per-256-column partial sums of the RMS
  float* stats;     // [0] rho, [1] divisor max(rho/clip, 1)
  unsigned* ticket; // arrival counter of the finalize kernel
  size_t bytes;
};

static Scratch scratch_layout(void* base, int64_t rows, int64_t cols) {
  const int64_t npanels = (rows + kPanelRows - 1) / kPanelRows;
  const int64_t nchunks = (cols + 255) / 256;
  char* p = static_cast<char*>(base);
  size_t off = 0;
  auto take = [&](size_t n) {
    char* q = p ? p + off : nullptr;
    off += (n + 255) & ~size_t(255);
    return q;
  };
  Scratch s;
  s.partial = reinterpret_cast<float*>(take(static_cast<size_t>(npanels * cols) * 4));
  s.denom = reinterpret_cast<float*>(take(static_cast<size_t>(cols) * 4));
  s.chunk = reinterpret_cast<double*>(take(static_cast<size_t>(nchunks) * 8));
  s.stats = reinterpret_cast<float*>(take(16));
  s.ticket = reinterpret_cast<unsigned*>(take(16));
  s.bytes = off;
  return s;
}

static bool needs_stats(int direction, double clip) { return !(direction == BL_DIR_SIGN && clip >= 1.0); }

// ------------------------------------------------------------------------------------------------ column statistics

// partial[p][c] = sum over the rows of panel p, in ascending order, of U0[r][c]^2; U0 = G or sign(G)
template <typename GT, bool SIGN>
__global__ void __launch_bounds__(kThreads) colstats_kernel(const GT* __restrict__ G, int64_t rows, int64_t cols,
                                                            float* __restrict__ partial) {
  const int64_t cc = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (cc * 8 >= cols) return;
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * kPanelRows;
  const int64_t r1 = min(rows, r0 + kPanelRows);
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
  const GT* p = G + r0 * cols + cc * 8;
#pragma unroll 4
  for (int64_t r = r0; r < r1; ++r, p += cols) {
    float v[8];
    load8(p, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float u = v[i];
      if (SIGN) u = static_cast<float>((u > 0.0f) - (u < 0.0f));
      acc[i] = acc[i] + u * u;
    }
  }
  float* out = partial + static_cast<int64_t>(blockIdx.y) * cols + cc * 8;
  reinterpret_cast<float4*>(out)[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
  reinterpret_cast<float4*>(out)[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
}

// colsq[c] = ascending sum of the panel partials; colnorm: denom[c] = sqrt(colsq/rows) + 1e-30 and the column's sum
// of U^2 is taken as colsq / denom^2. The RMS sums 256-column chunks with a fixed halving tree in double, then the
// chunks in ascending order; the last block to arrive publishes rho and the divisor.
__global__ void __launch_bounds__(256) finalize_kernel(const float* __restrict__ partial, int64_t rows, int64_t cols,
                                                       int npanels, int colnorm, float clip, float* __restrict__ denom,
                                                       double* __restrict__ chunk, float* __restrict__ stats,
                                                       unsigned* __restrict__ ticket) {
  __shared__ double red[256];
  __shared__ bool last;
  const int64_t c = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
  double colu = 0.0;
  if (c < cols) {
    float tot = 0.0f;
    for (int p = 0; p < npanels; ++p) tot = tot + partial[static_cast<int64_t>(p) * cols + c];
    if (colnorm) {
      const float d = sqrtf(tot / static_cast<float>(rows)) + 1e-30f;
      denom[c] = d;
      colu = static_cast<double>(tot / (d * d));
    } else {
      colu = static_cast<double>(tot);
    }
  }
  red[threadIdx.x] = colu;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if (threadIdx.x < s) red[threadIdx.x] = red[threadIdx.x] + red[threadIdx.x + s];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    chunk[blockIdx.x] = red[0];
    __threadfence();
    last = atomicAdd(ticket, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (last && threadIdx.x == 0) {
    __threadfence();
    double acc = 0.0;
    for (unsigned i = 0; i < gridDim.x; ++i) acc = acc + reinterpret_cast<volatile double*>(chunk)[i];
    const float rho = static_cast<float>(sqrt(acc / (static_cast<double>(rows) * static_cast<double>(cols))));
    stats[0] = rho;
    stats[1] = fmaxf(rho / clip, 1.0f);
    *ticket = 0u;
  }
}

// ------------------------------------------------------------------------------------------------ the update

struct StepParams {
  float lr, decay;
  int pb;            // phase bits 0..8
  int rule;          // BL_RULE_*
  float r_lo, r_hi;  // exp(-kappa), exp(+kappa)
  RoundParams rp;
  uint32_t offset;   // RNG index of element (0, 0), low 32 bits
};

// ---- per-thread work unit: one scale group of 16 consecutive elements ------------------------------------------------
// A thread loads the group's 8 code bytes, its phase bytes, its 16 gradient values and the scale byte, keeps its 16
// columns while it walks down the rows, and needs no communication with other threads.
//
// Exactness notes (every shortcut below returns the reference's bits; the parity tests compare bit for bit):
//  * (a, latent) of an element depend only on its code nibble and phase bits: a shared-memory table built with the
//    reference's formula at kernel start replaces the per-element level / neighbour / latent arithmetic;
//  * divisions sharing a divisor (the old and new group scale, a column's denominator, the RMS divisor) go through
//    div_rn with one correctly rounded reciprocal per divisor;
//  * the nearest level comes from the hardware E2M1 conversion (ties to even). The reference breaks ties to the lower
//    level, but the projection is invariant to that choice: a target exactly half-way between levels L < U gives
//    (U, phase -half) from either side (from L the phase code reaches +half and carries over), and with 0 phase bits
//    both sides draw U with probability 1/2 from the same random number;
//  * gaps between neighbouring levels are powers of two read off the exponent of the level, so dividing by a half
//    gap is a multiplication by an exact reciprocal and (t - w) / width needs no clamp (|t - w| <= width).

template <int PCB> struct PhaseWord;
template <> struct PhaseWord<0> { using type = uint32_t; };
template <> struct PhaseWord<1> { using type = uint16_t; };
template <> struct PhaseWord<2> { using type = uint32_t; };
template <> struct PhaseWord<4> { using type = uint2; };
template <> struct PhaseWord<8> { using type = uint4; };

// raw container value (PCB bits) of element i of the group
template <int PCB>
__device__ __forceinline__ uint32_t phase_raw(const typename PhaseWord<PCB>::type& w, int i) {
  if constexpr (PCB == 0) return 0u;
  else if constexpr (PCB == 1) return (static_cast<uint32_t>(w) >> i) & 1u;
  else if constexpr (PCB == 2) return (w >> (2 * i)) & 3u;
  else if constexpr (PCB == 4) return ((i < 8 ? w.x : w.y) >> (4 * (i & 7))) & 15u;
  else {
    const uint32_t word = i < 4 ? w.x : (i < 8 ? w.y : (i < 12 ? w.z : w.w));
    return (word >> (8 * (i & 3))) & 255u;
  }
}

template <int PCB>
__device__ __forceinline__ void phase_put(typename PhaseWord<PCB>::type& w, int i, uint32_t v) {
  if constexpr (PCB == 1) w = static_cast<uint16_t>(w | (v << i));
  else if constexpr (PCB == 2) w |= v << (2 * i);
  else if constexpr (PCB == 4) (i < 8 ? w.x : w.y) |= v << (4 * (i & 7));
  else if constexpr (PCB == 8) (i < 4 ? w.x : (i < 8 ? w.y : (i < 12 ? w.z : w.w))) |= v << (8 * (i & 3));
}

// distance from level w to its neighbour on the side `up` (0 at the ends of the lattice): 0.5 below 2, 1 up to 4, 2
// above, the interval being the one that contains the neighbour
__device__ __forceinline__ float level_gap(float w, bool up) {
  const float m = fabsf(w);
  const bool outward = (w == 0.0f) || (up == (w > 0.0f));
  const float x = outward ? m : m - 0.25f;
  const uint32_t e = __float_as_uint(fmaxf(x, 1.0f)) & 0x7F800000u;
  const float g = __uint_as_float(e - 0x00800000u);
  return (outward && m == 6.0f) ? 0.0f : g;
}

// reciprocal of a power of two in the normal range
__device__ __forceinline__ float rcp_pow2(float x) { return __uint_as_float(0x7F000000u - __float_as_uint(x)); }

constexpr float kMagic = 12582912.0f;     // 1.5 * 2^23: adding it leaves the integer part in the low mantissa bits

// DIR: 0 = D given as fp32, 1 = raw, 2 = sign, 3 = colnorm (the gradient is read as GT)
// SRMODE: the rounding mode is known to be 'sr' (the draw needs no mode switch)
template <int PCB, int DIR, typename GT, bool SRMODE>
__global__ void __launch_bounds__(kThreads, 3) update_kernel(uint8_t* __restrict__ codes, uint8_t* __restrict__ phase,
                                                          const uint8_t* scales_in, uint8_t* scales_out,
                                                          const float* __restrict__ global_scale,
                                                          const GT* __restrict__ grad, const float* __restrict__ denom,
                                                          const float* __restrict__ stats, int64_t rows, int64_t cols,
                                                          StepParams P) {
  using PW = typename PhaseWord<PCB>::type;
  __shared__ float2 lut[16 << PCB];                 // (level a, latent) by code nibble | phase container << 4
  {
    const float inv_half = 1.0f / static_cast<float>(1 << (P.pb > 0 ? P.pb - 1 : 0));
    const int sh = 32 - P.pb;
    for (int e = threadIdx.y * blockDim.x + threadIdx.x; e < (16 << PCB); e += kThreads) {
      const int rk = rank_of_code(e & 15);
      const float av = level_of_rank(rk);
      float lam = av;
      if (PCB != 0) {
        const int ph = static_cast<int>(static_cast<uint32_t>(e >> 4) << sh) >> sh;     // sign-extend pb bits
        const float c = static_cast<float>(ph) * inv_half;
        const float lo = level_of_rank(max(rk - 1, 0)), hi = level_of_rank(min(rk + 1, 14));
        lam = c < 0.0f ? av + c * (av - lo) * 0.5f : av + c * (hi - av) * 0.5f;
      }
      lut[e] = make_float2(av, lam);
    }
  }
  // by code nibble: the level w, half / (half the distance to the next level above / below) -- 0 at the ends of the
  // lattice -- and the next level above: (t - w) times one of the two factors is the phase coordinate of a target t
  // whose nearest level is w
  __shared__ float4 plut[16];
  if (threadIdx.y * blockDim.x + threadIdx.x < 16) {
    const int c = threadIdx.y * blockDim.x + threadIdx.x;
    const int rk = rank_of_code(c);
    const float w = level_of_rank(rk);
    const float hf = static_cast<float>(1 << (P.pb > 0 ? P.pb - 1 : 0));
    const float wu = rk < 14 ? level_of_rank(rk + 1) : w, wd = rk > 0 ? level_of_rank(rk - 1) : w;
    const float su = rk < 14 ? hf / ((wu - w) * 0.5f) : 0.0f, sd = rk > 0 ? hf / ((w - wd) * 0.5f) : 0.0f;
    plut[c] = make_float4(w, su, sd, wu);
  }
  __syncthreads();

  const int64_t cg = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;   // 16-column group of this thread
  if (cg * 16 >= cols) return;
  const float gs = global_scale[0];
  const float rgs = __frcp_rn(gs);
  const float div = stats != nullptr ? stats[1] : 1.0f;
  const bool use_div = DIR != 0 && stats != nullptr && div != 1.0f;
  const float rdiv = __frcp_rn(div);
  float den[DIR == 3 ? 16 : 1], rden[DIR == 3 ? 16 : 1];
  if constexpr (DIR == 3) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      den[i] = denom[cg * 16 + i];
      rden[i] = __frcp_rn(den[i]);
    }
  }
  const float half = static_cast<float>(1 << (P.pb > 0 ? P.pb - 1 : 0));
  const uint32_t pmask = (1u << P.pb) - 1u;
  const int64_t code_stride = cols / 2, phase_stride = cols * PCB / 8, scale_stride = cols / 16;
  const int64_t row_step = static_cast<int64_t>(gridDim.y) * blockDim.y;

  for (int64_t r = static_cast<int64_t>(blockIdx.y) * blockDim.y + threadIdx.y; r < rows; r += row_step) {
    // ---- loads
    const uint2 cw = *reinterpret_cast<const uint2*>(codes + r * code_stride + cg * 8);
    PW pw{};
    if constexpr (PCB != 0) pw = *reinterpret_cast<const PW*>(phase + r * phase_stride + cg * (2 * PCB));
    float gv[16];
    load8(grad + r * cols + cg * 16, gv);
    load8(grad + r * cols + cg * 16 + 8, gv + 8);
    const uint32_t sb_old = scales_in[r * scale_stride + cg];
    const float s_old = e4m3_decode(sb_old) * gs;
    const float inv_s = __frcp_rn(s_old);

    // ---- latent target and the sums of the scale fit
    float tau[16];
    float saa[2] = {0.0f, 0.0f}, sat[2] = {0.0f, 0.0f}, stt[2] = {0.0f, 0.0f};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t code = ((i < 8 ? cw.x : cw.y) >> (4 * (i & 7))) & 15u;
      const float2 al = lut[code | (phase_raw<PCB>(pw, i) << 4)];
      float d;
      if (DIR == 2 && !use_div) {
        d = gv[i] > 0.0f ? inv_s : (gv[i] < 0.0f ? -inv_s : 0.0f);        // (+-1) / s_old
      } else {
        float u = gv[i];
        if (DIR == 2) u = static_cast<float>((u > 0.0f) - (u < 0.0f));
        if (DIR == 3) u = div_rn(u, den[i], rden[i]);
        if (use_div) u = div_rn(u, div, rdiv);
        d = div_rn(u, s_old, inv_s);
      }
      const float lrd = P.lr * d;
      tau[i] = al.y * P.decay - lrd;
      if (P.rule != BL_RULE_FIXED) {
        const float tf = P.rule == BL_RULE_FIT_LATENT ? tau[i] : al.x * P.decay - lrd;
        const int h = i >> 3;
        saa[h] = saa[h] + al.x * al.x;
        sat[h] = sat[h] + al.x * tf;
        stt[h] = stt[h] + tf * tf;
      }
    }

    // ---- group scale inside the trust region (bitlattice/reference.py:307-321)
    float s_new = s_old, inv_new = inv_s;
    uint32_t sb_new = sb_old;
    if (P.rule != BL_RULE_FIXED) {
      const float SAA = saa[0] + saa[1], SAT = sat[0] + sat[1], STT = stt[0] + stt[1];
      float rr = SAA > 0.0f ? SAT / SAA : 1.0f;
      rr = fminf(fmaxf(rr, P.r_lo), P.r_hi);
      const uint32_t bits = e4m3_encode(div_rn(s_old * rr, gs, rgs));
      const float cand = e4m3_decode(bits) * gs;
      const float q = div_rn(cand, s_old, inv_s);
      const float before = STT - 2.0f * SAT + SAA;
      const float after = q * q * SAA - 2.0f * q * SAT + STT;
      if ((after <= before) && isfinite(cand) && cand > 0.0f && bits != sb_old) {
        s_new = cand;
        sb_new = bits;
        inv_new = __frcp_rn(s_new);
      }
    }
    scales_out[r * scale_stride + cg] = static_cast<uint8_t>(sb_new);

    // ---- projection back to (code, phase) (bitlattice/reference.py:250-274, 324-334)
    const uint32_t idx0 = P.offset + static_cast<uint32_t>(static_cast<uint64_t>(r) * cols + cg * 16);
    uint2 cout = make_uint2(0u, 0u);
    PW pout{};
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
      float fin[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float t = div_rn(tau[i + e] * s_old, s_new, inv_new);
        t = fminf(fmaxf(t, -6.0f), 6.0f);
        fin[e] = t;
      }
      // nearest levels of the pair through the hardware conversion (ties to even: see the notes above)
      const uint32_t near2 = cvt_e2m1x2(fin[1], fin[0]);
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float t = fin[e];
        const float u = SRMODE ? hash_uniform(idx0 + i + e, P.rp.key) : rounding_u(P.rp, idx0 + i + e);
        float out;
        if (PCB == 0) {
          float w;
          {
            uint32_t h2;
            asm("{\n\t.reg .b8 b;\n\tcvt.u8.u32 b, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, b;\n\t}" : "=r"(h2) : "r"(near2));
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h2));
            w = e == 0 ? f.x : f.y;
          }
          const bool up = !(t < w);
          const float gap = level_gap(w, up);
          const float a = up ? w : w - gap;
          const float p = gap > 0.0f ? (t - a) * rcp_pow2(gap) : 0.0f;
          out = (u < p) ? a + gap : a;
        } else {
          const float4 L = plut[(near2 >> (4 * e)) & 15u];
          const float q = (t - L.x) * (t < L.x ? L.z : L.y);       // phase coordinate times half; exact scaling
          const float flm = __fadd_rd(q, kMagic);                  // kMagic + floor(q), exact
          const float flo = flm - kMagic;
          const bool ci = u < q - flo;
          uint32_t k = __float_as_uint(flm) + (ci ? 1u : 0u);      // low bits: floor(q) + carry-in, two's complement
          const bool carry = flo + (ci ? 1.0f : 0.0f) >= half;
          out = carry ? L.w : L.x;                                 // a carry implies a level above (not the top one)
          if (carry) k = static_cast<uint32_t>(-static_cast<int>(half));
          phase_put<PCB>(pout, i + e, k & pmask);
        }
        fin[e] = out;
      }
      const uint32_t byte = cvt_e2m1x2(fin[1], fin[0]);            // exact: both are levels
      (i < 8 ? cout.x : cout.y) |= byte << (4 * (i & 7));
    }
    cout.x = e2m1_drop_negative_zero(cout.x);
    cout.y = e2m1_drop_negative_zero(cout.y);
    *reinterpret_cast<uint2*>(codes + r * code_stride + cg * 8) = cout;
    if constexpr (PCB != 0) *reinterpret_cast<PW*>(phase + r * phase_stride + cg * (2 * PCB)) = pout;
  }
}

// fp32 direction written out (the reference's `direction` operator)
template <int DIR, typename GT>
__global__ void __launch_bounds__(kThreads) direction_kernel(const GT* __restrict__ grad, const float* __restrict__ denom,
                                                             const float* __restrict__ stats, int64_t rows,
                                                             int64_t cols, float* __restrict__ D) {
  const int64_t cc = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (cc * 8 >= cols) return;
  const bool use_div = stats != nullptr;
  const float div = use_div ? stats[1] : 1.0f;
  float den[8];
  if (DIR == 3) {
#pragma unroll
    for (int i = 0; i < 8; ++i) den[i] = denom[cc * 8 + i];
  }
  const int64_t row_step = static_cast<int64_t>(gridDim.y) * blockDim.y;
  for (int64_t r = static_cast<int64_t>(blockIdx.y) * blockDim.y + threadIdx.y; r < rows; r += row_step) {
    float gv[8];
    load8(grad + r * cols + cc * 8, gv);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float u = gv[i];
      if (DIR == 2) u = static_cast<float>((u > 0.0f) - (u < 0.0f));
      if (DIR == 3) u = u / den[i];
      if (use_div) u = u / div;
      gv[i] = u;
    }
    float* out = D + r * cols + cc * 8;
    reinterpret_cast<float4*>(out)[0] = make_float4(gv[0], gv[1], gv[2], gv[3]);
    reinterpret_cast<float4*>(out)[1] = make_float4(gv[4], gv[5], gv[6], gv[7]);
  }
}

// ------------------------------------------------------------------------------------------------ host side

struct Geometry {
  dim3 block, grid;
};

// threads along x cover `per`-column chunks (a power of two >= 32 so a warp never spans two rows), y covers rows
static Geometry geometry(int64_t rows, int64_t cols, int device, int per = 16) {
  const int64_t cpr = cols / per;
  int bx = 32;
  while (bx < 256 && bx < cpr) bx <<= 1;
  const int by = kThreads / bx;
  const int64_t gx = (cpr + bx - 1) / bx;
  const int64_t want = static_cast<int64_t>(sm_count(device)) * 8;           // CTAs for a few waves per SM
  int64_t gy = (want + gx - 1) / gx;
  const int64_t max_gy = (rows + by - 1) / by;
  gy = gy < 1 ? 1 : (gy > max_gy ? max_gy : gy);
  if (gy > 65535) gy = 65535;
  Geometry g;
  g.block = dim3(bx, by);
  g.grid = dim3(static_cast<unsigned>(gx), static_cast<unsigned>(gy));
  return g;
}

static int check_common(int64_t rows, int64_t cols, int phase_bits, int phase_cb, const void* phase, int rounding,
                        int rule) {
  BL_REQUIRE(rows > 0 && cols > 0, "lattice update: empty tensor (%lld x %lld)", (long long)rows, (long long)cols);
  BL_REQUIRE(cols % 16 == 0, "lattice update: last dimension %lld must be a multiple of 16 (NVFP4 groups)",
             (long long)cols);
  BL_REQUIRE(phase_bits >= 0 && phase_bits <= 8, "lattice update: phase_bits %d outside [0, 8]", phase_bits);
  const int want_cb = phase_bits == 0 ? 0 : phase_bits == 1 ? 1 : phase_bits == 2 ? 2 : phase_bits <= 4 ? 4 : 8;
  BL_REQUIRE(phase_bits == 0 || phase_cb == want_cb, "lattice update: %d-bit phase needs %d-bit containers, got %d",
             phase_bits, want_cb, phase_cb);
  BL_REQUIRE(phase_bits == 0 || phase != nullptr, "lattice update: phase buffer missing for %d-bit phase", phase_bits);
  BL_REQUIRE(rounding >= 0 && rounding <= 2, "lattice update: unknown rounding %d", rounding);
  BL_REQUIRE(rule >= 0 && rule <= 2, "lattice update: unknown scale rule %d", rule);
  return 0;
}

static StepParams make_params(double lr, double decay, int pb, int rule, double kappa, int rounding, uint32_t seed,
                              uint32_t step, int strat_j, int strat_k, uint64_t offset) {
  StepParams P;
  P.lr = static_cast<float>(lr);
  P.decay = static_cast<float>(decay);
  P.pb = pb;
  P.rule = rule;
  P.r_lo = static_cast<float>(exp(-kappa));
  P.r_hi = static_cast<float>(exp(kappa));
  P.rp.mode = rounding;
  P.rp.key = hash_key(seed, rounding == BL_ROUND_STRAT ? 0u : step);
  P.rp.strat_j = static_cast<float>(strat_j);
  P.rp.strat_k = static_cast<float>(strat_k > 0 ? strat_k : 1);
  P.offset = static_cast<uint32_t>(offset);
  return P;
}

template <int DIR, typename GT, bool SRMODE>
static void launch_update_mode(int pcb, const Geometry& g, cudaStream_t st, uint8_t* codes, uint8_t* phase,
                               const uint8_t* sin, uint8_t* sout, const float* gs, const GT* grad, const float* denom,
                               const float* stats, int64_t rows, int64_t cols, const StepParams& P) {
  switch (pcb) {
    case 0: update_kernel<0, DIR, GT, SRMODE><<<g.grid, g.block, 0, st>>>(codes, phase, sin, sout, gs, grad, denom, stats, rows, cols, P); break;
    case 1: update_kernel<1, DIR, GT, SRMODE><<<g.grid, g.block, 0, st>>>(codes, phase, sin, sout, gs, grad, denom, stats, rows, cols, P); break;
    case 2: update_kernel<2, DIR, GT, SRMODE><<<g.grid, g.block, 0, st>>>(codes, phase, sin, sout, gs, grad, denom, stats, rows, cols, P); break;
    case 4: update_kernel<4, DIR, GT, SRMODE><<<g.grid, g.block, 0, st>>>(codes, phase, sin, sout, gs, grad, denom, stats, rows, cols, P); break;
    default: update_kernel<8, DIR, GT, SRMODE><<<g.grid, g.block, 0, st>>>(codes, phase, sin, sout, gs, grad, denom, stats, rows, cols, P); break;
  }
}

template <int DIR, typename GT>
static void launch_update(int pcb, const Geometry& g, cudaStream_t st, uint8_t* codes, uint8_t* phase,
                          const uint8_t* sin, uint8_t* sout, const float* gs, const GT* grad, const float* denom,
                          const float* stats, int64_t rows, int64_t cols, const StepParams& P) {
  if (P.rp.mode == BL_ROUND_SR)
    launch_update_mode<DIR, GT, true>(pcb, g, st, codes, phase, sin, sout, gs, grad, denom, stats, rows, cols, P);
  else
    launch_update_mode<DIR, GT, false>(pcb, g, st, codes, phase, sin, sout, gs, grad, denom, stats, rows, cols, P);
}

// column statistics + finalize into scratch; returns pointers for the consumer kernel
template <typename GT>
static int run_stats(const GT* grad, int64_t rows, int64_t cols, int direction, double clip, const Scratch& s,
                     cudaStream_t st) {
  const int64_t cpr = cols / 8;
  int bx = 32;
  while (bx < 256 && bx < cpr) bx <<= 1;
  const int64_t npanels = (rows + kPanelRows - 1) / kPanelRows;
  BL_REQUIRE(npanels <= 65535, "direction: %lld rows exceed the supported 8388480", (long long)rows);
  const dim3 grid(static_cast<unsigned>((cpr + bx - 1) / bx), static_cast<unsigned>(npanels));
  BL_CUDA(cudaMemsetAsync(s.ticket, 0, sizeof(unsigned), st));
  if (direction == BL_DIR_SIGN)
    colstats_kernel<GT, true><<<grid, bx, 0, st>>>(grad, rows, cols, s.partial);
  else
    colstats_kernel<GT, false><<<grid, bx, 0, st>>>(grad, rows, cols, s.partial);
  BL_CUDA(cudaGetLastError());
  const unsigned nchunks = static_cast<unsigned>((cols + 255) / 256);
  finalize_kernel<<<nchunks, 256, 0, st>>>(s.partial, rows, cols, static_cast<int>(npanels),
                                           direction == BL_DIR_COLNORM ? 1 : 0, static_cast<float>(clip), s.denom,
                                           s.chunk, s.stats, s.ticket);
  BL_CUDA(cudaGetLastError());
  return 0;
}

template <typename GT>
static int update_typed(uint8_t* codes, uint8_t* phase, uint8_t* scales, const float* gs, const GT* grad, int64_t rows,
                        int64_t cols, int pcb, const StepParams& P, int direction, double clip, void* scratch,
                        int device, cudaStream_t st) {
  const float* denom = nullptr;
  const float* stats = nullptr;
  if (needs_stats(direction, clip)) {
    const Scratch s = scratch_layout(scratch, rows, cols);
    if (int rc = run_stats(grad, rows, cols, direction, clip, s, st)) return rc;
    denom = s.denom;
    stats = s.stats;
  }
  const Geometry g = geometry(rows, cols, device);
  if (direction == BL_DIR_RAW) launch_update<1, GT>(pcb, g, st, codes, phase, scales, scales, gs, grad, denom, stats, rows, cols, P);
  else if (direction == BL_DIR_SIGN) launch_update<2, GT>(pcb, g, st, codes, phase, scales, scales, gs, grad, denom, stats, rows, cols, P);
  else launch_update<3, GT>(pcb, g, st, codes, phase, scales, scales, gs, grad, denom, stats, rows, cols, P);
  BL_CUDA(cudaGetLastError());
  return 0;
}

template <typename GT>
static int direction_typed(const GT* grad, int64_t rows, int64_t cols, int direction, double clip, float* D,
                           void* scratch, int device, cudaStream_t st) {
  const float* denom = nullptr;
  const float* stats = nullptr;
  if (needs_stats(direction, clip)) {
    const Scratch s = scratch_layout(scratch, rows, cols);
    if (int rc = run_stats(grad, rows, cols, direction, clip, s, st)) return rc;
    denom = s.denom;
    stats = s.stats;
  }
  const Geometry g = geometry(rows, cols, device, 8);
  if (direction == BL_DIR_RAW) direction_kernel<1, GT><<<g.grid, g.block, 0, st>>>(grad, denom, stats, rows, cols, D);
  else if (direction == BL_DIR_SIGN) direction_kernel<2, GT><<<g.grid, g.block, 0, st>>>(grad, denom, stats, rows, cols, D);
  else direction_kernel<3, GT><<<g.grid, g.block, 0, st>>>(grad, denom, stats, rows, cols, D);
  BL_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace blb

using namespace blb;

extern "C" size_t bl_update_scratch_bytes(int64_t rows, int64_t cols, int direction, double clip) {
  if (rows <= 0 || cols <= 0 || !needs_stats(direction, clip)) return 0;
  return scratch_layout(nullptr, rows, cols).bytes;
}

extern "C" int bl_nvfp4_step_quantized(uint8_t* codes, uint8_t* phase, const uint8_t* scales_in, uint8_t* scales_out,
                                       const float* global_scale, const float* D, int64_t rows, int64_t cols,
                                       uint64_t offset, int phase_bits, int phase_cb, double lr, double decay,
                                       int rounding, uint32_t seed, uint32_t step, int strat_j, int strat_k, int rule,
                                       double kappa, int device, bl_stream_t stream) {
  if (int rc = check_common(rows, cols, phase_bits, phase_cb, phase, rounding, rule)) return rc;
  BL_REQUIRE(codes && scales_in && scales_out && global_scale && D, "step_quantized: null buffer");
  BL_REQUIRE(aligned16(codes) && aligned16(D) && (phase == nullptr || aligned16(phase)),
             "step_quantized: codes, phase and D must be 16-byte aligned");
  BL_DEVICE(device);
  const StepParams P = make_params(lr, decay, phase_bits, rule, kappa, rounding, seed, step, strat_j, strat_k, offset);
  const Geometry g = geometry(rows, cols, device);
  launch_update<0, float>(phase_bits ? phase_cb : 0, g, reinterpret_cast<cudaStream_t>(stream), codes, phase, scales_in,
                          scales_out, global_scale, D, nullptr, nullptr, rows, cols, P);
  BL_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int bl_nvfp4_lattice_update(uint8_t* codes, uint8_t* phase, uint8_t* scales, const float* global_scale,
                                       const void* grad, int grad_dtype, int64_t rows, int64_t cols, uint64_t offset,
                                       int phase_bits, int phase_cb, double lr, double decay, int rounding,
                                       uint32_t seed, uint32_t step, int strat_j, int strat_k, int rule, double kappa,
                                       int direction, double clip, void* scratch, size_t scratch_bytes, int device,
                                       bl_stream_t stream) {
  if (int rc = check_common(rows, cols, phase_bits, phase_cb, phase, rounding, rule)) return rc;
  BL_REQUIRE(codes && scales && global_scale && grad, "lattice_update: null buffer");
  BL_REQUIRE(direction >= BL_DIR_RAW && direction <= BL_DIR_COLNORM,
             "lattice_update: direction %d is not built (raw, sign and colnorm are)", direction);
  BL_REQUIRE(clip > 0.0, "lattice_update: clip must be positive");
  BL_REQUIRE(grad_dtype >= BL_F32 && grad_dtype <= BL_F16, "lattice_update: unknown gradient dtype %d", grad_dtype);
  BL_REQUIRE(aligned16(codes) && aligned16(grad) && (phase == nullptr || aligned16(phase)),
             "lattice_update: codes, phase and gradient must be 16-byte aligned");
  const size_t need = bl_update_scratch_bytes(rows, cols, direction, clip);
  BL_REQUIRE(need == 0 || (scratch != nullptr && scratch_bytes >= need && aligned16(scratch)),
             "lattice_update: needs %zu bytes of 16-byte aligned scratch, got %zu", need, scratch_bytes);
  BL_DEVICE(device);
  const StepParams P = make_params(lr, decay, phase_bits, rule, kappa, rounding, seed, step, strat_j, strat_k, offset);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int pcb = phase_bits ? phase_cb : 0;
  if (grad_dtype == BL_BF16)
    return update_typed(codes, phase, scales, global_scale, static_cast<const __nv_bfloat16*>(grad), rows, cols, pcb, P,
                        direction, clip, scratch, device, st);
  if (grad_dtype == BL_F16)
    return update_typed(codes, phase, scales, global_scale, static_cast<const __half*>(grad), rows, cols, pcb, P,
                        direction, clip, scratch, device, st);
  return update_typed(codes, phase, scales, global_scale, static_cast<const float*>(grad), rows, cols, pcb, P, direction,
                      clip, scratch, device, st);
}

extern "C" int bl_nvfp4_lattice_update_many(int count, uint8_t* const* codes, uint8_t* const* phase,
                                            uint8_t* const* scales, const float* const* global_scale,
                                            const void* const* grad, const int64_t* rows, const int64_t* cols,
                                            const uint64_t* offset, const uint32_t* seed, const uint32_t* step,
                                            const int* strat_j, int grad_dtype, int phase_bits, int phase_cb, double lr,
                                            double decay, int rounding, int strat_k, int rule, double kappa,
                                            int direction, double clip, void* scratch, size_t scratch_bytes, int device,
                                            bl_stream_t stream) {
  BL_REQUIRE(count >= 0, "lattice_update_many: negative count");
  BL_REQUIRE(count == 0 || (codes && scales && global_scale && grad && rows && cols && offset && seed && step),
             "lattice_update_many: null array");
  BL_REQUIRE(phase_bits == 0 || phase != nullptr, "lattice_update_many: null phase array");
  // the tensors are updated one after the other on the stream and share the scratch, whose size must cover the largest
  for (int i = 0; i < count; ++i) {
    const size_t need = bl_update_scratch_bytes(rows[i], cols[i], direction, clip);
    BL_REQUIRE(need == 0 || (scratch != nullptr && scratch_bytes >= need),
               "lattice_update_many: tensor %d needs %zu bytes of scratch, got %zu", i, need, scratch_bytes);
  }
  for (int i = 0; i < count; ++i) {
    const int rc = bl_nvfp4_lattice_update(codes[i], phase_bits ? phase[i] : nullptr, scales[i], global_scale[i], grad[i],
                                           grad_dtype, rows[i], cols[i], offset[i], phase_bits, phase_cb, lr, decay,
                                           rounding, seed[i], step[i], strat_j ? strat_j[i] : 0, strat_k, rule, kappa,
                                           direction, clip, scratch, scratch_bytes, device, stream);
    if (rc != 0) return rc;
  }
  return 0;
}

extern "C" int bl_direction(const void* grad, int grad_dtype, int64_t rows, int64_t cols, int direction, double clip,
                            float* D, void* scratch, size_t scratch_bytes, int device, bl_stream_t stream) {
  BL_REQUIRE(rows > 0 && cols > 0 && cols % 8 == 0, "direction: [rows, cols] with cols a multiple of 8, got %lld x %lld",
             (long long)rows, (long long)cols);
  BL_REQUIRE(grad && D, "direction: null buffer");
  BL_REQUIRE(direction >= BL_DIR_RAW && direction <= BL_DIR_COLNORM,
             "direction: kind %d is not built (raw, sign and colnorm are)", direction);
  BL_REQUIRE(clip > 0.0, "direction: clip must be positive");
  BL_REQUIRE(grad_dtype >= BL_F32 && grad_dtype <= BL_F16, "direction: unknown gradient dtype %d", grad_dtype);
  BL_REQUIRE(aligned16(grad) && aligned16(D), "direction: buffers must be 16-byte aligned");
  const size_t need = bl_update_scratch_bytes(rows, cols, direction, clip);
  BL_REQUIRE(need == 0 || (scratch != nullptr && scratch_bytes >= need && aligned16(scratch)),
             "direction: needs %zu bytes of 16-byte aligned scratch, got %zu", need, scratch_bytes);
  BL_DEVICE(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (grad_dtype == BL_BF16)
    return direction_typed(static_cast<const __nv_bfloat16*>(grad), rows, cols, direction, clip, D, scratch, device, st);
  if (grad_dtype == BL_F16)
    return direction_typed(static_cast<const __half*>(grad), rows, cols, direction, clip, D, scratch, device, st);
  return direction_typed(static_cast<const float*>(grad), rows, cols, direction, clip, D, scratch, device, st);
}

// ------------------------------------------------------------------------------------------------ fixed-scratch variant
// The column statistics of the update live here instead of in a caller-provided buffer. The array is part of the
// library image: every GPU that loads the library keeps these bytes until the process exits.
constexpr size_t kFixedScratchBytes = size_t(4) << 20;
static __device__ __align__(256) unsigned char g_fixed_scratch[kFixedScratchBytes];

// In host code `g_fixed_scratch` is only a handle for the runtime, never an address a kernel may use: the device
// address is asked for once per device, with that device current, and kept.
static int fixed_scratch_address(int device, void** out) {
  static std::mutex mu;
  static void* cached[64];
  BL_REQUIRE(device >= 0 && device < 64, "lattice_update_fixed_scratch: device index %d out of range", device);
  std::lock_guard<std::mutex> lock(mu);
  if (cached[device] == nullptr) {
    void* p = nullptr;
    BL_CUDA(cudaGetSymbolAddress(&p, g_fixed_scratch));
    BL_REQUIRE(p != nullptr, "lattice_update_fixed_scratch: no device address for the scratch array");
    cached[device] = p;
  }
  *out = cached[device];
  return 0;
}

extern "C" size_t bl_update_fixed_scratch_capacity(void) { return kFixedScratchBytes; }

extern "C" int bl_nvfp4_lattice_update_fixed_scratch(uint8_t* codes, uint8_t* phase, uint8_t* scales,
                                                     const float* global_scale, const void* grad, int grad_dtype,
                                                     int64_t rows, int64_t cols, uint64_t offset, int phase_bits,
                                                     int phase_cb, double lr, double decay, int rounding,
                                                     uint32_t seed, uint32_t step, int strat_j, int strat_k, int rule,
                                                     double kappa, int direction, double clip, int device,
                                                     bl_stream_t stream) {
  if (int rc = check_common(rows, cols, phase_bits, phase_cb, phase, rounding, rule)) return rc;
  BL_REQUIRE(codes && scales && global_scale && grad, "lattice_update_fixed_scratch: null buffer");
  BL_REQUIRE(direction >= BL_DIR_RAW && direction <= BL_DIR_COLNORM,
             "lattice_update_fixed_scratch: direction %d is not built (raw, sign and colnorm are)", direction);
  BL_REQUIRE(clip > 0.0, "lattice_update_fixed_scratch: clip must be positive");
  BL_REQUIRE(grad_dtype >= BL_F32 && grad_dtype <= BL_F16, "lattice_update_fixed_scratch: unknown gradient dtype %d",
             grad_dtype);
  BL_REQUIRE(aligned16(codes) && aligned16(grad) && (phase == nullptr || aligned16(phase)),
             "lattice_update_fixed_scratch: codes, phase and gradient must be 16-byte aligned");
  const size_t need = bl_update_scratch_bytes(rows, cols, direction, clip);
  BL_REQUIRE(need <= kFixedScratchBytes,
             "lattice_update_fixed_scratch: a %lld x %lld gradient needs %zu bytes of column statistics, the built-in "
             "scratch holds %zu; use bl_nvfp4_lattice_update with a buffer of your own",
             (long long)rows, (long long)cols, need, kFixedScratchBytes);
  BL_DEVICE(device);
  void* scratch = nullptr;
  if (int rc = fixed_scratch_address(device, &scratch)) return rc;
  const StepParams P = make_params(lr, decay, phase_bits, rule, kappa, rounding, seed, step, strat_j, strat_k, offset);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int pcb = phase_bits ? phase_cb : 0;
  // run_stats clears the arrival counter and overwrites every statistic it later reads, so what an earlier call left
  // in the array does not matter
  if (grad_dtype == BL_BF16)
    return update_typed(codes, phase, scales, global_scale, static_cast<const __nv_bfloat16*>(grad), rows, cols, pcb, P,
                        direction, clip, scratch, device, st);
  if (grad_dtype == BL_F16)
    return update_typed(codes, phase, scales, global_scale, static_cast<const __half*>(grad), rows, cols, pcb, P,
                        direction, clip, scratch, device, st);
  return update_typed(codes, phase, scales, global_scale, static_cast<const float*>(grad), rows, cols, pcb, P, direction,
                      clip, scratch, device, st);
}
