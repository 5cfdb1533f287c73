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
#include <atomic>
#include <mutex>

#include "common.cuh"

namespace blb {

constexpr int kPanelRows = 128;   // rows summed sequentially into one partial column sum
constexpr int kThreads = 256;

// Scratch of one tensor's column statistics (bytes; every part rounded up to 256):
//   partial [npanels, cols] fp32 partial column sums of U0^2, denom [cols] fp32 colnorm denominators,
//   chunk [ceil(cols / 256)] fp64 partial sums of the RMS, stats: [0] rho, [1] divisor max(rho / clip, 1).
// A batch of tensors uses 256 bytes of arrival counters followed by the tensors' regions.
static size_t tensor_scratch_bytes(int64_t rows, int64_t cols) {
  auto up = [](size_t n) { return (n + 255) & ~size_t(255); };
  const int64_t npanels = (rows + kPanelRows - 1) / kPanelRows;
  const int64_t nchunks = (cols + 255) / 256;
  return up(static_cast<size_t>(npanels * cols) * 4) + up(static_cast<size_t>(cols) * 4) +
         up(static_cast<size_t>(nchunks) * 8) + 256;
}

static bool needs_stats(int direction, double clip) { return !(direction == BL_DIR_SIGN && clip >= 1.0); }

// ------------------------------------------------------------------------------------------------ batches
// Several tensors share every launch: a batch carries up to kMaxBatch tensor descriptors by value in the kernel
// parameters, and each CTA finds its tensor by walking the (short) list. One statistics launch, one finalize launch
// and one update launch then serve a whole parameter group, which matters for row shards of a few hundred thousand
// weights where four launches per tensor would cost more than the work.

constexpr int kMaxBatch = 40;

struct TensorDesc {
  uint8_t* codes;
  uint8_t* phase;
  const uint8_t* scales_in;
  uint8_t* scales_out;      // may equal scales_in
  const float* gs;
  const void* grad;
  int rows, cols;
  uint32_t offset, key;     // RNG: index of element (0, 0) and hash key of (seed, step)
  float strat_j;
  uint32_t scratch256;      // offset of the tensor's scratch region in the batch scratch, in units of 256 bytes
  // A row shard whose statistics cover the whole weight: stat_rows = rows of the whole weight, stat_panel0 = the
  // shard's first 128-row panel in it, stat_local = panels per owner, and the panel sums live in the batch's exchange
  // area (one block per owner, Batch::stat_stride floats apart): gather256 = offset, in units of 256 bytes, of this
  // tensor's slice in owner 0's block. Everything else: stat_rows = rows, stat_panel0 = 0, gather256 = 0 (the panel
  // sums are the head of the tensor's own scratch region).
  int stat_rows, stat_panel0, stat_local;
  uint32_t gather256;
};

struct Batch {
  int count;
  uint32_t stat_stride;     // floats between the blocks of consecutive owners in the exchange area (row shards)
  TensorDesc t[kMaxBatch];
};

__host__ __device__ inline int stats_col_chunks(int cols) { return (cols + 255) / 256; }
__host__ __device__ inline int stats_panels(int rows) { return (rows + kPanelRows - 1) / kPanelRows; }

// scratch region of one tensor, device side (same layout as scratch_layout)
struct ScratchDev {
  float* partial;
  float* denom;
  double* chunk;
  float* stats;
  unsigned* ticket;
};

// The first 256 bytes of a batch's scratch hold the arrival counters of its tensors (cleared by one memset per batch);
// the tensors' regions follow.
__device__ __forceinline__ ScratchDev scratch_of(unsigned char* base, const TensorDesc& t, int index) {
  unsigned char* p = base + static_cast<size_t>(t.scratch256) * 256;
  auto up = [](size_t n) { return (n + 255) & ~size_t(255); };
  ScratchDev s;
  s.partial = reinterpret_cast<float*>(p);
  p += up(static_cast<size_t>(stats_panels(t.stat_rows)) * t.cols * 4);
  s.denom = reinterpret_cast<float*>(p);
  p += up(static_cast<size_t>(t.cols) * 4);
  s.chunk = reinterpret_cast<double*>(p);
  p += up(static_cast<size_t>(stats_col_chunks(t.cols)) * 8);
  s.stats = reinterpret_cast<float*>(p);
  s.ticket = reinterpret_cast<unsigned*>(base) + index;
  return s;
}

// the sums of 128-row panel p of tensor t, [cols] floats
__device__ __forceinline__ float* panel_sums(unsigned char* base, const Batch& B, const TensorDesc& t, const ScratchDev& S,
                                             int p) {
  if (t.gather256 == 0) return S.partial + static_cast<int64_t>(p) * t.cols;
  const int owner = p / t.stat_local, local = p - owner * t.stat_local;
  return reinterpret_cast<float*>(base + static_cast<size_t>(t.gather256) * 256) +
         static_cast<size_t>(owner) * B.stat_stride + static_cast<int64_t>(local) * t.cols;
}

// ------------------------------------------------------------------------------------------------ column statistics

constexpr int kSubRows = 16;      // rows one warp sums sequentially; 8 warps cover a 128-row panel

// partial[p][c] of a 128-row panel: warp w sums the 16 rows [128 p + 16 w, + 16) in ascending order (lanes along the
// columns, 8 columns per lane, so every row is read as full lines), then the eight sub-sums are added in ascending w.
// U0 = G or sign(G). One CTA per (tensor, 256-column chunk, panel).
template <typename GT, bool SIGN>
__global__ void __launch_bounds__(kThreads) colstats_kernel(const __grid_constant__ Batch B, unsigned char* __restrict__ scratch) {
  __shared__ float sub[kPanelRows / kSubRows][256];
  int ti = 0;
  int blk = blockIdx.x;
  for (;; ++ti) {
    const int n = stats_col_chunks(B.t[ti].cols) * stats_panels(B.t[ti].rows);
    if (blk < n || ti == B.count - 1) break;
    blk -= n;
  }
  const TensorDesc& T = B.t[ti];
  const int chunks = stats_col_chunks(T.cols);
  const int panel = blk / chunks, chunk = blk - panel * chunks;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c0 = chunk * 256 + lane * 8;
  const GT* G = static_cast<const GT*>(T.grad);
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
  if (c0 < T.cols) {
    const int64_t r0 = static_cast<int64_t>(panel) * kPanelRows + warp * kSubRows;
    const int nr = static_cast<int>(min(static_cast<int64_t>(kSubRows), static_cast<int64_t>(T.rows) - r0));
    const GT* p = G + r0 * T.cols + c0;
    if (nr == kSubRows) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {                 // eight rows in flight at a time
        float v[kSubRows / 2][8];
#pragma unroll
        for (int r = 0; r < kSubRows / 2; ++r) load8(p + static_cast<int64_t>(half * (kSubRows / 2) + r) * T.cols, v[r]);
#pragma unroll
        for (int r = 0; r < kSubRows / 2; ++r) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float u = v[r][i];
            if (SIGN) u = static_cast<float>((u > 0.0f) - (u < 0.0f));
            acc[i] = acc[i] + u * u;
          }
        }
      }
    } else {
      for (int r = 0; r < nr; ++r) {
        float v[8];
        load8(p + static_cast<int64_t>(r) * T.cols, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float u = v[i];
          if (SIGN) u = static_cast<float>((u > 0.0f) - (u < 0.0f));
          acc[i] = acc[i] + u * u;
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) sub[warp][lane * 8 + i] = acc[i];
  __syncthreads();
  const int c = chunk * 256 + threadIdx.x;
  if (c < T.cols) {
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < kPanelRows / kSubRows; ++w) tot = tot + sub[w][threadIdx.x];
    panel_sums(scratch, B, T, scratch_of(scratch, T, ti), panel + T.stat_panel0)[c] = tot;
  }
}

// colsq[c] = ascending sum of the panel partials; colnorm: denom[c] = sqrt(colsq/rows) + 1e-30 and the column's sum
// of U^2 is taken as colsq / denom^2. The RMS sums 256-column chunks with a fixed halving tree in double, then the
// chunks in ascending order; the last block of a tensor to arrive publishes rho and the divisor and resets the
// tensor's arrival counter. One CTA per (tensor, 256-column chunk).
__global__ void __launch_bounds__(256) finalize_kernel(const __grid_constant__ Batch B, unsigned char* __restrict__ scratch, int colnorm,
                                                       float clip) {
  __shared__ double red[256];
  __shared__ bool last;
  int ti = 0;
  int blk = blockIdx.x;
  for (;; ++ti) {
    const int n = stats_col_chunks(B.t[ti].cols);
    if (blk < n || ti == B.count - 1) break;
    blk -= n;
  }
  const TensorDesc& T = B.t[ti];
  const ScratchDev S = scratch_of(scratch, T, ti);
  const int npanels = stats_panels(T.stat_rows);
  const int nchunks = stats_col_chunks(T.cols);
  const int c = blk * 256 + threadIdx.x;
  double colu = 0.0;
  if (c < T.cols) {
    // ascending sum; the loads of a run of panels are independent and issued ahead of the additions
    float tot = 0.0f;
    const int owners = T.gather256 == 0 ? 1 : npanels / T.stat_local;
    const int per = T.gather256 == 0 ? npanels : T.stat_local;
    for (int o = 0; o < owners; ++o) {
      const float* q = panel_sums(scratch, B, T, S, o * per) + c;
#pragma unroll 8
      for (int p = 0; p < per; ++p) tot = tot + q[static_cast<int64_t>(p) * T.cols];
    }
    if (colnorm) {
      const float d = sqrtf(tot / static_cast<float>(T.stat_rows)) + 1e-30f;
      S.denom[c] = d;
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
    S.chunk[blk] = red[0];
    __threadfence();
    last = atomicAdd(S.ticket, 1u) == static_cast<unsigned>(nchunks) - 1u;
  }
  __syncthreads();
  if (last && threadIdx.x == 0) {
    __threadfence();
    double acc = 0.0;
    for (int i = 0; i < nchunks; ++i) acc = acc + reinterpret_cast<volatile double*>(S.chunk)[i];
    const float rho = static_cast<float>(sqrt(acc / (static_cast<double>(T.stat_rows) * static_cast<double>(T.cols))));
    S.stats[0] = rho;
    S.stats[1] = fmaxf(rho / clip, 1.0f);
    *S.ticket = 0u;
  }
}

// ------------------------------------------------------------------------------------------------ the update

struct StepParams {
  float lr, decay;
  int pb;            // phase bits 0..8
  int rule;          // BL_RULE_*
  float r_lo, r_hi;  // exp(-kappa), exp(+kappa)
  int mode;          // BL_ROUND_*
  float strat_k;
};

// ---- per-thread work unit: one scale group of 16 consecutive elements ------------------------------------------------
// A thread loads the group's 8 code bytes, its phase bytes, its 16 gradient values and the scale byte, keeps its 16
// columns while it walks down the rows, and needs no communication with other threads.
//
// Exactness notes (every shortcut below returns the reference's bits; the parity tests compare bit for bit):
//  * (a, latent) of an element depend only on its code nibble and phase bits: shared-memory tables built with the
//    reference's formula at kernel start replace the per-element level / neighbour / latent arithmetic;
//  * divisions sharing a divisor (the old and new group scale, a column's denominator, the RMS divisor) go through
//    one correctly rounded reciprocal per divisor and two fused residual corrections (div_rn);
//  * the nearest level comes from the hardware E2M1 conversion (ties to even). The reference breaks ties to the lower
//    level, but the projection is invariant to that choice: a target exactly half-way between levels L < U gives
//    (U, phase -half) from either side (from L the phase code reaches +half and carries over), and with 0 phase bits
//    both sides draw U with probability 1/2 from the same random number;
//  * gaps between neighbouring levels are powers of two read off the exponent of the level, so dividing by a half
//    gap is a multiplication by an exact reciprocal and (t - w) / width needs no clamp (|t - w| <= width);
//  * a phase code that reaches +half carries to the next level with phase -half, and +half and -half have the same
//    low phase bits, so the stored bits are those of the uncorrected code;
//  * the sum of squared levels of a group is a sum of multiples of 1/4 below 2^24: exact in fp32 in any order, so
//    it is formed with integer arithmetic.

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

// Shared-memory tables of a CTA:
//   lutAL [16 << PCB]        (level a, latent value) by (code nibble | phase container << 4)
//   plut [16]                by code nibble: the level w, half / (half the distance to the next level above / below)
//                            -- 0 at the ends of the lattice -- and the code of the next level above: (t - w) times
//                            one of the two factors is the phase coordinate of a target t whose nearest level is w
template <int PCB>
__device__ __forceinline__ void build_tables(float2* lutAL, float4* plut, int pb, int tid, float4* plut24 = nullptr) {
  const float inv_half = 1.0f / static_cast<float>(1 << (pb > 0 ? pb - 1 : 0));
  const int sh = 32 - pb;
  for (int e = tid; e < (16 << PCB); e += kThreads) {
    const int rk = rank_of_code(e & 15);
    const float av = level_of_rank(rk);
    float lam = av;
    if (PCB != 0) {
      const int ph = static_cast<int>(static_cast<uint32_t>(e >> 4) << sh) >> sh;     // sign-extend pb bits
      const float c = static_cast<float>(ph) * inv_half;
      const float lo = level_of_rank(max(rk - 1, 0)), hi = level_of_rank(min(rk + 1, 14));
      lam = c < 0.0f ? av + c * (av - lo) * 0.5f : av + c * (hi - av) * 0.5f;
    }
    lutAL[e] = make_float2(av, lam);
  }
  if (tid < 16) {
    const int rk = rank_of_code(tid);
    const float w = level_of_rank(rk);
    const float hf = static_cast<float>(1 << (pb > 0 ? pb - 1 : 0));
    const float wu = rk < 14 ? level_of_rank(rk + 1) : w, wd = rk > 0 ? level_of_rank(rk - 1) : w;
    const float su = rk < 14 ? hf / ((wu - w) * 0.5f) : 0.0f, sd = rk > 0 ? hf / ((w - wd) * 0.5f) : 0.0f;
    plut[tid] = make_float4(w, su, sd, __uint_as_float(code_of_rank(min(rk + 1, 14))));
    // the same with the two factors times 2^24 (powers of two: exact): the phase coordinate in 2^-24 fixed point
    if (plut24) plut24[tid] = make_float4(w, su * 16777216.0f, sd * 16777216.0f,
                                          __uint_as_float(code_of_rank(min(rk + 1, 14))));
  }
}

__device__ __forceinline__ float draw_u(int mode, uint32_t idx, uint32_t key, float strat_j, float strat_k) {
  RoundParams rp;
  rp.mode = mode;
  rp.key = key;
  rp.strat_j = strat_j;
  rp.strat_k = strat_k;
  return rounding_u(rp, idx);
}

// One group by the general route: any rounding mode, any phase width, every division through the range-checked
// div_rn. It re-reads its inputs, writes its outputs and is kept out of line: the kernels use it for the
// configurations the fast route does not cover and for single groups whose values leave the fast route's range.
// DIR: 0 = D given as fp32, 1 = raw, 2 = sign, 3 = colnorm (the gradient is read as GT).
template <int PCB, int DIR, typename GT>
static __device__ __noinline__ void update_group_general(const TensorDesc& T, int64_t r, int64_t cg,
                                                         const float* __restrict__ denom, float div, bool use_div,
                                                         const float2* lutAL, const float4* plut,
                                                         const StepParams& P) {
  using PW = typename PhaseWord<PCB>::type;
  const int64_t cols = T.cols;
  const int64_t code_stride = cols / 2, phase_stride = cols * PCB / 8, scale_stride = cols / 16;
  const float gs = T.gs[0];
  const float rgs = __frcp_rn(gs);
  const float rdiv = __frcp_rn(div);
  const float half = static_cast<float>(1 << (P.pb > 0 ? P.pb - 1 : 0));
  const uint32_t pmask = (1u << P.pb) - 1u;
  const GT* grad = static_cast<const GT*>(T.grad);

  const uint2 cw = *reinterpret_cast<const uint2*>(T.codes + r * code_stride + cg * 8);
  PW pw{};
  if constexpr (PCB != 0) pw = *reinterpret_cast<const PW*>(T.phase + r * phase_stride + cg * (2 * PCB));
  float gv[16];
  load8(grad + r * cols + cg * 16, gv);
  load8(grad + r * cols + cg * 16 + 8, gv + 8);
  const uint32_t sb_old = T.scales_in[r * scale_stride + cg];
  const float s_old = e4m3_decode(sb_old) * gs;
  const float inv_s = __frcp_rn(s_old);

  // ---- latent target and the sums of the scale fit
  float tau[16];
  float saa[2] = {0.0f, 0.0f}, sat[2] = {0.0f, 0.0f}, stt[2] = {0.0f, 0.0f};
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const uint32_t code = ((i < 8 ? cw.x : cw.y) >> (4 * (i & 7))) & 15u;
    const uint32_t li = code | (phase_raw<PCB>(pw, i) << 4);
    const float2 al = lutAL[li];
    const float a = al.x, lam = al.y;
    float d;
    if (DIR == 2 && !use_div) {
      d = gv[i] > 0.0f ? inv_s : (gv[i] < 0.0f ? -inv_s : 0.0f);        // (+-1) / s_old
    } else {
      float u = gv[i];
      if (DIR == 2) u = static_cast<float>((u > 0.0f) - (u < 0.0f));
      if (DIR == 3) {
        const float den = denom[cg * 16 + i];
        u = div_rn(u, den, __frcp_rn(den));
      }
      if (use_div) u = div_rn(u, div, rdiv);
      d = div_rn(u, s_old, inv_s);
    }
    const float lrd = P.lr * d;
    tau[i] = lam * P.decay - lrd;
    if (P.rule != BL_RULE_FIXED) {
      const float tf = P.rule == BL_RULE_FIT_LATENT ? tau[i] : a * P.decay - lrd;
      const int h = i >> 3;
      saa[h] = saa[h] + a * a;
      sat[h] = sat[h] + a * tf;
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
  T.scales_out[r * scale_stride + cg] = static_cast<uint8_t>(sb_new);

  // ---- projection back to (code, phase) (bitlattice/reference.py:250-274, 324-334)
  const uint32_t idx0 = T.offset + static_cast<uint32_t>(static_cast<uint64_t>(r) * cols + cg * 16);
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
      const float u = draw_u(P.mode, idx0 + i + e, T.key, T.strat_j, P.strat_k);
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
        const uint32_t k = __float_as_uint(flm) + (ci ? 1u : 0u);   // low bits: floor(q) + carry-in, two's complement
        const bool carry = flo + (ci ? 1.0f : 0.0f) >= half;
        out = carry ? level_of_rank(rank_of_code(__float_as_uint(L.w))) : L.x;   // a carry implies a level above
        phase_put<PCB>(pout, i + e, k & pmask);                  // +half and -half share their low bits
      }
      fin[e] = out;
    }
    const uint32_t byte = cvt_e2m1x2(fin[1], fin[0]);            // exact: both are levels
    (i < 8 ? cout.x : cout.y) |= byte << (4 * (i & 7));
  }
  cout.x = e2m1_drop_negative_zero(cout.x);
  cout.y = e2m1_drop_negative_zero(cout.y);
  *reinterpret_cast<uint2*>(T.codes + r * code_stride + cg * 8) = cout;
  if constexpr (PCB != 0) *reinterpret_cast<PW*>(T.phase + r * phase_stride + cg * (2 * PCB)) = pout;
}

// sum over the 8 codes of a word of 4 * level^2 (byte table through PRMT, bytes summed by a dot product)
__device__ __forceinline__ uint32_t sum_sq4(uint32_t codes) {
  const uint32_t sel = codes & 0x77777777u;                       // magnitudes; bit 3 of a selector would replicate signs
  const uint32_t lo = __byte_perm(0x09040100u, 0x90402410u, sel);
  const uint32_t hi = __byte_perm(0x09040100u, 0x90402410u, sel >> 16);
  return __dp4a(lo, 0x01010101u, __dp4a(hi, 0x01010101u, 0u));
}

constexpr int kRowsPerThread = 8;     // rows a thread of the update kernel walks at most

__host__ __device__ inline int update_bx(int cols) {
  const int cpr = cols / 16;
  int bx = 32;
  while (bx < kThreads && bx < cpr) bx <<= 1;
  return bx;
}
__host__ __device__ inline int update_blocks(int rows, int cols) {
  const int bx = update_bx(cols), by = kThreads / bx;
  const int gx = (cols / 16 + bx - 1) / bx;
  const int gy = (rows + by * kRowsPerThread - 1) / (by * kRowsPerThread);
  return gx * gy;
}

// FAST: stochastic rounding with 1..7 phase bits. Its arithmetic runs on packed pairs (element i with element i + 8,
// the two halves of the group whose sums the reference accumulates separately) and its divisions skip div_rn's
// per-quotient range check. Instead one check per element on the gradient, against bounds derived per row from the
// divisors, establishes that every quotient of the chain g / den / div / s_old and of tau * s_old / s_new stays
// inside the range where the unchecked sequence is exact (zero excepted, which is exact anywhere); a group with a
// value outside goes through update_group_general. The bounds (fp32, conservative; 2^-98 .. 2^98 is the safe range of
// a quotient and of a dividend, the fit keeps s_new within a factor 4 of s_old):
//   |g| >= 2^-98 * max(1, dmax * div * max(1, 1/lr) * max(1, 4 s_old))      dmax, dmin: extremes of the thread's
//   |g| <= dmin * min(2^98, 2^60 * div * s_old)                             16 column denominators (1 without colnorm)
// together with s_old in [2^-40, 2^20], lr in [2^-30, 2^8], decay in [2^-20, 2], div <= 2^30, r_hi <= 2.
template <int PCB, int DIR, typename GT, bool FAST>
__global__ void __launch_bounds__(kThreads, 2) update_kernel(const __grid_constant__ Batch B, unsigned char* __restrict__ scratch, int has_stats,
                                                            StepParams P) {
  using PW = typename PhaseWord<PCB>::type;
  __shared__ float2 lutAL[16 << PCB];                       // (level, latent) pairs: one load per element
  __shared__ float4 plut[16];
  __shared__ float4 plut24[FAST ? 16 : 1];
  build_tables<PCB>(lutAL, plut, P.pb, threadIdx.x, FAST ? plut24 : nullptr);
  __syncthreads();

  int ti = 0;
  int blk = blockIdx.x;
  for (;; ++ti) {
    const int n = update_blocks(B.t[ti].rows, B.t[ti].cols);
    if (blk < n || ti == B.count - 1) break;
    blk -= n;
  }
  const TensorDesc& T = B.t[ti];
  const int64_t rows = T.rows, cols = T.cols;
  const int bx = update_bx(T.cols), by = kThreads / bx;
  const int gx = (T.cols / 16 + bx - 1) / bx;
  const int gy = (T.rows + by * kRowsPerThread - 1) / (by * kRowsPerThread);
  const int tx = threadIdx.x & (bx - 1), ty = threadIdx.x / bx;
  const int64_t cg = static_cast<int64_t>(blk % gx) * bx + tx;      // 16-column group of this thread
  if (cg * 16 >= cols) return;
  const int64_t row_first = static_cast<int64_t>(blk / gx) * by + ty, row_step = static_cast<int64_t>(gy) * by;

  const float* denom = nullptr;
  float div = 1.0f;
  if (has_stats) {
    const ScratchDev S = scratch_of(scratch, T, ti);
    denom = S.denom;
    div = S.stats[1];
  }
  const bool use_div = DIR != 0 && has_stats && div != 1.0f;

  if constexpr (!FAST) {
    for (int64_t r = row_first; r < rows; r += row_step)
      update_group_general<PCB, DIR, GT>(T, r, cg, denom, div, use_div, lutAL, plut, P);
    return;
  } else {
    const float gs = T.gs[0];
    const float rgs = __frcp_rn(gs);
    const GT* grad = static_cast<const GT*>(T.grad);
    const int64_t code_stride = cols / 2, phase_stride = cols * PCB / 8, scale_stride = cols / 16;
    const uint32_t pmask = (1u << P.pb) - 1u;
    const int half_i = 1 << (P.pb - 1);
    const bool fit = P.rule != BL_RULE_FIXED, latent = P.rule == BL_RULE_FIT_LATENT;
    const bool decay_one = P.decay == 1.0f;                   // no weight decay: the products by it are exact copies
    const f32x2 ndiv2 = pk(-div, -div), rdiv2 = pk(__frcp_rn(div), __frcp_rn(div));
    const f32x2 nlr2 = pk(-P.lr, -P.lr), decay2 = pk(P.decay, P.decay);

    // column denominators of the thread's group as pairs (i, i + 8), and the range bounds that depend on them
    f32x2 nden2[DIR == 3 ? 8 : 1], rden2[DIR == 3 ? 8 : 1];
    float dmax = 1.0f, dmin = 1.0f;
    if constexpr (DIR == 3) {
      dmax = 0.0f;
      dmin = 3.0e38f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float d0 = denom[cg * 16 + i], d1 = denom[cg * 16 + 8 + i];
        nden2[i] = pk(-d0, -d1);
        rden2[i] = pk(__frcp_rn(d0), __frcp_rn(d1));
        dmax = fmaxf(dmax, fmaxf(d0, d1));
        dmin = fminf(dmin, fminf(d0, d1));
      }
    }
    // the bounds of this thread; a kernel-wide parameter outside its range makes every group take the general route
    const bool params_ok = P.lr >= 9.3132257e-10f && P.lr <= 256.0f && P.decay >= 9.5367432e-7f && P.decay <= 2.0f &&
                           div <= 1073741824.0f && P.r_hi <= 2.0f && dmin >= 3.2e-30f && dmax <= 3.0e29f;
    const float inv_lr1 = fmaxf(1.0f, 1.0f / P.lr);
    const float lo_c = params_ok ? 3.1554436e-30f : 3.0e38f;                         // 2^-98
    const float lo_w = 3.1554436e-30f * dmax * div * inv_lr1;
    const float hi_c = dmin * 3.1691265e29f;                                         // 2^98 (may overflow to +inf: no bound)
    const float hi_w = dmin * div * 1.1529215e18f;                                   // 2^60

    for (int64_t r = row_first; r < rows; r += row_step) {
      // ---- loads
      const uint2 cw = *reinterpret_cast<const uint2*>(T.codes + r * code_stride + cg * 8);
      const PW pw = *reinterpret_cast<const PW*>(T.phase + r * phase_stride + cg * (2 * PCB));
      float gv[16];
      load8(grad + r * cols + cg * 16, gv);
      load8(grad + r * cols + cg * 16 + 8, gv + 8);
      const uint32_t sb_old = T.scales_in[r * scale_stride + cg];
      const float s_old = e4m3_decode(sb_old) * gs;
      const float inv_s = __frcp_rn(s_old);
      const f32x2 sold2 = pk(s_old, s_old), nsold2 = pk(-s_old, -s_old), rsold2 = pk(inv_s, inv_s);
      bool ok = s_old >= 9.0949470e-13f && s_old <= 1048576.0f;                     // 2^-40 .. 2^20
      const float g_lo = fmaxf(lo_c, lo_w * fmaxf(1.0f, 4.0f * s_old));
      const float g_hi = fminf(hi_c, hi_w * s_old);

      // sign direction: every element moves by the same +-L, L = lr * ((1 / div) / s_old)
      float nL = 0.0f;
      if constexpr (DIR == 2) {
        const float D0 = use_div ? div_rn(div_rn(1.0f, div, __frcp_rn(div)), s_old, inv_s) : inv_s;
        nL = -(P.lr * D0);
        const float xs = fabsf(nL) * s_old;                   // magnitude of tau * s_old where the latent value is 0
        ok = ok && xs >= 1.2621775e-29f && xs <= 1.1529215e18f;                      // 2^-96 .. 2^60
      }

      // ---- latent target and the sums of the scale fit
      f32x2 tau2[8];
      f32x2 sat2 = pk(0.0f, 0.0f), stt2 = pk(0.0f, 0.0f);
      // table indices (code | phase << 4). With 4-bit containers the nibbles of a code word and of a phase word are
      // interleaved into index bytes four at a time: even elements (c & 0x0F0F0F0F) | ((p << 4) & 0xF0F0F0F0), odd
      // elements ((c >> 4) & 0x0F0F0F0F) | (p & 0xF0F0F0F0); an index is then one byte extraction.
      [[maybe_unused]] uint32_t ev[2], od[2];
      if constexpr (PCB == 4) {
        ev[0] = (cw.x & 0x0F0F0F0Fu) | ((pw.x << 4) & 0xF0F0F0F0u);
        od[0] = ((cw.x >> 4) & 0x0F0F0F0Fu) | (pw.x & 0xF0F0F0F0u);
        ev[1] = (cw.y & 0x0F0F0F0Fu) | ((pw.y << 4) & 0xF0F0F0F0u);
        od[1] = ((cw.y >> 4) & 0x0F0F0F0Fu) | (pw.y & 0xF0F0F0F0u);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        uint32_t ia, ib;
        if constexpr (PCB == 4) {
          ia = __byte_perm((i & 1) ? od[0] : ev[0], 0u, 0x4440u | static_cast<uint32_t>(i >> 1));
          ib = __byte_perm((i & 1) ? od[1] : ev[1], 0u, 0x4440u | static_cast<uint32_t>(i >> 1));
        } else {
          ia = ((cw.x >> (4 * i)) & 15u) | (phase_raw<PCB>(pw, i) << 4);
          ib = ((cw.y >> (4 * i)) & 15u) | (phase_raw<PCB>(pw, i + 8) << 4);
        }
        const float2 al0 = lutAL[ia], al1 = lutAL[ib];
        const float a0 = al0.x, a1 = al1.x, l0 = al0.y, l1 = al1.y;
        f32x2 nl2;                                               // -(lr * d) of the pair
        if constexpr (DIR == 2) {
          const float g0 = gv[i], g1 = gv[i + 8];
          const float n0 = __uint_as_float(__float_as_uint(nL) ^ (__float_as_uint(g0) & 0x80000000u));
          const float n1 = __uint_as_float(__float_as_uint(nL) ^ (__float_as_uint(g1) & 0x80000000u));
          nl2 = pk(g0 == 0.0f ? 0.0f : n0, g1 == 0.0f ? 0.0f : n1);
        } else {
          const float g0 = gv[i], g1 = gv[i + 8];
          ok = ok && fabsf(g0) >= g_lo && fabsf(g0) <= g_hi && fabsf(g1) >= g_lo && fabsf(g1) <= g_hi;
          f32x2 u = pk(g0, g1);
          if constexpr (DIR == 3) u = div2p(u, nden2[i], rden2[i]);
          if (use_div) u = div2p(u, ndiv2, rdiv2);
          nl2 = prod2p(nlr2, div2p(u, nsold2, rsold2));
        }
        // Products that feed a sum keep their own rounding (prod2p; the sign of a zero product is immaterial: sums
        // start at +0 and the targets' zeros are normalised when the codes are written).
        const f32x2 a2 = pk(a0, a1);
        const f32x2 ld2 = decay_one ? pk(l0, l1) : prod2p(pk(l0, l1), decay2);
        tau2[i] = add2p(ld2, nl2);
        if (fit) {
          f32x2 tf2 = tau2[i];
          if (!latent) tf2 = add2p(decay_one ? a2 : prod2p(a2, decay2), nl2);
          sat2 = add2p(sat2, prod2p(a2, tf2));
          stt2 = add2p(stt2, prod2p(tf2, tf2));
        }
      }

      // ---- group scale inside the trust region (bitlattice/reference.py:307-321)
      float s_new = s_old, inv_new = inv_s;
      uint32_t sb_new = sb_old;
      if (fit) {
        float sat0, sat1, stt0, stt1;
        upk(sat2, sat0, sat1);
        upk(stt2, stt0, stt1);
        const float SAA = static_cast<float>(sum_sq4(cw.x)) * 0.25f + static_cast<float>(sum_sq4(cw.y)) * 0.25f;
        const float SAT = sat0 + sat1, STT = stt0 + stt1;
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
      ok = ok && s_new <= 4.0f * s_old && s_old <= 4.0f * s_new;
      if (!ok) {                                                // rare: values outside the unchecked divisions' range
        update_group_general<PCB, DIR, GT>(T, r, cg, denom, div, use_div, lutAL, plut, P);
        continue;
      }
      T.scales_out[r * scale_stride + cg] = static_cast<uint8_t>(sb_new);

      // ---- projection back to (code, phase) (bitlattice/reference.py:250-274, 324-334)
      const uint32_t h0 = (T.offset + static_cast<uint32_t>(static_cast<uint64_t>(r) * cols + cg * 16)) * 0x27D4EB2Fu +
                          T.key;
      const f32x2 nsnew2 = pk(-s_new, -s_new), rsnew2 = pk(inv_new, inv_new);
      uint2 cout = make_uint2(0u, 0u);
      PW pout{};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float tv[2];
        upk(div2p(mul2p(tau2[i], sold2), nsnew2, rsnew2), tv[0], tv[1]);
        // nearest levels of the pair through the hardware conversion (ties to even: see the notes above). It
        // saturates, and beyond the last level the table's factor is 0, so a target outside [-6, 6] needs no clamp
        // (the range check has made it finite): its phase coordinate is 0 either way.
        const uint32_t near2 = cvt_e2m1x2(tv[1], tv[0]);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float t = tv[e];
          const uint32_t nib = e == 0 ? (near2 & 15u) : (near2 >> 4);
          const float4 L = plut24[nib];
          // phase coordinate times half, in 2^-24 fixed point (exact scaling; |q| <= 64, so it fits 31 bits); the
          // draw n = hash >> 8 rounds up iff n * 2^-24 < frac(q), i.e. iff n < ceil(frac(q) * 2^24): the carry of
          // adding 2^24 - 1 - n to ceil(q * 2^24). k = floor(q) + carry, two's complement.
          const int q24 = __float2int_ru((t - L.x) * (t < L.x ? L.z : L.y));
          uint32_t h = h0 + static_cast<uint32_t>(i + 8 * e) * 0x27D4EB2Fu;
          h = (h ^ (h >> 16)) * 0x7FEB352Du;
          h = (h ^ (h >> 15)) * 0x846CA68Bu;
          h = ~(h ^ (h >> 16));
          const int k = (q24 + static_cast<int>(h >> 8)) >> 24;
          const uint32_t code = k == half_i ? __float_as_uint(L.w) : nib;      // +half: the level above, phase -half
          if (e == 0) cout.x += code << (4 * i);
          else cout.y += code << (4 * i);
          phase_put<PCB>(pout, i + 8 * e, static_cast<uint32_t>(k) & pmask);
        }
      }
      cout.x = e2m1_drop_negative_zero(cout.x);
      cout.y = e2m1_drop_negative_zero(cout.y);
      *reinterpret_cast<uint2*>(T.codes + r * code_stride + cg * 8) = cout;
      *reinterpret_cast<PW*>(T.phase + r * phase_stride + cg * (2 * PCB)) = pout;
    }
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

static std::atomic<int> g_update_route{0};     // 0: the fast route where it applies; 1: the general route everywhere

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
  BL_REQUIRE(rows < (1ll << 31) && cols < (1ll << 31), "lattice update: dimension exceeds 2^31 (%lld x %lld)",
             (long long)rows, (long long)cols);
  BL_REQUIRE(phase_bits >= 0 && phase_bits <= 8, "lattice update: phase_bits %d outside [0, 8]", phase_bits);
  const int want_cb = phase_bits == 0 ? 0 : phase_bits == 1 ? 1 : phase_bits == 2 ? 2 : phase_bits <= 4 ? 4 : 8;
  BL_REQUIRE(phase_bits == 0 || phase_cb == want_cb, "lattice update: %d-bit phase needs %d-bit containers, got %d",
             phase_bits, want_cb, phase_cb);
  BL_REQUIRE(phase_bits == 0 || phase != nullptr, "lattice update: phase buffer missing for %d-bit phase", phase_bits);
  BL_REQUIRE(rounding >= 0 && rounding <= 2, "lattice update: unknown rounding %d", rounding);
  BL_REQUIRE(rule >= 0 && rule <= 2, "lattice update: unknown scale rule %d", rule);
  return 0;
}

static StepParams make_params(double lr, double decay, int pb, int rule, double kappa, int rounding, int strat_k) {
  StepParams P;
  P.lr = static_cast<float>(lr);
  P.decay = static_cast<float>(decay);
  P.pb = pb;
  P.rule = rule;
  P.r_lo = static_cast<float>(exp(-kappa));
  P.r_hi = static_cast<float>(exp(kappa));
  P.mode = rounding;
  P.strat_k = static_cast<float>(strat_k > 0 ? strat_k : 1);
  return P;
}

static TensorDesc make_desc(uint8_t* codes, uint8_t* phase, const uint8_t* scales_in, uint8_t* scales_out,
                            const float* gs, const void* grad, int64_t rows, int64_t cols, uint64_t offset,
                            int rounding, uint32_t seed, uint32_t step, int strat_j) {
  TensorDesc d;
  d.codes = codes;
  d.phase = phase;
  d.scales_in = scales_in;
  d.scales_out = scales_out;
  d.gs = gs;
  d.grad = grad;
  d.rows = static_cast<int>(rows);
  d.cols = static_cast<int>(cols);
  d.offset = static_cast<uint32_t>(offset);
  d.key = hash_key(seed, rounding == BL_ROUND_STRAT ? 0u : step);
  d.strat_j = static_cast<float>(strat_j);
  d.scratch256 = 0;
  d.stat_rows = d.rows;
  d.stat_panel0 = 0;
  d.stat_local = stats_panels(d.rows);
  d.gather256 = 0;
  return d;
}

template <int DIR, typename GT, bool FAST>
static void launch_update_pcb(int pcb, unsigned blocks, cudaStream_t st, const Batch& B, unsigned char* scratch,
                              int has_stats, const StepParams& P) {
  switch (pcb) {
    case 0:
      if constexpr (!FAST) update_kernel<0, DIR, GT, false><<<blocks, kThreads, 0, st>>>(B, scratch, has_stats, P);
      break;
    case 1: update_kernel<1, DIR, GT, FAST><<<blocks, kThreads, 0, st>>>(B, scratch, has_stats, P); break;
    case 2: update_kernel<2, DIR, GT, FAST><<<blocks, kThreads, 0, st>>>(B, scratch, has_stats, P); break;
    case 4: update_kernel<4, DIR, GT, FAST><<<blocks, kThreads, 0, st>>>(B, scratch, has_stats, P); break;
    default: update_kernel<8, DIR, GT, FAST><<<blocks, kThreads, 0, st>>>(B, scratch, has_stats, P); break;
  }
}

// dir: 0 = D given (fp32), else BL_DIR_* + 1
template <typename GT>
static int launch_update(int dir, int pcb, cudaStream_t st, const Batch& B, unsigned char* scratch, int has_stats,
                         const StepParams& P) {
  int64_t blocks = 0;
  for (int i = 0; i < B.count; ++i) blocks += update_blocks(B.t[i].rows, B.t[i].cols);
  BL_REQUIRE(blocks > 0 && blocks <= 0x7FFFFFFF, "lattice update: too many blocks (%lld)", (long long)blocks);
  const unsigned nb = static_cast<unsigned>(blocks);
  const bool fast = P.mode == BL_ROUND_SR && P.pb >= 1 && P.pb <= 7 && g_update_route.load(std::memory_order_relaxed) == 0;
  if (fast) {
    if (dir == 0) launch_update_pcb<0, GT, true>(pcb, nb, st, B, scratch, has_stats, P);
    else if (dir == 1) launch_update_pcb<1, GT, true>(pcb, nb, st, B, scratch, has_stats, P);
    else if (dir == 2) launch_update_pcb<2, GT, true>(pcb, nb, st, B, scratch, has_stats, P);
    else launch_update_pcb<3, GT, true>(pcb, nb, st, B, scratch, has_stats, P);
  } else {
    if (dir == 0) launch_update_pcb<0, GT, false>(pcb, nb, st, B, scratch, has_stats, P);
    else if (dir == 1) launch_update_pcb<1, GT, false>(pcb, nb, st, B, scratch, has_stats, P);
    else if (dir == 2) launch_update_pcb<2, GT, false>(pcb, nb, st, B, scratch, has_stats, P);
    else launch_update_pcb<3, GT, false>(pcb, nb, st, B, scratch, has_stats, P);
  }
  BL_CUDA(cudaGetLastError());
  return 0;
}

// column statistics of a batch into its scratch (regions assigned in B): the panel sums only
template <typename GT>
static int run_colstats(const Batch& B, int direction, unsigned char* scratch, cudaStream_t st) {
  int64_t sblocks = 0;
  for (int i = 0; i < B.count; ++i)
    sblocks += static_cast<int64_t>(stats_col_chunks(B.t[i].cols)) * stats_panels(B.t[i].rows);
  BL_REQUIRE(sblocks <= 0x7FFFFFFF, "direction: too many statistics blocks (%lld)", (long long)sblocks);
  if (direction == BL_DIR_SIGN)
    colstats_kernel<GT, true><<<static_cast<unsigned>(sblocks), kThreads, 0, st>>>(B, scratch);
  else
    colstats_kernel<GT, false><<<static_cast<unsigned>(sblocks), kThreads, 0, st>>>(B, scratch);
  BL_CUDA(cudaGetLastError());
  return 0;
}

// panel sums -> denominators, RMS divisor
static int run_finalize(const Batch& B, int direction, double clip, unsigned char* scratch, cudaStream_t st) {
  int64_t fblocks = 0;
  for (int i = 0; i < B.count; ++i) fblocks += stats_col_chunks(B.t[i].cols);
  BL_CUDA(cudaMemsetAsync(scratch, 0, 256, st));                       // the batch's arrival counters
  finalize_kernel<<<static_cast<unsigned>(fblocks), 256, 0, st>>>(B, scratch, direction == BL_DIR_COLNORM ? 1 : 0,
                                                                 static_cast<float>(clip));
  BL_CUDA(cudaGetLastError());
  return 0;
}

template <typename GT>
static int run_stats(const Batch& B, int direction, double clip, unsigned char* scratch, cudaStream_t st) {
  if (int rc = run_colstats<GT>(B, direction, scratch, st)) return rc;
  return run_finalize(B, direction, clip, scratch, st);
}

// scratch regions of a batch, in order, behind the 256 bytes of arrival counters; returns the bytes used
static size_t assign_scratch(Batch& B) {
  size_t off = 256;
  for (int i = 0; i < B.count; ++i) {
    B.t[i].scratch256 = static_cast<uint32_t>(off / 256);
    off += tensor_scratch_bytes(B.t[i].stat_rows, B.t[i].cols);
  }
  return off;
}

// a batch through statistics (if the direction needs them) and the update; returns the kernels launched in *launches
template <typename GT>
static int run_batch(Batch& B, int pcb, const StepParams& P, int direction, double clip, void* scratch, cudaStream_t st,
                     int* launches) {
  const bool stats = needs_stats(direction, clip);
  if (stats) {
    assign_scratch(B);
    if (int rc = run_stats<GT>(B, direction, clip, static_cast<unsigned char*>(scratch), st)) return rc;
  }
  if (int rc = launch_update<GT>(direction + 1, pcb, st, B, static_cast<unsigned char*>(scratch), stats ? 1 : 0, P))
    return rc;
  if (launches) *launches += stats ? 3 : 1;
  return 0;
}

static int run_batch_dtype(Batch& B, int grad_dtype, int pcb, const StepParams& P, int direction, double clip,
                           void* scratch, cudaStream_t st, int* launches) {
  if (grad_dtype == BL_BF16) return run_batch<__nv_bfloat16>(B, pcb, P, direction, clip, scratch, st, launches);
  if (grad_dtype == BL_F16) return run_batch<__half>(B, pcb, P, direction, clip, scratch, st, launches);
  return run_batch<float>(B, pcb, P, direction, clip, scratch, st, launches);
}

template <typename GT>
static int direction_typed(const GT* grad, int64_t rows, int64_t cols, int direction, double clip, float* D,
                           void* scratch, int device, cudaStream_t st) {
  const float* denom = nullptr;
  const float* stats = nullptr;
  if (needs_stats(direction, clip)) {
    Batch B;
    B.stat_stride = 0;
  B.stat_stride = 0;
    B.count = 1;
    B.t[0] = make_desc(nullptr, nullptr, nullptr, nullptr, nullptr, grad, rows, cols, 0, 0, 0, 0, 0);
    B.t[0].scratch256 = 1;
    if (int rc = run_stats<GT>(B, direction, clip, static_cast<unsigned char*>(scratch), st)) return rc;
    auto up = [](size_t n) { return (n + 255) & ~size_t(255); };
    unsigned char* p = static_cast<unsigned char*>(scratch) + 256;
    p += up(static_cast<size_t>(stats_panels(static_cast<int>(rows))) * cols * 4);
    denom = reinterpret_cast<const float*>(p);
    p += up(static_cast<size_t>(cols) * 4) + up(static_cast<size_t>(stats_col_chunks(static_cast<int>(cols))) * 8);
    stats = reinterpret_cast<const float*>(p);
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

// Tests and experiments: 1 sends every group of every later update through the general route (any rounding mode and
// phase width, range-checked divisions), 0 hands the choice back. Both routes give identical results.
extern "C" int bl_update_select(int route) {
  BL_REQUIRE(route == 0 || route == 1, "update_select: unknown route %d", route);
  g_update_route.store(route, std::memory_order_relaxed);
  return 0;
}

extern "C" size_t bl_update_scratch_bytes(int64_t rows, int64_t cols, int direction, double clip) {
  if (rows <= 0 || cols <= 0 || !needs_stats(direction, clip)) return 0;
  return 256 + tensor_scratch_bytes(rows, cols);
}

// scratch that lets bl_nvfp4_lattice_update_many run its tensors in the fewest launches: the largest batch's needs
extern "C" size_t bl_update_many_scratch_bytes(int count, const int64_t* rows, const int64_t* cols, int direction,
                                               double clip) {
  if (count <= 0 || rows == nullptr || cols == nullptr || !needs_stats(direction, clip)) return 0;
  size_t best = 0;
  for (int i0 = 0; i0 < count; i0 += kMaxBatch) {
    size_t need = 256;
    for (int i = i0; i < count && i < i0 + kMaxBatch; ++i)
      if (rows[i] > 0 && cols[i] > 0) need += tensor_scratch_bytes(rows[i], cols[i]);
    best = need > best ? need : best;
  }
  return best;
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
  const StepParams P = make_params(lr, decay, phase_bits, rule, kappa, rounding, strat_k);
  Batch B;
  B.stat_stride = 0;
  B.count = 1;
  B.t[0] = make_desc(codes, phase, scales_in, scales_out, global_scale, D, rows, cols, offset, rounding, seed, step,
                     strat_j);
  return launch_update<float>(0, phase_bits ? phase_cb : 0, reinterpret_cast<cudaStream_t>(stream), B, nullptr, 0, P);
}

static int check_update_args(const char* who, const void* codes, const void* phase, const void* scales, const void* gs,
                             const void* grad, int grad_dtype, int direction, double clip) {
  BL_REQUIRE(codes && scales && gs && grad, "%s: null buffer", who);
  BL_REQUIRE(direction >= BL_DIR_RAW && direction <= BL_DIR_COLNORM,
             "%s: direction %d is not built (raw, sign and colnorm are)", who, direction);
  BL_REQUIRE(clip > 0.0, "%s: clip must be positive", who);
  BL_REQUIRE(grad_dtype >= BL_F32 && grad_dtype <= BL_F16, "%s: unknown gradient dtype %d", who, grad_dtype);
  BL_REQUIRE(aligned16(codes) && aligned16(grad) && (phase == nullptr || aligned16(phase)),
             "%s: codes, phase and gradient must be 16-byte aligned", who);
  return 0;
}

extern "C" int bl_nvfp4_lattice_update(uint8_t* codes, uint8_t* phase, uint8_t* scales, const float* global_scale,
                                       const void* grad, int grad_dtype, int64_t rows, int64_t cols, uint64_t offset,
                                       int phase_bits, int phase_cb, double lr, double decay, int rounding,
                                       uint32_t seed, uint32_t step, int strat_j, int strat_k, int rule, double kappa,
                                       int direction, double clip, void* scratch, size_t scratch_bytes, int device,
                                       bl_stream_t stream) {
  if (int rc = check_common(rows, cols, phase_bits, phase_cb, phase, rounding, rule)) return rc;
  if (int rc = check_update_args("lattice_update", codes, phase, scales, global_scale, grad, grad_dtype, direction, clip))
    return rc;
  const size_t need = bl_update_scratch_bytes(rows, cols, direction, clip);
  BL_REQUIRE(need == 0 || (scratch != nullptr && scratch_bytes >= need && aligned16(scratch)),
             "lattice_update: needs %zu bytes of 16-byte aligned scratch, got %zu", need, scratch_bytes);
  BL_DEVICE(device);
  const StepParams P = make_params(lr, decay, phase_bits, rule, kappa, rounding, strat_k);
  Batch B;
  B.stat_stride = 0;
  B.count = 1;
  B.t[0] = make_desc(codes, phase, scales, scales, global_scale, grad, rows, cols, offset, rounding, seed, step, strat_j);
  return run_batch_dtype(B, grad_dtype, phase_bits ? phase_cb : 0, P, direction, clip, scratch,
                         reinterpret_cast<cudaStream_t>(stream), nullptr);
}

extern "C" int bl_nvfp4_lattice_update_many(int count, uint8_t* const* codes, uint8_t* const* phase,
                                            uint8_t* const* scales, const float* const* global_scale,
                                            const void* const* grad, const int64_t* rows, const int64_t* cols,
                                            const uint64_t* offset, const uint32_t* seed, const uint32_t* step,
                                            const int* strat_j, int grad_dtype, int phase_bits, int phase_cb, double lr,
                                            double decay, int rounding, int strat_k, int rule, double kappa,
                                            int direction, double clip, void* scratch, size_t scratch_bytes, int device,
                                            bl_stream_t stream, int* launches) {
  BL_REQUIRE(count >= 0, "lattice_update_many: negative count");
  BL_REQUIRE(count == 0 || (codes && scales && global_scale && grad && rows && cols && offset && seed && step),
             "lattice_update_many: null array");
  BL_REQUIRE(phase_bits == 0 || phase != nullptr, "lattice_update_many: null phase array");
  if (launches) *launches = 0;
  const bool stats = needs_stats(direction, clip);
  for (int i = 0; i < count; ++i) {
    if (int rc = check_common(rows[i], cols[i], phase_bits, phase_cb, phase_bits ? phase[i] : nullptr, rounding, rule))
      return rc;
    if (int rc = check_update_args("lattice_update_many", codes[i], phase_bits ? phase[i] : nullptr, scales[i],
                                   global_scale[i], grad[i], grad_dtype, direction, clip))
      return rc;
    const size_t need = bl_update_scratch_bytes(rows[i], cols[i], direction, clip);
    BL_REQUIRE(need == 0 || (scratch != nullptr && scratch_bytes >= need && aligned16(scratch)),
               "lattice_update_many: tensor %d needs %zu bytes of 16-byte aligned scratch, got %zu", i, need,
               scratch_bytes);
  }
  BL_DEVICE(device);
  const StepParams P = make_params(lr, decay, phase_bits, rule, kappa, rounding, strat_k);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // Tensors are packed into batches in order: a batch closes when it holds kMaxBatch tensors or when the next
  // tensor's statistics would not fit the scratch beside those already in it. One launch chain per batch; batches
  // follow one another on the stream and reuse the scratch.
  int i = 0;
  while (i < count) {
    Batch B;
    B.stat_stride = 0;
  B.stat_stride = 0;
    B.count = 0;
    size_t used = 256;
    while (i < count && B.count < kMaxBatch) {
      const size_t need = stats ? tensor_scratch_bytes(rows[i], cols[i]) : 0;
      if (B.count > 0 && stats && used + need > scratch_bytes) break;
      B.t[B.count++] = make_desc(codes[i], phase_bits ? phase[i] : nullptr, scales[i], scales[i], global_scale[i],
                                 grad[i], rows[i], cols[i], offset[i], rounding, seed[i], step[i],
                                 strat_j ? strat_j[i] : 0);
      used += need;
      ++i;
    }
    if (int rc = run_batch_dtype(B, grad_dtype, phase_bits ? phase_cb : 0, P, direction, clip, scratch, st, launches))
      return rc;
  }
  return 0;
}

// ---- row shards whose direction normalises over the whole weight ----
// `world` owners hold equal row shards of every weight, owner r the rows [r * rows, (r + 1) * rows). Each sums its own
// 128-row panels into ITS block of the call's exchange area, the owners exchange the blocks (ONE all-gather in place
// per call: the host's job, between the two calls), and each finalizes over all panels in ascending order:
// denominators, RMS and therefore every code, phase and scale byte equal those of the unsharded update. A shard holds a
// multiple of 128 rows, so the panels are the unsharded ones.
//
// Scratch: [256 B arrival counters][exchange area: world blocks][the tensors' regions]. A block holds, per tensor of the
// call, the [rows / 128, cols] sums of one owner, each slice rounded up to 256 bytes. A call may hold any number of
// tensors: the kernels run over batches of up to kMaxBatch of them, the exchange covers them all at once.

struct ShardLayout {
  size_t block_bytes, area_offset, total_bytes;
};

static size_t shard_slice_bytes(int64_t rows, int64_t cols) {
  return (static_cast<size_t>(stats_panels(static_cast<int>(rows))) * cols * 4 + 255) & ~size_t(255);
}

static ShardLayout shard_layout(int count, const int64_t* rows, const int64_t* cols, int world) {
  ShardLayout L{0, 256, 0};
  size_t regions = 0;
  for (int i = 0; i < count; ++i) {
    L.block_bytes += shard_slice_bytes(rows[i], cols[i]);
    regions += tensor_scratch_bytes(rows[i] * world, cols[i]);
  }
  L.total_bytes = L.area_offset + L.block_bytes * world + regions;
  return L;
}

static int check_shards(const char* who, int count, const int64_t* rows, const int64_t* cols, int world, int rank,
                        int direction, double clip, const void* scratch, size_t scratch_bytes) {
  BL_REQUIRE(count >= 0, "%s: negative count", who);
  BL_REQUIRE(count == 0 || (rows && cols), "%s: null array", who);
  BL_REQUIRE(world >= 1 && rank >= 0 && rank < world, "%s: owner %d of %d", who, rank, world);
  BL_REQUIRE(needs_stats(direction, clip), "%s: this direction has no statistics (use the plain update)", who);
  for (int i = 0; i < count; ++i) {
    BL_REQUIRE(rows[i] > 0 && cols[i] > 0 && cols[i] % 8 == 0 && rows[i] * world < (1ll << 31) && cols[i] < (1ll << 31),
               "%s: tensor %d: [rows, cols] with cols a multiple of 8 and dimensions below 2^31", who, i);
    BL_REQUIRE(rows[i] % kPanelRows == 0 || world == 1, "%s: tensor %d: a shard holds a multiple of %d rows, got %lld",
               who, i, kPanelRows, (long long)rows[i]);
  }
  const ShardLayout L = shard_layout(count, rows, cols, world);
  BL_REQUIRE(L.total_bytes < (size_t(1) << 39) && L.block_bytes / 4 < (size_t(1) << 32), "%s: statistics of %zu bytes",
             who, L.total_bytes);
  BL_REQUIRE(count == 0 || (scratch != nullptr && aligned16(scratch) && scratch_bytes >= L.total_bytes),
             "%s: needs %zu bytes of 16-byte aligned scratch, got %zu", who, L.total_bytes, scratch_bytes);
  return 0;
}

// statistics fields and scratch offsets of the descriptors in B, which are the call's tensors [first, first + B.count),
// for owner `rank` of `world`
static void place_shards(Batch& B, int first, int count, const int64_t* rows, const int64_t* cols, int world, int rank) {
  const ShardLayout L = shard_layout(count, rows, cols, world);
  B.stat_stride = static_cast<uint32_t>(L.block_bytes / 4);
  size_t slice = L.area_offset, region = L.area_offset + L.block_bytes * world;
  for (int i = 0; i < first + B.count; ++i) {
    if (i >= first) {
      TensorDesc& t = B.t[i - first];
      t.stat_rows = static_cast<int>(rows[i] * world);
      t.stat_local = stats_panels(static_cast<int>(rows[i]));
      t.stat_panel0 = rank * t.stat_local;
      t.gather256 = static_cast<uint32_t>(slice / 256);
      t.scratch256 = static_cast<uint32_t>(region / 256);
    }
    slice += shard_slice_bytes(rows[i], cols[i]);
    region += tensor_scratch_bytes(rows[i] * world, cols[i]);
  }
}

extern "C" size_t bl_update_shards_scratch_bytes(int count, const int64_t* rows, const int64_t* cols, int world) {
  if (count <= 0 || rows == nullptr || cols == nullptr || world < 1) return 0;
  return shard_layout(count, rows, cols, world).total_bytes;
}

extern "C" int bl_update_shard_stats(int count, const void* const* grad, const int64_t* rows, const int64_t* cols,
                                     int world, int rank, int grad_dtype, int direction, double clip, void* scratch,
                                     size_t scratch_bytes, uint64_t* exchange_offset, uint64_t* block_bytes, int device,
                                     bl_stream_t stream, int* launches) {
  if (launches) *launches = 0;
  if (int rc = check_shards("update_shard_stats", count, rows, cols, world, rank, direction, clip, scratch, scratch_bytes))
    return rc;
  BL_REQUIRE(count == 0 || grad, "update_shard_stats: null array");
  BL_REQUIRE(exchange_offset && block_bytes, "update_shard_stats: null output");
  BL_REQUIRE(grad_dtype >= BL_F32 && grad_dtype <= BL_F16, "update_shard_stats: unknown gradient dtype %d", grad_dtype);
  const ShardLayout L = shard_layout(count, rows, cols, world);
  *exchange_offset = L.area_offset;
  *block_bytes = L.block_bytes;
  for (int i = 0; i < count; ++i)
    BL_REQUIRE(grad[i] != nullptr && aligned16(grad[i]), "update_shard_stats: gradient %d: null or not 16-byte aligned", i);
  BL_DEVICE(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  unsigned char* sc = static_cast<unsigned char*>(scratch);
  for (int first = 0; first < count; first += kMaxBatch) {
    Batch B;
    B.count = count - first < kMaxBatch ? count - first : kMaxBatch;
    for (int k = 0; k < B.count; ++k)
      B.t[k] = make_desc(nullptr, nullptr, nullptr, nullptr, nullptr, grad[first + k], rows[first + k], cols[first + k],
                         0, 0, 0, 0, 0);
    place_shards(B, first, count, rows, cols, world, rank);
    int rc;
    if (grad_dtype == BL_BF16) rc = run_colstats<__nv_bfloat16>(B, direction, sc, st);
    else if (grad_dtype == BL_F16) rc = run_colstats<__half>(B, direction, sc, st);
    else rc = run_colstats<float>(B, direction, sc, st);
    if (rc) return rc;
    if (launches) *launches += 1;
  }
  return 0;
}

template <typename GT>
static int shard_update_typed(Batch& B, int pcb, const StepParams& P, int direction, double clip, unsigned char* scratch,
                              cudaStream_t st) {
  if (int rc = run_finalize(B, direction, clip, scratch, st)) return rc;
  return launch_update<GT>(direction + 1, pcb, st, B, scratch, 1, P);
}

extern "C" int bl_nvfp4_lattice_update_shards(int count, uint8_t* const* codes, uint8_t* const* phase,
                                              uint8_t* const* scales, const float* const* global_scale,
                                              const void* const* grad, const int64_t* rows, const int64_t* cols,
                                              int world, int rank, const uint64_t* offset, const uint32_t* seed,
                                              const uint32_t* step, const int* strat_j, int grad_dtype, int phase_bits,
                                              int phase_cb, double lr, double decay, int rounding, int strat_k, int rule,
                                              double kappa, int direction, double clip, void* scratch,
                                              size_t scratch_bytes, int device, bl_stream_t stream, int* launches) {
  if (launches) *launches = 0;
  if (int rc = check_shards("lattice_update_shards", count, rows, cols, world, rank, direction, clip, scratch,
                            scratch_bytes))
    return rc;
  BL_REQUIRE(count == 0 || (codes && scales && global_scale && grad && offset && seed && step),
             "lattice_update_shards: null array");
  BL_REQUIRE(phase_bits == 0 || phase != nullptr, "lattice_update_shards: null phase array");
  for (int i = 0; i < count; ++i) {
    if (int rc = check_common(rows[i], cols[i], phase_bits, phase_cb, phase_bits ? phase[i] : nullptr, rounding, rule))
      return rc;
    if (int rc = check_update_args("lattice_update_shards", codes[i], phase_bits ? phase[i] : nullptr, scales[i],
                                   global_scale[i], grad[i], grad_dtype, direction, clip))
      return rc;
  }
  BL_DEVICE(device);
  const StepParams P = make_params(lr, decay, phase_bits, rule, kappa, rounding, strat_k);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  unsigned char* sc = static_cast<unsigned char*>(scratch);
  const int pcb = phase_bits ? phase_cb : 0;
  for (int first = 0; first < count; first += kMaxBatch) {
    Batch B;
    B.count = count - first < kMaxBatch ? count - first : kMaxBatch;
    for (int k = 0; k < B.count; ++k) {
      const int i = first + k;
      B.t[k] = make_desc(codes[i], phase_bits ? phase[i] : nullptr, scales[i], scales[i], global_scale[i], grad[i],
                         rows[i], cols[i], offset[i], rounding, seed[i], step[i], strat_j ? strat_j[i] : 0);
    }
    place_shards(B, first, count, rows, cols, world, rank);
    int rc;
    if (grad_dtype == BL_BF16) rc = shard_update_typed<__nv_bfloat16>(B, pcb, P, direction, clip, sc, st);
    else if (grad_dtype == BL_F16) rc = shard_update_typed<__half>(B, pcb, P, direction, clip, sc, st);
    else rc = shard_update_typed<float>(B, pcb, P, direction, clip, sc, st);
    if (rc) return rc;
    if (launches) *launches += 2;
  }
  return 0;
}

extern "C" int bl_direction(const void* grad, int grad_dtype, int64_t rows, int64_t cols, int direction, double clip,
                            float* D, void* scratch, size_t scratch_bytes, int device, bl_stream_t stream) {
  BL_REQUIRE(rows > 0 && cols > 0 && cols % 8 == 0, "direction: [rows, cols] with cols a multiple of 8, got %lld x %lld",
             (long long)rows, (long long)cols);
  BL_REQUIRE(rows < (1ll << 31) && cols < (1ll << 31), "direction: dimension exceeds 2^31");
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
  if (int rc = check_update_args("lattice_update_fixed_scratch", codes, phase, scales, global_scale, grad, grad_dtype,
                                 direction, clip))
    return rc;
  const size_t need = bl_update_scratch_bytes(rows, cols, direction, clip);
  BL_REQUIRE(need <= kFixedScratchBytes,
             "lattice_update_fixed_scratch: a %lld x %lld gradient needs %zu bytes of column statistics, the built-in "
             "scratch holds %zu; use bl_nvfp4_lattice_update with a buffer of your own",
             (long long)rows, (long long)cols, need, kFixedScratchBytes);
  BL_DEVICE(device);
  void* scratch = nullptr;
  if (int rc = fixed_scratch_address(device, &scratch)) return rc;
  const StepParams P = make_params(lr, decay, phase_bits, rule, kappa, rounding, strat_k);
  Batch B;
  B.stat_stride = 0;
  B.count = 1;
  B.t[0] = make_desc(codes, phase, scales, scales, global_scale, grad, rows, cols, offset, rounding, seed, step, strat_j);
  // the statistics pass clears the arrival counter it uses and overwrites every statistic it later reads, so what an
  // earlier call left in the array does not matter
  return run_batch_dtype(B, grad_dtype, phase_bits ? phase_cb : 0, P, direction, clip, scratch,
                         reinterpret_cast<cudaStream_t>(stream), nullptr);
}
