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
// One thread owns 8 consecutive elements of a row (one 32-bit code word, cb bytes of phase, 16 or 32 bytes of
// gradient); two neighbouring lanes share a 16-element scale group and exchange its three sums with one shuffle each.
// A thread keeps its 8 columns while it walks down the rows, so per-column statistics (colnorm) stay in registers.
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

template <int PCB>
__device__ __forceinline__ void load_phase(const uint8_t* p, int pb, int ph[8]) {
  if constexpr (PCB == 0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) ph[i] = 0;
  } else {
    uint64_t v;
    if constexpr (PCB == 1) v = *p;
    else if constexpr (PCB == 2) v = *reinterpret_cast<const uint16_t*>(p);
    else if constexpr (PCB == 4) v = *reinterpret_cast<const uint32_t*>(p);
    else v = *reinterpret_cast<const uint64_t*>(p);
    const int sh = 32 - pb;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t raw = static_cast<uint32_t>(v >> (i * PCB));
      ph[i] = static_cast<int>(raw << sh) >> sh;      // sign-extend the low pb bits
    }
  }
}

template <int PCB>
__device__ __forceinline__ void store_phase(uint8_t* p, int pb, const int ph[8]) {
  if constexpr (PCB != 0) {
    const uint32_t mask = (1u << pb) - 1u;
    uint64_t v = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) v |= static_cast<uint64_t>(static_cast<uint32_t>(ph[i]) & mask) << (i * PCB);
    if constexpr (PCB == 1) *p = static_cast<uint8_t>(v);
    else if constexpr (PCB == 2) *reinterpret_cast<uint16_t*>(p) = static_cast<uint16_t>(v);
    else if constexpr (PCB == 4) *reinterpret_cast<uint32_t*>(p) = static_cast<uint32_t>(v);
    else *reinterpret_cast<uint64_t*>(p) = v;
  }
}

// latent position from the phase code (bitlattice/reference.py:277-281)
__device__ __forceinline__ float latent(float w, float lo, float hi, int code, float inv_half) {
  const float c = static_cast<float>(code) * inv_half;   // division by 2^(pb-1) is exact either way
  return c < 0.0f ? w + c * (w - lo) * 0.5f : w + c * (hi - w) * 0.5f;
}

// projection of target t around the nearest level w with neighbours lo/hi (bitlattice/reference.py:250-274);
// returns the move (-1, 0, +1) and the new phase code
__device__ __forceinline__ int project(float t, float w, float lo, float hi, float u, int pb, float half, int* code) {
  if (pb == 0) {
    const bool up = t >= w;
    const float a = up ? w : lo, b = up ? hi : w;
    const float gap = b - a;
    const float p = gap > 0.0f ? (t - a) / gap : 0.0f;
    const bool take_b = u < p;
    *code = 0;
    return up ? (take_b ? 1 : 0) : (take_b ? 0 : -1);
  }
  const bool left = t < w;
  const float width = left ? (w - lo) * 0.5f : (hi - w) * 0.5f;
  float c = width > 0.0f ? (t - w) / width : 0.0f;
  c = fminf(fmaxf(c, -1.0f), 1.0f);
  const float q = c * half;
  const float fl = floorf(q);
  float k = fl + ((u < (q - fl)) ? 1.0f : 0.0f);
  int move = 0;
  if (k >= half) {
    if (hi > w) {
      move = 1;
      k = -half;
    } else {
      k = half - 1.0f;
    }
  }
  *code = static_cast<int>(k);
  return move;
}

// DIR: 0 = D given as fp32, 1 = raw, 2 = sign, 3 = colnorm (the gradient is read as GT)
template <int PCB, int DIR, typename GT>
__global__ void __launch_bounds__(kThreads) update_kernel(uint8_t* __restrict__ codes, uint8_t* __restrict__ phase,
                                                          const uint8_t* scales_in, uint8_t* scales_out,
                                                          const float* __restrict__ global_scale,
                                                          const GT* __restrict__ grad, const float* __restrict__ denom,
                                                          const float* __restrict__ stats, int64_t rows, int64_t cols,
                                                          StepParams P) {
  const int64_t cc = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;   // 8-column chunk of this thread
  const bool active = cc * 8 < cols;
  const float gs = global_scale[0];
  const float div = stats != nullptr ? stats[1] : 1.0f;
  const bool use_div = stats != nullptr;
  float den[8];
  if (DIR == 3 && active) {
    const float4 a = reinterpret_cast<const float4*>(denom + cc * 8)[0];
    const float4 b = reinterpret_cast<const float4*>(denom + cc * 8)[1];
    den[0] = a.x; den[1] = a.y; den[2] = a.z; den[3] = a.w;
    den[4] = b.x; den[5] = b.y; den[6] = b.z; den[7] = b.w;
  }
  const float half = static_cast<float>(1 << (P.pb > 0 ? P.pb - 1 : 0));
  const float inv_half = 1.0f / half;
  const int64_t code_stride = cols / 2, phase_stride = cols * PCB / 8, scale_stride = cols / 16;
  const int64_t row_step = static_cast<int64_t>(gridDim.y) * blockDim.y;

  for (int64_t r = static_cast<int64_t>(blockIdx.y) * blockDim.y + threadIdx.y; r < rows; r += row_step) {
    float a[8], tau[8], tf[8];
    float s_old = 1.0f;
    uint32_t sb_old = 0;
    if (active) {
      const uint32_t word = *reinterpret_cast<const uint32_t*>(codes + r * code_stride + cc * 4);
      int ph[8];
      load_phase<PCB>(phase + r * phase_stride + cc * PCB, P.pb, ph);
      float gv[8];
      load8(grad + r * cols + cc * 8, gv);
      sb_old = scales_in[r * scale_stride + (cc >> 1)];
      s_old = e4m3_decode(sb_old) * gs;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int rk = rank_of_code((word >> (4 * i)) & 0xFu);
        const float av = level_of_rank(rk);
        const float lo = level_of_rank(max(rk - 1, 0));
        const float hi = level_of_rank(min(rk + 1, 14));
        float u = gv[i];
        if (DIR == 2) u = static_cast<float>((u > 0.0f) - (u < 0.0f));
        if (DIR == 3) u = u / den[i];
        if (DIR != 0 && use_div) u = u / div;
        const float d = u / s_old;
        const float lam = P.pb == 0 ? av : latent(av, lo, hi, ph[i], inv_half);
        a[i] = av;
        tau[i] = lam * P.decay - P.lr * d;
        tf[i] = P.rule == BL_RULE_FIT_LATENT ? tau[i] : av * P.decay - P.lr * d;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) a[i] = tau[i] = tf[i] = 0.0f;
    }
    float s_new = s_old;
    uint32_t sb_new = sb_old;
    if (P.rule != BL_RULE_FIXED) {
      float saa = 0.0f, sat = 0.0f, stt = 0.0f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        saa = saa + a[i] * a[i];
        sat = sat + a[i] * tf[i];
        stt = stt + tf[i] * tf[i];
      }
      saa = saa + __shfl_xor_sync(0xffffffffu, saa, 1);
      sat = sat + __shfl_xor_sync(0xffffffffu, sat, 1);
      stt = stt + __shfl_xor_sync(0xffffffffu, stt, 1);
      float rr = saa > 0.0f ? sat / saa : 1.0f;
      rr = fminf(fmaxf(rr, P.r_lo), P.r_hi);
      const uint32_t bits = e4m3_encode(s_old * rr / gs);
      const float cand = e4m3_decode(bits) * gs;
      const float q = cand / s_old;
      const float before = stt - 2.0f * sat + saa;
      const float after = q * q * saa - 2.0f * q * sat + stt;
      if ((after <= before) && isfinite(cand) && cand > 0.0f) {
        s_new = cand;
        sb_new = bits;
      }
    }
    if (!active) continue;
    if ((threadIdx.x & 1) == 0) scales_out[r * scale_stride + (cc >> 1)] = static_cast<uint8_t>(sb_new);
    const uint32_t idx0 = P.offset + static_cast<uint32_t>(static_cast<uint64_t>(r) * cols + cc * 8);
    uint32_t word = 0;
    int ph[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float t = tau[i] * s_old / s_new;
      t = fminf(fmaxf(t, -6.0f), 6.0f);
      int rk = nearest_rank(t);
      const float w = level_of_rank(rk);
      const float lo = level_of_rank(max(rk - 1, 0));
      const float hi = level_of_rank(min(rk + 1, 14));
      const float u = rounding_u(P.rp, idx0 + i);
      rk += project(t, w, lo, hi, u, P.pb, half, &ph[i]);
      rk = min(max(rk, 0), 14);
      word |= code_of_rank(rk) << (4 * i);
    }
    *reinterpret_cast<uint32_t*>(codes + r * code_stride + cc * 4) = word;
    store_phase<PCB>(phase + r * phase_stride + cc * PCB, P.pb, ph);
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

// threads along x cover 8-column chunks (a power of two >= 32 so a warp never spans two rows), y covers rows
static Geometry geometry(int64_t rows, int64_t cols, int device) {
  const int64_t cpr = cols / 8;
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

template <int DIR, typename GT>
static void launch_update(int pcb, const Geometry& g, cudaStream_t st, uint8_t* codes, uint8_t* phase,
                          const uint8_t* sin, uint8_t* sout, const float* gs, const GT* grad, const float* denom,
                          const float* stats, int64_t rows, int64_t cols, const StepParams& P) {
  switch (pcb) {
    case 0: update_kernel<0, DIR, GT><<<g.grid, g.block, 0, st>>>(codes, phase, sin, sout, gs, grad, denom, stats, rows, cols, P); break;
    case 1: update_kernel<1, DIR, GT><<<g.grid, g.block, 0, st>>>(codes, phase, sin, sout, gs, grad, denom, stats, rows, cols, P); break;
    case 2: update_kernel<2, DIR, GT><<<g.grid, g.block, 0, st>>>(codes, phase, sin, sout, gs, grad, denom, stats, rows, cols, P); break;
    case 4: update_kernel<4, DIR, GT><<<g.grid, g.block, 0, st>>>(codes, phase, sin, sout, gs, grad, denom, stats, rows, cols, P); break;
    default: update_kernel<8, DIR, GT><<<g.grid, g.block, 0, st>>>(codes, phase, sin, sout, gs, grad, denom, stats, rows, cols, P); break;
  }
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
  const Geometry g = geometry(rows, cols, device);
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
