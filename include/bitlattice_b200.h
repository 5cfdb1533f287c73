/*
 * C ABI of libbitlattice_b200.so: the NVFP4 LatticeTensor linear layer (quantizers + block-scaled FP4 GEMM) and the
 * lattice optimizer update, hand-written CUDA for sm_100a.
 *
 * Every entry point replaces one operator of the reference's native extension (`torch.ops.bitlattice.*`, schemas in
 * the reference's csrc/bindings.cpp:75-134) for the NVFP4 format only. Conventions shared by all of them:
 *   - plain device pointers and sizes; the library never allocates or frees device memory (the caller owns every
 *     buffer, outputs included) -- scratch memory, where an operation needs some, is passed in and its size comes
 *     from the matching *_scratch_bytes function. Two exceptions, both stated at their declarations:
 *     bl_nvfp4_lattice_update_fixed_scratch keeps its scratch in an array inside the library image, and the
 *     diagnostic bl_selftest_division makes a temporary 8-byte allocation;
 *   - all buffers are contiguous and 16-byte aligned; shapes are validated before anything is launched;
 *   - work is enqueued on `stream` of CUDA device `device` and the call returns without synchronizing;
 *   - the return value is 0 on success, non-zero on failure; bl_last_error() then describes the failure
 *     (thread-local), which the Python layer raises as RuntimeError, as TORCH_CHECK does in the reference.
 *
 * Storage layout (bitlattice/formats.py:415, bitlattice/packing.py:22-33): a [rows, cols] NVFP4 tensor is
 *   codes   uint8 [rows, cols/2]   E2M1 nibbles, element 2j in the low nibble of byte j
 *   scales  uint8 [rows, cols/16]  E4M3 (float8_e4m3fn) bit patterns, one per 16 consecutive elements of a row
 *   global  float [1]              per-tensor scale; value = level(code) * scale * global
 * "Blocked" scales are the same bytes in the 128x4-tiled order of block-scaled GEMMs (bitlattice/backend.py:179-188):
 * offset(r, c) = ((r/128) * ceil(cols16/4) + c/4) * 512 + (r%32) * 16 + ((r/32)%4) * 4 + c%4, zero padded.
 */
#ifndef BITLATTICE_B200_H
#define BITLATTICE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define BL_API __attribute__((visibility("default")))
#else
#define BL_API
#endif

typedef struct CUstream_st* bl_stream_t; /* a cudaStream_t */

/* element types of dense inputs / outputs */
enum { BL_F32 = 0, BL_BF16 = 1, BL_F16 = 2 };
/* rounding of the lattice projection (bitlattice/_ops.py:22) */
enum { BL_ROUND_SR = 0, BL_ROUND_STRAT = 1, BL_ROUND_RTN = 2 };
/* group-scale rule (bitlattice/_ops.py:23) */
enum { BL_RULE_FIXED = 0, BL_RULE_FIT = 1, BL_RULE_FIT_LATENT = 2 };
/* update direction (bitlattice/_ops.py:24); only these three are built */
enum { BL_DIR_RAW = 0, BL_DIR_SIGN = 1, BL_DIR_COLNORM = 2 };
/* layout of block-scale outputs */
enum { BL_SF_ROWMAJOR = 0, BL_SF_BLOCKED = 1 };
/* four-over-six selection criterion: squared or absolute error of the dequantized block */
enum { BL_SELECT_MSE = 0, BL_SELECT_MAE = 1 };
enum { BL_Q_RTN = 0, BL_Q_SR = 1, BL_Q_EDEN = 2 };    /* modes of bl_nvfp4_quantize_general */

BL_API int bl_version(void);
BL_API const char* bl_last_error(void);

/* ---- lattice update ------------------------------------------------------------------------------------------- */

/* Replaces torch.ops.bitlattice.step_quantized for NVFP4 (csrc/bindings.cpp:77-81, csrc/lattice.cu:407-439,
 * kernel :125-175). One lattice step given the fp32 direction D [rows*cols]: codes and phase are updated in place,
 * the new scale bytes go to scales_out (scales_in is only read; the two may be the same buffer).
 * phase: phase_bits-bit two's complement values in phase_cb-bit containers {1,2,4,8} packed little-endian along
 * cols, [rows, cols*phase_cb/8]; NULL when phase_bits == 0. offset: RNG index of element (0, 0), so that a row
 * shard or row tile draws the numbers of the whole tensor (csrc/update.cpp:50). cols % 16 == 0. */
BL_API int bl_nvfp4_step_quantized(uint8_t* codes, uint8_t* phase, const uint8_t* scales_in, uint8_t* scales_out,
                            const float* global_scale, const float* D, int64_t rows, int64_t cols, uint64_t offset,
                            int phase_bits, int phase_cb, double lr, double decay, int rounding, uint32_t seed,
                            uint32_t step, int strat_j, int strat_k, int rule, double kappa, int device,
                            bl_stream_t stream);

/* Scratch bytes bl_nvfp4_lattice_update / bl_direction need for a [rows, cols] gradient (0 when none is needed). */
BL_API size_t bl_update_scratch_bytes(int64_t rows, int64_t cols, int direction, double clip);

/* Replaces torch.ops.bitlattice.lattice_update for NVFP4 (csrc/bindings.cpp:119-124, csrc/update.cpp:30-53) with the
 * direction fused: the gradient G [rows, cols] (grad_dtype BL_BF16 / BL_F32 / BL_F16) is read once by the update
 * kernel and the fp32 direction is never written to memory. D = U / max(rms(U)/clip, 1) with U = G, sign(G) or
 * G / (sqrt(mean_rows(G^2)) + 1e-30) (bitlattice/_ops.py:135-144, bitlattice/reference.py:488-490). Scales are
 * updated in place. Directions other than sign with clip >= 1 first reduce column statistics into `scratch`
 * (fixed reduction order: 16 rows summed sequentially, eight such sums in ascending order per 128-row panel, then the
 * panels in ascending order). */
BL_API int bl_nvfp4_lattice_update(uint8_t* codes, uint8_t* phase, uint8_t* scales, const float* global_scale,
                            const void* grad, int grad_dtype, int64_t rows, int64_t cols, uint64_t offset,
                            int phase_bits, int phase_cb, double lr, double decay, int rounding, uint32_t seed,
                            uint32_t step, int strat_j, int strat_k, int rule, double kappa, int direction,
                            double clip, void* scratch, size_t scratch_bytes, int device, bl_stream_t stream);

/* bl_nvfp4_lattice_update for `count` tensors in one call: the role of the reference's native tile loop
 * (csrc/update.cpp:30-53, which exists so that the loop runs without the interpreter lock), applied across the tensors
 * of a parameter group, whose shards can be so small that launches, not the GPU, set the pace. The tensors are
 * packed, in order, into batches of up to 40; a batch is ONE chain of launches (column statistics of all its tensors,
 * their reduction, the update of all its tensors), each kernel finding its tensor from a descriptor list passed in the
 * kernel parameters. Per-tensor arrays of length count (phase may be NULL when phase_bits == 0, strat_j when rounding
 * is not BL_ROUND_STRAT); the other settings are shared. `scratch` must cover the largest single
 * bl_update_scratch_bytes among the tensors; with bl_update_many_scratch_bytes(...) bytes every batch is full, with
 * less a batch closes when the next tensor's statistics would not fit beside those in it. launches (nullable) receives
 * the number of kernels launched. Results are identical to calling bl_nvfp4_lattice_update per tensor. */
BL_API size_t bl_update_many_scratch_bytes(int count, const int64_t* rows, const int64_t* cols, int direction, double clip);
BL_API int bl_nvfp4_lattice_update_many(int count, uint8_t* const* codes, uint8_t* const* phase, uint8_t* const* scales,
                                 const float* const* global_scale, const void* const* grad, const int64_t* rows,
                                 const int64_t* cols, const uint64_t* offset, const uint32_t* seed,
                                 const uint32_t* step, const int* strat_j, int grad_dtype, int phase_bits, int phase_cb,
                                 double lr, double decay, int rounding, int strat_k, int rule, double kappa,
                                 int direction, double clip, void* scratch, size_t scratch_bytes, int device,
                                 bl_stream_t stream, int* launches);

/* Row shards of weights whose direction normalises over ALL rows (colnorm; raw and sign with clip < 1). The reference
 * has no sharded update; its unsharded one (bitlattice/optim/lattice.py:671-694 with the colnorm of
 * bitlattice/_ops.py:110-144) is what the owners of the shards reproduce together, bit for bit. `world` owners hold
 * equal shards of every weight of the call, owner `rank` the rows [rank * rows, (rank + 1) * rows) of a weight
 * [world * rows, cols]; rows is a multiple of 128.
 *   1. bl_update_shard_stats: each owner sums the 128-row panels of ITS rows, all tensors of the call, into block
 *      number `rank` of the call's exchange area: `world` blocks of *block_bytes bytes starting *exchange_offset bytes
 *      into `scratch`;
 *   2. the host exchanges the blocks among the owners (ONE in-place all-gather of world * block_bytes bytes on the
 *      same stream, whatever the number of tensors) -- the library makes no collective call;
 *   3. bl_nvfp4_lattice_update_shards: every owner sums all panels in ascending order of their rows (the unsharded
 *      order), derives the column denominators and the RMS divisor of the whole weights, and updates its rows.
 *      `offset` is the RNG index of the shard's first element (rank * rows * cols for a weight that is not itself a
 *      tile of something larger).
 * Both calls get the same rows / cols / world / rank and the same scratch of
 * bl_update_shards_scratch_bytes(count, rows, cols, world) bytes, untouched in between except for step 2. Per 40
 * tensors the first call launches one kernel (statistics) and the second two (reduction, update); launches (nullable)
 * receives the number. */
BL_API size_t bl_update_shards_scratch_bytes(int count, const int64_t* rows, const int64_t* cols, int world);
BL_API int bl_update_shard_stats(int count, const void* const* grad, const int64_t* rows, const int64_t* cols, int world,
                          int rank, int grad_dtype, int direction, double clip, void* scratch, size_t scratch_bytes,
                          uint64_t* exchange_offset, uint64_t* block_bytes, int device, bl_stream_t stream,
                          int* launches);
BL_API int bl_nvfp4_lattice_update_shards(int count, uint8_t* const* codes, uint8_t* const* phase, uint8_t* const* scales,
                                   const float* const* global_scale, const void* const* grad, const int64_t* rows,
                                   const int64_t* cols, int world, int rank, const uint64_t* offset,
                                   const uint32_t* seed, const uint32_t* step, const int* strat_j, int grad_dtype,
                                   int phase_bits, int phase_cb, double lr, double decay, int rounding, int strat_k,
                                   int rule, double kappa, int direction, double clip, void* scratch,
                                   size_t scratch_bytes, int device, bl_stream_t stream, int* launches);

/* The update kernel has two routes with identical results: a fast one (stochastic rounding, 1..7 phase bits: packed
 * fp32 pairs, one range check per element instead of one per division; single groups whose values leave that range
 * fall back) and a general one. 1 forces the general route for every later update of this process (tests,
 * experiments), 0 hands the choice back. No counterpart in the reference. */
BL_API int bl_update_select(int route);

/* No counterpart in the reference. The same update as bl_nvfp4_lattice_update for callers that have no way to hand
 * over scratch memory: code running where cudaMalloc and the framework allocators are off limits -- a serving loop
 * with a frozen memory plan, a host thread that must not take the allocator's locks or trigger its implicit device
 * synchronisation, a plugin that only ever receives the tensors it works on. The column statistics go into an array
 * that is part of the library image (bl_update_fixed_scratch_capacity() bytes, 4 MiB; every GPU that loads the
 * library holds it until the process exits). Nothing is allocated or freed, here or in anything this calls.
 *  - Shapes whose statistics do not fit (bl_update_scratch_bytes(...) above the capacity) are refused with an error;
 *    4 MiB covers e.g. 12288 x 4096, 4096 x 12288 and 8192 x 8192.
 *  - The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that device
 *    current) and keeps it; make that first call before any stream capture.
 *  - All calls on a device share the one array. Each call resets the arrival counter it uses and overwrites every
 *    statistic before reading it, so earlier contents never matter; two calls whose kernels may run at the same time
 *    (different streams) race on it -- order them. */
BL_API size_t bl_update_fixed_scratch_capacity(void);
BL_API int bl_nvfp4_lattice_update_fixed_scratch(uint8_t* codes, uint8_t* phase, uint8_t* scales,
                                                 const float* global_scale, const void* grad, int grad_dtype,
                                                 int64_t rows, int64_t cols, uint64_t offset, int phase_bits,
                                                 int phase_cb, double lr, double decay, int rounding, uint32_t seed,
                                                 uint32_t step, int strat_j, int strat_k, int rule, double kappa,
                                                 int direction, double clip, int device, bl_stream_t stream);

/* Replaces torch.ops.bitlattice.direction for raw / sign / colnorm (csrc/bindings.cpp:90-92,
 * csrc/directions.cpp:145-191): writes the fp32 direction D [rows, cols]. */
BL_API int bl_direction(const void* grad, int grad_dtype, int64_t rows, int64_t cols, int direction, double clip, float* D,
                 void* scratch, size_t scratch_bytes, int device, bl_stream_t stream);

/* ---- storage <-> dense ---------------------------------------------------------------------------------------- */

/* Replaces torch.ops.bitlattice.dequantize for NVFP4 (csrc/bindings.cpp:86-88, csrc/lattice.cu:323-339,466-492):
 * out[r][c] = level * (scale * global) in out_dtype. */
BL_API int bl_nvfp4_dequantize(const uint8_t* codes, const uint8_t* scales, const float* global_scale, int64_t rows,
                        int64_t cols, void* out, int out_dtype, int device, bl_stream_t stream);

/* ---- operand quantizers --------------------------------------------------------------------------------------- */

/* The amax pass of bitlattice/backend.py:240-241: out[0] = max|x|, out[1] = max(out[0] / (6*448), 1e-12) (the
 * per-tensor scale), out[2] is used as a counter, out[3] = max(out[0] / (6*256), 1e-12) (the per-tensor scale of the
 * four-over-six recipe, bitlattice/fp4ref.py:110-113). out: 4 floats. */
BL_API int bl_nvfp4_amax(const void* x, int dtype, int64_t n, float* out, int device, bl_stream_t stream);

/* Replaces torch.ops.bitlattice.quantize_nvfp4 (csrc/bindings.cpp:96, csrc/act_quant.cu:180-225): x [rows, cols]
 * -> codes [rows, cols/2] + scales, blocks of 16 along cols, against the per-tensor scale *global_scale.
 * seed < 0: round to nearest, ties to the lower level, v / (scale*global) (== bitlattice/reference.py:164-235).
 * seed >= 0: stochastic rounding with u = hash(flat index, seed, step), v * (1/(scale*global))
 * (== bitlattice/fp4ref.py:71-78,135-137). sf_layout BL_SF_BLOCKED needs
 * bl_blocked_scale_bytes(rows, cols/16) bytes and receives the zero padding too. cols % 16 == 0. */
BL_API int bl_nvfp4_quantize(const void* x, int dtype, int64_t rows, int64_t cols, const float* global_scale, int64_t seed,
                      uint32_t step, uint8_t* codes, uint8_t* scales, int sf_layout, int device, bl_stream_t stream);

/* bl_nvfp4_amax followed by bl_nvfp4_quantize against the scale it finds (amax4[1]), enqueued by one call: the pair of
 * operators of bitlattice/backend.py:237-244 (quantize_fp4). amax4: 4 floats as bl_nvfp4_amax's out. */
BL_API int bl_nvfp4_amax_quantize(const void* x, int dtype, int64_t rows, int64_t cols, float* amax4, int64_t seed,
                           uint32_t step, uint8_t* codes, uint8_t* scales, int sf_layout, int device,
                           bl_stream_t stream);

/* The forward-activation quantizer of the '4over6' recipe (bitlattice/backend.py:131, the general quantizer
 * torch.ops.bitlattice.nvfp4_quantize with four_over_six, csrc/nvfp4.cu:553-600; Python twin bitlattice/fp4ref.py:103-135):
 * round to nearest with ties to the even code, v * (1 / (scale*global)); every block is quantized with its maximum
 * mapped to 6 and to 4 and keeps the candidate with the smaller error (select: BL_SELECT_MSE / BL_SELECT_MAE; six on
 * equality; error sums in element order). *global_scale is amax / (6 * 256) (out[3] of bl_nvfp4_amax). */
BL_API int bl_nvfp4_quantize_4over6(const void* x, int dtype, int64_t rows, int64_t cols, const float* global_scale,
                             int select, uint8_t* codes, uint8_t* scales, int sf_layout, int device,
                             bl_stream_t stream);

/* Replaces torch.ops.bitlattice.nvfp4_quantize (csrc/bindings.cpp schema "nvfp4_quantize", csrc/nvfp4.cu:553-600; Python
 * twin bitlattice/fp4ref.py:103-150): the quantizer of the 128-rotation recipes. x: dense [R, C] of `dtype`, or -- with
 * w_scales / w_global given -- the packed codes [R, C/2] of an NVFP4 matrix with its row-major scale bytes and
 * per-tensor scale (then transpose must be set; values are formed as (level * scale) * global). Output: codes and
 * scales of x (transpose = 0) or of x^T [C, R] (transpose = 1), blocks of 16 along the output's last dimension.
 *   mode           BL_Q_RTN: round to nearest, ties to the even code, v * (1 / (scale*global));
 *                  BL_Q_SR: stochastic rounding, u = hash(flat output index, seed, 0);
 *                  BL_Q_EDEN: round-to-nearest codes; per 128 elements S = <x,x> / <x,x_rtn>, every block scale times
 *                  S rounded stochastically to E4M3, u = hash(flat block index, seed ^ 0x9E3779B9, 0); needs rotate
 *   four_over_six  every block keeps the better (select: BL_SELECT_MSE / BL_SELECT_MAE) of "maximum mapped to 6" and
 *                  "maximum mapped to 4"; the per-tensor scale then uses 256 instead of 448
 *   rotate         x <- (x * signs) H_128 / sqrt(128) over consecutive 128-element blocks of the output's last
 *                  dimension (a multiple of 128), signs = hash(j, rotate_seed, 0x5151) < 0.5 ? -1 : 1 (rotate_seed < 0:
 *                  seed)
 *   given_global   device pointer to the per-tensor scale to use, or NULL: max|rotated x| / (6 * 448 or 256), at
 *                  least 1e-12, rounded up to a power of two when pow2 is set
 * Summation orders (the reference fixes none; its test allows 2e-3 of codes and scales to differ): butterflies with
 * strides 1 .. 64 then the normalisation; error and MS-EDEN sums over groups of four elements, then pairwise.
 * out_global: 1 float (written); scratch: 1 float of device memory (the amax). amax_out (nullable, 1 float): receives
 * max|rotated x| whether the per-tensor scale was given or computed -- the "seen" amax of the reference's delayed
 * scales (csrc/nvfp4.cu:435, 459-460). sf_layout as bl_nvfp4_quantize. */
BL_API int bl_nvfp4_quantize_general(const void* x, int dtype, int64_t R, int64_t C, int transpose, int mode,
                              int four_over_six, int select, int rotate, int64_t seed, int64_t rotate_seed,
                              const float* given_global, int pow2, const uint8_t* w_scales, const float* w_global,
                              uint8_t* codes, uint8_t* scales, int sf_layout, float* out_global, float* scratch,
                              float* amax_out, int device, bl_stream_t stream);

/* Replaces torch.ops.bitlattice.fp4_fold_scales (csrc/fold.cu:12-33; Python twin bitlattice/backend.py:688-697): the
 * blocked scale buffer of operands concatenated along K -- row_tiles x tiles_per_row tiles of 512 bytes, column tile t
 * belonging to piece piece[t] (device int32 [tiles_per_row]) whose per-tensor scale is the power of two g[piece] -- is
 * brought to the common scale max(g): every byte times g[piece] / max(g), rounded to E4M3. *g_max receives max(g);
 * *rounded (device, 64-bit) is incremented by the number of non-zero products below 2^-6 (rounded, not exact). */
BL_API int bl_fp4_fold_scales(uint8_t* scales, int64_t row_tiles, int64_t tiles_per_row, const int* piece, const float* g,
                       int pieces, float* g_max, unsigned long long* rounded, int device, bl_stream_t stream);

/* Replaces torch.ops.bitlattice.quantize_nvfp4_t (csrc/bindings.cpp:97-98, csrc/act_quant.cu:100-148,230-270):
 * x [M, K] -> NVFP4 of x^T, codes [K, M/2] + scales over [K, M/16], blocks of 16 along M, each block optionally
 * rotated v <- v H (H: fp32 [16,16] or NULL; sequential sum over the 16 inputs). global_bound (device, [1]): a
 * bound on the rotated tensor's per-tensor scale, used as max(bound*2688/2688, 1e-12); NULL: an amax pass over the
 * rotated tensor finds it (amax_scratch: 4 floats). global_out [1] receives the scale used. M % 16 == 0. */
BL_API int bl_nvfp4_quantize_t(const void* x, int dtype, int64_t M, int64_t K, const float* H, int64_t seed, uint32_t step,
                        const float* global_bound, float* amax_scratch, uint8_t* codes, uint8_t* scales,
                        float* global_out, int sf_layout, int device, bl_stream_t stream);

/* Replaces torch.ops.bitlattice.requantize_nvfp4_t (csrc/bindings.cpp:99, csrc/act_quant.cu:150-175,273-294):
 * NVFP4 W [N, K] -> NVFP4 of W^T, codes [K, N/2] + scales over [K, N/16], same per-tensor scale (copied to
 * global_out). N % 16 == 0, K % 16 == 0. */
BL_API int bl_nvfp4_requantize_t(const uint8_t* codes, const uint8_t* scales, const float* global_scale, int64_t N, int64_t K,
                          uint8_t* out_codes, uint8_t* out_scales, float* global_out, int sf_layout, int device,
                          bl_stream_t stream);

/* Bytes of a blocked scale buffer for [rows, cols16] scales. */
BL_API size_t bl_blocked_scale_bytes(int64_t rows, int64_t cols16);

/* Replaces bitlattice.backend.to_blocked (bitlattice/backend.py:179-188): row-major scale bytes [rows, cols16] ->
 * blocked layout with zero padding. */
BL_API int bl_nvfp4_scales_to_blocked(const uint8_t* scales, int64_t rows, int64_t cols16, uint8_t* out, int device,
                               bl_stream_t stream);

/* No counterpart in the reference (it has no tensor parallelism): GEMM operands of a full weight W [p*n, K] from the
 * p row shards an all-gather delivered. recv holds p buffers rank_stride bytes apart; inside each, at the given byte
 * offsets, the shard's codes [n, K/2], its blocked scales (bl_blocked_scale_bytes(n, K/16) bytes), the codes [K, n/2]
 * and the row-major scales [K, n/16] of its re-quantized W^T slice (bl_nvfp4_requantize_t of the shard). Outputs:
 * codes [p*n, K/2], sf (p blocked buffers in rank order = the blocked scales of W), tcodes [K, p*n/2], tsf (blocked
 * scales of W^T, bl_blocked_scale_bytes(K, p*n/16) bytes). n % 128 == 0, K % 64 == 0, offsets % 16 == 0. */
BL_API int bl_nvfp4_assemble_gathered(const uint8_t* recv, int64_t rank_stride, int p, int64_t n, int64_t K,
                               int64_t off_codes, int64_t off_sf, int64_t off_tcodes, int64_t off_tsf, uint8_t* codes,
                               uint8_t* sf, uint8_t* tcodes, uint8_t* tsf, int device, bl_stream_t stream);

/* ---- GEMM ----------------------------------------------------------------------------------------------------- */

/* Replaces bitlattice.backend.fp4_mm, i.e. torch._scaled_mm / F.scaled_mm on NVFP4 operands plus the per-tensor
 * scale kernel (bitlattice/backend.py:267-290, csrc/act_quant.cu:299-336):
 *   out[m][n] = (*a_global * *b_global) * sum_k A[m][k] * B[n][k],  A [M, K], B [N, K], both K-major NVFP4
 * on tcgen05 block-scaled FP4 tensor cores with fp32 accumulation in tensor memory. a_sf / b_sf: blocked scales.
 * out: [M, N] in out_dtype, row stride ldc elements. K % 32 == 0, N % 8 == 0. */
BL_API int bl_nvfp4_gemm(const uint8_t* a_codes, const uint8_t* a_sf, const float* a_global, const uint8_t* b_codes,
                  const uint8_t* b_sf, const float* b_global, int64_t M, int64_t N, int64_t K, void* out,
                  int out_dtype, int64_t ldc, int device, bl_stream_t stream);

/* out += (A B^T) * (*a_global * *b_global), same operands and rules as bl_nvfp4_gemm. Replaces the dense add autograd
 * performs when several projections read one input (the reference sums their input gradients as separate tensors,
 * bitlattice/tensor.py:269 + autograd): the product is rounded to out_dtype, then the fp32 sum of the old value and the
 * product is rounded to out_dtype -- the bits of `out + product` computed as two tensors. */
BL_API int bl_nvfp4_gemm_accumulate(const uint8_t* a_codes, const uint8_t* a_sf, const float* a_global,
                                    const uint8_t* b_codes, const uint8_t* b_sf, const float* b_global, int64_t M,
                                    int64_t N, int64_t K, void* out, int out_dtype, int64_t ldc, int device,
                                    bl_stream_t stream);

/* Every wait inside the GEMM kernel is bounded; when one expires the kernel records which (1 producer, 2 MMA issuer,
 * 3 epilogue), frees its tensor memory and returns. This call synchronizes `device`, stores the recorded code
 * (0: none) in *status and clears it. No counterpart in the reference (cuBLASLt reports nothing of the kind). */
BL_API int bl_nvfp4_gemm_status(int* status, int device);

/* The flag is sticky: once a wait has expired, every GEMM on the device gives up on its waits early (and leaves a
 * partial output) until bl_nvfp4_gemm_status has read and cleared it, so results are not to be trusted before that.
 * bl_nvfp4_gemm_status_async lets a training loop watch the flag without a synchronisation of its own: it enqueues,
 * behind the work already on `stream`, a copy of the flag (not cleared) into *host_status, which must be page-locked
 * host memory; read it once the stream has passed that point. The Python optimizer does this every step and raises
 * before applying updates computed from a failed GEMM. No counterpart in the reference. */
BL_API int bl_nvfp4_gemm_status_async(int* host_status, int device, bl_stream_t stream);

/* Diagnostic, no counterpart in the reference: runs the give-up path of the kernels' bounded waits in isolation -- one
 * warp waits, with a short limit, on a barrier nothing arrives on; no copy or tensor-memory operation is in flight.
 * *status receives the code the wait recorded (9), *returned 2 when the kernel ran to its end afterwards. Synchronous;
 * clears the error flag before and after; scratch: 4 bytes of device memory. */
BL_API int bl_selftest_bounded_wait(int* status, int* returned, int* scratch, int device);

/* Diagnostic, no counterpart in the reference: the tensor-pipe ceiling for block-scaled FP4. Every SM issues `iters`
 * k-tiles of four 128 x 256 x 64 MMAs on one resident pair of operand tiles, with no loads, scale copies or epilogue in
 * the loop (mma_n = 128: the same work issued as MMAs of 128 columns; mma_n = 1256: 256 columns with the twelve scale
 * copies of a k-tile issued in order before its MMAs); *ms receives the CUDA-event duration (after a
 * warm-up launch), *flops the work done. The GEMM kernels'
 * roofline fraction is quoted against flops / ms measured this way on the same GPU. Synchronous; scratch: 4 bytes of
 * device memory. */
BL_API int bl_selftest_mma_peak(int iters, int mma_n, float* ms, double* flops, int* scratch, int device);

/* SwiGLU glue between the gate/up and the down projection, every intermediate rounded to the activation type as
 * PyTorch autograd rounds F.silu(g) * u. Replaces torch.ops.bitlattice.swiglu_fwd / swiglu_bwd
 * (csrc/bindings.cpp:126-129, csrc/swiglu.cu:20-80):
 *   forward   a  = T(T(silu(g)) * u)
 *   backward  du = T(da * T(silu(g))),  dg = T(T(da * u) * sig * (1 + g * (1 - sig))),  sig = 1 / (1 + exp(-g))
 * g, u, da, a, dg, du: n contiguous elements of dtype BL_BF16 or BL_F16, 16-byte aligned. */
BL_API int bl_swiglu_fwd(const void* g, const void* u, void* a, int dtype, int64_t n, int device, bl_stream_t stream);
BL_API int bl_swiglu_bwd(const void* g, const void* u, const void* da, void* dg, void* du, int dtype, int64_t n,
                  int device, bl_stream_t stream);

/* bl_nvfp4_gemm picks among three kernels by problem size: 128 x 128 tiles, one CTA per tile (small problems);
 * persistent 128 x 256 tiles, one CTA per SM; persistent 256 x 256 tiles on pairs of SMs (tcgen05 cta_group::2), the
 * fastest on problems with at least as many such tiles as SMs (a quarter as many when K >= 16384). All give bit-identical results. This call forces
 * one of them for the rest of the process (tests, experiments) or, with BL_GEMM_AUTO, hands the choice back.
 * The environment variable BL_GEMM_KERNEL (same values) sets the initial choice. No counterpart in the reference. */
enum { BL_GEMM_AUTO = 0, BL_GEMM_TILE = 1, BL_GEMM_PERSISTENT = 2, BL_GEMM_PAIR = 3 };
BL_API int bl_nvfp4_gemm_select(int kernel);

/* Diagnostic, no counterpart in the reference: the kernels replace fp32 divisions that share a divisor by a product
 * with its correctly rounded reciprocal plus two fused residual corrections. This runs that routine against the
 * plain division on n pseudo-random operand pairs (synchronously, with a temporary 8-byte device allocation) and
 * stores the number of results that differ in any bit; the test-suite requires 0. */
BL_API int bl_selftest_division(uint64_t n, uint32_t seed, uint64_t* mismatches, int device);

#ifdef __cplusplus
}
#endif
#endif /* BITLATTICE_B200_H */
