// Block-scaled NVFP4 GEMM on the 5th-generation tensor cores (tcgen05) of sm_100a.
//
//   out[m][n] = (ga * gb) * sum_k A[m][k] * B[n][k]
//
// A [M, K] and B [N, K] are K-major packed E2M1 codes with one UE4M3 scale per 16 elements of K (the scales in the
// 128x4-tiled layout), ga / gb the fp32 per-tensor scales read on the device. This is the contraction the reference
// delegates to cuBLASLt through torch._scaled_mm (bitlattice/backend.py:267-290); forward, input-gradient and
// weight-gradient GEMMs of the layer are all of this form (bitlattice/backend.py:502-510, 606-624).
//
// Three kernels compute it with identical results, chosen by problem size (bl_nvfp4_gemm): gemm_kernel (below; one
// CTA per 128 x 128 tile), gemm_persistent_kernel (one CTA per SM walking 128 x 256 tiles) and gemm_pair_kernel (a
// cluster of two CTAs per SM pair walking 256 x 256 tiles with tcgen05.mma.cta_group::2). In the two persistent
// kernels the producer and MMA warps stay fully converged and issue each k-tile's burst of instructions under one
// elect.sync predicate: issued from a single lane of a diverged warp, every tcgen05 / TMA instruction cost about 90
// cycles and bounded the kernel.
//
// Structure of gemm_kernel (one CTA per 128 x BN output tile, 192 threads):
//   warp 0      producer: TMA loads of the A and B code tiles (128-byte swizzle) and bulk copies of their scale
//               blobs into a ring of shared-memory stages, signalled through mbarriers (full / empty)
//   warp 1      MMA issuer: owns the tensor-memory allocation; per stage copies the scale blobs into tensor memory
//               (tcgen05.cp) and issues four tcgen05.mma.kind::mxf4nvf4.block_scale (K = 64 each) accumulating in
//               tensor memory; tcgen05.commit releases the stage and finally publishes the accumulator
//   warps 2..5  epilogue: tcgen05.ld of the accumulator (each warp its 32-lane quarter), scale by ga*gb, convert and
//               store
// K per stage is 256 elements = one 128-byte swizzle row. Every wait on an mbarrier is bounded: on expiry the kernel
// raises an error flag, lets all warps fall through to the common exit and frees its tensor memory.
#include <cuda.h>

#include <cstdlib>
#include <atomic>
#include <mutex>

#include "common.cuh"

namespace blb {

constexpr int kBM = 128;          // rows of A per tile
constexpr int kBK = 256;          // elements of K per stage (128 bytes of packed codes)
constexpr int kGemmThreads = 192;
constexpr uint32_t kSpinLimit = 1u << 21;   // polls of one mbarrier wait before the kernel gives up

__device__ int g_gemm_error = 0;  // 0 ok; otherwise the code of the wait that expired

// ------------------------------------------------------------------------------------------------ PTX wrappers

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// mode 1: non-blocking test with cluster-scope acquire; mode 2: potentially blocking try with cluster-scope acquire
__device__ __forceinline__ bool mbar_probe_cluster(uint32_t bar, uint32_t parity, int mode) {
  uint32_t ok;
  if (mode == 1)
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
  else
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
  return ok != 0;
}

// Bounded wait: returns false when the limit expires, or when another warp of this CTA (*abort_flag) or another CTA
// (g_gemm_error) already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code,
                                          int mode = 0, uint32_t limit = kSpinLimit) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (mode == 0 ? mbar_try_wait(bar, parity) : mbar_probe_cluster(bar, parity, mode)) return true;
    if ((i & 1023u) == 1023u && (*abort_flag != 0 || *reinterpret_cast<volatile int*>(&g_gemm_error) != 0))
      return false;
  }
  *abort_flag = code;
  atomicCAS(&g_gemm_error, 0, code);
  return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
               : "memory");
}

__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// shared-memory matrix descriptor, K-major operand tile with 128-byte swizzle: 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t operand_desc(uint32_t saddr) {
  return static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

// descriptor of one 512-byte scale blob (32 rows of 16 bytes, no swizzle: 8-row groups 128 bytes apart)
__device__ __forceinline__ uint64_t scale_desc(uint32_t saddr) {
  return static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4) | (8ull << 32) | (1ull << 46);
}

// 32 rows x 128 bits of shared memory -> 4 columns of tensor memory, replicated into the four 32-lane quarters
__device__ __forceinline__ void tmem_copy_scales(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

__device__ __forceinline__ void mma_nvf4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa,
                                         uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
      : "memory");
}

// the mbarrier is arrived on once all tcgen05 operations issued so far by this thread have completed
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_load32(uint32_t taddr, uint32_t r[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_load32_async(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// One election for a burst of instructions: q is 1 in the elected lane and 0 elsewhere; the *_if wrappers issue their
// instruction under that predicate while the warp stays converged.
__device__ __forceinline__ uint32_t elect_one() {
  uint32_t q;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(q));
  return q;
}

__device__ __forceinline__ void mbar_expect_tx_if(uint32_t q, uint32_t bar, uint32_t bytes) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %0, 0;\n\t"
      "@p mbarrier.arrive.expect_tx.shared::cta.b64 _, [%1], %2;\n\t}" ::"r"(q), "r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void tma_load_2d_if(uint32_t q, uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %0, 0;\n\t"
      "@p cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%1], [%2, {%3, %4}], [%5];\n\t}"
      ::"r"(q), "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void bulk_load_if(uint32_t q, uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %0, 0;\n\t"
      "@p cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%1], [%2], %3, [%4];\n\t}"
      ::"r"(q), "r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
      : "memory");
}

template <int CG>
__device__ __forceinline__ void mma_commit_if(uint32_t q, uint32_t bar) {
  if constexpr (CG == 1)
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %0, 0;\n\t"
        "@p tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%1];\n\t}" ::"r"(q), "r"(bar)
        : "memory");
  else
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %0, 0;\n\t"
        "@p tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%1];\n\t}" ::"r"(q), "r"(bar)
        : "memory");
}

template <int CG>
__device__ __forceinline__ void tmem_copy_scales_if(uint32_t q, uint32_t taddr, uint64_t sdesc) {
  if constexpr (CG == 1)
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %0, 0;\n\t"
        "@p tcgen05.cp.cta_group::1.32x128b.warpx4 [%1], %2;\n\t}" ::"r"(q), "r"(taddr), "l"(sdesc) : "memory");
  else
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %0, 0;\n\t"
        "@p tcgen05.cp.cta_group::2.32x128b.warpx4 [%1], %2;\n\t}" ::"r"(q), "r"(taddr), "l"(sdesc) : "memory");
}

template <int CG>
__device__ __forceinline__ void mma_nvf4_if(uint32_t q, uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
  if constexpr (CG == 1)
    asm volatile(
        "{\n\t.reg .pred p, a;\n\t"
        "setp.ne.b32 p, %0, 0;\n\t"
        "setp.ne.b32 a, %7, 0;\n\t"
        "@p tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%1], %2, %3, %4, [%5], [%6], a;\n\t}"
        ::"r"(q), "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
        : "memory");
  else
    asm volatile(
        "{\n\t.reg .pred p, a;\n\t"
        "setp.ne.b32 p, %0, 0;\n\t"
        "setp.ne.b32 a, %7, 0;\n\t"
        "@p tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%1], %2, %3, %4, [%5], [%6], a;\n\t}"
        ::"r"(q), "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
        : "memory");
}

// Scale copies and MMAs of one full k-tile (4 blocks of 64 along K) of a 256-wide tile, from one elected lane.
//   sf_desc: descriptor of the stage's first A-scale blob; the B-scale blobs follow 2048 and 4096 bytes later
//   (two 128-row blobs of B scales per k block, whatever the tile width up to 256)
//   ORDER 0: all copies, then all MMAs; 1: copies of block j right before MMA j; 2: copies one block ahead of the MMAs
template <int CG, int ORDER, int NB = 2>
__device__ __forceinline__ void issue_k_tile(uint32_t q, uint32_t acc_t, uint32_t sfa_t, uint32_t sfb_t, uint64_t sf_desc,
                                             uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate,
                                             uint32_t sfb_first = 0u) {
  auto copies = [&](int j) {
    tmem_copy_scales_if<CG>(q, sfa_t + 4 * j, sf_desc + 32u * j);
    tmem_copy_scales_if<CG>(q, sfb_t + 4 * NB * j, sf_desc + 128u + 32u * j);
    if constexpr (NB == 2) tmem_copy_scales_if<CG>(q, sfb_t + 8 * j + 4, sf_desc + 256u + 32u * j);
  };
  auto mma = [&](int j) {
    // sfb_first: column, inside the copied blobs, of the tile's first 32 rows of B (tiles that start inside a blob)
    mma_nvf4_if<CG>(q, acc_t, a_desc + 2u * j, b_desc + 2u * j, idesc, sfa_t + 4 * j, sfb_t + 4 * NB * j + sfb_first,
                    j == 0 ? accumulate : 1u);
  };
  if constexpr (ORDER == 0) {
#pragma unroll
    for (int j = 0; j < 4; ++j) copies(j);
#pragma unroll
    for (int j = 0; j < 4; ++j) mma(j);
  } else if constexpr (ORDER == 1) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      copies(j);
      mma(j);
    }
  } else {
    copies(0);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (j < 3) copies(j + 1);
      mma(j);
    }
  }
}

// One asm block for the whole burst of a full k-tile of the pair kernel, so that the operand arithmetic of all 16
// instructions can be scheduled ahead of them: 12 scale copies, 4 MMAs, and the two commits that hand the stage back
// to the producers of both CTAs. Descriptors differ only in their low
// words (sf_lo, a_lo, b_lo); sf_hi / op_hi are the constant high words.
__device__ __forceinline__ void issue_k_tile_pair_block(uint32_t q, uint32_t acc_t, uint32_t sfa_t, uint32_t sfb_t,
                                                        uint32_t sf_lo, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                                        uint32_t accumulate, uint32_t sf_hi, uint32_t op_hi,
                                                        uint32_t sfb_mma_t, uint32_t empty_local, uint32_t empty_peer) {
  asm volatile(
      "{\n\t"
      ".reg .pred q, p, one;\n\t"
      ".reg .b32 t0, t1, lo;\n\t"
      ".reg .b64 d0, d1;\n\t"
      "setp.ne.b32 q, %0, 0;\n\t"
      "setp.ne.b32 p, %8, 0;\n\t"
      "setp.eq.b32 one, 0, 0;\n\t"
      "add.u32 t0, %2, 0;\n\t"
      "add.u32 lo, %4, 0;\n\t"
      "mov.b64 d0, {lo, %9};\n\t"
      "@q tcgen05.cp.cta_group::2.32x128b.warpx4 [t0], d0;\n\t"
      "add.u32 t0, %3, 0;\n\t"
      "add.u32 lo, %4, 128;\n\t"
      "mov.b64 d0, {lo, %9};\n\t"
      "@q tcgen05.cp.cta_group::2.32x128b.warpx4 [t0], d0;\n\t"
      "add.u32 t0, %3, 4;\n\t"
      "add.u32 lo, %4, 256;\n\t"
      "mov.b64 d0, {lo, %9};\n\t"
      "@q tcgen05.cp.cta_group::2.32x128b.warpx4 [t0], d0;\n\t"
      "add.u32 t0, %2, 4;\n\t"
      "add.u32 lo, %4, 32;\n\t"
      "mov.b64 d0, {lo, %9};\n\t"
      "@q tcgen05.cp.cta_group::2.32x128b.warpx4 [t0], d0;\n\t"
      "add.u32 t0, %3, 8;\n\t"
      "add.u32 lo, %4, 160;\n\t"
      "mov.b64 d0, {lo, %9};\n\t"
      "@q tcgen05.cp.cta_group::2.32x128b.warpx4 [t0], d0;\n\t"
      "add.u32 t0, %3, 12;\n\t"
      "add.u32 lo, %4, 288;\n\t"
      "mov.b64 d0, {lo, %9};\n\t"
      "@q tcgen05.cp.cta_group::2.32x128b.warpx4 [t0], d0;\n\t"
      "add.u32 t0, %2, 8;\n\t"
      "add.u32 lo, %4, 64;\n\t"
      "mov.b64 d0, {lo, %9};\n\t"
      "@q tcgen05.cp.cta_group::2.32x128b.warpx4 [t0], d0;\n\t"
      "add.u32 t0, %3, 16;\n\t"
      "add.u32 lo, %4, 192;\n\t"
      "mov.b64 d0, {lo, %9};\n\t"
      "@q tcgen05.cp.cta_group::2.32x128b.warpx4 [t0], d0;\n\t"
      "add.u32 t0, %3, 20;\n\t"
      "add.u32 lo, %4, 320;\n\t"
      "mov.b64 d0, {lo, %9};\n\t"
      "@q tcgen05.cp.cta_group::2.32x128b.warpx4 [t0], d0;\n\t"
      "add.u32 t0, %2, 12;\n\t"
      "add.u32 lo, %4, 96;\n\t"
      "mov.b64 d0, {lo, %9};\n\t"
      "@q tcgen05.cp.cta_group::2.32x128b.warpx4 [t0], d0;\n\t"
      "add.u32 t0, %3, 24;\n\t"
      "add.u32 lo, %4, 224;\n\t"
      "mov.b64 d0, {lo, %9};\n\t"
      "@q tcgen05.cp.cta_group::2.32x128b.warpx4 [t0], d0;\n\t"
      "add.u32 t0, %3, 28;\n\t"
      "add.u32 lo, %4, 352;\n\t"
      "mov.b64 d0, {lo, %9};\n\t"
      "@q tcgen05.cp.cta_group::2.32x128b.warpx4 [t0], d0;\n\t"
      "add.u32 t0, %2, 0;\n\t"
      "add.u32 t1, %11, 0;\n\t"
      "add.u32 lo, %5, 0;\n\t"
      "mov.b64 d0, {lo, %10};\n\t"
      "add.u32 lo, %6, 0;\n\t"
      "mov.b64 d1, {lo, %10};\n\t"
      "@q tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%1], d0, d1, %7, [t0], [t1], p;\n\t"
      "add.u32 t0, %2, 4;\n\t"
      "add.u32 t1, %11, 8;\n\t"
      "add.u32 lo, %5, 2;\n\t"
      "mov.b64 d0, {lo, %10};\n\t"
      "add.u32 lo, %6, 2;\n\t"
      "mov.b64 d1, {lo, %10};\n\t"
      "@q tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%1], d0, d1, %7, [t0], [t1], one;\n\t"
      "add.u32 t0, %2, 8;\n\t"
      "add.u32 t1, %11, 16;\n\t"
      "add.u32 lo, %5, 4;\n\t"
      "mov.b64 d0, {lo, %10};\n\t"
      "add.u32 lo, %6, 4;\n\t"
      "mov.b64 d1, {lo, %10};\n\t"
      "@q tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%1], d0, d1, %7, [t0], [t1], one;\n\t"
      "add.u32 t0, %2, 12;\n\t"
      "add.u32 t1, %11, 24;\n\t"
      "add.u32 lo, %5, 6;\n\t"
      "mov.b64 d0, {lo, %10};\n\t"
      "add.u32 lo, %6, 6;\n\t"
      "mov.b64 d1, {lo, %10};\n\t"
      "@q tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%1], d0, d1, %7, [t0], [t1], one;\n\t"
      "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%12];\n\t"
      "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%13];\n\t"
      "}"
      ::"r"(q), "r"(acc_t), "r"(sfa_t), "r"(sfb_t), "r"(sf_lo), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate),
        "r"(sf_hi), "r"(op_hi), "r"(sfb_mma_t), "r"(empty_local), "r"(empty_peer)
      : "memory");
}


template <int BN, int STAGES>
struct GemmSmem {
  static constexpr uint32_t kA = kBM * (kBK / 2);          // 16 KiB
  static constexpr uint32_t kB = BN * (kBK / 2);
  static constexpr uint32_t kSFA = (kBM / 128) * 4 * 512;  // four 512-byte blobs per 128 rows and 256 K
  static constexpr uint32_t kSFB = (BN / 128) * 4 * 512;
  static constexpr uint32_t kStage = kA + kB + kSFA + kSFB;
  static constexpr uint32_t kBars = 1024;                  // barriers + tensor-memory address + abort flag
  static constexpr uint32_t kTotal = STAGES * kStage + kBars + 1024;   // + slack to align the base to 1024 bytes
};

struct GemmArgs {
  const uint8_t* a_sf;
  const uint8_t* b_sf;
  const float* a_global;
  const float* b_global;
  void* out;
  int64_t M, N, K, ldc;
  int out_dtype;
  int num_m, num_n;
  int accumulate;          // 1: out += result, the sum rounded as a dense add of two tensors of the output type
};

// 32 bytes in one store instruction (a whole sector per lane); dst must be 32-byte aligned
__device__ __forceinline__ void store32B(void* dst, const uint32_t w[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]),
               "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
               : "memory");
}

__device__ __forceinline__ void load32B(const void* src, uint32_t w[8]) {
  asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
               : "l"(src)
               : "memory");
}

// 32 consecutive outputs of one row; ncols_valid is a multiple of 8. ACC: the result is added to what dst holds, as
// torch adds two tensors of type O: the product is rounded to O first, then the fp32 sum of the two is rounded to O.
template <typename O, bool ACC>
__device__ __forceinline__ void store_row32_impl(O* dst, const uint32_t acc[32], float alpha, int ncols_valid) {
  if constexpr (sizeof(O) == 2) {
    // full width and a 32-byte aligned row: two 32-byte stores instead of four 16-byte ones. Every lane writes its
    // own row, so a warp's store instruction touches 32 different sectors either way; filling each sector with one
    // instruction halves the write transactions of the epilogue.
    if (ncols_valid == 32 && (reinterpret_cast<uintptr_t>(dst) & 31u) == 0) {
#pragma unroll
      for (int c = 0; c < 32; c += 16) {
        O o[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) o[j] = from_f<O>(__uint_as_float(acc[c + j]) * alpha);
        if constexpr (ACC) {
          O old[16];
          load32B(dst + c, reinterpret_cast<uint32_t*>(old));
#pragma unroll
          for (int j = 0; j < 16; ++j) o[j] = from_f<O>(to_f<O>(old[j]) + to_f<O>(o[j]));
        }
        store32B(dst + c, reinterpret_cast<const uint32_t*>(o));
      }
      return;
    }
  }
#pragma unroll
  for (int c = 0; c < 32; c += 8) {
    if (c >= ncols_valid) break;
    if constexpr (sizeof(O) == 4) {
      float4 v0 = make_float4(__uint_as_float(acc[c]) * alpha, __uint_as_float(acc[c + 1]) * alpha,
                              __uint_as_float(acc[c + 2]) * alpha, __uint_as_float(acc[c + 3]) * alpha);
      float4 v1 = make_float4(__uint_as_float(acc[c + 4]) * alpha, __uint_as_float(acc[c + 5]) * alpha,
                              __uint_as_float(acc[c + 6]) * alpha, __uint_as_float(acc[c + 7]) * alpha);
      if constexpr (ACC) {      // (explicitly rounded adds: this file is compiled with fused multiply-adds allowed)
        const float4 p0 = reinterpret_cast<const float4*>(dst + c)[0], p1 = reinterpret_cast<const float4*>(dst + c)[1];
        v0 = make_float4(__fadd_rn(p0.x, v0.x), __fadd_rn(p0.y, v0.y), __fadd_rn(p0.z, v0.z), __fadd_rn(p0.w, v0.w));
        v1 = make_float4(__fadd_rn(p1.x, v1.x), __fadd_rn(p1.y, v1.y), __fadd_rn(p1.z, v1.z), __fadd_rn(p1.w, v1.w));
      }
      reinterpret_cast<float4*>(dst + c)[0] = v0;
      reinterpret_cast<float4*>(dst + c)[1] = v1;
    } else {
      O o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = from_f<O>(__uint_as_float(acc[c + j]) * alpha);
      if constexpr (ACC) {
        const uint4 raw = *reinterpret_cast<const uint4*>(dst + c);
        const O* old = reinterpret_cast<const O*>(&raw);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = from_f<O>(to_f<O>(old[j]) + to_f<O>(o[j]));
      }
      *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(o);
    }
  }
}

template <typename O>
__device__ __forceinline__ void store_row32(O* dst, const uint32_t acc[32], float alpha, int ncols_valid,
                                            int accumulate = 0) {
  if (accumulate) store_row32_impl<O, true>(dst, acc, alpha, ncols_valid);
  else store_row32_impl<O, false>(dst, acc, alpha, ncols_valid);
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(kGemmThreads) gemm_kernel(const __grid_constant__ CUtensorMap map_a,
                                                            const __grid_constant__ CUtensorMap map_b, GemmArgs args) {
  using S = GemmSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;                  // operand tiles need 1024-byte alignment
  uint8_t* base_ptr = smem_raw + (base - raw_addr);
  const uint32_t bars = base + STAGES * S::kStage;
  uint8_t* bars_ptr = base_ptr + STAGES * S::kStage;
  // barrier block: full[STAGES], empty[STAGES], accumulator-ready, then the tensor-memory address and the abort flag
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  const uint32_t acc_bar = bars + 8u * (2 * STAGES);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars_ptr + 8 * (2 * STAGES + 1));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars_ptr + 8 * (2 * STAGES + 1) + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // tile of this CTA: groups of 16 row tiles share their column tiles while they are hot in L2
  constexpr int kGroup = 16;
  const int pid = blockIdx.x;
  const int per_group = kGroup * args.num_n;
  const int group = pid / per_group;
  const int first_m = group * kGroup;
  const int group_m = min(args.num_m - first_m, kGroup);
  const int tile_m = first_m + (pid % per_group) % group_m;
  const int tile_n = (pid % per_group) / group_m;
  const int64_t m0 = static_cast<int64_t>(tile_m) * kBM, n0 = static_cast<int64_t>(tile_n) * BN;

  const int num_k_tiles = static_cast<int>((args.K + kBK - 1) / kBK);
  const int nkb = static_cast<int>((args.K + 63) / 64);               // scale blobs per 128 rows along K
  const int nrb_b = static_cast<int>((args.N + 127) / 128);           // 128-row scale blocks of B

  constexpr uint32_t kTmemCols = BN <= 64 ? 128 : (BN <= 192 ? 256 : 512);
  constexpr uint32_t kSfaCol = BN;            // accumulator: columns [0, BN); then 16 columns of A scales
  constexpr uint32_t kSfbCol = BN + 16;       // then (BN/32)*4 columns of B scales

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_b)) : "memory");
      for (int kt = 0; kt < num_k_tiles; ++kt) {
        const int s = kt % STAGES;
        const uint32_t round = kt / STAGES;
        if (round > 0 && !mbar_wait(empty_bar(s), (round - 1) & 1, abort_flag, 1)) break;
        const uint32_t stage = base + s * S::kStage;
        const int blobs = min(4, nkb - kt * 4);
        const uint32_t sf_bytes = blobs * 512u;
        const int b_blocks = min(BN / 128, nrb_b - tile_n * (BN / 128));     // 128-row scale blocks of B that exist
        mbar_expect_tx(full_bar(s), S::kA + S::kB + sf_bytes * (1 + b_blocks));
        tma_load_2d(stage, &map_a, kt * (kBK / 2), static_cast<int>(m0), full_bar(s));
        tma_load_2d(stage + S::kA, &map_b, kt * (kBK / 2), static_cast<int>(n0), full_bar(s));
        const uint8_t* sfa = args.a_sf + (static_cast<int64_t>(tile_m) * nkb + kt * 4) * 512;
        bulk_load(stage + S::kA + S::kB, sfa, sf_bytes, full_bar(s));
#pragma unroll
        for (int h = 0; h < b_blocks; ++h) {
          const uint8_t* sfb = args.b_sf + ((static_cast<int64_t>(tile_n) * (BN / 128) + h) * nkb + kt * 4) * 512;
          bulk_load(stage + S::kA + S::kB + S::kSFA + h * 2048, sfb, sf_bytes, full_bar(s));
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      // instruction descriptor: E2M1 x E2M1, UE4M3 scales, K-major A and B, N = BN, M = 128, dense K = 64
      constexpr uint32_t idesc = (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BN >> 3) << 17) | (8u << 24);
      bool ok = true;
      for (int kt = 0; kt < num_k_tiles && ok; ++kt) {
        const int s = kt % STAGES;
        ok = mbar_wait(full_bar(s), (kt / STAGES) & 1, abort_flag, 2);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t stage = base + s * S::kStage;
        const int blocks = min(4, nkb - kt * 4);
        for (int j = 0; j < blocks; ++j) {
          tmem_copy_scales(tmem_base + kSfaCol + 4 * j, scale_desc(stage + S::kA + S::kB + j * 512));
#pragma unroll
          for (int h = 0; h < BN / 128; ++h)
            tmem_copy_scales(tmem_base + kSfbCol + (BN / 32) * j + 4 * h,
                             scale_desc(stage + S::kA + S::kB + S::kSFA + h * 2048 + j * 512));
        }
        const uint64_t adesc = operand_desc(stage), bdesc = operand_desc(stage + S::kA);
        for (int j = 0; j < blocks; ++j)
          mma_nvf4(tmem_base, adesc + 2u * j, bdesc + 2u * j, idesc, tmem_base + kSfaCol + 4 * j,
                   tmem_base + kSfbCol + (BN / 32) * j, (kt | j) != 0);
        mma_commit(empty_bar(s));
      }
      if (ok) mma_commit(acc_bar);
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const bool ok = mbar_wait(acc_bar, 0, abort_flag, 3);
    tcgen05_fence_after();
    if (ok) {
      const int quarter = warp & 3;                       // the 32 accumulator lanes this warp may read
      const int64_t row = m0 + quarter * 32 + lane;
      const float alpha = args.a_global[0] * args.b_global[0];
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t acc[32];
        tmem_load32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + c, acc);
        const int64_t col = n0 + c;
        if (row < args.M && col < args.N) {
          const int64_t left = args.N - col;
          const int valid = left < 32 ? static_cast<int>(left) : 32;
          if (args.out_dtype == BL_BF16)
            store_row32(static_cast<__nv_bfloat16*>(args.out) + row * args.ldc + col, acc, alpha, valid, args.accumulate);
          else if (args.out_dtype == BL_F16)
            store_row32(static_cast<__half*>(args.out) + row * args.ldc + col, acc, alpha, valid, args.accumulate);
          else
            store_row32(static_cast<float*>(args.out) + row * args.ldc + col, acc, alpha, valid, args.accumulate);
        }
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------------ persistent kernel
// One CTA per SM walks over 128 x 256 output tiles (tile = blockIdx.x + i * gridDim.x, same grouped order). The
// producer warp runs ahead across tile boundaries, so the shared-memory ring stays full while the epilogue drains the
// accumulator; the MMA warp only waits for the drain (tmem_empty) before the first MMA of the next tile.
//   warp 0: producer   warp 1: MMA issuer + tensor-memory owner   warps 2..9: epilogue (two warps per 32-lane
//   quarter, each taking one 128-column half of the accumulator)
constexpr int kPersistThreads = 320;

// The "accumulator drained" arrivals carry no data through memory (tensor-memory reads are ordered by
// tcgen05.wait::ld and the tcgen05 fences on both sides), so they are relaxed: a release would first wait for the
// epilogue's outstanding global stores of the previous tile, about a microsecond per tile.
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.relaxed.cta.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

template <int STAGES, int ORDER>
__global__ void __launch_bounds__(kPersistThreads, 1) gemm_persistent_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                             const __grid_constant__ CUtensorMap map_b,
                                                                             GemmArgs args) {
  constexpr int BN = 256;
  using S = GemmSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw_addr);
  const uint32_t bars = base + STAGES * S::kStage;
  uint8_t* bars_ptr = base_ptr + STAGES * S::kStage;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  const uint32_t acc_full = bars + 8u * (2 * STAGES);        // accumulator of the current tile is complete
  const uint32_t acc_empty = bars + 8u * (2 * STAGES + 1);   // accumulator has been read out (8 warp arrivals)
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars_ptr + 8 * (2 * STAGES + 2));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars_ptr + 8 * (2 * STAGES + 2) + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = args.num_m * args.num_n;
  const int num_k_tiles = static_cast<int>((args.K + kBK - 1) / kBK);
  const int nkb = static_cast<int>((args.K + 63) / 64);
  const int nrb_b = static_cast<int>((args.N + 127) / 128);
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kSfaCol = BN, kSfbCol = BN + 16;

  constexpr int kGroup = 16;
  auto tile_coords = [&](int pid, int& tile_m, int& tile_n) {
    const int per_group = kGroup * args.num_n;
    const int group = pid / per_group;
    const int first_m = group * kGroup;
    const int group_m = min(args.num_m - first_m, kGroup);
    tile_m = first_m + (pid % per_group) % group_m;
    tile_n = (pid % per_group) / group_m;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 8);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer: whole warp converged, one lane issues
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_b)) : "memory");
    }
    __syncwarp();
    int s = 0;
    uint32_t phase = 1;                                    // parity that means "stage is free" (free at the start)
    bool ok = true;
    for (int pid = blockIdx.x; pid < num_tiles && ok; pid += gridDim.x) {
      int tile_m, tile_n;
      tile_coords(pid, tile_m, tile_n);
      const int b_blocks = min(BN / 128, nrb_b - tile_n * (BN / 128));
      const uint8_t* sfa = args.a_sf + static_cast<int64_t>(tile_m) * nkb * 512;
      const uint8_t* sfb = args.b_sf + static_cast<int64_t>(tile_n) * (BN / 128) * nkb * 512;
      for (int kt = 0; kt < num_k_tiles; ++kt) {
        ok = __all_sync(0xffffffffu, mbar_wait(empty_bar(s), phase, abort_flag, 1));
        if (!ok) break;
        const uint32_t q = elect_one();
        const uint32_t stage = base + s * S::kStage;
        const int blobs = min(4, nkb - kt * 4);
        const uint32_t sf_bytes = blobs * 512u;
        mbar_expect_tx_if(q, full_bar(s), S::kA + S::kB + sf_bytes * (1 + b_blocks));
        tma_load_2d_if(q, stage, &map_a, kt * (kBK / 2), tile_m * kBM, full_bar(s));
        tma_load_2d_if(q, stage + S::kA, &map_b, kt * (kBK / 2), tile_n * BN, full_bar(s));
        bulk_load_if(q, stage + S::kA + S::kB, sfa + kt * 2048, sf_bytes, full_bar(s));
        bulk_load_if(q, stage + S::kA + S::kB + S::kSFA, sfb + kt * 2048, sf_bytes, full_bar(s));
        if (b_blocks == 2)
          bulk_load_if(q, stage + S::kA + S::kB + S::kSFA + 2048, sfb + (static_cast<int64_t>(nkb) + kt * 4) * 512, sf_bytes,
                       full_bar(s));
        if (++s == STAGES) {
          s = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issue: whole warp converged, one lane issues
    constexpr uint32_t idesc = (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BN >> 3) << 17) | (8u << 24);
    int s = 0;
    uint32_t phase = 0, acc_phase = 1;                     // the accumulator starts out free
    bool ok = true;
    for (int pid = blockIdx.x; pid < num_tiles && ok; pid += gridDim.x) {
      ok = __all_sync(0xffffffffu, mbar_wait(acc_empty, acc_phase, abort_flag, 4));
      if (!ok) break;
      acc_phase ^= 1;
      tcgen05_fence_after();
      for (int kt = 0; kt < num_k_tiles; ++kt) {
        ok = __all_sync(0xffffffffu, mbar_wait(full_bar(s), phase, abort_flag, 2));
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t q = elect_one();
        const uint32_t stage = base + s * S::kStage;
        const int blocks = min(4, nkb - kt * 4);
        const uint64_t adesc = operand_desc(stage), bdesc = operand_desc(stage + S::kA);
        const uint64_t sdesc = scale_desc(stage + S::kA + S::kB);
        if (blocks == 4) {
          issue_k_tile<1, ORDER>(q, tmem_base, tmem_base + kSfaCol, tmem_base + kSfbCol, sdesc, adesc, bdesc, idesc,
                                 kt != 0);
        } else {
          for (int j = 0; j < blocks; ++j) {
            tmem_copy_scales_if<1>(q, tmem_base + kSfaCol + 4 * j, sdesc + 32u * j);
            tmem_copy_scales_if<1>(q, tmem_base + kSfbCol + 8 * j, sdesc + 128u + 32u * j);
            tmem_copy_scales_if<1>(q, tmem_base + kSfbCol + 8 * j + 4, sdesc + 256u + 32u * j);
          }
          for (int j = 0; j < blocks; ++j)
            mma_nvf4_if<1>(q, tmem_base, adesc + 2u * j, bdesc + 2u * j, idesc, tmem_base + kSfaCol + 4 * j,
                           tmem_base + kSfbCol + 8 * j, (kt | j) != 0);
        }
        mma_commit_if<1>(q, empty_bar(s));
        if (kt == num_k_tiles - 1) mma_commit_if<1>(q, acc_full);
        if (++s == STAGES) {
          s = 0;
          phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue: 8 warps, a 32-lane x 128-column block each
    const int quarter = warp & 3;                        // accumulator lanes this warp may read
    const int half = (warp - 2) >> 2;                    // 128-column half it drains
    const float alpha = args.a_global[0] * args.b_global[0];
    uint32_t acc_phase = 0;
    for (int pid = blockIdx.x; pid < num_tiles; pid += gridDim.x) {
      int tile_m, tile_n;
      tile_coords(pid, tile_m, tile_n);
      if (!mbar_wait(acc_full, acc_phase, abort_flag, 3)) break;
      acc_phase ^= 1;
      tcgen05_fence_after();
      // pull the whole block into registers first, so that the next tile's MMAs can start while this one is stored
      uint32_t acc[4][32];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        tmem_load32_async(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + half * 128 + i * 32, acc[i]);
      tmem_load_wait();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty);
      const int64_t row = static_cast<int64_t>(tile_m) * kBM + quarter * 32 + lane;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int64_t col = static_cast<int64_t>(tile_n) * BN + half * 128 + i * 32;
        if (row < args.M && col < args.N) {
          const int64_t left = args.N - col;
          const int valid = left < 32 ? static_cast<int>(left) : 32;
          if (args.out_dtype == BL_BF16)
            store_row32(static_cast<__nv_bfloat16*>(args.out) + row * args.ldc + col, acc[i], alpha, valid, args.accumulate);
          else if (args.out_dtype == BL_F16)
            store_row32(static_cast<__half*>(args.out) + row * args.ldc + col, acc[i], alpha, valid, args.accumulate);
          else
            store_row32(static_cast<float*>(args.out) + row * args.ldc + col, acc[i], alpha, valid, args.accumulate);
        }
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------------ CTA-pair kernel
// Two CTAs on neighbouring SMs (a cluster of 2) share one 256 x 256 output tile: CTA r holds rows [128 r, 128 r + 128)
// of the A tile and of the accumulator, and half of the B tile (rows [128 r, 128 r + 128) of B); one
// tcgen05.mma.cta_group::2 issued by CTA 0 multiplies the 256-row A by the 256-row B using both SMs' tensor cores and
// both shared memories. Per flop this halves the operand bytes each SM pulls from L2.
//
// Synchronisation (all mbarriers; every wait bounded):
//   full[s]    in CTA 0 only: the TMA loads of BOTH CTAs for stage s complete their bytes here (the loads carry
//              .cta_group::2, which lets a load signal the barrier of the other CTA of the pair)
//   empty[s]   each CTA: tcgen05.commit from CTA 0 after the MMAs that read stage s (one commit per CTA)
//   acc_full   each CTA: tcgen05.commit from CTA 0 after the last MMA of a tile
//   acc_empty  in CTA 0: 16 arrivals, one per epilogue warp of both CTAs, when the accumulator is in registers
// Every CTA loads its own operand halves; the only cross-CTA traffic is barrier signalling.
constexpr int kPairThreads = 320;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {   // shared::cluster address
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {   // relaxed: see mbar_arrive
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// TMA loads whose completion may be signalled on the other CTA of the pair (bar is a shared::cluster address)
__device__ __forceinline__ void tma_pair_load_2d_if(uint32_t q, uint32_t dst, const CUtensorMap* map, int x, int y,
                                                    uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %0, 0;\n\t"
      "@p cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%1], [%2, {%3, %4}], [%5];\n\t}"
      ::"r"(q), "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void tma_pair_load_3d_if(uint32_t q, uint32_t dst, const CUtensorMap* map, int x, int y, int z,
                                                    uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %0, 0;\n\t"
      "@p cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%1], [%2, {%3, %4, %5}], [%6];\n\t}"
      ::"r"(q), "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}

// BN = 256 (the one in use): one accumulator of 256 columns; a second one plus the scale columns would not fit the 512
// columns of tensor memory, so a tile's MMAs wait for the epilogue of the tile before it. The kernel is written for
// narrower tiles with two accumulators as well (BN = 192: a 192-row tile of B starts at row 0 or 64 of a 128-row
// scale blob, so the MMA is pointed two columns into the copied blobs for odd tiles; BN = 128: one blob). Both gave
// the same bits but were slower on B200 and are not instantiated: an MMA of N = 192 takes as long as one of N = 256
// (3.9 PFLOP/s against 4.6-5.1), and 256 x 128 tiles are bound by L2 -> shared-memory traffic (3.1 PFLOP/s).
template <int BN, int STAGES>
struct PairSmem {
  static constexpr uint32_t kA = 128 * (kBK / 2);       // this CTA's 128 rows of A
  static constexpr uint32_t kB = (BN / 2) * (kBK / 2);  // this CTA's half of the B tile
  static constexpr uint32_t kSFA = 4 * 512;             // scales of its A rows
  static constexpr int kBlobsB = BN > 128 ? 2 : 1;      // 128-row scale blobs the B tile touches
  static constexpr uint32_t kSFB = kBlobsB * 4 * 512;
  static constexpr uint32_t kStage = kA + kB + kSFA + kSFB;
  static constexpr uint32_t kTotal = STAGES * kStage + 1024 + 1024;
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(kPairThreads, 1) gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                    const __grid_constant__ CUtensorMap map_b,
                                                                    const __grid_constant__ CUtensorMap map_sfa,
                                                                    const __grid_constant__ CUtensorMap map_sfb,
                                                                    GemmArgs args) {
  using S = PairSmem<BN, STAGES>;
  constexpr int NACC = BN == 256 ? 1 : 2;                  // accumulator buffers
  constexpr int kHalf = BN / 2;                            // columns one epilogue warp drains
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw_addr);
  const uint32_t bars = base + STAGES * S::kStage;
  uint8_t* bars_ptr = base_ptr + STAGES * S::kStage;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto acc_full = [&](int a) { return bars + 8u * (2 * STAGES + a); };
  auto acc_empty = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars_ptr + 8 * (2 * STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars_ptr + 8 * (2 * STAGES + 4) + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();                 // 0: leader (issues the MMAs), 1: peer
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int num_tiles = args.num_m * args.num_n;           // 256 x BN tiles
  const int num_k_tiles = static_cast<int>((args.K + kBK - 1) / kBK);
  const int nkb = static_cast<int>((args.K + 63) / 64);
  constexpr uint32_t kTmemCols = 512, kSfaCol = NACC * BN, kSfbCol = kSfaCol + 16;
  static_assert(kSfbCol + 32 <= kTmemCols, "tensor memory budget");
  constexpr int kCluster = 2;                              // barriers signalled across the pair: cluster-scope acquire

  constexpr int kGroup = 8;
  auto tile_coords = [&](int pid, int& tile_m, int& tile_n) {
    const int per_group = kGroup * args.num_n;
    const int group = pid / per_group;
    const int first_m = group * kGroup;
    const int group_m = min(args.num_m - first_m, kGroup);
    tile_m = first_m + (pid % per_group) % group_m;
    tile_n = (pid % per_group) / group_m;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full(a), 1);
      mbar_init(acc_empty(a), 16);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();                                      // both CTAs' barriers exist before any remote signal
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (both CTAs, each for its own halves)
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_b)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_sfa)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_sfb)) : "memory");
    }
    __syncwarp();
    const uint32_t full_leader0 = map_to_cta(full_bar(0), 0);
    int s = 0;
    uint32_t phase = 1;
    bool ok = true;
    for (int pid = pair; pid < num_tiles && ok; pid += num_pairs) {
      int tile_m, tile_n;
      tile_coords(pid, tile_m, tile_n);
      const int rb_a = tile_m * 2 + static_cast<int>(rank);               // 128-row block of A this CTA owns
      const int row_b = tile_n * BN + static_cast<int>(rank) * (BN / 2);  // its half of the B tile
      const int blob_b = (tile_n * BN) >> 7;                              // first scale blob the B tile touches
      for (int kt = 0; kt < num_k_tiles; ++kt) {
        ok = __all_sync(0xffffffffu, mbar_wait(empty_bar(s), phase, abort_flag, 1, kCluster));
        if (!ok) break;
        const uint32_t q = elect_one();
        const uint32_t stage = base + s * S::kStage;
        const uint32_t bar = full_leader0 + 8u * s;
        // every load is a full box (bytes outside the tensors arrive as zeros), so the byte count is fixed
        if (rank == 0) mbar_expect_tx_if(q, full_bar(s), 2 * S::kStage);
        tma_pair_load_2d_if(q, stage, &map_a, kt * (kBK / 2), rb_a * 128, bar);
        tma_pair_load_2d_if(q, stage + S::kA, &map_b, kt * (kBK / 2), row_b, bar);
        tma_pair_load_3d_if(q, stage + S::kA + S::kB, &map_sfa, 0, kt * 4, rb_a, bar);
        tma_pair_load_3d_if(q, stage + S::kA + S::kB + S::kSFA, &map_sfb, 0, kt * 4, blob_b, bar);
        if (++s == STAGES) {
          s = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    if (rank == 0) {
      // ---------------------------------------------------------------- leader: scale copies + MMAs for the pair
      // E2M1 x E2M1, UE4M3 scales, K-major, N = BN, M = 256 (two CTAs), dense K = 64
      constexpr uint32_t idesc = (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BN >> 3) << 17) | (16u << 24);
      const uint32_t empty_peer0 = map_to_cta(empty_bar(0), 1);           // the peer's barriers, 8 bytes apart
      const uint32_t acc_full_peer0 = map_to_cta(acc_full(0), 1);
      int s = 0, ab = 0;
      uint32_t phase = 0, acc_phases = 3u;                                // bit a: parity to wait for on accumulator a
                                                                          // (both start out free)
      bool ok = true;
      for (int pid = pair; pid < num_tiles && ok; pid += num_pairs) {
        int tile_m, tile_n;
        tile_coords(pid, tile_m, tile_n);
        const uint32_t sfb_first = static_cast<uint32_t>(((tile_n * BN) & 127) >> 5);
        const uint32_t acc_t = tmem_base + static_cast<uint32_t>(ab * BN);
        ok = __all_sync(0xffffffffu, mbar_wait(acc_empty(ab), (acc_phases >> ab) & 1u, abort_flag, 4, kCluster));
        if (!ok) break;
        acc_phases ^= 1u << ab;
        tcgen05_fence_after();
        for (int kt = 0; kt < num_k_tiles; ++kt) {
          ok = __all_sync(0xffffffffu, mbar_wait(full_bar(s), phase, abort_flag, 2, kCluster));
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t q = elect_one();
          const uint32_t stage = base + s * S::kStage;
          const int blocks = min(4, nkb - kt * 4);
          const uint64_t adesc = operand_desc(stage), bdesc = operand_desc(stage + S::kA);
          const uint64_t sdesc = scale_desc(stage + S::kA + S::kB);
          if (blocks == 4 && S::kBlobsB == 2) {
            issue_k_tile_pair_block(q, acc_t, tmem_base + kSfaCol, tmem_base + kSfbCol, static_cast<uint32_t>(sdesc),
                                    static_cast<uint32_t>(adesc), static_cast<uint32_t>(bdesc), idesc, kt != 0,
                                    static_cast<uint32_t>(sdesc >> 32), static_cast<uint32_t>(adesc >> 32),
                                    tmem_base + kSfbCol + sfb_first, empty_bar(s), empty_peer0 + 8u * s);
          } else {
            if (blocks == 4) {
              issue_k_tile<2, 0, S::kBlobsB>(q, acc_t, tmem_base + kSfaCol, tmem_base + kSfbCol, sdesc, adesc, bdesc, idesc,
                                             kt != 0, sfb_first);
            } else {
              for (int j = 0; j < blocks; ++j) {
                tmem_copy_scales_if<2>(q, tmem_base + kSfaCol + 4 * j, sdesc + 32u * j);
                tmem_copy_scales_if<2>(q, tmem_base + kSfbCol + 4 * S::kBlobsB * j, sdesc + 128u + 32u * j);
                if (S::kBlobsB == 2) tmem_copy_scales_if<2>(q, tmem_base + kSfbCol + 8 * j + 4, sdesc + 256u + 32u * j);
              }
              for (int j = 0; j < blocks; ++j)
                mma_nvf4_if<2>(q, acc_t, adesc + 2u * j, bdesc + 2u * j, idesc, tmem_base + kSfaCol + 4 * j,
                               tmem_base + kSfbCol + 4 * S::kBlobsB * j + sfb_first, (kt | j) != 0);
            }
            mma_commit_if<2>(q, empty_bar(s));
            mma_commit_if<2>(q, empty_peer0 + 8u * s);
          }
          if (kt == num_k_tiles - 1) {
            mma_commit_if<2>(q, acc_full(ab));
            mma_commit_if<2>(q, acc_full_peer0 + 8u * ab);
          }
          if (++s == STAGES) {
            s = 0;
            phase ^= 1;
          }
        }
        if (NACC == 2) ab ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    const float alpha = args.a_global[0] * args.b_global[0];
    const uint32_t acc_empty_leader0 = map_to_cta(acc_empty(0), 0);
    int ab = 0;
    uint32_t acc_phases = 0u;
    for (int pid = pair; pid < num_tiles; pid += num_pairs) {
      int tile_m, tile_n;
      tile_coords(pid, tile_m, tile_n);
      if (!mbar_wait(acc_full(ab), (acc_phases >> ab) & 1u, abort_flag, 3, kCluster)) break;
      acc_phases ^= 1u << ab;
      tcgen05_fence_after();
      uint32_t acc[kHalf / 32][32];
#pragma unroll
      for (int i = 0; i < kHalf / 32; ++i)
        tmem_load32_async(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + ab * BN + half * kHalf + i * 32,
                          acc[i]);
      tmem_load_wait();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty_leader0 + 8u * ab);
      const int64_t row = static_cast<int64_t>(tile_m) * 256 + rank * 128 + quarter * 32 + lane;
#pragma unroll
      for (int i = 0; i < kHalf / 32; ++i) {
        const int64_t col = static_cast<int64_t>(tile_n) * BN + half * kHalf + i * 32;
        if (row < args.M && col < args.N) {
          const int64_t left = args.N - col;
          const int valid = left < 32 ? static_cast<int>(left) : 32;
          if (args.out_dtype == BL_BF16)
            store_row32(static_cast<__nv_bfloat16*>(args.out) + row * args.ldc + col, acc[i], alpha, valid, args.accumulate);
          else if (args.out_dtype == BL_F16)
            store_row32(static_cast<__half*>(args.out) + row * args.ldc + col, acc[i], alpha, valid, args.accumulate);
          else
            store_row32(static_cast<float*>(args.out) + row * args.ldc + col, acc[i], alpha, valid, args.accumulate);
        }
      }
      if (NACC == 2) ab ^= 1;
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();                                      // no CTA frees tensor memory the pair's MMAs may still use
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

// The give-up path of mbar_wait on its own: one warp, one mbarrier that nothing ever arrives on, a short limit. No
// TMA copy or tensor-memory operation is in flight, so the kernel simply records the code and returns.
constexpr int kSelftestWaitCode = 9;

__global__ void selftest_bounded_wait_kernel(int* returned) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  bool ok = true;
  if (threadIdx.x == 0) ok = mbar_wait(smem_u32(&bar), 0, &abort_flag, kSelftestWaitCode, 0, 4096u);
  __syncwarp();
  if (threadIdx.x == 0) *returned = ok ? 1 : 2;            // 2: the wait gave up and the kernel still reached its end
}

// Tensor-pipe ceiling: every SM issues block-scaled FP4 MMAs (M 128, N 256, K 64, the persistent kernel's shape) on
// one resident pair of operand tiles filled with pseudo-random codes, with nothing else in the loop -- no loads, no
// scale copies, no epilogue. The result is meaningless; the time is what the MMA pipe alone needs, under the power cap,
// and serves as the measured peak the GEMM kernels are compared with.
// SCALES: 0 = scale columns written once (the ceiling); 1 = the twelve tcgen05.cp of a k-tile issued in order before
// its MMAs, as the GEMM kernels do (on one SM they cost nothing: 8.10 against 8.13 PFLOP/s).
template <int BN, int SCALES>
__global__ void __launch_bounds__(128, 1) mma_peak_kernel(int iters, int* status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_storage;
  __shared__ uint32_t tmem_slot_storage;
  __shared__ int abort_storage;
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw_addr);
  constexpr uint32_t kA = 128 * 128, kB = 256 * 128, kSF = 3 * 2048;      // A tile, B tile, scale blobs (A, B lo, B hi)
  const uint32_t bar = smem_u32(&bar_storage);
  volatile int* abort_flag = &abort_storage;
  const int warp = threadIdx.x >> 5;
  for (uint32_t i = threadIdx.x; i < (kA + kB) / 4; i += blockDim.x) {
    uint32_t h = (i + blockIdx.x * 7919u) * 0x9E3779B1u;
    h = (h ^ (h >> 15)) * 0x85EBCA77u;
    reinterpret_cast<uint32_t*>(base_ptr)[i] = h ^ (h >> 13);
  }
  for (uint32_t i = threadIdx.x; i < kSF / 4; i += blockDim.x)
    reinterpret_cast<uint32_t*>(base_ptr + kA + kB)[i] = 0x38383838u;      // UE4M3 1.0
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 0) tmem_alloc(smem_u32(&tmem_slot_storage), 512);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = tmem_slot_storage;
  if (warp == 0) {
    constexpr uint32_t idesc = (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BN >> 3) << 17) | (8u << 24);
    constexpr uint32_t kSfaCol = 256, kSfbCol = 272;
    const uint64_t adesc = operand_desc(base), bdesc = operand_desc(base + kA);
    const uint64_t sdesc = scale_desc(base + kA + kB);
    uint32_t q = elect_one();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      tmem_copy_scales_if<1>(q, tmem_base + kSfaCol + 4 * j, sdesc + 32u * j);
      tmem_copy_scales_if<1>(q, tmem_base + kSfbCol + 8 * j, sdesc + 128u + 32u * j);
      tmem_copy_scales_if<1>(q, tmem_base + kSfbCol + 8 * j + 4, sdesc + 256u + 32u * j);
    }
    uint32_t parity = 0;
    bool ok = true;
    for (int it = 0; it < iters && ok; ++it) {
      q = elect_one();
      if constexpr (SCALES == 1) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          tmem_copy_scales_if<1>(q, tmem_base + kSfaCol + 4 * j, sdesc + 32u * j);
          tmem_copy_scales_if<1>(q, tmem_base + kSfbCol + 8 * j, sdesc + 128u + 32u * j);
          tmem_copy_scales_if<1>(q, tmem_base + kSfbCol + 8 * j + 4, sdesc + 256u + 32u * j);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if constexpr (BN == 256) {
          mma_nvf4_if<1>(q, tmem_base, adesc + 2u * j, bdesc + 2u * j, idesc, tmem_base + kSfaCol + 4 * j,
                         tmem_base + kSfbCol + 8 * j, (it | j) != 0);
        } else {                                    // the same work as two MMAs of 128 columns (B rows 128 apart)
          mma_nvf4_if<1>(q, tmem_base, adesc + 2u * j, bdesc + 2u * j, idesc, tmem_base + kSfaCol + 4 * j,
                         tmem_base + kSfbCol + 8 * j, (it | j) != 0);
          mma_nvf4_if<1>(q, tmem_base + 128, adesc + 2u * j, bdesc + 1024u + 2u * j, idesc,
                         tmem_base + kSfaCol + 4 * j, tmem_base + kSfbCol + 8 * j + 4, (it | j) != 0);
        }
      }
      if ((it & 63) == 63 || it == iters - 1) {               // bound the work in flight; every wait has a limit
        mma_commit_if<1>(q, bar);
        ok = __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, 8));
        parity ^= 1u;
        tcgen05_fence_after();
      }
    }
    if (!ok && (threadIdx.x & 31) == 0) *status = 8;
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 0) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------------ host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// Encoded tensor maps are a function of (address, shape, box) alone, so they are kept: a training step multiplies
// the same operands (weights of a version, cached activations) and the same shapes at the same addresses again and
// again, and the driver call costs more than the look-up. Direct-mapped, a few hundred KiB, one lock.
struct MapKey {
  const void* ptr;
  int64_t rows, K;
  int box, kind;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && K == o.K && box == o.box && kind == o.kind;
  }
};

struct MapSlot {
  MapKey key;
  CUtensorMap map;
  bool used;
};

constexpr size_t kMapSlots = 2048;
static MapSlot g_map_cache[kMapSlots];
static std::mutex g_map_mutex;

static size_t map_slot(const MapKey& k) {
  uint64_t h = reinterpret_cast<uintptr_t>(k.ptr) * 0x9E3779B97F4A7C15ull;
  h ^= static_cast<uint64_t>(k.rows) * 0xC2B2AE3D27D4EB4Full + static_cast<uint64_t>(k.K) * 0x165667B19E3779F9ull +
       static_cast<uint64_t>(k.box * 4 + k.kind);
  h ^= h >> 29;
  return static_cast<size_t>(h % kMapSlots);
}

static bool cached_map(const MapKey& k, CUtensorMap* out) {
  std::lock_guard<std::mutex> lock(g_map_mutex);
  const MapSlot& s = g_map_cache[map_slot(k)];
  if (!s.used || !(s.key == k)) return false;
  *out = s.map;
  return true;
}

static void keep_map(const MapKey& k, const CUtensorMap& m) {
  std::lock_guard<std::mutex> lock(g_map_mutex);
  MapSlot& s = g_map_cache[map_slot(k)];
  s.key = k;
  s.map = m;
  s.used = true;
}

// [rows, K/2] bytes, box of 128 bytes x box_rows rows, 128-byte swizzle, zero fill outside the tensor
static int make_operand_map(CUtensorMap* map, const uint8_t* codes, int64_t rows, int64_t K, int box_rows) {
  const MapKey key{codes, rows, K, box_rows, 0};
  if (cached_map(key, map)) return 0;
  EncodeTiledFn enc = encode_tiled_fn();
  BL_REQUIRE(enc != nullptr, "gemm: the CUDA driver does not provide cuTensorMapEncodeTiled");
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K / 2), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(K / 2)};
  const cuuint32_t box[2] = {128u, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem[2] = {1u, 1u};
  const CUresult rc = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(codes), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  BL_REQUIRE(rc == CUDA_SUCCESS, "gemm: cuTensorMapEncodeTiled failed with code %d (rows %lld, K %lld)", (int)rc,
             (long long)rows, (long long)K);
  keep_map(key, *map);
  return 0;
}

// Blocked scales seen as [row blocks][k blocks][512 bytes]; one box is 4 k blocks of box_row_blocks row blocks, landing
// in shared memory as consecutive 512-byte blobs. Blocks outside the tensor arrive as zeros.
static int make_scale_map(CUtensorMap* map, const uint8_t* sf, int64_t rows, int64_t K, int box_row_blocks) {
  const MapKey key{sf, rows, K, box_row_blocks, 1};
  if (cached_map(key, map)) return 0;
  EncodeTiledFn enc = encode_tiled_fn();
  BL_REQUIRE(enc != nullptr, "gemm: the CUDA driver does not provide cuTensorMapEncodeTiled");
  const cuuint64_t nkb = static_cast<cuuint64_t>((K + 63) / 64), nrb = static_cast<cuuint64_t>((rows + 127) / 128);
  const cuuint64_t dims[3] = {128u, nkb, nrb};                        // 32-bit words
  const cuuint64_t strides[2] = {512u, nkb * 512u};
  const cuuint32_t box[3] = {128u, 4u, static_cast<cuuint32_t>(box_row_blocks)};
  const cuuint32_t elem[3] = {1u, 1u, 1u};
  const CUresult rc = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<uint8_t*>(sf), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  BL_REQUIRE(rc == CUDA_SUCCESS, "gemm: cuTensorMapEncodeTiled failed with code %d for scales (rows %lld, K %lld)", (int)rc,
             (long long)rows, (long long)K);
  keep_map(key, *map);
  return 0;
}

template <int BN, int STAGES>
static int launch_gemm(const uint8_t* a_codes, const uint8_t* b_codes, GemmArgs args, cudaStream_t st) {
  using S = GemmSmem<BN, STAGES>;
  CUtensorMap map_a, map_b;
  if (int rc = make_operand_map(&map_a, a_codes, args.M, args.K, kBM)) return rc;
  if (int rc = make_operand_map(&map_b, b_codes, args.N, args.K, BN)) return rc;
  args.num_m = static_cast<int>((args.M + kBM - 1) / kBM);
  args.num_n = static_cast<int>((args.N + BN - 1) / BN);
  BL_CUDA(cudaFuncSetAttribute(gemm_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
  const int64_t tiles = static_cast<int64_t>(args.num_m) * args.num_n;
  BL_REQUIRE(tiles <= 0x7FFFFFFF, "gemm: too many output tiles (%lld)", (long long)tiles);
  gemm_kernel<BN, STAGES><<<static_cast<unsigned>(tiles), kGemmThreads, S::kTotal, st>>>(map_a, map_b, args);
  BL_CUDA(cudaGetLastError());
  return 0;
}

template <int STAGES, int ORDER>
static int launch_persistent(const uint8_t* a_codes, const uint8_t* b_codes, GemmArgs args, int device, cudaStream_t st) {
  using S = GemmSmem<256, STAGES>;
  CUtensorMap map_a, map_b;
  if (int rc = make_operand_map(&map_a, a_codes, args.M, args.K, kBM)) return rc;
  if (int rc = make_operand_map(&map_b, b_codes, args.N, args.K, 256)) return rc;
  args.num_m = static_cast<int>((args.M + kBM - 1) / kBM);
  args.num_n = static_cast<int>((args.N + 255) / 256);
  const int64_t tiles = static_cast<int64_t>(args.num_m) * args.num_n;
  BL_REQUIRE(tiles <= 0x7FFFFFFF, "gemm: too many output tiles (%lld)", (long long)tiles);
  BL_CUDA(cudaFuncSetAttribute(gemm_persistent_kernel<STAGES, ORDER>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
  const int sms = sm_count(device);
  const unsigned grid = static_cast<unsigned>(tiles < sms ? tiles : sms);
  gemm_persistent_kernel<STAGES, ORDER><<<grid, kPersistThreads, S::kTotal, st>>>(map_a, map_b, args);
  BL_CUDA(cudaGetLastError());
  return 0;
}

template <int BN, int STAGES>
static int launch_pair(const uint8_t* a_codes, const uint8_t* b_codes, GemmArgs args, int device, cudaStream_t st) {
  using S = PairSmem<BN, STAGES>;
  CUtensorMap map_a, map_b;
  if (int rc = make_operand_map(&map_a, a_codes, args.M, args.K, 128)) return rc;
  if (int rc = make_operand_map(&map_b, b_codes, args.N, args.K, BN / 2)) return rc;
  CUtensorMap map_sfa, map_sfb;
  if (int rc = make_scale_map(&map_sfa, args.a_sf, args.M, args.K, 1)) return rc;
  if (int rc = make_scale_map(&map_sfb, args.b_sf, args.N, args.K, S::kBlobsB)) return rc;
  args.num_m = static_cast<int>((args.M + 255) / 256);
  args.num_n = static_cast<int>((args.N + BN - 1) / BN);
  const int64_t tiles = static_cast<int64_t>(args.num_m) * args.num_n;
  BL_REQUIRE(tiles <= 0x3FFFFFFF, "gemm: too many output tiles (%lld)", (long long)tiles);
  BL_CUDA(cudaFuncSetAttribute(gemm_pair_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(sm_count(device) & ~1);
  cfg.blockDim = dim3(kPairThreads);
  cfg.dynamicSmemBytes = S::kTotal;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // The tile list is strided over the pairs, so every pair must be resident at once: ask how many clusters of two
  // the device can hold (fewer than SMs / 2 where a GPC has an odd number of usable SMs).
  static std::mutex mu;
  static int resident[64] = {};
  int max_pairs;
  {
    std::lock_guard<std::mutex> lock(mu);
    BL_REQUIRE(device >= 0 && device < 64, "gemm: device index %d out of range", device);
    if (resident[device] == 0) {
      int n = 0;
      BL_CUDA(cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel<BN, STAGES>, &cfg));
      BL_REQUIRE(n > 0, "gemm: the device cannot hold a cluster of two CTAs of the pair kernel");
      resident[device] = n;
    }
    max_pairs = resident[device];
  }
  const unsigned pairs = static_cast<unsigned>(tiles < max_pairs ? tiles : max_pairs);
  cfg.gridDim = dim3(pairs * 2);
  BL_CUDA(cudaLaunchKernelEx(&cfg, gemm_pair_kernel<BN, STAGES>, map_a, map_b, map_sfa, map_sfb, args));
  return 0;
}

}  // namespace blb

using namespace blb;

static std::atomic<int> g_kernel_choice{[] {
  const char* e = getenv("BL_GEMM_KERNEL");     // same values as bl_nvfp4_gemm_select
  const int v = e ? atoi(e) : 0;
  return v >= BL_GEMM_AUTO && v <= BL_GEMM_PAIR ? v : 0;
}()};

static int gemm_entry(const uint8_t* a_codes, const uint8_t* a_sf, const float* a_global, const uint8_t* b_codes,
                      const uint8_t* b_sf, const float* b_global, int64_t M, int64_t N, int64_t K, void* out,
                      int out_dtype, int64_t ldc, int accumulate, int device, bl_stream_t stream) {
  BL_REQUIRE(a_codes && a_sf && a_global && b_codes && b_sf && b_global && out, "gemm: null buffer");
  BL_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: empty problem %lld x %lld x %lld", (long long)M, (long long)N, (long long)K);
  BL_REQUIRE(K % 32 == 0, "gemm: K = %lld is not a multiple of 32", (long long)K);
  BL_REQUIRE(N % 8 == 0, "gemm: N = %lld is not a multiple of 8", (long long)N);
  BL_REQUIRE(ldc >= N && ldc % 8 == 0, "gemm: output row stride %lld must be a multiple of 8 and at least N", (long long)ldc);
  BL_REQUIRE(out_dtype >= BL_F32 && out_dtype <= BL_F16, "gemm: unknown output dtype %d", out_dtype);
  BL_REQUIRE(aligned16(a_codes) && aligned16(b_codes) && aligned16(a_sf) && aligned16(b_sf) && aligned16(out),
             "gemm: operands, scales and output must be 16-byte aligned");
  BL_REQUIRE(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31), "gemm: dimension exceeds 2^31");
  BL_DEVICE(device);
  GemmArgs args;
  args.a_sf = a_sf;
  args.b_sf = b_sf;
  args.a_global = a_global;
  args.b_global = b_global;
  args.out = out;
  args.M = M;
  args.N = N;
  args.K = K;
  args.ldc = ldc;
  args.out_dtype = out_dtype;
  args.num_m = args.num_n = 0;
  args.accumulate = accumulate ? 1 : 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int kernel = g_kernel_choice.load(std::memory_order_relaxed);
  if (kernel == BL_GEMM_AUTO) {
    // Measured on B200: the pair kernel wins from two waves of 256 x 256 tiles, or from a quarter wave when K is long
    // enough to amortise its start-up; below that 128 x 256 tiles on single SMs fill the machine better, and small
    // problems spread best as 128 x 128 tiles.
    const int64_t tiles = ((M + 255) / 256) * ((N + 255) / 256);
    const int64_t tiles_1sm = ((M + 127) / 128) * ((N + 255) / 256);
    const int sms = sm_count(device);
    if (tiles >= sms || (tiles >= sms / 4 && K >= 16384)) kernel = BL_GEMM_PAIR;
    else if (tiles_1sm >= sms / 2) kernel = BL_GEMM_PERSISTENT;
    else kernel = BL_GEMM_TILE;
  }
  if (kernel == BL_GEMM_PAIR) return launch_pair<256, 5>(a_codes, b_codes, args, device, st);
  if (kernel == BL_GEMM_PERSISTENT) return launch_persistent<4, 0>(a_codes, b_codes, args, device, st);
  return launch_gemm<128, 3>(a_codes, b_codes, args, st);
}

extern "C" int bl_nvfp4_gemm(const uint8_t* a_codes, const uint8_t* a_sf, const float* a_global, const uint8_t* b_codes,
                             const uint8_t* b_sf, const float* b_global, int64_t M, int64_t N, int64_t K, void* out,
                             int out_dtype, int64_t ldc, int device, bl_stream_t stream) {
  return gemm_entry(a_codes, a_sf, a_global, b_codes, b_sf, b_global, M, N, K, out, out_dtype, ldc, 0, device, stream);
}

// out += (A B^T) * ga * gb: the sum of the input gradients of projections that read one input (q / k / v, gate / up)
// without a separate pass over the gradient. Bits of `out + product` as a dense add of two tensors of the output type.
extern "C" int bl_nvfp4_gemm_accumulate(const uint8_t* a_codes, const uint8_t* a_sf, const float* a_global,
                                        const uint8_t* b_codes, const uint8_t* b_sf, const float* b_global, int64_t M,
                                        int64_t N, int64_t K, void* out, int out_dtype, int64_t ldc, int device,
                                        bl_stream_t stream) {
  return gemm_entry(a_codes, a_sf, a_global, b_codes, b_sf, b_global, M, N, K, out, out_dtype, ldc, 1, device, stream);
}

// Forces one of the GEMM kernels (BL_GEMM_TILE, BL_GEMM_PERSISTENT, BL_GEMM_PAIR) for every later bl_nvfp4_gemm call
// of this process, or returns the choice to the library (BL_GEMM_AUTO). All kernels give identical results.
extern "C" int bl_nvfp4_gemm_select(int kernel) {
  BL_REQUIRE(kernel >= BL_GEMM_AUTO && kernel <= BL_GEMM_PAIR, "gemm_select: unknown kernel %d", kernel);
  g_kernel_choice.store(kernel, std::memory_order_relaxed);
  return 0;
}

// Reads (and clears) the device-side error flag of the GEMM kernels: 0 = no bounded wait expired so far.
// Synchronizes the device.
extern "C" int bl_nvfp4_gemm_status(int* status, int device) {
  BL_REQUIRE(status != nullptr, "gemm_status: null output");
  BL_DEVICE(device);
  int zero = 0;
  BL_CUDA(cudaMemcpyFromSymbol(status, g_gemm_error, sizeof(int)));
  BL_CUDA(cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int)));
  return 0;
}

// Copies the error flag (without clearing it) to `host_status`, which must be page-locked host memory, behind the
// work already enqueued on `stream`; the caller reads it after a later synchronisation of that stream. This is how a
// training loop watches the flag without a device synchronisation of its own.
extern "C" int bl_nvfp4_gemm_status_async(int* host_status, int device, bl_stream_t stream) {
  BL_REQUIRE(host_status != nullptr, "gemm_status_async: null output");
  BL_DEVICE(device);
  BL_CUDA(cudaMemcpyFromSymbolAsync(host_status, g_gemm_error, sizeof(int), 0, cudaMemcpyDeviceToHost,
                                    reinterpret_cast<cudaStream_t>(stream)));
  return 0;
}

// Runs the give-up path of the kernels' bounded waits in isolation (see selftest_bounded_wait_kernel) and reports
// what bl_nvfp4_gemm_status would: *status receives the recorded code (9 when the path works), *returned 2 when the
// kernel ran to its end after giving up. Synchronous; clears the flag; `scratch`: 4 bytes of device memory.
extern "C" int bl_selftest_bounded_wait(int* status, int* returned, int* scratch, int device) {
  BL_REQUIRE(status != nullptr && returned != nullptr && scratch != nullptr, "selftest_bounded_wait: null argument");
  BL_DEVICE(device);
  int zero = 0;
  BL_CUDA(cudaDeviceSynchronize());
  BL_CUDA(cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int)));
  BL_CUDA(cudaMemcpy(scratch, &zero, sizeof(int), cudaMemcpyHostToDevice));
  selftest_bounded_wait_kernel<<<1, 32>>>(scratch);
  BL_CUDA(cudaGetLastError());
  BL_CUDA(cudaMemcpy(returned, scratch, sizeof(int), cudaMemcpyDeviceToHost));
  BL_CUDA(cudaMemcpyFromSymbol(status, g_gemm_error, sizeof(int)));
  BL_CUDA(cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int)));
  return 0;
}

// Measures the tensor-pipe ceiling with mma_peak_kernel: `iters` k-tiles (4 MMAs of 128 x 256 x 64 each, or with
// mma_n = 128 the same work as 8 MMAs of 128 x 128 x 64) per SM, timed
// with CUDA events after one warm-up launch. *ms receives the duration, *flops the work (2 * 128 * 256 * 256 * iters
// * SMs). Synchronous; scratch: 4 bytes of device memory for the kernel's give-up code (returned as an error).
extern "C" int bl_selftest_mma_peak(int iters, int mma_n, float* ms, double* flops, int* scratch, int device) {
  BL_REQUIRE(iters > 0 && iters <= (1 << 20) && ms && flops && scratch, "selftest_mma_peak: bad argument");
  const int scales = mma_n / 1000;                  // thousands digit: how the scale columns are refreshed (see kernel)
  mma_n %= 1000;
  BL_REQUIRE(mma_n == 256 || mma_n == 128, "selftest_mma_peak: the MMA width is 256 or 128 columns");
  BL_REQUIRE(scales >= 0 && scales <= 1 && (scales == 0 || mma_n == 256), "selftest_mma_peak: unknown scale mode");
  auto kernel = mma_n == 128 ? mma_peak_kernel<128, 0> : scales == 0 ? mma_peak_kernel<256, 0> : mma_peak_kernel<256, 1>;
  BL_DEVICE(device);
  constexpr int kSmem = 128 * 128 + 256 * 128 + 3 * 2048 + 1024;
  BL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
  const int sms = sm_count(device);
  cudaEvent_t a, b;
  BL_CUDA(cudaEventCreate(&a));
  BL_CUDA(cudaEventCreate(&b));
  int zero = 0, code = 0;
  cudaError_t rc = cudaMemcpy(scratch, &zero, sizeof(int), cudaMemcpyHostToDevice);
  if (rc == cudaSuccess) {
    kernel<<<sms, 128, kSmem>>>(64, scratch);
    cudaEventRecord(a);
    kernel<<<sms, 128, kSmem>>>(iters, scratch);
    cudaEventRecord(b);
    rc = cudaEventSynchronize(b);
  }
  if (rc == cudaSuccess) rc = cudaGetLastError();
  if (rc == cudaSuccess) rc = cudaEventElapsedTime(ms, a, b);
  if (rc == cudaSuccess) rc = cudaMemcpy(&code, scratch, sizeof(int), cudaMemcpyDeviceToHost);
  cudaEventDestroy(a);
  cudaEventDestroy(b);
  BL_CUDA(rc);
  BL_REQUIRE(code == 0, "selftest_mma_peak: a bounded wait expired (code %d)", code);
  *flops = 2.0 * 128.0 * 256.0 * 256.0 * static_cast<double>(iters) * static_cast<double>(sms);
  return 0;
}
