// GEMM operands of a full NVFP4 weight assembled from the row shards that an all-gather delivered.
//
// Every rank r of p sends one buffer holding, for a weight W [N, K] of which it owns n = N / p rows,
//   codes      [n, K/2]      its rows of W's E2M1 codes,
//   tiled_sf   tiled bytes   its rows of W's E4M3 scales in the GEMM's 128x4-tiled layout (n % 128 == 0: whole tiles),
//   t_codes    [K, n/2]      its column slice of the re-quantized W^T's codes,
//   t_sf       [K, n/16]     its column slice of W^T's scales, row-major,
// each at its own byte offset inside the buffer; the all-gather stacks the p buffers `rank_stride` bytes apart. One
// launch cuts the stacked buffers back into the two operands the GEMMs read: W (codes and tiled scales are plain
// rank-order concatenations) and W^T (column slices put side by side, scales re-tiled on the way). Pure byte movement,
// HBM-bound: 16-byte words for the codes and concatenations, 4-byte words for the transposed scales (four consecutive
// scale columns are four consecutive bytes of a tile row).
#include "common.cuh"

namespace blb {

constexpr int kGatherThreads = 256;

struct GatherArgs {
  const uint8_t* recv;
  int64_t rank_stride;
  int p;
  int64_t n, K;
  int64_t off_codes, off_sf, off_tcodes, off_tsf;
  int64_t sf_bytes;                       // tiled scale bytes of one shard
  uint8_t *codes, *sf, *tcodes, *tsf;
};

__global__ void __launch_bounds__(kGatherThreads) assemble_gathered_kernel(GatherArgs a) {
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t code_w = a.n * a.K / 32;             // 16-byte words of one shard's codes (and of its W^T slice)
  const int64_t sf_w = a.sf_bytes / 16;
  // W: codes and tiled scales, rank after rank
  for (int64_t i = tid; i < code_w * a.p; i += nthreads) {
    const int64_t r = i / code_w, j = i - r * code_w;
    reinterpret_cast<uint4*>(a.codes)[i] =
        reinterpret_cast<const uint4*>(a.recv + r * a.rank_stride + a.off_codes)[j];
  }
  for (int64_t i = tid; i < sf_w * a.p; i += nthreads) {
    const int64_t r = i / sf_w, j = i - r * sf_w;
    reinterpret_cast<uint4*>(a.sf)[i] = reinterpret_cast<const uint4*>(a.recv + r * a.rank_stride + a.off_sf)[j];
  }
  // W^T codes: row k of the result is the p slices' rows k side by side; n/2 bytes per slice row = n/32 words
  const int64_t row_w = a.n / 32;
  for (int64_t i = tid; i < code_w * a.p; i += nthreads) {
    const int64_t k = i / (row_w * a.p), rem = i - k * (row_w * a.p);
    const int64_t r = rem / row_w, j = rem - r * row_w;
    reinterpret_cast<uint4*>(a.tcodes)[i] =
        reinterpret_cast<const uint4*>(a.recv + r * a.rank_stride + a.off_tcodes)[k * row_w + j];
  }
  // W^T scales [K, N/16] into the tiled layout: offset(k, c) = ((k/128) * ceil(C/4) + c/4) * 512 + (k%32) * 16 +
  // ((k/32)%4) * 4 + c%4 with C = N/16; groups of four columns move as one 32-bit word (n/16 is a multiple of 8)
  const int64_t slice_q = a.n / 64;                  // 4-byte words per slice row
  const int64_t C4 = a.p * slice_q;                  // = ceil(C/4), C a multiple of 4
  for (int64_t i = tid; i < a.K * C4; i += nthreads) {
    const int64_t k = i / C4, q = i - k * C4;        // q: group of four scale columns of the full matrix
    const int64_t r = q / slice_q, j = q - r * slice_q;
    const uint32_t v = reinterpret_cast<const uint32_t*>(a.recv + r * a.rank_stride + a.off_tsf)[k * slice_q + j];
    const int64_t dst = ((k >> 7) * C4 + q) * 512 + (k & 31) * 16 + ((k >> 5) & 3) * 4;
    *reinterpret_cast<uint32_t*>(a.tsf + dst) = v;
  }
}

}  // namespace blb

using namespace blb;

extern "C" int bl_nvfp4_assemble_gathered(const uint8_t* recv, int64_t rank_stride, int p, int64_t n, int64_t K,
                                          int64_t off_codes, int64_t off_sf, int64_t off_tcodes, int64_t off_tsf,
                                          uint8_t* codes, uint8_t* sf, uint8_t* tcodes, uint8_t* tsf, int device,
                                          bl_stream_t stream) {
  BL_REQUIRE(recv && codes && sf && tcodes && tsf, "assemble_gathered: null buffer");
  BL_REQUIRE(p > 0 && n > 0 && K > 0, "assemble_gathered: empty shard (%d x %lld x %lld)", p, (long long)n, (long long)K);
  BL_REQUIRE(n % 128 == 0 && K % 64 == 0, "assemble_gathered: shards of %lld rows x %lld columns (rows %% 128, columns "
             "%% 64 are required)", (long long)n, (long long)K);
  BL_REQUIRE(rank_stride % 16 == 0 && off_codes % 16 == 0 && off_sf % 16 == 0 && off_tcodes % 16 == 0 && off_tsf % 16 == 0,
             "assemble_gathered: offsets and the rank stride must be multiples of 16 bytes");
  BL_REQUIRE(aligned16(recv) && aligned16(codes) && aligned16(sf) && aligned16(tcodes) && aligned16(tsf),
             "assemble_gathered: buffers must be 16-byte aligned");
  BL_DEVICE(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  GatherArgs a;
  a.recv = recv;
  a.rank_stride = rank_stride;
  a.p = p;
  a.n = n;
  a.K = K;
  a.off_codes = off_codes;
  a.off_sf = off_sf;
  a.off_tcodes = off_tcodes;
  a.off_tsf = off_tsf;
  a.sf_bytes = static_cast<int64_t>(bl_blocked_scale_bytes(n, K / 16));
  a.codes = codes;
  a.sf = sf;
  a.tcodes = tcodes;
  a.tsf = tsf;
  // W^T scales: K rows in tiles of 128 -- rows of a last partial tile that no k reaches must read as zero
  if (K % 128 != 0) BL_CUDA(cudaMemsetAsync(tsf, 0, bl_blocked_scale_bytes(K, static_cast<int64_t>(p) * n / 16), st));
  const int64_t work = static_cast<int64_t>(p) * n * K / 32;
  int64_t blocks = (work + kGatherThreads - 1) / kGatherThreads;
  const int64_t cap = static_cast<int64_t>(sm_count(device)) * 16;
  if (blocks > cap) blocks = cap;
  assemble_gathered_kernel<<<static_cast<unsigned>(blocks), kGatherThreads, 0, st>>>(a);
  BL_CUDA(cudaGetLastError());
  return 0;
}
