// SwiGLU glue between the gate/up and the down projection: a = T(T(silu(g)) * u) and its backward, every
// intermediate rounded to the activation type T (bf16 or fp16) exactly where PyTorch autograd rounds
// `F.silu(g) * u` -- so the op can replace the autograd expression bit for bit in the forward and in du.
// Reference operators: torch.ops.bitlattice.swiglu_fwd / swiglu_bwd (csrc/swiglu.cu:20-80, csrc/bindings.cpp:126-129).
//
// Pure streaming work: 2 reads + 1 write (forward), 3 reads + 2 writes (backward) of 2-byte elements; one thread
// handles 8 consecutive elements (16-byte accesses), grid-stride over the tensor.
#include "common.cuh"

namespace blb {

constexpr int kGluThreads = 256;

// ATen's silu in its op-math type: x / (1 + exp(-x)), true division
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }

template <typename T>
struct Pack8 {
  uint4 raw;
  __device__ __forceinline__ float get(int i) const { return to_f<T>(reinterpret_cast<const T*>(&raw)[i]); }
  __device__ __forceinline__ void set(int i, float v) { reinterpret_cast<T*>(&raw)[i] = from_f<T>(v); }
};

template <typename T>
__device__ __forceinline__ float round_to(float v) { return to_f<T>(from_f<T>(v)); }

template <typename T>
__device__ __forceinline__ float glu_forward(float g, float u) { return round_to<T>(silu_f(g)) * u; }

// (dg, du) for one element; the order of operations is ATen's silu_backward: d * sig * (1 + g * (1 - sig))
template <typename T>
__device__ __forceinline__ void glu_backward(float g, float u, float da, float& dg, float& du) {
  du = da * round_to<T>(silu_f(g));
  const float ds = round_to<T>(da * u);
  const float sig = 1.0f / (1.0f + expf(-g));
  dg = ds * sig * (1.0f + g * (1.0f - sig));
}

template <typename T>
__global__ void __launch_bounds__(kGluThreads) swiglu_fwd_kernel(const T* __restrict__ g, const T* __restrict__ u,
                                                                 T* __restrict__ a, int64_t n) {
  const int64_t nvec = n / 8, stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec; v += stride) {
    Pack8<T> pg, pu, pa;
    pg.raw = __ldcs(reinterpret_cast<const uint4*>(g) + v);
    pu.raw = __ldcs(reinterpret_cast<const uint4*>(u) + v);
#pragma unroll
    for (int i = 0; i < 8; ++i) pa.set(i, glu_forward<T>(pg.get(i), pu.get(i)));
    reinterpret_cast<uint4*>(a)[v] = pa.raw;
  }
  // ragged tail: the last n % 8 elements, one per thread of block 0
  const int64_t t = nvec * 8 + threadIdx.x;
  if (blockIdx.x == 0 && t < n) a[t] = from_f<T>(glu_forward<T>(to_f<T>(g[t]), to_f<T>(u[t])));
}

template <typename T>
__global__ void __launch_bounds__(kGluThreads) swiglu_bwd_kernel(const T* __restrict__ g, const T* __restrict__ u,
                                                                 const T* __restrict__ da, T* __restrict__ dg,
                                                                 T* __restrict__ du, int64_t n) {
  const int64_t nvec = n / 8, stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec; v += stride) {
    Pack8<T> pg, pu, pd, og, ou;
    pg.raw = __ldcs(reinterpret_cast<const uint4*>(g) + v);
    pu.raw = __ldcs(reinterpret_cast<const uint4*>(u) + v);
    pd.raw = __ldcs(reinterpret_cast<const uint4*>(da) + v);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float x, y;
      glu_backward<T>(pg.get(i), pu.get(i), pd.get(i), x, y);
      og.set(i, x);
      ou.set(i, y);
    }
    reinterpret_cast<uint4*>(dg)[v] = og.raw;
    reinterpret_cast<uint4*>(du)[v] = ou.raw;
  }
  const int64_t t = nvec * 8 + threadIdx.x;
  if (blockIdx.x == 0 && t < n) {
    float x, y;
    glu_backward<T>(to_f<T>(g[t]), to_f<T>(u[t]), to_f<T>(da[t]), x, y);
    dg[t] = from_f<T>(x);
    du[t] = from_f<T>(y);
  }
}

static int glu_grid(int64_t n, int device) {
  const int64_t blocks = (n / 8 + kGluThreads - 1) / kGluThreads;
  const int64_t cap = static_cast<int64_t>(sm_count(device)) * 8;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace blb

using namespace blb;

extern "C" int bl_swiglu_fwd(const void* g, const void* u, void* a, int dtype, int64_t n, int device,
                             bl_stream_t stream) {
  BL_REQUIRE(g && u && a && n > 0, "swiglu_fwd: null or empty buffer");
  BL_REQUIRE(dtype == BL_BF16 || dtype == BL_F16, "swiglu_fwd: activations must be bf16 or fp16, got dtype %d", dtype);
  BL_REQUIRE(aligned16(g) && aligned16(u) && aligned16(a), "swiglu_fwd: buffers must be 16-byte aligned");
  BL_DEVICE(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int grid = glu_grid(n, device);
  if (dtype == BL_BF16)
    swiglu_fwd_kernel<<<grid, kGluThreads, 0, st>>>(static_cast<const __nv_bfloat16*>(g),
                                                    static_cast<const __nv_bfloat16*>(u),
                                                    static_cast<__nv_bfloat16*>(a), n);
  else
    swiglu_fwd_kernel<<<grid, kGluThreads, 0, st>>>(static_cast<const __half*>(g), static_cast<const __half*>(u),
                                                    static_cast<__half*>(a), n);
  BL_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int bl_swiglu_bwd(const void* g, const void* u, const void* da, void* dg, void* du, int dtype, int64_t n,
                             int device, bl_stream_t stream) {
  BL_REQUIRE(g && u && da && dg && du && n > 0, "swiglu_bwd: null or empty buffer");
  BL_REQUIRE(dtype == BL_BF16 || dtype == BL_F16, "swiglu_bwd: activations must be bf16 or fp16, got dtype %d", dtype);
  BL_REQUIRE(aligned16(g) && aligned16(u) && aligned16(da) && aligned16(dg) && aligned16(du),
             "swiglu_bwd: buffers must be 16-byte aligned");
  BL_DEVICE(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int grid = glu_grid(n, device);
  if (dtype == BL_BF16)
    swiglu_bwd_kernel<<<grid, kGluThreads, 0, st>>>(
        static_cast<const __nv_bfloat16*>(g), static_cast<const __nv_bfloat16*>(u),
        static_cast<const __nv_bfloat16*>(da), static_cast<__nv_bfloat16*>(dg), static_cast<__nv_bfloat16*>(du), n);
  else
    swiglu_bwd_kernel<<<grid, kGluThreads, 0, st>>>(static_cast<const __half*>(g), static_cast<const __half*>(u),
                                                    static_cast<const __half*>(da), static_cast<__half*>(dg),
                                                    static_cast<__half*>(du), n);
  BL_CUDA(cudaGetLastError());
  return 0;
}
