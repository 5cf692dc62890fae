// Quantizer-side kernels (offline toolchain, not the serving path).
//
// nvq_assign: nearest lattice codeword under a weighted squared error, fused.  For every vector v of `vec` weights
// (4 or 8) with per-element importance w and a scale s, find
//     argmin_c  sum_i w_i * (s * c_i - x_i)^2  =  argmin_c  sum_i c_i * (s^2 w_i c_i - 2 s w_i x_i)
// over a codebook of C entries.  The PyTorch formulation materialises two [V, C] matrices (gigabytes for a few hundred
// rows of a real layer) and re-reads them for every candidate scale of the search; here a thread keeps its vector in
// registers, the codebook streams through shared memory in slices, and nothing of size V x C ever exists.
// Ties go to the lowest index.
//
// The reference does this step in its JIT quantizer extension (mfq/quantize/cuda: nvq_quant_assign.cu and the
// nvq2j / nvq3j assign kernels).
#include "common.cuh"

#include <cfloat>

namespace mfq {

constexpr int kAssignSlice = 1024;  // codewords per shared-memory slice (32 KB of float at vec = 8)

template <int VEC>
__global__ void __launch_bounds__(256) nvq_assign_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                         const float* __restrict__ scale, const float* __restrict__ table,
                                                         int* __restrict__ idx, long long V, int C) {
  __shared__ float tab[kAssignSlice * VEC];
  const long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const bool live = v < V;
  float a[VEC], b[VEC];
  if (live) {
    const float s = scale[v];
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const float wi = w[v * VEC + i];
      a[i] = s * s * wi;
      b[i] = 2.f * s * wi * x[v * VEC + i];
    }
  }
  float best = FLT_MAX;
  int best_i = 0;
  for (int c0 = 0; c0 < C; c0 += kAssignSlice) {
    const int n = min(kAssignSlice, C - c0);
    __syncthreads();
    for (int i = threadIdx.x; i < n * VEC; i += blockDim.x) tab[i] = table[size_t(c0) * VEC + i];
    __syncthreads();
    if (live) {
      for (int c = 0; c < n; ++c) {
        float cost = 0.f;
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          const float ci = tab[c * VEC + i];  // every thread reads the same address: a broadcast
          cost = fmaf(ci, fmaf(a[i], ci, -b[i]), cost);
        }
        if (cost < best) { best = cost; best_i = c0 + c; }
      }
    }
  }
  if (live) idx[v] = best_i;
}

}  // namespace mfq

// x, w: [V, vec] fp32; scale: [V] fp32; table: [C, vec] fp32; idx: [V] int32.  vec in {4, 8}.
extern "C" int mfq_nvq_assign(const float* x, const float* w, const float* scale, const float* table, int* idx,
                              long long V, int C, int vec, cudaStream_t stream) {
  if (V <= 0 || C <= 0 || (vec != 4 && vec != 8)) return -1;
  const unsigned blocks = unsigned((V + 255) / 256);
  if (vec == 8) mfq::nvq_assign_kernel<8><<<blocks, 256, 0, stream>>>(x, w, scale, table, idx, V, C);
  else mfq::nvq_assign_kernel<4><<<blocks, 256, 0, stream>>>(x, w, scale, table, idx, V, C);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}
