// Stochastic sampling for continuous batching: one CTA per row applies penalties, temperature, top-k and top-p and
// draws a token, without sorting the vocabulary.  The top-k cut and the nucleus cut are both found by bisection on
// the logit value (count / probability mass above a threshold), the token by a block-wide prefix scan in index order,
// with a counter-based random number per (seed, step), so a request replays identically.
// Reference: mfq/kernels/cuda/sampling.cu (radix-select top-k, top-p, presence/frequency/repetition penalties,
// batched transform/resolve).
#include "common.cuh"

#include <cfloat>

namespace mfq {

struct SampleRow {
  float temperature;     // <= 0: greedy
  int top_k;             // <= 0: off
  float top_p;           // >= 1: off
  float presence, frequency, repetition;  // 0, 0, 1: off
  unsigned long long seed;
};

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < (blockDim.x >> 5); ++i) t += red[i];
  return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = -FLT_MAX;
  for (int i = 0; i < (blockDim.x >> 5); ++i) t = fmaxf(t, red[i]);
  return t;
}
// splitmix64-style counter hash -> uniform in [0, 1)
__device__ __forceinline__ float uniform01(unsigned long long seed, unsigned long long step) {
  unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (step + 1);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return float(z >> 40) * (1.f / 16777216.f);
}

// logits [B, V] bf16 (row stride `stride`); counts [B, V] uint16 occurrences of each token in the row's sequence
// (may be null); work [B, V] fp32 scratch; out [B] sampled ids; steps [B] per-row draw counter (read only).
//
// Speculative verification (`window` > 1, `draft` given): the B rows are `window` consecutive positions of B / window
// sequences; `rows` / `steps` are per SEQUENCE, position i draws with counter steps[seq] + i.  Positions 0 .. window-2
// carry a draft token x = draft[seq][i] that was proposed deterministically (the draft head's arg-max), i.e. from a
// one-hot proposal, so speculative sampling keeps it with probability p(x) under this row's processed target
// distribution and otherwise draws from p with x removed -- the emitted token is then distributed exactly as p.  The
// last position has no draft and is a plain draw.  Greedy rows return the arg-max either way, so comparing `out` with
// the draft (what the accept kernel does) is the verification in both modes.
__global__ void __launch_bounds__(1024)
sample_kernel(const __nv_bfloat16* __restrict__ logits, int V, int stride, const unsigned short* __restrict__ counts,
              const SampleRow* __restrict__ rows, const int* __restrict__ steps, float* __restrict__ work,
              int* __restrict__ out, int window, const int* __restrict__ draft) {
  __shared__ float red[32];
  __shared__ float s_scan[33];
  const int b = blockIdx.x, tid = threadIdx.x;
  const int seq = b / window, pos = b - seq * window;
  const SampleRow r = rows[seq];
  const int x = (draft && pos < window - 1) ? draft[seq * (window - 1) + pos] : -1;
  const __nv_bfloat16* lr = logits + size_t(b) * stride;
  float* w = work + size_t(b) * V;
  const unsigned short* cr = counts ? counts + size_t(b) * V : nullptr;
  const bool greedy = r.temperature <= 0.f;
  const float inv_t = greedy ? 1.f : 1.f / r.temperature;
  float mx = -FLT_MAX;
  int mi = 0x7fffffff;
  for (int i = tid; i < V; i += blockDim.x) {
    float l = __bfloat162float(lr[i]);
    if (cr) {
      const int c = cr[i];
      if (c > 0) {
        l = l > 0.f ? l / r.repetition : l * r.repetition;
        l -= r.presence + r.frequency * float(c);
      }
    }
    l *= inv_t;
    w[i] = l;
    if (l > mx) { mx = l; mi = i; }
  }
  const float gmax = block_max(mx, red);
  {
    // lowest index among the maxima: the greedy answer, and the fallback should the draw below hit a rounding edge
    int cand = (mx == gmax) ? mi : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
    __shared__ int s_idx[32];
    __syncthreads();
    if ((tid & 31) == 0) s_idx[tid >> 5] = cand;
    __syncthreads();
    if (tid == 0) {
      int best = 0x7fffffff;
      for (int i = 0; i < (blockDim.x >> 5); ++i) best = min(best, s_idx[i]);
      out[b] = best;
    }
    if (greedy) return;
  }
  // ---- top-k: lowest threshold (in logit units below the maximum) that keeps at most k tokens ----
  float lo_cut = gmax - 80.f;  // exp(-80) of the maximum: below that a token has no measurable mass
  if (r.top_k > 0 && r.top_k < V) {
    float lo = gmax - 80.f, hi = gmax;
    for (int it = 0; it < 24; ++it) {
      const float mid = 0.5f * (lo + hi);
      float cnt = 0.f;
      for (int i = tid; i < V; i += blockDim.x) cnt += w[i] >= mid ? 1.f : 0.f;
      cnt = block_sum(cnt, red);
      if (cnt > float(r.top_k)) lo = mid; else hi = mid;
    }
    lo_cut = hi;
  }
  // ---- probabilities of the kept set, then the nucleus cut ----
  float z = 0.f;
  for (int i = tid; i < V; i += blockDim.x) z += w[i] >= lo_cut ? __expf(w[i] - gmax) : 0.f;
  z = block_sum(z, red);
  float cut = lo_cut;
  if (r.top_p < 1.f) {
    float lo = lo_cut, hi = gmax;  // mass(lo) >= p * z by construction; find the highest cut that still has it
    for (int it = 0; it < 24; ++it) {
      const float mid = 0.5f * (lo + hi);
      float m = 0.f;
      for (int i = tid; i < V; i += blockDim.x) m += w[i] >= mid ? __expf(w[i] - gmax) : 0.f;
      m = block_sum(m, red);
      if (m >= r.top_p * z) lo = mid; else hi = mid;
    }
    cut = lo;
  }
  // mass of the draft token inside the kept set (0: no draft, or the cuts removed it -> it can only be rejected)
  const float e_x = (x >= 0 && x < V && w[x] >= cut) ? __expf(w[x] - gmax) : 0.f;
  // ---- draw: inverse CDF over index order, the draft token left out; each thread owns a contiguous slice ----
  const int per = (V + blockDim.x - 1) / blockDim.x;
  const int i0 = tid * per, i1 = min(V, i0 + per);
  float mine = 0.f;
  for (int i = i0; i < i1; ++i) mine += (w[i] >= cut && i != x) ? __expf(w[i] - gmax) : 0.f;
  // block exclusive scan of `mine`
  float incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, incl, o);
    if ((tid & 31) >= o) incl += n;
  }
  __syncthreads();
  if ((tid & 31) == 31) s_scan[tid >> 5] = incl;
  __syncthreads();
  if (tid == 0) {
    float run = 0.f;
    for (int i = 0; i < (blockDim.x >> 5); ++i) { const float t = s_scan[i]; s_scan[i] = run; run += t; }
    s_scan[32] = run;
  }
  __syncthreads();
  const float total = s_scan[32];  // without the draft token
  const unsigned long long step = (unsigned long long)(steps[seq] + pos);
  if (x >= 0) {
    // keep the draft with probability p(x) = e_x / (total + e_x); every thread takes the same branch
    const float ua = uniform01(r.seed ^ 0x5DEECE66Dull, step);
    if (ua * (total + e_x) < e_x || total <= 0.f) {
      if (tid == 0) out[b] = x;
      return;
    }
  }
  const float before = s_scan[tid >> 5] + incl - mine;
  const float target = uniform01(r.seed, step) * total;
  if (target >= before && (target < before + mine || (tid == blockDim.x - 1))) {
    float run = before;
    int pick = -1;
    for (int i = i0; i < i1; ++i) {
      if (w[i] >= cut && i != x) {
        run += __expf(w[i] - gmax);
        pick = i;
        if (run > target) break;
      }
    }
    if (pick >= 0) out[b] = pick;
  }
}

}  // namespace mfq

// rows: device array of B records {temperature, top_k, top_p, presence, frequency, repetition, seed} (see SampleRow).
extern "C" int mfq_sample(const void* logits, int B, int V, int stride, const void* counts, const void* rows,
                          const int* steps, float* work, int* out, cudaStream_t stream) {
  if (B <= 0 || V <= 0) return -1;
  mfq::sample_kernel<<<B, 1024, 0, stream>>>(static_cast<const __nv_bfloat16*>(logits), V, stride,
                                             static_cast<const unsigned short*>(counts),
                                             static_cast<const mfq::SampleRow*>(rows), steps, work, out, 1, nullptr);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

// Verification draw for speculative decoding: logits [B * window, V] (window consecutive positions per sequence), rows /
// steps [B] per sequence, draft [B, window - 1] proposed tokens; out [B * window] = the token each position emits (the
// draft where it was kept).  See sample_kernel.
extern "C" int mfq_sample_verify(const void* logits, int B, int window, int V, int stride, const void* rows, const int* steps,
                                 const int* draft, float* work, int* out, cudaStream_t stream) {
  if (B <= 0 || V <= 0 || window < 1) return -1;
  mfq::sample_kernel<<<B * window, 1024, 0, stream>>>(static_cast<const __nv_bfloat16*>(logits), V, stride, nullptr,
                                                      static_cast<const mfq::SampleRow*>(rows), steps, work, out, window,
                                                      window > 1 ? draft : nullptr);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}
