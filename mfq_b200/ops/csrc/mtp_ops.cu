// Device-side bookkeeping of the MTP draft/verify cycle, so that the whole cycle replays as one CUDA graph.
//
// State before a cycle, per row: seq_len tokens are in the KV cache, `sampled` is the last confirmed token (not yet
// cached) and draft[0..K) are the head's guesses for the tokens after it.
//   mtp_prepare: lays out the verify window  [sampled, draft_0 .. draft_{K-1}]  with positions, KV slots and the
//                window-inclusive sequence length the attention kernel expects.
//   mtp_accept:  compares drafts with the verify arg-maxes (greedy acceptance: the longest matching prefix), emits
//                the confirmed tokens, advances seq_len by accepted + 1, makes the last confirmed token the new
//                `sampled`, and takes the next cycle's first draft from the head's prediction at that position.
// Rejected positions leave stale KV rows behind that the next window overwrites; nothing needs to be rolled back
// for attention layers.  Reference: the greedy chain verification of cpp_runtime/engine/include/mtp_policy.h:51 and
// the graph-captured predictor of backends/cuda/engine/mtp.cpp.
#include "common.cuh"

namespace mfq {

__global__ void mtp_prepare_kernel(const int* __restrict__ sampled, const int* __restrict__ draft,
                                   const int* __restrict__ seq_lens, const int* __restrict__ block_table,
                                   const int* __restrict__ active, int* __restrict__ input_ids, int* __restrict__ positions,
                                   int* __restrict__ slots, int* __restrict__ window_lens, int B, int K, int max_pages,
                                   int page_size) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int W = K + 1;
  if (i >= B * W) return;
  const int b = i / W, j = i % W;
  const bool on = !active || active[b];
  const int len = seq_lens[b];
  input_ids[i] = j == 0 ? sampled[b] : draft[b * K + j - 1];
  const int pos = len + j;
  positions[i] = pos;
  const int page = block_table[size_t(b) * max_pages + min(pos / page_size, max_pages - 1)];
  slots[i] = on ? page * page_size + pos % page_size : -1;
  if (j == 0) window_lens[b] = on ? len + W : len;
}

// targets[b, W]: arg-max of the verify logits at each window position; head_next[b, W]: the head's arg-max when fed
// (hidden of window position j, target_j).  out_tokens[b, W] gets the confirmed tokens (-1 padded), n_out[b] their count.
__global__ void mtp_accept_kernel(const int* __restrict__ targets, const int* __restrict__ head_next,
                                  const int* __restrict__ active, int* __restrict__ draft, int* __restrict__ sampled,
                                  int* __restrict__ seq_lens, int* __restrict__ out_tokens, int* __restrict__ n_out,
                                  int* __restrict__ accept_row, unsigned long long* __restrict__ stats, int B, int K) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const int W = K + 1;
  if (active && !active[b]) { n_out[b] = 0; accept_row[b] = 0; return; }
  int a = 0;
  while (a < K && draft[b * K + a] == targets[b * W + a]) ++a;
  for (int j = 0; j < W; ++j) out_tokens[b * W + j] = j <= a ? targets[b * W + j] : -1;
  n_out[b] = a + 1;
  accept_row[b] = a;
  sampled[b] = targets[b * W + a];
  seq_lens[b] += a + 1;
  draft[b * K] = head_next[b * W + a];
  if (stats) { atomicAdd(&stats[0], (unsigned long long)K); atomicAdd(&stats[1], (unsigned long long)a); }
}

// rows_out[b] = rows_in[b * W + accept_row[b]]  (hidden state of the last confirmed position, for chained drafts)
__global__ void mtp_select_rows_kernel(const __nv_bfloat16* __restrict__ in, const int* __restrict__ accept_row,
                                       __nv_bfloat16* __restrict__ out, int W, int H) {
  const int b = blockIdx.x;
  const uint4* src = reinterpret_cast<const uint4*>(in + (size_t(b) * W + accept_row[b]) * H);
  uint4* dst = reinterpret_cast<uint4*>(out + size_t(b) * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

}  // namespace mfq

extern "C" int mfq_mtp_prepare(const int* sampled, const int* draft, const int* seq_lens, const int* block_table,
                               const int* active, int* input_ids, int* positions, int* slots, int* window_lens, int B,
                               int K, int max_pages, int page_size, cudaStream_t stream) {
  if (B <= 0 || K < 1) return -1;
  const int n = B * (K + 1);
  mfq::mtp_prepare_kernel<<<(n + 127) / 128, 128, 0, stream>>>(sampled, draft, seq_lens, block_table, active, input_ids,
                                                             positions, slots, window_lens, B, K, max_pages, page_size);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

extern "C" int mfq_mtp_accept(const int* targets, const int* head_next, const int* active, int* draft, int* sampled,
                              int* seq_lens, int* out_tokens, int* n_out, int* accept_row, void* stats, int B, int K,
                              cudaStream_t stream) {
  if (B <= 0 || K < 1) return -1;
  mfq::mtp_accept_kernel<<<(B + 127) / 128, 128, 0, stream>>>(targets, head_next, active, draft, sampled, seq_lens,
                                                            out_tokens, n_out, accept_row,
                                                            static_cast<unsigned long long*>(stats), B, K);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

extern "C" int mfq_mtp_select_rows(const void* in, const int* accept_row, void* out, int B, int W, int H,
                                   cudaStream_t stream) {
  if (B <= 0 || H % 8) return -1;
  mfq::mtp_select_rows_kernel<<<B, 128, 0, stream>>>(static_cast<const __nv_bfloat16*>(in), accept_row,
                                                     static_cast<__nv_bfloat16*>(out), W, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}
