// Speculative-decoding verification kernels for sm_100a (one thread per request; the work
// per request is at most max_spec_len + 1 steps).
//
//   rejection_greedy   accept draft tokens while they equal the target argmax, then emit the
//                      target token at the first mismatch or the bonus token
//   rejection_random   accept draft token x with probability min(1, p_target(x) / p_draft(x))
//                      (p_draft = 1 for draft-free proposers), else emit the recovered token
//   recovered_tokens   the token emitted in place of a rejected draft token
//   expand_batch_to_tokens  repeat a per-request value for each of its tokens
//
// Output rows are int32 [max_spec_len + 1], pre-filled with -1.
// Reference: csrc/src/rejection_greedy_sample.cpp:21, rejection_random_sample.cpp:24,31,
// expand_batch_to_tokens.cpp:18; torch oracles in
// vllm_gcu/patch/patch_0_9_2/rejection_sampler.py:11-120.
#include "common.cuh"

namespace b200 {
namespace spec {

__global__ void rejection_greedy_kernel(int* out, const int* draft_ids, const long long* target_argmax,
                                        const long long* bonus_ids, const int* num_draft, int B, int S) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  int* o = out + static_cast<long long>(b) * (S + 1);
  for (int i = 0; i <= S; ++i) o[i] = -1;
  const int n = min(num_draft[b], S);
  bool rejected = false;
  for (int i = 0; i < n; ++i) {
    const int t = static_cast<int>(target_argmax[static_cast<long long>(b) * (S + 1) + i]);
    o[i] = t;
    if (draft_ids[static_cast<long long>(b) * S + i] != t) {
      rejected = true;
      break;
    }
  }
  // the bonus token is the target's choice at the position after the last draft token
  if (!rejected)
    o[n] = bonus_ids ? static_cast<int>(bonus_ids[b])
                     : static_cast<int>(target_argmax[static_cast<long long>(b) * (S + 1) + n]);
}

__global__ void rejection_random_kernel(int* out, const int* draft_ids, const float* draft_probs,
                                        const float* target_probs, const long long* bonus_ids,
                                        const int* recovered_ids, const float* uniform,
                                        const int* num_draft, int B, int S, int V) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  int* o = out + static_cast<long long>(b) * (S + 1);
  for (int i = 0; i <= S; ++i) o[i] = -1;
  const int n = min(num_draft[b], S);
  bool rejected = false;
  for (int i = 0; i < n; ++i) {
    const long long bi = static_cast<long long>(b) * S + i;
    const int x = draft_ids[bi];
    const float pt = target_probs[bi * V + x];
    const float pd = draft_probs ? draft_probs[bi * V + x] : 1.0f;
    if (pd > 0.0f && pt / pd >= uniform[bi]) {
      o[i] = x;
    } else {
      o[i] = recovered_ids[bi];
      rejected = true;
      break;
    }
  }
  if (!rejected) o[n] = static_cast<int>(bonus_ids[b]);
}

// Recovered token of one (request, draft position): argmax over the vocabulary of
// max(0, p_target - p_draft) / noise (noise ~ Exp(1)); for draft-free proposers the draft
// token itself is excluded instead of subtracting a draft distribution.  One CTA per row;
// ties go to the smaller id, as torch.argmax does.
__global__ void __launch_bounds__(256)
    recovered_tokens_kernel(int* out, const int* draft_ids, const float* draft_probs,
                            const float* target_probs, const float* noise, int V) {
  __shared__ float s_val[8];
  __shared__ int s_idx[8];
  const long long row = blockIdx.x;
  const float* pt = target_probs + row * V;
  const float* pd = draft_probs ? draft_probs + row * V : nullptr;
  const float* nz = noise + row * V;
  const int skip = pd ? -1 : draft_ids[row];
  float best = -1.0f;
  int bi = 0x7fffffff;
  for (int v = threadIdx.x; v < V; v += blockDim.x) {
    float a = pd ? fmaxf(pt[v] - pd[v], 0.0f) : (v == skip ? 0.0f : pt[v]);
    a = a / fmaxf(nz[v], 1e-30f);
    if (a > best) { best = a; bi = v; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { s_val[threadIdx.x >> 5] = best; s_idx[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x < 32) {
    best = threadIdx.x < (blockDim.x >> 5) ? s_val[threadIdx.x] : -1.0f;
    bi = threadIdx.x < (blockDim.x >> 5) ? s_idx[threadIdx.x] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (threadIdx.x == 0) out[row] = bi == 0x7fffffff ? 0 : bi;
  }
}

__global__ void expand_batch_kernel(long long* out, const long long* x, const int* cu_num_tokens,
                                    int B, long long replace_from, long long replace_to) {
  const int b = blockIdx.x;
  if (b >= B) return;
  const int lo = b == 0 ? 0 : cu_num_tokens[b - 1], hi = cu_num_tokens[b];
  long long v = x[b];
  if (v == replace_from) v = replace_to;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) out[i] = v;
}

}  // namespace spec
}  // namespace b200

// target_argmax is [B, S + 1] (argmax of the target at every draft position and at the bonus
// position); bonus_ids may be null, in which case column S of target_argmax is the bonus.
B200_API int b200_rejection_greedy(int* out, const int* draft_ids, const long long* target_argmax,
                                   const long long* bonus_ids, const int* num_draft, int B, int S,
                                   void* stream) {
  if (B <= 0) return 0;
  b200::spec::rejection_greedy_kernel<<<(B + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      out, draft_ids, target_argmax, bonus_ids, num_draft, B, S);
  return static_cast<int>(cudaGetLastError());
}

B200_API int b200_rejection_random(int* out, const int* draft_ids, const float* draft_probs,
                                   const float* target_probs, const long long* bonus_ids,
                                   const int* recovered_ids, const float* uniform,
                                   const int* num_draft, int B, int S, int V, void* stream) {
  if (B <= 0) return 0;
  b200::spec::rejection_random_kernel<<<(B + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      out, draft_ids, draft_probs, target_probs, bonus_ids, recovered_ids, uniform, num_draft, B, S, V);
  return static_cast<int>(cudaGetLastError());
}

// out[b, i] (int32 [B, S]) = recovered token of draft position i of request b; probs and noise
// are fp32 [B, S, V] (draft_probs may be null for draft-free proposers).  Reference:
// vllm_gcu/patch/patch_0_9_2/rejection_sampler.py:94-120,174 (sample_recovered_tokens).
B200_API int b200_sample_recovered_tokens(int* out, const int* draft_ids,
                                          const float* draft_probs, const float* target_probs,
                                          const float* noise, int B, int S, int V, void* stream) {
  if (B <= 0 || S <= 0) return 0;
  if (V <= 0) return -2;
  b200::spec::recovered_tokens_kernel<<<B * S, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      out, draft_ids, draft_probs, target_probs, noise, V);
  return static_cast<int>(cudaGetLastError());
}

B200_API int b200_expand_batch_to_tokens(long long* out, const long long* x, const int* cu_num_tokens,
                                         int B, long long replace_from, long long replace_to,
                                         void* stream) {
  if (B <= 0) return 0;
  b200::spec::expand_batch_kernel<<<B, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      out, x, cu_num_tokens, B, replace_from, replace_to);
  return static_cast<int>(cudaGetLastError());
}
