// On-device step bookkeeping for sm_100a: multi-step advance and the
// device-side next-token feed of the asynchronous runner.
//
//   advance_step      input_tokens <- sampled, positions <- seq_lens,
//                     slot = block_table[seq / bs] * bs + seq % bs, seq_lens += 1
//   feed_tokens       input_ids[dst[i]] <- prev_sampled[src[i]] (scatter of the
//                     previous step's sampled ids, no host round trip)
//
// Reference: csrc/src/advance_step_kernel.tops:7-129,
// csrc/src/advance_step_flashattn.cpp:34 (contract in
// tests/kernels/test_advance_step.py:8-27) and
// vllm_gcu/v1/gcu_async_model_runner.py:370-473.
#include "common.cuh"

namespace b200 {
namespace step {

__global__ void advance_step_kernel(int num_seqs, int num_queries, int block_size,
                                    long long* input_tokens, const long long* sampled,
                                    long long* positions, int* seq_lens, long long* slot_mapping,
                                    const int* block_tables, int max_blocks, int active_only,
                                    unsigned int* status) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= num_seqs) return;
  if (i >= num_queries) {  // padded tail of a captured batch: keep it inert
    if (slot_mapping != nullptr) slot_mapping[i] = -1;
    return;
  }
  const int sl = seq_lens[i];
  if (active_only && sl <= 0) {  // inactive row of a padded batch
    if (slot_mapping != nullptr) slot_mapping[i] = -1;
    return;
  }
  input_tokens[i] = sampled[i];
  positions[i] = sl;
  const int blk_idx = sl / block_size;
  if (blk_idx >= max_blocks) {
    report_status(status, kStatusBounds, 40u, static_cast<unsigned>(i));
    slot_mapping[i] = -1;
  } else {
    slot_mapping[i] =
        static_cast<long long>(block_tables[static_cast<long long>(i) * max_blocks + blk_idx]) *
            block_size + sl % block_size;
  }
  seq_lens[i] = sl + 1;
}

__global__ void feed_tokens_kernel(long long* input_ids, const long long* prev_sampled,
                                   const int* dst_idx, const int* src_idx, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) input_ids[dst_idx[i]] = prev_sampled[src_idx[i]];
}

}  // namespace step
}  // namespace b200

B200_API int b200_advance_step(int num_seqs, int num_queries, int block_size,
                               long long* input_tokens, const long long* sampled,
                               long long* positions, int* seq_lens, long long* slot_mapping,
                               const int* block_tables, int max_blocks, int active_only,
                               void* stream) {
  if (num_seqs <= 0) return 0;
  b200::step::advance_step_kernel<<<(num_seqs + 255) / 256, 256, 0,
                                    static_cast<cudaStream_t>(stream)>>>(
      num_seqs, num_queries, block_size, input_tokens, sampled, positions, seq_lens, slot_mapping,
      block_tables, max_blocks, active_only, b200::status_ptr());
  return static_cast<int>(cudaGetLastError());
}

B200_API int b200_feed_tokens(long long* input_ids, const long long* prev_sampled,
                              const int* dst_idx, const int* src_idx, int n, void* stream) {
  if (n <= 0) return 0;
  b200::step::feed_tokens_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      input_ids, prev_sampled, dst_idx, src_idx, n);
  return static_cast<int>(cudaGetLastError());
}
