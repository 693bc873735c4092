// Device half of the sampler (sampler.cu) and the host half shared with the CPU-testable entry points.
#pragma once
#include <cuda_runtime.h>

#include "../../include/tenzo.h"

namespace tz {

constexpr int kMaxCandidates = 2048;   // candidates (logits >= the k-th largest) the device hands to the host

cudaError_t launch_penalty(float* logits, int vocab, const int* tokens, const int* counts, int n, float penalty, cudaStream_t st);
cudaError_t launch_select_candidates(const float* logits, int vocab, int k, int* out_count, float* out_val, int* out_idx, cudaStream_t st);

// The reference's streaming top-k + softmax + top-p + draw over (value, index) pairs given in ascending index order
// (the whole vocabulary, or the candidates of launch_select_candidates). r in [0,1] replaces rand()/RAND_MAX; r < 0
// draws from rand(). temperature <= 0: first maximum.
int sample_pairs(const float* vals, const int* idxs, int n, const tenzo_sampling_params_t& p, float r);

}  // namespace tz
