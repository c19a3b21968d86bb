// Fused attention launcher (see attention.cu).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace gcb {
// O = softmax(Q K^T * scale [+ causal mask]) V for `bh` independent (batch, head)
// units; Q, K, V, O are [bh][seq][dim] bf16, contiguous.
void attention_bf16(const void *Q, const void *K, const void *V, void *O, int64_t bh, int64_t seq, int64_t dim,
                    float scale, int causal, cudaStream_t stream);
} // namespace gcb
