// The encoder / head MLP under the bfloat16 autocast contract on tensor-core tiles (mlp_kernels.cu).
#pragma once
#include <cuda_runtime.h>

namespace bnb {
namespace mlp {

// Whether the tiled kernel serves these widths (else the caller uses the CUDA-core engine).
bool supported(int in_pad, int hidden, int out_dim);

// Linear(in, hidden) + b1 -> RMSNorm(g1) -> GELU -> Linear(hidden, out) + b2 [-> RMSNorm(g2)], bfloat16 result,
// the first out_store columns of each row stored.  w1 is (hidden, in_pad) with zero columns beyond in_dim.
// x holds float32 rows, or with x_bf16 bfloat16 rows (then in_dim == in_pad and x on a 16-byte boundary).
int encoder_mlp_bf16(const float* w1, const float* b1, const float* g1, const float* w2, const float* b2, const float* g2,
                     int in_dim, int in_pad, int hidden, int out_dim, int out_store, const void* x, bool x_bf16, void* y,
                     int n_rows, cudaStream_t st);

}  // namespace mlp
}  // namespace bnb
