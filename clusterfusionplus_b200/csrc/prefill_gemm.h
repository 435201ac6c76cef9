// Internal interface between the C ABI (capi.cu) and the tensor-core prefill GEMM
// (prefill_gemm.cu), which is compiled on its own because of its template weight.
#pragma once
#include <cuda_runtime.h>

namespace cfb {

enum : int { PREFILL_ACT_NONE = 0, PREFILL_ACT_GELU_TANH = 1, PREFILL_ACT_GELU_ERF = 2 };

// out[m,n] = act(x[m,k] . w[n,k]^T + bias[n] + residual[m,n]); bias and residual may be null.
// Returns null on success, else a static message.  Asynchronous on `st`.
const char* prefill_linear(const void* x, const void* w, const void* bias, const void* residual, void* out, int m, int n,
                           int k, int act, cudaStream_t st);

}  // namespace cfb
