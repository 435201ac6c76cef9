// Host-side helpers shared by the translation units of the library (defined in capi.cu).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

typedef CUresult (*CfEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// the driver's cuTensorMapEncodeTiled, looked up once through the runtime (nullptr if unavailable)
CfEncodeTiledFn cf_host_encode_fn();
// records the thread-local message behind cf_last_error() and returns `code`
int cf_host_fail(int code, const char* fmt, ...);
// CF_ERR_INVALID (with a message naming `what`) while `st` is being captured, CF_OK otherwise
int cf_host_refuse_in_capture(cudaStream_t st, const char* what);
// status word of the batched Llama path on device `dev` (0 when unused); cleared when it was set
int cf_host_lb_probe_status(int dev, int* status);
