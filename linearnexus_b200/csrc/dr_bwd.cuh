// placeholder until the backward lands
#pragma once
#include "dr_common.cuh"
namespace dr {
inline int64_t bwd_workspace_bytes(const DrDesc*) { return DR_ERR_UNSUPPORTED; }
inline cudaError_t launch_bwd(const DrDesc*, const void*, const void*, const void*, const void*, const float*, const float*, const void*, const float*, void*, void*, void*, float*, float*, float*, void*, cudaStream_t, int*) { return cudaErrorNotSupported; }
}
