// placeholder until the tcgen05 kernel lands
#pragma once
#include "dr_common.cuh"
namespace dr { namespace sm100 {
constexpr bool kAvailable = false;
inline cudaError_t launch_chunk(const FwdParams&, cudaStream_t) { return cudaErrorNotSupported; }
}}
