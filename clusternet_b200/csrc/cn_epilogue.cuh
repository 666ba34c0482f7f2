// Elementwise pieces shared by the stand-alone kernels and the GEMM tile stores.
#pragma once
#include <float.h>
#include "cn_internal.h"

// rectified_linear / logistic / doubleRectifiedLinear / LinearUnit exactly as the reference kernels
// compute them (source/clusterKernels.cu:803-811,382-390,823-834,836-844).  The logistic keeps the
// reference's mixed precision: `1.0f / (1.0 + expf(-x))` adds and divides in double.
__device__ __forceinline__ float cn_apply_activation(float x, int act)
{
    switch (act) {
        case CN_ACT_RELU: return x > 0.0f ? x : 0.0f;
        case CN_ACT_LOGISTIC: return (float)(1.0f / (1.0 + expf(-x)));
        case CN_ACT_DOUBLE_RELU: { float v = x > 0.0f ? x : 0.0f; return v < 1.0f ? v : 1.0f; }
        default: return x;
    }
}
