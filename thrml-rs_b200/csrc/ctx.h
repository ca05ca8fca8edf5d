// Device context shared by the translation units of the library, and the CUDA error-check macro.
#pragma once
#include <cuda_runtime.h>

#include <string>

#include "tables.h"

struct thrml_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    int sm_count = 148;
};

#define CU_TRY(expr)                                                                                                      \
    do {                                                                                                                  \
        cudaError_t e__ = (expr);                                                                                         \
        if (e__ != cudaSuccess) return thrml::fail(THRML_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(e__)); \
    } while (0)
