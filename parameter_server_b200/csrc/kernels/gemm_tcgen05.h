// Host interface of the tcgen05 bf16 GEMM (see gemm_tcgen05.cu).
#pragma once
#include <cuda_bf16.h>

#include <cstdint>

namespace psb {

struct GemmOperand {
    const void* ptr = nullptr;  // bf16, row-major 2-D tensor
    int64_t ld = 0;             // leading dimension in elements (multiple of 8)
    bool mn_major = false;      // false: [M or N rows][K cols]; true: [K rows][M or N cols]
};

struct GemmEpilogue {
    __nv_bfloat16* out_bf16 = nullptr;  // either or both outputs
    float* out_f32 = nullptr;
    int64_t ldd = 0;                    // leading dimension of the output(s)
    const float* bias = nullptr;        // [N], added before the activation
    const __nv_bfloat16* bias_bf16 = nullptr;  // same, stored as bf16 (parameters of a dense table)
    int relu = 0;
    const __nv_bfloat16* mask = nullptr;  // [M][N]: result is zeroed where mask <= 0 (ReLU backward)
    int64_t ldmask = 0;
    int accumulate = 0;                 // fp32 output: add to what is there
    int split_k = 1;                    // >1: K is split over gridDim.z and partial sums are added with
                                        // red.global.add.f32 into a zero-initialised fp32 output
};

// D = epilogue(A * B^T-style contraction over K). err_flag: device word, set non-zero when a bounded wait
// inside the kernel ran out. Returns 0, a cudaError_t, -2 (alignment) or -3 (tensor map).
int gemm_bf16(const GemmOperand& A, const GemmOperand& B, const GemmEpilogue& ep, int M, int N, int K, unsigned* err_flag,
              double wait_limit_s, void* stream);

}  // namespace psb
