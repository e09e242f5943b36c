// Host interface of the non-GEMM model kernels (see model_kernels.cu). All pointers are device
// pointers; bf16 tensors are passed as void*. Return value: 0, a cudaError_t, or -2 (unsupported shape).
#pragma once
#include <cstdint>

namespace pybind11 { class module_; }

namespace psb {

// emb: fp32 [B][F][D], or bf16 when emb_bf16 != 0
int interaction_fwd(const void* bottom, int64_t ldb, const void* emb, int emb_bf16, int F, int D, void* out, int64_t ldo,
                    int B, void* stream);
int interaction_bwd(const void* dout, int64_t ldo, const void* bottom, int64_t ldb, const void* emb, int emb_bf16, int F,
                    int D, void* dbottom, int64_t lddb, float* demb, int B, int relu_mask, void* stream);
int bce_head(const void* h, int64_t ldh, const void* w, const void* bias, const float* y, int B, int K, float inv_batch,
             float* loss_sum, float* logits, void* dz_prev, int64_t lddz, float* dw, float* db, void* stream);
int bias_grad(const void* dz, int64_t ld, int M, int N, float* db, void* stream);
// db_i[n] += sum_m dz_i[m][n] for up to 8 tensors with the same number of rows M, in one launch.
struct BiasGradSet {
    const void* dz[8];
    int64_t ld[8];
    int N[8];
    float* db[8];
    int group_end[8];  // filled by bias_grad_multi
    int count = 0;
    int M = 0;
};
int bias_grad_multi(BiasGradSet set, void* stream);
int cast_pad(const float* x, int B, int Kin, void* out, int64_t ldo, void* stream);
int timestamp(unsigned long long* slot, void* stream);

}  // namespace psb

void bind_model_kernels(pybind11::module_& m);
