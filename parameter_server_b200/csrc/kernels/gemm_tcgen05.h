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

// All-gather fused into the GEMM (dense pull fused with its first consumer): operand B ([N][K], K-major,
// contiguous rows) is sharded by rows over `world` ranks, rank r holding the current values of rows
// [r*rows_per_rank, (r+1)*rows_per_rank) in ITS copy of the tensor. `gather_ctas` CTAs of the launch pull the
// remote row blocks over NVLink into this GPU's copy (bulk copies global -> shared -> global, no multicast)
// and publish one flag per n-tile; the GEMM CTAs start with the tiles of the local rows and wait (bounded) for
// the flag of a remote n-tile right before their TMA loads of it, so the transfer overlaps the math.
struct GemmGather {
    int enabled = 0;
    int world = 1, rank = 0;
    const __nv_bfloat16* peer_b[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    __nv_bfloat16* local_b = nullptr;
    int rows_per_rank = 0;     // multiple of the n-tile height (256)
    unsigned* ready = nullptr; // [N / 256] in local memory; n-tile j has landed when ready[j] >= epoch
    unsigned epoch = 0;
    int gather_ctas = 8;
};

// D = epilogue(A * B^T-style contraction over K). err_flag: device word, set non-zero when a bounded wait
// inside the kernel ran out. Returns 0, a cudaError_t, -2 (alignment) or -3 (tensor map).
int gemm_bf16(const GemmOperand& A, const GemmOperand& B, const GemmEpilogue& ep, int M, int N, int K, unsigned* err_flag,
              double wait_limit_s, void* stream, const GemmGather* gather = nullptr);

// Up to 8 independent GEMMs in ONE persistent launch (same operand majors for all; 128 x 256 tiles when every
// N >= 256, else 128 x 128). Meant for work that becomes available together, e.g. the weight gradients of all
// layers of an MLP at the end of the backward pass. Same return codes as gemm_bf16.
//
// With `chain_done` (device scratch of gemm_chain_scratch_words() unsigned, zeroed by the call) the problems form a
// CHAIN: problem i + 1 takes the bf16 output of problem i as its A operand (the layers of an MLP in the forward
// pass, or the dgrad sequence of the backward pass). All layers then run in this one launch: the work units are
// ordered row block by row block, the epilogue counts the stored tiles of every row block, and the TMA producer
// of the next layer waits (bounded) for the row block it is about to load, so the tail of one layer overlaps the
// head of the next instead of paying a kernel boundary per layer. Every problem must have the same M and a
// K-major A; split_k is not allowed.
int gemm_bf16_grouped(const GemmOperand* A, const GemmOperand* B, const GemmEpilogue* ep, const int* M, const int* N,
                      const int* K, int count, unsigned* err_flag, double wait_limit_s, void* stream,
                      unsigned* chain_done = nullptr);
int gemm_chain_scratch_words();
// Upper bound on the CTAs (= SMs) of the following launches; 0 = all SMs. A GEMM CTA fills its SM, so a smaller grid
// leaves whole SMs to kernels of another stream that run at the same time (the sparse push beside the dense backward).
void gemm_set_cta_limit(int ctas);
// CTA pairs (two CTAs of a cluster per 256-row tile) on or off for the following launches. A pair needs two free SMs
// of one TPC at the same moment; launches that share the GPU with another kernel run better without.
void gemm_set_pair(int on);
// Tracing of the following launches (nullptr = off): CTA 0 writes %globaltimer stamps for the first 8 work units it runs
// into this device buffer of 256 x u64, 32 slots per unit (producer, MMA and epilogue milestones; unit index in slot 7). The tool behind the per-tile timelines in profiles/.
void gemm_set_trace(void* device_buffer_of_256_u64);

}  // namespace psb
