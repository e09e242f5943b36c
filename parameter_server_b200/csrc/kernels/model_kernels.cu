// Model-side kernels of the DLRM workload that are not GEMMs: feature interaction (pairwise dots),
// the 1-wide output layer fused with sigmoid + binary cross-entropy (forward and backward in one
// pass), bias gradients and the dense-feature cast. Not in the reference (it ships no model code);
// they exist so that a full CTR training step runs on hand-written sm_100a kernels.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "model_kernels.h"

namespace psb {

namespace {

constexpr int kMaxT = 32;  // interaction vectors per sample (fields + 1)

// ---- interaction forward -----------------------------------------------------------------------
// T[0] = bottom (bf16), T[1..F] = emb (fp32). out[b] = [bottom (D) | dot(T_i, T_j) for i > j | 0 pad].
template <int D>
__global__ void __launch_bounds__(128) interaction_fwd_kernel(const __nv_bfloat16* __restrict__ bottom, int64_t ldb,
                                                              const float* __restrict__ emb, int F,
                                                              __nv_bfloat16* __restrict__ out, int64_t ldo, int B) {
    __shared__ float T[kMaxT][D + 1];
    const int nT = F + 1;
    const int npairs = nT * (nT - 1) / 2;
    for (int b = blockIdx.x; b < B; b += gridDim.x) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < nT * D; idx += 128) {
            const int i = idx / D, d = idx % D;
            T[i][d] = (i == 0) ? __bfloat162float(bottom[(size_t)b * ldb + d]) : emb[((size_t)b * F + (i - 1)) * D + d];
        }
        __syncthreads();
        __nv_bfloat16* o = out + (size_t)b * ldo;
        for (int d = threadIdx.x; d < D; d += 128) o[d] = __float2bfloat16_rn(T[0][d]);
        for (int p = threadIdx.x; p < npairs; p += 128) {
            int i = (int)((1.0f + sqrtf(1.0f + 8.0f * (float)p)) * 0.5f);
            while (i * (i - 1) / 2 > p) --i;
            while ((i + 1) * i / 2 <= p) ++i;
            const int j = p - i * (i - 1) / 2;
            float acc = 0.f;
#pragma unroll 8
            for (int d = 0; d < D; ++d) acc = fmaf(T[i][d], T[j][d], acc);
            o[D + p] = __float2bfloat16_rn(acc);
        }
        for (int c = D + npairs + threadIdx.x; c < ldo; c += 128) o[c] = __float2bfloat16_rn(0.f);
    }
}

// ---- interaction backward ----------------------------------------------------------------------
// dT_i = sum_{j != i} G[i][j] T_j with G the symmetric matrix of pair gradients.
// d_bottom (bf16) = (dout[:, :D] + dT_0) masked by (bottom > 0) when relu_mask; d_emb (fp32) = dT_{1..F}.
template <int D>
__global__ void __launch_bounds__(D) interaction_bwd_kernel(const __nv_bfloat16* __restrict__ dout, int64_t ldo,
                                                            const __nv_bfloat16* __restrict__ bottom, int64_t ldb,
                                                            const float* __restrict__ emb, int F,
                                                            __nv_bfloat16* __restrict__ dbottom, int64_t lddb,
                                                            float* __restrict__ demb, int B, int relu_mask) {
    __shared__ float T[kMaxT][D + 1];
    __shared__ float G[kMaxT][kMaxT + 1];
    const int nT = F + 1;
    const int npairs = nT * (nT - 1) / 2;
    for (int b = blockIdx.x; b < B; b += gridDim.x) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < nT * D; idx += D) {
            const int i = idx / D, d = idx % D;
            T[i][d] = (i == 0) ? __bfloat162float(bottom[(size_t)b * ldb + d]) : emb[((size_t)b * F + (i - 1)) * D + d];
        }
        const __nv_bfloat16* go = dout + (size_t)b * ldo;
        for (int p = threadIdx.x; p < npairs; p += D) {
            int i = (int)((1.0f + sqrtf(1.0f + 8.0f * (float)p)) * 0.5f);
            while (i * (i - 1) / 2 > p) --i;
            while ((i + 1) * i / 2 <= p) ++i;
            const int j = p - i * (i - 1) / 2;
            const float g = __bfloat162float(go[D + p]);
            G[i][j] = g;
            G[j][i] = g;
        }
        if (threadIdx.x < nT) G[threadIdx.x][threadIdx.x] = 0.f;
        __syncthreads();
        const int d = threadIdx.x;
        for (int i = 0; i < nT; ++i) {
            float acc = 0.f;
            for (int j = 0; j < nT; ++j) acc = fmaf(G[i][j], T[j][d], acc);
            if (i == 0) {
                float v = acc + __bfloat162float(go[d]);
                if (relu_mask && !(T[0][d] > 0.f)) v = 0.f;
                dbottom[(size_t)b * lddb + d] = __float2bfloat16_rn(v);
            } else {
                demb[((size_t)b * F + (i - 1)) * D + d] = acc;
            }
        }
    }
}

// ---- output layer + sigmoid + BCE, forward and backward ------------------------------------------
// h: bf16 [B][K] (ReLU output of the last hidden layer), w: bf16 [K], bias fp32 [1], y: fp32 [B].
// loss_sum += sum_b bce(z_b, y_b) * inv_batch;  dz_prev[b][k] = dlogit_b * w[k] * (h > 0);
// dw[k] += sum_b dlogit_b * h[b][k];  db += sum_b dlogit_b, with dlogit_b = (sigmoid(z_b) - y_b) * inv_batch.
__global__ void __launch_bounds__(256) bce_head_kernel(const __nv_bfloat16* __restrict__ h, int64_t ldh,
                                                       const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ bias,
                                                       const float* __restrict__ y, int B, int K, float inv_batch,
                                                       float* __restrict__ loss_sum, float* __restrict__ logits,
                                                       __nv_bfloat16* __restrict__ dz_prev, int64_t lddz,
                                                       float* __restrict__ dw, float* __restrict__ db) {
    extern __shared__ float s_dw[];  // [K] per-CTA partial of dw
    __shared__ float s_loss, s_db;
    for (int k = threadIdx.x; k < K; k += blockDim.x) s_dw[k] = 0.f;
    if (threadIdx.x == 0) { s_loss = 0.f; s_db = 0.f; }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const float b0 = bias ? __bfloat162float(bias[0]) : 0.f;
    for (int b = blockIdx.x * nwarps + warp; b < B; b += gridDim.x * nwarps) {
        const __nv_bfloat16* hr = h + (size_t)b * ldh;
        float acc = 0.f;
        for (int k = lane; k < K; k += 32) acc = fmaf(__bfloat162float(hr[k]), __bfloat162float(w[k]), acc);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        const float z = acc + b0;
        const float yy = y[b];
        const float p = 1.f / (1.f + __expf(-z));
        const float loss = fmaxf(z, 0.f) - z * yy + log1pf(__expf(-fabsf(z)));
        const float dl = (p - yy) * inv_batch;
        if (lane == 0) {
            atomicAdd(&s_loss, loss * inv_batch);
            atomicAdd(&s_db, dl);
            if (logits) logits[b] = z;
        }
        if (dz_prev != nullptr) {
            __nv_bfloat16* dr = dz_prev + (size_t)b * lddz;
            for (int k = lane; k < K; k += 32) {
                const float hv = __bfloat162float(hr[k]);
                dr[k] = __float2bfloat16_rn(hv > 0.f ? dl * __bfloat162float(w[k]) : 0.f);
                atomicAdd(&s_dw[k], dl * hv);
            }
        }
    }
    __syncthreads();
    if (dw != nullptr)
        for (int k = threadIdx.x; k < K; k += blockDim.x) atomicAdd(&dw[k], s_dw[k]);
    if (threadIdx.x == 0) {
        atomicAdd(loss_sum, s_loss);
        if (db != nullptr) atomicAdd(db, s_db);
    }
}

// ---- bias gradient: db[n] = sum_m dz[m][n] -------------------------------------------------------------
__global__ void __launch_bounds__(256) bias_grad_kernel(const __nv_bfloat16* __restrict__ dz, int64_t ld, int M, int N,
                                                        float* __restrict__ db) {
    // CTA handles 32 columns x a stripe of rows; threads (tx: column, ty: row lane)
    __shared__ float part[8][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int col = blockIdx.x * 32 + tx;
    float acc = 0.f;
    if (col < N)
        for (int m = blockIdx.y * 8 + ty; m < M; m += gridDim.y * 8) acc += __bfloat162float(dz[(size_t)m * ld + col]);
    part[ty][tx] = acc;
    __syncthreads();
    if (ty == 0 && col < N) {
        float s = 0.f;
#pragma unroll
        for (int r = 0; r < 8; ++r) s += part[r][tx];
        atomicAdd(&db[col], s);
    }
}

__global__ void cast_pad_kernel(const float* __restrict__ x, int B, int Kin, __nv_bfloat16* __restrict__ out, int64_t ldo) {
    const size_t total = (size_t)B * ldo;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t b = i / ldo;
        const int k = (int)(i % ldo);
        out[i] = __float2bfloat16_rn(k < Kin ? x[b * Kin + k] : 0.f);
    }
}

}  // namespace

int interaction_fwd(const void* bottom, int64_t ldb, const float* emb, int F, int D, void* out, int64_t ldo, int B,
                    void* stream) {
    if (D != 128 && D != 64) return -2;
    if (F + 1 > kMaxT) return -2;
    const int grid = B < 148 * 16 ? B : 148 * 16;
    if (D == 128)
        interaction_fwd_kernel<128><<<grid, 128, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)bottom, ldb, emb, F,
                                                                            (__nv_bfloat16*)out, ldo, B);
    else
        interaction_fwd_kernel<64><<<grid, 128, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)bottom, ldb, emb, F,
                                                                           (__nv_bfloat16*)out, ldo, B);
    return (int)cudaGetLastError();
}

int interaction_bwd(const void* dout, int64_t ldo, const void* bottom, int64_t ldb, const float* emb, int F, int D,
                    void* dbottom, int64_t lddb, float* demb, int B, int relu_mask, void* stream) {
    if (D != 128 && D != 64) return -2;
    if (F + 1 > kMaxT) return -2;
    const int grid = B < 148 * 16 ? B : 148 * 16;
    if (D == 128)
        interaction_bwd_kernel<128><<<grid, 128, 0, (cudaStream_t)stream>>>(
            (const __nv_bfloat16*)dout, ldo, (const __nv_bfloat16*)bottom, ldb, emb, F, (__nv_bfloat16*)dbottom, lddb, demb,
            B, relu_mask);
    else
        interaction_bwd_kernel<64><<<grid, 64, 0, (cudaStream_t)stream>>>(
            (const __nv_bfloat16*)dout, ldo, (const __nv_bfloat16*)bottom, ldb, emb, F, (__nv_bfloat16*)dbottom, lddb, demb,
            B, relu_mask);
    return (int)cudaGetLastError();
}

int bce_head(const void* h, int64_t ldh, const void* w, const void* bias, const float* y, int B, int K, float inv_batch,
             float* loss_sum, float* logits, void* dz_prev, int64_t lddz, float* dw, float* db, void* stream) {
    const int grid = 148 * 2;
    bce_head_kernel<<<grid, 256, K * sizeof(float), (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)h, ldh, (const __nv_bfloat16*)w, (const __nv_bfloat16*)bias, y, B, K, inv_batch, loss_sum, logits,
        (__nv_bfloat16*)dz_prev, lddz, dw, db);
    return (int)cudaGetLastError();
}

int bias_grad(const void* dz, int64_t ld, int M, int N, float* db, void* stream) {
    dim3 grid((N + 31) / 32, 64);
    bias_grad_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)dz, ld, M, N, db);
    return (int)cudaGetLastError();
}

int cast_pad(const float* x, int B, int Kin, void* out, int64_t ldo, void* stream) {
    cast_pad_kernel<<<148 * 4, 256, 0, (cudaStream_t)stream>>>(x, B, Kin, (__nv_bfloat16*)out, ldo);
    return (int)cudaGetLastError();
}

}  // namespace psb
