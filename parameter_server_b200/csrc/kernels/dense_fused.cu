// Dense push for sm_100a: reduce-scatter of the ranks' gradient buffers fused with the partitioned
// optimizer step on the fp32 master shard and with the all-gather of the updated bf16 parameters,
// all in ONE kernel over NVLink peer memory.
//
// Parity: DenseTablePushOperator splits a dense value into slices, each owned by one shard, and the
// owner applies the update rule per slice (pico-ps/operator/DensePushOperator.h:76-84, :171-193);
// DenseTablePullOperator reassembles the slices on the worker (pico-ps/operator/DensePullOperator.h:
// 153-169, :197-216). Here slice r is the r-th contiguous 1/world of the flat parameter buffer:
//   1. every rank announces "my gradients are complete" with a release flag on every peer;
//   2. rank r sums slice r of every peer's gradient buffer with vector peer loads (a warp reads one contiguous span), in rank order
//      (bitwise reproducible), scales, and runs SGD / Adam(W) on its fp32 master + moments;
//   3. it stores the new bf16 values of slice r into EVERY rank's parameter buffer (peer stores),
//      which is the all-gather of the next dense pull;
//   4. a second flag round tells every rank that all slices of its parameter buffer have landed and
//      that its gradient buffer may be overwritten.
// All waits are bounded; world == 1 runs the optimizer only.
#include <cuda_bf16.h>

#include "dense_fused.h"

namespace psb {

namespace {

constexpr int kThreadsSmall = 256;   // four CTAs per SM
constexpr int kThreadsWide = 1024;   // one CTA fills an SM: the shape for sharing the GPU by SMs with another kernel

template <typename GT>
struct Vec4;  // four gradient elements; a warp's loads cover one contiguous 512-byte (fp32) / 256-byte (bf16) span
template <>
struct Vec4<float> {
    float4 a;
    __device__ __forceinline__ void load(const float* p) { a = *(const float4*)p; }
    __device__ __forceinline__ void to_float(float* f) const { f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; }
};
template <>
struct Vec4<__nv_bfloat16> {
    uint2 raw;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { raw = *(const uint2*)p; }
    __device__ __forceinline__ void to_float(float* f) const {
        const __nv_bfloat162* h = (const __nv_bfloat162*)&raw;
        float2 t0 = __bfloat1622float2(h[0]), t1 = __bfloat1622float2(h[1]);
        f[0] = t0.x; f[1] = t0.y; f[2] = t1.x; f[3] = t1.y;
    }
};

template <typename GT, int kThreads>
__global__ void __launch_bounds__(kThreads, 1024 / kThreads) dense_rs_opt_ag_kernel(const DenseArgs a) {
    const int me = a.rank;
    const unsigned epoch = *((volatile unsigned*)&a.ctl->epoch) + 1u;
    const int W = a.world;
    OptConfig opt = a.opt;
    if (opt.step_from_epoch) opt_set_step(opt, epoch);
    // ---- 1. announce + wait: gradients of every rank are complete --------------------------------
    if (W > 1) {
        if (blockIdx.x == 0 && threadIdx.x < (unsigned)W && (int)threadIdx.x != me) {
            __threadfence_system();
            st_release_sys(a.peer_flags[threadIdx.x] + me, epoch);
        }
        int ok = 1;
        if (threadIdx.x < (unsigned)W && (int)threadIdx.x != me) {
            if (!wait_flag_ge(a.peer_flags[me] + threadIdx.x, epoch, a.limit_ns)) {
                set_status(a.ctl, kStTimeout, 1);
                ok = 0;
            }
        }
        if (!__syncthreads_and(ok)) return;
    }
    // ---- 2+3. reduce, update, scatter bf16 ------------------------------------------------------------
    const size_t n4 = a.shard_len / 4;
    // peer pointers are read from the kernel parameters (constant bank) where they are used: keeping
    // sixteen of them in registers would cost a third of the register budget
#pragma unroll 1
    for (size_t c = blockIdx.x * (size_t)kThreads + threadIdx.x; c < n4; c += (size_t)gridDim.x * kThreads) {
        const size_t i = c * 4;
        float g[4];
        {
            Vec4<GT> v;
            v.load((const GT*)a.peer_grads[0] + a.shard_lo + i);
            v.to_float(g);
        }
#pragma unroll
        for (int r = 1; r < kMaxWorld; ++r) {
            if (r < W) {
                Vec4<GT> v;
                v.load((const GT*)a.peer_grads[r] + a.shard_lo + i);
                float t[4];
                v.to_float(t);
#pragma unroll
                for (int k = 0; k < 4; ++k) g[k] += t[k];
            }
        }
        __align__(16) float w[4], m[4], s[4];
        *(float4*)w = *(const float4*)(a.master + i);
        if (a.n_slots > 0) *(float4*)m = *(const float4*)(a.slot0 + i);
        if (a.n_slots > 1) *(float4*)s = *(const float4*)(a.slot1 + i);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float s0 = a.n_slots > 0 ? m[k] : 0.f, s1 = a.n_slots > 1 ? s[k] : 0.f;
            opt_update(opt, w[k], s0, s1, g[k] * a.grad_scale);
            m[k] = s0;
            s[k] = s1;
        }
        *(float4*)(a.master + i) = *(float4*)w;
        if (a.n_slots > 0) *(float4*)(a.slot0 + i) = *(float4*)m;
        if (a.n_slots > 1) *(float4*)(a.slot1 + i) = *(float4*)s;
        uint2 packed;
        __nv_bfloat162* h = (__nv_bfloat162*)&packed;
        h[0] = __floats2bfloat162_rn(w[0], w[1]);
        h[1] = __floats2bfloat162_rn(w[2], w[3]);
#pragma unroll
        for (int r = 0; r < kMaxWorld; ++r)
            if (r < W && (a.scatter_peers || r == me)) *(uint2*)(a.peer_params[r] + a.shard_lo + i) = packed;
    }
    // ---- 4. all slices landed everywhere ----------------------------------------------------------
    if (W == 1) {
        // single rank: the epoch is only the step counter; the last CTA out publishes it
        __syncthreads();
        if (threadIdx.x == 0 && atomicAdd(&a.ctl->done_blocks, 1u) == gridDim.x - 1u) {
            a.ctl->done_blocks = 0;
            a.ctl->epoch = epoch;
        }
    }
    if (W > 1) {
        __threadfence_system();
        __syncthreads();
        __shared__ unsigned s_last;
        if (threadIdx.x == 0) s_last = (atomicAdd(&a.ctl->done_blocks, 1u) == gridDim.x - 1u);
        __syncthreads();
        if (s_last) {
            // every CTA has read the epoch by now (it counted itself done after reading it)
            if (threadIdx.x == 0) {
                a.ctl->done_blocks = 0;
                a.ctl->epoch = epoch;
            }
            if (threadIdx.x < (unsigned)W && (int)threadIdx.x != me) {
                st_release_sys(a.peer_flags[threadIdx.x] + kMaxWorld + me, epoch);
                if (!wait_flag_ge(a.peer_flags[me] + kMaxWorld + threadIdx.x, epoch, a.limit_ns))
                    set_status(a.ctl, kStTimeout, 2);
            }
        }
    }
}

}  // namespace

int launch_dense_rs_opt_ag(const DenseArgs& a, int grad_is_bf16, int nblocks, bool wide, void* stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (wide) {
        if (grad_is_bf16) dense_rs_opt_ag_kernel<__nv_bfloat16, kThreadsWide><<<nblocks, kThreadsWide, 0, s>>>(a);
        else dense_rs_opt_ag_kernel<float, kThreadsWide><<<nblocks, kThreadsWide, 0, s>>>(a);
    } else {
        if (grad_is_bf16) dense_rs_opt_ag_kernel<__nv_bfloat16, kThreadsSmall><<<nblocks, kThreadsSmall, 0, s>>>(a);
        else dense_rs_opt_ag_kernel<float, kThreadsSmall><<<nblocks, kThreadsSmall, 0, s>>>(a);
    }
    return (int)cudaGetLastError();
}

}  // namespace psb
