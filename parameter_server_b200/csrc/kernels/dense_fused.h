// Argument block of the fused dense push (reduce-scatter + optimizer + all-gather) kernel.
#pragma once
#include <cuda_bf16.h>

#include "common.cuh"
#include "optim.cuh"

namespace psb {

struct DenseArgs {
    int world;
    int rank;
    unsigned long long limit_ns;
    const void* peer_grads[kMaxWorld];       // every rank's full gradient buffer
    __nv_bfloat16* peer_params[kMaxWorld];   // every rank's full bf16 parameter buffer
    unsigned* peer_flags[kMaxWorld];         // every rank's flag block: [0..8) ready, [8..16) done
    float* master;                           // fp32 master weights of this rank's slice
    float* slot0;                            // optimizer moments of the slice
    float* slot1;
    int n_slots;
    size_t shard_lo;                         // first element of this rank's slice
    size_t shard_len;                        // elements in the slice (multiple of 8)
    float grad_scale;                        // e.g. 1/world for a mean over data-parallel ranks
    int scatter_peers;                       // 1: store the new bf16 values into every rank's buffer (all-gather);
                                             // 0: only into this rank's own buffer (the consumer gathers lazily)
    OptConfig opt;
    KernelCtl* ctl;
};

// wide: 1024-thread CTAs (one per SM, nblocks = SMs used) instead of 256-thread ones
int launch_dense_rs_opt_ag(const DenseArgs& a, int grad_is_bf16, int nblocks, bool wide, void* stream);

}  // namespace psb
