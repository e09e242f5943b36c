// DenseEngine: one dense table (a flat parameter buffer holding any number of tensors) sharded by
// contiguous slices over the ranks, with its gradient and bf16 parameter buffers in symmetric peer
// memory. The B200 counterpart of DenseTablePush/PullOperator + Push/PullHandler for dense keys
// (pico-ps/operator/DensePushOperator.h:59-126, pico-ps/operator/DensePullOperator.h:49-116).
#pragma once
#include <memory>
#include <string>
#include <vector>

#include "../comm/symmetric.h"
#include "../kernels/dense_fused.h"

namespace psb {

class DenseEngine {
public:
    // numel is rounded up to a multiple of 8*world; grads are bf16 or fp32.
    DenseEngine(int device, int world, int rank, size_t numel, bool grad_bf16, int opt_type, double wait_limit_s);
    ~DenseEngine();

    std::string ipc_handle() const { return symm_->ipc_handle(); }
    Status connect(const std::vector<std::string>& handles);
    void connect_local(const std::vector<DenseEngine*>& engines);

    size_t numel() const { return numel_; }
    size_t shard_lo() const { return shard_len_ * rank_; }
    size_t shard_len() const { return shard_len_; }
    void* params_ptr() const { return (char*)symm_->local() + off_params_; }  // bf16[numel]
    void* grads_ptr() const { return (char*)symm_->local() + off_grads_; }    // GT[numel]
    void* peer_params_ptr(int r) const { return (char*)symm_->peer(r) + off_params_; }
    float* master_ptr() const { return master_; }
    float* slot_ptr(int s) const { return s == 0 ? slot0_ : slot1_; }
    bool grad_bf16() const { return grad_bf16_; }

    // Initialise from a full fp32 device vector (same values on every rank): master slice + local bf16 copy.
    Status load_full(const float* full, void* stream);
    // Collective: reduce-scatter + optimizer + all-gather.
    Status step(const OptConfig& opt, float grad_scale, void* stream);
    Status check(void* stream);
    // Re-arm after a time-out: clears the status word, the call epoch and the flags on THIS rank (every rank must).
    Status reset(void* stream);
    uint64_t kernel_launches() const { return launches_; }
    // false: dense push leaves the other ranks' copies of this table stale; they are gathered by the
    // consuming kernel (all-gather fused with the first GEMM).
    void set_scatter_peers(bool on) { scatter_peers_ = on; }
    // n > 0: the push runs as 1024-thread CTAs (each fills an SM) on at most n SMs and leaves the others, whole, to a
    // kernel of another stream (the sparse push of the same step); 0 = the whole GPU.
    void set_sm_budget(int sms) { sm_budget_ = sms > 0 ? sms : 0; }
    int world() const { return world_; }
    int rank() const { return rank_; }

private:
    int device_, world_, rank_;
    size_t numel_, shard_len_;
    bool grad_bf16_;
    int n_slots_;
    double wait_limit_s_;
    std::unique_ptr<SymmetricBuffer> symm_;
    size_t off_flags_ = 0, off_params_ = 0, off_grads_ = 0;
    float *master_ = nullptr, *slot0_ = nullptr, *slot1_ = nullptr;
    KernelCtl* ctl_ = nullptr;
    unsigned epoch_ = 0;
    uint64_t launches_ = 0;
    bool scatter_peers_ = true;
    int sm_budget_ = 0;
};

}  // namespace psb
