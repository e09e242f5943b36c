#include "dense_engine.h"

#include <cuda_runtime.h>

#include <stdexcept>

namespace psb {

namespace {
size_t align_up(size_t v, size_t a = 256) { return (v + a - 1) / a * a; }

__global__ void load_full_kernel(const float* full, size_t numel, size_t lo, size_t len, float* master,
                                 __nv_bfloat16* params) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < numel; i += stride) {
        const float v = full[i];
        params[i] = __float2bfloat16_rn(v);
        if (i >= lo && i < lo + len) master[i - lo] = v;
    }
}
}  // namespace

DenseEngine::DenseEngine(int device, int world, int rank, size_t numel, bool grad_bf16, int opt_type,
                         double wait_limit_s)
    : device_(device), world_(world), rank_(rank), grad_bf16_(grad_bf16), wait_limit_s_(wait_limit_s) {
    if (world < 1 || world > kMaxWorld) throw std::invalid_argument("DenseEngine: world must be 1..8");
    cudaSetDevice(device_);
    const size_t q = 8 * (size_t)world;
    numel_ = (numel + q - 1) / q * q;
    shard_len_ = numel_ / world;
    n_slots_ = opt_num_slots(opt_type);
    size_t off = 0;
    off_flags_ = off; off = align_up(off + 2 * kMaxWorld * sizeof(unsigned));
    off_params_ = off; off = align_up(off + numel_ * 2);
    off_grads_ = off; off = align_up(off + numel_ * (grad_bf16 ? 2 : 4));
    symm_.reset(new SymmetricBuffer(device_, off));
    auto alloc = [&](float** p) {
        if (cudaMalloc(p, shard_len_ * 4) != cudaSuccess) throw std::runtime_error("DenseEngine: cudaMalloc");
        cudaMemset(*p, 0, shard_len_ * 4);
    };
    alloc(&master_);
    if (n_slots_ > 0) alloc(&slot0_);
    if (n_slots_ > 1) alloc(&slot1_);
    if (cudaMalloc(&ctl_, sizeof(KernelCtl)) != cudaSuccess) throw std::runtime_error("DenseEngine: cudaMalloc");
    cudaMemset(ctl_, 0, sizeof(KernelCtl));
    cudaDeviceSynchronize();
    if (world == 1) symm_->connect_local(std::vector<void*>(1, symm_->local()), 0);
}

DenseEngine::~DenseEngine() {
    cudaSetDevice(device_);
    cudaDeviceSynchronize();
    cudaFree(master_);
    if (slot0_) cudaFree(slot0_);
    if (slot1_) cudaFree(slot1_);
    cudaFree(ctl_);
}

Status DenseEngine::connect(const std::vector<std::string>& handles) {
    if ((int)handles.size() != world_) return Status::InvalidConfig("connect: need one handle per rank");
    return symm_->connect(handles, rank_);
}

void DenseEngine::connect_local(const std::vector<DenseEngine*>& engines) {
    std::vector<void*> ptrs;
    for (auto* e : engines) ptrs.push_back(e->symm_->local());
    symm_->connect_local(ptrs, rank_);
}

Status DenseEngine::load_full(const float* full, void* stream) {
    cudaSetDevice(device_);
    load_full_kernel<<<148 * 4, 256, 0, (cudaStream_t)stream>>>(full, numel_, shard_lo(), shard_len_, master_,
                                                                (__nv_bfloat16*)params_ptr());
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return Status::Error(cudaGetErrorString(e));
    return Status::Ok();
}

Status DenseEngine::step(const OptConfig& opt, float grad_scale, void* stream) {
    cudaSetDevice(device_);
    if (symm_->world() != world_) return Status::Error("dense step: peers are not connected");
    DenseArgs a;
    a.world = world_;
    a.rank = rank_;
    ++epoch_;
    a.limit_ns = (unsigned long long)(wait_limit_s_ * 1e9);
    for (int r = 0; r < kMaxWorld; ++r) {
        if (r < world_) {
            char* base = (char*)symm_->peer(r);
            a.peer_grads[r] = base + off_grads_;
            a.peer_params[r] = (__nv_bfloat16*)(base + off_params_);
            a.peer_flags[r] = (unsigned*)(base + off_flags_);
        } else {
            a.peer_grads[r] = nullptr;
            a.peer_params[r] = nullptr;
            a.peer_flags[r] = nullptr;
        }
    }
    a.master = master_;
    a.slot0 = slot0_;
    a.slot1 = slot1_;
    a.n_slots = n_slots_;
    a.shard_lo = shard_lo();
    a.shard_len = shard_len_;
    a.grad_scale = grad_scale;
    a.scatter_peers = scatter_peers_ ? 1 : 0;
    a.opt = opt;
    a.ctl = ctl_;
    const size_t chunks = shard_len_ / 4;
    int nblocks = (int)std::min<size_t>(148 * 4, std::max<size_t>(1, (chunks + 255) / 256));  // 4 resident CTAs per SM, one wave
    const bool wide = sm_budget_ > 0;
    if (wide) nblocks = (int)std::min<size_t>((size_t)sm_budget_, std::max<size_t>(1, (chunks + 1023) / 1024));
    int rc = launch_dense_rs_opt_ag(a, grad_bf16_ ? 1 : 0, nblocks, wide, stream);
    ++launches_;
    if (rc != 0) return Status::Error(std::string("dense_rs_opt_ag launch: ") + cudaGetErrorString((cudaError_t)rc));
    return Status::Ok();
}

Status DenseEngine::reset(void* stream) {
    cudaSetDevice(device_);
    cudaStream_t s = (cudaStream_t)stream;
    cudaStreamSynchronize(s);
    cudaMemsetAsync(ctl_, 0, sizeof(KernelCtl), s);
    cudaMemsetAsync((char*)symm_->local() + off_flags_, 0, 2 * kMaxWorld * sizeof(unsigned), s);
    cudaError_t e = cudaStreamSynchronize(s);
    epoch_ = 0;
    if (e != cudaSuccess) return Status::Fatal(cudaGetErrorString(e));
    return Status::Ok();
}

Status DenseEngine::check(void* stream) {
    cudaSetDevice(device_);
    cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) return Status::Fatal(std::string("stream: ") + cudaGetErrorString(e));
    KernelCtl h;
    e = cudaMemcpy(&h, ctl_, sizeof(h), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return Status::Fatal(cudaGetErrorString(e));
    if (h.status == kStTimeout)
        return Status::Timeout(h.where == 1 ? "dense push: waiting for a peer's gradients"
                                            : "dense push: waiting for a peer's completion flag");
    if (h.status != 0) return Status::Error("dense push failed");
    return Status::Ok();
}

}  // namespace psb
