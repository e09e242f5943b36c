#include "symmetric.h"

#include <cuda_runtime.h>

#include <cstring>
#include <stdexcept>

namespace psb {

SymmetricBuffer::SymmetricBuffer(int device, size_t bytes) : device_(device), bytes_(bytes) {
    cudaSetDevice(device_);
    cudaError_t e = cudaMalloc(&local_, bytes_);
    if (e != cudaSuccess)
        throw std::runtime_error(std::string("SymmetricBuffer: cudaMalloc: ") + cudaGetErrorString(e));
    e = cudaMemset(local_, 0, bytes_);
    if (e != cudaSuccess)
        throw std::runtime_error(std::string("SymmetricBuffer: cudaMemset: ") + cudaGetErrorString(e));
    cudaDeviceSynchronize();
    peers_.assign(1, local_);
    opened_.assign(1, false);
}

SymmetricBuffer::~SymmetricBuffer() {
    cudaSetDevice(device_);
    for (size_t r = 0; r < peers_.size(); ++r)
        if (opened_[r] && peers_[r] != nullptr) cudaIpcCloseMemHandle(peers_[r]);
    if (local_) cudaFree(local_);
}

std::string SymmetricBuffer::ipc_handle() const {
    cudaSetDevice(device_);
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, local_);
    if (e != cudaSuccess)
        throw std::runtime_error(std::string("SymmetricBuffer: cudaIpcGetMemHandle: ") + cudaGetErrorString(e));
    return std::string((const char*)&h, sizeof(h));
}

Status SymmetricBuffer::connect(const std::vector<std::string>& handles, int rank) {
    cudaSetDevice(device_);
    rank_ = rank;
    peers_.assign(handles.size(), nullptr);
    opened_.assign(handles.size(), false);
    for (size_t r = 0; r < handles.size(); ++r) {
        if ((int)r == rank) {
            peers_[r] = local_;
            continue;
        }
        if (handles[r].size() != sizeof(cudaIpcMemHandle_t)) return Status::InvalidConfig("bad IPC handle size");
        cudaIpcMemHandle_t h;
        std::memcpy(&h, handles[r].data(), sizeof(h));
        void* p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return Status::Error(std::string("cudaIpcOpenMemHandle(rank ") + std::to_string(r) + "): " +
                                 cudaGetErrorString(e));
        }
        peers_[r] = p;
        opened_[r] = true;
    }
    return Status::Ok();
}

void SymmetricBuffer::connect_local(const std::vector<void*>& ptrs, int rank) {
    rank_ = rank;
    peers_ = ptrs;
    peers_[rank] = local_;
    opened_.assign(ptrs.size(), false);
}

}  // namespace psb
