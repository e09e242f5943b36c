// Symmetric peer memory: every rank allocates a buffer of the same size, exports a CUDA IPC handle,
// and maps every peer's buffer, so that a kernel on any GPU can ld/st/red any peer's HBM over
// NVLink 5 / NVSwitch.
//
// Parity: this is the data-plane transport that replaces prpc's c2s/s2s dealer sockets and the
// RPC-registered zero-copy memory (RpcVector / PSAllocator, pico-ps/common/message.h:238-276): a
// "request" is a peer store into the owner's mailbox plus a release flag, a "response" is a peer
// store back into the requester's buffer.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "../common/status.h"

namespace psb {

class SymmetricBuffer {
public:
    SymmetricBuffer(int device, size_t bytes);
    ~SymmetricBuffer();
    SymmetricBuffer(const SymmetricBuffer&) = delete;
    SymmetricBuffer& operator=(const SymmetricBuffer&) = delete;

    // 64-byte CUDA IPC handle of the local buffer (exchange through any host channel).
    std::string ipc_handle() const;
    // Map the peers. handles[r] is rank r's ipc_handle(); handles[rank] is ignored.
    Status connect(const std::vector<std::string>& handles, int rank);
    // Single-process use (world == 1 or several buffers of one process): peers given as raw pointers.
    void connect_local(const std::vector<void*>& ptrs, int rank);

    void* local() const { return local_; }
    void* peer(int r) const { return peers_.at(r); }
    int world() const { return (int)peers_.size(); }
    size_t bytes() const { return bytes_; }
    int device() const { return device_; }

private:
    int device_;
    size_t bytes_;
    void* local_ = nullptr;
    int rank_ = 0;
    std::vector<void*> peers_;
    std::vector<bool> opened_;
};

}  // namespace psb
