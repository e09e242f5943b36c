// The allocation-free variant of dedup_partition (contract in dedup_noalloc.h). Its scratch is the
// file-scope device arrays below. In host code the NAME of such an array is only a handle for the
// CUDA runtime, not an address a kernel may be given, so the device address is looked up once per
// device with cudaGetSymbolAddress (with that device current) and that pointer is what the kernels get.
#include "dedup_noalloc.h"

#include <mutex>

#include "dedup.h"

namespace psb {
namespace {

constexpr unsigned long long kNoAllocSlots = 2ull * PSB_DEDUP_NOALLOC_MAX_KEYS;  // power of two, >= 2n
constexpr int kMaxDevices = 64;

static __device__ __align__(256) Slot g_dedup_slots[kNoAllocSlots];
static __device__ __align__(256) unsigned g_dedup_pos[PSB_DEDUP_NOALLOC_MAX_KEYS];

struct PerDevice {
    bool ready = false;
    Slot* slots = nullptr;
    unsigned* pos = nullptr;
};
PerDevice g_per_device[kMaxDevices];
std::mutex g_setup_mutex;  // host threads making the first call on a device take turns at the set-up

}  // namespace
}  // namespace psb

extern "C" __attribute__((visibility("default"))) int psb_dedup_partition_noalloc(
    const long long* keys, unsigned n, const int* shard_owner, int n_shards, int world, long long* uniq_keys, int* uniq_owner,
    int* inverse, unsigned* counts, void* stream) {
    using namespace psb;
    if (n > PSB_DEDUP_NOALLOC_MAX_KEYS) return PSB_DEDUP_ERR_TOO_LARGE;
    if (world < 1 || world > kMaxWorld || (shard_owner != nullptr && n_shards < 1)) return PSB_DEDUP_ERR_BAD_ARGUMENT;
    if (counts == nullptr || (n > 0 && (keys == nullptr || uniq_keys == nullptr || uniq_owner == nullptr || inverse == nullptr)))
        return PSB_DEDUP_ERR_BAD_ARGUMENT;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return PSB_DEDUP_ERR_BAD_ARGUMENT;
    PerDevice d;
    {
        std::lock_guard<std::mutex> guard(g_setup_mutex);
        PerDevice& slot = g_per_device[dev];
        if (!slot.ready) {
            // one-time set-up for this device: turn the symbols into device addresses
            e = cudaGetSymbolAddress((void**)&slot.slots, g_dedup_slots);
            if (e != cudaSuccess) return (int)e;
            e = cudaGetSymbolAddress((void**)&slot.pos, g_dedup_pos);
            if (e != cudaSuccess) return (int)e;
            slot.ready = true;
        }
        d = slot;
    }
    // The array still holds the previous call's state (an interrupted call may have left claimed
    // slots): empty it first, in stream order with the work that follows.
    int rc = dedup_fill_scratch(d.slots, kNoAllocSlots, stream);
    if (rc != 0) return rc;
    return dedup_partition(keys, n, d.slots, kNoAllocSlots, d.pos, shard_owner, n_shards, world, uniq_keys, uniq_owner, inverse,
                           counts, stream);
}
