// dedup_partition: the client-side preparation of a sparse request as a stand-alone operation.
//
// Given a batch of int64 keys it returns the distinct keys, the inverse map (position -> index of its
// distinct key), the owning rank of every distinct key (jump_consistent_hash(murmur(key)) -> shard ->
// shard_owner) and the number of distinct keys per owner. This is what the reference's client does in
// SparseTablePullOperator::generate_request_data (pico-ps/operator/SparsePullOperator.h:91-101) with an
// EasyHashMap (pico-ps/common/EasyHashMap.h:145-163) and the partitioner (pico-ps/common/Partitioner.h:
// 43-45); the fused pull kernel does the same work in its first phase, this entry point serves callers
// that batch or route requests themselves (the RPC path, the NCCL-only baseline, tests).
//
// Scratch: an open-addressing table of at least 2n slots that must be all-empty on entry; the second
// kernel empties every slot it used, so the table is ready for the next call.
#include "dedup.h"

namespace psb {

namespace {

constexpr int kThreads = 256;

// Bit 31 of counts[0] is the error mark of a call: the scratch table was exhausted (it was not empty on entry:
// two calls overlapped on it), a key equals one of the two reserved values, or a shard owner is outside
// [0, world). Positions of such keys get inverse -1; everything else is still valid.
__global__ void dedup_claim_kernel(const long long* __restrict__ keys, unsigned n, Slot* table, unsigned long long mask,
                                   const int* __restrict__ shard_owner, int n_shards, int world, long long* uniq_keys,
                                   int* uniq_owner, unsigned* pos_slot, unsigned* counts) {
    const unsigned lane = threadIdx.x & 31u;
    const unsigned nthreads = gridDim.x * kThreads;
    for (unsigned i0 = ((blockIdx.x * kThreads + threadIdx.x) & ~31u); i0 < n; i0 += nthreads) {
        const unsigned i = i0 + lane;
        long long key = 0;
        unsigned long long h = 0;
        bool won = false;
        if (i < n) {
            key = keys[i];
            bool found = false;
            if (key > kTombstoneKey) {
                h = slot_hash(key) & mask;
                // every probe sequence ends: at most mask + 1 slots are examined
                for (unsigned long long probes = 0; probes <= mask; ++probes) {
                    long long cur = *((volatile long long*)&table[h].key);
                    if (cur == key) { found = true; break; }
                    if (cur == kEmptyKey) {
                        long long prev = (long long)atomicCAS((unsigned long long*)&table[h].key, (unsigned long long)kEmptyKey,
                                                              (unsigned long long)key);
                        if (prev == kEmptyKey) { won = true; found = true; break; }
                        if (prev == key) { found = true; break; }
                    }
                    h = (h + 1) & mask;
                }
            }
            if (!found) atomicOr(&counts[0], kDedupErrorBit);
            pos_slot[i] = found ? (unsigned)h : kNoSlot;
        }
        const unsigned wmask = __ballot_sync(0xffffffffu, won);
        if (wmask == 0) continue;
        unsigned base = 0;
        const int leader = __ffs(wmask) - 1;
        if ((int)lane == leader) base = atomicAdd(&counts[0], (unsigned)__popc(wmask)) & ~kDedupErrorBit;
        base = __shfl_sync(0xffffffffu, base, leader);
        if (won) {
            const unsigned u = base + __popc(wmask & ((1u << lane) - 1u));
            int owner = shard_owner ? shard_owner[sparse_shard_of(key, n_shards)] : 0;
            if (owner < 0 || owner >= world) {
                atomicOr(&counts[0], kDedupErrorBit);
                owner = 0;
            }
            table[h].row = u;
            uniq_keys[u] = key;
            uniq_owner[u] = owner;
            atomicAdd(&counts[1 + owner], 1u);
        }
    }
}

__global__ void dedup_inverse_kernel(unsigned n, Slot* table, const unsigned* __restrict__ pos_slot, int* inverse) {
    for (unsigned i = blockIdx.x * kThreads + threadIdx.x; i < n; i += gridDim.x * kThreads) {
        const unsigned h = pos_slot[i];
        inverse[i] = (h == kNoSlot) ? -1 : (int)table[h].row;
    }
}

__global__ void dedup_clear_kernel(unsigned n, Slot* table, const unsigned* __restrict__ pos_slot) {
    for (unsigned i = blockIdx.x * kThreads + threadIdx.x; i < n; i += gridDim.x * kThreads)
        if (pos_slot[i] != kNoSlot) table[pos_slot[i]].key = kEmptyKey;
}

__global__ void dedup_fill_kernel(Slot* table, unsigned long long slots) {
    for (unsigned long long i = blockIdx.x * (unsigned long long)kThreads + threadIdx.x; i < slots;
         i += (unsigned long long)gridDim.x * kThreads) {
        Slot e;
        e.key = kEmptyKey;
        e.row = kNoRow;
        e.aux = kNoRow;
        table[i] = e;
    }
}

__global__ void shard_of_kernel(const long long* __restrict__ keys, unsigned long long n, int n_shards,
                                const int* __restrict__ shard_owner, int* __restrict__ out) {
    for (unsigned long long i = blockIdx.x * (unsigned long long)kThreads + threadIdx.x; i < n;
         i += (unsigned long long)gridDim.x * kThreads) {
        const int s = sparse_shard_of(keys[i], n_shards);
        out[i] = shard_owner ? shard_owner[s] : s;
    }
}

int run(const long long* keys, unsigned n, Slot* table, unsigned long long slots, unsigned* pos_slot, const int* shard_owner,
        int n_shards, int world, long long* uniq_keys, int* uniq_owner, int* inverse, unsigned* counts, cudaStream_t s) {
    cudaError_t e = cudaMemsetAsync(counts, 0, (size_t)(1 + world) * sizeof(unsigned), s);
    if (e != cudaSuccess) return (int)e;
    if (n == 0) return 0;
    const int blocks = (int)((n + kThreads - 1) / kThreads) < 148 * 8 ? (int)((n + kThreads - 1) / kThreads) : 148 * 8;
    dedup_claim_kernel<<<blocks, kThreads, 0, s>>>(keys, n, table, slots - 1, shard_owner, n_shards, world, uniq_keys,
                                                   uniq_owner, pos_slot, counts);
    dedup_inverse_kernel<<<blocks, kThreads, 0, s>>>(n, table, pos_slot, inverse);
    dedup_clear_kernel<<<blocks, kThreads, 0, s>>>(n, table, pos_slot);
    return (int)cudaGetLastError();
}

}  // namespace

int shard_of_keys(const long long* keys, unsigned long long n, int n_shards, const int* shard_owner, int* out, void* stream) {
    if (n == 0) return 0;
    if (n_shards < 1) return -2;
    const unsigned long long want = (n + kThreads - 1) / kThreads;
    shard_of_kernel<<<(unsigned)(want < 148 * 8 ? want : 148 * 8), kThreads, 0, (cudaStream_t)stream>>>(keys, n, n_shards,
                                                                                                       shard_owner, out);
    return (int)cudaGetLastError();
}

int dedup_fill_scratch(void* scratch, unsigned long long slots, void* stream) {
    dedup_fill_kernel<<<148 * 4, kThreads, 0, (cudaStream_t)stream>>>((Slot*)scratch, slots);
    return (int)cudaGetLastError();
}

int dedup_partition(const long long* keys, unsigned n, void* scratch, unsigned long long scratch_slots, unsigned* pos_scratch,
                    const int* shard_owner, int n_shards, int world, long long* uniq_keys, int* uniq_owner, int* inverse,
                    unsigned* counts, void* stream) {
    if (scratch_slots < 2ull * n || (scratch_slots & (scratch_slots - 1))) return -2;  // power of two, >= 2n
    if (world < 1 || world > kMaxWorld) return -2;
    return run(keys, n, (Slot*)scratch, scratch_slots, pos_scratch, shard_owner, n_shards, world, uniq_keys, uniq_owner,
               inverse, counts, (cudaStream_t)stream);
}

}  // namespace psb
