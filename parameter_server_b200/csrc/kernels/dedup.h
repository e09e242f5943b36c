// Host interface of the stand-alone key dedup + partition operation (see dedup.cu).
#pragma once
#include "common.cuh"

namespace psb {

// Fill `slots` scratch slots (16 bytes each) with the empty marker; needed once after allocation.
int dedup_fill_scratch(void* scratch, unsigned long long slots, void* stream);

// Error mark of a call in counts[0] (see below); the number of distinct keys is counts[0] & ~kDedupErrorBit.
constexpr unsigned kDedupErrorBit = 0x80000000u;

// keys[n] -> uniq_keys[n_uniq], uniq_owner[n_uniq], inverse[n], counts[0] = n_uniq, counts[1 + r] = distinct keys
// owned by rank r. scratch: `scratch_slots` (power of two, >= 2n) empty slots; pos_scratch: n unsigned.
// shard_owner may be null (every key is owned by rank 0). Returns 0, a cudaError_t, or -2 (bad sizes).
// The kernels never wait without a bound: when the scratch table is not empty on entry (two calls overlapping on
// it), a key equals a reserved value (INT64_MIN, INT64_MIN + 1) or a shard owner lies outside [0, world), the call
// still ends and sets kDedupErrorBit in counts[0]; the positions concerned get inverse -1.
int dedup_partition(const long long* keys, unsigned n, void* scratch, unsigned long long scratch_slots, unsigned* pos_scratch,
                    const int* shard_owner, int n_shards, int world, long long* uniq_keys, int* uniq_owner, int* inverse,
                    unsigned* counts, void* stream);

// out[i] = shard of keys[i] under n_shards, or the owner of that shard when shard_owner (device, n_shards ints) is given.
int shard_of_keys(const long long* keys, unsigned long long n, int n_shards, const int* shard_owner, int* out, void* stream);

}  // namespace psb
