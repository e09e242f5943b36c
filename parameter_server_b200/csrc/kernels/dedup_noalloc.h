/* psb_dedup_partition_noalloc: key dedup + partition for callers that must not allocate.
 *
 * This entry point has no counterpart in the reference (pico-ps allocates freely on the host heap). It
 * exists for code that runs where device allocation is off limits: inside a serving loop with a fixed
 * memory budget, inside another framework's stream callback or graph-managed region, or in a plug-in
 * that is handed buffers by its host application and is forbidden to call cudaMalloc. Such callers pass
 * every input and output buffer themselves; the only scratch the operation needs (an open-addressing
 * table and one index per key) lives in a fixed array inside this library.
 *
 * Limits and rules
 *   - At most PSB_DEDUP_NOALLOC_MAX_KEYS keys per call; more is refused with PSB_DEDUP_ERR_TOO_LARGE.
 *   - The scratch array (about 2.3 MB) is part of the library image: every GPU that loads the library
 *     holds it until the process exits, whether or not this function is ever called.
 *   - No cudaMalloc, cudaFree or allocating library routine is called, on any call.
 *   - The FIRST call on each device looks up the device address of the scratch array (with that device
 *     current). Make that first call before any stream capture is started.
 *   - Every call on a device shares the one array, which still holds what the previous call left; the
 *     function empties it on the caller's stream before use. Two calls whose kernels overlap on the
 *     GPU (different streams without ordering, or different host threads) race on it: serialise them.
 *     Such a race cannot hang a kernel (every probe loop is bounded by the size of the array); it shows
 *     as wrong output or as the error mark below. The one-time address look-up is guarded by a mutex,
 *     so host threads may make their first calls concurrently.
 *   - Error mark: bit 31 of counts[0] (PSB_DEDUP_COUNT_ERROR_BIT) is set when the array was found
 *     occupied (overlapping calls), when a key equals INT64_MIN or INT64_MIN + 1 (reserved), or when a
 *     shard_owner entry lies outside [0, world). Positions of such keys get inverse -1. The call is
 *     asynchronous, so the mark is read with the outputs; counts[0] & 0x7fffffff is the distinct count.
 *   - All pointers are device pointers valid on the current device; `stream` is a cudaStream_t.
 *
 * Outputs (same meaning as psb::dedup_partition): uniq_keys[n], uniq_owner[n] (first counts[0] entries are
 * valid), inverse[n], counts[1 + world] with counts[0] = number of distinct keys and counts[1 + r] = how many
 * of them rank r owns. shard_owner may be NULL (every key belongs to rank 0; n_shards is then ignored).
 *
 * Returns 0 on success, a positive cudaError_t value, or one of the negative codes below.
 */
#pragma once

#define PSB_DEDUP_NOALLOC_MAX_KEYS 65536u
#define PSB_DEDUP_ERR_TOO_LARGE (-10)
#define PSB_DEDUP_ERR_BAD_ARGUMENT (-11)
#define PSB_DEDUP_COUNT_ERROR_BIT 0x80000000u

#ifdef __cplusplus
extern "C" {
#endif

int psb_dedup_partition_noalloc(const long long* keys, unsigned n, const int* shard_owner, int n_shards, int world,
                                long long* uniq_keys, int* uniq_owner, int* inverse, unsigned* counts, void* stream);

#ifdef __cplusplus
}
#endif
