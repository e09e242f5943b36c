// Order-preserving pre-aggregation of duplicate keys for the fused push (reproducible mode).
//
// The fused push normally sums the gradients of duplicate keys with fp32 atomics, whose order changes from run to
// run. The reference merges duplicates in a map in arrival order before it applies them once
// (pico-ps/operator/SparsePushOperator.h:130-146 apply_push_arg, :377-409 merge_push_value), so its result is a
// function of the request alone. This pre-pass restores that property: the positions are sorted by their unique id
// with a STABLE radix sort (position order survives inside a key's segment) and every segment is summed in a fixed
// order with non-contracted fp32 adds: the occurrences of a key, in position order, are cut into blocks of 64, every
// block is added front to back, then the block sums are added front to back (a key with up to 64 occurrences is a
// plain left-to-right sum). A host loop that adds in that order gets the same bits; the blocks of a hot key are summed
// in parallel, so the head of a skewed batch does not serialise the pass.
#pragma once
#include <cstddef>
#include <cstdint>

namespace psb {

// Bytes of temporary device storage needed for batches of up to max_n positions.
size_t ordered_segment_sum_temp_bytes(unsigned max_n, unsigned dim);

// inverse[n]: unique id of every position; counters / plan_epoch: the pull's counter block ([2][16] words, word 0 of
// a half = number of unique ids) and the device word whose parity selects the half; grads:
// [n / bag][dim]; agg: [n_uniq][dim] output. `scale` multiplies every gradient (mean pooling), 1 for none.
// sorted_ids / sorted_pos: device scratch of max_n unsigned each; temp: ordered_segment_sum_temp_bytes(max_n, dim)
// bytes (max_n = the size the storage was made for, n <= max_n). Returns 0 or a cudaError_t.
int ordered_segment_sum(const int* inverse, unsigned n, unsigned max_n, const unsigned* counters, const unsigned* plan_epoch,
                        const float* grads, unsigned bag, unsigned dim, float scale, float* agg, unsigned* sorted_ids,
                        unsigned* sorted_pos, void* temp, size_t temp_bytes, void* stream);

}  // namespace psb
