// Order-preserving pre-aggregation of duplicate keys for the fused push (reproducible mode).
//
// The fused push normally sums the gradients of duplicate keys with fp32 atomics, whose order changes from run to
// run. The reference merges duplicates in a map in arrival order before it applies them once
// (pico-ps/operator/SparsePushOperator.h:130-146 apply_push_arg, :377-409 merge_push_value), so its result is a
// function of the request alone. This pre-pass restores that property: the positions are sorted by their unique id
// with a STABLE radix sort (position order survives inside a key's segment) and every segment is summed front to
// back with non-contracted fp32 adds, which is bit for bit what a host loop over the positions computes.
#pragma once
#include <cstddef>
#include <cstdint>

namespace psb {

// Bytes of temporary device storage needed for batches of up to max_n positions.
size_t ordered_segment_sum_temp_bytes(unsigned max_n);

// inverse[n]: unique id of every position; counters / plan_epoch: the pull's counter block ([2][16] words, word 0 of
// a half = number of unique ids) and the device word whose parity selects the half; grads:
// [n / bag][dim]; agg: [n_uniq][dim] output. `scale` multiplies every gradient (mean pooling), 1 for none.
// sorted_ids / sorted_pos: device scratch of n unsigned each; temp: ordered_segment_sum_temp_bytes(n) bytes.
// Returns 0 or a cudaError_t.
int ordered_segment_sum(const int* inverse, unsigned n, const unsigned* counters, const unsigned* plan_epoch, const float* grads, unsigned bag,
                        unsigned dim, float scale, float* agg, unsigned* sorted_ids, unsigned* sorted_pos, void* temp,
                        size_t temp_bytes, void* stream);

}  // namespace psb
