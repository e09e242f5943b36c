// See segment_sum.h. The sort is cub::DeviceRadixSort (a stable LSD radix sort that ships with the CUDA toolkit);
// the segmented, ordered sum is the kernel below.
#include "segment_sum.h"

#include <cub/device/device_radix_sort.cuh>

#include "common.cuh"

namespace psb {

namespace {

constexpr int kThreads = 256;

__global__ void iota_kernel(unsigned* p, unsigned n) {
    for (unsigned i = blockIdx.x * kThreads + threadIdx.x; i < n; i += gridDim.x * kThreads) p[i] = i;
}

// One lane group per unique id u: its positions are the run of `sorted_ids == u`, found by binary search; the rows
// are added in ascending position order. A very hot key makes one group walk a long run: this is the price of a
// fixed order, and the reason the atomic path stays the default.
__global__ void __launch_bounds__(kThreads) ordered_sum_kernel(const unsigned* __restrict__ sorted_ids,
                                                              const unsigned* __restrict__ sorted_pos, unsigned n,
                                                              const unsigned* __restrict__ counters,
                                                              const unsigned* __restrict__ plan_epoch,
                                                              const float* __restrict__ grads, unsigned bag, unsigned dim,
                                                              float scale, float* __restrict__ agg) {
    const unsigned lanes = lanes_for_dim(dim);
    const unsigned tid = blockIdx.x * kThreads + threadIdx.x;
    const unsigned group = tid / lanes, ngroups = (gridDim.x * kThreads) / lanes, lane = tid % lanes;
    // the counters of a pull live in the half selected by the parity of the pull's call epoch (device memory: a
    // launch replayed from a CUDA graph sees the current one)
    const unsigned n_uniq = counters[(*plan_epoch & 1u) * 16];
    for (unsigned u = group; u < n_uniq; u += ngroups) {
        // lower bounds of u and u + 1
        unsigned lo = 0, hi = n;
        while (lo < hi) {
            const unsigned mid = (lo + hi) >> 1;
            if ((sorted_ids[mid] & 0x7fffffffu) < u) lo = mid + 1; else hi = mid;
        }
        unsigned end = lo, top = n;
        while (end < top) {
            const unsigned mid = (end + top) >> 1;
            if ((sorted_ids[mid] & 0x7fffffffu) <= u) end = mid + 1; else top = mid;
        }
        for (unsigned d = lane * 4; d < dim; d += lanes * 4) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (unsigned j = lo; j < end; ++j) {
                const unsigned pos = sorted_pos[j];
                float4 v = *(const float4*)(grads + (size_t)(pos / bag) * dim + d);
                if (scale != 1.0f) {
                    v.x = __fmul_rn(v.x, scale); v.y = __fmul_rn(v.y, scale);
                    v.z = __fmul_rn(v.z, scale); v.w = __fmul_rn(v.w, scale);
                }
                if (j == lo) {
                    acc = v;
                } else {
                    acc.x = __fadd_rn(acc.x, v.x); acc.y = __fadd_rn(acc.y, v.y);
                    acc.z = __fadd_rn(acc.z, v.z); acc.w = __fadd_rn(acc.w, v.w);
                }
            }
            *(float4*)(agg + (size_t)u * dim + d) = acc;
        }
    }
}

}  // namespace

size_t ordered_segment_sum_temp_bytes(unsigned max_n) {
    size_t bytes = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, bytes, (const unsigned*)nullptr, (unsigned*)nullptr, (const unsigned*)nullptr,
                                    (unsigned*)nullptr, (int)max_n);
    return bytes + (size_t)max_n * sizeof(unsigned);   // + the identity permutation that is sorted along
}

int ordered_segment_sum(const int* inverse, unsigned n, const unsigned* counters, const unsigned* plan_epoch, const float* grads, unsigned bag,
                        unsigned dim, float scale, float* agg, unsigned* sorted_ids, unsigned* sorted_pos, void* temp,
                        size_t temp_bytes, void* stream) {
    if (n == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    unsigned* iota = (unsigned*)temp;
    void* cub_temp = (char*)temp + (size_t)n * sizeof(unsigned);
    size_t cub_bytes = temp_bytes - (size_t)n * sizeof(unsigned);
    iota_kernel<<<148 * 2, kThreads, 0, s>>>(iota, n);
    int bits = 1;
    while (bits < 31 && (1ull << bits) < (unsigned long long)n) ++bits;   // unique ids are below n; bit 31 is a flag, not part of the id
    cudaError_t e = cub::DeviceRadixSort::SortPairs(cub_temp, cub_bytes, (const unsigned*)inverse, sorted_ids, (const unsigned*)iota,
                                                    sorted_pos, (int)n, 0, bits, s);
    if (e != cudaSuccess) return (int)e;
    const unsigned lanes = lanes_for_dim(dim);
    const unsigned long long want = ((unsigned long long)n * lanes + kThreads - 1) / kThreads;
    ordered_sum_kernel<<<(unsigned)(want < 148 * 16 ? want : 148 * 16), kThreads, 0, s>>>(sorted_ids, sorted_pos, n, counters, plan_epoch, grads,
                                                                                      bag, dim, scale, agg);
    return (int)cudaGetLastError();
}

}  // namespace psb
