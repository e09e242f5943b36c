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

constexpr unsigned kBlock = 64;   // occurrences per block of the blocked sum

__device__ __forceinline__ float4 load_grad(const float* grads, unsigned pos, unsigned bag, unsigned dim, unsigned d, float scale) {
    float4 v = *(const float4*)(grads + (size_t)(pos / bag) * dim + d);
    if (scale != 1.0f) {
        v.x = __fmul_rn(v.x, scale); v.y = __fmul_rn(v.y, scale);
        v.z = __fmul_rn(v.z, scale); v.w = __fmul_rn(v.w, scale);
    }
    return v;
}
__device__ __forceinline__ void add_rn(float4& acc, const float4& v) {
    acc.x = __fadd_rn(acc.x, v.x); acc.y = __fadd_rn(acc.y, v.y);
    acc.z = __fadd_rn(acc.z, v.z); acc.w = __fadd_rn(acc.w, v.w);
}

// Left-to-right sum of the gradient rows of sorted entries [lo, end) for the lane's 4 columns at d. The adds are
// chained, the loads are not: four rows are requested before the first is added.
__device__ __forceinline__ float4 run_sum(const unsigned* __restrict__ sorted_pos, unsigned lo, unsigned end,
                                          const float* __restrict__ grads, unsigned bag, unsigned dim, unsigned d, float scale) {
    float4 acc = load_grad(grads, sorted_pos[lo], bag, dim, d, scale);
    unsigned j = lo + 1;
    for (; j + 4 <= end; j += 4) {
        const unsigned p0 = sorted_pos[j], p1 = sorted_pos[j + 1], p2 = sorted_pos[j + 2], p3 = sorted_pos[j + 3];
        const float4 v0 = load_grad(grads, p0, bag, dim, d, scale), v1 = load_grad(grads, p1, bag, dim, d, scale);
        const float4 v2 = load_grad(grads, p2, bag, dim, d, scale), v3 = load_grad(grads, p3, bag, dim, d, scale);
        add_rn(acc, v0); add_rn(acc, v1); add_rn(acc, v2); add_rn(acc, v3);
    }
    for (; j < end; ++j) add_rn(acc, load_grad(grads, sorted_pos[j], bag, dim, d, scale));
    return acc;
}

// The order of the sum (the definition the tests' oracle restates): the occurrences of a key, in position order, are
// cut into blocks of kBlock; every block is added front to back, then the block sums are added front to back. A key
// with up to kBlock occurrences is thus a plain left-to-right sum. The order depends on the batch alone, not on
// which unique id a key happened to get, and the blocks of a hot key are summed by different lane groups.
//
// Pass 1, one lane group per unique id u: its run in the sorted arrays is found by binary search; a run of up to
// kBlock entries is summed here, a longer one is put on the list of long runs.
__global__ void __launch_bounds__(kThreads) ordered_sum_kernel(const unsigned* __restrict__ sorted_ids,
                                                              const unsigned* __restrict__ sorted_pos, unsigned n,
                                                              const unsigned* __restrict__ counters,
                                                              const unsigned* __restrict__ plan_epoch,
                                                              const float* __restrict__ grads, unsigned bag, unsigned dim,
                                                              float scale, float* __restrict__ agg, unsigned* __restrict__ long_cnt,
                                                              uint3* __restrict__ long_runs) {
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
        if (end <= lo) continue;
        if (end - lo > kBlock) {
            if (lane == 0) long_runs[atomicAdd(long_cnt, 1u)] = make_uint3(u, lo, end);
            continue;
        }
        for (unsigned d = lane * 4; d < dim; d += lanes * 4)
            *(float4*)(agg + (size_t)u * dim + d) = run_sum(sorted_pos, lo, end, grads, bag, dim, d, scale);
    }
}

// Pass 2, one CTA per long run (grid-stride): the lane groups of the CTA sum the blocks of the run into a scratch row
// each, then the first group adds the block sums front to back.
__global__ void __launch_bounds__(kThreads) long_run_kernel(const unsigned* __restrict__ sorted_pos, const float* __restrict__ grads,
                                                           unsigned bag, unsigned dim, float scale, float* __restrict__ agg,
                                                           unsigned* __restrict__ long_cnt, const uint3* __restrict__ long_runs,
                                                           float* __restrict__ partials) {
    const unsigned lanes = lanes_for_dim(dim);
    const unsigned lgroup = threadIdx.x / lanes, lgroups = kThreads / lanes, lane = threadIdx.x % lanes;
    const unsigned n_long = long_cnt[0];
    __shared__ unsigned s_base;
    for (unsigned r = blockIdx.x; r < n_long; r += gridDim.x) {
        const uint3 run = long_runs[r];
        const unsigned lo = run.y, end = run.z;
        const unsigned nblk = (end - lo + kBlock - 1) / kBlock;
        __syncthreads();   // s_base of the previous run has been read
        if (threadIdx.x == 0) s_base = atomicAdd(long_cnt + 1, nblk);   // rows of the scratch area for this run's block sums
        __syncthreads();
        float* part = partials + (size_t)s_base * dim;
        for (unsigned k = lgroup; k < nblk; k += lgroups) {
            const unsigned b_lo = lo + k * kBlock, b_end = min(end, b_lo + kBlock);
            for (unsigned d = lane * 4; d < dim; d += lanes * 4)
                *(float4*)(part + (size_t)k * dim + d) = run_sum(sorted_pos, b_lo, b_end, grads, bag, dim, d, scale);
        }
        __syncthreads();   // orders the block sums (global memory) before their reader below
        if (lgroup == 0) {
            for (unsigned d = lane * 4; d < dim; d += lanes * 4) {
                float4 acc = *(const float4*)(part + d);
                unsigned k = 1;
                for (; k + 4 <= nblk; k += 4) {
                    const float4 v0 = *(const float4*)(part + (size_t)k * dim + d), v1 = *(const float4*)(part + (size_t)(k + 1) * dim + d);
                    const float4 v2 = *(const float4*)(part + (size_t)(k + 2) * dim + d), v3 = *(const float4*)(part + (size_t)(k + 3) * dim + d);
                    add_rn(acc, v0); add_rn(acc, v1); add_rn(acc, v2); add_rn(acc, v3);
                }
                for (; k < nblk; ++k) add_rn(acc, *(const float4*)(part + (size_t)k * dim + d));
                *(float4*)(agg + (size_t)run.x * dim + d) = acc;
            }
        }
    }
}

}  // namespace

namespace {
// layout of the temporary storage after the identity permutation and cub's own scratch
struct Scratch {
    size_t counters, runs, partials, total;
};
Scratch scratch_layout(unsigned max_n, unsigned dim, size_t cub_bytes) {
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    Scratch l;
    size_t o = up((size_t)max_n * sizeof(unsigned)) + up(cub_bytes);
    l.counters = o; o += 256;
    const size_t max_long = (size_t)max_n / kBlock + 1;                 // runs longer than kBlock
    l.runs = o; o += up(max_long * sizeof(uint3));
    l.partials = o; o += up((2 * max_long + 1) * (size_t)dim * sizeof(float));   // sum of ceil(len / kBlock) over the long runs
    l.total = o;
    return l;
}
size_t cub_sort_bytes(unsigned max_n) {
    size_t bytes = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, bytes, (const unsigned*)nullptr, (unsigned*)nullptr, (const unsigned*)nullptr,
                                    (unsigned*)nullptr, (int)max_n);
    return bytes;
}
}  // namespace

size_t ordered_segment_sum_temp_bytes(unsigned max_n, unsigned dim) { return scratch_layout(max_n, dim, cub_sort_bytes(max_n)).total; }

int ordered_segment_sum(const int* inverse, unsigned n, unsigned max_n, const unsigned* counters, const unsigned* plan_epoch,
                        const float* grads, unsigned bag, unsigned dim, float scale, float* agg, unsigned* sorted_ids,
                        unsigned* sorted_pos, void* temp, size_t temp_bytes, void* stream) {
    if (n == 0) return 0;
    if (n > max_n) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t cub_bytes = cub_sort_bytes(max_n);
    const Scratch l = scratch_layout(max_n, dim, cub_bytes);
    if (l.total > temp_bytes) return (int)cudaErrorInvalidValue;
    unsigned* iota = (unsigned*)temp;
    void* cub_temp = (char*)temp + ((size_t)max_n * sizeof(unsigned) + 255) / 256 * 256;
    unsigned* long_cnt = (unsigned*)((char*)temp + l.counters);
    uint3* long_runs = (uint3*)((char*)temp + l.runs);
    float* partials = (float*)((char*)temp + l.partials);
    cudaError_t e = cudaMemsetAsync(long_cnt, 0, 8, s);
    if (e != cudaSuccess) return (int)e;
    iota_kernel<<<148 * 2, kThreads, 0, s>>>(iota, n);
    int bits = 1;
    while (bits < 31 && (1ull << bits) < (unsigned long long)n) ++bits;   // unique ids are below n; bit 31 is a flag, not part of the id
    size_t cb = cub_bytes;
    e = cub::DeviceRadixSort::SortPairs(cub_temp, cb, (const unsigned*)inverse, sorted_ids, (const unsigned*)iota, sorted_pos, (int)n, 0,
                                        bits, s);
    if (e != cudaSuccess) return (int)e;
    const unsigned lanes = lanes_for_dim(dim);
    const unsigned long long want = ((unsigned long long)n * lanes + kThreads - 1) / kThreads;
    ordered_sum_kernel<<<(unsigned)(want < 148 * 16 ? want : 148 * 16), kThreads, 0, s>>>(sorted_ids, sorted_pos, n, counters, plan_epoch, grads,
                                                                                      bag, dim, scale, agg, long_cnt, long_runs);
    long_run_kernel<<<148 * 4, kThreads, 0, s>>>(sorted_pos, grads, bag, dim, scale, agg, long_cnt, long_runs, partials);
    return (int)cudaGetLastError();
}

}  // namespace psb
