// GpuTable implementation: memory management on the host, scan / set / erase / store kernels on the
// device. The hot pull / push path is in kernels/sparse_fused.cu; what is here serves dump, load,
// restore, reshard, for_each, erase_if, sync-push store and statistics
// (pico-ps/operator/{DumpOperator,LoadOperator,RestoreOperator,UpdateContextOperator,ForEachOperator,
// EraseIfOperator}.h).
#include "gpu_table.h"

#include <algorithm>
#include <cstdio>
#include <stdexcept>

namespace psb {

#define PSB_CUDA_OK(expr)                                                                            \
    do {                                                                                             \
        cudaError_t _e = (expr);                                                                     \
        if (_e != cudaSuccess)                                                                       \
            return Status::Error(std::string(#expr) + ": " + cudaGetErrorString(_e));                \
    } while (0)

namespace {

constexpr int kThreads = 256;

inline int grid_for(uint64_t n, int per_thread = 1) {
    uint64_t b = (n + (uint64_t)kThreads * per_thread - 1) / ((uint64_t)kThreads * per_thread);
    return (int)std::max<uint64_t>(1, std::min<uint64_t>(b, 148 * 16));
}

uint64_t pow2_ceil(uint64_t v) {
    uint64_t p = 1;
    while (p < v) p <<= 1;
    return p;
}

__global__ void fill_slots_kernel(Slot* s, uint64_t n) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        Slot e;
        e.key = kEmptyKey;
        e.row = kNoRow;
        e.aux = kNoRow;
        s[i] = e;
    }
}

__device__ __forceinline__ bool filter_match(const ShardFilter& f, const TableView& t, long long key, unsigned row) {
    switch (f.mode) {
        case 0: return true;
        case 1: return sparse_shard_of(key, f.n_shards) == f.shard;
        case 2: return f.shard_owner[sparse_shard_of(key, f.n_shards)] != f.rank;
        case 3: return f.shard_owner[sparse_shard_of(key, f.n_shards)] == f.rank;
        case 4: return row < kRowPending && t.dirty_bits != nullptr && ((t.dirty_bits[row >> 5] >> (row & 31u)) & 1u);
        default: return false;
    }
}

// Scan slots [begin, end); matching live entries are appended (warp-aggregated) to out_keys/out_rows.
__global__ void export_kernel(TableView t, ShardFilter f, uint64_t begin, uint64_t end, long long* out_keys,
                              float* out_rows, unsigned long long* out_count) {
    const unsigned lane = threadIdx.x & 31u;
    const uint64_t warp = (blockIdx.x * (uint64_t)blockDim.x + threadIdx.x) >> 5;
    const uint64_t nwarps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
    for (uint64_t base = begin + warp * 32; base < end; base += nwarps * 32) {
        const uint64_t s = base + lane;
        long long key = kEmptyKey;
        unsigned row = kNoRow;
        bool hit = false;
        if (s < end) {
            key = t.slots[s].key;
            row = t.slots[s].row;
            hit = key != kEmptyKey && key != kTombstoneKey && filter_match(f, t, key, row);
        }
        const unsigned ballot = __ballot_sync(0xffffffffu, hit);
        if (ballot == 0) continue;
        unsigned long long pos0 = 0;
        if (lane == 0) pos0 = atomicAdd(out_count, (unsigned long long)__popc(ballot));
        pos0 = __shfl_sync(0xffffffffu, pos0, 0);
        const unsigned my_off = __popc(ballot & ((1u << lane) - 1u));
        if (hit) out_keys[pos0 + my_off] = key;
        if (out_rows == nullptr) continue;
        // cooperative row copy: the whole warp copies each hit's row
        unsigned rem = ballot;
        unsigned k = 0;
        while (rem) {
            const int src_lane = __ffs(rem) - 1;
            rem &= rem - 1;
            const unsigned r = __shfl_sync(0xffffffffu, row, src_lane);
            const long long rk = __shfl_sync(0xffffffffu, key, src_lane);
            float* dst = out_rows + (pos0 + k) * t.stride;
            if (r < kRowPending) {
                const float* src = t.row_ptr(r);
                for (unsigned d = lane * 4; d < t.stride; d += 128) *(float4*)(dst + d) = *(const float4*)(src + d);
            } else {
                // key without a backing row: export its initial value
                for (unsigned d = lane; d < t.stride; d += 32) {
                    float v = 0.f;
                    if (d < t.dim) v = init_uniform(rk, d, t.init_seed, t.init_range);
                    else if (d < t.dim * (1 + t.n_opt_slots)) v = t.slot_init[(d / t.dim - 1) < 2 ? (d / t.dim - 1) : 1];
                    dst[d] = v;
                }
            }
            ++k;
        }
    }
}

// set_rows pass 1: find-or-insert + attach a row; records the slot and whether the row is new.
__global__ void set_resolve_kernel(TableView t, const long long* keys, uint64_t n, unsigned* out_slot,
                                   unsigned char* out_new, unsigned* status) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        bool inserted = false, oom = false;
        unsigned slot = table_find_or_insert(t, keys[i], true, &inserted);
        unsigned char is_new = 0;
        if (slot == kNoSlot) {
            atomicCAS(status, 0u, kStOom);
        } else {
            if (table_attach_row(t, slot, &oom)) is_new = 1;
            if (inserted) atomicAdd(t.n_items, 1ull);
            if (oom) atomicCAS(status, 0u, kStOom);
        }
        out_slot[i] = slot;
        out_new[i] = is_new;
    }
}

// set_rows pass 2: write the row payload.
__global__ void set_write_kernel(TableView t, const long long* keys, const float* rows, uint64_t n,
                                 const unsigned* slot_of, const unsigned char* is_new, int emb_only) {
    const unsigned lanes = lanes_for_dim(t.dim);
    const uint64_t tid = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x;
    const uint64_t group = tid / lanes, ngroups = ((uint64_t)gridDim.x * blockDim.x) / lanes;
    const unsigned lane = tid % lanes;
    for (uint64_t i = group; i < n; i += ngroups) {
        const unsigned slot = slot_of[i];
        if (slot == kNoSlot) continue;
        const unsigned row = t.slots[slot].row;
        if (row >= kRowPending) continue;
        float* dst = t.row_ptr(row);
        if (emb_only) {
            if (is_new[i]) row_init(t, dst, keys[i], lane, lanes);
            const float* src = rows + i * t.dim;
            for (unsigned d = lane * 4; d < t.dim; d += lanes * 4) *(float4*)(dst + d) = *(const float4*)(src + d);
        } else {
            const float* src = rows + i * t.stride;
            for (unsigned d = lane * 4; d < t.stride; d += lanes * 4) *(float4*)(dst + d) = *(const float4*)(src + d);
        }
        if (t.dirty_bits != nullptr && lane == 0) atomicOr(&t.dirty_bits[row >> 5], 1u << (row & 31u));
    }
}

__global__ void get_rows_kernel(TableView t, const long long* keys, uint64_t n, float* out, int* found,
                                int emb_only) {
    const unsigned lanes = lanes_for_dim(t.dim);
    const uint64_t tid = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x;
    const uint64_t group = tid / lanes, ngroups = ((uint64_t)gridDim.x * blockDim.x) / lanes;
    const unsigned lane = tid % lanes;
    const unsigned width = emb_only ? t.dim : t.stride;
    for (uint64_t i = group; i < n; i += ngroups) {
        bool ins;
        const unsigned slot = table_find_or_insert(t, keys[i], false, &ins);
        unsigned row = kNoRow;
        if (slot != kNoSlot) row = t.slots[slot].row;
        float* dst = out + i * width;
        if (slot != kNoSlot && row < kRowPending) {
            const float* src = t.row_ptr(row);
            for (unsigned d = lane * 4; d < width; d += lanes * 4) *(float4*)(dst + d) = *(const float4*)(src + d);
        } else if (slot != kNoSlot) {
            // key without a backing row: its value is the initial one (same rule as the export kernel)
            for (unsigned d = lane; d < width; d += lanes) {
                float v = 0.f;
                if (d < t.dim) v = init_uniform(keys[i], d, t.init_seed, t.init_range);
                else if (d < t.dim * (1 + t.n_opt_slots)) v = t.slot_init[(d / t.dim - 1) < 2 ? (d / t.dim - 1) : 1];
                dst[d] = v;
            }
        } else {
            for (unsigned d = lane * 4; d < width; d += lanes * 4) *(float4*)(dst + d) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (found != nullptr && lane == 0) found[i] = (slot != kNoSlot) ? 1 : 0;
    }
}

__device__ __forceinline__ void erase_slot(const TableView& t, uint64_t s, long long key, unsigned long long* n_erased) {
    // Only the thread that swings the key to the tombstone releases the row.
    long long prev = (long long)atomicCAS((unsigned long long*)&t.slots[s].key, (unsigned long long)key,
                                          (unsigned long long)kTombstoneKey);
    if (prev != key) return;
    const unsigned row = t.slots[s].row;
    t.slots[s].row = kNoRow;
    t.slots[s].aux = kNoRow;
    if (row < kRowPending) {
        if (t.touched_bits != nullptr) atomicAnd(&t.touched_bits[row >> 5], ~(1u << (row & 31u)));
        if (t.dirty_bits != nullptr) atomicAnd(&t.dirty_bits[row >> 5], ~(1u << (row & 31u)));
        const int pos = atomicAdd(t.free_count, 1);
        t.free_rows[pos] = row;
    }
    atomicAdd(t.n_items, (unsigned long long)-1ll);
    atomicAdd(n_erased, 1ull);
}

__global__ void erase_keys_kernel(TableView t, const long long* keys, uint64_t n, unsigned long long* n_erased) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        bool ins;
        const unsigned slot = table_find_or_insert(t, keys[i], false, &ins);
        if (slot != kNoSlot) erase_slot(t, slot, keys[i], n_erased);
    }
}

__global__ void erase_filter_kernel(TableView t, ShardFilter f, uint64_t cap, unsigned long long* n_erased) {
    for (uint64_t s = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; s < cap; s += (uint64_t)gridDim.x * blockDim.x) {
        const long long key = t.slots[s].key;
        if (key == kEmptyKey || key == kTombstoneKey) continue;
        if (filter_match(f, t, key, t.slots[s].row)) erase_slot(t, s, key, n_erased);
    }
}

// ---- scans evaluated where the rows live -------------------------------------------------------------------
// A warp examines 32 consecutive slots; the entries that pass the shard filter are then visited one by one by the
// whole warp, which reads the row with 16-byte loads and reduces across lanes. Only counters leave the GPU.
struct DeviceScan {
    int pred_type;          // ScanPredicate::Type, or -1: statistics over `section`
    long long mod, rem;
    double threshold;
    unsigned section;
};

__device__ __forceinline__ float row_value(const TableView& t, const float* row, long long key, unsigned d) {
    // value of float d of the full row; a key without a backing row has its initial value
    if (row != nullptr) return row[d];
    if (d < t.dim) return init_uniform(key, d, t.init_seed, t.init_range);
    if (d < t.dim * (1 + t.n_opt_slots)) return t.slot_init[(d / t.dim - 1) < 2 ? (d / t.dim - 1) : 1];
    return 0.f;
}

__global__ void scan_kernel(TableView t, ShardFilter f, DeviceScan sc, uint64_t cap, unsigned long long* n_erased,
                            double* stats /* count, sum, sum_sq, max_abs (bits) */) {
    const unsigned lane = threadIdx.x & 31u;
    const uint64_t warp = (blockIdx.x * (uint64_t)blockDim.x + threadIdx.x) >> 5;
    const uint64_t nwarps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
    double w_count = 0, w_sum = 0, w_sq = 0, w_max = 0;   // per-warp partials (lane 0 holds them)
    for (uint64_t base = warp * 32; base < cap; base += nwarps * 32) {
        const uint64_t s = base + lane;
        long long key = kEmptyKey;
        unsigned row = kNoRow;
        bool cand = false;
        if (s < cap) {
            key = t.slots[s].key;
            row = t.slots[s].row;
            cand = key != kEmptyKey && key != kTombstoneKey && filter_match(f, t, key, row);
        }
        bool doomed = false;
        if (cand && sc.pred_type == 0) doomed = ((key % sc.mod) + sc.mod) % sc.mod == sc.rem;   // KEY_MOD needs no row
        if (cand && sc.pred_type == 3) doomed = true;                                          // ALL
        const bool need_row = cand && (sc.pred_type < 0 || sc.pred_type == 1 || sc.pred_type == 2);
        unsigned rem = __ballot_sync(0xffffffffu, need_row);
        while (rem) {
            const int src = __ffs(rem) - 1;
            rem &= rem - 1;
            const unsigned r = __shfl_sync(0xffffffffu, row, src);
            const long long rk = __shfl_sync(0xffffffffu, key, src);
            const float* rp = r < kRowPending ? t.row_ptr(r) : nullptr;
            const unsigned sec = sc.pred_type == 2 ? 1u : (sc.pred_type == 1 ? 0u : sc.section);
            double a = 0, q = 0, m = 0;
            for (unsigned d = lane; d < t.dim; d += 32) {
                const double v = (double)row_value(t, rp, rk, sec * t.dim + d);
                a += v;
                q += v * v;
                m = fmax(m, fabs(v));
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                a += __shfl_xor_sync(0xffffffffu, a, o);
                q += __shfl_xor_sync(0xffffffffu, q, o);
                m = fmax(m, __shfl_xor_sync(0xffffffffu, m, o));
            }
            if (sc.pred_type < 0) {
                w_count += 1;
                w_sum += a;
                w_sq += q;
                w_max = fmax(w_max, m);
            } else if ((int)lane == src) {
                doomed = sc.pred_type == 1 ? sqrt(q) < sc.threshold : a / (double)t.dim < sc.threshold;
            }
        }
        if (doomed) erase_slot(t, s, key, n_erased);
    }
    if (sc.pred_type < 0 && lane == 0 && w_count > 0) {
        atomicAdd(&stats[0], w_count);
        atomicAdd(&stats[1], w_sum);
        atomicAdd(&stats[2], w_sq);
        atomicMax((unsigned long long*)&stats[3], (unsigned long long)__double_as_longlong(w_max));  // non-negative doubles order like their bits
    }
}

__global__ void shard_count_kernel(TableView t, uint64_t cap, int n_shards, unsigned long long* counts) {
    for (uint64_t s = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; s < cap; s += (uint64_t)gridDim.x * blockDim.x) {
        const long long key = t.slots[s].key;
        if (key == kEmptyKey || key == kTombstoneKey) continue;
        atomicAdd(&counts[sparse_shard_of(key, n_shards)], 1ull);
    }
}

// OP_STORE: apply the optimizer once per touched row with the accumulated delta, then zero it.
__global__ void store_delta_kernel(TableView t, OptConfig opt, unsigned n_touched) {
    const unsigned lanes = lanes_for_dim(t.dim);
    const unsigned tid = blockIdx.x * blockDim.x + threadIdx.x;
    const unsigned group = tid / lanes, ngroups = (gridDim.x * blockDim.x) / lanes, lane = tid % lanes;
    const unsigned dim = t.dim;
    for (unsigned j = group; j < n_touched; j += ngroups) {
        const unsigned row = t.touched_list[j];
        // Test-and-clear: a row that was erased (and maybe recycled and touched again) since it entered the list
        // may be listed twice or with its bit already clear; only the entry that clears the bit applies the delta.
        unsigned had = 0;
        if (lane == 0) had = atomicAnd(&t.touched_bits[row >> 5], ~(1u << (row & 31u))) & (1u << (row & 31u));
        const unsigned gl0 = (threadIdx.x & 31u) / lanes * lanes;  // first lane of this group inside its warp
        const unsigned gmask = (lanes >= 32u ? 0xffffffffu : ((1u << lanes) - 1u)) << gl0;
        had = __shfl_sync(gmask, had, gl0);
        if (!had) continue;
        float* w = t.row_ptr(row);
        float* delta = w + (size_t)(t.n_opt_slots + 1) * dim;
        for (unsigned d = lane * 4; d < dim; d += lanes * 4) {
            float4 gv = *(float4*)(delta + d);
            float4 wv = *(float4*)(w + d);
            float4 s0 = make_float4(0.f, 0.f, 0.f, 0.f), s1 = s0;
            if (t.n_opt_slots > 0) s0 = *(float4*)(w + dim + d);
            if (t.n_opt_slots > 1) s1 = *(float4*)(w + 2 * dim + d);
            opt_update(opt, wv.x, s0.x, s1.x, gv.x);
            opt_update(opt, wv.y, s0.y, s1.y, gv.y);
            opt_update(opt, wv.z, s0.z, s1.z, gv.z);
            opt_update(opt, wv.w, s0.w, s1.w, gv.w);
            *(float4*)(w + d) = wv;
            if (t.n_opt_slots > 0) *(float4*)(w + dim + d) = s0;
            if (t.n_opt_slots > 1) *(float4*)(w + 2 * dim + d) = s1;
            *(float4*)(delta + d) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (lane == 0 && t.dirty_bits != nullptr) atomicOr(&t.dirty_bits[row >> 5], 1u << (row & 31u));
    }
}

// Puts the election word of every slot back to its rest value (after a push that was cut short).
__global__ void clear_aux_kernel(Slot* s, uint64_t n) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
        s[i].aux = kNoRow;
}

__global__ void rehash_kernel(const Slot* old_slots, uint64_t old_cap, Slot* new_slots, unsigned long long new_mask,
                              unsigned* status) {
    for (uint64_t s = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; s < old_cap; s += (uint64_t)gridDim.x * blockDim.x) {
        const Slot e = old_slots[s];
        if (e.key == kEmptyKey || e.key == kTombstoneKey) continue;
        unsigned long long h = slot_hash(e.key) & new_mask;
        bool placed = false;
        for (unsigned long long probe = 0; probe <= new_mask; ++probe) {
            long long prev = (long long)atomicCAS((unsigned long long*)&new_slots[h].key, (unsigned long long)kEmptyKey,
                                                  (unsigned long long)e.key);
            if (prev == kEmptyKey) {
                new_slots[h].row = e.row;
                placed = true;
                break;
            }
            h = (h + 1) & new_mask;
        }
        if (!placed) atomicCAS(status, 0u, kStOom);
    }
}

}  // namespace

GpuTable::GpuTable(const GpuTableConfig& cfg) : cfg_(cfg) {
    cudaSetDevice(cfg_.device);
    n_slots_ = (uint32_t)opt_num_slots(cfg_.opt_type);
    stride_ = cfg_.dim * (1 + n_slots_ + (cfg_.sync_delta ? 1 : 0));
    capacity_ = pow2_ceil(std::max<uint64_t>(cfg_.index_capacity, 1024));
    max_rows_ = cfg_.max_rows ? cfg_.max_rows : capacity_ / 4 * 3;
    if (max_rows_ > 0xFFFFFF00ull) max_rows_ = 0xFFFFFF00ull;
    const uint64_t slab_rows = 1ull << cfg_.slab_shift;
    max_slabs_ = (uint32_t)((max_rows_ + slab_rows - 1) / slab_rows);
    max_rows_ = (uint64_t)max_slabs_ * slab_rows;
    auto must = [](cudaError_t e, const char* what) {
        if (e != cudaSuccess) throw std::runtime_error(std::string("GpuTable: ") + what + ": " + cudaGetErrorString(e));
    };
    must(cudaMalloc(&slots_, capacity_ * sizeof(Slot)), "index");
    bytes_ += capacity_ * sizeof(Slot);
    fill_slots_kernel<<<grid_for(capacity_, 4), kThreads>>>(slots_, capacity_);
    must(cudaMalloc(&slabs_dev_, (size_t)max_slabs_ * sizeof(float*)), "slab table");
    must(cudaMemset(slabs_dev_, 0, (size_t)max_slabs_ * sizeof(float*)), "slab table");
    free_cap_ = max_rows_;
    must(cudaMalloc(&free_rows_, free_cap_ * sizeof(unsigned)), "free stack");
    bytes_ += free_cap_ * sizeof(unsigned);
    const uint64_t bit_words = (max_rows_ + 31) / 32;
    must(cudaMalloc(&touched_bits_, bit_words * 4), "touched bits");
    must(cudaMemset(touched_bits_, 0, bit_words * 4), "touched bits");
    bytes_ += bit_words * 4;
    if (cfg_.sync_delta) {
        touched_cap_ = (uint32_t)std::min<uint64_t>(max_rows_, 0xFFFFFFFFull);
        must(cudaMalloc(&touched_list_, (size_t)touched_cap_ * 4), "touched list");
        bytes_ += (uint64_t)touched_cap_ * 4;
    }
    must(cudaMalloc(&scratch_, 64 * sizeof(unsigned long long)), "scratch");
    must(cudaMemset(scratch_, 0, 64 * sizeof(unsigned long long)), "scratch");
    // scratch layout (8-byte words): 0 n_items, 1 row_bump(u32), 2 free_count(i32), 3 touched_count(u32),
    //                                4 op counter, 5 op status, 6 rows_avail(u32)
    n_items_ = scratch_ + 0;
    row_bump_ = (unsigned*)(scratch_ + 1);
    free_count_ = (int*)(scratch_ + 2);
    touched_count_ = (unsigned*)(scratch_ + 3);
    must(cudaHostAlloc((void**)&host_mirror_, 64, cudaHostAllocDefault), "pinned mirror");
    host_mirror_[0] = host_mirror_[1] = 0;
    must(cudaMalloc(&view_dev_, sizeof(TableView)), "device view");
    auto_grow_ = cfg_.max_rows == 0;   // an explicit row ceiling is a limit the caller wants kept
    if (!publish_view().ok()) throw std::runtime_error("GpuTable: cannot publish the device view");
    must(cudaDeviceSynchronize(), "init");
}

GpuTable::~GpuTable() {
    cudaSetDevice(cfg_.device);
    for (float* s : slabs_) cudaFree(s);
    cudaFree(slots_);
    cudaFree(slabs_dev_);
    cudaFree(free_rows_);
    cudaFree(touched_bits_);
    if (touched_list_) cudaFree(touched_list_);
    if (dirty_bits_) cudaFree(dirty_bits_);
    cudaFree(scratch_);
    if (view_dev_) cudaFree(view_dev_);
    if (host_mirror_) cudaFreeHost((void*)host_mirror_);
}

Status GpuTable::publish_view() {
    const TableView v = view();
    PSB_CUDA_OK(cudaMemcpy(view_dev_, &v, sizeof(TableView), cudaMemcpyHostToDevice));
    return Status::Ok();
}

// Raise the row ceiling: the free stack, the per-row bit sets and the slab pointer table are sized by it.
Status GpuTable::grow_row_ceiling(uint64_t new_max_rows) {
    const uint64_t slab_rows = 1ull << cfg_.slab_shift;
    if (new_max_rows > 0xFFFFFF00ull) new_max_rows = 0xFFFFFF00ull;
    const uint32_t new_slabs = (uint32_t)((new_max_rows + slab_rows - 1) / slab_rows);
    new_max_rows = (uint64_t)new_slabs * slab_rows;
    if (new_max_rows <= max_rows_) return Status::Ok();
    const uint64_t old_words = (max_rows_ + 31) / 32, new_words = (new_max_rows + 31) / 32;
    auto regrow = [&](void** p, uint64_t old_bytes, uint64_t new_bytes, bool zero_tail) -> Status {
        void* q = nullptr;
        if (cudaMalloc(&q, new_bytes) != cudaSuccess) {
            cudaGetLastError();
            return Status::OOM("GpuTable: no memory to raise the row ceiling");
        }
        if (*p != nullptr && old_bytes) cudaMemcpy(q, *p, old_bytes, cudaMemcpyDeviceToDevice);
        if (zero_tail && new_bytes > old_bytes) cudaMemset((char*)q + old_bytes, 0, new_bytes - old_bytes);
        if (*p != nullptr) cudaFree(*p);
        *p = q;
        bytes_ += new_bytes - old_bytes;
        return Status::Ok();
    };
    PSB_RETURN_IF_ERROR(check_budget((new_max_rows - max_rows_) * 4 + (new_words - old_words) * 8));
    PSB_RETURN_IF_ERROR(regrow((void**)&free_rows_, free_cap_ * 4, new_max_rows * 4, false));
    PSB_RETURN_IF_ERROR(regrow((void**)&touched_bits_, old_words * 4, new_words * 4, true));
    if (dirty_bits_) PSB_RETURN_IF_ERROR(regrow((void**)&dirty_bits_, old_words * 4, new_words * 4, true));
    if (touched_list_) {
        PSB_RETURN_IF_ERROR(regrow((void**)&touched_list_, (uint64_t)touched_cap_ * 4, new_max_rows * 4, false));
        touched_cap_ = (uint32_t)std::min<uint64_t>(new_max_rows, 0xFFFFFFFFull);
    }
    {
        uint64_t before = bytes_;
        PSB_RETURN_IF_ERROR(regrow((void**)&slabs_dev_, (uint64_t)max_slabs_ * sizeof(float*), (uint64_t)new_slabs * sizeof(float*), true));
        bytes_ = before;   // the pointer table is not counted (it never was)
    }
    free_cap_ = new_max_rows;
    max_rows_ = new_max_rows;
    max_slabs_ = new_slabs;
    return Status::Ok();
}

Status GpuTable::maybe_grow(uint64_t n_new) {
    if (!auto_grow_) return Status::Ok();
    // live keys as of the last completed usage refresh, plus a margin for calls still in flight (as reserve_rows)
    const uint64_t bump = (unsigned)host_mirror_[0];
    const int freec = (int)(unsigned)host_mirror_[1];
    const uint64_t used = bump - (uint64_t)std::max(freec, 0);
    if ((used + 3 * n_new) * 2 <= capacity_) return Status::Ok();
    cudaSetDevice(cfg_.device);
    PSB_CUDA_OK(cudaDeviceSynchronize());   // nothing may still be probing the old index
    uint64_t want = capacity_;
    while ((rows_used() + 3 * n_new) * 2 > want) want *= 2;
    if (want == capacity_) return Status::Ok();   // the mirror was stale: there is room
    PSB_RETURN_IF_ERROR(rebuild_index(want, nullptr));
    PSB_RETURN_IF_ERROR(grow_row_ceiling(capacity_ / 4 * 3));
    ++grows_;
    return publish_view();
}

Status GpuTable::check_budget(uint64_t extra) {
    if (cfg_.hard_limit_bytes && bytes_ + extra > cfg_.hard_limit_bytes) {
        healthy_ = false;
        return Status::OOM("row pool would exceed the hard memory limit");
    }
    if (cfg_.soft_limit_bytes && bytes_ + extra > cfg_.soft_limit_bytes) {
        healthy_ = false;
        return Status::OOM("row pool would exceed the soft memory limit");
    }
    return Status::Ok();
}

Status GpuTable::add_slab() {
    if (slabs_.size() >= max_slabs_) {
        healthy_ = false;
        return Status::OOM("row pool reached max_rows");
    }
    const uint64_t bytes = (uint64_t)(1ull << cfg_.slab_shift) * stride_ * sizeof(float);
    PSB_RETURN_IF_ERROR(check_budget(bytes));
    float* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        healthy_ = false;
        return Status::OOM(std::string("cudaMalloc slab: ") + cudaGetErrorString(e));
    }
    PSB_CUDA_OK(cudaMemcpy(slabs_dev_ + slabs_.size(), &p, sizeof(float*), cudaMemcpyHostToDevice));
    slabs_.push_back(p);
    bytes_ += bytes;
    rows_avail_ = (uint32_t)(slabs_.size() << cfg_.slab_shift);
    PSB_CUDA_OK(cudaMemcpy(scratch_ + 6, &rows_avail_, sizeof(uint32_t), cudaMemcpyHostToDevice));
    return Status::Ok();
}

Status GpuTable::reserve_rows(uint64_t n) {
    cudaSetDevice(cfg_.device);
    // The pinned mirror holds the counters as of the last completed refresh_usage_async(); calls
    // still in flight may each have attached up to n rows since, hence the margin. No host sync.
    const uint64_t bump = (unsigned)host_mirror_[0];
    const int freec = (int)(unsigned)host_mirror_[1];
    const uint64_t used = bump - (uint64_t)std::max(freec, 0);
    const uint64_t need = used + 3 * n;
    if (need <= rows_avail_) return Status::Ok();
    // grow geometrically (at least a quarter of the pool) so that allocation calls are amortised
    const uint64_t target = std::max<uint64_t>(need, (uint64_t)rows_avail_ + rows_avail_ / 4);
    while (need > rows_avail_ || (target > rows_avail_ && slabs_.size() < max_slabs_)) {
        Status st = add_slab();
        if (!st.ok()) return need <= rows_avail_ ? Status::Ok() : st;  // the kernel reports what does not fit
    }
    return Status::Ok();
}

Status GpuTable::reserve_exact(uint64_t n_new) {
    // Explicit pre-allocation: reads the counters synchronously, so no margin for calls in flight is needed.
    const uint64_t need = rows_used() + n_new;
    while (need > rows_avail_) PSB_RETURN_IF_ERROR(add_slab());
    return Status::Ok();
}

void GpuTable::refresh_usage_async(void* stream) {
    cudaMemcpyAsync((void*)host_mirror_, scratch_ + 1, 16, cudaMemcpyDeviceToHost, (cudaStream_t)stream);
}

TableView GpuTable::view() const {
    TableView v;
    v.slots = slots_;
    v.mask = capacity_ - 1;
    v.slabs = slabs_dev_;
    v.slab_shift = cfg_.slab_shift;
    v.stride = stride_;
    v.dim = cfg_.dim;
    v.n_opt_slots = n_slots_;
    v.has_delta = cfg_.sync_delta ? 1 : 0;
    v.rows_avail = (const unsigned*)(scratch_ + 6);
    v.max_probe = (unsigned)std::min<uint64_t>(cfg_.max_probe, capacity_);
    v.row_bump = row_bump_;
    v.free_rows = free_rows_;
    v.free_count = free_count_;
    v.n_items = n_items_;
    v.touched_bits = touched_bits_;
    v.touched_list = touched_list_;
    v.touched_count = touched_count_;
    v.touched_cap = touched_cap_;
    v.dirty_bits = dirty_bits_;
    v.init_seed = cfg_.init_seed;
    v.init_range = cfg_.init_range;
    v.slot_init[0] = cfg_.slot_init0;
    v.slot_init[1] = cfg_.slot_init1;
    return v;
}

uint64_t GpuTable::size() {
    cudaSetDevice(cfg_.device);
    unsigned long long v = 0;
    cudaMemcpy(&v, n_items_, sizeof(v), cudaMemcpyDeviceToHost);
    return v;
}

uint64_t GpuTable::rows_used() {
    cudaSetDevice(cfg_.device);
    unsigned long long w[3];
    cudaMemcpy(w, scratch_ + 1, sizeof(unsigned long long) * 2, cudaMemcpyDeviceToHost);
    const unsigned bump = (unsigned)w[0];
    const int freec = (int)(unsigned)w[1];
    return (uint64_t)bump - (uint64_t)std::max(freec, 0);
}

Status GpuTable::export_window(uint64_t cursor, uint64_t window, const ShardFilter& f, long long* out_keys,
                               float* out_rows, uint64_t* n_out, uint64_t* next_cursor, void* stream) {
    cudaSetDevice(cfg_.device);
    cudaStream_t s = (cudaStream_t)stream;
    const uint64_t end = std::min(capacity_, cursor + window);
    *n_out = 0;
    *next_cursor = end;
    if (cursor >= end) return Status::Ok();
    PSB_CUDA_OK(cudaMemsetAsync(scratch_ + 4, 0, 8, s));
    export_kernel<<<grid_for(end - cursor), kThreads, 0, s>>>(view(), f, cursor, end, out_keys, out_rows, scratch_ + 4);
    unsigned long long c = 0;
    PSB_CUDA_OK(cudaMemcpyAsync(&c, scratch_ + 4, 8, cudaMemcpyDeviceToHost, s));
    PSB_CUDA_OK(cudaStreamSynchronize(s));
    *n_out = c;
    return Status::Ok();
}

Status GpuTable::set_rows(const long long* keys, const float* rows, uint64_t n, bool emb_only, void* stream) {
    cudaSetDevice(cfg_.device);
    if (n == 0) return Status::Ok();
    cudaStream_t s = (cudaStream_t)stream;
    Status reserve = reserve_rows(n);
    unsigned* slot_of = nullptr;
    unsigned char* is_new = nullptr;
    PSB_CUDA_OK(cudaMallocAsync(&slot_of, n * sizeof(unsigned), s));
    PSB_CUDA_OK(cudaMallocAsync(&is_new, n, s));
    PSB_CUDA_OK(cudaMemsetAsync(scratch_ + 5, 0, 8, s));
    TableView v = view();
    set_resolve_kernel<<<grid_for(n), kThreads, 0, s>>>(v, keys, n, slot_of, is_new, (unsigned*)(scratch_ + 5));
    const unsigned lanes = lanes_for_dim(cfg_.dim);
    set_write_kernel<<<grid_for(n * lanes), kThreads, 0, s>>>(v, keys, rows, n, slot_of, is_new, emb_only ? 1 : 0);
    unsigned long long st = 0;
    PSB_CUDA_OK(cudaMemcpyAsync(&st, scratch_ + 5, 8, cudaMemcpyDeviceToHost, s));
    refresh_usage_async(s);
    PSB_CUDA_OK(cudaFreeAsync(slot_of, s));
    PSB_CUDA_OK(cudaFreeAsync(is_new, s));
    PSB_CUDA_OK(cudaStreamSynchronize(s));
    if ((unsigned)st == kStOom) {
        healthy_ = false;
        return Status::OOM(reserve.ok() ? "table index or row pool full during set_rows" : reserve.msg());
    }
    return Status::Ok();
}

Status GpuTable::get_rows(const long long* keys, uint64_t n, float* out, int* found, bool emb_only, void* stream) {
    cudaSetDevice(cfg_.device);
    if (n == 0) return Status::Ok();
    const unsigned lanes = lanes_for_dim(cfg_.dim);
    get_rows_kernel<<<grid_for(n * lanes), kThreads, 0, (cudaStream_t)stream>>>(view(), keys, n, out, found,
                                                                                 emb_only ? 1 : 0);
    PSB_CUDA_OK(cudaGetLastError());
    return Status::Ok();
}

Status GpuTable::erase_keys(const long long* keys, uint64_t n, uint64_t* n_erased, void* stream) {
    cudaSetDevice(cfg_.device);
    cudaStream_t s = (cudaStream_t)stream;
    *n_erased = 0;
    if (n == 0) return Status::Ok();
    PSB_CUDA_OK(cudaMemsetAsync(scratch_ + 4, 0, 8, s));
    erase_keys_kernel<<<grid_for(n), kThreads, 0, s>>>(view(), keys, n, scratch_ + 4);
    unsigned long long c = 0;
    PSB_CUDA_OK(cudaMemcpyAsync(&c, scratch_ + 4, 8, cudaMemcpyDeviceToHost, s));
    PSB_CUDA_OK(cudaStreamSynchronize(s));
    *n_erased = c;
    tombstones_ += c;
    return Status::Ok();
}

Status GpuTable::erase_filter(const ShardFilter& f, uint64_t* n_erased, void* stream) {
    cudaSetDevice(cfg_.device);
    cudaStream_t s = (cudaStream_t)stream;
    PSB_CUDA_OK(cudaMemsetAsync(scratch_ + 4, 0, 8, s));
    erase_filter_kernel<<<grid_for(capacity_), kThreads, 0, s>>>(view(), f, capacity_, scratch_ + 4);
    unsigned long long c = 0;
    PSB_CUDA_OK(cudaMemcpyAsync(&c, scratch_ + 4, 8, cudaMemcpyDeviceToHost, s));
    PSB_CUDA_OK(cudaStreamSynchronize(s));
    *n_erased = c;
    tombstones_ += c;
    return Status::Ok();
}

Status GpuTable::erase_if(const ShardFilter& f, int pred_type, long long mod, long long rem, double threshold,
                          uint64_t* n_erased, void* stream) {
    cudaSetDevice(cfg_.device);
    cudaStream_t s = (cudaStream_t)stream;
    if (pred_type == 2 && n_slots_ == 0) return Status::InvalidConfig("erase_if slot0_below: table has no optimizer slot");
    PSB_CUDA_OK(cudaMemsetAsync(scratch_ + 4, 0, 8, s));
    DeviceScan sc{pred_type, mod, rem, threshold, 0};
    scan_kernel<<<grid_for(capacity_), kThreads, 0, s>>>(view(), f, sc, capacity_, scratch_ + 4, nullptr);
    unsigned long long c = 0;
    PSB_CUDA_OK(cudaMemcpyAsync(&c, scratch_ + 4, 8, cudaMemcpyDeviceToHost, s));
    PSB_CUDA_OK(cudaStreamSynchronize(s));
    *n_erased = c;
    tombstones_ += c;
    return Status::Ok();
}

Status GpuTable::reduce_section(const ShardFilter& f, uint32_t section, uint64_t* count, double* sum, double* sum_sq,
                                double* max_abs, void* stream) {
    cudaSetDevice(cfg_.device);
    cudaStream_t s = (cudaStream_t)stream;
    if ((section + 1) * cfg_.dim > stride_) return Status::InvalidConfig("for_each: no such row section");
    double* d = (double*)(scratch_ + 8);   // words 8..11 of the scratch block
    PSB_CUDA_OK(cudaMemsetAsync(d, 0, 4 * sizeof(double), s));
    DeviceScan sc{-1, 1, 0, 0.0, section};
    scan_kernel<<<grid_for(capacity_), kThreads, 0, s>>>(view(), f, sc, capacity_, scratch_ + 4, d);
    double h[4];
    PSB_CUDA_OK(cudaMemcpyAsync(h, d, sizeof(h), cudaMemcpyDeviceToHost, s));
    PSB_CUDA_OK(cudaStreamSynchronize(s));
    *count = (uint64_t)h[0];
    *sum = h[1];
    *sum_sq = h[2];
    *max_abs = h[3];
    return Status::Ok();
}

Status GpuTable::shard_counts(int n_shards, std::vector<uint64_t>* counts, void* stream) {
    cudaSetDevice(cfg_.device);
    cudaStream_t s = (cudaStream_t)stream;
    unsigned long long* d = nullptr;
    PSB_CUDA_OK(cudaMallocAsync(&d, (size_t)n_shards * 8, s));
    PSB_CUDA_OK(cudaMemsetAsync(d, 0, (size_t)n_shards * 8, s));
    shard_count_kernel<<<grid_for(capacity_), kThreads, 0, s>>>(view(), capacity_, n_shards, d);
    counts->assign(n_shards, 0);
    PSB_CUDA_OK(cudaMemcpyAsync(counts->data(), d, (size_t)n_shards * 8, cudaMemcpyDeviceToHost, s));
    PSB_CUDA_OK(cudaFreeAsync(d, s));
    PSB_CUDA_OK(cudaStreamSynchronize(s));
    return Status::Ok();
}

Status GpuTable::store_delta(const OptConfig& opt, void* stream) {
    cudaSetDevice(cfg_.device);
    if (!cfg_.sync_delta) return Status::InvalidConfig("table was created without sync_delta");
    cudaStream_t s = (cudaStream_t)stream;
    unsigned n_touched = 0;
    PSB_CUDA_OK(cudaMemcpyAsync(&n_touched, touched_count_, 4, cudaMemcpyDeviceToHost, s));
    PSB_CUDA_OK(cudaStreamSynchronize(s));
    if (n_touched == 0) return Status::Ok();
    n_touched = std::min(n_touched, touched_cap_);
    const unsigned lanes = lanes_for_dim(cfg_.dim);
    store_delta_kernel<<<grid_for((uint64_t)n_touched * lanes), kThreads, 0, s>>>(view(), opt, n_touched);
    PSB_CUDA_OK(cudaMemsetAsync(touched_count_, 0, 4, s));
    PSB_CUDA_OK(cudaGetLastError());
    return Status::Ok();
}

Status GpuTable::clear_aux(void* stream) {
    cudaSetDevice(cfg_.device);
    clear_aux_kernel<<<grid_for(capacity_, 4), kThreads, 0, (cudaStream_t)stream>>>(slots_, capacity_);
    PSB_CUDA_OK(cudaGetLastError());
    return Status::Ok();
}

Status GpuTable::clear(void* stream) {
    cudaSetDevice(cfg_.device);
    cudaStream_t s = (cudaStream_t)stream;
    fill_slots_kernel<<<grid_for(capacity_, 4), kThreads, 0, s>>>(slots_, capacity_);
    PSB_CUDA_OK(cudaMemsetAsync(scratch_, 0, 64 * sizeof(unsigned long long), s));
    PSB_CUDA_OK(cudaMemsetAsync(touched_bits_, 0, ((max_rows_ + 31) / 32) * 4, s));
    if (dirty_bits_) PSB_CUDA_OK(cudaMemsetAsync(dirty_bits_, 0, ((max_rows_ + 31) / 32) * 4, s));
    PSB_CUDA_OK(cudaMemcpyAsync(scratch_ + 6, &rows_avail_, sizeof(uint32_t), cudaMemcpyHostToDevice, s));
    PSB_CUDA_OK(cudaStreamSynchronize(s));
    host_mirror_[0] = host_mirror_[1] = 0;
    tombstones_ = 0;
    healthy_ = true;
    return Status::Ok();
}

Status GpuTable::rebuild_index(uint64_t new_capacity, void* stream) {
    cudaSetDevice(cfg_.device);
    cudaStream_t s = (cudaStream_t)stream;
    const uint64_t ncap = pow2_ceil(std::max<uint64_t>(new_capacity, 1024));
    const int64_t extra = (int64_t)(ncap * sizeof(Slot));
    PSB_RETURN_IF_ERROR(check_budget((uint64_t)extra));
    Slot* ns = nullptr;
    cudaError_t e = cudaMalloc(&ns, ncap * sizeof(Slot));
    if (e != cudaSuccess) {
        cudaGetLastError();
        return Status::OOM(std::string("cudaMalloc index: ") + cudaGetErrorString(e));
    }
    fill_slots_kernel<<<grid_for(ncap, 4), kThreads, 0, s>>>(ns, ncap);
    PSB_CUDA_OK(cudaMemsetAsync(scratch_ + 5, 0, 8, s));
    rehash_kernel<<<grid_for(capacity_), kThreads, 0, s>>>(slots_, capacity_, ns, ncap - 1, (unsigned*)(scratch_ + 5));
    unsigned long long st = 0;
    PSB_CUDA_OK(cudaMemcpyAsync(&st, scratch_ + 5, 8, cudaMemcpyDeviceToHost, s));
    PSB_CUDA_OK(cudaStreamSynchronize(s));
    if ((unsigned)st != 0) {
        cudaFree(ns);
        return Status::OOM("new index too small for the live keys");
    }
    cudaFree(slots_);
    bytes_ = bytes_ - capacity_ * sizeof(Slot) + ncap * sizeof(Slot);
    slots_ = ns;
    capacity_ = ncap;
    tombstones_ = 0;
    return publish_view();
}

void GpuTable::enable_dirty_tracking() {
    if (dirty_bits_) return;
    cudaSetDevice(cfg_.device);
    const uint64_t bit_words = (max_rows_ + 31) / 32;
    if (cudaMalloc(&dirty_bits_, bit_words * 4) != cudaSuccess) {
        dirty_bits_ = nullptr;
        throw std::runtime_error("GpuTable: cudaMalloc dirty bits failed");
    }
    cudaMemset(dirty_bits_, 0, bit_words * 4);
    bytes_ += bit_words * 4;
    publish_view();
}

Status GpuTable::clear_dirty(void* stream) {
    if (!dirty_bits_) return Status::Ok();
    cudaSetDevice(cfg_.device);
    PSB_CUDA_OK(cudaMemsetAsync(dirty_bits_, 0, ((max_rows_ + 31) / 32) * 4, (cudaStream_t)stream));
    return Status::Ok();
}

}  // namespace psb
