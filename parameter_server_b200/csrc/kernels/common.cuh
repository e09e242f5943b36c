// Device-side building blocks shared by the sm_100a kernels: the open-addressing slot layout, the
// row pool view, bounded waits (grid barrier, cross-GPU flags) and the kernel status word.
//
// Every wait in this file is bounded by a wall-clock limit read from %globaltimer; when a wait runs
// out the kernel records StatusCode::TIMEOUT in its status word and every CTA leaves at its next
// barrier, so the CUDA context stays usable and the host maps the word to Status::Timeout (the
// role of the per-request RPC timeout in pico-ps/common/DistributedAsyncReturn.cpp:46-54).
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

#include "../common/hash.h"

namespace psb {

constexpr int kMaxWorld = 8;
constexpr long long kEmptyKey = (long long)0x8000000000000000ull;      // reserved: never a user key
constexpr long long kTombstoneKey = (long long)0x8000000000000001ull;  // reserved: erased slot
constexpr unsigned kNoRow = 0xFFFFFFFFu;
constexpr unsigned kNoSlot = 0xFFFFFFFFu;
constexpr unsigned kRowPending = 0xFFFFFFFEu;  // transient: a thread is attaching a row to the slot

// Device status word values (low byte = StatusCode).
constexpr unsigned kStOk = 0, kStOom = 3, kStTimeout = 4, kStError = 10;

// One slot of an open-addressing table: 16 bytes so that a probe touches one 32-byte sector.
struct __align__(16) Slot {
    long long key;  // kEmptyKey / kTombstoneKey / user key
    unsigned row;   // row-pool index, kNoRow while the key has no backing row
    unsigned aux;   // scratch for cross-rank leader election during a push; kNoRow at rest
};

// Row pool: rows of `stride` floats ([embedding dim | optimizer slots | optional sync delta]) carved
// from slabs of 2^slab_shift rows; slabs are added by the host without moving existing rows, so
// capacity grows without the 2x rehash spike that the reference's memory governor fights
// (pico-ps/storage/Storage.cpp:154-204).
struct TableView {
    Slot* slots;
    unsigned long long mask;  // slot capacity - 1 (capacity is a power of two)
    float* const* slabs;      // device array of slab base pointers
    unsigned slab_shift;
    unsigned stride;          // floats per row
    unsigned dim;             // embedding floats per row
    unsigned n_opt_slots;     // optimizer slot count (each dim floats)
    unsigned has_delta;       // 1 when rows carry a sync-push delta section after the slots
    const unsigned* rows_avail;  // device word: rows backed by memory (the host raises it when it adds slabs, so a
                                 // launch captured in a CUDA graph sees the growth)
    unsigned max_probe;
    unsigned* row_bump;       // next never-used row
    unsigned* free_rows;      // stack of recycled rows
    int* free_count;
    unsigned long long* n_items;  // live keys
    unsigned* touched_bits;   // 1 bit per row: row is in the sync-push touched list
    unsigned* touched_list;
    unsigned* touched_count;
    unsigned touched_cap;
    unsigned* dirty_bits;     // 1 bit per row: row changed since the last incremental sync (nullptr = off)
    // row initialisation
    unsigned long long init_seed;
    float init_range;
    float slot_init[2];

    __device__ __forceinline__ float* row_ptr(unsigned row) const {
        return slabs[row >> slab_shift] + (size_t)(row & ((1u << slab_shift) - 1)) * stride;
    }
};

// ------------------------------------------------------------------------------------------------
// memory-order helpers
__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_relaxed_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Control block of one kernel family on one GPU (device global memory, zero-initialised).
struct KernelCtl {
    unsigned bar_count;  // grid barrier arrivals
    unsigned bar_gen;    // grid barrier generation
    unsigned status;     // first error (StatusCode) seen by the kernel, 0 = OK
    unsigned where;      // site id of the wait or check that failed
    unsigned done_blocks;
    unsigned epoch;      // number of completed calls; a kernel runs as call epoch+1 and publishes it at its end,
                         // so a launch captured in a CUDA graph advances the epoch on every replay
    unsigned soft;       // first NON-fatal condition (OUT_OF_MEMORY: a key without a row); the call still runs to
                         // its end, so scratch state and epochs stay consistent; the host reports and clears it
    unsigned soft_where;
    unsigned arrive[4];  // "last CTA publishes" counters, one per hand-off point of a kernel
    unsigned pad[4];
};

// Fatal: every CTA leaves at its next barrier. The word is sticky until the host resets the engine.
__device__ __forceinline__ void set_status(KernelCtl* ctl, unsigned code, unsigned where) {
    if (atomicCAS(&ctl->status, 0u, code) == 0u) ctl->where = where;
}
// Non-fatal (memory pressure): recorded, the call completes. Reads of a row-less key see the initial value,
// writes to it are dropped - the analogue of the reference answering OUT_OF_MEMORY while a shard's overflow
// list is non-empty (pico-ps/operator/SparsePullOperator.h:195-199).
__device__ __forceinline__ void set_soft_status(KernelCtl* ctl, unsigned code, unsigned where) {
    if (atomicCAS(&ctl->soft, 0u, code) == 0u) ctl->soft_where = where;
}

// Hand-off without a grid barrier: every CTA calls this after its last store of a phase; it returns true
// (uniformly per CTA) in the CTA that arrived last, which may then publish the phase's flags to the peers.
// The fences make every CTA's stores visible system-wide before the flag can be written.
__device__ __forceinline__ bool cta_arrive_last(unsigned* counter, unsigned nblocks) {
    __shared__ unsigned s_last_arrival;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned prev = atomicAdd(counter, 1u);
        const unsigned last = (prev == nblocks - 1u) ? 1u : 0u;
        if (last) {
            *((volatile unsigned*)counter) = 0;  // re-armed for the next call (ordered by the stream)
            __threadfence_system();
        }
        s_last_arrival = last;
    }
    __syncthreads();
    return s_last_arrival != 0u;
}

// Bounded grid-wide barrier for cooperative launches. Returns false (uniformly per CTA) when the
// wait ran out or another CTA already failed; the caller must then return from the kernel.
__device__ __forceinline__ bool grid_sync(KernelCtl* ctl, unsigned nblocks, unsigned long long limit_ns,
                                          unsigned where) {
    __syncthreads();
    int ok = 1;
    if (threadIdx.x == 0) {
        unsigned gen = ld_acquire_gpu(&ctl->bar_gen);
        __threadfence();
        unsigned arrived = atomicAdd(&ctl->bar_count, 1u) + 1u;
        if (arrived == nblocks) {
            ctl->bar_count = 0;
            __threadfence();
            atomicAdd(&ctl->bar_gen, 1u);
        } else {
            unsigned long long t0 = global_timer_ns();
            unsigned spins = 0;
            while (ld_acquire_gpu(&ctl->bar_gen) == gen) {
                if ((++spins & 63u) == 0) {
                    // a CTA that failed leaves without arriving: do not wait for it
                    if (ld_acquire_gpu(&ctl->status) != 0u) {
                        ok = 0;
                        break;
                    }
                    if (global_timer_ns() - t0 > limit_ns) {
                        set_status(ctl, kStTimeout, where);
                        ok = 0;
                        break;
                    }
                }
            }
        }
        __threadfence();
        if (ld_acquire_gpu(&ctl->status) != 0u) ok = 0;
    }
    return __syncthreads_and(ok) != 0;
}

// Bounded wait until *flag >= target (flags are monotonically increasing epochs written by a peer
// GPU with st.release.sys). Called by ONE thread; returns false on time-out.
__device__ __forceinline__ bool wait_flag_ge(const unsigned* flag, unsigned target, unsigned long long limit_ns) {
    unsigned long long t0 = global_timer_ns();
    unsigned spins = 0;
    while ((int)(ld_acquire_sys(flag) - target) < 0) {
        if ((++spins & 15u) == 0) {
            if (global_timer_ns() - t0 > limit_ns) return false;
            __nanosleep(64);
        }
    }
    return true;
}

// ------------------------------------------------------------------------------------------------
// Find `key` or claim an empty slot for it. Returns the slot index, or kNoSlot when the probe limit is
// hit (index full). `inserted` tells whether THIS call created the entry. With insert=false a
// missing key returns kNoSlot.
__device__ __forceinline__ unsigned table_find_or_insert(const TableView& t, long long key, bool insert,
                                                         bool* inserted) {
    *inserted = false;
    unsigned long long h = slot_hash(key) & t.mask;
    for (unsigned probe = 0; probe < t.max_probe; ++probe) {
        long long cur = *((volatile long long*)&t.slots[h].key);
        if (cur == key) return (unsigned)h;
        if (cur == kEmptyKey) {
            if (!insert) return kNoSlot;
            long long prev = (long long)atomicCAS((unsigned long long*)&t.slots[h].key,
                                                  (unsigned long long)kEmptyKey, (unsigned long long)key);
            if (prev == kEmptyKey) {
                *inserted = true;
                return (unsigned)h;
            }
            if (prev == key) return (unsigned)h;
        }
        h = (h + 1) & t.mask;
    }
    return kNoSlot;
}

// Give the entry in `slot` a backing row if it has none. Returns true when THIS call attached the
// row (the caller must then initialise it). Rows come from the free stack first, then the bump
// pointer; when the pool is exhausted the entry stays row-less (reads see the init value, writes
// are dropped and the kernel reports OUT_OF_MEMORY), the analogue of the reference parking items in
// the shard's overflow vector (pico-ps/operator/SparsePushOperator.h:257-259).
__device__ __forceinline__ bool table_attach_row(const TableView& t, unsigned slot, bool* oom) {
    if (*((volatile unsigned*)&t.slots[slot].row) != kNoRow) return false;
    // Claim the attachment first so that only one thread allocates for this slot; everybody else
    // reads the row index after the next grid barrier.
    if (atomicCAS(&t.slots[slot].row, kNoRow, kRowPending) != kNoRow) return false;
    unsigned row = kNoRow;
    // the free stack is only popped in this kernel family, so an empty stack stays empty: skip its atomics
    int f = (*((volatile int*)t.free_count) > 0) ? atomicSub(t.free_count, 1) : 0x7fffffff;
    if (f > 0 && f != 0x7fffffff) {
        row = t.free_rows[f - 1];
    } else {
        if (f != 0x7fffffff) atomicAdd(t.free_count, 1);
        unsigned b = atomicAdd(t.row_bump, 1u);
        if (b < *((volatile const unsigned*)t.rows_avail)) {
            row = b;
        } else {
            atomicSub(t.row_bump, 1u);
            *oom = true;
        }
    }
    *((volatile unsigned*)&t.slots[slot].row) = row;  // kNoRow again when the pool is exhausted
    return row != kNoRow;
}

// Cooperative row helpers: `lanes` consecutive lanes of a warp (a power of two <= 32) handle one row
// with 16-byte accesses; `lane` is the index inside the group.
__device__ __forceinline__ void row_init(const TableView& t, float* row, long long key, unsigned lane,
                                         unsigned lanes) {
    for (unsigned d = lane * 4; d < t.dim; d += lanes * 4) {
        float4 v;
        v.x = init_uniform(key, d + 0, t.init_seed, t.init_range);
        v.y = init_uniform(key, d + 1, t.init_seed, t.init_range);
        v.z = init_uniform(key, d + 2, t.init_seed, t.init_range);
        v.w = init_uniform(key, d + 3, t.init_seed, t.init_range);
        *(float4*)(row + d) = v;
    }
    for (unsigned s = 0; s < t.n_opt_slots; ++s) {
        const float iv = s == 0 ? t.slot_init[0] : t.slot_init[1];   // static indices: the view stays in registers
        float4 v = make_float4(iv, iv, iv, iv);
        for (unsigned d = lane * 4; d < t.dim; d += lanes * 4) *(float4*)(row + (s + 1) * t.dim + d) = v;
    }
    if (t.has_delta) {
        float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
        for (unsigned d = lane * 4; d < t.dim; d += lanes * 4)
            *(float4*)(row + (t.n_opt_slots + 1) * t.dim + d) = z;
    }
}

__host__ __device__ __forceinline__ unsigned lanes_for_dim(unsigned dim) {
    unsigned v = dim / 4;
    unsigned l = 1;
    while (l < v && l < 32) l <<= 1;
    return l;
}

}  // namespace psb
