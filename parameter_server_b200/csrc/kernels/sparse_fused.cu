// Fused sparse pull and push for sm_100a: ONE cooperative kernel per call does the client side, the
// transport and the server side of the reference's sparse operators, with the transport being plain
// peer stores over NVLink/NVSwitch issued from inside the kernel.
//
// fused_pull_kernel  (pico-ps/operator/SparsePullOperator.h:81-110 generate_request_data,
//                     :112-154 generate_request, :156-254 apply_request, :278-304 fill_pull_items)
//   P1  dedup the key batch (warp-local match first, then an open-addressing scratch table), partition the
//       unique keys by jump_consistent_hash(murmur(key)) -> shard -> owning GPU, stage per-owner key lists
//   P2  copy the staged lists into the owners' mailboxes (coalesced peer stores); the CTA that finishes last
//       publishes count + flag to every owner (no grid barrier)
//   P3  owner: resolve the local requester's keys at once, then wait for every source's flag and resolve
//       theirs: find-or-insert in the local table, attach + initialise rows of new keys, store each row
//       (fp32, or bf16 when the consumer wants bf16) into the requesting GPU's row buffer; last CTA publishes
//   P5  consumer: resolve position -> row while the remote rows are in flight, wait for every owner's flag,
//       un-dedup and sum/mean-pool rows into the activation buffer; leave behind the "plan" (inverse map,
//       per-owner lists, owner-side slots) for the push
// fused_push_kernel  (pico-ps/operator/SparsePushOperator.h:109-154 generate_request_data,
//                     :197-276 async apply, :278-320 sync apply, :377-409 merge before store)
//   Q0  owner: chain the received entries that name the same table row (one entry per source rank)
//   Q1  segment-sum the gradients of duplicate keys into one row per unique key
//   Q2  store the merged gradient rows into the owners' mailboxes, last CTA publishes the flag
//   Q3  owner: wait for every source; the head entry of each row's chain folds the sources' gradients in
//       rank order (reproducible) and applies the optimizer once per row (or accumulates into the sync-push
//       delta section); last CTA acknowledges the sources. With replication the head also appends (key, folded
//       gradient) to a log in the memory of the GPU that mirrors this rank's shards
//   Q4  replica holder: wait for the mirrored rank's log, find-or-insert its keys in the mirror table and apply the
//       same optimizer step to the mirror rows, so a replica is exact after every push
//       (pico-ps/operator/SparsePushOperator.h:161-168: a push reaches every node that hosts the shard)
// A kernel on one GPU waits for kernels on the other GPUs; each GPU runs exactly one of them per
// call, all waits are bounded, and with world == 1 no cross-GPU wait is executed at all. The grid is a
// parameter: a full-residency grid when the kernel runs alone, a bounded CTA budget when it shares the SMs
// with the dense GEMMs of the same training step on another stream.
#include <cooperative_groups.h>
#include <cuda_bf16.h>

#include "sparse_fused.h"

namespace psb {

namespace {

// Two CTA shapes, same code: 256 threads (four CTAs per SM; fastest on an idle GPU, whose large batches like many small
// row caches) and 1024 threads (one CTA fills an SM: the shape for sharing the GPU by SMs with another kernel).
constexpr int kThreadsSmall = 256;
constexpr int kThreadsWide = 1024;
// block-local accumulation of hot gradient rows in the push (Q1)
// push, per CTA: counting table of kHotSlots keys, at most kHotRows rows cached (FusedArgs::hot_rows may ask for fewer)
template <int kThreads> struct HotCfg {
    static constexpr int kHotSlots = kThreads >= 1024 ? 2048 : 512;
    static constexpr int kHotRows = kThreads >= 1024 ? 64 : 24;
};
constexpr unsigned kHotMaxDim = 128;
template <int kThreads> constexpr size_t push_smem_bytes() { return (size_t)HotCfg<kThreads>::kHotRows * kHotMaxDim * sizeof(float); }

enum Where : unsigned {
    W_P1 = 1, W_P2, W_KEYFLAG, W_P3A, W_P3B, W_P3C, W_ROWFLAG, W_MAILBOX_OVERFLOW, W_INDEX_FULL, W_POOL_FULL,
    W_DEDUP_FULL, W_RESERVED_KEY,
    W_Q1 = 32, W_ACK, W_Q2, W_GRADFLAG, W_Q3A, W_Q3B, W_NOROW, W_REPACK, W_REPFLAG, W_REP_A, W_REP_FULL,
};

// Initial value of four columns of a key that has no row (read-only pulls of unknown keys): rare, so out of line in
// the gather loops, whose bodies should stay small.
__device__ __noinline__ float4 init4_rare(long long key, unsigned d, unsigned long long seed, float range) {
    float4 v;
    v.x = init_uniform(key, d + 0, seed, range);
    v.y = init_uniform(key, d + 1, seed, range);
    v.z = init_uniform(key, d + 2, seed, range);
    v.w = init_uniform(key, d + 3, seed, range);
    return v;
}
__device__ __forceinline__ float4 init4(const TableView& t, long long key, unsigned d) {
    float4 v;
    v.x = init_uniform(key, d + 0, t.init_seed, t.init_range);
    v.y = init_uniform(key, d + 1, t.init_seed, t.init_range);
    v.z = init_uniform(key, d + 2, t.init_seed, t.init_range);
    v.w = init_uniform(key, d + 3, t.init_seed, t.init_range);
    return v;
}

__device__ __forceinline__ float4 unpack_bf16x4(const uint2& p) {
    const __nv_bfloat162 lo = *(const __nv_bfloat162*)&p.x, hi = *(const __nv_bfloat162*)&p.y;
    const float2 a = __bfloat1622float2(lo), b = __bfloat1622float2(hi);
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ uint2 pack_bf16x4(const float4& v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 p;
    p.x = *(const unsigned*)&lo;
    p.y = *(const unsigned*)&hi;
    return p;
}

// The update rule on four coordinates, any rule, out of line (for paths that are not worth four inlined copies).
__device__ __noinline__ void opt_update4_any(const OptConfig& opt, float4& w, float4& s0, float4& s1, const float4& g) {
    opt_update(opt, w.x, s0.x, s1.x, g.x);
    opt_update(opt, w.y, s0.y, s1.y, g.y);
    opt_update(opt, w.z, s0.z, s1.z, g.z);
    opt_update(opt, w.w, s0.w, s1.w, g.w);
}

// Each CTA waits until every peer's flag in `flags` (local memory, written remotely) reached `target`.
__device__ __forceinline__ bool wait_all_flags(const unsigned* flags, unsigned target, const FusedArgs& a,
                                               unsigned where) {
    int ok = 1;
    if (threadIdx.x < (unsigned)a.world && (int)threadIdx.x != a.rank) {
        if (!wait_flag_ge(flags + threadIdx.x, target, a.limit_ns)) {
            set_status(a.ctl, kStTimeout, where);
            ok = 0;
        }
    }
    if (ld_acquire_gpu(&a.ctl->status) != 0u) ok = 0;
    return __syncthreads_and(ok) != 0;
}

// Row source of one key position in P5.
struct RowSrc {
    const float* f32;            // table row or fp32 row returned by a remote owner
    const __nv_bfloat16* b16;    // bf16 row returned by a remote owner
};

}  // namespace

// Phase timestamps (the kernel-side counterpart of the reference's VTIMER scopes): CTA 0 records
// %globaltimer when it enters each phase.
// Per-CTA stamps (same switch): when each CTA started and when it reached a grid barrier; the spread tells a phase
// that is bound by throughput (all CTAs arrive late) from one that waits for stragglers.
#define PROF_CTA(k)                                                                                              \
    do {                                                                                                         \
        if (a.prof != nullptr && threadIdx.x == 0 && blockIdx.x < kProfMaxCtas)                                  \
            a.prof[16 + (k) * kProfMaxCtas + blockIdx.x] = global_timer_ns();                                    \
    } while (0)
#define PROF(slot)                                                                 \
    do {                                                                           \
        if (a.prof != nullptr && blockIdx.x == 0 && threadIdx.x == 0) a.prof[slot] = global_timer_ns(); \
    } while (0)

// MULTI = false: the single-rank variant; `W` is then the constant 1 and all code for peers drops out of the kernel
// (less code in the phase loops, which the instruction fetch of these long kernels feels).
template <int kThreads, bool MULTI>
__global__ void __launch_bounds__(kThreads, 1024 / kThreads) fused_pull_kernel(const FusedArgs a) {
    const unsigned nblocks = gridDim.x;
    const unsigned tid = blockIdx.x * kThreads + threadIdx.x;
    const unsigned nthreads = nblocks * kThreads;
    // a fatal status of an earlier call stays until the host resets the engine: do nothing, touch nothing
    if (ld_acquire_gpu(&a.ctl->status) != 0u) return;
    const unsigned epoch = *((volatile unsigned*)&a.ctl->epoch) + 1u;
    const unsigned par = epoch & 1u;
    unsigned* cnt = a.counters + par * 16;
    unsigned* send_cnt = cnt + 4;
    unsigned* in_cnt = a.in_cnt + par * kMaxWorld;
    const int me = a.rank;
    const int W = MULTI ? a.world : 1;
    const unsigned C = a.C;
    const TableView T = *a.table;
    const PeerBufs& mine = a.peer[me];
    const unsigned lanes = lanes_for_dim(a.dim);
    const unsigned group = tid / lanes, ngroups = nthreads / lanes, lane = tid % lanes;
    const bool out16 = (a.flags & FUSED_OUT_BF16) != 0;
    const bool rows16 = out16 && a.bag_size == 1;  // remote rows travel as bf16

    __shared__ unsigned s_pre[kMaxWorld + 1];

    // ---- P1: dedup + partition ------------------------------------------------------------------
    // Duplicates inside a warp are folded with a match before anything touches memory (the head of a Zipf
    // batch otherwise sends many lanes to one slot); counters are bumped once per warp and owner (ballot /
    // match), not once per key: same-address atomics serialise in L2 and would otherwise bound the phase.
    PROF(0);
    PROF_CTA(0);
    const unsigned wlane = threadIdx.x & 31u;
    const unsigned long long probe_limit = a.dmask + 1ull;
    const unsigned dup_tag = (epoch << 1) | 1u;
    // Unique ids and per-owner mailbox positions are handed out per CTA: the warps add their counts to shared
    // counters, one thread per counter fetches the CTA's base from global memory, and every winner adds its rank
    // inside the CTA. One global atomic per CTA and counter instead of one per warp: all of them hit the same two
    // or three addresses, and that many same-address atomics serialised in L2 left the last warps waiting.
    __shared__ unsigned s_cnt[kMaxWorld + 1];    // [0] uniques, [1 + o] keys for owner o (this iteration)
    __shared__ unsigned s_base[kMaxWorld + 1];
    if (threadIdx.x <= (unsigned)kMaxWorld) s_cnt[threadIdx.x] = 0;
    __syncthreads();
    const unsigned n_ceil = (a.n + kThreads - 1) / kThreads * kThreads;
    for (unsigned i0 = blockIdx.x * kThreads; i0 < n_ceil; i0 += nthreads) {   // trip count uniform in the CTA
        const unsigned i = i0 + threadIdx.x;
        bool active = i < a.n;
        long long key = kEmptyKey;
        if (active) {
            key = a.keys[i];
            if (key <= kTombstoneKey) {  // the two reserved values can never be stored
                set_status(a.ctl, kStError, W_RESERVED_KEY);
                active = false;
                key = kEmptyKey;
            }
        }
        const unsigned same = __match_any_sync(0xffffffffu, key);
        const int klead = __ffs(same) - 1;
        unsigned h = 0;
        bool won = false;
        if (active && (int)wlane == klead) {
            unsigned long long hh = slot_hash(key) & a.dmask;
            unsigned long long probes = 0;
            for (; probes < probe_limit; ++probes) {
                long long cur = *((volatile long long*)&a.dedup[hh].key);
                if (cur == key) break;
                if (cur == kEmptyKey) {
                    long long prev = (long long)atomicCAS((unsigned long long*)&a.dedup[hh].key,
                                                          (unsigned long long)kEmptyKey, (unsigned long long)key);
                    if (prev == kEmptyKey) { won = true; break; }
                    if (prev == key) break;
                }
                hh = (hh + 1) & a.dmask;
            }
            // A key met more than once (by another warp before, or by several lanes of this warp) is tagged with
            // this call's epoch: the push then knows which gradient rows need summing and which are plain copies.
            // Nobody ever clears the tag: a value left by an earlier call differs from the current one. Read before
            // write: the head keys of a skewed batch are met by thousands of warps, and that many stores to one
            // address serialise in L2 where the reads (same sector as the key just probed) do not.
            if (probes < probe_limit && (!won || __popc(same) > 1) &&
                *((volatile unsigned*)&a.dedup[hh].aux) != dup_tag)
                a.dedup[hh].aux = dup_tag;
            // the table holds >= 2n slots and is emptied by every call; a full table means an earlier call was
            // cut short or two calls overlap on one engine
            if (probes == probe_limit) set_status(a.ctl, kStError, W_DEDUP_FULL);
            h = (unsigned)hh;
        }
        h = __shfl_sync(0xffffffffu, h, klead);
        if (active) a.pos_slot[i] = h;
        const unsigned wmask = __ballot_sync(0xffffffffu, won);
        const int owner = won ? a.shard_owner[sparse_shard_of(key, a.n_shards)] : -1;
        // rank of this winner among the CTA's winners (all, and of the same owner)
        unsigned uoff = 0, poff = 0;
        const unsigned peers = __match_any_sync(0xffffffffu, owner);
        if (wmask) {
            const int uleader = __ffs(wmask) - 1;
            if ((int)wlane == uleader) uoff = atomicAdd(&s_cnt[0], (unsigned)__popc(wmask));
            uoff = __shfl_sync(0xffffffffu, uoff, uleader) + __popc(wmask & ((1u << wlane) - 1u));
            const int pleader = __ffs(peers) - 1;
            if (won && (int)wlane == pleader) poff = atomicAdd(&s_cnt[1 + owner], (unsigned)__popc(peers));
            poff = __shfl_sync(0xffffffffu, poff, pleader) + __popc(peers & ((1u << wlane) - 1u));
        }
        __syncthreads();
        if (threadIdx.x <= (unsigned)W) {
            const unsigned c = s_cnt[threadIdx.x];
            s_base[threadIdx.x] = c ? atomicAdd(threadIdx.x == 0 ? &cnt[0] : &send_cnt[threadIdx.x - 1], c) : 0u;
            s_cnt[threadIdx.x] = 0;
        }
        __syncthreads();
        if (won) {
            const unsigned u = s_base[0] + uoff;
            const unsigned p = s_base[1 + owner] + poff;
            if (p < C) {
                a.send_keys[(size_t)owner * C + p] = key;
                a.send_ret[(size_t)owner * C + p] = u;
            } else {
                set_status(a.ctl, kStError, W_MAILBOX_OVERFLOW);
            }
            a.dedup[h].row = u;
            a.uniq_slot[u] = h;
            a.uniq_row[u] = (owner == me) ? kNoSlot : kRemoteRow;
        }
    }
    PROF_CTA(1);
    if (!grid_sync(a.ctl, nblocks, a.limit_ns, W_P1)) return;

    // ---- P2: ship staged key lists to the owners ------------------------------------------------
    PROF(1);
    if (W > 1) {
        if (threadIdx.x == 0) {
            unsigned acc = 0;
            for (int o = 0; o < W; ++o) {
                s_pre[o] = acc;
                acc += (o == me) ? 0u : min(send_cnt[o], C);
            }
            s_pre[W] = acc;
        }
        __syncthreads();
        const unsigned total = s_pre[W];
        // every rank starts with its right-hand neighbour and walks the ring, so that at any moment the ranks
        // write to different peers (starting at peer 0 everywhere would funnel all traffic into one link)
        const unsigned rot = s_pre[(me + 1) % W];
        for (unsigned e0 = tid; e0 < total; e0 += nthreads) {
            unsigned e = e0 + rot;
            if (e >= total) e -= total;
            int o = 0;
            while (e >= s_pre[o + 1]) ++o;
            const unsigned p = e - s_pre[o];
            a.peer[o].mail_keys[(size_t)me * C + p] = a.send_keys[(size_t)o * C + p];
            a.peer[o].mail_ret[(size_t)me * C + p] = a.send_ret[(size_t)o * C + p];
        }
        if (cta_arrive_last(&a.ctl->arrive[0], nblocks)) {
            if (threadIdx.x < (unsigned)W && (int)threadIdx.x != me) {
                const int o = threadIdx.x;
                a.peer[o].key_cnt[me] = min(send_cnt[o], C);
                __threadfence_system();
                st_release_sys(&a.peer[o].key_flag[me], epoch);
            }
        }
        __syncthreads();  // s_pre is rewritten below
    }

    // ---- P3a: resolve keys in the local table: the local requester's list first (nothing to wait for), then
    // the lists of the other source ranks as one flattened range ---------------------------------------
    const bool do_insert = (a.flags & FUSED_INSERT) != 0;
    PROF(2);
    for (int pass = 0; pass < (W > 1 ? 2 : 1); ++pass) {
        unsigned total_e;
        if (pass == 0) {
            total_e = min(send_cnt[me], C);
        } else {
            if (!wait_all_flags(mine.key_flag, epoch, a, W_KEYFLAG)) return;
            if (threadIdx.x == 0) {
                unsigned acc = 0;
                for (int r = 0; r < W; ++r) {
                    s_pre[r] = acc;
                    acc += (r == me) ? 0u : min(ld_relaxed_sys(&mine.key_cnt[r]), C);
                }
                s_pre[W] = acc;
            }
            __syncthreads();
            total_e = s_pre[W];
            if (blockIdx.x == 0 && threadIdx.x < (unsigned)W)
                in_cnt[threadIdx.x] = ((int)threadIdx.x == me) ? min(send_cnt[me], C)
                                                               : s_pre[threadIdx.x + 1] - s_pre[threadIdx.x];
        }
        for (unsigned e0 = (tid & ~31u); e0 < total_e; e0 += nthreads) {
            const unsigned e = e0 + wlane;
            bool attached = false, inserted = false;
            unsigned slot = kNoSlot;
            if (e < total_e) {
                int r = me;
                unsigned p = e;
                if (pass == 1) {
                    r = 0;
                    while (e >= s_pre[r + 1]) ++r;
                    p = e - s_pre[r];
                }
                const long long key = (r == me) ? a.send_keys[(size_t)me * C + p] : mine.mail_keys[(size_t)r * C + p];
                slot = table_find_or_insert(T, key, do_insert, &inserted);
                if (slot == kNoSlot) {
                    if (do_insert) set_soft_status(a.ctl, kStOom, W_INDEX_FULL);
                } else if (do_insert) {
                    bool oom = false;
                    attached = table_attach_row(T, slot, &oom);
                    if (oom) set_soft_status(a.ctl, kStOom, W_POOL_FULL);
                }
                a.res_slot[(size_t)r * C + p] = slot;
                // a local requester reads the table directly in P5: it only needs the slot
                if (r == me) a.uniq_row[a.send_ret[(size_t)me * C + p]] = slot;
            }
            // list of freshly attached rows and the live-key counter: one atomic per warp each
            const unsigned amask = __ballot_sync(0xffffffffu, attached);
            if (amask) {
                const int al = __ffs(amask) - 1;
                unsigned base = 0;
                if ((int)wlane == al) base = atomicAdd(&cnt[1], (unsigned)__popc(amask));
                base = __shfl_sync(0xffffffffu, base, al);
                if (attached) a.new_list[base + __popc(amask & ((1u << wlane) - 1u))] = slot;
            }
            const unsigned imask = __ballot_sync(0xffffffffu, inserted);
            if (imask && (int)wlane == __ffs(imask) - 1) atomicAdd(T.n_items, (unsigned long long)__popc(imask));
        }
    }
    if (W == 1 && blockIdx.x == 0 && threadIdx.x == 0) in_cnt[0] = min(send_cnt[0], C);
    PROF_CTA(2);
    if (!grid_sync(a.ctl, nblocks, a.limit_ns, W_P3A)) return;

    // ---- P3b: initialise the rows attached by this call -----------------------------------------
    PROF(3);
    const unsigned n_new = cnt[1];
    if (n_new > 0) {
        for (unsigned j = group; j < n_new; j += ngroups) {
            const unsigned slot = a.new_list[j];
            const unsigned row = T.slots[slot].row;
            row_init(T, T.row_ptr(row), T.slots[slot].key, lane, lanes);
        }
        if (!grid_sync(a.ctl, nblocks, a.limit_ns, W_P3B)) return;
    }

    // ---- P3c: return rows to the remote requesters by peer stores -------------------------------------
    PROF(4);
    if (W > 1) {
        if (a.flags & FUSED_COPY_ROWS) {
            // one lane group per entry, two entries in flight; every owner starts with the requester to its right
            // and walks the ring: if all owners served requester 0 first, its one link would carry everything
            // while the others idle
            const unsigned total_rem = s_pre[W];
            const unsigned rot = s_pre[(me + 1) % W];
            constexpr int kIn = 2;
            for (unsigned e0 = group; e0 < total_rem; e0 += ngroups * kIn) {
                const float* src[kIn];
                long long key[kIn];
                size_t dst_off[kIn];
                int rr[kIn];
                bool act[kIn];
#pragma unroll
                for (int k = 0; k < kIn; ++k) {
                    unsigned e = e0 + (unsigned)k * ngroups;
                    act[k] = e < total_rem;
                    src[k] = nullptr;
                    key[k] = 0;
                    dst_off[k] = 0;
                    rr[k] = 0;
                    if (!act[k]) continue;
                    e += rot;
                    if (e >= total_rem) e -= total_rem;
                    int r = 0;
                    while (e >= s_pre[r + 1]) ++r;
                    const unsigned p = e - s_pre[r];
                    const unsigned slot = a.res_slot[(size_t)r * C + p];
                    unsigned row = kNoRow;
                    if (slot != kNoSlot) row = T.slots[slot].row;
                    rr[k] = r;
                    dst_off[k] = (size_t)mine.mail_ret[(size_t)r * C + p] * a.dim;
                    if (row < kRowPending) src[k] = T.row_ptr(row);
                    else key[k] = mine.mail_keys[(size_t)r * C + p];
                }
                for (unsigned d = lane * 4; d < a.dim; d += lanes * 4) {
                    float4 v[kIn];
#pragma unroll
                    for (int k = 0; k < kIn; ++k)
                        if (act[k]) v[k] = src[k] != nullptr ? *(const float4*)(src[k] + d) : init4_rare(key[k], d, T.init_seed, T.init_range);
#pragma unroll
                    for (int k = 0; k < kIn; ++k) {
                        if (!act[k]) continue;
                        if (rows16) *(uint2*)((__nv_bfloat16*)a.peer[rr[k]].rows_in + dst_off[k] + d) = pack_bf16x4(v[k]);
                        else *(float4*)(a.peer[rr[k]].rows_in + dst_off[k] + d) = v[k];
                    }
                }
            }
        }
        // the row flag also tells the requester that its key mailbox on this owner may be overwritten
        if (cta_arrive_last(&a.ctl->arrive[1], nblocks)) {
            if (threadIdx.x < (unsigned)W && (int)threadIdx.x != me)
                st_release_sys(&a.peer[threadIdx.x].row_flag[me], epoch);
        }
    }

    // ---- P5 (consumer): un-dedup + pool into the activation buffer ------------------------------
    PROF(5);
    // Every CTA owns a contiguous range of bags: pass (a) resolves the index chain
    // position -> dedup slot -> unique id -> table slot -> row with one THREAD per position (independent loads
    // in flight; it needs nothing from the peers, so it runs while their rows are still arriving), pass (b)
    // gathers and pools with one lane group per bag. Only a CTA barrier in between.
    const unsigned L = a.bag_size;
    {
        const unsigned nbags = a.n / L;
        const unsigned per = (nbags + nblocks - 1) / nblocks;
        const unsigned b_lo = min(nbags, blockIdx.x * per), b_hi = min(nbags, b_lo + per);
        for (unsigned i = b_lo * L + threadIdx.x; i < b_hi * L; i += kThreads) {
            const unsigned h = a.pos_slot[i];
            const Slot ds = a.dedup[h];
            const unsigned u = ds.row;
            // bit 31 of the inverse map: the key occurs more than once in this batch
            a.inverse[i] = (int)(u | (ds.aux == dup_tag ? kDupBit : 0u));
            const unsigned s = a.uniq_row[u];
            unsigned row = s;  // kRemoteRow stays
            if (!MULTI || s != kRemoteRow) row = (s == kNoSlot) ? kNoRow : T.slots[s].row;
            a.pos_slot[i] = row;  // from here on: the row of position i
        }
        if (W > 1) {
            if (!wait_all_flags(mine.row_flag, epoch, a, W_ROWFLAG)) return;
        } else {
            __syncthreads();
        }
        if (a.flags & FUSED_COPY_ROWS) {
            const float scale = (a.flags & FUSED_MEAN) ? 1.0f / (float)L : 1.0f;
            const unsigned lgroup = threadIdx.x / lanes, lgroups = kThreads / lanes;
            float* outf = (float*)a.out;
            __nv_bfloat16* outh = (__nv_bfloat16*)a.out;
            const __nv_bfloat16* rin16 = (const __nv_bfloat16*)mine.rows_in;
            if (L == 1) {
                // one key per bag (the common embedding lookup): four bags per lane group and iteration, so that
                // four row loads are in flight before the first store (the loop is bound by load latency)
                constexpr int kBags = 4;
                for (unsigned b0 = b_lo; b0 < b_hi; b0 += lgroups * kBags) {
                    unsigned bb[kBags];
                    RowSrc src[kBags];
                    bool act[kBags];
#pragma unroll
                    for (int k = 0; k < kBags; ++k) {
                        bb[k] = b0 + (unsigned)k * lgroups + lgroup;
                        act[k] = bb[k] < b_hi;
                        src[k].f32 = nullptr;
                        src[k].b16 = nullptr;
                        if (act[k]) {
                            const unsigned row = a.pos_slot[bb[k]];
                            if (MULTI && row == kRemoteRow) {
                                const size_t uq = (unsigned)a.inverse[bb[k]] & ~kDupBit;
                                if (rows16) src[k].b16 = rin16 + uq * a.dim;
                                else src[k].f32 = mine.rows_in + uq * a.dim;
                            } else if (row < kRowPending) {
                                src[k].f32 = T.row_ptr(row);
                            }
                        }
                    }
                    for (unsigned d = lane * 4; d < a.dim; d += lanes * 4) {
                        float4 v[kBags];
                        uint2 hv[kBags];
#pragma unroll
                        for (int k = 0; k < kBags; ++k) {
                            if (!act[k]) continue;
                            if (MULTI && src[k].b16 != nullptr) hv[k] = *(const uint2*)(src[k].b16 + d);
                            else v[k] = src[k].f32 != nullptr ? *(const float4*)(src[k].f32 + d) : init4_rare(a.keys[bb[k]], d, T.init_seed, T.init_range);
                        }
#pragma unroll
                        for (int k = 0; k < kBags; ++k) {
                            if (!act[k]) continue;
                            if (out16) {
                                if (!MULTI || src[k].b16 == nullptr) hv[k] = pack_bf16x4(v[k]);
                                *(uint2*)(outh + (size_t)bb[k] * a.dim + d) = hv[k];
                            } else {
                                *(float4*)(outf + (size_t)bb[k] * a.dim + d) = v[k];
                            }
                        }
                    }
                }
            } else
            for (unsigned b = b_lo + lgroup; b < b_hi; b += lgroups) {
                for (unsigned d = lane * 4; d < a.dim; d += lanes * 4) {
                    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (unsigned j = 0; j < L; ++j) {
                        const unsigned i = b * L + j;
                        const unsigned row = a.pos_slot[i];
                        float4 v;
                        if (MULTI && row == kRemoteRow) v = *(const float4*)(mine.rows_in + (size_t)((unsigned)a.inverse[i] & ~kDupBit) * a.dim + d);
                        else if (row < kRowPending) v = *(const float4*)(T.row_ptr(row) + d);
                        else v = init4_rare(a.keys[i], d, T.init_seed, T.init_range);
                        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                    }
                    if (L > 1) { acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale; }
                    if (out16) *(uint2*)(outh + (size_t)b * a.dim + d) = pack_bf16x4(acc);
                    else *(float4*)(outf + (size_t)b * a.dim + d) = acc;
                }
            }
        }
    }
    // leave the scratch table empty for the next call: one store per DISTINCT key (clearing per position would
    // make every duplicate of a hot key store to the same address)
    for (unsigned u = tid; u < cnt[0]; u += nthreads) a.dedup[a.uniq_slot[u]].key = kEmptyKey;
    if (a.flags & FUSED_PREPARE_PUSH) {
        // the push adds the gradients of a duplicated key into its aggregation row, which must start at zero; the
        // rows of keys that occur once are written with a plain store and need nothing
        const unsigned n_uniq = cnt[0];
        if (n_uniq != a.n) {
            for (unsigned u = group; u < n_uniq; u += ngroups) {
                if (a.dedup[a.uniq_slot[u]].aux != dup_tag) continue;
                float4* z = (float4*)(a.agg + (size_t)u * a.dim);
                for (unsigned d = lane; d < a.dim / 4; d += lanes) z[d] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
    }
    if (blockIdx.x == 0 && threadIdx.x < 16) a.counters[(par ^ 1u) * 16 + threadIdx.x] = 0;
    PROF(6);
    if (blockIdx.x == 0 && threadIdx.x == 0) a.ctl->epoch = epoch;
}

// PLAIN: the common push (no replication, no sync delta): those two features drop out of the update loop.
template <int kThreads, bool MULTI, bool PLAIN>
__global__ void __launch_bounds__(kThreads, 1024 / kThreads) fused_push_kernel(const FusedArgs a) {
    constexpr int kHotSlots = HotCfg<kThreads>::kHotSlots;
    constexpr int kHotRows = HotCfg<kThreads>::kHotRows;
    const unsigned nblocks = gridDim.x;
    const unsigned tid = blockIdx.x * kThreads + threadIdx.x;
    const unsigned nthreads = nblocks * kThreads;
    // a fatal status of this family or of the pull that made the plan: do nothing
    if (ld_acquire_gpu(&a.ctl->status) != 0u || ld_acquire_gpu(&a.plan_ctl->status) != 0u) return;
    const unsigned epoch = *((volatile unsigned*)&a.ctl->epoch) + 1u;
    const unsigned plan_par = *((volatile const unsigned*)&a.plan_ctl->epoch) & 1u;
    const unsigned* cnt = a.counters + plan_par * 16;
    const unsigned* send_cnt = cnt + 4;
    const unsigned* in_cnt = a.in_cnt + plan_par * kMaxWorld;
    const int me = a.rank;
    const int W = MULTI ? a.world : 1;
    const unsigned C = a.C;
    const TableView T = *a.table;
    const PeerBufs& mine = a.peer[me];
    const unsigned lanes = lanes_for_dim(a.dim);
    const bool grads16 = (a.flags & FUSED_GRAD_BF16) != 0;
    const unsigned group = tid / lanes, ngroups = nthreads / lanes, lane = tid % lanes;
    const unsigned L = a.bag_size;

    __shared__ unsigned s_pre[kMaxWorld + 1];   // shipment prefix (Q2)
    __shared__ unsigned s_in[kMaxWorld + 1];    // received-entry prefix (Q0 / Q3)
    __shared__ unsigned s_nheads;               // chain heads this CTA found in its stripe (world > 1)
    if (threadIdx.x == 0) {
        unsigned acc = 0;
        for (int r = 0; r < W; ++r) {
            s_in[r] = acc;
            acc += in_cnt[r];
        }
        s_in[W] = acc;
    }
    __syncthreads();
    const unsigned total_in = s_in[W];

    // ---- Q0 (owner): one thread per received entry resolves entry -> slot -> row once (Q3 then starts from the row
    // index instead of walking that chain of dependent loads per lane group) and, with several ranks, chains the
    // entries that name the same table row. Each source rank sends a key at most once, so a chain holds at most one
    // entry per rank. All of this needs the slots resolved by the pull, not the gradients.
    PROF(8);
    unsigned* ent_row = a.new_list;   // free during a push: [world*C] row of every received entry
    for (unsigned e = tid; e < total_in; e += nthreads) {
        int r = 0;
        while (e >= s_in[r + 1]) ++r;
        const unsigned id = (unsigned)r * C + (e - s_in[r]);
        const unsigned slot = a.res_slot[id];
        unsigned row = kNoRow;
        if (slot != kNoSlot) {
            row = T.slots[slot].row;
            if (row >= kRowPending) row = kNoRow;
            if (W > 1) a.ent_next[id] = atomicExch(&T.slots[slot].aux, id);
        }
        ent_row[id] = row;
    }

    // ---- Q1: segment-sum gradients of duplicate keys --------------------------------------------
    // Every CTA owns a contiguous range of positions. Keys that occur several times inside the range
    // (the head of a Zipf distribution occurs in every range) are first summed in shared memory and reach
    // global memory once per CTA; everything else goes straight to the per-key row with a vector atomic.
    if (!(a.flags & FUSED_AGG_READY)) {
        const unsigned n_uniq = cnt[0];
        const bool dups = (n_uniq != a.n);
        const float scale = (a.flags & FUSED_MEAN) ? 1.0f / (float)L : 1.0f;
        const bool do_scale = L > 1 && (a.flags & FUSED_MEAN);
        const unsigned per = (a.n + nblocks - 1) / nblocks;
        const unsigned lo = min(a.n, blockIdx.x * per), hi = min(a.n, lo + per);
        const unsigned lgroup = threadIdx.x / lanes, lgroups = kThreads / lanes;
        extern __shared__ __align__(16) float s_cache[];  // [kHotRows][dim]
        __shared__ unsigned s_hkey[kHotSlots], s_hcnt[kHotSlots];
        __shared__ int s_hrow[kHotSlots];
        __shared__ unsigned s_cache_u[kHotRows];
        __shared__ unsigned s_ncache;
        const unsigned hot_rows = min(a.hot_rows, (unsigned)kHotRows);
        // the block-local sums pay for their three extra passes only when a CTA's range is long enough to hold a hot
        // key many times
        const bool use_cache = dups && hot_rows > 0 && a.dim <= kHotMaxDim && (hi - lo) >= 1024;
        if (use_cache) {
            for (unsigned t = threadIdx.x; t < kHotSlots; t += kThreads) { s_hkey[t] = 0xFFFFFFFFu; s_hcnt[t] = 0; s_hrow[t] = -1; }
            if (threadIdx.x == 0) s_ncache = 0;
            __syncthreads();
            // 1. count the keys of this range
            for (unsigned i = lo + threadIdx.x; i < hi; i += kThreads) {
                const unsigned iv = (unsigned)a.inverse[i];
                if (!(iv & kDupBit)) continue;   // a key that occurs once in the batch needs no summing
                const unsigned u = iv & ~kDupBit;
                unsigned h = (u * 2654435761u) & (kHotSlots - 1);
                for (int probe = 0; probe < 8; ++probe) {
                    const unsigned prev = atomicCAS(&s_hkey[h], 0xFFFFFFFFu, u);
                    if (prev == 0xFFFFFFFFu || prev == u) { atomicAdd(&s_hcnt[h], 1u); break; }
                    h = (h + 1) & (kHotSlots - 1);
                }
            }
            __syncthreads();
            // 2. keys seen at least 4 times get a shared-memory row
            for (unsigned t = threadIdx.x; t < kHotSlots; t += kThreads)
                if (s_hkey[t] != 0xFFFFFFFFu && s_hcnt[t] >= 4) {
                    const unsigned c = atomicAdd(&s_ncache, 1u);
                    if (c < hot_rows) { s_hrow[t] = (int)c; s_cache_u[c] = s_hkey[t]; }
                }
            __syncthreads();
            const unsigned nc = min(s_ncache, hot_rows);
            for (unsigned t = threadIdx.x; t < nc * a.dim; t += kThreads) s_cache[t] = 0.f;
            __syncthreads();
        }
        PROF(13);
        const unsigned gl0 = (threadIdx.x & 31u) / lanes * lanes;  // first lane of this group inside its warp
        // Four positions per lane group and iteration: their index lookups and gradient-row loads are all issued
        // before the first accumulation (the loop is bound by load latency, not by bytes).
        constexpr int kPos = 4;
        for (unsigned base = lo; base < hi; base += lgroups * kPos) {
            unsigned pos[kPos], u[kPos];
            int crow[kPos];
            bool active[kPos], dup[kPos];
#pragma unroll
            for (int k = 0; k < kPos; ++k) {
                pos[k] = base + (unsigned)k * lgroups + lgroup;
                active[k] = pos[k] < hi;
                const unsigned iv = active[k] ? (unsigned)a.inverse[pos[k]] : 0u;
                u[k] = iv & ~kDupBit;
                dup[k] = (iv & kDupBit) != 0u;
                crow[k] = -1;
            }
            if (use_cache) {
#pragma unroll
                for (int k = 0; k < kPos; ++k) {
                    if (active[k] && dup[k] && lane == 0) {
                        unsigned h = (u[k] * 2654435761u) & (kHotSlots - 1);
                        for (int probe = 0; probe < 8; ++probe) {
                            const unsigned key = s_hkey[h];
                            if (key == u[k]) { crow[k] = s_hrow[h]; break; }
                            if (key == 0xFFFFFFFFu) break;
                            h = (h + 1) & (kHotSlots - 1);
                        }
                    }
                    crow[k] = __shfl_sync(0xffffffffu, crow[k], gl0);
                }
            }
            for (unsigned d = lane * 4; d < a.dim; d += lanes * 4) {
                float4 v[kPos];
#pragma unroll
                for (int k = 0; k < kPos; ++k)
                    if (active[k]) v[k] = *(const float4*)(a.grads + (size_t)(pos[k] / L) * a.dim + d);
#pragma unroll
                for (int k = 0; k < kPos; ++k) {
                    if (!active[k]) continue;
                    float4 w = v[k];
                    if (do_scale) { w.x *= scale; w.y *= scale; w.z *= scale; w.w *= scale; }
                    if (crow[k] >= 0) {
                        float* c = s_cache + (size_t)crow[k] * a.dim + d;
                        atomicAdd(c + 0, w.x); atomicAdd(c + 1, w.y); atomicAdd(c + 2, w.z); atomicAdd(c + 3, w.w);
                    } else if (dup[k]) {
                        atomicAdd((float4*)(a.agg + (size_t)u[k] * a.dim + d), w);
                    } else {
                        *(float4*)(a.agg + (size_t)u[k] * a.dim + d) = w;
                    }
                }
            }
        }
        PROF(14);
        if (use_cache) {
            __syncthreads();
            const unsigned nc = min(s_ncache, hot_rows);
            for (unsigned c = lgroup; c < nc; c += lgroups) {
                float* dst = a.agg + (size_t)s_cache_u[c] * a.dim;
                for (unsigned d = lane * 4; d < a.dim; d += lanes * 4)
                    atomicAdd((float4*)(dst + d), *(const float4*)(s_cache + (size_t)c * a.dim + d));
            }
        }
    }
    PROF(15);
    PROF_CTA(3);
    if (!grid_sync(a.ctl, nblocks, a.limit_ns, W_Q1)) return;

    if (W > 1) {
        // the owners must have consumed the previous push before their mailboxes are overwritten
        if (!wait_all_flags(mine.push_ack, epoch - 1u, a, W_ACK)) return;
        // ---- Q2: ship merged gradient rows to the owners, two rows in flight per lane group
        PROF(9);
        if (threadIdx.x == 0) {
            unsigned acc = 0;
            for (int o = 0; o < W; ++o) {
                s_pre[o] = acc;
                acc += (o == me) ? 0u : min(send_cnt[o], C);
            }
            s_pre[W] = acc;
        }
        __syncthreads();
        const unsigned total = s_pre[W];
        const unsigned rot = s_pre[(me + 1) % W];  // ring order, see the key shipment of the pull
        constexpr int kIn = 2;
        for (unsigned e0 = group; e0 < total; e0 += ngroups * kIn) {
            const float* src[kIn];
            float* dst[kIn];
            bool act[kIn];
#pragma unroll
            for (int k = 0; k < kIn; ++k) {
                unsigned e = e0 + (unsigned)k * ngroups;
                act[k] = e < total;
                src[k] = nullptr;
                dst[k] = nullptr;
                if (!act[k]) continue;
                e += rot;
                if (e >= total) e -= total;
                int o = 0;
                while (e >= s_pre[o + 1]) ++o;
                const unsigned p = e - s_pre[o];
                src[k] = a.agg + (size_t)a.send_ret[(size_t)o * C + p] * a.dim;
                // bf16 on the wire: the same mailbox, rows packed at half the pitch
                dst[k] = grads16 ? (float*)((__nv_bfloat16*)a.peer[o].mail_grad + ((size_t)me * C + p) * a.dim)
                                 : a.peer[o].mail_grad + ((size_t)me * C + p) * a.dim;
            }
            for (unsigned d = lane * 4; d < a.dim; d += lanes * 4) {
                float4 v[kIn];
#pragma unroll
                for (int k = 0; k < kIn; ++k)
                    if (act[k]) v[k] = *(const float4*)(src[k] + d);
#pragma unroll
                for (int k = 0; k < kIn; ++k) {
                    if (!act[k]) continue;
                    if (grads16) *(uint2*)((__nv_bfloat16*)dst[k] + d) = pack_bf16x4(v[k]);
                    else *(float4*)(dst[k] + d) = v[k];
                }
            }
        }
        if (cta_arrive_last(&a.ctl->arrive[0], nblocks)) {
            if (threadIdx.x < (unsigned)W && (int)threadIdx.x != me)
                st_release_sys(&a.peer[threadIdx.x].grad_flag[me], epoch);
        }
        // While the peers' gradient rows are on their way: find the chain heads of this CTA's stripe of the received
        // entries and write out every head's chain in rank order, one THREAD per entry. The walk is a string of
        // dependent loads (slot, head test, up to world - 1 links); done here it runs thousands at a time, done by
        // the lane groups of the update loop below it was the longer part of that loop from two ranks on.
        {
            if (threadIdx.x == 0) s_nheads = 0;
            __syncthreads();
            const unsigned per_e = (total_in + nblocks - 1) / nblocks;
            const unsigned e_lo = min(total_in, blockIdx.x * per_e), e_hi = min(total_in, e_lo + per_e);
            for (unsigned e = e_lo + threadIdx.x; e < e_hi; e += kThreads) {
                int r = 0;
                while (e >= s_in[r + 1]) ++r;
                const unsigned id = (unsigned)r * C + (e - s_in[r]);
                const unsigned slot = a.res_slot[id];
                if (slot == kNoSlot) {
                    set_soft_status(a.ctl, kStOom, W_NOROW);
                    continue;
                }
                if (*((volatile unsigned*)&T.slots[slot].aux) != id) continue;  // not the head of its chain
                unsigned ids[kMaxWorld];
                ids[0] = id;
                unsigned cur = id;
#pragma unroll
                for (int k = 1; k < kMaxWorld; ++k) {
                    if (cur != kNoRow) cur = a.ent_next[cur];
                    ids[k] = cur;
                }
                // ascending entry id = ascending source rank (sorting network for 8 keys; kNoRow sorts last)
#define PSB_CSWAP(i, j)                                          \
    do {                                                         \
        const unsigned lo_ = min(ids[i], ids[j]), hi_ = max(ids[i], ids[j]); \
        ids[i] = lo_;                                            \
        ids[j] = hi_;                                            \
    } while (0)
                PSB_CSWAP(0, 1); PSB_CSWAP(2, 3); PSB_CSWAP(4, 5); PSB_CSWAP(6, 7);
                PSB_CSWAP(0, 2); PSB_CSWAP(1, 3); PSB_CSWAP(4, 6); PSB_CSWAP(5, 7);
                PSB_CSWAP(1, 2); PSB_CSWAP(5, 6); PSB_CSWAP(0, 4); PSB_CSWAP(3, 7);
                PSB_CSWAP(1, 5); PSB_CSWAP(2, 6);
                PSB_CSWAP(1, 4); PSB_CSWAP(3, 6);
                PSB_CSWAP(2, 4); PSB_CSWAP(3, 5);
                PSB_CSWAP(3, 4);
#undef PSB_CSWAP
                const unsigned pos = atomicAdd(&s_nheads, 1u);
                a.head_ids[e_lo + pos] = id;
#pragma unroll
                for (int k = 0; k < kMaxWorld; ++k)
                    if (k < W) a.chain_buf[(size_t)id * W + k] = ids[k];
                T.slots[slot].aux = kNoRow;   // the chain is consumed: the slot is clean for the next call
            }
            __syncthreads();
        }
        if (!wait_all_flags(mine.grad_flag, epoch, a, W_GRADFLAG)) return;
    }

    // ---- Q3 (owner): one optimizer step per touched row. With several ranks the head of each row's chain
    // collects the chain (at most one entry per source rank), orders it by source rank and adds the gradients in
    // that order, so the result does not depend on which entry arrived first.
    PROF(10);
    PROF(11);
    OptConfig opt = a.opt;
    if (opt.step_from_epoch) opt_set_step(opt, epoch);
    const bool sync_mode = !PLAIN && (a.flags & FUSED_SYNC_PUSH) != 0;
    const unsigned dim = a.dim;
    // Replication: this rank's updates go to the GPU to its right, and it applies the updates of the GPU to its left.
    // (a sync push only buffers deltas: it appends nothing, but it keeps the hand-shake of the log going so that
    // the epochs of later pushes line up)
    const bool replicate = !PLAIN && (a.flags & FUSED_REPLICATE) != 0;
    const bool rep_log = replicate && !sync_mode;
    const int partner = (me + 1) % W, mirrored = (me + W - 1) % W;
    unsigned* rep_fill = a.ctl->pad;   // entries appended to the partner's log by this call (reset by the last CTA)
    if (replicate) {
        // the partner must have applied the log of the previous push before it is overwritten
        int ok = 1;
        if (threadIdx.x == 0 && !wait_flag_ge(mine.rep_ack, epoch - 1u, a.limit_ns)) {
            set_status(a.ctl, kStTimeout, W_REPACK);
            ok = 0;
        }
        if (!__syncthreads_and(ok)) return;
    }
    const unsigned gl0 = (threadIdx.x & 31u) / lanes * lanes;  // first lane of this group inside its warp
    const unsigned gmask = (lanes >= 32u ? 0xffffffffu : ((1u << lanes) - 1u)) << gl0;
    // the row index and (single rank) the gradient row of the NEXT entry are fetched while the current one is updated
    unsigned row_nx = kNoRow, u_nx = 0;
    auto entry_id = [&](unsigned e, int* r_out) -> unsigned {
        int r = 0;
        while (e >= s_in[r + 1]) ++r;
        *r_out = r;
        return (unsigned)r * C + (e - s_in[r]);
    };
    // Work list: every received entry (one rank), or the chain heads this CTA found in its stripe (several ranks).
    const unsigned lgroup3 = threadIdx.x / lanes, lgroups3 = kThreads / lanes;
    const unsigned per_e3 = (total_in + nblocks - 1) / nblocks;
    const unsigned h_lo = min(total_in, blockIdx.x * per_e3);
    const unsigned n_work = (W == 1) ? total_in : s_nheads;
    const unsigned w_first = (W == 1) ? group : lgroup3, w_step = (W == 1) ? ngroups : lgroups3;
    unsigned id_nx = kNoRow;
    if (w_first < n_work) {
        if (W == 1) {
            int r0;
            id_nx = entry_id(w_first, &r0);
            u_nx = a.send_ret[id_nx];
        } else {
            id_nx = a.head_ids[h_lo + w_first];
        }
        row_nx = ent_row[id_nx];
    }
    for (unsigned e = w_first; e < n_work; e += w_step) {
        const unsigned id = id_nx;
        const int r = (int)(id / C);
        const unsigned row = row_nx, u_own = u_nx;
        if (e + w_step < n_work) {
            if (W == 1) {
                int rn;
                id_nx = entry_id(e + w_step, &rn);
                u_nx = a.send_ret[id_nx];
            } else {
                id_nx = a.head_ids[h_lo + e + w_step];
            }
            row_nx = ent_row[id_nx];
        }
        unsigned ids[kMaxWorld];
        ids[0] = id;
#pragma unroll
        for (int k = 1; k < kMaxWorld; ++k) ids[k] = kNoRow;
        if (W > 1) {
#pragma unroll
            for (int k = 0; k < kMaxWorld; ++k)
                if (k < W) ids[k] = a.chain_buf[(size_t)id * W + k];
        }
        if (row == kNoRow) {
            if (lane == 0) set_soft_status(a.ctl, kStOom, W_NOROW);
            continue;
        }
        // at most one entry of a chain is this rank's own (its gradient sits in `agg`, the others in the mailbox)
        const float* own = nullptr;
        if (W == 1) {
            own = a.agg + (size_t)u_own * dim;
        } else {
#pragma unroll
            for (int k = 0; k < kMaxWorld; ++k)
                if (ids[k] != kNoRow && (int)(ids[k] / C) == me)
                    own = a.agg + (size_t)a.send_ret[(size_t)me * C + (ids[k] - (unsigned)me * C)] * dim;
        }
        float* w = T.row_ptr(row);
        float* delta = w + (size_t)(T.n_opt_slots + 1) * dim;
        float* rep_dst = nullptr;
        if (rep_log) {
            unsigned j = 0;
            if (lane == 0) {
                j = atomicAdd(rep_fill, 1u);
                if (j < (unsigned)W * C)
                    a.peer[partner].rep_keys[j] = (r == me) ? a.send_keys[(size_t)me * C + (id - (unsigned)me * C)] : mine.mail_keys[id];
                else set_status(a.ctl, kStError, W_REP_FULL);
            }
            j = __shfl_sync(gmask, j, gl0);
            if (j < (unsigned)W * C) rep_dst = a.peer[partner].rep_grad + (size_t)j * dim;
        }
        // gradient row of chain entry k: this rank's own sum (fp32) or a row of the mailbox (fp32 or bf16)
        auto grad4 = [&](int k, unsigned d) -> float4 {
            if ((int)(ids[k] / C) == me) return *(const float4*)(own + d);
            if (grads16) return unpack_bf16x4(*(const uint2*)((const __nv_bfloat16*)mine.mail_grad + (size_t)ids[k] * dim + d));
            return *(const float4*)(mine.mail_grad + (size_t)ids[k] * dim + d);
        };
        for (unsigned d = lane * 4; d < dim; d += lanes * 4) {
            float4 gv = grad4(0, d);
#pragma unroll
            for (int k = 1; k < kMaxWorld; ++k) {
                if (ids[k] == kNoRow) continue;
                const float4 o = grad4(k, d);
                gv.x = __fadd_rn(gv.x, o.x); gv.y = __fadd_rn(gv.y, o.y);
                gv.z = __fadd_rn(gv.z, o.z); gv.w = __fadd_rn(gv.w, o.w);
            }
            if (rep_dst != nullptr) *(float4*)(rep_dst + d) = gv;   // the replica gets what the row is updated with
            if (sync_mode) {
                float4 dv = *(float4*)(delta + d);
                dv.x += gv.x; dv.y += gv.y; dv.z += gv.z; dv.w += gv.w;
                *(float4*)(delta + d) = dv;
            } else {
                float4 wv = *(float4*)(w + d);
                float4 s0 = make_float4(0.f, 0.f, 0.f, 0.f), s1 = s0;
                if (T.n_opt_slots > 0) s0 = *(float4*)(w + dim + d);
                if (T.n_opt_slots > 1) s1 = *(float4*)(w + 2 * dim + d);
                opt_update(opt, wv.x, s0.x, s1.x, gv.x);
                opt_update(opt, wv.y, s0.y, s1.y, gv.y);
                opt_update(opt, wv.z, s0.z, s1.z, gv.z);
                opt_update(opt, wv.w, s0.w, s1.w, gv.w);
                *(float4*)(w + d) = wv;
                if (T.n_opt_slots > 0) *(float4*)(w + dim + d) = s0;
                if (T.n_opt_slots > 1) *(float4*)(w + 2 * dim + d) = s1;
            }
        }
        if (sync_mode && lane == 0) {
            unsigned bit = 1u << (row & 31u);
            unsigned old = atomicOr(&T.touched_bits[row >> 5], bit);
            if (!(old & bit)) {
                unsigned j = atomicAdd(T.touched_count, 1u);
                if (j < T.touched_cap) T.touched_list[j] = row;
                else set_soft_status(a.ctl, kStOom, W_NOROW);
            }
        }
        if (T.dirty_bits != nullptr && lane == 0) atomicOr(&T.dirty_bits[row >> 5], 1u << (row & 31u));
    }

    if (W > 1) {
        // last CTA out acknowledges the sources: their next push may overwrite our mailboxes
        if (cta_arrive_last(&a.ctl->arrive[1], nblocks)) {
            if (threadIdx.x < (unsigned)W && (int)threadIdx.x != me)
                st_release_sys(&a.peer[threadIdx.x].push_ack[me], epoch);
        }
    }
    // ---- Q4 (replica holder) -----------------------------------------------------------------------------
    if (replicate) {
        TableView R = *a.mirror;
        // a mirror row starts from the OWNER's initial value of the key
        R.init_seed = T.init_seed;
        R.init_range = T.init_range;
        R.slot_init[0] = T.slot_init[0];
        R.slot_init[1] = T.slot_init[1];
        // the log this rank WROTE is complete when every CTA is past Q3: the last one publishes count + flag
        if (cta_arrive_last(&a.ctl->arrive[2], nblocks)) {
            if (threadIdx.x == 0) {
                const unsigned filled = min(*((volatile unsigned*)rep_fill), (unsigned)W * C);
                *rep_fill = 0;
                *a.peer[partner].rep_cnt = filled;
                __threadfence_system();
                st_release_sys(a.peer[partner].rep_flag, epoch);
            }
        }
        // the log this rank RECEIVES (from the rank it mirrors)
        {
            int ok = 1;
            if (threadIdx.x == 0 && !wait_flag_ge(mine.rep_flag, epoch, a.limit_ns)) {
                set_status(a.ctl, kStTimeout, W_REPFLAG);
                ok = 0;
            }
            if (ld_acquire_gpu(&a.ctl->status) != 0u) ok = 0;
            if (!__syncthreads_and(ok)) return;
        }
        const unsigned n_log = min(ld_relaxed_sys(mine.rep_cnt), (unsigned)W * C);
        unsigned* n_new_rep = a.ctl->pad + 1;
        // (a) one thread per entry: find or insert the key in the mirror and give it a row
        const unsigned wl = threadIdx.x & 31u;
        for (unsigned j0 = (tid & ~31u); j0 < n_log; j0 += nthreads) {
            const unsigned j = j0 + wl;
            bool attached = false, inserted = false;
            unsigned slot = kNoSlot;
            if (j < n_log) {
                slot = table_find_or_insert(R, mine.rep_keys[j], true, &inserted);
                if (slot == kNoSlot) {
                    set_soft_status(a.ctl, kStOom, W_INDEX_FULL);
                } else {
                    bool oom = false;
                    attached = table_attach_row(R, slot, &oom);
                    if (oom) set_soft_status(a.ctl, kStOom, W_POOL_FULL);
                }
                a.rep_slot[j] = slot;
            }
            const unsigned amask = __ballot_sync(0xffffffffu, attached);
            if (amask) {
                const int al = __ffs(amask) - 1;
                unsigned base = 0;
                if ((int)wl == al) base = atomicAdd(n_new_rep, (unsigned)__popc(amask));
                base = __shfl_sync(0xffffffffu, base, al);
                if (attached) a.rep_new[base + __popc(amask & ((1u << wl) - 1u))] = slot;
            }
            const unsigned imask = __ballot_sync(0xffffffffu, inserted);
            if (imask && (int)wl == __ffs(imask) - 1) atomicAdd(R.n_items, (unsigned long long)__popc(imask));
        }
        if (!grid_sync(a.ctl, nblocks, a.limit_ns, W_REP_A)) return;
        // (b) rows the mirror did not have yet start from the key's initial value, exactly like on the owner
        const unsigned n_new = *((volatile unsigned*)n_new_rep);
        for (unsigned j = group; j < n_new; j += ngroups) {
            const unsigned slot = a.rep_new[j];
            const unsigned row = R.slots[slot].row;
            if (row < kRowPending) row_init(R, R.row_ptr(row), R.slots[slot].key, lane, lanes);
        }
        if (n_new > 0) {
            if (!grid_sync(a.ctl, nblocks, a.limit_ns, W_REP_A)) return;
        }
        // (c) the same optimizer step with the same gradient: the mirror row stays bit-identical to the owner's
        for (unsigned j = group; j < n_log; j += ngroups) {
            const unsigned slot = a.rep_slot[j];
            if (slot == kNoSlot) continue;
            const unsigned row = R.slots[slot].row;
            if (row >= kRowPending) continue;
            float* w = R.row_ptr(row);
            const float* g = mine.rep_grad + (size_t)j * dim;
            for (unsigned d = lane * 4; d < dim; d += lanes * 4) {
                const float4 gv = *(const float4*)(g + d);
                float4 wv = *(float4*)(w + d);
                float4 s0 = make_float4(0.f, 0.f, 0.f, 0.f), s1 = s0;
                if (R.n_opt_slots > 0) s0 = *(float4*)(w + dim + d);
                if (R.n_opt_slots > 1) s1 = *(float4*)(w + 2 * dim + d);
                opt_update4_any(opt, wv, s0, s1, gv);   // out of line: the replica path is the rare one
                *(float4*)(w + d) = wv;
                if (R.n_opt_slots > 0) *(float4*)(w + dim + d) = s0;
                if (R.n_opt_slots > 1) *(float4*)(w + 2 * dim + d) = s1;
            }
        }
        // last CTA out: the log may be overwritten by the mirrored rank's next push
        if (cta_arrive_last(&a.ctl->arrive[3], nblocks)) {
            if (threadIdx.x == 0) {
                *n_new_rep = 0;
                st_release_sys(a.peer[mirrored].rep_ack, epoch);
            }
        }
    }
    PROF(12);
    // every CTA read the epoch before the first grid barrier, so CTA 0 may publish it when it leaves
    if (blockIdx.x == 0 && threadIdx.x == 0) a.ctl->epoch = epoch;
}

namespace {
template <int kThreads>
const void* push_kernel_of(bool multi, bool plain) {
    if (plain) return multi ? (const void*)fused_push_kernel<kThreads, true, true> : (const void*)fused_push_kernel<kThreads, false, true>;
    return multi ? (const void*)fused_push_kernel<kThreads, true, false> : (const void*)fused_push_kernel<kThreads, false, false>;
}

template <int kThreads>
int max_blocks_of(const cudaDeviceProp& prop, int* pull_blocks, int* push_blocks) {
    int per_sm = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fused_pull_kernel<kThreads, true>, kThreads, 0);
    if (e != cudaSuccess) return (int)e;
    *pull_blocks = per_sm * prop.multiProcessorCount;
    // static counting tables + the dynamic row cache may exceed the 48 KB a kernel gets without asking
    for (int v = 0; v < 4; ++v) {
        e = cudaFuncSetAttribute(push_kernel_of<kThreads>((v & 1) != 0, (v & 2) != 0), cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)push_smem_bytes<kThreads>());
        if (e != cudaSuccess) return (int)e;
    }
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fused_push_kernel<kThreads, true, false>, kThreads, push_smem_bytes<kThreads>());
    if (e != cudaSuccess) return (int)e;
    *push_blocks = per_sm * prop.multiProcessorCount;
    return 0;
}
template <int kThreads>
int launch_push_of(const FusedArgs& a, int nblocks, void* stream) {
    void* params[] = {(void*)&a};
    const unsigned cap = (unsigned)HotCfg<kThreads>::kHotRows;
    const size_t smem = (size_t)(a.hot_rows < cap ? a.hot_rows : cap) * kHotMaxDim * sizeof(float);
    const void* kern = push_kernel_of<kThreads>(a.world > 1, (a.flags & (FUSED_SYNC_PUSH | FUSED_REPLICATE)) == 0);
    return (int)cudaLaunchCooperativeKernel(kern, dim3(nblocks), dim3(kThreads), params, smem, (cudaStream_t)stream);
}
}  // namespace

int fused_max_blocks(int device, bool wide, int* pull_blocks, int* push_blocks) {
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) return (int)e;
    return wide ? max_blocks_of<kThreadsWide>(prop, pull_blocks, push_blocks)
                : max_blocks_of<kThreadsSmall>(prop, pull_blocks, push_blocks);
}

int launch_fused_pull(const FusedArgs& a, int nblocks, bool wide, void* stream) {
    void* params[] = {(void*)&a};
    const bool multi = a.world > 1;
    const void* kern = wide ? (multi ? (const void*)fused_pull_kernel<kThreadsWide, true> : (const void*)fused_pull_kernel<kThreadsWide, false>)
                            : (multi ? (const void*)fused_pull_kernel<kThreadsSmall, true> : (const void*)fused_pull_kernel<kThreadsSmall, false>);
    return (int)cudaLaunchCooperativeKernel(kern, dim3(nblocks), dim3(wide ? kThreadsWide : kThreadsSmall), params, 0, (cudaStream_t)stream);
}

int launch_fused_push(const FusedArgs& a, int nblocks, bool wide, void* stream) {
    return wide ? launch_push_of<kThreadsWide>(a, nblocks, stream) : launch_push_of<kThreadsSmall>(a, nblocks, stream);
}

}  // namespace psb
