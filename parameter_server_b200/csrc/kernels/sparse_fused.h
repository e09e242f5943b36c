// Argument blocks of the fused sparse pull / push kernels (host + device view).
#pragma once
#include <cstdint>

#include "common.cuh"
#include "optim.cuh"

namespace psb {

// Pointers into ONE rank's symmetric (peer-mapped) buffer, as seen from the calling process.
struct PeerBufs {
    unsigned* key_flag;    // [kMaxWorld] epoch written by source rank r at index r once its keys landed
    unsigned* key_cnt;     // [kMaxWorld] number of keys rank r sent
    unsigned* row_flag;    // [kMaxWorld] epoch written by owner o once the rows for this rank landed
    unsigned* grad_flag;   // [kMaxWorld] epoch written by source rank r once its gradients landed
    unsigned* push_ack;    // [kMaxWorld] epoch written by owner o once it consumed this rank's gradients
    long long* mail_keys;  // [world][C]
    unsigned* mail_ret;    // [world][C] index in the sender's unique list (where the row must return)
    float* rows_in;        // [N][dim] rows returned by remote owners, indexed by unique id (fp32, or bf16 in the
                           // first half of the buffer when the pull asked for bf16 output without pooling)
    float* mail_grad;      // [world][C][dim] merged gradients sent by each source rank
    // ---- replica log (only with replication): written by the rank whose shards this GPU mirrors ----
    unsigned* rep_flag;    // [1] epoch written by the mirrored rank once its log of this push is complete
    unsigned* rep_cnt;     // [1] entries in the log
    unsigned* rep_ack;     // [1] epoch written by the rank that holds MY mirror once it has applied my log
    long long* rep_keys;   // [world*C] keys of the rows the mirrored rank updated
    float* rep_grad;       // [world*C][dim] the gradient each of them was updated with (all sources folded)
};

enum FusedFlags : unsigned {
    FUSED_INSERT = 1u,        // missing keys are inserted (pull of a non read-only operator)
    FUSED_COPY_ROWS = 2u,     // return rows (pull); off when only a push plan is built
    FUSED_PREPARE_PUSH = 4u,  // zero the gradient aggregation rows for a following push
    FUSED_MEAN = 8u,          // mean instead of sum pooling
    FUSED_SYNC_PUSH = 16u,    // push accumulates into the delta section instead of updating
    FUSED_OUT_BF16 = 32u,     // pull output is bf16 (the consumer's activation dtype); with bag_size 1 the rows
                              // also cross NVLink as bf16, which halves the bytes of the row-return phase
    FUSED_AGG_READY = 64u,    // push: the per-unique gradient sums are already in `agg` (deterministic pre-pass)
    FUSED_REPLICATE = 128u,   // push: every row update is also applied to the row's replica on the partner GPU
    FUSED_GRAD_BF16 = 256u,   // push: merged gradient rows cross NVLink as bf16 (summed in fp32 on both sides)
};

struct FusedArgs {
    int world;
    int rank;
    unsigned C;  // capacity of one (source, owner) mailbox, in entries
    unsigned N;  // capacity of one call, in key positions
    unsigned dim;
    unsigned flags;
    unsigned long long limit_ns;
    PeerBufs peer[kMaxWorld];  // peer[rank] is this GPU's own buffer
    // ---- local scratch -------------------------------------------------------------------
    Slot* dedup;
    unsigned long long dmask;
    unsigned* pos_slot;    // [N] dedup slot of each key position
    int* inverse;          // [N] unique id of each key position (bit 31: kDupBit)
    unsigned* uniq_row;    // [N] local row index of a unique key, kRemoteRow when the owner is a peer
    unsigned* uniq_slot;   // [N] dedup-table slot of a unique key (to empty the table afterwards)
    long long* send_keys;  // [world][C] staged per-owner key lists
    unsigned* send_ret;    // [world][C] unique id of each staged key
    float* agg;            // [N][dim] per-unique-key gradient sums
    unsigned* res_slot;    // [world][C] owner side: table slot of each received key
    unsigned* new_list;    // [world*C] owner side: slots whose rows were attached by this call
    unsigned* ent_next;    // [world*C] owner side, push: next entry (other source rank) that holds the same table row
    unsigned* head_ids;    // [world*C] push, world > 1: chain heads found by each CTA in its stripe of the entries
    unsigned* chain_buf;   // [world*C][world] push, world > 1: entry ids of a head's chain in ascending (= rank) order
    unsigned* counters;    // [2][16] per epoch parity: 0 n_uniq, 1 n_new, 4.. send_cnt[world]
    unsigned* in_cnt;      // [2][kMaxWorld] per epoch parity: keys received from each source rank
    KernelCtl* ctl;       // control block of this kernel family (holds the call epoch)
    const KernelCtl* plan_ctl;  // push: control block of the pull family (parity of the plan)
    unsigned long long* prof;  // [16] phase timestamps written by CTA 0 (nullptr = off)
    const int* shard_owner;  // [n_shards] owning rank of every global shard
    int n_shards;
    // The table views live in device memory (GpuTable::view_dev): a launch replayed from a CUDA graph then sees an
    // index that the host has grown, or dirty tracking that was switched on, since the capture.
    const TableView* table;
    const TableView* mirror;  // push with FUSED_REPLICATE: the local table that mirrors rank (rank - 1) % world
    unsigned* rep_slot;       // [world*C] mirror slot of each log entry (scratch of the replica phase)
    unsigned* rep_new;        // [world*C] list of log entries whose mirror row was attached by this call
    // ---- call inputs / outputs ----------------------------------------------------------------
    const long long* keys;  // [n]
    unsigned n;
    unsigned bag_size;      // keys pooled per output row (1 = no pooling)
    unsigned hot_rows;      // push: gradient rows of hot keys a CTA may sum in shared memory (0..24; 512 B each at dim 128)
    void* out;              // [n / bag_size][dim] fp32, or bf16 with FUSED_OUT_BF16
    const float* grads;     // [n / bag_size][dim] gradient w.r.t. `out`
    OptConfig opt;
};

constexpr unsigned kRemoteRow = 0xFFFFFFFDu;
constexpr unsigned kProfMaxCtas = 2048;   // per-CTA profile stamps: prof[16 + k * kProfMaxCtas + cta], k < 4
constexpr unsigned kDupBit = 0x80000000u;   // in FusedArgs::inverse: the position's key occurs more than once in the batch

// Host launchers (defined in sparse_fused.cu). `stream` is a cudaStream_t. Return cudaError_t as int.
// wide = the 1024-thread CTA shape (one CTA per SM); otherwise 256 threads, four CTAs per SM
int launch_fused_pull(const FusedArgs& a, int nblocks, bool wide, void* stream);
int launch_fused_push(const FusedArgs& a, int nblocks, bool wide, void* stream);
int fused_max_blocks(int device, bool wide, int* pull_blocks, int* push_blocks);

}  // namespace psb
