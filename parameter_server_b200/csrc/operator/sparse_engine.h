// SparseEngine: the collective (all training ranks call together) pull / push path of one sparse
// table, i.e. the B200 replacement of PullHandler::pull + SparseTablePullOperator and
// PushHandler::async_push / sync_push + SparseTablePushOperator
// (pico-ps/handler/PullHandler.cpp:101-141, pico-ps/handler/PushHandler.cpp:53-86). It owns the
// symmetric mailboxes, the local scratch and the per-call epoch, and launches the fused kernels.
#pragma once
#include <memory>
#include <string>
#include <vector>

#include "../comm/symmetric.h"
#include "../kernels/sparse_fused.h"
#include "../storage/gpu_table.h"

namespace psb {

struct SparseEngineConfig {
    int world = 1;
    int rank = 0;
    uint32_t max_keys = 1u << 20;   // N: key positions per call per rank
    uint32_t pair_capacity = 0;     // C: entries per (source, owner) mailbox; 0 = automatic
    int n_shards = 1;               // global shard count G
    double wait_limit_s = 10.0;     // bound of every device-side wait
    bool replicate = false;         // allocate the replica log: pushes can keep a mirror on the next rank exact
};

class SparseEngine {
public:
    SparseEngine(GpuTable* table, const SparseEngineConfig& cfg);
    ~SparseEngine();

    std::string ipc_handle() const { return symm_->ipc_handle(); }
    Status connect(const std::vector<std::string>& handles);
    // In-process multi-engine wiring (tests, single process driving several GPUs).
    void connect_local(const std::vector<SparseEngine*>& engines);

    // shard -> owning rank map (length n_shards); may be changed between calls (reshard).
    Status set_shard_owner(const std::vector<int>& owner);
    const std::vector<int>& shard_owner() const { return shard_owner_host_; }

    // Collective pull. keys: device int64[n]; out: device [n/bag_size][dim], fp32 or (FUSED_OUT_BF16) bf16; may be
    // null when flags lacks FUSED_COPY_ROWS. Leaves a plan for one following push().
    Status pull(const long long* keys, uint32_t n, uint32_t bag_size, void* out, unsigned flags, void* stream);
    // Collective push with the plan of the last pull: grads is device float[n_rows][dim] and n_rows must equal the
    // plan's n / bag_size (0 skips the check: the caller vouches for the buffer).
    Status push(const float* grads, uint32_t n_rows, const OptConfig& opt, unsigned flags, void* stream);
    // Synchronise the stream and translate the device status words of pull and push. OUT_OF_MEMORY is reported
    // once and cleared (the call that met it ran to its end); TIMEOUT / ERROR stay until reset() and make the
    // engine refuse further launches.
    Status check(void* stream);
    // Re-arm after an error (clears scratch, barriers and flags on THIS rank; every rank must do it).
    Status reset(void* stream);
    // SM budget of the two kernels. 0 = the whole GPU (256-thread CTAs, four per SM). n > 0 = the call runs as
    // 1024-thread CTAs, each of which fills its SM (the whole register file), on n SMs, and leaves the others, whole,
    // to kernels of another stream (the dense GEMMs of the same step, whose CTAs also fill an SM each: whichever
    // starts first, the two share the GPU by SMs).
    void set_sm_budget(int pull_sms, int push_sms);
    // Reproducible pushes: duplicate keys of a batch are summed in position order (a stable sort + an ordered
    // segment sum before the fused kernel) instead of with fp32 atomics. Together with the rank-ordered fold of the
    // owners this makes the table after a push a function of the requests alone. Allocates its scratch on first use.
    Status set_deterministic(bool on);
    // Gradient rows that go to another rank cross NVLink as bf16 (half the bytes of the push's link-bound phase); each
    // rank's partial sum is rounded once, the owner adds the rows in fp32. Off by default: results then differ from
    // the fp32 oracle in the last bits of a bf16 value.
    void set_grad_wire_bf16(bool on) { grad_wire_bf16_ = on; }
    // Replication inside the push (needs SparseEngineConfig::replicate on every rank): `mirror` is the table on THIS
    // GPU that mirrors the shards of rank (rank - 1) % world (with world 1: of this rank). From then on every push
    // forwards, per updated row, the key and the folded gradient to rank (rank + 1) % world, whose kernel applies
    // the same optimizer step to its mirror row: the mirror is exact after every push, no separate sync needed.
    // nullptr switches it off again (collectively).
    Status set_mirror(GpuTable* mirror);
    bool deterministic() const { return deterministic_; }
    int pull_blocks() const { return pull_blocks_; }
    int push_blocks() const { return push_blocks_; }

    uint32_t last_unique(void* stream);  // unique keys of the last pull (synchronises)
    const SparseEngineConfig& config() const { return cfg_; }
    GpuTable* table() const { return table_; }
    uint32_t pair_capacity() const { return C_; }
    uint64_t scratch_bytes() const { return scratch_bytes_; }
    uint64_t kernel_launches() const { return launches_; }
    void set_wait_limit(double s) { cfg_.wait_limit_s = s; }
    // Phase tracing: when on, CTA 0 of each kernel records a timestamp at every phase boundary.
    void set_profile(bool on) { profile_ = on; }
    // Raw %globaltimer stamps of the last pull (slots 0..6) and push (slots 8..12), in ns.
    std::vector<uint64_t> phase_stamps(void* stream);
    // Per-CTA %globaltimer stamps of the last profiled calls: 0 = CTA entered the pull, 1 = reached the barrier after
    // the dedup phase, 2 = after the resolve phase, 3 = (push) after the segment sum. Zero where a CTA did not run.
    std::vector<uint64_t> cta_stamps(int which, void* stream);

private:
    void fill_common(FusedArgs& a) const;

    GpuTable* table_;
    SparseEngineConfig cfg_;
    uint32_t C_ = 0;
    std::unique_ptr<SymmetricBuffer> symm_;
    size_t off_flags_ = 0, off_mail_keys_ = 0, off_mail_ret_ = 0, off_rows_in_ = 0, off_mail_grad_ = 0;
    size_t off_rep_words_ = 0, off_rep_keys_ = 0, off_rep_grad_ = 0;
    GpuTable* mirror_ = nullptr;
    unsigned *rep_slot_ = nullptr, *rep_new_ = nullptr;
    char* scratch_ = nullptr;
    uint64_t scratch_bytes_ = 0;
    // carved from scratch_
    Slot* dedup_ = nullptr;
    uint64_t dedup_slots_ = 0;
    unsigned *pos_slot_ = nullptr, *uniq_row_ = nullptr, *uniq_slot_ = nullptr, *send_ret_ = nullptr, *res_slot_ = nullptr,
             *new_list_ = nullptr, *ent_next_ = nullptr, *counters_ = nullptr, *in_cnt_ = nullptr;
    int* inverse_ = nullptr;
    long long* send_keys_ = nullptr;
    float* agg_ = nullptr;
    KernelCtl* ctl_pull_ = nullptr;
    KernelCtl* ctl_push_ = nullptr;
    int* shard_owner_dev_ = nullptr;
    std::vector<int> shard_owner_host_;
    unsigned pull_epoch_ = 0, push_epoch_ = 0;
    int pull_blocks_ = 0, push_blocks_ = 0;          // grid of the next launches
    int max_pull_blocks_ = 0, max_push_blocks_ = 0;  // full residency on the idle GPU (256-thread CTAs)
    int max_pull_wide_ = 0, max_push_wide_ = 0;      // the same for the 1024-thread shape (one CTA per SM)
    unsigned* head_ids_ = nullptr;
    unsigned* chain_buf_ = nullptr;
    bool pull_wide_ = false, push_wide_ = false;
    bool grad_wire_bf16_ = false;
    int num_sms_ = 0;
    unsigned hot_rows_ = 24;
    bool failed_ = false;                            // a fatal device status was seen: reset() first
    bool deterministic_ = false;
    unsigned *sorted_ids_ = nullptr, *sorted_pos_ = nullptr;   // scratch of the ordered pre-aggregation
    void* sort_temp_ = nullptr;
    size_t sort_temp_bytes_ = 0;
    // last pull (the plan)
    const long long* plan_keys_ = nullptr;
    uint32_t plan_n_ = 0, plan_bag_ = 1;
    unsigned plan_flags_ = 0;
    bool plan_valid_ = false, plan_used_ = false;
    uint64_t launches_ = 0;
    unsigned long long* prof_ = nullptr;
    bool profile_ = false;
};

}  // namespace psb
