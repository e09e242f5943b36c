#include "sparse_engine.h"

#include <cuda_runtime.h>

#include "../kernels/segment_sum.h"

#include <algorithm>
#include <stdexcept>

namespace psb {

namespace {
size_t align_up(size_t v, size_t a = 256) { return (v + a - 1) / a * a; }
uint64_t pow2_ceil64(uint64_t v) {
    uint64_t p = 1;
    while (p < v) p <<= 1;
    return p;
}
__global__ void fill_dedup_kernel(Slot* s, uint64_t n) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        Slot e;
        e.key = kEmptyKey;
        e.row = kNoRow;
        e.aux = kNoRow;
        s[i] = e;
    }
}
const char* where_name(unsigned w) {
    switch (w) {
        case 1: return "pull: grid barrier after dedup";
        case 2: return "pull: grid barrier after key shipment";
        case 3: return "pull: waiting for a source rank's keys";
        case 4: return "pull: grid barrier after key resolution";
        case 5: return "pull: grid barrier after row initialisation";
        case 6: return "pull: grid barrier after row return";
        case 7: return "pull: waiting for an owner's rows";
        case 8: return "pull: (source, owner) mailbox overflow - raise pair_capacity";
        case 9: return "pull: table index full";
        case 10: return "pull: row pool exhausted";
        case 11: return "pull: dedup scratch table full (an earlier call was cut short, or two calls overlap on one engine)";
        case 12: return "pull: a key equals one of the two reserved values (INT64_MIN, INT64_MIN + 1)";
        case 32: return "push: grid barrier after gradient merge";
        case 33: return "push: waiting for an owner's acknowledgement of the previous push";
        case 34: return "push: grid barrier after gradient shipment";
        case 35: return "push: waiting for a source rank's gradients";
        case 36: return "push: grid barrier after leader election";
        case 37: return "push: grid barrier after cross-rank merge";
        case 38: return "push: key without a backing row (pool exhausted)";
        case 39: return "push: waiting for the replica holder to apply the previous push's log";
        case 40: return "push: waiting for the mirrored rank's replica log";
        case 41: return "push: grid barrier of the replica phase";
        case 42: return "push: replica log overflow";
        default: return "unknown site";
    }
}
}  // namespace

SparseEngine::SparseEngine(GpuTable* table, const SparseEngineConfig& cfg) : table_(table), cfg_(cfg) {
    if (cfg_.world < 1 || cfg_.world > kMaxWorld) throw std::invalid_argument("SparseEngine: world must be 1..8");
    if (table_->dim() % 4 != 0) throw std::invalid_argument("SparseEngine: dim must be a multiple of 4");
    cudaSetDevice(table_->device());
    const uint64_t N = cfg_.max_keys;
    const int W = cfg_.world;
    if (cfg_.pair_capacity) C_ = cfg_.pair_capacity;
    else if (W <= 2) C_ = (uint32_t)N;
    else C_ = (uint32_t)std::min<uint64_t>(N, std::max<uint64_t>(65536, 2 * N / W + 4096));
    const uint64_t dim = table_->dim();

    // symmetric part
    size_t off = 0;
    off_flags_ = off; off = align_up(off + 5 * kMaxWorld * sizeof(unsigned));
    if (W > 1) {
        off_mail_keys_ = off; off = align_up(off + (size_t)W * C_ * 8);
        off_mail_ret_ = off; off = align_up(off + (size_t)W * C_ * 4);
        off_rows_in_ = off; off = align_up(off + (size_t)N * dim * 4);
        off_mail_grad_ = off; off = align_up(off + (size_t)W * C_ * dim * 4);
    }
    if (cfg_.replicate) {
        off_rep_words_ = off; off = align_up(off + 4 * sizeof(unsigned));
        off_rep_keys_ = off; off = align_up(off + (size_t)W * C_ * 8);
        off_rep_grad_ = off; off = align_up(off + (size_t)W * C_ * dim * 4);
    }
    symm_.reset(new SymmetricBuffer(table_->device(), off));

    // local scratch
    dedup_slots_ = pow2_ceil64(2 * N);
    size_t s = 0;
    auto carve = [&](size_t bytes) { size_t o = s; s = align_up(s + bytes); return o; };
    const size_t o_dedup = carve(dedup_slots_ * sizeof(Slot));
    const size_t o_pos = carve(N * 4), o_inv = carve(N * 4), o_urow = carve(N * 4), o_uslot = carve(N * 4);
    const size_t o_skeys = carve((size_t)W * C_ * 8), o_sret = carve((size_t)W * C_ * 4);
    const size_t o_agg = carve(N * dim * 4);
    const size_t o_res = carve((size_t)W * C_ * 4), o_new = carve((size_t)W * C_ * 4), o_next = carve((size_t)W * C_ * 4);
    // push, several ranks: per-CTA lists of chain heads and the sorted chain of every head
    const size_t o_heads = carve(W > 1 ? (size_t)W * C_ * 4 : 0), o_chain = carve(W > 1 ? (size_t)W * C_ * (size_t)W * 4 : 0);
    const size_t o_rslot = carve(cfg_.replicate ? (size_t)W * C_ * 4 : 0), o_rnew = carve(cfg_.replicate ? (size_t)W * C_ * 4 : 0);
    const size_t o_cnt = carve(2 * 16 * 4), o_in = carve(2 * kMaxWorld * 4);
    const size_t o_ctl1 = carve(sizeof(KernelCtl)), o_ctl2 = carve(sizeof(KernelCtl));
    const size_t o_prof = carve((16 + 4 * kProfMaxCtas) * 8);
    const size_t o_owner = carve((size_t)std::max(cfg_.n_shards, 1) * 4);
    scratch_bytes_ = s;
    cudaError_t e = cudaMalloc(&scratch_, s);
    if (e != cudaSuccess) throw std::runtime_error(std::string("SparseEngine: cudaMalloc scratch: ") + cudaGetErrorString(e));
    cudaMemset(scratch_, 0, s);
    dedup_ = (Slot*)(scratch_ + o_dedup);
    pos_slot_ = (unsigned*)(scratch_ + o_pos);
    inverse_ = (int*)(scratch_ + o_inv);
    uniq_row_ = (unsigned*)(scratch_ + o_urow);
    uniq_slot_ = (unsigned*)(scratch_ + o_uslot);
    send_keys_ = (long long*)(scratch_ + o_skeys);
    send_ret_ = (unsigned*)(scratch_ + o_sret);
    agg_ = (float*)(scratch_ + o_agg);
    res_slot_ = (unsigned*)(scratch_ + o_res);
    new_list_ = (unsigned*)(scratch_ + o_new);
    ent_next_ = (unsigned*)(scratch_ + o_next);
    head_ids_ = (unsigned*)(scratch_ + o_heads);
    chain_buf_ = (unsigned*)(scratch_ + o_chain);
    rep_slot_ = (unsigned*)(scratch_ + o_rslot);
    rep_new_ = (unsigned*)(scratch_ + o_rnew);
    counters_ = (unsigned*)(scratch_ + o_cnt);
    in_cnt_ = (unsigned*)(scratch_ + o_in);
    ctl_pull_ = (KernelCtl*)(scratch_ + o_ctl1);
    ctl_push_ = (KernelCtl*)(scratch_ + o_ctl2);
    prof_ = (unsigned long long*)(scratch_ + o_prof);
    shard_owner_dev_ = (int*)(scratch_ + o_owner);
    fill_dedup_kernel<<<148 * 4, 256>>>(dedup_, dedup_slots_);
    // default placement: shard s lives on rank s % world
    std::vector<int> owner(std::max(cfg_.n_shards, 1));
    for (size_t i = 0; i < owner.size(); ++i) owner[i] = (int)(i % (size_t)W);
    set_shard_owner(owner);
    int rc = fused_max_blocks(table_->device(), false, &max_pull_blocks_, &max_push_blocks_);
    if (rc == 0) rc = fused_max_blocks(table_->device(), true, &max_pull_wide_, &max_push_wide_);
    if (rc != 0) throw std::runtime_error("SparseEngine: occupancy query failed");
    cudaDeviceGetAttribute(&num_sms_, cudaDevAttrMultiProcessorCount, table_->device());
    set_sm_budget(0, 0);
    cudaDeviceSynchronize();
    std::vector<void*> self(1, symm_->local());
    if (W == 1) symm_->connect_local(self, 0);
}

SparseEngine::~SparseEngine() {
    cudaSetDevice(table_->device());
    cudaDeviceSynchronize();
    if (scratch_) cudaFree(scratch_);
    if (sorted_ids_) cudaFree(sorted_ids_);
    if (sorted_pos_) cudaFree(sorted_pos_);
    if (sort_temp_) cudaFree(sort_temp_);
}

Status SparseEngine::set_mirror(GpuTable* mirror) {
    if (mirror != nullptr) {
        if (!cfg_.replicate) return Status::InvalidConfig("set_mirror: the engine was built without the replica log (replicate=false)");
        if (mirror->dim() != table_->dim() || mirror->stride() != table_->stride() || mirror->device() != table_->device())
            return Status::InvalidConfig("set_mirror: the mirror table must have the layout and the device of the primary");
    }
    mirror_ = mirror;
    return Status::Ok();
}

Status SparseEngine::set_deterministic(bool on) {
    if (on && sort_temp_ == nullptr) {
        cudaSetDevice(table_->device());
        sort_temp_bytes_ = ordered_segment_sum_temp_bytes(cfg_.max_keys, table_->dim());
        if (cudaMalloc(&sorted_ids_, (size_t)cfg_.max_keys * 4) != cudaSuccess || cudaMalloc(&sorted_pos_, (size_t)cfg_.max_keys * 4) != cudaSuccess ||
            cudaMalloc(&sort_temp_, sort_temp_bytes_) != cudaSuccess) {
            cudaGetLastError();
            return Status::OOM("set_deterministic: no memory for the sort scratch");
        }
    }
    deterministic_ = on;
    return Status::Ok();
}

Status SparseEngine::connect(const std::vector<std::string>& handles) {
    if ((int)handles.size() != cfg_.world) return Status::InvalidConfig("connect: need one handle per rank");
    return symm_->connect(handles, cfg_.rank);
}

void SparseEngine::set_sm_budget(int pull_sms, int push_sms) {
    // No budget: 256-thread CTAs, four per SM, on every SM. With a budget the call runs as 1024-thread CTAs, each of
    // which fills an SM, so the grid size is the number of SMs the call occupies.
    pull_wide_ = pull_sms > 0;
    push_wide_ = push_sms > 0;
    pull_blocks_ = pull_wide_ ? std::min(max_pull_wide_, pull_sms) : max_pull_blocks_;
    push_blocks_ = push_wide_ ? std::min(max_push_wide_, push_sms) : max_push_blocks_;
    hot_rows_ = push_wide_ ? 64u : 24u;
}

void SparseEngine::connect_local(const std::vector<SparseEngine*>& engines) {
    std::vector<void*> ptrs;
    for (auto* e : engines) ptrs.push_back(e->symm_->local());
    symm_->connect_local(ptrs, cfg_.rank);
}

Status SparseEngine::set_shard_owner(const std::vector<int>& owner) {
    if ((int)owner.size() != std::max(cfg_.n_shards, 1)) return Status::InvalidConfig("shard_owner length != n_shards");
    for (int o : owner)
        if (o < 0 || o >= cfg_.world) return Status::InvalidConfig("shard owner out of range");
    cudaSetDevice(table_->device());
    cudaError_t e = cudaMemcpy(shard_owner_dev_, owner.data(), owner.size() * 4, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return Status::Error(cudaGetErrorString(e));
    shard_owner_host_ = owner;
    plan_valid_ = false;
    return Status::Ok();
}

void SparseEngine::fill_common(FusedArgs& a) const {
    a.world = cfg_.world;
    a.rank = cfg_.rank;
    a.C = C_;
    a.N = cfg_.max_keys;
    a.dim = table_->dim();
    a.limit_ns = (unsigned long long)(cfg_.wait_limit_s * 1e9);
    for (int r = 0; r < cfg_.world; ++r) {
        char* base = (char*)symm_->peer(r);
        unsigned* fl = (unsigned*)(base + off_flags_);
        a.peer[r].key_flag = fl;
        a.peer[r].key_cnt = fl + kMaxWorld;
        a.peer[r].row_flag = fl + 2 * kMaxWorld;
        a.peer[r].grad_flag = fl + 3 * kMaxWorld;
        a.peer[r].push_ack = fl + 4 * kMaxWorld;
        a.peer[r].mail_keys = (long long*)(base + off_mail_keys_);
        a.peer[r].mail_ret = (unsigned*)(base + off_mail_ret_);
        a.peer[r].rows_in = (float*)(base + off_rows_in_);
        a.peer[r].mail_grad = (float*)(base + off_mail_grad_);
        unsigned* rw = (unsigned*)(base + off_rep_words_);
        a.peer[r].rep_flag = rw;
        a.peer[r].rep_cnt = rw + 1;
        a.peer[r].rep_ack = rw + 2;
        a.peer[r].rep_keys = (long long*)(base + off_rep_keys_);
        a.peer[r].rep_grad = (float*)(base + off_rep_grad_);
    }
    a.dedup = dedup_;
    a.dmask = dedup_slots_ - 1;
    a.pos_slot = pos_slot_;
    a.inverse = inverse_;
    a.uniq_row = uniq_row_;
    a.uniq_slot = uniq_slot_;
    a.send_keys = send_keys_;
    a.send_ret = send_ret_;
    a.agg = agg_;
    a.res_slot = res_slot_;
    a.new_list = new_list_;
    a.ent_next = ent_next_;
    a.head_ids = head_ids_;
    a.chain_buf = chain_buf_;
    a.counters = counters_;
    a.in_cnt = in_cnt_;
    a.prof = profile_ ? prof_ : nullptr;
    a.shard_owner = shard_owner_dev_;
    a.n_shards = std::max(cfg_.n_shards, 1);
    a.table = table_->view_dev();
    a.mirror = mirror_ != nullptr ? mirror_->view_dev() : a.table;
    a.rep_slot = rep_slot_;
    a.rep_new = rep_new_;
}

Status SparseEngine::pull(const long long* keys, uint32_t n, uint32_t bag_size, void* out, unsigned flags,
                          void* stream) {
    if (failed_) return Status::Error("pull: the engine saw a fatal device status; call reset() on every rank first");
    if (n > cfg_.max_keys) return Status::InvalidConfig("pull: n exceeds max_keys of the engine");
    if ((flags & FUSED_OUT_BF16) && (table_->dim() % 8)) return Status::InvalidConfig("pull: bf16 output needs dim % 8 == 0");
    if (bag_size == 0 || n % bag_size != 0) return Status::InvalidConfig("pull: n must be a multiple of bag_size");
    if (symm_->world() != cfg_.world) return Status::Error("pull: peers are not connected");
    cudaSetDevice(table_->device());
    Status reserve = Status::Ok();
    if (flags & FUSED_INSERT) {
        // worst case every rank sends n new keys to this owner; bounded by the mailboxes
        const uint64_t worst = std::min<uint64_t>((uint64_t)cfg_.world * C_, (uint64_t)cfg_.world * n);  // keys this owner may receive
        Status grown = table_->maybe_grow(worst);   // index load: grows between launches, also under graph replay
        if (!grown.ok() && grown.code() != StatusCode::OUT_OF_MEMORY) return grown;
        reserve = table_->reserve_rows(worst);
    }
    FusedArgs a;
    fill_common(a);
    a.flags = flags;
    ++pull_epoch_;
    a.ctl = ctl_pull_;
    a.plan_ctl = ctl_pull_;
    a.keys = keys;
    a.n = n;
    a.bag_size = bag_size;
    a.out = out;
    a.grads = nullptr;
    a.hot_rows = 0;
    int rc = launch_fused_pull(a, pull_blocks_, pull_wide_, stream);
    ++launches_;
    if (flags & FUSED_INSERT) table_->refresh_usage_async(stream);
    if (rc != 0) return Status::Error(std::string("fused_pull launch: ") + cudaGetErrorString((cudaError_t)rc));
    plan_keys_ = keys;
    plan_n_ = n;
    plan_bag_ = bag_size;
    plan_flags_ = flags;
    plan_valid_ = true;
    plan_used_ = false;
    if (!reserve.ok() && reserve.code() != StatusCode::OUT_OF_MEMORY) return reserve;
    return Status::Ok();
}

Status SparseEngine::push(const float* grads, uint32_t n_rows, const OptConfig& opt, unsigned flags, void* stream) {
    if (failed_) return Status::Error("push: the engine saw a fatal device status; call reset() on every rank first");
    if (!plan_valid_) return Status::Error("push: no plan (call pull or plan first)");
    if (n_rows != 0 && n_rows != plan_n_ / plan_bag_)
        return Status::InvalidConfig("push: gradient rows (" + std::to_string(n_rows) + ") != pulled bags (" +
                                     std::to_string(plan_n_ / plan_bag_) + ")");
    cudaSetDevice(table_->device());
    if (plan_used_ || !(plan_flags_ & FUSED_PREPARE_PUSH)) {
        // a plan pushed twice, or made by a pull that did not prepare a push: the aggregation rows must start
        // from zero
        cudaMemsetAsync(agg_, 0, (size_t)plan_n_ * table_->dim() * 4, (cudaStream_t)stream);
    }
    if (deterministic_ && !(flags & FUSED_AGG_READY)) {
        // position-ordered sums of the duplicates, then the fused kernel without its own (atomic) segment sum
        const float scale = (plan_flags_ & FUSED_MEAN) && plan_bag_ > 1 ? 1.0f / (float)plan_bag_ : 1.0f;
        int rc0 = ordered_segment_sum(inverse_, plan_n_, cfg_.max_keys, counters_, &ctl_pull_->epoch, grads, plan_bag_, table_->dim(), scale,
                                      agg_, sorted_ids_, sorted_pos_, sort_temp_, sort_temp_bytes_, stream);
        if (rc0 != 0) return Status::Error(std::string("ordered_segment_sum: ") + cudaGetErrorString((cudaError_t)rc0));
        flags |= FUSED_AGG_READY;
    }
    FusedArgs a;
    fill_common(a);
    a.flags = (plan_flags_ & FUSED_MEAN) | (flags & (FUSED_SYNC_PUSH | FUSED_AGG_READY));
    if (grad_wire_bf16_) a.flags |= FUSED_GRAD_BF16;
    if (mirror_ != nullptr) {
        a.flags |= FUSED_REPLICATE;
        // the mirror may get a row for every entry of the mirrored rank's log
        Status rs = mirror_->reserve_rows(std::min<uint64_t>((uint64_t)cfg_.world * C_, (uint64_t)cfg_.world * plan_n_));
        if (!rs.ok() && rs.code() != StatusCode::OUT_OF_MEMORY) return rs;
    }
    ++push_epoch_;
    a.ctl = ctl_push_;
    a.plan_ctl = ctl_pull_;
    a.keys = plan_keys_;
    a.n = plan_n_;
    a.bag_size = plan_bag_;
    a.out = nullptr;
    a.grads = grads;
    a.opt = opt;
    a.hot_rows = hot_rows_;
    int rc = launch_fused_push(a, push_blocks_, push_wide_, stream);
    ++launches_;
    if (mirror_ != nullptr) mirror_->refresh_usage_async(stream);
    if (rc != 0) return Status::Error(std::string("fused_push launch: ") + cudaGetErrorString((cudaError_t)rc));
    plan_used_ = true;
    return Status::Ok();
}

Status SparseEngine::check(void* stream) {
    cudaSetDevice(table_->device());
    KernelCtl h[2];
    cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) return Status::Fatal(std::string("stream: ") + cudaGetErrorString(e));
    e = cudaMemcpy(&h[0], ctl_pull_, sizeof(KernelCtl), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess) e = cudaMemcpy(&h[1], ctl_push_, sizeof(KernelCtl), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return Status::Fatal(std::string("status read: ") + cudaGetErrorString(e));
    for (int k = 0; k < 2; ++k) {
        if (h[k].status == 0) continue;
        failed_ = true;
        std::string msg = where_name(h[k].where);
        switch (h[k].status) {
            case kStTimeout: return Status::Timeout(msg);
            default: return Status::Error(msg);
        }
    }
    for (int k = 0; k < 2; ++k) {
        if (h[k].soft == 0) continue;
        // memory pressure: the call ran to its end (reads of a row-less key saw its initial value, writes to it
        // were dropped); report it once
        KernelCtl* ctl = k == 0 ? ctl_pull_ : ctl_push_;
        cudaMemset(&ctl->soft, 0, 2 * sizeof(unsigned));
        if (k == 0) cudaMemset(&ctl_push_->soft, 0, 2 * sizeof(unsigned));
        table_->set_healthy(false);
        return Status::OOM(where_name(h[k].soft_where));
    }
    return Status::Ok();
}

Status SparseEngine::reset(void* stream) {
    cudaSetDevice(table_->device());
    cudaStream_t s = (cudaStream_t)stream;
    cudaStreamSynchronize(s);
    // keep the shard map (last carve) and the table; clear everything else
    const size_t keep_from = (char*)shard_owner_dev_ - scratch_;
    cudaMemsetAsync(scratch_, 0, keep_from, s);
    fill_dedup_kernel<<<148 * 4, 256, 0, s>>>(dedup_, dedup_slots_);
    cudaMemsetAsync((char*)symm_->local() + off_flags_, 0, 5 * kMaxWorld * sizeof(unsigned), s);
    if (cfg_.replicate) cudaMemsetAsync((char*)symm_->local() + off_rep_words_, 0, 4 * sizeof(unsigned), s);
    table_->clear_aux(s);  // a push that was cut short leaves its row chains behind
    cudaError_t e = cudaStreamSynchronize(s);
    pull_epoch_ = push_epoch_ = 0;
    plan_valid_ = false;
    failed_ = false;
    if (e != cudaSuccess) return Status::Fatal(cudaGetErrorString(e));
    return Status::Ok();
}

std::vector<uint64_t> SparseEngine::phase_stamps(void* stream) {
    cudaSetDevice(table_->device());
    cudaStreamSynchronize((cudaStream_t)stream);
    std::vector<uint64_t> v(16, 0);
    cudaMemcpy(v.data(), prof_, 16 * 8, cudaMemcpyDeviceToHost);
    return v;
}

std::vector<uint64_t> SparseEngine::cta_stamps(int which, void* stream) {
    cudaSetDevice(table_->device());
    cudaStreamSynchronize((cudaStream_t)stream);
    std::vector<uint64_t> v(kProfMaxCtas, 0);
    if (which < 0 || which > 3) return v;
    cudaMemcpy(v.data(), prof_ + 16 + (size_t)which * kProfMaxCtas, kProfMaxCtas * 8, cudaMemcpyDeviceToHost);
    return v;
}

uint32_t SparseEngine::last_unique(void* stream) {
    cudaSetDevice(table_->device());
    cudaStreamSynchronize((cudaStream_t)stream);
    KernelCtl h;
    cudaMemcpy(&h, ctl_pull_, sizeof(h), cudaMemcpyDeviceToHost);
    unsigned v = 0;
    cudaMemcpy(&v, counters_ + (h.epoch & 1u) * 16, 4, cudaMemcpyDeviceToHost);
    return v;
}

}  // namespace psb
