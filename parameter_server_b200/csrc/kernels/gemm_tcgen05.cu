// bf16 GEMM for sm_100a on the 5th-generation tensor cores: tcgen05.mma issued by one elected
// thread, operands staged in shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle, no
// multicast), fp32 accumulators in TMEM, read back with tcgen05.ld for a fused epilogue.
//
//   D[M,N] = epilogue( sum_k A(m,k) * B(n,k) )
//
// Each operand is described by a 2-D row-major tensor in global memory and a "major":
//   K-major  : the tensor is [rows = M or N][cols = K]   (contraction index contiguous)
//   MN-major : the tensor is [rows = K][cols = M or N]   (contraction index strided)
// so that the three GEMMs of a linear layer y = x W^T run without any transposed copy:
//   forward  y  = x  W^T   : A = x  (K-major),  B = W  (K-major)
//   dgrad    dx = dy W     : A = dy (K-major),  B = W  (MN-major; W is [N_out][K_in] = [k][n])
//   wgrad    dW = dy^T x   : A = dy (MN-major), B = x  (MN-major)
// Epilogue (all optional): + bias[n], ReLU, multiply by (mask[m,n] > 0) (ReLU backward), add to the
// existing fp32 output; output bf16 or fp32, row-major with leading dimension ldd.
//
// Not in the reference (it has no model code); this is the dense-MLP kernel of the DLRM and GPT
// workloads and the compute half of the fused dense pull.
//
// Structure per CTA (320 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 2..9 = epilogue (two warps per 32-lane quarter of TMEM, each taking half of the tile's columns; the
// TMEM load of the next 32-column chunk is in flight while the current one is converted and stored, and the
// tile's bias is staged in shared memory before the accumulator is ready). One 128 x BN tile per CTA,
// BK = 64 (one 128-byte swizzle span), kStages-deep mbarrier ring. Every mbarrier wait is bounded;
// on a time-out the CTA records an error, still frees its TMEM and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "gemm_tcgen05.h"

namespace psb {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kEpilogueWarps = 8;
// Warp roles: warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2-9 epilogue, warp 10 publisher (chain mode:
// bumps the completion counters for the epilogue warps). Moving registers from the single-thread roles to the
// epilogue warps (setmaxnreg) was tried and dropped: the producer and MMA code paths need about as many registers
// as the epilogue, and with 168 for everybody nothing spills.
constexpr int kFirstEpilogueWarp = 2;
constexpr int kPublisherWarp = kFirstEpilogueWarp + kEpilogueWarps;
constexpr int kThreads = 32 * (kPublisherWarp + 1);

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long gtimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait; returns false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned long long limit_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = gtimer();
    unsigned spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 255u) == 0 && gtimer() - t0 > limit_ns) return false;
    }
    return true;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

// Output path of the epilogue: a warp stages a [32 rows][64 bytes] piece of the tile in shared memory and one lane
// hands it to the TMA unit, which writes whole lines (rows and columns outside the tensor are clipped by the map).
// A thread-per-row store would touch 32 different lines per instruction and keeps the load/store unit busy for
// longer than the MMAs of a small-K tile take.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"((uint64_t)map), "r"(smem_u32(src)), "r"(c0), "r"(c1)
                 : "memory");
}
// Same, adding to what is in global memory (fp32): the split-K partial sums and `accumulate` outputs.
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, const void* src, int c0, int c1) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"((uint64_t)map), "r"(smem_u32(src)), "r"(c0), "r"(c1)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ uint4 ld_nc_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void bulk_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Shared-memory matrix descriptor (version 1 = Blackwell), 128-byte swizzle.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;  // descriptor version
    d |= (uint64_t)2 << 61;  // SWIZZLE_128B
    return d;
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// ---- CTA pairs (cta_group::2) -------------------------------------------------------------------------
// Two CTAs of a cluster work on one 256-row tile: each holds its own 128 rows of A, HALF of the B tile and the
// accumulator of its 128 rows in its own TMEM; one thread of the leader (cluster rank 0) issues the MMAs for both.
// Each SM then reads and fills half as many B bytes per flop: the 1-CTA 128 x 256 tile needs about 96 B/clk of
// operand reads plus as much again for the TMA fill, more than one SM's shared memory delivers.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of `local` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_cluster(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Loads of a pair: the data lands in this CTA, the bytes are counted on the LEADER's barrier (no multicast: every
// CTA fetches its own tiles).
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(bar_cluster), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(bar_cluster), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on the barrier at this offset in BOTH CTAs of the pair once the MMAs issued so far have completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"((uint16_t)3)
                 : "memory");
}

// Issue the load of 32 accumulator columns (one row per lane); the registers are valid after tmem_wait_ld.
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
// Wait for every TMEM load this thread has issued. The registers of the chunk about to be used are operands, so
// that nothing that reads them can be scheduled ahead of the wait.
__device__ __forceinline__ void tmem_wait_ld(uint32_t* v) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]),
                   "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15]),
                   "+r"(v[16]), "+r"(v[17]), "+r"(v[18]), "+r"(v[19]), "+r"(v[20]), "+r"(v[21]), "+r"(v[22]), "+r"(v[23]),
                   "+r"(v[24]), "+r"(v[25]), "+r"(v[26]), "+r"(v[27]), "+r"(v[28]), "+r"(v[29]), "+r"(v[30]), "+r"(v[31])
                 :
                 : "memory");
}

template <int BN, bool PAIR = false>
struct SmemLayout {
    static constexpr int kABytes = BM * BK * 2;   // 16 KB
    static constexpr int kBBytes = (PAIR ? BN / 2 : BN) * BK * 2;   // a CTA of a pair holds half of the B tile
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kStages = PAIR ? ((BN == 256) ? 6 : 8) : ((BN == 256) ? 4 : 6);
    static constexpr int kTileBytes = kStages * kStageBytes;
    static constexpr int kBarBytes = 256;
    static constexpr int kBiasBytes = 2 * 256 * 4;  // the bias of a tile's columns, double-buffered with the accumulator
    static constexpr int kStageOutBytes = kEpilogueWarps * 2048;  // per epilogue warp: [32 rows][64 bytes] output staging
    static constexpr int kTotal = kTileBytes + kBarBytes + kBiasBytes + kStageOutBytes + 1024;  // + alignment slack
};

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
constexpr uint32_t kPubExit = 0xFFFFFFFFu;
__device__ __forceinline__ uint32_t ld_acquire_cta_smem(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_cta_smem(uint32_t* p, uint32_t v) {
    asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}
// One lane of an epilogue warp hands a request to the publisher warp (waits, bounded, for the slot to be free).
__device__ __forceinline__ void post_publish(uint32_t* box, uint32_t req, unsigned long long limit_ns, unsigned* err_flag) {
    if (ld_acquire_cta_smem(box) != 0u) {
        const unsigned long long t0 = gtimer();
        unsigned spins = 0;
        while (ld_acquire_cta_smem(box) != 0u) {
            if ((++spins & 63u) == 0 && gtimer() - t0 > limit_ns) {
                atomicCAS(err_flag, 0u, 8u);
                return;
            }
        }
    }
    st_release_cta_smem(box, req);
}


// ReLU-backward mask of one piece read straight from global memory (rows whose mask was not prefetched).
__device__ __noinline__ void apply_mask_slow(const GemmEpilogue& ep, float* f, int row, int col0, int N) {
    const bool full = (col0 + 32 <= N);
    {
        const __nv_bfloat16* mp = ep.mask + (size_t)row * ep.ldmask + col0;
        if (full && (ep.ldmask % 8 == 0)) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
                uint4 raw = *(const uint4*)(mp + j);
                const __nv_bfloat16* h = (const __nv_bfloat16*)&raw;
#pragma unroll
                for (int t = 0; t < 8; ++t)
                    if (!(__bfloat162float(h[t]) > 0.f)) f[j + t] = 0.f;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (col0 + j < N && !(__bfloat162float(mp[j]) > 0.f)) f[j] = 0.f;
        }
    }
}

// Epilogue of one 32-column chunk held by one thread (one output row). `bias_s`: the chunk's 32 bias values in
// shared memory (every lane reads the same words: a broadcast), or nullptr.
// mpre != nullptr: the chunk's 32 mask values were loaded ahead of time (4 x uint4, this lane's row).
// LEAN_FWD / LEAN_BWD: the lean launches of a forward layer (bias and activation, never a mask) and of a dgrad layer
// (a prefetched mask, never bias or activation) carry only their own code.
template <bool LEAN_FWD = false, bool LEAN_BWD = false>
__device__ __forceinline__ void epilogue_chunk(const GemmEpilogue& ep, float* f, int row, int col0, int N,
                                               const float* bias_s, bool row_valid, const uint4* mpre = nullptr) {
    constexpr bool LEAN = LEAN_FWD || LEAN_BWD;
    if constexpr (!LEAN_BWD) {
    if (bias_s != nullptr) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
            const float4 b = *(const float4*)(bias_s + j);
            f[j] += b.x; f[j + 1] += b.y; f[j + 2] += b.z; f[j + 3] += b.w;
        }
    }
    if constexpr (!LEAN_FWD) {   // the lean forward kernel applies the activation to the packed pairs
    if (ep.relu) {
#pragma unroll
        for (int j = 0; j < 32; ++j) f[j] = fmaxf(f[j], 0.f);
    }
    }
    }
    if constexpr (LEAN) return;
    if (mpre != nullptr) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
            const __nv_bfloat16* h = (const __nv_bfloat16*)&mpre[j / 8];
#pragma unroll
            for (int t = 0; t < 8; ++t)
                if (!(__bfloat162float(h[t]) > 0.f)) f[j + t] = 0.f;
        }
        return;
    }
    if constexpr (LEAN) return;   // a mask of a lean launch is always prefetched
    if (ep.mask != nullptr && row_valid) {
        // not prefetched (partial piece or unaligned mask): the slow path, kept out of the loop's code
        float tmp[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) tmp[j] = f[j];
        apply_mask_slow(ep, tmp, row, col0, N);
#pragma unroll
        for (int j = 0; j < 32; ++j) f[j] = tmp[j];
    }
}

// fp32 output of one 32-column piece: two [32 rows][16 cols] halves through the warp's staging piece and the TMA unit
// (store, or reduce-add for split-K partial sums and `accumulate`). Called by the whole warp.
__device__ __noinline__ void store_piece_f32(const CUtensorMap* map_d, int d_mode, uint8_t* stage, int lane, const float* f,
                                             int col0, int row0, int N) {
    uint8_t* my_stage = stage + lane * 64;
#pragma unroll 1
    for (int hcol = 0; hcol < 32; hcol += 16) {
        if (col0 + hcol >= N) break;   // warp-uniform
#pragma unroll
        for (int j = 0; j < 16; j += 4)
            *(float4*)(my_stage + j * 4) = make_float4(f[hcol + j], f[hcol + j + 1], f[hcol + j + 2], f[hcol + j + 3]);
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
            if (d_mode == 2) tma_reduce_add_2d(map_d, stage, col0 + hcol, row0);
            else tma_store_2d(map_d, stage, col0 + hcol, row0);
            bulk_commit();
            if (hcol == 0) bulk_wait_read0();   // the second half follows at once
        }
        if (hcol == 0) __syncwarp();
    }
}

// The thread-per-row output path (d_mode 0). Out of line, like every rarely taken path of the epilogue: the loop
// over a tile's pieces must stay small enough for the instruction cache close to the schedulers; with all paths
// inlined a piece cost about 8 cycles per instruction.
__device__ __noinline__ void store_chunk_rows(const GemmEpilogue& ep, const float* f, int row, int col0, int N) {
    const bool full = (col0 + 32 <= N);
    if (ep.out_f32 != nullptr) {
        float* op = ep.out_f32 + (size_t)row * ep.ldd + col0;
        if (ep.split_k > 1) {
            if (full && (ep.ldd % 4 == 0)) {
#pragma unroll
                for (int j = 0; j < 32; j += 4) atomicAdd((float4*)(op + j), make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]));
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (col0 + j < N) atomicAdd(op + j, f[j]);
            }
        } else if (full && (ep.ldd % 4 == 0)) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
                float4 o = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
                if (ep.accumulate) {
                    float4 old = *(float4*)(op + j);
                    o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                *(float4*)(op + j) = o;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (col0 + j < N) op[j] = ep.accumulate ? op[j] + f[j] : f[j];
        }
    }
    if (ep.out_bf16 != nullptr) {
        __nv_bfloat16* op = ep.out_bf16 + (size_t)row * ep.ldd + col0;
        if (full && (ep.ldd % 8 == 0)) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
                uint4 raw;
                __nv_bfloat162* h = (__nv_bfloat162*)&raw;
                h[0] = __floats2bfloat162_rn(f[j], f[j + 1]);
                h[1] = __floats2bfloat162_rn(f[j + 2], f[j + 3]);
                h[2] = __floats2bfloat162_rn(f[j + 4], f[j + 5]);
                h[3] = __floats2bfloat162_rn(f[j + 6], f[j + 7]);
                *(uint4*)(op + j) = raw;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (col0 + j < N) op[j] = __float2bfloat16_rn(f[j]);
        }
    }
}

__device__ __forceinline__ unsigned ld_acquire_gpu_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// All-gather role of a CTA: copy the row blocks of B that other ranks own and that are assigned to this CTA from the
// owners' memory into the local copy of B with bulk async copies staged through shared memory, and publish each
// n-tile's flag. One thread drives a ring of kDepth staging buffers: the load of piece j + kDepth - 1 is issued
// before the store of piece j, a buffer is reloaded as soon as the store that used it has READ it
// (`wait_group.read`), and nothing waits for a store to complete except the flag of an n-tile. So kDepth - 1 loads
// are always in flight over NVLink while the stores drain into local memory (one round trip per piece otherwise).
template <int BN>
__device__ void gather_rows(const GemmGather& ag, int K, uint8_t* smem, uint64_t* bars, unsigned* err_flag,
                            unsigned long long limit_ns, int N) {
    constexpr int kDepth = 6;
    constexpr uint32_t kPiece = 32768;
    if (threadIdx.x != 0) return;
    for (int d = 0; d < kDepth; ++d) mbar_init(&bars[d], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const int n_tiles = (N + BN - 1) / BN;
    const int tpr = ag.rows_per_rank / BN;
    const size_t tile_bytes = (size_t)BN * K * 2;
    const uint32_t pieces_per_tile = (uint32_t)((tile_bytes + kPiece - 1) / kPiece);
    // this CTA's n-tiles, in the order the GEMM CTAs will ask for them
    int my_tiles = 0;
    for (int j = tpr, order = 0; j < n_tiles; ++j, ++order)
        if (order % ag.gather_ctas == (int)blockIdx.x) ++my_tiles;
    const uint32_t total = (uint32_t)my_tiles * pieces_per_tile;
    auto tile_of = [&](uint32_t t) -> int {   // t-th tile of this CTA -> n-tile index
        const int j = tpr + (int)blockIdx.x + (int)t * ag.gather_ctas;
        return (j + ag.rank * tpr) % n_tiles;
    };
    auto issue_load = [&](uint32_t q) {
        const uint32_t t = q / pieces_per_tile, i = q % pieces_per_tile;
        const int nt = tile_of(t);
        const size_t o = (size_t)i * kPiece;
        const uint32_t bytes = (uint32_t)min((size_t)kPiece, tile_bytes - o);
        const uint8_t* src = (const uint8_t*)ag.peer_b[nt / tpr] + (size_t)nt * tile_bytes + o;
        const int d = (int)(q % kDepth);
        mbar_expect_tx(&bars[d], bytes);
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                         smem_u32(smem + (size_t)d * kPiece)),
                     "l"(src), "r"(bytes), "r"(smem_u32(&bars[d]))
                     : "memory");
    };
    // prologue: kDepth - 1 loads in flight
    for (uint32_t q = 0; q < total && q < (uint32_t)(kDepth - 1); ++q) issue_load(q);
    for (uint32_t q = 0; q < total; ++q) {
        const int d = (int)(q % kDepth);
        // next load: its buffer was last used by the store of piece q - 1, committed one group ago
        const uint32_t qn = q + (uint32_t)(kDepth - 1);
        if (qn < total) {
            if (q > 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            issue_load(qn);
        }
        if (!mbar_wait(&bars[d], (q / kDepth) & 1u, limit_ns)) {
            atomicCAS(err_flag, 0u, 6u);
            // the loads still in flight land in this CTA's shared memory: let them finish (bounded) before leaving
            for (uint32_t w = q + 1; w < total && w <= qn; ++w) mbar_wait(&bars[w % kDepth], (w / kDepth) & 1u, limit_ns);
            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
            return;
        }
        const uint32_t t = q / pieces_per_tile, i = q % pieces_per_tile;
        const int nt = tile_of(t);
        const size_t o = (size_t)i * kPiece;
        const uint32_t bytes = (uint32_t)min((size_t)kPiece, tile_bytes - o);
        uint8_t* dst = (uint8_t*)ag.local_b + (size_t)nt * tile_bytes + o;
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst),
                     "r"(smem_u32(smem + (size_t)d * kPiece)), "r"(bytes)
                     : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        if (i + 1 == pieces_per_tile) {
            // the n-tile is complete once its stores are: publish its flag (loads of the next tile stay in flight)
            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
            asm volatile("fence.proxy.async.global;" ::: "memory");
            __threadfence();
            asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(ag.ready + nt), "r"(ag.epoch) : "memory");
        }
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// One launch can carry several independent GEMMs (a "group": e.g. the weight gradients of every layer of an
// MLP, which all become computable at the end of the backward pass). The persistent CTAs walk one list of
// work units that covers the problems back to back, so small problems fill the machine together and pay one
// prologue. All problems of a launch share the tile shape and the operand majors.
constexpr int kMaxGroup = 8;
struct GemmProblemSet {
    CUtensorMap map_a[kMaxGroup];
    CUtensorMap map_b[kMaxGroup];
    GemmEpilogue ep[kMaxGroup];
    int M[kMaxGroup], N[kMaxGroup], K[kMaxGroup];
    int unit_end[kMaxGroup];  // running total of work units (m tile x n tile x k split) up to and including problem i
    // An MN-major operand whose MN extent is a multiple of 64 is described by a 3-D tensor map
    // (64 elements, K rows, MN / 64 column blocks), so that ONE bulk-tensor load brings all the 64-wide column blocks
    // of a stage (2 for A, BN / 64 for B) instead of one load per block: the single producer thread then issues two
    // loads per k-step for every operand layout.
    unsigned char a_blocked[kMaxGroup], b_blocked[kMaxGroup];
    // How the epilogue writes problem i: 0 = one thread per row (any alignment, both outputs), 1 = bf16 through a
    // shared-memory piece and 16-byte stores that cover whole row segments, 2 = TMA reduce-add of fp32
    // [32 rows][16 cols] pieces (split-K partial sums, `accumulate`), 3 = TMA store of fp32 pieces (map_d: 2 and 3).
    CUtensorMap map_d[kMaxGroup];
    unsigned char d_mode[kMaxGroup];
    // Tracing (off when null): CTA 0 writes %globaltimer stamps, 32 slots for each of the first 8 work units it runs:
    // 0 producer starts the unit's loads, 1 producer issued the last load, 2 MMA warp owns an accumulator buffer,
    // 3 first operand stage arrived, 4 accumulator complete (committed), 8 epilogue warp 0 sees the accumulator,
    // 5 all epilogue warps do, 9 first TMEM piece in registers, 10 first piece staged, 11 first piece handed to
    // the TMA store, 6 last piece handed to the TMA store, 7 unit index, 20 / 21 the SM's cycle counter at 3 and 4 (their ratio to the timer gives the SM clock); inside the first piece:
    // 15 bias / activation / mask applied, 16 piece written to shared memory.
    unsigned long long* trace;
    int epi_skip;   // diagnosis only (PSB_GEMM_EPI_SKIP): 1 = no bias / activation / mask, 2 = no staging and no stores, 4 = no global stores
    int count;
    // Chain: problem i + 1 reads the output of problem i as its A operand (the layers of an MLP, forward or dgrad).
    // done[i * kMaxChainMTiles + m] counts the epilogue warps that have stored their part of an n-tile of row block m
    // of problem i; a unit of problem i + 1 waits until all of row block m is there. Zeroed before every launch.
    int chain;
    unsigned* done;
};
constexpr int kMaxChainMTiles = 1024;

struct WorkUnit {
    int p;                    // problem index
    int tile_m, tile_n, nt;   // element offsets of the tile, n-tile index
    int kt_begin, num_kt;     // k-tile range of this split
};

// PAIR: a unit covers 256 rows; the CTA of cluster rank `cr` works on rows [tile_m, tile_m + 128) = the unit's
// rows + 128 * cr (which may lie past M: the loads then read zeros and the stores are clipped).
template <int BN, bool PAIR>
__device__ __forceinline__ WorkUnit decode_unit(const GemmProblemSet& ps, int u, const GemmGather& ag, int cr) {
    constexpr int BMU = PAIR ? 2 * BM : BM;
    WorkUnit w;
    int p = 0;
    while (p + 1 < ps.count && u >= ps.unit_end[p]) ++p;
    w.p = p;
    const int local = u - (p > 0 ? ps.unit_end[p - 1] : 0);
    const int m_tiles = (ps.M[p] + BMU - 1) / BMU;
    const int n_tiles = (ps.N[p] + BN - 1) / BN;
    const int splits = ps.ep[p].split_k > 1 ? ps.ep[p].split_k : 1;
    const int total_kt = (ps.K[p] + BK - 1) / BK;
    const int kt_per = (total_kt + splits - 1) / splits;
    const int z = local / (m_tiles * n_tiles);
    const int rem = local - z * (m_tiles * n_tiles);
    int nt = rem / m_tiles;  // m fastest: CTAs that run together share the B tile in L2
    int mt = rem % m_tiles;
    if (ps.chain) {
        // n fastest: a row block of this layer is complete after n_tiles consecutive units, so the next layer can
        // start on it while this layer is still working on later row blocks (the weights stay in L2 either way)
        nt = rem % n_tiles;
        mt = rem / n_tiles;
    }
    if (ag.enabled) nt = (nt + ag.rank * (ag.rows_per_rank / BN)) % n_tiles;  // local rows first, then ring order
    w.nt = nt;
    w.tile_n = nt * BN;
    w.tile_m = mt * BMU + cr * BM;
    w.kt_begin = z * kt_per;
    w.num_kt = max(0, min(total_kt - w.kt_begin, kt_per));
    return w;
}

// Persistent kernel: gridDim.x CTAs (one per SM) walk the tile list t = blockIdx.x, +gridDim.x, ...;
// a tile is (split z, n tile, m tile) with m fastest so that concurrently running CTAs share the B
// tile in L2. The accumulator is double-buffered in TMEM (2 x BN columns): while the epilogue warps
// drain buffer b, the MMA warp already fills buffer b^1 with the next tile.
// AMN / BMN: operand is MN-major. The box of an MN-major operand is [64 k-rows][64 mn-elements].
// PAIR: launched as clusters of two CTAs that share every work unit (see the CTA-pair helpers above); the gather
// role exists only without it.
// LEAN: every problem of the launch writes bf16 through the staged path, N is a multiple of 32 and a mask (if any) has
// 16-byte aligned rows: the epilogue loop is compiled without the other output paths, the partial-piece code, the
// tracing stamps and the diagnostic switch. The loop is bound by instruction fetch, so less code is less time.
template <int BN, bool AMN, bool BMN, bool PAIR, bool LEAN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ GemmProblemSet ps, unsigned* err_flag, unsigned long long limit_ns,
                         const GemmGather ag) {
    using L = SmemLayout<BN, PAIR>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full_bar = (uint64_t*)(smem + L::kTileBytes);
    uint64_t* empty_bar = full_bar + L::kStages;
    uint64_t* tfull_bar = empty_bar + L::kStages;   // [2] accumulator buffer complete
    uint64_t* tempty_bar = tfull_bar + 2;           // [2] accumulator buffer drained
    uint32_t* tmem_slot = (uint32_t*)(tempty_bar + 2);
    // Chain mode: one mailbox per epilogue warp. The warp posts (index of a completion counter) + 1 once the stores
    // of a tile are complete; a lane of the publisher warp fences and bumps the counter, so that no epilogue warp
    // ever waits for a device-scope fence. 0 = empty, kPubExit = no more requests.
    uint32_t* pub_req = tmem_slot + 2;   // [kEpilogueWarps]
    float* bias_smem = (float*)(smem + L::kTileBytes + L::kBarBytes);   // [2][256]
    uint8_t* stage_out = smem + L::kTileBytes + L::kBarBytes + L::kBiasBytes;   // [kEpilogueWarps][2048]

    // ---- all-gather role: the first ag.gather_ctas CTAs move remote row blocks of B into the local copy ----
    const int n_gather = (!PAIR && ag.enabled) ? ag.gather_ctas : 0;
    if constexpr (!PAIR) {
        if ((int)blockIdx.x < n_gather) {
            gather_rows<BN>(ag, ps.K[0], smem, full_bar, err_flag, limit_ns, ps.N[0]);
            return;
        }
    }
    // the walker index: a CTA, or a pair of CTAs
    const int cr = PAIR ? (int)cluster_ctarank() : 0;
    const int cta = PAIR ? (int)blockIdx.x / 2 : (int)blockIdx.x - n_gather;
    const int n_cta = PAIR ? (int)gridDim.x / 2 : (int)gridDim.x - n_gather;
    const bool leader = cr == 0;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int total_units = ps.unit_end[ps.count - 1];

    if (threadIdx.x < kEpilogueWarps) pub_req[threadIdx.x] = 0;
    if (threadIdx.x == 0) {
        for (int s = 0; s < L::kStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tfull_bar[b], 1);
            // one arrival per epilogue warp (of both CTAs of a pair: the leader's barrier collects them)
            mbar_init(&tempty_bar[b], PAIR ? 2 * kEpilogueWarps : kEpilogueWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        if constexpr (PAIR) {
            // executed by one warp of each CTA of the pair: the columns are allocated in both tensor memories
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                         "r"((uint32_t)(2 * BN))
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                         "r"((uint32_t)(2 * BN))
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    if constexpr (PAIR) cluster_sync_all();   // the peer's barriers must exist before anything is signalled on them
    else __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *((volatile uint32_t*)tmem_slot);
    // Programmatic dependent launch: everything above (barriers, TMEM) touched no global memory, so it may
    // run while the previous kernel of the stream drains; from here on its results are needed. Without the
    // launch attribute both instructions do nothing.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            for (int p = 0; p < ps.count; ++p) {
                asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&ps.map_a[p]) : "memory");
                asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&ps.map_b[p]) : "memory");
                if (ps.d_mode[p] >= 2) asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&ps.map_d[p]) : "memory");
            }
            uint32_t it = 0;  // k-tile counter across all tiles of this CTA (drives the stage ring)
            bool ok = true;
            for (int unit = cta; unit < total_units && ok; unit += n_cta) {
                const WorkUnit w = decode_unit<BN, PAIR>(ps, unit, ag, cr);
                if (ag.enabled) {
                    // a remote n-tile must have landed before it is loaded
                    const int tpr = ag.rows_per_rank / BN;
                    const int nt = w.nt;
                    if (nt / tpr != ag.rank) {
                        const unsigned long long t0 = gtimer();
                        unsigned spins = 0;
                        while ((int)(ld_acquire_gpu_u32(ag.ready + nt) - ag.epoch) < 0) {
                            if ((++spins & 63u) == 0 && gtimer() - t0 > limit_ns) {
                                atomicCAS(err_flag, 0u, 5u);
                                ok = false;
                                break;
                            }
                        }
                        if (!ok) break;
                        asm volatile("fence.proxy.async.global;" ::: "memory");
                    }
                }
                if (ps.chain && w.p > 0 && w.tile_m < ps.M[w.p]) {
                    // the A operand is the previous layer's output: all n-tiles of this row block must be stored
                    const int prev_n_tiles = (ps.N[w.p - 1] + BN - 1) / BN;
                    const unsigned target = (unsigned)kEpilogueWarps * (unsigned)prev_n_tiles;  // every epilogue warp of every tile
                    const unsigned* cnt = ps.done + (size_t)(w.p - 1) * kMaxChainMTiles + w.tile_m / BM;
                    const unsigned long long t0 = gtimer();
                    unsigned spins = 0;
                    while (ld_acquire_gpu_u32(cnt) < target) {
                        if ((++spins & 63u) == 0 && gtimer() - t0 > limit_ns) {
                            atomicCAS(err_flag, 0u, 7u);
                            ok = false;
                            break;
                        }
                    }
                    if (!ok) break;
                    // the rows were written with ordinary stores; the loads below go through the async proxy
                    asm volatile("fence.proxy.async.global;" ::: "memory");
                }
                const CUtensorMap* map_a = &ps.map_a[w.p];
                const CUtensorMap* map_b = &ps.map_b[w.p];
                const int tile_n = w.tile_n, tile_m = w.tile_m, kt_begin = w.kt_begin, num_kt = w.num_kt;
                const int tslot = (unit - cta) / n_cta;
                if (ps.trace != nullptr && cta == 0 && leader && tslot < 8) {
                    ps.trace[tslot * 32 + 0] = gtimer();
                    ps.trace[tslot * 32 + 7] = (unsigned long long)unit;
                }
                for (int kt = 0; kt < num_kt; ++kt, ++it) {
                    const int s = it % L::kStages;
                    const uint32_t ph = (it / L::kStages) & 1u;
                    if (!mbar_wait(&empty_bar[s], ph ^ 1u, limit_ns)) {
                        atomicCAS(err_flag, 0u, 1u);
                        ok = false;
                        break;
                    }
                    uint8_t* sa = smem + s * L::kStageBytes;
                    uint8_t* sb = sa + L::kABytes;
                    const int k0 = (kt_begin + kt) * BK;
                    if constexpr (PAIR) {
                        // both CTAs' bytes are counted on the leader's barrier
                        if (leader) mbar_expect_tx(&full_bar[s], 2u * (uint32_t)L::kStageBytes);
                        const uint32_t fb = mapa_cluster(smem_u32(&full_bar[s]), 0);
                        const int bn0 = tile_n + cr * (BN / 2);   // this CTA's half of the B tile
                        if (!AMN) {
                            tma_load_2d_pair(sa, map_a, fb, k0, tile_m);  // box [128 rows][64 k]
                        } else if (ps.a_blocked[w.p]) {
                            tma_load_3d_pair(sa, map_a, fb, 0, k0, tile_m / 64);  // box [2 blocks][64 k][64 m]
                        } else {
                            tma_load_2d_pair(sa, map_a, fb, tile_m, k0);  // box [64 k][64 m]
                            tma_load_2d_pair(sa + 64 * 128, map_a, fb, tile_m + 64, k0);
                        }
                        if (!BMN) {
                            tma_load_2d_pair(sb, map_b, fb, k0, bn0);  // box [BN / 2 rows][64 k]
                        } else if (ps.b_blocked[w.p]) {
                            tma_load_3d_pair(sb, map_b, fb, 0, k0, bn0 / 64);  // box [BN / 128 blocks][64 k][64 n]
                        } else {
#pragma unroll
                            for (int j = 0; j < BN / 128; ++j)
                                tma_load_2d_pair(sb + j * 64 * 128, map_b, fb, bn0 + 64 * j, k0);
                        }
                        continue;
                    }
                    mbar_expect_tx(&full_bar[s], (uint32_t)L::kStageBytes);
                    if (!AMN) {
                        tma_load_2d(sa, map_a, &full_bar[s], k0, tile_m);  // box [128 rows][64 k]
                    } else if (ps.a_blocked[w.p]) {
                        tma_load_3d(sa, map_a, &full_bar[s], 0, k0, tile_m / 64);  // box [2 blocks][64 k][64 m]
                    } else {
                        tma_load_2d(sa, map_a, &full_bar[s], tile_m, k0);  // box [64 k][64 m]
                        tma_load_2d(sa + 64 * 128, map_a, &full_bar[s], tile_m + 64, k0);
                    }
                    if (!BMN) {
                        tma_load_2d(sb, map_b, &full_bar[s], k0, tile_n);  // box [BN rows][64 k]
                    } else if (ps.b_blocked[w.p]) {
                        tma_load_3d(sb, map_b, &full_bar[s], 0, k0, tile_n / 64);  // box [BN / 64 blocks][64 k][64 n]
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j)
                            tma_load_2d(sb + j * 64 * 128, map_b, &full_bar[s], tile_n + 64 * j, k0);
                    }
                }
                if (ps.trace != nullptr && cta == 0 && leader && tslot < 8) ps.trace[tslot * 32 + 1] = gtimer();
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer --------------------------------
        if (lane == 0 && leader) {
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((AMN ? 1u : 0u) << 15) |
                                   ((BMN ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) |
                                   ((uint32_t)((PAIR ? 2 * BM : BM) >> 4) << 24);
            uint32_t it = 0, tc = 0;
            bool ok = true;
            for (int unit = cta; unit < total_units && ok; unit += n_cta) {
                const int num_kt = decode_unit<BN, PAIR>(ps, unit, ag, cr).num_kt;
                if (num_kt == 0) continue;
                const uint32_t buf = tc & 1u, tph = (tc >> 1) & 1u;
                if (!mbar_wait(&tempty_bar[buf], tph ^ 1u, limit_ns)) {
                    atomicCAS(err_flag, 0u, 4u);
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + buf * (uint32_t)BN;
                const int tslot = (unit - cta) / n_cta;
                const bool tr = ps.trace != nullptr && cta == 0 && leader && tslot < 8;
                if (tr) ps.trace[tslot * 32 + 2] = gtimer();
                for (int kt = 0; kt < num_kt; ++kt, ++it) {
                    const int s = it % L::kStages;
                    const uint32_t ph = (it / L::kStages) & 1u;
                    // consumers wait longer than producers, so that the wait that reports is the one at the root
                    if (!mbar_wait(&full_bar[s], ph, limit_ns * 2)) {
                        atomicCAS(err_flag, 0u, 2u);
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    if (tr && kt == 0) {
                        ps.trace[tslot * 32 + 3] = gtimer();
                        ps.trace[tslot * 32 + 20] = (unsigned long long)clock64();
                    }
                    const uint32_t sa = smem_u32(smem + s * L::kStageBytes);
                    const uint32_t sb = sa + L::kABytes;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // K-major: 8-row groups are 1024 B apart, a K step of 16 elements is 32 B inside the
                        // swizzle span. MN-major: 64-element column blocks are one box (8192 B) apart,
                        // 8-k-row groups 1024 B apart, a K step of 16 rows is 2048 B.
                        const uint64_t da = AMN ? make_desc(sa + k * 2048, 8192, 1024) : make_desc(sa + k * 32, 16, 1024);
                        const uint64_t db = BMN ? make_desc(sb + k * 2048, 8192, 1024) : make_desc(sb + k * 32, 16, 1024);
                        if constexpr (PAIR) umma_bf16_pair(tmem_d, da, db, idesc, (kt | k) ? 1u : 0u);
                        else umma_bf16(tmem_d, da, db, idesc, (kt | k) ? 1u : 0u);
                    }
                    // frees the stage (in both CTAs of a pair) when these MMAs have read it
                    if constexpr (PAIR) umma_commit_pair(&empty_bar[s]);
                    else umma_commit(&empty_bar[s]);
                }
                // accumulator complete (also on error, so the epilogue moves on)
                if constexpr (PAIR) umma_commit_pair(&tfull_bar[buf]);
                else umma_commit(&tfull_bar[buf]);
                if (tr) {
                    ps.trace[tslot * 32 + 4] = gtimer();
                    ps.trace[tslot * 32 + 21] = (unsigned long long)clock64();
                }
                ++tc;
            }
        }
    } else if (warp == kPublisherWarp) {
        // ------------------------------ publisher (chain mode) --------------------
        if (ps.chain && lane < kEpilogueWarps) {
            uint32_t* box = pub_req + lane;
            const unsigned long long t0 = gtimer();
            unsigned spins = 0;
            for (;;) {
                const uint32_t r = ld_acquire_cta_smem(box);
                if (r == kPubExit) break;
                if (r != 0u) {
                    // the epilogue warp saw its stores complete before it posted: fence, then tell the next layer
                    __threadfence();
                    atomicAdd(ps.done + (r - 1u), 1u);
                    st_release_cta_smem(box, 0u);
                    continue;
                }
                __nanosleep(40);
                // every epilogue warp posts kPubExit on its way out, also after an error: this bound only guards
                // against a warp that never gets there
                if ((++spins & 255u) == 0 && gtimer() - t0 > limit_ns * 64) {
                    atomicCAS(err_flag, 0u, 9u);
                    break;
                }
            }
        }
    } else {
        // ------------------------------ epilogue ----------------------------------
        const int ew = warp - kFirstEpilogueWarp;   // 0 .. kEpilogueWarps-1
        const int q = warp & 3;              // TMEM lane quarter this warp may read
        const int half = ew >> 2;            // which half of the tile's columns this warp drains
        const int etid = ew * 32 + lane;     // 0 .. 255
        constexpr int kChunks = BN / 64;     // 32-column chunks per warp
        uint32_t tc = 0;
        bool store_in_flight = false;        // lane 0: a TMA store may still be reading this warp's staging piece
        int bias_unit = -1;                  // the unit whose bias the previous tile already staged
        for (int unit = cta; unit < total_units; unit += n_cta) {
            const WorkUnit w = decode_unit<BN, PAIR>(ps, unit, ag, cr);
            const int tile_n = w.tile_n, tile_m = w.tile_m, num_kt = w.num_kt;
            const GemmEpilogue& ep = ps.ep[w.p];
            const int M = ps.M[w.p], N = ps.N[w.p];
            if (num_kt == 0) continue;
            const uint32_t buf = tc & 1u, tph = (tc >> 1) & 1u;
            // The bias of the tile's columns, staged in shared memory (double-buffered with the accumulator). It was
            // fetched during the tile before this one; only the first tile of a CTA waits for the load here.
            float* bs = bias_smem + buf * 256;
            const bool has_bias = !(LEAN && BMN) && (ep.bias != nullptr || ep.bias_bf16 != nullptr);
            if (has_bias && etid < BN && bias_unit != unit) {
                const int col = tile_n + etid;
                float v = 0.f;
                if (col < N) v = ep.bias != nullptr ? ep.bias[col] : __bfloat162float(ep.bias_bf16[col]);
                bs[etid] = v;
            }
            // Mask (ReLU backward) of this lane's row: the first piece is requested here, before the wait for the
            // accumulator, and each following piece while the one before it is converted and stored, so that no
            // piece waits for memory.
            const int row = tile_m + q * 32 + lane;
            const int cbase = half * (BN / 2);
            const bool mask_fast = !(LEAN && !BMN) && ep.mask != nullptr && (ep.ldmask % 8 == 0) && row < M;
            const __nv_bfloat16* mrow = mask_fast ? ep.mask + (size_t)row * ep.ldmask + tile_n + cbase : nullptr;
            uint4 mreg[4];
            bool mhave = false;
            if (mask_fast && tile_n + cbase + 32 <= N) {
#pragma unroll
                for (int j = 0; j < 4; ++j) mreg[j] = ld_nc_v4(mrow + j * 8);
                mhave = true;
            }
            const bool waited = mbar_wait(&tfull_bar[buf], tph, limit_ns * 4);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (!LEAN && ps.trace != nullptr && cta == 0 && leader && (unit - cta) / n_cta < 8 && ew == 0 && lane == 0)
                ps.trace[(unit - cta) / n_cta * 32 + 8] = gtimer();
            // One barrier of the epilogue warps per tile: it publishes the staged bias and makes the decision to give
            // up uniform (a warp that timed out must not leave the others waiting at the next tile's barrier).
            uint32_t all_ok;
            asm volatile(
                "{\n\t.reg .pred p, q;\n\t"
                "setp.ne.u32 q, %1, 0;\n\t"
                "bar.red.and.pred p, 1, %2, q;\n\t"
                "selp.u32 %0, 1, 0, p;\n\t}"
                : "=r"(all_ok)
                : "r"(waited ? 1u : 0u), "r"(32 * kEpilogueWarps)
                : "memory");
            if (!all_ok) {
                if (!waited && lane == 0) atomicCAS(err_flag, 0u, 3u);
                break;
            }
            const int tslot = (unit - cta) / n_cta;
            const bool tr = !LEAN && ps.trace != nullptr && cta == 0 && leader && tslot < 8 && ew == 0 && lane == 0;
            if (tr) ps.trace[tslot * 32 + 5] = gtimer();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * (uint32_t)BN + (uint32_t)cbase;
            // One register buffer for the accumulator pieces and ONE copy of the loop body: the load of piece c + 1 is
            // issued once the values of piece c are packed. (Two buffers with the load issued right after the wait
            // hide the TMEM latency, but need two copies of the body, and the loop is bound by instruction fetch:
            // 74.7 instead of 69.6 us for the top forward chain.)
            uint32_t va[32];
            if (tile_n + cbase < N) tmem_ld32_issue(taddr, va);
            const int d_mode = LEAN ? 1 : ps.d_mode[w.p];
            const CUtensorMap* map_d = &ps.map_d[w.p];
            uint8_t* my_stage = stage_out + ew * 2048 + lane * 64;   // this lane's row of the warp's staging piece
            const int row0 = tile_m + q * 32;
            // one piece: returns false when the tile has no more columns
            auto piece = [&](uint32_t* v, const int c) -> bool {
                const int col0 = tile_n + cbase + c * 32;
                if (col0 >= N) return false;  // warp-uniform
                const bool more = c + 1 < kChunks && col0 + 32 < N;
                tmem_wait_ld(v);
                if (tr && c == 0) ps.trace[tslot * 32 + 9] = gtimer();
                float f[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
                if (!LEAN && d_mode == 0) {
                    if (row < M) {
                        epilogue_chunk(ep, f, row, col0, N, has_bias ? bs + cbase + c * 32 : nullptr, true);
                        float tmp[32];   // a copy: the values of the common path must not live in local memory
#pragma unroll
                        for (int j = 0; j < 32; ++j) tmp[j] = f[j];
                        store_chunk_rows(ep, tmp, row, col0, N);
                    }
                    if (more) tmem_ld32_issue(taddr + (uint32_t)(c + 1) * 32u, v);
                    return true;
                }
                if constexpr (!(LEAN && BMN)) {   // (the lean dgrad kernel has neither bias nor activation)
                    if (LEAN || !(ps.epi_skip & 1))
                        epilogue_chunk<LEAN && !BMN, LEAN && BMN>(ep, f, row, col0, N, has_bias ? bs + cbase + c * 32 : nullptr,
                                                                  row < M, mhave ? mreg : nullptr);
                }
                uint4 raw[4];
                if constexpr (LEAN) {
                    // Lean kernels finish on the packed pairs: ReLU as a packed max, the ReLU-backward mask as a packed
                    // compare + AND (the same values as on fp32: rounding keeps sign and zero), a third of the
                    // instructions.
                    const __nv_bfloat162 zero2 = __floats2bfloat162_rn(0.f, 0.f);
                    const bool relu = !BMN && ep.relu != 0;
                    const bool masked = BMN && mhave;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        __nv_bfloat162* h = (__nv_bfloat162*)&raw[j];
                        const __nv_bfloat162* m2 = (const __nv_bfloat162*)&mreg[j];
                        uint32_t* hb = (uint32_t*)&raw[j];
#pragma unroll
                        for (int t = 0; t < 4; ++t) {
                            h[t] = __floats2bfloat162_rn(f[8 * j + 2 * t], f[8 * j + 2 * t + 1]);
                            if constexpr (!BMN) {
                                if (relu) h[t] = __hmax2(h[t], zero2);
                            } else {
                                if (masked) hb[t] &= __hgt2_mask(m2[t], zero2);
                            }
                        }
                    }
                }
                mhave = false;
                if (mask_fast && c + 1 < kChunks && col0 + 64 <= N) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) mreg[j] = ld_nc_v4(mrow + (c + 1) * 32 + j * 8);
                    mhave = true;
                }
                if (tr && c == 0) ps.trace[tslot * 32 + 15] = gtimer();
                if (LEAN || d_mode == 1) {
                    // bf16: the warp's [32 rows][32 cols] piece goes through shared memory so that every store
                    // instruction writes whole 64-byte row segments (8 rows per instruction) instead of 16 bytes
                    // in each of 32 rows. Lane l writes row l; the 16-byte column blocks of a row are XOR-swizzled
                    // by (row / 2) % 4, which makes both the row-wise writes and the 8-row reads conflict-free.
                    if constexpr (!LEAN) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            __nv_bfloat162* h = (__nv_bfloat162*)&raw[j];
                            h[0] = __floats2bfloat162_rn(f[8 * j], f[8 * j + 1]);
                            h[1] = __floats2bfloat162_rn(f[8 * j + 2], f[8 * j + 3]);
                            h[2] = __floats2bfloat162_rn(f[8 * j + 4], f[8 * j + 5]);
                            h[3] = __floats2bfloat162_rn(f[8 * j + 6], f[8 * j + 7]);
                        }
                    }
                    if (more) tmem_ld32_issue(taddr + (uint32_t)(c + 1) * 32u, v);   // the values are packed: v is free
                    if (!LEAN && (ps.epi_skip & 2)) {
                        if (raw[0].x == 0x7fc07fc1u && raw[3].w == 0x12345678u) atomicAdd(err_flag, 0u);   // keeps the values alive
                        return true;
                    }
                    __syncwarp();   // the reads of the previous piece are done
                    {
                        const int sw = (lane >> 1) & 3;
#pragma unroll
                        for (int j = 0; j < 4; ++j) *(uint4*)(my_stage + ((j ^ sw) << 4)) = raw[j];
                    }
                    if (tr && c == 0) ps.trace[tslot * 32 + 16] = gtimer();
                    __syncwarp();
                    {
                        const int cb = lane & 3;            // 16-byte column block of this lane
                        const int gcol = col0 + cb * 8;
                        __nv_bfloat16* orow = ep.out_bf16 + (size_t)row0 * ep.ldd + gcol;
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int r = i * 8 + (lane >> 2);
                            const uint4 d = *(const uint4*)(stage_out + ew * 2048 + r * 64 + ((cb ^ ((r >> 1) & 3)) << 4));
                            if (row0 + r < M && (LEAN || !(ps.epi_skip & 4))) {
                                __nv_bfloat16* op = orow + (size_t)r * ep.ldd;
                                if (LEAN || gcol + 8 <= N) {
                                    *(uint4*)op = d;
                                } else {
                                    const __nv_bfloat16* h = (const __nv_bfloat16*)&d;
                                    for (int t = 0; t < 8; ++t)
                                        if (gcol + t < N) op[t] = h[t];
                                }
                            }
                        }
                    }
                    if (tr && c == 0) ps.trace[tslot * 32 + 10] = gtimer();
                } else if constexpr (!LEAN) {
                    // fp32 (weight gradients, split-K partial sums): out of line, once per long K loop
                    if (store_in_flight) {
                        if (lane == 0) bulk_wait_read0();
                        __syncwarp();
                    }
                    if constexpr (AMN && BMN) {
                        // the weight-gradient variant of the kernel: this IS its output path, kept in line
#pragma unroll
                        for (int hcol = 0; hcol < 32; hcol += 16) {
                            if (col0 + hcol >= N) break;   // warp-uniform
#pragma unroll
                            for (int j = 0; j < 16; j += 4)
                                *(float4*)(my_stage + j * 4) = make_float4(f[hcol + j], f[hcol + j + 1], f[hcol + j + 2], f[hcol + j + 3]);
                            fence_async_smem();
                            __syncwarp();
                            if (lane == 0) {
                                if (d_mode == 2) tma_reduce_add_2d(map_d, stage_out + ew * 2048, col0 + hcol, row0);
                                else tma_store_2d(map_d, stage_out + ew * 2048, col0 + hcol, row0);
                                bulk_commit();
                                if (hcol == 0) bulk_wait_read0();   // the second half follows at once
                            }
                            if (hcol == 0) __syncwarp();
                        }
                    } else {
                        float tmp[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) tmp[j] = f[j];
                        store_piece_f32(map_d, d_mode, stage_out + ew * 2048, lane, tmp, col0, row0, N);
                    }
                    store_in_flight = true;
                    if (more) tmem_ld32_issue(taddr + (uint32_t)(c + 1) * 32u, v);
                }
                return true;
            };
#pragma unroll 1
            for (int c = 0; c < kChunks; ++c)
                if (!piece(va, c)) break;
            if (tr) ps.trace[tslot * 32 + 6] = gtimer();
            // this warp is done reading the buffer: hand it back to the MMA warp
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                if constexpr (PAIR) mbar_arrive_cluster(mapa_cluster(smem_u32(&tempty_bar[buf]), 0));
                else mbar_arrive(&tempty_bar[buf]);
                // Chain mode: this warp's part of the tile is handed to the publisher at once. The output of a chained
                // layer is bf16 and written with ordinary stores (by all lanes, ordered before this hand-off by the
                // warp barrier above), so there is nothing to wait for here: the publisher's fence covers them.
                if (ps.chain && tile_m < M)
                    post_publish(pub_req + ew, (uint32_t)(w.p * kMaxChainMTiles + tile_m / BM) + 1u, limit_ns, err_flag);
            }
            // fetch the bias of the next tile now: its latency hides behind the rest of this iteration
            {
                const int nu = unit + n_cta;
                if (nu < total_units) {
                    const WorkUnit nw = decode_unit<BN, PAIR>(ps, nu, ag, cr);
                    const GemmEpilogue& nep = ps.ep[nw.p];
                    if (!(LEAN && BMN) && nw.num_kt != 0 && (nep.bias != nullptr || nep.bias_bf16 != nullptr) && etid < BN) {
                        const int col = nw.tile_n + etid;
                        float v = 0.f;
                        if (col < ps.N[nw.p]) v = nep.bias != nullptr ? nep.bias[col] : __bfloat162float(nep.bias_bf16[col]);
                        bias_smem[(buf ^ 1u) * 256 + etid] = v;
                    }
                    bias_unit = nu;
                }
            }
            ++tc;
        }
        __syncwarp();
        if (lane == 0) {
            if (store_in_flight) bulk_wait_read0();   // the staging piece must outlive the store that reads it
            if (ps.chain) post_publish(pub_req + ew, kPubExit, limit_ns, err_flag);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    // a pair leaves together: until here the peer may still signal this CTA's barriers or read its shared memory
    if constexpr (PAIR) cluster_sync_all();
    else __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if constexpr (PAIR)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(2 * BN))
                         : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(2 * BN))
                         : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode() {
    static EncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeFn)p;
    });
    return fn;
}

// 2-D bf16 row-major tensor [rows][cols] with leading dimension ld (elements); box [box_rows][64 cols].
bool make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
    EncodeFn enc = get_encode();
    if (!enc) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld * 2};
    cuuint32_t box[2] = {64, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// MN-major operand [K rows][MN cols] (MN a multiple of 64) as (64, K, MN / 64) with box (64, 64, blocks): the box
// lands in shared memory block by block ([block][64 k][64 mn], 8 KB per block), which is the layout the MMA
// descriptors of an MN-major operand walk.
bool make_map_blocked(CUtensorMap* map, const void* base, uint64_t k_rows, uint64_t mn, uint64_t ld, uint32_t blocks) {
    EncodeFn enc = get_encode();
    if (!enc) return false;
    cuuint64_t dims[3] = {64, k_rows, mn / 64};
    cuuint64_t strides[2] = {ld * 2, 128};
    cuuint32_t box[3] = {64, 64, blocks};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// Output tensor [rows][cols] (bf16 or fp32, leading dimension ld) with a [32 rows][64 bytes] box, no swizzle.
bool make_map_out(CUtensorMap* map, void* base, bool f32, uint64_t rows, uint64_t cols, uint64_t ld) {
    EncodeFn enc = get_encode();
    if (!enc) return false;
    const uint64_t elem = f32 ? 4 : 2;
    if (((uintptr_t)base % 16) || ((ld * elem) % 16)) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld * elem};
    cuuint32_t box[2] = {f32 ? 16u : 32u, 32u};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

extern int g_gemm_cta_limit;

bool pdl_enabled() {
    static const bool on = [] {
        const char* e = std::getenv("PSB_GEMM_PDL");
        return e != nullptr && e[0] != '\0' && e[0] != '0';
    }();
    return on;
}

template <int BN, bool AMN, bool BMN, bool PAIR, bool LEAN>
cudaError_t launch_variant(const GemmProblemSet& ps, unsigned* err, unsigned long long limit_ns, cudaStream_t s,
                           const GemmGather& ag) {
    auto kern = gemm_bf16_tcgen05_kernel<BN, AMN, BMN, PAIR, LEAN>;
    static bool configured = false;
    static int max_pairs = 0;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemLayout<BN, PAIR>::kTotal);
        if (e != cudaSuccess) return e;
        if (PAIR) {
            // how many 2-CTA clusters the device can hold at once (one CTA per SM): the size of the persistent grid
            cudaLaunchConfig_t q = {};
            q.gridDim = dim3(2);
            q.blockDim = dim3(kThreads);
            q.dynamicSmemBytes = SmemLayout<BN, PAIR>::kTotal;
            cudaLaunchAttribute qa[1];
            qa[0].id = cudaLaunchAttributeClusterDimension;
            qa[0].val.clusterDim.x = 2;
            qa[0].val.clusterDim.y = 1;
            qa[0].val.clusterDim.z = 1;
            q.attrs = qa;
            q.numAttrs = 1;
            int n = 0;
            e = cudaOccupancyMaxActiveClusters(&n, kern, &q);
            if (e != cudaSuccess) return e;
            if (n <= 0) return cudaErrorLaunchOutOfResources;
            max_pairs = n;
        }
        configured = true;
    }
    static int num_sms = 0;
    if (num_sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
    }
    const int units = ps.unit_end[ps.count - 1];
    int ctas = units < num_sms ? units : num_sms;
    if (ag.enabled) ctas = std::max(ag.gather_ctas + 1, std::min(num_sms, units + ag.gather_ctas));
    int sms = num_sms;
    if (g_gemm_cta_limit > 0 && !ag.enabled) sms = std::max(2, std::min(num_sms, g_gemm_cta_limit));
    if (!ag.enabled) ctas = std::min(ctas, sms);
    if (PAIR) ctas = 2 * std::min(units, std::min(max_pairs, sms / 2));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = SmemLayout<BN, PAIR>::kTotal;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (PAIR) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 2;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    if (pdl_enabled() && !ag.enabled) {  // the prologue of this launch may overlap the previous kernel's tail
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return cudaLaunchKernelEx(&cfg, kern, ps, err, limit_ns, ag);
}

template <bool PAIR, bool LEAN>
cudaError_t dispatch_mode(int BN, bool a_mn, bool b_mn, const GemmProblemSet& ps, unsigned* err, unsigned long long lim,
                          cudaStream_t s, const GemmGather& ag) {
    const int v = (a_mn ? 2 : 0) | (b_mn ? 1 : 0);
    if constexpr (LEAN) {
        // lean launches are forward / dgrad layers: A is K-major
        if (BN == 256) return v == 0 ? launch_variant<256, false, false, PAIR, true>(ps, err, lim, s, ag)
                                     : launch_variant<256, false, true, PAIR, true>(ps, err, lim, s, ag);
        return v == 0 ? launch_variant<128, false, false, PAIR, true>(ps, err, lim, s, ag)
                      : launch_variant<128, false, true, PAIR, true>(ps, err, lim, s, ag);
    } else {
        if (BN == 256) {
            switch (v) {
                case 0: return launch_variant<256, false, false, PAIR, false>(ps, err, lim, s, ag);
                case 1: return launch_variant<256, false, true, PAIR, false>(ps, err, lim, s, ag);
                case 2: return launch_variant<256, true, false, PAIR, false>(ps, err, lim, s, ag);
                default: return launch_variant<256, true, true, PAIR, false>(ps, err, lim, s, ag);
            }
        }
        switch (v) {
            case 0: return launch_variant<128, false, false, PAIR, false>(ps, err, lim, s, ag);
            case 1: return launch_variant<128, false, true, PAIR, false>(ps, err, lim, s, ag);
            case 2: return launch_variant<128, true, false, PAIR, false>(ps, err, lim, s, ag);
            default: return launch_variant<128, true, true, PAIR, false>(ps, err, lim, s, ag);
        }
    }
}

// Whether every problem of the set qualifies for the lean epilogue.
bool lean_ok(const GemmProblemSet& ps, bool a_mn, bool b_mn, const GemmGather& ag) {
    if (a_mn || ag.enabled || ps.trace != nullptr || ps.epi_skip != 0) return false;
    for (int i = 0; i < ps.count; ++i) {
        const GemmEpilogue& e = ps.ep[i];
        if (ps.d_mode[i] != 1 || (ps.N[i] % 32) != 0) return false;
        if (b_mn) {   // the lean dgrad kernel: a mask (aligned rows) or nothing
            if (e.bias != nullptr || e.bias_bf16 != nullptr || e.relu) return false;
            if (e.mask != nullptr && ((e.ldmask % 8) != 0 || ((uintptr_t)e.mask % 16) != 0)) return false;
        } else if (e.mask != nullptr) {   // the lean forward kernel: bias and activation, no mask
            return false;
        }
    }
    return true;
}

cudaError_t dispatch(int BN, bool pair, bool a_mn, bool b_mn, const GemmProblemSet& ps, unsigned* err, unsigned long long lim,
                     cudaStream_t s, const GemmGather& ag) {
    if (lean_ok(ps, a_mn, b_mn, ag))
        return pair ? dispatch_mode<true, true>(BN, a_mn, b_mn, ps, err, lim, s, ag)
                    : dispatch_mode<false, true>(BN, a_mn, b_mn, ps, err, lim, s, ag);
    return pair ? dispatch_mode<true, false>(BN, a_mn, b_mn, ps, err, lim, s, ag)
                : dispatch_mode<false, false>(BN, a_mn, b_mn, ps, err, lim, s, ag);
}

// CTA pairs are used whenever a problem has more than one 128-row block (and never with the gather role, whose
// copy CTAs are not part of a pair). PSB_GEMM_PAIR=0 forces the 1-CTA kernel.
int epi_skip_env() {
    static const int v = [] {
        const char* e = std::getenv("PSB_GEMM_EPI_SKIP");
        return e != nullptr ? std::atoi(e) : 0;
    }();
    return v;
}
int g_gemm_pair = 1;
bool pair_enabled() {
    static const bool on = [] {
        const char* e = std::getenv("PSB_GEMM_PAIR");
        return !(e != nullptr && e[0] == '0');
    }();
    return on && g_gemm_pair != 0;
}

// Fills slot i of a problem set; returns 0, -2 (alignment) or -3 (tensor map).
unsigned long long* g_gemm_trace = nullptr;
int g_gemm_cta_limit = 0;   // 0 = one CTA per SM

int add_problem(GemmProblemSet* ps, int i, int BN, bool pair, const GemmOperand& A, const GemmOperand& B, const GemmEpilogue& ep,
                int M, int N, int K) {
    const int BNL = pair ? BN / 2 : BN;   // rows of B that one CTA loads per stage
    if ((A.ld % 8) || (B.ld % 8) || ((uintptr_t)A.ptr % 16) || ((uintptr_t)B.ptr % 16)) return -2;  // TMA: 16-byte rule
    // K-major: tensor [MN rows][K cols], box [tile rows][64]; MN-major: tensor [K rows][MN cols], box [64][64], or the
    // blocked 3-D form (one load per stage) when the MN extent is a whole number of 64-wide blocks covering the tile
    ps->a_blocked[i] = (A.mn_major && M % 64 == 0 && M >= BM) ? 1 : 0;
    ps->b_blocked[i] = (B.mn_major && N % 64 == 0 && N >= BN) ? 1 : 0;
    if (pair && BNL < 64) ps->b_blocked[i] = 0;
    // (if the driver refuses the blocked form, the per-block form does the same job with more loads)
    if (ps->a_blocked[i] && !make_map_blocked(&ps->map_a[i], A.ptr, (uint64_t)K, (uint64_t)M, (uint64_t)A.ld, BM / 64)) ps->a_blocked[i] = 0;
    if (ps->b_blocked[i] && !make_map_blocked(&ps->map_b[i], B.ptr, (uint64_t)K, (uint64_t)N, (uint64_t)B.ld, BNL / 64)) ps->b_blocked[i] = 0;
    bool ok = A.mn_major ? (ps->a_blocked[i] ? make_map_blocked(&ps->map_a[i], A.ptr, (uint64_t)K, (uint64_t)M, (uint64_t)A.ld, BM / 64)
                                             : make_map(&ps->map_a[i], A.ptr, (uint64_t)K, (uint64_t)M, (uint64_t)A.ld, 64))
                         : make_map(&ps->map_a[i], A.ptr, (uint64_t)M, (uint64_t)K, (uint64_t)A.ld, BM);
    ok = ok && (B.mn_major ? (ps->b_blocked[i] ? make_map_blocked(&ps->map_b[i], B.ptr, (uint64_t)K, (uint64_t)N, (uint64_t)B.ld, BNL / 64)
                                               : make_map(&ps->map_b[i], B.ptr, (uint64_t)K, (uint64_t)N, (uint64_t)B.ld, 64))
                           : make_map(&ps->map_b[i], B.ptr, (uint64_t)N, (uint64_t)K, (uint64_t)B.ld, BNL));
    if (!ok) return -3;
    ps->d_mode[i] = 0;
    if (ep.out_bf16 != nullptr && ep.out_f32 == nullptr) {
        // coalesced 16-byte stores through a staging piece: rows must start on 16-byte boundaries
        if (((uintptr_t)ep.out_bf16 % 16) == 0 && (ep.ldd % 8) == 0) ps->d_mode[i] = 1;
    } else if (ep.out_f32 != nullptr && ep.out_bf16 == nullptr) {
        if (make_map_out(&ps->map_d[i], ep.out_f32, true, (uint64_t)M, (uint64_t)N, (uint64_t)ep.ldd))
            ps->d_mode[i] = (ep.split_k > 1 || ep.accumulate) ? 2 : 3;
    }
    ps->ep[i] = ep;
    ps->M[i] = M;
    ps->N[i] = N;
    ps->K[i] = K;
    const int bmu = pair ? 2 * BM : BM;
    const int units = ((N + BN - 1) / BN) * ((M + bmu - 1) / bmu) * (ep.split_k > 1 ? ep.split_k : 1);
    ps->unit_end[i] = (i > 0 ? ps->unit_end[i - 1] : 0) + units;
    return 0;
}

}  // namespace

int gemm_bf16(const GemmOperand& A, const GemmOperand& B, const GemmEpilogue& ep, int M, int N, int K, unsigned* err_flag,
              double wait_limit_s, void* stream, const GemmGather* gather) {
    GemmGather ag;
    if (gather != nullptr) ag = *gather;
    if (ag.enabled) {
        // the gather path moves whole 256-row blocks of a contiguous K-major B and never splits K
        if (A.mn_major || B.mn_major || B.ld != K || N < 256 || (ag.rows_per_rank % 256) || ag.rows_per_rank * ag.world != N ||
            ep.split_k > 1 || ((size_t)K * 2) % 16)
            return -2;
    }
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    // 128 x 256 tiles halve the operand bytes per flop (the 128 x 128 tile is bound by the L2 -> SMEM feed);
    // they are used whenever N fills them.
    const int BN = (N >= 256) ? 256 : 128;
    GemmProblemSet ps;
    ps.count = 1;
    ps.chain = 0;
    ps.done = nullptr;
    ps.trace = g_gemm_trace;
    ps.epi_skip = epi_skip_env();
    const bool pair = pair_enabled() && !ag.enabled && M > BM;
    int rc = add_problem(&ps, 0, BN, pair, A, B, ep, M, N, K);
    if (rc != 0) return rc;
    const unsigned long long lim = (unsigned long long)(wait_limit_s * 1e9);
    return (int)dispatch(BN, pair, A.mn_major, B.mn_major, ps, err_flag, lim, (cudaStream_t)stream, ag);
}

void gemm_set_cta_limit(int ctas) { g_gemm_cta_limit = ctas > 0 ? ctas : 0; }
void gemm_set_pair(int on) { g_gemm_pair = on ? 1 : 0; }

void gemm_set_trace(void* device_buffer_of_256_u64) { g_gemm_trace = (unsigned long long*)device_buffer_of_256_u64; }

int gemm_chain_scratch_words() { return kMaxGroup * kMaxChainMTiles; }

int gemm_bf16_grouped(const GemmOperand* A, const GemmOperand* B, const GemmEpilogue* ep, const int* M, const int* N,
                      const int* K, int count, unsigned* err_flag, double wait_limit_s, void* stream, unsigned* chain_done) {
    if (count <= 0) return 0;
    if (count > kMaxGroup) return -2;
    int BN = 256;
    for (int i = 0; i < count; ++i) {
        if (M[i] <= 0 || N[i] <= 0 || K[i] <= 0) return -2;
        if (A[i].mn_major != A[0].mn_major || B[i].mn_major != B[0].mn_major) return -2;  // one kernel variant per launch
        if (N[i] < 256) BN = 128;
    }
    GemmProblemSet ps;
    ps.count = count;
    ps.chain = chain_done != nullptr ? 1 : 0;
    ps.done = chain_done;
    ps.trace = g_gemm_trace;
    ps.epi_skip = epi_skip_env();
    if (ps.chain) {
        // layer i + 1 consumes the bf16 output of layer i: same rows, K of the consumer = N of the producer
        for (int i = 0; i < count; ++i) {
            if (M[i] != M[0] || A[i].mn_major || ep[i].split_k > 1) return -2;
            if (i > 0 && (K[i] != N[i - 1] || A[i].ptr != (const void*)ep[i - 1].out_bf16)) return -2;
        }
        if ((M[0] + BM - 1) / BM > kMaxChainMTiles) return -2;
        cudaError_t e = cudaMemsetAsync(chain_done, 0, (size_t)count * kMaxChainMTiles * sizeof(unsigned), (cudaStream_t)stream);
        if (e != cudaSuccess) return (int)e;
    }
    bool pair = false;
    for (int i = 0; i < count; ++i) pair = pair || M[i] > BM;
    pair = pair && pair_enabled();
    for (int i = 0; i < count; ++i) {
        int rc = add_problem(&ps, i, BN, pair, A[i], B[i], ep[i], M[i], N[i], K[i]);
        if (rc != 0) return rc;
    }
    const unsigned long long lim = (unsigned long long)(wait_limit_s * 1e9);
    GemmGather none;
    return (int)dispatch(BN, pair, A[0].mn_major, B[0].mn_major, ps, err_flag, lim, (cudaStream_t)stream, none);
}

}  // namespace psb
