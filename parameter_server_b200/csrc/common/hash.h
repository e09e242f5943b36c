// Key hashing and partitioning shared by host C++ and device CUDA code.
//
// Parity: the reference partitions a sparse key with
//   jump_consistent_hash(murmur_hash(key), global_shard_num)      (pico-ps/common/Partitioner.h:43-45)
// and dense slices with hash % num_buckets                         (pico-ps/common/dense_common.h:58-65).
// The body of murmur_hash lives in the absent prpc submodule; this build uses the MurmurHash3 64-bit
// finalizer (fmix64) for integral keys and MurmurHash3_x64_128 for strings, plus the Lamping-Veach
// jump consistent hash. Every function here is usable from __host__ and __device__ code so that the
// CPU oracle, the host storage back-end and the sm_100a kernels agree bit for bit.
#pragma once
#include <cstdint>
#include <cstddef>
#include <cstring>

#if defined(__CUDACC__)
#define PSB_HD __host__ __device__ __forceinline__
#else
#define PSB_HD inline
#endif

namespace psb {

constexpr uint64_t kMurmurSeed = 0x9E3779B97F4A7C15ull;

PSB_HD uint64_t fmix64(uint64_t k) {
    k ^= k >> 33;
    k *= 0xff51afd7ed558ccdull;
    k ^= k >> 33;
    k *= 0xc4ceb9fe1a85ec53ull;
    k ^= k >> 33;
    return k;
}

PSB_HD uint64_t murmur_hash_u64(uint64_t key) { return fmix64(key); }

// Lamping & Veach, "A Fast, Minimal Memory, Consistent Hash Algorithm" (2014).
PSB_HD int32_t jump_consistent_hash(uint64_t key, int32_t num_buckets) {
    int64_t b = -1, j = 0;
    while (j < num_buckets) {
        b = j;
        key = key * 2862933555777941757ull + 1;
        j = (int64_t)((double)(b + 1) * ((double)(1ll << 31) / (double)((key >> 33) + 1)));
    }
    return (int32_t)b;
}

// Sparse key -> global shard id.
PSB_HD int32_t sparse_shard_of(int64_t key, int32_t global_shard_num) {
    return jump_consistent_hash(murmur_hash_u64((uint64_t)key), global_shard_num);
}

// Dense (id, slice) -> shard id: plain modulo of a mixed hash, as in the reference's dense partitioner.
PSB_HD int32_t dense_shard_of(int64_t id, int32_t slice_id, int32_t num_shards) {
    uint64_t h = fmix64((uint64_t)id * 0x9E3779B97F4A7C15ull + (uint64_t)(uint32_t)slice_id);
    return (int32_t)(h % (uint64_t)num_shards);
}

// Key -> shard id by plain modulo (non-negative for negative keys too): for tables whose producer lays the keys out.
PSB_HD int32_t modulo_shard_of(int64_t key, int32_t num_shards) {
    const int64_t r = key % (int64_t)num_shards;
    return (int32_t)(r < 0 ? r + num_shards : r);
}

// Slot hash for the open-addressing tables (decorrelated from the shard hash by a second mix).
PSB_HD uint64_t slot_hash(int64_t key) { return fmix64((uint64_t)key ^ kMurmurSeed); }

// Counter-based deterministic initialiser: value d of the row of `key`, uniform in [-range, range).
// The same arithmetic runs in the CPU oracle and in the insert kernels, so freshly inserted rows are
// bitwise identical on both sides.
PSB_HD float init_uniform(int64_t key, uint32_t d, uint64_t seed, float range) {
    uint64_t h = fmix64(((uint64_t)key + 0x632BE59BD9B4E019ull * (uint64_t)(d + 1)) ^ seed);
    // 24 random mantissa bits -> [0,1)
    float u = (float)(h >> 40) * (1.0f / 16777216.0f);
    return (2.0f * u - 1.0f) * range;
}

// host-only helpers (strings never reach device code)
inline uint64_t rotl64(uint64_t x, int8_t r) { return (x << r) | (x >> (64 - r)); }

// MurmurHash3_x64_128 (public domain, Austin Appleby); returns the first 64-bit half.
inline uint64_t murmur3_x64_128_first(const void* key, size_t len, uint32_t seed) {
    const uint8_t* data = (const uint8_t*)key;
    const size_t nblocks = len / 16;
    uint64_t h1 = seed, h2 = seed;
    const uint64_t c1 = 0x87c37b91114253d5ull, c2 = 0x4cf5ad432745937full;
    for (size_t i = 0; i < nblocks; i++) {
        uint64_t k1, k2;
        std::memcpy(&k1, data + i * 16, 8);
        std::memcpy(&k2, data + i * 16 + 8, 8);
        k1 *= c1; k1 = rotl64(k1, 31); k1 *= c2; h1 ^= k1;
        h1 = rotl64(h1, 27); h1 += h2; h1 = h1 * 5 + 0x52dce729;
        k2 *= c2; k2 = rotl64(k2, 33); k2 *= c1; h2 ^= k2;
        h2 = rotl64(h2, 31); h2 += h1; h2 = h2 * 5 + 0x38495ab5;
    }
    const uint8_t* tail = data + nblocks * 16;
    uint64_t k1 = 0, k2 = 0;
    switch (len & 15) {
        case 15: k2 ^= ((uint64_t)tail[14]) << 48; [[fallthrough]];
        case 14: k2 ^= ((uint64_t)tail[13]) << 40; [[fallthrough]];
        case 13: k2 ^= ((uint64_t)tail[12]) << 32; [[fallthrough]];
        case 12: k2 ^= ((uint64_t)tail[11]) << 24; [[fallthrough]];
        case 11: k2 ^= ((uint64_t)tail[10]) << 16; [[fallthrough]];
        case 10: k2 ^= ((uint64_t)tail[9]) << 8; [[fallthrough]];
        case 9:  k2 ^= ((uint64_t)tail[8]) << 0;
                 k2 *= c2; k2 = rotl64(k2, 33); k2 *= c1; h2 ^= k2; [[fallthrough]];
        case 8:  k1 ^= ((uint64_t)tail[7]) << 56; [[fallthrough]];
        case 7:  k1 ^= ((uint64_t)tail[6]) << 48; [[fallthrough]];
        case 6:  k1 ^= ((uint64_t)tail[5]) << 40; [[fallthrough]];
        case 5:  k1 ^= ((uint64_t)tail[4]) << 32; [[fallthrough]];
        case 4:  k1 ^= ((uint64_t)tail[3]) << 24; [[fallthrough]];
        case 3:  k1 ^= ((uint64_t)tail[2]) << 16; [[fallthrough]];
        case 2:  k1 ^= ((uint64_t)tail[1]) << 8; [[fallthrough]];
        case 1:  k1 ^= ((uint64_t)tail[0]) << 0;
                 k1 *= c1; k1 = rotl64(k1, 31); k1 *= c2; h1 ^= k1;
    }
    h1 ^= len; h2 ^= len;
    h1 += h2; h2 += h1;
    h1 = fmix64(h1); h2 = fmix64(h2);
    h1 += h2;
    return h1;
}

inline int32_t string_shard_of(const char* s, size_t n, int32_t global_shard_num) {
    return jump_consistent_hash(murmur3_x64_128_first(s, n, (uint32_t)kMurmurSeed), global_shard_num);
}

}  // namespace psb
