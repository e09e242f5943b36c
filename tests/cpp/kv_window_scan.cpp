// The window-walking defaults of KVStorage::scan_shard / update_shard - the code that a storage without a
// snapshot scan of its own runs (the GPU back-end) - exercised on the CPU: a storage that keeps the host table's
// data but answers scans through the base-class defaults, with the index rebuilt under a scan on purpose.
//
//   g++ -std=c++17 -I parameter_server_b200/csrc tests/cpp/kv_window_scan.cpp -o kv_window_scan -lpthread
#include <cstdio>
#include <set>

#include "storage/kv_storage.h"

using namespace psb;

#define CHECK(c)                                                        \
    do {                                                                \
        if (!(c)) {                                                     \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #c);  \
            return 1;                                                   \
        }                                                               \
    } while (0)

class WindowOnly : public HostKVStorage {
public:
    using HostKVStorage::HostKVStorage;
    Status scan_shard(int s, uint64_t window, bool dirty_only, const ScanFn& fn, const std::function<void()>& restart = nullptr) override {
        return KVStorage::scan_shard(s, window, dirty_only, fn, restart);
    }
    Status update_shard(int s, uint64_t window, const UpdateFn& fn, uint64_t* changed) override {
        return KVStorage::update_shard(s, window, fn, changed);
    }
};

int main() {
    HostTableConfig cfg;
    cfg.dim = 4;
    cfg.n_shards = 1;
    cfg.init_range = 0.f;
    WindowOnly st(cfg);
    CHECK(st.create_shard(0).ok());
    const size_t n = 5000;
    std::vector<int64_t> keys(n);
    std::vector<float> rows(n * 4);
    for (size_t i = 0; i < n; ++i) {
        keys[i] = (int64_t)i * 7 + 1;
        for (int d = 0; d < 4; ++d) rows[i * 4 + d] = (float)(i % 11);
    }
    CHECK(st.set_rows(keys.data(), rows.data(), n, true).ok());

    // 1. a quiet table: many windows, every key exactly once
    std::multiset<int64_t> seen;
    size_t calls = 0;
    CHECK(st.scan_shard(0, 512, false, [&](const std::vector<int64_t>& k, const std::vector<float>& r) {
                ++calls;
                if (r.size() != k.size() * st.stride()) return Status::Error("row width");
                seen.insert(k.begin(), k.end());
                return Status::Ok();
            }).ok());
    CHECK(calls > 4 && seen.size() == n && std::set<int64_t>(seen.begin(), seen.end()).size() == n);

    // 2. the index is rebuilt under the scan (somebody inserts enough new keys between two windows): a consumer that
    //    can forget starts over and ends with every old key exactly once
    seen.clear();
    int restarts = 0;
    bool grown = false;
    int64_t next_key = 1 << 30;
    auto grow = [&] {   // more new keys than the table holds: the index doubles at least once
        std::vector<int64_t> nk((size_t)st.size() + 1000);
        std::vector<float> nr(nk.size() * 4, 1.f);
        for (auto& k : nk) k = next_key++;
        return st.set_rows(nk.data(), nr.data(), nk.size(), true);
    };
    CHECK(st.scan_shard(0, 512, false,
                        [&](const std::vector<int64_t>& k, const std::vector<float>&) {
                            for (int64_t x : k)
                                if (x < (1 << 30)) seen.insert(x);
                            if (!grown && seen.size() > 1000) {
                                grown = true;
                                return grow();
                            }
                            return Status::Ok();
                        },
                        [&] {
                            ++restarts;
                            seen.clear();
                        }).ok());
    CHECK(grown && restarts == 1 && seen.size() == n && std::set<int64_t>(seen.begin(), seen.end()).size() == n);

    // 3. a consumer that cannot forget is told, instead of getting keys twice or not at all
    grown = false;
    size_t got = 0;
    Status s3 = st.scan_shard(0, 512, false, [&](const std::vector<int64_t>& k, const std::vector<float>&) {
        got += k.size();
        if (!grown && got > 1000) {
            grown = true;
            return grow();
        }
        return Status::Ok();
    });
    CHECK(grown && !s3.ok() && s3.msg().find("rebuilt") != std::string::npos);

    // 4. the writing scan: changed rows are written back, exactly once, the others are left alone
    uint64_t changed = 0;
    CHECK(st.update_shard(0, 700, [&](int64_t key, float* row) {
                  if (key >= (1 << 30) || key % 2 == 0) return false;
                  row[0] += 100.f;
                  return true;
              }, &changed).ok());
    std::vector<float> out(n * 4);
    CHECK(st.pull(0, keys.data(), n, out.data(), false).ok());
    size_t odd = 0;
    for (size_t i = 0; i < n; ++i) {
        const bool hit = keys[i] % 2 != 0;
        odd += hit;
        CHECK(out[i * 4] == (float)(i % 11) + (hit ? 100.f : 0.f) && out[i * 4 + 1] == (float)(i % 11));
    }
    CHECK(changed == odd);

    // 5. a rebuild under the writing scan ends it with an error; no row was changed twice
    grown = false;
    size_t visited = 0;
    Status s5 = st.update_shard(0, 700, [&](int64_t key, float* row) {
        if (key >= (1 << 30)) return false;
        if (++visited == 1500 && !grown) {
            grown = true;
            Status g = grow();
            if (!g.ok()) std::printf("grow failed\n");
        }
        row[1] += 1000.f;
        return true;
    }, &changed);
    CHECK(grown && !s5.ok());
    CHECK(st.pull(0, keys.data(), n, out.data(), false).ok());
    size_t once = 0;
    for (size_t i = 0; i < n; ++i) {
        const float d = out[i * 4 + 1] - (float)(i % 11);
        CHECK(d == 0.f || d == 1000.f);
        once += d == 1000.f;
    }
    CHECK(once == changed && once < n);
    std::printf("WINDOW SCAN OK\n");
    return 0;
}
