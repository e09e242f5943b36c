// A plug-in operator library as a user of the framework would write one: it derives from the operator base classes,
// registers its classes under its own library name and is opened with Client::load_operator_library. What the
// reference allows through REGISTER_OPERATOR(lib, Class) + virtual hooks (pico-ps/operator/Operator.h:118-130,
// ForEachOperator.h:214-232, EraseIfOperator.h:57, UpdateContextOperator.h:59-213, common/dense_common.h:135-171).
//
//   g++ -std=c++17 -shared -fPIC -DPSB_OPERATOR_PLUGIN -I parameter_server_b200/csrc tests/cpp/plugin_ops.cpp -o libplugin_ops.so
#include <fstream>

#include "operator/operators.h"

using namespace psb;

// erase_if with a predicate the built-in menu does not have: even keys whose first embedding value exceeds a bound.
class EraseEvenAbove : public EraseIfOperatorBase {
public:
    explicit EraseEvenAbove(const Json& c) : EraseIfOperatorBase(c) {}
    bool erase_if(int64_t key, const float* row, uint32_t, uint32_t, const Json& carried) const override {
        return key % 2 == 0 && row[0] > (float)carried.at("bound").as_double(0);
    }
};

// for_each with its own result type: how many keys fall in each residue class modulo 4, and the smallest key.
class KeyHistogram : public ForEachOperatorBase {
public:
    struct Result {
        int64_t bucket[4];
        int64_t min_key;
    };
    explicit KeyHistogram(const Json& c) : ForEachOperatorBase(c) {}
    std::string init_result(const Json&) const override {
        Result r{{0, 0, 0, 0}, INT64_MAX};
        return std::string((const char*)&r, sizeof(r));
    }
    void for_each(int64_t key, const float*, uint32_t, uint32_t, const Json&, std::string* result) const override {
        Result* r = (Result*)&(*result)[0];
        ++r->bucket[((key % 4) + 4) % 4];
        r->min_key = std::min(r->min_key, key);
    }
    void merge_result(const std::string& in, std::string* out) const override {
        const Result* a = (const Result*)in.data();
        Result* b = (Result*)&(*out)[0];
        for (int i = 0; i < 4; ++i) b->bucket[i] += a->bucket[i];
        b->min_key = std::min(b->min_key, a->min_key);
    }
};

// A writing scan: rows of odd keys get their first value replaced by the key; the result counts them (one int64).
class StampOddKeys : public ForEachWriteOperatorBase {
public:
    explicit StampOddKeys(const Json& c) : ForEachWriteOperatorBase(c) {}
    std::string init_result(const Json&) const override { return std::string(8, '\0'); }
    bool for_each_write(int64_t key, float* row, uint32_t, uint32_t, const Json&, std::string* result) const override {
        if (key % 2 == 0) return false;
        row[0] = (float)key;
        ++*(int64_t*)&(*result)[0];
        return true;
    }
    void merge_result(const std::string& in, std::string* out) const override { *(int64_t*)&(*out)[0] += *(const int64_t*)in.data(); }
};

// A dense value cut back to front: slice j holds the j-th block counted from the END of the tensor.
static void reversed_partition(int64_t id, size_t numel, uint32_t slice_len, std::vector<DenseSlice>* out) {
    dense_default_partition(id, numel, slice_len, out);
    const size_t ns = out->size();
    for (size_t j = 0; j < ns / 2; ++j) {
        std::swap((*out)[j].offset, (*out)[ns - 1 - j].offset);
        std::swap((*out)[j].len, (*out)[ns - 1 - j].len);
    }
}
class ReversedDensePull : public DenseTablePullOperator {
public:
    explicit ReversedDensePull(const Json& c) : DenseTablePullOperator(c) {}
    void partition(int64_t id, size_t numel, uint32_t slice_len, std::vector<DenseSlice>* out) const override {
        reversed_partition(id, numel, slice_len, out);
    }
};
class ReversedDensePush : public DenseTablePushOperator {
public:
    explicit ReversedDensePush(const Json& c) : DenseTablePushOperator(c) {}
    void partition(int64_t id, size_t numel, uint32_t slice_len, std::vector<DenseSlice>* out) const override {
        reversed_partition(id, numel, slice_len, out);
    }
};

// A reshard codec that leaves a trace: every purge appends a line to the file named in its config.
class TracingUpdateContext : public ShardUpdateContextOperator {
public:
    explicit TracingUpdateContext(const Json& c) : ShardUpdateContextOperator(c), trace_(c.at("trace").as_string()) {}
    Status apply_purge_request(TableEntry& e) const override {
        std::ofstream(trace_, std::ios::app) << "purge " << e.sid << "\n";
        return ShardUpdateContextOperator::apply_purge_request(e);
    }
    Status generate_shuffle_requests(TableEntry& e, int32_t old_shard, const SendBlock& send) const override {
        std::ofstream(trace_, std::ios::app) << "shuffle " << old_shard << "\n";
        return ShardUpdateContextOperator::generate_shuffle_requests(e, old_shard, send);
    }

private:
    std::string trace_;
};

PSB_REGISTER_OPERATOR(testplugin, EraseEvenAbove);
PSB_REGISTER_OPERATOR(testplugin, KeyHistogram);
PSB_REGISTER_OPERATOR(testplugin, StampOddKeys);
PSB_REGISTER_OPERATOR(testplugin, ReversedDensePull);
PSB_REGISTER_OPERATOR(testplugin, ReversedDensePush);
PSB_REGISTER_OPERATOR(testplugin, TracingUpdateContext);
