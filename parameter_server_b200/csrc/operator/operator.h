// Operator base class and the (lib_name, op_name) -> producer registry.
//
// Parity: pico-ps/operator/Operator.h:51-130 (Operator(conf), OperatorFactory singleton,
// REGISTER_OPERATOR static registration) and pico-ps/operator/Operator.cpp:15-61. The pair
// (lib_name, op_name) is the cross-process identity of an operator: it travels in the context JSON
// so that every client and server builds the same object. load_library is real here (dlopen of a
// shared object whose static initialisers register more operators); in the reference it is a stub.
// A plug-in includes operators.h, derives from the *Base classes (or from a built-in operator), registers its classes
// with PSB_REGISTER_OPERATOR(lib, Class) and is compiled with
//   g++ -std=c++17 -shared -fPIC -DPSB_OPERATOR_PLUGIN -I <csrc> plugin.cpp -o libplugin.so
// Every process that builds operators from the context (servers AND clients) must load it: Client::load_operator_library
// does so locally and on every server.
#pragma once
#include <dlfcn.h>

#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <string>

#include "../common/json.h"
#include "../common/status.h"

namespace psb {

class Operator {
public:
    explicit Operator(const Json& config) : config_(config) {}
    virtual ~Operator() = default;
    const Json& config() const { return config_; }
    // What the operator is, for dispatch checks: "storage", "pull", "push", "direct_push", "for_each",
    // "erase_if", "dump", "load", "restore", "update_ctx", "sync", "udf".
    virtual const char* kind() const = 0;

protected:
    Json config_;
};

class OperatorFactory;
}  // namespace psb

// The one registry of a process. The host (the Python module or the psb_node executable) defines and exports this
// accessor; a plug-in library compiled with -DPSB_OPERATOR_PLUGIN leaves it undefined, so that the dynamic loader
// binds it to the host's registry when the library is opened and the plug-in's static registrations land there.
extern "C" void* psb_operator_factory();

namespace psb {

class OperatorFactory {
public:
    using Producer = std::function<std::shared_ptr<Operator>(const Json&)>;

    static OperatorFactory& instance() { return *static_cast<OperatorFactory*>(psb_operator_factory()); }
    void register_producer(const std::string& lib, const std::string& op, Producer p) {
        std::lock_guard<std::mutex> g(mu_);
        producers_[lib + "\x1f" + op] = std::move(p);
    }
    Status create(const std::string& lib, const std::string& op, const std::string& config_str,
                  std::shared_ptr<Operator>* out) {
        Json cfg = Json::object();
        if (!config_str.empty() && !Json::parse_config(config_str, &cfg))
            return Status::InvalidConfig("operator config of " + lib + "/" + op + " is neither valid JSON nor YAML");
        Producer p;
        {
            std::lock_guard<std::mutex> g(mu_);
            auto it = producers_.find(lib + "\x1f" + op);
            if (it == producers_.end()) return Status::InvalidConfig("no operator registered as (" + lib + ", " + op + ")");
            p = it->second;
        }
        try {
            *out = p(cfg);
        } catch (const std::exception& e) {
            return Status::InvalidConfig(std::string("operator ") + op + ": " + e.what());
        }
        return Status::Ok();
    }
    bool has(const std::string& lib, const std::string& op) {
        std::lock_guard<std::mutex> g(mu_);
        return producers_.count(lib + "\x1f" + op) != 0;
    }
    Status load_library(const std::string& path) {
        void* h = dlopen(path.c_str(), RTLD_NOW | RTLD_GLOBAL);
        if (!h) return Status::Error(std::string("load_library: ") + dlerror());
        return Status::Ok();
    }

private:
    std::mutex mu_;
    std::map<std::string, Producer> producers_;
};

template <class OP>
struct OperatorRegisterer {
    OperatorRegisterer(const char* lib, const char* name) {
        OperatorFactory::instance().register_producer(lib, name, [](const Json& c) { return std::make_shared<OP>(c); });
    }
};

#define PSB_REGISTER_OPERATOR(lib, cls) \
    static ::psb::OperatorRegisterer<cls> psb_register_##cls(#lib, #cls)

}  // namespace psb
