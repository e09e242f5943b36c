// Request types, message meta and the request/response envelope of the control plane.
//
// Parity: RequestType values are those of pico-ps/common/message.h:15-42; PSMessageMeta mirrors
// pico-ps/common/message.h:45-51 and rides at the TAIL of every request and response, popped with
// read_back (pico-ps/common/DistributedAsyncReturn.cpp:67-70,88-90). On B200 the bulk data plane
// (keys, rows, gradients) moves through NVLink peer memory from inside the fused kernels; this
// envelope carries the control plane and the non-collective (RPC) data path.
#pragma once
#include <cctype>
#include <string>
#include <cstdint>

#include "archive.h"
#include "status.h"

namespace psb {

enum class RequestType : int8_t {
    STORAGE_CREATE = 0,
    STORAGE_DELETE = 1,
    STORAGE_CLEAR = 2,
    STORAGE_STATISTIC = 3,
    HANDLER_REGISTER = 4,
    HANDLER_DEREGISTER = 5,
    OP_FOREACH = 6,
    OP_ERASEIF = 7,
    OP_DUMP = 8,
    OP_LOAD = 9,
    OP_PULL = 10,
    OP_PUSH_ASYNC = 11,
    OP_PUSH_SYNC = 12,
    OP_STORE = 13,
    OP_LOAD_LIBRARY = 14,
    EXIT = 15,
    NEW_CTX_CREATE_SHARD = 16,
    NEW_CTX_SHUFFLE = 17,
    NEW_CTX_STORE = 18,
    NEW_CTX_PURGE = 19,
    CTX_UPDATE = 20,
    OP_SYNC = 21,
    MEMORY_INFO = 22,
    OP_COORDINATED_RESTORE_ITERATE = 23,
    HEALTH_CHECK = 24,
    OP_UDF = 25,
};

inline const char* request_type_name(RequestType t) {
    static const char* names[] = {
        "STORAGE_CREATE", "STORAGE_DELETE", "STORAGE_CLEAR", "STORAGE_STATISTIC", "HANDLER_REGISTER",
        "HANDLER_DEREGISTER", "OP_FOREACH", "OP_ERASEIF", "OP_DUMP", "OP_LOAD", "OP_PULL",
        "OP_PUSH_ASYNC", "OP_PUSH_SYNC", "OP_STORE", "OP_LOAD_LIBRARY", "EXIT", "NEW_CTX_CREATE_SHARD",
        "NEW_CTX_SHUFFLE", "NEW_CTX_STORE", "NEW_CTX_PURGE", "CTX_UPDATE", "OP_SYNC", "MEMORY_INFO",
        "OP_COORDINATED_RESTORE_ITERATE", "HEALTH_CHECK", "OP_UDF"};
    int i = (int)t;
    return (i >= 0 && i < 26) ? names[i] : "UNKNOWN";
}

// The request type as the metric series name it: the reference's labels where it has them (c2s_pull, c2s_async_push,
// c2s_store, c2s_udf_op, s2s_async_push: pico-ps/service/Service.cpp:703-764,820-862,872-894,937-974), the enum name in
// lower case without its OP_ prefix for the rest.
inline std::string request_type_label(RequestType t) {
    switch (t) {
        case RequestType::OP_PULL: return "pull";
        case RequestType::OP_PUSH_ASYNC: return "async_push";
        case RequestType::OP_PUSH_SYNC: return "sync_push";
        case RequestType::OP_STORE: return "store";
        case RequestType::OP_UDF: return "udf_op";
        default: break;
    }
    std::string n = request_type_name(t);
    if (n.compare(0, 3, "OP_") == 0) n = n.substr(3);
    for (auto& c : n) c = (char)std::tolower((unsigned char)c);
    return n;
}

struct PSMessageMeta {
    int32_t sid = -1;        // storage id
    int32_t hid = -1;        // handler id
    int32_t ctx_ver = -1;    // context version the sender believes in
    int32_t ctx_u_ver = -1;  // update (reshard transaction) version, -1 outside a reshard
    RequestType req_type = RequestType::HEALTH_CHECK;
};
static_assert(sizeof(PSMessageMeta) == 20, "meta layout is part of the wire format");

// A request or response: body archive + meta appended last.
struct PSMessage {
    Archive ar;
    PSMessageMeta meta;

    std::vector<uint8_t> seal() {
        Archive out = ar;  // copy: a request may be re-sent on retry
        out << meta;
        return out.release();
    }
    static PSMessage open(std::vector<uint8_t> bytes) {
        PSMessage m;
        m.ar = Archive(std::move(bytes));
        m.ar.read_back(m.meta);
        return m;
    }
};

inline Archive& operator<<(Archive& ar, const Status& st) {
    ar << (int32_t)st.code();
    ar << st.msg();
    return ar;
}
inline Archive& operator>>(Archive& ar, Status& st) {
    int32_t c = 0;
    std::string m;
    ar >> c;
    ar >> m;
    st = Status((StatusCode)c, std::move(m));
    return ar;
}

// Names fixed by the reference (pico-ps/common/defs.h:10-16).
constexpr const char* PSERVER_LOCK_NAME = "PSERVER_LOCK";
constexpr const char* STORAGE_ID_KEY = "storage_id";
constexpr const char* HANDLER_ID_KEY = "handler";
constexpr const char* PSERVER_C2S_RPC_NAME = "pserver_c2s_rpc_api";
constexpr const char* PSERVER_S2S_RPC_NAME = "pserver_s2s_rpc_api";

}  // namespace psb
