// Status taxonomy of the parameter server.
//
// Parity: code values and names follow pico-ps/common/Status.h:15-29 so that the client-side retry
// policy (timeout / no-replica -> dead-node detection, too-new-ctx -> refresh, out-of-memory -> wait
// for a context change; pico-ps/handler/Handler.cpp:65-103) can be expressed on the same codes.
// Device kernels report through a 32-bit status word whose low byte is one of these codes.
#pragma once
#include <cstdint>
#include <string>
#include <utility>

namespace psb {

enum class StatusCode : int32_t {
    OK = 0,
    INVALID_CONFIG = 1,
    INVALID_ID = 2,
    OUT_OF_MEMORY = 3,
    TIMEOUT = 4,
    SERVER_TOO_NEW_CTX = 5,
    SERVER_TOO_OLD_CTX = 6,
    SERVER_TOO_NEW_CTX_U = 7,
    SERVER_TOO_OLD_CTX_U = 8,
    NO_REPLICA = 9,
    ERROR = 10,
    FATAL = 11,
    EMPTY = 12,
};

inline const char* status_code_name(StatusCode c) {
    switch (c) {
        case StatusCode::OK: return "OK";
        case StatusCode::INVALID_CONFIG: return "InvalidConfig";
        case StatusCode::INVALID_ID: return "InvalidID";
        case StatusCode::OUT_OF_MEMORY: return "OutOfMemory";
        case StatusCode::TIMEOUT: return "Timeout";
        case StatusCode::SERVER_TOO_NEW_CTX: return "ServerTooNewCtx";
        case StatusCode::SERVER_TOO_OLD_CTX: return "ServerTooOldCtx";
        case StatusCode::SERVER_TOO_NEW_CTX_U: return "ServerTooNewCtxU";
        case StatusCode::SERVER_TOO_OLD_CTX_U: return "ServerTooOldCtxU";
        case StatusCode::NO_REPLICA: return "NoReplica";
        case StatusCode::ERROR: return "Error";
        case StatusCode::FATAL: return "Fatal";
        case StatusCode::EMPTY: return "Empty";
    }
    return "Unknown";
}

class Status {
public:
    Status() = default;
    Status(StatusCode c, std::string m) : code_(c), msg_(std::move(m)) {}

    static Status Ok() { return Status(); }
    static Status InvalidConfig(std::string m) { return {StatusCode::INVALID_CONFIG, std::move(m)}; }
    static Status InvalidID(std::string m) { return {StatusCode::INVALID_ID, std::move(m)}; }
    static Status OOM(std::string m) { return {StatusCode::OUT_OF_MEMORY, std::move(m)}; }
    static Status Timeout(std::string m) { return {StatusCode::TIMEOUT, std::move(m)}; }
    static Status ServerTooNewCtx(std::string m) { return {StatusCode::SERVER_TOO_NEW_CTX, std::move(m)}; }
    static Status ServerTooOldCtx(std::string m) { return {StatusCode::SERVER_TOO_OLD_CTX, std::move(m)}; }
    static Status ServerTooNewCtxU(std::string m) { return {StatusCode::SERVER_TOO_NEW_CTX_U, std::move(m)}; }
    static Status ServerTooOldCtxU(std::string m) { return {StatusCode::SERVER_TOO_OLD_CTX_U, std::move(m)}; }
    static Status NoReplica(std::string m) { return {StatusCode::NO_REPLICA, std::move(m)}; }
    static Status Error(std::string m) { return {StatusCode::ERROR, std::move(m)}; }
    static Status Fatal(std::string m) { return {StatusCode::FATAL, std::move(m)}; }
    static Status Empty(std::string m) { return {StatusCode::EMPTY, std::move(m)}; }

    bool ok() const { return code_ == StatusCode::OK; }
    StatusCode code() const { return code_; }
    const std::string& msg() const { return msg_; }
    bool is(StatusCode c) const { return code_ == c; }

    std::string to_string() const {
        if (ok()) return "OK";
        return std::string(status_code_name(code_)) + ": " + msg_;
    }

private:
    StatusCode code_ = StatusCode::OK;
    std::string msg_;
};

#define PSB_RETURN_IF_ERROR(expr)            \
    do {                                     \
        ::psb::Status _st = (expr);          \
        if (!_st.ok()) return _st;           \
    } while (0)

}  // namespace psb
