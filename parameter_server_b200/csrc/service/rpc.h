// Host control-plane transport: length-framed request / response messages over TCP on localhost.
//
// Parity: stands for the slice of prpc that pico-ps uses (pico-ps/common/core.h:124-141: RpcService,
// RpcServer, RpcClient, Dealer): a server accepts requests and answers them (possibly later, from
// another thread: the UDF operator keeps the dealer), a client fans requests out to several servers
// and collects the answers with a timeout; a broken or missing peer surfaces as Status::Timeout, the
// analogue of prpc's ENOSUCHSERVER (pico-ps/common/DistributedAsyncReturn.cpp:46-54). On B200 this
// channel only carries control messages and the non-collective data path; bulk keys / rows /
// gradients of training ranks move through NVLink peer memory inside the fused kernels.
//
// Frame: u32 payload_len | u64 request_id | u8 kind (0 request, 1 response) | payload bytes.
#pragma once
#include <arpa/inet.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstdlib>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "../common/status.h"

namespace psb {

using Bytes = std::vector<uint8_t>;

namespace rpc_detail {
// The address this process publishes for its servers: $PSB_HOST, else loopback.
inline std::string local_host() {
    const char* h = std::getenv("PSB_HOST");
    return h && *h ? std::string(h) : std::string("127.0.0.1");
}
// Dotted address or host name -> IPv4 address.
inline bool resolve(const std::string& host, in_addr* out) {
    if (::inet_pton(AF_INET, host.c_str(), out) == 1) return true;
    addrinfo hints{}, *res = nullptr;
    hints.ai_family = AF_INET;
    hints.ai_socktype = SOCK_STREAM;
    if (::getaddrinfo(host.c_str(), nullptr, &hints, &res) != 0 || !res) return false;
    *out = ((sockaddr_in*)res->ai_addr)->sin_addr;
    ::freeaddrinfo(res);
    return true;
}
inline bool read_full(int fd, void* buf, size_t n) {
    uint8_t* p = (uint8_t*)buf;
    while (n) {
        ssize_t r = ::recv(fd, p, n, 0);
        if (r <= 0) {
            if (r < 0 && (errno == EINTR)) continue;
            return false;
        }
        p += r;
        n -= (size_t)r;
    }
    return true;
}
inline bool write_full(int fd, const void* buf, size_t n) {
    const uint8_t* p = (const uint8_t*)buf;
    while (n) {
        ssize_t r = ::send(fd, p, n, MSG_NOSIGNAL);
        if (r <= 0) {
            if (r < 0 && errno == EINTR) continue;
            return false;
        }
        p += r;
        n -= (size_t)r;
    }
    return true;
}
constexpr uint32_t kMaxFrameBytes = 1u << 30;

inline bool write_frame(int fd, std::mutex& mu, uint64_t id, uint8_t kind, const Bytes& payload) {
    uint8_t hdr[13];
    uint32_t len = (uint32_t)payload.size();
    std::memcpy(hdr, &len, 4);
    std::memcpy(hdr + 4, &id, 8);
    hdr[12] = kind;
    std::lock_guard<std::mutex> g(mu);
    return write_full(fd, hdr, 13) && (payload.empty() || write_full(fd, payload.data(), payload.size()));
}
inline bool read_frame(int fd, uint64_t* id, uint8_t* kind, Bytes* payload) {
    uint8_t hdr[13];
    if (!read_full(fd, hdr, 13)) return false;
    uint32_t len;
    std::memcpy(&len, hdr, 4);
    std::memcpy(id, hdr + 4, 8);
    *kind = hdr[12];
    if (len > kMaxFrameBytes) return false;  // nobody sends this: drop the connection instead of allocating for it
    payload->resize(len);
    return len == 0 || read_full(fd, payload->data(), len);
}
}  // namespace rpc_detail

// ---------------------------------------------------------------------------------------------------
class RpcServer {
public:
    struct Conn {
        int fd = -1;
        uint64_t id = 0;
        std::mutex wmu;
        std::atomic<bool> alive{true};
    };
    // The way to answer one request; may be copied and called later from any thread (once).
    class Responder {
    public:
        Responder() = default;
        Responder(std::shared_ptr<Conn> c, uint64_t req) : conn_(std::move(c)), req_(req) {}
        bool send(const Bytes& payload) const {
            if (!conn_ || !conn_->alive) return false;
            return rpc_detail::write_frame(conn_->fd, conn_->wmu, req_, 1, payload);
        }
        uint64_t conn_id() const { return conn_ ? conn_->id : 0; }
    private:
        std::shared_ptr<Conn> conn_;
        uint64_t req_ = 0;
    };
    using Handler = std::function<void(Bytes&&, Responder)>;
    using DisconnectHandler = std::function<void(uint64_t conn_id)>;

    // port 0 = any free port (the usual case: addresses are published through the master); a fixed port is for the
    // master itself, which clients must find again after it was restarted
    RpcServer(Handler h, int n_threads, DisconnectHandler on_disconnect = nullptr, int port = 0)
        : handler_(std::move(h)), on_disconnect_(std::move(on_disconnect)) {
        listen_fd_ = ::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
        int one = 1;
        ::setsockopt(listen_fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
        sockaddr_in addr{};
        addr.sin_family = AF_INET;
        // One box is the default: listen on loopback. With $PSB_HOST (psb_node --host) set to this machine's address
        // or name the servers listen on every interface and publish that address, so that masters, servers and
        // clients may sit on different machines (the reference's deployment; its tests use localhost as well).
        host_ = rpc_detail::local_host();
        if (host_ == "127.0.0.1") addr.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
        else if (host_.compare(0, 4, "127.") == 0) ::inet_pton(AF_INET, host_.c_str(), &addr.sin_addr);
        else addr.sin_addr.s_addr = htonl(INADDR_ANY);
        addr.sin_port = htons((uint16_t)port);
        if (::bind(listen_fd_, (sockaddr*)&addr, sizeof addr) != 0 || ::listen(listen_fd_, 256) != 0) {
            ::close(listen_fd_);
            throw std::runtime_error("RpcServer: cannot listen on port " + std::to_string(port));
        }
        socklen_t len = sizeof addr;
        ::getsockname(listen_fd_, (sockaddr*)&addr, &len);
        port_ = ntohs(addr.sin_port);
        for (int i = 0; i < n_threads; ++i) workers_.emplace_back([this] { work(); });
        accept_thread_ = std::thread([this] { accept_loop(); });
    }
    ~RpcServer() { stop(); }

    int port() const { return port_; }
    std::string address() const { return host_ + ":" + std::to_string(port_); }

    void stop() {
        bool was = running_.exchange(false);
        if (!was) return;
        ::shutdown(listen_fd_, SHUT_RDWR);
        ::close(listen_fd_);
        {
            std::lock_guard<std::mutex> g(mu_);
            for (auto& c : conns_) {
                c->alive = false;
                ::shutdown(c->fd, SHUT_RDWR);
            }
        }
        cv_.notify_all();
        if (accept_thread_.joinable()) accept_thread_.join();
        for (auto& t : workers_) if (t.joinable()) t.join();
        std::vector<std::thread> readers;
        {
            std::lock_guard<std::mutex> g(mu_);
            readers.swap(readers_);
        }
        for (auto& t : readers) if (t.joinable()) t.join();
        std::lock_guard<std::mutex> g(mu_);
        for (auto& c : conns_) ::close(c->fd);
        conns_.clear();
    }

private:
    struct Task { Bytes req; Responder resp; };

    void accept_loop() {
        while (running_) {
            int fd = ::accept4(listen_fd_, nullptr, nullptr, SOCK_CLOEXEC);   // not inherited by commands that a server starts
            if (fd < 0) {
                if (!running_) break;
                continue;
            }
            int one = 1;
            ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
            auto c = std::make_shared<Conn>();
            c->fd = fd;
            c->id = ++next_conn_;
            std::lock_guard<std::mutex> g(mu_);
            conns_.push_back(c);
            readers_.emplace_back([this, c] { read_loop(c); });
        }
    }
    void read_loop(std::shared_ptr<Conn> c) {
        for (;;) {
            uint64_t id;
            uint8_t kind;
            Bytes payload;
            if (!rpc_detail::read_frame(c->fd, &id, &kind, &payload)) break;
            std::lock_guard<std::mutex> g(mu_);
            tasks_.push_back(Task{std::move(payload), Responder(c, id)});
            cv_.notify_one();
        }
        c->alive = false;
        if (on_disconnect_ && running_) on_disconnect_(c->id);
    }
    void work() {
        for (;;) {
            Task t;
            {
                std::unique_lock<std::mutex> g(mu_);
                cv_.wait(g, [this] { return !tasks_.empty() || !running_; });
                if (tasks_.empty()) return;
                t = std::move(tasks_.front());
                tasks_.pop_front();
            }
            try {
                handler_(std::move(t.req), t.resp);
            } catch (...) {
                // a handler must answer with a Status itself; swallow to keep the pool alive
            }
        }
    }

    Handler handler_;
    DisconnectHandler on_disconnect_;
    int listen_fd_ = -1, port_ = 0;
    std::string host_ = "127.0.0.1";
    std::atomic<bool> running_{true};
    std::atomic<uint64_t> next_conn_{0};
    std::thread accept_thread_;
    std::vector<std::thread> workers_, readers_;
    std::vector<std::shared_ptr<Conn>> conns_;
    std::deque<Task> tasks_;
    std::mutex mu_;
    std::condition_variable cv_;
};

// ---------------------------------------------------------------------------------------------------
class RpcClient {
public:
    struct Pending {
        std::mutex mu;
        std::condition_variable cv;
        bool done = false, broken = false;
        Bytes payload;
    };
    using Ticket = std::shared_ptr<Pending>;

    RpcClient() = default;
    ~RpcClient() { close_all(); }

    // Fire a request; the ticket is redeemed with wait(). A peer that cannot be reached yields a
    // ticket that is already broken.
    Ticket send(const std::string& address, const Bytes& payload) {
        auto p = std::make_shared<Pending>();
        auto ch = channel(address);
        if (!ch) {
            p->done = p->broken = true;
            return p;
        }
        uint64_t id = ++next_id_;
        {
            std::lock_guard<std::mutex> g(ch->mu);
            ch->pending[id] = p;
        }
        if (!rpc_detail::write_frame(ch->fd, ch->wmu, id, 0, payload)) {
            drop(address);
            std::lock_guard<std::mutex> g(p->mu);
            p->done = p->broken = true;
        }
        return p;
    }
    // OK with the payload, or Timeout (limit ran out / peer gone: the caller decides which by asking
    // the master whether the node is still registered).
    Status wait(const Ticket& t, int timeout_ms, Bytes* out) {
        std::unique_lock<std::mutex> g(t->mu);
        if (timeout_ms < 0) t->cv.wait(g, [&] { return t->done; });
        else if (!t->cv.wait_for(g, std::chrono::milliseconds(timeout_ms), [&] { return t->done; }))
            return Status::Timeout("rpc: no response within " + std::to_string(timeout_ms) + " ms");
        if (t->broken) return Status::Timeout("rpc: no such server / connection broken");
        *out = std::move(t->payload);
        return Status::Ok();
    }
    Status call(const std::string& address, const Bytes& payload, int timeout_ms, Bytes* out) {
        return wait(send(address, payload), timeout_ms, out);
    }
    void drop(const std::string& address) {
        std::shared_ptr<Channel> ch;
        {
            std::lock_guard<std::mutex> g(mu_);
            auto it = channels_.find(address);
            if (it == channels_.end()) return;
            ch = it->second;
            channels_.erase(it);
        }
        // Other threads may still hold this channel and be writing to it: shut the socket down (their calls
        // fail) but leave the descriptor open until the last holder lets go, or its number could be handed to
        // a new connection under their feet.
        ::shutdown(ch->fd, SHUT_RDWR);
        std::lock_guard<std::mutex> g(ch->join_mu);
        if (ch->reader.joinable()) {
            if (ch->reader.get_id() == std::this_thread::get_id()) ch->reader.detach();
            else ch->reader.join();
        }
    }
    void close_all() {
        std::vector<std::string> addrs;
        {
            std::lock_guard<std::mutex> g(mu_);
            for (auto& kv : channels_) addrs.push_back(kv.first);
        }
        for (auto& a : addrs) drop(a);
    }
    bool connected(const std::string& address) {
        std::lock_guard<std::mutex> g(mu_);
        auto it = channels_.find(address);
        return it != channels_.end() && it->second->alive;
    }

private:
    struct Channel {
        int fd = -1;
        std::mutex mu, wmu, join_mu;
        std::map<uint64_t, Ticket> pending;
        std::thread reader;
        std::atomic<bool> alive{true};
        ~Channel() {
            if (reader.joinable()) reader.detach();  // only reached on the reader thread itself, as its last act
            if (fd >= 0) ::close(fd);
        }
    };

    std::shared_ptr<Channel> channel(const std::string& address) {
        std::lock_guard<std::mutex> g(mu_);
        auto it = channels_.find(address);
        if (it != channels_.end()) {
            if (it->second->alive) return it->second;
            auto dead = it->second;
            channels_.erase(it);
            std::lock_guard<std::mutex> jg(dead->join_mu);
            if (dead->reader.joinable()) dead->reader.join();   // the descriptor closes with the last holder
        }
        auto colon = address.rfind(':');
        if (colon == std::string::npos) return nullptr;
        sockaddr_in addr{};
        addr.sin_family = AF_INET;
        addr.sin_port = htons((uint16_t)std::stoi(address.substr(colon + 1)));
        if (!rpc_detail::resolve(address.substr(0, colon), &addr.sin_addr)) return nullptr;
        int fd = ::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
        if (fd < 0) return nullptr;
        if (::connect(fd, (sockaddr*)&addr, sizeof addr) != 0) {
            ::close(fd);
            return nullptr;
        }
        int one = 1;
        ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
        auto ch = std::make_shared<Channel>();
        ch->fd = fd;
        ch->reader = std::thread([ch] {
            for (;;) {
                uint64_t id;
                uint8_t kind;
                Bytes payload;
                if (!rpc_detail::read_frame(ch->fd, &id, &kind, &payload)) break;
                Ticket t;
                {
                    std::lock_guard<std::mutex> g(ch->mu);
                    auto it = ch->pending.find(id);
                    if (it == ch->pending.end()) continue;
                    t = it->second;
                    ch->pending.erase(it);
                }
                std::lock_guard<std::mutex> g(t->mu);
                t->payload = std::move(payload);
                t->done = true;
                t->cv.notify_all();
            }
            ch->alive = false;
            std::map<uint64_t, Ticket> rest;
            {
                std::lock_guard<std::mutex> g(ch->mu);
                rest.swap(ch->pending);
            }
            for (auto& kv : rest) {
                std::lock_guard<std::mutex> g(kv.second->mu);
                kv.second->done = kv.second->broken = true;
                kv.second->cv.notify_all();
            }
        });
        channels_[address] = ch;
        return ch;
    }

    std::mutex mu_;
    std::map<std::string, std::shared_ptr<Channel>> channels_;
    std::atomic<uint64_t> next_id_{0};
};

}  // namespace psb
