// A minimal HTTP endpoint that serves one text document (the Prometheus exposition of a server's request series)
// on GET, for native processes without Python. One accept thread, one short-lived connection at a time: scrapes
// are rare and small.
//
// Parity: the reference's servers export their ps_* series through prpc's metrics service
// (pico-ps/service/Service.cpp:23-33); the series themselves are produced by Server::metrics_text.
#pragma once
#include <arpa/inet.h>
#include <netinet/in.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <functional>
#include <stdexcept>
#include <string>
#include <thread>

namespace psb {

class MetricsHttpServer {
public:
    // port 0 = any free port (see port()). `body` is called for every scrape.
    MetricsHttpServer(int port, std::function<std::string()> body) : body_(std::move(body)) {
        fd_ = ::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
        if (fd_ < 0) throw std::runtime_error("metrics: socket failed");
        int one = 1;
        ::setsockopt(fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
        sockaddr_in addr{};
        addr.sin_family = AF_INET;
        addr.sin_addr.s_addr = htonl(INADDR_ANY);
        addr.sin_port = htons((uint16_t)port);
        if (::bind(fd_, (sockaddr*)&addr, sizeof addr) != 0 || ::listen(fd_, 16) != 0) {
            ::close(fd_);
            throw std::runtime_error("metrics: cannot listen on port " + std::to_string(port));
        }
        socklen_t len = sizeof addr;
        ::getsockname(fd_, (sockaddr*)&addr, &len);
        port_ = ntohs(addr.sin_port);
        thread_ = std::thread([this] { loop(); });
    }
    ~MetricsHttpServer() { stop(); }
    MetricsHttpServer(const MetricsHttpServer&) = delete;
    MetricsHttpServer& operator=(const MetricsHttpServer&) = delete;

    int port() const { return port_; }
    void stop() {
        if (!running_.exchange(false)) return;
        if (thread_.joinable()) thread_.join();   // the loop polls with a timeout and sees the flag
        ::close(fd_);
    }

private:
    void loop() {
        while (running_) {
            pollfd p{fd_, POLLIN, 0};
            if (::poll(&p, 1, 100) <= 0) continue;
            const int c = ::accept4(fd_, nullptr, nullptr, SOCK_CLOEXEC);
            if (c < 0) continue;
            serve(c);
            ::close(c);
        }
    }
    void serve(int c) {
        // read the request head (bounded in size and time); only the request line matters
        std::string head;
        char buf[1024];
        for (int spins = 0; spins < 50 && head.size() < 8192 && head.find("\r\n\r\n") == std::string::npos; ++spins) {
            pollfd p{c, POLLIN, 0};
            if (::poll(&p, 1, 100) <= 0) continue;
            const ssize_t n = ::recv(c, buf, sizeof buf, 0);
            if (n <= 0) break;
            head.append(buf, (size_t)n);
        }
        std::string status = "200 OK", body;
        if (head.compare(0, 4, "GET ") != 0) {
            status = "405 Method Not Allowed";
        } else {
            const size_t sp = head.find(' ', 4);
            const std::string path = head.substr(4, sp == std::string::npos ? std::string::npos : sp - 4);
            if (path == "/metrics" || path == "/") body = body_();
            else status = "404 Not Found";
        }
        const std::string resp = "HTTP/1.1 " + status + "\r\nContent-Type: text/plain; version=0.0.4\r\nContent-Length: " +
                                 std::to_string(body.size()) + "\r\nConnection: close\r\n\r\n" + body;
        for (size_t off = 0; off < resp.size();) {
            const ssize_t n = ::send(c, resp.data() + off, resp.size() - off, MSG_NOSIGNAL);
            if (n <= 0) break;
            off += (size_t)n;
        }
    }

    std::function<std::string()> body_;
    int fd_ = -1, port_ = 0;
    std::atomic<bool> running_{true};
    std::thread thread_;
};

}  // namespace psb
