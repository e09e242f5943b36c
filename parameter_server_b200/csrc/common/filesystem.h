// Files of dumps and loads: local paths, or a Hadoop file system reached through the `hadoop fs` command line.
//
// Parity: the reference reads and writes its dump files through prpc's FileSystem / ShellUtility, which serve
// `hdfs://` URIs by piping through `<hadoop_bin> fs -cat / -put / -ls / -mkdir -p / -rm` (the `hadoop_bin` argument of
// its Server constructor, DumpArgs and LoadHandler: pico-ps/service/Server.h:52-55, pico-ps/operator/DumpOperator.h:17-43,
// pico-ps/handler/LoadHandler.cpp:75-137). The same here: a path that starts with a remote scheme goes through
// the configured command (argv, no shell), everything else through the local file system. Files are moved whole,
// which is how the dump codec works anyway (one compressed block per file).
#pragma once
#include <dirent.h>
#include <fcntl.h>
#include <signal.h>
#include <sys/stat.h>
#include <sys/wait.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iterator>
#include <mutex>
#include <string>
#include <vector>

#include "status.h"

namespace psb {
namespace fs {

inline std::mutex& config_mu() {
    static std::mutex m;
    return m;
}
inline std::string& hadoop_bin_ref() {
    static std::string bin = [] {
        const char* env = std::getenv("PSB_HADOOP_BIN");
        return std::string(env && *env ? env : "hadoop");
    }();
    return bin;
}
// The command that serves remote paths (default: $PSB_HADOOP_BIN, else "hadoop" on PATH). Process-wide.
inline void set_hadoop_bin(const std::string& bin) {
    std::lock_guard<std::mutex> g(config_mu());
    hadoop_bin_ref() = bin.empty() ? "hadoop" : bin;
}
inline std::string hadoop_bin() {
    std::lock_guard<std::mutex> g(config_mu());
    return hadoop_bin_ref();
}

inline bool is_remote(const std::string& path) {
    for (const char* scheme : {"hdfs://", "viewfs://", "s3a://", "gs://", "abfs://"})
        if (path.compare(0, std::strlen(scheme), scheme) == 0) return true;
    return false;
}

// Runs argv (no shell), feeds `in` to its stdin, collects its stdout. A non-zero exit is an error.
inline Status run(const std::vector<std::string>& argv, const uint8_t* in, size_t in_len, std::vector<uint8_t>* out) {
    static std::once_flag once;
    std::call_once(once, [] { ::signal(SIGPIPE, SIG_IGN); });   // a child that dies early must not take the server along
    int to_child[2] = {-1, -1}, from_child[2] = {-1, -1};
    // close-on-exec: a command started by another thread at the same time must not inherit (and hold open) these ends
    if (::pipe2(to_child, O_CLOEXEC) != 0) return Status::Error("pipe failed");
    if (::pipe2(from_child, O_CLOEXEC) != 0) {
        ::close(to_child[0]);
        ::close(to_child[1]);
        return Status::Error("pipe failed");
    }
    // everything the child needs is laid out before the fork: in a process with other threads the child may only
    // make async-signal-safe calls (no allocation) until it has exec'ed
    std::vector<char*> args;
    for (auto& a : argv) args.push_back(const_cast<char*>(a.c_str()));
    args.push_back(nullptr);
    const int fds[4] = {to_child[0], to_child[1], from_child[0], from_child[1]};
    const pid_t pid = ::fork();
    if (pid < 0) {
        for (int fd : fds) ::close(fd);
        return Status::Error("fork failed");
    }
    if (pid == 0) {
        ::dup2(to_child[0], 0);
        ::dup2(from_child[1], 1);
        for (int fd : fds) ::close(fd);
        ::execvp(args[0], args.data());
        ::_exit(127);
    }
    ::close(to_child[0]);
    ::close(from_child[1]);
    // the commands used here either take input (put) or give output (cat, ls), never much of both: write, then read
    bool write_ok = true;
    for (size_t off = 0; off < in_len;) {
        const ssize_t n = ::write(to_child[1], in + off, in_len - off);
        if (n < 0) {
            if (errno == EINTR) continue;
            write_ok = false;
            break;
        }
        off += (size_t)n;
    }
    ::close(to_child[1]);
    uint8_t buf[1 << 16];
    for (;;) {
        const ssize_t n = ::read(from_child[0], buf, sizeof buf);
        if (n < 0 && errno == EINTR) continue;
        if (n <= 0) break;
        if (out) out->insert(out->end(), buf, buf + n);
    }
    ::close(from_child[0]);
    int status = 0;
    while (::waitpid(pid, &status, 0) < 0 && errno == EINTR) {}
    if (!write_ok || !WIFEXITED(status) || WEXITSTATUS(status) != 0) {
        std::string cmd;
        for (auto& a : argv) cmd += (cmd.empty() ? "" : " ") + a;
        const int code = WIFEXITED(status) ? WEXITSTATUS(status) : -1;
        return Status::Error("command failed (" + std::to_string(code) + (code == 127 ? ", not found" : "") + "): " + cmd);
    }
    return Status::Ok();
}
inline Status hadoop(std::vector<std::string> args, const uint8_t* in = nullptr, size_t in_len = 0, std::vector<uint8_t>* out = nullptr) {
    std::vector<std::string> argv = {hadoop_bin(), "fs"};
    argv.insert(argv.end(), args.begin(), args.end());
    return run(argv, in, in_len, out);
}

inline Status mkdir_p(const std::string& path) {
    if (is_remote(path)) return hadoop({"-mkdir", "-p", path});
    std::string cur;
    for (size_t i = 0; i <= path.size(); ++i) {
        if (i == path.size() || path[i] == '/') {
            if (!cur.empty() && ::mkdir(cur.c_str(), 0777) != 0 && errno != EEXIST) return Status::Error("mkdir " + cur + " failed");
        }
        if (i < path.size()) cur += path[i];
    }
    return Status::Ok();
}

inline Status write_file(const std::string& path, const std::vector<uint8_t>& data) {
    if (is_remote(path)) return hadoop({"-put", "-f", "-", path}, data.data(), data.size());
    std::ofstream f(path, std::ios::binary | std::ios::trunc);
    if (!f) return Status::Error("cannot open " + path + " for writing");
    f.write((const char*)data.data(), (std::streamsize)data.size());
    return f.good() ? Status::Ok() : Status::Error("write to " + path + " failed");
}

inline Status read_file(const std::string& path, std::vector<uint8_t>* data) {
    data->clear();
    if (is_remote(path)) return hadoop({"-cat", path}, nullptr, 0, data);
    std::ifstream f(path, std::ios::binary);
    if (!f) return Status::Error("cannot open " + path);
    data->assign(std::istreambuf_iterator<char>(f), std::istreambuf_iterator<char>());
    return Status::Ok();
}

// Full paths of the entries of `dir` whose name starts with `prefix`, sorted. A directory that cannot be listed
// gives an empty list.
inline std::vector<std::string> list(const std::string& dir, const std::string& prefix) {
    std::vector<std::string> out;
    if (is_remote(dir)) {
        std::vector<uint8_t> text;
        if (!hadoop({"-ls", dir}, nullptr, 0, &text).ok()) return out;
        // one entry per line, the path is the last column ("Found N items" and the like have no '/' in it)
        std::string line;
        text.push_back('\n');
        for (uint8_t c : text) {
            if (c != '\n') {
                line += (char)c;
                continue;
            }
            const size_t sp = line.find_last_of(" \t");
            const std::string path = sp == std::string::npos ? line : line.substr(sp + 1);
            const size_t slash = path.rfind('/');
            if ((line[0] == '-' || line[0] == 'd') && slash != std::string::npos && path.compare(slash + 1, prefix.size(), prefix) == 0)
                out.push_back(path);
            line.clear();
        }
    } else if (DIR* d = ::opendir(dir.c_str())) {
        while (dirent* e = ::readdir(d)) {
            const std::string n = e->d_name;
            if (n != "." && n != ".." && n.compare(0, prefix.size(), prefix) == 0) out.push_back(dir + "/" + n);
        }
        ::closedir(d);
    }
    std::sort(out.begin(), out.end());
    return out;
}

inline Status remove_file(const std::string& path) {
    if (is_remote(path)) return hadoop({"-rm", "-f", path});
    return ::remove(path.c_str()) == 0 || errno == ENOENT ? Status::Ok() : Status::Error("cannot remove " + path);
}

}  // namespace fs
}  // namespace psb
