// A keyed rendezvous store over TCP: a threaded server inside the master rank's process and a blocking client in
// every rank, the counterpart of the reference's store (lumen/distributed/store.rs:43-72,100-230): set, get (waits
// until the key exists), add (an integer counter), wait (for a set of keys) and delete. EVERY wait carries a deadline -
// a peer that never arrives makes the others return LB_ERR_TIMEOUT instead of hanging - and so does every socket
// read. The process group's barrier and the exchange of the NCCL unique id (comm.cpp) are built on it.
//
// Wire format (this library's own): a request is `u32 op, i64 number, u32 n_strings, then n_strings x (u32 length,
// bytes)`; a reply is `u32 status (0 found, 1 timed out), i64 number, u32 length, bytes`. Little-endian.
#include <arpa/inet.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <thread>

#include "common.h"

namespace lb {
namespace {

using Clock = std::chrono::steady_clock;
enum Op : uint32_t { OP_SET = 1, OP_GET = 2, OP_ADD = 3, OP_WAIT = 4, OP_DELETE = 5 };

struct Table {
    std::mutex mutex;
    std::condition_variable changed;
    std::map<std::string, std::string> values;
};

// Reads exactly n bytes or fails; `deadline_ms` < 0 waits without limit (server side: a client may stay idle).
bool read_all(int fd, void* buf, size_t n, int deadline_ms) {
    char* p = (char*)buf;
    auto until = Clock::now() + std::chrono::milliseconds(deadline_ms < 0 ? 0 : deadline_ms);
    while (n > 0) {
        if (deadline_ms >= 0) {
            auto left = std::chrono::duration_cast<std::chrono::milliseconds>(until - Clock::now()).count();
            if (left <= 0) return false;
            pollfd pfd{fd, POLLIN, 0};
            int rc = poll(&pfd, 1, (int)std::min<long long>(left, 1000));
            if (rc < 0 && errno != EINTR) return false;
            if (rc <= 0) continue;
        }
        ssize_t got = recv(fd, p, n, 0);
        if (got == 0) return false;
        if (got < 0) {
            if (errno == EINTR) continue;
            return false;
        }
        p += got, n -= (size_t)got;
    }
    return true;
}

bool write_all(int fd, const void* buf, size_t n) {
    const char* p = (const char*)buf;
    while (n > 0) {
        ssize_t put = send(fd, p, n, MSG_NOSIGNAL);
        if (put < 0) {
            if (errno == EINTR) continue;
            return false;
        }
        p += put, n -= (size_t)put;
    }
    return true;
}

struct Frame {
    uint32_t op = 0;  // request: Op; reply: status
    int64_t number = 0;
    std::vector<std::string> strings;
};

bool send_frame(int fd, const Frame& f) {
    std::string out;
    auto put = [&](const void* p, size_t n) { out.append((const char*)p, n); };
    uint32_t count = (uint32_t)f.strings.size();
    put(&f.op, 4), put(&f.number, 8), put(&count, 4);
    for (auto& s : f.strings) {
        uint32_t len = (uint32_t)s.size();
        put(&len, 4), put(s.data(), s.size());
    }
    return write_all(fd, out.data(), out.size());
}

bool recv_frame(int fd, Frame& f, int deadline_ms) {
    uint32_t count = 0;
    if (!read_all(fd, &f.op, 4, deadline_ms) || !read_all(fd, &f.number, 8, deadline_ms) || !read_all(fd, &count, 4, deadline_ms)) return false;
    if (count > 4096) return false;
    f.strings.clear();
    for (uint32_t k = 0; k < count; k++) {
        uint32_t len = 0;
        if (!read_all(fd, &len, 4, deadline_ms) || len > (64u << 20)) return false;
        std::string s(len, '\0');
        if (len && !read_all(fd, s.data(), len, deadline_ms)) return false;
        f.strings.push_back(std::move(s));
    }
    return true;
}

// Serves one connection until the client closes it. Waits (GET, WAIT) sleep on the table's condition variable up to
// the deadline the client sent (`number`, milliseconds).
void serve(int fd, std::shared_ptr<Table> table, std::shared_ptr<std::atomic<bool>> stop) {
    Frame req;
    while (!stop->load() && recv_frame(fd, req, -1)) {
        Frame reply;
        std::unique_lock<std::mutex> lock(table->mutex);
        auto have_all = [&](size_t from) {
            for (size_t k = from; k < req.strings.size(); k++)
                if (!table->values.count(req.strings[k])) return false;
            return true;
        };
        auto wait_keys = [&](size_t from) {
            auto until = Clock::now() + std::chrono::milliseconds(std::max<int64_t>(req.number, 0));
            while (!have_all(from)) {
                if (stop->load() || table->changed.wait_until(lock, until) == std::cv_status::timeout) return have_all(from);
            }
            return true;
        };
        switch (req.op) {
            case OP_SET:
                if (req.strings.size() == 2) {
                    table->values[req.strings[0]] = req.strings[1];
                    table->changed.notify_all();
                } else {
                    reply.op = 1;
                }
                break;
            case OP_GET:
                if (req.strings.size() == 1 && wait_keys(0)) reply.strings.push_back(table->values[req.strings[0]]);
                else reply.op = 1;
                break;
            case OP_ADD:
                if (req.strings.size() == 1) {
                    std::string& v = table->values[req.strings[0]];
                    long long current = 0;
                    try {
                        current = v.empty() ? 0 : std::stoll(v);
                    } catch (...) {
                        current = 0;
                    }
                    reply.number = current + req.number;
                    v = std::to_string(reply.number);
                    table->changed.notify_all();
                } else {
                    reply.op = 1;
                }
                break;
            case OP_WAIT: reply.op = wait_keys(0) ? 0 : 1; break;
            case OP_DELETE:
                reply.op = req.strings.size() == 1 && table->values.erase(req.strings[0]) ? 0 : 1;
                table->changed.notify_all();
                break;
            default: reply.op = 1;
        }
        lock.unlock();
        if (!send_frame(fd, reply)) break;
    }
    close(fd);
}

}  // namespace
}  // namespace lb

struct lb_store {
    int fd = -1;  // client connection
    int port = 0;
    int timeout_ms = 30000;
    std::mutex mutex;  // one request/reply exchange at a time
    // master only
    int listen_fd = -1;
    std::thread acceptor;
    std::shared_ptr<lb::Table> table;
    std::shared_ptr<std::atomic<bool>> stop;
};

namespace lb {
namespace {

void accept_loop(int listen_fd, std::shared_ptr<Table> table, std::shared_ptr<std::atomic<bool>> stop) {
    while (!stop->load()) {
        pollfd pfd{listen_fd, POLLIN, 0};
        int rc = poll(&pfd, 1, 100);
        if (rc <= 0) continue;
        int fd = accept(listen_fd, nullptr, nullptr);
        if (fd < 0) continue;
        int one = 1;
        setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
        std::thread(serve, fd, table, stop).detach();  // holds the table alive by its own reference
    }
}

Frame exchange(lb_store* s, const Frame& req, int wait_ms) {
    std::lock_guard<std::mutex> lock(s->mutex);
    if (s->fd < 0) fail(LB_ERR_INVALID, "store: not connected");
    Frame reply;
    // the server answers a wait at its deadline at the latest; allow the network a margin on top
    if (!send_frame(s->fd, req) || !recv_frame(s->fd, reply, wait_ms + 5000)) {
        close(s->fd);
        s->fd = -1;
        fail(LB_ERR_TIMEOUT, "store: the master did not answer (connection lost or deadline passed)");
    }
    return reply;
}

}  // namespace
}  // namespace lb

extern "C" {

void lb_store_destroy(lb_store* s) {
    if (!s) return;
    if (s->fd >= 0) close(s->fd);
    if (s->stop) {
        s->stop->store(true);
        if (s->table) s->table->changed.notify_all();
    }
    if (s->acceptor.joinable()) s->acceptor.join();
    if (s->listen_fd >= 0) close(s->listen_fd);
    delete s;
}

int lb_store_create(const char* host, int port, int is_master, int timeout_ms, lb_store** out) {
    return lb::guarded([&] {
        if (!host || !out || port < 0 || port > 65535) lb::fail(LB_ERR_INVALID, "lb_store_create: host, a port in 0..65535 and an out pointer");
        std::unique_ptr<lb_store, void (*)(lb_store*)> s(new lb_store, lb_store_destroy);
        s->timeout_ms = timeout_ms > 0 ? timeout_ms : 30000;
        s->port = port;
        if (is_master) {
            s->listen_fd = socket(AF_INET, SOCK_STREAM, 0);
            if (s->listen_fd < 0) lb::fail(LB_ERR_INVALID, "store: socket() failed");
            int one = 1;
            setsockopt(s->listen_fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
            sockaddr_in addr{};
            addr.sin_family = AF_INET;
            addr.sin_addr.s_addr = htonl(INADDR_ANY);
            addr.sin_port = htons((uint16_t)port);
            if (bind(s->listen_fd, (sockaddr*)&addr, sizeof(addr)) != 0 || listen(s->listen_fd, 128) != 0)
                lb::fail(LB_ERR_INVALID, lb::format("store: cannot listen on port %d: %s", port, strerror(errno)));
            socklen_t len = sizeof(addr);
            getsockname(s->listen_fd, (sockaddr*)&addr, &len);
            s->port = ntohs(addr.sin_port);
            s->table = std::make_shared<lb::Table>();
            s->stop = std::make_shared<std::atomic<bool>>(false);
            s->acceptor = std::thread(lb::accept_loop, s->listen_fd, s->table, s->stop);
        }
        // connect, retrying until the deadline so that workers may start before the master
        addrinfo hints{}, *res = nullptr;
        hints.ai_family = AF_INET, hints.ai_socktype = SOCK_STREAM;
        const std::string port_text = std::to_string(s->port);
        auto until = lb::Clock::now() + std::chrono::milliseconds(s->timeout_ms);
        for (;;) {
            if (getaddrinfo(is_master ? "127.0.0.1" : host, port_text.c_str(), &hints, &res) == 0 && res) {
                int fd = socket(res->ai_family, res->ai_socktype, res->ai_protocol);
                if (fd >= 0 && connect(fd, res->ai_addr, res->ai_addrlen) == 0) {
                    int one = 1;
                    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
                    s->fd = fd;
                    freeaddrinfo(res);
                    break;
                }
                if (fd >= 0) close(fd);
                freeaddrinfo(res);
                res = nullptr;
            }
            if (lb::Clock::now() >= until)
                lb::fail(LB_ERR_TIMEOUT, lb::format("store: no master at %s:%d within %d ms", host, s->port, s->timeout_ms));
            std::this_thread::sleep_for(std::chrono::milliseconds(10));
        }
        *out = s.release();
    });
}

int lb_store_port(const lb_store* s) { return s ? s->port : -1; }

int lb_store_set(lb_store* s, const char* key, const void* value, size_t n) {
    return lb::guarded([&] {
        if (!s || !key || (!value && n)) lb::fail(LB_ERR_INVALID, "lb_store_set: null argument");
        lb::Frame req;
        req.op = lb::OP_SET;
        req.strings = {key, std::string((const char*)value, n)};
        if (lb::exchange(s, req, 0).op != 0) lb::fail(LB_ERR_INVALID, "store: set was refused");
    });
}

int lb_store_get(lb_store* s, const char* key, void* out, size_t capacity, size_t* n, int timeout_ms) {
    return lb::guarded([&] {
        if (!s || !key || !n) lb::fail(LB_ERR_INVALID, "lb_store_get: null argument");
        const int wait_ms = timeout_ms > 0 ? timeout_ms : s->timeout_ms;
        lb::Frame req;
        req.op = lb::OP_GET, req.number = wait_ms, req.strings = {key};
        lb::Frame reply = lb::exchange(s, req, wait_ms);
        if (reply.op != 0 || reply.strings.size() != 1)
            lb::fail(LB_ERR_TIMEOUT, lb::format("store: key '%s' was not set within %d ms", key, wait_ms));
        *n = reply.strings[0].size();
        if (*n > capacity) lb::fail(LB_ERR_INVALID, lb::format("store: the value of '%s' has %zu bytes, the buffer %zu", key, *n, capacity));
        if (*n) memcpy(out, reply.strings[0].data(), *n);
    });
}

int lb_store_add(lb_store* s, const char* key, int64_t amount, int64_t* result) {
    return lb::guarded([&] {
        if (!s || !key) lb::fail(LB_ERR_INVALID, "lb_store_add: null argument");
        lb::Frame req;
        req.op = lb::OP_ADD, req.number = amount, req.strings = {key};
        lb::Frame reply = lb::exchange(s, req, 0);
        if (reply.op != 0) lb::fail(LB_ERR_INVALID, "store: add was refused");
        if (result) *result = reply.number;
    });
}

int lb_store_wait(lb_store* s, const char* const* keys, int n_keys, int timeout_ms) {
    return lb::guarded([&] {
        if (!s || (!keys && n_keys)) lb::fail(LB_ERR_INVALID, "lb_store_wait: null argument");
        const int wait_ms = timeout_ms > 0 ? timeout_ms : s->timeout_ms;
        lb::Frame req;
        req.op = lb::OP_WAIT, req.number = wait_ms;
        for (int k = 0; k < n_keys; k++) req.strings.push_back(keys[k]);
        if (lb::exchange(s, req, wait_ms).op != 0) {
            std::string names;
            for (auto& k : req.strings) names += (names.empty() ? "" : ", ") + k;
            lb::fail(LB_ERR_TIMEOUT, lb::format("store: keys [%s] were not all set within %d ms", names.c_str(), wait_ms));
        }
    });
}

int lb_store_delete(lb_store* s, const char* key) {
    return lb::guarded([&] {
        if (!s || !key) lb::fail(LB_ERR_INVALID, "lb_store_delete: null argument");
        lb::Frame req;
        req.op = lb::OP_DELETE, req.strings = {key};
        lb::exchange(s, req, 0);
    });
}
}
