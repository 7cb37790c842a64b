// Framed TCP RPC used by the config store: one Endpoint owns epoll worker threads, an optional
// listener and any number of links (accepted or dialled). The wire format is byte-compatible with
// the reference's acc_links layer so either side can be the reference implementation:
//   handshake  client -> server : ConnReq  (16 bytes)   server -> client : ConnResp (2 bytes)
//   frames     MsgHeader (16 bytes) + bodyLen bytes
// All integers are host-endian raw structs.
// Parity: src/acc_links/include/acc_def.h:45-115, src/acc_links/include/acc_tcp_server.h:64-166,
// src/acc_links/csrc/acc_tcp_listener.cpp:189-240, src/acc_links/csrc/acc_tcp_worker.cpp.
#pragma once
#include <condition_variable>
#include <map>
#include <unordered_map>

#include "mf_tls.h"

#include "../util/mf_util.h"

namespace mf {
namespace net {

#pragma pack(push, 1)
struct ConnReq {
    int16_t magic = 0;
    int16_t version = 0;
    int8_t reconnect = 0;
    int8_t reserved[3] = {0, 0, 0};
    uint64_t rankId = 0;  // (worldSize << 32) | rank ; rank 0xFFFFFFFF = "assign me one"
};
struct ConnResp {
    int16_t result = 0;
};
struct MsgHeader {
    int16_t type = 0;
    int16_t result = 0;
    uint32_t bodyLen = 0;
    uint32_t seqNo = 0;
    uint32_t crc = 0;
};
#pragma pack(pop)
static_assert(sizeof(ConnReq) == 16, "handshake must be 16 bytes");
static_assert(sizeof(ConnResp) == 2, "handshake reply must be 2 bytes");
static_assert(sizeof(MsgHeader) == 16, "frame header must be 16 bytes");

constexpr uint32_t kMaxBodyLen = 80u << 20;  // a store value may be 64 MiB plus framing

class Endpoint;

class Link : public std::enable_shared_from_this<Link> {
public:
    Link(int fd, uint64_t id, uint64_t peerTag, bool accepted) : fd_(fd), id_(id), peerTag_(peerTag), accepted_(accepted) {}
    ~Link();
    uint64_t Id() const { return id_; }
    uint64_t PeerTag() const { return peerTag_; }  // ConnReq.rankId seen (server side) or sent (client side)
    bool Accepted() const { return accepted_; }
    bool Alive() const { return !closed_.load(); }
    // Sends one frame; thread-safe. Returns OK or ERR_NOT_CONNECTED.
    int Send(int16_t type, int16_t result, uint32_t seqNo, const void *body, uint32_t len);
    void Shutdown();  // wakes the worker which then reports the link as broken
    std::atomic<void *> userData{nullptr};  // set by a handler thread, read by timers
    std::atomic<uint64_t> lastSeenMs{0};

private:
    friend class Endpoint;
    bool WriteRaw(const void *buf, size_t len);                   // through TLS when the link has a session
    bool ReadRawTimed(void *buf, size_t len, uint32_t timeoutMs);
    int fd_;
    std::unique_ptr<TlsSession> tls_;  // set once, before the link is shared between threads
    uint64_t id_;
    uint64_t peerTag_;
    bool accepted_;
    std::atomic<bool> closed_{false};
    std::mutex sendMu_;
    // input state (touched only by the owning worker thread)
    std::vector<uint8_t> in_;
    size_t inUsed_ = 0;
};
using LinkPtr = std::shared_ptr<Link>;

struct EndpointOptions {
    uint16_t workers = 2;
    int16_t magic = 0;
    int16_t version = 0;
    uint32_t pollMs = 500;
    bool reusePort = false;
    std::shared_ptr<TlsContext> tls;  // set: every link is TLS 1.3 with mutual certificate verification
};

class Endpoint {
public:
    // Return 0 to admit the link, non-zero to refuse (sent back in ConnResp.result).
    using NewLinkFn = std::function<int(const ConnReq &, const LinkPtr &)>;
    using MsgFn = std::function<void(const LinkPtr &, const MsgHeader &, std::string &body)>;
    using BrokenFn = std::function<void(const LinkPtr &)>;

    explicit Endpoint(const EndpointOptions &opt = EndpointOptions());
    ~Endpoint();

    void OnNewLink(NewLinkFn f) { newLink_ = std::move(f); }
    void OnMessage(MsgFn f) { msg_ = std::move(f); }
    void OnBroken(BrokenFn f) { broken_ = std::move(f); }

    int Start();                                       // workers only
    int Listen(const std::string &ip, uint16_t port);  // Start() must have been called
    uint16_t ListenPort() const { return listenPort_; }
    // Dial + handshake. result receives ConnResp.result when the server refuses.
    int Connect(const std::string &ip, uint16_t port, const ConnReq &req, uint32_t timeoutMs, LinkPtr &out,
                int16_t *refused = nullptr);
    void Stop();
    size_t LinkCount();

private:
    struct Worker {
        int epfd = -1;
        int wakefd = -1;
        std::thread th;
        std::mutex mu;
        std::unordered_map<int, LinkPtr> links;
    };
    void WorkerLoop(Worker *w);
    void AcceptLoop();
    void Admit(int fd);
    void Attach(const LinkPtr &l);
    bool Drain(Worker *w, const LinkPtr &l);  // false => link finished
    void Drop(Worker *w, const LinkPtr &l);

    EndpointOptions opt_;
    NewLinkFn newLink_;
    MsgFn msg_;
    BrokenFn broken_;
    std::vector<std::unique_ptr<Worker>> workers_;
    std::thread acceptor_;
    static constexpr uint32_t kMaxHandshakes = 64;
    std::mutex hsMu_;
    std::condition_variable hsCv_;
    uint32_t handshakes_ = 0;  // TLS admissions in flight (their threads are detached; the accept loop waits for them before it ends)
    int listenFd_ = -1;
    uint16_t listenPort_ = 0;
    std::atomic<bool> running_{false};
    std::atomic<uint64_t> nextLinkId_{1};
    std::atomic<uint32_t> rr_{0};
};

// "ip:port" / "tcp://ip:port" helpers. Returns false on malformed input.
bool ParseIpPort(const std::string &s, std::string &ip, uint16_t &port);
// Finds a TCP port that can be bound on `ip`, scanning upward from `from`. Returns 0 when none.
uint16_t FindFreePort(const std::string &ip, uint16_t from, uint16_t span = 200);
// True when a TCP connect to ip:port succeeds within timeoutMs.
bool ProbeReachable(const std::string &ip, uint16_t port, uint32_t timeoutMs);

}  // namespace net
}  // namespace mf
