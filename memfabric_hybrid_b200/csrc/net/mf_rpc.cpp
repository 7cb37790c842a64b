#include "mf_rpc.h"

#include <arpa/inet.h>
#include <fcntl.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/epoll.h>
#include <sys/eventfd.h>
#include <sys/socket.h>
#include <unistd.h>

namespace mf {
namespace net {

namespace {
void TuneSocket(int fd)
{
    int one = 1;
    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    setsockopt(fd, SOL_SOCKET, SO_KEEPALIVE, &one, sizeof(one));
    int idle = 32, cnt = 7, intvl = 2;
    setsockopt(fd, IPPROTO_TCP, TCP_KEEPIDLE, &idle, sizeof(idle));
    setsockopt(fd, IPPROTO_TCP, TCP_KEEPCNT, &cnt, sizeof(cnt));
    setsockopt(fd, IPPROTO_TCP, TCP_KEEPINTVL, &intvl, sizeof(intvl));
    struct timeval tv = {30, 0};  // a peer that stops reading cannot wedge a sender forever
    setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof(tv));
}

bool WriteAll(int fd, const void *buf, size_t len)
{
    const char *p = static_cast<const char *>(buf);
    while (len > 0) {
        ssize_t n = ::send(fd, p, len, MSG_NOSIGNAL);
        if (n < 0) {
            if (errno == EINTR) continue;
            return false;
        }
        p += n;
        len -= (size_t)n;
    }
    return true;
}

bool ReadAllTimed(int fd, void *buf, size_t len, uint32_t timeoutMs)
{
    char *p = static_cast<char *>(buf);
    uint64_t deadline = NowMs() + timeoutMs;
    while (len > 0) {
        uint64_t now = NowMs();
        if (now >= deadline) return false;
        struct pollfd pfd = {fd, POLLIN, 0};
        int pr = poll(&pfd, 1, (int)(deadline - now));
        if (pr < 0 && errno == EINTR) continue;
        if (pr <= 0) return false;
        ssize_t n = ::recv(fd, p, len, 0);
        if (n == 0) return false;
        if (n < 0) {
            if (errno == EINTR || errno == EAGAIN) continue;
            return false;
        }
        p += n;
        len -= (size_t)n;
    }
    return true;
}

bool MakeAddr(const std::string &ip, uint16_t port, sockaddr_in &sa)
{
    memset(&sa, 0, sizeof(sa));
    sa.sin_family = AF_INET;
    sa.sin_port = htons(port);
    std::string host = (ip.empty() || ip == "localhost") ? "127.0.0.1" : ip;
    return inet_pton(AF_INET, host.c_str(), &sa.sin_addr) == 1;
}
}  // namespace

Link::~Link()
{
    tls_.reset();  // close_notify goes out while the socket is still open
    if (fd_ >= 0) ::close(fd_);
}

bool Link::WriteRaw(const void *buf, size_t len) { return tls_ ? tls_->WriteAll(buf, len) : WriteAll(fd_, buf, len); }
bool Link::ReadRawTimed(void *buf, size_t len, uint32_t timeoutMs)
{
    return tls_ ? tls_->ReadAll(buf, len, timeoutMs) : ReadAllTimed(fd_, buf, len, timeoutMs);
}

int Link::Send(int16_t type, int16_t result, uint32_t seqNo, const void *body, uint32_t len)
{
    if (closed_.load()) return ERR_NOT_CONNECTED;
    MsgHeader h;
    h.type = type;
    h.result = result;
    h.bodyLen = len;
    h.seqNo = seqNo;
    h.crc = 0;
    std::lock_guard<std::mutex> g(sendMu_);
    if (len <= 1024) {  // one syscall for small frames
        char tmp[sizeof(MsgHeader) + 1024];
        memcpy(tmp, &h, sizeof(h));
        if (len > 0) memcpy(tmp + sizeof(h), body, len);
        if (!WriteRaw(tmp, sizeof(h) + len)) {
            Shutdown();
            return ERR_NOT_CONNECTED;
        }
        return OK;
    }
    if (!WriteRaw(&h, sizeof(h)) || !WriteRaw(body, len)) {
        Shutdown();
        return ERR_NOT_CONNECTED;
    }
    return OK;
}

void Link::Shutdown()
{
    if (!closed_.exchange(true)) ::shutdown(fd_, SHUT_RDWR);
}

Endpoint::Endpoint(const EndpointOptions &opt) : opt_(opt) {}
Endpoint::~Endpoint() { Stop(); }

int Endpoint::Start()
{
    if (running_.exchange(true)) return OK;
    uint16_t n = opt_.workers == 0 ? 1 : opt_.workers;
    for (uint16_t i = 0; i < n; i++) {
        auto w = std::make_unique<Worker>();
        w->epfd = epoll_create1(EPOLL_CLOEXEC);
        w->wakefd = eventfd(0, EFD_NONBLOCK | EFD_CLOEXEC);
        if (w->epfd < 0 || w->wakefd < 0) return MF_FAIL(ERR_NO_RESOURCES, "epoll/eventfd create failed: %s", strerror(errno));
        struct epoll_event ev = {};
        ev.events = EPOLLIN;
        ev.data.fd = w->wakefd;
        epoll_ctl(w->epfd, EPOLL_CTL_ADD, w->wakefd, &ev);
        Worker *raw = w.get();
        w->th = std::thread([this, raw, i] {
            char nm[16];
            snprintf(nm, sizeof(nm), "mf-rpc-%u", i);
            pthread_setname_np(pthread_self(), nm);
            WorkerLoop(raw);
        });
        workers_.push_back(std::move(w));
    }
    return OK;
}

int Endpoint::Listen(const std::string &ip, uint16_t port)
{
    if (!running_) return ERR_NOT_STARTED;
    sockaddr_in sa;
    if (!MakeAddr(ip, port, sa)) return MF_FAIL(ERR_INVALID_PARAM, "bad listen address %s", ip.c_str());
    int fd = socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (fd < 0) return MF_FAIL(ERR_NO_RESOURCES, "socket failed: %s", strerror(errno));
    int one = 1;
    setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    if (opt_.reusePort) setsockopt(fd, SOL_SOCKET, SO_REUSEPORT, &one, sizeof(one));
    if (bind(fd, (sockaddr *)&sa, sizeof(sa)) != 0) {
        int e = errno;
        ::close(fd);
        LastError::Set(e == EADDRINUSE ? ERR_IN_USE : ERR, "bind %s:%u failed: %s", ip.c_str(), port, strerror(e));
        return e == EADDRINUSE ? ERR_IN_USE : ERR;
    }
    if (listen(fd, 512) != 0) {
        ::close(fd);
        return MF_FAIL(ERR, "listen failed: %s", strerror(errno));
    }
    socklen_t sl = sizeof(sa);
    getsockname(fd, (sockaddr *)&sa, &sl);
    listenPort_ = ntohs(sa.sin_port);
    listenFd_ = fd;
    acceptor_ = std::thread([this] {
        pthread_setname_np(pthread_self(), "mf-rpc-accept");
        AcceptLoop();
    });
    return OK;
}

void Endpoint::AcceptLoop()
{
    while (running_) {
        struct pollfd pfd = {listenFd_, POLLIN, 0};
        int pr = poll(&pfd, 1, 200);
        if (pr <= 0) continue;
        int fd = accept4(listenFd_, nullptr, nullptr, SOCK_CLOEXEC);
        if (fd < 0) continue;
        TuneSocket(fd);
        if (!opt_.tls) {
            Admit(fd);
            continue;
        }
        // TLS: the handshake (several round trips, up to 5 s for a slow or silent peer) runs beside the accept loop, so that
        // one stalled client cannot hold up the others; at most kMaxHandshakes at a time
        {
            std::unique_lock<std::mutex> g(hsMu_);
            if (handshakes_ >= kMaxHandshakes) {
                g.unlock();
                ::close(fd);
                MF_WARN("refused a connection: %u TLS handshakes are already in progress", kMaxHandshakes);
                continue;
            }
            handshakes_++;
        }
        std::thread([this, fd] {
            pthread_setname_np(pthread_self(), "mf-rpc-tls");
            Admit(fd);
            std::lock_guard<std::mutex> g(hsMu_);
            handshakes_--;
            hsCv_.notify_all();
        }).detach();
    }
    // no admission thread may outlive the endpoint
    std::unique_lock<std::mutex> g(hsMu_);
    hsCv_.wait(g, [this] { return handshakes_ == 0; });
}

// Handshake (TLS when configured), admission request / reply, hand-over to a worker. Owns fd until a Link does.
void Endpoint::Admit(int fd)
{
    std::unique_ptr<TlsSession> session;
    if (opt_.tls) {
        std::string why;
        session = opt_.tls->Handshake(fd, true, 5000, why);
        if (!session) {
            MF_WARN("refused a connection: %s", why.c_str());
            ::close(fd);
            return;
        }
    }
    ConnReq req;
    if (!(session ? session->ReadAll(&req, sizeof(req), 5000) : ReadAllTimed(fd, &req, sizeof(req), 5000))) {
        session.reset();
        ::close(fd);
        return;
    }
    ConnResp resp;
    auto link = std::make_shared<Link>(fd, nextLinkId_.fetch_add(1), req.rankId, true);
    link->tls_ = std::move(session);
    link->lastSeenMs = NowMs();
    if (!running_) return;  // the endpoint is stopping: the link's destructor closes the socket
    if (req.magic != opt_.magic || req.version != opt_.version) {
        resp.result = -1;
    } else if (newLink_) {
        resp.result = (int16_t)newLink_(req, link);
    }
    if (!link->WriteRaw(&resp, sizeof(resp)) || resp.result != 0) {
        link->closed_ = true;
        if (resp.result == 0 && broken_) broken_(link);  // admitted but the peer vanished
        return;  // link destructor closes fd
    }
    Attach(link);
}

void Endpoint::Attach(const LinkPtr &l)
{
    Worker *w = workers_[rr_.fetch_add(1) % workers_.size()].get();
    {
        std::lock_guard<std::mutex> g(w->mu);
        w->links[l->fd_] = l;
    }
    struct epoll_event ev = {};
    ev.events = EPOLLIN | EPOLLRDHUP;
    ev.data.fd = l->fd_;
    epoll_ctl(w->epfd, EPOLL_CTL_ADD, l->fd_, &ev);
}

int Endpoint::Connect(const std::string &ip, uint16_t port, const ConnReq &req, uint32_t timeoutMs, LinkPtr &out,
                      int16_t *refused)
{
    if (!running_) return ERR_NOT_STARTED;
    sockaddr_in sa;
    if (!MakeAddr(ip, port, sa)) return MF_FAIL(ERR_INVALID_PARAM, "bad address %s", ip.c_str());
    int fd = socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (fd < 0) return ERR_NO_RESOURCES;
    int fl = fcntl(fd, F_GETFL, 0);
    fcntl(fd, F_SETFL, fl | O_NONBLOCK);
    int rc = ::connect(fd, (sockaddr *)&sa, sizeof(sa));
    if (rc != 0 && errno != EINPROGRESS) {
        ::close(fd);
        return ERR_NOT_CONNECTED;
    }
    if (rc != 0) {
        struct pollfd pfd = {fd, POLLOUT, 0};
        int pr = poll(&pfd, 1, (int)timeoutMs);
        int err = 0;
        socklen_t el = sizeof(err);
        getsockopt(fd, SOL_SOCKET, SO_ERROR, &err, &el);
        if (pr <= 0 || err != 0) {
            ::close(fd);
            return ERR_NOT_CONNECTED;
        }
    }
    fcntl(fd, F_SETFL, fl);
    TuneSocket(fd);
    ConnReq r = req;
    r.magic = opt_.magic;
    r.version = opt_.version;
    ConnResp resp;
    std::unique_ptr<TlsSession> session;
    if (opt_.tls) {
        std::string why;
        session = opt_.tls->Handshake(fd, false, timeoutMs == 0 ? 5000 : timeoutMs, why);
        if (!session) {
            ::close(fd);
            return MF_FAIL(ERR_NOT_CONNECTED, "TLS to %s:%u: %s", ip.c_str(), (unsigned)port, why.c_str());
        }
    }
    const uint32_t respMs = timeoutMs == 0 ? 5000 : timeoutMs;
    const bool sent = session ? session->WriteAll(&r, sizeof(r)) : WriteAll(fd, &r, sizeof(r));
    if (!sent || !(session ? session->ReadAll(&resp, sizeof(resp), respMs) : ReadAllTimed(fd, &resp, sizeof(resp), respMs))) {
        session.reset();
        ::close(fd);
        return ERR_NOT_CONNECTED;
    }
    if (resp.result != 0) {
        session.reset();
        ::close(fd);
        if (refused != nullptr) *refused = resp.result;
        return ERR_RECONNECT;
    }
    out = std::make_shared<Link>(fd, nextLinkId_.fetch_add(1), req.rankId, false);
    out->tls_ = std::move(session);
    out->lastSeenMs = NowMs();
    Attach(out);
    return OK;
}

bool Endpoint::Drain(Worker *, const LinkPtr &l)
{
    for (;;) {
        if (l->in_.size() - l->inUsed_ < 65536) l->in_.resize(std::max<size_t>(l->in_.size() * 2, 131072));
        ssize_t n;
        if (l->tls_) {
            n = l->tls_->ReadSome(l->in_.data() + l->inUsed_, l->in_.size() - l->inUsed_);
            if (n == 0) break;  // everything the socket and the TLS layer held has been taken
            if (n < 0) return false;
        } else {
            n = ::recv(l->fd_, l->in_.data() + l->inUsed_, l->in_.size() - l->inUsed_, MSG_DONTWAIT);
            if (n == 0) return false;
            if (n < 0) {
                if (errno == EINTR) continue;
                if (errno == EAGAIN || errno == EWOULDBLOCK) break;
                return false;
            }
        }
        l->inUsed_ += (size_t)n;
        l->lastSeenMs.store(NowMs(), std::memory_order_relaxed);
        size_t off = 0;
        while (l->inUsed_ - off >= sizeof(MsgHeader)) {
            MsgHeader h;
            memcpy(&h, l->in_.data() + off, sizeof(h));
            if (h.bodyLen > kMaxBodyLen) {
                MF_WARN("link %lu: frame of %u bytes exceeds the limit, closing", (unsigned long)l->id_, h.bodyLen);
                return false;
            }
            size_t need = sizeof(h) + h.bodyLen;
            if (l->in_.size() < need) l->in_.resize(need + 65536);
            if (l->inUsed_ - off < need) break;
            std::string body(reinterpret_cast<char *>(l->in_.data() + off + sizeof(h)), h.bodyLen);
            off += need;
            if (msg_) msg_(l, h, body);
        }
        if (off > 0) {
            memmove(l->in_.data(), l->in_.data() + off, l->inUsed_ - off);
            l->inUsed_ -= off;
        }
        if (l->in_.size() > (4u << 20) && l->inUsed_ < 65536) {
            l->in_.resize(131072);
            l->in_.shrink_to_fit();
        }
    }
    return !l->closed_.load();
}

void Endpoint::Drop(Worker *w, const LinkPtr &l)
{
    epoll_ctl(w->epfd, EPOLL_CTL_DEL, l->fd_, nullptr);
    {
        std::lock_guard<std::mutex> g(w->mu);
        w->links.erase(l->fd_);
    }
    l->closed_ = true;
    ::shutdown(l->fd_, SHUT_RDWR);
    if (broken_ && running_) broken_(l);
}

void Endpoint::WorkerLoop(Worker *w)
{
    struct epoll_event evs[64];
    while (running_) {
        int n = epoll_wait(w->epfd, evs, 64, (int)opt_.pollMs);
        if (n < 0) {
            if (errno == EINTR) continue;
            break;
        }
        for (int i = 0; i < n; i++) {
            int fd = evs[i].data.fd;
            if (fd == w->wakefd) {
                uint64_t v;
                (void)!::read(w->wakefd, &v, sizeof(v));
                continue;
            }
            LinkPtr l;
            {
                std::lock_guard<std::mutex> g(w->mu);
                auto it = w->links.find(fd);
                if (it != w->links.end()) l = it->second;
            }
            if (!l) continue;
            bool ok = true;
            if (evs[i].events & EPOLLIN) ok = Drain(w, l);
            if (ok && (evs[i].events & (EPOLLERR | EPOLLHUP | EPOLLRDHUP))) ok = false;
            if (!ok) Drop(w, l);
        }
    }
}

void Endpoint::Stop()
{
    if (!running_.exchange(false)) return;
    JoinOrDetach(acceptor_);
    if (listenFd_ >= 0) {
        ::close(listenFd_);
        listenFd_ = -1;
    }
    for (auto &w : workers_) {
        uint64_t one = 1;
        (void)!::write(w->wakefd, &one, sizeof(one));
    }
    for (auto &w : workers_) {
        JoinOrDetach(w->th);
        std::unordered_map<int, LinkPtr> links;
        {
            std::lock_guard<std::mutex> g(w->mu);
            links.swap(w->links);
        }
        for (auto &kv : links) {
            kv.second->closed_ = true;
            ::shutdown(kv.second->fd_, SHUT_RDWR);
        }
        ::close(w->epfd);
        ::close(w->wakefd);
    }
    workers_.clear();
}

size_t Endpoint::LinkCount()
{
    size_t n = 0;
    for (auto &w : workers_) {
        std::lock_guard<std::mutex> g(w->mu);
        n += w->links.size();
    }
    return n;
}

bool ParseIpPort(const std::string &s, std::string &ip, uint16_t &port)
{
    std::string t = s;
    size_t p = t.find("://");
    if (p != std::string::npos) t = t.substr(p + 3);
    p = t.find('#');
    if (p != std::string::npos) t = t.substr(0, p);
    p = t.rfind(':');
    if (p == std::string::npos || p == 0 || p + 1 >= t.size()) return false;
    ip = t.substr(0, p);
    uint64_t v = 0;
    if (!ParseU64(t.substr(p + 1), v) || v == 0 || v > 65535) return false;
    port = (uint16_t)v;
    return true;
}

uint16_t FindFreePort(const std::string &ip, uint16_t from, uint16_t span)
{
    for (uint32_t p = from; p < (uint32_t)from + span && p <= 65535; p++) {
        sockaddr_in sa;
        if (!MakeAddr(ip, (uint16_t)p, sa)) return 0;
        int fd = socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
        if (fd < 0) return 0;
        int one = 1;
        setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
        int rc = bind(fd, (sockaddr *)&sa, sizeof(sa));
        ::close(fd);
        if (rc == 0) return (uint16_t)p;
    }
    return 0;
}

bool ProbeReachable(const std::string &ip, uint16_t port, uint32_t timeoutMs)
{
    sockaddr_in sa;
    if (!MakeAddr(ip, port, sa)) return false;
    int fd = socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC | SOCK_NONBLOCK, 0);
    if (fd < 0) return false;
    bool ok = false;
    int rc = ::connect(fd, (sockaddr *)&sa, sizeof(sa));
    if (rc == 0) {
        ok = true;
    } else if (errno == EINPROGRESS) {
        struct pollfd pfd = {fd, POLLOUT, 0};
        if (poll(&pfd, 1, (int)timeoutMs) > 0) {
            int err = 0;
            socklen_t el = sizeof(err);
            getsockopt(fd, SOL_SOCKET, SO_ERROR, &err, &el);
            ok = err == 0;
        }
    }
    ::close(fd);
    return ok;
}

}  // namespace net
}  // namespace mf
