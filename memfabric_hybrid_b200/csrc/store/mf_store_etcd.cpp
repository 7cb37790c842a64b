#include "mf_store_etcd.h"

#include <arpa/inet.h>
#include <errno.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <cstring>

namespace mf {
namespace store {

namespace {

constexpr int64_t kLockTtlSec = 10;
constexpr uint32_t kLockWaitMs = 30000;
constexpr const char *kClusterRoot = "/memfabric_hybrid/config_store/clusters/";

// ---- base64 (the gateway carries keys and values as base64 strings) ----------------------------------
const char kB64[] = "ABCDEFGHIJKLMNOPQRSTUVWXYZabcdefghijklmnopqrstuvwxyz0123456789+/";

std::string B64Encode(const std::string &in)
{
    std::string out;
    out.reserve((in.size() + 2) / 3 * 4);
    size_t i = 0;
    for (; i + 2 < in.size(); i += 3) {
        uint32_t v = ((uint8_t)in[i] << 16) | ((uint8_t)in[i + 1] << 8) | (uint8_t)in[i + 2];
        out += kB64[v >> 18];
        out += kB64[(v >> 12) & 63];
        out += kB64[(v >> 6) & 63];
        out += kB64[v & 63];
    }
    if (i + 1 == in.size()) {
        uint32_t v = (uint8_t)in[i] << 16;
        out += kB64[v >> 18];
        out += kB64[(v >> 12) & 63];
        out += "==";
    } else if (i + 2 == in.size()) {
        uint32_t v = ((uint8_t)in[i] << 16) | ((uint8_t)in[i + 1] << 8);
        out += kB64[v >> 18];
        out += kB64[(v >> 12) & 63];
        out += kB64[(v >> 6) & 63];
        out += '=';
    }
    return out;
}

bool B64Decode(const std::string &in, std::string &out)
{
    static int8_t table[256];
    static bool ready = [] {
        memset(table, -1, sizeof(table));
        for (int i = 0; i < 64; i++) table[(uint8_t)kB64[i]] = (int8_t)i;
        table[(uint8_t)'-'] = 62;  // the URL-safe alphabet is accepted as well
        table[(uint8_t)'_'] = 63;
        return true;
    }();
    (void)ready;
    out.clear();
    uint32_t acc = 0;
    int bits = 0;
    for (char c : in) {
        if (c == '=' || c == '\n' || c == '\r') continue;
        int8_t v = table[(uint8_t)c];
        if (v < 0) return false;
        acc = (acc << 6) | (uint32_t)v;
        bits += 6;
        if (bits >= 8) {
            bits -= 8;
            out += (char)((acc >> bits) & 0xff);
        }
    }
    return true;
}

// ---- a JSON reader for the gateway's replies ---------------------------------------------------------
struct Json {
    enum Kind { NUL, BOOL, NUM, STR, ARR, OBJ } kind = NUL;
    bool b = false;
    std::string s;  // STR: the text; NUM: the digits as written (64-bit ids do not fit a double)
    std::vector<Json> arr;
    std::vector<std::pair<std::string, Json>> obj;

    const Json *Find(const char *name) const
    {
        if (kind != OBJ) return nullptr;
        for (auto &kv : obj)
            if (kv.first == name) return &kv.second;
        return nullptr;
    }
    // int64 fields arrive as strings ("ID":"7587862...") from the gateway and as numbers from some proxies
    int64_t Int(const char *name, int64_t dflt = 0) const
    {
        const Json *j = Find(name);
        if (j == nullptr || (j->kind != STR && j->kind != NUM) || j->s.empty()) return dflt;
        return strtoll(j->s.c_str(), nullptr, 10);
    }
    std::string Str(const char *name) const
    {
        const Json *j = Find(name);
        return j != nullptr && j->kind == STR ? j->s : std::string();
    }
    bool Bool(const char *name) const
    {
        const Json *j = Find(name);
        return j != nullptr && j->kind == BOOL && j->b;
    }
};

class JsonParser {
public:
    explicit JsonParser(const std::string &t) : t_(t) {}
    bool Parse(Json &out)
    {
        bool ok = Value(out, 0);
        Skip();
        return ok;
    }

private:
    void Skip()
    {
        while (p_ < t_.size() && (t_[p_] == ' ' || t_[p_] == '\n' || t_[p_] == '\r' || t_[p_] == '\t')) p_++;
    }
    bool Lit(const char *w)
    {
        size_t n = strlen(w);
        if (t_.compare(p_, n, w) != 0) return false;
        p_ += n;
        return true;
    }
    bool String(std::string &out)
    {
        if (p_ >= t_.size() || t_[p_] != '"') return false;
        p_++;
        out.clear();
        while (p_ < t_.size() && t_[p_] != '"') {
            char c = t_[p_++];
            if (c != '\\') {
                out += c;
                continue;
            }
            if (p_ >= t_.size()) return false;
            char e = t_[p_++];
            switch (e) {
                case 'n': out += '\n'; break;
                case 't': out += '\t'; break;
                case 'r': out += '\r'; break;
                case 'b': out += '\b'; break;
                case 'f': out += '\f'; break;
                case 'u': {
                    if (p_ + 4 > t_.size()) return false;
                    unsigned cp = (unsigned)strtoul(t_.substr(p_, 4).c_str(), nullptr, 16);
                    p_ += 4;
                    if (cp < 0x80) out += (char)cp;
                    else if (cp < 0x800) {
                        out += (char)(0xc0 | (cp >> 6));
                        out += (char)(0x80 | (cp & 0x3f));
                    } else {
                        out += (char)(0xe0 | (cp >> 12));
                        out += (char)(0x80 | ((cp >> 6) & 0x3f));
                        out += (char)(0x80 | (cp & 0x3f));
                    }
                    break;
                }
                default: out += e;  // \" \\ \/
            }
        }
        if (p_ >= t_.size()) return false;
        p_++;
        return true;
    }
    bool Value(Json &out, int depth)
    {
        if (depth > 32) return false;
        Skip();
        if (p_ >= t_.size()) return false;
        char c = t_[p_];
        if (c == '{') {
            out.kind = Json::OBJ;
            p_++;
            Skip();
            if (p_ < t_.size() && t_[p_] == '}') {
                p_++;
                return true;
            }
            while (true) {
                Skip();
                std::string k;
                if (!String(k)) return false;
                Skip();
                if (p_ >= t_.size() || t_[p_++] != ':') return false;
                Json v;
                if (!Value(v, depth + 1)) return false;
                out.obj.emplace_back(std::move(k), std::move(v));
                Skip();
                if (p_ >= t_.size()) return false;
                if (t_[p_] == ',') {
                    p_++;
                    continue;
                }
                if (t_[p_] == '}') {
                    p_++;
                    return true;
                }
                return false;
            }
        }
        if (c == '[') {
            out.kind = Json::ARR;
            p_++;
            Skip();
            if (p_ < t_.size() && t_[p_] == ']') {
                p_++;
                return true;
            }
            while (true) {
                Json v;
                if (!Value(v, depth + 1)) return false;
                out.arr.push_back(std::move(v));
                Skip();
                if (p_ >= t_.size()) return false;
                if (t_[p_] == ',') {
                    p_++;
                    continue;
                }
                if (t_[p_] == ']') {
                    p_++;
                    return true;
                }
                return false;
            }
        }
        if (c == '"') {
            out.kind = Json::STR;
            return String(out.s);
        }
        if (c == 't' || c == 'f') {
            out.kind = Json::BOOL;
            out.b = c == 't';
            return Lit(c == 't' ? "true" : "false");
        }
        if (c == 'n') return Lit("null");
        size_t b = p_;
        while (p_ < t_.size() && (isdigit((unsigned char)t_[p_]) || strchr("+-.eE", t_[p_]) != nullptr)) p_++;
        if (p_ == b) return false;
        out.kind = Json::NUM;
        out.s = t_.substr(b, p_ - b);
        return true;
    }
    const std::string &t_;
    size_t p_ = 0;
};

std::string Quoted(const std::string &s)
{
    std::string o = "\"";
    for (char c : s) {
        if (c == '"' || c == '\\') {
            o += '\\';
            o += c;
        } else if ((unsigned char)c < 0x20) {
            char buf[8];
            snprintf(buf, sizeof(buf), "\\u%04x", c);
            o += buf;
        } else {
            o += c;
        }
    }
    return o + "\"";
}

// The smallest key greater than every key that starts with `prefix` ("\0" = to the end of the key space).
std::string RangeEnd(const std::string &prefix)
{
    std::string e = prefix;
    while (!e.empty()) {
        if ((uint8_t)e.back() != 0xff) {
            e.back() = (char)((uint8_t)e.back() + 1);
            return e;
        }
        e.pop_back();
    }
    return std::string(1, '\0');
}

// ---- one HTTP/1.1 POST on a fresh connection ----------------------------------------------------------
int DialTimed(const std::string &ip, uint16_t port, uint32_t timeoutMs)
{
    sockaddr_in sa;
    memset(&sa, 0, sizeof(sa));
    sa.sin_family = AF_INET;
    sa.sin_port = htons(port);
    if (inet_pton(AF_INET, ip.c_str(), &sa.sin_addr) != 1) return -1;
    int fd = socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC | SOCK_NONBLOCK, 0);
    if (fd < 0) return -1;
    int rc = ::connect(fd, (sockaddr *)&sa, sizeof(sa));
    if (rc != 0 && errno != EINPROGRESS) {
        ::close(fd);
        return -1;
    }
    if (rc != 0) {
        struct pollfd pfd = {fd, POLLOUT, 0};
        int err = 0;
        socklen_t el = sizeof(err);
        if (poll(&pfd, 1, (int)timeoutMs) <= 0 || getsockopt(fd, SOL_SOCKET, SO_ERROR, &err, &el) != 0 || err != 0) {
            ::close(fd);
            return -1;
        }
    }
    int one = 1;
    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    return fd;
}

bool SendAllTimed(int fd, const std::string &data, uint64_t deadlineMs)
{
    size_t off = 0;
    while (off < data.size()) {
        ssize_t n = ::send(fd, data.data() + off, data.size() - off, MSG_NOSIGNAL);
        if (n > 0) {
            off += (size_t)n;
            continue;
        }
        if (n < 0 && errno == EINTR) continue;
        if (n < 0 && (errno == EAGAIN || errno == EWOULDBLOCK)) {
            uint64_t now = NowMs();
            if (now >= deadlineMs) return false;
            struct pollfd pfd = {fd, POLLOUT, 0};
            poll(&pfd, 1, (int)(deadlineMs - now));
            continue;
        }
        return false;
    }
    return true;
}

// Reads until the peer closes (the request says "Connection: close") or the reply is complete by its own framing.
bool ReadReply(int fd, uint64_t deadlineMs, int &status, std::string &body)
{
    std::string raw;
    size_t headEnd = std::string::npos;
    long contentLen = -1;
    bool chunked = false;
    char buf[8192];
    auto complete = [&]() -> bool {
        if (headEnd == std::string::npos) return false;
        if (contentLen >= 0) return raw.size() >= headEnd + (size_t)contentLen;
        if (chunked) return raw.size() >= headEnd + 5 && raw.compare(raw.size() - 5, 5, "0\r\n\r\n") == 0;
        return false;
    };
    while (!complete()) {
        uint64_t now = NowMs();
        if (now >= deadlineMs) return false;
        struct pollfd pfd = {fd, POLLIN, 0};
        int pr = poll(&pfd, 1, (int)(deadlineMs - now));
        if (pr < 0 && errno == EINTR) continue;
        if (pr <= 0) return false;
        ssize_t n = ::recv(fd, buf, sizeof(buf), 0);
        if (n < 0 && (errno == EINTR || errno == EAGAIN || errno == EWOULDBLOCK)) continue;
        if (n < 0) return false;
        if (n == 0) break;  // closed: what we have is the reply
        raw.append(buf, (size_t)n);
        if (raw.size() > (64u << 20)) return false;
        if (headEnd == std::string::npos) {
            size_t p = raw.find("\r\n\r\n");
            if (p == std::string::npos) continue;
            headEnd = p + 4;
            std::string head = raw.substr(0, headEnd);
            for (auto &ch : head) ch = (char)tolower((unsigned char)ch);
            size_t cl = head.find("\r\ncontent-length:");
            if (cl != std::string::npos) contentLen = strtol(head.c_str() + cl + 17, nullptr, 10);
            size_t te = head.find("\r\ntransfer-encoding:");
            if (te != std::string::npos) {
                size_t eol = head.find("\r\n", te + 2);
                chunked = head.substr(te, eol - te).find("chunked") != std::string::npos;
            }
        }
    }
    if (headEnd == std::string::npos || raw.compare(0, 5, "HTTP/") != 0) return false;
    size_t sp = raw.find(' ');
    if (sp == std::string::npos || sp > 16) return false;
    status = atoi(raw.c_str() + sp + 1);
    if (!chunked) {
        body = contentLen >= 0 ? raw.substr(headEnd, (size_t)contentLen) : raw.substr(headEnd);
        return contentLen < 0 || body.size() == (size_t)contentLen;
    }
    body.clear();
    size_t p = headEnd;
    while (p < raw.size()) {
        size_t eol = raw.find("\r\n", p);
        if (eol == std::string::npos) return false;
        unsigned long len = strtoul(raw.c_str() + p, nullptr, 16);
        p = eol + 2;
        if (len == 0) return true;
        if (p + len > raw.size()) return false;
        body.append(raw, p, len);
        p += len + 2;
    }
    return !body.empty();  // closed after a chunk without the terminating one (a stream the server ended)
}

}  // namespace

struct EtcdBackend::Reply {
    int status = 0;
    Json json;
};

EtcdBackend::EtcdBackend(std::string ip, uint16_t port, std::string instance, std::string user, std::string password)
    : ip_(std::move(ip)), port_(port), user_(std::move(user)), password_(std::move(password))
{
    if (!instance.empty()) root_ = std::string(kClusterRoot) + instance;
    api_ = EnvStr("MF_ETCD_API_PREFIX", nullptr, "/v3");  // "/v3beta" on etcd 3.3
    timeoutMs_ = (uint32_t)EnvInt("MF_ETCD_TIMEOUT_MS", nullptr, 3000, 50, 600000);
    if (user_.empty()) {
        user_ = EnvStr("MF_ETCD_USER", nullptr, "");
        password_ = EnvStr("MF_ETCD_PASSWORD", nullptr, "");
    }
    char host[128] = "host";
    gethostname(host, sizeof(host) - 1);
    char tail[64];
    snprintf(tail, sizeof(tail), ":%d:%p", (int)getpid(), (void *)this);
    owner_ = std::string(host) + tail;
}

EtcdBackend::~EtcdBackend()
{
    {
        std::lock_guard<std::mutex> g(kaMu_);
        stop_ = true;
    }
    kaCv_.notify_all();
    if (keepAlive_.joinable()) keepAlive_.join();
    std::map<std::string, int64_t> locks;
    {
        std::lock_guard<std::mutex> g(mu_);
        locks.swap(locks_);
    }
    for (auto &kv : locks) RevokeLease(kv.second);  // a closing holder frees its locks at once
}

void EtcdBackend::SetError(const std::string &e)
{
    std::lock_guard<std::mutex> g(mu_);
    lastError_ = e;
}

std::string EtcdBackend::LastError()
{
    std::lock_guard<std::mutex> g(mu_);
    return lastError_;
}

std::string EtcdBackend::Qualify(const std::string &key) const
{
    if (root_.empty() || key.compare(0, root_.size(), root_) == 0) return key;
    if (!key.empty() && key.front() == '/') return root_ + key;
    return root_ + "/" + key;
}

int EtcdBackend::CallOnce(const std::string &path, const std::string &body, Reply &reply, bool withToken)
{
    uint32_t to = timeoutMs_.load();
    int fd = DialTimed(ip_, port_, to);
    if (fd < 0) {
        SetError("cannot reach etcd at " + ip_ + ":" + std::to_string(port_));
        return ERR_NOT_CONNECTED;
    }
    std::string token;
    if (withToken) {
        std::lock_guard<std::mutex> g(mu_);
        token = token_;
    }
    std::string req = "POST " + api_ + path + " HTTP/1.1\r\nHost: " + ip_ + ":" + std::to_string(port_) +
                      "\r\nContent-Type: application/json\r\nAccept: application/json\r\nConnection: close\r\nContent-Length: " +
                      std::to_string(body.size()) + "\r\n";
    if (!token.empty()) req += "Authorization: " + token + "\r\n";
    req += "\r\n" + body;
    uint64_t deadline = NowMs() + to;
    std::string text;
    bool ok = SendAllTimed(fd, req, deadline) && ReadReply(fd, deadline, reply.status, text);
    ::close(fd);
    if (!ok) {
        SetError("no complete reply from etcd for " + path);
        return ERR_NOT_CONNECTED;
    }
    reply.json = Json();
    // a streaming call answers {"result":{...}}; one JSON document per line
    size_t nl = text.find('\n');
    if (nl != std::string::npos && nl + 1 < text.size()) text.resize(nl);
    if (!text.empty() && !JsonParser(text).Parse(reply.json)) {
        SetError("unreadable reply from etcd for " + path);
        return ERR;
    }
    return OK;
}

int EtcdBackend::Authenticate()
{
    Reply r;
    int rc = CallOnce("/auth/authenticate", "{\"name\":" + Quoted(user_) + ",\"password\":" + Quoted(password_) + "}", r, false);
    if (rc != OK) return rc;
    std::string tok = r.json.Str("token");
    if (r.status != 200 || tok.empty()) {
        SetError("etcd refused the credentials of user " + user_ + ": " + r.json.Str("error") + r.json.Str("message"));
        return ERR_NOT_CONNECTED;
    }
    std::lock_guard<std::mutex> g(mu_);
    token_ = tok;
    return OK;
}

int EtcdBackend::Call(const std::string &path, const std::string &body, Reply &reply)
{
    bool auth = !user_.empty();
    if (auth) {
        bool have;
        {
            std::lock_guard<std::mutex> g(mu_);
            have = !token_.empty();
        }
        if (!have) {
            int rc = Authenticate();
            if (rc != OK) return rc;
        }
    }
    int rc = CallOnce(path, body, reply, auth);
    if (rc == OK && auth && reply.status == 401) {  // the token ran out: log in again, once
        rc = Authenticate();
        if (rc == OK) rc = CallOnce(path, body, reply, true);
    }
    if (rc != OK) return rc;
    if (reply.status != 200) {
        std::string why = reply.json.Str("error");
        if (why.empty()) why = reply.json.Str("message");
        SetError("etcd answered " + std::to_string(reply.status) + " to " + path + ": " + why);
        return ERR;
    }
    return OK;
}

int EtcdBackend::Connect()
{
    // a range over a key that nobody writes: cheap, and it passes through authentication
    Reply r;
    int rc = Call("/kv/range", "{\"key\":\"" + B64Encode(Qualify("/memfabric_hybrid/ping")) + "\",\"count_only\":true}", r);
    return rc == OK ? OK : ERR_NOT_CONNECTED;
}

int EtcdBackend::GrantLease(int64_t ttlSec, int64_t &id)
{
    Reply r;
    int rc = Call("/lease/grant", "{\"TTL\":\"" + std::to_string(ttlSec) + "\"}", r);
    if (rc != OK) return rc;
    id = r.json.Int("ID");
    if (id == 0) {
        SetError("etcd granted no lease: " + r.json.Str("error"));
        return ERR;
    }
    return OK;
}

void EtcdBackend::RevokeLease(int64_t id)
{
    Reply r;
    Call("/lease/revoke", "{\"ID\":\"" + std::to_string(id) + "\"}", r);
}

int EtcdBackend::Put(const std::string &key, const std::string &value, uint32_t ttlMs)
{
    std::string k = Qualify(key);
    int64_t lease = 0;
    if (ttlMs != 0) {
        int rc = GrantLease(((int64_t)ttlMs + 999) / 1000, lease);
        if (rc != OK) return rc;
    }
    std::string body = "{\"key\":\"" + B64Encode(k) + "\",\"value\":\"" + B64Encode(value) + "\"";
    if (lease != 0) body += ",\"lease\":\"" + std::to_string(lease) + "\"";
    body += "}";
    Reply r;
    int rc = Call("/kv/put", body, r);
    if (rc != OK) {
        if (lease != 0) RevokeLease(lease);
        return rc;
    }
    int64_t old = 0;
    {
        std::lock_guard<std::mutex> g(mu_);
        auto it = putLeases_.find(k);
        if (it != putLeases_.end()) {
            old = it->second;
            putLeases_.erase(it);
        }
        if (lease != 0) putLeases_[k] = lease;
    }
    if (old != 0) RevokeLease(old);  // the key hangs on the new lease (or on none) by now
    return OK;
}

int EtcdBackend::Get(const std::string &key, std::string &value)
{
    Reply r;
    int rc = Call("/kv/range", "{\"key\":\"" + B64Encode(Qualify(key)) + "\"}", r);
    if (rc != OK) return rc;
    const Json *kvs = r.json.Find("kvs");
    if (kvs == nullptr || kvs->kind != Json::ARR || kvs->arr.empty()) return ERR_NOT_EXIST;
    if (!B64Decode(kvs->arr[0].Str("value"), value)) return ERR;  // an empty value has no "value" member
    return OK;
}

int EtcdBackend::PrefixGet(const std::string &prefix, std::vector<std::pair<std::string, std::string>> &out)
{
    std::string p = Qualify(prefix);
    Reply r;
    int rc = Call("/kv/range", "{\"key\":\"" + B64Encode(p.empty() ? std::string(1, '\0') : p) + "\",\"range_end\":\"" +
                                   B64Encode(RangeEnd(p)) + "\",\"sort_order\":\"ASCEND\",\"sort_target\":\"KEY\"}",
                  r);
    if (rc != OK) return rc;
    out.clear();
    const Json *kvs = r.json.Find("kvs");
    if (kvs == nullptr || kvs->kind != Json::ARR) return OK;
    for (auto &kv : kvs->arr) {
        std::string k, v;
        if (!B64Decode(kv.Str("key"), k) || !B64Decode(kv.Str("value"), v)) return ERR;
        // callers see the names they wrote: without the cluster root
        if (!root_.empty() && k.compare(0, root_.size(), root_) == 0 && prefix.compare(0, root_.size(), root_) != 0) {
            k = k.substr(root_.size());
            if (!prefix.empty() && prefix.front() != '/' && !k.empty() && k.front() == '/') k = k.substr(1);
        }
        out.emplace_back(std::move(k), std::move(v));
    }
    return OK;
}

int EtcdBackend::Delete(const std::string &key)
{
    std::string k = Qualify(key);
    Reply r;
    int rc = Call("/kv/deleterange", "{\"key\":\"" + B64Encode(k) + "\"}", r);
    if (rc != OK) return rc;
    {
        std::lock_guard<std::mutex> g(mu_);
        putLeases_.erase(k);  // the lease, if any, runs out by itself
    }
    return r.json.Int("deleted") > 0 ? OK : ERR_NOT_EXIST;
}

int EtcdBackend::Clear(const std::string &prefix)
{
    std::string p = Qualify(prefix);
    Reply r;
    int rc = Call("/kv/deleterange",
                  "{\"key\":\"" + B64Encode(p.empty() ? std::string(1, '\0') : p) + "\",\"range_end\":\"" + B64Encode(RangeEnd(p)) + "\"}", r);
    if (rc != OK) return rc;
    std::lock_guard<std::mutex> g(mu_);
    for (auto it = putLeases_.lower_bound(p); it != putLeases_.end() && it->first.compare(0, p.size(), p) == 0;) it = putLeases_.erase(it);
    return OK;
}

int EtcdBackend::Acquire(const std::string &name, bool wait)
{
    {
        std::lock_guard<std::mutex> g(mu_);
        if (locks_.count(name)) return ERR_IN_USE;  // not re-entrant: this object holds it already
    }
    int64_t lease = 0;
    int rc = GrantLease(kLockTtlSec, lease);
    if (rc != OK) return rc;
    std::string k64 = B64Encode(Qualify("/memfabric_hybrid/config_store/locks/" + name));
    std::string body = "{\"compare\":[{\"key\":\"" + k64 + "\",\"target\":\"CREATE\",\"result\":\"EQUAL\",\"create_revision\":\"0\"}],"
                       "\"success\":[{\"request_put\":{\"key\":\"" + k64 + "\",\"value\":\"" + B64Encode(owner_) + "\",\"lease\":\"" +
                       std::to_string(lease) + "\"}}]}";
    uint64_t deadline = NowMs() + kLockWaitMs;
    uint64_t renewAt = NowMs() + kLockTtlSec * 1000 / 3;
    uint32_t pause = 20;
    while (true) {
        Reply r;
        rc = Call("/kv/txn", body, r);
        if (rc != OK) break;
        if (r.json.Bool("succeeded")) {
            {
                std::lock_guard<std::mutex> g(mu_);
                locks_[name] = lease;
            }
            std::lock_guard<std::mutex> g(kaMu_);
            if (!keepAlive_.joinable() && !stop_) keepAlive_ = std::thread([this] { KeepAliveLoop(); });
            return OK;
        }
        if (!wait) {
            rc = ERR_IN_USE;
            break;
        }
        if (NowMs() >= deadline) {
            rc = ERR_TIMEOUT;
            break;
        }
        std::this_thread::sleep_for(std::chrono::milliseconds(pause));
        pause = std::min<uint32_t>(pause * 2, 250);
        if (NowMs() >= renewAt) {  // the lease we are waiting with must not run out before we win
            Reply ka;
            Call("/lease/keepalive", "{\"ID\":\"" + std::to_string(lease) + "\"}", ka);
            renewAt = NowMs() + kLockTtlSec * 1000 / 3;
        }
    }
    RevokeLease(lease);
    return rc;
}

int EtcdBackend::Lock(const std::string &name) { return Acquire(name, true); }

int EtcdBackend::TryLock(const std::string &name) { return Acquire(name, false); }

int EtcdBackend::Unlock(const std::string &name)
{
    int64_t lease = 0;
    {
        std::lock_guard<std::mutex> g(mu_);
        auto it = locks_.find(name);
        if (it == locks_.end()) return ERR_NOT_EXIST;
        lease = it->second;
        locks_.erase(it);
    }
    RevokeLease(lease);  // takes the lock key with it
    return OK;
}

void EtcdBackend::KeepAliveLoop()
{
    std::unique_lock<std::mutex> lk(kaMu_);
    while (!stop_) {
        kaCv_.wait_for(lk, std::chrono::milliseconds(kLockTtlSec * 1000 / 3), [this] { return stop_; });
        if (stop_) break;
        lk.unlock();
        std::vector<int64_t> leases;
        {
            std::lock_guard<std::mutex> g(mu_);
            for (auto &kv : locks_) leases.push_back(kv.second);
        }
        for (int64_t id : leases) {
            Reply r;
            int rc = Call("/lease/keepalive", "{\"ID\":\"" + std::to_string(id) + "\"}", r);
            const Json *res = rc == OK ? r.json.Find("result") : nullptr;
            if (rc == OK && (res == nullptr ? r.json.Int("TTL") : res->Int("TTL")) <= 0)
                MF_WARN("etcd lease %lld of a held lock has run out", (long long)id);
        }
        lk.lock();
    }
}

}  // namespace store
}  // namespace mf
