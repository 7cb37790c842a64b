#include "mf_tls.h"

#include <dlfcn.h>
#include <fcntl.h>
#include <poll.h>
#include <string.h>
#include <time.h>
#include <unistd.h>

#include <pthread.h>

#include <algorithm>
#include <chrono>
#include <climits>
#include <fstream>
#include <sstream>
#include <thread>

#include "../util/mf_util.h"

namespace mf {
namespace net {
namespace {

// The handful of OpenSSL 3 constants this file needs (stable ABI values of the public headers).
constexpr int kSslCtrlMode = 33, kSslCtrlSetMinProto = 123, kSslCtrlSetMaxProto = 124;
constexpr long kTls13 = 0x0304;
constexpr long kModePartialWrite = 0x1, kModeMovingBuffer = 0x2;
constexpr int kVerifyPeer = 0x1, kVerifyFailIfNoPeerCert = 0x2;
constexpr int kFiletypePem = 1;
constexpr int kErrWantRead = 2, kErrWantWrite = 3, kErrZeroReturn = 6;
constexpr unsigned long kCrlCheck = 0x4, kCrlCheckAll = 0x8;

struct Api {
    void *ssl = nullptr, *crypto = nullptr;
    // libssl
    const void *(*TLS_method)() = nullptr;
    void *(*SSL_CTX_new)(const void *) = nullptr;
    void (*SSL_CTX_free)(void *) = nullptr;
    long (*SSL_CTX_ctrl)(void *, int, long, void *) = nullptr;
    int (*SSL_CTX_use_certificate_chain_file)(void *, const char *) = nullptr;
    int (*SSL_CTX_use_PrivateKey_file)(void *, const char *, int) = nullptr;
    int (*SSL_CTX_use_PrivateKey)(void *, void *) = nullptr;
    int (*SSL_CTX_check_private_key)(const void *) = nullptr;
    int (*SSL_CTX_load_verify_locations)(void *, const char *, const char *) = nullptr;
    void (*SSL_CTX_set_verify)(void *, int, void *) = nullptr;
    void (*SSL_CTX_set_default_passwd_cb_userdata)(void *, void *) = nullptr;
    void *(*SSL_CTX_get_cert_store)(const void *) = nullptr;
    void *(*SSL_CTX_get0_certificate)(const void *) = nullptr;
    void *(*SSL_new)(void *) = nullptr;
    void (*SSL_free)(void *) = nullptr;
    int (*SSL_set_fd)(void *, int) = nullptr;
    int (*SSL_accept)(void *) = nullptr;
    int (*SSL_connect)(void *) = nullptr;
    int (*SSL_read)(void *, void *, int) = nullptr;
    int (*SSL_write)(void *, const void *, int) = nullptr;
    int (*SSL_get_error)(const void *, int) = nullptr;
    int (*SSL_shutdown)(void *) = nullptr;
    void *(*SSL_get1_peer_certificate)(const void *) = nullptr;
    long (*SSL_get_verify_result)(const void *) = nullptr;
    // libcrypto
    void *(*BIO_new_mem_buf)(const void *, int) = nullptr;
    int (*BIO_free)(void *) = nullptr;
    void *(*PEM_read_bio_PrivateKey)(void *, void **, void *, void *) = nullptr;
    void (*EVP_PKEY_free)(void *) = nullptr;
    int (*X509_STORE_load_locations)(void *, const char *, const char *) = nullptr;
    int (*X509_STORE_set_flags)(void *, unsigned long) = nullptr;
    void (*X509_free)(void *) = nullptr;
    void *(*X509_get_subject_name)(const void *) = nullptr;
    char *(*X509_NAME_oneline)(const void *, char *, int) = nullptr;
    const void *(*X509_get0_notAfter)(const void *) = nullptr;
    int (*ASN1_TIME_diff)(int *, int *, const void *, const void *) = nullptr;
    unsigned long (*ERR_get_error)() = nullptr;
    void (*ERR_error_string_n)(unsigned long, char *, size_t) = nullptr;
    void (*ERR_clear_error)() = nullptr;
};

std::mutex g_apiMu;
Api g_api;
bool g_apiLoaded = false;

void *OpenLib(const std::string &dir, const char *const *names)
{
    for (const char *const *n = names; *n != nullptr; n++) {
        std::string path = dir.empty() ? std::string(*n) : dir + "/" + *n;
        void *h = dlopen(path.c_str(), RTLD_NOW | RTLD_GLOBAL);
        if (h != nullptr) return h;
    }
    return nullptr;
}

template <typename F> bool Sym(void *lib, const char *name, F &out)
{
    out = reinterpret_cast<F>(dlsym(lib, name));
    return out != nullptr;
}

bool LoadApi(const std::string &packagePath, std::string &err)
{
    std::lock_guard<std::mutex> g(g_apiMu);
    if (g_apiLoaded) return true;
    static const char *const cryptoNames[] = {"libcrypto.so.3", "libcrypto.so", nullptr};
    static const char *const sslNames[] = {"libssl.so.3", "libssl.so", nullptr};
    Api a;
    a.crypto = OpenLib(packagePath, cryptoNames);
    a.ssl = OpenLib(packagePath, sslNames);
    if (a.crypto == nullptr || a.ssl == nullptr) {
        const char *d = dlerror();
        err = std::string("cannot open libssl / libcrypto") + (packagePath.empty() ? "" : " under " + packagePath) + (d ? std::string(": ") + d : "");
        return false;
    }
    bool ok = true;
#define MF_SSL(name) ok = Sym(a.ssl, #name, a.name) && ok
#define MF_CRYPTO(name) ok = Sym(a.crypto, #name, a.name) && ok
    MF_SSL(TLS_method);
    MF_SSL(SSL_CTX_new);
    MF_SSL(SSL_CTX_free);
    MF_SSL(SSL_CTX_ctrl);
    MF_SSL(SSL_CTX_use_certificate_chain_file);
    MF_SSL(SSL_CTX_use_PrivateKey_file);
    MF_SSL(SSL_CTX_use_PrivateKey);
    MF_SSL(SSL_CTX_check_private_key);
    MF_SSL(SSL_CTX_load_verify_locations);
    MF_SSL(SSL_CTX_set_verify);
    MF_SSL(SSL_CTX_set_default_passwd_cb_userdata);
    MF_SSL(SSL_CTX_get_cert_store);
    MF_SSL(SSL_CTX_get0_certificate);
    MF_SSL(SSL_new);
    MF_SSL(SSL_free);
    MF_SSL(SSL_set_fd);
    MF_SSL(SSL_accept);
    MF_SSL(SSL_connect);
    MF_SSL(SSL_read);
    MF_SSL(SSL_write);
    MF_SSL(SSL_get_error);
    MF_SSL(SSL_shutdown);
    MF_SSL(SSL_get_verify_result);
    if (!Sym(a.ssl, "SSL_get1_peer_certificate", a.SSL_get1_peer_certificate))  // OpenSSL 1.1 name
        ok = Sym(a.ssl, "SSL_get_peer_certificate", a.SSL_get1_peer_certificate) && ok;
    MF_CRYPTO(BIO_new_mem_buf);
    MF_CRYPTO(BIO_free);
    MF_CRYPTO(PEM_read_bio_PrivateKey);
    MF_CRYPTO(EVP_PKEY_free);
    MF_CRYPTO(X509_STORE_load_locations);
    MF_CRYPTO(X509_STORE_set_flags);
    MF_CRYPTO(X509_free);
    MF_CRYPTO(X509_get_subject_name);
    MF_CRYPTO(X509_NAME_oneline);
    MF_CRYPTO(X509_get0_notAfter);
    MF_CRYPTO(ASN1_TIME_diff);
    MF_CRYPTO(ERR_get_error);
    MF_CRYPTO(ERR_error_string_n);
    MF_CRYPTO(ERR_clear_error);
#undef MF_SSL
#undef MF_CRYPTO
    if (!ok) {
        err = "libssl / libcrypto lack an entry point this build needs (OpenSSL 1.1.1 or 3.x expected)";
        return false;
    }
    g_api = a;
    g_apiLoaded = true;
    return true;
}

std::string LastSslError()
{
    char buf[256] = "no OpenSSL error queued";
    unsigned long e = g_api.ERR_get_error();
    if (e != 0) g_api.ERR_error_string_n(e, buf, sizeof(buf));
    g_api.ERR_clear_error();
    return buf;
}

std::string Trim(const std::string &s)
{
    size_t a = s.find_first_not_of(" \t\r\n"), b = s.find_last_not_of(" \t\r\n");
    return a == std::string::npos ? std::string() : s.substr(a, b - a + 1);
}

std::vector<std::string> SplitList(const std::string &s)
{
    std::vector<std::string> out;
    std::stringstream ss(s);
    std::string item;
    while (std::getline(ss, item, ',')) {
        item = Trim(item);
        if (!item.empty()) out.push_back(item);
    }
    return out;
}

bool ReadFile(const std::string &path, std::string &out)
{
    std::ifstream f(path, std::ios::binary);
    if (!f) return false;
    std::stringstream ss;
    ss << f.rdbuf();
    out = ss.str();
    return true;
}

std::string Join(const std::string &dir, const std::string &name)
{
    if (name.empty() || name[0] == '/' || dir.empty()) return name;
    return dir.back() == '/' ? dir + name : dir + "/" + name;
}

bool IsDir(const std::string &p)
{
    int fd = open(p.c_str(), O_RDONLY | O_DIRECTORY | O_CLOEXEC);
    if (fd < 0) return false;
    close(fd);
    return true;
}

uint64_t NowMsMono()
{
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (uint64_t)ts.tv_sec * 1000 + (uint64_t)ts.tv_nsec / 1000000;
}

int EnvInt(const char *name, int lo, int hi, int dflt)
{
    const char *e = getenv(name);
    if (e == nullptr || *e == 0) return dflt;
    char *end = nullptr;
    long v = strtol(e, &end, 10);
    if (end == e || *end != 0 || v < lo || v > hi) return dflt;
    return (int)v;
}
}  // namespace

// ---- periodic certificate check: one detached thread per process, started with the first context -------------------
std::mutex g_checkMu;
std::vector<std::weak_ptr<TlsContext>> g_contexts;
bool g_checkerStarted = false;

void RegisterForChecks(const std::shared_ptr<TlsContext> &c)
{
    std::lock_guard<std::mutex> g(g_checkMu);
    g_contexts.push_back(c);
    if (g_checkerStarted) return;
    g_checkerStarted = true;
    std::thread([] {
        pthread_setname_np(pthread_self(), "mf-tls-check");
        for (;;) {
            const int hours = EnvInt("MF_ACC_CHECK_PERIOD_HOURS", 24, 24 * 30, 7 * 24);
            std::this_thread::sleep_for(std::chrono::hours(hours));
            (void)TlsCheckAllNow();
        }
    }).detach();  // sleeps for days and touches only objects it keeps alive: it ends with the process
}

bool TlsSettings::Parse(const std::string &info, TlsSettings &out, std::string &err)
{
    TlsSettings s;
    s.enable = true;
    std::stringstream ss(info);
    std::string field;
    while (std::getline(ss, field, ';')) {
        field = Trim(field);
        if (field.empty()) continue;
        size_t c = field.find(':');
        if (c == std::string::npos) {
            err = "TLS info field without ':' : " + field;
            return false;
        }
        std::string k = Trim(field.substr(0, c)), v = Trim(field.substr(c + 1));
        if (k == "tlsCaPath") s.caPath = v;
        else if (k == "tlsCaFile") s.caFiles = SplitList(v);
        else if (k == "tlsCert") s.certPath = v;
        else if (k == "tlsPk") s.keyPath = v;
        else if (k == "tlsPkPwd") s.keyPassPath = v;
        else if (k == "tlsCrlPath") s.crlPath = v;
        else if (k == "tlsCrlFile") s.crlFiles = SplitList(v);
        else if (k == "packagePath") s.packagePath = v;
        else if (k == "decrypterLibPath") s.decrypterLibPath = v;
        else {
            err = "unknown TLS info key: " + k;
            return false;
        }
    }
    if (s.certPath.empty() || (s.caPath.empty() && s.caFiles.empty())) {
        err = "TLS info needs tlsCert and tlsCaPath / tlsCaFile";
        return false;
    }
    out = s;
    return true;
}

bool TlsAvailable(const std::string &packagePath, std::string &err) { return LoadApi(packagePath, err); }

std::shared_ptr<TlsContext> TlsContext::Create(const TlsSettings &s, std::string &err)
{
    if (!LoadApi(s.packagePath, err)) return nullptr;
    const Api &A = g_api;
    std::shared_ptr<TlsContext> c(new TlsContext());
    A.ERR_clear_error();
    c->ctx_ = A.SSL_CTX_new(A.TLS_method());
    if (c->ctx_ == nullptr) {
        err = "SSL_CTX_new: " + LastSslError();
        return nullptr;
    }
    A.SSL_CTX_ctrl(c->ctx_, kSslCtrlSetMinProto, kTls13, nullptr);
    A.SSL_CTX_ctrl(c->ctx_, kSslCtrlSetMaxProto, kTls13, nullptr);
    A.SSL_CTX_ctrl(c->ctx_, kSslCtrlMode, kModePartialWrite | kModeMovingBuffer, nullptr);

    // trust store
    int loaded = 0;
    for (const auto &f : s.caFiles) {
        std::string p = Join(s.caPath, f);
        if (A.SSL_CTX_load_verify_locations(c->ctx_, p.c_str(), nullptr) != 1) {
            err = "cannot load CA file " + p + ": " + LastSslError();
            return nullptr;
        }
        loaded++;
    }
    if (loaded == 0) {
        // one path: a PEM file, or a directory in OpenSSL's hashed layout
        const bool dir = IsDir(s.caPath);
        if (A.SSL_CTX_load_verify_locations(c->ctx_, dir ? nullptr : s.caPath.c_str(), dir ? s.caPath.c_str() : nullptr) != 1) {
            err = "cannot load CA from " + s.caPath + ": " + LastSslError();
            return nullptr;
        }
    }
    // revocation lists
    if (!s.crlFiles.empty()) {
        void *store = A.SSL_CTX_get_cert_store(c->ctx_);
        for (const auto &f : s.crlFiles) {
            std::string p = Join(s.crlPath, f);
            if (A.X509_STORE_load_locations(store, p.c_str(), nullptr) != 1) {
                err = "cannot load CRL " + p + ": " + LastSslError();
                return nullptr;
            }
        }
        A.X509_STORE_set_flags(store, kCrlCheck | kCrlCheckAll);
    }
    // certificate
    if (A.SSL_CTX_use_certificate_chain_file(c->ctx_, s.certPath.c_str()) != 1) {
        err = "cannot load certificate " + s.certPath + ": " + LastSslError();
        return nullptr;
    }
    void *cert = A.SSL_CTX_get0_certificate(c->ctx_);
    if (cert != nullptr) {
        int days = 0, secs = 0;
        if (A.ASN1_TIME_diff(&days, &secs, nullptr, A.X509_get0_notAfter(cert)) == 1) {
            c->certDaysLeft_ = (days < 0 || secs < 0) ? -1 : days;
            c->notAfterUnix_ = (int64_t)time(nullptr) + (int64_t)days * 86400 + secs;
            c->certPath_ = s.certPath;
            const int ahead = EnvInt("MF_ACC_CERT_CHECK_AHEAD_DAYS", 7, 180, 30);
            if (c->certDaysLeft_ < 0) {
                err = "certificate " + s.certPath + " has expired";
                return nullptr;
            }
            if (c->certDaysLeft_ < ahead) MF_WARN("TLS certificate %s expires in %d days", s.certPath.c_str(), c->certDaysLeft_);
        }
    }
    // pass phrase of the key: plain, from a file, optionally through the caller's decrypter
    std::string pass = s.keyPass;
    if (pass.empty() && !s.keyPassPath.empty() && !ReadFile(s.keyPassPath, pass)) {
        err = "cannot read the key pass phrase file " + s.keyPassPath;
        return nullptr;
    }
    while (!pass.empty() && (pass.back() == '\n' || pass.back() == '\r')) pass.pop_back();
    TlsDecryptFn dec = s.decrypt;
    if (dec == nullptr && !s.decrypterLibPath.empty()) {
        void *lib = dlopen(s.decrypterLibPath.c_str(), RTLD_NOW);
        if (lib != nullptr) dec = reinterpret_cast<TlsDecryptFn>(dlsym(lib, "DecryptPassword"));
        if (dec == nullptr) {
            err = "cannot load DecryptPassword from " + s.decrypterLibPath;
            return nullptr;
        }
    }
    if (!pass.empty() && dec != nullptr) {
        std::string plain(pass.size() + 256, '\0');
        size_t n = plain.size();
        if (dec(pass.data(), pass.size(), &plain[0], n) != 0 || n > plain.size()) {
            err = "the decrypt handler rejected the key pass phrase";
            return nullptr;
        }
        plain.resize(n);
        pass = plain;
    }
    c->keyPassPlain_ = pass;
    // OpenSSL's default callback copies the userdata string when one is set
    if (!c->keyPassPlain_.empty()) A.SSL_CTX_set_default_passwd_cb_userdata(c->ctx_, const_cast<char *>(c->keyPassPlain_.c_str()));
    // key
    if (!s.keyPem.empty()) {
        void *bio = A.BIO_new_mem_buf(s.keyPem.data(), (int)s.keyPem.size());
        void *pkey = bio != nullptr
                         ? A.PEM_read_bio_PrivateKey(bio, nullptr, nullptr,
                                                     c->keyPassPlain_.empty() ? nullptr : const_cast<char *>(c->keyPassPlain_.c_str()))
                         : nullptr;
        if (bio != nullptr) A.BIO_free(bio);
        if (pkey == nullptr) {
            err = "cannot parse the private key: " + LastSslError();
            return nullptr;
        }
        int rc = A.SSL_CTX_use_PrivateKey(c->ctx_, pkey);
        A.EVP_PKEY_free(pkey);
        if (rc != 1) {
            err = "cannot use the private key: " + LastSslError();
            return nullptr;
        }
    } else if (!s.keyPath.empty()) {
        if (A.SSL_CTX_use_PrivateKey_file(c->ctx_, s.keyPath.c_str(), kFiletypePem) != 1) {
            err = "cannot load the private key " + s.keyPath + ": " + LastSslError();
            return nullptr;
        }
    } else {
        err = "TLS is enabled but no private key was given (tlsPk in the TLS info, keyPath, or smem_set_config_store_tls_key)";
        return nullptr;
    }
    if (A.SSL_CTX_check_private_key(c->ctx_) != 1) {
        err = "the private key does not match the certificate: " + LastSslError();
        return nullptr;
    }
    A.SSL_CTX_set_verify(c->ctx_, kVerifyPeer | kVerifyFailIfNoPeerCert, nullptr);
    RegisterForChecks(c);
    return c;
}

int TlsContext::CheckExpiry()
{
    if (notAfterUnix_ == 0) return certDaysLeft_;
    const int64_t left = notAfterUnix_ - (int64_t)time(nullptr);
    certDaysLeft_ = left < 0 ? -1 : (int)(left / 86400);
    const int ahead = EnvInt("MF_ACC_CERT_CHECK_AHEAD_DAYS", 7, 180, 30);
    if (certDaysLeft_ < 0) {
        MF_ERROR("TLS certificate %s has expired", certPath_.c_str());
        Logger::Get().Alarm(0x7101, "TLS certificate expired");
    } else if (certDaysLeft_ < ahead) {
        MF_WARN("TLS certificate %s expires in %d days", certPath_.c_str(), certDaysLeft_);
        Logger::Get().Alarm(0x7100, "TLS certificate close to expiry");
    }
    return certDaysLeft_;
}

int TlsCheckAllNow()
{
    int least = INT32_MAX;
    std::vector<std::shared_ptr<TlsContext>> live;
    {
        std::lock_guard<std::mutex> g(g_checkMu);
        for (auto it = g_contexts.begin(); it != g_contexts.end();) {
            if (auto c = it->lock()) {
                live.push_back(c);
                ++it;
            } else {
                it = g_contexts.erase(it);
            }
        }
    }
    for (auto &c : live) least = std::min(least, c->CheckExpiry());
    return least;
}

TlsContext::~TlsContext()
{
    if (ctx_ != nullptr && g_apiLoaded) g_api.SSL_CTX_free(ctx_);
    // the pass phrase does not outlive the context
    for (auto &ch : keyPassPlain_) ch = 0;
}

std::unique_ptr<TlsSession> TlsContext::Handshake(int fd, bool asServer, uint32_t timeoutMs, std::string &err)
{
    const Api &A = g_api;
    int fl = fcntl(fd, F_GETFL, 0);
    fcntl(fd, F_SETFL, fl | O_NONBLOCK);
    A.ERR_clear_error();
    void *ssl = A.SSL_new(ctx_);
    if (ssl == nullptr || A.SSL_set_fd(ssl, fd) != 1) {
        err = "SSL_new / SSL_set_fd: " + LastSslError();
        if (ssl != nullptr) A.SSL_free(ssl);
        return nullptr;
    }
    const uint64_t deadline = NowMsMono() + (timeoutMs == 0 ? 5000 : timeoutMs);
    for (;;) {
        A.ERR_clear_error();
        int rc = asServer ? A.SSL_accept(ssl) : A.SSL_connect(ssl);
        if (rc == 1) break;
        int e = A.SSL_get_error(ssl, rc);
        uint64_t now = NowMsMono();
        if ((e != kErrWantRead && e != kErrWantWrite) || now >= deadline) {
            err = (now >= deadline ? std::string("TLS handshake timed out") : "TLS handshake failed: " + LastSslError());
            A.SSL_free(ssl);
            return nullptr;
        }
        struct pollfd pfd = {fd, (short)(e == kErrWantRead ? POLLIN : POLLOUT), 0};
        poll(&pfd, 1, (int)(deadline - now));
    }
    if (A.SSL_get_verify_result(ssl) != 0) {
        err = "the peer's certificate did not verify";
        A.SSL_free(ssl);
        return nullptr;
    }
    return std::unique_ptr<TlsSession>(new TlsSession(ssl, fd));
}

TlsSession::~TlsSession()
{
    if (ssl_ != nullptr) {
        g_api.ERR_clear_error();
        (void)g_api.SSL_shutdown(ssl_);  // one non-blocking attempt at close_notify
        g_api.SSL_free(ssl_);
    }
}

bool TlsSession::WriteAll(const void *buf, size_t len, uint32_t timeoutMs)
{
    const Api &A = g_api;
    const char *p = static_cast<const char *>(buf);
    while (len > 0) {
        int n, e = 0;
        {
            std::lock_guard<std::mutex> g(mu_);
            A.ERR_clear_error();
            n = A.SSL_write(ssl_, p, (int)std::min<size_t>(len, 1 << 20));
            if (n <= 0) e = A.SSL_get_error(ssl_, n);
        }
        if (n > 0) {
            p += n;
            len -= (size_t)n;
            continue;
        }
        if (e != kErrWantRead && e != kErrWantWrite) return false;
        struct pollfd pfd = {fd_, (short)(e == kErrWantRead ? POLLIN : POLLOUT), 0};
        if (poll(&pfd, 1, (int)timeoutMs) <= 0) return false;
    }
    return true;
}

long TlsSession::ReadSome(void *buf, size_t len)
{
    const Api &A = g_api;
    std::lock_guard<std::mutex> g(mu_);
    A.ERR_clear_error();
    int n = A.SSL_read(ssl_, buf, (int)std::min<size_t>(len, 1 << 30));
    if (n > 0) return n;
    int e = A.SSL_get_error(ssl_, n);
    if (e == kErrWantRead || e == kErrWantWrite) return 0;
    return e == kErrZeroReturn ? -1 : -2;
}

bool TlsSession::ReadAll(void *buf, size_t len, uint32_t timeoutMs)
{
    char *p = static_cast<char *>(buf);
    const uint64_t deadline = NowMsMono() + timeoutMs;
    while (len > 0) {
        long n = ReadSome(p, len);
        if (n < 0) return false;
        if (n > 0) {
            p += n;
            len -= (size_t)n;
            continue;
        }
        uint64_t now = NowMsMono();
        if (now >= deadline) return false;
        struct pollfd pfd = {fd_, POLLIN, 0};
        poll(&pfd, 1, (int)std::min<uint64_t>(deadline - now, 100));
    }
    return true;
}

std::string TlsSession::PeerSubject()
{
    const Api &A = g_api;
    std::lock_guard<std::mutex> g(mu_);
    void *cert = A.SSL_get1_peer_certificate(ssl_);
    if (cert == nullptr) return std::string();
    char buf[512] = {0};
    A.X509_NAME_oneline(A.X509_get_subject_name(cert), buf, sizeof(buf) - 1);
    A.X509_free(cert);
    return buf;
}

}  // namespace net
}  // namespace mf
