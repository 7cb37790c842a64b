// TLS 1.3 for the framed TCP RPC, on an OpenSSL 3 that is opened at run time (dlopen of libssl / libcrypto, so that the
// library itself links against neither). Both ends present a certificate and verify the peer against the same CA set
// (mutual TLS); certificate revocation lists are honoured when given.
// Counterpart of the reference's acc_links security layer (src/acc_links/csrc/security/acc_tcp_ssl_helper.cpp and
// the OpenSSL wrapper beside it).
#pragma once
#include <stdint.h>

#include <memory>
#include <mutex>
#include <string>
#include <vector>

namespace mf {
namespace net {

// plainText receives at most plainTextLen bytes; plainTextLen is updated to what was written. Returns 0 on success.
using TlsDecryptFn = int (*)(const char *cipherText, size_t cipherTextLen, char *plainText, size_t &plainTextLen);

struct TlsSettings {
    bool enable = false;
    std::string caPath;             // directory of the CA files (or, with no caFiles, one CA file / a hashed directory)
    std::vector<std::string> caFiles;
    std::string certPath;           // this end's certificate (PEM, chain allowed)
    std::string keyPath;            // private key file (PEM) ...
    std::string keyPem;             // ... or its content
    std::string keyPass;            // pass phrase of the key (plain, or cipher text when `decrypt` is set)
    std::string keyPassPath;        // file holding the pass phrase (same rule)
    std::string crlPath;            // directory of the revocation lists
    std::vector<std::string> crlFiles;
    std::string packagePath;        // directory of libssl.so / libcrypto.so (empty: the loader's search path)
    std::string decrypterLibPath;   // shared object exporting "DecryptPassword" with the TlsDecryptFn signature
    TlsDecryptFn decrypt = nullptr;

    // "tlsCaPath: /dir/; tlsCaFile: a.pem,b.pem; tlsCert: /x/server.crt; tlsPk: /x/server.key; tlsPkPwd: /x/pass;
    //  tlsCrlPath: /crl/; tlsCrlFile: r.pem; packagePath: /usr/lib64" -> settings. Unknown keys are an error.
    static bool Parse(const std::string &info, TlsSettings &out, std::string &err);
};

class TlsSession;

// One SSL_CTX: certificate, key and trust store are loaded once and shared by every link of an endpoint.
class TlsContext {
public:
    static std::shared_ptr<TlsContext> Create(const TlsSettings &s, std::string &err);
    ~TlsContext();
    // Handshake over a connected socket (made non-blocking here). nullptr + err when it fails or runs out of time.
    std::unique_ptr<TlsSession> Handshake(int fd, bool asServer, uint32_t timeoutMs, std::string &err);
    // Days until this end's certificate expires (negative: expired), as of the last check.
    int CertDaysLeft() const { return certDaysLeft_; }
    // Re-computes the days left from the certificate's end date and warns (log + alarm hook) inside the warning window
    // (MF_ACC_CERT_CHECK_AHEAD_DAYS, default 30) or after expiry. Run every MF_ACC_CHECK_PERIOD_HOURS (default 168) by a
    // process-wide thread for every live context; tests call it directly. -> days left.
    int CheckExpiry();

private:
    TlsContext() = default;
    void *ctx_ = nullptr;  // SSL_CTX
    int certDaysLeft_ = 0;
    int64_t notAfterUnix_ = 0;  // end of the certificate's validity, seconds since the epoch (0: unknown)
    std::string certPath_;
    std::string keyPassPlain_;
    friend class TlsSession;
};

// One SSL object on a non-blocking socket. OpenSSL allows one thread at a time in an SSL object, so every call takes the
// session's mutex; waiting for the socket happens outside it, which lets the reader make progress while a writer waits
// for buffer space (two ends that are both blocked in a write would otherwise never drain each other).
class TlsSession {
public:
    ~TlsSession();
    // Writes all of buf or fails (false). Waits for the socket at most timeoutMs per stall.
    bool WriteAll(const void *buf, size_t len, uint32_t timeoutMs = 30000);
    // Reads exactly len bytes or fails / runs out of time.
    bool ReadAll(void *buf, size_t len, uint32_t timeoutMs);
    // Non-blocking read: > 0 bytes read, 0 = nothing available now, < 0 = closed or failed.
    long ReadSome(void *buf, size_t len);
    // After the handshake: the peer's certificate subject (one line).
    std::string PeerSubject();

private:
    friend class TlsContext;
    TlsSession(void *ssl, int fd) : ssl_(ssl), fd_(fd) {}
    void *ssl_;
    int fd_;
    std::mutex mu_;
};

// True when libssl / libcrypto could be opened and every entry point resolved (packagePath: see TlsSettings).
bool TlsAvailable(const std::string &packagePath, std::string &err);
// For tests: runs the periodic certificate check of every live context now; -> the smallest number of days left (INT_MAX: none).
int TlsCheckAllNow();

}  // namespace net
}  // namespace mf
