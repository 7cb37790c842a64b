// URL parsing and per-URL store singletons.
// tcp://ip:port            plain TCP store (server started by whoever asks for it)
// etcd://ip:port[#inst]    HA store over etcd v3 at ip:port (native client, mf_store_etcd.h), or over the user-registered op
//                          table when one is set; the store leader listens at MF_CONFIG_STORE_IP : MF_CONFIG_STORE_PORT (or above)
// reg://name[#inst]        HA store over the user-registered op table, or over the in-process backend `name`
// Parity: src/smem/csrc/config_store/smem_store_factory.cpp:50-125,174-251,292-310.
#include "mf_store_backend.h"
#include "mf_store_etcd.h"
#include "mf_store_ha.h"

namespace mf {
namespace store {

bool StoreUrl::Parse(const std::string &url, StoreUrl &out)
{
    out.raw = url;
    std::string rest = url;
    size_t p = rest.find("://");
    std::string scheme = "tcp";
    if (p != std::string::npos) {
        scheme = rest.substr(0, p);
        rest = rest.substr(p + 3);
    }
    if (scheme == "tcp") out.scheme = TCP;
    else if (scheme == "etcd") out.scheme = ETCD;
    else if (scheme == "reg") out.scheme = REG;
    else return false;
    p = rest.find('#');
    if (p != std::string::npos) {
        out.instance = rest.substr(p + 1);
        rest = rest.substr(0, p);
    }
    if (out.scheme == REG && rest.find(':') == std::string::npos) {
        out.ip = rest;  // registry name only
        out.port = 0;
        return !rest.empty();
    }
    return net::ParseIpPort(rest, out.ip, out.port);
}

namespace {
struct Entry {
    StorePtr client;
    std::shared_ptr<StoreServer> server;
    std::shared_ptr<HaConfigStore> ha;
    uint32_t refs = 0;
    bool pinnedServer = false;  // started by smem_create_config_store: outlives the clients of this process
};
std::mutex g_mu;
std::map<std::string, Entry> g_stores;
TlsOptions g_tls;
std::mutex g_tlsMu;  // g_tls and the context below (taken alone, never while g_mu is wanted)
std::shared_ptr<net::TlsContext> g_tlsCtx;
std::string g_tlsKey, g_tlsKeyPass;
net::TlsDecryptFn g_tlsDecrypt = nullptr;
}  // namespace

int StoreFactory::SetTls(bool enable, const std::string &info)
{
    std::lock_guard<std::mutex> g(g_tlsMu);
    g_tlsCtx.reset();
    g_tls.enable = false;
    g_tls.info = info;
    if (!enable) return OK;
    std::string err;
    if (!net::TlsSettings::Parse(info, g_tls.settings, err)) return MF_FAIL(ERR_INVALID_PARAM, "%s", err.c_str());
    if (!net::TlsAvailable(g_tls.settings.packagePath, err)) return MF_FAIL(ERR, "%s", err.c_str());
    g_tls.enable = true;
    return OK;
}

int StoreFactory::SetTlsConfig(const net::TlsSettings &s)
{
    std::lock_guard<std::mutex> g(g_tlsMu);
    g_tlsCtx.reset();
    g_tls.enable = false;
    if (!s.enable) return OK;
    std::string err;
    if (s.certPath.empty() || s.caPath.empty()) return MF_FAIL(ERR_INVALID_PARAM, "TLS config needs caPath and certPath");
    if (!net::TlsAvailable(s.packagePath, err)) return MF_FAIL(ERR, "%s", err.c_str());
    g_tls.settings = s;
    g_tls.enable = true;
    return OK;
}

int StoreFactory::SetTlsKey(const std::string &pk, const std::string &pass, net::TlsDecryptFn decrypt)
{
    std::lock_guard<std::mutex> g(g_tlsMu);
    g_tlsCtx.reset();
    g_tlsKey = pk;
    g_tlsKeyPass = pass;
    g_tlsDecrypt = decrypt;
    return OK;
}

std::shared_ptr<net::TlsContext> StoreFactory::TlsContextFor(int &rc)
{
    std::lock_guard<std::mutex> g(g_tlsMu);
    rc = OK;
    if (!g_tls.enable) return nullptr;
    if (g_tlsCtx) return g_tlsCtx;
    net::TlsSettings s = g_tls.settings;
    if (!g_tlsKey.empty()) {  // the key given through the key call wins over a path in the info string
        if (g_tlsKey.find("-----BEGIN") != std::string::npos) s.keyPem = g_tlsKey;
        else s.keyPath = g_tlsKey;
        s.keyPass = g_tlsKeyPass;
        s.decrypt = g_tlsDecrypt;
    }
    std::string err;
    g_tlsCtx = net::TlsContext::Create(s, err);
    if (!g_tlsCtx) rc = MF_FAIL(ERR, "config-store TLS: %s", err.c_str());
    return g_tlsCtx;
}

const TlsOptions &StoreFactory::Tls() { return g_tls; }

std::shared_ptr<StoreServer> StoreFactory::ServerOf(const std::string &url)
{
    std::lock_guard<std::mutex> g(g_mu);
    auto it = g_stores.find(url);
    return it == g_stores.end() ? nullptr : it->second.server;
}

int StoreFactory::CreateServerOnly(const std::string &url, uint32_t worldSize, uint64_t flags)
{
    StoreUrl u;
    if (!StoreUrl::Parse(url, u) || u.scheme != StoreUrl::TCP) return MF_FAIL(ERR_INVALID_PARAM, "bad store url %s", url.c_str());
    std::lock_guard<std::mutex> g(g_mu);
    Entry &e = g_stores[url];
    if (e.server) return OK;
    auto s = std::make_shared<StoreServer>(u.ip, u.port, worldSize, flags);
    int rc = s->Startup();
    if (rc != OK) {
        if (!e.client) g_stores.erase(url);
        return rc;
    }
    e.server = s;
    e.pinnedServer = true;
    return OK;
}

void StoreFactory::DestroyServer(const std::string &url)
{
    Entry e;
    {
        std::lock_guard<std::mutex> g(g_mu);
        auto it = g_stores.find(url);
        if (it == g_stores.end()) return;
        it->second.pinnedServer = false;
        if (it->second.client) {  // a client of this process still uses it: the last DestroyStore ends the server
            return;
        }
        e = it->second;
        g_stores.erase(it);
    }
    if (e.ha) e.ha->Shutdown();
    if (e.server) e.server->Shutdown();
}

StorePtr StoreFactory::CreateStore(const std::string &url, bool isServer, uint32_t worldSize, uint32_t rank,
                                   uint32_t timeoutMs, uint64_t serverFlags, int *err)
{
    auto fail = [&](int code) -> StorePtr {
        if (err != nullptr) *err = code;
        return nullptr;
    };
    StoreUrl u;
    if (!StoreUrl::Parse(url, u)) {
        MF_FAIL(ERR_INVALID_PARAM, "bad store url %s", url.c_str());
        return fail(ERR_INVALID_PARAM);
    }
    std::unique_lock<std::mutex> g(g_mu);
    Entry &e = g_stores[url];
    if (e.client) {
        e.refs++;
        if (err != nullptr) *err = OK;
        return e.client;
    }
    if (u.scheme != StoreUrl::TCP) {
        BackendPtr backend;
        smem_conf_store_backend_op_t ops;
        if (GetExternalBackendOps(ops)) backend = std::make_shared<ExternalBackend>(ops, u.ip, u.instance);
        else if (u.scheme == StoreUrl::REG) backend = std::make_shared<LocalMemoryBackend>(u.ip, true);
        else {
            auto etcd = std::make_shared<EtcdBackend>(u.ip, u.port, u.instance);
            if (etcd->Connect() != OK) {
                g_stores.erase(url);
                MF_FAIL(ERR_NOT_CONNECTED, "etcd backend of %s: %s", url.c_str(), etcd->LastError().c_str());
                return fail(ERR_NOT_CONNECTED);
            }
            backend = etcd;
        }
        std::string ip = EnvStr("MF_CONFIG_STORE_IP", nullptr, "127.0.0.1");
        // the port of an etcd:// URL is etcd's own: the store leader listens elsewhere
        uint16_t port = (u.port != 0 && u.scheme != StoreUrl::ETCD) ? u.port : (uint16_t)EnvInt("MF_CONFIG_STORE_PORT", nullptr, 36100, 1024, 65000);
        auto ha = std::make_shared<HaConfigStore>(ip, port, worldSize, rank, backend, isServer);
        g.unlock();
        int rc = ha->Startup(timeoutMs);
        g.lock();
        if (rc != OK) {
            g_stores.erase(url);
            return fail(rc);
        }
        Entry &e2 = g_stores[url];
        e2.ha = ha;
        e2.client = ha;
        e2.refs = 1;
        if (err != nullptr) *err = OK;
        return ha;
    }
    if (isServer && !e.server) {
        auto s = std::make_shared<StoreServer>(u.ip, u.port, worldSize, serverFlags);
        int rc = s->Startup();
        if (rc == OK) e.server = s;
        else if (rc != ERR_IN_USE) {  // somebody else serving on that port is fine: we are a client then
            g_stores.erase(url);
            return fail(rc);
        }
    }
    auto c = std::make_shared<TcpStoreClient>(u.ip, u.port, worldSize, rank);
    g.unlock();
    int rc = c->Startup(timeoutMs);
    g.lock();
    Entry &e3 = g_stores[url];
    if (rc != OK) {
        if (e3.server) e3.server->Shutdown();
        g_stores.erase(url);
        return fail(rc);
    }
    e3.client = c;
    e3.refs = 1;
    if (err != nullptr) *err = OK;
    return c;
}

void StoreFactory::DestroyStore(const std::string &url)
{
    Entry e;
    {
        std::lock_guard<std::mutex> g(g_mu);
        auto it = g_stores.find(url);
        if (it == g_stores.end()) return;
        if (it->second.refs > 1) {
            it->second.refs--;
            return;
        }
        e = it->second;
        if (e.pinnedServer && !e.ha) {  // keep serving other processes; only this process's client goes
            it->second.client.reset();
            it->second.refs = 0;
            e.server.reset();
        } else {
            g_stores.erase(it);
        }
    }
    if (e.ha) e.ha->Shutdown();
    else if (e.client) std::static_pointer_cast<TcpStoreClient>(e.client)->Shutdown();
    if (e.server) e.server->Shutdown();
}

void StoreFactory::DestroyAll()
{
    std::map<std::string, Entry> all;
    {
        std::lock_guard<std::mutex> g(g_mu);
        all.swap(g_stores);
    }
    for (auto &kv : all) {
        if (kv.second.ha) kv.second.ha->Shutdown();
        else if (kv.second.client) std::static_pointer_cast<TcpStoreClient>(kv.second.client)->Shutdown();
        if (kv.second.server) kv.second.server->Shutdown();
    }
}

StorePtr StoreFactory::Prefixed(const StorePtr &base, const std::string &prefix)
{
    return std::make_shared<PrefixStore>(base, prefix);
}

}  // namespace store
}  // namespace mf
