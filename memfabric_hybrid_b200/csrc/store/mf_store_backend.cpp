#include "mf_store_backend.h"

namespace mf {
namespace store {

struct LocalMemoryBackend::Shared {
    std::mutex mu;
    std::condition_variable cv;
    struct Entry {
        std::string value;
        uint64_t expireMs = 0;  // 0 = never
    };
    std::map<std::string, Entry> kv;
    std::set<std::string> locks;
    bool reachable = true;
};

namespace {
std::mutex g_regMu;
std::map<std::string, std::shared_ptr<LocalMemoryBackend::Shared>> *g_reg = nullptr;
smem_conf_store_backend_op_t g_extOps;
bool g_extSet = false;
}  // namespace

static std::shared_ptr<LocalMemoryBackend::Shared> SharedOf(const std::string &name);

LocalMemoryBackend::LocalMemoryBackend(const std::string &name, bool pretendDistributed)
    : s_(SharedOf(name)), distributed_(pretendDistributed)
{
}

static std::shared_ptr<LocalMemoryBackend::Shared> SharedOf(const std::string &name)
{
    std::lock_guard<std::mutex> g(g_regMu);
    if (g_reg == nullptr) g_reg = new std::map<std::string, std::shared_ptr<LocalMemoryBackend::Shared>>();
    auto &slot = (*g_reg)[name];
    if (!slot) slot = std::make_shared<LocalMemoryBackend::Shared>();
    return slot;
}

void LocalMemoryBackend::SetReachable(const std::string &name, bool reachable)
{
    auto s = SharedOf(name);
    std::lock_guard<std::mutex> g(s->mu);
    s->reachable = reachable;
}

void LocalMemoryBackend::Reset(const std::string &name)
{
    auto s = SharedOf(name);
    std::lock_guard<std::mutex> g(s->mu);
    s->kv.clear();
    s->locks.clear();
    s->reachable = true;
    s->cv.notify_all();
}

int LocalMemoryBackend::Connect()
{
    std::lock_guard<std::mutex> g(s_->mu);
    return s_->reachable ? OK : ERR_NOT_CONNECTED;
}

int LocalMemoryBackend::Put(const std::string &key, const std::string &value, uint32_t ttlMs)
{
    std::lock_guard<std::mutex> g(s_->mu);
    if (!s_->reachable) return ERR_NOT_CONNECTED;
    auto &e = s_->kv[key];
    e.value = value;
    e.expireMs = ttlMs == 0 ? 0 : NowMs() + ttlMs;
    return OK;
}

int LocalMemoryBackend::Get(const std::string &key, std::string &value)
{
    std::lock_guard<std::mutex> g(s_->mu);
    if (!s_->reachable) return ERR_NOT_CONNECTED;
    auto it = s_->kv.find(key);
    if (it == s_->kv.end()) return ERR_NOT_EXIST;
    if (it->second.expireMs != 0 && NowMs() >= it->second.expireMs) {
        s_->kv.erase(it);
        return ERR_NOT_EXIST;
    }
    value = it->second.value;
    return OK;
}

int LocalMemoryBackend::PrefixGet(const std::string &prefix, std::vector<std::pair<std::string, std::string>> &out)
{
    std::lock_guard<std::mutex> g(s_->mu);
    if (!s_->reachable) return ERR_NOT_CONNECTED;
    uint64_t now = NowMs();
    for (auto it = s_->kv.lower_bound(prefix); it != s_->kv.end() && it->first.compare(0, prefix.size(), prefix) == 0; ++it) {
        if (it->second.expireMs != 0 && now >= it->second.expireMs) continue;
        out.emplace_back(it->first, it->second.value);
    }
    return OK;
}

int LocalMemoryBackend::Delete(const std::string &key)
{
    std::lock_guard<std::mutex> g(s_->mu);
    if (!s_->reachable) return ERR_NOT_CONNECTED;
    return s_->kv.erase(key) ? OK : ERR_NOT_EXIST;
}

int LocalMemoryBackend::Clear(const std::string &prefix)
{
    std::lock_guard<std::mutex> g(s_->mu);
    if (!s_->reachable) return ERR_NOT_CONNECTED;
    for (auto it = s_->kv.lower_bound(prefix); it != s_->kv.end() && it->first.compare(0, prefix.size(), prefix) == 0;)
        it = s_->kv.erase(it);
    return OK;
}

int LocalMemoryBackend::Lock(const std::string &name)
{
    std::unique_lock<std::mutex> lk(s_->mu);
    if (!s_->reachable) return ERR_NOT_CONNECTED;
    bool ok = s_->cv.wait_for(lk, std::chrono::seconds(30), [&] { return !s_->reachable || s_->locks.count(name) == 0; });
    if (!ok) return ERR_TIMEOUT;
    if (!s_->reachable) return ERR_NOT_CONNECTED;
    s_->locks.insert(name);
    return OK;
}

int LocalMemoryBackend::TryLock(const std::string &name)
{
    std::lock_guard<std::mutex> g(s_->mu);
    if (!s_->reachable) return ERR_NOT_CONNECTED;
    if (s_->locks.count(name)) return ERR_IN_USE;
    s_->locks.insert(name);
    return OK;
}

int LocalMemoryBackend::Unlock(const std::string &name)
{
    std::lock_guard<std::mutex> g(s_->mu);
    s_->locks.erase(name);
    s_->cv.notify_all();
    return OK;
}

// ---------------------------------------------------------------------------------------------
int SetExternalBackendOps(const smem_conf_store_backend_op_t *ops)
{
    std::lock_guard<std::mutex> g(g_regMu);
    if (ops == nullptr) {
        g_extSet = false;
        return OK;
    }
    if (ops->create == nullptr || ops->destroy == nullptr || ops->put == nullptr || ops->get == nullptr ||
        ops->remove == nullptr)
        return ERR_INVALID_PARAM;
    g_extOps = *ops;
    g_extSet = true;
    return OK;
}

bool GetExternalBackendOps(smem_conf_store_backend_op_t &ops)
{
    std::lock_guard<std::mutex> g(g_regMu);
    if (!g_extSet) return false;
    ops = g_extOps;
    return true;
}

ExternalBackend::ExternalBackend(const smem_conf_store_backend_op_t &ops, const std::string &name,
                                 const std::string &prefix)
    : ops_(ops), name_(name), prefix_(prefix)
{
}

ExternalBackend::~ExternalBackend()
{
    if (handle_ != nullptr) ops_.destroy(handle_);
}

bool ExternalBackend::Distributed() const { return ops_.distributed != nullptr && ops_.distributed(0); }

int ExternalBackend::Connect()
{
    if (handle_ != nullptr) return OK;
    int rc = ops_.create(name_.c_str(), prefix_.c_str(), 0, &handle_);
    if (rc != 0 || handle_ == nullptr) {
        handle_ = nullptr;
        return MF_FAIL(ERR_NOT_CONNECTED, "external store backend create(%s) failed: %d", name_.c_str(), rc);
    }
    return OK;
}

static int MapExt(int rc)
{
    switch (rc) {
        case SMEM_STORE_BACKEND_CODE_OK: return OK;
        case SMEM_STORE_BACKEND_CODE_NOENT: return ERR_NOT_EXIST;
        case SMEM_STORE_BACKEND_CODE_LOCKED: return ERR_IN_USE;
        case SMEM_STORE_BACKEND_CODE_INVAL: return ERR_INVALID_PARAM;
        case SMEM_STORE_BACKEND_CODE_NORES: return ERR_NO_RESOURCES;
        default: return ERR;
    }
}

int ExternalBackend::Put(const std::string &key, const std::string &value, uint32_t ttlMs)
{
    if (Connect() != OK) return ERR_NOT_CONNECTED;
    // The op table has no TTL argument; the lease length in seconds travels in `flags` (0 = no expiry).
    return MapExt(ops_.put(handle_, key.c_str(), value.data(), value.size(), (ttlMs + 999) / 1000));
}

int ExternalBackend::Get(const std::string &key, std::string &value)
{
    if (Connect() != OK) return ERR_NOT_CONNECTED;
    std::string buf(4096, '\0');
    uint64_t size = 0;
    int rc = ops_.get(handle_, key.c_str(), &buf[0], buf.size(), 0, &size);
    if (rc == SMEM_STORE_BACKEND_CODE_BUFEX && size > buf.size()) {
        buf.resize(size);
        rc = ops_.get(handle_, key.c_str(), &buf[0], buf.size(), 0, &size);
    }
    if (rc != 0) return MapExt(rc);
    buf.resize(size);
    value.swap(buf);
    return OK;
}

int ExternalBackend::PrefixGet(const std::string &prefix, std::vector<std::pair<std::string, std::string>> &out)
{
    if (Connect() != OK) return ERR_NOT_CONNECTED;
    if (ops_.prefix_get == nullptr) return ERR;
    smem_store_prefix_get_ctx_t ctx;
    ctx.prefix = prefix.c_str();
    ctx.marker = "";
    ctx.context = &out;
    ctx.fill = [](const char *key, const void *value, uint64_t size, void *c) -> bool {
        auto *v = static_cast<std::vector<std::pair<std::string, std::string>> *>(c);
        v->emplace_back(key, std::string(static_cast<const char *>(value), size));
        return true;
    };
    return MapExt(ops_.prefix_get(handle_, &ctx, 0));
}

int ExternalBackend::Delete(const std::string &key)
{
    if (Connect() != OK) return ERR_NOT_CONNECTED;
    return MapExt(ops_.remove(handle_, key.c_str(), 0));
}

int ExternalBackend::Clear(const std::string &prefix)
{
    std::vector<std::pair<std::string, std::string>> all;
    int rc = PrefixGet(prefix, all);
    if (rc != OK) return rc;
    for (auto &kv : all) Delete(kv.first);
    return OK;
}

int ExternalBackend::Lock(const std::string &name)
{
    if (Connect() != OK) return ERR_NOT_CONNECTED;
    return ops_.lock ? MapExt(ops_.lock(handle_, name.c_str(), 0)) : ERR;
}

int ExternalBackend::TryLock(const std::string &name)
{
    if (Connect() != OK) return ERR_NOT_CONNECTED;
    return ops_.try_lock ? MapExt(ops_.try_lock(handle_, name.c_str(), 0)) : ERR;
}

int ExternalBackend::Unlock(const std::string &name)
{
    if (Connect() != OK) return ERR_NOT_CONNECTED;
    return ops_.unlock ? MapExt(ops_.unlock(handle_, name.c_str(), 0)) : ERR;
}

}  // namespace store
}  // namespace mf
