// StoreMessage pack/unpack. See mf_store.h for the byte layout.
#include "mf_store.h"

namespace mf {
namespace store {

namespace {
inline void PutRaw(std::string &out, const void *p, size_t n) { out.append(static_cast<const char *>(p), n); }

struct Reader {
    const uint8_t *p;
    size_t left;
    template <typename T> bool Take(T &v)
    {
        if (left < sizeof(T)) return false;
        memcpy(&v, p, sizeof(T));
        p += sizeof(T);
        left -= sizeof(T);
        return true;
    }
    bool TakeBytes(uint64_t n, std::string &out)
    {
        if (left < n) return false;
        out.assign(reinterpret_cast<const char *>(p), n);
        p += n;
        left -= n;
        return true;
    }
};
}  // namespace

std::string StoreMessage::Pack() const
{
    uint64_t total = sizeof(uint64_t) + sizeof(int64_t) + sizeof(int16_t) + 2 * sizeof(uint64_t);
    for (auto &k : keys) total += sizeof(uint64_t) + k.size();
    for (auto &v : values) total += sizeof(uint64_t) + v.size();
    std::string out;
    out.reserve(total);
    PutRaw(out, &total, sizeof(total));
    PutRaw(out, &userDef, sizeof(userDef));
    int16_t t = mt;
    PutRaw(out, &t, sizeof(t));
    uint64_t n = keys.size();
    PutRaw(out, &n, sizeof(n));
    for (auto &k : keys) {
        uint64_t l = k.size();
        PutRaw(out, &l, sizeof(l));
        PutRaw(out, k.data(), k.size());
    }
    n = values.size();
    PutRaw(out, &n, sizeof(n));
    for (auto &v : values) {
        uint64_t l = v.size();
        PutRaw(out, &l, sizeof(l));
        PutRaw(out, v.data(), v.size());
    }
    return out;
}

bool StoreMessage::Unpack(const std::string &buf, StoreMessage &out) { return Unpack(buf.data(), buf.size(), out); }

bool StoreMessage::Unpack(const void *buf, size_t len, StoreMessage &out)
{
    Reader r{static_cast<const uint8_t *>(buf), len};
    uint64_t total = 0, n = 0;
    int16_t t = 0;
    if (!r.Take(total) || total != len) return false;
    if (!r.Take(out.userDef) || !r.Take(t)) return false;
    if (t < 0 || t >= MT_COUNT) return false;
    out.mt = static_cast<MsgType>(t);
    if (!r.Take(n) || n > kMaxKeys) return false;
    out.keys.clear();
    out.keys.reserve(n);
    for (uint64_t i = 0; i < n; i++) {
        uint64_t l = 0;
        std::string s;
        if (!r.Take(l) || l > kMaxKeyLen || !r.TakeBytes(l, s)) return false;
        out.keys.emplace_back(std::move(s));
    }
    if (!r.Take(n) || n > kMaxValues) return false;
    out.values.clear();
    out.values.reserve(n);
    for (uint64_t i = 0; i < n; i++) {
        uint64_t l = 0;
        std::string s;
        if (!r.Take(l) || l > kMaxValueLen || !r.TakeBytes(l, s)) return false;
        out.values.emplace_back(std::move(s));
    }
    return r.left == 0;
}

uint32_t HeartbeatMs()
{
    static uint32_t v = (uint32_t)EnvInt("MF_STORE_HEARTBEAT_MS", nullptr, 2000, 20, 60000);
    return v;
}

}  // namespace store
}  // namespace mf
