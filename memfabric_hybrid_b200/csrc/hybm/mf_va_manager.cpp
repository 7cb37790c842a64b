#include "mf_hybm_types.h"

namespace mf {
namespace hybm {

uint64_t WindowBase(hybm_mem_type t, uint32_t entityId, uint32_t attempt)
{
    // MF_GVA_DRAM_BASE / MF_GVA_HBM_BASE move a space (every process of the job must be given the same value): for
    // address spaces in which the defaults are taken, e.g. under ThreadSanitizer, whose shadow memory covers them.
    static const uint64_t dramBase = (uint64_t)EnvInt("MF_GVA_DRAM_BASE", nullptr, (int64_t)kDramWindowBase, 1LL << 32, 1LL << 47);
    static const uint64_t hbmBase = (uint64_t)EnvInt("MF_GVA_HBM_BASE", nullptr, (int64_t)kHbmWindowBase, 1LL << 32, 1LL << 47);
    uint64_t base = t == HYBM_MEM_TYPE_HOST ? dramBase : hbmBase;
    // A retry after a collision moves to another of the 64 windows, the same one in every process.
    uint32_t window = (entityId + attempt * 17u) % (kMaxEntityId + 1);
    return base + (uint64_t)window * kWindowStride;
}

uint64_t Gva56WindowBase(hybm_mem_type t, uint32_t entityId, uint32_t attempt)
{
    const uint32_t half = kGva56Windows / 2;
    return kGva56Base + (uint64_t)((entityId + attempt * 17u) % half + (t == HYBM_MEM_TYPE_HOST ? 0 : half)) * kGva56WindowStride;
}

uint64_t CompactSlot(uint32_t ranks)
{
    uint64_t per = kCompactThreshold / (ranks == 0 ? 1 : ranks), slot = 2ULL << 20;
    while (slot * 2 <= per) slot *= 2;
    return slot;
}

VaManager &VaManager::Get()
{
    static VaManager inst;
    return inst;
}

int VaManager::AddReserved(const ReservedRange &r)
{
    if (r.slot == 0 || r.ranks == 0) return ERR_INVALID_PARAM;
    std::unique_lock<std::shared_mutex> g(mu_);
    for (auto &kv : reserved_) {
        if (r.base < kv.second.End() && kv.second.base < r.End())
            return MF_FAIL(ERR_IN_USE, "GVA range %#lx+%#lx overlaps a reserved range at %#lx", (unsigned long)r.base,
                           (unsigned long)(r.slot * r.ranks), (unsigned long)kv.second.base);
    }
    reserved_[r.base] = r;
    return OK;
}

void VaManager::RemoveReserved(uint64_t base)
{
    std::unique_lock<std::shared_mutex> g(mu_);
    reserved_.erase(base);
}

bool VaManager::Locate(uint64_t va, ReservedRange &out, uint32_t &rank) const
{
    std::shared_lock<std::shared_mutex> g(mu_);
    auto it = reserved_.upper_bound(va);
    if (it == reserved_.begin()) return false;
    --it;
    if (va >= it->second.End()) return false;
    out = it->second;
    rank = (uint32_t)((va - out.base) / out.slot);
    return true;
}

void VaManager::AddLocal(uint64_t va, uint64_t size, bool device)
{
    std::unique_lock<std::shared_mutex> g(mu_);
    locals_[va] = Local{size, device};
}

void VaManager::RemoveLocal(uint64_t va)
{
    std::unique_lock<std::shared_mutex> g(mu_);
    locals_.erase(va);
}

uint8_t VaManager::Classify(uint64_t va, uint64_t len) const
{
    std::shared_lock<std::shared_mutex> g(mu_);
    auto it = reserved_.upper_bound(va);
    if (it != reserved_.begin()) {
        auto p = std::prev(it);
        if (va < p->second.End()) {
            if (va + len > p->second.End()) return AC_NONE;  // straddles the end of the pool
            return p->second.type == HYBM_MEM_TYPE_HOST ? AC_GH : AC_GD;
        }
    }
    auto lt = locals_.upper_bound(va);
    if (lt != locals_.begin()) {
        auto p = std::prev(lt);
        if (va + len <= p->first + p->second.size) return p->second.device ? AC_LD : AC_LH;
    }
    return AC_NONE;
}

namespace {
struct DirRow {
    uint8_t src, dst;
    hybm_data_copy_direction dir;
};
const DirRow kDirs[] = {
    {AC_LH, AC_GH, HYBM_LOCAL_HOST_TO_GLOBAL_HOST},     {AC_LH, AC_GD, HYBM_LOCAL_HOST_TO_GLOBAL_DEVICE},
    {AC_LD, AC_GH, HYBM_LOCAL_DEVICE_TO_GLOBAL_HOST},   {AC_LD, AC_GD, HYBM_LOCAL_DEVICE_TO_GLOBAL_DEVICE},
    {AC_GH, AC_GH, HYBM_GLOBAL_HOST_TO_GLOBAL_HOST},    {AC_GH, AC_GD, HYBM_GLOBAL_HOST_TO_GLOBAL_DEVICE},
    {AC_GH, AC_LH, HYBM_GLOBAL_HOST_TO_LOCAL_HOST},     {AC_GH, AC_LD, HYBM_GLOBAL_HOST_TO_LOCAL_DEVICE},
    {AC_GD, AC_GH, HYBM_GLOBAL_DEVICE_TO_GLOBAL_HOST},  {AC_GD, AC_GD, HYBM_GLOBAL_DEVICE_TO_GLOBAL_DEVICE},
    {AC_GD, AC_LH, HYBM_GLOBAL_DEVICE_TO_LOCAL_HOST},   {AC_GD, AC_LD, HYBM_GLOBAL_DEVICE_TO_LOCAL_DEVICE},
};
// 256-entry table indexed by (srcClass << 4 | dstClass); built once.
struct DirLut {
    hybm_data_copy_direction t[256];
    DirLut()
    {
        for (auto &d : t) d = HYBM_DATA_COPY_DIRECTION_BUTT;
        for (auto &r : kDirs) t[(r.src << 4) | r.dst] = r.dir;
    }
};
const DirLut &Lut()
{
    static DirLut l;
    return l;
}
}  // namespace

hybm_data_copy_direction VaManager::DirectionOf(uint8_t s, uint8_t d)
{
    if (s > 15 || d > 15) return HYBM_DATA_COPY_DIRECTION_BUTT;
    return Lut().t[(s << 4) | d];
}

bool VaManager::DirectionMatches(hybm_data_copy_direction dir, uint8_t s, uint8_t d)
{
    for (auto &r : kDirs) {
        if (r.dir != dir) continue;
        // An unknown (AC_NONE) side is accepted as the local side the caller named.
        bool sOk = s == r.src || (s == AC_NONE && (r.src == AC_LH || r.src == AC_LD));
        bool dOk = d == r.dst || (d == AC_NONE && (r.dst == AC_LH || r.dst == AC_LD));
        return sOk && dOk;
    }
    return false;
}

std::string VaManager::Dump() const
{
    std::shared_lock<std::shared_mutex> g(mu_);
    std::ostringstream os;
    for (auto &kv : reserved_)
        os << "reserved " << std::hex << kv.second.base << "-" << kv.second.End() << std::dec << " slot " << kv.second.slot
           << " ranks " << kv.second.ranks << (kv.second.type == HYBM_MEM_TYPE_HOST ? " DRAM" : " HBM") << " entity "
           << kv.second.entityId << "\n";
    for (auto &kv : locals_)
        os << "local " << std::hex << kv.first << std::dec << " size " << kv.second.size << (kv.second.device ? " device" : " host") << "\n";
    return os.str();
}

const char *ErrorString(int32_t code)
{
    switch (code) {
        case BM_OK: return "ok";
        case BM_ERROR: return "error";
        case BM_INVALID_PARAM: return "invalid parameter";
        case BM_MALLOC_FAILED: return "allocation failed";
        case BM_NEW_OBJECT_FAILED: return "object creation failed";
        case BM_FILE_NOT_ACCESS: return "file not accessible";
        case BM_DL_FUNCTION_FAILED: return "backend library call failed";
        case BM_TIMEOUT: return "timeout";
        case BM_UNDER_API_UNLOAD: return "backend library not loaded";
        case BM_NOT_INITIALIZED: return "not initialized";
        case BM_NOT_SUPPORT_FUNC: return "function not supported";
        case BM_NOT_SUPPORTED: return "not supported";
        case BM_NOT_CONNECTED: return "not connected";
        default: return "unknown error";
    }
}

}  // namespace hybm
}  // namespace mf
