#include "mf_trace.h"

#include <fstream>
#include <sys/stat.h>
#include <unistd.h>

namespace mf {

static const char *kTpNames[TP_COUNT] = {
    "TP_STORE_SET",        "TP_STORE_GET",         "TP_STORE_CAS",       "TP_GROUP_BARRIER",  "TP_GROUP_ALLGATHER",
    "TP_GROUP_JOIN",       "TP_GROUP_LEAVE",       "TP_BM_CREATE",       "TP_BM_JOIN",        "TP_BM_COPY",
    "TP_BM_COPY_BATCH",    "TP_SHM_CREATE",        "TP_TRANS_REGISTER",  "TP_TRANS_BATCH_WRITE", "TP_TRANS_BATCH_READ",
    "TP_HYBM_RESERVE",     "TP_HYBM_ALLOC",        "TP_HYBM_EXPORT",     "TP_HYBM_IMPORT",    "TP_HYBM_MMAP",
    "TP_HYBM_LH_TO_LH",    "TP_HYBM_LH_TO_GH",     "TP_HYBM_GH_TO_LH",   "TP_HYBM_GH_TO_GH",  "TP_HYBM_LD_TO_GD",
    "TP_HYBM_GD_TO_LD",    "TP_HYBM_GD_TO_GD",     "TP_HYBM_LH_TO_GD",   "TP_HYBM_GD_TO_LH",  "TP_HYBM_LD_TO_GH",
    "TP_HYBM_GH_TO_LD",    "TP_HYBM_GD_TO_GH",     "TP_HYBM_GH_TO_GD",   "TP_HYBM_BATCH_KERNEL", "TP_HYBM_BATCH_HOST_LEG",
    "TP_HYBM_WAIT",        "TP_ZBAL_COLLECTIVE",
};

const char *TracePointName(uint32_t id) { return id < TP_COUNT ? kTpNames[id] : "TP_UNKNOWN"; }

namespace {
struct Cell {
    std::atomic<uint64_t> begin{0}, good{0}, bad{0}, total{0};
    std::atomic<uint64_t> mn{UINT64_MAX}, mx{0};
    std::atomic<uint64_t> hist[PTracer::kHistBuckets + 1] = {};
    std::atomic<uint64_t> histSum{0};
};
Cell g_cells[TP_COUNT];
Tracer g_tracer;
std::thread g_dumper;
std::mutex g_mu;
std::condition_variable g_cv;
bool g_run = false;
std::string g_path;
constexpr uint64_t kMaxFileBytes = 10ULL << 20;

void DefBegin(uint32_t id, uint64_t) { if (id < TP_COUNT) g_cells[id].begin.fetch_add(1, std::memory_order_relaxed); }
void DefEnd(uint32_t id, uint64_t t0, uint64_t t1, int32_t ret)
{
    if (id >= TP_COUNT) return;
    Cell &c = g_cells[id];
    uint64_t d = t1 > t0 ? t1 - t0 : 0;
    (ret == 0 ? c.good : c.bad).fetch_add(1, std::memory_order_relaxed);
    c.total.fetch_add(d, std::memory_order_relaxed);
    uint32_t b = 0;   // smallest i with d <= 1000 ns << i
    while (b < PTracer::kHistBuckets && d > (1000ULL << b)) b++;
    c.hist[b].fetch_add(1, std::memory_order_relaxed);
    c.histSum.fetch_add(d, std::memory_order_relaxed);
    uint64_t cur = c.mn.load(std::memory_order_relaxed);
    while (d < cur && !c.mn.compare_exchange_weak(cur, d)) {}
    cur = c.mx.load(std::memory_order_relaxed);
    while (d > cur && !c.mx.compare_exchange_weak(cur, d)) {}
}
}  // namespace

const Tracer &PTracer::Current() { return g_tracer; }
void PTracer::Install(const Tracer &t) { g_tracer = t; }
std::string PTracer::FilePath() { return g_path; }

PTracer::Row PTracer::Snapshot(uint32_t id)
{
    Row r{};
    if (id >= TP_COUNT) return r;
    Cell &c = g_cells[id];
    r.begin = c.begin.load();
    r.goodEnd = c.good.load();
    r.badEnd = c.bad.load();
    r.minNs = c.mn.load();
    r.maxNs = c.mx.load();
    r.totalNs = c.total.load();
    return r;
}

uint64_t PTracer::Histogram(uint32_t id, uint64_t counts[kHistBuckets + 1], uint64_t *sumNs)
{
    uint64_t n = 0;
    for (uint32_t i = 0; i <= kHistBuckets; i++) {
        counts[i] = id < TP_COUNT ? g_cells[id].hist[i].load(std::memory_order_relaxed) : 0;
        n += counts[i];
    }
    if (sumNs != nullptr) *sumNs = id < TP_COUNT ? g_cells[id].histSum.load(std::memory_order_relaxed) : 0;
    return n;
}

std::string PTracer::DumpTable(bool reset)
{
    char line[512];
    std::string out;
    time_t now = time(nullptr);
    struct tm tmv;
    localtime_r(&now, &tmv);
    char ts[32];
    strftime(ts, sizeof(ts), "%Y-%m-%d %H:%M:%S", &tmv);
    bool any = false;
    for (uint32_t i = 0; i < TP_COUNT; i++) {
        Cell &c = g_cells[i];
        uint64_t b = c.begin.load();
        if (b == 0) continue;
        if (!any) {
            snprintf(line, sizeof(line), "%-23s%-40s%-15s%-15s%-15s%-15s%-15s%-15s%-15s%-15s\n", "TIME", "NAME", "BEGIN",
                     "GOOD_END", "BAD_END", "ON_FLY", "MIN(us)", "MAX(us)", "AVG(us)", "TOTAL(us)");
            out += line;
            any = true;
        }
        uint64_t g = c.good.load(), bd = c.bad.load(), tot = c.total.load();
        uint64_t done = g + bd;
        double mn = c.mn.load() == UINT64_MAX ? 0.0 : c.mn.load() / 1000.0;
        snprintf(line, sizeof(line), "%-23s%-40s%-15lu%-15lu%-15lu%-15lu%-15.3f%-15.3f%-15.3f%-15.3f\n", ts, kTpNames[i],
                 (unsigned long)b, (unsigned long)g, (unsigned long)bd, (unsigned long)(b > done ? b - done : 0), mn,
                 c.mx.load() / 1000.0, done ? tot / 1000.0 / done : 0.0, tot / 1000.0);
        out += line;
        if (reset) {
            c.begin.store(b > done ? b - done : 0);
            c.good.store(0);
            c.bad.store(0);
            c.total.store(0);
            c.mn.store(UINT64_MAX);
            c.mx.store(0);
        }
    }
    return out;
}

int PTracer::Start(const std::string &dir, uint32_t periodMs)
{
    std::lock_guard<std::mutex> g(g_mu);
    if (g_run) return OK;
    std::string d = dir.empty() ? EnvStr("MF_PTRACER_DIR", nullptr, "/var/log/memfabric_hybrid") : dir;
    if (mkdir(d.c_str(), 0750) != 0 && errno != EEXIST) d = "/tmp";
    if (access(d.c_str(), W_OK) != 0) d = "/tmp";
    g_path = d + "/ptracer_" + std::to_string(getpid()) + ".dat";
    g_tracer.begin = DefBegin;
    g_tracer.end = DefEnd;
    g_tracer.enabled = true;
    g_run = true;
    uint32_t period = periodMs == 0 ? 10000 : periodMs;
    g_dumper = std::thread([period] {
        pthread_setname_np(pthread_self(), "mf-ptracer");
        std::unique_lock<std::mutex> lk(g_mu);
        while (g_run) {
            g_cv.wait_for(lk, std::chrono::milliseconds(period));
            std::string tbl = DumpTable(true);
            if (tbl.empty()) continue;
            struct stat st;
            bool trunc = stat(g_path.c_str(), &st) == 0 && (uint64_t)st.st_size > kMaxFileBytes;
            std::ofstream f(g_path, trunc ? std::ios::trunc : std::ios::app);
            f << tbl;
        }
    });
    return OK;
}

void PTracer::Stop()
{
    {
        std::lock_guard<std::mutex> g(g_mu);
        if (!g_run) return;
        g_run = false;
        g_tracer.enabled = false;
    }
    g_cv.notify_all();
    if (g_dumper.joinable()) g_dumper.join();
}

// ---------------------------------------------------------------------------------------------
namespace {
struct Point {
    FipCallback cb = nullptr;
    bool registered = false;
    bool active = false;
    FipType type = FipType::CALLBACK;
    int32_t hits = 0;  // remaining hits; <0 = unlimited
    int64_t param = 0;
};
std::shared_mutex g_fmu;
std::map<std::string, Point> g_points;
std::string g_conf;
time_t g_confMtime = 0;
off_t g_confSize = -1;
std::atomic<bool> g_fipInit{false};
std::atomic<uint64_t> g_lastCheckMs{0};

void DefaultFailCb(FipParam *p, int32_t *ret)
{
    if (ret != nullptr) *ret = p->value != 0 ? (int32_t)p->value : -1;
    p->skipBlock = true;
}
}  // namespace

std::string FaultPoints::ConfPath() { return g_conf; }

void FaultPoints::Init(const std::string &confPath)
{
    std::unique_lock<std::shared_mutex> g(g_fmu);
    g_conf = confPath.empty() ? "/tmp/mf_failpoints_" + std::to_string(getpid()) + ".conf" : confPath;
    g_confMtime = 0;
    g_confSize = -1;
    g_fipInit = true;
}

void FaultPoints::Exit()
{
    std::unique_lock<std::shared_mutex> g(g_fmu);
    g_points.clear();
    g_fipInit = false;
}

int FaultPoints::Register(const std::string &name, FipCallback cb)
{
    std::unique_lock<std::shared_mutex> g(g_fmu);
    Point &p = g_points[name];  // keeps an activation that was read from the file before registration
    p.cb = cb;
    p.registered = true;
    return 0;
}

int FaultPoints::Unregister(const std::string &name)
{
    std::unique_lock<std::shared_mutex> g(g_fmu);
    return g_points.erase(name) ? 0 : 3;
}

int FaultPoints::Activate(const std::string &name, FipType type, int32_t hits, int64_t param)
{
    std::unique_lock<std::shared_mutex> g(g_fmu);
    Point &p = g_points[name];
    p.active = true;
    p.type = type;
    p.hits = hits;
    p.param = param;
    return 0;
}

int FaultPoints::Deactivate(const std::string &name)
{
    std::unique_lock<std::shared_mutex> g(g_fmu);
    auto it = g_points.find(name);
    if (it == g_points.end()) return 3;
    it->second.active = false;
    return 0;
}

void FaultPoints::DeactivateAll()
{
    std::unique_lock<std::shared_mutex> g(g_fmu);
    for (auto &kv : g_points) kv.second.active = false;
}

bool FaultPoints::IsActive(const std::string &name)
{
    std::shared_lock<std::shared_mutex> g(g_fmu);
    auto it = g_points.find(name);
    return it != g_points.end() && it->second.active && it->second.hits != 0;
}

void FaultPoints::Reload()
{
    if (!g_fipInit) return;
    struct stat st;
    std::string path;
    {
        std::shared_lock<std::shared_mutex> g(g_fmu);
        path = g_conf;
    }
    if (stat(path.c_str(), &st) != 0) {
        std::unique_lock<std::shared_mutex> g(g_fmu);
        if (g_confSize >= 0) {  // file removed: clear file-driven activations
            for (auto &kv : g_points) kv.second.active = false;
            g_confSize = -1;
            g_confMtime = 0;
        }
        return;
    }
    {
        std::shared_lock<std::shared_mutex> g(g_fmu);
        if (st.st_mtime == g_confMtime && st.st_size == g_confSize) return;
    }
    std::ifstream f(path);
    std::string line;
    std::map<std::string, Point> parsed;
    while (std::getline(f, line)) {
        if (line.empty() || line[0] == '#') continue;
        std::istringstream is(line);
        std::string name, type;
        int32_t hits = -1;
        int64_t param = 0;
        if (!(is >> name >> type)) continue;
        is >> hits;
        is >> param;
        Point p;
        p.active = true;
        p.hits = hits;
        p.param = param;
        if (type == "callback") p.type = FipType::CALLBACK;
        else if (type == "pause") p.type = FipType::PAUSE;
        else if (type == "reset") p.type = FipType::RESET;
        else if (type == "abort") p.type = FipType::ABORT;
        else continue;
        parsed[name] = p;
    }
    std::unique_lock<std::shared_mutex> g(g_fmu);
    for (auto &kv : g_points) kv.second.active = false;
    for (auto &kv : parsed) {
        Point &p = g_points[kv.first];
        p.active = true;
        p.type = kv.second.type;
        p.hits = kv.second.hits;
        p.param = kv.second.param;
    }
    g_confMtime = st.st_mtime;
    g_confSize = st.st_size;
}

bool FaultPoints::Begin(const char *name, int32_t *ret)
{
    if (!g_fipInit.load(std::memory_order_relaxed)) return false;
    uint64_t now = NowMs();
    uint64_t last = g_lastCheckMs.load();
    if (now - last >= 200 && g_lastCheckMs.compare_exchange_strong(last, now)) Reload();
    FipCallback cb = nullptr;
    FipType type;
    FipParam param;
    {
        std::unique_lock<std::shared_mutex> g(g_fmu);
        auto it = g_points.find(name);
        if (it == g_points.end() || !it->second.active || !it->second.registered || it->second.hits == 0) return false;
        Point &p = it->second;
        if (p.hits > 0) p.hits--;
        type = p.type;
        cb = p.cb;
        param.value = p.param;
        if (type == FipType::RESET) p.active = false;
    }
    switch (type) {
        case FipType::CALLBACK:
            (cb != nullptr ? cb : DefaultFailCb)(&param, ret);
            return param.skipBlock;
        case FipType::PAUSE:
            std::this_thread::sleep_for(std::chrono::milliseconds(param.value > 0 ? param.value : 100));
            return false;
        case FipType::RESET:
            return false;
        case FipType::ABORT:
            MF_ERROR("fault point %s: abort requested", name);
            abort();
    }
    return false;
}

void FaultPoints::RegisterBuiltins()
{
    if (!g_fipInit) Init();
    for (const char *n : {"ALLOC_LOCAL_MEMORY", "MMAP", "IMPORT", "STORE_CONNECT"}) Register(n, DefaultFailCb);
}

void FaultPoints::UnregisterBuiltins()
{
    for (const char *n : {"ALLOC_LOCAL_MEMORY", "MMAP", "IMPORT", "STORE_CONNECT"}) Unregister(n);
}

}  // namespace mf
