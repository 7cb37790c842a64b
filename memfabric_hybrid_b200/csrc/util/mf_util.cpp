#include "mf_util.h"

#include <ctime>
#include <sys/syscall.h>
#include <unistd.h>

namespace mf {

Logger::Logger()
{
    // MF_LOG_LEVEL is honoured at start-up so tools that never call set_log_level can be made verbose.
    const char *e = getenv("MF_LOG_LEVEL");
    if (e != nullptr && *e != 0) {
        int v = atoi(e);
        if (v >= LOG_DEBUG && v <= LOG_OFF) level_.store(v);
    }
}

Logger &Logger::Get()
{
    static Logger inst;
    return inst;
}

void Logger::Alarm(uint16_t code, const char *msg)
{
    auto fn = alarm_.load();
    if (fn != nullptr) fn(code, msg);
}

void Logger::Resume(uint16_t code)
{
    auto fn = resume_.load();
    if (fn != nullptr) fn(code);
}

void Logger::Write(int lv, const char *file, int line, const char *fmt, ...)
{
    char body[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(body, sizeof(body), fmt, ap);
    va_end(ap);
    const char *base = strrchr(file, '/');
    base = base ? base + 1 : file;
    char full[1200];
    auto sink = sink_.load();
    if (sink != nullptr) {
        snprintf(full, sizeof(full), "[%s:%d] %s", base, line, body);
        sink(lv, full);
        return;
    }
    static const char *names[] = {"DEBUG", "INFO", "WARN", "ERROR"};
    struct timespec ts;
    clock_gettime(CLOCK_REALTIME, &ts);
    struct tm tmv;
    localtime_r(&ts.tv_sec, &tmv);
    snprintf(full, sizeof(full), "%02d:%02d:%02d.%03ld %d/%ld %s [%s:%d] %s\n", tmv.tm_hour, tmv.tm_min, tmv.tm_sec,
             ts.tv_nsec / 1000000, (int)getpid(), (long)syscall(SYS_gettid), names[lv < 0 ? 0 : (lv > 3 ? 3 : lv)], base,
             line, body);
    fputs(full, lv >= LOG_WARN ? stderr : stdout);
}

namespace {
struct ErrSlot {
    int32_t code = 0;
    std::string msg;
    std::string taken;
};
thread_local ErrSlot g_err;
}  // namespace

void LastError::Set(int32_t code, const char *fmt, ...)
{
    char body[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(body, sizeof(body), fmt, ap);
    va_end(ap);
    g_err.code = code;
    g_err.msg = body;
}
int FailImpl(int32_t code, const char *file, int line, const char *fmt, ...)
{
    char body[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(body, sizeof(body), fmt, ap);
    va_end(ap);
    g_err.code = code;
    g_err.msg = body;
    if (LOG_ERROR >= Logger::Get().Level()) Logger::Get().Write(LOG_ERROR, file, line, "%s", body);
    return code;
}
const char *LastError::Msg() { return g_err.msg.c_str(); }
int32_t LastError::Code() { return g_err.code; }
const char *LastError::TakeMsg()
{
    g_err.taken.swap(g_err.msg);
    g_err.msg.clear();
    g_err.code = 0;
    return g_err.taken.c_str();
}
void LastError::Clear()
{
    g_err.msg.clear();
    g_err.code = 0;
}

std::string EnvStr(const char *name, const char *alias, const char *dflt)
{
    const char *v = getenv(name);
    if (v != nullptr && *v != 0) return v;
    if (alias != nullptr) {
        v = getenv(alias);
        if (v != nullptr && *v != 0) {
            static std::atomic<int> warned{0};
            if (warned.fetch_add(1) < 8) MF_WARN("environment variable %s is deprecated, use %s", alias, name);
            return v;
        }
    }
    return dflt;
}

int64_t EnvInt(const char *name, const char *alias, int64_t dflt, int64_t lo, int64_t hi)
{
    std::string s = EnvStr(name, alias, "");
    if (s.empty()) return dflt;
    int64_t v = 0;
    if (!ParseI64(s, v) || v < lo || v > hi) {
        MF_WARN("environment variable %s=%s out of range [%ld,%ld], using %ld", name, s.c_str(), (long)lo, (long)hi,
                (long)dflt);
        return dflt;
    }
    return v;
}

uint32_t Crc32(const void *data, size_t len, uint32_t seed)
{
    static uint32_t table[256];
    static std::once_flag once;
    std::call_once(once, [] {
        for (uint32_t i = 0; i < 256; i++) {
            uint32_t c = i;
            for (int k = 0; k < 8; k++) c = (c & 1) ? (0xEDB88320u ^ (c >> 1)) : (c >> 1);
            table[i] = c;
        }
    });
    uint32_t c = ~seed;
    const uint8_t *p = static_cast<const uint8_t *>(data);
    for (size_t i = 0; i < len; i++) c = table[(c ^ p[i]) & 0xff] ^ (c >> 8);
    return ~c;
}

ThreadPool::ThreadPool(size_t n, const char *name)
{
    for (size_t i = 0; i < n; i++) {
        workers_.emplace_back([this, name, i] {
            char tn[16];
            snprintf(tn, sizeof(tn), "%.10s-%zu", name, i);
            pthread_setname_np(pthread_self(), tn);
            for (;;) {
                std::function<void()> job;
                {
                    std::unique_lock<std::mutex> lk(mu_);
                    cv_.wait(lk, [this] { return stop_ || !q_.empty(); });
                    if (stop_ && q_.empty()) return;
                    job = std::move(q_.front());
                    q_.pop_front();
                }
                job();
            }
        });
    }
}

ThreadPool::~ThreadPool()
{
    {
        std::lock_guard<std::mutex> g(mu_);
        stop_ = true;
    }
    cv_.notify_all();
    for (auto &t : workers_) t.join();
}

std::vector<std::string> Split(const std::string &s, char delim)
{
    std::vector<std::string> out;
    size_t pos = 0;
    while (pos <= s.size()) {
        size_t e = s.find(delim, pos);
        if (e == std::string::npos) e = s.size();
        if (e > pos) out.emplace_back(s.substr(pos, e - pos));
        pos = e + 1;
    }
    return out;
}

bool ParseU64(const std::string &s, uint64_t &out)
{
    if (s.empty() || s[0] == '-') return false;
    char *end = nullptr;
    errno = 0;
    unsigned long long v = strtoull(s.c_str(), &end, 10);
    if (errno != 0 || end == s.c_str() || *end != 0) return false;
    out = v;
    return true;
}

bool ParseI64(const std::string &s, int64_t &out)
{
    if (s.empty()) return false;
    char *end = nullptr;
    errno = 0;
    long long v = strtoll(s.c_str(), &end, 10);
    if (errno != 0 || end == s.c_str() || *end != 0) return false;
    out = v;
    return true;
}

}  // namespace mf
