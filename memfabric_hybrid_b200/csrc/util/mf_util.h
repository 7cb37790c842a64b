// Base utilities shared by every native layer: result codes, logger with external sink and alarm
// callbacks, per-thread last-error text, environment lookups with deprecated aliases, monotonic
// time, CRC32 and a small fixed-size thread pool.
//
// Parity: src/util/csrc/mf_out_logger.h, src/util/csrc/mf_env_define.h:40-66,
// src/smem/csrc/common/smem_last_error.h, src/smem/csrc/common/smem_thread_pool.cpp.
#pragma once
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <functional>
#include <future>
#include <memory>
#include <mutex>
#include <sstream>
#include <string>
#include <thread>
#include <vector>

namespace mf {

// Internal result codes. Store status values travel on the wire in the frame header `result`.
enum Result : int32_t {
    OK = 0,
    ERR = -1,
    ERR_INVALID_PARAM = -2000,
    ERR_MALLOC = -2001,
    ERR_NO_RESOURCES = -2002,
    ERR_NOT_STARTED = -2003,
    ERR_TIMEOUT = -2004,
    ERR_REPEAT = -2005,
    ERR_DUPLICATED = -2006,
    ERR_NOT_EXIST = -2007,
    ERR_NOT_INIT = -2008,
    ERR_IN_USE = -2009,
    ERR_BUSY = -2010,        // interrupted by a membership change: caller may retry
    ERR_RECONNECT = -2011,   // server in its recovery window: dial again later
    ERR_PARTIAL = -2012,
    ERR_NOT_CONNECTED = -2014,
};

// Status values carried in the store reply header.
enum StoreStatus : int16_t {
    ST_OK = 0,
    ST_ERROR = -1,
    ST_INVALID_MESSAGE = -400,
    ST_INVALID_KEY = -401,
    ST_NOT_EXIST = -404,
    ST_RESTORE = -405,
    ST_TIMEOUT = -601,
    ST_IO_ERROR = -602,
};

enum LogLevel : int { LOG_DEBUG = 0, LOG_INFO = 1, LOG_WARN = 2, LOG_ERROR = 3, LOG_OFF = 4 };

using ExternLogFn = void (*)(int level, const char *msg);
using ExternAlarmFn = void (*)(uint16_t code, const char *msg);
using ExternResumeFn = void (*)(uint16_t code);

class Logger {
public:
    static Logger &Get();
    void SetLevel(int lv) { level_.store(lv); }
    int Level() const { return level_.load(); }
    void SetSink(ExternLogFn fn) { sink_.store(fn); }
    void SetAlarm(ExternAlarmFn a, ExternResumeFn r) { alarm_.store(a); resume_.store(r); }
    void Alarm(uint16_t code, const char *msg);
    void Resume(uint16_t code);
    void Write(int lv, const char *file, int line, const char *fmt, ...) __attribute__((format(printf, 5, 6)));

private:
    Logger();
    std::atomic<int> level_{LOG_WARN};
    std::atomic<ExternLogFn> sink_{nullptr};
    std::atomic<ExternAlarmFn> alarm_{nullptr};
    std::atomic<ExternResumeFn> resume_{nullptr};
};

#define MF_LOG(lv, ...)                                                            \
    do {                                                                           \
        if ((lv) >= ::mf::Logger::Get().Level())                                   \
            ::mf::Logger::Get().Write((lv), __FILE__, __LINE__, __VA_ARGS__);      \
    } while (0)
#define MF_DEBUG(...) MF_LOG(::mf::LOG_DEBUG, __VA_ARGS__)
#define MF_INFO(...) MF_LOG(::mf::LOG_INFO, __VA_ARGS__)
#define MF_WARN(...) MF_LOG(::mf::LOG_WARN, __VA_ARGS__)
#define MF_ERROR(...) MF_LOG(::mf::LOG_ERROR, __VA_ARGS__)

// Per-thread last error (code + text); cleared by the *_and_clear accessor of the C API.
class LastError {
public:
    static void Set(int32_t code, const char *fmt, ...) __attribute__((format(printf, 2, 3)));
    static const char *Msg();
    static int32_t Code();
    static const char *TakeMsg();  // returns the text and clears it
    static void Clear();
};

// Records the failure in LastError, logs it and evaluates to the code.
int FailImpl(int32_t code, const char *file, int line, const char *fmt, ...) __attribute__((format(printf, 4, 5)));
#define MF_FAIL(code, ...) ::mf::FailImpl((code), __FILE__, __LINE__, __VA_ARGS__)

// Environment access. `alias` is a deprecated spelling: honoured with a one-time warning.
std::string EnvStr(const char *name, const char *alias = nullptr, const char *dflt = "");
int64_t EnvInt(const char *name, const char *alias, int64_t dflt, int64_t lo, int64_t hi);

inline uint64_t NowNs()
{
    return std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch())
        .count();
}
inline uint64_t NowMs() { return NowNs() / 1000000ULL; }

uint32_t Crc32(const void *data, size_t len, uint32_t seed = 0);

inline uint64_t AlignUp(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }
inline uint64_t AlignDown(uint64_t v, uint64_t a) { return v / a * a; }

// Fixed-size pool; Submit returns a future so batch copies can collect per-item results.
class ThreadPool {
public:
    explicit ThreadPool(size_t n, const char *name = "mf-pool");
    ~ThreadPool();
    template <typename F> auto Submit(F &&f) -> std::future<decltype(f())>
    {
        using R = decltype(f());
        auto task = std::make_shared<std::packaged_task<R()>>(std::forward<F>(f));
        auto fut = task->get_future();
        {
            std::lock_guard<std::mutex> g(mu_);
            q_.emplace_back([task] { (*task)(); });
        }
        cv_.notify_one();
        return fut;
    }
    size_t Size() const { return workers_.size(); }

private:
    std::mutex mu_;
    std::condition_variable cv_;
    std::deque<std::function<void()>> q_;
    std::vector<std::thread> workers_;
    bool stop_ = false;
};

// Joins a thread, unless the caller IS that thread (an object released from its own callback):
// then the thread is detached, since joining oneself throws.
inline void JoinOrDetach(std::thread &t)
{
    if (!t.joinable()) return;
    if (t.get_id() == std::this_thread::get_id()) t.detach();
    else t.join();
}

// Splits "a,b,c" on a delimiter, dropping empty pieces.
std::vector<std::string> Split(const std::string &s, char delim);
bool ParseU64(const std::string &s, uint64_t &out);
bool ParseI64(const std::string &s, int64_t &out);

}  // namespace mf
