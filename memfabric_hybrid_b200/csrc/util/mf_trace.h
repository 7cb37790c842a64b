// Host trace points and fault-injection points.
//
// Trace points: MF_TRACE_BEGIN(id) / MF_TRACE_END(id, ret) bracket an operation; a pluggable tracer
// receives begin/end. The default tracer keeps BEGIN / GOOD_END / BAD_END / ON_FLY / MIN / MAX / AVG /
// TOTAL per point and a thread writes the table every period to ptracer_<pid>.dat (size capped).
// Parity: src/util/csrc/ptracer/include/ptracer.h:15-56, src/util/csrc/ptracer/tracers/ptracer_default.h,
// table format of doc/ptracer.md:19-39.
//
// Fault points: MF_FIP_START(NAME, &ret) { real code } MF_FIP_END. An active point can run a callback
// that rewrites `ret` and skips the block, pause for N ms, reset (deactivate itself) or abort the
// process, with a hit budget. Points are activated by API or by a config file
// "<name> <type> <hits> [param]" that is reloaded when its mtime changes.
// Parity: src/util/csrc/mf_fault_injection_point.h:30-192, doc/fault_injection.md.
#pragma once
#include <map>
#include <shared_mutex>

#include "mf_util.h"

namespace mf {

// Trace point identifiers. Names are printed in the table.
enum TracePoint : uint32_t {
    TP_STORE_SET = 0,
    TP_STORE_GET,
    TP_STORE_CAS,
    TP_GROUP_BARRIER,
    TP_GROUP_ALLGATHER,
    TP_GROUP_JOIN,
    TP_GROUP_LEAVE,
    TP_BM_CREATE,
    TP_BM_JOIN,
    TP_BM_COPY,
    TP_BM_COPY_BATCH,
    TP_SHM_CREATE,
    TP_TRANS_REGISTER,
    TP_TRANS_BATCH_WRITE,
    TP_TRANS_BATCH_READ,
    TP_HYBM_RESERVE,
    TP_HYBM_ALLOC,
    TP_HYBM_EXPORT,
    TP_HYBM_IMPORT,
    TP_HYBM_MMAP,
    TP_HYBM_LH_TO_LH,
    TP_HYBM_LH_TO_GH,
    TP_HYBM_GH_TO_LH,
    TP_HYBM_GH_TO_GH,
    TP_HYBM_LD_TO_GD,
    TP_HYBM_GD_TO_LD,
    TP_HYBM_GD_TO_GD,
    TP_HYBM_LH_TO_GD,
    TP_HYBM_GD_TO_LH,
    TP_HYBM_LD_TO_GH,
    TP_HYBM_GH_TO_LD,
    TP_HYBM_GD_TO_GH,
    TP_HYBM_GH_TO_GD,
    TP_HYBM_BATCH_KERNEL,
    TP_HYBM_BATCH_HOST_LEG,
    TP_HYBM_WAIT,
    TP_ZBAL_COLLECTIVE,
    TP_COUNT
};
const char *TracePointName(uint32_t id);

struct Tracer {
    bool enabled = false;
    void (*begin)(uint32_t id, uint64_t nowNs) = nullptr;
    void (*end)(uint32_t id, uint64_t beginNs, uint64_t nowNs, int32_t ret) = nullptr;
};

class PTracer {
public:
    // Starts the default aggregating tracer. `dir` empty => $MF_PTRACER_DIR or /var/log/memfabric_hybrid
    // (falls back to /tmp when not writable). periodMs 0 => 10 s.
    static int Start(const std::string &dir = "", uint32_t periodMs = 0);
    static void Stop();
    static void Install(const Tracer &t);  // replace the tracer (tests, external profilers)
    static const Tracer &Current();
    static std::string DumpTable(bool reset);  // formats one period of the default tracer
    static std::string FilePath();
    struct Row {
        uint64_t begin, goodEnd, badEnd, minNs, maxNs, totalNs;
    };
    static Row Snapshot(uint32_t id);
    // Latency histogram of a point since the tracer started (never reset by the periodic table): counts[i] for
    // i < kHistBuckets = completed operations that took at most 1 us * 2^i, counts[kHistBuckets] = the slower ones.
    // Not cumulative over buckets. -> number of completed operations; *sumNs their total duration.
    static constexpr uint32_t kHistBuckets = 24;
    static uint64_t Histogram(uint32_t id, uint64_t counts[kHistBuckets + 1], uint64_t *sumNs);
};

struct TraceScope {
    uint32_t id;
    uint64_t t0;
};

#define MF_TRACE_BEGIN(ID)                                                    \
    ::mf::TraceScope _tp_##ID{::mf::ID, 0};                                   \
    do {                                                                      \
        const auto &_t = ::mf::PTracer::Current();                            \
        if (_t.enabled) {                                                     \
            _tp_##ID.t0 = ::mf::NowNs();                                      \
            if (_t.begin) _t.begin(::mf::ID, _tp_##ID.t0);                    \
        }                                                                     \
    } while (0)
#define MF_TRACE_END(ID, RET)                                                 \
    do {                                                                      \
        const auto &_t = ::mf::PTracer::Current();                            \
        if (_t.enabled && _t.end) _t.end(::mf::ID, _tp_##ID.t0, ::mf::NowNs(), (int32_t)(RET)); \
    } while (0)

// ---------------------------------------------------------------------------------------------
enum class FipType : int32_t { CALLBACK = 0, PAUSE = 1, RESET = 2, ABORT = 3 };

struct FipParam {
    int64_t value = 0;       // optional numeric parameter from the activation (pause ms, forced code, ...)
    bool skipBlock = false;  // set by a callback to skip the guarded block
};

using FipCallback = void (*)(FipParam *param, int32_t *ret);

class FaultPoints {
public:
    static void Init(const std::string &confPath = "");  // default /tmp/mf_failpoints_<pid>.conf
    static void Exit();
    static int Register(const std::string &name, FipCallback cb);
    static int Unregister(const std::string &name);
    static int Activate(const std::string &name, FipType type, int32_t hits, int64_t param);
    static int Deactivate(const std::string &name);
    static void DeactivateAll();
    static bool IsActive(const std::string &name);
    static void Reload();  // re-reads the config file if it changed
    // Returns true when the guarded block must be skipped.
    static bool Begin(const char *name, int32_t *ret);
    static void RegisterBuiltins();    // ALLOC_LOCAL_MEMORY, MMAP, IMPORT, STORE_CONNECT
    static void UnregisterBuiltins();
    static std::string ConfPath();
};

#define MF_FIP_START(NAME, RETPTR) if (!::mf::FaultPoints::Begin(#NAME, (RETPTR))) {
#define MF_FIP_END }

}  // namespace mf
