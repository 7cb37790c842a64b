// Host side of the device timeline: owns the ring (pinned, device-writable host memory), points the
// kernel translation units at it, and writes a Chrome-trace JSON ("X" events: pid = rank, tid = CTA).
// Parity of role: app/zbal/src/csrc/common/zbal_trace_viewer_dumper.h:63-132 of the reference.
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "mf_devtrace.cuh"

extern "C" int mf_coll_set_devtrace(unsigned long long *, uint32_t, uint32_t);
extern "C" int mf_moe_set_devtrace(unsigned long long *, uint32_t, uint32_t);

namespace {
std::mutex g_mu;
unsigned long long *g_host = nullptr, *g_dev = nullptr;
uint32_t g_perCta = 0, g_ctas = 0;

const char *FrameName(uint32_t f)
{
    switch (f) {
        case mfk::PF_STAGE_IN: return "stage_in";
        case mfk::PF_SYNC: return "sync";
        case mfk::PF_REDUCE: return "reduce";
        case mfk::PF_COPY_OUT: return "copy_out";
        case mfk::PF_PUSH: return "push";
        case mfk::PF_LAYOUT: return "moe_layout";
        case mfk::PF_DISPATCH: return "moe_dispatch";
        case mfk::PF_WAIT_PEERS: return "wait_peers";
        case mfk::PF_COMBINE: return "moe_combine";
        default: return "frame";
    }
}

int PointAll(unsigned long long *ring, uint32_t per, uint32_t ctas)
{
    int rc = mf_coll_set_devtrace(ring, per, ctas);
    if (rc == 0) rc = mf_moe_set_devtrace(ring, per, ctas);
    return rc;
}
}  // namespace

extern "C" {

// ctas lanes of per_cta records each (16 bytes of host memory per 2 records). Returns 0 or a CUDA error.
int mf_devtrace_enable(uint32_t ctas, uint32_t per_cta)
{
    std::lock_guard<std::mutex> g(g_mu);
    if (g_host != nullptr) return 0;
    if (ctas == 0 || per_cta == 0 || (uint64_t)ctas * (per_cta + 1) * 8 > (1ull << 30)) return -1;
    const size_t bytes = (size_t)ctas * (per_cta + 1) * sizeof(unsigned long long);
    cudaError_t e = cudaHostAlloc(reinterpret_cast<void **>(&g_host), bytes, cudaHostAllocMapped);
    if (e != cudaSuccess) return (int)e;
    memset(g_host, 0, bytes);
    e = cudaHostGetDevicePointer(reinterpret_cast<void **>(&g_dev), g_host, 0);
    if (e != cudaSuccess) {
        cudaFreeHost(g_host);
        g_host = nullptr;
        return (int)e;
    }
    g_perCta = per_cta;
    g_ctas = ctas;
    return PointAll(g_dev, per_cta, ctas);
}

int mf_devtrace_disable(void)
{
    std::lock_guard<std::mutex> g(g_mu);
    if (g_host == nullptr) return 0;
    cudaDeviceSynchronize();
    PointAll(nullptr, 0, 0);
    cudaFreeHost(g_host);
    g_host = g_dev = nullptr;
    g_perCta = g_ctas = 0;
    return 0;
}

// Number of records currently held (after a device synchronisation).
long long mf_devtrace_count(void)
{
    std::lock_guard<std::mutex> g(g_mu);
    if (g_host == nullptr) return 0;
    cudaDeviceSynchronize();
    long long n = 0;
    for (uint32_t c = 0; c < g_ctas; c++) n += (long long)g_host[(size_t)c * (g_perCta + 1)];
    return n;
}

// Writes the Chrome-trace file and, when reset != 0, empties the lanes. Returns the number of events
// written or a negative value on failure.
long long mf_devtrace_dump(const char *path, int rank, int reset)
{
    std::lock_guard<std::mutex> g(g_mu);
    if (g_host == nullptr || path == nullptr) return -1;
    cudaDeviceSynchronize();
    FILE *f = fopen(path, "w");
    if (f == nullptr) return -2;
    fprintf(f, "{\"displayTimeUnit\":\"ns\",\"traceEvents\":[\n");
    long long events = 0;
    unsigned long long t0 = ~0ull;
    for (uint32_t c = 0; c < g_ctas; c++) {
        const unsigned long long *lane = g_host + (size_t)c * (g_perCta + 1);
        for (unsigned long long i = 0; i < lane[0] && i < g_perCta; i++) t0 = std::min(t0, lane[1 + i] & ((1ull << 56) - 1));
    }
    bool first = true;
    for (uint32_t c = 0; c < g_ctas; c++) {
        unsigned long long *lane = g_host + (size_t)c * (g_perCta + 1);
        const unsigned long long n = std::min<unsigned long long>(lane[0], g_perCta);
        unsigned long long open[128];
        bool has[128] = {false};
        for (unsigned long long i = 0; i < n; i++) {
            const unsigned long long r = lane[1 + i];
            const uint32_t frame = (uint32_t)((r >> 56) & 0x7f);
            const unsigned long long t = r & ((1ull << 56) - 1);
            if ((r >> 63) == 0) {
                open[frame] = t;
                has[frame] = true;
            } else if (has[frame]) {
                has[frame] = false;
                fprintf(f, "%s{\"name\":\"%s\",\"ph\":\"X\",\"pid\":%d,\"tid\":%u,\"ts\":%.3f,\"dur\":%.3f}", first ? "" : ",\n", FrameName(frame),
                        rank, c, (double)(open[frame] - t0) / 1000.0, (double)(t - open[frame]) / 1000.0);
                first = false;
                events++;
            }
        }
        if (reset) lane[0] = 0;
    }
    fprintf(f, "\n]}\n");
    fclose(f);
    return events;
}

}  // extern "C"
