// Device-side timeline marks. A kernel brackets a phase with MF_PROF_START(frame) / MF_PROF_STOP(frame);
// thread 0 of each CTA appends one 64-bit record  [63] end flag | [62:56] frame | [55:0] %globaltimer (ns)
// to the CTA's lane of a ring in pinned host memory that the device can write. The host turns the lanes
// into a Chrome-trace file (mf_devtrace.cu). When tracing is off the cost is one load of a device global.
// Counterpart of the per-core trace ring of the reference (operators/npu/aicore/common/zbal_kernel_trace.h:21-63).
//
// The control block is a static device global of each translation unit; MF_DEVTRACE_DEFINE_SETTER(name)
// emits the host function through which the tracer points that unit at the ring.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace mfk {

struct DevTraceCtl {
    unsigned long long *ring;  // [ctas][1 + per_cta]: word 0 of a lane counts its records
    uint32_t per_cta;
    uint32_t ctas;
};

static __device__ DevTraceCtl g_devtrace = {nullptr, 0, 0};

enum ProfFrame : uint32_t {
    PF_STAGE_IN = 1,    // copy of the input into the staging area
    PF_SYNC = 2,        // handshake with the peers (includes the wait)
    PF_REDUCE = 3,      // reduction over the peers' data
    PF_COPY_OUT = 4,    // staging -> output
    PF_PUSH = 5,        // stores into peers' buffers
    PF_LAYOUT = 6,      // MoE: histogram and count exchange
    PF_DISPATCH = 7,    // MoE: quantise + push of the token rows
    PF_WAIT_PEERS = 8,  // MoE: wait for every peer's completion flag
    PF_COMBINE = 9,     // MoE: push home / slot reduce
};

__device__ __forceinline__ void prof_mark(uint32_t frame, uint32_t end)
{
    if (threadIdx.x != 0) return;
    const DevTraceCtl c = g_devtrace;
    if (c.ring == nullptr) return;
    const uint32_t cta = blockIdx.x + gridDim.x * blockIdx.y;
    if (cta >= c.ctas) return;
    unsigned long long *lane = c.ring + (size_t)cta * (c.per_cta + 1);
    const unsigned long long idx = lane[0];
    if (idx >= c.per_cta) return;
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    lane[1 + idx] = ((unsigned long long)(end & 1) << 63) | ((unsigned long long)(frame & 0x7f) << 56) | (t & ((1ull << 56) - 1));
    lane[0] = idx + 1;
}

}  // namespace mfk

#define MF_PROF_START(frame) ::mfk::prof_mark((frame), 0)
#define MF_PROF_STOP(frame) ::mfk::prof_mark((frame), 1)
#define MF_DEVTRACE_DEFINE_SETTER(name)                                                              \
    extern "C" int name(unsigned long long *ring, uint32_t per_cta, uint32_t ctas)                 \
    {                                                                                                \
        ::mfk::DevTraceCtl c{ring, per_cta, ctas};                                                   \
        return (int)cudaMemcpyToSymbol(::mfk::g_devtrace, &c, sizeof(c));                            \
    }
