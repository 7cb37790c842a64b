// Process-wide state of zbal: what bootstrap set up, the communicator registry, and the launcher table
// of the CUDA kernel library (resolved at run time: this library does not link the CUDA runtime).
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../include/smem_shm.h"
#include "../include/zbal.h"

namespace zbal {

// ---- argument blocks of the kernel launchers (layout shared with kernels/mf_team.cuh, mf_coll.cu) ----
struct MfTeam {
    uint64_t heap_base;
    uint64_t stride;
    uint64_t mc_base;
    uint32_t rank;
    uint32_t world;
    uint32_t emu;
    uint32_t spin_limit;
};
struct MfCollArgs {
    MfTeam team;
    uint64_t in, out, in_rank_stride, out_rank_stride, n, stage_a, stage_b;
    float scale;
    int op;
    uint32_t epoch, zero_copy, root, algo;
    uint64_t part_stride;
};
struct MfA2AArgs {
    MfTeam team;
    uint64_t in, out, in_rank_stride, out_rank_stride, meta, meta_rank_stride, in_bytes, stage_a;
    uint32_t epoch;
};
struct MfP2PArgs {
    MfTeam team;
    uint64_t buf, bytes, stage_off;
    uint32_t peer, epoch, channel;
};

struct Launchers {
    int (*coll)(int kind, int in_dtype, int out_dtype, const MfCollArgs *, int ctas, int threads, void *stream) = nullptr;
    int (*a2a)(const MfA2AArgs *, int ctas, int threads, void *stream) = nullptr;
    int (*send)(const MfP2PArgs *, int ctas, void *stream) = nullptr;
    int (*recv)(const MfP2PArgs *, int ctas, void *stream) = nullptr;
    int (*barrier)(const MfTeam *, uint32_t channel, uint32_t epoch, void *stream) = nullptr;
    unsigned (*argsSize)() = nullptr;
    int (*smCount)() = nullptr;
    bool ok = false;
};
// Resolves the table once; false (with the last error set) when the CUDA library cannot be loaded.
const Launchers *GetLaunchers();

constexpr uint64_t kSignalBytes = 1ull << 20;  // flags at the start of every communicator slot
constexpr uint32_t kStageCount = 5;            // A0, B0, A1, B1, point-to-point landing

class Comm {
public:
    std::string name;
    uint32_t id = 0, first = 0, step = 1, size = 1, groupRank = 0;
    MfTeam team{};
    uint64_t stageBytes = 0;
    uint64_t stageOff[4] = {0, 0, 0, 0};  // relative to the communicator slot
    uint64_t p2pOff = 0, p2pBytes = 0;
    uint64_t epoch = 0;
    std::map<std::pair<uint32_t, uint32_t>, uint32_t> p2pEpochs;
    int maxCtas = 128;
    std::mutex mu;

    uint32_t Next(uint64_t &a, uint64_t &b)
    {
        epoch++;
        a = stageOff[(epoch & 1) * 2];
        b = stageOff[(epoch & 1) * 2 + 1];
        return (uint32_t)epoch;
    }
    int Ctas(uint64_t bytes) const;
};

struct State {
    std::mutex mu;
    bool up = false;
    zbal_bootstrap_options_t opts{};
    zbal_bootstrap_output_t out{};
    smem_shm_t shm = nullptr;
    std::vector<smem_shm_t> extraShm;  // expansion segments of the heap (zbal_heap_expand), destroyed with the first one
    std::vector<uint64_t> extraLocal;  // address of this rank's slot in each of them
    uint64_t commSlotBytes = 0;
    bool ownSmem = false, ownShm = false, ownSma = false;
    std::map<std::string, std::shared_ptr<Comm>> comms;
    std::shared_ptr<Comm> world;
    uint32_t spinLimit = 1u << 22;
    uint64_t mcBase = 0;  // NVLink multicast alias of a slice (0: not set up); only the world communicator can use it
};
State &S();

// communicator lookup for the operation entry points (nullptr + last error when the handle is stale)
std::shared_ptr<Comm> FindComm(zbal_comm_t h);

}  // namespace zbal
