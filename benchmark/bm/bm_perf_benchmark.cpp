// bm_perf_benchmark: bandwidth / latency of every copy direction of the BigMemory API, with the data checked after each.
//
//   bm_perf_benchmark -bw -t all -s 2097152 -bs 16 -cc 200 -ws 2 -lrs 2 -ip tcp://127.0.0.1:8570
//
// One process per rank (forked here), one GPU per rank. Rank r works against the slices of rank (r + 1) % ws:
//   h2d  d2h              local host  <-> this rank's pooled HBM
//   h2rd rd2h             local host  <-> the peer's pooled HBM
//   h2rh rh2h             local host  <-> the peer's pooled DRAM
//   d2rd rd2d             local HBM   <-> the peer's pooled HBM      (NVLink)
//   d2rh rh2d             local HBM   <-> the peer's pooled DRAM
//   g2g_d2rd g2g_rh2d     pooled -> pooled: own HBM slice -> peer HBM slice, peer DRAM slice -> own HBM slice
// Same role and command line as the reference's benchmark/bm tool (its ten directions plus the two pooled-to-pooled ones);
// -ot accepts the reference's operator names, which all select the one device data path of this build except host_shm.
#include <cuda_runtime.h>
#include <fcntl.h>
#include <poll.h>
#include <pthread.h>
#include <signal.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/wait.h>
#include <unistd.h>

#include <chrono>
#include <string>
#include <vector>

#include "smem.h"
#include "smem_bm.h"

namespace {

struct Options {
    bool latency = false;
    std::string direction = "all";
    std::string op = "sdma";
    std::string url = "tcp://127.0.0.1:8570";
    uint64_t blockSize = 2 << 20;
    uint32_t batch = 1;
    uint32_t count = 100;
    uint32_t world = 2, localRanks = 2, rankStart = 0, deviceStart = 0;
};

enum Side { LOCAL_HOST, LOCAL_DEV, POOL_DEV_OWN, POOL_DEV_PEER, POOL_HOST_PEER };

struct Direction {
    const char *name;
    Side src, dst;
    smem_bm_copy_type type;
};

const Direction kDirections[] = {
    {"h2d", LOCAL_HOST, POOL_DEV_OWN, SMEMB_COPY_H2G},
    {"d2h", POOL_DEV_OWN, LOCAL_HOST, SMEMB_COPY_G2H},
    {"h2rd", LOCAL_HOST, POOL_DEV_PEER, SMEMB_COPY_H2G},
    {"h2rh", LOCAL_HOST, POOL_HOST_PEER, SMEMB_COPY_H2GH},
    {"d2rh", LOCAL_DEV, POOL_HOST_PEER, SMEMB_COPY_L2GH},
    {"d2rd", LOCAL_DEV, POOL_DEV_PEER, SMEMB_COPY_L2G},
    {"rh2d", POOL_HOST_PEER, LOCAL_DEV, SMEMB_COPY_GH2L},
    {"rh2h", POOL_HOST_PEER, LOCAL_HOST, SMEMB_COPY_GH2H},
    {"rd2d", POOL_DEV_PEER, LOCAL_DEV, SMEMB_COPY_G2L},
    {"rd2h", POOL_DEV_PEER, LOCAL_HOST, SMEMB_COPY_G2H},
    {"g2g_d2rd", POOL_DEV_OWN, POOL_DEV_PEER, SMEMB_COPY_G2G},
    {"g2g_rh2d", POOL_HOST_PEER, POOL_DEV_OWN, SMEMB_COPY_G2G},
};

struct Row {
    char name[16];
    uint32_t rank, device;
    uint64_t blockSize, batch, count;
    double totalUs;
    int64_t wrong;  // bytes that differ after the last copy, -1: the copy itself failed
    int32_t valid;
};

struct Shared {  // lives in a MAP_SHARED mapping made before the fork
    pthread_barrier_t barrier;
};

#define CHECK(cond, ...)                   \
    do {                                   \
        if (!(cond)) {                     \
            fprintf(stderr, __VA_ARGS__);  \
            fprintf(stderr, "\n");         \
            return -1;                     \
        }                                  \
    } while (0)

uint8_t PatternByte(uint32_t rank, uint32_t dir, uint64_t i) { return (uint8_t)(i * 131 + (i >> 11) * 7 + rank * 17 + dir * 29 + 1); }

void Fill(std::vector<uint8_t> &v, uint32_t rank, uint32_t dir)
{
    for (uint64_t i = 0; i < v.size(); i++) v[i] = PatternByte(rank, dir, i);
}

struct RankCtx {
    Options opt;
    uint32_t rank = 0, peer = 0, device = 0;
    smem_bm_t bm = nullptr;
    uint64_t bytes = 0;      // blockSize * batch
    uint8_t *localHost = nullptr, *localDev = nullptr;
    uint8_t *poolDevOwn = nullptr, *poolDevPeer = nullptr, *poolHostPeer = nullptr;

    uint8_t *Base(Side s) const
    {
        switch (s) {
            case LOCAL_HOST: return localHost;
            case LOCAL_DEV: return localDev;
            case POOL_DEV_OWN: return poolDevOwn;
            case POOL_DEV_PEER: return poolDevPeer;
            default: return poolHostPeer;
        }
    }
    static bool PoolIsDram(Side s) { return s == POOL_HOST_PEER; }

    // one contiguous copy with the blocking call, retried while the peer's slice is not mapped yet
    int CopyOnce(const void *src, void *dst, uint64_t n, smem_bm_copy_type t)
    {
        smem_copy_params p{};
        p.src = src;
        p.dest = dst;
        p.dataSize = n;
        int rc = -1;
        for (int tries = 0; tries < 600; tries++) {
            rc = smem_bm_copy(bm, &p, t, 0);
            if (rc == 0) return 0;
            usleep(50 * 1000);
        }
        fprintf(stderr, "rank %u: copy type %d failed: %d (%s)\n", rank, (int)t, rc, smem_get_last_err_msg());
        return rc;
    }
    // host <-> any side, through the API for pooled memory and the runtime for the private buffers
    int Upload(Side s, const std::vector<uint8_t> &v)
    {
        if (s == LOCAL_HOST) return memcpy(localHost, v.data(), v.size()), 0;
        if (s == LOCAL_DEV) return cudaMemcpy(localDev, v.data(), v.size(), cudaMemcpyHostToDevice) == cudaSuccess ? 0 : -1;
        return CopyOnce(v.data(), Base(s), v.size(), PoolIsDram(s) ? SMEMB_COPY_H2GH : SMEMB_COPY_H2G);
    }
    int Download(Side s, std::vector<uint8_t> &v)
    {
        if (s == LOCAL_HOST) return memcpy(v.data(), localHost, v.size()), 0;
        if (s == LOCAL_DEV) return cudaMemcpy(v.data(), localDev, v.size(), cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : -1;
        return CopyOnce(Base(s), v.data(), v.size(), PoolIsDram(s) ? SMEMB_COPY_GH2H : SMEMB_COPY_G2H);
    }

    int RunDirection(uint32_t idx, Row &row)
    {
        const Direction &d = kDirections[idx];
        memset(&row, 0, sizeof(row));
        snprintf(row.name, sizeof(row.name), "%s", d.name);
        row.rank = rank;
        row.device = device;
        row.blockSize = opt.blockSize;
        row.batch = opt.batch;
        row.count = opt.count;
        row.valid = 1;
        std::vector<uint8_t> pattern(bytes), zeros(bytes, 0), back(bytes);
        Fill(pattern, rank, idx);
        if (Upload(d.src, pattern) != 0 || Upload(d.dst, zeros) != 0) {
            row.wrong = -1;
            return -1;
        }
        std::vector<void *> srcs(opt.batch), dsts(opt.batch);
        std::vector<uint64_t> sizes(opt.batch, opt.blockSize);
        for (uint32_t i = 0; i < opt.batch; i++) {
            srcs[i] = Base(d.src) + (uint64_t)i * opt.blockSize;
            dsts[i] = Base(d.dst) + (uint64_t)i * opt.blockSize;
        }
        smem_batch_copy_params bp{};
        bp.sources = srcs.data();
        bp.destinations = dsts.data();
        bp.dataSizes = sizes.data();
        bp.batchSize = opt.batch;
        smem_copy_params one{};
        one.src = srcs[0];
        one.dest = dsts[0];
        one.dataSize = opt.blockSize;
        auto issue = [&]() { return opt.batch == 1 ? smem_bm_copy(bm, &one, d.type, 0) : smem_bm_copy_batch(bm, &bp, d.type, 0); };
        for (int w = 0; w < 3; w++) {
            int rc = issue();
            if (rc != 0) {
                fprintf(stderr, "rank %u: %s failed: %d (%s)\n", rank, d.name, rc, smem_get_last_err_msg());
                row.wrong = -1;
                return -1;
            }
        }
        auto t0 = std::chrono::steady_clock::now();
        for (uint32_t c = 0; c < opt.count; c++) {
            if (issue() != 0) {
                row.wrong = -1;
                return -1;
            }
        }
        auto t1 = std::chrono::steady_clock::now();
        row.totalUs = std::chrono::duration<double, std::micro>(t1 - t0).count();
        if (Download(d.dst, back) != 0) {
            row.wrong = -1;
            return -1;
        }
        int64_t wrong = 0;
        for (uint64_t i = 0; i < bytes; i++) wrong += back[i] != pattern[i];
        row.wrong = wrong;
        return 0;
    }
};

int ParseArgs(int argc, char **argv, Options &o)
{
    for (int i = 1; i < argc; i++) {
        std::string a = argv[i];
        auto next = [&]() -> const char * { return i + 1 < argc ? argv[++i] : ""; };
        if (a == "-bw") o.latency = false;
        else if (a == "-lat") o.latency = true;
        else if (a == "-t") o.direction = next();
        else if (a == "-ot") o.op = next();
        else if (a == "-s") o.blockSize = strtoull(next(), nullptr, 0);
        else if (a == "-bs") o.batch = (uint32_t)strtoul(next(), nullptr, 0);
        else if (a == "-cc") o.count = (uint32_t)strtoul(next(), nullptr, 0);
        else if (a == "-ws") o.world = (uint32_t)strtoul(next(), nullptr, 0);
        else if (a == "-lrs") o.localRanks = (uint32_t)strtoul(next(), nullptr, 0);
        else if (a == "-rs") o.rankStart = (uint32_t)strtoul(next(), nullptr, 0);
        else if (a == "-d") o.deviceStart = (uint32_t)strtoul(next(), nullptr, 0);
        else if (a == "-ip") o.url = next();
        else if (a == "-rdma") (void)next();  // accepted for command-line compatibility; there is no RDMA NIC leg here
        else if (a == "-h" || a == "--help") return 1;
        else {
            fprintf(stderr, "unknown option %s\n", a.c_str());
            return -1;
        }
    }
    if (o.blockSize == 0 || o.batch == 0 || o.count == 0 || o.world == 0 || o.localRanks == 0) return -1;
    if (o.world != o.localRanks || o.rankStart != 0) {
        fprintf(stderr, "all ranks of a run live on this box (NVLink domain): -ws must equal -lrs and -rs must be 0\n");
        return -1;
    }
    if (o.direction != "all") {
        bool known = false;
        for (const auto &d : kDirections) known = known || o.direction == d.name;
        if (!known) {
            fprintf(stderr, "unknown direction %s\n", o.direction.c_str());
            return -1;
        }
    }
    return 0;
}

void Usage()
{
    printf("bm_perf_benchmark [-bw|-lat] [-ot sdma|device_rdma|host_rdma|host_urma|host_tcp|host_shm] [-t DIRECTION|all]\n"
           "                  [-s BLOCK_SIZE] [-bs BLOCKS_PER_CALL] [-cc CALLS] [-ws WORLD] [-lrs LOCAL_RANKS] [-rs 0]\n"
           "                  [-d FIRST_DEVICE] [-ip tcp://ip:port]\n  directions:");
    for (const auto &d : kDirections) printf(" %s", d.name);
    printf("\n");
}

int RunRank(const Options &opt, uint32_t localIdx, Shared *sh, int pipeFd)
{
    RankCtx c;
    c.opt = opt;
    c.rank = opt.rankStart + localIdx;
    c.peer = (c.rank + 1) % opt.world;
    c.device = opt.deviceStart + localIdx;
    c.bytes = opt.blockSize * opt.batch;
    int nDev = 0;
    const bool gpu = cudaGetDeviceCount(&nDev) == cudaSuccess && nDev > 0;
    if (gpu) {
        c.device %= (uint32_t)nDev;
        CHECK(cudaSetDevice((int)c.device) == cudaSuccess, "cudaSetDevice(%u) failed", c.device);
    } else {
        (void)cudaGetLastError();  // no device: only the host <-> pooled DRAM directions can run
        c.device = 0;
    }
    CHECK(smem_init(0) == 0, "smem_init: %s", smem_get_last_err_msg());
    smem_set_log_level(3);
    smem_bm_config_t cfg;
    smem_bm_config_init(&cfg);
    cfg.autoRanking = false;
    cfg.rankId = c.rank;
    cfg.startConfigStoreServer = c.rank == 0;
    CHECK(smem_bm_init(opt.url.c_str(), opt.world, (uint16_t)c.device, &cfg) == 0, "smem_bm_init: %s", smem_get_last_err_msg());
    // two regions per slice: [0, bytes) is written by the previous rank, [bytes, 2 bytes) by the owner
    const uint64_t slice = ((2 * c.bytes + (64ull << 20) - 1) >> 26) << 26;
    const smem_bm_data_op_type op = (opt.op == "host_shm" || !gpu) ? SMEMB_DATA_OP_HOST_SHM : SMEMB_DATA_OP_SDMA;
    c.bm = smem_bm_create(0, opt.world, op, slice, gpu ? slice : 0, 0);
    CHECK(c.bm != nullptr, "smem_bm_create: %s", smem_get_last_err_msg());
    CHECK(smem_bm_join(c.bm, 0) == 0, "smem_bm_join: %s", smem_get_last_err_msg());
    if (gpu) {
        CHECK(cudaMalloc(&c.localDev, c.bytes) == cudaSuccess, "cudaMalloc of %lu bytes failed", (unsigned long)c.bytes);
        CHECK(cudaHostAlloc(&c.localHost, c.bytes, cudaHostAllocDefault) == cudaSuccess, "cudaHostAlloc failed");
        c.poolDevOwn = static_cast<uint8_t *>(smem_bm_ptr_by_mem_type(c.bm, SMEM_MEM_TYPE_DEVICE, (uint16_t)c.rank)) + c.bytes;
        c.poolDevPeer = static_cast<uint8_t *>(smem_bm_ptr_by_mem_type(c.bm, SMEM_MEM_TYPE_DEVICE, (uint16_t)c.peer));
    } else {
        CHECK(posix_memalign(reinterpret_cast<void **>(&c.localHost), 4096, c.bytes) == 0, "host allocation failed");
    }
    c.poolHostPeer = static_cast<uint8_t *>(smem_bm_ptr_by_mem_type(c.bm, SMEM_MEM_TYPE_HOST, (uint16_t)c.peer));
    pthread_barrier_wait(&sh->barrier);  // everybody has joined

    int failures = 0;
    for (uint32_t i = 0; i < sizeof(kDirections) / sizeof(kDirections[0]); i++) {
        if (opt.direction != "all" && opt.direction != kDirections[i].name) continue;
        const Direction &d = kDirections[i];
        const bool hostOnly = (d.src == LOCAL_HOST || d.src == POOL_HOST_PEER) && (d.dst == LOCAL_HOST || d.dst == POOL_HOST_PEER);
        if (!gpu && !hostOnly) continue;  // every rank skips the same directions, so the barriers below stay matched
        Row row;
        if (c.RunDirection(i, row) != 0 || row.wrong != 0) failures++;
        if (write(pipeFd, &row, sizeof(row)) != (ssize_t)sizeof(row)) failures++;
        pthread_barrier_wait(&sh->barrier);  // the ranks move through the directions together, as concurrent traffic
    }
    pthread_barrier_wait(&sh->barrier);  // nobody unmaps a slice that a peer still reads
    if (gpu) {
        cudaFree(c.localDev);
        cudaFreeHost(c.localHost);
    } else {
        free(c.localHost);
    }
    smem_bm_leave(c.bm, 0);
    if (c.rank == 0) usleep(500 * 1000);  // the store's host leaves last
    smem_bm_destroy(c.bm);
    smem_bm_uninit(0);
    smem_uninit();
    return failures;
}

}  // namespace

int main(int argc, char **argv)
{
    Options opt;
    int pr = ParseArgs(argc, argv, opt);
    if (pr != 0) {
        Usage();
        return pr > 0 ? 0 : 2;
    }
    Shared *sh = static_cast<Shared *>(mmap(nullptr, sizeof(Shared), PROT_READ | PROT_WRITE, MAP_SHARED | MAP_ANONYMOUS, -1, 0));
    if (sh == MAP_FAILED) return 2;
    pthread_barrierattr_t ba;
    pthread_barrierattr_init(&ba);
    pthread_barrierattr_setpshared(&ba, PTHREAD_PROCESS_SHARED);
    pthread_barrier_init(&sh->barrier, &ba, opt.localRanks);
    int fds[2];
    if (pipe(fds) != 0) return 2;
    std::vector<pid_t> kids;
    for (uint32_t i = 0; i < opt.localRanks; i++) {
        pid_t pid = fork();  // before any CUDA call of this process
        if (pid == 0) {
            close(fds[0]);
            int rc = RunRank(opt, i, sh, fds[1]);
            fflush(nullptr);
            _exit(rc == 0 ? 0 : 1);
        }
        kids.push_back(pid);
    }
    close(fds[1]);
    std::vector<Row> rows;
    int bad = 0;
    size_t live = kids.size();
    std::vector<bool> done(kids.size(), false);
    while (live > 0) {
        // rows arrive on the pipe; a rank that dies would leave the others in a barrier, so they are ended with it
        struct pollfd pfd = {fds[0], POLLIN, 0};
        if (poll(&pfd, 1, 200) > 0 && (pfd.revents & POLLIN)) {
            Row r;
            if (read(fds[0], &r, sizeof(r)) == (ssize_t)sizeof(r)) rows.push_back(r);
        }
        for (size_t k = 0; k < kids.size(); k++) {
            if (done[k]) continue;
            int st = 0;
            if (waitpid(kids[k], &st, WNOHANG) != kids[k]) continue;
            done[k] = true;
            live--;
            if (!WIFEXITED(st) || WEXITSTATUS(st) != 0) {
                bad++;
                for (size_t j = 0; j < kids.size(); j++)
                    if (!done[j]) kill(kids[j], SIGKILL);
            }
        }
    }
    {
        Row r;  // what was still in the pipe
        int fl = fcntl(fds[0], F_GETFL, 0);
        fcntl(fds[0], F_SETFL, fl | O_NONBLOCK);
        while (read(fds[0], &r, sizeof(r)) == (ssize_t)sizeof(r)) rows.push_back(r);
    }
    printf("%-10s %5s %5s %12s %6s %8s %14s %12s %12s %8s\n", "direction", "rank", "dev", "block_bytes", "batch", "calls", "total_us",
           opt.latency ? "us_per_call" : "GB_per_s", opt.latency ? "GB_per_s" : "us_per_call", "wrong");
    for (const auto &d : kDirections) {
        for (uint32_t rank = 0; rank < opt.world; rank++) {
            for (const auto &row : rows) {
                if (strcmp(row.name, d.name) != 0 || row.rank != rank) continue;
                const double bytes = (double)row.blockSize * row.batch * row.count;
                const double gbs = row.totalUs > 0 ? bytes / row.totalUs / 1e3 : 0.0;
                const double lat = row.count > 0 ? row.totalUs / row.count : 0.0;
                printf("%-10s %5u %5u %12lu %6lu %8lu %14.1f %12.2f %12.2f %8ld\n", row.name, row.rank, row.device,
                       (unsigned long)row.blockSize, (unsigned long)row.batch, (unsigned long)row.count, row.totalUs,
                       opt.latency ? lat : gbs, opt.latency ? gbs : lat, (long)row.wrong);
                if (row.wrong != 0) bad++;
            }
        }
    }
    printf("%s\n", bad == 0 ? "ALL DIRECTIONS VERIFIED" : "FAILED");
    return bad == 0 ? 0 : 1;
}
