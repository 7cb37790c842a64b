// transfer_perf: latency and throughput of the TRANS API between two ranks, block sizes 32 KiB .. 16 MiB, 32 blocks per call.
//
//   transfer_perf {rankSize} {rankId} {deviceId} {useSdma} tcp://{ip}:{port}        one process per rank, or
//   transfer_perf fork {deviceOfRank0} {deviceOfRank1} tcp://{ip}:{port}             both ranks forked from here
//
// Rank 0 is the sender, rank 1 the receiver. The receiver registers a device buffer and publishes its address through the
// SHM control plane (all-gather); the sender writes every block size `kRounds` times with smem_trans_batch_write, then
// reads the blocks back with smem_trans_batch_read and compares. Output lines have the reference tool's form
// ("Test completed: latency ..us, block size ..KB, total size ..KB , throughput .. GB/s"; benchmark/transfer/perf_cpp).
#include <cuda_runtime.h>
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
#include "smem_shm.h"
#include "smem_trans.h"

namespace {
constexpr uint32_t kBlocks = 32;
constexpr uint64_t kMinBlock = 32 << 10;
uint64_t kMaxBlock = 16 << 20;  // MF_PERF_MAX_BLOCK_KB lowers it (quick runs)
bool g_gpu = true;              // false: no CUDA device, the buffers are host memory (the API moves those as well)

uint8_t *AllocBuf(uint64_t n, int fill)
{
    uint8_t *p = nullptr;
    if (g_gpu) {
        if (cudaMalloc(&p, n) != cudaSuccess || cudaMemset(p, fill, n) != cudaSuccess) return nullptr;
        return p;
    }
    if (posix_memalign(reinterpret_cast<void **>(&p), 4096, n) != 0) return nullptr;
    memset(p, fill, n);
    return p;
}
void FreeBuf(uint8_t *p)
{
    if (g_gpu) cudaFree(p);
    else free(p);
}
bool ToBuf(uint8_t *dst, const uint8_t *hostSrc, uint64_t n)
{
    if (g_gpu) return cudaMemcpy(dst, hostSrc, n, cudaMemcpyHostToDevice) == cudaSuccess;
    memcpy(dst, hostSrc, n);
    return true;
}
bool FromBuf(uint8_t *hostDst, const uint8_t *src, uint64_t n)
{
    if (g_gpu) return cudaMemcpy(hostDst, src, n, cudaMemcpyDeviceToHost) == cudaSuccess;
    memcpy(hostDst, src, n);
    return true;
}
constexpr int kWarmup = 3, kRounds = 20;

#define CHECK(cond, ...)                  \
    do {                                  \
        if (!(cond)) {                    \
            fprintf(stderr, __VA_ARGS__); \
            fprintf(stderr, "\n");        \
            return 1;                     \
        }                                 \
    } while (0)

struct Published {
    uint64_t addr;
    char id[56];
};

// Address exchange and barriers of the two ranks: the SHM control plane when the ranks are separate commands, a shared
// mapping with a process-shared barrier when both were forked from one command (works without a GPU as well).
struct ForkShared {
    pthread_barrier_t barrier;
    Published slots[2];
};
struct Control {
    ForkShared *forked = nullptr;
    smem_shm_t shm = nullptr;
    int AllGather(uint32_t rank, uint32_t world, const Published &mine, std::vector<Published> &all)
    {
        if (forked != nullptr) {
            forked->slots[rank] = mine;
            pthread_barrier_wait(&forked->barrier);
            all.assign(forked->slots, forked->slots + 2);
            return 0;
        }
        return smem_shm_control_allgather(shm, reinterpret_cast<const char *>(&mine), sizeof(mine), reinterpret_cast<char *>(all.data()),
                                          (uint32_t)(sizeof(mine) * world));
    }
    void Barrier()
    {
        if (forked != nullptr) pthread_barrier_wait(&forked->barrier);
        else smem_shm_control_barrier(shm);
    }
};

int RunRank(uint32_t world, uint32_t rank, int device, bool sdma, const std::string &url, ForkShared *forked)
{
    int nDev = 0;
    g_gpu = cudaGetDeviceCount(&nDev) == cudaSuccess && nDev > 0;
    if (g_gpu) {
        device %= nDev;
        CHECK(cudaSetDevice(device) == cudaSuccess, "cudaSetDevice(%d) failed", device);
    } else {
        (void)cudaGetLastError();
        if (rank == 0) printf("no CUDA device: host buffers\n");
    }
    if (const char *e = getenv("MF_PERF_MAX_BLOCK_KB")) {
        uint64_t kb = strtoull(e, nullptr, 0);
        if (kb >= 32 && kb <= 16384) kMaxBlock = kb << 10;
    }
    CHECK(smem_init(0) == 0, "smem_init: %s", smem_get_last_err_msg());
    smem_set_log_level(3);
    if (rank == 0) CHECK(smem_create_config_store(url.c_str(), 0) == 0, "config store: %s", smem_get_last_err_msg());

    smem_trans_config_t tc;
    smem_trans_config_init(&tc);
    tc.role = rank == 0 ? SMEM_TRANS_SENDER : SMEM_TRANS_RECEIVER;
    tc.deviceId = (uint32_t)device;
    tc.dataOpType = sdma ? SMEMB_DATA_OP_SDMA : SMEMB_DATA_OP_DEVICE_RDMA;
    CHECK(smem_trans_init(&tc) == 0, "smem_trans_init: %s", smem_get_last_err_msg());
    const std::string myId = "127.0.0.1:" + std::to_string(20000 + rank);
    smem_trans_t trans = smem_trans_create(url.c_str(), myId.c_str(), &tc);
    CHECK(trans != nullptr, "smem_trans_create: %s", smem_get_last_err_msg());

    Control ctl;
    ctl.forked = forked;
    if (forked == nullptr) {
        smem_shm_config_t sc;
        smem_shm_config_init(&sc);
        sc.startConfigStoreServer = false;
        CHECK(smem_shm_init(url.c_str(), world, rank, (uint16_t)device, &sc) == 0, "smem_shm_init: %s", smem_get_last_err_msg());
        void *gva = nullptr;
        ctl.shm = smem_shm_create(0, world, rank, 2 << 20, SMEMS_DATA_OP_MTE, 0, &gva);
        CHECK(ctl.shm != nullptr, "smem_shm_create: %s", smem_get_last_err_msg());
    }

    const uint64_t total = kMaxBlock * kBlocks;
    uint8_t *buf = AllocBuf(total, rank == 0 ? 0x5A : 0);
    CHECK(buf != nullptr, "cannot allocate %lu bytes", (unsigned long)total);
    CHECK(smem_trans_register_mem(trans, buf, total, 0) == 0, "register_mem: %s", smem_get_last_err_msg());

    std::vector<Published> all(world);
    Published mine{};
    mine.addr = reinterpret_cast<uint64_t>(buf);
    snprintf(mine.id, sizeof(mine.id), "%s", myId.c_str());
    CHECK(ctl.AllGather(rank, world, mine, all) == 0, "allgather: %s", smem_get_last_err_msg());

    int rc = 0;
    if (rank == 0) {
        const Published &peer = all[1];
        uint8_t *scratch = AllocBuf(total, 0);
        CHECK(scratch != nullptr, "cannot allocate %lu bytes", (unsigned long)total);
        CHECK(smem_trans_register_mem(trans, scratch, total, 0) == 0, "register_mem: %s", smem_get_last_err_msg());
        std::vector<uint8_t> host(total), expect(total);
        for (uint64_t bs = kMinBlock; bs <= kMaxBlock && rc == 0; bs <<= 1) {
            std::vector<const void *> src(kBlocks);
            std::vector<void *> dst(kBlocks), back(kBlocks);
            std::vector<const void *> rsrc(kBlocks);
            std::vector<size_t> sizes(kBlocks, bs);
            for (uint32_t i = 0; i < kBlocks; i++) {
                src[i] = buf + i * bs;
                dst[i] = reinterpret_cast<void *>(peer.addr + i * bs);
                rsrc[i] = dst[i];
                back[i] = scratch + i * bs;
            }
            // a pattern of this block size, so that a stale block of the previous size cannot pass
            for (uint64_t i = 0; i < bs * kBlocks; i++) expect[i] = (uint8_t)(i * 31 + (i >> 13) + bs / kMinBlock);
            CHECK(ToBuf(buf, expect.data(), bs * kBlocks), "upload failed");
            for (int w = 0; w < kWarmup && rc == 0; w++) {
                // the receiver's registration becomes visible shortly after its create: retry the first writes
                for (int tries = 0; tries < 200; tries++) {
                    rc = smem_trans_batch_write(trans, src.data(), peer.id, dst.data(), sizes.data(), kBlocks, 0);
                    if (rc == 0) break;
                    usleep(50 * 1000);
                }
            }
            CHECK(rc == 0, "batch_write: %d %s", rc, smem_get_last_err_msg());
            auto t0 = std::chrono::steady_clock::now();
            for (int r = 0; r < kRounds && rc == 0; r++)
                rc = smem_trans_batch_write(trans, src.data(), peer.id, dst.data(), sizes.data(), kBlocks, 0);
            auto t1 = std::chrono::steady_clock::now();
            CHECK(rc == 0, "batch_write: %d %s", rc, smem_get_last_err_msg());
            const double us = std::chrono::duration<double, std::micro>(t1 - t0).count() / kRounds;
            // read back and compare
            memset(host.data(), 0, bs * kBlocks);
            CHECK(ToBuf(scratch, host.data(), bs * kBlocks), "clearing the read-back buffer failed");
            rc = smem_trans_batch_read(trans, back.data(), peer.id, rsrc.data(), sizes.data(), kBlocks, 0);
            CHECK(rc == 0, "batch_read: %d %s", rc, smem_get_last_err_msg());
            CHECK(FromBuf(host.data(), scratch, bs * kBlocks), "download failed");
            uint64_t wrong = 0;
            for (uint64_t i = 0; i < bs * kBlocks; i++) wrong += host[i] != expect[i];
            printf("Test completed: latency %.1fus, block size %luKB, total size %luKB , throughput %.2f GB/s, verified %s\n", us,
                   (unsigned long)(bs >> 10), (unsigned long)((bs * kBlocks) >> 10), (double)(bs * kBlocks) / us / 1e3,
                   wrong == 0 ? "yes" : "NO");
            if (wrong != 0) rc = 1;
        }
        FreeBuf(scratch);
    }
    fflush(stdout);
    ctl.Barrier();  // the receiver keeps its buffer until the sender is done
    FreeBuf(buf);
    if (ctl.shm != nullptr) {
        smem_shm_destroy(ctl.shm, 0);
        smem_shm_uninit(0);
    }
    smem_trans_destroy(trans, 0);
    smem_trans_uninit(0);
    if (rank == 0) {
        usleep(300 * 1000);
        smem_destroy_config_store(url.c_str());
    }
    smem_uninit();
    return rc;
}
}  // namespace

int main(int argc, char **argv)
{
    if (argc == 5 && strcmp(argv[1], "fork") == 0) {
        const int dev[2] = {atoi(argv[2]), atoi(argv[3])};
        const std::string url = argv[4];
        ForkShared *sh = static_cast<ForkShared *>(mmap(nullptr, sizeof(ForkShared), PROT_READ | PROT_WRITE, MAP_SHARED | MAP_ANONYMOUS, -1, 0));
        if (sh == MAP_FAILED) return 2;
        pthread_barrierattr_t ba;
        pthread_barrierattr_init(&ba);
        pthread_barrierattr_setpshared(&ba, PTHREAD_PROCESS_SHARED);
        pthread_barrier_init(&sh->barrier, &ba, 2);
        pid_t kids[2];
        for (int r = 0; r < 2; r++) {
            kids[r] = fork();  // before any CUDA call of this process
            if (kids[r] == 0) {
                if (r == 1) usleep(300 * 1000);  // the store is served by rank 0
                int rc = RunRank(2, (uint32_t)r, dev[r], true, url, sh);
                fflush(nullptr);
                _exit(rc);
            }
        }
        int bad = 0;
        for (int left = 2; left > 0; left--) {
            int st = 0;
            pid_t who = wait(&st);
            if (who <= 0) break;
            if (!WIFEXITED(st) || WEXITSTATUS(st) != 0) {
                bad++;
                for (int r = 0; r < 2; r++)  // its partner would wait in a barrier for ever
                    if (kids[r] != who) kill(kids[r], SIGKILL);
            }
        }
        return bad == 0 ? 0 : 1;
    }
    if (argc != 6) {
        printf("usage: transfer_perf {rankSize} {rankId} {deviceId} {useSdma} tcp://{ip}:{port}\n"
               "       transfer_perf fork {deviceOfRank0} {deviceOfRank1} tcp://{ip}:{port}\n");
        return 2;
    }
    return RunRank((uint32_t)atoi(argv[1]), (uint32_t)atoi(argv[2]), atoi(argv[3]), atoi(argv[4]) != 0, argv[5], nullptr);
}
