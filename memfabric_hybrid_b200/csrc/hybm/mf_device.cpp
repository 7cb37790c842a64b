#include "mf_device.h"

#include <dlfcn.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cmath>
#include <map>
#include <mutex>

#include "../util/mf_util.h"

#ifndef MAP_FIXED_NOREPLACE
#define MAP_FIXED_NOREPLACE 0x100000
#endif

namespace mf {
namespace hybm {

namespace {

// "Device memory" of the fake backend is memfd-backed host memory; handles are the memfds.
class FakeBackend : public DeviceBackend {
public:
    FakeBackend()
    {
        caps_.present = false;
        caps_.vmm = true;
        caps_.posixFd = true;
        caps_.deviceCount = 1;
        caps_.granularity = 2ULL << 20;
        caps_.totalMem = 64ULL << 30;
        snprintf(caps_.name, sizeof(caps_.name), "fake-device");
    }
    const char *Name() const override { return "fake"; }
    int Init(int deviceId) override
    {
        dev_ = deviceId;
        return OK;
    }
    int DeviceId() const override { return dev_; }
    const DeviceCaps &Caps() const override { return caps_; }
    int BindThread() override { return OK; }

    int Reserve(uint64_t hint, uint64_t size, uint64_t *va) override
    {
        void *p = mmap(reinterpret_cast<void *>(hint), size, PROT_NONE,
                       MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE | (hint ? MAP_FIXED_NOREPLACE : 0), -1, 0);
        if (p == MAP_FAILED) return MF_FAIL(ERR_NO_RESOURCES, "fake reserve %#lx+%#lx: %s", (unsigned long)hint, (unsigned long)size, strerror(errno));
        if (hint != 0 && reinterpret_cast<uint64_t>(p) != hint) {
            munmap(p, size);
            return ERR_NO_RESOURCES;
        }
        *va = reinterpret_cast<uint64_t>(p);
        return OK;
    }
    int ReleaseVa(uint64_t va, uint64_t size) override { return munmap(reinterpret_cast<void *>(va), size) == 0 ? OK : ERR; }
    int CreatePhys(uint64_t size, PhysHandle *h) override
    {
        int fd = memfd_create("mf-fake-hbm", MFD_CLOEXEC);
        if (fd < 0) return MF_FAIL(ERR_NO_RESOURCES, "memfd_create: %s", strerror(errno));
        if (ftruncate(fd, (off_t)size) != 0) {
            close(fd);
            return MF_FAIL(ERR_MALLOC, "ftruncate(%lu): %s", (unsigned long)size, strerror(errno));
        }
        *h = (PhysHandle)fd;
        return OK;
    }
    int ExportFd(PhysHandle h, int *fd) override
    {
        *fd = fcntl((int)h, F_DUPFD_CLOEXEC, 0);
        return *fd >= 0 ? OK : ERR;
    }
    int ImportFd(int fd, uint64_t, PhysHandle *h) override
    {
        *h = (PhysHandle)fd;
        return OK;
    }
    int Map(uint64_t va, uint64_t size, PhysHandle h) override
    {
        void *p = mmap(reinterpret_cast<void *>(va), size, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_FIXED, (int)h, 0);
        return p == MAP_FAILED ? MF_FAIL(ERR, "fake map %#lx: %s", (unsigned long)va, strerror(errno)) : OK;
    }
    int Unmap(uint64_t va, uint64_t size) override
    {
        void *p = mmap(reinterpret_cast<void *>(va), size, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE | MAP_FIXED,
                       -1, 0);
        return p == MAP_FAILED ? ERR : OK;
    }
    int ReleasePhys(PhysHandle h) override
    {
        close((int)h);
        return OK;
    }
    int Malloc(uint64_t size, uint64_t *ptr) override
    {
        void *p = nullptr;
        if (posix_memalign(&p, 4096, size) != 0) return ERR_MALLOC;
        std::lock_guard<std::mutex> g(mu_);
        allocs_[reinterpret_cast<uint64_t>(p)] = size;
        *ptr = reinterpret_cast<uint64_t>(p);
        return OK;
    }
    int Free(uint64_t ptr) override
    {
        {
            std::lock_guard<std::mutex> g(mu_);
            allocs_.erase(ptr);
        }
        free(reinterpret_cast<void *>(ptr));
        return OK;
    }
    int HostAlloc(uint64_t size, void **ptr) override { return posix_memalign(ptr, 4096, size) == 0 ? OK : ERR_MALLOC; }
    int HostFree(void *ptr) override
    {
        free(ptr);
        return OK;
    }
    int HostRegister(void *, uint64_t) override { return OK; }
    int HostUnregister(void *) override { return OK; }
    int IpcExport(uint64_t, uint8_t *, uint64_t *, uint64_t *) override { return ERR; }
    int IpcOpen(const uint8_t *, uint64_t *) override { return ERR; }
    int IpcClose(uint64_t) override { return ERR; }
    bool IsDevicePointer(uint64_t ptr) override
    {
        std::lock_guard<std::mutex> g(mu_);
        auto it = allocs_.upper_bound(ptr);
        if (it == allocs_.begin()) return false;
        --it;
        return ptr < it->first + it->second;
    }
    int EnablePeerAccess(int) override { return OK; }
    int CanAccessPeer(int) override { return 1; }
    int StreamCreate(void **s) override
    {
        *s = reinterpret_cast<void *>(0x1);
        return OK;
    }
    int StreamDestroy(void *) override { return OK; }
    int StreamSync(void *) override { return OK; }
    int MemcpyAsync(uint64_t dst, uint64_t src, uint64_t len, MemcpyKind, void *) override
    {
        memmove(reinterpret_cast<void *>(dst), reinterpret_cast<const void *>(src), len);
        return OK;
    }
    int MemsetAsync(uint64_t dst, int value, uint64_t len, void *) override
    {
        memset(reinterpret_cast<void *>(dst), value, len);
        return OK;
    }
    int LaunchBatchCopy(const CopyItem *items, uint32_t count, void *, bool) override
    {
        for (uint32_t i = 0; i < count; i++)
            memmove(reinterpret_cast<void *>(items[i].dst), reinterpret_cast<const void *>(items[i].src), items[i].len);
        return OK;
    }
    // Reference arithmetic of the quantising copy, also used as the CPU oracle of the CUDA kernel.
    int LaunchQuantCopy(const QuantItem *items, uint32_t count, uint32_t unit, int inputFp16, int mode, void *) override
    {
        if (mode != 0 || unit == 0) return ERR_INVALID_PARAM;  // fp8 needs the device
        for (uint32_t i = 0; i < count; i++) {
            const uint16_t *in = reinterpret_cast<const uint16_t *>(items[i].src);
            int8_t *out = reinterpret_cast<int8_t *>(items[i].dst);
            float *sc = reinterpret_cast<float *>(items[i].scale);
            uint64_t units = (items[i].elems + unit - 1) / unit;
            for (uint64_t u = 0; u < units; u++) {
                uint64_t b = u * unit, e = std::min<uint64_t>(items[i].elems, b + unit);
                float amax = 0.f;
                for (uint64_t k = b; k < e; k++) amax = std::max(amax, std::fabs(ToFloat(in[k], inputFp16)));
                float s = amax > 0.f ? 127.f / amax : 1.f;
                for (uint64_t k = b; k < e; k++) {
                    float q = std::nearbyint(ToFloat(in[k], inputFp16) * s);
                    out[k] = (int8_t)std::max(-127.f, std::min(127.f, q));
                }
                sc[u] = amax > 0.f ? amax / 127.f : 1.f;
            }
        }
        return OK;
    }

private:
    static float ToFloat(uint16_t h, int fp16)
    {
        if (!fp16) {
            uint32_t w = (uint32_t)h << 16;
            float f;
            memcpy(&f, &w, 4);
            return f;
        }
        uint32_t sign = (h >> 15) & 1, exp = (h >> 10) & 0x1f, man = h & 0x3ff;
        float v;
        if (exp == 0) v = std::ldexp((float)man, -24);
        else if (exp == 31) v = man ? NAN : INFINITY;
        else v = std::ldexp((float)(man | 0x400), (int)exp - 25);
        return sign ? -v : v;
    }
    int dev_ = 0;
    DeviceCaps caps_;
    std::mutex mu_;
    std::map<uint64_t, uint64_t> allocs_;
};

std::mutex g_mu;
DeviceBackend *g_backend = nullptr;
void *g_cudaLib = nullptr;
int g_refs = 0;

std::string SelfDir()
{
    Dl_info info;
    if (dladdr(reinterpret_cast<void *>(&CreateFakeBackend), &info) == 0 || info.dli_fname == nullptr) return ".";
    std::string p = info.dli_fname;
    size_t s = p.rfind('/');
    return s == std::string::npos ? "." : p.substr(0, s);
}

}  // namespace

DeviceBackend *CreateFakeBackend() { return new FakeBackend(); }

DeviceBackend *CurrentBackend()
{
    std::lock_guard<std::mutex> g(g_mu);
    return g_backend;
}

DeviceBackend *AcquireBackend(int deviceId, std::string *why)
{
    std::lock_guard<std::mutex> g(g_mu);
    if (g_backend != nullptr) {
        g_refs++;
        return g_backend;
    }
    std::string mode = EnvStr("MF_DEVICE_BACKEND", nullptr, "auto");
    auto say = [&](const std::string &s) {
        if (why != nullptr) *why = s;
    };
    if (mode == "none") {
        say("MF_DEVICE_BACKEND=none");
        return nullptr;
    }
    if (mode == "fake") {
        g_backend = new FakeBackend();
        g_backend->Init(deviceId);
        g_refs = 1;
        return g_backend;
    }
    std::string path = EnvStr("MF_CUDA_BACKEND_LIB", nullptr, (SelfDir() + "/libmf_cuda.so").c_str());
    g_cudaLib = dlopen(path.c_str(), RTLD_NOW | RTLD_GLOBAL);
    if (g_cudaLib == nullptr) {
        say(std::string("cannot load ") + path + ": " + dlerror());
        if (mode == "cuda") MF_ERROR("MF_DEVICE_BACKEND=cuda but %s", why ? why->c_str() : "load failed");
        return nullptr;
    }
    auto fn = reinterpret_cast<MfCreateCudaBackendFn>(dlsym(g_cudaLib, "mf_create_cuda_backend"));
    if (fn == nullptr) {
        say("libmf_cuda.so lacks mf_create_cuda_backend");
        return nullptr;
    }
    DeviceBackend *b = fn();
    int rc = b->Init(deviceId);
    if (rc != OK) {
        say("no usable CUDA device (init returned " + std::to_string(rc) + ")");
        delete b;
        return nullptr;
    }
    g_backend = b;
    g_refs = 1;
    return g_backend;
}

void *CudaSymbol(const char *name)
{
    std::lock_guard<std::mutex> g(g_mu);
    if (g_cudaLib == nullptr) {
        std::string path = EnvStr("MF_CUDA_BACKEND_LIB", nullptr, (SelfDir() + "/libmf_cuda.so").c_str());
        g_cudaLib = dlopen(path.c_str(), RTLD_NOW | RTLD_GLOBAL);
        if (g_cudaLib == nullptr) {
            MF_WARN("cannot load %s: %s", path.c_str(), dlerror());
            return nullptr;
        }
    }
    return dlsym(g_cudaLib, name);
}

void ReleaseBackend()
{
    std::lock_guard<std::mutex> g(g_mu);
    if (g_refs > 0 && --g_refs == 0) {
        delete g_backend;
        g_backend = nullptr;
    }
}

}  // namespace hybm
}  // namespace mf
