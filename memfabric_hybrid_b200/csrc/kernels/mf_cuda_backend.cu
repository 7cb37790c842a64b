// CUDA implementation of the device backend: CUDA VMM for the pooled HBM (fixed-address reserve,
// POSIX-FD shareable physical allocations, peer mapping), host registration of the pooled DRAM, CUDA
// IPC for caller-registered device buffers, streams / copy engines, and the launches of the xcopy
// kernels. Driver entry points are looked up through the runtime (no link-time libcuda), so this
// library also loads on a machine without a GPU, where Init reports "no device".
// Parity of role: src/hybm/csrc/under_api/dl_cuda_api.cpp:42-82 plus the driver calls of
// src/hybm/csrc/mm/hybm_vmm_based_segment.cpp:71-101,252-336,395-445,551-631 restated for CUDA.
#include <cuda.h>
#include <cuda_runtime.h>
#include <unistd.h>

#include <map>
#include <mutex>

#include "../hybm/mf_device.h"
#include "../util/mf_util.h"
#include "mf_xcopy.cuh"

namespace mf {
namespace hybm {
namespace {

#define DRV(name) decltype(&name) p_##name = nullptr
struct DriverApi {
    DRV(cuMemAddressReserve);
    DRV(cuMemAddressFree);
    DRV(cuMemCreate);
    DRV(cuMemRelease);
    DRV(cuMemMap);
    DRV(cuMemUnmap);
    DRV(cuMemSetAccess);
    DRV(cuMemExportToShareableHandle);
    DRV(cuMemImportFromShareableHandle);
    DRV(cuMemGetAllocationGranularity);
    DRV(cuMemGetAddressRange);
    DRV(cuPointerGetAttribute);
    DRV(cuMulticastCreate);
    DRV(cuMulticastAddDevice);
    DRV(cuMulticastBindAddr);
    DRV(cuMulticastUnbind);
    DRV(cuMulticastGetGranularity);
    DRV(cuDeviceGet);
    DRV(cuGetErrorString);
    bool ok = false;
};
#undef DRV

template <typename F> bool Load(const char *name, F &fn)
{
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr) {
        (void)cudaGetLastError();
        return false;
    }
    fn = reinterpret_cast<F>(p);
    return true;
}

#define CU_CHECK(call, what)                                                                         \
    do {                                                                                             \
        CUresult _r = (call);                                                                        \
        if (_r != CUDA_SUCCESS) {                                                                    \
            const char *_s = nullptr;                                                                \
            if (drv_.p_cuGetErrorString) drv_.p_cuGetErrorString(_r, &_s);                           \
            return MF_FAIL(ERR, "%s failed: %s (%d)", what, _s ? _s : "?", (int)_r);                 \
        }                                                                                            \
    } while (0)

#define RT_CHECK(call, what)                                                                         \
    do {                                                                                             \
        cudaError_t _e = (call);                                                                     \
        if (_e != cudaSuccess) {                                                                     \
            (void)cudaGetLastError();                                                                \
            return MF_FAIL(ERR, "%s failed: %s", what, cudaGetErrorString(_e));                      \
        }                                                                                            \
    } while (0)

class CudaBackend : public DeviceBackend {
public:
    const char *Name() const override { return "cuda"; }

    int Init(int deviceId) override
    {
        int n = 0;
        if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
            (void)cudaGetLastError();
            return ERR_NOT_EXIST;
        }
        if (deviceId < 0 || deviceId >= n) return MF_FAIL(ERR_INVALID_PARAM, "device %d outside [0, %d)", deviceId, n);
        dev_ = deviceId;
        RT_CHECK(cudaSetDevice(dev_), "cudaSetDevice");
        RT_CHECK(cudaFree(nullptr), "context creation");
        cudaDeviceProp prop;
        RT_CHECK(cudaGetDeviceProperties(&prop, dev_), "cudaGetDeviceProperties");
        caps_.present = true;
        caps_.deviceCount = n;
        caps_.smCount = prop.multiProcessorCount;
        caps_.ccMajor = prop.major;
        caps_.ccMinor = prop.minor;
        caps_.totalMem = prop.totalGlobalMem;
        snprintf(caps_.name, sizeof(caps_.name), "%s", prop.name);
        cudaDriverGetVersion(&caps_.driverVersion);
        cudaRuntimeGetVersion(&caps_.runtimeVersion);
        bool ok = Load("cuMemAddressReserve", drv_.p_cuMemAddressReserve) && Load("cuMemAddressFree", drv_.p_cuMemAddressFree) &&
                  Load("cuMemCreate", drv_.p_cuMemCreate) && Load("cuMemRelease", drv_.p_cuMemRelease) &&
                  Load("cuMemMap", drv_.p_cuMemMap) && Load("cuMemUnmap", drv_.p_cuMemUnmap) &&
                  Load("cuMemSetAccess", drv_.p_cuMemSetAccess) &&
                  Load("cuMemExportToShareableHandle", drv_.p_cuMemExportToShareableHandle) &&
                  Load("cuMemImportFromShareableHandle", drv_.p_cuMemImportFromShareableHandle) &&
                  Load("cuMemGetAllocationGranularity", drv_.p_cuMemGetAllocationGranularity) &&
                  Load("cuMemGetAddressRange", drv_.p_cuMemGetAddressRange) &&
                  Load("cuPointerGetAttribute", drv_.p_cuPointerGetAttribute);
        Load("cuGetErrorString", drv_.p_cuGetErrorString);
        drv_.ok = ok;
        {
            const bool have = Load("cuMulticastCreate", drv_.p_cuMulticastCreate) && Load("cuMulticastAddDevice", drv_.p_cuMulticastAddDevice) &&
                              Load("cuMulticastBindAddr", drv_.p_cuMulticastBindAddr) && Load("cuMulticastUnbind", drv_.p_cuMulticastUnbind) &&
                              Load("cuMulticastGetGranularity", drv_.p_cuMulticastGetGranularity) && Load("cuDeviceGet", drv_.p_cuDeviceGet);
            caps_.multicast = have && ok && McSupported();
        }
        // Every GPU this library targets (sm_100) has virtual memory management; the entry points being
        // present is the remaining condition.
        caps_.vmm = ok;
        caps_.posixFd = ok;  // POSIX file descriptors are the handle type of every Linux driver
        int hostPtr = 0;
        cudaDeviceGetAttribute(&hostPtr, cudaDevAttrCanUseHostPointerForRegisteredMem, dev_);
        caps_.hostPtrForRegistered = hostPtr != 0;
        if (caps_.vmm) {
            CUmemAllocationProp ap = AllocProp();
            size_t g = 0;
            if (drv_.p_cuMemGetAllocationGranularity(&g, &ap, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && g != 0)
                caps_.granularity = g;
        }
        grid_ = (int)EnvInt("MF_XCOPY_CTAS_PER_SM", nullptr, 2, 1, 4) * caps_.smCount;
        SetupBulk();
        return OK;
    }

    // Shape of the bulk-copy kernel: MF_XCOPY_BULK = "pipelines per CTA, stages, piece KiB" (0 pipelines: use the
    // register-copy kernel only). As many CTAs per SM as the stage rings leave room for.
    void SetupBulk()
    {
        int pipes = 2, stages = 4, pieceKb = 16;
        if (const char *e = getenv("MF_XCOPY_BULK")) {
            if (sscanf(e, "%d,%d,%d", &pipes, &stages, &pieceKb) < 1) pipes = 0;
        }
        ConfigureBulkCopy(pipes, stages, pieceKb);
    }
    int ConfigureBulkCopy(int pipes, int stages, int pieceKb) override
    {
        bulkPipes_ = 0;
        if (pipes <= 0) return OK;
        pipes = std::min(pipes, 4);
        stages = std::min(std::max(stages, 4), mfk::kBulkMaxStages);
        pieceKb = std::min(std::max(pieceKb, 1), 48);
        const uint32_t smem = (uint32_t)pipes * stages * pieceKb * 1024u;
        if (smem > 220u * 1024u) return ERR_INVALID_PARAM;
        if (cudaFuncSetAttribute(mfk::mf_xcopy_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            (void)cudaGetLastError();
            return ERR_NO_RESOURCES;
        }
        if (copyStatus_ == nullptr) {
            void *st = nullptr;
            if (cudaHostAlloc(&st, 64, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
                (void)cudaGetLastError();
                return ERR_MALLOC;
            }
            memset(st, 0, 64);
            copyStatus_ = static_cast<uint32_t *>(st);
        }
        bulkStages_ = (uint32_t)stages;
        bulkPiece_ = (uint32_t)pieceKb * 1024u;
        const int perSm = std::max(1, std::min(8, (int)((227u * 1024u) / (smem + 1024u))));
        bulkGrid_ = perSm * caps_.smCount;
        bulkPipes_ = (uint32_t)pipes;
        return OK;
    }

    bool McSupported()
    {
        // CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED through the driver attribute query
        using AttrFn = CUresult (*)(int *, CUdevice_attribute, CUdevice);
        AttrFn fn = nullptr;
        if (!Load("cuDeviceGetAttribute", fn)) return false;
        CUdevice d;
        if (drv_.p_cuDeviceGet(&d, dev_) != CUDA_SUCCESS) return false;
        int v = 0;
        return fn(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, d) == CUDA_SUCCESS && v != 0;
    }
    CUmulticastObjectProp McProp(uint64_t size, uint32_t devices) const
    {
        CUmulticastObjectProp p;
        memset(&p, 0, sizeof(p));
        p.numDevices = devices;
        p.size = size;
        p.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
        return p;
    }
    int McGranularity(uint64_t size, uint32_t devices, uint64_t *gran) override
    {
        if (!caps_.multicast) return ERR;
        CUmulticastObjectProp p = McProp(size, devices);
        size_t g = 0;
        CU_CHECK(drv_.p_cuMulticastGetGranularity(&g, &p, CU_MULTICAST_GRANULARITY_MINIMUM), "cuMulticastGetGranularity");
        *gran = g;
        return OK;
    }
    int McCreate(uint64_t size, uint32_t devices, PhysHandle *h) override
    {
        if (!caps_.multicast) return ERR;
        CUmulticastObjectProp p = McProp(size, devices);
        CUmemGenericAllocationHandle mc;
        CU_CHECK(drv_.p_cuMulticastCreate(&mc, &p), "cuMulticastCreate");
        *h = (PhysHandle)mc;
        return OK;
    }
    int McAddDevice(PhysHandle h) override
    {
        CUdevice d;
        CU_CHECK(drv_.p_cuDeviceGet(&d, dev_), "cuDeviceGet");
        CU_CHECK(drv_.p_cuMulticastAddDevice((CUmemGenericAllocationHandle)h, d), "cuMulticastAddDevice");
        return OK;
    }
    int McBindAddr(PhysHandle h, uint64_t mcOffset, uint64_t va, uint64_t size) override
    {
        CU_CHECK(drv_.p_cuMulticastBindAddr((CUmemGenericAllocationHandle)h, mcOffset, (CUdeviceptr)va, size, 0), "cuMulticastBindAddr");
        return OK;
    }
    int McUnbind(PhysHandle h, uint64_t mcOffset, uint64_t size) override
    {
        CUdevice d;
        CU_CHECK(drv_.p_cuDeviceGet(&d, dev_), "cuDeviceGet");
        CU_CHECK(drv_.p_cuMulticastUnbind((CUmemGenericAllocationHandle)h, d, mcOffset, size), "cuMulticastUnbind");
        return OK;
    }

    int DeviceId() const override { return dev_; }
    const DeviceCaps &Caps() const override { return caps_; }
    int BindThread() override
    {
        int cur = -1;
        if (cudaGetDevice(&cur) == cudaSuccess && cur == dev_) return OK;
        RT_CHECK(cudaSetDevice(dev_), "cudaSetDevice");
        return OK;
    }

    // ---- VMM
    int Reserve(uint64_t hint, uint64_t size, uint64_t *va) override
    {
        if (!caps_.vmm) return ERR_NOT_INIT;
        CUdeviceptr p = 0;
        CU_CHECK(drv_.p_cuMemAddressReserve(&p, size, caps_.granularity, (CUdeviceptr)hint, 0), "cuMemAddressReserve");
        if (hint != 0 && (uint64_t)p != hint) {
            drv_.p_cuMemAddressFree(p, size);
            return MF_FAIL(ERR_NO_RESOURCES, "cuMemAddressReserve gave %#lx instead of %#lx", (unsigned long)p, (unsigned long)hint);
        }
        *va = (uint64_t)p;
        return OK;
    }
    int ReleaseVa(uint64_t va, uint64_t size) override
    {
        CU_CHECK(drv_.p_cuMemAddressFree((CUdeviceptr)va, size), "cuMemAddressFree");
        return OK;
    }
    int CreatePhys(uint64_t size, PhysHandle *h) override
    {
        CUmemAllocationProp ap = AllocProp();
        CUmemGenericAllocationHandle handle;
        CU_CHECK(drv_.p_cuMemCreate(&handle, size, &ap, 0), "cuMemCreate");
        *h = (PhysHandle)handle;
        return OK;
    }
    int ExportFd(PhysHandle h, int *fd) override
    {
        int out = -1;
        CU_CHECK(drv_.p_cuMemExportToShareableHandle(&out, (CUmemGenericAllocationHandle)h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
                 "cuMemExportToShareableHandle");
        *fd = out;
        return OK;
    }
    int ImportFd(int fd, uint64_t, PhysHandle *h) override
    {
        CUmemGenericAllocationHandle handle;
        CUresult r = drv_.p_cuMemImportFromShareableHandle(&handle, (void *)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
        close(fd);
        CU_CHECK(r, "cuMemImportFromShareableHandle");
        *h = (PhysHandle)handle;
        return OK;
    }
    int Map(uint64_t va, uint64_t size, PhysHandle h) override
    {
        CU_CHECK(drv_.p_cuMemMap((CUdeviceptr)va, size, 0, (CUmemGenericAllocationHandle)h, 0), "cuMemMap");
        CUmemAccessDesc ad{};
        ad.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        ad.location.id = dev_;
        ad.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
        CUresult r = drv_.p_cuMemSetAccess((CUdeviceptr)va, size, &ad, 1);
        if (r != CUDA_SUCCESS) {
            drv_.p_cuMemUnmap((CUdeviceptr)va, size);
            CU_CHECK(r, "cuMemSetAccess");
        }
        return OK;
    }
    int Unmap(uint64_t va, uint64_t size) override
    {
        CU_CHECK(drv_.p_cuMemUnmap((CUdeviceptr)va, size), "cuMemUnmap");
        return OK;
    }
    int ReleasePhys(PhysHandle h) override
    {
        CU_CHECK(drv_.p_cuMemRelease((CUmemGenericAllocationHandle)h), "cuMemRelease");
        return OK;
    }

    // ---- plain memory
    int Malloc(uint64_t size, uint64_t *ptr) override
    {
        void *p = nullptr;
        RT_CHECK(cudaMalloc(&p, size), "cudaMalloc");
        *ptr = (uint64_t)p;
        return OK;
    }
    int Free(uint64_t ptr) override
    {
        RT_CHECK(cudaFree((void *)ptr), "cudaFree");
        return OK;
    }
    int HostAlloc(uint64_t size, void **ptr) override
    {
        RT_CHECK(cudaHostAlloc(ptr, size, cudaHostAllocPortable | cudaHostAllocMapped), "cudaHostAlloc");
        return OK;
    }
    int HostFree(void *ptr) override
    {
        RT_CHECK(cudaFreeHost(ptr), "cudaFreeHost");
        return OK;
    }
    int HostRegister(void *ptr, uint64_t size) override
    {
        cudaError_t e = cudaHostRegister(ptr, size, cudaHostRegisterPortable | cudaHostRegisterMapped);
        if (e == cudaErrorHostMemoryAlreadyRegistered) {
            (void)cudaGetLastError();
            return OK;
        }
        RT_CHECK(e, "cudaHostRegister");
        return OK;
    }
    int HostUnregister(void *ptr) override
    {
        cudaError_t e = cudaHostUnregister(ptr);
        if (e != cudaSuccess) (void)cudaGetLastError();
        return OK;
    }
    int IpcExport(uint64_t ptr, uint8_t blob[64], uint64_t *base, uint64_t *size) override
    {
        CUdeviceptr b = 0;
        size_t sz = 0;
        CU_CHECK(drv_.p_cuMemGetAddressRange(&b, &sz, (CUdeviceptr)ptr), "cuMemGetAddressRange");
        cudaIpcMemHandle_t h;
        RT_CHECK(cudaIpcGetMemHandle(&h, (void *)b), "cudaIpcGetMemHandle");
        static_assert(sizeof(h) == 64, "IPC handle is 64 bytes");
        memcpy(blob, &h, sizeof(h));
        *base = (uint64_t)b;
        *size = sz;
        return OK;
    }
    int IpcOpen(const uint8_t blob[64], uint64_t *ptr) override
    {
        cudaIpcMemHandle_t h;
        memcpy(&h, blob, sizeof(h));
        std::lock_guard<std::mutex> g(mu_);
        std::string key(reinterpret_cast<const char *>(blob), 64);
        auto it = ipc_.find(key);
        if (it != ipc_.end()) {  // one allocation may carry several registered buffers: open it once
            it->second.refs++;
            *ptr = it->second.ptr;
            return OK;
        }
        void *p = nullptr;
        RT_CHECK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
        ipc_[key] = IpcRec{(uint64_t)p, 1};
        *ptr = (uint64_t)p;
        return OK;
    }
    int IpcClose(uint64_t ptr) override
    {
        std::lock_guard<std::mutex> g(mu_);
        for (auto it = ipc_.begin(); it != ipc_.end(); ++it) {
            if (it->second.ptr != ptr) continue;
            if (--it->second.refs == 0) {
                cudaIpcCloseMemHandle((void *)ptr);
                ipc_.erase(it);
            }
            return OK;
        }
        return ERR_NOT_EXIST;
    }
    bool IsDevicePointer(uint64_t ptr) override
    {
        cudaPointerAttributes a;
        if (cudaPointerGetAttributes(&a, (const void *)ptr) != cudaSuccess) {
            (void)cudaGetLastError();
            return false;
        }
        return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
    }
    bool IsPinnedHost(uint64_t ptr, uint64_t len) override
    {
        if (!caps_.hostPtrForRegistered || len == 0) return false;
        auto pinned = [](uint64_t a) {
            cudaPointerAttributes at;
            if (cudaPointerGetAttributes(&at, (const void *)a) != cudaSuccess) {
                (void)cudaGetLastError();
                return false;
            }
            return at.type == cudaMemoryTypeHost && at.devicePointer == (void *)a;
        };
        return pinned(ptr) && pinned(ptr + len - 1);
    }
    int EnablePeerAccess(int peer) override
    {
        if (peer == dev_) return OK;
        cudaError_t e = cudaDeviceEnablePeerAccess(peer, 0);
        if (e == cudaErrorPeerAccessAlreadyEnabled) {
            (void)cudaGetLastError();
            return OK;
        }
        RT_CHECK(e, "cudaDeviceEnablePeerAccess");
        return OK;
    }
    int CanAccessPeer(int peer) override
    {
        if (peer == dev_) return 1;
        int can = 0;
        if (cudaDeviceCanAccessPeer(&can, dev_, peer) != cudaSuccess) (void)cudaGetLastError();
        return can;
    }

    // ---- execution
    int StreamCreate(void **s) override
    {
        cudaStream_t st;
        RT_CHECK(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking), "cudaStreamCreate");
        *s = st;
        return OK;
    }
    int StreamDestroy(void *s) override
    {
        cudaStreamDestroy((cudaStream_t)s);
        return OK;
    }
    int StreamSync(void *s) override
    {
        RT_CHECK(cudaStreamSynchronize((cudaStream_t)s), "cudaStreamSynchronize");
        return OK;
    }
    int MemcpyAsync(uint64_t dst, uint64_t src, uint64_t len, MemcpyKind, void *s) override
    {
        RT_CHECK(cudaMemcpyAsync((void *)dst, (const void *)src, len, cudaMemcpyDefault, (cudaStream_t)s), "cudaMemcpyAsync");
        return OK;
    }
    int MemsetAsync(uint64_t dst, int value, uint64_t len, void *s) override
    {
        RT_CHECK(cudaMemsetAsync((void *)dst, value, len, (cudaStream_t)s), "cudaMemsetAsync");
        return OK;
    }
    int LaunchBatchCopy(const CopyItem *items, uint32_t count, void *s, bool bulkOk) override
    {
        if (count == 0) return OK;
        static_assert(sizeof(CopyItem) == sizeof(mfk::CopyItem), "descriptor layout");
        if (bulkOk && bulkPipes_ > 0 && copyStatus_ != nullptr) {
            const uint32_t smem = bulkPipes_ * bulkStages_ * bulkPiece_;
            const uint32_t grid = std::min<uint32_t>((count + bulkPipes_ - 1) / bulkPipes_, (uint32_t)bulkGrid_);
            mfk::mf_xcopy_bulk_kernel<<<grid, 32 * bulkPipes_, smem, (cudaStream_t)s>>>(reinterpret_cast<const mfk::CopyItem *>(items), count,
                                                                                      bulkStages_, bulkPiece_, copyStatus_, window_);
            RT_CHECK(cudaGetLastError(), "xcopy bulk launch");
            return OK;
        }
        int grid = (int)std::min<uint32_t>(count, (uint32_t)grid_);
        mfk::mf_xcopy_batch_kernel<<<grid, mfk::kCopyThreads, 0, (cudaStream_t)s>>>(reinterpret_cast<const mfk::CopyItem *>(items), count,
                                                                                    copyStatus_ != nullptr ? window_ : nullptr, copyStatus_);
        RT_CHECK(cudaGetLastError(), "xcopy batch launch");
        return OK;
    }
    bool SetCopyWindow(uint64_t base, uint64_t slot, uint32_t ranks, const uint64_t *mapped) override
    {
        if (copyStatus_ == nullptr || ranks > 64) return false;
        if (window_ == nullptr) {
            if (base == 0) return true;
            void *p = nullptr;
            if (cudaHostAlloc(&p, sizeof(mfk::CopyWindow), cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
                (void)cudaGetLastError();
                return false;
            }
            memset(p, 0, sizeof(mfk::CopyWindow));
            window_ = static_cast<mfk::CopyWindow *>(p);
        }
        // launches already queued read the table when they run: callers change it between batches, not under them
        window_->slot = slot;
        window_->ranks = ranks;
        for (uint32_t r = 0; r < 64; r++) window_->mapped[r] = (mapped != nullptr && r < ranks) ? mapped[r] : 0;
        window_->base = base;
        return true;
    }
    uint32_t CopyStatus(bool clear) override
    {
        if (copyStatus_ == nullptr) return 0;
        const uint32_t v = *reinterpret_cast<volatile uint32_t *>(copyStatus_);
        if (clear && v != 0) *reinterpret_cast<volatile uint32_t *>(copyStatus_) = 0;
        return v;
    }
    int LaunchQuantCopy(const QuantItem *items, uint32_t count, uint32_t unit, int inputFp16, int mode, void *s) override
    {
        if (count == 0) return OK;
        if (unit == 0 || (mode == 1 && unit != 128) || mode < 0 || mode > 1) return MF_FAIL(ERR_INVALID_PARAM, "quant copy: unit %u / mode %d unsupported", unit, mode);
        static_assert(sizeof(QuantItem) == sizeof(mfk::QuantItem), "descriptor layout");
        auto *q = reinterpret_cast<const mfk::QuantItem *>(items);
        for (uint32_t off = 0; off < count; off += 65535) {
            uint32_t n = std::min<uint32_t>(65535, count - off);
            // Every CTA fetches its descriptor from the pinned host ring (a PCIe read), so the grid is kept near the
            // number of CTAs the GPU can hold: with many items one CTA walks all units of its item, with few items the
            // units of an item are spread over several CTAs (8 units, one per warp, per CTA and step).
            uint64_t maxUnits = 1;
            for (uint32_t i = 0; i < n; i++) maxUnits = std::max<uint64_t>(maxUnits, (items[off + i].elems + unit - 1) / unit);
            const uint64_t perItem = std::max<uint64_t>(1, (2ull * (uint64_t)std::max(1, grid_) + n - 1) / n);
            dim3 grid((unsigned)std::min<uint64_t>({perItem, (maxUnits + 15) / 16, 65535ull}), n);  // a CTA takes at least 16 units per step
            cudaStream_t st = (cudaStream_t)s;
            // units of 128 elements on aligned addresses (the fp8 1 x 128 format, and int8 with that unit): the kernel
            // that keeps eight loads per lane in flight
            bool fast = unit == 128;
            for (uint32_t i = 0; i < n && fast; i++) {
                const QuantItem &q0 = items[off + i];
                fast = (q0.src & 15) == 0 && (q0.dst & 7) == 0 && (q0.scale & 3) == 0 && (q0.elems % 128) == 0 && q0.elems != 0;
            }
            if (fast) {
                dim3 g2((unsigned)std::min<uint64_t>({perItem, (maxUnits + 127) / 128, 65535ull}), n);  // a CTA takes 128 units per step
                if (inputFp16) {
                    if (mode == 0) mfk::mf_xcopy_quant128_kernel<__half, 0><<<g2, 256, 0, st>>>(q + off);
                    else mfk::mf_xcopy_quant128_kernel<__half, 1><<<g2, 256, 0, st>>>(q + off);
                } else {
                    if (mode == 0) mfk::mf_xcopy_quant128_kernel<__nv_bfloat16, 0><<<g2, 256, 0, st>>>(q + off);
                    else mfk::mf_xcopy_quant128_kernel<__nv_bfloat16, 1><<<g2, 256, 0, st>>>(q + off);
                }
                RT_CHECK(cudaGetLastError(), "xcopy quant launch");
                continue;
            }
            if (inputFp16) {
                if (mode == 0) mfk::mf_xcopy_quant_kernel<__half, 0><<<grid, 256, 0, st>>>(q + off, unit);
                else mfk::mf_xcopy_quant_kernel<__half, 1><<<grid, 256, 0, st>>>(q + off, unit);
            } else {
                if (mode == 0) mfk::mf_xcopy_quant_kernel<__nv_bfloat16, 0><<<grid, 256, 0, st>>>(q + off, unit);
                else mfk::mf_xcopy_quant_kernel<__nv_bfloat16, 1><<<grid, 256, 0, st>>>(q + off, unit);
            }
            RT_CHECK(cudaGetLastError(), "xcopy quant launch");
        }
        return OK;
    }

private:
    CUmemAllocationProp AllocProp() const
    {
        CUmemAllocationProp ap{};
        ap.type = CU_MEM_ALLOCATION_TYPE_PINNED;
        ap.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        ap.location.id = dev_;
        ap.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
        return ap;
    }
    struct IpcRec {
        uint64_t ptr;
        int refs;
    };
    int dev_ = 0;
    int grid_ = 296;
    uint32_t bulkPipes_ = 0, bulkStages_ = 4, bulkPiece_ = 16384;
    int bulkGrid_ = 148;
    uint32_t *copyStatus_ = nullptr;
    mfk::CopyWindow *window_ = nullptr;  // debug table of the copy kernels (pinned, device-visible), null unless MF_XCOPY_DEBUG is on
    DeviceCaps caps_;
    DriverApi drv_;
    std::mutex mu_;
    std::map<std::string, IpcRec> ipc_;
};

}  // namespace
}  // namespace hybm
}  // namespace mf

extern "C" mf::hybm::DeviceBackend *mf_create_cuda_backend() { return new mf::hybm::CudaBackend(); }

// Small runtime helpers for the host-only library, which does not link the CUDA runtime itself.
extern "C" int mf_cuda_device_sync(int device)
{
    (void)device;  // one device per process: the current device is the one in use
    return (int)cudaDeviceSynchronize();
}
extern "C" int mf_cuda_memset(void *ptr, int value, size_t bytes) { return (int)cudaMemset(ptr, value, bytes); }
extern "C" int mf_cuda_copy_d2h(void *dst, const void *src, size_t bytes) { return (int)cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost); }
extern "C" int mf_cuda_sm_count(void)
{
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return sms;
}

// Self-check of the copy kernels' debug window (see mfk::CopyWindow): runs `n` descriptors (src, dst, len triples) through
// the register-copy kernel (bulk == 0) or the bulk-copy kernel (bulk != 0) against a window described by the caller, on
// the default stream, and returns the status word the kernel left (0: every descriptor passed, 0x7D1: at least one was
// refused and skipped). Descriptors that fail are never dereferenced, so a test may name an address in an unmapped part
// of the window. Returns a negative number when the launch could not be made.
extern "C" int mf_xcopy_debug_probe(const uint64_t *triples, uint32_t n, uint64_t win_base, uint64_t slot, uint32_t ranks,
                                    const uint64_t *mapped, int bulk)
{
    if (triples == nullptr || n == 0 || n > 1024 || ranks > 64) return -1;
    void *mem = nullptr;
    const size_t bytes = sizeof(mfk::CopyWindow) + 64 + (size_t)n * sizeof(mfk::CopyItem);
    if (cudaHostAlloc(&mem, bytes, cudaHostAllocMapped) != cudaSuccess) {
        (void)cudaGetLastError();
        return -2;
    }
    memset(mem, 0, bytes);
    auto *w = static_cast<mfk::CopyWindow *>(mem);
    auto *status = reinterpret_cast<uint32_t *>(static_cast<char *>(mem) + sizeof(mfk::CopyWindow));
    auto *items = reinterpret_cast<mfk::CopyItem *>(static_cast<char *>(mem) + sizeof(mfk::CopyWindow) + 64);
    w->base = win_base;
    w->slot = slot;
    w->ranks = ranks;
    for (uint32_t r = 0; r < ranks; r++) w->mapped[r] = mapped != nullptr ? mapped[r] : 0;
    for (uint32_t i = 0; i < n; i++) items[i] = mfk::CopyItem{triples[3 * i], triples[3 * i + 1], triples[3 * i + 2]};
    int rc = 0;
    if (bulk) {
        const uint32_t smem = 4 * 16384;
        if (cudaFuncSetAttribute(mfk::mf_xcopy_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024) != cudaSuccess) rc = -3;
        if (rc == 0) mfk::mf_xcopy_bulk_kernel<<<2, 32, smem>>>(items, n, 4, 16384, status, w);
    } else {
        mfk::mf_xcopy_batch_kernel<<<2, mfk::kCopyThreads>>>(items, n, w, status);
    }
    if (rc == 0 && (cudaGetLastError() != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess)) rc = -4;
    if (rc == 0) rc = (int)*reinterpret_cast<volatile uint32_t *>(status);
    cudaFreeHost(mem);
    return rc;
}
