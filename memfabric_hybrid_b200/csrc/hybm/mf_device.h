// Device backend seam. Everything the memory layer needs from "a GPU runtime" is behind this
// interface so that the whole GVA / segment / entity / data-operation stack also runs on a machine
// without a GPU:
//   * CudaBackend (built by nvcc into libmf_cuda.so, loaded on demand): CUDA VMM
//     (cuMemAddressReserve / cuMemCreate / POSIX-FD export+import / cuMemMap / cuMemSetAccess),
//     host registration, CUDA IPC, streams, copy engines and the sm_100a xcopy kernels.
//   * FakeBackend (always available): the same operations on memfd-backed host memory, used by the
//     CPU test tier in the way the reference's unit tests run against fake vendor libraries
//     (test/ut/mock/hal_stub.cpp, test/ut/mock/CMakeLists.txt:11-90).
// Parity of role: src/hybm/csrc/under_api/dl_hybrid_api.h:28-120 (NPU/GPU switch),
// src/hybm/csrc/under_api/dl_cuda_api.cpp:42-82.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace mf {
namespace hybm {

using PhysHandle = uint64_t;  // opaque: CUmemGenericAllocationHandle or a memfd

struct CopyItem {
    uint64_t src;
    uint64_t dst;
    uint64_t len;
};

// Per-unit dynamic quantisation while copying (see LaunchQuantCopy).
struct QuantItem {
    uint64_t src;    // bf16/fp16 input, local
    uint64_t dst;    // int8 (or fp8) output, usually remote
    uint64_t scale;  // fp32 dequant factors, one per unit, usually remote
    uint64_t elems;  // number of input elements
};

enum MemcpyKind : int { CPY_H2H = 0, CPY_H2D = 1, CPY_D2H = 2, CPY_D2D = 3, CPY_AUTO = 4 };

struct DeviceCaps {
    bool present = false;       // a real device is attached
    bool vmm = false;           // virtual memory management usable
    bool posixFd = false;       // POSIX-FD shareable handles
    bool fabric = false;        // fabric handles (IMEX)
    bool multicast = false;     // NVLS multicast objects
    bool hostPtrForRegistered = true;
    int deviceCount = 0;
    int smCount = 0;
    int ccMajor = 0, ccMinor = 0;
    uint64_t granularity = 2ULL << 20;
    uint64_t totalMem = 0;
    int driverVersion = 0, runtimeVersion = 0;
    char name[64] = {0};
};

class DeviceBackend {
public:
    virtual ~DeviceBackend() = default;
    virtual const char *Name() const = 0;
    virtual int Init(int deviceId) = 0;
    virtual int DeviceId() const = 0;
    virtual const DeviceCaps &Caps() const = 0;
    virtual int BindThread() = 0;  // make the device current on the calling thread

    // ---- virtual memory management
    virtual int Reserve(uint64_t hint, uint64_t size, uint64_t *va) = 0;  // *va == hint or failure
    virtual int ReleaseVa(uint64_t va, uint64_t size) = 0;
    virtual int CreatePhys(uint64_t size, PhysHandle *h) = 0;
    virtual int ExportFd(PhysHandle h, int *fd) = 0;
    virtual int ImportFd(int fd, uint64_t size, PhysHandle *h) = 0;  // takes ownership of fd
    virtual int Map(uint64_t va, uint64_t size, PhysHandle h) = 0;   // maps and grants read/write
    virtual int Unmap(uint64_t va, uint64_t size) = 0;
    virtual int ReleasePhys(PhysHandle h) = 0;

    // ---- NVLink multicast objects (in-switch reduction / broadcast, "NVLS"); optional: a backend without
    // them returns an error from McCreate and Caps().multicast is false
    virtual int McGranularity(uint64_t size, uint32_t devices, uint64_t *gran) { (void)size, (void)devices, (void)gran; return -1; }
    virtual int McCreate(uint64_t size, uint32_t devices, PhysHandle *h) { (void)size, (void)devices, (void)h; return -1; }
    virtual int McAddDevice(PhysHandle h) { (void)h; return -1; }
    // binds [va, va + size) of THIS device's mapped memory at mcOffset of the object; every device must have
    // been added (by every process) before the first bind
    virtual int McBindAddr(PhysHandle h, uint64_t mcOffset, uint64_t va, uint64_t size) { (void)h, (void)mcOffset, (void)va, (void)size; return -1; }
    virtual int McUnbind(PhysHandle h, uint64_t mcOffset, uint64_t size) { (void)h, (void)mcOffset, (void)size; return -1; }

    // ---- plain allocations, host registration, IPC of caller-owned device buffers
    virtual int Malloc(uint64_t size, uint64_t *ptr) = 0;
    virtual int Free(uint64_t ptr) = 0;
    virtual int HostAlloc(uint64_t size, void **ptr) = 0;  // pinned + device-mapped
    virtual int HostFree(void *ptr) = 0;
    virtual int HostRegister(void *ptr, uint64_t size) = 0;
    virtual int HostUnregister(void *ptr) = 0;
    virtual int IpcExport(uint64_t ptr, uint8_t blob[64], uint64_t *base, uint64_t *size) = 0;
    virtual int IpcOpen(const uint8_t blob[64], uint64_t *ptr) = 0;
    virtual int IpcClose(uint64_t ptr) = 0;
    virtual bool IsDevicePointer(uint64_t ptr) = 0;
    // True when [ptr, ptr + len) is pinned host memory that kernels of this device can address at the same
    // value (cudaHostAlloc / cudaHostRegister under unified addressing).
    virtual bool IsPinnedHost(uint64_t ptr, uint64_t len) { (void)ptr, (void)len; return false; }
    virtual int EnablePeerAccess(int peerDevice) = 0;
    virtual int CanAccessPeer(int peerDevice) = 0;  // 1 yes, 0 no

    // ---- execution
    virtual int StreamCreate(void **stream) = 0;
    virtual int StreamDestroy(void *stream) = 0;
    virtual int StreamSync(void *stream) = 0;
    virtual int MemcpyAsync(uint64_t dst, uint64_t src, uint64_t len, MemcpyKind kind, void *stream) = 0;
    virtual int MemsetAsync(uint64_t dst, int value, uint64_t len, void *stream) = 0;
    // items live in pinned, device-visible memory (ring slots) until the stream passes this launch.
    // bulkOk: every item has source, destination and length in multiples of 16 bytes and both ends in device
    // memory, so the backend may move it with the bulk-copy (TMA) variant of the kernel.
    virtual int LaunchBatchCopy(const CopyItem *items, uint32_t count, void *stream, bool bulkOk = false) = 0;
    // Code left by a copy kernel whose bounded wait ran out (0: none); `clear` resets it.
    virtual uint32_t CopyStatus(bool clear) { (void)clear; return 0; }
    // Debug aid (MF_XCOPY_DEBUG=1): the pool window the copy kernels check every descriptor against before their first
    // access (base 0 switches the check off). Returns false when the backend has no such check.
    virtual bool SetCopyWindow(uint64_t base, uint64_t slot, uint32_t ranks, const uint64_t *mapped) { (void)base, (void)slot, (void)ranks, (void)mapped; return false; }
    // Shape of the bulk-copy kernel (pipelines per CTA, stages per pipeline, KiB per stage); 0 pipelines
    // switches it off. Takes effect for the launches that follow.
    virtual int ConfigureBulkCopy(int pipes, int stages, int pieceKb) { (void)pipes, (void)stages, (void)pieceKb; return -1; }
    // mode 0: int8 with scale = absmax/127 per `unit` elements; mode 1: fp8 e4m3 with scale = absmax/448 per 128.
    virtual int LaunchQuantCopy(const QuantItem *items, uint32_t count, uint32_t unit, int inputFp16, int mode,
                                void *stream) = 0;
};

// The fake backend; `deviceId` only labels it.
DeviceBackend *CreateFakeBackend();

// Process-wide backend selection. MF_DEVICE_BACKEND = cuda | fake | none | auto (default auto: cuda when
// libmf_cuda.so loads and sees a device, else none). Returns nullptr for "none".
DeviceBackend *AcquireBackend(int deviceId, std::string *why = nullptr);
DeviceBackend *CurrentBackend();
void ReleaseBackend();
// Address of an exported function of the CUDA library (kernel launchers), loading the library if it is not
// loaded yet; nullptr when the library or the symbol is missing.
void *CudaSymbol(const char *name);

// Symbol exported by libmf_cuda.so.
extern "C" typedef DeviceBackend *(*MfCreateCudaBackendFn)();

}  // namespace hybm
}  // namespace mf
