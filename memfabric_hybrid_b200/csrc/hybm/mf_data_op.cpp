#include "mf_data_op.h"

#include <sys/uio.h>

#include <algorithm>

#include "../util/mf_trace.h"

namespace mf {
namespace hybm {

namespace {
constexpr uint64_t kKiB = 1024;
bool DeviceVisible(const Endpoint &e, bool devPresent)
{
    return e.kind == EP_DEVICE || (e.kind == EP_HOST_PINNED && devPresent);
}
bool HostAddressable(const Endpoint &e, bool devPresent)
{
    // With the fake backend "device" memory is host memory, so every local kind is memcpy-able.
    return e.kind == EP_HOST || e.kind == EP_HOST_PINNED || (e.kind == EP_DEVICE && !devPresent);
}
}  // namespace

ComposeDataOp::ComposeDataOp(DeviceBackend *dev, uint32_t opMask) : dev_(dev), mask_(opMask)
{
    chunk_ = (uint64_t)EnvInt("MF_XCOPY_CHUNK_KB", nullptr, 256, 4, 65536) * kKiB;
    hostSplit_ = 1ULL << 20;
    engineMin_ = (uint64_t)EnvInt("MF_XCOPY_ENGINE_MIN_MB", nullptr, 64, 0, 1 << 20) << 20;  // 0: never
    size_t threads = (size_t)EnvInt("MF_HOST_COPY_THREADS", nullptr, 4, 1, 64);
    pool_ = std::make_unique<ThreadPool>(threads, "mf-hcopy");
}

ComposeDataOp::~ComposeDataOp()
{
    Wait();
    if (dev_ != nullptr) {
        if (ring_ != nullptr) dev_->HostFree(ring_);
        if (stream_ != nullptr) dev_->StreamDestroy(stream_);
    }
}

int ComposeDataOp::EnsureRing()
{
    if (ring_ != nullptr) return OK;
    if (dev_ == nullptr) return ERR_NOT_INIT;
    uint64_t bytes = (uint64_t)EnvInt("MF_XCOPY_RING_MB", nullptr, 32, 1, 1024) << 20;  // 1.4 M descriptors: a dozen of the largest batches between wraps
    void *p = nullptr;
    int rc = dev_->HostAlloc(bytes, &p);
    if (rc != OK) return MF_FAIL(rc, "cannot allocate the %lu-byte pinned descriptor ring", (unsigned long)bytes);
    ring_ = static_cast<CopyItem *>(p);
    ringCap_ = bytes / sizeof(CopyItem);
    ringHead_ = 0;
    return OK;
}

void *ComposeDataOp::StreamFor(void *userStream, uint32_t flags)
{
    if (userStream != nullptr && (flags & (1u << 2)) != 0) return userStream;  // caller's stream flag
    if (stream_ == nullptr && dev_ != nullptr) {
        dev_->BindThread();
        if (dev_->StreamCreate(&stream_) != OK) stream_ = nullptr;
    }
    return stream_;
}

int ComposeDataOp::CheckCopyStatus()
{
    if (dev_ == nullptr) return OK;
    const uint32_t code = dev_->CopyStatus(true);
    if (code == 0) return OK;
    return MF_FAIL(ERR_TIMEOUT, "copy kernel gave up a bounded wait (code %#x): the data of that batch is incomplete", code);
}

bool ComposeDataOp::HostFast(const ResolvedCopy &c)
{
    const bool devPresent = dev_ != nullptr && dev_->Caps().present;
    if (c.len >= 2 * hostSplit_ || !HostAddressable(c.src, devPresent) || !HostAddressable(c.dst, devPresent)) return false;
    MF_TRACE_BEGIN(TP_HYBM_LH_TO_GH);
    memmove(reinterpret_cast<void *>(c.dst.addr), reinterpret_cast<const void *>(c.src.addr), c.len);
    MF_TRACE_END(TP_HYBM_LH_TO_GH, 0);
    fastHost_.fetch_add(1, std::memory_order_relaxed);
    return true;
}

int ComposeDataOp::RunHost(const ResolvedCopy &c)
{
    char *d = reinterpret_cast<char *>(c.dst.addr);
    const char *s = reinterpret_cast<const char *>(c.src.addr);
    if (c.len < 2 * hostSplit_ || pool_->Size() <= 1) {
        memmove(d, s, c.len);
        return OK;
    }
    bool overlap = (d < s + c.len) && (s < d + c.len);
    if (overlap) {
        memmove(d, s, c.len);
        return OK;
    }
    size_t parts = std::min<size_t>(pool_->Size(), (size_t)(c.len / hostSplit_));
    uint64_t per = AlignUp(c.len / parts, 4096);
    std::vector<std::future<int>> futs;
    for (size_t i = 1; i < parts; i++) {
        uint64_t off = per * i;
        if (off >= c.len) break;
        uint64_t n = std::min(per, c.len - off);
        futs.push_back(pool_->Submit([d, s, off, n]() -> int {
            memcpy(d + off, s + off, n);
            return 0;
        }));
    }
    memcpy(d, s, std::min(per, c.len));
    for (auto &f : futs) f.get();
    return OK;
}

int ComposeDataOp::RunVm(const ResolvedCopy &c)
{
    // Exactly one side lives in another process. The local side must be host-addressable.
    bool read = c.src.kind == EP_REMOTE_VM;
    const Endpoint &remote = read ? c.src : c.dst;
    const Endpoint &local = read ? c.dst : c.src;
    bool devPresent = dev_ != nullptr && dev_->Caps().present;
    std::vector<char> bounce;
    uint64_t localAddr = local.addr;
    if (!HostAddressable(local, devPresent)) {
        bounce.resize(c.len);
        localAddr = reinterpret_cast<uint64_t>(bounce.data());
        if (!read) {
            int rc = dev_->MemcpyAsync(localAddr, local.addr, c.len, CPY_D2H, StreamFor(nullptr, 0));
            if (rc == OK) rc = dev_->StreamSync(StreamFor(nullptr, 0));
            if (rc != OK) return rc;
        }
    }
    uint64_t done = 0;
    while (done < c.len) {
        struct iovec l = {reinterpret_cast<void *>(localAddr + done), (size_t)(c.len - done)};
        struct iovec r = {reinterpret_cast<void *>(remote.addr + done), (size_t)(c.len - done)};
        ssize_t n = read ? process_vm_readv(remote.pid, &l, 1, &r, 1, 0) : process_vm_writev(remote.pid, &l, 1, &r, 1, 0);
        if (n <= 0)
            return MF_FAIL(ERR_NOT_CONNECTED, "process_vm_%s pid %d addr %#lx: %s", read ? "readv" : "writev", remote.pid,
                           (unsigned long)remote.addr, n == 0 ? "no progress" : strerror(errno));
        done += (uint64_t)n;
    }
    if (!bounce.empty() && read) {
        int rc = dev_->MemcpyAsync(local.addr, localAddr, c.len, CPY_H2D, StreamFor(nullptr, 0));
        if (rc == OK) rc = dev_->StreamSync(StreamFor(nullptr, 0));
        if (rc != OK) return rc;
    }
    return OK;
}

int ComposeDataOp::RunEngine(const ResolvedCopy &c, void *stream)
{
    MemcpyKind k = CPY_AUTO;
    bool sd = c.src.kind == EP_DEVICE, dd = c.dst.kind == EP_DEVICE;
    if (sd && dd) k = CPY_D2D;
    else if (sd) k = CPY_D2H;
    else if (dd) k = CPY_H2D;
    else k = CPY_H2H;
    return dev_->MemcpyAsync(c.dst.addr, c.src.addr, c.len, k, stream);
}

int ComposeDataOp::RunKernel(const std::vector<const ResolvedCopy *> &items, void *stream)
{
    int rc = EnsureRing();
    if (rc != OK) return rc;
    uint64_t total = 0, alignMask = 0;
    bool allDevice = true;
    for (auto *c : items) {
        total += c->len;
        alignMask |= c->src.addr | c->dst.addr | c->len;
        allDevice = allDevice && c->src.kind == EP_DEVICE && c->dst.kind == EP_DEVICE;
    }
    const bool bulkOk = allDevice && (alignMask & 15) == 0;
    // Equal work chunks: small enough to fill every SM a few times over, large enough to amortise the
    // descriptor fetch. Multiples of 4 KiB keep the alignment of every chunk equal to that of its item.
    uint64_t sms = std::max(1, dev_->Caps().smCount);
    uint64_t chunk = AlignUp(std::max<uint64_t>(total / (sms * 8), 1), 4096);
    chunk = std::min(std::max<uint64_t>(chunk, 16 * kKiB), chunk_);
    MF_TRACE_BEGIN(TP_HYBM_BATCH_KERNEL);
    size_t i = 0;
    uint64_t off = 0;
    while (i < items.size()) {
        if (ringHead_ >= ringCap_) {  // every slot handed out: wait for the launches that may still read them
            for (void *s : ringUsers_) dev_->StreamSync(s);
            ringUsers_.clear();
            ringHead_ = 0;
        }
        uint64_t first = ringHead_, n = 0;
        while (i < items.size() && first + n < ringCap_) {
            const ResolvedCopy *c = items[i];
            uint64_t len = std::min(chunk, c->len - off);
            ring_[first + n] = CopyItem{c->src.addr + off, c->dst.addr + off, len};
            n++;
            off += len;
            if (off >= c->len) {
                i++;
                off = 0;
            }
        }
        if (n == 0) continue;
        rc = dev_->LaunchBatchCopy(ring_ + first, (uint32_t)n, stream, bulkOk);
        if (rc != OK) break;
        ringHead_ = first + n;
        if (std::find(ringUsers_.begin(), ringUsers_.end(), stream) == ringUsers_.end()) ringUsers_.push_back(stream);
        stats_.kernelLaunches++;
        stats_.kernelItems += n;
    }
    MF_TRACE_END(TP_HYBM_BATCH_KERNEL, rc);
    return rc;
}

int ComposeDataOp::Submit(std::vector<ResolvedCopy> &items, void *userStream, uint32_t flags, int32_t *perItem)
{
    if (items.empty()) return OK;
    std::lock_guard<std::mutex> g(mu_);
    bool devPresent = dev_ != nullptr && dev_->Caps().present;
    if (dev_ != nullptr) dev_->BindThread();

    // 1. merge address-adjacent neighbours (same kinds, same process)
    if (perItem == nullptr && items.size() > 1) {
        size_t w = 0;
        for (size_t r = 1; r < items.size(); r++) {
            ResolvedCopy &a = items[w];
            const ResolvedCopy &b = items[r];
            if (a.src.kind == b.src.kind && a.dst.kind == b.dst.kind && a.src.pid == b.src.pid && a.dst.pid == b.dst.pid &&
                a.src.addr + a.len == b.src.addr && a.dst.addr + a.len == b.dst.addr) {
                a.len += b.len;
                stats_.coalesced++;
            } else {
                items[++w] = b;
            }
        }
        items.resize(w + 1);
    }

    // 2. route
    std::vector<const ResolvedCopy *> kernelItems;
    std::vector<const ResolvedCopy *> engineItems;
    int firstErr = OK;
    auto fail = [&](const ResolvedCopy &c, int rc) {
        if (perItem != nullptr) perItem[c.index] = rc;
        if (firstErr == OK) firstErr = rc;
    };
    bool forceKernel = (flags & (1u << 1)) != 0;  // COPY_EXTEND_FLAG
    for (auto &c : items) {
        if (c.len == 0) continue;
        if (c.src.kind == EP_REMOTE_VM || c.dst.kind == EP_REMOTE_VM) {
            if (c.src.kind == EP_REMOTE_VM && c.dst.kind == EP_REMOTE_VM) {
                fail(c, ERR_INVALID_PARAM);
                continue;
            }
            int rc = RunVm(c);
            stats_.vmCopies++;
            if (rc != OK) fail(c, rc);
            continue;
        }
        bool sHost = c.src.kind != EP_DEVICE, dHost = c.dst.kind != EP_DEVICE;
        if ((sHost && dHost) || !devPresent) {
            if (dev_ != nullptr && !devPresent && (c.src.kind == EP_DEVICE || c.dst.kind == EP_DEVICE)) {
                kernelItems.push_back(&c);  // fake backend: exercise the batch path
                continue;
            }
            MF_TRACE_BEGIN(TP_HYBM_LH_TO_GH);
            int rc = RunHost(c);
            MF_TRACE_END(TP_HYBM_LH_TO_GH, rc);
            stats_.hostCopies++;
            if (rc != OK) fail(c, rc);
            continue;
        }
        if (dev_ == nullptr) {
            fail(c, ERR_NOT_INIT);
            continue;
        }
        bool bothVisible = DeviceVisible(c.src, devPresent) && DeviceVisible(c.dst, devPresent);
        bool d2d = !sHost && !dHost;
        // Device<->device always goes to the SM kernel. A pinned host leg goes to the kernel when the
        // pieces are small (one launch instead of one engine submission per segment).
        // A long contiguous device<->device run is better off on a copy engine (its NVLink writes are wider than what
        // SM stores produce: 772 against 709 GB/s measured between two B200s), unless the caller asks for the kernel.
        const bool bigD2d = d2d && !forceKernel && engineMin_ != 0 && c.len >= engineMin_;
        if (bothVisible && !bigD2d && (d2d || forceKernel || c.len <= (4ULL << 20))) kernelItems.push_back(&c);
        else engineItems.push_back(&c);
    }

    void *stream = StreamFor(userStream, flags);
    int rc = OK;
    if (!kernelItems.empty()) {
        rc = RunKernel(kernelItems, stream);
        if (rc != OK) {
            MF_WARN("xcopy kernel launch failed (%d): falling back to the copy engine for %zu items", rc, kernelItems.size());
            for (auto *c : kernelItems) engineItems.push_back(c);
            rc = OK;
        }
    }
    if (!engineItems.empty()) {
        MF_TRACE_BEGIN(TP_HYBM_BATCH_HOST_LEG);
        for (auto *c : engineItems) {
            int r = RunEngine(*c, stream);
            stats_.engineCopies++;
            if (r != OK) fail(*c, r);
        }
        MF_TRACE_END(TP_HYBM_BATCH_HOST_LEG, firstErr);
    }
    if (!kernelItems.empty() || !engineItems.empty()) {
        if ((flags & 1u) != 0) {  // ASYNC_COPY_FLAG
            pending_ = true;
        } else if (dev_ != nullptr) {
            int r = dev_->StreamSync(stream);
            if (r == OK) r = CheckCopyStatus();
            if (r != OK && firstErr == OK) firstErr = r;
            if (stream == stream_) {
                ringUsers_.erase(std::remove(ringUsers_.begin(), ringUsers_.end(), stream), ringUsers_.end());
                if (ringUsers_.empty()) ringHead_ = 0;
            }
        }
    }
    return firstErr != OK ? firstErr : rc;
}

// ------------------------------------------------------------------------------------------------
KernelBatch::KernelBatch(ComposeDataOp &op, void *userStream, uint32_t flags, uint64_t totalBytes)
    : op_(op), lock_(op.mu_), flags_(flags)
{
    if (op_.dev_ == nullptr) {
        rc_ = ERR_NOT_INIT;
        return;
    }
    op_.dev_->BindThread();
    rc_ = op_.EnsureRing();
    if (rc_ != OK) return;
    stream_ = op_.StreamFor(userStream, flags);
    uint64_t sms = std::max(1, op_.dev_->Caps().smCount);
    uint64_t chunk = AlignUp(std::max<uint64_t>(totalBytes / (sms * 8), 1), 4096);
    chunk_ = std::min(std::max<uint64_t>(chunk, 16 * kKiB), op_.chunk_);
    if (op_.ringHead_ >= op_.ringCap_) Wrap();
    first_ = op_.ringHead_;
}

int KernelBatch::Launch()
{
    uint64_t n = op_.ringHead_ - first_;
    if (n == 0) return OK;
    int rc = op_.dev_->LaunchBatchCopy(op_.ring_ + first_, (uint32_t)n, stream_, (alignMask_ & 15) == 0);
    if (rc != OK) return rc;
    if (std::find(op_.ringUsers_.begin(), op_.ringUsers_.end(), stream_) == op_.ringUsers_.end()) op_.ringUsers_.push_back(stream_);
    op_.stats_.kernelLaunches++;
    op_.stats_.kernelItems += n;
    first_ = op_.ringHead_;
    return OK;
}

void KernelBatch::Wrap()
{
    // every slot is handed out: launch what this batch wrote, wait for all readers, start over
    int rc = Launch();
    if (rc != OK && rc_ == OK) rc_ = rc;
    for (void *s : op_.ringUsers_) op_.dev_->StreamSync(s);
    op_.ringUsers_.clear();
    op_.ringHead_ = 0;
    first_ = 0;
}

int KernelBatch::Finish()
{
    if (rc_ != OK) return rc_;
    if (pendLen_ != 0) Emit();
    MF_TRACE_BEGIN(TP_HYBM_BATCH_KERNEL);
    int rc = Launch();
    if (rc == OK && rc_ != OK) rc = rc_;
    if (rc == OK) {
        if ((flags_ & 1u) != 0) {
            op_.pending_ = true;
        } else {
            rc = op_.dev_->StreamSync(stream_);
            if (rc == OK) rc = op_.CheckCopyStatus();
            if (stream_ == op_.stream_) {
                auto &u = op_.ringUsers_;
                u.erase(std::remove(u.begin(), u.end(), stream_), u.end());
                if (u.empty()) op_.ringHead_ = 0;
            }
        }
    }
    MF_TRACE_END(TP_HYBM_BATCH_KERNEL, rc);
    return rc;
}

int ComposeDataOp::Prepare(const std::vector<ResolvedCopy> &items, PreparedBatch &out)
{
    if (dev_ == nullptr) return ERR_NOT_INIT;
    // merge neighbours, then cut into equal work chunks exactly as RunKernel does
    std::vector<CopyItem> runs;
    uint64_t total = 0, alignMask = 0;
    for (const auto &c : items) {
        if (c.len == 0) continue;
        if (c.src.kind != EP_DEVICE || c.dst.kind != EP_DEVICE) return MF_FAIL(ERR_INVALID_PARAM, "a prepared batch holds device-to-device copies only");
        total += c.len;
        alignMask |= c.src.addr | c.dst.addr | c.len;
        if (!runs.empty() && runs.back().src + runs.back().len == c.src.addr && runs.back().dst + runs.back().len == c.dst.addr) runs.back().len += c.len;
        else runs.push_back(CopyItem{c.src.addr, c.dst.addr, c.len});
    }
    if (runs.empty()) return MF_FAIL(ERR_INVALID_PARAM, "a prepared batch needs at least one non-empty copy");
    const uint64_t sms = std::max(1, dev_->Caps().smCount);
    uint64_t chunk = AlignUp(std::max<uint64_t>(total / (sms * 8), 1), 4096);
    chunk = std::min(std::max<uint64_t>(chunk, 16 * kKiB), chunk_);
    uint64_t n = 0;
    for (const auto &r : runs) n += (r.len + chunk - 1) / chunk;
    if (n > UINT32_MAX) return MF_FAIL(ERR_INVALID_PARAM, "batch too large");
    dev_->BindThread();
    void *mem = nullptr;
    int rc = dev_->HostAlloc(n * sizeof(CopyItem), &mem);
    if (rc != OK) return MF_FAIL(rc, "cannot allocate %lu pinned descriptors", (unsigned long)n);
    auto *d = static_cast<CopyItem *>(mem);
    uint64_t w = 0;
    for (const auto &r : runs)
        for (uint64_t off = 0; off < r.len; off += chunk) d[w++] = CopyItem{r.src + off, r.dst + off, std::min(chunk, r.len - off)};
    out.desc = d;
    out.count = (uint32_t)n;
    out.bytes = total;
    out.bulkOk = (alignMask & 15) == 0;
    return OK;
}

int ComposeDataOp::LaunchPrepared(const PreparedBatch &b, void *stream)
{
    if (dev_ == nullptr || b.desc == nullptr) return ERR_INVALID_PARAM;
    // no lock, no shared state: the descriptors belong to the batch; the launch is all there is (graph-capturable)
    int rc = dev_->LaunchBatchCopy(b.desc, b.count, stream, b.bulkOk);
    if (rc == OK) {
        fastLaunches_.fetch_add(1, std::memory_order_relaxed);
        fastItems_.fetch_add(b.count, std::memory_order_relaxed);
    }
    return rc;
}

void ComposeDataOp::ReleasePrepared(PreparedBatch &b)
{
    if (dev_ != nullptr && b.desc != nullptr) dev_->HostFree(b.desc);
    b = PreparedBatch();
}

int ComposeDataOp::Quant(const std::vector<QuantItem> &items, uint32_t unit, int inputFp16, int mode, void *userStream)
{
    if (dev_ == nullptr) return ERR_NOT_INIT;
    if (items.empty()) return OK;
    std::lock_guard<std::mutex> g(mu_);
    dev_->BindThread();
    int rc = EnsureRing();
    if (rc != OK) return rc;
    static_assert(sizeof(QuantItem) <= 2 * sizeof(CopyItem), "quant descriptors borrow ring slots");
    void *stream = userStream != nullptr ? userStream : StreamFor(nullptr, 0);
    size_t done = 0;
    while (done < items.size()) {
        uint64_t need = 2;  // slots per descriptor
        if (ringHead_ + need > ringCap_) {
            for (void *s : ringUsers_) dev_->StreamSync(s);
            ringUsers_.clear();
            ringHead_ = 0;
        }
        uint64_t room = (ringCap_ - ringHead_) / need;
        size_t n = std::min<size_t>(items.size() - done, (size_t)room);
        QuantItem *slot = reinterpret_cast<QuantItem *>(ring_ + ringHead_);
        memcpy(slot, items.data() + done, n * sizeof(QuantItem));
        rc = dev_->LaunchQuantCopy(slot, (uint32_t)n, unit, inputFp16, mode, stream);
        if (rc != OK) return rc;
        ringHead_ += n * need;
        if (std::find(ringUsers_.begin(), ringUsers_.end(), stream) == ringUsers_.end()) ringUsers_.push_back(stream);
        done += n;
    }
    if (userStream == nullptr) rc = dev_->StreamSync(stream);
    return rc;
}

int ComposeDataOp::Wait()
{
    std::lock_guard<std::mutex> g(mu_);
    if (dev_ == nullptr) return OK;
    MF_TRACE_BEGIN(TP_HYBM_WAIT);
    int rc = OK;
    if (stream_ != nullptr) rc = dev_->StreamSync(stream_);
    for (void *s : ringUsers_)
        if (s != stream_) dev_->StreamSync(s);
    ringUsers_.clear();
    ringHead_ = 0;
    pending_ = false;
    if (rc == OK) rc = CheckCopyStatus();
    MF_TRACE_END(TP_HYBM_WAIT, rc);
    return rc;
}

}  // namespace hybm
}  // namespace mf
