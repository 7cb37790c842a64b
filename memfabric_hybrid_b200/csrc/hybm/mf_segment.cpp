#include "mf_segment.h"

#include <dirent.h>

#include <fcntl.h>
#include <poll.h>
#include <sys/file.h>
#include <sys/mman.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <sys/un.h>
#include <unistd.h>

#include <algorithm>
#include <mutex>
#include <random>
#include <set>

#include "../util/mf_trace.h"

#ifndef MAP_FIXED_NOREPLACE
#define MAP_FIXED_NOREPLACE 0x100000
#endif

namespace mf {
namespace hybm {

// ------------------------------------------------------------------------------------------------
FdChannel &FdChannel::Get()
{
    static FdChannel *inst = new FdChannel();  // intentionally leaked: outlives static destructors
    return *inst;
}

static socklen_t AbstractAddr(const std::string &name, sockaddr_un &sa)
{
    memset(&sa, 0, sizeof(sa));
    sa.sun_family = AF_UNIX;
    size_t n = std::min(name.size(), sizeof(sa.sun_path) - 2);
    memcpy(sa.sun_path + 1, name.data(), n);  // leading NUL: abstract namespace, nothing to unlink
    return (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
}

const std::string &FdChannel::Name()
{
    std::lock_guard<std::mutex> g(mu_);
    if (run_) return name_;
    std::random_device rd;
    name_ = "mfb200-fd-" + std::to_string(getpid()) + "-" + std::to_string(rd());
    listenFd_ = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    sockaddr_un sa;
    socklen_t sl = AbstractAddr(name_, sa);
    if (listenFd_ < 0 || bind(listenFd_, (sockaddr *)&sa, sl) != 0 || listen(listenFd_, 64) != 0) {
        MF_ERROR("fd channel: cannot listen on %s: %s", name_.c_str(), strerror(errno));
        if (listenFd_ >= 0) close(listenFd_);
        listenFd_ = -1;
        return name_;
    }
    run_ = true;
    th_ = std::thread([this] {
        pthread_setname_np(pthread_self(), "mf-fd-channel");
        Serve();
    });
    th_.detach();
    return name_;
}

void FdChannel::Serve()
{
    while (run_) {
        struct pollfd pfd = {listenFd_, POLLIN, 0};
        if (poll(&pfd, 1, 200) <= 0) continue;
        int c = accept4(listenFd_, nullptr, nullptr, SOCK_CLOEXEC);
        if (c < 0) continue;
        uint64_t token = 0;
        struct timeval tv = {2, 0};
        setsockopt(c, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
        if (recv(c, &token, sizeof(token), MSG_WAITALL) == (ssize_t)sizeof(token)) {
            int fd = -1;
            {
                std::lock_guard<std::mutex> g(mu_);
                auto it = fds_.find(token);
                if (it != fds_.end()) fd = it->second;
            }
            char ok = fd >= 0 ? 1 : 0;
            struct iovec iov = {&ok, 1};
            struct msghdr msg = {};
            msg.msg_iov = &iov;
            msg.msg_iovlen = 1;
            char ctrl[CMSG_SPACE(sizeof(int))] = {0};
            if (fd >= 0) {
                msg.msg_control = ctrl;
                msg.msg_controllen = sizeof(ctrl);
                struct cmsghdr *cm = CMSG_FIRSTHDR(&msg);
                cm->cmsg_level = SOL_SOCKET;
                cm->cmsg_type = SCM_RIGHTS;
                cm->cmsg_len = CMSG_LEN(sizeof(int));
                memcpy(CMSG_DATA(cm), &fd, sizeof(int));
            }
            sendmsg(c, &msg, MSG_NOSIGNAL);
        }
        close(c);
    }
}

uint64_t FdChannel::Publish(int fd)
{
    Name();
    std::lock_guard<std::mutex> g(mu_);
    uint64_t t = next_++;
    fds_[t] = fd;
    return t;
}

void FdChannel::Withdraw(uint64_t token)
{
    std::lock_guard<std::mutex> g(mu_);
    auto it = fds_.find(token);
    if (it == fds_.end()) return;
    close(it->second);
    fds_.erase(it);
}

int FdChannel::Fetch(const std::string &name, uint64_t token, int *fd)
{
    int s = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (s < 0) return ERR_NO_RESOURCES;
    sockaddr_un sa;
    socklen_t sl = AbstractAddr(name, sa);
    int rc = -1;
    for (int i = 0; i < 50 && rc != 0; i++) {  // the exporter may still be starting its server thread
        rc = connect(s, (sockaddr *)&sa, sl);
        if (rc != 0) usleep(10000);
    }
    if (rc != 0) {
        close(s);
        return MF_FAIL(ERR_NOT_CONNECTED, "fd channel %s unreachable: %s", name.c_str(), strerror(errno));
    }
    struct timeval tv = {5, 0};
    setsockopt(s, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
    if (send(s, &token, sizeof(token), MSG_NOSIGNAL) != (ssize_t)sizeof(token)) {
        close(s);
        return ERR_NOT_CONNECTED;
    }
    char ok = 0;
    struct iovec iov = {&ok, 1};
    char ctrl[CMSG_SPACE(sizeof(int))] = {0};
    struct msghdr msg = {};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    ssize_t n = recvmsg(s, &msg, MSG_CMSG_CLOEXEC);
    close(s);
    if (n != 1 || ok != 1) return MF_FAIL(ERR_NOT_EXIST, "fd channel %s has no token %lu", name.c_str(), (unsigned long)token);
    struct cmsghdr *cm = CMSG_FIRSTHDR(&msg);
    if (cm == nullptr || cm->cmsg_type != SCM_RIGHTS) return ERR;
    memcpy(fd, CMSG_DATA(cm), sizeof(int));
    return OK;
}

void FdChannel::Stop() { run_ = false; }

// ------------------------------------------------------------------------------------------------
int Segment::Reserve(uint32_t attempt)
{
    if (base_ != 0) return OK;
    if (opt_.slot == 0 || opt_.rankCount == 0) return ERR_INVALID_PARAM;
    MF_TRACE_BEGIN(TP_HYBM_RESERVE);
    uint64_t total = opt_.slot * opt_.rankCount;
    uint64_t hint = WindowBase(opt_.type, opt_.entityId, attempt);
    ReservedRange r;
    r.base = hint;
    r.slot = opt_.slot;
    r.ranks = opt_.rankCount;
    r.type = opt_.type;
    r.entityId = opt_.entityId;
    r.localRank = opt_.rank;
    int rc = VaManager::Get().AddReserved(r);
    if (rc == OK) {
        rc = ReserveRange(hint, total);
        if (rc != OK) VaManager::Get().RemoveReserved(hint);
        else base_ = hint;
    }
    if (rc == OK && Compact()) {
        // the window of 56-bit addresses callers see: registered so that classification and gva_to_va know it
        ReservedRange pub = r;
        pub.base = Gva56WindowBase(opt_.type, opt_.entityId, attempt);
        pub.slot = opt_.publicSlot;
        pub.localBase = base_;
        pub.localSlot = opt_.slot;
        rc = VaManager::Get().AddReserved(pub);
        if (rc == OK) {
            pubBase_ = pub.base;
        } else {
            ReleaseRange(base_, total);
            VaManager::Get().RemoveReserved(base_);
            base_ = 0;
        }
    }
    MF_TRACE_END(TP_HYBM_RESERVE, rc);
    return rc;
}

void Segment::RecomputeMapped(uint32_t rank)
{
    if (rank >= mappedBytes_.size()) return;
    // slices are laid out back to back from offset 0, so the mapped prefix is the largest run without a hole
    std::vector<std::pair<uint64_t, uint64_t>> spans;
    if (rank == opt_.rank) {
        for (auto &l : locals_) spans.emplace_back(l.slice->offset, l.slice->size);
    } else {
        for (auto &p : peers_)
            if (p.rank == rank && p.mapped) spans.emplace_back(p.offset, p.size);
    }
    std::sort(spans.begin(), spans.end());
    uint64_t end = 0;
    for (auto &sp : spans) {
        if (sp.first > end) break;
        end = std::max(end, sp.first + sp.second);
    }
    mappedBytes_[rank].store(end, std::memory_order_release);
}

int Segment::Unreserve()
{
    if (base_ == 0) return OK;
    UnmapAll();
    {
        std::lock_guard<std::mutex> g(mu_);
        for (auto &l : locals_) UnmapLocal(*l.slice);
        locals_.clear();
        localUsed_ = 0;
        for (auto &m : mappedBytes_) m.store(0);
    }
    ReleaseRange(base_, opt_.slot * opt_.rankCount);
    VaManager::Get().RemoveReserved(base_);
    if (pubBase_ != 0) VaManager::Get().RemoveReserved(pubBase_);
    pubBase_ = 0;
    base_ = 0;
    return OK;
}

int Segment::AllocLocal(uint64_t size, std::shared_ptr<MemSlice> &out)
{
    if (base_ == 0) return MF_FAIL(ERR_NOT_STARTED, "segment has no reserved range");
    uint64_t sz = AlignUp(size, Granule());
    std::lock_guard<std::mutex> g(mu_);
    if (size == 0 || localUsed_ + sz > opt_.slot)
        return MF_FAIL(ERR_NO_RESOURCES, "local slice of %lu bytes does not fit the %lu-byte slot (used %lu)%s",
                       (unsigned long)size, (unsigned long)opt_.slot, (unsigned long)localUsed_,
                       Compact() ? ": with 56-bit addresses a rank's slices share the compact slot of 16 TiB / ranks" : "");
    auto s = std::make_shared<MemSlice>();
    s->index = (uint32_t)locals_.size();
    s->memType = opt_.type;
    s->origin = SL_POOL;
    s->offset = localUsed_;
    s->size = sz;
    s->gva = base_ + opt_.slot * opt_.rank + s->offset;
    LocalRec rec;
    int rc = MapLocal(*s, rec.source, rec.token);
    if (rc != OK) return rc;
    rec.slice = s;
    locals_.push_back(rec);
    localUsed_ += sz;
    RecomputeMapped(opt_.rank);
    out = s;
    return OK;
}

int Segment::FreeLocal(const std::shared_ptr<MemSlice> &s)
{
    std::lock_guard<std::mutex> g(mu_);
    for (auto it = locals_.begin(); it != locals_.end(); ++it) {
        if (it->slice.get() != s.get()) continue;
        UnmapLocal(*it->slice);
        if (it->slice->offset + it->slice->size == localUsed_) localUsed_ = it->slice->offset;
        locals_.erase(it);
        RecomputeMapped(opt_.rank);
        return OK;
    }
    return ERR_NOT_EXIST;
}

std::vector<std::shared_ptr<MemSlice>> Segment::LocalSlices()
{
    std::lock_guard<std::mutex> g(mu_);
    std::vector<std::shared_ptr<MemSlice>> v;
    for (auto &l : locals_) v.push_back(l.slice);
    return v;
}

int Segment::Export(const MemSlice &s, hybm_exchange_info *out)
{
    std::lock_guard<std::mutex> g(mu_);
    const LocalRec *rec = nullptr;
    for (auto &l : locals_)
        if (l.slice->index == s.index && l.slice->offset == s.offset) rec = &l;
    if (rec == nullptr) return MF_FAIL(ERR_NOT_EXIST, "slice %u is not a live slice of this segment", s.index);
    ExWriter w(out);
    ExHeader h;
    h.kind = EX_SLICE;
    h.rank = opt_.rank;
    h.entityId = opt_.entityId;
    uint32_t type = opt_.type;
    int32_t pid = getpid();
    bool ok = w.Put(h) && w.Put(type) && w.Put(s.index) && w.Put(s.offset) && w.Put(s.size) && w.Put(opt_.slot) &&
              w.Put(base_) && w.Put(pid) && w.Put(rec->token) && w.PutStr(rec->source);
    return ok ? OK : MF_FAIL(ERR, "slice export does not fit the exchange blob");
}

int Segment::Import(const hybm_exchange_info &in, uint64_t *addr)
{
    ExReader r(&in);
    ExHeader h;
    uint32_t type = 0;
    PeerSlice p;
    uint64_t slot = 0, base = 0;
    if (!r.Take(h) || h.magic != kExMagic || h.version != kExVersion || h.kind != EX_SLICE || !r.Take(type) ||
        !r.Take(p.index) || !r.Take(p.offset) || !r.Take(p.size) || !r.Take(slot) || !r.Take(base) || !r.Take(p.pid) ||
        !r.Take(p.token) || !r.TakeStr(p.source))
        return MF_FAIL(ERR_INVALID_PARAM, "malformed slice exchange blob");
    if (type != (uint32_t)opt_.type) return ERR_NOT_EXIST;  // belongs to the entity's other segment
    // offset and size come from another process: compared one by one, their sum could wrap
    if (h.rank >= opt_.rankCount || slot != opt_.slot || p.size == 0 || p.offset > opt_.slot || p.size > opt_.slot - p.offset)
        return MF_FAIL(ERR_INVALID_PARAM, "slice of rank %u does not match this pool's layout (slot %lu vs %lu)", h.rank,
                       (unsigned long)slot, (unsigned long)opt_.slot);
    if (base != base_)
        return MF_FAIL(ERR_INVALID_PARAM, "rank %u reserved its pool at %#lx, this rank at %#lx", h.rank, (unsigned long)base,
                       (unsigned long)base_);
    p.rank = h.rank;
    if (addr != nullptr) *addr = ToPublic(base_ + opt_.slot * p.rank + p.offset);
    if (p.rank == opt_.rank) return OK;  // our own slice is already mapped
    std::lock_guard<std::mutex> g(mu_);
    for (auto &e : peers_)
        if (e.rank == p.rank && e.index == p.index && e.offset == p.offset) {
            if (e.token == p.token && e.source == p.source) return OK;
            if (e.mapped) UnmapPeer(e);  // the peer came back with a new incarnation
            e = p;
            return OK;
        }
    peers_.push_back(p);
    return OK;
}

int Segment::Mmap()
{
    MF_TRACE_BEGIN(TP_HYBM_MMAP);
    std::lock_guard<std::mutex> g(mu_);
    int rc = OK;
    for (auto &p : peers_) {
        if (p.mapped) continue;
        int r = MapPeer(p);
        if (r != OK) {
            rc = r;
            break;
        }
        p.mapped = true;
        RecomputeMapped(p.rank);
    }
    MF_TRACE_END(TP_HYBM_MMAP, rc);
    return rc;
}

void Segment::UnmapAll()
{
    std::lock_guard<std::mutex> g(mu_);
    for (auto &p : peers_)
        if (p.mapped) {
            UnmapPeer(p);
            p.mapped = false;
        }
    peers_.clear();
    for (uint32_t r = 0; r < mappedBytes_.size(); r++)
        if (r != opt_.rank) mappedBytes_[r].store(0);
}

int Segment::RemoveImported(uint32_t rank)
{
    std::lock_guard<std::mutex> g(mu_);
    for (auto it = peers_.begin(); it != peers_.end();) {
        if (it->rank != rank) {
            ++it;
            continue;
        }
        if (it->mapped) UnmapPeer(*it);
        it = peers_.erase(it);
    }
    RecomputeMapped(rank);
    return OK;
}

bool Segment::RankMapped(uint32_t rank)
{
    if (rank == opt_.rank) return true;
    std::lock_guard<std::mutex> g(mu_);
    for (auto &p : peers_)
        if (p.rank == rank && p.mapped) return true;
    return false;
}

// ------------------------------------------------------------------------------------------------
namespace {

class HostShmSegment : public Segment {
public:
    using Segment::Segment;
    ~HostShmSegment() override { Unreserve(); }

protected:
    uint64_t Granule() const override { return 2ULL << 20; }

    int ReserveRange(uint64_t hint, uint64_t size) override
    {
        void *p = mmap(reinterpret_cast<void *>(hint), size, PROT_NONE,
                       MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE | MAP_FIXED_NOREPLACE, -1, 0);
        if (p == MAP_FAILED || reinterpret_cast<uint64_t>(p) != hint) {
            if (p != MAP_FAILED) munmap(p, size);
            return MF_FAIL(ERR_NO_RESOURCES, "cannot reserve DRAM window %#lx+%#lx: %s", (unsigned long)hint,
                           (unsigned long)size, strerror(errno));
        }
        return OK;
    }
    int ReleaseRange(uint64_t base, uint64_t size) override { return munmap(reinterpret_cast<void *>(base), size) == 0 ? OK : ERR; }

    int MapAt(uint64_t va, uint64_t size, int fd, bool populate)
    {
        int flags = MAP_SHARED | MAP_FIXED | (populate ? MAP_POPULATE : 0);
        void *p = mmap(reinterpret_cast<void *>(va), size, PROT_READ | PROT_WRITE, flags, fd, 0);
        if (p == MAP_FAILED) return MF_FAIL(ERR, "mmap of pooled DRAM at %#lx failed: %s", (unsigned long)va, strerror(errno));
        if (opt_.dev != nullptr && opt_.dev->Caps().present) {
            int rc = opt_.dev->HostRegister(p, size);
            if (rc != OK) MF_WARN("pooled DRAM at %#lx could not be pinned (rc %d): device copies will be staged", (unsigned long)va, rc);
        }
        return OK;
    }
    void UnmapAt(uint64_t va, uint64_t size)
    {
        if (opt_.dev != nullptr && opt_.dev->Caps().present) opt_.dev->HostUnregister(reinterpret_cast<void *>(va));
        mmap(reinterpret_cast<void *>(va), size, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE | MAP_FIXED, -1, 0);
    }

    // Backing files this process created and has not unlinked yet: whatever is left when the process exits normally
    // (a pool that was never destroyed) is unlinked then.
    struct OwnedFiles {
        std::mutex mu;
        std::set<std::string> paths;
        void Add(const std::string &p)
        {
            std::lock_guard<std::mutex> g(mu);
            paths.insert(p);
        }
        void Drop(const std::string &p)
        {
            std::lock_guard<std::mutex> g(mu);
            paths.erase(p);
        }
        ~OwnedFiles()
        {
            for (auto &p : paths) unlink(p.c_str());
        }
    };
    static OwnedFiles &Owned()
    {
        static OwnedFiles o;
        return o;
    }

    // Backing files of this user whose owner no longer lives (it held an exclusive flock for its lifetime and never
    // got to unlink them: killed, or exited without destroying its pool) are removed, once per process. Peers that
    // still map such a file keep their mapping. Parity: src/hybm/csrc/mm/hybm_host_shm_segment.cpp:390-466 (stale cleanup).
    static void RemoveStaleFiles(const char *dir)
    {
        static std::once_flag once;
        std::call_once(once, [dir] {
            DIR *d = opendir(dir);
            if (d == nullptr) return;
            const std::string prefix = "memfabric_b200_" + std::to_string(geteuid()) + "_";
            while (struct dirent *e = readdir(d)) {
                if (strncmp(e->d_name, prefix.c_str(), prefix.size()) != 0) continue;
                const std::string path = std::string(dir) + "/" + e->d_name;
                int fd = open(path.c_str(), O_RDWR | O_CLOEXEC);
                if (fd < 0) continue;
                struct stat st;
                // a file younger than a minute may belong to a process that has created it and not locked it yet
                if (fstat(fd, &st) != 0 || time(nullptr) - st.st_ctime < 60) {
                    close(fd);
                    continue;
                }
                if (flock(fd, LOCK_EX | LOCK_NB) == 0) {
                    unlink(path.c_str());
                    MF_INFO("removed the stale pool file %s", path.c_str());
                }
                close(fd);
            }
            closedir(d);
        });
    }

    int MapLocal(MemSlice &s, std::string &source, uint64_t &token) override
    {
        int fd = -1;
        if ((opt_.flags & HYBM_FLAG_CREATE_WITH_SHM) != 0 && opt_.shmFd >= 0 && s.index == 0) {
            // Caller-provided backing file: peers receive it through the fd channel.
            fd = fcntl(opt_.shmFd, F_DUPFD_CLOEXEC, 0);
            struct stat st;
            if (fd < 0 || fstat(fd, &st) != 0 || (uint64_t)st.st_size < s.size) {
                if (fd >= 0) close(fd);
                return MF_FAIL(ERR_INVALID_PARAM, "dramShmFd is not a file of at least %lu bytes", (unsigned long)s.size);
            }
            source = "@" + FdChannel::Get().Name();
            token = FdChannel::Get().Publish(fcntl(fd, F_DUPFD_CLOEXEC, 0));
        } else if (EnvInt("MF_DRAM_POOL_FILES", nullptr, 0, 0, 1) == 0) {
            // Default: an anonymous memory file handed to the peers as a descriptor through the fd channel. It has no
            // name, so nothing can be left behind in /dev/shm however the process ends (children of Python's
            // multiprocessing leave through _exit and run no destructor).
            fd = memfd_create("memfabric_b200_pool", MFD_CLOEXEC);
            if (fd < 0) return MF_FAIL(ERR_NO_RESOURCES, "memfd_create: %s", strerror(errno));
            if (ftruncate(fd, (off_t)s.size) != 0) {
                int e = errno;
                close(fd);
                return MF_FAIL(ERR_MALLOC, "cannot size the pool's memory file to %lu bytes: %s", (unsigned long)s.size, strerror(e));
            }
            source = "@" + FdChannel::Get().Name();
            token = FdChannel::Get().Publish(fcntl(fd, F_DUPFD_CLOEXEC, 0));
        } else {
            std::random_device rd;
            const char *dir = access("/dev/shm", W_OK) == 0 ? "/dev/shm" : "/tmp";
            RemoveStaleFiles(dir);
            for (int attempt = 0; attempt < 8 && fd < 0; attempt++) {
                source = std::string(dir) + "/memfabric_b200_" + std::to_string(geteuid()) + "_" + std::to_string(opt_.entityId) +
                         "_" + std::to_string(opt_.rank) + "_" + std::to_string(s.index) + "_" + std::to_string(rd());
                fd = open(source.c_str(), O_CREAT | O_EXCL | O_RDWR | O_CLOEXEC, 0600);
            }
            if (fd < 0) return MF_FAIL(ERR_NO_RESOURCES, "cannot create %s: %s", source.c_str(), strerror(errno));
            flock(fd, LOCK_EX | LOCK_NB);  // marks the file as owned by a live process
            if (ftruncate(fd, (off_t)s.size) != 0) {
                int e = errno;
                close(fd);
                unlink(source.c_str());
                return MF_FAIL(ERR_MALLOC, "cannot size %s to %lu bytes: %s", source.c_str(), (unsigned long)s.size, strerror(e));
            }
        }
        int rc = MapAt(s.gva, s.size, fd, s.size <= (4ULL << 30));  // larger slices fault in on first touch
        if (rc != OK) {
            close(fd);
            if (source[0] != '@') unlink(source.c_str());
            else FdChannel::Get().Withdraw(token);
            return rc;
        }
        ownFds_[s.index] = fd;
        ownFiles_[s.index] = source;
        if (source[0] == '@') ownTokens_[s.index] = token;
        else Owned().Add(source);
        return OK;
    }
    int UnmapLocal(MemSlice &s) override
    {
        UnmapAt(s.gva, s.size);
        auto f = ownFds_.find(s.index);
        if (f != ownFds_.end()) {
            close(f->second);
            ownFds_.erase(f);
        }
        auto t = ownTokens_.find(s.index);
        if (t != ownTokens_.end()) {
            FdChannel::Get().Withdraw(t->second);  // the descriptor kept for peers: without this the memory file outlives the pool
            ownTokens_.erase(t);
        }
        auto n = ownFiles_.find(s.index);
        if (n != ownFiles_.end()) {
            if (!n->second.empty() && n->second[0] != '@') {
                unlink(n->second.c_str());
                Owned().Drop(n->second);
            }
            ownFiles_.erase(n);
        }
        return OK;
    }
    int MapPeer(PeerSlice &p) override
    {
        int fd = -1;
        if (!p.source.empty() && p.source[0] == '@') {
            int rc = FdChannel::Fetch(p.source.substr(1), p.token, &fd);
            if (rc != OK) return rc;
        } else {
            for (int i = 0; i < 50 && fd < 0; i++) {
                fd = open(p.source.c_str(), O_RDWR | O_CLOEXEC);
                if (fd < 0) usleep(10000);
            }
            if (fd < 0) return MF_FAIL(ERR_NOT_EXIST, "peer rank %u DRAM file %s: %s", p.rank, p.source.c_str(), strerror(errno));
        }
        uint64_t va = base_ + opt_.slot * p.rank + p.offset;
        // the owner has touched every page already: filling this process's page table now (as the reference does on
        // import, hybm_host_shm_segment.cpp:468-540) keeps minor faults out of the first copies; very large slices are
        // left to fault in on demand so that a join does not stall
        int rc = MapAt(va, p.size, fd, p.size <= (4ULL << 30));
        close(fd);
        return rc;
    }
    int UnmapPeer(PeerSlice &p) override
    {
        UnmapAt(base_ + opt_.slot * p.rank + p.offset, p.size);
        return OK;
    }

private:
    std::map<uint32_t, int> ownFds_;
    std::map<uint32_t, std::string> ownFiles_;
    std::map<uint32_t, uint64_t> ownTokens_;  // fd-channel tokens of the descriptors published for peers
};

class VmmSegment : public Segment {
public:
    using Segment::Segment;
    ~VmmSegment() override { Unreserve(); }

protected:
    uint64_t Granule() const override { return std::max<uint64_t>(opt_.dev->Caps().granularity, kHbmGranule); }
    // The driver honours a fixed-address request reliably only for large ranges (observed on B200, driver 580:
    // below 512 MiB the hint is ignored once another allocator of the process has initialised), so the
    // reservation, not the slot, is rounded up to a whole GiB; address space inside a window is plentiful.
    static uint64_t ReserveBytes(uint64_t size) { return AlignUp(size, 1ULL << 30); }
    int ReserveRange(uint64_t hint, uint64_t size) override
    {
        size = ReserveBytes(size);
        uint64_t va = 0;
        int rc = opt_.dev->Reserve(hint, size, &va);
        if (rc != OK || va != hint) {
            if (rc == OK) opt_.dev->ReleaseVa(va, size);
            return MF_FAIL(ERR_NO_RESOURCES, "cannot reserve HBM window %#lx+%#lx on %s", (unsigned long)hint,
                           (unsigned long)size, opt_.dev->Name());
        }
        return OK;
    }
    int ReleaseRange(uint64_t base, uint64_t size) override { return opt_.dev->ReleaseVa(base, ReserveBytes(size)); }
    int MapLocal(MemSlice &s, std::string &source, uint64_t &token) override
    {
        PhysHandle h = 0;
        int rc = opt_.dev->CreatePhys(s.size, &h);
        if (rc != OK) return rc;
        rc = opt_.dev->Map(s.gva, s.size, h);
        if (rc != OK) {
            opt_.dev->ReleasePhys(h);
            return rc;
        }
        int fd = -1;
        rc = opt_.dev->ExportFd(h, &fd);
        if (rc != OK) {
            opt_.dev->Unmap(s.gva, s.size);
            opt_.dev->ReleasePhys(h);
            return MF_FAIL(rc, "cannot export HBM slice as a file descriptor");
        }
        source = FdChannel::Get().Name();
        token = FdChannel::Get().Publish(fd);
        ownPhys_[s.index] = h;
        ownTokens_[s.index] = token;
        return OK;
    }
    int UnmapLocal(MemSlice &s) override
    {
        opt_.dev->Unmap(s.gva, s.size);
        auto it = ownPhys_.find(s.index);
        if (it != ownPhys_.end()) {
            opt_.dev->ReleasePhys(it->second);
            ownPhys_.erase(it);
        }
        auto t = ownTokens_.find(s.index);
        if (t != ownTokens_.end()) {
            FdChannel::Get().Withdraw(t->second);
            ownTokens_.erase(t);
        }
        return OK;
    }
    int MapPeer(PeerSlice &p) override
    {
        int fd = -1;
        int rc = FdChannel::Fetch(p.source, p.token, &fd);
        if (rc != OK) return rc;
        rc = opt_.dev->ImportFd(fd, p.size, &p.phys);
        if (rc != OK) return MF_FAIL(rc, "cannot import HBM slice of rank %u", p.rank);
        rc = opt_.dev->Map(base_ + opt_.slot * p.rank + p.offset, p.size, p.phys);
        if (rc != OK) {
            opt_.dev->ReleasePhys(p.phys);
            p.phys = 0;
        }
        return rc;
    }
    int UnmapPeer(PeerSlice &p) override
    {
        opt_.dev->Unmap(base_ + opt_.slot * p.rank + p.offset, p.size);
        if (p.phys != 0) opt_.dev->ReleasePhys(p.phys);
        p.phys = 0;
        return OK;
    }

private:
    std::map<uint32_t, PhysHandle> ownPhys_;
    std::map<uint32_t, uint64_t> ownTokens_;
};

}  // namespace

std::shared_ptr<Segment> Segment::Create(const SegmentOptions &o)
{
    if (o.type == HYBM_MEM_TYPE_HOST) return std::make_shared<HostShmSegment>(o);
    if (o.dev == nullptr || !o.dev->Caps().vmm) {
        MF_FAIL(ERR_NOT_INIT, "an HBM pool needs a device backend with virtual memory management");
        return nullptr;
    }
    return std::make_shared<VmmSegment>(o);
}

}  // namespace hybm
}  // namespace mf
