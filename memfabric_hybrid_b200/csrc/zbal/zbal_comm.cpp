// zbal communicators and operations.
//
// A communicator covers the world ranks first, first+step, ..., first+(size-1)*step and owns one slot of
// the communicator area: [1 MiB signals][stage A0][stage B0][stage A1][stage B1][p2p landing]. Its device
// view is a Team whose base is the slot of the group's first member and whose stride is step x the
// symmetric stride, so the kernels written for the whole world serve any strided sub-group unchanged,
// and groups never share flags. The slot index is agreed through the config store (the group's first
// member draws a unique value, the members learn it by a sub-group all-gather), so members may create
// different communicators in different orders. Point-to-point communicators are 2-member groups
// (low, high): also strided.
//
// Operations enqueue kernels on the caller's stream and return. Payloads larger than a staging buffer
// are cut into pieces; calls alternate between the two staging sets, so no trailing synchronisation is
// needed between consecutive calls.
//
// Parity of role: app/zbal/src/csrc/operators/zbal_communicator.cpp, zbal_comm_group_meta.cpp,
// zbal_operations.cpp:117-457 of the reference.
#include <algorithm>
#include <cstring>

#include "../hybm/mf_device.h"
#include "../util/mf_util.h"
#include "zbal_state.h"

namespace zbal {

int Comm::Ctas(uint64_t bytes) const
{
    int c;
    if (bytes <= (16u << 10)) c = 1;
    else if (bytes <= (64u << 10)) c = 4;
    else if (bytes <= (256u << 10)) c = 16;
    else if (bytes <= (1u << 20)) c = 32;
    else if (bytes <= (8u << 20)) c = 64;
    else c = maxCtas;
    return std::max(1, std::min(c, maxCtas));
}

std::shared_ptr<Comm> FindComm(zbal_comm_t h)
{
    State &st = S();
    std::lock_guard<std::mutex> g(st.mu);
    if (!st.up) {
        mf::LastError::Set(Z_NOT_INITIALIZED, "zbal is not bootstrapped");
        return nullptr;
    }
    for (auto &kv : st.comms)
        if (kv.second.get() == h) return kv.second;
    mf::LastError::Set(Z_INVALID_PARAM, "unknown communicator handle %p", h);
    return nullptr;
}

namespace {

// zbal dtype -> (kernel dtype for reductions, element size); kernel dtype -1: copy-only type
struct TypeInfo {
    int kdt;
    uint32_t size;
};
bool TypeOf(zbal_datatype_t t, TypeInfo &o)
{
    switch (t) {
        case ZBAL_DT_INT8: o = {-1, 1}; return true;
        case ZBAL_DT_UINT8: o = {-1, 1}; return true;
        case ZBAL_DT_INT16: o = {-1, 2}; return true;
        case ZBAL_DT_UINT16: o = {-1, 2}; return true;
        case ZBAL_DT_INT32: o = {3, 4}; return true;
        case ZBAL_DT_UINT32: o = {-1, 4}; return true;
        case ZBAL_DT_INT64: o = {-1, 8}; return true;
        case ZBAL_DT_UINT64: o = {-1, 8}; return true;
        case ZBAL_DT_FP64: o = {-1, 8}; return true;
        case ZBAL_DT_FP16: o = {1, 2}; return true;
        case ZBAL_DT_FP32: o = {2, 4}; return true;
        case ZBAL_DT_BF16: o = {0, 2}; return true;
        default: return false;
    }
}
int OpOf(zbal_reduce_op_t op)
{
    switch (op) {
        case ZBAL_REDUCE_SUM: return 0;
        case ZBAL_REDUCE_MAX: return 1;
        case ZBAL_REDUCE_MIN: return 2;
        case ZBAL_REDUCE_PROD: return 3;
        default: return -1;
    }
}

// Byte payloads travel as 4-byte or 2-byte units (the copy kernels are typed); odd byte counts are refused.
bool UnitOf(uint64_t bytes, uint64_t a, uint64_t b, int &kdt, uint32_t &unit)
{
    if (bytes % 4 == 0 && a % 4 == 0 && b % 4 == 0) {
        kdt = 2;
        unit = 4;
        return true;
    }
    if (bytes % 2 == 0 && a % 2 == 0 && b % 2 == 0) {
        kdt = 0;
        unit = 2;
        return true;
    }
    return false;
}

int Launched(int rc, const char *what)
{
    if (rc == 0) return Z_OK;
    return MF_FAIL(Z_LAUNCH_FAILED, "%s: kernel launch failed (%d)", what, rc);
}

MfCollArgs BaseArgs(Comm &c, const void *in, void *out, uint64_t n, float scale, int op, uint32_t root, uint32_t algo)
{
    MfCollArgs a{};
    a.team = c.team;
    a.in = reinterpret_cast<uint64_t>(in);
    a.out = reinterpret_cast<uint64_t>(out);
    a.n = n;
    a.scale = scale;
    a.op = op;
    a.root = root;
    a.algo = algo;
    a.epoch = c.Next(a.stage_a, a.stage_b);
    return a;
}

constexpr uint64_t kOneShotMax = 256u << 10;

// Direct mode: a buffer that lies inside this rank's slice of the symmetric heap (a tensor from the
// symmetric allocator) is reachable by the peers, so the kernels skip the staging copies. Small payloads
// stay on the staged path: it needs one handshake where direct mode needs two.
bool InSlice(const void *p, uint64_t bytes)
{
    State &st = S();
    const uint64_t a = reinterpret_cast<uint64_t>(p);
    if (p == nullptr) return false;
    if (a >= st.out.localGva && a + bytes <= st.out.localGva + st.opts.deviceMemorySize) return true;
    // expansion segments: rank r's slot of segment k starts at the segment's base + r * symmetricSize
    std::lock_guard<std::mutex> g(st.mu);
    for (uint64_t segLocal : st.extraLocal)
        if (a >= segLocal && a + bytes <= segLocal + st.opts.deviceMemorySize) return true;
    return false;
}
// The multicast alias covers the first segment only: a buffer of an expansion segment is reached by peer loads / stores.
bool InFirstSegment(const void *p, uint64_t bytes)
{
    State &st = S();
    const uint64_t a = reinterpret_cast<uint64_t>(p);
    return p != nullptr && a >= st.out.localGva && a + bytes <= st.out.localGva + st.opts.deviceMemorySize;
}
uint64_t DirectMin()
{
    static const uint64_t v = (uint64_t)mf::EnvInt("ZBAL_DIRECT_MIN_BYTES", nullptr, 256 << 10, 0, INT64_MAX);
    return v;
}

int AllReduce(Comm &c, const void *in, void *out, uint64_t n, int kdt, int odt, uint32_t es, uint32_t oes, int op, float scale, void *stream)
{
    const Launchers *L = GetLaunchers();
    if (L == nullptr) return Z_NOT_SUPPORTED;
    std::lock_guard<std::mutex> g(c.mu);
    if (n * es > DirectMin() && InSlice(in, n * es) && InSlice(out, n * oes)) {
        MfCollArgs a = BaseArgs(c, in, out, n, scale, op, 0, 1);
        const bool mc = c.team.mc_base != 0 && InFirstSegment(in, n * es) && InFirstSegment(out, n * oes);
        a.zero_copy = (mc && op == 0 && kdt == odt && kdt != 3) ? 3 : 2;  // the switch adds when it can
        return Launched(L->coll(0, kdt, odt, &a, c.Ctas(n * es), 512, stream), "all_reduce (direct)");
    }
    uint64_t piece = c.stageBytes / std::max(es, oes);
    piece -= piece % (8ull * c.size);
    uint64_t done = 0;
    while (done < n) {
        const uint64_t cnt = std::min(piece, n - done);
        MfCollArgs a = BaseArgs(c, static_cast<const char *>(in) + done * es, static_cast<char *>(out) + done * oes, cnt, scale, op, 0,
                                cnt * es <= kOneShotMax ? 0 : 1);
        int rc = Launched(L->coll(0, kdt, odt, &a, c.Ctas(cnt * es), 512, stream), "all_reduce");
        if (rc != Z_OK) return rc;
        done += cnt;
    }
    return Z_OK;
}

// A byte-wise all-gather of `bytes` per member (the building block of gather and of typed all_gather).
int AllGatherBytes(Comm &c, const void *in, void *out, uint64_t bytes, void *stream)
{
    const Launchers *L = GetLaunchers();
    if (L == nullptr) return Z_NOT_SUPPORTED;
    int kdt;
    uint32_t unit;
    if (!UnitOf(bytes, reinterpret_cast<uint64_t>(in), reinterpret_cast<uint64_t>(out), kdt, unit))
        return MF_FAIL(Z_NOT_SUPPORTED, "all_gather: %lu bytes per member at odd addresses or of odd size", (unsigned long)bytes);
    std::lock_guard<std::mutex> g(c.mu);
    const uint64_t m = bytes / unit;
    if (bytes * c.size > DirectMin() && InSlice(out, bytes * c.size)) {
        MfCollArgs a = BaseArgs(c, in, out, m, 1.f, 0, 0, 0);
        a.zero_copy = (c.team.mc_base != 0 && InFirstSegment(out, bytes * c.size)) ? 3 : 2;  // one multicast store per 16 bytes instead of one store per peer
        return Launched(L->coll(2, kdt, kdt, &a, c.Ctas(bytes * c.size), 512, stream), "all_gather (direct)");
    }
    uint64_t piece = c.stageBytes / unit / c.size;
    piece -= piece % 8;
    // a payload larger than the staging is gathered piece by piece: piece [done, done + cnt) of member r
    // lands at out[r * m + done ...], i.e. the output rows stay m apart (part_stride)
    uint64_t done = 0;
    while (done < m) {
        const uint64_t cnt = std::min(piece, m - done);
        MfCollArgs a = BaseArgs(c, static_cast<const char *>(in) + done * unit, static_cast<char *>(out) + done * unit, cnt, 1.f, 0, 0, 0);
        a.part_stride = m;
        int rc = Launched(L->coll(2, kdt, kdt, &a, c.Ctas(cnt * c.size * unit), 512, stream), "all_gather");
        if (rc != Z_OK) return rc;
        done += cnt;
    }
    return Z_OK;
}

int BroadcastBytes(Comm &c, const void *in, void *out, uint64_t bytes, uint32_t root, void *stream)
{
    const Launchers *L = GetLaunchers();
    if (L == nullptr) return Z_NOT_SUPPORTED;
    int kdt;
    uint32_t unit;
    if (!UnitOf(bytes, reinterpret_cast<uint64_t>(in), reinterpret_cast<uint64_t>(out), kdt, unit))
        return MF_FAIL(Z_NOT_SUPPORTED, "broadcast: %lu bytes at odd addresses or of odd size", (unsigned long)bytes);
    std::lock_guard<std::mutex> g(c.mu);
    const uint64_t total = bytes / unit;
    if (bytes > DirectMin() && InSlice(out, bytes)) {
        MfCollArgs a = BaseArgs(c, in, out, total, 1.f, 0, root, 0);
        a.zero_copy = (c.team.mc_base != 0 && InFirstSegment(out, bytes)) ? 3 : 2;
        return Launched(L->coll(3, kdt, kdt, &a, c.Ctas(bytes), 512, stream), "broadcast (direct)");
    }
    uint64_t piece = c.stageBytes / unit;
    piece -= piece % 8;
    uint64_t done = 0;
    while (done < total) {
        const uint64_t cnt = std::min(piece, total - done);
        MfCollArgs a = BaseArgs(c, static_cast<const char *>(in) + done * unit, static_cast<char *>(out) + done * unit, cnt, 1.f, 0, root, 0);
        int rc = Launched(L->coll(3, kdt, kdt, &a, c.Ctas(cnt * unit), 512, stream), "broadcast");
        if (rc != Z_OK) return rc;
        done += cnt;
    }
    return Z_OK;
}

int P2P(Comm &c, void *buf, uint64_t bytes, uint32_t peer, bool sending, void *stream)
{
    const Launchers *L = GetLaunchers();
    if (L == nullptr) return Z_NOT_SUPPORTED;
    if (peer >= c.size || peer == c.groupRank) return MF_FAIL(Z_INVALID_PARAM, "peer %u is not another member of '%s'", peer, c.name.c_str());
    std::lock_guard<std::mutex> g(c.mu);
    const uint32_t src = sending ? c.groupRank : peer, dst = sending ? peer : c.groupRank;
    uint64_t done = 0;
    while (done < bytes) {
        const uint64_t cnt = std::min(c.p2pBytes, bytes - done);
        MfP2PArgs a{};
        a.team = c.team;
        a.buf = reinterpret_cast<uint64_t>(buf) + done;
        a.bytes = cnt;
        a.stage_off = c.p2pOff + (uint64_t)src * c.p2pBytes;  // one landing area per sender in the receiver's slot
        a.peer = peer;
        a.epoch = ++c.p2pEpochs[{src, dst}];
        a.channel = 16 + src % 48;
        const int ctas = std::min(c.Ctas(cnt), 32);
        int rc = Launched(sending ? L->send(&a, ctas, stream) : L->recv(&a, ctas, stream), sending ? "send" : "recv");
        if (rc != Z_OK) return rc;
        done += cnt;
    }
    return Z_OK;
}

}  // namespace
}  // namespace zbal

using namespace zbal;

extern "C" int32_t zbal_is_symmetric(const void *ptr, uint64_t bytes) { return S().up && InSlice(ptr, bytes) ? 1 : 0; }

extern "C" {

int32_t zbal_comm_create(zbal_comm_options_t *o, zbal_comm_t *comm)
{
    if (o == nullptr || comm == nullptr) return MF_FAIL(Z_INVALID_PARAM, "options or comm is NULL");
    State &st = S();
    zbal_bootstrap_output_t bo;
    smem_shm_t shm;
    uint64_t slotBytes;
    uint32_t cap, spin;
    uint64_t mcBase;
    {
        std::lock_guard<std::mutex> g(st.mu);
        if (!st.up) return MF_FAIL(Z_NOT_INITIALIZED, "zbal is not bootstrapped");
        if (st.comms.count(o->name)) return MF_FAIL(Z_DUPLICATED, "communicator '%s' exists", o->name);
        bo = st.out;
        shm = st.shm;
        slotBytes = st.commSlotBytes;
        cap = st.opts.commGroupCap;
        spin = st.spinLimit;
        mcBase = st.mcBase;
    }
    if (o->name[0] == 0) return MF_FAIL(Z_INVALID_PARAM, "communicator name is empty");
    if (o->groupSize == 0 || o->groupSize > 16) return MF_FAIL(Z_INVALID_PARAM, "group size %u is outside 1..16", o->groupSize);
    const uint32_t step = o->groupSize == 1 ? 1 : o->rankStep;
    if (step == 0) return MF_FAIL(Z_INVALID_PARAM, "rank step is 0");
    const uint64_t last = (uint64_t)o->firstRank + (uint64_t)(o->groupSize - 1) * step;
    if (last >= bo.worldSize) return MF_FAIL(Z_INVALID_PARAM, "group %u:%lu:%u leaves the world of %u", o->firstRank, (unsigned long)last, step, bo.worldSize);
    if (bo.rankId < o->firstRank || (bo.rankId - o->firstRank) % step != 0 || (bo.rankId - o->firstRank) / step >= o->groupSize)
        return MF_FAIL(Z_INVALID_PARAM, "rank %u is not a member of group %u:%lu:%u", bo.rankId, o->firstRank, (unsigned long)last, step);
    const uint32_t groupRank = (bo.rankId - o->firstRank) / step;

    // slot index: the world takes 0; for others the first member draws a unique value and tells the rest
    int32_t slot = 0;
    const bool isWorld = o->firstRank == 0 && step == 1 && o->groupSize == bo.worldSize && strcmp(o->name, "zbal_world") == 0;
    if (!isWorld) {
        int32_t mine = -1;
        if (groupRank == 0) {
            int rc = smem_shm_atomic_alloc_value(shm, cap - 1, &mine);
            if (rc != 0 || mine < 0) return MF_FAIL(Z_NO_MEMORY, "all %u communicator slots are taken (%d)", cap, rc);
            mine += 1;  // slot 0 belongs to the world
        }
        if (o->groupSize > 1) {
            std::vector<int32_t> all(o->groupSize, -1);
            std::string key = std::string("zbal_comm/") + o->name;
            int rc = smem_shm_subgroup_allgather(shm, key.c_str(), o->groupSize, groupRank, reinterpret_cast<const char *>(&mine), sizeof(mine),
                                                 reinterpret_cast<char *>(all.data()), (uint32_t)(all.size() * sizeof(int32_t)));
            if (rc != 0) return MF_FAIL(Z_ERROR, "communicator '%s': members could not agree on a slot (%d): %s", o->name, rc, mf::LastError::Msg());
            slot = all[0];
        } else {
            slot = mine;
        }
        if (slot <= 0 || (uint32_t)slot >= cap) return MF_FAIL(Z_ERROR, "communicator '%s': bad slot %d", o->name, slot);
    }

    auto c = std::make_shared<Comm>();
    c->name = o->name;
    c->id = (uint32_t)slot;
    c->first = o->firstRank;
    c->step = step;
    c->size = o->groupSize;
    c->groupRank = groupRank;
    const uint64_t slotOff = (uint64_t)slot * slotBytes;
    c->team.heap_base = bo.baseGva + (uint64_t)o->firstRank * bo.symmetricSize + slotOff;
    c->team.stride = (uint64_t)step * bo.symmetricSize;
    // a multimem access reaches EVERY rank of the job, so only a communicator over all of them may use the alias
    c->team.mc_base = (o->groupSize == bo.worldSize && step == 1) ? (mcBase ? mcBase + slotOff : 0) : 0;
    c->team.rank = groupRank;
    c->team.world = o->groupSize;
    c->team.emu = 0;
    c->team.spin_limit = spin;
    c->stageBytes = mf::AlignDown((slotBytes - kSignalBytes) / kStageCount, 4096);
    for (int i = 0; i < 4; i++) c->stageOff[i] = kSignalBytes + (uint64_t)i * c->stageBytes;
    c->p2pOff = kSignalBytes + 4 * c->stageBytes;
    c->p2pBytes = mf::AlignDown(c->stageBytes / o->groupSize, 4096);
    const Launchers *L = GetLaunchers();
    int sms = (L != nullptr && L->smCount != nullptr) ? L->smCount() : 0;
    c->maxCtas = sms > 0 ? std::min(sms, 256) : 128;

    // a slot may have served an earlier communicator: its flags restart from zero, and every member must
    // have cleared before anybody signals
    auto *be = mf::hybm::CurrentBackend();
    if (be != nullptr && !isWorld) {
        be->BindThread();
        be->MemsetAsync(bo.localGva + slotOff, 0, kSignalBytes, nullptr);
        be->StreamSync(nullptr);
    }
    if (o->groupSize > 1 && !isWorld) {
        std::string key = std::string("zbal_comm_ready/") + o->name;
        int rc = smem_shm_subgroup_barrier(shm, key.c_str(), o->groupSize, groupRank);
        if (rc != 0) return MF_FAIL(Z_ERROR, "communicator '%s': barrier failed (%d)", o->name, rc);
    }
    {
        std::lock_guard<std::mutex> g(st.mu);
        st.comms[c->name] = c;
        if (isWorld) st.world = c;
    }
    *comm = c.get();
    return Z_OK;
}

int32_t zbal_comm_get_property(zbal_comm_t comm, zbal_comm_property_t *p)
{
    auto c = FindComm(comm);
    if (!c || p == nullptr) return Z_INVALID_PARAM;
    memset(p, 0, sizeof(*p));
    snprintf(p->name, sizeof(p->name), "%s", c->name.c_str());
    p->groupId = c->id;
    p->groupSize = c->size;
    p->groupRank = c->groupRank;
    p->firstRank = c->first;
    p->rankStep = c->step;
    p->signalGva = c->team.heap_base + (uint64_t)c->groupRank * c->team.stride;
    p->stageBytes = c->stageBytes;
    p->epoch = c->epoch;
    return Z_OK;
}

zbal_comm_t zbal_comm_get_global(void)
{
    std::lock_guard<std::mutex> g(S().mu);
    return S().world.get();
}

zbal_comm_t zbal_comm_get_by_name(const char *name)
{
    if (name == nullptr) return nullptr;
    std::lock_guard<std::mutex> g(S().mu);
    auto it = S().comms.find(name);
    return it == S().comms.end() ? nullptr : it->second.get();
}

int32_t zbal_comm_destroy(zbal_comm_t comm, uint32_t flags)
{
    (void)flags;
    auto c = FindComm(comm);
    if (!c) return Z_INVALID_PARAM;
    State &st = S();
    smem_shm_t shm;
    {
        std::lock_guard<std::mutex> g(st.mu);
        if (st.world == c) return MF_FAIL(Z_INVALID_PARAM, "the world communicator goes away with zbal_unbootstrap");
        st.comms.erase(c->name);
        shm = st.shm;
    }
    if (c->groupRank == 0 && c->id > 0) smem_shm_atomic_release_value(shm, (int32_t)c->id - 1);
    return Z_OK;
}

void zbal_comm_destroy_all(uint32_t flags)
{
    std::vector<zbal_comm_t> hs;
    {
        std::lock_guard<std::mutex> g(S().mu);
        for (auto &kv : S().comms)
            if (kv.second != S().world) hs.push_back(kv.second.get());
    }
    for (auto h : hs) zbal_comm_destroy(h, flags);
}

int32_t zbal_comm_get_device_status(zbal_comm_t comm, uint32_t status[4])
{
    auto c = FindComm(comm);
    if (!c || status == nullptr) return Z_INVALID_PARAM;
    auto *be = mf::hybm::CurrentBackend();
    if (be == nullptr) return Z_NOT_SUPPORTED;
    const uint64_t src = c->team.heap_base + (uint64_t)c->groupRank * c->team.stride;
    int rc = be->MemcpyAsync(reinterpret_cast<uint64_t>(status), src, 16, mf::hybm::CPY_D2H, nullptr);
    if (rc == 0) rc = be->StreamSync(nullptr);
    return rc == 0 ? Z_OK : Z_ERROR;
}

int32_t zbal_all_reduce_scaled(const void *send, void *recv, size_t count, zbal_datatype_t dt, zbal_datatype_t odt, zbal_reduce_op_t op,
                               float scale, zbal_comm_t comm, zbal_stream_t stream)
{
    auto c = FindComm(comm);
    if (!c) return Z_INVALID_PARAM;
    if (send == nullptr || count == 0) return Z_OK;
    if (recv == nullptr) return MF_FAIL(Z_INVALID_PARAM, "recv buffer is NULL");
    TypeInfo ti, to;
    const int kop = OpOf(op);
    if (!TypeOf(dt, ti) || !TypeOf(odt, to) || kop < 0) return MF_FAIL(Z_INVALID_PARAM, "bad data type or reduce op");
    if (ti.kdt < 0) return MF_FAIL(Z_NOT_SUPPORTED, "all_reduce supports bf16, fp16, fp32 and int32");
    if (!(odt == dt || (dt == ZBAL_DT_FP32 && odt == ZBAL_DT_BF16))) return MF_FAIL(Z_NOT_SUPPORTED, "the fused cast goes from fp32 to bf16 only");
    if (c->size == 1 && send == recv && scale == 1.f) return Z_OK;
    return AllReduce(*c, send, recv, count, ti.kdt, to.kdt, ti.size, to.size, kop, scale, stream);
}

int32_t zbal_all_reduce(const void *send, void *recv, void *buffer, size_t count, zbal_datatype_t dt, zbal_reduce_op_t op, zbal_comm_t comm,
                        zbal_stream_t stream)
{
    (void)buffer;
    return zbal_all_reduce_scaled(send, recv, count, dt, dt, op, 1.f, comm, stream);
}

int32_t zbal_reduce_scatter(const void *send, void *recv, size_t recv_count, zbal_datatype_t dt, zbal_reduce_op_t op, zbal_comm_t comm,
                            zbal_stream_t stream)
{
    auto c = FindComm(comm);
    if (!c) return Z_INVALID_PARAM;
    if (send == nullptr || recv_count == 0) return Z_OK;
    if (recv == nullptr) return MF_FAIL(Z_INVALID_PARAM, "recv buffer is NULL");
    TypeInfo ti;
    const int kop = OpOf(op);
    if (!TypeOf(dt, ti) || kop < 0) return MF_FAIL(Z_INVALID_PARAM, "bad data type or reduce op");
    if (ti.kdt < 0) return MF_FAIL(Z_NOT_SUPPORTED, "reduce_scatter supports bf16, fp16, fp32 and int32");
    const Launchers *L = GetLaunchers();
    if (L == nullptr) return Z_NOT_SUPPORTED;
    std::lock_guard<std::mutex> g(c->mu);
    const uint64_t m = recv_count;
    if (m * c->size * ti.size > DirectMin() && InSlice(send, m * c->size * ti.size)) {
        MfCollArgs a = BaseArgs(*c, send, recv, m * c->size, 1.f, kop, 0, 0);
        const bool mc = c->team.mc_base != 0 && InFirstSegment(send, m * c->size * ti.size);
        a.zero_copy = (mc && kop == 0 && ti.kdt != 3) ? 3 : 2;  // the switch adds when it can
        return Launched(L->coll(1, ti.kdt, ti.kdt, &a, c->Ctas(m * c->size * ti.size), 512, stream), "reduce_scatter (direct)");
    }
    uint64_t piece = c->stageBytes / ti.size / c->size;
    piece -= piece % 8;
    // pieces are column blocks of the [members, m] view of the input: rows stay m apart (part_stride)
    uint64_t done = 0;
    while (done < m) {
        const uint64_t cnt = std::min(piece, m - done);
        MfCollArgs a = BaseArgs(*c, static_cast<const char *>(send) + done * ti.size, static_cast<char *>(recv) + done * ti.size, cnt * c->size,
                                1.f, kop, 0, 0);
        a.part_stride = m;
        int rc = Launched(L->coll(1, ti.kdt, ti.kdt, &a, c->Ctas(cnt * c->size * ti.size), 512, stream), "reduce_scatter");
        if (rc != Z_OK) return rc;
        done += cnt;
    }
    return Z_OK;
}

int32_t zbal_all_gather(const void *send, void *recv, size_t send_count, zbal_datatype_t dt, zbal_comm_t comm, zbal_stream_t stream)
{
    auto c = FindComm(comm);
    if (!c) return Z_INVALID_PARAM;
    if (send == nullptr || send_count == 0) return Z_OK;
    if (recv == nullptr) return MF_FAIL(Z_INVALID_PARAM, "recv buffer is NULL");
    TypeInfo ti;
    if (!TypeOf(dt, ti)) return MF_FAIL(Z_INVALID_PARAM, "bad data type");
    return AllGatherBytes(*c, send, recv, (uint64_t)send_count * ti.size, stream);
}

int32_t zbal_all_to_all_v(const void *send, void *recv, const uint64_t *meta, uint64_t buffer_bytes, zbal_comm_t comm, zbal_stream_t stream)
{
    auto c = FindComm(comm);
    if (!c) return Z_INVALID_PARAM;
    if (send == nullptr) return Z_OK;
    if (recv == nullptr || meta == nullptr) return MF_FAIL(Z_INVALID_PARAM, "recv buffer or meta table is NULL");
    const Launchers *L = GetLaunchers();
    if (L == nullptr) return Z_NOT_SUPPORTED;
    std::lock_guard<std::mutex> g(c->mu);
    if (buffer_bytes + 4096 > c->stageBytes)
        return MF_FAIL(Z_NOT_SUPPORTED, "all_to_all_v: buffers of %lu bytes exceed the staging capacity of %lu", (unsigned long)buffer_bytes,
                       (unsigned long)(c->stageBytes - 4096));
    MfA2AArgs a{};
    a.team = c->team;
    a.in = reinterpret_cast<uint64_t>(send);
    a.out = reinterpret_cast<uint64_t>(recv);
    a.meta = reinterpret_cast<uint64_t>(meta);
    a.in_bytes = buffer_bytes;
    uint64_t b;
    a.epoch = c->Next(a.stage_a, b);
    return Launched(L->a2a(&a, c->Ctas(buffer_bytes), 512, stream), "all_to_all_v");
}

int32_t zbal_broadcast(void *buf, uint64_t count, zbal_datatype_t dt, uint16_t root, zbal_comm_t comm, zbal_stream_t stream)
{
    auto c = FindComm(comm);
    if (!c) return Z_INVALID_PARAM;
    if (buf == nullptr || count == 0) return Z_OK;
    TypeInfo ti;
    if (!TypeOf(dt, ti)) return MF_FAIL(Z_INVALID_PARAM, "bad data type");
    if (root >= c->size) return MF_FAIL(Z_INVALID_PARAM, "root %u is outside the group of %u", root, c->size);
    return BroadcastBytes(*c, buf, buf, count * ti.size, root, stream);
}

int32_t zbal_scatter(const void *send, void *recv, uint64_t count, zbal_datatype_t dt, uint16_t root, zbal_comm_t comm, zbal_stream_t stream)
{
    auto c = FindComm(comm);
    if (!c) return Z_INVALID_PARAM;
    if (recv == nullptr || count == 0) return Z_OK;
    TypeInfo ti;
    if (!TypeOf(dt, ti)) return MF_FAIL(Z_INVALID_PARAM, "bad data type");
    if (root >= c->size) return MF_FAIL(Z_INVALID_PARAM, "root %u is outside the group of %u", root, c->size);
    if (c->groupRank == root && send == nullptr) return MF_FAIL(Z_INVALID_PARAM, "the root's send buffer is NULL");
    const Launchers *L = GetLaunchers();
    if (L == nullptr) return Z_NOT_SUPPORTED;
    const uint64_t bytes = count * ti.size;
    int kdt;
    uint32_t unit;
    if (!UnitOf(bytes, reinterpret_cast<uint64_t>(send), reinterpret_cast<uint64_t>(recv), kdt, unit))
        return MF_FAIL(Z_NOT_SUPPORTED, "scatter: %lu bytes per member at odd addresses or of odd size", (unsigned long)bytes);
    std::lock_guard<std::mutex> g(c->mu);
    // the rooted-copy kernel in scatter mode: the root pushes part r (part_stride apart) to member r only
    const uint64_t total = bytes / unit;
    uint64_t piece = c->stageBytes / unit;
    piece -= piece % 8;
    uint64_t done = 0;
    while (done < total) {
        const uint64_t cnt = std::min(piece, total - done);
        const char *src = send != nullptr ? static_cast<const char *>(send) + done * unit : nullptr;
        MfCollArgs a = BaseArgs(*c, src, static_cast<char *>(recv) + done * unit, cnt, 1.f, 0, root, 1);
        a.part_stride = total;
        int rc = Launched(L->coll(3, kdt, kdt, &a, c->Ctas(cnt * unit), 512, stream), "scatter");
        if (rc != Z_OK) return rc;
        done += cnt;
    }
    return Z_OK;
}

int32_t zbal_gather(const void *send, void *recv, uint64_t count, zbal_datatype_t dt, uint16_t root, zbal_comm_t comm, zbal_stream_t stream)
{
    auto c = FindComm(comm);
    if (!c) return Z_INVALID_PARAM;
    if (send == nullptr || count == 0) return Z_OK;
    if (recv == nullptr) return MF_FAIL(Z_INVALID_PARAM, "gather needs a receive buffer of groupSize * count elements on every member");
    if (root >= c->size) return MF_FAIL(Z_INVALID_PARAM, "root %u is outside the group of %u", root, c->size);
    TypeInfo ti;
    if (!TypeOf(dt, ti)) return MF_FAIL(Z_INVALID_PARAM, "bad data type");
    return AllGatherBytes(*c, send, recv, count * ti.size, stream);
}

int32_t zbal_barrier(zbal_comm_t comm, zbal_stream_t stream)
{
    auto c = FindComm(comm);
    if (!c) return Z_INVALID_PARAM;
    const Launchers *L = GetLaunchers();
    if (L == nullptr) return Z_NOT_SUPPORTED;
    std::lock_guard<std::mutex> g(c->mu);
    uint64_t a, b;
    const uint32_t epoch = c->Next(a, b);
    return Launched(L->barrier(&c->team, 0, epoch, stream), "barrier");
}

int32_t zbal_send(const void *buf, size_t count, zbal_datatype_t dt, uint32_t peer, zbal_comm_t comm, zbal_stream_t stream)
{
    auto c = FindComm(comm);
    if (!c) return Z_INVALID_PARAM;
    if (buf == nullptr || count == 0) return Z_OK;
    TypeInfo ti;
    if (!TypeOf(dt, ti)) return MF_FAIL(Z_INVALID_PARAM, "bad data type");
    return P2P(*c, const_cast<void *>(buf), count * ti.size, peer, true, stream);
}

int32_t zbal_recv(void *buf, size_t count, zbal_datatype_t dt, uint32_t peer, zbal_comm_t comm, zbal_stream_t stream)
{
    auto c = FindComm(comm);
    if (!c) return Z_INVALID_PARAM;
    if (buf == nullptr || count == 0) return Z_OK;
    TypeInfo ti;
    if (!TypeOf(dt, ti)) return MF_FAIL(Z_INVALID_PARAM, "bad data type");
    return P2P(*c, buf, count * ti.size, peer, false, stream);
}

}  // extern "C"
