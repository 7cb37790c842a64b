// Core types of the memory layer: options, copy directions, the opaque 1280-byte exchange blob and
// its writer/reader, slices, and the process-wide VA manager (reserved GVA windows, address
// classification, direction lookup table).
// Parity: src/hybm/include/hybm_def.h:105-162, src/hybm/csrc/mm/hybm_ex_info_transfer.h:1-187,
// src/hybm/csrc/mm/hybm_mem_slice.h, src/hybm/csrc/mm/hybm_va_manager.{h,cpp}:24-36,140-168,221-339,506-549.
#pragma once
#include <map>
#include <shared_mutex>

#include "../include/hybm_def.h"
#include "../util/mf_util.h"

namespace mf {
namespace hybm {

constexpr uint64_t kGiB = 1ULL << 30;
constexpr uint64_t kTiB = 1ULL << 40;
constexpr uint64_t kHbmGranule = 2ULL << 20;

// GVA windows. Every process derives the same addresses from (space, entity id, attempt), so no
// negotiation is needed unless a reservation collides with something already mapped; then all
// ranks move to the next attempt together. Each space is 32 TiB cut into 128 windows of 256 GiB; a
// pool larger than one window runs into the following ids' windows (the overlap check refuses a real
// collision), so very large pools should use ids spaced accordingly. The spaces stay clear of where
// Linux puts PIE executables and the heap (0x55..-0x56..) and of the top-down mmap area (0x7f..).
//   pooled DRAM  : 0x1000_0000_0000 .. 0x3000_0000_0000   (host mmap, MAP_FIXED_NOREPLACE)
//   pooled HBM   : 0x3000_0000_0000 .. 0x5000_0000_0000   (cuMemAddressReserve with a fixed address)
//   trans imports: 0x6000_0000_0000 .. 0x7000_0000_0000   (peer-registered buffers mapped on demand)
constexpr uint64_t kDramWindowBase = 0x100000000000ULL;
constexpr uint64_t kHbmWindowBase = 0x300000000000ULL;
constexpr uint64_t kTransWindowBase = 0x600000000000ULL;
constexpr uint64_t kTransWindowEnd = 0x700000000000ULL;
constexpr uint64_t kWindowStride = 256 * kGiB;
constexpr uint32_t kMaxEntityId = 127;  // 0-63 Big Memory pools, 64-127 symmetric (SHM) heaps
constexpr uint32_t kShmEntityBase = 64;
constexpr uint32_t kReserveAttempts = 4;
uint64_t WindowBase(hybm_mem_type t, uint32_t entityId, uint32_t attempt);
// 56-bit global addresses (enable56BitsGva) for pooled DRAM whose window (slot x ranks) does not fit the 32 TiB DRAM space
// above, e.g. 1 024 ranks x 1 TiB. The addresses a caller sees then are NUMBERS in [2^55, 2^56), 32 windows of 1 PiB
// (the lower 16 for pooled DRAM, the upper 16 for pooled HBM):
// they name (rank, offset) and are only ever passed to the copy calls. Inside the process every rank's slice is mapped
// in a compact window of the ordinary DRAM space whose slot is as large as 16 TiB / ranks allows (a power of two); the
// copy paths and gva_to_va translate. A rank's slices together may not exceed the compact slot.
constexpr uint64_t kGva56Base = 1ULL << 55;
constexpr uint64_t kGva56WindowStride = 1ULL << 50;
constexpr uint32_t kGva56Windows = 32;
constexpr uint64_t kCompactThreshold = 16 * kTiB;   // larger windows than this go compact when 56-bit addresses are enabled
uint64_t Gva56WindowBase(hybm_mem_type t, uint32_t entityId, uint32_t attempt);
uint64_t CompactSlot(uint32_t ranks);               // bytes per rank of the compact window

// Address classes (bit mask): local host / pooled host / local device / pooled device.
enum AddrClass : uint8_t { AC_NONE = 0, AC_LH = 1, AC_GH = 2, AC_LD = 4, AC_GD = 8 };

struct ReservedRange {
    uint64_t base = 0;
    uint64_t slot = 0;    // bytes per rank
    uint32_t ranks = 0;
    hybm_mem_type type = HYBM_MEM_TYPE_DEVICE;
    uint32_t entityId = 0;
    uint32_t localRank = 0;
    uint64_t localBase = 0;  // != 0: a window of 56-bit addresses; rank r's slot is mapped at localBase + r * localSlot here
    uint64_t localSlot = 0;
    uint64_t End() const { return base + slot * ranks; }
};

class VaManager {
public:
    static VaManager &Get();
    int AddReserved(const ReservedRange &r);  // rejects overlap
    void RemoveReserved(uint64_t base);
    // O(#entities): which window holds va, and which rank's slot.
    bool Locate(uint64_t va, ReservedRange &out, uint32_t &rank) const;
    // User-registered local device/host ranges (outside any window).
    void AddLocal(uint64_t va, uint64_t size, bool device);
    void RemoveLocal(uint64_t va);
    // Class of [va, va+len). Unknown addresses are AC_NONE (the caller's copy type decides).
    uint8_t Classify(uint64_t va, uint64_t len) const;
    // Direction from classes; HYBM_DATA_COPY_DIRECTION_BUTT when the pair is not a valid copy.
    static hybm_data_copy_direction DirectionOf(uint8_t srcClass, uint8_t dstClass);
    static bool DirectionMatches(hybm_data_copy_direction d, uint8_t srcClass, uint8_t dstClass);
    std::string Dump() const;

private:
    mutable std::shared_mutex mu_;
    std::map<uint64_t, ReservedRange> reserved_;
    struct Local {
        uint64_t size;
        bool device;
    };
    std::map<uint64_t, Local> locals_;
};

// ---- exchange blob ---------------------------------------------------------------------------
constexpr uint32_t kExMagic = 0x4D464232u;  // "MFB2"
constexpr uint16_t kExVersion = 1;
enum ExKind : uint16_t { EX_ENTITY = 1, EX_SLICE = 2 };

class ExWriter {
public:
    explicit ExWriter(hybm_exchange_info *out) : out_(out) { out_->descLen = 0; }
    template <typename T> bool Put(const T &v) { return PutBytes(&v, sizeof(T)); }
    bool PutStr(const std::string &s)
    {
        uint16_t n = (uint16_t)s.size();
        return Put(n) && PutBytes(s.data(), n);
    }
    bool PutBytes(const void *p, size_t n)
    {
        if (out_->descLen + n > sizeof(out_->desc)) return false;
        memcpy(out_->desc + out_->descLen, p, n);
        out_->descLen += (uint32_t)n;
        return true;
    }

private:
    hybm_exchange_info *out_;
};

class ExReader {
public:
    explicit ExReader(const hybm_exchange_info *in) : in_(in) {}
    template <typename T> bool Take(T &v) { return TakeBytes(&v, sizeof(T)); }
    bool TakeStr(std::string &s)
    {
        uint16_t n = 0;
        if (!Take(n) || off_ + n > in_->descLen) return false;
        s.assign(reinterpret_cast<const char *>(in_->desc + off_), n);
        off_ += n;
        return true;
    }
    bool TakeBytes(void *p, size_t n)
    {
        if (in_->descLen > sizeof(in_->desc) || off_ + n > in_->descLen) return false;
        memcpy(p, in_->desc + off_, n);
        off_ += (uint32_t)n;
        return true;
    }

private:
    const hybm_exchange_info *in_;
    uint32_t off_ = 0;
};

struct ExHeader {
    uint32_t magic = kExMagic;
    uint16_t version = kExVersion;
    uint16_t kind = 0;
    uint32_t rank = 0;
    uint32_t entityId = 0;
};

// ---- slices ------------------------------------------------------------------------------------
enum SliceOrigin : uint8_t { SL_POOL = 0, SL_USER = 1 };

struct MemSlice {
    uint32_t magic = 0x534C4943u;  // checked when an opaque handle comes back from the caller
    uint32_t index = 0;
    hybm_mem_type memType = HYBM_MEM_TYPE_DEVICE;
    SliceOrigin origin = SL_POOL;
    uint64_t gva = 0;   // address inside the GVA window (pool) or the registered address (user)
    uint64_t size = 0;
    uint64_t offset = 0;  // offset inside this rank's slot
    bool Valid() const { return magic == 0x534C4943u; }
};

const char *ErrorString(int32_t code);

}  // namespace hybm
}  // namespace mf
