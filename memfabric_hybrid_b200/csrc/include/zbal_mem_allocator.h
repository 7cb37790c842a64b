/*
 * SMA, the allocator that hands out device memory from the symmetric heap so that tensors allocated in
 * the same order on every rank sit at the same offset of every rank's slice. The zbal_pluggable_* pair
 * has the signature PyTorch's pluggable CUDA allocator expects
 * (parity: app/zbal/src/include/zbal_mem_allocator.h of the reference).
 */
#ifndef MF_B200_ZBAL_MEM_ALLOCATOR_H
#define MF_B200_ZBAL_MEM_ALLOCATOR_H

#include "zbal_def.h"

#ifdef __cplusplus
extern "C" {
#endif

int32_t zbal_sma_init(zbal_allocator_options_t *options, int32_t flags);
void zbal_sma_uninit(int32_t flags);

void zbal_pluggable_init(int32_t device_count);
void *zbal_pluggable_malloc(size_t size, int32_t device, zbal_stream_t stream);
void zbal_pluggable_free(void *ptr, size_t size, int32_t device, zbal_stream_t stream);
/* Returns every cached block to the heap. With check_error a block still in use is reported as an error. */
void zbal_pluggable_empty_cache(bool check_error);

/* Runs the allocator over a made-up address range with no device behind it (replay, tests). */
void zbal_simulate_init(int64_t addr, int64_t size);

typedef struct {
    uint64_t heapSize;
    uint64_t inUseBytes;       /* handed out to callers now */
    uint64_t cachedBytes;      /* free blocks kept per stream for reuse */
    uint64_t peakInUseBytes;
    uint64_t largestFreeBlock; /* in the heap, caches not counted */
    uint64_t mallocCalls;
    uint64_t freeCalls;
    uint64_t cacheHits;
    uint64_t heapCarves;       /* mallocs that had to go to the heap */
    uint64_t failedMallocs;
    uint64_t poolCount;        /* private pools that exist (capturing or kept alive by a CUDA graph) */
    uint64_t poolCachedBytes;  /* free blocks parked in private pools (not counted in cachedBytes) */
    uint64_t segments;         /* address ranges the heap spans (1 until it was expanded) */
    uint64_t segmentsAdded;    /* of those, added by the grow hook on exhaustion */
} zbal_sma_stats_t;

/* Expandable segments. zbal_sma_add_segment hands the allocator another address range; with
 * ZBAL_ALLOC_CONF=expandable_segments:True a request that the heap cannot serve calls the grow hook (set by
 * zbal_bootstrap to the collective zbal_heap_expand), which returns 0 after it added a segment, and is tried again. */
typedef int (*zbal_sma_grow_hook_t)(uint64_t need_bytes, void *ctx);
int32_t zbal_sma_add_segment(uint64_t base, uint64_t size);
void zbal_sma_set_grow_hook(zbal_sma_grow_hook_t hook, void *ctx);

/* Private pools for CUDA-graph capture. A graph replays with the addresses it saw while it was captured, so
 * what it allocated must never be handed to anyone else while the graph exists:
 *   begin   allocations on streams the filter accepts (NULL: every stream) are served from the pool's own blocks,
 *           else carved from the heap and tagged with the pool;
 *   end     stops routing (capture finished); the pool and its blocks stay;
 *   release the graphs that used the pool are gone: parked blocks return to the heap, blocks still in use
 *           become ordinary blocks.
 * A tagged block that is freed is parked in its pool (reused only by the same pool); zbal_pluggable_empty_cache
 * leaves pools alone. The pool id is PyTorch's MempoolId_t pair. */
typedef bool (*zbal_pool_filter_t)(void *ctx, zbal_stream_t stream);
int32_t zbal_sma_begin_pool(uint64_t pool_hi, uint64_t pool_lo, zbal_pool_filter_t filter, void *ctx);
int32_t zbal_sma_end_pool(uint64_t pool_hi, uint64_t pool_lo);
int32_t zbal_sma_release_pool(uint64_t pool_hi, uint64_t pool_lo);

int32_t zbal_sma_get_stats(zbal_sma_stats_t *stats);
void zbal_sma_reset_peak(void);
/* History of malloc/free events (bounded ring) for the offline replay tool. Recording is off by default. */
void zbal_sma_record_history(bool enable, uint32_t max_entries);
/* Writes a JSON snapshot {"heap":…, "blocks":[…], "history":[…]} into buf; returns the bytes needed (call
 * with buf == NULL to size the buffer). */
int64_t zbal_sma_snapshot(char *buf, int64_t cap);

#ifdef __cplusplus
}
#endif
#endif
