/*
 * zbal library-wide calls: version, logging, last error. Include this header to get the whole zbal C
 * surface (parity: app/zbal/src/include/zbal.h:28-60 of the reference).
 */
#ifndef MF_B200_ZBAL_H
#define MF_B200_ZBAL_H

#include "zbal_def.h"
#include "zbal_bootstrap.h"
#include "zbal_mem_allocator.h"
#include "zbal_operations.h"
#include "zbal_moe.h"

#ifdef __cplusplus
extern "C" {
#endif

const char *zbal_version(void);
/* func receives (level, message); NULL restores the default sink (stderr) */
int32_t zbal_set_logger(void (*func)(int, const char *));
/* 0 debug, 1 info, 2 warn, 3 error */
int32_t zbal_set_logger_level(int level);
/* Collective: adds one more segment (deviceMemorySize bytes per rank) to the symmetric heap. Every rank must call it at
 * the same point of its allocation sequence. With ZBAL_ALLOC_CONF=expandable_segments:True the allocator calls it by
 * itself when a request does not fit; since symmetric allocation already requires the same sequence of requests on
 * every rank, all ranks reach that point together. */
int32_t zbal_heap_expand(uint64_t *segmentBase, uint64_t *segmentBytes);
/* 1 when [ptr, ptr + bytes) lies inside this rank's part of the symmetric memory (any segment), else 0. */
int32_t zbal_is_symmetric(const void *ptr, uint64_t bytes);
const char *zbal_get_last_error_msg(void);
const char *zbal_get_and_clear_last_error_msg(void);

#ifdef __cplusplus
}
#endif
#endif
