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
const char *zbal_get_last_error_msg(void);
const char *zbal_get_and_clear_last_error_msg(void);

#ifdef __cplusplus
}
#endif
#endif
