/*
 * Process-level entry points of the memory fabric: library init, config-store creation, logging,
 * TLS knobs and the per-thread last error.
 * ABI parity: src/smem/include/host/smem.h:24-182 of the reference.
 */
#ifndef MF_B200_SMEM_H
#define MF_B200_SMEM_H

#include <stddef.h>
#include <stdint.h>
#include <stdbool.h>
#include "smem_def.h"

#ifdef __cplusplus
extern "C" {
#endif

/* copy flags */
#define ASYNC_COPY_FLAG                  (1UL << (0)) /* return after enqueue; smem_bm_wait completes it */
#define COPY_EXTEND_FLAG                 (1UL << (1)) /* force the SM copy kernel instead of the copy engine */
#define SMEM_BM_FLAG_USE_EXTERNAL_STREAM (1UL << (2)) /* params.stream is a caller CUDA stream */
#define SMEM_WORLD_SIZE_MAX              1024U
#define SMEM_INVALID_DEV_ID              (-1)

/* smem_create_config_store flags */
#define SMEM_STORE_SKIP_RECOVER          (1UL << (0))

#define SMEM_OK              (0)
#define SMEM_ERROR           (-1)
#define SMEM_INVALID_PARAM   (-2000)
#define SMEM_MALLOC_FAILED   (-2001)
#define SMEM_NO_RESOURCES    (-2002)
#define SMEM_NOT_STARTED     (-2003)
#define SMEM_TIMEOUT         (-2004)
#define SMEM_REPEAT_INVOKE   (-2005)
#define SMEM_DUPLICATED      (-2006)
#define SMEM_NOT_EXIST       (-2007)
#define SMEM_NOT_INIT        (-2008)
#define SMEM_RES_IN_USE      (-2009)
#define SMEM_PARTIAL_FAILED  (-2012)
#define SMEM_NOT_CONNECTED   (-2014)

int32_t smem_init(uint32_t flags);
/* storeUrl: tcp://ip:port | etcd://ip:port[#instance] | reg://name[#instance]. Starts a store server. */
int32_t smem_create_config_store(const char *storeUrl, uint64_t flags);
void smem_destroy_config_store(const char *storeUrl);
int32_t smem_config_store_set_backend_op(const smem_conf_store_backend_op_t *backendOp);
int32_t smem_set_extern_logger(void (*func)(int level, const char *msg));
int32_t smem_set_extern_alarm(void (*alarm)(uint16_t code, const char *msg), void (*resume)(uint16_t code));
int32_t smem_set_log_level(int level); /* 0 debug, 1 info, 2 warn, 3 error, 4 off */
int32_t smem_set_conf_store_tls(bool enable, const char *tls_info, const uint32_t tls_info_len);
#ifdef __cplusplus
typedef int (*smem_decrypt_handler)(const char *cipherText, size_t cipherTextLen, char *plainText,
                                    size_t &plainTextLen);
#else
typedef int (*smem_decrypt_handler)(const char *cipherText, size_t cipherTextLen, char *plainText,
                                    size_t *plainTextLen);
#endif
int32_t smem_set_config_store_tls_key(const char *tls_pk, const uint32_t tls_pk_len, const char *tls_pk_pw,
                                      const uint32_t tls_pk_pw_len, const smem_decrypt_handler h);
void smem_uninit(void);
const char *smem_get_last_err_msg(void);
int32_t smem_get_last_err_code(void);
const char *smem_get_and_clear_last_err_msg(void);

#ifdef __cplusplus
}
#endif
#endif
