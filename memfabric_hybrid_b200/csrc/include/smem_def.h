/*
 * Types shared by the smem C API: the op table through which a caller plugs its own durable or
 * distributed key/value service (etcd, a registry, ...) under the config store.
 * ABI parity: src/smem/include/host/smem_def.h:22-96 of the reference.
 */
#ifndef MF_B200_SMEM_DEF_H
#define MF_B200_SMEM_DEF_H

#include <stdbool.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Return codes an op-table function may use. 0 is success. */
#define SMEM_STORE_BACKEND_CODE_OK       (0)
#define SMEM_STORE_BACKEND_CODE_BASE     (-3000)
#define SMEM_STORE_BACKEND_CODE_INTERNAL (SMEM_STORE_BACKEND_CODE_BASE)
#define SMEM_STORE_BACKEND_CODE_INVAL    (SMEM_STORE_BACKEND_CODE_BASE - 1)
#define SMEM_STORE_BACKEND_CODE_BUFEX    (SMEM_STORE_BACKEND_CODE_BASE - 2) /* caller buffer too small */
#define SMEM_STORE_BACKEND_CODE_PERM     (SMEM_STORE_BACKEND_CODE_BASE - 3)
#define SMEM_STORE_BACKEND_CODE_NORES    (SMEM_STORE_BACKEND_CODE_BASE - 4)
#define SMEM_STORE_BACKEND_CODE_NOENT    (SMEM_STORE_BACKEND_CODE_BASE - 5) /* key absent */
#define SMEM_STORE_BACKEND_CODE_LOCKED   (SMEM_STORE_BACKEND_CODE_BASE - 6) /* try_lock lost */
#define SMEM_STORE_BACKEND_CODE_UNLOCKED (SMEM_STORE_BACKEND_CODE_BASE - 7)

/* Cursor for a prefix scan: keys strictly after `marker`, in lexicographic order; `fill` is invoked per
 * match and stops the scan by returning false. */
typedef struct smem_store_prefix_get_ctx {
    const char *prefix;
    const char *marker;
    void *context;
    bool (*fill)(const char *key, const void *value, uint64_t size, void *context);
} smem_store_prefix_get_ctx_t;

typedef struct {
    bool (*distributed)(uint32_t flags);                                               /* true: shared by several nodes */
    int32_t (*create)(const char *name, const char *prefix, uint32_t flags, void **handle);
    void (*destroy)(void *handle);
    int32_t (*put)(void *handle, const char *key, const void *value, uint64_t size, uint32_t flags);
    int32_t (*get)(void *handle, const char *key, void *value, uint64_t capacity, uint32_t flags, uint64_t *size);
    int32_t (*prefix_get)(void *handle, const smem_store_prefix_get_ctx_t *ctx, uint32_t flags);
    int32_t (*remove)(void *handle, const char *key, uint32_t flags);
    int32_t (*lock)(void *handle, const char *name, uint32_t flags);                   /* may block */
    int32_t (*try_lock)(void *handle, const char *name, uint32_t flags);
    int32_t (*unlock)(void *handle, const char *name, uint32_t flags);
} smem_conf_store_backend_op_t;

#ifdef __cplusplus
}
#endif
#endif
