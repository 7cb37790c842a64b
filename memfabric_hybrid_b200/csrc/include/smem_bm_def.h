/*
 * Big Memory (BM) pool types: memory kinds, data-operation bitmask, copy directions, configuration
 * and batch-copy parameter blocks.
 * ABI parity: src/smem/include/host/smem_bm_def.h:22-166 of the reference. On this platform
 * SMEMB_DATA_OP_SDMA selects the NVLink path (SM copy kernels + copy engines on mapped peer HBM);
 * the RDMA/URMA/TCP bits are accepted and served by the same intra-box paths.
 */
#ifndef MF_B200_SMEM_BM_DEF_H
#define MF_B200_SMEM_BM_DEF_H

#include <stdint.h>
#include <stddef.h>
#include <stdbool.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *smem_bm_t;
#define SMEM_BM_TIMEOUT_MAX UINT32_MAX
#define SMEM_TLS_PATH_SIZE  256

/* smem_bm_create flags: bits 0-6 NUMA node to bind the DRAM slice to (0x7f = follow the GPU's affinity),
 * bit 7 performance mode, bit 8 back the DRAM slice with a caller shm fd, bit 9 map DRAM at a host VA. */
#define SMEM_BM_BIND_NUMA_FLAG_INDEX         0
#define SMEM_BM_BIND_NUMA_FLAG_LEN           7
#define SMEM_BM_PERFORMANCE_MODE_FLAG_INDEX  7
#define SMEM_BM_PERFORMANCE_MODE_FLAG_LEN    1
#define SMEM_BM_BIND_NUMA_AUTO_AFFINITY_FLAG ((1U << SMEM_BM_BIND_NUMA_FLAG_LEN) - 1)
#define SMEM_BM_FLAG_CREATE_WITH_SHM         (1U << 8)
#define SMEM_BM_FLAG_DRAM_MAP_HOST_VA        (1U << 9)

typedef enum {
    SMEM_MEM_TYPE_LOCAL_DEVICE = 0, /* private device memory of the caller */
    SMEM_MEM_TYPE_LOCAL_HOST,       /* private host memory of the caller */
    SMEM_MEM_TYPE_DEVICE,           /* pooled HBM (GVA) */
    SMEM_MEM_TYPE_HOST,             /* pooled DRAM (GVA) */
    SMEM_MEM_TYPE_BUTT
} smem_bm_mem_type;
typedef smem_bm_mem_type smem_bm_mem_type_t;

typedef enum {
    SMEMB_DATA_OP_SDMA = 1U << 0,
    SMEMB_DATA_OP_HOST_RDMA = 1U << 1,
    SMEMB_DATA_OP_HOST_TCP = 1U << 2,
    SMEMB_DATA_OP_DEVICE_RDMA = 1U << 3,
    SMEMB_DATA_OP_HOST_URMA = 1U << 4,
    SMEMB_DATA_OP_HOST_SHM = 1U << 5,
    SMEMB_DATA_OP_DEVICE_URMA = 1U << 6,
    SMEMB_DATA_OP_BUTT
} smem_bm_data_op_type;
typedef smem_bm_data_op_type smem_bm_data_op_type_t;

typedef enum {
    SMEMB_COPY_L2G = 0,  /* local HBM        -> pooled HBM  */
    SMEMB_COPY_G2L = 1,  /* pooled HBM       -> local HBM   */
    SMEMB_COPY_G2H = 2,  /* pooled HBM       -> local host  */
    SMEMB_COPY_H2G = 3,  /* local host       -> pooled HBM  */
    SMEMB_COPY_L2GH = 4, /* local HBM        -> pooled DRAM */
    SMEMB_COPY_GH2L = 5, /* pooled DRAM      -> local HBM   */
    SMEMB_COPY_GH2H = 6, /* pooled DRAM      -> local host  */
    SMEMB_COPY_H2GH = 7, /* local host       -> pooled DRAM */
    SMEMB_COPY_G2G = 8,  /* pooled           -> pooled      */
    SMEMB_COPY_AUTO = 9, /* infer from the two addresses    */
    SMEMB_COPY_BUTT
} smem_bm_copy_type;
typedef smem_bm_copy_type smem_bm_copy_type_t;

typedef struct {
    bool tlsEnable;
    char caPath[SMEM_TLS_PATH_SIZE];
    char crlPath[SMEM_TLS_PATH_SIZE];
    char certPath[SMEM_TLS_PATH_SIZE];
    char keyPath[SMEM_TLS_PATH_SIZE];
    char keyPassPath[SMEM_TLS_PATH_SIZE];
    char packagePath[SMEM_TLS_PATH_SIZE];
    char decrypterLibPath[SMEM_TLS_PATH_SIZE];
} smem_tls_config;
typedef smem_tls_config smem_tls_config_t;

typedef struct {
    uint32_t initTimeout;             /* seconds, default 120 */
    uint32_t createTimeout;           /* seconds, default 120 */
    uint32_t controlOperationTimeout; /* seconds, default 120 */
    bool startConfigStoreServer;      /* default true: rank 0 (or the first racer) hosts the store */
    bool startConfigStoreOnly;
    bool dynamicWorldSize;
    bool unifiedAddressSpace;         /* must stay true */
    bool autoRanking;
    uint32_t rankId;                  /* used when autoRanking is false */
    uint32_t flags;
    char hcomUrl[64];
    smem_tls_config hcomTlsConfig;
    smem_tls_config storeTlsConfig;
} smem_bm_config_t;

typedef struct {
    uint64_t maxDramSize;   /* per-rank DRAM slot size of the GVA layout */
    uint64_t maxHbmSize;    /* per-rank HBM slot size of the GVA layout */
    uint64_t localDRAMSize; /* what this rank contributes now */
    uint64_t localHBMSize;
    smem_bm_data_op_type dataOpType;
    bool enable56BitsGva;
    uint32_t flags;
    char tag[32];
    char tagOpInfo[256];    /* "tagA:OPTYPE:tagB,..." routing between tagged members */
    int dramShmFd;
} smem_bm_create_option_t;

typedef struct {
    const void *src;
    void *dest;
    size_t dataSize;
    void *stream;
} smem_copy_params;
typedef smem_copy_params smem_copy_params_t;

typedef struct {
    void **sources;
    void **destinations;
    const uint64_t *dataSizes;
    uint32_t batchSize;
    void *stream;
} smem_batch_copy_params;
typedef smem_batch_copy_params smem_batch_copy_params_t;

typedef struct {
    int32_t *results;   /* one code per item */
    uint32_t batchSize;
} smem_batch_copy_result;
typedef smem_batch_copy_result smem_batch_copy_result_t;

typedef enum {
    SMEM_GROUP_EVENT_JOIN,
    SMEM_GROUP_EVENT_LEAVE,
    SMEM_MEMBER_EVENT_BUTT
} smem_bm_group_event_t;

typedef void (*smem_bm_group_event_cb)(smem_bm_t handle, uint32_t rankId, smem_bm_group_event_t event, void *context);

#ifdef __cplusplus
}
#endif
#endif
