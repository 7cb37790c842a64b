/*
 * hybm ("hybrid big memory") layer types: the memory/data/transport engine under the smem API.
 * ABI parity: src/hybm/include/hybm_def.h:30-190 of the reference (enums, error codes, the 1280-byte
 * exchange blob, options, the 12 copy directions and the copy parameter blocks).
 * Data-operation bits on this platform: MTE = SM kernels doing peer load/store, SDMA = copy engines,
 * HOST_SHM = mapped host shared memory; RDMA/URMA/TCP bits are accepted and served by those paths.
 */
#ifndef MF_B200_HYBM_DEF_H
#define MF_B200_HYBM_DEF_H

#include <stdint.h>
#include <stdbool.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *hybm_entity_t;
typedef void *hybm_mem_slice_t;

#define HYBM_TLS_PATH_SIZE               256
#define HYBM_BIND_NUMA_FLAG_INDEX        0
#define HYBM_BIND_NUMA_FLAG_LEN          7
#define HYBM_PERFORMANCE_MODE_FLAG_INDEX 7
#define HYBM_PERFORMANCE_MODE_FLAG_LEN   1
#define HYBM_BIND_NUMA_AUTO_AFFINITY_FLAG ((1U << HYBM_BIND_NUMA_FLAG_LEN) - 1)
#define HYBM_FLAG_CREATE_WITH_SHM         (1U << 8)
#define HYBM_FLAG_DRAM_MAP_HOST_VA        (1U << 9)
#define HYBM_FLAG_INIT_SHMEM_META         (1ULL << 63)
#define HYBM_PRE_REG_SIZE_THRES           (8192U * 1024)

#define BM_OK                 (0)
#define BM_ERROR              (-1)
#define BM_INVALID_PARAM      (-2)
#define BM_MALLOC_FAILED      (-3)
#define BM_NEW_OBJECT_FAILED  (-4)
#define BM_FILE_NOT_ACCESS    (-5)
#define BM_DL_FUNCTION_FAILED (-6)
#define BM_TIMEOUT            (-7)
#define BM_UNDER_API_UNLOAD   (-8)
#define BM_NOT_INITIALIZED    (-9)
#define BM_NOT_SUPPORT_FUNC   (-10)
#define BM_NOT_SUPPORTED      (-100)
#define BM_NOT_CONNECTED      (-101)

typedef enum {
    HYBM_TYPE_AI_CORE_INITIATE = 0, /* copies issued from device kernels */
    HYBM_TYPE_HOST_INITIATE,        /* copies issued by host API calls */
    HYBM_TYPE_AICPU_INITIATE,
    HYBM_TYPE_BUTT
} hybm_type;

typedef enum {
    HYBM_DOP_TYPE_DEFAULT = 0U,
    HYBM_DOP_TYPE_MTE = 1U << 0,
    HYBM_DOP_TYPE_SDMA = 1U << 1,
    HYBM_DOP_TYPE_DEVICE_RDMA = 1U << 2,
    HYBM_DOP_TYPE_HOST_RDMA = 1U << 3,
    HYBM_DOP_TYPE_HOST_TCP = 1U << 4,
    HYBM_DOP_TYPE_HOST_URMA = 1U << 5,
    HYBM_DOP_TYPE_HOST_SHM = 1U << 6,
    HYBM_DOP_TYPE_AIV_SDMA = 1U << 7,
    HYBM_DOP_TYPE_DEVICE_URMA = 1U << 8,
    HYBM_DOP_TYPE_BUTT
} hybm_data_op_type;

typedef enum {
    HYBM_MEM_TYPE_DEVICE = 1U << 0,
    HYBM_MEM_TYPE_HOST = 1U << 1,
    HYBM_MEM_TYPE_BUTT
} hybm_mem_type;

typedef enum {
    HYBM_SCENE_DEFAULT = 1U << 0,
    HYBM_SCENE_TRANS = 1U << 1,
    HYBM_SCENE_SHM = 1U << 2,
    HYBM_SCENE_BUTT
} hybm_scene;

typedef enum {
    HYBM_ROLE_PEER = 0,
    HYBM_ROLE_SENDER,
    HYBM_ROLE_RECEIVER,
    HYBM_ROLE_BUTT
} hybm_role_type;

typedef struct {
    uint8_t desc[1280L];
    uint32_t descLen;
} hybm_exchange_info;

typedef struct {
    bool tlsEnable;
    char caPath[HYBM_TLS_PATH_SIZE];
    char crlPath[HYBM_TLS_PATH_SIZE];
    char certPath[HYBM_TLS_PATH_SIZE];
    char keyPath[HYBM_TLS_PATH_SIZE];
    char keyPassPath[HYBM_TLS_PATH_SIZE];
    char packagePath[HYBM_TLS_PATH_SIZE];
    char decrypterLibPath[HYBM_TLS_PATH_SIZE];
} hybm_tls_config;

typedef struct {
    hybm_type bmType;
    hybm_mem_type memType;           /* bit mask of the pools this entity owns */
    hybm_data_op_type bmDataOpType;  /* bit mask of permitted data operators */
    uint32_t rankCount;
    uint32_t rankId;
    uint16_t devId;
    uint64_t maxHBMSize;             /* per-rank HBM slot */
    uint64_t maxDRAMSize;            /* per-rank DRAM slot */
    uint64_t deviceVASpace;
    uint64_t hostVASpace;
    hybm_scene scene;
    bool enable56BitsGva;
    hybm_role_type role;
    uint32_t flags;
    char transUrl[64];
    char tag[32];
    char tagOpInfo[256];
    hybm_tls_config tlsOption;
    int dramShmFd;
} hybm_options;

typedef enum {
    HYBM_LOCAL_HOST_TO_GLOBAL_HOST = 0,
    HYBM_LOCAL_HOST_TO_GLOBAL_DEVICE = 1,
    HYBM_LOCAL_DEVICE_TO_GLOBAL_HOST = 2,
    HYBM_LOCAL_DEVICE_TO_GLOBAL_DEVICE = 3,
    HYBM_GLOBAL_HOST_TO_GLOBAL_HOST = 4,
    HYBM_GLOBAL_HOST_TO_GLOBAL_DEVICE = 5,
    HYBM_GLOBAL_HOST_TO_LOCAL_HOST = 6,
    HYBM_GLOBAL_HOST_TO_LOCAL_DEVICE = 7,
    HYBM_GLOBAL_DEVICE_TO_GLOBAL_HOST = 8,
    HYBM_GLOBAL_DEVICE_TO_GLOBAL_DEVICE = 9,
    HYBM_GLOBAL_DEVICE_TO_LOCAL_HOST = 10,
    HYBM_GLOBAL_DEVICE_TO_LOCAL_DEVICE = 11,
    HYBM_DATA_COPY_DIRECTION_AUTO = 12,
    HYBM_DATA_COPY_DIRECTION_BUTT
} hybm_data_copy_direction;

typedef struct {
    void *src;
    void *dest;
    uint64_t dataSize;
} hybm_copy_params;

typedef struct {
    void **sources;
    void **destinations;
    const uint64_t *dataSizes;
    uint32_t batchSize;
} hybm_batch_copy_params;

typedef struct {
    void **sources;
    void **destinations;
    const uint64_t *dataSizes;
    void **scale;
    void **offset;
    uint32_t batchSize;
    uint32_t unitNum;   /* elements per quantisation unit */
    void *stream;
    uint32_t inputType; /* 0 bf16, 1 fp16 */
    uint32_t flags;     /* HYBM_QUANT_FP8_E4M3: fp8 e4m3 with one factor per 128 elements (unitNum must be 128) instead of int8 */
} hybm_quant_copy_params;

#define HYBM_QUANT_FP8_E4M3 (1u << 0)

#ifdef __cplusplus
}
#endif
#endif
