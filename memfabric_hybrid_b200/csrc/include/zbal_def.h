/*
 * zbal: collectives, MoE exchange and a symmetric allocator on top of one smem_shm object per job.
 * Types shared by the zbal C entry points. Enum values are part of the ABI that Python and torch layers
 * rely on (parity: app/zbal/src/include/zbal_def.h:31-155 of the reference). Streams are CUDA streams.
 */
#ifndef MF_B200_ZBAL_DEF_H
#define MF_B200_ZBAL_DEF_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *zbal_comm_t;
typedef void *zbal_stream_t; /* cudaStream_t */

typedef enum {
    ZBAL_DT_INT8 = 0,
    ZBAL_DT_INT16 = 1,
    ZBAL_DT_INT32 = 2,
    ZBAL_DT_INT64 = 3,
    ZBAL_DT_UINT64 = 4,
    ZBAL_DT_FP64 = 5,
    ZBAL_DT_FP16 = 6,
    ZBAL_DT_FP32 = 7,
    ZBAL_DT_BF16 = 8,
    ZBAL_DT_UINT8 = 9,
    ZBAL_DT_UINT16 = 10,
    ZBAL_DT_UINT32 = 11,
    ZBAL_DT_BUTT
} zbal_datatype_t;

typedef enum { ZBAL_REDUCE_PROD = 0, ZBAL_REDUCE_SUM = 1, ZBAL_REDUCE_MAX = 2, ZBAL_REDUCE_MIN = 3, ZBAL_REDUCE_BUTT } zbal_reduce_op_t;

/* How a communicator moves data. On B200 every value selects SM load/store kernels over NVLink peer
 * mappings; the enum is kept so that option structs written for the reference still parse. */
typedef enum { ZBAL_DATA_OP_MTE = 0, ZBAL_DATA_OP_AIV_SDMA = 1, ZBAL_DATA_OP_AICPU_SDMA = 2, ZBAL_DATA_OP_BUTT } zbal_data_op_type_t;

typedef enum { ZBAL_BT_MEMFABRIC = 0, ZBAL_BT_BUTT } zbal_bootstrap_type_t;

typedef enum { ZBAL_NO_QUANT = 0, ZBAL_QUANT_BF16_TO_INT8 = 1, ZBAL_QUANT_BF16_TO_FP8_1X128 = 2, ZBAL_QUANT_BUTT } zbal_quant_mode_t;

/* result codes of every zbal_* call */
typedef enum {
    Z_OK = 0,
    Z_ERROR = -1,
    Z_INVALID_PARAM = -2,
    Z_NOT_INITIALIZED = -3,
    Z_ALREADY_INITIALIZED = -4,
    Z_NO_MEMORY = -5,
    Z_NOT_SUPPORTED = -6,
    Z_TIMEOUT = -7,
    Z_NOT_FOUND = -8,
    Z_LAUNCH_FAILED = -9,
    Z_DUPLICATED = -10
} zbal_result_t;

#define ZBAL_IP_PORT_MAX        128
#define ZBAL_COMM_NAME_MAX      128
#define ZBAL_GROUP_CAP_MAX      256u
#define ZBAL_GROUP_CAP_DEFAULT  16u
#define ZBAL_TENSOR_MAX_DIM     12

typedef struct {
    uint32_t flags;
    zbal_bootstrap_type_t btType;
    char ipPort[ZBAL_IP_PORT_MAX]; /* config store, "tcp://ip:port" or "ip:port" */
    uint32_t worldSize;
    uint32_t rankId;
    int32_t deviceId;
    bool startConfigServer;        /* default: rank 0 hosts the store */
    uint64_t deviceMemorySize;     /* bytes of this rank's symmetric slice */
    zbal_data_op_type_t dataOperationType;
    uint64_t commMetaSpaceSize;    /* bytes per communicator: 1 MiB of signals + 4 staging buffers; 0 = derive from the slice */
    uint32_t commGroupCap;         /* communicators that can exist at once (1..256), default 16 */
} zbal_bootstrap_options_t;

/* Where things ended up. [localGva, +commAreaSize) holds the communicator slots, the rest is the
 * allocator heap; rank r's slice starts at baseGva + r * symmetricSize on every rank. */
typedef struct {
    uint64_t baseGva;
    uint64_t localGva;
    uint64_t symmetricSize;
    uint64_t commAreaSize;
    uint64_t heapGva;
    uint64_t heapSize;
    uint32_t worldSize;
    uint32_t rankId;
} zbal_bootstrap_output_t;

typedef struct {
    uint64_t baseAddress;     /* start of the heap (device address) */
    uint64_t size;
    uint64_t smallThreshold;  /* requests below it are carved from the low end, others from the high end; 0 = 1 MiB */
    int32_t deviceId;
    uint32_t flags;
} zbal_allocator_options_t;

/* A communicator over world ranks first, first+step, ..., first+(size-1)*step. */
typedef struct {
    char name[ZBAL_COMM_NAME_MAX];
    uint32_t firstRank;
    uint32_t rankStep;
    uint32_t groupSize;
    uint32_t flags;
} zbal_comm_options_t;

typedef struct {
    char name[ZBAL_COMM_NAME_MAX];
    uint32_t groupId;
    uint32_t groupSize;
    uint32_t groupRank;
    uint32_t firstRank;
    uint32_t rankStep;
    uint64_t signalGva;    /* this rank's signal area of the communicator */
    uint64_t stageBytes;   /* bytes of each of its 4 staging buffers */
    uint64_t epoch;        /* collectives issued so far */
} zbal_comm_property_t;

typedef struct {
    void *data;
    zbal_datatype_t dtype;
    uint32_t dim;
    int64_t shape[ZBAL_TENSOR_MAX_DIM];
} zbal_tensor_info_t;

#ifdef __cplusplus
}
#endif
#endif
