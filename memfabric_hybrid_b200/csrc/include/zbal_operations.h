/*
 * zbal communicators and the operations on them. Every operation is enqueued on the caller's CUDA
 * stream and returns at once; all cross-GPU traffic is issued by the kernel itself as loads/stores to
 * peer slices. All members of a communicator must issue the same sequence of operations.
 * A NULL send buffer makes a collective a successful no-op.
 * Parity: app/zbal/src/include/zbal_operations.h of the reference (whole file); differences are noted
 * at the declarations.
 */
#ifndef MF_B200_ZBAL_OPERATIONS_H
#define MF_B200_ZBAL_OPERATIONS_H

#include "zbal_def.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Collective over the members named by options (a strided set of world ranks). The communicator slot is
 * agreed through the config store, so members may create different communicators in different orders. */
int32_t zbal_comm_create(zbal_comm_options_t *options, zbal_comm_t *comm);
int32_t zbal_comm_get_property(zbal_comm_t comm, zbal_comm_property_t *property);
zbal_comm_t zbal_comm_get_global(void);
zbal_comm_t zbal_comm_get_by_name(const char *name);
int32_t zbal_comm_destroy(zbal_comm_t comm, uint32_t flags);
void zbal_comm_destroy_all(uint32_t flags);
/* Reads the device-side status words of this rank: code 0 = no wait of any kernel ever ran out. */
int32_t zbal_comm_get_device_status(zbal_comm_t comm, uint32_t status[4]);

/* recv = reduce(send over members). buffer is unused (the reduce-scatter landing area is the
 * communicator's own staging) and may be NULL. In place (send == recv) is allowed. */
int32_t zbal_all_reduce(const void *send_buff, void *recv_buff, void *buffer, size_t count, zbal_datatype_t data_type,
                        zbal_reduce_op_t op, zbal_comm_t comm, zbal_stream_t stream);
/* Extension: out = cast(scale * reduce(send)) in one pass; out_type is data_type or BF16 (from FP32). */
int32_t zbal_all_reduce_scaled(const void *send_buff, void *recv_buff, size_t count, zbal_datatype_t data_type,
                               zbal_datatype_t out_type, zbal_reduce_op_t op, float scale, zbal_comm_t comm, zbal_stream_t stream);
int32_t zbal_reduce_scatter(const void *sendBuff, void *recvBuff, size_t recv_count, zbal_datatype_t dataType, zbal_reduce_op_t op,
                            zbal_comm_t comm, zbal_stream_t stream);
int32_t zbal_all_gather(const void *sendBuff, void *recvBuff, size_t send_count, zbal_datatype_t dataType, zbal_comm_t comm,
                        zbal_stream_t stream);
/* meta: DEVICE array [groupSize][4] of uint64 {send offset, send bytes, recv offset, recv bytes} for each
 * peer; buffer_bytes: size of the larger of the two buffers (the pieces land in the receiver's staging area, which must
 * hold the whole receive buffer). (The reference passes cumulative sums and counts in three device arrays; here one
 * table carries the same information.) */
int32_t zbal_all_to_all_v(const void *sendBuff, void *recvBuff, const uint64_t *meta, uint64_t buffer_bytes, zbal_comm_t comm,
                          zbal_stream_t stream);
int32_t zbal_broadcast(void *buf, uint64_t data_count, zbal_datatype_t dataType, uint16_t root, zbal_comm_t comm, zbal_stream_t stream);
/* root's sendBuff holds groupSize * data_count elements; every member receives its data_count elements */
int32_t zbal_scatter(const void *sendBuff, void *recvBuff, uint64_t data_count, zbal_datatype_t dataType, uint16_t root,
                     zbal_comm_t comm, zbal_stream_t stream);
/* every member contributes data_count elements; recvBuff (groupSize * data_count) is filled on every
 * member (only the root's copy is specified by the interface) */
int32_t zbal_gather(const void *sendBuff, void *recvBuff, uint64_t data_count, zbal_datatype_t dataType, uint16_t root,
                    zbal_comm_t comm, zbal_stream_t stream);
int32_t zbal_barrier(zbal_comm_t comm, zbal_stream_t stream);
/* peer is a rank of the communicator. A send pairs with the peer's recv of the same byte count. */
int32_t zbal_send(const void *sendBuff, size_t sendCount, zbal_datatype_t dataType, uint32_t peer, zbal_comm_t comm, zbal_stream_t stream);
int32_t zbal_recv(void *recvBuff, size_t recvCount, zbal_datatype_t dataType, uint32_t peer, zbal_comm_t comm, zbal_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif
