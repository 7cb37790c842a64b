/*
 * zbal bootstrap: bring up the config store connection, create the job-wide symmetric object
 * (smem_init -> smem_shm_init -> smem_shm_create) and split this rank's slice into the communicator
 * area and the allocator heap (parity: app/zbal/src/include/zbal_bootstrap.h of the reference).
 */
#ifndef MF_B200_ZBAL_BOOTSTRAP_H
#define MF_B200_ZBAL_BOOTSTRAP_H

#include "zbal_def.h"

#ifdef __cplusplus
extern "C" {
#endif

int32_t zbal_bootstrap_options_init(zbal_bootstrap_options_t *options);
/* Collective over all ranks of the job. Also creates the world communicator ("zbal_world"). */
int32_t zbal_bootstrap(zbal_bootstrap_options_t *options, zbal_bootstrap_output_t *output);
int32_t zbal_unbootstrap(uint32_t flags);
/* 1 after a successful zbal_bootstrap, else 0 */
int32_t zbal_is_bootstrapped(void);
int32_t zbal_bootstrap_get_output(zbal_bootstrap_output_t *output);

#ifdef __cplusplus
}
#endif
#endif
