/* Internal interface between the sharding layer (shard.cu) and the host-buffer pipeline (host_pipeline.cu). */
#ifndef RPB_SHARD_INTERNAL_H
#define RPB_SHARD_INTERNAL_H

#include <cuda_runtime.h>
#include "rpb_common.h"

int rpb_shard_rank_of(const RpbShard* s);
int rpb_shard_world_of(const RpbShard* s);
int rpb_shard_device_of(const RpbShard* s);
/* NCCL broadcast of raw bytes on `stream` (no-op for a single rank) */
int rpb_shard_broadcast_bytes(RpbShard* s, void* buf, size_t bytes, int root, cudaStream_t stream);
/* partial dB GEMM on `stream` + its reduction over the ranks on the shard's side stream */
int rpb_shard_db_begin(RpbShard* s, void* dB, const void* A_rows, const void* dC_rows, long long rows, int k, int n,
                       int dtype, int flags, cudaStream_t stream);
/* which elements of dB are valid on this rank after rpb_shard_db_begin(..., flags, ...) */
void rpb_shard_db_slice(const RpbShard* s, int k, int n, int dtype, int flags, long long* begin, long long* end);
/* makes `stream` wait for the reduction started by rpb_shard_db_begin */
int rpb_shard_db_end(RpbShard* s, cudaStream_t stream);

#endif
