/*
 * dataflow_b200_exchange.h -- the one collective of the token-sharded step, from C.
 *
 * Every op on the path is independent per token except two sums over tokens: the cross-entropy loss sum and the RMSNorm weight
 * gradients. Ranks (one process per GPU) therefore exchange one small packed fp32 buffer per step,
 *     [ loss sum, valid rows | dW of norm 0 | dW of norm 1 | ... ]
 * with a single sum all-reduce over NCCL. The kernels write their fp32 results straight into their slots of that buffer --
 * submit_softmax_cross_entropy takes the two loss floats as its loss_sum argument, submit_rms_norm_bwd_w_sums a dW slot as its
 * column_sums -- so nothing is packed or unpacked around the collective, and after it every rank holds the global sums in place.
 *
 * The reference has no counterpart: its handle interface leaves the network section open
 * (src/dataflow_handle/include/dataflow_handle.h:120, "TODO: Network") and offers only submit_peer_transfer
 * (src/dataflow_handle/nvidia/src/cuda_dataflow_handle.c:639-651). These calls follow the handle's conventions instead: a handle
 * and a stream id in, 0 / -1 out, message on stderr, work enqueued on the handle's stream without synchronising.
 *
 * NCCL is resolved at run time (the copy already loaded into the process, e.g. by a framework, else libnccl.so.2 from the loader
 * path), so the library itself does not depend on it; a world of one needs no NCCL at all.
 */
#ifndef DATAFLOW_B200_EXCHANGE_H
#define DATAFLOW_B200_EXCHANGE_H

#include "dataflow_abi.h"

#ifdef __cplusplus
extern "C" {
#endif

#define DATAFLOW_EXCHANGE_ID_BYTES 128

typedef struct dataflow_exchange {
	Dataflow_Handle * handle;       /* the rank's handle: its device and streams are the exchange's */
	int world_size;
	int rank;
	void * comm;                    /* ncclComm_t, NULL in a world of one */
	void * nccl_lib;                /* dlopen handle of the NCCL library in use */
	void * fn[6];                   /* resolved NCCL entry points */
} Dataflow_Exchange;

/* Rank 0 makes the id (ncclGetUniqueId) and hands its 128 bytes to the other ranks by whatever channel the job has (a store, MPI, a
 * file); every rank then calls dataflow_exchange_init with the same bytes. */
int dataflow_exchange_unique_id(uint8_t id[DATAFLOW_EXCHANGE_ID_BYTES]);

/* Joins the communicator of `world_size` ranks on the handle's device (ncclCommInitRank: collective over the ranks, blocks until
 * all have called). world_size == 1 sets up a no-op exchange and ignores `id` (may be NULL). */
int dataflow_exchange_init(Dataflow_Exchange * exchange, Dataflow_Handle * handle, int world_size, int rank,
                           const uint8_t id[DATAFLOW_EXCHANGE_ID_BYTES]);

/* packed[0 .. count) <- sum over the ranks, in place, fp32, enqueued on stream `stream_id` of the handle (-1 = default stream).
 * Orders like any op of that stream: make the stream wait for the kernels that fill the buffer (submit_dependency) and the
 * consumers wait for the stream. Every rank must call it with the same count, once per step, in the same order. */
int dataflow_exchange_all_reduce_f32(Dataflow_Exchange * exchange, int stream_id, float * packed, uint64_t count);

/* Leaves the communicator (outstanding work on the handle's streams should have completed). */
void dataflow_exchange_destroy(Dataflow_Exchange * exchange);

#ifdef __cplusplus
}
#endif
#endif
