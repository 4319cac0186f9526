// Layout of the peer-exchange memory behind dalib200_allreduce and the cross-rank
// reductions of generated kernels.  Plain C declarations only: this text is compiled
// by g++ (comm.cc), by nvcc (peer_exchange.cu) and, spliced in front of the device
// prelude, by NVRTC for every generated kernel.
//
// Every rank (one GPU each, all on one NVLink / NVSwitch box) owns one block of
// DALI_PEER_BYTES in its own HBM that every other rank can address (CUDA IPC mapping
// between processes).  A collective is "one shot": each rank stores its contribution
// into slot [parity][its rank] of EVERY rank's block with plain stores over NVLink,
// then raises that slot's flag to the call's epoch with a release store at system
// scope; each rank then waits (bounded) until all flags of its own block show the
// epoch, and folds the slots of its own block in rank order -- the same order on every
// rank, so the result is bit-identical everywhere.  No reads cross NVLink, nothing is
// multicast, and no library kernel is handed a peer pointer.
//
// Epochs count collectives per region and live in device memory (a replayed CUDA graph
// advances them like an eager launch).  Slots are double-buffered by epoch parity: a
// rank can only be one collective ahead of the slowest rank, because finishing call k
// needs every rank's contribution to call k.
#ifndef DALI_B200_CSRC_PEER_H
#define DALI_B200_CSRC_PEER_H

#define DALI_PEER_MAX_WORLD 8                      /* the GPUs of one box */
#define DALI_PEER_SLOT_BYTES (256 * 1024)           /* payload per rank per collective (standalone kernels) */
#define DALI_PEER_CHUNK_BYTES 4096                  /* one CTA of 256 threads x 16 bytes; one flag per chunk */
#define DALI_PEER_CHUNKS (DALI_PEER_SLOT_BYTES / DALI_PEER_CHUNK_BYTES)
#define DALI_PEER_FUSED_SLOT_BYTES 256              /* 16 reductions x 16 bytes (generated all-axis kernels) */

/* byte offsets inside a rank's block */
#define DALI_PEER_OFF_DATA 0ull
#define DALI_PEER_OFF_FLAGS (DALI_PEER_OFF_DATA + 2ull * DALI_PEER_MAX_WORLD * DALI_PEER_SLOT_BYTES)
#define DALI_PEER_OFF_FUSED_DATA (DALI_PEER_OFF_FLAGS + 2ull * DALI_PEER_MAX_WORLD * DALI_PEER_CHUNKS * 8ull)
#define DALI_PEER_OFF_FUSED_FLAGS (DALI_PEER_OFF_FUSED_DATA + 2ull * DALI_PEER_MAX_WORLD * DALI_PEER_FUSED_SLOT_BYTES)
#define DALI_PEER_BYTES (DALI_PEER_OFF_FUSED_FLAGS + 2ull * DALI_PEER_MAX_WORLD * 8ull)

/* What a kernel needs to take part; lives in the rank's own device memory. */
struct DaliPeerTable {
    int world;
    int rank;
    unsigned long long wait_ns;                     /* a wait that lasts longer gives up and raises *error */
    unsigned long long* epoch;                      /* local: [0] standalone collectives, [1] generated kernels */
    int* error;                                     /* local, sticky: 0 ok, 1 a wait expired */
    unsigned int* ticket;                           /* local, wraps to 0: last CTA of a standalone kernel advances the epoch */
    char* block[DALI_PEER_MAX_WORLD];               /* rank r's block as addressed from this GPU */
};

#endif
