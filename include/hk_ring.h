/* hk_ring.h -- the ring hop of the sequence-sharded attention, issued from native code.
 *
 * The reference (BlubridgeAI/HyperKernels) has no multi-GPU path; this is the transport under
 * hyperkernels_b200/ring.py.  One hop = ncclGroupStart / ncclSend / ncclRecv / ncclGroupEnd on a
 * communication stream, ordered against the compute stream with two events, so that the host does
 * nothing per hop but call one function.  Only local buffers are ever handed to NCCL or to a kernel:
 * no peer pointer reaches a tensor map.
 *
 * The library (libhk_ring.so) resolves NCCL at run time (dlopen of libnccl.so.2: in a PyTorch process
 * the copy torch already loaded), so it loads -- and every function returns an error code instead of
 * crashing -- on a machine without NCCL or without a GPU.
 *
 * Every function returns HK_RING_OK (0) or a negative code; hk_ring_error_string gives the text.
 */
#ifndef HK_RING_H
#define HK_RING_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

enum hk_ring_status {
    HK_RING_OK = 0,
    HK_RING_ERR_NO_NCCL = -1,   /* libnccl.so.2 could not be loaded */
    HK_RING_ERR_NCCL = -2,      /* an NCCL call failed; hk_ring_last_nccl_error() has NCCL's text */
    HK_RING_ERR_CUDA = -3,      /* a CUDA runtime call failed */
    HK_RING_ERR_ARG = -4,       /* null pointer, bad rank */
    HK_RING_ERR_TIMEOUT = -5,   /* hk_ring_wait: the hop did not complete in time */
    HK_RING_ERR_ASYNC = -6      /* ncclCommGetAsyncError reported a failure (a peer died, the network failed) */
};

#define HK_RING_UNIQUE_ID_BYTES 128

typedef struct hk_ring hk_ring_t;

/* rank 0 of the ring makes the id and hands it to the others (any out-of-band channel; ring.py broadcasts it) */
int hk_ring_get_unique_id(void* id /* HK_RING_UNIQUE_ID_BYTES */);

/* collective over the ring's ranks; the communicator lives on the calling thread's current device */
int hk_ring_create(hk_ring_t** ring, const void* id, int rank, int world);

#define HK_RING_SLOTS 4 /* hops that may be in flight at once (the backward keeps two) */

/* One hop: when everything enqueued on compute_stream so far is done, send `bytes` from `send` to rank
 * send_peer and receive as many into `recv` from rank recv_peer, on comm_stream.  Returns at once.
 * `slot` (0 .. HK_RING_SLOTS-1) names the hop for hk_ring_join / hk_ring_wait; a slot is reused only after
 * its previous hop has been joined or waited for. */
int hk_ring_exchange(hk_ring_t* ring, int slot, const void* send, int send_peer, void* recv, int recv_peer,
                     size_t bytes, void* compute_stream, void* comm_stream);

/* make compute_stream wait for the hop of `slot` (device-side ordering only, the host does not block) */
int hk_ring_join(hk_ring_t* ring, int slot, void* compute_stream);

/* host-side wait for the hop of `slot` with a limit: polls the hop's event and ncclCommGetAsyncError.
 * HK_RING_ERR_TIMEOUT / HK_RING_ERR_ASYNC leave the communicator aborted (ncclCommAbort): destroy it. */
int hk_ring_wait(hk_ring_t* ring, int slot, double timeout_s);

/* ncclCommGetAsyncError once: HK_RING_OK or HK_RING_ERR_ASYNC */
int hk_ring_poll(hk_ring_t* ring);

int hk_ring_destroy(hk_ring_t* ring);

/* like hk_ring_destroy, but with ncclCommAbort: for a ring whose peers may be gone (never blocks on them) */
int hk_ring_abort(hk_ring_t* ring);

const char* hk_ring_error_string(int status);
const char* hk_ring_last_nccl_error(void);

#ifdef __cplusplus
}
#endif
#endif /* HK_RING_H */
