/*
 * Buffer table: the replacement of the reference's rpcmem buffers.  There the host allocates
 * shared memory (rpcmem_alloc, rpcmem_to_fd, fastrpc_mmap: src/host/test.c:30-53), names it by
 * file descriptor in every request, and the DSP side turns fd into pointer through a cache
 * (src/dsp/mmap_mgr.cc:15-37).  Here the "fd" is a small integer handle of a cudaMalloc'd device
 * buffer (or of a pinned host buffer for the message channel, or of a shared buffer - pinned host
 * memory the device addresses, for results the host reads in place); device memory is not host
 * addressable, so upload/download are explicit.  None of these have a reference counterpart
 * beyond the lines cited.
 *
 * All functions need an open session and act on its device.  Handles are > 0.
 */
#ifndef HTP_OPS_HOST_BUFFERS_H
#define HTP_OPS_HOST_BUFFERS_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Device buffer of `size` bytes (256-byte aligned, zero-filled).  Handle, or -1. */
int htp_buf_alloc(size_t size);
/* Pinned host buffer (for the message channel; also usable as a staging area).  Handle, or -1. */
int htp_buf_alloc_host(size_t size);
/* Pinned host memory that the device addresses directly (mapped; the host pointer is the device
 * pointer): the closest thing to an rpcmem buffer - operators take it as output, activation or weight,
 * the host reads results through htp_buf_ptr once the message is done (or after
 * htp_session_synchronize) without a download.  Every device access crosses PCIe: meant for small
 * activations and outputs (a token's logits), not for weights.  htp_buf_upload / htp_buf_download on it
 * wait for the session stream first and then copy on the host.  Handle, or -1. */
int htp_buf_alloc_shared(size_t size);
/* Registers caller-owned device memory (for example a tensor of another framework) under a
 * handle; htp_buf_free forgets it without freeing the memory.  Handle, or -1. */
int htp_buf_wrap(void *device_ptr, size_t size);
/* Releases the handle (test.c:55-58).  0, or -1 for an unknown handle. */
int htp_buf_free(int fd);

/* Synchronous copies between caller memory and a buffer region.  0, or -1 (unknown handle,
 * region outside the buffer, copy failure). */
int htp_buf_upload(int fd, size_t offset, const void *src, size_t size);
int htp_buf_download(int fd, size_t offset, void *dst, size_t size);
/* The same copies, only ENQUEUED on the session stream: operators submitted afterwards (a message, a
 * direct call) see an upload's bytes, and a download sees the results of operators submitted before
 * it, but the call does not wait.  For pinned caller memory (pageable memory makes CUDA stage the
 * copy and wait anyway).  The caller leaves `src` unchanged, and does not read `dst`, until the
 * next completed message or htp_session_synchronize.  rpcmem needs no such calls: its bytes are
 * shared with the DSP (src/host/test.c:30-53). */
int htp_buf_upload_async(int fd, size_t offset, const void *src, size_t size);
int htp_buf_download_async(int fd, size_t offset, void *dst, size_t size);

/* Base address: device pointer of a device buffer, host pointer of a host buffer; NULL if unknown. */
void *htp_buf_ptr(int fd);
/* 1 for a host buffer, 2 for a shared (host memory, device-addressable) buffer, 0 for a device buffer,
 * -1 if unknown. */
int htp_buf_is_host(int fd);
size_t htp_buf_size(int fd);

/* The session's stream as a cudaStream_t, for callers that enqueue their own work in order with
 * the operators; NULL when no session is open. */
void *htp_session_stream(void);
/* Waits for everything enqueued on the session stream; returns like htp_b200_stream_status. */
int htp_session_synchronize(void);

#ifdef __cplusplus
}
#endif

#endif /* HTP_OPS_HOST_BUFFERS_H */
