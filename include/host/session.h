/*
 * Session API of the host shim.  Same five symbols as the reference's include/host/session.h:5-11
 * (implemented there in src/host/session.c:10-96 over FastRPC); here a session is a CUDA device
 * plus one stream and one servicer thread.
 */
#ifndef HTP_OPS_HOST_SESSION_H
#define HTP_OPS_HOST_SESSION_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* The reference takes this type from the Hexagon SDK's remote.h. */
typedef uint64_t remote_handle64;

/*
 * Opens the process-global session (reference session.c:14-84).  domain_id selects the CUDA
 * device: the environment variable HTP_OPS_CUDA_DEVICE wins when set; otherwise domain_id is used
 * as the device ordinal when such a device exists, else device 0 (the reference's callers pass
 * the cDSP domain id, 3).  unsigned_pd_enabled is accepted and ignored.  Returns 0, or -1 when no
 * CUDA device can be used - there is no CPU fallback.
 */
int open_dsp_session(int domain_id, int unsigned_pd_enabled);

/* Stops the message channel if one is active, frees library-owned buffers, closes the session
 * (reference session.c:86-88 -> commu.c:225-234). */
void close_dsp_session(void);

/* Handle of the open session, (remote_handle64) -1 when none (reference session.c:8-12). */
remote_handle64 get_global_handle(void);

/* Creates the stream and kernel scratch of the open session (reference session.c:90-92 ->
 * commu.c:239-249, which brought up power, VTCM and HMX instead). */
void init_htp_backend(void);

/*
 * Starts the servicer thread on the message buffer `fd` (a host buffer from
 * htp_buf_alloc_host) of max_msg_size bytes (reference session.c:94-96 -> commu.c:252-258,
 * 151-195).  The buffer is zeroed first.  Returns 0; non-zero when a channel is already active,
 * the handle is not a host buffer, or the size exceeds the buffer.
 */
int create_htp_message_channel(int fd, unsigned int max_msg_size);

#ifdef __cplusplus
}
#endif

#endif /* HTP_OPS_HOST_SESSION_H */
