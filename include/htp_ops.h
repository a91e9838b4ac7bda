/*
 * The remote interface of the reference (include/htp_ops.idl:9-20, implemented in
 * src/dsp/commu.c:215-396) as ordinary C functions: same names and argument order as the stubs
 * the IDL compiler generates, nothing remote behind them.  Every function returns an AEEResult:
 * 0 on success, one of the HTP_AEE_* codes otherwise (callers should test for non-zero; the
 * numeric values are this library's own).
 */
#ifndef HTP_OPS_RPC_H
#define HTP_OPS_RPC_H

#include <stdint.h>

#include "host/session.h" /* remote_handle64 */

#ifdef __cplusplus
extern "C" {
#endif

typedef int AEEResult;

#define HTP_AEE_SUCCESS      0
#define HTP_AEE_EFAILED      1
#define HTP_AEE_EBADPARM     14
#define HTP_AEE_EALREADY     9
#define HTP_AEE_EUNSUPPORTED 20

/* commu.c:215-222.  `uri` selects the device like open_dsp_session's domain_id when it ends in a
 * number ("...&_dom=3" or "cuda:3"); NULL means device 0. */
AEEResult htp_ops_open(const char *uri, remote_handle64 *handle);
/* commu.c:225-234 */
AEEResult htp_ops_close(remote_handle64 handle);
/* commu.c:239-249 */
AEEResult htp_ops_init_backend(remote_handle64 handle);
/* commu.c:252-258: a second channel while one is active -> HTP_AEE_EALREADY */
AEEResult htp_ops_create_channel(remote_handle64 handle, int32_t fd, uint32_t size);
/* commu.c:261-263 */
AEEResult htp_ops_destroy_channel(remote_handle64 handle);
/* commu.c:266-317: RMSNorm of ne1 rows of ne0 floats, fd0/offset0 = dst, fd1/offset1 = src; runs and
 * completes before returning.  HTP_AEE_EFAILED when the session is not ready or the operator rejects
 * its arguments. */
AEEResult htp_ops_rms_norm_f32(remote_handle64 handle, int32_t fd0, int32_t offset0, int32_t fd1, int32_t offset1,
                               int32_t ne0, int32_t ne1);
/* commu.c:320-385: output (fd0) = activation (fd1, fp32 [m][k]) x fp16 weights in the reference's tile
 * order (fd2, as written by src/host/test.c:303-313); synchronous; HTP_AEE_EFAILED as above. */
AEEResult htp_ops_mat_mul_permuted_w16a32(remote_handle64 handle, int32_t fd0, int32_t offset0, int32_t fd1,
                                          int32_t offset1, int32_t fd2, int32_t offset2, int32_t m, int32_t k,
                                          int32_t n);
/* commu.c:390-396 ran Hexagon micro-benchmarks; here a no-op that returns success. */
AEEResult htp_ops_test_ops(remote_handle64 handle);

#ifdef __cplusplus
}
#endif

#endif /* HTP_OPS_RPC_H */
