/*
 * Direct (non-channel) operator calls, same two symbols as the reference's
 * include/host/op_export.h:3-5 (src/host/op_export.c:6-14): synchronous RMSNorm and fp16-weight
 * matmul on buffer handles, through the session's global handle.  0 on success, an HTP_AEE_* code
 * otherwise (unknown handle, region outside its buffer, arguments the operator rejects).
 */
#ifndef HTP_OPS_HOST_OP_EXPORT_H
#define HTP_OPS_HOST_OP_EXPORT_H

#ifdef __cplusplus
extern "C" {
#endif

int htp_ops_rpc_rms_norm_f32(int dst_fd, int dst_offset, int src_fd, int src_offset, int ne0, int ne1);
int htp_ops_rpc_mat_mul_permuted_w16a32(int output_fd, int output_offset, int activation_fd, int activation_offset,
                                        int weight_fd, int weight_offset, int m, int k, int n);

#ifdef __cplusplus
}
#endif

#endif /* HTP_OPS_HOST_OP_EXPORT_H */
