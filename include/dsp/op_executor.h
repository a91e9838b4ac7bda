/*
 * Operator dispatch.  Same symbol as the reference's include/dsp/op_executor.h:9
 * (src/dsp/op_executor.cc:52-204): decode the op index, resolve the three buffer handles, check
 * sizes and alignment, run the kernel, return its code.
 */
#ifndef HTP_OPS_DSP_OP_EXECUTOR_H
#define HTP_OPS_DSP_OP_EXECUTOR_H

#include "message.h"

#ifdef __cplusplus
extern "C" {
#endif

/*
 * Runs one request on the open session and waits for it.  Returns 0 on success and -1 for: no
 * open session, an unknown or unbuilt op index (the reference returns 0 there without doing
 * anything, op_executor.cc:200-203; reporting it is a documented deviation), an unknown buffer
 * handle, a region that does not fit its buffer, and every argument the kernel rejects
 * (src/dsp/ops/mat_mul.c:878-892).  A positive value is a kernel-side error code.
 */
int execute_op_simple(struct OpComputeRequest *req);

#ifdef __cplusplus
}
#endif

#endif /* HTP_OPS_DSP_OP_EXECUTOR_H */
