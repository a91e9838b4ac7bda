/*
 * Batched-request container exchanged over the message channel.
 *
 * Wire-compatible restatement of the reference's include/message.h (:6-58): same struct
 * and helper names, same packed sizes (MessageState 8, MessageHeader 16, RequestHeader 8,
 * RpcmemMapRequest 8, OpComputeRequest 4), same RequestType values.
 *
 * Protocol (reference src/host/test.c:182-204, src/dsp/commu.c:46-133): the host zeroes
 * state.d, writes n_reqs, req_offsets[0..n_reqs] (byte offsets from the start of the message;
 * the last entry is the total size) and the requests, then sets state.v[0] = 1. The servicer
 * executes every request in order, stores each return code in RequestHeader.state and then
 * sets state.v[1] = 1. One request on the wire is RequestHeader || body, unpadded, so request
 * bodies are only 4-byte aligned: read them through these packed structs or memcpy.
 */
#ifndef HTP_OPS_MESSAGE_H
#define HTP_OPS_MESSAGE_H

#include <stddef.h>
#include <stdint.h>

#define HTP_MSG_PACKED __attribute__((packed))

struct MessageState {
  union {
    volatile uint8_t  v[8]; /* v[0]: host "go"; v[1]: servicer "done" */
    volatile uint64_t d;
  };
} HTP_MSG_PACKED;

struct MessageHeader {
  struct MessageState state;
  uint32_t            checksum; /* carried, never verified (reference commu.c:78) */
  int32_t             n_reqs;
  int32_t             req_offsets[0]; /* n_reqs + 1 entries */
} HTP_MSG_PACKED;

struct RequestHeader {
  int32_t state; /* out: return code of this request */
  int32_t type;  /* enum RequestType */
  uint8_t data[0];
} HTP_MSG_PACKED;

enum RequestType {
  REQUEST_TYPE_NO_OP      = 0,
  REQUEST_TYPE_RPCMEM_MAP = 1,
  REQUEST_TYPE_OP_COMPUTE = 2,
  REQUEST_TYPE_COUNT,
};

struct RpcmemMapRequest {
  int32_t n_puts; /* handles whose cached mapping is dropped */
  int32_t n_gets; /* ignored, as in the reference (commu.c:104-108) */
  int32_t fds[0];
} HTP_MSG_PACKED;

struct OpComputeRequest {
  uint32_t op; /* enum HtpOpsIndex */
  uint8_t  payload[0];
} HTP_MSG_PACKED;

static inline size_t message_header_size(const struct MessageHeader *h) {
  return sizeof(struct MessageHeader) + ((size_t) h->n_reqs + 1) * sizeof(int32_t);
}

static inline size_t message_total_size(const struct MessageHeader *h) {
  return (size_t) h->req_offsets[h->n_reqs];
}

static inline size_t message_header_get_request_size(const struct MessageHeader *h, int req_idx) {
  return (size_t) (h->req_offsets[req_idx + 1] - h->req_offsets[req_idx]);
}

static inline struct RequestHeader *message_header_get_request_ptr(struct MessageHeader *h, int req_idx) {
  return (struct RequestHeader *) ((uintptr_t) h + (uintptr_t) h->req_offsets[req_idx]);
}

#if defined(__cplusplus)
static_assert(sizeof(struct MessageState) == 8, "wire size");
static_assert(sizeof(struct MessageHeader) == 16, "wire size");
static_assert(sizeof(struct RequestHeader) == 8, "wire size");
static_assert(sizeof(struct RpcmemMapRequest) == 8, "wire size");
static_assert(sizeof(struct OpComputeRequest) == 4, "wire size");
#else
_Static_assert(sizeof(struct MessageState) == 8, "wire size");
_Static_assert(sizeof(struct MessageHeader) == 16, "wire size");
_Static_assert(sizeof(struct RequestHeader) == 8, "wire size");
_Static_assert(sizeof(struct RpcmemMapRequest) == 8, "wire size");
_Static_assert(sizeof(struct OpComputeRequest) == 4, "wire size");
#endif

#endif /* HTP_OPS_MESSAGE_H */
