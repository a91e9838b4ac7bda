// Host layer: session, buffer table, operator dispatch and the message-channel servicer.
//
// Mirrors, over CUDA, what the reference spreads across src/host/session.c (session),
// src/dsp/mmap_mgr.cc (handle -> pointer table), src/dsp/op_executor.cc (dispatch) and
// src/dsp/commu.c (channel servicer and the remote-interface functions).  One process-global
// session, one stream, one servicer thread; like the reference, the library is not re-entrant.
#include <cuda_runtime.h>

#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iterator>
#include <map>
#include <mutex>
#include <thread>
#include <unordered_map>
#include <vector>

#include "device_ctx.h"
#include "dsp/op_executor.h"
#include "host/buffers.h"
#include "host/op_export.h"
#include "host/session.h"
#include "htp_ops.h"
#include "htp_ops_b200.h"
#include "message.h"
#include "op_reg.h"

namespace {

enum BufKind { kDeviceBuf = 0, kHostBuf = 1, kWrappedBuf = 2, kSharedBuf = 3 };  // shared: pinned host memory the device addresses

struct Buffer {
  uint8_t *ptr  = nullptr;
  size_t   size = 0;
  int      kind = kDeviceBuf;
};

// Set of disjoint address intervals (merged on insertion); used to detect operators that touch
// memory an earlier, still pending operator writes or reads.
class IntervalSet {
 public:
  bool overlaps(uintptr_t lo, uintptr_t hi) const {
    if (lo >= hi || m_.empty()) {
      return false;
    }
    auto it = m_.lower_bound(hi);  // first interval starting at or after hi
    if (it == m_.begin()) {
      return false;
    }
    --it;
    return it->second > lo;  // intervals are disjoint: the last one starting below hi decides
  }
  void add(uintptr_t lo, uintptr_t hi) {
    if (lo >= hi) {
      return;
    }
    auto it = m_.lower_bound(lo);
    if (it != m_.begin()) {
      auto prev = std::prev(it);
      if (prev->second >= lo) {
        it = prev;
      }
    }
    while (it != m_.end() && it->first <= hi) {
      lo = it->first < lo ? it->first : lo;
      hi = it->second > hi ? it->second : hi;
      it = m_.erase(it);
    }
    m_[lo] = hi;
  }
  void clear() { m_.clear(); }
  bool empty() const { return m_.empty(); }

 private:
  std::map<uintptr_t, uintptr_t> m_;
};

// Decode-sized operators of one kind that do not depend on each other, collected while a message
// is being read and issued as ONE persistent launch.
struct PendingBatch {
  std::vector<htp::MatMulDesc> ops;
  std::vector<RequestHeader *> owners;  // where to report a launch failure
  int                          m = 0, weight_type = 0, act_type = 0;
  IntervalSet                  writes, reads;
  bool                         weights_hazard = false;  // a weight overlaps an earlier pending output
  void clear() {
    ops.clear();
    owners.clear();
    writes.clear();
    reads.clear();
    weights_hazard = false;
  }
};

struct Session {
  std::mutex                      mu;  // buffer table and session fields
  bool                            open    = false;
  bool                            backend = false;
  int                             device  = -1;
  cudaStream_t                    stream  = nullptr;
  std::unordered_map<int, Buffer> bufs;
  int                             next_fd = 16;
  // regions written by operators enqueued since the stream was last waited for; a weight buffer
  // that overlaps one of them must not be prefetched ahead of stream order
  IntervalSet  pending_out;
  PendingBatch batch;
  // Operator state (the pending batch, pending_out, the stream's error word) is touched by the
  // channel servicer AND by callers of execute_op_simple / the RPC-named functions; whoever
  // enqueues or waits holds this lock - the servicer for a whole message, a direct call for itself.
  std::mutex   op_mu;
  // message channel
  std::thread       servicer;
  std::atomic<bool> stop{ false };
  uint8_t          *msg        = nullptr;
  size_t            max_msg    = 0;
  int               chan_fd    = -1;
};

Session g;
int     dummy_handle_target;

remote_handle64 session_handle() {
  return (remote_handle64) (uintptr_t) &dummy_handle_target;
}

bool set_session_device() {
  return g.open && cudaSetDevice(g.device) == cudaSuccess;
}

bool lookup(int fd, Buffer *out) {
  std::lock_guard<std::mutex> lk(g.mu);
  auto                        it = g.bufs.find(fd);
  if (it == g.bufs.end()) {
    return false;
  }
  *out = it->second;
  return true;
}

int register_buffer(const Buffer &b) {
  std::lock_guard<std::mutex> lk(g.mu);
  const int                   fd = g.next_fd++;
  g.bufs[fd]                     = b;
  return fd;
}

// handle + offset + size -> device address; nullptr when the handle is unknown, is a host
// buffer, or the region does not fit (the reference resolves an unknown fd to NULL and lets the
// operator's null check fail, op_executor.cc:57-61).
uint8_t *resolve(const RpcmemBufAddr &a, size_t bytes) {
  Buffer b;
  if (!lookup(a.fd, &b) || b.kind == kHostBuf || a.offset < 0) {
    return nullptr;
  }
  const size_t off = (size_t) a.offset;
  if (off > b.size || bytes > b.size - off) {
    return nullptr;
  }
  return b.ptr + off;
}

constexpr int kFlushOps = 64;  // operators collected before a batch is issued without waiting for more

// Issues the collected batch (if any).  Returns 0 or the launch error.
int flush_batch() {
  PendingBatch &b = g.batch;
  if (b.ops.empty()) {
    return 0;
  }
  int rc;
  if (b.ops.size() == 1) {
    const htp::MatMulDesc &d = b.ops[0];
    rc = htp::mul_mat_checked(d.y, d.x, d.w, b.m, d.k, d.n, b.weight_type, b.act_type, g.stream, !b.weights_hazard);
  } else {
    rc = htp::mul_mat_batch_checked(b.ops.data(), (int) b.ops.size(), b.m, b.weight_type, b.act_type, g.stream,
                                    !b.weights_hazard);
  }
  if (rc != 0) {
    for (RequestHeader *rh : b.owners) {
      if (rh) {
        rh->state = rc;
      }
    }
  }
  b.clear();
  return rc;
}

// Enqueue one operator on the session stream.  Returns the synchronous part of the result
// (argument validation); launch and kernel-side errors surface later (flush / stream wait).
// `owner` is the request to blame if the batch the operator joins fails to launch.
int enqueue_op(const OpComputeRequest *req, RequestHeader *owner) {
  if (!g.open || !g.backend) {
    return -1;
  }
  uint32_t op;
  memcpy(&op, &req->op, sizeof(op));
  if (op == HTP_OPS_RMS_NORM_F32) {
    // op_executor.cc:81-93: one size for both buffers, ne0 * ne1 floats
    RmsNormF32Params rp;
    memcpy(&rp, req->payload, sizeof(rp));
    if (rp.ne0 <= 0 || rp.ne1 <= 0) {
      return -1;
    }
    const size_t bytes = (size_t) rp.ne0 * (size_t) rp.ne1 * sizeof(float);
    uint8_t     *dst   = resolve(rp.dst, bytes);
    uint8_t     *src   = resolve(rp.src, bytes);
    if (!dst || !src) {
      return -1;
    }
    if (!g.batch.ops.empty()) {
      flush_batch();  // stream order then covers every dependence on the pending mat-vecs
    }
    const int rc = htp_b200_rms_norm_f32(reinterpret_cast<float *>(dst), reinterpret_cast<const float *>(src), rp.ne0,
                                         rp.ne1, g.stream);
    if (rc == 0) {
      g.pending_out.add((uintptr_t) dst, (uintptr_t) dst + bytes);
    }
    return rc;
  }
  int weight_type, act_type;
  switch (op) {
    case HTP_OPS_MAT_MUL_PERMUTED_W16A32: weight_type = HTP_B200_WT_F16_TILED, act_type = HTP_B200_ACT_F32; break;
    case HTP_OPS_MAT_MUL_PERMUTED_W4D16A32: weight_type = 2, act_type = HTP_B200_ACT_F32; break;
    case HTP_OPS_MAT_MUL_PERMUTED_W8D16A32: weight_type = 8, act_type = HTP_B200_ACT_F32; break;
    case HTP_OPS_MAT_MUL_PERMUTED_W4D16A32_IQ4_NL: weight_type = 20, act_type = HTP_B200_ACT_F32; break;
    case HTP_OPS_MAT_MUL_W4D16A16: weight_type = 2, act_type = HTP_B200_ACT_F16; break;
    case HTP_OPS_MAT_MUL_W8D16A16: weight_type = 8, act_type = HTP_B200_ACT_F16; break;
    default: return -1;  // unknown, or not built in this library
  }
  if (htp::g_opt_permuted_weights && op >= HTP_OPS_MAT_MUL_PERMUTED_W4D16A32 &&
      op <= HTP_OPS_MAT_MUL_PERMUTED_W4D16A32_IQ4_NL) {
    weight_type |= HTP_B200_WT_PERMUTED;  // the reference's own buffers for these op numbers
  }
  MatMulParams p;
  memcpy(&p, req->payload, sizeof(p));
  if (p.m <= 0 || p.k <= 0 || p.n <= 0 || p.k % 32 != 0 || p.n % 32 != 0) {
    return -1;
  }
  // sizes as in op_executor.cc:124-126, in 64 bits
  const size_t out_bytes = (size_t) p.m * (size_t) p.n * sizeof(float);
  const size_t act_bytes = (size_t) p.m * (size_t) p.k * (act_type == HTP_B200_ACT_F16 ? 2 : 4);
  const size_t w_bytes   = htp_b200_weight_bytes(weight_type, p.k, p.n);
  uint8_t     *out = resolve(p.output, out_bytes);
  uint8_t     *act = resolve(p.activation, act_bytes);
  uint8_t     *w   = resolve(p.weight, w_bytes);
  if (!out || !act || !w || (((uintptr_t) out | (uintptr_t) act | (uintptr_t) w) & 127u)) {
    return -1;
  }
  const uintptr_t o0 = (uintptr_t) out, a0 = (uintptr_t) act, w0 = (uintptr_t) w;
  PendingBatch   &b  = g.batch;
  const bool batchable = htp::mul_mat_batchable(p.m, p.k, p.n, weight_type, act_type);
  if (!b.ops.empty()) {
    const bool same_kind = batchable && b.m == p.m && b.weight_type == weight_type && b.act_type == act_type;
    const bool hazard    = b.writes.overlaps(a0, a0 + act_bytes) || b.writes.overlaps(w0, w0 + w_bytes) ||
                        b.writes.overlaps(o0, o0 + out_bytes) || b.reads.overlaps(o0, o0 + out_bytes);
    if (!same_kind || hazard) {
      flush_batch();  // a failure is reported in the owners' request states
    }
  }
  const bool weights_hazard = g.pending_out.overlaps(w0, w0 + w_bytes);
  if (!batchable) {
    const int rc = htp::mul_mat_checked(out, act, w, p.m, p.k, p.n, weight_type, act_type, g.stream, !weights_hazard);
    if (rc == 0) {
      g.pending_out.add(o0, o0 + out_bytes);
    }
    return rc;
  }
  if (b.ops.empty()) {
    b.m = p.m, b.weight_type = weight_type, b.act_type = act_type;
  }
  b.ops.push_back(htp::MatMulDesc{ reinterpret_cast<float *>(out), act, w, p.k, p.n });
  b.owners.push_back(owner);
  b.writes.add(o0, o0 + out_bytes);
  b.reads.add(a0, a0 + act_bytes);
  b.reads.add(w0, w0 + w_bytes);
  b.weights_hazard = b.weights_hazard || weights_hazard;
  g.pending_out.add(o0, o0 + out_bytes);
  // A long message (a decoder's 224 requests) is issued in pieces: the GPU starts on the first
  // kFlushOps operators while the host is still reading the rest (about half a microsecond per
  // request), instead of idling until the whole message has been parsed.
  if ((int) b.ops.size() >= kFlushOps) {
    flush_batch();  // a launch failure lands in the owners' request states
  }
  return 0;
}

int wait_stream() {
  const int frc = flush_batch();
  const int rc  = htp_b200_stream_status(g.stream);
  g.pending_out.clear();
  return rc != 0 ? rc : frc;
}

// ---------------------------------------------------------------- message channel servicer

inline uint64_t load_acquire64(volatile uint64_t *p) {
  return __atomic_load_n((uint64_t *) p, __ATOMIC_ACQUIRE);
}
inline void store_release64(volatile uint64_t *p, uint64_t v) {
  __atomic_store_n((uint64_t *) p, v, __ATOMIC_RELEASE);
}

// Checks that the request table of a published message stays inside the buffer.
bool message_is_sane(const MessageHeader *h, size_t max_msg) {
  if (h->n_reqs < 0) {
    return false;
  }
  const size_t hdr = sizeof(MessageHeader) + ((size_t) h->n_reqs + 1) * sizeof(int32_t);
  if (hdr > max_msg) {
    return false;
  }
  int32_t prev = (int32_t) hdr;
  if (h->n_reqs > 0 && h->req_offsets[0] < prev) {
    return false;
  }
  for (int i = 0; i <= h->n_reqs; ++i) {
    const int32_t o = h->req_offsets[i];
    if (o < prev || (size_t) o > max_msg) {
      return false;
    }
    prev = o;
  }
  return true;
}

void servicer_loop() {
  cudaSetDevice(g.device);
  MessageHeader *hdr   = reinterpret_cast<MessageHeader *>(g.msg);
  unsigned       idle  = 0;
  while (!g.stop.load(std::memory_order_acquire)) {
    const uint64_t d  = load_acquire64(&hdr->state.d);
    const uint8_t  v0 = d & 0xff, v1 = (d >> 8) & 0xff;
    if (v0 == 0 || v1 != 0) {
      // nothing published, or the last message has not been taken back yet
      if (++idle < 4096) {
        __builtin_ia32_pause();
      } else if (idle < 65536) {
        std::this_thread::yield();
      } else {
        std::this_thread::sleep_for(std::chrono::microseconds(50));
      }
      continue;
    }
    idle = 0;
    std::vector<int>            enqueued;
    std::unique_lock<std::mutex> op_lock(g.op_mu);
    if (message_is_sane(hdr, g.max_msg)) {
      for (int i = 0; i < hdr->n_reqs; ++i) {
        RequestHeader *rh    = message_header_get_request_ptr(hdr, i);
        const size_t   rsize = message_header_get_request_size(hdr, i);
        if (rsize < sizeof(RequestHeader)) {
          continue;
        }
        switch (rh->type) {
          case REQUEST_TYPE_OP_COMPUTE: {
            // the payload must hold the parameter block of the op it names
            size_t need = sizeof(RequestHeader) + sizeof(OpComputeRequest);
            if (rsize >= need) {
              uint32_t op;
              memcpy(&op, reinterpret_cast<const uint8_t *>(rh) + sizeof(RequestHeader), sizeof(op));
              need += op == HTP_OPS_RMS_NORM_F32 ? sizeof(RmsNormF32Params) : sizeof(MatMulParams);
            }
            if (rsize < need) {
              rh->state = -1;
              break;
            }
            rh->state = enqueue_op(reinterpret_cast<OpComputeRequest *>(rh->data), rh);
            if (rh->state == 0) {
              enqueued.push_back(i);
            }
          } break;
          case REQUEST_TYPE_RPCMEM_MAP: {
            // The reference drops its cached mapping of n_puts handles (commu.c:102-110);
            // there is no mapping cache here, the handles stay valid until freed.
            rh->state = 0;
          } break;
          default: break;
        }
      }
    }
    // (a message whose offset table leaves the buffer is not executed: the host sees "done"
    // with untouched request states)
    // all requests of a message complete before "done" is published (commu.c:91-126)
    const int rc = wait_stream();
    if (rc != 0) {
      for (int i : enqueued) {
        message_header_get_request_ptr(hdr, i)->state = rc;
      }
    }
    op_lock.unlock();
    store_release64(&hdr->state.d, (uint64_t) v0 | (1ull << 8));
  }
}

void stop_channel() {
  if (g.msg == nullptr) {
    return;
  }
  g.stop.store(true, std::memory_order_release);
  if (g.servicer.joinable()) {
    g.servicer.join();
  }
  g.stop.store(false, std::memory_order_release);
  g.msg     = nullptr;
  g.max_msg = 0;
  g.chan_fd = -1;
}

int pick_device(int domain_id) {
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) {
    cudaGetLastError();
    return -1;
  }
  if (const char *env = getenv("HTP_OPS_CUDA_DEVICE")) {
    const int d = atoi(env);
    return (d >= 0 && d < count) ? d : -1;
  }
  return (domain_id >= 0 && domain_id < count) ? domain_id : 0;
}

}  // namespace

extern "C" {

// ---------------------------------------------------------------- session

int open_dsp_session(int domain_id, int unsigned_pd_enabled) {
  (void) unsigned_pd_enabled;
  if (g.open) {
    return 0;
  }
  const int dev = pick_device(domain_id);
  if (dev < 0) {
    fprintf(stderr, "htp-ops-b200: no usable CUDA device (there is no CPU fallback)\n");
    return -1;
  }
  if (cudaSetDevice(dev) != cudaSuccess || cudaFree(0) != cudaSuccess) {
    cudaGetLastError();
    fprintf(stderr, "htp-ops-b200: cannot initialise CUDA device %d\n", dev);
    return -1;
  }
  g.device  = dev;
  g.open    = true;
  g.backend = false;
  return 0;
}

void close_dsp_session(void) {
  if (!g.open) {
    return;
  }
  stop_channel();
  cudaSetDevice(g.device);
  if (g.stream) {
    cudaStreamSynchronize(g.stream);
  }
  {
    std::lock_guard<std::mutex> lk(g.mu);
    for (auto &kv : g.bufs) {
      if (kv.second.kind == kDeviceBuf) {
        cudaFree(kv.second.ptr);
      } else if (kv.second.kind == kHostBuf || kv.second.kind == kSharedBuf) {
        cudaFreeHost(kv.second.ptr);
      }
    }
    g.bufs.clear();
  }
  g.pending_out.clear();
  g.batch.clear();
  htp::release_all_scratch();
  if (g.stream) {
    cudaStreamDestroy(g.stream);
    g.stream = nullptr;
  }
  g.open    = false;
  g.backend = false;
  g.device  = -1;
}

remote_handle64 get_global_handle(void) {
  return g.open ? session_handle() : (remote_handle64) -1;
}

void init_htp_backend(void) {
  if (!set_session_device() || g.backend) {
    return;
  }
  if (cudaStreamCreateWithFlags(&g.stream, cudaStreamNonBlocking) != cudaSuccess) {
    cudaGetLastError();
    g.stream = nullptr;
    return;
  }
  htp::DeviceCtx *ctx = htp::current_device_ctx();
  if (!ctx || !htp::stream_scratch(ctx, g.stream)) {
    return;
  }
  g.backend = true;
}

int create_htp_message_channel(int fd, unsigned int max_msg_size) {
  if (!g.open || !g.backend) {
    return HTP_AEE_EFAILED;
  }
  if (g.msg != nullptr) {
    return HTP_AEE_EALREADY;
  }
  Buffer b;
  if (!lookup(fd, &b) || b.kind != kHostBuf || max_msg_size < sizeof(MessageHeader) + sizeof(int32_t) ||
      max_msg_size > b.size) {
    return HTP_AEE_EBADPARM;
  }
  memset(b.ptr, 0, max_msg_size);
  g.msg     = b.ptr;
  g.max_msg = max_msg_size;
  g.chan_fd = fd;
  g.stop.store(false);
  g.servicer = std::thread(servicer_loop);
  return 0;
}

// ---------------------------------------------------------------- remote-interface names

AEEResult htp_ops_open(const char *uri, remote_handle64 *handle) {
  int dom = 0;
  if (uri) {
    const char *e = uri + strlen(uri);
    while (e > uri && e[-1] >= '0' && e[-1] <= '9') {
      --e;
    }
    if (*e) {
      dom = atoi(e);
    }
  }
  if (open_dsp_session(dom, 1) != 0) {
    return HTP_AEE_EFAILED;
  }
  if (handle) {
    *handle = session_handle();
  }
  return HTP_AEE_SUCCESS;
}

AEEResult htp_ops_close(remote_handle64 handle) {
  (void) handle;
  close_dsp_session();
  return HTP_AEE_SUCCESS;
}

AEEResult htp_ops_init_backend(remote_handle64 handle) {
  (void) handle;
  init_htp_backend();
  return g.backend ? HTP_AEE_SUCCESS : HTP_AEE_EFAILED;
}

AEEResult htp_ops_create_channel(remote_handle64 handle, int32_t fd, uint32_t size) {
  (void) handle;
  return create_htp_message_channel(fd, size);
}

AEEResult htp_ops_destroy_channel(remote_handle64 handle) {
  (void) handle;
  stop_channel();
  return HTP_AEE_SUCCESS;
}

// Synchronous, like the FastRPC call it stands for (src/dsp/commu.c: htp_ops_rms_norm_f32 maps the
// two buffers and runs hvx_rms_norm_f32): fd0/offset0 = dst, fd1/offset1 = src.
AEEResult htp_ops_rms_norm_f32(remote_handle64 handle, int32_t fd0, int32_t offset0, int32_t fd1, int32_t offset1,
                               int32_t ne0, int32_t ne1) {
  (void) handle;
  if (!set_session_device() || !g.backend) {
    return HTP_AEE_EFAILED;
  }
  alignas(8) uint8_t raw[sizeof(OpComputeRequest) + sizeof(RmsNormF32Params)];
  OpComputeRequest  *req = reinterpret_cast<OpComputeRequest *>(raw);
  req->op                = HTP_OPS_RMS_NORM_F32;
  RmsNormF32Params rp;
  rp.dst.fd = fd0, rp.dst.offset = offset0, rp.src.fd = fd1, rp.src.offset = offset1, rp.ne0 = ne0, rp.ne1 = ne1;
  memcpy(req->payload, &rp, sizeof(rp));
  return execute_op_simple(req) == 0 ? HTP_AEE_SUCCESS : HTP_AEE_EFAILED;
}

AEEResult htp_ops_mat_mul_permuted_w16a32(remote_handle64 handle, int32_t fd0, int32_t offset0, int32_t fd1,
                                          int32_t offset1, int32_t fd2, int32_t offset2, int32_t m, int32_t k,
                                          int32_t n) {
  (void) handle;
  if (!set_session_device() || !g.backend) {
    return HTP_AEE_EFAILED;
  }
  alignas(8) uint8_t raw[sizeof(OpComputeRequest) + sizeof(MatMulParams)];
  OpComputeRequest  *req = reinterpret_cast<OpComputeRequest *>(raw);
  req->op                = HTP_OPS_MAT_MUL_PERMUTED_W16A32;
  MatMulParams p;
  p.output.fd = fd0, p.output.offset = offset0, p.activation.fd = fd1, p.activation.offset = offset1;
  p.weight.fd = fd2, p.weight.offset = offset2, p.m = m, p.k = k, p.n = n;
  memcpy(req->payload, &p, sizeof(p));
  return execute_op_simple(req) == 0 ? HTP_AEE_SUCCESS : HTP_AEE_EFAILED;
}

AEEResult htp_ops_test_ops(remote_handle64 handle) {
  (void) handle;
  return HTP_AEE_SUCCESS;
}

int htp_ops_rpc_rms_norm_f32(int dst_fd, int dst_offset, int src_fd, int src_offset, int ne0, int ne1) {
  return htp_ops_rms_norm_f32(get_global_handle(), dst_fd, dst_offset, src_fd, src_offset, ne0, ne1);
}

int htp_ops_rpc_mat_mul_permuted_w16a32(int output_fd, int output_offset, int activation_fd, int activation_offset,
                                        int weight_fd, int weight_offset, int m, int k, int n) {
  return htp_ops_mat_mul_permuted_w16a32(get_global_handle(), output_fd, output_offset, activation_fd,
                                         activation_offset, weight_fd, weight_offset, m, k, n);
}

// ---------------------------------------------------------------- dispatch

int execute_op_simple(struct OpComputeRequest *req) {
  if (!req || !set_session_device() || !g.backend) {
    return -1;
  }
  std::lock_guard<std::mutex> op_lock(g.op_mu);
  const int                   rc = enqueue_op(req, nullptr);
  if (rc != 0) {
    return rc;
  }
  return wait_stream();
}

// ---------------------------------------------------------------- buffers

int htp_buf_alloc(size_t size) {
  if (!set_session_device() || size == 0) {
    return -1;
  }
  Buffer b;
  if (cudaMalloc(&b.ptr, size) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  // Zero-fill on the session stream and wait: a cudaMemset on the default stream is asynchronous
  // and NOT ordered with the (non-blocking) session stream, so it could land after an operator
  // had already written the buffer.
  if (cudaMemsetAsync(b.ptr, 0, size, g.stream) != cudaSuccess || cudaStreamSynchronize(g.stream) != cudaSuccess) {
    cudaGetLastError();
    cudaFree(b.ptr);
    return -1;
  }
  b.size = size;
  b.kind = kDeviceBuf;
  return register_buffer(b);
}

int htp_buf_alloc_host(size_t size) {
  if (!set_session_device() || size == 0) {
    return -1;
  }
  Buffer b;
  if (cudaHostAlloc(&b.ptr, size, cudaHostAllocDefault) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  memset(b.ptr, 0, size);
  b.size = size;
  b.kind = kHostBuf;
  return register_buffer(b);
}

int htp_buf_alloc_shared(size_t size) {
  if (!set_session_device() || size == 0) {
    return -1;
  }
  Buffer b;
  void  *dp = nullptr;
  if (cudaHostAlloc(&b.ptr, size, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  // unified addressing: the device reaches the bytes at the host address (anything else is not supported here)
  if (cudaHostGetDevicePointer(&dp, b.ptr, 0) != cudaSuccess || dp != b.ptr) {
    cudaGetLastError();
    cudaFreeHost(b.ptr);
    return -1;
  }
  memset(b.ptr, 0, size);
  b.size = size;
  b.kind = kSharedBuf;
  return register_buffer(b);
}

int htp_buf_wrap(void *device_ptr, size_t size) {
  if (!g.open || !device_ptr || size == 0) {
    return -1;
  }
  Buffer b;
  b.ptr  = static_cast<uint8_t *>(device_ptr);
  b.size = size;
  b.kind = kWrappedBuf;
  return register_buffer(b);
}

int htp_buf_free(int fd) {
  Buffer b;
  {
    std::lock_guard<std::mutex> lk(g.mu);
    auto                        it = g.bufs.find(fd);
    if (it == g.bufs.end() || fd == g.chan_fd) {
      return -1;  // unknown, or still the active message buffer
    }
    b = it->second;
    g.bufs.erase(it);
  }
  if (!set_session_device()) {
    return -1;
  }
  if (b.kind == kDeviceBuf) {
    if (g.stream) {
      cudaStreamSynchronize(g.stream);
    }
    cudaFree(b.ptr);
  } else if (b.kind == kHostBuf) {
    cudaFreeHost(b.ptr);
  } else if (b.kind == kSharedBuf) {
    if (g.stream) {
      cudaStreamSynchronize(g.stream);  // an operator may still be writing it
    }
    cudaFreeHost(b.ptr);
  }
  return 0;
}

static int copy_region(int fd, size_t offset, void *host, size_t size, bool upload, bool wait = true) {
  Buffer b;
  if (!host || !lookup(fd, &b) || offset > b.size || size > b.size - offset) {
    return -1;
  }
  if (size == 0) {
    return 0;
  }
  if (b.kind == kHostBuf || b.kind == kSharedBuf) {
    if (b.kind == kSharedBuf && set_session_device() && g.stream) {
      // the copy below is the host's own: operators enqueued before may still be reading or writing the
      // bytes, so the stream order a device buffer's copy would have is kept by waiting (also in the
      // "async" forms - a host that wants no wait writes and reads the shared bytes itself)
      cudaStreamSynchronize(g.stream);
    }
    if (upload) {
      memcpy(b.ptr + offset, host, size);
    } else {
      memcpy(host, b.ptr + offset, size);
    }
    return 0;
  }
  if (!set_session_device()) {
    return -1;
  }
  cudaError_t e = upload ? cudaMemcpyAsync(b.ptr + offset, host, size, cudaMemcpyHostToDevice, g.stream)
                         : cudaMemcpyAsync(host, b.ptr + offset, size, cudaMemcpyDeviceToHost, g.stream);
  if (e == cudaSuccess && wait) {
    e = cudaStreamSynchronize(g.stream);
  }
  if (e != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return 0;
}

int htp_buf_upload(int fd, size_t offset, const void *src, size_t size) {
  return copy_region(fd, offset, const_cast<void *>(src), size, true);
}

int htp_buf_upload_async(int fd, size_t offset, const void *src, size_t size) {
  return copy_region(fd, offset, const_cast<void *>(src), size, true, false);
}

int htp_buf_download_async(int fd, size_t offset, void *dst, size_t size) {
  return copy_region(fd, offset, dst, size, false, false);
}

int htp_buf_download(int fd, size_t offset, void *dst, size_t size) {
  return copy_region(fd, offset, dst, size, false);
}

void *htp_buf_ptr(int fd) {
  Buffer b;
  return lookup(fd, &b) ? b.ptr : nullptr;
}

int htp_buf_is_host(int fd) {
  Buffer b;
  return lookup(fd, &b) ? (b.kind == kHostBuf ? 1 : (b.kind == kSharedBuf ? 2 : 0)) : -1;
}

size_t htp_buf_size(int fd) {
  Buffer b;
  return lookup(fd, &b) ? b.size : 0;
}

void *htp_session_stream(void) {
  return g.open ? (void *) g.stream : nullptr;
}

int htp_session_synchronize(void) {
  if (!set_session_device() || !g.backend) {
    return -2;
  }
  std::lock_guard<std::mutex> op_lock(g.op_mu);
  return wait_stream();
}

}  // extern "C"
