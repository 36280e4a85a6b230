// Host side of the row reduction whose reduced axis is sharded over GPUs: the mailbox every rank owns, the
// handle that describes it to the other ranks, and the launch that fills in the kernel's exchange record.
// The device side is exchangeTail() in kernels/row_reduce.cu.
//
// Mailbox layout (one cudaMalloc, so that one IPC handle covers it):
//   [256, 260)   CTAs or warps of the running launch that are done (local use)
//   [260, 264)   status word (local use)
//   [272, 280)   {completed calls : arrivals of the running launch} (local use): every CTA of a launch adds one
//                and learns the call's number from what it gets back; the last one moves the word on, so a launch
//                has no argument that changes from call to call
//   [512, ...)   entries[2][world][maxRows], eight bytes each: {f32 partial sum, epoch}.  The epoch's parity picks
//                the half, so a rank that is already sending call e+1 cannot overwrite an entry a slower rank has
//                not yet read for call e; it can send call e+2 only after it finished e+1, which needs every
//                rank's e+1 entries, which they send after they finished reading e.
#include "runtime/rowsum_exchange.h"

#include "runtime/caller_device.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <unistd.h>

namespace {

constexpr size_t kDoneOffset = 256, kStatusOffset = 260, kCallWordOffset = 272, kSlotsOffset = 512;

struct Handle {  // AFIRT_EXCHANGE_HANDLE_BYTES
  cudaIpcMemHandle_t ipc;  // 64 bytes
  uint64_t pid;
  uint64_t address;        // the mailbox as its owner sees it (used inside one process)
  int32_t device;
  int32_t rank;
  int64_t maxRows;
};
static_assert(sizeof(Handle) == AFIRT_EXCHANGE_HANDLE_BYTES, "handle layout");

void fail(char *buf, size_t len, const char *what, cudaError_t e = cudaSuccess) {
  if (!buf || len == 0) return;
  if (e != cudaSuccess) std::snprintf(buf, len, "%s: %s", what, cudaGetErrorString(e));
  else std::snprintf(buf, len, "%s", what);
}

} // namespace

struct AfirtRowsumExchange_s {
  int device = 0, rank = 0, world = 1;
  int64_t maxRows = 0;
  char *mailbox = nullptr;
  char *peer[AFIRT_EXCHANGE_MAX_RANKS] = {nullptr};
  bool viaIpc[AFIRT_EXCHANGE_MAX_RANKS] = {false};
  bool connected = false;
  unsigned long long callsIssued = 0;  // launches enqueued through this handle (the call number itself lives in the mailbox)
  int64_t slotStride() const { return maxRows; }  // entries
  size_t slotsBytesPerHalf() const { return static_cast<size_t>(world) * static_cast<size_t>(slotStride()) * sizeof(unsigned long long); }
};

#define AFIRT_EXPORT extern "C" __attribute__((visibility("default")))

AFIRT_EXPORT int afirt_rowsum_exchange_create(int device_id, int rank, int world_size, int64_t max_rows,
                                              AfirtRowsumExchange *out_exchange, uint8_t *out_handle, char *err_buf, size_t err_len) {
  if (!out_exchange || !out_handle) { fail(err_buf, err_len, "out_exchange and out_handle are required"); return 1; }
  *out_exchange = nullptr;
  if (device_id < 0) { fail(err_buf, err_len, "device id must not be negative"); return 1; }
  if (world_size < 1 || world_size > AFIRT_EXCHANGE_MAX_RANKS) { fail(err_buf, err_len, "world_size must be 1..8"); return 1; }
  if (rank < 0 || rank >= world_size) { fail(err_buf, err_len, "rank must be in [0, world_size)"); return 1; }
  if (max_rows < 1 || max_rows > (1ll << 28)) { fail(err_buf, err_len, "max_rows must be in [1, 2^28]"); return 1; }
  afir::CallerDeviceScope keepCallerDevice;
  cudaError_t e = cudaSetDevice(device_id);
  if (e != cudaSuccess) { fail(err_buf, err_len, "cudaSetDevice", e); return 1; }
  auto *x = new AfirtRowsumExchange_s;
  x->device = device_id;
  x->rank = rank;
  x->world = world_size;
  x->maxRows = max_rows;
  const size_t bytes = kSlotsOffset + 2 * x->slotsBytesPerHalf();
  e = cudaMalloc(reinterpret_cast<void **>(&x->mailbox), bytes);
  if (e == cudaSuccess) e = cudaMemset(x->mailbox, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  Handle h;
  std::memset(&h, 0, sizeof(h));
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h.ipc, x->mailbox);
  if (e != cudaSuccess) {
    fail(err_buf, err_len, "mailbox allocation", e);
    if (x->mailbox) cudaFree(x->mailbox);
    delete x;
    return 1;
  }
  h.pid = static_cast<uint64_t>(getpid());
  h.address = reinterpret_cast<uint64_t>(x->mailbox);
  h.device = device_id;
  h.rank = rank;
  h.maxRows = max_rows;
  std::memcpy(out_handle, &h, sizeof(h));
  *out_exchange = x;
  return 0;
}

AFIRT_EXPORT int afirt_rowsum_exchange_connect(AfirtRowsumExchange x, const uint8_t *all_handles, char *err_buf, size_t err_len) {
  if (!x || !all_handles) { fail(err_buf, err_len, "exchange and all_handles are required"); return 1; }
  if (x->connected) { fail(err_buf, err_len, "exchange is already connected"); return 1; }
  afir::CallerDeviceScope keepCallerDevice;
  cudaError_t e = cudaSetDevice(x->device);
  if (e != cudaSuccess) { fail(err_buf, err_len, "cudaSetDevice", e); return 1; }
  for (int p = 0; p < x->world; ++p) {
    Handle h;
    std::memcpy(&h, all_handles + static_cast<size_t>(p) * sizeof(Handle), sizeof(h));
    if (h.rank != p || h.maxRows != x->maxRows) {
      char msg[160];
      std::snprintf(msg, sizeof(msg), "handle %d describes rank %d with max_rows %lld; expected rank %d with max_rows %lld", p,
                    h.rank, static_cast<long long>(h.maxRows), p, static_cast<long long>(x->maxRows));
      fail(err_buf, err_len, msg);
      return 1;
    }
    if (p == x->rank) {
      if (h.address != reinterpret_cast<uint64_t>(x->mailbox) || h.pid != static_cast<uint64_t>(getpid())) {
        fail(err_buf, err_len, "the handle at this rank's position is not this exchange's own");
        return 1;
      }
      x->peer[p] = x->mailbox;
      continue;
    }
    if (h.device == x->device) {
      fail(err_buf, err_len, "two ranks share a GPU: ranks that wait for one another need a device each");
      return 1;
    }
    if (h.pid == static_cast<uint64_t>(getpid())) {
      int can = 0;
      e = cudaDeviceCanAccessPeer(&can, x->device, h.device);
      if (e == cudaSuccess && !can) { fail(err_buf, err_len, "no peer access between the two devices"); return 1; }
      if (e == cudaSuccess) {
        e = cudaDeviceEnablePeerAccess(h.device, 0);
        if (e == cudaErrorPeerAccessAlreadyEnabled) { e = cudaSuccess; (void)cudaGetLastError(); }
      }
      if (e != cudaSuccess) { fail(err_buf, err_len, "enabling peer access", e); return 1; }
      x->peer[p] = reinterpret_cast<char *>(h.address);
    } else {
      void *mapped = nullptr;
      e = cudaIpcOpenMemHandle(&mapped, h.ipc, cudaIpcMemLazyEnablePeerAccess);
      if (e != cudaSuccess) { fail(err_buf, err_len, "cudaIpcOpenMemHandle", e); return 1; }
      x->peer[p] = static_cast<char *>(mapped);
      x->viaIpc[p] = true;
    }
  }
  x->connected = true;
  return 0;
}

AFIRT_EXPORT int afirt_bcast_add_rowsum_exchange(AfirtRowsumExchange x, int elem_type, const void *a, const void *b, void *out,
                                                 int64_t rows, int64_t cols, int64_t b_row_stride, void *cuda_stream,
                                                 char *err_buf, size_t err_len) {
  using namespace afir::kernels;
  if (!x || !x->connected) { fail(err_buf, err_len, "exchange is not connected"); return 1; }
  if (elem_type != kF32 && elem_type != kF16 && elem_type != kBF16) { fail(err_buf, err_len, "elem_type must be 0 (f32), 1 (f16) or 2 (bf16)"); return 1; }
  if (rows < 1 || rows > x->maxRows) { fail(err_buf, err_len, "rows must be in [1, max_rows]"); return 1; }
  if (cols < 0 || b_row_stride < cols) { fail(err_buf, err_len, "cols must not be negative and b_row_stride at least cols"); return 1; }
  if (!a || !out || (!b && cols > 0)) { fail(err_buf, err_len, "a, b and out are required"); return 1; }
  afir::CallerDeviceScope keepCallerDevice;
  cudaError_t e = cudaSetDevice(x->device);
  if (e != cudaSuccess) { fail(err_buf, err_len, "cudaSetDevice", e); return 1; }

  RowReduceExchange rx = {};
  int mailboxDevice = 0;
  if (afir::Status st = afir::nextExchangeCall(x, rx, mailboxDevice); !st) { fail(err_buf, err_len, st.message().c_str()); return 1; }

  RowReduceLaunch l = {};
  l.elemType = elem_type;
  l.rows = rows;
  l.cols = cols;
  l.numViews = 2;
  l.views[0].base = a;  // a[m]: follows the row, broadcast along the columns
  l.views[0].rowStride = 1;
  l.views[0].colStride = 0;
  l.views[1].base = b;  // this rank's column slice of b[m, n]
  l.views[1].rowStride = b_row_stride;
  l.views[1].colStride = 1;
  l.out = out;
  l.body.numOps = 1;
  l.body.ops[0].op = kOpAdd;
  l.body.ops[0].a = {kSrcView, 0, 0.0f};
  l.body.ops[0].b = {kSrcView, 1, 0.0f};
  l.exchange = &rx;
  int launched = 0;
  const int rc = launchRowReduce(l, static_cast<cudaStream_t>(cuda_stream), &launched);
  if (rc != 0) { fail(err_buf, err_len, "launch", static_cast<cudaError_t>(rc)); return 1; }
  afir::commitExchangeCall(x, rx);
  return 0;
}

// A run of `count` independent reductions of the same shape (operands a[i], b[i], out[i]) enqueued back to back
// on one stream by one call: what a caller with a queue of work (layers, micro-batches) does, without paying the
// language binding once per reduction.  Collective like the single call: every rank passes the same count.
AFIRT_EXPORT int afirt_bcast_add_rowsum_exchange_batch(AfirtRowsumExchange x, int elem_type, int count, const void *const *a,
                                                       const void *const *b, void *const *out, int64_t rows, int64_t cols,
                                                       int64_t b_row_stride, void *cuda_stream, char *err_buf, size_t err_len) {
  if (count < 0 || (count > 0 && (!a || !b || !out))) { fail(err_buf, err_len, "count must not be negative and the pointer arrays are required"); return 1; }
  for (int i = 0; i < count; ++i)
    if (afirt_bcast_add_rowsum_exchange(x, elem_type, a[i], b[i], out[i], rows, cols, b_row_stride, cuda_stream, err_buf, err_len) != 0) return 1;
  return 0;
}

namespace afir {

Status nextExchangeCall(AfirtRowsumExchange x, kernels::RowReduceExchange &rx, int &device) {
  if (!x || !x->connected) return Status::error("exchange is not connected");
  rx = kernels::RowReduceExchange();
  for (int p = 0; p < x->world; ++p)
    rx.peerEntries[p] = reinterpret_cast<unsigned long long *>(x->peer[p] + kSlotsOffset) + static_cast<size_t>(x->rank) * x->slotStride();
  rx.myEntries = reinterpret_cast<const unsigned long long *>(x->mailbox + kSlotsOffset);
  rx.doneCounter = reinterpret_cast<unsigned int *>(x->mailbox + kDoneOffset);
  rx.status = reinterpret_cast<unsigned int *>(x->mailbox + kStatusOffset);
  rx.callWord = reinterpret_cast<unsigned long long *>(x->mailbox + kCallWordOffset);
  rx.world = x->world;
  rx.slotStride = x->slotStride();
  rx.halfStride = static_cast<long long>(x->slotsBytesPerHalf() / sizeof(unsigned long long));
  device = x->device;
  return Status::success();
}

void commitExchangeCall(AfirtRowsumExchange x, const kernels::RowReduceExchange &) { ++x->callsIssued; }

} // namespace afir

AFIRT_EXPORT int afirt_rowsum_exchange_status(AfirtRowsumExchange x, char *err_buf, size_t err_len) {
  if (!x) { fail(err_buf, err_len, "exchange is required"); return 1; }
  afir::CallerDeviceScope keepCallerDevice;
  cudaError_t e = cudaSetDevice(x->device);
  unsigned int words[2] = {0, 0};  // done counter, status
  if (e == cudaSuccess) e = cudaMemcpy(words, x->mailbox + kDoneOffset, sizeof(words), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) { fail(err_buf, err_len, "reading the status word", e); return 1; }
  char stagedText[256];
  const int staged = afir::kernels::rowReduceCheckStatus(x->device, stagedText);
  if (words[1] == 0 && !staged) return 0;
  cudaMemset(x->mailbox + kDoneOffset, 0, sizeof(words));
  if (words[1] != 0)
    fail(err_buf, err_len, "row-sum exchange: gave up waiting for another rank's partial sums after 2 s");
  else
    fail(err_buf, err_len, stagedText);
  return 1;
}

AFIRT_EXPORT void afirt_rowsum_exchange_destroy(AfirtRowsumExchange x) {
  if (!x) return;
  afir::CallerDeviceScope keepCallerDevice;
  if (cudaSetDevice(x->device) == cudaSuccess) {
    cudaDeviceSynchronize();
    for (int p = 0; p < x->world; ++p)
      if (x->viaIpc[p] && x->peer[p]) cudaIpcCloseMemHandle(x->peer[p]);
    if (x->mailbox) cudaFree(x->mailbox);
  }
  delete x;
}
