// Collectives over NCCL (NVLink / NVSwitch).  The reference is single-device and
// has nothing here; this file gives the data-parallel trainer its gradient
// all-reduce and the column-sharded INT8 path its max-reduce and all-gather.
// libnccl.so.2 is loaded on first use so that the library itself has no link
// dependency on NCCL; single-GPU users never touch it.
#include <dlfcn.h>
#include <nccl.h>

#include "common.cuh"

namespace {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommSplit)(ncclComm_t, int, int, ncclComm_t*, void*) = nullptr;  // optional (NCCL >= 2.18)
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                            cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t,
                            cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
};
NcclApi g_nccl;

int load_nccl(vtlb_ctx* ctx) {
  if (g_nccl.handle) return VTLB_OK;
  void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  if (!h) return vtlb_fail(ctx, VTLB_ENCCL, "cannot load libnccl.so.2: %s", dlerror());
#define VTLB_SYM(field, name)                                                    \
  *(void**)(&g_nccl.field) = dlsym(h, name);                                     \
  if (!g_nccl.field) return vtlb_fail(ctx, VTLB_ENCCL, "libnccl lacks %s", name)
  VTLB_SYM(GetUniqueId, "ncclGetUniqueId");
  VTLB_SYM(CommInitRank, "ncclCommInitRank");
  VTLB_SYM(CommDestroy, "ncclCommDestroy");
  VTLB_SYM(AllReduce, "ncclAllReduce");
  VTLB_SYM(AllGather, "ncclAllGather");
  VTLB_SYM(GetErrorString, "ncclGetErrorString");
#undef VTLB_SYM
  *(void**)(&g_nccl.CommSplit) = dlsym(h, "ncclCommSplit");
  g_nccl.handle = h;
  return VTLB_OK;
}

#define VTLB_NCCL(ctx, call)                                                      \
  do {                                                                            \
    ncclResult_t r__ = (call);                                                    \
    if (r__ != ncclSuccess)                                                       \
      return vtlb_fail((ctx), VTLB_ENCCL, "%s: %s -> %s", __func__, #call,        \
                       g_nccl.GetErrorString(r__));                               \
  } while (0)

// Orders a communication stream after everything enqueued on the compute stream.
int comm_after_compute(vtlb_ctx* ctx, cudaStream_t lane) {
  VTLB_CUDA(ctx, cudaEventRecord(ctx->ev_compute, ctx->stream));
  VTLB_CUDA(ctx, cudaStreamWaitEvent(lane, ctx->ev_compute, 0));
  return VTLB_OK;
}
int comm_after_compute(vtlb_ctx* ctx) { return comm_after_compute(ctx, ctx->comm_stream); }

int need_comm(vtlb_ctx* ctx, const char* fn) {
  if (!ctx->comm) return vtlb_fail(ctx, VTLB_ESTATE, "%s: vtlb_comm_init_rank has not been called", fn);
  return VTLB_OK;
}

}  // namespace

VTLB_API int vtlb_comm_unique_id(void* h_id128) {
  if (!h_id128) return vtlb_fail(nullptr, VTLB_EINVAL, "vtlb_comm_unique_id: null out");
  int rc = load_nccl(nullptr);
  if (rc) return rc;
  static_assert(sizeof(ncclUniqueId) == 128, "unique id size");
  ncclUniqueId id;
  VTLB_NCCL(nullptr, g_nccl.GetUniqueId(&id));
  memcpy(h_id128, &id, sizeof id);
  return VTLB_OK;
}

namespace {
bool open_small_lane(vtlb_ctx* ctx) {
  if (ctx->comm_small) return true;
  if (!g_nccl.CommSplit || ctx->nranks < 2) return false;
  ncclComm_t small = nullptr;
  if (g_nccl.CommSplit((ncclComm_t)ctx->comm, 0, ctx->rank, &small, nullptr) != ncclSuccess || !small) return false;
  if (cudaStreamCreateWithFlags(&ctx->comm_small_stream, cudaStreamNonBlocking) != cudaSuccess) {
    cudaGetLastError();
    g_nccl.CommDestroy(small);
    return false;
  }
  ctx->comm_small = small;
  return true;
}
}  // namespace

VTLB_API int vtlb_comm_init_rank(vtlb_ctx* ctx, int nranks, int rank, const void* h_id128) {
  VTLB_ENTER(ctx);
  if (nranks < 1 || rank < 0 || rank >= nranks || !h_id128)
    return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_comm_init_rank: bad arguments (nranks %d, rank %d)", nranks, rank);
  if (ctx->comm) return vtlb_fail(ctx, VTLB_ESTATE, "vtlb_comm_init_rank: communicator already exists");
  int rc = load_nccl(ctx);
  if (rc) return rc;
  ncclUniqueId id;
  memcpy(&id, h_id128, sizeof id);
  ncclComm_t comm = nullptr;
  VTLB_NCCL(ctx, g_nccl.CommInitRank(&comm, nranks, id, rank));
  ctx->comm = comm;
  ctx->nranks = nranks;
  ctx->rank = rank;
  // the lane for small collectives: a communicator of its own, so that NCCL may run both at once
  static int two_lanes = -1;
  if (two_lanes < 0) {
    const char* e = getenv("VTLB_COMM_TWO_LANES");
    two_lanes = e ? atoi(e) != 0 : 0;  // off by default: on 2 GPUs two NCCL kernels at once cost the GEMMs more than the queueing
  }
  if (two_lanes) open_small_lane(ctx);
  return VTLB_OK;
}

// A lane of its own for the small collectives of this communicator (collective: every rank calls it).
// Worth it when the bulk lane carries copy-engine transfers (vtlb_allgather_push_async): a 32 KB
// all-reduce then runs beside them instead of queueing behind 200 MB of copies.  Beside NCCL's own
// bulk kernels it measured no gain (two NCCL kernels at once cost the GEMMs as much as the queueing).
VTLB_API int vtlb_comm_small_lane(vtlb_ctx* ctx) {
  VTLB_ENTER(ctx);
  int rc = need_comm(ctx, __func__);
  if (rc) return rc;
  if (ctx->comm_small || ctx->nranks < 2) return VTLB_OK;
  if (!g_nccl.CommSplit) return vtlb_fail(ctx, VTLB_ESTATE, "vtlb_comm_small_lane: this NCCL has no ncclCommSplit");
  if (!open_small_lane(ctx)) return vtlb_fail(ctx, VTLB_ECUDA, "vtlb_comm_small_lane: could not split the communicator");
  return VTLB_OK;
}

VTLB_API int vtlb_comm_destroy(vtlb_ctx* ctx) {
  if (!ctx || !ctx->comm) return VTLB_OK;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->comm_stream);
  if (ctx->comm_small) {
    cudaStreamSynchronize(ctx->comm_small_stream);
    g_nccl.CommDestroy((ncclComm_t)ctx->comm_small);
    cudaStreamDestroy(ctx->comm_small_stream);
    ctx->comm_small = nullptr;
    ctx->comm_small_stream = nullptr;
  }
  if (ctx->comm_barrier_word) {
    cudaFree(ctx->comm_barrier_word);
    ctx->comm_barrier_word = nullptr;
  }
  for (auto& ev : ctx->comm_marks)
    if (ev) {
      cudaEventDestroy(ev);
      ev = nullptr;
    }
  g_nccl.CommDestroy((ncclComm_t)ctx->comm);
  ctx->comm = nullptr;
  ctx->nranks = 1;
  ctx->rank = 0;
  return VTLB_OK;
}

VTLB_API int vtlb_allreduce_sum_f32_async(vtlb_ctx* ctx, void* d_buf, size_t n) {
  VTLB_ENTER(ctx);
  int rc = need_comm(ctx, __func__);
  if (rc) return rc;
  if (n == 0) return VTLB_OK;
  if ((rc = comm_after_compute(ctx))) return rc;
  VTLB_NCCL(ctx, g_nccl.AllReduce(d_buf, d_buf, n, ncclFloat32, ncclSum, (ncclComm_t)ctx->comm, ctx->comm_stream));
  vtlb_comm_track(ctx, d_buf, n * sizeof(float));
  return VTLB_OK;
}

VTLB_API int vtlb_allreduce_max_f32_async(vtlb_ctx* ctx, void* d_buf, size_t n) {
  VTLB_ENTER(ctx);
  int rc = need_comm(ctx, __func__);
  if (rc) return rc;
  if (n == 0) return VTLB_OK;
  const bool small = ctx->comm_small != nullptr;
  cudaStream_t lane = small ? ctx->comm_small_stream : ctx->comm_stream;
  if ((rc = comm_after_compute(ctx, lane))) return rc;
  VTLB_NCCL(ctx, g_nccl.AllReduce(d_buf, d_buf, n, ncclFloat32, ncclMax,
                                  (ncclComm_t)(small ? ctx->comm_small : ctx->comm), lane));
  vtlb_comm_track(ctx, d_buf, n * sizeof(float));
  return VTLB_OK;
}

VTLB_API int vtlb_allgather_async(vtlb_ctx* ctx, const void* d_send, void* d_recv, size_t bytes_per_rank) {
  VTLB_ENTER(ctx);
  int rc = need_comm(ctx, __func__);
  if (rc) return rc;
  if (bytes_per_rank == 0) return VTLB_OK;
  if ((rc = comm_after_compute(ctx))) return rc;
  VTLB_NCCL(ctx, g_nccl.AllGather(d_send, d_recv, bytes_per_rank, ncclInt8, (ncclComm_t)ctx->comm, ctx->comm_stream));
  vtlb_comm_track(ctx, d_send, bytes_per_rank);
  vtlb_comm_track(ctx, d_recv, bytes_per_rank * (size_t)ctx->nranks);
  return VTLB_OK;
}

// ---------------------------------------------------------------- all-gather by copy engines
// NCCL's all-gather runs as a kernel on 16 to 32 SMs.  Beside a persistent GEMM that wants every SM
// (one CTA pair per TPC, tiles assigned statically) that costs far more than its share: pairs that
// start late finish late, and the column-sharded inference pipeline measured its GEMMs 50 % slower
// while an all-gather was in flight.  Here the copy engines move the data: every rank exports its
// receive buffer to the other processes (CUDA IPC), and an all-gather is each rank copying its part
// straight into every peer's buffer over NVLink, followed by an all-reduce of one word -- when that
// completes on a rank, every rank has entered it, which it does only after its own copies: all parts
// have landed everywhere.  No SM is used except by that one-word collective.
VTLB_API int vtlb_shared_alloc(vtlb_ctx* ctx, size_t bytes, void** d_out, void* h_handle64) {
  VTLB_ENTER(ctx);
  if (!d_out || !h_handle64 || bytes == 0) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_shared_alloc: bad arguments");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  *d_out = nullptr;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return vtlb_fail(ctx, VTLB_ENOMEM, "vtlb_shared_alloc(%zu bytes): %s", bytes, cudaGetErrorString(e));
  }
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    cudaFree(p);
    return vtlb_fail(ctx, VTLB_ECUDA, "vtlb_shared_alloc: cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
  }
  VTLB_CUDA(ctx, cudaMemset(p, 0, bytes));
  memcpy(h_handle64, &h, sizeof h);
  *d_out = p;
  return VTLB_OK;
}

VTLB_API int vtlb_shared_free(vtlb_ctx* ctx, void* d_ptr) {
  VTLB_ENTER(ctx);
  if (!d_ptr) return VTLB_OK;
  VTLB_CUDA(ctx, cudaDeviceSynchronize());
  VTLB_CUDA(ctx, cudaFree(d_ptr));
  return VTLB_OK;
}

VTLB_API int vtlb_shared_open(vtlb_ctx* ctx, const void* h_handle64, void** d_peer_out) {
  VTLB_ENTER(ctx);
  if (!h_handle64 || !d_peer_out) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_shared_open: null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, h_handle64, sizeof h);
  *d_peer_out = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(d_peer_out, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return vtlb_fail(ctx, VTLB_ECUDA, "vtlb_shared_open: cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
  }
  return VTLB_OK;
}

VTLB_API int vtlb_shared_close(vtlb_ctx* ctx, void* d_peer) {
  VTLB_ENTER(ctx);
  if (!d_peer) return VTLB_OK;
  VTLB_CUDA(ctx, cudaDeviceSynchronize());
  VTLB_CUDA(ctx, cudaIpcCloseMemHandle(d_peer));
  return VTLB_OK;
}

VTLB_API int vtlb_allgather_push_async(vtlb_ctx* ctx, const void* d_src, void* const* d_peer_dst, int npeers,
                                       size_t bytes) {
  VTLB_ENTER(ctx);
  int rc = need_comm(ctx, __func__);
  if (rc) return rc;
  if (!d_src || !d_peer_dst || npeers < 0) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_allgather_push_async: bad arguments");
  if (!ctx->comm_barrier_word) {
    VTLB_CUDA(ctx, cudaMalloc(&ctx->comm_barrier_word, 256));
    VTLB_CUDA(ctx, cudaMemset(ctx->comm_barrier_word, 0, 256));
  }
  if ((rc = comm_after_compute(ctx))) return rc;
  // rank r starts with peer r + 1: at every moment the ranks write to different receivers, so no
  // receiver's link carries more than one copy at a time.  (Dealing the seven copies of a push to two
  // or four streams, so that they overlap, breaks exactly that: 2.39 -> 3.11 / 3.25 ms per forward
  // of the column-sharded MLP on 8 GPUs.)
  for (int i = 1; i <= npeers; ++i) {
    const int r = (ctx->rank + i) % npeers;
    if (d_peer_dst[r] && bytes)
      VTLB_CUDA(ctx, cudaMemcpyAsync(d_peer_dst[r], d_src, bytes, cudaMemcpyDeviceToDevice, ctx->comm_stream));
  }
  VTLB_NCCL(ctx, g_nccl.AllReduce(ctx->comm_barrier_word, ctx->comm_barrier_word, 1, ncclFloat32, ncclSum,
                                  (ncclComm_t)ctx->comm, ctx->comm_stream));
  vtlb_comm_track(ctx, d_src, bytes);
  return VTLB_OK;
}

VTLB_API int vtlb_comm_mark(vtlb_ctx* ctx, int lane, int slot) {
  VTLB_ENTER(ctx);
  if (slot < 0 || slot >= vtlb_ctx::kCommMarks || lane < 0 || lane > 1)
    return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_comm_mark: lane %d / slot %d out of range", lane, slot);
  if (!ctx->comm_marks[slot]) VTLB_CUDA(ctx, cudaEventCreateWithFlags(&ctx->comm_marks[slot], cudaEventDisableTiming));
  cudaStream_t s = (lane == VTLB_COMM_LANE_SMALL && ctx->comm_small) ? ctx->comm_small_stream : ctx->comm_stream;
  VTLB_CUDA(ctx, cudaEventRecord(ctx->comm_marks[slot], s));
  return VTLB_OK;
}

VTLB_API int vtlb_comm_wait_mark(vtlb_ctx* ctx, int slot) {
  VTLB_ENTER(ctx);
  if (slot < 0 || slot >= vtlb_ctx::kCommMarks || !ctx->comm_marks[slot])
    return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_comm_wait_mark: slot %d was never marked", slot);
  vtlb_prof_scope prof(ctx, VTLB_PHASE_COMM_WAIT);
  VTLB_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->comm_marks[slot], 0));
  return VTLB_OK;
}

VTLB_API int vtlb_comm_wait(vtlb_ctx* ctx) {
  VTLB_ENTER(ctx);
  vtlb_prof_scope prof(ctx, VTLB_PHASE_COMM_WAIT);  // how long the compute stream stands idle here
  if (ctx->comm_small) {
    VTLB_CUDA(ctx, cudaEventRecord(ctx->ev_comm, ctx->comm_small_stream));
    VTLB_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->ev_comm, 0));
  }
  VTLB_CUDA(ctx, cudaEventRecord(ctx->ev_comm, ctx->comm_stream));
  VTLB_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->ev_comm, 0));
  ctx->comm_inflight.clear();  // the compute stream is now ordered after every collective enqueued so far
  return VTLB_OK;
}
