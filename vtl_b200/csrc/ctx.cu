// Context, device memory and status: the part of the C ABI that stands where
// vtl's CudaStorage (storage/cuda_d_cuda.v) and DeviceSession buffers
// (autograd_cuda/device_session_gpu_d_cuda.v:24-45) stand in the reference.
#include <stdarg.h>

#include <new>

#include "common.cuh"

thread_local char g_vtlb_err[512] = {0};

int vtlb_fail(vtlb_ctx* ctx, int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  memcpy(g_vtlb_err, buf, sizeof buf);
  if (ctx) memcpy(ctx->err, buf, sizeof buf);
  return code;
}

VTLB_API const char* vtlb_last_error(vtlb_ctx* ctx) { return ctx ? ctx->err : g_vtlb_err; }

VTLB_API int vtlb_device_count(int* count) {
  if (!count) return vtlb_fail(nullptr, VTLB_EINVAL, "vtlb_device_count: null out");
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) {
    *count = 0;
    return vtlb_fail(nullptr, VTLB_ECUDA, "cudaGetDeviceCount: %s", cudaGetErrorString(e));
  }
  *count = n;
  return VTLB_OK;
}

VTLB_API int vtlb_ctx_create(int device, vtlb_ctx** out) {
  if (!out) return vtlb_fail(nullptr, VTLB_EINVAL, "vtlb_ctx_create: null out");
  *out = nullptr;
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0)
    return vtlb_fail(nullptr, VTLB_ECUDA, "vtlb_ctx_create: no usable CUDA device (%s)",
                     e == cudaSuccess ? "count is 0" : cudaGetErrorString(e));
  if (device < 0 || device >= n)
    return vtlb_fail(nullptr, VTLB_EINVAL, "vtlb_ctx_create: device %d out of range [0,%d)",
                     device, n);
  cudaDeviceProp prop;
  if ((e = cudaSetDevice(device)) != cudaSuccess ||
      (e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess)
    return vtlb_fail(nullptr, VTLB_ECUDA, "vtlb_ctx_create: %s", cudaGetErrorString(e));
  if (prop.major != 10)
    return vtlb_fail(nullptr, VTLB_ECUDA,
                     "vtlb_ctx_create: device %d is sm_%d%d; this library is built for sm_100a only",
                     device, prop.major, prop.minor);
  vtlb_ctx* ctx = new (std::nothrow) vtlb_ctx();
  if (!ctx) return vtlb_fail(nullptr, VTLB_ENOMEM, "vtlb_ctx_create: host allocation failed");
  ctx->device = device;
  ctx->sm_count = prop.multiProcessorCount;
  {  // keep freed blocks in the pool instead of returning them to the driver at every sync
    cudaMemPool_t pool;
    unsigned long long keep = ~0ull;
    if (cudaDeviceGetDefaultMemPool(&pool, device) == cudaSuccess)
      cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
  }
  if ((e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking)) != cudaSuccess ||
      (e = cudaStreamCreateWithFlags(&ctx->comm_stream, cudaStreamNonBlocking)) != cudaSuccess ||
      (e = cudaStreamCreateWithFlags(&ctx->copy_in, cudaStreamNonBlocking)) != cudaSuccess ||
      (e = cudaStreamCreateWithFlags(&ctx->copy_out, cudaStreamNonBlocking)) != cudaSuccess ||
      (e = cudaEventCreateWithFlags(&ctx->ev_copy, cudaEventDisableTiming)) != cudaSuccess ||
      (e = cudaEventCreateWithFlags(&ctx->ev_compute, cudaEventDisableTiming)) != cudaSuccess ||
      (e = cudaEventCreateWithFlags(&ctx->ev_comm, cudaEventDisableTiming)) != cudaSuccess ||
      (e = cudaMalloc(&ctx->d_status, 256)) != cudaSuccess ||
      (e = cudaMemset(ctx->d_status, 0, 256)) != cudaSuccess ||
      (e = cudaMalloc(&ctx->ksplit_buf, vtlb_ctx::kKsplitBytes)) != cudaSuccess ||
      (e = cudaMemset(ctx->ksplit_buf, 0, vtlb_ctx::kKsplitFlagBytes)) != cudaSuccess) {
    int rc = vtlb_fail(nullptr, VTLB_ECUDA, "vtlb_ctx_create: %s", cudaGetErrorString(e));
    vtlb_ctx_destroy(ctx);
    return rc;
  }
  *out = ctx;
  return VTLB_OK;
}

VTLB_API int vtlb_ctx_destroy(vtlb_ctx* ctx) {
  if (!ctx) return VTLB_OK;
  cudaSetDevice(ctx->device);
  if (ctx->comm) vtlb_comm_destroy(ctx);
  if (ctx->stream) cudaStreamSynchronize(ctx->stream);
  if (ctx->comm_stream) cudaStreamSynchronize(ctx->comm_stream);
  if (ctx->copy_in) cudaStreamSynchronize(ctx->copy_in);
  if (ctx->copy_out) cudaStreamSynchronize(ctx->copy_out);
  for (auto& kv : ctx->small_free)
    for (void* p : kv.second) cudaFreeAsync(p, ctx->stream);
  if (ctx->stream) cudaStreamSynchronize(ctx->stream);
  if (ctx->prof_ev) {
    for (int i = 0; i < 2 * vtlb_ctx::kProfSlots; ++i)
      if (ctx->prof_ev[i]) cudaEventDestroy(ctx->prof_ev[i]);
    delete[] ctx->prof_ev;
    delete[] ctx->prof_phase;
  }
  if (ctx->scratch) cudaFree(ctx->scratch);
  if (ctx->ksplit_buf) cudaFree(ctx->ksplit_buf);
  if (ctx->d_status) cudaFree(ctx->d_status);
  if (ctx->ev_compute) cudaEventDestroy(ctx->ev_compute);
  if (ctx->ev_comm) cudaEventDestroy(ctx->ev_comm);
  if (ctx->stream) cudaStreamDestroy(ctx->stream);
  if (ctx->comm_stream) cudaStreamDestroy(ctx->comm_stream);
  if (ctx->ev_copy) cudaEventDestroy(ctx->ev_copy);
  if (ctx->copy_in) cudaStreamDestroy(ctx->copy_in);
  if (ctx->copy_out) cudaStreamDestroy(ctx->copy_out);
  delete ctx;
  return VTLB_OK;
}

VTLB_API int vtlb_sync(vtlb_ctx* ctx) {
  VTLB_ENTER(ctx);
  VTLB_CUDA(ctx, cudaStreamSynchronize(ctx->copy_in));
  VTLB_CUDA(ctx, cudaStreamSynchronize(ctx->comm_stream));
  if (ctx->comm_small_stream) VTLB_CUDA(ctx, cudaStreamSynchronize(ctx->comm_small_stream));
  VTLB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  VTLB_CUDA(ctx, cudaStreamSynchronize(ctx->copy_out));
  return VTLB_OK;
}

// ---------------------------------------------------------------- input pipeline copies
VTLB_API int vtlb_copy_h2d_async(vtlb_ctx* ctx, void* d_dst, const void* h_src, size_t bytes) {
  VTLB_ENTER(ctx);
  if (bytes == 0) return VTLB_OK;
  if (!d_dst || !h_src) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_copy_h2d_async: null pointer");
  // the destination may still be read by compute work enqueued so far (the step that used this
  // buffer last): the copy starts after it
  VTLB_CUDA(ctx, cudaEventRecord(ctx->ev_copy, ctx->stream));
  VTLB_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_in, ctx->ev_copy, 0));
  VTLB_CUDA(ctx, cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, ctx->copy_in));
  return VTLB_OK;
}

VTLB_API int vtlb_copy_d2h_async(vtlb_ctx* ctx, void* h_dst, const void* d_src, size_t bytes) {
  VTLB_ENTER(ctx);
  if (bytes == 0) return VTLB_OK;
  if (!h_dst || !d_src) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_copy_d2h_async: null pointer");
  VTLB_CUDA(ctx, cudaEventRecord(ctx->ev_copy, ctx->stream));  // after the work that produces d_src
  VTLB_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_out, ctx->ev_copy, 0));
  VTLB_CUDA(ctx, cudaMemcpyAsync(h_dst, d_src, bytes, cudaMemcpyDeviceToHost, ctx->copy_out));
  return VTLB_OK;
}

VTLB_API int vtlb_copy_wait(vtlb_ctx* ctx, int what) {
  VTLB_ENTER(ctx);
  if (what & ~(VTLB_COPY_IN_BEFORE_COMPUTE | VTLB_COPY_OUT_BEFORE_COMPUTE | VTLB_COPY_OUT_DONE))
    return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_copy_wait: unknown bits 0x%x", what);
  if (what & VTLB_COPY_IN_BEFORE_COMPUTE) {
    VTLB_CUDA(ctx, cudaEventRecord(ctx->ev_copy, ctx->copy_in));
    VTLB_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->ev_copy, 0));
  }
  if (what & VTLB_COPY_OUT_BEFORE_COMPUTE) {
    VTLB_CUDA(ctx, cudaEventRecord(ctx->ev_copy, ctx->copy_out));
    VTLB_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->ev_copy, 0));
  }
  if (what & VTLB_COPY_OUT_DONE) VTLB_CUDA(ctx, cudaStreamSynchronize(ctx->copy_out));
  return VTLB_OK;
}

VTLB_API int vtlb_check_status(vtlb_ctx* ctx, uint32_t* status) {
  VTLB_ENTER(ctx);
  if (!status) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_check_status: null out");
  uint32_t st = 0;
  VTLB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  VTLB_CUDA(ctx, cudaMemcpy(&st, ctx->d_status, 4, cudaMemcpyDeviceToHost));
  if (st) VTLB_CUDA(ctx, cudaMemset(ctx->d_status, 0, 4));
  *status = st;
  if (st & VTLB_ST_GEMM_TIMEOUT)
    return vtlb_fail(ctx, VTLB_ETIMEOUT,
                     "a tcgen05 GEMM pipeline wait ran out (status 0x%x); its output is invalid",
                     st);
  return VTLB_OK;
}

VTLB_API uint64_t vtlb_launch_count(vtlb_ctx* ctx) { return ctx ? ctx->launches : 0; }
VTLB_API void* vtlb_stream(vtlb_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

VTLB_API int vtlb_profile_gemm(vtlb_ctx* ctx, int enable) {
  VTLB_ENTER(ctx);
  if (enable && !ctx->prof_ev) {
    ctx->prof_ev = new (std::nothrow) cudaEvent_t[2 * vtlb_ctx::kProfSlots]();
    if (!ctx->prof_ev) return vtlb_fail(ctx, VTLB_ENOMEM, "vtlb_profile_gemm: host allocation failed");
    ctx->prof_phase = new (std::nothrow) uint8_t[vtlb_ctx::kProfSlots]();
    if (!ctx->prof_phase) return vtlb_fail(ctx, VTLB_ENOMEM, "vtlb_profile_gemm: host allocation failed");
    for (int i = 0; i < 2 * vtlb_ctx::kProfSlots; ++i) VTLB_CUDA(ctx, cudaEventCreate(&ctx->prof_ev[i]));
  }
  ctx->prof_on = enable != 0;
  if (enable) {
    ctx->prof_n = 0;
    ctx->prof_flops = 0.0;
    memset(ctx->prof_phase, 0, vtlb_ctx::kProfSlots);
  }
  return VTLB_OK;
}

VTLB_API int vtlb_profile_read_phase(vtlb_ctx* ctx, int phase, double* total_ms, uint64_t* spans) {
  VTLB_ENTER(ctx);
  if (!total_ms || !spans) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_profile_read_phase: null out");
  if (phase < 0 || phase >= VTLB_PHASE_COUNT)
    return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_profile_read_phase: unknown phase %d", phase);
  *total_ms = 0.0;
  *spans = 0;
  if (!ctx->prof_ev) return VTLB_OK;
  VTLB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  for (int i = 0; i < ctx->prof_n; ++i) {
    if (ctx->prof_phase[i] != phase) continue;
    float t = 0.f;
    VTLB_CUDA(ctx, cudaEventElapsedTime(&t, ctx->prof_ev[2 * i], ctx->prof_ev[2 * i + 1]));
    *total_ms += t;
    ++*spans;
  }
  return VTLB_OK;
}

VTLB_API int vtlb_profile_gemm_read(vtlb_ctx* ctx, double* total_ms, uint64_t* launches, double* total_ops) {
  VTLB_ENTER(ctx);
  if (!total_ms || !launches || !total_ops) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_profile_gemm_read: null out");
  VTLB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  double ms = 0.0;
  uint64_t n = 0;
  for (int i = 0; i < ctx->prof_n; ++i) {
    if (ctx->prof_phase[i] != VTLB_PHASE_GEMM) continue;
    float t = 0.f;
    VTLB_CUDA(ctx, cudaEventElapsedTime(&t, ctx->prof_ev[2 * i], ctx->prof_ev[2 * i + 1]));
    ms += t;
    ++n;
  }
  *total_ms = ms;
  *launches = n;
  *total_ops = ctx->prof_flops;
  ctx->prof_n = 0;
  ctx->prof_flops = 0.0;
  memset(ctx->prof_phase, 0, vtlb_ctx::kProfSlots);
  return VTLB_OK;
}

VTLB_API int vtlb_event_create(vtlb_ctx* ctx, void** ev_out) {
  VTLB_ENTER(ctx);
  if (!ev_out) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_event_create: null out");
  cudaEvent_t ev;
  VTLB_CUDA(ctx, cudaEventCreate(&ev));
  *ev_out = (void*)ev;
  return VTLB_OK;
}
VTLB_API int vtlb_event_record(vtlb_ctx* ctx, void* ev) {
  VTLB_ENTER(ctx);
  if (!ev) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_event_record: null event");
  VTLB_CUDA(ctx, cudaEventRecord((cudaEvent_t)ev, ctx->stream));
  return VTLB_OK;
}
VTLB_API int vtlb_event_elapsed_ms(vtlb_ctx* ctx, void* ev_start, void* ev_stop, float* ms) {
  VTLB_ENTER(ctx);
  if (!ev_start || !ev_stop || !ms) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_event_elapsed_ms: null argument");
  VTLB_CUDA(ctx, cudaEventSynchronize((cudaEvent_t)ev_stop));
  VTLB_CUDA(ctx, cudaEventElapsedTime(ms, (cudaEvent_t)ev_start, (cudaEvent_t)ev_stop));
  return VTLB_OK;
}
VTLB_API int vtlb_event_destroy(vtlb_ctx* ctx, void* ev) {
  VTLB_ENTER(ctx);
  if (ev) VTLB_CUDA(ctx, cudaEventDestroy((cudaEvent_t)ev));
  return VTLB_OK;
}

// ---------------------------------------------------------------- memory

VTLB_API int vtlb_alloc(vtlb_ctx* ctx, size_t bytes, void** d_out) {
  VTLB_ENTER(ctx);
  if (!d_out) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_alloc: null out");
  *d_out = nullptr;
  if (bytes == 0) return VTLB_OK;
  const bool small = bytes <= vtlb_ctx::kCacheBlockMax;
  if (small) {
    bytes = vtlb_round_up(bytes, 256);
    auto it = ctx->small_free.find(bytes);
    if (it != ctx->small_free.end() && !it->second.empty()) {
      *d_out = it->second.back();
      it->second.pop_back();
      ctx->small_cached_bytes -= bytes;
      ctx->small_live.emplace(*d_out, bytes);
      return VTLB_OK;
    }
  }
  // Stream-ordered allocation from the device's pool: no device-wide synchronisation,
  // and freed blocks are reused by later allocations on the same stream.
  cudaError_t e = cudaMallocAsync(d_out, bytes, ctx->stream);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return vtlb_fail(ctx, VTLB_ENOMEM, "vtlb_alloc(%zu bytes): %s", bytes, cudaGetErrorString(e));
  }
  if (small)
    ctx->small_live.emplace(*d_out, bytes);
  else
    ctx->big_live.emplace(*d_out, bytes);
  return VTLB_OK;
}

VTLB_API int vtlb_free(vtlb_ctx* ctx, void* d_ptr) {
  VTLB_ENTER(ctx);
  if (!d_ptr) return VTLB_OK;
  // The free is ordered after the work already enqueued on the compute stream.  Only a block
  // that a collective still in flight on the communication stream reads or writes needs more:
  // the compute stream then waits for the communication stream first.  Every other free leaves
  // the two streams independent, so a gradient all-reduce keeps running beside backprop.
  auto it = ctx->small_live.find(d_ptr);
  if (!ctx->comm_inflight.empty()) {
    size_t bytes = 0;
    bool known = false;
    if (it != ctx->small_live.end()) {
      bytes = it->second;
      known = true;
    } else {
      auto bit = ctx->big_live.find(d_ptr);
      if (bit != ctx->big_live.end()) {
        bytes = bit->second;
        known = true;
      }
    }
    const uintptr_t b = (uintptr_t)d_ptr, e = b + bytes;
    bool hit = !known;  // a pointer this context did not hand out: be conservative
    for (size_t i = 0; i < ctx->comm_inflight.size() && !hit; ++i)
      hit = ctx->comm_inflight[i].first < e && b < ctx->comm_inflight[i].second;
    if (hit) {
      if (ctx->comm_small) {
        VTLB_CUDA(ctx, cudaEventRecord(ctx->ev_comm, ctx->comm_small_stream));
        VTLB_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->ev_comm, 0));
      }
      VTLB_CUDA(ctx, cudaEventRecord(ctx->ev_comm, ctx->comm_stream));
      VTLB_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->ev_comm, 0));
      ctx->comm_inflight.clear();
    }
  }
  ctx->big_live.erase(d_ptr);
  if (it != ctx->small_live.end()) {
    const size_t bytes = it->second;
    ctx->small_live.erase(it);
    if (ctx->small_cached_bytes + bytes <= vtlb_ctx::kCacheTotalMax) {
      // the next owner's work is enqueued on the same stream, after everything that used the block
      ctx->small_free[bytes].push_back(d_ptr);
      ctx->small_cached_bytes += bytes;
      return VTLB_OK;
    }
  }
  VTLB_CUDA(ctx, cudaFreeAsync(d_ptr, ctx->stream));
  return VTLB_OK;
}

VTLB_API int vtlb_h2d(vtlb_ctx* ctx, void* d_dst, const void* h_src, size_t bytes) {
  VTLB_ENTER(ctx);
  if (bytes == 0) return VTLB_OK;
  if (!d_dst || !h_src) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_h2d: null pointer");
  VTLB_CUDA(ctx, cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, ctx->stream));
  return VTLB_OK;
}

VTLB_API int vtlb_d2h(vtlb_ctx* ctx, void* h_dst, const void* d_src, size_t bytes) {
  VTLB_ENTER(ctx);
  if (bytes == 0) return VTLB_OK;
  if (!h_dst || !d_src) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_d2h: null pointer");
  VTLB_CUDA(ctx, cudaMemcpyAsync(h_dst, d_src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  VTLB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return VTLB_OK;
}

VTLB_API int vtlb_d2d(vtlb_ctx* ctx, void* d_dst, const void* d_src, size_t bytes) {
  VTLB_ENTER(ctx);
  if (bytes == 0) return VTLB_OK;
  if (!d_dst || !d_src) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_d2d: null pointer");
  VTLB_CUDA(ctx, cudaMemcpyAsync(d_dst, d_src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
  return VTLB_OK;
}

VTLB_API int vtlb_memset0(vtlb_ctx* ctx, void* d_dst, size_t bytes) {
  VTLB_ENTER(ctx);
  if (bytes == 0) return VTLB_OK;
  if (!d_dst) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_memset0: null pointer");
  VTLB_CUDA(ctx, cudaMemsetAsync(d_dst, 0, bytes, ctx->stream));
  return VTLB_OK;
}

VTLB_API int vtlb_host_alloc(size_t bytes, void** h_out) {
  if (!h_out) return vtlb_fail(nullptr, VTLB_EINVAL, "vtlb_host_alloc: null out");
  *h_out = nullptr;
  if (bytes == 0) return VTLB_OK;
  cudaError_t e = cudaMallocHost(h_out, bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return vtlb_fail(nullptr, VTLB_ENOMEM, "vtlb_host_alloc(%zu): %s", bytes,
                     cudaGetErrorString(e));
  }
  return VTLB_OK;
}

VTLB_API int vtlb_host_free(void* h_ptr) {
  if (!h_ptr) return VTLB_OK;
  cudaError_t e = cudaFreeHost(h_ptr);
  if (e != cudaSuccess)
    return vtlb_fail(nullptr, VTLB_ECUDA, "vtlb_host_free: %s", cudaGetErrorString(e));
  return VTLB_OK;
}

int vtlb_scratch(vtlb_ctx* ctx, size_t bytes, void** out) {
  if (bytes > ctx->scratch_bytes) {
    VTLB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (ctx->scratch) VTLB_CUDA(ctx, cudaFree(ctx->scratch));
    ctx->scratch = nullptr;
    ctx->scratch_bytes = 0;
    size_t want = vtlb_round_up(bytes + bytes / 8, (size_t)1 << 20);
    cudaError_t e = cudaMalloc(&ctx->scratch, want);
    if (e != cudaSuccess) {
      cudaGetLastError();
      want = vtlb_round_up(bytes, 256);
      e = cudaMalloc(&ctx->scratch, want);
    }
    if (e != cudaSuccess) {
      cudaGetLastError();
      return vtlb_fail(ctx, VTLB_ENOMEM, "scratch of %zu bytes: %s", bytes, cudaGetErrorString(e));
    }
    ctx->scratch_bytes = want;
  }
  *out = ctx->scratch;
  return VTLB_OK;
}

VTLB_API int vtlb_reserve_scratch(vtlb_ctx* ctx, size_t bytes) {
  VTLB_ENTER(ctx);
  void* p;
  return vtlb_scratch(ctx, bytes, &p);
}
