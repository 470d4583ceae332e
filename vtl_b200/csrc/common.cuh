// Shared host-side plumbing of libvtlb200.so: the context object, error
// reporting and launch bookkeeping.  Nothing here is visible through the C ABI
// except the opaque vtlb_ctx pointer.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <unordered_map>
#include <utility>
#include <vector>

#include "../../include/vtlb.h"

#define VTLB_API extern "C" __attribute__((visibility("default")))

// Bits of the device status word (vtlb_check_status).
#define VTLB_ST_GEMM_TIMEOUT 0x1u  // a pipeline wait inside a tcgen05 GEMM ran out

struct vtlb_ctx {
  int device = 0;
  int sm_count = 0;
  cudaStream_t stream = nullptr;       // compute
  cudaStream_t comm_stream = nullptr;  // collectives
  cudaEvent_t ev_compute = nullptr;    // compute -> comm ordering
  cudaEvent_t ev_comm = nullptr;       // comm -> compute ordering
  // input pipeline: host -> device and device -> host copies on streams of their own, so that the
  // next batch comes in and the last result goes out while the current step computes
  cudaStream_t copy_in = nullptr, copy_out = nullptr;
  cudaEvent_t ev_copy = nullptr;       // ordering between the copy streams and compute
  uint32_t* d_status = nullptr;        // device status word
  void* scratch = nullptr;             // operand-split buffers, partial sums
  size_t scratch_bytes = 0;
  // INT8 pair GEMM, K-split tiles: flags + parked accumulators (kKsplitBytes, allocated with the
  // context so that no launch ever allocates); every launch that splits stamps its flags with a
  // fresh epoch, so nothing is ever reset.
  static constexpr size_t kKsplitTiles = 64;  // cut tiles per launch at most (half of the CTA pairs)
  static constexpr size_t kKsplitFlagBytes = kKsplitTiles * 2 * 8 * 4;       // [tile][rank][epilogue warp]
  static constexpr size_t kKsplitBytes = kKsplitFlagBytes + kKsplitTiles * 256 * 256 * 4;
  void* ksplit_buf = nullptr;
  uint32_t ksplit_epoch = 0;
  // Small blocks (<= kCacheBlockMax) are recycled by the context itself: a training step of a small
  // model makes dozens of sub-megabyte allocations, and a pool call per tensor costs more host time
  // than the kernels that use it take to run.  Blocks are reused in stream order, like the pool's.
  static constexpr size_t kCacheBlockMax = 1u << 20, kCacheTotalMax = 256u << 20;
  std::unordered_map<void*, size_t> small_live;                 // block -> rounded size
  std::unordered_map<size_t, std::vector<void*>> small_free;    // rounded size -> free blocks
  size_t small_cached_bytes = 0;
  void* comm = nullptr;  // ncclComm_t
  int nranks = 1, rank = 0;
  // A second communicator (split off the first) on a stream of its own carries the small,
  // latency-critical collectives (the max all-reduce of row maxima), so that they do not queue
  // behind a bulk all-gather or gradient all-reduce still running on the first.  Null when the
  // NCCL at hand cannot split communicators: both lanes then share the first.
  void* comm_small = nullptr;
  cudaStream_t comm_small_stream = nullptr;
  // Marks: events recorded behind the collectives enqueued so far on one lane, for which the compute
  // stream can wait individually (vtlb_comm_mark / vtlb_comm_wait_mark).
  float* comm_barrier_word = nullptr;  // one word all-reduced behind pushed copies (vtlb_allgather_push_async)
  static constexpr int kCommMarks = 64;
  cudaEvent_t comm_marks[kCommMarks] = {};
  // Byte ranges handed to collectives on the communication stream since the compute stream last
  // waited for it.  Freeing (or recycling) a block that overlaps one of them must first order the
  // compute stream after the communication stream; every other free needs no such wait, which is
  // what lets a gradient all-reduce run beside the rest of backprop.
  std::vector<std::pair<uintptr_t, uintptr_t>> comm_inflight;  // [begin, end)
  std::unordered_map<void*, size_t> big_live;                  // blocks above kCacheBlockMax -> bytes
  uint64_t launches = 0;
  // f32 GEMMs of at most this many flops (2*M*N*K) run on the CUDA-core kernel of
  // f32_small.cu instead of the tensor-core path (vtlb_set_small_gemm_limit; 0 = never).
  double small_gemm_flops = 1.4e8;
  // Optional timing of the tensor-core GEMM launches (vtlb_profile_gemm): a ring of event
  // pairs recorded around each launch plus the algorithmic work of the launches timed.
  bool prof_on = false;
  static constexpr int kProfSlots = 2048;
  cudaEvent_t* prof_ev = nullptr;  // 2 * kProfSlots events, created on first enable
  uint8_t* prof_phase = nullptr;   // phase of each slot (VTLB_PHASE_*; the GEMM launch sites leave 0)
  int prof_n = 0;
  double prof_flops = 0.0;
  char err[512] = {0};
};

extern thread_local char g_vtlb_err[512];

int vtlb_fail(vtlb_ctx* ctx, int code, const char* fmt, ...);

// Makes ctx's device current; every entry point starts with it.
#define VTLB_ENTER(ctx)                                                         \
  do {                                                                          \
    if (!(ctx)) return vtlb_fail(nullptr, VTLB_EINVAL, "%s: null ctx", __func__); \
    cudaError_t e__ = cudaSetDevice((ctx)->device);                             \
    if (e__ != cudaSuccess)                                                     \
      return vtlb_fail((ctx), VTLB_ECUDA, "%s: cudaSetDevice(%d): %s", __func__, \
                       (ctx)->device, cudaGetErrorString(e__));                 \
  } while (0)

#define VTLB_CUDA(ctx, call)                                                          \
  do {                                                                                \
    cudaError_t e__ = (call);                                                         \
    if (e__ != cudaSuccess)                                                           \
      return vtlb_fail((ctx), VTLB_ECUDA, "%s: %s -> %s", __func__, #call,            \
                       cudaGetErrorString(e__));                                      \
  } while (0)

// After a kernel launch: count it and surface launch-configuration errors.
#define VTLB_LAUNCHED(ctx)                                                            \
  do {                                                                                \
    (ctx)->launches++;                                                                \
    cudaError_t e__ = cudaGetLastError();                                             \
    if (e__ != cudaSuccess)                                                           \
      return vtlb_fail((ctx), VTLB_ECUDA, "%s: kernel launch: %s", __func__,          \
                       cudaGetErrorString(e__));                                      \
  } while (0)

// Brackets the launches of its scope with one event pair of the timing ring, filed under `phase`
// (include/vtlb.h: VTLB_PHASE_*), while vtlb_profile_gemm is enabled; free otherwise.
struct vtlb_prof_scope {
  vtlb_ctx* ctx;
  int slot;
  vtlb_prof_scope(vtlb_ctx* c, int phase) : ctx(c), slot(-1) {
    if (c->prof_on && c->prof_ev && c->prof_n < vtlb_ctx::kProfSlots) {
      slot = c->prof_n++;
      c->prof_phase[slot] = (uint8_t)phase;
      cudaEventRecord(c->prof_ev[2 * slot], c->stream);
    }
  }
  ~vtlb_prof_scope() {
    if (slot >= 0) cudaEventRecord(ctx->prof_ev[2 * slot + 1], ctx->stream);
  }
  vtlb_prof_scope(const vtlb_prof_scope&) = delete;
  vtlb_prof_scope& operator=(const vtlb_prof_scope&) = delete;
};

// Notes that a collective enqueued on the communication stream reads or writes [p, p + bytes).
inline void vtlb_comm_track(vtlb_ctx* ctx, const void* p, size_t bytes) {
  if (!p || !bytes) return;
  auto& v = ctx->comm_inflight;
  if (v.size() >= 1024) {  // a caller that never waits: fold the list into its bounding range
    uintptr_t lo = v[0].first, hi = v[0].second;
    for (const auto& r : v) {
      lo = r.first < lo ? r.first : lo;
      hi = r.second > hi ? r.second : hi;
    }
    v.assign(1, std::make_pair(lo, hi));
  }
  v.emplace_back((uintptr_t)p, (uintptr_t)p + bytes);
}

// Returns a scratch region of at least `bytes` (grown on demand; growth
// synchronises the stream first because earlier kernels may still use the old one).
int vtlb_scratch(vtlb_ctx* ctx, size_t bytes, void** out);

// Launch with programmatic stream serialisation: the kernel's CTAs may become resident while
// the kernel in front of it in the stream is still finishing, which hides the launch latency
// of short dependent kernels.  Only for kernels that execute griddepcontrol.wait before their
// first access to memory (the wait returns once the kernel in front has completed and its
// writes are visible).  VTLB_EARLY_LAUNCH=0 turns the attribute off (measurements).
template <typename... KArgs, typename... Args>
static inline cudaError_t vtlb_launch_early(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                            cudaStream_t stream, Args&&... args) {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("VTLB_EARLY_LAUNCH");
    on = e ? atoi(e) != 0 : 1;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = on ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<Args&&>(args)...);
}

static inline bool vtlb_aligned16(const void* p) { return (((uintptr_t)p) & 15u) == 0; }
static inline size_t vtlb_round_up(size_t x, size_t m) { return (x + m - 1) / m * m; }
