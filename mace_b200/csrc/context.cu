// Runtime part of the C ABI: context creation, device and pinned-host memory,
// stream copies and synchronisation.  It plays the role that CpuRuntime and
// its allocator play for the CPU path (mace/runtimes/cpu/cpu_runtime.cc:28-109)
// for a CUDA device.
#include <atomic>
#include <cstdarg>
#include <cstdlib>

#include "common.cuh"

int mb_fail(mb_context *ctx, int code, const char *fmt, ...) {
  if (ctx != nullptr) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(ctx->last_error, sizeof(ctx->last_error), fmt, ap);
    va_end(ap);
  }
  return code;
}

int mb_check_cuda(mb_context *ctx, cudaError_t e, const char *what) {
  if (e == cudaSuccess) return MB_SUCCESS;
  const int code =
      (e == cudaErrorMemoryAllocation) ? MB_OUT_OF_RESOURCES : MB_RUNTIME_ERROR;
  return mb_fail(ctx, code, "%s: %s", what, cudaGetErrorString(e));
}

int mb_scratch(mb_context *ctx, size_t bytes, void **ptr) {
  if (bytes > ctx->scratch_bytes) {
    if (ctx->capturing)
      return mb_fail(ctx, MB_RUNTIME_ERROR,
                     "scratch arena would grow during graph capture; run the sequence once first");
    // Growing invalidates earlier carve-outs, so drain the stream first.
    MB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (ctx->scratch != nullptr) {
      MB_CUDA(ctx, cudaFree(ctx->scratch));
      ctx->scratch = nullptr;
      ctx->scratch_bytes = 0;
    }
    const size_t want = align_up(bytes + bytes / 4, 1 << 20);
    MB_CUDA(ctx, cudaMalloc(&ctx->scratch, want));
    ctx->scratch_bytes = want;
  }
  *ptr = ctx->scratch;
  return MB_SUCCESS;
}

extern "C" {

int mb_init(int device, mb_context **out) {
  if (out == nullptr) return MB_INVALID_ARGS;
  *out = nullptr;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 ||
      device >= count) {
    return MB_RUNTIME_ERROR;  // no CUDA device: there is no CPU fallback
  }
  mb_context *ctx = new mb_context();
  ctx->device = device;
  cudaDeviceProp prop;
  if (cudaSetDevice(device) != cudaSuccess ||
      cudaGetDeviceProperties(&prop, device) != cudaSuccess) {
    delete ctx;
    return MB_RUNTIME_ERROR;
  }
  if (prop.major != 10) {
    // The kernels are built for sm_100a only.
    delete ctx;
    return MB_UNSUPPORTED;
  }
  ctx->num_sms = prop.multiProcessorCount;
  ctx->max_smem_optin = static_cast<int>(prop.sharedMemPerBlockOptin);
  if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) !=
          cudaSuccess ||
      cudaMalloc(&ctx->dev_status, sizeof(int)) != cudaSuccess ||
      cudaMemset(ctx->dev_status, 0, sizeof(int)) != cudaSuccess ||
      cudaMallocHost(&ctx->host_status, sizeof(int)) != cudaSuccess) {
    delete ctx;
    return MB_RUNTIME_ERROR;
  }
  *ctx->host_status = 0;
  // The tensor-map encoder lives in the driver; resolve it at run time so the
  // library has no link-time dependency on libcuda.
  cudaDriverEntryPointQueryResult qres;
  void *fn = nullptr;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault,
                              &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess) {
    fn = nullptr;
  }
  ctx->encode_tiled = fn;
  *out = ctx;
  return MB_SUCCESS;
}

int mb_destroy(mb_context *ctx) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  cudaSetDevice(ctx->device);
  if (ctx->stream) cudaStreamSynchronize(ctx->stream);
  if (ctx->download_stream) {
    cudaStreamSynchronize(ctx->download_stream);
    cudaEventDestroy(ctx->download_event);
    cudaStreamDestroy(ctx->download_stream);
  }
  if (ctx->upload_stream) {
    cudaStreamSynchronize(ctx->upload_stream);
    cudaEventDestroy(ctx->upload_event);
    cudaStreamDestroy(ctx->upload_stream);
  }
  if (ctx->scratch) cudaFree(ctx->scratch);
  if (ctx->skinny_ws) cudaFree(ctx->skinny_ws);
  if (ctx->dev_status) cudaFree(ctx->dev_status);
  if (ctx->host_status) cudaFreeHost(ctx->host_status);
  if (ctx->stream) cudaStreamDestroy(ctx->stream);
  delete ctx;
  return MB_SUCCESS;
}

const char *mb_last_error(const mb_context *ctx) {
  return ctx ? ctx->last_error : "null context";
}

// ---- allocator fault injection ------------------------------------------------------------
// The reference's allocators fail at random when MACE_RUNTIME_FAILURE_RATIO is set
// (ShouldMockRuntimeFailure, mace/core/runtime_failure_mock.cc:25-53, called at the top of every
// allocator's New(), e.g. mace/runtimes/cpu/cpu_ref_allocator.cc:33), so that callers' handling
// of MACE_OUT_OF_RESOURCES can be exercised.  The same switch here: the ratio comes from the
// environment variable, read once, unless mb_set_runtime_failure_ratio has set it.
namespace {
std::atomic<float> g_failure_ratio{-1.f};   // < 0: not decided yet (read the environment)
std::atomic<uint64_t> g_failure_draws{0x9e3779b97f4a7c15ull};

float failure_ratio() {
  float r = g_failure_ratio.load();
  if (r < 0.f) {
    const char *env = getenv("MACE_RUNTIME_FAILURE_RATIO");
    r = env != nullptr ? static_cast<float>(atof(env)) : 0.f;
    if (!(r >= 0.f)) r = 0.f;
    g_failure_ratio.store(r);
  }
  return r;
}
}  // namespace

int mb_set_runtime_failure_ratio(float ratio) {
  if (!(ratio >= 0.f && ratio <= 1.f)) return MB_INVALID_ARGS;
  g_failure_ratio.store(ratio);
  return MB_SUCCESS;
}

int mb_should_mock_runtime_failure(void) {
  const float ratio = failure_ratio();
  if (!(ratio > 1e-6f)) return 0;
  // one draw of a 64-bit mixing generator per call; thread-safe through the atomic counter
  uint64_t z = g_failure_draws.fetch_add(0x9e3779b97f4a7c15ull);
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  z ^= z >> 31;
  const float u = static_cast<float>(z >> 40) * (1.0f / 16777216.0f);  // [0, 1)
  return u < ratio ? 1 : 0;
}

int mb_malloc(mb_context *ctx, size_t bytes, void **dptr) {
  if (ctx == nullptr || dptr == nullptr) return MB_INVALID_ARGS;
  *dptr = nullptr;
  if (bytes == 0) return MB_SUCCESS;
  if (mb_should_mock_runtime_failure())
    return mb_fail(ctx, MB_OUT_OF_RESOURCES, "mb_malloc: mock runtime failure (MACE_RUNTIME_FAILURE_RATIO)");
  MB_CUDA(ctx, cudaSetDevice(ctx->device));
  MB_CUDA(ctx, cudaMalloc(dptr, bytes));
  return MB_SUCCESS;
}

int mb_free(mb_context *ctx, void *dptr) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  if (dptr == nullptr) return MB_SUCCESS;
  MB_CUDA(ctx, cudaSetDevice(ctx->device));
  MB_CUDA(ctx, cudaFree(dptr));
  return MB_SUCCESS;
}

int mb_host_alloc(mb_context *ctx, size_t bytes, void **hptr) {
  if (ctx == nullptr || hptr == nullptr) return MB_INVALID_ARGS;
  *hptr = nullptr;
  if (bytes == 0) return MB_SUCCESS;
  MB_CUDA(ctx, cudaSetDevice(ctx->device));
  // host_alloc_wc: write-combined pinned memory -- for buffers the host only writes and the GPU
  // only reads (input staging): the copy engine reads them without snooping the CPU caches
  MB_CUDA(ctx, cudaHostAlloc(hptr, bytes, ctx->host_alloc_wc ? cudaHostAllocWriteCombined : cudaHostAllocDefault));
  return MB_SUCCESS;
}

int mb_host_free(mb_context *ctx, void *hptr) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  if (hptr == nullptr) return MB_SUCCESS;
  MB_CUDA(ctx, cudaFreeHost(hptr));
  return MB_SUCCESS;
}

int mb_memcpy_h2d(mb_context *ctx, void *dst, const void *src, size_t bytes) {
  if (ctx == nullptr || (bytes && (!dst || !src))) return MB_INVALID_ARGS;
  if (bytes == 0) return MB_SUCCESS;
  MB_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice,
                               ctx->stream));
  return MB_SUCCESS;
}

int mb_memcpy_d2h(mb_context *ctx, void *dst, const void *src, size_t bytes) {
  if (ctx == nullptr || (bytes && (!dst || !src))) return MB_INVALID_ARGS;
  if (bytes == 0) return MB_SUCCESS;
  MB_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost,
                               ctx->stream));
  return MB_SUCCESS;
}

int mb_memcpy_d2d(mb_context *ctx, void *dst, const void *src, size_t bytes) {
  if (ctx == nullptr || (bytes && (!dst || !src))) return MB_INVALID_ARGS;
  if (bytes == 0) return MB_SUCCESS;
  MB_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
  return MB_SUCCESS;
}

static int upload_stream_ready(mb_context *ctx) {
  if (ctx->upload_stream == nullptr) {
    MB_CUDA(ctx, cudaSetDevice(ctx->device));
    MB_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->upload_stream, cudaStreamNonBlocking));
    MB_CUDA(ctx, cudaEventCreateWithFlags(&ctx->upload_event, cudaEventDisableTiming));
  }
  return MB_SUCCESS;
}

int mb_upload_h2d(mb_context *ctx, void *dst, const void *src, size_t bytes) {
  if (ctx == nullptr || (bytes && (!dst || !src))) return MB_INVALID_ARGS;
  if (ctx->capturing) return mb_fail(ctx, MB_INVALID_ARGS, "mb_upload_h2d: not inside a graph capture");
  MB_RETURN_IF_ERROR(upload_stream_ready(ctx));
  if (bytes == 0) return MB_SUCCESS;
  MB_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->upload_stream));
  return MB_SUCCESS;
}

int mb_upload_wait_event(mb_context *ctx, void *event) {
  if (ctx == nullptr || event == nullptr) return MB_INVALID_ARGS;
  MB_RETURN_IF_ERROR(upload_stream_ready(ctx));
  MB_CUDA(ctx, cudaStreamWaitEvent(ctx->upload_stream, static_cast<cudaEvent_t>(event), 0));
  return MB_SUCCESS;
}

int mb_upload_signal(mb_context *ctx) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  if (ctx->capturing) return mb_fail(ctx, MB_INVALID_ARGS, "mb_upload_signal: not inside a graph capture");
  MB_RETURN_IF_ERROR(upload_stream_ready(ctx));
  MB_CUDA(ctx, cudaEventRecord(ctx->upload_event, ctx->upload_stream));
  MB_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->upload_event, 0));
  return MB_SUCCESS;
}

int mb_download_d2h(mb_context *ctx, void *dst, const void *src, size_t bytes, void *done_event) {
  if (ctx == nullptr || (bytes && (!dst || !src))) return MB_INVALID_ARGS;
  if (ctx->capturing) return mb_fail(ctx, MB_INVALID_ARGS, "mb_download_d2h: not inside a graph capture");
  if (ctx->download_stream == nullptr) {
    MB_CUDA(ctx, cudaSetDevice(ctx->device));
    MB_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->download_stream, cudaStreamNonBlocking));
    MB_CUDA(ctx, cudaEventCreateWithFlags(&ctx->download_event, cudaEventDisableTiming));
  }
  MB_CUDA(ctx, cudaEventRecord(ctx->download_event, ctx->stream));
  MB_CUDA(ctx, cudaStreamWaitEvent(ctx->download_stream, ctx->download_event, 0));
  if (bytes != 0) MB_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->download_stream));
  if (done_event != nullptr) MB_CUDA(ctx, cudaEventRecord(static_cast<cudaEvent_t>(done_event), ctx->download_stream));
  return MB_SUCCESS;
}

int mb_stream_wait_event(mb_context *ctx, void *event) {
  if (ctx == nullptr || event == nullptr) return MB_INVALID_ARGS;
  if (ctx->capturing) return mb_fail(ctx, MB_INVALID_ARGS, "mb_stream_wait_event: not inside a graph capture");
  MB_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, static_cast<cudaEvent_t>(event), 0));
  return MB_SUCCESS;
}

int mb_event_sync(mb_context *ctx, void *event) {
  if (ctx == nullptr || event == nullptr) return MB_INVALID_ARGS;
  MB_CUDA(ctx, cudaEventSynchronize(static_cast<cudaEvent_t>(event)));
  return MB_SUCCESS;
}

int mb_memset(mb_context *ctx, void *dst, int value, size_t bytes) {
  if (ctx == nullptr || (bytes && !dst)) return MB_INVALID_ARGS;
  if (bytes == 0) return MB_SUCCESS;
  MB_CUDA(ctx, cudaMemsetAsync(dst, value, bytes, ctx->stream));
  return MB_SUCCESS;
}

int mb_stream_sync(mb_context *ctx) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  MB_CUDA(ctx, cudaMemcpyAsync(ctx->host_status, ctx->dev_status, sizeof(int),
                               cudaMemcpyDeviceToHost, ctx->stream));
  MB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (*ctx->host_status != 0) {
    const int code = *ctx->host_status;
    *ctx->host_status = 0;
    cudaMemsetAsync(ctx->dev_status, 0, sizeof(int), ctx->stream);
    return mb_fail(ctx, MB_RUNTIME_ERROR,
                   "a kernel gave up a bounded wait (device status %d)", code);
  }
  return MB_SUCCESS;
}

int mb_event_create(mb_context *ctx, void **event) {
  if (ctx == nullptr || event == nullptr) return MB_INVALID_ARGS;
  cudaEvent_t e;
  MB_CUDA(ctx, cudaSetDevice(ctx->device));
  MB_CUDA(ctx, cudaEventCreate(&e));
  *event = e;
  return MB_SUCCESS;
}

int mb_event_record(mb_context *ctx, void *event) {
  if (ctx == nullptr || event == nullptr) return MB_INVALID_ARGS;
  // Inside a graph capture the record becomes an event-record NODE of the graph (the "external"
  // flag), so that replays of the graph stamp the event and the time between two such nodes can
  // be read after a replay has finished.
  MB_CUDA(ctx, cudaEventRecordWithFlags(static_cast<cudaEvent_t>(event), ctx->stream,
                                        ctx->capturing ? cudaEventRecordExternal : cudaEventRecordDefault));
  return MB_SUCCESS;
}

int mb_event_elapsed_ms(mb_context *ctx, void *start, void *stop, float *ms) {
  if (ctx == nullptr || start == nullptr || stop == nullptr || ms == nullptr)
    return MB_INVALID_ARGS;
  MB_CUDA(ctx, cudaEventSynchronize(static_cast<cudaEvent_t>(stop)));
  MB_CUDA(ctx, cudaEventElapsedTime(ms, static_cast<cudaEvent_t>(start),
                                    static_cast<cudaEvent_t>(stop)));
  return MB_SUCCESS;
}

int mb_event_destroy(mb_context *ctx, void *event) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  if (event != nullptr) MB_CUDA(ctx, cudaEventDestroy(static_cast<cudaEvent_t>(event)));
  return MB_SUCCESS;
}

// A captured sequence and the number of kernel launches one replay stands for.
struct mb_graph {
  cudaGraphExec_t exec = nullptr;
  uint64_t launches = 0, launches_tc = 0;
};

int mb_graph_begin(mb_context *ctx) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  if (ctx->capturing) return mb_fail(ctx, MB_INVALID_ARGS, "a capture is already in progress");
  MB_CUDA(ctx, cudaSetDevice(ctx->device));
  MB_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
  ctx->capturing = 1;
  ctx->capture_launches0 = ctx->launches;
  ctx->capture_launches_tc0 = ctx->launches_tc;
  return MB_SUCCESS;
}

int mb_graph_end(mb_context *ctx, void **graph_exec) {
  if (ctx == nullptr || graph_exec == nullptr) return MB_INVALID_ARGS;
  if (!ctx->capturing) return mb_fail(ctx, MB_INVALID_ARGS, "no capture in progress");
  ctx->capturing = 0;
  cudaGraph_t graph = nullptr;
  MB_CUDA(ctx, cudaStreamEndCapture(ctx->stream, &graph));
  cudaGraphExec_t exec = nullptr;
  cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  MB_CUDA(ctx, e);
  mb_graph *g = new mb_graph();
  g->exec = exec;
  // the launches counted during capture were recorded, not executed
  g->launches = ctx->launches - ctx->capture_launches0;
  g->launches_tc = ctx->launches_tc - ctx->capture_launches_tc0;
  ctx->launches = ctx->capture_launches0;
  ctx->launches_tc = ctx->capture_launches_tc0;
  *graph_exec = g;
  return MB_SUCCESS;
}

int mb_graph_launch(mb_context *ctx, void *graph_exec) {
  if (ctx == nullptr || graph_exec == nullptr) return MB_INVALID_ARGS;
  mb_graph *g = static_cast<mb_graph *>(graph_exec);
  MB_CUDA(ctx, cudaGraphLaunch(g->exec, ctx->stream));
  ctx->launches += g->launches;
  ctx->launches_tc += g->launches_tc;
  return MB_SUCCESS;
}

int mb_graph_destroy(mb_context *ctx, void *graph_exec) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  if (graph_exec != nullptr) {
    mb_graph *g = static_cast<mb_graph *>(graph_exec);
    cudaError_t e = cudaGraphExecDestroy(g->exec);
    delete g;
    MB_CUDA(ctx, e);
  }
  return MB_SUCCESS;
}

// Profiling aid, not part of the public header: give the tensor-core GEMM a
// device buffer of 32 long longs into which CTA 0 writes clock stamps of its
// pipeline milestones (null switches it off).
int mb_internal_set_tc_timeline(mb_context *ctx, long long *device_buffer) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  ctx->tc_timeline = device_buffer;
  return MB_SUCCESS;
}

void *mb_stream(mb_context *ctx) { return ctx ? ctx->stream : nullptr; }

uint64_t mb_launch_count(const mb_context *ctx) { return ctx ? ctx->launches : 0; }

uint64_t mb_launch_count_tensor_core(const mb_context *ctx) {
  return ctx ? ctx->launches_tc : 0;
}

uint64_t mb_launch_count_pair(const mb_context *ctx) { return ctx ? ctx->launches_pair : 0; }

int mb_pair_clusters(const mb_context *ctx) { return ctx ? ctx->max_pair_clusters : 0; }

int mb_set_option(mb_context *ctx, const char *name, int value) {
  if (ctx == nullptr || name == nullptr) return MB_INVALID_ARGS;
  if (strcmp(name, "tensor_cores") == 0) {
    ctx->use_tensor_cores = value;
  } else if (strcmp(name, "mn_major") == 0) {
    ctx->use_mn_major = value;
  } else if (strcmp(name, "host_alloc_wc") == 0) {
    ctx->host_alloc_wc = value;
  } else if (strcmp(name, "tc_rowsum") == 0) {
    ctx->tc_rowsum = value;
  } else if (strcmp(name, "dw_tma") == 0) {
    ctx->dw_tma = value;
  } else if (strcmp(name, "dw_waves") == 0) {
    if (value < 1) return mb_fail(ctx, MB_INVALID_ARGS, "dw_waves must be at least 1");
    ctx->dw_waves = value;
  } else if (strcmp(name, "skinny_max_m") == 0) {
    if (value < 0 || value > 16) return mb_fail(ctx, MB_INVALID_ARGS, "skinny_max_m must be 0 .. 16");
    ctx->skinny_max_m = value;
  } else if (strcmp(name, "stem_tc") == 0) {
    ctx->stem_tc = value;
  } else if (strcmp(name, "thin_pw") == 0) {
    ctx->thin_pw = value;
  } else if (strcmp(name, "dw_fixed_groups") == 0) {
    ctx->dw_fixed_groups = value;
  } else if (strcmp(name, "dw_lane_setup") == 0) {
    ctx->dw_lane_setup = value;
  } else if (strcmp(name, "b_prefetch") == 0) {
    ctx->b_prefetch = value;
  } else if (strcmp(name, "conv_filter_const") == 0) {
    ctx->conv_filter_const = value;
  } else if (strcmp(name, "stem_grid") == 0) {
    if (value < 1 || value > 16) return mb_fail(ctx, MB_INVALID_ARGS, "stem_grid: 1..16");
    ctx->stem_grid = value;
  } else if (strcmp(name, "dw_tma_fill") == 0) {
    if (value < 1 || value > 64) return mb_fail(ctx, MB_INVALID_ARGS, "dw_tma_fill: 1..64");
    ctx->dw_tma_fill = value;
  } else if (strcmp(name, "pair") == 0) {
    ctx->pair_gemm = value;
  } else if (strcmp(name, "runs_min_m") == 0) {
    ctx->runs_min_m = value;
  } else if (strcmp(name, "split_k") == 0) {
    ctx->split_k = value;
  } else if (strcmp(name, "gemv_stream") == 0) {
    ctx->gemv_stream = value;
  } else if (strcmp(name, "gemv_lhs_const") == 0) {
    ctx->gemv_lhs_const = value;
  } else if (strcmp(name, "gemv_chain_chunks") == 0) {
    ctx->gemv_chain_chunks = value;
  } else if (strcmp(name, "gemv_const_one_per_sm") == 0) {
    ctx->gemv_const_one_per_sm = value;
  } else if (strcmp(name, "force_bn") == 0) {
    if (value != 0 && value != 64 && value != 128 && value != 256)
      return mb_fail(ctx, MB_INVALID_ARGS, "force_bn must be 0, 64, 128 or 256");
    ctx->force_bn = value;
  } else if (strcmp(name, "pdl") == 0) {
    ctx->pdl_chain = value;
  } else if (strcmp(name, "wino_plane") == 0) {
    ctx->wino_plane = value;
  } else if (strcmp(name, "col_budget_mb") == 0) {
    if (value < 1) return mb_fail(ctx, MB_INVALID_ARGS, "col_budget_mb must be at least 1");
    ctx->col_budget_bytes = static_cast<int64_t>(value) << 20;
  } else {
    return mb_fail(ctx, MB_INVALID_ARGS, "unknown option %s", name);
  }
  return MB_SUCCESS;
}

}  // extern "C"
