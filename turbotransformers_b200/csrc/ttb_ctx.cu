// Context, status word and the stream-ordered device pool behind the C ABI.
#include "ttb_common.cuh"

using namespace ttb;

extern "C" const char* ttb_version(void) { return "ttb-b200 0.1 (sm_100a)"; }

extern "C" int ttb_ctx_create(int device, void* cuda_stream, ttb_ctx** out) {
  if (!out) return TTB_ERR_INVALID;
  *out = nullptr;
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || device < 0 || device >= n) return TTB_ERR_CUDA;
  DeviceGuard g(device);
  ttb_ctx* c = new ttb_ctx();
  c->device = device;
  auto bail = [&](const char* what, cudaError_t e) {
    fprintf(stderr, "ttb_ctx_create: %s: %s\n", what, cudaGetErrorString(e));
    delete c;
    return (int)TTB_ERR_CUDA;
  };
  cudaError_t e;
  // NULL selects the legacy default stream: ordered with every blocking stream of the process, which is
  // what a caller that mixes these kernels with other libraries on "the default stream" expects.
  c->stream = cuda_stream ? static_cast<cudaStream_t>(cuda_stream) : cudaStreamLegacy;
  cudaMemPoolProps props = {};
  props.allocType = cudaMemAllocationTypePinned;
  props.handleTypes = cudaMemHandleTypeNone;
  props.location.type = cudaMemLocationTypeDevice;
  props.location.id = device;
  if ((e = cudaMemPoolCreate(&c->pool, &props)) != cudaSuccess) return bail("mempool", e);
  c->owns_pool = true;
  uint64_t keep = UINT64_MAX;  // freed blocks stay cached in the pool: steady state makes no driver calls
  cudaMemPoolSetAttribute(c->pool, cudaMemPoolAttrReleaseThreshold, &keep);
  // [0] the status word; [1], [2] the work counters of the attention kernel (zero between launches)
  if ((e = cudaMalloc(&c->d_status, 4 * sizeof(int))) != cudaSuccess) return bail("status word", e);
  if ((e = cudaMemset(c->d_status, 0, 4 * sizeof(int))) != cudaSuccess) return bail("status memset", e);
  if ((e = cudaMallocHost(&c->h_status, sizeof(int))) != cudaSuccess) return bail("pinned status", e);
  *c->h_status = 0;
  cudaDeviceGetAttribute(&c->sm_count, cudaDevAttrMultiProcessorCount, device);
  *out = c;
  return TTB_OK;
}

extern "C" int ttb_ctx_destroy(ttb_ctx* c) {
  if (!c) return TTB_ERR_INVALID;
  DeviceGuard g(c->device);
  cudaStreamSynchronize(c->stream);
  for (auto& kv : c->live) cudaFreeAsync(kv.first, c->stream);
  cudaStreamSynchronize(c->stream);
  for (auto& a : c->arenas) cudaFree(a.first);
  if (c->ln_ws) cudaFree(c->ln_ws);
  if (c->d_status) cudaFree(c->d_status);
  if (c->h_status) cudaFreeHost(c->h_status);
  if (c->owns_pool && c->pool) cudaMemPoolDestroy(c->pool);
  if (c->owns_stream && c->stream) cudaStreamDestroy(c->stream);
  delete c;
  return TTB_OK;
}

extern "C" int ttb_ctx_set_stream(ttb_ctx* c, void* s) {
  if (!c) return TTB_ERR_INVALID;
  if (c->owns_stream && c->stream) {
    DeviceGuard g(c->device);
    cudaStreamSynchronize(c->stream);
    cudaStreamDestroy(c->stream);
    c->owns_stream = false;
  }
  cudaStream_t next = s ? static_cast<cudaStream_t>(s) : cudaStreamLegacy;
  if (next != c->stream) {
    // Work already queued through this context (kernels, and the stream-ordered frees of its buffers) stays ahead of
    // whatever is queued next: the new stream waits for an event recorded on the old one. While either stream is being
    // captured into a graph the event cannot be recorded; the capture code orders its streams itself.
    DeviceGuard g(c->device);
    cudaStreamCaptureStatus a = cudaStreamCaptureStatusNone, b = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(c->stream, &a);
    cudaStreamIsCapturing(next, &b);
    cudaGetLastError();
    if (a == cudaStreamCaptureStatusNone && b == cudaStreamCaptureStatusNone) {
      cudaEvent_t ev = nullptr;
      if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) == cudaSuccess) {
        if (cudaEventRecord(ev, c->stream) == cudaSuccess) cudaStreamWaitEvent(next, ev, 0);
        cudaEventDestroy(ev);
      }
      cudaGetLastError();
    }
    c->stream = next;
  }
  return TTB_OK;
}

extern "C" void* ttb_ctx_stream(ttb_ctx* c) { return c ? (void*)c->stream : nullptr; }
extern "C" int ttb_ctx_device(ttb_ctx* c) { return c ? c->device : -1; }

extern "C" int ttb_ctx_sync(ttb_ctx* c) {
  if (!c) return TTB_ERR_INVALID;
  DeviceGuard g(c->device);
  TTB_CUDA(c, cudaStreamSynchronize(c->stream));
  return TTB_OK;
}

extern "C" const char* ttb_last_error(ttb_ctx* c) {
  if (!c) return "null context";
  return c->last_error.c_str();
}

extern "C" uint64_t ttb_launch_count(ttb_ctx* c) { return c ? c->launches.load() : 0; }

extern "C" int ttb_device_status(ttb_ctx* c) {
  if (!c) return TTB_ERR_INVALID;
  DeviceGuard g(c->device);
  TTB_CUDA(c, cudaMemcpyAsync(c->h_status, c->d_status, sizeof(int), cudaMemcpyDeviceToHost, c->stream));
  TTB_CUDA(c, cudaMemsetAsync(c->d_status, 0, sizeof(int), c->stream));
  TTB_CUDA(c, cudaStreamSynchronize(c->stream));
  int s = *c->h_status;
  if (s == TTB_ERR_DEVICE_WAIT) return fail(c, s, "a bounded device-side wait expired inside a kernel");
  if (s == TTB_ERR_BAD_INDEX) return fail(c, s, "an embedding id was outside its table (clamped)");
  if (s != 0) return fail(c, TTB_ERR_CUDA, "device status word holds %d", s);
  return TTB_OK;
}

extern "C" int ttb_memcpy_h2d(ttb_ctx* c, void* dst, const void* src, size_t bytes) {
  if (!c) return TTB_ERR_INVALID;
  if (bytes == 0) return TTB_OK;
  TTB_REQUIRE(c, dst && src, "memcpy_h2d: null pointer");
  DeviceGuard g(c->device);
  TTB_CUDA(c, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, c->stream));
  TTB_CUDA(c, cudaStreamSynchronize(c->stream));
  return TTB_OK;
}

extern "C" int ttb_memcpy_d2h(ttb_ctx* c, void* dst, const void* src, size_t bytes) {
  if (!c) return TTB_ERR_INVALID;
  if (bytes == 0) return TTB_OK;
  TTB_REQUIRE(c, dst && src, "memcpy_d2h: null pointer");
  DeviceGuard g(c->device);
  TTB_CUDA(c, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, c->stream));
  TTB_CUDA(c, cudaStreamSynchronize(c->stream));
  return TTB_OK;
}

extern "C" int ttb_copy_2d(ttb_ctx* c, void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width, size_t rows) {
  if (!c) return TTB_ERR_INVALID;
  if (width == 0 || rows == 0) return TTB_OK;
  TTB_REQUIRE(c, dst && src && dst_pitch >= width && src_pitch >= width, "copy_2d: bad arguments");
  DeviceGuard g(c->device);
  TTB_CUDA(c, cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width, rows, cudaMemcpyDeviceToDevice, c->stream));
  return TTB_OK;
}

// ---------------------------------------------------------------------------------------------
// pool
// ---------------------------------------------------------------------------------------------
extern "C" int ttb_alloc(ttb_ctx* c, size_t bytes, const char* name, void** out) {
  if (!c || !out) return TTB_ERR_INVALID;
  *out = nullptr;
  if (bytes == 0) return TTB_OK;
  {
    std::lock_guard<std::mutex> g(c->mu);
    c->bytes_allocated_total += bytes;
    if (c->arena_active) {  // fixed placement, no driver call: what a CUDA-graph capture of a forward pass needs
      const size_t off = (c->arena_off + 255) & ~(size_t)255;
      if (off + bytes > c->arena_size) {
        c->last_error = std::string("arena exhausted allocating '") + (name ? name : "") + "'";
        return TTB_ERR_OOM;
      }
      c->arena_off = off + bytes;
      if (c->arena_off > c->arena_peak) c->arena_peak = c->arena_off;
      c->n_allocs++;
      *out = c->arena + off;
      return TTB_OK;
    }
    if (c->limit && c->in_use + bytes > c->limit) {
      c->last_error = std::string("pool limit exceeded allocating '") + (name ? name : "") + "'";
      return TTB_ERR_OOM;
    }
  }
  DeviceGuard g(c->device);
  void* p = nullptr;
  cudaError_t e = cudaMallocFromPoolAsync(&p, bytes, c->pool, c->stream);
  if (e == cudaErrorMemoryAllocation) {
    // Same recovery the reference's caching allocator had (naive_allocator.h:50-63): drop cached blocks, retry once.
    cudaGetLastError();
    cudaStreamSynchronize(c->stream);
    cudaMemPoolTrimTo(c->pool, 0);
    e = cudaMallocFromPoolAsync(&p, bytes, c->pool, c->stream);
  }
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(c, e == cudaErrorMemoryAllocation ? TTB_ERR_OOM : TTB_ERR_CUDA, "allocating %zu bytes for '%s': %s",
                bytes, name ? name : "", cudaGetErrorString(e));
  }
  std::lock_guard<std::mutex> lk(c->mu);
  c->live[p] = bytes;
  c->in_use += bytes;
  if (c->in_use > c->high_water) c->high_water = c->in_use;
  c->n_allocs++;
  *out = p;
  return TTB_OK;
}

extern "C" int ttb_free(ttb_ctx* c, void* p, const char* /*name*/) {
  if (!c) return TTB_ERR_INVALID;
  if (!p) return TTB_OK;
  {
    std::lock_guard<std::mutex> lk(c->mu);
    for (auto& a : c->arenas)
      if (p >= (void*)a.first && p < (void*)(a.first + a.second)) return TTB_OK;  // arena memory is not recycled
    auto it = c->live.find(p);
    if (it == c->live.end()) {
      c->last_error = "ttb_free: pointer was not allocated by this context";
      return TTB_ERR_INVALID;
    }
    c->in_use -= it->second;
    c->live.erase(it);
  }
  DeviceGuard g(c->device);
  TTB_CUDA(c, cudaFreeAsync(p, c->stream));
  return TTB_OK;
}

extern "C" int ttb_arena_begin(ttb_ctx* c, size_t bytes) {
  if (!c) return TTB_ERR_INVALID;
  TTB_REQUIRE(c, bytes > 0, "arena_begin: zero size");
  TTB_REQUIRE(c, !c->arena_active, "arena_begin: an arena is already active");
  DeviceGuard g(c->device);
  // a buffer of its own for every begin: buffers of earlier arenas may be in use by graphs that were captured over them
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(c, e == cudaErrorMemoryAllocation ? TTB_ERR_OOM : TTB_ERR_CUDA, "reserving an arena of %zu bytes: %s", bytes, cudaGetErrorString(e));
  }
  std::lock_guard<std::mutex> lk(c->mu);
  c->arena = static_cast<char*>(p);
  c->arena_size = bytes;
  c->arenas.emplace_back(c->arena, bytes);
  c->arena_off = 0;
  c->arena_peak = 0;
  c->arena_active = true;
  return TTB_OK;
}

extern "C" int ttb_arena_end(ttb_ctx* c, size_t* bytes_used, void** arena_out) {
  if (!c) return TTB_ERR_INVALID;
  std::lock_guard<std::mutex> lk(c->mu);
  if (!c->arena_active) {
    c->last_error = "arena_end: no arena is active";
    return TTB_ERR_INVALID;
  }
  if (bytes_used) *bytes_used = c->arena_peak;
  if (arena_out) *arena_out = c->arena;
  c->arena_active = false;
  c->arena = nullptr;
  c->arena_size = 0;
  return TTB_OK;
}

extern "C" int ttb_arena_release(ttb_ctx* c, void* arena) {
  if (!c) return TTB_ERR_INVALID;
  if (!arena) return TTB_OK;
  {
    std::lock_guard<std::mutex> lk(c->mu);
    size_t i = 0;
    while (i < c->arenas.size() && c->arenas[i].first != arena) ++i;
    if (i == c->arenas.size()) {
      c->last_error = "arena_release: not an arena of this context";
      return TTB_ERR_INVALID;
    }
    if (c->arena_active && c->arena == arena) {
      c->last_error = "arena_release: the arena is active";
      return TTB_ERR_INVALID;
    }
    c->arenas.erase(c->arenas.begin() + (long)i);
  }
  DeviceGuard g(c->device);
  TTB_CUDA(c, cudaDeviceSynchronize());  // graphs replayed on any stream may still be using the buffer
  TTB_CUDA(c, cudaFree(arena));
  return TTB_OK;
}

extern "C" int ttb_bytes_allocated_total(ttb_ctx* c, uint64_t* bytes) {
  if (!c || !bytes) return TTB_ERR_INVALID;
  std::lock_guard<std::mutex> lk(c->mu);
  *bytes = c->bytes_allocated_total;
  return TTB_OK;
}

extern "C" int ttb_pool_stats(ttb_ctx* c, size_t* in_use, size_t* high_water, uint64_t* n_allocs) {
  if (!c) return TTB_ERR_INVALID;
  std::lock_guard<std::mutex> lk(c->mu);
  if (in_use) *in_use = c->in_use;
  if (high_water) *high_water = c->high_water;
  if (n_allocs) *n_allocs = c->n_allocs;
  return TTB_OK;
}

extern "C" int ttb_pool_set_limit(ttb_ctx* c, size_t bytes) {
  if (!c) return TTB_ERR_INVALID;
  std::lock_guard<std::mutex> lk(c->mu);
  c->limit = bytes;
  return TTB_OK;
}

// Activation bytes live at once in one encoder layer of the fused path, for `tokens` packed tokens:
// hidden in [T,H] + qkv [T,3H] + context [T,H] + attention out [T,H] + intermediate [T,F] + layer out [T,H],
// times the reference planner's 1.2 safety factor (model_aware_memory_scheduler.h:31-32). The arena is
// taken from the pool once and returned to it, so the pool holds that much memory from then on.
extern "C" int ttb_plan_activations(ttb_ctx* c, int64_t batch, int64_t tokens, int64_t heads, int64_t hidden,
                                    int64_t ffn, int64_t layers, int dtype, size_t* arena_bytes) {
  if (!c) return TTB_ERR_INVALID;
  TTB_REQUIRE(c, batch > 0 && tokens > 0 && heads > 0 && hidden > 0 && ffn > 0 && layers > 0, "plan: non-positive shape");
  size_t es = dtype_size(dtype);
  TTB_REQUIRE(c, es == 2 || es == 4, "plan: dtype must be F32/F16/BF16");
  size_t per_token = (size_t)(hidden * 7 + ffn) * es;
  size_t arena = (size_t)((double)tokens * (double)per_token * 1.2) + (size_t)(batch + 1) * 4 + (2u << 20);
  arena = (arena + (2u << 20) - 1) / (2u << 20) * (2u << 20);
  void* p = nullptr;
  int s = ttb_alloc(c, arena, "plan/arena", &p);
  if (s != TTB_OK) return s;
  s = ttb_free(c, p, "plan/arena");
  if (arena_bytes) *arena_bytes = arena;
  return s;
}
