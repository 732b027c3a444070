// Context lifetime, scratch buffer, error string, seeded synthetic-input generators.
#include <math.h>
#include <stdio.h>
#include <string.h>

#include <mutex>
#include <unordered_map>
#include <vector>

#include "common.cuh"

static thread_local std::string g_last_error;
void talos_set_last_error(const std::string& msg) { g_last_error = msg; }

TALOS_API const char* talos_last_error_string(void) { return g_last_error.c_str(); }

static void* grow_scratch(talos_ctx* ctx, void** buf, size_t* have, size_t bytes) {
  if (bytes <= *have) return *buf;
  size_t want = bytes + (bytes >> 2);
  want = (want + 255) & ~size_t(255);
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, want);
  if (e != cudaSuccess) { cudaGetLastError(); throw talos_error(TALOS_ERR_ALLOC, "workspace cudaMalloc failed"); }
  if (*buf) { TALOS_CHECK_CUDA(cudaStreamSynchronize(ctx->stream)); cudaFree(*buf); }
  *buf = p; *have = want;
  return p;
}
void* talos_workspace(talos_ctx* ctx, size_t bytes) { return grow_scratch(ctx, &ctx->ws, &ctx->ws_bytes, bytes); }
void* talos_workspace2(talos_ctx* ctx, size_t bytes) { return grow_scratch(ctx, &ctx->ws2, &ctx->ws2_bytes, bytes); }

// ---- caching device allocator -----------------------------------------------------------------------------------
// The reference allocates a fresh result (and a fresh gradient buffer) for every op (src/autograd.rs:94-107), so the
// host mirror above this ABI asks for device memory thousands of times per training step.  cudaMalloc / cudaFree cost
// tens of microseconds and cudaFree synchronises the device; blocks are therefore kept per context in free lists by
// size class and handed out again without touching the driver.  A block freed by the host may still be read by work
// already enqueued, and is only ever handed to work enqueued LATER on the same stream (one ctx = one stream), so reuse
// needs no synchronisation.  Size classes: powers of two up to 1 MiB, then multiples of 1 MiB.
struct talos_pool {
  std::mutex mu;
  std::unordered_map<size_t, std::vector<void*>> free_lists;       // class size -> idle blocks
  std::unordered_map<void*, size_t> live;                          // block -> class size
  size_t cached_bytes = 0, live_bytes = 0;
  int64_t driver_allocs = 0, reuses = 0;
  static size_t size_class(size_t bytes) {
    if (bytes <= 256) return 256;
    if (bytes <= (size_t(1) << 20)) { size_t c = 256; while (c < bytes) c <<= 1; return c; }
    return (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
  }
};

// Returns every idle block to the driver (after the stream has drained: an idle block may still be read by queued work).
static void pool_trim(talos_ctx* ctx) {
  talos_pool* pl = ctx->pool;
  if (!pl || pl->cached_bytes == 0) return;
  cudaStreamSynchronize(ctx->stream);
  for (auto& kv : pl->free_lists) { for (void* p : kv.second) cudaFree(p); kv.second.clear(); }
  pl->cached_bytes = 0;
}

void talos_sync_and_check(talos_ctx* ctx) {
  // the status word rides along with the wait the caller needs anyway: one 4-byte copy enqueued before the sync
  TALOS_CHECK_CUDA(cudaMemcpyAsync(ctx->host_status, ctx->dev_status, sizeof(int32_t), cudaMemcpyDeviceToHost, ctx->stream));
  TALOS_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));
  const int32_t st = *ctx->host_status;
  if (st != 0) {
    *ctx->host_status = 0;
    TALOS_CHECK_CUDA(cudaMemsetAsync(ctx->dev_status, 0, 64, ctx->stream));
    if (st >= TALOS_DEV_BAD_INDEX)
      throw talos_error(TALOS_ERR_ARG, "an index read from device memory was out of range (an action outside [0, n_actions)); the kernel skipped it (status " + std::to_string(st) + ")");
    throw talos_error(TALOS_ERR_TIMEOUT, "a bounded device-side wait gave up (status " + std::to_string(st) + ")");
  }
}

TALOS_API talos_status talos_ctx_create(int32_t device, void* stream, talos_ctx** out) {
  TALOS_ENTRY_BEGIN
  TALOS_REQUIRE(out != nullptr, TALOS_ERR_ARG, "null out pointer");
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0) { cudaGetLastError(); throw talos_error(TALOS_ERR_CUDA, "no CUDA device: this library has no CPU path"); }
  TALOS_REQUIRE(device >= 0 && device < count, TALOS_ERR_ARG, "device index out of range");
  TALOS_CHECK_CUDA(cudaSetDevice(device));
  cudaDeviceProp prop;
  TALOS_CHECK_CUDA(cudaGetDeviceProperties(&prop, device));
  TALOS_REQUIRE(prop.major == 10, TALOS_ERR_UNSUPPORTED, "this library is built for sm_100a (B200) only");
  talos_ctx* c = new talos_ctx();
  c->device = device; c->sm_count = prop.multiProcessorCount;
  c->stream = (cudaStream_t)stream; c->own_stream = false;     // NULL is the device's default stream
  TALOS_CHECK_CUDA(cudaMalloc(&c->dev_status, 64));
  TALOS_CHECK_CUDA(cudaMemset(c->dev_status, 0, 64));
  TALOS_CHECK_CUDA(cudaMallocHost(&c->host_status, 64));
  memset(c->host_status, 0, 64);
  c->pool = new talos_pool();
  talos_colsum_noalloc_prepare(device);     // resolve the fixed scratch array's address now, not inside a trainer thread's first call
  *out = c;
  TALOS_ENTRY_END
}

static void timeline_destroy(talos_timeline* t);
TALOS_API talos_status talos_ctx_destroy(talos_ctx* ctx) {
  TALOS_ENTRY_BEGIN
  if (!ctx) return TALOS_OK;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  timeline_destroy(ctx->timeline);
  if (ctx->pool) {
    pool_trim(ctx);
    for (auto& kv : ctx->pool->live) cudaFree(kv.first);          // blocks the host never returned
    delete ctx->pool;
  }
  if (ctx->host_status) cudaFreeHost(ctx->host_status);
  if (ctx->ws) cudaFree(ctx->ws);
  if (ctx->ws2) cudaFree(ctx->ws2);
  if (ctx->dev_status) cudaFree(ctx->dev_status);
  if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
  delete ctx;
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_ctx_synchronize(talos_ctx* ctx) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  talos_sync_and_check(ctx);
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_debug_set_device_status(talos_ctx* ctx, int32_t code) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_CHECK_CUDA(cudaMemcpyAsync(ctx->dev_status, &code, sizeof(code), cudaMemcpyHostToDevice, ctx->stream));
  TALOS_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_debug_gemm_stall(talos_ctx* ctx, int32_t skip_k_block, uint32_t wait_spins) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(skip_k_block >= -1 && (wait_spins == 0 || wait_spins >= 1024), TALOS_ERR_ARG, "bad stall parameters");
  ctx->dbg_skip_kb = skip_k_block; ctx->dbg_wait_spins = wait_spins;
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_ctx_set_stream(talos_ctx* ctx, void* stream) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));
  if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
  ctx->stream = (cudaStream_t)stream; ctx->own_stream = false;
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_ctx_reserve_workspace(talos_ctx* ctx, size_t bytes) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  talos_workspace(ctx, bytes);
  talos_workspace2(ctx, bytes);
  TALOS_ENTRY_END
}

TALOS_API int32_t talos_ctx_tensor_cores_active(talos_ctx* ctx) { return ctx && ctx->tc_state == 1 ? 1 : 0; }
TALOS_API int32_t talos_ctx_tensor_cores_state(talos_ctx* ctx) { return ctx ? ctx->tc_state : 0; }
TALOS_API int64_t talos_ctx_launch_count(talos_ctx* ctx) { return ctx ? ctx->launches.load() : 0; }

// ---- device memory for hosts that bind only this ABI ----
TALOS_API talos_status talos_malloc(talos_ctx* ctx, size_t bytes, void** out) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(out != nullptr, TALOS_ERR_ARG, "null out pointer");
  *out = nullptr;
  if (bytes == 0) return TALOS_OK;
  talos_pool* pl = ctx->pool;
  const size_t cls = talos_pool::size_class(bytes);
  std::lock_guard<std::mutex> lock(pl->mu);
  auto it = pl->free_lists.find(cls);
  void* p = nullptr;
  if (it != pl->free_lists.end() && !it->second.empty()) {
    p = it->second.back(); it->second.pop_back(); pl->cached_bytes -= cls; pl->reuses += 1;
  } else {
    cudaError_t e = cudaMalloc(&p, cls);
    if (e != cudaSuccess) {                                         // give the idle blocks back to the driver and try once more
      cudaGetLastError(); pool_trim(ctx);
      e = cudaMalloc(&p, cls);
      if (e != cudaSuccess) { cudaGetLastError(); throw talos_error(TALOS_ERR_ALLOC, "device allocation failed"); }
    }
    pl->driver_allocs += 1;
  }
  pl->live[p] = cls; pl->live_bytes += cls;
  *out = p;
  TALOS_ENTRY_END
}
TALOS_API talos_status talos_free(talos_ctx* ctx, void* ptr) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  if (!ptr) return TALOS_OK;
  talos_pool* pl = ctx->pool;
  std::lock_guard<std::mutex> lock(pl->mu);
  auto it = pl->live.find(ptr);
  TALOS_REQUIRE(it != pl->live.end(), TALOS_ERR_ARG, "talos_free: pointer was not returned by talos_malloc on this context");
  const size_t cls = it->second;
  pl->live.erase(it); pl->live_bytes -= cls;
  pl->free_lists[cls].push_back(ptr); pl->cached_bytes += cls;
  TALOS_ENTRY_END
}
TALOS_API talos_status talos_ctx_trim(talos_ctx* ctx) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  std::lock_guard<std::mutex> lock(ctx->pool->mu);
  pool_trim(ctx);
  TALOS_ENTRY_END
}
TALOS_API talos_status talos_ctx_memory_stats(talos_ctx* ctx, int64_t* stats4) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(stats4 != nullptr, TALOS_ERR_ARG, "null pointer");
  std::lock_guard<std::mutex> lock(ctx->pool->mu);
  stats4[0] = (int64_t)ctx->pool->live_bytes; stats4[1] = (int64_t)ctx->pool->cached_bytes;
  stats4[2] = ctx->pool->driver_allocs; stats4[3] = ctx->pool->reuses;
  TALOS_ENTRY_END
}
// ---- launch timeline (measurement aid): while recording, every launch is followed by an event on the ctx stream ----
struct talos_timeline {
  static constexpr int MAX_MARKS = 512;
  cudaEvent_t start = nullptr;
  std::vector<cudaEvent_t> events;       // created once, reused
  std::vector<const char*> names;        // string literals passed to talos_launched
  int used = 0;
};
void talos_timeline_mark(talos_ctx* ctx, const char* what) {
  talos_timeline* t = ctx->timeline;
  if (!t || t->used >= talos_timeline::MAX_MARKS) return;
  if ((int)t->events.size() <= t->used) { cudaEvent_t e; if (cudaEventCreate(&e) != cudaSuccess) { cudaGetLastError(); return; } t->events.push_back(e); t->names.push_back(what); }
  t->names[t->used] = what;
  cudaEventRecord(t->events[t->used], ctx->stream);
  t->used += 1;
}
static void timeline_destroy(talos_timeline* t) {
  if (!t) return;
  for (cudaEvent_t e : t->events) cudaEventDestroy(e);
  if (t->start) cudaEventDestroy(t->start);
  delete t;
}
TALOS_API talos_status talos_ctx_timeline_begin(talos_ctx* ctx) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  if (!ctx->timeline) { ctx->timeline = new talos_timeline(); TALOS_CHECK_CUDA(cudaEventCreate(&ctx->timeline->start)); }
  ctx->timeline->used = 0;
  TALOS_CHECK_CUDA(cudaEventRecord(ctx->timeline->start, ctx->stream));
  TALOS_ENTRY_END
}
TALOS_API talos_status talos_ctx_timeline_end(talos_ctx* ctx, int32_t capacity, int32_t* count_out, float* us_out, char* names_out, int32_t name_stride) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(count_out != nullptr && capacity >= 0 && (capacity == 0 || (us_out && names_out && name_stride > 1)), TALOS_ERR_ARG, "bad timeline buffers");
  talos_timeline* t = ctx->timeline;
  TALOS_REQUIRE(t != nullptr, TALOS_ERR_ARG, "no timeline is being recorded");
  talos_sync_and_check(ctx);
  const int n = std::min<int>(t->used, capacity);
  for (int i = 0; i < n; ++i) {
    float ms = 0.f;
    TALOS_CHECK_CUDA(cudaEventElapsedTime(&ms, i ? t->events[i - 1] : t->start, t->events[i]));
    us_out[i] = ms * 1000.f;
    snprintf(names_out + (size_t)i * name_stride, (size_t)name_stride, "%s", t->names[i]);
  }
  *count_out = t->used;
  timeline_destroy(t); ctx->timeline = nullptr;
  TALOS_ENTRY_END
}

TALOS_API talos_status talos_memset_zero(talos_ctx* ctx, void* ptr, size_t bytes) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  if (bytes) { TALOS_REQUIRE(ptr != nullptr, TALOS_ERR_ARG, "null pointer"); TALOS_CHECK_CUDA(cudaMemsetAsync(ptr, 0, bytes, ctx->stream)); }
  TALOS_ENTRY_END
}
TALOS_API talos_status talos_copy_from_host(talos_ctx* ctx, void* dst, const void* src, size_t bytes) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  if (bytes) {
    TALOS_REQUIRE(dst && src, TALOS_ERR_ARG, "null pointer");
    TALOS_CHECK_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    TALOS_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));
  }
  TALOS_ENTRY_END
}
TALOS_API talos_status talos_copy_to_host(talos_ctx* ctx, void* dst, const void* src, size_t bytes) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  if (bytes) {
    TALOS_REQUIRE(dst && src, TALOS_ERR_ARG, "null pointer");
    TALOS_CHECK_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    talos_sync_and_check(ctx);
  }
  TALOS_ENTRY_END
}
TALOS_API talos_status talos_copy_device(talos_ctx* ctx, void* dst, const void* src, size_t bytes) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  if (bytes) {
    TALOS_REQUIRE(dst && src, TALOS_ERR_ARG, "null pointer");
    TALOS_CHECK_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
  }
  TALOS_ENTRY_END
}
TALOS_API talos_status talos_upload_f64(talos_ctx* ctx, float* dst, const double* src, int64_t n) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(n >= 0 && ((dst && src) || n == 0), TALOS_ERR_ARG, "null pointer");
  if (n == 0) return TALOS_OK;
  std::string buf(sizeof(float) * (size_t)n, '\0');
  float* f = (float*)&buf[0];
  for (int64_t i = 0; i < n; ++i) f[i] = (float)src[i];
  TALOS_CHECK_CUDA(cudaMemcpyAsync(dst, f, sizeof(float) * (size_t)n, cudaMemcpyHostToDevice, ctx->stream));
  TALOS_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));
  TALOS_ENTRY_END
}
TALOS_API talos_status talos_download_f64(talos_ctx* ctx, double* dst, const float* src, int64_t n) {
  TALOS_ENTRY_BEGIN
  talos_check_ctx(ctx);
  TALOS_REQUIRE(n >= 0 && ((dst && src) || n == 0), TALOS_ERR_ARG, "null pointer");
  if (n == 0) return TALOS_OK;
  std::string buf(sizeof(float) * (size_t)n, '\0');
  float* f = (float*)&buf[0];
  TALOS_CHECK_CUDA(cudaMemcpyAsync(f, src, sizeof(float) * (size_t)n, cudaMemcpyDeviceToHost, ctx->stream));
  talos_sync_and_check(ctx);
  for (int64_t i = 0; i < n; ++i) dst[i] = (double)f[i];
  TALOS_ENTRY_END
}

// ---- src/rng.rs:14-117 restated: SplitMix64 seeding, xoshiro256**, 53-bit uniform, Box-Muller z0 ----
namespace {
struct Xoshiro {
  uint64_t s[4];
  explicit Xoshiro(uint64_t seed) {
    for (int i = 0; i < 4; ++i) {
      seed += 0x9e3779b97f4a7c15ULL; uint64_t z = seed;
      z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ULL; z = (z ^ (z >> 27)) * 0x94d049bb133111ebULL; s[i] = z ^ (z >> 31);
    }
  }
  static uint64_t rotl(uint64_t x, int k) { return (x << k) | (x >> (64 - k)); }
  uint64_t next() {
    uint64_t r = rotl(s[1] * 5, 7) * 9, t = s[1] << 17;
    s[2] ^= s[0]; s[3] ^= s[1]; s[1] ^= s[2]; s[0] ^= s[3]; s[2] ^= t; s[3] = rotl(s[3], 45); return r;
  }
  double f64() { return (double)(next() >> 11) * (1.0 / 9007199254740992.0); }
};
}  // namespace

TALOS_API talos_status talos_rng_uniform_host(uint64_t seed, float lo, float hi, float* out, int64_t n) {
  TALOS_ENTRY_BEGIN
  TALOS_REQUIRE(out || n == 0, TALOS_ERR_ARG, "null output");
  Xoshiro r(seed);
  for (int64_t i = 0; i < n; ++i) out[i] = (float)((double)lo + ((double)hi - (double)lo) * r.f64());
  TALOS_ENTRY_END
}
TALOS_API talos_status talos_rng_normal_host(uint64_t seed, float mean, float std, float* out, int64_t n) {
  TALOS_ENTRY_BEGIN
  TALOS_REQUIRE(out || n == 0, TALOS_ERR_ARG, "null output");
  Xoshiro r(seed);
  for (int64_t i = 0; i < n; ++i) {
    double u1; do { u1 = r.f64(); } while (!(u1 > 0.0));
    double u2 = r.f64();
    out[i] = (float)((double)mean + (double)std * (sqrt(-2.0 * log(u1)) * cos(2.0 * M_PI * u2)));
  }
  TALOS_ENTRY_END
}
TALOS_API talos_status talos_rng_bounded_host(uint64_t seed, uint32_t range, int32_t* out, int64_t n) {
  TALOS_ENTRY_BEGIN
  TALOS_REQUIRE(range > 0 && (out || n == 0), TALOS_ERR_ARG, "bad range or null output");
  Xoshiro r(seed);
  uint64_t rg = range, threshold = (0ULL - rg) % rg;
  for (int64_t i = 0; i < n; ++i) { uint64_t x; do { x = r.next(); } while (x < threshold); out[i] = (int32_t)(x % rg); }
  TALOS_ENTRY_END
}
TALOS_API talos_status talos_lcg_rand_host(uint64_t seed, double lo, double hi, double* out, int64_t n) {
  TALOS_ENTRY_BEGIN
  TALOS_REQUIRE(out || n == 0, TALOS_ERR_ARG, "null output");
  uint64_t x = seed;
  for (int64_t i = 0; i < n; ++i) {
    x = x * 6364136223846793005ULL + 1ULL;
    out[i] = lo + ((double)(x >> 33) / 4294967295.0) * (hi - lo);
  }
  TALOS_ENTRY_END
}
