// Context, status and error plumbing of the C ABI (see include/b200graft.h).
// Replaces the reference's rt::Device error model (sticky first error,
// metal_pjrt/runtime/metal_runtime.h:43-53) and its host-side fault
// injection (metal_pjrt/runtime/metal_runtime.cc:1646-1653).
#include <cstdlib>

#include "common.cuh"

namespace b200 {

static thread_local char g_error[1024] = "";

void SetError(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

b200_status Fail(b200_status code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

b200_status Stick(b200_context* ctx, b200_status code) {
  if (ctx == nullptr || code == B200_OK) return code;
  int expected = 0;
  if (ctx->sticky.compare_exchange_strong(expected, static_cast<int>(code))) {
    std::lock_guard<std::mutex> lock(ctx->mu);
    ctx->sticky_message = g_error;
  }
  return code;
}

bool PdlDisabled() {
  static const bool off = [] {
    const char* v = std::getenv("B200_NO_PDL");
    return v != nullptr && v[0] != '\0' && v[0] != '0';
  }();
  return off;
}

b200_status BeginLaunch(b200_context* ctx) {
  if (ctx == nullptr) return Fail(B200_INVALID_ARGUMENT, "null context");
  const int sticky = ctx->sticky.load();
  if (sticky != 0) {
    std::lock_guard<std::mutex> lock(ctx->mu);
    SetError("context is in a failed state: %s", ctx->sticky_message.c_str());
    return static_cast<b200_status>(sticky);
  }
  const int64_t fail_at = ctx->fail_at.load();
  if (fail_at > 0 && ctx->launches.load() + 1 >= fail_at) {
    ctx->fail_at.store(0);
    return Stick(ctx, Fail(B200_INTERNAL, "injected launch failure (launch %lld refused before enqueue)",
                           static_cast<long long>(fail_at)));
  }
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e != cudaSuccess)
    return Stick(ctx, Fail(B200_INTERNAL, "cudaSetDevice(%d): %s", ctx->device, cudaGetErrorString(e)));
  return B200_OK;
}

b200_status EndLaunch(b200_context* ctx, const char* what, int kernels) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return Stick(ctx, Fail(B200_INTERNAL, "%s: %s", what, cudaGetErrorString(e)));
  ctx->launches.fetch_add(kernels);
  return B200_OK;
}

}  // namespace b200

using namespace b200;

namespace {

// Waits on an mbarrier that nobody ever arrives at, with the caller's limit, and reports the
// way every bounded wait of this library reports: first report wins, B200_TIMEOUT and the
// wait's id in the status word; then it returns normally (no trap, the context stays usable).
__global__ void wait_probe_kernel(long long limit_cycles, int* status) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
    const long long t0 = clock64();
    bool ok = false;
    while (!ok && clock64() - t0 <= limit_cycles) ok = mbar_try_wait(&bar, 0);
    if (!ok) report_timeout(status, 900);
  }
}

}  // namespace

extern "C" {

int b200_abi_version(void) { return B200_ABI_VERSION; }

b200_status b200_context_wait_probe(b200_context* ctx, b200_stream stream, int64_t limit_cycles) {
  b200_status s = BeginLaunch(ctx);
  if (s != B200_OK) return s;
  if (limit_cycles < 1 || limit_cycles > 4000000000ll)
    return Fail(B200_INVALID_ARGUMENT, "b200_context_wait_probe: limit of %lld cycles (1 .. 4e9)", static_cast<long long>(limit_cycles));
  wait_probe_kernel<<<1, 32, 0, stream>>>(limit_cycles, ctx->dev_status);
  return EndLaunch(ctx, "b200_context_wait_probe");
}

const char* b200_last_error(void) { return g_error; }

b200_status b200_context_create(int device_ordinal, b200_context** out) {
  if (out == nullptr) return Fail(B200_INVALID_ARGUMENT, "b200_context_create: null out");
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0) {
    (void)cudaGetLastError();
    return Fail(B200_FAILED_PRECONDITION, "no CUDA device: %s (this library has no CPU fallback)",
                e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0");
  }
  if (device_ordinal < 0 || device_ordinal >= count)
    return Fail(B200_INVALID_ARGUMENT, "device ordinal %d out of range [0, %d)", device_ordinal, count);
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, device_ordinal);
  if (e != cudaSuccess) return Fail(B200_INTERNAL, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
  if (prop.major != 10)
    return Fail(B200_FAILED_PRECONDITION, "device %d is sm_%d%d; this library holds sm_100a code only",
                device_ordinal, prop.major, prop.minor);
  e = cudaSetDevice(device_ordinal);
  if (e != cudaSuccess) return Fail(B200_INTERNAL, "cudaSetDevice: %s", cudaGetErrorString(e));
  b200_context* ctx = new b200_context();
  ctx->device = device_ordinal;
  ctx->sm_count = prop.multiProcessorCount;
  ctx->max_smem_optin = static_cast<int>(prop.sharedMemPerBlockOptin);
  e = cudaMalloc(&ctx->dev_status, 4 * sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(ctx->dev_status, 0, 4 * sizeof(int));
  if (e == cudaSuccess) e = cudaMallocHost(&ctx->host_status, 4 * sizeof(int));
  ctx->qtc_parts_floats = 4u << 20;   // 16 MB
  ctx->qtc_tiles_max = 1 << 16;
  if (e == cudaSuccess) e = cudaMalloc(&ctx->qtc_parts, ctx->qtc_parts_floats * sizeof(float));
  if (e == cudaSuccess) e = cudaMalloc(&ctx->qtc_counters, ctx->qtc_tiles_max * sizeof(unsigned));
  if (e == cudaSuccess) e = cudaMemset(ctx->qtc_counters, 0, ctx->qtc_tiles_max * sizeof(unsigned));
  if (e != cudaSuccess) {
    b200_status s = Fail(B200_RESOURCE_EXHAUSTED, "context allocation: %s", cudaGetErrorString(e));
    if (ctx->dev_status) cudaFree(ctx->dev_status);
    if (ctx->qtc_parts) cudaFree(ctx->qtc_parts);
    if (ctx->qtc_counters) cudaFree(ctx->qtc_counters);
    delete ctx;
    return s;
  }
  ctx->host_status[0] = 0;
  if (AttnStaticScratchInit(ctx) != B200_OK) {
    b200_context_destroy(ctx);
    return B200_INTERNAL;
  }
  *out = ctx;
  return B200_OK;
}

void b200_context_destroy(b200_context* ctx) {
  if (ctx == nullptr) return;
  cudaSetDevice(ctx->device);
  if (ctx->dev_status) cudaFree(ctx->dev_status);
  if (ctx->qtc_parts) cudaFree(ctx->qtc_parts);
  if (ctx->qtc_counters) cudaFree(ctx->qtc_counters);
  if (ctx->qmm_ws) cudaFree(ctx->qmm_ws);
  if (ctx->host_status) cudaFreeHost(ctx->host_status);
  delete ctx;
}

b200_status b200_context_error(b200_context* ctx) {
  if (ctx == nullptr) return Fail(B200_INVALID_ARGUMENT, "null context");
  int sticky = ctx->sticky.load();
  if (sticky == 0 && ctx->dev_status != nullptr) {
    // Plain blocking read of four ints; callers use this after synchronising.
    int word[4] = {0, 0, 0, 0};
    cudaSetDevice(ctx->device);
    cudaError_t e = cudaMemcpy(word, ctx->dev_status, sizeof(word), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) {
      Stick(ctx, Fail(B200_INTERNAL, "reading the device status word: %s", cudaGetErrorString(e)));
    } else if (word[0] != 0) {
      if (word[0] == B200_TIMEOUT)
        Stick(ctx, Fail(B200_TIMEOUT, "a kernel reported B200_TIMEOUT: bounded wait %d gave up", word[1]));
      else if (word[0] == B200_INVALID_ARGUMENT)
        Stick(ctx, Fail(B200_INVALID_ARGUMENT,
                        "a kernel reported B200_INVALID_ARGUMENT: device-side argument check %d failed (a position "
                        "outside the cache or a token id outside the vocabulary)", word[1]));
      else
        Stick(ctx, Fail(static_cast<b200_status>(word[0]), "a kernel reported status %d (site %d)", word[0], word[1]));
    }
    sticky = ctx->sticky.load();
  }
  if (sticky != 0) {
    std::lock_guard<std::mutex> lock(ctx->mu);
    SetError("%s", ctx->sticky_message.c_str());
  }
  return static_cast<b200_status>(sticky);
}

void b200_context_fail_launch_after(b200_context* ctx, int64_t n) {
  if (ctx == nullptr) return;
  ctx->fail_at.store(n <= 0 ? 0 : ctx->launches.load() + n);
}

int64_t b200_context_launch_count(b200_context* ctx) { return ctx == nullptr ? 0 : ctx->launches.load(); }

void b200_qmm_force_route(b200_context* ctx, int route) {
  if (ctx != nullptr) ctx->qmm_route.store(route);
}

void b200_gemm_force_route(b200_context* ctx, int route) {
  if (ctx != nullptr) ctx->force_route.store(route);
}

}  // extern "C"
