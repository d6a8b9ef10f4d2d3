/* The h3_gpu_* operator layer of libh3q8: opaque context and tensors, command
 * scope, file loading, and the linear operators that dispatch on a weight's
 * q8 descriptor -- the subset of h3cli's src/gpu.h that the DiT block's linear
 * path uses, with the reference's conventions:
 *   - int results: 1 ok, 0 failure; the reason is kept per context (h3_gpu_error)
 *   - operators need an open command scope (h3_gpu_begin), enqueue on the
 *     context's compute stream and never block; h3_gpu_submit waits and reports
 *     deferred errors (CUDA errors, a kernel's bounded wait that ran out,
 *     non-finite activations seen by the quantiser)
 *   - the caller owns tensors, the context owns scratch
 * (src/cuda/gpu_cuda.cu:128-230, 429-489, 595-666 are the behaviour followed.) */
#include <algorithm>
#include <cerrno>
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fcntl.h>
#include <mutex>
#include <new>
#include <sys/stat.h>
#include <unistd.h>
#include <string>
#include <vector>

#include "h3q8.h"
#include "h3q8_internal.h"
#include "kernels_misc.cuh"

using namespace h3q8;

struct h3_gpu_tensor {
    h3_gpu *owner = nullptr;
    void *data = nullptr;
    size_t elements = 0, bytes = 0;
    h3_gpu_dtype dtype = H3_GPU_F32;
    h3_gpu_storage storage = H3_GPU_DEVICE_ONLY;
    cudaEvent_t ready = nullptr;    /* recorded on the copy stream after an async fill   */
    cudaEvent_t released = nullptr; /* recorded on the compute stream after the last use */
    bool ready_recorded = false, release_recorded = false;
    /* q8 descriptor: int8 [n,k] at offset 0, fp32 scales [n, ceil(k/group)] at scale_offset */
    int q8 = 0;
    uint32_t q8_n = 0, q8_k = 0, q8_group = 0;
    size_t q8_scale_offset = 0;
    bool borrowed = false; /* a view into a weight-stream slot: the memory is not this tensor's */
};
struct h3_gpu_event { h3_gpu *owner = nullptr; cudaEvent_t value = nullptr; bool recorded = false; };

struct h3_gpu {
    int device = 0;
    cudaStream_t compute = nullptr, copy = nullptr; /* copy: host to device and weight streaming */
    cudaStream_t copy_out = nullptr;                /* device to host, so that both PCIe directions run at once */
    bool active = false, deferred_error = false;
    char error[1024] = {0};
    h3_gpu_stats stats = {};
    h3q8_gpu_profile profile = {};
    int quant_mode = 0;         /* 0 off, 1 W8A16, 2 W8A8 */
    uint32_t group = 0;
    bool group_set = false;
    int w8a16_scratch_rows = -1; /* rows at or above which W8A16 dequantises to scratch first; 0 = never; -1 = by shape */
    void *arena[4] = {nullptr, nullptr, nullptr, nullptr}; /* 0 int8 activations, 1 activation scales, 2 bf16 weight scratch, 3 reserved for a split-K workspace (unused: few-row problems reduce on chip) */
    size_t arena_bytes[4] = {0, 0, 0, 0};
    int dependent_launch = 1;   /* GEMMs start as programmatic dependents of their conversion kernel; H3Q8_DEPENDENT_LAUNCH=0 turns it off */
    int skinny_direct = 1;      /* W8A16 with at most 128 rows: main-loop dequantisation on the weight-streaming kernel (the weight is read once as int8) */
    uint32_t *flags = nullptr;  /* [0] kernel wait status, [1] non-finite seen */
    unsigned long long *diagnostics = nullptr;   /* [0] clipped, [1] non-zero values quantised to zero; H3_QUANT_DIAGNOSTICS=1 */
    void *bounce[2] = {nullptr, nullptr};
    cudaEvent_t bounce_free[2] = {nullptr, nullptr};
    bool bounce_used[2] = {false, false};
    std::string quant_cache;    /* directory of packed-weight artifacts; empty = no cache */
    uint64_t allocation_budget = 0; /* H3_CUDA_TEST_MEMORY_BUDGET: fail allocations beyond this many live bytes */
    h3_weight_options weight_options = {H3_WEIGHTS_AUTO, -1, 0, 0};
    h3_weight_plan weight_plan = {};
    bool allocation_failed = false; /* an allocation ran out of memory: an automatic plan may retry with fewer resident blocks */
    std::mutex mutex, copy_mutex;
    std::vector<h3_gpu_tensor *> accessed;
    /* profiling: event pairs per kernel, category 0 = GEMM, 7 = conversion */
    bool profiling = false;
    struct Span { cudaEvent_t start, stop; int category; };
    std::vector<Span> spans;
    std::vector<cudaEvent_t> spare_events;
    std::mutex span_mutex;      /* copies may be issued from another thread than the operators */
    std::string label = "DiT";  /* names the context in profile reports */
    double created = 0;
};

/* Brackets work on one stream (the compute stream unless another is named) with an event
 * pair while profiling; finished pairs are read back after the next synchronising submit.
 * Categories as in src/cuda/gpu_cuda.cu:231-273: 0 GEMM, 3 slot wait, 4 host to device,
 * 5 device to host, 7 quantisation conversion.  No fence or cross-stream dependency is added. */
struct ProfileScope {
    h3_gpu *g;
    cudaStream_t stream;
    h3_gpu::Span span{};
    bool live = false;
    static cudaEvent_t event(h3_gpu *g) {
        cudaEvent_t e = nullptr;
        if (!g->spare_events.empty()) { e = g->spare_events.back(); g->spare_events.pop_back(); }
        else cudaEventCreate(&e);
        return e;
    }
    ProfileScope(h3_gpu *gpu, int category, cudaStream_t target = nullptr) : g(gpu), stream(target ? target : gpu->compute) {
        if (!g->profiling) return;
        {
            std::lock_guard<std::mutex> lock(g->span_mutex);
            span.start = event(g); span.stop = event(g); span.category = category;
        }
        live = span.start && span.stop && cudaEventRecord(span.start, stream) == cudaSuccess;
    }
    ~ProfileScope() {
        if (!live || cudaEventRecord(span.stop, stream) != cudaSuccess) return;
        std::lock_guard<std::mutex> lock(g->span_mutex);
        g->spans.push_back(span);
    }
};
static void harvest_profile(h3_gpu *g) {
    std::lock_guard<std::mutex> lock(g->span_mutex);
    std::vector<h3_gpu::Span> pending;
    for (auto &s : g->spans) {
        float ms = 0;
        if (cudaEventQuery(s.stop) == cudaErrorNotReady) { pending.push_back(s); continue; } /* a copy still in flight */
        if (cudaEventElapsedTime(&ms, s.start, s.stop) == cudaSuccess) {
            if (s.category == 0) { g->stats.linear_seconds += ms * 1e-3; g->profile.linear_kernel_launches++; }
            else if (s.category == 3) { /* slot wait: time the compute stream sat idle waiting for a weight copy */
                g->stats.stream_wait_seconds += ms * 1e-3;
                if (ms > 0.02f) g->stats.stream_stalls++;
            }
            else if (s.category == 4) g->stats.h2d_seconds += ms * 1e-3;
            else if (s.category == 5) g->stats.d2h_seconds += ms * 1e-3;
            else { g->stats.quant_conversion_seconds += ms * 1e-3; g->profile.conversion_kernel_launches++; }
        }
        g->spare_events.push_back(s.start);
        g->spare_events.push_back(s.stop);
    }
    g->spans.swap(pending);
}

static const size_t BOUNCE_BYTES = 16u << 20; /* src/cuda/gpu_cuda.cu:79-82 */

static double now_seconds() {
    return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
static int set_error(h3_gpu *g, const char *format, ...) {
    if (g) {
        va_list args;
        va_start(args, format);
        vsnprintf(g->error, sizeof g->error, format, args);
        va_end(args);
    }
    return 0;
}
static int checked(h3_gpu *g, cudaError_t e, const char *what, size_t bytes = 0) {
    if (e == cudaSuccess) return 1;
    if (g) g->deferred_error = true;
    return set_error(g, "CUDA %s: %s (%zu bytes, device %d)", what, cudaGetErrorString(e), bytes, g ? g->device : -1);
}
static int selected(h3_gpu *g) { return g && checked(g, cudaSetDevice(g->device), "select device"); }
static int launch_ready(h3_gpu *g) {
    return selected(g) && (g->active || set_error(g, "CUDA operation requires h3_gpu_begin"));
}
static size_t item_size(h3_gpu_dtype t) { return t == H3_GPU_I8 ? 1 : (t == H3_GPU_BF16 || t == H3_GPU_F16) ? 2 : 4; }

static int require(h3_gpu *g, const h3_gpu_tensor *t, h3_gpu_dtype dtype, size_t elements, const char *label) {
    if (!t) return set_error(g, "%s: tensor is missing", label);
    if (t->owner != g) return set_error(g, "%s: tensor belongs to another context", label);
    if (t->dtype != dtype) return set_error(g, "%s: wrong element type", label);
    if (t->elements < elements) return set_error(g, "%s: %zu elements, need %zu", label, t->elements, elements);
    return 1;
}
/* Device pointer of a tensor for use on the compute stream: waits for an
 * asynchronous fill, and notes the tensor so its 'released' event is recorded
 * after the launch (src/cuda/gpu_cuda.cu:223-230, 208-220). */
static void *pointer(const h3_gpu_tensor *t) {
    if (!t) return nullptr;
    h3_gpu *g = t->owner;
    if (t->ready_recorded) cudaStreamWaitEvent(g->compute, t->ready, 0);
    g->accessed.push_back(const_cast<h3_gpu_tensor *>(t));
    return t->data;
}
static int launch_status(h3_gpu *g, const char *what, unsigned dispatches) {
    g->stats.direct_dispatches += dispatches;
    int ok = checked(g, cudaGetLastError(), what);
    for (h3_gpu_tensor *t : g->accessed)
        if (t->released) {
            if (!checked(g, cudaEventRecord(t->released, g->compute), "tensor release event")) ok = 0;
            else t->release_recorded = true;
        }
    g->accessed.clear();
    return ok && !g->deferred_error;
}
static int arena(h3_gpu *g, int which, size_t bytes) {
    if (g->arena_bytes[which] >= bytes) { g->stats.native_scratch_reuses++; return 1; }
    if (g->arena[which]) {
        cudaStreamSynchronize(g->compute);
        cudaFree(g->arena[which]);
        g->stats.live_bytes -= g->arena_bytes[which];
        g->stats.native_scratch_bytes -= g->arena_bytes[which];
        g->arena[which] = nullptr;
        g->arena_bytes[which] = 0;
    }
    if (!checked(g, cudaMalloc(&g->arena[which], bytes), "scratch allocation", bytes)) return 0;
    g->arena_bytes[which] = bytes;
    g->stats.native_scratch_bytes += bytes;
    g->stats.native_scratch_allocations++;
    g->stats.live_bytes += bytes;
    if (g->stats.live_bytes > g->stats.peak_live_bytes) g->stats.peak_live_bytes = g->stats.live_bytes;
    return 1;
}

/* ------------------------------------------------------------------ context */
extern "C" h3_gpu *h3_gpu_create(const char *, char *error, size_t error_size) {
    auto refuse = [&](const char *why) -> h3_gpu * {
        if (error && error_size) snprintf(error, error_size, "%s", why);
        return nullptr;
    };
    int device = 0, count = 0;
    const char *chosen = getenv("H3_CUDA_DEVICE"); /* src/cuda/cuda_probe.c:31-40 */
    if (cudaGetDeviceCount(&count) != cudaSuccess || !count) return refuse("no CUDA device: libh3q8 has no CPU path");
    if (chosen && *chosen) {
        char *end = nullptr;
        long v = strtol(chosen, &end, 10);
        if (*end || v < 0 || v >= count) return refuse("H3_CUDA_DEVICE is not a valid device index");
        device = (int)v;
    }
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return refuse("cannot query the CUDA device");
    if (prop.major != 10) return refuse("libh3q8 is built for sm_100a (B200) only");
    h3_gpu *g = new (std::nothrow) h3_gpu;
    if (!g) return refuse("out of host memory");
    g->device = device;
    g->created = now_seconds();
    {   /* src/cuda/gpu_cuda.cu:305: residency options are read once, when the context is made */
        char why[160] = {0};
        if (!h3_weight_options_read(&g->weight_options, 0, why, sizeof why)) { delete g; return refuse(why); }
        g->allocation_budget = g->weight_options.allocation_limit;
    }
    g->profiling = getenv("H3_PROFILE") != nullptr;
    const char *dependent = getenv("H3Q8_DEPENDENT_LAUNCH");
    if (dependent && *dependent) g->dependent_launch = atoi(dependent);
    const char *skinny = getenv("H3Q8_SKINNY_DIRECT");
    if (skinny && *skinny) g->skinny_direct = atoi(skinny);
    const char *policy = getenv("H3Q8_W8A16_SCRATCH_ROWS");
    /* unset: the policy is chosen per problem (w8a16_to_scratch); a number fixes the row threshold, 0 the main-loop kernels */
    g->w8a16_scratch_rows = policy && *policy ? atoi(policy) : -1;
    bool ok = cudaSetDevice(device) == cudaSuccess &&
              cudaStreamCreateWithFlags(&g->compute, cudaStreamNonBlocking) == cudaSuccess &&
              cudaStreamCreateWithFlags(&g->copy, cudaStreamNonBlocking) == cudaSuccess &&
              cudaStreamCreateWithFlags(&g->copy_out, cudaStreamNonBlocking) == cudaSuccess &&
              cudaMalloc(&g->flags, 2 * sizeof(uint32_t)) == cudaSuccess &&
              cudaMemset(g->flags, 0, 2 * sizeof(uint32_t)) == cudaSuccess;
    const char *diagnose = getenv("H3_QUANT_DIAGNOSTICS");   /* src/cuda/cuda_quant.cuh:156 */
    if (ok && diagnose && !strcmp(diagnose, "1"))
        ok = cudaMalloc(&g->diagnostics, 2 * sizeof(unsigned long long)) == cudaSuccess &&
             cudaMemset(g->diagnostics, 0, 2 * sizeof(unsigned long long)) == cudaSuccess;
    if (!ok) {
        snprintf(error ? error : g->error, error ? error_size : sizeof g->error, "CUDA context setup failed: %s",
                 cudaGetErrorString(cudaGetLastError()));
        h3_gpu_free(g);
        return nullptr;
    }
    return g;
}

extern "C" void h3_gpu_cancel(h3_gpu *g) {
    if (!g) return;
    cudaSetDevice(g->device);
    cudaStreamSynchronize(g->compute);
    cudaStreamSynchronize(g->copy);
    cudaStreamSynchronize(g->copy_out);
    cudaGetLastError();
    if (g->flags) cudaMemset(g->flags, 0, 2 * sizeof(uint32_t));
    g->accessed.clear();
    harvest_profile(g);
    g->active = false;
    g->deferred_error = false;
}

extern "C" void h3_gpu_free(h3_gpu *g) {
    if (!g) return;
    h3_gpu_cancel(g);
    for (auto &s : g->spans) { cudaEventDestroy(s.start); cudaEventDestroy(s.stop); }
    for (cudaEvent_t e : g->spare_events) cudaEventDestroy(e);
    for (int i = 0; i < 4; i++) if (g->arena[i]) cudaFree(g->arena[i]);
    for (int i = 0; i < 2; i++) {
        if (g->bounce[i]) cudaFreeHost(g->bounce[i]);
        if (g->bounce_free[i]) cudaEventDestroy(g->bounce_free[i]);
    }
    if (g->flags) cudaFree(g->flags);
    if (g->diagnostics) cudaFree(g->diagnostics);
    if (g->compute) cudaStreamDestroy(g->compute);
    if (g->copy) cudaStreamDestroy(g->copy);
    if (g->copy_out) cudaStreamDestroy(g->copy_out);
    delete g;
}

/* src/cuda/gpu_cuda.cu:497-524: the H3_PROFILE report, limited to the lines this path feeds --
 * weight placement, quantisation, transfers and the GEMM / conversion event categories. */
extern "C" void h3_gpu_profile_set_label(h3_gpu *g, const char *label) {
    if (g && label) g->label = label;
}
extern "C" void h3_gpu_profile_mark(h3_gpu *g, const char *phase) {
    if (!g || !getenv("H3_PROFILE")) return;
    if (!phase) phase = "";
    const h3_gpu_stats &s = g->stats;
    const double gib = 1073741824.;
    if (s.active_weight_blocks)
        fprintf(stderr, "h3cli: weight placement %s: resident=%llu/%llu resident_bytes=%llu slot_bytes=%llu pinned_bytes=%llu uploaded_bytes=%llu\n",
                phase, (unsigned long long)s.resident_blocks, (unsigned long long)s.active_weight_blocks,
                (unsigned long long)s.resident_weight_bytes, (unsigned long long)s.stream_slot_bytes,
                (unsigned long long)s.pinned_bytes, (unsigned long long)s.streamed_bytes);
    if (g->quant_mode)
        fprintf(stderr, "h3cli: quant profile %s / %s: mode=%s group=%u native_calls=%llu cache_hits=%llu prepared=%llu conversion=%.6fs (%llu kernels)\n",
                g->label.c_str(), phase, g->quant_mode == 2 ? "w8a8" : "w8a16", g->group,
                (unsigned long long)s.quant_projection_dispatches, (unsigned long long)s.quant_cache_hits,
                (unsigned long long)s.quant_cache_misses, s.quant_conversion_seconds, (unsigned long long)g->profile.conversion_kernel_launches);
    fprintf(stderr, "h3cli: CUDA profile %s / %s: wall %.3fs peak %.3f GiB, GEMM %llu, H2D %.3f GiB D2H %.3f GiB stream %.3f GiB wait %.3fs\n",
            g->label.c_str(), phase, now_seconds() - g->created, s.peak_live_bytes / gib, (unsigned long long)s.linear_dispatches,
            s.h2d_bytes / gib, s.d2h_bytes / gib, s.streamed_bytes / gib, s.stream_wait_seconds);
    fprintf(stderr, "h3cli: CUDA category seconds: GEMM %.6f (%llu kernels) conversion %.6f; stream stalls %llu / %.6fs\n", s.linear_seconds,
            (unsigned long long)g->profile.linear_kernel_launches, s.quant_conversion_seconds, (unsigned long long)s.stream_stalls, s.stream_wait_seconds);
    fprintf(stderr, "h3cli: CUDA transfer events: H2D %.6fs (%.3f GiB/s), D2H %.6fs (%.3f GiB/s)\n", s.h2d_seconds,
            s.h2d_seconds > 0 ? s.h2d_bytes / gib / s.h2d_seconds : 0.0, s.d2h_seconds, s.d2h_seconds > 0 ? s.d2h_bytes / gib / s.d2h_seconds : 0.0);
}

extern "C" const char *h3_gpu_error(const h3_gpu *g) { return g ? g->error : "no GPU context"; }
extern "C" int h3_gpu_get_stats(const h3_gpu *g, h3_gpu_stats *stats) {
    if (!g || !stats) return 0;
    *stats = g->stats;
    return 1;
}
extern "C" int h3q8_gpu_get_profile(const h3_gpu *g, h3q8_gpu_profile *profile) {
    if (!g || !profile) return 0;
    *profile = g->profile;
    return 1;
}
extern "C" const char *h3_gpu_backend_name(const h3_gpu *) { return "cuda-b200-q8"; }
extern "C" int h3_gpu_has_int8_mlp(const h3_gpu *g) { return g != nullptr; }

/* ------------------------------------------------------------ command scope */
extern "C" int h3_gpu_begin(h3_gpu *g) {
    if (!selected(g)) return 0;
    if (g->active) return set_error(g, "command scope already active");
    if (g->deferred_error) return set_error(g, "context has a pending error; call h3_gpu_cancel");
    g->active = true;
    return 1;
}
extern "C" int h3_gpu_continue(h3_gpu *g) {
    return launch_ready(g) && !g->deferred_error;
}
static int drain(h3_gpu *g) {
    if (!checked(g, cudaStreamSynchronize(g->compute), "synchronize")) return 0;
    harvest_profile(g);
    uint32_t flags[2] = {0, 0};
    if (!checked(g, cudaMemcpy(flags, g->flags, sizeof flags, cudaMemcpyDeviceToHost), "read device flags")) return 0;
    if (g->diagnostics) {   /* cumulative, like the reference's counters (src/cuda/gpu_cuda.cu:447-449) */
        unsigned long long counts[2] = {0, 0};
        if (cudaMemcpy(counts, g->diagnostics, sizeof counts, cudaMemcpyDeviceToHost) == cudaSuccess) {
            g->stats.quant_clipped_values = counts[0];
            g->stats.quant_zeroed_values = counts[1];
        }
    }
    uint32_t shared_status = h3q8_device_status(g->compute);
    if (flags[0] || flags[1] || shared_status) {
        cudaMemset(g->flags, 0, sizeof flags);
        g->deferred_error = true;
        if (flags[1] || (!flags[0] && (shared_status & 0x80000000u))) return set_error(g, "non-finite activation reached the int8 quantiser");
        uint32_t code = flags[0] ? flags[0] : shared_status;
        return set_error(g, "a linear kernel gave up a bounded wait (code %u, CTA %u)", code & 0xffu, code >> 8);
    }
    return 1;
}
extern "C" int h3_gpu_submit(h3_gpu *g) {
    if (!launch_ready(g)) return 0;
    g->active = false;
    g->stats.submissions++;
    int ok = drain(g);
    return ok && !g->deferred_error;
}
extern "C" int h3_gpu_synchronize(h3_gpu *g) {
    if (!selected(g)) return 0;
    return checked(g, cudaStreamSynchronize(g->compute), "synchronize") &&
           checked(g, cudaStreamSynchronize(g->copy), "synchronize copy stream") &&
           checked(g, cudaStreamSynchronize(g->copy_out), "synchronize download stream");
}

/* ------------------------------------------------------------------ tensors */
extern "C" h3_gpu_tensor *h3_gpu_tensor_alloc(h3_gpu *g, size_t elements, h3_gpu_dtype dtype, h3_gpu_storage storage) {
    if (!selected(g) || !elements) { set_error(g, "tensor allocation: no elements"); return nullptr; }
    size_t bytes = elements * item_size(dtype);
    std::lock_guard<std::mutex> lock(g->mutex);
    if (g->allocation_budget && g->stats.live_bytes + bytes > g->allocation_budget) {
        set_error(g, "CUDA allocation: out of memory (test budget %llu, live %llu, requested %zu)",
                  (unsigned long long)g->allocation_budget, (unsigned long long)g->stats.live_bytes, bytes);
        g->allocation_failed = true;
        return nullptr;
    }
    h3_gpu_tensor *t = new (std::nothrow) h3_gpu_tensor;
    if (!t) return nullptr;
    cudaError_t e = storage == H3_GPU_DEVICE_ONLY ? cudaMalloc(&t->data, bytes)
                  : storage == H3_GPU_HOST_PINNED ? cudaMallocHost(&t->data, bytes)
                                                  : cudaMallocManaged(&t->data, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        set_error(g, "CUDA allocation: %s; requested %zu bytes", cudaGetErrorString(e), bytes);
        delete t;
        return nullptr;
    }
    t->owner = g; t->elements = elements; t->bytes = bytes; t->dtype = dtype; t->storage = storage;
    cudaEventCreateWithFlags(&t->ready, cudaEventDisableTiming);
    cudaEventCreateWithFlags(&t->released, cudaEventDisableTiming);
    g->stats.tensor_allocations++;
    g->stats.allocated_bytes += bytes;
    g->stats.live_bytes += bytes;
    if (storage == H3_GPU_HOST_PINNED) {
        g->stats.pinned_bytes += bytes;
        if (g->stats.pinned_bytes > g->stats.peak_pinned_bytes) g->stats.peak_pinned_bytes = g->stats.pinned_bytes;
    } else if (storage == H3_GPU_DEVICE_ONLY) g->stats.device_bytes += bytes;
    if (g->stats.live_bytes > g->stats.peak_live_bytes) g->stats.peak_live_bytes = g->stats.live_bytes;
    return t;
}
extern "C" void h3_gpu_tensor_free(h3_gpu_tensor *t) {
    if (!t) return;
    h3_gpu *g = t->owner;
    cudaSetDevice(g->device);
    { /* work in flight may still use it: cudaFree waits, host memory needs an explicit wait */
        std::lock_guard<std::mutex> lock(g->mutex);
        for (auto it = g->accessed.begin(); it != g->accessed.end();) it = *it == t ? g->accessed.erase(it) : it + 1;
        if (t->borrowed) { /* nothing to release */ }
        else if (t->storage == H3_GPU_HOST_PINNED) { cudaStreamSynchronize(g->compute); cudaStreamSynchronize(g->copy); cudaStreamSynchronize(g->copy_out); cudaFreeHost(t->data); }
        else { if (t->ready_recorded) cudaEventSynchronize(t->ready); cudaFree(t->data); }
        if (!t->borrowed) g->stats.live_bytes -= t->bytes;
        if (!t->borrowed && t->storage == H3_GPU_HOST_PINNED) g->stats.pinned_bytes -= t->bytes;
        if (!t->borrowed && t->storage == H3_GPU_DEVICE_ONLY && g->stats.device_bytes >= t->bytes) g->stats.device_bytes -= t->bytes;
    }
    if (t->ready) cudaEventDestroy(t->ready);
    if (t->released) cudaEventDestroy(t->released);
    delete t;
}
extern "C" void *h3_gpu_tensor_contents(h3_gpu_tensor *t) {
    if (!t || t->storage == H3_GPU_DEVICE_ONLY) return nullptr;
    cudaSetDevice(t->owner->device);
    cudaStreamSynchronize(t->owner->compute);
    cudaStreamSynchronize(t->owner->copy);
    cudaStreamSynchronize(t->owner->copy_out);
    return t->data;
}
extern "C" size_t h3_gpu_tensor_elements(const h3_gpu_tensor *t) { return t ? t->elements : 0; }
extern "C" h3_gpu_dtype h3_gpu_tensor_dtype(const h3_gpu_tensor *t) { return t ? t->dtype : H3_GPU_F32; }
extern "C" h3_gpu_tensor *h3_gpu_tensor_new_f32(h3_gpu *g, size_t n) { return h3_gpu_tensor_alloc(g, n, H3_GPU_F32, H3_GPU_DEVICE_ONLY); }
extern "C" h3_gpu_tensor *h3_gpu_tensor_new_bf16(h3_gpu *g, size_t n) { return h3_gpu_tensor_alloc(g, n, H3_GPU_BF16, H3_GPU_DEVICE_ONLY); }
extern "C" h3_gpu_tensor *h3_gpu_tensor_new_i8(h3_gpu *g, size_t n) { return h3_gpu_tensor_alloc(g, n, H3_GPU_I8, H3_GPU_DEVICE_ONLY); }

/* Host <-> device copies order themselves after everything already enqueued on
 * the compute stream and return when the bytes have moved. */
static int upload(h3_gpu_tensor *t, size_t offset_bytes, const void *values, size_t bytes) {
    h3_gpu *g = t->owner;
    if (!selected(g)) return 0;
    if (offset_bytes > t->bytes || bytes > t->bytes - offset_bytes) return set_error(g, "tensor write out of range");
    if (!checked(g, cudaMemcpyAsync((char *)t->data + offset_bytes, values, bytes, cudaMemcpyDefault, g->compute), "host to device copy", bytes) ||
        !checked(g, cudaStreamSynchronize(g->compute), "host to device copy wait")) return 0;
    g->stats.h2d_bytes += bytes;
    return 1;
}
static int download(const h3_gpu_tensor *t, void *values, size_t bytes) {
    h3_gpu *g = t->owner;
    if (!selected(g)) return 0;
    if (bytes > t->bytes) return set_error(g, "tensor read out of range");
    if (t->ready_recorded) cudaStreamWaitEvent(g->compute, t->ready, 0);
    if (!checked(g, cudaMemcpyAsync(values, t->data, bytes, cudaMemcpyDefault, g->compute), "device to host copy", bytes) ||
        !checked(g, cudaStreamSynchronize(g->compute), "device to host copy wait")) return 0;
    g->stats.d2h_bytes += bytes;
    return 1;
}
static h3_gpu_tensor *from_host(h3_gpu *g, const void *values, size_t elements, h3_gpu_dtype dtype) {
    if (!values) { set_error(g, "tensor upload: no source"); return nullptr; }
    h3_gpu_tensor *t = h3_gpu_tensor_alloc(g, elements, dtype, H3_GPU_DEVICE_ONLY);
    if (t && !upload(t, 0, values, t->bytes)) { h3_gpu_tensor_free(t); t = nullptr; }
    return t;
}
extern "C" h3_gpu_tensor *h3_gpu_tensor_from_f32(h3_gpu *g, const float *v, size_t n) { return from_host(g, v, n, H3_GPU_F32); }
extern "C" h3_gpu_tensor *h3_gpu_tensor_from_bf16(h3_gpu *g, const uint16_t *v, size_t n) { return from_host(g, v, n, H3_GPU_BF16); }
extern "C" h3_gpu_tensor *h3_gpu_tensor_from_u32(h3_gpu *g, const uint32_t *v, size_t n) { return from_host(g, v, n, H3_GPU_U32); }
#define TYPED_IO(name, ctype, dt)                                                                              \
    extern "C" int h3_gpu_tensor_read_##name(const h3_gpu_tensor *t, ctype *values, size_t elements) {        \
        if (!t || !values) return 0;                                                                           \
        if (t->dtype != dt) return set_error(t->owner, "tensor read: wrong element type");                     \
        return download(t, values, elements * sizeof(ctype));                                                  \
    }                                                                                                          \
    extern "C" int h3_gpu_tensor_write_##name(h3_gpu_tensor *t, const ctype *values, size_t elements) {       \
        if (!t || !values) return 0;                                                                           \
        if (t->dtype != dt) return set_error(t->owner, "tensor write: wrong element type");                    \
        return upload(t, 0, values, elements * sizeof(ctype));                                                 \
    }
TYPED_IO(f32, float, H3_GPU_F32)
TYPED_IO(bf16, uint16_t, H3_GPU_BF16)
TYPED_IO(i8, int8_t, H3_GPU_I8)
extern "C" int h3_gpu_tensor_read_u32(const h3_gpu_tensor *t, uint32_t *values, size_t elements) {
    if (!t || !values) return 0;
    if (t->dtype != H3_GPU_U32) return set_error(t->owner, "tensor read: wrong element type");
    return download(t, values, elements * 4);
}
extern "C" int h3_gpu_tensor_write_bf16_range(h3_gpu_tensor *t, size_t offset, const uint16_t *values, size_t elements) {
    if (!t || !values) return 0;
    if (t->dtype != H3_GPU_BF16) return set_error(t->owner, "tensor write: wrong element type");
    return upload(t, offset * 2, values, elements * 2);
}

extern "C" int h3q8_gpu_tensor_upload_async(h3_gpu_tensor *t, const void *host, size_t bytes) {
    if (!t || !host) return 0;
    h3_gpu *g = t->owner;
    if (bytes > t->bytes) return set_error(g, "tensor write out of range");
    std::lock_guard<std::mutex> lock(g->copy_mutex);
    if (!selected(g)) return 0;
    if (t->release_recorded) cudaStreamWaitEvent(g->copy, t->released, 0);
    if (t->ready_recorded) cudaStreamWaitEvent(g->copy, t->ready, 0); /* an earlier download of this tensor */
    ProfileScope timing(g, 4, g->copy);
    if (!checked(g, cudaMemcpyAsync(t->data, host, bytes, cudaMemcpyHostToDevice, g->copy), "asynchronous host to device copy", bytes) ||
        !checked(g, cudaEventRecord(t->ready, g->copy), "tensor ready event")) return 0;
    t->ready_recorded = true;
    g->stats.h2d_bytes += bytes;
    return 1;
}
extern "C" int h3q8_gpu_tensor_download_async(h3_gpu_tensor *t, void *host, size_t bytes) {
    if (!t || !host) return 0;
    h3_gpu *g = t->owner;
    if (bytes > t->bytes) return set_error(g, "tensor read out of range");
    std::lock_guard<std::mutex> lock(g->copy_mutex);
    if (!selected(g)) return 0;
    if (t->release_recorded) cudaStreamWaitEvent(g->copy_out, t->released, 0);
    if (t->ready_recorded) cudaStreamWaitEvent(g->copy_out, t->ready, 0); /* an earlier upload of this tensor */
    ProfileScope timing(g, 5, g->copy_out);
    if (!checked(g, cudaMemcpyAsync(host, t->data, bytes, cudaMemcpyDeviceToHost, g->copy_out), "asynchronous device to host copy", bytes) ||
        !checked(g, cudaEventRecord(t->ready, g->copy_out), "tensor ready event")) return 0;
    t->ready_recorded = true; /* the next operator that writes the tensor waits for this copy */
    g->stats.d2h_bytes += bytes;
    return 1;
}
/* Host-side wait for the tensor's last asynchronous copy only: nothing else is drained, so later
 * uploads and operators already queued keep running. */
extern "C" int h3q8_gpu_tensor_wait(h3_gpu_tensor *t) {
    if (!t) return 0;
    h3_gpu *g = t->owner;
    if (!selected(g)) return 0;
    return !t->ready_recorded || checked(g, cudaEventSynchronize(t->ready), "tensor copy wait");
}

extern "C" h3_gpu_event *h3_gpu_event_new(h3_gpu *g) {
    if (!selected(g)) return nullptr;
    h3_gpu_event *e = new (std::nothrow) h3_gpu_event;
    if (e && cudaEventCreateWithFlags(&e->value, cudaEventDisableTiming) != cudaSuccess) { delete e; e = nullptr; }
    if (e) e->owner = g;
    return e;
}
extern "C" int h3_gpu_event_record(h3_gpu *g, h3_gpu_event *e) {
    if (!selected(g) || !e || e->owner != g) return 0;
    e->recorded = true;
    return checked(g, cudaEventRecord(e->value, g->compute), "event record");
}
extern "C" int h3_gpu_event_wait(h3_gpu *g, h3_gpu_event *e) {
    if (!selected(g) || !e || !e->recorded) return 0;
    return checked(g, cudaStreamWaitEvent(g->compute, e->value, 0), "event wait");
}
extern "C" void h3_gpu_event_free(h3_gpu_event *e) {
    if (!e) return;
    cudaEventDestroy(e->value);
    delete e;
}

/* ---------------------------------------------------------------- file I/O */
/* pread -> pinned bounce buffer -> cudaMemcpyAsync on the copy stream, two
 * bounce buffers in rotation, each guarded by a reuse event.  Safe to call from
 * an I/O thread while the owner thread enqueues compute: only the copy stream
 * and the copy mutex are touched (src/cuda/gpu_cuda.cu:761-841). */
static int file_into(h3_gpu_tensor *t, size_t dst_offset, const char *path, uint64_t file_offset, size_t bytes,
                     char *error, size_t error_size) {
    h3_gpu *g = t->owner;
    auto refuse = [&](const char *format, ...) {
        char text[512];
        va_list args;
        va_start(args, format);
        vsnprintf(text, sizeof text, format, args);
        va_end(args);
        if (error && error_size) snprintf(error, error_size, "%s", text);
        set_error(g, "%s", text);
        return 0;
    };
    if (dst_offset > t->bytes || bytes > t->bytes - dst_offset) return refuse("file read exceeds the tensor");
    std::lock_guard<std::mutex> lock(g->copy_mutex);
    if (cudaSetDevice(g->device) != cudaSuccess) return refuse("cannot select the CUDA device");
    int fd = open(path, O_RDONLY);
    if (fd < 0) return refuse("cannot open %s: %s", path, strerror(errno));
    /* a slot that compute may still be reading must not be overwritten */
    if (t->release_recorded) cudaStreamWaitEvent(g->copy, t->released, 0);
    double start = now_seconds();
    size_t done = 0;
    int slot = 0, ok = 1;
    while (ok && done < bytes) {
        if (!g->bounce[slot]) {
            if (cudaMallocHost(&g->bounce[slot], BOUNCE_BYTES) != cudaSuccess ||
                cudaEventCreateWithFlags(&g->bounce_free[slot], cudaEventDisableTiming) != cudaSuccess) {
                ok = refuse("cannot allocate a pinned staging buffer");
                break;
            }
            g->stats.pinned_bytes += BOUNCE_BYTES;
        }
        if (g->bounce_used[slot]) {   /* only time spent waiting for a busy staging buffer is a stream wait (src/cuda/gpu_cuda.cu:823-827) */
            const double waiting = now_seconds();
            if (cudaEventQuery(g->bounce_free[slot]) == cudaErrorNotReady) g->stats.stream_stalls++;
            cudaEventSynchronize(g->bounce_free[slot]);
            g->stats.stream_wait_seconds += now_seconds() - waiting;
        }
        size_t chunk = bytes - done < BOUNCE_BYTES ? bytes - done : BOUNCE_BYTES, got = 0;
        while (got < chunk) {
            ssize_t r = pread(fd, (char *)g->bounce[slot] + got, chunk - got, (off_t)(file_offset + done + got));
            if (r < 0 && errno == EINTR) continue;
            if (r <= 0) { ok = refuse("short read from %s at offset %llu", path, (unsigned long long)(file_offset + done + got)); break; }
            got += (size_t)r;
        }
        if (!ok) break;
        if (cudaMemcpyAsync((char *)t->data + dst_offset + done, g->bounce[slot], chunk, cudaMemcpyDefault, g->copy) != cudaSuccess ||
            cudaEventRecord(g->bounce_free[slot], g->copy) != cudaSuccess) {
            ok = refuse("CUDA copy from the staging buffer failed: %s", cudaGetErrorString(cudaGetLastError()));
            break;
        }
        g->bounce_used[slot] = true;
        done += chunk;
        slot ^= 1;
    }
    close(fd);
    if (ok) {
        cudaEventRecord(t->ready, g->copy);
        t->ready_recorded = true;
        g->stats.h2d_bytes += bytes;
        g->stats.streamed_bytes += bytes;
        g->stats.transfer_seconds += now_seconds() - start;
    }
    return ok;
}
extern "C" int h3_gpu_tensor_read_file_bf16(h3_gpu_tensor *t, const char *path, uint64_t offset, size_t elements,
                                            char *error, size_t error_size) {
    if (!t || !path || t->dtype != H3_GPU_BF16) return 0;
    return file_into(t, 0, path, offset, elements * 2, error, error_size);
}
extern "C" int h3_gpu_tensor_stream_file_bf16(h3_gpu_tensor *t, const char *path, uint64_t offset, size_t elements,
                                              char *error, size_t error_size) {
    return h3_gpu_tensor_read_file_bf16(t, path, offset, elements, error, error_size);
}
extern "C" h3_gpu_tensor *h3_gpu_tensor_load_bf16(h3_gpu *g, const char *path, uint64_t offset, size_t elements) {
    h3_gpu_tensor *t = h3_gpu_tensor_new_bf16(g, elements);
    if (t && !file_into(t, 0, path, offset, elements * 2, nullptr, 0)) { h3_gpu_tensor_free(t); t = nullptr; }
    return t;
}

/* ---------------------------------------------------------------- planning */
/* 0 resident, 1 streamed (two layer slots), -1 not even that.  The reserve is
 * max(1 GiB, total/10) as in src/cuda/gpu_cuda.cu:548-568. */
extern "C" int h3_gpu_plan_weights(h3_gpu *g, uint64_t weights, uint64_t activations) {
    if (!selected(g)) return -1;
    size_t free_bytes = 0, total = 0;
    if (!checked(g, cudaMemGetInfo(&free_bytes, &total), "memory query")) return -1;
    if (g->allocation_budget) {
        uint64_t left = g->allocation_budget > g->stats.live_bytes ? g->allocation_budget - g->stats.live_bytes : 0;
        if (left < free_bytes) free_bytes = left;
    }
    uint64_t reserve = total / 10 > (1ull << 30) ? total / 10 : (1ull << 30);
    if (g->allocation_budget) reserve = 0;
    uint64_t fixed = activations + reserve;
    if (free_bytes >= fixed && weights <= free_bytes - fixed) return 0;
    if (free_bytes >= fixed) return 1;
    set_error(g, "insufficient CUDA capacity for activations plus reserve");
    return -1;
}
extern "C" int h3_gpu_release_weight_cache(h3_gpu *g) { return g != nullptr; }

/* src/cuda/gpu_cuda.cu:559-578: plan which blocks stay resident from the device's free memory,
 * the context's live bytes and a reserve of max(1 GiB, 10 % of the device). */
extern "C" int h3_gpu_plan_bf16_weights(h3_gpu *g, uint64_t active_mask, uint64_t block_bytes, uint64_t future_bytes,
                                        int force_stream, int retry_cap, h3_weight_plan *plan) {
    if (!selected(g) || !plan) return 0;
    size_t available = 0, total = 0;
    if (!checked(g, cudaMemGetInfo(&available, &total), "weight planner")) return 0;
    h3_weight_options options = g->weight_options;
    if (force_stream && options.mode == H3_WEIGHTS_RESIDENT)
        return set_error(g, "--ssd-streaming conflicts with CUDA resident weight mode");
    if (force_stream) options.mode = H3_WEIGHTS_STREAM;
    if (retry_cap >= 0 && (options.max_resident < 0 || retry_cap < options.max_resident)) options.max_resident = retry_cap;
    uint64_t reserve = total / 10 > (1ull << 30) ? total / 10 : (1ull << 30);
    char why[256] = {0};
    if (!h3_weight_plan_build(plan, options, active_mask, block_bytes, available, g->stats.live_bytes, future_bytes, reserve,
                              why, sizeof why))
        return set_error(g, "%s", why);
    g->weight_plan = *plan;
    g->allocation_failed = false;
    g->stats.resident_weight_bytes = plan->resident_bytes;
    g->stats.stream_slot_bytes = plan->slot_bytes;
    g->stats.resident_blocks = plan->resident_count;
    g->stats.active_weight_blocks = plan->active_count;
    g->stats.resident_block_mask = plan->resident_mask;
    return 1;
}
extern "C" int h3_gpu_should_retry_streaming(const h3_gpu *g) {
    return g && g->allocation_failed && g->weight_options.mode == H3_WEIGHTS_AUTO;
}
/* src/cuda/gpu_cuda.cu:579-594: may a context made under earlier options be kept for this request? */
extern "C" int h3_gpu_weight_plan_compatible(h3_gpu *g, int force_stream) {
    if (!g) return 0;
    h3_weight_options requested, old = g->weight_options;
    char why[160];
    if (!h3_weight_options_read(&requested, force_stream, why, sizeof why)) return 0;
    if (force_stream) { requested.mode = H3_WEIGHTS_STREAM; old.mode = H3_WEIGHTS_STREAM; }
    if (!h3_weight_options_equal(&requested, &old)) return 0;
    if (old.mode == H3_WEIGHTS_AUTO && g->weight_plan.active_count && g->weight_plan.resident_count < g->weight_plan.active_count)
        return 0; /* a constrained automatic plan reconsiders capacity on every request */
    size_t free_bytes = 0, total = 0;
    return selected(g) && cudaMemGetInfo(&free_bytes, &total) == cudaSuccess &&
           free_bytes >= (total / 10 > (1ull << 30) ? total / 10 : (1ull << 30));
}

/* -------------------------------------------------------- quantised weights */
extern "C" int h3q8_gpu_set_group(h3_gpu *g, uint32_t group) {
    if (!g) return 0;
    if (group && group % 16) return set_error(g, "scale group must be 0 (per channel) or a multiple of 16");
    g->group = group;
    g->group_set = true;
    return 1;
}
extern "C" void *h3q8_gpu_tensor_device_pointer(const h3_gpu_tensor *t) { return t ? t->data : nullptr; }
extern "C" void *h3q8_gpu_compute_stream(h3_gpu *g) { return g ? (void *)g->compute : nullptr; }
extern "C" int h3q8_gpu_set_profiling(h3_gpu *g, int enabled) {
    if (!g) return 0;
    g->profiling = enabled != 0;
    return 1;
}
extern "C" int h3q8_gpu_set_w8a16_scratch_rows(h3_gpu *g, uint32_t rows) {
    if (!g) return 0;
    g->w8a16_scratch_rows = (int)rows;
    return 1;
}
static int make_directories(const std::string &path) {
    for (size_t i = 1; i <= path.size(); i++)
        if (i == path.size() || path[i] == '/') {
            std::string part = path.substr(0, i);
            if (mkdir(part.c_str(), 0755) && errno != EEXIST) return 0;
        }
    struct stat st;
    return !stat(path.c_str(), &st) && S_ISDIR(st.st_mode);
}
extern "C" int h3_gpu_quant_configure(h3_gpu *g, int mode, const char *cache, uint64_t weights, uint64_t activations, int force_stream) {
    if (!g) return 0;
    if (mode < 0 || mode > 2) return set_error(g, "quantisation mode must be 0 (off), 1 (W8A16) or 2 (W8A8)");
    if (!mode) return 1;
    if (g->quant_mode) return set_error(g, "quantized GPU context already configured");
    if (cache && *cache) { /* src/cuda/cuda_quant.cpp:137-139: the cache directory is created at configure time */
        if (!make_directories(cache)) return set_error(g, "cannot create quantization cache %s: %s", cache, strerror(errno));
        g->quant_cache = cache;
    }
    if (weights || activations) {
        int plan = h3_gpu_plan_weights(g, weights / 2, activations);
        if (plan < 0) return 0;
        (void)force_stream;
    }
    if (!g->group_set) {
        const char *env = getenv("H3Q8_GROUP");
        g->group = env && *env ? (uint32_t)strtoul(env, nullptr, 10) : 0;
    }
    g->quant_mode = mode;
    return 1;
}

static h3_gpu_tensor *q8_blob(h3_gpu *g, uint32_t rows, uint32_t columns, uint32_t group) {
    size_t offset, bytes;
    if (!h3q8_q8_layout(rows, columns, group, &offset, &bytes)) {
        set_error(g, "q8 weight %ux%u: invalid or too large shape", rows, columns);
        return nullptr;
    }
    /* scales start on a 16-byte boundary so kernels can fetch them as vectors */
    size_t aligned = (offset + 15) & ~(size_t)15;
    h3_gpu_tensor *t = h3_gpu_tensor_alloc(g, aligned + (bytes - offset), H3_GPU_I8, H3_GPU_DEVICE_ONLY);
    if (!t) return nullptr;
    t->elements = (size_t)rows * columns;
    t->q8 = 1; t->q8_n = rows; t->q8_k = columns; t->q8_group = group; t->q8_scale_offset = aligned;
    return t;
}

static h3_gpu_tensor *q8_load_file(h3_gpu *g, const char *path, uint64_t offset, uint32_t rows, uint32_t columns, uint32_t group) {
    if (!selected(g) || !path) return nullptr;
    if (offset & 1) { set_error(g, "q8 load: bf16 payload offset must be even"); return nullptr; }
    double start = now_seconds();
    h3_gpu_tensor *t = q8_blob(g, rows, columns, group);
    if (!t) return nullptr;
    /* Bounded staging: bf16 rows pass through a device buffer of at most 32 MiB
     * (src/metal/q8_host.inc:3-51 bounds its staging the same way). */
    size_t row_bytes = (size_t)columns * 2;
    uint32_t chunk_rows = (uint32_t)((32u << 20) / row_bytes);
    if (!chunk_rows) chunk_rows = 1;
    if (chunk_rows > rows) chunk_rows = rows;
    h3_gpu_tensor *staging = h3_gpu_tensor_new_bf16(g, (size_t)chunk_rows * columns);
    const uint32_t width = group ? group : columns;
    const uint32_t groups = (uint32_t)(((uint64_t)columns + width - 1) / width);
    int ok = staging != nullptr;
    cudaMemsetAsync(t->data, 0, t->bytes, g->compute);
    for (uint32_t r = 0; ok && r < rows; r += chunk_rows) {
        uint32_t n = rows - r < chunk_rows ? rows - r : chunk_rows;
        /* the previous chunk's pack kernel must be done with the staging buffer */
        cudaEventRecord(staging->released, g->compute);
        staging->release_recorded = true;
        ok = file_into(staging, 0, path, offset + (uint64_t)r * row_bytes, (size_t)n * row_bytes, nullptr, 0);
        if (!ok) break;
        cudaStreamWaitEvent(g->compute, staging->ready, 0);
        const uint64_t items = (uint64_t)n * groups;
        q8_pack_rows_kernel<<<(unsigned)((items + 7) / 8), 256, 0, g->compute>>>(
            (const uint16_t *)staging->data, (int8_t *)t->data + (size_t)r * columns,
            (float *)((char *)t->data + t->q8_scale_offset) + (size_t)r * groups, n, columns, width, groups, g->flags + 1);
        if (g->diagnostics)   /* weights count on cold preparation, as in the reference */
            quant_diagnostics_kernel<<<(unsigned)std::min<uint64_t>(4096, ((uint64_t)n * columns + 255) / 256), 256, 0, g->compute>>>(
                (const uint16_t *)staging->data, (const int8_t *)t->data + (size_t)r * columns,
                (const float *)((char *)t->data + t->q8_scale_offset) + (size_t)r * groups, n, columns, width, groups, g->diagnostics);
        count_launch(1);
        ok = checked(g, cudaGetLastError(), "q8 pack launch");
    }
    uint32_t nonfinite = 0;
    if (ok) ok = checked(g, cudaStreamSynchronize(g->compute), "q8 pack wait") &&
                 checked(g, cudaMemcpy(&nonfinite, g->flags + 1, 4, cudaMemcpyDeviceToHost), "q8 pack flag");
    if (ok && nonfinite) {
        cudaMemset(g->flags + 1, 0, 4);
        ok = set_error(g, "q8 load: non-finite weight in %s", path);
    }
    h3_gpu_tensor_free(staging);
    if (!ok) { h3_gpu_tensor_free(t); return nullptr; }
    g->stats.q8_weights++;
    g->stats.q8_source_bytes += (uint64_t)rows * row_bytes;
    g->stats.q8_storage_bytes += t->bytes;
    g->stats.q8_load_seconds += now_seconds() - start;
    g->stats.quant_conversion_seconds += now_seconds() - start;
    return t;
}
extern "C" h3_gpu_tensor *h3_gpu_q8_load(h3_gpu *g, const char *path, uint64_t offset, uint32_t rows, uint32_t columns) {
    return q8_load_file(g, path, offset, rows, columns, g && g->group_set ? g->group : H3_Q8_GROUP);
}
extern "C" h3_gpu_tensor *h3_gpu_quant_load(h3_gpu *g, const char *path, uint64_t offset, uint32_t rows, uint32_t columns) {
    if (!g) return nullptr;
    if (!g->quant_mode || !rows || !columns || rows % 128 || columns % 128 || (uint64_t)rows * columns > UINT32_MAX) {
        set_error(g, "quantized weight shape must be nonzero and a multiple of 128"); /* src/cuda/cuda_quant.cuh:293-295 */
        return nullptr;
    }
    if (g->quant_cache.empty()) {
        h3_gpu_tensor *t = q8_load_file(g, path, offset, rows, columns, g->group);
        if (t) g->stats.quant_cache_misses++;
        return t;
    }
    /* src/cuda/cuda_quant.cuh:292-333: artifact hit -> upload the packed bytes; miss -> pack on the
     * device, read the blob back, publish it; the source is re-checked before either is accepted */
    /* H3_QUANT_VERIFY=1 selects the content-keyed, payload-verified kind (src/weights/quant.c:10-13) */
    const char *verify = getenv("H3_QUANT_VERIFY");
    h3q8_cache *entry = verify && !strcmp(verify, "1")
        ? h3q8_cache_open_content(g->quant_cache.c_str(), path, offset, rows, columns, g->group, g->error, sizeof g->error)
        : h3q8_cache_open(g->quant_cache.c_str(), path, offset, rows, columns, g->group, g->error, sizeof g->error);
    if (!entry) return nullptr;
    const size_t bytes = h3q8_cache_payload_bytes(entry);
    std::vector<unsigned char> payload;
    try { payload.resize(bytes); } catch (const std::bad_alloc &) {
        h3q8_cache_close(entry);
        set_error(g, "host allocation failed for %zu-byte packed weight", bytes);
        return nullptr;
    }
    int status = h3q8_cache_read(entry, payload.data(), g->error, sizeof g->error);
    h3_gpu_tensor *t = nullptr;
    if (status == 1) {
        t = q8_blob(g, rows, columns, g->group);
        if (t && !upload(t, 0, payload.data(), t->bytes < bytes ? t->bytes : bytes)) { h3_gpu_tensor_free(t); t = nullptr; }
        if (t) { g->stats.quant_cache_hits++; g->stats.q8_weights++; g->stats.q8_storage_bytes += t->bytes; }
    } else if (status == 0) {
        t = q8_load_file(g, path, offset, rows, columns, g->group);
        if (t) {
            memset(payload.data(), 0, bytes);
            if (!download(t, payload.data(), t->bytes < bytes ? t->bytes : bytes) ||
                !h3q8_cache_write(entry, payload.data(), g->error, sizeof g->error)) { h3_gpu_tensor_free(t); t = nullptr; }
            else g->stats.quant_cache_misses++;
        }
    }
    if (t && !h3q8_cache_unchanged(entry, g->error, sizeof g->error)) { h3_gpu_tensor_free(t); t = nullptr; }
    h3q8_cache_close(entry);
    return t;
}
extern "C" h3_gpu_tensor *h3q8_gpu_q8_from_host(h3_gpu *g, const int8_t *weights, const float *scales,
                                                uint32_t rows, uint32_t columns, uint32_t group) {
    if (!selected(g) || !weights || !scales) return nullptr;
    h3_gpu_tensor *t = q8_blob(g, rows, columns, group);
    if (!t) return nullptr;
    const uint32_t width = group ? group : columns;
    const size_t groups = ((size_t)columns + width - 1) / width;
    if (!upload(t, 0, weights, (size_t)rows * columns) ||
        !upload(t, t->q8_scale_offset, scales, (size_t)rows * groups * sizeof(float))) { h3_gpu_tensor_free(t); return nullptr; }
    g->stats.q8_weights++;
    g->stats.q8_storage_bytes += t->bytes;
    return t;
}

/* ------------------------------------------------------ packed-weight streaming */
struct h3q8_weight_stream {
    h3_gpu *owner = nullptr;
    size_t slot_bytes = 0;
    uint32_t slots = 0, next = 0;
    std::vector<void *> memory;
    std::vector<cudaEvent_t> ready, released;
    std::vector<bool> ready_recorded, released_recorded;
};

extern "C" size_t h3q8_q8_blob_bytes(uint32_t rows, uint32_t columns, uint32_t group, size_t *scale_offset) {
    size_t offset, bytes;
    if (!h3q8_q8_layout(rows, columns, group, &offset, &bytes)) return 0;
    size_t aligned = (offset + 15) & ~(size_t)15;
    if (scale_offset) *scale_offset = aligned;
    return (aligned + (bytes - offset) + 255) & ~(size_t)255;
}

/* src/weights/residency.h:31-33, for this library's packing: payload = int8 [rows, columns], scale plane at the next
 * 16-byte boundary (fp32 [rows, ceil(columns / group)]), no global-scale slot (global == end of the scales), total
 * rounded up to 256 bytes.  mode 1 (W8A16) uses the process default group (H3Q8_GROUP, else the reference's 64),
 * mode 2 (W8A8) per-channel scales. */
extern "C" int h3_weight_packed_size(uint32_t rows, uint32_t columns, int mode, uint64_t *scale, uint64_t *global, uint64_t *bytes) {
    if (!rows || !columns || (mode != 1 && mode != 2) || !scale || !global || !bytes) return 0;
    uint32_t group = 0;
    if (mode == 1) {
        const char *env = getenv("H3Q8_GROUP");
        group = env && *env ? (uint32_t)strtoul(env, nullptr, 10) : H3_Q8_GROUP;
    }
    size_t offset = 0, raw_offset = 0, raw_bytes = 0;
    const size_t total = h3q8_q8_blob_bytes(rows, columns, group, &offset);
    if (!total || !h3q8_q8_layout(rows, columns, group, &raw_offset, &raw_bytes)) return 0;
    *scale = offset;
    *global = offset + (raw_bytes - raw_offset);
    *bytes = total;
    return 1;
}

extern "C" h3q8_weight_stream *h3q8_gpu_weight_stream_create(h3_gpu *g, size_t slot_bytes, uint32_t slots) {
    if (!selected(g)) return nullptr;
    if (!slot_bytes || slots < 2 || slots > 8) { set_error(g, "weight stream: needs 2..8 slots of non-zero size"); return nullptr; }
    if (g->allocation_budget && g->stats.live_bytes + slot_bytes * slots > g->allocation_budget) {
        set_error(g, "CUDA allocation: out of memory (test budget) for %u weight-stream slots of %zu bytes", slots, slot_bytes);
        return nullptr;
    }
    auto *s = new (std::nothrow) h3q8_weight_stream;
    if (!s) return nullptr;
    s->owner = g; s->slot_bytes = slot_bytes; s->slots = slots;
    for (uint32_t i = 0; i < slots; i++) {
        void *memory = nullptr;
        cudaEvent_t a = nullptr, b = nullptr;
        if (cudaMalloc(&memory, slot_bytes) != cudaSuccess || cudaEventCreateWithFlags(&a, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&b, cudaEventDisableTiming) != cudaSuccess) {
            cudaGetLastError();
            set_error(g, "weight stream: cannot allocate slot %u of %zu bytes", i, slot_bytes);
            if (memory) cudaFree(memory);
            h3q8_gpu_weight_stream_free(s);
            return nullptr;
        }
        s->memory.push_back(memory); s->ready.push_back(a); s->released.push_back(b);
        s->ready_recorded.push_back(false); s->released_recorded.push_back(false);
        g->stats.live_bytes += slot_bytes;
        g->stats.stream_slot_bytes += slot_bytes;
    }
    if (g->stats.live_bytes > g->stats.peak_live_bytes) g->stats.peak_live_bytes = g->stats.live_bytes;
    return s;
}

extern "C" void h3q8_gpu_weight_stream_free(h3q8_weight_stream *s) {
    if (!s) return;
    h3_gpu *g = s->owner;
    cudaSetDevice(g->device);
    cudaStreamSynchronize(g->copy);
    cudaStreamSynchronize(g->compute);
    for (size_t i = 0; i < s->memory.size(); i++) {
        cudaFree(s->memory[i]);
        cudaEventDestroy(s->ready[i]);
        cudaEventDestroy(s->released[i]);
        g->stats.live_bytes -= s->slot_bytes;
        g->stats.stream_slot_bytes -= s->slot_bytes;
    }
    delete s;
}

extern "C" int h3q8_gpu_weight_stream_prefetch(h3q8_weight_stream *s, const void *host_blob, size_t bytes) {
    if (!s || !host_blob) return -1;
    h3_gpu *g = s->owner;
    if (!bytes || bytes > s->slot_bytes) { set_error(g, "weight stream: %zu bytes do not fit a %zu-byte slot", bytes, s->slot_bytes); return -1; }
    std::lock_guard<std::mutex> lock(g->copy_mutex);
    if (cudaSetDevice(g->device) != cudaSuccess) return -1;
    const int slot = (int)s->next;
    s->next = (s->next + 1) % s->slots;
    /* the copy may not overwrite a slot the compute stream is still reading */
    if (s->released_recorded[slot] && !checked(g, cudaStreamWaitEvent(g->copy, s->released[slot], 0), "weight stream wait")) return -1;
    ProfileScope timing(g, 4, g->copy);
    if (!checked(g, cudaMemcpyAsync(s->memory[slot], host_blob, bytes, cudaMemcpyHostToDevice, g->copy), "weight stream copy", bytes) ||
        !checked(g, cudaEventRecord(s->ready[slot], g->copy), "weight stream ready event")) return -1;
    s->ready_recorded[slot] = true;
    g->stats.h2d_bytes += bytes;
    g->stats.streamed_bytes += bytes;
    return slot;
}

/* A slot filled by the caller's own stream instead of a host copy (an NCCL all-gather of the ranks'
 * slices, a peer copy): reserve hands out the next slot and makes `producer_stream` wait until the
 * compute stream has released it; publish records the slot's ready event on that stream.  The slot is
 * plain local device memory before any kernel of this library reads it. */
extern "C" int h3q8_gpu_weight_stream_reserve(h3q8_weight_stream *s, void *producer_stream, void **device_pointer) {
    if (!s || !device_pointer) return -1;
    h3_gpu *g = s->owner;
    std::lock_guard<std::mutex> lock(g->copy_mutex);
    if (cudaSetDevice(g->device) != cudaSuccess) return -1;
    const int slot = (int)s->next;
    s->next = (s->next + 1) % s->slots;
    if (s->released_recorded[slot] &&
        !checked(g, cudaStreamWaitEvent((cudaStream_t)producer_stream, s->released[slot], 0), "weight stream reserve")) return -1;
    *device_pointer = s->memory[slot];
    return slot;
}
extern "C" int h3q8_gpu_weight_stream_publish(h3q8_weight_stream *s, int slot, void *producer_stream, size_t bytes) {
    if (!s || slot < 0 || (uint32_t)slot >= s->slots) return 0;
    h3_gpu *g = s->owner;
    if (bytes > s->slot_bytes) return set_error(g, "weight stream: %zu bytes do not fit a %zu-byte slot", bytes, s->slot_bytes);
    std::lock_guard<std::mutex> lock(g->copy_mutex);
    if (cudaSetDevice(g->device) != cudaSuccess) return 0;
    if (!checked(g, cudaEventRecord(s->ready[slot], (cudaStream_t)producer_stream), "weight stream publish event")) return 0;
    s->ready_recorded[slot] = true;
    g->stats.streamed_bytes += bytes;
    return 1;
}

extern "C" int h3q8_gpu_weight_stream_acquire(h3q8_weight_stream *s, int slot) {
    if (!s || slot < 0 || (uint32_t)slot >= s->slots) return 0;
    h3_gpu *g = s->owner;
    if (!selected(g)) return 0;
    if (!s->ready_recorded[slot]) return set_error(g, "weight stream: slot %d was never filled", slot);
    /* with profiling on, an event pair around the wait measures how long the compute
     * stream really stalled for the copy (category 3, slot wait) */
    ProfileScope timing(g, 3);
    return checked(g, cudaStreamWaitEvent(g->compute, s->ready[slot], 0), "weight stream acquire");
}

extern "C" int h3q8_gpu_weight_stream_release(h3q8_weight_stream *s, int slot) {
    if (!s || slot < 0 || (uint32_t)slot >= s->slots) return 0;
    h3_gpu *g = s->owner;
    if (!selected(g)) return 0;
    if (!checked(g, cudaEventRecord(s->released[slot], g->compute), "weight stream release event")) return 0;
    s->released_recorded[slot] = true;
    return 1;
}

extern "C" h3_gpu_tensor *h3q8_gpu_weight_stream_view(h3q8_weight_stream *s, int slot, size_t offset, uint32_t rows,
                                                      uint32_t columns, uint32_t group) {
    if (!s || slot < 0 || (uint32_t)slot >= s->slots) return nullptr;
    h3_gpu *g = s->owner;
    size_t scale_offset = 0, bytes = h3q8_q8_blob_bytes(rows, columns, group, &scale_offset);
    if (!bytes || (offset & 255) || offset > s->slot_bytes || bytes > s->slot_bytes - offset) {
        set_error(g, "weight stream view: %ux%u at offset %zu does not fit the slot (offsets are multiples of 256)", rows, columns, offset);
        return nullptr;
    }
    h3_gpu_tensor *t = new (std::nothrow) h3_gpu_tensor;
    if (!t) return nullptr;
    t->owner = g; t->data = (char *)s->memory[slot] + offset; t->elements = (size_t)rows * columns; t->bytes = bytes;
    t->dtype = H3_GPU_I8; t->storage = H3_GPU_DEVICE_ONLY; t->borrowed = true;
    t->q8 = 1; t->q8_n = rows; t->q8_k = columns; t->q8_group = group; t->q8_scale_offset = scale_offset;
    return t;
}

/* The row / K-group activation quantiser on the compute stream, followed by the diagnostics scan when that is on. */
static void quantise_activations(h3_gpu *g, const uint16_t *in, int8_t *out, float *scales, uint64_t live, uint64_t total, uint32_t segment,
                                 float clip) {
    launch_quantize_rows(in, out, scales, live, total, segment, clip, g->flags + 1, g->compute);
    if (g->diagnostics && live)
        quant_diagnostics_kernel<<<(unsigned)std::min<uint64_t>(4096, (live * segment + 255) / 256), 256, 0, g->compute>>>(
            in, out, scales, live, segment, segment, 1, g->diagnostics);
}
/* src/metal/gpu.m:3379-3384: H3_INT8_ACTIVATION_CLIP in [0.1, 1] shrinks the range the MLP's row quantisers map to +-127 */
static float mlp_activation_clip() {
    const char *text = getenv("H3_INT8_ACTIVATION_CLIP");
    if (!text) return 1.0f;
    const float parsed = strtof(text, nullptr);
    return parsed >= 0.1f && parsed <= 1.0f ? parsed : 1.0f;
}

/* ------------------------------------------------------------------ linears */
static size_t round256(size_t n) { return (n + 255) & ~(size_t)255; }

/* Which of the two W8A16 policies a problem of more than 128 rows takes.  Dequantise-then-GEMM pays one pass over the
 * weight (3 bytes of HBM traffic per element and a launch) and then runs at the bf16 kernel's rate; main-loop
 * dequantisation pays nothing up front but is bound by shared-memory bandwidth (80 KB instead of 64 KB per k-block and
 * SM), about three quarters of that rate.  The up-front pass is the larger cost only while the GEMM itself is short:
 * few rows and a short K. */
static bool w8a16_to_scratch(const h3_gpu *g, const h3_gpu_linear_problem &q) {
    if (q.activation == H3Q8_ACT_SWIGLU) return g->w8a16_scratch_rows != 0;
    if (g->w8a16_scratch_rows < 0) return q.rows > 1024 || q.input_dim > 4096;
    return g->w8a16_scratch_rows && q.rows >= (uint32_t)g->w8a16_scratch_rows;
}

/* Whether the GEMM of a problem starts as a programmatic dependent of its conversion kernel (set-up overlapped with
 * that kernel's tail).  Worth 2-3 us per call, which is 3-4 % of a 4 096-row projection; at 32 400 rows it is lost in the
 * noise for K = 3 072 and costs 1 % at K = 12 288, where the early-resident GEMM blocks take thread slots from a
 * conversion grid of many waves.  Never with profiling: the event between the two kernels breaks the dependency. */
static bool dependent_launch(const h3_gpu *g, const h3_gpu_linear_problem &q) {
    return g->dependent_launch && !g->profiling && q.rows <= 8192;
}

/* Scratch a problem needs from the context arenas: [0] int8 activations, [1] their scales, [2] bf16 weight,
 * [3] nothing any more (problems of at most 128 rows reduce their K slices on chip). */
static void linear_scratch(const h3_gpu *g, const h3_gpu_linear_problem &q, size_t need[4]) {
    need[0] = need[1] = need[2] = need[3] = 0;
    if (!q.weight) return;
    const bool swiglu = q.activation == H3Q8_ACT_SWIGLU;
    uint32_t mode = H3Q8_MODE_BF16;
    if (q.weight->q8 && g->quant_mode == 2) {
        size_t padded = ((size_t)q.rows + 127u) & ~(size_t)127u;
        need[0] = round256(padded * q.input_dim);
        need[1] = round256(padded * sizeof(float));
        mode = H3Q8_MODE_W8A8;
    } else if (q.weight->q8) {
        /* few rows: the int8 weight is read once with main-loop dequantisation (the weight-streaming kernel), when the
         * weight is large enough for that to matter */
        const bool skinny = g->skinny_direct && !swiglu && q.rows <= 128 && (uint64_t)q.input_dim * q.output_dim >= (1u << 20);
        if (q.input_dim % 16 == 0 && !skinny && w8a16_to_scratch(g, q)) {
            need[2] = round256((size_t)q.output_dim * (swiglu ? 2 : 1) * q.input_dim * 2);
        } else mode = H3Q8_MODE_W8A16;
    }
    (void)mode;   /* problems of at most 128 rows run on the weight-streaming kernel, which needs no split-K workspace */
}

/* The linear operators: validate every problem, run the conversion kernels each needs
 * (per-token quantiser for W8A8, weight dequantiser for the W8A16 scratch policy), then
 * hand all of them to the raw layer in one grouped call. */
static int linear_dispatch_many(h3_gpu *g, const h3_gpu_linear_problem *problems, uint32_t count, const h3q8_rope_desc *rope = nullptr,
                                h3_gpu_tensor *partial_sums = nullptr) {
    if (!launch_ready(g)) return 0;
    if (partial_sums) {
        if (!problems || count != 1 || rope || g->quant_mode == 2 || problems[0].output || problems[0].activation != H3Q8_ACT_NONE)
            return set_error(g, "linear partial sums: one problem with bf16 or W8A16 operands, no output tensor and no activation");
        if (!require(g, partial_sums, H3_GPU_F32, (size_t)problems[0].rows * problems[0].output_dim, "linear partial sums")) return 0;
    }
    if (!problems || !count || count > 16) return set_error(g, "linear: between 1 and 16 problems per call");
    size_t total[4] = {0, 0, 0, 0};
    for (uint32_t i = 0; i < count; i++) {
        const h3_gpu_linear_problem &q = problems[i];
        const uint32_t rows = q.rows, k = q.input_dim, n = q.output_dim;
        if (!rows || !k || !n) return set_error(g, "linear %ux%ux%u: invalid tensor shape/type", rows, n, k);
        if (!q.weight || q.weight->owner != g) return set_error(g, "linear %ux%ux%u: weight is missing or foreign", rows, n, k);
        if (!require(g, q.input, H3_GPU_BF16, (size_t)rows * k, "linear input") ||
            ((q.output || (!rope && !partial_sums)) && !require(g, q.output, H3_GPU_BF16, (size_t)rows * n, "linear output"))) return 0;
        const uint32_t wrows = q.activation == H3Q8_ACT_SWIGLU ? 2 * n : n; /* SwiGLU weight: [gate n | up n] rows */
        if (q.bias && !require(g, q.bias, H3_GPU_BF16, wrows, "linear bias")) return 0;
        if (q.gate && !require(g, q.gate, H3_GPU_BF16, n, "linear gate")) return 0;
        if (q.residual && !require(g, q.residual, H3_GPU_BF16, (size_t)rows * n, "linear residual")) return 0;
        if (q.output == q.input || q.output == q.weight) return set_error(g, "linear %ux%ux%u: output aliases an operand", rows, n, k);
        if (q.activation < 0 || q.activation > H3Q8_ACT_SWIGLU) return set_error(g, "linear: unknown activation %d", q.activation);
        if (q.weight->q8) {
            if (q.weight->q8_n != wrows || q.weight->q8_k != k)
                return set_error(g, "linear %ux%ux%u: q8 weight is %ux%u", rows, n, k, q.weight->q8_n, q.weight->q8_k);
        } else if (q.weight->dtype != H3_GPU_BF16 || q.weight->elements < (size_t)wrows * k) {
            return set_error(g, "linear %ux%ux%u: invalid tensor shape/type", rows, n, k);
        }
        size_t need[4];
        linear_scratch(g, q, need);
        for (int a = 0; a < 4; a++) total[a] += need[a];
    }
    for (int a = 0; a < 4; a++)
        if (total[a] && !arena(g, a, total[a])) return 0;

    h3q8_linear_desc descs[16];
    size_t offset[4] = {0, 0, 0, 0};
    unsigned dispatches = 0;
    for (uint32_t i = 0; i < count; i++) {
        const h3_gpu_linear_problem &q = problems[i];
        const h3_gpu_tensor *w = q.weight;
        h3q8_linear_desc &d = descs[i];
        d = h3q8_linear_desc{};
        d.rows = q.rows; d.input_dim = q.input_dim; d.output_dim = q.output_dim;
        d.bias = q.bias ? (const uint16_t *)pointer(q.bias) : nullptr;
        d.gate = q.gate ? (const uint16_t *)pointer(q.gate) : nullptr;
        d.residual = q.residual ? (const uint16_t *)pointer(q.residual) : nullptr;
        d.activation = (uint32_t)q.activation;
        d.output = q.output ? (uint16_t *)pointer(q.output) : nullptr;
        d.accumulators = partial_sums ? (int32_t *)pointer(partial_sums) : nullptr;
        d.rope = rope;
        d.input = pointer(q.input);
        d.weight = pointer(w);
        size_t need[4];
        linear_scratch(g, q, need);
        if (need[3] && !rope) { d.workspace = (char *)g->arena[3] + offset[3]; d.workspace_bytes = need[3]; }
        if (w->q8) {
            d.weight_scales = (const float *)((const char *)w->data + w->q8_scale_offset);
            d.weight_group = w->q8_group;
            if (need[0]) { /* W8A8: per-token quantise into context scratch, then the int8 GEMM */
                const uint32_t padded = (q.rows + 127u) & ~127u;
                int8_t *xq = (int8_t *)g->arena[0] + offset[0];
                float *xs = (float *)((char *)g->arena[1] + offset[1]);
                {
                    ProfileScope timing(g, 7);
                    quantise_activations(g, (const uint16_t *)d.input, xq, xs, q.rows, padded, q.input_dim, 1.0f);
                }
                count_launch(1);
                dispatches++;
                d.mode = H3Q8_MODE_W8A8;
                d.input = xq;
                d.input_scales = xs;
                d.after_producer = dependent_launch(g, q);   /* the quantiser is the kernel right before the GEMM */
            } else if (need[2]) {
                /* policy 0 of the reference: dequantise once, then a bf16 GEMM (src/metal/q8_host.inc:75-88) */
                uint16_t *wb = (uint16_t *)((char *)g->arena[2] + offset[2]);
                ProfileScope timing(g, 7);
                if (!h3q8_q8_dequant((const int8_t *)d.weight, d.weight_scales, wb, w->q8_n, q.input_dim, d.weight_group, g->compute)) {
                    g->accessed.clear();
                    return set_error(g, "%s", h3q8_last_error());
                }
                dispatches++;
                d.mode = H3Q8_MODE_BF16;
                d.weight = wb;
                d.weight_scales = nullptr;
                d.weight_group = 0;
                d.after_producer = dependent_launch(g, q);   /* the dequantiser is the kernel right before the GEMM */
            } else d.mode = H3Q8_MODE_W8A16;
            g->stats.q8_dispatches++;
            g->stats.quant_projection_dispatches++;
        } else d.mode = H3Q8_MODE_BF16;
        for (int a = 0; a < 4; a++) offset[a] += need[a];
    }
    const uint64_t before = h3q8_kernel_launches();
    {
        ProfileScope timing(g, 0);
        int ok = count == 1 ? h3q8_linear(&descs[0], g->compute) : h3q8_linear_grouped(descs, count, g->compute);
        if (!ok) { g->accessed.clear(); return set_error(g, "%s", h3q8_last_error()); }
    }
    dispatches += (unsigned)(h3q8_kernel_launches() - before);
    g->stats.linear_dispatches += count;
    return launch_status(g, "linear", dispatches);
}

static int linear_dispatch(h3_gpu *g, h3_gpu_tensor *out, const h3_gpu_tensor *in, const h3_gpu_tensor *w,
                           const h3_gpu_tensor *bias, const h3_gpu_tensor *gate, const h3_gpu_tensor *residual,
                           uint32_t rows, uint32_t k, uint32_t n, int activation) {
    h3_gpu_linear_problem q = {out, in, w, bias, gate, residual, rows, k, n, activation};
    return linear_dispatch_many(g, &q, 1);
}

extern "C" int h3_gpu_linear_bf16(h3_gpu *g, h3_gpu_tensor *out, const h3_gpu_tensor *in, const h3_gpu_tensor *w,
                                  const h3_gpu_tensor *bias, uint32_t rows, uint32_t k, uint32_t n) {
    return linear_dispatch(g, out, in, w, bias, nullptr, nullptr, rows, k, n, H3Q8_ACT_NONE);
}
extern "C" int h3_gpu_linear_fused_bf16(h3_gpu *g, h3_gpu_tensor *out, const h3_gpu_tensor *in, const h3_gpu_tensor *w,
                                        const h3_gpu_tensor *bias, const h3_gpu_tensor *gate, const h3_gpu_tensor *residual,
                                        uint32_t rows, uint32_t k, uint32_t n, int activation) {
    return linear_dispatch(g, out, in, w, bias, gate, residual, rows, k, n, activation);
}
/* A linear cut along K (or across GPUs): the fp32 partial sums of one K slice, before any epilogue term, and the
 * call that turns summed partial sums into the bf16 result with the usual epilogue. */
extern "C" int h3q8_gpu_linear_partial_f32(h3_gpu *g, h3_gpu_tensor *sums, const h3_gpu_tensor *in, const h3_gpu_tensor *w,
                                           uint32_t rows, uint32_t k, uint32_t n) {
    h3_gpu_linear_problem q = {nullptr, in, w, nullptr, nullptr, nullptr, rows, k, n, H3Q8_ACT_NONE};
    return linear_dispatch_many(g, &q, 1, nullptr, sums);
}
extern "C" int h3q8_gpu_linear_finish_bf16(h3_gpu *g, h3_gpu_tensor *out, const h3_gpu_tensor *sums, const h3_gpu_tensor *bias,
                                           const h3_gpu_tensor *gate, const h3_gpu_tensor *residual, uint32_t rows, uint32_t n, int activation) {
    if (!launch_ready(g)) return 0;
    if (!require(g, out, H3_GPU_BF16, (size_t)rows * n, "linear finish output") || !require(g, sums, H3_GPU_F32, (size_t)rows * n, "linear finish sums") ||
        (bias && !require(g, bias, H3_GPU_BF16, n, "linear finish bias")) || (gate && !require(g, gate, H3_GPU_BF16, n, "linear finish gate")) ||
        (residual && !require(g, residual, H3_GPU_BF16, (size_t)rows * n, "linear finish residual"))) return 0;
    if (activation < 0 || activation > H3Q8_ACT_GELU_TANH) return set_error(g, "linear finish: activation must be none or GELU-tanh");
    if (!h3q8_linear_finish((const float *)pointer(sums), rows, n, bias ? (const uint16_t *)pointer(bias) : nullptr,
                            gate ? (const uint16_t *)pointer(gate) : nullptr, residual ? (const uint16_t *)pointer(residual) : nullptr,
                            (uint32_t)activation, (uint16_t *)pointer(out), g->compute)) {
        g->accessed.clear();
        return set_error(g, "%s", h3q8_last_error());
    }
    return launch_status(g, "linear finish", 1);
}

/* Several projections of different shapes in one call: with bf16 or W8A8 operands (and
 * the W8A16 scratch policy) all of them run in ONE GEMM launch on the two-CTA kernel. */
extern "C" int h3_gpu_linear_grouped_bf16(h3_gpu *g, const h3_gpu_linear_problem *problems, uint32_t count) {
    if (!g) return 0;
    return linear_dispatch_many(g, problems, count);
}

extern "C" int h3_gpu_quantize_weight_int8(h3_gpu *g, h3_gpu_tensor *out, h3_gpu_tensor *scales, const h3_gpu_tensor *in,
                                           uint32_t rows, uint32_t columns) {
    if (!launch_ready(g)) return 0;
    if (!rows || !columns || !require(g, in, H3_GPU_BF16, (size_t)rows * columns, "BF16 weight to quantize") ||
        !require(g, out, H3_GPU_I8, (size_t)rows * columns, "int8 quantized output") ||
        !require(g, scales, H3_GPU_F32, rows, "int8 quantization scales")) return 0;
    quantise_activations(g, (const uint16_t *)pointer(in), (int8_t *)pointer(out), (float *)pointer(scales), rows, rows, columns, 1.0f);
    count_launch(1);
    return launch_status(g, "weight quantiser", 1);
}

/* src/metal/gpu.m:3183-3249: quantise the rows (padded to 128) into the caller's
 * scratch tensors, then the int8 GEMM with the dequantising epilogue. */
extern "C" int h3_gpu_linear_int8_bf16(h3_gpu *g, h3_gpu_tensor *out, h3_gpu_tensor *qin, h3_gpu_tensor *in_scales,
                                       const h3_gpu_tensor *in, const h3_gpu_tensor *w, const h3_gpu_tensor *w_scales,
                                       uint32_t rows, uint32_t k, uint32_t n, int) {
    if (!launch_ready(g)) return 0;
    uint32_t padded = (rows + 127u) & ~127u;
    if (rows < 128 || k % 128 || n % 128) return set_error(g, "int8 linear needs rows >= 128 and K, N multiples of 128");
    if (!require(g, w, H3_GPU_I8, (size_t)n * k, "int8 linear weight") || !require(g, w_scales, H3_GPU_F32, n, "int8 linear weight scales") ||
        !require(g, out, H3_GPU_BF16, (size_t)rows * n, "int8 linear output") || !require(g, in, H3_GPU_BF16, (size_t)rows * k, "int8 linear input") ||
        !require(g, qin, H3_GPU_I8, (size_t)padded * k, "int8 quantized output") ||
        !require(g, in_scales, H3_GPU_F32, padded, "int8 quantization scales")) return 0;
    quantise_activations(g, (const uint16_t *)pointer(in), (int8_t *)pointer(qin), (float *)pointer(in_scales), rows, padded, k, 1.0f);
    count_launch(1);
    h3q8_linear_desc d = {};
    d.mode = H3Q8_MODE_W8A8; d.rows = rows; d.input_dim = k; d.output_dim = n;
    d.input = qin->data; d.input_scales = (const float *)in_scales->data;
    d.weight = pointer(w); d.weight_scales = (const float *)pointer(w_scales);
    d.output = (uint16_t *)pointer(out);
    if (!h3q8_linear(&d, g->compute)) { g->accessed.clear(); return set_error(g, "%s", h3q8_last_error()); }
    g->stats.linear_dispatches++;
    return launch_status(g, "int8 linear", 2);
}

/* src/gpu.h:630-642, src/metal/gpu.m:3837-3900: gate + residual, RMS/AdaLN and the per-row int8
 * quantiser in one pass; the output feeds h3_gpu_linear_fused_int8_bf16 without another
 * look at the bf16 activations. */
extern "C" int h3_gpu_gate_adaln_quantize_int8(h3_gpu *g, h3_gpu_tensor *gated_residual, h3_gpu_tensor *quantized_output,
                                               h3_gpu_tensor *quantized_scales, const h3_gpu_tensor *residual,
                                               const h3_gpu_tensor *branch, const h3_gpu_tensor *norm_weight,
                                               const h3_gpu_tensor *gate_modulation, const h3_gpu_tensor *norm_modulation,
                                               const h3_gpu_tensor *row_map, uint32_t rows, uint32_t padded_rows, uint32_t width,
                                               uint32_t slots, uint32_t gate_slot, uint32_t shift_slot, uint32_t scale_slot,
                                               float epsilon) {
    if (!launch_ready(g)) return 0;
    const size_t n = (size_t)rows * width;
    if (!rows || padded_rows < rows || !width || width > 24576 || !slots || gate_slot >= slots || shift_slot >= slots || scale_slot >= slots)
        return set_error(g, "gate/AdaLN/quantize: invalid shape or slot");
    if (!require(g, residual, H3_GPU_BF16, n, "gate residual") || !require(g, branch, H3_GPU_BF16, n, "gate branch") ||
        !require(g, gated_residual, H3_GPU_BF16, n, "gated residual") || !require(g, norm_weight, H3_GPU_BF16, width, "AdaLN norm weight") ||
        !require(g, gate_modulation, H3_GPU_BF16, (size_t)slots * width, "gate modulation") ||
        !require(g, norm_modulation, H3_GPU_BF16, (size_t)slots * width, "AdaLN modulation") ||
        !require(g, quantized_output, H3_GPU_I8, (size_t)padded_rows * width, "int8 quantized output") ||
        !require(g, quantized_scales, H3_GPU_F32, padded_rows, "int8 quantization scales") ||
        (row_map && !require(g, row_map, H3_GPU_U32, rows, "row map"))) return 0;
    const uint16_t *res_p = (const uint16_t *)pointer(residual), *branch_p = (const uint16_t *)pointer(branch);
    const uint16_t *gate_p = (const uint16_t *)pointer(gate_modulation), *norm_p = (const uint16_t *)pointer(norm_weight);
    const uint16_t *mod_p = (const uint16_t *)pointer(norm_modulation);
    const uint32_t *map_p = row_map ? (const uint32_t *)pointer(row_map) : nullptr;
    uint16_t *gated_p = (uint16_t *)pointer(gated_residual);
    int8_t *q_p = (int8_t *)pointer(quantized_output);
    float *s_p = (float *)pointer(quantized_scales);
    const uintptr_t alignment = (uintptr_t)res_p | (uintptr_t)branch_p | (uintptr_t)gate_p | (uintptr_t)norm_p | (uintptr_t)mod_p |
                                (uintptr_t)gated_p | (uintptr_t)q_p;
    /* rows of at most 6144 elements on 16-byte aligned operands: one warp per row, the row stays in registers */
    /* rows on 16-byte aligned operands: one warp per row, the row in that warp's shared memory */
    const size_t row_bytes = (size_t)4 * width * 2;
    if (width % 8 == 0 && row_bytes <= 200 * 1024 && (alignment & 15u) == 0) {
        static bool opted_in[64] = {};
        if (row_bytes > 48 * 1024 && !opted_in[g->device]) {
            if (!checked(g, cudaFuncSetAttribute(gate_adaln_quantize_warp_smem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024),
                         "shared memory opt-in")) return 0;
            opted_in[g->device] = true;
        }
        gate_adaln_quantize_warp_smem_kernel<<<(padded_rows + 3) / 4, 128, row_bytes, g->compute>>>(
            res_p, branch_p, gate_p, map_p, norm_p, mod_p, gated_p, q_p, s_p, rows, padded_rows, width, slots, gate_slot, shift_slot,
            scale_slot, epsilon, g->flags + 1);
    } else
        gate_adaln_quantize_kernel<<<padded_rows, 256, width * sizeof(uint16_t), g->compute>>>(
            res_p, branch_p, gate_p, map_p, norm_p, mod_p, gated_p, q_p, s_p, rows, width, slots, gate_slot, shift_slot, scale_slot, epsilon,
            g->flags + 1);
    count_launch(1);
    return launch_status(g, "gate/AdaLN/quantize", 1);
}

/* The fused projection on activations that are already int8 (from the call above or from
 * h3q8_quantize_rows): weight is a q8 descriptor with per-channel scales, or per-K-group
 * activation scales when input_group != 0 (input_scales is then [rows, K/input_group]). */
extern "C" int h3_gpu_linear_fused_int8_bf16(h3_gpu *g, h3_gpu_tensor *out, const h3_gpu_tensor *quantized_input,
                                             const h3_gpu_tensor *input_scales, uint32_t input_group, const h3_gpu_tensor *w,
                                             const h3_gpu_tensor *bias, const h3_gpu_tensor *gate, const h3_gpu_tensor *residual,
                                             uint32_t rows, uint32_t k, uint32_t n, int activation) {
    if (!launch_ready(g)) return 0;
    if (!rows || !k || !n || activation < 0 || activation > H3Q8_ACT_SWIGLU) return set_error(g, "int8 linear %ux%ux%u: invalid arguments", rows, n, k);
    const uint32_t wrows = activation == H3Q8_ACT_SWIGLU ? 2 * n : n;
    if (!w || w->owner != g || !w->q8 || w->q8_n != wrows || w->q8_k != k) return set_error(g, "int8 linear %ux%ux%u: needs a matching q8 weight", rows, n, k);
    if (input_group && k % input_group) return set_error(g, "int8 linear: K must be a multiple of the activation scale group");
    if (!require(g, quantized_input, H3_GPU_I8, (size_t)rows * k, "int8 linear input") ||
        !require(g, input_scales, H3_GPU_F32, (size_t)rows * (input_group ? k / input_group : 1), "int8 linear input scales") ||
        !require(g, out, H3_GPU_BF16, (size_t)rows * n, "int8 linear output") ||
        (bias && !require(g, bias, H3_GPU_BF16, wrows, "linear bias")) || (gate && !require(g, gate, H3_GPU_BF16, n, "linear gate")) ||
        (residual && !require(g, residual, H3_GPU_BF16, (size_t)rows * n, "linear residual"))) return 0;
    h3q8_linear_desc d = {};
    d.mode = H3Q8_MODE_W8A8; d.rows = rows; d.input_dim = k; d.output_dim = n; d.activation = (uint32_t)activation;
    d.input = pointer(quantized_input); d.input_scales = (const float *)pointer(input_scales); d.input_group = input_group;
    d.weight = pointer(w); d.weight_scales = (const float *)((const char *)w->data + w->q8_scale_offset); d.weight_group = w->q8_group;
    d.bias = bias ? (const uint16_t *)pointer(bias) : nullptr; d.gate = gate ? (const uint16_t *)pointer(gate) : nullptr;
    d.residual = residual ? (const uint16_t *)pointer(residual) : nullptr; d.output = (uint16_t *)pointer(out);
    {
        ProfileScope timing(g, 0);
        if (!h3q8_linear(&d, g->compute)) { g->accessed.clear(); return set_error(g, "%s", h3q8_last_error()); }
    }
    g->stats.linear_dispatches++;
    g->stats.q8_dispatches++;
    return launch_status(g, "int8 linear", 1);
}

/* ------------------------------------------- unfused epilogue operators */
static __global__ void gelu_kernel(const uint16_t *in, uint16_t *out, uint32_t count) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) out[i] = (uint16_t)f32_to_bf16_bits(gelu_tanh_f32(bf16_bits_to_f32(in[i])));
}
static __global__ void gate_kernel(const uint16_t *residual, const uint16_t *branch, const uint16_t *modulation, const uint32_t *row_map,
                            uint16_t *out, uint32_t rows, uint32_t width, uint32_t slots, uint32_t gate_slot) {
    uint32_t c = blockIdx.x * blockDim.x + threadIdx.x, r = blockIdx.y;
    if (c >= width || r >= rows) return;
    size_t base = (size_t)(row_map ? row_map[r] : 0) * slots * width;
    float gate = bf16_bits_to_f32(modulation[base + (size_t)gate_slot * width + c]);
    size_t i = (size_t)r * width + c;
    out[i] = (uint16_t)f32_to_bf16_bits(__fadd_rn(bf16_bits_to_f32(residual[i]), __fmul_rn(bf16_bits_to_f32(branch[i]), gate)));
}
static __global__ void add_kernel(const uint16_t *a, const uint16_t *b, uint16_t *out, uint32_t count) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) out[i] = (uint16_t)f32_to_bf16_bits(__fadd_rn(bf16_bits_to_f32(a[i]), bf16_bits_to_f32(b[i])));
}
extern "C" int h3_gpu_gelu_bf16(h3_gpu *g, h3_gpu_tensor *out, const h3_gpu_tensor *in, uint32_t elements, int approximate) {
    if (!launch_ready(g)) return 0;
    if (!approximate) return set_error(g, "only the tanh GELU is on this path");
    if (!elements || !require(g, in, H3_GPU_BF16, elements, "gelu input") || !require(g, out, H3_GPU_BF16, elements, "gelu output")) return 0;
    gelu_kernel<<<(elements + 255) / 256, 256, 0, g->compute>>>((const uint16_t *)pointer(in), (uint16_t *)pointer(out), elements);
    count_launch(1);
    return launch_status(g, "gelu", 1);
}
extern "C" int h3_gpu_gate_bf16(h3_gpu *g, h3_gpu_tensor *out, const h3_gpu_tensor *residual, const h3_gpu_tensor *branch,
                                const h3_gpu_tensor *modulation, const h3_gpu_tensor *row_map, uint32_t rows, uint32_t width,
                                uint32_t slots, uint32_t gate_slot) {
    if (!launch_ready(g)) return 0;
    size_t n = (size_t)rows * width;
    if (!rows || !width || !slots || gate_slot >= slots || rows > 65535 ||
        !require(g, residual, H3_GPU_BF16, n, "gate residual") || !require(g, branch, H3_GPU_BF16, n, "gate branch") ||
        !require(g, out, H3_GPU_BF16, n, "gate output") || !require(g, modulation, H3_GPU_BF16, (size_t)slots * width, "gate modulation") ||
        (row_map && !require(g, row_map, H3_GPU_U32, rows, "gate row map"))) return set_error(g, "gate: invalid arguments");
    gate_kernel<<<dim3((width + 255) / 256, rows), 256, 0, g->compute>>>(
        (const uint16_t *)pointer(residual), (const uint16_t *)pointer(branch), (const uint16_t *)pointer(modulation),
        row_map ? (const uint32_t *)pointer(row_map) : nullptr, (uint16_t *)pointer(out), rows, width, slots, gate_slot);
    count_launch(1);
    return launch_status(g, "gate", 1);
}
/* RMS norm with the AdaLN modulation, the producer of every block linear's input (src/cuda/cuda_kernels.cuh:936-971,
 * src/gpu.h:586-592): out = bf16(fma(x * rsqrt(mean(x^2) + eps) * weight, 1 + scale[class], shift[class])).  One
 * 256-thread CTA per row; lane t sums columns t, t + 256, ... in order with fma and the lanes are combined by the
 * reference's halving tree, so the mean has the reference's bits. */
static __global__ void __launch_bounds__(256) adaln_rows_kernel(const uint16_t *__restrict__ input, const uint16_t *__restrict__ norm_weight,
                                                               const uint16_t *__restrict__ modulation, const uint32_t *__restrict__ row_map,
                                                               uint16_t *__restrict__ output, uint32_t width, uint32_t slots,
                                                               uint32_t shift_slot, uint32_t scale_slot, float epsilon) {
    __shared__ float lanes[256];
    const uint32_t row = blockIdx.x, tid = threadIdx.x;
    const uint16_t *x = input + (size_t)row * width;
    float sum = 0.0f;
    for (uint32_t c = tid; c < width; c += 256) {
        const float v = bf16_bits_to_f32(x[c]);
        sum = fmaf(v, v, sum);
    }
    lanes[tid] = sum;
    __syncthreads();
    for (uint32_t stride = 128; stride; stride >>= 1) {
        if (tid < stride) lanes[tid] = __fadd_rn(lanes[tid], lanes[tid + stride]);
        __syncthreads();
    }
    const float inverse = rsqrtf(__fadd_rn(__fdiv_rn(lanes[0], (float)width), epsilon));
    const size_t base = (size_t)(row_map ? row_map[row] : 0) * slots * width;
    const uint16_t *shift = modulation + base + (size_t)shift_slot * width, *scale = modulation + base + (size_t)scale_slot * width;
    for (uint32_t c = tid; c < width; c += 256) {
        const float normalized = __fmul_rn(__fmul_rn(bf16_bits_to_f32(x[c]), inverse), bf16_bits_to_f32(norm_weight[c]));
        output[(size_t)row * width + c] = (uint16_t)f32_to_bf16_bits(fmaf(normalized, __fadd_rn(1.0f, bf16_bits_to_f32(scale[c])), bf16_bits_to_f32(shift[c])));
    }
}
extern "C" int h3_gpu_adaln_bf16(h3_gpu *g, h3_gpu_tensor *out, const h3_gpu_tensor *in, const h3_gpu_tensor *norm_weight,
                                 const h3_gpu_tensor *modulation, const h3_gpu_tensor *row_map, uint32_t rows, uint32_t width,
                                 uint32_t slots, uint32_t shift_slot, uint32_t scale_slot, float epsilon) {
    if (!launch_ready(g)) return 0;
    const size_t n = (size_t)rows * width;
    if (!rows || !width || !slots || shift_slot >= slots || scale_slot >= slots) return set_error(g, "AdaLN: invalid arguments");
    if (!require(g, in, H3_GPU_BF16, n, "AdaLN input") || !require(g, out, H3_GPU_BF16, n, "AdaLN output") ||
        !require(g, norm_weight, H3_GPU_BF16, width, "AdaLN norm weight") ||
        !require(g, modulation, H3_GPU_BF16, (size_t)slots * width, "AdaLN modulation") ||
        (row_map && !require(g, row_map, H3_GPU_U32, rows, "AdaLN row map"))) return 0;
    adaln_rows_kernel<<<rows, 256, 0, g->compute>>>((const uint16_t *)pointer(in), (const uint16_t *)pointer(norm_weight),
                                                     (const uint16_t *)pointer(modulation), row_map ? (const uint32_t *)pointer(row_map) : nullptr,
                                                     (uint16_t *)pointer(out), width, slots, shift_slot, scale_slot, epsilon);
    count_launch(1);
    return launch_status(g, "AdaLN", 1);
}
/* src/gpu.h:618-629; on CUDA the reference composes the two operators (src/cuda/gpu_cuda.cu:1118-1120) and so does this. */
extern "C" int h3_gpu_gate_adaln_bf16(h3_gpu *g, h3_gpu_tensor *gated_residual, h3_gpu_tensor *out, const h3_gpu_tensor *residual,
                                      const h3_gpu_tensor *branch, const h3_gpu_tensor *norm_weight, const h3_gpu_tensor *gate_modulation,
                                      const h3_gpu_tensor *norm_modulation, const h3_gpu_tensor *row_map, uint32_t rows, uint32_t width,
                                      uint32_t slots, uint32_t gate_slot, uint32_t shift_slot, uint32_t scale_slot, float epsilon) {
    return h3_gpu_gate_bf16(g, gated_residual, residual, branch, gate_modulation, row_map, rows, width, slots, gate_slot) &&
           h3_gpu_adaln_bf16(g, out, gated_residual, norm_weight, norm_modulation, row_map, rows, width, slots, shift_slot, scale_slot, epsilon);
}
/* src/gpu.h:506-511: fc1 over the [gate | up] weight with SwiGLU in its epilogue, then fc2 (weights: bf16 or q8 descriptors). */
extern "C" int h3_gpu_mlp_bf16(h3_gpu *g, h3_gpu_tensor *out, const h3_gpu_tensor *in, const h3_gpu_tensor *fc1, const h3_gpu_tensor *fc2,
                               uint32_t rows, uint32_t input_dim, uint32_t hidden_dim, uint32_t output_dim) {
    if (!launch_ready(g)) return 0;
    h3_gpu_tensor *activated = h3_gpu_tensor_new_bf16(g, (size_t)rows * hidden_dim);
    if (!activated) return 0;
    const int ok = linear_dispatch(g, activated, in, fc1, nullptr, nullptr, nullptr, rows, input_dim, hidden_dim, H3Q8_ACT_SWIGLU) &&
                   linear_dispatch(g, out, activated, fc2, nullptr, nullptr, nullptr, rows, hidden_dim, output_dim, H3Q8_ACT_NONE);
    h3_gpu_tensor_free(activated);   /* legal with work in flight: the release waits for it */
    return ok;
}
/* src/cuda/cuda_kernels.cuh:988-1045 with grouped = 1: one thread per (row, head, dimension);
 * every thread accumulates the head's squares in dimension order like the reference. */
static __global__ void __launch_bounds__(128) grouped_qkv_rope_kernel(const uint16_t *__restrict__ qkv, const uint16_t *__restrict__ q_weight,
                                                                     const uint16_t *__restrict__ k_weight, const uint16_t *__restrict__ rope_cos,
                                                                     const uint16_t *__restrict__ rope_sin, uint16_t *query, uint16_t *key,
                                                                     uint16_t *value, uint32_t heads, uint32_t head_dim, uint32_t rope_half,
                                                                     float epsilon) {
    const uint32_t row = blockIdx.y, head = blockIdx.x;
    const size_t q_base = ((size_t)row * heads + head) * head_dim * 3, k_base = q_base + head_dim, v_base = k_base + head_dim;
    float q_sum = 0.0f, k_sum = 0.0f;
    for (uint32_t d = 0; d < head_dim; d++) {
        const float q = bf16_bits_to_f32(qkv[q_base + d]), k = bf16_bits_to_f32(qkv[k_base + d]);
        q_sum = fmaf(q, q, q_sum);
        k_sum = fmaf(k, k, k_sum);
    }
    const float q_inverse = rsqrtf(__fadd_rn(__fdiv_rn(q_sum, (float)head_dim), epsilon));
    const float k_inverse = rsqrtf(__fadd_rn(__fdiv_rn(k_sum, (float)head_dim), epsilon));
    for (uint32_t d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float q0 = __fmul_rn(__fmul_rn(bf16_bits_to_f32(qkv[q_base + d]), q_inverse), bf16_bits_to_f32(q_weight[d]));
        float k0 = __fmul_rn(__fmul_rn(bf16_bits_to_f32(qkv[k_base + d]), k_inverse), bf16_bits_to_f32(k_weight[d]));
        if (d < 2 * rope_half) {
            const bool low = d < rope_half;
            const uint32_t pair = low ? d + rope_half : d - rope_half, first = low ? d : pair;
            const float q1 = __fmul_rn(__fmul_rn(bf16_bits_to_f32(qkv[q_base + pair]), q_inverse), bf16_bits_to_f32(q_weight[pair]));
            const float k1 = __fmul_rn(__fmul_rn(bf16_bits_to_f32(qkv[k_base + pair]), k_inverse), bf16_bits_to_f32(k_weight[pair]));
            const float c = bf16_bits_to_f32(rope_cos[(size_t)row * rope_half + first]), s = bf16_bits_to_f32(rope_sin[(size_t)row * rope_half + first]);
            q0 = low ? __fsub_rn(__fmul_rn(q0, c), __fmul_rn(q1, s)) : __fadd_rn(__fmul_rn(q0, c), __fmul_rn(q1, s));
            k0 = low ? __fsub_rn(__fmul_rn(k0, c), __fmul_rn(k1, s)) : __fadd_rn(__fmul_rn(k0, c), __fmul_rn(k1, s));
        }
        const size_t o = ((size_t)row * heads + head) * head_dim + d;
        query[o] = (uint16_t)f32_to_bf16_bits(q0);
        key[o] = (uint16_t)f32_to_bf16_bits(k0);
        value[o] = qkv[v_base + d];
    }
}
static int rope_operands(h3_gpu *g, const h3_gpu_tensor *q, const h3_gpu_tensor *k, const h3_gpu_tensor *v, const h3_gpu_tensor *qw,
                         const h3_gpu_tensor *kw, const h3_gpu_tensor *c, const h3_gpu_tensor *s, uint32_t rows, uint32_t heads,
                         uint32_t dim, uint32_t half) {
    const size_t count = (size_t)rows * heads * dim;
    if (!rows || !heads || !dim || half * 2 > dim || rows > 65535u * 64u) return set_error(g, "QKV norm/RoPE: invalid shape");
    return require(g, q, H3_GPU_BF16, count, "Q") && require(g, k, H3_GPU_BF16, count, "K") && require(g, v, H3_GPU_BF16, count, "V") &&
           require(g, qw, H3_GPU_BF16, dim, "Q norm") && require(g, kw, H3_GPU_BF16, dim, "K norm") &&
           require(g, c, H3_GPU_BF16, (size_t)rows * half, "RoPE cos") && require(g, s, H3_GPU_BF16, (size_t)rows * half, "RoPE sin");
}
extern "C" int h3_gpu_grouped_qkv_rope_bf16(h3_gpu *g, h3_gpu_tensor *q, h3_gpu_tensor *k, h3_gpu_tensor *v, const h3_gpu_tensor *qkv,
                                            const h3_gpu_tensor *qw, const h3_gpu_tensor *kw, const h3_gpu_tensor *c, const h3_gpu_tensor *s,
                                            uint32_t rows, uint32_t heads, uint32_t dim, uint32_t half, float epsilon) {
    if (!launch_ready(g)) return 0;
    if (!rope_operands(g, q, k, v, qw, kw, c, s, rows, heads, dim, half) ||
        !require(g, qkv, H3_GPU_BF16, (size_t)rows * heads * dim * 3, "QKV")) return 0;
    if (rows > 65535) return set_error(g, "QKV norm/RoPE: at most 65535 rows per call");
    grouped_qkv_rope_kernel<<<dim3(heads, rows), 128, 0, g->compute>>>(
        (const uint16_t *)pointer(qkv), (const uint16_t *)pointer(qw), (const uint16_t *)pointer(kw), (const uint16_t *)pointer(c),
        (const uint16_t *)pointer(s), (uint16_t *)pointer(q), (uint16_t *)pointer(k), (uint16_t *)pointer(v), heads, dim, half, epsilon);
    count_launch(1);
    return launch_status(g, "QKV norm/RoPE", 1);
}
extern "C" int h3_gpu_grouped_qkv_linear_rope_bf16(h3_gpu *g, h3_gpu_tensor *q, h3_gpu_tensor *k, h3_gpu_tensor *v, h3_gpu_tensor *qkv,
                                                   const h3_gpu_tensor *input, const h3_gpu_tensor *w, const h3_gpu_tensor *qw,
                                                   const h3_gpu_tensor *kw, const h3_gpu_tensor *c, const h3_gpu_tensor *s, uint32_t rows,
                                                   uint32_t width, uint32_t heads, uint32_t dim, uint32_t half, float epsilon) {
    if (!launch_ready(g)) return 0;
    if (!rope_operands(g, q, k, v, qw, kw, c, s, rows, heads, dim, half)) return 0;
    const uint32_t n = heads * dim * 3;
    /* one kernel when the epilogue can hold a head row: head_dim 128, rotary half 48 or 64, operands the two-CTA kernel takes */
    const bool grouped_scales = w && w->q8 && g->quant_mode == 2 && w->q8_group;
    const bool fusable = dim == 128 && (half == 48 || half == 64) && width % 16 == 0 && rows > 0 && !grouped_scales &&
                         (!w || !w->q8 || g->quant_mode == 2 || g->w8a16_scratch_rows);
    if (fusable) {
        h3q8_rope_desc rope = {(const uint16_t *)pointer(qw), (const uint16_t *)pointer(kw), (const uint16_t *)pointer(c),
                               (const uint16_t *)pointer(s), (uint16_t *)pointer(q), (uint16_t *)pointer(k), (uint16_t *)pointer(v),
                               heads, dim, half, epsilon};
        h3_gpu_linear_problem problem = {qkv, input, w, nullptr, nullptr, nullptr, rows, width, n, H3Q8_ACT_NONE};
        const int saved = g->w8a16_scratch_rows;
        if (w && w->q8 && g->quant_mode != 2) g->w8a16_scratch_rows = 1; /* the fused epilogue wants bf16 operands */
        int ok = linear_dispatch_many(g, &problem, 1, &rope);
        g->w8a16_scratch_rows = saved;
        return ok;
    }
    if (!qkv) return set_error(g, "QKV projection: this shape needs the qkv tensor for the unfused route");
    return h3_gpu_linear_bf16(g, qkv, input, w, nullptr, rows, width, n) &&
           h3_gpu_grouped_qkv_rope_bf16(g, q, k, v, qkv, qw, kw, c, s, rows, heads, dim, half, epsilon);
}

/* ----------------------------------------------- the int8 operator family */
/* One W8A8 projection on int8 activations and a separate int8 weight + fp32 per-channel scale tensor pair
 * (the layout of the reference's int8 family, src/gpu.h:521-563): optional SwiGLU (weight rows [gate n | up n]),
 * per-K-group activation scales, or the QKV norm + rotary epilogue. */
static int int8_projection(h3_gpu *g, const h3_gpu_tensor *q_in, const h3_gpu_tensor *in_scales, uint32_t input_group,
                           const h3_gpu_tensor *w, const h3_gpu_tensor *w_scales, h3_gpu_tensor *out, uint32_t rows, uint32_t k,
                           uint32_t n, uint32_t activation, const h3q8_rope_desc *rope, const char *what) {
    h3q8_linear_desc d = {};
    d.mode = H3Q8_MODE_W8A8; d.rows = rows; d.input_dim = k; d.output_dim = n; d.activation = activation;
    d.input = pointer(q_in); d.input_scales = (const float *)pointer(in_scales); d.input_group = input_group;
    d.weight = pointer(w); d.weight_scales = (const float *)pointer(w_scales);
    d.output = out ? (uint16_t *)pointer(out) : nullptr;
    d.rope = rope;
    {
        ProfileScope timing(g, 0);
        if (!h3q8_linear(&d, g->compute)) { g->accessed.clear(); return set_error(g, "%s: %s", what, h3q8_last_error()); }
    }
    g->stats.linear_dispatches++;
    return 1;
}

/* Per-row int8 of a [head, row, dimension] bf16 tensor gathered into row-major [row, head * dimension]
 * (src/gpu.h:536-546: the projection after attention reads SDPA's native layout without a bf16 transpose). */
static __global__ void __launch_bounds__(256) quantize_rows_head_major_kernel(const uint16_t *__restrict__ in, int8_t *__restrict__ out,
                                                                       float *__restrict__ scales, uint32_t rows, uint32_t heads,
                                                                       uint32_t head_dim, uint32_t *nonfinite) {
    __shared__ uint32_t scratch[8];
    const uint32_t row = blockIdx.x, columns = heads * head_dim, vectors = columns / 8;
    uint2 *q = reinterpret_cast<uint2 *>(out + (size_t)row * columns);
    if (row >= rows) {
        for (uint32_t c = threadIdx.x; c < vectors; c += 256) q[c] = make_uint2(0, 0);
        if (threadIdx.x == 0) scales[row] = 1.0f;
        return;
    }
    auto vector = [&](uint32_t c) {
        const uint32_t column = c * 8, head = column / head_dim, inside = column - head * head_dim;
        return *reinterpret_cast<const uint4 *>(in + ((size_t)head * rows + row) * head_dim + inside);
    };
    uint32_t peak_bits = 0;
    for (uint32_t c = threadIdx.x; c < vectors; c += 256) {
        const uint4 v = vector(c);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; j++) peak_bits = absmax2(peak_bits, w[j]);
    }
    peak_bits = block_max_256_u32(absmax_fold(peak_bits), scratch);
    const float peak = bf16_bits_to_f32(peak_bits);
    const float scale = peak > 0.0f ? __fdiv_rn(peak, 127.0f) : __fdiv_rn(1.0f, 127.0f);
    const float inverse = peak > 0.0f ? __fdiv_rn(127.0f, peak) : 127.0f;
    if (threadIdx.x == 0) {
        scales[row] = scale;
        if (absmax_nonfinite(peak_bits) && nonfinite) atomicOr(nonfinite, STATUS_NONFINITE);
    }
    for (uint32_t c = threadIdx.x; c < vectors; c += 256) {
        const uint4 v = vector(c);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t o[2] = {0, 0};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            uint32_t lo = (uint32_t)quantize_one(bf16_lo(w[j]), inverse) & 0xffu, hi = (uint32_t)quantize_one(bf16_hi(w[j]), inverse) & 0xffu;
            o[j >> 1] |= (lo | (hi << 8)) << ((j & 1) * 16);
        }
        q[c] = make_uint2(o[0], o[1]);
    }
}

extern "C" int h3_gpu_linear_int8_head_major_bf16(h3_gpu *g, h3_gpu_tensor *out, h3_gpu_tensor *qin, h3_gpu_tensor *in_scales,
                                                  const h3_gpu_tensor *in, const h3_gpu_tensor *w, const h3_gpu_tensor *w_scales,
                                                  uint32_t rows, uint32_t heads, uint32_t head_dim, uint32_t n) {
    if (!launch_ready(g)) return 0;
    const uint32_t k = heads * head_dim, padded = (rows + 127u) & ~127u;
    if (rows < 128 || !heads || !head_dim || head_dim % 8 || k % 128 || n % 128)
        return set_error(g, "int8 head-major linear needs rows >= 128, head_dim %% 8 == 0 and K, N multiples of 128");
    if (!require(g, w, H3_GPU_I8, (size_t)n * k, "int8 linear weight") || !require(g, w_scales, H3_GPU_F32, n, "int8 linear weight scales") ||
        !require(g, out, H3_GPU_BF16, (size_t)rows * n, "int8 linear output") || !require(g, in, H3_GPU_BF16, (size_t)rows * k, "int8 linear input") ||
        !require(g, qin, H3_GPU_I8, (size_t)padded * k, "int8 quantized output") ||
        !require(g, in_scales, H3_GPU_F32, padded, "int8 quantization scales")) return 0;
    {
        ProfileScope timing(g, 7);
        quantize_rows_head_major_kernel<<<padded, 256, 0, g->compute>>>((const uint16_t *)pointer(in), (int8_t *)pointer(qin),
                                                                        (float *)pointer(in_scales), rows, heads, head_dim, g->flags + 1);
    }
    count_launch(1);
    if (!int8_projection(g, qin, in_scales, 0, w, w_scales, out, rows, k, n, H3Q8_ACT_NONE, nullptr, "int8 head-major linear")) return 0;
    return launch_status(g, "int8 head-major linear", 2);
}

/* src/gpu.h:547-563, src/metal/gpu.m:3281-3490: the block's MLP on int8 tensor cores.  fc1 + SwiGLU reads the
 * per-row quantised input (quantised here unless the caller's gate/AdaLN pass already did), `activated` is stored as
 * bf16, re-quantised per row and per 1024 hidden features (or per row with use_int8_row_fc2) and fed to fc2.
 * The diagnostic bf16 stages of the reference (H3_INT8_MLP_STAGE, the fc1_bf16 / fc2_bf16 weights) are not part of
 * this path; the slower-variant switches select equal results there and are accepted and ignored. */
extern "C" int h3_gpu_mlp_int8_bf16(h3_gpu *g, h3_gpu_tensor *out, h3_gpu_tensor *activated, h3_gpu_tensor *q_act, h3_gpu_tensor *act_scales,
                                    const h3_gpu_tensor *in, const h3_gpu_tensor *fc1_w, const h3_gpu_tensor *fc1_s,
                                    const h3_gpu_tensor *fc2_w, const h3_gpu_tensor *fc2_s, const h3_gpu_tensor *, const h3_gpu_tensor *,
                                    uint32_t rows, uint32_t k, uint32_t hidden, uint32_t n, int, int, int use_int8_row_fc2,
                                    int input_is_quantized) {
    if (!launch_ready(g)) return 0;
    if (getenv("H3_INT8_MLP_STAGE")) return set_error(g, "int8 MLP: the diagnostic bf16 stages are not available on this backend");
    const uint32_t padded = (rows + 127u) & ~127u, groups = hidden / 1024u;
    if (rows < 128 || k % 128 || hidden % 128 || n % 128 || (!use_int8_row_fc2 && hidden % 1024))
        return set_error(g, "int8 MLP needs rows >= 128, dimensions that are multiples of 128 and a hidden width that is a multiple of 1024");
    const size_t capacity = (size_t)padded * (k > hidden ? k : hidden);
    if (!require(g, q_act, H3_GPU_I8, capacity, "int8 MLP activation") ||
        !require(g, act_scales, H3_GPU_F32, (size_t)padded * (groups ? groups : 1u), "int8 MLP activation scales") ||
        !require(g, fc1_w, H3_GPU_I8, (size_t)hidden * 2 * k, "int8 MLP FC1 weight") || !require(g, fc1_s, H3_GPU_F32, (size_t)hidden * 2, "int8 MLP FC1 scales") ||
        !require(g, fc2_w, H3_GPU_I8, (size_t)n * hidden, "int8 MLP FC2 weight") || !require(g, fc2_s, H3_GPU_F32, n, "int8 MLP FC2 scales") ||
        (!input_is_quantized && !require(g, in, H3_GPU_BF16, (size_t)rows * k, "int8 MLP input")) ||
        !require(g, activated, H3_GPU_BF16, (size_t)rows * hidden, "int8 MLP activated") ||
        !require(g, out, H3_GPU_BF16, (size_t)rows * n, "int8 MLP output")) return 0;
    unsigned launched = 0;
    const float clip = mlp_activation_clip();   /* the MLP's row quantisers only; the per-1024 one has no clip (gpu.m:3405-3451) */
    if (!input_is_quantized) {
        ProfileScope timing(g, 7);
        quantise_activations(g, (const uint16_t *)pointer(in), (int8_t *)pointer(q_act), (float *)pointer(act_scales), rows, padded, k, clip);
        count_launch(1);
        launched++;
    }
    if (!int8_projection(g, q_act, act_scales, 0, fc1_w, fc1_s, activated, rows, k, hidden, H3Q8_ACT_SWIGLU, nullptr, "int8 MLP FC1")) return 0;
    {
        ProfileScope timing(g, 7);
        if (use_int8_row_fc2)
            quantise_activations(g, (const uint16_t *)pointer(activated), (int8_t *)pointer(q_act), (float *)pointer(act_scales), rows, padded, hidden,
                                 clip);
        else  /* every (row, 1024-feature group) is a segment of the same contiguous matrix */
            quantise_activations(g, (const uint16_t *)pointer(activated), (int8_t *)pointer(q_act), (float *)pointer(act_scales),
                                 (uint64_t)rows * groups, (uint64_t)padded * groups, 1024, 1.0f);
        count_launch(1);
        launched++;
    }
    if (!int8_projection(g, q_act, act_scales, use_int8_row_fc2 ? 0u : 1024u, fc2_w, fc2_s, out, rows, hidden, n, H3Q8_ACT_NONE, nullptr,
                         "int8 MLP FC2")) return 0;
    return launch_status(g, "int8 MLP", launched + 2);
}

/* src/gpu.h:682-702: QKV projection on int8 tensor cores with the per-head RMS norm and rotary embedding in the
 * epilogue.  The input is quantised per row here unless the caller's gate/AdaLN pass already did.  The slower-variant
 * switches select equal results in the reference and are accepted and ignored. */
extern "C" int h3_gpu_grouped_qkv_linear_rope_int8(h3_gpu *g, h3_gpu_tensor *q, h3_gpu_tensor *k, h3_gpu_tensor *v, h3_gpu_tensor *qin,
                                                   h3_gpu_tensor *in_scales, const h3_gpu_tensor *in, const h3_gpu_tensor *w,
                                                   const h3_gpu_tensor *w_scales, const h3_gpu_tensor *qw, const h3_gpu_tensor *kw,
                                                   const h3_gpu_tensor *c, const h3_gpu_tensor *s, uint32_t rows, uint32_t width,
                                                   uint32_t heads, uint32_t dim, uint32_t half, float epsilon, int input_is_quantized,
                                                   int, int, int) {
    if (!launch_ready(g)) return 0;
    if (!rope_operands(g, q, k, v, qw, kw, c, s, rows, heads, dim, half)) return 0;
    const uint32_t n = heads * dim * 3, padded = (rows + 127u) & ~127u;
    if (rows < 128 || width % 128 || dim != 128 || (half != 48 && half != 64))
        return set_error(g, "int8 QKV projection needs rows >= 128, K %% 128 == 0, head_dim 128 and rope_half 48 or 64");
    if (!require(g, w, H3_GPU_I8, (size_t)n * width, "int8 QKV weight") || !require(g, w_scales, H3_GPU_F32, n, "int8 QKV weight scales") ||
        !require(g, qin, H3_GPU_I8, (size_t)padded * width, "int8 QKV quantized input") ||
        !require(g, in_scales, H3_GPU_F32, padded, "int8 QKV input scales") ||
        (!input_is_quantized && !require(g, in, H3_GPU_BF16, (size_t)rows * width, "int8 QKV input"))) return 0;
    unsigned launched = 1;
    if (!input_is_quantized) {
        ProfileScope timing(g, 7);
        quantise_activations(g, (const uint16_t *)pointer(in), (int8_t *)pointer(qin), (float *)pointer(in_scales), rows, padded, width, 1.0f);
        count_launch(1);
        launched++;
    }
    h3q8_rope_desc rope = {(const uint16_t *)pointer(qw), (const uint16_t *)pointer(kw), (const uint16_t *)pointer(c),
                           (const uint16_t *)pointer(s), (uint16_t *)pointer(q), (uint16_t *)pointer(k), (uint16_t *)pointer(v),
                           heads, dim, half, epsilon};
    if (!int8_projection(g, qin, in_scales, 0, w, w_scales, nullptr, rows, width, n, H3Q8_ACT_NONE, &rope, "int8 QKV projection")) return 0;
    return launch_status(g, "int8 QKV projection", launched);
}

/* src/gpu.h:714-716, src/cuda/cuda_kernels.cuh:1047-1059: fused row = [gate width | up width] */
static __global__ void swiglu_kernel(const uint16_t *fused, uint16_t *out, uint32_t rows, uint32_t width) {
    uint32_t c = blockIdx.x * blockDim.x + threadIdx.x, r = blockIdx.y;
    if (c >= width || r >= rows) return;
    size_t base = (size_t)r * width * 2;
    out[(size_t)r * width + c] = (uint16_t)f32_to_bf16_bits(swiglu_f32(bf16_bits_to_f32(fused[base + c]), bf16_bits_to_f32(fused[base + width + c]), true));
}
extern "C" int h3_gpu_swiglu_bf16(h3_gpu *g, h3_gpu_tensor *out, const h3_gpu_tensor *fused, uint32_t rows, uint32_t width) {
    if (!launch_ready(g)) return 0;
    if (!rows || !width || rows > 65535 || !require(g, fused, H3_GPU_BF16, (size_t)rows * width * 2, "swiglu input") ||
        !require(g, out, H3_GPU_BF16, (size_t)rows * width, "swiglu output")) return set_error(g, "swiglu: invalid arguments");
    swiglu_kernel<<<dim3((width + 255) / 256, rows), 256, 0, g->compute>>>((const uint16_t *)pointer(fused), (uint16_t *)pointer(out), rows, width);
    count_launch(1);
    return launch_status(g, "swiglu", 1);
}
extern "C" int h3_gpu_add_bf16(h3_gpu *g, h3_gpu_tensor *out, const h3_gpu_tensor *a, const h3_gpu_tensor *b, uint32_t elements) {
    if (!launch_ready(g)) return 0;
    if (!elements || !require(g, a, H3_GPU_BF16, elements, "add left") || !require(g, b, H3_GPU_BF16, elements, "add right") ||
        !require(g, out, H3_GPU_BF16, elements, "add output")) return 0;
    add_kernel<<<(elements + 255) / 256, 256, 0, g->compute>>>((const uint16_t *)pointer(a), (const uint16_t *)pointer(b), (uint16_t *)pointer(out), elements);
    count_launch(1);
    return launch_status(g, "add", 1);
}
