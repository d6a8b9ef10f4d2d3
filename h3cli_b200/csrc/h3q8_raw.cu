/* Raw C entry points of libh3q8: validation, kernel selection, TMA descriptor
 * construction and launches.  Device pointers in, work enqueued on the caller's
 * stream, nothing allocated per call (one 4-byte status word per device is
 * allocated on first use).  See include/h3q8.h for the contract. */
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <cstdlib>
#include <mutex>

#include "h3q8.h"
#include "h3q8_internal.h"
#include "gemm_tcgen05_skinny.cuh"
#include "kernels_misc.cuh"

namespace h3q8 {

static thread_local char last_error[512];
static std::atomic<uint64_t> launches{0};
/* host-side fault injection for the failure-path tests (h3q8_fault_injection) */
static std::atomic<long long> injected_wait_limit{0};
static std::atomic<uint32_t> injected_skip_first_load{0};

int fail(const char *format, ...) {
    va_list args;
    va_start(args, format);
    vsnprintf(last_error, sizeof last_error, format, args);
    va_end(args);
    return 0;
}
void count_launch(unsigned n) { launches.fetch_add(n, std::memory_order_relaxed); }

static int cuda_ok(cudaError_t e, const char *what) {
    return e == cudaSuccess ? 1 : fail("CUDA %s: %s", what, cudaGetErrorString(e));
}

/* ------------------------------------------------------------ per-device state */
struct DeviceState {
    bool ready = false;
    int sms = 0;
    uint32_t *status = nullptr;
};
static DeviceState devices[64];
static std::mutex device_mutex;
typedef CUresult (*encode_tiled_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static encode_tiled_fn encode_tiled = nullptr;

static DeviceState *device_state() {
    int device = 0;
    if (!cuda_ok(cudaGetDevice(&device), "get device")) return nullptr;
    if (device < 0 || device >= 64) { fail("device index %d out of range", device); return nullptr; }
    std::lock_guard<std::mutex> lock(device_mutex);
    DeviceState &d = devices[device];
    if (d.ready) return &d;
    cudaDeviceProp prop;
    if (!cuda_ok(cudaGetDeviceProperties(&prop, device), "device properties")) return nullptr;
    if (prop.major != 10) {
        fail("libh3q8 needs an sm_100 GPU (B200); device %d is sm_%d%d", device, prop.major, prop.minor);
        return nullptr;
    }
    d.sms = prop.multiProcessorCount;
    if (!cuda_ok(cudaMalloc(&d.status, sizeof(uint32_t)), "status word") ||
        !cuda_ok(cudaMemset(d.status, 0, sizeof(uint32_t)), "status word clear")) return nullptr;
    if (!encode_tiled) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (!cuda_ok(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &result), "driver entry point") ||
            result != cudaDriverEntryPointSuccess || !fn) {
            fail("cuTensorMapEncodeTiled is not available from this driver");
            return nullptr;
        }
        encode_tiled = (encode_tiled_fn)fn;
    }
    d.ready = true;
    return &d;
}

uint32_t *device_status_word() {
    DeviceState *d = device_state();
    return d ? d->status : nullptr;
}

/* 2-D row-major [rows, columns] tensor, box = [box_rows, box_bytes worth of columns] */
static int make_map(CUtensorMap *map, const void *base, uint32_t element_bytes, uint64_t rows, uint64_t columns,
                    uint32_t box_columns, uint32_t box_rows, CUtensorMapSwizzle swizzle) {
    cuuint64_t dims[2] = {columns, rows};
    cuuint64_t strides[1] = {columns * element_bytes};
    cuuint32_t box[2] = {box_columns, box_rows};
    cuuint32_t element_strides[2] = {1, 1};
    CUresult r = encode_tiled(map, element_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                              const_cast<void *>(base), dims, strides, box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 1 : fail("cuTensorMapEncodeTiled failed (%d) for a %llu x %llu tensor", (int)r,
                                        (unsigned long long)rows, (unsigned long long)columns);
}

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

/* ------------------------------------------------------------------ launches */
template <int MODE, int BN, int MT, bool GROUPED>
static int launch_tcgen05(const h3q8_linear_desc &d, GemmParams p, DeviceState *dev, cudaStream_t stream) {
    using C = GemmConfig<MODE, BN, MT, GROUPED>;
    CUtensorMap map_a, map_b;
    const uint32_t a_bytes = MODE == MODE_W8A8 ? 1 : 2, b_bytes = MODE == MODE_BF16 ? 2 : 1;
    if (!make_map(&map_a, d.input, a_bytes, d.rows, d.input_dim, C::BKE, 128, CU_TENSOR_MAP_SWIZZLE_128B)) return 0;
    if (!make_map(&map_b, d.weight, b_bytes, d.output_dim, d.input_dim, C::BKE, BN,
                  MODE == MODE_W8A16 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B)) return 0;
    p.m_blocks = (d.rows + C::BM - 1) / C::BM;
    p.n_blocks = (d.output_dim + BN - 1) / BN;
    p.tiles = p.m_blocks * p.n_blocks;
    p.band = p.m_blocks < 16 ? p.m_blocks : 16;
    auto kernel = gemm_tcgen05_kernel<MODE, BN, MT, GROUPED>;
    static bool configured[64] = {};
    int device = 0;
    cudaGetDevice(&device);
    if (!configured[device]) {
        if (!cuda_ok(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES),
                     "shared memory opt-in")) return 0;
        configured[device] = true;
    }
    const uint32_t grid = p.tiles < (uint32_t)dev->sms ? p.tiles : (uint32_t)dev->sms;
    kernel<<<grid, C::THREADS, C::SMEM_BYTES, stream>>>(map_a, map_b, p);
    count_launch(1);
    return cuda_ok(cudaGetLastError(), "tcgen05 linear launch");
}

/* Two-CTA clusters: the grid is twice the number of clusters that can be resident at once. */
/* `count` problems (1..PAIR_MAX_PROBLEMS) of one operand mode in ONE launch. */
template <int MODE, bool ROPE, int EPILOGUE_WARPS>
static int launch_pair_with(const h3q8_linear_desc *descs, const GemmParams *params, uint32_t count, DeviceState *dev, cudaStream_t stream) {
    using C = PairConfig<MODE, ROPE, EPILOGUE_WARPS>;
    static_assert(sizeof(PairArgs) <= 4000, "kernel parameter block too large");
    PairArgs args;
    memset(&args, 0, sizeof args);
    args.count = count;
    const uint32_t bytes = MODE == MODE_W8A8 ? 1 : 2;
    uint32_t tiles = 0;
    for (uint32_t i = 0; i < count; i++) {
        const h3q8_linear_desc &d = descs[i];
        GemmParams &p = args.p[i];
        p = params[i];
        if (!make_map(&args.map_a[i], d.input, bytes, d.rows, d.input_dim, C::BKE, 128, CU_TENSOR_MAP_SWIZZLE_128B)) return 0;
        const bool swiglu = d.activation == H3Q8_ACT_SWIGLU; /* weight rows [gate N | up N], 128 outputs per tile */
        if (!make_map(&args.map_b[i], d.weight, bytes, (uint64_t)d.output_dim * (swiglu ? 2 : 1), d.input_dim, C::BKE, 128,
                      CU_TENSOR_MAP_SWIZZLE_128B)) return 0;
        p.m_blocks = (d.rows + C::BM - 1) / C::BM;
        p.n_blocks = swiglu ? (d.output_dim + 127) / 128 : (d.output_dim + C::BN - 1) / C::BN;
        p.tiles = p.m_blocks * p.n_blocks;
        /* measured: bands of 16 row blocks are best while a 256-row block of X is small (K*bytes <= 8 KB per row),
         * 8 beyond that (FFN-down); L2 eviction hints (activations first, weights last) lost 3-5 % everywhere */
        const uint32_t band = (uint64_t)d.input_dim * bytes <= 8192 ? 16 : 8;
        p.band = p.m_blocks < band ? p.m_blocks : band;
        p.l2_policy_a = L2_EVICT_NORMAL;
        p.l2_policy_b = L2_EVICT_NORMAL;
        args.tile_start[i] = tiles;
        tiles += p.tiles;
    }
    args.tile_start[count] = tiles;
    auto kernel = gemm_tcgen05_pair_kernel<MODE, ROPE, EPILOGUE_WARPS>;
    static int clusters[64] = {};
    int device = 0;
    cudaGetDevice(&device);
    if (!clusters[device]) {
        if (!cuda_ok(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES),
                     "shared memory opt-in")) return 0;
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(dev->sms & ~1u);
        config.blockDim = dim3(C::THREADS);
        config.dynamicSmemBytes = C::SMEM_BYTES;
        cudaLaunchAttribute attribute;
        attribute.id = cudaLaunchAttributeClusterDimension;
        attribute.val.clusterDim.x = 2; attribute.val.clusterDim.y = 1; attribute.val.clusterDim.z = 1;
        config.attrs = &attribute;
        config.numAttrs = 1;
        int active = 0;
        if (!cuda_ok(cudaOccupancyMaxActiveClusters(&active, kernel, &config), "cluster occupancy query")) return 0;
        if (active < 1) return fail("the device cannot co-schedule a two-CTA cluster of the pair kernel");
        clusters[device] = active < dev->sms / 2 ? active : dev->sms / 2;
    }
    const uint32_t pairs = tiles < (uint32_t)clusters[device] ? tiles : (uint32_t)clusters[device];
    bool dependent = false;
    for (uint32_t i = 0; i < count; i++) dependent = dependent || params[i].wait_previous;
    args.p[0].wait_previous = dependent;
    if (!dependent) {
        kernel<<<2 * pairs, C::THREADS, C::SMEM_BYTES, stream>>>(args);
        count_launch(1);
        return cuda_ok(cudaGetLastError(), "tcgen05 pair linear launch");
    }
    /* programmatic dependent of the conversion kernel enqueued just before: resident and set up while that kernel
     * drains; its producer role waits for the conversion's completion before the first operand load */
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(2 * pairs);
    config.blockDim = dim3(C::THREADS);
    config.dynamicSmemBytes = C::SMEM_BYTES;
    config.stream = stream;
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&config, kernel, args);
    count_launch(1);
    return cuda_ok(e != cudaSuccess ? e : cudaGetLastError(), "tcgen05 pair linear launch");
}

/* Epilogue warps by mode and size: sixteen for int8 tiles (their main loop is half as long for the same epilogue) and
 * for bf16 problems of few tile waves (the last tile's epilogue is exposed), eight for large bf16 problems and for the
 * rotary epilogue. */
template <int MODE, bool ROPE = false>
static int launch_pair(const h3q8_linear_desc *descs, const GemmParams *params, uint32_t count, DeviceState *dev, cudaStream_t stream) {
    if constexpr (ROPE) return launch_pair_with<MODE, true, 8>(descs, params, count, dev, stream);
    else if constexpr (MODE == MODE_W8A8) return launch_pair_with<MODE, false, 16>(descs, params, count, dev, stream);
    else {
        uint64_t rows = 0;
        for (uint32_t i = 0; i < count; i++) rows += descs[i].rows;
        return rows <= 8192 ? launch_pair_with<MODE, false, 16>(descs, params, count, dev, stream)
                            : launch_pair_with<MODE, false, 8>(descs, params, count, dev, stream);
    }
}

/* W8A16 with main-loop dequantisation on the two-CTA tile (one problem per launch). */
static int launch_pair_w8a16(const h3q8_linear_desc &d, const GemmParams &params, DeviceState *dev, cudaStream_t stream) {
    using C = PairW8A16Config;
    PairArgs args;
    memset(&args, 0, sizeof args);
    args.count = 1;
    GemmParams &p = args.p[0];
    p = params;
    const bool swiglu = d.activation == H3Q8_ACT_SWIGLU; /* weight rows [gate N | up N], 128 outputs per tile */
    if (!make_map(&args.map_a[0], d.input, 2, d.rows, d.input_dim, C::BKE, 128, CU_TENSOR_MAP_SWIZZLE_128B)) return 0;
    if (!make_map(&args.map_b[0], d.weight, 1, (uint64_t)d.output_dim * (swiglu ? 2 : 1), d.input_dim, C::KSUB * C::BKE, 128,
                  CU_TENSOR_MAP_SWIZZLE_128B)) return 0;
    p.m_blocks = (d.rows + C::BM - 1) / C::BM;
    p.n_blocks = swiglu ? (d.output_dim + 127) / 128 : (d.output_dim + C::BN - 1) / C::BN;
    p.tiles = p.m_blocks * p.n_blocks;
    /* bands of four row blocks: this kernel's X tiles wait longer in L2 than the bf16 kernel's (measured 2 ... 32) */
    const uint32_t band = 4;
    p.band = p.m_blocks < band ? p.m_blocks : band;
    p.l2_policy_a = L2_EVICT_NORMAL;
    p.l2_policy_b = L2_EVICT_NORMAL;
    args.tile_start[0] = 0;
    args.tile_start[1] = p.tiles;
    static const bool packed = [] { const char *e = getenv("H3Q8_W8A16_PACKED"); return e && *e ? atoi(e) != 0 : true; }();
    auto kernel = packed ? gemm_tcgen05_pair_w8a16_kernel<true> : gemm_tcgen05_pair_w8a16_kernel<false>;
    static int clusters[64] = {};
    int device = 0;
    cudaGetDevice(&device);
    if (!clusters[device]) {
        if (!cuda_ok(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES), "shared memory opt-in")) return 0;
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(dev->sms & ~1u);
        config.blockDim = dim3(C::THREADS);
        config.dynamicSmemBytes = C::SMEM_BYTES;
        cudaLaunchAttribute attribute;
        attribute.id = cudaLaunchAttributeClusterDimension;
        attribute.val.clusterDim.x = 2; attribute.val.clusterDim.y = 1; attribute.val.clusterDim.z = 1;
        config.attrs = &attribute;
        config.numAttrs = 1;
        int active = 0;
        if (!cuda_ok(cudaOccupancyMaxActiveClusters(&active, kernel, &config), "cluster occupancy query")) return 0;
        if (active < 1) return fail("the device cannot co-schedule a two-CTA cluster of the W8A16 pair kernel");
        clusters[device] = active < dev->sms / 2 ? active : dev->sms / 2;
    }
    const uint32_t pairs = p.tiles < (uint32_t)clusters[device] ? p.tiles : (uint32_t)clusters[device];
    kernel<<<2 * pairs, C::THREADS, C::SMEM_BYTES, stream>>>(args);
    count_launch(1);
    return cuda_ok(cudaGetLastError(), "tcgen05 pair W8A16 linear launch");
}

/* W8A8 with per-K-group scales on the two-CTA kernel (one problem per launch). */
template <bool MAGIC>
static int launch_pair_grouped(const h3q8_linear_desc &d, const GemmParams &params, DeviceState *dev, cudaStream_t stream) {
    /* PairGroupedConfig: 256 x 128 tiles while the per-group combine is the bound, 256 x 256 for groups of 512 and more;
     * each CTA stages half of the tile's weight rows */
    /* with groups of 512 and more the combine runs once per four or more k-blocks and bounds nothing, so the wider tile's
     * lower operand traffic wins; with narrower groups the combine is the bound and the narrow tile's 16 epilogue warps win */
    static const int wide_tiles = [] { const char *e = getenv("H3Q8_GROUPED_WIDE"); return e && *e ? atoi(e) : 1; }();
    const bool wide = wide_tiles && params.scale_group >= 512;
    const uint32_t BM = 256, BN = wide ? 256 : 128, BKE = 128;
    PairArgs args;
    memset(&args, 0, sizeof args);
    args.count = 1;
    GemmParams &p = args.p[0];
    p = params;
    if (!make_map(&args.map_a[0], d.input, 1, d.rows, d.input_dim, BKE, 128, CU_TENSOR_MAP_SWIZZLE_128B)) return 0;
    if (!make_map(&args.map_b[0], d.weight, 1, d.output_dim, d.input_dim, BKE, BN / 2, CU_TENSOR_MAP_SWIZZLE_128B)) return 0;
    p.m_blocks = (d.rows + BM - 1) / BM;
    p.n_blocks = (d.output_dim + BN - 1) / BN;
    p.tiles = p.m_blocks * p.n_blocks;
    const uint32_t band = d.input_dim <= 8192 ? 16 : 8;
    p.band = p.m_blocks < band ? p.m_blocks : band;
    p.l2_policy_a = L2_EVICT_NORMAL;
    p.l2_policy_b = L2_EVICT_NORMAL;
    args.tile_start[0] = 0;
    args.tile_start[1] = p.tiles;
    return launch_pair_grouped_kernel(args, MAGIC, wide, dev->sms, stream);
}

/* Split-K plan for one problem: how many CTAs share an output tile and how many k-blocks each takes.
 * At least four k-blocks per split, at most as many CTAs as SMs, bounded by the workspace. */
static bool plan_splitk(uint32_t mode, uint32_t rows, uint32_t k, uint32_t n, int sms, size_t workspace_bytes, uint32_t &splits,
                        uint32_t &kb_per_split) {
    const uint32_t bke = mode == H3Q8_MODE_W8A8 ? 128 : 64, num_kb = (k + bke - 1) / bke;
    const uint64_t tiles = (uint64_t)((rows + 127) / 128) * ((n + 127) / 128);
    /* a few work items per SM (the kernel is persistent), unless the tiles alone already fill the GPU */
    /* three work items per SM (the kernel is persistent and a work item is short) and at least eight k-blocks per split
     * (below that the fixed cost of a work item -- first TMA round trip, accumulator hand-off -- outweighs the streaming) */
    static const int waves = [] { const char *e = getenv("H3Q8_SPLITK_WAVES"); return e && *e && atoi(e) > 0 ? atoi(e) : 3; }();
    static const int min_kb = [] { const char *e = getenv("H3Q8_SPLITK_MIN_KB"); return e && *e && atoi(e) > 0 ? atoi(e) : 8; }();
    uint64_t want = tiles && tiles < (uint64_t)sms ? ((uint64_t)waves * sms + tiles - 1) / tiles : 0;
    if (want > num_kb / (uint32_t)min_kb) want = num_kb / (uint32_t)min_kb;
    if (want > 32) want = 32;
    const uint64_t per_split = (uint64_t)rows * n * 4;
    /* the partial sums are written and read once: keep them below twice the weight bytes they help to stream */
    const uint64_t weight_bytes = (uint64_t)n * k * (mode == H3Q8_MODE_BF16 ? 2 : 1);
    if (per_split && want > 2 * weight_bytes / per_split) want = 2 * weight_bytes / per_split;
    if (per_split && want > workspace_bytes / per_split) want = workspace_bytes / per_split;
    if (want < 2) return false;
    kb_per_split = (uint32_t)((num_kb + want - 1) / want);
    splits = (num_kb + kb_per_split - 1) / kb_per_split;
    return splits >= 2;
}

template <int MODE>
static int launch_splitk(const h3q8_linear_desc &d, GemmParams p, DeviceState *dev, cudaStream_t stream) {
    using C = GemmConfig<MODE, 128, 1, false>;
    if (!plan_splitk(d.mode, d.rows, d.input_dim, d.output_dim, dev->sms, d.workspace_bytes, p.splits, p.kb_per_split))
        return fail("linear: split-K needs a workspace of at least 2 * rows * output_dim * 4 bytes and K of 16 k-blocks or more");
    p.partials = static_cast<uint32_t *>(d.workspace);
    CUtensorMap map_a, map_b;
    const uint32_t a_bytes = MODE == MODE_W8A8 ? 1 : 2, b_bytes = MODE == MODE_BF16 ? 2 : 1;
    if (!make_map(&map_a, d.input, a_bytes, d.rows, d.input_dim, C::BKE, 128, CU_TENSOR_MAP_SWIZZLE_128B)) return 0;
    if (!make_map(&map_b, d.weight, b_bytes, d.output_dim, d.input_dim, C::BKE, 128,
                  MODE == MODE_W8A16 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B)) return 0;
    p.m_blocks = (d.rows + 127) / 128;
    p.n_blocks = (d.output_dim + 127) / 128;
    p.tiles = p.m_blocks * p.n_blocks;
    p.band = p.m_blocks < 16 ? p.m_blocks : 16;
    auto kernel = gemm_tcgen05_kernel<MODE, 128, 1, false, true>;
    static bool configured[64] = {};
    int device = 0;
    cudaGetDevice(&device);
    if (!configured[device]) {
        if (!cuda_ok(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES), "shared memory opt-in")) return 0;
        configured[device] = true;
    }
    const uint32_t items = p.tiles * p.splits;
    kernel<<<items < (uint32_t)dev->sms ? items : (uint32_t)dev->sms, C::THREADS, C::SMEM_BYTES, stream>>>(map_a, map_b, p);
    const uint64_t outputs8 = (uint64_t)d.rows * (d.output_dim / 8);
    /* the finishing grid is launched with programmatic stream serialisation: its blocks become resident while the
     * GEMM drains and wait (griddepcontrol.wait) for the GEMM's completion before they read the partial sums */
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)((outputs8 + 255) / 256));
    config.blockDim = dim3(256);
    config.stream = stream;
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&config, splitk_finish_kernel<MODE>, p);
    count_launch(2);
    return cuda_ok(e != cudaSuccess ? e : cudaGetLastError(), "tcgen05 split-K linear launch");
}

static int launch_skinny(const h3q8_linear_desc &d, const GemmParams &p, DeviceState *dev, cudaStream_t stream) {
    SkinnyArgs args;
    memset(&args, 0, sizeof args);
    args.p = p;
    args.tokens16 = (d.rows + 15u) & ~15u;
    const uint32_t w_bytes = d.mode == H3Q8_MODE_BF16 ? 2 : 1, x_bytes = d.mode == H3Q8_MODE_W8A8 ? 1 : 2;
    /* 128-byte operand rows: 64 bf16 or 128 int8 (the raw W8A16 tile covers two 64-wide k-blocks) */
    if (!make_map(&args.map_w, d.weight, w_bytes, d.output_dim, d.input_dim, 128 / w_bytes, 128, CU_TENSOR_MAP_SWIZZLE_128B)) return 0;
    /* token tiles are exactly as tall as the padded row count, which leaves the shared memory to the weight stream */
    if (!make_map(&args.map_x, d.input, x_bytes, d.rows, d.input_dim, 128 / x_bytes, args.tokens16, CU_TENSOR_MAP_SWIZZLE_128B)) return 0;
    return launch_skinny_kernel(args, d.mode, dev->sms, stream);   /* chooses the K split */
}

template <int MODE>
static int launch_plain(const h3q8_linear_desc &d, const GemmParams &p, cudaStream_t stream) {
    dim3 grid((d.output_dim + 63) / 64, (d.rows + 63) / 64);
    linear_plain_kernel<MODE><<<grid, 256, 0, stream>>>(d.input, d.weight, p);
    count_launch(1);
    return cuda_ok(cudaGetLastError(), "plain linear launch");
}

template <int MODE>
static int launch_mode(const h3q8_linear_desc &d, const GemmParams &p, uint32_t kernel, DeviceState *dev, cudaStream_t stream) {
    const bool grouped8 = MODE == MODE_W8A8 && p.scale_group != 0;
    if (kernel == H3Q8_KERNEL_PLAIN) return launch_plain<MODE>(d, p, stream);
    if (kernel == H3Q8_KERNEL_TCGEN05_SPLITK) return launch_splitk<MODE>(d, p, dev, stream);
    if (kernel == H3Q8_KERNEL_TCGEN05_SKINNY) return launch_skinny(d, p, dev, stream);
    if (grouped8) {
        if (MODE != MODE_W8A8) return fail("grouped W8A8 reached a non-W8A8 launch");
        if (kernel == H3Q8_KERNEL_TCGEN05_PAIR)
            return p.scale_group <= 256 ? launch_pair_grouped<true>(d, p, dev, stream) : launch_pair_grouped<false>(d, p, dev, stream);
        return launch_tcgen05<MODE_W8A8, 128, 1, true>(d, p, dev, stream);
    }
    if (kernel == H3Q8_KERNEL_TCGEN05_PAIR) {
        if constexpr (MODE == MODE_W8A16) return launch_pair_w8a16(d, p, dev, stream);
        else return d.rope ? launch_pair<MODE, true>(&d, &p, 1, dev, stream) : launch_pair<MODE>(&d, &p, 1, dev, stream);
    }
    if (kernel == H3Q8_KERNEL_TCGEN05_M256) return launch_tcgen05<MODE, 256, 2, false>(d, p, dev, stream);
    if (kernel == H3Q8_KERNEL_TCGEN05_N128) return launch_tcgen05<MODE, 128, 1, false>(d, p, dev, stream);
    return launch_tcgen05<MODE, 256, 1, false>(d, p, dev, stream);
}

/* Validation, kernel parameters and kernel choice for one problem. */
static int plan_linear(const h3q8_linear_desc &d, GemmParams &p, uint32_t &kernel, DeviceState *&dev) {
    if (!d.rows || !d.input_dim || !d.output_dim) return fail("linear %ux%ux%u: empty dimension", d.rows, d.output_dim, d.input_dim);
    if (!d.input || !d.weight || (!d.output && !d.rope && !d.accumulators)) return fail("linear %ux%ux%u: null operand", d.rows, d.output_dim, d.input_dim);
    if (d.rope) {
        const h3q8_rope_desc &r = *d.rope;
        if (d.activation || d.bias || d.gate || d.residual || d.accumulators || d.weight_group || d.input_group || d.mode == H3Q8_MODE_W8A16)
            return fail("linear: the QKV rotary epilogue takes bf16 or per-channel W8A8 operands and no other epilogue term");
        if (r.head_dim != 128 || (r.rope_half != 48 && r.rope_half != 64) || !r.heads || d.output_dim != r.heads * 3 * 128)
            return fail("linear: fused QKV rotary epilogue needs head_dim 128, rope_half 48 or 64 and output_dim = heads * 384");
        if (!r.q_norm || !r.k_norm || !r.rope_cos || !r.rope_sin || !r.query || !r.key || !r.value)
            return fail("linear: QKV rotary epilogue operand missing");
    }
    if (d.mode > H3Q8_MODE_W8A8) return fail("linear: unknown mode %u", d.mode);
    if (d.activation > H3Q8_ACT_SWIGLU) return fail("linear: unknown activation %u", d.activation);
    const bool swiglu = d.activation == H3Q8_ACT_SWIGLU;
    if (swiglu && (d.gate || d.residual || d.input_group || d.accumulators || (d.mode == H3Q8_MODE_W8A8 && d.weight_group)))
        return fail("linear: SwiGLU takes no gate, residual or accumulator dump, and per-channel scales on the int8 path");
    if (swiglu && d.output_dim % 8) return fail("linear: SwiGLU needs output_dim %% 8 == 0");
    if (d.mode != H3Q8_MODE_BF16 && !d.weight_scales) return fail("linear: int8 weights need weight_scales");
    if (d.mode == H3Q8_MODE_W8A8 && !d.input_scales) return fail("linear: W8A8 needs per-token input_scales");
    if (d.accumulators && d.mode == H3Q8_MODE_W8A8 && d.weight_group)
        return fail("linear: the int32 dump exists only for W8A8 with per-channel weight scales");
    if (d.accumulators && swiglu) return fail("linear: no accumulator dump with SwiGLU");
    if ((uint64_t)d.output_dim * (swiglu ? 2u : 1u) * d.input_dim > UINT32_MAX - 31u) return fail("linear: weight exceeds 32-bit indexing");
    if (static_cast<const void *>(d.output) == d.input) return fail("linear: output aliases the input");
    dev = device_state();
    if (!dev) return 0;

    const uint32_t width = d.weight_group ? d.weight_group : d.input_dim;
    if (d.input_group && d.mode != H3Q8_MODE_W8A8) return fail("linear: input_group applies to W8A8 only");
    if (d.input_group && d.weight_group && d.input_group != d.weight_group)
        return fail("linear: activation and weight scale groups must have the same width");
    if (d.input_group && d.input_dim % d.input_group) return fail("linear: input_dim must be a multiple of input_group");
    if (d.accumulators && d.input_group) return fail("linear: the int32 dump exists only for ungrouped W8A8");
    p = GemmParams{};
    p.M = d.rows; p.N = d.output_dim; p.K = d.input_dim;
    p.scale_group = d.mode == H3Q8_MODE_BF16 ? 0 : d.weight_group ? d.weight_group : d.input_group;
    p.scale_groups = d.mode == H3Q8_MODE_BF16 || !d.weight_group ? 1 : (d.input_dim + width - 1) / width;
    p.a_scale_groups = d.input_group ? d.input_dim / d.input_group : 1;
    p.w_scales = d.weight_scales; p.a_scales = d.input_scales;
    p.ep.bias = d.bias; p.ep.gate = d.gate; p.ep.residual = d.residual; p.ep.activation = d.activation;
    p.out = d.output; p.acc_dump = d.accumulators; p.status = dev->status;
    p.wait_previous = d.after_producer != 0;
    p.wait_limit = injected_wait_limit.load(std::memory_order_relaxed);
    p.skip_first_load = injected_skip_first_load.load(std::memory_order_relaxed);
    if (d.rope) {
        const h3q8_rope_desc &r = *d.rope;
        p.ep.activation = ACT_QKV_ROPE;
        p.ep.rope = RopeParams{r.q_norm, r.k_norm, r.rope_cos, r.rope_sin, r.query, r.key, r.value, r.heads, r.rope_half, r.epsilon};
    }

    /* What the TMA path needs: 16-byte aligned bases and row pitches, output rows
     * that take 16-byte stores, scale groups that align with the k-blocks. */
    const uint32_t k_multiple = d.mode == H3Q8_MODE_BF16 ? 8 : 16;
    bool tma_ok = d.input_dim % k_multiple == 0 && d.output_dim % 8 == 0 && aligned16(d.input) && aligned16(d.weight) &&
                  (!d.output || aligned16(d.output)) && (!d.bias || aligned16(d.bias)) && (!d.gate || aligned16(d.gate)) &&
                  (!d.residual || aligned16(d.residual)) && (!d.accumulators || aligned16(d.accumulators)) &&
                  (d.mode != H3Q8_MODE_W8A8 || aligned16(d.weight_scales));
    if (d.mode == H3Q8_MODE_W8A16 && d.weight_group && d.weight_group % 64) tma_ok = false;
    if (d.mode == H3Q8_MODE_W8A8 && p.scale_group && p.scale_group % 128) tma_ok = false;
    /* the grouped two-CTA kernel hands whole scale groups to the epilogue: groups of whole k-blocks that tile K */
    const bool grouped_pair_ok = d.mode == H3Q8_MODE_W8A8 && p.scale_group && p.scale_group % 128 == 0 &&
                                 d.input_dim % p.scale_group == 0 && !swiglu && !d.rope;
    kernel = d.kernel;
    if (kernel > H3Q8_KERNEL_TCGEN05_SKINNY) return fail("linear: unknown kernel selector %u", kernel);
    /* the weight-streaming kernel: at most 128 rows, per-channel int8 scales, bias / GELU / gate / residual epilogue */
    const bool skinny_ok = d.rows <= 128 && !(d.mode == H3Q8_MODE_W8A8 && p.scale_group) && !swiglu && !d.rope && !d.accumulators &&
                           d.output;
    /* split-K: raw sums go through the workspace, so no per-group combine, second accumulator, rotary epilogue or dump */
    const bool splitk_ok = !(d.mode == H3Q8_MODE_W8A8 && p.scale_group) && !swiglu && !d.rope && !d.accumulators && d.workspace &&
                           aligned16(d.workspace);
    if (kernel == H3Q8_KERNEL_AUTO) {
        const bool tiny = (uint64_t)d.rows * d.input_dim * d.output_dim <= (1u << 22);
        /* two-CTA tiles need both CTAs to have rows */
        const bool pair_ok = d.rows > 128 && (d.mode != H3Q8_MODE_W8A8 || !p.scale_group || grouped_pair_ok) &&
                             !(d.mode == H3Q8_MODE_W8A16 && d.accumulators);
        kernel = !tma_ok || tiny ? H3Q8_KERNEL_PLAIN : d.output_dim <= 128 ? H3Q8_KERNEL_TCGEN05_N128
               : pair_ok ? H3Q8_KERNEL_TCGEN05_PAIR : H3Q8_KERNEL_TCGEN05;
        /* SwiGLU runs on the two-CTA kernel (gate rows in one CTA, up rows in its peer) or on the plain kernel */
        /* one row tile: the weight is streamed once and the problem is bandwidth bound, so spread K over the idle SMs */
        uint32_t splits, kb_per_split;
        if (kernel != H3Q8_KERNEL_PLAIN && skinny_ok) kernel = H3Q8_KERNEL_TCGEN05_SKINNY;
        else if (kernel != H3Q8_KERNEL_PLAIN && d.rows <= 128 && splitk_ok &&
                 plan_splitk(d.mode, d.rows, d.input_dim, d.output_dim, dev->sms, d.workspace_bytes, splits, kb_per_split))
            kernel = H3Q8_KERNEL_TCGEN05_SPLITK;
        if (swiglu) kernel = tma_ok ? H3Q8_KERNEL_TCGEN05_PAIR : H3Q8_KERNEL_PLAIN;
        if (d.rope) kernel = H3Q8_KERNEL_TCGEN05_PAIR;
    }
    if (d.rope) {
        const h3q8_rope_desc &r = *d.rope;
        if (kernel != H3Q8_KERNEL_TCGEN05_PAIR || !tma_ok || !aligned16(r.q_norm) || !aligned16(r.k_norm) || !aligned16(r.rope_cos) ||
            !aligned16(r.rope_sin) || !aligned16(r.query) || !aligned16(r.key) || !aligned16(r.value))
            return fail("linear: the fused QKV rotary epilogue runs on the two-CTA kernel with 16-byte aligned operands");
        return 1;
    }
    /* an explicitly requested kernel must be able to take the problem */
    if (swiglu && kernel != H3Q8_KERNEL_PLAIN && kernel != H3Q8_KERNEL_TCGEN05_PAIR) {
        return fail("linear: SwiGLU is available on the two-CTA and the plain kernel");
    } else if (kernel == H3Q8_KERNEL_TCGEN05_PAIR && d.mode == H3Q8_MODE_W8A8 && p.scale_group && !grouped_pair_ok) {
        return fail("linear: the two-CTA W8A8 kernel takes scale groups that are multiples of 128 and divide K");
    } else if (kernel == H3Q8_KERNEL_TCGEN05_PAIR && d.mode == H3Q8_MODE_W8A16 && d.accumulators) {
        return fail("linear: the two-CTA W8A16 kernel has no accumulator dump");
    } else if (kernel == H3Q8_KERNEL_TCGEN05_SKINNY && !skinny_ok) {
        return fail("linear: the weight-streaming kernel takes at most 128 rows, ungrouped W8A8 scales, and no SwiGLU / rotary epilogue / accumulator dump");
    } else if (kernel == H3Q8_KERNEL_TCGEN05_SPLITK && !splitk_ok) {
        return fail("linear: split-K takes ungrouped scales, no SwiGLU / rotary epilogue / accumulator dump, and a 16-byte aligned workspace");
    } else if (kernel != H3Q8_KERNEL_PLAIN && !tma_ok) {
        return fail("linear %ux%ux%u: shape or alignment not supported by the tcgen05 kernel "
                    "(K %% %u, N %% 8, 16-byte aligned operands, scale group %% 64/128)",
                    d.rows, d.output_dim, d.input_dim, k_multiple);
    }
    if (kernel == H3Q8_KERNEL_PLAIN && d.mode == H3Q8_MODE_W8A8 && p.scale_group % 16)
        return fail("linear: W8A8 weight scale group must be a multiple of 16");
    return 1;
}

static int launch_planned(const h3q8_linear_desc &d, const GemmParams &p, uint32_t kernel, DeviceState *dev, cudaStream_t stream) {
    switch (d.mode) {
    case H3Q8_MODE_BF16: return launch_mode<MODE_BF16>(d, p, kernel, dev, stream);
    case H3Q8_MODE_W8A16: return launch_mode<MODE_W8A16>(d, p, kernel, dev, stream);
    default: return launch_mode<MODE_W8A8>(d, p, kernel, dev, stream);
    }
}

} /* namespace h3q8 */

using namespace h3q8;

static int linear_one(const h3q8_linear_desc &d, cudaStream_t stream) {
    GemmParams p;
    uint32_t kernel;
    DeviceState *dev;
    return plan_linear(d, p, kernel, dev) && launch_planned(d, p, kernel, dev, stream);
}

extern "C" size_t h3q8_linear_workspace_bytes(uint32_t mode, uint32_t rows, uint32_t input_dim, uint32_t output_dim) {
    DeviceState *dev = device_state();
    uint32_t splits = 0, kb_per_split = 0;
    if (!dev || rows > 128 || !plan_splitk(mode, rows, input_dim, output_dim, dev->sms, SIZE_MAX, splits, kb_per_split)) return 0;
    return (size_t)splits * rows * output_dim * 4;
}

/* Second half of a linear whose fp32 partial sums were produced elsewhere (several K slices summed by the caller, or by
 * an all-reduce across GPUs): sums fp32 [rows, output_dim] -> the usual epilogue -> bf16. */
extern "C" int h3q8_linear_finish(const float *sums, uint32_t rows, uint32_t output_dim, const uint16_t *bias, const uint16_t *gate,
                                  const uint16_t *residual, uint32_t activation, uint16_t *output, void *cuda_stream) {
    if (!sums || !output || !rows || !output_dim) return fail("linear finish: null operand or empty dimension");
    if (activation > H3Q8_ACT_GELU_TANH) return fail("linear finish: activation must be none or GELU-tanh");
    if (output_dim % 8 || !aligned16(sums) || !aligned16(output) || (bias && !aligned16(bias)) || (gate && !aligned16(gate)) ||
        (residual && !aligned16(residual)))
        return fail("linear finish: needs output_dim %% 8 == 0 and 16-byte aligned operands");
    uint32_t *status = device_status_word();
    if (!status) return 0;
    GemmParams p = {};
    p.M = rows; p.N = output_dim; p.K = 0;
    p.ep.bias = bias; p.ep.gate = gate; p.ep.residual = residual; p.ep.activation = activation;
    p.out = output; p.status = status;
    p.splits = 1; p.partials = reinterpret_cast<uint32_t *>(const_cast<float *>(sums));
    const uint64_t outputs8 = (uint64_t)rows * (output_dim / 8);
    splitk_finish_kernel<MODE_BF16><<<(unsigned)((outputs8 + 255) / 256), 256, 0, (cudaStream_t)cuda_stream>>>(p);
    count_launch(1);
    return cuda_ok(cudaGetLastError(), "linear finish launch");
}

extern "C" int h3q8_linear(const h3q8_linear_desc *desc, void *cuda_stream) {
    if (!desc) return fail("linear: null descriptor");
    return linear_one(*desc, (cudaStream_t)cuda_stream);
}

extern "C" int h3q8_linear_grouped(const h3q8_linear_desc *problems, uint32_t count, void *cuda_stream) {
    if (!problems || !count) return fail("grouped linear: no problems");
    cudaStream_t stream = (cudaStream_t)cuda_stream;
    /* One launch when every problem runs on the two-CTA kernel in the same operand mode;
     * otherwise the problems are enqueued back to back. */
    if (count <= PAIR_MAX_PROBLEMS) {
        GemmParams params[PAIR_MAX_PROBLEMS];
        DeviceState *dev = nullptr;
        bool together = true;
        for (uint32_t i = 0; i < count; i++) {
            uint32_t kernel;
            if (!plan_linear(problems[i], params[i], kernel, dev)) return 0;
            together = together && kernel == H3Q8_KERNEL_TCGEN05_PAIR && problems[i].mode == problems[0].mode && !problems[i].rope &&
                       problems[i].mode != H3Q8_MODE_W8A16 &&
                       !(problems[i].mode == H3Q8_MODE_W8A8 && params[i].scale_group);
        }
        if (together && count > 1)
            return problems[0].mode == H3Q8_MODE_BF16 ? launch_pair<MODE_BF16>(problems, params, count, dev, stream)
                                                       : launch_pair<MODE_W8A8>(problems, params, count, dev, stream);
    }
    for (uint32_t i = 0; i < count; i++)
        if (!linear_one(problems[i], stream)) return 0;
    return 1;
}

extern "C" int h3q8_quantize_rows(const uint16_t *input, int8_t *output, float *scales, uint32_t rows,
                                  uint32_t dispatch_rows, uint32_t columns, float clip, void *cuda_stream) {
    if (!input || !output || !scales || !rows || !columns || dispatch_rows < rows)
        return fail("quantize rows: invalid arguments");
    if (!(clip > 0.0f) || clip > 1.0f) return fail("quantize rows: clip must be in (0, 1]");
    uint32_t *status = device_status_word();
    if (!status) return 0;
    cudaError_t e = launch_quantize_rows(input, output, scales, rows, dispatch_rows, columns, clip, status, (cudaStream_t)cuda_stream);
    count_launch(1);
    return cuda_ok(e, "quantize rows launch");
}

extern "C" int h3q8_quantize_rows_grouped(const uint16_t *input, int8_t *output, float *scales, uint32_t rows,
                                          uint32_t dispatch_rows, uint32_t columns, uint32_t group, void *cuda_stream) {
    if (!group || columns % group) return fail("quantize rows: columns must be a multiple of the group width");
    const uint64_t groups = columns / group;
    if (dispatch_rows * groups > UINT32_MAX) return fail("quantize rows: too many row groups");
    /* every (row, group) is an independent row of `group` columns of the same contiguous matrix */
    return h3q8_quantize_rows(input, output, scales, (uint32_t)(rows * groups), (uint32_t)(dispatch_rows * groups), group, 1.0f, cuda_stream);
}

extern "C" int h3q8_q8_pack_rows_device(const uint16_t *source, int8_t *weights, float *scales, uint32_t rows,
                                        uint32_t columns, uint32_t group, void *cuda_stream) {
    size_t offset, bytes;
    if (!source || !weights || !scales || !h3q8_q8_layout(rows, columns, group, &offset, &bytes))
        return fail("q8 pack: invalid arguments");
    uint32_t *status = device_status_word();
    if (!status) return 0;
    const uint32_t width = group ? group : columns;
    const uint32_t groups = (uint32_t)(((uint64_t)columns + width - 1) / width);
    const uint64_t items = (uint64_t)rows * groups;
    q8_pack_rows_kernel<<<(unsigned)((items + 7) / 8), 256, 0, (cudaStream_t)cuda_stream>>>(source, weights, scales, rows, columns,
                                                                                           width, groups, status);
    count_launch(1);
    return cuda_ok(cudaGetLastError(), "q8 pack launch");
}

extern "C" int h3q8_q8_dequant(const int8_t *weights, const float *scales, uint16_t *output, uint32_t rows,
                               uint32_t columns, uint32_t group, void *cuda_stream) {
    if (!weights || !scales || !output || !rows || !columns) return fail("q8 dequant: invalid arguments");
    if (!device_status_word()) return 0;
    const uint32_t width = group ? group : columns;
    const uint32_t groups = (uint32_t)(((uint64_t)columns + width - 1) / width);
    unsigned per_row = (columns / 16 + 255) / 256;
    if (!per_row) per_row = 1;
    q8_dequant_kernel<<<dim3(per_row, rows), 256, 0, (cudaStream_t)cuda_stream>>>(weights, scales, output, rows, columns, width, groups);
    count_launch(1);
    return cuda_ok(cudaGetLastError(), "q8 dequant launch");
}

extern "C" uint32_t h3q8_device_status(void *cuda_stream) {
    uint32_t *word = device_status_word();
    if (!word) return 0xffffffffu;
    uint32_t value = 0;
    if (cudaStreamSynchronize((cudaStream_t)cuda_stream) != cudaSuccess ||
        cudaMemcpy(&value, word, sizeof value, cudaMemcpyDeviceToHost) != cudaSuccess) {
        fail("CUDA error while reading the device status: %s", cudaGetErrorString(cudaGetLastError()));
        return 0xffffffffu;
    }
    if (value) cudaMemset(word, 0, sizeof value);
    else value = static_status_take();   /* h3q8_linear_w8a8_static called without a status word of the caller's */
    if (value == 0xffffffffu) fail("CUDA error while reading the device status: %s", cudaGetErrorString(cudaGetLastError()));
    else if (value & STATUS_NONFINITE) fail("non-finite value (Inf or NaN) in the input of a quantiser or of the weight packer");
    else if (value) fail("a kernel gave up a bounded wait: code %u in CTA %u", value & 0xffu, value >> 8);
    return value;
}

extern "C" void h3q8_fault_injection(uint64_t wait_limit_cycles, uint32_t skip_first_load) {
    injected_wait_limit.store((long long)wait_limit_cycles);
    injected_skip_first_load.store(skip_first_load);
}
extern "C" const char *h3q8_last_error(void) { return last_error; }
extern "C" uint64_t h3q8_kernel_launches(void) { return launches.load(); }
