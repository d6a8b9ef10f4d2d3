/* h3q8_linear_w8a8_static: the W8A8 projection for callers that must not
 * allocate GPU memory.
 *
 * Who that is: code that runs where cudaMalloc is off limits -- inside a
 * latency-critical render loop that has already handed every byte of HBM to
 * its own pools, inside a host callback or another library's hook where
 * allocating could deadlock or synchronise the whole device, or in a process
 * whose memory budget was fixed at start-up and is audited.  The regular W8A8
 * path needs scratch for the per-token int8 activations and their scales; the
 * caller (h3q8_linear + h3q8_quantize_rows) or the context (h3_gpu_*) has to
 * allocate it.  Here that scratch is a fixed array compiled into the library's
 * device image, so the call itself allocates nothing: no cudaMalloc, no
 * cudaFree, no allocating library routine.
 *
 * The price, stated plainly:
 *   - every GPU whose context loads this library holds the array (16 MiB + 64 KiB
 *     + one status word) from load until the process exits, used or not;
 *   - the problem must fit: rows * input_dim <= 16 MiB of int8 activations and
 *     rows <= 16384; anything larger is refused with an error, never truncated;
 *   - all calls on a device share the one array.  Each call overwrites the part
 *     it later reads (activations and scales of its own rows), so nothing has to
 *     start at zero and stale bytes of an earlier, larger call are never read;
 *     but two calls that overlap on the GPU (different streams, or different
 *     host threads) race on it.  Keep calls on one stream, or order them.
 *   - the first call on a device resolves the array's device address
 *     (cudaGetSymbolAddress) and opts the kernel into its shared-memory size.
 *     Make that first call outside any stream capture.
 */
#include <mutex>

#include "h3q8.h"
#include "h3q8_internal.h"
#include "kernels_misc.cuh"

using namespace h3q8;

namespace {

constexpr size_t ACTIVATION_BYTES = H3Q8_STATIC_MAX_ACTIVATION_BYTES;
constexpr uint32_t MAX_ROWS = H3Q8_STATIC_MAX_ROWS;
constexpr size_t SCALE_OFFSET = ACTIVATION_BYTES;
constexpr size_t STATUS_OFFSET = SCALE_OFFSET + MAX_ROWS * sizeof(float);
constexpr size_t SCRATCH_BYTES = STATUS_OFFSET + 256;

/* The scratch itself.  In host code this name is only a handle for the runtime;
 * the address kernels can use comes from cudaGetSymbolAddress below. */
static __device__ __align__(256) unsigned char static_scratch[SCRATCH_BYTES];

/* Device code may name the array directly; this also keeps it in the device image. */
static __global__ void clear_status_kernel() { *reinterpret_cast<uint32_t *>(static_scratch + STATUS_OFFSET) = 0u; }

struct PerDevice {
    bool ready = false;
    unsigned char *base = nullptr; /* device address of static_scratch on this device */
    int sms = 0;
};
PerDevice per_device[64];
std::mutex setup_mutex;

typedef CUresult (*encode_tiled_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
encode_tiled_fn encode_tiled = nullptr;

using StaticConfig = GemmConfig<MODE_W8A8, 256, 1, false>;

/* Once per device, with that device current: find where the array lives there. */
PerDevice *setup(cudaStream_t stream) {
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) { fail("static W8A8: cudaGetDevice: %s", cudaGetErrorString(e)); return nullptr; }
    if (device < 0 || device >= 64) { fail("static W8A8: device index %d out of range", device); return nullptr; }
    std::lock_guard<std::mutex> lock(setup_mutex);
    PerDevice &d = per_device[device];
    if (d.ready) return &d;
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess || major != 10) {
        fail("static W8A8: needs an sm_100 GPU (B200)");
        return nullptr;
    }
    if (cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || d.sms <= 0) {
        fail("static W8A8: cannot read the SM count");
        return nullptr;
    }
    void *address = nullptr;
    e = cudaGetSymbolAddress(&address, static_scratch);
    if (e != cudaSuccess || !address) {
        fail("static W8A8: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        return nullptr;
    }
    d.base = static_cast<unsigned char *>(address);
    e = cudaFuncSetAttribute(gemm_tcgen05_kernel<MODE_W8A8, 256, 1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             StaticConfig::SMEM_BYTES);
    if (e != cudaSuccess) { fail("static W8A8: shared memory opt-in: %s", cudaGetErrorString(e)); return nullptr; }
    /* the one word that must start at zero; cleared on the caller's stream, ahead of the first use */
    clear_status_kernel<<<1, 1, 0, stream>>>();
    e = cudaGetLastError();
    if (e != cudaSuccess) { fail("static W8A8: clearing the status word: %s", cudaGetErrorString(e)); return nullptr; }
    if (!encode_tiled) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &result) != cudaSuccess ||
            result != cudaDriverEntryPointSuccess || !fn) {
            fail("static W8A8: cuTensorMapEncodeTiled is not available from this driver");
            return nullptr;
        }
        encode_tiled = reinterpret_cast<encode_tiled_fn>(fn);
    }
    d.ready = true;
    return &d;
}

bool int8_map(CUtensorMap *map, const void *base, uint64_t rows, uint64_t columns, uint32_t box_rows) {
    cuuint64_t dims[2] = {columns, rows};
    cuuint64_t strides[1] = {columns};
    cuuint32_t box[2] = {StaticConfig::BKE, box_rows};
    cuuint32_t element_strides[2] = {1, 1};
    return encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, element_strides,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

} /* namespace */

/* The status word inside the static array, for calls that passed device_status == NULL: read (and cleared when set) by
 * h3q8_device_status after it has synchronised the stream.  0 when this device never ran the static entry point. */
uint32_t h3q8::static_status_take() {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 0;
    unsigned char *base;
    {
        std::lock_guard<std::mutex> lock(setup_mutex);
        if (!per_device[device].ready) return 0;
        base = per_device[device].base;
    }
    uint32_t value = 0;
    if (cudaMemcpy(&value, base + STATUS_OFFSET, sizeof value, cudaMemcpyDeviceToHost) != cudaSuccess) return 0xffffffffu;
    if (value) cudaMemset(base + STATUS_OFFSET, 0, sizeof value);
    return value;
}

extern "C" int h3q8_linear_w8a8_static(const h3q8_linear_desc *desc, uint32_t *device_status, void *cuda_stream) {
    if (!desc) return fail("static W8A8: null descriptor");
    const h3q8_linear_desc &d = *desc;
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    if (d.mode != H3Q8_MODE_W8A8) return fail("static W8A8: desc.mode must be H3Q8_MODE_W8A8");
    if (!d.rows || !d.input_dim || !d.output_dim || !d.input || !d.weight || !d.weight_scales || !d.output)
        return fail("static W8A8: missing operand or empty dimension");
    if (d.input_scales) return fail("static W8A8: input is bf16 here; leave input_scales NULL (the scales live in the static scratch)");
    if (d.weight_group || d.input_group || d.accumulators) return fail("static W8A8: per-channel weight scales only, no accumulator dump");
    if (d.activation > H3Q8_ACT_GELU_TANH) return fail("static W8A8: unknown activation %u", d.activation);
    if (d.rope) return fail("static W8A8: the QKV rotary epilogue is not available here; use h3q8_linear");
    if (d.workspace || d.workspace_bytes) return fail("static W8A8: takes no workspace (split-K is not available here)");
    if (d.kernel != H3Q8_KERNEL_AUTO) return fail("static W8A8: desc.kernel must be H3Q8_KERNEL_AUTO (one fixed kernel runs here)");
    if (d.rows > MAX_ROWS || (uint64_t)d.rows * d.input_dim > ACTIVATION_BYTES)
        return fail("static W8A8: %u x %u activations exceed the built-in scratch (rows <= %u and rows * input_dim <= %zu bytes); "
                    "use h3q8_quantize_rows + h3q8_linear with your own scratch instead",
                    d.rows, d.input_dim, MAX_ROWS, ACTIVATION_BYTES);
    if (d.input_dim % 16 || d.output_dim % 8 || !aligned16(d.input) || !aligned16(d.weight) || !aligned16(d.weight_scales) ||
        !aligned16(d.output) || (d.bias && !aligned16(d.bias)) || (d.gate && !aligned16(d.gate)) ||
        (d.residual && !aligned16(d.residual)))
        return fail("static W8A8: needs input_dim %% 16 == 0, output_dim %% 8 == 0 and 16-byte aligned operands");
    if ((uint64_t)d.output_dim * d.input_dim > UINT32_MAX - 31u) return fail("static W8A8: weight exceeds 32-bit indexing");
    PerDevice *dev = setup(stream);
    if (!dev) return 0;

    int8_t *activations = reinterpret_cast<int8_t *>(dev->base);
    float *scales = reinterpret_cast<float *>(dev->base + SCALE_OFFSET);
    uint32_t *status = device_status ? device_status : reinterpret_cast<uint32_t *>(dev->base + STATUS_OFFSET);

    /* 1. per-token quantisation of exactly the rows this call will read */
    quantize_rows_kernel<<<d.rows, 256, 0, stream>>>(static_cast<const uint16_t *>(d.input), activations, scales, d.rows,
                                                     d.input_dim, 1.0f, nullptr);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail("static W8A8: quantiser launch: %s", cudaGetErrorString(e));

    /* 2. int8 GEMM + fused epilogue; the activation map covers d.rows rows only, so TMA
     *    zero-fills the tail of the last row tile instead of reading older contents */
    CUtensorMap map_a, map_b;
    if (!int8_map(&map_a, activations, d.rows, d.input_dim, 128) || !int8_map(&map_b, d.weight, d.output_dim, d.input_dim, 256))
        return fail("static W8A8: cuTensorMapEncodeTiled failed");
    GemmParams p = {};
    p.M = d.rows; p.N = d.output_dim; p.K = d.input_dim;
    p.scale_group = 0; p.scale_groups = 1; p.a_scale_groups = 1;
    p.w_scales = d.weight_scales; p.a_scales = scales;
    p.ep.bias = d.bias; p.ep.gate = d.gate; p.ep.residual = d.residual; p.ep.activation = d.activation;
    p.out = d.output; p.acc_dump = nullptr; p.status = status;
    p.m_blocks = (d.rows + StaticConfig::BM - 1) / StaticConfig::BM;
    p.n_blocks = (d.output_dim + 255) / 256;
    p.tiles = p.m_blocks * p.n_blocks;
    p.band = p.m_blocks < 16 ? p.m_blocks : 16;
    const uint32_t grid = p.tiles < (uint32_t)dev->sms ? p.tiles : (uint32_t)dev->sms;
    gemm_tcgen05_kernel<MODE_W8A8, 256, 1, false><<<grid, StaticConfig::THREADS, StaticConfig::SMEM_BYTES, stream>>>(map_a, map_b, p);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail("static W8A8: GEMM launch: %s", cudaGetErrorString(e));
    count_launch(2);
    return 1;
}
