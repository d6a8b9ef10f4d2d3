/* Launch of the weight-streaming kernel for linears of at most 64 rows (a translation unit of its own). */
#include <cuda.h>
#include <cuda_runtime.h>
#include "h3q8.h"
#include "h3q8_internal.h"
#include "gemm_tcgen05_skinny.cuh"

namespace h3q8 {

/* K slices: as many CTAs per 128-channel tile as the machine can hold at once (a cluster of at most 8; a cluster size
 * whose clusters cannot all be resident together would run in two waves), each with at least two K units. */
template <int MODE>
static int launch(SkinnyArgs &args, int sms, cudaStream_t stream) {
    using C = SkinnyConfig<MODE>;
    auto kernel = gemm_tcgen05_skinny_kernel<MODE>;
    static int resident[64][9] = {};                 /* clusters of each size that fit on the device; 0 = not asked yet */
    int device = 0;
    cudaGetDevice(&device);
    if (device < 0 || device >= 64) return fail("skinny linear: device index out of range");
    if (!resident[device][0]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return fail("CUDA shared memory opt-in: %s", cudaGetErrorString(e));
        resident[device][0] = 1;
    }
    const uint32_t tiles = (args.p.N + 127) / 128, units = (args.p.K + C::UNIT - 1) / C::UNIT;
    cudaLaunchConfig_t config = {};
    config.blockDim = dim3(C::THREADS);
    config.dynamicSmemBytes = C::SMEM_BYTES;
    config.stream = stream;
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeClusterDimension;
    attribute.val.clusterDim.y = 1; attribute.val.clusterDim.z = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    uint32_t want = tiles ? (uint32_t)sms / tiles : 1;
    if (want > 8) want = 8;
    if (want > units / 2) want = units / 2;
    if (want < 1) want = 1;
    for (; want > 1; want--) {
        if (!resident[device][want]) {
            attribute.val.clusterDim.x = want;
            config.gridDim = dim3(want * ((uint32_t)sms / want));
            int clusters = 0;
            cudaError_t e = cudaOccupancyMaxActiveClusters(&clusters, kernel, &config);
            if (e != cudaSuccess) return fail("CUDA cluster occupancy query: %s", cudaGetErrorString(e));
            resident[device][want] = clusters > 0 ? clusters : -1;
        }
        if (resident[device][want] >= (int)tiles) break;
    }
    args.units_per_split = (units + want - 1) / want;
    args.splits = (units + args.units_per_split - 1) / args.units_per_split;
    attribute.val.clusterDim.x = args.splits;
    config.gridDim = dim3(tiles * args.splits);
    cudaError_t e = cudaLaunchKernelEx(&config, kernel, args);
    count_launch(1);
    if (e == cudaSuccess) e = cudaGetLastError();
    return e == cudaSuccess ? 1 : fail("CUDA tcgen05 skinny linear launch: %s", cudaGetErrorString(e));
}

int launch_skinny_kernel(SkinnyArgs &args, uint32_t mode, int sms, void *stream) {
    switch (mode) {
    case H3Q8_MODE_BF16: return launch<MODE_BF16>(args, sms, (cudaStream_t)stream);
    case H3Q8_MODE_W8A16: return launch<MODE_W8A16>(args, sms, (cudaStream_t)stream);
    default: return launch<MODE_W8A8>(args, sms, (cudaStream_t)stream);
    }
}

} /* namespace h3q8 */
