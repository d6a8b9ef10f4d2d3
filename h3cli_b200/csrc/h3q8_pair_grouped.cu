/* Launch of the grouped-scale two-CTA W8A8 kernel (a translation unit of its own keeps the
 * build of the other kernels unchanged while this one is tuned). */
#include <cuda.h>
#include <cuda_runtime.h>
#include "h3q8.h"
#include "h3q8_internal.h"
#include "gemm_tcgen05_pair_grouped.cuh"

namespace h3q8 {

template <bool MAGIC, bool WIDE>
static int launch(const PairArgs &args, int sms, cudaStream_t stream) {
    using C = PairGroupedConfig<WIDE>;
    auto kernel = gemm_tcgen05_pair_grouped_kernel<MAGIC, WIDE>;
    static int clusters[64] = {};
    int device = 0;
    cudaGetDevice(&device);
    if (device < 0 || device >= 64) return fail("grouped pair linear: device index out of range");
    if (!clusters[device]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return fail("CUDA shared memory opt-in: %s", cudaGetErrorString(e));
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(sms & ~1u);
        config.blockDim = dim3(C::THREADS);
        config.dynamicSmemBytes = C::SMEM_BYTES;
        cudaLaunchAttribute attribute;
        attribute.id = cudaLaunchAttributeClusterDimension;
        attribute.val.clusterDim.x = 2; attribute.val.clusterDim.y = 1; attribute.val.clusterDim.z = 1;
        config.attrs = &attribute;
        config.numAttrs = 1;
        int active = 0;
        e = cudaOccupancyMaxActiveClusters(&active, kernel, &config);
        if (e != cudaSuccess) return fail("CUDA cluster occupancy query: %s", cudaGetErrorString(e));
        if (active < 1) return fail("the device cannot co-schedule a two-CTA cluster of the grouped pair kernel");
        clusters[device] = active < sms / 2 ? active : sms / 2;
    }
    const uint32_t tiles = args.tile_start[args.count];
    const uint32_t pairs = tiles < (uint32_t)clusters[device] ? tiles : (uint32_t)clusters[device];
    kernel<<<2 * pairs, C::THREADS, C::SMEM_BYTES, stream>>>(args);
    count_launch(1);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 1 : fail("CUDA tcgen05 grouped pair linear launch: %s", cudaGetErrorString(e));
}

int launch_pair_grouped_kernel(const PairArgs &args, bool magic, bool wide, int sms, void *stream) {
    if (wide) return launch<false, true>(args, sms, (cudaStream_t)stream);     /* wide tiles serve groups of 512 and more */
    return magic ? launch<true, false>(args, sms, (cudaStream_t)stream) : launch<false, false>(args, sms, (cudaStream_t)stream);
}

} /* namespace h3q8 */
