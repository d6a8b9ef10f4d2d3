/* Linears of at most 128 token rows: the weight is the wide operand.
 *
 *   out[m, n] = epilogue( sum_k X[m, k] * W[n, k] )        rows (m) <= 128
 *
 * With so few rows the weight matrix is streamed once and the problem is bound by HBM, so the
 * kernel is built around the weight stream instead of around an output tile:
 *
 *   - operands are swapped: the MMA's M side is 128 WEIGHT rows (every TMEM lane carries a
 *     real output channel), its N side the token rows padded to a multiple of 16, so the
 *     accumulator is [128 channels x tokens] and all 128 epilogue threads have work;
 *   - K is split over the CTAs of a thread-block cluster (1 to 8) so that tiles x splits
 *     fills the machine; each CTA streams its K range through a deep TMA ring (up to eight
 *     16 KB weight tiles in flight per SM; the token tile beside each is as tall as the call's
 *     padded row count, so few rows leave the shared memory to the weight stream);
 *   - the four K steps of a k-block accumulate into four separate TMEM accumulators, so that
 *     consecutive narrow MMAs do not chain on one accumulator (the epilogue adds the four);
 *   - the partial sums never leave the chip: each CTA writes its [tokens x 128] partial tile
 *     into its own shared memory, the cluster synchronises once, and CTA s sums token rows
 *     s, s + splits, ... over all CTAs in ascending split order through distributed shared
 *     memory, eight channels per thread and step (int32 exactly, fp32 in one fixed order:
 *     results do not depend on scheduling), runs the usual epilogue and stores bf16 -- one
 *     launch, no workspace.
 *
 * Modes: bf16 x bf16, W8A8 (int8 x int8 -> int32, per-token and per-channel scales in the
 * epilogue) and W8A16 (int8 weights dequantised in the main loop, bf16(float(q) * scale),
 * src/metal/shaders.metal:825-827, by two groups of four warps on alternate 128-wide blocks
 * of K, with the conversion of the two-CTA W8A16 kernel).
 *
 * Every mbarrier wait is bounded; a role that gives up raises the CTA's abort flag, all roles
 * fall through to the two cluster barriers and the common exit, the status word is set and
 * TMEM is freed.
 */
#pragma once
#include "gemm_tcgen05_pair_w8a16.cuh"

namespace h3q8 {

struct SkinnyArgs {
    GemmParams p;            /* M = token rows, N = output channels, K                        */
    CUtensorMap map_w, map_x;
    uint32_t tokens16;       /* token rows rounded up to a multiple of 16 (the MMA's N)       */
    uint32_t splits;         /* CTAs per cluster = K slices                                   */
    uint32_t units_per_split;/* K units (k-blocks; 128-wide blocks for W8A16) per slice       */
};

template <int MODE>
struct SkinnyConfig {
    static constexpr int MAX_TOKENS = 128;
    static constexpr int BKE = MODE == MODE_W8A8 ? 128 : 64;     /* K elements per 128-byte operand row             */
    static constexpr int SUB = MODE == MODE_W8A16 ? 2 : 1;       /* k-blocks per K unit (weight hand-off)           */
    static constexpr int UNIT = BKE * SUB;                        /* K elements per unit                             */
    static constexpr int W_BYTES = 128 * 128;                     /* weight operand tile of one k-block              */
    static constexpr int RAW_BYTES = 128 * 128;                   /* W8A16: 128 rows x 128 int8 (one unit)           */
    /* rings in K units */
    static constexpr int STAGES = 8;                              /* at most; as many as the stage region holds at the
                                                                     call's row count (a token tile is tokens16 x 128 B) */
    /* W8A16: two groups of four dequantiser warps take alternate units, one converted pair each.  (Four groups, four
     * converted pairs or eight raw tiles measured the same or slower: the main loop, not the stream, is its bound.) */
    static constexpr int GROUPS = 2;
    static constexpr int RAW_STAGES = MODE == MODE_W8A16 ? 5 : 0;
    static constexpr int CONV_BUFFERS = MODE == MODE_W8A16 ? GROUPS : 0;
    /* stage region: token tiles only (W8A16, 64 KB) or weight tile + token tile (192 KB) */
    static constexpr int STAGE_REGION = MODE == MODE_W8A16 ? 64 * 1024 : 192 * 1024;
    static constexpr int EPILOGUE_WARPS = 4, PRODUCER_WARP = 4, MMA_WARP = 5, FIRST_DEQUANT_WARP = 6;
    static constexpr int GROUP_WARPS = 4, DEQUANT_WARPS = MODE == MODE_W8A16 ? GROUPS * GROUP_WARPS : 0;
    static constexpr int WARPS = FIRST_DEQUANT_WARP + DEQUANT_WARPS, THREADS = WARPS * 32;
    static constexpr int RING_BYTES = STAGE_REGION + RAW_STAGES * RAW_BYTES + CONV_BUFFERS * SUB * W_BYTES;
    static constexpr int PARTIAL_BYTES = MAX_TOKENS * 128 * 4;   /* aliases the rings once the main loop is done    */
    static constexpr int BARRIERS = 2 * STAGES + 2 * RAW_STAGES + 2 * CONV_BUFFERS + 1;
    static constexpr int SMEM_BYTES = RING_BYTES + 1024 + 512;
    static constexpr int ACCUMULATORS = 4;      /* independent partial accumulators, see the MMA issuer */
    static constexpr int TMEM_COLUMNS = ACCUMULATORS * MAX_TOKENS;
    static_assert(PARTIAL_BYTES <= RING_BYTES, "the partial tile lives in the drained rings");
    static_assert(SMEM_BYTES <= 227 * 1024 && BARRIERS * 8 + 16 <= 512, "shared memory budget");
};

__device__ __forceinline__ uint32_t cluster_cta_count() {
    uint32_t count;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(count));
    return count;
}
__device__ __forceinline__ uint4 load_cluster_u128(uint32_t cluster_addr) {
    uint4 v;
    /* volatile keeps it behind the cluster barrier; no memory clobber, so independent loads around it may be batched */
    asm volatile("ld.shared::cluster.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(cluster_addr));
    return v;
}

template <int MODE>
static __global__ void __launch_bounds__(SkinnyConfig<MODE>::THREADS, 1)
gemm_tcgen05_skinny_kernel(const __grid_constant__ SkinnyArgs args) {
    using C = SkinnyConfig<MODE>;
    const GemmParams &p = args.p;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *ring = smem;                                             /* per stage: [W tile] X tile(s)            */
    uint8_t *conv = ring + C::STAGE_REGION;                           /* W8A16: converted weight tiles            */
    uint8_t *raw_ring = conv + C::CONV_BUFFERS * C::SUB * C::W_BYTES; /* W8A16: raw int8 weight tiles             */
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + C::RING_BYTES);
    uint64_t *full = bars, *empty = full + C::STAGES;
    uint64_t *rfull = empty + C::STAGES, *rempty = rfull + C::RAW_STAGES;
    uint64_t *bfull = rempty + C::RAW_STAGES, *bempty = bfull + C::CONV_BUFFERS;
    uint64_t *tfull = bempty + C::CONV_BUFFERS;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tfull + 1);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    uint32_t *partial = reinterpret_cast<uint32_t *>(smem);          /* [token][128 channels], after the main loop */

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t split = cluster_cta_rank(), splits = cluster_cta_count();
    const uint32_t tile = blockIdx.x / splits;                        /* 128 output channels                       */
    const uint32_t n0 = tile * 128;
    const uint32_t units = (p.K + C::UNIT - 1) / C::UNIT;
    const uint32_t unit_begin = min(units, split * args.units_per_split);
    const uint32_t unit_end = min(units, unit_begin + args.units_per_split);
    const uint32_t num_kb = (p.K + C::BKE - 1) / C::BKE;
    const uint32_t tokens16 = args.tokens16;
    /* a token tile holds tokens16 rows (the TMA box of the call); a stage holds the tiles of one unit */
    const uint32_t x_tile_bytes = tokens16 * 128;
    const uint32_t stage_bytes = MODE == MODE_W8A16 ? C::SUB * x_tile_bytes : C::W_BYTES + x_tile_bytes;
    const uint32_t stages = min((uint32_t)C::STAGES, C::STAGE_REGION / stage_bytes);

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int s = 0; s < C::RAW_STAGES; s++) { mbar_init(&rfull[s], 1); mbar_init(&rempty[s], C::GROUP_WARPS); }
        for (int s = 0; s < C::CONV_BUFFERS; s++) { mbar_init(&bfull[s], C::GROUP_WARPS); mbar_init(&bempty[s], 1); }
        mbar_init(tfull, 1);
        control_block_init(tmem_slot, p.wait_limit);
        fence_barrier_init();
        fence_proxy_async_smem();
    }
    if (warp == C::PRODUCER_WARP && lane == 0) { tma_prefetch_descriptor(&args.map_w); tma_prefetch_descriptor(&args.map_x); }
    if (warp == C::MMA_WARP) { tmem_alloc(tmem_slot, C::TMEM_COLUMNS); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    uint32_t failure = STATUS_OK;

    if (warp == C::PRODUCER_WARP) {
        /* ------------------------------------------------ TMA producer */
        if (lane == 0) {
            PipeState st, sr;
            for (uint32_t u = unit_begin; u < unit_end; u++) {
                if (MODE == MODE_W8A16) {
                    if (!wait_or_abort(&rempty[sr.index], sr.phase ^ 1, abort_flag)) { failure = STATUS_WAIT_PRODUCER; break; }
                    mbar_arrive_expect_tx(&rfull[sr.index], C::RAW_BYTES);
                    if (!(p.skip_first_load && blockIdx.x == 0 && u == unit_begin))
                        tma_load_2d(raw_ring + sr.index * C::RAW_BYTES, &args.map_w, &rfull[sr.index], (int32_t)(u * C::UNIT), (int32_t)n0);
                    sr.advance(C::RAW_STAGES);
                }
                if (!wait_or_abort(&empty[st.index], st.phase ^ 1, abort_flag)) { failure = STATUS_WAIT_PRODUCER; break; }
                uint8_t *stage = ring + st.index * stage_bytes;
                mbar_arrive_expect_tx(&full[st.index], MODE == MODE_W8A16 && u * C::SUB + 1 >= num_kb ? x_tile_bytes : stage_bytes);
                if (MODE != MODE_W8A16) {
                    if (!(p.skip_first_load && blockIdx.x == 0 && u == unit_begin))
                        tma_load_2d(stage, &args.map_w, &full[st.index], (int32_t)(u * C::UNIT), (int32_t)n0);
                    tma_load_2d(stage + C::W_BYTES, &args.map_x, &full[st.index], (int32_t)(u * C::UNIT), 0);
                } else {
                    /* a k-block that starts beyond K is neither loaded nor multiplied */
#pragma unroll
                    for (int sub = 0; sub < C::SUB; sub++)
                        if (u * C::SUB + sub < num_kb)
                            tma_load_2d(stage + sub * x_tile_bytes, &args.map_x, &full[st.index], (int32_t)(u * C::UNIT + sub * C::BKE), 0);
                }
                st.advance(stages);
            }
        }
    } else if (warp == C::MMA_WARP) {
        /* ------------------------------------------------ MMA issuer */
        if (lane == 0 && unit_begin < unit_end) {
            const uint32_t idesc = MODE == MODE_W8A8 ? umma_idesc(2, 1, 128, tokens16) : umma_idesc(1, 1, 128, tokens16);
            /* The four K steps of a k-block go to four accumulators (columns j * tokens16), so that MMAs this narrow do not
             * chain on one accumulator; the epilogue adds the four in a fixed order.  Each MMA still reads its 4 KB of
             * weights from shared memory, about 60 clocks, which is the floor of this formulation. */
            PipeState st, cv;
            for (uint32_t u = unit_begin; u < unit_end && !failure; u++) {
                if (!wait_or_abort(&full[st.index], st.phase, abort_flag)) { failure = STATUS_WAIT_MMA; break; }
                if (MODE == MODE_W8A16 && !wait_or_abort(&bfull[cv.index], cv.phase, abort_flag)) { failure = STATUS_WAIT_MMA; break; }
                tc_fence_after_sync();
                const uint8_t *stage = ring + st.index * stage_bytes;
#pragma unroll
                for (int sub = 0; sub < C::SUB; sub++) {
                    if (u * C::SUB + sub >= num_kb) break;
                    const uint8_t *w_tile = MODE == MODE_W8A16 ? conv + (cv.index * C::SUB + sub) * C::W_BYTES : stage;
                    const uint8_t *x_tile = MODE == MODE_W8A16 ? stage + sub * x_tile_bytes : stage + C::W_BYTES;
                    const uint64_t w_desc = umma_smem_desc_sw128(smem_u32(w_tile)), x_desc = umma_smem_desc_sw128(smem_u32(x_tile));
                    const uint32_t accumulate = u > unit_begin || sub > 0;
#pragma unroll
                    for (int k4 = 0; k4 < 4; k4++) {
                        if (MODE == MODE_W8A8) umma_i8(tmem_base + k4 * tokens16, w_desc + 2 * k4, x_desc + 2 * k4, idesc, accumulate);
                        else umma_bf16(tmem_base + k4 * tokens16, w_desc + 2 * k4, x_desc + 2 * k4, idesc, accumulate);
                    }
                }
                umma_commit(&empty[st.index]);
                st.advance(stages);
                if (MODE == MODE_W8A16) { umma_commit(&bempty[cv.index]); cv.advance(C::CONV_BUFFERS); }
            }
            if (!failure) umma_commit(tfull);
        }
    } else if (MODE == MODE_W8A16 && warp >= C::FIRST_DEQUANT_WARP) {
        /* ------------------------------------------------ dequantisers: group g converts units g, g + GROUPS, ... */
        const uint32_t group = (warp - C::FIRST_DEQUANT_WARP) / C::GROUP_WARPS;
        const uint32_t r = threadIdx.x - (C::FIRST_DEQUANT_WARP + C::GROUP_WARPS * group) * 32;   /* weight row of the tile */
        const uint32_t twist = r & 7;
        const uint32_t width = p.scale_group ? p.scale_group : p.K;
        const bool live = n0 + r < p.N;
        const float *row_scales = p.w_scales + (size_t)(live ? n0 + r : 0) * p.scale_groups;
        auto scales_of = [&](uint32_t u, float &s0, float &s1) {
            const uint32_t k0 = u * C::UNIT, k1 = k0 + C::BKE;
            s0 = live ? row_scales[k0 / width] : 0.0f;
            s1 = live && k1 < p.K ? row_scales[k1 / width] : s0;
        };
        PipeState sr, cv;
        float upcoming0 = 0.0f, upcoming1 = 0.0f;
        if (unit_begin + group < unit_end) scales_of(unit_begin + group, upcoming0, upcoming1);
        for (uint32_t u = unit_begin; u < unit_end; u++) {
            if ((u - unit_begin) % C::GROUPS != group) { sr.advance(C::RAW_STAGES); cv.advance(C::CONV_BUFFERS); continue; }
            const float scale[2] = {upcoming0, upcoming1};
            if (p.scale_groups > 1 && u + C::GROUPS < unit_end) scales_of(u + C::GROUPS, upcoming0, upcoming1);
            bool ready = wait_or_abort(&rfull[sr.index], sr.phase, abort_flag);
            ready = ready && wait_or_abort(&bempty[cv.index], cv.phase ^ 1, abort_flag);
            if (!__all_sync(0xffffffffu, ready)) { failure = STATUS_WAIT_DEQUANT; break; }
            const uint8_t *raw = raw_ring + sr.index * C::RAW_BYTES + r * 128;
            uint8_t *dst = conv + cv.index * C::SUB * C::W_BYTES + r * 128;
            uint4 q[8];
#pragma unroll
            for (int c = 0; c < 8; c++) q[c] = *reinterpret_cast<const uint4 *>(raw + ((c ^ twist) << 4));
            __syncwarp();
            if (lane == 0) mbar_arrive(&rempty[sr.index]);     /* the raw tile is in registers */
#pragma unroll
            for (int c = 0; c < 8; c++) {
                uint4 lo, hi;
                dequant16<true>(q[c], scale[c >> 2], lo, hi);
                uint8_t *tile_row = dst + (c >> 2) * C::W_BYTES;
                *reinterpret_cast<uint4 *>(tile_row + (((2 * (c & 3)) ^ twist) << 4)) = lo;
                *reinterpret_cast<uint4 *>(tile_row + (((2 * (c & 3) + 1) ^ twist) << 4)) = hi;
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bfull[cv.index]);
            sr.advance(C::RAW_STAGES);
            cv.advance(C::CONV_BUFFERS);
        }
    } else if (warp < C::EPILOGUE_WARPS) {
        /* ------------------------------------------------ accumulator -> this CTA's partial tile */
        /* thread = output channel n0 + 32 * warp + lane (its TMEM lane), registers = token rows */
        const uint32_t channel = warp * 32 + lane;
        if (unit_begin < unit_end) {
            bool ready = wait_or_abort(tfull, 0, abort_flag);
            if (!__all_sync(0xffffffffu, ready)) failure = STATUS_WAIT_EPILOGUE;
            tc_fence_after_sync();
        }
        /* tfull: every MMA of this CTA is done, so every tile the rings held has been read and no TMA write is pending */
        for (uint32_t c = 0; c < tokens16 / 16; c++) {
            uint32_t v[16];
            if (unit_begin < unit_end && !failure) {
                uint32_t more[3][16];
                tmem_load_32x16(tmem_base + ((warp * 32u) << 16) + c * 16, v);
#pragma unroll
                for (int j = 1; j < C::ACCUMULATORS; j++) tmem_load_32x16(tmem_base + ((warp * 32u) << 16) + j * tokens16 + c * 16, more[j - 1]);
                tmem_load_wait();
#pragma unroll
                for (int j = 1; j < C::ACCUMULATORS; j++)
#pragma unroll
                    for (int i = 0; i < 16; i++)
                        v[i] = MODE == MODE_W8A8 ? v[i] + more[j - 1][i]
                                                 : __float_as_uint(__fadd_rn(__uint_as_float(v[i]), __uint_as_float(more[j - 1][i])));
            } else {
#pragma unroll
                for (int j = 0; j < 16; j++) v[j] = 0;       /* a K slice without work contributes zeros */
            }
#pragma unroll
            for (int j = 0; j < 16; j++) partial[(c * 16 + j) * 128 + channel] = v[j];
        }
        tc_fence_before_sync();
    }

    /* ---------------------------------------------------------- reduction across the cluster and epilogue */
    if (failure) {
        *abort_flag = 1;
        atomicCAS(p.status, 0u, failure | (blockIdx.x << 8));
    }
    cluster_sync();                                   /* every CTA's partial tile is complete and visible */
    if (warp < C::EPILOGUE_WARPS) {
        /* CTA s owns token rows s, s + splits, ...; one work item = 8 consecutive channels of one such row: the partial
         * sums of every CTA (two 16-byte loads each through distributed shared memory), scales, bias, gate and residual
         * are all requested before the first is used, then summed in ascending split order */
        const bool gated = p.ep.gate != nullptr || p.ep.residual != nullptr;
        const uint32_t my_rows = split < p.M ? (p.M - split + splits - 1) / splits : 0;
        for (uint32_t item = threadIdx.x; item < my_rows * 16; item += C::EPILOGUE_WARPS * 32) {
            const uint32_t m = split + (item >> 4) * splits, col = (item & 15) * 8, n = n0 + col;
            if (n >= p.N) continue;
            const uint32_t own = smem_u32(partial + m * 128 + col);
            uint32_t bias[4] = {0, 0, 0, 0}, gate[4] = {0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u}, res[4] = {0, 0, 0, 0};
            if (p.ep.bias) *reinterpret_cast<uint4 *>(bias) = *reinterpret_cast<const uint4 *>(p.ep.bias + n);
            if (p.ep.gate) *reinterpret_cast<uint4 *>(gate) = *reinterpret_cast<const uint4 *>(p.ep.gate + n);
            if (p.ep.residual) *reinterpret_cast<uint4 *>(res) = *reinterpret_cast<const uint4 *>(p.ep.residual + (size_t)m * p.N + n);
            float lin[8];
            if (MODE == MODE_W8A8) {
                const float a_scale = p.a_scales[m];
                const float4 s0 = *reinterpret_cast<const float4 *>(p.w_scales + n), s1 = *reinterpret_cast<const float4 *>(p.w_scales + n + 4);
                const float ws[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
                int32_t sum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                for (uint32_t first = 0; first < splits; first += 4) {           /* four CTAs' sums in flight at a time */
                    uint4 v[4][2];
#pragma unroll
                    for (int s = 0; s < 4; s++) {
                        const uint32_t peer = map_to_cta(own, first + s < splits ? first + s : 0);
                        v[s][0] = first + s < splits ? load_cluster_u128(peer) : make_uint4(0, 0, 0, 0);
                        v[s][1] = first + s < splits ? load_cluster_u128(peer + 16) : make_uint4(0, 0, 0, 0);
                    }
#pragma unroll
                    for (int s = 0; s < 4; s++) {
                        const uint32_t w[8] = {v[s][0].x, v[s][0].y, v[s][0].z, v[s][0].w, v[s][1].x, v[s][1].y, v[s][1].z, v[s][1].w};
#pragma unroll
                        for (int j = 0; j < 8; j++) sum[j] += (int32_t)w[j];
                    }
                }
#pragma unroll
                for (int j = 0; j < 8; j++) lin[j] = __fmul_rn(__fmul_rn((float)sum[j], a_scale), ws[j]);
            } else {
                for (uint32_t first = 0; first < splits; first += 4) {
                    uint4 v[4][2];
#pragma unroll
                    for (int s = 0; s < 4; s++) {
                        const uint32_t peer = map_to_cta(own, first + s < splits ? first + s : 0);
                        v[s][0] = first + s < splits ? load_cluster_u128(peer) : make_uint4(0, 0, 0, 0);
                        v[s][1] = first + s < splits ? load_cluster_u128(peer + 16) : make_uint4(0, 0, 0, 0);
                    }
#pragma unroll
                    for (int s = 0; s < 4; s++) {
                        const uint32_t w[8] = {v[s][0].x, v[s][0].y, v[s][0].z, v[s][0].w, v[s][1].x, v[s][1].y, v[s][1].z, v[s][1].w};
#pragma unroll
                        for (int j = 0; j < 8; j++)
                            if (first + s == 0) lin[j] = __uint_as_float(w[j]);
                            else if (first + s < splits) lin[j] = __fadd_rn(lin[j], __uint_as_float(w[j]));
                    }
                }
            }
            uint32_t packed[4];
#pragma unroll
            for (int j = 0; j < 4; j++)
                packed[j] = epilogue_pair(lin[2 * j], lin[2 * j + 1], bias[j], p.ep.bias != nullptr, p.ep.activation, gated, gate[j], res[j]);
            *reinterpret_cast<uint4 *>(p.out + (size_t)m * p.N + n) = *reinterpret_cast<uint4 *>(packed);
        }
    }
    cluster_sync();                                   /* no CTA leaves while a peer may still read its partial tile */
    if (*abort_flag) {
        /* give any TMA copy still in flight time to land before the shared memory is released */
        long long start = clock64();
        while (clock64() - start < 2000000ll) { }
        __syncthreads();
    }
    if (warp == C::MMA_WARP) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, C::TMEM_COLUMNS);
    }
}

} /* namespace h3q8 */
