/* Two-CTA W8A8 GEMM with per-K-group scales (weight scales per group, activation scales
 * per group, or both): the int32 sum of every scale group is finished on the tensor cores,
 * handed to the epilogue warps through TMEM and combined there in fp32,
 *     total = sum over g ascending of (float(acc_g) * in_scale[m, g]) * w_scale[n, g],
 * which is the arithmetic of the reference's per-1024 FC2 recipe
 * (src/metal/shaders.metal:2701-2741) with the group scale on either operand.
 *
 * Differences from the per-channel pair kernel:
 *   - the fp32 totals of a tile live in registers for all of its groups, so the tile is
 *     256 x 128 per pair (each CTA: 128 rows x 128 columns = a quarter of the register file);
 *     a 256-wide tile spilled, and with 200 KB of shared memory carved out of L1 every
 *     spill goes to L2;
 *   - four TMEM accumulators of 128 columns are handed over per GROUP, not per tile: the MMA
 *     issuer runs up to three groups ahead of the epilogue;
 *   - 16 epilogue warps (TMEM lane quadrant = warp % 4, 32-column quarter = warp / 4): each
 *     thread owns one output row x 32 columns, pulls a group's sums in two 16-column TMEM
 *     loads and releases the accumulator once the second is in registers;
 *   - the two scale multiplies are packed f32x2 instructions; the running sum is a scalar
 *     add.rn per element, because the assembler contracts a packed multiply that feeds a
 *     packed add into one fused multiply-add, which is not the reference's rounding;
 *   - for groups of at most 256 the int32 -> fp32 conversion is the exact 1.5 * 2^23 bias
 *     trick (|acc_g| < 2^22 there): an integer add and a packed subtract per pair;
 *   - each warp stages the 32 weight scales of its columns for the group in its own
 *     shared memory (one load per lane, read back as broadcast vectors).
 * With 128-wide groups the epilogue (about 3.5 issue slots per element) is the bound, not
 * the tensor pipe: 128 x 128 elements per 256 MMA clocks per CTA. */
#pragma once
#include "gemm_tcgen05_pair.cuh"

namespace h3q8 {

/* WIDE = false: the shape described above, for narrow groups where the combine is the bound.
 * WIDE = true: 256 x 256 tiles, two accumulators, 8 epilogue warps with one row x 128 columns of totals per thread
 * (a quarter of the register file again, now in half as many threads): for groups of 512 and more the combine runs
 * once per four or more k-blocks and no longer bounds anything, so the tile that halves the operand traffic per flop
 * wins (the reference's per-1024 FC2 recipe). */
template <bool WIDE>
struct PairGroupedConfig {
    static constexpr int BM = 256, BN = WIDE ? 256 : 128, BKE = 128, ROW_BYTES = 128;
    static constexpr int A_BYTES = 128 * ROW_BYTES, B_BYTES = (BN / 2) * ROW_BYTES, STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = WIDE ? 6 : 8;
    static constexpr int ACC_COLS = BN, ACC_BUFFERS = 512 / BN;
    static constexpr int EPILOGUE_WARPS = WIDE ? 8 : 16, PRODUCER_WARP = EPILOGUE_WARPS, MMA_WARP = EPILOGUE_WARPS + 1;
    static constexpr int WARPS = EPILOGUE_WARPS + 2, THREADS = WARPS * 32;
    static constexpr int COLS = BN / (EPILOGUE_WARPS / 4);          /* output columns per epilogue thread: 32 or 128 */
    static constexpr int SCALE_BYTES = EPILOGUE_WARPS * 2 * COLS * 4; /* per warp: two buffers of COLS floats */
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + SCALE_BYTES + 1024 + 256;
    static constexpr uint32_t IDESC = umma_idesc(2, 1, 256, BN);
};

/* MAGIC: scale groups of at most 256 elements, so every group sum fits the 2^22 bias trick. */
template <bool MAGIC, bool WIDE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PairGroupedConfig<WIDE>::THREADS, 1)
gemm_tcgen05_pair_grouped_kernel(const __grid_constant__ PairArgs args) {
    using C = PairGroupedConfig<WIDE>;
    const uint32_t total_tiles = args.tile_start[args.count];
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *stages = smem;
    float *scale_stage = reinterpret_cast<float *>(stages + C::STAGES * C::STAGE_BYTES);
    uint64_t *bars = reinterpret_cast<uint64_t *>(stages + C::STAGES * C::STAGE_BYTES + C::SCALE_BYTES);
    uint64_t *full = bars, *empty = full + C::STAGES;
    uint64_t *tfull = empty + C::STAGES, *tempty = tfull + C::ACC_BUFFERS;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tempty + C::ACC_BUFFERS);
    volatile uint32_t *abort_flag = tmem_slot + 1;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();               /* 0 = leader */
    const uint32_t pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int s = 0; s < C::ACC_BUFFERS; s++) { mbar_init(&tfull[s], 1); mbar_init(&tempty[s], 2 * C::EPILOGUE_WARPS); }
        control_block_init(tmem_slot, args.p[0].wait_limit);
        fence_barrier_init();
        fence_proxy_async_smem();
    }
    if (warp == C::PRODUCER_WARP && lane == 0)
        for (uint32_t g = 0; g < args.count; g++) { tma_prefetch_descriptor(&args.map_a[g]); tma_prefetch_descriptor(&args.map_b[g]); }
    if (warp == C::MMA_WARP) { tmem_alloc_pair(tmem_slot, 512); tmem_relinquish_pair(); }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync();           /* both CTAs' barriers exist before anything crosses the pair */
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    uint32_t failure = STATUS_OK;

    if (warp == C::PRODUCER_WARP) {
        if (lane == 0) {
            PipeState st;
            for (uint32_t tile = pair; tile < total_tiles && !failure; tile += pairs) {
                uint32_t local, mb, nb;
                const uint32_t g = locate_problem(args, tile, local);
                const GemmParams &p = args.p[g];
                const CUtensorMap &map_a = args.map_a[g], &map_b = args.map_b[g];
                const uint32_t num_kb = p.K / C::BKE;
                tile_coordinates(p, local, mb, nb);
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    if (!wait_or_abort(&empty[st.index], st.phase ^ 1, abort_flag)) { failure = STATUS_WAIT_PRODUCER; break; }
                    uint8_t *stage = stages + st.index * C::STAGE_BYTES;
                    if (rank == 0) mbar_arrive_expect_tx(&full[st.index], 2 * C::STAGE_BYTES);
                    const uint32_t leader_full = map_to_cta(smem_u32(&full[st.index]), 0);
                    tma_load_2d_pair(stage, &map_a, leader_full, (int32_t)(kb * C::BKE), (int32_t)(mb * C::BM + rank * 128), p.l2_policy_a);
                    tma_load_2d_pair(stage + C::A_BYTES, &map_b, leader_full, (int32_t)(kb * C::BKE), (int32_t)(nb * C::BN + rank * (C::BN / 2)),
                                     p.l2_policy_b);
                    st.advance(C::STAGES);
                }
            }
        }
    } else if (warp == C::MMA_WARP) {
        if (lane == 0 && rank == 0) {
            PipeState st, acc;
            for (uint32_t tile = pair; tile < total_tiles && !failure; tile += pairs) {
                uint32_t local;
                const uint32_t g = locate_problem(args, tile, local);
                const uint32_t group_kb = args.p[g].scale_group / C::BKE, groups = args.p[g].K / args.p[g].scale_group;
                for (uint32_t group = 0; group < groups && !failure; group++) {
                    if (!wait_or_abort(&tempty[acc.index], acc.phase ^ 1, abort_flag)) { failure = STATUS_WAIT_MMA; break; }
                    tc_fence_after_sync();
                    const uint32_t d = tmem_base + acc.index * C::ACC_COLS;
                    for (uint32_t kb = 0; kb < group_kb; kb++) {
                        if (!wait_or_abort(&full[st.index], st.phase, abort_flag)) { failure = STATUS_WAIT_MMA; break; }
                        tc_fence_after_sync();
                        uint8_t *stage = stages + st.index * C::STAGE_BYTES;
                        const uint64_t a_desc = umma_smem_desc_sw128(smem_u32(stage));
                        const uint64_t b_desc = umma_smem_desc_sw128(smem_u32(stage + C::A_BYTES));
#pragma unroll
                        for (int k4 = 0; k4 < 4; k4++) umma_i8_pair(d, a_desc + 2 * k4, b_desc + 2 * k4, C::IDESC, kb | k4);
                        umma_commit_pair(&empty[st.index], 3);   /* frees the stage in both CTAs */
                        st.advance(C::STAGES);
                    }
                    if (failure) break;
                    umma_commit_pair(&tfull[acc.index], 3);      /* this group's int32 sums are complete */
                    acc.advance(C::ACC_BUFFERS);
                }
            }
        }
    } else {
        /* epilogue: this CTA's 128 rows; TMEM lane quadrant warp % 4, columns (warp / 4) * COLS .. + COLS - 1 */
        constexpr int COLS = C::COLS, PER_LANE = COLS / 32;
        const uint32_t quadrant = warp & 3, quarter = warp >> 2;
        float *my_scales = scale_stage + warp * 2 * COLS;
        const uint64_t bias2 = f32x2(-12582912.0f, -12582912.0f);
        PipeState acc;
        for (uint32_t tile = pair; tile < total_tiles && !failure; tile += pairs) {
            uint32_t local, mb, nb;
            const uint32_t problem = locate_problem(args, tile, local);
            const GemmParams &p = args.p[problem];
            const bool gated = p.ep.gate != nullptr || p.ep.residual != nullptr;
            tile_coordinates(p, local, mb, nb);
            const uint32_t n0 = nb * C::BN + quarter * COLS;
            const uint32_t groups = p.K / p.scale_group, wg = p.scale_groups, ag = p.a_scale_groups;
            const uint32_t row = mb * C::BM + rank * 128 + quadrant * 32 + lane;
            const bool row_ok = row < p.M;
            const float *a_row = p.a_scales + (size_t)(row_ok ? row : 0) * ag;
            /* this lane fetches the scales of columns n0 + lane + 32 i for the whole warp */
            float next_w[PER_LANE], next_a = row_ok ? a_row[0] : 0.0f;
            auto weight_scale = [&](int i, uint32_t group) {
                const uint32_t column = n0 + lane + 32 * i;
                return column < p.N ? p.w_scales[(size_t)column * wg + group] : 0.0f;
            };
#pragma unroll
            for (int i = 0; i < PER_LANE; i++) next_w[i] = weight_scale(i, 0);
            /* -0 + x == x for every x, so the first group's value is taken as it is */
            float total[COLS];
#pragma unroll
            for (int i = 0; i < COLS; i++) total[i] = -0.0f;

            /* every lane has finished reading the scales the previous tile staged (lanes diverge on row_ok before this) */
            __syncwarp();
            for (uint32_t group = 0; group < groups; group++) {
                float *buffer = my_scales + (wg > 1 ? (group & 1u) * COLS : 0u);
                if (group == 0 || wg > 1) {
#pragma unroll
                    for (int i = 0; i < PER_LANE; i++) buffer[lane + 32 * i] = next_w[i];
                }
                const uint64_t a2 = f32x2(next_a, next_a);
                __syncwarp();
                if (group + 1 < groups) {           /* next group's scales travel while this group is combined */
                    if (wg > 1) {
#pragma unroll
                        for (int i = 0; i < PER_LANE; i++) next_w[i] = weight_scale(i, group + 1);
                    }
                    if (ag > 1) next_a = row_ok ? a_row[group + 1] : 0.0f;
                }
                bool ready = wait_or_abort(&tfull[acc.index], acc.phase, abort_flag);
                if (!__all_sync(0xffffffffu, ready)) { failure = STATUS_WAIT_EPILOGUE; break; }
                tc_fence_after_sync();
                const uint32_t taddr = tmem_base + ((quadrant * 32u) << 16) + acc.index * C::ACC_COLS + quarter * COLS;
#pragma unroll
                for (int c2 = 0; c2 < COLS / 16; c2++) {
                    uint32_t v[16];
                    tmem_load_32x16(taddr + c2 * 16, v);
                    tmem_load_wait();
                    if (c2 == COLS / 16 - 1) {      /* everything this warp needs is in registers: the MMA issuer may refill */
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) {
                            if (rank == 0) mbar_arrive(&tempty[acc.index]);
                            else mbar_arrive_remote(map_to_cta(smem_u32(&tempty[acc.index]), 0));
                        }
                    }
#pragma unroll
                    for (int j4 = 0; j4 < 4; j4++) {
                        const float4 w = *reinterpret_cast<const float4 *>(buffer + c2 * 16 + j4 * 4);
                        uint64_t f0, f1;
                        if (MAGIC) {
                            f0 = add_f32x2(f32x2(__int_as_float((int32_t)v[j4 * 4 + 0] + 0x4B400000), __int_as_float((int32_t)v[j4 * 4 + 1] + 0x4B400000)), bias2);
                            f1 = add_f32x2(f32x2(__int_as_float((int32_t)v[j4 * 4 + 2] + 0x4B400000), __int_as_float((int32_t)v[j4 * 4 + 3] + 0x4B400000)), bias2);
                        } else {
                            f0 = f32x2((float)(int32_t)v[j4 * 4 + 0], (float)(int32_t)v[j4 * 4 + 1]);
                            f1 = f32x2((float)(int32_t)v[j4 * 4 + 2], (float)(int32_t)v[j4 * 4 + 3]);
                        }
                        float p0, p1, p2, p3;
                        f32x2_unpack(mul_f32x2(mul_f32x2(f0, a2), f32x2(w.x, w.y)), p0, p1);
                        f32x2_unpack(mul_f32x2(mul_f32x2(f1, a2), f32x2(w.z, w.w)), p2, p3);
                        const int t = c2 * 16 + j4 * 4;
                        total[t + 0] = __fadd_rn(total[t + 0], p0);
                        total[t + 1] = __fadd_rn(total[t + 1], p1);
                        total[t + 2] = __fadd_rn(total[t + 2], p2);
                        total[t + 3] = __fadd_rn(total[t + 3], p3);
                    }
                }
                acc.advance(C::ACC_BUFFERS);
            }
            if (failure) break;
            if (row_ok) {
#pragma unroll
                for (int j8 = 0; j8 < COLS / 8; j8++) {
                    const uint32_t col = n0 + j8 * 8;
                    if (col >= p.N) continue;       /* N is a multiple of 8 on this path */
                    float lin[8];
#pragma unroll
                    for (int j = 0; j < 8; j++) lin[j] = total[j8 * 8 + j];
                    uint32_t bias[4] = {0, 0, 0, 0}, gate[4] = {0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u};
                    uint32_t res[4] = {0, 0, 0, 0};
                    if (p.ep.bias) *reinterpret_cast<uint4 *>(bias) = *reinterpret_cast<const uint4 *>(p.ep.bias + col);
                    if (p.ep.gate) *reinterpret_cast<uint4 *>(gate) = *reinterpret_cast<const uint4 *>(p.ep.gate + col);
                    if (p.ep.residual)
                        *reinterpret_cast<uint4 *>(res) = *reinterpret_cast<const uint4 *>(p.ep.residual + (size_t)row * p.N + col);
                    uint32_t packed[4];
#pragma unroll
                    for (int j = 0; j < 4; j++)
                        packed[j] = epilogue_pair(lin[2 * j], lin[2 * j + 1], bias[j], p.ep.bias != nullptr, p.ep.activation,
                                                  gated, gate[j], res[j]);
                    *reinterpret_cast<uint4 *>(p.out + (size_t)row * p.N + col) = *reinterpret_cast<uint4 *>(packed);
                }
            }
        }
    }

    if (failure) {
        *abort_flag = 1;
        atomicCAS(args.p[0].status, 0u, failure | (blockIdx.x << 8));
    }
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        long long start = clock64();
        while (clock64() - start < 2000000ll) { }
        __syncthreads();
    }
    cluster_sync();           /* the peer may still be read by the leader's MMAs until here */
    if (warp == C::MMA_WARP) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

} /* namespace h3q8 */
