/* Two-CTA variant of the tcgen05 GEMM: a cluster of two CTAs (one SM each)
 * computes a 256 x 256 output tile with `tcgen05.mma.cta_group::2`.
 *
 * Why: with one CTA per tile every 128 x 256 x 16 MMA reads 12 KB of operands
 * from that SM's shared memory while TMA writes the same amount, and shared
 * memory bandwidth (not the tensor pipe) sets the pace.  In a pair each CTA
 * stages its own 128 rows of A and only HALF of the weight tile (128 of the 256
 * output channels); the tensor cores of the two SMs exchange the B halves, so
 * per-SM shared-memory traffic per flop drops by a third and the stage shrinks
 * from 48 KB to 32 KB (6 stages instead of 4).
 *
 * Protocol (leader = CTA rank 0 of the pair):
 *   - both CTAs run a TMA producer for their own tiles; completion bytes of both
 *     are counted on the leader's `full` barrier (the loads carry `.cta_group::2`
 *     and name the leader's barrier); each CTA has its own `empty` barriers
 *   - only the leader issues MMAs; `tcgen05.commit` arrives on the `empty` /
 *     `tfull` barriers of both CTAs at once
 *   - both CTAs run the epilogue on their own 128 accumulator rows (their own
 *     TMEM); epilogue warps of both arrive on the leader's `tempty` barrier
 *   - TMEM is allocated and freed by the same warp of both CTAs; a cluster
 *     barrier brackets the kernel so that neither CTA leaves while the other can
 *     still touch its shared memory or TMEM
 * Modes: MODE_BF16 and MODE_W8A8 (per-channel scales).  All waits are bounded
 * as in the single-CTA kernel.
 *
 * One launch can carry up to PAIR_MAX_PROBLEMS independent problems of different
 * shapes (the video and audio streams of the DiT): the tile index space is the
 * concatenation of the problems' tiles, each with its own tensor maps and
 * parameters, and all of them flow through the same TMA / MMA / TMEM pipeline
 * without draining it between problems.
 */
#pragma once
#include "gemm_tcgen05.cuh"

namespace h3q8 {

/* EPILOGUE_WARPS: 8 = each warp a column half of the tile, 16 = a column quarter (the rotary epilogue keeps a whole
 * 128-wide head row per thread and stays at 8).  Sixteen warps cover the TMEM and global-memory latencies of the
 * epilogue better; they pay where the epilogue is exposed: int8 tiles, whose main loop is half as long for the same
 * epilogue (measured on one box at M = 32 400: QKV 2 302 -> 2 513, attention-out 1 770 -> 1 842, FFN-up 2 154 -> 2 487,
 * FFN-down 2 319 -> 2 296 TOP/s; the 4 096-row W8A8 linear 58.1 -> 45.1 us), and bf16 problems of few tile waves, where
 * the last tile's epilogue is not hidden (4 096 x 3 072 x 3 072: 66.9 -> 63.8 us).  At M = 32 400 the bf16 kernel loses
 * 1 % with sixteen, so the launcher picks by mode and row count. */
template <int MODE, bool ROPE = false, int EPILOGUE_WARPS_ = 8>
struct PairConfig {
    static constexpr int BM = 256, BN = 256;           /* per pair */
    static constexpr int ROW_BYTES = 128;
    static constexpr int BKE = MODE == MODE_W8A8 ? 128 : 64;
    static constexpr int A_BYTES = 128 * ROW_BYTES;     /* this CTA's 128 rows of A         */
    static constexpr int B_BYTES = 128 * ROW_BYTES;     /* this CTA's 128 output channels   */
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = 6;
    static constexpr int ACC_COLS = BN, ACC_BUFFERS = 2;
    static constexpr int EPILOGUE_WARPS = EPILOGUE_WARPS_;
    static constexpr int PRODUCER_WARP = EPILOGUE_WARPS, MMA_WARP = EPILOGUE_WARPS + 1, WARPS = EPILOGUE_WARPS + 2, THREADS = WARPS * 32;
    static_assert(EPILOGUE_WARPS == 8 || (EPILOGUE_WARPS == 16 && !ROPE), "column halves, or quarters for the plain epilogues");
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
    static constexpr uint32_t IDESC = MODE == MODE_W8A8 ? umma_idesc(2, 1, 256, BN) : umma_idesc(1, 1, 256, BN);
    static_assert(MODE == MODE_BF16 || MODE == MODE_W8A8, "pair kernel: bf16 or int8 operands");
};

constexpr int PAIR_MAX_PROBLEMS = 4;
struct alignas(64) PairArgs {
    CUtensorMap map_a[PAIR_MAX_PROBLEMS];
    CUtensorMap map_b[PAIR_MAX_PROBLEMS];
    GemmParams p[PAIR_MAX_PROBLEMS];
    uint32_t tile_start[PAIR_MAX_PROBLEMS + 1]; /* first global tile index of each problem; [count] = total */
    uint32_t count;
};
/* problem that owns global tile `tile`, and the tile's index inside it */
__device__ __forceinline__ uint32_t locate_problem(const PairArgs &args, uint32_t tile, uint32_t &local) {
    uint32_t g = 0;
#pragma unroll
    for (int i = 1; i < PAIR_MAX_PROBLEMS; i++)
        if (i < (int)args.count && tile >= args.tile_start[i]) g = i;
    local = tile - args.tile_start[g];
    return g;
}

/* ROPE selects the QKV norm + rotary epilogue (its own instantiation: it keeps a whole
 * 128-wide head row in registers, which the other epilogues should not pay for). */
template <int MODE, bool ROPE, int EPILOGUE_WARPS>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PairConfig<MODE, ROPE, EPILOGUE_WARPS>::THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ PairArgs args) {
    using C = PairConfig<MODE, ROPE, EPILOGUE_WARPS>;
    const uint32_t total_tiles = args.tile_start[args.count];
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *stages = smem;
    uint64_t *bars = reinterpret_cast<uint64_t *>(stages + C::STAGES * C::STAGE_BYTES);
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
            if (args.p[0].wait_previous) grid_dependency_wait();   /* an operand is still being written by the previous kernel */
            PipeState st;
            for (uint32_t tile = pair; tile < total_tiles && !failure; tile += pairs) {
                uint32_t local, mb, nb;
                const uint32_t g = locate_problem(args, tile, local);
                const GemmParams &p = args.p[g];
                const CUtensorMap &map_a = args.map_a[g], &map_b = args.map_b[g];
                const uint32_t num_kb = (p.K + C::BKE - 1) / C::BKE;
                tile_coordinates(p, local, mb, nb);
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    if (!wait_or_abort(&empty[st.index], st.phase ^ 1, abort_flag)) { failure = STATUS_WAIT_PRODUCER; break; }
                    uint8_t *stage = stages + st.index * C::STAGE_BYTES;
                    if (p.skip_first_load && tile == pair && kb == 0) { st.advance(C::STAGES); continue; }   /* injected fault */
                    /* the leader arms its barrier for the bytes of both CTAs */
                    if (rank == 0) mbar_arrive_expect_tx(&full[st.index], 2 * C::STAGE_BYTES);
                    const uint32_t leader_full = map_to_cta(smem_u32(&full[st.index]), 0);
                    tma_load_2d_pair(stage, &map_a, leader_full, (int32_t)(kb * C::BKE), (int32_t)(mb * C::BM + rank * 128), p.l2_policy_a);
                    /* SwiGLU: the leader stages 128 gate rows, its peer the matching 128 up rows (weight rows N + n) */
                    const uint32_t b_row = p.ep.activation == ACT_SWIGLU ? nb * 128 + rank * p.N : nb * C::BN + rank * 128;
                    tma_load_2d_pair(stage + C::A_BYTES, &map_b, leader_full, (int32_t)(kb * C::BKE), (int32_t)b_row, p.l2_policy_b);
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
                const uint32_t num_kb = (args.p[g].K + C::BKE - 1) / C::BKE;
                if (!wait_or_abort(&tempty[acc.index], acc.phase ^ 1, abort_flag)) { failure = STATUS_WAIT_MMA; break; }
                tc_fence_after_sync();
                const uint32_t d = tmem_base + acc.index * C::ACC_COLS;
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    if (!wait_or_abort(&full[st.index], st.phase, abort_flag)) { failure = STATUS_WAIT_MMA; break; }
                    tc_fence_after_sync();
                    uint8_t *stage = stages + st.index * C::STAGE_BYTES;
                    const uint64_t a_desc = umma_smem_desc_sw128(smem_u32(stage));
                    const uint64_t b_desc = umma_smem_desc_sw128(smem_u32(stage + C::A_BYTES));
#pragma unroll
                    for (int k4 = 0; k4 < 4; k4++) {
                        if (MODE == MODE_W8A8) umma_i8_pair(d, a_desc + 2 * k4, b_desc + 2 * k4, C::IDESC, kb | k4);
                        else umma_bf16_pair(d, a_desc + 2 * k4, b_desc + 2 * k4, C::IDESC, kb | k4);
                    }
                    umma_commit_pair(&empty[st.index], 3);   /* frees the stage in both CTAs */
                    st.advance(C::STAGES);
                }
                if (failure) break;
                umma_commit_pair(&tfull[acc.index], 3);
                acc.advance(C::ACC_BUFFERS);
            }
        }
    } else {
        /* epilogue: this CTA's 128 rows, TMEM lane quadrant warp % 4, column half warp / 4 */
        constexpr int SPLIT = C::EPILOGUE_WARPS / 4;          /* column parts of the tile: halves or quarters */
        constexpr int HALF_CHUNKS = C::BN / 32 / SPLIT;        /* 32-column chunks per warp */
        static_assert(!ROPE || SPLIT == 2, "the rotary epilogue owns a 128-column group per warp");
        const uint32_t quadrant = warp & 3, half = warp >> 2;
        PipeState acc;
        for (uint32_t tile = pair; tile < total_tiles && !failure; tile += pairs) {
            uint32_t local, mb, nb;
            const uint32_t g = locate_problem(args, tile, local);
            const GemmParams &p = args.p[g];
            const bool gated = p.ep.gate != nullptr || p.ep.residual != nullptr;
            tile_coordinates(p, local, mb, nb);
            const bool swiglu = p.ep.activation == ACT_SWIGLU;
            const uint32_t n0 = swiglu ? nb * 128 : nb * C::BN;
            bool ready = wait_or_abort(&tfull[acc.index], acc.phase, abort_flag);
            if (!__all_sync(0xffffffffu, ready)) { failure = STATUS_WAIT_EPILOGUE; break; }
            tc_fence_after_sync();
            const uint32_t row = mb * C::BM + rank * 128 + quadrant * 32 + lane;
            const bool row_ok = row < p.M;
            float a_scale = 1.0f;
            if (MODE == MODE_W8A8) a_scale = row_ok ? p.a_scales[row] : 0.0f;
            if (ROPE) {
                /* each 128-column group is one (head, q|k|v) stream; this warp owns the group `half` of the tile and
                 * every thread keeps its row's 128 bf16 values in registers between the norm and the rotation */
                const uint32_t block = nb * 2 + half;
                if (block * 128 < p.N) {
                    const uint32_t head = block / 3, which = block - head * 3;
                    uint32_t xp[64];
                    float sum = 0.0f;
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        uint32_t v[32];
                        tmem_load_32x32(tmem_base + ((quadrant * 32u) << 16) + acc.index * C::ACC_COLS + half * 128 + c * 32, v);
                        tmem_load_wait();
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            float l0, l1;
                            if (MODE == MODE_W8A8) {
                                const float2 ws = *reinterpret_cast<const float2 *>(p.w_scales + block * 128 + c * 32 + 2 * j);
                                l0 = __fmul_rn(__fmul_rn((float)(int32_t)v[2 * j], a_scale), ws.x);
                                l1 = __fmul_rn(__fmul_rn((float)(int32_t)v[2 * j + 1], a_scale), ws.y);
                            } else { l0 = __uint_as_float(v[2 * j]); l1 = __uint_as_float(v[2 * j + 1]); }
                            const uint32_t packed = pack_bf16_pair(l0, l1);
                            xp[c * 16 + j] = packed;
                            sum = fmaf(bf16_lo(packed), bf16_lo(packed), sum);
                            sum = fmaf(bf16_hi(packed), bf16_hi(packed), sum);
                        }
                    }
                    if (row_ok) {
                        if (p.out) {
#pragma unroll
                            for (int i = 0; i < 16; i++)
                                reinterpret_cast<uint4 *>(p.out + (size_t)row * p.N + block * 128)[i] = *reinterpret_cast<uint4 *>(&xp[4 * i]);
                        }
                        const RopeParams &rp = p.ep.rope;
                        uint16_t *dst = (which == 0 ? rp.query : which == 1 ? rp.key : rp.value) + ((size_t)row * rp.heads + head) * 128;
                        if (which == 2) {
#pragma unroll
                            for (int i = 0; i < 16; i++) reinterpret_cast<uint4 *>(dst)[i] = *reinterpret_cast<uint4 *>(&xp[4 * i]);
                        } else {
                            const uint16_t *norm = which == 0 ? rp.q_norm : rp.k_norm;
                            const uint16_t *cos_row = rp.cos + (size_t)row * rp.rope_half, *sin_row = rp.sin + (size_t)row * rp.rope_half;
                            if (rp.rope_half == 48) qkv_rope_store<48>(xp, sum, norm, cos_row, sin_row, rp.epsilon, dst);
                            else qkv_rope_store<64>(xp, sum, norm, cos_row, sin_row, rp.epsilon, dst);
                        }
                    }
                }
            } else if (!ROPE && swiglu) {
                /* accumulator columns 0..127 hold the gate, 128..255 the up projection of the same 128 outputs */
#pragma unroll 1
                for (int hc = 0; hc < 4 / SPLIT; hc++) {
                    const int c = half * (4 / SPLIT) + hc;
                    uint32_t vg[32], vu[32];
                    const uint32_t taddr = tmem_base + ((quadrant * 32u) << 16) + acc.index * C::ACC_COLS + c * 32;
                    tmem_load_32x32(taddr, vg);
                    tmem_load_32x32(taddr + 128, vu);
                    tmem_load_wait();
                    if (!row_ok) continue;
#pragma unroll
                    for (int j8 = 0; j8 < 4; j8++) {
                        const uint32_t col = n0 + c * 32 + j8 * 8;
                        if (col >= p.N) continue;
                        float gl[8], ul[8];
                        if (MODE == MODE_W8A8) {
                            float4 g0 = *reinterpret_cast<const float4 *>(p.w_scales + col), g1 = *reinterpret_cast<const float4 *>(p.w_scales + col + 4);
                            float4 u0 = *reinterpret_cast<const float4 *>(p.w_scales + p.N + col), u1 = *reinterpret_cast<const float4 *>(p.w_scales + p.N + col + 4);
                            const float wg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
                            const float wu[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
                            for (int j = 0; j < 8; j++) {
                                gl[j] = __fmul_rn(__fmul_rn((float)(int32_t)vg[j8 * 8 + j], a_scale), wg[j]);
                                ul[j] = __fmul_rn(__fmul_rn((float)(int32_t)vu[j8 * 8 + j], a_scale), wu[j]);
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 8; j++) { gl[j] = __uint_as_float(vg[j8 * 8 + j]); ul[j] = __uint_as_float(vu[j8 * 8 + j]); }
                        }
                        if (p.ep.bias) {
                            uint32_t bg[4], bu[4];
                            *reinterpret_cast<uint4 *>(bg) = *reinterpret_cast<const uint4 *>(p.ep.bias + col);
                            *reinterpret_cast<uint4 *>(bu) = *reinterpret_cast<const uint4 *>(p.ep.bias + p.N + col);
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                gl[2 * j] = __fadd_rn(gl[2 * j], bf16_lo(bg[j])); gl[2 * j + 1] = __fadd_rn(gl[2 * j + 1], bf16_hi(bg[j]));
                                ul[2 * j] = __fadd_rn(ul[2 * j], bf16_lo(bu[j])); ul[2 * j + 1] = __fadd_rn(ul[2 * j + 1], bf16_hi(bu[j]));
                            }
                        }
                        uint32_t packed[4];
#pragma unroll
                        for (int j = 0; j < 4; j++)
                            packed[j] = pack_bf16_pair(swiglu_f32(gl[2 * j], ul[2 * j], MODE != MODE_W8A8),
                                                       swiglu_f32(gl[2 * j + 1], ul[2 * j + 1], MODE != MODE_W8A8));
                        *reinterpret_cast<uint4 *>(p.out + (size_t)row * p.N + col) = *reinterpret_cast<uint4 *>(packed);
                    }
                }
            } else if (!ROPE)
#pragma unroll 1
            for (int hc = 0; hc < HALF_CHUNKS; hc++) {
                const int c = half * HALF_CHUNKS + hc;
                uint32_t v[32];
                tmem_load_32x32(tmem_base + ((quadrant * 32u) << 16) + acc.index * C::ACC_COLS + c * 32, v);
                tmem_load_wait();
                const uint32_t col0 = n0 + c * 32;
                if (!row_ok) continue;
                if (p.acc_dump) {   /* raw accumulators: int32 sums (W8A8) or fp32 partial sums (bf16 operands) */
#pragma unroll
                    for (int j8 = 0; j8 < 4; j8++)
                        if (col0 + j8 * 8 < p.N) {
                            int4 *dst = reinterpret_cast<int4 *>(p.acc_dump + (size_t)row * p.N + col0 + j8 * 8);
                            dst[0] = make_int4(v[j8 * 8 + 0], v[j8 * 8 + 1], v[j8 * 8 + 2], v[j8 * 8 + 3]);
                            dst[1] = make_int4(v[j8 * 8 + 4], v[j8 * 8 + 5], v[j8 * 8 + 6], v[j8 * 8 + 7]);
                        }
                    if (!p.out) continue;   /* a partial-sum call stores nothing else */
                }
#pragma unroll
                for (int j8 = 0; j8 < 4; j8++) {
                    const uint32_t col = col0 + j8 * 8;
                    if (col >= p.N) continue;
                    float lin[8];
                    if (MODE == MODE_W8A8) {
                        float4 s0 = *reinterpret_cast<const float4 *>(p.w_scales + col);
                        float4 s1 = *reinterpret_cast<const float4 *>(p.w_scales + col + 4);
                        const float ws[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
                        for (int j = 0; j < 8; j++)
                            lin[j] = __fmul_rn(__fmul_rn((float)(int32_t)v[j8 * 8 + j], a_scale), ws[j]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; j++) lin[j] = __uint_as_float(v[j8 * 8 + j]);
                    }
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
            /* this warp is done with the accumulator: tell the leader's MMA issuer */
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if (rank == 0) mbar_arrive(&tempty[acc.index]);
                else mbar_arrive_remote(map_to_cta(smem_u32(&tempty[acc.index]), 0));
            }
            acc.advance(C::ACC_BUFFERS);
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
