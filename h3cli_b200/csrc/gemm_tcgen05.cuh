/* Persistent, warp-specialised tcgen05 GEMM for the q8 DiT linears (sm_100a).
 *
 *   out[M,N] = epilogue( X[M,K] . W[N,K]^T )
 *
 * Three operand modes share one pipeline:
 *   MODE_BF16   X bf16, W bf16            TMA -> smem -> kind::f16 MMA  (fp32 in TMEM)
 *   MODE_W8A16  X bf16, W int8 + scales   TMA -> smem -> dequant warps write
 *                                         bf16(float(q)*scale) tiles -> kind::f16 MMA
 *   MODE_W8A8   X int8, W int8            TMA -> smem -> kind::i8 MMA   (int32 in TMEM)
 *
 * One CTA per SM, static round-robin over output tiles of (128*MT) x BN.
 * Warp roles: 0-7 epilogue (TMEM lane quadrant = warp % 4, column half = warp / 4),
 * 8 TMA producer, 9 MMA issuer and TMEM owner, 10-17 dequantisers (MODE_W8A16 only).
 * Operand tiles are rows of 128 bytes in the 128-byte swizzle; one k-block is
 * 64 bf16 or 128 int8 elements = four MMA instructions per 128-row sub-tile.
 * Accumulators are double-buffered in TMEM whenever 2*MT*BN <= 512 columns so
 * the epilogue of one tile overlaps the main loop of the next.
 *
 * Every CTA fetches its own operand tiles; tiles that share weights are
 * co-scheduled so they meet in L2.
 */
#pragma once
#include "epilogue.cuh"

namespace h3q8 {

enum : int { MODE_BF16 = 0, MODE_W8A16 = 1, MODE_W8A8 = 2 };

enum : uint32_t {
    STATUS_OK = 0,
    STATUS_WAIT_PRODUCER = 1,  /* TMA producer gave up waiting for a free stage   */
    STATUS_WAIT_MMA = 2,       /* MMA issuer gave up waiting for operands / TMEM  */
    STATUS_WAIT_EPILOGUE = 3,  /* epilogue gave up waiting for an accumulator     */
    STATUS_WAIT_DEQUANT = 4,   /* dequantiser gave up waiting                     */
    STATUS_NONFINITE = 0x80000000u, /* OR-ed in by a quantiser or packer that met an Inf or a NaN */
};

struct GemmParams {
    uint32_t M, N, K;
    uint32_t scale_group;   /* K elements per scale group (weights and/or activations); 0 = none */
    uint32_t scale_groups;  /* scales per weight row (1 = per output channel)                    */
    uint32_t a_scale_groups;/* scales per activation row (1 = per token), MODE_W8A8              */
    const float *w_scales;  /* [N, scale_groups] (MODE_W8A16, MODE_W8A8)                     */
    const float *a_scales;  /* [M] per-token scales (MODE_W8A8)                              */
    EpilogueParams ep;
    uint16_t *out;          /* bf16 [M,N]                                                    */
    int32_t *acc_dump;      /* optional [M,N] raw accumulators: int32 (MODE_W8A8, ungrouped) or fp32 bits */
    uint32_t *status;       /* device error word, 0 = ok                                     */
    uint32_t m_blocks, n_blocks, tiles, band;
    uint64_t l2_policy_a, l2_policy_b; /* TMA L2 eviction policies for activations / weights (two-CTA kernel) */
    /* split-K (skinny M): `splits` CTAs share one output tile, each accumulates kb_per_split k-blocks and stores its raw
     * 32-bit accumulators at partials[(split * M + row) * N + col]; splitk_finish_kernel sums them and runs the epilogue */
    uint32_t splits, kb_per_split;
    uint32_t *partials;
    /* failure-path testing, set from the host (h3q8_fault_injection): a shorter limit for every bounded wait, and a
     * producer that leaves out the very first operand load, so that a wait runs out and the error path is exercised */
    long long wait_limit;
    uint32_t skip_first_load;
    /* launched as a programmatic dependent of the kernel that writes one of the operands: the producer role waits for
     * that grid (griddepcontrol.wait) before its first load */
    uint32_t wait_previous;
};

template <int MODE, int BN, int MT, bool GROUPED>
struct GemmConfig {
    static constexpr int BM = 128 * MT;
    static constexpr int ROW_BYTES = 128;
    static constexpr int BKE = MODE == MODE_W8A8 ? 128 : 64;   /* K elements per k-block */
    static constexpr int A_BYTES = BM * ROW_BYTES;
    static constexpr int B_BYTES = BN * ROW_BYTES;              /* MMA operand tile        */
    static constexpr int RAW_BYTES = MODE == MODE_W8A16 ? BN * 64 : 0;
    static constexpr int STAGE_BYTES = A_BYTES + (MODE == MODE_W8A16 ? RAW_BYTES : B_BYTES);
    /* converted-tile ring: four deep for the 128-wide tile (16 KB each), where skinny problems live on the latency of
     * the TMA -> convert -> MMA chain and the dequantisers must be able to run ahead of the tensor core */
    static constexpr int CONV_BUFFERS = MODE == MODE_W8A16 ? (BN == 128 && MT == 1 ? 4 : 2) : 0;
    static constexpr int SMEM_BUDGET = 227 * 1024 - 2048;
    static constexpr int STAGES_FIT = (SMEM_BUDGET - CONV_BUFFERS * B_BYTES) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_FIT > 6 ? 6 : STAGES_FIT;
    static constexpr int ACC_COLS = BN * MT;
    static constexpr int ACC_BUFFERS = 512 / ACC_COLS >= 2 ? 2 : 1;
    static constexpr int DEQUANT_WARPS = MODE == MODE_W8A16 ? 8 : 0;
    static constexpr int EPILOGUE_WARPS = 8;
    static constexpr int PRODUCER_WARP = EPILOGUE_WARPS, MMA_WARP = EPILOGUE_WARPS + 1, FIRST_DEQUANT_WARP = EPILOGUE_WARPS + 2;
    static constexpr int WARPS = EPILOGUE_WARPS + 2 + DEQUANT_WARPS;
    static constexpr int THREADS = WARPS * 32;
    static constexpr int BARRIERS = 2 * STAGES + 2 * CONV_BUFFERS + 2 * ACC_BUFFERS;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + CONV_BUFFERS * B_BYTES + 1024 /* align */ + 256;
    static constexpr uint32_t IDESC = MODE == MODE_W8A8 ? umma_idesc(2, 1, 128, BN) : umma_idesc(1, 1, 128, BN);
    static_assert(STAGES >= 2, "pipeline needs at least two stages");
    static_assert(ACC_COLS <= 512, "accumulator exceeds TMEM");
    static_assert(!GROUPED || (MODE == MODE_W8A8 && BN == 128 && MT == 1), "grouped epilogue shape");
};

struct PipeState {
    uint32_t index = 0, phase = 0;
    __device__ __forceinline__ void advance(uint32_t count) {
        if (++index == count) { index = 0; phase ^= 1; }
    }
};

/* Shared-memory control block behind the barriers of every kernel here: [0] TMEM base, [1] abort flag, [2..3] the
 * wait limit in clocks (GemmParams::wait_limit, else WAIT_LIMIT_CYCLES), written once by thread 0. */
__device__ __forceinline__ void control_block_init(uint32_t *tmem_slot, long long wait_limit) {
    tmem_slot[1] = 0;
    *reinterpret_cast<volatile long long *>(tmem_slot + 2) = wait_limit > 0 ? wait_limit : WAIT_LIMIT_CYCLES;
}
/* Bounded wait of a pipeline role.  False: this wait ran out, or another role of the CTA already gave up. */
__device__ __forceinline__ bool wait_or_abort(uint64_t *bar, uint32_t parity, volatile uint32_t *abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64(), limit = *reinterpret_cast<const volatile long long *>(abort_flag + 1);
    for (;;) {
#pragma unroll 1
        for (int spin = 0; spin < 128; spin++)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - start > limit) return false;
    }
}

/* Tile order: bands of `band` row blocks; inside a band the row block varies
 * fastest, so the CTAs running at one time share a few weight column blocks
 * and a few activation row blocks in L2. */
__device__ __forceinline__ void tile_coordinates(const GemmParams &p, uint32_t tile, uint32_t &mb, uint32_t &nb) {
    uint32_t per_band = p.band * p.n_blocks;
    uint32_t b = tile / per_band, within = tile - b * per_band;
    uint32_t first = b * p.band;
    uint32_t height = p.m_blocks - first < p.band ? p.m_blocks - first : p.band;
    nb = within / height;
    mb = first + (within - nb * height);
}

/* int8 x4 -> four fp32 holding float(q)*scale, exactly as fp32 multiply rounds it.
 * (q ^ 0x80) placed in the low mantissa byte of 2^23 gives 2^23 + q + 128. */
__device__ __forceinline__ void dequant4(uint32_t packed, float scale, float (&f)[4]) {
    uint32_t biased = packed ^ 0x80808080u;
    f[0] = __fmul_rn(__fsub_rn(__uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7650)), 8388736.0f), scale);
    f[1] = __fmul_rn(__fsub_rn(__uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7651)), 8388736.0f), scale);
    f[2] = __fmul_rn(__fsub_rn(__uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7652)), 8388736.0f), scale);
    f[3] = __fmul_rn(__fsub_rn(__uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7653)), 8388736.0f), scale);
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

template <int MODE, int BN, int MT, bool GROUPED, bool SPLITK = false>
__global__ void __launch_bounds__(GemmConfig<MODE, BN, MT, GROUPED>::THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const GemmParams p) {
    using C = GemmConfig<MODE, BN, MT, GROUPED>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *stages = smem;
    uint8_t *conv = stages + C::STAGES * C::STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(conv + C::CONV_BUFFERS * C::B_BYTES);
    uint64_t *full = bars, *empty = full + C::STAGES;
    uint64_t *bfull = empty + C::STAGES, *bempty = bfull + C::CONV_BUFFERS;
    uint64_t *tfull = bempty + C::CONV_BUFFERS, *tempty = tfull + C::ACC_BUFFERS;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tempty + C::ACC_BUFFERS);
    volatile uint32_t *abort_flag = tmem_slot + 1;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t num_kb = (p.K + C::BKE - 1) / C::BKE;
    /* k-blocks accumulated before the accumulator is handed to the epilogue */
    const uint32_t kb_per_chunk = GROUPED ? p.scale_group / C::BKE : num_kb;
    const uint32_t chunks = GROUPED ? (num_kb + kb_per_chunk - 1) / kb_per_chunk : 1;
    static_assert(!(GROUPED && SPLITK), "split-K hands raw sums to a second kernel; grouped scales are combined in this one");
    /* work items: output tiles, or (tile, K split) pairs */
    const uint32_t items = SPLITK ? p.tiles * p.splits : p.tiles;
#define H3Q8_ITEM(item, tile, kb_first, kb_last)                                                        \
    const uint32_t tile = SPLITK ? (item) / p.splits : (item);                                           \
    const uint32_t kb_first = SPLITK ? ((item) - tile * p.splits) * p.kb_per_split : 0;                  \
    const uint32_t kb_last = SPLITK ? (kb_first + p.kb_per_split < num_kb ? kb_first + p.kb_per_split : num_kb) : num_kb;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int s = 0; s < C::CONV_BUFFERS; s++) { mbar_init(&bfull[s], C::DEQUANT_WARPS / 2); mbar_init(&bempty[s], 1); }
        for (int s = 0; s < C::ACC_BUFFERS; s++) { mbar_init(&tfull[s], 1); mbar_init(&tempty[s], C::EPILOGUE_WARPS); }
        control_block_init(tmem_slot, p.wait_limit);
        fence_barrier_init();
        fence_proxy_async_smem();
    }
    if (warp == C::PRODUCER_WARP && lane == 0) { tma_prefetch_descriptor(&map_a); tma_prefetch_descriptor(&map_b); }
    if (warp == C::MMA_WARP) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    uint32_t failure = STATUS_OK;
    /* split-K: let the finishing grid be scheduled as SMs drain (it waits for this grid's completion before reading) */
    if (SPLITK) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == C::PRODUCER_WARP) {
        /* ------------------------------------------------ TMA producer */
        if (lane == 0) {
            PipeState st;
            for (uint32_t item = blockIdx.x; item < items && !failure; item += gridDim.x) {
                H3Q8_ITEM(item, tile, kb_first, kb_last)
                uint32_t mb, nb;
                tile_coordinates(p, tile, mb, nb);
                for (uint32_t kb = kb_first; kb < kb_last; kb++) {
                    if (!wait_or_abort(&empty[st.index], st.phase ^ 1, abort_flag)) { failure = STATUS_WAIT_PRODUCER; break; }
                    uint8_t *stage = stages + st.index * C::STAGE_BYTES;
                    if (p.skip_first_load && item == blockIdx.x && kb == kb_first) { st.advance(C::STAGES); continue; }   /* injected fault */
                    mbar_arrive_expect_tx(&full[st.index], C::STAGE_BYTES);
#pragma unroll
                    for (int mt = 0; mt < MT; mt++)
                        tma_load_2d(stage + mt * 128 * C::ROW_BYTES, &map_a, &full[st.index],
                                    (int32_t)(kb * C::BKE), (int32_t)(mb * C::BM + mt * 128));
                    tma_load_2d(stage + C::A_BYTES, &map_b, &full[st.index], (int32_t)(kb * C::BKE), (int32_t)(nb * BN));
                    st.advance(C::STAGES);
                }
            }
        }
    } else if (warp == C::MMA_WARP) {
        /* -------------------------------------------------- MMA issuer */
        if (lane == 0) {
            PipeState st, cv, acc;
            for (uint32_t item = blockIdx.x; item < items && !failure; item += gridDim.x) {
                H3Q8_ITEM(item, tile, kb_first, kb_last)
                (void)tile;
                uint32_t kb = kb_first;
                for (uint32_t chunk = 0; chunk < chunks && !failure; chunk++) {
                    if (!wait_or_abort(&tempty[acc.index], acc.phase ^ 1, abort_flag)) { failure = STATUS_WAIT_MMA; break; }
                    tc_fence_after_sync();
                    uint32_t last = kb + kb_per_chunk < kb_last ? kb + kb_per_chunk : kb_last;
                    uint32_t accumulate = 0;
                    for (; kb < last; kb++) {
                        if (!wait_or_abort(&full[st.index], st.phase, abort_flag)) { failure = STATUS_WAIT_MMA; break; }
                        uint8_t *stage = stages + st.index * C::STAGE_BYTES;
                        uint8_t *b_tile = stage + C::A_BYTES;
                        if (MODE == MODE_W8A16) {
                            if (!wait_or_abort(&bfull[cv.index], cv.phase, abort_flag)) { failure = STATUS_WAIT_MMA; break; }
                            b_tile = conv + cv.index * C::B_BYTES;
                        }
                        tc_fence_after_sync();
                        const uint64_t b_desc = umma_smem_desc_sw128(smem_u32(b_tile));
#pragma unroll
                        for (int mt = 0; mt < MT; mt++) {
                            const uint64_t a_desc = umma_smem_desc_sw128(smem_u32(stage + mt * 128 * C::ROW_BYTES));
                            const uint32_t d = tmem_base + acc.index * C::ACC_COLS + mt * BN;
#pragma unroll
                            for (int k4 = 0; k4 < 4; k4++) {
                                /* 32 bytes along K per instruction: +2 in 16-byte units */
                                if (MODE == MODE_W8A8) umma_i8(d, a_desc + 2 * k4, b_desc + 2 * k4, C::IDESC, accumulate | k4);
                                else umma_bf16(d, a_desc + 2 * k4, b_desc + 2 * k4, C::IDESC, accumulate | k4);
                            }
                        }
                        accumulate = 1;
                        umma_commit(&empty[st.index]);
                        st.advance(C::STAGES);
                        if (MODE == MODE_W8A16) { umma_commit(&bempty[cv.index]); cv.advance(C::CONV_BUFFERS); }
                    }
                    if (failure) break;
                    umma_commit(&tfull[acc.index]);
                    acc.advance(C::ACC_BUFFERS);
                }
            }
        }
    } else if (warp < C::EPILOGUE_WARPS) {
        /* ---------------------------------------------------- epilogue */
        /* warp w reads TMEM lanes 32*(w%4).. (its hardware quadrant) and the column half w/4 */
        constexpr int HALF_CHUNKS = BN / 64;
        const uint32_t quadrant = warp & 3, half = warp >> 2;
        PipeState acc;
        const bool gated = p.ep.gate != nullptr || p.ep.residual != nullptr;
        for (uint32_t item = blockIdx.x; item < items && !failure; item += gridDim.x) {
            H3Q8_ITEM(item, tile, kb_first, kb_last)
            (void)kb_last;
            uint32_t mb, nb;
            tile_coordinates(p, tile, mb, nb);
            const uint32_t n0 = nb * BN;
            float totals[GROUPED ? BN / 2 : 1];
            for (uint32_t chunk = 0; chunk < chunks && !failure; chunk++) {
                bool ready = wait_or_abort(&tfull[acc.index], acc.phase, abort_flag);
                if (!__all_sync(0xffffffffu, ready)) { failure = STATUS_WAIT_EPILOGUE; break; }
                tc_fence_after_sync();
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    const uint32_t row = mb * C::BM + mt * 128 + quadrant * 32 + lane;
                    const bool row_ok = row < p.M;
                    float a_scale = 1.0f;
                    if (MODE == MODE_W8A8)
                        a_scale = !row_ok ? 0.0f : !GROUPED || p.a_scale_groups == 1 ? p.a_scales[(size_t)row * p.a_scale_groups]
                                                 : p.a_scales[(size_t)row * p.a_scale_groups + chunk];
#pragma unroll(GROUPED ? HALF_CHUNKS : 1)
                    for (int hc = 0; hc < HALF_CHUNKS; hc++) {
                        const int c = half * HALF_CHUNKS + hc;
                        uint32_t v[32];
                        tmem_load_32x32(tmem_base + ((quadrant * 32u) << 16) + acc.index * C::ACC_COLS + mt * BN + c * 32, v);
                        tmem_load_wait();
                        const uint32_t col0 = n0 + c * 32;
                        if (GROUPED) {
#pragma unroll
                            for (int j = 0; j < 32; j++) {
                                uint32_t col = col0 + j;
                                float ws = col < p.N ? p.w_scales[(size_t)col * p.scale_groups + (p.scale_groups == 1 ? 0 : chunk)] : 0.0f;
                                float value = __fmul_rn(__fmul_rn((float)(int32_t)v[j], a_scale), ws);
                                totals[hc * 32 + j] = chunk ? __fadd_rn(totals[hc * 32 + j], value) : value;
                            }
                            if (chunk + 1 < chunks) continue;
                        }
                        if (!row_ok) continue;
                        if (SPLITK) {   /* raw 32-bit sums of this K range; the finishing kernel owns the epilogue */
                            uint32_t *dst = p.partials + ((size_t)(kb_first / p.kb_per_split) * p.M + row) * p.N + col0;
#pragma unroll
                            for (int j4 = 0; j4 < 8; j4++)
                                if (col0 + j4 * 4 < p.N)
                                    reinterpret_cast<uint4 *>(dst)[j4] = make_uint4(v[j4 * 4], v[j4 * 4 + 1], v[j4 * 4 + 2], v[j4 * 4 + 3]);
                            continue;
                        }
                        if (!GROUPED && p.acc_dump) {   /* raw accumulators: int32 sums (W8A8) or fp32 partial sums */
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
                            if (col >= p.N) continue; /* N is a multiple of 8 on this path */
                            float lin[8];
                            if (MODE == MODE_W8A8 && !GROUPED) {
                                float4 s0 = *reinterpret_cast<const float4 *>(p.w_scales + col);
                                float4 s1 = *reinterpret_cast<const float4 *>(p.w_scales + col + 4);
                                const float ws[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
                                for (int j = 0; j < 8; j++)
                                    lin[j] = __fmul_rn(__fmul_rn((float)(int32_t)v[j8 * 8 + j], a_scale), ws[j]);
                            } else if (GROUPED) {
#pragma unroll
                                for (int j = 0; j < 8; j++) lin[j] = totals[hc * 32 + j8 * 8 + j];
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
                }
                /* accumulator drained: hand the TMEM buffer back to the MMA issuer */
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&tempty[acc.index]);
                acc.advance(C::ACC_BUFFERS);
            }
        }
    } else if (MODE == MODE_W8A16) {
        /* ------------------------------------------------- dequantisers */
        /* Two groups of four warps take alternate k-blocks: a group turns a whole BN x 64 int8 tile (64-byte rows,
         * 64-byte swizzle) into a BN x 64 bf16 tile (128-byte rows, 128-byte swizzle), one 64-byte row per thread and
         * pass.  Each warp then pays the wait -> convert -> fence.proxy.async -> arrive latency once per TWO k-blocks,
         * and the groups overlap each other (that chain, not the arithmetic, set the pace with all eight warps on
         * every k-block). */
        constexpr int ROWS = BN / 128;                      /* rows per thread */
        const uint32_t group = (warp - C::FIRST_DEQUANT_WARP) >> 2;
        const uint32_t d = threadIdx.x - (C::FIRST_DEQUANT_WARP + 4 * group) * 32;   /* 0..127 inside the group */
        const uint32_t width = p.scale_group ? p.scale_group : p.K;
        PipeState st, cv;
        uint32_t turn = 0;                                  /* k-blocks seen so far, across tiles */
        for (uint32_t item = blockIdx.x; item < items && !failure; item += gridDim.x) {
            H3Q8_ITEM(item, tile, kb_first, kb_last)
            uint32_t mb, nb;
            tile_coordinates(p, tile, mb, nb);
            const float *row_scales[ROWS];
            bool live[ROWS];
            float upcoming[ROWS];
            /* this group's first k-block of the tile; its scales are fetched before they are needed */
            const uint32_t mine_first = kb_first + ((turn & 1u) == group ? 0u : 1u);
#pragma unroll
            for (int rr = 0; rr < ROWS; rr++) {
                const uint32_t n = nb * BN + d + rr * 128;
                live[rr] = n < p.N;
                row_scales[rr] = p.w_scales + (size_t)(live[rr] ? n : 0) * p.scale_groups;
                upcoming[rr] = live[rr] && mine_first < kb_last ? row_scales[rr][(mine_first * C::BKE) / width] : 0.0f;
            }
            for (uint32_t kb = kb_first; kb < kb_last; kb++, turn++) {
                if ((turn & 1u) != group) { st.advance(C::STAGES); cv.advance(C::CONV_BUFFERS); continue; }
                float scale[ROWS];
#pragma unroll
                for (int rr = 0; rr < ROWS; rr++) {
                    scale[rr] = upcoming[rr];
                    if (p.scale_groups > 1 && kb + 2 < kb_last && live[rr]) upcoming[rr] = row_scales[rr][((kb + 2) * C::BKE) / width];
                }
                bool ready = wait_or_abort(&full[st.index], st.phase, abort_flag) &&
                             wait_or_abort(&bempty[cv.index], cv.phase ^ 1, abort_flag);
                if (!__all_sync(0xffffffffu, ready)) { failure = STATUS_WAIT_DEQUANT; break; }
                const uint8_t *raw = stages + st.index * C::STAGE_BYTES + C::A_BYTES;
                uint8_t *dst = conv + cv.index * C::B_BYTES;
#pragma unroll
                for (int rr = 0; rr < ROWS; rr++) {
                    const uint32_t r = d + rr * 128;
#pragma unroll
                    for (int chunk = 0; chunk < 4; chunk++) {
                        const uint4 q = *reinterpret_cast<const uint4 *>(raw + r * 64 + ((chunk ^ ((r >> 1) & 3)) << 4));
                        const uint32_t words[4] = {q.x, q.y, q.z, q.w};
                        uint32_t o[8];
#pragma unroll
                        for (int w = 0; w < 4; w++) {
                            float f[4];
                            dequant4(words[w], scale[rr], f);
                            o[2 * w] = pack_bf16x2(f[0], f[1]);
                            o[2 * w + 1] = pack_bf16x2(f[2], f[3]);
                        }
                        uint8_t *row_dst = dst + r * 128;
                        *reinterpret_cast<uint4 *>(row_dst + (((2 * chunk) ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                        *reinterpret_cast<uint4 *>(row_dst + (((2 * chunk + 1) ^ (r & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
                    }
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bfull[cv.index]);
                st.advance(C::STAGES);
                cv.advance(C::CONV_BUFFERS);
            }
        }
    }

    /* ---------------------------------------------------------- teardown */
    if (failure) {
        *abort_flag = 1;
        atomicCAS(p.status, 0u, failure | (blockIdx.x << 8));
    }
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        /* Give any TMA copy still in flight time to land before the CTA's shared
         * memory is released. */
        long long start = clock64();
        while (clock64() - start < 2000000ll) { }
        __syncthreads();
    }
    if (warp == C::MMA_WARP) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 512);
    }
}

#undef H3Q8_ITEM

/* Second half of a split-K linear: sums the `splits` partial accumulators of every output in ascending split order
 * (int32: exact; fp32: one fixed order, so results do not depend on scheduling) and applies the usual epilogue.
 * One thread per 8 consecutive outputs of a row. */
template <int MODE>
__global__ void __launch_bounds__(256) splitk_finish_kernel(const GemmParams p) {
    const uint32_t per_row = p.N / 8;
    const uint64_t index = (uint64_t)blockIdx.x * 256 + threadIdx.x;
    /* launched with programmatic stream serialisation: this grid may be resident before the split GEMM has finished;
     * nothing it wrote is read before this point */
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (index >= (uint64_t)p.M * per_row) return;
    const uint32_t row = (uint32_t)(index / per_row), col = (uint32_t)(index % per_row) * 8;
    const bool gated = p.ep.gate != nullptr || p.ep.residual != nullptr;
    const uint32_t *src = p.partials + (size_t)row * p.N + col;
    const size_t stride = (size_t)p.M * p.N;
    float lin[8];
    if (MODE == MODE_W8A8) {
        int32_t sum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (uint32_t s = 0; s < p.splits; s++) {
            const uint4 a = reinterpret_cast<const uint4 *>(src + s * stride)[0], b = reinterpret_cast<const uint4 *>(src + s * stride)[1];
            const uint32_t v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
            for (int j = 0; j < 8; j++) sum[j] += (int32_t)v[j];
        }
        const float a_scale = p.a_scales[row];
        const float4 s0 = *reinterpret_cast<const float4 *>(p.w_scales + col), s1 = *reinterpret_cast<const float4 *>(p.w_scales + col + 4);
        const float ws[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
        for (int j = 0; j < 8; j++) lin[j] = __fmul_rn(__fmul_rn((float)sum[j], a_scale), ws[j]);
    } else {
#pragma unroll
        for (int j = 0; j < 8; j++) lin[j] = 0.0f;
        for (uint32_t s = 0; s < p.splits; s++) {
            const uint4 a = reinterpret_cast<const uint4 *>(src + s * stride)[0], b = reinterpret_cast<const uint4 *>(src + s * stride)[1];
            const uint32_t v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
            for (int j = 0; j < 8; j++) lin[j] = s ? __fadd_rn(lin[j], __uint_as_float(v[j])) : __uint_as_float(v[j]);
        }
    }
    uint32_t bias[4] = {0, 0, 0, 0}, gate[4] = {0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u}, res[4] = {0, 0, 0, 0};
    if (p.ep.bias) *reinterpret_cast<uint4 *>(bias) = *reinterpret_cast<const uint4 *>(p.ep.bias + col);
    if (p.ep.gate) *reinterpret_cast<uint4 *>(gate) = *reinterpret_cast<const uint4 *>(p.ep.gate + col);
    if (p.ep.residual) *reinterpret_cast<uint4 *>(res) = *reinterpret_cast<const uint4 *>(p.ep.residual + (size_t)row * p.N + col);
    uint32_t packed[4];
#pragma unroll
    for (int j = 0; j < 4; j++)
        packed[j] = epilogue_pair(lin[2 * j], lin[2 * j + 1], bias[j], p.ep.bias != nullptr, p.ep.activation, gated, gate[j], res[j]);
    *reinterpret_cast<uint4 *>(p.out + (size_t)row * p.N + col) = *reinterpret_cast<uint4 *>(packed);
}

} /* namespace h3q8 */
