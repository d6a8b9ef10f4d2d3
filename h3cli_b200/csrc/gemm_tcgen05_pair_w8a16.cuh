/* W8A16 with dequantisation in the main loop on the two-CTA tile.
 *
 *   out[M,N] = epilogue( X[M,K] (bf16) . bf16(float(Wq[N,K]) * scale[n, k/group])^T )
 *
 * A cluster of two CTAs computes a 256 x 256 output tile with `tcgen05.mma.cta_group::2`
 * exactly as gemm_tcgen05_pair_kernel does, but the weight arrives as int8: each CTA's TMA
 * brings its own 128 weight rows as 128 raw bytes per row (two k-blocks of 64), dequantiser warps
 * (two groups of four on alternate 128-wide blocks) turn them into two bf16 operand tiles (128-byte rows, 128-byte
 * swizzle) with the reference's arithmetic, bf16(float(q) * scale) (src/metal/shaders.metal:825-827), and the
 * leader's MMA issuer consumes the converted tiles of BOTH CTAs.  The hand-off covers 128 elements of K because
 * its fixed cost -- two waits, a proxy fence and an arrival per warp -- is a quarter of the conversion time of a
 * 64-wide block, and the dequantisers are what the tensor core waits for.
 *
 * Why two CTAs: a CTA converts only its own 128 of the tile's 256 weight rows, i.e. half
 * of the conversions per SM and MMA clock of a one-CTA 128 x 256 tile, and its tensor core
 * reads half of the B operand from its own shared memory.
 *
 * Per CTA and k-block (64 elements of K, 512 MMA clocks at full rate):
 *   TMA writes    A 16 KB (bf16, 128-byte swizzle) + raw W 8 KB (int8, 128-byte swizzle, 16 KB per two k-blocks)
 *   dequantisers  read 8 KB, write 16 KB (converted ring)
 *   tensor core   reads A 16 KB + converted W 16 KB
 *
 * Barriers (count; who arrives):
 *   afull[s]   leader only; 1 + tx bytes of both CTAs' A tiles      (producers of both CTAs)
 *   aempty[s]  per CTA;     1   tcgen05.commit of the leader, sent to both CTAs
 *   rfull[s]   per CTA;     1 + tx bytes of the CTA's own raw tile   (its own producer)          per two k-blocks
 *   rempty[s]  per CTA;     4   the warps of the group that converts the tile, once it is in registers
 *   bfull[c]   leader only; 8   one arrival per warp of that group in both CTAs                 per two k-blocks
 *   bempty[c]  per CTA;     1   tcgen05.commit of the leader, sent to both CTAs                per two k-blocks
 *   tfull[a] / tempty[a]    as in the bf16 pair kernel
 * Every wait is bounded; a role that gives up raises the CTA's abort flag and all roles
 * fall through to the common exit, where the status word is set and TMEM is freed.
 */
#pragma once
#include "gemm_tcgen05_pair.cuh"

/* dequantiser groups; three measured slightly slower than two (the bound is shared-memory bandwidth, not the conversion) */
#ifndef H3Q8_W8A16_GROUPS
#define H3Q8_W8A16_GROUPS 2
#endif

namespace h3q8 {

struct PairW8A16Config {
    static constexpr int BM = 256, BN = 256, BKE = 64;
    static constexpr int A_BYTES = 128 * 128;            /* this CTA's 128 rows of X, 64 bf16 each       */
    static constexpr int KSUB = 2;                       /* k-blocks per weight hand-off                 */
    static constexpr int RAW_BYTES = 128 * 64 * KSUB;    /* this CTA's 128 weight rows, 128 int8 each    */
    static constexpr int B_BYTES = 128 * 128;            /* converted tile of one k-block                */
    /* three rings: a raw tile is free again as soon as it has been converted, the X tile and the converted tile only
     * when the MMAs that read them are done; raw tiles are small, so that ring is the deep one */
    static constexpr int A_STAGES = 5, RAW_STAGES = 3, CONV_BUFFERS = 3;   /* raw and converted: units of KSUB k-blocks */
    static constexpr int ACC_COLS = BN, ACC_BUFFERS = 2;
    /* warps: epilogue (TMEM lane quadrant = warp % 4, column half = warp / 4), weight producer, activation producer,
     * MMA issuer and TMEM owner, dequantisers in two groups */
    /* eight dequantiser warps keep ahead of the tensor core; sixteen only add shared-memory and issue contention, and the
     * ring depths matter little once each covers the TMA latency: the kernel is bound by shared-memory bandwidth */
    static constexpr int EPILOGUE_WARPS = 8, RAW_PRODUCER_WARP = EPILOGUE_WARPS, A_PRODUCER_WARP = EPILOGUE_WARPS + 1,
                         MMA_WARP = EPILOGUE_WARPS + 2, FIRST_DEQUANT_WARP = EPILOGUE_WARPS + 3;
    static constexpr int GROUPS = H3Q8_W8A16_GROUPS, GROUP_WARPS = 4, DEQUANT_WARPS = GROUPS * GROUP_WARPS;
    static_assert((EPILOGUE_WARPS == 4 || EPILOGUE_WARPS == 8) && (GROUP_WARPS == 4 || GROUP_WARPS == 8), "role layout");
    static constexpr int WARPS = FIRST_DEQUANT_WARP + DEQUANT_WARPS, THREADS = WARPS * 32;
    static constexpr int BARRIERS = 2 * A_STAGES + 2 * RAW_STAGES + 2 * CONV_BUFFERS + 2 * ACC_BUFFERS;
    static constexpr int SMEM_BYTES = A_STAGES * A_BYTES + RAW_STAGES * RAW_BYTES + CONV_BUFFERS * KSUB * B_BYTES + 1024 + 512;
    static constexpr uint32_t IDESC = umma_idesc(1, 1, 256, BN);
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
    static_assert(BARRIERS * 8 + 16 <= 512, "barrier block");
};

/* sixteen int8 (one 16-byte vector) -> sixteen bf16 = bf16(float(q) * scale), as two 16-byte vectors.
 * (q ^ 0x80) in the low mantissa byte of 2^23 is 2^23 + 128 + q exactly; subtracting 2^23 + 128 and multiplying by the
 * scale are IEEE fp32 operations, then one round-to-nearest-even conversion per pair.  PACKED uses the two-lane fp32
 * instructions of sm_100 for the subtraction and the multiplication. */
template <bool PACKED>
__device__ __forceinline__ void dequant16(const uint4 q, const float scale, uint4 &lo, uint4 &hi) {
    const uint32_t words[4] = {q.x, q.y, q.z, q.w};
    uint32_t o[8];
    if (PACKED) {
        const uint64_t scale2 = f32x2(scale, scale), magic2 = f32x2(-8388736.0f, -8388736.0f);
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const uint32_t biased = words[w] ^ 0x80808080u;
            const uint64_t p01 = f32x2(__uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7650)), __uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7651)));
            const uint64_t p23 = f32x2(__uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7652)), __uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7653)));
            float f0, f1, f2, f3;
            f32x2_unpack(mul_f32x2(add_f32x2(p01, magic2), scale2), f0, f1);
            f32x2_unpack(mul_f32x2(add_f32x2(p23, magic2), scale2), f2, f3);
            o[2 * w] = pack_bf16_pair(f0, f1);
            o[2 * w + 1] = pack_bf16_pair(f2, f3);
        }
    } else {
#pragma unroll
        for (int w = 0; w < 4; w++) {
            float f[4];
            dequant4(words[w], scale, f);
            o[2 * w] = pack_bf16_pair(f[0], f[1]);
            o[2 * w + 1] = pack_bf16_pair(f[2], f[3]);
        }
    }
    lo = make_uint4(o[0], o[1], o[2], o[3]);
    hi = make_uint4(o[4], o[5], o[6], o[7]);
}

template <bool PACKED>
static __global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PairW8A16Config::THREADS, 1)
gemm_tcgen05_pair_w8a16_kernel(const __grid_constant__ PairArgs args) {
    using C = PairW8A16Config;
    const GemmParams &p = args.p[0];
    const CUtensorMap &map_a = args.map_a[0], &map_b = args.map_b[0];
    const uint32_t total_tiles = p.tiles;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *a_ring = smem;
    uint8_t *conv = a_ring + C::A_STAGES * C::A_BYTES;
    uint8_t *raw_ring = conv + C::CONV_BUFFERS * C::KSUB * C::B_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(raw_ring + C::RAW_STAGES * C::RAW_BYTES);
    uint64_t *afull = bars, *aempty = afull + C::A_STAGES;
    uint64_t *rfull = aempty + C::A_STAGES, *rempty = rfull + C::RAW_STAGES;
    uint64_t *bfull = rempty + C::RAW_STAGES, *bempty = bfull + C::CONV_BUFFERS;
    uint64_t *tfull = bempty + C::CONV_BUFFERS, *tempty = tfull + C::ACC_BUFFERS;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tempty + C::ACC_BUFFERS);
    volatile uint32_t *abort_flag = tmem_slot + 1;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();               /* 0 = leader */
    const uint32_t pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const uint32_t num_kb = (p.K + C::BKE - 1) / C::BKE;
    const uint32_t num_wb = (num_kb + C::KSUB - 1) / C::KSUB;   /* weight hand-offs per tile */
    const bool swiglu = p.ep.activation == ACT_SWIGLU;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::A_STAGES; s++) { mbar_init(&afull[s], 1); mbar_init(&aempty[s], 1); }
        for (int s = 0; s < C::RAW_STAGES; s++) { mbar_init(&rfull[s], 1); mbar_init(&rempty[s], C::GROUP_WARPS); }
        for (int s = 0; s < C::CONV_BUFFERS; s++) { mbar_init(&bfull[s], 2 * C::GROUP_WARPS); mbar_init(&bempty[s], 1); }
        for (int s = 0; s < C::ACC_BUFFERS; s++) { mbar_init(&tfull[s], 1); mbar_init(&tempty[s], 2 * C::EPILOGUE_WARPS); }
        control_block_init(tmem_slot, p.wait_limit);
        fence_barrier_init();
        fence_proxy_async_smem();
    }
    if (warp == C::RAW_PRODUCER_WARP && lane == 0) tma_prefetch_descriptor(&map_b);
    if (warp == C::A_PRODUCER_WARP && lane == 0) tma_prefetch_descriptor(&map_a);
    if (warp == C::MMA_WARP) { tmem_alloc_pair(tmem_slot, 512); tmem_relinquish_pair(); }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync();           /* both CTAs' barriers exist before anything crosses the pair */
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    uint32_t failure = STATUS_OK;

    if (warp == C::RAW_PRODUCER_WARP) {
        /* ------------------------------------------------ weight producer (both CTAs): raw int8 tiles */
        if (lane == 0) {
            PipeState sr;
            for (uint32_t tile = pair; tile < total_tiles && !failure; tile += pairs) {
                uint32_t mb, nb;
                tile_coordinates(p, tile, mb, nb);
                /* SwiGLU: the leader stages 128 gate rows, its peer the matching 128 up rows (weight rows N + n) */
                const uint32_t b_row = swiglu ? nb * 128 + rank * p.N : nb * C::BN + rank * 128;
                for (uint32_t wb = 0; wb < num_wb; wb++) {
                    if (!wait_or_abort(&rempty[sr.index], sr.phase ^ 1, abort_flag)) { failure = STATUS_WAIT_PRODUCER; break; }
                    mbar_arrive_expect_tx(&rfull[sr.index], C::RAW_BYTES);
                    tma_load_2d(raw_ring + sr.index * C::RAW_BYTES, &map_b, &rfull[sr.index], (int32_t)(wb * C::KSUB * C::BKE), (int32_t)b_row);
                    sr.advance(C::RAW_STAGES);
                }
            }
        }
    } else if (warp == C::A_PRODUCER_WARP) {
        /* ------------------------------------------------ activation producer (both CTAs): bf16 tiles of X */
        if (lane == 0) {
            PipeState sa;
            for (uint32_t tile = pair; tile < total_tiles && !failure; tile += pairs) {
                uint32_t mb, nb;
                tile_coordinates(p, tile, mb, nb);
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    if (!wait_or_abort(&aempty[sa.index], sa.phase ^ 1, abort_flag)) { failure = STATUS_WAIT_PRODUCER; break; }
                    /* the leader arms its barrier for the bytes of both CTAs */
                    if (rank == 0) mbar_arrive_expect_tx(&afull[sa.index], 2 * C::A_BYTES);
                    tma_load_2d_pair(a_ring + sa.index * C::A_BYTES, &map_a, map_to_cta(smem_u32(&afull[sa.index]), 0), (int32_t)(kb * C::BKE),
                                     (int32_t)(mb * C::BM + rank * 128), p.l2_policy_a);
                    sa.advance(C::A_STAGES);
                }
            }
        }
    } else if (warp == C::MMA_WARP) {
        /* ------------------------------------------------ MMA issuer (leader only) */
        if (lane == 0 && rank == 0) {
            PipeState st, cv, acc;
            for (uint32_t tile = pair; tile < total_tiles && !failure; tile += pairs) {
                if (!wait_or_abort(&tempty[acc.index], acc.phase ^ 1, abort_flag)) { failure = STATUS_WAIT_MMA; break; }
                tc_fence_after_sync();
                const uint32_t d = tmem_base + acc.index * C::ACC_COLS;
                for (uint32_t wb = 0; wb < num_wb && !failure; wb++) {
                    if (!wait_or_abort(&bfull[cv.index], cv.phase, abort_flag)) { failure = STATUS_WAIT_MMA; break; }
#pragma unroll
                    for (int sub = 0; sub < C::KSUB; sub++) {
                        const uint32_t kb = wb * C::KSUB + sub;
                        if (kb >= num_kb) break;
                        if (!wait_or_abort(&afull[st.index], st.phase, abort_flag)) { failure = STATUS_WAIT_MMA; break; }
                        tc_fence_after_sync();
                        const uint64_t a_desc = umma_smem_desc_sw128(smem_u32(a_ring + st.index * C::A_BYTES));
                        const uint64_t b_desc = umma_smem_desc_sw128(smem_u32(conv + (cv.index * C::KSUB + sub) * C::B_BYTES));
#pragma unroll
                        for (int k4 = 0; k4 < 4; k4++) umma_bf16_pair(d, a_desc + 2 * k4, b_desc + 2 * k4, C::IDESC, kb | k4);
                        umma_commit_pair(&aempty[st.index], 3);   /* frees the X tile in both CTAs */
                        st.advance(C::A_STAGES);
                    }
                    if (failure) break;
                    umma_commit_pair(&bempty[cv.index], 3);       /* frees the converted tiles in both CTAs */
                    cv.advance(C::CONV_BUFFERS);
                }
                if (failure) break;
                umma_commit_pair(&tfull[acc.index], 3);
                acc.advance(C::ACC_BUFFERS);
            }
        }
    } else if (warp >= C::FIRST_DEQUANT_WARP) {
        /* ------------------------------------------------ dequantisers (both CTAs) */
        /* Two groups of four warps take alternate weight blocks of 128 k-values.  Thread t owns weight row t of this
         * CTA's 128: eight 16-byte loads from the raw tile (128-byte rows, 128-byte swizzle), 16 conversions per load,
         * 16-byte stores into the two operand tiles (128-byte rows, 128-byte swizzle); consecutive lanes take
         * consecutive rows, which keeps both swizzles free of bank conflicts.  A warp pays two waits, one proxy fence
         * and one arrival per block, and while one group sits in its fence the other converts. */
        static_assert(C::GROUP_WARPS == 4 && C::KSUB == 2, "one thread per weight row, two k-blocks per hand-off");
        const uint32_t group = (warp - C::FIRST_DEQUANT_WARP) / C::GROUP_WARPS;
        const uint32_t r = threadIdx.x - (C::FIRST_DEQUANT_WARP + C::GROUP_WARPS * group) * 32;
        const uint32_t twist = r & 7;
        const uint32_t width = p.scale_group ? p.scale_group : p.K;
        const uint32_t leader_bfull = map_to_cta(smem_u32(bfull), 0);
        auto scale_pointer = [&](uint32_t tile, bool &live) {
            uint32_t mb, nb;
            tile_coordinates(p, tile, mb, nb);
            const uint32_t n = swiglu ? nb * 128 + r : nb * C::BN + rank * 128 + r;       /* output channel (bounds)  */
            live = n < p.N;
            const size_t scale_row = swiglu ? (size_t)rank * p.N + n : n;                  /* row of the weight matrix */
            return p.w_scales + (live ? scale_row : 0) * p.scale_groups;
        };
        /* the scales of the two k-blocks of weight block wb (the same one unless the scale group is 64) */
        auto scales_of = [&](const float *row, bool row_live, uint32_t wb, float &s0, float &s1) {
            const uint32_t k0 = wb * C::KSUB * C::BKE, k1 = k0 + C::BKE;
            s0 = row_live ? row[k0 / width] : 0.0f;
            s1 = row_live && k1 < p.K ? row[k1 / width] : s0;
        };
        PipeState st, cv;
        uint32_t turn = 0;                                  /* weight blocks seen so far, across tiles */
        bool live = false;
        const float *row_scales = pair < total_tiles ? scale_pointer(pair, live) : p.w_scales;
        float first0 = 0.0f, first1 = 0.0f;                 /* block 0 of the coming tile, fetched one tile ahead */
        if (pair < total_tiles) scales_of(row_scales, live, 0, first0, first1);
        for (uint32_t tile = pair; tile < total_tiles && !failure; tile += pairs) {
            const float *scales_now = row_scales;
            const bool live_now = live;
            float upcoming0 = first0, upcoming1 = first1;
            const uint32_t mine_first = (group + C::GROUPS - turn % C::GROUPS) % C::GROUPS;   /* this group's first block of the tile */
            if (p.scale_groups > 1 && mine_first && mine_first < num_wb) scales_of(scales_now, live_now, mine_first, upcoming0, upcoming1);
            if (tile + pairs < total_tiles) {
                row_scales = scale_pointer(tile + pairs, live);
                scales_of(row_scales, live, 0, first0, first1);
            }
            for (uint32_t wb = 0; wb < num_wb; wb++, turn++) {
                if (turn % C::GROUPS != group) { st.advance(C::RAW_STAGES); cv.advance(C::CONV_BUFFERS); continue; }
                const float scale[2] = {upcoming0, upcoming1};
                if (p.scale_groups > 1 && wb + C::GROUPS < num_wb) scales_of(scales_now, live_now, wb + C::GROUPS, upcoming0, upcoming1);
                bool ready = wait_or_abort(&rfull[st.index], st.phase, abort_flag);
                ready = ready && wait_or_abort(&bempty[cv.index], cv.phase ^ 1, abort_flag);
                if (!__all_sync(0xffffffffu, ready)) { failure = STATUS_WAIT_DEQUANT; break; }
                const uint8_t *raw = raw_ring + st.index * C::RAW_BYTES + r * 128;
                uint8_t *dst = conv + cv.index * C::KSUB * C::B_BYTES + r * 128;
                uint4 q[8];
#pragma unroll
                for (int c = 0; c < 8; c++) q[c] = *reinterpret_cast<const uint4 *>(raw + ((c ^ twist) << 4));
                /* the raw tile is in registers: its slot may be refilled */
                __syncwarp();
                if (lane == 0) mbar_arrive(&rempty[st.index]);
#pragma unroll
                for (int c = 0; c < 8; c++) {
                    uint4 lo, hi;
                    dequant16<PACKED>(q[c], scale[c >> 2], lo, hi);
                    uint8_t *tile_row = dst + (c >> 2) * C::B_BYTES;
                    *reinterpret_cast<uint4 *>(tile_row + (((2 * (c & 3)) ^ twist) << 4)) = lo;
                    *reinterpret_cast<uint4 *>(tile_row + (((2 * (c & 3) + 1) ^ twist) << 4)) = hi;
                }
                /* The converted tiles are read by the tensor core of THIS SM (each CTA supplies its own half of B), so all
                 * that has to cross the pair is the news that the writes are done: every writer makes its stores visible
                 * to the async proxy, then one lane per warp arrives on the leader's barrier with the plain remote arrive.
                 * (A cluster-scope release on this arrival is a memory barrier of about 900 clocks per warp and hand-off,
                 * which alone holds the kernel to a third of the MMA rate.) */
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    if (rank == 0) mbar_arrive(&bfull[cv.index]);
                    else mbar_arrive_remote(leader_bfull + cv.index * 8);
                }
                st.advance(C::RAW_STAGES);
                cv.advance(C::CONV_BUFFERS);
            }
        }
    } else {
        /* ------------------------------------------------ epilogue (both CTAs, own 128 rows) */
        /* warp w owns TMEM lane quadrant w (rows 32 w .. 32 w + 31 of this CTA's 128) and walks all 256 columns; the
         * reference's operator chain in registers (epilogue.cuh) */
        constexpr int SPLIT = C::EPILOGUE_WARPS / 4;   /* column halves */
        const uint32_t quadrant = warp & 3, half = warp >> 2;
        const bool gated = p.ep.gate != nullptr || p.ep.residual != nullptr;
        PipeState acc;
        for (uint32_t tile = pair; tile < total_tiles && !failure; tile += pairs) {
            uint32_t mb, nb;
            tile_coordinates(p, tile, mb, nb);
            const uint32_t n0 = swiglu ? nb * 128 : nb * C::BN;
            bool ready = wait_or_abort(&tfull[acc.index], acc.phase, abort_flag);
            if (!__all_sync(0xffffffffu, ready)) { failure = STATUS_WAIT_EPILOGUE; break; }
            tc_fence_after_sync();
            const uint32_t row = mb * C::BM + rank * 128 + quadrant * 32 + lane;
            const bool row_ok = row < p.M;
            const uint32_t lane_base = tmem_base + ((quadrant * 32u) << 16) + acc.index * C::ACC_COLS;
            if (swiglu) {
                /* accumulator columns 0..127 hold the gate, 128..255 the up projection of the same 128 outputs */
#pragma unroll 1
                for (int hc = 0; hc < 8 / SPLIT; hc++) {
                    const int c = half * (8 / SPLIT) + hc;
                    uint32_t vg[16], vu[16];
                    tmem_load_32x16(lane_base + c * 16, vg);
                    tmem_load_32x16(lane_base + 128 + c * 16, vu);
                    tmem_load_wait();
                    if (!row_ok) continue;
#pragma unroll
                    for (int j8 = 0; j8 < 2; j8++) {
                        const uint32_t col = n0 + c * 16 + j8 * 8;
                        if (col >= p.N) continue;
                        uint32_t bg[4] = {0, 0, 0, 0}, bu[4] = {0, 0, 0, 0};
                        if (p.ep.bias) {
                            *reinterpret_cast<uint4 *>(bg) = *reinterpret_cast<const uint4 *>(p.ep.bias + col);
                            *reinterpret_cast<uint4 *>(bu) = *reinterpret_cast<const uint4 *>(p.ep.bias + p.N + col);
                        }
                        uint32_t packed[4];
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            float g0 = __uint_as_float(vg[j8 * 8 + 2 * j]), g1 = __uint_as_float(vg[j8 * 8 + 2 * j + 1]);
                            float u0 = __uint_as_float(vu[j8 * 8 + 2 * j]), u1 = __uint_as_float(vu[j8 * 8 + 2 * j + 1]);
                            if (p.ep.bias) {
                                g0 = __fadd_rn(g0, bf16_lo(bg[j])); g1 = __fadd_rn(g1, bf16_hi(bg[j]));
                                u0 = __fadd_rn(u0, bf16_lo(bu[j])); u1 = __fadd_rn(u1, bf16_hi(bu[j]));
                            }
                            packed[j] = pack_bf16_pair(swiglu_f32(g0, u0, true), swiglu_f32(g1, u1, true));
                        }
                        *reinterpret_cast<uint4 *>(p.out + (size_t)row * p.N + col) = *reinterpret_cast<uint4 *>(packed);
                    }
                }
            } else {
#pragma unroll 1
                for (int hc = 0; hc < 16 / SPLIT; hc++) {
                    const int c = half * (16 / SPLIT) + hc;
                    uint32_t v[16];
                    tmem_load_32x16(lane_base + c * 16, v);
                    tmem_load_wait();
                    if (!row_ok) continue;
#pragma unroll
                    for (int j8 = 0; j8 < 2; j8++) {
                        const uint32_t col = n0 + c * 16 + j8 * 8;
                        if (col >= p.N) continue;
                        uint32_t bias[4] = {0, 0, 0, 0}, gate[4] = {0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u};
                        uint32_t res[4] = {0, 0, 0, 0};
                        if (p.ep.bias) *reinterpret_cast<uint4 *>(bias) = *reinterpret_cast<const uint4 *>(p.ep.bias + col);
                        if (p.ep.gate) *reinterpret_cast<uint4 *>(gate) = *reinterpret_cast<const uint4 *>(p.ep.gate + col);
                        if (p.ep.residual)
                            *reinterpret_cast<uint4 *>(res) = *reinterpret_cast<const uint4 *>(p.ep.residual + (size_t)row * p.N + col);
                        uint32_t packed[4];
#pragma unroll
                        for (int j = 0; j < 4; j++)
                            packed[j] = epilogue_pair(__uint_as_float(v[j8 * 8 + 2 * j]), __uint_as_float(v[j8 * 8 + 2 * j + 1]), bias[j],
                                                      p.ep.bias != nullptr, p.ep.activation, gated, gate[j], res[j]);
                        *reinterpret_cast<uint4 *>(p.out + (size_t)row * p.N + col) = *reinterpret_cast<uint4 *>(packed);
                    }
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

    /* ---------------------------------------------------------- teardown */
    if (failure) {
        *abort_flag = 1;
        atomicCAS(p.status, 0u, failure | (blockIdx.x << 8));
    }
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        /* give any TMA copy still in flight time to land before the shared memory is released */
        long long start = clock64();
        while (clock64() - start < 2000000ll) { }
        __syncthreads();
    }
    cluster_sync();           /* the peer's shared memory and TMEM are in use by the leader's MMAs until here */
    if (warp == C::MMA_WARP) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

} /* namespace h3q8 */
