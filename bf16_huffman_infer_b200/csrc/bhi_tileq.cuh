// Fused decode + tensor-core product with the four-row decoders of the GEMV kernel (sm_100a: tcgen05 + TMEM), for up to
// 32 activation rows.
//
// Same product and same roles as tile_kernel (bhi_tile.cuh): decoder warps fill K-major W stages in shared memory, one
// warp issues the MMAs, one requests the X blocks by TMA, four read the accumulators back.  What differs is where the
// decoders get their streams from: here the records of a QUAD (four rows) are copied whole into a two-ended ring by the
// bulk-copy engine, as in quad_kernel (bhi_quad.cuh), and decoded with its cursor-in-shared-memory loop: two table
// look-ups per window fetch, 47 to 52 instructions per row and 128-column block instead of 73.  Eight groups of two warps hold
// eight quads, so a SET is 32 weight rows (MMA N = 32) and a W stage is a PAIR of 128-column blocks (16 MMAs), because
// one decoder step yields two blocks.  The rings take the shared memory the larger X stages of more than 32 rows would
// need; beyond that (and for records that do not fit a ring slot pair) tile_kernel runs.
//
// Lane (r = lane >> 3, j = lane & 7) of warp w of group g decodes, for pass p of its two passes, streams
// sigma = 8 (2 w + p) + j and sigma + 32 of row 4 g + r of the set: the words of columns 2 sigma, 2 sigma + 1 and
// 64 + 2 sigma, 65 + 2 sigma.  W stage layout: 16-byte units at unit index kc * 36 + row (kc = K-chunk of 8 columns), so
// the 32 lanes of a store hit 32 different banks.
//
// Measured on B200 (16 rows of X; 4096 x 4096 / 12288 x 4096 / 4096 x 12288): 23.2 / 60.3 / 59.4 us, against 22.5 / 59.3 /
// 62.1 us for decode-to-dense + library GEMM and 32.7 / 64.9 / 88.3 us for tile_kernel.  Without its MMAs (results wrong)
// the same kernel takes 17.1 us on the first shape: the decoders run at the GEMV kernel's pace.  What holds it back is the
// issue rate of tcgen05.mma while the decoders run: with the issuer and the decoders uncoupled (no waits between them,
// results wrong) the 256 MMAs of a CTA's set take 16.5 us, 64 ns (122 clocks) each against 52 clocks on an idle SM, whatever
// N (8 or 32) and M (64 or 128).  At 8 MMAs per block of 32 rows that is 0.51 us against 0.38 us of decoding.  Tried without
// effect: three W stages, up to eight X stages, polling instead of parked waits, the 8 MMAs of a block as one piece of
// inline assembly, a scheduler without decoder warps for the issuer, four issuer warps (one per scheduler) taking the
// stages in turn (slower: 25.6 us).  Tensor pipe 8 % busy, shared-memory data pipe 35 %, issue slots 26 %.  Fewer, larger
// MMAs need more rows per set, and a set's records must fit the rings.
#pragma once

#include "bhi_quad.cuh"
#include "bhi_tile.cuh"

namespace bhi {

constexpr int kTqDecoders = 16;                 // decoder warps: 8 groups of 2
constexpr int kTqIssuer = 16;
constexpr int kTqLoader = 17;                   // 18, 19 idle (a warpgroup of four keeps setmaxnreg aligned)
constexpr int kTqEpilogue = 20;                 // 20..23: TMEM lane quarters 0..3
constexpr int kTqWarps = 24;
constexpr int kTqThreads = kTqWarps * 32;
constexpr int kTqRows = 32;                     // rows per set = MMA N
constexpr uint32_t kTqLbo = 36;                 // 16-byte units between K-chunks of a W half-stage (576 bytes: 16 banks apart)
constexpr uint32_t kTqHalf = 16u * kTqLbo * 16u;        // bytes of one 128-column block of a W stage
constexpr uint32_t kTqWStage = 2u * kTqHalf;
constexpr int kTqWStages = 2;
constexpr int kTqXStagesMax = 8;

struct TqPlan {
    QuadGeom G;            // table region, ring geometry (part / acc / ys / x fields unused)
    uint32_t x_rows, x_atom, x_stage, x_stages;
    uint32_t x_off, w_off, total;
    int sets_per_cta;
};

template <class Codec>
__global__ void __launch_bounds__(kTqThreads, 1)
tileq_kernel(Layer L, typename Codec::Args targs, const uint8_t *prepared, const __grid_constant__ CUtensorMap xmap, uint16_t *Y, int B,
             TqPlan P, Consts kc) {
    extern __shared__ __align__(1024) uint8_t smem[];
    using Tables = typename Codec::Tables;
    using Dec = typename QuadOf<Codec>::type;
    constexpr bool kHuff = std::is_same<Codec, HuffCodec>::value;
    constexpr int PPW = 2, kWG = 2;                  // passes per warp, warps per group
    constexpr int kRG = 4;                           // blocks per sign/mantissa prefetch group
    const QuadGeom &G = P.G;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint32_t *fast = reinterpret_cast<uint32_t *>(smem);
    Tables &tab = *reinterpret_cast<Tables *>(smem + G.lut_bytes);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + G.lut_bytes + kExactBytes);
    const uint32_t smem_base = smem_addr(smem);
    const uint32_t table_bar = smem_addr(&bars[16]);
    const uint32_t full_bar = smem_addr(&bars[17]);        // + 8 * W stage
    const uint32_t xfull_bar = smem_addr(&bars[23]);       // + 8 * X stage
    const uint32_t sdone_bar = smem_addr(&bars[31]);       // + 8 * (stage number % 8): the stage's MMAs are complete
    const uint32_t done_bar = smem_addr(&bars[39]);        // + 8 * accumulator
    const uint32_t free_bar = smem_addr(&bars[41]);        // + 8 * accumulator
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(&bars[43]);
    static_assert(44 * 8 <= kQuadCtrlBytes, "control block too small");

    const int nsets = (L.M + kTqRows - 1) / kTqRows;
    const int set_lo = blockIdx.x * P.sets_per_cta;
    const int my_sets = max(0, min(nsets - set_lo, P.sets_per_cta));
    const int nblk = L.Nc >> 7;
    const int npair = (nblk + 1) >> 1;               // W stages per chunk
    const uint32_t stages_per_set = static_cast<uint32_t>(L.S * npair);
    const uint32_t my_stages = static_cast<uint32_t>(my_sets) * stages_per_set;

    pdl_launch_dependents();
    if (tid == 0) {
        mbar_init(table_bar, 1);
        for (int g = 0; g < 2 * kQuadGroups; g++) mbar_init(smem_addr(&bars[g]), 1);
        for (int s = 0; s < kTqWStages; s++) {
            mbar_init(full_bar + 8 * s, kTqDecoders);
        }
        for (int s = 0; s < kTqXStagesMax; s++) {
            mbar_init(xfull_bar + 8 * s, 1);
            mbar_init(sdone_bar + 8 * s, 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(done_bar + 8 * a, 1);
            mbar_init(free_bar + 8 * a, 4);
        }
        mbar_fence_init();
    }
    if (warp == kTqIssuer) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(64) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    if (prepared != nullptr && tid == 0) {
        mbar_expect_tx(table_bar, kPreparedBytes);
        bulk_copy_g2s(smem_base + G.lut_bytes - kPairEntries * 4, prepared, kPreparedBytes, table_bar);
    }

    // X stage u (counted over all sets of this CTA) holds the two blocks of W stage u: four atoms of 64 columns
    auto request_x = [&](uint32_t u) {               // one thread; the stage must be free
        const uint32_t s = u % P.x_stages;
        const uint32_t bar = xfull_bar + 8u * s;
        const uint32_t dst = smem_base + P.x_off + s * P.x_stage;
        const uint32_t v = u % stages_per_set;
        const int k = static_cast<int>(v) / npair, pr = static_cast<int>(v) % npair;
        const int col = k * L.Nc + pr * 256;
        const int atoms = (2 * pr + 1 < nblk) ? 4 : 2;
        mbar_expect_tx(bar, static_cast<uint32_t>(atoms) * P.x_atom);
        for (int a = 0; a < atoms; a++) tma_load_2d(dst + a * P.x_atom, &xmap, col + a * kXAtomCols, 0, bar);
    };

    pdl_wait();
    if (warp == kTqLoader && lane == 0)
        for (uint32_t u = 0; u < P.x_stages && u < my_stages; u++) request_x(u);

    // ---- units of the decoder groups (weights only: started before the tables are ready) ------------------------
    const int group = warp >> 1, wig = warp & 1;     // decoders only
    const int r = lane >> 3;
    const uint32_t sigma4 = 4u * (8 * (wig * PPW) + (lane & 7));
    const uint32_t bar0 = smem_addr(&bars[2 * (group & 7)]);
    const uint32_t ring = G.ring_off + (group & 7) * G.ring_bytes;
    const int nrec = L.S * L.M;
    const int nc4 = L.Nc >> 2;
    const int q_lo = 8 * set_lo, nq = 8 * my_sets;

    auto describe = [&](int qi, int k, QuadUnit &u) {
        u.qi = qi;
        u.k = k;
        const int m = min(4 * (q_lo + qi) + r, L.M - 1);      // rows past the end decode the last row again; nobody reads them
        u.rec = k * L.M + m;
        u.off = static_cast<uint32_t>(__ldg(L.offsets + u.rec));
        const int64_t end = (u.rec + 1 < nrec) ? static_cast<int64_t>(static_cast<uint32_t>(__ldg(L.offsets + u.rec + 1)))
                                               : L.exp_words;
        const int64_t words = end - static_cast<int64_t>(u.off);
        const bool ok = words > 0 && (words & 63) == 0 && (u.off & 3u) == 0 && end <= L.exp_words && words <= (1 << 16);
        uint32_t rows = ok ? static_cast<uint32_t>(words >> 6) : 0u;
        u.bytes = rows * 256u;
        rows = max(rows, __shfl_xor_sync(0xFFFFFFFFu, rows, 8));
        rows = max(rows, __shfl_xor_sync(0xFFFFFFFFu, rows, 16));
        u.rows = rows;
        u.staged = __all_sync(0xFFFFFFFFu, ok) && u.foot() <= G.ring_bytes;
        u.valid = true;
    };
    auto place = [&](QuadUnit &u, int slot) { u.base = slot == 0 ? ring : ring + G.ring_bytes - u.foot(); };
    auto issue = [&](QuadUnit &u, int slot) {
        place(u, slot);
        if (wig == 0) {
            const uint32_t bar = bar0 + 8u * slot;
            uint32_t total = u.bytes;
            total += __shfl_xor_sync(0xFFFFFFFFu, total, 8);
            total += __shfl_xor_sync(0xFFFFFFFFu, total, 16);
            if (lane == 0) mbar_expect_tx(bar, total);
            __syncwarp();
            if ((lane & 7) == 0) {
                bulk_copy_g2s(smem_base + u.base + r * u.stride(), L.exp + u.off, u.bytes, bar);
                prefetch_l2(L.rem + static_cast<int64_t>(u.rec) * L.Nc, static_cast<uint32_t>(L.Nc));
            }
        }
    };
    // units of a group: its quad of each set in turn, and for each the chunks in order
    auto next_unit = [&](const QuadUnit &c, QuadUnit &u) {
        u.valid = false;
        if (c.k + 1 < L.S) describe(c.qi, c.k + 1, u);
        else if (c.qi + kQuadGroups < nq) describe(c.qi + kQuadGroups, 0, u);
    };
    QuadUnit cur, nxt;
    cur.valid = false;
    if (warp < kTqDecoders && group < nq) {
        describe(group, 0, cur);
        if (cur.staged) issue(cur, 0);
        else place(cur, 0);
    }

    // ---- tables: every warp helps ------------------------------------------------------------------------------------
    uint32_t flagged = 1u;
    const uint32_t copies = 1u << (G.copy_shift - 2);
    if (prepared == nullptr) {
        load_tables(tab, targs, tid, kTqThreads);
        __syncthreads();
        if constexpr (kHuff) {
            for (int v = tid; v < kPairEntries; v += kTqThreads) {
                const uint32_t e = pair_entry(tab, v);
                for (uint32_t c = 0; c < copies; c++) fast[v * copies + c] = e;
            }
        } else {
            for (int v = tid; v < (1 << kc.ans_bits); v += kTqThreads) {
                const uint32_t e = __ldg(targs.lut + v);
                for (uint32_t c = 0; c < copies; c++) fast[v * copies + c] = e;
            }
        }
    } else {
        if (!mbar_wait_bounded(table_bar, 0u) && tid == 0) atomicExch(&g_staged_status, 2);
        flagged = prepared_flagged(smem + G.lut_bytes);
        if (copies > 1) {
            // fan out: entry v (one word at the tail of the region) -> `copies` words at v * copies; the targets overlap the
            // raw copy, so every thread reads its raw entries before anybody writes
            constexpr int kPer = (kPairEntries + kTqThreads - 1) / kTqThreads;
            const uint32_t *raw = fast + (G.lut_bytes - kPairEntries * 4) / 4;
            uint32_t mine[kPer];
#pragma unroll
            for (int i = 0; i < kPer; i++) {
                const int v = tid + i * kTqThreads;
                mine[i] = v < kPairEntries ? raw[v] : 0u;
            }
            __syncthreads();
#pragma unroll
            for (int i = 0; i < kPer; i++) {
                const int v = tid + i * kTqThreads;
                if (v < kPairEntries)
                    for (uint32_t c = 0; c < copies; c++) fast[v * copies + c] = mine[i];
            }
        }
    }
    const bool checked = kHuff && flagged != 0u;
    __syncthreads();

    if (warp < kTqDecoders) {
        QuadCtx ctx;
        ctx.smem = smem;
        ctx.k = kc;
        ctx.copy_shift = G.copy_shift;
        ctx.copy_off = 4u * (lane & ((1u << (G.copy_shift - 2)) - 1u));
        ctx.index_mask = G.index_mask;
        ctx.bias = kHuff ? G.copy_shift : 0u;
        ctx.lut_bytes = G.lut_bytes;

        // this lane's word of pass 0, block half 0, inside a W stage: row 4 group + r, K-chunk 4 wig + (j >> 2), word j & 3
        const uint32_t j8 = lane & 7;
        const uint32_t ws_lane = P.w_off + (((4u * wig + (j8 >> 2)) * kTqLbo + 4u * group + r) * 4u + (j8 & 3u)) * 4u;
        uint32_t stage = 0u, un = 0u;                // slot in the W ring and stage number; every decoder warp and the issuer walk the same sequence
        auto begin_pair = [&]() {
            // the slot is free once the MMAs that read it kTqWStages stages ago have completed
            if (un >= kTqWStages) {
                const uint32_t w = un - kTqWStages;
                if (!mbar_wait_parked(sdone_bar + 8u * (w & 7u), (w >> 3) & 1u) && lane == 0) atomicExch(&g_staged_status, 3);
            }
        };
        auto emit = [&](int pp, int half, uint32_t rw, uint32_t e0, uint32_t e1) {
            uint8_t *ws = smem + ws_lane + stage * kTqWStage + half * kTqHalf + pp * (2 * kTqLbo * 16);
            *reinterpret_cast<uint32_t *>(ws) = bitselect(prmt(rw, 0u, 0x1100u), e0, kRemMask);
            *reinterpret_cast<uint32_t *>(ws + 8 * kTqLbo * 16) = bitselect(prmt(rw, 0u, 0x3322u), e1, kRemMask);
        };
        auto commit_pair = [&]() {
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(full_bar + 8u * stage);
            un++;
            if (++stage == kTqWStages) stage = 0u;
        };

        uint32_t phases = 0u;
        int slot = 0;
        uint32_t r_cur[PPW][kRG], r_nxt[PPW][kRG];
        bool have_first = false;
        while (cur.valid) {
            next_unit(cur, nxt);
            const bool early = nxt.valid && nxt.staged && (!cur.staged || cur.foot() + nxt.foot() <= G.ring_bytes);
            if (early) issue(nxt, slot ^ 1);
            const uint32_t *rem = reinterpret_cast<const uint32_t *>(L.rem) + static_cast<int64_t>(cur.rec) * nc4 + (sigma4 >> 2);
            const uint32_t *rem_next =
                nxt.valid ? reinterpret_cast<const uint32_t *>(L.rem) + static_cast<int64_t>(nxt.rec) * nc4 + (sigma4 >> 2) : rem;
            bool next_first = false;
            bool decoded = false;

            if (cur.staged) {
                const int full = nblk / kRG;                // groups of kRG blocks whose sign/mantissa words are prefetched
                if (full > 0 && !have_first) {
#pragma unroll
                    for (int pp = 0; pp < PPW; pp++)
#pragma unroll
                        for (int j = 0; j < kRG; j++) r_cur[pp][j] = __ldg(rem + j * 32 + pp * 8);
                }
                const bool arrived = mbar_wait_bounded(bar0 + 8u * slot, (phases >> slot) & 1u);
                phases ^= 1u << slot;
                if (arrived) {
                    decoded = true;
                    Dec dec[PPW];
#pragma unroll
                    for (int pp = 0; pp < PPW; pp++) dec[pp].open(ctx, cur.base + r * cur.stride(), sigma4 + 32u * pp, cur.rows);
                    auto run = [&](auto checked_tag) {
                        constexpr bool kChecked = decltype(checked_tag)::value;
                        for (int gi = 0; gi < full; gi++) {
                            const uint32_t *src = (gi + 1 < full) ? rem + (gi + 1) * (kRG * 32) : rem_next;
#pragma unroll
                            for (int pp = 0; pp < PPW; pp++)
#pragma unroll
                                for (int j = 0; j < kRG; j++) r_nxt[pp][j] = __ldg(src + j * 32 + pp * 8);
#pragma unroll
                            for (int j = 0; j < kRG; j += 2) {
                                uint32_t eA0[PPW], eA1[PPW], eB0[PPW], eB1[PPW];
#pragma unroll
                                for (int pp = 0; pp < PPW; pp++) dec[pp].template two<kChecked>(ctx, eA0[pp], eA1[pp], eB0[pp], eB1[pp]);
                                begin_pair();
#pragma unroll
                                for (int pp = 0; pp < PPW; pp++) {
                                    emit(pp, 0, r_cur[pp][j], eA0[pp], eA1[pp]);
                                    emit(pp, 1, r_cur[pp][j + 1], eB0[pp], eB1[pp]);
                                }
                                commit_pair();
                            }
#pragma unroll
                            for (int pp = 0; pp < PPW; pp++) {
                                dec[pp].clamp();
#pragma unroll
                                for (int j = 0; j < kRG; j++) r_cur[pp][j] = r_nxt[pp][j];
                            }
                        }
                        // blocks past the last full group: sign/mantissa words fetched on the spot
                        for (int blk = full * kRG; blk < nblk; blk += 2) {
                            uint32_t eA0[PPW], eA1[PPW], eB0[PPW], eB1[PPW];
#pragma unroll
                            for (int pp = 0; pp < PPW; pp++) dec[pp].template two<kChecked>(ctx, eA0[pp], eA1[pp], eB0[pp], eB1[pp]);
                            begin_pair();
#pragma unroll
                            for (int pp = 0; pp < PPW; pp++) {
                                emit(pp, 0, __ldg(rem + blk * 32 + pp * 8), eA0[pp], eA1[pp]);
                                if (blk + 1 < nblk) emit(pp, 1, __ldg(rem + (blk + 1) * 32 + pp * 8), eB0[pp], eB1[pp]);
                            }
                            commit_pair();
                        }
                    };
                    if (checked) run(std::true_type{});
                    else run(std::false_type{});
                    next_first = nxt.valid && full > 0;
                } else if (lane == 0) {
                    atomicExch(&g_staged_status, 1);
                }
            } else {
                // direct unit: on-demand global loads with a bounds guard, table-exact decoders
                decoded = true;
                typename Codec::template Stream<GlobalWords> s0[PPW], s1[PPW];
#pragma unroll
                for (int pp = 0; pp < PPW; pp++) {
                    const int64_t w0 = static_cast<int64_t>(cur.off) + (sigma4 >> 2) + 8 * pp;
                    s0[pp].init(GlobalWords{L.exp, L.exp_words, w0});
                    s1[pp].init(GlobalWords{L.exp, L.exp_words, w0 + 32});
                }
                for (int blk = 0; blk < nblk; blk++) {
                    if (!(blk & 1)) begin_pair();
#pragma unroll
                    for (int pp = 0; pp < PPW; pp++) {
                        const uint32_t rw = __ldg(rem + blk * 32 + pp * 8);
                        const uint32_t a0 = s0[pp].next(tab);
                        const uint32_t b0 = s1[pp].next(tab);
                        const uint32_t a1 = s0[pp].next(tab);
                        const uint32_t b1 = s1[pp].next(tab);
                        emit(pp, blk & 1, rw, (a0 << 7) | (a1 << 23), (b0 << 7) | (b1 << 23));
                    }
                    if ((blk & 1) || blk + 1 == nblk) commit_pair();
                }
            }
            if (!decoded) {
                // the record never arrived (status set above): keep the pipeline moving, the products are garbage
                for (int pr = 0; pr < npair; pr++) {
                    begin_pair();
                    commit_pair();
                }
            }
            have_first = next_first;
            group_barrier(group, kWG * 32);          // the unit's ring space is free
            if (nxt.valid && !early) {
                if (nxt.staged) issue(nxt, slot ^ 1);
                else place(nxt, slot ^ 1);
            }
            cur = nxt;
            slot ^= 1;
        }
    } else if (warp == kTqIssuer) {
        // ---- issuer: 8 MMAs per 128-column block, two blocks per stage -------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t kIdesc = tile_idesc(kTqRows);
            uint32_t u = 0u;
            for (int nset = 0; nset < my_sets; nset++) {
                const uint32_t a = static_cast<uint32_t>(nset) & 1u;
                const uint32_t acc = tmem + a * kTqRows;
                if (nset >= 2 && !mbar_wait_parked(free_bar + 8u * a, ((static_cast<uint32_t>(nset) >> 1) - 1u) & 1u)) atomicExch(&g_staged_status, 7);
                for (uint32_t v = 0; v < stages_per_set; v++, u++) {
                    const uint32_t s = u % kTqWStages, wr = u / kTqWStages, xs = u % P.x_stages, xwr = u / P.x_stages;
                    const int pr = static_cast<int>(v) % npair;
                    const int halves = (2 * pr + 1 < nblk) ? 2 : 1;
                    if (!mbar_wait_parked(xfull_bar + 8u * xs, xwr & 1u)) atomicExch(&g_staged_status, 8);
                    if (!mbar_wait_parked(full_bar + 8u * s, wr & 1u)) atomicExch(&g_staged_status, 4);
                    tc_fence_after();
                    const uint32_t xt = smem_base + P.x_off + xs * P.x_stage, wt = smem_base + P.w_off + s * kTqWStage;
                    for (int h = 0; h < halves; h++) {
                        // descriptors of the 8 K-steps differ in the address field (low word) only: one add each
                        const uint64_t xd0 = umma_desc_sw128(xt + (2 * h) * P.x_atom), xd1 = umma_desc_sw128(xt + (2 * h + 1) * P.x_atom);
                        const uint64_t wd = umma_desc(wt + h * kTqHalf, kTqLbo);
#pragma unroll
                        for (int j = 0; j < 8; j++)
                            umma_bf16(acc, ((j >> 2) ? xd1 : xd0) + static_cast<uint64_t>((j & 3) * 2), wd + static_cast<uint64_t>(j * 2 * kTqLbo),
                                      kIdesc, (v | static_cast<uint32_t>(h) | static_cast<uint32_t>(j)) != 0u ? 1u : 0u);
                    }
                    // one commit per stage (each costs the issuing thread about 300 clocks): the decoders and the loader wait on the
                    // same barrier, a ring of eight so that neither can fall two phases behind
                    if (v + 1u == stages_per_set) umma_commit(done_bar + 8u * a);
                    umma_commit(sdone_bar + 8u * (u & 7u));
                }
            }
            tc_fence_before();
        }
        __syncwarp();
    } else if (warp == kTqLoader) {
        // ---- loader: X stage u + x_stages as soon as the MMAs of stage u are done ----------------------------------------
        if (lane == 0) {
            for (uint32_t u = 0; u + P.x_stages < my_stages; u++) {
                if (!mbar_wait_parked(sdone_bar + 8u * (u & 7u), (u >> 3) & 1u)) atomicExch(&g_staged_status, 6);
                request_x(u + P.x_stages);
            }
        }
        __syncwarp();
    } else if (warp >= kTqEpilogue) {
        // ---- epilogue: accumulator -> BF16 -> Y[b, set * 32 ..] ------------------------------------------------------------
        const uint32_t q = static_cast<uint32_t>(warp) & 3u;      // the TMEM lane quarter this warp may read
        const int b = static_cast<int>(q) * 32 + lane;
        for (int nset = 0; nset < my_sets; nset++) {
            const uint32_t a = static_cast<uint32_t>(nset) & 1u;
            const uint32_t acc = tmem + a * kTqRows;
            const int row0 = (set_lo + nset) * kTqRows;
            if (!mbar_wait_parked(done_bar + 8u * a, (static_cast<uint32_t>(nset) >> 1) & 1u) && lane == 0) atomicExch(&g_staged_status, 5);
            tc_fence_after();
            if (static_cast<int>(q) * 32 < B) {
#pragma unroll
                for (int c0 = 0; c0 < kTqRows; c0 += 8) {
                    uint32_t v[8];
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                                 : "r"(acc + ((q * 32u) << 16) + c0));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (b < B) {
#pragma unroll
                        for (int c = 0; c < 8; c++)
                            if (row0 + c0 + c < L.M) Y[static_cast<int64_t>(b) * L.M + row0 + c0 + c] = f32_to_bf16_rn(__uint_as_float(v[c]));
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(free_bar + 8u * a);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == kTqIssuer) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(64) : "memory");
}

// ---- host side ---------------------------------------------------------------------------------------
template <class Codec>
static bool tileq_plan(const Layer &L, int B, uint32_t ans_bits, TqPlan &P) {
    constexpr bool kHuff = std::is_same<Codec, HuffCodec>::value;
    const uint32_t one_table = kHuff ? kPairEntries * 4u : (4u << ans_bits);
    P.x_rows = static_cast<uint32_t>((B + 7) & ~7);
    P.x_atom = P.x_rows * 128u;                       // 64 columns; a multiple of 1024 bytes
    P.x_stage = 4u * P.x_atom;
    const uint32_t cap = static_cast<uint32_t>(kSmemMax);
    const uint32_t w_bytes = (kTqWStages * kTqWStage + 1023u) & ~1023u;
    // [tables][X ring][W stages][rings][slack].  A 128-row MMA reads 16 KB from the start of each X atom whatever the
    // batch; the W stages and rings behind the X ring keep that inside the allocation.
    for (int copies_log2 = 2; copies_log2 >= 0; copies_log2--) {
        const uint32_t lut = one_table << copies_log2;
        const uint32_t fixed = ((lut + kExactBytes + kQuadCtrlBytes + 1023u) & ~1023u);
        const uint32_t rest = fixed + w_bytes + kQuadGroups * kQuadRingWant + kSlackBytes;
        if (rest + 2u * P.x_stage > cap) continue;
        uint32_t xs = (cap - rest) / P.x_stage;
        if (xs > kTqXStagesMax) xs = kTqXStagesMax;
        P.x_stages = xs;
        P.G = QuadGeom{};
        P.G.lut_bytes = lut;
        P.G.copy_shift = 2u + copies_log2;
        P.G.index_mask = kHuff ? (static_cast<uint32_t>(kPairEntries - 1) << P.G.copy_shift) : (((1u << ans_bits) - 1u) << P.G.copy_shift);
        P.x_off = fixed;
        P.w_off = P.x_off + xs * P.x_stage;
        P.G.ring_off = P.w_off + w_bytes;
        uint32_t ring_bytes = ((cap - kSlackBytes - P.G.ring_off) / kQuadGroups) & ~255u;
        if (ring_bytes > 4u * kRingMax) ring_bytes = 4u * kRingMax;
        P.G.ring_bytes = ring_bytes;
        P.total = P.G.ring_off + kQuadGroups * ring_bytes + kSlackBytes;
        return true;
    }
    return false;
}

template <class Codec>
static int tileq_launch(const Layer &L, const typename Codec::Args &targs, const uint8_t *prepared, const uint16_t *X, uint16_t *Y,
                        int B, cudaStream_t st) {
    if (!staged_shape_ok(L) || !aligned(prepared, 16)) return kStagedDeclined;
    if (static_cast<int64_t>(L.S) * L.M >= (1ll << 31)) return kStagedDeclined;
    const uint32_t ans_bits = ans_bits_of(targs);
    TqPlan plan{};
    if (!tileq_plan<Codec>(L, B, ans_bits, plan)) return kStagedDeclined;
    auto kernel = tileq_kernel<Codec>;
    if (int rc = staged_prepare(kernel)) return rc;
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) return fail(BHI_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    // X as a [B, K] BF16 tensor; a box is 64 columns (one 128-byte swizzle atom) by the padded batch
    const uint64_t K = static_cast<uint64_t>(L.S) * L.Nc;
    alignas(64) CUtensorMap xmap;
    const cuuint64_t dims[2] = {K, static_cast<cuuint64_t>(B)};
    const cuuint64_t strides[1] = {K * 2};
    const cuuint32_t box[2] = {kXAtomCols, plan.x_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult cr = encode(&xmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t *>(X), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return fail(BHI_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(cr)));
    const int nsets = (L.M + kTqRows - 1) / kTqRows;
    const int sms = sm_count();
    plan.sets_per_cta = (nsets + sms - 1) / sms;
    const int grid = (nsets + plan.sets_per_cta - 1) / plan.sets_per_cta;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kTqThreads);
    cfg.dynamicSmemBytes = plan.total;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap_launches() ? 1 : 0;
    const Consts k{ans_bits, (1u << ans_bits) - 1u, 1u, 8u, 4u * kCopies, 65536u};
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, L, targs, prepared, xmap, Y, B, plan, k);
    return e == cudaSuccess ? BHI_OK : cuda_fail(e, "fused tensor-core kernel launch");
}

}  // namespace bhi
