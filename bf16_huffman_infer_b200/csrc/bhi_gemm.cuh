// Fused decode + tensor-core product for up to 128 activation rows (sm_100a: tcgen05.mma with the
// accumulator in tensor memory).
//
// Y[b, m] = sum_c X[b, c] * W[m, c].  The reference decodes W to a dense BF16 scratch in HBM and calls
// a library GEMM (functional.py:405-407), which moves every weight three times.  Here a CTA decodes
// SETS of 32 weight rows (one row per warp) into shared memory and multiplies them on the fly; W is
// read once, compressed, and its dense form never leaves the SM.
//
// MMA shape.  The batch is the M dimension (A operand = X, 128 rows; rows beyond the batch feed
// accumulator rows nobody reads), a set of 32 weight rows is N, K advances in blocks of 128 columns
// (8 MMAs of K = 16).  X blocks arrive by TMA (cp.async.bulk.tensor, two boxes of 64 columns x padded
// batch rows) in the 128-byte-swizzled K-major layout; rows past the batch are filled with zeros by
// the copy engine.  Decoded weights are K-major without swizzle: 16-byte units (8 BF16) at unit index
// kc * 33 + row, so the per-lane stores of decoded words are bank-conflict free.  The accumulator
// D[128 x 32] FP32 lives in tensor memory, double-buffered over sets; four warps read it back with
// tcgen05.ld and store BF16 while the next set is already being multiplied.
//
// Pipeline.  A K-block of both operands occupies one of NS stages.  Warps are not in lock step: a warp
// decodes its row's 128 columns (same decoders as the GEMV kernel), waits until the MMAs that last
// read the stage have completed (mbarrier `empty`, arrived on by tcgen05.commit), stores, fences to
// the async proxy and arrives on the stage's `full` mbarrier, which also counts the bytes of the X
// block.  For block t, lane 0 of warp t mod 32 additionally requests the X block NS - 1 blocks ahead,
// waits for `full`, issues the 8 MMAs and commits them to `empty`.  No CTA-wide barrier sits in the
// loop.  Every wait is bounded (status word, see bhi_debug_status).
//
// Cost model (measured on B200).  A tcgen05.mma of 128 x N x 16 occupies the tensor pipe for about
// 90 ns whether N is 32 or 256, and the issuing thread stalls for as long.  A set of 32 rows (what the
// rings can hold: one record per warp plus its successor) therefore pays 8 x 90 ns per 128-column
// block, about twice what the 32 warps need to decode it, and the stall lands on a warp that also
// has a row to decode.  So this kernel is tensor-issue bound and does NOT beat decoding to a dense
// scratch followed by a library GEMM (about 150 us against 81 us for a 12288 x 4096 layer); the host layer
// keeps the reference's decode + GEMM branch as the default above 8 rows and offers this path as an
// option.
#pragma once

#include <cuda.h>      // CUtensorMap and the encode entry point's types; the driver library is not linked

#include "bhi_staged.cuh"

namespace bhi {

constexpr int kGemmWarps = 32;
constexpr int kGemmRows = 32;                    // weight rows per set (MMA N)
constexpr int kGemmBatch = 128;                  // MMA M
constexpr int kWLbo = 33;                        // 16-byte units between K-chunks of the decoded-weight tile (odd)
constexpr int kWTileBytes = 16 * kWLbo * 16;     // 8 448
constexpr int kGemmCopies = 2;                   // fast-table copies (lane & 1 picks one): leaves more room for the rings
constexpr int kGemmLutBytes = kPairEntries * 4 * kGemmCopies;
constexpr int kGemmHeader = kGemmLutBytes + kExactBytes + kCtrlBytes;
constexpr int kGemmRingMax = 4608;
constexpr int kDirectState = 1024;               // ring bytes a record decoded from global memory keeps its state in
constexpr int kGemmStages = 2;                   // measured: deeper rings only add waiting warps that compete with the decoders
constexpr int kGemmStagesMax = 4;                // barrier slots reserved in the control block
constexpr int kTmemCols = 64;                    // two accumulators of 32 columns
constexpr int kXAtomCols = 64;                   // columns of one 128-byte swizzle atom

// instruction descriptor: D = F32, A = B = BF16, both K-major, N = 32, M = 128
constexpr uint32_t kGemmIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((kGemmRows >> 3) << 17) | ((kGemmBatch >> 4) << 24);

// Shared-memory plan of one launch, derived from the batch on the host.
struct GemmPlan {
    uint32_t x_rows;       // batch rounded up to 8: rows of a TMA box
    uint32_t x_stage;      // bytes per X stage (two atoms of x_rows * 128 bytes), a multiple of 1024
    uint32_t stages;
    uint32_t x_off, w_off, ring_off, ring_bytes, total;
};

__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_byte_addr, uint32_t lbo_units) {
    // K-major, no swizzle: start address, leading (K-chunk) offset, stride (8-row group) offset = 128 B,
    // all in 16-byte units; descriptor version 1
    return static_cast<uint64_t>((smem_byte_addr >> 4) & 0x3FFFu) | (static_cast<uint64_t>(lbo_units & 0x3FFFu) << 16) |
           (static_cast<uint64_t>(8u) << 32) | (static_cast<uint64_t>(1u) << 46);
}
// K-major, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart, stage base 1024-aligned
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_byte_addr) {
    return static_cast<uint64_t>((smem_byte_addr >> 4) & 0x3FFFu) | (static_cast<uint64_t>(1u) << 16) |
           (static_cast<uint64_t>(64u) << 32) | (static_cast<uint64_t>(1u) << 46) | (static_cast<uint64_t>(2u) << 61);
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// fast tables in kGemmCopies interleaved copies
__device__ __forceinline__ void gemm_fast_table(uint32_t *fast, const HuffTables &t, int tid, int n) {
    for (int v = tid; v < kPairEntries; v += n) {
        const uint32_t e = pair_entry(t, v);
        *reinterpret_cast<uint2 *>(fast + v * kGemmCopies) = make_uint2(e, e);
    }
}
__device__ __forceinline__ void gemm_fast_table(uint32_t *fast, const AnsTables &t, int tid, int n) {
    for (int i = tid; i < (1 << t.bits); i += n) {
        const uint32_t e = __ldg(t.lut + i);
        *reinterpret_cast<uint2 *>(fast + i * kGemmCopies) = make_uint2(e, e);
    }
}

// A record that cannot be staged (too large for the ring, or offsets out of storage order) is decoded
// from global memory by the table-exact decoder, one 128-column block per call.  All warps of the CTA
// advance block by block, so the two stream states of a lane rest in the warp's ring between calls
// (word j of lane l at st[32 * j + l]); out of line, such records are rare.
__device__ __forceinline__ void stream_save(const HuffStream<GlobalWords> &s, uint32_t *st, uint32_t off) {
    st[0] = static_cast<uint32_t>(s.src.at - off);
    st[32] = static_cast<uint32_t>(s.win);
    st[64] = static_cast<uint32_t>(s.win >> 32);
    st[96] = s.have;
}
__device__ __forceinline__ void stream_load(HuffStream<GlobalWords> &s, const uint32_t *st, uint32_t off) {
    s.src.at = static_cast<int64_t>(off) + st[0];
    s.win = static_cast<uint64_t>(st[32]) | (static_cast<uint64_t>(st[64]) << 32);
    s.have = st[96];
}
__device__ __forceinline__ void stream_save(const AnsStream<GlobalWords> &s, uint32_t *st, uint32_t off) {
    st[0] = static_cast<uint32_t>(s.src.at - off);
    st[32] = static_cast<uint32_t>(s.state);
    st[64] = static_cast<uint32_t>(s.state >> 32);
}
__device__ __forceinline__ void stream_load(AnsStream<GlobalWords> &s, const uint32_t *st, uint32_t off) {
    s.src.at = static_cast<int64_t>(off) + st[0];
    s.state = static_cast<uint64_t>(st[32]) | (static_cast<uint64_t>(st[64]) << 32);
}

template <class Codec>
__device__ __noinline__ uint2 direct_block(const uint32_t *exp, int64_t exp_words, uint32_t off, int lane, bool first,
                                           uint32_t *st, const typename Codec::Tables *tab) {
    typename Codec::template Stream<GlobalWords> s0, s1;
    if (first) {
        s0.init(GlobalWords{exp, exp_words, static_cast<int64_t>(off) + lane});
        s1.init(GlobalWords{exp, exp_words, static_cast<int64_t>(off) + 32 + lane});
    } else {
        s0.src.base = s1.src.base = exp;
        s0.src.limit = s1.src.limit = exp_words;
        stream_load(s0, st, off);
        stream_load(s1, st + 128, off);
    }
    const uint32_t a0 = s0.next(*tab);
    const uint32_t b0 = s1.next(*tab);
    const uint32_t a1 = s0.next(*tab);
    const uint32_t b1 = s1.next(*tab);
    stream_save(s0, st, off);
    stream_save(s1, st + 128, off);
    return make_uint2((a0 << 7) | (a1 << 23), (b0 << 7) | (b1 << 23));
}

template <class Codec>
__global__ void __launch_bounds__(kGemmWarps * 32, 1)
gemm_kernel(Layer L, typename Codec::Args targs, const uint8_t *prepared, const __grid_constant__ CUtensorMap xmap,
            uint16_t *Y, int B, GemmPlan P, Consts k) {
    extern __shared__ __align__(1024) uint8_t smem[];
    using Tables = typename Codec::Tables;
    using Dec = typename StagedOf<Codec>::type;
    constexpr int NW = kGemmWarps;

    uint32_t *fast = reinterpret_cast<uint32_t *>(smem);
    Tables &tab = *reinterpret_cast<Tables *>(smem + kGemmLutBytes);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kGemmLutBytes + kExactBytes);
    const uint32_t table_bar = smem_addr(&bars[2 * NW]);
    const uint32_t full_bar = smem_addr(&bars[2 * NW + 1]);                    // + 8 * stage
    const uint32_t empty_bar = smem_addr(&bars[2 * NW + 1 + kGemmStagesMax]);  // + 8 * stage
    const uint32_t done_bar = smem_addr(&bars[2 * NW + 1 + 2 * kGemmStagesMax]);   // + 8 * accumulator
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(&bars[2 * NW + 3 + 2 * kGemmStagesMax]);
    static_assert((2 * NW + 4 + 2 * kGemmStagesMax) * 8 <= kCtrlBytes, "control block too small");

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const uint32_t lane4 = 4u * lane;
    const uint32_t copy_off = 4u * (lane & (kGemmCopies - 1));
    const uint32_t ring_bytes = P.ring_bytes;
    const uint32_t ring = P.ring_off + warp * ring_bytes;
    const uint32_t smem_base = smem_addr(smem);
    const uint32_t bar0 = smem_addr(&bars[2 * warp]);

    const int64_t nrec = static_cast<int64_t>(L.S) * L.M;
    const int nblk = L.Nc >> 7;
    const int nsets = (L.M + kGemmRows - 1) / kGemmRows;
    const int first_set = blockIdx.x;

    pdl_launch_dependents();
    if (lane == 0 && first_set * kGemmRows + warp < L.M)
        prefetch_l2(L.rem + static_cast<int64_t>(first_set * kGemmRows + warp) * L.Nc, static_cast<uint32_t>(L.Nc));
    if (threadIdx.x == 0) {
        mbar_init(table_bar, 1);
        for (int s = 0; s < kGemmStagesMax; s++) {
            mbar_init(full_bar + 8 * s, NW + 1);   // one arrival per warp + the X block (arrival and bytes)
            mbar_init(empty_bar + 8 * s, 1);       // the commit of the MMAs that read the stage
        }
        mbar_init(done_bar, 1);
        mbar_init(done_bar + 8, 1);
    }
    if (lane == 0) {
        mbar_init(bar0, 1);
        mbar_init(bar0 + 8, 1);
        mbar_fence_init();
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    if (prepared != nullptr && threadIdx.x == 0) {
        mbar_expect_tx(table_bar, kPreparedBytes);
        bulk_copy_g2s(smem_base + kGemmLutBytes - kPairEntries * 4, prepared, kPreparedBytes, table_bar);
    }

    auto describe = [&](int m, int kk, Unit &u) {
        u.m = m;
        u.k = kk;
        u.rec = static_cast<int64_t>(kk) * L.M + m;
        u.off = static_cast<uint32_t>(__ldg(L.offsets + u.rec));
        const int64_t end = (u.rec + 1 < nrec) ? static_cast<int64_t>(static_cast<uint32_t>(__ldg(L.offsets + u.rec + 1)))
                                               : L.exp_words;
        const int64_t words = end - static_cast<int64_t>(u.off);
        u.staged = words > 0 && (words & 63) == 0 && (u.off & 3u) == 0 && end <= L.exp_words &&
                   words * 4 <= static_cast<int64_t>(ring_bytes);
        u.exp_bytes = u.staged ? static_cast<uint32_t>(words * 4) : 0u;
        u.valid = true;
    };
    auto issue = [&](Unit &u, int slot) {
        u.base = slot == 0 ? ring : ring + ring_bytes - u.exp_bytes;
        if (lane == 0) {
            const uint32_t bar = bar0 + 8u * slot;
            mbar_expect_tx(bar, u.exp_bytes);
            bulk_copy_g2s(smem_base + u.base, L.exp + u.off, u.exp_bytes, bar);
            prefetch_l2(L.rem + u.rec * L.Nc, static_cast<uint32_t>(L.Nc));
        }
    };

    Unit cur, nxt;
    cur.valid = false;
    if (first_set * kGemmRows + warp < L.M) {
        describe(first_set * kGemmRows + warp, 0, cur);
        if (cur.staged) issue(cur, 0);
    }

    // X blocks: block u of this CTA (counted over all of its sets) lives in stage u % NS and covers
    // columns 128 * (u % blocks_per_set).
    const uint32_t blocks_per_set = static_cast<uint32_t>(L.S * nblk);
    const uint32_t my_sets = first_set < nsets ? static_cast<uint32_t>((nsets - first_set + gridDim.x - 1) / gridDim.x) : 0u;
    const uint32_t my_blocks = my_sets * blocks_per_set;
    auto request_x = [&](uint32_t u) {               // one thread; the stage must be free
        const uint32_t s = u % P.stages;
        const uint32_t bar = full_bar + 8u * s;
        const uint32_t dst = smem_base + P.x_off + s * P.x_stage;
        const int col = static_cast<int>(u % blocks_per_set) * 128;
        mbar_expect_tx(bar, 2u * P.x_rows * 128u);
        tma_load_2d(dst, &xmap, col, 0, bar);
        tma_load_2d(dst + P.x_rows * 128u, &xmap, col + kXAtomCols, 0, bar);
    };

    pdl_wait();
    if (threadIdx.x == 0)
        for (uint32_t u = 0; u < P.stages && u < my_blocks; u++) request_x(u);
    if (prepared == nullptr) {
        load_tables(tab, targs, threadIdx.x, blockDim.x);
        __syncthreads();
        gemm_fast_table(fast, tab, threadIdx.x, blockDim.x);
    } else {
        if (!mbar_wait_bounded(table_bar, 0u) && threadIdx.x == 0) atomicExch(&g_staged_status, 2);
        // fan out: entry v (one word at the tail of the table region) -> kGemmCopies words at 2v; the slots
        // overlap the raw copy, so every thread reads all of its raw entries before anybody writes
        constexpr int kPer = kPairEntries / (NW * 32);
        const uint32_t *raw = fast + (kGemmLutBytes - kPairEntries * 4) / 4;
        uint32_t mine[kPer];
#pragma unroll
        for (int i = 0; i < kPer; i++) mine[i] = raw[threadIdx.x + i * NW * 32];
        __syncthreads();
#pragma unroll
        for (int i = 0; i < kPer; i++)
            *reinterpret_cast<uint2 *>(fast + (threadIdx.x + i * NW * 32) * kGemmCopies) = make_uint2(mine[i], mine[i]);
    }
    __syncthreads();

    // W tile: the lane's word of columns 2l, 2l+1 goes to K-chunk l / 4, the one of columns 64 + 2l to
    // K-chunk 8 + l / 4, row = warp.
    const uint32_t ws0 = P.w_off + (((lane >> 2) * kWLbo + warp) * 4 + (lane & 3)) * 4u;

    int slot = 0;
    uint32_t phases = 0u;
    uint32_t stage = 0u, wraps = 0u;           // position in the stage ring; every warp walks the same sequence
    uint32_t block_no = 0u;                    // blocks this CTA has been through (warp 0 requests X by it)
    uint32_t nset = 0u;                        // sets this CTA has finished
    uint32_t r_cur[4], r_nxt[4];
    bool have_first = false;

    for (int set = first_set; set < nsets; set += gridDim.x, nset++) {
        const uint32_t acc = tmem + (nset & 1u) * kGemmRows;
        for (int kk = 0; kk < L.S; kk++) {
            nxt.valid = false;
            if (cur.valid) {
                if (kk + 1 < L.S) {
                    describe(cur.m, kk + 1, nxt);
                } else {
                    const int s2 = set + gridDim.x;
                    if (s2 < nsets && s2 * kGemmRows + warp < L.M) describe(s2 * kGemmRows + warp, 0, nxt);
                }
            }
            // what `cur` holds of the ring: its staged words, or the decoder state of a direct record
            const uint32_t cur_bytes = cur.staged ? cur.exp_bytes : static_cast<uint32_t>(kDirectState);
            const bool early = nxt.valid && nxt.staged && cur_bytes + nxt.exp_bytes <= ring_bytes;
            if (early) issue(nxt, slot ^ 1);

            const uint32_t *rem = reinterpret_cast<const uint32_t *>(L.rem + (cur.valid ? cur.rec : 0) * L.Nc) + lane;
            const uint32_t *rem_next = reinterpret_cast<const uint32_t *>(L.rem + (nxt.valid ? nxt.rec : 0) * L.Nc) + lane;
            if (!have_first) {
#pragma unroll
                for (int j = 0; j < 4; j++) r_cur[j] = (cur.valid && j < nblk) ? __ldg(rem + j * 32) : 0u;
            }
            Dec dec;
            bool fast_path = false;
            if (cur.valid && cur.staged) {
                fast_path = mbar_wait_bounded(bar0 + 8u * slot, (phases >> slot) & 1u);
                phases ^= 1u << slot;
                if (fast_path) dec.open(smem, cur.base, cur.base + cur.exp_bytes + 256u, lane);
                else if (lane == 0) atomicExch(&g_staged_status, 1);
            }

            auto step = [&](int blk, uint32_t r) {
                const int gblk = kk * nblk + blk;
                uint32_t w0 = 0u, w1 = 0u;
                if (fast_path) {
                    uint32_t e0, e1;
                    dec.pairs(smem, k, tab, lane4, copy_off, e0, e1);
                    dec.clamp();
                    w0 = bitselect(prmt(r, 0u, 0x1100u), e0, kRemMask);
                    w1 = bitselect(prmt(r, 0u, 0x3322u), e1, kRemMask);
                } else if (cur.valid && !cur.staged) {
                    uint32_t *st = reinterpret_cast<uint32_t *>(smem + (slot == 0 ? ring : ring + ring_bytes - kDirectState)) + lane;
                    const uint2 e = direct_block<Codec>(L.exp, L.exp_words, cur.off, lane, blk == 0, st, &tab);
                    w0 = join_pair<0>(r, e.x);
                    w1 = join_pair<1>(r, e.y);
                }

                // the stage is free once the MMAs that read it NS blocks ago have completed
                if (wraps > 0u && !mbar_wait_bounded(empty_bar + 8u * stage, (wraps - 1u) & 1u) && lane == 0)
                    atomicExch(&g_staged_status, 3);
                uint8_t *ws = smem + ws0 + stage * kWTileBytes;
                *reinterpret_cast<uint32_t *>(ws) = w0;
                *reinterpret_cast<uint32_t *>(ws + 8 * kWLbo * 16) = w1;
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(full_bar + 8u * stage);
                // Blocks take turns in who issues: the issuing lane stalls while the tensor pipe works off the
                // previous block, and this spreads that stall over all warps.  The MMAs of block t are issued
                // before those of block t + 1 because their issuer arrives on block t + 1's barrier afterwards.
                if (warp == static_cast<int>(block_no & (kGemmWarps - 1))) {
                    if (lane == 0) {
                        // the stage of the previous block is free as soon as its MMAs are done: refill its X
                        if (block_no >= 1u && block_no - 1u + P.stages < my_blocks) {
                            const uint32_t ps = stage == 0u ? P.stages - 1u : stage - 1u;
                            const uint32_t pw = stage == 0u ? wraps - 1u : wraps;
                            if (!mbar_wait_bounded(empty_bar + 8u * ps, pw & 1u)) atomicExch(&g_staged_status, 6);
                            request_x(block_no - 1u + P.stages);
                        }
                        if (!mbar_wait_bounded(full_bar + 8u * stage, wraps & 1u)) atomicExch(&g_staged_status, 4);
                        tc_fence_after();
                        const uint32_t xt = smem_base + P.x_off + stage * P.x_stage, wt = smem_base + P.w_off + stage * kWTileBytes;
#pragma unroll
                        for (int j = 0; j < 8; j++)
                            umma_bf16(acc, umma_desc_sw128(xt + (j >> 2) * P.x_rows * 128u + (j & 3) * 32u),
                                      umma_desc(wt + j * 2 * kWLbo * 16, kWLbo), kGemmIdesc, (gblk | j) != 0 ? 1u : 0u);
                        umma_commit(empty_bar + 8u * stage);
                        if (kk == L.S - 1 && blk == nblk - 1) umma_commit(done_bar + 8u * (nset & 1u));
                        tc_fence_before();
                    }
                    __syncwarp();
                }
                block_no++;
                if (++stage == P.stages) {
                    stage = 0u;
                    wraps++;
                }
            };

            for (int g0 = 0; g0 < nblk; g0 += 4) {
                const bool last = g0 + 4 >= nblk;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    if (!last) r_nxt[j] = (cur.valid && g0 + 4 + j < nblk) ? __ldg(rem + (g0 + 4 + j) * 32) : 0u;
                    else r_nxt[j] = (nxt.valid && j < nblk) ? __ldg(rem_next + j * 32) : 0u;
                }
#pragma unroll
                for (int j = 0; j < 4; j++)
                    if (g0 + j < nblk) step(g0 + j, r_cur[j]);
#pragma unroll
                for (int j = 0; j < 4; j++) r_cur[j] = r_nxt[j];
            }
            have_first = true;

            __syncwarp();
            if (nxt.valid && nxt.staged && !early) issue(nxt, slot ^ 1);
            cur = nxt;
            slot ^= 1;
        }

        // ---- epilogue of the set: accumulator -> BF16 -> Y[b, set*32 .. set*32+31] --------------------
        // Warps 0..3 own TMEM lanes 32w..32w+31 = batch rows.  The other accumulator is already being
        // filled by the next set; this one is rewritten two sets from now, after these loads (ordered by
        // the warps' later arrivals on the stage barriers).
        if (warp < 4) {
            if (!mbar_wait_bounded(done_bar + 8u * (nset & 1u), (nset >> 1) & 1u) && lane == 0) atomicExch(&g_staged_status, 5);
            tc_fence_after();
            const int b = warp * 32 + lane;
            const int row0 = set * kGemmRows;
#pragma unroll
            for (int c0 = 0; c0 < kGemmRows; c0 += 8) {
                uint32_t v[8];
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                             : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                             : "r"(acc + (static_cast<uint32_t>(warp * 32) << 16) + c0));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (b < B) {
#pragma unroll
                    for (int c = 0; c < 8; c++)
                        if (row0 + c0 + c < L.M) Y[static_cast<int64_t>(b) * L.M + row0 + c0 + c] = f32_to_bf16_rn(__uint_as_float(v[c]));
                }
            }
            tc_fence_before();
        }
    }

    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
}

// Shared-memory plan for a batch: X stages sized by the batch, the rings get what is left.  A 128-row
// MMA reads 16 KB from the start of each atom whatever the batch; the W stages and rings that follow
// the X stages keep that inside the CTA's shared memory.
static GemmPlan gemm_plan(int B) {
    GemmPlan p{};
    p.x_rows = static_cast<uint32_t>((B + 7) & ~7);
    p.x_stage = (2u * p.x_rows * 128u + 1023u) & ~1023u;
    p.stages = kGemmStages;
    const uint32_t room = kSmemMax - kGemmHeader - kSlackBytes - p.stages * (p.x_stage + kWTileBytes);
    p.ring_bytes = (room / kGemmWarps) & ~255u;
    if (p.ring_bytes > kGemmRingMax) p.ring_bytes = kGemmRingMax;
    p.x_off = kGemmHeader;
    p.w_off = p.x_off + p.stages * p.x_stage;
    p.ring_off = p.w_off + ((p.stages * kWTileBytes + 255u) & ~255u);
    p.total = p.ring_off + kGemmWarps * p.ring_bytes + kSlackBytes;
    return p;
}
static_assert(kGemmHeader % 1024 == 0, "X stages must start on a 1024-byte boundary");

// The tensor-map encoder lives in the driver library, which this library does not link: it is
// looked up through the runtime once.
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                   const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

template <class Codec>
static int gemm_launch(const Layer &L, const typename Codec::Args &targs, const uint8_t *prepared, const uint16_t *X,
                       uint16_t *Y, int B, cudaStream_t st) {
    auto kernel = gemm_kernel<Codec>;
    if (int rc = staged_prepare(kernel)) return rc;
    const GemmPlan plan = gemm_plan(B);
    if (plan.total > static_cast<uint32_t>(kSmemMax) || plan.ring_bytes < 1024u) return fail(BHI_ERR_LIMIT, "no shared-memory plan for this batch");
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
    int grid = sm_count();
    const int nsets = (L.M + kGemmRows - 1) / kGemmRows;
    if (grid > nsets) grid = nsets;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kGemmWarps * 32);
    cfg.dynamicSmemBytes = plan.total;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap_launches() ? 1 : 0;
    const uint32_t ans_bits = ans_bits_of(targs);
    const Consts k{ans_bits, (1u << ans_bits) - 1u, 1u, 8u, 4u * kGemmCopies, 65536u};
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, L, targs, prepared, xmap, Y, B, plan, k);
    return e == cudaSuccess ? BHI_OK : cuda_fail(e, "fused tensor-core kernel launch");
}

}  // namespace bhi
