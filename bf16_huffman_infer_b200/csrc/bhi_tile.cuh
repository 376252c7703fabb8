// Fused decode + tensor-core product for up to 128 activation rows (sm_100a: tcgen05.mma, accumulators in tensor memory).
//
// Y[b, m] = sum_c X[b, c] * W[m, c].  The reference decodes W to a dense BF16 scratch in HBM and calls a library GEMM
// (functional.py:405-407, :460-462).  Here W is read once, compressed, and its dense form only ever exists as
// 128-column tiles in shared memory.
//
// Roles.  16 decoder warps each walk R weight rows (R = 2, 3 or 4, chosen per layer by the host), so a CTA holds a SET of
// 16 R rows; one warp issues the MMAs, one requests the X blocks by TMA, four read the accumulators back
// (TMEM -> BF16 -> Y).  No decoder ever waits for the tensor pipe or for an accumulator.
//
// Decoders keep no record in shared memory (128 records would not fit).  A stream is two 32-bit words of look-ahead and
// a bit cursor in registers; when the cursor leaves a word, the next one is loaded straight from global memory (a warp
// reads the 32 streams of a row as one 128-byte line; the load has a whole block time to arrive).  Lane l owns streams l
// and 32 + l of each of its R rows: 2 R independent dependency chains per lane.
//
// MMA shape: the batch is M (A operand = X, 128 rows; rows past the batch are accumulator lanes nobody reads), the set's
// rows are N = 16 R, K advances in blocks of 128 columns (8 instructions of K = 16).  X blocks arrive in the
// 128-byte-swizzled K-major layout; decoded weights are K-major without swizzle, 16-byte units at unit index
// kc * (N + 1) + row, so a warp's stores (one row, 32 lanes = 8 K-chunks x 4 words) are bank-conflict free.  Two
// accumulators of N columns alternate between sets.
//
// What was measured on B200 while building this (one thread issuing back to back, all 148 SMs busy):
//   * a tcgen05.mma of M x N x 16 costs max(52 clocks, N / 2 clocks) whether M is 64 or 128 and whatever the operand
//     layout: 52 is an issue floor, N / 2 the tensor pipe itself.  Anything the issuing thread computes between two
//     instructions adds to the floor: the 8 descriptors of a block are one base plus an add in the low word.
//   * every CTA wants the same X block at about the same time, and its way from L2 takes several block times: X has a ring
//     of its own, deeper than the W ring, fed by its own warp as soon as tcgen05.commit reports a stage free.
//   * with both out of the way the kernel runs at the speed of its decoders: about 86 warp instructions per row and block
//     (the GEMV kernel's four-row layout needs 36) at a third of the issue slots, the rest being global-load latency.
//     That is 0.8 to 1.0 us per block of 32 to 64 rows, against 0.45 us for the same rows in the decode-to-dense kernel,
//     so decode + library GEMM stays ahead (23 / 61 / 63 us against 31 / 62 / 83 us on 4096x4096, 12288x4096, 4096x12288 at
//     16 rows) and remains the default above 8 rows; this path is an option (BHI_TENSOR_ROWS in the host layer).
//
// Barriers (all waits bounded, failures reported through bhi_debug_status):
//   full[s]    16 decoder warps                          -> issuer may multiply W stage s
//   xfull[x]   the X block's bytes                        -> issuer may multiply X stage x
//   empty[s], xempty[x]  tcgen05.commit of a block's MMAs -> decoders may overwrite W[s]; the loader may refill X[x]
//   done[a]    commit after a set's last block            -> epilogue warps read accumulator a
//   free[a]    4 epilogue warps                           -> issuer may start a new set in accumulator a
#pragma once

#include <cuda.h>      // CUtensorMap and the encode entry point's types; the driver library is not linked

#include "bhi_staged.cuh"

namespace bhi {

constexpr int kXAtomCols = 64;                    // columns of one 128-byte swizzle atom

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

constexpr int kTileDecoders = 16;                 // decoder warps
constexpr int kTileIssuer = kTileDecoders;        // warp index of the TMA + MMA issuer
constexpr int kTileEpilogue = kTileDecoders + 1;  // first of four epilogue warps (17..20: TMEM lane quarters 1, 2, 3, 0)
constexpr int kTileLoader = kTileDecoders + 5;    // warp that requests the X blocks
constexpr int kTileWarps = kTileDecoders + 6;
constexpr int kTileThreads = kTileWarps * 32;
constexpr int kTileStagesMax = 8;                 // W stages
constexpr int kTileXStagesMax = 16;               // X stages: the same X block is wanted by every CTA at about the same time, and its
                                                  // way from L2 takes several block times
constexpr int kTileRowsMax = 4;                   // rows per decoder warp (more spill registers)

struct TilePlan {
    uint32_t x_rows;       // batch rounded up to 8: rows of a TMA box
    uint32_t x_stage;      // bytes per X stage (two atoms of x_rows * 128 bytes), a multiple of 1024
    uint32_t w_stage;      // bytes per W stage: 16 K-chunks of (N + 1) 16-byte units
    uint32_t stages;       // W stages
    uint32_t x_stages;
    uint32_t x_off, w_off, total;
    uint32_t tmem_cols;    // power of two >= 2 N
};

// ---- streams in registers ---------------------------------------------------------------------------
// Word i of stream g of a record lives at exp[off + 64 i + g].  `lim` is the last word of the buffer: reads past the
// end of the last record are redirected there (their values are never used).
//
// A stream keeps words i and i + 1 in registers.  When the cursor leaves word i, word i + 2 is loaded, and the line of
// word i + 3 is asked into L1 by a prefetch, which has no destination register: a load kept in flight across
// iterations instead would share its scoreboard with younger loads and make every use of an old value wait for them.
__device__ __forceinline__ void prefetch_l1(const void *p) { asm volatile("prefetch.global.L1 [%0];" ::"l"(p)); }
__device__ __forceinline__ uint32_t ld_keep(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::evict_last.b32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_stream(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.b32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
// try_wait with a suspend-time hint: the hardware may park the warp until the phase completes instead of letting it poll
// through the issue slots the decoders need (measured: 31 against 36 us on a 4096 x 4096 layer).  Bounded.
__device__ __forceinline__ bool mbar_wait_parked(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < (1u << 16); i++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity), "r"(20000u) : "memory");
        if (ok) return true;
    }
    return false;
}

// load `*dst = *p` only where `take` is set (one predicated instruction, no branch)
__device__ __forceinline__ void ld_keep_if(uint32_t &dst, const uint32_t *p, uint32_t take) {
    asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.u32 q, %2, 0;\n\t@q ld.global.nc.L1::evict_last.b32 %0, [%1];\n\t}"
                 : "+r"(dst) : "l"(p), "r"(take));
}

struct HuffReg {
    uint32_t w0, w1, c, ni;      // words i, i + 1 of the stream; c = 32 i + bit position inside w0; ni = index of word i + 2
    __device__ __forceinline__ void open(const uint32_t *exp, uint32_t at, uint32_t lim) {
        w0 = ld_keep(exp + min(at, lim));
        w1 = ld_keep(exp + min(at + 64u, lim));
        ni = at + 128u;
        c = 0u;
    }
    // n <= 32 bits used: at most one word is left behind.  Branch-free: in a warp some lane crosses a word at almost
    // every step.
    __device__ __forceinline__ void advance(const uint32_t *exp, uint32_t, uint32_t lim, uint32_t n) {
        const uint32_t c2 = c + n;
        const uint32_t crossed = (c2 ^ c) & 32u;
        w0 = crossed ? w1 : w0;
        ld_keep_if(w1, exp + min(ni, lim), crossed);
        ni += 2u * crossed;
        c = c2;
    }
    // the two exponents of the next column pair, at bits 7..14 and 23..30
    template <bool kChecked>
    __device__ __forceinline__ uint32_t pair(const uint8_t *smem, const Consts &k, const HuffTables &t, const uint32_t *exp,
                                             uint32_t at, uint32_t lim, uint32_t copy_off) {
        uint32_t win = __funnelshift_r(w0, w1, c);
        uint32_t e = HuffStaged::lookup(smem, k, win, copy_off);
        if (!kChecked || !(e & (kEntSingle | kEntExact))) {
            advance(exp, at, lim, e & kEntBits);
            return e;
        }
        if (e & kEntExact) {
            const uint2 f = huff_exact_symbol(win, &t);
            advance(exp, at, lim, f.y);
            e = f.x << 7;
        } else {
            advance(exp, at, lim, e & kEntBits);
        }
        win = __funnelshift_r(w0, w1, c);
        const uint32_t e2 = HuffStaged::lookup(smem, k, win, copy_off);
        uint32_t s1 = (e2 >> 7) & 0xFFu, l1 = (e2 >> 16) & 15u;
        if (e2 & kEntExact) {
            const uint2 f = huff_exact_symbol(win, &t);
            s1 = f.x;
            l1 = f.y;
        }
        advance(exp, at, lim, l1);
        return (e & 0x7F80u) | (s1 << 23);
    }
};

struct AnsReg {
    uint32_t lo, hi, i;          // state; words taken so far
    __device__ __forceinline__ void open(const uint32_t *exp, uint32_t at, uint32_t lim) {
        lo = ld_keep(exp + min(at, lim));
        prefetch_l1(exp + min(at + 64u, lim));
        hi = 0u;
        i = 0u;
    }
    __device__ __forceinline__ uint32_t symbol(const uint8_t *smem, const Consts &k, const uint32_t *exp, uint32_t at, uint32_t lim,
                                               uint32_t copy_off) {
        if (hi == 0u && lo <= k.ans_mask) {
            i++;
            hi = lo;
            lo = ld_keep(exp + min(at + i * 64u, lim));
            prefetch_l1(exp + min(at + (i + 1u) * 64u, lim));
        }
        const uint32_t e = *reinterpret_cast<const uint32_t *>(smem + umad(lo & k.ans_mask, k.entry, copy_off));
        const uint32_t shifted = __funnelshift_r(lo, hi, k.ans_bits);
        const uint64_t next = static_cast<uint64_t>((e >> 12) & 0xFFFu) * shifted + (e & 0xFFFu);
        lo = static_cast<uint32_t>(next);
        hi = static_cast<uint32_t>(next >> 32);
        return e >> 24;
    }
    template <bool kChecked>
    __device__ __forceinline__ uint32_t pair(const uint8_t *smem, const Consts &k, const AnsTables &, const uint32_t *exp, uint32_t at,
                                             uint32_t lim, uint32_t copy_off) {
        const uint32_t s0 = symbol(smem, k, exp, at, lim, copy_off);
        const uint32_t s1 = symbol(smem, k, exp, at, lim, copy_off);
        return (s0 << 7) | (s1 << 23);
    }
};

template <class Codec> struct RegOf;
template <> struct RegOf<HuffCodec> { using type = HuffReg; };
template <> struct RegOf<AnsCodec> { using type = AnsReg; };

// instruction descriptor: D = F32, A = B = BF16, both K-major, M = 128, N = 16 R
__host__ __device__ constexpr uint32_t tile_idesc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((static_cast<uint32_t>(n) >> 3) << 17) | ((128u >> 4) << 24);
}

template <class Codec, int R>
__global__ void __launch_bounds__(kTileThreads, 1)
tile_kernel(Layer L, typename Codec::Args targs, const uint8_t *prepared, const __grid_constant__ CUtensorMap xmap, uint16_t *Y, int B,
            TilePlan P, Consts k) {
    extern __shared__ __align__(1024) uint8_t smem[];
    using Tables = typename Codec::Tables;
    using Reg = typename RegOf<Codec>::type;
    constexpr int N = kTileDecoders * R;               // weight rows per set
    constexpr uint32_t kLbo = N + 1;                   // 16-byte units between K-chunks of a W stage
    constexpr bool kHuff = std::is_same<Codec, HuffCodec>::value;

    uint32_t *fast = reinterpret_cast<uint32_t *>(smem);
    Tables &tab = *reinterpret_cast<Tables *>(smem + kLutBytes);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kLutBytes + kExactBytes);
    const uint32_t full_bar = smem_addr(&bars[0]);                        // + 8 * W stage
    const uint32_t empty_bar = smem_addr(&bars[kTileStagesMax]);          // + 8 * W stage
    const uint32_t done_bar = smem_addr(&bars[2 * kTileStagesMax]);       // + 8 * accumulator
    const uint32_t free_bar = smem_addr(&bars[2 * kTileStagesMax + 2]);   // + 8 * accumulator
    const uint32_t table_bar = smem_addr(&bars[2 * kTileStagesMax + 4]);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(&bars[2 * kTileStagesMax + 5]);
    const uint32_t xfull_bar = smem_addr(&bars[2 * kTileStagesMax + 6]);                       // + 8 * X stage
    const uint32_t xempty_bar = smem_addr(&bars[2 * kTileStagesMax + 6 + kTileXStagesMax]);    // + 8 * X stage

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const uint32_t smem_base = smem_addr(smem);
    const int nblk = L.Nc >> 7;
    const int nsets = (L.M + N - 1) / N;
    const int first_set = blockIdx.x;
    const uint32_t blocks_per_set = static_cast<uint32_t>(L.S * nblk);
    const uint32_t my_sets = first_set < nsets ? static_cast<uint32_t>((nsets - first_set + gridDim.x - 1) / gridDim.x) : 0u;
    const uint32_t my_blocks = my_sets * blocks_per_set;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < kTileStagesMax; s++) {
            mbar_init(full_bar + 8 * s, kTileDecoders);       // one arrival per decoder warp
            mbar_init(empty_bar + 8 * s, 1);
        }
        for (int s = 0; s < kTileXStagesMax; s++) {
            mbar_init(xfull_bar + 8 * s, 1);                  // the X block (arrival and bytes)
            mbar_init(xempty_bar + 8 * s, 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(done_bar + 8 * a, 1);
            mbar_init(free_bar + 8 * a, 4);
        }
        mbar_init(table_bar, 1);
        mbar_fence_init();
    }
    if (warp == kTileIssuer) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(P.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    if (kHuff && prepared != nullptr && threadIdx.x == 0) {
        mbar_expect_tx(table_bar, kPreparedBytes);
        bulk_copy_g2s(smem_base + kLutBytes - kPairEntries * 4, prepared, kPreparedBytes, table_bar);
    }

    auto request_x = [&](uint32_t u) {               // one thread; the stage must be free
        const uint32_t s = u % P.x_stages;
        const uint32_t bar = xfull_bar + 8u * s;
        const uint32_t dst = smem_base + P.x_off + s * P.x_stage;
        const int col = static_cast<int>(u % blocks_per_set) * 128;
        mbar_expect_tx(bar, 2u * P.x_rows * 128u);
        tma_load_2d(dst, &xmap, col, 0, bar);
        tma_load_2d(dst + P.x_rows * 128u, &xmap, col + kXAtomCols, 0, bar);
    };

    pdl_wait();
    if (warp == kTileLoader && lane == 0)
        for (uint32_t u = 0; u < P.x_stages && u < my_blocks; u++) request_x(u);

    // ---- tables: every warp helps, then the roles part -------------------------------------------------
    uint32_t flagged = 1u;            // entries of the folded table that do not resolve two symbols (unknown: assume some)
    if (!kHuff || prepared == nullptr) {
        load_tables(tab, targs, threadIdx.x, blockDim.x);
        __syncthreads();
        build_fast_table(fast, tab, threadIdx.x, blockDim.x);
    } else {
        if (!mbar_wait_bounded(table_bar, 0u) && threadIdx.x == 0) atomicExch(&g_staged_status, 2);
        flagged = prepared_flagged(smem + kLutBytes);
        // fan out: entry v (one word at the tail of the table region) -> kCopies words at pair_slot(v); the slots overlap
        // the raw copy, so every thread reads all of its raw entries before anybody writes
        constexpr int kPer = (kPairEntries + kTileThreads - 1) / kTileThreads;
        const uint32_t *raw = fast + (kLutBytes - kPairEntries * 4) / 4;
        uint32_t mine[kPer];
#pragma unroll
        for (int i = 0; i < kPer; i++) {
            const int v = threadIdx.x + i * kTileThreads;
            mine[i] = v < kPairEntries ? raw[v] : 0u;
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < kPer; i++) {
            const int v = threadIdx.x + i * kTileThreads;
            if (v < kPairEntries) *reinterpret_cast<uint4 *>(fast + pair_slot(v)) = make_uint4(mine[i], mine[i], mine[i], mine[i]);
        }
    }
    __syncthreads();

    if (warp < kTileDecoders) {
        // ---- decoders: R rows per warp, lane l owns streams l and 32 + l of each ---------------------------
        const uint32_t copy_off = 4u * (lane & (kCopies - 1));
        const uint32_t lim = static_cast<uint32_t>(L.exp_words - 1);
        // W stage: row n = warp * R + j; the lane's word of columns 2l, 2l+1 goes to K-chunk l / 4, the one of columns
        // 64 + 2l to K-chunk 8 + l / 4
        const uint32_t ws0 = P.w_off + (((lane >> 2) * kLbo + warp * R) * 4 + (lane & 3)) * 4u;
        auto decode_sets = [&](auto checked) {
        constexpr bool kChecked = decltype(checked)::value;
        uint32_t stage = 0u, wraps = 0u;           // position in the stage ring; every warp and the issuer walk the same sequence
        for (int set = first_set; set < nsets; set += gridDim.x) {
            for (int kk = 0; kk < L.S; kk++) {
                Reg s0[R], s1[R];
                uint32_t at[R], r_cur[R], r_nxt[R];
                const uint32_t *rem32 = reinterpret_cast<const uint32_t *>(L.rem) + lane;
                uint32_t rem[R];                       // word index of the row's sign/mantissa bytes
#pragma unroll
                for (int j = 0; j < R; j++) {
                    // rows past the end of the matrix decode the last row again; nobody reads their products
                    const int m = min(set * N + warp * R + j, L.M - 1);
                    const int64_t rec = static_cast<int64_t>(kk) * L.M + m;
                    at[j] = static_cast<uint32_t>(__ldg(L.offsets + rec)) + lane;
                    rem[j] = static_cast<uint32_t>((rec * L.Nc) >> 2);
                }
#pragma unroll
                for (int j = 0; j < R; j++) {
                    s0[j].open(L.exp, at[j], lim);
                    s1[j].open(L.exp, at[j] + 32u, lim);
                    r_cur[j] = ld_stream(rem32 + rem[j]);
                }
                for (int blk = 0; blk < nblk; blk++) {
#pragma unroll
                    for (int j = 0; j < R; j++) r_nxt[j] = blk + 1 < nblk ? ld_stream(rem32 + rem[j] + (blk + 1) * 32) : 0u;
                    // the stage is free once the MMAs that read it `stages` blocks ago have completed
                    if (wraps > 0u && !mbar_wait_parked(empty_bar + 8u * stage, (wraps - 1u) & 1u) && lane == 0)
                        atomicExch(&g_staged_status, 3);
                    uint8_t *ws = smem + ws0 + stage * P.w_stage;
#pragma unroll
                    for (int j = 0; j < R; j++) {
                        const uint32_t e0 = s0[j].template pair<kChecked>(smem, k, tab, L.exp, at[j], lim, copy_off);
                        const uint32_t e1 = s1[j].template pair<kChecked>(smem, k, tab, L.exp, at[j] + 32u, lim, copy_off);
                        *reinterpret_cast<uint32_t *>(ws + j * 16) = bitselect(prmt(r_cur[j], 0u, 0x1100u), e0, kRemMask);
                        *reinterpret_cast<uint32_t *>(ws + j * 16 + 8 * kLbo * 16) = bitselect(prmt(r_cur[j], 0u, 0x3322u), e1, kRemMask);
                    }
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(full_bar + 8u * stage);
                    if (++stage == P.stages) {
                        stage = 0u;
                        wraps++;
                    }
#pragma unroll
                    for (int j = 0; j < R; j++) r_cur[j] = r_nxt[j];
                }
            }
        }
        };
        if (kHuff && flagged == 0u) decode_sets(std::false_type{});
        else decode_sets(std::true_type{});
    } else if (warp == kTileIssuer) {
        // ---- issuer: X blocks by TMA, 8 MMAs per block ---------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t kIdesc = tile_idesc(N);
            uint32_t u = 0u;
            for (uint32_t nset = 0; nset < my_sets; nset++) {
                const uint32_t a = nset & 1u;
                const uint32_t acc = tmem + a * N;
                if (nset >= 2u && !mbar_wait_parked(free_bar + 8u * a, ((nset >> 1) - 1u) & 1u)) atomicExch(&g_staged_status, 7);
                for (uint32_t b = 0; b < blocks_per_set; b++, u++) {
                    const uint32_t s = u % P.stages, wr = u / P.stages, xs = u % P.x_stages, xwr = u / P.x_stages;
                    if (!mbar_wait_parked(xfull_bar + 8u * xs, xwr & 1u)) atomicExch(&g_staged_status, 8);
                    if (!mbar_wait_parked(full_bar + 8u * s, wr & 1u)) atomicExch(&g_staged_status, 4);
                    tc_fence_after();
                    const uint32_t xt = smem_base + P.x_off + xs * P.x_stage, wt = smem_base + P.w_off + s * P.w_stage;
                    // descriptors of the 8 K-steps differ in the address field (low word) only: one add each
                    const uint64_t xd0 = umma_desc_sw128(xt), xd1 = umma_desc_sw128(xt + P.x_rows * 128u), wd = umma_desc(wt, kLbo);
#pragma unroll
                    for (int j = 0; j < 8; j++)
                        umma_bf16(acc, ((j >> 2) ? xd1 : xd0) + static_cast<uint64_t>((j & 3) * 2), wd + static_cast<uint64_t>(j * 2 * kLbo),
                                  kIdesc, (b | static_cast<uint32_t>(j)) != 0u ? 1u : 0u);
                    umma_commit(empty_bar + 8u * s);
                    umma_commit(xempty_bar + 8u * xs);
                    if (b + 1u == blocks_per_set) umma_commit(done_bar + 8u * a);
                }
            }
            tc_fence_before();
        }
        __syncwarp();
    } else if (warp == kTileLoader) {
        // ---- loader: X block u + x_stages as soon as the MMAs of block u are done ----------------------------------------
        if (lane == 0) {
            for (uint32_t u = 0; u + P.x_stages < my_blocks; u++) {
                if (!mbar_wait_parked(xempty_bar + 8u * (u % P.x_stages), (u / P.x_stages) & 1u)) atomicExch(&g_staged_status, 6);
                request_x(u + P.x_stages);
            }
        }
        __syncwarp();
    } else {
        // ---- epilogue: accumulator -> BF16 -> Y[b, set * N ..] ------------------------------------------------------
        const uint32_t q = static_cast<uint32_t>(warp) & 3u;      // the TMEM lane quarter this warp may read
        const int b = static_cast<int>(q) * 32 + lane;
        for (uint32_t nset = 0; nset < my_sets; nset++) {
            const uint32_t a = nset & 1u;
            const uint32_t acc = tmem + a * N;
            const int row0 = (first_set + static_cast<int>(nset) * static_cast<int>(gridDim.x)) * N;
            if (!mbar_wait_parked(done_bar + 8u * a, (nset >> 1) & 1u) && lane == 0) atomicExch(&g_staged_status, 5);
            tc_fence_after();
            if (static_cast<int>(q) * 32 < B) {
#pragma unroll
                for (int c0 = 0; c0 < N; c0 += 8) {
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
    if (warp == kTileIssuer) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(P.tmem_cols) : "memory");
}

// ---- host side ---------------------------------------------------------------------------------------
static bool tile_plan(int B, int rows_per_warp, TilePlan &p) {
    const uint32_t n = static_cast<uint32_t>(kTileDecoders * rows_per_warp);
    p.x_rows = static_cast<uint32_t>((B + 7) & ~7);
    p.x_stage = (2u * p.x_rows * 128u + 1023u) & ~1023u;
    p.w_stage = 16u * (n + 1u) * 16u;
    const uint32_t header = kLutBytes + kExactBytes + kCtrlBytes;
    // a 128-row MMA reads 16 KB from the start of each X atom whatever the batch: keep that inside the allocation
    const uint32_t tail = 16u * 1024u;
    const uint32_t room = static_cast<uint32_t>(kSmemMax) - header - tail;
    if (room < 2u * (p.x_stage + p.w_stage)) return false;
    // three W stages when they fit beside at least three X stages; X takes the rest
    p.stages = room >= 3u * (p.x_stage + p.w_stage) ? 3u : 2u;
    p.x_stages = (room - p.stages * p.w_stage) / p.x_stage;
    if (p.x_stages > kTileXStagesMax) p.x_stages = kTileXStagesMax;
    p.x_off = header;
    p.w_off = p.x_off + p.x_stages * p.x_stage;
    p.total = p.w_off + p.stages * p.w_stage + tail;
    p.tmem_cols = 32u;
    while (p.tmem_cols < 2u * n) p.tmem_cols <<= 1;
    return p.total <= static_cast<uint32_t>(kSmemMax);
}
static_assert((kLutBytes + kExactBytes + kCtrlBytes) % 1024 == 0, "X stages must start on a 1024-byte boundary");
static_assert((2 * kTileStagesMax + 6 + 2 * kTileXStagesMax) * 8 <= kCtrlBytes, "control block too small");

// Rows per decoder warp for a layer: the fewest waves times the measured time of one 128-column block (0.81 / 0.88 /
// 1.04 us for 2 / 3 / 4 rows per warp on B200; more rows per warp spill registers).
static int tile_rows_per_warp(const Layer &L, int grid) {
    static const struct { int rows; double us; } kChoices[] = {{2, 0.81}, {3, 0.88}, {4, 1.04}};
    int best = 2;
    double best_cost = 1e30;
    for (const auto &c : kChoices) {
        const int nsets = (L.M + kTileDecoders * c.rows - 1) / (kTileDecoders * c.rows);
        const int waves = (nsets + grid - 1) / grid;
        if (waves * c.us < best_cost - 1e-9) {
            best_cost = waves * c.us;
            best = c.rows;
        }
    }
    return best;
}

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

template <class Codec, int R>
static int tile_launch_r(const Layer &L, const typename Codec::Args &targs, const uint8_t *prepared, const CUtensorMap &xmap,
                         uint16_t *Y, int B, const TilePlan &plan, cudaStream_t st) {
    auto kernel = tile_kernel<Codec, R>;
    if (int rc = staged_prepare(kernel)) return rc;
    int grid = sm_count();
    const int nsets = (L.M + kTileDecoders * R - 1) / (kTileDecoders * R);
    if (grid > nsets) grid = nsets;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kTileThreads);
    cfg.dynamicSmemBytes = plan.total;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap_launches() ? 1 : 0;
    const uint32_t ans_bits = ans_bits_of(targs);
    const Consts k{ans_bits, (1u << ans_bits) - 1u, 1u, 8u, 4u * kCopies, 65536u};
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, L, targs, prepared, xmap, Y, B, plan, k);
    return e == cudaSuccess ? BHI_OK : cuda_fail(e, "fused tensor-core kernel launch");
}

template <class Codec>
static int tile_launch(const Layer &L, const typename Codec::Args &targs, const uint8_t *prepared, const uint16_t *X, uint16_t *Y,
                       int B, cudaStream_t st) {
    const int r = tile_rows_per_warp(L, sm_count());
    TilePlan plan{};
    if (!tile_plan(B, r, plan)) return fail(BHI_ERR_LIMIT, "no shared-memory plan for this batch");
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
    switch (r) {
    case 2: return tile_launch_r<Codec, 2>(L, targs, prepared, xmap, Y, B, plan, st);
    case 3: return tile_launch_r<Codec, 3>(L, targs, prepared, xmap, Y, B, plan, st);
    default: return tile_launch_r<Codec, 4>(L, targs, prepared, xmap, Y, B, plan, st);
    }
}

}  // namespace bhi
