// Fused decode + GEMV for 1..8 rows of X, "quad" mapping (sm_100a).
//
// Work mapping.  A *quad* is four consecutive weight rows.  A group of four warps owns one quad at a
// time; warp j of the group (its *pass*) decodes streams 8j..8j+7 and 32+8j..32+8j+7 of all four
// rows: lane (r = lane/8, s = (lane/4)%2, t = lane%4) runs the two streams sigma = 8j + 4s + t and
// sigma + 32 of row r.  Per 128-column block a lane therefore rebuilds two bf16x2 words, exactly the
// B fragment of one mma.sync.m16n8k16 whose eight columns n = lane/4 are (row r, half s): the tile
// is dense over the four weight rows, and its sixteen A rows are (half s, batch row b), b = 0..7.
// One tensor-core instruction per block thus serves EVERY batch row; the products of mismatched
// halves (c1, c2) are discarded and c0 + c3 of lane (b, t) is the dot product of batch row b with
// weight row t of the quad.  The cost of a launch is (almost) independent of the batch.
//
// Exponent records: the four records of a (quad, chunk) unit are brought into the group's ring by
// four bulk async copies on one mbarrier, one unit ahead, each record shifted by 32 bytes against
// the previous one so that the 32 lanes of a warp (4 rows x 8 streams) read 32 different banks.
//
// Huffman decoding: a stream is a bit cursor.  One 32-bit window fetched under the cursor serves TWO
// lookups of the folded pair table (two blocks, four symbols): the table index is taken from the
// window with a single logic instruction (the cursor runs a few bits behind the stream position so
// that the index is already scaled by the entry stride), the window is shifted by the bits the
// first entry used, and the cursor advances by the sum.  Windows a 12-bit index cannot resolve as
// two symbols are flagged in the entry; the warp then re-decodes those streams symbol by symbol
// out of line.  A table without any flagged entry (all codes <= 6 bits) selects a loop without the
// test.  rANS decoding follows the reference's state update, refills from the ring.
//
// X is staged in shared memory as ready-made A fragments (one 16-byte load per lane and block).
// When batch x K does not fit, the K-chunks are processed in stages with X restaged in between and
// per-quad partial sums parked in shared memory.
//
// Results: the four warps of a group add their partial sums through shared memory in pass order
// (deterministic).  Row-sharded layers stage their results and store them into every rank's output
// with coalesced peer stores at the end of the kernel (see ExchangeSink for the protocol).
#pragma once

#include "bhi_staged.cuh"

namespace bhi {

constexpr int kQuadGroups = 8;                                 // warp groups per CTA, one quad each at a time
constexpr int kQuadCtrlBytes = 1024;                           // mbarriers
constexpr int kQuadPartBytes = kQuadGroups * 2 * 4 * 32 * 4;   // [group][parity][warp of the group][lane] partial sums
constexpr uint32_t kQuadRingWant = 59u * 256u;                 // per group: two units of four 7-row records
constexpr uint32_t kQuadRingLeast = 8u * 1024u;                // below this the shape is declined
constexpr uint32_t kEntFlags = kEntSingle | kEntExact;

struct QuadGeom {
    uint32_t lut_bytes;        // fast table region (copies * one table)
    uint32_t copy_shift;       // log2(bytes between consecutive table entries) = 2 + log2(copies)
    uint32_t index_mask;       // table index bits, already at their place in a biased window
    uint32_t part_off, acc_off, ys_off, x_off, ring_off;
    uint32_t x_bytes;          // one stage of X
    uint32_t ring_bytes;       // per group
    int chunks_per_stage;
    int stages;
};

__device__ __forceinline__ uint32_t lds32(const uint8_t *smem, uint32_t a) { return *reinterpret_cast<const uint32_t *>(smem + a); }

// barrier among the warps of one group: hardware barrier group + 1 (0 is the CTA-wide one).  Literal
// barrier numbers, so that the kernel reserves nine barriers and not all sixteen.
__device__ __forceinline__ void group_barrier(int group, int threads) {
#define BHI_GROUP_BAR(g) \
    case g: asm volatile("bar.sync " #g " + 1, %0;" ::"r"(threads) : "memory"); break;
    switch (group) {
        BHI_GROUP_BAR(0) BHI_GROUP_BAR(1) BHI_GROUP_BAR(2) BHI_GROUP_BAR(3)
        BHI_GROUP_BAR(4) BHI_GROUP_BAR(5) BHI_GROUP_BAR(6) BHI_GROUP_BAR(7)
    }
#undef BHI_GROUP_BAR
}

// ---- Huffman, symbol by symbol (rare windows) --------------------------------------------------------
// Decodes the next four symbols of one stream with first-symbol lookups (and the exact cascade for
// codes longer than the table index).  `p` is the true bit cursor.  Returns the two entry words
// {block A, block B} with the exponents at bits 7..14 and 23..30.  Inlined: as a call it cost a
// quarter more on tables where a few percent of the windows need it.
__device__ __forceinline__ uint2 quad_huff_slow(uint32_t p, uint32_t off, uint32_t plim, uint32_t copy_shift, uint32_t lut_bytes,
                                             uint32_t *p_out) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const HuffTables &t = *reinterpret_cast<const HuffTables *>(smem + lut_bytes);
    uint32_t sym[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t a = ((p >> 5) << 8) + off;
        const uint32_t win = __funnelshift_r(lds32(smem, a), lds32(smem, a + 256), p);
        const uint32_t e = lds32(smem, (win & (kPairEntries - 1)) << copy_shift);
        uint32_t s = (e >> 7) & 0xFFu, l = (e >> 16) & 15u;
        if (e & kEntExact) {
            s = huff_cascade(t, win);
            l = t.len[s];
        }
        sym[i] = s;
        p = min(p + l, plim);
    }
    *p_out = p;
    return make_uint2((sym[0] << 7) | (sym[1] << 23), (sym[2] << 7) | (sym[3] << 23));
}

// Per-lane decoder state over the group's ring.  Interface shared by both coders:
//   open(base, sigma4, rows)  - record of this lane's row at byte `base`, `rows` word rows long
//   two<kChecked>(eA0, eA1, eB0, eB1) - entry words of the next two blocks (streams sigma, sigma+32)
//   clamp()
struct QuadCtx {
    const uint8_t *smem;
    Consts k;
    uint32_t copy_off, index_mask, bias, copy_shift, lut_bytes;
};

struct QuadHuff {
    uint32_t p0, p1, plim, off;          // cursors run `bias` bits behind the stream position
    __device__ __forceinline__ void open(const QuadCtx &c, uint32_t base, uint32_t sigma4, uint32_t rows) {
        off = (base & 255u) + sigma4;
        p0 = p1 = (base >> 8) * 32u - c.bias;
        plim = p0 + 32u * (rows + 1u);
    }
    static __device__ __forceinline__ uint32_t window(const QuadCtx &c, uint32_t p, uint32_t o) {
        const uint32_t a = umad(p & ~31u, c.k.eight, o);
        return __funnelshift_r(lds32(c.smem, a), lds32(c.smem, a + 256u), p);
    }
    static __device__ __forceinline__ uint32_t lookup(const QuadCtx &c, uint32_t win) {
        return lds32(c.smem, (win & c.index_mask) | c.copy_off);
    }
    template <bool kChecked>
    __device__ __forceinline__ void two(const QuadCtx &c, uint32_t &eA0, uint32_t &eA1, uint32_t &eB0, uint32_t &eB1) {
        const uint32_t q0 = p0, q1 = p1;
        const uint32_t w0 = window(c, p0, off);
        const uint32_t w1 = window(c, p1, off + 128u);
        eA0 = lookup(c, w0);
        eA1 = lookup(c, w1);
        eB0 = lookup(c, __funnelshift_r(w0, 0u, eA0));       // shift count = low five bits = bits used by A
        eB1 = lookup(c, __funnelshift_r(w1, 0u, eA1));
        p0 += (eA0 + eB0) & 31u;
        p1 += (eA1 + eB1) & 31u;
        if (kChecked) {
            if ((eA0 | eB0 | eA1 | eB1) & kEntFlags) {
                if ((eA0 | eB0) & kEntFlags) {
                    uint32_t p;
                    const uint2 f = quad_huff_slow(q0 + c.bias, off, plim + c.bias, c.copy_shift, c.lut_bytes, &p);
                    eA0 = f.x;
                    eB0 = f.y;
                    p0 = p - c.bias;
                }
                if ((eA1 | eB1) & kEntFlags) {
                    uint32_t p;
                    const uint2 f = quad_huff_slow(q1 + c.bias, off + 128u, plim + c.bias, c.copy_shift, c.lut_bytes, &p);
                    eA1 = f.x;
                    eB1 = f.y;
                    p1 = p - c.bias;
                }
            }
        }
    }
    __device__ __forceinline__ void clamp() {
        p0 = min(p0, plim);
        p1 = min(p1, plim);
    }
};

struct QuadAnsLane {
    uint32_t lo, hi, nx;
    __device__ __forceinline__ uint32_t symbol(const QuadCtx &c, uint32_t alim) {
        if (hi == 0 && lo <= c.k.ans_mask) {
            hi = lo;
            lo = lds32(c.smem, nx);
            nx = min(nx + 256u, alim);
        }
        const uint32_t e = lds32(c.smem, ((lo << c.copy_shift) & c.index_mask) | c.copy_off);
        const uint32_t shifted = __funnelshift_r(lo, hi, c.k.ans_bits);
        const uint64_t next = static_cast<uint64_t>((e >> 12) & 0xFFFu) * shifted + (e & 0xFFFu);
        lo = static_cast<uint32_t>(next);
        hi = static_cast<uint32_t>(next >> 32);
        return e >> 24;
    }
};

struct QuadAns {
    QuadAnsLane a0, a1;
    uint32_t alim;
    __device__ __forceinline__ void open(const QuadCtx &c, uint32_t base, uint32_t sigma4, uint32_t rows) {
        const uint32_t p = base + sigma4;
        a0.lo = lds32(c.smem, p);
        a1.lo = lds32(c.smem, p + 128u);
        a0.hi = a1.hi = 0;
        a0.nx = p + 256u;
        a1.nx = p + 128u + 256u;
        alim = p + rows * 256u;
    }
    template <bool>
    __device__ __forceinline__ void two(const QuadCtx &c, uint32_t &eA0, uint32_t &eA1, uint32_t &eB0, uint32_t &eB1) {
        const uint32_t s00 = a0.symbol(c, alim), s10 = a1.symbol(c, alim + 128u);
        const uint32_t s01 = a0.symbol(c, alim), s11 = a1.symbol(c, alim + 128u);
        const uint32_t s02 = a0.symbol(c, alim), s12 = a1.symbol(c, alim + 128u);
        const uint32_t s03 = a0.symbol(c, alim), s13 = a1.symbol(c, alim + 128u);
        eA0 = (s00 << 7) | (s01 << 23);
        eA1 = (s10 << 7) | (s11 << 23);
        eB0 = (s02 << 7) | (s03 << 23);
        eB1 = (s12 << 7) | (s13 << 23);
    }
    __device__ __forceinline__ void clamp() {}
};

template <class Codec> struct QuadOf;
template <> struct QuadOf<HuffCodec> { using type = QuadHuff; };
template <> struct QuadOf<AnsCodec> { using type = QuadAns; };

// number of flagged entries of the folded table (0 = every 12-bit window resolves two symbols)
__device__ __forceinline__ uint32_t prepared_flagged(const uint8_t *exact_region) {
    return *reinterpret_cast<const uint32_t *>(exact_region + sizeof(HuffTables));
}

struct QuadUnit {
    int qi, k;              // quad index inside the CTA, chunk
    int rec;                // this lane's row: record index (chunk * M + row)
    uint32_t off;           // this lane's row: first exponent word
    uint32_t bytes;         // this lane's row: staged bytes
    uint32_t rows;          // word rows of the longest of the four records
    uint32_t base;          // byte offset of the unit in shared memory
    bool valid, staged;
    __device__ __forceinline__ uint32_t stride() const { return rows * 256u + 32u; }      // bytes between the four records
    __device__ __forceinline__ uint32_t foot() const { return rows * 1024u + 128u; }      // bytes of the unit in the ring
};

// PPW = passes per warp: 1 (four warps per group, 32 warps) or 2 (two warps per group, 16 warps of twice the registers).
template <class Codec, int B, int PPW>
__global__ void __launch_bounds__(kQuadGroups * (4 / PPW) * 32, 1)
quad_kernel(Layer L, typename Codec::Args targs, const uint8_t *prepared, const uint32_t *X, uint16_t *Y, PeerSet peers,
            QuadGeom G, Consts kc) {
    extern __shared__ __align__(1024) uint8_t smem[];
    using Tables = typename Codec::Tables;
    using Dec = typename QuadOf<Codec>::type;
    constexpr bool kHuff = std::is_same<Codec, HuffCodec>::value;
    constexpr int kWG = 4 / PPW;                       // warps per group
    constexpr int kThreads = kQuadGroups * kWG * 32;
    constexpr int kRG = 4;                           // blocks per sign/mantissa prefetch group

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int group = warp / kWG, wig = warp % kWG;    // warp inside the group; its passes are wig * PPW + 0..PPW-1
    const int r = lane >> 3, t = lane & 3, gq = lane >> 2;
    const uint32_t sigma4 = 4u * (8 * (wig * PPW) + (lane & 7));   // byte offset of the first pass's stream inside a word row
    const bool exchange = peers.world > 0;

    uint32_t *fast = reinterpret_cast<uint32_t *>(smem);
    Tables &tab = *reinterpret_cast<Tables *>(smem + G.lut_bytes);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + G.lut_bytes + kExactBytes);
    const uint32_t smem_base = smem_addr(smem);
    const uint32_t bar0 = smem_addr(&bars[2 * group]);
    const uint32_t table_bar = smem_addr(&bars[2 * kQuadGroups]);
    float *part = reinterpret_cast<float *>(smem + G.part_off) + group * 256;
    float *acc = reinterpret_cast<float *>(smem + G.acc_off);
    uint16_t *ys = reinterpret_cast<uint16_t *>(smem + G.ys_off);
    const uint4 *xs = reinterpret_cast<const uint4 *>(smem + G.x_off);
    const uint32_t ring = G.ring_off + group * G.ring_bytes;

    QuadCtx ctx;
    ctx.smem = smem;
    ctx.k = kc;
    ctx.copy_shift = G.copy_shift;
    ctx.copy_off = 4u * (lane & ((1u << (G.copy_shift - 2)) - 1u));
    ctx.index_mask = G.index_mask;
    ctx.bias = kHuff ? G.copy_shift : 0u;
    ctx.lut_bytes = G.lut_bytes;

    const int nquads = (L.M + 3) >> 2;
    const int q_lo = static_cast<int>(static_cast<int64_t>(nquads) * blockIdx.x / gridDim.x);
    const int q_hi = static_cast<int>(static_cast<int64_t>(nquads) * (blockIdx.x + 1) / gridDim.x);
    const int nq = q_hi - q_lo;
    const int row_lo = 4 * q_lo;
    const int rows_cta = min(4 * q_hi, L.M) - row_lo;
    const int nrec = L.S * L.M;
    const int nblk = L.Nc >> 7;
    const int nc4 = L.Nc >> 2;

    pdl_launch_dependents();
    if (tid == 0) mbar_init(table_bar, 1);
    if (wig == 0 && lane == 0) {
        mbar_init(bar0, 1);
        mbar_init(bar0 + 8, 1);
    }
    if (lane == 0) mbar_fence_init();
    __syncthreads();
    if (prepared != nullptr && tid == 0) {
        // one copy of the folded table lands at the tail of the table region, the exact tables behind it
        mbar_expect_tx(table_bar, kPreparedBytes);
        bulk_copy_g2s(smem_base + G.lut_bytes - kPairEntries * 4, prepared, kPreparedBytes, table_bar);
    }

    auto describe = [&](int qi, int k, QuadUnit &u) {
        u.qi = qi;
        u.k = k;
        const int m = min(4 * (q_lo + qi) + r, L.M - 1);
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
    // the leader warp of the group starts the four record copies of a unit
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

    // units of this group inside a stage: quads group, group + 8, ... ; for each, the chunks of the stage in order
    int k_lo = 0, k_hi = min(L.S, G.chunks_per_stage);
    auto first_unit = [&](QuadUnit &u) {
        u.valid = false;
        if (group < nq) describe(group, k_lo, u);
    };
    auto next_unit = [&](const QuadUnit &c, QuadUnit &u) {
        u.valid = false;
        if (c.k + 1 < k_hi) describe(c.qi, c.k + 1, u);
        else if (c.qi + kQuadGroups < nq) describe(c.qi + kQuadGroups, k_lo, u);
    };

    QuadUnit cur, nxt;
    first_unit(cur);
    if (cur.valid && cur.staged) issue(cur, 0);
    else if (cur.valid) place(cur, 0);

    // Everything above read weights only and is in flight (record copies, table copy).  X (and Y) belong to the
    // previous kernel in the stream: wait for it here, and fetch the first stage of X while the tables arrive.
    pdl_wait();
    uint32_t launch_no = 0;
    if (exchange) {
        launch_no = *reinterpret_cast<const volatile uint32_t *>(peers.launches) + 1u;
        if (blockIdx.x == 0 && tid < peers.world) red_release_sys_add(pick(peers.ready, tid), 1u);
    }

    const int64_t row_pairs = (static_cast<int64_t>(L.S) * L.Nc) >> 1;
    auto stage_x = [&]() {
        // A fragments: [block][pass][batch row][t] -> {pair 8j+t, pair 8j+4+t, pair 32+8j+t, pair 32+8j+4+t} of the block
        uint4 *dst = reinterpret_cast<uint4 *>(smem + G.x_off);
        const int total = (k_hi - k_lo) * nblk * 16 * B;
        for (int i = tid; i < total; i += kThreads) {
            const int tt = i & 3, rest = i >> 2;
            const int b = rest % B, rest2 = rest / B;
            const int j = rest2 & 3, gb = rest2 >> 2;
            const uint32_t *s = X + b * row_pairs + (static_cast<int64_t>(k_lo) * nblk + gb) * 64 + 8 * j + tt;
            dst[i] = make_uint4(__ldg(s), __ldg(s + 4), __ldg(s + 32), __ldg(s + 36));
        }
    };
    stage_x();

    // tables (their copy was started before the wait above)
    uint32_t flagged = 1u;
    const uint32_t copies = 1u << (G.copy_shift - 2);
    if (prepared == nullptr) {
        load_tables(tab, targs, tid, kThreads);
        __syncthreads();
        if constexpr (kHuff) {
            for (int v = tid; v < kPairEntries; v += kThreads) {
                const uint32_t e = pair_entry(tab, v);
                for (uint32_t c = 0; c < copies; c++) fast[v * copies + c] = e;
            }
        } else {
            for (int v = tid; v < (1 << kc.ans_bits); v += kThreads) {
                const uint32_t e = __ldg(targs.lut + v);
                for (uint32_t c = 0; c < copies; c++) fast[v * copies + c] = e;
            }
        }
    } else {
        if (!mbar_wait_bounded(table_bar, 0u) && tid == 0) atomicExch(&g_staged_status, 2);
        flagged = prepared_flagged(smem + G.lut_bytes);
        if (copies > 1) {
            // fan out: entry v (one word at the tail of the region) -> `copies` words at v * copies.  The
            // targets overlap the raw copy, so every thread reads its raw entries before anybody writes.
            constexpr int kPer = kPairEntries / kThreads;
            const uint32_t *raw = fast + (G.lut_bytes - kPairEntries * 4) / 4;
            uint32_t mine[kPer];
#pragma unroll
            for (int i = 0; i < kPer; i++) mine[i] = raw[tid + i * kThreads];
            __syncthreads();
#pragma unroll
            for (int i = 0; i < kPer; i++)
                for (uint32_t c = 0; c < copies; c++) fast[(tid + i * kThreads) * copies + c] = mine[i];
        }
    }
    const bool checked = kHuff && flagged != 0u;

    float c[PPW][4];
#pragma unroll
    for (int pp = 0; pp < PPW; pp++) c[pp][0] = c[pp][1] = c[pp][2] = c[pp][3] = 0.f;
    uint32_t phases = 0u, parity = 0u;
    int slot = 0;
    const int gqx = gq < B ? gq : B - 1;      // lanes of unused batch rows read a used row (their products are discarded)

    for (int stage = 0; stage < G.stages; stage++) {
        if (stage > 0) {
            __syncthreads();                  // everybody is done with the previous stage of X
            k_lo = k_hi;
            k_hi = min(L.S, k_lo + G.chunks_per_stage);
            first_unit(cur);
            if (cur.valid && cur.staged) issue(cur, slot);
            else if (cur.valid) place(cur, slot);
        }
        if (stage > 0) stage_x();
        __syncthreads();

        uint32_t r_cur[PPW][kRG], r_nxt[PPW][kRG];
        bool have_first = false;

        while (cur.valid) {
            next_unit(cur, nxt);
            const bool early = nxt.valid && nxt.staged && (!cur.staged || cur.foot() + nxt.foot() <= G.ring_bytes);
            if (early) issue(nxt, slot ^ 1);

            // pass pp of this warp: streams at sigma4 + 32 * pp bytes, sign/mantissa words 8 * pp further, A fragments B * 4 further
            const uint32_t *rem = reinterpret_cast<const uint32_t *>(L.rem) + static_cast<int64_t>(cur.rec) * nc4 + (sigma4 >> 2);
            const uint32_t *rem_next =
                nxt.valid ? reinterpret_cast<const uint32_t *>(L.rem) + static_cast<int64_t>(nxt.rec) * nc4 + (sigma4 >> 2) : rem;
            const uint4 *xq = xs + (static_cast<int64_t>(cur.k - k_lo) * nblk * 4 + wig * PPW) * (B * 4) + gqx * 4 + t;
            bool next_first = false;

            auto mac = [&](int pp, int blk, uint32_t rw, uint32_t e0, uint32_t e1) {
                uint4 a = make_uint4(0u, 0u, 0u, 0u);
                if (B == 8 || gq < B) a = xq[blk * (16 * B) + pp * (B * 4)];     // lanes of unused batch rows feed zeros
                mma_bf16_16x8x16(c[pp], a.x, a.y, a.z, a.w, bitselect(prmt(rw, 0u, 0x1100u), e0, kRemMask),
                                 bitselect(prmt(rw, 0u, 0x3322u), e1, kRemMask));
            };

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
                    Dec dec[PPW];
#pragma unroll
                    for (int pp = 0; pp < PPW; pp++) dec[pp].open(ctx, cur.base + r * cur.stride(), sigma4 + 32u * pp, cur.rows);
                    auto run = [&](auto checked_tag) {
                        constexpr bool kChecked = decltype(checked_tag)::value;
                        for (int gi = 0; gi < full; gi++) {
                            // next group of this record, or the first group of the next unit (of this one again if there is none)
                            const uint32_t *src = (gi + 1 < full) ? rem + (gi + 1) * (kRG * 32) : rem_next;
#pragma unroll
                            for (int pp = 0; pp < PPW; pp++)
#pragma unroll
                                for (int j = 0; j < kRG; j++) r_nxt[pp][j] = __ldg(src + j * 32 + pp * 8);
                            const int g0 = gi * kRG;
#pragma unroll
                            for (int j = 0; j < kRG; j += 2) {
                                uint32_t eA0[PPW], eA1[PPW], eB0[PPW], eB1[PPW];
#pragma unroll
                                for (int pp = 0; pp < PPW; pp++) dec[pp].template two<kChecked>(ctx, eA0[pp], eA1[pp], eB0[pp], eB1[pp]);
#pragma unroll
                                for (int pp = 0; pp < PPW; pp++) {
                                    mac(pp, g0 + j, r_cur[pp][j], eA0[pp], eA1[pp]);
                                    mac(pp, g0 + j + 1, r_cur[pp][j + 1], eB0[pp], eB1[pp]);
                                }
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
#pragma unroll
                            for (int pp = 0; pp < PPW; pp++) {
                                uint32_t eA0, eA1, eB0, eB1;
                                dec[pp].template two<kChecked>(ctx, eA0, eA1, eB0, eB1);
                                mac(pp, blk, __ldg(rem + blk * 32 + pp * 8), eA0, eA1);
                                if (blk + 1 < nblk) mac(pp, blk + 1, __ldg(rem + (blk + 1) * 32 + pp * 8), eB0, eB1);
                            }
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
#pragma unroll
                for (int pp = 0; pp < PPW; pp++) {
                    typename Codec::template Stream<GlobalWords> s0, s1;
                    const int64_t w0 = static_cast<int64_t>(cur.off) + (sigma4 >> 2) + 8 * pp;
                    s0.init(GlobalWords{L.exp, L.exp_words, w0});
                    s1.init(GlobalWords{L.exp, L.exp_words, w0 + 32});
                    for (int blk = 0; blk < nblk; blk++) {
                        const uint32_t rw = __ldg(rem + blk * 32 + pp * 8);
                        const uint32_t a0 = s0.next(tab);
                        const uint32_t b0 = s1.next(tab);
                        const uint32_t a1 = s0.next(tab);
                        const uint32_t b1 = s1.next(tab);
                        mac(pp, blk, rw, (a0 << 7) | (a1 << 23), (b0 << 7) | (b1 << 23));
                    }
                }
            }
            have_first = next_first;

            const bool quad_done = !(nxt.valid && nxt.qi == cur.qi);       // last chunk of this quad in this stage
            if (quad_done) {
                float v = c[0][0] + c[0][3];
#pragma unroll
                for (int pp = 1; pp < PPW; pp++) v += c[pp][0] + c[pp][3];
                part[(parity * 4 + wig) * 32 + lane] = v;
#pragma unroll
                for (int pp = 0; pp < PPW; pp++) c[pp][0] = c[pp][1] = c[pp][2] = c[pp][3] = 0.f;
            }
            group_barrier(group, kWG * 32);  // the unit's ring space is free; partial sums are visible
            if (quad_done) {
                if (wig == 0) {
                    const float *pp = part + parity * 128 + lane;
                    float v = pp[0];
#pragma unroll
                    for (int w = 1; w < kWG; w++) v += pp[32 * w];
                    float *a = acc + cur.qi * 32 + lane;
                    if (stage > 0) v += *a;
                    if (stage + 1 < G.stages) {
                        *a = v;
                    } else {
                        const int row = 4 * (q_lo + cur.qi) + t;
                        if (gq < B && row < L.M) {
                            if (exchange) ys[gq * rows_cta + (row - row_lo)] = f32_to_bf16_rn(v);
                            else Y[static_cast<int64_t>(gq) * L.M + row] = f32_to_bf16_rn(v);
                        }
                    }
                }
                parity ^= 1u;
            }
            if (nxt.valid && !early) {
                if (nxt.staged) issue(nxt, slot ^ 1);
                else place(nxt, slot ^ 1);
            }
            cur = nxt;
            slot ^= 1;
        }
    }

    if (exchange) {
        // one thread asks whether every peer's buffer may be overwritten (an acquire at system scope); the barrier that
        // makes the staged results visible hands its answer to the others
        if (tid == 0 && !counter_wait_bounded(pick(peers.ready, peers.rank), launch_no * peers.world)) atomicExch(&g_staged_status, 8);
        __syncthreads();
        for (int i = tid; i < B * rows_cta; i += kThreads) {
            const int b = i / rows_cta, rr = i - b * rows_cta;
            const uint16_t v = ys[i];
            const int64_t at = static_cast<int64_t>(b) * peers.m_total + peers.row_base + row_lo + rr;
#pragma unroll
            for (int q = 0; q < kMaxPeers; q++)
                if (q < peers.world) peers.y[q][at] = v;
        }
        exchange_finish(peers, launch_no);
    }
}

// ---- host side -------------------------------------------------------------------------------------
// Shared-memory plan of a launch; false when the shape does not fit (the caller then uses another kernel).
template <class Codec, int B>
static bool quad_plan(const Layer &L, int grid, bool exchange, uint32_t ans_bits, QuadGeom &G, uint32_t &smem_bytes) {
    constexpr bool kHuff = std::is_same<Codec, HuffCodec>::value;
    const uint32_t one_table = kHuff ? kPairEntries * 4u : (4u << ans_bits);
    const uint32_t chunk_bytes = static_cast<uint32_t>(B) * L.Nc * 2u;
    const int nquads = (L.M + 3) / 4;
    const int nq = (nquads + grid - 1) / grid;
    const uint32_t ys_bytes = exchange ? ((static_cast<uint32_t>(B) * (4u * nq) * 2u + 255u) & ~255u) : 0u;
    const uint32_t cap = static_cast<uint32_t>(kSmemMax);
    for (int copies_log2 = 2; copies_log2 >= 0; copies_log2--) {
        const uint32_t lut = one_table << copies_log2;
        const uint32_t fixed = lut + kExactBytes + kQuadCtrlBytes + kQuadPartBytes + ys_bytes + kSlackBytes;
        const uint32_t ring_need = kQuadGroups * kQuadRingWant;
        if (fixed + ring_need + chunk_bytes > cap) continue;
        // as many chunks of X per stage as fit beside the wanted rings; partial sums are parked between stages
        int cps = static_cast<int>((cap - fixed - ring_need) / chunk_bytes);
        if (cps > L.S) cps = L.S;
        int stages = (L.S + cps - 1) / cps;
        uint32_t acc_bytes = 0;
        if (stages > 1) {
            acc_bytes = (static_cast<uint32_t>(nq) * 128u + 255u) & ~255u;
            while (cps > 0 && fixed + ring_need + acc_bytes + static_cast<uint32_t>(cps) * chunk_bytes > cap) cps--;
            if (cps == 0) continue;
            stages = (L.S + cps - 1) / cps;
        }
        const uint32_t x_bytes = (static_cast<uint32_t>(cps) * chunk_bytes + 255u) & ~255u;
        if (fixed + acc_bytes + x_bytes + kQuadGroups * kQuadRingLeast > cap) continue;
        uint32_t ring_bytes = ((cap - fixed - acc_bytes - x_bytes) / kQuadGroups) & ~255u;
        if (ring_bytes > 4u * kRingMax) ring_bytes = 4u * kRingMax;
        G.lut_bytes = lut;
        G.copy_shift = 2u + copies_log2;
        G.index_mask = kHuff ? (static_cast<uint32_t>(kPairEntries - 1) << G.copy_shift) : (((1u << ans_bits) - 1u) << G.copy_shift);
        G.part_off = lut + kExactBytes + kQuadCtrlBytes;
        G.acc_off = G.part_off + kQuadPartBytes;
        G.ys_off = G.acc_off + acc_bytes;
        G.x_off = G.ys_off + ys_bytes;
        G.ring_off = G.x_off + x_bytes;
        G.x_bytes = x_bytes;
        G.ring_bytes = ring_bytes;
        G.chunks_per_stage = cps;
        G.stages = stages;
        smem_bytes = G.ring_off + kQuadGroups * ring_bytes + kSlackBytes;
        return true;
    }
    return false;
}

int quad_passes_per_warp();      // 0 = by table kind, 1 = 32 warps, 2 = 16 warps: see bhi_set_quad_warps

template <class Codec, int B, int PPW>
static int quad_launch_p(const Layer &L, const typename Codec::Args &targs, const uint8_t *prepared, const uint16_t *X, uint16_t *Y,
                         const PeerSet *peers, cudaStream_t st) {
    int grid = sm_count();
    const int nquads = (L.M + 3) / 4;
    if (grid > nquads) grid = nquads;
    QuadGeom G{};
    uint32_t smem_bytes = 0;
    if (!quad_plan<Codec, B>(L, grid, peers != nullptr, ans_bits_of(targs), G, smem_bytes)) return kStagedDeclined;
    auto kernel = quad_kernel<Codec, B, PPW>;
    if (int rc = staged_prepare(kernel)) return rc;
    PeerSet ps{};
    if (peers) ps = *peers;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kQuadGroups * (4 / PPW) * 32);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap_launches() ? 1 : 0;
    const uint32_t ans_bits = ans_bits_of(targs);
    const Consts k{ans_bits, (1u << ans_bits) - 1u, 1u, 8u, 4u * kCopies, 65536u};
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, L, targs, prepared, reinterpret_cast<const uint32_t *>(X), Y, ps, G, k);
    return e == cudaSuccess ? BHI_OK : cuda_fail(e, "quad kernel launch");
}

// pair_complete: the caller knows that every window of the folded table resolves two symbols (no code
// longer than kPairBits / 2).  Such tables run fastest with two warps per group (a lane decodes four
// streams); tables with unresolved windows with four warps per group, where the divergent
// symbol-by-symbol detour stalls half as many streams.  Only a tuning hint: the kernel itself reads
// from the table header whether it may skip the per-step test.
template <class Codec, int B>
static int quad_launch_b(const Layer &L, const typename Codec::Args &targs, const uint8_t *prepared, const uint16_t *X, uint16_t *Y,
                         const PeerSet *peers, bool pair_complete, cudaStream_t st) {
    int ppw = quad_passes_per_warp();
    if (ppw == 0) ppw = (pair_complete || !std::is_same<Codec, HuffCodec>::value) ? 2 : 1;
    if (ppw == 2) return quad_launch_p<Codec, B, 2>(L, targs, prepared, X, Y, peers, st);
    return quad_launch_p<Codec, B, 1>(L, targs, prepared, X, Y, peers, st);
}

template <class Codec>
static int quad_launch(const Layer &L, const typename Codec::Args &targs, const uint8_t *prepared, const uint16_t *X, uint16_t *Y,
                       const PeerSet *peers, int B, bool pair_complete, cudaStream_t st) {
    if (!staged_shape_ok(L) || !aligned(prepared, 16)) return kStagedDeclined;
    if (static_cast<int64_t>(L.S) * L.M >= (1ll << 31)) return kStagedDeclined;
    switch (B) {
        case 1: return quad_launch_b<Codec, 1>(L, targs, prepared, X, Y, peers, pair_complete, st);
        case 2: return quad_launch_b<Codec, 2>(L, targs, prepared, X, Y, peers, pair_complete, st);
        case 3: return quad_launch_b<Codec, 3>(L, targs, prepared, X, Y, peers, pair_complete, st);
        case 4: return quad_launch_b<Codec, 4>(L, targs, prepared, X, Y, peers, pair_complete, st);
        case 5: return quad_launch_b<Codec, 5>(L, targs, prepared, X, Y, peers, pair_complete, st);
        case 6: return quad_launch_b<Codec, 6>(L, targs, prepared, X, Y, peers, pair_complete, st);
        case 7: return quad_launch_b<Codec, 7>(L, targs, prepared, X, Y, peers, pair_complete, st);
        case 8: return quad_launch_b<Codec, 8>(L, targs, prepared, X, Y, peers, pair_complete, st);
    }
    return kStagedDeclined;
}

}  // namespace bhi
