// Staged decode-side kernels for sm_100a.
//
// One persistent CTA per SM, 32 warps (16 for batches above 4, which need more registers).
//
// Memory plan.  The exponent record of a (chunk, row) pair is contiguous in global memory; lane 0
// of the warp that owns the row brings it into the warp's private shared-memory ring with ONE
// bulk async copy (cp.async.bulk, completion counted on an mbarrier) while the warp is still
// decoding the previous record.  Stream word w of stream g then sits at ring word 64*w + g, so
// lane l (streams l and l+32) always reads bank l: the data-dependent word fetches are
// conflict-free.  The sign/mantissa row needs no reordering between lanes (lane l owns bytes
// 4l..4l+3 of every 128-byte block), so it is read straight from global memory, 128 bytes per
// warp and block, eight blocks ahead of use and prefetched across record boundaries.  X is staged
// once per CTA in shared memory, permuted so that one 8-byte load gives a lane its four values of
// a block.
//
// Decode plan (Huffman).  The four byte tables of the format are folded, per CTA, into a
// 4096-entry table indexed by the next 12 bits of a stream.  An entry yields TWO symbols, already
// shifted to the exponent positions of a bf16x2 word, and the number of bits they use.  A stream
// keeps no window registers: its state is one bit cursor; each step re-reads the two ring words
// under the cursor, so there is no refill branch in the loop.  Windows the 12 bits cannot
// resolve as a pair give the first symbol only (the second comes from one more lookup) or, for
// codes longer than 12 bits, fall back to the exact four-table cascade; both are rare.
//
// Decode plan (rANS).  One table word per slot, 64-bit state kept as two registers,
// state' = freq * (state >> 8) + rem as one 32x32+64 multiply-add (a valid stream keeps
// state < 2^(32 + bits), bits <= 12), refill word fetched from the ring.
//
// Multiply-accumulate (GEMV sinks).  One mma.sync.m16n8k16 per block and pair of batch rows, with the
// words a lane has just rebuilt as its B fragment and its own X pairs as its A fragment; see the
// comment above GemvSink.
//
// A warp owns whole output rows (all K-chunks in order): no cross-warp reduction, fixed
// summation order.  Rows are dealt to CTAs in equal contiguous ranges and to the warps of a CTA
// through a shared counter.  (Layers with few rows per CTA and several K-chunks are split by
// record instead, with the partial sums added in chunk order at the end; row-sharded layers can
// write their results into every rank's buffer: ExchangeSink.)  Records too large for the ring,
// or whose offsets are not in storage order, are decoded from global memory by the table-exact
// decoder.
//
// Every wait on an mbarrier is bounded; on expiry the warp records a status code in a device
// word (bhi_debug_status), skips the record and carries on: a lost copy cannot hang the GPU.
// Cursors are clamped once per group of blocks, so corrupt tables or data cannot walk a read
// out of the CTA's shared memory.
#pragma once

#include <mutex>
#include <type_traits>
#include <unordered_map>

#include "bhi_common.cuh"

namespace bhi {

constexpr int kStagedDeclined = -1;

constexpr int kPairBits = 12;
constexpr int kPairEntries = 1 << kPairBits;
constexpr int kCopies = 4;                     // bank-interleaved copies of the fast table (lane & 3 picks one)
constexpr int kLutBytes = kPairEntries * 4 * kCopies;   // 64 KB (Huffman pair table; rANS uses the first 4 KB)
constexpr int kExactBytes = 2048;              // table-exact copies for rare windows / direct records
constexpr int kCtrlBytes = 1024;               // mbarriers (2 per warp) + row counter
constexpr int kHeaderBytes = kLutBytes + kExactBytes + kCtrlBytes;
constexpr int kSlackBytes = 2048;              // readable space above the last ring
constexpr int kSmemMax = 227 * 1024;
constexpr int kRingMax = 8192;
constexpr int kXStageMax = 32 * 1024;          // X is staged in shared memory up to this many bytes (32 warps)
constexpr int kXStageMax16 = 64 * 1024;        // ... with 16 warps, whose rings need half the room
constexpr int kPartMax = 16 * 1024;             // most shared memory spent on staged results
constexpr int kGroup = 8;                      // blocks per rem prefetch group (8 measured 2 % faster than 4)
constexpr uint32_t kSpinLimit = 1u << 22;

// pair-table entry fields
constexpr uint32_t kEntBits = 0xFu;            // bits 0..3: stream bits consumed (bit 4 stays zero: the word is also a shift count)
constexpr uint32_t kEntSingle = 0x20u;         // only the first symbol is resolved
constexpr uint32_t kEntExact = 0x40u;          // nothing resolved: use the exact tables
constexpr uint32_t kRemMask = 0x807F807Fu;     // sign + mantissa bits of a bf16x2 word; the rest is exponent

// Multipliers handed to the kernel at launch.  Integer multiply-add runs on the FMA pipe, plain
// shifts/adds on the (half-rate, saturated) integer pipe; because the compiler cannot see these
// values it has to keep the multiply-add form.
struct Consts {
    uint32_t ans_bits, ans_mask;             // rANS: probability precision of the layer's table and 2^bits - 1
    uint32_t one, eight, entry, shift16;     // entry = bytes between consecutive fast-table entries (4 * copies);
                                             // shift16 = 65536 (a left shift by 16 as a multiply)
};

// A prepared-table blob (Huffman): one copy of the folded pair table, then the exact tables.
constexpr int kPreparedBytes = kPairEntries * 4 + kExactBytes;

static_assert(sizeof(HuffTables) <= kExactBytes && sizeof(AnsTables) <= kExactBytes, "exact tables do not fit");
static_assert((4 << kAnsBitsMax) * kCopies <= kLutBytes, "the largest rANS table does not fit the fast-table region");

__device__ int g_staged_status = 0;            // 0 = fine; otherwise the last failure code

// ---- PTX wrappers ----------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
// global -> this CTA's shared memory; both addresses 16-byte aligned, size a multiple of 16
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void prefetch_l2(const void *p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}
// Programmatic dependent launch: let the next kernel in the stream start its weight-only prologue
// while this one is still running, and wait for the previous kernel's results before touching them.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kSpinLimit; i++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// ---- sinks: what happens to the two bf16x2 words a lane produces per 128-column block --------------
// gblk = index of the 128-column block inside the full row (chunk * blocks_per_chunk + block).
//
// The multiply-accumulate runs on the warp-level tensor-core instruction (mma.sync m16n8k16, BF16 in,
// FP32 accumulate) without any conversion or data movement: the two words w0, w1 a lane has just
// rebuilt ARE its B fragment (k = the 16 columns its lane group holds, n = its lane group), and the
// lane's own X pairs of the same columns are its A fragment (rows 0..7 = one batch row seen by the 8
// lane groups, rows 8..15 = the next batch row).  D[g][g'] is then the dot product of group g's X
// columns with group g''s W columns; only the diagonal g = g' is meaningful, and the sum of the 8
// diagonal entries is the block's contribution to the row's dot product.  One instruction replaces
// eight conversions and two packed FMAs per batch row; the seven off-diagonal products are waste the
// tensor pipe has room for.
__device__ __forceinline__ void mma_bf16_16x8x16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                                 uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int B, bool kXS>
struct GemvSink {
    static constexpr int kPairs = B / 2;       // batch rows handled two per instruction
    static constexpr bool kOdd = (B & 1) != 0; // ... and a last one alone
    float c[kPairs + (kOdd ? 1 : 0)][4];
    const uint32_t *x;      // X as bf16 pairs (global)
    const uint4 *xq;        // staged: [pair][gblk][lane] -> {b: pair at 2l, b+1: pair at 2l, b: pair at 64+2l, b+1: pair at 64+2l}
    const uint2 *xo;        // staged, last row of an odd batch: [gblk][lane] -> {pair at 2l, pair at 64+2l}
    int64_t row_pairs;      // K / 2
    int row_blocks;         // K / 128
    uint16_t *Y;
    int M;

    __device__ __forceinline__ void stage(uint8_t *x_region, int tid, int nthreads) {
        if (kXS) {
            uint4 *dq = reinterpret_cast<uint4 *>(x_region);
            const int per = row_blocks * 32;
            for (int i = tid; i < kPairs * per; i += nthreads) {
                const int l = i & 31, gb = i >> 5;
                const int p = gb / row_blocks, g = gb - p * row_blocks;
                const uint32_t *s0 = x + (2 * p) * row_pairs + g * 64 + l;
                const uint32_t *s1 = s0 + row_pairs;
                dq[i] = make_uint4(__ldg(s0), __ldg(s1), __ldg(s0 + 32), __ldg(s1 + 32));
            }
            uint2 *dk = reinterpret_cast<uint2 *>(dq + kPairs * per);
            if (kOdd) {
                for (int i = tid; i < per; i += nthreads) {
                    const uint32_t *s0 = x + (B - 1) * row_pairs + (i >> 5) * 64 + (i & 31);
                    dk[i] = make_uint2(__ldg(s0), __ldg(s0 + 32));
                }
            }
            xq = dq;
            xo = dk;
        }
    }
    __device__ __forceinline__ void clear() {
#pragma unroll
        for (int p = 0; p < kPairs + (kOdd ? 1 : 0); p++)
#pragma unroll
            for (int j = 0; j < 4; j++) c[p][j] = 0.f;
    }
    __device__ __forceinline__ void reset(int lane) {
        x += lane;
        xq += lane;
        xo += lane;
        clear();
    }
    __device__ __forceinline__ void begin_record(int) {}
    __device__ __forceinline__ void after_wait(int) {}        // right after the wait for the previous kernel
    __device__ __forceinline__ void finish_kernel() {}        // last thing the kernel does
    __device__ __forceinline__ void put(const Consts &, int gblk, uint32_t w0, uint32_t w1) {
#pragma unroll
        for (int p = 0; p < kPairs; p++) {
            uint4 q;
            if (kXS) {
                q = xq[(p * row_blocks + gblk) * 32];
            } else {
                const uint32_t *s0 = x + (2 * p) * row_pairs + gblk * 64;
                const uint32_t *s1 = s0 + row_pairs;
                q = make_uint4(__ldg(s0), __ldg(s1), __ldg(s0 + 32), __ldg(s1 + 32));
            }
            mma_bf16_16x8x16(c[p], q.x, q.y, q.z, q.w, w0, w1);
        }
        if (kOdd) {
            uint2 q;
            if (kXS) {
                q = xo[gblk * 32];
            } else {
                const uint32_t *s0 = x + (B - 1) * row_pairs + gblk * 64;
                q = make_uint2(__ldg(s0), __ldg(s0 + 32));
            }
            mma_bf16_16x8x16(c[kPairs], q.x, 0u, q.y, 0u, w0, w1);
        }
    }
    // The dot product of batch row b so far: the diagonal entries of its accumulator tile live in the lanes
    // whose column pair contains their lane group's index; everything else in the tile is discarded.
    __device__ __forceinline__ float row_value(int b, int lane) const {
        const bool holds = (lane & 3) == (lane >> 3);
        const bool second = ((lane >> 2) & 1) != 0;
        const float *t = c[b >> 1];
        const float lo = second ? t[1] : t[0], hi = second ? t[3] : t[2];
        return warp_sum(holds ? ((b & 1) ? hi : lo) : 0.f);
    }
    __device__ __forceinline__ void finish_row(int m, int lane) {
#pragma unroll
        for (int b = 0; b < B; b++) {
            const float v = row_value(b, lane);
            if (lane == 0) Y[static_cast<int64_t>(b) * M + m] = f32_to_bf16_rn(v);
        }
        clear();
    }
    // staged results: part[(b * rows + r) * slots + slot]
    static constexpr int kBatch = B;
    static constexpr bool kStagesResults = false;      // only when the launch asks for split work
    __device__ __forceinline__ void finish_part(float *part, int r, int slot, int rows, int slots, int lane) {
#pragma unroll
        for (int b = 0; b < B; b++) {
            const float v = row_value(b, lane);
            if (lane == 0) part[(b * rows + r) * slots + slot] = v;
        }
        clear();
    }
    static __device__ __forceinline__ float part_sum(const float *part, int i, int slots) {
        float v = part[i * slots];
        for (int s = 1; s < slots; s++) v += part[i * slots + s];
        return v;
    }
    __device__ __forceinline__ void combine(const float *part, int row_lo, int rows, int slots, int) {
        for (int i = threadIdx.x; i < B * rows; i += blockDim.x) {
            const int b = i / rows, r = i - b * rows;
            Y[static_cast<int64_t>(b) * M + row_lo + r] = f32_to_bf16_rn(part_sum(part, i, slots));
        }
    }
};

struct DenseSink {
    uint32_t *out;          // Y as bf16 pairs
    int64_t row_pairs;      // K / 2
    uint32_t *row;
    __device__ __forceinline__ void stage(uint8_t *, int, int) {}
    __device__ __forceinline__ void reset(int lane) { out += lane; }
    __device__ __forceinline__ void begin_record(int m) { row = out + static_cast<int64_t>(m) * row_pairs; }
    __device__ __forceinline__ void after_wait(int) {}
    __device__ __forceinline__ void finish_kernel() {}
    __device__ __forceinline__ void put(const Consts &, int gblk, uint32_t w0, uint32_t w1) {
        row[gblk * 64] = w0;
        row[gblk * 64 + 32] = w1;
    }
    __device__ __forceinline__ void finish_row(int, int) {}
    static constexpr int kBatch = 0;
    static constexpr bool kStagesResults = false;
    __device__ __forceinline__ void finish_part(float *, int, int, int, int, int) {}
    __device__ __forceinline__ void combine(const float *, int, int, int, int) {}
};

// ---- row-sharded GEMV whose epilogue is the all-gather ------------------------------------------------
// Every rank computes the rows [row_base, row_base + M) of Y [B, M_total] and needs all of it.  Instead
// of a collective after the kernel, the lanes that hold a finished dot product store it straight into
// the Y buffer of every rank (plain stores to peer-mapped pointers over NVLink; lane r serves rank r).
// Four counter words per layer and rank make that safe without any other kernel:
//   ready  - each rank adds 1 on every peer when its launch may be written to (its earlier consumers of
//            Y are done: the add comes after the wait for the previous kernel in the stream); a warp
//            checks its own copy (>= world * launch number) before its first remote store;
//   arrive (local) - every CTA adds 1 after its stores; the CTA that brings it to the grid size is the last
//            one of this launch on this GPU and puts it back to zero;
//   done   - that last CTA adds 1 on every peer (release at system scope, cumulative over all CTAs'
//            stores through the arrive counter) and then waits until its own copy shows
//            world * launch number, so whatever runs next on the stream sees the whole of Y.  One
//            system-scope signal per peer and launch, whatever the grids of the ranks are;
//   launches (local) - how often this layer has run; written by the one waiting thread at the end.
// launches and arrive are two consecutive words (PeerSet::launches points at the first).
// Both waits are bounded; on expiry the status word is set (8 = peers not ready, 9 = peers not done)
// and the kernel carries on.
constexpr int kMaxPeers = BHI_MAX_PEERS;

struct PeerSet {
    uint16_t *y[kMaxPeers];
    uint32_t *ready[kMaxPeers];
    uint32_t *done[kMaxPeers];
    uint32_t *launches;
    int world, rank, row_base, m_total;
};

__device__ __forceinline__ void red_release_sys_add(uint32_t *p, uint32_t v) {
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_relaxed_sys_add(uint32_t *p, uint32_t v) {
    asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// waits until the counter has reached `target` (wrap-safe); false when a second has passed without it
constexpr uint64_t kPeerWaitNs = 1000ull * 1000ull * 1000ull;
__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ bool counter_wait_bounded(const uint32_t *p, uint32_t target) {
    if (static_cast<int32_t>(ld_acquire_sys(p) - target) >= 0) return true;
    const uint64_t t0 = global_ns();
    for (uint32_t i = 0; i < kSpinLimit; i++) {            // the iteration bound is a second line of defence
        if (static_cast<int32_t>(ld_relaxed_sys(p) - target) >= 0) {
            asm volatile("fence.acq_rel.sys;" ::: "memory");
            return true;
        }
        if ((i & 15u) == 15u && global_ns() - t0 > kPeerWaitNs) return false;
        __nanosleep(40);
    }
    return false;
}

// a[i] without indexing the array by a register (that would move the whole kernel-parameter struct to
// local memory, accumulators included)
template <class T>
__device__ __forceinline__ T pick(T const (&a)[kMaxPeers], int i) {
    T v = a[0];
#pragma unroll
    for (int r = 1; r < kMaxPeers; r++)
        if (i == r) v = a[r];
    return v;
}

__device__ __forceinline__ uint32_t atom_add_acq_rel_gpu(uint32_t *p, uint32_t v) {
    uint32_t old;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
}

// End of an exchange kernel (every thread of the CTA calls it after its stores to the peers).
__device__ __forceinline__ void exchange_finish(const PeerSet &peers, uint32_t launch_no) {
    // The barrier orders every warp's stores before thread 0; its release is cumulative over them, and the
    // last CTA's acquire of the arrive counter, then its release at system scope, carry them to the peers.
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t before = atom_add_acq_rel_gpu(peers.launches + 1, 1u);
        if (before + 1u == gridDim.x) {
            // last CTA of this launch.  The arrival counter goes back to zero for the next launch of the layer,
            // whatever grid that one uses (its CTAs arrive only after this whole grid has completed).
            *reinterpret_cast<volatile uint32_t *>(peers.launches + 1) = 0u;
            // one system-scope fence, then a relaxed add per peer: a release per peer would be a fence per peer, one after
            // the other (7 us more per launch on 8 GPUs than on 4)
            asm volatile("fence.acq_rel.sys;" ::: "memory");
#pragma unroll
            for (int q = 0; q < kMaxPeers; q++)
                if (q < peers.world) red_relaxed_sys_add(peers.done[q], 1u);
            if (!counter_wait_bounded(pick(peers.done, peers.rank), launch_no * peers.world)) atomicExch(&g_staged_status, 9);
            *peers.launches = launch_no;
            __threadfence();
        }
    }
}

template <int B, bool kXS>
struct ExchangeSink : GemvSink<B, kXS> {
    using Base = GemvSink<B, kXS>;
    PeerSet peers;
    uint16_t *dst;          // this lane's destination rank's Y (lanes >= world: unused)
    uint32_t launch_no;     // 1-based number of this launch of the layer
    bool peers_ready;

    __device__ __forceinline__ void after_wait(int lane) {
        launch_no = *reinterpret_cast<const volatile uint32_t *>(peers.launches) + 1u;   // written by this layer's previous launch
        peers_ready = false;
        dst = pick(peers.y, lane < peers.world ? lane : peers.rank);
        if (blockIdx.x == 0 && threadIdx.x < peers.world) red_release_sys_add(pick(peers.ready, threadIdx.x), 1u);
    }
    __device__ __forceinline__ void finish_row(int m, int lane) {
        if (!peers_ready) {
            if (!counter_wait_bounded(pick(peers.ready, peers.rank), launch_no * peers.world) && lane == 0) atomicExch(&g_staged_status, 8);
            peers_ready = true;
        }
#pragma unroll
        for (int b = 0; b < B; b++) {
            const float v = Base::row_value(b, lane);                            // every lane holds the sum
            if (lane < peers.world) dst[static_cast<int64_t>(b) * peers.m_total + peers.row_base + m] = f32_to_bf16_rn(v);
        }
        Base::clear();
    }
    // Results staged in shared memory leave for every rank at the end, consecutive threads writing
    // consecutive rows (coalesced peer stores instead of one 2-byte store per row and rank).
    static constexpr bool kStagesResults = true;
    __device__ __forceinline__ void combine(const float *part, int row_lo, int rows, int slots, int lane) {
        if (!counter_wait_bounded(pick(peers.ready, peers.rank), launch_no * peers.world) && lane == 0) atomicExch(&g_staged_status, 8);
        for (int i = threadIdx.x; i < B * rows; i += blockDim.x) {
            const int b = i / rows, r = i - b * rows;
            const uint16_t v = f32_to_bf16_rn(Base::part_sum(part, i, slots));
            const int64_t at = static_cast<int64_t>(b) * peers.m_total + peers.row_base + row_lo + r;
#pragma unroll
            for (int q = 0; q < kMaxPeers; q++)
                if (q < peers.world) peers.y[q][at] = v;
        }
    }
    __device__ __forceinline__ void finish_kernel() { exchange_finish(peers, launch_no); }
};

// ---- Huffman: folded pair table ---------------------------------------------------------------------
__device__ __forceinline__ uint32_t umad(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// (a & mask) | (b & ~mask) in one logic instruction
__device__ __forceinline__ uint32_t bitselect(uint32_t a, uint32_t b, uint32_t mask) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xE4;" : "=r"(d) : "r"(a), "r"(b), "r"(mask));
    return d;
}

// Resolve one symbol from `known` valid low bits of `v` (other bits zero).  Returns its length, 0
// if the known bits do not determine it.
__device__ __forceinline__ uint32_t resolve_symbol(const HuffTables &t, uint32_t v, uint32_t known, uint32_t &sym) {
    sym = t.lut[0][v & 0xFF];
    if (sym != 255) {
        const uint32_t n = t.len[sym];
        return (n >= 1 && n <= 8 && n <= known) ? n : 0;
    }
    if (known <= 8) return 0;
    sym = t.lut[1][(v >> 8) & 0xFF];
    if (sym == 255) return 0;
    const uint32_t n = t.len[sym];
    return (n >= 9 && n <= known) ? n : 0;
}

// entry: bits 0..3 stream bits consumed, bit 5 single, bit 6 exact, bits 7..14 first exponent,
// bits 16..19 length of the first symbol, bits 23..30 second exponent
__device__ __forceinline__ uint32_t pair_entry(const HuffTables &t, uint32_t v) {
    uint32_t s0, s1;
    const uint32_t l0 = resolve_symbol(t, v, kPairBits, s0);
    if (!l0) return kEntExact;
    const uint32_t l1 = resolve_symbol(t, v >> l0, kPairBits - l0, s1);
    return l1 ? ((s0 << 7) | (s1 << 23) | (l0 << 16) | (l0 + l1)) : ((s0 << 7) | (l0 << 16) | l0 | kEntSingle);
}

// Where the kCopies copies of entry v live (word index of copy 0): interleaved, so copy c only ever
// touches banks congruent to c mod kCopies.  (Picking the bank from the top index bits instead was
// measured slower: two more integer instructions per lookup cost more than the conflicts they save.)
__device__ __forceinline__ uint32_t pair_slot(uint32_t v) { return v * kCopies; }

__device__ __forceinline__ void build_pair_table(uint32_t *dst, const HuffTables &t, int tid, int nthreads) {
    for (int v = tid; v < kPairEntries; v += nthreads) {
        const uint32_t e = pair_entry(t, v);
        *reinterpret_cast<uint4 *>(dst + pair_slot(v)) = make_uint4(e, e, e, e);
    }
}

// A code longer than the table index: resolve one symbol with the exact four-table cascade.
// Returns {symbol, length}.  Out of line on purpose: it is rare and must not bloat the loop.
__device__ __noinline__ uint2 huff_exact_symbol(uint32_t win, const HuffTables *t) {
    const uint32_t s = huff_cascade(*t, win);
    return make_uint2(s, t->len[s]);
}

// A stream is a bit cursor p = (bit position) + (byte offset of the record in shared memory) / 8.
// Records start on 256-byte boundaries, so (p & ~31) * 8 is the byte address of the current word
// row and p & 31 the bit inside the word.
struct HuffStaged {
    uint32_t p0, p1, plim;
    __device__ __forceinline__ void open(const uint8_t *, uint32_t base, uint32_t limit, int) {
        p0 = p1 = base >> 3;
        plim = limit >> 3;
    }
    static __device__ __forceinline__ uint32_t window(const uint8_t *smem, const Consts &k, uint32_t p, uint32_t lane_off) {
        const uint32_t a = umad(p & ~31u, k.eight, lane_off);
        const uint32_t w0 = *reinterpret_cast<const uint32_t *>(smem + a);
        const uint32_t w1 = *reinterpret_cast<const uint32_t *>(smem + a + 256);
        return __funnelshift_r(w0, w1, p);
    }
    // this lane's copy of entry (win & 0xFFF): see pair_slot
    static __device__ __forceinline__ uint32_t lookup(const uint8_t *smem, const Consts &k, uint32_t win, uint32_t copy_off) {
        return *reinterpret_cast<const uint32_t *>(smem + umad(win & (kPairEntries - 1), k.entry, copy_off));
    }
    // entry is "single" (or was "exact" and its first symbol has just been taken): one more lookup
    __device__ __forceinline__ void second(const uint8_t *smem, const Consts &k, const HuffTables &t, uint32_t lane_off,
                                           uint32_t copy_off, uint32_t &p, uint32_t &e) {
        const uint32_t win = window(smem, k, p, lane_off);
        const uint32_t e2 = lookup(smem, k, win, copy_off);
        uint32_t s1 = (e2 >> 7) & 0xFFu, l1 = (e2 >> 16) & 15u;
        if (e2 & kEntExact) {
            const uint2 f = huff_exact_symbol(win, &t);
            s1 = f.x;
            l1 = f.y;
        }
        p = min(p + l1, plim);
        e = (e & 0x7F80u) | (s1 << 23);
    }
    __device__ __forceinline__ void first_exact(uint32_t win, const HuffTables &t, uint32_t &p, uint32_t &e) {
        const uint2 f = huff_exact_symbol(win, &t);
        p = min(p + f.y, plim);
        e = (f.x << 7) | kEntSingle;
    }
    __device__ __forceinline__ void pairs(const uint8_t *smem, const Consts &k, const HuffTables &t, uint32_t lane4,
                                          uint32_t copy_off, uint32_t &e0, uint32_t &e1) {
        const uint32_t win0 = window(smem, k, p0, lane4);
        const uint32_t win1 = window(smem, k, p1, lane4 + 128);
        e0 = lookup(smem, k, win0, copy_off);
        e1 = lookup(smem, k, win1, copy_off);
        p0 = umad(e0 & kEntBits, k.one, p0);
        p1 = umad(e1 & kEntBits, k.one, p1);
        if ((e0 | e1) & (kEntSingle | kEntExact)) {
            if ((e0 | e1) & kEntExact) {
                if (e0 & kEntExact) first_exact(win0, t, p0, e0);
                if (e1 & kEntExact) first_exact(win1, t, p1, e1);
            }
            // one pass serves every lane that needs a second symbol on exactly one of its streams
            const bool on1 = !(e0 & kEntSingle);
            if ((e0 | e1) & kEntSingle) {
                uint32_t p = on1 ? p1 : p0, e = on1 ? e1 : e0;
                second(smem, k, t, on1 ? lane4 + 128 : lane4, copy_off, p, e);
                if (on1) { p1 = p; e1 = e; } else { p0 = p; e0 = e; }
            }
            if (e1 & kEntSingle) second(smem, k, t, lane4 + 128, copy_off, p1, e1);      // both streams needed one
        }
    }
    __device__ __forceinline__ void clamp() {
        p0 = min(p0, plim);
        p1 = min(p1, plim);
    }
};

// ---- rANS over the ring ----------------------------------------------------------------------------
struct AnsLane {
    uint32_t lo, hi, nx;     // state, byte address of the next word of this stream
    __device__ __forceinline__ uint32_t symbol(const uint8_t *smem, const Consts &k, uint32_t copy_off, uint32_t alim) {
        if (hi == 0 && lo <= k.ans_mask) {
            hi = lo;
            lo = *reinterpret_cast<const uint32_t *>(smem + nx);
            nx = min(nx + 256u, alim);
        }
        const uint32_t e = *reinterpret_cast<const uint32_t *>(smem + umad(lo & k.ans_mask, k.entry, copy_off));
        const uint32_t shifted = __funnelshift_r(lo, hi, k.ans_bits);    // state >> bits, fits 32 bits
        const uint64_t next = static_cast<uint64_t>((e >> 12) & 0xFFFu) * shifted + (e & 0xFFFu);
        lo = static_cast<uint32_t>(next);
        hi = static_cast<uint32_t>(next >> 32);
        return e >> 24;
    }
};

struct AnsStaged {
    AnsLane a0, a1;
    uint32_t alim;
    __device__ __forceinline__ void open(const uint8_t *smem, uint32_t base, uint32_t limit, int lane) {
        const uint32_t p = base + 4u * lane;
        a0.lo = *reinterpret_cast<const uint32_t *>(smem + p);
        a1.lo = *reinterpret_cast<const uint32_t *>(smem + p + 128);
        a0.hi = a1.hi = 0;
        a0.nx = p + 256;
        a1.nx = p + 128 + 256;
        alim = limit + 4u * lane;
    }
    __device__ __forceinline__ void pairs(const uint8_t *smem, const Consts &k, const AnsTables &, uint32_t,
                                          uint32_t copy_off, uint32_t &e0, uint32_t &e1) {
        const uint32_t s00 = a0.symbol(smem, k, copy_off, alim);
        const uint32_t s10 = a1.symbol(smem, k, copy_off, alim + 128);
        const uint32_t s01 = a0.symbol(smem, k, copy_off, alim);
        const uint32_t s11 = a1.symbol(smem, k, copy_off, alim + 128);
        e0 = (s00 << 7) | (s01 << 23);
        e1 = (s10 << 7) | (s11 << 23);
    }
    __device__ __forceinline__ void clamp() {}
};

template <class Codec> struct StagedOf;
template <> struct StagedOf<HuffCodec> { using type = HuffStaged; };
template <> struct StagedOf<AnsCodec> { using type = AnsStaged; };

__device__ __forceinline__ void build_fast_table(uint32_t *fast, const HuffTables &t, int tid, int n) { build_pair_table(fast, t, tid, n); }
__device__ __forceinline__ void build_fast_table(uint32_t *fast, const AnsTables &t, int tid, int n) {
    for (int i = tid; i < (1 << t.bits); i += n) {
        const uint32_t e = __ldg(t.lut + i);
        *reinterpret_cast<uint4 *>(fast + i * kCopies) = make_uint4(e, e, e, e);
    }
}

// ---- the kernel ------------------------------------------------------------------------------------
struct Unit {
    int m, k;
    int64_t rec;
    uint32_t off;          // first exponent word
    uint32_t exp_bytes;    // staged exponent bytes (0 if the record is read from global memory)
    uint32_t base;         // byte offset of the record inside dynamic shared memory
    bool valid, staged;
};

// kPart: results are staged in shared memory (and work may be split by record); a compile-time switch so
// that the plain instantiation carries none of it.
template <class Codec, class Sink, int NW, bool kPart>
__global__ void __launch_bounds__(NW * 32, 1)
staged_kernel(Layer L, typename Codec::Args targs, const uint8_t *prepared, Sink sink_proto, uint32_t x_bytes,
              uint32_t ring_bytes, Consts k, uint32_t part_bytes_arg, int split_arg) {
    const uint32_t part_bytes = kPart ? part_bytes_arg : 0u;
    const bool split = kPart && split_arg != 0;
    extern __shared__ __align__(1024) uint8_t smem[];
    using Tables = typename Codec::Tables;
    using Dec = typename StagedOf<Codec>::type;

    uint32_t *fast = reinterpret_cast<uint32_t *>(smem);
    Tables &tab = *reinterpret_cast<Tables *>(smem + kLutBytes);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kLutBytes + kExactBytes);
    int *row_counter = reinterpret_cast<int *>(bars + 2 * NW);
    const uint32_t table_bar = smem_addr(reinterpret_cast<uint8_t *>(row_counter) + 8);   // for the prepared-table copy

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const uint32_t lane4 = 4u * lane;
    const uint32_t copy_off = 4u * (lane & (kCopies - 1));            // this lane's copy of the fast table
    // Optional result staging (part_bytes > 0): dot products go to part[b][row][slot] in shared memory and
    // are written out by the whole CTA at the end.  With `split` a unit of work is one (row, chunk) record
    // instead of a whole row - for layers with fewer rows than warps - and slot = chunk; the chunks of a row
    // are summed in chunk order at the end, so the result does not depend on which warp took which.
    float *part = reinterpret_cast<float *>(smem + kHeaderBytes + x_bytes);
    const uint32_t ring = kHeaderBytes + x_bytes + part_bytes + warp * ring_bytes;     // byte offset in smem, 256-aligned
    const uint32_t smem_base = smem_addr(smem);
    const uint32_t bar0 = smem_addr(&bars[2 * warp]);                      // slot s uses the barrier at bar0 + 8*s

    const int row_lo = static_cast<int>(static_cast<int64_t>(L.M) * blockIdx.x / gridDim.x);
    const int row_hi = static_cast<int>(static_cast<int64_t>(L.M) * (blockIdx.x + 1) / gridDim.x);
    const int64_t nrec = static_cast<int64_t>(L.S) * L.M;
    const int nblk = L.Nc >> 7;
    const int rows_cta = row_hi - row_lo;
    const int slots = split ? L.S : 1;             // partial sums kept per row when results are staged
    pdl_launch_dependents();
    // The first row of every warp is fixed (row_lo + warp), so its sign/mantissa row can be
    // requested from HBM before anything else is known; later rows come from the shared counter.
    if (lane == 0 && !split && row_lo + warp < row_hi)
        prefetch_l2(L.rem + static_cast<int64_t>(row_lo + warp) * L.Nc, static_cast<uint32_t>(L.Nc));
    if (threadIdx.x == 0) {
        *row_counter = NW;
        mbar_init(table_bar, 1);
    }
    if (lane == 0) {
        mbar_init(bar0, 1);
        mbar_init(bar0 + 8, 1);
        mbar_fence_init();
    }
    __syncthreads();
    if (prepared != nullptr && threadIdx.x == 0) {
        // Folded + exact tables were built once for this layer.  The blob holds ONE copy of the folded
        // table followed by the exact tables; it lands at the tail of the table region (so that the
        // exact tables fall into their place) and is fanned out into the interleaved copies below.
        mbar_expect_tx(table_bar, kPreparedBytes);
        bulk_copy_g2s(smem_base + kLutBytes - kPairEntries * 4, prepared, kPreparedBytes, table_bar);
    }

    auto next_index = [&]() -> int {               // next row (or, with `split`, next record) of this CTA
        int v = 0;
        if (lane == 0) v = atomicAdd(row_counter, 1);
        return __shfl_sync(0xFFFFFFFFu, v, 0);
    };
    auto describe = [&](int m, int k, Unit &u) {
        u.m = m;
        u.k = k;
        u.rec = static_cast<int64_t>(k) * L.M + m;
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
    auto rem_ptr = [&](const Unit &u) { return reinterpret_cast<const uint32_t *>(L.rem + u.rec * L.Nc) + lane; };

    // index v of the CTA's work list -> unit: row row_lo + v, or record (row_lo + v / S, v % S)
    auto unit_at = [&](int v, Unit &u) {
        if (split) {
            if (v < rows_cta * L.S) describe(row_lo + v / L.S, v % L.S, u);
        } else if (row_lo + v < row_hi) {
            describe(row_lo + v, 0, u);
        }
    };

    Unit cur, nxt;
    cur.valid = false;
    unit_at(warp, cur);
    if (cur.valid && cur.staged) issue(cur, 0);
    // Tables first: they belong to the layer, so this still overlaps the previous kernel in the stream
    // (and the first record copy in flight).
    Sink sink = sink_proto;
    if (prepared == nullptr) {
        load_tables(tab, targs, threadIdx.x, blockDim.x);
        __syncthreads();
        build_fast_table(fast, tab, threadIdx.x, blockDim.x);
    } else {
        if (!mbar_wait_bounded(table_bar, 0u) && threadIdx.x == 0) atomicExch(&g_staged_status, 2);
        // fan out: entry v (one word at the tail) -> kCopies words at pair_slot(v).  Slots overlap the raw
        // copy, so every thread reads all of its raw entries before anybody writes.
        constexpr int kPer = kPairEntries / (NW * 32);
        static_assert(kPairEntries % (NW * 32) == 0, "table size must divide by the CTA size");
        const uint32_t *raw = fast + (kLutBytes - kPairEntries * 4) / 4;
        uint32_t mine[kPer];
#pragma unroll
        for (int i = 0; i < kPer; i++) mine[i] = raw[threadIdx.x + i * NW * 32];
        __syncthreads();
#pragma unroll
        for (int i = 0; i < kPer; i++)
            *reinterpret_cast<uint4 *>(fast + pair_slot(threadIdx.x + i * NW * 32)) = make_uint4(mine[i], mine[i], mine[i], mine[i]);
    }
    // Everything above read weights only.  X (and Y) belong to the previous kernel in the stream.
    pdl_wait();
    sink.after_wait(lane);
    sink.stage(smem + kHeaderBytes, threadIdx.x, blockDim.x);
    __syncthreads();
    sink.reset(lane);
    int slot = 0;
    uint32_t phases = 0u;                          // bit s = parity the next wait on slot s expects
    uint32_t r_cur[kGroup], r_nxt[kGroup];
    bool have_first = false;                       // r_cur already holds the first group of `cur`

    while (cur.valid) {
        nxt.valid = false;
        if (!split && cur.k + 1 < L.S) describe(cur.m, cur.k + 1, nxt);
        else unit_at(next_index(), nxt);
        const bool early = nxt.valid && nxt.staged && (!cur.staged || cur.exp_bytes + nxt.exp_bytes <= ring_bytes);
        if (early) issue(nxt, slot ^ 1);

        const int gblk0 = cur.k * nblk;
        sink.begin_record(cur.m);
        const uint32_t *rem = rem_ptr(cur);
        const uint32_t *rem_next = nxt.valid ? rem_ptr(nxt) : rem;
        bool next_first = false;

        if (cur.staged) {
            if (!have_first) {
#pragma unroll
                for (int j = 0; j < kGroup; j++) r_cur[j] = (j < nblk) ? __ldg(rem + j * 32) : 0u;
            }
            const bool arrived = mbar_wait_bounded(bar0 + 8u * slot, (phases >> slot) & 1u);
            phases ^= 1u << slot;
            if (arrived) {
                Dec dec;
                // cursors may not pass the last word row that is still inside this CTA's shared memory window
                dec.open(smem, cur.base, cur.base + cur.exp_bytes + 256u, lane);
                for (int g0 = 0; g0 < nblk; g0 += kGroup) {
                    const bool last = g0 + kGroup >= nblk;
#pragma unroll
                    for (int j = 0; j < kGroup; j++) {
                        if (!last) r_nxt[j] = (g0 + kGroup + j < nblk) ? __ldg(rem + (g0 + kGroup + j) * 32) : 0u;
                        else r_nxt[j] = (nxt.valid && j < nblk) ? __ldg(rem_next + j * 32) : 0u;
                    }
                    auto step = [&](int j) {
                        uint32_t e0, e1;
                        dec.pairs(smem, k, tab, lane4, copy_off, e0, e1);
                        const uint32_t r = r_cur[j];
                        sink.put(k, gblk0 + g0 + j, bitselect(prmt(r, 0u, 0x1100u), e0, kRemMask),
                                 bitselect(prmt(r, 0u, 0x3322u), e1, kRemMask));
                    };
                    if (g0 + kGroup <= nblk) {
#pragma unroll
                        for (int j = 0; j < kGroup; j++) step(j);
                    } else {
#pragma unroll
                        for (int j = 0; j < kGroup; j++)
                            if (g0 + j < nblk) step(j);
                    }
                    dec.clamp();
#pragma unroll
                    for (int j = 0; j < kGroup; j++) r_cur[j] = r_nxt[j];
                }
                next_first = nxt.valid;
            } else if (lane == 0) {
                atomicExch(&g_staged_status, 1);
            }
        } else {
            // direct record: on-demand global loads with a bounds guard, table-exact decoders
            typename Codec::template Stream<GlobalWords> s0, s1;
            s0.init(GlobalWords{L.exp, L.exp_words, static_cast<int64_t>(cur.off) + lane});
            s1.init(GlobalWords{L.exp, L.exp_words, static_cast<int64_t>(cur.off) + 32 + lane});
            for (int blk = 0; blk < nblk; blk++) {
                const uint32_t r = __ldg(rem + blk * 32);
                const uint32_t a0 = s0.next(tab);
                const uint32_t b0 = s1.next(tab);
                const uint32_t a1 = s0.next(tab);
                const uint32_t b1 = s1.next(tab);
                sink.put(k, gblk0 + blk, join_pair<0>(r, (a0 << 7) | (a1 << 23)), join_pair<1>(r, (b0 << 7) | (b1 << 23)));
            }
        }
        have_first = next_first;
        if (kPart) {
            if (split || cur.k == L.S - 1) sink.finish_part(part, cur.m - row_lo, split ? cur.k : 0, rows_cta, slots, lane);
        } else if (cur.k == L.S - 1) {
            sink.finish_row(cur.m, lane);
        }
        __syncwarp();
        if (nxt.valid && nxt.staged && !early) issue(nxt, slot ^ 1);
        cur = nxt;
        slot ^= 1;
    }
    if (kPart) {
        __syncthreads();
        sink.combine(part, row_lo, rows_cta, slots, lane);
    }
    sink.finish_kernel();
}

// ---- host side -------------------------------------------------------------------------------------
bool overlap_launches();     // process-wide switch, see bhi_set_launch_overlap

template <class K>
static int staged_prepare(K kernel) {
    // Opt in to the large dynamic shared-memory carve-out once per device and kernel.  Keyed by the
    // kernel's address: instantiations that differ only in a non-type argument share their pointer type.
    static std::mutex mu;
    static std::unordered_map<const void *, uint64_t> done;      // kernel -> bit per device
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return BHI_ERR_CUDA;
    const void *key = reinterpret_cast<const void *>(kernel);
    std::lock_guard<std::mutex> lock(mu);
    uint64_t &bits = done[key];
    if (!(bits >> dev & 1u)) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax);
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(shared memory)");
        bits |= 1ull << dev;
    }
    return BHI_OK;
}

static bool staged_shape_ok(const Layer &L) { return aligned(L.rem, 16) && aligned(L.exp, 16); }


// blob = folded pair table (one copy), exact tables, then one word: how many folded entries do not
// resolve two symbols (0 lets the fused kernel run its loop without the per-step test)
__global__ void __launch_bounds__(1024) huffman_prepare_kernel(HuffArgs targs, uint8_t *blob) {
    __shared__ HuffTables tab;
    __shared__ uint32_t flagged;
    if (threadIdx.x == 0) flagged = 0u;
    load_tables(tab, targs, threadIdx.x, blockDim.x);
    __syncthreads();
    uint32_t mine = 0;
    for (int v = threadIdx.x; v < kPairEntries; v += blockDim.x) {
        const uint32_t e = pair_entry(tab, v);
        reinterpret_cast<uint32_t *>(blob)[v] = e;
        mine += (e & (kEntSingle | kEntExact)) ? 1u : 0u;
    }
    if (mine) atomicAdd(&flagged, mine);
    __syncthreads();
    uint32_t *dst = reinterpret_cast<uint32_t *>(blob + kPairEntries * 4);
    const uint32_t *src = reinterpret_cast<const uint32_t *>(&tab);
    constexpr int kTabWords = static_cast<int>(sizeof(HuffTables) / 4);
    for (int i = threadIdx.x; i < kExactBytes / 4; i += blockDim.x)
        dst[i] = i < kTabWords ? src[i] : (i == kTabWords ? flagged : 0u);
}

template <class Codec, class Sink, int NW>
static int staged_launch(const Layer &L, const typename Codec::Args &targs, const uint8_t *prepared, const Sink &sink,
                         uint32_t x_bytes, cudaStream_t st) {
    int grid = sm_count();
    if (grid > L.M) grid = L.M;
    // Work is split by (row, chunk) records when a CTA has fewer rows than warps and rows have several
    // chunks; results are then (and for sinks that ask for it) staged in shared memory, if they fit.
    const int rows_cta = (L.M + grid - 1) / grid;
    // (measured: with more than half the warps holding a row of their own, whole rows are faster)
    int split = (Sink::kBatch > 0 && L.S > 1 && 2 * rows_cta <= NW) ? 1 : 0;
    uint32_t part_bytes = 0;
    if (split || Sink::kStagesResults) {
        part_bytes = ((static_cast<uint32_t>(Sink::kBatch) * rows_cta * (split ? L.S : 1) * 4u) + 255u) & ~255u;
        if (part_bytes > kPartMax) {
            part_bytes = 0;
            split = 0;
        }
    }
    auto kernel = part_bytes ? staged_kernel<Codec, Sink, NW, true> : staged_kernel<Codec, Sink, NW, false>;
    if (int rc = staged_prepare(kernel)) return rc;
    const uint32_t avail = kSmemMax - kHeaderBytes - kSlackBytes - x_bytes - part_bytes;
    uint32_t ring_bytes = (avail / NW) & ~255u;
    if (ring_bytes > kRingMax) ring_bytes = kRingMax;
    const uint32_t smem_bytes = kHeaderBytes + x_bytes + part_bytes + NW * ring_bytes + kSlackBytes;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(NW * 32);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap_launches() ? 1 : 0;
    const uint32_t ans_bits = ans_bits_of(targs);
    const Consts k{ans_bits, (1u << ans_bits) - 1u, 1u, 8u, 4u * kCopies, 65536u};
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, L, targs, prepared, sink, x_bytes, ring_bytes, k, part_bytes, split);
    return e == cudaSuccess ? BHI_OK : cuda_fail(e, "staged kernel launch");
}

template <class Codec, int B>
static int staged_gemv_b(const Layer &L, const typename Codec::Args &targs, const uint8_t *prepared, const uint16_t *X,
                         uint16_t *Y, cudaStream_t st) {
    constexpr int NW = B <= 4 ? 32 : 16;      // measured: batches 5..8 are faster with 16 warps of twice the registers
    const int64_t K = static_cast<int64_t>(L.S) * L.Nc;
    const int64_t x_need = ((static_cast<int64_t>(B) * K * 2 + 255) / 256) * 256;
    if (x_need <= (NW == 16 ? kXStageMax16 : kXStageMax)) {
        GemvSink<B, true> sink{};
        sink.x = reinterpret_cast<const uint32_t *>(X);
        sink.row_pairs = K >> 1;
        sink.row_blocks = static_cast<int>(K >> 7);
        sink.Y = Y;
        sink.M = L.M;
        return staged_launch<Codec, GemvSink<B, true>, NW>(L, targs, prepared, sink, static_cast<uint32_t>(x_need), st);
    }
    GemvSink<B, false> sink{};
    sink.x = reinterpret_cast<const uint32_t *>(X);
    sink.row_pairs = K >> 1;
    sink.row_blocks = static_cast<int>(K >> 7);
    sink.Y = Y;
    sink.M = L.M;
    return staged_launch<Codec, GemvSink<B, false>, NW>(L, targs, prepared, sink, 0u, st);
}

template <class Codec>
static int staged_gemv(const Layer &L, const typename Codec::Args &targs, const uint8_t *prepared, const uint16_t *X,
                       uint16_t *Y, int B, cudaStream_t st) {
    if (!staged_shape_ok(L) || !aligned(prepared, 16)) return kStagedDeclined;
    switch (B) {
        case 1: return staged_gemv_b<Codec, 1>(L, targs, prepared, X, Y, st);
        case 2: return staged_gemv_b<Codec, 2>(L, targs, prepared, X, Y, st);
        case 3: return staged_gemv_b<Codec, 3>(L, targs, prepared, X, Y, st);
        case 4: return staged_gemv_b<Codec, 4>(L, targs, prepared, X, Y, st);
        case 5: return staged_gemv_b<Codec, 5>(L, targs, prepared, X, Y, st);
        case 6: return staged_gemv_b<Codec, 6>(L, targs, prepared, X, Y, st);
        case 7: return staged_gemv_b<Codec, 7>(L, targs, prepared, X, Y, st);
        case 8: return staged_gemv_b<Codec, 8>(L, targs, prepared, X, Y, st);
    }
    return kStagedDeclined;
}

template <class Codec, int B>
static int staged_exchange_b(const Layer &L, const typename Codec::Args &targs, const uint8_t *prepared, const uint16_t *X,
                             const PeerSet &peers, cudaStream_t st) {
    constexpr int NW = B <= 4 ? 32 : 16;      // measured: batches 5..8 are faster with 16 warps of twice the registers
    const int64_t K = static_cast<int64_t>(L.S) * L.Nc;
    const int64_t x_need = ((static_cast<int64_t>(B) * K * 2 + 255) / 256) * 256;
    auto fill = [&](auto &sink) {
        sink.x = reinterpret_cast<const uint32_t *>(X);
        sink.row_pairs = K >> 1;
        sink.row_blocks = static_cast<int>(K >> 7);
        sink.Y = nullptr;
        sink.M = L.M;
        sink.peers = peers;
    };
    if (x_need <= (NW == 16 ? kXStageMax16 : kXStageMax)) {
        ExchangeSink<B, true> sink{};
        fill(sink);
        return staged_launch<Codec, ExchangeSink<B, true>, NW>(L, targs, prepared, sink, static_cast<uint32_t>(x_need), st);
    }
    ExchangeSink<B, false> sink{};
    fill(sink);
    return staged_launch<Codec, ExchangeSink<B, false>, NW>(L, targs, prepared, sink, 0u, st);
}

template <class Codec>
static int staged_exchange(const Layer &L, const typename Codec::Args &targs, const uint8_t *prepared, const uint16_t *X,
                           const PeerSet &peers, int B, cudaStream_t st) {
    switch (B) {
        case 1: return staged_exchange_b<Codec, 1>(L, targs, prepared, X, peers, st);
        case 2: return staged_exchange_b<Codec, 2>(L, targs, prepared, X, peers, st);
        case 3: return staged_exchange_b<Codec, 3>(L, targs, prepared, X, peers, st);
        case 4: return staged_exchange_b<Codec, 4>(L, targs, prepared, X, peers, st);
        case 5: return staged_exchange_b<Codec, 5>(L, targs, prepared, X, peers, st);
        case 6: return staged_exchange_b<Codec, 6>(L, targs, prepared, X, peers, st);
        case 7: return staged_exchange_b<Codec, 7>(L, targs, prepared, X, peers, st);
        case 8: return staged_exchange_b<Codec, 8>(L, targs, prepared, X, peers, st);
    }
    return kStagedDeclined;
}

template <class Codec>
static int staged_decode(const Layer &L, const typename Codec::Args &targs, const uint8_t *prepared, uint16_t *Y,
                         cudaStream_t st) {
    if (!staged_shape_ok(L) || !aligned(prepared, 16)) return kStagedDeclined;
    DenseSink sink{};
    sink.out = reinterpret_cast<uint32_t *>(Y);
    sink.row_pairs = (static_cast<int64_t>(L.S) * L.Nc) >> 1;
    sink.row = nullptr;
    return staged_launch<Codec, DenseSink, 32>(L, targs, prepared, sink, 0u, st);
}

}  // namespace bhi
