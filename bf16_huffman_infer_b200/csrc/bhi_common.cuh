// Shared device helpers: BF16 reassembly, the two exponent decoders in their table-exact form,
// and small host utilities.  sm_100a only.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/bf16_huffman_b200.h"

namespace bhi {

constexpr int kAnsBitsMin = 8;                    // probability precision of an rANS table: 2^bits slots
constexpr int kAnsBitsMax = BHI_ANS_MAX_PRECISION;
constexpr int kStreamsPerRecord = 64;   // 2 per lane: stream lane (first 64 columns of a block) and lane+32

// ---- host side ---------------------------------------------------------------------------------
void set_error(const std::string &msg);
int fail(int code, const std::string &msg);
int cuda_fail(cudaError_t e, const char *what);
int sm_count();          // of the current device, cached

#define BHI_REQUIRE(cond, msg) \
    do { if (!(cond)) return ::bhi::fail(BHI_ERR_ARG, std::string(msg) + " [" #cond "]"); } while (0)

inline bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// ---- device side -------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// Two BF16 values from two sign+mantissa bytes and two exponents already placed at bits 7..14 and
// 23..30.  `r` is the little-endian word of the four bytes (h0,t0) (h0,t1) (h1,t0) (h1,t1) a lane
// owns in a 128-column block; `half` picks h.  Per 16-bit lane: bit 15 = sign, bits 14..7 =
// exponent, bits 6..0 = mantissa (reference src/kernel.cu:149-160).
template <int half>
__device__ __forceinline__ uint32_t join_pair(uint32_t r, uint32_t exp_at_7_and_23) {
    uint32_t doubled = prmt(r, 0u, half == 0 ? 0x1100u : 0x3322u);   // bytes: a a b b
    return (doubled & 0x807F807Fu) | exp_at_7_and_23;
}

__device__ __forceinline__ float bf16lo_to_f32(uint32_t pair) { return __uint_as_float(pair << 16); }
__device__ __forceinline__ float bf16hi_to_f32(uint32_t pair) { return __uint_as_float(pair & 0xFFFF0000u); }

__device__ __forceinline__ uint16_t f32_to_bf16_rn(float f) {
    uint16_t h;
    asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(h) : "f"(f));
    return h;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

// ---- table-exact decoders (generic path and the slow lane of the staged path) ---------------------
// Huffman: four byte-indexed tables + length table, reference src/kernel.cu:313-319, 354-380.
struct HuffTables {
    uint8_t lut[4][256];
    uint8_t len[256];
};

struct HuffArgs {
    const uint8_t *lut1, *lut2, *lut3, *lut4, *len;
};

__device__ __forceinline__ void load_tables(HuffTables &t, const HuffArgs &a, int tid, int nthreads) {
    for (int i = tid; i < 256; i += nthreads) {
        t.lut[0][i] = a.lut1[i];
        t.lut[1][i] = a.lut2[i];
        t.lut[2][i] = a.lut3[i];
        t.lut[3][i] = a.lut4[i];
        t.len[i] = a.len[i];
    }
}

__device__ __forceinline__ uint32_t huff_cascade(const HuffTables &t, uint32_t window) {
    uint32_t s = t.lut[0][window & 0xFF];
    if (s == 255) s = t.lut[1][(window >> 8) & 0xFF];
    if (s == 255) s = t.lut[2][(window >> 16) & 0xFF];
    if (s == 255) s = t.lut[3][window >> 24];
    return s;
}

// Word source over global memory with a hard upper bound: words past the buffer read as zero.
struct GlobalWords {
    const uint32_t *base;
    int64_t limit;
    int64_t at;     // next word of this stream (stride 64)
    __device__ __forceinline__ uint32_t pop() {
        uint32_t v = (at < limit) ? __ldg(base + at) : 0u;
        at += kStreamsPerRecord;
        return v;
    }
};

template <class Words>
struct HuffStream {
    Words src;
    uint64_t win;
    uint32_t have;
    __device__ __forceinline__ void init(const Words &w) { src = w; win = 0; have = 0; }
    __device__ __forceinline__ uint32_t next(const HuffTables &t) {
        if (have < 32) {
            win |= static_cast<uint64_t>(src.pop()) << have;
            have += 32;
        }
        uint32_t s = huff_cascade(t, static_cast<uint32_t>(win));
        uint32_t n = t.len[s];
        win >>= n;
        have -= n;
        return s;
    }
};

// rANS: one table word per slot = sym<<24 | freq<<12 | (slot - cum[sym]), reference
// src/kernel.cu:647-683.  The table has 2^bits slots (the reference fixes bits = 8; its word layout and
// its static_assert allow up to 12).  The table-exact decoder reads the caller's table in global memory.
struct AnsTables {
    const uint32_t *lut;
    uint32_t bits;
};

struct AnsArgs {
    const uint32_t *lut;
    int bits;
};

__device__ __forceinline__ void load_tables(AnsTables &t, const AnsArgs &a, int tid, int) {
    if (tid == 0) {
        t.lut = a.lut;
        t.bits = static_cast<uint32_t>(a.bits);
    }
}

template <class Words>
struct AnsStream {
    Words src;
    uint64_t state;
    __device__ __forceinline__ void init(const Words &w) { src = w; state = src.pop(); }
    __device__ __forceinline__ uint32_t next(const AnsTables &t) {
        if (state < (1ull << t.bits)) state = (state << 32) | src.pop();
        uint32_t e = __ldg(t.lut + (static_cast<uint32_t>(state) & ((1u << t.bits) - 1u)));
        state = static_cast<uint64_t>((e >> 12) & 0xFFFu) * (state >> t.bits) + (e & 0xFFFu);
        return e >> 24;
    }
};

// probability precision carried by a codec's table arguments (Huffman: unused)
__host__ __device__ inline uint32_t ans_bits_of(const HuffArgs &) { return kAnsBitsMin; }
__host__ __device__ inline uint32_t ans_bits_of(const AnsArgs &a) { return static_cast<uint32_t>(a.bits); }

struct HuffCodec {
    using Tables = HuffTables;
    using Args = HuffArgs;
    template <class W> using Stream = HuffStream<W>;
};
struct AnsCodec {
    using Tables = AnsTables;
    using Args = AnsArgs;
    template <class W> using Stream = AnsStream<W>;
};

// Geometry shared by every decode-side kernel.
struct Layer {
    const uint8_t *rem;        // [S, M, Nc]
    const uint32_t *exp;       // [exp_words]
    int64_t exp_words;
    const int32_t *offsets;    // [S, M]
    int S, M, Nc;
};

}  // namespace bhi
