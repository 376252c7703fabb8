// Encode-side kernels.  Two families:
//  * the two per-stream operators of the reference (character / word output, one thread per
//    stream, reference src/kernel.cu:590-610 and :767-811), kept for operator compatibility;
//  * the whole-layer two-pass encoder that writes the device format directly from the BF16
//    weight: one thread per stream, 64 consecutive threads per record, so that the BF16 reads
//    (2 columns per thread, 256 B per record and block) and the interleaved word stores
//    (64 words per record row) are coalesced.
#pragma once

#include "bhi_common.cuh"

namespace bhi {

// ---- operator-compatible per-stream encoders ------------------------------------------------------
__global__ void huffman_encode_chars_kernel(const uint8_t *__restrict__ data, int streams, int n,
                                            const uint8_t *__restrict__ lut, uint8_t *__restrict__ out,
                                            int32_t *__restrict__ out_len) {
    __shared__ uint8_t codes[256 * 32];
    for (int i = threadIdx.x; i < 256 * 32; i += blockDim.x) codes[i] = lut[i];
    __syncthreads();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= streams) return;
    const uint8_t *src = data + static_cast<int64_t>(t) * n;
    uint8_t *dst = out + static_cast<int64_t>(t) * n * 32;
    int32_t cnt = 0;
    for (int i = 0; i < n; i++) {
        const uint8_t *c = codes + 32 * src[i];
        for (int j = 0; j < 32 && c[j] != 0; j++) dst[cnt++] = c[j];
    }
    out_len[t] = cnt;
}

// Probability precision of an rANS model: its frequencies sum to 2^bits (cum[255] + freq[255] is that sum).
__device__ __forceinline__ uint32_t ans_model_bits(const uint32_t *sf, const uint32_t *sc) {
    const uint32_t total = sc[255] + sf[255];
    return total ? 31u - static_cast<uint32_t>(__clz(total)) : kAnsBitsMin;
}

// rANS step shared by all encoders: emits renormalisation words through `put(word)`.
template <class Put>
__device__ __forceinline__ void ans_push(uint64_t &state, uint32_t f, uint32_t c, uint32_t bits, Put &&put) {
    while ((state >> 32) >= f) {
        put(static_cast<uint32_t>(state));
        state >>= 32;
    }
    state = ((state / f) << bits) + (state % f) + c;
}

__global__ void ans_encode_words_kernel(const uint8_t *__restrict__ data, int streams, int n,
                                        const uint32_t *__restrict__ freq, const uint32_t *__restrict__ cum,
                                        uint32_t *__restrict__ out, int32_t *__restrict__ out_len) {
    __shared__ uint32_t sf[256], sc[256];
    for (int i = threadIdx.x; i < 256; i += blockDim.x) { sf[i] = freq[i]; sc[i] = cum[i]; }
    __syncthreads();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= streams) return;
    const uint8_t *src = data + static_cast<int64_t>(t) * n;
    uint32_t *dst = out + static_cast<int64_t>(t) * n * 8;
    const uint32_t bits = ans_model_bits(sf, sc);
    uint64_t state = 1ull << bits;
    int32_t cnt = 0;
    auto put = [&](uint32_t w) { dst[cnt++] = w; };
    for (int i = n - 1; i >= 0; i--) ans_push(state, sf[src[i]], sc[src[i]], bits, put);
    while (state > 0) { put(static_cast<uint32_t>(state)); state >>= 32; }
    for (int i = 0; i < cnt / 2; i++) {
        const uint32_t a = dst[i];
        dst[i] = dst[cnt - 1 - i];
        dst[cnt - 1 - i] = a;
    }
    out_len[t] = cnt;
}

// ---- whole-layer encoder ---------------------------------------------------------------------------
constexpr int kEncThreads = 256;                 // 4 records per block
constexpr int kEncRecords = kEncThreads / 64;

struct EncGeom {
    const uint16_t *W;     // [M, K]
    int M, K, S, Nc;
};

// thread -> (record, stream); returns false past the end
__device__ __forceinline__ bool enc_locate(const EncGeom &g, int64_t &rec, int &k, int &m, int &st) {
    rec = static_cast<int64_t>(blockIdx.x) * kEncRecords + (threadIdx.x >> 6);
    st = threadIdx.x & 63;
    if (rec >= static_cast<int64_t>(g.S) * g.M) return false;
    k = static_cast<int>(rec / g.M);
    m = static_cast<int>(rec - static_cast<int64_t>(k) * g.M);
    return true;
}

// the two BF16 values (as one u32) a stream owns in block `blk` of its record
__device__ __forceinline__ uint32_t enc_pair(const EncGeom &g, int k, int m, int st, int blk) {
    const uint16_t *p = g.W + static_cast<int64_t>(m) * g.K + static_cast<int64_t>(k) * g.Nc + blk * 128 + 2 * st;
    return __ldg(reinterpret_cast<const uint32_t *>(p));
}
__device__ __forceinline__ uint32_t exp_lo(uint32_t pair) { return (pair >> 7) & 0xFF; }
__device__ __forceinline__ uint32_t exp_hi(uint32_t pair) { return (pair >> 23) & 0xFF; }

// max over the 64 threads of a record (two warps) -> every thread of the record gets it
__device__ __forceinline__ uint32_t record_max(uint32_t v, uint32_t *scratch /*[kEncThreads/32]*/) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = max(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    const int w = threadIdx.x >> 5;
    if ((threadIdx.x & 31) == 0) scratch[w] = v;
    __syncthreads();
    return max(scratch[w & ~1], scratch[w | 1]);
}

__global__ void __launch_bounds__(kEncThreads)
huffman_size_kernel(EncGeom g, const uint8_t *__restrict__ code_len, int32_t *__restrict__ words_per_row) {
    __shared__ uint8_t len[256];
    __shared__ uint32_t scratch[kEncThreads / 32];
    for (int i = threadIdx.x; i < 256; i += blockDim.x) len[i] = code_len[i];
    __syncthreads();
    int64_t rec; int k, m, st;
    const bool live = enc_locate(g, rec, k, m, st);
    uint32_t bits = 0;
    if (live)
        for (int blk = 0; blk < (g.Nc >> 7); blk++) {
            const uint32_t p = enc_pair(g, k, m, st, blk);
            bits += len[exp_lo(p)] + len[exp_hi(p)];
        }
    const uint32_t worst = record_max(bits, scratch);
    if (live && st == 0) words_per_row[rec] = static_cast<int32_t>(((worst + 7) / 8 + 3) / 4);
}

__device__ __forceinline__ void store_rem(uint8_t *rem_row, int st, int blk, uint32_t pair) {
    // stream st = h*32 + lane owns bytes blk*128 + lane*4 + h*2 + {0,1} (reference functional.py:184)
    const uint32_t lo = ((pair >> 8) & 0x80) | (pair & 0x7F);
    const uint32_t hi = ((pair >> 24) & 0x80) | ((pair >> 16) & 0x7F);
    *reinterpret_cast<uint16_t *>(rem_row + blk * 128 + (st & 31) * 4 + (st >> 5) * 2) = static_cast<uint16_t>(lo | (hi << 8));
}

__global__ void __launch_bounds__(kEncThreads)
huffman_emit_kernel(EncGeom g, const uint8_t *__restrict__ code_len, const uint32_t *__restrict__ code_val,
                    const int32_t *__restrict__ offsets, uint8_t *__restrict__ rem, uint32_t *__restrict__ exp) {
    __shared__ uint8_t len[256];
    __shared__ uint32_t val[256];
    for (int i = threadIdx.x; i < 256; i += blockDim.x) { len[i] = code_len[i]; val[i] = code_val[i]; }
    __syncthreads();
    int64_t rec; int k, m, st;
    if (!enc_locate(g, rec, k, m, st)) return;
    uint8_t *rem_row = rem + rec * g.Nc;
    uint32_t *out = exp + static_cast<uint32_t>(offsets[rec]) + st;
    uint64_t acc = 0;
    uint32_t have = 0;
    for (int blk = 0; blk < (g.Nc >> 7); blk++) {
        const uint32_t p = enc_pair(g, k, m, st, blk);
        store_rem(rem_row, st, blk, p);
#pragma unroll
        for (int t = 0; t < 2; t++) {
            const uint32_t e = t ? exp_hi(p) : exp_lo(p);
            acc |= static_cast<uint64_t>(val[e]) << have;
            have += len[e];
            if (have >= 32) {
                *out = static_cast<uint32_t>(acc);
                out += kStreamsPerRecord;
                acc >>= 32;
                have -= 32;
            }
        }
    }
    if (have > 0) *out = static_cast<uint32_t>(acc);
}

// rANS over one stream of a record, symbols last to first; `put` sees words in emission order.
template <class Put>
__device__ __forceinline__ void ans_encode_record_stream(const EncGeom &g, int k, int m, int st,
                                                         const uint32_t *sf, const uint32_t *sc, Put &&put) {
    const uint32_t bits = ans_model_bits(sf, sc);
    uint64_t state = 1ull << bits;
    for (int blk = (g.Nc >> 7) - 1; blk >= 0; blk--) {
        const uint32_t p = enc_pair(g, k, m, st, blk);
        const uint32_t e1 = exp_hi(p), e0 = exp_lo(p);
        ans_push(state, sf[e1], sc[e1], bits, put);
        ans_push(state, sf[e0], sc[e0], bits, put);
    }
    while (state > 0) { put(static_cast<uint32_t>(state)); state >>= 32; }
}

__global__ void __launch_bounds__(kEncThreads)
ans_size_kernel(EncGeom g, const uint32_t *__restrict__ freq, const uint32_t *__restrict__ cum,
                int32_t *__restrict__ words_per_row, uint8_t *__restrict__ stream_words) {
    __shared__ uint32_t sf[256], sc[256];
    __shared__ uint32_t scratch[kEncThreads / 32];
    for (int i = threadIdx.x; i < 256; i += blockDim.x) { sf[i] = freq[i]; sc[i] = cum[i]; }
    __syncthreads();
    int64_t rec; int k, m, st;
    const bool live = enc_locate(g, rec, k, m, st);
    uint32_t cnt = 0;
    if (live) {
        ans_encode_record_stream(g, k, m, st, sf, sc, [&](uint32_t) { cnt++; });
        stream_words[rec * 64 + st] = static_cast<uint8_t>(cnt);
    }
    const uint32_t worst = record_max(cnt, scratch);
    if (live && st == 0) words_per_row[rec] = static_cast<int32_t>(worst);
}

__global__ void __launch_bounds__(kEncThreads)
ans_emit_kernel(EncGeom g, const uint32_t *__restrict__ freq, const uint32_t *__restrict__ cum,
                const int32_t *__restrict__ offsets, const uint8_t *__restrict__ stream_words,
                uint8_t *__restrict__ rem, uint32_t *__restrict__ exp) {
    __shared__ uint32_t sf[256], sc[256];
    for (int i = threadIdx.x; i < 256; i += blockDim.x) { sf[i] = freq[i]; sc[i] = cum[i]; }
    __syncthreads();
    int64_t rec; int k, m, st;
    if (!enc_locate(g, rec, k, m, st)) return;
    uint8_t *rem_row = rem + rec * g.Nc;
    for (int blk = 0; blk < (g.Nc >> 7); blk++) store_rem(rem_row, st, blk, enc_pair(g, k, m, st, blk));
    // the j-th emitted word is the (cnt-1-j)-th word the decoder reads
    uint32_t *out = exp + static_cast<uint32_t>(offsets[rec]) + st;
    int at = static_cast<int>(stream_words[rec * 64 + st]) - 1;
    ans_encode_record_stream(g, k, m, st, sf, sc, [&](uint32_t w) {
        if (at >= 0) out[static_cast<int64_t>(at) * kStreamsPerRecord] = w;
        at--;
    });
}

}  // namespace bhi
