// Generic decode-side kernels: one warp per record, exponent words fetched on demand from global
// memory with a bounds guard, table-exact decoders.  They accept every shape the format allows
// and are the fallback of the staged kernels (records too large for the shared-memory ring,
// unaligned buffers).  Semantics follow reference src/kernel.cu:46-310.
#pragma once

#include "bhi_common.cuh"

namespace bhi {

constexpr int kGenericThreads = 256;

// Y[b, m] for b < B.  One warp owns a whole output row: it walks the S chunk records of the row in
// order, so the K-split needs no cross-warp combine and the summation order is fixed.
template <class Codec, int B>
__global__ void __launch_bounds__(kGenericThreads)
gemv_generic_kernel(Layer L, typename Codec::Args targs, const uint16_t *__restrict__ X, uint16_t *__restrict__ Y) {
    __shared__ typename Codec::Tables tab;
    load_tables(tab, targs, threadIdx.x, blockDim.x);
    __syncthreads();

    const int lane = threadIdx.x & 31;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int nwarps = (gridDim.x * blockDim.x) >> 5;
    const int64_t K = static_cast<int64_t>(L.S) * L.Nc;
    const int nblk = L.Nc >> 7;

    for (int m = warp; m < L.M; m += nwarps) {
        float acc[B];
#pragma unroll
        for (int b = 0; b < B; b++) acc[b] = 0.f;

        for (int k = 0; k < L.S; k++) {
            const int64_t rec = static_cast<int64_t>(k) * L.M + m;
            const uint32_t *rem = reinterpret_cast<const uint32_t *>(L.rem + rec * L.Nc);
            const int64_t off = static_cast<uint32_t>(L.offsets[rec]);
            typename Codec::template Stream<GlobalWords> s0, s1;
            s0.init(GlobalWords{L.exp, L.exp_words, off + lane});
            s1.init(GlobalWords{L.exp, L.exp_words, off + 32 + lane});
            const uint32_t *x = reinterpret_cast<const uint32_t *>(X + static_cast<int64_t>(k) * L.Nc) + lane;

            for (int blk = 0; blk < nblk; blk++) {
                const uint32_t r = __ldg(rem + blk * 32 + lane);
                // decode order of the reference: stream0, stream1, stream0, stream1
                const uint32_t a0 = s0.next(tab);
                const uint32_t b0 = s1.next(tab);
                const uint32_t a1 = s0.next(tab);
                const uint32_t b1 = s1.next(tab);
                const uint32_t w0 = join_pair<0>(r, (a0 << 7) | (a1 << 23));
                const uint32_t w1 = join_pair<1>(r, (b0 << 7) | (b1 << 23));
                const float w00 = bf16lo_to_f32(w0), w01 = bf16hi_to_f32(w0);
                const float w10 = bf16lo_to_f32(w1), w11 = bf16hi_to_f32(w1);
#pragma unroll
                for (int b = 0; b < B; b++) {
                    const uint32_t x0 = __ldg(x + (b * K >> 1) + blk * 64);
                    const uint32_t x1 = __ldg(x + (b * K >> 1) + blk * 64 + 32);
                    acc[b] += (w00 * bf16lo_to_f32(x0) + w01 * bf16hi_to_f32(x0)) +
                              (w10 * bf16lo_to_f32(x1) + w11 * bf16hi_to_f32(x1));
                }
            }
        }
#pragma unroll
        for (int b = 0; b < B; b++) {
            const float v = warp_sum(acc[b]);
            if (lane == 0) Y[static_cast<int64_t>(b) * L.M + m] = f32_to_bf16_rn(v);
        }
    }
}

// Dense BF16 [M, S*Nc]; one warp per record (k, m), grid-stride.
template <class Codec>
__global__ void __launch_bounds__(kGenericThreads)
decode_generic_kernel(Layer L, typename Codec::Args targs, uint16_t *__restrict__ Y) {
    __shared__ typename Codec::Tables tab;
    load_tables(tab, targs, threadIdx.x, blockDim.x);
    __syncthreads();

    const int lane = threadIdx.x & 31;
    const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    const int64_t K = static_cast<int64_t>(L.S) * L.Nc;
    const int nblk = L.Nc >> 7;
    const int64_t nrec = static_cast<int64_t>(L.S) * L.M;

    for (int64_t rec = warp; rec < nrec; rec += nwarps) {
        const int k = static_cast<int>(rec / L.M);
        const int m = static_cast<int>(rec - static_cast<int64_t>(k) * L.M);
        const uint32_t *rem = reinterpret_cast<const uint32_t *>(L.rem + rec * L.Nc);
        const int64_t off = static_cast<uint32_t>(L.offsets[rec]);
        typename Codec::template Stream<GlobalWords> s0, s1;
        s0.init(GlobalWords{L.exp, L.exp_words, off + lane});
        s1.init(GlobalWords{L.exp, L.exp_words, off + 32 + lane});
        uint32_t *out = reinterpret_cast<uint32_t *>(Y + static_cast<int64_t>(m) * K + static_cast<int64_t>(k) * L.Nc) + lane;
        for (int blk = 0; blk < nblk; blk++) {
            const uint32_t r = __ldg(rem + blk * 32 + lane);
            const uint32_t a0 = s0.next(tab);
            const uint32_t b0 = s1.next(tab);
            const uint32_t a1 = s0.next(tab);
            const uint32_t b1 = s1.next(tab);
            out[blk * 64] = join_pair<0>(r, (a0 << 7) | (a1 << 23));
            out[blk * 64 + 32] = join_pair<1>(r, (b0 << 7) | (b1 << 23));
        }
    }
}

}  // namespace bhi
