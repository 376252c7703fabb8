/*
 * C ABI of the B200 (sm_100a) kernels for exponent-coded BF16 linear layers.
 *
 * Plain pointers and sizes only; every pointer is a DEVICE pointer unless said otherwise.  All
 * entry points enqueue work on `stream` (a cudaStream_t passed as void*) of the CURRENT CUDA
 * device and return without synchronising, so they may be called while the stream is being
 * captured into a CUDA graph.  None of them allocates memory.  Return value: 0 on success, a
 * BHI_ERR_* code otherwise; bhi_last_error() then returns a message for the calling thread.
 *
 * Each entry point replaces one operator of the reference project's torch extension
 * (lszxb/bf16_huffman_infer; paths below are relative to that project).  The compressed
 * format is the reference's: see bf16_huffman_infer/functional.py:161-238.
 *
 *   A_rem    u8  [split_k, M, Nc]   sign+mantissa bytes, permuted per 128-column block
 *   A_exp    u32 [exp_words]        entropy-coded exponents, 64 interleaved streams per record
 *   offsets  i32 [split_k, M]       first word of the record of (chunk, row)
 *   X        bf16 [batch, split_k*Nc]   activations (row-major)
 *   Y        bf16 [batch, M]        (gemv)   or   bf16 [M, split_k*Nc]  (decode)
 *   Nc % 128 == 0, 128 <= Nc <= 16384, 1 <= split_k, 1 <= batch <= 8.
 */
#ifndef BF16_HUFFMAN_B200_H_
#define BF16_HUFFMAN_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BHI_OK 0
#define BHI_ERR_ARG 1      /* a size, pointer or alignment the kernels do not accept */
#define BHI_ERR_CUDA 2     /* a CUDA runtime call failed (message holds cudaGetErrorString) */
#define BHI_ERR_LIMIT 3    /* a size beyond a documented fixed limit */

#define BHI_MAX_BATCH 8            /* rows of X the fused GEMV accepts */
#define BHI_MAX_PEERS 8            /* ranks one exchange entry point can serve */
#define BHI_MAX_LINEAR_BATCH 128   /* rows of X the fused tensor-core product accepts */
#define BHI_ANS_PRECISION 8        /* the reference's probability precision (2^8 table slots) */
#define BHI_ANS_MAX_PRECISION 12   /* largest precision the kernels take (the table word has 12-bit fields) */

/* Message describing the last error returned on this thread ("" if none). */
const char *bhi_last_error(void);

/* ABI revision of this library. */
int bhi_abi_version(void);

/* Which implementation the gemv / decode entry points use:
 *   0 = automatic (the four-rows-per-warp-group kernel when the shape allows it, else the
 *       one-row-per-warp staged kernel, else the generic path)
 *   1 = generic path only (one warp per record, direct global loads)
 *   2 = skip the four-rows-per-warp-group kernel (one-row-per-warp staged kernel, else generic)
 * The linear entry points choose between their two kernels the same way: 0 = the one whose decoders stage records in
 * shared memory when the batch leaves room for them (up to about 48 rows), else the one that keeps its streams in
 * registers; 2 = the latter always.
 * Process-wide; meant for tests and A/B measurements.  Returns the previous value. */
int bhi_set_kernel_path(int path);

/* Warps per block of the four-rows-per-warp-group kernel: 32 (a lane decodes two streams), 16 (a lane
 * decodes four streams, twice the registers per thread) or 0 = chosen per call (16 for rANS and for Huffman
 * tables declared pair-complete, see bhi_huffman_table_hint; else 32).  Process-wide; returns the previous
 * value, -1 for any other argument.  For A/B measurements. */
int bhi_set_quad_warps(int warps);

/* Launch overlap (programmatic dependent launch), process-wide, off by default.  When on, a fused
 * kernel may begin while the previous kernel in the stream is still running: it reads the layer's
 * weight buffers, offsets and tables right away and waits for the previous kernel only before it
 * touches X and Y.  Turn it on only if the weight buffers are complete in memory before the call
 * is enqueued (written by an earlier synchronised operation or a memory copy, never by a kernel
 * still in flight on the same stream).  Returns the previous value. */
int bhi_set_launch_overlap(int on);

/* Reads and clears the device-side status word of the current device.  0 = no incident; otherwise
 * the last bounded wait that ran out inside a kernel: 1 a record's bulk copy (the record was
 * skipped), 2 the prepared-table copy, 3-7 the tensor-core path's stage / accumulator barriers,
 * 8 peers not ready and 9 peers not done in an exchange kernel.  The kernels always run to their
 * end.  Synchronises the device; meant for tests and post-mortems, not for the launch path. */
int bhi_debug_status(int *status_out);

/* Y[b, m] = sum_c X[b, c] * W[m, c] computed straight from the Huffman-coded weight.
 * Replaces torch.ops.bf16_huffman_infer.gemv_bf16_huffman
 * (bf16_huffman_infer/src/kernel.cu:445-507, schema src/bf16_huffman_infer.cpp:29). */
int bhi_gemv_bf16_huffman(const uint8_t *A_rem, const uint32_t *A_exp, int64_t exp_words,
                          const uint16_t *X, uint16_t *Y, const int32_t *offsets,
                          const uint8_t *LUT1, const uint8_t *LUT2, const uint8_t *LUT3,
                          const uint8_t *LUT4, const uint8_t *code_lengths,
                          int split_k, int M, int Nc, int batch, void *stream);

/* Dense BF16 weight [M, split_k*Nc] from the Huffman-coded form.
 * Replaces torch.ops.bf16_huffman_infer.huffman_decode (src/kernel.cu:534-587, schema .cpp:31). */
int bhi_huffman_decode(const uint8_t *A_rem, const uint32_t *A_exp, int64_t exp_words,
                       uint16_t *Y, const int32_t *offsets,
                       const uint8_t *LUT1, const uint8_t *LUT2, const uint8_t *LUT3,
                       const uint8_t *LUT4, const uint8_t *code_lengths,
                       int split_k, int M, int Nc, void *stream);

/* ---- prepared Huffman tables ---------------------------------------------------------------
 * The fused kernels do not decode with the four byte tables directly: they fold them into a
 * 4096-entry two-symbols-per-lookup table (kept in four bank-interleaved copies).  The two entry points above rebuild that table inside
 * every launch, which costs a few microseconds per call.  A caller that keeps a layer around can
 * fold the tables once into a blob of bhi_huffman_prepared_bytes() bytes (16-byte aligned device
 * memory owned by the caller) and pass the blob instead of the five tables; the kernels then
 * fetch it with a single bulk copy.  Results are identical.  No counterpart in the reference
 * (its kernels index the byte tables directly, src/kernel.cu:370-377). */
int bhi_huffman_prepared_bytes(void);
/* Tuning hint for a prepared blob (host-side bookkeeping, no device work): pair_complete != 0 declares that
 * no code of the table is longer than 6 bits, so that any two consecutive codes fit the 12-bit index of the
 * folded table.  The fused kernels pick their warp layout by it; results never depend on it (whether the
 * per-step test can be skipped is read from the blob itself).  bhi_huffman_prepare clears the hint of the
 * blob it writes; give the hint after preparing.  Thread-safe. */
int bhi_huffman_table_hint(const uint8_t *prepared, int pair_complete);
int bhi_huffman_prepare(const uint8_t *LUT1, const uint8_t *LUT2, const uint8_t *LUT3, const uint8_t *LUT4,
                        const uint8_t *code_lengths, uint8_t *prepared, void *stream);
int bhi_gemv_bf16_huffman_prepared(const uint8_t *A_rem, const uint32_t *A_exp, int64_t exp_words,
                                   const uint16_t *X, uint16_t *Y, const int32_t *offsets,
                                   const uint8_t *prepared, int split_k, int M, int Nc, int batch, void *stream);
int bhi_huffman_decode_prepared(const uint8_t *A_rem, const uint32_t *A_exp, int64_t exp_words,
                                uint16_t *Y, const int32_t *offsets, const uint8_t *prepared,
                                int split_k, int M, int Nc, void *stream);

/* Same two operations for the rANS-coded form; LUT is u32[2^precision] with
 * sym<<24 | freq<<12 | (slot - cum[sym]), BHI_ANS_PRECISION (8, the reference's constant) <= precision <=
 * BHI_ANS_MAX_PRECISION (12, what the 12-bit fields of the word allow; the reference's kernel asserts the
 * same bound, src/kernel.cu:695).  The encoders below take the precision from the model itself
 * (its frequencies sum to 2^precision).
 * Replace torch.ops.bf16_huffman_infer.gemv_bf16_ans (src/kernel.cu:714-764, schema .cpp:33)
 * and torch.ops.bf16_huffman_infer.ans_decode (src/kernel.cu:878-919, schema .cpp:35). */
int bhi_gemv_bf16_ans(const uint8_t *A_rem, const uint32_t *A_exp, int64_t exp_words,
                      const uint16_t *X, uint16_t *Y, const int32_t *offsets, const uint32_t *LUT, int precision,
                      int split_k, int M, int Nc, int batch, void *stream);
int bhi_ans_decode(const uint8_t *A_rem, const uint32_t *A_exp, int64_t exp_words,
                   uint16_t *Y, const int32_t *offsets, const uint32_t *LUT, int precision,
                   int split_k, int M, int Nc, void *stream);

/* ---- fused decode + tensor-core product for up to 128 rows of X -----------------------------
 * Y[b, m] = sum_c X[b, c] * W[m, c] for 1 <= batch <= BHI_MAX_LINEAR_BATCH (meant for 9..128; the
 * GEMV entry points are faster up to 8).  The reference has no operator for this range: it decodes
 * the weight to a dense scratch with huffman_decode / ans_decode and calls a library GEMM
 * (bf16_huffman_infer/functional.py:398-407, 469-478).  These entry points replace that pair of
 * calls: a set of weight rows is decoded into shared memory and multiplied there by tcgen05.mma
 * with the accumulator in tensor memory, so the dense weight never reaches HBM and no scratch is
 * needed.  Accumulation is FP32 over the whole row, one rounding to BF16 at the end.  X must be
 * 16-byte aligned.  Measured on B200: within 5 % of decode + library GEMM up to 32 rows, behind it
 * beyond. */
int bhi_linear_bf16_huffman(const uint8_t *A_rem, const uint32_t *A_exp, int64_t exp_words,
                            const uint16_t *X, uint16_t *Y, const int32_t *offsets,
                            const uint8_t *LUT1, const uint8_t *LUT2, const uint8_t *LUT3,
                            const uint8_t *LUT4, const uint8_t *code_lengths,
                            int split_k, int M, int Nc, int batch, void *stream);
int bhi_linear_bf16_huffman_prepared(const uint8_t *A_rem, const uint32_t *A_exp, int64_t exp_words,
                                     const uint16_t *X, uint16_t *Y, const int32_t *offsets,
                                     const uint8_t *prepared, int split_k, int M, int Nc, int batch, void *stream);
int bhi_linear_bf16_ans(const uint8_t *A_rem, const uint32_t *A_exp, int64_t exp_words,
                        const uint16_t *X, uint16_t *Y, const int32_t *offsets, const uint32_t *LUT, int precision,
                        int split_k, int M, int Nc, int batch, void *stream);

/* ---- row-sharded GEMV with the all-gather in its epilogue --------------------------------------
 * For a weight whose output rows are split over `world` GPUs of one node (one process per GPU):
 * this rank holds rows [row_base, row_base + M) of an [M_total, K] weight and computes
 * Y[b, row_base + m]; every rank needs all of Y afterwards.  These entry points store each result
 * straight into the Y buffer of every rank (y[r], peer-mapped device pointers, e.g. from CUDA IPC
 * or torch symmetric memory) and return only when, in stream order, all ranks' rows have arrived
 * in y[rank]: no collective call follows.  All ranks must call them for the same layer in the
 * same order.  No counterpart in the reference (single GPU).
 *
 * ready[r], done[r]: one u32 word per rank for THIS layer, in peer-mapped memory, zero before the
 * first call and never touched by the caller afterwards; launches: TWO consecutive u32 words in local
 * memory (the layer's launch counter, then the kernel's block-arrival counter), zero before the first
 * call.  Every rank signals each peer once per launch, whatever its grid, so the ranks may hold
 * different numbers of rows.  The kernel signals the peers that y may be overwritten only after
 * everything earlier in `stream` has finished, so consumers of Y must be ordered on the same
 * stream.  Waits on peers are bounded (one second each); if one runs out the status word is set
 * (bhi_debug_status) and Y is incomplete.  batch <= BHI_MAX_BATCH, world <= BHI_MAX_PEERS. */
typedef struct {
    int world, rank;
    int row_base, M_total;
    uint16_t *y[BHI_MAX_PEERS];       /* Y [batch, M_total] bf16 of every rank */
    uint32_t *ready[BHI_MAX_PEERS];
    uint32_t *done[BHI_MAX_PEERS];
    uint32_t *launches;
} bhi_exchange_t;
int bhi_gemv_bf16_huffman_exchange(const uint8_t *A_rem, const uint32_t *A_exp, int64_t exp_words,
                                   const uint16_t *X, const int32_t *offsets, const uint8_t *prepared,
                                   int split_k, int M, int Nc, int batch, const bhi_exchange_t *exchange, void *stream);
int bhi_gemv_bf16_ans_exchange(const uint8_t *A_rem, const uint32_t *A_exp, int64_t exp_words,
                               const uint16_t *X, const int32_t *offsets, const uint32_t *LUT, int precision,
                               int split_k, int M, int Nc, int batch, const bhi_exchange_t *exchange, void *stream);

/* Single-GPU form of bhi_gemv_bf16_huffman_exchange whose counter words live inside the library
 * (no counterpart in the reference).  Y [batch, M] is an ordinary output buffer; the counter
 * words of the exchange protocol (ready, done, launches, block arrivals) are taken from a file-scope device array of
 * BHI_STATIC_EXCHANGE_LAYERS entries of 256 bytes (256 KB per device), entry `layer_slot`; slots
 * outside [0, BHI_STATIC_EXCHANGE_LAYERS) are rejected with BHI_ERR_LIMIT.  Nothing is allocated:
 * the array's address is looked up once per device (the first call on a device must therefore not be
 * made while `stream` is being captured; it returns BHI_ERR_ARG if it is); the array needs no clearing,
 * device memory of this kind starts out zero when the library is loaded.  Calls that use the same slot and may overlap in time (different streams, or threads) race on
 * its counters and must be serialised by the caller; different slots are independent. */
#define BHI_STATIC_EXCHANGE_LAYERS 1024
int bhi_gemv_bf16_huffman_exchange_static(const uint8_t *A_rem, const uint32_t *A_exp, int64_t exp_words,
                                          const uint16_t *X, uint16_t *Y, const int32_t *offsets,
                                          const uint8_t *prepared, int split_k, int M, int Nc, int batch,
                                          int layer_slot, void *stream);

/* Per-stream Huffman code emission as ASCII '0'/'1' characters.
 *   data u8 [streams, n]; LUT u8 [256, 32] code strings (root first, NUL padded);
 *   output u8 [streams, 32*n] (caller pre-fills with '0'); output_lengths i32 [streams] = bits.
 * Replaces torch.ops.bf16_huffman_infer.huffman_encode (src/kernel.cu:590-644, schema .cpp:30). */
int bhi_huffman_encode(const uint8_t *data, int streams, int n, const uint8_t *LUT,
                       uint8_t *output, int32_t *output_lengths, void *stream);

/* Per-stream rANS encode (64-bit state, 32-bit words, symbols taken last to first, words stored
 * in decode order).  data u8 [streams, n]; freq, cum u32 [256]; output u32 [streams, 8*n];
 * output_lengths i32 [streams] = words.
 * Replaces torch.ops.bf16_huffman_infer.ans_encode (src/kernel.cu:767-848, schema .cpp:34). */
int bhi_ans_encode(const uint8_t *data, int streams, int n, const uint32_t *freq,
                   const uint32_t *cum, uint32_t *output, int32_t *output_lengths, void *stream);

/* ---- whole-layer encoder -------------------------------------------------------------------
 * The reference drives the two per-stream operators above from Python and assembles the format
 * with tensor ops (functional.py:129-238, 297-310), expanding every symbol to 32 characters on
 * the way.  These entry points produce the same bytes directly from the BF16 weight W [M, K]
 * (row-major, K = split_k*Nc) in two passes: a size pass and an emit pass, with the record
 * offsets (a prefix sum with 64 padding words after every 4096 rows) computed in between by the
 * caller. */

/* Size pass: words_per_row i32 [split_k, M] = words per stream of each record
 * (functional.py:144-147 for Huffman: ceil(ceil(max bits / 8) / 4); :308 for rANS: max words).
 * The rANS variant also writes stream_words u8 [split_k, M, 64] for the emit pass. */
int bhi_huffman_size_pass(const uint16_t *W, int M, int K, int split_k, const uint8_t *code_lengths,
                          int32_t *words_per_row, void *stream);
int bhi_ans_size_pass(const uint16_t *W, int M, int K, int split_k, const uint32_t *freq,
                      const uint32_t *cum, int32_t *words_per_row, uint8_t *stream_words, void *stream);

/* Emit pass: writes A_rem (permuted bytes) and the coded words of every record at its offset.
 * A_exp must be zero-filled by the caller (padding words are never written).
 * code_values u32 [256]: code bits with the first path bit in bit 0. */
int bhi_huffman_emit_pass(const uint16_t *W, int M, int K, int split_k, const uint8_t *code_lengths,
                          const uint32_t *code_values, const int32_t *offsets,
                          uint8_t *A_rem, uint32_t *A_exp, void *stream);
int bhi_ans_emit_pass(const uint16_t *W, int M, int K, int split_k, const uint32_t *freq,
                      const uint32_t *cum, const int32_t *offsets, const uint8_t *stream_words,
                      uint8_t *A_rem, uint32_t *A_exp, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* BF16_HUFFMAN_B200_H_ */
