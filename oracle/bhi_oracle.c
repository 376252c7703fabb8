/*
 * CPU oracle for the exponent-coded BF16 weight format and its decode / decode+GEMV path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package calls into this file; it is the
 * checker the tests, the smoke test and the benchmark's CPU-baseline leg compare the CUDA
 * kernels against.  It is a plain-C restatement of the reference project's algorithm
 * (lszxb/bf16_huffman_infer), written from its behaviour; each function names the reference
 * lines it follows.  Paths are relative to the reference project root.
 *
 * Pinning: the bit conventions of both coders are checked against the reference's own slow
 * single-stream Python codecs and table builders through committed golden vectors
 * (tests/golden), and the whole-layer layout against buffers produced by the reference's CUDA
 * extension on a B200 (tests/golden/ref_layout_*.npz).
 *
 * Layout recap.  W is BF16 [M, K]; K is cut into S chunks of Nc = K/S columns (Nc % 128 == 0).
 *   rem  : u8  [S, M, Nc]   sign+mantissa bytes, permuted inside each 128-column block
 *   exp  : u32 [words]      per (chunk k, row m) a record of L rows of 64 words, word w of stream
 *                           g at offsets[k][m] + 64*w + g; 64 zero words after every slab of
 *                           4096 rows
 *   offs : i32 [S, M]       absolute word index of each record
 * Stream g = h*32 + lane of record (k, m) carries, for blk = 0..Nc/128-1 and t = 0,1, the
 * exponent of column k*Nc + blk*128 + 2*g + t.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define SLAB_ROWS 4096
/* Probability precision of the rANS model in use: the reference fixes 8 (functional.py:16, kernel.cu:25); its table
 * word and its static_assert (kernel.cu:647-649, :695) allow up to 12.  Set before a call, read-only during it. */
static int ANS_BITS = 8;
void bhi_oracle_set_ans_bits(int bits) {
    if (bits >= 8 && bits <= 12) ANS_BITS = bits;
}

/* ---- byte split / merge: bf16_huffman_infer/utils.py:7-12, src/kernel.cu:149-160 ---------- */
static inline uint8_t exp_of(uint16_t b) { return (uint8_t)((b >> 7) & 0xFF); }
static inline uint8_t rem_of(uint16_t b) { return (uint8_t)(((b >> 8) & 0x80) | (b & 0x7F)); }
static inline uint16_t join(uint8_t rem, uint8_t exp) {
    return (uint16_t)((((uint16_t)rem << 8) & 0x8000) | (rem & 0x7F) | ((uint16_t)exp << 7));
}

void bhi_oracle_split(const uint16_t *w, int64_t n, uint8_t *rem, uint8_t *exp) {
    for (int64_t i = 0; i < n; i++) { rem[i] = rem_of(w[i]); exp[i] = exp_of(w[i]); }
}

void bhi_oracle_merge(const uint8_t *rem, const uint8_t *exp, int64_t n, uint16_t *w) {
    for (int64_t i = 0; i < n; i++) w[i] = join(rem[i], exp[i]);
}

void bhi_oracle_histogram(const uint16_t *w, int64_t n, int64_t *counts /*[256]*/) {
    memset(counts, 0, 256 * sizeof(int64_t));
    for (int64_t i = 0; i < n; i++) counts[exp_of(w[i])]++;
}

/* ---- K-chunk chooser: bf16_huffman_infer/utils.py:15-31 ----------------------------------- */
int bhi_oracle_chunk_count(int K) {
    if (K <= 0 || K % 128) return -1;
    int nb = K / 128;
    for (int i = 32; i > 2; i--) if (nb % i == 0 && nb / i <= 8) return nb / i;
    for (int i = 32; i <= 128; i++) if (nb % i == 0 && nb / i <= 32) return nb / i;
    for (int i = 32; i > 2; i--) if (nb % i == 0 && nb / i <= 32) return nb / i;
    return -1;
}

/* column of symbol s of stream g in record (k, .): functional.py:171 (stream split) */
static inline int64_t col_of(int k, int Nc, int g, int s) {
    return (int64_t)k * Nc + (int64_t)(s >> 1) * 128 + 2 * g + (s & 1);
}

/* ---- rem permutation: functional.py:184 ---------------------------------------------------- */
void bhi_oracle_pack_rem(const uint16_t *W, int M, int K, int S, uint8_t *rem /*[S,M,Nc]*/) {
    int Nc = K / S;
    for (int k = 0; k < S; k++)
        for (int m = 0; m < M; m++) {
            const uint16_t *row = W + (int64_t)m * K + (int64_t)k * Nc;
            uint8_t *out = rem + ((int64_t)k * M + m) * Nc;
            for (int blk = 0; blk < Nc / 128; blk++)
                for (int h = 0; h < 2; h++)
                    for (int lane = 0; lane < 32; lane++)
                        for (int t = 0; t < 2; t++)
                            out[blk * 128 + lane * 4 + h * 2 + t] = rem_of(row[blk * 128 + h * 64 + lane * 2 + t]);
        }
}

/* ---- record placement: functional.py:175-182 (per slab) and :204-231 (slabs, chunks) -------
 * L[k*M+m] = words per stream of record (k,m).  Records are laid out chunk-major, rows ascending,
 * with 64 zero words appended after every slab of 4096 rows.  Returns the total word count. */
int64_t bhi_oracle_layout_offsets(const int32_t *L, int S, int M, int32_t *offsets) {
    int64_t at = 0;
    for (int k = 0; k < S; k++)
        for (int m = 0; m < M; m++) {
            offsets[(int64_t)k * M + m] = (int32_t)at;
            at += 64 * (int64_t)L[(int64_t)k * M + m];
            if ((m + 1) % SLAB_ROWS == 0 || m + 1 == M) at += 64;
        }
    return at;
}

/* ---- Huffman: size pass.  functional.py:144-147 -------------------------------------------- */
void bhi_oracle_huffman_row_words(const uint16_t *W, int M, int K, int S, const uint8_t *code_len,
                                  int32_t *L) {
    int Nc = K / S, n = Nc / 64;
#pragma omp parallel for collapse(2) schedule(static)
    for (int k = 0; k < S; k++)
        for (int m = 0; m < M; m++) {
            const uint16_t *row = W + (int64_t)m * K;
            uint32_t worst = 0;
            for (int g = 0; g < 64; g++) {
                uint32_t bits = 0;
                for (int s = 0; s < n; s++) bits += code_len[exp_of(row[col_of(k, Nc, g, s)])];
                if (bits > worst) worst = bits;
            }
            uint32_t bytes = (worst + 7) / 8;
            L[(int64_t)k * M + m] = (int32_t)((bytes + 3) / 4);
        }
}

/* ---- Huffman: emit pass.  src/kernel.cu:590-610 (code emission in root-first order) and
 * functional.py:149-157 (bit p of a stream -> byte p/8, bit p%8; bytes viewed little-endian). */
void bhi_oracle_huffman_emit(const uint16_t *W, int M, int K, int S, const uint8_t *code_len,
                             const uint32_t *code_val, const int32_t *offsets, uint32_t *exp) {
    int Nc = K / S, n = Nc / 64;
#pragma omp parallel for collapse(2) schedule(static)
    for (int k = 0; k < S; k++)
        for (int m = 0; m < M; m++) {
            const uint16_t *row = W + (int64_t)m * K;
            uint32_t *rec = exp + offsets[(int64_t)k * M + m];
            for (int g = 0; g < 64; g++) {
                uint64_t acc = 0; int have = 0; int w = 0;
                for (int s = 0; s < n; s++) {
                    uint8_t e = exp_of(row[col_of(k, Nc, g, s)]);
                    acc |= (uint64_t)code_val[e] << have;
                    have += code_len[e];
                    if (have >= 32) { rec[64 * w + g] = (uint32_t)acc; w++; acc >>= 32; have -= 32; }
                }
                if (have > 0) rec[64 * w + g] = (uint32_t)acc;
            }
        }
}

/* ---- rANS encode of one stream: src/kernel.cu:767-811.  Symbols are taken last to first; the
 * emitted words are reversed at the end.  Returns the word count; out may be NULL (size pass). */
static int ans_encode_stream(const uint8_t *sym, int n, const uint32_t *freq, const uint32_t *cum,
                             uint32_t *out /*capacity 8n*/) {
    uint64_t state = 1ull << ANS_BITS;
    int cnt = 0;
    for (int i = n - 1; i >= 0; i--) {
        uint32_t f = freq[sym[i]], c = cum[sym[i]];
        while ((state >> 32) >= f) { if (out) out[cnt] = (uint32_t)state; cnt++; state >>= 32; }
        state = ((state / f) << ANS_BITS) + (state % f) + c;
    }
    while (state > 0) { if (out) out[cnt] = (uint32_t)state; cnt++; state >>= 32; }
    if (out)
        for (int i = 0; i < cnt / 2; i++) { uint32_t t = out[i]; out[i] = out[cnt - 1 - i]; out[cnt - 1 - i] = t; }
    return cnt;
}

/* The reference's ans_encode operator: data u8 [streams, n] -> output u32 [streams, 8n]. */
void bhi_oracle_ans_encode_op(const uint8_t *data, int streams, int n, const uint32_t *freq,
                              const uint32_t *cum, uint32_t *output, int32_t *output_lengths) {
#pragma omp parallel for schedule(static)
    for (int t = 0; t < streams; t++)
        output_lengths[t] = ans_encode_stream(data + (int64_t)t * n, n, freq, cum, output + (int64_t)t * n * 8);
}

/* The reference's huffman_encode operator: src/kernel.cu:590-610.  LUT is [256][32] ASCII code
 * strings (root-first, NUL padded); output [streams, 32n] chars is written with the
 * concatenated codes, output_lengths gets the bit count. */
void bhi_oracle_huffman_encode_op(const uint8_t *data, int streams, int n, const char *LUT,
                                  char *output, int32_t *output_lengths) {
    for (int t = 0; t < streams; t++) {
        int32_t cnt = 0;
        for (int i = 0; i < n; i++) {
            const char *p = LUT + 32 * (int)data[(int64_t)t * n + i];
            for (int j = 0; j < 32 && p[j] != '\0'; j++) output[(int64_t)t * n * 32 + cnt++] = p[j];
        }
        output_lengths[t] = cnt;
    }
}

static void gather_stream(const uint16_t *row, int k, int Nc, int g, int n, uint8_t *sym) {
    for (int s = 0; s < n; s++) sym[s] = exp_of(row[col_of(k, Nc, g, s)]);
}

/* ---- rANS: size pass (functional.py:308, L = max words over the 64 streams) ---------------- */
void bhi_oracle_ans_row_words(const uint16_t *W, int M, int K, int S, const uint32_t *freq,
                              const uint32_t *cum, int32_t *L) {
    int Nc = K / S, n = Nc / 64;
#pragma omp parallel for collapse(2) schedule(static)
    for (int k = 0; k < S; k++)
        for (int m = 0; m < M; m++) {
            uint8_t sym[1024];
            int worst = 0;
            for (int g = 0; g < 64; g++) {
                gather_stream(W + (int64_t)m * K, k, Nc, g, n, sym);
                int c = ans_encode_stream(sym, n, freq, cum, NULL);
                if (c > worst) worst = c;
            }
            L[(int64_t)k * M + m] = worst;
        }
}

void bhi_oracle_ans_emit(const uint16_t *W, int M, int K, int S, const uint32_t *freq,
                         const uint32_t *cum, const int32_t *offsets, uint32_t *exp) {
    int Nc = K / S, n = Nc / 64;
#pragma omp parallel for collapse(2) schedule(static)
    for (int k = 0; k < S; k++)
        for (int m = 0; m < M; m++) {
            uint8_t sym[1024];
            uint32_t words[8 * 1024];
            uint32_t *rec = exp + offsets[(int64_t)k * M + m];
            for (int g = 0; g < 64; g++) {
                gather_stream(W + (int64_t)m * K, k, Nc, g, n, sym);
                int c = ans_encode_stream(sym, n, freq, cum, words);
                for (int w = 0; w < c; w++) rec[64 * w + g] = words[w];
            }
        }
}

/* ---- decoders ------------------------------------------------------------------------------ */
typedef struct {
    const uint32_t *base; int64_t limit;   /* whole exp buffer, for bounds */
    int64_t at;                            /* next word index of this stream */
    uint64_t win; int have;                /* Huffman window / valid bits; rANS state in win */
    int overrun;
} stream_t;

static inline uint32_t next_word(stream_t *s) {
    uint32_t v = 0;
    if (s->at >= 0 && s->at < s->limit) v = s->base[s->at]; else s->overrun = 1;
    s->at += 64;
    return v;
}

/* src/kernel.cu:354-380: refill one word when fewer than 32 bits remain, then take the first of
 * LUT1[b0], LUT2[b1], LUT3[b2], LUT4[b3] that is not 255 and drop code_lengths[sym] bits. */
static inline uint8_t huff_next(stream_t *s, const uint8_t *l1, const uint8_t *l2, const uint8_t *l3,
                                const uint8_t *l4, const uint8_t *len) {
    if (s->have < 32) { s->win |= (uint64_t)next_word(s) << s->have; s->have += 32; }
    uint8_t sym = l1[s->win & 0xFF];
    if (sym == 255) sym = l2[(s->win >> 8) & 0xFF];
    if (sym == 255) sym = l3[(s->win >> 16) & 0xFF];
    if (sym == 255) sym = l4[(s->win >> 24) & 0xFF];
    int n = len[sym];
    s->win >>= n;
    s->have = (uint8_t)(s->have - n);
    return sym;
}

/* src/kernel.cu:652-683; table word = sym<<24 | freq<<12 | (slot - cum[sym]) (functional.py:288-292) */
static inline uint8_t ans_next(stream_t *s, const uint32_t *lut) {
    if (s->win < (1u << ANS_BITS)) s->win = (s->win << 32) | next_word(s);
    uint32_t e = lut[s->win & ((1u << ANS_BITS) - 1)];
    s->win = (uint64_t)((e >> 12) & 0xFFF) * (s->win >> ANS_BITS) + (e & 0xFFF);
    return (uint8_t)(e >> 24);
}

/* Decode record (k,m) into exponents for the chunk's Nc columns, in source column order. */
static int decode_record(int algo, const uint32_t *exp, int64_t exp_words, int64_t off, int Nc,
                         const uint8_t *l1, const uint8_t *l2, const uint8_t *l3, const uint8_t *l4,
                         const uint8_t *len, const uint32_t *alut, uint8_t *e_out /*[Nc]*/) {
    int n = Nc / 64, bad = 0;
    for (int g = 0; g < 64; g++) {
        stream_t s = { exp, exp_words, off + g, 0, 0, 0 };
        if (algo == 1) s.win = next_word(&s);
        for (int i = 0; i < n; i++) {
            uint8_t sym = algo == 0 ? huff_next(&s, l1, l2, l3, l4, len) : ans_next(&s, alut);
            e_out[(i >> 1) * 128 + 2 * g + (i & 1)] = sym;
        }
        /* A Huffman stream may look one word past its record (kernel.cu:359-368); in a well-formed
         * buffer that word is slab padding or the next record, so it is still inside the buffer.
         * Leaving the buffer altogether means the offsets / tables do not belong to this data. */
        bad |= s.overrun;
    }
    return bad;
}

static int decode_layer(int algo, const uint8_t *rem, const uint32_t *exp, int64_t exp_words,
                        const int32_t *offsets, const uint8_t *l1, const uint8_t *l2, const uint8_t *l3,
                        const uint8_t *l4, const uint8_t *len, const uint32_t *alut,
                        int S, int M, int Nc, uint16_t *Wout) {
    int64_t K = (int64_t)S * Nc;
    int status = 0;
#pragma omp parallel for collapse(2) schedule(static)
    for (int k = 0; k < S; k++)
        for (int m = 0; m < M; m++) {
            uint8_t e[16384];
            if (decode_record(algo, exp, exp_words, offsets[(int64_t)k * M + m], Nc, l1, l2, l3, l4, len, alut, e)) {
#pragma omp atomic write
                status = 1;
            }
            const uint8_t *r = rem + ((int64_t)k * M + m) * Nc;
            uint16_t *out = Wout + (int64_t)m * K + (int64_t)k * Nc;
            for (int blk = 0; blk < Nc / 128; blk++)
                for (int lane = 0; lane < 32; lane++)
                    for (int h = 0; h < 2; h++)
                        for (int t = 0; t < 2; t++) {
                            int c = blk * 128 + h * 64 + lane * 2 + t;
                            out[c] = join(r[blk * 128 + lane * 4 + h * 2 + t], e[c]);
                        }
        }
    return status;
}

/* Dense BF16 [M, S*Nc] from the compressed form: src/kernel.cu:222-310 with either decoder. */
int bhi_oracle_huffman_decode(const uint8_t *rem, const uint32_t *exp, int64_t exp_words,
                              const int32_t *offsets, const uint8_t *l1, const uint8_t *l2,
                              const uint8_t *l3, const uint8_t *l4, const uint8_t *len,
                              int S, int M, int Nc, uint16_t *Wout) {
    if (Nc % 128 || Nc > 16384) return -1;
    return decode_layer(0, rem, exp, exp_words, offsets, l1, l2, l3, l4, len, NULL, S, M, Nc, Wout);
}

int bhi_oracle_ans_decode(const uint8_t *rem, const uint32_t *exp, int64_t exp_words,
                          const int32_t *offsets, const uint32_t *lut, int S, int M, int Nc, uint16_t *Wout) {
    if (Nc % 128 || Nc > 16384) return -1;
    return decode_layer(1, rem, exp, exp_words, offsets, NULL, NULL, NULL, NULL, NULL, lut, S, M, Nc, Wout);
}

static inline float bf16_to_f32(uint16_t b) { uint32_t u = (uint32_t)b << 16; float f; memcpy(&f, &u, 4); return f; }

/* Y[b][m] = sum_c X[b][c] * W[m][c] on dense BF16 inputs, accumulated in double so that it can
 * serve as the exact reference for the FP32-accumulating kernels (src/kernel.cu:163-166, 171-218). */
void bhi_oracle_matvec(const uint16_t *W, const uint16_t *X, int B, int M, int64_t K, float *Y) {
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; m++)
        for (int b = 0; b < B; b++) {
            double acc = 0.0;
            const uint16_t *w = W + (int64_t)m * K, *x = X + (int64_t)b * K;
            for (int64_t c = 0; c < K; c++) acc += (double)bf16_to_f32(w[c]) * (double)bf16_to_f32(x[c]);
            Y[(int64_t)b * M + m] = (float)acc;
        }
}

/* Fused CPU path used only as the timed CPU baseline: decode each record and dot it with X
 * without materialising W (what the fused kernel does, src/kernel.cu:46-219), FP32 accumulate. */
int bhi_oracle_gemv(int algo, const uint8_t *rem, const uint32_t *exp, int64_t exp_words,
                    const int32_t *offsets, const uint8_t *l1, const uint8_t *l2, const uint8_t *l3,
                    const uint8_t *l4, const uint8_t *len, const uint32_t *alut,
                    int S, int M, int Nc, const uint16_t *X, int B, float *Y) {
    if (Nc % 128 || Nc > 16384 || B > 8) return -1;
    int64_t K = (int64_t)S * Nc;
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; m++) {
        float acc[8] = {0};
        uint8_t e[16384];
        for (int k = 0; k < S; k++) {
            decode_record(algo, exp, exp_words, offsets[(int64_t)k * M + m], Nc, l1, l2, l3, l4, len, alut, e);
            const uint8_t *r = rem + ((int64_t)k * M + m) * Nc;
            for (int blk = 0; blk < Nc / 128; blk++)
                for (int lane = 0; lane < 32; lane++)
                    for (int h = 0; h < 2; h++)
                        for (int t = 0; t < 2; t++) {
                            int c = blk * 128 + h * 64 + lane * 2 + t;
                            float w = bf16_to_f32(join(r[blk * 128 + lane * 4 + h * 2 + t], e[c]));
                            for (int b = 0; b < B; b++) acc[b] += w * bf16_to_f32(X[(int64_t)b * K + (int64_t)k * Nc + c]);
                        }
        }
        for (int b = 0; b < B; b++) Y[(int64_t)b * M + m] = acc[b];
    }
    return 0;
}

/* Worker threads of the following calls (the benchmark sets it to the cores it may use, whatever OMP_NUM_THREADS says). */
void bhi_oracle_set_threads(int n) {
#ifdef _OPENMP
    if (n >= 1) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int bhi_oracle_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
