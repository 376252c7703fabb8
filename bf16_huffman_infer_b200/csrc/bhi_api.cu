// C ABI entry points: argument validation, launch geometry and dispatch.  No allocation, no
// synchronisation, no device-property query on the launch path (the SM count is cached per
// device on first use), so every call can be captured into a CUDA graph.
#include <atomic>
#include <mutex>
#include <unordered_map>

#include "bhi_common.cuh"
#include "bhi_encode.cuh"
#include "bhi_generic.cuh"
#include "bhi_staged.cuh"
#include "bhi_quad.cuh"
#include "bhi_tile.cuh"
#include "bhi_tileq.cuh"

namespace bhi {

static thread_local std::string g_error;
static std::atomic<int> g_path{0};
static std::atomic<int> g_overlap{0};
static std::atomic<int> g_quad_ppw{0};
bool overlap_launches() { return g_overlap.load() != 0; }
int quad_passes_per_warp() { return g_quad_ppw.load(); }

// Prepared blobs the caller has declared pair-complete (bhi_huffman_table_hint): device pointer -> true.
// A tuning hint only; bhi_huffman_prepare forgets the entry of the blob it rewrites.
static std::mutex g_hint_mu;
static std::unordered_map<const void *, bool> g_hints;
static bool pair_complete_hint(const void *prepared) {
    if (prepared == nullptr) return false;
    std::lock_guard<std::mutex> lock(g_hint_mu);
    auto it = g_hints.find(prepared);
    return it != g_hints.end() && it->second;
}

void set_error(const std::string &msg) { g_error = msg; }
int fail(int code, const std::string &msg) {
    g_error = msg;
    return code;
}
int cuda_fail(cudaError_t e, const char *what) {
    g_error = std::string(what) + ": " + cudaGetErrorString(e);
    return BHI_ERR_CUDA;
}

int sm_count() {
    static std::mutex mu;
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

static int check_layer(const void *rem, const void *exp, int64_t exp_words, const void *offsets,
                       int S, int M, int Nc) {
    BHI_REQUIRE(rem && exp && offsets, "null weight buffer");
    BHI_REQUIRE(S >= 1 && M >= 1, "empty layer");
    BHI_REQUIRE(Nc >= 128 && Nc % 128 == 0 && Nc <= 16384, "chunk width must be a multiple of 128 in [128, 16384]");
    BHI_REQUIRE(exp_words >= 64, "exponent buffer shorter than one record row");
    BHI_REQUIRE(aligned(rem, 4) && aligned(exp, 4) && aligned(offsets, 4), "weight buffers must be 4-byte aligned");
    return BHI_OK;
}

static int launch_status(const char *what) {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? BHI_OK : cuda_fail(e, what);
}

template <class Codec>
static int run_gemv(const Layer &L, const typename Codec::Args &targs, const uint8_t *prepared, const uint16_t *X,
                    uint16_t *Y, int B, cudaStream_t st) {
    BHI_REQUIRE(X && Y, "null activation buffer");
    BHI_REQUIRE(B >= 1 && B <= BHI_MAX_BATCH, "batch must be in [1, 8]");
    BHI_REQUIRE(aligned(X, 4) && aligned(Y, 2), "activation buffers must be 4-byte (X) / 2-byte (Y) aligned");
    const int path = g_path.load();
    const bool complete = pair_complete_hint(prepared);
    // One or two rows of X with rANS, or with Huffman tables that have unresolved windows: the one-row-per-warp
    // kernel is the faster one there (its single-symbol detour is cheaper, and its tensor-core tile covers two
    // rows of X anyway)
    const bool row_first = !(std::is_same<Codec, HuffCodec>::value && complete) && B <= 2;
    if (path == 0 && row_first) {
        int rc = staged_gemv<Codec>(L, targs, prepared, X, Y, B, st);
        if (rc != kStagedDeclined) return rc;
    }
    if (path == 0) {
        int rc = quad_launch<Codec>(L, targs, prepared, X, Y, nullptr, B, complete, st);
        if (rc != kStagedDeclined) return rc;
    }
    if (path == 0 || path == 2) {
        int rc = staged_gemv<Codec>(L, targs, prepared, X, Y, B, st);
        if (rc != kStagedDeclined) return rc;
    }
    // one warp per row, enough blocks to give every row its own warp up to 8 waves of blocks per SM
    const int warps_per_block = kGenericThreads / 32;
    int blocks = (L.M + warps_per_block - 1) / warps_per_block;
    const int cap = sm_count() * 64;
    if (blocks > cap) blocks = cap;
#define BHI_CASE(b)                                                                                  \
    case b:                                                                                          \
        gemv_generic_kernel<Codec, b><<<blocks, kGenericThreads, 0, st>>>(L, targs, X, Y);           \
        break;
    switch (B) {
        BHI_CASE(1) BHI_CASE(2) BHI_CASE(3) BHI_CASE(4) BHI_CASE(5) BHI_CASE(6) BHI_CASE(7) BHI_CASE(8)
    }
#undef BHI_CASE
    return launch_status("gemv launch");
}

template <class Codec>
static int run_decode(const Layer &L, const typename Codec::Args &targs, const uint8_t *prepared, uint16_t *Y,
                      cudaStream_t st) {
    BHI_REQUIRE(Y, "null output buffer");
    BHI_REQUIRE(aligned(Y, 4), "output must be 4-byte aligned");
    if (g_path.load() != 1) {
        int rc = staged_decode<Codec>(L, targs, prepared, Y, st);
        if (rc != kStagedDeclined) return rc;
    }
    const int64_t nrec = static_cast<int64_t>(L.S) * L.M;
    const int warps_per_block = kGenericThreads / 32;
    int64_t blocks = (nrec + warps_per_block - 1) / warps_per_block;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 64;
    if (blocks > cap) blocks = cap;
    decode_generic_kernel<Codec><<<static_cast<int>(blocks), kGenericThreads, 0, st>>>(L, targs, Y);
    return launch_status("decode launch");
}

template <class Codec>
static int run_linear(const Layer &L, const typename Codec::Args &targs, const uint8_t *prepared, const uint16_t *X,
                      uint16_t *Y, int B, cudaStream_t st) {
    BHI_REQUIRE(X && Y, "null activation buffer");
    BHI_REQUIRE(B >= 1 && B <= BHI_MAX_LINEAR_BATCH, "batch must be in [1, 128]");
    BHI_REQUIRE(aligned(X, 16) && aligned(Y, 2), "activation buffers must be 16-byte (X) / 2-byte (Y) aligned");
    BHI_REQUIRE(aligned(L.rem, 16) && aligned(L.exp, 16) && aligned(prepared, 16), "weight buffers must be 16-byte aligned");
    if (g_path.load() != 2) {
        const int rc = tileq_launch<Codec>(L, targs, prepared, X, Y, B, st);
        if (rc != kStagedDeclined) return rc;
    }
    return tile_launch<Codec>(L, targs, prepared, X, Y, B, st);
}

template <class Codec>
static int run_exchange(const Layer &L, const typename Codec::Args &targs, const uint8_t *prepared, const uint16_t *X, int B,
                        const bhi_exchange_t *ex, cudaStream_t st) {
    BHI_REQUIRE(X && ex, "null activation buffer or exchange descriptor");
    BHI_REQUIRE(B >= 1 && B <= BHI_MAX_BATCH, "batch must be in [1, 8]");
    BHI_REQUIRE(ex->world >= 1 && ex->world <= BHI_MAX_PEERS && ex->rank >= 0 && ex->rank < ex->world, "bad world / rank");
    BHI_REQUIRE(ex->row_base >= 0 && ex->M_total >= ex->row_base + L.M, "rows outside the full output");
    BHI_REQUIRE(ex->launches && aligned(ex->launches, 4), "null or unaligned launch counter");
    BHI_REQUIRE(aligned(X, 4), "X must be 4-byte aligned");
    BHI_REQUIRE(aligned(L.rem, 16) && aligned(L.exp, 16) && aligned(prepared, 16), "weight buffers must be 16-byte aligned");
    PeerSet peers{};
    for (int r = 0; r < ex->world; r++) {
        BHI_REQUIRE(ex->y[r] && ex->ready[r] && ex->done[r], "null peer pointer");
        BHI_REQUIRE(aligned(ex->y[r], 2) && aligned(ex->ready[r], 4) && aligned(ex->done[r], 4), "unaligned peer pointer");
        peers.y[r] = ex->y[r];
        peers.ready[r] = ex->ready[r];
        peers.done[r] = ex->done[r];
    }
    peers.launches = ex->launches;
    peers.world = ex->world;
    peers.rank = ex->rank;
    peers.row_base = ex->row_base;
    peers.m_total = ex->M_total;
    int rc = kStagedDeclined;
    const bool complete = pair_complete_hint(prepared);
    const bool row_first = !(std::is_same<Codec, HuffCodec>::value && complete) && B <= 2;
    if (g_path.load() == 0 && !row_first) rc = quad_launch<Codec>(L, targs, prepared, X, nullptr, &peers, B, complete, st);
    if (rc == kStagedDeclined) rc = staged_exchange<Codec>(L, targs, prepared, X, peers, B, st);
    if (rc == kStagedDeclined && g_path.load() == 0 && row_first) rc = quad_launch<Codec>(L, targs, prepared, X, nullptr, &peers, B, complete, st);
    return rc == kStagedDeclined ? fail(BHI_ERR_ARG, "shape not supported by the exchange kernel") : rc;
}

// ---- exchange counters kept inside the library (bhi_gemv_bf16_huffman_exchange_static) --------------
// One 256-byte entry per layer slot: ready counter at word 0, done counter at word 32, launch counter at
// word 48, block-arrival counter at word 49.  File-scope device memory: nothing is allocated; the address is
// looked up once per device.  No clearing: a file-scope device array without initialiser is zero when the
// module is loaded, and a clear enqueued on the first caller's stream could run under another stream's kernel.
constexpr int kStaticWordsPerLayer = 64;
static __device__ __align__(256) uint32_t g_static_exchange[BHI_STATIC_EXCHANGE_LAYERS * kStaticWordsPerLayer];

static int static_exchange_base(cudaStream_t st, uint32_t **base_out) {
    static std::mutex mu;
    static uint32_t *base[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(BHI_ERR_CUDA, "cudaGetDevice failed");
    std::lock_guard<std::mutex> lock(mu);
    if (base[dev] == nullptr) {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        cudaError_t e = cudaStreamIsCapturing(st, &cap);
        if (e != cudaSuccess) return cuda_fail(e, "cudaStreamIsCapturing");
        BHI_REQUIRE(cap == cudaStreamCaptureStatusNone, "the first call on a device must be made outside stream capture");
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_exchange);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress");
        base[dev] = static_cast<uint32_t *>(p);
    }
    *base_out = base[dev];
    return BHI_OK;
}

static int check_enc(const void *W, int M, int K, int S) {
    BHI_REQUIRE(W, "null weight");
    BHI_REQUIRE(M >= 1 && K >= 128 && S >= 1 && K % S == 0, "bad shape");
    const int Nc = K / S;
    BHI_REQUIRE(Nc % 128 == 0 && Nc <= 16384, "chunk width must be a multiple of 128, at most 16384");
    BHI_REQUIRE(aligned(W, 4), "weight must be 4-byte aligned");
    return BHI_OK;
}

static int enc_blocks(int M, int S) {
    return static_cast<int>((static_cast<int64_t>(S) * M + kEncRecords - 1) / kEncRecords);
}

}  // namespace bhi

using namespace bhi;

extern "C" {

const char *bhi_last_error(void) { return g_error.c_str(); }
int bhi_abi_version(void) { return 2; }
int bhi_set_kernel_path(int path) { return g_path.exchange(path); }
int bhi_set_launch_overlap(int on) { return g_overlap.exchange(on ? 1 : 0); }
int bhi_set_quad_warps(int warps) {
    if (warps != 0 && warps != 16 && warps != 32) return -1;
    const int prev = g_quad_ppw.exchange(warps == 16 ? 2 : warps == 32 ? 1 : 0);
    return prev == 2 ? 16 : prev == 1 ? 32 : 0;
}
int bhi_huffman_table_hint(const uint8_t *prepared, int pair_complete) {
    BHI_REQUIRE(prepared, "null prepared tables");
    std::lock_guard<std::mutex> lock(g_hint_mu);
    if (pair_complete) g_hints[prepared] = true;
    else g_hints.erase(prepared);
    return BHI_OK;
}

int bhi_debug_status(int *status_out) {
    BHI_REQUIRE(status_out, "null output");
    int v = 0, zero = 0;
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemcpyFromSymbol(&v, g_staged_status, sizeof(int));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_staged_status, &zero, sizeof(int));
    if (e != cudaSuccess) return cuda_fail(e, "status read");
    *status_out = v;
    return BHI_OK;
}

int bhi_gemv_bf16_huffman(const uint8_t *A_rem, const uint32_t *A_exp, int64_t exp_words,
                          const uint16_t *X, uint16_t *Y, const int32_t *offsets,
                          const uint8_t *LUT1, const uint8_t *LUT2, const uint8_t *LUT3,
                          const uint8_t *LUT4, const uint8_t *code_lengths,
                          int split_k, int M, int Nc, int batch, void *stream) {
    if (int rc = check_layer(A_rem, A_exp, exp_words, offsets, split_k, M, Nc)) return rc;
    BHI_REQUIRE(LUT1 && LUT2 && LUT3 && LUT4 && code_lengths, "null table");
    Layer L{A_rem, A_exp, exp_words, offsets, split_k, M, Nc};
    HuffArgs t{LUT1, LUT2, LUT3, LUT4, code_lengths};
    return run_gemv<HuffCodec>(L, t, nullptr, X, Y, batch, static_cast<cudaStream_t>(stream));
}

int bhi_huffman_decode(const uint8_t *A_rem, const uint32_t *A_exp, int64_t exp_words,
                       uint16_t *Y, const int32_t *offsets,
                       const uint8_t *LUT1, const uint8_t *LUT2, const uint8_t *LUT3,
                       const uint8_t *LUT4, const uint8_t *code_lengths,
                       int split_k, int M, int Nc, void *stream) {
    if (int rc = check_layer(A_rem, A_exp, exp_words, offsets, split_k, M, Nc)) return rc;
    BHI_REQUIRE(LUT1 && LUT2 && LUT3 && LUT4 && code_lengths, "null table");
    Layer L{A_rem, A_exp, exp_words, offsets, split_k, M, Nc};
    HuffArgs t{LUT1, LUT2, LUT3, LUT4, code_lengths};
    return run_decode<HuffCodec>(L, t, nullptr, Y, static_cast<cudaStream_t>(stream));
}

int bhi_huffman_prepared_bytes(void) { return kPreparedBytes; }

int bhi_huffman_prepare(const uint8_t *LUT1, const uint8_t *LUT2, const uint8_t *LUT3, const uint8_t *LUT4,
                        const uint8_t *code_lengths, uint8_t *prepared, void *stream) {
    BHI_REQUIRE(LUT1 && LUT2 && LUT3 && LUT4 && code_lengths && prepared, "null table");
    BHI_REQUIRE(aligned(prepared, 16), "prepared tables must be 16-byte aligned");
    HuffArgs t{LUT1, LUT2, LUT3, LUT4, code_lengths};
    {
        std::lock_guard<std::mutex> lock(g_hint_mu);
        g_hints.erase(prepared);
    }
    huffman_prepare_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(t, prepared);
    return launch_status("huffman_prepare launch");
}

// A prepared blob carries the exact tables too, so the five table pointers are not needed here.
int bhi_gemv_bf16_huffman_prepared(const uint8_t *A_rem, const uint32_t *A_exp, int64_t exp_words,
                                   const uint16_t *X, uint16_t *Y, const int32_t *offsets,
                                   const uint8_t *prepared, int split_k, int M, int Nc, int batch, void *stream) {
    if (int rc = check_layer(A_rem, A_exp, exp_words, offsets, split_k, M, Nc)) return rc;
    BHI_REQUIRE(prepared && aligned(prepared, 16), "null or unaligned prepared tables");
    Layer L{A_rem, A_exp, exp_words, offsets, split_k, M, Nc};
    const uint8_t *ex = prepared + kPairEntries * 4;
    HuffArgs t{ex, ex + 256, ex + 512, ex + 768, ex + 1024};
    return run_gemv<HuffCodec>(L, t, prepared, X, Y, batch, static_cast<cudaStream_t>(stream));
}

int bhi_huffman_decode_prepared(const uint8_t *A_rem, const uint32_t *A_exp, int64_t exp_words,
                                uint16_t *Y, const int32_t *offsets, const uint8_t *prepared,
                                int split_k, int M, int Nc, void *stream) {
    if (int rc = check_layer(A_rem, A_exp, exp_words, offsets, split_k, M, Nc)) return rc;
    BHI_REQUIRE(prepared && aligned(prepared, 16), "null or unaligned prepared tables");
    Layer L{A_rem, A_exp, exp_words, offsets, split_k, M, Nc};
    const uint8_t *ex = prepared + kPairEntries * 4;
    HuffArgs t{ex, ex + 256, ex + 512, ex + 768, ex + 1024};
    return run_decode<HuffCodec>(L, t, prepared, Y, static_cast<cudaStream_t>(stream));
}

int bhi_linear_bf16_huffman(const uint8_t *A_rem, const uint32_t *A_exp, int64_t exp_words,
                            const uint16_t *X, uint16_t *Y, const int32_t *offsets,
                            const uint8_t *LUT1, const uint8_t *LUT2, const uint8_t *LUT3,
                            const uint8_t *LUT4, const uint8_t *code_lengths,
                            int split_k, int M, int Nc, int batch, void *stream) {
    if (int rc = check_layer(A_rem, A_exp, exp_words, offsets, split_k, M, Nc)) return rc;
    BHI_REQUIRE(LUT1 && LUT2 && LUT3 && LUT4 && code_lengths, "null table");
    Layer L{A_rem, A_exp, exp_words, offsets, split_k, M, Nc};
    HuffArgs t{LUT1, LUT2, LUT3, LUT4, code_lengths};
    return run_linear<HuffCodec>(L, t, nullptr, X, Y, batch, static_cast<cudaStream_t>(stream));
}

int bhi_linear_bf16_huffman_prepared(const uint8_t *A_rem, const uint32_t *A_exp, int64_t exp_words,
                                     const uint16_t *X, uint16_t *Y, const int32_t *offsets,
                                     const uint8_t *prepared, int split_k, int M, int Nc, int batch, void *stream) {
    if (int rc = check_layer(A_rem, A_exp, exp_words, offsets, split_k, M, Nc)) return rc;
    BHI_REQUIRE(prepared && aligned(prepared, 16), "null or unaligned prepared tables");
    Layer L{A_rem, A_exp, exp_words, offsets, split_k, M, Nc};
    const uint8_t *ex = prepared + kPairEntries * 4;
    HuffArgs t{ex, ex + 256, ex + 512, ex + 768, ex + 1024};
    return run_linear<HuffCodec>(L, t, prepared, X, Y, batch, static_cast<cudaStream_t>(stream));
}

int bhi_linear_bf16_ans(const uint8_t *A_rem, const uint32_t *A_exp, int64_t exp_words,
                        const uint16_t *X, uint16_t *Y, const int32_t *offsets, const uint32_t *LUT, int precision,
                        int split_k, int M, int Nc, int batch, void *stream) {
    if (int rc = check_layer(A_rem, A_exp, exp_words, offsets, split_k, M, Nc)) return rc;
    BHI_REQUIRE(LUT && aligned(LUT, 4), "null or unaligned table");
    BHI_REQUIRE(precision >= BHI_ANS_PRECISION && precision <= BHI_ANS_MAX_PRECISION, "rANS precision must be in [8, 12]");
    Layer L{A_rem, A_exp, exp_words, offsets, split_k, M, Nc};
    AnsArgs t{LUT, precision};
    return run_linear<AnsCodec>(L, t, nullptr, X, Y, batch, static_cast<cudaStream_t>(stream));
}

int bhi_gemv_bf16_huffman_exchange(const uint8_t *A_rem, const uint32_t *A_exp, int64_t exp_words,
                                   const uint16_t *X, const int32_t *offsets, const uint8_t *prepared,
                                   int split_k, int M, int Nc, int batch, const bhi_exchange_t *exchange, void *stream) {
    if (int rc = check_layer(A_rem, A_exp, exp_words, offsets, split_k, M, Nc)) return rc;
    BHI_REQUIRE(prepared && aligned(prepared, 16), "null or unaligned prepared tables");
    Layer L{A_rem, A_exp, exp_words, offsets, split_k, M, Nc};
    const uint8_t *ex = prepared + kPairEntries * 4;
    HuffArgs t{ex, ex + 256, ex + 512, ex + 768, ex + 1024};
    return run_exchange<HuffCodec>(L, t, prepared, X, batch, exchange, static_cast<cudaStream_t>(stream));
}

int bhi_gemv_bf16_huffman_exchange_static(const uint8_t *A_rem, const uint32_t *A_exp, int64_t exp_words,
                                          const uint16_t *X, uint16_t *Y, const int32_t *offsets,
                                          const uint8_t *prepared, int split_k, int M, int Nc, int batch,
                                          int layer_slot, void *stream) {
    if (int rc = check_layer(A_rem, A_exp, exp_words, offsets, split_k, M, Nc)) return rc;
    BHI_REQUIRE(prepared && aligned(prepared, 16), "null or unaligned prepared tables");
    BHI_REQUIRE(Y && aligned(Y, 2), "null or unaligned output");
    if (layer_slot < 0 || layer_slot >= BHI_STATIC_EXCHANGE_LAYERS)
        return fail(BHI_ERR_LIMIT, "layer_slot outside [0, BHI_STATIC_EXCHANGE_LAYERS)");
    uint32_t *words = nullptr;
    if (int rc = static_exchange_base(static_cast<cudaStream_t>(stream), &words)) return rc;
    words += static_cast<size_t>(layer_slot) * kStaticWordsPerLayer;
    bhi_exchange_t ex = {};
    ex.world = 1;
    ex.rank = 0;
    ex.row_base = 0;
    ex.M_total = M;
    ex.y[0] = Y;
    ex.ready[0] = words;
    ex.done[0] = words + 32;
    ex.launches = words + 48;
    Layer L{A_rem, A_exp, exp_words, offsets, split_k, M, Nc};
    const uint8_t *t = prepared + kPairEntries * 4;
    HuffArgs args{t, t + 256, t + 512, t + 768, t + 1024};
    return run_exchange<HuffCodec>(L, args, prepared, X, batch, &ex, static_cast<cudaStream_t>(stream));
}

int bhi_gemv_bf16_ans_exchange(const uint8_t *A_rem, const uint32_t *A_exp, int64_t exp_words,
                               const uint16_t *X, const int32_t *offsets, const uint32_t *LUT, int precision,
                               int split_k, int M, int Nc, int batch, const bhi_exchange_t *exchange, void *stream) {
    if (int rc = check_layer(A_rem, A_exp, exp_words, offsets, split_k, M, Nc)) return rc;
    BHI_REQUIRE(LUT && aligned(LUT, 4), "null or unaligned table");
    BHI_REQUIRE(precision >= BHI_ANS_PRECISION && precision <= BHI_ANS_MAX_PRECISION, "rANS precision must be in [8, 12]");
    Layer L{A_rem, A_exp, exp_words, offsets, split_k, M, Nc};
    AnsArgs t{LUT, precision};
    return run_exchange<AnsCodec>(L, t, nullptr, X, batch, exchange, static_cast<cudaStream_t>(stream));
}

int bhi_gemv_bf16_ans(const uint8_t *A_rem, const uint32_t *A_exp, int64_t exp_words,
                      const uint16_t *X, uint16_t *Y, const int32_t *offsets, const uint32_t *LUT, int precision,
                      int split_k, int M, int Nc, int batch, void *stream) {
    if (int rc = check_layer(A_rem, A_exp, exp_words, offsets, split_k, M, Nc)) return rc;
    BHI_REQUIRE(LUT && aligned(LUT, 4), "null or unaligned table");
    BHI_REQUIRE(precision >= BHI_ANS_PRECISION && precision <= BHI_ANS_MAX_PRECISION, "rANS precision must be in [8, 12]");
    Layer L{A_rem, A_exp, exp_words, offsets, split_k, M, Nc};
    AnsArgs t{LUT, precision};
    return run_gemv<AnsCodec>(L, t, nullptr, X, Y, batch, static_cast<cudaStream_t>(stream));
}

int bhi_ans_decode(const uint8_t *A_rem, const uint32_t *A_exp, int64_t exp_words,
                   uint16_t *Y, const int32_t *offsets, const uint32_t *LUT, int precision,
                   int split_k, int M, int Nc, void *stream) {
    if (int rc = check_layer(A_rem, A_exp, exp_words, offsets, split_k, M, Nc)) return rc;
    BHI_REQUIRE(LUT && aligned(LUT, 4), "null or unaligned table");
    BHI_REQUIRE(precision >= BHI_ANS_PRECISION && precision <= BHI_ANS_MAX_PRECISION, "rANS precision must be in [8, 12]");
    Layer L{A_rem, A_exp, exp_words, offsets, split_k, M, Nc};
    AnsArgs t{LUT, precision};
    return run_decode<AnsCodec>(L, t, nullptr, Y, static_cast<cudaStream_t>(stream));
}

int bhi_huffman_encode(const uint8_t *data, int streams, int n, const uint8_t *LUT,
                       uint8_t *output, int32_t *output_lengths, void *stream) {
    BHI_REQUIRE(data && LUT && output && output_lengths, "null buffer");
    BHI_REQUIRE(streams >= 0 && n >= 0, "negative size");
    if (streams == 0) return BHI_OK;
    const int threads = 128;
    huffman_encode_chars_kernel<<<(streams + threads - 1) / threads, threads, 0, static_cast<cudaStream_t>(stream)>>>(
        data, streams, n, LUT, output, output_lengths);
    return launch_status("huffman_encode launch");
}

int bhi_ans_encode(const uint8_t *data, int streams, int n, const uint32_t *freq,
                   const uint32_t *cum, uint32_t *output, int32_t *output_lengths, void *stream) {
    BHI_REQUIRE(data && freq && cum && output && output_lengths, "null buffer");
    BHI_REQUIRE(streams >= 0 && n >= 0, "negative size");
    if (streams == 0) return BHI_OK;
    const int threads = 128;
    ans_encode_words_kernel<<<(streams + threads - 1) / threads, threads, 0, static_cast<cudaStream_t>(stream)>>>(
        data, streams, n, freq, cum, output, output_lengths);
    return launch_status("ans_encode launch");
}

int bhi_huffman_size_pass(const uint16_t *W, int M, int K, int split_k, const uint8_t *code_lengths,
                          int32_t *words_per_row, void *stream) {
    if (int rc = check_enc(W, M, K, split_k)) return rc;
    BHI_REQUIRE(code_lengths && words_per_row, "null buffer");
    EncGeom g{W, M, K, split_k, K / split_k};
    huffman_size_kernel<<<enc_blocks(M, split_k), kEncThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        g, code_lengths, words_per_row);
    return launch_status("huffman size pass launch");
}

int bhi_ans_size_pass(const uint16_t *W, int M, int K, int split_k, const uint32_t *freq,
                      const uint32_t *cum, int32_t *words_per_row, uint8_t *stream_words, void *stream) {
    if (int rc = check_enc(W, M, K, split_k)) return rc;
    BHI_REQUIRE(freq && cum && words_per_row && stream_words, "null buffer");
    EncGeom g{W, M, K, split_k, K / split_k};
    ans_size_kernel<<<enc_blocks(M, split_k), kEncThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        g, freq, cum, words_per_row, stream_words);
    return launch_status("rANS size pass launch");
}

int bhi_huffman_emit_pass(const uint16_t *W, int M, int K, int split_k, const uint8_t *code_lengths,
                          const uint32_t *code_values, const int32_t *offsets,
                          uint8_t *A_rem, uint32_t *A_exp, void *stream) {
    if (int rc = check_enc(W, M, K, split_k)) return rc;
    BHI_REQUIRE(code_lengths && code_values && offsets && A_rem && A_exp, "null buffer");
    BHI_REQUIRE(aligned(A_rem, 2) && aligned(A_exp, 4), "unaligned output");
    EncGeom g{W, M, K, split_k, K / split_k};
    huffman_emit_kernel<<<enc_blocks(M, split_k), kEncThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        g, code_lengths, code_values, offsets, A_rem, A_exp);
    return launch_status("huffman emit pass launch");
}

int bhi_ans_emit_pass(const uint16_t *W, int M, int K, int split_k, const uint32_t *freq,
                      const uint32_t *cum, const int32_t *offsets, const uint8_t *stream_words,
                      uint8_t *A_rem, uint32_t *A_exp, void *stream) {
    if (int rc = check_enc(W, M, K, split_k)) return rc;
    BHI_REQUIRE(freq && cum && offsets && stream_words && A_rem && A_exp, "null buffer");
    BHI_REQUIRE(aligned(A_rem, 2) && aligned(A_exp, 4), "unaligned output");
    EncGeom g{W, M, K, split_k, K / split_k};
    ans_emit_kernel<<<enc_blocks(M, split_k), kEncThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        g, freq, cum, offsets, stream_words, A_rem, A_exp);
    return launch_status("rANS emit pass launch");
}

}  // extern "C"
