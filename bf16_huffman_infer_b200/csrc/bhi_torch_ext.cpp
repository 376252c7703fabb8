// PyTorch stable-ABI glue: registers the operator schemas of the reference extension
// (bf16_huffman_infer/src/bf16_huffman_infer.cpp:28-36) under the same namespace and forwards
// each call to the C ABI of libbf16_huffman_b200.so.  No kernels and no CUDA headers here: the
// only torch facilities used are tensor metadata, the current stream and a device guard.
#define USE_CUDA
#include <Python.h>

#include <torch/csrc/inductor/aoti_torch/c/shim.h>
#include <torch/csrc/stable/accelerator.h>
#include <torch/csrc/stable/library.h>
#include <torch/csrc/stable/tensor.h>
#include <torch/headeronly/core/ScalarType.h>

#include <string>

#include "../../include/bf16_huffman_b200.h"

#ifndef BHI_TORCH_NAMESPACE
#define BHI_TORCH_NAMESPACE bf16_huffman_infer
#endif

extern "C" {
// An empty module: importing it loads this shared object, whose static initialisers register
// the operators (same arrangement as the reference's `_C`).
PyObject *PyInit__C(void) {
    static struct PyModuleDef def = {PyModuleDef_HEAD_INIT, "_C", nullptr, -1, nullptr, nullptr, nullptr, nullptr, nullptr};
    return PyModule_Create(&def);
}
}

namespace {

using torch::stable::Tensor;
using torch::headeronly::ScalarType;

Tensor arg(StableIValue *stack, int i) { return torch::stable::detail::to<Tensor>(stack[i]); }
int64_t iarg(StableIValue *stack, int i) { return torch::stable::detail::to<int64_t>(stack[i]); }

// The current stream of the tensor's device.  The low-level shim call is used because it is legal
// during CUDA-graph capture (the reference does the same, src/kernel.cu:30-38).
void *stream_of(const Tensor &t) {
    void *s = nullptr;
    TORCH_ERROR_CODE_CHECK(aoti_torch_get_current_cuda_stream(t.get_device_index(), &s));
    return s;
}

void want(const Tensor &t, ScalarType st, const char *name, int64_t min_dim = 1) {
    STD_TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
    STD_TORCH_CHECK(t.scalar_type() == st, name, " has the wrong dtype");
    STD_TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
    STD_TORCH_CHECK(t.dim() >= min_dim, name, " has too few dimensions");
}

void same_device(const Tensor &a, const Tensor &b, const char *name) {
    STD_TORCH_CHECK(a.get_device_index() == b.get_device_index(), name, " is on a different device");
}

void check(int rc) { STD_TORCH_CHECK(rc == BHI_OK, "bf16_huffman_b200: ", bhi_last_error()); }

template <class T> T *ptr(const Tensor &t) { return static_cast<T *>(t.data_ptr()); }

struct LayerView {
    int S, M, Nc;
    int64_t exp_words;
};

LayerView layer_of(const Tensor &rem, const Tensor &exp, const Tensor &offsets) {
    want(rem, ScalarType::Byte, "A_rem", 3);
    want(exp, ScalarType::Int, "A_exp");
    want(offsets, ScalarType::Int, "offsets");
    same_device(rem, exp, "A_exp");
    same_device(rem, offsets, "offsets");
    STD_TORCH_CHECK(rem.dim() == 3, "A_rem must be [split_k, M, Nc]");
    STD_TORCH_CHECK(offsets.numel() == rem.size(0) * rem.size(1), "offsets must hold split_k*M entries");
    return {static_cast<int>(rem.size(0)), static_cast<int>(rem.size(1)), static_cast<int>(rem.size(2)), exp.numel()};
}

void huff_tables(StableIValue *stack, int first, const Tensor &rem, const uint8_t *out[5]) {
    static const char *names[5] = {"LUT1", "LUT2", "LUT3", "LUT4", "code_lengths"};
    for (int i = 0; i < 5; i++) {
        Tensor t = arg(stack, first + i);
        want(t, ScalarType::Byte, names[i]);
        same_device(rem, t, names[i]);
        STD_TORCH_CHECK(t.numel() == 256, names[i], " must have 256 entries");
        out[i] = ptr<const uint8_t>(t);
    }
}

// gemv_bf16_huffman(A_rem, A_exp, X, Y(a!), offsets, LUT1, LUT2, LUT3, LUT4, code_lengths) -> ()
void boxed_gemv_bf16_huffman(StableIValue *stack, uint64_t, uint64_t) {
    Tensor rem = arg(stack, 0), exp = arg(stack, 1), X = arg(stack, 2), Y = arg(stack, 3), off = arg(stack, 4);
    LayerView v = layer_of(rem, exp, off);
    want(X, ScalarType::BFloat16, "X");
    want(Y, ScalarType::BFloat16, "Y", 2);
    same_device(rem, X, "X");
    same_device(rem, Y, "Y");
    const int64_t K = static_cast<int64_t>(v.S) * v.Nc;
    STD_TORCH_CHECK(X.numel() % K == 0, "X must hold whole rows of split_k*Nc values");
    const int64_t B = X.numel() / K;
    STD_TORCH_CHECK(B <= BHI_MAX_BATCH, "batch_size <= 8");
    STD_TORCH_CHECK(Y.numel() == B * v.M, "Y must be [batch, M]");
    const uint8_t *t[5];
    huff_tables(stack, 5, rem, t);
    torch::stable::accelerator::DeviceGuard guard(rem.get_device_index());
    check(bhi_gemv_bf16_huffman(ptr<const uint8_t>(rem), ptr<const uint32_t>(exp), v.exp_words, ptr<const uint16_t>(X),
                                ptr<uint16_t>(Y), ptr<const int32_t>(off), t[0], t[1], t[2], t[3], t[4], v.S, v.M,
                                v.Nc, static_cast<int>(B), stream_of(rem)));
}

// huffman_decode(A_rem, A_exp, Y(a!), offsets, LUT1, LUT2, LUT3, LUT4, code_lengths) -> ()
void boxed_huffman_decode(StableIValue *stack, uint64_t, uint64_t) {
    Tensor rem = arg(stack, 0), exp = arg(stack, 1), Y = arg(stack, 2), off = arg(stack, 3);
    LayerView v = layer_of(rem, exp, off);
    want(Y, ScalarType::BFloat16, "Y", 2);
    same_device(rem, Y, "Y");
    STD_TORCH_CHECK(Y.numel() == static_cast<int64_t>(v.S) * v.M * v.Nc, "Y must be [M, split_k*Nc]");
    const uint8_t *t[5];
    huff_tables(stack, 4, rem, t);
    torch::stable::accelerator::DeviceGuard guard(rem.get_device_index());
    check(bhi_huffman_decode(ptr<const uint8_t>(rem), ptr<const uint32_t>(exp), v.exp_words, ptr<uint16_t>(Y),
                             ptr<const int32_t>(off), t[0], t[1], t[2], t[3], t[4], v.S, v.M, v.Nc, stream_of(rem)));
}

// huffman_prepare(LUT1, LUT2, LUT3, LUT4, code_lengths, prepared(a!)) -> ()
void boxed_huffman_prepare(StableIValue *stack, uint64_t, uint64_t) {
    Tensor blob = arg(stack, 5);
    want(blob, ScalarType::Byte, "prepared");
    STD_TORCH_CHECK(blob.numel() == bhi_huffman_prepared_bytes(), "prepared must have bhi_huffman_prepared_bytes() bytes");
    const uint8_t *t[5];
    huff_tables(stack, 0, blob, t);
    torch::stable::accelerator::DeviceGuard guard(blob.get_device_index());
    check(bhi_huffman_prepare(t[0], t[1], t[2], t[3], t[4], ptr<uint8_t>(blob), stream_of(blob)));
}

// huffman_table_hint(prepared, pair_complete) -> ()
void boxed_huffman_table_hint(StableIValue *stack, uint64_t, uint64_t) {
    Tensor blob = arg(stack, 0);
    want(blob, ScalarType::Byte, "prepared");
    check(bhi_huffman_table_hint(ptr<const uint8_t>(blob), static_cast<int>(iarg(stack, 1))));
}

// Probability precision of an rANS table: it has 2^precision slots (the operator schemas carry no such argument).
int ans_precision_of(const Tensor &lut) {
    const int64_t n = lut.numel();
    int p = 0;
    while ((int64_t{1} << p) < n) p++;
    STD_TORCH_CHECK((int64_t{1} << p) == n && p >= BHI_ANS_PRECISION && p <= BHI_ANS_MAX_PRECISION,
                    "LUT must have 2^precision entries, 8 <= precision <= 12");
    return p;
}

// gemv_bf16_huffman_prepared(A_rem, A_exp, X, Y(a!), offsets, prepared) -> ()
void boxed_gemv_bf16_huffman_prepared(StableIValue *stack, uint64_t, uint64_t) {
    Tensor rem = arg(stack, 0), exp = arg(stack, 1), X = arg(stack, 2), Y = arg(stack, 3), off = arg(stack, 4),
           blob = arg(stack, 5);
    LayerView v = layer_of(rem, exp, off);
    want(X, ScalarType::BFloat16, "X");
    want(Y, ScalarType::BFloat16, "Y", 2);
    want(blob, ScalarType::Byte, "prepared");
    same_device(rem, X, "X");
    same_device(rem, Y, "Y");
    same_device(rem, blob, "prepared");
    STD_TORCH_CHECK(blob.numel() == bhi_huffman_prepared_bytes(), "prepared has the wrong size");
    const int64_t K = static_cast<int64_t>(v.S) * v.Nc;
    STD_TORCH_CHECK(X.numel() % K == 0, "X must hold whole rows of split_k*Nc values");
    const int64_t B = X.numel() / K;
    STD_TORCH_CHECK(B <= BHI_MAX_BATCH, "batch_size <= 8");
    STD_TORCH_CHECK(Y.numel() == B * v.M, "Y must be [batch, M]");
    torch::stable::accelerator::DeviceGuard guard(rem.get_device_index());
    check(bhi_gemv_bf16_huffman_prepared(ptr<const uint8_t>(rem), ptr<const uint32_t>(exp), v.exp_words,
                                         ptr<const uint16_t>(X), ptr<uint16_t>(Y), ptr<const int32_t>(off),
                                         ptr<const uint8_t>(blob), v.S, v.M, v.Nc, static_cast<int>(B), stream_of(rem)));
}

// huffman_decode_prepared(A_rem, A_exp, Y(a!), offsets, prepared) -> ()
void boxed_huffman_decode_prepared(StableIValue *stack, uint64_t, uint64_t) {
    Tensor rem = arg(stack, 0), exp = arg(stack, 1), Y = arg(stack, 2), off = arg(stack, 3), blob = arg(stack, 4);
    LayerView v = layer_of(rem, exp, off);
    want(Y, ScalarType::BFloat16, "Y", 2);
    want(blob, ScalarType::Byte, "prepared");
    same_device(rem, Y, "Y");
    same_device(rem, blob, "prepared");
    STD_TORCH_CHECK(blob.numel() == bhi_huffman_prepared_bytes(), "prepared has the wrong size");
    STD_TORCH_CHECK(Y.numel() == static_cast<int64_t>(v.S) * v.M * v.Nc, "Y must be [M, split_k*Nc]");
    torch::stable::accelerator::DeviceGuard guard(rem.get_device_index());
    check(bhi_huffman_decode_prepared(ptr<const uint8_t>(rem), ptr<const uint32_t>(exp), v.exp_words, ptr<uint16_t>(Y),
                                      ptr<const int32_t>(off), ptr<const uint8_t>(blob), v.S, v.M, v.Nc, stream_of(rem)));
}

// gemv_bf16_ans(A_rem, A_exp, X, Y(a!), offsets, LUT) -> ()
void boxed_gemv_bf16_ans(StableIValue *stack, uint64_t, uint64_t) {
    Tensor rem = arg(stack, 0), exp = arg(stack, 1), X = arg(stack, 2), Y = arg(stack, 3), off = arg(stack, 4),
           lut = arg(stack, 5);
    LayerView v = layer_of(rem, exp, off);
    want(X, ScalarType::BFloat16, "X");
    want(Y, ScalarType::BFloat16, "Y", 2);
    want(lut, ScalarType::Int, "LUT");
    same_device(rem, X, "X");
    same_device(rem, Y, "Y");
    same_device(rem, lut, "LUT");
    const int precision = ans_precision_of(lut);
    const int64_t K = static_cast<int64_t>(v.S) * v.Nc;
    STD_TORCH_CHECK(X.numel() % K == 0, "X must hold whole rows of split_k*Nc values");
    const int64_t B = X.numel() / K;
    STD_TORCH_CHECK(B <= BHI_MAX_BATCH, "batch_size <= 8");
    STD_TORCH_CHECK(Y.numel() == B * v.M, "Y must be [batch, M]");
    torch::stable::accelerator::DeviceGuard guard(rem.get_device_index());
    check(bhi_gemv_bf16_ans(ptr<const uint8_t>(rem), ptr<const uint32_t>(exp), v.exp_words, ptr<const uint16_t>(X),
                            ptr<uint16_t>(Y), ptr<const int32_t>(off), ptr<const uint32_t>(lut), precision, v.S, v.M, v.Nc,
                            static_cast<int>(B), stream_of(rem)));
}

// linear_bf16_huffman_prepared(A_rem, A_exp, X, Y(a!), offsets, prepared) -> ()   (up to 128 rows of X)
void boxed_linear_bf16_huffman_prepared(StableIValue *stack, uint64_t, uint64_t) {
    Tensor rem = arg(stack, 0), exp = arg(stack, 1), X = arg(stack, 2), Y = arg(stack, 3), off = arg(stack, 4),
           blob = arg(stack, 5);
    LayerView v = layer_of(rem, exp, off);
    want(X, ScalarType::BFloat16, "X");
    want(Y, ScalarType::BFloat16, "Y", 2);
    want(blob, ScalarType::Byte, "prepared");
    same_device(rem, X, "X");
    same_device(rem, Y, "Y");
    same_device(rem, blob, "prepared");
    STD_TORCH_CHECK(blob.numel() == bhi_huffman_prepared_bytes(), "prepared has the wrong size");
    const int64_t K = static_cast<int64_t>(v.S) * v.Nc;
    STD_TORCH_CHECK(X.numel() % K == 0, "X must hold whole rows of split_k*Nc values");
    const int64_t B = X.numel() / K;
    STD_TORCH_CHECK(B <= BHI_MAX_LINEAR_BATCH, "batch_size <= 128");
    STD_TORCH_CHECK(Y.numel() == B * v.M, "Y must be [batch, M]");
    torch::stable::accelerator::DeviceGuard guard(rem.get_device_index());
    check(bhi_linear_bf16_huffman_prepared(ptr<const uint8_t>(rem), ptr<const uint32_t>(exp), v.exp_words,
                                           ptr<const uint16_t>(X), ptr<uint16_t>(Y), ptr<const int32_t>(off),
                                           ptr<const uint8_t>(blob), v.S, v.M, v.Nc, static_cast<int>(B), stream_of(rem)));
}

// linear_bf16_ans(A_rem, A_exp, X, Y(a!), offsets, LUT) -> ()   (up to 128 rows of X)
void boxed_linear_bf16_ans(StableIValue *stack, uint64_t, uint64_t) {
    Tensor rem = arg(stack, 0), exp = arg(stack, 1), X = arg(stack, 2), Y = arg(stack, 3), off = arg(stack, 4),
           lut = arg(stack, 5);
    LayerView v = layer_of(rem, exp, off);
    want(X, ScalarType::BFloat16, "X");
    want(Y, ScalarType::BFloat16, "Y", 2);
    want(lut, ScalarType::Int, "LUT");
    same_device(rem, X, "X");
    same_device(rem, Y, "Y");
    same_device(rem, lut, "LUT");
    const int precision = ans_precision_of(lut);
    const int64_t K = static_cast<int64_t>(v.S) * v.Nc;
    STD_TORCH_CHECK(X.numel() % K == 0, "X must hold whole rows of split_k*Nc values");
    const int64_t B = X.numel() / K;
    STD_TORCH_CHECK(B <= BHI_MAX_LINEAR_BATCH, "batch_size <= 128");
    STD_TORCH_CHECK(Y.numel() == B * v.M, "Y must be [batch, M]");
    torch::stable::accelerator::DeviceGuard guard(rem.get_device_index());
    check(bhi_linear_bf16_ans(ptr<const uint8_t>(rem), ptr<const uint32_t>(exp), v.exp_words, ptr<const uint16_t>(X),
                              ptr<uint16_t>(Y), ptr<const int32_t>(off), ptr<const uint32_t>(lut), precision, v.S, v.M, v.Nc,
                              static_cast<int>(B), stream_of(rem)));
}

// Fills the C descriptor from a CPU int64 tensor [3 * world + 1]: y pointers, ready pointers, done
// pointers (one per rank each), then the local launch counter.
bhi_exchange_t exchange_of(const Tensor &peers, int64_t rank, int64_t row_base, int64_t m_total) {
    STD_TORCH_CHECK(!peers.is_cuda() && peers.scalar_type() == ScalarType::Long && peers.is_contiguous(),
                    "peers must be a contiguous CPU int64 tensor");
    const int64_t n = peers.numel();
    STD_TORCH_CHECK(n >= 4 && (n - 1) % 3 == 0 && (n - 1) / 3 <= BHI_MAX_PEERS, "peers must hold 3 * world + 1 pointers");
    const int world = static_cast<int>((n - 1) / 3);
    const int64_t *v = static_cast<const int64_t *>(peers.data_ptr());
    bhi_exchange_t ex = {};
    ex.world = world;
    ex.rank = static_cast<int>(rank);
    ex.row_base = static_cast<int>(row_base);
    ex.M_total = static_cast<int>(m_total);
    for (int r = 0; r < world; r++) {
        ex.y[r] = reinterpret_cast<uint16_t *>(v[r]);
        ex.ready[r] = reinterpret_cast<uint32_t *>(v[world + r]);
        ex.done[r] = reinterpret_cast<uint32_t *>(v[2 * world + r]);
    }
    ex.launches = reinterpret_cast<uint32_t *>(v[3 * world]);
    return ex;
}

// gemv_bf16_huffman_exchange(A_rem, A_exp, X, offsets, prepared, peers, rank, row_base, m_total) -> ()
void boxed_gemv_bf16_huffman_exchange(StableIValue *stack, uint64_t, uint64_t) {
    Tensor rem = arg(stack, 0), exp = arg(stack, 1), X = arg(stack, 2), off = arg(stack, 3), blob = arg(stack, 4),
           peers = arg(stack, 5);
    LayerView v = layer_of(rem, exp, off);
    want(X, ScalarType::BFloat16, "X");
    want(blob, ScalarType::Byte, "prepared");
    same_device(rem, X, "X");
    same_device(rem, blob, "prepared");
    STD_TORCH_CHECK(blob.numel() == bhi_huffman_prepared_bytes(), "prepared has the wrong size");
    const int64_t K = static_cast<int64_t>(v.S) * v.Nc;
    STD_TORCH_CHECK(X.numel() % K == 0, "X must hold whole rows of split_k*Nc values");
    const int64_t B = X.numel() / K;
    STD_TORCH_CHECK(B <= BHI_MAX_BATCH, "batch_size <= 8");
    const bhi_exchange_t ex = exchange_of(peers, iarg(stack, 6), iarg(stack, 7), iarg(stack, 8));
    torch::stable::accelerator::DeviceGuard guard(rem.get_device_index());
    check(bhi_gemv_bf16_huffman_exchange(ptr<const uint8_t>(rem), ptr<const uint32_t>(exp), v.exp_words, ptr<const uint16_t>(X),
                                         ptr<const int32_t>(off), ptr<const uint8_t>(blob), v.S, v.M, v.Nc,
                                         static_cast<int>(B), &ex, stream_of(rem)));
}

// gemv_bf16_ans_exchange(A_rem, A_exp, X, offsets, LUT, peers, rank, row_base, m_total) -> ()
void boxed_gemv_bf16_ans_exchange(StableIValue *stack, uint64_t, uint64_t) {
    Tensor rem = arg(stack, 0), exp = arg(stack, 1), X = arg(stack, 2), off = arg(stack, 3), lut = arg(stack, 4),
           peers = arg(stack, 5);
    LayerView v = layer_of(rem, exp, off);
    want(X, ScalarType::BFloat16, "X");
    want(lut, ScalarType::Int, "LUT");
    same_device(rem, X, "X");
    same_device(rem, lut, "LUT");
    const int precision = ans_precision_of(lut);
    const int64_t K = static_cast<int64_t>(v.S) * v.Nc;
    STD_TORCH_CHECK(X.numel() % K == 0, "X must hold whole rows of split_k*Nc values");
    const int64_t B = X.numel() / K;
    STD_TORCH_CHECK(B <= BHI_MAX_BATCH, "batch_size <= 8");
    const bhi_exchange_t ex = exchange_of(peers, iarg(stack, 6), iarg(stack, 7), iarg(stack, 8));
    torch::stable::accelerator::DeviceGuard guard(rem.get_device_index());
    check(bhi_gemv_bf16_ans_exchange(ptr<const uint8_t>(rem), ptr<const uint32_t>(exp), v.exp_words, ptr<const uint16_t>(X),
                                     ptr<const int32_t>(off), ptr<const uint32_t>(lut), precision, v.S, v.M, v.Nc, static_cast<int>(B),
                                     &ex, stream_of(rem)));
}

// ans_decode(A_rem, A_exp, Y(a!), offsets, LUT) -> ()
void boxed_ans_decode(StableIValue *stack, uint64_t, uint64_t) {
    Tensor rem = arg(stack, 0), exp = arg(stack, 1), Y = arg(stack, 2), off = arg(stack, 3), lut = arg(stack, 4);
    LayerView v = layer_of(rem, exp, off);
    want(Y, ScalarType::BFloat16, "Y", 2);
    want(lut, ScalarType::Int, "LUT");
    same_device(rem, Y, "Y");
    same_device(rem, lut, "LUT");
    const int precision = ans_precision_of(lut);
    STD_TORCH_CHECK(Y.numel() == static_cast<int64_t>(v.S) * v.M * v.Nc, "Y must be [M, split_k*Nc]");
    torch::stable::accelerator::DeviceGuard guard(rem.get_device_index());
    check(bhi_ans_decode(ptr<const uint8_t>(rem), ptr<const uint32_t>(exp), v.exp_words, ptr<uint16_t>(Y),
                         ptr<const int32_t>(off), ptr<const uint32_t>(lut), precision, v.S, v.M, v.Nc, stream_of(rem)));
}

// huffman_encode(data, LUT, output(a!), output_lengths(b!)) -> ()
void boxed_huffman_encode(StableIValue *stack, uint64_t, uint64_t) {
    Tensor data = arg(stack, 0), lut = arg(stack, 1), out = arg(stack, 2), lens = arg(stack, 3);
    want(data, ScalarType::Byte, "data", 2);
    want(lut, ScalarType::Byte, "LUT", 2);
    want(out, ScalarType::Byte, "output", 2);
    want(lens, ScalarType::Int, "output_lengths");
    same_device(data, lut, "LUT");
    same_device(data, out, "output");
    same_device(data, lens, "output_lengths");
    STD_TORCH_CHECK(lut.numel() == 256 * 32, "LUT must be [256, 32]");
    STD_TORCH_CHECK(out.numel() == data.numel() * 32, "output must be [streams, 32*n]");
    STD_TORCH_CHECK(lens.numel() == data.size(0), "output_lengths must be [streams]");
    torch::stable::accelerator::DeviceGuard guard(data.get_device_index());
    check(bhi_huffman_encode(ptr<const uint8_t>(data), static_cast<int>(data.size(0)), static_cast<int>(data.size(1)),
                             ptr<const uint8_t>(lut), ptr<uint8_t>(out), ptr<int32_t>(lens), stream_of(data)));
}

// ans_encode(data, freq, cum, output(a!), output_lengths(b!)) -> ()
void boxed_ans_encode(StableIValue *stack, uint64_t, uint64_t) {
    Tensor data = arg(stack, 0), freq = arg(stack, 1), cum = arg(stack, 2), out = arg(stack, 3), lens = arg(stack, 4);
    want(data, ScalarType::Byte, "data", 2);
    want(freq, ScalarType::Int, "freq");
    want(cum, ScalarType::Int, "cum");
    want(out, ScalarType::Int, "output", 2);
    want(lens, ScalarType::Int, "output_lengths");
    same_device(data, freq, "freq");
    same_device(data, cum, "cum");
    same_device(data, out, "output");
    same_device(data, lens, "output_lengths");
    STD_TORCH_CHECK(freq.numel() == 256 && cum.numel() == 256, "freq and cum must have 256 entries");
    STD_TORCH_CHECK(out.numel() == data.numel() * 8, "output must be [streams, 8*n]");
    STD_TORCH_CHECK(lens.numel() == data.size(0), "output_lengths must be [streams]");
    torch::stable::accelerator::DeviceGuard guard(data.get_device_index());
    check(bhi_ans_encode(ptr<const uint8_t>(data), static_cast<int>(data.size(0)), static_cast<int>(data.size(1)),
                         ptr<const uint32_t>(freq), ptr<const uint32_t>(cum), ptr<uint32_t>(out), ptr<int32_t>(lens),
                         stream_of(data)));
}

// set_launch_overlap(int on) -> int
void boxed_set_launch_overlap(StableIValue *stack, uint64_t, uint64_t) {
    const int64_t prev = bhi_set_launch_overlap(static_cast<int>(iarg(stack, 0)));
    stack[0] = torch::stable::detail::from(prev);
}

// ---- whole-layer encoder (no counterpart operator in the reference) -------------------------------
struct EncView {
    int M, K, S;
};

EncView enc_of(const Tensor &W, int64_t split_k) {
    want(W, ScalarType::BFloat16, "W", 2);
    STD_TORCH_CHECK(W.dim() == 2, "W must be [M, K]");
    STD_TORCH_CHECK(split_k >= 1 && W.size(1) % split_k == 0, "split_k must divide K");
    return {static_cast<int>(W.size(0)), static_cast<int>(W.size(1)), static_cast<int>(split_k)};
}

// huffman_size_pass(W, split_k, code_lengths, words_per_row(a!)) -> ()
void boxed_huffman_size_pass(StableIValue *stack, uint64_t, uint64_t) {
    Tensor W = arg(stack, 0), len = arg(stack, 2), rows = arg(stack, 3);
    EncView v = enc_of(W, iarg(stack, 1));
    want(len, ScalarType::Byte, "code_lengths");
    want(rows, ScalarType::Int, "words_per_row");
    same_device(W, len, "code_lengths");
    same_device(W, rows, "words_per_row");
    STD_TORCH_CHECK(len.numel() == 256, "code_lengths must have 256 entries");
    STD_TORCH_CHECK(rows.numel() == static_cast<int64_t>(v.S) * v.M, "words_per_row must be [split_k, M]");
    torch::stable::accelerator::DeviceGuard guard(W.get_device_index());
    check(bhi_huffman_size_pass(ptr<const uint16_t>(W), v.M, v.K, v.S, ptr<const uint8_t>(len), ptr<int32_t>(rows),
                                stream_of(W)));
}

// huffman_emit_pass(W, split_k, code_lengths, code_values, offsets, rem(a!), exp(b!)) -> ()
void boxed_huffman_emit_pass(StableIValue *stack, uint64_t, uint64_t) {
    Tensor W = arg(stack, 0), len = arg(stack, 2), val = arg(stack, 3), off = arg(stack, 4), rem = arg(stack, 5),
           exp = arg(stack, 6);
    EncView v = enc_of(W, iarg(stack, 1));
    want(len, ScalarType::Byte, "code_lengths");
    want(val, ScalarType::Int, "code_values");
    want(off, ScalarType::Int, "offsets");
    want(rem, ScalarType::Byte, "rem");
    want(exp, ScalarType::Int, "exp");
    for (const Tensor *t : {&len, &val, &off, &rem, &exp}) same_device(W, *t, "an encoder buffer");
    STD_TORCH_CHECK(len.numel() == 256 && val.numel() == 256, "code tables must have 256 entries");
    STD_TORCH_CHECK(off.numel() == static_cast<int64_t>(v.S) * v.M, "offsets must be [split_k, M]");
    STD_TORCH_CHECK(rem.numel() == W.numel(), "rem must be [split_k, M, K/split_k]");
    torch::stable::accelerator::DeviceGuard guard(W.get_device_index());
    check(bhi_huffman_emit_pass(ptr<const uint16_t>(W), v.M, v.K, v.S, ptr<const uint8_t>(len), ptr<const uint32_t>(val),
                                ptr<const int32_t>(off), ptr<uint8_t>(rem), ptr<uint32_t>(exp), stream_of(W)));
}

// ans_size_pass(W, split_k, freq, cum, words_per_row(a!), stream_words(b!)) -> ()
void boxed_ans_size_pass(StableIValue *stack, uint64_t, uint64_t) {
    Tensor W = arg(stack, 0), freq = arg(stack, 2), cum = arg(stack, 3), rows = arg(stack, 4), sw = arg(stack, 5);
    EncView v = enc_of(W, iarg(stack, 1));
    want(freq, ScalarType::Int, "freq");
    want(cum, ScalarType::Int, "cum");
    want(rows, ScalarType::Int, "words_per_row");
    want(sw, ScalarType::Byte, "stream_words");
    for (const Tensor *t : {&freq, &cum, &rows, &sw}) same_device(W, *t, "an encoder buffer");
    STD_TORCH_CHECK(freq.numel() == 256 && cum.numel() == 256, "freq and cum must have 256 entries");
    STD_TORCH_CHECK(rows.numel() == static_cast<int64_t>(v.S) * v.M, "words_per_row must be [split_k, M]");
    STD_TORCH_CHECK(sw.numel() == static_cast<int64_t>(v.S) * v.M * 64, "stream_words must be [split_k, M, 64]");
    torch::stable::accelerator::DeviceGuard guard(W.get_device_index());
    check(bhi_ans_size_pass(ptr<const uint16_t>(W), v.M, v.K, v.S, ptr<const uint32_t>(freq), ptr<const uint32_t>(cum),
                            ptr<int32_t>(rows), ptr<uint8_t>(sw), stream_of(W)));
}

// ans_emit_pass(W, split_k, freq, cum, offsets, stream_words, rem(a!), exp(b!)) -> ()
void boxed_ans_emit_pass(StableIValue *stack, uint64_t, uint64_t) {
    Tensor W = arg(stack, 0), freq = arg(stack, 2), cum = arg(stack, 3), off = arg(stack, 4), sw = arg(stack, 5),
           rem = arg(stack, 6), exp = arg(stack, 7);
    EncView v = enc_of(W, iarg(stack, 1));
    want(freq, ScalarType::Int, "freq");
    want(cum, ScalarType::Int, "cum");
    want(off, ScalarType::Int, "offsets");
    want(sw, ScalarType::Byte, "stream_words");
    want(rem, ScalarType::Byte, "rem");
    want(exp, ScalarType::Int, "exp");
    for (const Tensor *t : {&freq, &cum, &off, &sw, &rem, &exp}) same_device(W, *t, "an encoder buffer");
    STD_TORCH_CHECK(freq.numel() == 256 && cum.numel() == 256, "freq and cum must have 256 entries");
    STD_TORCH_CHECK(off.numel() == static_cast<int64_t>(v.S) * v.M, "offsets must be [split_k, M]");
    STD_TORCH_CHECK(sw.numel() == static_cast<int64_t>(v.S) * v.M * 64, "stream_words must be [split_k, M, 64]");
    STD_TORCH_CHECK(rem.numel() == W.numel(), "rem must be [split_k, M, K/split_k]");
    torch::stable::accelerator::DeviceGuard guard(W.get_device_index());
    check(bhi_ans_emit_pass(ptr<const uint16_t>(W), v.M, v.K, v.S, ptr<const uint32_t>(freq), ptr<const uint32_t>(cum),
                            ptr<const int32_t>(off), ptr<const uint8_t>(sw), ptr<uint8_t>(rem), ptr<uint32_t>(exp),
                            stream_of(W)));
}

}  // namespace

STABLE_TORCH_LIBRARY(BHI_TORCH_NAMESPACE, m) {
    // the six operators of the reference, schemas verbatim
    m.def("gemv_bf16_huffman(Tensor A_rem, Tensor A_exp, Tensor X, Tensor(a!) Y, Tensor offsets, Tensor LUT1, Tensor LUT2, Tensor LUT3, Tensor LUT4, Tensor code_lengths) -> ()");
    m.def("huffman_encode(Tensor data, Tensor LUT, Tensor(a!) output, Tensor(b!) output_lengths) -> ()");
    m.def("huffman_decode(Tensor A_rem, Tensor A_exp, Tensor(a!) Y, Tensor offsets, Tensor LUT1, Tensor LUT2, Tensor LUT3, Tensor LUT4, Tensor code_lengths) -> ()");
    m.def("gemv_bf16_ans(Tensor A_rem, Tensor A_exp, Tensor X, Tensor(a!) Y, Tensor offsets, Tensor LUT) -> ()");
    m.def("ans_encode(Tensor data, Tensor freq, Tensor cum, Tensor(a!) output, Tensor(b!) output_lengths) -> ()");
    m.def("ans_decode(Tensor A_rem, Tensor A_exp, Tensor(a!) Y, Tensor offsets, Tensor LUT) -> ()");
    // prepared Huffman tables
    m.def("huffman_prepare(Tensor LUT1, Tensor LUT2, Tensor LUT3, Tensor LUT4, Tensor code_lengths, Tensor(a!) prepared) -> ()");
    m.def("huffman_table_hint(Tensor prepared, int pair_complete) -> ()");
    m.def("gemv_bf16_huffman_prepared(Tensor A_rem, Tensor A_exp, Tensor X, Tensor(a!) Y, Tensor offsets, Tensor prepared) -> ()");
    m.def("huffman_decode_prepared(Tensor A_rem, Tensor A_exp, Tensor(a!) Y, Tensor offsets, Tensor prepared) -> ()");
    m.def("linear_bf16_huffman_prepared(Tensor A_rem, Tensor A_exp, Tensor X, Tensor(a!) Y, Tensor offsets, Tensor prepared) -> ()");
    m.def("linear_bf16_ans(Tensor A_rem, Tensor A_exp, Tensor X, Tensor(a!) Y, Tensor offsets, Tensor LUT) -> ()");
    m.def("gemv_bf16_huffman_exchange(Tensor A_rem, Tensor A_exp, Tensor X, Tensor offsets, Tensor prepared, Tensor peers, int rank, int row_base, int m_total) -> ()");
    m.def("gemv_bf16_ans_exchange(Tensor A_rem, Tensor A_exp, Tensor X, Tensor offsets, Tensor LUT, Tensor peers, int rank, int row_base, int m_total) -> ()");
    m.def("set_launch_overlap(int on) -> int");
    // whole-layer encoder
    m.def("huffman_size_pass(Tensor W, int split_k, Tensor code_lengths, Tensor(a!) words_per_row) -> ()");
    m.def("huffman_emit_pass(Tensor W, int split_k, Tensor code_lengths, Tensor code_values, Tensor offsets, Tensor(a!) rem, Tensor(b!) exp) -> ()");
    m.def("ans_size_pass(Tensor W, int split_k, Tensor freq, Tensor cum, Tensor(a!) words_per_row, Tensor(b!) stream_words) -> ()");
    m.def("ans_emit_pass(Tensor W, int split_k, Tensor freq, Tensor cum, Tensor offsets, Tensor stream_words, Tensor(a!) rem, Tensor(b!) exp) -> ()");
}

STABLE_TORCH_LIBRARY_IMPL(BHI_TORCH_NAMESPACE, CompositeExplicitAutograd, m) {
    m.impl("set_launch_overlap", &boxed_set_launch_overlap);
}

STABLE_TORCH_LIBRARY_IMPL(BHI_TORCH_NAMESPACE, CUDA, m) {
    m.impl("gemv_bf16_huffman", &boxed_gemv_bf16_huffman);
    m.impl("huffman_encode", &boxed_huffman_encode);
    m.impl("huffman_decode", &boxed_huffman_decode);
    m.impl("gemv_bf16_ans", &boxed_gemv_bf16_ans);
    m.impl("ans_encode", &boxed_ans_encode);
    m.impl("ans_decode", &boxed_ans_decode);
    m.impl("huffman_prepare", &boxed_huffman_prepare);
    m.impl("huffman_table_hint", &boxed_huffman_table_hint);
    m.impl("gemv_bf16_huffman_prepared", &boxed_gemv_bf16_huffman_prepared);
    m.impl("huffman_decode_prepared", &boxed_huffman_decode_prepared);
    m.impl("linear_bf16_huffman_prepared", &boxed_linear_bf16_huffman_prepared);
    m.impl("linear_bf16_ans", &boxed_linear_bf16_ans);
    m.impl("gemv_bf16_huffman_exchange", &boxed_gemv_bf16_huffman_exchange);
    m.impl("gemv_bf16_ans_exchange", &boxed_gemv_bf16_ans_exchange);
    m.impl("huffman_size_pass", &boxed_huffman_size_pass);
    m.impl("huffman_emit_pass", &boxed_huffman_emit_pass);
    m.impl("ans_size_pass", &boxed_ans_size_pass);
    m.impl("ans_emit_pass", &boxed_ans_emit_pass);
}
