"""The exchange entry point whose counters live inside the library: same results as the entry point that
takes caller-owned counters, on two calls in a row, without touching the device allocator."""
import ctypes as C
import os
import sys

import pytest
import torch

from _util import ROOT, Abi, bits_of, make_input, make_weight, tables_for, to_device

sys.path.insert(0, os.path.join(ROOT, "oracle"))
import oracle  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class Exchange(C.Structure):
    _fields_ = [("world", C.c_int), ("rank", C.c_int), ("row_base", C.c_int), ("M_total", C.c_int),
                ("y", C.c_void_p * 8), ("ready", C.c_void_p * 8), ("done", C.c_void_p * 8), ("launches", C.c_void_p)]


def test_static_counters_match_caller_owned_counters():
    abi = Abi()
    M, K, S = 640, 4096, 1
    Wb = bits_of(make_weight(M, K, 21))
    tabs = tables_for("huffman", oracle.histogram(Wb))
    rem, exp, offsets, _ = oracle.compress(Wb, "huffman", tabs, split_k=S)
    w = to_device(dict(rem=rem, exp=exp, offsets=offsets, **{k: tabs[k] for k in ("LUT1", "LUT2", "LUT3", "LUT4", "code_lengths")}), DEV)
    blob = abi.prepare(w)
    p = abi.p
    counters = torch.zeros(3, 32, dtype=torch.int32, device=DEV)
    y_ref = torch.zeros(8, M, dtype=torch.bfloat16, device=DEV)
    y_new = torch.zeros(8, M, dtype=torch.bfloat16, device=DEV)
    ex = Exchange(world=1, rank=0, row_base=0, M_total=M)
    ex.y[0] = y_ref.data_ptr()
    ex.ready[0] = counters[0].data_ptr()
    ex.done[0] = counters[1].data_ptr()
    ex.launches = counters[2].data_ptr()
    words = C.c_int64(w["exp"].numel())

    def both(x, slot):
        B = x.shape[0]
        abi.check(abi.lib.bhi_gemv_bf16_huffman_exchange(p(w["rem"]), p(w["exp"]), words, p(x), p(w["offsets"]), p(blob),
                                                         S, M, K // S, B, C.byref(ex), abi.stream()))
        abi.check(abi.lib.bhi_gemv_bf16_huffman_exchange_static(p(w["rem"]), p(w["exp"]), words, p(x), p(y_new), p(w["offsets"]),
                                                                p(blob), S, M, K // S, B, slot, abi.stream()))
        torch.cuda.synchronize()
        return y_ref[:B].clone(), y_new[:B].clone()

    x1, x2 = make_input(3, K, 1).to(DEV), make_input(3, K, 2).to(DEV)
    both(x1, 7)                                       # set-up happens here (address lookup, counters cleared)
    torch.cuda.synchronize()
    for x in (x1, x2):                                # two calls in a row on the same slot
        a, b = both(x, 7)
        assert torch.equal(a, b)
        assert not torch.equal(a, torch.zeros_like(a))
    a, b = both(x1, 1023)                             # the last slot works, independently of slot 7
    assert torch.equal(a, b)
    # nothing is allocated: free device memory is the same around calls that involve no torch allocation
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for slot in (7, 7, 500):
        abi.check(abi.lib.bhi_gemv_bf16_huffman_exchange_static(p(w["rem"]), p(w["exp"]), words, p(x2), p(y_new), p(w["offsets"]),
                                                                p(blob), S, M, K // S, 3, slot, abi.stream()))
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, "device memory was allocated"
    status = C.c_int(-1)
    abi.check(abi.lib.bhi_debug_status(C.byref(status)))
    assert status.value == 0
    for bad in (-1, 1024):
        rc = abi.lib.bhi_gemv_bf16_huffman_exchange_static(p(w["rem"]), p(w["exp"]), words, p(x1), p(y_new), p(w["offsets"]),
                                                           p(blob), S, M, K // S, 3, bad, abi.stream())
        assert rc == 3 and b"layer_slot" in abi.lib.bhi_last_error()
