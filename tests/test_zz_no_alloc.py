"""The entry point that allocates nothing (csrc/no_alloc.h): the greedy choice
with its scratch inside the library, for callers that cannot allocate device
memory (code under stream capture, hosts with a fixed memory budget, C callers
without torch).  It is called here the way such a caller would: through the
exported C symbol, with raw pointers, and compared with the entry point the
engine uses, on two calls in a row (the second meets what the first left in the
shared scratch).  This file is collected last on purpose."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_argmax_without_allocation_matches_the_engine_entry_point():
    from tokenizer_b200.kernels import load_library, ops

    lib = load_library("sampling.cu")
    lib.tokb200_argmax_no_alloc.restype = ctypes.c_int
    lib.tokb200_argmax_no_alloc.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                            ctypes.c_void_p, ctypes.c_void_p]
    lib.tokb200_no_alloc_error.restype = ctypes.c_char_p
    lib.tokb200_no_alloc_error.argtypes = [ctypes.c_int]
    limit = lib.tokb200_argmax_no_alloc_max_rows()
    assert limit == 256

    device = torch.device("cuda:0")
    with torch.cuda.device(device):
        stream = torch.cuda.current_stream().cuda_stream
        generator = torch.Generator().manual_seed(5)
        for call, (rows, vocab) in enumerate([(7, 151936), (64, 3001)]):
            logits = torch.randn(rows, vocab, generator=generator).to(device)
            logits[0, 11] = logits[0, vocab - 5] = 99.0       # ties keep the lower id
            logits[rows - 1, vocab - 1] = 100.0               # the last id of the last row
            want = torch.empty(rows, dtype=torch.int32, device=device)
            ops.argmax(logits, want)                          # the engine's entry point
            got = torch.full((rows,), -7, dtype=torch.int32, device=device)
            before = torch.cuda.memory_allocated(device)
            status = lib.tokb200_argmax_no_alloc(logits.data_ptr(), rows, vocab, got.data_ptr(), stream)
            assert status == 0, lib.tokb200_no_alloc_error(status).decode()
            torch.cuda.synchronize()
            assert torch.cuda.memory_allocated(device) == before
            assert got.tolist() == want.tolist(), f"call {call}"
            assert got[0].item() == 11 and got[rows - 1].item() == vocab - 1
            assert got.tolist() == logits.argmax(dim=1).tolist()

        # sizes beyond the built-in scratch are refused, with a reason, and nothing runs
        big = torch.zeros(limit + 1, 8, device=device)
        out = torch.full((limit + 1,), -7, dtype=torch.int32, device=device)
        status = lib.tokb200_argmax_no_alloc(big.data_ptr(), limit + 1, 8, out.data_ptr(), stream)
        assert status == -1 and b"256" in lib.tokb200_no_alloc_error(status)
        assert lib.tokb200_argmax_no_alloc(big.data_ptr(), 4, 0, out.data_ptr(), stream) == -1
        assert lib.tokb200_argmax_no_alloc(None, 4, 8, out.data_ptr(), stream) == -1
        torch.cuda.synchronize()
        assert out.tolist() == [-7] * (limit + 1)
        # exactly the limit still runs
        status = lib.tokb200_argmax_no_alloc(big.data_ptr(), limit, 8, out.data_ptr(), stream)
        assert status == 0
        torch.cuda.synchronize()
        assert out[:limit].tolist() == [0] * limit
