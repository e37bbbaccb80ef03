"""The allocation-free arg-max entry point (fixed device scratch) against the regular entry point.
Collected last on purpose: it must give the same answer alone and after every other GPU test."""
import ctypes
import gc

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, logits, out):
    dt = 2 if logits.dtype == torch.float32 else (1 if logits.dtype == torch.bfloat16 else 0)
    lib.telb_argmax_static.restype = ctypes.c_int
    return lib.telb_argmax_static(ctypes.c_void_p(logits.data_ptr()), ctypes.c_void_p(out.data_ptr()), ctypes.c_int(logits.shape[0]),
                                  ctypes.c_int(logits.shape[1]), ctypes.c_longlong(logits.stride(0)), ctypes.c_int(dt),
                                  ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("rows,vocab", [(1, 151936), (8, 32000), (64, 151936), (256, 5000), (3, 100)])
def test_static_argmax_matches_regular_entry_point(dtype, rows, vocab):
    from tensorrt_edge_llm_b200.ops import cuda
    lib = cuda.lib()
    g = torch.Generator(device="cuda").manual_seed(rows * 7 + vocab)
    logits = torch.randn(rows, vocab, device="cuda", generator=g).to(dtype)
    logits[0, vocab // 2] = logits[0, vocab - 1] = 50.0            # a tie: the lower index wins
    want = cuda.argmax(logits)
    out = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    assert _call(lib, logits, out) == 0                             # first call on the device also does the set-up
    torch.cuda.synchronize()
    assert torch.equal(out, want)
    assert torch.equal(logits.float().gather(1, out.long()[:, None])[:, 0], logits.float().max(-1).values)
    assert int(out[0]) == vocab // 2
    # second call straight after, other data, no allocation by torch in between
    logits2 = torch.randn(rows, vocab, device="cuda", generator=g).to(dtype)
    want2 = cuda.argmax(logits2)
    out2 = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    gc.collect()                       # cyclic garbage of earlier tests must not be freed inside the measured window
    gc.disable()
    try:
        before = torch.cuda.memory_allocated()
        assert _call(lib, logits2, out2) == 0
        assert _call(lib, logits, out) == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
    finally:
        gc.enable()
    assert torch.equal(out2, want2) and torch.equal(out, want)


def test_static_argmax_on_a_side_stream_and_wrong_device_stream():
    """A non-default stream of the current device works; a stream (or logits) of another device is refused."""
    from tensorrt_edge_llm_b200.ops import cuda
    lib = cuda.lib()
    g = torch.Generator(device="cuda").manual_seed(11)
    logits = torch.randn(16, 40000, device="cuda", generator=g).half()
    want = cuda.argmax(logits)
    out = torch.full((16,), -1, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        assert _call(lib, logits, out) == 0
        assert _call(lib, logits, out) == 0
    side.synchronize()
    assert torch.equal(out, want)
    if torch.cuda.device_count() > 1:
        other = torch.cuda.Stream(device=1)
        lib.telb_argmax_static.restype = ctypes.c_int
        rc = lib.telb_argmax_static(ctypes.c_void_p(logits.data_ptr()), ctypes.c_void_p(out.data_ptr()), ctypes.c_int(16), ctypes.c_int(40000),
                                    ctypes.c_longlong(logits.stride(0)), ctypes.c_int(0), ctypes.c_void_p(other.cuda_stream))
        assert rc == -1 and b"device" in lib.telb_last_error()
        torch.cuda.synchronize()


def test_static_argmax_rejects_oversize():
    from tensorrt_edge_llm_b200.ops import cuda
    lib = cuda.lib()
    logits = torch.zeros(257, 64, device="cuda")
    out = torch.zeros(257, dtype=torch.int32, device="cuda")
    assert _call(lib, logits, out) == -1
    assert b"256" in lib.telb_last_error()
    torch.cuda.synchronize()
