"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some hosts of this library cannot call cudaMalloc: the device's memory was handed out completely when
the process started (a serving runtime that reserved everything for weights and cache, or a plugin living
inside another allocator), or they sit in a latency-critical loop where the device-wide synchronisation of
cudaMalloc / cudaFree is not acceptable. For them the library carries its split-key scratch inside its own
image. This test calls that entry point twice in a row with different inputs and checks each result
against the ordinary entry point (which takes scratch from the caller), within the tolerance the kernel
tests use. The file sorts last so that a run that stops at the first failure has run everything else.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _call_noalloc(c, nh, nkv, D, page, n_seqs, window, max_splits, out):
    from tokenmill_b200.kernels import lib

    fn = lib.load().tm_decode_attention_bf16_noalloc
    fn.restype = ctypes.c_int
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [P, P, P, P, I, P, P, P, I, I, P, I, I, I, I, F, I, I, I, P]
    return fn(c["q"].data_ptr(), c["kc"].data_ptr(), c["vc"].data_ptr(), c["table"].data_ptr(), c["table"].stride(0),
              c["cu"].data_ptr(), c["before"].data_ptr(), c["seq_of"].data_ptr(), n_seqs, c["q"].shape[0],
              out.data_ptr(), nh, nkv, D, page, D ** -0.5, window, 256, max_splits,
              torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("nh,nkv,D,page", [(14, 2, 64, 16), (8, 2, 128, 8)])
def test_noalloc_entry_point_matches_the_ordinary_one_twice_in_a_row(nh, nkv, D, page):
    from kernel_cases import paged_case as _paged_case
    from tokenmill_b200.kernels import ops

    for call, (befores, window) in enumerate([([0, 255, 256, 700, 1000, 63, 511], 0), ([900, 3, 300, 64, 1, 513, 128], 150)]):
        q_lens = [1] * len(befores)
        c = _paged_case(nh, nkv, D, page, q_lens=q_lens, befores=befores, dtype=torch.bfloat16, seed=100 + call + D,
                        window=window)
        T = len(befores)
        max_splits = -(-(max(befores) + 1) // 256)
        ordinary = torch.empty_like(c["q"])
        part_acc = torch.empty(T * nh * max_splits * D, device=DEV)
        part_ml = torch.empty(T * nh * max_splits * 2, device=DEV)
        ops.decode_attention_bf16(c["q"], c["kc"], c["vc"], c["table"], c["cu"], c["before"], T, ordinary,
                                  scale=D ** -0.5, window=window, split_keys=256, max_splits=max_splits,
                                  part_acc=part_acc, part_ml=part_ml)
        out = torch.full_like(c["q"], float("nan"))
        before = torch.cuda.memory_allocated()
        status = _call_noalloc(c, nh, nkv, D, page, T, window, max_splits, out)
        torch.cuda.synchronize()
        assert status == 0
        assert torch.cuda.memory_allocated() == before           # nothing was taken from torch's allocator
        assert torch.equal(out, ordinary)                         # same kernels, same order of sums
        ref = c["ref"]
        assert (out.float().cpu() - ref).abs().max() <= 1e-2 * float(ref.abs().max())


def _status():
    from tokenmill_b200.kernels import lib
    fn = lib.load().tm_decode_attention_bf16_noalloc_status
    fn.restype, fn.argtypes = ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p]
    code = ctypes.c_int(-1)
    assert fn(ctypes.addressof(code), torch.cuda.current_stream().cuda_stream) == 0
    return code.value


def _reset():
    from tokenmill_b200.kernels import lib
    fn = lib.load().tm_decode_attention_bf16_noalloc_reset
    fn.restype, fn.argtypes = ctypes.c_int, [ctypes.c_void_p]
    assert fn(torch.cuda.current_stream().cuda_stream) == 0


def test_noalloc_entry_point_with_portions_of_a_few_tokens_three_calls_in_a_row():
    """Requests that bring 2 to 4 tokens (rows of several tokens share a 16-row tile at 4 heads per kv head), on the
    same request indices three times in a row: a counter that a call left non-zero would make the next call merge
    too early or never."""
    from kernel_cases import paged_case as _paged_case
    from tokenmill_b200.kernels import ops

    nh, nkv, D, page = 8, 2, 128, 16
    for call in range(3):
        q_lens, befores = [2, 4, 3, 1, 4], [300 + call, 0, 517, 64, 255]
        c = _paged_case(nh, nkv, D, page, q_lens=q_lens, befores=befores, dtype=torch.bfloat16, seed=7 + call)
        T, S = sum(q_lens), len(q_lens)
        max_splits = -(-(max(b + n for b, n in zip(befores, q_lens))) // 256)
        ordinary = torch.empty_like(c["q"])
        ops.decode_attention_bf16(c["q"], c["kc"], c["vc"], c["table"], c["cu"], c["before"], S, ordinary,
                                  scale=D ** -0.5, window=0, split_keys=256, max_splits=max_splits,
                                  part_acc=torch.empty(T * nh * max_splits * D, device=DEV),
                                  part_ml=torch.empty(T * nh * max_splits * 2, device=DEV))
        out = torch.full_like(c["q"], float("nan"))
        assert _call_noalloc(c, nh, nkv, D, page, S, 0, max_splits, out) == 0
        torch.cuda.synchronize()
        assert torch.equal(out, ordinary)
        ref = c["ref"]
        assert (out.float().cpu() - ref).abs().max() <= 1.5e-2 * float(ref.abs().max())     # the kernel tests' bound
        assert _status() == 0


def test_noalloc_entry_point_reports_what_the_host_cannot_check():
    """A context beyond max_splits * split_keys is only visible on the device: the launch says so through the
    library's error word, leaves the counters at zero, and after a reset the entry point works as before."""
    from kernel_cases import paged_case as _paged_case

    c = _paged_case(14, 2, 64, 16, q_lens=[1, 1], befores=[10, 700], dtype=torch.bfloat16, seed=3)
    out = torch.empty_like(c["q"])
    assert _call_noalloc(c, 14, 2, 64, 16, 2, 0, 2, out) == 0          # 2 splits of 256 keys: request 1 has 701
    torch.cuda.synchronize()
    assert _status() == 32
    _reset()
    assert _status() == 0
    good = torch.full_like(c["q"], float("nan"))
    assert _call_noalloc(c, 14, 2, 64, 16, 2, 0, 3, good) == 0
    torch.cuda.synchronize()
    assert _status() == 0
    assert (good.float().cpu() - c["ref"]).abs().max() <= 1.5e-2 * float(c["ref"].abs().max())


def test_noalloc_entry_point_refuses_what_does_not_fit():
    from kernel_cases import paged_case as _paged_case

    c = _paged_case(14, 2, 64, 16, q_lens=[1, 1], befores=[10, 20], dtype=torch.bfloat16, seed=1)
    out = torch.empty_like(c["q"])
    # 2 tokens x 14 heads x 100000 splits x 66 floats is far beyond the 2 Mi floats the library carries
    assert _call_noalloc(c, 14, 2, 64, 16, 2, 0, 100000, out) == 90004
    # more (request, kv head) pairs than the 4,096 counters; a head size the kernel does not have
    assert _call_noalloc(c, 14, 2, 64, 16, 2049, 0, 1, out) == 90004
    assert _call_noalloc(c, 14, 2, 96, 16, 2, 0, 1, out) == 90001
