"""The split attention kernel's entry point for callers that cannot allocate device memory
(`tl_paged_attention_split_static`, declared in tandemllm_b200/csrc/attention_noalloc.h).

Such callers (a serving loop that must not take the device-wide stall of cudaMalloc, a process whose device memory
all belongs to another allocator, a foreign host program with no device allocator) bring inputs and outputs only;
the kernel's scratch is a fixed array inside the library. The test calls the entry point the way they would,
through the exported C symbol with raw pointers, twice in a row on different inputs so that the second call runs
over whatever the first left in the shared array, and holds each result to the ordinary entry point's, which is
given scratch of its own, and to a plain softmax attention in torch. It also checks that a call too large for the
fixed array is refused with a message, that a table entry outside the pool and a row beyond the spans it was given
are recorded in the status word instead of being read, and that the device's free memory does not move across the
calls (which also sees an allocation made behind torch's back).

The file's name sorts last, so a run that stops at the first failure has run every other test before this one.
"""

import ctypes
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
STATIC_FLOATS = 2 * 1024 * 1024          # TL_STATIC_SCRATCH_FLOATS of attention_noalloc.h


def library():
    from tandemllm_b200.kernels import ops
    lib = ops.core()
    fn = lib.tl_paged_attention_split_static
    fn.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_int, c_void_p,
                   c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]
    fn.restype = c_int
    return ops, lib, fn


def case(seed: int, dtype, seqs, Hq=8, Hk=2, D=64, page=16):
    """Decode rows at the given context lengths over randomly placed pages."""
    from tests.test_gpu_kernels import paged_setup
    kc, vc, table, ks, vs = paged_setup(seqs, Hk, D, page, dtype, seed=seed)
    g = torch.Generator().manual_seed(seed + 1)
    q = torch.randn(len(seqs), Hq, D, generator=g).to(dtype)
    dev = dict(q=q.to(DEV), kc=kc.to(DEV), vc=vc.to(DEV), table=table.to(DEV),
               req=torch.arange(len(seqs), dtype=torch.int32, device=DEV),
               pos=torch.tensor([L - 1 for L in seqs], dtype=torch.int32, device=DEV), host_q=q, ks=ks, vs=vs)
    return dev, page, (Hq, Hk, D)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_entry_point_matches_the_ordinary_one_on_two_calls_in_a_row(dtype):
    ops, lib, fn = library()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    # the second call has fewer spans and other contents: it must not see what the first left in the array
    for seed, seqs, window in ((1, [1500, 300, 1024, 7], None), (2, [700, 513, 260], 400)):
        dev, page, (Hq, Hk, D) = case(seed, dtype, seqs)
        rows = len(seqs)
        spans = ops.attention_spans(max(seqs))
        assert ops.attention_scratch_floats(rows, Hq, D, spans) <= STATIC_FLOATS
        want = torch.full((rows, Hq, D), float("nan"), dtype=dtype, device=DEV)
        own = torch.full((ops.attention_scratch_floats(rows, Hq, D, spans),), float("nan"), device=DEV)
        ops.paged_attention_split(dev["q"], dev["kc"], dev["vc"], dev["table"], page, dev["req"], dev["pos"], 0.125,
                                  window, want, own, spans, status)
        got = torch.full((rows, Hq, D), float("nan"), dtype=dtype, device=DEV)
        torch.cuda.synchronize()
        before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
        code = fn(dev["q"].data_ptr(), dev["kc"].data_ptr(), dev["vc"].data_ptr(), dev["table"].data_ptr(),
                  dev["table"].shape[1], page, dev["kc"].shape[0], dev["req"].data_ptr(), dev["pos"].data_ptr(), 0.125,
                  window or 0, got.data_ptr(), rows, Hq, Hk, D, spans, ops.dtype_code(dtype), status.data_ptr(), ops.stream())
        assert code == 0, lib.tl_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.cuda.mem_get_info()[0] == free_before, "the device's free memory moved across the call"
        assert int(status) == 0
        scale = want.float().abs().max().clamp_min(1e-6)
        err = float((got.float() - want.float()).abs().max() / scale)
        assert err <= (2e-5 if dtype == torch.float32 else 2e-2), f"call with contexts {seqs}: error {err:.3g}"
        assert not bool(torch.isnan(got.float()).any())
        # and against a plain softmax attention over each request's own keys and values
        from tests.test_gpu_kernels import plain_attention
        for b in range(rows):
            plain = plain_attention(dev["host_q"][b:b + 1].float(), dev["ks"][b], dev["vs"][b], 0.125, window)[0]
            err = float((got[b].float().cpu() - plain).abs().max() / plain.abs().max())
            assert err <= (2e-5 if dtype == torch.float32 else 2e-2), f"row {b} of contexts {seqs}: error {err:.3g} against plain"


def test_a_call_too_large_for_the_fixed_array_is_refused():
    ops, lib, fn = library()
    dev, page, (Hq, Hk, D) = case(3, torch.bfloat16, [64] * 4)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.zeros(4, Hq, D, dtype=torch.bfloat16, device=DEV)
    spans = STATIC_FLOATS // (4 * Hq * (D + 2)) + 1          # one span more than the array can hold for these rows
    code = fn(dev["q"].data_ptr(), dev["kc"].data_ptr(), dev["vc"].data_ptr(), dev["table"].data_ptr(),
              dev["table"].shape[1], page, dev["kc"].shape[0], dev["req"].data_ptr(), dev["pos"].data_ptr(), 0.125, 0,
              out.data_ptr(), 4, Hq, Hk, D, spans, ops.dtype_code(torch.bfloat16), status.data_ptr(), ops.stream())
    assert code == ops.TL_BAD_ARGUMENT
    message = lib.tl_last_error().decode()
    assert "fixed array" in message and str(STATIC_FLOATS) in message
    torch.cuda.synchronize()
    assert int(status) == 0 and not bool(out.any())


def test_a_stale_table_entry_and_a_row_past_its_spans_are_recorded_not_read():
    ops, lib, fn = library()
    seqs = [700, 300]
    dev, page, (Hq, Hk, D) = case(4, torch.float32, seqs)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.zeros(2, Hq, D, device=DEV)

    def call(table, spans):
        code = fn(dev["q"].data_ptr(), dev["kc"].data_ptr(), dev["vc"].data_ptr(), table.data_ptr(), table.shape[1], page,
                  dev["kc"].shape[0], dev["req"].data_ptr(), dev["pos"].data_ptr(), 0.125, 0, out.data_ptr(), 2, Hq, Hk, D,
                  spans, ops.dtype_code(torch.float32), status.data_ptr(), ops.stream())
        assert code == 0, lib.tl_last_error().decode()
        torch.cuda.synchronize()
        code, _ = int(status), status.zero_()
        return code
    spans = ops.attention_spans(max(seqs))
    assert call(dev["table"], spans) == 0
    stale = dev["table"].clone()
    stale[1, 2] = dev["kc"].shape[0] + 5             # an entry that names no page of the pool
    assert call(stale, spans) == 3
    assert call(dev["table"], spans - 1) == 3        # the first row's position lies past the spans it was given
    assert call(dev["table"], spans) == 0            # and the next call is clean
