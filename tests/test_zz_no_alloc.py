"""The decode attention entry point that allocates nothing (csrc/attention_static_scratch.h).

Collected last on purpose (the file name sorts after every other test file): should it
fail, a run that stops at the first failure has already run everything else. It calls the
exported C symbol directly, twice in a row with different inputs, and compares each result
with the ordinary entry point's, whose scratch comes from the caller. It needs nothing from
the other tests and passes alone in a fresh process.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def case(seed, lengths, Hq=8, Hk=2, d=64):
    g = torch.Generator().manual_seed(seed)
    B = len(lengths)
    per_seq = max(-(-n // 64) for n in lengths)
    pages = B * per_seq
    k = torch.randn(pages, Hk, 64, d, generator=g).to(torch.bfloat16).to(DEV)
    v = torch.randn(pages, Hk, 64, d, generator=g).to(torch.bfloat16).to(DEV)
    table = torch.randperm(pages, generator=g).to(torch.int32).view(B, per_seq).contiguous().to(DEV)
    q = torch.randn(B, Hq, d, generator=g).to(torch.bfloat16).to(DEV)
    slots = torch.arange(B, dtype=torch.int32, device=DEV)
    lens = torch.tensor(lengths, dtype=torch.int32, device=DEV)
    return q, k, v, table, slots, lens


def p(t):
    return ctypes.c_void_p(t.data_ptr())


def run(lib, symbol, q, k, v, table, slots, lens, splits, scratch=None):
    B, Hq, d = q.shape
    out = torch.full((B, Hq * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    args = [p(q), p(k), p(v)]
    if scratch is not None:
        args.append(p(scratch))
    args += [p(out), p(table), table.shape[1], p(slots), p(lens), B, Hq, k.shape[1], d, 64,
             ctypes.c_float(d ** -0.5), 0, splits, stream]
    torch.cuda.synchronize()
    before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
    code = getattr(lib, symbol)(*args)
    torch.cuda.synchronize()
    # what torch's allocator handed out, and what the driver says is free on the device: the
    # second also sees an allocation made behind torch's back
    return code, out, (torch.cuda.memory_allocated() - before, free_before - torch.cuda.mem_get_info()[0])


def test_static_scratch_entry_point_matches_the_ordinary_one_twice_in_a_row():
    from llama_rs_metal_b200.kernels import library
    lib = library.load()
    lib.lrm_attention_static_scratch_error.restype = ctypes.c_char_p
    capacity = lib.lrm_attention_static_scratch_floats()
    assert capacity == 1 << 20
    # The first call on a device looks the array's address up (and may make the driver load the
    # module): it is made here, before anything is measured. It is also a large one, so that the
    # array is full of another problem's partials when the smaller problems below run; the last
    # of them has more splits than some sequences have pages (splits that see no key).
    q, k, v, table, slots, lens = case(9, [700] * 8, Hq=32, Hk=8)
    code, _, _ = run(lib, "lrm_attention_decode_tiled_static_scratch", q, k, v, table, slots, lens, 7)
    assert code == 0, lib.lrm_attention_static_scratch_error(code).decode()
    for seed, lengths, splits in ((1, [300, 64, 1, 129], 3), (2, [40, 513], 5), (3, [1, 64, 65], 6)):
        q, k, v, table, slots, lens = case(seed, lengths)
        scratch = torch.full((len(lengths) * 8 * splits * 66,), float("nan"), dtype=torch.float32, device=DEV)
        code, want, _ = run(lib, "lrm_attention_decode_tiled", q, k, v, table, slots, lens, splits, scratch)
        assert code == 0
        code, got, (from_torch, from_driver) = run(lib, "lrm_attention_decode_tiled_static_scratch", q, k, v, table,
                                                   slots, lens, splits)
        assert code == 0, lib.lrm_attention_static_scratch_error(code).decode()
        assert from_torch == 0 and from_driver <= 0             # nothing was allocated, by anyone
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got, want)                           # the same kernels in the same order: the same bits
    # a problem whose partials do not fit is refused, with a sentence that says why
    q, k, v, table, slots, lens = case(3, [64] * 64, Hq=32, Hk=8)
    code, _, _ = run(lib, "lrm_attention_decode_tiled_static_scratch", q, k, v, table, slots, lens, 8)
    assert code == -4
    assert b"do not fit" in lib.lrm_attention_static_scratch_error(code)
