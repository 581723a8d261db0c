"""The allocation-free K/V statistics entry point against the regular one.

Some callers of the library cannot create device memory (everything is owned by their framework's pool, or
cudaMalloc is banned on their thread), so `rh3_attn_kv_stats_noalloc` keeps its chunk partials in an array
inside the library instead of caller scratch. This file checks, through the C ABI, that it returns exactly
what `rh3_attn_kv_stats` returns, on two calls in a row with different inputs (the shared array keeps the
previous call's contents), and that a problem beyond the built-in limit is refused with a clear message.
It is named to be collected last, so a run that stops at the first failure has already run everything else.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _stats(lib, entry, k, v, with_scratch):
    l, h, _ = k.shape
    out = [torch.full((h, 128), float("nan"), device="cuda") for _ in range(3)]
    head = (k.data_ptr(), k.stride(0), k.stride(1), v.data_ptr(), v.stride(0), v.stride(1), l, h)
    tail = tuple(t.data_ptr() for t in out) + (lib.stream(),)
    if with_scratch:
        nbytes = lib.lib().rh3_attn_kv_stats_scratch_bytes(l, h)
        scratch = torch.empty(nbytes, device="cuda", dtype=torch.uint8)
        lib.call(entry, *head, scratch.data_ptr(), nbytes, *tail)
    else:
        lib.call(entry, *head, *tail)
    torch.cuda.synchronize()
    return out


def test_noalloc_kv_stats_equals_regular_entry_twice_in_a_row():
    from rapid_h3_b200 import _lib as lib
    assert torch.cuda.is_available()
    g = torch.Generator(device="cuda").manual_seed(7)
    for l, h in ((5000, 8), (777, 3)):  # second call: fewer chunks and heads than the array still holds
        k = (torch.randn(l, h, 128, device="cuda", generator=g) * 3 + 1).to(torch.bfloat16)
        v = torch.randn(l, 3 * h, 128, device="cuda", generator=g).to(torch.bfloat16)[:, h:2 * h]  # strided view
        before = torch.cuda.memory_allocated()
        got = _stats(lib, "rh3_attn_kv_stats_noalloc", k, v, with_scratch=False)
        ref = _stats(lib, "rh3_attn_kv_stats", k, v, with_scratch=True)
        for a, b in zip(got, ref):
            assert torch.equal(a, b)  # same kernels, same order of additions: bit-identical
        assert torch.isfinite(got[0]).all() and (got[2] > 0).all()
        del got, ref
        assert torch.cuda.memory_allocated() <= before + (1 << 20)
    lib.check_status()


@pytest.mark.parametrize("l, h", [(1, 8192), (65536, 32)])
def test_noalloc_kv_stats_at_exactly_the_builtin_limit(l, h):
    """8192 units, the last element of the built-in array included: many heads of one token, and many chunks of
    few heads. One unit more is refused."""
    from rapid_h3_b200 import _lib as lib
    g = torch.Generator(device="cuda").manual_seed(l + h)
    k = torch.randn(l, h, 128, device="cuda", generator=g).to(torch.bfloat16)
    v = (torch.randn(l, h, 128, device="cuda", generator=g) - 0.5).to(torch.bfloat16)
    got = _stats(lib, "rh3_attn_kv_stats_noalloc", k, v, with_scratch=False)
    ref = _stats(lib, "rh3_attn_kv_stats", k, v, with_scratch=True)
    for a, b in zip(got, ref):
        assert torch.equal(a, b)
    lib.check_status()
    out = torch.zeros(3, 1, 128, device="cuda")
    l2, h2 = (l, h + 1) if l == 1 else (l + 1, h)
    rc = lib.lib().rh3_attn_kv_stats_noalloc(k.data_ptr(), k.stride(0), k.stride(1), v.data_ptr(), v.stride(0),
                                             v.stride(1), l2, h2, out[0].data_ptr(), out[1].data_ptr(),
                                             out[2].data_ptr(), lib.stream())
    assert rc < 0 and "exceeds the built-in scratch limit" in lib.last_error()


def test_noalloc_kv_stats_rejects_sizes_beyond_the_builtin_scratch():
    from rapid_h3_b200 import _lib as lib
    k = torch.zeros(8, 1, 128, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(3, 40, 128, device="cuda")
    # 40 heads x ceil(60000/256) = 9400 units > 8192: must be refused before anything is launched
    rc = lib.lib().rh3_attn_kv_stats_noalloc(k.data_ptr(), 128, 128, k.data_ptr(), 128, 128, 60000, 40,
                                             out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr(), lib.stream())
    assert rc < 0
    assert "exceeds the built-in scratch limit" in lib.last_error()
