"""The give-up path of the bounded device waits, exercised without faulting or hanging anything: a small kernel
waits, with a limit of a few thousand polls, on a barrier nothing ever completes; it must come back by itself,
report its code through the device status word, and leave the context and the status word usable."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_reports_its_code_and_the_library_goes_on():
    from rapid_h3_b200 import _lib as lib, quantizers
    assert torch.cuda.is_available()
    lib.check_status()                                   # clean before
    left = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib.call("rh3_selftest_wait_expiry", 3000, left.data_ptr(), lib.stream())
    st = ctypes.c_int(0)
    lib.call("rh3_check_status", lib.stream(), ctypes.addressof(st))
    assert st.value == 190                               # ST_TIMEOUT_SELFTEST
    assert "gave up" in lib.last_error()
    assert left.item() == 1                              # every thread left through the give-up path
    # the word was cleared by the read, and kernels still run
    lib.check_status()
    x = torch.randn(64, 512, device="cuda").to(torch.bfloat16)
    q, s = quantizers.quant_rows_i8(x)
    torch.cuda.synchronize()
    assert (q.float().abs().amax(dim=1) == 127).all()
    lib.check_status()


def test_check_status_raises_on_a_recorded_code():
    from rapid_h3_b200 import _lib as lib
    left = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib.call("rh3_selftest_wait_expiry", 200, left.data_ptr(), lib.stream())
    with pytest.raises(RuntimeError, match="190"):
        lib.check_status()
    lib.check_status()


@pytest.mark.parametrize("kind", [0, 1, 2])
@pytest.mark.parametrize("random_operands", [0, 1])
def test_tensor_pipe_probe_returns_and_reports_a_plausible_rate(kind, random_operands):
    """The issue-rate probe (no reference counterpart) comes back by itself with a clean status word, counts its
    operations as documented, and retires above half of the nominal rate of its operand kind."""
    from rapid_h3_b200 import _lib as lib
    ops = ctypes.c_double(0)
    groups = 400

    def run():
        lib.call("rh3_selftest_mma_rate", kind, groups, random_operands, 0, ctypes.addressof(ops), lib.stream())

    run()
    lib.check_status()
    sms = lib.lib().rh3_sm_count()
    assert ops.value == sms * groups * 64 * 2 * 128 * 256 * (16 if kind == 2 else 32)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        run()
    e1.record()
    torch.cuda.synchronize()
    lib.check_status()
    tops = ops.value * 3 / e0.elapsed_time(e1) / 1e9
    assert tops > (1100 if kind == 2 else 2200), tops
    # pattern 4: the same with 128-column MMAs (half the work per instruction), the narrow tiles of the convolution
    lib.call("rh3_selftest_mma_rate", kind, groups, random_operands, 4, ctypes.addressof(ops), lib.stream())
    lib.check_status()
    assert ops.value == sms * groups * 64 * 2 * 128 * 128 * (16 if kind == 2 else 32)
    with pytest.raises(RuntimeError):
        lib.call("rh3_selftest_mma_rate", 3, groups, 0, 0, ctypes.addressof(ops), lib.stream())
    with pytest.raises(RuntimeError):
        lib.call("rh3_selftest_mma_rate", kind, groups, 0, 5, ctypes.addressof(ops), lib.stream())


@pytest.mark.parametrize("fill", [0, 16384, 49152])
def test_gemm_main_loop_probe_returns_by_itself(fill):
    """The main-loop probe (bulk copies into a four-stage ring + MMAs, no epilogue) comes back with a clean status
    word for stage counts that are and are not multiples of the ring size, and refuses bad arguments."""
    from rapid_h3_b200 import _lib as lib
    src = torch.randint(-127, 128, (8 << 20,), device="cuda", dtype=torch.int8)
    ops = ctypes.c_double(0)
    for stages in (1, 3, 4, 1001):
        lib.call("rh3_selftest_mma_feed", src.data_ptr(), src.numel(), stages, fill, ctypes.addressof(ops), lib.stream())
        lib.check_status()
        assert ops.value == lib.lib().rh3_sm_count() * stages * 4 * 2 * 128 * 256 * 32
    with pytest.raises(RuntimeError):
        lib.call("rh3_selftest_mma_feed", src.data_ptr(), src.numel(), 10, 1000, ctypes.addressof(ops), lib.stream())
    with pytest.raises(RuntimeError):
        lib.call("rh3_selftest_mma_feed", src.data_ptr(), 100, 10, 16384, ctypes.addressof(ops), lib.stream())
