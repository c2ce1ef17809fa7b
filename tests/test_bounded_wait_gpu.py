"""A bounded device-side wait that runs out: the kernel reports it and returns, and the device stays usable.

Every mbarrier wait of the tensor-memory kernels gives up after a number of polls, records IMP_WAIT_TIMEOUT
in the status word and leaves its loop; the CTA then frees its tensor memory and returns.  Here that path runs
once, in the one permitted form: one CTA of the few-rows product, the poll limit lowered to a few thousand, and
the producer told to leave one stage of the ring unfilled (a barrier that nothing completes).  Nothing faults
and nothing spins without a limit; the regular limit and the regular producer are restored afterwards.
"""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu

IMP_WAIT_TIMEOUT = 5


def test_a_wait_that_cannot_succeed_reports_a_timeout_and_frees_the_device():
    from imp_b200.ops import kernels as K
    from imp_b200.ops import library as L
    lib = L.load()
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(5)
    # 8 rows, 64 interleaved gate/up weight rows, 16 blocks of K: one CTA (the SwiGLU epilogue never splits K)
    M, N, Kdim = 8, 64, 1024
    a = (torch.randn(M, Kdim, generator=g) * 0.5).to(dev, torch.bfloat16)
    w = (torch.randn(N, Kdim, generator=g) * 0.05).to(dev, torch.bfloat16)
    out = torch.zeros(M, N // 2, dtype=torch.bfloat16, device=dev)
    status = K.new_status(dev)

    def product():
        assert K.gemm_bf16_tc_swap(out, a, w, epilogue=K.TC_OUT_SWIGLU, status=status)
        torch.cuda.synchronize()
        return int(status.item())

    def want():
        y = a.double().cpu() @ w.double().cpu().T                       # [M, N]: groups of 8 gate rows, then their 8 up rows
        y = y.view(M, N // 16, 2, 8)
        gate, up = y[:, :, 0], y[:, :, 1]
        return (gate / (1 + torch.exp(-gate)) * up).reshape(M, N // 2)

    assert product() == 0
    assert torch.allclose(out.double().cpu(), want(), atol=2e-2, rtol=2e-2)
    try:
        # block 7 of 16 stays unfilled: the MMA thread's wait for it, the producer's wait for that slot five blocks
        # later and its wait for its own copies all run out, each after 4096 polls
        L.check(lib.imp_gemm_tc_test_hooks(4096, 7), "imp_gemm_tc_test_hooks")
        t0 = time.perf_counter()
        code = product()
        seconds = time.perf_counter() - t0
    finally:
        L.check(lib.imp_gemm_tc_test_hooks(0, -1), "imp_gemm_tc_test_hooks")
    assert code == IMP_WAIT_TIMEOUT
    assert lib.imp_status_string(code).decode() == "a bounded device-side wait ran out"
    assert seconds < 2.0, f"the give-up path took {seconds:.2f} s"
    with pytest.raises(L.KernelError, match="bounded device-side wait"):
        K.check_status(status)                                           # reads, raises and clears the word
    # the regular limit is back, tensor memory was freed: the same product again, then one that takes all SMs
    out.zero_()
    assert product() == 0
    assert torch.allclose(out.double().cpu(), want(), atol=2e-2, rtol=2e-2)
    big_a = (torch.randn(512, 1024, generator=g) * 0.5).to(dev, torch.bfloat16)
    big_w = (torch.randn(lib.imp_device_sm_count() * 256, 1024, generator=g) * 0.05).to(dev, torch.bfloat16)
    big = K.linear(torch.empty(512, big_w.shape[0], dtype=torch.bfloat16, device=dev), big_a, big_w)
    torch.cuda.synchronize()
    ref = big_a.float() @ big_w.float().T
    assert torch.allclose(big.float(), ref, atol=0.1, rtol=3e-2)
