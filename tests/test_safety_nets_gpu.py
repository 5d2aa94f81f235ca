"""The library's safety nets, run on purpose: a bounded wait that runs out (the give-up
path of the tcgen05 kernels: status word, abort flag, drain, tensor memory freed), and
the host's reading of the status word.  Nothing here faults, traps or hangs: the wait is
on a barrier at which nobody arrives, with a limit of a millisecond, and the kernel
returns by itself."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from zlm_b200.kernels import get_kernels
    return get_kernels()


def _product_is_right(K):
    g = torch.Generator().manual_seed(5)
    x = (torch.randn((200, 256), generator=g) * 0.5).to(torch.bfloat16).cuda()
    w = (torch.randn((384, 256), generator=g) * 0.5).to(torch.bfloat16).cuda()
    out = torch.empty((200, 384), dtype=torch.bfloat16, device="cuda")
    K.linear(out, x, w, impl="tc")
    want = x.float() @ w.float().t()
    torch.testing.assert_close(out.float(), want, atol=3e-2, rtol=3e-2)


def test_a_bounded_wait_runs_out_and_the_library_goes_on(K):
    from zlm_b200.kernels import KernelError
    assert K.status(sync=True) == 0
    _product_is_right(K)
    code, released, ns, landed = K.test_bounded_wait(1_000_000)            # one millisecond
    assert code == (1 << 8) | 0x7e, "the waiting role did not give up with its own mark"
    assert released, "the other roles' waits were not ended by the abort flag"
    assert landed, "the producer did not let its copy land before the block ended"
    assert 1_000_000 <= ns < 500_000_000, f"the kernel took {ns} ns for a 1 ms limit"
    # the host sees the mark without any copy, and reading it as an error clears it
    assert K.status() == code
    with pytest.raises(KernelError, match="bounded wait inside a tcgen05 product kernel gave up"):
        K.check_status()
    assert K.status() == 0
    # tensor memory was given back and the context is whole: an ordinary product runs and is right
    _product_is_right(K)
    assert K.status(sync=True) == 0


def test_the_engine_raises_when_a_step_reported_a_give_up(K, tmp_path):
    """After a kernel has reported a give-up, the next place where the host waits for the
    device anyway (a prefill's tokens, a fetched decode step, the next step's start)
    raises instead of handing out what was computed."""
    from helpers import make_model
    from zlm_b200 import Engine
    from zlm_b200.kernels import KernelError
    folder, cfg, _ = make_model(tmp_path, "A", seed=1)
    eng = Engine.from_pretrained(folder, dtype="bfloat16", max_tokens=512)
    assert eng.generate([[1, 2, 3]], max_tokens=4).tokens[0]
    K.test_bounded_wait(1_000_000)
    with pytest.raises(KernelError, match="gave up"):
        eng.generate([[1, 2, 3]], max_tokens=4)
    assert K.status() == 0
    eng.cache.check()
    assert eng.cache.slots.held == 0, "the failed call kept its slots"
    assert eng.generate([[1, 2, 3]], max_tokens=4).tokens[0]
