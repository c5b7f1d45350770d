"""Runtime pieces on one GPU: bounded waits and the status block."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.expect_status
def test_wait_on_a_flag_nobody_sets_times_out_and_context_survives():
    from parallelkernelbench_b200 import _native as nv

    flag = torch.zeros(4, dtype=torch.int32, device="cuda")
    elapsed = torch.zeros(1, dtype=torch.int32, device="cuda")
    nv.clear_status()
    nv.check(nv.cuda_lib().pkb_wait_selftest(nv.ptr(flag), 1, nv.c_u64(3_000_000), nv.ptr(elapsed), nv.current_stream()))
    torch.cuda.synchronize()
    st = nv.read_status()
    assert st[0] == 2 and st[1] == 900              # PEER_TIMEOUT recorded by the self-test kernel
    assert 2500 <= elapsed.item() <= 50_000         # gave up after ~3 ms, not after seconds
    with pytest.raises(nv.KernelStatusError):
        nv.raise_on_status()
    # the context is still usable: the next kernel on the same stream runs fine
    flag.fill_(7)
    nv.check(nv.cuda_lib().pkb_wait_selftest(nv.ptr(flag), 1, nv.c_u64(3_000_000), nv.ptr(elapsed), nv.current_stream()))
    torch.cuda.synchronize()
    assert nv.read_status()[0] == 0 and elapsed.item() < 1000
    assert torch.equal(torch.ones(4, device="cuda") * 2, torch.full((4,), 2.0, device="cuda"))
