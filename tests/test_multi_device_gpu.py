"""One process driving two GPUs: per-device kernel attributes (the 227 KB shared-memory opt-in, the SM
count) must be set on each device the library launches on.  Skipped with fewer than two devices."""
import pytest
import torch

from helpers import Case, check_close

pytestmark = pytest.mark.gpu


def test_same_process_decodes_on_two_devices():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    outs = []
    for dev in ("cuda:0", "cuda:1"):
        with torch.cuda.device(dev):
            case = Case([1500], seed=5, device=dev)
            o, lse = case.run()
            want_o, _ = case.oracle_kernel_arith(split_pv=True)
            check_close(o, want_o, ctx="decode on " + dev)
            outs.append(o.cpu())
    assert torch.equal(outs[0], outs[1])
