"""GPU test of lum_op_sample_q8_0_static, the sampling entry for hosts that cannot allocate device memory when they
run a step (all of HBM already belongs to their own arenas, or a cudaMalloc's device-wide synchronisation is not
acceptable on their path).  Its scratch is a fixed array inside the library, so the things to check are that it
computes exactly what the allocating entry lum_op_sample_q8_0 computes, that a second call right after the first
(which finds the first call's leftovers in the array) still does, and that it refuses what it cannot hold.

Collected last on purpose: a run that stops at the first failure has then already run every other test.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _call(lib, fn, packed, n, k, x, torch):
    logits = torch.full((n,), float("nan"), device="cuda")
    best = torch.full((2,), -7, dtype=torch.int32, device="cuda")
    rc = fn(packed.data_ptr(), n, k, x.data_ptr(), logits.data_ptr(), best.data_ptr(), None)
    assert rc == 0, (lib.lum_last_error(None) or b"").decode()
    torch.cuda.synchronize()
    return logits.cpu().numpy(), best.cpu().numpy()


def test_static_scratch_entry_matches_allocating_entry_twice(pkg):
    import torch
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    lib = pkg.load_library()
    n, k = 16384, 4096                      # 4096 stage-units: every SM gets work, several chunks of partial maxima
    packed = torch.empty(lib.lum_q8_0_packed_bytes(n, k), dtype=torch.uint8, device="cuda")
    assert lib.lum_op_synth_q8_0_packed(11, 7, n, k, packed.data_ptr(), None) == 0
    gen = torch.Generator(device="cuda").manual_seed(5)
    for call in range(2):                   # two calls in a row: the second starts from the first one's leftovers
        x = torch.randn(k, device="cuda", generator=gen)
        want_logits, want_best = _call(lib, lib.lum_op_sample_q8_0, packed, n, k, x, torch)
        got_logits, got_best = _call(lib, lib.lum_op_sample_q8_0_static, packed, n, k, x, torch)
        # same kernel, same reduction order: bit-identical, which is also the tolerance the operator tests use between
        # launch paths of one kernel
        assert (got_logits.view(np.uint32) == want_logits.view(np.uint32)).all(), f"call {call}: logits differ"
        assert (got_best == want_best).all(), f"call {call}: {got_best} vs {want_best}"
        assert int(got_best[1]) == int(np.flatnonzero(want_logits == want_logits.max())[-1])


def test_static_scratch_entry_rejects_what_it_cannot_take(pkg):
    import torch
    torch.cuda.set_device(0)
    lib = pkg.load_library()
    x = torch.zeros(4096, device="cuda")
    out = torch.zeros(64, device="cuda")
    best = torch.zeros(2, dtype=torch.int32, device="cuda")
    # K = 96 cannot be packed: a clear error, nothing launched
    assert lib.lum_op_sample_q8_0_static(x.data_ptr(), 8, 96, x.data_ptr(), out.data_ptr(), best.data_ptr(), None) < 0
    assert b"cannot be packed" in lib.lum_last_error(None)
    assert lib.lum_op_sample_q8_0_static(None, 64, 4096, x.data_ptr(), out.data_ptr(), best.data_ptr(), None) < 0
