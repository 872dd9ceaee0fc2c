"""The allocation-free entry point `fsb_argmax_rows_static`, called through the C ABI and compared with the handle
based entry point on the same rows.  Collected last (file name), so that it also runs after every other test has
used the library in this process; it passes alone as well."""
import numpy as np
import pytest

import ferro_b200 as fb

pytestmark = pytest.mark.gpu


def _greedy_through_the_handle(engine, lg):
    p = fb.make_params(lg.shape[0], temperature=0.0, top_k=50, top_p=1.0, min_p=0.0, repetition_penalty=1.0)
    sids = engine.open_streams(p)
    try:
        return engine.sample_batch(sids, lg.copy(), [np.zeros(0, np.int32)] * lg.shape[0])
    finally:
        for s in sids:
            engine.close_stream(int(s))


# (1, 262144) and (3, 200000): one tile per CTA, so a row has 32 resp. 25 segments - more than a CTA has warps - and
# its candidates are merged by the gather-and-order route instead of the ordered-list route
@pytest.mark.parametrize("shape", [(64, 262144), (17, 65536), (5, 70001), (1, 33), (1, 262144), (3, 200000)])
def test_static_scratch_entry_point_matches_the_handle_based_one_twice_in_a_row(engine, shape):
    import torch
    B, V = shape
    rng = np.random.default_rng(2024 + V)
    out = torch.full((B,), -7, dtype=torch.int32, device="cuda")
    for call in range(2):                                   # two calls in a row share the one scratch array
        lg = (rng.standard_normal((B, V)) * 3).astype(np.float32)
        lg[:, ::5] = np.round(lg[:, ::5])                   # ties: the lowest index must win
        if call == 1:
            lg[0, :] = 2.5                                  # a row of equal values
        dev = torch.from_numpy(lg).cuda()
        out.fill_(-7)
        fb.argmax_rows_static(dev.data_ptr(), V, B, V, out.data_ptr(), device=0, cuda_stream=torch.cuda.current_stream().cuda_stream)
        got = out.cpu().numpy()
        assert np.array_equal(got, _greedy_through_the_handle(engine, lg)), f"call {call}"
        assert np.array_equal(got, np.argmax(lg, axis=1).astype(np.int32))


def test_static_scratch_entry_point_without_waiting_and_with_a_row_stride(engine):
    import torch
    B, V, ld = 8, 40000, 40960
    rng = np.random.default_rng(9)
    wide = (rng.standard_normal((B, ld)) * 2).astype(np.float32)
    wide[:, V:] = 100.0                                     # columns past n_vocab must not be looked at
    dev = torch.from_numpy(wide).cuda()
    out = torch.zeros(B, dtype=torch.int32, device="cuda")
    fb.argmax_rows_static(dev.data_ptr(), ld, B, V, out.data_ptr(), wait=False, cuda_stream=torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), np.argmax(wide[:, :V], axis=1).astype(np.int32))


def test_static_scratch_entry_point_recovers_from_an_error_nobody_waited_for():
    """A call without FSB_STATIC_WAIT whose kernel reports an error (a row without a finite logit) leaves the status
    word set; the next call clears it before its kernel runs and must succeed."""
    import torch
    B, V = 4, 20000
    bad = torch.full((B, V), float("nan"), device="cuda")
    out = torch.zeros(B, dtype=torch.int32, device="cuda")
    fb.argmax_rows_static(bad.data_ptr(), V, B, V, out.data_ptr(), wait=False, cuda_stream=torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    with pytest.raises(fb.SamplerError) as e:               # the same input, waited for: the error is reported
        fb.argmax_rows_static(bad.data_ptr(), V, B, V, out.data_ptr(), cuda_stream=torch.cuda.current_stream().cuda_stream)
    assert "FSB_ERR_DEVICE" in str(e.value)
    lg = (np.random.default_rng(5).standard_normal((B, V)) * 2).astype(np.float32)
    good = torch.from_numpy(lg).cuda()
    for _ in range(2):
        fb.argmax_rows_static(good.data_ptr(), V, B, V, out.data_ptr(), cuda_stream=torch.cuda.current_stream().cuda_stream)
        assert np.array_equal(out.cpu().numpy(), np.argmax(lg, axis=1).astype(np.int32))


def test_static_scratch_entry_point_refuses_what_its_array_cannot_hold():
    import torch
    dev = torch.zeros(fb.STATIC_MAX_ROWS + 1, 4096, device="cuda")
    out = torch.zeros(fb.STATIC_MAX_ROWS + 1, dtype=torch.int32, device="cuda")
    with pytest.raises(fb.SamplerError) as e:
        fb.argmax_rows_static(dev.data_ptr(), 4096, fb.STATIC_MAX_ROWS + 1, 4096, out.data_ptr())
    assert "FSB_ERR_CAPACITY" in str(e.value)
    with pytest.raises(fb.SamplerError):
        fb.argmax_rows_static(0, 4096, 1, 4096, out.data_ptr())          # null logits
    with pytest.raises(fb.SamplerError):
        fb.argmax_rows_static(dev.data_ptr(), 100, 1, 4096, out.data_ptr())   # row stride below n_vocab
