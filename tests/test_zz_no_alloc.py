"""-m gpu, collected last: the allocation-free entry point of the fused batch-1 FFN kernel.

Some users of the library cannot call cudaMalloc where they call us (a real-time decode loop, a
plugin living inside another program's reserved memory pool). For them
tffn_op_swiglu_bs1_noalloc takes device pointers the caller already owns and keeps its scratch in
a fixed array inside the library. This test drives it through the C ABI twice in a row, with
different shapes so that the second call meets the first call's leftovers in the shared scratch,
and checks each result against the ordinary entry point tffn_op_swiglu_bs1 on the same inputs.
The device buffers are made with torch here only because the test, unlike those users, may allocate.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 1.5e-2  # the kernel tolerance of the other GPU tests; the two entry points run the same kernel


def _case(seed, H, I):
    import synth
    import tffn
    rng = np.random.default_rng(seed)

    def rnd(shape, scale):
        return synth.f32_to_bf16((rng.standard_normal(shape, dtype=np.float32) * scale).reshape(-1)).reshape(shape)

    h = rnd((H,), 1.0)
    w = synth.f32_to_bf16(1.0 + 0.1 * rng.standard_normal(H, dtype=np.float32))
    pb = tffn.pack_ffn(rnd((I, H), 0.02), rnd((I, H), 0.02), rnd((H, I), 0.02))
    pe = tffn.pack_ffn(rnd((I, H), 0.02), rnd((I, H), 0.02), rnd((H, I), 0.02))
    return h, w, pb, pe


def test_no_alloc_entry_matches_allocating_entry_twice_in_a_row():
    import torch
    import synth
    import tffn

    def dev(a):
        return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).cuda()

    stream = torch.cuda.current_stream().cuda_stream
    for seed, H, I, expert in ((1, 896, 4864, True), (2, 448, 640, False), (3, 896, 4864, True), (4, 2048, 1184, True)):  # last: the largest hidden size the built-in scratch covers
        h, w, pb, pe = _case(seed, H, I)
        want = tffn.op_swiglu_bs1(h, w, pb, pe if expert else None, 0.1, 1e-6)
        d_h, d_w, d_pb, d_pe = dev(h), dev(w), dev(pb), dev(pe)
        torch.cuda.synchronize()
        tffn.op_swiglu_bs1_noalloc(d_h.data_ptr(), d_w.data_ptr(), d_pb.data_ptr(), d_pe.data_ptr() if expert else None,
                                   H, I, 0.1, 1e-6, stream)
        got = d_h.cpu().numpy().view(np.uint16)
        a, b = synth.bf16_to_f32(got), synth.bf16_to_f32(want)
        assert np.abs(a - b).max() / np.abs(b).max() <= TOL, (seed, H, I)
        assert (got == want).all(), "same kernel, same reduction order: expected identical bits"


def test_no_alloc_entry_rejects_sizes_beyond_its_scratch():
    import torch
    import tffn
    buf = torch.zeros(1 << 16, dtype=torch.int16, device="cuda")
    with pytest.raises(tffn.TffnError) as ei:
        tffn.op_swiglu_bs1_noalloc(buf.data_ptr(), buf.data_ptr(), buf.data_ptr(), None, 4096, 8)
    assert ei.value.code == -6 and "2048" in ei.value.msg


def test_no_alloc_entry_rejects_misaligned_pointers():
    """the caller's pointers reach 16-byte vector loads and bulk copies unchanged: an address that is
    not 16-byte aligned is refused on the host instead of faulting on the device"""
    import torch
    import tffn
    buf = torch.zeros(1 << 16, dtype=torch.int16, device="cuda")
    base = buf.data_ptr()
    for bad in range(4):
        ptrs = [base, base + 4096, base + 8192, base + 65536]
        ptrs[bad] += 2
        with pytest.raises(tffn.TffnError) as ei:
            tffn.op_swiglu_bs1_noalloc(ptrs[0], ptrs[1], ptrs[2], ptrs[3], 256, 8)
        assert ei.value.code == -1 and "aligned" in ei.value.msg
