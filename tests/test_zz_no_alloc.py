"""GPU: the no-allocation forward entry point gives the same result as the regular one.

`qla_chunk_fwd_noalloc` exists for hosts that own all device memory themselves and must not see a
cudaMalloc on the request path (for instance a serving process whose pools fill the card); it keeps the
chunk tables of packed (cu_seqlens) batches in a fixed array inside the library.  The test drives it
through the C ABI with ctypes on two consecutive calls and compares with `qla_chunk_fwd` (bitwise: both
run the same kernels on the same inputs).  A call with a different number of sequences runs in between,
so the second call finds another batch's tables in the shared array, and the device's free memory is
compared before and after to see that nothing was allocated.
"""
import ctypes as C

import pytest
import torch

from oracle import gdr_oracle as orc

pytestmark = pytest.mark.gpu


def _args(_cabi, t, out, cu, n_seqs, status):
    q, k, v, g, beta, h0 = t["q"], t["k"], t["v"], t["g"], t["beta"], t["h0"]
    return _cabi.QlaChunkFwdArgs(
        batch=1, seq_len=q.shape[1], num_seqs=n_seqs, num_k_heads=q.shape[2], num_v_heads=v.shape[2],
        qkv_dtype=_cabi.dtype_code(q.dtype), gate_dtype=_cabi.dtype_code(g.dtype),
        beta_dtype=_cabi.dtype_code(beta.dtype), flags=0, max_chunks_per_seq=0, scale=128 ** -0.5,
        q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), g=g.data_ptr(), beta=beta.data_ptr(),
        h0=h0.data_ptr(), cu_seqlens=cu.data_ptr(), seq_map=None, chunk_limit=None,
        g_cumsum=out["g_cumsum"].data_ptr(), A=out["A"].data_ptr(), w=out["w"].data_ptr(), o=out["o"].data_ptr(), h=None, v_new=None,
        final_state=out["fs"].data_ptr(), workspace=None, workspace_bytes=0, status=status.data_ptr())


def _outputs(t, n_seqs):
    v = t["v"]
    return dict(g_cumsum=torch.zeros(v.shape[:3], dtype=torch.float32, device=v.device),
                A=torch.zeros(*v.shape[:3], 64, dtype=v.dtype, device=v.device), w=torch.zeros_like(v),
                o=torch.zeros_like(v),
                fs=torch.zeros(n_seqs, v.shape[2], 128, 128, dtype=torch.float32, device=v.device))


def test_noalloc_forward_matches_regular_entry_point():
    from flashqla_b200 import _cabi
    lib = _cabi.lib()
    lens = [200, 64, 333, 1, 130]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    inp = orc.make_prefill_inputs(1, sum(lens), 2, 4, seed=77, with_h0=True, n_states=len(lens))
    t = {n: x.cuda() for n, x in inp.items()}
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream

    # regular entry point with a caller-provided workspace
    ref = _outputs(t, len(lens))
    a = _args(_cabi, t, ref, cu, len(lens), status)
    ws = torch.empty(lib.qla_chunk_fwd_workspace_bytes(a), dtype=torch.uint8, device="cuda")
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    assert lib.qla_chunk_fwd(a, stream) == 0, lib.qla_last_error()

    # another packed batch (different number of sequences, so its tables sit at other offsets of the array)
    lens2 = [70, 500]
    cu2 = torch.tensor([0, 70, 570], dtype=torch.int32, device="cuda")
    inp2 = orc.make_prefill_inputs(1, sum(lens2), 2, 4, seed=78, with_h0=True, n_states=len(lens2))
    t2 = {n: x.cuda() for n, x in inp2.items()}
    out2 = _outputs(t2, len(lens2))

    # the entry point under test, twice in a row (the second call reuses the shared array, which the call
    # in between has overwritten); the flag that would skip the table launch must not be honoured
    outs = [_outputs(t, len(lens)) for _ in range(2)]
    torch.cuda.synchronize()
    free_before, allocated_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
    for call in range(2):
        got = outs[call]
        b = _args(_cabi, t, got, cu, len(lens), status)
        if call == 1:
            b.flags |= _cabi.CHUNK_TABLES_READY
        assert lib.qla_chunk_fwd_noalloc(b, stream) == 0, lib.qla_last_error()
        if call == 0:
            assert lib.qla_chunk_fwd_noalloc(_args(_cabi, t2, out2, cu2, len(lens2), status), stream) == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        for name in ref:
            assert torch.equal(got[name], ref[name]), f"call {call}: {name} differs"
    assert torch.cuda.memory_allocated() == allocated_before
    assert torch.cuda.mem_get_info()[0] >= free_before, "device memory was allocated during the calls"
    ref2 = orc.chunk_gdr_fwd_varlen(inp2["q"], inp2["k"], inp2["v"], inp2["g"], inp2["beta"], cu2.cpu(), h0=inp2["h0"])
    assert orc.rel_rms(out2["o"].float().cpu(), ref2["o"]) <= 5e-3
    # and against the oracle, with the tolerance of the forward tests
    o_ref = orc.chunk_gdr_fwd_varlen(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], cu.cpu(), h0=inp["h0"])
    assert orc.rel_rms(got["o"].float().cpu(), o_ref["o"]) <= 5e-3
    assert orc.rel_rms(got["fs"].cpu(), o_ref["final_state"]) <= 5e-3


def test_noalloc_rejects_too_many_sequences():
    from flashqla_b200 import _cabi
    lib = _cabi.lib()
    dummy = torch.zeros(8, dtype=torch.int32, device="cuda")
    a = _cabi.QlaChunkFwdArgs(batch=1, seq_len=8192, num_seqs=4097, num_k_heads=1, num_v_heads=1,
                              cu_seqlens=dummy.data_ptr())
    assert lib.qla_chunk_fwd_noalloc(a, None) == -1
    assert b"at most 4096" in lib.qla_last_error()
