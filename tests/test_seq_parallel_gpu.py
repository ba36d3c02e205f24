"""GPU parity of the cross-GPU sequence-parallel forward, with the ranks run one after the other on ONE GPU:
the slices' kernels are ordinary launches in stream order (none waits for another), and the all-gather is a
torch.stack of the per-slice summaries.  Compared with the fp64 oracle on the whole sequence and with the
single-call forward.  Tolerances as for the forward: relative rms 5e-3 on o and on the final state."""
import pytest
import torch

from oracle import gdr_oracle as orc

pytestmark = pytest.mark.gpu

RMS_TOL = 5e-3


def _run_slices(sp, c, cuts, h0):
    ctxs = []
    t0 = 0
    for n in cuts:
        sl = slice(t0, t0 + n)
        ctxs.append(sp.slice_summary(c["q"][:, sl], c["k"][:, sl], c["v"][:, sl], c["g"][:, sl], c["beta"][:, sl]))
        t0 += n
    gathered = torch.stack([x.summary for x in ctxs])
    outs, end = [], None
    for r, ctx in enumerate(ctxs):
        incoming = sp.fold_incoming_state(gathered, r, h0) if (r > 0 or h0 is not None) else None
        o, end = sp.slice_forward(ctx, incoming)
        outs.append(o)
    return torch.cat(outs, dim=1), end, ctxs


@pytest.mark.parametrize("cuts,gate_div,with_h0", [
    ((1024, 1024), 1.0, False),          # slices long enough to be cut into local segments
    ((2048, 1024, 3072), 1.0, True),     # unequal slices, initial state
    ((512, 512), 64.0, True),            # weak gates, one segment per slice: transition matrices cross the ranks
    ((2048, 2048), 64.0, True),          # weak gates and local segments: prefix products of transition matrices
])
def test_slices_reproduce_whole_sequence(cuts, gate_div, with_h0):
    import flashqla_b200 as fq
    from flashqla_b200 import seq_parallel as sp
    T, Hk, Hv = sum(cuts), 2, 4
    inp = orc.make_prefill_inputs(1, T, Hk, Hv, seed=31, with_h0=with_h0, gate_div=gate_div)
    c = {n: t.cuda() for n, t in inp.items()}
    h0 = c.get("h0")
    o, end, ctxs = _run_slices(sp, c, cuts, h0)
    if cuts[0] >= 1024:
        assert ctxs[0].plan.n_seg > 1
    if gate_div > 1.0:
        assert float(ctxs[0].summary[1].abs().max()) > 0.0  # a transition matrix really crosses
    else:
        assert float(ctxs[0].summary[1].abs().max()) == 0.0
    ref = orc.chunk_gdr_fwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], h0=inp.get("h0"), dtype=torch.float64)
    assert orc.rel_rms(o.float().cpu(), ref["o"]) <= RMS_TOL
    assert orc.rel_rms(end.float().cpu(), ref["final_state"]) <= RMS_TOL
    _, _, o1, _, fs1 = fq.chunk_gated_delta_rule_fwd(c["q"], c["k"], c["v"], c["g"], c["beta"], initial_state=h0)
    assert orc.rel_rms(o.float().cpu(), o1.float().cpu()) <= RMS_TOL
    assert orc.rel_rms(end.cpu(), fs1.cpu()) <= RMS_TOL


def test_slice_must_be_whole_chunks():
    from flashqla_b200 import seq_parallel as sp
    inp = orc.make_prefill_inputs(1, 100, 1, 2, seed=1)
    c = {n: t.cuda() for n, t in inp.items()}
    with pytest.raises(ValueError):
        sp.slice_summary(c["q"], c["k"], c["v"], c["g"], c["beta"])
