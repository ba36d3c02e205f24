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


@pytest.mark.parametrize("cuts,gate_div", [((1024, 1024), 1.0), ((2048, 1024, 3072), 4.0), ((512, 512), 64.0)])
def test_backward_slices_reproduce_whole_sequence(cuts, gate_div):
    """Forward carry, then the reverse carry: per slice (G, Md) from one state-only launch of the reverse scan,
    the stack stands in for the all-gather, fold from the right, ordinary backward per slice.  Tolerance as for
    the backward: relative rms 5e-3 per gradient (dg 1e-2 with weak gates) against the fp64 oracle on the whole
    sequence."""
    from flashqla_b200 import seq_parallel as sp
    T, Hk, Hv = sum(cuts), 2, 4
    inp = orc.make_prefill_inputs(1, T, Hk, Hv, seed=35, with_h0=True, with_grads=True, gate_div=gate_div)
    c = {n: t.cuda() for n, t in inp.items()}
    _, _, fctx = _run_slices(sp, c, cuts, c["h0"])
    fgathered = torch.stack([x.summary for x in fctx])
    bctx, t0 = [], 0
    for r, n in enumerate(cuts):
        sl = slice(t0, t0 + n)
        incoming = sp.fold_incoming_state(fgathered, r, c["h0"]).unsqueeze(0)
        bctx.append(sp.slice_backward_summary(c["q"][:, sl], c["k"][:, sl], c["v"][:, sl], c["g"][:, sl],
                                              c["beta"][:, sl], c["do"][:, sl], incoming))
        t0 += n
    gathered = torch.stack([x.summary for x in bctx])
    if gate_div > 4.0:
        assert float(gathered[1, 1].abs().max()) > 1e-5   # a gradient transition matrix really crosses
    parts = [sp.slice_backward(ctx, sp.fold_incoming_gradient(gathered, r, c["dht"])) for r, ctx in enumerate(bctx)]
    import flashqla_b200 as fq
    fq.check_device_status()
    ref = orc.chunk_gdr_bwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], inp["do"], dht=inp["dht"],
                            h0=inp["h0"])
    for i, n in enumerate(("dq", "dk", "dv", "db", "dg")):
        got = torch.cat([p[i] for p in parts], dim=1).float().cpu()
        tol = 1e-2 if (n == "dg" and gate_div > 1.0) else RMS_TOL
        assert orc.rel_rms(got, ref[n]) <= tol, (n, orc.rel_rms(got, ref[n]))
    assert orc.rel_rms(parts[0][5].float().cpu(), ref["dh0"]) <= RMS_TOL


def test_slice_must_be_whole_chunks():
    from flashqla_b200 import seq_parallel as sp
    inp = orc.make_prefill_inputs(1, 100, 1, 2, seed=1)
    c = {n: t.cuda() for n, t in inp.items()}
    with pytest.raises(ValueError):
        sp.slice_summary(c["q"], c["k"], c["v"], c["g"], c["beta"])


def _nccl_rank(rank, world, port, out):
    import os
    import torch.distributed as dist
    import flashqla_b200 as fq
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    T, Hk, Hv = 4096, 2, 4
    inp = orc.make_prefill_inputs(1, T, Hk, Hv, seed=33, with_h0=True)
    sl = slice(rank * T // world, (rank + 1) * T // world)
    c = {n: (t[:, sl] if n != "h0" else t).cuda() for n, t in inp.items()}
    o, fs = fq.chunk_gated_delta_rule_fwd_sp(c["q"], c["k"], c["v"], c["g"], c["beta"], initial_state=c["h0"],
                                             broadcast_final_state=True)
    ref = orc.chunk_gdr_fwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], h0=inp["h0"], dtype=torch.float64)
    # backward: the reverse carry over the same group
    full = orc.make_prefill_inputs(1, T, Hk, Hv, seed=33, with_h0=True, with_grads=True)
    do, dht = full["do"][:, sl].cuda(), full["dht"].cuda()
    _, _, incoming = fq.chunk_gated_delta_rule_fwd_sp(c["q"], c["k"], c["v"], c["g"], c["beta"],
                                                      initial_state=c["h0"], return_incoming_state=True)
    grads = fq.chunk_gated_delta_rule_bwd_sp(c["q"], c["k"], c["v"], c["g"], c["beta"], do, incoming_state=incoming,
                                             dht=dht)
    bref = orc.chunk_gdr_bwd(full["q"], full["k"], full["v"], full["g"], full["beta"], full["do"], dht=full["dht"],
                             h0=full["h0"])
    e_b = max(orc.rel_rms(grads[i].float().cpu(), bref[n][:, sl]) for i, n in enumerate(("dq", "dk", "dv", "db", "dg")))
    if rank == 0:
        e_b = max(e_b, orc.rel_rms(grads[5].float().cpu(), bref["dh0"]))
    err = torch.tensor([orc.rel_rms(o.float().cpu(), ref["o"][:, sl]),
                        orc.rel_rms(fs.float().cpu(), ref["final_state"]), e_b], device="cuda")
    dist.all_reduce(err, op=dist.ReduceOp.MAX)
    if rank == 0:
        out.put(err.cpu().tolist())
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpus_nccl_all_gather():
    """The real collective: needs two GPUs, skipped on a single-GPU box."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import socket
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    procs = [ctx.Process(target=_nccl_rank, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    e_o, e_fs, e_b = out.get()
    assert e_o <= RMS_TOL and e_fs <= RMS_TOL and e_b <= RMS_TOL
