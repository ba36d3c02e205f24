"""CPU: work partitioning across ranks (no data-path collective) and the context-parallel planner.
The two-rank test runs real torch.distributed processes on the gloo backend."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flashqla_b200 import cp, sharding
from oracle import gdr_oracle as orc


def test_head_shards_keep_gqa_groups():
    for world in (1, 2, 4, 8):
        seen_k, seen_v = [], []
        for r in range(world):
            ks, vs = sharding.head_shard(16, 32, world, r)
            assert (vs.stop - vs.start) == 2 * (ks.stop - ks.start)
            assert vs.start == 2 * ks.start
            seen_k += list(range(ks.start, ks.stop))
            seen_v += list(range(vs.start, vs.stop))
        assert seen_k == list(range(16)) and seen_v == list(range(32))
    with pytest.raises(ValueError):
        sharding.head_shard(6, 12, 4, 0)


def test_sequence_balance_is_a_partition_and_balanced():
    gen = torch.Generator().manual_seed(2)
    lens = torch.randint(512, 16385, (64,), generator=gen).tolist()
    for world in (1, 2, 4, 8):
        parts = sharding.balance_sequences(lens, world)
        assert sorted(i for p in parts for i in p) == list(range(64))
        loads = [sum(lens[i] for i in p) for p in parts]
        assert max(loads) - min(loads) <= max(lens)
    assert sharding.balance_sequences([], 2) == [[], []]


def test_batch_shard_covers_batch():
    for B, world in ((4, 2), (4, 4), (5, 2), (3, 4)):
        rows = []
        for r in range(world):
            s = sharding.batch_shard(B, world, r)
            rows += list(range(s.start, s.stop))
        assert rows == list(range(B))


def test_cp_planner_rules():
    p = cp.plan_segments([32768], 32, 148)
    assert p.use_cp and p.cu[0] == 0 and p.cu[-1] == 32768
    assert p.seg_next[-1] == -1 and p.seg_raw[-1] == 0 and p.raw_first == [0, len(p.seg_next)]
    # every cut is a multiple of the chunk size, so chunk numbering is unchanged
    assert all(c % 64 == 0 for c in p.cu[:-1])
    # many chains already: no CP; short sequences: no CP
    assert not cp.plan_segments([4096] * 64, 8, 148).use_cp
    assert not cp.plan_segments([512], 4, 148).use_cp
    # mixed lengths: short sequences stay whole
    p = cp.plan_segments([3000, 100, 2077], 2, 148)
    assert p.use_cp and p.raw_first[1] - p.raw_first[0] > 1 and p.raw_first[2] - p.raw_first[1] == 1
    assert [p.cu[i] for i in p.raw_first] == [0, 3000, 3100, 5177]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    # every rank runs the oracle on its head shard of the same seeded problem; rank 0 gathers o
    inp = orc.make_prefill_inputs(1, 96, 2, 4, seed=5, with_h0=True)
    ks, vs = sharding.head_shard(2, 4, world, rank)
    res = orc.chunk_gdr_fwd(inp["q"][:, :, ks], inp["k"][:, :, ks], inp["v"][:, :, vs], inp["g"][:, :, vs],
                            inp["beta"][:, :, vs], h0=inp["h0"][:, vs])
    parts = [torch.empty_like(res["o"]) for _ in range(world)]
    dist.all_gather(parts, res["o"].contiguous())      # test plumbing only: the op itself needs no exchange
    t = torch.tensor([float(rank + 1)])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)            # the bench's max-over-ranks timing reduction
    if rank == 0:
        full = orc.chunk_gdr_fwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], h0=inp["h0"])
        out.put((float((torch.cat(parts, dim=2) - full["o"]).abs().max()), float(t.item())))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_head_sharding_reproduces_single_rank():
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    err, tmax = out.get()
    assert err < 1e-5 and tmax == 2.0


def _sp_rank_main(rank, world, port, out):
    """Sequence-parallel carry with the oracle standing in for the kernels: every rank summarises its slice
    as (end state from zero, transition matrix), one all_gather, fold, then the slice with its incoming state."""
    from flashqla_b200.seq_parallel import fold_incoming_state
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    Hv, K, T = 2, 64, 64 * 2 * world
    inp = orc.make_prefill_inputs(1, T, 1, Hv, K=K, V=K, seed=9, with_h0=True, dtype=torch.float32, gate_div=4.0)
    sl = slice(rank * T // world, (rank + 1) * T // world)
    mine = {n: inp[n][:, sl] for n in ("q", "k", "v", "g", "beta")}
    run = lambda v, h0: orc.chunk_gdr_fwd(mine["q"], mine["k"], v, mine["g"], mine["beta"], h0=h0, dtype=torch.float64)
    H = run(mine["v"], None)["final_state"][0]
    M = run(torch.zeros_like(mine["v"]), torch.eye(K).expand(1, Hv, K, K))["final_state"][0]
    summary = torch.stack((H, M)).float()
    gathered = [torch.empty_like(summary) for _ in range(world)]
    dist.all_gather(gathered, summary)
    incoming = fold_incoming_state(torch.stack(gathered), rank, inp["h0"])
    res = run(mine["v"], incoming[None].double())
    full = orc.chunk_gdr_fwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], h0=inp["h0"], dtype=torch.float64)
    err = float((res["o"] - full["o"][:, sl]).abs().max())
    if rank == world - 1:
        err = max(err, float((res["final_state"] - full["final_state"]).abs().max()))
    t = torch.tensor([err])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        out.put(float(t.item()))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sequence_parallel_carry_reproduces_single_rank(world):
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_sp_rank_main, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    assert out.get() < 1e-5


def _sp_bwd_rank_main(rank, world, port, out):
    """Reverse carry of the sequence-parallel backward with the oracle standing in for the kernels: every rank
    summarises its slice as (start-state gradient for a zero gradient behind it, gradient transition matrix),
    one all_gather, fold from the right, then the slice's backward with its incoming gradient."""
    from flashqla_b200.seq_parallel import fold_incoming_gradient, fold_incoming_state
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    Hv, K, T = 2, 64, 64 * 2 * world
    inp = orc.make_prefill_inputs(1, T, 1, Hv, K=K, V=K, seed=11, with_h0=True, with_grads=True,
                                  dtype=torch.float32, gate_div=4.0)
    sl = slice(rank * T // world, (rank + 1) * T // world)
    mine = {n: inp[n][:, sl] for n in ("q", "k", "v", "g", "beta", "do")}
    # forward carry first: the state entering the slice
    fwd = lambda v, h0: orc.chunk_gdr_fwd(mine["q"], mine["k"], v, mine["g"], mine["beta"], h0=h0, dtype=torch.float64)
    eye = torch.eye(K).expand(1, Hv, K, K)
    fsum = torch.stack((fwd(mine["v"], None)["final_state"][0], fwd(torch.zeros_like(mine["v"]), eye)["final_state"][0])).float()
    fg = [torch.empty_like(fsum) for _ in range(world)]
    dist.all_gather(fg, fsum)
    incoming = fold_incoming_state(torch.stack(fg), rank, inp["h0"])[None]
    bwd = lambda do, dht: orc.chunk_gdr_bwd(mine["q"], mine["k"], mine["v"], mine["g"], mine["beta"], do, dht=dht,
                                            h0=incoming)
    G = bwd(mine["do"], None)["dh0"][0]
    Md = bwd(torch.zeros_like(mine["do"]), eye.contiguous())["dh0"][0]
    bsum = torch.stack((G, Md)).float()
    bg = [torch.empty_like(bsum) for _ in range(world)]
    dist.all_gather(bg, bsum)
    D = fold_incoming_gradient(torch.stack(bg), rank, inp["dht"])
    res = bwd(mine["do"], D[None])
    full = orc.chunk_gdr_bwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], inp["do"], dht=inp["dht"], h0=inp["h0"])
    err = 0.0
    for n in ("dq", "dk", "dv", "db", "dg"):
        err = max(err, float((res[n].float() - full[n][:, sl].float()).abs().max() / full[n].float().abs().max()))
    if rank == 0:
        err = max(err, float((res["dh0"] - full["dh0"]).abs().max() / full["dh0"].abs().max()))
    t = torch.tensor([err])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        out.put(float(t.item()))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sequence_parallel_reverse_carry_reproduces_single_rank(world):
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_sp_bwd_rank_main, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    assert out.get() < 1e-4
