"""GPU parity against the CPU oracle at the sizes of the headline configurations.

Heads and sequences are independent, so where the oracle on everything would take too long it checks a
subset of heads / sequences of the full-size GPU call (which always runs at the full size: all CTAs, all
context-parallel segments, all rounds).

* config 1: one sequence of 32768 tokens, Hk 16 / Hv 32: output and final state, all heads;
* config 2: 64 packed sequences of 512..16384 tokens (seeded), Hk = Hv = 8, per-sequence initial state:
  the longest, the shortest and two more sequences;
* config 3: training step B=4, T=8192, Hk = Hv = 32: all six gradients of one batch row, three heads;
* config 4: decode and 4-token verify (fp32 and bf16 scratch, and a bf16 state pool) for 256 sequences,
  Hk 16 / Hv 32, against the per-token loop.

Tolerances: relative rms <= 5e-3 and max |err| <= 2 % of max |ref| (prefill, gradients); recurrent op
o <= 3e-3, fp32 states <= 1e-4, 16-bit states <= 1 % of max |ref| (one 16-bit rounding is 0.4 %).
"""
import pytest
import torch

from oracle import gdr_oracle as orc

pytestmark = pytest.mark.gpu
RMS, MAXR = 5e-3, 2e-2


def _close(name, got, ref, rms=RMS, maxr=MAXR):
    got, ref = got.float().cpu(), ref.float()
    e, m = orc.rel_rms(got, ref), orc.max_abs_ratio(got, ref)
    assert e <= rms and m <= maxr, f"{name}: rel_rms {e:.2e} (<= {rms}), max ratio {m:.2e} (<= {maxr})"


def test_config1_forward_all_heads():
    import flashqla_b200 as fq
    inp = orc.make_prefill_inputs(1, 32768, 16, 32, seed=1)
    c = {n: t.cuda() for n, t in inp.items()}
    _, _, o, _, fs = fq.chunk_gated_delta_rule_fwd(c["q"], c["k"], c["v"], c["g"], c["beta"])
    fq.check_device_status()
    torch.set_num_threads(max(1, torch.get_num_threads()))
    ref = orc.chunk_gdr_fwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"])
    _close("o", o, ref["o"])
    _close("final_state", fs, ref["final_state"])
    # the error must not grow along the 512 chunks: the last eighth of the sequence by itself
    _close("o[last 4096 tokens]", o[:, -4096:], ref["o"][:, -4096:])


def test_config2_varlen_forward_subset_of_sequences():
    import flashqla_b200 as fq
    gen = torch.Generator().manual_seed(2)
    lens = torch.randint(512, 16385, (64,), generator=gen).tolist()
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    inp = orc.make_prefill_inputs(1, cu[-1], 8, 8, seed=20, with_h0=True, n_states=64)
    c = {n: t.cuda() for n, t in inp.items()}
    cu_dev = torch.tensor(cu, dtype=torch.int32, device="cuda")
    _, _, o, _, fs = fq.chunk_gated_delta_rule_fwd(c["q"], c["k"], c["v"], c["g"], c["beta"], initial_state=c["h0"],
                                                   cu_seqlens=cu_dev)
    fq.check_device_status()
    order = sorted(range(64), key=lambda i: lens[i])
    for n in (order[-1], order[0], order[31], 63):
        a, b = cu[n], cu[n + 1]
        ref = orc.chunk_gdr_fwd(inp["q"][:, a:b], inp["k"][:, a:b], inp["v"][:, a:b], inp["g"][:, a:b],
                                inp["beta"][:, a:b], h0=inp["h0"][n:n + 1])
        _close(f"o[seq {n}, {b - a} tokens]", o[:, a:b], ref["o"])
        _close(f"final_state[seq {n}]", fs[n:n + 1], ref["final_state"])


def test_config3_gradients_subset_of_heads():
    import flashqla_b200 as fq
    B, T, H = 4, 8192, 32
    inp = orc.make_prefill_inputs(B, T, H, H, seed=3, with_h0=True, with_grads=True)
    c = {n: t.cuda() for n, t in inp.items()}
    g_cs, A, o, h, fs, vn = fq.chunk_gated_delta_rule_fwd(c["q"], c["k"], c["v"], c["g"], c["beta"],
                                                          initial_state=c["h0"], output_h=True, output_v_new=True)
    got = fq.chunk_gated_delta_rule_bwd(c["q"], c["k"], c["v"], g_cs, c["beta"], A, c["do"], dht=c["dht"],
                                        initial_state=c["h0"], h=h, v_new=vn)
    fq.check_device_status()
    dq, dk, dv, db, dg, dh0 = got
    row, heads = 2, [0, 13, 31]
    sl = lambda t: t[row:row + 1][:, :, heads]
    ref = orc.chunk_gdr_bwd(sl(inp["q"]), sl(inp["k"]), sl(inp["v"]), sl(inp["g"]), sl(inp["beta"]), sl(inp["do"]),
                            dht=inp["dht"][row:row + 1, heads], h0=inp["h0"][row:row + 1, heads])
    _close("o", sl(o), ref["o"])
    _close("final_state", fs[row:row + 1, heads], ref["final_state"])
    for name, t in (("dq", dq), ("dk", dk), ("dv", dv), ("db", db), ("dg", dg)):
        _close(name, sl(t), ref[name])
    _close("dh0", dh0[row:row + 1, heads], ref["dh0"])


def _recurrent_inputs(N, T, Hk, Hv, seed):
    gen = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=gen)
    return dict(q=orc.l2norm(rn(1, N * T, Hk, 128)).bfloat16(), k=orc.l2norm(rn(1, N * T, Hk, 128)).bfloat16(),
                v=rn(1, N * T, Hv, 128).bfloat16(), g=torch.nn.functional.logsigmoid(rn(1, N * T, Hv)),
                beta=torch.sigmoid(rn(1, N * T, Hv)), state=0.1 * rn(N, Hv, 128, 128))


@pytest.mark.parametrize("mode", ["decode", "verify_f32", "verify_bf16", "decode_bf16_pool"])
def test_config4_recurrent_against_per_token_loop(mode):
    import flashqla_b200 as fq
    N, Hk, Hv = 256, 16, 32
    verify = mode.startswith("verify")
    T = 4 if verify else 1
    inp = _recurrent_inputs(N, T, Hk, Hv, seed=4)
    c = {n: t.cuda() for n, t in inp.items()}
    pool_dtype = torch.bfloat16 if mode == "decode_bf16_pool" else torch.float32
    pool = c["state"].to(pool_dtype)
    inter_dtype = torch.bfloat16 if mode == "verify_bf16" else torch.float32
    inter = torch.zeros(N, T, Hv, 128, 128, dtype=inter_dtype, device="cuda") if verify else None
    o = fq.fused_sigmoid_gating_delta_rule_update(
        None, c["g"], None, c["q"], c["k"], c["v"], c["beta"], pool, use_qk_l2norm_in_kernel=False,
        a_is_log_decay=True, b_is_beta=True, disable_state_update=verify, intermediate_states_buffer=inter)
    fq.check_device_status()
    # the oracle on the first 64 sequences (the per-token Python loop); every sequence is independent
    n = 64
    state_ref = inp["state"][:n].to(pool_dtype).clone()
    inter_ref = torch.zeros(n, T, Hv, 128, 128, dtype=inter_dtype) if verify else None
    zeros = torch.zeros(Hv)
    o_ref = orc.recurrent_update_ref(zeros, inp["g"][:, :n * T], zeros, inp["q"][:, :n * T], inp["k"][:, :n * T],
                                     inp["v"][:, :n * T], inp["beta"][:, :n * T], state_ref, use_qk_l2norm=False,
                                     a_is_log_decay=True, b_is_beta=True, disable_state_update=verify,
                                     inter=inter_ref)
    assert orc.max_abs(o[:, :n * T].float().cpu(), o_ref) <= 3e-3
    if verify:
        assert torch.equal(pool.cpu(), inp["state"]), "verify must leave the pool untouched"
        if inter_dtype == torch.float32:
            assert orc.max_abs(inter[:n].cpu(), inter_ref) <= 1e-4
        else:
            assert orc.max_abs_ratio(inter[:n].float().cpu(), inter_ref.float()) <= 1e-2
    elif pool_dtype == torch.float32:
        assert orc.max_abs(pool[:n].cpu(), state_ref) <= 1e-4
    else:
        assert orc.max_abs_ratio(pool[:n].float().cpu(), state_ref.float()) <= 1e-2
