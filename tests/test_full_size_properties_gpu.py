"""Properties that hold at any size, checked at the full sizes of the headline configurations (where the
oracle would take minutes): the forward of config 1 (1 x 32768 tokens, Hk 16 / Hv 32) and the recurrent
op of config 4 (256 sequences, Hv 32).

* splitting a sequence at a chunk boundary and carrying the state gives the same outputs as one call;
* the context-parallel plan (segments, warm-up, chaining) gives the same outputs as the plain scan;
* with a zero initial state the op is linear in v;
* verifying T draft tokens in one call equals T decode calls, and the cached state of step t is the pool
  after t decode calls.

Tolerances: relative rms 5e-3 between two 16-bit results of the same quantity (each carries its own
rounding); 1e-4 max-abs for fp32 states of the recurrent op (the reference's gate,
benchmark/bench_recurrent_fused_matrix.py:515-517)."""
import pytest
import torch

from oracle import gdr_oracle as orc

pytestmark = pytest.mark.gpu

T, HK, HV = 32768, 16, 32


@pytest.fixture(scope="module")
def cfg1():
    gen = torch.Generator(device="cuda").manual_seed(1)
    rn = lambda *s: torch.randn(*s, generator=gen, device="cuda")
    unit = lambda x: x * torch.rsqrt((x * x).sum(-1, keepdim=True) + 1e-6)
    return dict(q=unit(rn(1, T, HK, 128)).bfloat16(), k=unit(rn(1, T, HK, 128)).bfloat16(),
                v=rn(1, T, HV, 128).bfloat16(), g=torch.nn.functional.logsigmoid(rn(1, T, HV)),
                beta=torch.sigmoid(rn(1, T, HV)))


def _rel(a, b):
    return orc.rel_rms(a.float(), b.float())


def test_split_with_carried_state_equals_one_call(cfg1):
    import flashqla_b200 as fq
    c = cfg1
    _, _, o, _, fs = fq.chunk_gated_delta_rule_fwd(c["q"], c["k"], c["v"], c["g"], c["beta"])
    cut = 64 * 201  # a chunk boundary that is not a segment boundary of the plan
    part = lambda a, b: [c[n][:, a:b].contiguous() for n in ("q", "k", "v", "g", "beta")]
    _, _, o1, _, s1 = fq.chunk_gated_delta_rule_fwd(*part(0, cut))
    _, _, o2, _, s2 = fq.chunk_gated_delta_rule_fwd(*part(cut, T), initial_state=s1)
    assert _rel(torch.cat((o1, o2), dim=1), o) <= 5e-3
    assert _rel(s2, fs) <= 5e-3


def test_context_parallel_plan_equals_plain_scan(cfg1):
    import flashqla_b200 as fq
    c = cfg1
    _, _, o_cp, _, fs_cp = fq.chunk_gated_delta_rule_fwd(c["q"], c["k"], c["v"], c["g"], c["beta"], auto_cp=True)
    _, _, o, _, fs = fq.chunk_gated_delta_rule_fwd(c["q"], c["k"], c["v"], c["g"], c["beta"], auto_cp=False)
    assert _rel(o_cp, o) <= 5e-3
    assert _rel(fs_cp, fs) <= 5e-3


def test_linear_in_v(cfg1):
    import flashqla_b200 as fq
    c = cfg1
    v2 = torch.roll(c["v"], 1, dims=1)
    run = lambda v: fq.chunk_gated_delta_rule_fwd(c["q"], c["k"], v, c["g"], c["beta"])
    _, _, oa, _, sa = run(c["v"])
    _, _, ob, _, sb = run(v2)
    _, _, oc, _, sc = run((c["v"].float() + v2.float()).bfloat16())
    # three 16-bit outputs and a 16-bit rounded sum of the inputs: a few roundings of 2^-9 each
    assert _rel(oa.float() + ob.float(), oc) <= 1e-2
    assert _rel(sa + sb, sc) <= 1e-2


def test_verify_equals_successive_decodes():
    import flashqla_b200 as fq
    N, steps = 256, 4
    gen = torch.Generator(device="cuda").manual_seed(4)
    rn = lambda *s: torch.randn(*s, generator=gen, device="cuda")
    unit = lambda x: x * torch.rsqrt((x * x).sum(-1, keepdim=True) + 1e-6)
    q, k = unit(rn(1, N * steps, HK, 128)).bfloat16(), unit(rn(1, N * steps, HK, 128)).bfloat16()
    v = rn(1, N * steps, HV, 128).bfloat16()
    g, beta = torch.nn.functional.logsigmoid(rn(1, N * steps, HV)), torch.sigmoid(rn(1, N * steps, HV))
    pool0 = 0.1 * rn(N, HV, 128, 128)
    kw = dict(use_qk_l2norm_in_kernel=False, a_is_log_decay=True, b_is_beta=True)
    # one verify call: tokens of sequence n are n * steps .. n * steps + steps - 1
    pool_v = pool0.clone()
    inter = torch.zeros(N, steps, HV, 128, 128, device="cuda")
    o_v = fq.fused_sigmoid_gating_delta_rule_update(None, g, None, q, k, v, beta, pool_v,
                                                    intermediate_states_buffer=inter, cache_steps=steps, **kw)
    # the same tokens as `steps` decode calls
    pool_d = pool0.clone()
    o_v = o_v.view(N, steps, HV, 128)
    for t in range(steps):
        sel = lambda x: x.view(N, steps, *x.shape[2:])[:, t].unsqueeze(0).contiguous()
        o_t = fq.fused_sigmoid_gating_delta_rule_update(None, sel(g), None, sel(q), sel(k), sel(v), sel(beta), pool_d,
                                                        assume_regular=True, **kw)
        assert orc.max_abs(o_t[0].float(), o_v[:, t].float()) <= 3e-3
        assert orc.max_abs(inter[:, t], pool_d) <= 1e-4
    assert orc.max_abs(pool_v, pool_d) <= 1e-4


def test_backward_is_linear_in_do_at_config3():
    """Config 3 (4 x 8192 tokens, 32 heads): for fixed inputs every gradient is linear in the output gradient."""
    import flashqla_b200 as fq
    B, T3, H = 4, 8192, 32
    gen = torch.Generator(device="cuda").manual_seed(3)
    rn = lambda *s: torch.randn(*s, generator=gen, device="cuda")
    unit = lambda x: x * torch.rsqrt((x * x).sum(-1, keepdim=True) + 1e-6)
    q, k = unit(rn(B, T3, H, 128)).bfloat16(), unit(rn(B, T3, H, 128)).bfloat16()
    v = rn(B, T3, H, 128).bfloat16()
    g, beta = torch.nn.functional.logsigmoid(rn(B, T3, H)), torch.sigmoid(rn(B, T3, H))
    g_cs, A, o, h, fs, v_new = fq.chunk_gated_delta_rule_fwd(q, k, v, g, beta, output_h=True, output_v_new=True)
    do1, do2 = rn(B, T3, H, 128).bfloat16(), rn(B, T3, H, 128).bfloat16()
    run = lambda do: fq.chunk_gated_delta_rule_bwd(q, k, v, g_cs, beta, A, do, h=h, v_new=v_new)[:5]
    ga, gb = run(do1), run(do2)
    gc = run((do1.float() + do2.float()).bfloat16())
    for name, a, b, c in zip(("dq", "dk", "dv", "dbeta", "dg"), ga, gb, gc):
        assert orc.rel_rms(a.float() + b.float(), c.float()) <= 2e-2, name
