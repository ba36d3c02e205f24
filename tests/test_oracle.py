"""CPU: pin oracle/gdr_oracle.py against fixtures produced by the reference's own CPU code
(tests/golden/make_golden.py: ref_gdr.chunk_gated_delta_rule_fwd/_bwd and cpu_ref)."""
import pytest
import torch

from oracle import gdr_oracle as orc


def _load(golden_dir, name):
    return torch.load(golden_dir / f"{name}.pt", weights_only=False)


@pytest.mark.parametrize("name", ["cfg0_fp32_k64", "tail_gqa_bwd", "weak_gate_bwd"])
def test_forward_matches_reference_oracle(golden_dir, name):
    fx = _load(golden_dir, name)
    i = fx["inputs"]
    res = orc.chunk_gdr_fwd(i["q"], i["k"], i["v"], i["g"], i["beta"], scale=fx["meta"]["scale"],
                            h0=i.get("h0"))
    assert orc.max_abs(res["g_cumsum"], fx["g_cumsum"]) < 1e-5
    assert orc.rel_rms(res["o"], fx["o"]) < 2e-6
    assert orc.rel_rms(res["final_state"], fx["final_state"]) < 2e-6
    # the per-token recurrence is the same map
    o2, s2 = orc.naive_recurrent_gdr(i["q"], i["k"], i["v"], i["g"], i["beta"],
                                     scale=fx["meta"]["scale"], h0=i.get("h0"))
    assert orc.rel_rms(o2, fx["o"]) < 5e-6
    assert orc.rel_rms(s2, fx["final_state"]) < 5e-6


def test_inputs_are_reproducible(golden_dir):
    """The seeded generator must give the same tensors on every machine (GPU tests rely on it)."""
    fx = _load(golden_dir, "tail_gqa_bwd")
    m = fx["meta"]
    again = orc.make_prefill_inputs(m["B"], m["T"], m["Hk"], m["Hv"], m["K"], m["V"], seed=m["seed"],
                                    with_h0=True, with_grads=True)
    for n, t in fx["inputs"].items():
        assert torch.equal(t, again[n]), n


@pytest.mark.parametrize("name", ["tail_gqa_bwd", "weak_gate_bwd"])
def test_backward_matches_reference_oracle(golden_dir, name):
    fx = _load(golden_dir, name)
    i = fx["inputs"]
    res = orc.chunk_gdr_bwd(i["q"], i["k"], i["v"], i["g"], i["beta"], i["do"], dht=i["dht"],
                            scale=fx["meta"]["scale"], h0=i["h0"])
    for n in ("dq", "dk", "dv", "db", "dg", "dh0"):
        assert orc.rel_rms(res[n], fx[n]) < 2e-5, n


def test_varlen_equals_per_sequence(golden_dir):
    fx = _load(golden_dir, "weak_gate_bwd")
    i = fx["inputs"]
    T = fx["meta"]["T"]
    pk = {n: i[n].reshape(1, -1, *i[n].shape[2:]) for n in ("q", "k", "v", "g", "beta")}
    res = orc.chunk_gdr_fwd_varlen(**pk, cu_seqlens=[0, T, 2 * T], scale=fx["meta"]["scale"], h0=i["h0"])
    assert orc.rel_rms(res["o"].reshape(fx["o"].shape), fx["o"]) < 2e-6
    assert orc.rel_rms(res["final_state"], fx["final_state"]) < 2e-6


@pytest.mark.parametrize("case", ["chain_f32", "chain_bf16", "hop_f32", "hop_bf16"])
def test_recurrent_matches_reference_cpu_loop(golden_dir, case):
    fx = _load(golden_dir, "recurrent_verify")
    i, m, c = fx["inputs"], fx["meta"], fx["cases"][case]
    dt = torch.float32 if case.endswith("f32") else torch.bfloat16
    inter = torch.zeros(m["N"], m["T"], m["HV"], 128, 128, dtype=dt)
    state = i["h0"].clone()
    o = orc.recurrent_update_ref(i["A_log"], i["a"], i["dt_bias"], i["q"], i["k"], i["v"], i["b"], state,
                                 scale=m["scale"], softplus_beta=m["softplus_beta"],
                                 softplus_threshold=m["softplus_threshold"], use_qk_l2norm=True,
                                 disable_state_update=True, inter=inter, parents=c["parents"])
    assert torch.equal(state, i["h0"])
    o = o.view(m["N"], m["T"], m["HV"], 128)
    assert orc.max_abs(o, c["o"]) < 2e-6
    assert orc.max_abs(inter[:, -1].float(), c["inter_last"]) < 2e-6
    assert orc.max_abs(inter.float().sum(-1), c["inter_rowsum"]) < 1e-4


def test_inverse_gate_roundtrip():
    g = torch.nn.functional.logsigmoid(torch.randn(64))
    beta = torch.sigmoid(torch.randn(64))
    a, b = orc.inverse_gate(g, beta)
    assert torch.allclose(-torch.nn.functional.softplus(a), g, atol=1e-5)
    assert torch.allclose(torch.sigmoid(b), beta, atol=1e-6)


def test_oracle_agrees_with_the_reference_file_when_present():
    """Where oracle/build_ref.py has placed the reference's own tests/ref_gdr.py under oracle/_ref/, the port and
    the reference's forward agree on fresh seeded inputs (a tail chunk, GQA, an initial state)."""
    import importlib.util
    from pathlib import Path
    import pytest
    ref_file = Path(__file__).resolve().parents[1] / "oracle" / "_ref" / "ref_gdr.py"
    if not ref_file.exists():
        pytest.skip("no reference checkout was at hand when the library was built")
    spec = importlib.util.spec_from_file_location("_ref_gdr", ref_file)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    inp = orc.make_prefill_inputs(2, 200, 2, 4, seed=11, dtype=torch.float32, with_h0=True)
    g_cs, o, A, h, fs = ref.chunk_gated_delta_rule_fwd(inp["q"], inp["k"], inp["v"], inp["g"].clone(), inp["beta"],
                                                       initial_state=inp["h0"], scale=128 ** -0.5)
    mine = orc.chunk_gdr_fwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], h0=inp["h0"])
    assert orc.max_abs(mine["o"], o) <= 2e-5
    assert orc.max_abs(mine["final_state"], fs) <= 2e-5
    assert orc.max_abs(mine["g_cumsum"], g_cs) <= 2e-6
