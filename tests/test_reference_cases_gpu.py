"""GPU parity on the shapes and input distributions of the reference's own precision and shape suites.

* tests/bench_precision_gdr.py:113-160 (SMOKE_CASES + FULL_EXTRA_CASES): 16 / 16 and 8 / 16 heads, tails of
  17, 48 and 96 tokens, batch 2, a 3-sequence packed mix, half of the heads without decay, and gates scaled
  by 128 / 16 (log decay down to about -400 per chunk); initial state ~ N(0, 1), dht ~ N(0, 1) / 8, beta
  stored in bf16 (its generator at :178-300) - forward and backward against the oracle;
* tests/settings/product.csv (eight packed batches of 16384 tokens with production length mixes) and
  tests/settings/varlen.csv (B=11 x 33 tokens, B=7 x 4321 tokens, packed batches with random cuts) - forward.

Tolerances as everywhere: relative rms <= 5e-3, max |err| <= 2 % of max |ref|.  The gradient of the gates
is compared on the heads that have a gate (the reference masks the others, bench_precision_gdr.py:250-262).
"""
import pytest
import torch

from oracle import gdr_oracle as orc

pytestmark = pytest.mark.gpu
RMS, MAXR = 5e-3, 2e-2

# name, B, T, Hk, Hv, h0, gate_scale, swa_ratio, cu_seqlens
PRECISION_CASES = [
    ("short_tail", 1, 17, 16, 16, True, 1.0, 1.0, None),
    ("tail_gate_stress", 1, 48, 16, 16, True, 128.0, 1.0, None),
    ("one_chunk", 1, 64, 16, 16, True, 1.0, 1.0, None),
    ("tail_2chunk", 1, 96, 16, 16, True, 1.0, 1.0, None),
    ("gva_tail", 1, 96, 8, 16, True, 1.0, 1.0, None),
    ("batch2", 2, 128, 16, 16, True, 1.0, 1.0, None),
    ("varlen_mix", 1, 160, 16, 16, True, 1.0, 1.0, (0, 17, 96, 160)),
    ("multi_chunk", 1, 256, 16, 16, True, 1.0, 1.0, None),
    ("multi_chunk_gva", 1, 256, 8, 16, True, 1.0, 1.0, None),
    ("no_h0", 1, 128, 16, 16, False, 1.0, 1.0, None),
    ("swa_half", 1, 192, 16, 16, True, 1.0, 0.5, None),
    ("gate_stress", 1, 128, 16, 16, True, 16.0, 1.0, None),
]


def _precision_inputs(B, T, Hk, Hv, h0, gate_scale, swa_ratio, cu, seed=0):
    gen = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=gen)
    q, k = orc.l2norm(rn(B, T, Hk, 128)).bfloat16(), orc.l2norm(rn(B, T, Hk, 128)).bfloat16()
    v = rn(B, T, Hv, 128).bfloat16()
    g = torch.nn.functional.logsigmoid(rn(B, T, Hv)) * (gate_scale / 16.0)
    beta = torch.sigmoid(rn(B, T, Hv)).bfloat16()
    gated = torch.ones(Hv, dtype=torch.bool)
    if swa_ratio < 1.0:
        active = max(1, int(-(-swa_ratio * Hv // 1)))
        gated = torch.zeros(Hv, dtype=torch.bool)
        gated[torch.randperm(Hv, generator=gen)[:active]] = True
        g[:, :, ~gated] = 0.0
    n_states = B if cu is None else len(cu) - 1
    out = dict(q=q, k=k, v=v, g=g, beta=beta, do=rn(B, T, Hv, 128).bfloat16(), dht=rn(n_states, Hv, 128, 128) / 8.0)
    if h0:
        out["h0"] = rn(n_states, Hv, 128, 128)
    return out, gated


@pytest.mark.parametrize("case", PRECISION_CASES, ids=[c[0] for c in PRECISION_CASES])
def test_reference_precision_case(case):
    import flashqla_b200 as fq
    name, B, T, Hk, Hv, h0, gate_scale, swa_ratio, cu = case
    inp, gated = _precision_inputs(B, T, Hk, Hv, h0, gate_scale, swa_ratio, cu)
    c = {n: t.cuda() for n, t in inp.items()}
    cu_dev = None if cu is None else torch.tensor(cu, dtype=torch.int32, device="cuda")
    g_cs, A, o, h, fs, vn = fq.chunk_gated_delta_rule_fwd(c["q"], c["k"], c["v"], c["g"], c["beta"],
                                                          initial_state=c.get("h0"), cu_seqlens=cu_dev,
                                                          output_h=True, output_v_new=True)
    dq, dk, dv, db, dg, dh0 = fq.chunk_gated_delta_rule_bwd(c["q"], c["k"], c["v"], g_cs, c["beta"], A, c["do"],
                                                            dht=c["dht"], initial_state=c.get("h0"),
                                                            cu_seqlens=cu_dev, h=h, v_new=vn)
    fq.check_device_status()
    ref = orc.chunk_gdr_bwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"].float(), inp["do"], dht=inp["dht"],
                            h0=inp.get("h0"), cu_seqlens=cu)
    errs = []

    def close(label, got, want):
        e, m = orc.rel_rms(got.float().cpu(), want), orc.max_abs_ratio(got.float().cpu(), want)
        if not (e <= RMS and m <= MAXR):
            errs.append(f"{label}: rel_rms {e:.2e}, max ratio {m:.2e}")

    close("o", o, ref["o"])
    close("final_state", fs, ref["final_state"])
    for label, got in (("dq", dq), ("dk", dk), ("dv", dv), ("db", db)):
        close(label, got, ref[label])
    close("dg", dg[:, :, gated.cuda()], ref["dg"][:, :, gated])
    if h0:
        close("dh0", dh0, ref["dh0"])
    else:
        assert dh0 is None
    assert not errs, f"{name}: " + "; ".join(errs)


PRODUCT_CU = [
    "0-268-1139-1179-1212-1476-2792-3202-3611-3726-3820-4096-4882-6417-8130-8192-8328-9426-10473-11002-11754-12288-14085-15370-16384",
    "0-3393-4096-4153-5636-5853-6318-6777-8192-8320-8931-9163-9494-10040-10113-10363-10561-11061-11388-11634-12288-14545-16288-16384",
    "0-4096-6111-6485-6589-7118-8192-9056-10448-12288-14032-14525-15884-16012-16384",
    "0-177-4096-8192-12288-12805-13171-13298-16055-16384",
    "0-308-1128-1678-4096-4748-8192-8506-9657-10252-12113-12288-16384",
    "0-4096-6893-7665-8192-12288-16384",
    "0-410-841-1135-2126-2512-4096-4682-5022-5375-6259-6335-6580-6648-7308-8192-10450-12058-12288-14215-15280-15701-16384",
    "0-2048-4096-6144-8192-10240-12288-14336-16384",
]


def _forward_case(B, T, cu, seed, Hk=2, Hv=4):
    import flashqla_b200 as fq
    n_states = B if cu is None else len(cu) - 1
    # the reference's test distribution: gates / 16, a quarter of the heads without decay (tests/test_gdr.py:48-112)
    inp = orc.make_prefill_inputs(B, T, Hk, Hv, seed=seed, with_h0=True, n_states=n_states, gate_div=16.0,
                                  zero_gate_heads=0.25)
    c = {n: t.cuda() for n, t in inp.items()}
    cu_dev = None if cu is None else torch.tensor(cu, dtype=torch.int32, device="cuda")
    _, _, o, _, fs = fq.chunk_gated_delta_rule_fwd(c["q"], c["k"], c["v"], c["g"], c["beta"], initial_state=c["h0"],
                                                   cu_seqlens=cu_dev)
    fq.check_device_status()
    if cu is None:
        ref = orc.chunk_gdr_fwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], h0=inp["h0"])
    else:
        ref = orc.chunk_gdr_fwd_varlen(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], cu, h0=inp["h0"])
    for label, got, want in (("o", o, ref["o"]), ("final_state", fs, ref["final_state"])):
        e, m = orc.rel_rms(got.float().cpu(), want), orc.max_abs_ratio(got.float().cpu(), want)
        assert e <= RMS and m <= MAXR, f"{label}: rel_rms {e:.2e}, max ratio {m:.2e}"


@pytest.mark.parametrize("row", range(len(PRODUCT_CU)))
def test_production_length_mixes(row):
    cu = [int(x) for x in PRODUCT_CU[row].split("-")]
    _forward_case(1, cu[-1], cu, seed=100 + row)


@pytest.mark.parametrize("B,T,varlen", [(11, 33, False), (7, 4321, False), (3, 16789, True), (5, 8192, True),
                                        (10, 1024, True), (20, 512, True)])
def test_shape_suite(B, T, varlen):
    if not varlen:
        _forward_case(B, T, None, seed=B * 1000 + T)
        return
    # B sequences packed into T tokens at random cuts, every sequence non-empty (tests/test_gdr.py:114-121)
    gen = torch.Generator().manual_seed(B * 1000 + T)
    cuts = sorted((torch.randperm(T - 1, generator=gen)[:B - 1] + 1).tolist())
    _forward_case(1, T, [0] + cuts + [T], seed=B * 1000 + T)
