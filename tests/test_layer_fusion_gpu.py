"""GPU: the GDN layer's prologue and epilogue folded into the op.

* output gated RMS norm as an epilogue of the scan (``out_norm_gate`` / ``out_norm_weight``) against the same
  formula applied by torch to the plain op's output and against the fp64 oracle;
* the fused prologue (q / k L2 norm, gate activation, beta sigmoid inside the kernels) under autograd: every
  gradient, including those of ``A_log`` and ``dt_bias``, against torch autograd through the oracle's chunked
  forward on the same raw inputs.

Tolerances: relative rms 5e-3 and max |err| <= 2 % of max |ref| (gradients of the raw gate inputs: 1e-2,
they pass through two more activations).
"""
import pytest
import torch

from oracle import gdr_oracle as orc

pytestmark = pytest.mark.gpu


def _norm(o, z, w, eps):
    of = o.double()
    return of * torch.rsqrt(of.pow(2).mean(-1, keepdim=True) + eps) * w.double() * torch.nn.functional.silu(z.double())


@pytest.mark.parametrize("B,T,Hk,Hv,cu", [(2, 200, 1, 2, None), (1, 4096 + 17, 1, 2, None), (1, 500, 2, 4, (0, 130, 194, 500))])
def test_output_gated_rmsnorm_epilogue(B, T, Hk, Hv, cu):
    import flashqla_b200 as fq
    inp = orc.make_prefill_inputs(B, T, Hk, Hv, seed=61, with_h0=True, n_states=B if cu is None else len(cu) - 1)
    gen = torch.Generator().manual_seed(9)
    z = torch.randn(B, T, Hv, 128, generator=gen).bfloat16()
    weight = 1.0 + 0.2 * torch.randn(128, generator=gen)
    c = {n: t.cuda() for n, t in inp.items()}
    cu_dev = None if cu is None else torch.tensor(cu, dtype=torch.int32, device="cuda")
    o_plain = fq.chunk_gated_delta_rule_fwd(c["q"], c["k"], c["v"], c["g"], c["beta"], initial_state=c["h0"],
                                            cu_seqlens=cu_dev)[2]
    out = fq.chunk_gated_delta_rule_fwd(c["q"], c["k"], c["v"], c["g"], c["beta"], initial_state=c["h0"],
                                        cu_seqlens=cu_dev, out_norm_gate=z.cuda(), out_norm_weight=weight.cuda(),
                                        out_norm_eps=1e-6)
    fq.check_device_status()
    o_fused = out[2]
    # the same formula on the plain output (which is what the epilogue sees, rounded to 16 bits)
    want = _norm(o_plain.cpu(), z, weight, 1e-6)
    assert orc.rel_rms(o_fused.float().cpu(), want) <= 4e-3  # one more 16-bit rounding
    # and end to end against the oracle
    if cu is None:
        ref = orc.chunk_gdr_fwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], h0=inp["h0"], dtype=torch.float64)
    else:
        ref = orc.chunk_gdr_fwd_varlen(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], cu, h0=inp["h0"],
                                       dtype=torch.float64)
    assert orc.rel_rms(o_fused.float().cpu(), _norm(ref["o"], z, weight, 1e-6)) <= 7e-3
    # the public op takes the same switches (inference path: inside the kernel)
    o_pub, _ = fq.chunk_gated_delta_rule(c["q"], c["k"], c["v"], c["g"], c["beta"], initial_state=c["h0"],
                                         cu_seqlens=cu_dev, output_norm_gate=z.cuda(), output_norm_weight=weight.cuda())
    assert torch.equal(o_pub, o_fused)


def test_fused_prologue_under_autograd():
    import flashqla_b200 as fq
    B, T, Hk, Hv = 2, 330, 2, 4
    gen = torch.Generator().manual_seed(71)
    rn = lambda *s: torch.randn(*s, generator=gen)
    raw = dict(q=rn(B, T, Hk, 128).bfloat16(), k=rn(B, T, Hk, 128).bfloat16(), v=rn(B, T, Hv, 128).bfloat16(),
               a=rn(B, T, Hv), b=rn(B, T, Hv), A_log=-0.5 + torch.rand(Hv, generator=gen), dt_bias=0.3 * rn(Hv),
               h0=0.1 * rn(B, Hv, 128, 128))
    do, dht = rn(B, T, Hv, 128).bfloat16(), 0.1 * rn(B, Hv, 128, 128)

    # reference: torch autograd through the oracle on the same raw inputs (fp64)
    leaves = {n: t.detach().double().requires_grad_(True) for n, t in raw.items()}
    unit = lambda x: x * torch.rsqrt(x.pow(2).sum(-1, keepdim=True) + 1e-6)
    g = -torch.exp(leaves["A_log"]) * torch.nn.functional.softplus(leaves["a"] + leaves["dt_bias"])
    res = orc.chunk_gdr_fwd(unit(leaves["q"]), unit(leaves["k"]), leaves["v"], g, torch.sigmoid(leaves["b"]),
                            h0=leaves["h0"], dtype=torch.float64)
    loss = (res["o"] * do.double()).sum() + (res["final_state"] * dht.double()).sum()
    names = ("q", "k", "v", "a", "b", "A_log", "dt_bias", "h0")
    want = dict(zip(names, torch.autograd.grad(loss, [leaves[n] for n in names])))

    dev = {n: t.cuda().requires_grad_(True) for n, t in raw.items()}
    o, fs = fq.chunk_gated_delta_rule(dev["q"], dev["k"], dev["v"], dev["a"], dev["b"], initial_state=dev["h0"],
                                      output_final_state=True, use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True,
                                      A_log=dev["A_log"], dt_bias=dev["dt_bias"], use_beta_sigmoid_in_kernel=True)
    ((o.float() * do.cuda().float()).sum() + (fs * dht.cuda()).sum()).backward()
    fq.check_device_status()
    assert orc.rel_rms(o.float().cpu(), res["o"].detach()) <= 5e-3
    bad = []
    for n in names:
        got = dev[n].grad.float().cpu()
        rms, ratio = orc.rel_rms(got, want[n]), orc.max_abs_ratio(got, want[n])
        tol = 1e-2 if n in ("a", "A_log", "dt_bias") else 5e-3
        if not (rms <= tol and ratio <= 2e-2):
            bad.append(f"d{n}: rel_rms {rms:.2e}, max ratio {ratio:.2e}")
    assert not bad, "; ".join(bad)
