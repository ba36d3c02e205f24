"""Generate the golden fixtures in this directory from the reference's own CPU code.

Run once, where a checkout of the reference is at hand (the tests only need the stored fixtures):

    python tests/golden/make_golden.py /path/to/FlashQLA

It imports the reference's fp32 oracle ``tests/ref_gdr.py`` (forward + hand-written backward)
and the per-token CPU loop ``cpu_ref`` of ``tests/test_recurrent_verify_scratch_dtype.py``,
feeds them seeded inputs and stores inputs + outputs as ``*.pt``.  The committed fixtures pin
``oracle/gdr_oracle.py`` (see ``tests/test_oracle.py``).
"""
import importlib.util
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))
from oracle import gdr_oracle as orc  # noqa: E402


def chunk_case(ref, name, *, B, T, Hk, Hv, K, V, seed, dtype, with_h0, gate_div=1.0, zero_gate=0.0,
               bwd=False):
    inp = orc.make_prefill_inputs(B, T, Hk, Hv, K, V, seed=seed, dtype=dtype, with_h0=with_h0,
                                  gate_div=gate_div, zero_gate_heads=zero_gate, with_grads=bwd)
    f = {n: t.float() for n, t in inp.items()}
    scale = K ** -0.5
    g_cs, o, A, h, fs = ref.chunk_gated_delta_rule_fwd(
        f["q"], f["k"], f["v"], f["g"].clone(), f["beta"], initial_state=f.get("h0"), scale=scale)
    out = dict(inputs=inp, meta=dict(B=B, T=T, Hk=Hk, Hv=Hv, K=K, V=V, seed=seed, scale=scale),
               o=o, final_state=fs, g_cumsum=g_cs)
    if bwd:
        dq, dk, dv, db, dg, dh0 = ref.chunk_gated_delta_rule_bwd(
            f["q"], f["k"], f["v"], g_cs, f["beta"], A, scale, f.get("h0"), f["do"], f["dht"])
        out.update(dq=dq, dk=dk, dv=dv, db=db, dg=dg, dh0=dh0)
    torch.save(out, HERE / f"{name}.pt")
    print(name, {n: tuple(t.shape) for n, t in out.items() if torch.is_tensor(t)})


def recurrent_cases(ref_root: Path):
    spec = importlib.util.spec_from_file_location(
        "ref_recurrent_test", ref_root / "tests" / "test_recurrent_verify_scratch_dtype.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    q, k, v, a, b, A_log, dt_bias, h0 = mod.make_inputs(torch, "cpu")
    out = dict(inputs=dict(q=q, k=k, v=v, a=a, b=b, A_log=A_log, dt_bias=dt_bias, h0=h0),
               meta=dict(N=mod.N, T=mod.T, H=mod.H, HV=mod.HV, scale=mod.SCALE,
                         softplus_beta=mod.SP_BETA, softplus_threshold=mod.SP_THRESH), cases={})
    for kind in ("chain", "hop"):
        for dt in (torch.float32, torch.bfloat16):
            o_ref, inter_ref = mod.cpu_ref(torch, kind, dt)
            out["cases"][f"{kind}_{'f32' if dt == torch.float32 else 'bf16'}"] = dict(
                parents=mod.make_parents(torch, kind, "cpu"), o=o_ref,
                inter_last=inter_ref[:, -1].clone(), inter_rowsum=inter_ref.sum(-1))
    torch.save(out, HERE / "recurrent_verify.pt")
    print("recurrent_verify", list(out["cases"]))


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path of the reference checkout>")
    ref_root = Path(sys.argv[1])
    sys.path[:0] = [str(ref_root), str(ref_root / "tests")]
    import ref_gdr as ref

    # the reference's CPU-runnable case: naive-size fp32, K=V=64
    chunk_case(ref, "cfg0_fp32_k64", B=1, T=256, Hk=4, Hv=4, K=64, V=64, seed=0,
               dtype=torch.float32, with_h0=True)
    # K=V=128, GQA, ragged tail (T % 64 != 0), bf16 inputs, h0, gradients
    chunk_case(ref, "tail_gqa_bwd", B=1, T=150, Hk=1, Hv=2, K=128, V=128, seed=1,
               dtype=torch.bfloat16, with_h0=True, bwd=True)
    # the reference's own gate distribution (g/16, a zero-gate head), two sequences
    chunk_case(ref, "weak_gate_bwd", B=2, T=128, Hk=1, Hv=2, K=128, V=128, seed=2,
               dtype=torch.bfloat16, with_h0=True, gate_div=16.0, zero_gate=0.5, bwd=True)
    recurrent_cases(ref_root)


if __name__ == "__main__":
    main()
