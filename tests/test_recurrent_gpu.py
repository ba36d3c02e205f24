"""GPU parity of the recurrent op (decode / verify / tree verify / ragged) through the C-ABI,
against oracle/gdr_oracle.py and the golden vectors of the reference's CPU loop.

Tolerances: o max-abs <= 3e-3, state max-abs <= 1e-4, cached states <= 1e-4 (fp32 scratch) -
the reference's own gates, benchmark/bench_recurrent_fused_matrix.py:515-517.
"""
import pytest
import torch

from oracle import gdr_oracle as orc

pytestmark = pytest.mark.gpu

O_TOL, STATE_TOL = 3e-3, 1e-4


@pytest.fixture(scope="module")
def fq():
    import flashqla_b200
    assert torch.cuda.is_available()
    return flashqla_b200


def _inputs(N, T, Hk, Hv, seed, dtype=torch.bfloat16, slots=None):
    gen = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=gen)
    NT = N * T
    d = dict(
        q=orc.l2norm(rn(1, NT, Hk, 128)).to(dtype), k=orc.l2norm(rn(1, NT, Hk, 128)).to(dtype),
        v=rn(1, NT, Hv, 128).to(dtype),
        g=torch.nn.functional.logsigmoid(rn(1, NT, Hv)), beta=torch.sigmoid(rn(1, NT, Hv)),
        a=rn(1, NT, Hv).bfloat16(), b=rn(1, NT, Hv).bfloat16(),
        A_log=(-0.1 - torch.rand(Hv, generator=gen) * 0.5), dt_bias=(0.4 * rn(Hv)).bfloat16(),
        state=0.1 * rn(slots or N, Hv, 128, 128))
    return d


def _cuda(d):
    return {n: (t.cuda() if torch.is_tensor(t) else t) for n, t in d.items()}


@pytest.mark.parametrize("case", ["chain_f32", "chain_bf16", "hop_f32", "hop_bf16"])
def test_golden_verify_cases(fq, golden_dir, case):
    """Geometry, seed and expected values of tests/test_recurrent_verify_scratch_dtype.py."""
    fx = torch.load(golden_dir / "recurrent_verify.pt", weights_only=False)
    i, m, c = _cuda(fx["inputs"]), fx["meta"], fx["cases"][case]
    dt = torch.float32 if case.endswith("f32") else torch.bfloat16
    inter = torch.zeros(m["N"], m["T"], m["HV"], 128, 128, dtype=dt, device="cuda")
    state = i["h0"].clone()
    o = fq.fused_sigmoid_gating_delta_rule_update(
        i["A_log"], i["a"], i["dt_bias"], i["q"], i["k"], i["v"], i["b"], state, scale=m["scale"],
        use_qk_l2norm_in_kernel=True, disable_state_update=True, intermediate_states_buffer=inter,
        retrieve_parent_token=c["parents"].cuda(), block_dv=4)
    torch.cuda.synchronize()
    assert torch.equal(state, i["h0"]), "disable_state_update must leave the pool untouched"
    o = o.float().cpu().view(m["N"], m["T"], m["HV"], 128)
    assert orc.max_abs(o, c["o"]) <= O_TOL
    tol = STATE_TOL if dt == torch.float32 else 4e-3  # bf16 snapshots: one bf16 ulp of |S| <~ 1
    assert orc.max_abs(inter[:, -1].float().cpu(), c["inter_last"]) <= tol


def test_verify_invariants(fq, golden_dir):
    """Known-answer invariants of the reference test (:9-18): linear-verify o is bitwise equal
    across scratch dtypes; the bf16 scratch equals round_bf16(fp32 scratch); a chain-shaped
    tree equals the linear run bitwise."""
    fx = torch.load(golden_dir / "recurrent_verify.pt", weights_only=False)
    i, m = _cuda(fx["inputs"]), fx["meta"]
    chain = fx["cases"]["chain_f32"]["parents"].cuda()

    def run(dt, parents):
        inter = torch.zeros(m["N"], m["T"], m["HV"], 128, 128, dtype=dt, device="cuda")
        o = fq.fused_sigmoid_gating_delta_rule_update(
            i["A_log"], i["a"], i["dt_bias"], i["q"], i["k"], i["v"], i["b"], i["h0"].clone(),
            scale=m["scale"], disable_state_update=True, intermediate_states_buffer=inter,
            retrieve_parent_token=parents)
        return o, inter

    o32, i32 = run(torch.float32, None)
    o16, i16 = run(torch.bfloat16, None)
    ot, it = run(torch.float32, chain)
    assert torch.equal(o32, o16)
    assert torch.equal(i32.bfloat16(), i16)
    assert torch.equal(o32, ot) and torch.equal(i32, it)


@pytest.mark.parametrize("rows", [None, 16, 32])
@pytest.mark.parametrize("precomputed", [True, False])
def test_decode_matches_oracle(fq, rows, precomputed):
    N, Hk, Hv = 6, 2, 4
    d = _inputs(N, 1, Hk, Hv, seed=10)
    c = _cuda(d)
    state = c["state"].clone()
    kw = dict(block_dv=rows, assume_regular=True)
    if precomputed:
        o = fq.fused_sigmoid_gating_delta_rule_update(
            None, c["g"], None, c["q"], c["k"], c["v"], c["beta"], state,
            use_qk_l2norm_in_kernel=False, a_is_log_decay=True, b_is_beta=True, **kw)
        ref_state = d["state"].clone()
        o_ref = orc.recurrent_update_ref(None or torch.zeros(Hv), d["g"], torch.zeros(Hv), d["q"], d["k"],
                                         d["v"], d["beta"], ref_state, use_qk_l2norm=False,
                                         a_is_log_decay=True, b_is_beta=True)
    else:
        o = fq.fused_sigmoid_gating_delta_rule_update(
            c["A_log"], c["a"], c["dt_bias"], c["q"], c["k"], c["v"], c["b"], state, **kw)
        ref_state = d["state"].clone()
        o_ref = orc.recurrent_update_ref(d["A_log"], d["a"], d["dt_bias"], d["q"], d["k"], d["v"],
                                         d["b"], ref_state)
    assert orc.max_abs(o.float().cpu(), o_ref) <= O_TOL
    assert orc.max_abs(state.cpu(), ref_state) <= STATE_TOL


@pytest.mark.parametrize("mode", ["identity", "reverse", "negative_last"])
def test_state_index_modes(fq, mode):
    """Index modes of benchmark/bench_recurrent_fused_matrix.py:162-172; -1 = zero state, no write-back."""
    N, T, Hk, Hv, slots = 5, 3, 1, 2, 7
    d = _inputs(N, T, Hk, Hv, seed=11, slots=slots)
    idx = {"identity": torch.arange(N), "reverse": torch.arange(N).flip(0) + 2,
           "negative_last": torch.tensor([0, 1, 2, 3, -1])}[mode].int()
    c = _cuda(d)
    state = c["state"].clone()
    o = fq.fused_sigmoid_gating_delta_rule_update(
        c["A_log"], c["a"], c["dt_bias"], c["q"], c["k"], c["v"], c["b"], state,
        initial_state_indices=idx.cuda())
    ref_state = d["state"].clone()
    o_ref = orc.recurrent_update_ref(d["A_log"], d["a"], d["dt_bias"], d["q"], d["k"], d["v"], d["b"],
                                     ref_state, state_indices=idx)
    assert orc.max_abs(o.float().cpu(), o_ref) <= O_TOL
    assert orc.max_abs(state.cpu(), ref_state) <= STATE_TOL


@pytest.mark.parametrize("rows", [16, 32])
def test_more_items_than_resident_ctas(fq, rows):
    """Enough (sequence, head, row tile) items that every CTA walks several of them, so the staged copy of the
    next state tile alternates its buffers; shuffled pool slots with some sequences on the zero state (-1,
    nothing staged for them, no write-back)."""
    N, T, Hk, Hv, slots = 96, 2, 2, 8, 100
    d = _inputs(N, T, Hk, Hv, seed=21, slots=slots)
    gen = torch.Generator().manual_seed(5)
    idx = torch.randperm(slots, generator=gen)[:N].int()
    idx[::7] = -1
    c = _cuda(d)
    state = c["state"].clone()
    o = fq.fused_sigmoid_gating_delta_rule_update(
        c["A_log"], c["a"], c["dt_bias"], c["q"], c["k"], c["v"], c["b"], state,
        initial_state_indices=idx.cuda(), block_dv=rows)
    ref_state = d["state"].clone()
    o_ref = orc.recurrent_update_ref(d["A_log"], d["a"], d["dt_bias"], d["q"], d["k"], d["v"], d["b"],
                                     ref_state, state_indices=idx)
    assert orc.max_abs(o.float().cpu(), o_ref) <= O_TOL
    assert orc.max_abs(state.cpu(), ref_state) <= STATE_TOL


def test_ragged_cu_seqlens_and_tree(fq):
    lens = [3, 1, 5, 2]
    N, Hk, Hv = len(lens), 2, 4
    cu = torch.tensor([0, 3, 4, 9, 11], dtype=torch.int64)
    d = _inputs(1, 11, Hk, Hv, seed=12, slots=N)
    c = _cuda(d)
    parents = torch.tensor([[-1, 0, 0, 0, 0], [-1, 0, 0, 0, 0], [-1, 0, 1, 1, 2], [-1, 0, 0, 0, 0]]).int()
    inter = torch.zeros(N, 5, Hv, 128, 128, device="cuda")
    state = c["state"].clone()
    o = fq.fused_sigmoid_gating_delta_rule_update(
        c["A_log"], c["a"], c["dt_bias"], c["q"], c["k"], c["v"], c["b"], state, cu_seqlens=cu.cuda(),
        intermediate_states_buffer=inter, retrieve_parent_token=parents.cuda())
    ref_state, ref_inter = d["state"].clone(), torch.zeros(N, 5, Hv, 128, 128)
    o_ref = orc.recurrent_update_ref(d["A_log"], d["a"], d["dt_bias"], d["q"], d["k"], d["v"], d["b"],
                                     ref_state, cu_seqlens=cu, inter=ref_inter, parents=parents)
    assert orc.max_abs(o.float().cpu(), o_ref) <= O_TOL
    assert orc.max_abs(state.cpu(), ref_state) <= STATE_TOL
    assert orc.max_abs(inter.cpu(), ref_inter) <= STATE_TOL


def test_fp16_inputs_and_repeatability(fq):
    N, T, Hk, Hv = 4, 2, 2, 2
    d = _inputs(N, T, Hk, Hv, seed=13, dtype=torch.float16)
    c = _cuda(d)
    outs = []
    for _ in range(20):
        state = c["state"].clone()
        o = fq.fused_sigmoid_gating_delta_rule_update(
            c["A_log"], c["a"], c["dt_bias"], c["q"], c["k"], c["v"], c["b"], state)
        outs.append((o.clone(), state))
    for o, s in outs[1:]:
        assert torch.equal(o, outs[0][0]) and torch.equal(s, outs[0][1])
    ref_state = d["state"].clone()
    o_ref = orc.recurrent_update_ref(d["A_log"], d["a"], d["dt_bias"], d["q"], d["k"], d["v"], d["b"], ref_state)
    assert orc.max_abs(outs[0][0].float().cpu(), o_ref) <= O_TOL
    assert orc.max_abs(outs[0][1].cpu(), ref_state) <= STATE_TOL


def test_python_api_errors_on_gpu(fq):
    q = torch.zeros(1, 4, 2, 128, dtype=torch.bfloat16, device="cuda")
    v = torch.zeros(1, 4, 4, 128, dtype=torch.bfloat16, device="cuda")
    ab = torch.zeros(1, 4, 4, device="cuda")
    hv = torch.zeros(4, device="cuda")
    st = torch.zeros(4, 4, 128, 128, device="cuda")
    with pytest.raises(ValueError, match="contiguous"):
        fq.fused_sigmoid_gating_delta_rule_update(hv, ab, hv, q, q, v, ab, st.transpose(2, 3))
    with pytest.raises(ValueError, match="a shape"):
        fq.fused_sigmoid_gating_delta_rule_update(hv, ab[:, :2], hv, q, q, v, ab, st)
    with pytest.raises(ValueError, match="K=V=128"):
        fq.fused_sigmoid_gating_delta_rule_update(hv, ab, hv, q[..., :64], q[..., :64], v, ab, st)


@pytest.mark.parametrize("scratch_dtype", [torch.float32, torch.bfloat16])
def test_commit_verified_state(scratch_dtype):
    """Verify (T=4, cached, pool untouched) followed by the commit of the accepted prefix equals running the
    accepted tokens through the decode path: the pool ends up with the state after token num_accepted - 1."""
    import flashqla_b200 as fq
    from oracle import gdr_oracle as orc
    N, T, Hk, Hv = 5, 4, 2, 4
    gen = torch.Generator().manual_seed(61)
    rn = lambda *s: torch.randn(*s, generator=gen)
    q = orc.l2norm(rn(1, N * T, Hk, 128)).bfloat16().cuda()
    k = orc.l2norm(rn(1, N * T, Hk, 128)).bfloat16().cuda()
    v = rn(1, N * T, Hv, 128).bfloat16().cuda()
    g = torch.nn.functional.logsigmoid(rn(1, N * T, Hv)).cuda()
    beta = torch.sigmoid(rn(1, N * T, Hv)).cuda()
    pool = (0.1 * rn(8, Hv, 128, 128)).cuda()
    slots = torch.tensor([6, 0, 3, 7, 2], dtype=torch.int32, device="cuda")
    inter = torch.zeros(N, T, Hv, 128, 128, dtype=scratch_dtype, device="cuda")
    before = pool.clone()
    fq.fused_sigmoid_gating_delta_rule_update(None, g, None, q, k, v, beta, pool, initial_state_indices=slots,
                                              use_qk_l2norm_in_kernel=False, a_is_log_decay=True, b_is_beta=True,
                                              assume_regular=True, disable_state_update=True,
                                              intermediate_states_buffer=inter)
    assert torch.equal(pool, before)
    accepted = torch.tensor([4, 0, 1, 3, 2], dtype=torch.int32, device="cuda")
    fq.commit_verified_state(pool, inter, accepted, initial_state_indices=slots)
    fq.check_device_status()
    for n in range(N):
        s, a = int(slots[n]), int(accepted[n])
        want = before[s] if a == 0 else inter[n, a - 1].float()
        assert torch.equal(pool[s], want), f"sequence {n}"
    untouched = [i for i in range(8) if i not in slots.tolist()]
    assert torch.equal(pool[untouched], before[untouched])
    # out-of-range slot: reported through the status word, nothing written
    bad = torch.tensor([99, 0, 3, 7, 2], dtype=torch.int32, device="cuda")
    fq.commit_verified_state(pool, inter, accepted, initial_state_indices=bad)
    with pytest.raises(Exception):
        fq.check_device_status()


@pytest.mark.parametrize("pool_dtype", [torch.float32, torch.bfloat16])
def test_prefill_then_decode_through_the_pool(fq, pool_dtype):
    """Prefill writes the final states into pool slots (one sequence without a slot), a second prefill call
    continues from the pool, then the recurrent op decodes one more token from the same slots: o of that token
    and the pool must be those of the per-token recurrence over all tokens.  The kernels index the slots
    themselves; the pool is fp32 or bf16 (then every hand-over rounds the state to 16 bits)."""
    N, Hk, Hv, T1, T2, slots = 3, 2, 4, 128, 64, 6
    inp = orc.make_prefill_inputs(N, T1 + T2 + 1, Hk, Hv, seed=51)
    c = {n: t.cuda() for n, t in inp.items()}
    idx = torch.tensor([4, -1, 1], dtype=torch.int32)
    pool = torch.full((slots, Hv, 128, 128), 7.0, device="cuda", dtype=pool_dtype)
    tol = 5e-3 if pool_dtype == torch.float32 else 1e-2
    part = lambda a, b: [c[n][:, a:b].contiguous() for n in ("q", "k", "v", "g", "beta")]
    o1, _ = fq.prefill_into_state_pool(*part(0, T1), pool, idx.cuda())
    o2, _ = fq.prefill_into_state_pool(*part(T1, T1 + T2), pool, idx.cuda(), continue_from_pool=True)
    assert float((pool[[0, 2, 3, 5]].float() - 7.0).abs().max()) == 0.0  # untouched slots
    # one decode token per sequence from the pool (packed [1, N, ...] layout of the recurrent op)
    t = T1 + T2
    tok = lambda n: c[n][:, t].unsqueeze(0).contiguous()
    o3 = fq.fused_sigmoid_gating_delta_rule_update(
        None, tok("g"), None, tok("q"), tok("k"), tok("v"), tok("beta"), pool, initial_state_indices=idx.cuda(),
        use_qk_l2norm_in_kernel=False, a_is_log_decay=True, b_is_beta=True, assume_regular=True)
    ref = orc.naive_recurrent_gdr(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], dtype=torch.float64)
    o_ref, s_ref = ref[0], ref[1]
    keep = [0, 2]  # sequence 1 has no slot: its second prefill and its decode start from zero
    assert orc.rel_rms(o1.float().cpu(), o_ref[:, :T1]) <= 5e-3
    assert orc.rel_rms(o2.float().cpu()[keep], o_ref[keep, T1:t]) <= tol
    assert orc.rel_rms(o3.float().cpu()[0, keep], o_ref[keep, t]) <= tol
    # pool layout is [V, K]; the oracle's state is [K, V]
    assert orc.rel_rms(pool[[4, 1]].float().cpu(), s_ref[keep].transpose(-1, -2).float()) <= tol


def test_pool_prefill_with_context_parallel_segments(fq):
    """The same slot-indexed prefill when the planner cuts the sequences into segments: the start states come
    out of the pool inside the plan kernel ([V, K] slots into the [K, V] segment states), the last segment of
    every sequence writes its slot."""
    lens = [4096 + 37, 2048]
    cu = torch.tensor([0, lens[0], lens[0] + lens[1]], dtype=torch.int32)
    inp = orc.make_prefill_inputs(1, sum(lens), 1, 2, seed=52, with_h0=True, n_states=2)
    c = {n: t.cuda() for n, t in inp.items()}
    idx = torch.tensor([3, 0], dtype=torch.int32, device="cuda")
    pool = torch.zeros(5, 2, 128, 128, device="cuda")
    pool[3], pool[0] = c["h0"][0].transpose(-1, -2), c["h0"][1].transpose(-1, -2)
    from flashqla_b200 import cp
    assert cp.get_plan(lens, 2, torch.device("cuda", 0)).use_cp
    o, _ = fq.prefill_into_state_pool(c["q"], c["k"], c["v"], c["g"], c["beta"], pool, idx, cu_seqlens=cu.cuda(),
                                      continue_from_pool=True)
    fq.check_device_status()
    ref = orc.chunk_gdr_fwd_varlen(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], cu, h0=inp["h0"])
    assert orc.rel_rms(o.float().cpu(), ref["o"]) <= 5e-3
    assert orc.rel_rms(pool[[3, 0]].cpu(), ref["final_state"].transpose(-1, -2)) <= 5e-3
    assert float(pool[[1, 2, 4]].abs().max()) == 0.0


def test_decode_step_in_a_cuda_graph(fq):
    """A decode step captured in a CUDA graph (how serving loops launch it; the reference skips its autotune
    under capture, recurrent_fused.py:234) replays with the same result as a plain call."""
    N, Hk, Hv = 8, 2, 4
    d = _inputs(N, 1, Hk, Hv, seed=61)
    c = _cuda(d)
    kw = dict(use_qk_l2norm_in_kernel=True)
    ref_state = c["state"].clone()
    o_ref = fq.fused_sigmoid_gating_delta_rule_update(c["A_log"], c["a"], c["dt_bias"], c["q"], c["k"], c["v"],
                                                      c["b"], ref_state, **kw)
    state = c["state"].clone()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            o = fq.fused_sigmoid_gating_delta_rule_update(c["A_log"], c["a"], c["dt_bias"], c["q"], c["k"], c["v"],
                                                          c["b"], state, **kw)
    torch.cuda.current_stream().wait_stream(side)
    state.copy_(c["state"])  # capture does not run the kernel; replay on the initial pool
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(o, o_ref) and torch.equal(state, ref_state)


def _reference_recurrent():
    """The reference's own recurrent op (TileLang kernels, compiled on this box), loaded by path from the copy
    that oracle/build_ref.py places under oracle/_ref/ (the way the reference's own test loads it,
    tests/test_recurrent_verify_scratch_dtype.py:93-107).  None when the file or TileLang is missing."""
    import importlib.util
    import os
    import sys
    from pathlib import Path
    src = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "recurrent_fused.py"
    if not src.exists():
        return None
    if "reference_recurrent_fused" in sys.modules:
        return sys.modules["reference_recurrent_fused"]
    try:
        import tilelang  # noqa: F401
    except Exception:
        return None
    os.environ.setdefault("TILELANG_CACHE_DIR", "/tmp/flashqla_b200_tilelang_cache")
    spec = importlib.util.spec_from_file_location("reference_recurrent_fused", src)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["reference_recurrent_fused"] = mod
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("mode", ["decode_plain", "decode_gated_l2norm", "verify_f32", "verify_bf16"])
def test_against_the_reference_kernel_on_this_gpu(fq, mode):
    """Same inputs through the reference's TileLang kernel and through this library: outputs, updated pool and
    cached per-token states, with the gates of the reference's own comparison
    (benchmark/bench_recurrent_fused_matrix.py:515-517).  Skips where the reference file is absent or its kernel
    does not compile for this GPU."""
    rec = _reference_recurrent()
    if rec is None:
        pytest.skip("reference recurrent op not available (oracle/_ref/recurrent_fused.py or TileLang missing)")
    verify = mode.startswith("verify")
    N, T, Hk, Hv = 48, (4 if verify else 1), 4, 8
    c = _cuda(_inputs(N, T, Hk, Hv, seed=71))
    # the reference's verify kernel applies the layer's gate activation whatever a_is_log_decay / b_is_beta say, so
    # the verify cases use raw gate inputs (as the reference's own verify test does)
    gated = mode != "decode_plain"
    kw = dict(use_qk_l2norm_in_kernel=gated, a_is_log_decay=not gated, b_is_beta=not gated, assume_regular=True)
    a_in, b_in = (c["a"], c["b"]) if gated else (c["g"], c["beta"])
    A_log = c["A_log"].float()
    dt_bias = c["dt_bias"]
    inter_dt = torch.bfloat16 if mode == "verify_bf16" else torch.float32
    outs = []
    for impl in ("reference", "ours"):
        pool = c["state"].clone()
        inter = torch.zeros(N, T, Hv, 128, 128, dtype=inter_dt, device="cuda") if verify else None
        fn = rec.fused_sigmoid_gating_delta_rule_update if impl == "reference" else fq.fused_sigmoid_gating_delta_rule_update
        try:
            o = fn(A_log, a_in, dt_bias, c["q"], c["k"], c["v"], b_in, pool, disable_state_update=verify,
                   intermediate_states_buffer=inter, **kw)
            torch.cuda.synchronize()
        except Exception as exc:  # the reference's JIT may not support this GPU or toolchain
            if impl == "reference":
                pytest.skip(f"reference kernel did not run here: {type(exc).__name__}: {str(exc)[:120]}")
            raise
        outs.append((o.float(), pool, inter))
    fq.check_device_status()
    (o_r, pool_r, inter_r), (o_m, pool_m, inter_m) = outs
    assert float((o_r - o_m).abs().max()) <= O_TOL
    assert float((pool_r - pool_m).abs().max()) <= STATE_TOL
    if verify:
        assert torch.equal(pool_m, c["state"]) and torch.equal(pool_r, c["state"])
        tol = STATE_TOL if inter_dt == torch.float32 else 8e-3  # two bf16 roundings of |S| ~ 1
        assert float((inter_r.float() - inter_m.float()).abs().max()) <= tol
