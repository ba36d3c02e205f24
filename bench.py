#!/usr/bin/env python
"""Benchmark of the GDN hot path on B200.  One JSON line on stdout (rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload = the configuration the headline metric is quoted on: chunked prefill forward,
B=1, T=32768, Hk=16, Hv=32, K=V=128, bf16 q/k/v, fp32 g/beta, zero initial state, final state
written.  With N > 1 (one process per GPU under torch.distributed.run) the v-heads (and their k-heads)
are split across ranks - no collective on the data path; the timed region is bracketed by a barrier and
the reported time is the max over ranks.

Other workloads (own measurements, same JSON shape): ``decode`` and ``verify`` (256 sequences, Hk=16,
Hv=32; HBM-bound, metric GB/s), ``varlen`` (64 packed sequences, Hk=Hv=8).

``--impl reference`` times the CPU restatement of the reference algorithm (oracle/gdr_oracle.py, all host
threads) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

K = V = 128
MEASURED_SCAN_DRAM_BYTES_PER_TOKEN_HK16_HV32 = 39648.0
CHUNK = 64


def peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        p = json.loads(f.read_text())
        return dict(hbm=p["hbm_gbs"], tf_burst=p["bf16_tflops"], tf_sus=p["bf16_tflops_sustained"], src="measured")
    return dict(hbm=6650.0, tf_burst=1590.0, tf_sus=1400.0, src="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index: int, period: float = 0.05):
        self.index, self.period = index, period
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None

    def __enter__(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None
            return self
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def _run(self):
        nv = self._nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        s = sorted(self.samples)
        med = s[len(s) // 2] if s else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(s)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


L2_BYTES = 126 * 2 ** 20


def timed(fn, steps, warmup, world, device, flush_l2=False):
    """W untimed steps, then exactly K steps between CUDA events on the current stream; barrier +
    synchronize on both sides; max over ranks.  With ``flush_l2`` (working sets that would fit the L2) a
    buffer of twice the L2 size is overwritten before every step and each step has its own event pair, so
    the flush is outside what is timed."""
    import torch.distributed as dist
    flush = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=device) if flush_l2 else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    if flush is None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize(device)
        ms = e0.elapsed_time(e1)
    else:
        pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        for a, b in pairs:
            flush.zero_()
            a.record()
            fn()
            b.record()
        torch.cuda.synchronize(device)
        ms = sum(a.elapsed_time(b) for a, b in pairs)
    if world > 1:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
        ms = float(t.item())
    return ms


MIN_TIMED_SECONDS = 1.0
MAX_BLOCKS = 400


def measure(fn, steps, warmup, world, device, flush_l2=False, min_seconds=None):
    """Median over repeated blocks of exactly K timed steps (``timed``): the block is repeated until the timed
    regions add up to at least ``MIN_TIMED_SECONDS`` (at most ``MAX_BLOCKS`` blocks), so that clocks and power
    have settled and the clock sampler sees the region.  Every rank runs the same number of blocks (the count
    comes from the first block's max-over-ranks time).  Returns (ms of the median block, number of blocks)."""
    min_seconds = MIN_TIMED_SECONDS if min_seconds is None else min_seconds
    first = timed(fn, steps, warmup, world, device, flush_l2=flush_l2)
    blocks = int(min(MAX_BLOCKS, max(1, -(-min_seconds * 1e3 // max(first, 1e-6)))))
    times = [first] + [timed(fn, steps, 0, world, device, flush_l2=flush_l2) for _ in range(blocks - 1)]
    times.sort()
    return times[len(times) // 2], len(times)


# ------------------------------------------------------------------------------------ workloads
def SCAN_DRAM_BYTES_PER_TOKEN_HEADS(Hk, Hv):
    """DRAM bytes per token moved by one launch of the chunk scan: dram__bytes_read + dram__bytes_write of an
    ncu capture of this kernel on a smaller case (8192 tokens, 16 k-heads / 32 v-heads: 324.8 MB = 39.6 KB
    per token), scaled by the head counts of this rank."""
    # the scan reads q, k per k-head (512 B) and v, w, A, gates per v-head and writes o (904 B)
    return MEASURED_SCAN_DRAM_BYTES_PER_TOKEN_HK16_HV32 * (Hk * 512 + Hv * 904) / (16 * 512 + 32 * 904)


def prefill_inputs(T, Hk, Hv, seed, n_seqs=1, with_h0=False):
    from oracle import gdr_oracle as orc
    return orc.make_prefill_inputs(1, T, Hk, Hv, seed=seed, with_h0=with_h0, n_states=n_seqs)


def run_prefill(args, rank, world, device, varlen=False):
    import flashqla_b200 as fq
    from flashqla_b200 import _cabi
    from oracle import gdr_oracle as orc
    if varlen:
        gen = torch.Generator().manual_seed(2)
        lens = torch.randint(512, 16385, (64,), generator=gen).tolist()
        # token-balanced longest-first assignment of sequences to ranks
        from flashqla_b200.sharding import balance_sequences
        mine = balance_sequences(lens, world)[rank]
        my_lens = [lens[i] for i in mine]
        Hk = Hv = 8
        T = sum(my_lens)
        total_tokens = sum(lens)
        cu = torch.tensor([0] + list(torch.tensor(my_lens).cumsum(0)), dtype=torch.int32)
        inp = prefill_inputs(T, Hk, Hv, seed=20 + rank, n_seqs=len(my_lens), with_h0=True)
        workload = "varlen_prefill_fwd_64seq_U512-16384_Hk8_Hv8"
        n_states_in = len(my_lens)
    else:
        T, Hk_all, Hv_all = args.tokens, 16, 32
        assert Hv_all % world == 0 and Hk_all % world == 0
        Hk, Hv = Hk_all // world, Hv_all // world
        total_tokens = T
        cu = None
        inp = prefill_inputs(T, Hk, Hv, seed=1 + rank)
        workload = f"prefill_fwd_B1_T{T}_Hk{Hk_all}_Hv{Hv_all}_K128_V128_chunk64"
        n_states_in = 0
    host = {n: t.pin_memory() for n, t in inp.items()}
    dev = {n: t.to(device, non_blocking=True) for n, t in host.items()}
    cu_dev = cu.to(device) if cu is not None else None
    h0 = dev.get("h0")
    torch.cuda.synchronize(device)

    def eager_step():
        return fq.chunk_gated_delta_rule_fwd(dev["q"], dev["k"], dev["v"], dev["g"], dev["beta"],
                                             initial_state=h0, cu_seqlens=cu_dev, output_final_state=True)

    # The timed step replays a CUDA graph of the same public call on the same buffers (what a serving loop
    # with static buffers does): after sharding over several GPUs the host would otherwise need longer to
    # issue the nine launches of a call than a GPU needs to run them.  --eager times the plain call.
    step, launch_mode = eager_step, "eager"
    if not args.eager:
        try:
            step = fq.GraphedForward(dev["q"], dev["k"], dev["v"], dev["g"], dev["beta"], initial_state=h0,
                                     cu_seqlens=cu_dev, output_final_state=True)
            launch_mode = "cuda_graph"
        except Exception as exc:  # capture is an optimisation, never a requirement
            launch_mode = f"eager (graph capture failed: {type(exc).__name__})"

    from flashqla_b200 import cp as _cp
    plan_lens = my_lens if varlen else [T]
    use_cp = _cp.get_plan(plan_lens, Hv, device).use_cp
    launches_per_step = fq.chunk.launches_per_forward(varlen=cu is not None, use_cp=use_cp)
    in_bytes = sum(t.numel() * t.element_size() for t in dev.values())
    flush_l2 = in_bytes < 2 * L2_BYTES  # head shards of 4 and 8 GPUs: the inputs of a rank would fit the L2
    with ClockSampler(torch.cuda.current_device() if device.index is None else device.index) as cs:
        ms, blocks = measure(step, args.steps, args.warmup, world, device, flush_l2=flush_l2)
    fq.check_device_status()

    # ---- dominant kernel alone (the chunk scan), for the roofline entry
    g_cs, A, o, _, fs = step()
    scan_only = fq.chunk.make_scan_only(dev["q"], dev["k"], dev["v"], dev["beta"], g_cs, A, o, fs,
                                        initial_state=h0, cu_seqlens=cu_dev)
    ms_scan = measure(scan_only, args.steps, args.warmup, world, device, flush_l2=flush_l2, min_seconds=0.2)[0] / args.steps

    # ---- end to end through the public API with host buffers
    o_host = torch.empty(o.shape, dtype=o.dtype).pin_memory()
    fs_host = torch.empty(fs.shape, dtype=fs.dtype).pin_memory()
    h2d = sum(host[n].numel() * host[n].element_size() for n in host)
    d2h = o_host.numel() * o_host.element_size() + fs_host.numel() * fs_host.element_size()

    def e2e_step():
        if not varlen:
            # one sequence in pinned host memory: copies and compute overlap piece by piece
            fq.chunk_gated_delta_rule_fwd_host(host["q"], host["k"], host["v"], host["g"], host["beta"],
                                               out=o_host, final_state_out=fs_host, device=device)
            return
        d = {n: t.to(device, non_blocking=True) for n, t in host.items()}
        _, _, oo, _, ff = fq.chunk_gated_delta_rule_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"],
                                                        initial_state=d.get("h0"), cu_seqlens=cu_dev,
                                                        output_final_state=True)
        o_host.copy_(oo, non_blocking=True)
        fs_host.copy_(ff, non_blocking=True)

    e2e_steps = max(2, min(args.steps, 10))
    ms_e2e = timed(e2e_step, e2e_steps, 2, world, device)
    fq.check_device_status()

    # ---- optional same-box bar: FLA's Triton kernels (the reference's own comparison baseline) on these inputs
    same_box = None
    if args.compare_fla:
        try:
            from fla.ops.gated_delta_rule import chunk_gated_delta_rule as fla_gdr
            cu64 = None if cu_dev is None else cu_dev.long()
            fla_step = lambda: fla_gdr(dev["q"], dev["k"], dev["v"], dev["g"], dev["beta"], scale=K ** -0.5,
                                       initial_state=h0, output_final_state=True, cu_seqlens=cu64)
            ms_fla = timed(fla_step, args.steps, args.warmup, world, device) / args.steps
            same_box = {"impl": "fla %s (Triton)" % __import__("fla").__version__, "ms_per_step": ms_fla,
                        "tokens_per_s": total_tokens / (ms_fla * 1e-3)}
        except Exception as exc:
            same_box = {"impl": "fla", "unavailable": f"{type(exc).__name__}: {str(exc)[:120]}"}

    pk = peaks()
    per_step = ms / args.steps
    value = total_tokens / (per_step * 1e-3)
    tok_heads_rank = T * Hv
    scan_flops = tok_heads_rank * (6 * CHUNK * K + 6 * K * V)  # QK^T, A W, Pg Vd + K S, Q S, K^T V'
    achieved = scan_flops / (ms_scan * 1e-3) / 1e12
    algo_bytes = orc.prefill_bytes(T, Hk, Hv, n_states_in, n_states_in if varlen else 1)
    gbs_scan = algo_bytes / (ms_scan * 1e-3) / 1e9
    line = {
        "metric": "gdn_prefill_fwd_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "blocks": blocks,
        "config": {"workload": workload, "sharding": f"v-heads/{world}" if not varlen else f"sequences/{world}",
                   "context_parallel": use_cp, "launch": launch_mode,
                   "l2": (f"inputs of a rank ({in_bytes / 1e6:.0f} MB) exceed the 126 MB L2; no flush needed" if not flush_l2
                          else f"inputs of a rank are {in_bytes / 1e6:.0f} MB: a 252 MB buffer is overwritten before "
                               "every timed step (per-step events, the flush is not timed)"),
                   "tokens": total_tokens},
        "clocks": cs.summary(),
        "e2e": {"value": total_tokens / (ms_e2e / e2e_steps * 1e-3), "unit": "tokens/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e / e2e_steps},
        "gpu_launches": launches_per_step * args.steps * blocks,
        # The chunk scan is the dominant kernel.  Its intensity (163 840 flop and 24 832 B per token at this
        # shape) is below the B200 ridge, so HBM is the binding roof; the tensor figures are given beside it.
        # traffic: DRAM bytes of one launch from an ncu capture (bytes per token measured on a smaller case
        # of the same kernel, times the tokens of this launch): above the algorithmic bytes by design,
        # because the prepared operands A and w make a round trip through HBM.
        "roofline": {"kernel": "chunk_fwd_kernel", "bound": "hbm", "achieved": gbs_scan, "peak": pk["hbm"],
                     "unit": "GB/s", "frac": gbs_scan / pk["hbm"], "peak_source": pk["src"],
                     "ms_per_launch": ms_scan,
                     # the same algorithmic bytes over the WHOLE call (preparation + context-parallel passes + scan)
                     "whole_call_frac": algo_bytes / (per_step * 1e-3) / 1e9 / pk["hbm"],
                     "traffic": None if varlen else SCAN_DRAM_BYTES_PER_TOKEN_HEADS(Hk, Hv) * T,
                     "tensor_achieved_tflops": achieved, "tensor_peak_tflops": pk["tf_burst"],
                     "tensor_frac": achieved / pk["tf_burst"]},
    }
    if same_box is not None:
        line["same_box"] = same_box
    return line


def run_prefill_sp(args, rank, world, device):
    """Config 1 with the TOKENS of the one sequence spread over the ranks (all heads on every rank) and the
    chunk-boundary states carried by one all-gather per call: the optional sequence-parallel mode.  The
    default multi-GPU prefill line shards heads instead, which needs no exchange."""
    import flashqla_b200 as fq
    Hk, Hv, T = 16, 32, args.tokens
    per = (T // world // 64) * 64
    lo = rank * per
    hi = T if rank == world - 1 else lo + per
    inp = prefill_inputs(T, Hk, Hv, seed=1)
    c = {n: t[:, lo:hi].contiguous().to(device) for n, t in inp.items()}

    def step():
        fq.chunk_gated_delta_rule_fwd_sp(c["q"], c["k"], c["v"], c["g"], c["beta"])

    with ClockSampler(device.index) as clocks:
        ms, blocks = measure(step, args.steps, args.warmup, world, device)
    ms_step = ms / args.steps
    tps = T / (ms_step * 1e-3)
    return {
        "metric": "gdn_prefill_fwd_tokens_per_s", "value": tps, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "blocks": blocks,
        "config": {"workload": f"prefill_fwd_B1_T{T}_Hk16_Hv32_K128_V128_chunk64", "sharding": f"tokens/{world}",
                   "exchange": f"one all_gather of {2 * Hv * 65536} B per rank", "launch": "eager",
                   "l2": "inputs exceed the 126 MB L2; no flush needed", "tokens": T},
        "clocks": clocks.summary(), "gpu_launches": args.steps * 7 * blocks}


def run_recurrent(args, rank, world, device, verify: bool):
    import flashqla_b200 as fq
    from oracle import gdr_oracle as orc
    N_all, Hk, Hv = 256, 16, 32
    assert N_all % world == 0
    N = N_all // world
    T = 4 if verify else 1
    gen = torch.Generator().manual_seed(4 + rank)
    rn = lambda *s: torch.randn(*s, generator=gen)
    q = orc.l2norm(rn(1, N * T, Hk, K)).bfloat16().to(device)
    k = orc.l2norm(rn(1, N * T, Hk, K)).bfloat16().to(device)
    v = rn(1, N * T, Hv, V).bfloat16().to(device)
    g = torch.nn.functional.logsigmoid(rn(1, N * T, Hv)).to(device)
    beta = torch.sigmoid(rn(1, N * T, Hv)).to(device)
    state = (0.1 * rn(N, Hv, V, K)).to(device)
    inter = torch.empty(N, T, Hv, V, K, dtype=torch.float32 if not args.bf16_scratch else torch.bfloat16,
                        device=device) if verify else None

    # The pool of one rank shrinks with the number of ranks (67 MB at 8 GPUs): steps then rotate over enough
    # copies of it that a pool is out of the 126 MB L2 again before its next use.
    copies = max(1, -(-512 * 2 ** 20 // (state.numel() * 4)))
    pools = [state] + [state.clone() for _ in range(copies - 1)]
    calls = [0]

    def step():
        calls[0] += 1
        return fq.fused_sigmoid_gating_delta_rule_update(
            None, g, None, q, k, v, beta, pools[calls[0] % copies], use_qk_l2norm_in_kernel=False,
            a_is_log_decay=True, b_is_beta=True, assume_regular=True, disable_state_update=verify,
            intermediate_states_buffer=inter, block_dv=args.block_dv)

    with ClockSampler(device.index or 0) as cs:
        ms, blocks = measure(step, args.steps, args.warmup, world, device)
    per_step = ms / args.steps
    same_box = []
    if args.compare_fla and not verify:
        # same-box bar: FLA's Triton recurrent kernel on the same inputs (what the reference compares its decode
        # kernels with); it returns the new states instead of updating the pool in place
        try:
            from fla.ops.gated_delta_rule import fused_recurrent_gated_delta_rule as fla_update
            cu_fla = torch.arange(N + 1, device=device, dtype=torch.long)
            fla_step = lambda: fla_update(q, k, v, g=g, beta=beta, scale=K ** -0.5, initial_state=pools[0],
                                          output_final_state=True, use_qk_l2norm_in_kernel=False, cu_seqlens=cu_fla,
                                          transpose_state_layout=True)
            ms_fla = measure(fla_step, args.steps, args.warmup, world, device, min_seconds=0.3)[0] / args.steps
            same_box.append({"impl": "fla %s fused_recurrent_gated_delta_rule (Triton)" % __import__("fla").__version__,
                             "ms_per_step": ms_fla})
        except Exception as exc:
            same_box.append({"impl": "fla fused_recurrent_gated_delta_rule",
                             "unavailable": f"{type(exc).__name__}: {str(exc)[:160]}"})
    if args.compare_fla:
        # same-box bar: the reference's own recurrent op (TileLang kernels compiled on this box), loaded by path
        # from the copy that oracle/build_ref.py places beside the oracle; same inputs, same pool rotation
        ref_file = ROOT / "oracle" / "_ref" / "recurrent_fused.py"
        if ref_file.exists():
            import contextlib
            import importlib.util
            import logging
            # TileLang logs its compilations to stdout, which carries this program's one JSON line: its loggers are
            # created (and anything it prints is sent) with stdout pointing at stderr
            redirect = contextlib.ExitStack()
            try:
                os.environ.setdefault("TILELANG_CACHE_DIR", "/tmp/flashqla_b200_tilelang_cache")
                redirect.enter_context(contextlib.redirect_stdout(sys.stderr))
                spec = importlib.util.spec_from_file_location("reference_recurrent_fused", ref_file)
                rec = importlib.util.module_from_spec(spec)
                sys.modules["reference_recurrent_fused"] = rec
                spec.loader.exec_module(rec)
                for name in list(logging.root.manager.loggerDict):
                    if name.lower().startswith("tilelang"):
                        logging.getLogger(name).setLevel(logging.ERROR)
                zeros_h = torch.zeros(Hv, dtype=torch.float32, device=device)  # A_log / dt_bias: unused with log decays
                rcalls = [0]

                # (its verify kernel applies the layer's gate activation whatever a_is_log_decay / b_is_beta say:
                # the arithmetic of that step differs a little, the memory traffic does not)
                def ref_step():
                    rcalls[0] += 1
                    return rec.fused_sigmoid_gating_delta_rule_update(
                        zeros_h, g, zeros_h, q, k, v, beta, pools[rcalls[0] % copies], use_qk_l2norm_in_kernel=False,
                        a_is_log_decay=True, b_is_beta=True, assume_regular=True, disable_state_update=verify,
                        intermediate_states_buffer=inter)
                ms_ref = measure(ref_step, args.steps, args.warmup, world, device, min_seconds=0.3)[0] / args.steps
                same_box.append({"impl": "reference flash_qla recurrent_fused.py (TileLang %s, compiled here)"
                                         % __import__("tilelang").__version__, "ms_per_step": ms_ref})
            except Exception as exc:
                same_box.append({"impl": "reference flash_qla recurrent_fused.py (TileLang)",
                                 "unavailable": f"{type(exc).__name__}: {str(exc)[:160]}"})
            finally:
                redirect.close()
    cache_b = 0 if not verify else (2 if args.bf16_scratch else 4)
    nbytes = orc.state_bytes_decode(N, Hv, T=T, Hk=Hk, cache_bytes=cache_b, write_back=not verify)
    gbs = nbytes * world / (per_step * 1e-3) / 1e9
    pk = peaks()
    for bar in same_box:
        if "ms_per_step" in bar:
            bar["gb_per_s"] = nbytes * world / (bar["ms_per_step"] * 1e-3) / 1e9
    return {
        **({"same_box": same_box} if same_box else {}),
        "metric": "gdn_%s_hbm_gb_per_s" % ("verify" if verify else "decode"), "value": gbs, "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "blocks": blocks,
        "config": {"workload": f"{'verify_T4' if verify else 'decode_T1'}_N{N_all}_Hk16_Hv32",
                   "scratch": None if not verify else ("bf16" if args.bf16_scratch else "fp32"),
                   "l2": ("state pool (>= 0.5 GB) exceeds the 126 MB L2" if copies == 1 else
                          f"steps rotate over {copies} copies of the rank's pool (>= 0.5 GB together), so no step "
                          "finds its pool in the 126 MB L2")},
        "clocks": cs.summary(), "gpu_launches": args.steps * blocks,
        "roofline": {"kernel": "recurrent_kernel", "bound": "hbm", "achieved": gbs / world, "peak": pk["hbm"],
                     "unit": "GB/s", "frac": gbs / world / pk["hbm"], "peak_source": pk["src"],
                     # ncu capture of the decode step (T=1, fp32 pool): 1.021 GB for 256 x 32 (sequence, v-head)
                     # states, i.e. 124.6 KB each (part of the written state is still in L2 at the end)
                     "traffic": None if verify else 124.6e3 * N_all * Hv / world},
    }


def run_train(args, rank, world, device):
    """Config 3: forward (saving h and v_new) + backward, B=4, T=8192, Hk=Hv=32, batch rows sharded."""
    import flashqla_b200 as fq
    from flashqla_b200.sharding import batch_shard
    B_all, T, H_all = 4, args.tokens if args.tokens != 32768 else 8192, 32
    if world <= B_all:
        rows = batch_shard(B_all, world, rank)
        B, H = rows.stop - rows.start, H_all
        sharding = f"batch/{world}"
    else:  # more ranks than batch rows: every row's heads are split as well
        per_row = world // B_all
        assert world % B_all == 0 and H_all % per_row == 0
        B, H = 1, H_all // per_row
        sharding = f"batch/{B_all} x heads/{per_row}"
    gen = torch.Generator(device=device).manual_seed(3 + rank)
    rn = lambda *s: torch.randn(*s, generator=gen, device=device)
    q = torch.nn.functional.normalize(rn(B, T, H, K), dim=-1).bfloat16()
    k = torch.nn.functional.normalize(rn(B, T, H, K), dim=-1).bfloat16()
    v = rn(B, T, H, V).bfloat16()
    g = torch.nn.functional.logsigmoid(rn(B, T, H))
    beta = torch.sigmoid(rn(B, T, H))
    h0 = 0.1 * rn(B, H, K, V)
    do = rn(B, T, H, V).bfloat16()
    dht = 0.1 * rn(B, H, K, V)

    def step():
        g_cs, A, o, h, fs, vn, w = fq.chunk_gated_delta_rule_fwd(q, k, v, g, beta, initial_state=h0, output_h=True,
                                                                 output_v_new=True, output_w=True)
        return fq.chunk_gated_delta_rule_bwd(q, k, v, g_cs, beta, A, do, dht=dht, initial_state=h0, h=h, v_new=vn,
                                             w=w)

    use_cp = fq.cp.get_plan([T] * B, H, device).use_cp
    launches_per_step = fq.chunk.launches_per_forward(False, use_cp) + fq.chunk.launches_per_backward(False, use_cp)
    with ClockSampler(device.index or 0) as cs:
        ms, blocks = measure(step, args.steps, args.warmup, world, device)
    fq.check_device_status()
    per_step = ms / args.steps
    tokens = B_all * T
    flops = tokens * H_all * (163840 + 409600)
    pk = peaks()
    return {
        "metric": "gdn_train_fwd_bwd_tokens_per_s", "value": tokens / (per_step * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "blocks": blocks,
        "config": {"workload": f"train_fwd_bwd_B{B_all}_T{T}_Hk{H_all}_Hv{H_all}_K128_V128_chunk64", "sharding": sharding,
                   "l2": "inputs (>= 1 GB per step) exceed the 126 MB L2; no flush needed", "tokens": tokens},
        "clocks": cs.summary(), "gpu_launches": launches_per_step * args.steps * blocks,
        "roofline": {"kernel": "fwd+bwd (kkt_solve, chunk scan, bwd_scan, bwd_chunk)", "bound": "tensor", "achieved": flops / world / (per_step * 1e-3) / 1e12,
                     "peak": pk["tf_sus"], "unit": "TFLOP/s",
                     "frac": flops / world / (per_step * 1e-3) / 1e12 / pk["tf_sus"], "peak_source": pk["src"],
                     "traffic": None},
    }


# ------------------------------------------------------------------------------------ CPU arms
def reference_forward():
    """The CPU forward the reference arm times: the reference's own fp32 PyTorch forward
    (tests/ref_gdr.py, placed under oracle/_ref/ by oracle/build_ref.py where a checkout of the reference was
    at hand) when it is there, else the oracle port.  Returns (callable, kind, description)."""
    from oracle import gdr_oracle as orc
    ref = ROOT / "oracle" / "_ref" / "ref_gdr.py"
    if ref.exists():
        try:
            import importlib.util
            spec = importlib.util.spec_from_file_location("_ref_gdr", ref)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            fwd = mod.chunk_gated_delta_rule_fwd

            def run(inp):
                return fwd(inp["q"].float(), inp["k"].float(), inp["v"].float(), inp["g"].clone(), inp["beta"],
                           scale=128 ** -0.5)
            return run, "reference", "the reference's tests/ref_gdr.py forward (fp32 PyTorch, all host threads)"
        except Exception:  # missing dependency of the reference's file on this box: the port stands in
            pass
    return (lambda inp: orc.chunk_gdr_fwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"]), "port",
            "fp32 oracle port (oracle/gdr_oracle.py, all host threads)")


def cpu_prefill_sample(tokens_sample: int, repeats: int = 2, fn=None):
    """CPU forward on the first `tokens_sample` tokens of the default workload, all host threads."""
    from oracle import gdr_oracle as orc
    torch.set_num_threads(os.cpu_count() or 1)
    inp = orc.make_prefill_inputs(1, tokens_sample, 16, 32, seed=1)
    if fn is None:
        fn = lambda i: orc.chunk_gdr_fwd(i["q"], i["k"], i["v"], i["g"], i["beta"])
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        fn(inp)
        best = min(best, time.perf_counter() - t0)
    return tokens_sample / best, best


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="prefill_fwd", choices=["prefill_fwd", "prefill_sp", "varlen", "decode", "verify", "train"])
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--bf16-scratch", action="store_true")
    ap.add_argument("--block-dv", type=int, default=None, help="recurrent workloads: rows of V per CTA (16 or 32)")
    ap.add_argument("--cpu-sample-tokens", type=int, default=32768)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true",
                    help="default workload only: skip the decode / verify / varlen / train records")
    ap.add_argument("--eager", action="store_true", help="time plain calls instead of CUDA-graph replays")
    ap.add_argument("--compare-fla", action="store_true",
                    help="also time FLA's Triton forward on the same inputs (adds a same_box entry)")
    ap.add_argument("--min-seconds", type=float, default=None,
                    help="total timed time to reach by repeating the K-step block (default 1.0; 0 = one block, "
                         "for profiler captures)")
    args = ap.parse_args()
    rank, world, local = dist_env()
    args.warmup = max(args.warmup, 3)
    if args.min_seconds is not None:
        global MIN_TIMED_SECONDS
        MIN_TIMED_SECONDS = args.min_seconds

    if args.impl == "reference":
        if rank != 0:
            return
        steps = max(1, min(args.steps, 3))
        ref_fn, kind, what = reference_forward()
        vals = []
        for _ in range(1 + steps):
            tps, sec = cpu_prefill_sample(args.cpu_sample_tokens, repeats=1, fn=ref_fn)
            vals.append(tps)
        tps = sum(vals[-steps:]) / steps
        sample = f"first {args.cpu_sample_tokens} tokens of the workload (all 32 v-heads), {what}"
        print(json.dumps({
            "impl": "reference", "metric": "gdn_prefill_fwd_tokens_per_s", "value": tps, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": 1, "ms_per_step": args.cpu_sample_tokens / tps * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "prefill_fwd_B1_T32768_Hk16_Hv32_K128_V128_chunk64", "tokens": 32768},
            "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": kind,
                             "sample": sample},
            "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}))
        return

    import torch.distributed as dist
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    if args.workload == "prefill_fwd":
        line = run_prefill(args, rank, world, device)
    elif args.workload == "prefill_sp":
        line = run_prefill_sp(args, rank, world, device)
    elif args.workload == "varlen":
        line = run_prefill(args, rank, world, device, varlen=True)
    elif args.workload == "train":
        line = run_train(args, rank, world, device)
    else:
        line = run_recurrent(args, rank, world, device, verify=args.workload == "verify")
    if args.workload == "prefill_fwd" and not args.no_secondary:
        # the other metrics of the path, measured after the headline's timed region with the same rules; every
        # rank takes part (the shards are those of the workloads themselves)
        import copy
        secondary = []
        workloads = [("decode", {}), ("verify", {}), ("verify", {"bf16_scratch": True}), ("varlen", {}), ("train", {})]
        if world > 1:  # the optional sequence-parallel mode: tokens over the ranks, one NCCL all-gather per call
            workloads.append(("prefill_sp", {}))
        for wl, extra in workloads:
            a2 = copy.copy(args)
            a2.workload, a2.steps, a2.tokens, a2.bf16_scratch = wl, min(args.steps, 20), 32768, False
            a2.compare_fla = wl in ("decode", "verify") and world == 1  # same-box bars: FLA (decode), the reference's own op
            for name, val in extra.items():
                setattr(a2, name, val)
            try:
                if wl == "varlen":
                    rec = run_prefill(a2, rank, world, device, varlen=True)
                elif wl == "train":
                    rec = run_train(a2, rank, world, device)
                elif wl == "prefill_sp":
                    rec = run_prefill_sp(a2, rank, world, device)
                else:
                    rec = run_recurrent(a2, rank, world, device, verify=wl == "verify")
                rec = {k: rec[k] for k in ("metric", "value", "unit", "ms_per_step", "steps", "blocks", "config",
                                           "roofline", "clocks", "gpu_launches", "same_box") if k in rec}
            except Exception as exc:
                rec = {"metric": wl, "error": f"{type(exc).__name__}: {str(exc)[:200]}"}
            secondary.append(rec)
        line["secondary"] = secondary
        line["gpu_launches"] += sum(r.get("gpu_launches", 0) for r in secondary)
    if rank == 0:
        if not args.no_cpu_baseline and args.workload == "prefill_fwd" and world == 1:
            ref_fn, kind, what = reference_forward()
            tps, sec = cpu_prefill_sample(args.cpu_sample_tokens, fn=ref_fn)
            line["cpu_baseline"] = {
                "value": tps, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": kind,
                "sample": f"first {args.cpu_sample_tokens} of the 32768 tokens (all 32 v-heads), {what}, best of 2, "
                          f"{sec:.2f} s"}
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
