#!/usr/bin/env python
"""Benchmark of the omni-attention forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload C4] [--no-c5]

One "step" = one forward pass of the block-mask attention over one batch of synthetic input.
Workload at every N: the 8K interleaved text/image configuration (C4: H32 N8192 D128 bf16, block
128), one batch element per GPU (batch*heads are independent, so ranks share nothing and there
is no collective on the data path: weak scaling). Metric: effective TFLOP/s counting only the
4*128*128*D flops of visited blocks. Prints ONE JSON line on rank 0.

Timing: W warm-up steps, then K steps each bracketed by CUDA events on the launching stream with a
256 MiB L2 flush before every step (not timed); the per-rank sum is reduced with MAX over ranks.
`e2e` is the same metric through the public Python operator with pinned HOST buffers, the
host->device copies of q, k, v and the device->host copy of the output inside the timed region;
`e2e.copy_only` is the same copy pattern with no kernel (the floor the host link sets).
Reported aside in the same line: the other configurations (`configs`), the reference's 13-argument
module entry (`dropin_13arg`), the same mask listed in 64x64 blocks (`blocks_64x64`), the 32K configuration sharded over the ranks with its optional
all-gather (`c5_sharded`), the backward pass and the soft-cap variant.
`--impl reference` times the reference's CPU torch path (the oracle's restatement of
omni_attn_torch.naive_attention_with_dense_mask, the additive mask of a head built beforehand) on
this host's cores; one step = one head of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from omni_attention_b200 import inputs  # noqa: E402

METRIC = "effective_tflops_nonempty_blocks"
UNIT = "TFLOP/s"


def workload_config(cfg):
    """The `config` object of the JSON line: the same in both arms."""
    return {"workload": f"{cfg.name}: one batch element per GPU, H={cfg.H} N={cfg.N} D={cfg.D} bf16, 128x128 blocks, "
                        f"interleaved text/image mask (1024-token images), mask seed = rank, batch*heads sharded over "
                        f"the GPUs, no collective",
            "B_per_gpu": 1, "H": cfg.H, "N": cfg.N, "D": cfg.D, "block": 128,
            "flop_count": "4*128*128*D per visited (listed FULL/CAUSAL/PARTIAL) block",
            "l2": "256 MiB flush before every timed GPU step; q,k,v,o of a step total 268 MB (> 126 MB L2)"}

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the timed kernel on this
# workload, from the ncu capture summarised in profiles/ (None until captured).
NCU_DRAM_BYTES_PER_LAUNCH = {"C4": 330.3e6}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), float(d.get("hbm_gbs", 0.0)), "measured"
    return 1590.0, 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs (read-only)."""

    def __init__(self, device_index: int, period_s: float = 0.005):
        super().__init__(daemon=True)
        self.period = period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml

            self.nv = pynvml
            pynvml.nvmlInit()
            try:
                uuid = torch.cuda.get_device_properties(device_index).uuid
                self.h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(uuid)).encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwPowerBrakeSlowdown", 0x80): "hw_power_brake_slowdown",
        }
        while not self._halt.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                try:
                    r = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                except Exception:
                    r = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._halt.set()
        self.join(timeout=1.0)
        s = sorted(self.samples)
        med = s[len(s) // 2] if s else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(s)}


def device_qkv(B, H, N, D, dtype, seed, device, scale):
    g = torch.Generator(device=device).manual_seed(seed)
    mk = lambda: (torch.randn(B, H, N, D, generator=g, device=device, dtype=torch.float32) * scale).to(dtype)
    return mk(), mk(), mk()


def time_steps(fn, steps, warmup, flush):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    evs = []
    for _ in range(steps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        evs.append((e0, e1))
    torch.cuda.synchronize()
    return sum(a.elapsed_time(b) for a, b in evs)  # ms over all steps


def _time_reference_heads(cfg, bm, heads, order):
    """The reference's function on one head per step: q, k, v of the head as fp32 and its additive
    [N, N] mask are made beforehand; the timed call is the matmul - add mask - softmax - matmul of
    omni_attn_torch.naive_attention_with_dense_mask and nothing else. Returns seconds per step in `order`."""
    from oracle import omni_oracle as orc

    q, k, v = inputs.make_qkv(1, cfg.H, cfg.N, cfg.D, cfg.dtype, 0, cfg.qkv_scale, bh_range=(0, heads))
    q, k, v = q.float(), k.float(), v.float()
    masks = [orc.to_score_mask(orc.to_dense_mask_slice(bm, 0, h))[None, None] for h in range(heads)]
    times = []
    for h in order:
        t0 = time.perf_counter()
        orc.attention_dense_mask(q[:, h:h + 1], k[:, h:h + 1], v[:, h:h + 1], masks[h], want_lse=False)
        times.append(time.perf_counter() - t0)
    return times


def cpu_baseline(cfg, bm, heads=3, budget_s=20.0):
    """Reference torch path on this host's cores on a bounded sample of the same workload."""
    per_head = [inputs.effective_flops(bm.slice_heads(h, h + 1), cfg.D) for h in range(heads)]
    order = [0] + list(range(heads))            # one untimed warm-up call
    times = _time_reference_heads(cfg, bm, heads, order)[1:]
    t_total, fl = sum(times), sum(per_head)
    return {"value": fl / t_total / 1e12, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{heads} of {cfg.H} heads of one {cfg.name} batch element; per head the reference's "
                      f"naive_attention_with_dense_mask on fp32 inputs with the head's additive [N,N] mask built "
                      f"beforehand (not timed), torch CPU",
            "ms_per_head": 1e3 * t_total / heads}


def run_reference(args, rank, world):
    """Reference arm: the reference's CPU torch path (oracle restatement) on the host cores."""
    if rank != 0:
        return
    cfg = inputs.CONFIGS[args.workload]
    torch.set_num_threads(os.cpu_count() or 1)
    bm, _ = inputs.make_block_mask(cfg, 0, B=1)
    heads = min(cfg.H, 4, args.steps + args.warmup)
    order = [i % heads for i in range(args.warmup + args.steps)]
    times = _time_reference_heads(cfg, bm, heads, order)[args.warmup:]
    fl = sum(inputs.effective_flops(bm.slice_heads(h, h + 1), cfg.D) for h in order[args.warmup:])
    t_total = sum(times)
    val = fl / t_total / 1e12
    cores = torch.get_num_threads()
    sample = (f"one step = one head ({cfg.N}x{cfg.N} fp32 scores) of the workload, heads 0..{heads - 1} in turn; the "
              f"reference's naive_attention_with_dense_mask with the additive mask built beforehand; torch CPU, {cores} threads")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * t_total / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(cfg),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }), flush=True)


def block_type_counts(bm):
    """Listed blocks by type (the entries the kernels visit)."""
    mb = bm.kv_indices.shape[-1]
    listed = torch.arange(mb) < bm.kv_num_blocks.long().clamp(0, mb).unsqueeze(-1)
    t = bm.block_mask_types
    return {"FULL": int((listed & (t == 2)).sum()), "CAUSAL": int((listed & (t == 1)).sum()),
            "PARTIAL": int((listed & (t == 3)).sum())}


def median_ms(fn, flush, steps=20, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(steps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2], ts[0]


def run_ours(args, rank, local_rank, world):
    import torch.distributed as dist

    import omni_attention_b200 as pkg
    from omni_attention_b200 import sharding
    from omni_attention_b200.ops import load_library, omni_attention, omni_attention_forward_out

    cfg = inputs.CONFIGS[args.workload]
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    peak_tf, peak_hbm, which = measured_peaks()
    # one batch element per rank; every rank draws its own image/text layout
    bm, mask_meta = inputs.make_block_mask(cfg, seed=rank, B=1)
    flops = inputs.effective_flops(bm, cfg.D)
    q, k, v = device_qkv(1, cfg.H, cfg.N, cfg.D, cfg.dtype, 1234 + rank, dev, cfg.qkv_scale)
    out = torch.empty_like(q)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def step():
        omni_attention_forward_out(q, k, v, out, bm, cfg.N, None, None, status, "ws")

    step()  # builds the cached device copy of the mask (+ bit-packed partial pool), not a timed step
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler.start()
    total_ms = time_steps(step, args.steps, args.warmup, flush)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    # ---- C5 (32K multi-image), batch*heads sharded over the ranks: strong scaling, reported aside --
    # Last on purpose: its 34 ms launches draw enough power to lower the SM clock for a while, which
    # would otherwise be carried into the short measurements above.
    c5 = None
    if not args.no_c5:
        c5cfg = inputs.CONFIGS["C5"]
        bm5, _ = inputs.make_block_mask(c5cfg, seed=0)
        BH = c5cfg.B * c5cfg.H
        shard, (lo, hi) = sharding.shard_block_mask(bm5, rank, world)
        fl5 = inputs.effective_flops(bm5, c5cfg.D)
        q5, k5, v5 = device_qkv(1, hi - lo, c5cfg.N, c5cfg.D, c5cfg.dtype, 99 + rank, dev, c5cfg.qkv_scale)
        o5 = torch.empty_like(q5)

        def step5():
            omni_attention_forward_out(q5, k5, v5, o5, shard, c5cfg.N, None, None, status, "ws")

        step5()
        if world > 1:
            dist.barrier()
        ms5 = time_steps(step5, 5, 3, flush) / 5
        c5 = {"ms": ms5, "flops_all_ranks": fl5, "gather_ms": 0.0, "gather_bytes": 0}
        if world > 1:
            # optional epilogue for callers that want the whole output on every GPU: one NCCL all-gather of
            # the ranks' own output buffers, timed on its own (not part of the forward)
            full = sharding.all_gather_outputs(o5, BH)      # warm-up (communicator set-up)
            del full
            torch.cuda.synchronize()
            dist.barrier()
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            g0.record()
            full = sharding.all_gather_outputs(o5, BH)
            g1.record()
            torch.cuda.synchronize()
            assert torch.equal(full[lo:hi], o5[0]), "gathered rows of the own range differ from the local output"
            c5["gather_ms"] = g0.elapsed_time(g1)
            c5["gather_bytes"] = (BH - (hi - lo)) * c5cfg.N * c5cfg.D * 2
            del full
        del q5, k5, v5, o5

    if int(status.item()) != 0:
        raise RuntimeError(f"kernel status {int(status.item()):#x}")

    # ---- end to end through the public operator with host buffers -------------------------------
    # Every step copies its q, k, v from pinned host memory, calls the public operator and copies the
    # output back. Steps alternate between two streams so that one step's device-to-host copy and
    # kernel run under the next step's host-to-device copy (the host link is full duplex); every step
    # still moves all of its own bytes inside the timed region. `copy_only` is the same loop without
    # the operator call (the output copy reads a tensor that is already there): the floor set by the
    # host link, against which the end-to-end time is to be read.
    hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
    e2e_streams = [torch.cuda.Stream(device=dev) for _ in range(2)]
    ho = [torch.empty_like(hq).pin_memory() for _ in e2e_streams]
    e2e_steps = max(4, min(args.steps, 20))

    def e2e_step(i, with_kernel=True):
        with torch.cuda.stream(e2e_streams[i & 1]):
            dq, dk, dv = (t.to(dev, non_blocking=True) for t in (hq, hk, hv))
            o = omni_attention(dq, dk, dv, bm) if with_kernel else out
            ho[i & 1].copy_(o, non_blocking=True)

    def timed_e2e(with_kernel):
        for i in range(4):
            e2e_step(i, with_kernel)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        main_stream = torch.cuda.current_stream()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for st_ in e2e_streams:
            st_.wait_event(e0)
        for i in range(e2e_steps):
            e2e_step(i, with_kernel)
        for st_ in e2e_streams:
            main_stream.wait_stream(st_)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    e2e_ms = timed_e2e(True)
    assert torch.equal(ho[0], ho[1])   # both streams computed the same inputs
    copy_ms = timed_e2e(False)

    # ---- the other configurations, both kernels (every rank runs them; rank 0's numbers are printed) ----
    configs = {}
    for cname in ("C1", "C2", "C3"):
        c = inputs.CONFIGS[cname]
        cbm, _ = inputs.make_block_mask(c, seed=0)
        cq, ck, cv = device_qkv(c.B, c.H, c.N, c.D, c.dtype, 7, dev, c.qkv_scale)
        co = torch.empty_like(cq)
        cfl = inputs.effective_flops(cbm, c.D)
        entry = {"shape": f"B={c.B} H={c.H} N={c.N} D={c.D} {str(c.dtype).replace('torch.', '')}", "blocks": block_type_counts(cbm),
                 "effective_gflop": cfl / 1e9}
        for kern in ("ws", "simple"):
            fn = lambda kern=kern: omni_attention_forward_out(cq, ck, cv, co, cbm, c.N, None, None, status, kern)
            fn()
            med, mn = median_ms(fn, flush)
            entry[kern] = {"ms": med, "ms_min": mn, "tflops": cfl / med / 1e9, "frac_of_peak": cfl / med / 1e9 / peak_tf}
        configs[cname] = entry
        del cq, ck, cv, co
    configs["C4"] = {"shape": f"B=1 H={cfg.H} N={cfg.N} D={cfg.D} bf16", "blocks": block_type_counts(bm),
                     "effective_gflop": flops / 1e9}
    fn = lambda: omni_attention_forward_out(q, k, v, out, bm, cfg.N, None, None, status, "simple")
    fn()
    med, mn = median_ms(fn, flush)
    configs["C4"]["simple"] = {"ms": med, "ms_min": mn, "tflops": flops / med / 1e9, "frac_of_peak": flops / med / 1e9 / peak_tf}

    # ---- the reference's own boundary: the 13-argument module function on torch tensors, byte-per-element
    # pool as the reference stores it -------------------------------------------------------------------
    mod = pkg.install_reference_module()
    m = bm._cache[(str(dev), True)]
    pool_bytes = bm.partial_block_masks.to(dev).contiguous()
    fn = lambda: mod.omni_attn_mma_stages_split_q_shared_kv(q, k, v, out, m["nb"], m["idx"], m["typ"], 128, 128, cfg.N,
                                                            m["pidx"], pool_bytes, True)
    fn()
    dropin_med, dropin_min = median_ms(fn, flush)
    del pool_bytes

    # ---- the same pattern listed in 64x64 blocks (the reference's other block shape), reported aside ----
    from omni_attention_b200.block_mask import block_mask_from_row_limits, row_limits_from_modality_positions

    limits64, causal_rows64 = row_limits_from_modality_positions(cfg.N, mask_meta["image_spans"])
    bm64 = block_mask_from_row_limits(limits64, cfg.H, causal_rows64, 64, True)
    out64 = torch.empty_like(out)
    fn64 = lambda: omni_attention_forward_out(q, k, v, out64, bm64, cfg.N, None, None, status, "ws")
    fn64()
    blk64_med, blk64_min = median_ms(fn64, flush)
    step()
    torch.cuda.synchronize()
    blk64_same = bool(torch.equal(out64, out))
    del out64

    # ---- backward pass on the same workload (three launches per step), reported aside ---------------
    bwd_ms = 0.0
    if not args.no_backward:
        from omni_attention_b200.ops import omni_attention_backward_out

        lse = torch.empty(1, cfg.H, cfg.N, dtype=torch.float32, device=dev)
        omni_attention_forward_out(q, k, v, out, bm, cfg.N, None, lse, status, "ws")
        d_out = (torch.randn(q.shape, device=dev, generator=torch.Generator(device=dev).manual_seed(77 + rank)) * 0.5).to(q.dtype)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
        wsp = torch.empty(int(load_library().omni_attn_bwd_workspace_bytes(1, cfg.H, cfg.N)), dtype=torch.uint8, device=dev)

        def bstep():
            omni_attention_backward_out(q, k, v, out, lse, d_out, dq, dk, dv, bm, cfg.N, None, status, wsp)

        bstep()
        if world > 1:
            dist.barrier()
        bwd_ms = time_steps(bstep, 10, 3, flush) / 10
        del d_out, dq, dk, dv, wsp

    # ---- the Transfusion model's variant of the forward (tanh soft-cap 50), reported aside -----------
    cap_ms = 0.0
    if not args.no_backward:
        def cstep():
            omni_attention_forward_out(q, k, v, out, bm, cfg.N, None, None, status, "ws", softcap=50.0)

        cstep()
        if world > 1:
            dist.barrier()
        cap_ms = time_steps(cstep, 10, 3, flush) / 10
    if int(status.item()) != 0:
        raise RuntimeError(f"kernel status {int(status.item()):#x}")

    # ---- reduce over ranks (MAX of time, SUM of work) ---------------------------------------------
    vals = torch.tensor([total_ms, e2e_ms, c5["ms"] if c5 else 0.0, float(flops), bwd_ms, cap_ms, copy_ms,
                         c5["gather_ms"] if c5 else 0.0, dropin_med], dtype=torch.float64, device=dev)
    if world > 1:
        mx = vals.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = vals.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        total_ms, e2e_ms, c5ms, flops_all, bwd_ms = float(mx[0]), float(mx[1]), float(mx[2]), float(sm[3]), float(mx[4])
        cap_ms, copy_ms, gather_ms, dropin_med = float(mx[5]), float(mx[6]), float(mx[7]), float(mx[8])
    else:
        c5ms, flops_all, gather_ms = float(vals[2]), float(flops), 0.0
    if rank != 0:
        return

    ms_per_step = total_ms / args.steps
    value = flops_all / (ms_per_step * 1e-3) / 1e12
    per_gpu_tf = flops / (ms_per_step * 1e-3) / 1e12
    e2e_val = flops_all / (e2e_ms / e2e_steps * 1e-3) / 1e12
    tensor_bytes = q.numel() * q.element_size()
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": workload_config(cfg),
        "kernel": "omni_fwd_ws_kernel<128,bf16> (persistent, dynamic unit hand-out)",
        "visited_blocks_per_gpu": bm.visited_blocks(), "effective_gflop_per_gpu": flops / 1e9,
        "fwd_ms": ms_per_step,
        "roofline": {"bound": "tensor", "achieved": per_gpu_tf, "peak": peak_tf, "unit": UNIT, "frac": per_gpu_tf / peak_tf,
                     "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get(cfg.name), "peak_source": f"MEASURED_PEAKS.json bf16_tflops ({which}, burst)",
                     "frac_of_nominal_2250": per_gpu_tf / 2250.0},
        "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": 3 * tensor_bytes, "d2h_bytes_per_step": tensor_bytes,
                "ms_per_step": e2e_ms / e2e_steps, "steps": e2e_steps, "streams": 2,
                "kernel_ms": ms_per_step,
                "copy_only": {"ms_per_step": copy_ms / e2e_steps,
                              "gb_per_s_per_gpu": 4 * tensor_bytes / (copy_ms / e2e_steps * 1e-3) / 1e9,
                              "note": "the same host-to-device and device-to-host copies per step with no kernel"},
                "over_copy_only": e2e_ms / copy_ms,
                "note": "steps alternate between two streams: copies of one step overlap the next step's"},
        "gpu_launches": args.steps,
        "clocks": clocks,
        "configs": configs,
        "blocks_64x64": {"ms": blk64_med, "ms_min": blk64_min, "tflops": flops / blk64_med / 1e9,
                         "over_headline": blk64_med / ms_per_step, "listed_blocks": int(bm64.visited_blocks()),
                         "bit_identical_to_128_blocks": blk64_same,
                         "what": "the same mask listed in 64x64 blocks (four times as many entries), same kernel"},
        "dropin_13arg": {"ms": dropin_med, "ms_min": dropin_min, "tflops": flops / dropin_med / 1e9,
                         "over_headline": dropin_med / ms_per_step,
                         "what": "omni_attn.omni_attn_mma_stages_split_q_shared_kv(13 positional arguments) on the same inputs: "
                                 "byte-per-element pool as the reference stores it; the module keeps a unit counter per stream"},
    }
    if c5 is not None:
        line["c5_sharded"] = {"workload": "C5: B=4 H=32 N=32768 D=128 bf16, 128 (batch,head) pairs split over the ranks (strong scaling)",
                              "fwd_ms": c5ms, "value": c5["flops_all_ranks"] / (c5ms * 1e-3) / 1e12, "unit": UNIT, "steps": 5}
        if world > 1:
            line["c5_sharded"]["all_gather_ms"] = gather_ms
            line["c5_sharded"]["all_gather_recv_bytes_per_gpu"] = c5["gather_bytes"]
            line["c5_sharded"]["all_gather_gb_per_s_per_gpu"] = c5["gather_bytes"] / (gather_ms * 1e-3) / 1e9
    if bwd_ms > 0:
        # five tile contractions per visited block (S, dP, dV, dK, dQ) = 2.5 x the forward count; the
        # kernels execute seven (S and dP are recomputed by the dQ kernel)
        bwd_tf = 2.5 * flops / (bwd_ms * 1e-3) / 1e12
        line["backward"] = {"ms": bwd_ms, "value": 2.5 * flops_all / (bwd_ms * 1e-3) / 1e12, "unit": UNIT, "steps": 10,
                            "launches_per_step": 3, "flop_count": "10*128*128*D per visited block",
                            "roofline_frac": bwd_tf / peak_tf,
                            "kernels": "omni_bwd_prep_kernel, omni_bwd_dkdv_kernel, omni_bwd_dq_kernel"}
    if cap_ms > 0:
        line["softcap_forward"] = {"ms": cap_ms, "value": flops_all / (cap_ms * 1e-3) / 1e12, "unit": UNIT, "softcap": 50.0,
                                   "steps": 10, "roofline_frac": flops / (cap_ms * 1e-3) / 1e12 / peak_tf}
    if world == 1 and not args.no_cpu_baseline:
        torch.set_num_threads(os.cpu_count() or 1)
        line["cpu_baseline"] = cpu_baseline(cfg, bm)
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="C4", choices=["C3", "C4"])
    ap.add_argument("--no-c5", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-backward", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_ours(args, rank, local_rank, world)
    finally:
        if world > 1:
            import torch.distributed as dist

            dist.destroy_process_group()


if __name__ == "__main__":
    main()
